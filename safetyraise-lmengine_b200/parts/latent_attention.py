"""Attention over a cached latent.

Per token the pages hold one vector: the RMS-normed latent c (kv_rank elements) and, behind it, one
rotated key part (rot_dim elements) that all heads share.  Head h's unrotated key is U_k,h c and its
value U_v,h c; the score of query i on key j is (q_i . U_k,h c_j + qr_i . kr_j) * scale.  Neither keys
nor values are formed: the up projection of the keys is folded into the query (U_k,h^T q_i), the
attention runs over [c | kr] with the values being c itself, and the up projection of the values is
applied to the attended latent.  The result does not depend on how a prompt is cut: every step runs
the same three kernels around the same attention kernel.  Each head's output is multiplied by the
sigmoid of a projection of the mixer's input before the output projection.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import PAGED_ALL
from ..config.spec import LatentAttentionSpec, RunStep
from ..errors import Unsupported
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import POSITION_ENCODINGS, ROTATION, CacheNeed, Part, lookup, register_mixer
from .linear import Linear


@register_mixer("latent_attention")
class LatentAttention(Part):
    def __init__(self, spec: LatentAttentionSpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        rows = [tensors[p + nm.q], tensors[p + nm.down]] + ([tensors[p + nm.gate]] if s.output_gate else [])
        self.proj = Linear(torch.cat(rows, dim=0).contiguous(), p + "q_down_gate")
        self.c_off = s.heads * (s.head_dim + s.rot_dim)
        self.g_off = self.c_off + s.kv_rank + s.rot_dim if s.output_gate else -1
        self.latent_norm_w = tensors[p + nm.latent_norm]
        self.uk = tensors[p + nm.up_k].view(s.heads, s.head_dim, s.kv_rank).contiguous()
        # per head [kv_rank, v_head_dim]: a thread of the expanding kernel owns one output column
        self.uv_t = tensors[p + nm.up_v].view(s.heads, s.v_head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.out = Linear(tensors[p + nm.o], p + nm.o)
        self.position = None
        if s.position is not None:
            self.position = lookup(POSITION_ENCODINGS, s.position.kind, "position encoding")(s.position, mctx)
            if getattr(self.position, "applies", ROTATION) != ROTATION:
                raise Unsupported(f"position encoding {s.position.kind!r} is not a rotation")

    @classmethod
    def tensor_decls(cls, s: LatentAttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        decls = [TensorDecl(p + nm.q, (s.heads * (s.head_dim + s.rot_dim), s.hidden_size), MATRIX),
                 TensorDecl(p + nm.down, (s.kv_rank + s.rot_dim, s.hidden_size), MATRIX),
                 TensorDecl(p + nm.latent_norm, (s.kv_rank,), VECTOR),
                 TensorDecl(p + nm.up_k, (s.heads * s.head_dim, s.kv_rank), MATRIX),
                 TensorDecl(p + nm.up_v, (s.heads * s.v_head_dim, s.kv_rank), MATRIX)]
        if s.output_gate:
            decls.append(TensorDecl(p + nm.gate, (s.heads, s.hidden_size), MATRIX))
        decls.append(TensorDecl(p + nm.o, (s.hidden_size, s.heads * s.v_head_dim), MATRIX))
        return decls

    @classmethod
    def cache_need_of(cls, s: LatentAttentionSpec) -> CacheNeed:
        # one KV head of kv_rank + rot_dim elements per token, and no value pool: the values are the latent
        return CacheNeed(PAGED_ALL, 1, s.kv_rank + s.rot_dim, None, v_head_dim=0)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        s = self.spec
        T = x.shape[0]
        proj = self.proj(ctx, x, "latent.proj", out_dtype=torch.float32)
        cache, _, group = ctx.cache.kv_of_entry(run_step.cache)
        rot = self.position.rotation(ctx) if self.position is not None else None
        if rot is not None and not rot.interleaved:
            raise Unsupported("the latent attention kernels rotate interleaved pairs only")
        if run_step.writes_cache:
            ops.latent_append(proj, self.c_off, self.latent_norm_w, s.latent_norm_eps, rot, cache, ctx.kv_slot[group],
                              s.kv_rank, s.rot_dim)
        qd = s.kv_rank + s.rot_dim
        q = ctx.workspace.get("latent.q", T, s.heads * qd, torch.float32)
        ops.latent_absorb(proj, self.uk, rot, q, s.heads, s.head_dim, s.rot_dim, s.kv_rank)
        o_lat = ctx.workspace.get("latent.o", T, s.heads * s.kv_rank, torch.float32)
        ops.paged_attention_general(ctx, q, cache, None, o_lat, ctx.block_tables[group], None, s.heads, 1, qd,
                                    s.kv_rank, s.softmax_scale)
        gated = ctx.workspace.get("latent.out", T, s.heads * s.v_head_dim, ctx.dtype)
        ops.latent_expand(o_lat, self.uv_t, proj, self.g_off, gated, s.heads, s.kv_rank, s.v_head_dim)
        return self.out(ctx, gated, "latent.proj_out")
