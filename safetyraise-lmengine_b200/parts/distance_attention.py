"""Grouped-query attention without a rotation, over a sliding window, whose scores fall with the
logarithm of the distance between query and key:

    q, k, v = W h;   q, k <- q, k / sqrt(mean(.^2) + eps) per head          (when the spec gives an eps)
    score(i, j) = (q_i . k_j) * scale * temperature_h - weight_h * ln(1 + rate_h * (i - j)),  0 <= i - j < window
    out_h = softmax(score) v * logistic((W_g h)_h)

temperature, weight and rate are learned numbers per query head; positions enter through i - j alone.
One stacked projection gives q | k | v | gate logits in float32, so the unit norms, the scores and the
gates see unrounded values; keys and values go to the pages in the cache's dtype.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import PAGED_ALL, PAGED_WINDOW
from ..config.spec import DistanceAttentionSpec, RunStep
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import CacheNeed, Part, register_mixer
from .linear import Linear


@register_mixer("distance_attention")
class DistanceAttention(Part):
    def __init__(self, spec: DistanceAttentionSpec, prefix: str, tensors: dict, mctx):
        self.spec = spec
        p, nm = prefix, spec.names
        rows = [tensors[p + nm.q], tensors[p + nm.k], tensors[p + nm.v]]
        if spec.output_gate:
            rows.append(tensors[p + nm.gate])
        self.proj = Linear(torch.cat(rows, dim=0).contiguous(), p + "qkvg")
        self.gate_offset = spec.heads * spec.head_dim + spec.kv_heads * (spec.head_dim + spec.v_head_dim)
        self.temperature = tensors[p + nm.temperature] if spec.temperature else None
        self.penalty = (tensors[p + nm.penalty_weight], tensors[p + nm.penalty_rate]) if spec.distance_penalty else None
        self.out = Linear(tensors[p + nm.o], p + nm.o)

    @classmethod
    def tensor_decls(cls, s: DistanceAttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        decls = [TensorDecl(p + nm.q, (s.heads * s.head_dim, s.hidden_size), MATRIX),
                 TensorDecl(p + nm.k, (s.kv_heads * s.head_dim, s.hidden_size), MATRIX),
                 TensorDecl(p + nm.v, (s.kv_heads * s.v_head_dim, s.hidden_size), MATRIX)]
        if s.distance_penalty:
            decls += [TensorDecl(p + nm.penalty_weight, (s.heads,), VECTOR),
                      TensorDecl(p + nm.penalty_rate, (s.heads,), VECTOR)]
        if s.temperature:
            decls.append(TensorDecl(p + nm.temperature, (s.heads,), VECTOR))
        if s.output_gate:
            decls.append(TensorDecl(p + nm.gate, (s.heads, s.hidden_size), MATRIX))
        decls.append(TensorDecl(p + nm.o, (s.hidden_size, s.heads * s.v_head_dim), MATRIX))
        return decls

    @classmethod
    def cache_need_of(cls, s: DistanceAttentionSpec) -> CacheNeed:
        return CacheNeed(PAGED_WINDOW if s.window else PAGED_ALL, s.kv_heads, s.head_dim, s.window,
                         v_head_dim=None if s.v_head_dim == s.head_dim else s.v_head_dim)

    def can_fuse(self, ctx) -> bool:
        return self.proj.can_fuse(ctx, ctx.T) and self.out.can_fuse(ctx, ctx.T)

    def forward_fused(self, ctx, nx, run_step: RunStep, residual: torch.Tensor, next_norm):
        """The same as forward for a lazily normalised input (the norm's scale is applied inside the stacked
        product), with the output projection adding into the residual stream and preparing the input of the
        part behind ``next_norm``."""
        proj = ctx.workspace.get("dist_attn.proj", ctx.T, self.proj.out_features, torch.float32)
        self.proj.from_normed(ctx, nx, proj)
        return self.out.into_residual(ctx, self._attend(ctx, proj, run_step), residual, next_norm, "a", early=False)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        proj = self.proj(ctx, x, "dist_attn.proj", out_dtype=torch.float32)
        return self.out(ctx, self._attend(ctx, proj, run_step), "dist_attn.o")

    def _attend(self, ctx, proj: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        """From the stacked projection to the gated heads' outputs [T, heads * v_head_dim]."""
        s = self.spec
        T = proj.shape[0]
        k_pool, v_pool, group = ctx.cache.kv_of_entry(run_step.cache)
        # prompts and portions with heads of 128 for keys and values: the framework's tensor-memory kernel, which
        # takes its queries in bfloat16 and changes a row of scores in registers before the softmax
        page_size = k_pool.shape[2]
        on_tcgen05 = (ctx.max_q_len > 4 and s.head_dim == s.v_head_dim
                      and ops.sinks_on_tcgen05(ctx, ctx.dtype, s.heads, s.kv_heads, s.head_dim, s.v_head_dim, page_size))
        q = ctx.workspace.get("dist_attn.q", T, s.heads * s.head_dim, ctx.dtype if on_tcgen05 else torch.float32)
        ops.attention_unit_norm_append(proj, s.unit_norm_eps, q, k_pool, v_pool, ctx.kv_slot[group], s.heads,
                                       s.kv_heads, s.head_dim, s.v_head_dim, run_step.writes_cache)
        gated = s.output_gate
        attended = ctx.workspace.get("dist_attn.out", T, s.heads * s.v_head_dim, ctx.dtype)
        if on_tcgen05:
            ops.paged_attention(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], s.heads, s.kv_heads,
                                s.head_dim, page_size, s.softmax_scale, s.window or 0,
                                mods=(self.temperature, self.penalty[0] if self.penalty else None,
                                      self.penalty[1] if self.penalty else None))
            if gated:
                ops.head_gate(attended, proj, self.gate_offset, attended, s.heads, s.v_head_dim)
            return attended
        # the gate is applied where the general kernels write a head's output (the kernel that adds key slices included)
        ops.paged_attention_general(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], None, s.heads, s.kv_heads,
                                    s.head_dim, s.v_head_dim, s.softmax_scale, s.window or 0,
                                    head_scale=self.temperature, penalty=self.penalty,
                                    gate=(proj, self.gate_offset) if gated else None)
        return attended
