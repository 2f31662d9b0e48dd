"""Grouped-query attention without a position encoding, with biases on the q / k / v projections,
a learned sink per head in the softmax denominator, keys and values of different sizes, and values
mixed with those of an earlier layer.

    score(i, j) = (q_i . k_j) * scale,  j <= i
    p_ij        = exp(score(i, j)) / (exp(sink_h) + sum_j' exp(score(i, j')))
    v           = (1 - lambda) v + lambda v_kept       (layers that mix; v_kept: the values, of the same
                                                         token, of the layer that keeps them)

The mixed values are what the pages hold.  The kept values live for one step in the step's tables:
a step's tokens only ever mix with their own.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import PAGED_ALL, PAGED_WINDOW
from ..config.spec import RunStep, SinkAttentionSpec
from ..errors import ConfigError
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import CacheNeed, Part, register_mixer
from .linear import Linear


@register_mixer("sink_attention")
class SinkAttention(Part):
    def __init__(self, spec: SinkAttentionSpec, prefix: str, tensors: dict, mctx):
        self.spec = spec
        p, nm = prefix, spec.names
        self.qkv = Linear(torch.cat([tensors[p + nm.q], tensors[p + nm.k], tensors[p + nm.v]], dim=0).contiguous(),
                          p + "qkv")
        self.bias = None
        if spec.bias:
            self.bias = torch.cat([tensors[p + n + nm.bias_suffix] for n in (nm.q, nm.k, nm.v)]).contiguous()
        self.sink = tensors[p + nm.sink] if spec.sink else None
        self.lam = tensors[p + nm.value_mix].reshape(1).contiguous() if spec.value_mix else None
        self.out = Linear(tensors[p + nm.o], p + nm.o)

    @classmethod
    def tensor_decls(cls, s: SinkAttentionSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        sizes = {nm.q: s.heads * s.head_dim, nm.k: s.kv_heads * s.head_dim, nm.v: s.kv_heads * s.v_head_dim}
        decls = [TensorDecl(p + n, (rows, s.hidden_size), MATRIX) for n, rows in sizes.items()]
        if s.bias:
            decls += [TensorDecl(p + n + nm.bias_suffix, (rows,), VECTOR) for n, rows in sizes.items()]
        if s.value_mix:
            decls.append(TensorDecl(p + nm.value_mix, (), VECTOR))     # unused by the layer that keeps, but stored
        if s.sink:
            decls.append(TensorDecl(p + nm.sink, (s.heads,), VECTOR))
        decls.append(TensorDecl(p + nm.o, (s.hidden_size, s.heads * s.v_head_dim), MATRIX))
        return decls

    @classmethod
    def cache_need_of(cls, s: SinkAttentionSpec) -> CacheNeed:
        return CacheNeed(PAGED_WINDOW if s.window else PAGED_ALL, s.kv_heads, s.head_dim, s.window,
                         v_head_dim=None if s.v_head_dim == s.head_dim else s.v_head_dim)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        s = self.spec
        T = x.shape[0]
        # the projection's result stays float32: the scores are float32 products of it
        qkv = self.qkv(ctx, x, "sink_attn.qkv", out_dtype=torch.float32)
        k_pool, v_pool, group = ctx.cache.kv_of_entry(run_step.cache)
        # prompts with heads of 128 for keys and values: the framework's tensor-memory kernel, which takes its
        # queries in bfloat16 and starts every row's softmax from the head's sink
        page_size = k_pool.shape[2]
        on_tcgen05 = (v_pool is not None and not s.window and ctx.max_q_len > 4 and s.sink
                      and ops.sinks_on_tcgen05(ctx, ctx.dtype, s.heads, s.kv_heads, s.head_dim, s.v_head_dim, page_size))
        q = ctx.workspace.get("sink_attn.q", T, s.heads * s.head_dim, ctx.dtype if on_tcgen05 else torch.float32)
        keep, mode = None, 0
        if s.value_mix:
            key = ("kept_values", s.kv_heads * s.v_head_dim)
            if s.value_mix == "keep":
                keep = ctx.tables[key] = ctx.workspace.get("sink_attn.kept_values", T, s.kv_heads * s.v_head_dim,
                                                           torch.float32)
                mode = 1
            else:
                keep = ctx.tables.get(key)
                if keep is None:
                    raise ConfigError("a layer mixes its values with kept ones, but no layer before it keeps any")
                mode = 2
        ops.attention_bias_append(qkv, self.bias, q, k_pool, v_pool, ctx.kv_slot[group], s.heads, s.kv_heads,
                                  s.head_dim, s.v_head_dim, keep, self.lam, mode, run_step.writes_cache)
        attended = ctx.workspace.get("sink_attn.out", T, s.heads * s.v_head_dim, ctx.dtype)
        if on_tcgen05:
            ops.paged_attention(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], s.heads, s.kv_heads,
                                s.head_dim, page_size, s.softmax_scale, 0, sinks=self.sink)
            return self.out(ctx, attended, "sink_attn.proj")
        ops.paged_attention_general(ctx, q, k_pool, v_pool, attended, ctx.block_tables[group], self.sink, s.heads,
                                    s.kv_heads, s.head_dim, s.v_head_dim, s.softmax_scale, s.window or 0)
        return self.out(ctx, attended, "sink_attn.proj")
