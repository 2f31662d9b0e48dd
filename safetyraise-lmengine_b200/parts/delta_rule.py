"""The gated delta rule: a recurrent mixer with a matrix of state S [head_dim, v_head_dim] per head.

Per token and head, with q and k unit vectors (q also divided by sqrt(head_dim)), q, k and v behind a
short causal convolution over time and SiLU, beta = sigmoid(B x), g = exp(-exp(A) softplus(a x + dt)):

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the token's own write.  o is RMS-normed per head, scaled by a weight shared by the
heads and by silu(G x), then projected.  Value head h reads q / k head h // (heads / kv_heads).

What a request carries from token to token is a fixed-size float32 state in the request's slot: S of every
head and the last taps-1 inputs of every convolved channel.  It starts at zero (the engine zeroes a
slot for its new occupant) and is put back when a step fails (the engine's snapshot).
"""
from __future__ import annotations

from typing import List

import torch

from ..cache.manager import FIXED_STATE
from ..config.spec import DeltaRuleSpec, RunStep
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, TensorDecl
from .base import CacheNeed, Part, register_mixer
from .linear import Linear


@register_mixer("delta_rule")
class DeltaRule(Part):
    def __init__(self, spec: DeltaRuleSpec, prefix: str, tensors: dict, mctx):
        self.spec = s = spec
        p, nm = prefix, spec.names
        stacked = [tensors[p + n] for n in (nm.q, nm.k, nm.v, nm.beta, nm.decay, nm.gate)]
        self.proj = Linear(torch.cat(stacked, dim=0).contiguous(), p + "q_k_v_b_a_g")
        self.channels = 2 * s.kv_heads * s.head_dim + s.heads * s.v_head_dim
        self.conv_w = torch.cat([tensors[p + n + nm.conv_suffix] for n in (nm.q, nm.k, nm.v)], dim=0).float().contiguous()
        self.decay_log, self.decay_bias = tensors[p + nm.decay_log], tensors[p + nm.decay_bias]
        self.out_norm_w = tensors[p + nm.out_norm]
        self.gate_off = self.channels + 2 * s.heads
        self.out = Linear(tensors[p + nm.o], p + nm.o)

    @classmethod
    def tensor_decls(cls, s: DeltaRuleSpec, prefix: str) -> List[TensorDecl]:
        p, nm = prefix, s.names
        qk, v = s.kv_heads * s.head_dim, s.heads * s.v_head_dim
        decls = []
        for n, rows in ((nm.q, qk), (nm.k, qk), (nm.v, v)):
            decls += [TensorDecl(p + n, (rows, s.hidden_size), MATRIX),
                      TensorDecl(p + n + nm.conv_suffix, (rows, s.conv_taps), MATRIX)]
        decls += [TensorDecl(p + nm.beta, (s.heads, s.hidden_size), MATRIX),
                  TensorDecl(p + nm.decay, (s.heads, s.hidden_size), MATRIX),
                  TensorDecl(p + nm.decay_log, (s.heads,), VECTOR),
                  TensorDecl(p + nm.decay_bias, (s.heads,), VECTOR),
                  TensorDecl(p + nm.out_norm, (s.v_head_dim,), VECTOR),
                  TensorDecl(p + nm.gate, (v, s.hidden_size), MATRIX),
                  TensorDecl(p + nm.o, (s.hidden_size, v), MATRIX)]
        return decls

    @staticmethod
    def state_size(s: DeltaRuleSpec) -> int:
        channels = 2 * s.kv_heads * s.head_dim + s.heads * s.v_head_dim
        return s.heads * s.head_dim * s.v_head_dim + channels * (s.conv_taps - 1)

    @classmethod
    def cache_need_of(cls, s: DeltaRuleSpec) -> CacheNeed:
        return CacheNeed(FIXED_STATE, state_shape=(cls.state_size(s),), state_dtype=torch.float32)

    def forward(self, ctx, x: torch.Tensor, run_step: RunStep) -> torch.Tensor:
        s = self.spec
        T, H, G, dk, dv = x.shape[0], s.heads, s.kv_heads, s.head_dim, s.v_head_dim
        proj = self.proj(ctx, x, "delta.proj", out_dtype=torch.float32)
        state = ctx.cache.state_of_entry(run_step.cache)                    # [slots, state_size]
        qkv = ctx.workspace.get("delta.qkv", T, self.channels, torch.float32)
        beta = ctx.workspace.get("delta.beta", T, H, torch.float32)
        decay = ctx.workspace.get("delta.decay", T, H, torch.float32)
        qk = ctx.workspace.get("delta.qk", T, G, torch.float32)
        ops.delta_prepare(ctx, proj, self.conv_w, self.decay_log, self.decay_bias, state, qkv, beta, decay, qk, H, G,
                          dk, dv, s.conv_taps, s.unit_eps)
        o = ctx.workspace.get("delta.o", T, H * dv, torch.float32)
        ops.delta_recurrence(ctx, qkv, beta, decay, qk, state, o, H, G, dk, dv)
        gated = ctx.workspace.get("delta.out", T, H * dv, ctx.dtype)
        ops.delta_output(o, self.out_norm_w, s.norm_eps, proj, self.gate_off, gated, H, dv)
        return self.out(ctx, gated, "delta.proj_out")
