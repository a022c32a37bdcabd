"""Gated linear attention: linear attention over a matrix state per head whose rows decay at a rate read from the
input, one rate per key channel and token.

For head h with queries and keys of ``head_dim`` (K) and values of ``v_head_dim`` (V) elements:

    q_t = W_q x_t * K^-1/2      k_t = W_k x_t      v_t = W_v x_t
    z_t = W_a2 (W_a1 x_t) + b                      a low-rank pair of matrices, laid out heads x K
    a_t = sigmoid(z_t)^(1/tau)                     the decay of every key channel, in (0, 1)
    S_t = diag(a_t) S_(t-1) + k_t v_t^T            S [K, V], zero before the request's first token
    o_t = S_t^T q_t
    out = concat_h( o_t / rms(o_t) * w ) * silu(W_g x_t),   rms over the head's V elements with ``eps``, w [V] shared by heads

followed by the output projection.  The state, the decay and everything else behind the projections is float32 in
either mode of the engine: the projections' float32 accumulators go to the recurrence unrounded.  The state is a
``StateNeed``: the engine gives the mixer a [slots, heads * K * V] tensor and the step's slot ids.  ``decay_rank`` is
the inner size of the low-rank pair; 0 takes it from the tensors' shapes."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import Mixer, WeightSpec, MATRIX, VECTOR, StateNeed, LayerContext


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, tau: float, eps: float,
                 decay_rank: int = 0, names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.tau, self.eps, self.decay_rank = float(tau), float(eps), int(decay_rank)
        if min(self.num_heads, self.head_dim, self.v_head_dim) <= 0 or not self.tau > 0 or self.decay_rank < 0:
            raise ValueError("gated_linear_attention: heads and sizes must be positive, tau > 0, decay_rank >= 0")
        self.names = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm", "decay_in": "a1",
                      "decay_out": "a2", "decay_bias": "a2.b"}
        self.names.update(names or {})
        self.qk_width = self.num_heads * self.head_dim
        self.v_width = self.num_heads * self.v_head_dim
        self.w_in = self.w_o = self.w_a1 = self.w_a2 = self.decay_bias = self.norm_w = None

    def cache_need(self):
        return StateNeed((self.num_heads * self.head_dim * self.v_head_dim,), "float32")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n, r = self.names, (self.decay_rank or -1)            # -1: whatever the file holds
        return {n["q"]: WeightSpec((self.qk_width, self.hidden_size), MATRIX),
                n["k"]: WeightSpec((self.qk_width, self.hidden_size), MATRIX),
                n["v"]: WeightSpec((self.v_width, self.hidden_size), MATRIX),
                n["gate"]: WeightSpec((self.v_width, self.hidden_size), MATRIX),
                n["o"]: WeightSpec((self.hidden_size, self.v_width), MATRIX),
                n["norm"]: WeightSpec((self.v_head_dim,), VECTOR, init="one_plus_normal"),
                n["decay_in"]: WeightSpec((r, self.hidden_size), MATRIX),
                n["decay_out"]: WeightSpec((self.qk_width, r), MATRIX, init_scale=0.3),
                n["decay_bias"]: WeightSpec((self.qk_width,), VECTOR, init="normal", init_scale=1.0)}

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]]
        dt = rows[0].dtype if all(r.dtype == rows[0].dtype for r in rows) else torch.float32
        w = torch.cat([r.to(dt) for r in rows], dim=0)
        pad = (-w.shape[0]) % 8               # the product's output rows are stored 16 bytes at a time
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=dt, device=w.device)], dim=0)
        self.w_in = w.contiguous()
        self.gate_off = 2 * self.qk_width + self.v_width
        self.w_o = tensors[n["o"]]
        a1, a2 = tensors[n["decay_in"]], tensors[n["decay_out"]]
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"gated_linear_attention: '{n['decay_in']}' has {a1.shape[0]} rows, '{n['decay_out']}' "
                             f"{a2.shape[1]} columns: the low-rank pair does not fit together")
        if a1.dtype != a2.dtype:
            a1, a2 = a1.to(torch.float32), a2.to(torch.float32)
        pad = (-a1.shape[0]) % 8              # zero rows and columns: the product of the pair is the same
        if pad:
            a1 = torch.cat([a1, torch.zeros((pad, a1.shape[1]), dtype=a1.dtype, device=a1.device)], dim=0)
            a2 = torch.cat([a2, torch.zeros((a2.shape[0], pad), dtype=a2.dtype, device=a2.device)], dim=1)
        self.w_a1, self.w_a2 = a1.contiguous(), a2.contiguous()
        self.decay_bias = tensors[n["decay_bias"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def forward(self, h, ctx: LayerContext, residual):
        if ctx.state is None:
            raise ValueError("gated_linear_attention needs a state tensor (StateNeed)")
        ops = ctx.ops
        T = h.shape[0]
        H, K, V = self.num_heads, self.head_dim, self.v_head_dim
        proj = ops.projection_buffer(T, self.w_in.shape[0], h.device, h.dtype)
        ops.gemm(h, self.w_in, proj)
        low = torch.empty((T, self.w_a1.shape[0]), dtype=h.dtype if self.w_a1.dtype == h.dtype else torch.float32,
                          device=h.device)
        ops.gemm(h, self.w_a1, low)
        raw = torch.empty((T, self.qk_width), dtype=torch.float32, device=h.device)
        ops.gemm(low, self.w_a2, raw)
        o = torch.empty((T, self.v_width), dtype=torch.float32, device=h.device)
        ops.linear_recurrence((proj, 0), (proj, self.qk_width), (proj, 2 * self.qk_width), (raw, 0), ctx.state, ctx.batch,
                              o, H, K, V, "gate", dec_bias=self.decay_bias, inv_tau=1.0 / self.tau, q_scale=float(K) ** -0.5)
        mixed = torch.empty((T, self.v_width), dtype=h.dtype, device=h.device)
        ops.gated_norm(o, V, proj, self.gate_off, self.norm_w, self.eps, False, mixed, clear_cols=(0, proj.shape[1]),
                       last_reader=True)
        if residual is None:
            out = ops.sublayer_output(T, self.hidden_size, h.device, h.dtype)
            ops.gemm(mixed, self.w_o, out)
            return out
        ops.gemm(mixed, self.w_o, residual, residual=residual)
        return residual
