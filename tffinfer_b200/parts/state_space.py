"""A selective state space mixer in the state-space-duality form (Mamba-2): a linear recurrence over a matrix state per
head with one decay per head and token, read from the input.

With heads of ``head_dim`` (P) channels, a state of ``state_size`` (N) rows and ``groups`` groups of heads that share B
and C (inner = heads * P, head h uses group h // (heads / groups)):

    [z | x | B | C | dt] = W_in h                          inner | inner | groups*N | groups*N | heads columns
    [x | B | C] <- silu(conv(. ) + conv bias)              a causal convolution of ``conv_taps`` taps on every channel
    dt = softplus(dt + dt_bias)                            per head, no clamp
    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T     S [N, P], zero before the request's first token
    y_t = S_t^T C_t + D_h x_t
    out = W_o ( rms_parts(y * silu(z)) * w )               the gate ahead of the norm; ``norm_groups`` equal parts of the
                                                           inner row, each divided by its own root mean square (``eps``)

Everything behind the input product is float32 in either mode of the engine (the product's accumulators go to the
convolution and the recurrence unrounded).  The mixer keeps one ``StateNeed`` of float32 per request: the last
conv_taps - 1 rows of [x | B | C] ahead of the convolution, then the heads' states.  It is a :class:`SplitMixer`: beside
another mixer (parts/parallel.py) its input and output products are shared."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import SplitMixer, WeightSpec, MATRIX, VECTOR, StateNeed, LayerContext


@register_part("mixer", "selective_state_space")
class SelectiveStateSpace(SplitMixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float, names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.state_size, self.groups, self.conv_taps = int(state_size), int(groups), int(conv_taps)
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        if min(self.num_heads, self.head_dim, self.state_size, self.groups, self.norm_groups) <= 0:
            raise ValueError("selective_state_space: heads, sizes and groups must be positive")
        if self.num_heads % self.groups:
            raise ValueError(f"selective_state_space: heads ({self.num_heads}) must be a multiple of groups ({self.groups})")
        if not 1 <= self.conv_taps <= 16:
            raise ValueError(f"selective_state_space: conv_taps must lie in 1 .. 16, got {self.conv_taps}")
        self.inner = self.num_heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"selective_state_space: norm_groups ({self.norm_groups}) must divide heads * head_dim ({self.inner})")
        self.bc = self.groups * self.state_size
        self.channels = self.inner + 2 * self.bc                       # what the convolution runs over: [x | B | C]
        self.in_rows = 2 * self.inner + 2 * self.bc + self.num_heads
        self.conv_state = (self.conv_taps - 1) * self.channels
        self.names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "rate": "A_log", "skip": "D",
                      "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.rate_log = self.skip = self.norm_w = None

    def cache_need(self):
        return StateNeed((self.conv_state + self.num_heads * self.state_size * self.head_dim,), "float32")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        return {n["in"]: WeightSpec((self.in_rows, self.hidden_size), MATRIX),
                n["conv"]: WeightSpec((self.channels, self.conv_taps), VECTOR, init="normal", init_scale=0.5),
                n["conv_bias"]: WeightSpec((self.channels,), VECTOR, init="normal", init_scale=0.2),
                n["dt_bias"]: WeightSpec((self.num_heads,), VECTOR, init="normal", init_scale=1.0),
                n["rate"]: WeightSpec((self.num_heads,), VECTOR, init="normal", init_scale=0.7),
                n["skip"]: WeightSpec((self.num_heads,), VECTOR, init="one_plus_normal", init_scale=0.3),
                n["norm"]: WeightSpec((self.inner,), VECTOR, init="one_plus_normal"),
                n["o"]: WeightSpec((self.hidden_size, self.inner), MATRIX)}

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.w_in, self.w_o = tensors[n["in"]], tensors[n["o"]]
        self.conv_w, self.conv_b = f32(tensors[n["conv"]]), f32(tensors[n["conv_bias"]])
        self.dt_bias, self.rate_log, self.skip = f32(tensors[n["dt_bias"]]), f32(tensors[n["rate"]]), f32(tensors[n["skip"]])
        self.norm_w = f32(tensors[n["norm"]])

    def input_rows(self):
        return self.w_in

    def mixed_width(self) -> int:
        return self.inner

    def output_cols(self):
        return self.w_o

    def mix(self, proj, col, ctx: LayerContext, mixed, mixed_col, out_scale, last_reader) -> None:
        if ctx.state is None:
            raise ValueError("selective_state_space needs a state tensor (StateNeed)")
        ops, batch = ctx.ops, ctx.batch
        T = proj.shape[0]
        H, P, N = self.num_heads, self.head_dim, self.state_size
        xbc = torch.empty((T, self.channels), dtype=torch.float32, device=proj.device)
        if not ops.causal_conv(proj, col + self.inner, self.channels, self.conv_w, self.conv_b, "silu", ctx.state, 0, batch,
                               xbc, update_state=True):          # single tokens: the rows move up in the same kernel
            ops.causal_conv_state(proj, col + self.inner, self.channels, self.conv_taps, ctx.state, 0, batch)
        y = torch.empty((T, self.inner), dtype=torch.float32, device=proj.device)
        ops.linear_recurrence((xbc, self.inner + self.bc), (xbc, self.inner), (xbc, 0),
                              (proj, col + 2 * self.inner + 2 * self.bc), ctx.state, batch, y, H, N, P, "step",
                              share=H // self.groups, dec_bias=self.dt_bias, rate_log=self.rate_log, skip=self.skip,
                              state_off=self.conv_state)
        ops.gated_norm(y, self.inner // self.norm_groups, proj, col, self.norm_w, self.eps, True, mixed, mixed_col,
                       out_scale, clear_cols=(col, proj.shape[1] if last_reader else col + self.in_rows),
                       last_reader=last_reader)
