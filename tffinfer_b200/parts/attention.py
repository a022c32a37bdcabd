"""Grouped-query attention over the paged cache, with optional per-head RMSNorm of
queries and keys and optional rotary encoding.

Order of operations, as the reference's Qwen3 graph states it
(src/core/model/qwen3/QWen3Creator.cpp:66-140): q,k,v projections without bias ->
reshape to heads -> RMSNorm over head_dim of q and of k with one weight vector each
(:93-101) -> K and V into the cache (:104-108) -> RoPE on q and k -> causal softmax
attention with scale 1/sqrt(head_dim), query head h reading kv head h // (heads/kv_heads)
(src/kernel/cuda/paged_flash_attention.cu:891-892, :1158) -> output projection ->
residual add.  The reference caches un-rotated keys and rotates them on every read;
here keys are rotated once, before they are written, which is algebraically the same.
A ``window`` > 0 lets a query at position p see keys p-window+1 .. p only.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import Mixer, SplitMixer, WeightSpec, MATRIX, VECTOR, KVNeed, StateNeed, LayerContext


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm: bool = True, qk_norm_eps: float = 0.0, window: int = 0,
                 softmax_scale: Optional[float] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.qk_norm = bool(qk_norm)
        self.qk_norm_eps = float(qk_norm_eps)
        self.window = int(window)
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.head_dim)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.qk_norm and not self.qk_norm_eps > 0:
            raise ValueError("qk_norm needs qk_norm_eps > 0")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {
            "q_proj.weight": WeightSpec((self.q_width, self.hidden_size), MATRIX),
            "k_proj.weight": WeightSpec((self.kv_width, self.hidden_size), MATRIX),
            "v_proj.weight": WeightSpec((self.kv_width, self.hidden_size), MATRIX),
            "o_proj.weight": WeightSpec((self.hidden_size, self.q_width), MATRIX),
        }
        if self.qk_norm:
            s["q_norm.weight"] = WeightSpec((self.head_dim,), VECTOR, init="one_plus_normal")
            s["k_norm.weight"] = WeightSpec((self.head_dim,), VECTOR, init="one_plus_normal")
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        q, k, v = tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]
        dt = q.dtype if (q.dtype == k.dtype == v.dtype) else torch.float32
        # one projection instead of three: rows [q heads | k heads | v heads]
        self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        if self.qk_norm:
            self.q_norm_w = tensors["q_norm.weight"]
            self.k_norm_w = tensors["k_norm.weight"]

    def forward(self, h, ctx: LayerContext, residual):
        ops, batch = ctx.ops, ctx.batch
        T = h.shape[0]
        # projection, q/k norm, rotation, cache write and attention: how many kernels that is, is the kernel
        # library's business; the projection's accumulators stay in float32 until q and k have been normalised
        rot = ctx.position.rotary() if ctx.position is not None else None
        attn = torch.empty((T, self.q_width), dtype=h.dtype, device=h.device)
        ops.attend(h, self.w_qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps,
                   rot[0] if rot else None, rot[1] if rot else 0,
                   batch, ctx.block_table, ctx.kv_cache, ctx.kv_layer, ctx.page_size, attn,
                   self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window, ctx.write_cache)
        ops.gemm(attn, self.w_o, residual, residual=residual)
        return residual


@register_part("mixer", "gated_sink_attention")
class GatedSinkAttention(Mixer):
    """Grouped-query attention over the paged cache with what several newer designs add to it, each a parameter:

    * keys/queries of ``head_dim`` and values of ``v_head_dim`` elements;
    * a rotation of part of the head given by the layer's position encoding (``frequencies()``);
    * scores ``(q . k) * softmax_scale``, then ``softcap * tanh(score / softcap)`` when ``softcap`` > 0;
    * a sliding ``window`` (a query at position p sees keys p-window+1 .. p; 0 = all earlier keys);
    * ``sink``: one more term in the softmax's denominator, a key without a value: True, of score 0; "learned", of a
      learned score per head (tensor "sink" [heads]), which is neither scaled nor capped;
    * ``conv_taps`` > 0: a short causal convolution over time on every channel of the projected q, k and v (tensors
      "q_conv", "k_conv", "v_conv" [channels, taps]; y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the
      sequence's start), directly behind the projection; a request's last taps-1 projected rows are kept in a state slot;
    * ``qk_norm`` "whole": an RMS norm over ALL of a token's q (and of its k) at once, with plain weights "q_norm"
      [heads * head_dim] and "k_norm" and ``qk_norm_eps``, behind the convolution and ahead of the rotation;
    * ``value_mix``: "source" leaves this layer's values of the step's tokens in ``ctx.shared[value_key]``;
      "mix" replaces its own by ``(1 - lambda) v + lambda v_source`` with a learned scalar lambda before they are
      cached; "none" does neither;
    * ``head_gate``: every head's output is multiplied by ``sigmoid(W_g h)`` of that head, W_g [heads, hidden], read
      from the mixer's input like the projections.

    The q, k, v and gate projections are one product.  ``names`` gives the tensor names of "q", "k", "v", "o",
    "gate" and "lambda" relative to the prefix."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int = 0,
                 softmax_scale: Optional[float] = None, softcap: float = 0.0, window: int = 0, sink: bool = False,
                 value_mix: str = "none", value_key: str = "values", head_gate: bool = False,
                 lambda_tensor: bool = False, conv_taps: int = 0, qk_norm: str = "none", qk_norm_eps: float = 0.0,
                 names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.v_head_dim = int(v_head_dim) if v_head_dim else int(head_dim)
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.softcap, self.window = float(softcap), int(window)
        if sink not in (False, True, "learned"):
            raise ValueError(f"sink must be False, True or 'learned', got {sink!r}")
        self.sink = sink
        self.conv_taps = int(conv_taps)
        if self.conv_taps < 0 or self.conv_taps > 8:
            raise ValueError(f"conv_taps must lie in 0 .. 8, got {self.conv_taps}")
        if qk_norm not in ("none", "whole"):
            raise ValueError(f"qk_norm must be 'none' or 'whole', got '{qk_norm}'")
        if qk_norm == "whole" and not qk_norm_eps > 0:
            raise ValueError("qk_norm needs qk_norm_eps > 0")
        self.qk_norm, self.qk_norm_eps = qk_norm, float(qk_norm_eps)
        if value_mix not in ("none", "source", "mix"):
            raise ValueError(f"value_mix must be 'none', 'source' or 'mix', got '{value_mix}'")
        self.value_mix, self.value_key, self.head_gate = value_mix, value_key, bool(head_gate)
        self.lambda_tensor = bool(lambda_tensor) or value_mix == "mix"   # a "source" layer may carry an unused one
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                      "gate": "gate_proj.weight", "lambda": "value_lambda", "sink": "sink", "q_conv": "q_conv",
                      "k_conv": "k_conv", "v_conv": "v_conv", "q_norm": "q_norm", "k_norm": "k_norm"}
        self.names.update(names or {})
        self.q_width = self.num_heads * self.head_dim
        self.k_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_kv_heads * self.v_head_dim
        self.cache_dim = max(self.head_dim, self.v_head_dim)     # a cache slot holds a key or a value
        self.w_in = self.w_o = self.lam = self.sink_w = None
        self.conv_w = self.conv_wt = self.norm_w = None

    def cache_need(self):
        kv = KVNeed(self.num_kv_heads, self.cache_dim, self.window)
        if self.conv_taps > 1:        # the projected rows the convolution still needs when the next step comes
            return kv, StateNeed((self.conv_taps - 1, self.q_width + self.k_width + self.v_width), "float32")
        return kv

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        s = {n["q"]: WeightSpec((self.q_width, self.hidden_size), MATRIX),
             n["k"]: WeightSpec((self.k_width, self.hidden_size), MATRIX),
             n["v"]: WeightSpec((self.v_width, self.hidden_size), MATRIX),
             n["o"]: WeightSpec((self.hidden_size, self.num_heads * self.v_head_dim), MATRIX)}
        if self.head_gate:
            s[n["gate"]] = WeightSpec((self.num_heads, self.hidden_size), MATRIX)
        # a layer that mixes nothing may still carry the scalar in a file: it is accepted and not used
        s[n["lambda"]] = WeightSpec((), VECTOR, init="normal", init_scale=0.3, optional=not self.lambda_tensor)
        if self.sink == "learned":
            s[n["sink"]] = WeightSpec((self.num_heads,), VECTOR, init="normal", init_scale=1.0)
        if self.conv_taps > 0:
            for which, width in (("q_conv", self.q_width), ("k_conv", self.k_width), ("v_conv", self.v_width)):
                s[n[which]] = WeightSpec((width, self.conv_taps), VECTOR, init="normal", init_scale=0.5)
        if self.qk_norm == "whole":
            s[n["q_norm"]] = WeightSpec((self.q_width,), VECTOR, init="one_plus_normal")
            s[n["k_norm"]] = WeightSpec((self.k_width,), VECTOR, init="one_plus_normal")
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        if self.head_gate:
            rows.append(tensors[n["gate"]])
        dt = rows[0].dtype if all(r.dtype == rows[0].dtype for r in rows) else torch.float32
        w = torch.cat([r.to(dt) for r in rows], dim=0)
        pad = (-w.shape[0]) % 8               # the product's output rows are stored 16 bytes at a time
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=dt, device=w.device)], dim=0)
        self.w_in = w.contiguous()
        self.gate_off = self.q_width + self.k_width + self.v_width
        self.w_o = tensors[n["o"]]
        if self.lambda_tensor:
            self.lam = tensors[n["lambda"]].reshape(1).contiguous()
        if self.sink == "learned":
            self.sink_w = tensors[n["sink"]].to(torch.float32).contiguous()
        if self.conv_taps > 0:
            self.conv_w = tuple(tensors[n[w]].to(torch.float32).contiguous() for w in ("q_conv", "k_conv", "v_conv"))
            self.conv_wt = tuple(w.t().contiguous() for w in self.conv_w)     # [taps, channels]: the fused kernel's layout
        if self.qk_norm == "whole":
            self.norm_w = (tensors[n["q_norm"]].to(torch.float32).contiguous(), tensors[n["k_norm"]].to(torch.float32).contiguous())

    def forward(self, h, ctx: LayerContext, residual):
        ops, batch = ctx.ops, ctx.batch
        T = h.shape[0]
        freq = ctx.position.frequencies() if ctx.position is not None else None
        share = None
        if self.value_mix == "source":
            share = torch.empty((T, self.v_width), dtype=torch.float32, device=h.device)
            ctx.shared[self.value_key] = share
        elif self.value_mix == "mix":
            share = ctx.shared.get(self.value_key)
            if share is None or tuple(share.shape) != (T, self.v_width):
                raise ValueError(f"value_mix='mix' needs the values of an earlier layer of this step under "
                                 f"'{self.value_key}' with {self.v_width} elements a token")
        attn = torch.empty((T, self.num_heads * self.v_head_dim), dtype=h.dtype, device=h.device)
        pre = None
        if self.conv_taps > 0 or self.qk_norm == "whole":
            pre = dict(taps=max(self.conv_taps, 1), conv=self.conv_w, conv_t=self.conv_wt, norm=self.norm_w, eps=self.qk_norm_eps,
                       state=ctx.state if self.conv_taps > 1 else None)
        ops.attend_gated(h, self.w_in, freq, batch, ctx.block_table, ctx.kv_cache, ctx.kv_layer, ctx.page_size, attn,
                         self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, self.scale, self.window,
                         self.softcap, self.sink_w if self.sink == "learned" else self.sink,
                         {"none": 0, "source": 1, "mix": 2}[self.value_mix], share,
                         self.lam if self.value_mix == "mix" else None,
                         self.gate_off if self.head_gate else -1, ctx.write_cache, pre=pre)
        if residual is None:
            out = ops.sublayer_output(T, self.hidden_size, h.device, h.dtype)
            ops.gemm(attn, self.w_o, out)
            return out
        ops.gemm(attn, self.w_o, residual, residual=residual)
        return residual


@register_part("mixer", "biased_chunk_attention")
class BiasedChunkAttention(SplitMixer):
    """Grouped-query softmax attention whose visibility is causal within blocks of ``chunk`` positions counted from
    position 0 of the sequence (key n is seen from p only if n // chunk == p // chunk; 0 = no blocks) and/or within a
    sliding ``window``, with, each a parameter:

    * scores that carry the positions, ``score(p, n) = (q_p . k_n) * softmax_scale * temp_h - r1_h * ln(1 + r2_h * (p - n))``
      with learned per-head numbers temp (``head_temperature``) and r1, r2 (``distance_bias``);
    * ``projection_bias``: biases of the q, k and v projections (tensors "<name>.b"), added in the projection;
    * ``rotary``: part of every q and k head rotated by the layer's position encoding (``frequencies()``);
    * ``unit_norm_eps`` > 0: every q and k head divided, behind the rotation, by sqrt(mean(x^2) + eps) (an RMS norm
      without a weight);
    * ``softcap`` > 0: the scaled product becomes softcap * tanh(. / softcap).

    Keys of ``head_dim`` and values of ``v_head_dim`` elements.  Everything behind the projections is float32 arithmetic
    (kernels/library.py ``attention_tile``).  The cache keeps what a later query can still see: the last ``chunk`` (or
    ``window``) tokens."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int = 0,
                 softmax_scale: Optional[float] = None, chunk: int = 0, window: int = 0, head_temperature: bool = False,
                 distance_bias: bool = False, projection_bias: bool = False, rotary: bool = False,
                 unit_norm_eps: float = 0.0, softcap: float = 0.0, names: Optional[Dict[str, str]] = None,
                 prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.v_head_dim = int(v_head_dim) if v_head_dim else int(head_dim)
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.chunk, self.window = int(chunk), int(window)
        self.head_temperature, self.distance_bias = bool(head_temperature), bool(distance_bias)
        self.projection_bias, self.rotary = bool(projection_bias), bool(rotary)
        self.unit_norm_eps, self.softcap = float(unit_norm_eps), float(softcap)
        if self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.chunk < 0 or self.window < 0 or self.unit_norm_eps < 0 or self.softcap < 0:
            raise ValueError("chunk, window, unit_norm_eps and softcap must not be negative")
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "temp": "temp", "r1": "r1", "r2": "r2", "q_bias": "q.b",
                      "k_bias": "k.b", "v_bias": "v.b"}
        self.names.update(names or {})
        self.q_width = self.num_heads * self.head_dim
        self.k_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_kv_heads * self.v_head_dim
        self.cache_dim = max(self.head_dim, self.v_head_dim)     # a cache slot holds a key or a value
        self.w_in = self.w_o = self.temp = self.r1 = self.r2 = self.bias = None

    def cache_need(self):
        spans = [s for s in (self.chunk, self.window) if s > 0]
        return KVNeed(self.num_kv_heads, self.cache_dim, min(spans) if spans else 0)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        n = self.names
        s = {n["q"]: WeightSpec((self.q_width, self.hidden_size), MATRIX),
             n["k"]: WeightSpec((self.k_width, self.hidden_size), MATRIX),
             n["v"]: WeightSpec((self.v_width, self.hidden_size), MATRIX),
             n["o"]: WeightSpec((self.hidden_size, self.num_heads * self.v_head_dim), MATRIX)}
        if self.head_temperature:
            s[n["temp"]] = WeightSpec((self.num_heads,), VECTOR, init="one_plus_normal", init_scale=0.2)
        if self.distance_bias:
            s[n["r1"]] = WeightSpec((self.num_heads,), VECTOR, init="one_plus_normal", init_scale=0.2)
            s[n["r2"]] = WeightSpec((self.num_heads,), VECTOR, init="one_plus_normal", init_scale=0.2)
        if self.projection_bias:
            for which, width in (("q_bias", self.q_width), ("k_bias", self.k_width), ("v_bias", self.v_width)):
                s[n[which]] = WeightSpec((width,), VECTOR, init="normal", init_scale=0.3)
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        rows = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        dt = rows[0].dtype if all(r.dtype == rows[0].dtype for r in rows) else torch.float32
        self.w_in = torch.cat([r.to(dt) for r in rows], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.temp = tensors[n["temp"]].contiguous() if self.head_temperature else None
        self.r1 = tensors[n["r1"]].contiguous() if self.distance_bias else None
        self.r2 = tensors[n["r2"]].contiguous() if self.distance_bias else None
        if self.projection_bias:                     # one vector laid out like the projection's q | k | v columns
            self.bias = torch.cat([tensors[n[w]].to(torch.float32) for w in ("q_bias", "k_bias", "v_bias")]).contiguous()

    def input_rows(self):
        return self.w_in

    def mixed_width(self) -> int:
        return self.num_heads * self.v_head_dim

    def output_cols(self):
        return self.w_o

    def mix(self, proj, col, ctx: LayerContext, mixed, mixed_col, out_scale, last_reader) -> None:
        if not ctx.write_cache:
            raise ValueError("biased_chunk_attention writes the keys and values it attends to; a borrowed cache is not supported")
        ops, batch = ctx.ops, ctx.batch
        freq = None
        if self.rotary:
            freq = ctx.position.frequencies() if ctx.position is not None else None
            if freq is None:
                raise ValueError("biased_chunk_attention with rotary=True needs a position encoding that gives frequencies")
            if freq[1] > self.head_dim:
                raise ValueError(f"the rotation covers {freq[1]} dimensions, a head has {self.head_dim}")
        q = torch.empty((proj.shape[0], self.q_width), dtype=mixed.dtype, device=mixed.device)
        ops.qkv_finish(proj, q, None, freq, batch, ctx.block_table, ctx.kv_cache, ctx.kv_layer, ctx.page_size,
                       self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, last_reader=last_reader,
                       proj_off=col, bias=self.bias, unit_eps=self.unit_norm_eps)
        ops.attention_tile(q, batch, ctx.block_table, ctx.kv_cache, ctx.kv_layer, ctx.page_size, mixed, self.num_heads,
                           self.num_kv_heads, self.head_dim, self.v_head_dim, self.scale, window=self.window,
                           chunk=self.chunk, temp=self.temp, r1=self.r1, r2=self.r2, out_scale=out_scale,
                           out_off=mixed_col, softcap=self.softcap)
