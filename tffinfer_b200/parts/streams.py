"""A residual of several streams (hyper-connections) with layer scale, and the pre-norm arrangement over it.

Instead of one residual x there are S copies x_1 .. x_S, all equal to the embedding output at the start.  A
sublayer with learned vectors a (read), b (write) and a learned matrix M [S, S] does

    u    = sum_s a[s] x_s                      what the sublayer's norm sees
    y    = sublayer(norm(u)) * g               g: layer scale, a learned vector over the width
    x_t <- sum_s M[s, t] x_s + b[t] y          all streams at once from the old ones (M indexed [from, to])

and the model's final norm reads sum_s x_s.  With ``learned`` off, a and b are ones and M the identity: S = 1 is
then the plain pre-norm residual with layer scale.

A write is not run when it is asked for: it is kept until the next read (of the next sublayer, or of the final
norm), and one kernel then updates the streams, combines them and applies that reader's norm
(``ops.stream_step``, csrc/streams.cu).  The streams live for one step only, so the last write before the final
norm is needed at the rows whose logits are wanted and nowhere else.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import Block, Connector, LayerContext, WeightSpec, VECTOR


class ResidualStreams:
    """float32 [T, S, hidden] and at most one write that has not been applied yet."""

    def __init__(self, x: torch.Tensor, ops):
        self.x = x
        self.ops = ops
        self.streams = x.shape[1]
        self.pending = None            # (y, scale, mix, out) of the write that is still to come
        self.pending_bias = None       # a vector [hidden] that is still to be added to every stream, behind that write

    @classmethod
    def from_embedding(cls, token_ids, table, scale: float, streams: int, ops) -> "ResidualStreams":
        x = torch.empty((token_ids.shape[0], streams, table.shape[1]), dtype=torch.float32, device=table.device)
        ops.embed(token_ids, table, x, scale, copies=streams)
        return cls(x, ops)

    @property
    def device(self):
        return self.x.device

    def write(self, y, scale, mix, out) -> None:
        self.flush()                   # (a vector still to be added comes ahead of this write)
        self.pending = (y, scale, mix, out)

    def add_vector(self, vec: torch.Tensor) -> None:
        """x_s <- x_s + vec for every stream (float32 [hidden]); like a write, it runs with the next read."""
        if self.pending_bias is not None:
            self.flush()
        self.pending_bias = vec

    def flush(self) -> None:
        if self.pending is not None or self.pending_bias is not None:
            y, scale, mix, out = self.pending if self.pending is not None else (None, None, None, None)
            bias, self.pending, self.pending_bias = self.pending_bias, None, None
            self.ops.stream_step(self.x, y=y, scale=scale, mix=mix, out=out, bias=bias)

    def read(self, read_w, norm, ops, out_dtype, row_index=None) -> torch.Tensor:
        """norm(sum_s read_w[s] x_s) at every row, or at the rows of ``row_index``; applies the write that is
        still to come in the same kernel.  With ``row_index`` the write feeds the read of those rows only and the
        streams are not updated: that is the model's last read, nothing looks at them afterwards."""
        rows = self.x.shape[0] if row_index is None else row_index.shape[0]
        h = torch.empty((rows, self.x.shape[2]), dtype=out_dtype, device=self.x.device)
        y, scale, mix, out = self.pending if self.pending is not None else (None, None, None, None)
        bias, self.pending, self.pending_bias = self.pending_bias, None, None
        ops.stream_step(self.x, y=y, scale=scale, mix=mix, out=out, read=read_w, norm_weight=norm.weight,
                        eps=norm.eps, h=h, row_index=row_index, bias=bias)
        return h

    def total(self) -> torch.Tensor:
        """sum_s x_s as float32 [T, hidden] (for looking at the residual between layers)."""
        self.flush()
        out = torch.empty((self.x.shape[0], self.x.shape[2]), dtype=torch.float32, device=self.x.device)
        self.ops.stream_step(self.x, total=out)
        return out


@register_part("connector", "hyper_connection")
class HyperConnection(Connector):
    """One sublayer's read vector, write vector, mixing matrix and layer scale.  ``names`` gives the tensor names
    (relative to the prefix) of "read" [S], "write" [S], "mix" [S, S] and "scale" [hidden]."""

    def __init__(self, streams: int, hidden_size: int, learned: bool = True, layer_scale: bool = True,
                 multiplier: float = 1.0, names: Optional[Dict[str, str]] = None, prefix: str = ""):
        super().__init__(prefix)
        self.streams = int(streams)
        self.hidden_size = int(hidden_size)
        self.learned = bool(learned)
        self.layer_scale = bool(layer_scale)
        self.multiplier = float(multiplier)       # a constant that multiplies every write (with the write vector)
        self.names = {"read": "in", "write": "out", "mix": "mix", "scale": "scale"}
        self.names.update(names or {})
        self.read_w = self.write_w = self.mix_w = self.scale_w = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        S, n, s = self.streams, self.names, {}
        if self.learned:
            s[n["read"]] = WeightSpec((S,), VECTOR, init="one_plus_normal", init_scale=0.3)
            s[n["write"]] = WeightSpec((S,), VECTOR, init="one_plus_normal", init_scale=0.3)
            s[n["mix"]] = WeightSpec((S, S), VECTOR, init="eye_plus_normal", init_scale=0.25)
        if self.layer_scale:
            s[n["scale"]] = WeightSpec((self.hidden_size,), VECTOR, init="one_plus_normal", init_scale=0.3)
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        n = self.names
        if self.learned:
            self.read_w, self.write_w, self.mix_w = tensors[n["read"]], tensors[n["write"]], tensors[n["mix"]]
            if self.multiplier != 1.0:
                self.write_w = (self.write_w.to(torch.float32) * self.multiplier).contiguous()
        if self.layer_scale:
            self.scale_w = tensors[n["scale"]]

    def read(self, x: ResidualStreams, norm, ops, out_dtype):
        return x.read(self.read_w, norm, ops, out_dtype)

    def write(self, x: ResidualStreams, y) -> None:
        if self.write_w is None and self.multiplier != 1.0:       # no learned write vector: the constant alone
            self.write_w = torch.full((self.streams,), self.multiplier, dtype=torch.float32, device=x.device)
        x.write(y, self.scale_w, self.mix_w, self.write_w)


@register_part("block", "stream_pre_norm")
class StreamPreNormBlock(Block):
    """Pre-norm sublayers over a residual of streams: the mixer, then the feed-forward if the layer has one, each
    reading and writing through its connector (``connectors["mixer"]``, ``connectors["ffn"]``)."""

    def __init__(self, mixer, feed_forward=None, mixer_norm=None, ffn_norm=None, extra_norms=None, connectors=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, extra_norms, connectors)
        if mixer_norm is None or "mixer" not in self.connectors:
            raise ValueError("the stream_pre_norm arrangement needs mixer_norm and a 'mixer' connector")
        if feed_forward is not None and (ffn_norm is None or "ffn" not in self.connectors):
            raise ValueError("a feed-forward in the stream_pre_norm arrangement needs ffn_norm and an 'ffn' connector")

    def forward(self, x: ResidualStreams, ctx: LayerContext, act_dtype):
        join = self.connectors["mixer"]
        h = join.read(x, self.mixer_norm, ctx.ops, act_dtype)
        join.write(x, self.mixer.forward(h, ctx, residual=None))
        if self.feed_forward is not None:
            join = self.connectors["ffn"]
            h = join.read(x, self.ffn_norm, ctx.ops, act_dtype)
            join.write(x, self.feed_forward.forward(h, ctx, residual=None))
        return x


@register_part("block", "stream_parallel")
class StreamParallelBlock(Block):
    """The mixer and the feed-forward side by side on ONE norm's output: ``x <- write(mixer(h) + feed_forward(h))`` with
    ``h = norm(read(x))``, through the connector ``connectors["layer"]`` (which carries any multiplier of the sum).  The
    feed-forward adds into the mixer's output rows; a layer without a feed-forward is the mixer alone."""

    def __init__(self, mixer, feed_forward=None, mixer_norm=None, ffn_norm=None, extra_norms=None, connectors=None):
        super().__init__(mixer, feed_forward, mixer_norm, ffn_norm, extra_norms, connectors)
        if mixer_norm is None or "layer" not in self.connectors:
            raise ValueError("the stream_parallel arrangement needs mixer_norm and a 'layer' connector")
        if ffn_norm is not None:
            raise ValueError("the stream_parallel arrangement has one norm: both sublayers read its output")

    def forward(self, x: ResidualStreams, ctx: LayerContext, act_dtype):
        join = self.connectors["layer"]
        h = join.read(x, self.mixer_norm, ctx.ops, act_dtype)
        y = self.mixer.forward(h, ctx, residual=None)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(h, ctx, residual=y)
        join.write(x, y)
        return x
