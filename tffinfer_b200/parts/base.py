"""Interfaces of the parts a layer is put together from.

Each part is constructed with its sizes and constants as keyword parameters, says
which tensors it wants (:meth:`Part.weight_specs`), receives them
(:meth:`Part.load`) and runs on the flat token rows of one step.  The kernels come
in through ``ops`` (kernels/library.py): a part never touches a device API itself.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch

# --- weights -----------------------------------------------------------------
MATRIX = "matrix"      # operand of a matrix product: held in the engine's compute dtype
VECTOR = "vector"      # small per-channel parameters (norm weights): always held in float32
INT_TABLE = "int"      # integer tables: held in int32


@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]                # a dimension of -1: whatever the file holds (random weights cannot be made then)
    role: str = MATRIX
    init: str = "normal"          # random-weights mode: "normal" | "one_plus_normal" | "eye_plus_normal" | "zeros"
    init_scale: Optional[float] = None   # std; None = the model's init_std (normal) or 0.1 (one_plus_normal)
    optional: bool = False               # a file may hold it or not (the part does not use it); never made at random


# --- cache needs ---------------------------------------------------------------
@dataclass(frozen=True)
class KVNeed:
    """Keys and values of every token (window == 0) or of the last ``window`` tokens.  ``planes`` 2: a page holds a
    plane of keys and a plane of values, slots of ``head_dim`` elements each; 1: one plane, a token's slot is one
    vector of ``head_dim`` elements from which the mixer makes both (a latent cache)."""
    num_kv_heads: int
    head_dim: int
    window: int = 0
    planes: int = 2


@dataclass(frozen=True)
class StateNeed:
    """A per-request state of fixed size (``shape`` elements of ``dtype`` per request)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


# --- run-time contexts ---------------------------------------------------------
@dataclass
class LayerContext:
    """What one run of one layer sees of the step.

    batch        the step's StepBatch (engine/batch.py): tokens, positions, per-request rows
    ops          the kernel library
    kv_cache     tensor [pages, layers_in_group, 2, kv_heads, page_size, head_dim] or None
    kv_layer     this run's index along the second axis of kv_cache
    block_table  int32 [requests_in_step, max_blocks] of the run's cache group, or None
    page_size    tokens per page
    write_cache  False when this run reads another run's cache
    state        tensor [slots, *StateNeed.shape] of this run, or None
    position     the layer's position-encoding part, or None
    shared       a dict that lives for one step, the same object for every layer run: a mixer may leave
                 tensors of this step's tokens there for the layers behind it (values that later layers mix
                 into their own, for instance)
    """
    batch: Any
    ops: Any
    kv_cache: Optional[torch.Tensor] = None
    kv_layer: int = 0
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    write_cache: bool = True
    state: Optional[torch.Tensor] = None
    position: Any = None
    shared: Optional[Dict[str, Any]] = None    # lives for one step: what a layer leaves for later layers of the step


class Part:
    """Base of every part.  ``prefix`` is prepended to the names in weight_specs()."""
    family = ""
    kind = ""

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Tensor names (relative to the prefix) -> what is expected in the file."""
        return {}

    def full_name(self, rel: str) -> str:
        return f"{self.prefix}.{rel}" if self.prefix else rel

    def load(self, tensors: Dict[str, torch.Tensor], ops, act_dtype: torch.dtype) -> None:
        """Receive the tensors named by weight_specs() (relative names), already on the
        device and in the dtype their role asks for.  Merging happens here."""


class Norm(Part):
    """x: float32 [rows, dim] -> activation dtype [rows or len(row_index), dim]."""
    def forward(self, x: torch.Tensor, ops, out_dtype: torch.dtype,
                row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into something a mixer applies.  ``prepare`` runs once after
    loading (tables); ``embed`` may change the residual stream after the embedding
    (absolute encodings); rotary encodings expose ``rotary()`` for mixers."""
    def prepare(self, ops, device, max_position: int) -> None:
        pass

    def embed(self, x: torch.Tensor, batch, ops) -> torch.Tensor:
        return x

    def rotary(self):
        """(cos_sin table float32 [max_position, rot_dim/2, 2], rot_dim) or None."""
        return None

    def frequencies(self):
        """For rotations computed from the position on the fly: (frequencies float32 [rot_dim/2] on the device,
        rot_dim, magnitude of cos and sin, interleaved pairs or halves), or None."""
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here).

    cache_need() -> KVNeed | StateNeed | None, or a tuple (KVNeed, StateNeed) for a mixer that keeps both (two
    mixers side by side): the layer context then carries pages and a state
    forward(h, ctx, residual) -> float32 [T, hidden]: residual + mixer(h); with ``residual`` None, mixer(h)
    alone in a tensor of its own (arrangements that do something else with it than add it to one stream).
    """
    def cache_need(self):
        return None

    def forward(self, h: torch.Tensor, ctx: LayerContext, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class SplitMixer(Mixer):
    """A mixer of the shape  input projection -> token mixing -> output projection  that lets somebody else run the
    two projections: several such mixers side by side then share ONE input product and ONE output product
    (parts/parallel.py).  After ``load``:

    input_rows()    the rows of its input projection [n_in, hidden] (its columns of the shared product, in its order)
    mixed_width()   how many columns its mixed activation has
    output_cols()   its output projection [hidden, mixed_width]
    mix(proj, col, ctx, mixed, mixed_col, out_scale, last_reader)
                    reads columns col .. col + n_in of the float32 rows ``proj`` (the product's accumulators) and writes
                    ``out_scale`` times its mixed activation into columns mixed_col .. of ``mixed`` (activation type).
                    ``last_reader``: nothing of the rows is left for anybody else (accumulator buffers that are kept at
                    zero between uses count as clean again).

    ``forward`` runs the same three steps alone."""
    def input_rows(self) -> torch.Tensor:
        raise NotImplementedError

    def mixed_width(self) -> int:
        raise NotImplementedError

    def output_cols(self) -> torch.Tensor:
        raise NotImplementedError

    def mix(self, proj, col: int, ctx: LayerContext, mixed, mixed_col: int, out_scale: float, last_reader: bool) -> None:
        raise NotImplementedError

    @staticmethod
    def padded_rows(w: torch.Tensor) -> torch.Tensor:
        pad = (-w.shape[0]) % 8               # a product's output rows are stored 16 bytes at a time
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        return w.contiguous()

    def forward(self, h, ctx: LayerContext, residual):
        ops = ctx.ops
        T = h.shape[0]
        w_in = getattr(self, "_w_in_alone", None)
        if w_in is None:
            w_in = self._w_in_alone = self.padded_rows(self.input_rows())
        proj = ops.projection_buffer(T, w_in.shape[0], h.device, h.dtype)
        ops.gemm(h, w_in, proj)
        mixed = torch.empty((T, self.mixed_width()), dtype=h.dtype, device=h.device)
        self.mix(proj, 0, ctx, mixed, 0, 1.0, True)
        if residual is None:
            out = ops.sublayer_output(T, self.output_cols().shape[0], h.device, h.dtype)
            ops.gemm(mixed, self.output_cols(), out)
            return out
        ops.gemm(mixed, self.output_cols(), residual, residual=residual)
        return residual


class FeedForward(Part):
    """forward(h, ctx, residual) -> float32 [T, hidden]: residual + f(h); with ``residual`` None, f(h) alone."""
    def forward(self, h: torch.Tensor, ctx: LayerContext, residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class EmbeddingExtra(Part):
    """Something added to the token embedding's output before the first layer (registry family "embedding").

    state_need() -> StateNeed | None: what it keeps per request between steps (the previous token, say)
    forward(x, batch, ops, state, copies): adds to x, float32 [T, hidden] (copies == 0) or [T, copies, hidden] with
    every copy getting the same; ``state`` is its [slots, ...] tensor, indexed with batch.slots on the device.
    """
    def state_need(self):
        return None

    def forward(self, x: torch.Tensor, batch, ops, state, copies: int = 0) -> None:
        raise NotImplementedError


class Connector(Part):
    """How a sublayer reads its input from the residual and how its output joins it, where that is more than
    ``norm(x)`` and ``x + y``: the residual is then a :class:`parts.streams.ResidualStreams`.

    read(x, norm, ops, out_dtype) -> activation rows [T, hidden]
    write(x, y) -> None (x is updated; the update may be deferred to the next read)
    """
    def read(self, x, norm, ops, out_dtype):
        raise NotImplementedError

    def write(self, x, y) -> None:
        raise NotImplementedError


class Block:
    """An arrangement of a mixer, a feed-forward and norms around the residual stream.  Which norms there
    are is the arrangement's business: the two of the pre-norm arrangement have names of their own, any
    others come in ``extra_norms`` under the names the layer's description gave them."""
    family = "block"
    kind = ""

    def __init__(self, mixer: Mixer, feed_forward: Optional[FeedForward], mixer_norm: Optional[Norm] = None,
                 ffn_norm: Optional[Norm] = None, extra_norms: Optional[Dict[str, Norm]] = None,
                 connectors: Optional[Dict[str, "Connector"]] = None):
        self.mixer = mixer
        self.feed_forward = feed_forward          # None: the layer has no feed-forward (where the arrangement allows)
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm
        self.extra_norms = dict(extra_norms or {})
        self.connectors = dict(connectors or {})  # by a name of the arrangement's choosing

    def parts(self):
        named = [self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward] + list(self.extra_norms.values()) + \
                list(self.connectors.values())
        return [p for p in named if p is not None]

    def forward(self, x: torch.Tensor, ctx: LayerContext, act_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError
