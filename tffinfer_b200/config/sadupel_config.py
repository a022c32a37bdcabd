"""Typed configuration of the Sadupel design: a decoder-only model whose config.json lists its layers one by one.  A
layer is one RMS norm whose output feeds an attention mixer and a mixture of experts side by side; their sum, times
``residual_mult``, joins the residual.  A range of layers may run several times in a row (``loop``), every pass with
caches of its own and a learned vector added to the residual ahead of it.  A table indexed by a hash of the previous
and the current token is added to the token embedding.

    {"architecture": "Sadupel", "vocab": V, "width": W, "residual_mult": m, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "loop": {"start": i, "stop": j, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv": taps, "scale", "softcap",
                           "rot": {"base", "dims", "scaling": {"factor"}}},
                 "mlp": {"kind": "moe", "expert": {"ff"}, "shared": {"ff"},
                         "router": {"experts", "top", "identity", "groups": {"count", "keep"}}} | null}, ...]}

Every size and constant of a checkpoint comes from there.  Optional keys: ``residual_mult`` (absent: 1),
``embedding.bigram`` (absent: no such table), ``loop`` (absent: every layer runs once), ``kv_heads`` (absent: heads),
``vdim`` (absent: dim), ``conv`` (absent or 0: no convolution), ``softcap`` (absent or 0: none), ``rot.dims`` (absent:
dim), ``rot.scaling`` (absent: factor 1), ``router.identity`` (absent: 0), ``router.groups`` (absent: one group),
``shared`` (absent or null: no shared expert), ``max_position`` (absent: MAX_POSITION_DEFAULT; the design itself has no
limit, the engine's block tables need one)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ModelConfig, ConfigError
from .tipezen_config import _need, _int, _float, MAX_POSITION_DEFAULT

MAX_CONV_TAPS = 8          # what the convolution kernel unrolls a channel's window to


@dataclass(frozen=True)
class SadupelExperts:
    ff: int
    experts: int
    top: int
    identity: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0


@dataclass(frozen=True)
class SadupelLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    softcap: float
    rot_base: float
    rot_dims: int
    rot_factor: float
    mlp: Optional[SadupelExperts] = None
    type: str = "attention"


@dataclass(frozen=True)
class SadupelConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    bigram: Optional[Tuple[int, int, int]] = None        # (buckets, mul_prev, mul_cur)
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)
    layers: Tuple[SadupelLayer, ...] = ()
    max_position: int = MAX_POSITION_DEFAULT

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def runs(self):
        """(layer, pass number or None) in the order the layers run; the pass number stands at the first layer of each
        pass of the loop."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, None) for i in range(start)]
        for t in range(times):
            out += [(i, t if i == start else None) for i in range(start, stop)]
        return out + [(i, None) for i in range(stop, n)]

    @staticmethod
    def from_json_dict(d: Dict[str, Any]) -> "SadupelConfig":
        from .model_config import architecture_name
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            if kind != "attention":
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design (attention)")
            m = _need(l, "mixer", where)
            mw = where + ".mixer"
            mlp = l.get("mlp")
            ex = None
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind '{mlp.get('kind')}' is not supported (moe only)")
                r = _need(mlp, "router", where + ".mlp")
                rw = where + ".mlp.router"
                g = r.get("groups") or {}
                shared = mlp.get("shared")
                ex = SadupelExperts(ff=_int(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert"),
                                    experts=_int(r, "experts", rw), top=_int(r, "top", rw),
                                    identity=_int(r, "identity", rw, 0), groups=_int(g, "count", rw + ".groups", 1),
                                    keep=_int(g, "keep", rw + ".groups", 1) if g else 1,
                                    shared_ff=_int(shared, "ff", where + ".mlp.shared") if shared is not None else 0)
                outputs = ex.experts + ex.identity
                if ex.ff <= 0 or ex.experts <= 0 or ex.identity < 0 or ex.shared_ff < 0 or not 0 < ex.top <= outputs:
                    raise ConfigError(f"config.json: {where}.mlp: ff and experts must be positive and 1 <= top <= experts + identity")
                if ex.groups < 1 or not 1 <= ex.keep <= ex.groups or outputs % ex.groups or ex.top > ex.keep * (outputs // ex.groups):
                    raise ConfigError(f"config.json: {rw}.groups: 'count' must divide experts + identity ({outputs}), "
                                      f"1 <= keep <= count, and the kept groups must hold at least 'top' outputs")
            rot = _need(m, "rot", mw)
            heads = _int(m, "heads", mw)
            dim = _int(m, "dim", mw)
            layer = SadupelLayer(
                heads=heads, kv_heads=_int(m, "kv_heads", mw, heads), dim=dim, vdim=_int(m, "vdim", mw, dim),
                conv=_int(m, "conv", mw, 0), scale=_float(m, "scale", mw), softcap=_float(m, "softcap", mw, 0.0),
                rot_base=_float(rot, "base", mw + ".rot"), rot_dims=_int(rot, "dims", mw + ".rot", dim),
                rot_factor=_float(rot.get("scaling") or {}, "factor", mw + ".rot.scaling", 1.0), mlp=ex)
            if layer.kv_heads <= 0 or heads <= 0 or heads % layer.kv_heads:
                raise ConfigError(f"config.json: {mw}: heads ({heads}) must be a multiple of kv_heads ({layer.kv_heads})")
            if min(layer.dim, layer.vdim) <= 0 or layer.softcap < 0 or not 0 <= layer.conv <= MAX_CONV_TAPS:
                raise ConfigError(f"config.json: {mw}: dim and vdim must be positive, softcap >= 0, 0 <= conv <= {MAX_CONV_TAPS}")
            if layer.rot_dims <= 0 or layer.rot_dims % 2 or layer.rot_dims > dim or not layer.rot_base > 0 or not layer.rot_factor > 0:
                raise ConfigError(f"config.json: {mw}.rot: 'dims' must be even, positive and at most dim, 'base' and the "
                                  f"scaling factor positive")
            layers.append(layer)
        bigram = (d.get("embedding") or {}).get("bigram")
        bg = None
        if bigram is not None:
            bg = (_int(bigram, "buckets", "embedding.bigram"), _int(bigram, "mul_prev", "embedding.bigram"),
                  _int(bigram, "mul_cur", "embedding.bigram"))
            if bg[0] <= 0:
                raise ConfigError("config.json: embedding.bigram.buckets must be positive")
        loop = d.get("loop")
        lp = None
        if loop is not None:
            lp = (_int(loop, "start", "loop"), _int(loop, "stop", "loop"), _int(loop, "times", "loop"))
            if not 0 <= lp[0] < lp[1] <= len(layers) or lp[2] < 1:
                raise ConfigError(f"config.json: loop: 0 <= start < stop <= {len(layers)} layers and times >= 1, got {lp}")
        cfg = SadupelConfig(
            architecture=architecture_name(d), vocab_size=_int(d, "vocab", "the top level"),
            hidden_size=_int(d, "width", "the top level"), norm_eps=_float(_need(d, "norm", "the top level"), "eps", "norm"),
            residual_mult=_float(d, "residual_mult", "the top level", 1.0), bigram=bg, loop=lp, layers=tuple(layers),
            max_position=_int(d, "max_position", "the top level", MAX_POSITION_DEFAULT))
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive and norm.eps > 0")
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        out = []
        for l in self.layers:
            m: Dict[str, Any] = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "conv": l.conv,
                                 "scale": l.scale, "softcap": l.softcap,
                                 "rot": {"base": l.rot_base, "dims": l.rot_dims, "scaling": {"factor": l.rot_factor}}}
            mlp = None
            if l.mlp is not None:
                e = l.mlp
                mlp = {"kind": "moe", "expert": {"ff": e.ff},
                       "router": {"experts": e.experts, "top": e.top, "identity": e.identity,
                                  "groups": {"count": e.groups, "keep": e.keep}},
                       "shared": {"ff": e.shared_ff} if e.shared_ff > 0 else None}
            out.append({"type": l.type, "mixer": m, "mlp": mlp})
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps}, "layers": out}
        if self.bigram is not None:
            d["embedding"] = {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_position != MAX_POSITION_DEFAULT:
            d["max_position"] = self.max_position
        return d
