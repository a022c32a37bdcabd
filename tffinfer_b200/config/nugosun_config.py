"""Typed configuration of the Nugosun design: a decoder-only model whose config.json lists its layers one by one.
A layer's mixer is ``gla`` (gated linear attention), ``parallel`` (a chunked rotary attention beside a Mamba-2 state
space) or ``latent_attention``; its feed-forward is dense, a mixture of experts, or absent.

    {"architecture": "Nugosun", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask": {"size"},
                                    "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}},
                           "right": {"heads", "vdim", "state", "groups", "conv", "norm_groups"},
                           "left_scale", "right_scale"}, "mlp": ...},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot": {"base", "dims"},
                           "kv_from": j (optional)}, "mlp": ...}, ...]}
    "mlp": {"kind": "dense", "ff": F} | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}} | null

Every size and constant of a checkpoint comes from there or from a tensor's shape (the inner size of the low-rank pair
that makes a gla layer's decay; ``rank`` gives it where weights are made at random).  Optional keys: ``embedding.scale``
(absent: 1), ``kv_heads`` (absent: heads), ``mask`` (absent: all earlier keys), ``softcap`` (absent or 0: none), ``rot``
of the left mixer and ``rot.scaling`` (absent: no rotation / plain frequencies), ``scale`` (absent: dim^-1/2; latent:
(dim + rot_dim)^-1/2), ``groups`` and ``norm_groups`` (absent: 1), ``left_scale`` / ``right_scale`` (absent: 1),
``rot.dims`` of a latent layer (absent: rot_dim), ``kv_from``, ``max_position`` (absent: MAX_POSITION_DEFAULT; the
design itself has no limit, the engine's block tables need one)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .model_config import ModelConfig, ConfigError, architecture_name
from .tipezen_config import _need, _int, _float, RotaryConfig, MAX_POSITION_DEFAULT


@dataclass(frozen=True)
class NugosunMlp:
    kind: str                          # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0

    @staticmethod
    def read(d, where: str) -> Optional["NugosunMlp"]:
        if d is None:
            return None
        kind = _need(d, "kind", where)
        if kind == "dense":
            m = NugosunMlp("dense", _int(d, "ff", where))
        elif kind == "moe":
            r = _need(d, "router", where)
            m = NugosunMlp("moe", _int(_need(d, "expert", where), "ff", where + ".expert"),
                           _int(r, "experts", where + ".router"), _int(r, "top", where + ".router"))
            if not 0 < m.top <= m.experts:
                raise ConfigError(f"config.json: {where}.router: 1 <= top <= experts is required")
        else:
            raise ConfigError(f"config.json: {where}.kind '{kind}' is not a feed-forward of this design (dense, moe)")
        if m.ff <= 0:
            raise ConfigError(f"config.json: {where}: ff must be positive")
        return m

    def to_json(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class NugosunGla:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0                      # inner size of the decay's low-rank pair; 0: the tensors' shapes say


@dataclass(frozen=True)
class NugosunAttention:                # the left mixer of a parallel layer
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0
    chunk: int = 0                     # mask.size; 0 = all earlier keys
    rot: Optional[RotaryConfig] = None


@dataclass(frozen=True)
class NugosunStateSpace:               # the right mixer of a parallel layer
    heads: int
    vdim: int
    state: int
    groups: int = 1
    conv: int = 1
    norm_groups: int = 1


@dataclass(frozen=True)
class NugosunLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class NugosunLayer:
    type: str                          # "gla" | "parallel" | "latent_attention"
    gla: Optional[NugosunGla] = None
    left: Optional[NugosunAttention] = None
    right: Optional[NugosunStateSpace] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    latent: Optional[NugosunLatent] = None
    mlp: Optional[NugosunMlp] = None


def _positive(where: str, **values) -> None:
    bad = [k for k, v in values.items() if not v > 0]
    if bad:
        raise ConfigError(f"config.json: {where}: {', '.join(bad)} must be positive")


@dataclass(frozen=True)
class NugosunConfig(ModelConfig):
    vocab_size: int = 0
    hidden_size: int = 0
    embed_scale: float = 1.0
    norm_eps: float = 0.0
    layers: Tuple[NugosunLayer, ...] = ()
    max_position: int = MAX_POSITION_DEFAULT

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_json_dict(d: Dict[str, Any]) -> "NugosunConfig":
        raw = _need(d, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            m = _need(l, "mixer", where)
            mw = where + ".mixer"
            mlp = NugosunMlp.read(l.get("mlp"), where + ".mlp")
            if kind == "gla":
                g = NugosunGla(_int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw), _float(m, "tau", mw),
                               _int(m, "rank", mw, 0))
                _positive(mw, heads=g.heads, dim=g.dim, vdim=g.vdim, tau=g.tau)
                layer = NugosunLayer(kind, gla=g, mlp=mlp)
            elif kind == "parallel":
                L, R = _need(m, "left", mw), _need(m, "right", mw)
                lw, rw = mw + ".left", mw + ".right"
                heads, dim = _int(L, "heads", lw), _int(L, "dim", lw)
                _positive(lw, heads=heads, dim=dim)
                mask = L.get("mask")
                left = NugosunAttention(
                    heads, _int(L, "kv_heads", lw, heads), dim, _int(L, "vdim", lw), _float(L, "scale", lw, dim ** -0.5),
                    _float(L, "softcap", lw, 0.0), _int(mask, "size", lw + ".mask") if mask is not None else 0,
                    RotaryConfig.read(L.get("rot"), lw + ".rot"))
                _positive(lw, kv_heads=left.kv_heads, vdim=left.vdim)
                if left.heads % left.kv_heads:
                    raise ConfigError(f"config.json: {lw}: heads ({left.heads}) must be a multiple of kv_heads ({left.kv_heads})")
                if left.chunk < 0 or left.softcap < 0:
                    raise ConfigError(f"config.json: {lw}: mask.size and softcap must not be negative")
                if left.rot is not None and left.rot.dims > left.dim:
                    raise ConfigError(f"config.json: {lw}.rot: 'dims' ({left.rot.dims}) exceeds dim ({left.dim})")
                right = NugosunStateSpace(_int(R, "heads", rw), _int(R, "vdim", rw), _int(R, "state", rw),
                                          _int(R, "groups", rw, 1), _int(R, "conv", rw, 1), _int(R, "norm_groups", rw, 1))
                _positive(rw, heads=right.heads, vdim=right.vdim, state=right.state, groups=right.groups, conv=right.conv,
                          norm_groups=right.norm_groups)
                if right.heads % right.groups or (right.heads * right.vdim) % right.norm_groups:
                    raise ConfigError(f"config.json: {rw}: groups must divide heads, norm_groups must divide heads * vdim")
                layer = NugosunLayer(kind, left=left, right=right, left_scale=_float(m, "left_scale", mw, 1.0),
                                     right_scale=_float(m, "right_scale", mw, 1.0), mlp=mlp)
            elif kind == "latent_attention":
                rot_dim, dim = _int(m, "rot_dim", mw), _int(m, "dim", mw)
                _positive(mw, dim=dim, rot_dim=rot_dim)
                rd = dict(_need(m, "rot", mw))
                rd.setdefault("dims", rot_dim)
                la = NugosunLatent(_int(m, "heads", mw), dim, rot_dim, _int(m, "vdim", mw), _int(m, "q_rank", mw),
                                   _int(m, "kv_rank", mw), _float(m, "scale", mw, (dim + rot_dim) ** -0.5),
                                   RotaryConfig.read(rd, mw + ".rot"),
                                   _int(m, "kv_from", mw) if m.get("kv_from") is not None else None)
                _positive(mw, heads=la.heads, vdim=la.vdim, q_rank=la.q_rank, kv_rank=la.kv_rank)
                if la.rot.dims > rot_dim:
                    raise ConfigError(f"config.json: {mw}.rot: 'dims' ({la.rot.dims}) exceeds rot_dim ({rot_dim})")
                if la.kv_from is not None:
                    j = la.kv_from
                    src = layers[j].latent if 0 <= j < i else None
                    if src is None or src.kv_from is not None:
                        raise ConfigError(f"config.json: {mw}.kv_from must name an earlier latent_attention layer that "
                                          f"keeps a cache of its own, got {j}")
                    if (src.kv_rank, src.rot_dim, src.rot) != (la.kv_rank, la.rot_dim, la.rot):
                        raise ConfigError(f"config.json: {mw}: kv_rank, rot_dim and rot must equal those of layer {j}")
                layer = NugosunLayer(kind, latent=la, mlp=mlp)
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design "
                                  f"(gla, parallel, latent_attention)")
            layers.append(layer)
        emb = d.get("embedding") or {}
        cfg = NugosunConfig(
            architecture=architecture_name(d), vocab_size=_int(d, "vocab", "the top level"),
            hidden_size=_int(d, "width", "the top level"), embed_scale=_float(emb, "scale", "embedding", 1.0),
            norm_eps=_float(_need(d, "norm", "the top level"), "eps", "norm"), layers=tuple(layers),
            max_position=_int(d, "max_position", "the top level", MAX_POSITION_DEFAULT))
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive, norm.eps > 0")
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        out = []
        for l in self.layers:
            if l.type == "gla":
                g = l.gla
                m: Dict[str, Any] = {"heads": g.heads, "dim": g.dim, "vdim": g.vdim, "tau": g.tau}
                if g.rank:
                    m["rank"] = g.rank
            elif l.type == "parallel":
                a, s = l.left, l.right
                left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                                        "scale": a.scale, "softcap": a.softcap}
                if a.chunk > 0:
                    left["mask"] = {"size": a.chunk}
                if a.rot is not None:
                    left["rot"] = a.rot.to_json()
                m = {"left": left, "left_scale": l.left_scale, "right_scale": l.right_scale,
                     "right": {"heads": s.heads, "vdim": s.vdim, "state": s.state, "groups": s.groups, "conv": s.conv,
                               "norm_groups": s.norm_groups}}
            else:
                a = l.latent
                m = {"heads": a.heads, "dim": a.dim, "rot_dim": a.rot_dim, "vdim": a.vdim, "q_rank": a.q_rank,
                     "kv_rank": a.kv_rank, "scale": a.scale, "rot": a.rot.to_json()}
                if a.kv_from is not None:
                    m["kv_from"] = a.kv_from
            out.append({"type": l.type, "mixer": m, "mlp": l.mlp.to_json() if l.mlp is not None else None})
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embed_scale}, "norm": {"eps": self.norm_eps}, "layers": out}
        if self.max_position != MAX_POSITION_DEFAULT:
            d["max_position"] = self.max_position
        return d
