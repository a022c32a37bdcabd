"""Nugosun as a model description: a decoder-only design whose layers are listed one by one in config.json.  A layer
adds both of its sublayers to the residual at once, each behind an RMS norm of its own that reads the same residual
(``x + mixer(norm1 x) + ff(norm2 x)``; norm weights stored around zero, multiplier 1 + w).  Its mixer is a gated linear
attention (parts/linear_attention.py), a latent attention (parts/latent.py; a layer with ``kv_from`` reads the cached
vectors of an earlier layer), or two mixers side by side (parts/parallel.py): a chunked attention with projection
biases, a partly rotated head with rescaled frequencies, unit-norm queries and keys and capped scores, and a selective
state space (parts/state_space.py).  The feed-forward is a gated dense one or a mixture of experts whose chosen
logits are weighted by a softmax among themselves.  The embedding is scaled and the output matrix is the embedding table.

Tensor names: ``embed``, ``final.norm``; layer i: ``l<i>.norm1/2``; gla ``l<i>.mix.{q,k,v,g,o,norm,a1,a2,a2.b}``; latent
attention ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}``; parallel ``l<i>.mix.left.{q,q.b,k,k.b,v,v.b,o}`` and
``l<i>.mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o}``; dense ``l<i>.mlp.{gate,up,down}``; experts
``l<i>.mlp.router``, ``l<i>.mlp.router.b`` and ``l<i>.mlp.e<j>.{gate,up,down}``."""
from __future__ import annotations

from ..config.nugosun_config import NugosunConfig
from ..parts.description import ModelDescription, LayerSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

ARCHITECTURE = "Nugosun"


def _position(positions: dict, rot, pairing: str):
    """The name of the position encoding for ``rot`` (made on first use), or None."""
    if rot is None:
        return None
    name = f"{pairing}:{rot.dims}:{rot.base!r}:{rot.scaling!r}"
    if name not in positions:
        positions[name] = PartSpec("scaled_rotary", dict(rotary_dim=rot.dims, theta=rot.base, pairing=pairing,
                                                         scaling=rot.scaling))
    return name


def describe_nugosun(cfg: NugosunConfig) -> ModelDescription:
    W, eps = cfg.hidden_size, cfg.norm_eps
    positions, layers, schedule = {}, [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        position, cache_of = None, None
        if l.type == "gla":
            g = l.gla
            mixer = PartSpec("gated_linear_attention", dict(hidden_size=W, num_heads=g.heads, head_dim=g.dim, v_head_dim=g.vdim,
                                                            tau=g.tau, eps=eps, decay_rank=g.rank), prefix=f"{p}.mix")
        elif l.type == "latent_attention":
            a = l.latent
            position, cache_of = _position(positions, a.rot, "interleaved"), a.kv_from
            mixer = PartSpec("latent_attention", dict(
                hidden_size=W, num_heads=a.heads, head_dim=a.dim, rot_dim=a.rot_dim, v_head_dim=a.vdim, q_rank=a.q_rank,
                kv_rank=a.kv_rank, eps=eps, softmax_scale=a.scale, shared_kv=a.kv_from is not None), prefix=f"{p}.mix")
        else:
            a, s = l.left, l.right
            position = _position(positions, a.rot, "halves")
            mixer = PartSpec("parallel", dict(hidden_size=W, branches=[
                dict(name="left", kind="biased_chunk_attention", scale=l.left_scale, params=dict(
                    hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim,
                    softmax_scale=a.scale, chunk=a.chunk, projection_bias=True, rotary=a.rot is not None,
                    unit_norm_eps=eps, softcap=a.softcap)),
                dict(name="right", kind="selective_state_space", scale=l.right_scale, params=dict(
                    hidden_size=W, num_heads=s.heads, head_dim=s.vdim, state_size=s.state, groups=s.groups,
                    conv_taps=s.conv, norm_groups=s.norm_groups, eps=eps)),
            ]), prefix=f"{p}.mix")
        ff = None
        if l.mlp is not None and l.mlp.kind == "dense":
            ff = PartSpec("swiglu", dict(hidden_size=W, intermediate_size=l.mlp.ff, activation="silu",
                                         names={"gate": "gate", "up": "up", "down": "down"}), prefix=f"{p}.mlp")
        elif l.mlp is not None:
            ff = PartSpec("routed_experts", dict(hidden_size=W, intermediate_size=l.mlp.ff, num_experts=l.mlp.experts,
                                                 top=l.mlp.top, activation="silu", weight_on="output",
                                                 router_score="softmax_chosen", router_bias=True), prefix=f"{p}.mlp")
        norm = lambda q: PartSpec("rms_norm", dict(dim=W, eps=eps, name=f"norm{q}", weight_offset=1.0), prefix=p)
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm(1),
                                ffn_norm=norm(2) if ff is not None else None, block="parallel_pre_norm", position=position))
        schedule.append(ScheduleEntry(layer=i, cache_of=cache_of))       # one run per layer: entry j is layer j
    return ModelDescription(
        hidden_size=W, vocab_size=cfg.vocab_size, max_position=cfg.max_position, embed_name="embed", lm_head_name=None,
        final_norm=PartSpec("rms_norm", dict(dim=W, eps=eps, name="norm", weight_offset=1.0), prefix="final"),
        layers=layers, schedule=schedule, positions=positions, embed_scale=cfg.embed_scale)


register_architecture(ARCHITECTURE, NugosunConfig.from_json_dict, describe_nugosun, replace=True)
