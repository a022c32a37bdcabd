"""Sadupel as a model description: a decoder-only design whose layers are listed one by one in config.json.  A layer
is ``x + m * (attention(h) + experts(h))`` with ONE RMS norm ``h = norm1(x)`` feeding both sublayers.  The attention
has grouped heads, a short causal convolution over time behind the q, k and v projections, an RMS norm over the whole
of q and of k, a rotate-half rotation of part of each head with linearly rescaled frequencies, capped scores, a learned
sink per head in the softmax, and a sigmoid gate per head read from the mixer's input.  The experts are not gated
(``down(relu(up h)^2)``); the router takes a softmax over experts and identity experts together, corrects the scores
for the choice only, and chooses within the best groups of neighbouring experts; a shared expert runs for every token.
A table indexed by a hash of the previous and the current token is added to the embedding, and a range of layers may
run several times in a row, every pass with caches of its own and a learned vector added to the residual ahead of it.

Tensor names: ``embed``, ``bigram``, ``loop.step``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.mix.{q,k,v,
g,o,sink}``, ``l<i>.mix.{q,k,v}.conv``, ``l<i>.mix.{q,k}.norm``, ``l<i>.mlp.router``, ``l<i>.mlp.correction``,
``l<i>.mlp.e<j>.{up,down}``, ``l<i>.mlp.shared.{up,down}``."""
from __future__ import annotations

from ..config.sadupel_config import SadupelConfig
from ..parts.description import ModelDescription, LayerSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

ARCHITECTURE = "Sadupel"


def describe_sadupel(cfg: SadupelConfig) -> ModelDescription:
    W = cfg.hidden_size
    positions, layers = {}, []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}"
        position = f"halves:{l.rot_dims}:{l.rot_base!r}:{l.rot_factor!r}"
        if position not in positions:
            positions[position] = PartSpec("scaled_rotary", dict(rotary_dim=l.rot_dims, theta=l.rot_base, pairing="halves",
                                                                 linear_factor=l.rot_factor))
        mixer = PartSpec("gated_sink_attention", dict(
            hidden_size=W, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim,
            softmax_scale=l.scale, softcap=l.softcap, sink="learned", head_gate=True, conv_taps=l.conv,
            qk_norm="whole", qk_norm_eps=cfg.norm_eps,
            names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "sink": "sink", "q_conv": "q.conv",
                   "k_conv": "k.conv", "v_conv": "v.conv", "q_norm": "q.norm", "k_norm": "k.norm", "lambda": "vmix"}),
            prefix=f"{p}.mix")
        ff = None
        if l.mlp is not None:
            e = l.mlp
            ff = PartSpec("routed_experts", dict(
                hidden_size=W, intermediate_size=e.ff, num_experts=e.experts, top=e.top, activation="relu2", gated=False,
                renormalize=False, weight_on="output", router_score="softmax", correction=True,
                groups=(e.groups, e.keep), identity_experts=e.identity, shared_intermediate=e.shared_ff), prefix=f"{p}.mlp")
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=ff, mixer_norm=PartSpec("rms_norm", dict(dim=W, eps=cfg.norm_eps, name="norm1"), prefix=p),
            block="stream_parallel", position=position,
            connectors={"layer": PartSpec("hyper_connection", dict(streams=1, hidden_size=W, learned=False,
                                                                    layer_scale=False, multiplier=cfg.residual_mult),
                                          prefix=p)}))
    schedule = [ScheduleEntry(layer=i, add_vector=("loop.step", t) if t is not None else None) for i, t in cfg.runs()]
    extras = []
    if cfg.bigram is not None:
        extras.append(PartSpec("hashed_pair", dict(hidden_size=W, buckets=cfg.bigram[0], mul_prev=cfg.bigram[1],
                                                   mul_cur=cfg.bigram[2], name="bigram")))
    return ModelDescription(
        hidden_size=W, vocab_size=cfg.vocab_size, max_position=cfg.max_position, embed_name="embed", lm_head_name="head",
        final_norm=PartSpec("rms_norm", dict(dim=W, eps=cfg.norm_eps, name="norm"), prefix="final"),
        layers=layers, schedule=schedule, positions=positions, streams=1, embed_extras=extras,
        vector_tables={"loop.step": cfg.loop[2]} if cfg.loop is not None else {})


register_architecture(ARCHITECTURE, SadupelConfig.from_json_dict, describe_sadupel, replace=True)
