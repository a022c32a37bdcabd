"""A plain, slow implementation of the Sadupel design in float64 (or float32), one function per mechanism, written
from the design's equations and sharing no code with the package.  It runs whole sequences at once on the CPU and
is what the framework's kernels, cache, state slots and batching are compared with.

Notation: T tokens at positions 0..T-1, W the model width, x the residual [T, W], m the residual multiplier.

    embedding:   x_t = E[tok_t] + B[(tok_(t-1) * a + tok_t * b) mod n]        (B[n] for t = 0)
    schedule:    layers start..stop-1 run ``times`` times in a row (own cache each pass), then the rest;
                 before every pass x <- x + step[pass]
    layer:       h = norm(x);  x <- x + m * (attention(h) + experts(h))       norm(x) = x / sqrt(mean(x^2) + eps) * w
    output:      head norm(x)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x, w, eps: float):
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


def bigram_rows(tokens, buckets: int, mul_prev: int, mul_cur: int):
    """Row of the bigram table for every token of one sequence: the pair's hash, or row ``buckets`` for the first."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens, table, bigram, buckets: int, mul_prev: int, mul_cur: int):
    idx = torch.tensor([int(t) for t in tokens], dtype=torch.long)
    return table[idx] + bigram[torch.tensor(bigram_rows(tokens, buckets, mul_prev, mul_cur), dtype=torch.long)]


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros((taps - 1, C), dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j][None, :]
    return y


def rotate_halves(x, positions, base: float, dims: int, factor: float = 1.0):
    """x [T, heads, D]: of the first ``dims`` elements of a head, element i is paired with i + dims/2 and the pair is
    turned by positions * base^(-2i/dims) / factor; the rest passes."""
    out = x.clone()
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) / factor for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def sink_softmax_attention(q, k, v, scale: float, softcap: float, sink, window: int = 0):
    """q [T, H, D], k [T, G, D], v [T, G, Dv], sink [H] or None -> [T, H, Dv].  Causal; scores (q.k) * scale, capped by
    softcap * tanh(. / softcap) when softcap > 0; the softmax's denominator has exp(sink_h) as one more term."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    i = torch.arange(T)
    visible = i[None, :] <= i[:, None]
    if window > 0:
        visible &= i[None, :] > i[:, None] - window
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~visible, float("-inf"))
        top = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].reshape(1, 1).to(s.dtype))
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h].to(s.dtype) - top)
        out[:, h] = (e / den) @ v[:, g]
    return out


def attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, positions=None):
    """The whole mixer on the rows h [T, W] of one sequence; ``w`` the model's tensors, ``p`` the mixer's prefix, ``m``
    its sizes and constants as the configuration lists them."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    positions = torch.arange(T) if positions is None else positions
    q, k, v = h @ w[p + ".q"].T, h @ w[p + ".k"].T, h @ w[p + ".v"].T
    if m.get("conv", 0) and m["conv"] > 0:
        q, k, v = causal_conv(q, w[p + ".q.conv"]), causal_conv(k, w[p + ".k.conv"]), causal_conv(v, w[p + ".v.conv"])
    q = rms_norm(q, w[p + ".q.norm"], eps)               # over the whole projection, not per head
    k = rms_norm(k, w[p + ".k.norm"], eps)
    q, k, v = q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, Dv)
    rot = m.get("rot")
    if rot is not None:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_halves(q, positions, float(rot["base"]), int(rot["dims"]), factor)
        k = rotate_halves(k, positions, float(rot["base"]), int(rot["dims"]), factor)
    o = sink_softmax_attention(q, k, v, float(m["scale"]), float(m.get("softcap", 0.0) or 0.0), w[p + ".sink"])
    gate = torch.sigmoid(h @ w[p + ".g"].T)               # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * Dv) @ w[p + ".o"].T


def route(h, w_router, correction, top: int, groups: int, keep: int, margin_out: Optional[list] = None):
    """Scores s = softmax(W_r h) over all router outputs; choice scores s + correction; only the ``keep`` groups (of
    ``groups`` equal groups of neighbours) with the largest best choice score stay eligible; the ``top`` largest choice
    scores among them are chosen (the lower index wins a tie); the weights are the chosen s.  -> (index [T, top], s [T, top]).
    ``margin_out`` receives a [T] tensor: how far the choice is from another one, the smaller of the gap between the last
    chosen and the first unchosen choice score and the gap between the last kept and the first dropped group."""
    s = torch.softmax(h @ w_router.T, dim=-1)
    c = s + correction[None, :]
    T, E = c.shape
    margin = torch.full((T,), float("inf"), dtype=c.dtype)
    if groups > 1 and keep < groups:
        per = E // groups
        best = c.reshape(T, groups, per).max(dim=-1).values
        ranked = torch.sort(best, dim=-1, descending=True).values
        margin = ranked[:, keep - 1] - ranked[:, keep]
        order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
        ok = torch.zeros((T, groups), dtype=torch.bool)
        ok.scatter_(1, order, True)
        c = c.masked_fill(~ok[:, :, None].expand(T, groups, per).reshape(T, E), float("-inf"))
    if top < E:
        ranked = torch.sort(c, dim=-1, descending=True).values
        margin = torch.minimum(margin, ranked[:, top - 1] - ranked[:, top])
    if margin_out is not None:
        margin_out.append(margin)
    idx = torch.sort(c, dim=-1, descending=True, stable=True).indices[:, :top]
    return idx, torch.gather(s, 1, idx)


def plain_expert(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def experts_mixer(h, w: Dict[str, torch.Tensor], p: str, mlp: dict, round_router_input: bool = False,
                  margin_out: Optional[list] = None):
    """``round_router_input``: the router reads the bfloat16 rounding of h (the design allows either); a token whose choice
    of experts changes with it is a close call."""
    r = mlp["router"]
    E, ident = int(r["experts"]), int(r.get("identity", 0) or 0)
    g = r.get("groups") or {}
    hr = h.to(torch.bfloat16).to(h.dtype) if round_router_input else h
    idx, wts = route(hr, w[p + ".router"], w[p + ".correction"], int(r["top"]), int(g.get("count", 1)), int(g.get("keep", 1)),
                     margin_out)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), wts[t]):
            if e >= E:                                   # an identity expert: the input itself
                out[t] += s * h[t]
            else:
                out[t] += s * plain_expert(h[t:t + 1], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + plain_expert(h, w[p + ".shared.up"], w[p + ".shared.down"])
    return out


def layer_runs(config: dict) -> List[tuple]:
    """(layer, pass number or None) in the order the layers run; the pass number on the first layer of each pass."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or int(loop.get("times", 1)) < 1:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None,
            round_router_input: bool = False, margins_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence; ``layers_out`` receives the residual after every layer run, ``margins_out`` a
    [T] tensor per routed layer run (see route)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    bg = config["embedding"]["bigram"]
    x = embed(tokens, w["embed"], w["bigram"], int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))
    for i, step in layer_runs(config):
        l, p = config["layers"][i], f"l{i}"
        if step is not None:
            x = x + w["loop.step"][step][None, :]
        h = rms_norm(x, w[p + ".norm1"], eps)
        y = attention_mixer(h, w, p + ".mix", l["mixer"], eps)
        if l.get("mlp") is not None:
            y = y + experts_mixer(h, w, p + ".mlp", l["mlp"], round_router_input, margins_out)
        x = x + mult * y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(config: dict, weights, prompt, new_tokens: int, dtype=torch.float64):
    toks = [int(t) for t in prompt]
    for _ in range(new_tokens):
        toks.append(int(torch.argmax(forward(config, weights, toks, dtype)[-1])))
    return toks[len(prompt):]
