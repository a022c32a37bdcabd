"""A plain, slow implementation of the Nugosun design in float64 (or float32), one function per mechanism, written
from the design's equations and sharing no code with the package.  It runs whole sequences at once on the CPU and is
what the framework's kernels, cache, state slots and batching are compared with.

Notation: T tokens at positions 0..T-1, W the model width, x the residual [T, W], h a sublayer's input.

    layer        x <- x + ( mixer(n1(x)) + ff(n2(x)) ),  n(x) = x / sqrt(mean(x^2) + eps) * (1 + w); both norms read the same x
    gla          S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t,  a_t = sigmoid(z_t)^(1/tau) per key channel
    parallel     c_l * chunked_attention(h) + c_r * ssd(h)
    ssd          S_t = exp(-exp(A) dt_t) S_(t-1) + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t   (Mamba-2)
    latent       attention whose keys and values are made from a small vector per token
    ff           down(silu(gate h) * (up h)), alone or as the chosen experts of a router
    output       E n(x), E the embedding table
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ small pieces
_ROUND = [None]     # set by forward(round_inputs=True): what an engine that computes in 16 bits rounds ahead of a product


def lin(x, w, b=None):
    """W x (+ b) for rows x; the rows are rounded first when forward() asks for it."""
    if _ROUND[0] is not None:
        x = _ROUND[0](x)
    y = x @ w.T
    return y if b is None else y + b


def rms_norm(x, w, eps: float, unit_offset: bool = False):
    """x / sqrt(mean(x^2) + eps) times (1 + w) or w; no weight when w is None."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * ((1.0 + w) if unit_offset else w)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rescaled_frequencies(rot: dict):
    """(frequencies [dims/2] as floats, magnitude of cos and sin).  Plain: base^(-2i/dims), magnitude 1.  With
    rot["scaling"] = {factor, original, fast, slow}: between the dimensions at which ``original`` positions make
    ``fast`` and ``slow`` turns a ramp takes f_i over to f_i / factor, and the magnitude is 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict, interleaved: bool):
    """x [T, ..., D]: the first rot["dims"] elements are turned by positions * f_i; pairs (2i, 2i+1) when
    ``interleaved``, else (i, i + dims/2).  The rest passes unchanged."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rescaled_frequencies(rot)
    ang = positions.to(x.dtype)[:, None] * torch.tensor(f, dtype=x.dtype)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def softmax_rows(scores, visible):
    s = scores.masked_fill(~visible, float("-inf"))
    s = s - s.max(dim=-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(dim=-1, keepdim=True)


# ------------------------------------------------------------------------------------------------ mixers
def decayed_outer_recurrence(q, k, v, log_decay, state=None):
    """The linear recurrence both state mixers share, one head: S_t = diag(exp(log_decay_t)) S_(t-1) + k_t v_t^T,
    o_t = S_t^T q_t.  q, k, log_decay [T, K] (the decay acts on the rows of S, which belong to the key channels), v [T, V].
    Returns (o [T, V], last state [K, V])."""
    T, K = k.shape
    S = torch.zeros((K, v.shape[1]), dtype=q.dtype) if state is None else state.clone()
    o = []
    for t in range(T):
        S = torch.exp(log_decay[t])[:, None] * S + k[t][:, None] * v[t][None, :]
        o.append(S.T @ q[t])
    return torch.stack(o), S


def gla_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, states: Optional[list] = None):
    """Gated linear attention with a decay per key channel read from the input through a low-rank pair of matrices."""
    T = h.shape[0]
    H, K, V, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    q = lin(h, w[p + ".q"]).reshape(T, H, K) * K ** -0.5
    k = lin(h, w[p + ".k"]).reshape(T, H, K)
    v = lin(h, w[p + ".v"]).reshape(T, H, V)
    z = lin(lin(h, w[p + ".a1"]), w[p + ".a2"], w[p + ".a2.b"]).reshape(T, H, K)
    log_alpha = torch.nn.functional.logsigmoid(z) / tau
    outs = []
    for hd in range(H):
        o, S = decayed_outer_recurrence(q[:, hd], k[:, hd], v[:, hd], log_alpha[:, hd])
        if states is not None:
            states.append(S)
        outs.append(rms_norm(o, w[p + ".norm"], float(m["eps"])))
    return lin(torch.cat(outs, dim=-1) * silu(lin(h, w[p + ".g"])), w[p + ".o"])


def chunked_attention(h, positions, w, p: str, m: dict, eps: float):
    """Grouped heads with biases; part of every q and k head rotated (halves pairing), then each head divided by its
    root mean square; score = cap * tanh(q.k * scale / cap); key j is seen from i if j <= i and both lie in the same
    block of mask.size positions counted from position 0."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = lin(h, w[p + ".q"], w[p + ".q.b"]).reshape(T, H, D)
    k = lin(h, w[p + ".k"], w[p + ".k.b"]).reshape(T, G, D)
    v = lin(h, w[p + ".v"], w[p + ".v.b"]).reshape(T, G, V)
    if m.get("rot"):
        q, k = rotate(q, positions, m["rot"], False), rotate(k, positions, m["rot"], False)
    q, k = rms_norm(q, None, eps), rms_norm(k, None, eps)
    visible = positions[None, :] <= positions[:, None]
    size = int((m.get("mask") or {}).get("size", 0))
    if size > 0:
        visible = visible & ((positions[:, None] // size) == (positions[None, :] // size))
    cap = float(m.get("softcap") or 0.0)
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        outs.append(softmax_rows(s, visible) @ v[:, g])
    return lin(torch.cat(outs, dim=-1), w[p + ".o"])


def causal_conv(u, weight, bias):
    """u [T, C], weight [C, taps]: y_t = bias + sum_j weight[:, j] u_(t - taps + 1 + j), zeros ahead of the sequence."""
    T, taps = u.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u) + bias
    for j in range(taps):
        y = y + padded[j:j + T] * weight[:, j]
    return y


def ssd_mixer(h, w, p: str, m: dict, eps: float, states: Optional[list] = None):
    """Mamba-2: one input product laid out [z | x | B | C | dt]; x, B, C through a short causal convolution and silu;
    a scalar decay per head and token; the gate ahead of a norm in equal parts of the concatenated heads."""
    T = h.shape[0]
    H, V, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * V
    proj = lin(h, w[p + ".in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + ".dt_bias"])                                 # [T, H]
    rate = torch.exp(w[p + ".A_log"])
    ys = []
    for hd in range(H):
        g = hd // (H // G)
        log_decay = (-rate[hd] * dt[:, hd])[:, None].expand(T, N)
        y, S = decayed_outer_recurrence(C[:, g], B[:, g] * dt[:, hd:hd + 1], x[:, hd], log_decay)
        if states is not None:
            states.append(S)
        ys.append(y + w[p + ".D"][hd] * x[:, hd])
    y = torch.cat(ys, dim=-1) * silu(z)
    parts = int(m["norm_groups"])
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * w[p + ".norm"]
    return lin(y, w[p + ".o"])


def latent_of(h, positions, w, p: str, m: dict, eps: float):
    """What a latent layer caches: (c [T, kv_rank] normed, r [T, rot_dim] rotated)."""
    kv_rank = int(m["kv_rank"])
    d = lin(h, w[p + ".dkv"])
    return rms_norm(d[:, :kv_rank], w[p + ".dkv.norm"], eps), rotate(d[:, kv_rank:], positions, m["rot"], True)


def latent_attention(h, positions, c, r, w, p: str, m: dict, eps: float):
    T = h.shape[0]
    H, D, R, V = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    q = lin(rms_norm(lin(h, w[p + ".dq"]), w[p + ".dq.norm"], eps), w[p + ".uq"]).reshape(T, H, D + R)
    q_rot = rotate(q[..., D:], positions, m["rot"], True)
    keys = lin(c, w[p + ".uk"]).reshape(T, H, D)
    vals = lin(c, w[p + ".uv"]).reshape(T, H, V)
    visible = positions[None, :] <= positions[:, None]
    outs = []
    for hd in range(H):
        s = (q[:, hd, :D] @ keys[:, hd].T + q_rot[:, hd] @ r.T) * float(m["scale"])
        outs.append(softmax_rows(s, visible) @ vals[:, hd])
    return lin(torch.cat(outs, dim=-1), w[p + ".o"])


# ------------------------------------------------------------------------------------------------ feed-forwards
def gated_ff(h, gate, up, down):
    return lin(silu(lin(h, gate)) * lin(h, up), down)


def routed_ff(h, w, p: str, mlp: dict, margins: Optional[list] = None):
    """Router logits W_r h + b; the ``top`` largest are chosen and weighted by the softmax over the chosen logits.
    ``margins`` collects one number a token: how close the choice was."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    logits = lin(h, w[p + ".router"], w[p + ".router.b"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(logits[t, e]), e))
        chosen = order[:top]
        if margins is not None:        # how far the last chosen logit is ahead of the best one left out, in units of the
            spread = float(logits[t].std()) if E > 1 else 1.0          # token's logits' standard deviation
            margins.append(float(logits[t, order[top - 1]] - logits[t, order[top]]) / max(spread, 1e-30) if top < E else float("inf"))
        wts = torch.softmax(logits[t, chosen], dim=0)
        for e, a in zip(chosen, wts):
            out[t] = out[t] + a * gated_ff(h[t:t + 1], w[f"{p}.e{e}.gate"], w[f"{p}.e{e}.up"], w[f"{p}.e{e}.down"])[0]
    return out


# ------------------------------------------------------------------------------------------------ the model
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None,
            margins: Optional[list] = None, round_inputs: bool = False):
    """Logits [T, vocab] of a whole sequence.  ``layers_out`` collects the residual after every layer.  With
    ``round_inputs`` the rows that enter a product with a weight matrix are rounded to bfloat16 first, as an engine that
    computes in 16 bits rounds them: how far that alone moves a position says how well conditioned the position is."""
    _ROUND[0] = (lambda t: t.to(torch.bfloat16).to(t.dtype)) if round_inputs else None
    try:
        return _forward(config, weights, tokens, dtype, layers_out, margins)
    finally:
        _ROUND[0] = None


def _forward(config, weights, tokens, dtype, layers_out, margins):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    latents = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = rms_norm(x, w[p + ".norm1"], eps, True)
        if layer["type"] == "gla":
            y = gla_mixer(h, w, p + ".mix", dict(m, eps=eps))
        elif layer["type"] == "parallel":
            y = float(m.get("left_scale", 1.0)) * chunked_attention(h, positions, w, p + ".mix.left", m["left"], eps) + \
                float(m.get("right_scale", 1.0)) * ssd_mixer(h, w, p + ".mix.right", m["right"], eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, positions, w, p + ".mix", m, eps)
                src = i
            c, r = latents[src]
            y = latent_attention(h, positions, c, r, w, p + ".mix", m, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = rms_norm(x, w[p + ".norm2"], eps, True)
            if mlp["kind"] == "dense":
                y = y + gated_ff(h2, w[p + ".mlp.gate"], w[p + ".mlp.up"], w[p + ".mlp.down"])
            else:
                y = y + routed_ff(h2, w, p + ".mlp", mlp, margins)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(rms_norm(x, w["final.norm"], eps, True), w["embed"])


def greedy(config: dict, weights, prompt, new_tokens: int, dtype=torch.float64):
    toks = list(prompt)
    for _ in range(new_tokens):
        toks.append(int(torch.argmax(forward(config, weights, toks, dtype)[-1])))
    return toks[len(prompt):]
