"""The Nugosun design in the engine against its plain implementation (plain_nugosun.py): every mechanism alone through
the kernel library, and whole models of several small configurations in every cut of the steps.  The configurations
differ in every size and option, with values that are unequal where a model might have them equal (key and value sizes,
heads and key/value heads, state rows and head channels, rotated dimensions and head) and 1 where it might have more
(heads, groups, experts, chosen experts, taps, block size)."""
import math
import random

import pytest
import torch

import plain_nugosun as P
from helpers import trace_whole, trace_tail_decode, trace_portions, trace_mixed, run_trace, first_bad
from test_tipezen_gpu import fake_batch
from tffinfer_b200.config import EngineConfig, NugosunConfig, NugosunLayer, NugosunMlp
from tffinfer_b200.config.nugosun_config import NugosunGla, NugosunAttention, NugosunStateSpace, NugosunLatent
from tffinfer_b200.config.tipezen_config import RotaryConfig
from tffinfer_b200.engine import ModelRunner
from tffinfer_b200.weights.random_init import random_state_dict

pytestmark = pytest.mark.gpu
TOL = {"float32": 3e-5, "bfloat16": 5e-2}


def gla(heads, dim, vdim, tau, rank, mlp=None):
    return NugosunLayer("gla", gla=NugosunGla(heads, dim, vdim, tau, rank), mlp=mlp)


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale=None, base=1e4, rot_dims=0, kv_from=None, mlp=None):
    return NugosunLayer("latent_attention", latent=NugosunLatent(
        heads, dim, rot_dim, vdim, q_rank, kv_rank, scale if scale is not None else (dim + rot_dim) ** -0.5,
        RotaryConfig(base, rot_dims or rot_dim), kv_from), mlp=mlp)


def par(heads, kv, dim, vdim, chunk, scale, cap, rot, s_heads, s_vdim, s_state, groups=1, conv=4, parts=1, ls=1.0, rs=1.0,
        mlp=None):
    return NugosunLayer("parallel", left=NugosunAttention(heads, kv, dim, vdim, scale, cap, chunk, rot),
                        right=NugosunStateSpace(s_heads, s_vdim, s_state, groups, conv, parts), left_scale=ls,
                        right_scale=rs, mlp=mlp)


YARN = (4.0, 64.0, 16.0, 2.0)          # factor, original, fast, slow


def config(name: str) -> NugosunConfig:
    if name == "a":      # sizes that take the tensor-core products; every kind of layer, a borrowed latent cache
        moe, dense = NugosunMlp("moe", 64, 6, 2), NugosunMlp("dense", 192)
        rot = RotaryConfig(1e4, 32, YARN)
        layers = (gla(2, 64, 32, 8.0, 16, mlp=dense),
                  par(8, 2, 64, 64, 24, 0.3, 6.0, rot, 4, 32, 16, groups=2, conv=4, parts=2, ls=0.7, rs=1.2, mlp=moe),
                  lat(4, 32, 16, 32, 48, 64, mlp=moe), gla(4, 16, 32, 2.0, 8, mlp=moe),
                  lat(4, 32, 16, 32, 48, 64, kv_from=2, mlp=dense),
                  par(8, 2, 64, 64, 24, 0.3, 6.0, rot, 4, 32, 16, groups=2, conv=4, parts=2, ls=0.7, rs=1.2, mlp=dense))
        return NugosunConfig("Nugosun", vocab_size=320, hidden_size=128, embed_scale=8.0, norm_eps=1e-5, layers=layers)
    if name == "b":      # odd sizes everywhere: FMA products, three query heads a key/value head, a block of 7 positions
        moe = NugosunMlp("moe", 22, 5, 5)                               # that no page size divides, every expert chosen,
        layers = (par(6, 2, 24, 40, 7, 0.25, 0.0, RotaryConfig(1e3, 10), 3, 20, 12, groups=3, conv=3, parts=5, rs=0.5),
                  gla(3, 12, 20, 1.0, 5, mlp=moe),                       # no cap, a layer without a feed-forward,
                  lat(3, 20, 6, 12, 10, 18, scale=0.2, base=1e3, rot_dims=4, mlp=moe),          # part of the rotated part
                  par(6, 2, 24, 40, 7, 0.25, 0.0, RotaryConfig(1e3, 10), 3, 20, 12, groups=3, conv=3, parts=5, rs=0.5,
                      mlp=NugosunMlp("dense", 70)),                      # not rotated
                  lat(3, 20, 6, 12, 10, 18, scale=0.2, base=1e3, rot_dims=4, kv_from=2, mlp=moe))
        return NugosunConfig("Nugosun", vocab_size=97, hidden_size=52, embed_scale=1.0, norm_eps=3e-6, layers=layers)
    if name == "c":      # one head, one group, one expert, one tap, blocks of one position and none, no rotation, values
        m1, m2 = NugosunMlp("moe", 48, 1, 1), NugosunMlp("moe", 16, 9, 1)          # wider than keys, a whole head rotated
        layers = (lat(1, 16, 8, 72, 24, 160, base=5e5, mlp=m1),
                  par(1, 1, 16, 32, 1, 0.5, 3.0, None, 1, 48, 8, conv=1, mlp=m2),
                  gla(1, 8, 96, 30.0, 24),
                  par(2, 1, 32, 16, 0, 0.2, 9.0, RotaryConfig(3e4, 32, YARN), 2, 8, 40, conv=2, ls=1.5, mlp=m2),
                  gla(2, 40, 8, 4.0, 3, mlp=NugosunMlp("dense", 32)))
        return NugosunConfig("Nugosun", vocab_size=264, hidden_size=64, embed_scale=3.0, norm_eps=1e-6, layers=layers)
    if name == "d":      # blocks of 64 over pages of 32, chains of borrowed vectors, a gla layer first and last, wide state
        moe = NugosunMlp("moe", 32, 12, 3)
        rot = RotaryConfig(3e5, 8, (6.0, 128.0, 24.0, 0.5))
        layers = (gla(2, 128, 24, 16.0, 32, mlp=moe), lat(2, 24, 8, 40, 32, 56, mlp=moe),
                  par(8, 8, 16, 16, 64, 0.4, 20.0, rot, 2, 64, 80, conv=5, parts=4, mlp=moe),
                  lat(2, 24, 8, 40, 32, 56, kv_from=1, mlp=moe), lat(4, 8, 8, 8, 8, 56, mlp=NugosunMlp("dense", 40)),
                  lat(2, 24, 8, 40, 32, 56, kv_from=1), gla(2, 128, 24, 16.0, 32, mlp=moe))
        return NugosunConfig("Nugosun", vocab_size=150, hidden_size=96, embed_scale=9.8, norm_eps=1e-6, layers=layers)
    raise KeyError(name)


PAGE = {"a": 16, "b": 4, "c": 8, "d": 32}
PROMPTS = {"a": [5, 90, 37, 200], "b": [1, 13, 40, 64], "c": [3, 29, 110, 71], "d": [2, 70, 133]}


def weights(cfg, seed=11, sharp=4.0):
    """Random weights; the latent queries and the routers are scaled up so that attention is far from uniform, a key
    that is wrongly seen or missed moves the logits, and router scores differ between experts."""
    sd = random_state_dict(cfg, seed, "bfloat16", norm_noise=0.2)
    for n in sd:
        if n.endswith(".mix.uq"):
            sd[n] = (sd[n].float() * sharp).to(torch.bfloat16)
        elif n.endswith(".router"):
            sd[n] = (sd[n].float() * 8.0).to(torch.bfloat16)
        elif n.endswith(".mix.k") or n.endswith(".mix.v") or n.endswith(".right.in"):
            sd[n] = (sd[n].float() * 3.0).to(torch.bfloat16)         # states that weigh beside the attention
    return sd


def runner_of(cfg, sd, dtype, page, tokens, live=4, graphs=False):
    return ModelRunner(config=cfg, tensors=dict(sd), engine_config=EngineConfig(
        dtype=dtype, page_size=page, max_cache_tokens=tokens, max_live_requests=live, use_cuda_graphs=graphs))


def plain_logits(cj, sd, reqs, dtype):
    """{request: (logits, bar of every position)} of the plain implementation.  In 32-bit the bar is TOL.  In bfloat16 a
    position may be ill-conditioned (a head's output normed when its query barely meets its key, a router's close call):
    how far rounding the rows that enter every product alone moves the plain logits there, times three, is then its bar, and a
    position at which a router's choice hangs on less than a hundredth of its logits' spread is not compared.  Such positions must be few, or the test
    says nothing."""
    out = {}
    for r, t in reqs.items():
        want = P.forward(cj, sd, t)
        bar = torch.full((want.shape[0],), TOL[dtype], dtype=torch.float64)
        if dtype == "bfloat16":
            margins = []
            moved = P.forward(cj, sd, t, round_inputs=True, margins=margins)
            bar = torch.maximum(bar, 3.0 * (moved - want).abs().amax(dim=-1) / want.abs().amax(dim=-1))
            if margins:        # a router's close call (per routed layer one margin a token): another expert may win in 16 bits
                closest = torch.tensor(margins, dtype=torch.float64).reshape(-1, want.shape[0]).amin(dim=0)
                bar[closest < 0.01] = float("inf")
        out[r] = (want, bar)
    raised = sum(int((b > TOL[dtype]).sum()) for _, b in out.values())
    assert raised <= 2 + sum(w.shape[0] for w, _ in out.values()) // 4, f"{raised} ill-conditioned positions: too many for a test"
    return out


def assert_within(got, want_bar, what):
    want, bar = want_bar
    err = torch.nan_to_num((got.double() - want).abs().amax(dim=-1) / want.abs().amax(dim=-1).clamp_min(1e-30), nan=float("inf"))
    bad = torch.nonzero(err > bar)
    assert bad.numel() == 0, f"{what}: token {int(bad[0])} off by {float(err[int(bad[0])]):.3g} (bar {float(bar[int(bad[0])]):.3g})"


def requests_of(cfg, name, decoded, seed=5):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + decoded)] for i, n in enumerate(PROMPTS[name])}


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cut_matches_plain(name, dtype):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and mixed batches in a pool
    small enough that pages and slots are used again (released pages are poisoned)."""
    cfg = config(name)
    sd = weights(cfg)
    reqs = requests_of(cfg, name, decoded=12)
    cj = cfg.to_json_dict()
    want = plain_logits(cj, sd, reqs, dtype)
    page = PAGE[name]
    most = max(-(-len(t) // page) * page for t in reqs.values())
    cuts = {"whole": (trace_whole(reqs), most), "tail": (trace_tail_decode(reqs, tail=12), most),
            "portions": (trace_portions(reqs), most),
            "mixed": (trace_mixed(reqs, PROMPTS[name], max_live=3, page_size=page, pool_tokens=most + most // 2,
                                  chunk=48), most + most // 2)}
    for cut, (steps, pool) in cuts.items():
        r = runner_of(cfg, sd, dtype, page, pool, live=3)
        stats = {}
        got = run_trace(r, reqs, steps, poison=True, stats=stats)
        for q in reqs:
            assert_within(got[q], want[q], f"{name} {dtype} {cut}: request {q}")
        if cut == "mixed":
            assert stats["pages_reused"] > 0


def test_cuts_agree_in_float32():
    """The logits of a position do not depend on how the prompt was cut beyond rounding: far tighter than the
    distance to the plain implementation allows."""
    cfg = config("a")
    sd = weights(cfg)
    reqs = requests_of(cfg, "a", decoded=8)
    most = max(-(-len(t) // 16) * 16 for t in reqs.values())
    ref = run_trace(runner_of(cfg, sd, "float32", 16, most), reqs, trace_whole(reqs))
    for steps in (trace_portions(reqs, sizes=(2, 31, 3, 16, 2, 33)), trace_tail_decode(reqs, tail=40)):
        got = run_trace(runner_of(cfg, sd, "float32", 16, most), reqs, steps)
        for q in reqs:
            assert first_bad(got[q], ref[q], 5e-6) is None


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.fixture(scope="module")
def ops():
    from tffinfer_b200.kernels.library import CudaKernels
    return CudaKernels()


def _steps_of(seqs, lens_by_step):
    """(lens, starts) of every step for sequences cut as lens_by_step[step][request] says."""
    starts = [0] * len(seqs)
    for lens in lens_by_step:
        yield lens, list(starts)
        starts = [s + n for s, n in zip(starts, lens)]


@pytest.mark.parametrize("H,K,V,share", [(2, 32, 16, 1), (3, 12, 20, 1), (1, 128, 24, 1), (4, 48, 40, 2), (2, 200, 8, 2),
                                         (1, 8, 130, 1)])
@pytest.mark.parametrize("mode", ["gate", "step", "log"])
@pytest.mark.parametrize("long", [150, 600])
def test_recurrence_steps_slots_and_a_far_key(ops, H, K, V, share, mode, long):
    """The recurrence through three steps (a long portion, short portions, one token each), slots out of order, other
    slots poisoned, state behind other elements of the slot, against the plain recurrence over the whole sequences.
    In the first request one key far back is planted with a query aimed at it under a slow decay: its value must
    arrive at the last token.  A portion of 600 tokens is walked as segments side by side (ragged last segment) beside
    short portions that are not."""
    if mode != "step" and share != 1:
        pytest.skip("shared q and k go with the per-head decay")
    dev = "cuda"
    g = torch.Generator().manual_seed(H * K + V)
    cuts = [[long, 3, 1], [2, 9, 1], [1, 1, 1]]
    total = [sum(c[i] for c in cuts) for i in range(3)]
    G = H // share
    off = 7                                                  # the state does not start at the slot's first element
    slots = [3, 0, 2]
    state = torch.full((5, off + H * K * V + 3), float("nan"), device=dev)
    tau = 3.0
    seqs = []
    for n in total:
        q, k = torch.randn(n, G * K, generator=g), torch.randn(n, G * K, generator=g)
        v = torch.randn(n, H * V, generator=g)
        dec = torch.randn(n, H if mode == "step" else H * K, generator=g)
        if mode == "log":
            dec = -dec.abs() * 0.2
        seqs.append([q, k, v, dec])
    bias = torch.randn(H if mode == "step" else H * K, generator=g)
    rate_log = torch.randn(H, generator=g) * 0.5
    skip = torch.randn(H, generator=g)
    # the planted key of request 0: token 4 holds a key nobody else resembles, the last token asks for it
    q0, k0, v0, d0 = seqs[0]
    k0[4, :K] = 0.0
    k0[4, 0] = 30.0
    q0[-1, :K] = 0.0
    q0[-1, 0] = 30.0
    if mode == "gate":
        d0[:, 0] = 12.0 - bias[0]                            # sigmoid(12)^(1/3): the channel forgets almost nothing
    elif mode == "log":
        d0[:, 0] = -1e-5
    else:
        d0[:, 0] = -9.0 - bias[0]                            # a tiny step: head 0 decays slowly
    want = []
    for q, k, v, dec in seqs:
        outs = []
        for h in range(H):
            gi = h // share
            qh, kh = q[:, gi * K:(gi + 1) * K].double() * 0.5, k[:, gi * K:(gi + 1) * K].double()
            vh = v[:, h * V:(h + 1) * V].double()
            if mode == "step":
                dt = P.softplus(dec[:, h].double() + bias[h].double())
                ld = (-torch.exp(rate_log[h].double()) * dt)[:, None].expand(-1, K)
                kh = kh * dt[:, None]
            elif mode == "gate":
                ld = torch.nn.functional.logsigmoid(dec[:, h * K:(h + 1) * K].double() + bias[h * K:(h + 1) * K].double()) / tau
            else:
                ld = dec[:, h * K:(h + 1) * K].double()
            o, _ = P.decayed_outer_recurrence(qh, kh, vh, ld)
            outs.append(o + (skip[h].double() * vh if mode == "step" else 0.0))
        want.append(torch.cat(outs, dim=-1))
    got = [[] for _ in seqs]
    pad = 5                                                  # the inputs are column blocks of wider rows
    for lens, starts in _steps_of(seqs, cuts):
        b = fake_batch(lens, starts, dev, 8, slots=slots)
        ops.reset_state_slots(state, b.slots, b.pos_start)
        rows = [torch.cat([s[j][st:st + n] for s, n, st in zip(seqs, lens, starts)]) for j in range(4)]
        wide = [torch.cat([torch.full((r.shape[0], pad), float("nan")), r], dim=1).to(dev).contiguous() for r in rows]
        out = torch.full((rows[0].shape[0], H * V), float("nan"), device=dev)
        ops.linear_recurrence((wide[0], pad), (wide[1], pad), (wide[2], pad), (wide[3], pad), state, b, out, H, K, V, mode,
                              share=share, dec_bias=bias.to(dev) if mode != "log" else None,
                              rate_log=rate_log.to(dev) if mode == "step" else None,
                              skip=skip.to(dev) if mode == "step" else None, inv_tau=1.0 / tau, q_scale=0.5, state_off=off)
        torch.cuda.synchronize()
        row = 0
        for i, n in enumerate(lens):
            got[i].append(out[row:row + n].double().cpu())
            row += n
    for i in range(len(seqs)):
        scale = float(want[i].abs().max())
        err = float((torch.cat(got[i]) - want[i]).abs().max()) / scale
        assert err < (2e-5 if long <= 256 else 5e-5), f"request {i} off by {err:.3g}"
    if mode != "step":                                       # (a slow decay there means a small step, which also scales k)
        assert float(want[0][-1, :V].abs().max()) > 100.0    # the far key's value dominates the last output of head 0
    assert torch.isnan(state[1]).all() and torch.isnan(state[4]).all()          # nobody's slots were left alone


@pytest.mark.parametrize("taps,C,act", [(1, 40, "silu"), (2, 300, "none"), (4, 96, "silu"), (7, 10, "silu")])
def test_causal_convolution_across_steps(ops, taps, C, act):
    """Portions shorter than the taps, single tokens, slots out of order and poisoned neighbours; an impulse must
    arrive exactly ``taps`` tokens long."""
    dev = "cuda"
    g = torch.Generator().manual_seed(taps)
    cuts = [[2, 9, 1], [1, 1, 1], [3, 1, 2], [1, 30, 1]]
    total = [sum(c[i] for c in cuts) for i in range(3)]
    w, bias = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    seqs = [torch.randn(n, C, generator=g) for n in total]
    seqs[1] = torch.zeros_like(seqs[1])
    seqs[1][2] = 1.0                                          # the impulse
    f = (lambda y: y) if act == "none" else P.silu
    want = [f(P.causal_conv(s.double(), w.double(), bias.double())) for s in seqs]
    off, col0 = 11, 6
    state = torch.full((5, off + max(taps - 1, 1) * C + 2), float("nan"), device=dev)
    slots = [4, 1, 2]
    got = [[] for _ in seqs]
    for lens, starts in _steps_of(seqs, cuts):
        b = fake_batch(lens, starts, dev, 8, slots=slots)
        ops.reset_state_slots(state, b.slots, b.pos_start)
        rows = torch.cat([s[st:st + n] for s, n, st in zip(seqs, lens, starts)])
        proj = torch.cat([torch.full((rows.shape[0], col0), float("nan")), rows, torch.full((rows.shape[0], 3), float("nan"))],
                         dim=1).to(dev).contiguous()
        out = torch.full((rows.shape[0], C), float("nan"), device=dev)
        # steps of single tokens let the convolution's kernel move the rows up itself
        if not ops.causal_conv(proj, col0, C, w.to(dev), bias.to(dev), act, state if taps > 1 else None, off, b, out,
                               update_state=True):
            ops.causal_conv_state(proj, col0, C, taps, state, off, b)
        torch.cuda.synchronize()
        row = 0
        for i, n in enumerate(lens):
            got[i].append(out[row:row + n].double().cpu())
            row += n
    for i in range(3):
        err = float((torch.cat(got[i]) - want[i]).abs().max())
        assert err < 1e-5, f"request {i} off by {err:.3g}"
    base = f(bias.double())
    moved = ((want[1] - base).abs().amax(dim=1) > 1e-9).nonzero().flatten().tolist()
    assert moved == list(range(2, 2 + taps))
    assert torch.isnan(state[0]).all() and torch.isnan(state[3]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,group,wlen,first", [(96, 32, 32, False), (96, 48, 96, True), (60, 12, 60, True),
                                                    (130, 130, 130, True), (40, 8, 8, False)])
def test_gated_group_norm(ops, dtype, width, group, wlen, first):
    dev = "cuda"
    g = torch.Generator().manual_seed(width)
    T, goff, ooff = 7, 5, 3
    o, gate = torch.randn(T, width, generator=g) * 3, torch.randn(T, goff + width + 2, generator=g)
    w = 1 + 0.3 * torch.randn(wlen, generator=g)
    z = gate[:, goff:goff + width].double()
    wfull = w.double().repeat(width // wlen)
    if first:
        want = P.rms_norm((o.double() * P.silu(z)).reshape(T, width // group, group), None, 1e-5).reshape(T, width) * wfull
    else:
        want = P.rms_norm(o.double().reshape(T, width // group, group), None, 1e-5).reshape(T, width) * wfull * P.silu(z)
    out = torch.full((T, ooff + width + 1), float("nan"), device=dev, dtype=dtype)
    ops.gated_norm(o.to(dev), group, gate.to(dev).contiguous(), goff, w.to(dev), 1e-5, first, out, ooff, 1.5)
    torch.cuda.synchronize()
    err = float((out[:, ooff:ooff + width].double().cpu() / 1.5 - want).abs().max()) / float(want.abs().max())
    assert err < (1e-5 if dtype == torch.float32 else 1e-2)
    assert torch.isnan(out[:, :ooff]).all() and torch.isnan(out[:, ooff + width:]).all()


def _rot(dims, base=1e4, scaling=None):
    d = {"dims": dims, "base": base}
    if scaling is not None:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def _attention_case(ops, dtype, H, G, d, dv, chunk, cap, rot, lens, starts, aim, page=8, splits=None):
    """Requests whose step brings lens[b] tokens after starts[b] cached ones.  The mixer's input is made so that, in
    every request, the LAST query resembles the key at position aim[b] far more than any other: if that key is
    visible the output is its value, if not it is a mix of the others.  Runs biases, rotation, unit norm and cache
    write (qkv_finish), then the chunked, capped attention (attention_tile), against the plain mixer."""
    from tffinfer_b200.parts.position import scaled_frequencies
    dev = "cuda"
    g = torch.Generator().manual_seed(H * d + chunk)
    W = 32
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.6, "softcap": cap, "mask": {"size": chunk}, "rot": rot}
    w = {"p.q": torch.randn(H * d, W, generator=g), "p.k": torch.randn(G * d, W, generator=g),
         "p.v": torch.randn(G * dv, W, generator=g), "p.q.b": torch.randn(H * d, generator=g) * 0.3,
         "p.k.b": torch.randn(G * d, generator=g) * 0.3, "p.v.b": torch.randn(G * dv, generator=g) * 0.3,
         "p.o": torch.eye(H * dv)}
    w = {k: v.double() for k, v in w.items()}
    seqs = []
    for n, s, a in zip(lens, starts, aim):
        h = torch.randn(s + n, W, generator=g).double()
        if rot is None:
            # without a rotation a query finds its key by content: the last token's input is the aimed token's, and
            # q and k projections are tied so that q.k is largest there
            h[-1] = h[a] * 3.0
        seqs.append(h)
    if rot is None:
        w["p.k"] = w["p.q"][:G * d].clone()
        w["p.k.b"] = w["p.q.b"][:G * d].clone()
    want = [P.chunked_attention(h, torch.arange(h.shape[0]), w, "p", m, 1e-6) for h in seqs]
    # the engine's side: two steps (the cached tokens, then the step's own), pages in order
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    freq = None
    if rot is not None:
        f, mag = scaled_frequencies(rot["dims"], rot["base"], tuple(rot["scaling"].values()) if "scaling" in rot else None)
        freq = (torch.tensor(f, dtype=torch.float64).float().to(dev), rot["dims"], mag, False)
    slot = max(d, dv)
    pages = sum(-(-(s + n) // page) for n, s in zip(lens, starts))
    cache = torch.full((pages + 1, 1, 2, G, page, slot), float("nan"), device=dev, dtype=tdt)
    w_in = torch.cat([w["p.q"], w["p.k"], w["p.v"]]).float().to(dev)
    bias = torch.cat([w["p.q.b"], w["p.k.b"], w["p.v.b"]]).float().to(dev)
    outs = None
    for phase in (0, 1):
        ln = [s for s in starts] if phase == 0 else list(lens)
        st = [0] * len(lens) if phase == 0 else list(starts)
        keep = [i for i, n in enumerate(ln) if n > 0]
        if not keep:
            continue
        b = fake_batch([ln[i] for i in keep], [st[i] for i in keep], dev, page)
        # the same pages in both phases: request i's pages are those of its whole length
        first = [0]
        for n, s in zip(lens, starts):
            first.append(first[-1] + -(-(s + n) // page))
        width = max(-(-(s + n) // page) for n, s in zip(lens, starts))
        table = [[first[i] + j if j < first[i + 1] - first[i] else -1 for j in range(width)] for i in keep]
        b.block_table = torch.tensor(table, dtype=torch.int32, device=dev)
        rows = torch.cat([seqs[i][st[i]:st[i] + ln[i]] for i in keep]).float().to(dev)
        proj = (rows @ w_in.T).contiguous()
        q = torch.empty((rows.shape[0], H * d), device=dev, dtype=tdt)
        ops.qkv_finish(proj, q, None, freq, b, b.block_table, cache, 0, page, H, G, d, dv, bias=bias, unit_eps=1e-6)
        out = torch.full((rows.shape[0], H * dv + 3), float("nan"), device=dev, dtype=tdt)
        ops.attention_tile(q, b, b.block_table, cache, 0, page, out, H, G, d, dv, 0.6, chunk=chunk, softcap=cap,
                           out_scale=2.0, out_off=3, num_splits=splits)
        torch.cuda.synchronize()
        if phase == 1:
            outs, row = [], 0
            for i in keep:
                outs.append(out[row:row + ln[i], 3:].double().cpu() / 2.0)
                row += ln[i]
    return outs, [wnt[s:] for wnt, s in zip(want, starts)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rot", [None, _rot(8), _rot(16, 1e3, YARN)])
@pytest.mark.parametrize("lens,starts,aim", [([40, 1, 1, 1, 1], [0, 39, 40, 47, 300], [24, 24, 24, 24, 288]),
                                             ([3, 2, 64, 9], [21, 46, 100, 0], [1, 24, 145, 0]),
                                             ([1, 1, 1], [23, 24, 71], [0, 23, 48])])
def test_attention_block_edges_and_far_keys(ops, dtype, rot, lens, starts, aim):
    """Blocks of 24 positions over pages of 8: keys just inside a block, just outside, one before the edge and far
    back; decoded tokens and the last token of a portion; with and without a cap, three heads a key/value head,
    unequal key and value sizes; the key range whole and in shares."""
    for H, G, d, dv, cap, splits in ((6, 2, 16, 24, 4.0, None), (2, 2, 64, 64, 0.0, 2), (3, 1, 20, 8, 7.0, None)):
        got, want = _attention_case(ops, dtype, H, G, d, dv, 24, cap, rot, lens, starts, aim, splits=splits)
        for i, (a, b) in enumerate(zip(got, want)):
            err = float((a - b).abs().max()) / float(b.abs().max())
            assert err < (2e-5 if dtype == "float32" else 4e-2), f"request {i} off by {err:.3g} ({H}, {G}, {d}, {dv})"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,ff,W,T", [(5, 1, 24, 40, 70), (7, 3, 64, 128, 130), (3, 3, 10, 52, 9), (1, 1, 16, 64, 3),
                                          (16, 2, 64, 128, 600)])
def test_routed_experts_with_a_bias_and_weights_among_the_chosen(ops, dtype, E, top, ff, W, T):
    """The router's bias moves the choice (it is large for one expert, which every token must then take), and the
    weights are the softmax over the chosen logits alone."""
    from tffinfer_b200.parts.moe import RoutedExperts
    dev = "cuda"
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(E * 100 + top)
    rnd = lambda *s: (torch.randn(*s, generator=g) * (s[-1] ** -0.5)).to(torch.bfloat16)
    w = {"m.router": (rnd(E, W).float() * 6).to(torch.bfloat16), "m.router.b": torch.randn(E, generator=g).to(torch.bfloat16)}
    w["m.router.b"][E - 1] = 25.0
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = rnd(ff, W), rnd(ff, W), rnd(W, ff)
    part = RoutedExperts(W, ff, E, top, activation="silu", weight_on="output", router_score="softmax_chosen",
                         router_bias=True, prefix="m")
    held = {k[2:]: (v.float() if k.endswith(".b") else v.to(tdt)).to(dev) for k, v in w.items()}
    part.load(held, ops, tdt)
    h = torch.randn(T, W, generator=g).to(torch.bfloat16)
    margins = []
    want = P.routed_ff(h.double(), {k: v.double() for k, v in w.items()}, "m", {"router": {"experts": E, "top": top}}, margins)
    from types import SimpleNamespace
    res = torch.zeros(T, W, device=dev)
    part.forward(h.to(tdt).to(dev), SimpleNamespace(ops=ops), res)
    torch.cuda.synchronize()
    sure = torch.tensor([m > 1e-3 for m in margins])
    err = float((res.double().cpu() - want)[sure].abs().max()) / float(want.abs().max())
    assert err < (2e-5 if dtype == "float32" else 3e-2)


def test_both_norms_of_a_layer_read_the_same_residual(ops):
    """The arrangement x + mixer(norm1 x) + ff(norm2 x): the feed-forward's norm must not see what the mixer added."""
    from tffinfer_b200.parts.block import ParallelPreNormBlock
    from tffinfer_b200.parts.norm import RMSNorm
    from types import SimpleNamespace
    dev = "cuda"
    g = torch.Generator().manual_seed(3)
    T, W = 9, 72
    x = torch.randn(T, W, generator=g)
    w1, w2 = torch.randn(W, generator=g) * 0.2, torch.randn(W, generator=g) * 0.2

    class Adds:
        def __init__(self, f):
            self.f = f

        def forward(self, h, ctx, residual):
            residual += self.f * h.float()
            return residual

    n1, n2 = RMSNorm(W, 1e-5, "norm1", 1.0), RMSNorm(W, 1e-5, "norm2", 1.0)
    n1.load({"norm1": w1.to(dev)}, ops, torch.float32)
    n2.load({"norm2": w2.to(dev)}, ops, torch.float32)
    block = ParallelPreNormBlock(Adds(100.0), Adds(1.0), n1, n2)
    got = block.forward(x.to(dev).clone(), SimpleNamespace(ops=ops), torch.float32).double().cpu()
    want = x.double() + 100.0 * P.rms_norm(x.double(), w1.double(), 1e-5, True) + P.rms_norm(x.double(), w2.double(), 1e-5, True)
    assert float((got - want).abs().max()) < 1e-4 * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [72, 50, 2048, 1026])
def test_two_norms_in_one_pass(ops, dtype, W):
    g = torch.Generator().manual_seed(W)
    x = torch.randn(11, W, generator=g) * 3
    wa, wb = torch.randn(W, generator=g), torch.randn(W, generator=g)
    a, b = torch.empty(11, W, device="cuda", dtype=dtype), torch.empty(11, W, device="cuda", dtype=dtype)
    ops.rmsnorm_pair(x.cuda(), wa.cuda(), wb.cuda(), 1e-5, a, b)
    one = torch.empty(11, W, device="cuda", dtype=dtype)
    ops.rmsnorm(x.cuda(), wb.cuda(), 1e-5, one)
    torch.cuda.synchronize()
    assert torch.equal(one, b)                               # the same bits as the single norm
    want = P.rms_norm(x.double(), wa.double(), 1e-5)
    assert float((a.double().cpu() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2) * float(want.abs().max())


# ------------------------------------------------------------------------------ through the engine's own entry point
@pytest.mark.parametrize("dtype,name", [("float32", "a"), ("float32", "b"), ("bfloat16", "a")])
def test_greedy_generation_through_the_engine(dtype, name):
    """Six requests on three state slots and a pool that holds two of them at a time, decode steps replayed as CUDA
    graphs, 60 new tokens each: the scheduler admits, preempts and frees; in 32-bit every request's tokens are those
    of the plain implementation decoding greedily (a token whose two best logits are closer than rounding may
    differ: from there on the rest is not compared)."""
    import tffinfer_b200 as tff
    cfg = config(name)
    sd = weights(cfg, sharp=2.0)
    rng = random.Random(2)
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in (3, 40, 17, 64, 9, 25)]
    new = 60
    runner = ModelRunner(config=cfg, tensors=dict(sd), engine_config=EngineConfig(
        dtype=dtype, page_size=PAGE[name], max_cache_tokens=256, max_live_requests=3, use_cuda_graphs=True,
        max_tokens_per_step=48))
    eng = tff.Engine(runner=runner)
    outs = eng.generate(prompts, max_new_tokens=new)
    assert all(len(o) == new for o in outs)
    if dtype != "float32":
        return
    cj = cfg.to_json_dict()
    for p, o in zip(prompts[:3], outs[:3]):
        seq = list(p)
        for i in range(new):
            logits = P.forward(cj, sd, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(logits.abs().max()):
                break
            assert int(logits.argmax()) == o[i], f"token {i} differs"
            seq.append(o[i])


def test_trace_replay_tool_on_a_model_folder(tmp_path):
    """bin/trace_run on a Nugosun folder written by the random-weights mode: a mixed schedule (portions beside single
    tokens, four live requests, a pool that makes later requests reuse pages and slots) in both number formats."""
    import numpy as np
    from test_trace_run_gpu import _replay, _max_tokens
    from helpers import steps_to_jsonl
    from tffinfer_b200.weights import write_random_model
    from tffinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = config("d")
    d = write_random_model(str(tmp_path / "model"), cfg, seed=5)
    f = SafetensorsFile(str(tmp_path / "model" / "model.safetensors"))
    sd = {n: f.tensor(n).clone() for n in f.names()}
    rng = random.Random(9)
    prompts = [70, 3, 130, 41, 18]
    reqs = {f"q{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + 10)] for i, n in enumerate(prompts)}
    want = {r: P.forward(cfg.to_json_dict(), sd, t) for r, t in reqs.items()}
    steps = trace_mixed(reqs, prompts, max_live=4, page_size=64, pool_tokens=384, chunk=33)
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        out.mkdir()
        assert _replay(d, dtype, _max_tokens(reqs, steps), steps_to_jsonl(reqs, steps), str(out)) == 0
        got = {r: [None] * len(t) for r, t in reqs.items()}
        for i, (entries, _) in enumerate(steps):
            rows = sum(n for _, _, n in entries)
            arr = torch.from_numpy(np.fromfile(str(out / f"{i}.f32"), dtype="<f4").reshape(rows, cfg.vocab_size))
            row = 0
            for r, start, n in entries:
                for k in range(n):
                    got[r][start + k] = arr[row]
                    row += 1
        for r in reqs:
            assert first_bad(torch.stack(got[r]), want[r], TOL[dtype]) is None, (dtype, r)


def test_command_line_generates(tmp_path):
    import json
    import subprocess
    import sys
    import os
    from tffinfer_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "model"), config("b"), seed=1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "tffinfer_b200", d, "--prompt-ids", "1,2,3,4,5", "--prompt-ids", "7,8",
                        "--n-predict", "12", "--max-live", "2", "--max-cache-tokens", "128", "--json"],
                       cwd=root, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = json.loads(p.stdout.strip().splitlines()[-1])
    assert [len(o) for o in out["outputs"]] == [12, 12]


# ------------------------------------------------------------------------------ configurations drawn at random
def draw(seed: int):
    """Layer orders, sizes and constants drawn at random: which products run (tensor-core or FMA) follows from the sizes."""
    rng = random.Random(seed)
    W = rng.choice([64, 96, 128, 192]) if rng.random() < 0.75 else rng.choice([36, 100, 150])
    n_layers = rng.choice([2, 3, 4, 6])
    heads = rng.choice([1, 2, 4, 8])
    dim, rot = rng.choice([8, 16, 32, 24]), rng.choice([4, 8, 16, 32])
    latent = dict(heads=heads, dim=dim, rot_dim=rot, vdim=rng.choice([8, 16, 40, 64]), q_rank=rng.choice([8, 24, 48, 13]),
                  kv_rank=rng.choice([16, 32, 72, 128, 27]), scale=rng.choice([None, 0.11, 0.3]),
                  base=rng.choice([1e4, 5e5]), rot_dims=rng.choice([0, 0, rot // 2 // 2 * 2 or rot]))
    a_heads = rng.choice([1, 2, 4, 6])
    a_kv = rng.choice([h for h in (1, 2, 3, 4, 6) if a_heads % h == 0])
    a_dim = rng.choice([16, 32, 64, 48])
    a_rot = rng.choice([None, RotaryConfig(rng.choice([1e4, 3e5]), rng.choice([4, 8, a_dim])),
                        RotaryConfig(1e4, rng.choice([8, a_dim]), (rng.choice([2.0, 8.0]), 256.0, 32.0, 1.0))])
    s_heads = rng.choice([1, 2, 4, 6])
    s_groups = rng.choice([h for h in (1, 2, 3) if s_heads % h == 0])
    s_vdim = rng.choice([8, 16, 24, 64])
    parallel = dict(heads=a_heads, kv=a_kv, dim=a_dim, vdim=a_dim if rng.random() < 0.5 else rng.choice([16, 32, 96]),
                    chunk=rng.choice([0, 1, 5, 16, 33, 64, 100]), scale=rng.choice([a_dim ** -0.5, 0.2, 0.5]),
                    cap=rng.choice([0.0, 5.0, 50.0]), rot=a_rot, s_heads=s_heads, s_vdim=s_vdim,
                    s_state=rng.choice([4, 16, 48, 100]), groups=s_groups, conv=rng.choice([1, 2, 4]),
                    parts=rng.choice([p for p in (1, 2, 4, s_heads) if (s_heads * s_vdim) % p == 0]),
                    ls=rng.choice([1.0, 0.6]), rs=rng.choice([1.0, 1.3]))
    gated = dict(heads=rng.choice([1, 2, 4]), dim=rng.choice([8, 16, 32, 100]), vdim=rng.choice([8, 16, 64, 36]),
                 tau=rng.choice([1.0, 4.0, 16.0]), rank=rng.choice([4, 8, 16, 7]))
    E = rng.choice([1, 4, 8, 12])
    moe = NugosunMlp("moe", rng.choice([16, 64, 40]), E, rng.randint(1, min(E, 4)))
    dense = NugosunMlp("dense", rng.choice([32, 100, 256]))
    layers, own = [], []
    for i in range(n_layers):
        m = rng.choice([moe, dense, moe, dense, None])
        kind = rng.choice(["gla", "parallel", "latent"])
        if kind == "latent":
            src = rng.choice(own) if own and rng.random() < 0.4 else None
            if src is None:
                own.append(i)
            layers.append(lat(kv_from=src, mlp=m, **latent))
        elif kind == "parallel":
            layers.append(par(mlp=m, **parallel))
        else:
            layers.append(gla(mlp=m, **gated))
    cfg = NugosunConfig("Nugosun", vocab_size=rng.choice([97, 256, 311, 1000]), hidden_size=W,
                        embed_scale=rng.choice([1.0, W ** 0.5]), norm_eps=rng.choice([1e-6, 1e-5]), layers=tuple(layers))
    return cfg, rng.choice([8, 16, 32]), [rng.randint(1, 40), rng.randint(60, 150), rng.randint(2, 230), rng.randint(20, 90)]


@pytest.mark.parametrize("seed", list(range(1, 17)))
def test_random_configuration_matches_plain(seed):
    cfg, page, prompts = draw(seed)
    sd = weights(cfg, seed=seed, sharp=3.0)
    rng = random.Random(50 + seed)
    reqs = {f"r{i}": [rng.randrange(cfg.vocab_size) for _ in range(n + 5)] for i, n in enumerate(prompts)}
    cj = cfg.to_json_dict()
    most = max(-(-len(t) // page) * page for t in reqs.values())
    pool = most + most // 2
    for dtype in ("float32", "bfloat16"):
        want = plain_logits(cj, sd, reqs, dtype)
        for steps, tokens in ((trace_mixed(reqs, prompts, max_live=3, page_size=page, pool_tokens=pool, chunk=48), pool),
                              (trace_portions(reqs, sizes=(64, 2, 17, 130, 3)), most)):
            got = run_trace(runner_of(cfg, sd, dtype, page, tokens, live=3), reqs, steps, poison=True)
            for q in reqs:
                assert_within(got[q], want[q], f"draw {seed} {dtype}: request {q}: {cj}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graph_replay(dtype):
    """Two requests decoded for 300 tokens, one token a step, the steps replayed as CUDA graphs: the blocks of the
    chunked attention pass over decoded tokens many times, pages are given back behind them, and the states of the
    recurrences and the convolution's rows are carried all the way."""
    cfg = config("a")
    sd = weights(cfg)
    rng = random.Random(4)
    reqs = {r: [rng.randrange(cfg.vocab_size) for _ in range(n + 300)] for r, n in (("r0", 21), ("r1", 3))}
    want = plain_logits(cfg.to_json_dict(), sd, reqs, dtype)
    steps = [([("r0", 0, 21), ("r1", 0, 3)], [])]
    steps += [([("r0", 21 + i, 1), ("r1", 3 + i, 1)], ["r0", "r1"] if i == 299 else []) for i in range(300)]
    r = runner_of(cfg, sd, dtype, 16, 2 * 336, live=2, graphs=True)
    got = run_trace(r, reqs, steps, poison=True)
    assert any(st["graphs"] for st in r._graphs.values()), "the decode steps were not replayed as graphs"
    for q in reqs:
        assert_within(got[q], want[q], f"{dtype}: request {q}")
