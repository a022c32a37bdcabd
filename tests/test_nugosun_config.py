"""Host side of the Nugosun design (no GPU): configuration round trip, defaults and errors; the description's tensor
names, cache needs and schedule; a size that only a tensor's shape gives; and the plain implementation against itself
(the recurrences run in two halves, the state space against its definition token by token, a routed feed-forward with
every expert chosen, the convolution's taps, the block mask's edges)."""
import copy

import pytest
import torch

import plain_nugosun as P
from tffinfer_b200.config import NugosunConfig, ConfigError
from tffinfer_b200.parts import Model, KVNeed, StateNeed
from tffinfer_b200.registry import get_architecture
import tffinfer_b200.models  # noqa: F401


def sample_json():
    moe = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}
    dense = {"kind": "dense", "ff": 70}
    latent = {"heads": 3, "dim": 20, "rot_dim": 6, "vdim": 12, "q_rank": 10, "kv_rank": 18, "scale": 0.2,
              "rot": {"base": 1000.0, "dims": 4}}
    par = {"left": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3, "softcap": 11.0, "mask": {"size": 7},
                    "rot": {"base": 5000.0, "dims": 10,
                            "scaling": {"factor": 4.0, "original": 64.0, "fast": 16.0, "slow": 2.0}}},
           "right": {"heads": 3, "vdim": 20, "state": 12, "groups": 3, "conv": 3, "norm_groups": 5},
           "left_scale": 0.75, "right_scale": 0.5}
    gla = {"heads": 3, "dim": 12, "vdim": 20, "tau": 4.0, "rank": 5}
    return {"architecture": "Nugosun", "vocab": 97, "width": 52, "embedding": {"scale": 2.5}, "norm": {"eps": 3e-6},
            "layers": [{"type": "parallel", "mixer": par, "mlp": None},
                       {"type": "latent_attention", "mixer": latent, "mlp": moe},
                       {"type": "gla", "mixer": gla, "mlp": dense},
                       {"type": "latent_attention", "mixer": dict(latent, kv_from=1), "mlp": moe}]}


def test_round_trip_and_defaults():
    cj = sample_json()
    cfg = NugosunConfig.from_json_dict(cj)
    assert cfg.to_json_dict() == cj
    assert cfg.layers[3].latent.kv_from == 1 and cfg.layers[0].left.chunk == 7 and cfg.layers[1].latent.rot.dims == 4
    d = copy.deepcopy(cj)
    left = d["layers"][0]["mixer"]["left"]
    del d["embedding"], left["mask"], left["softcap"], left["kv_heads"], left["rot"], left["scale"]
    del d["layers"][0]["mixer"]["left_scale"], d["layers"][0]["mixer"]["right"]["groups"]
    del d["layers"][0]["mixer"]["right"]["norm_groups"], d["layers"][2]["mixer"]["rank"]
    d["layers"][1]["mixer"]["rot"] = {"base": 1000.0}
    d["layers"][3]["mixer"]["rot"] = {"base": 1000.0}
    c2 = NugosunConfig.from_json_dict(d)
    a = c2.layers[0].left
    assert c2.embed_scale == 1.0 and a.chunk == 0 and a.softcap == 0.0 and a.kv_heads == 6 and a.rot is None
    assert a.scale == 24 ** -0.5 and c2.layers[0].left_scale == 1.0 and c2.layers[0].right.groups == 1
    assert c2.layers[0].right.norm_groups == 1 and c2.layers[1].latent.rot.dims == 6 and c2.layers[2].gla.rank == 0


@pytest.mark.parametrize("edit,word", [
    (lambda d: d["layers"][1].__setitem__("type", "convolution"), "type"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_rank", 20), "equal"),
    (lambda d: d["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["right"].__setitem__("groups", 2), "groups"),
    (lambda d: d["layers"][0]["mixer"]["right"].__setitem__("norm_groups", 7), "norm_groups"),
    (lambda d: d["layers"][0]["mixer"]["right"].pop("state"), "state"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 26), "dims"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("tau", 0.0), "tau"),
    (lambda d: d["layers"][2]["mlp"].pop("ff"), "ff"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_errors_name_the_key(edit, word):
    d = sample_json()
    edit(d)
    with pytest.raises(ConfigError) as e:
        NugosunConfig.from_json_dict(d)
    assert word in str(e.value)


def test_description_names_needs_and_schedule():
    arch = get_architecture("Nugosun")
    cfg = arch.read_config(sample_json())
    desc = arch.describe(cfg)
    model = Model(desc)
    names = model.expected_tensors()
    for n in ("embed", "final.norm", "l0.norm1", "l0.mix.left.q", "l0.mix.left.q.b", "l0.mix.left.v.b", "l0.mix.left.o",
              "l0.mix.right.in", "l0.mix.right.conv", "l0.mix.right.conv.b", "l0.mix.right.dt_bias", "l0.mix.right.A_log",
              "l0.mix.right.D", "l0.mix.right.norm", "l0.mix.right.o", "l1.mix.dkv", "l1.mlp.router", "l1.mlp.router.b",
              "l1.mlp.e4.down", "l2.norm2", "l2.mix.a1", "l2.mix.a2", "l2.mix.a2.b", "l2.mix.norm", "l2.mix.g", "l2.mlp.gate",
              "l3.mix.uk"):
        assert n in names, n
    assert "l0.norm2" not in names and "l3.mix.dkv" not in names and "lm_head" not in names
    assert names["l0.mix.right.in"].shape == (2 * 60 + 2 * 36 + 3, 52) and names["l0.mix.right.conv"].shape == (60 + 72, 3)
    assert names["l2.mix.a1"].shape == (5, 52) and names["l2.mix.a2"].shape == (36, 5) and names["l2.mix.norm"].shape == (20,)
    needs = model.cache_needs()
    assert needs[0] == (KVNeed(2, 40, 7, 2), StateNeed((2 * 132 + 3 * 12 * 20,), "float32"))
    assert needs[1] == KVNeed(1, 24, 0, 1) and needs[2] == StateNeed((3 * 12 * 20,), "float32") and needs[3] is None
    assert [e.cache_of for e in desc.schedule] == [None, None, None, 1]
    assert desc.embed_scale == 2.5 and desc.lm_head_name is None and all(l.block == "parallel_pre_norm" for l in desc.layers)


def test_a_size_that_only_the_file_gives():
    """Without ``rank`` the inner size of the decay's low-rank pair is whatever the tensors hold; the two must agree."""
    from tffinfer_b200.weights.loader import check_tensors, WeightError
    from tffinfer_b200.weights.random_init import random_state_dict
    cj = sample_json()
    cfg = NugosunConfig.from_json_dict(cj)
    sd = random_state_dict(cfg, 3)
    del cj["layers"][2]["mixer"]["rank"]
    open_cfg = NugosunConfig.from_json_dict(cj)
    arch = get_architecture("Nugosun")
    model = Model(arch.describe(open_cfg))
    held = check_tensors(sd, model.expected_tensors(), torch.float32, "cpu")
    assert held["l2.mix.a1"].shape == (5, 52)
    with pytest.raises(ValueError):
        random_state_dict(open_cfg, 3)                         # random weights need the size
    sd["l2.mix.q"] = sd["l2.mix.q"][:-1]
    with pytest.raises(WeightError):
        check_tensors(sd, model.expected_tensors(), torch.float32, "cpu")


def test_package_frequencies_equal_the_plain_ones():
    from tffinfer_b200.parts.position import scaled_frequencies
    for rot in ({"base": 70000.0, "dims": 24, "scaling": {"factor": 6.0, "original": 512, "fast": 24.0, "slow": 0.5}},
                {"base": 1e4, "dims": 64, "scaling": {"factor": 4.0, "original": 64.0, "fast": 16.0, "slow": 2.0}},
                {"base": 5e5, "dims": 6}):
        sc = rot.get("scaling")
        f, mag = scaled_frequencies(rot["dims"], rot["base"], (sc["factor"], sc["original"], sc["fast"], sc["slow"]) if sc else None)
        pf, pmag = P.rescaled_frequencies(rot)
        assert mag == pytest.approx(pmag, rel=1e-12) and f == pytest.approx(pf, rel=1e-12)


def test_plain_recurrence_in_two_halves_and_by_its_definition():
    g = torch.Generator().manual_seed(0)
    T, K, V = 23, 6, 5
    q, k, ld = torch.randn(T, K, generator=g).double(), torch.randn(T, K, generator=g).double(), -torch.rand(T, K, generator=g).double()
    v = torch.randn(T, V, generator=g).double()
    whole, S = P.decayed_outer_recurrence(q, k, v, ld)
    a, Sa = P.decayed_outer_recurrence(q[:9], k[:9], v[:9], ld[:9])
    b, Sb = P.decayed_outer_recurrence(q[9:], k[9:], v[9:], ld[9:], state=Sa)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12) and torch.allclose(S, Sb, atol=1e-12)
    # the closed form: o_t = sum_(s <= t) (q_t . (k_s * prod_(s < u <= t) a_u)) v_s
    cum = torch.cumsum(ld, dim=0)
    for t in (0, 7, 22):
        o = sum(((q[t] * k[s] * torch.exp(cum[t] - cum[s])).sum() * v[s] for s in range(t + 1)))
        assert torch.allclose(o, whole[t], atol=1e-10)


def test_plain_state_space_against_a_direct_loop():
    g = torch.Generator().manual_seed(1)
    W, T = 10, 9
    m = {"heads": 4, "vdim": 3, "state": 5, "groups": 2, "conv": 3, "norm_groups": 2}
    inner, bc = 12, 10
    w = {"p.in": torch.randn(2 * inner + 2 * bc + 4, W, generator=g), "p.conv": torch.randn(inner + 2 * bc, 3, generator=g),
         "p.conv.b": torch.randn(inner + 2 * bc, generator=g), "p.dt_bias": torch.randn(4, generator=g),
         "p.A_log": torch.randn(4, generator=g), "p.D": torch.randn(4, generator=g), "p.norm": torch.randn(inner, generator=g),
         "p.o": torch.eye(inner)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W, generator=g).double()
    got = P.ssd_mixer(h, w, "p", m, 1e-5)
    proj = h @ w["p.in"].T
    z, dt = proj[:, :inner], torch.log1p(torch.exp(proj[:, -4:] + w["p.dt_bias"]))
    u = torch.cat([torch.zeros(2, inner + 2 * bc).double(), proj[:, inner:inner + inner + 2 * bc]])
    xbc = torch.stack([sum(w["p.conv"][:, j] * u[t + j] for j in range(3)) + w["p.conv.b"] for t in range(T)])
    xbc = xbc * torch.sigmoid(xbc)
    S = torch.zeros(4, 5, 3).double()
    rows = []
    for t in range(T):
        y = []
        for hd in range(4):
            gi = hd // 2
            x, B, C = xbc[t, hd * 3:(hd + 1) * 3], xbc[t, inner + gi * 5:inner + (gi + 1) * 5], xbc[t, inner + bc + gi * 5:inner + bc + (gi + 1) * 5]
            S[hd] = torch.exp(-torch.exp(w["p.A_log"][hd]) * dt[t, hd]) * S[hd] + dt[t, hd] * B[:, None] * x[None, :]
            y.append(S[hd].T @ C + w["p.D"][hd] * x)
        y = torch.cat(y) * (z[t] * torch.sigmoid(z[t]))
        y = torch.cat([part / torch.sqrt((part * part).mean() + 1e-5) for part in y.reshape(2, 6)]) * w["p.norm"]
        rows.append(y)
    assert torch.allclose(torch.stack(rows), got, atol=1e-10)


def test_plain_router_with_every_expert_chosen_is_a_softmax_mixture():
    g = torch.Generator().manual_seed(2)
    W, E, ff, T = 8, 3, 5, 4
    w = {"m.router": torch.randn(E, W, generator=g).double(), "m.router.b": torch.randn(E, generator=g).double()}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = (torch.randn(ff, W, generator=g).double(),
                                                                torch.randn(ff, W, generator=g).double(),
                                                                torch.randn(W, ff, generator=g).double())
    h = torch.randn(T, W, generator=g).double()
    got = P.routed_ff(h, w, "m", {"router": {"experts": E, "top": E}})
    p = torch.softmax(h @ w["m.router"].T + w["m.router.b"], dim=-1)
    want = sum(p[:, e:e + 1] * P.gated_ff(h, w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"]) for e in range(E))
    assert torch.allclose(got, want, atol=1e-12)
    one = P.routed_ff(h, w, "m", {"router": {"experts": E, "top": 1}})
    best = (h @ w["m.router"].T + w["m.router.b"]).argmax(dim=-1)
    for t in range(T):
        e = int(best[t])
        assert torch.allclose(one[t], P.gated_ff(h[t:t + 1], w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"])[0], atol=1e-12)


def test_plain_model_runs_on_a_written_folder(tmp_path):
    """A model folder written by the random-weights mode, read back by name, through the plain implementation: the
    logits of a prefix do not change when tokens follow it (every mixer is causal)."""
    from tffinfer_b200.weights import write_random_model
    from tffinfer_b200.weights.safetensors_io import SafetensorsFile
    cfg = NugosunConfig.from_json_dict(sample_json())
    d = write_random_model(str(tmp_path / "m"), cfg, seed=4)
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    sd = {n: f.tensor(n).clone() for n in f.names()}
    toks = [(5 * i * i + 3) % 97 for i in range(30)]
    full = P.forward(sample_json(), sd, toks)
    assert full.shape == (30, 97) and torch.isfinite(full).all()
    assert torch.allclose(P.forward(sample_json(), sd, toks[:17]), full[:17], atol=1e-9)


def test_plain_attention_sees_the_block_edges():
    """A key planted one position inside the query's block is found, one position outside is not.  Queries and keys
    read the first half of the input, values the second: the last token copies the planted token's first half."""
    g = torch.Generator().manual_seed(1)
    W, d = 16, 8
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 4.0, "softcap": 0.0, "mask": {"size": 10}, "rot": None}
    wq = torch.cat([torch.randn(d, d, generator=g), torch.zeros(d, d)], dim=1).double()
    wv = torch.cat([torch.zeros(d, d), torch.randn(d, d, generator=g)], dim=1).double()
    zero = torch.zeros(d).double()
    w = {"p.q": wq, "p.k": wq, "p.v": wv, "p.q.b": zero, "p.k.b": zero, "p.v.b": zero, "p.o": torch.eye(d).double()}
    for aimed, seen in ((20, True), (19, False)):
        h = torch.randn(26, W, generator=g).double()
        h[25, :d] = h[aimed, :d]
        out = P.chunked_attention(h, torch.arange(26), w, "p", m, 1e-6)
        own, other = h[25] @ wv.T, h[aimed] @ wv.T
        if seen:                   # the query finds itself and the planted key alike: half of each value
            assert float((out[25] - 0.5 * (own + other)).abs().max()) < 1e-3 * float(other.abs().max())
        else:                      # the planted key is in the block before: the query finds only itself
            assert float((out[25] - own).abs().max()) < 1e-3 * float(own.abs().max())
