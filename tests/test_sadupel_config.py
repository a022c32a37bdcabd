"""Host-side tests of the Sadupel design: its configuration reader, its model description (tensor names, the order of
layer runs, cache and state needs), the rotation frequencies against the plain implementation's, and properties of the
plain implementation itself that the kernels' restatements rest on."""
import json
import math

import pytest
import torch

import plain_sadupel as P
import tffinfer_b200 as tff
from tffinfer_b200.config import ConfigError, read_config_json
from tffinfer_b200.config.sadupel_config import SadupelConfig, SadupelLayer, SadupelExperts
from tffinfer_b200.parts import Model, KVNeed, StateNeed
from tffinfer_b200.weights import write_random_model
from tffinfer_b200.weights.safetensors_io import SafetensorsFile


def small_config():
    m = SadupelExperts(ff=12, experts=4, top=2, identity=2, groups=3, keep=2, shared_ff=20)
    layers = (SadupelLayer(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, scale=0.25, softcap=15.0, rot_base=1e4, rot_dims=4,
                           rot_factor=2.0, mlp=m),
              SadupelLayer(heads=2, kv_heads=1, dim=16, vdim=8, conv=0, scale=0.3, softcap=0.0, rot_base=1e5, rot_dims=16,
                           rot_factor=1.0, mlp=None),
              SadupelLayer(heads=3, kv_heads=3, dim=6, vdim=6, conv=2, scale=0.4, softcap=5.0, rot_base=500.0, rot_dims=6,
                           rot_factor=4.0, mlp=SadupelExperts(ff=8, experts=3, top=1)))
    return SadupelConfig("Sadupel", vocab_size=50, hidden_size=24, norm_eps=1e-5, residual_mult=0.4, bigram=(13, 5, 7),
                         loop=(1, 3, 2), layers=layers)


def test_config_round_trip_and_defaults():
    cfg = small_config()
    d = cfg.to_json_dict()
    assert SadupelConfig.from_json_dict(json.loads(json.dumps(d))) == cfg
    assert cfg.runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None)]
    bare = {"architecture": "Sadupel", "vocab": 9, "width": 8, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 4, "scale": 0.5, "rot": {"base": 100.0}}, "mlp": None}]}
    c = SadupelConfig.from_json_dict(bare)
    l = c.layers[0]
    assert (l.kv_heads, l.vdim, l.conv, l.softcap, l.rot_dims, l.rot_factor) == (2, 4, 0, 0.0, 4, 1.0)
    assert c.residual_mult == 1.0 and c.bigram is None and c.loop is None and c.runs() == [(0, None)]


@pytest.mark.parametrize("change,key", [
    (lambda d: d["layers"][0].update(type="retention"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), "dims"),
    (lambda d: d["layers"][0]["mixer"].update(conv=9), "conv"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "groups"),
    (lambda d: d["loop"].update(stop=4), "loop"),
    (lambda d: d["embedding"]["bigram"].update(buckets=0), "buckets"),
])
def test_config_errors_name_the_key(change, key):
    d = small_config().to_json_dict()
    change(d)
    with pytest.raises(ConfigError) as e:
        SadupelConfig.from_json_dict(d)
    assert key in str(e.value)


def test_description_names_needs_and_passes():
    cfg = small_config()
    model = Model(tff.get_architecture("Sadupel").describe(cfg))
    names = model.expected_tensors()
    for n, shape in {"embed": (50, 24), "bigram": (14, 24), "loop.step": (2, 24), "head": (50, 24), "final.norm": (24,),
                     "l0.norm1": (24,), "l0.mix.q": (32, 24), "l0.mix.k": (16, 24), "l0.mix.v": (24, 24), "l0.mix.g": (4, 24),
                     "l0.mix.o": (24, 48), "l0.mix.sink": (4,), "l0.mix.q.conv": (32, 3), "l0.mix.v.conv": (24, 3),
                     "l0.mix.q.norm": (32,), "l0.mix.k.norm": (16,), "l0.mlp.router": (6, 24), "l0.mlp.correction": (6,),
                     "l0.mlp.e3.up": (12, 24), "l0.mlp.e3.down": (24, 12), "l0.mlp.shared.up": (20, 24),
                     "l2.mlp.router": (3, 24), "l2.mix.k.conv": (18, 2)}.items():
        assert tuple(names[n].shape) == shape, n
    for n in ("l0.mlp.e4.up", "l1.mlp.router", "l1.mix.q.conv", "l2.mlp.shared.up", "l0.norm2", "l0.mlp.e0.gate"):
        assert n not in names, n
    # every run of a layer keeps pages of its own, and a state where the convolution has more than one tap
    needs = model.cache_needs()
    assert len(needs) == 5
    assert needs[0] == (KVNeed(2, 12, 0), StateNeed((2, 32 + 16 + 24), "float32"))
    assert needs[1] == needs[3] == KVNeed(1, 16, 0)
    assert needs[2] == needs[4] == (KVNeed(3, 6, 0), StateNeed((1, 54), "float32"))
    assert model.extra_state_needs() == [StateNeed((1,), "int32")]
    sched = model.desc.schedule
    assert [e.layer for e in sched] == [0, 1, 2, 1, 2]
    assert [e.add_vector for e in sched] == [None, ("loop.step", 0), None, ("loop.step", 1), None]


def test_random_model_folder_runs_in_the_plain_implementation(tmp_path):
    cfg = small_config()
    d = write_random_model(str(tmp_path / "m"), cfg, seed=3)
    assert SadupelConfig.from_json_dict(read_config_json(d)) == cfg
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    w = {n: f.tensor(n).clone() for n in f.names()}
    layers = []
    logits = P.forward(cfg.to_json_dict(), w, [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], layers_out=layers)
    assert logits.shape == (11, 50) and len(layers) == 5 and torch.isfinite(logits).all()
    from tffinfer_b200.weights.loader import check_tensors, WeightError
    expected = Model(tff.get_architecture("Sadupel").describe(cfg)).expected_tensors()
    with pytest.raises(WeightError) as e:
        check_tensors({n: t for n, t in w.items() if n != "l0.mix.sink"}, expected, torch.float32, "cpu")
    assert "l0.mix.sink" in str(e.value)


@pytest.mark.parametrize("base,dims,factor", [(1e4, 64, 1.0), (3e5, 32, 2.5), (500.0, 6, 16.0)])
def test_frequencies_match_the_plain_ones(base, dims, factor):
    from tffinfer_b200.parts.model import build_part
    desc = tff.get_architecture("Sadupel").describe(SadupelConfig(
        "Sadupel", vocab_size=8, hidden_size=8, norm_eps=1e-5, layers=(SadupelLayer(
            heads=1, kv_heads=1, dim=dims, vdim=4, conv=0, scale=1.0, softcap=0.0, rot_base=base, rot_dims=dims, rot_factor=factor),)))
    part = build_part("position", next(iter(desc.positions.values())))
    part.prepare(None, "cpu", 0)
    f, rot, magnitude, interleaved = part.frequencies()
    want = [base ** (-2.0 * i / dims) / factor for i in range(dims // 2)]
    assert (rot, magnitude, interleaved) == (dims, 1.0, False)
    assert torch.equal(f, torch.tensor(want, dtype=torch.float64).to(torch.float32))
    # the plain rotation turns pair (i, i + dims/2) by position * frequency and leaves the rest of the head
    x = torch.zeros(1, 1, dims + 2, dtype=torch.float64)
    x[0, 0, 1], x[0, 0, dims] = 1.0, 7.0
    y = P.rotate_halves(x, torch.tensor([3]), base, dims, factor)
    assert y[0, 0, 1] == pytest.approx(math.cos(3 * want[1])) and y[0, 0, 1 + dims // 2] == pytest.approx(math.sin(3 * want[1]))
    assert y[0, 0, dims] == 7.0


def test_groups_choose_among_negative_scores():
    """With every choice score below zero, an expert outside the kept groups must not win over the kept ones."""
    h = torch.eye(4, dtype=torch.float64)[:1]
    router = torch.zeros(6, 4, dtype=torch.float64)            # equal scores 1/6
    corr = torch.tensor([-5.0, -1.0, -4.0, -4.5, -0.9, -3.0], dtype=torch.float64)
    idx, w = P.route(h, router, corr, top=2, groups=3, keep=1)
    assert idx.tolist() == [[4, 5]] and torch.allclose(w, torch.full((1, 2), 1 / 6, dtype=torch.float64))
    idx, _ = P.route(h, router, corr, top=2, groups=3, keep=2)
    assert idx.tolist() == [[4, 1]]
    idx, _ = P.route(h, router, torch.zeros(6, dtype=torch.float64), top=3, groups=1, keep=1)
    assert idx.tolist() == [[0, 1, 2]]                          # equal scores: the lower index first


def test_sink_share_and_first_token_of_the_plain_attention():
    one = torch.ones(1, 1, 1, dtype=torch.float64)
    o = P.sink_softmax_attention(torch.zeros(1, 1, 4, dtype=torch.float64), torch.zeros(1, 1, 4, dtype=torch.float64), one,
                                 0.3, 2.0, torch.tensor([1.5], dtype=torch.float64))
    assert float(o) == pytest.approx(1 / (1 + math.exp(1.5)))
    assert P.bigram_rows([4, 9, 2], 7, 3, 5) == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 2 * 5) % 7]
    y = P.causal_conv(torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64), torch.tensor([[2.0, 3.0]], dtype=torch.float64))
    assert y[:, 0].tolist() == [3.0, 32.0, 320.0]
