"""Fasunex's configuration, its spec, the cache's bookkeeping for mixers side by side, and the plain implementation's
own invariants (no GPU)."""
import copy
import math

import pytest
import torch

import wick_b200 as wick
from wick_b200.cache import Cache
from wick_b200.config.base import ConfigError
from wick_b200.weights.safetensors_io import SafeTensorsDir
from helpers import tmp_root
from plain import fasunex_plain as P

MOE = {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "identity": 2, "top": 3}}
LEFT = dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.3, mask={"size": 7}, rot={"dims": 4, "base": 50.0})
RIGHT = dict(heads=3, vdim=4, state=5, groups=3, conv=3, norm_groups=2)
CONFIG = dict(architecture="Fasunex", vocab=97, width=32, norm={"eps": 1e-5}, loop={"start": 1, "stop": 3, "times": 2}, layers=[
    dict(type="attention", mixer=dict(heads=2, kv_heads=1, dim=8, vdim=8, scale=0.4), mlp=MOE),
    dict(type="parallel", mixer=dict(left=LEFT, right=RIGHT, left_scale=0.7, right_scale=1.3), mlp=None),
    dict(type="attention", mixer=dict(heads=4, kv_heads=4, dim=4, vdim=4, scale=0.5),
         mlp={"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 3, "top": 1}}),
    dict(type="parallel", mixer=dict(left=LEFT, right=RIGHT, left_scale=1.0, right_scale=-0.5), mlp=MOE),
])


def test_config_round_trip_and_registry():
    cfg = wick.config_from_json(CONFIG)
    assert isinstance(cfg, wick.FasunexConfig) and cfg.vocab == 97 and len(cfg.layers) == 4
    assert cfg.layers[1].mixer.left.mask_size == 7 and cfg.layers[1].mixer.left.rot_dims == 4 and cfg.layers[1].mlp is None
    assert cfg.layers[1].mixer.right.channels == 12 + 2 * 15 and cfg.layers[3].mixer.right_scale == -0.5
    assert cfg.layers[0].mlp.identity == 2 and cfg.layers[2].mlp.identity == 0 and cfg.layers[2].mlp.top == 1
    assert [i for i, _ in cfg.run_order()] == [0, 1, 2, 1, 2, 3] and [e for _, e in cfg.run_order()] == [False, True, False, True, False, False]
    assert wick.config_from_json(cfg.to_json()) == cfg
    assert "Fasunex" in wick.architecture_names()
    bare = copy.deepcopy(CONFIG)
    bare.pop("loop")
    bare["layers"][1]["mixer"]["left"].pop("mask")
    bare["layers"][1]["mixer"]["left"].pop("rot")
    c2 = wick.config_from_json(bare)
    assert c2.loop is None and c2.layers[1].mixer.left.mask_size is None and c2.layers[1].mixer.left.rot_dims == 0
    assert [i for i, _ in c2.run_order()] == [0, 1, 2, 3] and not any(e for _, e in c2.run_order())
    assert wick.config_from_json(c2.to_json()) == c2


@pytest.mark.parametrize("breakage", [
    lambda c: c.pop("vocab"), lambda c: c.pop("norm"), lambda c: c["layers"][0]["mixer"].pop("scale"),
    lambda c: c["layers"][0].update(type="recurrent"), lambda c: c["layers"][0]["mlp"].update(kind="dense"),
    lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), lambda c: c["layers"][0]["mixer"].update(vdim=6),
    lambda c: c["layers"][1]["mixer"].pop("left_scale"), lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=3),
    lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=10), lambda c: c["layers"][1]["mixer"]["right"].update(groups=2),
    lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5), lambda c: c["layers"][1]["mixer"]["right"].pop("state"),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=8), lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"),
    lambda c: c["loop"].update(stop=5), lambda c: c["loop"].update(start=3), lambda c: c["loop"].pop("times"),
    lambda c: c.update(layers=[])])
def test_broken_configs_are_refused(breakage):
    c = copy.deepcopy(CONFIG)
    breakage(c)
    with pytest.raises(ConfigError):
        wick.config_from_json(c)


def test_spec_names_every_tensor_and_gives_every_pass_a_cache_of_its_own():
    cfg = wick.config_from_json(CONFIG)
    spec = wick.get_architecture("Fasunex").build_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert [e.before for e in spec.schedule] == [None, "pass_input", None, "pass_input", None, None]
    assert all(e.read_cache_of is None for e in spec.schedule)
    assert spec.layers[1].ffn.kind == "none" and spec.layers[0].mixer.params["values"] == "keys"
    m = wick.Model(spec, torch.float32, "cpu")
    names = set(m.tensor_table())
    for n in ("embed", "loop.in", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.k",
              "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.e4.gate", "l0.mlp.e0.up", "l0.mlp.e2.down",
              "l0.mlp.router", "l0.mlp.correction", "l1.mix.left.q", "l1.mix.left.k", "l1.mix.left.v", "l1.mix.left.sink", "l1.mix.left.g",
              "l1.mix.left.o", "l1.mix.right.in", "l1.mix.right.conv", "l1.mix.right.conv.b", "l1.mix.right.dt_bias", "l1.mix.right.A_log",
              "l1.mix.right.D", "l1.mix.right.norm", "l1.mix.right.o", "l1.norm1b", "l2.mlp.e2.gate"):
        assert n in names, n
    for n in ("l0.mix.v", "l1.mix.left.q.norm", "l0.mlp.e5.gate", "l2.mlp.e3.gate"):
        assert n not in names, n
    table = m.tensor_table()
    assert table["l0.mlp.router"].shape == (7, 32) and table["l2.mlp.router"].shape == (3, 32) and table["loop.in"].shape == (32, 64)
    assert table["l1.mix.right.in"].shape == (2 * 12 + 2 * 15 + 3, 32) and table["l1.mix.right.conv"].shape == (42, 3)
    needs = m.cache_needs()
    assert needs[0].kind == "paged_kv" and (needs[0].kv_heads, needs[0].head_dim) == (1, 8)
    assert needs[1].kind == "several" and [p.kind for p in needs[1].parts] == ["paged_kv", "state"]
    assert needs[1].parts[0].v_head_dim == 6 and needs[1].parts[1].shape == (2 * 42 + 3 * 4 * 5,) and needs[1].parts[1].dtype == torch.float32
    n_params = sum(math.prod(ts.shape) for name, ts in table.items() if ts.init != "absent")
    assert cfg.param_count() == n_params


def test_the_cache_places_every_branch_of_every_pass():
    cfg = wick.config_from_json(CONFIG)
    m = wick.Model(wick.get_architecture("Fasunex").build_spec(cfg), torch.float32, "cpu")
    cache = Cache(m.cache_needs(), max_tokens=256, dtype=torch.float32, device="cpu", allocate=False)
    kinds = sorted((g.need.kind, len(g.entries)) for g in cache.groups)
    # the three runs of a parallel layer (two passes over layer 1, layer 3) share one group of pages and one of records
    assert kinds == [("paged_kv", 1), ("paged_kv", 2), ("paged_kv", 3), ("state", 3)]
    left, right = cache.entry_place[1]
    left2, right2 = cache.entry_place[3]
    assert left[0] is left2[0] and left[1] != left2[1] and right[0] is right2[0] and right[1] != right2[1]


def test_random_model_folder_loads_into_the_plain_model():
    d = wick.write_random_model(wick.config_from_json(CONFIG), 3, tmp_root() + "/fas-cpu", std=0.3)
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    assert "l1.norm2" not in w and "l1.norm2b" not in w and w["loop.in"].shape == (32, 64) and w["l1.mix.right.conv"].shape == (42, 3)
    toks = list(range(40))
    taps = []
    z = P.forward(CONFIG, w, toks, taps=taps)
    assert z.shape == (40, 97) and len(taps) == 6 and torch.isfinite(z).all()
    other = list(toks)
    other[10] = 96
    z2 = P.forward(CONFIG, w, other)                          # causal; the recurrence carries a change to every later position
    assert torch.equal(z[:10], z2[:10]) and all(not torch.equal(z[i], z2[i]) for i in range(10, 40))


def test_plain_mechanisms_on_small_cases():
    assert P.visible(5, 2).int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 0, 1]]
    assert P.visible(3, None).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    w = P.sink_softmax(torch.zeros(1, 1, 1).double(), torch.ones(1, 1, dtype=torch.bool), torch.tensor([0.0]).double())
    assert torch.allclose(w, torch.full((1, 1, 1), 0.5).double())
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]]).double()
    r = P.rotate_halves(x, torch.tensor([1]), 2, 1.0)         # the pair (0, 1) turns by one radian; the rest passes
    assert torch.allclose(r[0, 0], torch.tensor([0.5403023, 0.8414710, 5.0, 7.0]).double(), atol=1e-6)
    u = torch.tensor([[1.0], [2.0], [4.0]]).double()
    c = P.causal_conv(u, torch.tensor([[0.5, 1.0]]).double(), torch.tensor([0.25]).double())
    assert torch.allclose(c[:, 0], torch.tensor([1.25, 2.75, 5.25]).double())
    assert abs(P.softplus(torch.tensor(0.0)).item() - math.log(2.0)) < 1e-7 and P.softplus(torch.tensor(50.0)).item() == 50.0
    # one expert and one identity output, both chosen: s_0 expert(h) + s_1 h
    t = {"m.router": torch.tensor([[1.0, 0.0], [0.0, 1.0]]).double(), "m.e0.gate": torch.eye(2).double(), "m.e0.up": torch.eye(2).double(),
         "m.e0.down": torch.eye(2).double()}
    h = torch.tensor([[2.0, 0.0]]).double()
    s = torch.softmax(h[0], -1)
    out = P.routed_experts(h, t, "m.", {"router": {"experts": 1, "identity": 1, "top": 2}})
    want = s[0] * (P.silu(h[0]) * h[0]) + s[1] * h[0]
    assert torch.allclose(out[0], want)
    # a state-space head without decay is a running sum: S_t = S_(t-1) + dt B x_t, y_t = C S_t; with z = h the gate is silu(h)
    m = dict(heads=1, vdim=1, state=1, groups=1, conv=1, norm_groups=1)
    big = 40.0                                                # B = C = silu(40) = 40 and dt = softplus(40) = 40, whatever h
    tt = {"s.in": torch.tensor([[1.0], [1.0], [0.0], [0.0], [0.0]]).double(), "s.conv": torch.ones(3, 1).double(),
          "s.conv.b": torch.tensor([0.0, big, big]).double(), "s.dt_bias": torch.tensor([big]).double(),
          "s.A_log": torch.tensor([-60.0]).double(), "s.D": torch.tensor([0.0]).double(), "s.norm": torch.ones(1).double(),
          "s.o": torch.eye(1).double()}
    hh = torch.tensor([[1.0], [2.0], [3.0]]).double()
    y = P.state_space(hh, tt, "s.", m, 1.0)
    run = torch.cumsum(big * big * P.silu(hh[:, 0]), 0) * big * P.silu(hh[:, 0])
    assert torch.allclose(y[:, 0], run / torch.sqrt(run * run + 1.0), rtol=1e-9)
