"""Sunosun's configuration, its spec, the cache's bookkeeping for its recurrent state, and the plain implementation's
own invariants (no GPU)."""
import copy
import math

import pytest
import torch

import wick_b200 as wick
from wick_b200.cache import Cache
from wick_b200.config.base import ConfigError
from wick_b200.weights.loader import WeightError, load_weights
from wick_b200.weights.safetensors_io import SafeTensorsDir, write_safetensors
from helpers import tmp_root
from plain import sunosun_plain as P

MOE = {"kind": "moe", "expert": {"ff": 12}, "shared": {"ff": 20},
       "router": {"experts": 6, "top": 3, "scale": 2.5, "groups": {"count": 3, "keep": 2}}}
GLA = dict(heads=3, dim=8, vdim=4, tau=4.0, rank=5)
LEFT = dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.3)
CONFIG = dict(architecture="Sunosun", vocab=97, width=32, norm={"eps": 1e-5}, embedding={"scale": 2.0}, logit_softcap=9.0,
              loop={"start": 1, "stop": 3, "times": 2}, layers=[
    dict(type="gla", mixer=GLA, mlp={"kind": "dense", "ff": 40}),
    dict(type="parallel", mixer=dict(left=LEFT, right=dict(heads=2, dim=4, vdim=10, tau=1.0), left_scale=0.7, right_scale=1.3), mlp=None),
    dict(type="gla", mixer=dict(heads=1, dim=6, vdim=6, tau=16.0), mlp={"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 3, "top": 1, "scale": 1.0}}),
    dict(type="gla", mixer=GLA, mlp=MOE),
])


def test_config_round_trip_and_registry():
    cfg = wick.config_from_json(CONFIG)
    assert isinstance(cfg, wick.SunosunConfig) and cfg.vocab == 97 and len(cfg.layers) == 4
    assert cfg.embedding_scale == 2.0 and cfg.logit_softcap == 9.0 and cfg.norm_eps == 1e-5
    assert cfg.layers[0].mixer.rank == 5 and cfg.layers[1].mixer.right.rank == 0 and cfg.layers[1].mlp is None
    assert cfg.layers[3].mlp.group_count == 3 and cfg.layers[3].mlp.group_keep == 2 and cfg.layers[3].mlp.shared_ff == 20
    assert cfg.layers[2].mlp.group_count == 0 and cfg.layers[2].mlp.shared_ff == 0 and cfg.layers[0].mlp.kind == "dense"
    assert [i for i, _ in cfg.run_order()] == [0, 1, 2, 1, 2, 3] and [t for _, t in cfg.run_order()] == [None, 0, None, 1, None, None]
    assert wick.config_from_json(cfg.to_json()) == cfg
    assert "Sunosun" in wick.architecture_names()
    bare = copy.deepcopy(CONFIG)
    for k in ("loop", "logit_softcap", "embedding"):
        bare.pop(k)
    c2 = wick.config_from_json(bare)
    assert c2.loop is None and c2.logit_softcap is None and c2.embedding_scale == 1.0
    assert [i for i, _ in c2.run_order()] == [0, 1, 2, 3] and all(t is None for _, t in c2.run_order())
    assert wick.config_from_json(c2.to_json()) == c2


@pytest.mark.parametrize("breakage", [
    lambda c: c.pop("vocab"), lambda c: c.pop("norm"), lambda c: c["layers"][0]["mixer"].pop("tau"),
    lambda c: c["layers"][0].update(type="attention"), lambda c: c["layers"][0]["mlp"].update(kind="gated"),
    lambda c: c["layers"][0]["mlp"].pop("ff"), lambda c: c["layers"][1]["mixer"]["left"].update(heads=3),
    lambda c: c["layers"][1]["mixer"].pop("right_scale"), lambda c: c["layers"][1]["mixer"]["left"].pop("scale"),
    lambda c: c["layers"][3]["mlp"]["router"].update(top=7), lambda c: c["layers"][3]["mlp"]["router"].pop("scale"),
    lambda c: c["layers"][3]["mlp"]["router"]["groups"].update(count=4), lambda c: c["layers"][3]["mlp"]["router"]["groups"].update(keep=1),
    lambda c: c["layers"][3]["mlp"]["router"]["groups"].update(keep=4), lambda c: c["layers"][3]["mlp"]["expert"].pop("ff"),
    lambda c: c["loop"].update(stop=5), lambda c: c["loop"].update(start=3), lambda c: c["loop"].pop("times"),
    lambda c: c.update(layers=[])])
def test_broken_configs_are_refused(breakage):
    c = copy.deepcopy(CONFIG)
    breakage(c)
    with pytest.raises(ConfigError):
        wick.config_from_json(c)


def test_spec_names_every_tensor_and_gives_every_pass_a_state_of_its_own():
    cfg = wick.config_from_json(CONFIG)
    spec = wick.get_architecture("Sunosun").build_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert [e.before for e in spec.schedule] == [None, "pass_offset", None, "pass_offset", None, None]
    assert [e.before_index for e in spec.schedule] == [0, 0, 0, 1, 0, 0]
    assert spec.layers[1].ffn.kind == "none" and spec.layers[0].ffn.kind == "gated_mlp" and spec.layers[3].ffn.kind == "routed_moe"
    assert spec.head.params["tied"] and spec.head.params["soft_cap"] == 9.0
    m = wick.Model(spec, torch.float32, "cpu")
    table = m.tensor_table()
    names = set(table)
    for n in ("embed", "loop.step", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g", "l0.mix.o",
              "l0.mix.norm", "l0.mix.a1", "l0.mix.a2", "l0.mix.a2.b", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.left.q",
              "l1.mix.left.q.b", "l1.mix.left.k.b", "l1.mix.left.v.b", "l1.mix.left.o", "l1.mix.right.a1", "l1.mix.right.norm",
              "l2.mlp.e2.up", "l2.mlp.e0.down", "l2.mlp.router", "l2.mlp.correction", "l3.mlp.e5.up", "l3.mlp.shared.up",
              "l3.mlp.shared.down", "l3.mlp.shared.sg"):
        assert n in names, n
    for n in ("l1.norm2", "l1.mix.left.sink", "l2.mlp.e0.gate", "l2.mlp.shared.up", "l2.mlp.shared.sg", "l3.mlp.e6.up", "l1.mlp.up"):
        assert n not in names or table[n].optional, n
    assert table["l0.mix.a1"].shape == (5, 32) and table["l0.mix.a2"].shape == (24, 5) and table["loop.step"].shape == (2, 32)
    assert table["l1.mix.right.a1"].shape == (-1, 32) and table["l1.mix.right.a2"].shape == (8, -1)      # (the checkpoint decides)
    assert table["l3.mlp.shared.sg"].shape == (1, 32) and table["l3.mlp.router"].shape == (6, 32)
    needs = m.cache_needs()
    assert needs[0].kind == "state" and needs[0].shape == (3 * 8 * 4,) and needs[0].dtype == torch.float32
    assert needs[1].kind == "several" and [p.kind for p in needs[1].parts] == ["paged_kv", "state"]
    assert needs[1].parts[0].v_head_dim == 6 and needs[1].parts[1].shape == (2 * 4 * 10,)
    n_params = sum(math.prod(16 if d == -1 else d for d in ts.shape) for name, ts in table.items() if ts.init != "absent" and not ts.optional)
    assert cfg.param_count() == n_params


def test_the_cache_places_every_pass():
    cfg = wick.config_from_json(CONFIG)
    m = wick.Model(wick.get_architecture("Sunosun").build_spec(cfg), torch.float32, "cpu")
    cache = Cache(m.cache_needs(), max_tokens=256, dtype=torch.float32, device="cpu", allocate=False)
    kinds = sorted((g.need.kind, tuple(g.need.shape), len(g.entries)) for g in cache.groups)
    # layer 0 and layer 3 keep records of one size; the two passes over layers 1 and 2 have records of their own each
    assert kinds == [("paged_kv", (), 2), ("state", (36,), 2), ("state", (80,), 2), ("state", (96,), 2)]
    left, right = cache.entry_place[1]
    left2, right2 = cache.entry_place[3]
    assert left[0] is left2[0] and left[1] != left2[1] and right[0] is right2[0] and right[1] != right2[1]


def test_random_model_folder_loads_into_the_plain_model_and_the_rank_comes_from_the_tensors():
    d = wick.write_random_model(wick.config_from_json(CONFIG), 3, tmp_root() + "/suno-cpu", std=0.3)
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    assert "l1.norm2" not in w and w["loop.step"].shape == (2, 32) and w["l0.mix.a1"].shape == (5, 32)
    assert w["l1.mix.right.a1"].shape == (16, 32) and w["l1.mix.right.a2"].shape == (8, 16)
    toks = list(range(40))
    taps = []
    z = P.forward(CONFIG, w, toks, taps=taps)
    assert z.shape == (40, 97) and len(taps) == 6 and torch.isfinite(z).all() and z.abs().max() <= 9.0
    other = list(toks)
    other[10] = 96
    z2 = P.forward(CONFIG, w, other)                          # causal; the state carries a change to every later position
    assert torch.allclose(z[:10], z2[:10], rtol=0, atol=1e-11) and all((z[i] - z2[i]).abs().max() > 1e-6 for i in range(10, 40))
    # a checkpoint whose decay projections have another rank loads where the configuration leaves the rank open ...
    cfg = wick.config_from_json(CONFIG)
    m = wick.Model(wick.get_architecture("Sunosun").build_spec(cfg), torch.float32, "cpu")
    w2 = dict(w)
    w2["l1.mix.right.a1"], w2["l1.mix.right.a2"] = torch.randn(3, 32), torch.randn(8, 3)
    d2 = tmp_root() + "/suno-cpu-rank3"
    import os, shutil
    os.makedirs(d2, exist_ok=True)
    shutil.copy(os.path.join(d, "config.json"), os.path.join(d2, "config.json"))
    write_safetensors(os.path.join(d2, "model.safetensors"), w2)
    load_weights(m, d2)
    assert m.tensor("l1.mix.right.a1").shape == (3, 32)
    # ... and is refused where the two tensors disagree, or where the configuration names a rank
    w2["l1.mix.right.a2"] = torch.randn(8, 4)
    write_safetensors(os.path.join(d2, "model.safetensors"), w2)
    with pytest.raises(ValueError):
        load_weights(m, d2)
    w3 = dict(w)
    w3["l0.mix.a1"] = torch.randn(6, 32)
    write_safetensors(os.path.join(d2, "model.safetensors"), w3)
    with pytest.raises(WeightError):
        load_weights(m, d2)


def test_plain_mechanisms_on_small_cases():
    pv = P.position_vectors(3, 5, torch.float64)
    assert torch.allclose(pv[0], torch.tensor([0.0, 1.0, 0.0, 1.0, 0.0]).double())
    assert torch.allclose(pv[2, :2], torch.tensor([math.sin(2.0), math.cos(2.0)]).double())
    assert abs(pv[2, 2].item() - math.sin(2.0 * 10000 ** (-2 / 5))) < 1e-12 and abs(pv[2, 4].item() - math.sin(2.0 * 10000 ** (-4 / 5))) < 1e-12
    # one key of score 0 and the further key of score 0: half the weight each
    w = P.one_more_softmax(torch.zeros(1, 1, 1).double(), torch.ones(1, 1, dtype=torch.bool))
    assert torch.allclose(w, torch.full((1, 1, 1), 0.5).double())
    w = P.one_more_softmax(torch.full((1, 1, 1), 200.0).double(), torch.ones(1, 1, dtype=torch.bool))
    assert torch.allclose(w, torch.ones(1, 1, 1).double())
    # a state of one key channel and one value: S_t = a S_(t-1) + k v, o = q S
    q, k, v = torch.ones(3, 1, 1).double(), torch.tensor([1.0, 2.0, 3.0]).double().view(3, 1, 1), torch.tensor([1.0, 1.0, 2.0]).double().view(3, 1, 1)
    a = torch.full((3, 1, 1), 0.5).double()
    o, S = P.decayed_outer_products(q, k, v, a)
    assert torch.allclose(o[:, 0, 0], torch.tensor([1.0, 2.5, 7.25]).double()) and S.item() == 7.25
    # the decay acts on key channels (rows): with a = (1, 0) only the first row keeps the past
    q2 = torch.ones(2, 1, 2).double()
    k2 = torch.ones(2, 1, 2).double()
    v2 = torch.tensor([[[1.0, 10.0]], [[2.0, 20.0]]]).double()
    a2 = torch.tensor([1.0, 0.0]).double().expand(2, 1, 2)
    o2, _ = P.decayed_outer_products(q2, k2, v2, a2)
    assert torch.allclose(o2[1, 0], torch.tensor([1.0 + 2 * 2.0, 10.0 + 2 * 20.0]).double())
    # sigmoid(0)^(1/tau)
    t = {"m.a1": torch.zeros(2, 3).double(), "m.a2": torch.zeros(4, 2).double(), "m.a2.b": torch.zeros(4).double()}
    d = P.decays(torch.ones(1, 3).double(), t, "m.", dict(heads=2, dim=2, tau=4.0))
    assert torch.allclose(d, torch.full((1, 2, 2), 0.5 ** 0.25).double())
    # groups: the best single expert sits in a group whose two largest add up to less than another group's
    r = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    z = torch.logit(torch.tensor([[0.9, 0.05, 0.6, 0.5, 0.1, 0.1]]).double())
    chosen, wts = P.choose_experts(z, torch.zeros(6).double(), r)
    assert sorted(chosen[0].tolist()) == [2, 3] and abs(wts.sum().item() - 3.0) < 1e-9
    # the correction decides the choice, not the weights; negative corrected scores still beat a masked group
    corr = torch.tensor([-2.0, -2.0, -5.0, -5.0, -5.0, -5.0]).double()
    chosen, wts = P.choose_experts(z, corr, r)
    assert sorted(chosen[0].tolist()) == [0, 1]
    assert torch.allclose(wts[0].sort().values, torch.tensor([0.05, 0.9]).double() / 0.95 * 3.0)
    # without groups the two best overall
    chosen, _ = P.choose_experts(z, torch.zeros(6).double(), {"experts": 6, "top": 2, "scale": 1.0})
    assert sorted(chosen[0].tolist()) == [0, 2]
    assert P.relu2(torch.tensor([-1.0, 3.0])).tolist() == [0.0, 9.0]
    assert P.run_order({"layers": [0, 1, 2], "loop": {"start": 0, "stop": 2, "times": 2}}) == [(0, 0), (1, None), (0, 1), (1, None), (2, None)]
