"""The Zudepel configuration on the CPU: what config.json keys are read, what may be absent, what is refused, which tensors a
model declares, the round trip through a model folder, a layer that asks the cache for pages and a state, and the plain
implementation's own pieces."""
import copy
import json
import os

import pytest
import torch

import plain_zudepel as plain
import zudepel_cases as zc
from tileinfer_b200.config import ConfigError, ZudepelConfig, config_from_dict, resolve_architecture
from tileinfer_b200.engine.model import tensor_declarations


def test_registry_resolves_the_design_by_its_name():
    assert resolve_architecture({"architecture": "Zudepel"}).config_class is ZudepelConfig
    assert resolve_architecture({"architectures": ["Zudepel"]}).config_class is ZudepelConfig
    assert resolve_architecture({"architecture": "Vogilix"}).name == "Vogilix"


@pytest.mark.parametrize("name", sorted(zc.CASES))
def test_round_trip_and_lowering(name):
    case = zc.CASES[name]
    cfg = config_from_dict(case)
    assert ZudepelConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict() == case
    spec = cfg.model_spec()
    assert spec.options["residual_dtype"] == "float32" and spec.embedding_kind == "lookup32" and spec.final_norm.kind == "rmsnorm32"
    for l, raw in zip(spec.layers, case["layers"]):
        m = raw["mixer"]
        assert l.block == "parallel" and l.feed_forward_norm is None and (l.feed_forward is None) == (raw["mlp"] is None)
        assert (l.mixer.num_heads, l.mixer.head_dim, l.mixer.options["value_dim"]) == (m["heads"], m["dim"], m["vdim"])
        if raw["type"] == "lightning":
            assert l.mixer.kind == "lightning" and list(l.mixer.options["decay"]) == m["decay"]
        else:
            assert l.mixer.kind == "conv_attention" and l.mixer.scale == m["scale"] and l.mixer.kv_source == m.get("kv_from")
            assert l.mixer.options["conv_taps"] == m.get("conv", 0) and l.mixer.num_kv_heads == m["kv_heads"]
            if "rot" in m:
                assert l.mixer.position.options["rotary_dim"] == m["rot"]["dims"] and l.mixer.position.theta == m["rot"]["base"]
            else:
                assert l.mixer.position.kind == "none"
        if raw["mlp"] and raw["mlp"]["kind"] == "moe":
            r, o = raw["mlp"]["router"], l.feed_forward.options
            g = r.get("groups") or {"count": 1, "keep": 1}
            assert (o["experts"], o["top"], o["pass_through"], tuple(o["groups"])) == (r["experts"], r["top"], r.get("identity", 0), (g["count"], g["keep"]))
            assert o["shared_size"] == (raw["mlp"].get("shared") or {}).get("ff", 0) and o["score"] == "softmax" and o["renormalize"]


def test_declared_tensors():
    decls = {d.name: tuple(d.shape) for d in tensor_declarations(config_from_dict(zc.CASE_A).model_spec())}
    assert decls["embed"] == (151, 72) and decls["head"] == (151, 72) and decls["final.norm"] == (72,) and decls["l3.norm1"] == (72,)
    assert not any(n.endswith("norm2") for n in decls)
    assert decls["l0.mix.q"] == (60, 72) and decls["l0.mix.k"] == (20, 72) and decls["l0.mix.v"] == (28, 72) and decls["l0.mix.o"] == (72, 84)
    assert decls["l0.mix.q.b"] == (60,) and decls["l0.mix.v.conv"] == (28, 3) and decls["l0.mix.k.norm"] == (20,) and decls["l0.mix.q.norm"] == (60,)
    assert "l0.mix.v.norm" not in decls and decls["l0.mix.sink"] == (6,) and decls["l0.mix.g"] == (84, 72)
    assert decls["l2.mix.q.conv"] == (60, 2) and not any(n.startswith(("l2.mix.k", "l2.mix.v", "l2.mlp")) for n in decls)
    assert decls["l1.mix.q"] == (36, 72) and decls["l1.mix.v"] == (60, 72) and decls["l1.mix.norm"] == (60,) and decls["l1.mix.o"] == (72, 60)
    assert decls["l1.mlp.gate"] == (100, 72) and decls["l1.mlp.down"] == (72, 100)
    assert decls["l0.mlp.router"] == (8, 72) and decls["l0.mlp.correction"] == (8,) and decls["l0.mlp.e5.up"] == (20, 72) and "l0.mlp.e6.up" not in decls
    assert decls["l0.mlp.shared.gate"] == (28, 72) and decls["l0.mlp.shared.sg"] == (1, 72)
    assert decls["l3.mlp.router"] == (5, 72) and not any(n.startswith("l3.mlp.shared") for n in decls)
    c = {d.name for d in tensor_declarations(config_from_dict(zc.CASE_C).model_spec())}
    assert "l0.mix.q.conv" not in c and "l0.mix.q.b" in c and "l1.mlp.router" in c


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="latent"), "not a mixer of this design"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay has 1 entries for 3 heads"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "must name an earlier attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "must name an earlier attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=12), "differ from those of layer 0"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "do not divide"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=12), "rot.dims 12 must be even and at most dim 10"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top 9 of 8 router outputs"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1), "groups"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "not a feed-forward of this design"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("width"), "width"),
])
def test_what_is_refused(edit, text):
    c = copy.deepcopy(zc.CASE_A)
    edit(c)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(c)


def test_model_folder_round_trip(tmp_path):
    folder = zc.write_folder(zc.CASE_C, 5, str(tmp_path / "m"))
    cfg, W = zc.load_folder(folder)
    assert {k: v for k, v in cfg.items() if k != "dtype"} == zc.CASE_C
    decls = tensor_declarations(config_from_dict(cfg).model_spec())
    assert sorted(W) == sorted(d.name for d in decls)
    from tileinfer_b200.weights import load_tensors
    assert sorted(load_tensors(folder, decls)) == sorted(W)
    logits = plain.forward(cfg, W, [3, 1, 4, 1, 5], torch.float32)
    assert logits.shape == (5, 97) and bool(torch.isfinite(logits).all())


def test_a_layer_with_pages_and_a_state_and_a_reader_of_its_pages():
    """A layer may ask the cache for pages and for a fixed-size state; a layer that reads its pages keeps a state of its own."""
    from tileinfer_b200.cache import Cache
    from tileinfer_b200.parts import CacheRequest
    pages = CacheRequest("paged_kv", kv_heads=2, head_dim=16)
    state = lambda c: CacheRequest("state", shape=(3, c), dtype=torch.float32)
    big = CacheRequest("state", shape=(2, 4, 8), dtype=torch.float32)
    cache = Cache([(pages, state(10)), big, (state(6),), None, (pages, state(10))], torch.float32, "cpu", max_tokens=256, max_seqs=3,
                  share={2: 0, 3: 0})
    assert len(cache.groups) == 4 and len(cache.paged_groups) == 1
    v0, v1, v2, v3, v4 = (cache.layer(i) for i in range(5))
    assert v0.k.shape[1:] == (2, 64, 16) and tuple(v0.state.shape) == (3, 3, 10) and v4.state.shape == v0.state.shape
    assert v0.k.data_ptr() != v4.k.data_ptr() and v0.state.data_ptr() != v4.state.data_ptr()
    assert v1.k is None and tuple(v1.state.shape) == (3, 2, 4, 8)
    assert v2.k.data_ptr() == v0.k.data_ptr() and tuple(v2.state.shape) == (3, 3, 6)        # the source's pages, its own state
    assert v3.k.data_ptr() == v0.k.data_ptr() and v3.state is None                          # a reader without a state sees none
    assert v2.group_index == v0.group_index == v3.group_index
    slot = cache.alloc_slot()
    v0.state[slot].fill_(1.0); v1.state[slot].fill_(2.0)
    cache.free_slot(slot)
    assert cache.alloc_slot() == slot and float(v0.state[slot].abs().max()) == 0.0 and float(v1.state[slot].abs().max()) == 0.0
    with pytest.raises(ValueError, match="two storages of the same kind"):
        Cache([(state(4), big)], torch.float32, "cpu")


def test_plain_pieces():
    """The plain implementation against formulas written out by hand at tiny sizes."""
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=torch.float64)
    c = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = plain.causal_conv(u, c)
    assert y.tolist() == [[100.0, 10.0], [210.0, 20.0], [321.0, 30.0]]
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64).repeat(2, 1, 1)
    r = plain.rotate(x, torch.tensor([0, 1]), 4, 100.0)
    assert torch.allclose(r[0], x[0]) and float(r[1, 0, 4]) == 5.0
    a0, a1 = 1.0, 100.0 ** -0.5
    import math
    assert abs(float(r[1, 0, 0]) - (1 * math.cos(a0) - 3 * math.sin(a0))) < 1e-12 and abs(float(r[1, 0, 3]) - (4 * math.cos(a1) + 2 * math.sin(a1))) < 1e-12
    # A router whose corrections make every choice score negative, and whose best group is not the one with the largest softmax value.
    W = {"r.router": torch.eye(4), "r.correction": torch.tensor([-1.0, -1.0, -0.2, -0.9])}
    h = torch.tensor([[3.0, 0.0, 0.0, 1.0]], dtype=torch.float64)
    mlp = {"router": {"experts": 3, "identity": 1, "top": 1, "groups": {"count": 2, "keep": 1}}}
    chosen, w, margin = plain.route(h, W, "r.", mlp, torch.float32)
    assert chosen.tolist() == [[2]] and abs(float(w[0, 0]) - 1.0) < 1e-12                  # group 1 wins by -0.2 + s2; its weight alone sums to one
    mlp["router"]["top"] = 2
    chosen, w, _ = plain.route(h, W, "r.", mlp, torch.float32)
    s = torch.softmax(h, -1)[0]
    assert chosen.tolist() == [[2, 3]] and abs(float(w[0, 1]) - float(s[3] / (s[2] + s[3]))) < 1e-12


def test_the_command_line_writes_a_model_folder_of_this_design(tmp_path, capsys):
    """``tileinfer random config.json out`` goes through the registry: a Zudepel config.json gives a folder that loads back."""
    from tileinfer_b200.cli import cli
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(zc.CASE_C))
    out = tmp_path / "model"
    assert cli(["random", str(cfg_path), str(out), "--seed", "3"]) == 0
    cfg, W = zc.load_folder(str(out))
    assert cfg["architecture"] == "Zudepel" and W["l1.mix.norm"].shape == (16,) and W["l1.mlp.router"].shape == (4, 64)
