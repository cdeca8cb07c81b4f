"""The Vogilix configuration on the CPU: what config.json keys are read, what is refused, which tensors a model
declares, the round trip through a model folder, and the plain implementation's own pieces."""
import copy
import json
import os

import pytest
import torch

import plain_vogilix as plain
import vogilix_cases as vc
from tileinfer_b200.config import ConfigError, VogilixConfig, config_from_dict, resolve_architecture
from tileinfer_b200.engine.model import tensor_declarations


def test_registry_resolves_the_design_by_its_name():
    assert resolve_architecture({"architecture": "Vogilix"}).config_class is VogilixConfig
    assert resolve_architecture({"architectures": ["Vogilix"]}).config_class is VogilixConfig
    assert resolve_architecture({"architectures": ["ApertusForCausalLM"]}).name == "ApertusForCausalLM"
    with pytest.raises(ConfigError):
        resolve_architecture({"architecture": "Nothing"})


@pytest.mark.parametrize("name", sorted(vc.CASES))
def test_round_trip_and_lowering(name):
    case = vc.CASES[name]
    cfg = config_from_dict(case)
    assert VogilixConfig.from_dict(cfg.to_dict()) == cfg
    again = cfg.to_dict()
    for key in case:
        assert again[key] == case[key], key
    spec = cfg.model_spec()
    assert spec.options["residual_dtype"] == "float32" and spec.embedding_kind == "lookup_learned_positions"
    assert len(spec.layers) == len(case["layers"])
    for l, raw in zip(spec.layers, case["layers"]):
        m = raw["mixer"]
        assert (l.mixer.num_heads, l.mixer.head_dim, l.mixer.scale) == (m["heads"], m["dim"], m["scale"])
        assert l.mixer.window == (m.get("mask") or {}).get("size")
        assert l.mixer.options["kv_rank"] == m["kv_rank"] and l.mixer.options["value_dim"] == m["vdim"]
        assert (l.feed_forward is None) == (raw["mlp"] is None) and (l.feed_forward_norm is None) == (raw["mlp"] is None)
        assert (l.token_input is None) == ("token_side" not in case)
        assert l.options["residual_mult"] == case.get("residual_mult", 1.0)


def test_declared_tensors():
    decls = {d.name: tuple(d.shape) for d in tensor_declarations(config_from_dict(vc.CASE_A).model_spec())}
    assert decls["embed"] == (151, 72) and decls["pos"] == (512, 72) and decls["head"] == (151, 72) and decls["final.norm"] == (72,)
    assert decls["side.embed"] == (151, 24) and decls["l1.side.gate"] == (8, 72) and decls["l1.side.proj"] == (72, 8)
    assert decls["l0.mix.dq"] == (40, 72) and decls["l0.mix.uq"] == (48, 40) and decls["l0.mix.dkv"] == (48, 72)
    assert decls["l0.mix.uk"] == (48, 48) and decls["l0.mix.uv"] == (72, 48) and decls["l0.mix.o"] == (72, 72)
    assert decls["l2.mix.uk"] == (64, 32) and decls["l2.mix.uv"] == (32, 32) and decls["l2.mix.o"] == (72, 32)
    assert decls["l0.mlp.up"] == (136, 72) and decls["l0.mlp.down"] == (72, 136)
    assert "l1.norm2" not in decls and not any(n.startswith("l1.mlp") for n in decls)
    assert decls["l2.mlp.router"] == (6, 72) and decls["l2.mlp.e5.gate"] == (40, 72) and decls["l2.mlp.e5.down"] == (72, 40)
    assert decls["l2.mlp.shared.up"] == (56, 72) and "l2.mlp.e6.gate" not in decls
    b = {d.name for d in tensor_declarations(config_from_dict(vc.CASE_B).model_spec())}
    assert "side.embed" not in b and not any("shared" in n or "side" in n for n in b)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="ring"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"].update(heads=0), "heads"),
])
def test_refusals(edit, text):
    c = copy.deepcopy(vc.CASE_A)
    edit(c)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(c)


def test_model_folder_round_trip(tmp_path):
    folder = vc.write_folder(vc.CASE_C, 5, str(tmp_path / "m"))
    with open(os.path.join(folder, "config.json")) as f:
        on_disk = json.load(f)
    assert config_from_dict(on_disk) == config_from_dict(vc.CASE_C)
    cfg, W = plain.load_folder(folder)
    assert W["l0.mlp.router"].shape == (5, 60) and W["l0.norm1"].dtype == torch.bfloat16
    assert float(W["l0.norm1"].float().abs().max()) < 1.0            # gains are stored as their distance from one
    logits = plain.forward(cfg, W, [3, 1, 4, 1, 5], torch.float32)
    assert logits.shape == (5, 97) and bool(torch.isfinite(logits).all())


def test_plain_pieces():
    """The plain implementation's mask, norms and the spreading of uncertain router calls."""
    ok = plain.window_mask(6, 3)
    assert ok.tolist() == [[j <= i and i - j < 3 for j in range(6)] for i in range(6)]
    assert plain.window_mask(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]
    y = torch.tensor([[3.0, -4.0]])
    assert torch.allclose(plain.norm_offset(y, torch.tensor([0.0, 1.0]), 0.0), torch.tensor([[3.0, -8.0]]) / 12.5 ** 0.5)
    assert torch.allclose(plain.norm_plain(y, torch.tensor([2.0, 1.0]), 0.0), torch.tensor([[6.0, -4.0]]) / 12.5 ** 0.5)
    cfg = {"layers": [{"mixer": {"mask": {"size": 3}}}, {"mixer": {"mask": {"size": 4}}}, {"mixer": {}}]}
    margins = [(0, torch.tensor([1.0, 1.0, 0.001, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0]))]
    bad = plain.unsure_positions({"layers": cfg["layers"][:2]}, margins, 10, 0.01)
    assert bad.tolist() == [False, False, True, True, True, True] + [False] * 4       # layer 1 carries it 3 further
    bad = plain.unsure_positions(cfg, margins, 10, 0.01)
    assert bad.tolist() == [False, False] + [True] * 8                                 # a layer without window: to the end
    last = plain.unsure_positions(cfg, [(2, margins[0][1])], 10, 0.01)
    assert last.tolist() == [False, False, True] + [False] * 7


def test_command_line_writes_a_model_folder_of_this_design(tmp_path, capsys):
    from tileinfer_b200.cli import cli
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(vc.CASE_B))
    out = tmp_path / "model"
    assert cli(["random", str(cfg), str(out), "--seed", "9"]) == 0 and "wrote" in capsys.readouterr().out
    again, W = plain.load_folder(str(out))
    assert again["architecture"] == "Vogilix" and again["layers"] == vc.CASE_B["layers"]
    assert "residual_mult" in again and again["residual_mult"] == 1.0          # what the file left out is written with its default
    assert W["l1.mlp.e3.up"].shape == (72, 128) and "l1.mlp.shared.up" not in W and "side.embed" not in W
