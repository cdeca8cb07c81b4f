"""Small Zudepel configurations for the tests, their random model folders and the comparison against the plain
implementation (``plain_zudepel``).

The configurations differ from one another in every size and constant, and none keeps two sizes equal that a kernel could
mix up (query/key size and value size, heads and key/value heads, taps, groups and experts).
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_zudepel as plain


def lightning(heads, dim, vdim, decay, mlp):
    return {"mixer": {"decay": decay, "dim": dim, "heads": heads, "vdim": vdim}, "mlp": mlp, "type": "lightning"}


def attention(heads, kv_heads, dim, vdim, scale, mlp, conv=None, rot=None, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if conv:
        m["conv"] = conv
    if rot:
        m["rot"] = {"base": rot[1], "dims": rot[0]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"mixer": m, "mlp": mlp, "type": "attention"}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, top, ff, identity=0, groups=None, shared=0):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if identity:
        r["identity"] = identity
    m = {"expert": {"ff": ff}, "kind": "moe", "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# Odd sizes that no fast kernel takes: key and value sizes differ, three query heads per key/value head, part of a head
# rotated, an attention layer first (routed, with groups, pass-through choices and a shared expert larger than an expert), a
# layer that reads the first layer's keys and values with another number of taps and no feed-forward, lightning layers of
# different shapes, a router without groups, pass-through choices or shared expert that takes one expert.
CASE_A = {
    "architecture": "Zudepel", "vocab": 151, "width": 72, "norm": {"eps": 1e-5},
    "layers": [attention(6, 2, 10, 14, 0.4, moe(6, 3, 20, identity=2, groups=(4, 2), shared=28), conv=3, rot=(6, 500.0)),
               lightning(3, 12, 20, [0.5, 0.9, 0.995], dense(100)),
               attention(6, 2, 10, 14, 0.4, None, conv=2, rot=(6, 500.0), kv_from=0),
               lightning(2, 40, 8, [0.97, 0.75], moe(5, 1, 24))],
}
# Sizes the tensor-core kernels take (widths in steps of 8, heads of 64): lightning first, two query heads per key/value
# head, keys shorter than values (filled up in the pages), one tap (a scale per channel, no state), a whole head rotated,
# every group kept, more pass-through choices than a token takes.
CASE_B = {
    "architecture": "Zudepel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
    "layers": [lightning(2, 32, 64, [0.8, 0.999], moe(8, 2, 64, groups=(2, 1), shared=64)),
               attention(4, 2, 64, 64, 0.125, dense(256), conv=4, rot=(32, 10000.0)),
               attention(4, 1, 32, 64, 0.2, moe(4, 1, 40, identity=4, groups=(4, 4)), conv=1, rot=(32, 100.0)),
               attention(4, 2, 64, 64, 0.11, dense(136), conv=5, rot=(32, 10000.0), kv_from=1)],
}
# What may be absent is absent: no convolution, no rotation, as many key/value heads as heads, one lightning head, a router
# that takes every output it has (a pass-through choice among them).
CASE_C = {
    "architecture": "Zudepel", "vocab": 97, "width": 64, "norm": {"eps": 3e-6},
    "layers": [attention(2, 2, 16, 16, 0.25, dense(48)),
               lightning(1, 16, 16, [0.93], moe(3, 4, 24, identity=1))],
}
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}


def write_folder(case: dict, seed: int, out_dir: str) -> str:
    """A model folder with random weights for ``case``, made without a device. The routers' rows are made three times as
    long as a random matrix's and the corrections ten times as large: choices then rest on gaps that rounding does not
    close at most positions (the weights still come from the softmax alone)."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.weights import write_model_folder
    from tileinfer_b200.weights.safetensors_io import SafetensorsFile, save_file
    write_model_folder(config_from_dict(case), seed, out_dir, device="cpu")
    path = os.path.join(out_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.entries}
    for n in tensors:
        if n.endswith(".mlp.router"):
            tensors[n] = (tensors[n].float() * 3.0).to(tensors[n].dtype)
        if n.endswith(".mlp.correction"):
            tensors[n] = (tensors[n].float() * 10.0).to(tensors[n].dtype)
    del f
    save_file(tensors, path)
    return out_dir


def load_folder(folder):
    """(config dict, tensors) of a model folder, read with the safetensors package."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    W = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            W[k] = f.get_tensor(k)
    return cfg, W


class Model:
    """A case's folder, the plain implementation's view of it and cached reference logits."""

    def __init__(self, name: str, seed: int, tmp: str):
        self.name = name
        self.folder = write_folder(CASES[name], seed, os.path.join(tmp, f"zudepel_{name}_{seed}"))
        self.cfg, self.W = load_folder(self.folder)
        self.vocab = self.cfg["vocab"]
        self._refs = {}

    def reference(self, tokens, dtype):
        """(logits [n, vocab] as numpy, positions at which a router's choice rests on a gap that rounding can close [n] bool)."""
        key = (tuple(tokens), dtype)
        if key not in self._refs:
            logits, _, margins = plain.forward(self.cfg, self.W, tokens, dtype, return_layers=True)
            # A choice score is a softmax value plus a constant; rounding the router's input to bfloat16 moves it, with what earlier layers rounded, by up to
            # five thousandths (choices with such margins were seen to turn), 32-bit arithmetic by a few millionths.
            unsure = margins < (2e-2 if dtype == torch.bfloat16 else 2e-5)
            self._refs[key] = (logits.float().numpy(), unsure.numpy())
        return self._refs[key]

    def engine(self, dtype: str, **kw):
        from tileinfer_b200.engine import Engine
        args = dict(max_tokens=2048, max_seqs=6, max_context=1024)
        args.update(kw)
        return Engine.load(self.folder, dtype=dtype, **args)


def tolerance(dtype, ref: np.ndarray) -> float:
    scale = max(float(np.abs(ref).max()), 1.0)
    return 1e-4 * scale if dtype == torch.float32 else 8 * scale * 2.0 ** -8


def compare(model: Model, tokens, got: dict, dtype, what: str = "", need: float = 0.6):
    """``got``: position -> logits row. Every position whose own router choices are settled must be within the tolerance
    (a choice that rounding turns changes its own position by an expert's whole share; what later positions see of it
    through states and keys is one token's part among many, and stays within the tolerance); at least ``need`` of the
    positions (of 20 or more) must be of that kind."""
    ref, unsure = model.reference(tokens, dtype)
    tol = tolerance(dtype, ref)
    sure = [p for p in got if not unsure[p]]
    if len(got) >= 20:
        assert len(sure) >= need * len(got), f"{what}: only {len(sure)} of {len(got)} positions are free of close router calls"
    for p in sure:
        err = float(np.abs(got[p] - ref[p]).max())
        assert err <= tol, f"{what}: position {p} of {len(tokens)}: |d| = {err:.3g} > {tol:.3g}"
    return len(sure)


def prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
