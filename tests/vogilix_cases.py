"""Small Vogilix configurations for the tests, their random model folders and the comparison against the plain
implementation (``plain_vogilix``).

The configurations differ from one another in every size and constant, and none keeps two sizes equal that a
kernel could mix up (query/key size and value size, the two latent ranks, heads and experts).
"""
from __future__ import annotations

import os

import numpy as np
import torch

import plain_vogilix as plain


def mixer(heads, dim, vdim, q_rank, kv_rank, scale, window):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "vdim": vdim}
    if window:
        m["mask"] = {"size": window}
    return m


def moe(experts, top, ff, limit, shared=None):
    m = {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mix, mlp):
    return {"mixer": mix, "mlp": mlp, "type": "latent_attention"}


# Odd sizes, two attention groups with different windows and latents, a layer without feed-forward, the routed layer
# last (a turned router choice then changes one position only), a sharp softmax (scale well above 1 / sqrt(dim)).
CASE_A = {
    "architecture": "Vogilix", "vocab": 151, "width": 72, "max_positions": 512, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
    "token_side": {"dim": 8},
    "layers": [layer(mixer(3, 16, 24, 40, 48, 0.7, 37), {"ff": 136, "kind": "dense"}),
               layer(mixer(3, 16, 24, 40, 48, 0.7, 37), None),
               layer(mixer(2, 32, 16, 24, 32, 0.5, 70), moe(6, 2, 40, 1.5, (56, 2.5)))],
}
# Sizes that the tensor-core kernels take (widths in steps of 8, a latent of 64), a layer that sees every earlier
# position, no token input, no shared expert, no residual multiplier in the file (1), one expert per token.
CASE_B = {
    "architecture": "Vogilix", "vocab": 320, "width": 128, "max_positions": 1024, "norm": {"eps": 1e-6},
    "layers": [layer(mixer(4, 32, 48, 80, 64, 0.6, 100), {"ff": 264, "kind": "dense"}),
               layer(mixer(4, 32, 48, 80, 64, 0.6, None), moe(4, 1, 72, 0.75))],
}
# Sizes no fast kernel takes (a width that is no multiple of 8, a latent that is no multiple of 16), a routed layer
# first, three experts per token, a window shorter than a page.
CASE_C = {
    "architecture": "Vogilix", "vocab": 97, "width": 60, "max_positions": 300, "norm": {"eps": 3e-6}, "residual_mult": 1.25,
    "token_side": {"dim": 5},
    "layers": [layer(mixer(5, 10, 6, 18, 40, 0.9, 23), moe(5, 3, 22, 3.0, (30, 1.0))),
               layer(mixer(2, 14, 26, 50, 20, 0.4, 129), {"ff": 90, "kind": "dense"})],
}
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}


def write_folder(case: dict, seed: int, out_dir: str) -> str:
    """A model folder with random weights for ``case``, made without a device."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.weights import write_model_folder
    return write_model_folder(config_from_dict(case), seed, out_dir, device="cpu")


class Model:
    """A case's folder, the plain implementation's view of it and cached reference logits."""

    def __init__(self, name: str, seed: int, tmp: str, bf16_margin: float = 0.1):
        self.name, self.bf16_margin = name, bf16_margin
        self.folder = write_folder(CASES[name], seed, os.path.join(tmp, f"vogilix_{name}_{seed}"))
        self.cfg, self.W = plain.load_folder(self.folder)
        self.vocab = self.cfg["vocab"]
        self._refs = {}

    def reference(self, tokens, dtype):
        """(logits [n, vocab] as numpy, positions that a turned router choice could have changed [n] bool)."""
        key = (tuple(tokens), dtype)
        if key not in self._refs:
            margins = []
            logits = plain.forward(self.cfg, self.W, tokens, dtype, margins=margins)
            # How far rounding can move a router logit relative to the row's size. In bfloat16 the cases' sharp softmax
            # turns the rounding of queries and keys into a stream error of about a hundredth of its size, and
            # choices with margins up to 0.05 were seen to turn; in 32-bit the error is a few millionths.
            unsure = plain.unsure_positions(self.cfg, margins, len(tokens), self.bf16_margin if dtype == torch.bfloat16 else 1e-4)
            self._refs[key] = (logits.numpy(), unsure.numpy())
        return self._refs[key]

    def engine(self, dtype: str, **kw):
        from tileinfer_b200.engine import Engine
        args = dict(max_tokens=2048, max_seqs=6, max_context=self.cfg["max_positions"])
        args.update(kw)
        return Engine.load(self.folder, dtype=dtype, **args)


def tolerance(dtype, ref: np.ndarray) -> float:
    scale = max(float(np.abs(ref).max()), 1.0)
    return 1e-4 * scale if dtype == torch.float32 else 8 * scale * 2.0 ** -8


def compare(model: Model, tokens, got: dict, dtype, what: str = "", need: float = 0.5):
    """``got``: position -> logits row. Every position that no close router call could have changed must be within
    the tolerance; at least ``need`` of the positions (of 20 or more) must be of that kind."""
    ref, unsure = model.reference(tokens, dtype)
    tol = tolerance(dtype, ref)
    sure = [p for p in got if not unsure[p]]
    if len(got) >= 20:                                  # a handful of positions may all be close calls
        assert len(sure) >= need * len(got), f"{what}: only {len(sure)} of {len(got)} positions are free of close router calls"
    for p in sure:
        err = float(np.abs(got[p] - ref[p]).max())
        assert err <= tol, f"{what}: position {p} of {len(tokens)}: |d| = {err:.3g} > {tol:.3g}"
    return len(sure)


def prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
