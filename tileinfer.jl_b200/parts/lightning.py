"""Linear attention with a decay per head, its state carried from token to token ("lightning" attention).

Per token, from the mixer's input h:

    q = act(Wq h), k = act(Wk h)   [heads, dim]        v = act(Wv h)   [heads, value_dim]        act = SiLU
    S_t = a_head * S_(t-1) + k_t v_t^T                  a matrix [dim, value_dim] per head, 32-bit, zero at the start
    o_t = S_t^T q_t                                     no other scale
    out = Wo ( rms_norm(concat_heads o_t; w) * sigmoid(Wg h) )

The only thing a sequence keeps is S: a fixed-size state per layer (the cache's "state" kind), however long the sequence is.
The four projections read the same input and run as one product; the recurrence (``csrc/lightning.cu``) reads its rows, applies
the activation, and serves prompts and one-token steps alike. State, decay, o and the norm are 32-bit in every element type.

Record: ``num_heads``, ``head_dim`` (query/key size) and the options ``value_dim``, ``decay`` (one number per head), ``norm_eps``,
``gate`` (default True), ``activation`` ("silu" or "none").
"""
from __future__ import annotations

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Mixer, register_mixer
from .linear import Linear


@register_mixer("lightning")
class LightningAttention(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        o = spec.options
        self.heads, self.dim, self.vdim = spec.num_heads, spec.head_dim, int(o["value_dim"])
        decay = [float(a) for a in o["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"lightning: {len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.eps = float(o.get("norm_eps", 1e-6))
        self.gated = bool(o.get("gate", True))
        act = o.get("activation", "silu")
        if act not in ("silu", "none"):
            raise ValueError(f"lightning: activation {act!r} (known: silu, none)")
        self.act = act == "silu"
        n, p = spec.tensor_names, spec.prefix
        get = lambda k: rt.param(tensors[p + n[k]])
        mats = [get("q"), get("k"), get("v")] + ([get("g")] if self.gated else [])
        self.proj = Linear(torch.cat(mats, 0).contiguous(), rt, "lightning_in")
        self.norm_w = get("norm")
        self.o = Linear(get("o"), rt, "o")
        self.o.partials_name = "mixer.partials"

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        W, H, D, V = spec.hidden_size, spec.num_heads, spec.head_dim, int(o["value_dim"])
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        out = [TensorDecl(p + n["q"], (H * D, W), std(W)), TensorDecl(p + n["k"], (H * D, W), std(W)),
               TensorDecl(p + n["v"], (H * V, W), std(W)), TensorDecl(p + n["o"], (W, H * V), std(H * V)),
               TensorDecl(p + n["norm"], (H * V,), ("one_plus_normal", 0.1))]
        if o.get("gate", True):
            out.append(TensorDecl(p + n["g"], (H * V, W), std(W)))
        return out

    def cache_request(self):
        return CacheRequest("state", shape=(self.heads, self.dim, self.vdim), dtype=torch.float32)

    def forward(self, h, step, cache):
        rt = self.rt
        n = h.shape[0]
        H, D, V = self.heads, self.dim, self.vdim
        rows = rt.buffer("lightning.rows", (n, self.proj.out_features))
        self.proj.forward(h, rows)
        o = rt.buffer("lightning.o", (n, H * V), torch.float32)
        ops.lightning_scan(o, rows, 0, H * D, 2 * H * D, cache.state, self.decay, step.cu_seqlens, step.seq_slots, step.n_seqs, H, D, V,
                           act=self.act)
        y = rt.buffer("lightning.normed", (n, H * V))
        ops.lightning_out(y, o, rows[:, 2 * H * D + H * V:] if self.gated else None, self.norm_w, self.eps)
        out = rt.buffer("mixer.delta", (n, self.spec.hidden_size))
        return self.o.forward(y, out, allow_partials=True)
