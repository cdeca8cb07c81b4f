"""A plain, slow implementation of the Vogilix design on the CPU, one function per mechanism.

It shares no code with the library: it reads the same config.json keys and tensor names, and computes
every sequence alone, all positions at once, from full keys and values (nothing is cached, nothing is
absorbed into the queries). ``dtype`` bfloat16 rounds the matrix products' inputs and outputs and the
activations to bfloat16 and keeps what the design wants in 32-bit there: the residual stream, every
norm, the router, attention scores and weights.

The design, in this file's notation (x: residual stream in 32-bit, m: the residual multiplier):

* x0 = E[token] + P[position].
* a layer: x += m * N1(mixer(x)); x += m * N2(ff(x)); x += m * side(x, token). N(y) = y / rms(y) * (1 + w),
  rms(y) = sqrt(mean(y^2) + eps). The sublayers read x itself; a layer may have no feed-forward.
* mixer "latent_attention": cq = rmsw(Wdq x, w_q), q = Wuq cq; c = rmsw(Wdkv x, w_kv); per head k = Wuk c,
  v = Wuv c; position i sees j with 0 <= i - j < window; softmax(scale * q.k); out = Wo [heads' outputs].
  rmsw(y, w) = y / rms(y) * w.
* dense feed-forward: Wdown gelu_erf(Wup x).
* expert(h; limit) = Wdown (g * sigmoid(1.702 g) * (u + 1)), g = min(Wgate h, limit), u = clamp(Wup h, +-limit).
  routed: s = sigmoid(Wrouter x); the `top` largest s; sum over them of expert_e(s_e * x); plus shared(x).
* side(x, token) = y / rms(y) * w_side, y = Wproj (gelu_tanh(Wgate x) * S[token, layer's slice]).
* logits = Whead N_final(x).
"""
from __future__ import annotations

import json
import math
import os

import torch

F32 = torch.float32


def rnd(x: torch.Tensor, dtype) -> torch.Tensor:
    return x if dtype == F32 else x.to(dtype).to(F32)


def linear(x, w, dtype):
    """y = W x with 32-bit accumulation, inputs and output in ``dtype``."""
    return rnd(rnd(x, dtype).double() @ w.double().t(), dtype).to(F32) if dtype != F32 else (x.double() @ w.double().t()).to(F32)


def rms(y, eps):
    return torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + eps)


def norm_offset(y, w, eps):
    """y / rms(y) * (1 + w), in 32-bit."""
    return (y.double() / rms(y, eps) * (1.0 + w.double())).to(F32)


def norm_plain(y, w, eps):
    """y / rms(y) * w, in 32-bit."""
    return (y.double() / rms(y, eps) * w.double()).to(F32)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embed(W, tokens, positions):
    return W["embed"][tokens].to(F32) + W["pos"][positions].to(F32)


def window_mask(n, window):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    d = i - j
    ok = d >= 0
    if window:
        ok &= d < window
    return ok


def latent_attention(x, W, p, mix, eps, dtype):
    """x: [n, width] of one sequence from its first position on. Returns the mixer's output [n, width]."""
    n = x.shape[0]
    H, D, V = mix["heads"], mix["dim"], mix["vdim"]
    h = rnd(x, dtype)
    cq = rnd(norm_plain(linear(h, W[p + "dq"], dtype), W[p + "dq.norm"], eps), dtype)
    q = linear(cq, W[p + "uq"], dtype).view(n, H, D)
    c = rnd(norm_plain(linear(h, W[p + "dkv"], dtype), W[p + "dkv.norm"], eps), dtype)
    k = linear(c, W[p + "uk"], dtype).view(n, H, D)
    v = linear(c, W[p + "uv"], dtype).view(n, H, V)
    window = (mix.get("mask") or {}).get("size")
    ok = window_mask(n, window)
    s = torch.einsum("ihd,jhd->hij", q.double(), k.double()) * mix["scale"]
    s = s.masked_fill(~ok[None], float("-inf"))
    w = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhv->ihv", w, v.double()).to(F32).reshape(n, H * V)
    return linear(o, W[p + "o"], dtype)


def dense_ff(x, W, p, dtype):
    h = rnd(x, dtype)
    a = rnd(gelu_erf(linear(h, W[p + "up"], dtype).double()).to(F32), dtype)
    return linear(a, W[p + "down"], dtype)


def expert(h, W, p, limit, dtype):
    g = linear(h, W[p + "gate"], dtype).clamp(max=limit)
    u = linear(h, W[p + "up"], dtype).clamp(-limit, limit)
    y = rnd((g.double() * torch.sigmoid(1.702 * g.double()) * (u.double() + 1.0)).to(F32), dtype)
    return linear(y, W[p + "down"], dtype)


def router(x, W, p, top, dtype, margins=None):
    """(expert ids [n, top], their scores [n, top]); logits in 32-bit from the rounded input. ``margins``: a list
    that receives, per row, how far the last chosen logit is above the first one left out, relative to the row's
    root mean square (a small value marks a choice that rounding could turn)."""
    z = (rnd(x, dtype).double() @ W[p + "router"].double().t()).to(F32)
    val, idx = torch.topk(z, top, dim=-1)
    if margins is not None:
        if top < z.shape[1]:
            srt = torch.sort(z, dim=-1, descending=True).values
            margins.append((srt[:, top - 1] - srt[:, top]) / z.pow(2).mean(-1).sqrt().clamp_min(1e-30))
        else:
            margins.append(torch.full((z.shape[0],), float("inf")))
    return idx, torch.sigmoid(val)


def moe_ff(x, W, p, mlp, dtype, margins=None):
    n = x.shape[0]
    r = mlp["router"]
    idx, val = router(x, W, p, r["top"], dtype, margins)
    h = rnd(x, dtype)
    out = torch.zeros(n, x.shape[1], dtype=torch.float64)
    for t in range(n):
        for j in range(r["top"]):
            e = int(idx[t, j])
            scaled = rnd(val[t, j] * h[t:t + 1], dtype)
            out[t] += expert(scaled, W, f"{p}e{e}.", mlp["expert"]["limit"], dtype)[0].double()
    if mlp.get("shared"):
        out += expert(h, W, p + "shared.", mlp["shared"]["limit"], dtype).double()
    return rnd(out.to(F32), dtype)


def side_input(x, tokens, W, layer, i, dim, eps, dtype):
    """y / rms(y) * w for layer i's slice of the per-token table."""
    e = W["side.embed"][tokens, i * dim:(i + 1) * dim].to(F32)
    g = rnd(gelu_tanh(linear(rnd(x, dtype), W[layer + "side.gate"], dtype).double()).to(F32) * e, dtype)
    y = linear(g, W[layer + "side.proj"], dtype)
    return norm_plain(y, W[layer + "side.norm"], eps)


def forward(cfg, W, tokens, dtype=F32, layers_out=None, margins=None):
    """Logits [n, vocab] of one sequence from position 0; ``layers_out``: a list that receives the residual
    stream after every layer; ``margins``: a list that receives (layer, router margins [n]) of every routed layer."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    n = tokens.shape[0]
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    W = {k: v.to(F32) for k, v in W.items()}
    x = embed(W, tokens, torch.arange(n))
    side = cfg.get("token_side")
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        y = latent_attention(x, W, L + "mix.", layer["mixer"], eps, dtype)
        x = x + m * norm_offset(y, W[L + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] == "dense":
                y = dense_ff(x, W, L + "mlp.", dtype)
            else:
                got = [] if margins is not None else None
                y = moe_ff(x, W, L + "mlp.", mlp, dtype, got)
                if got:
                    margins.append((i, got[0]))
            x = x + m * norm_offset(y, W[L + "norm2"], eps)
        if side:
            x = x + m * side_input(x, tokens, W, L, i, side["dim"], eps, dtype)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = rnd(norm_offset(x, W["final.norm"], eps), dtype)
    return (h.double() @ W["head"].double().t()).to(F32)


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


def unsure_positions(cfg, margins, n, threshold):
    """Positions of a sequence of ``n`` tokens whose result a turned router choice could have changed: the positions
    whose margin in some routed layer is below ``threshold``, and the later positions that can see them through the
    attention of the layers after it (each such layer carries a change forward by its window, less one)."""
    bad = torch.zeros(n, dtype=torch.bool)
    by_layer = dict(margins)
    for i, layer in enumerate(cfg["layers"]):
        if bad.any():                                   # this layer's attention spreads what earlier layers changed
            window = (layer["mixer"].get("mask") or {}).get("size") or n
            idx = torch.nonzero(bad).flatten()
            for p in idx.tolist():
                bad[p:min(n, p + window)] = True
        if i in by_layer:
            bad |= by_layer[i] < threshold
    return bad
