"""A plain, slow implementation of the Zudepel design on the CPU, one function per mechanism.

It shares no code with the library: it reads the same config.json keys and tensor names and computes every
sequence alone, all positions at once, in 64-bit arithmetic on the stored weights (``dtype`` bfloat16 rounds the
products' inputs and outputs and the activations, and keeps what the design wants in 32-bit unrounded). Nothing is
cached: a recurrence is a loop over the positions, a convolution reads the earlier rows, attention builds all keys.

The design in this file's notation (x: the residual stream, N(y; w) = y / sqrt(mean(y^2) + eps) * w):

* x0 = E[token]; a layer: h = N(x; w1), x += mixer(h) + ff(h) (both read the same h; a layer may have no ff);
  logits = Whead N(x; w_final).
* mixer "lightning": q, k = silu(Wq h), silu(Wk h) [heads, dim], v = silu(Wv h) [heads, vdim]; per head
  S_t = a_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; out = Wo (N(concat o; w_norm) * sigmoid(Wg h)).
* mixer "attention": u = W h + b for q, k, v; a causal convolution over time on every channel,
  y_t = sum_j c[:, j] u_(t - taps + 1 + j); q and k normed over their whole rows; the first `dims` elements of every
  head rotated (element i with i + dims/2, angle p * base^(-2i/dims)); p_ij = exp(scale q_i.k_j) for j <= i, divided
  by their sum plus exp(sink_h); out = Wo (concat(sum_j p_ij v_j) * sigmoid(Wg h)). Query head a reads KV head
  a // (heads / kv_heads). With ``kv_from`` the keys and values are those of an earlier layer.
* dense ff: Wdown (gelu_tanh(Wgate h) * Wup h).
* routed ff: s = softmax(Wr h) over experts and identity experts; choice c = s + correction; experts in `count` equal
  groups of neighbours, a group's score its largest c, only the best `keep` groups stay; the `top` largest c of
  those; weights s_e / (sum of the chosen s + 1e-20); out = sum w_e expert_e(h) with expert = Wdown (silu(Wgate h) *
  Wup h) and identity experts (the last `identity` router outputs) returning h; plus sigmoid(Wsg h) * shared(h).
"""
from __future__ import annotations

import math

import torch

F32, F64 = torch.float32, torch.float64


def rnd(x, dtype):
    return x if dtype == F32 else x.to(dtype).to(F64)


def linear(x, w, dtype, bias=None):
    y = rnd(x, dtype).to(F64) @ w.to(F64).t()
    if bias is not None:
        y = y + bias.to(F64)
    return rnd(y, dtype)


def rms_norm(y, w, eps):
    y = y.to(F64)
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w.to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def lightning(h, W, p, mix, eps, dtype):
    """h [n, width] of one sequence from its first position. The recurrence is run position by position."""
    H, D, V = mix["heads"], mix["dim"], mix["vdim"]
    n = h.shape[0]
    q = rnd(silu(linear(h, W[p + "q"], dtype)), dtype).view(n, H, D)
    k = rnd(silu(linear(h, W[p + "k"], dtype)), dtype).view(n, H, D)
    v = rnd(silu(linear(h, W[p + "v"], dtype)), dtype).view(n, H, V)
    decay = torch.tensor(mix["decay"], dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(n, H, V, dtype=F64)
    for t in range(n):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms_norm(o.reshape(n, H * V), W[p + "norm"], eps)
    y = y * torch.sigmoid(linear(h, W[p + "g"], dtype))
    return linear(y, W[p + "o"], dtype)


def causal_conv(u, c):
    """u [n, channels], c [channels, taps]: y_t = sum_j c[:, j] u_(t - taps + 1 + j), zeros before the start."""
    n, taps = u.shape[0], c.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < n:
            y[shift:] += c[:, j].to(F64) * u[:n - shift]
    return y


def rotate(x, positions, dims, base):
    """x [n, heads, dim]: element i of the first `dims` is paired with i + dims / 2."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    a = positions.to(F64)[:, None] * f[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def projected(h, W, name, mix, dtype):
    """W h + b through the convolution, where the layer has one."""
    u = linear(h, W[name], dtype, W[name + ".b"])
    return rnd(causal_conv(u, W[name + ".conv"]), dtype) if mix.get("conv") else u


def rotated(x, mix):
    rot = mix.get("rot")
    return rotate(x, torch.arange(x.shape[0]), rot["dims"], rot["base"]) if rot else x


def attention_keys_values(h, W, p, mix, eps, dtype):
    """What a layer with projections of its own keeps of a sequence: keys after convolution, norm and rotation, values
    after convolution. [n, kv_heads, dim], [n, kv_heads, vdim]."""
    n = h.shape[0]
    G, D, V = mix["kv_heads"], mix["dim"], mix["vdim"]
    k = projected(h, W, p + "k", mix, dtype)
    v = projected(h, W, p + "v", mix, dtype)
    k = rms_norm(k, W[p + "k.norm"], eps).view(n, G, D)
    return rnd(rotated(k, mix), dtype), v.view(n, G, V)


def attention(h, W, p, mix, eps, dtype, keys_values):
    """keys_values: (k, v) of this layer or of the layer that ``kv_from`` names."""
    n = h.shape[0]
    H, G, D, V = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    q = rms_norm(projected(h, W, p + "q", mix, dtype), W[p + "q.norm"], eps).view(n, H, D)
    q = rnd(rotated(q, mix), dtype)
    k, v = keys_values
    rep = H // G
    k = k.repeat_interleave(rep, 1)
    v = v.repeat_interleave(rep, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * mix["scale"]
    causal = torch.arange(n)[:, None] >= torch.arange(n)[None, :]
    s = s.masked_fill(~causal, -math.inf)
    sink = W[p + "sink"].to(F64)
    m = torch.maximum(s.max(-1).values, sink[:, None])
    e = torch.exp(s - m[..., None])
    w = e / (e.sum(-1) + torch.exp(sink[:, None] - m))[..., None]
    o = torch.einsum("hij,jhv->ihv", w, v).reshape(n, H * V)
    o = rnd(o, dtype) * torch.sigmoid(linear(h, W[p + "g"], dtype))
    return linear(o, W[p + "o"], dtype)


def gated_unit(h, W, p, act, dtype):
    return linear(rnd(act(linear(h, W[p + "gate"], dtype)) * linear(h, W[p + "up"], dtype), dtype), W[p + "down"], dtype)


def dense(h, W, p, dtype):
    return gated_unit(h, W, p, gelu_tanh, dtype)


def route(h, W, p, mlp, dtype):
    """Returns (chosen [n, top] indices, weights [n, top], margin [n]): the margin is the gap between the last choice
    score taken and the best one left out (groups that lose by little count too), so that a caller can tell close
    calls from settled ones."""
    r = mlp["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = rnd(h, dtype).to(F64) @ W[p + "router"].to(F64).t()
    s = torch.softmax(z, -1)
    c = s + W[p + "correction"].to(F64)
    n, total = c.shape
    per = total // groups["count"]
    gs = c.view(n, groups["count"], per).max(-1).values
    order = gs.sort(-1, descending=True)
    kept = torch.zeros(n, groups["count"], dtype=torch.bool)
    kept.scatter_(1, order.indices[:, :groups["keep"]], True)
    margin = torch.full((n,), math.inf, dtype=F64)
    if groups["keep"] < groups["count"]:
        margin = order.values[:, groups["keep"] - 1] - order.values[:, groups["keep"]]
    allowed = kept.repeat_interleave(per, 1)
    c = c.masked_fill(~allowed, -math.inf)
    best = c.sort(-1, descending=True)
    chosen = best.indices[:, :top]
    if top < total:
        margin = torch.minimum(margin, best.values[:, top - 1] - best.values[:, top])
    w = s.gather(1, chosen)
    w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return chosen, w, margin


def routed(h, W, p, mlp, dtype):
    r = mlp["router"]
    E = r["experts"]
    chosen, w, margin = route(h, W, p, mlp, dtype)
    n = h.shape[0]
    out = torch.zeros(n, h.shape[1], dtype=F64)
    hr = rnd(h, dtype)
    for t in range(n):
        for e, we in zip(chosen[t].tolist(), w[t].tolist()):
            if e >= E:
                out[t] += we * hr[t]
            else:
                out[t] += we * gated_unit(h[t:t + 1], W, f"{p}e{e}.", silu, dtype)[0]
    if mlp.get("shared"):
        sg = torch.sigmoid(rnd(h, dtype).to(F64) @ W[p + "shared.sg"].to(F64).t())
        out = out + sg * gated_unit(h, W, p + "shared.", silu, dtype)
    return out, margin


def forward(config, W, tokens, dtype=F32, return_layers=False):
    """Logits [n, vocab] (64-bit) of one sequence; with ``return_layers`` also the stream after every layer and the
    smallest router margin seen at every position."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"][tokens].to(F64)
    kept = {}
    streams = []
    margins = torch.full((len(tokens),), math.inf, dtype=F64)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mix = layer["mixer"]
        h = rnd(rms_norm(x, W[p + "norm1"], eps), dtype)
        if layer["type"] == "lightning":
            d = lightning(h, W, p + "mix.", mix, eps, dtype)
        elif layer["type"] == "attention":
            if mix.get("kv_from") is None:
                kept[i] = attention_keys_values(h, W, p + "mix.", mix, eps, dtype)
                kv = kept[i]
            else:
                kv = kept[mix["kv_from"]]
            d = attention(h, W, p + "mix.", mix, eps, dtype, kv)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                d = d + dense(h, W, p + "mlp.", dtype)
            else:
                f, m = routed(h, W, p + "mlp.", mlp, dtype)
                d = d + f
                margins = torch.minimum(margins, m)
        x = x + d
        streams.append(x.clone())
    logits = rnd(rms_norm(x, W["final.norm"], eps), dtype) @ W["head"].to(F64).t()
    if return_layers:
        return logits, torch.stack(streams), margins
    return logits
