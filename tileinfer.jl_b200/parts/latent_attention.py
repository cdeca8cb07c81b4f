"""Attention through low-rank latents, with only the key/value latent cached.

Per token, from the mixer's input h (no positions are applied anywhere inside):

    cq = rms_w(Wdq h, w_q)          query latent   [q_rank]
    c  = rms_w(Wdkv h, w_kv)        key/value latent [kv_rank], the ONLY thing the cache keeps (one row per position)
    q_h = Wuq_h cq                  per head [dim];   k_h(j) = Wuk_h c(j) [dim];   v_h(j) = Wuv_h c(j) [value_dim]
    out = Wo concat_h( sum_j softmax_j(scale q_h . k_h(j)) v_h(j) )      over the visible j (causal, optional window)

rms_w(y, w) = y / sqrt(mean(y^2) + eps) * w in 32-bit. Keys and values are never built: since q_h . (Wuk_h c) =
(Wuk_h^T q_h) . c, the head's query is carried into the latent's space (one small matrix per head), attention runs
over the cached latents as ONE key/value head of size kv_rank shared by all query heads, with the latent as key and
as value, and the attended latent goes through Wuv_h afterwards. That is multi-query attention, so the library's
paged attention kernels (prefill, split-KV decode, plain) serve it unchanged, window included.

Sizes and constants come from the record: ``num_heads``, ``head_dim`` (query/key size), ``scale``, ``window`` and the
options ``value_dim``, ``q_rank``, ``kv_rank``, ``latent_norm_eps``.
"""
from __future__ import annotations

import dataclasses

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Mixer, register_mixer
from .linear import Linear


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        o = spec.options
        self.heads, self.dim, self.vdim = spec.num_heads, spec.head_dim, int(o["value_dim"])
        self.q_rank, self.kv_rank = int(o["q_rank"]), int(o["kv_rank"])
        self.eps = float(o.get("latent_norm_eps", 1e-6))
        if self.kv_rank > ops.MAX_HEAD_DIM:
            raise ValueError(f"latent_attention: a key/value latent of {self.kv_rank} exceeds the attention kernels' {ops.MAX_HEAD_DIM}")
        n, p = spec.tensor_names, spec.prefix
        get = lambda k: rt.param(tensors[p + n[k]])
        # The two down projections read the same input: one product, query latent first.
        self.down = Linear(torch.cat([get("dq"), get("dkv")], 0).contiguous(), rt, "latent_down")
        self.w_q_norm, self.w_kv_norm = get("dq_norm"), get("dkv_norm")
        self.uq = Linear(get("uq"), rt, "uq")
        H, D, V, R = self.heads, self.dim, self.vdim, self.kv_rank
        # Wuk_h [dim, kv_rank] is used transposed (query -> latent space); stored so, head after head.
        self.uk_t = get("uk").view(H, D, R).transpose(1, 2).contiguous()          # [H, kv_rank, dim]
        self.uv = get("uv").view(H, V, R).contiguous()                            # [H, value_dim, kv_rank]
        self.o = Linear(get("o"), rt, "o")
        # What the attention kernels see: one KV head of size kv_rank.
        self.attn_spec = dataclasses.replace(spec, num_kv_heads=1, head_dim=R)

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        W, H, D, V = spec.hidden_size, spec.num_heads, spec.head_dim, int(o["value_dim"])
        Q, R = int(o["q_rank"]), int(o["kv_rank"])
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        return [TensorDecl(p + n["dq"], (Q, W), std(W)), TensorDecl(p + n["dq_norm"], (Q,), ("one_plus_normal", 0.1)),
                TensorDecl(p + n["uq"], (H * D, Q), std(Q)), TensorDecl(p + n["dkv"], (R, W), std(W)),
                TensorDecl(p + n["dkv_norm"], (R,), ("one_plus_normal", 0.1)), TensorDecl(p + n["uk"], (H * D, R), std(R)),
                TensorDecl(p + n["uv"], (H * V, R), std(R)), TensorDecl(p + n["o"], (W, H * V), std(H * V))]

    def cache_request(self):
        return CacheRequest("paged_latent", kv_heads=1, head_dim=self.kv_rank, window=self.spec.window)

    def decode_plan(self, group):
        if not (self.rt.fast and self.rt.dtype == torch.bfloat16):
            return None
        from ..kernels import fast
        return fast.SplitKvPlan(1, group.page_size, group.num_pages * group.page_size)

    def forward(self, h, step, cache):
        rt, s = self.rt, self.spec
        n = h.shape[0]
        H, D, V, Q, R = self.heads, self.dim, self.vdim, self.q_rank, self.kv_rank
        rows = rt.buffer("latent.down", (n, Q + R))
        rows = self.down.forward(h, rows, allow_partials=n <= 256)
        cq = rt.buffer("latent.cq", (n, Q))
        meta = step.group(cache.group_index)
        ops.latent_inputs(rows, cq, cache.k, self.w_q_norm, self.w_kv_norm, self.eps, meta.slot_mapping, Q, R)
        q = rt.buffer("latent.q", (n, H, D))
        self.uq.forward(cq, q.view(n, H * D))
        fast = None
        if rt.fast:
            from ..kernels import fast
        q_lat = rt.buffer("latent.q_latent", (n, H, R))
        if not (fast is not None and fast.head_linear(q_lat, q, self.uk_t)):
            ops.head_gemm(q_lat, q, self.uk_t)
        attn = rt.buffer("latent.attended", (n, H, R))
        done = False
        if fast is not None:
            done = fast.attention(attn.view(n, H * R), q_lat, cache, meta, step, self.attn_spec)
        if not done:
            ops.attention_plain(attn.view(n, H * R), q_lat, cache.k, cache.v, meta.block_table, step.tok_slot, step.positions,
                                s.scale, H, 1, R, cache.page_size, window=s.window or 0)
        values = rt.buffer("latent.values", (n, H, V))
        if not (fast is not None and fast.head_linear(values, attn, self.uv)):
            ops.head_gemm(values, attn, self.uv)
        proj = rt.buffer("mixer.delta", (n, s.hidden_size))
        return self.o.forward(values.view(n, H * V), proj, allow_partials=True)
