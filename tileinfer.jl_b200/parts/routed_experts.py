"""A routed feed-forward: a router picks ``top`` of ``experts`` small gated units per token; a shared unit may run for
every token and is added.

    z = Wr h (32-bit), score = sigmoid(z); the `top` largest scores choose the experts (ties to the smaller index)
    unit(u; limit) = Wdown( a * sigmoid(slope * a) * (b + shift) ),  a = min(Wgate u, limit),  b = clamp(Wup u, -limit, limit)
    out = sum_chosen unit_e(score_e * h)  [+ unit_shared(h)]         with ``scale_input`` (the score scales the INPUT)
    out = sum_chosen score_e * unit_e(h)  [+ unit_shared(h)]         without it

Options of the record: ``experts``, ``top``, ``limit``, ``sigmoid_slope``, ``up_shift``, ``scale_input``, ``renormalize``
(divide the chosen scores by their sum), ``shared_size`` / ``shared_limit`` (0: no shared unit). ``intermediate_size`` is
an expert's size. Tensor names: ``router``, ``expert`` (a prefix pattern with ``{}`` for the expert's number), ``shared``
(a prefix), and inside a unit ``gate``, ``up``, ``down``.

On the device the (token, choice) pairs are grouped by expert and every expert's rows go through its matrices in
tiles (``csrc/routed_experts.cu``, on the tensor cores ``csrc/gemm_tcgen05.cu``); no count is read on the host, so a
one-token step stays capturable. The shared unit rides along as units of an expert's size that every token takes.
"""
from __future__ import annotations

import torch

from ..config.spec import FeedForwardSpec, TensorDecl
from ..kernels import ops
from .base import FeedForward, register_feed_forward
from .linear import Linear
from .norm import GatheredRows


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec: FeedForwardSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        o, n, p = spec.options, spec.tensor_names, spec.prefix
        self.experts, self.top = int(o["experts"]), int(o["top"])
        self.limit = float(o["limit"])
        self.slope, self.shift = float(o.get("sigmoid_slope", 1.0)), float(o.get("up_shift", 0.0))
        self.scale_input = bool(o.get("scale_input", False))
        if o.get("renormalize", False) or o.get("score", "sigmoid") != "sigmoid":
            raise ValueError("routed_experts: only unnormalised sigmoid scores are built")
        get = lambda name: rt.param(tensors[p + name])
        self.router = get(n["router"])
        self.router_linear = Linear(self.router, rt, "router")
        units = [p + n["expert"].format(e) for e in range(self.experts)]
        unit = lambda u, k: rt.param(tensors[u + n[k]])
        F, W = spec.intermediate_size, spec.hidden_size
        gate_up = [torch.cat([unit(u, "gate"), unit(u, "up")], 0) for u in units]
        down = [unit(u, "down") for u in units]
        limits = [self.limit] * self.experts
        # The shared unit runs as further units of an expert's size that every token takes with score one: a gated unit is
        # a sum over its inner rows, so slices of F of them (the last one filled up with zero rows, which add nothing)
        # are units of their own, and the grouped products carry them along with the routed experts.
        self.shared_size = int(o.get("shared_size", 0))
        self.always = -(-self.shared_size // F) if self.shared_size else 0
        if self.shared_size:
            u = p + n["shared"]
            g, up, d = unit(u, "gate"), unit(u, "up"), unit(u, "down")
            pad = self.always * F - self.shared_size
            if pad:
                zeros = torch.zeros(pad, W, dtype=g.dtype, device=g.device)
                g, up = torch.cat([g, zeros], 0), torch.cat([up, zeros], 0)
                d = torch.cat([d, torch.zeros(W, pad, dtype=d.dtype, device=d.device)], 1)
            for c in range(self.always):
                gate_up.append(torch.cat([g[c * F:(c + 1) * F], up[c * F:(c + 1) * F]], 0))
                down.append(d[:, c * F:(c + 1) * F])
                limits.append(float(o["shared_limit"]))
        # Every unit's gate rows then its up rows, unit after unit; the down matrices likewise.
        self.gate_up = torch.stack(gate_up).contiguous()
        self.down = torch.stack(down).contiguous()
        self.limits = torch.tensor(limits, dtype=torch.float32, device=rt.device)
        self.units = self.experts + self.always

    @classmethod
    def tensors(cls, spec: FeedForwardSpec):
        o, n, p = spec.options, spec.tensor_names, spec.prefix
        W, F = spec.hidden_size, spec.intermediate_size
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        out = [TensorDecl(p + n["router"], (int(o["experts"]), W), std(W))]

        def unit(u, size):
            return [TensorDecl(u + n["gate"], (size, W), std(W)), TensorDecl(u + n["up"], (size, W), std(W)),
                    TensorDecl(u + n["down"], (W, size), std(size))]
        for e in range(int(o["experts"])):
            out += unit(p + n["expert"].format(e), F)
        if int(o.get("shared_size", 0)):
            out += unit(p + n["shared"], int(o["shared_size"]))
        return out

    def forward(self, h, step):
        rt, spec = self.rt, self.spec
        n, W = h.shape
        F, top, E, per_token = spec.intermediate_size, self.top, self.experts, self.top + self.always
        pairs = n * per_token
        fast = None
        if rt.fast:
            from ..kernels import fast
        ids = rt.buffer("experts.ids", (n, per_token), torch.int32)
        scores = rt.buffer("experts.scores", (n, per_token), torch.float32)
        tile = fast.grouped_tile(pairs, self.units) if fast is not None else ops.EXPERT_TILE_ROWS
        max_tiles, rows = ops.expert_plan_sizes(pairs, self.units, tile)
        pair_row = rt.buffer("experts.pair_row", (n, per_token), torch.int32)
        row_pair = rt.buffer("experts.row_pair", (rows,), torch.int32)
        plan = rt.buffer("experts.plan", (1 + max_tiles,), torch.int32)
        xs = rt.buffer("experts.rows", (rows, W))
        logits = None
        if fast is not None:                     # the router's 32-bit sums from a product kernel, where one takes the sizes
            logits = fast.linear_f32(self.router_linear, h, rt.buffer("experts.logits", (n, E), torch.float32))
        ops.router_topk(h, self.router, top, ids, scores, logits, always=self.always)
        ops.expert_plan(ids, self.units, tile, pair_row, row_pair, plan)
        ops.expert_gather(xs, h, pair_row, scores, per_token, self.scale_input)
        act = rt.buffer("experts.act", (rows, F))
        gu = rt.buffer("experts.gate_up", (rows, 2 * F))
        if fast is not None and fast.grouped_linear(gu, xs, self.gate_up, plan, tile):
            ops.gated_unit_limit(act, gu, 0.0, self.slope, self.shift, plan=plan, tile=tile, limits=self.limits)
        else:
            ops.grouped_gemm(act, xs, self.gate_up, plan, tile, gated=True, limits=self.limits, slope=self.slope, shift=self.shift)
        ys = rt.buffer("experts.out_rows", (rows, W))
        if not (fast is not None and fast.grouped_linear(ys, act, self.down, plan, tile)):
            ops.grouped_gemm(ys, act, self.down, plan, tile)
        if self.scale_input:
            return GatheredRows(ys, pair_row)    # the norm that reads the output adds a token's rows up itself
        out = rt.buffer("feed_forward.delta", (n, W))
        ops.expert_combine(out, ys, pair_row, scores, None, per_token, scale_output=True)
        return out
