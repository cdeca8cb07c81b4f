"""The Vogilix design through the engine against the plain implementation (``plain_vogilix``): whole prompts, prompts
in portions down to two tokens, token-by-token decoding across page and window borders, batches of unequal requests
against each alone, slots and pages that are used again, long decoding, greedy generation through the public entry
point, and trace replay through ``bin/trace_run``; in 32-bit and in bfloat16, at three sets of sizes."""
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_vogilix as plain
import vogilix_cases as vc
from replay_util import Trace, run_trace

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Case C's routed layer comes first and its second layer sees 129 positions back: in bfloat16 a close router call
# anywhere leaves most of a sequence uncertain, so there only what is certain is compared, however little.
NEED = {("C", "bfloat16"): 0.0}


@pytest.fixture(scope="module")
def models():
    with tempfile.TemporaryDirectory() as tmp:
        # Case C routes in its first layer, whose output a second layer with a multiplier above one carries on: there
        # wider margins count as close calls in bfloat16.
        yield {name: vc.Model(name, seed, tmp, margin) for name, seed, margin in (("A", 11, 0.1), ("B", 12, 0.1), ("C", 13, 0.3))}


def rows(logits, positions):
    a = logits.detach().float().cpu().numpy()
    return {p: a[i].copy() for i, p in enumerate(positions)}


def run_cut(engine, tokens, cuts):
    """One sequence fed in portions of the given sizes (the rest one token at a time); logits at every position."""
    slot = engine.new_sequence()
    got, at = {}, 0
    sizes = list(cuts)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        got.update(rows(engine.step([(slot, tokens[at:at + n])], [list(range(n))]), range(at, at + n)))
        at += n
    engine.free_sequence(slot)
    engine.check_health()
    return got


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_prompts_in_portions(models, name, dtype):
    m = models[name]
    engine = m.engine(dtype)
    need = NEED.get((name, dtype), 0.5)
    longest = min(m.cfg["max_positions"], 600)
    for tokens in vc.prompts(m.vocab, [1, 2, 7, 64, 65, 150, longest], 21):
        got = run_cut(engine, tokens, [len(tokens)])
        vc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} whole {len(tokens)}", need)
    tokens = vc.prompts(m.vocab, [230], 22)[0]
    for cuts in ([2, 2, 3, 57, 1, 64, 2, 90], [63, 2, 64, 1, 1, 2, 97], [128, 2, 100], [1, 1, 1, 200, 2, 2]):
        got = run_cut(engine, tokens, cuts)                # whatever is left after the portions goes one token at a time
        assert sorted(got) == list(range(len(tokens)))
        vc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} portions {cuts}", need)


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_past_windows_and_pages(models, name, dtype):
    """A short prompt, then more than 200 single tokens: every window of the case passes over decoded tokens only, and
    pages fill up and (behind a window) are given back while decoding."""
    m = models[name]
    engine = m.engine(dtype, max_tokens=512, max_seqs=2)
    tokens = vc.prompts(m.vocab, [300], 23)[0]
    got = run_cut(engine, tokens, [5])
    vc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_batches_of_unequal_requests_and_reuse_of_slots_and_pages(models, name, dtype):
    """Requests of unequal lengths prefilled in one step and decoded together, the shorter ones leaving first; then a
    second batch in the slots and pages that the first gave back. Every request is compared with the plain
    implementation of that request alone."""
    m = models[name]
    need = NEED.get((name, dtype), 0.5)
    engine = m.engine(dtype, max_tokens=1024, max_seqs=4)
    cap = m.cfg["max_positions"]
    for seed, lengths, tails in ((31, [1, 40, 129, min(cap, 330)], [0, 12, 40, 3]), (32, [70, 3, min(cap, 260), 64], [6, 2, 65, 33])):
        reqs = vc.prompts(m.vocab, lengths, seed)
        slots = [engine.new_sequence() for _ in reqs]
        got = [dict() for _ in reqs]
        heads = [len(t) - d for t, d in zip(reqs, tails)]
        out = engine.step([(s, t[:h]) for s, t, h in zip(slots, reqs, heads)], [list(range(h)) for h in heads])
        a = out.detach().float().cpu().numpy()
        at = 0
        for i, h in enumerate(heads):
            got[i].update({p: a[at + p].copy() for p in range(h)})
            at += h
        fed = list(heads)
        live = [i for i in range(len(reqs)) if fed[i] < len(reqs[i])]
        for i in range(len(reqs)):
            if i not in live:
                engine.free_sequence(slots[i])
        while live:
            out = engine.step([(slots[i], [reqs[i][fed[i]]]) for i in live]).detach().float().cpu().numpy()
            for r, i in enumerate(live):
                got[i][fed[i]] = out[r].copy()
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(reqs[i])]:
                engine.free_sequence(slots[i])
            live = [i for i in live if fed[i] < len(reqs[i])]
        engine.check_health()
        for i, t in enumerate(reqs):
            assert sorted(got[i]) == list(range(len(t)))
            vc.compare(m, t, got[i], DTYPES[dtype], f"{name} {dtype} batch seed {seed} request {i}", need)
    assert engine.cache.slots.held == 0


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_a_single_key_just_inside_and_just_outside_the_window(dtype):
    """One layer, one head, weights made by hand so that a score stands out: the key/value latent of a marked token
    points along one axis, every query looks along that axis, and the value carried back is the marker. A query sees
    the marked token while it is among the last `window` positions and not one step longer; with the marker far
    away, at a page border, at the first position, in a prompt and while decoding."""
    from tileinfer_b200.config import MixerSpec
    from tileinfer_b200.parts import Runtime, lookup
    from test_parts_gpu import OneStep
    T = DTYPES[dtype]
    W, R, Q, D, V, window = 16, 16, 16, 16, 16, 70
    names = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
    spec = MixerSpec("latent_attention", "m.", W, 1, 1, D, scale=8.0, window=window, tensor_names=names,
                     options={"value_dim": V, "q_rank": Q, "kv_rank": R, "latent_norm_eps": 1e-6})
    eye = torch.eye(16)
    # Hidden vectors: a marked token is e0 + small e2, an ordinary one is e1. The latents are the hidden vector,
    # normalised. Queries: every token asks along e0 (uq sends both e0 and e1 to e0). Values: the latent itself.
    uq = torch.zeros(D, Q); uq[0, 0] = uq[0, 1] = 1.0
    tensors = {"m.dq": eye.clone(), "m.dq.norm": torch.ones(Q), "m.uq": uq, "m.dkv": eye.clone(), "m.dkv.norm": torch.ones(R),
               "m.uk": eye.clone(), "m.uv": eye.clone(), "m.o": eye.clone()}
    rt = Runtime(T)
    mixer = lookup("mixer", "latent_attention")(spec, {k: v.to(T) for k, v in tensors.items()}, rt, None)
    marked = torch.zeros(W); marked[0] = 1.0; marked[2] = 0.25
    plain_tok = torch.zeros(W); plain_tok[1] = 1.0
    for mark_at, prompt_len, total in ((0, 1, 150), (63, 64, 200), (64, 140, 220), (5, 80, 90), (128, 129, 260)):
        h = plain_tok.repeat(total, 1)
        h[mark_at] = marked
        env = OneStep(mixer, T, max_tokens=512, max_seqs=2)
        slot = env.cache.alloc_slot()
        out = [env.run(mixer, [(slot, h[:prompt_len].to(T))], W)]
        out += [env.run(mixer, [(slot, h[t:t + 1].to(T))], W) for t in range(prompt_len, total)]
        out = torch.cat(out)
        # Element 2 of the output is the marker's share of the attention: close to its 0.25 / |marked| * sqrt(16)
        # while the marked token is visible (its score exceeds the others' by 8 * 15), exactly zero afterwards.
        seen = out[:, 2] > 0.5
        expect = torch.tensor([mark_at <= t < mark_at + window for t in range(total)])
        assert torch.equal(seen, expect), f"marker at {mark_at}: visible at {torch.nonzero(seen).flatten().tolist()[:3]}..{int(seen.sum())} positions"
        assert float(out[~expect][:, 2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_mixer_alone_in_steps_of_every_kind(models, dtype):
    """The latent-attention mixer alone on random inputs (sizes of case A's last layer): two sequences, whole, in
    portions, token by token, the order of the entries swapped between steps, against the plain mixer."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.parts import Runtime, lookup
    from test_parts_gpu import OneStep
    T = DTYPES[dtype]
    m = models["A"]
    spec = config_from_dict(m.cfg).model_spec().layers[2].mixer
    rt = Runtime(T)
    mixer = lookup("mixer", "latent_attention")(spec, {k: v.to(T) for k, v in m.W.items()}, rt, None)
    torch.manual_seed(3)
    hs = [plain.rnd(torch.randn(n, spec.hidden_size), T) for n in (190, 75)]
    refs = [plain.latent_attention(h, {k: v.float() for k, v in m.W.items()}, "l2.mix.", m.cfg["layers"][2]["mixer"], m.cfg["norm"]["eps"], T)
            for h in hs]
    env = OneStep(mixer, T)
    a, b = env.cache.alloc_slot(), env.cache.alloc_slot()
    got = {a: [], b: []}
    cut = lambda i, lo, hi: hs[i][lo:hi].to(T)
    plan = [[(a, 0, 0, 100), (b, 1, 0, 2)], [(b, 1, 2, 40), (a, 0, 100, 101)], [(a, 0, 101, 103), (b, 1, 40, 41)]]
    plan += [[(a, 0, t, t + 1)] + ([(b, 1, t - 62, t - 61)] if t - 62 < 75 else []) for t in range(103, 190)]
    for entries in plan:
        out = env.run(mixer, [(s, cut(i, lo, hi)) for s, i, lo, hi in entries], spec.hidden_size)
        at = 0
        for s, i, lo, hi in entries:
            got[s].append(out[at:at + hi - lo])
            at += hi - lo
    for s, ref in ((a, refs[0]), (b, refs[1])):
        g = torch.cat(got[s])
        assert g.shape == ref.shape
        tol = (2e-5 if T == torch.float32 else 6 * 2.0 ** -8) * float(ref.abs().max())
        assert float((g - ref).abs().max()) <= tol


def test_greedy_generation_through_the_public_entry_point(models):
    """``generate`` (batches, scheduler, sampler, decode loop) on several prompts at once, in 32-bit: every generated
    token is the plain implementation's most likely next token for the same prefix."""
    import tileinfer_b200 as ti
    m = models["A"]
    engine = ti.load_model(m.folder, dtype="float32", max_context=256, max_seqs=3)
    reqs = vc.prompts(m.vocab, [3, 41, 90, 17], 41)
    outs = ti.generate(engine, reqs, max_new_tokens=40, stop_ids=[])
    assert [len(o) for o in outs] == [40] * 4
    for p, o in zip(reqs, outs):
        ref = plain.forward(m.cfg, m.W, p + o, torch.float32).numpy()
        for k, tok in enumerate(o):
            row = ref[len(p) + k - 1]
            assert row[tok] >= row.max() - 1e-4, f"token {k}: generated {tok}, plain argmax {int(row.argmax())}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_trace_replay(models, dtype):
    """The same requests through ``bin/trace_run``: whole, with the tail one by one, and in two batches one after the
    other (the second in the first one's slots and pages)."""
    m = models["B"]
    reqs = {f"r{i}": t for i, t in enumerate(vc.prompts(m.vocab, [1, 9, 70, 130, 200], 51))}
    t = Trace()
    t.whole(reqs)
    t.tail_one_by_one(reqs, tail=20)
    names = list(reqs)
    t.batch({r: reqs[r] for r in names[:3]}, {r: min(len(reqs[r]) - 1, 4 + 3 * i) for i, r in enumerate(names[:3])}, tag="x")
    t.batch({r: reqs[r] for r in names[2:]}, {r: min(len(reqs[r]) - 1, 30) for r in names[2:]}, tag="y")
    with tempfile.TemporaryDirectory() as out:
        got = run_trace(m.folder, dtype, t, out, sum(-(-len(x) // 64) * 64 for x in reqs.values()), m.vocab)
    by_request = {}
    for (rid, pos), row in got.items():
        by_request.setdefault(rid, {})[pos] = row
    assert len(by_request) == 5 + 5 + 3 + 3
    for rid, g in by_request.items():
        vc.compare(m, reqs[rid[1:]], g, DTYPES[dtype], f"replay {dtype} {rid}")


def test_bfloat16_steps_take_the_tensor_core_kernels(models):
    """Case B's sizes are ones the fast kernels take: a prompt and a decode step in bfloat16 go through the grouped and the
    per-head tensor-core products and the paged attention kernels, not through their plain stand-ins."""
    from tileinfer_b200.kernels import library
    m = models["B"]
    engine = m.engine("bfloat16", graphs=False)
    slot = engine.new_sequence()
    library.call_counts.clear()
    engine.step([(slot, vc.prompts(m.vocab, [450], 61)[0])])
    engine.step([(slot, [5])])
    engine.free_sequence(slot)
    engine.check_health()
    used = library.call_counts
    assert used.get("ti_gemm_tcgen05_grouped", 0) == 4 and used.get("ti_gemm_tcgen05_heads", 0) == 8
    assert used.get("ti_attention_prefill_tc", 0) == 2 and used.get("ti_attention_decode_shared", 0) == 2
    assert "ti_grouped_gemm" not in used and "ti_head_gemm" not in used and "ti_attention_plain" not in used


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_mechanisms_alone(dtype):
    """The kernels of the design one at a time against the plain implementation's functions, at sizes of their own:
    the 32-bit stream's update, the norms, the latents, a product per head, the activations, the router, the routed
    units with and without a shared one."""
    from tileinfer_b200.kernels import ops
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(7)
    R = lambda *shape, s=1.0: plain.rnd(torch.randn(*shape, generator=g) * s, T)
    dev = lambda t: t.to(T).cuda() if t.is_floating_point() else t.cuda()
    close = lambda got, ref, what: _close(got, ref, T, what)
    n, size = 9, 88
    # x += m * d / rms(d) * (1 + w); h = x / rms(x) * w2, or h = x
    x, d, w, w2 = torch.randn(n, size, generator=g), R(n, size, s=3.0), R(size, s=0.2), R(size) + 1
    for parts in (None, 3):
        for out_norm in (None, (dev(w2), 2e-5, False)):
            xs, h = x.clone().cuda(), torch.empty(n, size, dtype=T, device="cuda")
            delta = dev(d) if parts is None else torch.stack([d.float() * f for f in (0.5, 0.25, 0.25)]).cuda()
            ops.branch_norm_add32(xs, delta, dev(w), 1e-5, 0.7, True, h, out_norm)
            ref = x + 0.7 * plain.norm_offset(d, w, 1e-5)
            assert xs.dtype == torch.float32 and float((xs.cpu() - ref).abs().max()) < 1e-5
            close(h, ref if out_norm is None else plain.norm_plain(ref, w2, 2e-5), "stream update")
    # rows gathered and added up by the update itself
    rows, index = R(20, size), torch.randint(0, 20, (n, 3), generator=g, dtype=torch.int32)
    xs = x.clone().cuda()
    ops.branch_norm_add32(xs, dev(rows), dev(w), 1e-5, 1.0, False, None, None, gather=index.cuda())
    ref = x + plain.norm_plain(rows[index.long()].sum(1), w, 1e-5)
    assert float((xs.cpu() - ref).abs().max()) < 1e-5
    # norms of a 32-bit or a rounded input
    y = torch.empty(n, size, dtype=T, device="cuda")
    ops.norm32(y, x.cuda(), dev(w), 1e-6, True)
    close(y, plain.norm_offset(x, w, 1e-6), "norm of the stream")
    ops.norm32(y, dev(d), dev(w2), 1e-6, False)
    close(y, plain.norm_plain(d, w2, 1e-6), "norm of a rounded input")
    # embedding + learned positions
    E, P = R(30, size), R(40, size)
    ids, pos = torch.tensor([3, 29, 0, 7], dtype=torch.int32), torch.tensor([0, 39, 5, 5], dtype=torch.int32)
    xs, status = torch.empty(4, size, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_positions32(xs, dev(E), dev(P), ids.cuda(), pos.cuda(), status)
    assert torch.equal(xs.cpu(), E[ids.long()] + P[pos.long()]) and int(status.item()) == 0
    # latents: two norms with plain weights, one to a buffer, one to the pool at scattered places
    q_rank, kv_rank = 24, 40
    raw, wq, wkv = R(n, q_rank + kv_rank, s=2.0), R(q_rank) + 1, R(kv_rank) + 1
    cq, pool = torch.empty(n, q_rank, dtype=T, device="cuda"), torch.zeros(64, kv_rank, dtype=T, device="cuda")
    places = torch.tensor([5, 63, 0, 17, 18, 40, 2, 9, 33], dtype=torch.int32)
    ops.latent_inputs(dev(raw), cq, pool, dev(wq), dev(wkv), 1e-6, places.cuda(), q_rank, kv_rank)
    close(cq, plain.norm_plain(raw[:, :q_rank], wq, 1e-6), "query latent")
    close(pool[places.long().cuda()], plain.norm_plain(raw[:, q_rank:], wkv, 1e-6), "key/value latent")
    assert float(pool.float().abs().sum(1)[1]) == 0.0
    # a product per head
    heads, out_h, in_h = 3, 40, 24
    xh, wh = R(n, heads, in_h), R(heads, out_h, in_h, s=0.3)
    yh = torch.empty(n, heads, out_h, dtype=T, device="cuda")
    ops.head_gemm(yh, dev(xh), dev(wh))
    close(yh, torch.einsum("hoi,nhi->nho", wh.double(), xh.double()).float(), "product per head")
    if T == torch.bfloat16:
        from tileinfer_b200.kernels import fast
        xb = R(300, heads, in_h)
        yb = torch.empty(300, heads, out_h, dtype=T, device="cuda")
        assert fast.head_linear(yb, dev(xb), dev(wh))
        fast.check_status()
        close(yb, torch.einsum("hoi,nhi->nho", wh.double(), xb.double()).float(), "product per head on the tensor cores")
    # activations
    z = R(n, size, s=2.0)
    ops.gelu(y, dev(z), ops.ACT_GELU_ERF)
    close(y, plain.gelu_erf(z.double()).float(), "gelu")
    table, tok = R(30, 2 * size), torch.randint(0, 30, (n,), generator=g, dtype=torch.int32)
    gz = dev(z).clone()
    ops.gated_token_embedding(gz, dev(table), tok.cuda(), size)
    close(gz, (plain.gelu_tanh(z.double()) * table[tok.long(), size:].double()).float(), "gated token vector")
    gu = R(n, 2 * 48, s=2.0)
    act = torch.empty(n, 48, dtype=T, device="cuda")
    ops.gated_unit_limit(act, dev(gu), 1.25, 1.702, 1.0)
    a, b = gu[:, :48].clamp(max=1.25).double(), gu[:, 48:].clamp(-1.25, 1.25).double()
    close(act, (a * torch.sigmoid(1.702 * a) * (b + 1)).float(), "gated unit")
    # router: the largest logits, ties to the smaller index, always-on units behind them
    hr, wr = R(n, size), R(7, size, s=0.3)
    wr[4] = wr[2]                                                  # two experts with equal logits
    ids_out = torch.empty(n, 5, dtype=torch.int32, device="cuda")
    sc_out = torch.empty(n, 5, dtype=torch.float32, device="cuda")
    ops.router_topk(dev(hr), dev(wr), 3, ids_out, sc_out, always=2)
    zr = (hr.double() @ wr.double().t())
    order = sorted(range(7), key=lambda e: (-float(zr[0, e]), e))[:3]
    assert ids_out[0].tolist() == order + [7, 8] and sc_out[0, 3:].tolist() == [1.0, 1.0]
    assert torch.allclose(sc_out[:, :3].cpu(), torch.sigmoid(torch.sort(zr, descending=True).values[:, :3]).float(), atol=1e-5)
    for row in ids_out.cpu().tolist():
        assert not (4 in row[:3] and 2 not in row[:3])             # of equal logits the smaller index goes first


def _close(got, ref, T, what):
    tol = (1e-5 if T == torch.float32 else 2.0 ** -7) * max(1.0, float(ref.abs().max()))
    err = float((got.float().cpu() - ref.float()).abs().max())
    assert err <= tol, f"{what}: |d| = {err:.3g} > {tol:.3g}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("shared", [0, 56, 40])
def test_routed_units_alone(dtype, shared):
    """The routed feed-forward part alone on random inputs against the plain implementation: without a shared unit, with
    one that is no multiple of an expert's size, and with one of exactly an expert's size; few rows and many."""
    from tileinfer_b200.config import FeedForwardSpec
    from tileinfer_b200.parts import Runtime, lookup
    from tileinfer_b200.parts.norm import GatheredRows
    T = DTYPES[dtype]
    W, F, E, top = 72, 40, 6, 2
    names = {"router": "router", "expert": "e{}.", "shared": "shared.", "gate": "gate", "up": "up", "down": "down"}
    spec = FeedForwardSpec("routed_experts", "f.", W, F, names,
                           {"experts": E, "top": top, "limit": 1.5, "scale_input": True, "sigmoid_slope": 1.702, "up_shift": 1.0,
                            "shared_size": shared, "shared_limit": 0.8})
    cls = lookup("feed_forward", "routed_experts")
    g = torch.Generator().manual_seed(5 + shared)
    tensors = {d.name: plain.rnd(torch.randn(d.shape, generator=g) * d.init[1] * 2, T) for d in cls.tensors(spec)}
    assert ("f.shared.gate" in tensors) == bool(shared)
    part = cls(spec, {k: v.to(T) for k, v in tensors.items()}, Runtime(T))
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": 1.5}}
    if shared:
        mlp["shared"] = {"ff": shared, "limit": 0.8}
    for n in (1, 5, 300):
        h = plain.rnd(torch.randn(n, W, generator=g), T)
        margins = []
        ref = plain.moe_ff(h, tensors, "f.", mlp, T, margins)
        out = part.forward(h.to(T).cuda(), None)
        assert isinstance(out, GatheredRows)
        got = out.rows.float()[out.index.long()].sum(1).cpu()
        sure = margins[0] > (0.02 if T == torch.bfloat16 else 1e-5)
        tol = (2e-5 if T == torch.float32 else 2.0 ** -6) * float(ref.abs().max())
        assert int(sure.sum()) >= n // 2
        if bool(sure.any()):
            assert float((got - ref)[sure].abs().max()) <= tol
