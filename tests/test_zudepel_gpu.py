"""The Zudepel design through the engine against the plain implementation (``plain_zudepel``): whole prompts, prompts in
portions down to two tokens, token-by-token decoding, batches of unequal requests against each alone, slots, pages and
states that are used again, long decoding, hand-made weights that make one key, one sink, one decay or one tap stand out,
every kernel alone, greedy generation through the public entry point and trace replay; in 32-bit and in bfloat16, at three
sets of sizes."""
import math
import tempfile

import numpy as np
import pytest
import torch

import plain_zudepel as plain
import zudepel_cases as zc
from replay_util import Trace, run_trace

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


@pytest.fixture(scope="module")
def models():
    with tempfile.TemporaryDirectory() as tmp:
        yield {name: zc.Model(name, seed, tmp) for name, seed in (("A", 11), ("B", 12), ("C", 13))}


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
    for tokens in zc.prompts(m.vocab, [1, 2, 7, 64, 65, 150, 420], 21):
        got = run_cut(engine, tokens, [len(tokens)])
        zc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} whole {len(tokens)}")
    tokens = zc.prompts(m.vocab, [300], 22)[0]
    # Portions that start and end inside and at page borders, shorter than the taps, two tokens, one token.
    for cuts in ([100, 100, 100], [63, 1, 64, 2, 2, 128, 40], [2, 2, 2, 58, 64, 3, 1, 1, 120, 47], [129, 2, 61, 2, 70, 36]):
        got = run_cut(engine, tokens, cuts)
        zc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} portions {cuts[:4]}")


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_a_short_prompt(models, name, dtype):
    """A prompt shorter than the longest convolution, then almost 300 single tokens: pages fill up while decoding, the states
    and the convolutions' histories are carried by one-token steps alone."""
    m = models[name]
    engine = m.engine(dtype, max_tokens=512, max_seqs=2)
    tokens = zc.prompts(m.vocab, [300], 23)[0]
    got = run_cut(engine, tokens, [3])
    zc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_batches_of_unequal_requests_and_reuse_of_slots_pages_and_states(models, name, dtype):
    """Requests of unequal lengths prefilled in one step and decoded together, the shorter ones leaving first; then a second
    batch in the slots, pages and states that the first gave back. Every request is compared with the plain implementation
    of that request alone."""
    m = models[name]
    engine = m.engine(dtype, max_tokens=1024, max_seqs=4)
    for seed, lengths, tails in ((31, [1, 40, 129, 330], [0, 12, 40, 3]), (32, [70, 3, 260, 64], [6, 2, 65, 33])):
        reqs = zc.prompts(m.vocab, lengths, seed)
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
            zc.compare(m, t, got[i], DTYPES[dtype], f"{name} {dtype} batch seed {seed} request {i}")
    assert engine.cache.slots.held == 0


# ---------------------------------------------------------------- mixers alone, on inputs and weights made by hand
def _conv_attention(T, W, heads, kv_heads, dim, vdim, scale, taps, rot, tensors, kv_source=None):
    from tileinfer_b200.config import MixerSpec, PositionSpec
    from tileinfer_b200.parts import Runtime, lookup
    rt = Runtime(T)
    position = None
    pspec = PositionSpec(kind="none")
    if rot:
        pspec = PositionSpec(kind="rope", head_dim=dim, theta=rot[1], max_positions=4096,
                             options={"rotary_dim": rot[0], "table_dtype": "float32", "angles": "float64"})
        position = lookup("position", "rope")(pspec, rt, 1024)
    names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "sink": "sink", "bias_suffix": ".b", "conv_suffix": ".conv", "norm_suffix": ".norm"}
    spec = MixerSpec("conv_attention", "m.", W, heads, kv_heads, dim, True, 1e-6, scale, None, kv_source, pspec, names,
                     {"value_dim": vdim, "conv_taps": taps, "bias": True, "row_norm": True, "sink": True, "gate": True})
    return lookup("mixer", "conv_attention")(spec, {k: v.to(T) if v.dtype.is_floating_point else v for k, v in tensors.items()}, rt, position), spec


def _identity_attention_weights(W, taps, sink):
    """One head of size W whose projections, convolution (the newest tap alone), norms and output are the identity, the gate
    wide open."""
    eye = torch.eye(W)
    conv = torch.zeros(W, taps); conv[:, -1] = 1.0
    t = {"m.o": eye.clone(), "m.g": torch.zeros(W, W), "m.sink": torch.tensor([sink])}
    for k in "qkv":
        t[f"m.{k}"] = eye.clone(); t[f"m.{k}.b"] = torch.zeros(W); t[f"m.{k}.conv"] = conv.clone()
    t["m.q.norm"] = torch.ones(W); t["m.k.norm"] = torch.ones(W)
    t["m.g.b"] = None
    del t["m.g.b"]
    return t


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_one_far_key_stands_out_among_hundreds_and_the_sink_takes_its_share(dtype):
    """One head, identity weights: an ordinary token is the unit vector e1, a marked one e0 with a little e2, and every
    query looks along e0 too (the query projection sends e1 to e0). The marked key's score exceeds the others' by
    scale * 16 * (1 - 0) = 24, so whatever stands at e2 of the output is the marker's share: seen from every later position,
    however far, across page borders, from prompts and from single tokens. With a sink as large as the marked score the
    share halves, and with a sink far below it nothing changes."""
    from test_parts_gpu import OneStep
    T = DTYPES[dtype]
    W, scale = 16, 1.5
    marked_score = scale * 4.0 / math.sqrt(1.0625 / 16)              # an ordinary query (4 e0 after the norm) on the marked key
    for sink, share in ((-30.0, 1.0), (marked_score, 0.5)):
        tensors = _identity_attention_weights(W, 2, sink)
        tensors["m.q"][0, 1] = 1.0; tensors["m.q"][1, 1] = 0.0       # e1 -> e0: ordinary tokens ask along e0 as well
        mixer, spec = _conv_attention(T, W, 1, 1, W, W, scale, 2, None, tensors)
        marked = torch.zeros(W); marked[0] = 1.0; marked[2] = 0.25
        ordinary = torch.zeros(W); ordinary[1] = 1.0
        for mark_at, prompt_len, total in ((0, 1, 150), (63, 64, 200), (64, 140, 330), (5, 300, 310), (128, 129, 260)):
            h = ordinary.repeat(total, 1)
            h[mark_at] = marked
            env = OneStep(mixer, T, max_tokens=512, max_seqs=2)
            slot = env.cache.alloc_slot()
            out = [env.run(mixer, [(slot, h[:prompt_len].to(T))], W)]
            out += [env.run(mixer, [(slot, h[t:t + 1].to(T))], W) for t in range(prompt_len, total)]
            out = torch.cat(out)
            # Values are not normed: the marker's 0.25 at e2 reaches the output times the share and the half-open gate.
            want = 0.25 * share * 0.5
            seen = out[mark_at + 1:, 2]                           # (the marked token's own query is longer: its share differs)
            assert float((seen - want).abs().max()) <= (0.005 if T == torch.float32 else 0.04) * want, \
                f"sink {sink}, marker at {mark_at}: {seen[:3].tolist()} .. {seen[-3:].tolist()}, want {want}"
            assert float(out[:mark_at, 2].abs().max()) == 0.0 if mark_at else True


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_every_tap_reads_its_own_row_across_steps(dtype):
    """Identity weights but a convolution whose taps are 1, 10, 100, 1000 from the oldest to the newest on the VALUE channels:
    with a single marked token (value 1 in one channel, scores flat) the values of the following positions carry the taps'
    digits. Sequences are cut so that the history comes from the step itself, from the state, and from before the start."""
    from test_parts_gpu import OneStep
    T = torch.float32 if dtype == "float32" else torch.bfloat16
    W, taps = 16, 4
    tensors = _identity_attention_weights(W, taps, -30.0)
    tensors["m.v.conv"] = torch.tensor([1.0, 8.0, 64.0, 512.0]).repeat(W, 1)
    tensors["m.q"] = torch.zeros(W, W)                                # flat scores: every position averages the values so far
    mixer, spec = _conv_attention(T, W, 1, 1, W, W, 1.0, taps, None, tensors)
    total, mark_at = 12, 2
    h = torch.zeros(total, W); h[:, 5] = 1.0                          # keys and queries need a non-zero row for the norm
    h[mark_at, 9] = 1.0
    # values y_t[9] = sum_j c[j] u_(t - 3 + j)[9]: 512 at the mark, 64 one later, 8, 1, then 0.
    y = torch.zeros(total); y[mark_at:mark_at + 4] = torch.tensor([512.0, 64.0, 8.0, 1.0])
    want = torch.cumsum(y, 0) / torch.arange(1, total + 1) * 0.5
    for cuts in ([12], [1] * 12, [3, 1, 1, 7], [2, 2, 2, 6], [4, 8], [5, 1, 6]):
        env = OneStep(mixer, T, max_tokens=512, max_seqs=2)
        slot, at, out = env.cache.alloc_slot(), 0, []
        for n in cuts:
            out.append(env.run(mixer, [(slot, h[at:at + n].to(T))], W))
            at += n
        got = torch.cat(out)[:, 9]
        assert float((got - want).abs().max()) <= (1e-4 if T == torch.float32 else 0.01) * float(want.max()), f"cuts {cuts}: {got.tolist()}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_a_marked_token_fades_by_the_decay_and_no_faster(dtype):
    """The lightning mixer with identity-like weights: one marked token writes k v^T into the state, every later query reads it
    back times decay^(distance). Two heads with different decays; whole, token by token and in portions; a second sequence
    in the batch must not see it, nor a new sequence in the same slot."""
    from tileinfer_b200.config import MixerSpec
    from tileinfer_b200.parts import Runtime, lookup
    from test_parts_gpu import OneStep
    T = DTYPES[dtype]
    W, H, D, V = 16, 2, 4, 8
    decay = [0.5, 0.98]
    # Inputs far from zero so that SiLU is close to the identity: channel c of q, k is h[c] (heads 0, 1 <- elements 0..7), v likewise.
    sel = lambda rows, first: torch.eye(W)[first:first + rows]
    tensors = {"m.q": sel(H * D, 0), "m.k": sel(H * D, 0), "m.v": torch.cat([sel(V, 8), sel(V, 8)]), "m.g": torch.zeros(H * V, W),
               "m.o": torch.eye(W, H * V), "m.norm": torch.ones(H * V)}
    names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}
    spec = MixerSpec(kind="lightning", prefix="m.", hidden_size=W, num_heads=H, head_dim=D, tensor_names=names,
                     options={"value_dim": V, "decay": decay, "norm_eps": 1e-6, "gate": True, "activation": "none"})
    mixer = lookup("mixer", "lightning")(spec, {k: v.to(T) for k, v in tensors.items()}, Runtime(T), None)
    total, mark_at = 140, 3
    # Ordinary tokens have q = e0 per head (elements 0 and 4) and k = 0 elsewhere... they write k v^T with v = 0: nothing.
    h = torch.zeros(total, W); h[:, 0] = 1.0; h[:, 4] = 1.0
    h[mark_at, 8 + 2] = 1.0                                            # the marked token alone has a value: e2
    ref = torch.zeros(total, H * V, dtype=F64)
    for t in range(mark_at, total):
        for hd in range(H):
            ref[t, hd * V + 2] = decay[hd] ** (t - mark_at)
    ref = (ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + 1e-6) * 0.5).float()
    other = torch.zeros(40, W); other[:, 0] = 1.0
    for cuts in ([total], [1] * total, [2, 1, 1, 60, 2, 74], [4, 136]):
        env = OneStep(mixer, T, max_tokens=512, max_seqs=2)
        a, b = env.cache.alloc_slot(), env.cache.alloc_slot()
        at, out = 0, []
        for i, n in enumerate(cuts):
            entries = [(a, h[at:at + n].to(T))]
            if i < 40:
                entries = [(b, other[i:i + 1].to(T))] + entries          # a neighbour in the batch, in front
            r = env.run(mixer, entries, W)
            if i < 40:
                assert float(r[0].abs().max()) == 0.0                    # the neighbour's state stays empty
                r = r[1:]
            out.append(r)
            at += n
        got = torch.cat(out)[:, :H * V]
        tol = 2e-5 if T == torch.float32 else 2.0 ** -7
        assert float((got - ref).abs().max()) <= tol, f"cuts {cuts[:5]}"
        env.cache.free_slot(a)
        again = env.cache.alloc_slot()                                   # the slot's state starts from zero again
        assert again == a and float(env.run(mixer, [(again, other[:5].to(T))], W).abs().max()) == 0.0


# ---------------------------------------------------------------- kernels alone
def _tol(T, ref, f32=2e-5, bf=2.0 ** -7):
    return (f32 if T == torch.float32 else bf) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_lightning_scan_alone(dtype):
    """The recurrence kernel against a loop, at sizes of its own: value sizes that are no multiple of a block's 32 columns, key
    sizes up to the largest, sequences of unequal lengths in one launch, continued from a state."""
    from tileinfer_b200.kernels import ops
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(5)
    for H, D, V, lens in ((3, 12, 20, [1, 37, 5]), (2, 130, 33, [70]), (1, 256, 64, [3, 18]), (5, 8, 96, [16, 17, 15, 1]), (2, 400, 36, [1, 1]),
                          (1, 512, 32, [40]), (3, 24, 132, [1, 1, 1, 1])):
        n = sum(lens)
        rows_ = plain.rnd(torch.randn(n, 2 * H * D + H * V + 7, generator=g).to(F64), T).to(T)
        decay = torch.rand(H, generator=g) * 0.5 + 0.5
        state0 = torch.randn(len(lens) + 2, H, D, V, generator=g)
        slots = torch.tensor([len(lens) + 1 - i for i in range(len(lens))], dtype=torch.int32)       # slots in another order than the sequences
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        state = state0.clone().cuda()
        o = torch.empty(n, H * V, dtype=torch.float32, device="cuda")
        ops.lightning_scan(o, rows_.cuda(), 0, H * D, 2 * H * D, state, decay.cuda(), cu.cuda(), slots.cuda(), len(lens), H, D, V, act=True)
        x = rows_.to(F64)
        act = lambda z: plain.rnd(plain.silu(z), T)
        q, k, v = act(x[:, :H * D]).view(n, H, D), act(x[:, H * D:2 * H * D]).view(n, H, D), act(x[:, 2 * H * D:2 * H * D + H * V]).view(n, H, V)
        ref = torch.zeros(n, H, V, dtype=F64)
        for b, L in enumerate(lens):
            S = state0[slots[b]].to(F64)
            for t in range(int(cu[b]), int(cu[b]) + L):
                S = decay.to(F64)[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
                ref[t] = torch.einsum("hdv,hd->hv", S, q[t])
            assert float((state[slots[b]].cpu() - S.float()).abs().max()) <= 1e-4 * max(1.0, float(S.abs().max()))
        assert float((o.cpu() - ref.view(n, -1).float()).abs().max()) <= 1e-4 * max(1.0, float(ref.abs().max()))
        assert torch.equal(state[0].cpu(), state0[0])                                              # a slot of no sequence is left alone


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_router_with_groups_corrections_and_pass_through_choices_alone(dtype):
    """router_select against the plain router, with corrections large enough to make choice scores negative and to send the
    choice elsewhere than the largest softmax values, groups that lose, ties, and a gate for the always-on units."""
    from tileinfer_b200.kernels import ops
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(9)
    for E, I, top, groups, keep, always in ((6, 2, 3, 4, 2, 2), (15, 5, 3, 5, 2, 1), (5, 0, 1, 1, 1, 0), (3, 1, 4, 1, 1, 0), (8, 4, 2, 6, 1, 1)):
        n, width, total = 70, 24, E + I
        h = plain.rnd(torch.randn(n, width, generator=g).to(F64), T)
        wr = plain.rnd(torch.randn(total + 1, width, generator=g).to(F64) * 0.7, T)
        corr = torch.randn(total, generator=g) * 0.3 - 0.2
        mlp = {"router": {"experts": E, "identity": I, "top": top, "groups": {"count": groups, "keep": keep}}}
        W = {"r.router": wr[:total], "r.correction": corr}
        chosen, w, margin = plain.route(h, W, "r.", mlp, T)
        ids = torch.empty(n, top + always, dtype=torch.int32, device="cuda")
        scores = torch.empty(n, top + always, dtype=torch.float32, device="cuda")
        pass_w = torch.empty(n, dtype=torch.float32, device="cuda")
        for logits in (None, (h @ wr.t()).float().cuda()):
            ops.router_select(h.to(T).cuda(), wr.to(T).cuda(), logits, E, total, top, ids, scores, pass_w, softmax=True, correction=corr.cuda(),
                              groups=groups, keep=keep, renormalize=True, always=always, gate=True)
            gi, gs, gp = ids.cpu(), scores.cpu(), pass_w.cpu()
            sg = torch.sigmoid(h @ wr[total])
            for t in range(n):
                if margin[t] < 1e-4:
                    continue
                want = {int(e): float(x) for e, x in zip(chosen[t], w[t])}
                got = {int(e): float(x) for e, x in zip(gi[t, :top], gs[t, :top]) if e >= 0}
                assert set(got) == {e for e in want if e < E}, f"token {t}: {got} against {want}"
                assert all(abs(got[e] - want[e]) <= 1e-5 for e in got)
                assert abs(float(gp[t]) - sum(x for e, x in want.items() if e >= E)) <= 1e-5
                assert int((gi[t, :top] < 0).sum()) == sum(1 for e in want if e >= E)
                assert gi[t, top:].tolist() == list(range(E, E + always)) and all(abs(float(x) - float(sg[t])) <= 1e-5 for x in gs[t, top:])


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_small_kernels_alone(dtype):
    """The stream's update by two sublayers at once, the gated activations, the output gate, the norm with a gate."""
    from tileinfer_b200.kernels import ops
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(7)
    R = lambda *shape, s=1.0: plain.rnd(torch.randn(*shape, generator=g).to(F64) * s, T)
    n, size = 37, 72
    x, d1, d2, w = torch.randn(n, size, generator=g), R(n, size), R(n, size), R(size)
    parts = torch.randn(3, n, size, generator=g)
    for a, b, ref_d in ((d1, d2, d1 + d2), (d1, None, d1), (parts, d2, parts.sum(0).to(F64) + d2), (d1, parts, d1 + parts.sum(0).to(F64))):
        xs, h = x.clone().cuda(), torch.empty(n, size, dtype=T, device="cuda")
        dev = lambda t: None if t is None else (t.float().cuda() if t.dim() == 3 else t.to(T).cuda())
        ops.sum_add_norm32(xs, dev(a), dev(b), h, w.to(T).cuda(), 1e-5)
        ref_x = x.to(F64) + ref_d
        assert float((xs.cpu() - ref_x.float()).abs().max()) <= 1e-5
        ref_h = plain.rms_norm(ref_x, w, 1e-5)
        assert float((h.float().cpu() - ref_h.float()).abs().max()) <= _tol(T, ref_h)
    for kind, act in ((ops.ACT_SILU_GATED, plain.silu), (ops.ACT_GELU_TANH_GATED, plain.gelu_tanh)):
        gu = R(n, 2 * 50, s=2.0)
        y = torch.empty(n, 50, dtype=T, device="cuda")
        ops.gated_act(y, gu.to(T).cuda(), kind)
        ref = act(gu[:, :50]) * gu[:, 50:]
        assert float((y.float().cpu() - ref.float()).abs().max()) <= _tol(T, ref)
    heads, V, Dp = 3, 14, 16
    attn, gate = R(n, heads, Dp), R(n, heads * V + 5)
    y = torch.empty(n, heads * V, dtype=T, device="cuda")
    ops.sigmoid_gate(y, attn.to(T).cuda(), gate.to(T).cuda()[:, 5:], heads, V, Dp)
    ref = attn[:, :, :V].reshape(n, -1) * torch.sigmoid(gate[:, 5:])
    assert float((y.float().cpu() - ref.float()).abs().max()) <= _tol(T, ref)
    o = torch.randn(n, size, generator=g) * 30
    ops.lightning_out(h, o.cuda(), d1.to(T).cuda(), w.to(T).cuda(), 1e-5)
    ref = plain.rms_norm(o, w, 1e-5) * torch.sigmoid(d1)
    assert float((h.float().cpu() - ref.float()).abs().max()) <= _tol(T, ref)


def test_every_attention_kernel_counts_the_sink():
    """The mixer alone in bfloat16 at sizes that the tensor-memory kernel (heads of 64, long prompt), the mma.sync kernel (short
    prompt), the split decode kernel with one and with several parts, and the plain kernel take: against the plain
    implementation with sinks large enough to take a third of the weight."""
    from tileinfer_b200.kernels import library
    from test_parts_gpu import OneStep
    T = torch.bfloat16
    g = torch.Generator().manual_seed(17)
    W, H, G, D, V = 64, 4, 2, 64, 48
    R = lambda *shape, s=1.0: plain.rnd(torch.randn(*shape, generator=g).to(F64) * s, T)
    tensors = {"m.q": R(H * D, W, s=W ** -0.5), "m.k": R(G * D, W, s=W ** -0.5), "m.v": R(G * V, W, s=W ** -0.5), "m.g": R(H * V, W, s=W ** -0.5),
               "m.o": R(W, H * V, s=(H * V) ** -0.5), "m.sink": torch.tensor([2.0, -1.0, 4.0, 0.5])}
    for k, r in (("q", H * D), ("k", G * D), ("v", G * V)):
        tensors[f"m.{k}.b"] = R(r, s=0.1)
        tensors[f"m.{k}.conv"] = R(r, 3, s=0.5)
    tensors["m.q.norm"], tensors["m.k.norm"] = 1 + R(H * D, s=0.1), 1 + R(G * D, s=0.1)
    mix = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.3, "conv": 3, "rot": {"dims": 32, "base": 1000.0}}
    for kernels, lens in (("fast", [480]), ("fast", [90, 30]), ("plain", [130])):
        mixer, spec = _conv_attention(T, W, H, G, D, V, 0.3, 3, (32, 1000.0), tensors)
        mixer.rt.kernels = kernels
        hs = [R(n + 24, W) for n in lens]
        env = OneStep(mixer, T, max_tokens=2048, max_seqs=2)
        slots = [env.cache.alloc_slot() for _ in lens]
        library.call_counts.clear()
        out = env.run(mixer, [(s, h[:n].to(T)) for s, h, n in zip(slots, hs, lens)], W)
        outs = [list(out.split(lens))]
        for t in range(24):
            outs.append(list(env.run(mixer, [(s, h[n + t:n + t + 1].to(T)) for s, h, n in zip(slots, hs, lens)], W).split([1] * len(lens))))
        used = dict(library.call_counts)
        if kernels == "fast":
            assert used.get("ti_attention_decode_sink", 0) == 24 and "ti_attention_plain" not in used
            assert used.get("ti_attention_prefill_tc_sink" if lens[0] > 400 else "ti_attention_prefill_sink", 0) == 1
        else:
            assert used.get("ti_attention_plain", 0) == 25
        W64 = {k: v.to(F64) for k, v in tensors.items()}
        for i, h in enumerate(hs):
            kv = plain.attention_keys_values(h, W64, "m.", mix, 1e-6, T)
            ref = plain.attention(h, W64, "m.", mix, 1e-6, T, kv).float()
            got = torch.cat([o[i] for o in outs])
            err = (got - ref).abs().max(-1).values
            assert float(err.max()) <= 6 * 2.0 ** -8 * float(ref.abs().max()), \
                f"{kernels} {lens} sequence {i}: worst at {int(err.argmax())}: {float(err.max()):.3g} (scale {float(ref.abs().max()):.3g}); first bad {int((err > 6 * 2.0 ** -8 * float(ref.abs().max())).float().argmax())}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_models_of_one_kind_of_layer_and_of_one_layer(dtype):
    """Layers of lightning alone (a cache without pages), of attention alone (no state but the taps'), a single layer without
    feed-forward: whole, in portions and decoded, against the plain implementation."""
    T = DTYPES[dtype]
    cases = {
        "lightning only": {"architecture": "Zudepel", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
                           "layers": [zc.lightning(2, 8, 12, [0.9, 0.6], zc.dense(40)), zc.lightning(3, 16, 4, [0.99, 0.5, 0.8], None)]},
        "attention only": {"architecture": "Zudepel", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
                           "layers": [zc.attention(4, 2, 8, 12, 0.3, zc.dense(40), conv=2, rot=(4, 50.0)),
                                      zc.attention(4, 2, 8, 12, 0.3, None, conv=3, rot=(4, 50.0), kv_from=0)]},
        "one layer": {"architecture": "Zudepel", "vocab": 33, "width": 32, "norm": {"eps": 1e-6}, "layers": [zc.lightning(1, 32, 32, [0.95], None)]},
    }
    with tempfile.TemporaryDirectory() as tmp:
        for name, case in cases.items():
            zc.CASES[name] = case
            try:
                m = zc.Model(name, 3, tmp)
            finally:
                del zc.CASES[name]
            engine = m.engine(dtype, max_tokens=512, max_seqs=2, max_context=256)
            tokens = zc.prompts(m.vocab, [130], 5)[0]
            for cuts in ([130], [2, 64, 3], [70, 1, 1, 58]):
                zc.compare(m, tokens, run_cut(engine, tokens, cuts), T, f"{name} {dtype} {cuts}")


# ---------------------------------------------------------------- through the public entry points
def test_greedy_generation_through_the_public_entry_point(models):
    """``generate`` (batches, scheduler, sampler, decode loop) on several prompts at once, in 32-bit: every generated token is
    the plain implementation's most likely next token for the same prefix."""
    import tileinfer_b200 as ti
    m = models["A"]
    engine = ti.load_model(m.folder, dtype="float32", max_context=256, max_seqs=3)
    reqs = zc.prompts(m.vocab, [3, 41, 90, 17], 41)
    outs = ti.generate(engine, reqs, max_new_tokens=40, stop_ids=[])
    assert [len(o) for o in outs] == [40] * 4
    for p, o in zip(reqs, outs):
        ref = plain.forward(m.cfg, m.W, p + o, torch.float32).numpy()
        for k, tok in enumerate(o):
            row = ref[len(p) + k - 1]
            assert row[tok] >= row.max() - 1e-4, f"token {k}: generated {tok}, plain argmax {int(row.argmax())}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_trace_replay(models, dtype):
    """The same requests through ``bin/trace_run``: whole, with the tail one by one, and in two batches one after the other (the
    second in the first one's slots, pages and states)."""
    m = models["B"]
    reqs = {f"r{i}": t for i, t in enumerate(zc.prompts(m.vocab, [1, 9, 70, 130, 200], 51))}
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
        zc.compare(m, reqs[rid[1:]], g, DTYPES[dtype], f"replay {dtype} {rid}")


def test_bfloat16_steps_take_the_fast_kernels(models):
    """Case B's sizes are ones the fast kernels take: a prompt and a decode step in bfloat16 go through the tensor-core products
    (grouped ones for the experts) and the paged attention kernels with a sink, not through their plain stand-ins."""
    from tileinfer_b200.kernels import library
    m = models["B"]
    engine = m.engine("bfloat16", graphs=False)
    slot = engine.new_sequence()
    library.call_counts.clear()
    engine.step([(slot, zc.prompts(m.vocab, [600], 61)[0])])
    engine.step([(slot, [5])])
    engine.free_sequence(slot)
    engine.check_health()
    used = library.call_counts
    assert used.get("ti_gemm_tcgen05_grouped", 0) == 8 and used.get("ti_router_select", 0) == 4
    assert used.get("ti_attention_prefill_tc_sink", 0) == 3 and used.get("ti_attention_decode_sink", 0) == 3
    assert used.get("ti_lightning_scan", 0) == 2 and used.get("ti_conv_attention_inputs", 0) == 6
    assert "ti_grouped_gemm" not in used and "ti_attention_plain" not in used and "ti_gemm_plain" not in used
