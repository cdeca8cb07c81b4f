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
