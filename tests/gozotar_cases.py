"""Test bodies for the Gozotar decoder that run the same way on the CPU stand-in of the kernel layer and on the
GPU: each takes ``make_engine(cfg_dict, tensors, **kw)`` and a band (how close the engine has to be), and compares
the engine with the plain implementation in float64."""
from __future__ import annotations

import copy

import torch

import plain_gozotar as plain
from safuvik_tiny import tokens_for, run_cut, rel_err
from vaderax_cases import Band                                     # the same measure of closeness
from gozotar_tiny import CONFIGS, make_tensors, model, latent_layer, attention_layer, parallel_layer, rot
from rbitnet_b200.engine.step import StepEntry


def reference(cfg, tensors, tokens):
    return plain.forward(cfg, tensors, tokens, torch.float64)


def whole(make_engine, name, band, n=150):
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=11, spread=band.spread)
    toks = tokens_for(cfg, n, 5)
    assert band.ok(run_cut(make_engine(cfg, tensors), toks, []), reference(cfg, tensors, toks))


def prefill_against_decoding(make_engine, name, band, n=90, prompt=37):
    """A prompt in one step and the rest token by token, and everything token by token, against the whole."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=12, spread=band.spread)
    toks = tokens_for(cfg, n, 6)
    ref = reference(cfg, tensors, toks)
    eng = make_engine(cfg, tensors)
    assert band.ok(run_cut(eng, toks, list(range(prompt, n))), ref)
    assert band.ok(run_cut(eng, toks, list(range(1, n))), ref)


def portions(make_engine, name, band, n=140):
    """Portions of 2 tokens, of a page, of odd sizes, portions shorter than the convolution's taps, and a last
    portion of one token."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=13, spread=band.spread)
    toks = tokens_for(cfg, n, 7)
    ref = reference(cfg, tensors, toks)
    eng = make_engine(cfg, tensors)
    for cuts in (list(range(2, n, 2)), [64, 128], [3, 8, 9, 63, 65, 127, n - 1], [1, 2, 4, 70], [1, 3, 4, 5, 66, 67, 69]):
        assert band.ok(run_cut(eng, toks, cuts), ref), cuts


def batches_against_alone(make_engine, name, band, lengths=(1, 2, 75, 9, 131), decode=12):
    """Unequal prompts in one step, then decoded together, the shorter requests ending earlier; the slots and pages of
    those that ended are used again by a second batch.  Against each request alone (plain model)."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=14, spread=band.spread)
    eng = make_engine(cfg, tensors, max_tokens=64 * 8)
    for round_ in range(2):
        reqs = [tokens_for(cfg, n + (decode if i % 2 else decode // 2), 20 + 10 * round_ + i) for i, n in enumerate(lengths)]
        refs = [reference(cfg, tensors, r) for r in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step([StepEntry(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, lengths)])
        at = 0
        for i, n in enumerate(lengths):
            got[i].append(out[at:at + n])
            at += n
        fed = list(lengths)
        live = list(range(len(reqs)))
        while live:
            out = eng.step([StepEntry(slots[i], [reqs[i][fed[i]]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(reqs[i])]:
                eng.end_sequence(slots[i])
                live.remove(i)
        assert band.ok_all([(torch.cat(got[i]).float().cpu(), refs[i]) for i in range(len(reqs))]), round_


def slots_and_pages_used_again(make_engine, name, band):
    """A cache of three pages: every sequence gets the pages, the memory's slot, the convolutions' ring and the
    previous token that the one before gave back; nothing of the earlier sequence may show."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=15, spread=band.spread)
    eng = make_engine(cfg, tensors, max_tokens=64 * 3)
    for k, n in enumerate((130, 70, 150, 5, 129)):
        toks = tokens_for(cfg, n, 40 + k)
        got = run_cut(eng, toks, [n // 2, n - 3, n - 2, n - 1])
        assert band.ok(got, reference(cfg, tensors, toks)), k


def long_decoding(make_engine, name, band, n=200, prompt=3):
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=16, spread=band.spread)
    toks = tokens_for(cfg, n, 8)
    assert band.ok(run_cut(make_engine(cfg, tensors), toks, list(range(prompt, n))), reference(cfg, tensors, toks))


def first_tokens(make_engine, name, band):
    """Sequences of one to five tokens (shorter than, as long as and longer than the convolution's taps), whole and
    token by token."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=17, spread=band.spread)
    eng = make_engine(cfg, tensors)
    pairs = []
    for n in (1, 2, 3, 4, 5):
        toks = tokens_for(cfg, n, 50 + n)
        ref = reference(cfg, tensors, toks)
        pairs += [(run_cut(eng, toks, []), ref), (run_cut(eng, toks, list(range(1, n))), ref)]
    assert band.ok_all(pairs)


def random_configuration(make_engine, seed, band, n=100):
    """A configuration drawn from ``seed``: whole, the last tokens one by one, and two unequal requests together."""
    from gozotar_tiny import random_config
    cfg = random_config(seed)
    tensors = make_tensors(cfg, seed=seed, spread=band.spread)
    toks = tokens_for(cfg, n, seed)
    ref = reference(cfg, tensors, toks)
    eng = make_engine(cfg, tensors)
    assert band.ok(run_cut(eng, toks, []), ref), cfg
    assert band.ok(run_cut(eng, toks, [70] + list(range(90, n))), ref), cfg
    other = tokens_for(cfg, 31, seed + 1)
    slots = [eng.new_sequence(), eng.new_sequence()]
    out = eng.step([StepEntry(slots[0], toks[:66], list(range(66))), StepEntry(slots[1], other[:29], list(range(29)))])
    got = [[out[:66]], [out[66:]]]
    for k in range(2):
        out = eng.step([StepEntry(slots[0], [toks[66 + k]], [0]), StepEntry(slots[1], [other[29 + k]], [0])])
        got[0].append(out[:1])
        got[1].append(out[1:])
    for s_ in slots:
        eng.end_sequence(s_)
    assert band.ok_all([(torch.cat(got[0]).float().cpu(), ref[:68]), (torch.cat(got[1]).float().cpu(), reference(cfg, tensors, other))]), cfg


def retention_only():
    """Retention beside an attention branch that is switched off: what a far token does to the last logits went through
    the memory."""
    return model(40, 32, [
        parallel_layer((2, 1, 8, 0.3, 2, rot(100.0, 8)), (2, 16, 8, [0.995, 0.999], rot(1000.0, 16)), 0.0, 1.0, ff=None)])


def far_token_moves_the_logits(make_engine, cfg, tol, n=180, seed=19, least=20.0):
    """Changing the FIRST token must move the last logits, in the engine as in the plain model, whether the sequence
    came whole or was decoded through the memory."""
    tensors = make_tensors(cfg, seed=seed)
    toks = tokens_for(cfg, n, 10)
    other = [(toks[0] + 3) % cfg["vocab"]] + toks[1:]
    ref_a, ref_b = reference(cfg, tensors, toks)[-1], reference(cfg, tensors, other)[-1]
    moved = float((ref_a - ref_b).abs().max() / ref_a.abs().max())
    assert moved > least * tol, f"the configuration forgets too fast for this test ({moved})"
    eng = make_engine(cfg, tensors)
    for cuts in ([], list(range(100, n))):
        a, b = run_cut(eng, toks, cuts)[-1], run_cut(eng, other, cuts)[-1]
        assert rel_err(a[None], ref_a[None]) <= tol and rel_err(b[None], ref_b[None]) <= tol


def _sharp(kind):
    """One attention layer of the given kind alone, without feed-forward and embeddings beside the first."""
    if kind == "latent":
        return model(40, 32, [latent_layer(2, 8, 8, 8, 16, 1.0, base=10000.0, ff=None)])
    if kind == "attention":
        return model(40, 32, [attention_layer(2, 1, 32, 8, 1.0, rot(10000.0, 8), 50.0, True, ff=None)])
    return model(40, 32, [parallel_layer((2, 1, 32, 1.0, 2, rot(10000.0, 8)), (1, 8, 8, [0.9], rot(10.0, 8)), 1.0, 0.0, ff=None)])


def one_far_key_stands_out(make_engine, kind, tol, n, far, cuts, last_only=False):
    """One attention layer.  Position ``far`` holds a token that occurs nowhere else.  The queries' matrix is made the
    keys' matrix (per group), so that a token's query points at the key of an equal token; the last token's embedding is
    the far one's plus a smaller random vector, so that its query still points at the far key (and at its own) while
    its values differ, and the matrices are scaled so that these two scores stand far above the others.  Rotation then turns query and key by the distance
    between them, which only the part of a head that is not turned survives: the test's heads keep such a part.  The
    last logits then carry the far position's values: the engine must agree with the plain model, and exchanging the
    far token must move them a lot.  ``last_only``: only the last position is compared."""
    cfg = copy.deepcopy(_sharp(kind))
    tensors = make_tensors(cfg, seed=23, spread=10.0)
    V = cfg["vocab"]
    toks = [1 + (i * 7) % (V - 3) for i in range(n)]
    toks[far] = V - 1
    toks[-1] = V - 2
    noise = torch.randn(cfg["width"], generator=torch.Generator().manual_seed(7)) * float(tensors["embed"][V - 1].std())
    tensors["embed"][V - 2] = tensors["embed"][V - 1] + 0.3 * noise
    m = cfg["layers"][0]["mixer"]
    if kind == "latent":
        # q_c = U_k^T-aligned: make W_q's unrotated rows U_k D_c and leave the turned rows small
        H, D, R, C = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
        dkv, uk = tensors["l0.mix.dkv"], tensors["l0.mix.uk"]
        q = tensors["l0.mix.q"].view(H, D + R, -1).clone()
        q[:, :D] = (uk.view(H, D, C) @ dkv[:C]) * 0.5
        q[:, D:] *= 0.05
        tensors["l0.mix.q"] = q.reshape(H * (D + R), -1)
        tensors["l0.mix.dkv"][C:] *= 0.05
        tensors["l0.mix.sink"] = torch.full_like(tensors["l0.mix.sink"], -4.0)
        # sharp: the far key's score is 30, the others' a fraction of it
        x_far = tensors["embed"][V - 1].double()
        c_far = plain.rms((dkv[:C].double() @ x_far)[None], cfg["norm"]["eps"])[0] * tensors["l0.mix.dkv.norm"].double()
        match = ((q[:, :D].double() @ x_far) * (uk.double() @ c_far).view(H, D)).sum(-1)
        m["scale"] = 30.0 / float(match.min())
    elif kind == "attention":
        H, G, D = m["heads"], m["kv_heads"], m["dim"]
        k = tensors["l0.mix.k"].view(G, D, -1).clone()
        k[:, :m["rot"]["dims"]] *= 0.05                          # the turned prefix carries little
        tensors["l0.mix.k"] = k.reshape(G * D, -1)
        tensors["l0.mix.q"] = k.repeat_interleave(H // G, dim=0).reshape(H * D, -1).clone()
        tensors["l0.mix.q.norm"] = tensors["l0.mix.k.norm"].clone()
        m["scale"] = 1.5
    else:
        left = m["left"]
        H, G, D = left["heads"], left["kv_heads"], left["dim"]
        k = tensors["l0.mix.left.k"].view(G, D, -1).clone()
        k[:, :left["rot"]["dims"]] *= 0.05
        tensors["l0.mix.left.k"] = k.reshape(G * D, -1)
        tensors["l0.mix.left.q"] = k.repeat_interleave(H // G, dim=0).reshape(H * D, -1).clone()
        tensors["l0.mix.left.q.norm"] = tensors["l0.mix.left.k.norm"].repeat(H // G).clone()
        taps = torch.zeros_like(tensors["l0.mix.left.k.conv"])
        taps[:, -1] = 1.0                                         # the convolution passes the current row
        tensors["l0.mix.left.k.conv"] = taps
        tensors["l0.mix.left.q.conv"] = taps.repeat(H // G, 1)
        left["scale"] = 0.6
    tensors = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in tensors.items()}
    ref = reference(cfg, tensors, toks)
    other = list(toks)
    other[far] = 2
    ref_other = reference(cfg, tensors, other)
    assert float((ref[-1] - ref_other[-1]).abs().max() / ref[-1].abs().max()) > 0.03, "the far key does not stand out"
    eng = make_engine(cfg, tensors)
    pick = (lambda x: x[-1:]) if last_only else (lambda x: x)
    assert rel_err(pick(run_cut(eng, toks, cuts)), pick(ref)) <= tol
    assert rel_err(pick(run_cut(eng, other, cuts)), pick(ref_other)) <= tol


def sink_counts(make_engine, tol):
    """A heavy sink halves the attention's result; one that is left out, scaled or counted per key would show."""
    cfg = copy.deepcopy(_sharp("latent"))
    tensors = make_tensors(cfg, seed=29)
    toks = tokens_for(cfg, 70, 3)
    for sink in (torch.tensor([4.0, -2.0]), torch.tensor([-30.0, 9.0])):
        tensors["l0.mix.sink"] = sink
        ref = reference(cfg, tensors, toks)
        eng = make_engine(cfg, tensors)
        assert rel_err(run_cut(eng, toks, [65]), ref) <= tol
    tensors["l0.mix.sink"] = torch.tensor([-200.0, -200.0])
    without = reference(cfg, tensors, toks)
    assert float((without - ref).abs().max() / ref.abs().max()) > 0.02


def greedy_generation(make_engine, name, prompts=(7, 1, 30), new=24):
    """``Engine.generate`` (scheduler, batches, the captured decode step where there is one) against a greedy loop
    over the plain model."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, seed=21)
    eng = make_engine(cfg, tensors, graphs=True)
    ps = [tokens_for(cfg, n, 60 + i) for i, n in enumerate(prompts)]
    results = eng.generate(ps, max_tokens=new, temperature=0.0, stop_ids=[])
    for p, r in zip(ps, results):
        seq = list(p)
        for step, tok in enumerate(r.tokens):
            logits = reference(cfg, tensors, seq)[-1]
            best = int(torch.argmax(logits))
            if best != tok:
                # a tie within rounding is not a fault; anything else is
                assert float(logits[best] - logits[tok]) <= 1e-4 * float(logits.abs().max()), (step, best, tok)
            seq.append(tok)
        assert len(r.tokens) == new
