"""Test bodies for the Nifarax decoder that run the same way on the CPU stand-in of the kernel layer and on the
GPU: each takes ``make_engine(cfg_dict, tensors, **kw)`` and a band (how close the engine has to be), and compares
the engine with the plain implementation in float64."""
from __future__ import annotations

import torch

import plain_nifarax as plain
from safuvik_tiny import tokens_for, run_cut, rel_err
from vaderax_cases import Band                                     # the same measure of closeness
from nifarax_tiny import CONFIGS, make_tensors, gla_layer, latent_layer, model
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
    """A cache of three pages: every sequence gets the pages, the memory's slot and the convolutions' rings that the
    one before gave back; nothing of the earlier sequence may show."""
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


def gla_only(taps=3):
    """Memory layers alone: what a far token does to the last logits went through the memory."""
    return model(40, 32, 2, taps, 25.0, [gla_layer(2, 16, 8, 16.0, 4, None), gla_layer(4, 8, 8, 32.0, 3, None)])


def far_token_moves_the_logits(make_engine, cfg, tol, n=180, seed=19, least=20.0):
    """Changing the FIRST token must move the last logits, in the engine as in the plain model, whether the sequence
    came whole or was decoded through the memory."""
    tensors = make_tensors(cfg, seed=seed, long_memory=True)
    toks = tokens_for(cfg, n, 10)
    other = [(toks[0] + 3) % cfg["vocab"]] + toks[1:]
    ref_a, ref_b = reference(cfg, tensors, toks)[-1], reference(cfg, tensors, other)[-1]
    moved = float((ref_a - ref_b).abs().max() / ref_a.abs().max())
    assert moved > least * tol, f"the configuration forgets too fast for this test ({moved})"
    eng = make_engine(cfg, tensors)
    for cuts in ([], list(range(100, n))):
        a, b = run_cut(eng, toks, cuts)[-1], run_cut(eng, other, cuts)[-1]
        assert rel_err(a[None], ref_a[None]) <= tol and rel_err(b[None], ref_b[None]) <= tol


def latent_only(kv_rank=16):
    """One attention layer without feed-forward, one tap (the filter only scales), one norm group."""
    return model(40, 32, 1, 1, 25.0, [latent_layer(2, 16, 8, kv_rank, kv_rank, 1.0, None)])


def one_far_key_stands_out(make_engine, tol, n, far, cuts, last_only=False, kv_rank=16):
    """One attention layer.  Position ``far`` holds a token that occurs nowhere else, and the last token's query is made
    to point at that token's key, far above every other score.  The last logits then carry that position's latent: the
    engine must agree with the plain model, and exchanging the far token must move them a lot.  ``last_only``: only the
    last position is compared (in bfloat16 the sharp scores of the other positions, which nothing here arranges,
    amplify the rounding of queries and latents)."""
    cfg = latent_only(kv_rank)
    tensors = make_tensors(cfg, seed=23, spread=10.0)
    V = cfg["vocab"]
    toks = [1 + (i * 7) % (V - 3) for i in range(n)]
    toks[far] = V - 1
    toks[-1] = V - 2
    # The last token's embedding is the far token's with its values permuted; the queries' way through their latent is
    # the keys' way with the first matrix's columns permuted alike, and everything before the two is blind to a
    # permutation (one norm group without weights, the same tap on every channel).  So q(last) = k(far), |k|^2 of them.
    perm = torch.randperm(cfg["width"], generator=torch.Generator().manual_seed(5))
    emb = tensors["embed"]
    emb[V - 2] = emb[V - 1][perm]
    for name in ("embed.norm", "l0.norm1"):
        tensors[name] = torch.ones_like(tensors[name])
    tensors["l0.canon1"] = torch.full_like(tensors["l0.canon1"], 0.25)
    tensors["l0.mix.dq"] = tensors["l0.mix.dkv"][:, perm].clone()
    tensors["l0.mix.dq.norm"] = tensors["l0.mix.dkv.norm"].clone()
    tensors["l0.mix.uq"] = tensors["l0.mix.uk"].clone()
    # sharp: the far key's score is |k|^2 * scale, the others' a fraction of it
    k_far = (plain.rms(1.25 * plain.rms(emb[V - 1].double()[None], 1e-5) @ tensors["l0.mix.dkv"].double().T, 1e-5)
             * tensors["l0.mix.dkv.norm"].double()) @ tensors["l0.mix.uk"].double().T
    cfg["layers"][0]["mixer"]["scale"] = 60.0 / float((k_far.view(2, 16) ** 2).sum(-1).min())
    ref = reference(cfg, tensors, toks)
    other = list(toks)
    other[far] = 2
    ref_other = reference(cfg, tensors, other)
    assert float((ref[-1] - ref_other[-1]).abs().max() / ref[-1].abs().max()) > 0.05
    eng = make_engine(cfg, tensors)
    pick = (lambda x: x[-1:]) if last_only else (lambda x: x)
    assert rel_err(pick(run_cut(eng, toks, cuts)), pick(ref)) <= tol
    assert rel_err(pick(run_cut(eng, other, cuts)), pick(ref_other)) <= tol


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
