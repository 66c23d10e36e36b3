"""The Gozotar decoder on the GPU: the package's kernels against the plain implementation (whole models in both
dtypes, the same cases as on the CPU), and each new kernel alone against the plain functions."""
import copy

import numpy as np
import pytest
import torch

import plain_gozotar as plain
import gozotar_cases as cases
from safuvik_tiny import tokens_for, rel_err
from gozotar_tiny import CONFIGS, make_tensors, rot
from rbitnet_b200.config import config_from_dict

pytestmark = pytest.mark.gpu

# Fractions of the largest reference value.  float32: the weights are scaled up so that faults show, which amplifies
# rounding.  bfloat16: operands of the products, q, the cache, the attention's P and the rows between a feed-forward's
# products are rounded to 8 bits.
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
# whole models in bfloat16, matrices spread by 4: a retention head's outputs are divided by their root mean square, which
# at a sequence's first positions is |k . q| |v| of one or two tokens and can be as small as its own rounding; such
# single positions may lie outside the band (one in twenty), while the median stays within a third of it
BAND = {"float32": cases.Band(2e-4), "bfloat16": cases.Band(6e-2, spikes=0.05, spread=4.0)}
DTYPES = ["float32", "bfloat16"]


def engine_maker(dtype):
    from rbitnet_b200.engine import Engine

    def make(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
        return Engine(config_from_dict(cfg), dict(tensors), dtype=dtype, max_tokens=max_tokens, max_seq=1024,
                      use_graphs=graphs, **kw)
    return make


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole(name, dtype):
    cases.whole(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prefill_against_decoding(name, dtype):
    cases.prefill_against_decoding(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", list(range(1, 17)))
def test_random_configurations(seed, dtype):
    cases.random_configuration(engine_maker(dtype), seed, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_portions(name, dtype):
    cases.portions(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_batches(name, dtype):
    cases.batches_against_alone(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_slots_and_pages_used_again(name, dtype):
    cases.slots_and_pages_used_again(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding(name, dtype):
    cases.long_decoding(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
def test_first_tokens(name, dtype):
    cases.first_tokens(engine_maker(dtype), name, BAND[dtype])


def test_far_token_through_the_memory():
    # float32 only: what the first token of 180 leaves in the last logits is of the size of bfloat16's rounding
    cases.far_token_moves_the_logits(engine_maker("float32"), cases.retention_only(), TOL["float32"], least=10.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["latent", "attention", "left"])
@pytest.mark.parametrize("n,far,cuts", [(300, 2, []), (300, 63, [250] + list(range(290, 300))), (200, 64, list(range(1, 200))),
                                        (700, 0, [64, 128, 699]), (130, 127, [129])])
def test_one_far_key(n, far, cuts, kind, dtype):
    cases.one_far_key_stands_out(engine_maker(dtype), kind, TOL[dtype], n, far, cuts, last_only=dtype == "bfloat16")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink(dtype):
    cases.sink_counts(engine_maker(dtype), TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_greedy_generation_through_captured_steps(name):
    cases.greedy_generation(engine_maker("float32"), name)


def test_captured_step_in_bfloat16():
    """The captured decode step (padding rows, state saved around the trial run) against the plain model."""
    from rbitnet_b200.engine.step import StepEntry
    cfg = CONFIGS["C"]
    tensors = make_tensors(cfg, 23, spread=4.0)
    eng = engine_maker("bfloat16")(cfg, tensors, graphs=True)
    reqs = [tokens_for(cfg, n, 70 + n) for n in (20, 9, 33)]
    slots = [eng.new_sequence() for _ in reqs]
    eng.step([StepEntry(s, r[:-6], []) for s, r in zip(slots, reqs)])
    got = [[] for _ in reqs]
    for k in range(6, 0, -1):
        out = eng.step([StepEntry(s, [r[-k]], [0]) for s, r in zip(slots, reqs)], captured=True)
        for i in range(len(reqs)):
            got[i].append(out[i:i + 1])
    assert BAND["bfloat16"].ok_all([(torch.cat(got[i]).float().cpu(), plain.forward(cfg, tensors, r)[-6:])
                                    for i, r in enumerate(reqs)])


def _mid_sizes():
    """Sizes that every tensor-core kernel takes: cached rows of 128 (tcgen05 prefill, TMA decode) with sinks, heads of
    128 and of 64 with the soft cap, products of 512 to 2,048 columns."""
    from gozotar_tiny import model, latent_layer, attention_layer, parallel_layer
    stretched = (8.0, 1.0, 4.0, 128)
    return model(1000, 512, [
        latent_layer(8, 64, 32, 64, 96, 0.1, base=10000.0, ff=1536),
        attention_layer(8, 2, 128, 64, 0.09, rot(100000.0, 64, stretched), 15.0, True, ff=1536),
        parallel_layer((8, 2, 64, 0.12, 4, rot(10000.0, 32)), (4, 64, 128, [0.9, 0.97, 0.99, 0.999], rot(5000.0, 64)), 0.7, 0.6,
                       ff=1536),
        attention_layer(8, 2, 128, 64, 0.09, rot(100000.0, 64), None, True, ff=1536)], bigram=(4099, 211, 17), side=64)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mid_sizes(dtype):
    """Whole, the last 40 tokens one by one, and an unequal batch decoded together, at sizes of the tensor-core kernels."""
    from safuvik_tiny import run_cut
    from rbitnet_b200.engine.step import StepEntry
    cfg = _mid_sizes()
    band = BAND[dtype]
    tensors = make_tensors(cfg, seed=31, spread=band.spread)
    eng = engine_maker(dtype)(cfg, tensors, max_tokens=64 * 16)
    toks = tokens_for(cfg, 200, 9)
    ref = plain.forward(cfg, tensors, toks)
    assert band.ok(run_cut(eng, toks, []), ref)
    assert band.ok(run_cut(eng, toks, list(range(160, 200))), ref)
    reqs = [toks[:150], tokens_for(cfg, 70, 10), tokens_for(cfg, 9, 11)]
    refs = [ref[:150]] + [plain.forward(cfg, tensors, r) for r in reqs[1:]]
    slots = [eng.new_sequence() for _ in reqs]
    cut = [len(r) - 5 for r in reqs]
    out = eng.step([StepEntry(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, cut)])
    got, at = [], 0
    for n in cut:
        got.append([out[at:at + n]])
        at += n
    for k in range(5):
        out = eng.step([StepEntry(s, [r[n + k]], [0]) for s, r, n in zip(slots, reqs, cut)])
        for i in range(len(reqs)):
            got[i].append(out[i:i + 1])
    assert band.ok_all([(torch.cat(g).float().cpu(), r) for g, r in zip(got, refs)])


def test_command_line_and_trace_replay(tmp_path):
    """``python -m rbitnet_b200 random`` makes a model of the design from its config.json; ``generate --temperature 0``
    prints the plain model's greedy ids; ``bin/trace_run`` replays a schedule of two unequal requests on the same folder."""
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    from rbitnet_b200.weights import read_safetensors
    root = Path(__file__).resolve().parent.parent
    cfg = CONFIGS["D"]
    (tmp_path / "cfg.json").write_text(json.dumps(cfg))
    env = dict(os.environ, PYTHONPATH=str(root))
    model = tmp_path / "model"
    p = subprocess.run([sys.executable, "-m", "rbitnet_b200", "random", "--config", str(tmp_path / "cfg.json"), "--out", str(model),
                        "--seed", "5", "--dtype", "float32"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    tensors = {k: v.float() for k, v in read_safetensors(model / "model.safetensors").items()}
    ps = [tokens_for(cfg, 7, 1), tokens_for(cfg, 3, 2)]
    cmd = [sys.executable, "-m", "rbitnet_b200", "generate", "--model", str(model), "--dtype", "float32", "--temperature", "0",
           "--max-tokens", "6", "--cache-tokens", "512"]
    for q in ps:
        cmd += ["--prompt-ids", " ".join(map(str, q))]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [json.loads(x) for x in p.stdout.strip().splitlines()]
    assert len(lines) == 2
    for q, rec in zip(ps, lines):
        seq = list(q)
        for tok in rec["tokens"]:
            logits = plain.forward(cfg, tensors, seq)[-1]
            best = int(torch.argmax(logits))
            assert best == tok or float(logits[best] - logits[tok]) <= 1e-4 * float(logits.abs().max())
            seq.append(tok)
        assert len(rec["tokens"]) == 6
    a, b = tokens_for(cfg, 70, 3), tokens_for(cfg, 5, 4)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 64, 65]}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[4:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:], "want": [0, 1]}], "end": ["a"]}]
    ra, rb = plain.forward(cfg, tensors, a), plain.forward(cfg, tensors, b)
    want = {0: torch.stack([ra[0], ra[64], ra[65], rb[3]]), 1: torch.stack([ra[66], rb[4]]), 3: torch.stack([ra[68], ra[69]])}
    for dtype in DTYPES:
        out = tmp_path / f"out_{dtype}"
        p = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "128"], input="\n".join(json.dumps(x) for x in steps) + "\n", capture_output=True,
                           text=True, env=env, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [x for x in p.stdout.split("\n") if x.startswith("done")] == [f"done {i}" for i in range(4)]
        assert not (out / "2.f32").exists()
        for step, ref in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(ref.shape[0], -1).copy())
            assert rel_err(got, ref) <= (2e-4 if dtype == "float32" else 6e-2), (dtype, step)


# ---------------------------------------------------------------- kernels alone
def _ops(dtype):
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(dtype)


def _meta(ops, runs, tokens=None):
    """runs: (slot, start, n) per sequence."""
    from rbitnet_b200.engine.step import SeqChunk, build_meta
    chunks, at = [], 0
    for slot, start, n in runs:
        chunks.append(SeqChunk(slot, start, n, at))
        at += n
    toks = np.zeros(at, dtype=np.int32) if tokens is None else np.asarray(tokens, dtype=np.int32)
    return build_meta(chunks, toks, np.zeros(0, dtype=np.int32), ops.device)


class _Ctx:
    def __init__(self, ops, meta=None, state=None, cache=None):
        self.ops, self.meta, self._state, self._cache = ops, meta, state, cache
        self.pass_state = {}

    def state_view(self, entry):
        return self._state

    def cache_view(self, entry):
        return self._cache.view(0)


def _random_weights(part, g, scale=0.3):
    return {k: (torch.randn(tuple(shape), generator=g) * (scale if len(shape) > 1 else 1.0)).to(torch.bfloat16).double()
            for k, (shape, _) in part.weight_shapes().items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E", [(1, 64), (7, 100), (300, 1024), (3, 4104), (5, 7)])
def test_normed_result_added(dtype, T, E):
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(E)
    x, y = torch.randn(T, E, generator=g, dtype=torch.float64), torch.randn(T, E, generator=g, dtype=torch.float64) * 30.0
    w = torch.randn(E, generator=g, dtype=torch.float64)
    want = x + plain.rms(y, 1e-5) * w
    xd = x.float().cuda()
    rounded = ops.norm_add(xd, y.float().cuda(), w.float().cuda(), 1e-5, want_rounded=True)
    assert rel_err(xd.cpu(), want) <= 1e-6
    assert rounded.dtype == dtype and rel_err(rounded.float().cpu(), want) <= (1e-6 if dtype == torch.float32 else 5e-3)
    assert ops.norm_add(xd, y.float().cuda(), w.float().cuda(), 1e-5) is None
    got = ops.round_rows(x.float().cuda())
    assert got.dtype == dtype and rel_err(got.float().cpu(), x) <= (1e-7 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_and_token_gate(dtype):
    """Whole runs, portions and single rows; two sequences in one step; a slot whose last token is another sequence's
    counts as empty at position 0; the hash at the largest ids."""
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(1)
    V, E, buckets = 50, 24, 13
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": 40003, "mul_cur": 30011}}}
    t = {"embed": torch.randn(V, E, generator=g).to(torch.bfloat16).double(), "bigram": torch.randn(buckets + 1, E, generator=g).to(torch.bfloat16).double()}
    a = [49, 49, 0, 7, 48, 3, 3, 21, 49, 5]
    b = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    want_a, want_b = plain.embed(cfg, t, a), plain.embed(cfg, t, b)
    table, pairs = ops.prepare_embedding(t["embed"].float().cuda()), ops.prepare_embedding(t["bigram"].float().cuda())
    for cuts in ([0, 10], [0, 1, 2, 5, 9, 10], list(range(11))):
        previous = torch.full((4, 1), 33, dtype=torch.int32, device="cuda")
        outs_a, outs_b = [], []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            meta = _meta(ops, [(2, lo, hi - lo), (1, lo, hi - lo)], a[lo:hi] + b[lo:hi])
            out = ops.embed_pairs(meta, table, 1.0, pairs, (buckets, 40003, 30011), previous)
            outs_a.append(out[:hi - lo])
            outs_b.append(out[hi - lo:])
        assert rel_err(torch.cat(outs_a).cpu(), want_a) <= 1e-6 and rel_err(torch.cat(outs_b).cpu(), want_b) <= 1e-6, cuts
        assert previous.flatten().tolist() == [33, 10, 5, 33]
    rows = torch.randn(10, 6, generator=g, dtype=torch.float64) * 3
    side = torch.randn(V, 6, generator=g).to(torch.bfloat16).double()
    got = ops.token_gate(rows.float().cuda(), ops.prepare_embedding(side.float().cuda()), torch.tensor(a, dtype=torch.int32).cuda())
    assert rel_err(got.float().cpu(), plain.gelu_tanh(rows) * side[a]) <= (1e-6 if dtype == torch.float32 else 5e-3)


def _attention_case(kind, H, G, D, Dv, E, g):
    """(part, plain mixer description) of a grouped attention with this design's options."""
    from rbitnet_b200.parts.attention import Attention
    r = {"base": 300.0, "dims": D // 2 if kind != "whole" else D}
    position = {"kind": "rotary", "params": {"head_dim": D, "theta": r["base"], "pairing": "half", "rot_dim": r["dims"]}}
    if kind == "left":
        part = Attention(E, H, G, D, position=position, scale=0.3, value_dim=D, qk_norm="projection", norm_eps=1e-5,
                         head_gate=True, conv_taps=3, values="keys")
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": 0.3, "rot": r, "conv": 3}
    else:
        part = Attention(E, H, G, D, position=position, scale=0.3, value_dim=Dv, qk_norm="head_weight", norm_eps=1e-5,
                         softcap=4.0, value_mix=True)
        m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.3, "rot": r, "softcap": 4.0, "v_mix": True}
    return part, m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,H,G,D,Dv", [("left", 4, 2, 16, 16), ("left", 8, 4, 64, 64), ("left", 3, 3, 24, 24),
                                           ("capped", 4, 2, 16, 8), ("capped", 8, 2, 64, 48), ("capped", 2, 2, 40, 56),
                                           ("whole", 4, 4, 128, 128), ("capped", 16, 2, 8, 8)])
def test_prepared_attention_part(dtype, kind, H, G, D, Dv):
    """Grouped attention behind the kernel that prepares q, k and v, over the paged cache: whole, in portions across a
    page border and shorter than the taps, and token by token; two sequences in one step; head sizes that the
    tensor-core kernels take and refuse; mixed values against a second layer's own."""
    from rbitnet_b200.cache import SequenceCache
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(H * 100 + D)
    E, T = 64, 90
    part, m = _attention_case(kind, H, G, D, Dv, E, g)
    w = _random_weights(part, g, 0.4)
    if "vmix" in w:
        w["vmix"] = torch.tensor(0.35, dtype=torch.float64)
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    ha, hb = (torch.randn(T, E, generator=g).to(torch.bfloat16).double() for _ in range(2))
    if kind == "left":
        want = [plain.conv_attention(h, m, w, 1e-5) for h in (ha, hb)]
    else:
        # the layer mixes its values with those a first layer made: that layer's projections are given
        first = torch.randn(2 * T, G * Dv + 5, generator=g).float().cuda()
        want = []
        for i, h in enumerate((ha, hb)):
            shared = {"v_first": first[i * T:(i + 1) * T, 5:].double().cpu().view(T, G, Dv)}
            want.append(plain.attention(h, m, w, 1e-5, shared))
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    need = part.state_need()
    for cuts in ([0, T], [0, 1, 2, 3, 5, 63, 64, 66, T], list(range(T + 1))):
        cache = SequenceCache({0: part.cache_need()}, {}, {}, 64 * 8, 256, dtype, ops.device)
        slots = [cache.alloc(), cache.alloc(), cache.alloc()]
        state = {k: torch.full((4, *n.shape), 9.0, device="cuda") for k, n in need.items()} if need else None
        if state:
            for s in state.values():
                s[slots[1]].zero_(), s[slots[2]].zero_()
        outs = [[], []]
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            for s in slots[1:]:
                cache.reserve(s, hi - lo)
            cache.upload_tables()
            meta = _meta(ops, [(slots[1], lo, hi - lo), (slots[2], lo, hi - lo)])
            ctx = _Ctx(ops, meta, state=state, cache=cache)
            if kind != "left":
                rows = torch.cat([first[lo:hi], first[T + lo:T + hi]]).contiguous()
                ctx.pass_state["value_mix_first"] = (rows, 5, G * Dv)
            out = part.forward(ctx, torch.cat([ha[lo:hi], hb[lo:hi]]).to(dtype).cuda(), 0)
            outs[0].append(out[:hi - lo])
            outs[1].append(out[hi - lo:])
            for s in slots[1:]:
                cache.advance(s, hi - lo)
        for i in range(2):
            assert rel_err(torch.cat(outs[i]).cpu(), want[i]) <= tol, (cuts, i)
    ops.check_errors()


@pytest.mark.parametrize("H,D,Dv,dims", [(2, 16, 24, 16), (1, 40, 8, 20), (3, 8, 12, 4), (4, 128, 64, 64), (2, 100, 33, 2),
                                         (6, 32, 32, 32), (2, 8, 130, 8)])
@pytest.mark.parametrize("chunks", [True, False])
def test_retention_part(H, D, Dv, dims, chunks):
    """Whole runs, portions and single tokens through the memory; decays of one (nothing is forgotten), near one and of
    one half; two sequences in one step with the neighbouring slots untouched; runs of several tokens in chunks and
    token by token."""
    from rbitnet_b200.parts.retention import Retention
    ops = _ops(torch.float32)
    ops.gla_in_chunks = chunks
    g = torch.Generator().manual_seed(H * 1000 + D)
    E, T = 32, 100
    decay = ([1.0, 0.999, 0.5, 0.9, 0.97, 0.75] * 2)[:H]
    r = {"base": 200.0, "dims": dims}
    part = Retention(E, H, D, Dv, decay, 1e-5, position={"kind": "rotary", "params": {
        "head_dim": D, "theta": 200.0, "pairing": "half", "rot_dim": dims}})
    w = _random_weights(part, g, 0.3)
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    ha, hb = (torch.randn(T, E, generator=g, dtype=torch.float64) for _ in range(2))
    m = {"heads": H, "dim": D, "vdim": Dv, "decay": decay, "rot": r}
    want_a, want_b = plain.retention(ha, m, w, 1e-5), plain.retention(hb, m, w, 1e-5)
    for cuts in ([0, T], [0, 1, 2, 20, 36, 37, T], list(range(T + 1)), [0, 16, 17, 97, T]):
        state = {k: torch.zeros((4, *n.shape), device="cuda") for k, n in part.state_need().items()}
        outs_a, outs_b = [], []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ctx = _Ctx(ops, _meta(ops, [(1, a, b - a), (2, a, b - a)]), state=state)
            out = part.forward(ctx, torch.cat([ha[a:b], hb[a:b]]).float().cuda(), 0, scale_result=0.5)
            outs_a.append(out[:b - a])
            outs_b.append(out[b - a:])
        assert rel_err(torch.cat(outs_a).cpu(), 0.5 * want_a) <= 2e-4 and rel_err(torch.cat(outs_b).cpu(), 0.5 * want_b) <= 2e-4, cuts
        assert float(state["S"][0].abs().max()) == 0.0 and float(state["S"][3].abs().max()) == 0.0
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,Dv,C", [(4, 16, 8, 8, 24), (2, 24, 4, 40, 12), (8, 64, 16, 64, 80), (4, 32, 32, 32, 96),
                                        (1, 8, 2, 8, 200), (2, 64, 64, 16, 64), (16, 16, 16, 32, 240)])
def test_latent_attention_with_a_turned_key_part(dtype, H, D, R, Dv, C):
    """Attention through latents with a shared turned key part and sinks, over the paged cache: whole, in portions
    across a page border, and token by token; cache rows of sizes that the tensor-core attention kernels take and
    refuse."""
    from rbitnet_b200.cache import SequenceCache
    from rbitnet_b200.parts.latent import LatentAttention
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(H * 100 + D)
    E, T = 64, 90
    part = LatentAttention(E, H, D, Dv, 0, C, scale=0.3, norm_eps=1e-5, rot_dim=R, sinks=True, position={
        "kind": "rotary", "params": {"head_dim": R, "theta": 50.0, "pairing": "interleaved", "rot_dim": R}})
    w = _random_weights(part, g, 0.4)
    w["sink"] = w["sink"] * 2.0
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": Dv, "kv_rank": C, "scale": 0.3, "rot": {"base": 50.0, "dims": R}}
    want = plain.latent_attention(h, m, w, 1e-5)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    for cuts in ([0, T], [0, 1, 2, 63, 64, 66, T], list(range(T + 1))):
        cache = SequenceCache({0: part.cache_need()}, {}, {}, 64 * 4, 256, dtype, ops.device)
        cache.alloc()
        slot = cache.alloc()
        outs = []
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            cache.reserve(slot, hi - lo)
            cache.upload_tables()
            ctx = _Ctx(ops, _meta(ops, [(slot, lo, hi - lo)]), cache=cache)
            outs.append(part.forward(ctx, h[lo:hi].to(dtype).cuda(), 0))
            cache.advance(slot, hi - lo)
        assert rel_err(torch.cat(outs).cpu(), want) <= tol, cuts
    ops.check_errors()


@pytest.mark.parametrize("D", [64, 128, 112, 32])
def test_sinks_and_soft_cap_in_the_split_decode(D):
    """One token per sequence over 900 and 70 cached positions: the keys are split over several CTAs and warps, and
    the sink must count once in all of them together.  Against the float32 kernel on the same rounded inputs."""
    from rbitnet_b200.cache import SequenceCache
    from rbitnet_b200.parts.base import CacheNeed
    g = torch.Generator().manual_seed(D)
    H, G, lengths = 8, 2, (900, 70, 1)
    results = {}
    for dtype in (torch.float32, torch.bfloat16):
        ops = _ops(dtype)
        cache = SequenceCache({0: CacheNeed(G, D)}, {}, {}, 64 * 20, 1024, dtype, ops.device)
        slots = [cache.alloc() for _ in lengths]
        for s, n in zip(slots, lengths):
            cache.reserve(s, n)
        cache.upload_tables()
        view = cache.view(0)
        gen = torch.Generator().manual_seed(D + 1)
        view.k.copy_((torch.randn(view.k.shape, generator=gen) * 0.5).to(dtype))
        view.v.copy_(torch.randn(view.v.shape, generator=gen).to(dtype))
        q = (torch.randn(len(lengths), H, D, generator=gen) * 0.5).to(dtype).cuda()
        sinks = (torch.randn(H, generator=gen) * 3.0 + 3.0).float().cuda()
        meta = _meta(ops, [(s, n - 1, 1) for s, n in zip(slots, lengths)])
        results[dtype] = {
            "both": ops.attention(q, meta, view, H, 0.4, None, sinks=sinks, softcap=3.0).float().cpu(),
            "sinks": ops.attention(q, meta, view, H, 0.4, None, sinks=sinks).float().cpu(),
            "none": ops.attention(q, meta, view, H, 0.4, None).float().cpu()}
        ops.check_errors()
    for key in ("both", "sinks", "none"):
        assert rel_err(results[torch.bfloat16][key], results[torch.float32][key].double()) <= 2e-2, key
    assert rel_err(results[torch.float32]["sinks"], results[torch.float32]["none"].double()) > 0.05
