"""The Nifarax decoder on the GPU: the package's kernels against the plain implementation (whole models in both
dtypes, the same cases as on the CPU), and each new kernel alone against the plain functions."""
import numpy as np
import pytest
import torch

import plain_nifarax as plain
import nifarax_cases as cases
from safuvik_tiny import tokens_for, rel_err
from nifarax_tiny import CONFIGS, make_tensors
from rbitnet_b200.config import config_from_dict

pytestmark = pytest.mark.gpu

# Fractions of the largest reference value.  float32: the weights are scaled up so that faults show, which amplifies
# rounding.  bfloat16: operands of the products, the cached latents, the attention's P and the experts' inner rows are
# rounded to 8 bits.
TOL = {"float32": 2e-4, "bfloat16": 6e-2}
# whole models in bfloat16, matrices spread by 4: single positions where a router's choice fell the other way may lie
# outside the band (one in ten), while the median stays within a third of it
BAND = {"float32": cases.Band(2e-4), "bfloat16": cases.Band(6e-2, spikes=0.1, spread=4.0)}
DTYPES = ["float32", "bfloat16"]


def engine_maker(dtype):
    from rbitnet_b200.engine import Engine

    def make(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
        return Engine(config_from_dict(cfg), dict(tensors), dtype=dtype, max_tokens=max_tokens, max_seq=1024,
                      use_graphs=graphs, **kw)
    return make


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole(name, dtype):
    cases.whole(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_prefill_against_decoding(name, dtype):
    cases.prefill_against_decoding(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_portions(name, dtype):
    cases.portions(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_batches(name, dtype):
    cases.batches_against_alone(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_slots_and_pages_used_again(name, dtype):
    cases.slots_and_pages_used_again(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "E"])
def test_long_decoding(name, dtype):
    cases.long_decoding(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens(name, dtype):
    cases.first_tokens(engine_maker(dtype), name, BAND[dtype])


@pytest.mark.parametrize("taps", [1, 3])
def test_far_token_through_the_memory(taps):
    # float32 only: what the first token of 180 leaves in the last logits is of the size of bfloat16's rounding
    cases.far_token_moves_the_logits(engine_maker("float32"), cases.gla_only(taps), TOL["float32"], least=10.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kv_rank", [16, 64])
@pytest.mark.parametrize("n,far,cuts", [(300, 2, []), (300, 63, [250] + list(range(290, 300))), (200, 64, list(range(1, 200))),
                                        (700, 0, [64, 128, 699]), (130, 127, [129])])
def test_one_far_key(n, far, cuts, kv_rank, dtype):
    cases.one_far_key_stands_out(engine_maker(dtype), TOL[dtype], n, far, cuts, last_only=dtype == "bfloat16", kv_rank=kv_rank)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_through_captured_steps(name):
    cases.greedy_generation(engine_maker("float32"), name)


def test_captured_step_in_bfloat16():
    """The captured decode step (padding rows, state saved around the trial run) against the plain model."""
    from rbitnet_b200.engine.step import StepEntry
    cfg = CONFIGS["A"]
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


# ---------------------------------------------------------------- kernels alone
def _ops(dtype):
    from rbitnet_b200.kernels.ops import CudaOps
    return CudaOps(dtype)


def _meta(ops, runs):
    """runs: (slot, start, n) per sequence."""
    from rbitnet_b200.engine.step import SeqChunk, build_meta
    chunks, at = [], 0
    for slot, start, n in runs:
        chunks.append(SeqChunk(slot, start, n, at))
        at += n
    return build_meta(chunks, np.zeros(at, dtype=np.int32), np.zeros(0, dtype=np.int32), ops.device)


class _Ctx:
    def __init__(self, ops, meta=None, state=None, cache=None):
        self.ops, self.meta, self._state, self._cache = ops, meta, state, cache

    def state_view(self, entry):
        return self._state

    def cache_view(self, entry):
        return self._cache.view(0)


def _random_weights(part, g, scale=0.3):
    return {k: (torch.randn(*shape, generator=g) * (scale if len(shape) > 1 else 1.0)).to(torch.bfloat16).double()
            for k, (shape, _) in part.weight_shapes().items()}


@pytest.mark.parametrize("T,E,groups", [(1, 64, 2), (7, 100, 5), (300, 1024, 1), (3, 4104, 3), (5, 7, 7), (40, 96, 96)])
def test_norm_in_groups(T, E, groups):
    """Parts of very different sizes in one row: a group's statistics are its own."""
    ops = _ops(torch.float32)
    g = torch.Generator().manual_seed(E)
    x = torch.randn(T, E, generator=g, dtype=torch.float64)
    x = x * (10.0 ** torch.arange(groups).repeat_interleave(E // groups).double() ** 0.5)
    w = torch.randn(E, generator=g, dtype=torch.float64)
    got = ops.rmsnorm_grouped(x.float().cuda(), w.float().cuda(), groups, 1e-5, out_dtype=torch.float32)
    assert rel_err(got.cpu(), plain.group_norm(x, w, groups, 1e-5)) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,K,T", [(64, 3, 50), (100, 1, 50), (33, 4, 50), (512, 2, 50), (8, 7, 50), (256, 4, 601)])
def test_input_filter(dtype, C, K, T):
    """Whole runs, portions shorter than the taps and single rows through the ring; two sequences in one step; a slot
    whose ring holds another sequence's rows counts as empty at position 0.  Widths that allow 16 bytes a load and
    widths that do not; more taps than the kernel of wide loads keeps; steps of so many rows that a block takes several."""
    from rbitnet_b200.parts.sublayer import CausalTapsFilter
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(C + K)
    part = CausalTapsFilter(C, K)
    taps = torch.randn(C, K, generator=g, dtype=torch.float64)
    part.bind({"taps": taps.float().cuda()}, ops)
    ha = torch.randn(T, C, generator=g).to(torch.bfloat16).double()
    hb = torch.randn(T, C, generator=g).to(torch.bfloat16).double()
    want_a, want_b = plain.canon(ha, taps), plain.canon(hb, taps)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    need = part.state_need()
    for cuts in ([0, T], [0, 1, 2, 3, 4, 6, 9, 30, T], list(range(T + 1)) if T <= 100 else [0, 299, T]):
        ring = torch.full((4, *need.shape), 7.0, device="cuda") if need is not None else None      # stale rows
        outs_a, outs_b = [], []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ctx = _Ctx(ops, _meta(ops, [(2, a, b - a), (1, a, b - a)]))
            out = part.forward(ctx, torch.cat([ha[a:b], hb[a:b]]).to(dtype).cuda(), ring)
            outs_a.append(out[:b - a])
            outs_b.append(out[b - a:])
        assert rel_err(torch.cat(outs_a).cpu(), want_a) <= tol and rel_err(torch.cat(outs_b).cpu(), want_b) <= tol, cuts
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,groups,K,with_add", [(64, 2, 3, True), (100, 5, 4, False), (96, 1, 1, True), (2048, 2, 4, True),
                                                 (72, 9, 6, True), (70, 5, 3, True)])
def test_rows_between_two_sublayers_in_one_kernel(dtype, E, groups, K, with_add):
    """A decode step's gated addition, norm in groups and filter as one kernel against the three kernels: the same
    residual stream, and normed rows, filtered rows and ring that agree to rounding, at positions before and after the ring is full and in a slot
    whose ring holds stale rows."""
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(E + K)
    T = 5
    w = torch.randn(E, generator=g).cuda()
    taps = torch.randn(E, K, generator=g).cuda()
    bias = torch.randn(E, generator=g).cuda()
    ring_a = torch.randn(8, K, E, generator=g).cuda() if K > 1 else None
    ring_b = ring_a.clone() if K > 1 else None
    x_a = torch.randn(T, E, generator=g).cuda()
    x_b = x_a.clone()
    from rbitnet_b200.engine.step import SeqChunk, build_meta
    for pos in (0, 1, 2, 7, 100):
        meta = build_meta([SeqChunk(slot, pos, 1, i) for i, slot in enumerate((3, 0, 5, 1, 6))], np.zeros(T, dtype=np.int32),
                          np.zeros(0, dtype=np.int32), ops.device)
        y = torch.randn(T, E, generator=g).cuda()
        z = torch.randn(T, E, generator=g).cuda()
        ops.fuse_norm_filter = True
        got = ops.norm_filter_rows(x_a, w, groups, 1e-5, taps, ring_a, meta, add=(y, z, bias) if with_add else None)
        if (E // groups) % 4:
            assert got is None                       # parts that do not allow 16 bytes a load: the three kernels
            return
        assert got is not None
        if with_add:
            ops.gated_add(x_b, y, z, bias)
        h = ops.rmsnorm_grouped(x_b, w, groups, 1e-5)
        hf = ops.input_filter(h, taps, ring_b, meta)
        tol = 1e-6 if dtype == torch.float32 else 1e-2        # (the norm alone adds its squares up in another order)
        assert torch.equal(x_a, x_b)
        assert rel_err(got[0].float().cpu(), h.double().cpu()) <= tol and rel_err(got[1].float().cpu(), hf.double().cpu()) <= tol
        assert K == 1 or rel_err(ring_a.cpu(), ring_b.double().cpu()) <= tol
    ops.check_errors()


def test_gated_add_and_softcap():
    ops = _ops(torch.float32)
    g = torch.Generator().manual_seed(3)
    T, E = 37, 100
    x, y, z = (torch.randn(T, E, generator=g, dtype=torch.float64) * 3 for _ in range(3))
    b = torch.randn(E, generator=g, dtype=torch.float64) * 4
    got = ops.gated_add(x.float().cuda(), y.float().cuda(), z.float().cuda(), b.float().cuda())
    assert rel_err(got.cpu(), x + y * torch.sigmoid(z + b)) <= 1e-6
    v = torch.randn(T, E, generator=g, dtype=torch.float64) * 40
    assert rel_err(ops.softcap(v.float().cuda(), 12.5).cpu(), 12.5 * torch.tanh(v / 12.5)) <= 1e-6


@pytest.mark.parametrize("H,D,Dv,R,tau", [(2, 16, 24, 8, 8.0), (1, 40, 8, 4, 1.0), (3, 8, 12, 5, 2.0), (4, 128, 64, 16, 16.0),
                                          (2, 100, 33, 3, 4.0), (1, 300, 20, 7, 64.0), (2, 8, 130, 2, 16.0), (2, 512, 8, 9, 3.0),
                                          (2, 100, 36, 3, 0.5), (1, 64, 20, 4, 0.25)])
@pytest.mark.parametrize("chunks", [True, False])
def test_gated_linear_attention_kernels(H, D, Dv, R, tau, chunks):
    """Whole runs, portions and single tokens through the memory; key sizes that one to thirty-two lanes hold; decays
    near one, so that the memory of the first tokens is still there at the end, and decays near zero in some channels
    (a small tau: a channel that loses everything within a few tokens of a chunk); two sequences in one step with the
    neighbouring slots untouched.  Runs of several tokens in chunks of 32 (a run of 100 tokens ends inside its fourth
    chunk; value sizes that fill a tile of columns and that do not) and token by token."""
    from rbitnet_b200.parts.gla import GatedLinearAttention
    ops = _ops(torch.float32)
    ops.gla_in_chunks = chunks
    g = torch.Generator().manual_seed(H * 1000 + D)
    E, T = 32, 100
    part = GatedLinearAttention(E, H, D, Dv, R, tau, norm_eps=1e-5)
    w = {k: torch.randn(*shape, generator=g, dtype=torch.float64) * (0.3 if len(shape) > 1 else 1.0)
         for k, (shape, _) in part.weight_shapes().items()}
    w["a2.b"] = w["a2.b"] * 3.0 + 3.0
    w["a2"] = w["a2"] * 5.0
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    ha, hb = (torch.randn(T, E, generator=g, dtype=torch.float64) for _ in range(2))
    m = {"heads": H, "dim": D, "vdim": Dv, "tau": tau}
    want_a, want_b = plain.gla_mixer(ha, m, w, 1e-5), plain.gla_mixer(hb, m, w, 1e-5)
    for cuts in ([0, T], [0, 1, 2, 20, 36, 37, T], list(range(T + 1)), [0, 16, 17, 97, T]):
        state = {k: torch.zeros((4, *n.shape), device="cuda") for k, n in part.state_need().items()}
        outs_a, outs_b = [], []
        for a, b in zip(cuts[:-1], cuts[1:]):
            ctx = _Ctx(ops, _meta(ops, [(1, a, b - a), (2, a, b - a)]), state=state)
            out = part.forward(ctx, torch.cat([ha[a:b], hb[a:b]]).float().cuda(), 0)
            outs_a.append(out[:b - a])
            outs_b.append(out[b - a:])
        assert rel_err(torch.cat(outs_a).cpu(), want_a) <= 2e-4 and rel_err(torch.cat(outs_b).cpu(), want_b) <= 2e-4, cuts
        assert float(state["S"][0].abs().max()) == 0.0 and float(state["S"][3].abs().max()) == 0.0
    ops.check_errors()


def test_the_memory_keeps_a_far_token():
    """One key channel that never decays and a first token that alone writes to it: the last token, which alone reads
    it, gets the first token's values back after 600 steps, whole and decoded."""
    from rbitnet_b200.parts.gla import GatedLinearAttention
    ops = _ops(torch.float32)
    E, H, D, Dv, T = 16, 1, 16, 8, 600
    part = GatedLinearAttention(E, H, D, Dv, 2, 1.0, norm_eps=1e-5)
    g = torch.Generator().manual_seed(9)
    w = {k: torch.randn(*shape, generator=g, dtype=torch.float64) * 0.3 for k, (shape, _) in part.weight_shapes().items()}
    w["a2"] = torch.zeros_like(w["a2"])
    w["a2.b"] = torch.full_like(w["a2.b"], -1.0)            # everything else fades fast
    w["a2.b"][5] = 40.0                                     # channel 5 stays
    w["k"][5] = 0.0
    w["k"][5, 0] = 1.0                                      # written by input channel 0 only
    w["q"][5] = 0.0
    w["q"][5, 1] = 50.0                                     # read by input channel 1 only
    h = torch.randn(T, E, generator=g, dtype=torch.float64)
    h[:, 0] = 0.0
    h[:, 1] = 0.0
    h[0, 0] = 3.0
    h[-1, 1] = 3.0
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    m = {"heads": H, "dim": D, "vdim": Dv, "tau": 1.0}
    want = plain.gla_mixer(h, m, w, 1e-5)
    h2 = h.clone()
    h2[0] = torch.randn(E, generator=g, dtype=torch.float64)
    h2[0, 1] = 0.0
    h2[0, 0] = -3.0
    want2 = plain.gla_mixer(h2, m, w, 1e-5)
    assert float((want[-1] - want2[-1]).abs().max() / want[-1].abs().max()) > 0.5
    for rows, ref in ((h, want), (h2, want2)):
        for cuts in ([0, T], [0, 500] + list(range(501, T + 1))):
            state = {k: torch.zeros((2, *n.shape), device="cuda") for k, n in part.state_need().items()}
            outs = []
            for a, b in zip(cuts[:-1], cuts[1:]):
                ctx = _Ctx(ops, _meta(ops, [(1, a, b - a)]), state=state)
                outs.append(part.forward(ctx, rows[a:b].float().cuda(), 0))
            assert rel_err(torch.cat(outs)[-1:].cpu(), ref[-1:]) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv,Rq,R", [(4, 16, 8, 24, 32), (2, 24, 40, 16, 16), (3, 24, 24, 20, 40), (4, 32, 64, 96, 64),
                                         (16, 16, 32, 64, 128), (1, 8, 8, 8, 200), (2, 64, 16, 7, 9), (2, 16, 16, 24, 320)])
def test_latent_attention_part(dtype, H, D, Dv, Rq, R):
    """Attention through latents over the paged cache: whole, in portions across a page border, and token by token;
    latents of sizes that the tensor-core attention kernels take and refuse, and one wider than any of them takes."""
    from rbitnet_b200.cache import SequenceCache
    from rbitnet_b200.parts.latent import LatentAttention
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(H * 100 + D)
    E, T = 64, 90
    scale = 0.35 if R <= 256 else 0.12        # (a wide latent's sums are large: scores that bfloat16 still resolves)
    part = LatentAttention(E, H, D, Dv, Rq, R, scale=scale, norm_eps=1e-5)
    w = _random_weights(part, g, 0.4)
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()
    m = {"heads": H, "dim": D, "vdim": Dv, "scale": scale}
    want = plain.latent_attention(h, m, w, 1e-5)
    for cuts in ([0, T], [0, 60, 64, 65, T], [0, 50] + list(range(51, T + 1))):
        cache = SequenceCache({0: part.cache_need()}, {}, {}, 64 * 4, 1024, dtype, ops.device)
        cache.alloc()
        slot = cache.alloc()
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            cache.reserve(slot, b - a)
            cache.upload_tables()
            ctx = _Ctx(ops, _meta(ops, [(slot, a, b - a)]), cache=cache)
            outs.append(part.forward(ctx, h[a:b].to(dtype).cuda(), 0))
            cache.advance(slot, b - a)
        assert rel_err(torch.cat(outs).cpu(), want) <= (2e-5 if dtype == torch.float32 else 3e-2), cuts
    ops.check_errors()


@pytest.mark.parametrize("n,top,T,K", [(16, 1, 50, 48), (5, 2, 333, 100), (3, 3, 7, 70), (60, 6, 200, 64), (2, 1, 1, 32)])
@pytest.mark.parametrize("extra", [0, 1])
def test_router_with_sigmoid_scores(n, top, T, K, extra):
    """The best ``top`` sigmoid scores and the scores themselves as weights; the rows of the matrix that are no
    outputs (a shared expert's gate) come back as plain sums."""
    ops = _ops(torch.float32)
    g = torch.Generator().manual_seed(n * 10 + top)
    h = torch.randn(T, K, generator=g).double()
    router = torch.randn(n + extra, K, generator=g).double() * 0.3
    ids, weights, gate = ops.route_scored(h.float().cuda(), router.float().cuda(), None, top, 0, 0, scoring="sigmoid",
                                          extra_rows=extra)
    s = torch.sigmoid(h @ router[:n].T)
    want = torch.topk(s, top, dim=-1)
    ids, weights = ids.cpu().long(), weights.cpu().double()
    for t in range(T):
        assert sorted(ids[t].tolist()) == sorted(want.indices[t].tolist()), t
        assert float((weights[t].sort().values - want.values[t].sort().values).abs().max()) <= 3e-6
    if extra:
        assert rel_err(gate.cpu(), h @ router[n:].T) <= 1e-5
    else:
        assert gate is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,N,K", [(1, 3, 8, 16), (8, 16, 128, 128), (16, 2, 33, 100), (17, 2, 33, 100), (5, 4, 7, 300), (300, 3, 40, 24)])
def test_a_matrix_per_head(dtype, T, H, N, K):
    """Few rows (a warp per output) and many (tiles) through the product with one matrix per head."""
    ops = _ops(dtype)
    g = torch.Generator().manual_seed(T * 10 + H)
    x = torch.randn(T, H * K, generator=g).to(torch.bfloat16).double()
    w = (torch.randn(H, N, K, generator=g) * 0.3).to(torch.bfloat16).double()
    weight = ops.prepare_per_head(w.float().cuda())
    got = ops.per_head_linear(x.to(dtype).cuda(), weight).float().cpu()
    want = torch.einsum("thk,hnk->thn", x.view(T, H, K), w).reshape(T, H * N)
    assert rel_err(got, want) <= (1e-5 if dtype == torch.float32 else 1e-2)
    ops.check_errors()


@pytest.mark.parametrize("n,top,T,K,extra", [(16, 4, 200, 64, 1), (5, 1, 64, 128, 0), (33, 8, 700, 256, 1), (6, 2, 63, 64, 1),
                                             (32, 4, 8, 256, 1), (7, 3, 1, 64, 0)])
def test_router_sums_on_the_tensor_cores(n, top, T, K, extra):
    """In bfloat16 mode a router whose float32 values are bfloat16 values has its sums (outputs and extra rows) made by
    the tensor-core product, for a decode step's few rows as for a prompt's many; the choice and the weights are those
    of the plain sums."""
    ops = _ops(torch.bfloat16)
    g = torch.Generator().manual_seed(n * 7 + top)
    h = torch.randn(T, K, generator=g).to(torch.bfloat16).double()
    router = (torch.randn(n + extra, K, generator=g) * 0.3).to(torch.bfloat16).double()
    tc = ops.prepare_router(router.float().cuda())
    assert tc is not None
    ids, weights, gate = ops.route_scored(h.to(torch.bfloat16).cuda(), router.float().cuda(), None, top, 0, 0,
                                          scoring="sigmoid", extra_rows=extra, router_tc=tc)
    s = torch.sigmoid(h @ router[:n].T)
    want = torch.topk(s, top, dim=-1)
    ids, weights = ids.cpu().long(), weights.cpu().double()
    for t in range(T):
        assert sorted(ids[t].tolist()) == sorted(want.indices[t].tolist()), t
        assert float((weights[t].sort().values - want.values[t].sort().values).abs().max()) <= 3e-6
    if extra:
        assert rel_err(gate.cpu(), h @ router[n:].T) <= 1e-5
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,F,n,top,shared", [(1, 64, 40, 6, 2, (48, 1.0)), (3, 64, 40, 6, 6, None), (70, 64, 24, 3, 1, (24, 2.5)),
                                                (300, 128, 72, 16, 4, (256, 0.7)), (45, 100, 36, 4, 2, (20, 1.0)),
                                                (2500, 64, 32, 5, 2, None), (9, 64, 44, 2, 1, (8, 1.0))])
@pytest.mark.parametrize("fused", [True, False])
def test_experts_weighted_on_their_inputs(dtype, T, E, F, n, top, shared, fused):
    """Few pairs and many, tiles of every size, experts without any token, a width and an inner size that the
    tensor-core products refuse, with and without the shared expert.  The weight multiplies what the expert reads: with
    limits that bite, that differs from weighing its result.  The activation in the grouped product's epilogue and as
    a kernel of its own."""
    from rbitnet_b200.parts.feed_forward import RoutedExperts
    if dtype == torch.float32 and not fused:
        pytest.skip("float32 has the one form")
    ops = _ops(dtype)
    ops.fuse_gated_act = fused
    g = torch.Generator().manual_seed(T + E)
    part = RoutedExperts(E, F, n, top, correction=False, activation="swish_limited", scoring="sigmoid", weight_on="input",
                         limit=0.8, shared={"inner": shared[0], "limit": shared[1]} if shared else None)
    w = {k: (torch.randn(*shape, generator=g) * 0.5).to(torch.bfloat16).double() for k, (shape, _) in part.weight_shapes().items()}
    if n > 2:
        w["router"][1] = 0.0
        w["router"][1, 0] = -1.0              # with the first input value large: an expert that nobody chooses
    part.bind({k: v.float().cuda() for k, v in w.items()}, ops)
    h = torch.randn(T, E, generator=g).to(torch.bfloat16).double()
    h[:, 0] = 6.0
    mlp = {"router": {"experts": n, "top": top}, "expert": {"ff": F, "limit": 0.8}}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    want = plain.experts_ff(h, mlp, w)
    ctx = _Ctx(ops)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(part.forward(ctx, h.to(dtype).cuda()).cpu(), want) <= tol
    x = torch.randn(T, E, generator=g).float().cuda()
    before = x.clone()
    part.forward(ctx, h.to(dtype).cuda(), accumulate_into=x)
    assert rel_err((x - before).cpu(), want) <= tol
    ops.check_errors()
