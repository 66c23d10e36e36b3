"""The Gozotar decoder through the package's host logic (configuration, parts, cache and state manager, step
function, scheduler, generation, trace replay, command line) on the CPU stand-in of the kernel layer, against the
plain implementation."""
import json

import pytest
import torch

import plain_gozotar as plain
import gozotar_cases as cases
from safuvik_tiny import write_model, tokens_for
from gozotar_tiny import CONFIGS, make_tensors, spec_of
from torch_ops import TorchOps
from rbitnet_b200.config import config_from_dict, ConfigError, load_config
from rbitnet_b200.engine import Engine

# float32 against float64 on weights that are scaled up so that faults show
TOL = 2e-4
BAND = cases.Band(TOL)


def make_engine(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
    return Engine(config_from_dict(cfg), dict(tensors), dtype="float32", ops=TorchOps(torch.float32),
                  max_tokens=max_tokens, max_seq=1024, **kw)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole(name):
    cases.whole(make_engine, name, BAND, n=70)


@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_against_decoding(name):
    cases.prefill_against_decoding(make_engine, name, BAND, n=30, prompt=13)


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_configurations(seed):
    cases.random_configuration(make_engine, seed, BAND, n=100)


def test_portions():
    cases.portions(make_engine, "A", BAND, n=132)


def test_batches():
    cases.batches_against_alone(make_engine, "B", BAND, lengths=(1, 2, 67, 9), decode=6)


def test_slots_and_pages_used_again():
    cases.slots_and_pages_used_again(make_engine, "A", BAND)


def test_first_tokens():
    cases.first_tokens(make_engine, "D", BAND)


def test_far_token_through_the_memory():
    cases.far_token_moves_the_logits(make_engine, cases.retention_only(), TOL, n=110)


@pytest.mark.parametrize("kind", ["latent", "attention", "left"])
def test_one_far_key(kind):
    cases.one_far_key_stands_out(make_engine, kind, TOL, n=150, far=3, cuts=[100, 148, 149])


def test_sink():
    cases.sink_counts(make_engine, TOL)


def test_greedy_generation():
    cases.greedy_generation(make_engine, "B", prompts=(5, 1, 12), new=8)


# ---- every mechanism of the plain implementation against an independent statement of it
def test_plain_rotation_layouts_and_stretched_frequencies():
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    r = {"base": 100.0, "dims": 4}
    half, inter = plain.rotate(x, r, "half"), plain.rotate(x, r, "interleaved")
    f = [1.0, 100.0 ** -0.5]
    for t in range(5):
        for i in range(2):
            c, s = torch.cos(torch.tensor(t * f[i])), torch.sin(torch.tensor(t * f[i]))
            assert torch.allclose(half[t, :, i], x[t, :, i] * c - x[t, :, i + 2] * s)
            assert torch.allclose(half[t, :, i + 2], x[t, :, i + 2] * c + x[t, :, i] * s)
            assert torch.allclose(inter[t, :, 2 * i], x[t, :, 2 * i] * c - x[t, :, 2 * i + 1] * s)
    assert torch.equal(half[..., 4:], x[..., 4:]) and torch.equal(half[0], x[0])
    # wavelengths 2 pi, 2 pi 10, 2 pi 100, 2 pi 1000 against original/high = 16 and original/low = 64
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    got = plain.frequencies({"base": 10000.0, "dims": 8, "scaling": sc}, torch.float64)
    s = (64 / (2 * torch.pi * 10) - 1.0) / 3.0
    want = torch.tensor([1.0, 0.1 * ((1 - s) / 8.0 + s), 0.01 / 8.0, 0.001 / 8.0], dtype=torch.float64)
    assert torch.allclose(got, want)


def test_plain_attention_pieces():
    torch.manual_seed(0)
    q, k, v = torch.randn(4, 2, 3).double(), torch.randn(4, 1, 3).double(), torch.randn(4, 1, 5).double()
    sink = torch.tensor([0.3, -1.0]).double()
    out = plain.causal_softmax_attention(q, k, v, 0.7, softcap=2.0, sink=sink)
    for t in range(4):
        for h in range(2):
            s = torch.stack([2.0 * torch.tanh((q[t, h] @ k[j, 0]) * 0.7 / 2.0) for j in range(t + 1)])
            w = torch.exp(s) / (torch.exp(s).sum() + torch.exp(sink[h]))
            assert torch.allclose(out[t, h], (w[:, None] * v[:t + 1, 0]).sum(0))
    u, taps = torch.randn(6, 3).double(), torch.randn(3, 3).double()
    y = plain.short_conv(u, taps)
    assert torch.allclose(y[0], taps[:, 2] * u[0]) and torch.allclose(y[4], taps[:, 0] * u[2] + taps[:, 1] * u[3] + taps[:, 2] * u[4])


def test_plain_embedding_and_norms():
    cfg = {"embedding": {"bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 2}}}
    t = {"embed": torch.arange(12.0).view(6, 2), "bigram": 100.0 * torch.arange(12.0).view(6, 2)}
    x = plain.embed(cfg, t, [4, 1, 5])
    assert torch.equal(x[0], t["embed"][4] + t["bigram"][5])
    assert torch.equal(x[1], t["embed"][1] + t["bigram"][(4 * 3 + 1 * 2) % 5])
    assert torch.equal(x[2], t["embed"][5] + t["bigram"][(1 * 3 + 5 * 2) % 5])
    y = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain.norm_one_plus(y, torch.tensor([0.0, 1.0]), 0.0), torch.tensor([[3.0, 8.0]]) / (12.5 ** 0.5))


def test_value_mixing_takes_the_first_such_layer():
    """The second and third mixing layers mix with the FIRST one's values, not with the layer before them; a layer
    without the option between them neither takes part nor resets it."""
    cfg = CONFIGS["C"]
    tensors = make_tensors(cfg, 3)
    toks = tokens_for(cfg, 20, 1)
    ref = plain.forward(cfg, tensors, toks)
    other = dict(tensors)
    other["l0.mix.vmix"] = torch.tensor(0.9)                     # the first layer's own weight is not used
    assert torch.equal(plain.forward(cfg, other, toks), ref)
    other["l5.mix.vmix"] = torch.tensor(0.9)
    assert not torch.allclose(plain.forward(cfg, other, toks), ref)
    eng = make_engine(cfg, other)
    assert cases.rel_err(cases.run_cut(eng, toks, [7]), plain.forward(cfg, other, toks)) <= TOL


def test_one_tap_and_tensors_a_model_does_not_use(tmp_path):
    """A convolution of one tap only scales the channels and keeps no ring; a folder may hold a mixing weight for a
    layer that mixes nothing, norms of a feed-forward that a layer does not have, and embeddings the configuration
    does not ask for."""
    from gozotar_tiny import model, parallel_layer, attention_layer, rot
    cfg = model(40, 32, [parallel_layer((2, 1, 8, 0.3, 1, rot(100.0, 8)), (2, 16, 8, [0.9, 0.99], rot(1000.0, 16)), 0.5, 1.0),
                         attention_layer(2, 1, 8, 4, 0.3, rot(50.0, 4), None, False, ff=None)])
    tensors = make_tensors(cfg, 3)
    assert tensors["l0.mix.left.q.conv"].shape == (16, 1)
    toks = tokens_for(cfg, 20, 1)
    eng = make_engine(cfg, tensors)
    _, _, states = eng.model.cache_plan()
    assert set(states[0]) == {"right.S"}
    assert cases.rel_err(cases.run_cut(eng, toks, [5, 6]), plain.forward(cfg, tensors, toks)) <= TOL
    extra = dict(tensors, **{"l1.mix.vmix": torch.tensor(0.5), "l1.norm2": torch.zeros(32), "l1.ls2": torch.ones(32),
                             "bigram": torch.zeros(8, 32), "side.embed": torch.zeros(40, 6), "l0.side.gate": torch.zeros(3, 32)})
    folder = write_model(tmp_path / "m", cfg, extra)
    eng = Engine.load_path(folder, dtype="float32", ops=TorchOps(torch.float32), max_tokens=256, verbose=False)
    assert cases.rel_err(cases.run_cut(eng, toks, []), plain.forward(cfg, tensors, toks)) <= TOL
    with pytest.raises(Exception):
        Engine.load_path(write_model(tmp_path / "n", cfg, dict(tensors, other=torch.zeros(3))), dtype="float32",
                         ops=TorchOps(torch.float32), max_tokens=256, verbose=False)


def test_sizes_that_only_a_tensor_gives(tmp_path):
    """config.json may leave out the sizes that a tensor's shape gives; what nothing gives is an error."""
    cfg = CONFIGS["A"]
    tensors = make_tensors(cfg, 4)
    bare = json.loads(json.dumps(cfg))
    bare["layers"][0]["mlp"].pop("ff")
    bare["layers"][0]["mixer"]["left"].pop("conv")
    bare["layers"][3]["mixer"].pop("kv_rank")
    bare["embedding"]["bigram"].pop("buckets")
    bare["token_side"]["dim"] = None
    toks = tokens_for(cfg, 12, 2)
    eng = Engine.load_path(write_model(tmp_path / "m", bare, tensors), dtype="float32", ops=TorchOps(torch.float32),
                           max_tokens=256, verbose=False)
    assert cases.rel_err(cases.run_cut(eng, toks, [7]), plain.forward(cfg, tensors, toks)) <= TOL
    with pytest.raises(ConfigError):
        spec_of(bare)


def test_state_and_cache_of_a_model():
    eng = make_engine(CONFIGS["A"], make_tensors(CONFIGS["A"], 1))
    caches, _, states = eng.model.cache_plan()
    assert set(caches) == {0, 1, 2, 3}
    assert set(states[0]) == {"left.tail", "right.S"} and ("model", "previous_token") in states
    assert states[0]["left.tail"].shape == (3, (4 + 2) * 16) and states[0]["right.S"].shape == (2, 24, 16)
    assert caches[3].streams == ((1, 24),) and caches[1].head_dim == 16
    eng = make_engine(CONFIGS["B"], make_tensors(CONFIGS["B"], 1))
    _, _, states = eng.model.cache_plan()
    assert ("model", "previous_token") not in states


def test_residual_after_every_layer():
    """``ctx.layer_outputs`` receives the residual stream after every layer."""
    import numpy as np
    from rbitnet_b200.engine.step import build_meta, SeqChunk, StepContext
    cfg = CONFIGS["A"]
    tensors = make_tensors(cfg, 2)
    toks = tokens_for(cfg, 19, 3)
    eng = make_engine(cfg, tensors)
    slot = eng.new_sequence()
    eng.cache.reserve(slot, len(toks))
    eng.cache.upload_tables()
    meta = build_meta([SeqChunk(slot, 0, len(toks), 0)], np.asarray(toks, dtype=np.int32), np.arange(len(toks), dtype=np.int32),
                      eng.ops.device)
    ctx = StepContext(eng.ops, meta, eng.cache)
    ctx.layer_outputs = []
    eng.model.forward(ctx)
    want = []
    plain.forward(cfg, tensors, toks, torch.float64, want)
    assert len(ctx.layer_outputs) == len(want) == 4
    for got, ref in zip(ctx.layer_outputs, want):
        assert cases.rel_err(got, ref) <= TOL


def test_config_is_read_and_checked(tmp_path):
    cfg = CONFIGS["A"]
    tensors = make_tensors(cfg, 1)
    folder = write_model(tmp_path / "m", cfg, tensors)
    assert load_config(folder).token_side == {"dim": 6}
    shapes = spec_of(cfg).expected_shapes()
    assert shapes["bigram"] == (54, 64) and shapes["side.embed"] == (96, 4 * 6) and shapes["l2.side.proj"] == (64, 6)
    assert shapes["l0.mix.left.q.conv"] == (64, 3) and shapes["l0.mix.left.k.norm"] == (32,) and shapes["l0.mix.left.g"] == (4, 64)
    assert "l0.mix.left.v" not in shapes and shapes["l0.mix.right.g"] == (48, 64) and shapes["l0.ls1"] == (64,)
    assert shapes["l1.mix.q.norm"] == (16,) and shapes["l1.mix.vmix"] == () and shapes["l1.mix.v"] == (16, 64)
    assert shapes["l3.mix.q"] == (2 * 12, 64) and shapes["l3.mix.dkv"] == (24, 64) and shapes["l3.mix.sink"] == (2,)
    assert "l3.norm2" not in shapes and "l3.mlp.gate" not in shapes and shapes["final.norm"] == (64,) and shapes["head"] == (96, 64)
    for path, value in ((("layers", 1, "type"), "other"), (("layers", 3, "mixer", "kv_rank"), 0), (("norm", "eps"), 0),
                        (("layers", 0, "mixer", "right", "decay"), [0.5]), (("layers", 0, "mixer", "right", "decay"), [0.5, 1.5]),
                        (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 1, "mixer", "rot", "dims"), 7),
                        (("layers", 2, "mixer", "vdim"), 16), (("layers", 0, "mlp", "kind"), "moe"),
                        (("layers", 3, "mixer", "rot", "dims"), 2), (("embedding", "bigram", "buckets"), 0),
                        (("token_side", "dim"), 0), (("layers", 0, "mixer", "left", "vdim"), 8),
                        (("layers", 1, "mixer", "rot", "scaling"), {"factor": 2.0})):
        bad = json.loads(json.dumps(cfg))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_engine_from_a_model_folder_and_trace_replay(tmp_path):
    """The folder's config.json chooses the model class; trace replay drives the same engine."""
    from rbitnet_b200 import replay
    import io
    cfg = CONFIGS["D"]
    tensors = make_tensors(cfg, 5)
    folder = write_model(tmp_path / "m", cfg, tensors, store=torch.bfloat16)
    a, b = tokens_for(cfg, 9, 1), tokens_for(cfg, 4, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:6], "want": [0, 5]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[6:7], "want": []}, {"id": "b", "tokens": b[3:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[7:], "want": [1]}], "end": ["a"]}]
    out = io.StringIO()
    rc = replay.main(["--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                     stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out, ops=TorchOps(torch.float32))
    assert rc == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    import numpy as np
    ra, rb = plain.forward(cfg, tensors, a), plain.forward(cfg, tensors, b)
    got0 = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(3, -1))
    got1 = torch.from_numpy(np.fromfile(tmp_path / "o" / "1.f32", dtype="<f4").reshape(1, -1))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(1, -1))
    assert cases.rel_err(got0, torch.stack([ra[0], ra[5], rb[2]])) <= TOL
    assert cases.rel_err(got1, rb[3:4]) <= TOL and cases.rel_err(got2, ra[8:9]) <= TOL
