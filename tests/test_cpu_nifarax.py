"""The Nifarax decoder through the package's host logic (configuration, parts, cache and state manager, step
function, scheduler, generation, trace replay, command line) on the CPU stand-in of the kernel layer, against the
plain implementation."""
import json

import pytest
import torch

import plain_nifarax as plain
import nifarax_cases as cases
from safuvik_tiny import write_model, tokens_for
from nifarax_tiny import CONFIGS, make_tensors, spec_of
from torch_ops import TorchOps
from rbitnet_b200.config import config_from_dict, ConfigError, load_config
from rbitnet_b200.engine import Engine

# float32 against float64 on weights that are scaled up so that faults show
TOL = 2e-4
BAND = cases.Band(TOL)


def make_engine(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
    return Engine(config_from_dict(cfg), dict(tensors), dtype="float32", ops=TorchOps(torch.float32),
                  max_tokens=max_tokens, max_seq=1024, **kw)


@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_whole(name):
    cases.whole(make_engine, name, BAND, n=70)


@pytest.mark.parametrize("name", ["A", "C"])
def test_prefill_against_decoding(name):
    cases.prefill_against_decoding(make_engine, name, BAND, n=30, prompt=13)


def test_portions():
    cases.portions(make_engine, "A", BAND, n=132)


def test_batches():
    cases.batches_against_alone(make_engine, "C", BAND, lengths=(1, 2, 67, 9), decode=6)


def test_slots_and_pages_used_again():
    cases.slots_and_pages_used_again(make_engine, "A", BAND)


def test_first_tokens():
    cases.first_tokens(make_engine, "C", BAND)


def test_far_token_through_the_memory():
    cases.far_token_moves_the_logits(make_engine, cases.gla_only(), TOL, n=110)


def test_one_far_key():
    cases.one_far_key_stands_out(make_engine, TOL, n=150, far=3, cuts=[100, 148, 149])


def test_greedy_generation():
    cases.greedy_generation(make_engine, "B", prompts=(5, 1, 12), new=8)


def test_layers_that_use_another_layers_tensors():
    """Such a layer has no tensors and no block of its own, but a run, a cache or memory and rings of its own."""
    spec = spec_of(CONFIGS["A"])
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 2] and len(spec.layers) == 3
    shapes = spec.expected_shapes()
    assert not any(name.startswith("l2.") for name in shapes) and "l3.mix.dq" in shapes and "l3.norm2" not in shapes
    eng = make_engine(CONFIGS["A"], make_tensors(CONFIGS["A"], 1))
    _, _, states = eng.model.cache_plan()
    assert 0 in states and 2 in states and ("part", 2, "mixer_filter") in states and ("part", 3, "ffn_filter") not in states
    spec = spec_of(CONFIGS["B"])
    assert [e.layer for e in spec.schedule] == [0, 1, 0]
    eng = make_engine(CONFIGS["B"], make_tensors(CONFIGS["B"], 1))
    caches, _, states = eng.model.cache_plan()
    assert set(caches) == {0, 2} and not any(isinstance(k, tuple) for k in states)      # one tap: no ring anywhere


def test_residual_after_every_run_of_a_layer():
    """``ctx.layer_outputs`` receives the residual stream after every run of a layer."""
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
    assert load_config(folder).canon == {"taps": 3}
    shapes = spec_of(cfg).expected_shapes()
    assert shapes["l0.mix.a1"] == (8, 64) and shapes["l0.mix.a2"] == (32, 8) and shapes["l0.mix.a2.b"] == (32,)
    assert shapes["l0.mix.norm"] == (24,) and shapes["l0.canon2"] == (64, 3) and shapes["l0.rg1"] == (64, 64)
    assert shapes["l0.mlp.router"] == (6, 64) and shapes["l0.mlp.shared.sg"] == (1, 64) and shapes["l0.mlp.e5.gate"] == (40, 64)
    assert shapes["l1.mix.uk"] == (4 * 16, 32) and shapes["l1.mix.uv"] == (4 * 8, 32) and shapes["l1.mix.dq.norm"] == (24,)
    assert "l1.mlp.shared.gate" not in shapes and shapes["embed.norm"] == (64,) and shapes["final.norm"] == (64,)
    for path, value in ((("layers", 1, "type"), "other"), (("layers", 1, "mixer", "kv_rank"), 0), (("norm", "groups"), 5),
                        (("layers", 0, "mlp", "router", "top"), 7), (("layers", 2, "weights_of"), 1), (("canon", "taps"), 0),
                        (("layers", 2, "weights_of"), 2), (("layers", 0, "mlp", "kind"), "other"), (("logit_softcap"), 0),
                        (("layers", 0, "mixer", "tau"), 0.0), (("layers", 0, "mlp", "shared", "limit"), -1.0)):
        bad = json.loads(json.dumps(cfg))
        at = bad
        path = (path,) if isinstance(path, str) else path
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_the_decays_rank_comes_from_the_tensors(tmp_path):
    """config.json need not name the rank of the decays' low-rank product: the stored tensor's shape gives it, also to
    a layer that uses that layer's tensors."""
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    tensors = make_tensors(cfg, 5)
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
    folder = write_model(tmp_path / "m", cfg, tensors)
    eng = Engine.load_path(folder, dtype="float32", ops=TorchOps(torch.float32), max_tokens=256, max_seq=256)
    toks = tokens_for(cfg, 21, 4)
    assert BAND.ok(cases.run_cut(eng, toks, [9, 20]), plain.forward(cfg, tensors, toks))
    with pytest.raises(ConfigError):
        spec_of(cfg)


def test_replay_runs_the_design(tmp_path):
    """Trace replay chooses the model class by config.json and writes the wanted rows."""
    import io
    import numpy as np
    from rbitnet_b200.replay import main
    cfg = CONFIGS["C"]
    tensors = make_tensors(cfg, 3)
    folder = write_model(tmp_path / "m", cfg, tensors, store=torch.bfloat16)
    a, b = tokens_for(cfg, 20, 1), tokens_for(cfg, 7, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:15], "want": [0, 14]}, {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[15:16], "want": []}, {"id": "b", "tokens": b[6:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[16:], "want": [3]}], "end": ["a"]}]
    out = io.StringIO()
    rc = main(["--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128"],
              stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out, ops=TorchOps(torch.float32))
    assert rc == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    ref_a, ref_b = plain.forward(cfg, tensors, a, torch.float64), plain.forward(cfg, tensors, b, torch.float64)
    read = lambda n, rows: torch.from_numpy(np.fromfile(tmp_path / "o" / f"{n}.f32", dtype="<f4").reshape(rows, -1))
    assert cases.rel_err(read(0, 2), ref_a[[0, 14]]) <= TOL and cases.rel_err(read(1, 1), ref_b[[6]]) <= TOL
    assert cases.rel_err(read(2, 1), ref_a[[19]]) <= TOL


def test_command_line_serves_the_design(tmp_path, capsys):
    """random -> inspect -> generate, the same verbs as for the other decoders."""
    from rbitnet_b200.cli import main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["B"]))
    assert main(["random", "--config", str(cfg_path), "--out", str(tmp_path / "m"), "--seed", "4", "--dtype", "float32"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "Nifarax: 2 layers (3 runs of a layer in a pass), width 80" in out and "tensors fit the model" in out
    assert main(["generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt-ids", "1 2 3", "--max-tokens", "5",
                 "--temperature", "0", "--max-seq", "256", "--cache-tokens", "256"], ops=TorchOps(torch.float32)) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    from rbitnet_b200.weights import read_model_tensors
    tensors = read_model_tensors(tmp_path / "m")
    seq = [1, 2, 3]
    for t in line["tokens"]:
        assert int(torch.argmax(plain.forward(CONFIGS["B"], tensors, seq)[-1])) == t
        seq.append(t)
    assert len(line["tokens"]) == 5
