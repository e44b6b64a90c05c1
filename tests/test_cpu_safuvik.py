"""The Safuvik decoder through the package's host logic (configuration, parts, cache and state
manager, step function, scheduler, generation) on the CPU stand-in of the kernel layer, against the
plain implementation."""
import json

import pytest
import torch

import safuvik_cases as cases
import plain_safuvik as plain
from safuvik_tiny import CONFIGS, make_tensors, write_model, tokens_for, spec_of
from torch_ops import TorchOps
from rbitnet_b200.config import config_from_dict, ConfigError, load_config
from rbitnet_b200.engine import Engine

# float32 against float64: these weights are scaled up so that faults show, which also amplifies rounding
# (the plain implementation run in float32 differs from itself in float64 by 2e-5 here)
TOL = 2e-4


def make_engine(cfg, tensors, max_tokens=64 * 16, graphs=False, **kw):
    return Engine(config_from_dict(cfg), dict(tensors), dtype="float32", ops=TorchOps(torch.float32),
                  max_tokens=max_tokens, max_seq=1024, **kw)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole(name):
    cases.whole_and_layers(make_engine, name, TOL, n=80)


@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_prefill_against_decoding(name):
    cases.prefill_against_decoding(make_engine, name, TOL, n=40, prompt=17)


def test_portions():
    cases.portions(make_engine, "A", TOL, n=132)


@pytest.mark.parametrize("name", ["A", "C"])
def test_batches(name):
    cases.batches_against_alone(make_engine, name, TOL, lengths=(1, 2, 67, 9), decode=6)


def test_slots_and_pages_used_again():
    cases.slots_and_pages_used_again(make_engine, "B", TOL)


def test_first_tokens():
    cases.first_tokens(make_engine, "A", TOL)


def test_window_edges():
    cases.window_edges(make_engine, 2e-4, window=5, n=24, cuts=[11, 20, 21, 22, 23])


def test_far_token():
    cases.far_token_moves_the_logits(make_engine, "B", 2e-4, n=110)


def test_greedy_generation():
    cases.greedy_generation(make_engine, "C", prompts=(5, 1, 12), new=8)


def test_config_is_read_and_checked(tmp_path):
    cfg = CONFIGS["A"]
    folder = write_model(tmp_path / "m", cfg, make_tensors(cfg, 1))
    assert load_config(folder).streams == 3
    spec = spec_of(cfg)
    assert spec.residual_streams == 3 and spec.logit_scale == 0.5 and "l2.norm2" not in spec.expected_shapes()
    assert spec.expected_shapes()["l1.mix.left.q.norm"] == (4 * 32,)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][1]["type"] = "other"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    bad = json.loads(json.dumps(cfg))
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_frequencies_of_the_position_part():
    """The position part's table against the plain implementation's sines and cosines."""
    from rbitnet_b200.parts.position import RotaryEncoding
    rot = CONFIGS["A"]["layers"][1]["mixer"]["left"]["rot"]
    part = RotaryEncoding(32, rot["base"], "interleaved", rot_dim=rot["dims"], scaling=rot["scaling"])
    f, mag = part.frequencies()
    cos, sin = plain.rotary_tables(rot, 50, torch.float64)
    ang = torch.arange(50, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(torch.cos(ang) * mag, cos, atol=1e-12) and torch.allclose(torch.sin(ang) * mag, sin, atol=1e-12)
    assert mag > 1.0 and float(f[-1]) < rot["base"] ** (-2.0 * (rot["dims"] // 2 - 1) / rot["dims"])


def test_replay_runs_the_design(tmp_path):
    """Trace replay chooses the model class by config.json and writes the wanted rows."""
    import io
    import numpy as np
    from rbitnet_b200.replay import main
    cfg = CONFIGS["C"]
    tensors = make_tensors(cfg, 3)
    folder = write_model(tmp_path / "m", cfg, tensors)
    toks = tokens_for(cfg, 20, 1)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:15], "want": [0, 14]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[15:16], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[16:], "want": [3]}], "end": ["a"]}]
    out = io.StringIO()
    rc = main(["--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128"],
              stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out, ops=TorchOps(torch.float32))
    assert rc == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    ref = plain.forward(cfg, tensors, toks, torch.float64)
    got0 = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, -1))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "o" / "2.f32", dtype="<f4").reshape(1, -1))
    assert not (tmp_path / "o" / "1.f32").exists()
    assert cases.rel_err(got0, ref[[0, 14]]) <= TOL and cases.rel_err(got2, ref[[19]]) <= TOL


def test_command_line_serves_the_design(tmp_path, capsys):
    """random -> inspect -> generate, the same verbs as for the Llama decoder."""
    from rbitnet_b200.cli import main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["C"]))
    assert main(["random", "--config", str(cfg_path), "--out", str(tmp_path / "m"), "--seed", "4", "--dtype", "float32"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "Safuvik: 2 layers, width 48" in out and "tensors fit the model" in out
    assert main(["generate", "--model", str(tmp_path / "m"), "--dtype", "float32", "--prompt-ids", "1 2 3", "--max-tokens", "5",
                 "--temperature", "0", "--max-seq", "256", "--cache-tokens", "256"], ops=TorchOps(torch.float32)) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    from rbitnet_b200.weights import read_model_tensors
    tensors = read_model_tensors(tmp_path / "m")
    seq = [1, 2, 3]
    for t in line["tokens"]:
        assert int(torch.argmax(plain.forward(CONFIGS["C"], tensors, seq)[-1])) == t
        seq.append(t)
    assert len(line["tokens"]) == 5
