"""The command line without a GPU: ``create`` writes a model folder that loads, ``show`` prints the
configuration and the parameter count (for the Llama-3.2-1B sizes without writing a tensor), unknown
commands and bad folders end with an error line and a non-zero code (cmd/hfee/main.go:21-48)."""
import json
import os

import numpy as np
import pytest

from conftest import TINY_B
from hfee_b200 import cli

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 131072,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True,
}


def test_create_then_show_round_trip(tmp_path, capsys):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(TINY_B))
    model = tmp_path / "model"
    assert cli.main(["create", str(model), str(cfg_path), "--seed", "3", "--dtype", "float32"]) == 0
    assert "wrote" in capsys.readouterr().out
    assert sorted(os.listdir(model)) == ["config.json", "model.safetensors"]
    assert json.load(open(model / "config.json"))["hidden_size"] == TINY_B["hidden_size"]
    # what was written loads without a complaint and holds what the model asks for
    from hfee_b200.config import read_config_json, resolve
    from hfee_b200.parts.model import model_tensor_needs
    from hfee_b200.weights import Checkpoint
    arch, cfg = resolve(read_config_json(str(model)))
    needs = model_tensor_needs(arch.build_spec(cfg))
    Checkpoint(str(model)).check(needs)
    want = sum(int(np.prod(n.shape)) for n in needs.values() if not n.optional)
    assert cli.main(["show", str(model)]) == 0
    out = capsys.readouterr().out
    assert "LlamaForCausalLM" in out and f"{want:,}" in out
    assert "num_key_value_heads" in out and "rope_theta" in out
    # a second seed gives other weights, the same seed the same bytes
    again = tmp_path / "again"
    assert cli.main(["create", str(again), str(cfg_path), "--seed", "3", "--dtype", "float32"]) == 0
    assert open(model / "model.safetensors", "rb").read() == open(again / "model.safetensors", "rb").read()
    other = tmp_path / "other"
    assert cli.main(["create", str(other), str(cfg_path), "--seed", "4", "--dtype", "float32"]) == 0
    assert open(model / "model.safetensors", "rb").read() != open(other / "model.safetensors", "rb").read()


def test_show_counts_the_parameters_of_the_1b_shape_from_config_alone(tmp_path, capsys):
    (tmp_path / "config.json").write_text(json.dumps(LLAMA_1B))
    assert cli.main(["show", str(tmp_path)]) == 0
    assert "1,235,814,400" in capsys.readouterr().out


def test_errors_are_one_line_and_a_code(tmp_path, capsys):
    assert cli.main(["show", str(tmp_path / "nothing")]) == 1
    assert capsys.readouterr().err.startswith("Error:")
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NoSuchModel"]}))
    assert cli.main(["show", str(tmp_path)]) == 1
    assert "NoSuchModel" in capsys.readouterr().err
    assert cli.main(["frobnicate"]) == 1
    assert "unknown command" in capsys.readouterr().err
    assert cli.main(["version"]) == 0
    assert "version" in capsys.readouterr().out
