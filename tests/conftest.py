import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 172, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 128,
    "tie_word_embeddings": False, "rope_pairing": "half",
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "max_position_embeddings": 256, "tie_word_embeddings": True,
    "rope_pairing": "interleaved",
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1)}


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """Model folders (float32 weights) of the two tiny configurations."""
    from hfee_b200.weights import write_random_model
    out = {}
    for name, (cfg, seed) in TINY.items():
        d = str(tmp_path_factory.mktemp(f"tiny{name}"))
        write_random_model(d, cfg, seed=seed, dtype="float32")
        out[name] = d
    return out


@pytest.fixture
def cpu_ops(monkeypatch):
    import cpu_ops as doubles
    doubles.install(monkeypatch)
    return doubles
