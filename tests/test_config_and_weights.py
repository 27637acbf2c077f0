"""Configuration reading, the architecture registry, weight checks and random weights (CPU)."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import TINY_A, TINY_B
from hfee_b200.config import ConfigError, LlamaConfig, PartSpec, RunSpec, check_schedule, resolve
from hfee_b200.config.registry import architecture, known_architectures, read_config_json
from hfee_b200.models.llama import llama_spec
from hfee_b200.parts.model import model_tensor_needs
from hfee_b200.weights import (Checkpoint, TensorFiles, TensorNeed, WeightError, WeightFormatError, check_tensors,
                               write_file, write_random_model)


def test_config_reads_every_key_and_defaults():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (96, 3, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (32, 256, 384)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and c.tie_word_embeddings
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert c.rope_pairing == "interleaved" and c.max_position_embeddings == 256
    # defaults of the reference: kv heads = heads, head_dim = hidden/heads, eps 1e-5, theta 10000, ctx 2048
    d = LlamaConfig.from_dict({"hidden_size": 64, "num_hidden_layers": 1, "num_attention_heads": 4,
                               "intermediate_size": 8, "vocab_size": 10})
    assert (d.num_key_value_heads, d.head_dim, d.rms_norm_eps, d.rope_theta, d.max_position_embeddings) == \
           (4, 16, 1e-5, 10000.0, 2048)
    assert d.rope_scaling is None and not d.tie_word_embeddings and d.rope_pairing == "half"
    assert LlamaConfig.from_dict(c.to_dict()) == c
    assert LlamaConfig.from_dict({**TINY_A, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)
    assert LlamaConfig.from_dict({**TINY_A, "eos_token_id": 5}).eos_token_ids == (5,)


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "missing key 'hidden_size'"),
    ({"num_hidden_layers": 0}, "positive integer"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"head_dim": 15}, "must be even"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2}}, "not supported"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2}}, "missing"),
    ({"rope_pairing": "spiral"}, "rope_pairing"),
])
def test_config_errors_name_the_key(change, match):
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict({**TINY_A, **change})


def test_registry(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    arch, cfg = resolve(TINY_A)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    with pytest.raises(ConfigError, match="unsupported model architecture 'MambaForCausalLM'"):
        resolve({**TINY_A, "architectures": ["MambaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in TINY_A.items() if k != "architectures"})
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path))


def test_llama3_scaling_bands():
    c = LlamaConfig.from_dict(TINY_B)
    inv = [1.0 / (c.rope_theta ** (2 * i / c.head_dim)) for i in range(c.head_dim // 2)]
    out = c.rope_scaling.apply(inv)
    s = c.rope_scaling
    for a, b in zip(inv, out):
        wavelen = 2 * np.pi / a
        if wavelen < s.original_max_position_embeddings / s.high_freq_factor:
            assert b == a
        elif wavelen > s.original_max_position_embeddings / s.low_freq_factor:
            assert b == a / s.factor
        else:
            assert a / s.factor < b < a
    assert any(b == a for a, b in zip(inv, out)) and any(b == a / s.factor for a, b in zip(inv, out))


def test_spec_is_data_and_schedule_is_checked():
    spec = llama_spec(LlamaConfig.from_dict(TINY_A))
    assert len(spec.layers) == 2 and [r.layer for r in spec.schedule] == [0, 1]
    assert sorted(spec.layers[0].parts) == ["ffn", "ffn_norm", "mixer", "mixer_norm"]       # a layer's parts are data
    category, mixer = spec.layers[0].parts["mixer"]
    assert category == "mixer" and mixer.kind == "attention" and mixer.position.kind == "rotary"
    assert spec.layers[0].parts["ffn"] == ("feed_forward", spec.layers[1].parts["ffn"][1])
    assert mixer == spec.layers[1].parts["mixer"][1] and hash(mixer) == hash(spec.layers[1].parts["mixer"][1])
    assert mixer.replace(window=8) != mixer
    check_schedule(spec.layers, [RunSpec(0, 0), RunSpec(1, 1), RunSpec(1, 2), RunSpec(0, 0, writes_cache=False)])
    with pytest.raises(ValueError, match="already has a writer"):
        check_schedule(spec.layers, [RunSpec(0, 0), RunSpec(1, 0)])
    with pytest.raises(ValueError, match="before any run has written"):
        check_schedule(spec.layers, [RunSpec(0, 3, writes_cache=False)])
    with pytest.raises(ValueError, match="names layer 5"):
        check_schedule(spec.layers, [RunSpec(5, 0)])


def test_tensor_needs_cover_the_checkpoint_names():
    needs = model_tensor_needs(llama_spec(LlamaConfig.from_dict(TINY_A)))
    assert needs["model.embed_tokens.weight"].shape == (256, 64)
    assert needs["lm_head.weight"].shape == (256, 64)
    assert needs["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert needs["model.layers.0.mlp.down_proj.weight"].shape == (64, 172)
    assert needs["model.norm.weight"].role == "scale"
    assert len(needs) == 3 + 2 * 9
    tied = model_tensor_needs(llama_spec(LlamaConfig.from_dict(TINY_B)))
    assert tied["lm_head.weight"].optional and len(tied) == 3 + 3 * 9      # a tied model may still store a head
    # an architecture that gives an optional tensor no name simply never reads it; a required one must be named
    import dataclasses
    spec = llama_spec(LlamaConfig.from_dict(TINY_B))
    unnamed = dataclasses.replace(spec, names={k: v for k, v in spec.names.items() if k != "head.weight"})
    assert "lm_head.weight" not in model_tensor_needs(unnamed) and len(model_tensor_needs(unnamed)) == 2 + 3 * 9
    with pytest.raises(ValueError, match="no checkpoint name"):
        model_tensor_needs(dataclasses.replace(spec, names={k: v for k, v in spec.names.items() if k != "final_norm.weight"}))


def test_buffers_the_architecture_names_as_ignorable_are_skipped_with_a_warning(tmp_path):
    """Older exports store ``rotary_emb.inv_freq`` beside every layer's weights: the load goes through
    and says what it skipped; any other stranger still fails, in the same single error."""
    d = str(tmp_path / "m")
    write_random_model(d, TINY_A, seed=0)
    files = TensorFiles(d)
    tensors = {n: files.tensor(n).clone() for n in files.names()}
    for i in range(2):
        tensors[f"model.layers.{i}.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_file(os.path.join(d, "model.safetensors"), tensors)
    spec = llama_spec(LlamaConfig.from_dict(TINY_A))
    assert spec.ignorable == ("*.rotary_emb.inv_freq",)
    with pytest.warns(UserWarning, match="2 tensors of the checkpoint are not used"):
        Checkpoint(d).check(model_tensor_needs(spec), spec.ignorable)
    with pytest.raises(WeightError) as e:
        Checkpoint(d).check(model_tensor_needs(spec))                      # without the patterns they are strangers
    assert len(e.value.unexpected) == 2
    tensors["model.layers.0.self_attn.something_else"] = torch.zeros(3)
    write_file(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        Checkpoint(d).check(model_tensor_needs(spec), spec.ignorable)
    assert e.value.unexpected == ["model.layers.0.self_attn.something_else"]


def test_a_config_without_the_feed_forward_width_takes_it_from_the_gate_projection(tmp_path):
    """config.json without ``intermediate_size``: a model folder's width comes from the rows of the first
    layer's gate matrix (as the reference reads it); the content of config.json alone still names the key."""
    import json
    from hfee_b200.config import resolve, resolve_model_dir
    d = str(tmp_path / "m")
    write_random_model(d, TINY_A, seed=0)
    short = {k: v for k, v in TINY_A.items() if k != "intermediate_size"}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(short, f)
    arch, cfg = resolve_model_dir(d)
    assert cfg.intermediate_size == TINY_A["intermediate_size"]
    assert cfg == resolve(TINY_A)[1]
    with pytest.raises(ConfigError, match="intermediate_size"):
        resolve(short)
    spec = arch.build_spec(cfg)
    Checkpoint(d).check(model_tensor_needs(spec), spec.ignorable)          # and the checkpoint fits it


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, TINY_A, seed=0)
    files = TensorFiles(d)
    tensors = {n: files.tensor(n).clone() for n in files.names()}
    del tensors["model.layers.0.self_attn.q_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.9.mlp.up_proj.weight"] = torch.zeros(2, 2)
    tensors["lm_head.weight"] = torch.zeros(256, 65)
    tensors["model.layers.1.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_file(os.path.join(d, "model.safetensors"), tensors)
    needs = model_tensor_needs(llama_spec(LlamaConfig.from_dict(TINY_A)))
    with pytest.raises(WeightError) as e:
        Checkpoint(d).check(needs)
    err = e.value
    assert err.missing == ["model.layers.0.self_attn.q_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.9.mlp.up_proj.weight"]
    assert err.wrong_shape == [("lm_head.weight", (256, 65), (256, 64))]
    assert err.wrong_dtype == [("model.layers.1.input_layernorm.weight", "torch.int32")]
    msg = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [256, 65], expected [256, 64]"):
        assert piece in msg


def test_safetensors_round_trip_and_format_errors(tmp_path):
    p = str(tmp_path / "t.safetensors")
    src = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    write_file(p, src)
    os.rename(p, str(tmp_path / "model.safetensors"))
    files = TensorFiles(str(tmp_path))
    for k, v in src.items():
        assert torch.equal(files.tensor(k), v) and files.info(k).dtype == v.dtype
    with open(str(tmp_path / "model.safetensors"), "r+b") as f:
        f.truncate(40)
    with pytest.raises(WeightFormatError):
        TensorFiles(str(tmp_path))
    with pytest.raises(WeightFormatError, match="no model.safetensors"):
        TensorFiles(str(tmp_path / "nowhere"))


def test_dtype_policy():
    from hfee_b200.weights import kept_dtype
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(TensorNeed((2, 2), "matrix"), f32, bf) == bf
    assert kept_dtype(TensorNeed((2, 2), "table"), bf, f32) == f32
    assert kept_dtype(TensorNeed((2,), "scale"), bf, bf) == f32          # norm scales stay 32-bit
    assert kept_dtype(TensorNeed((2,), "vector"), f32, bf) == f32
    assert kept_dtype(TensorNeed((2,), "index"), torch.int64, bf) == torch.int32


def test_random_weights_are_seeded_per_tensor(tmp_path):
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    write_random_model(a, TINY_A, seed=4)
    write_random_model(b, TINY_A, seed=4)
    write_random_model(c, {**TINY_A, "num_hidden_layers": 1}, seed=4)
    fa, fb, fc = TensorFiles(a), TensorFiles(b), TensorFiles(c)
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    # a tensor's values do not depend on which other tensors were written
    assert torch.equal(fa.tensor("model.layers.0.mlp.up_proj.weight"), fc.tensor("model.layers.0.mlp.up_proj.weight"))
    w = fa.tensor("model.layers.0.mlp.up_proj.weight")
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(fa.tensor("model.norm.weight").mean()) - 1.0) < 0.02
    assert json.load(open(os.path.join(a, "config.json")))["torch_dtype"] == "float32"
    write_random_model(str(tmp_path / "d"), TINY_B, seed=1, dtype="bfloat16")
    assert TensorFiles(str(tmp_path / "d")).info("model.embed_tokens.weight").dtype == torch.bfloat16
