"""The layer sizes of Llama-3.2-1B (hidden 2048, 32 heads over 8 kv heads of size 64, intermediate
8192, llama3 rope scaling, tied embeddings, pages of 64) with two layers and a reduced vocabulary:
every production kernel runs at its real tile counts (tcgen05 tiles with K = 2048 and 8192 and
ragged M, the skinny and streaming products, attention with 4 query heads per kv head) and is
compared with the plain implementation, whole, in portions and mixed with decoding."""
import numpy as np
import pytest

import plain_llama as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 16032, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from hfee_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("llama1b_shape"))
    write_random_model(d, CFG, seed=3, dtype="bfloat16")
    cfg, w = plain.load_model_dir(d)
    rng = np.random.default_rng(1)
    seqs = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (300, 70, 130, 20)]
    want = [[len(s) - 1] if i == 0 else list(range(len(s) - 3, len(s))) for i, s in enumerate(seqs)]
    refs = [plain.forward(cfg, w, s) for s in seqs]
    return d, cfg, seqs, refs


@pytest.mark.parametrize("dtype,tol", [("bfloat16", 2e-2), ("float32", 1e-4)])
def test_whole_portions_and_mixed(model, dtype, tol):
    from hfee_b200 import EngineConfig, ModelRunner
    d, cfg, seqs, refs = model
    e = EngineConfig(dtype=dtype, page_size=64, max_requests=4, max_context=512, max_cache_tokens=9 * 64,
                     max_batch_tokens=512, use_cuda_graphs=True)
    runner = ModelRunner(d, e)
    for steps in (ru.whole(seqs), ru.prefill_then_decode(seqs, tail=20), ru.mixed(seqs, live=4, seed=3,
                                                                                 chunk_sizes=(2, 17, 64, 100, 129))):
        got = ru.run_in_process(runner, steps)
        for i in range(len(seqs)):
            err = ru.rel_err(got[i], refs[i])
            assert err < tol, f"{dtype} request {i}: relative error {err:.3g}"
