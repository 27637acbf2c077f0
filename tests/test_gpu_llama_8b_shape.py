"""The layer sizes of Llama-3.1-8B (hidden 4096, 32 heads over 8 kv heads of size 128, intermediate
14336, pages of 64) with one layer and a reduced vocabulary: the kernels at another set of real tile
counts (head size 128, which the tcgen05 attention does not take, K = 4096 and 14336, two passes of
the decode product, a width above the fused-norm limit), compared with the plain implementation
whole, token by token and mixed."""
import numpy as np
import pytest

import plain_llama as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 1, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 14336, "vocab_size": 4000, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": False,
}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from hfee_b200.weights import write_random_model
    d = str(tmp_path_factory.mktemp("llama8b_shape"))
    write_random_model(d, CFG, seed=5, dtype="bfloat16")
    cfg, w = plain.load_model_dir(d)
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (200, 70, 130, 9)]
    refs = [plain.forward(cfg, w, s) for s in seqs]
    return d, cfg, seqs, refs


@pytest.mark.parametrize("dtype,tol", [("bfloat16", 2e-2), ("float32", 1e-4)])
def test_whole_token_by_token_and_mixed(model, dtype, tol):
    from hfee_b200 import EngineConfig, ModelRunner
    from hfee_b200.kernels import ops
    d, cfg, seqs, refs = model
    e = EngineConfig(dtype=dtype, page_size=64, max_requests=4, max_context=256, max_cache_tokens=11 * 64,
                     max_batch_tokens=256, use_cuda_graphs=True)
    runner = ModelRunner(d, e)
    for steps in (ru.whole(seqs), ru.prefill_then_decode(seqs, tail=12),
                  ru.mixed(seqs, live=4, seed=4, chunk_sizes=(2, 17, 64, 100, 129))):
        got = ru.run_in_process(runner, steps)
        ops.check_status()
        for i in range(len(seqs)):
            err = ru.rel_err(got[i], refs[i])
            assert err < tol, f"{dtype} request {i}: relative error {err:.3g}"
