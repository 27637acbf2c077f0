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


# ---------------------------------------------------------------------------------------------
# The batches the benchmark runs: 16 and 64 live requests decoding together.

def _tails(n):
    """Decoded tokens per request: all ``n`` stay for 40 steps, then one leaves per step, and the
    last eight stay ten steps longer (so batch sizes n ... 9 are seen once each, 8 eleven times)."""
    return [40 + i if i < n - 8 else 40 + (n - 8) + 10 + (i - (n - 8)) for i in range(n)]


@pytest.fixture(scope="module")
def crowd(model):
    """64 requests: prompts of 5 to 60 tokens followed by as many tokens as the longest schedule decodes."""
    d, cfg, _, _ = model
    _, w = plain.load_model_dir(d)
    rng = np.random.default_rng(7)
    heads = [int(rng.integers(5, 61)) for _ in range(64)]
    seqs = [rng.integers(0, cfg.vocab, size=h + t).tolist() for h, t in zip(heads, _tails(64))]
    refs = [plain.forward(cfg, w, s) for s in seqs]
    return heads, seqs, refs


@pytest.mark.parametrize("live", [16, 64])
@pytest.mark.parametrize("dtype,tol", [("bfloat16", 2e-2), ("float32", 1e-4)])
def test_many_requests_decoding_together(model, crowd, live, dtype, tol):
    """Prompts one after the other, then decode-only steps of the whole batch through CUDA graphs
    (the batch sizes at which the step changes its kernels: 64 ... 17, 16 ... 9, 8 ...), requests
    leaving at different steps; every row of every step against the plain implementation."""
    from hfee_b200 import EngineConfig, ModelRunner
    d, cfg, _, _ = model
    heads, full, full_refs = crowd
    tails = _tails(live)
    pick = range(64 - live, 64)                                        # the longest ones
    heads = [heads[i] for i in pick]
    seqs = [full[i][:h + t] for i, h, t in zip(pick, heads, tails)]    # a prefix of a sequence has the same logits
    assert all(len(s) == h + t for s, h, t in zip(seqs, heads, tails))
    refs = [full_refs[i][:len(s)] for i, s in zip(pick, seqs)]
    e = EngineConfig(dtype=dtype, page_size=64, max_requests=live, max_context=4096, max_cache_tokens=live * 256,
                     max_batch_tokens=512, use_cuda_graphs=True)
    runner = ModelRunner(d, e)
    steps = ru.batched_decode(seqs, tails, want_head="last")
    sizes = [len(st["entries"]) for st in steps if all(len(t) == 1 for _, t, _ in st["entries"])]
    assert sizes.count(live) >= 40 and sizes.count(8) >= 10 and set(range(8, live + 1)) <= set(sizes)
    got = ru.run_in_process(runner, steps)
    want = ru.expected_rows(refs, steps)
    assert runner.graph_replays >= 38 + 8              # the full batch and the last eight ran from their graphs
    worst = max(ru.rel_err(got[i], want[i]) for i in range(len(seqs)))
    assert worst < tol, f"{dtype}, {live} live: relative error {worst:.3g}"
    if dtype == "bfloat16":
        # where the plain top-1 margin is clear the engine picks the same token
        checked = 0
        for i in range(len(seqs)):
            for row, r in zip(got[i], want[i]):
                top = np.sort(r)[-2:]
                if top[1] - top[0] > 2 * tol * np.abs(r).max():
                    assert int(np.argmax(row)) == int(np.argmax(r))
                    checked += 1
        assert checked > 100
