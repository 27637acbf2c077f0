"""Replay on the GPU in float32 and bfloat16, compared with the plain implementation:
whole requests, prefill then token by token, portions of changing size, and mixed
batches with so few pages that they are used again."""
import numpy as np
import pytest

import plain_llama as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

# Largest |difference| relative to the largest |logit| of the plain float64 result.
# float32: rounding of float32 arithmetic only.  bfloat16: weights are the same
# bfloat16 values on both sides; activations and cache entries are rounded to 8
# mantissa bits between kernels while sums and the residual stream stay float32.
TOL = {"float32": 1e-4, "bfloat16": 2e-2}


def make_runner(model_dir, dtype, max_tokens, page_size=16, max_requests=4, batch=None):
    from hfee_b200 import EngineConfig, ModelRunner
    e = EngineConfig(dtype=dtype, page_size=page_size, max_requests=max_requests, max_context=max_tokens,
                     max_cache_tokens=max_tokens, max_batch_tokens=batch or max_tokens, use_cuda_graphs=False)
    return ModelRunner(model_dir, e)


def sequences(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


@pytest.fixture(scope="module")
def refs(tiny_dirs):
    """Plain logits of the test sequences, per config and weight rounding."""
    out = {}
    for name in ("A", "B"):
        for dtype in ("float32", "bfloat16"):
            cfg, w = plain.load_model_dir(tiny_dirs[name], round_to_bf16=(dtype == "bfloat16"))
            seqs = sequences(cfg.vocab, (5, 17, 33, 100, 1, 71, 40, 9), seed=11)
            out[name, dtype] = (cfg, seqs, [plain.forward(cfg, w, s) for s in seqs])
    return out


def check(got, seqs, ref, dtype):
    assert sorted(got) == list(range(len(seqs)))
    for i in range(len(seqs)):
        assert got[i].shape == ref[i].shape
        err = ru.rel_err(got[i], ref[i])
        assert err < TOL[dtype], f"request {i}: relative error {err:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("scheme", ["whole", "prefill_then_decode", "portions", "mixed"])
def test_replay(tiny_dirs, refs, name, dtype, scheme):
    cfg, seqs, ref = refs[name, dtype]
    if scheme == "mixed":
        steps = ru.mixed(seqs, live=4, seed=2)
        # pages for the four longest at once would be 100+71+40+33 -> 16 pages of 16; give 17
        runner = make_runner(tiny_dirs[name], dtype, max_tokens=17 * 16)
    else:
        steps = getattr(ru, scheme)(seqs)
        runner = make_runner(tiny_dirs[name], dtype, max_tokens=112)      # 7 pages: every request reuses pages
    got = ru.run_in_process(runner, steps)
    check(got, seqs, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("scheme", ["equal_portions", "two_sizes", "mixed"])
def test_steps_whose_shape_repeats_replay_from_cuda_graphs(tiny_dirs, refs, name, dtype, scheme):
    """Prompt portions of one size (the usual case under a token budget), of two alternating sizes, and
    mixed steps: from the third step of a shape on they are replayed from a captured graph, at other
    positions, on other pages and for other requests than the captured step's."""
    from hfee_b200 import EngineConfig, ModelRunner
    cfg, seqs, ref = refs[name, dtype]
    if scheme == "mixed":
        steps, tokens = ru.mixed(seqs, live=4, seed=2, chunk_sizes=(2, 5, 16)), 17 * 16
    else:
        steps, tokens = ru.portions(seqs, sizes=(8,) if scheme == "equal_portions" else (16, 3)), 112
    e = EngineConfig(dtype=dtype, page_size=16, max_requests=4, max_context=tokens, max_cache_tokens=tokens,
                     max_batch_tokens=tokens, use_cuda_graphs=True)
    runner = ModelRunner(tiny_dirs[name], e)
    got = ru.run_in_process(runner, steps)
    check(got, seqs, ref, dtype)
    assert runner.graph_replays >= (20 if scheme != "mixed" else 1), runner.graph_replays


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_binary(tiny_dirs, refs, tmp_path, dtype):
    cfg, seqs, ref = refs["B", dtype]
    steps = ru.mixed(seqs, live=4, seed=4)
    got = ru.run_trace_binary(tiny_dirs["B"], dtype, steps, str(tmp_path / "out"), max_tokens=384,
                              vocab=cfg.vocab)
    check(got, seqs, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode_through_cuda_graphs(tiny_dirs, refs, dtype):
    """Three requests decoded token by token for 150 steps across many pages, with the
    decode steps captured in and replayed from CUDA graphs; one request ends early so the
    batch size (and the graph) changes."""
    import plain_llama as plain
    from hfee_b200 import EngineConfig, ModelRunner, StepEntry
    cfg, w = plain.load_model_dir(tiny_dirs["B"], round_to_bf16=(dtype == "bfloat16"))
    seqs = sequences(cfg.vocab, (160, 151, 90), seed=21)
    ref = [plain.forward(cfg, w, s) for s in seqs]
    e = EngineConfig(dtype=dtype, page_size=16, max_requests=4, max_context=256, max_cache_tokens=27 * 16,
                     max_batch_tokens=64, use_cuda_graphs=True)
    runner = ModelRunner(tiny_dirs["B"], e)
    slots = [runner.open() for _ in seqs]
    heads = [10, 1, 5]
    runner.step([StepEntry(s, q[:h], []) for s, q, h in zip(slots, seqs, heads)])
    at = list(heads)
    got = [[] for _ in seqs]
    live = [0, 1, 2]
    while live:
        entries = [StepEntry(slots[i], [seqs[i][at[i]]], [0]) for i in live]
        rows = runner.step(entries).float().cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(rows[j].copy())
            at[i] += 1
        for i in list(live):
            if at[i] == len(seqs[i]):
                runner.close(slots[i])
                live.remove(i)
    assert runner.graph_replays > 100
    for i in range(3):
        err = ru.rel_err(np.stack(got[i]), ref[i][heads[i]:])
        assert err < TOL[dtype], f"request {i}: relative error {err:.3g}"
