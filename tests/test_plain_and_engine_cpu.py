"""Host logic end to end on the CPU: the engine's batching, cache and layer schedule
driven through torch stand-ins for the kernels, against the plain implementation."""
import numpy as np
import pytest

import plain_llama as plain
from hfee_b200 import EngineConfig, ModelRunner, StepEntry


def _runner(model_dir, page_size=16, max_tokens=256, max_requests=4):
    e = EngineConfig(dtype="float32", page_size=page_size, max_requests=max_requests, max_context=max_tokens,
                     max_cache_tokens=max_tokens, max_batch_tokens=max_tokens, device="cpu")
    return ModelRunner(model_dir, e)


def _rel(a, b):
    return float(np.max(np.abs(a - b)) / (np.max(np.abs(b)) + 1e-30))


@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompt_matches_plain(tiny_dirs, cpu_ops, name):
    cfg, w = plain.load_model_dir(tiny_dirs[name])
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg.vocab, size=37).tolist()
    ref = plain.forward(cfg, w, toks)
    r = _runner(tiny_dirs[name])
    s = r.open()
    out = r.step([StepEntry(s, toks, list(range(len(toks))))]).numpy()
    assert _rel(out, ref) < 2e-5


@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_and_mixed_match_plain(tiny_dirs, cpu_ops, name):
    cfg, w = plain.load_model_dir(tiny_dirs[name])
    rng = np.random.default_rng(5)
    seqs = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (41, 23, 64)]
    refs = [plain.forward(cfg, w, t) for t in seqs]
    r = _runner(tiny_dirs[name], page_size=16, max_tokens=96)      # 6 pages: reuse is forced
    cuts = [[7, 2, 16, 3, 2, 11], [1, 5, 2, 15], [30, 2, 2, 30]]
    got = [[] for _ in seqs]
    # request 0 and 1 interleaved, then 2 after 0 ended (its pages are reused)
    slots = {0: r.open(), 1: r.open()}
    cur = [0, 0, 0]
    order = [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (0, 3), (1, 3), (0, 4), (0, 5)]
    pending = []
    for which, ci in order:
        n = cuts[which][ci]
        pending.append((which, n))
        if len(pending) == 2 or which == 0 and ci >= 4:
            entries = []
            for wch, k in pending:
                entries.append(StepEntry(slots[wch], seqs[wch][cur[wch]:cur[wch] + k], list(range(k))))
            out = r.step(entries).numpy().copy()
            at = 0
            for wch, k in pending:
                got[wch].append(out[at:at + k]); at += k; cur[wch] += k
            pending = []
    r.close(slots[0]); r.close(slots[1])
    r.cache.check_invariants()
    slots[2] = r.open()
    for k in cuts[2]:
        out = r.step([StepEntry(slots[2], seqs[2][cur[2]:cur[2] + k], list(range(k)))]).numpy().copy()
        got[2].append(out); cur[2] += k
    for i in range(3):
        g = np.concatenate(got[i])
        assert g.shape[0] == len(seqs[i]) or i < 2
        assert _rel(g, refs[i][:g.shape[0]]) < 2e-5


@pytest.mark.parametrize("scheme", ["whole", "prefill_then_decode", "portions", "mixed"])
def test_replay_schemes_on_cpu(tiny_dirs, cpu_ops, scheme):
    import replay_util as ru
    cfg, w = plain.load_model_dir(tiny_dirs["B"])
    rng = np.random.default_rng(11)
    seqs = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (5, 17, 33, 50, 1, 40)]
    refs = [plain.forward(cfg, w, s) for s in seqs]
    steps = ru.mixed(seqs, live=4, seed=2) if scheme == "mixed" else getattr(ru, scheme)(seqs)
    r = _runner(tiny_dirs["B"], page_size=16, max_tokens=9 * 16 if scheme == "mixed" else 64)
    got = ru.run_in_process(r, steps)
    for i in range(len(seqs)):
        assert got[i].shape == refs[i].shape
        assert ru.rel_err(got[i], refs[i]) < 2e-5


def test_bfloat16_weight_layouts_on_cpu(tiny_dirs, cpu_ops):
    """bfloat16 mode fuses and interleaves projection rows at load; the result must not change."""
    cfg, w = plain.load_model_dir(tiny_dirs["A"], round_to_bf16=True)
    rng = np.random.default_rng(1)
    toks = rng.integers(0, cfg.vocab, size=21).tolist()
    ref = plain.forward(cfg, w, toks)
    e = EngineConfig(dtype="bfloat16", page_size=16, max_requests=2, max_context=64, max_cache_tokens=64,
                     max_batch_tokens=64, device="cpu")
    r = ModelRunner(tiny_dirs["A"], e)
    out = r.step([StepEntry(r.open(), toks, list(range(len(toks))))]).numpy()
    assert r.model.blocks[0].feed_forward.granule == 4
    assert float(np.max(np.abs(out - ref)) / np.max(np.abs(ref))) < 2e-2


@pytest.mark.parametrize("pipeline", [False, True])
def test_generate_on_cpu_doubles_pipelined_and_not(tiny_dirs, cpu_ops, pipeline):
    """Engine.generate end to end over the CPU doubles: greedy tokens equal the plain
    implementation's with and without pipelining, with an end token, and under a cache so small
    that requests are preempted and recomputed."""
    import json, os, shutil, tempfile
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (20, 25, 30)]
    want = [plain.greedy_generate(cfg, w, p, 12) for p in prompts]
    eng = Engine(tiny_dirs["A"], dtype="float32", page_size=16, max_requests=3, max_context=128,
                 max_batch_tokens=64, max_cache_tokens=6 * 16, device="cpu")
    eng.pipeline = pipeline
    seen = [[] for _ in prompts]
    res = eng.generate(prompts, SamplingOptions.greedy(num_predict=12), on_token=lambda i, t: seen[i].append(t))
    assert [r.token_ids for r in res] == want and seen == want
    assert sum(r.stats.preemptions for r in res) > 0
    assert eng.runner.cache.free_pages() == 6 and eng.runner.cache.free_slots() == 3
    # an end token: generation stops before it
    d = tempfile.mkdtemp()
    shutil.copytree(tiny_dirs["A"], d, dirs_exist_ok=True)
    c = json.load(open(os.path.join(d, "config.json")))
    c["eos_token_id"] = want[0][5]
    json.dump(c, open(os.path.join(d, "config.json"), "w"))
    eng2 = Engine(d, dtype="float32", page_size=16, max_requests=3, max_context=128, max_batch_tokens=64, device="cpu")
    eng2.pipeline = pipeline
    res2 = eng2.generate(prompts, SamplingOptions.greedy(num_predict=12))
    for r, wnt in zip(res2, want):
        cut = wnt.index(want[0][5]) if want[0][5] in wnt else len(wnt)
        assert r.token_ids == wnt[:cut]
        assert r.stats.done_reason == ("stop" if cut < len(wnt) else "length") and r.stats.eval_tokens == cut
    shutil.rmtree(d)


def test_tied_model_with_a_stored_head_uses_it(tiny_dirs, cpu_ops, tmp_path):
    """tie_word_embeddings with lm_head.weight in the file: accepted, and the stored head is used
    (the reference takes output.weight whenever the file has one, internal/llm/model.go:118-121)."""
    import os, shutil, torch
    from hfee_b200.weights import TensorFiles, write_file
    d = str(tmp_path / "m")
    shutil.copytree(tiny_dirs["B"], d)
    files = TensorFiles(d)
    tensors = {n: files.tensor(n).clone() for n in files.names()}
    tensors["lm_head.weight"] = torch.randn(384, 96, generator=torch.Generator().manual_seed(0)) * 0.02
    write_file(os.path.join(d, "model.safetensors"), tensors)
    cfg, w = plain.load_model_dir(d)
    toks = list(range(3, 20))
    ref = plain.forward(cfg, w, toks)                       # the plain model prefers lm_head.weight too
    r = _runner(d)
    out = r.step([StepEntry(r.open(), toks, list(range(len(toks))))]).numpy()
    assert _rel(out, ref) < 2e-5
