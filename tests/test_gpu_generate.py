"""Generation through the Python entry point: greedy tokens equal the plain implementation's,
seeded sampling does not depend on the batch, preemption under a tiny cache changes nothing."""
import numpy as np
import pytest

import plain_llama as plain

pytestmark = pytest.mark.gpu


def prompts_for(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg.vocab, size=n).tolist() for n in lengths]


@pytest.mark.parametrize("name,lengths,steps", [("A", (5, 17, 33), 16), ("B", (1, 9, 40, 100), 24)])
def test_greedy_generation_float32_equals_plain(tiny_dirs, name, lengths, steps):
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs[name])
    prompts = prompts_for(cfg, lengths, seed=3)
    want = [plain.greedy_generate(cfg, w, p, steps) for p in prompts]
    eng = Engine(tiny_dirs[name], dtype="float32", page_size=16, max_requests=4, max_context=128,
                 max_batch_tokens=64, prefill_chunk=16)
    res = eng.generate(prompts, SamplingOptions.greedy(num_predict=steps))
    assert [r.token_ids for r in res] == want
    for r, p in zip(res, prompts):
        assert r.stats.prompt_tokens == len(p) and r.stats.eval_tokens == steps and r.stats.done_reason == "length"
        assert r.stats.eval_seconds > 0 and r.text is None


def test_greedy_generation_bfloat16_follows_plain_where_the_margin_allows(tiny_dirs):
    """bfloat16 may flip a near-tie; wherever the plain top-1 margin exceeds the tolerance the
    engine must pick the same token (teacher-forced along the plain continuation)."""
    from hfee_b200 import EngineConfig, ModelRunner, StepEntry
    cfg, w = plain.load_model_dir(tiny_dirs["B"], round_to_bf16=True)
    prompt = prompts_for(cfg, (40,), seed=5)[0]
    cont = plain.greedy_generate(cfg, w, prompt, 24)
    seq = prompt + cont
    ref = plain.forward(cfg, w, seq)
    runner = ModelRunner(tiny_dirs["B"], EngineConfig(dtype="bfloat16", page_size=16, max_requests=2, max_context=128,
                                                      max_batch_tokens=64))
    s = runner.open()
    got = [runner.step([StepEntry(s, seq[:40], [39])]).float().cpu().numpy()[0].copy()]
    for t in range(40, len(seq) - 1):
        got.append(runner.step([StepEntry(s, [seq[t]], [0])]).float().cpu().numpy()[0].copy())
    checked = 0
    for row, r in zip(got, ref[39:]):
        top = np.sort(r)[::-1]
        if top[0] - top[1] > 2 * 2e-2 * np.abs(r).max():
            assert int(np.argmax(row)) == int(np.argmax(r))
            checked += 1
    assert checked >= 5


@pytest.mark.parametrize("name", ["A", "B"])
def test_pipelined_generation_bfloat16_picks_the_plain_top1_where_the_margin_allows(tiny_dirs, name):
    """Engine.generate in bfloat16 with its defaults (pipelined, tokens fed back on the device, CUDA
    graphs): along each request's own continuation every token whose plain top-1 margin is clear is
    the plain argmax, and the callback saw the same tokens."""
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs[name], round_to_bf16=True)
    prompts = prompts_for(cfg, (5, 40, 17, 33), seed=13)
    eng = Engine(tiny_dirs[name], dtype="bfloat16", page_size=16, max_requests=4, max_context=128, max_batch_tokens=64)
    assert eng.pipeline and eng.config.use_cuda_graphs
    seen = [[] for _ in prompts]
    res = eng.generate(prompts, SamplingOptions.greedy(num_predict=30), on_token=lambda i, t: seen[i].append(t))
    assert eng.runner.graph_replays > 20
    checked = 0
    for p, r, s in zip(prompts, res, seen):
        assert len(r.token_ids) == 30 and s == r.token_ids and r.stats.done_reason == "length"
        ref = plain.forward(cfg, w, p + r.token_ids[:-1])
        for t, tok in enumerate(r.token_ids):
            row = ref[len(p) - 1 + t]
            top = np.sort(row)[-2:]
            if top[1] - top[0] > 2 * 2e-2 * np.abs(row).max():
                assert tok == int(np.argmax(row)), (name, t)
                checked += 1
    assert checked >= 20


class _Letters:
    """A tokenizer for tests: token id -> one or two letters."""

    def piece(self, t):
        return (chr(ord("a") + t % 26) + (chr(ord("A") + (t // 26) % 26) if t % 3 == 0 else "")).encode()

    def decode(self, ids):
        return b"".join(self.piece(t) for t in ids).decode()

    def encode(self, text):
        raise NotImplementedError


def test_stop_string_and_cancel_through_the_pipelined_engine(tiny_dirs):
    """On the GPU with device-side token feedback: a stop string found one step late cuts the request
    where it belongs, a cancelled request ends with "abort", the others are untouched, and every
    page and slot is free afterwards."""
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    prompts = prompts_for(cfg, (20, 25, 30), seed=21)
    want = [plain.greedy_generate(cfg, w, p, 16) for p in prompts]
    tok = _Letters()
    text0 = tok.decode(want[0])
    ends = np.cumsum([len(tok.piece(t)) for t in want[0]])
    at = int(ends[6])
    stop = text0[at:at + 3]
    assert text0.find(stop) == at
    eng = Engine(tiny_dirs["A"], tokenizer=tok, dtype="float32", page_size=16, max_requests=3, max_context=128,
                 max_batch_tokens=64)
    assert eng.pipeline
    shown = ["", "", ""]

    def on_text(i, s):
        shown[i] += s

    opts = [SamplingOptions.greedy(num_predict=16).with_(stop=[stop]), SamplingOptions.greedy(num_predict=16),
            SamplingOptions.greedy(num_predict=16)]
    res = eng.generate(prompts, opts, on_text=on_text,
                       on_token=lambda i, t: not (i == 2 and t == want[2][4]))
    assert res[0].token_ids == want[0][:7] and res[0].text == text0[:at] == shown[0] and res[0].stats.done_reason == "stop"
    assert res[1].token_ids == want[1] and res[1].stats.done_reason == "length" and shown[1] == tok.decode(want[1])
    cut = want[2].index(want[2][4]) + 1
    assert res[2].stats.done_reason == "abort" and res[2].token_ids[:cut] == want[2][:cut] and len(res[2].token_ids) <= cut + 1
    eng.runner.cache.check_invariants()
    assert eng.runner.cache.free_pages() == eng.runner.cache.num_pages and eng.runner.cache.free_slots() == 3


def test_first_tokens_of_a_sequence(tiny_dirs):
    """Positions 0, 1, 2 one by one (a one-token prompt, then single tokens) in both dtypes."""
    from hfee_b200 import EngineConfig, ModelRunner, StepEntry
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 2e-2)):
        cfg, w = plain.load_model_dir(tiny_dirs["A"], round_to_bf16=(dtype == "bfloat16"))
        seq = [7, 200, 31, 0]
        ref = plain.forward(cfg, w, seq)
        runner = ModelRunner(tiny_dirs["A"], EngineConfig(dtype=dtype, page_size=16, max_requests=2, max_context=64,
                                                          max_batch_tokens=16, use_cuda_graphs=False))
        s = runner.open()
        for t, tok in enumerate(seq):
            row = runner.step([StepEntry(s, [tok], [0])]).float().cpu().numpy()[0]
            assert np.abs(row - ref[t]).max() / np.abs(ref[t]).max() < tol, (dtype, t)


def test_long_prompts_in_equal_portions_beside_decoding_requests_replay_graphs(tiny_dirs):
    """Ten requests with prompts of 70 to 120 tokens, four at a time, prompts cut into portions of 32: the
    shapes of the mixed steps repeat and are replayed from CUDA graphs; every token equals the plain
    implementation's."""
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["B"])
    prompts = prompts_for(cfg, (70, 96, 120, 75, 100, 88, 111, 97, 105, 80), seed=13)
    want = [plain.greedy_generate(cfg, w, p, 8) for p in prompts]
    eng = Engine(tiny_dirs["B"], dtype="float32", page_size=16, max_requests=4, max_context=160,
                 max_batch_tokens=64, prefill_chunk=32)
    assert eng.config.use_cuda_graphs
    res = eng.generate(prompts, SamplingOptions.greedy(num_predict=8))
    assert [r.token_ids for r in res] == want
    shapes = [k for k in eng.runner._graphs if isinstance(k, tuple)]
    assert shapes and eng.runner.graph_replays > 0, (shapes, eng.runner.graph_replays)


def test_preemption_under_a_tiny_cache_changes_no_token(tiny_dirs):
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    prompts = prompts_for(cfg, (20, 25, 30), seed=8)
    want = [plain.greedy_generate(cfg, w, p, 20) for p in prompts]
    eng = Engine(tiny_dirs["A"], dtype="float32", page_size=16, max_requests=3, max_context=128,
                 max_batch_tokens=64, max_cache_tokens=7 * 16)        # 7 pages: not enough for all three to finish
    sched_holder = {}
    orig = eng.new_scheduler

    def spy():
        sched_holder["s"] = orig()
        return sched_holder["s"]

    eng.new_scheduler = spy
    res = eng.generate(prompts, SamplingOptions.greedy(num_predict=20))
    assert sched_holder["s"].preemptions > 0
    assert [r.token_ids for r in res] == want
    assert eng.runner.cache.free_pages() == 7 and eng.runner.cache.free_slots() == 3


def test_seeded_sampling_does_not_depend_on_the_batch(tiny_dirs):
    from hfee_b200 import Engine, SamplingOptions
    cfg, _ = plain.load_model_dir(tiny_dirs["A"])
    prompts = prompts_for(cfg, (6, 11, 19), seed=4)
    eng = Engine(tiny_dirs["A"], dtype="float32", page_size=16, max_requests=4, max_context=128, max_batch_tokens=64)
    plain_t = SamplingOptions(temperature=0.9, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=11, num_predict=12)
    chain = SamplingOptions(temperature=0.9, seed=11, num_predict=12)          # top-k 40, top-p 0.9, penalty 1.1
    for opts in (plain_t, chain):
        together = [r.token_ids for r in eng.generate(prompts, opts)]
        alone = [eng.generate([p], opts)[0].token_ids for p in prompts]
        assert together == alone
        assert together != [r.token_ids for r in eng.generate(prompts, opts.with_(seed=12))]
    greedy = [r.token_ids for r in eng.generate(prompts, SamplingOptions.greedy(12))]
    assert greedy != together


def test_eos_stops_generation_without_emitting_it(tiny_dirs, tmp_path):
    import json, os, shutil
    from hfee_b200 import Engine, SamplingOptions
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    prompt = prompts_for(cfg, (9,), seed=2)[0]
    cont = plain.greedy_generate(cfg, w, prompt, 10)
    d = str(tmp_path / "m")
    shutil.copytree(tiny_dirs["A"], d)
    c = json.load(open(os.path.join(d, "config.json")))
    c["eos_token_id"] = cont[4]
    json.dump(c, open(os.path.join(d, "config.json"), "w"))
    eng = Engine(d, dtype="float32", page_size=16, max_requests=2, max_context=64, max_batch_tokens=32)
    r = eng.generate([prompt], SamplingOptions.greedy())[0]
    first = cont.index(cont[4])
    assert r.token_ids == cont[:first] and r.stats.done_reason == "stop"


def test_cli_run_with_prompt_ids(tiny_dirs):
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, w = plain.load_model_dir(tiny_dirs["A"])
    want = plain.greedy_generate(cfg, w, [5, 6, 7], 6)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "hfee-b200"), "run", tiny_dirs["A"], "--prompt-ids",
                        "5,6,7", "--temperature", "0", "--repeat-penalty", "1", "--num-predict", "6", "--dtype",
                        "float32", "--num-ctx", "256", "--verbose"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    assert p.stdout.split("\n")[0].split() == [str(t) for t in want]
    assert "eval count:           6 token(s)" in p.stdout and "prompt eval count:    3 token(s)" in p.stdout
