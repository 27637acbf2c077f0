#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Llama-3.2-1B shape with random
bfloat16 weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 1b|8b|13b] [--layers L] [--dtype bfloat16|float32] [--breakdown]

A "step" is one decode step of a batch of 8 requests whose prompts of 2,048 tokens
are already cached (context limit 4,096).  The JSON line carries: ``value`` (decoded
tokens a second, timed on the device over exactly K steps), ``e2e`` (the same through
``Engine.generate``: host tokens in, host tokens out), ``prefill`` (one prompt of
2,048 tokens), ``roofline`` (bytes a decode step must read over its time, against the
measured HBM copy bandwidth), ``points`` (decode at batch 1 and 64), ``clocks`` and
``gpu_launches``.  Weights (2.5 GB) and the cache of the live requests are far larger
than the 126 MB L2, so no L2 flush is needed between steps.

``--shape 8b`` / ``13b`` run the layer sizes of Llama-3.1-8B / Llama-2-13B (by default with fewer
layers, named beside the full number in ``config``), ``--dtype float32`` the true 32-bit path.
``--breakdown`` prints, instead of the line above, what each class of kernels costs inside the decode
step at batch 1, 8 and 64 and inside the prompt pass: the step is timed again with that class's
launches left out (results wrong, timing not), and the difference is the class's cost in place.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Llama-3.2-1B shape.
MODEL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
}
# BASELINE.json configs[3] and configs[4]: the Llama-3.1-8B and Llama-2-13B shapes.
SHAPES = {
    "1b": (MODEL, "llama-3.2-1b-shape", 16),
    "8b": ({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
        "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": False,
    }, "llama-3.1-8b-shape", 8),
    "13b": ({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 40,
        "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0,
        "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    }, "llama-2-13b-shape", 8),
}
E2E_MIN_STEPS = 128                               # the wall-clock window of the end-to-end number never shrinks below this
PROMPT = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PUBLISHED_TOK_S = 7.0      # "about 7" tokens/s for llama3.2:1b on a 2-core VPS, the reference's README


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in list(out) + ["sm_max_mhz"]:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi sampling SM clocks and throttle reasons while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self):
        self.stop()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, layers, elem=2):
    """Sizes a decode step reads: every matrix once (the embedding table only as the head, or the
    head of its own), ``elem`` bytes per weight and cache element."""
    d, h, kv, hd, i, v = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                          cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    layer_params = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i
    return {"layer_params": layer_params, "head_params": v * d,
            "weight_bytes": elem * (layers * layer_params + v * d) + 4 * (2 * layers + 1) * d,
            "kv_bytes_per_token": 2 * layers * kv * hd * elem}


def prefill_flops(cfg, layers, t):
    n = model_numbers(cfg, layers)
    attn = 4 * layers * cfg["num_attention_heads"] * cfg["head_dim"] * t * (t + 1) // 2
    return 2 * t * layers * n["layer_params"] + attn + 2 * n["head_params"]


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "hostfog/hfee is a Go program with no Python package (pip: 'neither setup.py nor "
                      "pyproject.toml found') and no Go toolchain is installed, so it cannot be built or run here"}))
    return 0


def main():
    global PROMPT, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes: Llama-3.2-1B (the headline), 3.1-8B, 2-13B")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers of the same sizes, if memory or time needs it (config names both numbers)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--breakdown", action="store_true", help="cost of each class of kernels inside the steps, instead of the bench line")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="profiling aid: run just one of the measurements (the JSON line is then partial)")
    ap.add_argument("--prompt", type=int, default=PROMPT,
                    help="tokens of the prompts (other context lengths than the headline's 2,048; the cache holds twice as many per request)")
    ap.add_argument("--no-graphs", action="store_true", help="profiling aid: launch decode kernels one by one")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.prompt != PROMPT:
        PROMPT, CONTEXT = args.prompt, max(CONTEXT, 2 * args.prompt)

    import numpy as np
    import torch
    from hfee_b200 import Engine, SamplingOptions, StepEntry, write_random_model
    from hfee_b200.kernels import ops

    pk = peaks()
    model, model_name, default_layers = SHAPES[args.shape]
    full_layers = model["num_hidden_layers"]
    layers = args.layers or default_layers
    f32 = args.dtype == "float32"
    elem = 4 if f32 else 2
    cfg = dict(model, num_hidden_layers=layers)
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], CONTEXT)
    nums = model_numbers(cfg, layers, elem)
    context = min(CONTEXT, cfg["max_position_embeddings"])
    if f32:      # no tensor cores on this path: FFMA rate of this device at its highest clock
        props = torch.cuda.get_device_properties(0)
        compute_peak = props.multi_processor_count * 128 * 2 * (pk.get("sm_max_mhz") or 1965.0) * 1e6
    else:
        compute_peak = pk["bf16_tflops"] * 1e12
    rng = np.random.default_rng(0)
    tmp = tempfile.mkdtemp(prefix="hfee_bench_")
    t0 = time.time()
    write_random_model(tmp, cfg, seed=0, dtype="bfloat16")
    print(f"[bench] random model written in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)

    if args.only != "all":
        args.no_points = args.no_e2e = True
    max_b = 64 if (args.breakdown or not args.no_points) else args.batch
    max_b = max(max_b, args.batch)
    engine = Engine(tmp, dtype=args.dtype, page_size=64, max_requests=max_b, max_context=context,
                    max_batch_tokens=PROMPT, max_cache_tokens=max_b * context, use_cuda_graphs=not args.no_graphs)
    runner = engine.runner
    import shutil
    shutil.rmtree(tmp, ignore_errors=True)
    vocab = cfg["vocab_size"]
    sample_out = torch.zeros(max_b, dtype=torch.int32, device=runner.device)
    argmax_scratch = engine.sampler.argmax_scratch

    def timed(fn, iters):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(iters):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    prompt = rng.integers(0, vocab, size=PROMPT).tolist()

    def prefill_once(_):
        s = runner.open()
        runner.step([StepEntry(s, prompt, [PROMPT - 1])])
        runner.close(s)

    def decode_point(batch, steps, warmup, quiet=False):
        """Time ``steps`` decode steps of ``batch`` requests with prompts of PROMPT tokens cached."""
        slots = [runner.open() for _ in range(batch)]
        for s in slots:
            runner.step([StepEntry(s, rng.integers(0, vocab, size=PROMPT).tolist(), [])])
        start = PROMPT
        feed = rng.integers(0, vocab, size=(warmup + steps, batch)).tolist()

        def one(i):
            logits = runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.tag("sample")
            ops.argmax(logits, sample_out[:batch], argmax_scratch)

        for i in range(warmup):
            one(i)
        before = ops.launch_count()
        if not quiet:
            print(f"[bench] timed decode (batch {batch}) starts after {before} launches", file=sys.stderr, flush=True)
        ms = timed(lambda i: one(warmup + i), steps)
        launches = ops.launch_count() - before
        ctx = start + warmup + (steps - 1) / 2.0 + 1
        for s in slots:
            runner.close(s)
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launches,
                "bytes": nums["weight_bytes"] + batch * ctx * nums["kv_bytes_per_token"], "context": ctx}

    config = {"model": model_name, "global_batch": args.batch, "seq_len": context,
              "prompt_len": PROMPT, "parallelism": "single_gpu", "layers": layers,
              "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
              "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
              "intermediate": cfg["intermediate_size"], "vocab": vocab, "tied_embeddings": bool(cfg["tie_word_embeddings"]),
              "page_size": 64, "weights": "random bf16 seed 0", "l2": "inputs larger than L2",
              "peaks": pk["source"] + (", float32 against the FFMA rate" if f32 else "")}

    # ---------------------------------------------------------------- cost of each class of kernels
    if args.breakdown:
        per_layer = ["norm", "qkv", "rope", "attention", "o", "gate_up", "down"]
        once = ["embed", "head", "sample"]
        out = {"breakdown": "step time minus step time with the class left out; us per layer for layer classes, us per step for the rest",
               "config": config, "dtype": "bf16" if not f32 else "fp32"}

        def forget_graphs():
            runner._graphs.clear()
            runner._graph_seen.clear()

        def classes_of(measure, rounds=3):
            """Whole step and step without a class back to back, ``rounds`` times; the class costs the median
            of the differences of such pairs (the clocks move under the power cap during a run this long,
            and the two halves of a pair see the same clocks)."""
            whole_all = []
            res = {}
            for c in per_layer + once:
                diffs = []
                for _ in range(rounds):
                    ops.leave_out([])
                    forget_graphs()
                    whole = measure()
                    ops.leave_out([c])
                    forget_graphs()
                    diffs.append(whole - measure())
                    whole_all.append(whole)
                res[c] = round(statistics.median(diffs) * 1e3 / (layers if c in per_layer else 1), 2)
            ops.leave_out([])
            forget_graphs()
            res["step_ms"] = round(statistics.median(whole_all), 4)
            res["step_ms_spread"] = round(max(whole_all) - min(whole_all), 4)
            res["sum_ms"] = round(sum(res[c] * (layers if c in per_layer else 1) for c in per_layer + once) / 1e3, 4)
            return res

        clocks = ClockSampler()
        clocks.start()
        for b in (1, 8, 64):            # every measurement on freshly read prompts: the same context each time
            out[f"decode_b{b}"] = classes_of(lambda: decode_point(b, 64, 4, quiet=True)["ms_per_step"])
        for _ in range(args.warmup):
            prefill_once(0)
        out["prefill_2048"] = classes_of(lambda: timed(prefill_once, 2) / 2, rounds=7)
        out["clocks"] = clocks.summary()
        print(json.dumps(out))
        return 0

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    clocks = ClockSampler()
    prefill = None
    if args.only in ("all", "prefill"):
        for _ in range(args.warmup):
            prefill_once(0)
        clocks.start()
        p_iters = 5 if args.only == "all" else 1
        print(f"[bench] timed prefill starts after {ops.launch_count()} launches", file=sys.stderr, flush=True)
        p_ms = timed(prefill_once, p_iters) / p_iters
        p_flops = prefill_flops(cfg, layers, PROMPT)
        prefill = {"value": round(PROMPT / (p_ms / 1e3), 1), "tokens": PROMPT, "ms": round(p_ms, 3),
                   "frac": round(p_flops / (p_ms / 1e3) / compute_peak, 4)}
    else:
        clocks.start()
    if args.only == "prefill":
        print(json.dumps({"prefill": prefill, "clocks": clocks.summary()}))
        return 0

    # ---------------------------------------------------------------- decode
    main_pt = decode_point(args.batch, args.steps, args.warmup)
    clock_summary = clocks.summary()
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode_point(b, min(args.steps, 64), args.warmup)["tok_s"], 1)

    # ---------------------------------------------------------------- end to end through generate()
    # Host tokens in, host tokens out: every step copies its token ids and positions from pinned
    # host memory and reads the sampled ids back.  Prompts are read first; the timed window opens
    # when every request has produced `warmup` tokens (all are decoding by then) and closes when
    # the first one ends, so it holds decode steps of the full batch only.  It is a wall-clock
    # window, so it never holds fewer than E2E_MIN_STEPS steps, whatever --steps is.
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(args.steps, E2E_MIN_STEPS)
        e2e_warm = max(args.warmup, 8)         # the decode step's CUDA graph is captured in the first few steps
        prompts = [rng.integers(0, vocab, size=PROMPT).tolist() for _ in range(args.batch)]
        opts = SamplingOptions.greedy(num_predict=e2e_warm + e2e_steps)
        counts = [0] * args.batch
        marks = {}

        def on_token(i, tok):
            counts[i] += 1
            if "start" not in marks and min(counts) >= e2e_warm:
                marks["start"] = (time.perf_counter(), sum(counts), engine.h2d_bytes, engine.d2h_bytes, runner.steps_run)
            if "start" in marks and "end" not in marks and max(counts) >= e2e_warm + e2e_steps:
                marks["end"] = (time.perf_counter(), sum(counts), engine.h2d_bytes, engine.d2h_bytes, runner.steps_run)

        engine.generate(prompts, opts, on_token=on_token)
        (t0_, n0_, h0, d0, s0), (t1_, n1_, h1, d1, s1) = marks["start"], marks["end"]
        n_steps = max(1, s1 - s0)
        e2e = {"value": round((n1_ - n0_) / (t1_ - t0_), 1), "unit": "tokens/s",
               "h2d_bytes_per_step": round((h1 - h0) / n_steps, 1),
               "d2h_bytes_per_step": round((d1 - d0) / n_steps, 1), "steps": n_steps}

    achieved = main_pt["bytes"] / (main_pt["ms_per_step"] / 1e3) / 1e9
    # The reference publishes one figure: "about 7" tokens/s for one conversation with llama3.2:1b (a
    # 2-core CPU, quantised weights).  The like-for-like point here is decode at batch 1 of the 1B shape.
    single = points.get("decode_b1") if args.shape == "1b" and not f32 else None
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({model_name.replace('-shape', '').replace('llama', 'Llama')} shape)",
        "value": round(main_pt["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_pt["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(single / PUBLISHED_TOK_S, 1) if single else None,
        "vs_baseline_of": "decode_b1 over the reference's published single-conversation rate (CPU, quantised weights)",
        "dtype": "fp32" if f32 else "bf16", "data": "synthetic",
        "impl": "ours",
        "config": config,
        "e2e": e2e,
        "gpu_launches": int(main_pt["launches"]),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
