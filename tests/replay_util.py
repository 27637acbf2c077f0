"""Helpers shared by the replay tests: build traces over given sequences, run them
through the engine's step function, collect logits per (request, position)."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def rel_err(got, ref):
    """Largest absolute difference relative to the largest reference magnitude."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(got - ref)) / (np.max(np.abs(ref)) + 1e-30))


# A trace is a list of steps; a step is {"entries": [(rid, tokens, want)], "end": [rid]}.
def whole(seqs):
    """Each request alone and whole, one step per request."""
    return [{"entries": [(i, s, list(range(len(s))))], "end": [i]} for i, s in enumerate(seqs)]


def prefill_then_decode(seqs, tail=32):
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for i, s in enumerate(seqs):
        head = max(len(s) - tail, 1)
        steps.append({"entries": [(i, s[:head], list(range(head)))], "end": []})
        for t in range(head, len(s)):
            steps.append({"entries": [(i, s[t:t + 1], [0])], "end": [i] if t == len(s) - 1 else []})
        if head == len(s):
            steps[-1]["end"] = [i]
    return steps


def portions(seqs, sizes=(7, 2, 16, 3, 2, 33, 2, 5, 64, 2)):
    """Each request alone in portions of changing size, down to two tokens."""
    steps = []
    for i, s in enumerate(seqs):
        at, k = 0, 0
        while at < len(s):
            n = min(sizes[k % len(sizes)], len(s) - at)
            k += 1
            steps.append({"entries": [(i, s[at:at + n], list(range(n)))], "end": [i] if at + n == len(s) else []})
            at += n
    return steps


def mixed(seqs, live=4, seed=0, chunk_sizes=(2, 3, 5, 9, 16, 31)):
    """Up to ``live`` requests at a time: each step gives every live request either one
    token (once it is past a random point: 'decoding') or a portion of random size;
    a request that ends is replaced by the next one, so its pages are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(range(len(seqs)))
    active = {}
    steps = []
    switch = {i: int(rng.integers(1, max(2, len(s)))) for i, s in enumerate(seqs)}
    while waiting or active:
        while waiting and len(active) < live:
            active[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(active):
            if rng.random() < 0.2 and len(active) > 1:
                continue                                    # left out of this step, goes on later
            at, s = active[rid], seqs[rid]
            if at >= switch[rid]:
                n = 1
            else:
                n = int(min(rng.choice(chunk_sizes), switch[rid] - at))
            n = min(n, len(s) - at)
            entries.append((rid, s[at:at + n], list(range(n))))
            active[rid] = at + n
            if at + n == len(s):
                end.append(rid)
                del active[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def batched_decode(seqs, tails, live=None, want_head="all"):
    """Every request's head (all but its last ``tails[i]`` tokens) in a step of its own, then
    decode-only steps that give every live request one token.  Requests end after their last
    token, so with different tails the batch shrinks step by step; with ``live`` smaller than
    ``len(seqs)`` the waiting requests join as others leave (their head in a step of its own
    between the decode steps, in the slot that just became free).  ``want_head``: "all" asks for
    the logits of every head position, "last" for the last one only."""
    live = live or len(seqs)
    waiting = list(range(len(seqs)))
    active = {}
    steps = []
    while waiting or active:
        while waiting and len(active) < live:
            rid = waiting.pop(0)
            head = max(len(seqs[rid]) - tails[rid], 1)
            want = list(range(head)) if want_head == "all" else [head - 1]
            done = head == len(seqs[rid])
            steps.append({"entries": [(rid, seqs[rid][:head], want)], "end": [rid] if done else []})
            if not done:
                active[rid] = head
        if not active:
            continue
        entries, end = [], []
        for rid in list(active):
            at = active[rid]
            entries.append((rid, seqs[rid][at:at + 1], [0]))
            active[rid] = at + 1
            if at + 1 == len(seqs[rid]):
                end.append(rid)
                del active[rid]
        steps.append({"entries": entries, "end": end})
    return steps


def expected_rows(refs, steps):
    """For traces that do not ask for every position: {rid: reference rows in the order the trace
    asks for them}."""
    at = {}
    out = {}
    for st in steps:
        for rid, toks, want in st["entries"]:
            base = at.get(rid, 0)
            for w in want:
                out.setdefault(rid, []).append(refs[rid][base + w])
            at[rid] = base + len(toks)
    return {rid: np.stack(v) for rid, v in out.items()}


def run_in_process(runner, steps):
    """Feed a trace to a ModelRunner; returns {rid: [logits rows in position order]}."""
    from hfee_b200 import StepEntry
    slots, out = {}, {}
    for st in steps:
        entries = []
        for rid, toks, want in st["entries"]:
            if rid not in slots:
                slots[rid] = runner.open()
            entries.append(StepEntry(slots[rid], toks, want))
        logits = runner.step(entries)
        if logits is not None:
            rows = logits.float().cpu().numpy()
            at = 0
            for rid, toks, want in st["entries"]:
                for _ in want:
                    out.setdefault(rid, []).append(rows[at].copy())
                    at += 1
        for rid in st["end"]:
            runner.close(slots.pop(rid))
        runner.cache.check_invariants()
    return {rid: np.stack(v) for rid, v in out.items()}


def run_trace_binary(model_dir, dtype, steps, out_dir, max_tokens, vocab, extra_args=(), env=None):
    """Feed a trace to bin/trace_run over its standard input, waiting for ``done``
    after each step as the contract requires; returns {rid: rows}."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), *extra_args]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    out = {}
    try:
        for no, st in enumerate(steps):
            rec = {"step": no, "entries": [{"id": str(r), "tokens": list(map(int, t)), "want": list(w)}
                                           for r, t, w in st["entries"]], "end": [str(r) for r in st["end"]]}
            p.stdin.write(json.dumps(rec) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {no}", f"expected 'done {no}', got {line!r}"
            wanted = sum(len(w) for _, _, w in st["entries"])
            path = os.path.join(out_dir, f"{no}.f32")
            if wanted:
                rows = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
                at = 0
                for rid, toks, want in st["entries"]:
                    for _ in want:
                        out.setdefault(rid, []).append(rows[at])
                        at += 1
            else:
                assert not os.path.exists(path)
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    return {rid: np.stack(v) for rid, v in out.items()}
