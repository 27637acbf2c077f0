"""Command line in the manner of hostfog/hfee's ``hfee`` (cmd/hfee/main.go:21-48, run.go):

    hfee-b200 run <model_dir> [prompt] [--verbose]     generate (one shot, or a prompt loop)
    hfee-b200 create <model_dir> <config.json>         write a model folder with random weights
    hfee-b200 show <model_dir>                         print the model's configuration
    hfee-b200 version

``run`` joins piped standard input and the prompt arguments like run.go:46-53, prints the
reply as it is generated and, with ``--verbose``, the counters of run.go:210-223.  Sampling
options carry the reference's names (``--temperature``, ``--top-k``, ``--top-p``, ``--min-p``,
``--repeat-penalty``, ``--repeat-last-n``, ``--seed``, ``--num-predict``, ``--stop``) and
defaults (internal/llm/sampler.go:23-34); ``HFEE_NUM_CTX`` and ``HFEE_NUM_PARALLEL`` are read as
in internal/server/server.go:46-57.  A model folder without ``tokenizer.json`` takes
``--prompt-ids 1,2,3`` and prints token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import List, Optional

USAGE = __doc__


def _sampling_args(ap: argparse.ArgumentParser) -> None:
    from .sampling import SamplingOptions
    d = SamplingOptions()
    ap.add_argument("--temperature", type=float, default=d.temperature)
    ap.add_argument("--top-k", type=int, default=d.top_k)
    ap.add_argument("--top-p", type=float, default=d.top_p)
    ap.add_argument("--min-p", type=float, default=d.min_p)
    ap.add_argument("--repeat-penalty", type=float, default=d.repeat_penalty)
    ap.add_argument("--repeat-last-n", type=int, default=d.repeat_last_n)
    ap.add_argument("--seed", type=int, default=d.seed)
    ap.add_argument("--num-predict", type=int, default=d.num_predict)
    ap.add_argument("--stop", action="append", default=[])


def _rate(n: int, seconds: float) -> str:
    return "-" if seconds <= 0 else f"{n / seconds:.2f} tokens/s"


def _generate_once(engine, prompt, opts, verbose: bool, load_seconds: float, as_ids: bool) -> List[int]:
    t0 = time.perf_counter()

    def show_id(_i: int, tok: int) -> None:
        print(tok, end=" ", flush=True)

    def show_text(_i: int, text: str) -> None:       # whole characters, never a stop string (text.go:16-78)
        print(text, end="", flush=True)

    res = engine.generate([prompt], opts, on_token=show_id if as_ids else None,
                          on_text=None if as_ids else show_text)[0]
    print("\n")
    if verbose:
        st = res.stats
        print(f"total duration:       {time.perf_counter() - t0 + load_seconds:.3f}s")
        print(f"load duration:        {load_seconds:.3f}s")
        print(f"prompt eval count:    {st.prompt_tokens} token(s)")
        print(f"prompt eval rate:     {_rate(st.prompt_tokens, st.prompt_seconds)}")
        print(f"eval count:           {st.eval_tokens} token(s)")
        print(f"eval rate:            {_rate(st.eval_tokens, st.eval_seconds)}")
        print(f"done reason:          {st.done_reason}\n")
    return res.token_ids


def cmd_run(argv: List[str]) -> int:
    ap = argparse.ArgumentParser(prog="hfee-b200 run", description="Generate with a model folder.")
    ap.add_argument("model")
    ap.add_argument("prompt", nargs="*")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--prompt-ids", help="comma separated token ids instead of text")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--num-ctx", type=int, default=None, help="context window (HFEE_NUM_CTX, default 4096)")
    ap.add_argument("--num-parallel", type=int, default=None, help="requests at once (HFEE_NUM_PARALLEL, default 4)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--device", default="cuda:0")
    _sampling_args(ap)
    a = ap.parse_args(argv)

    from . import Engine, SamplingOptions
    opts = SamplingOptions(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p,
                           repeat_penalty=a.repeat_penalty, repeat_last_n=a.repeat_last_n, seed=a.seed,
                           num_predict=a.num_predict, stop=list(a.stop))
    settings = {"dtype": a.dtype, "page_size": a.page_size, "device": a.device}
    if a.num_ctx is not None:
        settings["max_context"] = a.num_ctx
    if a.num_parallel is not None:
        settings["max_requests"] = a.num_parallel
    t0 = time.perf_counter()
    engine = Engine(a.model, **settings)
    load_seconds = time.perf_counter() - t0

    if a.prompt_ids:
        ids = [int(t) for t in a.prompt_ids.replace(" ", "").split(",") if t]
        _generate_once(engine, ids, opts, a.verbose, load_seconds, as_ids=True)
        return 0

    prompt = " ".join(a.prompt)
    if not sys.stdin.isatty():                                   # run.go:46-53
        piped = sys.stdin.read().strip()
        prompt = (piped + "\n\n" + prompt).strip()
    if engine.tokenizer is None:
        print("Error: this model folder has no tokenizer.json; pass --prompt-ids 1,2,3", file=sys.stderr)
        return 1
    if prompt:
        _generate_once(engine, prompt, opts, a.verbose, load_seconds, as_ids=False)
        return 0
    return _repl(engine, opts, a.verbose)


def _repl(engine, opts, verbose: bool) -> int:
    """A prompt loop after run.go:69-155: ``\"\"\"`` starts and ends a multi-line message, /clear
    forgets the conversation, /bye exits.  The conversation is kept as token ids, so a follow-up
    continues from everything said so far."""
    print('Type a message, or /? for help. Use """ to begin a multi-line message.')
    history: List[int] = []
    while True:
        try:
            line = input(">>> ").strip()
        except EOFError:
            print()
            return 0
        if line.startswith('"""'):
            parts = [line[3:]]
            while not parts[-1].rstrip().endswith('"""') or (len(parts) == 1 and not parts[0]):
                try:
                    parts.append(input("... "))
                except EOFError:
                    break
            line = "\n".join(parts).rstrip()
            line = line[:-3].strip() if line.endswith('"""') else line
        if not line:
            continue
        if line in ("/bye", "/exit"):
            return 0
        if line in ("/?", "/help"):
            print('  /clear   Forget the conversation\n  /bye     Exit\n  """      Start or end a multi-line message')
            continue
        if line == "/clear":
            history = []
            print("Cleared session context")
            continue
        if line.startswith("/"):
            print(f"Unknown command {line.split()[0]}. Type /? for help.")
            continue
        ids = engine.encode(line) if not history else engine.tokenizer.encode(line)
        prompt = history + ids
        if len(prompt) >= engine.max_context:
            print("Error: the conversation no longer fits the context window; /clear starts over", file=sys.stderr)
            continue
        out = _generate_once(engine, prompt, opts, verbose, 0.0, as_ids=False)
        history = prompt + out


def cmd_create(argv: List[str]) -> int:
    ap = argparse.ArgumentParser(prog="hfee-b200 create",
                                 description="Write config.json and model.safetensors with random weights.")
    ap.add_argument("model_dir")
    ap.add_argument("config", help="a config.json naming the architecture and its sizes")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    a = ap.parse_args(argv)
    from .weights import write_random_model
    with open(a.config) as f:
        cfg = json.load(f)
    write_random_model(a.model_dir, cfg, seed=a.seed, dtype=a.dtype)
    print(f"wrote {a.model_dir} (seed {a.seed}, {a.dtype})")
    return 0


def cmd_show(argv: List[str]) -> int:
    ap = argparse.ArgumentParser(prog="hfee-b200 show")
    ap.add_argument("model")
    a = ap.parse_args(argv)
    from .config import resolve_model_dir
    from .parts.model import model_tensor_needs
    arch, cfg = resolve_model_dir(a.model)
    spec = arch.build_spec(cfg)
    params = 0
    for need in model_tensor_needs(spec).values():
        if need.optional:               # a head of its own that a tied model may store but does not need
            continue
        n = 1
        for s in need.shape:
            n *= s
        params += n
    print(f"architecture   {arch.name}")
    print(f"parameters     {params:,}")
    for k, v in cfg.to_dict().items() if hasattr(cfg, "to_dict") else []:
        if k not in ("architectures",):
            print(f"{k:<28} {v}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("help", "--help", "-h"):
        print(USAGE)
        return 0 if argv else 1
    cmd, rest = argv[0], argv[1:]
    try:
        if cmd == "run":
            return cmd_run(rest)
        if cmd == "create":
            return cmd_create(rest)
        if cmd == "show":
            return cmd_show(rest)
        if cmd in ("version", "--version", "-v"):
            from . import __version__
            print("hfee-b200 version", __version__)
            return 0
    except (ValueError, RuntimeError, OSError) as e:
        print("Error:", e, file=sys.stderr)
        return 1
    print(f"unknown command {cmd!r}\n\n{USAGE}", file=sys.stderr)
    return 1


if __name__ == "__main__":
    sys.exit(main())
