"""The sampling chain on the device (repeat penalty over a ring of recent tokens, top-k, float64
probabilities, top-p, min-p, draw) against the host chain, which follows the reference's
sampler step by step; and generation with the reference's default options, pipelined on the
device, against the same generation through the host chain."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _params(opts, u):
    return [max(opts.temperature, 0.0), opts.top_k, float(np.float32(opts.top_p)), float(np.float32(opts.min_p)),
            float(np.float32(opts.repeat_penalty)) if opts.penalises else 1.0, opts.repeat_last_n if opts.penalises else 0,
            u, 0.0]


@pytest.mark.parametrize("vocab", [1000, 5000, 128256])
def test_device_chain_equals_host_chain(vocab):
    from hfee_b200.kernels import ops
    from hfee_b200.sampling import SamplingOptions
    from hfee_b200.sampling.sampler import sample_host
    g = torch.Generator().manual_seed(vocab)
    rng = np.random.default_rng(vocab)
    option_sets = [
        SamplingOptions(),                                                          # the reference's defaults
        SamplingOptions(temperature=0.0),                                           # greedy with the default penalty
        SamplingOptions(temperature=1.3, top_k=64, top_p=1.0, min_p=0.05, repeat_penalty=1.0),
        SamplingOptions(temperature=0.5, top_k=1, repeat_penalty=1.5, repeat_last_n=200),
        SamplingOptions(temperature=0.8, top_k=7, top_p=0.5, min_p=0.2, repeat_penalty=0.8, repeat_last_n=3),
        SamplingOptions.greedy(),
    ]
    rows = 2 * len(option_sets)
    logits = (torch.randn(rows, vocab, generator=g) * 3).to(DEV)
    logits[0, 5] = logits[0, 77] = 12.0                                             # ties: the lower id comes first
    logits[1, vocab - 1] = 15.0
    cap = ops.CHAIN_HISTORY
    slots = torch.tensor(rng.permutation(rows + 3)[:rows], dtype=torch.int32, device=DEV)
    history = torch.zeros(rows + 3, cap, dtype=torch.int32, device=DEV)
    history_len = torch.zeros(rows + 3, dtype=torch.int32, device=DEV)
    hist_host = []
    for r in range(rows):
        n = int(rng.integers(0, 600))                                               # some rings have wrapped around
        toks = rng.integers(0, vocab, size=n).tolist()
        if n > 3:
            toks[-1] = toks[-3] = int(torch.argmax(logits[r]))                      # the best token twice: penalised once
        hist_host.append(toks)
        s = int(slots[r])
        for i, t in enumerate(toks):
            history[s, i % cap] = t
        history_len[s] = n
    scratch = torch.empty(ops.chain_scratch_floats(rows, vocab), dtype=torch.float32, device=DEV)
    feedback = torch.full((rows + 3,), -7, dtype=torch.int32, device=DEV)
    for trial in range(6):
        us = rng.random(rows).tolist()
        opts = [option_sets[(r + trial) % len(option_sets)] for r in range(rows)]
        want = [sample_host(logits[r].cpu().numpy(), hist_host[r], opts[r], us[r]) for r in range(rows)]
        params = torch.tensor([_params(o, u) for o, u in zip(opts, us)], dtype=torch.float64, device=DEV)
        work = logits.clone()
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        lens_before = history_len.clone()
        ops.sample_chain(work, params, out, scratch, slots, feedback, history, history_len, penalise=True)
        got = out.tolist()
        assert got == want, (trial, got, want)
        assert feedback[slots.long()].tolist() == got
        assert (history_len - lens_before)[slots.long()].tolist() == [1] * rows
        for r in range(rows):                                                       # the choice joined the ring and the host copy
            s = int(slots[r])
            assert int(history[s, int(lens_before[s]) % cap]) == got[r]
            hist_host[r].append(got[r])


def test_generation_with_default_options_is_the_same_on_device_and_host(tiny_dirs):
    """The reference's default options (temperature 0.8, top-k 40, top-p 0.9, repeat penalty 1.1 over
    64 tokens) pipelined on the device give the tokens of the host chain, request by request, whatever
    the batch; a tiny cache (preemption) changes nothing either."""
    from hfee_b200 import Engine, SamplingOptions
    rng = np.random.default_rng(5)
    opts = SamplingOptions(seed=11, num_predict=40)
    for name in ("A", "B"):
        d = tiny_dirs[name]
        eng = Engine(d, dtype="float32", page_size=16, max_requests=4, max_context=256, max_batch_tokens=64)
        vocab = eng.runner.spec.vocab
        prompts = [rng.integers(0, vocab, size=n).tolist() for n in (5, 70, 33)]
        assert opts.device_chain and not opts.device_only
        dev = [r.token_ids for r in eng.generate(prompts, opts)]
        eng.pipeline = False
        assert [r.token_ids for r in eng.generate(prompts, opts)] == dev          # device chain, step by step
        eng.sampler.use_device_chain = False
        host = [r.token_ids for r in eng.generate(prompts, opts)]                 # logits to the host, numpy chain
        assert dev == host
        alone = [eng.generate([p], opts)[0].token_ids for p in prompts]
        assert alone == host
        eng.pipeline, eng.sampler.use_device_chain = True, True
        assert [eng.generate([p], opts)[0].token_ids for p in prompts] == host
        small = Engine(d, dtype="float32", page_size=16, max_requests=4, max_context=256, max_batch_tokens=64,
                       max_cache_tokens=160)
        got = small.generate(prompts, opts)
        assert [r.token_ids for r in got] == host
        assert sum(r.stats.preemptions for r in got) > 0          # a request came back and its ring was loaded again
