"""The host sampling chain and the plain implementation's own parts (CPU)."""
import math

import numpy as np
import pytest

import plain_llama as plain
from hfee_b200.sampling import SamplingOptions, apply_repeat_penalty, sample_host, uniform


def test_defaults_are_the_references():
    o = SamplingOptions()
    assert (o.temperature, o.top_k, o.top_p, o.min_p, o.repeat_penalty, o.repeat_last_n, o.seed, o.num_predict) == \
           (0.8, 40, 0.9, 0.0, 1.1, 64, -1, -1)
    g = SamplingOptions.greedy(5)
    assert g.temperature == 0 and not g.penalises and g.device_only and g.num_predict == 5
    assert not o.device_only and SamplingOptions(temperature=0.7, top_k=0, top_p=1.0, repeat_penalty=1.0).device_only


def test_which_options_the_device_kernels_take():
    o = SamplingOptions()
    assert o.device_chain and not o.device_only                        # the reference's defaults: the chain kernels
    assert SamplingOptions.greedy().device_chain and SamplingOptions.greedy().device_only
    assert SamplingOptions(temperature=0.0).device_chain                # greedy with the default penalty: k = 1 after the penalty
    assert not SamplingOptions(top_k=65).device_chain and SamplingOptions(top_k=64).device_chain
    assert not SamplingOptions(top_k=0).device_chain                    # top-p over all tokens needs the full sort: host
    assert not SamplingOptions(repeat_last_n=-1).device_chain and not SamplingOptions(repeat_last_n=257).device_chain
    assert SamplingOptions(repeat_last_n=256).device_chain and SamplingOptions(repeat_last_n=0, top_k=5).device_chain


def test_equal_logits_are_taken_in_the_order_of_their_ids():
    logits = np.zeros(50, dtype=np.float32)
    logits[[40, 7, 23]] = 3.0
    o = SamplingOptions(temperature=1.0, top_k=2, top_p=1.0, repeat_penalty=1.0)
    # the two candidates are ids 7 and 23 (not 40), each with probability one half, 7 first
    assert [sample_host(logits, [], o, u) for u in (0.1, 0.49, 0.51, 0.99)] == [7, 7, 23, 23]


def test_uniform_is_a_pure_function_in_unit_interval():
    xs = [uniform(3, 0, i) for i in range(2000)]
    assert all(0 <= x < 1 for x in xs) and abs(np.mean(xs) - 0.5) < 0.03
    assert uniform(3, 0, 5) == uniform(3, 0, 5) != uniform(4, 0, 5)


def test_greedy_takes_the_first_maximum_and_penalty_applies_before_it():
    logits = np.array([1.0, 5.0, 5.0, -2.0], dtype=np.float32)
    assert sample_host(logits, [], SamplingOptions.greedy(), 0.3) == 1
    o = SamplingOptions(temperature=0.0, repeat_penalty=2.0, repeat_last_n=2)
    # only the last 2 of the history count; 5.0 / 2 = 2.5 loses against the other 5.0
    assert sample_host(logits, [1, 3, 1], o, 0.0) == 2
    l2 = logits.copy()
    apply_repeat_penalty(l2, [3, 3, 0], SamplingOptions(repeat_penalty=2.0, repeat_last_n=-1))
    assert l2.tolist() == [0.5, 5.0, 5.0, -4.0]                       # each id once; negative logits multiplied


def test_top_k_top_p_min_p_and_draw():
    logits = np.log(np.array([0.5, 0.25, 0.125, 0.0625, 0.0625], dtype=np.float64)).astype(np.float32)
    base = dict(temperature=1.0, repeat_penalty=1.0, top_k=0, top_p=1.0, min_p=0.0)
    # plain temperature: inverse CDF over the probabilities in descending order
    assert [sample_host(logits, [], SamplingOptions(**base), u) for u in (0.0, 0.49, 0.51, 0.76, 0.99)] == [0, 0, 1, 2, 4]
    # top_k 2 renormalises over {0.5, 0.25}
    assert [sample_host(logits, [], SamplingOptions(**{**base, "top_k": 2}), u) for u in (0.6, 0.7)] == [0, 1]
    # top_p 0.7: smallest prefix whose mass reaches 0.7 is {0.5, 0.25}
    assert sample_host(logits, [], SamplingOptions(**{**base, "top_p": 0.7}), 0.99) == 1
    # min_p 0.3: cut where p < 0.3 * p_max = 0.15 -> keeps {0.5, 0.25}
    assert sample_host(logits, [], SamplingOptions(**{**base, "min_p": 0.3}), 0.99) == 1
    # a low temperature sharpens: 0.1 -> essentially greedy
    assert sample_host(logits, [], SamplingOptions(**{**base, "temperature": 0.1}), 0.9) == 0


def test_plain_parts():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 8))
    w = rng.normal(size=8)
    y = plain.rms_norm(x, w, 1e-5)
    assert np.allclose(y[1], x[1] / math.sqrt(np.mean(x[1] ** 2) + 1e-5) * w)
    assert np.allclose(plain.softmax(np.array([1.0, 2.0, 3.0])).sum(), 1.0)
    g, u = np.array([0.0, 2.0]), np.array([3.0, 0.5])
    assert np.allclose(plain.swiglu(g, u), [0.0, 2.0 / (1 + math.exp(-2.0)) * 0.5])
    # rotation keeps norms, position 0 is the identity, and the two pairings differ only by a permutation
    inv = plain.rope_inv_freq(8, 10000.0)
    v = rng.normal(size=(2, 16))
    assert np.allclose(plain.rope(v, 2, 8, [0, 0], inv, "half"), v)
    r = plain.rope(v, 2, 8, [5, 9], inv, "half")
    assert np.allclose(np.linalg.norm(r, axis=1), np.linalg.norm(v, axis=1))
    perm = [0, 4, 1, 5, 2, 6, 3, 7]                      # interleaved slot j holds half-layout element perm[j]
    vi = v.reshape(2, 2, 8)[:, :, perm].reshape(2, 16)
    ri = plain.rope(vi, 2, 8, [5, 9], inv, "interleaved")
    assert np.allclose(ri.reshape(2, 2, 8)[:, :, np.argsort(perm)].reshape(2, 16), r)
    # causal attention: the first token attends to itself only; a window of 1 returns v itself
    q, k, vv = rng.normal(size=(4, 8)), rng.normal(size=(4, 4)), rng.normal(size=(4, 4))
    out = plain.attention(q, k, vv, heads=2, kv_heads=1, head_dim=4)
    assert np.allclose(out[0], np.concatenate([vv[0], vv[0]]))
    assert np.allclose(plain.attention(q, k, vv, 2, 1, 4, window=1), np.concatenate([vv, vv], axis=1))


def test_plain_bf16_rounding_is_round_to_nearest_even():
    import torch
    a = np.array([1.0, 1.00390625, 1.01171875, -3.3333, 1e-8, 65504.0], dtype=np.float32)
    want = torch.tensor(a).to(torch.bfloat16).float().numpy()
    assert np.array_equal(plain.to_bf16_grid(a).astype(np.float32), want)
