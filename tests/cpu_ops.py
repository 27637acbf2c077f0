"""Torch-on-CPU stand-ins for ``hfee_b200.kernels.ops``, for tests only.

The product has no CPU path.  These doubles let the ``-m "not gpu"`` tests drive
the engine's host logic (batch flattening, block tables, page reuse, the schedule
of layers, the scheduler) end to end on a machine without a GPU; a test installs
them with ``monkeypatch`` over the functions of the ops module.
"""
import math

import torch


def embed(table, tokens, out, slot_of_token=None, feedback=None):
    tok = tokens.long()
    if feedback is not None:
        tok = torch.where(tok < 0, feedback[slot_of_token.long()].long(), tok)
    out.copy_(table[tok].float())


def rmsnorm(x, weight, out, eps, rows=None, add_unit=False):
    src = x if rows is None else x[rows.long()]
    w = weight + 1.0 if add_unit else weight
    scale = torch.rsqrt((src * src).mean(dim=1, keepdim=True) + eps)
    out.copy_((src * scale * w).to(out.dtype))


def rope_table(positions, inv_freq, out):
    ang = positions.double()[:, None] * inv_freq[None, :]
    out.copy_(torch.stack([ang.cos(), ang.sin()], dim=-1).float().reshape(out.shape))


def rope_cache_write(qkv, cs, positions, slot_of_token, q_out, k_pool, v_pool, block_table, page_size,
                     heads, kv_heads, head_dim, rope_dim, interleaved):
    n = qkv.shape[0]
    total = heads + (2 * kv_heads if k_pool is not None else 0)
    x = qkv.float().reshape(n, total, head_dim).clone()
    if cs is not None:
        half = rope_dim // 2
        c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
        rot = x[:, :heads + (kv_heads if k_pool is not None else 0)]
        if interleaved:
            a, b = rot[..., 0:rope_dim:2].clone(), rot[..., 1:rope_dim:2].clone()
            rot[..., 0:rope_dim:2] = a * c - b * s
            rot[..., 1:rope_dim:2] = a * s + b * c
        else:
            a, b = rot[..., :half].clone(), rot[..., half:rope_dim].clone()
            rot[..., :half] = a * c - b * s
            rot[..., half:rope_dim] = a * s + b * c
    q_out.copy_(x[:, :heads].reshape(n, heads * head_dim).to(q_out.dtype))
    if k_pool is None:
        return
    for i in range(n):
        pos, slot = int(positions[i]), int(slot_of_token[i])
        page = int(block_table[slot, pos // page_size])
        assert page >= 0, "write to a position without a page"
        k_pool[page, :, pos % page_size, :] = x[i, heads:heads + kv_heads].to(k_pool.dtype)
        v_pool[page, :, pos % page_size, :] = x[i, heads + kv_heads:].to(v_pool.dtype)


def swiglu(gate_up, out, granule=None):
    inter = out.shape[1]
    granule = granule or inter
    x = gate_up.float().reshape(gate_up.shape[0], inter // granule, 2, granule)
    g, u = x[:, :, 0].reshape(-1, inter), x[:, :, 1].reshape(-1, inter)
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def linear_swiglu(a, w_gate_up, out, granule, scratch):
    linear(a, w_gate_up, scratch)
    swiglu(scratch, out, granule)


def linear(a, w, out, accumulate=False):
    y = a.float() @ w.float().t()
    if accumulate:
        out.add_(y)
    else:
        out.copy_(y.to(out.dtype))


def paged_attention(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                    head_dim, scale, window=0, step=None, scratch=None):
    n = q.shape[0]
    group = heads // kv_heads
    for i in range(n):
        pos, slot = int(positions[i]), int(slot_of_token[i])
        lo = max(0, pos + 1 - window) if window else 0
        idx = torch.arange(lo, pos + 1)
        pages = block_table[slot, (idx // page_size).long()].long()
        assert (pages >= 0).all(), "read of a position whose page was given back"
        k = k_pool[pages, :, (idx % page_size).long(), :].float()      # [span, kv_heads, hd]
        v = v_pool[pages, :, (idx % page_size).long(), :].float()
        for h in range(heads):
            qh = q[i, h * head_dim:(h + 1) * head_dim].float()
            s = (k[:, h // group, :] @ qh) * scale
            p = torch.softmax(s, dim=0)
            out[i, h * head_dim:(h + 1) * head_dim] = (p @ v[:, h // group, :]).to(out.dtype)


def sample(logits, out, temperature=None, uniform=None, slots=None, feedback=None):
    _sample(logits, out, temperature, uniform)
    if feedback is not None:
        feedback[slots.long()] = out


def _sample(logits, out, temperature=None, uniform=None):
    for r in range(logits.shape[0]):
        t = float(temperature[r]) if temperature is not None else 0.0
        if t <= 0:
            out[r] = int(torch.argmax(logits[r]))
        else:
            p = torch.exp((logits[r].double() - logits[r].max().double()) / t)
            cum = torch.cumsum(p, 0)
            out[r] = int(torch.searchsorted(cum, float(uniform[r]) * float(cum[-1])).clamp(max=logits.shape[1] - 1))


def linear_normed(inp, w, out, accumulate=False):
    linear(inp if isinstance(inp, torch.Tensor) else inp.tensor(), w, out, accumulate)


def linear_swiglu_normed(inp, w_gate_up, out, granule, scratch):
    linear_swiglu(inp if isinstance(inp, torch.Tensor) else inp.tensor(), w_gate_up, out, granule, scratch)


def argmax(logits, out, scratch, slots=None, feedback=None):
    out.copy_(torch.argmax(logits, dim=1).to(torch.int32))
    if feedback is not None:
        feedback[slots.long()] = out


ALL = ("argmax", "linear_normed", "linear_swiglu_normed", "embed", "rmsnorm", "rope_table", "rope_cache_write", "swiglu", "linear", "linear_swiglu",
       "paged_attention", "sample")


def install(monkeypatch):
    from hfee_b200.kernels import ops
    import sys
    me = sys.modules[__name__]
    for name in ALL:
        monkeypatch.setattr(ops, name, getattr(me, name))
    monkeypatch.setattr(ops, "ARGMAX_CHUNKS", 1, raising=False)
    # kernel fusions have no double: the parts take their unfused paths
    monkeypatch.setattr(ops, "FUSE_ROPE_INTO_DECODE_ATTENTION", False, raising=False)
    monkeypatch.setattr(ops, "FUSE_ROPE_INTO_QKV", False, raising=False)
