"""Plain torch twins of the CUDA kernels' Python faces, for tests only.

Each function has the signature of its namesake in ``simple_inference_b200.ops``
and does the same thing with elementary torch operations on whatever device
its tensors live on.  Two uses: (1) the GPU tests compare every kernel with its
twin at sizes other than the engine's; (2) the CPU tests swap the twins in for
the kernels (``use_twins``) so that the step function, the cache and the
scheduler can be exercised on a machine without a GPU.  The package itself
never imports this file and has no CPU path.
"""

from __future__ import annotations

import contextlib
import math

import torch

from tests import plain_llama


def embed_gather(table, ids, out):
    out.copy_(table[ids[: out.shape[0]].long()].float())
    return out


def rmsnorm(residual, weight, eps, out, delta=None, rows=None):
    n = out.shape[0]
    if rows is None:
        x = residual[:n]
        if delta is not None:
            x += delta[:n].float()
    else:
        idx = rows[:n].long()
        x = residual[idx]
        if delta is not None:
            x = x + delta[idx].float()
    var = x.pow(2).mean(dim=-1, keepdim=True)
    out.copy_((x * torch.rsqrt(var + eps) * weight.float()).to(out.dtype))
    return out


def swiglu(gate_up, out):
    inter = out.shape[1]
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))
    return out


def linear(x, weight, out):
    out.copy_((x.float() @ weight.float().T).to(out.dtype))
    return out


def rope_kv_store(qkv, positions, inv_freq, kv_slots, pool, num_q_heads, num_kv_heads, head_dim,
                  page_size, write_kv):
    n = qkv.shape[0]
    qw, kw = num_q_heads * head_dim, num_kv_heads * head_dim
    angles = torch.outer(positions[:n].float(), inv_freq)
    angles = torch.cat([angles, angles], dim=-1)
    cos, sin = angles.cos(), angles.sin()
    q = qkv[:, :qw].float().view(n, num_q_heads, head_dim)
    k = qkv[:, qw:qw + kw].float().view(n, num_kv_heads, head_dim)
    v = qkv[:, qw + kw:].view(n, num_kv_heads, head_dim)
    q = plain_llama.apply_rope(q, cos, sin)
    k = plain_llama.apply_rope(k, cos, sin)
    qkv[:, :qw] = q.reshape(n, qw).to(qkv.dtype)
    if not write_kv:
        return
    slots = kv_slots[:n].long()
    page, off = slots // page_size, slots % page_size
    pool[page, 0, :, off, :] = k.to(pool.dtype)
    pool[page, 1, :, off, :] = v.to(pool.dtype)


def attention_generic(q, pool, block_table, tok_seq, positions, out, num_q_heads, num_kv_heads,
                      head_dim, scale, window):
    n = out.shape[0]
    page_size = pool.shape[3]
    groups = num_q_heads // num_kv_heads
    for t in range(n):
        s, p = int(tok_seq[t]), int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1, device=pool.device)
        pages = block_table[s][js // page_size].long()
        offs = js % page_size
        k = pool[pages, 0, :, offs, :].float()   # [keys, Hkv, D]
        v = pool[pages, 1, :, offs, :].float()
        qt = q[t, :num_q_heads * head_dim].float().view(num_q_heads, head_dim)
        for h in range(num_q_heads):
            kh = h // groups
            sc = (k[:, kh, :] @ qt[h]) * scale
            pr = torch.softmax(sc, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (pr @ v[:, kh, :]).to(out.dtype)
    return out


def paged_attention(q, pool, ctx, plan, group, out, num_q_heads, num_kv_heads, head_dim, scale, window):
    return attention_generic(q, pool, ctx.block_tables[group], ctx.tok_seq, ctx.positions, out,
                             num_q_heads, num_kv_heads, head_dim, scale, window)


def sample(logits, temperature, top_k, top_p, seed, stream_id, counter, out):
    for r in range(logits.shape[0]):
        out[r] = plain_llama.sample(
            logits[r].cpu(), float(temperature[r]), int(top_k[r]), float(top_p[r]),
            int(seed[r]) & 0xFFFFFFFF, int(stream_id[r]) & 0xFFFFFFFF, int(counter[r]) & 0xFFFFFFFF)
    return out


_NAMES = ["embed_gather", "rmsnorm", "swiglu", "linear", "rope_kv_store", "attention_generic",
          "paged_attention", "sample"]


@contextlib.contextmanager
def use_twins():
    """Swap the twins in for the kernels (CPU tests of the host-side logic)."""
    from simple_inference_b200 import ops
    saved = {n: getattr(ops, n) for n in _NAMES}
    try:
        for n in _NAMES:
            setattr(ops, n, globals()[n])
        yield
    finally:
        for n, f in saved.items():
            setattr(ops, n, f)
