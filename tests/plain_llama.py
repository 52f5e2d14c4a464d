"""Plain, slow implementation of the Llama decoder, the oracle of the tests.

Whole sequences, no cache, float32 (float64 on request), one function for each
part, written from the reference's formulas; every function cites the file and
lines of Prathmesh234/simple-inference it restates.  It shares no code with the
package under test: it reads ``config.json`` and ``model.safetensors`` itself
and uses nothing but elementary torch operations.

``tests/golden/make_golden.py`` compared this file once with the reference's
own ``LlamaModel`` on the CPU (tiny random models); the outputs it wrote are
checked by ``tests/test_plain.py``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file


# ---------------------------------------------------------------------------
# model folder
# ---------------------------------------------------------------------------

def read_folder(folder, dtype=torch.float32):
    """(config dict, {tensor name: tensor in ``dtype``}) of a model folder."""
    folder = Path(folder)
    with open(folder / "config.json") as f:
        cfg = json.load(f)
    weights = {k: v.to(dtype) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, weights


def head_dim_of(cfg):
    # reference config.py:81: head_dim = hidden_size // num_attention_heads
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------

def rope_frequencies(head_dim, theta, scaling):
    """Rotation frequencies, float32 [head_dim/2].

    reference ops/rope.py:97-98: freq_i = 1 / theta^(2i/head_dim), float32;
    ops/rope.py:136-155: llama3 scaling by wavelength, per frequency in Python
    floats, stored back as float32; ops/rope.py:101: only rope_type "llama3"
    scales.
    """
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
    freqs = 1.0 / (theta ** (idx / head_dim))
    if not scaling or scaling.get("rope_type", "default") != "llama3":
        return freqs
    factor = scaling["factor"]
    low_f, high_f = scaling["low_freq_factor"], scaling["high_freq_factor"]
    orig = scaling["original_max_position_embeddings"]
    low_wl, high_wl = orig / low_f, orig / high_f
    out = []
    for f in freqs.tolist():
        wl = 2 * math.pi / f
        if wl < high_wl:
            out.append(f)
        elif wl > low_wl:
            out.append(f / factor)
        else:
            s = (orig / wl - low_f) / (high_f - low_f)
            out.append((1 - s) * f / factor + s * f)
    return torch.tensor(out, dtype=torch.float32)


def rope_tables(freqs, positions, dtype=torch.float32):
    """cos, sin [T, head_dim] for integer positions.

    reference ops/rope.py:108-118: angles = outer(positions as float32, freqs)
    in float32, duplicated cat([a, a]) to full width, then cos and sin.
    """
    pos = torch.as_tensor(positions, dtype=torch.float32)
    angles = torch.outer(pos, freqs)            # float32 product, as the reference
    angles = torch.cat([angles, angles], dim=-1).to(dtype)
    return angles.cos(), angles.sin()


def rotate_half(x):
    # reference ops/rope.py:167-184: cat(-x[half:], x[:half])
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x, cos, sin):
    """x [T, heads, D]; reference ops/rope.py:205-215: x*cos + rotate_half(x)*sin."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def rmsnorm(x, weight, eps):
    """reference ops/rmsnorm.py:41-46: x * rsqrt(mean(x^2) + eps) * weight."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def attention(q, k, v, positions, window=None, scale=None):
    """q [T, Hq, D], k, v [T, Hkv, D] (k already rotated) -> [T, Hq, D].

    reference kernels/attention_kernel.py:188 (query head h uses kv head
    h // groups), :223,289-290 (scores = q.k * 1/sqrt(D)),
    serving/paged_kv_cache.py:366-372 (key j allowed iff j <= query position),
    softmax over keys, O = P V.  ``window`` w (not in the reference) further
    restricts to keys with position > query position - w.
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    groups = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    pos = torch.as_tensor(positions)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty_like(q)
    for h in range(Hq):
        kh = h // groups
        scores = (q[:, h, :] @ k[:, kh, :].T) * scale
        scores = scores.masked_fill(~allowed, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, kh, :]
    return out


def attention_layer(x, w, prefix, cfg, positions, freqs, window=None):
    """reference ops/attention.py:128-151 and :223-226: q,k,v projections without
    bias, heads of head_dim columns, rope on q and k, attention, merge heads, o-proj."""
    T = x.shape[0]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, Hq, D)
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, Hkv, D)
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, Hkv, D)
    cos, sin = rope_tables(freqs, positions, x.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = attention(q, k, v, positions, window)
    return o.reshape(T, Hq * D) @ w[prefix + "o_proj.weight"].T


def mlp(x, w, prefix):
    """reference ops/mlp.py:117-128: down( silu(gate(x)) * up(x) ), silu(g) = g*sigmoid(g)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[prefix + "down_proj.weight"].T


def block(x, w, i, cfg, positions, freqs):
    """reference model/block.py:134-146: x + attn(norm(x)); then + mlp(norm(.))."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    x = x + attention_layer(rmsnorm(x, w[p + "input_layernorm.weight"], eps), w,
                            p + "self_attn.", cfg, positions, freqs)
    x = x + mlp(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return x


def forward(cfg, w, token_ids, run_order=None):
    """Logits [T, vocab] of one whole sequence.

    reference model/llama.py:174-186: embed, blocks in order, final norm, head;
    the head is the embedding matrix when tied (model/llama.py:111), otherwise
    lm_head.weight.  ``run_order`` (default 0..L-1) lists the layers to run.
    """
    dtype = w["model.embed_tokens.weight"].dtype
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = list(range(len(ids)))
    freqs = rope_frequencies(head_dim_of(cfg), cfg["rope_theta"], cfg.get("rope_scaling"))
    x = w["model.embed_tokens.weight"][ids]      # reference ops/embedding.py:57-60
    order = range(cfg["num_hidden_layers"]) if run_order is None else run_order
    for i in order:
        x = block(x, w, i, cfg, positions, freqs)
    x = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", True) \
        else w["lm_head.weight"]
    return (x @ head.T).to(dtype)


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

def _mix32(x):
    x &= 0xFFFFFFFF
    x ^= x >> 16
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x ^= x >> 15
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x ^= x >> 16
    return x


def uniform_from_hash(h):
    """float32 uniform strictly inside (0, 1) from 32-bit hashes: 23 bits plus a half."""
    import numpy as np
    return ((h.astype(np.uint64) >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) \
        * np.float32(1.0 / 8388608.0)


def gumbel_noise(seed, stream, counter, vocab):
    """float32 Gumbel noise per vocabulary entry from a counter-based hash."""
    import numpy as np
    base = _mix32(counter + _mix32(stream + _mix32(seed)))
    v = np.arange(vocab, dtype=np.uint64)

    def mix(x):
        x = x & 0xFFFFFFFF
        x ^= x >> np.uint64(16)
        x = (x * np.uint64(0x7FEB352D)) & np.uint64(0xFFFFFFFF)
        x ^= x >> np.uint64(15)
        x = (x * np.uint64(0x846CA68B)) & np.uint64(0xFFFFFFFF)
        x ^= x >> np.uint64(16)
        return x

    h = mix(np.uint64(base) ^ mix(v + np.uint64(0x9E3779B9)))
    u = uniform_from_hash(h)
    return torch.from_numpy(-np.log(-np.log(u, dtype=np.float32), dtype=np.float32))


def filter_logits(logits, temperature, top_k, top_p):
    """Scaled logits with everything outside top-k / top-p set to -inf.

    reference sampling.py:39-52 (divide by temperature), :68-83 (keep logits >=
    the k-th largest), :95-128 (sort descending, softmax, cumulative sum, drop
    where the sum BEFORE a token already exceeds p, so the crossing token stays).
    """
    z = logits.float() / temperature
    V = z.shape[-1]
    if 0 < top_k < V:
        kth = torch.topk(z, top_k).values[-1]
        z = torch.where(z < kth, torch.full_like(z, float("-inf")), z)
    if top_p < 1.0:
        if top_p <= 0.0:
            z = torch.where(z < z.max(), torch.full_like(z, float("-inf")), z)
        else:
            sz, idx = torch.sort(z, descending=True)
            cum = torch.softmax(sz, dim=-1).cumsum(-1)
            remove = cum > top_p
            remove[1:] = remove[:-1].clone()
            remove[0] = False
            mask = torch.zeros_like(remove)
            mask[idx] = remove
            z = z.masked_fill(mask, float("-inf"))
    return z


def sample(logits, temperature, top_k=0, top_p=1.0, seed=0, stream=0, counter=0):
    """One token from a row of logits; reference sampling.py:140-172 except the draw,
    which is argmax(z + Gumbel noise) instead of torch.multinomial."""
    if temperature == 0:
        return int(torch.argmax(logits.float()))       # sampling.py:159-160
    z = filter_logits(logits, temperature, top_k, top_p)
    g = gumbel_noise(seed, stream, counter, z.shape[-1])
    return int(torch.argmax(z + g))


def generate_greedy(cfg, w, prompt, n_new):
    """Greedy continuation by recomputing the whole sequence each time."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(cfg, w, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out
