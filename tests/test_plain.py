"""The plain implementation itself (no GPU): anchored to the reference, and self-consistent."""

import json
import math
from pathlib import Path

import pytest
import torch

from simple_inference_b200.weights import write_random_model
from tests import plain_llama
from tests.conftest import TINY_A, TINY_B, random_ids

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_matches_outputs_of_the_reference_model(name, tmp_path):
    """golden_*.json holds what the reference's own LlamaModel computed (make_golden.py)."""
    rec = json.loads((GOLDEN / f"golden_{name}.json").read_text())
    write_random_model(tmp_path, rec["config"], seed=rec["weights_seed"])
    cfg, w = plain_llama.read_folder(tmp_path)
    logits = plain_llama.forward(cfg, w, rec["prompt"])
    want = torch.tensor(rec["reference_logits_last4_first16"])
    assert (logits[-4:, :16] - want).abs().max() < 5e-6
    assert logits.argmax(-1).tolist() == rec["reference_argmax"]


def test_llama3_scaling_bands():
    # reference ops/rope.py:136-155: short wavelengths untouched, long ones divided by factor
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    base = plain_llama.rope_frequencies(32, 500000.0, None)
    scaled = plain_llama.rope_frequencies(32, 500000.0, sc)
    wl = 2 * math.pi / base
    assert torch.equal(scaled[wl < 16], base[wl < 16])
    assert torch.allclose(scaled[wl > 64], base[wl > 64] / 8.0)
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and ((scaled[mid] < base[mid]) & (scaled[mid] > base[mid] / 8.0)).all()
    assert torch.equal(plain_llama.rope_frequencies(32, 500000.0, {"rope_type": "default"}), base)


def test_causality_and_prefix_property(tmp_path):
    write_random_model(tmp_path, TINY_B, seed=4)
    cfg, w = plain_llama.read_folder(tmp_path)
    ids = random_ids(30, cfg["vocab_size"], 1)
    full = plain_llama.forward(cfg, w, ids)
    part = plain_llama.forward(cfg, w, ids[:11])
    assert (full[:11] - part).abs().max() < 1e-5      # later tokens do not change earlier logits
    other = list(ids)
    other[20] = (other[20] + 1) % cfg["vocab_size"]
    changed = plain_llama.forward(cfg, w, other)
    assert (changed[:20] - full[:20]).abs().max() < 1e-5
    assert (changed[20:] - full[20:]).abs().max() > 1e-4


def test_float64_agrees_with_float32(tmp_path):
    write_random_model(tmp_path, TINY_A, seed=4)
    cfg, w32 = plain_llama.read_folder(tmp_path)
    _, w64 = plain_llama.read_folder(tmp_path, torch.float64)
    ids = random_ids(50, cfg["vocab_size"], 2)
    assert (plain_llama.forward(cfg, w32, ids).double()
            - plain_llama.forward(cfg, w64, ids)).abs().max() < 1e-5


def test_attention_window_and_groups():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(9, 4, 16, generator=g)
    k = torch.randn(9, 2, 16, generator=g)
    v = torch.randn(9, 2, 16, generator=g)
    pos = list(range(9))
    full = plain_llama.attention(q, k, v, pos)
    win = plain_llama.attention(q, k, v, pos, window=3)
    assert torch.allclose(full[:3], win[:3], atol=1e-6) and not torch.allclose(full[5], win[5])
    # query head 1 reads kv head 0, query head 2 reads kv head 1
    q2 = q.clone()
    q2[:, 2] = q[:, 1]
    assert not torch.allclose(plain_llama.attention(q2, k, v, pos)[:, 2], full[:, 1])
    assert torch.allclose(full[0, 0], v[0, 0], atol=1e-6)   # the first token sees only itself


def test_sampling_rules():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(500, generator=g) * 2
    assert plain_llama.sample(logits, 0.0, top_k=5, top_p=0.1) == int(logits.argmax())
    z = plain_llama.filter_logits(logits, 1.0, 7, 1.0)
    assert int(torch.isfinite(z).sum()) == 7
    z = plain_llama.filter_logits(logits, 0.7, 0, 0.5)
    kept = torch.isfinite(z)
    probs = torch.softmax(logits / 0.7, -1)
    order = probs.argsort(descending=True)
    n = int(kept.sum())
    assert kept[order[:n]].all() and probs[order[:n]].sum() >= 0.5 > probs[order[:n - 1]].sum()
    assert int(torch.isfinite(plain_llama.filter_logits(logits, 1.0, 0, 0.0)).sum()) == 1
    draws = {plain_llama.sample(logits, 1.0, seed=1, stream=0, counter=c) for c in range(40)}
    assert len(draws) > 5
    assert plain_llama.sample(logits, 1.0, seed=1, counter=3) == plain_llama.sample(logits, 1.0, seed=1, counter=3)
    # the draw follows softmax: frequencies of the two likeliest tokens over many counters
    small = torch.tensor([2.0, 1.0, 0.0, -1.0])
    counts = torch.zeros(4)
    for c in range(3000):
        counts[plain_llama.sample(small, 1.0, seed=9, counter=c)] += 1
    assert (counts / 3000 - torch.softmax(small, -1)).abs().max() < 0.03


def test_uniform_of_every_hash_lies_strictly_inside_the_unit_interval():
    """The Gumbel draw takes -log(-log(u)): u = 0 or u = 1 would give infinite noise and make
    its token win (or lose) whatever its logit.  The uniform keeps 23 bits of the hash; sweep
    all of them, with the dropped low bits both clear and set."""
    import numpy as np
    top = np.arange(1 << 23, dtype=np.uint64) << np.uint64(9)
    for low in (0, 0x1FF):
        u = plain_llama.uniform_from_hash(top | np.uint64(low))
        assert u.dtype == np.float32
        assert float(u.min()) > 0.0 and float(u.max()) < 1.0
        noise = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
        assert np.isfinite(noise).all()
    assert np.isfinite(plain_llama.gumbel_noise(3, 1, 2, 200_000).numpy()).all()


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_one_wrong_key_moves_the_logits_by_more_than_the_bfloat16_tolerance(name, tmp_path):
    """The point of a tolerance: a fault must not fit under it.  Take the key and value of one
    token from another token, in one layer, and the logits of the plain model move by more
    than the bound that the bfloat16 replay tests allow between engine and plain model."""
    from tests.conftest import TINY
    from tests.test_replay_gpu import TOL
    write_random_model(tmp_path, TINY[name], seed=11 + "ABCD".index(name))
    cfg, w = plain_llama.read_folder(tmp_path)
    ids = random_ids(97, cfg["vocab_size"], 101)
    base = plain_llama.forward(cfg, w, ids)
    plain_attention = plain_llama.attention
    try:
        for layer in range(cfg["num_hidden_layers"]):
            for wrong, taken_from in ((10, 50), (40, 3)):
                calls = [0]

                def with_one_wrong_key(q, k, v, positions, window=None, scale=None):
                    if calls[0] == layer:
                        k, v = k.clone(), v.clone()
                        k[wrong], v[wrong] = k[taken_from], v[taken_from]
                    calls[0] += 1
                    return plain_attention(q, k, v, positions, window, scale)

                plain_llama.attention = with_one_wrong_key
                moved = float((plain_llama.forward(cfg, w, ids) - base).abs().max())
                assert moved > 1.2 * TOL["bfloat16"], (layer, wrong, moved)
    finally:
        plain_llama.attention = plain_attention


def test_sampling_filters_keep_what_the_reference_keeps():
    """golden_sampling.json holds which entries the reference's own filter_top_k and
    filter_top_p (sampling.py:69-128, after its division by the temperature, :39-52) leave
    finite, for rows with ties at the top and across the k-th place and for a peaked row."""
    rec = json.loads((GOLDEN / "golden_sampling.json").read_text())
    rows = torch.tensor(rec["rows"])
    for (temperature, top_k, top_p), per_row in zip(rec["settings"], rec["reference_kept"]):
        for row, want in zip(rows, per_row):
            z = plain_llama.filter_logits(row, temperature, int(top_k), top_p)
            assert torch.isfinite(z).nonzero().flatten().tolist() == want, (temperature, top_k, top_p)
            assert torch.equal(z[want], (row / temperature)[want])
