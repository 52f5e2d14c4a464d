"""Each part alone on the GPU against the plain functions, and the parts' generality:
a window, another position encoding, a run order that repeats a layer or shares a cache."""

import math

import pytest
import torch

from tests import plain_llama
from tests.conftest import random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


class Harness:
    """A cache, a batch builder and a workspace around parts under test."""

    def __init__(self, specs, dtype, page_size=4, pages=80, max_tokens=256, max_seqs=4,
                 max_seq_len=256, parts=()):
        from simple_inference_b200.cache import CacheManager
        from simple_inference_b200.engine.batch import BatchBuilder, Workspace
        from simple_inference_b200.parts import Runtime
        self.rt = Runtime(torch.device(DEV), dtype)
        # a request brings at most 64 tokens per step; a batch may hold max_tokens in all
        self.cache = CacheManager(specs, page_size, pages, max_seqs, 64, dtype, DEV)
        planners = {cls.name: cls for part in parts for cls in part.step_planners()}
        self.builder = BatchBuilder(self.cache, max_tokens, max_seqs, max_seq_len, self.rt.device,
                                    planners=planners)
        self.ws = Workspace(self.rt.device, max_tokens)
        self.views = self.cache.layer_caches()

    def ctx(self, entries):
        """entries: [(request, n_tokens)]; admits unknown requests for 150 tokens."""
        from simple_inference_b200.engine.batch import StepEntry
        for r, n in entries:
            if not self.cache.is_admitted(r):
                self.cache.admit(r, 150)
        starts = [self.cache.extend(r, n) for r, n in entries]
        return self.builder.build([StepEntry(r, [0] * n, []) for r, n in entries], starts, self.ws)


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


# tolerances relative to the largest magnitude of the expected tensor: float32 differs by
# summation order, bfloat16 by a handful of roundings of 2^-8 each
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def close(got, want, dtype):
    scale = max(1.0, float(want.abs().max()))
    return float((got - want).abs().max()) < TOL[dtype] * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from simple_inference_b200.parts import NORMS, PartSpec
    h = Harness([], dtype)
    norm = NORMS.build(PartSpec("rmsnorm", {"hidden_size": 120, "eps": 3e-6}))
    assert norm.tensors()["weight"].shape == (120,)
    w = 1 + rnd(120, seed=1, scale=0.1)
    norm.bind({"weight": w.to(DEV).to(dtype)}, h.rt)
    x, d = rnd(9, 120, seed=2), rnd(9, 120, seed=3).to(dtype)
    ctx = h.ctx([("a", 9)])
    res = x.to(DEV)
    out = norm.add_forward(res, d.to(DEV), ctx)
    assert (res.cpu() - (x + d.float())).abs().max() < 1e-6
    want = plain_llama.rmsnorm(x + d.float(), w.to(dtype).float(), 3e-6)
    assert close(out.float().cpu(), want, dtype)


def test_rotary_frequencies_match_plain():
    from simple_inference_b200.parts.rope import rope_inverse_frequencies
    sc = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
    for d, theta, s in ((128, 500000.0, sc), (32, 500000.0, dict(sc, factor=8.0,
                        original_max_position_embeddings=64)), (16, 10000.0, None),
                        (48, 25000.0, {"rope_type": "linear", "factor": 4.0})):
        assert torch.equal(rope_inverse_frequencies(d, theta, s), plain_llama.rope_frequencies(d, theta, s))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_in_portions_and_with_a_window(dtype, window):
    """The mixer alone: two requests fed in portions through the cache, one with pages given
    back as the window passes them, against plain whole-sequence attention."""
    from simple_inference_b200.parts import MIXERS, PartSpec
    H, hq, hkv, d = 72, 6, 2, 16
    scaling = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
               "high_freq_factor": 2.0, "original_max_position_embeddings": 32}
    mixer = MIXERS.build(PartSpec("attention", {
        "hidden_size": H, "num_heads": hq, "num_kv_heads": hkv, "head_dim": d, "window": window,
        "position": PartSpec("rope", {"head_dim": d, "theta": 1000.0, "scaling": scaling})}))
    assert mixer.cache_spec().window == window
    h = Harness([mixer.cache_spec()], dtype, page_size=4, pages=40 if window else 80, parts=[mixer])
    ws = {n: rnd(*s.shape, seed=i, scale=0.2).to(dtype) for i, (n, s) in enumerate(mixer.tensors().items())}
    mixer.bind({n: t.to(DEV) for n, t in ws.items()}, h.rt)
    cfg = {"num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": d}
    pw = {"q_proj.weight": ws["wq"].float(), "k_proj.weight": ws["wk"].float(),
          "v_proj.weight": ws["wv"].float(), "o_proj.weight": ws["wo"].float()}
    freqs = plain_llama.rope_frequencies(d, 1000.0, scaling)
    xs = {"a": rnd(150, H, seed=10).to(dtype), "b": rnd(60, H, seed=11).to(dtype)}
    want = {r: plain_llama.attention_layer(x.float(), pw, "", cfg, list(range(len(x))), freqs, window)
            for r, x in xs.items()}
    fed = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    plan = [[("a", 40)], [("a", 1), ("b", 7)], [("b", 2), ("a", 64)], [("a", 1), ("b", 1)],
            [("a", 44), ("b", 50)]]
    for step in plan:
        ctx = h.ctx(step)
        x = torch.cat([xs[r][fed[r]:fed[r] + n] for r, n in step]).to(DEV)
        out = mixer.forward(x, ctx, h.views[0]).float().cpu()
        o = 0
        for r, n in step:
            got[r].append(out[o:o + n])
            o += n
            fed[r] += n
        h.cache.check()
    for r in xs:
        assert close(torch.cat(got[r]), want[r], dtype), r
    if window:
        live = [p for p in h.cache.block_table("a", 0) if p >= 0]
        assert len(live) <= (window + 64) // 4 + 2 and h.cache.block_table("a", 0)[0] == -1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_embedding_head_and_block(dtype):
    from simple_inference_b200.parts import BLOCKS, FEED_FORWARDS, PartSpec
    from simple_inference_b200.parts.embedding import OutputHead, TokenEmbedding
    H, I, V = 72, 200, 331
    h = Harness([], dtype)
    ffn = FEED_FORWARDS.build(PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}))
    ws = {n: rnd(*s.shape, seed=i, scale=0.2).to(dtype) for i, (n, s) in enumerate(ffn.tensors().items())}
    ffn.bind({n: t.to(DEV) for n, t in ws.items()}, h.rt)
    x = rnd(11, H, seed=5).to(dtype)
    ctx = h.ctx([("a", 11)])
    want = plain_llama.mlp(x.float(), {"gate_proj.weight": ws["w_gate"].float(),
                                       "up_proj.weight": ws["w_up"].float(),
                                       "down_proj.weight": ws["w_down"].float()}, "")
    assert close(ffn.forward(x.to(DEV), ctx).float().cpu(), want, dtype)

    table = rnd(V, H, seed=6).to(dtype)
    emb = TokenEmbedding(V, H)
    emb.bind({"weight": table.to(DEV)}, h.rt)
    ids = torch.tensor(random_ids(11, V, 1), dtype=torch.int32)
    assert torch.equal(emb.forward(ids.to(DEV), ctx).cpu(), table[ids.long()].float())
    for tied in (True, False):
        head = OutputHead(V, H, tied)
        hw = rnd(V, H, seed=7).to(dtype)
        head.bind({} if tied else {"weight": hw.to(DEV)}, h.rt, embedding=emb)
        logits = head.forward(x.to(DEV), ctx)
        assert logits.dtype == torch.float32
        ref = x.float() @ (table if tied else hw).float().T
        assert close(logits.cpu(), ref, dtype)


def test_block_and_a_run_order_that_repeats_a_layer_and_shares_a_cache(model_folders):
    """The order layers run in is data.  Tiny A (2 layers) run as [0, 1, 0, 1-reading-the-
    cache-of-the-first-1]: the plain model runs the same order on whole sequences; a layer
    that reads another's cache must see that layer's keys, so the plain side feeds it the
    first run's keys and values."""
    from simple_inference_b200.config import read_config
    from simple_inference_b200.models.plan import DecoderModel, RunStep
    from simple_inference_b200.models.load import runtime_for
    from simple_inference_b200.weights import load_tensors
    from simple_inference_b200.cache import CacheManager
    from simple_inference_b200.engine import ModelRunner, StepEntry
    arch, cfg = read_config(model_folders["A"])
    plan = arch.plan(cfg)
    plan.run_order = [RunStep(0, 0), RunStep(1, 1), RunStep(0, 2), RunStep(1, 1, writes_cache=False)]
    model = DecoderModel(plan)
    assert len(model.cache_specs()) == 3
    rt = runtime_for("float32", DEV)
    model.bind(load_tensors(model_folders["A"], model.tensor_specs(), model.optional_tensor_names(), rt), rt)
    cache = CacheManager(model.cache_specs(), 4, 40, 2, 64, torch.float32, DEV)
    runner = ModelRunner(model, cache, rt, 64, 2, 128, max_logit_rows=64)
    pcfg, w = plain_llama.read_folder(model_folders["A"])
    ids = random_ids(50, pcfg["vocab_size"], 9)

    # plain: whole sequence, same order; the fourth run attends with its own queries over the
    # keys and values that the second run (same layer, earlier input) produced
    pos = list(range(len(ids)))
    freqs = plain_llama.rope_frequencies(plain_llama.head_dim_of(pcfg), pcfg["rope_theta"], None)
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    x = plain_llama.block(x, w, 0, pcfg, pos, freqs)
    x_in_1 = x
    x = plain_llama.block(x, w, 1, pcfg, pos, freqs)
    x = plain_llama.block(x, w, 0, pcfg, pos, freqs)
    p, eps = "model.layers.1.", pcfg["rms_norm_eps"]
    Hq, Hkv, D = pcfg["num_attention_heads"], pcfg["num_key_value_heads"], plain_llama.head_dim_of(pcfg)
    cos, sin = plain_llama.rope_tables(freqs, pos)
    n1 = plain_llama.rmsnorm(x_in_1, w[p + "input_layernorm.weight"], eps)
    k = plain_llama.apply_rope((n1 @ w[p + "self_attn.k_proj.weight"].T).view(-1, Hkv, D), cos, sin)
    v = (n1 @ w[p + "self_attn.v_proj.weight"].T).view(-1, Hkv, D)
    n4 = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    q = plain_llama.apply_rope((n4 @ w[p + "self_attn.q_proj.weight"].T).view(-1, Hq, D), cos, sin)
    a = plain_llama.attention(q, k, v, pos).reshape(len(ids), Hq * D) @ w[p + "self_attn.o_proj.weight"].T
    x = x + a
    x = x + plain_llama.mlp(plain_llama.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    want = plain_llama.rmsnorm(x, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T

    cache.admit("r", 50)
    rows, fed = [], 0
    for c in (17, 2, 1, 30):
        rows.append(runner.step([StepEntry("r", ids[fed:fed + c], list(range(c)))]).clone())
        fed += c
    assert (torch.cat(rows).cpu() - want).abs().max() < 2e-5
    with pytest.raises(ValueError):
        plan.run_order = [RunStep(0, 0, writes_cache=False)]
        DecoderModel(plan)                          # reads a cache nobody wrote
