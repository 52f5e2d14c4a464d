"""Generation through the Python entry point and the command line, on the GPU."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import plain_llama
from tests.conftest import random_ids

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _engine(folder, dtype, **kw):
    from simple_inference_b200 import InferenceEngine
    opts = dict(max_running=4, max_seq_len=128, block_size=4, eos_id=-1, max_tokens_per_step=32,
                chunk_size=9)
    opts.update(kw)
    return InferenceEngine.from_folder(folder, dtype, "cuda", **opts)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_float32_equals_plain_in_every_regime(name, model_folders):
    """BASELINE's workload for Tiny A: prompts of 5, 17 and 32 ids, 16 greedy tokens each,
    page size 4; alone, together, and with so few pages that requests queue."""
    cfg, w = plain_llama.read_folder(model_folders[name])
    prompts = [random_ids(n, cfg["vocab_size"], 60 + n) for n in (5, 17, 32)]
    want = [plain_llama.generate_greedy(cfg, w, p, 16) for p in prompts]
    together = _engine(model_folders[name], "float32")
    reqs = [together.add_request(p, 16) for p in prompts]
    together.run()
    assert [r.generated for r in reqs] == want
    few = _engine(model_folders[name], "float32", num_kv_blocks=14, max_running=2)
    reqs = [few.add_request(p, 16) for p in prompts]
    few.run()
    assert [r.generated for r in reqs] == want
    assert few.cache.free_pages() == 14
    few.cache.check()
    alone = _engine(model_folders[name], "float32", chunk_size=None)
    for p, g in zip(prompts, want):
        assert list(alone.generate(p, 16)) == g


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_greedy_bfloat16_graphs_on_and_off_agree_with_plain(name, model_folders):
    cfg, w = plain_llama.read_folder(model_folders[name])
    prompts = [random_ids(n, cfg["vocab_size"], 80 + n) for n in (5, 17, 32, 3)]
    outs = []
    for graphs in (True, False):
        eng = _engine(model_folders[name], "bfloat16", use_cuda_graphs=graphs)
        assert eng.use_cuda_graphs == graphs
        reqs = [eng.add_request(p, 12) for p in prompts]
        eng.run()
        outs.append([r.generated for r in reqs])
    _agree_where_the_plain_model_is_sure(cfg, w, prompts, outs[0], outs[1])


def _agree_where_the_plain_model_is_sure(cfg, w, prompts, with_graphs, without):
    """The same kernels run inside and outside the graph.  Padding rows of a bucket must
    not disturb real rows: compare token by token, allowing a split only where the plain
    model's top two logits are within bfloat16 noise of each other."""
    for a, b, p in zip(with_graphs, without, prompts):
        ids = list(p)
        for x, y in zip(a, b):
            logits = plain_llama.forward(cfg, w, ids)[-1]
            top2 = logits.topk(2).values
            if x != y or x != int(logits.argmax()):
                assert (top2[0] - top2[1]) < 0.05, "engines disagree where the plain model is sure"
                break
            ids.append(x)


@pytest.mark.parametrize("name", ["B", "D"])
def test_forty_requests_decoding_together(name, model_folders):
    """max_running 64 and forty short prompts: decoding runs in the graph buckets of 32 and 64
    (with up to 24 padding rows), through the matrix products for 17 to 64 rows and the split
    planning for many sequences; greedy tokens against the plain model."""
    cfg, w = plain_llama.read_folder(model_folders[name])
    top = min(60, cfg["max_position_embeddings"] - 16)
    prompts = [random_ids(3 + (7 * i) % top, cfg["vocab_size"], 300 + i) for i in range(40)]
    outs = []
    for graphs in (True, False):
        eng = _engine(model_folders[name], "bfloat16", use_cuda_graphs=graphs, max_running=64,
                      block_size=16, max_tokens_per_step=256, chunk_size=None)
        reqs = [eng.add_request(p, 8 + i % 5) for i, p in enumerate(prompts)]
        live = []
        while eng.has_work():
            eng.step()
            live.append(sum(r.state.value == "decode" for r in eng.scheduler.running))
        assert max(live) > 32, "the run must reach the largest bucket"
        outs.append([r.generated for r in reqs])
        eng.cache.check()
    _agree_where_the_plain_model_is_sure(cfg, w, prompts, outs[0], outs[1])


@pytest.mark.parametrize("name", ["D", "E"])
def test_a_hundred_and_ten_requests_decoding_together(name, model_folders):
    """max_running 128 and 110 short prompts: decoding reaches the graph bucket of 128, whose
    matrix products have enough rows for the tcgen05 kernels (the projections that feed the
    residual stream cut along k, their slices added by the norms) inside a captured graph;
    greedy tokens against the plain model."""
    cfg, w = plain_llama.read_folder(model_folders[name])
    prompts = [random_ids(3 + (5 * i) % 40, cfg["vocab_size"], 700 + i) for i in range(110)]
    outs = []
    for graphs in (True, False):
        eng = _engine(model_folders[name], "bfloat16", use_cuda_graphs=graphs, max_running=128,
                      block_size=16, max_tokens_per_step=512, chunk_size=None, max_seq_len=96)
        reqs = [eng.add_request(p, 6 + i % 4) for i, p in enumerate(prompts)]
        live = []
        while eng.has_work():
            eng.step()
            live.append(sum(r.state.value == "decode" for r in eng.scheduler.running))
        assert max(live) >= 96, "the run must reach the rows of the tcgen05 products"
        outs.append([r.generated for r in reqs])
        eng.cache.check()
    _agree_where_the_plain_model_is_sure(cfg, w, prompts, outs[0], outs[1])


def test_temperature_sampling_matches_the_plain_sampler(model_folders):
    """BASELINE's workload for Tiny B: prompts of 1, 9, 40 and 100 ids, portions of 16 mixed
    with decoding, temperature 0.8, seed 0, page size 8."""
    from simple_inference_b200 import SamplingParams
    cfg, w = plain_llama.read_folder(model_folders["B"])
    prompts = [random_ids(n, cfg["vocab_size"], 90 + n) for n in (1, 9, 40, 100)]
    eng = _engine(model_folders["B"], "float32", block_size=8, chunk_size=16, max_seq_len=160)
    sp = SamplingParams(temperature=0.8, seed=0)
    reqs = [eng.add_request(p, 10, sp) for p in prompts]
    eng.run()
    for r, p in zip(reqs, prompts):
        ids = list(p)
        for c, tok in enumerate(r.generated):
            logits = plain_llama.forward(cfg, w, ids)[-1]
            z = logits / 0.8 + plain_llama.gumbel_noise(0, 0, c, cfg["vocab_size"])
            assert z[tok] >= z.max() - 1e-4, "the engine drew a token the plain sampler would not"
            ids.append(tok)


def test_top_k_top_p_through_the_engine(model_folders):
    from simple_inference_b200 import SamplingParams
    cfg, w = plain_llama.read_folder(model_folders["A"])
    prompt = random_ids(12, cfg["vocab_size"], 5)
    eng = _engine(model_folders["A"], "float32")
    sp = SamplingParams(temperature=1.5, top_k=3, top_p=0.9, seed=4)
    r = eng.add_request(prompt, 12, sp)
    eng.run()
    ids = list(prompt)
    for tok in r.generated:
        z = plain_llama.filter_logits(plain_llama.forward(cfg, w, ids)[-1], 1.5, 3, 0.9)
        assert torch.isfinite(z[tok]), "drew a token outside top-k / top-p"
        ids.append(tok)


def test_command_line(model_folders, tmp_path):
    cfg, w = plain_llama.read_folder(model_folders["A"])
    prompt = random_ids(9, cfg["vocab_size"], 2)
    want = plain_llama.generate_greedy(cfg, w, prompt, 8)
    stats = tmp_path / "stats.json"
    out = subprocess.run(
        [sys.executable, str(ROOT / "generate.py"), "--model", str(model_folders["A"]),
         "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "8",
         "--temperature", "0", "--eos-id", "-1", "--max-seq-len", "64", "--block-size", "4",
         "--stats-json", str(stats)],
        capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert out.returncode == 0, out.stderr
    assert json.loads(out.stdout.strip().splitlines()[-1])["tokens"] == want
    rec = json.loads(stats.read_text())
    assert rec["metrics"]["new_tokens"] == 8 and rec["metrics"]["prompt_tokens"] == 9
