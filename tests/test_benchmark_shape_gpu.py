"""The engine at the layer sizes of the benchmark's model (Llama 3.2 3B: width 3072, 24 query
and 8 key/value heads of 128, feed-forward 8192, vocabulary 128,256, llama3 scaling by 32,
tied head), with two layers instead of 28.  The tiny configurations of the other tests never
reach these sizes: a product that goes wrong only at K = 8192, a head that goes wrong only
at 128,256 rows, or decode attention that goes wrong only with 64 sequences would pass them
all and still print a tokens-per-second figure.

float32 path against the plain model on a short prompt; bfloat16 against the float32 path on
a 300-token prompt cut three ways; one decode step of 64 sequences at contexts between 1 and
2,047 and one of 100 sequences (the rows of the tcgen05 products, cut along k), both replayed
from CUDA graphs, against the float32 path.
"""

import pytest
import torch

from tests import plain_llama
from tests.conftest import random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPE_3B_TWO_LAYERS = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 3072, "num_attention_heads": 24,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    "torch_dtype": "bfloat16",
}
PAGE = 16


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    from simple_inference_b200.weights import write_random_model
    return write_random_model(tmp_path_factory.mktemp("shape_3b"), SHAPE_3B_TWO_LAYERS, seed=31)


def _runner(folder, dtype, max_seqs, max_seq_len, graphs=False, step_tokens=2048):
    from simple_inference_b200 import load_model
    from simple_inference_b200.cache import CacheManager, pages_for
    from simple_inference_b200.engine import ModelRunner
    _, model = load_model(folder, dtype, DEV)
    cache = CacheManager(model.cache_specs(), PAGE, max_seqs * pages_for(max_seq_len, PAGE), max_seqs,
                         step_tokens, dtype=model.rt.dtype, device=DEV)
    return cache, ModelRunner(model, cache, model.rt, step_tokens, max_seqs, max_seq_len,
                              cuda_graphs=graphs, max_logit_rows=320)


def _spread(logits):
    """Standard deviation of the logits: the yardstick for a tolerance on them."""
    return float(logits.float().std())


def test_float32_path_equals_the_plain_model_at_these_sizes(folder):
    from simple_inference_b200.engine import StepEntry
    cfg, w = plain_llama.read_folder(folder)
    ids = random_ids(40, cfg["vocab_size"], 3)
    want = plain_llama.forward(cfg, w, ids)
    cache, runner = _runner(folder, "float32", 1, 64)
    cache.admit("p", 40)
    got = runner.step([StepEntry("p", ids, list(range(40)))]).cpu()
    assert got.shape == (40, 128256)
    diff = float((got - want).abs().max())
    print(f"float32 engine against the plain model at 3B layer sizes: {diff:.2e}, "
          f"logit spread {_spread(want):.3f}")
    assert diff < 1e-4 * max(1.0, _spread(want))
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_bfloat16_against_the_float32_path_three_cuts_and_64_and_100_sequences_decoding(folder):
    from simple_inference_b200.engine import StepEntry
    vocab = SHAPE_3B_TWO_LAYERS["vocab_size"]
    ids = random_ids(300, vocab, 4)
    lens = [1 + (i * 997) % 2047 for i in range(64)]       # contexts from 1 to 2,047, all distinct
    lens[5], lens[17] = 1, 2047
    seqs = [random_ids(n, vocab, 500 + i) for i, n in enumerate(lens)]

    def run(dtype, graphs):
        out = {}
        cache, runner = _runner(folder, dtype, 128, 2048, graphs=graphs)
        cache.admit("w", 300)
        out["whole"] = runner.step([StepEntry("w", ids, list(range(300)))]).clone()
        cache.release("w")
        if dtype == "bfloat16":
            cache.admit("two", 300)
            a = runner.step([StepEntry("two", ids[:171], list(range(171)))]).clone()
            b = runner.step([StepEntry("two", ids[171:], list(range(129)))]).clone()
            out["two portions"] = torch.cat([a, b])
            cache.release("two")
            cache.admit("tail", 300)
            rows = [runner.step([StepEntry("tail", ids[:284], [283])]).clone()]
            for p in range(284, 300):
                rows.append(runner.step([StepEntry("tail", [ids[p]], [0])]).clone())
            out["last 16 one by one"] = torch.cat(rows)
            cache.release("tail")
        # 64 sequences: all but the last token in steps of at most 2,048 tokens, then ONE decode step
        for i, s in enumerate(seqs):
            cache.admit(i, len(s) + 1)
        batch, room = [], 2048
        for i, s in enumerate(seqs):
            if len(s) == 1:
                continue
            if len(s) - 1 > room:
                runner.step(batch)
                batch, room = [], 2048
            batch.append(StepEntry(i, s[:-1], []))
            room -= len(s) - 1
        if batch:
            runner.step(batch)
        out["decode 64"] = runner.step([StepEntry(i, [s[-1]], [0]) for i, s in enumerate(seqs)]).clone()
        if graphs:
            assert 64 in runner._graphs, "the decode step of 64 sequences ran from a captured graph"
        # 36 more sequences join, then ONE decode step of 100: enough rows for the tcgen05 products,
        # whose projections into the residual stream are cut along k at these sizes
        more = [random_ids(2 + (i * 7) % 40, vocab, 900 + i) for i in range(36)]
        for i, s in enumerate(more):
            cache.admit(64 + i, len(s) + 1)
        runner.step([StepEntry(64 + i, s, []) for i, s in enumerate(more)])
        nxt = random_ids(100, vocab, 77)
        out["decode 100"] = runner.step([StepEntry(i, [nxt[i]], [0]) for i in range(100)]).clone()
        if graphs:
            assert 128 in runner._graphs, "the decode step of 100 sequences ran from a captured graph"
        cache.check()
        return {k: v.float().cpu() for k, v in out.items()}

    ref = run("float32", False)
    got = run("bfloat16", True)
    spread = _spread(ref["whole"])
    pairs = [("whole", ref["whole"]), ("two portions", ref["whole"]),
             ("last 16 one by one", ref["whole"][283:]), ("decode 64", ref["decode 64"]),
             ("decode 100", ref["decode 100"])]
    for what, want in pairs:
        diff = float((got[what] - want).abs().max())
        agree = float((got[what].argmax(-1) == want.argmax(-1)).float().mean())
        print(f"bfloat16 against float32 at 3B layer sizes, {what}: max diff {diff:.3e} "
              f"(logit spread {spread:.3f}), top-1 agreement {agree:.3f}")
        assert torch.isfinite(got[what]).all()
        assert diff < BF16_TOL_IN_SPREADS * spread, what
        # where the float32 path is sure of its token (a margin over the runner-up larger than the
        # tolerance allows both to move), the bfloat16 path names the same token
        top2 = want.topk(2, dim=-1).values
        sure = (top2[:, 0] - top2[:, 1]) > 2 * BF16_TOL_IN_SPREADS * spread
        assert torch.equal(got[what].argmax(-1)[sure], want.argmax(-1)[sure]), what


# measured: 0.064 to 0.066 of the logits' standard deviation (sums of 3072 and 8192 bfloat16
# products); a product that drops or repeats a k-block is off by a whole standard deviation
BF16_TOL_IN_SPREADS = 0.15
