"""A mixer with state of its own, a position encoding of its own and an architecture of
its own, all defined HERE, are registered, built, given random weights, and stepped in
portions and mixed batches, without a change to any file of the framework.  Further down:
a feed-forward that routes each token to one of several experts, a norm of another kind,
and a run order that runs a layer twice.

The toy mixer keeps a decaying sum per request: s <- decay * s + x_t, y_t = W s.  Its state
is one row of fixed size per request (the cache manager's slots), so it must be carried
across portions, zeroed when a slot is handed to a new request, and kept apart between
requests that share a batch.
"""

from dataclasses import dataclass

import pytest
import torch

from tests.conftest import random_ids

pytestmark = pytest.mark.gpu
DEV = "cuda"


def define_toy():
    from simple_inference_b200 import ops
    from simple_inference_b200.config import ModelConfig, register_architecture
    from simple_inference_b200.models.llama import llama_layer_plan
    from simple_inference_b200.models.plan import LayerPlan, ModelPlan
    from simple_inference_b200.config.model_config import LlamaConfig
    from simple_inference_b200.parts import (Mixer, PartSpec, PositionEncoding, StateSpec, TensorSpec,
                                             register_mixer, register_position_encoding)

    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
        def __init__(self, hidden_size: int, decay: float):
            self.hidden_size, self.decay = hidden_size, decay

        def tensors(self):
            return {"w": TensorSpec((self.hidden_size, self.hidden_size))}

        def cache_spec(self):
            return StateSpec((self.hidden_size,), "float32")

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w = tensors["w"]

        def forward(self, x, ctx, cache):
            sums = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            slots = ctx.seq_slots.tolist()
            t = 0
            for s, n in enumerate(ctx.q_lens):
                state = cache.state[slots[s]]
                for i in range(n):
                    state.mul_(self.decay).add_(x[t + i].float())
                    sums[t + i] = state
                t += n
            out = ctx.ws.get("toy.out", (x.shape[0], self.hidden_size), x.dtype)
            return ops.linear(sums.to(x.dtype), self.w, out)

    @register_position_encoding("toy_half_rotary")
    class HalfSpeedRotary(PositionEncoding):
        """Rotary encoding whose every frequency is one constant: another position encoding."""

        def __init__(self, head_dim: int, freq: float):
            self.head_dim, self.freq = head_dim, freq

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.inv_freq = torch.full((self.head_dim // 2,), self.freq, dtype=torch.float32,
                                       device=rt.device)

        def encode_and_store(self, qkv, num_q_heads, num_kv_heads, head_dim, ctx, cache):
            ops.rope_kv_store(qkv, ctx.positions, self.inv_freq, ctx.kv_slots[cache.group],
                              cache.pool, num_q_heads, num_kv_heads, head_dim, cache.page_size,
                              cache.writes)

    @dataclass(kw_only=True)
    class ToyConfig(LlamaConfig):
        decay: float = 0.5
        toy_freq: float = 0.25

    def toy_plan(cfg: ToyConfig) -> ModelPlan:
        layers = []
        for i in range(cfg.num_hidden_layers):
            lp = llama_layer_plan(cfg, i)
            params = dict(lp.block.params)
            if i % 2 == 1:      # odd layers: the state mixer instead of attention
                params["mixer"] = PartSpec("toy_decay", {"hidden_size": cfg.hidden_size,
                                                         "decay": cfg.decay})
                names = {k: v for k, v in lp.tensor_names.items() if not k.startswith("mixer.")}
                names["mixer.w"] = f"model.layers.{i}.toy.w"
            else:               # even layers: attention with the toy position encoding
                mixer = dict(params["mixer"].params)
                mixer["position"] = PartSpec("toy_half_rotary", {"head_dim": cfg.head_dim,
                                                                 "freq": cfg.toy_freq})
                params["mixer"] = PartSpec("attention", mixer)
                names = lp.tensor_names
            layers.append(LayerPlan(PartSpec("prenorm", params), names))
        return ModelPlan(
            hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=layers,
            run_order=ModelPlan.sequential(len(layers)),
            final_norm=PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
            tie_embeddings=cfg.tie_word_embeddings, embedding_names={"weight": "model.embed_tokens.weight"},
            final_norm_names={"weight": "model.norm.weight"}, head_names={"weight": "lm_head.weight"},
            max_positions=cfg.max_position_embeddings)

    register_architecture("ToyForCausalLM", ToyConfig, toy_plan)


def plain_toy(cfg, w, ids):
    """Whole-sequence plain model of the toy architecture."""
    from tests import plain_llama as pl
    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    pos = list(range(len(ids)))
    D = pl.head_dim_of(cfg)
    freqs = torch.full((D // 2,), cfg["toy_freq"])
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = pl.rmsnorm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        if i % 2 == 1:
            s = torch.zeros(cfg["hidden_size"])
            rows = []
            for t in range(len(ids)):
                s = cfg["decay"] * s + h[t]
                rows.append(s)
            x = x + torch.stack(rows) @ w[p + "toy.w"].T
        else:
            x = x + pl.attention_layer(h, w, p + "self_attn.", cfg, pos, freqs)
        x = x + pl.mlp(pl.rmsnorm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), w, p + "mlp.")
    x = pl.rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    return x @ w["model.embed_tokens.weight"].T


def test_toy_architecture_registers_builds_and_steps(tmp_path):
    define_toy()
    from simple_inference_b200 import load_model, write_random_model, known_architectures
    from simple_inference_b200.cache import CacheManager
    from simple_inference_b200.engine import ModelRunner, StepEntry
    from simple_inference_b200.parts import PagedKVSpec, StateSpec
    from tests import plain_llama
    assert "ToyForCausalLM" in known_architectures()
    config = {
        "architectures": ["ToyForCausalLM"], "num_hidden_layers": 4, "hidden_size": 48,
        "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16,
        "intermediate_size": 72, "vocab_size": 101, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": True, "max_position_embeddings": 128, "torch_dtype": "float32",
        "decay": 0.75, "toy_freq": 0.125,
    }
    write_random_model(tmp_path, config, seed=2)
    cfg, model = load_model(tmp_path, "float32", DEV)
    specs = model.cache_specs()
    assert [type(s) for s in specs] == [PagedKVSpec, StateSpec, PagedKVSpec, StateSpec]
    cache = CacheManager(specs, 4, 30, 2, 64, torch.float32, DEV)
    assert len(cache.groups) == 1 and sorted(cache.state) == [1, 3]
    runner = ModelRunner(model, cache, model.rt, 64, 2, 128, max_logit_rows=64)
    pcfg, w = plain_llama.read_folder(tmp_path)
    seqs = [random_ids(n, 101, 20 + n) for n in (45, 30, 12)]
    want = [plain_toy(pcfg, w, s) for s in seqs]
    got = {i: [] for i in range(3)}
    fed = {i: 0 for i in range(3)}

    def feed(step):
        entries = [StepEntry(i, seqs[i][fed[i]:fed[i] + n], list(range(n))) for i, n in step]
        out = runner.step(entries).clone().cpu()
        o = 0
        for i, n in step:
            got[i].append(out[o:o + n])
            o += n
            fed[i] += n

    cache.admit(0, 45)
    cache.admit(1, 30)
    for step in ([(0, 20)], [(0, 1), (1, 9)], [(1, 2), (0, 5)], [(0, 19), (1, 19)]):
        feed(step)
    cache.release(1)                  # request 2 takes over request 1's slot and pages:
    cache.admit(2, 12)                # its state row must start from zero
    assert cache.slot(2) == 1
    for step in ([(2, 3)], [(2, 1)], [(2, 8)]):
        feed(step)
    for i in range(3):
        assert (torch.cat(got[i]) - want[i]).abs().max() < 2e-5, f"sequence {i}"


# --------------------------------------------------------------------------------------
# A feed-forward with routing and a norm of another kind, again defined here.
# --------------------------------------------------------------------------------------

def define_routed():
    from simple_inference_b200 import ops
    from simple_inference_b200.config import register_architecture
    from simple_inference_b200.config.model_config import LlamaConfig
    from simple_inference_b200.models.llama import llama_layer_plan
    from simple_inference_b200.models.plan import LayerPlan, ModelPlan, RunStep
    from simple_inference_b200.parts import (FeedForward, Norm, PartSpec, TensorSpec,
                                             register_feed_forward, register_norm)

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(FeedForward):
        """Every token goes to the one expert its router logit (float32) is largest for, and the
        expert's output is scaled by the softmax weight of that logit: y = p_e W2_e relu(W1_e x)."""

        def __init__(self, hidden_size: int, expert_size: int, num_experts: int):
            self.h, self.f, self.e = hidden_size, expert_size, num_experts

        def tensors(self):
            t = {"router": TensorSpec((self.e, self.h))}
            for e in range(self.e):
                t[f"w1_{e}"] = TensorSpec((self.f, self.h))
                t[f"w2_{e}"] = TensorSpec((self.h, self.f))
            return t

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.t = tensors

        def forward(self, x, ctx):
            n = x.shape[0]
            logits = torch.empty(n, self.e, dtype=torch.float32, device=x.device)
            ops.linear(x.float(), self.t["router"].float(), logits)       # router in float32
            prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            out = ctx.ws.get("toy.experts", (n, self.h), x.dtype)
            out.zero_()
            for e in range(self.e):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                xe = x[rows].contiguous()
                mid = torch.empty(rows.numel(), self.f, dtype=x.dtype, device=x.device)
                ops.linear(xe, self.t[f"w1_{e}"], mid)
                mid.relu_()
                ye = torch.empty(rows.numel(), self.h, dtype=x.dtype, device=x.device)
                ops.linear(mid, self.t[f"w2_{e}"], ye)
                out[rows] = (ye.float() * prob[rows, None]).to(x.dtype)
            return out

    @register_norm("toy_centred")
    class CentredNorm(Norm):
        """Subtracts the mean, divides by the standard deviation, multiplies by a gain."""

        def __init__(self, hidden_size: int, eps: float):
            self.h, self.eps = hidden_size, eps

        def tensors(self):
            return {"weight": TensorSpec((self.h,), kind="vector", init="gain")}

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.weight = tensors["weight"]

        def forward(self, residual, ctx, tag="norm"):
            return self.add_forward(residual, None, ctx, None, tag)

        def add_forward(self, residual, delta, ctx, rows=None, tag="norm"):
            if rows is None:
                if delta is not None:
                    residual.add_(delta.float())
                x = residual
            else:
                x = residual[rows.long()]
                if delta is not None:
                    x = x + delta[rows.long()].float()
            x = x - x.mean(-1, keepdim=True)
            y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
            return y.to(self.rt.dtype)

    @dataclass(kw_only=True)
    class RoutedConfig(LlamaConfig):
        num_experts: int = 3
        expert_size: int = 40

    def routed_plan(cfg: RoutedConfig) -> ModelPlan:
        layers = []
        norm = PartSpec("toy_centred", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
        for i in range(cfg.num_hidden_layers):
            lp = llama_layer_plan(cfg, i)
            params = dict(lp.block.params)
            names = dict(lp.tensor_names)
            params["feed_forward_norm"] = norm
            if i % 2 == 0:  # even layers: experts; odd layers keep the dense feed-forward
                params["feed_forward"] = PartSpec("toy_top1_experts", {
                    "hidden_size": cfg.hidden_size, "expert_size": cfg.expert_size,
                    "num_experts": cfg.num_experts})
                names = {k: v for k, v in names.items() if not k.startswith("feed_forward.")}
                names["feed_forward.router"] = f"model.layers.{i}.moe.router"
                for e in range(cfg.num_experts):
                    names[f"feed_forward.w1_{e}"] = f"model.layers.{i}.moe.{e}.w1"
                    names[f"feed_forward.w2_{e}"] = f"model.layers.{i}.moe.{e}.w2"
            layers.append(LayerPlan(PartSpec("prenorm", params), names))
        # the run order is data: layer 1 runs twice, its second run with a cache of its own
        order = [RunStep(0, 0), RunStep(1, 1), RunStep(1, 2)]
        return ModelPlan(
            hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=layers, run_order=order,
            final_norm=norm, tie_embeddings=cfg.tie_word_embeddings,
            embedding_names={"weight": "model.embed_tokens.weight"},
            final_norm_names={"weight": "model.norm.weight"}, head_names={"weight": "lm_head.weight"},
            max_positions=cfg.max_position_embeddings)

    register_architecture("RoutedToyForCausalLM", RoutedConfig, routed_plan)


def plain_routed(cfg, w, ids):
    from tests import plain_llama as pl
    eps = cfg["rms_norm_eps"]

    def centred(x, g):
        x = x - x.mean(-1, keepdim=True)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g

    x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    pos = list(range(len(ids)))
    freqs = pl.rope_frequencies(pl.head_dim_of(cfg), cfg["rope_theta"], None)
    for i in (0, 1, 1):
        p = f"model.layers.{i}."
        h = pl.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        x = x + pl.attention_layer(h, w, p + "self_attn.", cfg, pos, freqs)
        h = centred(x, w[p + "post_attention_layernorm.weight"])
        if i % 2 == 0:
            prob, choice = torch.softmax(h @ w[p + "moe.router"].T, dim=-1).max(dim=-1)
            y = torch.zeros_like(h)
            for t in range(len(ids)):
                e = int(choice[t])
                y[t] = prob[t] * (w[f"{p}moe.{e}.w2"] @ torch.relu(w[f"{p}moe.{e}.w1"] @ h[t]))
            x = x + y
        else:
            x = x + pl.mlp(h, w, p + "mlp.")
    return centred(x, w["model.norm.weight"]) @ w["model.embed_tokens.weight"].T


def test_routed_feed_forward_another_norm_and_a_layer_run_twice(tmp_path):
    define_routed()
    from simple_inference_b200 import load_model, write_random_model
    from simple_inference_b200.cache import CacheManager
    from simple_inference_b200.engine import ModelRunner, StepEntry
    from tests import plain_llama
    config = {
        "architectures": ["RoutedToyForCausalLM"], "num_hidden_layers": 2, "hidden_size": 56,
        "num_attention_heads": 2, "num_key_value_heads": 2, "head_dim": 32,
        "intermediate_size": 88, "vocab_size": 77, "rope_theta": 5000.0, "rms_norm_eps": 1e-4,
        "tie_word_embeddings": True, "max_position_embeddings": 128, "torch_dtype": "float32",
        "num_experts": 3, "expert_size": 40,
    }
    write_random_model(tmp_path, config, seed=4)
    cfg, model = load_model(tmp_path, "float32", DEV)
    specs = model.cache_specs()
    assert len(specs) == 3, "two layers, three runs, three caches"
    cache = CacheManager(specs, 4, 40, 2, 64, torch.float32, DEV)
    runner = ModelRunner(model, cache, model.rt, 64, 2, 128, max_logit_rows=64)
    pcfg, w = plain_llama.read_folder(tmp_path)
    seqs = [random_ids(n, 77, 40 + n) for n in (37, 21)]
    want = [plain_routed(pcfg, w, s) for s in seqs]
    got = {0: [], 1: []}
    fed = {0: 0, 1: 0}
    cache.admit(0, 37)
    cache.admit(1, 21)
    for step in ([(0, 16)], [(0, 1), (1, 9)], [(1, 2), (0, 20)], [(1, 10)]):
        entries = [StepEntry(i, seqs[i][fed[i]:fed[i] + n], list(range(n))) for i, n in step]
        out = runner.step(entries).clone().cpu()
        o = 0
        for i, n in step:
            got[i].append(out[o:o + n])
            o += n
            fed[i] += n
    for i in range(2):
        assert (torch.cat(got[i]) - want[i]).abs().max() < 3e-5, f"sequence {i}"


# --------------------------------------------------------------------------------------
# A state mixer that a CUDA graph can hold: decode steps replay from a graph that is
# captured inside a live step, and the state must advance exactly once per step.
# --------------------------------------------------------------------------------------

def define_graph_toy():
    from simple_inference_b200 import ops
    from simple_inference_b200.config import register_architecture
    from simple_inference_b200.config.model_config import LlamaConfig
    from simple_inference_b200.models.llama import llama_layer_plan
    from simple_inference_b200.models.plan import LayerPlan, ModelPlan
    from simple_inference_b200.parts import Mixer, PartSpec, StateSpec, TensorSpec, register_mixer

    @register_mixer("toy_decay_on_device")
    class DeviceDecayMixer(Mixer):
        """s <- decay * s + x_t, y_t = W s, with single-token steps done by device-side index
        arithmetic alone (no read-back), so that they can be recorded in a CUDA graph."""

        def __init__(self, hidden_size: int, decay: float):
            self.hidden_size, self.decay = hidden_size, decay

        def tensors(self):
            return {"w": TensorSpec((self.hidden_size, self.hidden_size))}

        def cache_spec(self):
            return StateSpec((self.hidden_size,), "float32")

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.w = tensors["w"]

        def forward(self, x, ctx, cache):
            out = ctx.ws.get("toy.out", (x.shape[0], self.hidden_size), x.dtype)
            if ctx.max_q_len == 1:          # one token per sequence: rows of x are sequences
                idx = ctx.seq_slots.long()
                new = cache.state[idx] * self.decay + x.float()
                cache.state.index_copy_(0, idx, new)   # padding rows all hit the scratch slot
                return ops.linear(new.to(x.dtype), self.w, out)
            sums = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            slots = ctx.seq_slots.tolist()
            t = 0
            for s, n in enumerate(ctx.q_lens):
                state = cache.state[slots[s]]
                for i in range(n):
                    state.mul_(self.decay).add_(x[t + i].float())
                    sums[t + i] = state
                t += n
            return ops.linear(sums.to(x.dtype), self.w, out)

    @dataclass(kw_only=True)
    class GraphToyConfig(LlamaConfig):
        decay: float = 0.5

    def plan(cfg: GraphToyConfig) -> ModelPlan:
        layers = []
        for i in range(cfg.num_hidden_layers):
            lp = llama_layer_plan(cfg, i)
            params, names = dict(lp.block.params), lp.tensor_names
            if i % 2 == 1:
                params["mixer"] = PartSpec("toy_decay_on_device", {"hidden_size": cfg.hidden_size,
                                                                   "decay": cfg.decay})
                names = {k: v for k, v in names.items() if not k.startswith("mixer.")}
                names["mixer.w"] = f"model.layers.{i}.toy.w"
            layers.append(LayerPlan(PartSpec("prenorm", params), names))
        return ModelPlan(
            hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=layers,
            run_order=ModelPlan.sequential(len(layers)),
            final_norm=PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
            tie_embeddings=True, embedding_names={"weight": "model.embed_tokens.weight"},
            final_norm_names={"weight": "model.norm.weight"}, head_names={"weight": "lm_head.weight"},
            max_positions=cfg.max_position_embeddings)

    register_architecture("GraphToyForCausalLM", GraphToyConfig, plan)


def test_state_mixer_in_bfloat16_with_graphs_captured_inside_a_live_step(tmp_path):
    """Decode steps of a model with a state mixer, replayed from CUDA graphs that are captured
    when their batch size is first met (no warm-up): the logits must equal those of the same
    steps run without graphs.  A capture that ran the live step more than once would advance
    the state more than once and part from the eager run at the first graph step."""
    define_graph_toy()
    from simple_inference_b200 import load_model, write_random_model
    from simple_inference_b200.cache import CacheManager
    from simple_inference_b200.engine import ModelRunner, StepEntry
    config = {
        "architectures": ["GraphToyForCausalLM"], "num_hidden_layers": 4, "hidden_size": 64,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
        "intermediate_size": 96, "vocab_size": 120, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": True, "max_position_embeddings": 128, "torch_dtype": "bfloat16",
        "decay": 0.8,
    }
    write_random_model(tmp_path, config, seed=6)
    _, model = load_model(tmp_path, "bfloat16", DEV)
    seqs = [random_ids(n, 120, 70 + n) for n in (30, 22, 17)]

    def run(graphs: bool):
        cache = CacheManager(model.cache_specs(), 4, 60, 4, 64, torch.bfloat16, DEV)
        runner = ModelRunner(model, cache, model.rt, 64, 4, 128, cuda_graphs=graphs)
        out = []
        for i in range(3):
            cache.admit(i, 40)
        runner.step([StepEntry(i, seqs[i][:10], []) for i in range(3)])        # prompts
        for t in range(10, 17):                                                # three decoding
            out.append(runner.step([StepEntry(i, [seqs[i][t]], [0]) for i in range(3)]).clone())
        cache.release(2)
        for t in range(17, 22):                                                # two: another bucket
            out.append(runner.step([StepEntry(i, [seqs[i][t]], [0]) for i in range(2)]).clone())
        if graphs:
            assert sorted(runner._graphs) == [2, 4], "both buckets were captured on the way"
        return torch.cat(out).float().cpu()

    eager, replayed = run(False), run(True)
    assert torch.isfinite(eager).all()
    # the same kernels on the same numbers but for the number of key splits, which a graph plans
    # for the longest context: a rounding apart at most; a state advanced twice is far off
    assert (eager - replayed).abs().max() < 2e-2 * float(eager.abs().max())


# --------------------------------------------------------------------------------------
# A cache that is one vector per token in pages of its own size, an embedding with a
# scale and a head with a cap: registered kinds, no framework file touched.
# --------------------------------------------------------------------------------------

def define_latent_toy():
    from simple_inference_b200 import ops
    from simple_inference_b200.config import register_architecture
    from simple_inference_b200.config.model_config import LlamaConfig
    from simple_inference_b200.models.llama import llama_layer_plan
    from simple_inference_b200.models.plan import LayerPlan, ModelPlan
    from simple_inference_b200.parts import (Embedding, Head, Mixer, PartSpec, TensorSpec,
                                             register_embedding, register_head, register_mixer)

    @dataclass(frozen=True)
    class LatentSpec:
        """One vector of `width` numbers per token, in pages of 8 tokens whatever the engine's
        page size: a cache kind the framework has never heard of."""
        width: int
        window: int | None = None
        page_size: int | None = 8
        storage = "pages"

        def page_shape(self, page_size):
            return (page_size, self.width)

    @register_mixer("toy_latent_mean")
    class LatentMeanMixer(Mixer):
        """c_t = Wc x_t is stored per token; y_t = Wo * mean of c_j over the request's j <= t."""

        def __init__(self, hidden_size: int, width: int):
            self.hidden_size, self.width = hidden_size, width

        def tensors(self):
            return {"wc": TensorSpec((self.width, self.hidden_size)),
                    "wo": TensorSpec((self.hidden_size, self.width))}

        def cache_spec(self):
            return LatentSpec(self.width)

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.wc, self.wo = tensors["wc"], tensors["wo"]

        def forward(self, x, ctx, cache):
            n = x.shape[0]
            c = torch.empty(n, self.width, dtype=x.dtype, device=x.device)
            ops.linear(x, self.wc, c)
            flat = cache.pool.view(-1, self.width)            # [(pages+1) * page_size, width]
            flat[ctx.kv_slots[cache.group].long()] = c
            table = ctx.block_tables[cache.group].tolist()
            means = torch.empty_like(c)
            t = 0
            for s, (q, kv) in enumerate(zip(ctx.q_lens, ctx.kv_lens)):
                rows = torch.tensor([table[s][j // cache.page_size] * cache.page_size
                                     + j % cache.page_size for j in range(kv)], device=x.device)
                run = flat[rows].float().cumsum(0) / torch.arange(1, kv + 1, device=x.device)[:, None]
                means[t:t + q] = run[kv - q:].to(x.dtype)
                t += q
            out = ctx.ws.get("toy.latent_out", (n, self.hidden_size), x.dtype)
            return ops.linear(means, self.wo, out)

    @register_embedding("toy_scaled_embedding")
    class ScaledEmbedding(Embedding):
        def __init__(self, vocab_size: int, hidden_size: int, scale: float):
            self.v, self.h, self.scale = vocab_size, hidden_size, scale

        def tensors(self):
            return {"weight": TensorSpec((self.v, self.h))}

        def bind(self, tensors, rt):
            super().bind(tensors, rt)
            self.weight = tensors["weight"]

        def forward(self, token_ids, ctx):
            residual = ctx.ws.get("residual", (token_ids.shape[0], self.h), torch.float32)
            ops.embed_gather(self.weight, token_ids, residual)
            return residual.mul_(self.scale)

        def output_matrix(self):
            return self.weight

    @register_head("toy_capped_head")
    class CappedHead(Head):
        """logits = cap * tanh(x E^T / cap) + bias, with the embedding's matrix."""

        def __init__(self, vocab_size: int, hidden_size: int, cap: float):
            self.v, self.h, self.cap = vocab_size, hidden_size, cap

        def tensors(self):
            return {"bias": TensorSpec((self.v,), kind="vector", init="normal")}

        def bind(self, tensors, rt, embedding=None):
            super().bind(tensors, rt, embedding)
            self.weight, self.bias = embedding.output_matrix(), tensors["bias"]

        def forward(self, x, ctx):
            logits = ctx.ws.get("logits", (x.shape[0], self.v), torch.float32,
                                row_cap=ctx.ws.max_logit_rows)
            ops.linear(x, self.weight, logits)
            return torch.tanh(logits / self.cap) * self.cap + self.bias.float()

    @dataclass(kw_only=True)
    class LatentToyConfig(LlamaConfig):
        latent_width: int = 12
        embedding_scale: float = 3.0
        logit_cap: float = 2.0

    def plan(cfg: LatentToyConfig) -> ModelPlan:
        layers = []
        for i in range(cfg.num_hidden_layers):
            lp = llama_layer_plan(cfg, i)
            params, names = dict(lp.block.params), lp.tensor_names
            if i % 2 == 1:
                params["mixer"] = PartSpec("toy_latent_mean", {"hidden_size": cfg.hidden_size,
                                                               "width": cfg.latent_width})
                names = {k: v for k, v in names.items() if not k.startswith("mixer.")}
                names["mixer.wc"] = f"model.layers.{i}.latent.wc"
                names["mixer.wo"] = f"model.layers.{i}.latent.wo"
            layers.append(LayerPlan(PartSpec("prenorm", params), names))
        return ModelPlan(
            hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, layers=layers,
            run_order=ModelPlan.sequential(len(layers)),
            final_norm=PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
            tie_embeddings=True,
            embedding=PartSpec("toy_scaled_embedding", {
                "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                "scale": cfg.embedding_scale}),
            head=PartSpec("toy_capped_head", {"vocab_size": cfg.vocab_size,
                                              "hidden_size": cfg.hidden_size, "cap": cfg.logit_cap}),
            embedding_names={"weight": "model.embed_tokens.weight"},
            final_norm_names={"weight": "model.norm.weight"}, head_names={"bias": "lm_head.bias"},
            max_positions=cfg.max_position_embeddings)

    register_architecture("LatentToyForCausalLM", LatentToyConfig, plan)


def plain_latent(cfg, w, ids):
    from tests import plain_llama as pl
    eps = cfg["rms_norm_eps"]
    x = w["model.embed_tokens.weight"][torch.tensor(ids)] * cfg["embedding_scale"]
    pos = list(range(len(ids)))
    freqs = pl.rope_frequencies(pl.head_dim_of(cfg), cfg["rope_theta"], None)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = pl.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        if i % 2 == 1:
            c = h @ w[p + "latent.wc"].T
            mean = c.cumsum(0) / torch.arange(1, len(ids) + 1)[:, None]
            x = x + mean @ w[p + "latent.wo"].T
        else:
            x = x + pl.attention_layer(h, w, p + "self_attn.", cfg, pos, freqs)
        x = x + pl.mlp(pl.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    logits = pl.rmsnorm(x, w["model.norm.weight"], eps) @ w["model.embed_tokens.weight"].T
    return torch.tanh(logits / cfg["logit_cap"]) * cfg["logit_cap"] + w["lm_head.bias"]


def test_a_latent_cache_in_pages_of_its_own_a_scaled_embedding_and_a_capped_head(tmp_path):
    define_latent_toy()
    from simple_inference_b200 import load_model, write_random_model
    from simple_inference_b200.cache import CacheManager
    from simple_inference_b200.engine import ModelRunner, StepEntry
    from tests import plain_llama
    config = {
        "architectures": ["LatentToyForCausalLM"], "num_hidden_layers": 4, "hidden_size": 40,
        "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
        "intermediate_size": 56, "vocab_size": 90, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": True, "max_position_embeddings": 128, "torch_dtype": "float32",
        "latent_width": 12, "embedding_scale": 3.0, "logit_cap": 2.0,
    }
    write_random_model(tmp_path, config, seed=8)
    cfg, model = load_model(tmp_path, "float32", DEV)
    specs = model.cache_specs()
    assert [s.storage for s in specs] == ["pages"] * 4 and specs[0] != specs[1]
    # attention pages of 4 tokens (the manager's size), latent pages of 8 (their own): 16 and 9
    # pages hold 64 and 72 tokens, fewer than the 86 the three requests need together
    cache = CacheManager(specs, 4, {0: 16, 1: 9}, 2, 64, torch.float32, DEV)
    assert [g.page_size for g in cache.groups] == [4, 8]
    assert tuple(cache.groups[1].pool.shape) == (2, 10, 8, 12)
    runner = ModelRunner(model, cache, model.rt, 64, 2, 128, max_logit_rows=64)
    pcfg, w = plain_llama.read_folder(tmp_path)
    seqs = [random_ids(n, 90, 50 + n) for n in (41, 26, 19)]
    want = [plain_latent(pcfg, w, s) for s in seqs]
    got = {i: [] for i in range(3)}
    fed = {i: 0 for i in range(3)}

    def feed(step):
        entries = [StepEntry(i, seqs[i][fed[i]:fed[i] + n], list(range(n))) for i, n in step]
        out = runner.step(entries).clone().cpu()
        o = 0
        for i, n in step:
            got[i].append(out[o:o + n])
            o += n
            fed[i] += n
        cache.check()

    cache.admit(0, 28)
    cache.admit(1, 26)
    for step in ([(0, 13)], [(0, 1), (1, 9)], [(1, 17), (0, 2)], [(0, 12)]):
        feed(step)
    cache.release(1)                 # its pages of both sizes go to request 2
    cache.admit(2, 19)
    cache.reserve_to(0, 41)
    for step in ([(2, 3), (0, 1)], [(2, 16), (0, 12)]):
        feed(step)
    for i in range(3):
        assert (torch.cat(got[i]) - want[i]).abs().max() < 3e-5, f"sequence {i}"
