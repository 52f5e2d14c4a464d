"""``LlamaForCausalLM``: a dense decoder of pre-norm blocks with grouped-query
attention, rotary positions (llama3 scaling), RMSNorm and a SwiGLU feed-forward
(reference ``model/llama.py:65-186``, ``model/block.py:55-146``).

This module only translates a ``LlamaConfig`` into a ``ModelPlan``; every
number in the plan comes from the configuration.  Tensor names are the
checkpoint's own (reference ``loader.py:74-93``).
"""

from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .plan import LayerPlan, ModelPlan


def llama_layer_plan(cfg: LlamaConfig, index: int) -> LayerPlan:
    scaling = cfg.rope_scaling.to_dict() if cfg.rope_scaling is not None else None
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "scaling": scaling})
    mixer = PartSpec("attention", {
        "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "position": position, "window": None,
    })
    norm = PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                              "intermediate_size": cfg.intermediate_size})
    block = PartSpec("prenorm", {"mixer": mixer, "mixer_norm": norm, "feed_forward": ffn,
                                 "feed_forward_norm": norm})
    p = f"model.layers.{index}"
    names = {
        "mixer_norm.weight": f"{p}.input_layernorm.weight",
        "mixer.wq": f"{p}.self_attn.q_proj.weight",
        "mixer.wk": f"{p}.self_attn.k_proj.weight",
        "mixer.wv": f"{p}.self_attn.v_proj.weight",
        "mixer.wo": f"{p}.self_attn.o_proj.weight",
        "feed_forward_norm.weight": f"{p}.post_attention_layernorm.weight",
        "feed_forward.w_gate": f"{p}.mlp.gate_proj.weight",
        "feed_forward.w_up": f"{p}.mlp.up_proj.weight",
        "feed_forward.w_down": f"{p}.mlp.down_proj.weight",
    }
    return LayerPlan(block, names)


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    return ModelPlan(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=[llama_layer_plan(cfg, i) for i in range(cfg.num_hidden_layers)],
        run_order=ModelPlan.sequential(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps}),
        tie_embeddings=cfg.tie_word_embeddings,
        embedding_names={"weight": "model.embed_tokens.weight"},
        final_norm_names={"weight": "model.norm.weight"},
        head_names={"weight": "lm_head.weight"},
        max_positions=cfg.max_position_embeddings,
        eos_token_ids=cfg.eos_ids(),
        bos_token_id=cfg.bos_token_id,
    )


register_architecture("LlamaForCausalLM", LlamaConfig, llama_plan)
