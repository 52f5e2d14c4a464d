"""Compares the plain implementation (tests/plain_llama.py) with the reference's own
model code on the CPU, once, and writes the small outputs next to this script.

Run from the repository root on a machine that has the reference checked out:

    PYTHONDONTWRITEBYTECODE=1 HF_HUB_OFFLINE=1 python tests/golden/make_golden.py /path/to/reference

It builds two tiny random Llama models (the tests' Tiny A and Tiny B; weights
from the repository's own random-weights mode, stored as float32), loads the
same tensors into the reference's ``LlamaModel`` (``model/llama.py:65-186``,
float32, CPU, PyTorch branches of every op) and into the plain implementation,
runs one prompt through both and stores

    golden_<name>.json   prompt ids, the reference's logits at the last 4
                         positions (first 16 vocabulary entries) and the
                         reference's argmax at every position
    golden_sampling.json rows of logits (with ties) and, for several settings of
                         temperature, top-k and top-p, which entries the reference's
                         filters keep (``sampling.py:39-52,69-128``, composed in the
                         order of its ``sample``, ``:159-167``)

``tests/test_plain.py`` recomputes these with the plain implementation alone, so
the oracle of all other tests stays anchored to the reference without the
reference being present.  Two facts about the reference shape the comparison:
its head is always tied (``model/llama.py:111``), so for the untied Tiny B the
reference's final hidden state is taken (embed, layers, norm) and the plain
head applied to it; and ``rope_scaling: null`` crashes it
(``model/llama.py:77-86``), so Tiny A passes rope_type "default".
"""

from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests import plain_llama  # noqa: E402
from tests.conftest import TINY_A, TINY_B, random_ids  # noqa: E402
from simple_inference_b200.weights import write_random_model  # noqa: E402


def reference_logits(ref_root: str, cfg: dict, w: dict, ids: list[int]) -> torch.Tensor:
    sys.path.insert(0, ref_root)
    from config import ModelConfig, RopeScalingConfig  # type: ignore
    from model.llama import LlamaModel  # type: ignore

    rs = cfg.get("rope_scaling") or {"rope_type": "default", "factor": 1.0, "low_freq_factor": 1.0,
                                     "high_freq_factor": 4.0,
                                     "original_max_position_embeddings": cfg["max_position_embeddings"]}
    mc = ModelConfig(
        hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"],
        num_hidden_layers=cfg["num_hidden_layers"], vocab_size=cfg["vocab_size"],
        num_attention_heads=cfg["num_attention_heads"],
        num_key_value_heads=cfg["num_key_value_heads"], rms_norm_eps=cfg["rms_norm_eps"],
        rope_theta=cfg["rope_theta"], max_position_embeddings=cfg["max_position_embeddings"],
        rope_scaling=RopeScalingConfig(rs["rope_type"], rs["factor"], rs["low_freq_factor"],
                                       rs["high_freq_factor"],
                                       rs["original_max_position_embeddings"]),
        tie_word_embeddings=True, torch_dtype="float32")
    model = LlamaModel(mc, torch.device("cpu")).eval()
    with torch.no_grad():
        model.embed.weight.copy_(w["model.embed_tokens.weight"])
        for i, layer in enumerate(model.layers):
            p = f"model.layers.{i}."
            layer.attn_norm.weight.copy_(w[p + "input_layernorm.weight"])
            layer.attn.wq.copy_(w[p + "self_attn.q_proj.weight"])
            layer.attn.wk.copy_(w[p + "self_attn.k_proj.weight"])
            layer.attn.wv.copy_(w[p + "self_attn.v_proj.weight"])
            layer.attn.wo.copy_(w[p + "self_attn.o_proj.weight"])
            layer.mlp_norm.weight.copy_(w[p + "post_attention_layernorm.weight"])
            layer.mlp.w_gate_up.copy_(torch.cat([w[p + "mlp.gate_proj.weight"],
                                                 w[p + "mlp.up_proj.weight"]], dim=0))
            layer.mlp.w_down.copy_(w[p + "mlp.down_proj.weight"])
        model.norm.weight.copy_(w["model.norm.weight"])
        x = model.embed(torch.tensor([ids]))
        for layer in model.layers:
            x = layer(x, start_pos=0, kv_cache=None)
        x = model.norm(x)[0]
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", True) else w["lm_head.weight"]
    return x @ head.T


SAMPLING_SETTINGS = [(1.0, 0, 1.0), (0.7, 5, 1.0), (1.3, 0, 0.9), (0.8, 20, 0.5), (1.0, 3, 0.0),
                     (2.0, 64, 0.3), (0.5, 1, 0.99), (1.0, 0, 0.05), (1.0, 7, 1.0), (0.9, 100, 0.95)]


def sampling_rows() -> torch.Tensor:
    """Rows of 64 logits: random, with exact ties at the top and at the top-k edge, one peaked."""
    g = torch.Generator().manual_seed(5)
    rows = torch.randn(4, 64, generator=g) * 2.0
    rows[1, 10] = rows[1, 20] = rows[1].max() + 0.5          # a tie for the top
    order = rows[2].argsort(descending=True)
    rows[2, order[6]] = rows[2, order[7]] = rows[2, order[5]] - 0.25   # a tie across the 7th place
    rows[3, 33] = rows[3].max() + 9.0                        # one token holds nearly all the mass
    return rows


def reference_kept(ref_root: str, rows: torch.Tensor) -> list[list[list[int]]]:
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    import sampling as ref  # type: ignore
    out = []
    for temperature, top_k, top_p in SAMPLING_SETTINGS:
        z = ref.apply_temperature(rows.clone(), temperature)
        if top_k > 0:
            z = ref.filter_top_k(z, top_k)
        if top_p < 1.0:
            z = ref.filter_top_p(z, top_p)
        out.append([torch.isfinite(r).nonzero().flatten().tolist() for r in z])
    return out


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <folder of the reference project>")
    ref_root = sys.argv[1]
    here = Path(__file__).resolve().parent
    rows = sampling_rows()
    kept = reference_kept(ref_root, rows)
    for (temperature, top_k, top_p), per_row in zip(SAMPLING_SETTINGS, kept):
        for row, want in zip(rows, per_row):
            mine = torch.isfinite(plain_llama.filter_logits(row, temperature, top_k, top_p))
            assert mine.nonzero().flatten().tolist() == want, (temperature, top_k, top_p)
    print(f"sampling filters: plain keeps what the reference keeps in all "
          f"{len(SAMPLING_SETTINGS) * len(rows)} cases")
    with open(here / "golden_sampling.json", "w") as f:
        json.dump({"rows": rows.tolist(), "settings": SAMPLING_SETTINGS, "reference_kept": kept}, f)
    for name, cfg in (("A", TINY_A), ("B", TINY_B)):
        cfg = dict(cfg, torch_dtype="float32")
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(tmp, cfg, seed=101)
            pcfg, w = plain_llama.read_folder(tmp)
        ids = random_ids(40, cfg["vocab_size"], seed=7)
        ref = reference_logits(ref_root, pcfg, w, ids)
        ours = plain_llama.forward(pcfg, w, ids)
        diff = (ref - ours).abs().max().item()
        print(f"tiny {name}: max |reference - plain| = {diff:.3e} over {tuple(ref.shape)} logits")
        assert diff < 2e-5, diff
        record = {
            "config": cfg, "weights_seed": 101, "prompt_seed": 7, "prompt": ids,
            "max_abs_diff_plain_vs_reference": diff,
            "reference_logits_last4_first16": ref[-4:, :16].tolist(),
            "reference_argmax": ref.argmax(-1).tolist(),
        }
        with open(here / f"golden_{name}.json", "w") as f:
            json.dump(record, f, indent=1)


if __name__ == "__main__":
    main()
