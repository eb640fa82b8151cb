"""Writes tests/golden/rope_llama3.pt: cos/sin rows of the HF rotary module
(transformers.models.llama.modeling_llama.LlamaRotaryEmbedding, which the reference's
python/tilemega/serving/state.py:30-59 calls) for the rope_scaling blocks of the
Llama-3.1-8B and Llama-3.2-1B checkpoints, and for a linear scaling, at a few positions.

    python tests/golden/make_golden_rope.py

Needs `transformers` (any 4.45+/5.x); the fixture it writes is what the tests read.
"""
from pathlib import Path

import torch
from transformers import LlamaConfig
from transformers.models.llama.modeling_llama import LlamaRotaryEmbedding

CASES = {
    "llama31_8b": dict(head_dim=128, rope_theta=500000.0,
                       rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                         original_max_position_embeddings=8192)),
    "llama32_1b": dict(head_dim=64, rope_theta=500000.0,
                       rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                         original_max_position_embeddings=8192)),
    "linear4": dict(head_dim=128, rope_theta=10000.0, rope_scaling=dict(rope_type="linear", factor=4.0)),
}
POSITIONS = [0, 1, 2, 17, 255, 1000, 4097, 8191, 20000, 131071]


def main() -> None:
    out = {}
    for name, case in CASES.items():
        scaling = dict(case["rope_scaling"], rope_theta=case["rope_theta"])
        config = LlamaConfig(hidden_size=case["head_dim"] * 4, num_attention_heads=4, num_key_value_heads=4,
                             head_dim=case["head_dim"], rope_theta=case["rope_theta"], rope_scaling=scaling,
                             rope_parameters=scaling, max_position_embeddings=131072)
        module = LlamaRotaryEmbedding(config)
        positions = torch.tensor([POSITIONS])
        cos, sin = module(torch.zeros(1, len(POSITIONS), case["head_dim"], dtype=torch.bfloat16), positions)
        out[name] = {"config": {"head_dim": case["head_dim"], "rope_theta": case["rope_theta"],
                                "rope_scaling": case["rope_scaling"]},
                     "positions": POSITIONS, "inv_freq": module.inv_freq.clone(), "cos": cos[0].clone(), "sin": sin[0].clone()}
    torch.save(out, Path(__file__).resolve().parent / "rope_llama3.pt")
    print({name: (item["cos"].dtype, tuple(item["cos"].shape)) for name, item in out.items()})


if __name__ == "__main__":
    main()
