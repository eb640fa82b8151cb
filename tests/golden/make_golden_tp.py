"""Generate the tensor-parallel golden fixture from the reference's rank modules.

    python tests/golden/make_golden_tp.py /path/to/TileMega

The reference exports ONE RANK's graph when the config carries `tilemega_tp`
(python/tilemega/serving/export.py:39-47,107-112,152-163): its SelfAttention and MLP
then return that rank's partial o_proj / down_proj output, and lm_head scores that
rank's slice of the vocabulary. This script builds the rank modules of the TINY
config at T = 2, gives each its slice of the seeded weights exactly as the reference's
loader narrows them (python/tilemega/serving/weights.py:78-96), runs layer 0's two
blocks and the head on a seeded bf16 input with a seeded KV history, and stores the
per-rank outputs. tests/test_oracle_golden.py checks the oracle's per-rank partials
against them bit for bit.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilemega_b200 import synthetic  # noqa: E402
from make_golden import rope  # noqa: E402

ROW_SHARDED = ("o_proj.weight", "down_proj.weight")


def rank_state(weights: dict[str, torch.Tensor], rank: int, world: int) -> dict[str, torch.Tensor]:
    state = {}
    for name, tensor in weights.items():
        if tensor.ndim == 2 and name != "model.embed_tokens.weight":
            axis = 1 if name.endswith(ROW_SHARDED) else 0
            size = tensor.shape[axis] // world
            tensor = tensor.narrow(axis, rank * size, size)
        state[name] = tensor.contiguous()
    return state


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + Path(__file__).name + " /path/to/TileMega [case ...]")
    reference = Path(sys.argv[1])
    sys.path.insert(0, str(reference / "python"))
    from tilemega.serving.export import Decoder
    world, batch, past = 2, 2, 19
    config = dict(synthetic.TINY, tie_word_embeddings=False)
    weights = synthetic.seeded_weights(config, seed=0, dtype=torch.bfloat16)
    weights.setdefault("lm_head.weight", weights["model.embed_tokens.weight"])
    dim, hkv, hidden = synthetic.head_dim_of(config), config["num_key_value_heads"], config["hidden_size"]
    generator = torch.Generator().manual_seed(17)
    x = torch.randn((batch, 1, hidden), generator=generator).to(torch.bfloat16)
    past_k = (0.5 * torch.randn((batch, hkv, past, dim), generator=generator)).to(torch.bfloat16)
    past_v = (0.5 * torch.randn((batch, hkv, past, dim), generator=generator)).to(torch.bfloat16)
    cos, sin = rope(config, past + 1, torch.bfloat16)
    record = {"config": config, "world": world, "batch": batch, "past": past, "x": x, "past_k": past_k,
              "past_v": past_v, "torch": str(torch.__version__), "attention": [], "mlp": [], "head": []}
    for rank in range(world):
        model = Decoder(dict(config, tilemega_tp=world)).eval().to(torch.bfloat16)
        missing = model.load_state_dict(rank_state(weights, rank, world), strict=False)
        assert not missing.unexpected_keys and not missing.missing_keys, missing
        layer = model.model.layers[0]
        share = hkv // world
        with torch.inference_mode():
            update, _, _ = layer.self_attn(layer.input_layernorm(x), past_k[:, rank * share:(rank + 1) * share],
                                           past_v[:, rank * share:(rank + 1) * share], cos, sin)
            record["attention"].append(update)
            record["mlp"].append(layer.mlp(layer.post_attention_layernorm(x)))
            record["head"].append(model.lm_head(model.model.norm(x)))
        print("rank", rank, update.float().abs().mean().item(), flush=True)
    torch.save(record, Path(__file__).resolve().parent / "tiny_tp2.pt")


if __name__ == "__main__":
    main()
