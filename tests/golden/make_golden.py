"""Generate the golden fixtures from the reference's own PyTorch forward.

Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/TileMega

It imports `tilemega.serving.export.Decoder` from <reference>/python, loads the
seeded synthetic weights of tilemega_b200.synthetic into it, runs prefill +
greedy decode on CPU, and writes small .pt files next to this script. The tests
read only those files; nothing at test time needs the reference tree.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilemega_b200 import synthetic  # noqa: E402


def rope(config: dict, capacity: int, dtype: torch.dtype):
    dim = synthetic.head_dim_of(config)
    inv = 1.0 / (float(config["rope_theta"]) ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    angles = torch.arange(capacity, dtype=torch.float32)[:, None] * inv[None, :]
    table = torch.cat((angles, angles), -1)
    return table.cos().to(torch.bfloat16).to(dtype), table.sin().to(torch.bfloat16).to(dtype)


def module_state(config: dict, state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """The checkpoint holds one tensor per expert projection (HF names); the reference's
    module keeps them stacked (python/tilemega/moe/export.py:54-65: gate rows then up rows)."""
    if not synthetic.is_moe(config):
        return state
    out = {name: tensor for name, tensor in state.items() if ".mlp.experts." not in name}
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}.mlp.experts."
        out[p + "gate_up_proj"] = torch.stack([torch.cat((state[p + f"{e}.gate_proj.weight"],
                                                          state[p + f"{e}.up_proj.weight"]))
                                               for e in range(config["num_experts"])])
        out[p + "down_proj"] = torch.stack([state[p + f"{e}.down_proj.weight"] for e in range(config["num_experts"])])
    return out


def run_reference(Decoder, config: dict, dtype: torch.dtype, prompt: torch.Tensor, new_tokens: int,
                  weight_rounding: torch.dtype):
    """Greedy decode with the reference module; weights rounded to `weight_rounding` first."""
    model = Decoder(config).eval()
    weights = synthetic.seeded_weights(config, seed=0, dtype=torch.float32)
    state = {name: tensor.to(weight_rounding).to(torch.float32) for name, tensor in weights.items()}
    state = module_state(config, state)
    missing = model.load_state_dict(state, strict=False)
    assert not missing.unexpected_keys and set(missing.missing_keys) <= {"lm_head.weight"}, missing
    model = model.to(dtype)
    batch, length = prompt.shape
    dim = synthetic.head_dim_of(config)
    cos, sin = rope(config, length + new_tokens + 1, dtype)
    caches = tuple(torch.zeros((batch, config["num_key_value_heads"], 0, dim), dtype=dtype)
                   for _ in range(2 * config["num_hidden_layers"]))
    tokens, history = [], []
    with torch.inference_mode():
        out = model.execute(prompt, caches, cos, sin)
        for step in range(new_tokens):
            logits = out[0][:, -1].float()
            history.append(logits.clone())
            chosen = logits.argmax(-1)
            tokens.append(chosen)
            if step + 1 < new_tokens:
                out = model.execute(chosen.view(batch, 1).to(torch.int32), tuple(out[1:]), cos, sin)
    return torch.stack(tokens, 1).to(torch.int32), torch.stack(history)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + Path(__file__).name + " /path/to/TileMega [case ...]")
    reference = Path(sys.argv[1])
    sys.path.insert(0, str(reference / "python"))
    from tilemega.serving.export import Decoder
    torch.set_num_threads(8)
    out_dir = Path(__file__).resolve().parent
    cases = (
        ("tiny", synthetic.TINY, 2, 21, 8, True),
        ("tiny_d128", synthetic.TINY_D128, 3, 37, 6, True),
        ("llama_3_2_1b", synthetic.LLAMA_3_2_1B, 1, 128, 32, False),
        ("tiny_moe", synthetic.TINY_MOE, 2, 19, 6, True),
    )
    only = set(sys.argv[2:])
    for name, config, batch, prompt_len, new_tokens, keep_logits in cases:
        if only and name not in only:
            continue
        prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
        record = {"config": config, "batch": batch, "prompt_len": prompt_len, "new_tokens": new_tokens,
                  "prompt": prompt, "torch": str(torch.__version__)}
        for label, dtype, rounding in (("fp32", torch.float32, torch.float32),
                                       ("fp32_bf16w", torch.float32, torch.bfloat16),
                                       ("bf16", torch.bfloat16, torch.bfloat16)):
            tokens, logits = run_reference(Decoder, config, dtype, prompt, new_tokens, rounding)
            top = logits.topk(8, dim=-1)
            record[label] = {"tokens": tokens, "top_values": top.values, "top_indices": top.indices.to(torch.int32)}
            if keep_logits:
                record[label]["logits"] = logits
            print(name, label, tokens[0, :8].tolist(), flush=True)
        torch.save(record, out_dir / f"{name}.pt")


if __name__ == "__main__":
    main()
