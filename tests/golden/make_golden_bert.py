"""Writes tests/golden/tiny_bert.pt: inputs and outputs of transformers.BertModel (the module the reference exports
and checks against, python/tilemega/dnn/export.py:50-59) on the seeded weights of tilemega_b200.synthetic.TINY_BERT.

Run from the repository root where transformers is installed: python tests/golden/make_golden_bert.py
"""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tilemega_b200.synthetic import TINY_BERT, encoder_inputs, encoder_weights   # noqa: E402


def module_outputs(config: dict, weights: dict, ids: torch.Tensor, types: torch.Tensor, mask: torch.Tensor | None = None):
    from transformers import BertConfig, BertModel
    keys = ("hidden_size", "intermediate_size", "num_attention_heads", "num_hidden_layers", "vocab_size",
            "max_position_embeddings", "type_vocab_size", "layer_norm_eps", "hidden_act")
    bert_config = BertConfig(**{key: config[key] for key in keys})
    bert_config._attn_implementation = "sdpa"
    module = BertModel(bert_config).eval()
    missing, unexpected = module.load_state_dict(weights, strict=False)
    if unexpected or any("position_ids" not in name for name in missing):
        raise RuntimeError(f"state dict mismatch: missing {missing}, unexpected {unexpected}")
    with torch.inference_mode():
        out = module(input_ids=ids, token_type_ids=types) if mask is None else module(input_ids=ids, token_type_ids=types, attention_mask=mask)
    return out.last_hidden_state.clone(), out.pooler_output.clone()


if __name__ == "__main__":
    torch.manual_seed(0)
    weights = encoder_weights(TINY_BERT, seed=0)
    ids, types = encoder_inputs(TINY_BERT, batch=2, seed=1)
    hidden, pooled = module_outputs(TINY_BERT, weights, ids, types)
    # the same inputs with padded tails (the reference's masked check: python/tilemega/dnn/check.py:151-171, 251-253)
    mask = (torch.arange(ids.shape[1])[None, :] < torch.tensor([[77], [128 - 19]])).to(torch.int64)
    masked_hidden, masked_pooled = module_outputs(TINY_BERT, weights, ids, types, mask)
    target = Path(__file__).with_name("tiny_bert.pt")
    torch.save({"config": TINY_BERT, "input_ids": ids, "token_type_ids": types, "last_hidden_state": hidden,
                "pooler_output": pooled, "attention_mask": mask, "masked_last_hidden_state": masked_hidden,
                "masked_pooler_output": masked_pooled}, target)
    print(target, hidden.shape, float(hidden.abs().max()))
