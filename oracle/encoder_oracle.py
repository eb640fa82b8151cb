"""CPU oracle for the encoder forward path: a functional restatement of the BertModel forward.

TEST INFRASTRUCTURE ONLY. Nothing on the product path imports this file; only tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs may.

The reference does not hold this arithmetic itself: its oracle for the BERT workload is the third-party module
`transformers.BertModel(BertConfig())` with `attn_implementation='sdpa'` (reference call sites:
python/tilemega/dnn/export.py:50-59 builds it, python/tilemega/dnn/check.py:229-270 compares the native forward
with its fp32 and 16-bit runs; the reference pins transformers 5.19.0 in requirements/dnn-export.txt, 5.5.0 is
installed here). What is restated below is that module's published algorithm (BertEmbeddings: word + segment +
position embeddings, LayerNorm; BertLayer: scaled dot-product self-attention over all positions, output projection +
residual + LayerNorm, erf-GELU feed-forward + residual + LayerNorm; BertPooler: tanh of a projection of position 0).

Pinned: tests/golden/tiny_bert.pt holds inputs and outputs of the transformers module itself on seeded weights
(tests/golden/make_golden_bert.py); tests/test_encoder_host.py checks this restatement against the fixture and,
when transformers is importable, against the module run in the same test.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def encoder_forward(weights: dict[str, torch.Tensor], config: dict, input_ids: torch.Tensor, token_type_ids: torch.Tensor,
                    dtype: torch.dtype = torch.float32, attention_mask: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(last_hidden_state [B, S, H], pooler_output [B, H]) in `dtype` arithmetic (every module output rounded to it,
    as a module cast to that dtype does). `attention_mask` [B, S] (0 = hidden key position) becomes the module's
    additive mask: the most negative finite number of the score type on hidden keys, for every query."""
    w = {name: tensor.to(dtype) for name, tensor in weights.items()}
    hidden, heads, eps = config["hidden_size"], config["num_attention_heads"], float(config.get("layer_norm_eps", 1e-12))
    dim = hidden // heads
    batch, seq = input_ids.shape
    norm = lambda x, prefix: F.layer_norm(x, (hidden,), w[prefix + ".weight"], w[prefix + ".bias"], eps)
    positions = torch.arange(seq)
    x = (w["embeddings.word_embeddings.weight"][input_ids] + w["embeddings.token_type_embeddings.weight"][token_type_ids]
         + w["embeddings.position_embeddings.weight"][positions])
    x = norm(x, "embeddings.LayerNorm")
    for layer in range(config["num_hidden_layers"]):
        p = f"encoder.layer.{layer}."
        split = lambda t: t.view(batch, seq, heads, dim).transpose(1, 2)
        q = split(F.linear(x, w[p + "attention.self.query.weight"], w[p + "attention.self.query.bias"]))
        k = split(F.linear(x, w[p + "attention.self.key.weight"], w[p + "attention.self.key.bias"]))
        v = split(F.linear(x, w[p + "attention.self.value.weight"], w[p + "attention.self.value.bias"]))
        scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(dim)
        if attention_mask is not None:
            hidden_keys = (attention_mask == 0)[:, None, None, :]
            scores = scores.masked_fill(hidden_keys, torch.finfo(scores.dtype).min)
        context = torch.matmul(torch.softmax(scores.float(), dim=-1).to(dtype), v)
        context = context.transpose(1, 2).reshape(batch, seq, hidden)
        attended = F.linear(context, w[p + "attention.output.dense.weight"], w[p + "attention.output.dense.bias"])
        x = norm(attended + x, p + "attention.output.LayerNorm")
        inner = F.gelu(F.linear(x, w[p + "intermediate.dense.weight"], w[p + "intermediate.dense.bias"]))
        out = F.linear(inner, w[p + "output.dense.weight"], w[p + "output.dense.bias"])
        x = norm(out + x, p + "output.LayerNorm")
    pooled = torch.tanh(F.linear(x[:, 0], w["pooler.dense.weight"], w["pooler.dense.bias"]))
    return x, pooled


def token_cosine(actual: torch.Tensor, expected: torch.Tensor) -> torch.Tensor:
    """Cosine similarity per token (the quantity the reference gates on: python/tilemega/dnn/check.py:27-29)."""
    return F.cosine_similarity(actual.double().flatten(0, -2), expected.double().flatten(0, -2), dim=-1)
