"""Seeded synthetic workloads with the shapes of the benchmark configurations.

No dataset or checkpoint is involved: weights are N(0, 0.02) draws from a seeded
generator (norm weights 1), token ids and context lengths are seeded uniform
draws. The draw order is fixed here so every consumer (GPU path, CPU oracle,
fixture generator) sees the same tensors.
"""
from __future__ import annotations

import torch

LLAMA_3_2_1B = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=8192,
                    num_attention_heads=32, num_key_value_heads=8, head_dim=64, num_hidden_layers=16,
                    vocab_size=128256, rms_norm_eps=1e-5, tie_word_embeddings=True, rope_theta=500000.0)
LLAMA_3_1_8B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336,
                    num_attention_heads=32, num_key_value_heads=8, head_dim=128, num_hidden_layers=32,
                    vocab_size=128256, rms_norm_eps=1e-5, tie_word_embeddings=False, rope_theta=500000.0)
LLAMA_3_1_70B = dict(architectures=["LlamaForCausalLM"], hidden_size=8192, intermediate_size=28672,
                     num_attention_heads=64, num_key_value_heads=8, head_dim=128, num_hidden_layers=80,
                     vocab_size=128256, rms_norm_eps=1e-5, tie_word_embeddings=False, rope_theta=500000.0)
# Two-layer models (under 150 MB of bf16 weights) with every structural feature of
# the above: 4 query heads per KV head, head_dim 64 / 128, every K a multiple of 2048.
TINY = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=2048,
            num_attention_heads=32, num_key_value_heads=8, head_dim=64, num_hidden_layers=2,
            vocab_size=1024, rms_norm_eps=1e-5, tie_word_embeddings=True, rope_theta=500000.0)
TINY_D128 = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=4096,
                 num_attention_heads=16, num_key_value_heads=4, head_dim=128, num_hidden_layers=2,
                 vocab_size=2048, rms_norm_eps=1e-5, tie_word_embeddings=False, rope_theta=500000.0)


# 8 query heads per KV head (the 70B-shaped grouping)
TINY_GQ8 = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=2048,
                num_attention_heads=16, num_key_value_heads=2, head_dim=128, num_hidden_layers=2,
                vocab_size=1024, rms_norm_eps=1e-5, tie_word_embeddings=False, rope_theta=500000.0)


# Mixture of experts (Qwen3-30B-A3B-shaped): per-head QK norm, top-k routing over a
# softmax, expert SwiGLU FFNs; router weights N(0, 0.1) so the expert load is uneven.
QWEN3_30B_A3B = dict(architectures=["Qwen3MoeForCausalLM"], hidden_size=2048, intermediate_size=6144,
                     moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8, norm_topk_prob=True,
                     num_attention_heads=32, num_key_value_heads=4, head_dim=128, num_hidden_layers=48,
                     vocab_size=151936, rms_norm_eps=1e-6, tie_word_embeddings=False, rope_theta=1000000.0)
TINY_MOE = dict(architectures=["Qwen3MoeForCausalLM"], hidden_size=2048, intermediate_size=6144,
                moe_intermediate_size=768, num_experts=16, num_experts_per_tok=4, norm_topk_prob=True,
                num_attention_heads=16, num_key_value_heads=2, head_dim=128, num_hidden_layers=2,
                vocab_size=1024, rms_norm_eps=1e-6, tie_word_embeddings=False, rope_theta=1000000.0)


def is_moe(config: dict) -> bool:
    return int(config.get("num_experts", 0)) > 0


def head_dim_of(config: dict) -> int:
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


def parameter_shapes(config: dict) -> list[tuple[str, tuple[int, ...]]]:
    """HF tensor names and shapes in state-dict order (the draw order)."""
    hidden, inter = config["hidden_size"], config["intermediate_size"]
    dim = head_dim_of(config)
    q, kv = config["num_attention_heads"] * dim, config["num_key_value_heads"] * dim
    shapes: list[tuple[str, tuple[int, ...]]] = [("model.embed_tokens.weight", (config["vocab_size"], hidden))]
    qk_norm = config["architectures"][0].startswith("Qwen3")
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        shapes += [
            (p + "input_layernorm.weight", (hidden,)),
            (p + "self_attn.q_proj.weight", (q, hidden)),
            (p + "self_attn.k_proj.weight", (kv, hidden)),
            (p + "self_attn.v_proj.weight", (kv, hidden)),
            (p + "self_attn.o_proj.weight", (hidden, q)),
        ]
        if qk_norm:
            shapes += [(p + "self_attn.q_norm.weight", (dim,)), (p + "self_attn.k_norm.weight", (dim,))]
        shapes.append((p + "post_attention_layernorm.weight", (hidden,)))
        if is_moe(config):
            expert_inter = int(config.get("moe_intermediate_size") or inter)
            shapes.append((p + "mlp.gate.weight", (config["num_experts"], hidden)))
            for expert in range(config["num_experts"]):
                e = p + f"mlp.experts.{expert}."
                shapes += [(e + "gate_proj.weight", (expert_inter, hidden)), (e + "up_proj.weight", (expert_inter, hidden)),
                           (e + "down_proj.weight", (hidden, expert_inter))]
        else:
            shapes += [
                (p + "mlp.gate_proj.weight", (inter, hidden)),
                (p + "mlp.up_proj.weight", (inter, hidden)),
                (p + "mlp.down_proj.weight", (hidden, inter)),
            ]
    shapes.append(("model.norm.weight", (hidden,)))
    if not config.get("tie_word_embeddings", False):
        shapes.append(("lm_head.weight", (config["vocab_size"], hidden)))
    return shapes


ROUTER_STD = 0.1


def seeded_weights(config: dict, seed: int = 0, dtype: torch.dtype = torch.float32,
                   device: str | torch.device = "cpu", std: float = 0.02) -> dict[str, torch.Tensor]:
    """Every matrix N(0, std) from one generator seeded with `seed`; norm weights 1.

    On the CPU the draws are fp32 and then cast, so a bf16 copy is exactly the
    rounding of the fp32 copy. On a CUDA device the generator is the device's
    (a different stream of numbers: use it for throughput runs, not for parity).
    """
    device = torch.device(device)
    generator = torch.Generator(device=device).manual_seed(seed)
    weights: dict[str, torch.Tensor] = {}
    for name, shape in parameter_shapes(config):
        if len(shape) == 1:
            weights[name] = torch.ones(shape, dtype=dtype, device=device)
        else:
            draw = torch.randn(shape, generator=generator, dtype=torch.float32, device=device)
            weights[name] = (draw * (ROUTER_STD if name.endswith("mlp.gate.weight") else std)).to(dtype)
    return weights


class LazySeededCheckpoint:
    """A checkpoint whose tensors are drawn when asked for, each from its own generator
    seeded by (seed, tensor name): for models too large to hold unpacked (a 70B-shaped
    model is 140 GB in bf16). Every process that asks for a name gets the same values,
    so tensor-parallel ranks cut their slices out of one consistent model. Throughput
    runs only: the draws are the device generator's, not the CPU draws of seeded_weights."""

    def __init__(self, config: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                 device: str | torch.device = "cuda", std: float = 0.02):
        self.shapes = dict(parameter_shapes(config))
        self.tie_word_embeddings = bool(config.get("tie_word_embeddings", False))
        self.seed, self.dtype, self.device, self.std = seed, dtype, torch.device(device), std

    def tensor(self, name: str) -> torch.Tensor:
        import zlib
        if name == "lm_head.weight" and name not in self.shapes and self.tie_word_embeddings:
            name = "model.embed_tokens.weight"
        if name not in self.shapes:
            raise KeyError(f"checkpoint has no {name}")
        shape = self.shapes[name]
        if len(shape) == 1:
            return torch.ones(shape, dtype=self.dtype, device=self.device)
        generator = torch.Generator(device=self.device).manual_seed((self.seed << 32) ^ zlib.crc32(name.encode()))
        draw = torch.empty(shape, dtype=self.dtype, device=self.device)
        return draw.normal_(0.0, ROUTER_STD if name.endswith("mlp.gate.weight") else self.std, generator=generator)


def seeded_tokens(batch: int, length: int, vocab: int, seed: int = 1) -> torch.Tensor:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (batch, length), generator=generator, dtype=torch.int64).to(torch.int32)


def seeded_contexts(batch: int, low: int, high: int, seed: int = 2) -> torch.Tensor:
    """Per-sequence context lengths uniform in [low, high]."""
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(low, high + 1, (batch,), generator=generator, dtype=torch.int64).to(torch.int32)


# BERT-base-shaped encoder (the forward workload) and a two-layer model with the same structure for tests.
BERT_BASE = dict(architectures=["BertModel"], hidden_size=768, intermediate_size=3072, num_attention_heads=12,
                 num_hidden_layers=12, vocab_size=30522, max_position_embeddings=512, type_vocab_size=2,
                 layer_norm_eps=1e-12, hidden_act="gelu", position_embedding_type="absolute")
TINY_BERT = dict(architectures=["BertModel"], hidden_size=256, intermediate_size=512, num_attention_heads=4,
                 num_hidden_layers=2, vocab_size=1000, max_position_embeddings=128, type_vocab_size=2,
                 layer_norm_eps=1e-12, hidden_act="gelu", position_embedding_type="absolute")


def encoder_parameter_shapes(config: dict) -> list[tuple[str, tuple[int, ...]]]:
    """BertModel tensor names and shapes in state-dict order (the draw order)."""
    hidden, inter = config["hidden_size"], config["intermediate_size"]
    shapes = [("embeddings.word_embeddings.weight", (config["vocab_size"], hidden)),
              ("embeddings.position_embeddings.weight", (config["max_position_embeddings"], hidden)),
              ("embeddings.token_type_embeddings.weight", (config["type_vocab_size"], hidden)),
              ("embeddings.LayerNorm.weight", (hidden,)), ("embeddings.LayerNorm.bias", (hidden,))]
    for layer in range(config["num_hidden_layers"]):
        p = f"encoder.layer.{layer}."
        for part in ("query", "key", "value"):
            shapes += [(p + f"attention.self.{part}.weight", (hidden, hidden)), (p + f"attention.self.{part}.bias", (hidden,))]
        shapes += [(p + "attention.output.dense.weight", (hidden, hidden)), (p + "attention.output.dense.bias", (hidden,)),
                   (p + "attention.output.LayerNorm.weight", (hidden,)), (p + "attention.output.LayerNorm.bias", (hidden,)),
                   (p + "intermediate.dense.weight", (inter, hidden)), (p + "intermediate.dense.bias", (inter,)),
                   (p + "output.dense.weight", (hidden, inter)), (p + "output.dense.bias", (hidden,)),
                   (p + "output.LayerNorm.weight", (hidden,)), (p + "output.LayerNorm.bias", (hidden,))]
    return shapes + [("pooler.dense.weight", (hidden, hidden)), ("pooler.dense.bias", (hidden,))]


def encoder_weights(config: dict, seed: int = 0) -> dict[str, torch.Tensor]:
    """Seeded N(0, 0.02) draws for every tensor (LayerNorm weights 1 + the draw, so that every scale and bias of
    the forward pass is exercised), fp32."""
    generator = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, shape in encoder_parameter_shapes(config):
        draw = torch.randn(shape, generator=generator, dtype=torch.float32) * 0.02
        tensors[name] = 1.0 + draw if name.endswith("LayerNorm.weight") else draw
    return tensors


def encoder_inputs(config: dict, batch: int, seq: int = 128, seed: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """Token ids uniform in [0, vocab) and segment ids in [0, type_vocab), int64 [batch, seq]."""
    generator = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, config["vocab_size"], (batch, seq), generator=generator, dtype=torch.int64)
    types = torch.randint(0, config["type_vocab_size"], (batch, seq), generator=generator, dtype=torch.int64)
    return ids, types
