"""CPU oracle for the decode path: a functional restatement of the reference's
PyTorch forward, python/tilemega/serving/export.py:18-172 (RMSNorm :18-27,
rotate_half :30-32, SelfAttention.forward :69-100, MLP :115-116, Layer :134-140,
Decoder.execute :165-172), with the KV cache held in 16-token blocks behind a
block table instead of being passed in and out as whole tensors.

TEST INFRASTRUCTURE ONLY. Nothing on the product path imports this file; only
tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may.

Pinned: tests/golden/*.pt hold logits and greedy tokens produced by the
reference module itself (tests/golden/make_golden.py imports it from the
reference tree); tests/test_oracle_golden.py checks this restatement against
them in fp32 and bf16.

Tensor parallelism (tp > 1) is restated as what T ranks compute together: the
rank modules of export.py:39-47,107-112,152-163 each produce the partial o_proj /
down_proj output of their contiguous slice of heads / intermediate columns (the
slices of python/tilemega/serving/weights.py:78-96), and the kernel epilogue
adds the ranks' partials, each already rounded to the model dtype, in fp32 in
ascending rank order, rounds the sum and then adds the residual
(include/tilemega/Backend/Sm90DenseEpilogue.h:43-86). The per-rank partials are
pinned by tests/golden/tiny_tp2.pt (made by tests/golden/make_golden_tp.py from
the reference's rank modules); the summation rule is read from the kernel source.
The sharded lm_head changes nothing: each rank scores a slice of the rows and the
ranks' winners are compared with ties to the smaller index (Sm90DenseHead.cuh:139-201).

Mixture of experts (config `num_experts`): the router, top-k and expert sum of
python/tilemega/moe/export.py:12-37,68-93 (softmax in fp32 over the router's
model-dtype logits, top-k, optional renormalisation kept in fp32, expert outputs in
the model dtype times the fp32 routing weight, fp32 sum over the k ranks, one
rounding), and the per-head QK norm of Qwen3 (serving/export.py:63-65,82-84).
`last_route[layer]` keeps the chosen expert indices [tokens][k] for the tests.

Every op is the same torch op on the same dtype as the reference, so in bf16 the
rounding sites are the reference's: one rounding per linear output, RMSNorm
`w * (x.float() * rsqrt(mean x^2 + eps)).to(dtype)`, RoPE product-product-sum,
scores rounded then divided by sqrt(D), softmax in fp32 cast back, SwiGLU and
residual adds in the model dtype.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

KV_BLOCK = 16


def head_dim_of(config: dict) -> int:
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    # export.py:24-27
    value = x.float()
    value = value * torch.rsqrt(value.square().mean(-1, keepdim=True) + eps)
    return weight * value.to(x.dtype)


def rotate_half(value: torch.Tensor) -> torch.Tensor:
    # export.py:30-32
    half = value.shape[-1] // 2
    return torch.cat((-value[..., half:], value[..., :half]), dim=-1)


def rope_tables(config: dict, capacity: int, dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [capacity][D]: default RoPE, computed in fp32, stored in bf16 (the
    reference hands bf16 tables to both the GPU plan and its module,
    python/tilemega/serving/state.py:30-59), then cast to the compute dtype."""
    dim = head_dim_of(config)
    theta = float(config.get("rope_theta", 10000.0))
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    angles = torch.arange(capacity, dtype=torch.float32)[:, None] * inv_freq[None, :]
    table = torch.cat((angles, angles), dim=-1)
    return table.cos().to(torch.bfloat16).to(dtype), table.sin().to(torch.bfloat16).to(dtype)


class PagedKV:
    """[L][2][num_blocks][Hkv][16][D] pool + int32 block table [B][max_blocks]."""

    def __init__(self, config: dict, batch: int, capacity: int, dtype: torch.dtype,
                 block_table: torch.Tensor | None = None, num_blocks: int | None = None):
        self.max_blocks = capacity // KV_BLOCK
        self.num_blocks = num_blocks or batch * self.max_blocks
        self.table = (block_table.clone().to(torch.int64) if block_table is not None
                      else torch.arange(batch * self.max_blocks).reshape(batch, self.max_blocks))
        if int(self.table.max()) >= self.num_blocks or int(self.table.min()) < 0:
            raise ValueError("block table entry outside the pool")
        self.pool = torch.zeros((config["num_hidden_layers"], 2, self.num_blocks, config["num_key_value_heads"],
                                 KV_BLOCK, head_dim_of(config)), dtype=dtype)

    def rows(self, positions: torch.Tensor, b: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(pool block, row in block) of each position of sequence b."""
        return self.table[b, positions // KV_BLOCK], positions % KV_BLOCK

    def append(self, layer: int, b: int, start: int, k: torch.Tensor, v: torch.Tensor) -> None:
        # k, v: [S][Hkv][D] for positions start .. start+S-1
        positions = torch.arange(start, start + k.shape[0])
        block, row = self.rows(positions, b)
        self.pool[layer, 0, block, :, row] = k
        self.pool[layer, 1, block, :, row] = v

    def gather(self, layer: int, b: int, length: int) -> tuple[torch.Tensor, torch.Tensor]:
        # -> [Hkv][length][D] in logical order
        block, row = self.rows(torch.arange(length), b)
        k = self.pool[layer, 0, block, :, row].transpose(0, 1)
        v = self.pool[layer, 1, block, :, row].transpose(0, 1)
        return k, v


class OracleDecoder:
    """forward(ids [B][S], start [B]) -> logits [B][S][V]; appends to the cache."""

    def __init__(self, config: dict, weights: dict[str, torch.Tensor], dtype: torch.dtype = torch.float32,
                 capacity: int = 256, attention_fp32: bool = False, tp: int = 1):
        # attention_fp32 restates the numerics of the reference's *kernel* instead of
        # its module: scores, softmax and the probability-value product stay in fp32
        # and only the context is rounded to the model dtype
        # (include/tilemega/Backend/Sm90DenseAttentionBody.cuh:248-302,371-403; the
        # module rounds scores and probabilities to bf16, export.py:94-99). With
        # dtype fp32 the two modes are the same computation.
        self.config = config
        self.dtype = dtype
        self.attention_fp32 = attention_fp32
        self.tp = tp
        for key in ("num_attention_heads", "num_key_value_heads", "intermediate_size", "vocab_size"):
            if config[key] % tp:
                raise ValueError(f"{key} does not divide by the tensor parallel degree {tp}")
        self.w = {name: tensor.to(dtype) for name, tensor in weights.items()}
        if "lm_head.weight" not in self.w:
            if not config.get("tie_word_embeddings", False):
                raise KeyError("untied model without lm_head.weight")
            self.w["lm_head.weight"] = self.w["model.embed_tokens.weight"]
        self.eps = float(config.get("rms_norm_eps", 1e-5))
        self.heads = config["num_attention_heads"]
        self.kv_heads = config["num_key_value_heads"]
        self.dim = head_dim_of(config)
        self.cos, self.sin = rope_tables(config, capacity, dtype)
        self.qk_norm = config["architectures"][0].startswith("Qwen3") if "architectures" in config else False
        self.experts = int(config.get("num_experts", 0))
        self.last_route: dict[int, torch.Tensor] = {}
        if self.experts and tp != 1:
            raise ValueError("tensor parallel MoE is out of scope (export.py:191-192)")

    def row_sharded_partials(self, x: torch.Tensor, weight: torch.Tensor) -> list[torch.Tensor]:
        """The ranks' partial outputs of a linear whose reduction axis is split into tp
        contiguous parts (o_proj, down_proj): one model-dtype rounding per rank."""
        width = weight.shape[1] // self.tp
        return [F.linear(x[..., q * width:(q + 1) * width], weight[:, q * width:(q + 1) * width])
                for q in range(self.tp)]

    def all_reduce(self, partials: list[torch.Tensor]) -> torch.Tensor:
        """Sm90DenseEpilogue.h:64-86: fp32 sum in ascending rank order, then one rounding."""
        if len(partials) == 1:
            return partials[0]
        total = torch.zeros_like(partials[0], dtype=torch.float32)
        for part in partials:
            total = total + part.float()
        return total.to(partials[0].dtype)

    def attention(self, layer: int, x: torch.Tensor, start: list[int], kv: PagedKV) -> torch.Tensor:
        return self.all_reduce(self.attention_partials(layer, x, start, kv))

    def mlp(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        return self.all_reduce(self.mlp_partials(layer, x))

    def attention_partials(self, layer: int, x: torch.Tensor, start: list[int], kv: PagedKV) -> list[torch.Tensor]:
        # export.py:69-100, one sequence at a time because lengths differ
        p = f"model.layers.{layer}.self_attn."
        batch, seq, _ = x.shape
        q = F.linear(x, self.w[p + "q_proj.weight"]).view(batch, seq, self.heads, self.dim)
        k = F.linear(x, self.w[p + "k_proj.weight"]).view(batch, seq, self.kv_heads, self.dim)
        v = F.linear(x, self.w[p + "v_proj.weight"]).view(batch, seq, self.kv_heads, self.dim)
        if self.qk_norm:
            # serving/export.py:82-84: each head normalised over its own D values, before RoPE
            q = rms_norm(q, self.w[p + "q_norm.weight"], self.eps)
            k = rms_norm(k, self.w[p + "k_norm.weight"], self.eps)
        context = torch.empty((batch, seq, self.heads * self.dim), dtype=x.dtype)
        for b in range(batch):
            positions = torch.arange(start[b], start[b] + seq)
            cosine = self.cos.index_select(0, positions).view(seq, 1, self.dim)
            sine = self.sin.index_select(0, positions).view(seq, 1, self.dim)
            qb = q[b] * cosine + rotate_half(q[b]) * sine
            kb = k[b] * cosine + rotate_half(k[b]) * sine
            kv.append(layer, b, start[b], kb, v[b])
            full_k, full_v = kv.gather(layer, b, start[b] + seq)
            query = qb.transpose(0, 1)                                   # [Hq][S][D]
            keys = torch.repeat_interleave(full_k, self.heads // self.kv_heads, dim=0)
            values = torch.repeat_interleave(full_v, self.heads // self.kv_heads, dim=0)
            key_position = torch.arange(start[b] + seq)[None, :]
            if self.attention_fp32:
                score = torch.matmul(query.float(), keys.float().transpose(-1, -2)) / math.sqrt(self.dim)
                score = score.masked_fill(key_position > positions[:, None], float("-inf"))
                attended = torch.matmul(torch.softmax(score, dim=-1), values.float()).to(x.dtype)
            else:
                score = torch.matmul(query, keys.transpose(-1, -2)) / math.sqrt(self.dim)
                score = score.masked_fill(key_position > positions[:, None], float("-inf"))
                probability = torch.softmax(score.float(), dim=-1).to(x.dtype)
                attended = torch.matmul(probability, values)
            context[b] = attended.transpose(0, 1).reshape(seq, self.heads * self.dim)
        return self.row_sharded_partials(context, self.w[p + "o_proj.weight"])

    def sparse_mlp(self, layer: int, x: torch.Tensor) -> torch.Tensor:
        # moe/export.py:68-93 (router) and :12-37 (experts)
        p = f"model.layers.{layer}.mlp."
        shape = x.shape
        rows = x.reshape(-1, shape[-1])
        logits = F.linear(rows, self.w[p + "gate.weight"])
        probability = torch.softmax(logits, -1, dtype=torch.float32)
        weight, index = torch.topk(probability, int(self.config["num_experts_per_tok"]), dim=-1)
        if self.config.get("norm_topk_prob", False):
            weight = weight / weight.sum(-1, keepdim=True)
        else:
            weight = weight.to(rows.dtype)
        self.last_route[layer] = index.clone()
        partials = torch.empty((rows.shape[0], index.shape[1], shape[-1]),
                               dtype=torch.promote_types(rows.dtype, weight.dtype))
        for expert in range(self.experts):
            token, rank = torch.where(index == expert)
            if token.numel():
                e = p + f"experts.{expert}."
                gate = F.linear(rows[token], self.w[e + "gate_proj.weight"])
                up = F.linear(rows[token], self.w[e + "up_proj.weight"])
                projected = F.linear(F.silu(gate) * up, self.w[e + "down_proj.weight"])
                partials[token, rank] = projected * weight[token, rank, None]
        return partials.sum(1, dtype=torch.float32).to(rows.dtype).reshape(shape)

    def mlp_partials(self, layer: int, x: torch.Tensor) -> list[torch.Tensor]:
        if self.experts:
            return [self.sparse_mlp(layer, x)]
        # export.py:115-116
        p = f"model.layers.{layer}.mlp."
        hidden = F.silu(F.linear(x, self.w[p + "gate_proj.weight"])) * F.linear(x, self.w[p + "up_proj.weight"])
        return self.row_sharded_partials(hidden, self.w[p + "down_proj.weight"])

    @torch.inference_mode()
    def forward(self, ids: torch.Tensor, start: list[int], kv: PagedKV,
                last_only: bool = False, head_fp32: bool = False) -> torch.Tensor:
        # export.py:134-140,165-172. head_fp32 returns the lm_head products of the
        # same (model-dtype) normalised hidden state accumulated and kept in fp32,
        # i.e. the logits before their final rounding to the model dtype.
        x = F.embedding(ids.long(), self.w["model.embed_tokens.weight"])
        for layer in range(self.config["num_hidden_layers"]):
            p = f"model.layers.{layer}."
            x = x + self.attention(layer, rms_norm(x, self.w[p + "input_layernorm.weight"], self.eps), start, kv)
            x = x + self.mlp(layer, rms_norm(x, self.w[p + "post_attention_layernorm.weight"], self.eps))
        if last_only:
            x = x[:, -1:]
        normed = rms_norm(x, self.w["model.norm.weight"], self.eps)
        if head_fp32:
            return F.linear(normed.float(), self.w["lm_head.weight"].float())
        return F.linear(normed, self.w["lm_head.weight"])

    @torch.inference_mode()
    def greedy(self, prompt: torch.Tensor, new_tokens: int, kv: PagedKV, start: list[int] | None = None,
               forced: torch.Tensor | None = None, head_fp32: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
        """Prefill `prompt` [B][P], then decode. Returns (tokens [B][new], logits
        [new][B][V] as fp32). Ties go to the smaller index (torch.argmax on CPU
        returns the first maximum). With `forced` [B][new] the history follows
        `forced` instead of the oracle's own argmax (teacher forcing). The argmax
        always sees the logits rounded to the model dtype (the reference compares
        rounded logits); head_fp32 only changes what is returned."""
        batch, length = prompt.shape
        start = list(start) if start is not None else [0] * batch
        logits = self.forward(prompt, start, kv, last_only=True, head_fp32=head_fp32)[:, -1].float()
        tokens, history = [], []
        for step in range(new_tokens):
            history.append(logits)
            chosen = logits.to(self.dtype).float().argmax(-1)
            tokens.append(chosen)
            if step + 1 == new_tokens:
                break
            feed = forced[:, step].long() if forced is not None else chosen
            position = [s + length + step for s in start]
            logits = self.forward(feed.view(batch, 1).to(torch.int32), position, kv,
                                  head_fp32=head_fp32)[:, -1].float()
        return torch.stack(tokens, dim=1).to(torch.int32), torch.stack(history)
