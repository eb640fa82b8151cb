"""Device-resident request state of a decode plan: token ids, RoPE tables, KV.

Mirrors python/tilemega/serving/state.py:62-112 of the reference (one contiguous
[L][2][B][Hkv][capacity][D] bf16 allocation exposed as kv_cache.k.{l} /
kv_cache.v.{l}) and adds the block-table form: a pool
[L][2][num_blocks][Hkv][16][D] with `serving.block_table` i32 [B][capacity/16]
and `serving.context_base` i32 [B] (per-sequence position offset).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .plan import PlanLibrary

KV_BLOCK = 16


@dataclass
class ServingState:
    tensors: dict[str, torch.Tensor]
    kv_storage: torch.Tensor
    tokens: torch.Tensor
    block_table: torch.Tensor | None = None
    context_base: torch.Tensor | None = None
    extras: dict = field(default_factory=dict)

    @property
    def pointers(self) -> dict[str, int]:
        return {name: tensor.data_ptr() for name, tensor in self.tensors.items()}


def head_dim_of(config: dict) -> int:
    return int(config.get("head_dim") or config["hidden_size"] // config["num_attention_heads"])


def inverse_frequencies(config: dict) -> torch.Tensor:
    """inv_freq [D/2] in fp32: theta^(-2i/D), then the checkpoint's `rope_scaling`.

    The reference takes its tables from the HF rotary module (python/tilemega/serving/state.py:30-59),
    which applies the scaling the config names. Built here: "default", "linear" (every frequency
    divided by `factor`) and "llama3" (Llama 3.1/3.2 checkpoints: wavelengths longer than
    original_max_position_embeddings / low_freq_factor are slowed by `factor`, wavelengths shorter than
    original / high_freq_factor are kept, the band between is interpolated). All three leave the
    attention scale at 1. Anything else is refused."""
    dim = head_dim_of(config)
    theta = float(config.get("rope_theta", 10000.0))
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
    scaling = config.get("rope_scaling") or {}
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    if kind == "default":
        return inv_freq
    if kind not in ("linear", "llama3"):
        raise ValueError(f"rope_scaling of type {kind!r} is not built (default, linear, llama3 are)")
    factor = float(scaling["factor"])
    if kind == "linear":
        return inv_freq / factor
    if kind == "llama3":
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position_embeddings"])
        wavelength = 2.0 * math.pi / inv_freq
        slowed = torch.where(wavelength > original / low, inv_freq / factor, inv_freq)
        blend = (original / wavelength - low) / (high - low)
        between = (1.0 - blend) * slowed / factor + blend * slowed
        in_band = (wavelength >= original / high) & (wavelength <= original / low)
        return torch.where(in_band, between, slowed)
    raise AssertionError(kind)


def rotary_tables(config: dict, capacity: int, device: torch.device | str) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 cos/sin [capacity][D], the half duplicated (rotate-half convention): angles
    position * inv_freq in fp32, cosine and sine in fp32, cast to the model dtype."""
    inv_freq = inverse_frequencies(config)
    angles = torch.arange(capacity, dtype=torch.float32)[:, None] * inv_freq[None, :]
    table = torch.cat((angles, angles), dim=-1)
    return (table.cos().to(torch.bfloat16).to(device).contiguous(),
            table.sin().to(torch.bfloat16).to(device).contiguous())


def kv_row_swizzle(rows: torch.Tensor) -> torch.Tensor:
    """Convert KV rows between logical order and the plan's storage order.

    `rows` is [..., T, D] with T the row position inside its allocation (a 16-row
    block of the pool, or the capacity axis of the contiguous cache). The kernel
    keeps 16-byte chunk c of the row at position t at chunk c ^ (t mod 8), so that
    the eight rows of a shared-memory matrix load sit on different banks. The
    mapping is its own inverse: call it to bring history into a cache, and again
    to read rows back. The reference's driver only zero-fills its cache
    (python/tilemega/serving/state.py:86-98), for which this is the identity.
    """
    t, d = rows.shape[-2], rows.shape[-1]
    if d % 8:
        raise ValueError("head_dim must be a multiple of 8")
    chunk = torch.arange(d // 8, device=rows.device)[None, :] ^ (torch.arange(t, device=rows.device)[:, None] & 7)
    index = (chunk[:, :, None] * 8 + torch.arange(8, device=rows.device)).reshape(t, d)
    return torch.gather(rows, -1, index.expand(rows.shape))


def shuffled_block_table(batch: int, max_blocks: int, num_blocks: int, seed: int = 0) -> torch.Tensor:
    """A seeded permutation of the pool dealt to the sequences: [B][max_blocks] int32."""
    if num_blocks < batch * max_blocks:
        raise ValueError("the pool is smaller than batch * max_blocks")
    generator = torch.Generator().manual_seed(seed)
    order = torch.randperm(num_blocks, generator=generator)[:batch * max_blocks]
    return order.reshape(batch, max_blocks).to(torch.int32)


def allocate_state(config: dict, batch: int, decode: PlanLibrary, device: str | torch.device = "cuda",
                   block_table: torch.Tensor | None = None,
                   context_base: torch.Tensor | None = None, tp: int = 1,
                   shared_blocks: bool = False, kv_storage: torch.Tensor | None = None) -> ServingState:
    """`tp`: a tensor-parallel rank's state holds only its num_key_value_heads / tp KV heads
    (reference state.py:64-82); token state and RoPE tables are whole on every rank."""
    if decode.info.phase != 1:
        raise ValueError("allocate_state needs a decode plan")
    if not decode.info.batch_lo <= batch <= decode.info.batch_hi:
        raise ValueError("batch outside the plan's solved interval")
    device = torch.device(device)
    capacity = decode.info.capacity
    layers = int(config["num_hidden_layers"])
    hkv = int(config["num_key_value_heads"])
    if tp < 1 or hkv % tp:
        raise ValueError(f"{hkv} KV heads do not split across tensor parallel degree {tp}")
    hkv //= tp
    dim = head_dim_of(config)
    names = {buffer.name for buffer in decode.buffers}
    tokens = torch.zeros((batch, capacity), dtype=torch.int32, device=device)
    cos, sin = rotary_tables(config, capacity, device)
    result: dict[str, torch.Tensor] = {"serving.tokens": tokens, "serving.rope_cos": cos, "serving.rope_sin": sin}
    table = base = None
    if "serving.block_table" in names:
        num_blocks = int(decode.manifest["kv"]["num_blocks"])
        max_blocks = capacity // KV_BLOCK
        # rows past a sequence's length are masked by selection, so the pool starts zeroed
        # `kv_storage`: the pool of another plan of the same model (a prefill plan and a decode plan serve the
        # same sequences out of one pool)
        shape = (layers, 2, num_blocks, hkv, KV_BLOCK, dim)
        if kv_storage is None:
            kv_storage = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        elif tuple(kv_storage.shape) != shape or kv_storage.dtype != torch.bfloat16 or kv_storage.device != device:
            raise ValueError("the shared KV pool has another shape, dtype or device than this plan's")
        table = (block_table if block_table is not None
                 else torch.arange(batch * max_blocks, dtype=torch.int32).reshape(batch, max_blocks))
        if tuple(table.shape) != (batch, max_blocks) or table.dtype != torch.int32:
            raise ValueError("block table must be int32 [batch][capacity/16]")
        if int(table.min()) < 0 or int(table.max()) >= num_blocks:
            raise ValueError("block table entry outside the pool")
        # a static batch owns every block it names; a scheduler that parks idle rows on one scratch block
        # (serving/continuous.py) passes shared_blocks=True and keeps the live rows disjoint itself
        if not shared_blocks and table.reshape(-1).unique().numel() != table.numel():
            raise ValueError("block table maps two logical blocks to one pool block")
        table = table.to(device).contiguous()
        base = (context_base if context_base is not None else torch.zeros(batch, dtype=torch.int32))
        if tuple(base.shape) != (batch,) or base.dtype != torch.int32 or int(base.min()) < 0:
            raise ValueError("context_base must be non-negative int32 [batch]")
        base = base.to(device).contiguous()
        result["serving.block_table"] = table
        result["serving.context_base"] = base
        for layer in range(layers):
            result[f"kv_pool.k.{layer}"] = kv_storage[layer, 0]
            result[f"kv_pool.v.{layer}"] = kv_storage[layer, 1]
    else:
        if block_table is not None or context_base is not None:
            raise ValueError("this plan has a contiguous KV cache; it takes no block table")
        kv_storage = torch.zeros((layers, 2, batch, hkv, capacity, dim), dtype=torch.bfloat16, device=device)
        for layer in range(layers):
            result[f"kv_cache.k.{layer}"] = kv_storage[layer, 0]
            result[f"kv_cache.v.{layer}"] = kv_storage[layer, 1]
    for buffer in decode.buffers:
        if buffer.role != 1 or buffer.pack_json:
            continue
        tensor = result.get(buffer.name)
        if tensor is None:
            raise KeyError(f"unknown external request buffer {buffer.name}")
        expected = {0: torch.bfloat16, 1: torch.float32, 2: torch.int32}[buffer.dtype]
        if tensor.dtype != expected or tensor.numel() != buffer.elements_constant + batch * buffer.elements_per_batch:
            raise ValueError(f"{buffer.name} conflicts with plan metadata")
        if not tensor.is_contiguous():
            raise ValueError(f"{buffer.name} is not contiguous")
    return ServingState(result, kv_storage, tokens, table, base)
