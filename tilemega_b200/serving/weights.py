"""Checkpoint tensors -> the packed device buffers a plan's table asks for.

Same role as python/tilemega/serving/weights.py:99-313 of the reference: every
weight buffer of a plan carries a `pack_json` recipe that names checkpoint
tensors by their HF names; this module evaluates the recipe kinds the dense
decode plan uses (alias, qkv_group_interleave, gate_up_interleave, tile_pages).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Mapping

import torch

from .plan import Buffer, PlanLibrary

DTYPES = {0: torch.bfloat16, 1: torch.float32, 2: torch.int32, 3: torch.int64, 4: torch.uint8,   # 4: e4m3 bytes, 5: fp16 (additions
          5: torch.float16}                                                                     # of this library)
E4M3_MAX = 448.0


def _tied_name(name: str, known, tied: bool) -> str:
    """A tied model has no lm_head tensor of its own: the embedding table stands in."""
    return "model.embed_tokens.weight" if tied and name == "lm_head.weight" and name not in known else name


class Checkpoint:
    """The *.safetensors files of a model directory, addressed by HF tensor name. Tensors are
    read one at a time when a recipe asks for them (the reference's loader works the same
    way, python/tilemega/serving/weights.py:17-49), so the host never holds the whole model."""

    def __init__(self, model_dir: str | Path):
        from safetensors import safe_open
        self._reader = lambda path: safe_open(path, framework="pt", device="cpu")
        self.model_dir = Path(model_dir)
        self.tie_word_embeddings = False
        config = self.model_dir / "config.json"
        if config.exists():
            self.tie_word_embeddings = bool(json.loads(config.read_text()).get("tie_word_embeddings", False))
        self.files: dict[str, Path] = {}
        for shard in sorted(self.model_dir.glob("*.safetensors")):
            with self._reader(shard) as handle:
                names = list(handle.keys())
            clash = [name for name in names if name in self.files]
            if clash:
                raise ValueError(f"duplicate checkpoint tensor {clash[0]}")
            self.files.update((name, shard) for name in names)
        if not self.files:
            raise FileNotFoundError(f"no safetensors in {self.model_dir}")

    def tensor(self, name: str) -> torch.Tensor:
        name = _tied_name(name, self.files, self.tie_word_embeddings)
        if name not in self.files:
            raise KeyError(f"checkpoint has no {name}")
        with self._reader(self.files[name]) as handle:
            return handle.get_tensor(name)


class TensorCheckpoint:
    """An in-memory checkpoint (name -> tensor), e.g. seeded random weights."""

    def __init__(self, tensors: Mapping[str, torch.Tensor], tie_word_embeddings: bool = False):
        self.tensors = tensors
        self.tie_word_embeddings = tie_word_embeddings

    def tensor(self, name: str) -> torch.Tensor:
        name = _tied_name(name, self.tensors, self.tie_word_embeddings)
        if name not in self.tensors:
            raise KeyError(f"checkpoint has no {name}")
        return self.tensors[name]


def tile_pages(weight: torch.Tensor, tile_n: int, tile_k: int) -> torch.Tensor:
    """[N][K] -> [N/tn][K/tk][tn*tk] pages, each 8x64 atom 128-byte XOR swizzled.

    Layout contract (reference weights.py:239-240, tk >= 64): element (row, col)
    of a page sits at 512*(row//8 + (tn//8)*(col//64)) + 64*(row%8) +
    8*((col%64//8) ^ (row%8)) + col%8. Built here as a reshape: the page is
    [col//64][row//8][row%8][chunk][8] and the chunk axis is permuted by row%8.
    """
    if weight.ndim != 2 or tile_n <= 0 or tile_k <= 0 or tile_n % 8 or tile_k % 64:
        raise ValueError("invalid tile_pages source or geometry")
    if weight.is_cuda and weight.element_size() == 2 and weight.shape[1] % 8 == 0:
        return tile_pages_on_device(weight, tile_n, tile_k)
    return tile_pages_by_indexing(weight, tile_n, tile_k)


_PACKER = None


def tile_pages_on_device(weight: torch.Tensor, tile_n: int, tile_k: int) -> torch.Tensor:
    """The same layout written by the library's pack kernel (tm_pack_tile_pages): one pass over
    the matrix on the device instead of a chain of indexing ops."""
    global _PACKER
    if _PACKER is None:
        import ctypes as C
        from ..build import build_library
        _PACKER = C.CDLL(str(build_library())).tm_pack_tile_pages
        _PACKER.restype = C.c_int
        _PACKER.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    if weight.stride(1) != 1 or weight.stride(0) % 8 or weight.data_ptr() % 16:
        weight = weight.contiguous()
    n, k = weight.shape
    pages = -(-n // tile_n) * -(-k // tile_k)
    packed = torch.empty(pages * tile_n * tile_k, dtype=weight.dtype, device=weight.device)
    with torch.cuda.device(weight.device):
        status = _PACKER(weight.data_ptr(), n, k, weight.stride(0), tile_n, tile_k, packed.data_ptr(),
                         torch.cuda.current_stream().cuda_stream)
    if status != 0:
        raise RuntimeError(f"tm_pack_tile_pages failed ({status})")
    return packed


def tile_pages_by_indexing(weight: torch.Tensor, tile_n: int, tile_k: int) -> torch.Tensor:
    """The layout of tile_pages as tensor indexing (any device and dtype): the definition the
    pack kernel is tested against."""
    n, k = weight.shape
    nt, kt = -(-n // tile_n), -(-k // tile_k)
    if (nt * tile_n, kt * tile_k) != (n, k):
        padded = torch.zeros((nt * tile_n, kt * tile_k), dtype=weight.dtype, device=weight.device)
        padded[:n, :k] = weight
        weight = padded
    # axes: nt, row-group, row-in-group, kt, column-block, chunk, element
    view = weight.reshape(nt, tile_n // 8, 8, kt, tile_k // 64, 8, 8)
    view = view.permute(0, 3, 4, 1, 2, 5, 6)  # nt, kt, cb, rg, r, chunk, e
    rows = torch.arange(8, device=weight.device)
    source_chunk = rows[:, None] ^ rows[None, :]  # physical chunk c' of row r holds logical chunk c' ^ r
    swizzled = view[:, :, :, :, rows[:, None], source_chunk, :]
    return swizzled.reshape(-1).contiguous()


def sharded(recipe: Mapping[str, object], source: Callable[[str], torch.Tensor],
            tp_rank: int) -> Callable[[str], torch.Tensor]:
    """Megatron tensor parallelism (reference weights.py:78-96): a recipe with
    "shard": {"axis", "parts"} names whole checkpoint tensors, and a rank packs only
    its contiguous part of each of them: rows (axis 0) for q/k/v, gate/up and
    lm_head, columns (axis 1) for o and down."""
    spec = recipe.get("shard")
    if spec is None:
        return source
    axis, parts = int(spec["axis"]), int(spec["parts"])
    if axis not in (0, 1) or parts < 2 or not 0 <= tp_rank < parts:
        raise ValueError(f"invalid shard {spec} for tensor parallel rank {tp_rank}")

    def narrowed(name: str) -> torch.Tensor:
        tensor = source(name)
        if tensor.ndim != 2 or tensor.shape[axis] % parts:
            raise ValueError(f"{name} {tuple(tensor.shape)} does not split into {parts} on axis {axis}")
        size = tensor.shape[axis] // parts
        return tensor.narrow(axis, tp_rank * size, size).contiguous()
    return narrowed


def _sources(recipe: Mapping[str, object], source: Callable[[str], torch.Tensor]) -> list[torch.Tensor]:
    tensors = [source(str(name)) for name in recipe["sources"]]
    if not all(item.ndim == 2 for item in tensors) or len({item.shape[1] for item in tensors}) != 1:
        raise ValueError("packed GEMM sources must be matrices with one K")
    return tensors


def expert_matrices(recipe: Mapping[str, object], source: Callable[[str], torch.Tensor]):
    """The per-expert matrices of an expert_stack recipe, in expert order: gate/up rows
    interleaved in units of `u` (as gate_up_interleave), or the down projection
    (reference python/tilemega/moe/weights.py:15-47,56-76; names are the HF per-expert ones)."""
    prefix, part = str(recipe["prefix"]), recipe["part"]
    experts, hidden, inter, unit = (int(recipe[key]) for key in ("experts", "hidden", "intermediate", "u"))
    if part not in ("gate_up", "down") or min(experts, hidden, inter, unit) <= 0 or inter % unit or not prefix.endswith("."):
        raise ValueError("invalid expert stack recipe")
    for expert in range(experts):
        if part == "gate_up":
            gate = source(f"{prefix}{expert}.gate_proj.weight")
            up = source(f"{prefix}{expert}.up_proj.weight")
            if tuple(gate.shape) != (inter, hidden) or tuple(up.shape) != (inter, hidden):
                raise ValueError("expert projection has an incompatible shape")
            yield torch.stack((gate.reshape(-1, unit, hidden), up.reshape(-1, unit, hidden)), dim=1).reshape(-1, hidden)
        else:
            down = source(f"{prefix}{expert}.down_proj.weight")
            if tuple(down.shape) != (hidden, inter):
                raise ValueError("expert projection has an incompatible shape")
            yield down


def quantize_e4m3(matrix: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Row-wise e4m3 quantisation of a weight matrix [N][K]: scale[n] = max_k |W[n][k]| * fp32(1/448) (1 for an
    all-zero row), code[n][k] = e4m3(W[n][k] / scale[n]) rounded to nearest even. Returns the codes as
    uint8 [N][K] and the scales as float32 [N]; code * scale is the weight the kernel multiplies with."""
    if matrix.ndim != 2:
        raise ValueError("e4m3 quantisation takes a matrix")
    values = matrix.float()
    peak = values.abs().amax(dim=1)
    # (a multiplication by the rounded reciprocal, not a division by 448: libraries may turn a division by a
    # constant into exactly this on one device and not on another, and the scales must not depend on that)
    scale = torch.where(peak > 0, peak * torch.tensor(1.0 / E4M3_MAX, dtype=torch.float32, device=peak.device),
                        torch.ones_like(peak))
    # The rounding is spelled out in exact float operations (power-of-two steps, round half to even) so
    # that every device and library version derives the same codes; the cast at the end is then exact.
    scaled = values / scale[:, None]
    magnitude = scaled.abs()
    _, exponent = torch.frexp(magnitude)                       # magnitude = m * 2^exponent, m in [0.5, 1)
    step = torch.ldexp(torch.ones_like(magnitude), (exponent - 1).clamp_min(-6) - 3)   # 3 mantissa bits; subnormals below 2^-6
    rounded = (torch.round(magnitude / step) * step).clamp_max(E4M3_MAX)
    codes = torch.copysign(rounded, scaled).to(torch.float8_e4m3fn)
    return codes.view(torch.uint8), scale


def dequantize_e4m3(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """float32 [N][K]: the weights an e4m3 plan computes with."""
    return codes.view(torch.float8_e4m3fn).float() * scale[:, None].float()


def pack(recipe: Mapping[str, object], source: Callable[[str], torch.Tensor], tp_rank: int = 0) -> torch.Tensor:
    kind = recipe["kind"]
    if kind in ("e4m3_pairs", "e4m3_scale"):
        # the inner recipe's matrix (this rank's slice, rows already interleaved), quantised row by row
        codes, scale = quantize_e4m3(pack(recipe["source"], source, tp_rank))
        if kind == "e4m3_scale":
            return scale.contiguous()
        if codes.shape[1] % 2:
            raise ValueError("e4m3 weight rows need an even number of columns")
        return codes.contiguous().view(torch.bfloat16)   # two codes per 2-byte unit: tile_pages applies unchanged
    source = sharded(recipe, source, tp_rank)
    if kind == "alias":
        return source(str(recipe["source"]))
    if kind == "tile_pages":
        inner = recipe["source"]
        if isinstance(inner, Mapping) and inner.get("kind") == "expert_stack":
            # every expert packed by itself, the packed experts one after the other
            # (reference python/tilemega/moe/weights.py:56-88)
            return torch.cat([tile_pages(matrix, int(recipe["tile_n"]), int(recipe["tile_k"]))
                              for matrix in expert_matrices(inner, source)])
        return tile_pages(pack(inner, source, tp_rank), int(recipe["tile_n"]), int(recipe["tile_k"]))
    if kind == "qkv_group_interleave":
        # rows per KV head: its query heads, then its key head, then its value head
        # (reference weights.py:246-256)
        q, k, v = _sources(recipe, source)
        hkv, qperkv, dim = (int(recipe[key]) for key in ("hkv", "qperkv", "head_dim"))
        if q.shape[0] != hkv * qperkv * dim or k.shape[0] != hkv * dim or v.shape[0] != hkv * dim:
            raise ValueError("QKV recipe and checkpoint shapes disagree")
        width = q.shape[1]
        grouped = torch.cat((q.reshape(hkv, qperkv * dim, width), k.reshape(hkv, dim, width),
                             v.reshape(hkv, dim, width)), dim=1)
        return grouped.reshape(-1, width)
    if kind == "gate_up_interleave":
        # u gate rows, then the u matching up rows (reference weights.py:257-264)
        gate, up = _sources(recipe, source)
        unit = int(recipe["u"])
        if gate.shape != up.shape or unit <= 0 or gate.shape[0] % unit:
            raise ValueError("gate/up interleave shape mismatch")
        width = gate.shape[1]
        return torch.stack((gate.reshape(-1, unit, width), up.reshape(-1, unit, width)), dim=1).reshape(-1, width)
    raise ValueError(f"unsupported packing recipe {kind}")


def weight_recipes(*plans: PlanLibrary) -> dict[str, Buffer]:
    """Every buffer of the plans that carries a packing recipe, by name; plans that share a
    weight must describe it identically."""
    chosen: dict[str, Buffer] = {}
    for buffer in (buffer for plan in plans for buffer in plan.buffers if buffer.pack_json):
        seen = chosen.setdefault(buffer.name, buffer)
        if (seen.pack_json, seen.dtype, seen.elements_constant) != (buffer.pack_json, buffer.dtype, buffer.elements_constant):
            raise ValueError(f"plans disagree on weight {buffer.name}")
    return chosen


def load_weights(checkpoint: str | Path | Checkpoint | TensorCheckpoint, *plans: PlanLibrary,
                 device: str | torch.device = "cuda", tp: tuple[int, int] = (0, 1)) -> dict[str, torch.Tensor]:
    """Pack every recipe buffer of the plans on `device` (bf16 unless the table says otherwise).
    `tp` = (rank, world): this rank's slices of a tensor-parallel plan's weights."""
    tp_rank, tp_world = tp
    if any(plan.tp_world != tp_world for plan in plans):
        raise ValueError("the plans' tensor parallel degree differs from the requested one")
    if isinstance(checkpoint, (str, Path)):
        checkpoint = Checkpoint(checkpoint)
    device = torch.device(device)
    result: dict[str, torch.Tensor] = {}
    packed: dict[str, torch.Tensor] = {}
    for name, buffer in weight_recipes(*plans).items():
        if buffer.pack_json not in packed:
            recipe = json.loads(buffer.pack_json)
            # checkpoint tensors are staged in the model dtype; e4m3 codes and their scales are both derived from that
            derived = buffer.dtype == 4 or recipe.get("kind") == "e4m3_scale"
            dtype = torch.bfloat16 if derived else DTYPES[buffer.dtype]
            staged: dict[str, torch.Tensor] = {}

            def source(fqn: str) -> torch.Tensor:
                if fqn not in staged:
                    staged[fqn] = checkpoint.tensor(fqn).to(device=device, dtype=dtype).contiguous()
                return staged[fqn]

            packed[buffer.pack_json] = pack(recipe, source, tp_rank).contiguous()
        tensor = packed[buffer.pack_json]
        if buffer.dtype == 4:
            tensor = packed[buffer.pack_json] = tensor.view(torch.uint8)   # one element per e4m3 byte
        if tensor.numel() != buffer.elements_constant:
            raise ValueError(f"{name} has {tensor.numel()} elements; plan expects {buffer.elements_constant}")
        result[name] = tensor
    return result
