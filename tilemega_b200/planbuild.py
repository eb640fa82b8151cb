"""Emit one plan library: a copy of libtilemega_b200.so next to its JSON sidecar.

TileMega's compiler produces one shared object per (model, phase, batch
interval) and `tm_plan_query` takes no argument (reference:
include/tilemega/Codegen/tasks/ServingAbi.h:33). Here the kernels are generic
over the model dimensions, so "compiling a plan" is writing the sidecar the
library reads at load time; the copy gives each plan its own file identity, which
is what `ctypes.CDLL` keys loaded libraries on.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from pathlib import Path

from .build import LIB_DIR, LIBRARY, build_library

# Plan libraries are emitted inside the package tree (a git-ignored folder next to the built
# library), so that every shared object a process loads is one of this repository's files.
PLAN_DIR = LIB_DIR / "plans"

MODEL_KEYS = ("hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads",
              "head_dim", "num_hidden_layers", "vocab_size", "rms_norm_eps", "tie_word_embeddings",
              "rope_theta", "architectures", "num_experts", "num_experts_per_tok", "moe_intermediate_size",
              "norm_topk_prob")


ENCODER_KEYS = ("hidden_size", "intermediate_size", "num_attention_heads", "num_hidden_layers", "vocab_size",
                "max_position_embeddings", "type_vocab_size", "layer_norm_eps", "hidden_act", "position_embedding_type")


def forward_document(config: dict, *, batch_lo: int = 1, batch_hi: int | None = None, seq: int = 128,
                     dtype: str = "f16", mask: bool = False) -> dict:
    """The sidecar of a forward plan (phase 2): a stateless BERT-shaped encoder pass over batch x seq tokens."""
    model = {key: config[key] for key in ENCODER_KEYS if key in config}
    batch_hi = batch_lo if batch_hi is None else batch_hi
    if not 1 <= batch_lo <= batch_hi <= 512:
        raise ValueError("forward batch interval must lie in [1, 512]")
    if seq != 128:
        raise ValueError("forward plans run sequences of 128 positions")
    if dtype not in ("f16", "bf16"):
        raise ValueError("dtype must be 'f16' or 'bf16'")
    if config["hidden_size"] != 64 * config["num_attention_heads"] or config["hidden_size"] % 128 or config["hidden_size"] > 1024:
        raise ValueError("encoder heads must be 64 wide, the hidden size a multiple of 128 up to 1024")
    if config["intermediate_size"] % 128:
        raise ValueError("encoder intermediate size must be a multiple of 128")
    document = {"execution": "graph", "arch": "sm_100a", "phase": "forward", "model": model, "batch_lo": batch_lo,
                "batch_hi": batch_hi, "seq": seq, "dtype": dtype}
    if mask:
        document["mask"] = True   # a third input, "attention_mask" (int64 [batch, seq]; 0 hides a key position)
    return document


def plan_document(config: dict, *, batch_lo: int = 1, batch_hi: int | None = None, capacity: int,
                  kv_layout: str = "contiguous", num_blocks: int = 0, geometry: dict | None = None,
                  grid: int = 0, slots: int = 0, write_logits: bool = True,
                  tp: int = 1,
                  attn_min_slots: int | None = None,
                  weights: str = "bf16", chunk_rows: bool = False, phase: str = "decode", seq: int = 0) -> dict:
    """The sidecar for one decode plan; raises ValueError on shapes the kernels do not cover."""
    model = {key: config[key] for key in MODEL_KEYS if key in config}
    model.setdefault("head_dim", config["hidden_size"] // config["num_attention_heads"])
    model.setdefault("rms_norm_eps", 1e-5)
    batch_hi = batch_lo if batch_hi is None else batch_hi
    if phase not in ("decode", "prefill"):
        raise ValueError("phase must be 'decode' or 'prefill'")
    prefill = phase == "prefill"
    if prefill and (not 1 <= batch_lo <= batch_hi <= 64 or not 1 <= seq < capacity):
        raise ValueError("a prefill plan covers 1..64 sequences of seq positions, 1 <= seq < capacity")
    # batch 16..64 (and every prefill plan): the GEMM stages run on tcgen05 tiles, weight pages are 128 x 128
    dense_batch = batch_hi > 8 or prefill
    if dense_batch and not prefill and (batch_lo <= 8 or batch_hi > 64 or batch_lo % 16 or batch_hi % 16 or batch_lo > batch_hi):
        raise ValueError("a dense-batch plan covers batch sizes 16, 32, 48, 64 (interval bounds multiples of 16)")
    if not dense_batch and not 1 <= batch_lo <= batch_hi:
        raise ValueError("batch interval must lie in [1, 8], or in [16, 64] in steps of 16")
    if capacity < 16 or capacity % 16:
        raise ValueError("capacity must be a positive multiple of the KV block (16)")
    if kv_layout not in ("contiguous", "paged"):
        raise ValueError("kv_layout must be 'contiguous' or 'paged'")
    # the pool may be smaller than batch_hi * capacity / 16 blocks: a scheduler that knows its sequences' lengths
    # (serving/continuous.py) hands out blocks on demand; a static batch with full-length rows needs that many
    if kv_layout == "paged" and num_blocks < 2:
        raise ValueError("a paged plan needs a pool of at least 2 blocks (kv num_blocks)")
    if tp not in (1, 2, 4, 8):
        raise ValueError("tensor parallel degree must be 1, 2, 4 or 8")
    for key in ("num_attention_heads", "num_key_value_heads", "intermediate_size", "vocab_size"):
        if config[key] % tp:
            raise ValueError(f"{key}={config[key]} is not divisible by the tp degree {tp}")
    document = {
        "execution": "megakernel", "pg": "ring", "arch": "sm_100a", "phase": phase,
        "model": model, "batch_lo": batch_lo, "batch_hi": batch_hi, "capacity": capacity,
        "kv": {"layout": kv_layout, "block": 16, "num_blocks": num_blocks},
        "geometry": geometry or {}, "grid": grid, "slots": slots, "write_logits": write_logits,
    }
    if tp > 1:
        document["tp"] = tp   # the plan is ONE rank's: every rank loads the same library
    if weights not in ("bf16", "e4m3"):
        raise ValueError("weights must be 'bf16' or 'e4m3'")
    if weights == "e4m3":
        document["weights"] = "e4m3"   # GEMV matrices as e4m3 bytes + one fp32 scale per output row
    if prefill:
        # the plan's ONE step runs the prompts of batch sequences, seq positions each, as (sequence, position) rows
        document["seq"] = seq
    if chunk_rows:
        if not dense_batch or kv_layout != "paged":
            raise ValueError("chunk_rows (rows of one sequence at consecutive positions) needs a paged dense-batch plan")
        document["chunk_rows"] = True   # every row's key and value are appended before any row attends
    if attn_min_slots is not None:
        document["attn_min_slots"] = attn_min_slots   # least ring slots of keys per attention task
    return document


def emit_plan(config: dict, out_dir: str | Path | None = None, **options) -> Path:
    """Write `<out_dir>/<digest>.so` + `.so.plan.json` and return the library path
    (`out_dir` defaults to PLAN_DIR, inside the package tree)."""
    out_dir = PLAN_DIR if out_dir is None else out_dir
    if options.get("phase") == "forward":
        document = forward_document(config, **{key: value for key, value in options.items() if key != "phase"})
    else:
        document = plan_document(config, **options)
    text = json.dumps(document, indent=1, sort_keys=True) + "\n"
    digest = hashlib.sha256(text.encode()).hexdigest()[:16]
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    library = build_library()
    target = out_dir / f"tilemega_b200_{digest}.so"
    sidecar = Path(str(target) + ".plan.json")
    # Several processes (the ranks of one job) may emit the same plan at once: every file
    # appears under its final name complete or not at all, and an identical plan is left alone.
    unique = f".{os.getpid()}.tmp"
    if not target.exists() or target.stat().st_mtime < library.stat().st_mtime:
        tmp = Path(str(target) + unique)
        shutil.copyfile(library, tmp)
        os.replace(tmp, target)
    if not sidecar.exists() or sidecar.read_text() != text:
        tmp = Path(str(sidecar) + unique)
        tmp.write_text(text)
        os.replace(tmp, sidecar)
    if document.get("phase") == "forward":
        _write_bridge(target, document, unique)
    return target


def _write_bridge(target: Path, document: dict, unique: str) -> None:
    """The export bridge the reference's forward driver reads (python/tilemega/dnn/check.py:40, 45-49), as
    `<so>.bridge.json`: the graph's user inputs and outputs with shape and dtype. No `<so>.identity.json` is written:
    that file is the reference compiler's build record (hashes of its generated source and ptxas log, checked by
    python/tilemega/build/identity.py:99-130), and the reference's PlanLibrary loads a library without one."""
    model, seq, batch = document["model"], document["seq"], document["batch_lo"]
    element = "torch.float16" if document["dtype"] == "f16" else "torch.bfloat16"
    inputs = ["input_ids", "token_type_ids"] + (["attention_mask"] if document.get("mask") else [])
    nodes = [{"name": name, "shape": [batch, seq], "dtype": "torch.int64"} for name in inputs]
    nodes += [{"name": "last_hidden_state", "shape": [batch, seq, model["hidden_size"]], "dtype": element},
              {"name": "pooler_output", "shape": [batch, model["hidden_size"]], "dtype": element}]
    bridge = {"nodes": nodes,
              "signature": {"inputs": [{"name": name, "kind": "USER_INPUT"} for name in inputs],
                            "outputs": [{"name": name, "kind": "USER_OUTPUT"} for name in ("last_hidden_state", "pooler_output")]}}
    path = Path(str(target) + ".bridge.json")
    text = json.dumps(bridge, indent=1, sort_keys=True) + "\n"
    if not path.exists() or path.read_text() != text:
        tmp = Path(str(path) + unique)
        tmp.write_text(text)
        os.replace(tmp, path)


def remove_plans(out_dir: str | Path) -> None:
    """Delete the plan libraries (and sidecars) this module wrote into `out_dir`."""
    out_dir = Path(out_dir)
    if out_dir.is_dir():
        for path in out_dir.glob("tilemega_b200_*.so*"):
            path.unlink(missing_ok=True)
        if not any(out_dir.iterdir()):
            out_dir.rmdir()


__all__ = ["emit_plan", "forward_document", "plan_document", "remove_plans", "LIBRARY", "PLAN_DIR"]
