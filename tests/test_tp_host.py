"""Host side of tensor parallelism, on CPU: the rank plan's tables, the sharded packing
recipes, the region sizes, and (world_size 2, gloo) that two ranks packing their slices
cover the checkpoint exactly."""
import json
import os
import socket
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan, plan_document
from tilemega_b200.serving.plan import PlanLibrary
from tilemega_b200.serving.weights import TensorCheckpoint, load_weights, pack, tile_pages


def test_rank_plan_tables(plan_dir):
    config = synthetic.TINY_D128
    lib = PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=2, capacity=64, tp=2))
    assert lib.tp_world == 2
    table = {buffer.name: buffer for buffer in lib.buffers}
    hidden, dim = config["hidden_size"], 128
    heads, hkv, inter, vocab = 16 // 2, 4 // 2, config["intermediate_size"] // 2, config["vocab_size"] // 2
    # one rank's shares; the o reduction of 1024 columns is padded to one 2048-column page
    assert table["serving.qkv"].elements_per_batch == (heads + 2 * hkv) * dim
    assert table["serving.attention"].elements_per_batch == heads * dim
    assert table["serving.mlp"].elements_per_batch == inter
    assert table["serving.logits"].elements_per_batch == vocab
    assert table["kv_cache.k.0"].elements_per_batch == hkv * 64 * dim
    assert table["l0.o.weight"].elements_constant == hidden * 2048
    assert table["l0.down.weight"].elements_constant == hidden * 2048
    assert table["lm_head.weight"].elements_constant == vocab * hidden
    assert table["model.embed_tokens.weight"].elements_constant == config["vocab_size"] * hidden   # whole on every rank
    recipe = json.loads(table["l0.o.weight"].pack_json)
    assert recipe["source"]["shard"] == {"axis": 1, "parts": 2}
    assert json.loads(table["l0.qkv.weight"].pack_json)["source"]["shard"] == {"axis": 0, "parts": 2}
    assert json.loads(table["l0.gate_up.weight"].pack_json)["source"]["shard"] == {"axis": 0, "parts": 2}
    assert json.loads(table["lm_head.weight"].pack_json)["source"]["shard"] == {"axis": 0, "parts": 2}
    # two regions of [ranks][batch_hi][hidden/2] 8-byte packets; [ranks][8] exchange packets
    assert lib.tp_bytes(0) == 2 * 2 * 2 * (hidden // 2) * 8
    assert lib.tp_bytes(1) == 2 * 8 * 8


def test_tensor_parallel_needs_head_dim_128(plan_dir):
    so = emit_plan(synthetic.TINY, plan_dir, batch_lo=1, batch_hi=1, capacity=64, tp=2)
    with pytest.raises(RuntimeError, match="head_dim 128"):
        PlanLibrary(so)


def test_unsharded_plan_reports_world_one(plan_dir):
    lib = PlanLibrary(emit_plan(synthetic.TINY, plan_dir, batch_lo=1, batch_hi=1, capacity=64))
    assert lib.tp_world == 1
    with pytest.raises(ValueError):
        lib.tp_bytes(0)


def test_tp_degree_must_divide():
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY, capacity=64, tp=3)
    with pytest.raises(ValueError):
        plan_document(dict(synthetic.TINY, num_key_value_heads=4, num_attention_heads=16), capacity=64, tp=8)


def test_sharded_recipe_takes_the_rank_slice():
    weight = torch.arange(16 * 128, dtype=torch.float32).reshape(16, 128)
    source = {"w": weight}.__getitem__
    by_rows = {"kind": "alias", "source": "w", "shard": {"axis": 0, "parts": 2}}
    by_cols = {"kind": "alias", "source": "w", "shard": {"axis": 1, "parts": 2}}
    assert torch.equal(pack(by_rows, source, 1), weight[8:])
    assert torch.equal(pack(by_cols, source, 1), weight[:, 64:])
    paged = {"kind": "tile_pages", "tile_n": 8, "tile_k": 128, "source": by_cols}
    # the 64 columns of the slice are zero-padded to the 128-column page
    padded = torch.zeros(16, 128)
    padded[:, :64] = weight[:, :64]
    assert torch.equal(pack(paged, source, 0), tile_pages(padded, 8, 128))
    with pytest.raises(ValueError):
        pack(by_rows, source, 2)


def _rank_main(rank: int, world: int, port: int, plan_path: str, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    config = dict(synthetic.TINY_D128, num_hidden_layers=1)
    lib = PlanLibrary(plan_path)
    weights = synthetic.seeded_weights(config, seed=0, dtype=torch.bfloat16)
    packed = load_weights(TensorCheckpoint(weights, False), lib, device="cpu", tp=(rank, world))
    # element sums are layout-independent: the two ranks' slices must add up to the whole tensor
    mine = torch.tensor([packed[name].double().sum().item() for name in ("l0.qkv.weight", "l0.o.weight",
                                                                            "l0.gate_up.weight", "l0.down.weight",
                                                                            "lm_head.weight")], dtype=torch.float64)
    dist.all_reduce(mine)
    p = "model.layers.0."
    whole = torch.tensor([
        sum(weights[p + f"self_attn.{k}_proj.weight"].double().sum().item() for k in "qkv"),
        weights[p + "self_attn.o_proj.weight"].double().sum().item(),
        weights[p + "mlp.gate_proj.weight"].double().sum().item() + weights[p + "mlp.up_proj.weight"].double().sum().item(),
        weights[p + "mlp.down_proj.weight"].double().sum().item(),
        weights["lm_head.weight"].double().sum().item()], dtype=torch.float64)
    ok = bool(torch.allclose(mine, whole, rtol=0, atol=1e-6))
    Path(out_dir, f"rank{rank}.txt").write_text("ok" if ok else f"mismatch {mine.tolist()} {whole.tolist()}")
    dist.destroy_process_group()


def test_two_ranks_pack_disjoint_slices_that_cover_the_checkpoint(plan_dir, tmp_path):
    config = dict(synthetic.TINY_D128, num_hidden_layers=1)
    so = emit_plan(config, plan_dir, batch_lo=1, batch_hi=1, capacity=32, tp=2)
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, str(so), str(tmp_path)), nprocs=2, join=True)
    assert [Path(tmp_path, f"rank{r}.txt").read_text() for r in range(2)] == ["ok", "ok"]
