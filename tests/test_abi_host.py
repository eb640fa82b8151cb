"""Host-side checks of the C ABI that need no GPU: the library loads, exports
every declared symbol, publishes the buffer table of its sidecar, and refuses
loudly to create a plan without a CUDA device."""
import ctypes
import json
import re
from pathlib import Path

import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan, plan_document
from tilemega_b200.serving.plan import DECODE, PlanLibrary

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    header = (ROOT / "include" / "tilemega_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(tm_\w+)\s*\(", header)))


def test_library_exports_every_declared_symbol(library):
    lib = ctypes.CDLL(str(library))
    names = declared_symbols()
    assert len(names) >= 28
    for extra in ("tm_watchdog_probe_static", "tm_ipc_alloc", "tm_ipc_free", "tm_ipc_export", "tm_ipc_open", "tm_ipc_close",
                  "tm_pack_tile_pages", "tm_plan_launch_steps_ranks"):
        assert extra in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/tilemega_b200.h but not exported"


def test_binding_table_covers_the_header():
    """Every entry point the header declares has a row in the ctypes binding, and the other way round."""
    from tilemega_b200.serving.plan import SIGNATURES
    assert sorted(SIGNATURES) == declared_symbols()


def test_query_without_sidecar_fails(library, tmp_path, monkeypatch):
    import shutil
    orphan = tmp_path / "orphan.so"
    shutil.copyfile(library, orphan)
    with pytest.raises(RuntimeError):
        PlanLibrary(orphan)


def test_buffer_table_of_tiny_plan(plan_dir):
    config = synthetic.TINY
    so = emit_plan(config, plan_dir, batch_lo=1, batch_hi=4, capacity=64)
    lib = PlanLibrary(so)
    assert lib.info.abi_version == 1 and lib.info.phase == DECODE and lib.info.seq == 1
    assert (lib.info.batch_lo, lib.info.batch_hi, lib.info.capacity) == (1, 4, 64)
    assert (lib.info.past_lo, lib.info.past_hi) == (0, 63)
    assert lib.info.modes == 3
    table = {b.name: b for b in lib.buffers}
    hidden, dim = config["hidden_size"], config["head_dim"]
    assert table["serving.tokens"].elements_per_batch == 64 and table["serving.tokens"].dtype == 2
    assert table["serving.rope_cos"].elements_constant == 64 * dim
    assert table["kv_cache.k.1"].elements_per_batch == config["num_key_value_heads"] * 64 * dim
    qkv = table["l0.qkv.weight"]
    rows = (config["num_attention_heads"] + 2 * config["num_key_value_heads"]) * dim
    assert qkv.elements_constant == rows * hidden and qkv.role == 1
    recipe = json.loads(qkv.pack_json)
    assert recipe["kind"] == "tile_pages" and (recipe["tile_n"], recipe["tile_k"]) == (8, 2048)
    assert recipe["source"]["kind"] == "qkv_group_interleave" and recipe["source"]["qperkv"] == 4
    assert recipe["source"]["sources"][1] == "model.layers.0.self_attn.k_proj.weight"
    assert json.loads(table["l1.gate_up.weight"].pack_json)["source"]["u"] == 4
    assert json.loads(table["lm_head.weight"].pack_json)["source"] == {"kind": "alias", "source": "lm_head.weight"}
    assert table["serving.logits"].role == 0 and table["serving.logits"].elements_per_batch == config["vocab_size"]
    # external pointers are mandatory and checked before anything touches a device
    with pytest.raises(KeyError):
        lib.create(1, {}, 0)
    with pytest.raises(ValueError):
        lib.create(5, {}, 0)   # outside this plan's interval [1, 4]


def test_paged_plan_lists_block_table(plan_dir):
    so = emit_plan(synthetic.TINY, plan_dir, batch_lo=2, batch_hi=2, capacity=64, kv_layout="paged", num_blocks=24)
    lib = PlanLibrary(so)
    table = {b.name: b for b in lib.buffers}
    assert table["serving.block_table"].elements_per_batch == 4 and table["serving.block_table"].dtype == 2
    assert table["serving.context_base"].elements_per_batch == 1
    assert table["kv_pool.k.0"].elements_constant == 24 * 8 * 16 * 64 and "kv_cache.k.0" not in table


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_create_without_a_gpu_fails_loudly(plan_dir):
    so = emit_plan(synthetic.TINY, plan_dir, batch_lo=1, batch_hi=1, capacity=32)
    lib = PlanLibrary(so)
    pointers = {b.name: 4096 for b in lib.buffers if b.role == 1}
    with pytest.raises(RuntimeError, match="no such CUDA device|rejected"):
        lib.create(1, pointers, 0)


def test_unsupported_shapes_are_rejected(plan_dir):
    bad = dict(synthetic.TINY, hidden_size=1028)   # neither rows nor reductions in whole 16-byte chunks
    so = emit_plan(bad, plan_dir, batch_lo=1, batch_hi=1, capacity=32)
    with pytest.raises(RuntimeError, match="must be a multiple"):
        PlanLibrary(so)
    # a reduction that is not a whole number of pages is padded, not rejected
    padded = PlanLibrary(emit_plan(dict(synthetic.TINY, intermediate_size=1536), plan_dir, batch_lo=1, batch_hi=1,
                                   capacity=32))
    table = {buffer.name: buffer for buffer in padded.buffers}
    assert table["l0.down.weight"].elements_constant == synthetic.TINY["hidden_size"] * 2048
    assert table["serving.mlp"].elements_per_batch == 1536
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY, batch_lo=1, batch_hi=9, capacity=32)
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY, batch_lo=1, capacity=40)
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY, batch_lo=2, capacity=64, kv_layout="paged", num_blocks=1)


def test_prefill_plan_tables(plan_dir):
    """A prefill plan (phase 0) as the reference's driver sees it: seq = the prompt length, one step, the
    sequences' state buffers shared with the decode plan by name, GEMM weights under names of their own."""
    config = synthetic.TINY_D128
    so = emit_plan(config, plan_dir, batch_lo=1, batch_hi=4, capacity=64, phase="prefill", seq=21)
    lib = PlanLibrary(so)
    assert (lib.info.phase, lib.info.seq, lib.info.batch_lo, lib.info.batch_hi, lib.info.capacity) == (0, 21, 1, 4, 64)
    assert (lib.info.past_lo, lib.info.past_hi) == (0, 0)
    table = {buffer.name: buffer for buffer in lib.buffers}
    decode = {buffer.name: buffer for buffer in PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=4, capacity=64)).buffers}
    for name in ("serving.tokens", "serving.rope_cos", "kv_cache.k.0", "kv_cache.v.1", "model.embed_tokens.weight", "l0.norm1.weight"):
        assert (table[name].elements_constant, table[name].elements_per_batch, table[name].pack_json) == \
               (decode[name].elements_constant, decode[name].elements_per_batch, decode[name].pack_json), name
    hidden = config["hidden_size"]
    assert (table["serving.hidden"].elements_constant, table["serving.hidden"].elements_per_batch) == (64 * hidden, 0)
    assert "prefill.l0.qkv.weight" in table and "l0.qkv.weight" not in table and "prefill.lm_head.weight" in table
    assert '"tile_n":128' in table["prefill.l1.down.weight"].pack_json.replace(" ", "")
    with pytest.raises(ValueError):
        emit_plan(config, plan_dir, batch_lo=1, batch_hi=2, capacity=64, phase="prefill", seq=64)
