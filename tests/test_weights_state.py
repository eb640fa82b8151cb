"""Packing recipes and request state on the CPU."""
import json

import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.serving.state import rotary_tables, shuffled_block_table
from tilemega_b200.serving.weights import TensorCheckpoint, pack, tile_pages

GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"


def closed_form_offset(row, col, tn):
    # the layout contract of the reference's tile_pages recipe
    # (python/tilemega/serving/weights.py:239-240), written out per element
    return 512 * (row // 8 + (tn // 8) * (col // 64)) + 64 * (row % 8) + 8 * ((col % 64 // 8) ^ (row % 8)) + col % 8


@pytest.mark.parametrize("tn,tk,n,k", [(8, 2048, 24, 4096), (8, 64, 8, 128), (16, 128, 32, 256), (8, 2048, 20, 3000)])
def test_tile_pages_matches_closed_form(tn, tk, n, k):
    weight = torch.arange(n * k, dtype=torch.float32).reshape(n, k)
    packed = tile_pages(weight, tn, tk)
    nt, kt = -(-n // tn), -(-k // tk)
    assert packed.numel() == nt * tn * kt * tk
    pages = packed.reshape(nt, kt, tn * tk)
    generator = torch.Generator().manual_seed(3)
    for _ in range(400):
        row = int(torch.randint(0, nt * tn, (1,), generator=generator))
        col = int(torch.randint(0, kt * tk, (1,), generator=generator))
        expect = weight[row, col].item() if row < n and col < k else 0.0
        got = pages[row // tn, col // tk, closed_form_offset(row % tn, col % tk, tn)].item()
        assert got == expect


def test_qkv_and_gate_up_interleave():
    config = dict(synthetic.TINY, num_hidden_layers=1)
    hkv, dim, hidden = config["num_key_value_heads"], config["head_dim"], 16
    q = torch.arange(hkv * 4 * dim * hidden, dtype=torch.float32).reshape(hkv * 4 * dim, hidden)
    k = -torch.arange(hkv * dim * hidden, dtype=torch.float32).reshape(hkv * dim, hidden) - 1
    v = torch.full((hkv * dim, hidden), 0.5)
    source = TensorCheckpoint({"q": q, "k": k, "v": v}).tensor
    out = pack(dict(kind="qkv_group_interleave", sources=["q", "k", "v"], hkv=hkv, qperkv=4, head_dim=dim), source)
    group = 6 * dim
    for g in (0, 3, hkv - 1):
        assert torch.equal(out[g * group:g * group + 4 * dim], q[g * 4 * dim:(g + 1) * 4 * dim])
        assert torch.equal(out[g * group + 4 * dim:g * group + 5 * dim], k[g * dim:(g + 1) * dim])
        assert torch.equal(out[g * group + 5 * dim:(g + 1) * group], v[g * dim:(g + 1) * dim])
    gate = torch.arange(32 * 4, dtype=torch.float32).reshape(32, 4)
    up = gate + 1000
    both = pack(dict(kind="gate_up_interleave", sources=["g", "u"], u=4), TensorCheckpoint({"g": gate, "u": up}).tensor)
    assert torch.equal(both[0:4], gate[0:4]) and torch.equal(both[4:8], up[0:4]) and torch.equal(both[8:12], gate[4:8])
    with pytest.raises(ValueError):
        pack(dict(kind="unknown"), source)
    with pytest.raises(KeyError):
        TensorCheckpoint({}, True).tensor("lm_head.weight")


def test_tied_head_aliases_the_embedding():
    table = torch.randn(8, 4)
    assert TensorCheckpoint({"model.embed_tokens.weight": table}, True).tensor("lm_head.weight") is table


def test_rotary_tables_and_block_tables():
    config = synthetic.LLAMA_3_2_1B
    cos, sin = rotary_tables(config, 32, "cpu")
    assert cos.shape == (32, 64) and cos.dtype == torch.bfloat16
    assert torch.equal(cos[:, :32], cos[:, 32:]) and float(cos[0, 0]) == 1.0 and float(sin[0, 5]) == 0.0
    reference = torch.tensor(1.0 / 500000.0 ** (2 * 3 / 64)) * 7
    assert abs(float(sin[7, 3]) - float(torch.sin(reference))) < 4e-3
    table = shuffled_block_table(3, 8, 40, seed=5)
    assert table.shape == (3, 8) and table.unique().numel() == 24 and int(table.max()) < 40
    assert torch.equal(table, shuffled_block_table(3, 8, 40, seed=5))
    with pytest.raises(ValueError):
        shuffled_block_table(3, 8, 10)
    with pytest.raises(ValueError):
        rotary_tables(dict(config, rope_scaling={"rope_type": "yarn", "factor": 4.0}), 8, "cpu")


def test_seeded_weights_are_reproducible_and_ordered():
    config = synthetic.TINY
    names = [name for name, _ in synthetic.parameter_shapes(config)]
    assert names[0] == "model.embed_tokens.weight" and names[-1] == "model.norm.weight"
    assert "lm_head.weight" not in names and "lm_head.weight" in dict(synthetic.parameter_shapes(synthetic.TINY_D128))
    small = dict(config, vocab_size=64, num_hidden_layers=1)
    a, b = synthetic.seeded_weights(small, 0), synthetic.seeded_weights(small, 0)
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert torch.equal(a["model.norm.weight"], torch.ones(2048))
    assert 0.019 < float(a["model.layers.0.mlp.up_proj.weight"].std()) < 0.021
    assert not torch.equal(a["model.embed_tokens.weight"], synthetic.seeded_weights(small, 1)["model.embed_tokens.weight"])


def test_kv_row_swizzle_is_an_involution_with_the_kernel_mapping():
    from tilemega_b200.serving.state import kv_row_swizzle
    rows = torch.arange(2 * 32 * 64, dtype=torch.int32).reshape(2, 32, 64)
    stored = kv_row_swizzle(rows)
    assert torch.equal(kv_row_swizzle(stored), rows)
    for t, d in ((0, 5), (13, 42), (31, 63), (8, 17)):
        assert stored[1, t, (((d >> 3) ^ (t & 7)) << 3) | (d & 7)] == rows[1, t, d]


@pytest.mark.parametrize("case", ["llama31_8b", "llama32_1b", "linear4"])
def test_scaled_rope_tables_match_the_hf_rotary_module(case):
    """rope_scaling of the real Llama-3.1/3.2 checkpoints ("llama3") and "linear": inv_freq and
    the bf16 cos/sin rows against the fixture written from the HF rotary module the reference
    calls (tests/golden/make_golden_rope.py)."""
    from tilemega_b200.serving.state import inverse_frequencies, rotary_tables
    record = torch.load(GOLDEN / "rope_llama3.pt")[case]
    config = dict(record["config"], hidden_size=record["config"]["head_dim"] * 4, num_attention_heads=4)
    assert torch.allclose(inverse_frequencies(config), record["inv_freq"], rtol=1e-6, atol=0)
    capacity = max(record["positions"]) + 1
    cos, sin = rotary_tables(config, capacity, "cpu")
    rows = torch.tensor(record["positions"])
    # angles of ~1e5 rad in fp32 carry ~1e-2 rad of rounding, so two correct evaluations may
    # round a few table entries to neighbouring bf16 values; almost all must be identical
    for ours, theirs in ((cos[rows], record["cos"]), (sin[rows], record["sin"])):
        assert (ours.float() - theirs.float()).abs().max().item() <= 2 ** -7
        assert (ours == theirs).float().mean().item() >= 0.98
    with pytest.raises(ValueError):
        rotary_tables(dict(config, rope_scaling={"rope_type": "yarn", "factor": 2.0}), 16, "cpu")


def test_safetensors_directory_loads_like_an_in_memory_checkpoint(tmp_path, plan_dir):
    """A model directory of sharded *.safetensors files (the reference's input, python/tilemega/serving/
    weights.py:17-49): tensors are read one at a time as the recipes ask for them, tied embeddings resolve
    through config.json, and the packed buffers are those of the same tensors held in memory."""
    import json
    from safetensors.torch import save_file
    from tilemega_b200 import synthetic
    from tilemega_b200.planbuild import emit_plan
    from tilemega_b200.serving.plan import PlanLibrary
    from tilemega_b200.serving.weights import Checkpoint, TensorCheckpoint, load_weights
    config = dict(synthetic.TINY, num_hidden_layers=1, tie_word_embeddings=True)
    tensors = {name: tensor.to(torch.bfloat16).contiguous() for name, tensor in synthetic.seeded_weights(config, 0).items()}
    tensors.pop("lm_head.weight", None)                       # tied: the head is the embedding table
    names = sorted(tensors)
    save_file({name: tensors[name] for name in names[::2]}, tmp_path / "model-00001-of-00002.safetensors")
    save_file({name: tensors[name] for name in names[1::2]}, tmp_path / "model-00002-of-00002.safetensors")
    (tmp_path / "config.json").write_text(json.dumps(config))
    lib = PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=1, capacity=32))
    from_files = load_weights(tmp_path, lib, device="cpu")
    in_memory = load_weights(TensorCheckpoint(tensors, True), lib, device="cpu")
    assert set(from_files) == set(in_memory) and "lm_head.weight" in from_files
    for name in in_memory:
        assert torch.equal(from_files[name], in_memory[name]), name
    assert Checkpoint(tmp_path).tie_word_embeddings
    with pytest.raises(KeyError):
        Checkpoint(tmp_path).tensor("model.layers.7.mlp.up_proj.weight")
