"""e4m3 weight plans on the CPU: the row-wise quantisation, the two recipes that carry codes and
scales, and the plan's buffer table."""
import json

import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan, plan_document
from tilemega_b200.serving.plan import PlanLibrary
from tilemega_b200.serving.weights import (TensorCheckpoint, dequantize_e4m3, load_weights, pack, quantize_e4m3,
                                           tile_pages_by_indexing)


def test_row_wise_e4m3_quantisation():
    generator = torch.Generator().manual_seed(3)
    weight = (torch.randn(24, 512, generator=generator) * 0.02).to(torch.bfloat16)
    weight[5] = 0
    codes, scale = quantize_e4m3(weight)
    assert codes.dtype == torch.uint8 and codes.shape == weight.shape and scale.dtype == torch.float32
    assert scale[5].item() == 1.0 and codes[5].abs().max().item() == 0
    # every row uses the format's full range: its largest magnitude maps to the top code, 448
    decoded = codes.view(torch.float8_e4m3fn).float()
    rows = [r for r in range(24) if r != 5]
    assert torch.equal(decoded[rows].abs().amax(dim=1), torch.full((23,), 448.0))
    assert not decoded.isnan().any()
    # e4m3 keeps 3 mantissa bits: relative error at most 2^-4 for normal values, and the codes are a
    # fixed point of the quantiser (quantising the decoded weights changes nothing)
    back = dequantize_e4m3(codes, scale)
    big = weight.float().abs() > scale[:, None] * 2.0 ** -6
    assert ((back - weight.float()).abs()[big] <= weight.float().abs()[big] * 2.0 ** -4).all()
    again, scale_again = quantize_e4m3(back)
    assert torch.equal(again, codes) and torch.allclose(scale_again, scale, rtol=1e-6)


def test_e4m3_recipes_pack_codes_as_two_byte_units():
    weight = (torch.randn(16, 256, generator=torch.Generator().manual_seed(4)) * 0.02).to(torch.bfloat16)
    source = {"w": weight}.__getitem__
    inner = {"kind": "alias", "source": "w"}
    codes, scale = quantize_e4m3(weight)
    assert torch.equal(pack({"kind": "e4m3_scale", "source": inner}, source), scale)
    pairs = pack({"kind": "e4m3_pairs", "source": inner}, source)
    assert pairs.dtype == torch.bfloat16 and tuple(pairs.shape) == (16, 128)
    assert torch.equal(pairs.view(torch.uint8), codes)
    # pages: the codes seen as 2-byte units go through tile_pages unchanged (zero padding = code 0 = 0.0)
    paged = pack({"kind": "tile_pages", "tile_n": 8, "tile_k": 2048, "source": {"kind": "e4m3_pairs", "source": inner}}, source)
    assert paged.numel() == 2 * 8 * 2048
    assert torch.equal(paged, tile_pages_by_indexing(codes.view(torch.bfloat16), 8, 2048))
    # a column shard is quantised by itself: its own row maxima give its scales
    sharded = {"kind": "alias", "source": "w", "shard": {"axis": 1, "parts": 2}}
    assert torch.equal(pack({"kind": "e4m3_scale", "source": sharded}, source, 1), quantize_e4m3(weight[:, 128:])[1])


def test_e4m3_plan_tables_and_loader(plan_dir):
    config = synthetic.TINY_D128
    lib = PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=2, capacity=64, weights="e4m3"))
    table = {buffer.name: buffer for buffer in lib.buffers}
    hidden, inter = config["hidden_size"], config["intermediate_size"]
    rows = (16 + 2 * 4) * 128
    # one byte per element, reductions padded to whole pages of 4096 columns; one fp32 scale per row
    assert table["l0.qkv.weight"].dtype == 4 and table["l0.qkv.weight"].elements_constant == rows * 4096
    assert table["l0.qkv.scale"].dtype == 1 and table["l0.qkv.scale"].elements_constant == rows
    assert table["l1.down.weight"].elements_constant == hidden * 4096 and table["l1.down.scale"].elements_constant == hidden
    assert table["l0.gate_up.scale"].elements_constant == 2 * inter
    assert table["lm_head.weight"].dtype == 4 and table["lm_head.scale"].elements_constant == config["vocab_size"]
    assert table["model.embed_tokens.weight"].dtype == 0   # the embedding table stays bf16
    recipe = json.loads(table["l0.o.weight"].pack_json)
    assert recipe["kind"] == "tile_pages" and recipe["tile_k"] == 2048 and recipe["source"]["kind"] == "e4m3_pairs"
    assert json.loads(table["l0.o.scale"].pack_json) == {"kind": "e4m3_scale", "source": recipe["source"]["source"]}
    small = dict(config, num_hidden_layers=1, vocab_size=256)
    lib = PlanLibrary(emit_plan(small, plan_dir, batch_lo=1, batch_hi=1, capacity=32, weights="e4m3"))
    weights = synthetic.seeded_weights(small, dtype=torch.bfloat16)
    packed = load_weights(TensorCheckpoint(weights, False), lib, device="cpu")
    assert packed["l0.o.weight"].dtype == torch.uint8 and packed["l0.o.weight"].numel() == hidden * 4096
    codes, scale = quantize_e4m3(weights["model.layers.0.self_attn.o_proj.weight"])
    assert torch.equal(packed["l0.o.scale"], scale)
    assert torch.equal(packed["l0.o.weight"].view(torch.bfloat16), tile_pages_by_indexing(codes.view(torch.bfloat16), 8, 2048))


def test_e4m3_plans_refuse_what_is_not_built(plan_dir):
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY_D128, capacity=64, weights="int4")
    for config, options in ((synthetic.TINY, {}), (synthetic.TINY_MOE, {}), (synthetic.TINY_D128, {"batch_lo": 16, "batch_hi": 16})):
        with pytest.raises(RuntimeError):
            PlanLibrary(emit_plan(config, plan_dir, capacity=64, weights="e4m3", **{"batch_lo": 1, "batch_hi": 1, **options}))
