"""Host side of the mixture-of-experts plan, on CPU: tables, the expert_stack recipe, limits."""
import json

import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.plan import PlanLibrary
from tilemega_b200.serving.weights import pack, tile_pages


def test_moe_plan_tables(plan_dir):
    config = synthetic.TINY_MOE
    lib = PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=1, capacity=64))
    table = {buffer.name: buffer for buffer in lib.buffers}
    hidden, experts, inter, topk = config["hidden_size"], config["num_experts"], config["moe_intermediate_size"], 4
    assert table["serving.router_logits"].elements_per_batch == experts
    assert table["serving.mlp"].elements_per_batch == topk * inter            # one row per chosen expert
    assert table["serving.route_index"].elements_per_batch == config["num_hidden_layers"] * topk   # [layers][batch][topk]
    assert table["l0.router.weight"].elements_constant == experts * hidden
    assert table["l0.gate_up.weight"].elements_constant == experts * 2 * inter * hidden
    assert table["l0.down.weight"].elements_constant == experts * hidden * 2048   # 768 columns padded to one page
    assert table["l0.q_norm.weight"].elements_constant == 128
    recipe = json.loads(table["l1.down.weight"].pack_json)
    assert recipe["kind"] == "tile_pages" and recipe["source"] == {
        "kind": "expert_stack", "prefix": "model.layers.1.mlp.experts.", "part": "down", "experts": experts,
        "hidden": hidden, "intermediate": inter, "u": 4}


def test_expert_stack_recipe_packs_every_expert_by_itself():
    experts, hidden, inter = 3, 128, 16
    generator = torch.Generator().manual_seed(0)
    tensors = {}
    for e in range(experts):
        for kind, shape in (("gate", (inter, hidden)), ("up", (inter, hidden)), ("down", (hidden, inter))):
            tensors[f"m.experts.{e}.{kind}_proj.weight"] = torch.randn(shape, generator=generator)
    leaf = {"kind": "expert_stack", "prefix": "m.experts.", "experts": experts, "hidden": hidden, "intermediate": inter, "u": 4}
    packed = pack({"kind": "tile_pages", "tile_n": 8, "tile_k": 128, "source": dict(leaf, part="gate_up")},
                  tensors.__getitem__)
    per_expert = 2 * inter * hidden
    for e in range(experts):
        gate, up = tensors[f"m.experts.{e}.gate_proj.weight"], tensors[f"m.experts.{e}.up_proj.weight"]
        rows = torch.stack((gate.reshape(-1, 4, hidden), up.reshape(-1, 4, hidden)), dim=1).reshape(-1, hidden)
        assert torch.equal(packed[e * per_expert:(e + 1) * per_expert], tile_pages(rows, 8, 128))
    down = pack({"kind": "tile_pages", "tile_n": 8, "tile_k": 64, "source": dict(leaf, part="down")}, tensors.__getitem__)
    padded = torch.zeros(hidden, 64)
    padded[:, :inter] = tensors["m.experts.2.down_proj.weight"]
    assert torch.equal(down[2 * hidden * 64:], tile_pages(padded, 8, 64))


def test_moe_limits(plan_dir):
    assert PlanLibrary(emit_plan(synthetic.TINY_MOE, plan_dir, batch_lo=1, batch_hi=8, capacity=64)).info.batch_hi == 8
    with pytest.raises((RuntimeError, ValueError)):      # 16 and more rows would need the experts on the dense-batch tiles
        PlanLibrary(emit_plan(synthetic.TINY_MOE, plan_dir, batch_lo=16, batch_hi=16, capacity=64))
    with pytest.raises(RuntimeError, match="norm_topk_prob"):
        PlanLibrary(emit_plan(dict(synthetic.TINY_MOE, norm_topk_prob=False), plan_dir, batch_lo=1, batch_hi=1, capacity=64))
