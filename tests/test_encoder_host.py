"""Host-side checks of the encoder forward path that need no GPU: the oracle against the golden fixture made
by the third-party module the reference exports (and against that module itself when it is importable), and the
forward plan's tables as the reference's driver reads them."""
import pytest
import torch

from oracle.encoder_oracle import encoder_forward, token_cosine
from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan, forward_document
from tilemega_b200.serving.plan import FORWARD, PlanLibrary

from pathlib import Path

GOLDEN = Path(__file__).parent / "golden" / "tiny_bert.pt"


def test_oracle_matches_the_module_fixture():
    golden = torch.load(GOLDEN)
    weights = synthetic.encoder_weights(golden["config"], seed=0)
    hidden, pooled = encoder_forward(weights, golden["config"], golden["input_ids"], golden["token_type_ids"])
    # fp32 against fp32: only the order of summation differs
    assert (hidden - golden["last_hidden_state"]).abs().max() < 2e-5
    assert (pooled - golden["pooler_output"]).abs().max() < 2e-5
    # padded tails: every position of the module's output, the padded ones included
    hidden, pooled = encoder_forward(weights, golden["config"], golden["input_ids"], golden["token_type_ids"],
                                     attention_mask=golden["attention_mask"])
    assert (hidden - golden["masked_last_hidden_state"]).abs().max() < 2e-5
    assert (pooled - golden["masked_pooler_output"]).abs().max() < 2e-5
    assert (golden["masked_last_hidden_state"] - golden["last_hidden_state"]).abs().max() > 1e-2   # the mask matters


def test_oracle_matches_the_module_run_here():
    pytest.importorskip("transformers")
    import sys
    sys.path.insert(0, str(GOLDEN.parent))
    from make_golden_bert import module_outputs
    config = dict(synthetic.TINY_BERT, num_hidden_layers=3, intermediate_size=384)
    weights = synthetic.encoder_weights(config, seed=5)
    ids, types = synthetic.encoder_inputs(config, batch=1, seed=6)
    hidden, pooled = module_outputs(config, weights, ids, types)
    mine, mine_pooled = encoder_forward(weights, config, ids, types)
    assert (mine - hidden).abs().max() < 2e-5 and (mine_pooled - pooled).abs().max() < 2e-5
    # the 16-bit yardstick the GPU tests use: the same forward with every module output rounded to fp16
    half, _ = encoder_forward(weights, config, ids, types, torch.float16)
    assert token_cosine(half, hidden).min() > 0.9999


def test_forward_plan_tables(plan_dir):
    """A forward plan (phase 2) as the reference's driver sees it (python/tilemega/dnn/check.py:33-66): stateless,
    the module's parameters under their names, int64 inputs, outputs per batch."""
    config = synthetic.BERT_BASE
    lib = PlanLibrary(emit_plan(config, plan_dir, phase="forward", batch_lo=1, batch_hi=32, dtype="f16"))
    info = lib.info
    assert (info.phase, info.seq, info.batch_lo, info.batch_hi, info.capacity, info.past_lo, info.past_hi) == (FORWARD, 128, 1, 32, 0, 0, 0)
    table = {buffer.name: buffer for buffer in lib.buffers}
    shapes = dict(synthetic.encoder_parameter_shapes(config))
    for name, shape in shapes.items():
        count = 1
        for extent in shape:
            count *= extent
        assert (table[name].role, table[name].dtype, table[name].elements_constant, table[name].elements_per_batch) == (1, 5, count, 0), name
        assert '"alias"' in table[name].pack_json
    assert (table["input_ids"].role, table["input_ids"].dtype, table["input_ids"].elements_per_batch) == (1, 3, 128)
    assert (table["token_type_ids"].dtype, table["token_type_ids"].elements_per_batch) == (3, 128)
    assert (table["last_hidden_state"].role, table["last_hidden_state"].elements_per_batch) == (1, 128 * 768)
    assert (table["pooler_output"].role, table["pooler_output"].elements_per_batch) == (1, 768)
    assert {name for name, buffer in table.items() if buffer.role == 0} == {"forward.hidden", "forward.qkv", "forward.context", "forward.ffn"}
    bf16 = PlanLibrary(emit_plan(config, plan_dir, phase="forward", batch_lo=8, dtype="bf16"))
    assert {buffer.dtype for buffer in bf16.buffers} == {0, 3}
    assert "attention_mask" not in table
    masked = {buffer.name: buffer for buffer in PlanLibrary(emit_plan(config, plan_dir, phase="forward", batch_lo=8, mask=True)).buffers}
    assert (masked["attention_mask"].role, masked["attention_mask"].dtype, masked["attention_mask"].elements_per_batch) == (1, 3, 128)
    # without a CUDA device the plan refuses loudly
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            lib.create(1, {name: 16 for name, buffer in table.items() if buffer.role == 1}, 0)


def test_forward_plan_bridge_file(plan_dir):
    """The export bridge the reference's forward driver reads (python/tilemega/dnn/check.py:40, 45-59): its user
    inputs and outputs are exactly the external buffers that carry no packing recipe, and its dtypes are the ones
    that driver maps (a bf16 plan). No identity file is written (it is the reference compiler's build record, and the
    reference's PlanLibrary verifies one when it finds one)."""
    import json
    so = emit_plan(synthetic.TINY_BERT, plan_dir, phase="forward", batch_lo=2, dtype="bf16", mask=True)
    assert not Path(str(so) + ".identity.json").exists()
    bridge = json.loads(Path(str(so) + ".bridge.json").read_text())
    nodes = {node["name"]: node for node in bridge["nodes"]}
    inputs = [item["name"] for item in bridge["signature"]["inputs"] if item["kind"] == "USER_INPUT"]
    outputs = [item["name"] for item in bridge["signature"]["outputs"] if item["kind"] == "USER_OUTPUT"]
    lib = PlanLibrary(so)
    unpacked = {buffer.name for buffer in lib.buffers if buffer.role == 1 and not buffer.pack_json}
    assert set(inputs) | set(outputs) == unpacked and inputs == ["input_ids", "token_type_ids", "attention_mask"]
    assert all(nodes[name]["dtype"] == "torch.int64" and nodes[name]["shape"] == [2, 128] for name in inputs)
    assert {nodes[name]["dtype"] for name in outputs} == {"torch.bfloat16"}
    assert nodes["last_hidden_state"]["shape"] == [2, 128, 256] and nodes["pooler_output"]["shape"] == [2, 256]


def test_reference_driver_classes_accept_a_forward_plan(plan_dir):
    """Where the reference tree is at hand: its own PlanLibrary loads a forward plan emitted here and sees a stateless
    forward library, and its recipe table lists exactly the module's parameters."""
    import sys
    sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "oracle"))
    from build_ref import reference_tree
    tree = reference_tree()
    if tree is None or not (tree / "python" / "tilemega" / "serving" / "plan.py").is_file():
        pytest.skip("no reference tree on this machine")
    reference = tree / "python"
    sys.path.insert(0, str(reference))
    try:
        from tilemega.serving.plan import FORWARD as THEIR_FORWARD, PlanLibrary as TheirLibrary
        from tilemega.serving.weights import weight_recipes
    except Exception as error:   # a dependency of the reference's package that is not installed here
        pytest.skip(f"the reference's driver does not import here: {error}")
    finally:
        sys.path.remove(str(reference))
    so = emit_plan(synthetic.TINY_BERT, plan_dir, phase="forward", batch_lo=2, dtype="bf16")
    theirs = TheirLibrary(so)
    assert theirs.info.phase == THEIR_FORWARD and not theirs.info.capacity and theirs.info.batch_lo <= 2 <= theirs.info.batch_hi
    assert set(weight_recipes(theirs)) == {name for name, _ in synthetic.encoder_parameter_shapes(synthetic.TINY_BERT)}


def test_forward_plan_rejects_shapes_it_does_not_cover():
    with pytest.raises(ValueError):
        forward_document(synthetic.BERT_BASE, seq=64)
    with pytest.raises(ValueError):
        forward_document(dict(synthetic.BERT_BASE, num_attention_heads=8))
    with pytest.raises(ValueError):
        forward_document(synthetic.BERT_BASE, dtype="f32")
    with pytest.raises(ValueError):
        forward_document(synthetic.BERT_BASE, batch_lo=0)
