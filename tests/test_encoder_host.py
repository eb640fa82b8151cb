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


def test_forward_plan_rejects_shapes_it_does_not_cover():
    with pytest.raises(ValueError):
        forward_document(synthetic.BERT_BASE, seq=64)
    with pytest.raises(ValueError):
        forward_document(dict(synthetic.BERT_BASE, num_attention_heads=8))
    with pytest.raises(ValueError):
        forward_document(synthetic.BERT_BASE, dtype="f32")
    with pytest.raises(ValueError):
        forward_document(synthetic.BERT_BASE, batch_lo=0)
