"""Dense-batch plans (batch 16..64): the GEMM stages run on tcgen05 tiles (weights as the
128-row A operand, the batch rows as the N side, fp32 accumulators in tensor memory, split
reductions summed by the last arriver in ascending order), RMSNorm is a stage of its own and
attention is the small-batch kernel's code. Checked the same two ways as the small-batch path:
every stage recomputed on the CPU from the buffers the GPU had (tests/test_gpu_stages.py has
the method and the bounds), and the whole forward against the CPU oracle with the reference's
own bf16-against-fp32 distance as the yardstick (tests/test_gpu_decode.py)."""
import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.serving.state import shuffled_block_table

from harness import GpuRun, bf16_weights
from test_gpu_decode import assert_as_accurate_as_reference_bf16
from test_gpu_stages import check_every_stage

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("base,batch,history", [
    ("TINY_D128", 16, 40), ("TINY_GQ8", 32, 21), ("TINY_D128", 64, 33), ("TINY_D128", 48, 300),
    ("TINY_D128", 64, 420),    # 1792 attention slots on 148 CTAs: equal ranges of 13 slots across units of 7
    # the Llama-3.1-8B shape's own widths, one layer: hidden 4096, FFN 14336 (112 chunks in 14 parts),
    # vocabulary 128256 (1002 row tiles)
    ("LLAMA_3_1_8B", 16, 37), ("LLAMA_3_1_8B", 64, 70)])
def test_every_stage_of_one_layer_at_dense_batch(base, batch, history, plan_dir):
    check_every_stage(dict(getattr(synthetic, base), num_hidden_layers=1), batch, history, plan_dir)


@pytest.mark.parametrize("base,batch", [("TINY_D128", 16), ("TINY_GQ8", 32)])
def test_dense_batch_decode_matches_oracle(base, batch, plan_dir):
    config = getattr(synthetic, base)
    prompt_len, new_tokens, capacity = 9, 5, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, f"{base} batch {batch}")
    # one persistent launch per phase gives the tokens of one launch per step, and a rerun is bit-identical
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    again, logits_again = run.greedy(prompt, new_tokens)
    assert torch.equal(again, tokens) and torch.equal(logits_again, logits)
    run.close()
    # a shuffled block table changes nothing, bit for bit
    table = shuffled_block_table(batch, capacity // 16, batch * (capacity // 16) + 5, seed=3)
    paged = GpuRun(config, weights, batch, capacity, plan_dir, kv_layout="paged", block_table=table,
                   num_blocks=batch * (capacity // 16) + 5)
    paged_tokens, paged_logits = paged.greedy(prompt, new_tokens)
    assert torch.equal(paged_tokens, tokens) and torch.equal(paged_logits, logits)
    paged.close()


def test_dense_batch_plan_limits(plan_dir):
    from tilemega_b200.planbuild import emit_plan, plan_document
    from tilemega_b200.serving.plan import PlanLibrary
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY_D128, batch_lo=24, batch_hi=24, capacity=32)
    with pytest.raises(ValueError):
        plan_document(synthetic.TINY_D128, batch_lo=4, batch_hi=16, capacity=32)
    with pytest.raises(RuntimeError, match="head_dim 128"):
        PlanLibrary(emit_plan(synthetic.TINY, plan_dir, batch_lo=16, batch_hi=16, capacity=32))
