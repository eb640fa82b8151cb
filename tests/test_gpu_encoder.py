"""The encoder forward on the GPU, through the plan ABI, against the CPU oracle (the restated BertModel forward
that tests/golden/tiny_bert.pt pins to the third-party module).

Tolerances, floating point. The reference gates a native forward on cosine >= 0.999 per token against the fp32
module (python/tilemega/dnn/check.py:312, python/tilemega/dnn/gates.py:19) and reads the module's own 16-bit run as
the yardstick (check.py:259-268). Here: cosine >= 0.9999 per token and pooled row, and the largest absolute
deviation from the fp32 oracle at most 1.5 times that of the oracle run in the plan's 16-bit type (+ 1e-3)."""
from pathlib import Path

import pytest
import torch

from oracle.encoder_oracle import encoder_forward, token_cosine
from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.encoder import EncoderEngine
from tilemega_b200.serving.plan import L1, L2
from tilemega_b200.serving.weights import TensorCheckpoint

pytestmark = pytest.mark.gpu
COSINE = 0.9999
NOISE_FACTOR = 1.5


def run_case(config, batch, dtype_name, plan_dir, seed):
    dtype = torch.float16 if dtype_name == "f16" else torch.bfloat16
    # the weights every arm sees are the 16-bit roundings of the seeded draws
    weights = {name: tensor.to(dtype).float() for name, tensor in synthetic.encoder_weights(config, seed=seed).items()}
    ids, types = synthetic.encoder_inputs(config, batch, seed=seed + 1)
    so = emit_plan(config, plan_dir, phase="forward", batch_lo=batch, dtype=dtype_name)
    with EncoderEngine(TensorCheckpoint(weights), so, batch) as engine:
        hidden, pooled = engine(ids.cuda(), types.cuda(), mode=L2)
        again, pooled_again = engine(ids.cuda(), types.cuda(), mode=L1)
        # both executor modes, and a repeated launch, give the same bits (check.py:96-98)
        assert torch.equal(hidden, again) and torch.equal(pooled, pooled_again)
    truth, truth_pooled = encoder_forward(weights, config, ids, types)
    yard, yard_pooled = encoder_forward(weights, config, ids, types, dtype)
    hidden, pooled = hidden.float().cpu(), pooled.float().cpu()
    assert torch.isfinite(hidden).all() and torch.isfinite(pooled).all()
    assert token_cosine(hidden, truth).min() >= COSINE
    assert token_cosine(pooled, truth_pooled).min() >= COSINE
    noise = (yard.float() - truth).abs().max().item()
    assert (hidden - truth).abs().max().item() <= NOISE_FACTOR * noise + 1e-3
    noise_pooled = (yard_pooled.float() - truth_pooled).abs().max().item()
    assert (pooled - truth_pooled).abs().max().item() <= NOISE_FACTOR * noise_pooled + 1e-3
    return hidden, pooled


@pytest.mark.parametrize("dtype_name", ["f16", "bf16"])
@pytest.mark.parametrize("batch", [1, 3])
def test_tiny_encoder_matches_the_oracle(batch, dtype_name, plan_dir):
    run_case(synthetic.TINY_BERT, batch, dtype_name, plan_dir, seed=10 + batch)


def test_tiny_encoder_matches_the_module_fixture(plan_dir):
    """The committed outputs of the third-party module itself, on its seeded inputs."""
    golden = torch.load(Path(__file__).parent / "golden" / "tiny_bert.pt")
    config = golden["config"]
    weights = synthetic.encoder_weights(config, seed=0)
    so = emit_plan(config, plan_dir, phase="forward", batch_lo=2, dtype="f16")
    with EncoderEngine(TensorCheckpoint(weights), so, 2) as engine:
        hidden, pooled = engine(golden["input_ids"].cuda(), golden["token_type_ids"].cuda())
    assert token_cosine(hidden.float().cpu(), golden["last_hidden_state"]).min() >= COSINE
    assert (hidden.float().cpu() - golden["last_hidden_state"]).abs().max() < 3e-2
    assert (pooled.float().cpu() - golden["pooler_output"]).abs().max() < 1e-2


def test_padded_sequences_match_the_oracle_and_the_module_fixture(plan_dir):
    """A plan with the attention_mask input: the module's own outputs on padded inputs (every position, the padded
    ones included), then BERT-base shapes with a different visible length per sequence, one of them a single token."""
    golden = torch.load(Path(__file__).parent / "golden" / "tiny_bert.pt")
    config = golden["config"]
    weights = synthetic.encoder_weights(config, seed=0)
    so = emit_plan(config, plan_dir, phase="forward", batch_lo=2, dtype="f16", mask=True)
    with EncoderEngine(TensorCheckpoint(weights), so, 2) as engine:
        hidden, pooled = engine(golden["input_ids"].cuda(), golden["token_type_ids"].cuda(), golden["attention_mask"].cuda())
        plain, _ = engine(golden["input_ids"].cuda(), golden["token_type_ids"].cuda())   # no mask given: all visible
    assert token_cosine(hidden.float().cpu(), golden["masked_last_hidden_state"]).min() >= COSINE
    assert (hidden.float().cpu() - golden["masked_last_hidden_state"]).abs().max() < 3e-2
    assert (pooled.float().cpu() - golden["masked_pooler_output"]).abs().max() < 1e-2
    assert (plain.float().cpu() - golden["last_hidden_state"]).abs().max() < 3e-2
    config, batch = synthetic.BERT_BASE, 4
    weights = {name: tensor.half().float() for name, tensor in synthetic.encoder_weights(config, seed=40).items()}
    ids, types = synthetic.encoder_inputs(config, batch, seed=41)
    mask = (torch.arange(128)[None, :] < torch.tensor([[128], [1], [64], [97]])).to(torch.int64)
    so = emit_plan(config, plan_dir, phase="forward", batch_lo=batch, dtype="f16", mask=True)
    with EncoderEngine(TensorCheckpoint(weights), so, batch) as engine:
        hidden, pooled = engine(ids.cuda(), types.cuda(), mask.cuda())
    truth, truth_pooled = encoder_forward(weights, config, ids, types, attention_mask=mask)
    yard, _ = encoder_forward(weights, config, ids, types, torch.float16, attention_mask=mask)
    hidden, pooled = hidden.float().cpu(), pooled.float().cpu()
    assert token_cosine(hidden, truth).min() >= COSINE and token_cosine(pooled, truth_pooled).min() >= COSINE
    assert (hidden - truth).abs().max().item() <= NOISE_FACTOR * (yard.float() - truth).abs().max().item() + 1e-3


@pytest.mark.parametrize("batch,dtype_name", [(1, "f16"), (8, "f16"), (8, "bf16")])
def test_bert_base_shape_matches_the_oracle(batch, dtype_name, plan_dir):
    """The benchmark's shapes: 12 layers, hidden 768, 12 heads, FFN 3072, vocabulary 30522, batch x 128 tokens
    (batch 1: 32-row weight tiles and K split in 4; batch 8: 128-row tiles, K split in 2)."""
    run_case(synthetic.BERT_BASE, batch, dtype_name, plan_dir, seed=20)


def test_forward_plan_refuses_misuse(plan_dir):
    config = synthetic.TINY_BERT
    weights = synthetic.encoder_weights(config, seed=0)
    so = emit_plan(config, plan_dir, phase="forward", batch_lo=1, batch_hi=2, dtype="f16")
    with EncoderEngine(TensorCheckpoint(weights), so, 2) as engine:
        with pytest.raises(ValueError):
            engine.plan.set_steps([1])
        with pytest.raises(ValueError):
            engine.plan.launch(1, L2, 0)
        with pytest.raises(RuntimeError):
            engine.plan.launch_steps(0, 2, L2, 0)
        with pytest.raises(ValueError):
            engine(torch.zeros(1, 128, dtype=torch.int64).cuda(), torch.zeros(1, 128, dtype=torch.int64).cuda())
        assert engine.plan.watchdog() is None
