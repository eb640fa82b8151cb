"""The CPU oracle against fixtures produced by the reference's own module
(tests/golden/make_golden.py), in fp32 and in bf16."""
from pathlib import Path

import pytest
import torch

from oracle.decoder_oracle import OracleDecoder, PagedKV
from tilemega_b200 import synthetic

GOLDEN = Path(__file__).resolve().parent / "golden"
MODES = (("fp32", torch.float32, torch.float32), ("fp32_bf16w", torch.float32, torch.bfloat16),
         ("bf16", torch.bfloat16, torch.bfloat16))


def run_oracle(record, dtype, rounding, block_table=None, num_blocks=None):
    config = record["config"]
    weights = {name: tensor.to(rounding) for name, tensor in synthetic.seeded_weights(config, seed=0).items()}
    capacity = (record["prompt_len"] + record["new_tokens"] + 16) // 16 * 16
    decoder = OracleDecoder(config, weights, dtype, capacity)
    kv = PagedKV(config, record["batch"], capacity, dtype, block_table, num_blocks)
    return decoder.greedy(record["prompt"], record["new_tokens"], kv)


@pytest.mark.parametrize("name", ["tiny", "tiny_d128"])
@pytest.mark.parametrize("mode", MODES, ids=[m[0] for m in MODES])
def test_oracle_reproduces_reference_small(name, mode):
    label, dtype, rounding = mode
    record = torch.load(GOLDEN / f"{name}.pt")
    assert (record["prompt"] == synthetic.seeded_tokens(record["batch"], record["prompt_len"],
                                                        record["config"]["vocab_size"], seed=1)).all()
    tokens, logits = run_oracle(record, dtype, rounding)
    golden = record[label]
    assert torch.equal(tokens, golden["tokens"])
    # the same ops on the same dtypes; the only freedom is the GEMM blocking over
    # [B*S] rows (the oracle runs attention per sequence), far below one bf16 ulp
    tolerance = 2e-5 if dtype == torch.float32 else 0.04
    assert (logits - golden["logits"]).abs().max().item() <= tolerance


def test_oracle_block_table_is_transparent():
    """Shuffling the pool blocks must not change a single bit."""
    record = torch.load(GOLDEN / "tiny.pt")
    capacity = (record["prompt_len"] + record["new_tokens"] + 16) // 16 * 16
    from tilemega_b200.serving.state import shuffled_block_table
    table = shuffled_block_table(record["batch"], capacity // 16, 3 * record["batch"] * capacity // 16, seed=7)
    base_tokens, base_logits = run_oracle(record, torch.bfloat16, torch.bfloat16)
    tokens, logits = run_oracle(record, torch.bfloat16, torch.bfloat16, table, 3 * record["batch"] * capacity // 16)
    assert torch.equal(tokens, base_tokens) and torch.equal(logits, base_logits)


@pytest.mark.parametrize("mode", [MODES[2]], ids=["bf16"])
def test_oracle_reproduces_reference_llama_1b(mode):
    """Config 1 of the benchmark list: Llama-3.2-1B shape, batch 1, prompt 128, 32 greedy steps."""
    label, dtype, rounding = mode
    record = torch.load(GOLDEN / "llama_3_2_1b.pt")
    tokens, logits = run_oracle(record, dtype, rounding)
    golden = record[label]
    assert torch.equal(tokens, golden["tokens"])
    top = logits.topk(8, dim=-1)
    assert torch.equal(top.indices.to(torch.int32), golden["top_indices"])
    assert (top.values - golden["top_values"]).abs().max().item() <= 0.04
