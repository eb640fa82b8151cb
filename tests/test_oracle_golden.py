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


@pytest.mark.parametrize("name", ["tiny", "tiny_d128", "tiny_moe"])
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


def test_oracle_tensor_parallel_partials_match_reference_rank_modules():
    """The oracle's per-rank o_proj / down_proj partials and vocabulary slices are the
    outputs of the reference's own rank modules (tests/golden/make_golden_tp.py), bit
    for bit; and the rank-ordered sum of T = 1 is the unsharded linear."""
    from oracle.decoder_oracle import rms_norm
    import torch.nn.functional as F
    record = torch.load(GOLDEN / "tiny_tp2.pt")
    config, world, batch, past = record["config"], record["world"], record["batch"], record["past"]
    weights = synthetic.seeded_weights(config, seed=0, dtype=torch.bfloat16)
    weights.setdefault("lm_head.weight", weights["model.embed_tokens.weight"])
    decoder = OracleDecoder(config, weights, torch.bfloat16, capacity=32, tp=world)
    kv = PagedKV(config, batch, 32, torch.bfloat16)
    for b in range(batch):
        kv.append(0, b, 0, record["past_k"][b].transpose(0, 1), record["past_v"][b].transpose(0, 1))
    x = record["x"]
    normed = rms_norm(x, decoder.w["model.layers.0.input_layernorm.weight"], decoder.eps)
    attention = decoder.attention_partials(0, normed, [past] * batch, kv)
    mlp = decoder.mlp_partials(0, rms_norm(x, decoder.w["model.layers.0.post_attention_layernorm.weight"], decoder.eps))
    assert len(attention) == len(mlp) == world
    for rank in range(world):
        # the rank module runs the whole batch in one GEMM; the oracle one sequence at a
        # time for attention: identical ops per row, so the bf16 outputs agree exactly
        assert torch.equal(attention[rank], record["attention"][rank])
        assert torch.equal(mlp[rank], record["mlp"][rank])
    head = F.linear(rms_norm(x, decoder.w["model.norm.weight"], decoder.eps), decoder.w["lm_head.weight"])
    assert torch.equal(head, torch.cat(record["head"], dim=-1))
    # the all-reduce rule: fp32 sum of the bf16 partials in rank order, one rounding
    total = (record["mlp"][0].float() + record["mlp"][1].float()).to(torch.bfloat16)
    assert torch.equal(decoder.mlp(0, rms_norm(x, decoder.w["model.layers.0.post_attention_layernorm.weight"],
                                               decoder.eps)), total)
    single = OracleDecoder(config, weights, torch.bfloat16, capacity=32, tp=1)
    assert len(single.mlp_partials(0, x)) == 1
