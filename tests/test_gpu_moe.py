"""Mixture-of-experts decode (router, top-k, chosen experts, weighted sum) and the per-head QK
norm, batch 1, through the C ABI against the CPU oracle."""
from pathlib import Path

import pytest
import torch

from oracle.decoder_oracle import OracleDecoder, PagedKV
from tilemega_b200 import synthetic

from harness import GpuRun, assert_parity, bf16_weights

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
LOGIT_TOLERANCE = 2e-2


def forced_oracle(config, weights, prompt, forced, capacity, dtype):
    decoder = OracleDecoder(config, weights, dtype, capacity)
    kv = PagedKV(config, prompt.shape[0], capacity, dtype)
    _, logits = decoder.greedy(prompt, forced.shape[1], kv, forced=forced, head_fp32=True)
    return decoder, logits


def test_moe_decode_matches_oracle_and_routes_identically(plan_dir):
    config = synthetic.TINY_MOE
    record = torch.load(GOLDEN / "tiny_moe.pt")
    prompt, new_tokens, capacity = record["prompt"][:1], record["new_tokens"], 64
    weights = bf16_weights(config)
    run = GpuRun(config, weights, 1, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    route = run.read("serving.route_index", torch.int32).reshape(config["num_hidden_layers"], -1)
    route_weight = run.read("serving.route_weight", torch.float32).reshape(config["num_hidden_layers"], -1)
    exact_decoder, exact = forced_oracle(config, weights, prompt, tokens, capacity, torch.float32)
    module_decoder, module = forced_oracle(config, weights, prompt, tokens, capacity, torch.bfloat16)
    ours, theirs = (logits - exact).abs(), (module - exact).abs()
    assert ours.max().item() <= 1.25 * theirs.max().item(), (ours.max().item(), theirs.max().item())
    assert ours.mean().item() <= 1.25 * theirs.mean().item(), (ours.mean().item(), theirs.mean().item())
    assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), "tiny moe")
    # routing of the last step: layer 0 sees the same input on the GPU and in the bf16 oracle up to the
    # attention block's rounding noise; indices must be identical (in rank order) unless two experts tie
    expected = module_decoder.last_route[0][0].to(torch.int32)
    assert torch.equal(route[0], expected), (route[0].tolist(), expected.tolist())
    assert abs(route_weight[0].sum().item() - 1.0) < 1e-5 and (route_weight[0][:-1] >= route_weight[0][1:]).all()
    # the fixture is the reference module's own free-running bf16 decode of the first sequence's batch
    # of two; sequence 0 alone must give the same tokens while the margins are decided
    golden = record["bf16"]
    margin = (golden["top_values"][..., 0] - golden["top_values"][..., 1])[:, 0]
    if (margin > 2 * LOGIT_TOLERANCE).all():
        assert torch.equal(tokens[0], golden["tokens"][0])
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()
