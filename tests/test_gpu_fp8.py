"""e4m3 weight plans on the GPU (the second variant of the 70B-shaped benchmark configuration: FP8
e4m3 weights with per-output-channel fp32 scales). The reference has no 8-bit path, so the oracle is
its forward run with the weights the pages hold: every matrix quantised row by row exactly as the
loader does and scaled back to fp32. Per stage (tests/test_gpu_stages.py has the method) and as a
whole forward; also across tensor-parallel ranks launched together on one device."""
import pytest
import torch

from oracle.decoder_oracle import OracleDecoder, PagedKV
from tilemega_b200 import synthetic
from tilemega_b200.serving.weights import dequantize_e4m3, quantize_e4m3

from harness import GpuRun, assert_parity, bf16_weights
from test_gpu_stages import check_every_stage

pytestmark = pytest.mark.gpu
LOGIT_TOLERANCE = 2e-2


def held_weights(weights, dtype, ranks=1):
    """What an e4m3 plan multiplies with, as `dtype` tensors for the oracle. A tensor-parallel rank
    quantises its own slice: the column-sharded matrices (o, down) get their row scales per column part."""
    def held(name, t):
        if t.ndim != 2 or "embed_tokens" in name:
            return t.float()
        if ranks > 1 and (name.endswith("o_proj.weight") or name.endswith("down_proj.weight")):
            return torch.cat([dequantize_e4m3(*quantize_e4m3(part.contiguous())) for part in t.chunk(ranks, dim=1)], dim=1)
        return dequantize_e4m3(*quantize_e4m3(t))
    out = {name: held(name, t).to(dtype) for name, t in weights.items()}
    if "lm_head.weight" not in out:
        out["lm_head.weight"] = dequantize_e4m3(*quantize_e4m3(weights["model.embed_tokens.weight"])).to(dtype)
    return out


@pytest.mark.parametrize("base,batch,history", [
    ("TINY_D128", 1, 40), ("TINY_D128", 3, 70), ("TINY_GQ8", 8, 21),
    # the 8B shape's widths (FFN 14336: a down task of 3.5 pages of 4096 columns) and the 70B shape's hidden size
    ("LLAMA_3_1_8B", 1, 50), ("LLAMA_3_1_8B", 8, 33)])
def test_every_stage_with_e4m3_weights(base, batch, history, plan_dir):
    check_every_stage(dict(getattr(synthetic, base), num_hidden_layers=1), batch, history, plan_dir, weights="e4m3")


def test_e4m3_decode_matches_the_forward_with_the_held_weights(plan_dir):
    config = dict(synthetic.TINY_D128, tie_word_embeddings=False)
    batch, prompt_len, new_tokens, capacity = 2, 9, 6, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    run = GpuRun(config, weights, batch, capacity, plan_dir, weights="e4m3")
    tokens, logits = run.greedy(prompt, new_tokens)
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()
    config_untied = dict(config)

    def forced(dtype):
        decoder = OracleDecoder(config_untied, held_weights(weights, dtype), dtype, capacity)
        return decoder.greedy(prompt, new_tokens, PagedKV(config_untied, batch, capacity, dtype), forced=tokens, head_fp32=True)[1]

    exact, module = forced(torch.float32), forced(torch.bfloat16)
    ours, theirs = (logits - exact).abs(), (module - exact).abs()
    # the bf16 forward also rounds the held weights to bf16, which the kernel does not: the GPU must be at
    # least as close to the exact forward as that
    assert ours.max().item() <= 1.25 * theirs.max().item(), (ours.max().item(), theirs.max().item())
    assert ours.mean().item() <= 1.25 * theirs.mean().item(), (ours.mean().item(), theirs.mean().item())
    assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), "e4m3 tiny_d128")
    # and the 8-bit weights do change the result against the bf16 plan (the test is not vacuous)
    plain = GpuRun(config, weights, batch, capacity, plan_dir)
    _, plain_logits = plain.greedy(prompt, new_tokens)
    plain.close()
    assert (plain_logits - logits).abs().max().item() > 1e-3


@pytest.mark.parametrize("base,ranks,batch", [("TINY_D128", 2, 2), ("TINY_GQ8", 2, 1)])
def test_e4m3_tensor_parallel_ranks_on_one_device(base, ranks, batch, plan_dir):
    """The benchmark's tensor-parallel configuration in its e4m3 variant: every rank quantises its own
    slices; the ranks run as one cooperative launch on this GPU (tests/test_gpu_tp_one_device.py)."""
    from test_gpu_tp_one_device import RanksOnOneDevice
    config = dict(getattr(synthetic, base), tie_word_embeddings=False)
    prompt_len, new_tokens, capacity = 11, 5, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    run = RanksOnOneDevice(config, weights, batch, capacity, plan_dir, ranks, weights="e4m3")
    tokens, logits = run.greedy(prompt, new_tokens)
    run.close()

    def forced(dtype):
        decoder = OracleDecoder(config, held_weights(weights, dtype, ranks), dtype, capacity, tp=ranks)
        return decoder.greedy(prompt, new_tokens, PagedKV(config, batch, capacity, dtype), forced=tokens, head_fp32=True)[1]

    exact, module = forced(torch.float32), forced(torch.bfloat16)
    ours, theirs = (logits - exact).abs(), (module - exact).abs()
    assert ours.max().item() <= 1.25 * theirs.max().item(), (ours.max().item(), theirs.max().item())
    assert ours.mean().item() <= 1.25 * theirs.mean().item(), (ours.mean().item(), theirs.mean().item())
    assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), f"e4m3 {base} tp{ranks}")
