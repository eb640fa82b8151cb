"""Stage-by-stage parity of the CUDA decode step with the reference's math.

Rounding to bf16 amplifies any fp32-level difference to full bf16 noise within a
few consecutive roundings, so two correct implementations drift apart over a
whole forward no matter how exact each op is (the reference's own bf16 and fp32
CPU forwards differ by 0.13 max-abs on its 1B-shaped config). The exact check is
therefore made per stage: every stage's output buffer is recomputed on the CPU
from the INPUT BUFFERS THE GPU ACTUALLY HAD, with the reference's op sequence and
rounding sites, and must agree to within one bf16 unit in the last place, with
almost every element bit-identical. The logits (kept in fp32) must agree to 2e-2,
the bound the benchmark states, and in practice agree far closer."""
import pytest
import torch
import torch.nn.functional as F

from oracle.decoder_oracle import rms_norm, rotate_half, rope_tables
from tilemega_b200 import synthetic
from tilemega_b200.serving.state import kv_row_swizzle

from harness import GpuRun, bf16_ulp, bf16_weights

pytestmark = pytest.mark.gpu


def agreement(got, ref, what, ulps=1.0, exact_fraction=0.99, floor=1e-6, outliers=0.0, outlier_bound=0.0):
    """`outliers`: fraction of the elements that may miss the bound, by at most `outlier_bound` in
    absolute terms (an output that is a sum of much larger addends inherits THEIR rounding: among
    tens of thousands of elements a handful cancel that far)."""
    got, ref = got.float(), ref.float()
    diff = (got - ref).abs()
    within = diff <= ulps * bf16_ulp(ref) + floor   # absolute floor: outputs that cancel to ~0
    exact = (diff == 0).float().mean().item()
    if outliers:
        assert (diff[~within] <= outlier_bound).all(), f"{what}: an element differs by {diff[~within].max().item()}"
        assert (~within).float().mean().item() <= outliers, f"{what}: {int((~within).sum())} elements beyond {ulps} ulp"
        within = torch.ones_like(within)
    assert within.all(), f"{what}: {int((~within).sum())} elements differ by more than {ulps} ulp (max {diff.max().item()})"
    assert exact >= exact_fraction, f"{what}: only {exact:.4f} of the elements are bit-identical"
    return exact


@pytest.mark.parametrize("base,batch,history", [("TINY", 2, 37), ("TINY_D128", 3, 70), ("TINY", 1, 129),
                                                ("TINY", 8, 21), ("TINY_D128", 5, 33), ("TINY_GQ8", 2, 75),
                                                # long histories: several chunks per KV head, merged by the last arriver
                                                ("TINY_D128", 2, 701), ("TINY", 1, 1533), ("TINY_GQ8", 3, 389)])
def test_every_stage_of_one_layer(base, batch, history, plan_dir):
    check_every_stage(dict(getattr(synthetic, base), num_hidden_layers=1), batch, history, plan_dir)


# Much attention work per CTA (forced here with a small grid): the slots of all (sequence, KV head) units are cut
# into equal ranges, one per CTA, and a range crosses unit boundaries -- units of 11 slots in ranges of 9, units
# of 3 slots in ranges of 12.
@pytest.mark.parametrize("base,batch,history,grid,min_slots", [("TINY_D128", 3, 701, 8, 1), ("TINY", 8, 300, 16, 2),
                                                              ("TINY_GQ8", 2, 1100, 3, 1)])
def test_attention_in_equal_ranges(base, batch, history, grid, min_slots, plan_dir):
    check_every_stage(dict(getattr(synthetic, base), num_hidden_layers=1), batch, history, plan_dir, grid=grid,
                      attn_min_slots=min_slots)


# The benchmark configurations' own widths, one layer each: the Llama-3.2-1B shape (hidden 2048, head_dim
# 64, FFN 8192, vocabulary 128256, tied) and the Llama-3.1-8B shape (hidden 4096, head_dim 128, FFN 14336 =
# seven 2048-column pages per down task, vocabulary 128256) at batch 1 and at the GEMV path's widest batch.
@pytest.mark.parametrize("base,batch,history", [("LLAMA_3_2_1B", 1, 130), ("LLAMA_3_1_8B", 1, 150),
                                                ("LLAMA_3_1_8B", 8, 45)])
def test_every_stage_at_benchmark_widths(base, batch, history, plan_dir):
    check_every_stage(dict(getattr(synthetic, base), num_hidden_layers=1), batch, history, plan_dir)


def linear(x, weight):
    """One linear layer as the kernels compute it: fp32 products and sums, one rounding to bf16
    (for bf16 weights this is what the module's bf16 F.linear does)."""
    return F.linear(x.float(), weight.float()).to(torch.bfloat16)


def check_every_stage(config, batch, history, plan_dir, weights="bf16", grid=0, attn_min_slots=None):
    dim, heads, hkv = config["head_dim"], config["num_attention_heads"], config["num_key_value_heads"]
    hidden, eps = config["hidden_size"], config["rms_norm_eps"]
    capacity = (history + 18) // 16 * 16
    w = bf16_weights(config)
    run = GpuRun(config, w, batch, capacity, plan_dir, weights=weights, grid=grid, attn_min_slots=attn_min_slots)
    if weights == "e4m3":
        # the CPU side multiplies with what the plan's pages hold: every matrix quantised row by row and
        # scaled back (fp32), exactly as the loader derives codes and scales from the bf16 checkpoint
        from tilemega_b200.serving.weights import dequantize_e4m3, quantize_e4m3
        w = {name: dequantize_e4m3(*quantize_e4m3(t)) if t.ndim == 2 and "embed_tokens" not in name else t
             for name, t in w.items()}
        if "lm_head.weight" not in w:   # a tied head is quantised too, the embedding table is not
            w["lm_head.weight"] = dequantize_e4m3(*quantize_e4m3(w["model.embed_tokens.weight"]))
    ids = synthetic.seeded_tokens(batch, history + 2, config["vocab_size"], seed=9)
    run.state.tokens.zero_()
    run.state.tokens[:, :history + 2].copy_(ids)
    run.plan.set_prompt_len(history + 2)
    run.plan.set_steps(list(range(history + 1)))
    run.plan.launch_steps(0, history, 2, run.stream)      # positions 0 .. history-1 fill the cache
    run.plan.launch(history, 2, run.stream)               # the step under test: position `history`
    run.check_alive()
    pos = history
    gq = heads // hkv
    qkv_gpu = run.read("serving.qkv").reshape(batch, hkv, gq + 2, dim)
    attn_gpu = run.read("serving.attention").reshape(batch, heads * dim)
    h_gpu = run.read("serving.mlp").reshape(batch, -1)
    x_gpu = run.read("serving.hidden").reshape(batch, hidden)
    logits_gpu = run.read("serving.logits", torch.float32).reshape(batch, -1)
    cache = kv_row_swizzle(run.state.kv_storage.cpu())    # [1][2][B][Hkv][cap][D], logical column order
    p = "model.layers.0."
    # stage 1: RMSNorm + QKV
    x_in = F.embedding(ids[:, pos].long(), w["model.embed_tokens.weight"])
    xn = rms_norm(x_in, w[p + "input_layernorm.weight"], eps)
    q = linear(xn, w[p + "self_attn.q_proj.weight"]).view(batch, hkv, gq, dim)
    k = linear(xn, w[p + "self_attn.k_proj.weight"]).view(batch, hkv, 1, dim)
    v = linear(xn, w[p + "self_attn.v_proj.weight"]).view(batch, hkv, 1, dim)
    # (a handful of elements per hundred thousand may sit two steps apart: the CPU's bf16 GEMM and the GPU
    # sum 2048+ products in different orders and block sizes)
    reference_qkv = torch.cat((q, k, v), dim=2)
    agreement(qkv_gpu, reference_qkv, "qkv", outliers=2e-5, outlier_bound=2 * bf16_ulp(reference_qkv.float().abs().max()).item())
    # stage 2: RoPE, KV append, attention -- from the qkv the GPU produced
    cos, sin = rope_tables(config, capacity, torch.bfloat16)
    q_gpu, k_gpu, v_gpu = qkv_gpu[:, :, :gq], qkv_gpu[:, :, gq], qkv_gpu[:, :, gq + 1]
    q_rot = q_gpu * cos[pos] + rotate_half(q_gpu) * sin[pos]
    k_rot = k_gpu * cos[pos] + rotate_half(k_gpu) * sin[pos]
    assert torch.equal(cache[0, 0, :, :, pos], k_rot), "appended key row is not the roped key, bit for bit"
    assert torch.equal(cache[0, 1, :, :, pos], v_gpu), "appended value row is not the projected value"
    assert cache[0, :, :, :, pos + 1:].abs().max().item() == 0, "rows past the context were written"
    keys = cache[0, 0, :, :, :pos + 1].float()            # [B][Hkv][T][D] (the GPU's own history)
    values = cache[0, 1, :, :, :pos + 1].float()
    score = torch.einsum("bgqd,bgtd->bgqt", q_rot.float(), keys) / dim ** 0.5
    context = torch.einsum("bgqt,bgtd->bgqd", torch.softmax(score, dim=-1), values).to(torch.bfloat16)
    # the oracle rounds the probabilities to bf16 before the value product (2^-9 relative), the kernel
    # keeps about 16 bits of them: where one key dominates and the output nearly cancels, the two
    # differ by up to that fraction of the values' magnitude
    agreement(attn_gpu, context.reshape(batch, heads * dim), "attention", outliers=1e-4,
              outlier_bound=2.0 ** -8 * values.abs().max().item())
    # stage 3: o projection + residual (from the GPU's attention output)
    x_mid = x_in + linear(attn_gpu, w[p + "self_attn.o_proj.weight"])
    # stage 4: RMSNorm + gate/up + SwiGLU
    xm = rms_norm(x_mid, w[p + "post_attention_layernorm.weight"], eps)
    gate_ref, up_ref = F.silu(linear(xm, w[p + "mlp.gate_proj.weight"])), linear(xm, w[p + "mlp.up_proj.weight"])
    h_ref = gate_ref * up_ref
    # a product of two bf16 values that may each be one ulp off: the error scales with the
    # factors, not with a product that happens to be small: one ulp of the up projection times the gate
    # factor, three of the gate factor times the up projection (a gate pre-activation one ulp off moves
    # silu by up to ~1.5 of ITS ulps before its own rounding), plus the product's own rounding
    # (the CPU chain starts from the GPU's attention output, so the GPU's own roundings of the residual
    # stream and of the norm sit in between as well: a few elements in a hundred thousand land further out)
    agreement(h_gpu, h_ref, "swiglu", ulps=2.0, exact_fraction=0.93,
              floor=1e-3 + 3 * bf16_ulp(gate_ref.float()) * up_ref.float().abs() + bf16_ulp(up_ref.float()) * gate_ref.float().abs(),
              outliers=1e-4, outlier_bound=4 * bf16_ulp(h_ref.float().abs().max()).item())
    # stage 5: down projection + residual (from the GPU's own activations)
    # the sum may cancel to something much smaller than its addends, whose own ulp bounds the error
    agreement(x_gpu, x_mid + linear(h_gpu, w[p + "mlp.down_proj.weight"]), "residual stream", ulps=2.0,
              exact_fraction=0.93, floor=2e-3, outliers=1e-4, outlier_bound=2 * bf16_ulp(x_mid.float().abs().max()).item())
    # stage 6: final norm + lm_head, accumulators in fp32
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    logits_ref = F.linear(rms_norm(x_gpu, w["model.norm.weight"], eps).float(), head.float())
    diff = (logits_gpu - logits_ref).abs().max().item()
    assert diff <= 2e-2 and diff <= 1e-3 * max(1.0, logits_ref.abs().max().item()), diff
    # the token written for the next position is the argmax of the bf16-rounded logits, ties to the smaller index
    rounded = logits_gpu.to(torch.bfloat16).float()
    expect = torch.stack([torch.nonzero(row == row.max())[0, 0] for row in rounded]).to(torch.int32)
    assert torch.equal(run.state.tokens[:, pos + 1].cpu(), ids[:, pos + 1]), "teacher-forced token was overwritten"
    run.plan.set_prompt_len(0)
    run.plan.set_steps(list(range(history + 1)))
    run.plan.launch(history, 2, run.stream)               # same position again, now free-running
    run.check_alive()
    assert torch.equal(run.state.tokens[:, pos + 1].cpu(), expect)
    run.close()
