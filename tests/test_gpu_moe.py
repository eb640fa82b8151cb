"""Mixture-of-experts decode (router, top-k, chosen experts, weighted sum) and the per-head QK
norm, batch 1 to 8 (the experts' MLP runs token by token), through the C ABI against the CPU oracle."""
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


@pytest.mark.parametrize("batch", [1, 2])
def test_moe_decode_matches_oracle_and_routes_identically(batch, plan_dir):
    config = synthetic.TINY_MOE
    record = torch.load(GOLDEN / "tiny_moe.pt")
    prompt, new_tokens, capacity = record["prompt"][:batch], record["new_tokens"], 64
    weights = bf16_weights(config)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    # [layers][batch][topk]
    route = run.read("serving.route_index", torch.int32).reshape(config["num_hidden_layers"], batch, -1)
    route_weight = run.read("serving.route_weight", torch.float32).reshape(config["num_hidden_layers"], batch, -1)
    exact_decoder, exact = forced_oracle(config, weights, prompt, tokens, capacity, torch.float32)
    module_decoder, module = forced_oracle(config, weights, prompt, tokens, capacity, torch.bfloat16)
    ours, theirs = (logits - exact).abs(), (module - exact).abs()
    assert ours.max().item() <= 1.25 * theirs.max().item(), (ours.max().item(), theirs.max().item())
    assert ours.mean().item() <= 1.25 * theirs.mean().item(), (ours.mean().item(), theirs.mean().item())
    assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), "tiny moe")
    # routing of the last step: layer 0 sees the same input on the GPU and in the bf16 oracle up to the
    # attention block's rounding noise; indices must be identical (in rank order) unless two experts tie
    for b in range(batch):
        expected = module_decoder.last_route[0][b].to(torch.int32)      # layer 0, token b: [k]
        assert torch.equal(route[0, b], expected), (b, route[0, b].tolist(), expected.tolist())
        assert abs(route_weight[0, b].sum().item() - 1.0) < 1e-5 and (route_weight[0, b][:-1] >= route_weight[0, b][1:]).all()
    # the fixture is the reference module's own free-running bf16 decode of a batch of two; the same
    # sequences (alone or together) must give the same tokens while the margins are decided
    golden = record["bf16"]
    for b in range(batch):
        margin = (golden["top_values"][..., 0] - golden["top_values"][..., 1])[:, b]
        if (margin > 2 * LOGIT_TOLERANCE).all():
            assert torch.equal(tokens[b], golden["tokens"][b])
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()


# TINY_MOE has 16 experts and 4 per token; the Qwen3-30B-A3B shape is the benchmark's own: 128 experts,
# 8 per token (all eight slots of the routing and of the down stage's sub-tasks), vocabulary 151936.
@pytest.mark.parametrize("base", ["TINY_MOE", "QWEN3_30B_A3B"])
def test_every_moe_stage_of_one_layer(base, plan_dir):
    """Router logits, routing, expert SwiGLU rows and the weighted expert sum, each recomputed on
    the CPU from the buffers the GPU had (see tests/test_gpu_stages.py for the method); the QK norm
    is checked through the appended key row."""
    import torch.nn.functional as F
    from oracle.decoder_oracle import rms_norm, rotate_half, rope_tables
    from tilemega_b200.serving.state import kv_row_swizzle
    from test_gpu_stages import agreement

    config = dict(getattr(synthetic, base), num_hidden_layers=1)
    hidden, eps, dim = config["hidden_size"], config["rms_norm_eps"], config["head_dim"]
    heads, hkv, topk = config["num_attention_heads"], config["num_key_value_heads"], config["num_experts_per_tok"]
    inter = config["moe_intermediate_size"]
    history = 41
    capacity = (history + 18) // 16 * 16
    w = bf16_weights(config)
    run = GpuRun(config, w, 1, capacity, plan_dir)
    ids = synthetic.seeded_tokens(1, history + 2, config["vocab_size"], seed=9)
    run.state.tokens.zero_()
    run.state.tokens[:, :history + 2].copy_(ids)
    run.plan.set_prompt_len(history + 2)
    run.plan.set_steps(list(range(history + 1)))
    run.plan.launch_steps(0, history, 2, run.stream)
    run.plan.launch(history, 2, run.stream)
    run.check_alive()
    pos = history
    gq = heads // hkv
    qkv_gpu = run.read("serving.qkv").reshape(1, hkv, gq + 2, dim)
    attn_gpu = run.read("serving.attention").reshape(1, heads * dim)
    router_gpu = run.read("serving.router_logits").reshape(-1)
    route = run.read("serving.route_index", torch.int32).reshape(-1)
    route_weight = run.read("serving.route_weight", torch.float32).reshape(-1)
    h_gpu = run.read("serving.mlp").reshape(topk, inter)
    x_gpu = run.read("serving.hidden").reshape(1, hidden)
    cache = kv_row_swizzle(run.state.kv_storage.cpu())
    p = "model.layers.0."
    # QK norm + RoPE of the new key, from the GPU's own projection
    cos, sin = rope_tables(config, capacity, torch.bfloat16)
    k_normed = rms_norm(qkv_gpu[:, :, gq], w[p + "self_attn.k_norm.weight"], eps)
    k_rot = k_normed * cos[pos] + rotate_half(k_normed) * sin[pos]
    agreement(cache[0, 0, :, :, pos], k_rot, "normalised, roped key row", ulps=1.0, exact_fraction=0.97)
    # residual stream after attention, from the GPU's attention output
    x_in = F.embedding(ids[:, pos].long(), w["model.embed_tokens.weight"])
    x_mid = x_in + F.linear(attn_gpu, w[p + "self_attn.o_proj.weight"])
    xm = rms_norm(x_mid, w[p + "post_attention_layernorm.weight"], eps)
    # router: one bf16 rounding per logit
    agreement(router_gpu, F.linear(xm, w[p + "mlp.gate.weight"]).reshape(-1), "router logits", ulps=1.0, exact_fraction=0.9)
    # routing from the GPU's own logits: indices bit-exact and in rank order, weights renormalised in fp32
    probability = torch.softmax(router_gpu.float(), -1)
    # descending probability, ties to the smaller expert index (include/tilemega/Backend/Sm90DenseMoe.cuh:30-35;
    # torch.topk leaves the order of exact ties open, and bf16 logits of 128 experts do tie)
    order = sorted(range(probability.numel()), key=lambda e: (-probability[e].item(), e))[:topk]
    assert route.tolist() == order, (route.tolist(), order)
    weight = probability[order]
    assert torch.allclose(route_weight, weight / weight.sum(), rtol=0, atol=2e-6)
    # expert SwiGLU rows, one per chosen expert
    for slot in range(topk):
        e = p + f"mlp.experts.{int(route[slot])}."
        h_ref = F.silu(F.linear(xm, w[e + "gate_proj.weight"])) * F.linear(xm, w[e + "up_proj.weight"])
        agreement(h_gpu[slot], h_ref.reshape(-1), f"expert {int(route[slot])} swiglu", ulps=2.0, exact_fraction=0.95, floor=1e-3)
    # weighted sum of the experts' down projections (from the GPU's rows and weights), then the residual
    total = torch.zeros(hidden)
    for slot in range(topk):
        e = p + f"mlp.experts.{int(route[slot])}."
        total = total + F.linear(h_gpu[slot], w[e + "down_proj.weight"]).float() * route_weight[slot]
    agreement(x_gpu, x_mid + total.to(torch.bfloat16).reshape(1, hidden), "residual stream after the experts", ulps=2.0,
              exact_fraction=0.95, floor=2e-3)
    run.close()


def test_every_token_of_a_batch_goes_through_its_own_experts(plan_dir):
    """Batch 3, one layer: every token's router scores and routing from the buffers the GPU had, the
    last token's expert rows (the buffer holds the rows of the token served last), and every token's
    residual stream after its experts."""
    import torch.nn.functional as F
    from oracle.decoder_oracle import rms_norm
    from test_gpu_stages import agreement

    config = dict(synthetic.TINY_MOE, num_hidden_layers=1)
    batch, history = 3, 23
    hidden, eps = config["hidden_size"], config["rms_norm_eps"]
    heads, dim, topk, inter = config["num_attention_heads"], config["head_dim"], config["num_experts_per_tok"], config["moe_intermediate_size"]
    capacity = (history + 18) // 16 * 16
    w = bf16_weights(config)
    run = GpuRun(config, w, batch, capacity, plan_dir)
    ids = synthetic.seeded_tokens(batch, history + 2, config["vocab_size"], seed=9)
    run.state.tokens.zero_()
    run.state.tokens[:, :history + 2].copy_(ids)
    run.plan.set_prompt_len(history + 2)
    run.plan.set_steps(list(range(history + 1)))
    run.plan.launch_steps(0, history, 2, run.stream)
    run.plan.launch(history, 2, run.stream)
    run.check_alive()
    attn_gpu = run.read("serving.attention").reshape(batch, heads * dim)
    router_gpu = run.read("serving.router_logits").reshape(batch, -1)
    route = run.read("serving.route_index", torch.int32).reshape(1, batch, topk)[0]
    route_weight = run.read("serving.route_weight", torch.float32).reshape(1, batch, topk)[0]
    h_gpu = run.read("serving.mlp").reshape(-1)[:topk * inter].reshape(topk, inter)
    x_gpu = run.read("serving.hidden").reshape(batch, hidden)
    p = "model.layers.0."
    x_in = F.embedding(ids[:, history].long(), w["model.embed_tokens.weight"])
    x_mid = x_in + F.linear(attn_gpu, w[p + "self_attn.o_proj.weight"])
    xm = rms_norm(x_mid, w[p + "post_attention_layernorm.weight"], eps)
    agreement(router_gpu, F.linear(xm, w[p + "mlp.gate.weight"]), "router logits", ulps=1.0, exact_fraction=0.9)
    for b in range(batch):
        probability = torch.softmax(router_gpu[b].float(), -1)
        order = sorted(range(probability.numel()), key=lambda e: (-probability[e].item(), e))[:topk]
        assert route[b].tolist() == order, (b, route[b].tolist(), order)
        weight = probability[order]
        assert torch.allclose(route_weight[b], weight / weight.sum(), rtol=0, atol=2e-6)
        total = torch.zeros(hidden)
        for slot in range(topk):
            e = p + f"mlp.experts.{int(route[b, slot])}."
            h_ref = F.silu(F.linear(xm[b:b + 1], w[e + "gate_proj.weight"])) * F.linear(xm[b:b + 1], w[e + "up_proj.weight"])
            if b == batch - 1:      # the rows the GPU kept are the last token's
                agreement(h_gpu[slot], h_ref.reshape(-1), f"token {b} expert {int(route[b, slot])} swiglu", ulps=2.0,
                          exact_fraction=0.95, floor=1e-3)
                h_ref = h_gpu[slot].reshape(1, -1)
            total = total + F.linear(h_ref, w[e + "down_proj.weight"]).float().reshape(-1) * route_weight[b, slot]
        # (tokens before the last: the CPU's own expert rows stand in for the GPU's, which differ by their last bit)
        agreement(x_gpu[b], (x_mid[b] + total.to(torch.bfloat16)), f"token {b}: residual stream after the experts",
                  ulps=2.0 if b == batch - 1 else 3.0, exact_fraction=0.95 if b == batch - 1 else 0.8, floor=2e-3)
    run.close()
