"""Whole-forward parity of the CUDA decode path (through the C ABI) with the CPU
oracle and with fixtures made by the reference's own module.

Over a whole forward two correct bf16 implementations drift apart to bf16 noise
(see tests/test_gpu_stages.py for the exact per-stage check), so the yardstick
here is the reference's own: its bf16 CPU forward against its fp32 CPU forward
on the same bf16-rounded weights and the same token history. The CUDA path must
be at least as close to the fp32 forward as that (factor 1.25 on max-abs and on
the mean), its greedy token must be one of the fp32 forward's near-ties at every
step and equal to it wherever the top-2 margin is decided, and block tables,
token ids and appended KV rows are compared bit for bit."""
from pathlib import Path

import pytest
import torch

from oracle.decoder_oracle import OracleDecoder, PagedKV
from tilemega_b200 import synthetic
from tilemega_b200.serving.state import kv_row_swizzle, shuffled_block_table

from harness import GpuRun, assert_parity, bf16_ulp, bf16_weights

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
LOGIT_TOLERANCE = 2e-2


def oracle_logits_for(config, weights, prompt, forced, capacity, dtype=torch.bfloat16):
    decoder = OracleDecoder(config, weights, dtype, capacity)
    kv = PagedKV(config, prompt.shape[0], capacity, dtype)
    _, logits = decoder.greedy(prompt, forced.shape[1], kv, forced=forced, head_fp32=True)
    return logits


def assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, label):
    """d(GPU, fp32 forward) <= 1.25 * d(reference bf16 forward, fp32 forward), teacher
    forced on the GPU's tokens; token decisions checked against the fp32 forward."""
    exact = oracle_logits_for(config, weights, prompt, tokens, capacity, torch.float32)
    module = oracle_logits_for(config, weights, prompt, tokens, capacity, torch.bfloat16)
    ours, theirs = (logits - exact).abs(), (module - exact).abs()
    assert ours.max().item() <= 1.25 * theirs.max().item(), (label, ours.max().item(), theirs.max().item())
    assert ours.mean().item() <= 1.25 * theirs.mean().item(), (label, ours.mean().item(), theirs.mean().item())
    assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), label)
    return ours.max().item(), ours.mean().item(), theirs.max().item(), theirs.mean().item()


@pytest.mark.parametrize("name", ["tiny", "tiny_d128"])
def test_small_models_match_oracle_and_reference_fixture(name, plan_dir):
    record = torch.load(GOLDEN / f"{name}.pt")
    config, batch = record["config"], record["batch"]
    prompt, new_tokens = record["prompt"], record["new_tokens"]
    capacity = 64
    weights = bf16_weights(config)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    stats = assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, name)
    # the fixture is the reference module's own free-running bf16 decode
    golden = record["bf16"]
    margin = golden["top_values"][..., 0] - golden["top_values"][..., 1]
    if (margin > 2 * LOGIT_TOLERANCE).all():
        assert torch.equal(tokens, golden["tokens"])
        # two bf16 forwards, each within stats[2] of the fp32 one; the fixture's logits are rounded to bf16
        rounded = logits.to(torch.bfloat16).float()
        assert ((rounded - golden["logits"]).abs() <= bf16_ulp(golden["logits"]) + 2.5 * stats[2]).all()
    # one persistent launch for all decode steps gives the same tokens as step-by-step launches
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()


def test_batch_eight_matches_oracle(plan_dir):
    """The largest batch of the GEMV path (all eight rows of the tensor-pipe A operand, two epilogue passes)."""
    config = synthetic.TINY
    batch, prompt_len, new_tokens, capacity = 8, 19, 5, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=3)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, "tiny batch 8")
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()


def test_block_table_gather_is_bit_exact(plan_dir):
    """A shuffled block table over a larger pool must reproduce the contiguous
    cache bit for bit: tokens, logits and the gathered KV rows."""
    record = torch.load(GOLDEN / "tiny_d128.pt")
    config, batch, prompt, new_tokens = record["config"], record["batch"], record["prompt"], record["new_tokens"]
    capacity = 64
    weights = bf16_weights(config)
    base = GpuRun(config, weights, batch, capacity, plan_dir)
    base_tokens, base_logits = base.greedy(prompt, new_tokens)
    num_blocks = 3 * batch * capacity // 16
    table = shuffled_block_table(batch, capacity // 16, num_blocks, seed=11)
    paged = GpuRun(config, weights, batch, capacity, plan_dir, kv_layout="paged", block_table=table,
                   num_blocks=num_blocks)
    tokens, logits = paged.greedy(prompt, new_tokens)
    assert torch.equal(tokens, base_tokens) and torch.equal(logits, base_logits)
    length = prompt.shape[1] + new_tokens - 1
    contiguous = base.state.kv_storage.cpu()   # [L][2][B][Hkv][cap][D]
    pool = paged.state.kv_storage.cpu()        # [L][2][blocks][Hkv][16][D]
    positions = torch.arange(length)
    for b in range(batch):
        by_row = pool.permute(2, 4, 0, 1, 3, 5)[table[b, positions // 16].long(), positions % 16]  # [len][L][2][Hkv][D]
        assert torch.equal(by_row.permute(1, 2, 3, 0, 4), contiguous[:, :, b, :, :length])
    used = set(table.reshape(-1).tolist())
    untouched = [blk for blk in range(num_blocks) if blk not in used]
    assert pool[:, :, untouched].abs().max().item() == 0
    base.close()
    paged.close()


@pytest.mark.parametrize("bases,capacity,grid,min_slots", [
    ([0, 37, 70], 128, 0, None),
    ([0, 137, 300], 384, 4, 1)])   # 1, 2 and 3 slots per KV head, cut into equal ranges over 4 CTAs
def test_ragged_contexts_match_oracle(bases, capacity, grid, min_slots, plan_dir):
    """Sequences at different positions in one batch (context_base), paged KV."""
    config = synthetic.TINY
    batch, new_tokens = 3, 4
    weights = bf16_weights(config)
    num_blocks = batch * capacity // 16 + 5
    table = shuffled_block_table(batch, capacity // 16, num_blocks, seed=3)
    run = GpuRun(config, weights, batch, capacity, plan_dir, kv_layout="paged", block_table=table,
                 context_base=torch.tensor(bases, dtype=torch.int32), num_blocks=num_blocks, grid=grid,
                 attn_min_slots=min_slots)
    decoder = OracleDecoder(config, weights, torch.bfloat16, capacity)
    kv = PagedKV(config, batch, capacity, torch.bfloat16, table, num_blocks)
    # history: every sequence is prefilled by the oracle up to its own base, and the
    # oracle's cache is copied into the device pool (same layout up to the row swizzle)
    history = synthetic.seeded_tokens(batch, max(bases) + 8, config["vocab_size"], seed=5)
    for b in range(batch):
        if bases[b]:
            sub = PagedKV(config, 1, capacity, torch.bfloat16, table[b:b + 1], num_blocks)
            sub.pool = kv.pool
            decoder.forward(history[b:b + 1, :bases[b]], [0], sub)
    run.state.kv_storage.copy_(kv_row_swizzle(kv.pool))
    prompt_len = 8
    for b in range(batch):
        run.state.tokens[b, bases[b]:bases[b] + prompt_len] = history[b, bases[b]:bases[b] + prompt_len].cuda()
    run.plan.set_prompt_len(0)
    run.plan.set_steps(list(range(prompt_len + new_tokens)))
    # teacher-force the 8 "prompt" positions per sequence by launching them one by one
    # and restoring the known next token before each launch
    logits_gpu = []
    feed = history[:, :].clone()
    for step in range(prompt_len):
        run.plan.launch(step, 2, run.stream)
        torch.cuda.synchronize()
        logits_gpu.append(run.read("serving.logits", torch.float32).reshape(batch, -1))
        for b in range(batch):
            if step + 1 < prompt_len:
                run.state.tokens[b, bases[b] + step + 1] = int(history[b, bases[b] + step + 1])
    run.check_alive()
    logits_cpu = []
    for step in range(prompt_len):
        ids = torch.stack([history[b, bases[b] + step] for b in range(batch)]).view(batch, 1)
        logits_cpu.append(decoder.forward(ids, [bases[b] + step for b in range(batch)], kv,
                                          head_fp32=True)[:, -1].float())
    # two-layer model, eight steps: bf16 drift stays a small multiple of one rounding
    diff = (torch.stack(logits_gpu) - torch.stack(logits_cpu)).abs()
    assert diff.max().item() <= 3 * LOGIT_TOLERANCE and diff.mean().item() <= LOGIT_TOLERANCE / 2, diff.max().item()
    assert (torch.stack(logits_gpu).argmax(-1) == torch.stack(logits_cpu).argmax(-1)).float().mean().item() >= 0.9
    run.close()


def test_llama_3_2_1b_shape_32_greedy_steps(plan_dir):
    """Benchmark configuration 1: batch 1, prompt 128, 32 greedy steps, paged KV block 16."""
    record = torch.load(GOLDEN / "llama_3_2_1b.pt")
    config, prompt, new_tokens = record["config"], record["prompt"], record["new_tokens"]
    capacity = 160
    weights = bf16_weights(config)
    table = shuffled_block_table(1, capacity // 16, 16, seed=1)
    run = GpuRun(config, weights, 1, capacity, plan_dir, kv_layout="paged", block_table=table, num_blocks=16)
    tokens, logits = run.greedy(prompt, new_tokens)
    stats = assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, "llama_3_2_1b")
    # free-running tokens against the reference module's own fp32 run on the same bf16-rounded weights:
    # identical at least up to the first step whose top-2 margin is below the drift of a bf16 forward
    golden = record["fp32_bf16w"]
    same = 0
    while same < new_tokens and int(tokens[0, same]) == int(golden["tokens"][0, same]):
        same += 1
    margin = golden["top_values"][..., 0] - golden["top_values"][..., 1]
    first_close = next((i for i in range(new_tokens) if float(margin[i, 0]) <= 2 * stats[2]), new_tokens)
    assert same >= first_close, (same, first_close)
    print(f"llama_3_2_1b: |gpu-fp32| max {stats[0]:.4f} mean {stats[1]:.4f}; reference bf16 forward |bf16-fp32| max "
          f"{stats[2]:.4f} mean {stats[3]:.4f}; free-running tokens identical to the fp32 reference for {same}/{new_tokens}")
    run.close()


def test_abi_refuses_misuse(plan_dir):
    config = synthetic.TINY
    run = GpuRun(config, bf16_weights(config), 1, 32, plan_dir)
    run.plan.set_steps([0, 1, 2])
    assert run.plan.library.lib.tm_plan_launch(run.plan.handle, 0, 2, 5, run.stream) == -2
    assert run.plan.library.lib.tm_plan_launch(run.plan.handle, 3, 2, 0, run.stream) == -2
    assert run.plan.library.lib.tm_plan_launch(run.plan.handle, 0, 4, 0, run.stream) == -3
    with pytest.raises(ValueError):
        run.plan.set_steps([40])
    run.plan.launch(0, 2, run.stream)
    run.check_alive()
    assert run.plan.iteration[2] == 1
    run.close()


def test_bounded_wait_gives_up_and_returns(plan_dir):
    """A waiter whose producer never arrives must end by itself with a status
    record; the context stays usable and a normal launch still works after it."""
    config = synthetic.TINY
    run = GpuRun(config, bf16_weights(config), 1, 32, plan_dir)
    assert run.plan.watchdog_probe(withhold=False, limit_us=200000) is False
    assert run.plan.watchdog_probe(withhold=True, limit_us=2000) is True
    run.plan.set_steps([0])
    run.state.tokens[:, 0] = 5
    run.plan.launch(0, 2, run.stream)
    run.check_alive()
    run.close()


def test_reduction_padded_to_whole_pages(plan_dir):
    """A reduction length that is not a multiple of the 2048-column page (down-proj over
    1536 columns): the weights' pad columns are zero and the staged rows' too."""
    config = dict(synthetic.TINY, intermediate_size=1536)
    batch, prompt_len, new_tokens, capacity = 2, 11, 4, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=5)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, "padded reduction")
    run.close()


def test_eight_query_heads_per_kv_head(plan_dir):
    """The 70B-shaped grouping: 8 query heads share a KV head (all 8 rows of the attention A operand)."""
    config = synthetic.TINY_GQ8
    batch, prompt_len, new_tokens, capacity = 3, 23, 5, 48
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=8)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, "8 query heads per KV head")
    run.close()


def test_wide_batch_takes_the_down_reduction_in_parts(plan_dir):
    """Batch 8 with a down reduction of four pages: its rows do not fit beside the ring at once,
    so the stage runs as two parts with fp32 running sums in between (and the RMSNorm stages
    re-read their rows instead of parking them)."""
    config = dict(synthetic.TINY, intermediate_size=8192)
    batch, prompt_len, new_tokens, capacity = 8, 9, 4, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=6)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, new_tokens)
    assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits, capacity, "split down, batch 8")
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()


def test_generation_up_to_the_last_position_of_the_cache(plan_dir):
    """The last decode step runs position capacity - 1: its token has no slot in the token
    state and must not be written anywhere; everything before it matches the oracle."""
    config = synthetic.TINY_D128
    batch, prompt_len, capacity = 2, 20, 32
    steps = capacity - prompt_len + 1               # the last one decodes position capacity - 1
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=12)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, logits = run.greedy(prompt, steps)      # tokens: the capacity - prompt_len that fit
    assert tokens.shape == (batch, capacity - prompt_len) and logits.shape[0] == steps
    assert_as_accurate_as_reference_bf16(config, weights, prompt, tokens, logits[:tokens.shape[1]], capacity, "full cache")
    state = run.state.tokens.cpu()
    assert torch.equal(state[:, :prompt_len], prompt) and torch.equal(state[:, prompt_len:], tokens)
    looped, _ = run.greedy(prompt, steps, stepwise=False)
    assert torch.equal(looped, tokens)
    run.close()


def test_serving_engine_generates_the_tokens_of_the_stepwise_run(plan_dir):
    """The reference-facing driver class (ServingEngine.generate) in each of its launch
    schedules -- one persistent launch for all decode steps, chunks of two steps, one launch
    per step, mode L1 -- against the step-by-step run of the same plan."""
    from tilemega_b200.planbuild import emit_plan
    from tilemega_b200.serving.engine import ServingEngine
    from tilemega_b200.serving.weights import TensorCheckpoint

    config = synthetic.TINY
    batch, prompt_len, new_tokens, capacity = 2, 7, 6, 32
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    run = GpuRun(config, weights, batch, capacity, plan_dir)
    tokens, _ = run.greedy(prompt, new_tokens)
    run.close()
    so = emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity)
    checkpoint = TensorCheckpoint(weights, config["tie_word_embeddings"])
    for options in ({}, {"decode_chunk": 2}, {"decode_loop": False}, {"mode": "L1"}):
        with ServingEngine(checkpoint, config, so, batch, prompt_len=prompt_len, max_new_tokens=new_tokens,
                           **options) as engine:
            result = engine.generate(prompt)
            assert torch.equal(result.tokens, tokens), options
            assert result.decode_loop_used == options.get("decode_loop", True)
            assert len(result.step_ms) == new_tokens and result.step_ns_read and result.ttft_ms > 0
            assert all(ms > 0 for ms in result.step_ms)
            shorter = engine.generate(prompt, 3)     # the same engine again, fewer tokens
            assert torch.equal(shorter.tokens, tokens[:, :3])
            with pytest.raises(ValueError):
                engine.generate(prompt[:, :3])
            with pytest.raises(ValueError):
                engine.generate(prompt, new_tokens + 1)
    with pytest.raises(ValueError):
        ServingEngine(checkpoint, config, so, batch, prompt_len=prompt_len, max_new_tokens=capacity)


def test_a_fired_wait_blocks_launches_until_cleared(plan_dir):
    """Status -4: after a bounded wait gave up and tm_plan_watchdog reported it, the plan
    refuses launches until tm_plan_clear_watchdog (the record makes every other wait fall through)."""
    config = dict(synthetic.TINY, num_hidden_layers=1)
    run = GpuRun(config, bf16_weights(config), 1, 32, plan_dir)
    run.plan.set_steps([0, 1])
    run.state.tokens[:, 0] = 3
    # the probe leaves a clean plan behind: it clears the record it provoked
    assert run.plan.watchdog_probe(withhold=True, limit_us=2000)
    run.plan.launch(0, 2, run.stream)
    run.check_alive()
    # withhold = 2 leaves the record standing, as a real abandoned launch does
    assert run.lib.lib.tm_plan_watchdog_probe(run.plan.handle, 2, 2000, run.stream) == 1
    record = run.plan.watchdog()
    assert record is not None and record["fired"] == 1 and record["site"] == 5
    with pytest.raises(RuntimeError, match=r"\(-4\)"):
        run.plan.launch(1, 2, run.stream)
    run.plan.clear_watchdog()
    assert run.plan.watchdog() is None
    run.plan.launch(1, 2, run.stream)
    run.check_alive()
    run.close()


@pytest.mark.parametrize("rows,cols,tile_n,tile_k", [(64, 4096, 8, 2048), (24, 1536, 8, 2048), (256, 256, 128, 128),
                                                     (1000, 1096, 128, 128), (6144, 4096, 8, 2048)])
def test_pack_kernel_writes_the_tile_pages_layout(rows, cols, tile_n, tile_k):
    """tm_pack_tile_pages against the indexing definition of the recipe
    (python/tilemega/serving/weights.py:204-242 of the reference), bit for bit, ragged edges included."""
    from tilemega_b200.serving.weights import tile_pages, tile_pages_by_indexing

    generator = torch.Generator().manual_seed(5)
    weight = torch.randn(rows, cols, generator=generator).to(torch.bfloat16)
    expect = tile_pages_by_indexing(weight, tile_n, tile_k)
    got = tile_pages(weight.cuda(), tile_n, tile_k)
    assert torch.equal(got.cpu(), expect)
    # a view whose rows are further apart than their length (a column shard of a larger matrix)
    wide = torch.randn(rows, cols + 64, generator=generator).to(torch.bfloat16)
    got = tile_pages(wide.cuda()[:, :cols], tile_n, tile_k)
    assert torch.equal(got.cpu(), tile_pages_by_indexing(wide[:, :cols].contiguous(), tile_n, tile_k))
