"""Chunked prefill on the GPU: prompts run through a dense-batch plan whose rows are consecutive
positions (tcgen05 GEMM stages, every row's key and value appended behind a grid barrier before any
row attends), checked against the oracle's prefill forward -- the reference module's causal forward
over the whole prompt (python/tilemega/serving/export.py:134-172), which the fixtures under
tests/golden pin -- at every position; then decoding continues from the prefilled pool."""
import pytest
import torch

from oracle.decoder_oracle import OracleDecoder, PagedKV
from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.continuous import ContinuousEngine, Request
from tilemega_b200.serving.prefill import ChunkedPrefill
from tilemega_b200.serving.state import kv_row_swizzle
from tilemega_b200.serving.weights import TensorCheckpoint

from harness import bf16_ulp, bf16_weights

pytestmark = pytest.mark.gpu
LOGIT_TOLERANCE = 2e-2


def oracle_prefill(config, weights, prompt, capacity, dtype):
    decoder = OracleDecoder(config, weights, dtype, capacity)
    kv = PagedKV(config, 1, capacity, dtype)
    logits = decoder.forward(torch.tensor([prompt], dtype=torch.int32), [0], kv, head_fp32=True)[0].float()
    return logits, kv


@pytest.mark.parametrize("base,rows,lengths", [("TINY_D128", 16, [37, 20, 1]), ("TINY_GQ8", 32, [70])])
def test_chunked_prefill_matches_the_oracle_at_every_position(base, rows, lengths, plan_dir):
    config = getattr(synthetic, base)
    capacity, num_blocks = 96, 40
    weights = bf16_weights(config)
    prompts = [synthetic.seeded_tokens(1, length, config["vocab_size"], seed=30 + i)[0].tolist()
               for i, length in enumerate(lengths)]
    so = emit_plan(config, plan_dir, batch_lo=rows, batch_hi=rows, capacity=capacity, kv_layout="paged",
                   num_blocks=num_blocks, chunk_rows=True)
    layers, hkv, dim = config["num_hidden_layers"], config["num_key_value_heads"], config["head_dim"]
    pool = torch.zeros((layers, 2, num_blocks, hkv, 16, dim), dtype=torch.bfloat16, device="cuda:0")
    # blocks handed out in a scattered order, block 0 left to the pad rows
    order = (torch.randperm(num_blocks - 1, generator=torch.Generator().manual_seed(4)) + 1).tolist()
    blocks, taken = [], 0
    for length in lengths:
        need = -(-(length + 1) // 16)
        blocks.append(order[taken:taken + need])
        taken += need
    checkpoint = TensorCheckpoint(weights, config.get("tie_word_embeddings", False))
    with ChunkedPrefill(checkpoint, config, so, rows, pool) as prefill:
        results = prefill.run(prompts, blocks, want_logits=True)
        assert prefill.chunks_run == -(-sum(lengths) // rows)
    cache = kv_row_swizzle(pool.cpu())          # [L][2][blocks][Hkv][16][D], logical column order
    for prompt, owned, result in zip(prompts, blocks, results):
        exact, _ = oracle_prefill(config, weights, prompt, capacity, torch.float32)
        module, kv = oracle_prefill(config, weights, prompt, capacity, torch.bfloat16)
        ours, theirs = (result.logits - exact).abs(), (module - exact).abs()
        bound = max(LOGIT_TOLERANCE, 1.25 * theirs.max().item())
        assert ours.max().item() <= bound, (len(prompt), ours.max().item(), theirs.max().item())
        assert ours.mean().item() <= max(1.25 * theirs.mean().item(), LOGIT_TOLERANCE / 4)
        # the token after the prompt: the fp32 forward's choice wherever that is not a near tie
        top2 = exact[-1].topk(2).values
        if (top2[0] - top2[1]).item() > 2 * bound:
            assert result.first_token == int(exact[-1].argmax())
        assert exact[-1, result.first_token].item() >= top2[0].item() - 2 * bound
        # the cache rows the prefill wrote: the module's own keys and values, up to the bf16 drift of a two-layer model
        length = len(prompt)
        positions = torch.arange(length)
        # (index tensors on two separated axes move to the front: [len][L][2][Hkv][D] -> [L][2][len][Hkv][D])
        mine = cache[:, :, torch.tensor(owned)[positions // 16], :, positions % 16].permute(1, 2, 0, 3, 4)
        reference = kv.pool[:, :, kv.table[0, positions // 16].long(), :, positions % 16].permute(1, 2, 0, 3, 4)
        first_layer = (mine[0].float() - reference[0].float()).abs()
        assert (first_layer <= 2 * bf16_ulp(reference[0].float()) + 1e-6).float().mean().item() >= 0.999
        assert (mine.float() - reference.float()).abs().max().item() <= 0.05 * reference.float().abs().max().item()


def test_continuous_engine_decodes_on_from_a_prefilled_pool(plan_dir):
    config = synthetic.TINY_D128
    capacity, slots, num_blocks, rows = 64, 2, 9, 16
    weights = bf16_weights(config)
    shapes = [(21, 5), (3, 6), (40, 4), (17, 1)]
    requests = [Request(i, synthetic.seeded_tokens(1, length, config["vocab_size"], seed=50 + i)[0].tolist(), new)
                for i, (length, new) in enumerate(shapes)]
    decode_so = emit_plan(config, plan_dir, batch_lo=slots, batch_hi=slots, capacity=capacity, kv_layout="paged",
                          num_blocks=num_blocks)
    prefill_so = emit_plan(config, plan_dir, batch_lo=rows, batch_hi=rows, capacity=capacity, kv_layout="paged",
                           num_blocks=num_blocks, chunk_rows=True, write_logits=False)
    checkpoint = TensorCheckpoint(weights, config.get("tie_word_embeddings", False))
    with ContinuousEngine(checkpoint, config, decode_so, slots, prefill_so=prefill_so, prefill_rows=rows) as engine:
        for request in requests:
            engine.submit(request)
        finished = engine.run_until_done()
        # the prompts never went through the decode plan: steps = generated tokens after the first, shared by two slots
        assert engine.steps_run <= sum(new - 1 for _, new in shapes)
        assert len(engine.scheduler.pool.free) == num_blocks - 1
    assert sorted(request.id for request in finished) == [0, 1, 2, 3]
    decoder = OracleDecoder(config, weights, torch.float32, capacity)
    for request in finished:
        assert len(request.generated) == shapes[request.id][1]
        # teacher-forced on what the engine generated, every token must be the fp32 forward's choice or a near tie of it
        history = torch.tensor([request.prompt + request.generated[:-1]], dtype=torch.int32)
        kv = PagedKV(config, 1, capacity, torch.float32)
        logits = decoder.forward(history, [0], kv, head_fp32=True)[0].float()[len(request.prompt) - 1:]
        chosen = logits[torch.arange(len(request.generated)), torch.tensor(request.generated)]
        assert (chosen >= logits.max(dim=-1).values - 4 * LOGIT_TOLERANCE).all(), (request.id, request.generated)


def test_llama_8b_shape_prefill_is_chunk_size_invariant_and_agrees_with_the_decode_path(plan_dir):
    """At the benchmark's widths (hidden 4096, FFN 14336, vocabulary 128256; 8 of the 32 layers keep it
    quick), where the CPU oracle is too slow: properties. (1) Chunks of 16 and of 64 positions write the
    same cache bit for bit and sample the same token -- a row's sums do not depend on how many other
    rows share its tile; (2) a rerun is bit-identical; (3) the decode plan teacher-forced over the same
    prompt (GEMV path, other summation order) writes a cache that agrees to bf16 drift and samples the
    same token or a near tie of it."""
    from tilemega_b200.serving.plan import PlanLibrary
    from tilemega_b200.serving.state import allocate_state
    from tilemega_b200.serving.weights import load_weights
    config = dict(synthetic.LLAMA_3_1_8B, num_hidden_layers=8)
    length, capacity, num_blocks = 150, 192, 16
    device = torch.device("cuda", 0)
    checkpoint = synthetic.LazySeededCheckpoint(config, seed=0, device=device)
    prompt = synthetic.seeded_tokens(1, length, config["vocab_size"], seed=8)[0].tolist()
    blocks = [5, 2, 9, 1, 7, 3, 11, 4, 6, 8]            # ten scattered blocks: 160 positions
    layers, hkv, dim = config["num_hidden_layers"], config["num_key_value_heads"], config["head_dim"]
    pools, tokens = {}, {}
    for run, rows in enumerate((16, 64, 64)):
        so = emit_plan(config, plan_dir, batch_lo=rows, batch_hi=rows, capacity=capacity, kv_layout="paged",
                       num_blocks=num_blocks, chunk_rows=True, write_logits=False)
        pool = torch.zeros((layers, 2, num_blocks, hkv, 16, dim), dtype=torch.bfloat16, device=device)
        with ChunkedPrefill(checkpoint, config, so, rows, pool) as prefill:
            result = prefill.run([prompt], [blocks])[0]
        pools[run], tokens[run] = pool[:, :, blocks].clone(), result.first_token
        del pool
        torch.cuda.empty_cache()
    assert torch.equal(pools[0], pools[1]) and tokens[0] == tokens[1], "chunks of 16 and of 64 positions disagree"
    assert torch.equal(pools[1], pools[2]) and tokens[1] == tokens[2], "a rerun is not bit-identical"
    # the same prompt teacher-forced through the batch-1 decode plan
    so = emit_plan(config, plan_dir, batch_lo=1, batch_hi=1, capacity=capacity, kv_layout="paged", num_blocks=num_blocks)
    lib = PlanLibrary(so)
    weights = load_weights(checkpoint, lib, device=device)
    table = torch.zeros((1, capacity // 16), dtype=torch.int32)
    table[0, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
    table[0, len(blocks):] = torch.tensor([12, 13], dtype=torch.int32)
    state = allocate_state(config, 1, lib, device, block_table=table)
    plan = lib.create(1, {name: t.data_ptr() for name, t in weights.items()} | state.pointers, 0)
    state.tokens[0, :length] = torch.tensor(prompt, dtype=torch.int32, device=device)
    plan.set_prompt_len(length)
    plan.set_steps(list(range(length)))
    plan.launch_steps(0, length, 2, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert plan.watchdog() is None
    decoded = state.kv_storage[:, :, blocks].float()
    prefilled = pools[1].float()
    used = slice(0, length)                                    # positions written: rows of the ten blocks in order
    a = decoded.permute(0, 1, 3, 2, 4, 5).reshape(layers, 2, hkv, -1, dim)[:, :, :, used]
    b = prefilled.permute(0, 1, 3, 2, 4, 5).reshape(layers, 2, hkv, -1, dim)[:, :, :, used]
    assert torch.equal(a[0], b[0]) or ((a[0] - b[0]).abs() <= 2 * bf16_ulp(b[0]) + 1e-6).float().mean().item() >= 0.999
    assert (a - b).abs().mean().item() <= 0.01 * b.abs().max().item()
    assert (a - b).abs().max().item() <= 0.10 * b.abs().max().item()
    host = torch.empty(config["vocab_size"], dtype=torch.float32)
    plan.read_buffer("serving.logits", host.data_ptr(), host.numel() * 4)
    best = host.max().item()
    assert host[int(state.tokens[0, length])].item() >= best - 4 * LOGIT_TOLERANCE      # the decode path's own choice
    assert host[tokens[1]].item() >= best - 4 * LOGIT_TOLERANCE                         # the prefill's choice
    plan.close()


@pytest.mark.parametrize("kv_layout", ["contiguous", "paged"])
def test_prefill_plan_behind_the_abi_feeds_the_decode_plan(kv_layout, plan_dir):
    """The reference driver's flow with a prefill binary (python/tilemega/serving/engine.py:41-57,89-92,
    144-146): a phase-0 plan whose ONE step runs the whole batch of prompts over the state the decode plan
    shares, then the decode plan's steps behind the prompt. Checked against the engine's prompt mode (the
    prompt teacher-forced through the decode plan) and, teacher-forced, against the fp32 forward."""
    from tilemega_b200.serving.engine import ServingEngine
    from tilemega_b200.serving.state import shuffled_block_table
    config = synthetic.TINY_D128
    batch, prompt_len, new_tokens, capacity = 3, 37, 6, 64      # 111 (sequence, position) rows: two kernel steps
    weights = bf16_weights(config)
    checkpoint = TensorCheckpoint(weights, config.get("tie_word_embeddings", False))
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=12)
    num_blocks = batch * capacity // 16 + 3
    layout = dict(kv_layout=kv_layout, num_blocks=num_blocks if kv_layout == "paged" else 0)
    table = shuffled_block_table(batch, capacity // 16, num_blocks, seed=2) if kv_layout == "paged" else None
    decode_so = emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity, **layout)
    prefill_so = emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity, phase="prefill",
                           seq=prompt_len, **layout)
    with ServingEngine(checkpoint, config, decode_so, batch, prompt_len, new_tokens, block_table=table) as engine:
        by_decode = engine.generate(prompt).tokens.clone()
        cache_by_decode = engine.state.kv_storage.clone()
    with ServingEngine(checkpoint, config, decode_so, batch, prompt_len, new_tokens, block_table=table,
                       prefill_so=prefill_so) as engine:
        result = engine.generate(prompt)
        tokens = result.tokens.clone()
        again = engine.generate(prompt).tokens.clone()          # a second request through the same plans
        cache = engine.state.kv_storage.clone()
    assert torch.equal(again, tokens)
    # the two paths differ in the summation order of their GEMMs only: bf16 drift of a two-layer model
    drift = (cache.float() - cache_by_decode.float()).abs()
    assert drift.max().item() <= 0.05 * cache_by_decode.float().abs().max().item()
    decoder = OracleDecoder(config, weights, torch.float32, capacity)
    for b in range(batch):
        history = torch.cat((prompt[b], tokens[b, :-1].to(prompt.dtype))).view(1, -1).to(torch.int32)
        kv = PagedKV(config, 1, capacity, torch.float32)
        logits = decoder.forward(history, [0], kv, head_fp32=True)[0].float()[prompt_len - 1:]
        chosen = logits[torch.arange(new_tokens), tokens[b].long()]
        assert (chosen >= logits.max(dim=-1).values - 4 * LOGIT_TOLERANCE).all(), (b, tokens[b].tolist())
        decided = (logits.topk(2).values[:, 0] - logits.topk(2).values[:, 1]) > 4 * LOGIT_TOLERANCE
        if decided.all():
            assert torch.equal(tokens[b], by_decode[b])


def test_prefill_plan_continues_behind_cached_history(plan_dir):
    """serving.context_base shifts a prefill plan's positions: a prompt prefilled in two pieces (32 positions,
    then 21 more behind them) must leave the cache and sample the token of the same prompt prefilled at once,
    bit for bit (both run the same rows through the same arithmetic, only cut into kernel steps differently)."""
    from tilemega_b200.serving.plan import L2, PlanLibrary
    from tilemega_b200.serving.state import allocate_state, shuffled_block_table
    from tilemega_b200.serving.weights import load_weights
    config = synthetic.TINY_D128
    capacity, num_blocks, first, second = 96, 9, 32, 21
    weights = bf16_weights(config)
    checkpoint = TensorCheckpoint(weights, config.get("tie_word_embeddings", False))
    prompt = synthetic.seeded_tokens(1, first + second, config["vocab_size"], seed=21).to(torch.int32)
    layout = dict(batch_lo=1, batch_hi=1, capacity=capacity, kv_layout="paged", num_blocks=num_blocks)
    decode_lib = PlanLibrary(emit_plan(config, plan_dir, **layout))
    table = shuffled_block_table(1, capacity // 16, num_blocks, seed=5)
    stream = torch.cuda.current_stream().cuda_stream

    def prefill(pieces):
        state = allocate_state(config, 1, decode_lib, "cuda:0", block_table=table)
        done = 0
        for length in pieces:
            # (a piece writes the token it samples behind its last position; the driver knows the prompt goes on)
            state.tokens[0, :first + second] = prompt[0].cuda()
            lib = PlanLibrary(emit_plan(config, plan_dir, phase="prefill", seq=length, **layout))
            packed = load_weights(checkpoint, lib, device="cuda:0")
            plan = lib.create(1, {name: t.data_ptr() for name, t in packed.items()} | state.pointers, 0)
            state.context_base.fill_(done)
            plan.set_steps([0])
            plan.launch(0, L2, stream)
            torch.cuda.synchronize()
            assert plan.watchdog() is None
            plan.close()
            done += length
        return state.kv_storage.clone(), state.tokens[0, :first + second + 1].cpu()

    cache_once, tokens_once = prefill([first + second])
    cache_twice, tokens_twice = prefill([first, second])
    assert torch.equal(tokens_twice[:first + second], prompt[0])          # the prompt itself is never overwritten
    assert torch.equal(cache_twice, cache_once) and torch.equal(tokens_twice, tokens_once)
