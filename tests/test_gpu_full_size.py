"""Size-independent properties at the benchmark's full shape (Llama-3.1-8B-shaped,
32 layers, vocab 128256, bf16): the CPU oracle cannot run this in test time, so the
checks are properties that hold bit for bit whatever the weights are."""
import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.plan import PlanLibrary
from tilemega_b200.serving.state import allocate_state, shuffled_block_table
from tilemega_b200.serving.weights import TensorCheckpoint, load_weights

pytestmark = pytest.mark.gpu


def make_plan(lib, config, weights, batch, table):
    state = allocate_state(config, batch, lib, "cuda:0", block_table=table)
    pointers = {name: tensor.data_ptr() for name, tensor in weights.items()}
    pointers.update(state.pointers)
    return lib.create(batch, pointers, 0), state


def logits_of(lib, plan, batch, vocab):
    host = torch.empty(batch * vocab, dtype=torch.float32)
    torch.cuda.synchronize()
    plan.read_buffer("serving.logits", host.data_ptr(), host.numel() * 4)
    return host.reshape(batch, vocab)


def test_llama_8b_shape_block_tables_launch_splits_and_reruns_are_bit_identical(plan_dir):
    config = synthetic.LLAMA_3_1_8B
    batch, prompt_len, new_tokens = 2, 40, 6
    capacity = 64
    device = torch.device("cuda", 0)
    raw = synthetic.seeded_weights(config, seed=0, dtype=torch.bfloat16, device=device)
    contiguous = PlanLibrary(emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity))
    weights = load_weights(TensorCheckpoint(raw, False), contiguous, device=device)
    keep = {tensor.data_ptr() for tensor in weights.values()}
    raw = {name: tensor for name, tensor in raw.items() if tensor.data_ptr() in keep}
    torch.cuda.empty_cache()
    num_blocks = 3 * batch * capacity // 16
    paged = PlanLibrary(emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity,
                                  kv_layout="paged", num_blocks=num_blocks))
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    stream = torch.cuda.current_stream().cuda_stream
    steps = list(range(prompt_len + new_tokens - 1))

    def run(lib, table, split):
        plan, state = make_plan(lib, config, weights, batch, table)
        state.tokens[:, :prompt_len].copy_(prompt)
        plan.set_prompt_len(prompt_len)
        plan.set_steps(steps)
        if split:   # prompt in one launch, then one launch per decode step
            plan.launch_steps(0, prompt_len, 2, stream)
            for step in range(prompt_len, len(steps)):
                plan.launch(step, 2, stream)
        else:       # everything in a single persistent launch
            plan.launch_steps(0, len(steps), 2, stream)
        torch.cuda.synchronize()
        assert plan.watchdog() is None
        tokens = state.tokens[:, prompt_len:prompt_len + new_tokens].cpu()
        logits = logits_of(lib, plan, batch, config["vocab_size"])
        kv = state.kv_storage.cpu()
        plan.close()
        return tokens, logits, kv

    base_tokens, base_logits, base_kv = run(contiguous, None, split=False)
    assert int(base_tokens.min()) >= 0 and int(base_tokens.max()) < config["vocab_size"]
    assert torch.isfinite(base_logits).all()
    # 1. a second run reproduces every bit (tasks are claimed dynamically; results must not depend on who ran them)
    again_tokens, again_logits, again_kv = run(contiguous, None, split=False)
    assert torch.equal(again_tokens, base_tokens) and torch.equal(again_logits, base_logits)
    assert torch.equal(again_kv, base_kv)
    # 2. one launch per step == one launch for all steps
    split_tokens, split_logits, split_kv = run(contiguous, None, split=True)
    assert torch.equal(split_tokens, base_tokens) and torch.equal(split_logits, base_logits)
    assert torch.equal(split_kv, base_kv)
    # 3. a shuffled block table over a larger pool == the contiguous cache, row for row
    table = shuffled_block_table(batch, capacity // 16, num_blocks, seed=5)
    paged_tokens, paged_logits, pool = run(paged, table, split=False)
    assert torch.equal(paged_tokens, base_tokens) and torch.equal(paged_logits, base_logits)
    length = prompt_len + new_tokens - 1
    positions = torch.arange(length)
    for b in range(batch):
        rows = pool.permute(2, 4, 0, 1, 3, 5)[table[b, positions // 16].long(), positions % 16]   # [len][L][2][Hkv][D]
        assert torch.equal(rows.permute(1, 2, 3, 0, 4), base_kv[:, :, b, :, :length])
    # 4. the argmax written to the token state is the argmax of the bf16-rounded logits (ties to the smaller index)
    rounded = base_logits.to(torch.bfloat16).float()
    expect = torch.stack([torch.nonzero(row == row.max())[0, 0] for row in rounded]).to(torch.int32)
    assert torch.equal(base_tokens[:, -1], expect)
