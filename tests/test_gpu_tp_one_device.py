"""Tensor parallelism on ONE GPU: all ranks of a job as a single cooperative launch
(tm_plan_launch_steps_ranks), CTAs [0, g) running rank 0's plan, the next g rank 1's and so on.

The ranks' kernels wait for one another's all-reduce packets, so they must run at the same
time; on one GPU only a single launch guarantees that (separate launches, streams or
processes do not). The exchange code is the multi-GPU one unchanged: packets stored with
st.relaxed.sys into the peer's receive region (here a region in the same device's memory),
polled with ld.relaxed.sys, summed in ascending rank order; argmax winners exchanged the
same way. Checked against OracleDecoder(tp=T), whose per-rank partial sums are pinned bit for
bit by the reference's own rank modules (tests/golden/tiny_tp2.pt), with the yardstick of
tests/test_gpu_decode.py; the bit-for-bit rank-order sum is the rule the reference tests in
test/unit/sm90_dense_tp_test.cu:5-15.

The last cases run ONE layer at the 70B-shaped benchmark configuration's per-rank widths:
hidden 8192, 8 query heads per KV head, o / down reductions of 1024 / 3584 columns per rank
at 8 ranks (padded last pages) and 2048 / 7168 at 4 ranks.
"""
import pytest
import torch

from oracle.decoder_oracle import OracleDecoder, PagedKV
from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.plan import L1, PlanLibrary
from tilemega_b200.serving.state import allocate_state
from tilemega_b200.serving.weights import TensorCheckpoint, load_weights

from harness import assert_parity, bf16_weights

pytestmark = pytest.mark.gpu
LOGIT_TOLERANCE = 2e-2

# One layer with the 70B shape's hidden size, head grouping and FFN width; a smaller vocabulary keeps the
# CPU oracle quick (the head's row sharding does not depend on it).
WIDE_70B_LAYER = dict(synthetic.LLAMA_3_1_70B, num_hidden_layers=1, vocab_size=16384)


class RanksOnOneDevice:
    """T rank plans of one library on cuda:0, bound to one another's regions, launched together."""

    def __init__(self, config, weights_cpu, batch, capacity, plan_dir, ranks, weights="bf16"):
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        so = emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity, tp=ranks, grid=sms // ranks,
                       weights=weights)
        self.lib = PlanLibrary(so)
        self.ranks, self.batch, self.config = ranks, batch, config
        checkpoint = TensorCheckpoint(weights_cpu, config.get("tie_word_embeddings", False))
        self.weights, self.states, self.plans = [], [], []
        for rank in range(ranks):
            packed = load_weights(checkpoint, self.lib, device="cuda:0", tp=(rank, ranks))
            state = allocate_state(config, batch, self.lib, "cuda:0", tp=ranks)
            pointers = {name: tensor.data_ptr() for name, tensor in packed.items()} | state.pointers
            self.weights.append(packed)
            self.states.append(state)
            self.plans.append(self.lib.create(batch, pointers, 0))
        # every rank's receive region and exchange block: zeroed device memory, here all on one device
        self.regions = [torch.zeros(self.lib.tp_bytes(0) // 8, dtype=torch.int64, device="cuda:0") for _ in range(ranks)]
        self.blocks = [torch.zeros(self.lib.tp_bytes(1) // 8, dtype=torch.int64, device="cuda:0") for _ in range(ranks)]
        for rank, plan in enumerate(self.plans):
            plan.bind_tp(rank, [t.data_ptr() for t in self.regions], [t.data_ptr() for t in self.blocks])
        self.stream = torch.cuda.current_stream().cuda_stream

    def logits(self):
        """[B][V]: the ranks' row slices side by side."""
        rows = self.config["vocab_size"] // self.ranks
        torch.cuda.synchronize()
        parts = []
        for plan in self.plans:
            host = torch.empty(self.batch * rows, dtype=torch.float32)
            plan.read_buffer("serving.logits", host.data_ptr(), host.numel() * 4)
            parts.append(host.reshape(self.batch, rows))
        return torch.cat(parts, dim=-1)

    def greedy(self, prompt, new_tokens, stepwise=True):
        length = prompt.shape[1]
        for state, plan in zip(self.states, self.plans):
            state.tokens.zero_()
            state.tokens[:, :length].copy_(prompt)
            plan.set_prompt_len(length)
            plan.set_steps(list(range(length + new_tokens - 1)))
        self.lib.launch_steps_ranks(self.plans, 0, length, L1, self.stream)
        history = None
        if stepwise:
            history = [self.logits()]
            for step in range(new_tokens - 1):
                self.lib.launch_steps_ranks(self.plans, length + step, 1, L1, self.stream)
                history.append(self.logits())
            history = torch.stack(history)
        elif new_tokens > 1:
            self.lib.launch_steps_ranks(self.plans, length, new_tokens - 1, L1, self.stream)
        torch.cuda.synchronize()
        for rank, plan in enumerate(self.plans):
            fired = plan.watchdog()
            assert fired is None, f"rank {rank}: a bounded device wait gave up: {fired}"
        tokens = [state.tokens[:, length:length + new_tokens].cpu() for state in self.states]
        for rank in range(1, self.ranks):
            assert torch.equal(tokens[rank], tokens[0]), f"rank {rank} wrote tokens that differ from rank 0's"
        return tokens[0], history

    def close(self):
        for plan in self.plans:
            plan.close()


def forced_oracle(config, weights, prompt, forced, capacity, dtype, tp):
    decoder = OracleDecoder(config, weights, dtype, capacity, tp=tp)
    kv = PagedKV(config, prompt.shape[0], capacity, dtype)
    return decoder.greedy(prompt, forced.shape[1], kv, forced=forced, head_fp32=True)[1]


@pytest.mark.parametrize("name,config,ranks,batch,prompt_len,new_tokens,capacity", [
    ("tiny_d128 tp2", synthetic.TINY_D128, 2, 3, 13, 5, 32),      # o reduction of 1024 columns per rank: a padded page
    ("tiny_gq8 tp2", synthetic.TINY_GQ8, 2, 2, 21, 6, 64),        # 8 query heads per KV head, one KV head per rank
    ("tiny_d128 tp4", synthetic.TINY_D128, 4, 1, 17, 4, 48),      # one KV head per rank, 37 CTAs per rank
    ("70b-width layer tp8", WIDE_70B_LAYER, 8, 1, 9, 3, 32),      # per-rank reductions 1024 (o) and 3584 (down)
    ("70b-width layer tp4", WIDE_70B_LAYER, 4, 2, 9, 3, 32),      # per-rank reductions 2048 (o) and 7168 (down)
])
def test_ranks_on_one_device_match_tensor_parallel_oracle(name, config, ranks, batch, prompt_len, new_tokens, capacity,
                                                           plan_dir):
    weights = bf16_weights(config)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    run = RanksOnOneDevice(config, weights, batch, capacity, plan_dir, ranks)
    tokens, logits = run.greedy(prompt, new_tokens)
    run.close()
    # one launch for all steps of a phase must give the tokens of one launch per step
    run = RanksOnOneDevice(config, weights, batch, capacity, plan_dir, ranks)
    looped, _ = run.greedy(prompt, new_tokens, stepwise=False)
    run.close()
    assert torch.equal(looped, tokens), "one launch for all steps and one launch per step disagree"
    exact = forced_oracle(config, weights, prompt, tokens, capacity, torch.float32, ranks)
    module = forced_oracle(config, weights, prompt, tokens, capacity, torch.bfloat16, ranks)
    ours, theirs = (logits - exact).abs(), (module - exact).abs()
    assert ours.max().item() <= 1.25 * theirs.max().item(), (name, ours.max().item(), theirs.max().item())
    assert ours.mean().item() <= 1.25 * theirs.mean().item(), (name, ours.mean().item(), theirs.mean().item())
    assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), name)


def test_rank_group_launch_refuses_misuse(plan_dir):
    config = synthetic.TINY_D128
    run = RanksOnOneDevice(config, bf16_weights(config), 1, 32, plan_dir, 2)
    for plan in run.plans:
        plan.set_steps([0, 1])
    with pytest.raises(RuntimeError):   # ranks out of order
        run.lib.launch_steps_ranks(run.plans[::-1], 0, 1, L1, run.stream)
    with pytest.raises(RuntimeError):   # one plan is not a job
        run.lib.launch_steps_ranks(run.plans[:1], 0, 1, L1, run.stream)
    run.close()
