"""Shared helpers for the GPU parity tests: drive the CUDA path through the C ABI
(via the ctypes mirror of the reference driver) and collect tokens and logits."""
from __future__ import annotations

import torch

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.plan import PlanLibrary
from tilemega_b200.serving.state import allocate_state
from tilemega_b200.serving.weights import TensorCheckpoint, load_weights


class GpuRun:
    """One plan + state + weights on cuda:0."""

    def __init__(self, config, weights_cpu, batch, capacity, plan_dir, kv_layout="contiguous",
                 block_table=None, context_base=None, num_blocks=0, geometry=None, slots=0, grid=0, weights="bf16",
                 attn_min_slots=None):
        self.config = config
        self.batch = batch
        self.capacity = capacity
        so = emit_plan(config, plan_dir, batch_lo=batch, batch_hi=batch, capacity=capacity, kv_layout=kv_layout,
                       num_blocks=num_blocks, geometry=geometry, slots=slots, grid=grid, weights=weights,
                       attn_min_slots=attn_min_slots)
        self.lib = PlanLibrary(so)
        checkpoint = TensorCheckpoint(weights_cpu, config.get("tie_word_embeddings", False))
        self.weights = load_weights(checkpoint, self.lib, device="cuda:0")
        self.state = allocate_state(config, batch, self.lib, "cuda:0", block_table, context_base)
        pointers = {name: tensor.data_ptr() for name, tensor in self.weights.items()}
        pointers.update(self.state.pointers)
        self.plan = self.lib.create(batch, pointers, 0)
        self.stream = torch.cuda.current_stream().cuda_stream

    def read(self, name, dtype=torch.bfloat16):
        buffer = self.lib.buffers[self.lib.index[name]]
        count = buffer.elements_constant + self.batch * buffer.elements_per_batch
        host = torch.empty(count, dtype=dtype)
        torch.cuda.synchronize()
        self.plan.read_buffer(name, host.data_ptr(), host.numel() * host.element_size())
        return host

    def check_alive(self):
        torch.cuda.synchronize()
        fired = self.plan.watchdog()
        assert fired is None, f"a bounded device wait gave up: {fired}"

    def greedy(self, prompt, new_tokens, stepwise=True, mode=2):
        """Teacher-forced prompt, then greedy decode. Returns (tokens [B][new] int32 cpu,
        logits [new][B][V] fp32 cpu or None when not stepwise)."""
        batch, length = prompt.shape
        vocab = self.config["vocab_size"]
        self.state.tokens.zero_()
        self.state.tokens[:, :length].copy_(prompt)
        self.plan.set_prompt_len(length)
        self.plan.set_steps(list(range(length + new_tokens - 1)))
        self.plan.launch_steps(0, length, mode, self.stream)
        history = None
        if stepwise:
            history = [self.read("serving.logits", torch.float32).reshape(batch, vocab)]
            for step in range(new_tokens - 1):
                self.plan.launch(length + step, mode, self.stream)
                history.append(self.read("serving.logits", torch.float32).reshape(batch, vocab))
            history = torch.stack(history)
        elif new_tokens > 1:
            self.plan.launch_steps(length, new_tokens - 1, mode, self.stream)
        self.check_alive()
        tokens = self.state.tokens[:, length:length + new_tokens].cpu()
        return tokens, history

    def close(self):
        self.plan.close()


def bf16_weights(config, seed=0):
    return {name: tensor.to(torch.bfloat16) for name, tensor in synthetic.seeded_weights(config, seed).items()}


def bf16_ulp(values):
    """Spacing of bf16 numbers at the magnitude of `values` (8 significant bits)."""
    return torch.exp2(torch.floor(torch.log2(values.abs().clamp_min(1e-30))) - 7)


def assert_parity(gpu_tokens, gpu_logits, oracle_logits, tolerance, label=""):
    """GPU logits vs oracle logits computed on the SAME token history (teacher
    forced on the GPU's tokens), both before the final rounding to bf16: max-abs
    within `tolerance`, and the greedy token identical wherever the oracle's
    top-2 margin exceeds twice the tolerance."""
    diff = (gpu_logits - oracle_logits).abs().max().item()
    assert diff <= tolerance, f"{label}: logits differ by {diff} > {tolerance}"
    top2 = oracle_logits.topk(2, dim=-1).values
    margin = top2[..., 0] - top2[..., 1]
    oracle_tokens = oracle_logits.argmax(-1).transpose(0, 1).to(torch.int32)
    decided = (margin > 2 * tolerance).transpose(0, 1)
    assert torch.equal(gpu_tokens[decided], oracle_tokens[decided]), f"{label}: greedy token differs at a decided step"
    gpu_choice = torch.gather(oracle_logits, 2, gpu_tokens.transpose(0, 1).long().unsqueeze(-1)).squeeze(-1)
    assert ((top2[..., 0] - gpu_choice) <= 2 * tolerance).all(), f"{label}: GPU token is not a near-tie of the oracle's"
    return diff, int(decided.sum()), int(decided.numel())
