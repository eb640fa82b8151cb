"""Chunked prefill: a prompt runs through a dense-batch plan whose rows are consecutive positions.

The reference's native path has no prefill binary: its driver teacher-forces every prompt position
through the decode plan, one token per step (python/tilemega/serving/engine.py:38-41,144-148), and
its generic path lowers prefill to tiled GEMM tasks plus causal attention
(include/tilemega/Codegen/tasks/GemmStageTaskBody.h, FusedAttentionTaskBody.h:116-210). Here a
prompt is cut into chunks of up to `rows` positions (16, 32, 48 or 64) and every chunk is ONE step of
a dense-batch plan emitted with `chunk_rows=True`: row i of the batch is position p0 + i of the
sequence (`serving.context_base[i] = p0 + i`, every row's `serving.block_table` row names the
sequence's blocks), the weights stream once per chunk instead of once per token, the GEMM stages run
on tcgen05 tiles, and causality falls out of each row attending to positions <= its own -- the plan
appends all rows' keys and values behind a grid barrier before any row attends. Rows of several
sequences may share a chunk. The KV pool is the decode plan's own (`kv_storage`), so decoding goes
on from the prefilled cache without a copy.
"""
from __future__ import annotations

from dataclasses import dataclass

KV_BLOCK = 16


@dataclass
class PrefillResult:
    first_token: int        # the token sampled after the prompt's last position
    logits: object | None   # fp32 [prompt length][vocab], every position's logits (on request, plans that write logits)


def pack_rows(lengths: list[int], rows: int) -> list[list[tuple[int, int]]]:
    """Chunks of at most `rows` (sequence, position) pairs, sequences in order, positions ascending,
    so that a position's predecessors are in the same chunk or an earlier one."""
    if rows < 1:
        raise ValueError("rows must be positive")
    flat = [(index, position) for index, length in enumerate(lengths) for position in range(length)]
    return [flat[at:at + rows] for at in range(0, len(flat), rows)]


class ChunkedPrefill:
    """A `chunk_rows` dense-batch plan bound to a KV pool, driven chunk by chunk."""

    def __init__(self, checkpoint, config: dict, prefill_so, rows: int, kv_storage, device: int = 0, weights=None):
        import torch

        from .plan import L2, PlanLibrary
        from .state import allocate_state
        from .weights import load_weights
        if not torch.cuda.is_available():
            raise RuntimeError("ChunkedPrefill needs a CUDA device; there is no CPU path")
        self.torch = torch
        torch.cuda.set_device(device)
        self.library = PlanLibrary(prefill_so)
        if not self.library.manifest.get("chunk_rows"):
            raise ValueError("chunked prefill needs a plan emitted with chunk_rows=True")
        self.rows, self.mode = rows, L2
        self.capacity = self.library.info.capacity
        self.max_blocks = self.capacity // KV_BLOCK
        where = torch.device("cuda", device)
        self.weights = load_weights(checkpoint, self.library, device=where) if weights is None else weights
        table = torch.zeros((rows, self.max_blocks), dtype=torch.int32)          # every row on the scratch block 0
        self.state = allocate_state(config, rows, self.library, where, block_table=table, shared_blocks=True,
                                    kv_storage=kv_storage)
        bound = {name: tensor.data_ptr() for name, tensor in self.weights.items()} | self.state.pointers
        self.plan = self.library.create(rows, bound, device)
        self.plan.set_prompt_len(0)
        self.plan.set_steps([0])
        self.stream = torch.cuda.current_stream()
        self.vocab = int(config["vocab_size"])
        self.has_logits = "serving.logits" in self.library.index
        self.chunks_run = 0
        self.device_ms = 0.0    # kernel time of the chunks run so far (CUDA events around each launch)
        self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

    def run(self, prompts: list[list[int]], blocks: list[list[int]], want_logits: bool = False) -> list[PrefillResult]:
        """Prefill every prompt into its blocks of the pool. `blocks[s]` are sequence s's pool blocks in
        logical order (enough for its prompt; block 0 is the pad rows' scratch block and may not be used)."""
        torch = self.torch
        if len(prompts) != len(blocks) or not prompts:
            raise ValueError("one block list per prompt")
        rows_of = []
        for prompt, owned in zip(prompts, blocks):
            if not prompt or len(prompt) >= self.capacity:
                raise ValueError("a prompt needs 1 .. capacity - 1 tokens")
            if len(owned) > self.max_blocks or len(owned) * KV_BLOCK < len(prompt) or 0 in owned:
                raise ValueError("a sequence's blocks do not cover its prompt (or name the scratch block 0)")
            row = torch.zeros(self.max_blocks, dtype=torch.int32)
            row[:len(owned)] = torch.tensor(owned, dtype=torch.int32)
            rows_of.append(row)
        results: list[PrefillResult | None] = [None] * len(prompts)
        keep = want_logits and self.has_logits
        logits_of = [torch.empty((len(prompt), self.vocab), dtype=torch.float32) if keep else None for prompt in prompts]
        for chunk in pack_rows([len(prompt) for prompt in prompts], self.rows):
            table = torch.zeros((self.rows, self.max_blocks), dtype=torch.int32)
            base = torch.zeros(self.rows, dtype=torch.int32)
            ids = torch.zeros(self.rows, dtype=torch.int32)
            for row, (sequence, position) in enumerate(chunk):
                table[row], base[row], ids[row] = rows_of[sequence], position, prompts[sequence][position]
            self.state.block_table.copy_(table)
            self.state.context_base.copy_(base)
            rows = torch.arange(self.rows, device=self.state.tokens.device)
            self.state.tokens[rows, base.to(rows.device).long()] = ids.to(rows.device)
            self._events[0].record(self.stream)
            self.plan.launch(0, self.mode, self.stream.cuda_stream)
            self._events[1].record(self.stream)
            self.stream.synchronize()
            self.device_ms += self._events[0].elapsed_time(self._events[1])
            gave_up = self.plan.watchdog()
            if gave_up is not None:
                raise RuntimeError(f"a bounded device wait gave up: {gave_up}")
            self.chunks_run += 1
            chunk_logits = self.read_logits() if keep else None
            for row, (sequence, position) in enumerate(chunk):
                if keep:
                    logits_of[sequence][position] = chunk_logits[row]
                if position + 1 == len(prompts[sequence]):
                    results[sequence] = PrefillResult(int(self.state.tokens[row, position + 1]), logits_of[sequence])
        return results

    def read_logits(self):
        """fp32 [rows][vocab] of the last chunk (plans emitted with write_logits)."""
        torch = self.torch
        host = torch.empty(self.rows * self.vocab, dtype=torch.float32)
        self.plan.read_buffer("serving.logits", host.data_ptr(), host.numel() * 4)
        return host.reshape(self.rows, self.vocab)

    def close(self) -> None:
        self.plan.close()

    def __enter__(self) -> "ChunkedPrefill":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
