"""Tensor-parallel serving driver, one process per GPU.

Same role as python/tilemega/serving/tp_engine.py:47-181 of the reference, which
drives all T devices from a single process. Here every rank is its own process
(`torch.distributed`, any backend: it only carries the set-up and the checks):
the rank loads its slice of the weights, allocates its request state, its
all-reduce receive region and its argmax exchange block, publishes the two
regions to its peers as CUDA IPC handles, and binds its plan to all ranks'
regions. After that the ranks' persistent kernels talk to each other directly
over NVLink from inside the GEMV epilogues; the host is not involved in a step.

As in the reference (tp_engine.py:115-131) every rank launches the same steps, and
every generation checks that all ranks wrote identical tokens.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path

import torch
import torch.distributed as dist

from .engine import Generation
from .plan import PlanLibrary
from .state import allocate_state
from .weights import Checkpoint, TensorCheckpoint, load_weights

L1 = 1


@dataclass
class TpGeneration(Generation):
    # (first, last) %globaltimer stamps of this rank's decode steps
    rank_span: tuple[int, int] = (0, 0)
    rank_spans: list[tuple[int, int]] = field(default_factory=list)


def exchange_handles(library: PlanLibrary, pointer: int, group=None) -> list[int]:
    """All ranks' copies of one region, as pointers valid in this process (own copy in place)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    handles: list[bytes | None] = [None] * world
    dist.all_gather_object(handles, library.ipc_export(pointer), group=group)
    return [pointer if q == rank else library.ipc_open(handles[q]) for q in range(world)]


class TpServingEngine:
    def __init__(self, checkpoint: str | Path | Checkpoint | TensorCheckpoint, config: dict,
                 decode_so: str | Path, batch: int, prompt_len: int = 64, max_new_tokens: int = 1024,
                 device: int | None = None, group=None, block_table: torch.Tensor | None = None,
                 context_base: torch.Tensor | None = None, weights: dict[str, torch.Tensor] | None = None):
        if not dist.is_initialized():
            raise RuntimeError("tensor parallel serving needs an initialised torch.distributed group")
        if not torch.cuda.is_available():
            raise RuntimeError("TpServingEngine needs a CUDA device; there is no CPU path")
        if prompt_len < 1 or max_new_tokens < 1:
            raise ValueError("prompt length and output length must be positive")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.library = PlanLibrary(decode_so)
        if self.library.tp_world != self.world or self.world < 2:
            raise ValueError(f"plan is sharded {self.library.tp_world} ways; the group has {self.world} ranks")
        info = self.library.info
        if info.seq != 1 or prompt_len + max_new_tokens > info.capacity:
            raise ValueError("plan metadata does not cover this generation")
        self.device = self.rank % torch.cuda.device_count() if device is None else device
        torch.cuda.set_device(self.device)
        torch.cuda.init()
        # identical grids on every rank: the ranks' o/down tiles are claimed in the same
        # order and a tile's owner waits for the same tile of its peers
        sms: list[int | None] = [None] * self.world
        dist.all_gather_object(sms, torch.cuda.get_device_properties(self.device).multi_processor_count, group=group)
        if len(set(sms)) != 1:
            raise RuntimeError("tensor parallel ranks must have identical SM counts")
        self.batch, self.prompt_len, self.max_new_tokens = batch, prompt_len, max_new_tokens
        where = torch.device("cuda", self.device)
        self.weights = weights if weights is not None else load_weights(
            checkpoint, self.library, device=where, tp=(self.rank, self.world))
        self.state = allocate_state(config, batch, self.library, device=where, block_table=block_table,
                                    context_base=context_base, tp=self.world)
        pointers = {name: tensor.data_ptr() for name, tensor in self.weights.items()}
        pointers.update(self.state.pointers)
        self.plan = self.library.create(batch, pointers, self.device)
        # zeroed by the allocator: epoch 0 never matches a live step
        self.ar_region = self.library.ipc_alloc(self.device, self.library.tp_bytes(0))
        self.exchange_block = self.library.ipc_alloc(self.device, self.library.tp_bytes(1))
        self.ar = exchange_handles(self.library, self.ar_region, group)
        self.exchange = exchange_handles(self.library, self.exchange_block, group)
        self.plan.bind_tp(self.rank, self.ar, self.exchange)
        self.plan.set_prompt_len(prompt_len)
        self.plan.set_steps(list(range(0, prompt_len + max_new_tokens - 1)))
        self.stream = torch.cuda.Stream(device=where)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)   # nobody launches before every rank's regions are mapped everywhere
        self.decode = self.plan

    def generate(self, prompt_ids: torch.Tensor, new_tokens: int | None = None) -> TpGeneration:
        count = new_tokens or self.max_new_tokens
        if count < 1 or count > self.max_new_tokens:
            raise ValueError("token count outside allocated step ring")
        if tuple(prompt_ids.shape) != (self.batch, self.prompt_len):
            raise ValueError("prompt tensor shape disagrees with plan")
        source = prompt_ids.to(device="cpu", dtype=torch.int32).contiguous().pin_memory()
        start, boundary, final = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        output = torch.empty((self.batch, count), dtype=torch.int32, pin_memory=True)
        wall_start = time.perf_counter()
        with torch.cuda.stream(self.stream):
            self.state.tokens[:, :self.prompt_len].copy_(source, non_blocking=True)
            start.record(self.stream)
            self.plan.launch_steps(0, self.prompt_len, L1, self.stream.cuda_stream)
            boundary.record(self.stream)
            if count > 1:
                self.plan.launch_steps(self.prompt_len, count - 1, L1, self.stream.cuda_stream)
            final.record(self.stream)
            output.copy_(self.state.tokens[:, self.prompt_len:self.prompt_len + count], non_blocking=True)
        self.stream.synchronize()
        e2e_ms = (time.perf_counter() - wall_start) * 1e3
        fired = self.plan.watchdog()
        failures: list[object] = [None] * self.world
        dist.all_gather_object(failures, fired, group=self.group)
        if any(item is not None for item in failures):
            raise RuntimeError(f"a bounded device wait gave up: {failures}")
        tokens: list[torch.Tensor | None] = [None] * self.world
        dist.all_gather_object(tokens, output.clone(), group=self.group)
        for rank in range(1, self.world):
            if not torch.equal(tokens[0], tokens[rank]):
                raise AssertionError(f"rank {rank} generated tokens differing from rank 0")
        step_ms = [start.elapsed_time(boundary)]
        span = (0, 0)
        if count > 1:
            ns = self.plan.read_step_ns(self.prompt_len, count)
            step_ms.extend((ns[i] - ns[i - 1]) / 1e6 for i in range(1, count))
            span = (int(ns[0]), int(ns[-1]))
        spans: list[tuple[int, int] | None] = [None] * self.world
        dist.all_gather_object(spans, span, group=self.group)
        return TpGeneration(output, step_ms[0], step_ms, e2e_ms, count > 1, count > 1, span, list(spans))

    def close(self) -> None:
        if getattr(self, "plan", None) is not None:
            torch.cuda.synchronize(self.device)
            self.plan.close()
            self.plan = None
            dist.barrier(group=self.group)   # peers may still hold mappings of this rank's regions
            for q in range(self.world):
                if q != self.rank:
                    self.library.ipc_close(self.ar[q])
                    self.library.ipc_close(self.exchange[q])
            dist.barrier(group=self.group)
            self.library.ipc_free(self.ar_region)
            self.library.ipc_free(self.exchange_block)

    def __enter__(self) -> "TpServingEngine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
