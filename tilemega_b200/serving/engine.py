"""Static-batch serving driver over one decode plan.

Mirrors python/tilemega/serving/engine.py:27-178 of the reference in its prompt
mode: there is no prefill binary, the prompt positions run teacher-forced
through the decode plan (engine.py:38-41,144-148) and the whole generation is
one or two persistent launches.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from pathlib import Path

import torch

from .plan import PlanLibrary
from .state import allocate_state
from .weights import Checkpoint, TensorCheckpoint, load_weights


@dataclass
class Generation:
    tokens: torch.Tensor
    ttft_ms: float
    step_ms: list[float]
    e2e_ms: float
    decode_loop_used: bool = False
    step_ns_read: bool = False


class ServingEngine:
    def __init__(self, checkpoint: str | Path | Checkpoint | TensorCheckpoint, config: dict,
                 decode_so: str | Path, batch: int, prompt_len: int = 64, max_new_tokens: int = 1024,
                 mode: str = "auto", device: int = 0, decode_loop: bool = True,
                 decode_chunk: int | None = None, step_events: bool = True,
                 block_table: torch.Tensor | None = None, weights: dict[str, torch.Tensor] | None = None):
        if prompt_len < 1 or max_new_tokens < 1:
            raise ValueError("prompt length and output length must be positive")
        if not torch.cuda.is_available():
            raise RuntimeError("ServingEngine needs a CUDA device; there is no CPU path")
        torch.cuda.set_device(device)
        torch.cuda.init()
        self.decode_lib = PlanLibrary(decode_so)
        if self.decode_lib.info.seq != 1 or prompt_len + max_new_tokens > self.decode_lib.info.capacity:
            raise ValueError("plan metadata does not cover this generation")
        self.batch = batch
        self.prompt_len = prompt_len
        self.max_new_tokens = max_new_tokens
        self.decode_loop = bool(decode_loop)
        self.decode_chunk = decode_chunk
        self.step_events = bool(step_events)
        if mode not in ("auto", "L1", "L2"):
            raise ValueError(f"unknown serving mode {mode}")
        self.decode_mode = 1 if mode == "L1" else 2
        if not self.decode_lib.info.modes & self.decode_mode:
            raise ValueError("requested mode is not in the plan library")
        target = torch.device("cuda", device)
        self.weights = weights if weights is not None else load_weights(checkpoint, self.decode_lib, device=target)
        self.state = allocate_state(config, batch, self.decode_lib, device=target, block_table=block_table)
        pointers = {name: tensor.data_ptr() for name, tensor in self.weights.items()}
        pointers.update(self.state.pointers)
        self.decode = self.decode_lib.create(batch, pointers, device)
        self.loop_modes = self.decode.loop_modes()
        # step s runs position s: the prompt's positions, then the decode steps
        self.decode.set_prompt_len(prompt_len)
        self.decode.set_steps(list(range(0, prompt_len + max_new_tokens - 1)))

    def generate(self, prompt_ids: torch.Tensor, new_tokens: int | None = None) -> Generation:
        count = new_tokens or self.max_new_tokens
        if count < 1 or count > self.max_new_tokens:
            raise ValueError("token count outside allocated step ring")
        if tuple(prompt_ids.shape) != (self.batch, self.prompt_len):
            raise ValueError("prompt tensor shape disagrees with plan")
        source = prompt_ids.to(device="cpu", dtype=torch.int32).contiguous()
        if not source.is_pinned():
            source = source.pin_memory()
        stream = torch.cuda.current_stream()
        start, first, final = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        cpu_tokens = torch.empty((self.batch, count), dtype=torch.int32, pin_memory=True)
        use_loop = bool(self.loop_modes & self.decode_mode) and self.decode_loop and count > 1
        wall_start = time.perf_counter()
        self.state.tokens[:, :self.prompt_len].copy_(source, non_blocking=True)
        start.record(stream)
        self.decode.launch_steps(0, self.prompt_len, self.decode_mode, stream.cuda_stream)
        first.record(stream)
        offset = self.prompt_len
        if use_loop:
            chunk = self.decode_chunk or count - 1
            if chunk < 1:
                raise ValueError("decode_chunk must be positive")
            for begin in range(0, count - 1, chunk):
                self.decode.launch_steps(offset + begin, min(chunk, count - 1 - begin), self.decode_mode,
                                         stream.cuda_stream)
        else:
            for step in range(count - 1):
                self.decode.launch(offset + step, self.decode_mode, stream.cuda_stream)
        final.record(stream)
        cpu_tokens.copy_(self.state.tokens[:, self.prompt_len:self.prompt_len + count], non_blocking=True)
        stream.synchronize()
        e2e_ms = (time.perf_counter() - wall_start) * 1e3
        fired = self.decode.watchdog()
        if fired is not None:
            raise RuntimeError(f"a bounded device wait gave up: {fired}")
        step_ms = [start.elapsed_time(first)]
        step_ns_read = False
        if count > 1 and self.step_events:
            ns = self.decode.read_step_ns(offset, count)
            step_ms.extend((ns[i] - ns[i - 1]) / 1e6 for i in range(1, count))
            step_ns_read = True
        return Generation(cpu_tokens, step_ms[0], step_ms, e2e_ms, use_loop, step_ns_read)

    def close(self) -> None:
        self.decode.close()

    def __enter__(self) -> "ServingEngine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
