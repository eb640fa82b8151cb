"""Static-batch generation over one decode plan.

Same entry point as the reference's driver (python/tilemega/serving/engine.py:27-178:
`ServingEngine(checkpoint, config, decode_so, batch, ...)`, `generate(prompt_ids)`
returning a `Generation`), in its prompt mode: no prefill binary exists, the prompt's
positions run teacher-forced through the decode plan (engine.py:38-41 of the
reference) and the sampled tokens never leave the device until the end.

A generation is a list of spans of plan steps (step s decodes position s): one span
for the prompt, then the decode steps in spans of `decode_chunk` (one span when the
plan loops on the device, one span per step otherwise). Each span is one launch.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from pathlib import Path

import torch

from .plan import L1, L2, PlanLibrary
from .state import allocate_state
from .weights import Checkpoint, TensorCheckpoint, load_weights

MODES = {"auto": L2, "L1": L1, "L2": L2}


@dataclass
class Generation:
    tokens: torch.Tensor          # int32 [batch][new tokens], pinned host memory
    ttft_ms: float                # the prompt span, timed on the device
    step_ms: list[float]          # [ttft, then one entry per decode step when the plan stamps them]
    e2e_ms: float                 # host wall clock from the prompt upload to the tokens on the host
    decode_loop_used: bool = False
    step_ns_read: bool = False


def decode_spans(first: int, steps: int, chunk: int | None, looped: bool) -> list[tuple[int, int]]:
    """(first step, count) of every launch that covers decode steps [first, first + steps)."""
    if steps <= 0:
        return []
    if not looped:
        return [(first + offset, 1) for offset in range(steps)]
    size = steps if chunk is None else chunk
    if size < 1:
        raise ValueError("decode_chunk must be positive")
    return [(first + offset, min(size, steps - offset)) for offset in range(0, steps, size)]


class ServingEngine:
    def __init__(self, checkpoint: str | Path | Checkpoint | TensorCheckpoint, config: dict,
                 decode_so: str | Path, batch: int, prompt_len: int = 64, max_new_tokens: int = 1024,
                 mode: str = "auto", device: int = 0, decode_loop: bool = True,
                 decode_chunk: int | None = None, step_events: bool = True,
                 block_table: torch.Tensor | None = None, weights: dict[str, torch.Tensor] | None = None,
                 prefill_so: str | Path | None = None):
        if min(prompt_len, max_new_tokens) < 1:
            raise ValueError("prompt length and output length must be positive")
        if mode not in MODES:
            raise ValueError(f"unknown serving mode {mode}")
        if not torch.cuda.is_available():
            raise RuntimeError("ServingEngine needs a CUDA device; there is no CPU path")
        torch.cuda.set_device(device)
        self.decode_lib = PlanLibrary(decode_so)
        described = self.decode_lib.info
        if described.seq != 1 or prompt_len + max_new_tokens > described.capacity:
            raise ValueError("plan metadata does not cover this generation")
        self.decode_mode = MODES[mode]
        if not described.modes & self.decode_mode:
            raise ValueError("requested mode is not in the plan library")
        self.batch, self.prompt_len, self.max_new_tokens = batch, prompt_len, max_new_tokens
        self.decode_loop, self.decode_chunk, self.step_events = bool(decode_loop), decode_chunk, bool(step_events)
        where = torch.device("cuda", device)
        self.weights = load_weights(checkpoint, self.decode_lib, device=where) if weights is None else weights
        self.state = allocate_state(config, batch, self.decode_lib, device=where, block_table=block_table)
        bound = {name: tensor.data_ptr() for name, tensor in self.weights.items()} | self.state.pointers
        self.decode = self.decode_lib.create(batch, bound, device)
        self.loop_modes = self.decode.loop_modes()
        # With a prefill plan (phase 0, seq == prompt_len, same capacity and KV layout: the reference's
        # engine.py:41-57,89-92) the prompt runs as ONE step of that plan over the shared state; the decode plan
        # then starts behind the prompt. Without one the decode plan runs the prompt teacher-forced.
        self.prefill = self.prefill_lib = None
        if prefill_so is not None:
            self.prefill_lib = PlanLibrary(prefill_so)
            shape = self.prefill_lib.info
            if shape.phase != 0 or shape.seq != prompt_len or shape.capacity != described.capacity:
                raise ValueError("the prefill plan does not cover this prompt length and capacity")
            self.prefill_weights = load_weights(checkpoint, self.prefill_lib, device=where)
            both = bound | {name: tensor.data_ptr() for name, tensor in self.prefill_weights.items()}
            try:
                self.prefill = self.prefill_lib.create(batch, both, device)
            except BaseException:
                self.decode.close()
                raise
            self.prefill.set_steps([0])
            self.decode.set_steps(list(range(prompt_len, prompt_len + max_new_tokens - 1)) or [prompt_len])
        else:
            self.decode.set_prompt_len(prompt_len)
            self.decode.set_steps(list(range(prompt_len + max_new_tokens - 1)))

    def generate(self, prompt_ids: torch.Tensor, new_tokens: int | None = None) -> Generation:
        wanted = self.max_new_tokens if new_tokens is None else new_tokens
        if not 1 <= wanted <= self.max_new_tokens:
            raise ValueError("token count outside allocated step ring")
        if tuple(prompt_ids.shape) != (self.batch, self.prompt_len):
            raise ValueError("prompt tensor shape disagrees with plan")
        looped = self.decode_loop and wanted > 1 and bool(self.loop_modes & self.decode_mode)
        # plan steps of the decode plan: with a prefill plan its step s decodes position prompt_len + s
        first_decode = 0 if self.prefill is not None else self.prompt_len
        spans = [(0, self.prompt_len)] + decode_spans(first_decode, wanted - 1, self.decode_chunk, looped)
        host_prompt = prompt_ids.to(device="cpu", dtype=torch.int32).contiguous()
        host_prompt = host_prompt if host_prompt.is_pinned() else host_prompt.pin_memory()
        host_tokens = torch.empty((self.batch, wanted), dtype=torch.int32, pin_memory=True)
        stream = torch.cuda.current_stream()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        began = time.perf_counter()
        self.state.tokens[:, :self.prompt_len].copy_(host_prompt, non_blocking=True)
        for number, (first, count) in enumerate(spans):
            if number == 0:
                marks[0].record(stream)
            if number == 0 and self.prefill is not None:
                self.prefill.launch(0, self.decode_mode, stream.cuda_stream)
            elif count == 1 and not looped and number > 0:
                self.decode.launch(first, self.decode_mode, stream.cuda_stream)
            else:
                self.decode.launch_steps(first, count, self.decode_mode, stream.cuda_stream)
            if number == 0:
                marks[1].record(stream)
        host_tokens.copy_(self.state.tokens[:, self.prompt_len:self.prompt_len + wanted], non_blocking=True)
        stream.synchronize()
        e2e_ms = (time.perf_counter() - began) * 1e3
        gave_up = self.decode.watchdog() or (self.prefill.watchdog() if self.prefill is not None else None)
        if gave_up is not None:
            raise RuntimeError(f"a bounded device wait gave up: {gave_up}")
        step_ms = [marks[0].elapsed_time(marks[1])]
        stamped = self.step_events and wanted > 1
        if stamped:
            stamps = self.decode.read_step_ns(first_decode, wanted)
            step_ms += [(later - earlier) / 1e6 for earlier, later in zip(stamps, stamps[1:])]
        return Generation(host_tokens, step_ms[0], step_ms, e2e_ms, looped, stamped)

    def close(self) -> None:
        if self.prefill is not None:
            self.prefill.close()
        self.decode.close()

    def __enter__(self) -> "ServingEngine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
