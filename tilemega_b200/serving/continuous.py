"""Continuous batching over one paged decode plan: requests join and leave the batch between steps.

The reference's driver is static-batch (python/tilemega/serving/engine.py:27-178: every sequence
starts and ends together); its design notes list request admission and block allocation as the
step after the decode path (TileMega_skeleton.md:874-885). This module is that front end on the
host side, for a plan emitted with `kv_layout="paged"`:

* the batch is a fixed number of SLOTS; a slot holds one request or idles on a scratch block;
* a request gets ceil((prompt + new tokens + 1) / 16) blocks of the KV pool on admission (`BlockPool`)
  and gives them back when it ends; its row of `serving.block_table` names them;
* every decode step is one launch of plan step 0 with `serving.context_base[b]` = slot b's
  position, so sequences of any lengths and ages share a step; a slot still inside its prompt is
  teacher-forced (the next prompt token overwrites the sampled one, which is how the reference's
  prompt mode runs a prompt through the decode plan, engine.py:38-41);
* a request ends after `max_new_tokens` tokens or at its `eos` token.

With a `chunk_rows` prefill plan (serving/prefill.py) an admitted prompt is prefilled in chunks into the
same pool and decoding starts behind it; without one the prompt is teacher-forced as described above.

`SlotScheduler` (admission, block accounting, completion) is plain Python and tested on the CPU;
`ContinuousEngine` binds it to a plan and needs a CUDA device.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

KV_BLOCK = 16


@dataclass
class Request:
    id: int
    prompt: list[int]
    max_new_tokens: int
    eos: int | None = None
    generated: list[int] = field(default_factory=list)


class BlockPool:
    """Free list of KV pool blocks (block 0 is kept back as the idle slots' scratch block)."""

    def __init__(self, num_blocks: int):
        if num_blocks < 2:
            raise ValueError("the pool needs a scratch block and at least one more")
        self.free = deque(range(1, num_blocks))

    def take(self, count: int) -> list[int] | None:
        if count > len(self.free):
            return None
        return [self.free.popleft() for _ in range(count)]

    def give_back(self, blocks: list[int]) -> None:
        self.free.extend(blocks)


@dataclass
class Slot:
    request: Request | None = None
    blocks: list[int] = field(default_factory=list)
    position: int = 0     # position the next step decodes (= tokens of this request already in the cache)


class SlotScheduler:
    """Which request sits in which slot, at which position, on which blocks."""

    def __init__(self, slots: int, num_blocks: int, max_blocks_per_sequence: int):
        self.slots = [Slot() for _ in range(slots)]
        self.pool = BlockPool(num_blocks)
        self.max_blocks = max_blocks_per_sequence
        self.waiting: deque[Request] = deque()

    def submit(self, request: Request) -> None:
        if not request.prompt or request.max_new_tokens < 1:
            raise ValueError("a request needs a prompt and at least one new token")
        if self.blocks_needed(request) > self.max_blocks:
            raise ValueError("request is longer than the plan's capacity")
        self.waiting.append(request)

    @staticmethod
    def blocks_needed(request: Request) -> int:
        # one position more than the tokens: the kernel writes the token sampled at position p to p + 1
        return -(-(len(request.prompt) + request.max_new_tokens + 1) // KV_BLOCK)

    def admit(self) -> list[int]:
        """Fill free slots from the queue, in order, while the pool has blocks. Returns the slots filled."""
        filled = []
        for index, slot in enumerate(self.slots):
            if slot.request is not None or not self.waiting:
                continue
            blocks = self.pool.take(self.blocks_needed(self.waiting[0]))
            if blocks is None:
                break       # first come, first served: a later, smaller request does not overtake
            slot.request, slot.blocks, slot.position = self.waiting.popleft(), blocks, 0
            filled.append(index)
        return filled

    def active(self) -> list[int]:
        return [index for index, slot in enumerate(self.slots) if slot.request is not None]

    def advance(self, sampled: dict[int, int]) -> list[Request]:
        """One step has run. `sampled[b]` is the token the kernel chose for slot b. Returns the requests that ended."""
        ended = []
        for index in self.active():
            slot = self.slots[index]
            request = slot.request
            slot.position += 1
            if slot.position < len(request.prompt):
                continue                      # still inside the prompt: the sampled token is discarded
            token = sampled[index]
            request.generated.append(token)
            if len(request.generated) >= request.max_new_tokens or token == request.eos:
                self.pool.give_back(slot.blocks)
                self.slots[index] = Slot()
                ended.append(request)
        return ended

    def prefilled(self, index: int, first_token: int) -> Request | None:
        """The slot's whole prompt went through a prefill plan, which sampled `first_token` after its last
        position: decoding starts behind the prompt. Returns the request if that token already ends it."""
        slot = self.slots[index]
        request = slot.request
        slot.position = len(request.prompt)
        request.generated.append(first_token)
        if len(request.generated) >= request.max_new_tokens or first_token == request.eos:
            self.pool.give_back(slot.blocks)
            self.slots[index] = Slot()
            return request
        return None

    def forced_token(self, index: int) -> int | None:
        """The prompt token that must stand at the slot's NEXT position (None once the prompt is consumed)."""
        slot = self.slots[index]
        upcoming = slot.position + 1
        return slot.request.prompt[upcoming] if slot.request is not None and upcoming < len(slot.request.prompt) else None

    def idle(self) -> bool:
        return not self.waiting and not self.active()


class ContinuousEngine:
    """A paged decode plan driven one step at a time with a changing set of sequences."""

    def __init__(self, checkpoint, config: dict, decode_so, batch: int, device: int = 0, weights=None,
                 prefill_so=None, prefill_rows: int = 16):
        import torch

        from .plan import L2, PlanLibrary
        from .state import allocate_state
        from .weights import load_weights
        if not torch.cuda.is_available():
            raise RuntimeError("ContinuousEngine needs a CUDA device; there is no CPU path")
        self.torch = torch
        torch.cuda.set_device(device)
        self.library = PlanLibrary(decode_so)
        if "serving.block_table" not in self.library.index:
            raise ValueError("continuous batching needs a plan with a block-table KV pool (kv_layout='paged')")
        self.batch, self.mode = batch, L2
        capacity = self.library.info.capacity
        self.max_blocks = capacity // KV_BLOCK
        num_blocks = int(self.library.manifest["kv"]["num_blocks"])
        where = torch.device("cuda", device)
        self.weights = load_weights(checkpoint, self.library, device=where) if weights is None else weights
        # every row of the table starts on the scratch block; rows of admitted requests are rewritten
        table = torch.zeros((batch, self.max_blocks), dtype=torch.int32)
        self.state = allocate_state(config, batch, self.library, where, block_table=table, shared_blocks=True)
        bound = {name: tensor.data_ptr() for name, tensor in self.weights.items()} | self.state.pointers
        self.plan = self.library.create(batch, bound, device)
        self.plan.set_prompt_len(0)
        self.plan.set_steps([0])
        self.scheduler = SlotScheduler(batch, num_blocks, self.max_blocks)
        self.stream = torch.cuda.current_stream()
        self.host_positions = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.host_tokens = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.rows = torch.arange(batch, device=where)
        self.steps_run = 0
        # with a chunk_rows plan of the same model and pool size, prompts are prefilled in chunks of `prefill_rows`
        # positions into this engine's pool instead of being teacher-forced through the decode plan
        self.prefill = None
        if prefill_so is not None:
            from .prefill import ChunkedPrefill
            self.prefill = ChunkedPrefill(checkpoint, config, prefill_so, prefill_rows, self.state.kv_storage, device)

    def submit(self, request: Request) -> None:
        self.scheduler.submit(request)

    def _place(self, index: int) -> None:
        """Write an admitted request's block-table row and its first token."""
        torch = self.torch
        slot = self.scheduler.slots[index]
        row = torch.zeros(self.max_blocks, dtype=torch.int32)
        row[:len(slot.blocks)] = torch.tensor(slot.blocks, dtype=torch.int32)
        self.state.block_table[index].copy_(row, non_blocking=False)
        self.state.tokens[index, 0] = int(slot.request.prompt[0])

    def step(self) -> list[Request]:
        """Admit what fits, run one decode step for every slot, collect the tokens. Returns the requests that ended."""
        torch = self.torch
        admitted = self.scheduler.admit()
        for index in admitted:
            self._place(index)
        ended_in_prefill = []
        if self.prefill is not None and admitted:
            slots = [self.scheduler.slots[index] for index in admitted]
            results = self.prefill.run([slot.request.prompt for slot in slots], [slot.blocks for slot in slots])
            for index, slot, result in zip(admitted, slots, results):
                self.state.tokens[index, len(slot.request.prompt)] = result.first_token
                done = self.scheduler.prefilled(index, result.first_token)
                if done is not None:
                    ended_in_prefill.append(done)
        if not self.scheduler.active():
            return ended_in_prefill
        for index, slot in enumerate(self.scheduler.slots):
            self.host_positions[index] = slot.position if slot.request is not None else 0
        self.state.context_base.copy_(self.host_positions, non_blocking=True)
        self.plan.launch(0, self.mode, self.stream.cuda_stream)
        # teacher forcing: a slot inside its prompt gets the prompt's next token in place of the sampled one
        for index in self.scheduler.active():
            forced = self.scheduler.forced_token(index)
            if forced is not None:
                self.state.tokens[index, self.scheduler.slots[index].position + 1] = forced
        upcoming = (self.state.context_base.long() + 1).clamp_max(self.state.tokens.shape[1] - 1)
        self.host_tokens.copy_(self.state.tokens[self.rows, upcoming], non_blocking=True)
        self.stream.synchronize()
        gave_up = self.plan.watchdog()
        if gave_up is not None:
            raise RuntimeError(f"a bounded device wait gave up: {gave_up}")
        self.steps_run += 1
        sampled = {index: int(self.host_tokens[index]) for index in self.scheduler.active()}
        return ended_in_prefill + self.scheduler.advance(sampled)

    def run_until_done(self, limit: int = 100000) -> list[Request]:
        finished = []
        while not self.scheduler.idle():
            finished += self.step()
            if self.steps_run > limit:
                raise RuntimeError("step limit reached")
        return finished

    def close(self) -> None:
        if self.prefill is not None:
            self.prefill.close()
        self.plan.close()

    def __enter__(self) -> "ContinuousEngine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
