"""ctypes binding of one serving plan library (tm_plan_* ABI, version 1).

The public surface is the reference driver's (python/tilemega/serving/plan.py:44-266:
`PlanLibrary`, `Plan`, their method names, argument meaning and the exception types
they raise), so code written against the reference reads the same here; the
reference's own, unmodified `PlanLibrary` loads the same `.so`. The binding itself
is table driven: every entry point of include/tilemega_b200.h is one row of
`SIGNATURES`, and every status-returning call goes through one checker that turns a
non-zero status into an exception carrying the library's last error text. The
library behind it is this repository's CUDA library; nothing else can stand in.
"""
from __future__ import annotations

import ctypes as C
import json
from pathlib import Path
from typing import NamedTuple

ABI_VERSION = 1
PREFILL, DECODE, FORWARD = 0, 1, 2
L1, L2 = 1, 2
STATIC_PROBE_MAX_WAITERS = 32
WATCHDOG_FIELDS = ("fired", "site", "block", "thread", "waiter_stage", "waiter_task", "producer_stage", "group", "row",
                   "need", "value", "iteration")


class PlanInfo(C.Structure):
    """tm_plan_info (include/tilemega_b200.h; ServingAbi.h:17-23 of the reference)."""
    _fields_ = ([(name, C.c_uint32) for name in ("abi_version", "phase")] +
                [(name, C.c_int32) for name in ("batch_lo", "batch_hi", "seq", "past_lo", "past_hi", "capacity", "grid",
                                                "residency")] +
                [(name, C.c_uint32) for name in ("modes", "buffer_count")])


class BufferInfo(C.Structure):
    """tm_buffer_info (ServingAbi.h:25-31 of the reference)."""
    _fields_ = [("name", C.c_char_p), ("role", C.c_uint32), ("dtype", C.c_uint32), ("elements_constant", C.c_uint64),
                ("elements_per_batch", C.c_uint64), ("pack_json", C.c_char_p)]


class Buffer(NamedTuple):
    name: str
    role: int
    dtype: int
    elements_constant: int
    elements_per_batch: int
    pack_json: str


_P, _U32, _U64, _I = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
# name -> (result type, argument types, required by the ABI)
SIGNATURES = {
    "tm_plan_query": (_I, [C.POINTER(PlanInfo)], True),
    "tm_plan_buffer": (_I, [_U32, C.POINTER(BufferInfo)], True),
    "tm_plan_create": (_P, [_I, C.POINTER(_P), _I], True),
    "tm_plan_set_steps": (_I, [_P, C.POINTER(C.c_int32), _U32], True),
    "tm_plan_launch": (_I, [_P, _U32, _U32, _U64, _P], True),
    "tm_plan_destroy": (None, [_P], True),
    "tm_plan_launch_steps": (_I, [_P, _U32, _U32, _U32, _U64, _P], False),
    "tm_plan_launch_steps_ranks": (_I, [C.POINTER(_P), _U32, _U32, _U32, _U32, _U64, _P], False),
    "tm_plan_loop_modes": (C.c_uint, [_P], False),
    "tm_plan_read_step_ns": (_I, [_P, _U32, _U32, C.POINTER(_U64)], False),
    "tm_plan_read_buffer": (_I, [_P, _U32, _P, _U64], False),
    "tm_plan_watchdog": (_I, [_P, C.POINTER(_U64)], False),
    "tm_plan_set_prompt_len": (_I, [_P, _I], False),
    "tm_plan_pdl_enabled": (C.c_uint, [_P], False),
    "tm_plan_execution_smem": (_U64, [_P, C.c_uint], False),
    "tm_plan_tp_world": (C.c_uint, [], False),
    "tm_plan_tp_bytes": (C.c_ulonglong, [C.c_uint], False),
    "tm_plan_bind_tp": (_I, [_P, _I, C.POINTER(_P), C.POINTER(_P)], False),
    "tm_plan_last_error": (C.c_char_p, [], False),
    "tm_plan_clear_watchdog": (_I, [_P], False),
    "tm_plan_watchdog_probe": (_I, [_P, _I, _U32, _P], False),
    "tm_plan_step_bytes": (_U64, [_P, _U64], False),
    "tm_plan_trace_step": (_I, [_P, _I], False),
    "tm_plan_read_trace": (C.c_longlong, [_P, C.POINTER(_U64), _U64], False),
    "tm_pack_tile_pages": (_I, [_P, _U64, _U64, _U64, _U32, _U32, _P, _P], False),
    "tm_calibrate": (_I, [_I, C.c_char_p, C.POINTER(C.c_double), _I], False),
    "tm_watchdog_probe_static": (_I, [_I, _I, _I, _U32, _P, _P], False),
    "tm_ipc_alloc": (_I, [_I, _U64, C.POINTER(_P)], False),
    "tm_ipc_free": (_I, [_P], False),
    "tm_ipc_export": (_I, [_P, C.c_char_p], False),
    "tm_ipc_open": (_I, [C.c_char_p, C.POINTER(_P)], False),
    "tm_ipc_close": (_I, [_P], False),
}


class PlanLibrary:
    """One loaded plan library: its static description, buffer table and sidecar."""

    def __init__(self, path: str | Path):
        self.path = Path(path).resolve(strict=True)
        self.lib = C.CDLL(str(self.path), mode=C.RTLD_LOCAL)
        sidecar = Path(f"{self.path}.plan.json")
        self.manifest = json.loads(sidecar.read_text()) if sidecar.exists() else {}
        self.execution = self.manifest.get("execution", "megakernel")
        for name, (result, arguments, required) in SIGNATURES.items():
            entry = getattr(self.lib, name, None)
            if entry is None:
                if required:
                    raise RuntimeError(f"{path}: required entry point {name} is missing")
                continue
            entry.restype, entry.argtypes = result, arguments
        self.info = PlanInfo()
        if self.lib.tm_plan_query(C.byref(self.info)) != 0 or self.info.abi_version != ABI_VERSION:
            raise RuntimeError(f"incompatible serving plan ABI: {path}: {self.last_error()}")
        info = self.info
        if info.phase == FORWARD and (info.past_lo or info.past_hi or info.capacity or info.seq < 1):
            raise RuntimeError("forward plan has invalid sequence or KV state metadata")
        self.buffers = tuple(self._buffer(index) for index in range(info.buffer_count))
        self.index = {buffer.name: position for position, buffer in enumerate(self.buffers)}

    def _buffer(self, index: int) -> Buffer:
        raw = BufferInfo()
        if self.lib.tm_plan_buffer(index, C.byref(raw)) != 0:
            raise RuntimeError(f"buffer {index} could not be queried")
        return Buffer(raw.name.decode(), raw.role, raw.dtype, raw.elements_constant, raw.elements_per_batch,
                      (raw.pack_json or b"").decode())

    def optional(self, name: str):
        return getattr(self.lib, name, None)

    def last_error(self) -> str:
        query = self.optional("tm_plan_last_error")
        return (query() or b"").decode() if query is not None else ""

    def checked(self, name: str, *arguments) -> None:
        """Call a status-returning entry point; a non-zero status raises with the library's message."""
        status = getattr(self.lib, name)(*arguments)
        if status != 0:
            raise RuntimeError(f"{name} failed ({status}): {self.last_error()}")

    # -- tensor parallelism ------------------------------------------------
    @property
    def tp_world(self) -> int:
        query = self.optional("tm_plan_tp_world")
        return int(query()) if query is not None else 1

    def tp_bytes(self, which: int) -> int:
        if self.tp_world == 1:
            raise ValueError("an unsharded plan has no tensor parallel buffers")
        return int(self.lib.tm_plan_tp_bytes(which))

    def ipc_alloc(self, device: int, nbytes: int) -> int:
        """A zeroed device region that is one allocation of its own (what an IPC handle names)."""
        pointer = _P()
        self.checked("tm_ipc_alloc", device, nbytes, C.byref(pointer))
        return int(pointer.value)

    def ipc_free(self, device_pointer: int) -> None:
        self.checked("tm_ipc_free", device_pointer)

    def ipc_export(self, device_pointer: int) -> bytes:
        """64-byte CUDA IPC handle of a device allocation (its base address)."""
        handle = C.create_string_buffer(64)
        self.checked("tm_ipc_export", device_pointer, handle)
        return handle.raw

    def ipc_open(self, handle: bytes) -> int:
        """Map a peer process's allocation; returns the pointer valid in this process."""
        pointer = _P()
        self.checked("tm_ipc_open", C.create_string_buffer(handle, 64), C.byref(pointer))
        return int(pointer.value)

    def ipc_close(self, device_pointer: int) -> None:
        self.checked("tm_ipc_close", device_pointer)

    # -- probes --------------------------------------------------------------
    def watchdog_probe_static(self, device: int, waiters: int, withhold: bool, limit_us: int,
                              records_pointer: int, stream: int = 0) -> None:
        """The bounded-wait self test without a plan and without any allocation: for
        callers whose device memory is fully committed or budgeted. `records_pointer`
        is a device buffer of waiters*12 uint64 owned by the caller; synchronise the
        stream before reading it. Calls share one scratch array inside the library:
        do not let two of them overlap on the GPU."""
        self.checked("tm_watchdog_probe_static", device, waiters, int(withhold), limit_us, records_pointer, stream)

    # -- plans ---------------------------------------------------------------
    def create(self, batch: int, pointers: dict[str, int], device: int) -> "Plan":
        if not self.info.batch_lo <= batch <= self.info.batch_hi:
            raise ValueError("batch outside the solved interval")
        table = (_P * len(self.buffers))()
        for position, buffer in enumerate(self.buffers):
            supplied = buffer.name in pointers
            if buffer.role == 1 and not supplied:
                raise KeyError(f"missing external buffer: {buffer.name}")
            if buffer.role != 1 and supplied:
                raise ValueError(f"internal buffer supplied externally: {buffer.name}")
            if supplied:
                table[position] = pointers[buffer.name]
        handle = self.lib.tm_plan_create(batch, table, device)
        if not handle:
            raise RuntimeError(f"tm_plan_create rejected the plan or its buffers: {self.last_error()}")
        return Plan(self, handle, batch)

    def launch_steps_ranks(self, plans: list["Plan"], first: int, count: int, mode: int, stream: int) -> None:
        """All ranks of a tensor-parallel job that live on ONE device, as one cooperative launch."""
        handles = (_P * len(plans))(*[plan.handle for plan in plans])
        self.checked("tm_plan_launch_steps_ranks", handles, len(plans), first, count, mode, plans[0].iteration[mode], stream)
        for plan in plans:
            plan.iteration[mode] += count


class Plan:
    """One created plan (device buffers bound). Keeps the per-mode launch count the ABI wants back."""

    def __init__(self, library: PlanLibrary, handle: int, batch: int = 0):
        self.library = library
        self.handle = handle
        self.batch = batch
        self.iteration = {L1: 0, L2: 0}
        self.prompt_len = 0

    def _call(self, name: str, *arguments) -> None:
        self.library.checked(name, self.handle, *arguments)

    def _mode_present(self, mode: int) -> None:
        if not self.library.info.modes & mode:
            raise ValueError("mode not present in this plan")

    def set_prompt_len(self, prompt_len: int) -> None:
        if self.library.optional("tm_plan_set_prompt_len") is None:
            raise RuntimeError("this plan was built without the prompt mode")
        self._call("tm_plan_set_prompt_len", prompt_len)
        self.prompt_len = prompt_len

    def set_steps(self, past: list[int]) -> None:
        info = self.library.info
        if info.phase == FORWARD and past != [0]:
            raise ValueError("forward plans accept only step zero")
        inside = lambda position: 0 <= position <= info.past_hi and (position >= info.past_lo or position < self.prompt_len)
        if not past or not all(inside(position) for position in past):
            raise ValueError("past outside the solved interval")
        self._call("tm_plan_set_steps", (C.c_int32 * len(past))(*past), len(past))

    def launch(self, step: int, mode: int, stream: int) -> None:
        if self.library.info.phase == FORWARD and step != 0:
            raise ValueError("forward plans accept only step zero")
        self._mode_present(mode)
        self._call("tm_plan_launch", step, mode, self.iteration[mode], stream)
        self.iteration[mode] += 1

    def launch_steps(self, first: int, count: int, mode: int, stream: int) -> None:
        self._mode_present(mode)
        self._call("tm_plan_launch_steps", first, count, mode, self.iteration[mode], stream)
        self.iteration[mode] += count

    def loop_modes(self) -> int:
        query = self.library.optional("tm_plan_loop_modes")
        return int(query(self.handle)) if query is not None else 0

    def bind_tp(self, rank: int, ar: list[int], exchange: list[int]) -> None:
        """Give this rank's plan every rank's all-reduce region and exchange block
        (python/tilemega/serving/plan.py:207-218 of the reference)."""
        world = self.library.tp_world
        if len(ar) != world or len(exchange) != world:
            raise ValueError("bind_tp needs one region and one exchange block per rank")
        self._call("tm_plan_bind_tp", rank, (_P * world)(*ar), (_P * world)(*exchange))

    def read_step_ns(self, first: int, count: int) -> list[int]:
        stamps = (_U64 * count)()
        self._call("tm_plan_read_step_ns", first, count, stamps)
        return list(stamps)

    def read_buffer(self, name: str, host_pointer: int, nbytes: int) -> None:
        """Copy table entry `name` into host memory (synchronise the stream first)."""
        self._call("tm_plan_read_buffer", self.library.index[name], host_pointer, nbytes)

    def watchdog(self) -> dict[str, int] | None:
        """The record of a bounded device wait that gave up, or None. Read it after
        synchronising a launch: a plan with a fired wait refuses further launches (-4)
        until clear_watchdog()."""
        read = self.library.optional("tm_plan_watchdog")
        if read is None or not self.handle:
            return None
        record = (_U64 * len(WATCHDOG_FIELDS))()
        if read(self.handle, record) != 1:
            return None
        return {field: int(value) for field, value in zip(WATCHDOG_FIELDS, record)}

    def clear_watchdog(self) -> None:
        self._call("tm_plan_clear_watchdog")

    def watchdog_probe(self, withhold: bool, limit_us: int, stream: int = 0) -> bool:
        """Run the two-CTA bounded-wait self test; True when the wait gave up."""
        outcome = self.library.lib.tm_plan_watchdog_probe(self.handle, int(withhold), limit_us, stream)
        if outcome < 0:
            raise RuntimeError(f"tm_plan_watchdog_probe failed: {self.library.last_error()}")
        return outcome == 1

    def trace_step(self, step: int) -> None:
        self._call("tm_plan_trace_step", step)

    def read_trace(self) -> list[int]:
        """Stage stamps [grid][stages][4] of the traced step, flattened."""
        read = self.library.lib.tm_plan_read_trace
        size = read(self.handle, None, 0)
        if size <= 0:
            raise RuntimeError("no trace was requested")
        stamps = (_U64 * (size // 8))()
        if read(self.handle, stamps, size) != size:
            raise RuntimeError("tm_plan_read_trace failed")
        return list(stamps)

    def step_bytes(self, cached_tokens_total: int) -> int:
        return int(self.library.lib.tm_plan_step_bytes(self.handle, cached_tokens_total))

    def execution_smem(self, mode: int = L2) -> int:
        return int(self.library.lib.tm_plan_execution_smem(self.handle, mode))

    def close(self) -> None:
        if self.handle:
            self.library.lib.tm_plan_destroy(self.handle)
            self.handle = 0

    def __enter__(self) -> "Plan":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
