"""ctypes binding of one serving plan library (tm_plan_* ABI, version 1).

Mirrors python/tilemega/serving/plan.py:44-266 of the reference: the same
classes, method names, argument meaning and error behaviour, so code and tests
written against the reference driver read the same here. The library behind it
is this repository's CUDA library; there is no other implementation to fall
back to.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass
from pathlib import Path

ABI_VERSION = 1
PREFILL, DECODE, FORWARD = 0, 1, 2
L1, L2 = 1, 2


class PlanInfo(C.Structure):
    _fields_ = [
        ("abi_version", C.c_uint32), ("phase", C.c_uint32),
        ("batch_lo", C.c_int32), ("batch_hi", C.c_int32),
        ("seq", C.c_int32), ("past_lo", C.c_int32),
        ("past_hi", C.c_int32), ("capacity", C.c_int32),
        ("grid", C.c_int32), ("residency", C.c_int32),
        ("modes", C.c_uint32), ("buffer_count", C.c_uint32),
    ]


class BufferInfo(C.Structure):
    _fields_ = [
        ("name", C.c_char_p), ("role", C.c_uint32), ("dtype", C.c_uint32),
        ("elements_constant", C.c_uint64), ("elements_per_batch", C.c_uint64),
        ("pack_json", C.c_char_p),
    ]


@dataclass(frozen=True)
class Buffer:
    name: str
    role: int
    dtype: int
    elements_constant: int
    elements_per_batch: int
    pack_json: str


_OPTIONAL = (
    ("tm_plan_launch_steps", C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_void_p]),
    ("tm_plan_loop_modes", C.c_uint, [C.c_void_p]),
    ("tm_plan_read_step_ns", C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64)]),
    ("tm_plan_read_buffer", C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64]),
    ("tm_plan_watchdog", C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    ("tm_plan_set_prompt_len", C.c_int, [C.c_void_p, C.c_int]),
    ("tm_plan_pdl_enabled", C.c_uint, [C.c_void_p]),
    ("tm_plan_execution_smem", C.c_uint64, [C.c_void_p, C.c_uint]),
    ("tm_plan_tp_world", C.c_uint, []),
    ("tm_plan_tp_bytes", C.c_ulonglong, [C.c_uint]),
    ("tm_plan_bind_tp", C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    ("tm_plan_last_error", C.c_char_p, []),
    ("tm_plan_clear_watchdog", C.c_int, [C.c_void_p]),
    ("tm_plan_watchdog_probe", C.c_int, [C.c_void_p, C.c_int, C.c_uint32, C.c_void_p]),
    ("tm_plan_step_bytes", C.c_uint64, [C.c_void_p, C.c_uint64]),
    ("tm_plan_trace_step", C.c_int, [C.c_void_p, C.c_int]),
    ("tm_plan_read_trace", C.c_longlong, [C.c_void_p, C.POINTER(C.c_uint64), C.c_uint64]),
    ("tm_watchdog_probe_static", C.c_int, [C.c_int, C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_void_p]),
    ("tm_ipc_alloc", C.c_int, [C.c_int, C.c_uint64, C.POINTER(C.c_void_p)]),
    ("tm_ipc_free", C.c_int, [C.c_void_p]),
    ("tm_ipc_export", C.c_int, [C.c_void_p, C.c_char_p]),
    ("tm_ipc_open", C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    ("tm_ipc_close", C.c_int, [C.c_void_p]),
)
STATIC_PROBE_MAX_WAITERS = 32


class PlanLibrary:
    def __init__(self, path: str | Path):
        self.path = Path(path).resolve(strict=True)
        self.lib = C.CDLL(str(self.path), mode=C.RTLD_LOCAL)
        manifest_path = Path(str(self.path) + ".plan.json")
        self.manifest = json.loads(manifest_path.read_text()) if manifest_path.exists() else {}
        self.execution = self.manifest.get("execution", "megakernel")
        lib = self.lib
        lib.tm_plan_query.argtypes = [C.POINTER(PlanInfo)]
        lib.tm_plan_query.restype = C.c_int
        lib.tm_plan_buffer.argtypes = [C.c_uint32, C.POINTER(BufferInfo)]
        lib.tm_plan_buffer.restype = C.c_int
        lib.tm_plan_create.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.c_int]
        lib.tm_plan_create.restype = C.c_void_p
        lib.tm_plan_set_steps.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_uint32]
        lib.tm_plan_set_steps.restype = C.c_int
        lib.tm_plan_launch.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_void_p]
        lib.tm_plan_launch.restype = C.c_int
        lib.tm_plan_destroy.argtypes = [C.c_void_p]
        lib.tm_plan_destroy.restype = None
        for name, result, arguments in _OPTIONAL:
            symbol = getattr(lib, name, None)
            if symbol is not None:
                symbol.restype = result
                symbol.argtypes = arguments
        info = PlanInfo()
        if lib.tm_plan_query(C.byref(info)) != 0 or info.abi_version != ABI_VERSION:
            raise RuntimeError(f"incompatible serving plan ABI: {path}: {self.last_error()}")
        if info.phase == FORWARD and (info.past_lo or info.past_hi or info.capacity or info.seq < 1):
            raise RuntimeError("forward plan has invalid sequence or KV state metadata")
        self.info = info
        buffers = []
        for index in range(info.buffer_count):
            item = BufferInfo()
            if lib.tm_plan_buffer(index, C.byref(item)) != 0:
                raise RuntimeError(f"buffer {index} could not be queried")
            buffers.append(Buffer(item.name.decode(), item.role, item.dtype, item.elements_constant,
                                  item.elements_per_batch, item.pack_json.decode() if item.pack_json else ""))
        self.buffers = tuple(buffers)
        self.index = {buffer.name: number for number, buffer in enumerate(buffers)}

    def last_error(self) -> str:
        query = getattr(self.lib, "tm_plan_last_error", None)
        text = query() if query is not None else b""
        return text.decode() if text else ""

    def watchdog_probe_static(self, device: int, waiters: int, withhold: bool, limit_us: int,
                              records_pointer: int, stream: int = 0) -> None:
        """The bounded-wait self test without a plan and without any allocation: for
        callers whose device memory is fully committed or budgeted. `records_pointer`
        is a device buffer of waiters*12 uint64 owned by the caller; synchronise the
        stream before reading it. Calls share one scratch array inside the library:
        do not let two of them overlap on the GPU."""
        status = self.lib.tm_watchdog_probe_static(device, waiters, int(withhold), limit_us, records_pointer, stream)
        if status != 0:
            raise RuntimeError(f"tm_watchdog_probe_static failed ({status})")

    @property
    def tp_world(self) -> int:
        query = getattr(self.lib, "tm_plan_tp_world", None)
        return int(query()) if query is not None else 1

    def tp_bytes(self, which: int) -> int:
        if self.tp_world == 1:
            raise ValueError("an unsharded plan has no tensor parallel buffers")
        return int(self.lib.tm_plan_tp_bytes(which))

    def ipc_alloc(self, device: int, nbytes: int) -> int:
        """A zeroed device region that is one allocation of its own (what an IPC handle names)."""
        pointer = C.c_void_p()
        if self.lib.tm_ipc_alloc(device, nbytes, C.byref(pointer)) != 0:
            raise RuntimeError(f"tm_ipc_alloc failed: {self.last_error()}")
        return int(pointer.value)

    def ipc_free(self, device_pointer: int) -> None:
        if self.lib.tm_ipc_free(device_pointer) != 0:
            raise RuntimeError(f"tm_ipc_free failed: {self.last_error()}")

    def ipc_export(self, device_pointer: int) -> bytes:
        """64-byte CUDA IPC handle of a device allocation (its base address)."""
        handle = C.create_string_buffer(64)
        if self.lib.tm_ipc_export(device_pointer, handle) != 0:
            raise RuntimeError(f"tm_ipc_export failed: {self.last_error()}")
        return handle.raw

    def ipc_open(self, handle: bytes) -> int:
        """Map a peer process's allocation; returns the pointer valid in this process."""
        pointer = C.c_void_p()
        if self.lib.tm_ipc_open(C.create_string_buffer(handle, 64), C.byref(pointer)) != 0:
            raise RuntimeError(f"tm_ipc_open failed: {self.last_error()}")
        return int(pointer.value)

    def ipc_close(self, device_pointer: int) -> None:
        if self.lib.tm_ipc_close(device_pointer) != 0:
            raise RuntimeError(f"tm_ipc_close failed: {self.last_error()}")

    def create(self, batch: int, pointers: dict[str, int], device: int) -> "Plan":
        if not self.info.batch_lo <= batch <= self.info.batch_hi:
            raise ValueError("batch outside the solved interval")
        addresses = (C.c_void_p * len(self.buffers))()
        for index, buffer in enumerate(self.buffers):
            if buffer.role == 1:
                if buffer.name not in pointers:
                    raise KeyError(f"missing external buffer: {buffer.name}")
                addresses[index] = pointers[buffer.name]
            elif buffer.name in pointers:
                raise ValueError(f"internal buffer supplied externally: {buffer.name}")
        handle = self.lib.tm_plan_create(batch, addresses, device)
        if not handle:
            raise RuntimeError(f"tm_plan_create rejected the plan or its buffers: {self.last_error()}")
        return Plan(self, handle, batch)


class Plan:
    def __init__(self, library: PlanLibrary, handle: int, batch: int = 0):
        self.library = library
        self.handle = handle
        self.batch = batch
        self.iteration = {1: 0, 2: 0}
        self.prompt_len = 0

    def set_prompt_len(self, prompt_len: int) -> None:
        setter = getattr(self.library.lib, "tm_plan_set_prompt_len", None)
        if setter is None:
            raise RuntimeError("this plan was built without the prompt mode")
        if setter(self.handle, prompt_len) != 0:
            raise RuntimeError("tm_plan_set_prompt_len failed")
        self.prompt_len = prompt_len

    def set_steps(self, past: list[int]) -> None:
        if self.library.info.phase == FORWARD and past != [0]:
            raise ValueError("forward plans accept only step zero")
        lo = self.library.info.past_lo
        if not past or any(not (lo <= p or p < self.prompt_len) or p < 0 or
                           p > self.library.info.past_hi for p in past):
            raise ValueError("past outside the solved interval")
        values = (C.c_int32 * len(past))(*past)
        if self.library.lib.tm_plan_set_steps(self.handle, values, len(past)) != 0:
            raise RuntimeError(f"tm_plan_set_steps failed: {self.library.last_error()}")

    def launch(self, step: int, mode: int, stream: int) -> None:
        if self.library.info.phase == FORWARD and step != 0:
            raise ValueError("forward plans accept only step zero")
        if not self.library.info.modes & mode:
            raise ValueError("mode not present in this plan")
        status = self.library.lib.tm_plan_launch(self.handle, step, mode, self.iteration[mode], stream)
        if status != 0:
            raise RuntimeError(f"tm_plan_launch failed ({status}): {self.library.last_error()}")
        self.iteration[mode] += 1

    def bind_tp(self, rank: int, ar: list[int], exchange: list[int]) -> None:
        """Give this rank's plan every rank's all-reduce region and exchange block
        (python/tilemega/serving/plan.py:207-218 of the reference)."""
        world = self.library.tp_world
        if len(ar) != world or len(exchange) != world:
            raise ValueError("bind_tp needs one region and one exchange block per rank")
        regions = (C.c_void_p * world)(*ar)
        blocks = (C.c_void_p * world)(*exchange)
        status = self.library.lib.tm_plan_bind_tp(self.handle, rank, regions, blocks)
        if status != 0:
            raise RuntimeError(f"tm_plan_bind_tp failed ({status}): {self.library.last_error()}")

    def loop_modes(self) -> int:
        query = getattr(self.library.lib, "tm_plan_loop_modes", None)
        return int(query(self.handle)) if query is not None else 0

    def launch_steps(self, first: int, count: int, mode: int, stream: int) -> None:
        if not self.library.info.modes & mode:
            raise ValueError("mode not present in this plan")
        status = self.library.lib.tm_plan_launch_steps(self.handle, first, count, mode,
                                                       self.iteration[mode], stream)
        if status != 0:
            raise RuntimeError(f"tm_plan_launch_steps failed ({status}): {self.library.last_error()}")
        self.iteration[mode] += count

    def read_step_ns(self, first: int, count: int) -> list[int]:
        values = (C.c_uint64 * count)()
        if self.library.lib.tm_plan_read_step_ns(self.handle, first, count, values) != 0:
            raise RuntimeError("tm_plan_read_step_ns failed")
        return list(values)

    def read_buffer(self, name: str, host_pointer: int, nbytes: int) -> None:
        """Copy table entry `name` into host memory (synchronise the stream first)."""
        index = self.library.index[name]
        if self.library.lib.tm_plan_read_buffer(self.handle, index, host_pointer, nbytes) != 0:
            raise RuntimeError(f"tm_plan_read_buffer failed: {self.library.last_error()}")

    def watchdog(self) -> dict[str, int] | None:
        read = getattr(self.library.lib, "tm_plan_watchdog", None)
        if read is None or not self.handle:
            return None
        values = (C.c_uint64 * 12)()
        if read(self.handle, values) != 1:
            return None
        return dict(zip(("fired", "site", "block", "thread", "waiter_stage", "waiter_task",
                         "producer_stage", "group", "row", "need", "value", "iteration"),
                        map(int, values)))

    def clear_watchdog(self) -> None:
        if self.library.lib.tm_plan_clear_watchdog(self.handle) != 0:
            raise RuntimeError("tm_plan_clear_watchdog failed")

    def watchdog_probe(self, withhold: bool, limit_us: int, stream: int = 0) -> bool:
        """Run the two-CTA bounded-wait self test; True when the wait gave up."""
        result = self.library.lib.tm_plan_watchdog_probe(self.handle, int(withhold), limit_us, stream)
        if result < 0:
            raise RuntimeError(f"tm_plan_watchdog_probe failed: {self.library.last_error()}")
        return result == 1

    def trace_step(self, step: int) -> None:
        if self.library.lib.tm_plan_trace_step(self.handle, step) != 0:
            raise RuntimeError("tm_plan_trace_step failed")

    def read_trace(self) -> list[int]:
        """Stage stamps [grid][stages][4] of the traced step, flattened."""
        size = self.library.lib.tm_plan_read_trace(self.handle, None, 0)
        if size <= 0:
            raise RuntimeError("no trace was requested")
        values = (C.c_uint64 * (size // 8))()
        if self.library.lib.tm_plan_read_trace(self.handle, values, size) != size:
            raise RuntimeError("tm_plan_read_trace failed")
        return list(values)

    def step_bytes(self, cached_tokens_total: int) -> int:
        return int(self.library.lib.tm_plan_step_bytes(self.handle, cached_tokens_total))

    def execution_smem(self, mode: int = 2) -> int:
        return int(self.library.lib.tm_plan_execution_smem(self.handle, mode))

    def close(self) -> None:
        if self.handle:
            self.library.lib.tm_plan_destroy(self.handle)
            self.handle = 0

    def __enter__(self) -> "Plan":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
