"""The allocation-free bounded-wait probe (tm_watchdog_probe_static) against the
plan-based one (tm_plan_watchdog_probe), through the C ABI.

It exists for callers that cannot take device memory from the allocator: a server
whose HBM already belongs to its weight and KV pools, or a health check that must
not trigger cudaMalloc's device-wide synchronisation. Its scratch is a fixed array
inside the library; the caller only brings the output buffer. The file name keeps
this test last in collection order."""
import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.serving.plan import STATIC_PROBE_MAX_WAITERS

from harness import GpuRun, bf16_weights

pytestmark = pytest.mark.gpu


def test_static_probe_agrees_with_plan_probe_twice_in_a_row(plan_dir):
    config = dict(synthetic.TINY, num_hidden_layers=1)
    run = GpuRun(config, bf16_weights(config), 1, 32, plan_dir)
    lib = run.lib
    waiters = 3
    records = torch.full((waiters, 12), 7, dtype=torch.int64, device="cuda:0")   # caller-owned output
    # the first call may load the kernel's module (lazy loading takes device memory once); from the second on the
    # driver's own count of free device memory must not move either, which also covers cudaMalloc calls that
    # bypass torch's allocator
    lib.watchdog_probe_static(0, waiters, False, 3000, records.data_ptr(), run.stream)
    torch.cuda.synchronize()
    for withhold in (True, False, True, False):        # two rounds in a row: the shared scratch must be cleared each time
        expected = run.plan.watchdog_probe(withhold=withhold, limit_us=3000)
        records.fill_(7)
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        lib.watchdog_probe_static(0, waiters, withhold, 3000, records.data_ptr(), run.stream)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        host = records.cpu()
        assert host[:, 0].tolist() == [int(expected)] * waiters            # gave up exactly when the plan-based probe did
        assert host[:, 2].tolist() == [1, 2, 3]                            # waiting CTA
        assert host[:, 9].tolist() == [1] * waiters                        # arrivals needed
        assert host[:, 10].tolist() == [0 if withhold else 1] * waiters    # arrivals seen
        assert host[:, 1].tolist() == [5 if withhold else 0] * waiters     # wait site of the record
    # sizes beyond the fixed scratch are refused, not truncated
    with pytest.raises(RuntimeError):
        lib.watchdog_probe_static(0, STATIC_PROBE_MAX_WAITERS + 1, True, 1000, records.data_ptr(), run.stream)
    with pytest.raises(RuntimeError):
        lib.watchdog_probe_static(0, 0, True, 1000, records.data_ptr(), run.stream)
    # the plan is still alive afterwards
    run.plan.set_steps([0])
    run.state.tokens[:, 0] = 3
    run.plan.launch(0, 2, run.stream)
    run.check_alive()
    run.close()
