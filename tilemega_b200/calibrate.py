"""Writes the sm_100 target description from measurements on the device at hand.

    python -m tilemega_b200.calibrate [--device 0] [--out tilemega_b200/configs/targets/sm_100.json]

The file follows the reference's target schema (parsed by `TargetSpec::FromJson`,
lib/Target/TargetSpec.cpp:396-494; the "calibration" block by `ParseCalibration`, :60-330),
so the reference's solver could read real Blackwell constants from it. The reference fills
the block with its own calibration kernels (lib/Target/Calibration.cu and siblings); here the
numbers come from the library's `tm_calibrate` microbenchmarks (csrc/calibrate.cu) and the
device properties. Keys of the schema that describe things this decode path does not have
(stream-K GEMM points, the split-K combine fit, the compute/copy interference ratio) are
present with neutral values and listed under "not_measured". Needs a CUDA device; reads
settings only, changes none.
"""
from __future__ import annotations

import argparse
import ctypes as C
import datetime
import json
from pathlib import Path

from .build import build_library

TARGET = Path(__file__).resolve().parent / "configs" / "targets" / "sm_100.json"


def measure(lib, device: int, what: str, capacity: int = 64) -> list[float]:
    out = (C.c_double * capacity)()
    count = lib.tm_calibrate(device, what.encode(), out, capacity)
    if count < 0:
        raise RuntimeError(f"tm_calibrate({what}) failed with status {count}")
    return [float(value) for value in out[:count]]


BENCHMARKS = ("clock", "pipes", "tensor", "smem", "latency", "l2_curve", "dram", "sync", "atomic_contention", "grid_barrier")


def describe(device: int = 0) -> dict:
    """Run every microbenchmark on `device` and assemble the target description."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("calibration needs a CUDA device")
    lib = C.CDLL(str(build_library()))
    lib.tm_calibrate.restype = C.c_int
    lib.tm_calibrate.argtypes = [C.c_int, C.c_char_p, C.POINTER(C.c_double), C.c_int]
    props = torch.cuda.get_device_properties(device)
    properties = {"name": props.name, "major": props.major, "minor": props.minor, "sms": props.multi_processor_count,
                  "l2_bytes": int(props.L2_cache_size), "smem_per_sm": int(props.shared_memory_per_multiprocessor),
                  "smem_optin": int(props.shared_memory_per_block_optin), "regs_per_sm": int(props.regs_per_multiprocessor),
                  "threads_per_sm": int(props.max_threads_per_multi_processor), "warp_size": int(props.warp_size),
                  "memory_bytes": int(props.total_memory)}
    stamp = datetime.datetime.now(datetime.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")
    return assemble(properties, {what: measure(lib, device, what) for what in BENCHMARKS}, stamp)


def assemble(props: dict, measured: dict[str, list[float]], stamp: str) -> dict:
    """The target description in the reference's schema from device properties and the raw
    benchmark outputs (`measured[what]` = what tm_calibrate(what) wrote)."""
    clock_mhz, = measured["clock"]
    fp32, int32, ex2, rsqrt = measured["pipes"]
    tc_fp16, tc_bf16 = measured["tensor"]
    *smem_by_occupancy, conflict_slope = measured["smem"]
    l1_ns, l2_ns, dram_ns = measured["latency"]
    curve_bytes, curve_gbps = measured["l2_curve"][0::2], measured["l2_curve"][1::2]
    dram_gbps, = measured["dram"]
    atomic_ns, fence_ns, syncthreads_ns, named_ns, cluster_ns = measured["sync"]
    contention, barrier = measured["atomic_contention"], measured["grid_barrier"]
    l2_gbps = max(curve_gbps)
    knee = max(size for size, rate in zip(curve_bytes, curve_gbps) if rate >= 0.8 * l2_gbps)
    return {
        "arch_tag": "sm_100", "nvcc_arch": "sm_100a", "sm_major": props["major"], "sm_minor": props["minor"],
        "caps": {"cluster": True, "tma": True, "warp_specialized": True, "tcgen05": True, "l1_5": True, "net": False,
                 "cp_async": True, "mbarrier": True, "mbarrier_try_wait": True, "mbarrier_tx": True, "bulk_copy": True,
                 "bulk_prefetch": True, "pdl": True, "wgmma": False, "setmaxnreg": True, "tma_im2col": True,
                 "bulk_reduce": True, "dsmem": True, "elect_sync": True},
        "resources_provenance": "cudaGetDeviceProperties of the calibrated device",
        "resources": {"num_sms": props["sms"], "l2_bytes": props["l2_bytes"], "max_smem_per_sm": props["smem_per_sm"],
                      "max_dynamic_smem_per_cta": props["smem_optin"], "regs_per_sm": props["regs_per_sm"],
                      "max_cluster_size": 8, "max_threads_per_sm": props["threads_per_sm"],
                      "warp_size": props["warp_size"], "dram_capacity_bytes": props["memory_bytes"]},
        "calibration": {
            "calibrated": True, "device": props["name"], "measured_at": stamp,
            "method": "tm_calibrate microbenchmarks of libtilemega_b200 (csrc/calibrate.cu), best of three, "
                      f"SM clock under load {clock_mhz:.0f} MHz",
            "not_measured": ["streamk", "combine_fixed_ns", "combine_d_dram_ns", "interference_ratio"],
            "pipelines": {
                "tc_fp16_gflops": tc_fp16, "tc_bf16_gflops": tc_bf16, "tc_path": "mma.sync.m16n8k16",
                "cuda_fp32_gflops": fp32, "cuda_int32_gops": int32, "sfu_exp2_gops": ex2, "sfu_rsqrt_gops": rsqrt,
                "smem_gbps": max(smem_by_occupancy), "smem_conflict_slope": conflict_slope,
                "l1_latency_ns": l1_ns, "l2_latency_ns": l2_ns, "dram_latency_ns": dram_ns,
                "l2_gbps": l2_gbps, "l2_knee_bytes": knee, "dram_gbps": dram_gbps,
                "l2_curve_bytes": curve_bytes, "l2_curve_gbps": curve_gbps,
                "smem_occupancy_ctas": [1, 2, 4, 8], "smem_occupancy_gbps": smem_by_occupancy,
                "sm_mhz_under_load": clock_mhz,
            },
            "sync": {
                "atomic_uncontended_ns": atomic_ns, "atomic_contention_ctas": contention[0::2],
                "atomic_contention_ns": contention[1::2], "threadfence_ns": fence_ns, "syncthreads_ns": syncthreads_ns,
                "named_barrier_ns": named_ns, "cluster_sync_ns": cluster_ns, "cluster_sync_calibrated": True,
                "grid_barrier_ctas": barrier[0::2], "grid_barrier_ns": barrier[1::2],
                "wait_protocol": "red.release.gpu + ld.acquire.gpu on one monotonic counter",
            },
            "streamk": [],
            "combine_fixed_ns": 0.0, "combine_fixed_resolved": False, "combine_d_dram_ns": 0.0,
            "interference_ratio": 1.0,
        },
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--device", type=int, default=0)
    parser.add_argument("--out", type=Path, default=TARGET)
    args = parser.parse_args()
    document = describe(args.device)
    args.out.write_text(json.dumps(document, indent=1) + "\n")
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
