"""The sm_100 target description: it carries every field the reference's TargetSpec parser
requires (lib/Target/TargetSpec.cpp:60-330, 396-494), and -- where the reference tree is at
hand -- the reference's OWN parser, compiled from its sources as the checker, loads both the
committed file and a file assembled by the calibration writer."""
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
TARGET = ROOT / "tilemega_b200" / "configs" / "targets" / "sm_100.json"
sys.path.insert(0, str(ROOT / "oracle"))

REQUIRED_PIPELINES = ("tc_fp16_gflops", "cuda_fp32_gflops", "cuda_int32_gops", "sfu_exp2_gops", "sfu_rsqrt_gops", "smem_gbps",
                      "smem_conflict_slope", "l1_latency_ns", "l2_latency_ns", "dram_latency_ns", "l2_gbps", "l2_knee_bytes",
                      "dram_gbps", "l2_curve_bytes", "l2_curve_gbps", "smem_occupancy_ctas", "smem_occupancy_gbps")
REQUIRED_SYNC = ("atomic_uncontended_ns", "atomic_contention_ctas", "atomic_contention_ns", "threadfence_ns", "syncthreads_ns",
                 "named_barrier_ns", "cluster_sync_ns", "cluster_sync_calibrated", "grid_barrier_ctas", "grid_barrier_ns")


def fake_measurements():
    return {"clock": [1900.0], "pipes": [70000.0, 35000.0, 9000.0, 9000.0], "tensor": [600000.0, 600000.0],
            "smem": [20000.0, 30000.0, 33000.0, 33000.0, 0.9], "latency": [20.0, 300.0, 800.0],
            "l2_curve": [4e6, 15000.0, 64e6, 12000.0, 1e9, 6000.0], "dram": [6500.0],
            "sync": [700.0, 400.0, 20.0, 15.0, 150.0], "atomic_contention": [1, 700.0, 148, 2500.0],
            "grid_barrier": [1, 900.0, 148, 1800.0]}


def fake_properties():
    return {"name": "test device", "major": 10, "minor": 0, "sms": 148, "l2_bytes": 132120576, "smem_per_sm": 233472,
            "smem_optin": 232448, "regs_per_sm": 65536, "threads_per_sm": 2048, "warp_size": 32, "memory_bytes": 190000000000}


def check_schema(target):
    assert (target["arch_tag"], target["sm_major"], target["sm_minor"]) == ("sm_100", 10, 0)
    for cap in ("cluster", "tma", "warp_specialized", "tcgen05", "l1_5", "net", "cp_async", "mbarrier"):
        assert isinstance(target["caps"][cap], bool)
    for key in ("num_sms", "max_smem_per_sm", "max_dynamic_smem_per_cta", "regs_per_sm", "max_cluster_size",
                "max_threads_per_sm", "warp_size"):
        assert target["resources"][key] > 0
    calibration = target["calibration"]
    assert calibration["calibrated"] is True
    for key in REQUIRED_PIPELINES:
        assert key in calibration["pipelines"], key
    for key in REQUIRED_SYNC:
        assert key in calibration["sync"], key
    for key in ("streamk", "combine_fixed_ns", "combine_d_dram_ns", "interference_ratio"):
        assert key in calibration, key
    curve = calibration["pipelines"]
    assert len(curve["l2_curve_bytes"]) == len(curve["l2_curve_gbps"]) >= 3
    assert len(calibration["sync"]["grid_barrier_ctas"]) == len(calibration["sync"]["grid_barrier_ns"]) >= 2


def test_committed_target_has_the_required_schema_and_measured_values():
    target = json.loads(TARGET.read_text())
    check_schema(target)
    assert target["resources"]["num_sms"] == 148 and target["resources"]["max_dynamic_smem_per_cta"] == 232448
    pipelines = target["calibration"]["pipelines"]
    assert 5000 < pipelines["dram_gbps"] < 8200 and pipelines["l2_gbps"] > pipelines["dram_gbps"]
    assert pipelines["l1_latency_ns"] < pipelines["l2_latency_ns"] < pipelines["dram_latency_ns"]


def test_calibration_writer_assembles_the_schema():
    from tilemega_b200.calibrate import assemble
    check_schema(assemble(fake_properties(), fake_measurements(), "2026-01-01T00:00:00Z"))


@pytest.fixture(scope="module")
def reference_parser(tmp_path_factory):
    """The reference's TargetSpec::FromJson behind oracle/target_check.cpp, built from the reference
    tree's own sources (skipped where the tree, a CUTLASS header tree or the CUDA headers are absent)."""
    from build_ref import reference_tree
    tree = reference_tree()
    if tree is None:
        pytest.skip("no reference tree on this machine")
    import importlib.util
    cutlass = None
    for package in ("flashinfer", "tilelang"):
        found = importlib.util.find_spec(package)
        for relative in ("data/cutlass/include", "3rdparty/cutlass/include"):
            if found and found.submodule_search_locations:
                candidate = Path(list(found.submodule_search_locations)[0]) / relative
                if (candidate / "cutlass" / "arch" / "arch.h").exists():
                    cutlass = candidate
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    if cutlass is None or not (cuda / "include" / "cuda_runtime_api.h").exists() or shutil.which("g++") is None:
        pytest.skip("no CUTLASS header tree, CUDA headers or g++")
    binary = ROOT / "oracle" / "_ref" / "target_check"
    binary.parent.mkdir(exist_ok=True)
    command = ["g++", "-std=c++17", "-O1", f"-I{tree / 'include'}", f"-I{cutlass}", f"-I{cuda / 'include'}",
               str(ROOT / "oracle" / "target_check.cpp"), str(tree / "lib" / "Target" / "TargetSpec.cpp"),
               str(tree / "lib" / "Support" / "Json.cpp"), "-o", str(binary), f"-L{cuda / 'lib64'}", "-lcudart"]
    subprocess.run(command, check=True)
    environment = dict(os.environ, LD_LIBRARY_PATH=f"{cuda / 'lib64'}:{os.environ.get('LD_LIBRARY_PATH', '')}")
    return lambda path: subprocess.run([str(binary), str(path)], capture_output=True, text=True, env=environment)


def test_reference_parser_loads_the_committed_target(reference_parser):
    done = reference_parser(TARGET)
    assert done.returncode == 0, done.stderr
    assert "arch=sm_100 sms=148 tcgen05=1" in done.stdout and "calibrated=1" in done.stdout


def test_reference_parser_loads_what_the_writer_assembles(reference_parser, tmp_path):
    from tilemega_b200.calibrate import assemble
    path = tmp_path / "assembled.json"
    path.write_text(json.dumps(assemble(fake_properties(), fake_measurements(), "2026-01-01T00:00:00Z")))
    done = reference_parser(path)
    assert done.returncode == 0, done.stderr
    # and it does reject a file without the calibration keys (what the parser is strict about)
    broken = json.loads(path.read_text())
    del broken["calibration"]["pipelines"]["tc_fp16_gflops"]
    path.write_text(json.dumps(broken))
    assert reference_parser(path).returncode == 1
