"""The sm_100 target description carries the fields the reference's TargetSpec parser
requires (lib/Target/TargetSpec.cpp:447-494) and real, measured values."""
import json
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_sm_100_target_has_required_schema_and_measured_values():
    target = json.loads((ROOT / "tilemega_b200" / "configs" / "targets" / "sm_100.json").read_text())
    assert (target["arch_tag"], target["sm_major"], target["sm_minor"]) == ("sm_100", 10, 0)
    for cap in ("cluster", "tma", "warp_specialized", "tcgen05", "l1_5", "net", "cp_async", "mbarrier"):
        assert isinstance(target["caps"][cap], bool)
    resources = target["resources"]
    for key in ("num_sms", "max_smem_per_sm", "max_dynamic_smem_per_cta", "regs_per_sm", "max_cluster_size",
                "max_threads_per_sm", "warp_size"):
        assert resources[key] > 0
    assert resources["num_sms"] == 148 and resources["max_dynamic_smem_per_cta"] == 232448
    calibration = target["calibration"]
    assert calibration["calibrated"] is True and calibration["pipelines"]["dram_gbps"] > 5000
