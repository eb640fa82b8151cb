// Checker for the sm_100 target description: loads a target JSON with the REFERENCE's own
// parser (TargetSpec::FromJson, lib/Target/TargetSpec.cpp:396-494) and prints a few parsed
// fields. TEST INFRASTRUCTURE ONLY: tests/test_target_json.py compiles this file together with
// the reference's lib/Target/TargetSpec.cpp and lib/Support/Json.cpp where the reference tree
// is at hand (into oracle/_ref/, git-ignored) and runs it on
// tilemega_b200/configs/targets/sm_100.json.
#include <tilemega/Target/TargetSpec.h>

#include <cstdio>
#include <exception>

int main(int argc, char** argv) {
  if (argc != 2) {
    std::fprintf(stderr, "usage: target_check <target.json>\n");
    return 2;
  }
  try {
    const tilemega::TargetSpec spec = tilemega::TargetSpec::FromJson(argv[1]);
    std::printf("arch=%s sms=%d tcgen05=%d dram_gbps=%.1f l2_gbps=%.1f grid_barrier_points=%zu calibrated=%d\n",
                spec.arch_tag.c_str(), spec.res.num_sms, int(spec.caps.tcgen05), spec.calib.dram_gbps, spec.calib.l2_gbps,
                spec.calib.grid_barrier_ns.size(), int(spec.calib.calibrated));
  } catch (const std::exception& error) {
    std::fprintf(stderr, "rejected: %s\n", error.what());
    return 1;
  }
  return 0;
}
