// Host interface of the encoder forward plans (phase TM_SERVING_FORWARD): a BERT-shaped encoder over
// batch x seq tokens, run as one CUDA graph of hand-written sm_100a kernels. The runtime's ABI entry
// points branch here for a plan whose sidecar says "phase": "forward"
// (reference: include/tilemega/Codegen/tasks/Sm90F3Runtime.cuh:95-200 is the forward runtime behind the
// same tm_plan_* names; include/tilemega/Codegen/tasks/Sm90F3Program.cuh:690-732 the forward kernel).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "plan_spec.h"

namespace tmb {

struct EncoderPlan;

// Builds the launch graph for `batch` sequences over the table's buffers (`buffers[i]` = device pointer of
// table entry i). Returns null and an error text when the shapes are not covered or a CUDA call fails.
EncoderPlan* EncoderCreate(const PlanSpec& spec, int batch, const std::vector<void*>& buffers, int sm_count,
                           std::string* error);
// One forward pass on `stream`; a cudaError_t as int.
int EncoderLaunch(EncoderPlan* plan, cudaStream_t stream);
// 1 and a record (word 0 = code of the wait that gave up) when a bounded device wait ran out, else 0.
int EncoderStatus(EncoderPlan* plan, uint64_t* record12);
void EncoderClear(EncoderPlan* plan);
void EncoderDestroy(EncoderPlan* plan);

}  // namespace tmb
