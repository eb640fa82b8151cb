// Host-side description of one plan: model dimensions, request geometry, the
// buffer table with its packing recipes, and the GEMV page geometry. This is the
// part of the reference's code generator output that the runtime needs
// (lib/Frontend/ModelPlan.cpp:1005-1100 buffer names and recipes;
// lib/Codegen/Codegen.cpp:2164-2615 tables), written by hand instead of emitted.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "json.h"
#include "params.h"

namespace tmb {

struct BufferSpec {
  std::string name;
  uint32_t role = 0;   // 0 internal, 1 external
  uint32_t dtype = 0;  // 0 bf16, 1 f32, 2 i32, 3 i64, 4 e4m3, 5 f16
  uint64_t elements_constant = 0, elements_per_batch = 0;
  std::string pack_json;
};

// Index of the buffers the runtime binds, into PlanSpec::buffers.
struct LayerBuffers {
  int norm1, qkv, k, v, o, norm2, gate_up, down, router = -1, q_norm = -1, k_norm = -1;
  int qkv_scale = -1, o_scale = -1, gate_up_scale = -1, down_scale = -1;   // e4m3 weight plans: fp32 row scales
};

struct PlanSpec {
  // model
  // (heads, kv_heads, inter and head_rows are ONE RANK's shares when tp > 1: Megatron
  // sharding as in python/tilemega/serving/export.py:39-47,107-112,152-163)
  int hidden = 0, inter = 0, heads = 0, kv_heads = 0, head_dim = 0, layers = 0, vocab = 0;
  int tp = 1, head_rows = 0;
  // mixture of experts (experts == 0: dense MLP); `inter` is then ONE expert's width
  int experts = 0, topk = 0;
  bool norm_topk = false, qk_norm = false;
  double eps = 1e-5;
  bool tied = false;
  // request geometry
  int batch_lo = 1, batch_hi = 1, capacity = 0;
  bool paged = false;
  int num_blocks = 0, max_blocks = 0;
  // execution
  int grid = 0, slots = 0, attn_min_slots = 4;
  bool write_logits = true;
  int down_splits = 1;
  GemvGeo down_part[kMaxDownSplits] = {};
  GemvGeo geo[kNumGemv] = {};   // stages a plan does not have (kRouter in a dense plan) stay zero
  // dense-batch plans (batch_hi > kMaxBatch): GEMM stages on tcgen05 tiles; geo[] then describes the
  // page stream only (one task = cps pages of 128 rows x 128 columns)
  bool fp8 = false;             // GEMV matrices as e4m3 bytes + fp32 row scales
  int lm_head_scale = -1;
  bool dense_batch = false;
  bool chunk_rows = false;      // dense-batch plans: several rows of the batch may be consecutive positions of ONE sequence
  // prefill plans (phase 0): batch_lo..batch_hi count SEQUENCES of `prefill_seq` prompt positions each; the kernel
  // runs kDenseMaxBatch rows per step, (sequence, position) pairs in order, ceil(batch * seq / rows) steps per launch
  bool prefill = false;
  int prefill_seq = 0;
  // forward plans (phase 2): a stateless encoder pass over batch x forward_seq tokens (csrc/encoder.cu); hidden,
  // inter, heads, layers, vocab and eps describe the encoder, none of the decode fields above applies
  bool forward = false;
  bool f16 = false;             // activations and weights in fp16 (else bf16)
  int forward_seq = 0, max_position = 0, type_vocab = 0;
  bool forward_mask = false;    // the plan takes an "attention_mask" input (int64 [batch][seq], 0 = key position hidden)
  DenseGeo dgeo[kNumGemv] = {};
  int normed_buf = -1;
  // buffer table
  std::vector<BufferSpec> buffers;
  int tokens = -1, rope_cos = -1, rope_sin = -1, block_table = -1, context_base = -1;
  int embed = -1, final_norm = -1, lm_head = -1;
  int hidden_buf = -1, qkv_buf = -1, attn_buf = -1, mlp_buf = -1, logits_buf = -1, router_buf = -1,
      route_idx_buf = -1, route_weight_buf = -1;
  std::vector<LayerBuffers> layer;

  // Throws std::invalid_argument with a precise message on any unsupported field.
  static PlanSpec FromJson(const Json& plan);

  int qkv_rows() const { return (heads + 2 * kv_heads) * head_dim; }
  int max_k() const;
  // stages of a layer at a batch size: QKV, attention, O, gate/up, down (in parts for a wide batch); with
  // experts a router stage, and gate/up + down once per token
  int stages_per_layer(int batch) const { return experts ? 4 + 2 * batch : 5 + down_splits - 1; }
  // algorithmic bytes of one decode step (weights of every GEMV + KV rows read; with experts:
  // the dense matrices, the router, and batch * topk experts per layer)
  uint64_t weight_bytes() const;
  uint64_t kv_bytes_per_token() const { return 4ull * layers * kv_heads * head_dim; }
};

}  // namespace tmb
