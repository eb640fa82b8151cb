// Structures shared by the host runtime and the persistent decode kernel.
// Plain C++ (no CUDA types) so the host side can be unit-tested without a GPU.
#pragma once
#include <stdint.h>

#ifndef __CUDACC__
#define __host__
#define __device__
#endif

namespace tmb {

constexpr int kConsumerWarps = 8;                       // warps that do arithmetic
constexpr int kConsumerThreads = kConsumerWarps * 32;   // 256
constexpr int kThreads = kConsumerThreads + 32;         // + one streaming warp (one thread of it works)
constexpr int kSlotBytes = 32768;                       // one ring slot = one weight page / KV group
constexpr int kMaxSlots = 6;
constexpr int kTileN = 8;                               // weight rows per page (one 128B-swizzle atom)
constexpr int kKvBlock = 16;                            // tokens per KV block
constexpr int kMaxBatch = 8;                            // batch rows of the mma A operand (rows 0..7)
constexpr int kPartialRing = 8;                         // GEMV tasks whose warp partials may be in flight (> ring slots + 1)
constexpr int kAttnHalfBytes = kSlotBytes / 2;          // K part, then V part, of an attention slot
constexpr int kMaxTp = 8;                               // tensor-parallel ranks of one plan
// Dense-batch plans (batch 16..64, a multiple of 16): the GEMM stages run on the 5th-generation tensor
// cores. A weight page is 128 rows x 128 columns (two 64-column swizzle blocks of 128 rows x 128 bytes:
// the K-major 128-byte-swizzled operand layout of tcgen05.mma, which is what the tile_pages recipe
// writes for tile_n = 128), again one 32 KB ring slot; the batch rows are the N side of the tile.
constexpr int kDenseTileN = 128;
constexpr int kDenseTileK = 128;
constexpr int kDenseMaxBatch = 64;
constexpr int kDenseXSlots = 4;                         // at most this many activation chunks (batch x 128 columns) in flight per CTA
// ... as many of them as fit 48 KB: 3 at batch 64, 4 below
__host__ __device__ inline int dense_x_slots(int batch) {
  const int fit = 49152 / (batch * kDenseTileK * 2);
  return fit < kDenseXSlots ? fit : kDenseXSlots;
}
constexpr int kDenseThreads = kThreads + 32;            // + the warp whose lane 0 loads activations and issues tcgen05.mma
constexpr int kDenseTmemColumns = 128;                  // two accumulators of up to 64 fp32 columns

// kRouter exists in mixture-of-experts plans only; there kGateUp / kDown describe ONE expert.
enum StageKind : int { kQkv = 0, kOProj = 1, kGateUp = 2, kDown = 3, kHead = 4, kRouter = 5, kNumGemv = 6 };
constexpr int kMaxTopK = 8;                             // experts per token
constexpr int kMaxDownSplits = 8;                       // stages a down projection's reduction may be cut into
// kEpiResidualAllReduce: kEpiResidual after the ranks' bf16 partial sums are added in rank order.
// kEpiPartial: the fp32 sums of one part of a split reduction, kept in global memory for the next part.
enum Epilogue : int { kEpiStore = 0, kEpiResidual = 1, kEpiSwiGLU = 2, kEpiHead = 3, kEpiResidualAllReduce = 4, kEpiPartial = 5 };

// Geometry of one GEMV stage. Weights are packed [N/8][K/tile_k][8*tile_k]
// with the 8x64 128-byte XOR swizzle of the reference's tile_pages recipe
// (python/tilemega/serving/weights.py:204-242), so one page is one contiguous
// bulk copy.
struct GemvGeo {
  int n, k;            // output rows, reduction length (k: a multiple of tile_k; columns past k_src are zero)
  int k_src;           // columns the activation rows really have (the packing recipe zero-pads the weights to k)
  int tile_k;          // columns per page (2048)
  int pages_per_task;  // k / tile_k: a task is one 8-row tile over the whole reduction
  int last_page_bytes; // bytes of a task's last page that are copied: k_src rounded up to 256 columns (a warp's share)
  int ntasks;          // n / 8
  // A stage may cover only pages [page0, page0 + pages_per_task) of every task's run of
  // task_pages pages (the reduction of a wide-batch down projection is taken in several
  // stages, so that its activation rows fit in shared memory); its rows then start src_off
  // columns into source rows that are src_stride columns apart.
  int page0, task_pages, src_off, src_stride;
  int claim_chunk;     // tasks taken per claim: about 64 KB of pages, so a claim's round trip hides behind the copies
  int page_bytes;      // bytes of one page = one ring slot (8 rows x tile_k columns of 2 bytes, or of 1 byte for e4m3 weights)
};

// Geometry of one GEMM stage of a dense-batch plan: `tiles` row tiles of 128 weight rows, the
// reduction cut into `nsplit` parts of `cps` 128-column chunks each, so that there are enough tasks
// (tile, part) for every SM to stream; task id = tile * nsplit + part, its pages are contiguous.
// With nsplit > 1 every task leaves its fp32 partial tile in global memory and the last arriver of a
// tile adds the parts in ascending order (bit-reproducible) and runs the epilogue.
struct DenseGeo {
  int n, k;
  int tiles, nsplit, cps, ntasks;
};

struct LayerPtrs {
  // e4m3 weight plans: fp32 scale per output row of the four matrices (else null)
  const float* qkv_scale;
  const float* o_scale;
  const float* gate_up_scale;
  const float* down_scale;
  const void* qkv;       // packed pages, rows group-interleaved [Gq q heads][k][v] per KV head
  const void* o;
  const void* gate_up;   // packed pages, rows interleaved 4 gate / 4 up
  const void* down;
  const void* norm1;     // bf16 [H]
  const void* norm2;     // bf16 [H]
  const void* router;    // packed pages [E/8][H/tile_k] (mixture of experts), else null
  const void* q_norm;    // bf16 [D] per-head RMSNorm weights applied before RoPE (Qwen3), else null
  const void* k_norm;
  void* k_pool;          // bf16, addressed by block table
  void* v_pool;
};

// Status words written by the device (index into MegaParams::status).
enum StatusWord : int {
  kStFired = 0, kStSite, kStBlock, kStThread, kStStage, kStTask, kStProducer,
  kStGroup, kStRow, kStNeed, kStValue, kStIteration, kStWords
};
enum WaitSite : int { kSiteGrid = 1, kSiteFull = 2, kSiteEmpty = 3, kSiteTest = 5, kSitePeer = 6 };

struct MegaParams {
  // model
  // (heads, kv_heads, inter are this rank's shares of a tensor-parallel plan; vocab is the
  // whole vocabulary, of which this rank's head scores rows [head_base, head_base + geo[kHead].n))
  int batch, hidden, inter, heads, kv_heads, head_dim, layers, vocab;
  int head_base;
  // mixture of experts (experts == 0: dense MLP). gate_up / down of a layer are stacks of
  // `experts` packed matrices; geo[kGateUp] / geo[kDown] describe one of them.
  int experts, topk, norm_topk;
  int qk_norm;              // per-head RMSNorm of q and k before RoPE (Qwen3)
  int stages_per_layer;     // 5 dense, 6 with a router stage
  int trace_stages;         // stage records per CTA of a traced step (dense-batch plans record their RMSNorm stages too)
  float eps;
  float qk_scale_log2;      // log2(e) / sqrt(head_dim)
  // request state
  int capacity, max_blocks; // tokens per sequence; block-table row length
  int kv_max_entry;         // block-table entries are clamped to [0, kv_max_entry]
  long long kv_block_stride, kv_head_stride;   // elements
  int first_step, nsteps, prompt_len;
  int write_logits;
  int grid, nslots, xs_bytes;
  int attn_min_spt;         // least ring slots of keys per attention task (a task's fixed cost wants amortising)
  int bars_per_step;        // grid-wide arrivals of one decode step
  unsigned long long bar_base;     // grid-barrier arrivals before this launch
  unsigned long long watchdog_ns;  // per-wait limit
  GemvGeo geo[kNumGemv];
  int down_splits;                       // 1: geo[kDown] is the whole stage; else down_part[0..down_splits-1] run in turn
  GemvGeo down_part[kMaxDownSplits];
  // external buffers
  int* tokens;                 // [B][capacity]
  const void* rope_cos;        // bf16 [capacity][D]
  const void* rope_sin;
  const int* block_table;      // [B][max_blocks]
  const int* ctx_base;         // [B] position offset of each sequence (may be null)
  const int* past;             // [steps] position run by each step
  const void* embed;           // bf16 [V][H]
  const void* final_norm;      // bf16 [H]
  const void* lm_head;         // packed pages [V/8][H/tile_k][8*tile_k]
  const float* lm_head_scale;  // e4m3 weight plans: fp32 scale per vocabulary row (else null)
  int fp8;                     // weights are e4m3 bytes with per-row scales: pages of 8 rows x 4096 columns
  const LayerPtrs* layer;      // [L]
  // internal buffers
  void* x;                     // bf16 [B][H] residual stream
  void* qkv;                   // bf16 [B][(Hq+2Hkv)*D]
  void* attn;                  // bf16 [B][Hq*D]
  void* h;                     // bf16 [B][I]
  void* logits;                // f32 [B][V]: head accumulators before the bf16 rounding
  void* router_logits;         // bf16 [B][experts]
  int* route_idx;              // [layers][topk] chosen experts of the last step, in rank order (batch 1)
  float* route_w;              // [layers][topk] their routing weights
  float* down_partial;         // f32 [B][H]: running sums of a split down projection
  float* attn_part;            // [attn_part_tasks][Gq][D+2]: one record per attention task
  int attn_part_tasks;         // 2*grid + B*Hkv + 2: about two tasks per CTA, plus the rounding up per (sequence, KV head)
  unsigned* attn_cnt;          // [B*Hkv]
  unsigned long long* qkv_ready;  // [Hkv] QKV row tiles stored per KV-head group (monotonic within a launch)
  float* argmax_val;           // [grid][B]
  int* argmax_idx;             // [grid][B]
  unsigned* stage_cnt;         // [nsteps*(5*layers+1)+2] task claim counters, zero at launch
  unsigned long long* bar;     // grid barrier arrivals (monotonic)
  unsigned long long* status;  // [kStWords]
  unsigned long long* step_ns; // [capacity+1] %globaltimer stamps
  unsigned long long* trace;   // [grid][5*layers+1][4] stage stamps of step trace_step, or null
  int trace_step;
  // dense-batch plans (dense != 0): GEMM stages on tcgen05 tiles
  int dense;
  int chunk_rows;              // rows may be consecutive positions of one sequence: append stage + barrier before attention
  // prefill plans: row r of step s is cache position row_pos[s * batch + r] (its position in the prompt plus the
  // sequence's context_base, resolved at launch) of sequence row_seq[s * batch + r]; the plan's `past` entry of
  // step s is s * batch (null: row b is sequence b at position past + context_base[b])
  const int* row_seq;
  const int* row_pos;
  DenseGeo dgeo[kNumGemv];     // indexed by StageKind (kRouter unused)
  void* xn;                    // bf16 [B][H]: the RMSNorm output a GEMM stage reads
  float* gemm_part;            // f32 [max tasks][128][B]: partial tiles of split reductions
  unsigned* gemm_cnt;          // [max tiles]: parts of a tile that have arrived (zero between stages)
  const void* tmaps;           // three 128-byte tensor maps over [B][K] bf16 rows: 0 xn, 1 attention output, 2 mlp activations
  // tensor parallelism (tp_world == 1: unused). ar[q] / xchg[q] are rank q's receive
  // regions as mapped into this process; a rank stores into its peers' regions and
  // polls its own. Every 8-byte packet carries its epoch, so no flag or fence is needed.
  int tp_world, tp_rank;
  unsigned long long tp_steps;        // decode steps run on this plan before this launch (equal on all ranks)
  unsigned long long* ar[kMaxTp];     // [2 regions][tp_world sources][B][hidden/2] packets {epoch:32, bf16 pair:32}
  unsigned long long* xchg[kMaxTp];   // [tp_world sources][kMaxBatch] packets {epoch:28, bf16 value:16, index:20}
};

}  // namespace tmb
