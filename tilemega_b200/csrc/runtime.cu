// Host side of the tm_plan_* C ABI (include/tilemega_b200.h): reads the plan
// sidecar, publishes the buffer table, owns the internal device buffers and
// launches the persistent decode kernel. The reference's counterpart is
// include/tilemega/Codegen/tasks/Sm90DenseRuntime.cuh:244-559.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/tilemega_b200.h"
#include "params.h"
#include "encoder.h"
#include "plan_spec.h"

extern "C" int tmb_smem_bytes(const tmb::MegaParams* p);
extern "C" int tmb_prepare_decode(const tmb::MegaParams* p);
extern "C" int tmb_launch_decode(const tmb::MegaParams* p, void* stream);
extern "C" int tmb_launch_decode_ranks(const tmb::MegaParams* first, const tmb::MegaParams* ranks_dev, int count,
                                       int total_grid, void* stream);
extern "C" int tmb_launch_watchdog_probe(const tmb::MegaParams* p, int withhold, void* stream);

namespace {

thread_local std::string g_error;

int Fail(int code, const std::string& message) {
  g_error = message;
  std::fprintf(stderr, "tilemega_b200: %s\n", message.c_str());
  return code;
}

struct Library {
  bool ok = false;
  std::string error;
  std::string sidecar;
  tmb::PlanSpec spec;
};

std::string SidecarPath() {
  if (const char* env = std::getenv("TILEMEGA_PLAN_JSON")) return env;
  Dl_info info{};
  if (dladdr(reinterpret_cast<const void*>(&tm_plan_query), &info) && info.dli_fname)
    return std::string(info.dli_fname) + ".plan.json";
  return "";
}

const Library& Lib() {
  static Library lib;
  static std::once_flag once;
  std::call_once(once, [] {
    try {
      lib.sidecar = SidecarPath();
      std::ifstream in(lib.sidecar);
      if (!in) throw std::invalid_argument("cannot read plan sidecar '" + lib.sidecar + "'");
      std::stringstream text;
      text << in.rdbuf();
      lib.spec = tmb::PlanSpec::FromJson(tmb::Json::Parse(text.str()));
      lib.ok = true;
    } catch (const std::exception& e) {
      lib.error = e.what();
    }
  });
  return lib;
}

// Switch to the plan's device for one call and restore the caller's
// (include/tilemega/Codegen/tasks/Sm90DenseRuntime.cuh:112-119).
class DeviceScope {
 public:
  explicit DeviceScope(int device) {
    cudaGetDevice(&previous_);
    if (previous_ != device) cudaSetDevice(device);
    device_ = device;
  }
  ~DeviceScope() {
    if (previous_ != device_) cudaSetDevice(previous_);
  }

 private:
  int previous_ = 0, device_ = 0;
};

constexpr uint32_t kMagic = 0x544d4232u;  // "TMB2"

struct Plan {
  uint32_t magic = kMagic;
  int device = 0;
  int batch = 0;
  tmb::MegaParams params{};
  std::vector<void*> buffer_ptr;      // per table entry
  std::vector<uint64_t> buffer_bytes;
  std::vector<void*> owned;           // cudaMalloc'd by the plan
  int* past_dev = nullptr;
  uint32_t step_count = 0;
  uint64_t next_iteration[3] = {0, 0, 0};
  int prompt_len = 0;
  size_t smem_bytes = 0;
  unsigned long long* trace_dev = nullptr;
  size_t trace_bytes = 0;
  int trace_step = -1;
  bool tp_bound = false;                // tensor-parallel plan: tm_plan_bind_tp has been called
  uint64_t tp_steps = 0;                // decode steps launched so far (the all-reduce epochs count from it)
  unsigned char* sync_block = nullptr;  // barrier + counters, rezeroed by every launch
  bool abandoned = false;               // a bounded device wait was seen to give up: launches answer -4 until cleared
  tmb::MegaParams* ranks_dev = nullptr; // parameter records of a several-ranks-in-one-launch job (owned by its first plan)
  size_t sync_bytes = 0;
  size_t claim_offset = 0;
  uint32_t prefill_chunks = 0;          // prefill plan: kernel steps (64 rows each) behind its one plan step
  const int* row_seq_dev = nullptr;     // ... its (sequence, position in the prompt) pairs, one per kernel row,
  const int* row_rel_dev = nullptr;
  int* row_abs_dev = nullptr;           // ... and the pairs' positions in the cache, resolved at every launch
  tmb::EncoderPlan* encoder = nullptr;  // forward plan: the encoder's launch graph (none of the decode state above is used)
};

// Position in the cache of every row of a prefill plan: its position in the prompt plus its sequence's
// context_base (an external buffer the caller may change between launches), so that the kernel reads one word
// per row where it would chase two.
__global__ void ResolveRowPositions(const int* rel, const int* seq, const int* base, int* out, int count) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < count) out[r] = rel[r] + (base ? base[seq[r]] : 0);
}

Plan* AsPlan(void* handle) {
  Plan* plan = static_cast<Plan*>(handle);
  return plan && plan->magic == kMagic ? plan : nullptr;
}

uint64_t ElementBytes(uint32_t dtype) {
  return dtype == TM_DTYPE_BF16 || dtype == TM_DTYPE_F16 ? 2 : dtype == TM_DTYPE_E4M3 ? 1 : dtype == TM_DTYPE_I64 ? 8 : 4;
}

cudaError_t Alloc(Plan& plan, void** out, size_t bytes) {
  cudaError_t err = cudaMalloc(out, bytes ? bytes : 16);
  if (err != cudaSuccess) return err;
  plan.owned.push_back(*out);
  return cudaMemset(*out, 0, bytes ? bytes : 16);
}

void Destroy(Plan* plan) {
  DeviceScope scope(plan->device);
  tmb::EncoderDestroy(plan->encoder);
  for (void* p : plan->owned) cudaFree(p);
  plan->magic = 0;
  delete plan;
}

// Tiled tensor map over a row-major bf16 matrix [rows][cols]: boxes of two blocks of `rows` x 64 columns,
// 128-byte swizzle (what tcgen05.mma expects of a K-major operand). The encoder is the driver's; it is looked
// up at run time so that the library has no link-time dependency on the driver library.
const char* EncodeRowsMap(CUtensorMap* map, void* base, uint64_t rows, uint64_t cols) {
  using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = nullptr;
  if (!encode) {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult found{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) != cudaSuccess || !entry ||
        found != cudaDriverEntryPointSuccess)
      return "the driver does not offer cuTensorMapEncodeTiled";
    encode = reinterpret_cast<Encode>(entry);
  }
  // seen as [cols / 64][rows][64]: one copy fetches both 64-column swizzle blocks of a 128-column chunk,
  // block after block in shared memory (coordinates: column in block, row, block)
  const cuuint64_t dims[3] = {64, rows, cols / 64};
  const cuuint64_t strides[2] = {cols * 2, 128};
  const cuuint32_t box[3] = {64, cuuint32_t(rows), 2};
  const cuuint32_t steps[3] = {1, 1, 1};
  const CUresult status = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, steps,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return status == CUDA_SUCCESS ? nullptr : "cuTensorMapEncodeTiled rejected an activation buffer";
}

// What a dense-batch plan needs beyond the table's buffers: tensor maps over the three activation
// buffers its GEMM stages read, and the scratch of split reductions. Returns an error text or null.
const char* BindDense(Plan& plan, const tmb::PlanSpec& s, int batch) {
  tmb::MegaParams& p = plan.params;
  p.xn = plan.buffer_ptr[size_t(s.normed_buf)];
  alignas(64) CUtensorMap maps[3];
  void* const bases[3] = {p.xn, plan.buffer_ptr[size_t(s.attn_buf)], plan.buffer_ptr[size_t(s.mlp_buf)]};
  const uint64_t widths[3] = {uint64_t(s.hidden), uint64_t(s.heads) * s.head_dim, uint64_t(s.inter)};
  for (int i = 0; i < 3; ++i)
    if (const char* why = EncodeRowsMap(&maps[i], bases[i], uint64_t(batch), widths[i])) return why;
  static_assert(sizeof(CUtensorMap) == 128, "the kernel addresses the maps 128 bytes apart");
  void* dev = nullptr;
  if (Alloc(plan, &dev, sizeof(maps)) != cudaSuccess || cudaMemcpy(dev, maps, sizeof(maps), cudaMemcpyHostToDevice) != cudaSuccess)
    return "no device memory for the tensor maps";
  p.tmaps = dev;
  size_t part_tasks = 1, tiles = 1;
  for (int g : {tmb::kQkv, tmb::kOProj, tmb::kGateUp, tmb::kDown, tmb::kHead}) {
    tiles = std::max(tiles, size_t(s.dgeo[g].tiles));
    if (s.dgeo[g].nsplit > 1) part_tasks = std::max(part_tasks, size_t(s.dgeo[g].ntasks));
  }
  void *part = nullptr, *count = nullptr;
  if (Alloc(plan, &part, part_tasks * tmb::kDenseTileN * size_t(batch) * sizeof(float)) != cudaSuccess ||
      Alloc(plan, &count, tiles * sizeof(unsigned)) != cudaSuccess)
    return "no device memory for the split-reduction scratch";
  p.gemm_part = static_cast<float*>(part);
  p.gemm_cnt = static_cast<unsigned*>(count);
  return nullptr;
}

}  // namespace

extern "C" {

const char* tm_plan_last_error(void) { return g_error.c_str(); }

int tm_plan_query(tm_plan_info* out) {
  if (!out) return Fail(-1, "tm_plan_query: null output");
  const Library& lib = Lib();
  if (!lib.ok) return Fail(-1, "tm_plan_query: " + lib.error);
  const tmb::PlanSpec& s = lib.spec;
  std::memset(out, 0, sizeof(*out));
  out->abi_version = TM_SERVING_ABI_VERSION;
  out->phase = s.forward ? TM_SERVING_FORWARD : s.prefill ? TM_SERVING_PREFILL : TM_SERVING_DECODE;
  out->batch_lo = s.batch_lo;
  out->batch_hi = s.batch_hi;
  out->seq = s.forward ? s.forward_seq : s.prefill ? s.prefill_seq : 1;
  out->past_lo = 0;
  out->past_hi = s.prefill || s.forward ? 0 : s.capacity - 1;
  out->capacity = s.capacity;
  out->grid = s.grid;  // 0: one CTA per SM of the device the plan is created on
  out->residency = 1;
  out->modes = TM_SERVING_L1 | TM_SERVING_L2;
  out->buffer_count = uint32_t(s.buffers.size());
  return 0;
}

int tm_plan_buffer(uint32_t index, tm_buffer_info* out) {
  if (!out) return Fail(-1, "tm_plan_buffer: null output");
  const Library& lib = Lib();
  if (!lib.ok) return Fail(-1, "tm_plan_buffer: " + lib.error);
  if (index >= lib.spec.buffers.size()) return Fail(-1, "tm_plan_buffer: index out of range");
  const tmb::BufferSpec& b = lib.spec.buffers[index];
  out->name = b.name.c_str();
  out->role = b.role;
  out->dtype = b.dtype;
  out->elements_constant = b.elements_constant;
  out->elements_per_batch = b.elements_per_batch;
  out->pack_json = b.pack_json.empty() ? nullptr : b.pack_json.c_str();
  return 0;
}

void* tm_plan_create(int batch, void* const* external, int device) {
  const Library& lib = Lib();
  if (!lib.ok) {
    Fail(-1, "tm_plan_create: " + lib.error);
    return nullptr;
  }
  const tmb::PlanSpec& s = lib.spec;
  if (batch < s.batch_lo || batch > s.batch_hi || !external) {
    Fail(-1, "tm_plan_create: batch outside the plan's interval or null buffer list");
    return nullptr;
  }
  int device_count = 0;
  if (cudaGetDeviceCount(&device_count) != cudaSuccess || device < 0 || device >= device_count) {
    Fail(-1, "tm_plan_create: no such CUDA device (this library has no CPU path)");
    return nullptr;
  }
  for (size_t i = 0; i < s.buffers.size(); ++i) {
    if (s.buffers[i].role == TM_BUFFER_EXTERNAL && !external[i]) {
      Fail(-1, "tm_plan_create: external buffer '" + s.buffers[i].name + "' is null");
      return nullptr;
    }
    if (s.buffers[i].role == TM_BUFFER_EXTERNAL && (reinterpret_cast<uintptr_t>(external[i]) & 15u)) {
      Fail(-1, "tm_plan_create: external buffer '" + s.buffers[i].name + "' is not 16-byte aligned");
      return nullptr;
    }
  }
  if (s.dense_batch && !s.prefill && batch % 16) {
    Fail(-1, "tm_plan_create: a dense-batch plan runs batch sizes 16, 32, 48 or 64");
    return nullptr;
  }
  // rows of the kernel's batch: the sequences themselves, except in a prefill plan, whose `batch` sequences of
  // `seq` positions run as (sequence, position) rows, kDenseMaxBatch per kernel step
  const int seqs = batch;
  const int rows = s.prefill ? tmb::kDenseMaxBatch : batch;
  DeviceScope scope(device);
  cudaDeviceProp prop{};
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major < 10) {
    Fail(-1, "tm_plan_create: the kernels are built for sm_100a only");
    return nullptr;
  }
  auto plan = std::unique_ptr<Plan, void (*)(Plan*)>(new Plan, Destroy);
  plan->device = device;
  plan->batch = batch;
  plan->buffer_ptr.assign(s.buffers.size(), nullptr);
  plan->buffer_bytes.assign(s.buffers.size(), 0);
  auto fail = [&](const std::string& what, cudaError_t err) -> void* {
    Fail(int(err), "tm_plan_create: " + what + ": " + cudaGetErrorString(err));
    return nullptr;
  };
  for (size_t i = 0; i < s.buffers.size(); ++i) {
    const tmb::BufferSpec& b = s.buffers[i];
    plan->buffer_bytes[i] = (b.elements_constant + uint64_t(batch) * b.elements_per_batch) * ElementBytes(b.dtype);
    if (b.role == TM_BUFFER_EXTERNAL) {
      plan->buffer_ptr[i] = external[i];
    } else {
      cudaError_t err = Alloc(*plan, &plan->buffer_ptr[i], plan->buffer_bytes[i]);
      if (err != cudaSuccess) return fail("allocating " + b.name, err);
    }
  }
  if (s.forward) {
    // a stateless encoder pass: the launch graph over the table's buffers is all the plan holds
    std::string why;
    plan->encoder = tmb::EncoderCreate(s, batch, plan->buffer_ptr, prop.multiProcessorCount, &why);
    if (!plan->encoder) {
      Fail(-1, "tm_plan_create: " + why);
      return nullptr;
    }
    plan->step_count = 1;
    return plan.release();
  }
  tmb::MegaParams& p = plan->params;
  p.batch = rows;
  p.hidden = s.hidden;
  p.inter = s.inter;
  p.heads = s.heads;
  p.kv_heads = s.kv_heads;
  p.head_dim = s.head_dim;
  p.layers = s.layers;
  p.vocab = s.vocab;
  p.head_base = 0;   // set by tm_plan_bind_tp for a tensor-parallel plan
  p.tp_world = s.tp;
  p.tp_rank = 0;
  p.experts = s.experts;
  p.topk = s.topk;
  p.norm_topk = s.norm_topk ? 1 : 0;
  p.qk_norm = s.qk_norm ? 1 : 0;
  p.stages_per_layer = s.stages_per_layer(rows);
  p.dense = s.dense_batch ? 1 : 0;
  p.chunk_rows = s.chunk_rows ? 1 : 0;
  // a traced step: one record per stage; dense-batch plans have 7 per layer (two RMSNorm stages) and norm + head at the end
  p.trace_stages = s.dense_batch ? 7 * s.layers + 2 : s.stages_per_layer(rows) * s.layers + 1;
  // grid-wide arrivals of a step: one per stage except QKV (attention tasks wait per KV-head group)
  // plus the argmax hand-over; a dense-batch plan's RMSNorm stages arrive too
  // (with chunk_rows also the QKV stage and the append stage that follows it)
  p.bars_per_step = s.dense_batch ? (s.chunk_rows ? 8 : 6) * s.layers + 2 : (s.stages_per_layer(rows) - 1) * s.layers + 1;
  for (int g = 0; g < tmb::kNumGemv; ++g) p.dgeo[g] = s.dgeo[g];
  p.eps = float(s.eps);
  p.qk_scale_log2 = float(1.4426950408889634 / std::sqrt(double(s.head_dim)));
  p.capacity = s.capacity;
  p.max_blocks = s.max_blocks;
  p.first_step = 0;
  p.nsteps = 0;
  p.prompt_len = 0;
  p.write_logits = s.write_logits ? 1 : 0;
  p.grid = s.grid > 0 ? std::min(s.grid, prop.multiProcessorCount) : prop.multiProcessorCount;
  for (int g = 0; g < tmb::kNumGemv; ++g) p.geo[g] = s.geo[g];
  p.down_splits = s.down_splits;
  for (int i = 0; i < tmb::kMaxDownSplits; ++i) p.down_part[i] = s.down_part[i];
  p.bar_base = 0;
  const char* watchdog = std::getenv("TILEMEGA_WATCHDOG_MS");
  const double watchdog_ms = watchdog ? std::atof(watchdog) : 2000.0;
  p.watchdog_ns = (unsigned long long)(std::max(watchdog_ms, 0.001) * 1e6);
  // shared memory: activation rows (or the attention scratch, whichever is larger) + ring
  const int gq = s.heads / s.kv_heads;   // query heads per KV head (4 or 8)
  // roped q, new k and v, the warps' partial states, and the QK-normalised q/k rows
  const int attention_scratch = gq * s.head_dim * 2 + 2 * s.head_dim * 2 + 8 * gq * (s.head_dim + 2) * 4 +
                                (gq + 1) * s.head_dim * 2 + 64;
  // mixture of experts: the down stage stages one activation row per chosen expert
  const int expert_rows = s.experts ? s.topk * (s.geo[tmb::kDown].k + 8) * 2 : 0;
  // rows of the widest GEMV input; one extra hidden-wide row holds the RMSNorm weights
  // (rows are padded by 8 elements so that the batch rows of a k-chunk sit on distinct banks)
  // a normalised stage also parks its raw rows and the norm weights there: 2*batch + 1 hidden-wide rows
  // (batch > 4: the rows are normalised in a second pass over global memory instead: batch + 1 rows)
  int xs = std::max({rows * (s.max_k() + 8) * 2, (rows > 4 ? rows + 1 : 2 * rows + 1) * (s.geo[tmb::kQkv].k + 8) * 2, attention_scratch,
                     expert_rows});
  // dense-batch: the activation chunks of the GEMM stages (batch x 128 columns each) share the area
  // with the attention scratch; chunks must start on 1024-byte boundaries (128-byte swizzle)
  // (their attention tasks also hold the summed q, k, v rows of one KV head: gq + 2 more rows)
  if (s.dense_batch)
    xs = std::max(attention_scratch + (gq + 2) * s.head_dim * 2, tmb::dense_x_slots(rows) * rows * tmb::kDenseTileK * 2);
  xs = s.dense_batch ? (xs + 1023) & ~1023 : (xs + 127) & ~127;
  p.xs_bytes = xs;
  p.attn_min_spt = s.attn_min_slots;
  const int limit = int(prop.sharedMemPerBlockOptin);
  p.nslots = tmb::kMaxSlots;
  if (s.slots > 0) p.nslots = std::min(s.slots, tmb::kMaxSlots);
  while (p.nslots > 0 && tmb_smem_bytes(&p) > limit) --p.nslots;
  if (p.nslots < 2) {
    Fail(-1, "tm_plan_create: activation rows leave no room for a two-slot ring in shared memory");
    return nullptr;
  }
  plan->smem_bytes = size_t(tmb_smem_bytes(&p));
  // request state
  p.tokens = static_cast<int*>(plan->buffer_ptr[s.tokens]);
  p.rope_cos = plan->buffer_ptr[s.rope_cos];
  p.rope_sin = plan->buffer_ptr[s.rope_sin];
  const uint64_t D = s.head_dim;
  if (s.paged) {
    p.block_table = static_cast<const int*>(plan->buffer_ptr[s.block_table]);
    p.ctx_base = static_cast<const int*>(plan->buffer_ptr[s.context_base]);
    p.kv_block_stride = (long long)(s.kv_heads * tmb::kKvBlock * D);
    p.kv_head_stride = (long long)(tmb::kKvBlock * D);
    p.kv_max_entry = s.num_blocks - 1;
  } else {
    // The reference's contiguous [B][Hkv][capacity][D] cache seen as blocks of
    // 16 rows: entry (b, j) = b*Hkv*capacity/16 + j, heads capacity*D apart
    // (python/tilemega/serving/state.py:86-98).
    const int per_head = s.capacity / tmb::kKvBlock;
    std::vector<int> table(size_t(seqs) * s.max_blocks);
    for (int b = 0; b < seqs; ++b)
      for (int j = 0; j < s.max_blocks; ++j) table[size_t(b) * s.max_blocks + j] = b * s.kv_heads * per_head + j;
    void* dev = nullptr;
    cudaError_t err = Alloc(*plan, &dev, table.size() * sizeof(int));
    if (err == cudaSuccess) err = cudaMemcpy(dev, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return fail("block table", err);
    p.block_table = static_cast<const int*>(dev);
    p.ctx_base = nullptr;
    p.kv_block_stride = (long long)(tmb::kKvBlock * D);
    p.kv_head_stride = (long long)(uint64_t(s.capacity) * D);
    p.kv_max_entry = ((seqs - 1) * s.kv_heads + 1) * per_head - 1;
  }
  p.embed = plan->buffer_ptr[s.embed];
  p.final_norm = plan->buffer_ptr[s.final_norm];
  p.lm_head = plan->buffer_ptr[s.lm_head];
  p.fp8 = s.fp8 ? 1 : 0;
  p.lm_head_scale = s.fp8 ? static_cast<const float*>(plan->buffer_ptr[size_t(s.lm_head_scale)]) : nullptr;
  std::vector<tmb::LayerPtrs> layers(size_t(s.layers));
  for (int l = 0; l < s.layers; ++l) {
    const tmb::LayerBuffers& lb = s.layer[size_t(l)];
    auto optional = [&](int index) -> const void* { return index >= 0 ? plan->buffer_ptr[size_t(index)] : nullptr; };
    auto scale = [&](int index) { return static_cast<const float*>(optional(index)); };
    layers[size_t(l)] = tmb::LayerPtrs{scale(lb.qkv_scale),        scale(lb.o_scale),          scale(lb.gate_up_scale),
                                       scale(lb.down_scale),       plan->buffer_ptr[lb.qkv],   plan->buffer_ptr[lb.o],
                                       plan->buffer_ptr[lb.gate_up], plan->buffer_ptr[lb.down], plan->buffer_ptr[lb.norm1],
                                       plan->buffer_ptr[lb.norm2], optional(lb.router),        optional(lb.q_norm),
                                       optional(lb.k_norm),        plan->buffer_ptr[lb.k],     plan->buffer_ptr[lb.v]};
  }
  {
    void* dev = nullptr;
    cudaError_t err = Alloc(*plan, &dev, layers.size() * sizeof(tmb::LayerPtrs));
    if (err == cudaSuccess)
      err = cudaMemcpy(dev, layers.data(), layers.size() * sizeof(tmb::LayerPtrs), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return fail("layer table", err);
    p.layer = static_cast<const tmb::LayerPtrs*>(dev);
  }
  p.x = plan->buffer_ptr[s.hidden_buf];
  p.qkv = plan->buffer_ptr[s.qkv_buf];
  p.attn = plan->buffer_ptr[s.attn_buf];
  p.h = plan->buffer_ptr[s.mlp_buf];
  p.logits = plan->buffer_ptr[s.logits_buf];
  if (s.experts) {
    p.router_logits = plan->buffer_ptr[s.router_buf];
    p.route_idx = static_cast<int*>(plan->buffer_ptr[s.route_idx_buf]);
    p.route_w = static_cast<float*>(plan->buffer_ptr[s.route_weight_buf]);
  }
  // scratch
  struct Scratch {
    void** out;
    size_t bytes;
  };
  void *down_partial = nullptr, *attn_part = nullptr, *argmax_val = nullptr, *argmax_idx = nullptr, *status = nullptr,
       *step_ns = nullptr, *past = nullptr;
  const size_t attn_tasks = 2 * size_t(p.grid) + size_t(rows) * s.kv_heads + 2;
  p.attn_part_tasks = int(attn_tasks);
  const Scratch scratch[] = {
      {&down_partial, size_t(rows) * s.hidden * sizeof(float)},
      {&attn_part, attn_tasks * gq * (s.head_dim + 2) * sizeof(float)},
      {&argmax_val, size_t(p.grid) * rows * sizeof(float)},
      {&argmax_idx, size_t(p.grid) * rows * sizeof(int)},
      {&status, tmb::kStWords * sizeof(unsigned long long)},
      {&step_ns, size_t(s.capacity + 2) * sizeof(unsigned long long)},
      {&past, size_t(s.capacity) * sizeof(int)},
  };
  for (const Scratch& item : scratch) {
    cudaError_t err = Alloc(*plan, item.out, item.bytes);
    if (err != cudaSuccess) return fail("scratch", err);
  }
  // barrier word, then the attention arrival counters: one block, rezeroed per launch
  const size_t attn_cnt = size_t(rows) * s.kv_heads;
  // ... and the task claim counters of every stage instance of the longest possible launch
  const size_t stage_cnt = size_t(s.capacity) * (size_t(s.stages_per_layer(rows)) * size_t(s.layers) + 1) + 2;   // + the two look-ahead claims past the last stage
  const size_t ready_offset = (128 + attn_cnt * sizeof(unsigned) + 7) & ~size_t(7);
  plan->claim_offset = ready_offset + size_t(s.kv_heads) * sizeof(unsigned long long);
  plan->sync_bytes = plan->claim_offset + stage_cnt * sizeof(unsigned);
  {
    void* dev = nullptr;
    cudaError_t err = Alloc(*plan, &dev, plan->sync_bytes);
    if (err != cudaSuccess) return fail("counters", err);
    plan->sync_block = static_cast<unsigned char*>(dev);
  }
  p.bar = reinterpret_cast<unsigned long long*>(plan->sync_block);
  p.attn_cnt = reinterpret_cast<unsigned*>(plan->sync_block + 128);
  p.qkv_ready = reinterpret_cast<unsigned long long*>(plan->sync_block + ready_offset);
  p.stage_cnt = reinterpret_cast<unsigned*>(plan->sync_block + plan->claim_offset);
  if (s.dense_batch) {
    if (const char* why = BindDense(*plan, s, rows)) {
      Fail(-1, std::string("tm_plan_create: ") + why);
      return nullptr;
    }
  }
  p.down_partial = static_cast<float*>(down_partial);
  p.attn_part = static_cast<float*>(attn_part);
  p.argmax_val = static_cast<float*>(argmax_val);
  p.argmax_idx = static_cast<int*>(argmax_idx);
  p.status = static_cast<unsigned long long*>(status);
  p.step_ns = static_cast<unsigned long long*>(step_ns);
  plan->past_dev = static_cast<int*>(past);
  p.past = plan->past_dev;
  p.row_seq = p.row_pos = nullptr;
  if (s.prefill) {
    // The plan's one step covers seqs * seq (sequence, position) pairs: kernel step c takes pairs [c * rows,
    // (c + 1) * rows), sequences in order and positions ascending, so that a position's predecessors lie in the
    // same or an earlier kernel step; the last step's spare rows repeat the last pair (they recompute and
    // rewrite exactly what that pair writes). `past` of kernel step c is c * rows, the offset of its pairs.
    const int total = seqs * s.prefill_seq;
    const int chunks = (total + rows - 1) / rows;
    if (chunks > s.capacity) return fail("prefill plan", cudaErrorInvalidValue);
    std::vector<int> map, first;
    map.resize(size_t(2) * chunks * rows);
    first.resize(size_t(chunks));
    for (int r = 0; r < chunks * rows; ++r) {
      const int pair = std::min(r, total - 1);
      map[size_t(r)] = pair / s.prefill_seq;
      map[size_t(chunks) * rows + r] = pair % s.prefill_seq;
    }
    for (int ck = 0; ck < chunks; ++ck) first[size_t(ck)] = ck * rows;
    void* dev = nullptr;
    void* resolved = nullptr;
    cudaError_t err = Alloc(*plan, &dev, map.size() * sizeof(int));
    if (err == cudaSuccess) err = Alloc(*plan, &resolved, size_t(chunks) * rows * sizeof(int));
    if (err == cudaSuccess) err = cudaMemcpy(dev, map.data(), map.size() * sizeof(int), cudaMemcpyHostToDevice);
    if (err == cudaSuccess) err = cudaMemcpy(plan->past_dev, first.data(), first.size() * sizeof(int), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return fail("prefill row map", err);
    plan->row_seq_dev = static_cast<const int*>(dev);
    plan->row_rel_dev = plan->row_seq_dev + size_t(chunks) * rows;
    plan->row_abs_dev = static_cast<int*>(resolved);
    p.row_seq = plan->row_seq_dev;
    p.row_pos = plan->row_abs_dev;      // filled by ResolveRowPositions at every launch
    plan->prefill_chunks = uint32_t(chunks);
    plan->prompt_len = s.prefill_seq;   // positions before the prompt's end keep the caller's tokens
  }
  {
    const int status = tmb_prepare_decode(&p);
    if (status != 0) return fail("the persistent grid does not fit the device", cudaError_t(status));
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return fail("initialisation", cudaGetLastError());
  return plan.release();
}

int tm_plan_set_steps(void* handle, const int32_t* past, uint32_t count) {
  Plan* plan = AsPlan(handle);
  if (!plan || !past || count == 0) return Fail(-1, "tm_plan_set_steps: bad argument");
  const tmb::MegaParams& p = plan->params;
  if (plan->encoder) {
    // a forward plan has ONE step, at past 0 (include/tilemega/Codegen/tasks/Sm90F3Runtime.cuh:121-123)
    if (count != 1 || past[0] != 0) return Fail(-2, "tm_plan_set_steps: a forward plan has one step, at past 0");
    return 0;
  }
  if (plan->prefill_chunks) {
    // a prefill plan has ONE step, at past 0 (python/tilemega/serving/engine.py:89-90 sets exactly that)
    if (count != 1 || past[0] != 0) return Fail(-2, "tm_plan_set_steps: a prefill plan has one step, at past 0");
    plan->step_count = 1;
    return 0;
  }
  if (count > uint32_t(p.capacity)) return Fail(-2, "tm_plan_set_steps: more steps than the plan's capacity");
  for (uint32_t i = 0; i < count; ++i)
    if (past[i] < 0 || past[i] >= p.capacity) return Fail(-2, "tm_plan_set_steps: position outside [0, capacity)");
  DeviceScope scope(plan->device);
  cudaError_t err = cudaMemcpy(plan->past_dev, past, size_t(count) * sizeof(int32_t), cudaMemcpyHostToDevice);
  if (err != cudaSuccess) return Fail(int(err), std::string("tm_plan_set_steps: ") + cudaGetErrorString(err));
  plan->step_count = count;
  return 0;
}

int tm_plan_set_prompt_len(void* handle, int prompt_len) {
  Plan* plan = AsPlan(handle);
  if (!plan || prompt_len < 0 || prompt_len > plan->params.capacity)
    return Fail(-1, "tm_plan_set_prompt_len: bad argument");
  if (plan->prefill_chunks) return Fail(-1, "tm_plan_set_prompt_len: a prefill plan's prompt length is its seq");
  if (plan->encoder) return Fail(-1, "tm_plan_set_prompt_len: a forward plan has no prompt");
  plan->prompt_len = prompt_len;
  return 0;
}

}  // extern "C"

namespace {

// Everything a launch of `steps` steps checks and prepares before the kernel goes out:
// the argument and iteration rules, the counters rezeroed on the stream, the parameter
// record of this launch in `out`. Returns 0 or the error code to hand back.
int PrepareLaunch(Plan* plan, const char* who, uint32_t first_step, uint32_t steps, uint32_t mode, uint64_t base_iteration,
                  cudaStream_t s, tmb::MegaParams* out) {
  const std::string name = who;
  if (!plan || steps == 0) return Fail(-1, name + ": bad argument");
  if (mode != TM_SERVING_L1 && mode != TM_SERVING_L2) return Fail(-3, name + ": unknown mode");
  if (plan->abandoned)
    return Fail(-4, name + ": a bounded device wait gave up on this plan; read tm_plan_watchdog, then tm_plan_clear_watchdog");
  if (uint64_t(first_step) + steps > plan->step_count)
    return Fail(-2, name + ": steps outside the interval given to tm_plan_set_steps");
  // a prefill plan's one step is prefill_chunks kernel steps
  const uint32_t kernel_steps = plan->prefill_chunks ? plan->prefill_chunks : steps;
  if (base_iteration != plan->next_iteration[mode])
    return Fail(-2, name + ": iteration is not the number of previous launches of this mode");
  if (plan->params.tp_world > 1 && !plan->tp_bound)
    return Fail(-1, name + ": a tensor-parallel plan must be bound with tm_plan_bind_tp first");
  // only the claim counters this launch can touch are rezeroed
  const size_t used = plan->claim_offset +
                      (size_t(kernel_steps) * (size_t(plan->params.stages_per_layer) * size_t(plan->params.layers) + 1) + 2) * sizeof(unsigned);
  cudaError_t err = cudaMemsetAsync(plan->sync_block, 0, used, s);
  if (err != cudaSuccess) return Fail(int(err), name + ": " + cudaGetErrorString(err));
  if (plan->prefill_chunks) {
    const int count = int(plan->prefill_chunks) * plan->params.batch;
    ResolveRowPositions<<<(count + 255) / 256, 256, 0, s>>>(plan->row_rel_dev, plan->row_seq_dev, plan->params.ctx_base,
                                                            plan->row_abs_dev, count);
    err = cudaGetLastError();
    if (err != cudaSuccess) return Fail(int(err), name + ": " + cudaGetErrorString(err));
  }
  *out = plan->params;
  out->tp_steps = plan->tp_steps;
  out->first_step = int(first_step);
  out->nsteps = int(kernel_steps);
  out->prompt_len = plan->prompt_len;
  out->trace = plan->trace_step >= 0 ? plan->trace_dev : nullptr;
  out->trace_step = plan->trace_step;
  return 0;
}

void Launched(Plan* plan, uint32_t steps, uint32_t mode) {
  plan->next_iteration[mode] += steps;
  plan->tp_steps += steps;
}

}  // namespace

extern "C" {

int tm_plan_launch_steps(void* handle, uint32_t first_step, uint32_t steps, uint32_t mode, uint64_t base_iteration,
                         void* stream) {
  Plan* plan = AsPlan(handle);
  if (!plan) return Fail(-1, "tm_plan_launch_steps: bad argument");
  DeviceScope scope(plan->device);
  if (plan->encoder) {
    // one stateless pass; both executor modes run the same graph (their outputs are bit-identical by construction)
    if (first_step != 0 || steps != 1) return Fail(-2, "tm_plan_launch_steps: a forward plan has one step");
    if (mode != TM_SERVING_L1 && mode != TM_SERVING_L2) return Fail(-3, "tm_plan_launch_steps: unknown mode");
    if (plan->abandoned) return Fail(-4, "tm_plan_launch_steps: the plan was abandoned by a bounded wait; clear the watchdog first");
    const int status = tmb::EncoderLaunch(plan->encoder, static_cast<cudaStream_t>(stream));
    return status == 0 ? 0 : Fail(status, std::string("tm_plan_launch_steps: ") + cudaGetErrorString(cudaError_t(status)));
  }
  tmb::MegaParams p;
  const int ready = PrepareLaunch(plan, "tm_plan_launch_steps", first_step, steps, mode, base_iteration,
                                  static_cast<cudaStream_t>(stream), &p);
  if (ready != 0) return ready;
  const int status = tmb_launch_decode(&p, stream);
  if (status != 0)
    return Fail(status, std::string("tm_plan_launch_steps: ") + cudaGetErrorString(cudaError_t(status)));
  Launched(plan, steps, mode);
  return 0;
}

int tm_plan_launch_steps_ranks(void* const* handles, uint32_t count, uint32_t first_step, uint32_t steps, uint32_t mode,
                               uint64_t base_iteration, void* stream) {
  if (!handles || count < 2 || count > uint32_t(tmb::kMaxTp)) return Fail(-1, "tm_plan_launch_steps_ranks: bad argument");
  std::vector<Plan*> plans;
  for (uint32_t q = 0; q < count; ++q) {
    Plan* plan = AsPlan(handles[q]);
    if (!plan) return Fail(-1, "tm_plan_launch_steps_ranks: bad plan");
    plans.push_back(plan);
  }
  Plan* lead = plans[0];
  int total_grid = 0;
  for (uint32_t q = 0; q < count; ++q) {
    const tmb::MegaParams& p = plans[q]->params;
    if (plans[q]->device != lead->device || p.tp_world != int(count) || p.tp_rank != int(q) || p.batch != lead->params.batch ||
        plans[q]->smem_bytes != lead->smem_bytes)
      return Fail(-1, "tm_plan_launch_steps_ranks: the plans must be ranks 0..count-1 of one job, in order, on one device");
    total_grid += p.grid;
  }
  DeviceScope scope(lead->device);
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, lead->device);
  if (total_grid > sms)
    return Fail(-1, "tm_plan_launch_steps_ranks: the ranks' grids together exceed the device's SMs (emit the plans with a smaller \"grid\")");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!lead->ranks_dev) {
    void* dev = nullptr;
    cudaError_t err = Alloc(*lead, &dev, size_t(tmb::kMaxTp) * sizeof(tmb::MegaParams));
    if (err != cudaSuccess) return Fail(int(err), std::string("tm_plan_launch_steps_ranks: ") + cudaGetErrorString(err));
    lead->ranks_dev = static_cast<tmb::MegaParams*>(dev);
  }
  std::vector<tmb::MegaParams> records(count);
  for (uint32_t q = 0; q < count; ++q) {
    const int ready = PrepareLaunch(plans[q], "tm_plan_launch_steps_ranks", first_step, steps, mode, base_iteration, s, &records[q]);
    if (ready != 0) return ready;
  }
  // stream-ordered after the previous launch, which may still be reading its records
  cudaError_t err = cudaMemcpyAsync(lead->ranks_dev, records.data(), records.size() * sizeof(tmb::MegaParams),
                                    cudaMemcpyHostToDevice, s);
  if (err != cudaSuccess) return Fail(int(err), std::string("tm_plan_launch_steps_ranks: ") + cudaGetErrorString(err));
  const int status = tmb_launch_decode_ranks(&records[0], lead->ranks_dev, int(count), total_grid, stream);
  if (status != 0)
    return Fail(status, std::string("tm_plan_launch_steps_ranks: ") + cudaGetErrorString(cudaError_t(status)));
  for (Plan* plan : plans) Launched(plan, steps, mode);
  return 0;
}

int tm_plan_launch(void* handle, uint32_t step, uint32_t mode, uint64_t iteration, void* stream) {
  return tm_plan_launch_steps(handle, step, 1, mode, iteration, stream);
}

unsigned tm_plan_loop_modes(void* handle) { return AsPlan(handle) ? (TM_SERVING_L1 | TM_SERVING_L2) : 0u; }

int tm_plan_read_step_ns(void* handle, uint32_t first, uint32_t count, uint64_t* host) {
  Plan* plan = AsPlan(handle);
  if (!plan || !host || plan->encoder || uint64_t(first) + count > uint64_t(plan->params.capacity) + 2)
    return Fail(-1, "tm_plan_read_step_ns: bad argument");
  DeviceScope scope(plan->device);
  cudaError_t err =
      cudaMemcpy(host, plan->params.step_ns + first, size_t(count) * sizeof(uint64_t), cudaMemcpyDeviceToHost);
  return err == cudaSuccess ? 0 : Fail(int(err), std::string("tm_plan_read_step_ns: ") + cudaGetErrorString(err));
}

int tm_plan_read_buffer(void* handle, uint32_t index, void* host, uint64_t bytes) {
  Plan* plan = AsPlan(handle);
  if (!plan || !host || index >= plan->buffer_ptr.size() || bytes > plan->buffer_bytes[index])
    return Fail(-1, "tm_plan_read_buffer: bad argument");
  DeviceScope scope(plan->device);
  cudaError_t err = cudaMemcpy(host, plan->buffer_ptr[index], size_t(bytes), cudaMemcpyDeviceToHost);
  return err == cudaSuccess ? 0 : Fail(int(err), std::string("tm_plan_read_buffer: ") + cudaGetErrorString(err));
}

int tm_plan_watchdog(void* handle, uint64_t* record12) {
  Plan* plan = AsPlan(handle);
  if (!plan || !record12) return 0;
  DeviceScope scope(plan->device);
  if (plan->encoder) {
    const int fired = tmb::EncoderStatus(plan->encoder, record12);
    if (fired > 0) plan->abandoned = true;
    return fired > 0 ? 1 : 0;
  }
  unsigned long long words[tmb::kStWords] = {};
  if (cudaMemcpy(words, plan->params.status, sizeof(words), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
  for (int i = 0; i < 12; ++i) record12[i] = words[i];
  if (words[tmb::kStFired]) plan->abandoned = true;   // launches answer -4 until tm_plan_clear_watchdog
  return words[tmb::kStFired] ? 1 : 0;
}

int tm_plan_clear_watchdog(void* handle) {
  Plan* plan = AsPlan(handle);
  if (!plan) return Fail(-1, "tm_plan_clear_watchdog: bad plan");
  DeviceScope scope(plan->device);
  if (plan->encoder) {
    tmb::EncoderClear(plan->encoder);
    plan->abandoned = false;
    return 0;
  }
  cudaError_t err = cudaMemset(plan->params.status, 0, tmb::kStWords * sizeof(unsigned long long));
  if (err == cudaSuccess) plan->abandoned = false;
  return err == cudaSuccess ? 0 : Fail(int(err), cudaGetErrorString(err));
}

int tm_plan_watchdog_probe(void* handle, int withhold, uint32_t limit_us, void* stream) {
  Plan* plan = AsPlan(handle);
  if (!plan || plan->encoder || limit_us == 0 || limit_us > 1000000u) return Fail(-1, "tm_plan_watchdog_probe: bad argument");
  DeviceScope scope(plan->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemsetAsync(plan->sync_block, 0, plan->sync_bytes, s);
  if (err == cudaSuccess) err = cudaMemsetAsync(plan->params.status, 0, tmb::kStWords * sizeof(unsigned long long), s);
  if (err != cudaSuccess) return Fail(int(err), cudaGetErrorString(err));
  tmb::MegaParams p = plan->params;
  p.watchdog_ns = (unsigned long long)limit_us * 1000ull;
  const int status = tmb_launch_watchdog_probe(&p, withhold, stream);
  if (status != 0) return Fail(status, cudaGetErrorString(cudaError_t(status)));
  err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) return Fail(int(err), cudaGetErrorString(err));
  uint64_t record[12];
  const int fired = tm_plan_watchdog(handle, record);
  if (withhold != 2) tm_plan_clear_watchdog(handle);   // 2: the record stays, as after a real abandoned launch
  return fired;
}

int tm_plan_trace_step(void* handle, int step) {
  Plan* plan = AsPlan(handle);
  if (!plan || plan->encoder) return Fail(-1, "tm_plan_trace_step: bad plan");
  DeviceScope scope(plan->device);
  if (step >= 0 && !plan->trace_dev) {
    plan->trace_bytes = size_t(plan->params.grid) * size_t(plan->params.trace_stages) * 4 * sizeof(unsigned long long);
    void* dev = nullptr;
    cudaError_t err = Alloc(*plan, &dev, plan->trace_bytes);
    if (err != cudaSuccess) return Fail(int(err), cudaGetErrorString(err));
    plan->trace_dev = static_cast<unsigned long long*>(dev);
  }
  plan->trace_step = step;
  return 0;
}

long long tm_plan_read_trace(void* handle, uint64_t* host, uint64_t bytes) {
  Plan* plan = AsPlan(handle);
  if (!plan || !plan->trace_dev) return Fail(-1, "tm_plan_read_trace: no trace was requested");
  if (!host) return (long long)plan->trace_bytes;
  if (bytes < plan->trace_bytes) return Fail(-1, "tm_plan_read_trace: buffer too small");
  DeviceScope scope(plan->device);
  cudaError_t err = cudaMemcpy(host, plan->trace_dev, plan->trace_bytes, cudaMemcpyDeviceToHost);
  return err == cudaSuccess ? (long long)plan->trace_bytes : Fail(int(err), cudaGetErrorString(err));
}

unsigned tm_plan_pdl_enabled(void*) { return 0; }

uint64_t tm_plan_execution_smem(void* handle, unsigned) {
  Plan* plan = AsPlan(handle);
  return plan ? plan->smem_bytes : 0;
}

uint64_t tm_plan_step_bytes(void* handle, uint64_t cached_tokens_total) {
  Plan* plan = AsPlan(handle);
  if (!plan) return 0;
  const tmb::PlanSpec& s = Lib().spec;
  return s.weight_bytes() + s.kv_bytes_per_token() * cached_tokens_total;
}

// Tensor parallelism (include/tilemega/Codegen/tasks/ServingAbi.h:53-55). The caller
// allocates, zeroes and owns one all-reduce region (which = 0) and one argmax exchange
// block (which = 1) per rank, on that rank's device, and hands every rank the list of all
// of them as pointers valid in the calling process.
unsigned tm_plan_tp_world(void) {
  const Library& lib = Lib();
  return lib.ok ? unsigned(lib.spec.tp) : 1u;
}

unsigned long long tm_plan_tp_bytes(unsigned which) {
  const Library& lib = Lib();
  if (!lib.ok || lib.spec.tp < 2) return 0;
  const tmb::PlanSpec& s = lib.spec;
  if (which == 0) return 2ull * s.tp * s.batch_hi * (uint64_t(s.hidden) / 2) * 8ull;   // two regions of 8-byte packets
  if (which == 1) return uint64_t(s.tp) * tmb::kMaxBatch * 8ull;
  return 0;
}

int tm_plan_bind_tp(void* handle, int rank, void* const* ar, void* const* x) {
  Plan* plan = AsPlan(handle);
  if (!plan || !ar || !x) return Fail(-1, "tm_plan_bind_tp: bad argument");
  tmb::MegaParams& p = plan->params;
  if (p.tp_world < 2) return Fail(-1, "tm_plan_bind_tp: this plan is not tensor parallel");
  if (rank < 0 || rank >= p.tp_world) return Fail(-1, "tm_plan_bind_tp: rank outside the plan's degree");
  if (plan->tp_steps != 0) return Fail(-2, "tm_plan_bind_tp: the plan has already run");
  for (int q = 0; q < p.tp_world; ++q) {
    if (!ar[q] || !x[q] || (reinterpret_cast<uintptr_t>(ar[q]) & 7u) || (reinterpret_cast<uintptr_t>(x[q]) & 7u))
      return Fail(-1, "tm_plan_bind_tp: every rank needs an 8-byte aligned region and exchange block");
    p.ar[q] = static_cast<unsigned long long*>(ar[q]);
    p.xchg[q] = static_cast<unsigned long long*>(x[q]);
  }
  p.tp_rank = rank;
  p.head_base = rank * p.geo[tmb::kHead].n;
  plan->tp_bound = true;
  return 0;
}

// One process per GPU: a rank makes its regions visible to its peers through CUDA IPC.
// Additions without a reference counterpart (its driver runs every rank in one process,
// python/tilemega/serving/tp_engine.py:47-112).
int tm_ipc_alloc(int device, uint64_t bytes, void** device_pointer) {
  if (!device_pointer || bytes == 0) return Fail(-1, "tm_ipc_alloc: bad argument");
  DeviceScope scope(device);
  // its own cudaMalloc: an IPC handle names a whole allocation, so the region must not be
  // a slice of some pool
  cudaError_t err = cudaMalloc(device_pointer, size_t(bytes));
  if (err == cudaSuccess) err = cudaMemset(*device_pointer, 0, size_t(bytes));
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  return err == cudaSuccess ? 0 : Fail(int(err), std::string("tm_ipc_alloc: ") + cudaGetErrorString(err));
}

int tm_ipc_free(void* device_pointer) {
  cudaError_t err = cudaFree(device_pointer);
  return err == cudaSuccess ? 0 : Fail(int(err), std::string("tm_ipc_free: ") + cudaGetErrorString(err));
}

int tm_ipc_export(void* device_pointer, unsigned char* handle64) {
  if (!device_pointer || !handle64) return Fail(-1, "tm_ipc_export: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t handle;
  cudaError_t err = cudaIpcGetMemHandle(&handle, device_pointer);
  if (err != cudaSuccess) return Fail(int(err), std::string("tm_ipc_export: ") + cudaGetErrorString(err));
  std::memcpy(handle64, &handle, 64);
  return 0;
}

int tm_ipc_open(const unsigned char* handle64, void** device_pointer) {
  if (!handle64 || !device_pointer) return Fail(-1, "tm_ipc_open: bad argument");
  cudaIpcMemHandle_t handle;
  std::memcpy(&handle, handle64, 64);
  cudaError_t err = cudaIpcOpenMemHandle(device_pointer, handle, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) return Fail(int(err), std::string("tm_ipc_open: ") + cudaGetErrorString(err));
  return 0;
}

int tm_ipc_close(void* device_pointer) {
  cudaError_t err = cudaIpcCloseMemHandle(device_pointer);
  return err == cudaSuccess ? 0 : Fail(int(err), std::string("tm_ipc_close: ") + cudaGetErrorString(err));
}

void tm_plan_destroy(void* handle) {
  Plan* plan = AsPlan(handle);
  if (plan) Destroy(plan);
}

}  // extern "C"
