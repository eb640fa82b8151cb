// Encoder forward for sm_100a: a BERT-shaped stack (embedding sum + LayerNorm, then per layer QKV, bidirectional
// attention over 128 positions, output projection + residual + LayerNorm, GELU FFN + residual + LayerNorm, and the
// pooler) over batch x 128 tokens. The four projections of a layer are one GEMM kernel on the 5th-generation
// tensor cores: token tiles (128 rows) and weight tiles (32..128 rows) arrive in shared memory through TMA tensor
// maps with the 128-byte swizzle, one thread issues tcgen05.mma into a tensor-memory accumulator, eight warps read
// it back with tcgen05.ld for the epilogue. A forward pass is ONE CUDA graph of these kernels, each recorded as a
// programmatic dependent of the one before it.
//
// What the reference does for this path: include/tilemega/Codegen/tasks/Sm90F3Program.cuh:690-732 (one persistent
// wgmma kernel over a compile-time stage list), Backend/Sm90F3Gemm.cuh, Sm90F3Attention.cuh, tasks/LayerNormTaskBody.h,
// EncoderAttentionTaskBody.h, EmbeddingSumTaskBody.h. The arithmetic it must reproduce is the HF BertModel forward
// (python/tilemega/dnn/export.py:50-59).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdlib>
#include <string>
#include <vector>

#include "encoder.h"
#include "ptx.cuh"

namespace tmb {
namespace {

constexpr int kSeq = 128;            // positions per sequence the attention kernel is written for
constexpr int kHeadDim = 64;
constexpr int kTileM = 128;          // tokens per GEMM tile (the tensor-memory lanes)
constexpr int kTileK = 64;           // 16-bit elements per 128-byte swizzle row
constexpr int kABytes = kTileM * kTileK * 2;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // a device wait gives up after two seconds

enum Epilogue { kEpiBias = 0, kEpiBiasGelu = 1, kEpiPartial = 2 };

// ---- element types -------------------------------------------------------------------------------------------
template <typename T> struct Num;
template <> struct Num<__half> {
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
  static constexpr uint32_t kIdescFormat = 0;                                  // a, b = f16
};
template <> struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w)); }
  static constexpr uint32_t kIdescFormat = (1u << 7) | (1u << 10);             // a, b = bf16
};

template <typename T> __device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const float2 a = Num<T>::unpack(v.x), b = Num<T>::unpack(v.y), c = Num<T>::unpack(v.z), d = Num<T>::unpack(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(Num<T>::pack(f[0], f[1]), Num<T>::pack(f[2], f[3]), Num<T>::pack(f[4], f[5]), Num<T>::pack(f[6], f[7]));
}
template <typename T> __device__ __forceinline__ void unpack4(const uint2& v, float (&f)[4]) {
  const float2 a = Num<T>::unpack(v.x), b = Num<T>::unpack(v.y);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

// ---- programmatic dependent launch ---------------------------------------------------------------------------
// Every kernel of the pass is launched as a programmatic dependent of the one before it: it may start (and run its
// prologue: barriers, tensor-memory allocation, descriptor prefetch) while its predecessor drains, and reads or writes
// global memory only after dependency_wait(), which returns once the predecessor grid has completed and its writes
// are visible. allow_dependents() lets the successor start as soon as every CTA of this grid has issued it.
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// erf(x) by the rational approximation 7.1.26 of Abramowitz and Stegun (absolute error below 1e-6 in fp32
// arithmetic, far inside a 16-bit output's resolution): two special-function instructions and six multiply-adds, where the library's erff
// costs the GELU epilogue about as much as the tile's whole main loop.
__device__ __forceinline__ float erf_fast(float x) {
  const float a = fabsf(x);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, a, 1.0f));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float tail = poly * t * ex2(-1.4426950408889634f * a * a);
  return copysignf(1.0f - tail, x);
}

// ---- bounded waits -------------------------------------------------------------------------------------------
// Wait for a phase of an mbarrier, but not for ever: after kWaitLimitNs (or once another wait of the launch
// has given up) the caller gets `false`, leaves its loop and the kernel runs to its end. status[0] keeps the
// code of the first wait that gave up; the host reads it after synchronising.
__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, unsigned* status, unsigned where) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer();
  unsigned spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0) {
      if (*reinterpret_cast<volatile unsigned*>(status)) return false;
      if (global_timer() - start > kWaitLimitNs) {
        atomicCAS(status, 0u, where);
        return false;
      }
    }
  }
  return true;
}

// 32 consecutive fp32 columns of this thread's tensor-memory lane in one instruction.
__device__ __forceinline__ void tmem_load_32(uint32_t address, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// One 32-byte store (a whole sector) to a 32-byte aligned global address.
__device__ __forceinline__ void store_32_bytes(void* dst, const uint4& lo, const uint4& hi) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w),
               "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
               : "memory");
}

// ---- GEMM on tcgen05 -----------------------------------------------------------------------------------------
struct GemmArgs {
  const void* bias[3];     // one per weight map (QKV: query, key, value; otherwise the same three times)
  void* out;               // T [rows][ldc], or fp32 [splits][rows][ldc] partial sums (kEpiPartial)
  int ldc;
  int n_per_map;           // output columns covered by each weight map
  int kchunks;             // 64-column chunks of K one CTA walks (K / 64 / splits)
  unsigned long long part_stride;   // elements between the partial slabs
  unsigned* status;
};

template <int BN, bool DEEP = false> struct GemmShape {
  // about 100 KB of stages, so that two CTAs share an SM; the deep form (32-row weight tiles in a grid of at most one
  // CTA per SM) has ten stages, which puts nearly a whole K = 768 reduction in flight at once
  static constexpr int kStages = DEEP ? 10 : BN >= 128 ? 3 : BN == 64 ? 4 : 5;
  static constexpr int kBBytes = BN * kTileK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSmem = kStages * kStageBytes + 1024 /* alignment */ + 256 /* barriers */ + 512 /* the tile's bias */;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
};

// C[128 x BN tile] = A[rows x K] (tokens, K-major) * W[N x K]^T (nn.Linear layout, K-major), fp32 in tensor memory.
// blockIdx = (n tile, m tile, K split). Warp 0: TMA producer. Warp 1: tensor-memory owner and MMA issuer.
// Warps 2..9: epilogue, each on the 32 lanes its warp id modulo 4 may read and on one half of the tile's columns.
constexpr int kGemmThreads = 320;
template <typename T, int BN, int EPI, bool DEEP>
__global__ void __launch_bounds__(kGemmThreads) encoder_gemm(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap wmap0,
                                                    const __grid_constant__ CUtensorMap wmap1, const __grid_constant__ CUtensorMap wmap2,
                                                    const GemmArgs g) {
  using Shape = GemmShape<BN, DEEP>;
  constexpr int S = Shape::kStages;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + S * Shape::kStageBytes);
  uint64_t* empty = full + S;
  uint64_t* accum = empty + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  unsigned char* bias_tile = tiles + S * Shape::kStageBytes + 256;   // BN elements of T, staged by the epilogue warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * kTileM, k0 = blockIdx.z * g.kchunks;
  const int which = n0 / g.n_per_map, nm = n0 - which * g.n_per_map;   // weight map and the row inside it
  const CUtensorMap* wmap = which == 0 ? &wmap0 : which == 1 ? &wmap1 : &wmap2;

  if (threadIdx.x == 0) {
    prefetch_map(&amap);
    prefetch_map(wmap);
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Shape::kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = *tmem_slot;
  // weights do not depend on the kernel before this one: the first stages' weight tiles are requested at once
  const int early = g.kchunks < S ? g.kchunks : S;
  if (threadIdx.x == 0)
    for (int c = 0; c < early; ++c) {
      mbar_expect_tx(&full[c], Shape::kStageBytes);
      tma_load_2d(tiles + c * Shape::kStageBytes + kABytes, wmap, (k0 + c) * kTileK, nm, &full[c]);
    }
  dependency_wait();   // from here on the activations of the kernel before this one may be read, and outputs written

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int c = 0; c < g.kchunks && ok; ++c) {
        const int s = c % S;
        if (c >= S) ok = wait_bounded(&empty[s], uint32_t((c / S) - 1) & 1u, g.status, 1);
        if (!ok) break;
        unsigned char* a = tiles + s * Shape::kStageBytes;
        if (c >= early) {   // (the first stages' barriers were armed, and their weight tiles requested, above)
          mbar_expect_tx(&full[s], Shape::kStageBytes);
          tma_load_2d(a + kABytes, wmap, (k0 + c) * kTileK, nm, &full[s]);
        }
        tma_load_2d(a, &amap, (k0 + c) * kTileK, m0, &full[s]);
        issued = c + 1;
      }
      if (!ok)   // leaving early: first let the copies already issued land in this CTA's shared memory
        for (int c = issued > S ? issued - S : 0; c < issued; ++c) wait_bounded(&full[c % S], uint32_t(c / S) & 1u, g.status, 2);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | Num<T>::kIdescFormat | (uint32_t(BN >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
      bool ok = true;
      for (int c = 0; c < g.kchunks && ok; ++c) {
        const int s = c % S;
        ok = wait_bounded(&full[s], uint32_t(c / S) & 1u, g.status, 3);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a = smem_u32(tiles + s * Shape::kStageBytes), b = a + kABytes;
#pragma unroll
        for (int j = 0; j < kTileK / 16; ++j)
          umma_bf16(tmem, umma_desc_k_sw128(a + 32 * j, 1024), umma_desc_k_sw128(b + 32 * j, 1024), idesc, uint32_t((c | j) != 0));
        umma_commit(&empty[s]);
      }
      umma_commit(accum);   // arrives once everything issued above is done (at once if nothing was)
    }
  } else {
    // while the main loop runs: this tile's bias into shared memory (weights: no need to wait for the kernel before)
    if (EPI != kEpiPartial) {
      const int e = threadIdx.x - 64;
      if (e < BN / 8) reinterpret_cast<uint4*>(bias_tile)[e] = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(g.bias[which]) + nm) + e);
      asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps
    }
    const bool ok = wait_bounded(accum, 0, g.status, 4);
    tcgen05_fence_after();
    // the main loop is over: the next kernel may start (its CTAs then find the SMs this grid is about to leave,
    // and its prologue and first weight tiles run under this epilogue)
    allow_dependents();
    const int quarter = warp & 3, column_half = (warp - 2) >> 2;
    const int row = m0 + 32 * quarter + lane;
    constexpr int W = BN >= 64 ? 32 : 16;          // columns per tensor-memory load
    if (ok) {
#pragma unroll
      for (int c = column_half * (BN / 2); c < (column_half + 1) * (BN / 2); c += W) {
        float v[W];
        if constexpr (W == 32) {
          tmem_load_32(tmem + (uint32_t(32 * quarter) << 16) + uint32_t(c), v);
        } else {
          tmem_load_16(tmem + (uint32_t(32 * quarter) << 16) + uint32_t(c), v);
        }
        if (EPI == kEpiPartial) {
          float* dst = static_cast<float*>(g.out) + size_t(blockIdx.z) * g.part_stride + size_t(row) * g.ldc + n0 + c;
#pragma unroll
          for (int i = 0; i < W / 8; ++i)
            store_32_bytes(dst + 8 * i,
                           make_uint4(__float_as_uint(v[8 * i]), __float_as_uint(v[8 * i + 1]), __float_as_uint(v[8 * i + 2]), __float_as_uint(v[8 * i + 3])),
                           make_uint4(__float_as_uint(v[8 * i + 4]), __float_as_uint(v[8 * i + 5]), __float_as_uint(v[8 * i + 6]), __float_as_uint(v[8 * i + 7])));
        } else {
          T* dst = static_cast<T*>(g.out) + size_t(row) * g.ldc + n0 + c;
#pragma unroll
          for (int i = 0; i < W / 16; ++i) {
            float lo[8], hi[8];
            unpack8<T>(reinterpret_cast<const uint4*>(bias_tile)[(c + 16 * i) / 8], lo);
            unpack8<T>(reinterpret_cast<const uint4*>(bias_tile)[(c + 16 * i) / 8 + 1], hi);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              lo[j] += v[16 * i + j];
              hi[j] += v[16 * i + 8 + j];
              if (EPI == kEpiBiasGelu) {   // the exact (erf) GELU of the BERT feed-forward
                lo[j] = 0.5f * lo[j] * (1.0f + erf_fast(lo[j] * 0.70710678118654752f));
                hi[j] = 0.5f * hi[j] * (1.0f + erf_fast(hi[j] * 0.70710678118654752f));
              }
            }
            store_32_bytes(dst + 16 * i, pack8<T>(lo), pack8<T>(hi));
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem, Shape::kTmemCols);
  }
}

// ---- LayerNorm stages ----------------------------------------------------------------------------------------
constexpr int kMaxGroups = 8;   // hidden <= 32 lanes x 4 columns x 8 groups = 1024
constexpr int kMaxSplits = 4;   // partial slabs of a projection whose K is split

// LayerNorm of one row held as groups of 4 columns per lane: v[g][i] = column (g * 32 + lane) * 4 + i.
template <typename T>
__device__ __forceinline__ void layer_norm_row(float (&v)[kMaxGroups][4], int groups, int lane, int hidden, const T* gamma, const T* beta,
                                               float eps, T* out) {
  float sum = 0.f;
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g)
    if (g < groups) sum += (v[g][0] + v[g][1]) + (v[g][2] + v[g][3]);
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mean = sum / float(hidden);
  float sq = 0.f;
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g)
    if (g < groups)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float d = v[g][i] - mean;
        sq += d * d;
      }
#pragma unroll
  for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  const float inv = rsqrtf(sq / float(hidden) + eps);
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g)
    if (g < groups) {
      const int col = (g * 32 + lane) * 4;
      float w[4], b[4];
      unpack4<T>(__ldg(reinterpret_cast<const uint2*>(gamma + col)), w);
      unpack4<T>(__ldg(reinterpret_cast<const uint2*>(beta + col)), b);
      uint2 packed;
      packed.x = Num<T>::pack((v[g][0] - mean) * inv * w[0] + b[0], (v[g][1] - mean) * inv * w[1] + b[1]);
      packed.y = Num<T>::pack((v[g][2] - mean) * inv * w[2] + b[2], (v[g][3] - mean) * inv * w[3] + b[3]);
      *reinterpret_cast<uint2*>(out + col) = packed;
    }
}

// Token, position and segment embeddings summed, then LayerNorm (BertEmbeddings). One warp per token.
template <typename T>
__global__ void __launch_bounds__(256) encoder_embed(const long long* ids, const long long* types, const T* word, const T* position,
                                                     const T* segment, const T* gamma, const T* beta, T* out, int rows, int seq,
                                                     int hidden, int vocab, int segments, float eps) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  allow_dependents();
  dependency_wait();
  if (row >= rows) return;
  long long id = ids[row], ty = types[row];
  id = id < 0 ? 0 : id >= vocab ? vocab - 1 : id;          // an id outside the table reads its nearest row
  ty = ty < 0 ? 0 : ty >= segments ? segments - 1 : ty;
  const int groups = hidden / 128;
  float v[kMaxGroups][4];
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g)
    if (g < groups) {
      const int col = (g * 32 + lane) * 4;
      float a[4], b[4], c[4];
      unpack4<T>(__ldg(reinterpret_cast<const uint2*>(word + size_t(id) * hidden + col)), a);
      unpack4<T>(__ldg(reinterpret_cast<const uint2*>(segment + size_t(ty) * hidden + col)), b);
      unpack4<T>(__ldg(reinterpret_cast<const uint2*>(position + size_t(row % seq) * hidden + col)), c);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[g][i] = (a[i] + b[i]) + c[i];
    }
  layer_norm_row<T>(v, groups, lane, hidden, gamma, beta, eps, out + size_t(row) * hidden);
}

// Sum of a projection's partial slabs (in slab order: the result does not depend on the schedule) + bias + the
// residual row, then LayerNorm (BertSelfOutput / BertOutput). One warp per token.
template <typename T>
__global__ void __launch_bounds__(128) encoder_add_norm(const float* parts, int nparts, unsigned long long part_stride, const T* bias,
                                                        const T* residual, const T* gamma, const T* beta, T* out, int rows, int hidden,
                                                        float eps) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  allow_dependents();
  dependency_wait();
  if (row >= rows) return;
  const int groups = hidden / 128;
  float v[kMaxGroups][4];
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g)
    if (g < groups) {
      const int col = (g * 32 + lane) * 4;
      // every slab's load goes out before the first sum (the slabs are added in slab order)
      float4 slab[kMaxSplits];
#pragma unroll
      for (int s = 0; s < kMaxSplits; ++s)
        if (s < nparts) slab[s] = __ldcs(reinterpret_cast<const float4*>(parts + size_t(s) * part_stride + size_t(row) * hidden + col));
      float4 acc = slab[0];
#pragma unroll
      for (int s = 1; s < kMaxSplits; ++s)
        if (s < nparts) {
          acc.x += slab[s].x; acc.y += slab[s].y; acc.z += slab[s].z; acc.w += slab[s].w;
        }
      float b[4], r[4];
      unpack4<T>(__ldg(reinterpret_cast<const uint2*>(bias + col)), b);
      unpack4<T>(*reinterpret_cast<const uint2*>(residual + size_t(row) * hidden + col), r);
      v[g][0] = (acc.x + b[0]) + r[0];
      v[g][1] = (acc.y + b[1]) + r[1];
      v[g][2] = (acc.z + b[2]) + r[2];
      v[g][3] = (acc.w + b[3]) + r[3];
    }
  layer_norm_row<T>(v, groups, lane, hidden, gamma, beta, eps, out + size_t(row) * hidden);
}

// ---- attention -----------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared-memory address of 16-byte chunk `chunk` of row `row` in a [rows][64] 16-bit tile whose chunks are
// XOR-swizzled by the row (eight rows of one chunk column then sit in eight different bank groups).
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) { return base + row * 128 + ((chunk ^ (row & 7)) << 4); }

// Bidirectional attention of one (sequence, head) over 128 positions: softmax(Q K^T / sqrt(64) + mask) V, where a
// key position whose `mask` entry is 0 gets the most negative finite score (the additive mask the module builds from
// its attention_mask input; every query row still attends, a row with no visible key attends uniformly). `mask` may
// be null: every position visible. A CTA takes the 128 query rows (8 warps x 16) against the 128 keys; scores, softmax
// and the probability operand stay in registers.
template <typename T>
__global__ void __launch_bounds__(256) encoder_attention(const T* qkv, T* ctx, const long long* mask, int heads, int hidden,
                                                         float scale_log2) {
  __shared__ __align__(128) unsigned char ks[kSeq * 128], vs[kSeq * 128], qs[kSeq * 128];
  const int head = blockIdx.x % heads, seq = blockIdx.x / heads;
  const int ld = 3 * hidden, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* base = qkv + size_t(seq) * kSeq * ld + head * kHeadDim;
  allow_dependents();
  dependency_wait();
  {
    // 128 rows x 8 sixteen-byte chunks of q, k and v: four chunks of each per thread, all twelve loads in flight
    uint4 qv[4], kv[4], vv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * 256, r = i >> 3, ch = i & 7;
      const T* row = base + size_t(r) * ld + ch * 8;
      qv[j] = *reinterpret_cast<const uint4*>(row);
      kv[j] = *reinterpret_cast<const uint4*>(row + hidden);
      vv[j] = *reinterpret_cast<const uint4*>(row + 2 * hidden);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * 256, r = i >> 3, ch = i & 7, at = r * 128 + ((ch ^ (r & 7)) << 4);
      *reinterpret_cast<uint4*>(qs + at) = qv[j];
      *reinterpret_cast<uint4*>(ks + at) = kv[j];
      *reinterpret_cast<uint4*>(vs + at) = vv[j];
    }
  }
  __syncthreads();
  const uint32_t kbase = smem_u32(ks), vbase = smem_u32(vs), qbase = smem_u32(qs);

  // scores of this warp's 16 query rows against 128 keys: 16 column tiles of 8
  float s[16][4];
#pragma unroll
  for (int t = 0; t < 16; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < kHeadDim / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, tile_addr(qbase, warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4)));
#pragma unroll
    for (int tp = 0; tp < 8; ++tp) {   // two key tiles per load
      uint32_t b[4];
      ldmatrix_x4(b, tile_addr(kbase, tp * 16 + (lane & 7) + (lane >> 4) * 8, 2 * kk + ((lane >> 3) & 1)));
      mma_16816<T>(s[2 * tp], a, b[0], b[1]);
      mma_16816<T>(s[2 * tp + 1], a, b[2], b[3]);
    }
  }
  if (mask) {   // this thread's key columns of tile t: 8 t + 2 (lane % 4) and the next one
    const long long* visible = mask + size_t(seq) * kSeq + 2 * (lane & 3);
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const longlong2 m = *reinterpret_cast<const longlong2*>(visible + 8 * t);
      if (m.x == 0) s[t][0] = s[t][2] = -3.0e38f;
      if (m.y == 0) s[t][1] = s[t][3] = -3.0e38f;
    }
  }
  // softmax over the 128 keys of rows lane / 4 (values 0, 1 of a tile) and lane / 4 + 8 (values 2, 3)
  float top_lo = -INFINITY, top_hi = -INFINITY;
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    top_lo = fmaxf(top_lo, fmaxf(s[t][0], s[t][1]));
    top_hi = fmaxf(top_hi, fmaxf(s[t][2], s[t][3]));
  }
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
    top_lo = fmaxf(top_lo, __shfl_xor_sync(0xffffffffu, top_lo, o));
    top_hi = fmaxf(top_hi, __shfl_xor_sync(0xffffffffu, top_hi, o));
  }
  float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    s[t][0] = ex2((s[t][0] - top_lo) * scale_log2);
    s[t][1] = ex2((s[t][1] - top_lo) * scale_log2);
    s[t][2] = ex2((s[t][2] - top_hi) * scale_log2);
    s[t][3] = ex2((s[t][3] - top_hi) * scale_log2);
    sum_lo += s[t][0] + s[t][1];
    sum_hi += s[t][2] + s[t][3];
  }
#pragma unroll
  for (int o = 1; o <= 2; o <<= 1) {
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, o);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, o);
  }
  // context = probabilities (as the 16-bit A operand, straight from the score registers) x V
  float o[8][4];
#pragma unroll
  for (int t = 0; t < 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < kSeq / 16; ++kk) {
    uint32_t a[4];
    a[0] = Num<T>::pack(s[2 * kk][0], s[2 * kk][1]);
    a[1] = Num<T>::pack(s[2 * kk][2], s[2 * kk][3]);
    a[2] = Num<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = Num<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < 4; ++dp) {   // two column tiles of the head per load
      uint32_t b[4];
      ldmatrix_x4_trans(b, tile_addr(vbase, kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * dp + (lane >> 4)));
      mma_16816<T>(o[2 * dp], a, b[0], b[1]);
      mma_16816<T>(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
  const float inv_lo = 1.0f / sum_lo, inv_hi = 1.0f / sum_hi;
  T* out = ctx + (size_t(seq) * kSeq + warp * 16 + (lane >> 2)) * hidden + head * kHeadDim + 2 * (lane & 3);
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    *reinterpret_cast<uint32_t*>(out + t * 8) = Num<T>::pack(o[t][0] * inv_lo, o[t][1] * inv_lo);
    *reinterpret_cast<uint32_t*>(out + size_t(8) * hidden + t * 8) = Num<T>::pack(o[t][2] * inv_hi, o[t][3] * inv_hi);
  }
}

// ---- pooler --------------------------------------------------------------------------------------------------
// tanh(W h + b) on the first position of every sequence (BertPooler). One warp per output element.
template <typename T>
__global__ void __launch_bounds__(256) encoder_pooler(const T* hidden_out, const T* weight, const T* bias, T* out, int seq, int hidden) {
  const int n = blockIdx.x * 8 + (threadIdx.x >> 5), b = blockIdx.y, lane = threadIdx.x & 31;
  allow_dependents();
  dependency_wait();
  if (n >= hidden) return;
  const T* x = hidden_out + size_t(b) * seq * hidden;
  const T* w = weight + size_t(n) * hidden;
  float acc = 0.f;
  for (int col = lane * 4; col < hidden; col += 128) {
    float xv[4], wv[4];
    unpack4<T>(*reinterpret_cast<const uint2*>(x + col), xv);
    unpack4<T>(__ldg(reinterpret_cast<const uint2*>(w + col)), wv);
    acc += xv[0] * wv[0] + xv[1] * wv[1] + xv[2] * wv[2] + xv[3] * wv[3];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[size_t(b) * hidden + n] = Num<T>::from_float(tanhf(acc + Num<T>::to_float(bias[n])));
}

}  // namespace

// ---- host side -----------------------------------------------------------------------------------------------
struct GemmLaunch {
  CUtensorMap amap, wmap[3];
  GemmArgs args;
  dim3 grid;
  int bn, epilogue;
  bool dependent, deep;
};

struct EncoderPlan {
  bool f16 = false;
  int batch = 0, rows = 0, hidden = 0, inter = 0, heads = 0, layers = 0, vocab = 0, segments = 0, seq = 0;
  float eps = 1e-12f;
  std::vector<void*> owned;
  unsigned* status = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int kernels = 0;
  bool chained = true;   // kernels recorded as programmatic dependents of one another
};

namespace {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up at run time (the library does not link against the driver library).
EncodeTiled TensorMapEncoder() {
  static EncodeTiled encode = nullptr;
  if (!encode) {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult found{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) == cudaSuccess && entry &&
        found == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeTiled>(entry);
  }
  return encode;
}

// Map over a row-major 16-bit matrix [rows][cols] of this GPU's memory: boxes of `box_rows` x 64 columns, 128-byte
// swizzle. A copy's innermost coordinate is a multiple of 64 elements (128 bytes).
bool EncodeMatrix(CUtensorMap* map, bool f16, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiled encode = TensorMapEncoder();
  if (!encode) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {uint32_t(kTileK), box_rows};
  const cuuint32_t steps[2] = {1, 1};
  return encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One kernel launch; `dependent`: as a programmatic dependent of the launch before it on the stream.
template <typename... Params, typename... Args>
cudaError_t Launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool dependent, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = dependent ? &attribute : nullptr;
  config.numAttrs = dependent ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

template <typename T, int BN, int EPI, bool DEEP = false> cudaError_t LaunchGemmAs(const GemmLaunch& l, cudaStream_t stream) {
  auto kernel = encoder_gemm<T, BN, EPI, DEEP>;
  if (!stream)   // preparation pass (before the recording starts): only raise the kernel's shared-memory limit
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmShape<BN, DEEP>::kSmem);
  return Launch(kernel, l.grid, dim3(kGemmThreads), GemmShape<BN, DEEP>::kSmem, stream, l.dependent, l.amap, l.wmap[0], l.wmap[1], l.wmap[2], l.args);
}

template <typename T, int BN, bool DEEP = false> cudaError_t LaunchGemmTile(const GemmLaunch& l, cudaStream_t stream) {
  switch (l.epilogue) {
    case kEpiBias: return LaunchGemmAs<T, BN, kEpiBias, DEEP>(l, stream);
    case kEpiBiasGelu: return LaunchGemmAs<T, BN, kEpiBiasGelu, DEEP>(l, stream);
    default: return LaunchGemmAs<T, BN, kEpiPartial, DEEP>(l, stream);
  }
}

template <typename T> cudaError_t LaunchGemm(const GemmLaunch& l, cudaStream_t stream) {
  switch (l.bn) {
    case 128: return LaunchGemmTile<T, 128>(l, stream);
    case 64: return LaunchGemmTile<T, 64>(l, stream);
    default: return l.deep ? LaunchGemmTile<T, 32, true>(l, stream) : LaunchGemmTile<T, 32>(l, stream);
  }
}

// Tile width and K split of one projection. Wide weight tiles re-read the token tile less often from L2, so the
// widest tile that still gives three quarters of the SMs a CTA wins; a projection that ends in the add + LayerNorm
// stage may instead split K in up to kMaxSplits parts (its partial slabs are summed there, in slab order), and
// takes the fewest parts that occupy half of the SMs.
#ifndef TMB_ENCODER_WANTED_PLAIN
#define TMB_ENCODER_WANTED_PLAIN 100
#endif
#ifndef TMB_ENCODER_WANTED_SPLIT
#define TMB_ENCODER_WANTED_SPLIT 100
#endif
constexpr int kWantedPlainPercent = TMB_ENCODER_WANTED_PLAIN, kWantedSplitPercent = TMB_ENCODER_WANTED_SPLIT;

void ChooseTiling(int rows, int n, int k, int sm_count, bool may_split, int* bn, int* splits) {
  const int mtiles = rows / kTileM, chunks = k / kTileK;
  int widest_split = 1;
  if (may_split)
    for (int candidate = 1; candidate <= kMaxSplits; ++candidate)
      if (chunks % candidate == 0) widest_split = candidate;
  const int wanted = sm_count * (may_split ? kWantedSplitPercent : kWantedPlainPercent) / 100;
  *bn = 32;
  for (int candidate : {128, 64, 32})
    if (mtiles * (n / candidate) * widest_split >= wanted) {
      *bn = candidate;
      break;
    }
  *splits = 1;
  for (int candidate = 1; candidate <= widest_split; ++candidate) {
    if (chunks % candidate) continue;
    *splits = candidate;
    if (mtiles * (n / *bn) * candidate >= wanted) break;
  }
}

// Every instantiation a plan of this element type may launch gets its dynamic shared-memory limit raised.
template <typename T> cudaError_t PrepareGemms() {
  GemmLaunch l{};
  for (int form = 0; form < 4; ++form)
    for (int epilogue : {int(kEpiBias), int(kEpiBiasGelu), int(kEpiPartial)}) {
      l.bn = form == 0 ? 128 : form == 1 ? 64 : 32;
      l.deep = form == 3;
      l.epilogue = epilogue;
      const cudaError_t err = LaunchGemm<T>(l, nullptr);   // a null stream means: prepare only
      if (err != cudaSuccess) return err;
    }
  return cudaSuccess;
}

int Find(const PlanSpec& spec, const std::string& name) {
  for (size_t i = 0; i < spec.buffers.size(); ++i)
    if (spec.buffers[i].name == name) return int(i);
  return -1;
}

template <typename T> cudaError_t Enqueue(EncoderPlan& plan, const PlanSpec& spec, const std::vector<void*>& buffers, int sm_count,
                                         float* parts, cudaStream_t stream, bool chained, std::string* error) {
  auto at = [&](const std::string& name) -> void* {
    const int index = Find(spec, name);
    if (index < 0) {
      *error = "the buffer table has no '" + name + "'";
      return nullptr;
    }
    return buffers[size_t(index)];
  };
#define TMB_AT(var, name)        \
  void* var = at(name);          \
  if (!var) return cudaErrorInvalidValue;
  const int rows = plan.rows, hidden = plan.hidden, inter = plan.inter;
  TMB_AT(ids, "input_ids")
  TMB_AT(types, "token_type_ids")
  TMB_AT(word, "embeddings.word_embeddings.weight")
  TMB_AT(position, "embeddings.position_embeddings.weight")
  TMB_AT(segment, "embeddings.token_type_embeddings.weight")
  TMB_AT(embed_gamma, "embeddings.LayerNorm.weight")
  TMB_AT(embed_beta, "embeddings.LayerNorm.bias")
  TMB_AT(x, "forward.hidden")
  TMB_AT(qkv, "forward.qkv")
  TMB_AT(ctx, "forward.context")
  TMB_AT(ffn, "forward.ffn")
  TMB_AT(last_hidden, "last_hidden_state")
  TMB_AT(pooled, "pooler_output")
  TMB_AT(pool_w, "pooler.dense.weight")
  TMB_AT(pool_b, "pooler.dense.bias")
  void* mask = nullptr;
  if (spec.forward_mask) {
    TMB_AT(bound_mask, "attention_mask")
    mask = bound_mask;
  }
  cudaError_t err = cudaSuccess;
  plan.kernels = 0;
  // the first kernel of the pass is an ordinary launch: it follows whatever the caller's stream ran before
  err = Launch(encoder_embed<T>, dim3(unsigned((rows + 7) / 8)), dim3(256), 0, stream, false, static_cast<const long long*>(ids),
               static_cast<const long long*>(types), static_cast<const T*>(word), static_cast<const T*>(position),
               static_cast<const T*>(segment), static_cast<const T*>(embed_gamma), static_cast<const T*>(embed_beta), static_cast<T*>(x),
               rows, plan.seq, hidden, plan.vocab, plan.segments, plan.eps);
  ++plan.kernels;
  if (err != cudaSuccess) return err;

  // one projection: A = activation [rows][k], up to three weight matrices of n_per_map rows each
  auto gemm = [&](const void* a, int k, const void* const (&w)[3], const void* const (&bias)[3], int n, int n_per_map, int epilogue,
                  void* out) -> cudaError_t {
    GemmLaunch l{};
    int splits = 1;
    ChooseTiling(rows, n, k, sm_count, epilogue == kEpiPartial, &l.bn, &splits);
    if (!EncodeMatrix(&l.amap, plan.f16, a, uint64_t(rows), uint64_t(k), kTileM)) {
      *error = "cuTensorMapEncodeTiled rejected an activation buffer";
      return cudaErrorInvalidValue;
    }
    for (int i = 0; i < 3; ++i)
      if (!EncodeMatrix(&l.wmap[i], plan.f16, w[i], uint64_t(n_per_map), uint64_t(k), uint32_t(l.bn))) {
        *error = "cuTensorMapEncodeTiled rejected a weight buffer";
        return cudaErrorInvalidValue;
      }
    for (int i = 0; i < 3; ++i) l.args.bias[i] = bias[i];
    l.args.out = out;
    l.args.ldc = n;
    l.args.n_per_map = n_per_map;
    l.args.kchunks = k / kTileK / splits;
    l.args.part_stride = (unsigned long long)(rows) * n;
    l.args.status = plan.status;
    l.grid = dim3(unsigned(n / l.bn), unsigned(rows / kTileM), unsigned(splits));
    l.epilogue = epilogue;
    l.deep = l.bn == 32 && int(l.grid.x * l.grid.y * l.grid.z) <= sm_count;
    l.dependent = chained;
    ++plan.kernels;
    return LaunchGemm<T>(l, stream);
  };
  auto add_norm = [&](int k, const void* bias, const void* gamma, const void* beta, void* out) -> cudaError_t {
    int bn = 0, splits = 1;
    ChooseTiling(rows, hidden, k, sm_count, true, &bn, &splits);   // the slab count the projection before it wrote
    ++plan.kernels;
    return Launch(encoder_add_norm<T>, dim3(unsigned((rows + 3) / 4)), dim3(128), 0, stream, chained, static_cast<const float*>(parts), splits,
                  (unsigned long long)(rows) * hidden, static_cast<const T*>(bias), static_cast<const T*>(x), static_cast<const T*>(gamma),
                  static_cast<const T*>(beta), static_cast<T*>(out), rows, hidden, plan.eps);
  };
  const float scale_log2 = 1.4426950408889634f / 8.0f;   // log2(e) / sqrt(64)
  for (int layer = 0; layer < plan.layers; ++layer) {
    const std::string p = "encoder.layer." + std::to_string(layer) + ".";
    TMB_AT(wq, p + "attention.self.query.weight")
    TMB_AT(wk, p + "attention.self.key.weight")
    TMB_AT(wv, p + "attention.self.value.weight")
    TMB_AT(bq, p + "attention.self.query.bias")
    TMB_AT(bk, p + "attention.self.key.bias")
    TMB_AT(bv, p + "attention.self.value.bias")
    TMB_AT(wo, p + "attention.output.dense.weight")
    TMB_AT(bo, p + "attention.output.dense.bias")
    TMB_AT(g1, p + "attention.output.LayerNorm.weight")
    TMB_AT(b1, p + "attention.output.LayerNorm.bias")
    TMB_AT(wi, p + "intermediate.dense.weight")
    TMB_AT(bi, p + "intermediate.dense.bias")
    TMB_AT(wd, p + "output.dense.weight")
    TMB_AT(bd, p + "output.dense.bias")
    TMB_AT(g2, p + "output.LayerNorm.weight")
    TMB_AT(b2, p + "output.LayerNorm.bias")
    {
      const void* const w[3] = {wq, wk, wv};
      const void* const b[3] = {bq, bk, bv};
      if ((err = gemm(x, hidden, w, b, 3 * hidden, hidden, kEpiBias, qkv)) != cudaSuccess) return err;
    }
    err = Launch(encoder_attention<T>, dim3(unsigned(plan.batch * plan.heads)), dim3(256), 0, stream, chained, static_cast<const T*>(qkv),
                 static_cast<T*>(ctx), static_cast<const long long*>(mask), plan.heads, hidden, scale_log2);
    ++plan.kernels;
    if (err != cudaSuccess) return err;
    {
      const void* const w[3] = {wo, wo, wo};
      const void* const b[3] = {bo, bo, bo};
      if ((err = gemm(ctx, hidden, w, b, hidden, hidden, kEpiPartial, parts)) != cudaSuccess) return err;
    }
    if ((err = add_norm(hidden, bo, g1, b1, x)) != cudaSuccess) return err;
    {
      const void* const w[3] = {wi, wi, wi};
      const void* const b[3] = {bi, bi, bi};
      if ((err = gemm(x, hidden, w, b, inter, inter, kEpiBiasGelu, ffn)) != cudaSuccess) return err;
    }
    {
      const void* const w[3] = {wd, wd, wd};
      const void* const b[3] = {bd, bd, bd};
      if ((err = gemm(ffn, inter, w, b, hidden, hidden, kEpiPartial, parts)) != cudaSuccess) return err;
    }
    // the last layer's LayerNorm writes the caller's output buffer
    if ((err = add_norm(inter, bd, g2, b2, layer + 1 == plan.layers ? last_hidden : x)) != cudaSuccess) return err;
  }
  ++plan.kernels;
#undef TMB_AT
  return Launch(encoder_pooler<T>, dim3(unsigned((hidden + 7) / 8), unsigned(plan.batch)), dim3(256), 0, stream, chained,
                static_cast<const T*>(last_hidden), static_cast<const T*>(pool_w), static_cast<const T*>(pool_b), static_cast<T*>(pooled),
                plan.seq, hidden);
}

}  // namespace

EncoderPlan* EncoderCreate(const PlanSpec& spec, int batch, const std::vector<void*>& buffers, int sm_count, std::string* error) {
  auto plan = new EncoderPlan;
  plan->f16 = spec.f16;
  plan->batch = batch;
  plan->seq = spec.forward_seq;
  plan->rows = batch * spec.forward_seq;
  plan->hidden = spec.hidden;
  plan->inter = spec.inter;
  plan->heads = spec.heads;
  plan->layers = spec.layers;
  plan->vocab = spec.vocab;
  plan->segments = spec.type_vocab;
  plan->eps = float(spec.eps);
  auto fail = [&](const std::string& what) -> EncoderPlan* {
    if (error->empty()) *error = what;
    EncoderDestroy(plan);
    return nullptr;
  };
  if (!TensorMapEncoder()) return fail("the driver does not offer cuTensorMapEncodeTiled");
  // partial slabs of the two projections that end in add + LayerNorm: at most kMaxSplits slabs of rows x hidden fp32
  void* parts = nullptr;
  if (cudaMalloc(&parts, size_t(kMaxSplits) * plan->rows * plan->hidden * sizeof(float)) != cudaSuccess) return fail("no device memory for the partial sums");
  plan->owned.push_back(parts);
  void* status = nullptr;
  if (cudaMalloc(&status, 64) != cudaSuccess || cudaMemset(status, 0, 64) != cudaSuccess) return fail("no device memory for the status words");
  plan->owned.push_back(status);
  plan->status = static_cast<unsigned*>(status);
  // the forward pass is recorded once, on a stream of its own, and replayed as one graph launch
  if ((spec.f16 ? PrepareGemms<__half>() : PrepareGemms<__nv_bfloat16>()) != cudaSuccess) return fail("cannot raise the GEMM kernels' shared-memory limit");
  cudaStream_t recorder = nullptr;
  if (cudaStreamCreateWithFlags(&recorder, cudaStreamNonBlocking) != cudaSuccess) return fail("cannot create the recording stream");
  // TILEMEGA_ENCODER_CHAIN=0 records plain launches (each kernel starts when the one before it has ended)
  const char* chain = std::getenv("TILEMEGA_ENCODER_CHAIN");
  plan->chained = !(chain && chain[0] == '0');
  cudaError_t err = cudaStreamBeginCapture(recorder, cudaStreamCaptureModeThreadLocal);
  if (err == cudaSuccess) {
    err = spec.f16 ? Enqueue<__half>(*plan, spec, buffers, sm_count, static_cast<float*>(parts), recorder, plan->chained, error)
                   : Enqueue<__nv_bfloat16>(*plan, spec, buffers, sm_count, static_cast<float*>(parts), recorder, plan->chained, error);
    const cudaError_t ended = cudaStreamEndCapture(recorder, &plan->graph);
    if (err == cudaSuccess) err = ended;
  }
  cudaStreamDestroy(recorder);
  if (err != cudaSuccess) return fail(std::string("recording the forward pass: ") + cudaGetErrorString(err));
  err = cudaGraphInstantiate(&plan->exec, plan->graph, 0);
  if (err != cudaSuccess) return fail(std::string("cudaGraphInstantiate: ") + cudaGetErrorString(err));
  return plan;
}

int EncoderLaunch(EncoderPlan* plan, cudaStream_t stream) { return int(cudaGraphLaunch(plan->exec, stream)); }

int EncoderStatus(EncoderPlan* plan, uint64_t* record12) {
  unsigned words[4] = {0, 0, 0, 0};
  if (cudaMemcpy(words, plan->status, sizeof(words), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (record12) {
    for (int i = 0; i < 12; ++i) record12[i] = 0;
    record12[0] = words[0];   // 1: producer waiting for a free stage, 2: copies in flight, 3: MMA waiting for a stage, 4: epilogue
  }
  return words[0] ? 1 : 0;
}

void EncoderClear(EncoderPlan* plan) { cudaMemset(plan->status, 0, 64); }

void EncoderDestroy(EncoderPlan* plan) {
  if (!plan) return;
  if (plan->exec) cudaGraphExecDestroy(plan->exec);
  if (plan->graph) cudaGraphDestroy(plan->graph);
  for (void* p : plan->owned) cudaFree(p);
  delete plan;
}

}  // namespace tmb
