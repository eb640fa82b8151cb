// Microbenchmarks behind the sm_100 target description: the numbers the reference's
// TargetSpec parser requires under "calibration" (lib/Target/TargetSpec.cpp:60-200; the
// reference fills them with lib/Target/Calibration.cu and its siblings on its own hardware).
// Every benchmark here only reads and writes buffers it allocates itself, runs a fixed
// number of iterations, changes no device setting, and frees what it took. Waits between
// CTAs exist in the grid-barrier benchmark only: it is a cooperative launch (co-residency is
// guaranteed or the launch is refused) and its spin has an iteration limit all the same.
//
// One entry point, tm_calibrate(device, what, out, capacity): runs the benchmark named
// `what` and writes its numbers to out[]; returns how many it wrote, or a negative status.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/tilemega_b200.h"
#include "ptx.cuh"

namespace {

#define CAL_CHECK(expr)                                                                           \
  do {                                                                                            \
    cudaError_t status_ = (expr);                                                                 \
    if (status_ != cudaSuccess) {                                                                 \
      std::fprintf(stderr, "tilemega_b200: tm_calibrate: %s: %s\n", #expr, cudaGetErrorString(status_)); \
      return -int(status_) - 1000;                                                                \
    }                                                                                             \
  } while (0)

struct Timer {
  cudaEvent_t begin, end;
  Timer() {
    cudaEventCreate(&begin);
    cudaEventCreate(&end);
  }
  ~Timer() {
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
  }
  void start() { cudaEventRecord(begin); }
  double stop_ms() {
    cudaEventRecord(end);
    cudaEventSynchronize(end);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, begin, end);
    return double(ms);
  }
};

// ---- arithmetic pipes: long dependent-free chains per thread, all SMs busy ----
template <int Kind>
__global__ void pipe_kernel(float* sink, int iters) {
  float a0 = threadIdx.x * 1e-3f + 1.f, a1 = a0 + 1.f, a2 = a0 + 2.f, a3 = a0 + 3.f;
  float a4 = a0 + 4.f, a5 = a0 + 5.f, a6 = a0 + 6.f, a7 = a0 + 7.f;
  int i0 = threadIdx.x + 1, i1 = i0 + 1, i2 = i0 + 2, i3 = i0 + 3, i4 = i0 + 4, i5 = i0 + 5, i6 = i0 + 6, i7 = i0 + 7;
  const float m = 1.000001f, c = 1e-7f;
#pragma unroll 1
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (Kind == 0) {
        a0 = fmaf(a0, m, c); a1 = fmaf(a1, m, c); a2 = fmaf(a2, m, c); a3 = fmaf(a3, m, c);
        a4 = fmaf(a4, m, c); a5 = fmaf(a5, m, c); a6 = fmaf(a6, m, c); a7 = fmaf(a7, m, c);
      } else if (Kind == 1) {
        i0 = i0 * 3 + i1; i1 = i1 * 5 + i2; i2 = i2 * 7 + i3; i3 = i3 * 9 + i4;
        i4 = i4 * 3 + i5; i5 = i5 * 5 + i6; i6 = i6 * 7 + i7; i7 = i7 * 9 + i0;
      } else if (Kind == 2) {
        a0 = tmb::ex2(a0 * 1e-3f); a1 = tmb::ex2(a1 * 1e-3f); a2 = tmb::ex2(a2 * 1e-3f); a3 = tmb::ex2(a3 * 1e-3f);
        a4 = tmb::ex2(a4 * 1e-3f); a5 = tmb::ex2(a5 * 1e-3f); a6 = tmb::ex2(a6 * 1e-3f); a7 = tmb::ex2(a7 * 1e-3f);
      } else {
        a0 = rsqrtf(a0 + 1.f); a1 = rsqrtf(a1 + 1.f); a2 = rsqrtf(a2 + 1.f); a3 = rsqrtf(a3 + 1.f);
        a4 = rsqrtf(a4 + 1.f); a5 = rsqrtf(a5 + 1.f); a6 = rsqrtf(a6 + 1.f); a7 = rsqrtf(a7 + 1.f);
      }
    }
  }
  const float total = a0 + a1 + a2 + a3 + a4 + a5 + a6 + a7 + float(i0 ^ i1 ^ i2 ^ i3 ^ i4 ^ i5 ^ i6 ^ i7);
  if (total == 123.456f) sink[0] = total;   // never true: keeps the chains alive
}

// Tensor pipe through mma.sync m16n8k16 (the instruction the decode kernel's GEMV uses): eight
// independent accumulator sets per warp.
template <bool Bf16>
__global__ void mma_kernel(float* sink, int iters) {
  float d[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.f;
  const uint32_t a = 0x3c003c00u + threadIdx.x, b = 0x3c003c00u;
#pragma unroll 1
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (Bf16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[i][0]), "+f"(d[i][1]), "+f"(d[i][2]), "+f"(d[i][3])
                     : "r"(a), "r"(a), "r"(a), "r"(a), "r"(b), "r"(b));
      } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[i][0]), "+f"(d[i][1]), "+f"(d[i][2]), "+f"(d[i][3])
                     : "r"(a), "r"(a), "r"(a), "r"(a), "r"(b), "r"(b));
      }
    }
  }
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += d[i][0] + d[i][1] + d[i][2] + d[i][3];
  if (total == 123.456f) sink[0] = total;
}

// ---- shared memory: 128-bit loads, stride in 16-byte units selects the bank-conflict degree ----
__global__ void smem_kernel(float* sink, int iters, int stride) {
  extern __shared__ uint4 tile[];
  const int words = 2048;   // 32 KB
  for (int i = threadIdx.x; i < words; i += blockDim.x) tile[i] = make_uint4(i, i, i, i);
  __syncthreads();
  uint4 acc = make_uint4(0, 0, 0, 0);
  int index = (threadIdx.x * stride) & (words - 1);
#pragma unroll 1
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint4 v = tile[index];
      acc.x += v.x; acc.y ^= v.y; acc.z += v.z; acc.w ^= v.w;
      index = (index + 32 * stride) & (words - 1);
    }
  }
  if (acc.x + acc.y + acc.z + acc.w == 0x12345u) sink[0] = 1.f;
}

// ---- latency: one thread chases pointers through a footprint ----
__global__ void chase_kernel(const uint32_t* next, int hops, uint32_t* out, long long* cycles) {
  uint32_t at = 0;
  for (int i = 0; i < 64; ++i) at = next[at];   // warm the TLB path, not the lines (the footprint decides those)
  const long long t0 = clock64();
  for (int i = 0; i < hops; ++i) at = __ldcg(next + at);
  const long long t1 = clock64();
  out[0] = at;
  cycles[0] = t1 - t0;
}

__global__ void chase_l1_kernel(const uint32_t* next, int hops, uint32_t* out, long long* cycles) {
  uint32_t at = 0;
  for (int i = 0; i < 2 * hops; ++i) at = __ldca(next + at);
  const long long t0 = clock64();
  for (int i = 0; i < hops; ++i) at = __ldca(next + at);
  const long long t1 = clock64();
  out[0] = at;
  cycles[0] = t1 - t0;
}

// ---- bandwidth: every CTA streams its share of `bytes`, `passes` times ----
__global__ void read_kernel(const uint4* data, size_t chunks, int passes, float* sink) {
  uint4 acc = make_uint4(0, 0, 0, 0);
  for (int pass = 0; pass < passes; ++pass)
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < chunks; i += size_t(gridDim.x) * blockDim.x) {
      const uint4 v = __ldcg(data + i);
      acc.x ^= v.x; acc.y ^= v.y; acc.z ^= v.z; acc.w ^= v.w;
    }
  if ((acc.x ^ acc.y ^ acc.z ^ acc.w) == 0x12345u) sink[0] = 1.f;
}

__global__ void copy_kernel(const uint4* src, uint4* dst, size_t chunks) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < chunks; i += size_t(gridDim.x) * blockDim.x)
    dst[i] = __ldcs(src + i);
}

// ---- synchronisation primitives, timed in cycles by one thread / one CTA ----
__global__ void sync_kernel(unsigned long long* word, long long* cycles, int iters) {
  // [0] atomicAdd round trip, [1] __threadfence, [2] __syncthreads, [3] named barrier of 128 threads
  if (threadIdx.x == 0) {
    unsigned long long seen = 0;
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) seen += atomicAdd(word, 1ull);
    cycles[0] = (clock64() - t0) / iters + (seen == 1ull << 62 ? 1 : 0);
    t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      word[1] = i;
      __threadfence();
    }
    cycles[1] = (clock64() - t0) / iters;
  }
  __syncthreads();
  long long t0 = clock64();
  for (int i = 0; i < iters; ++i) __syncthreads();
  if (threadIdx.x == 0) cycles[2] = (clock64() - t0) / iters;
  if (threadIdx.x < 128) {
    t0 = clock64();
    for (int i = 0; i < iters; ++i) asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 0) cycles[3] = (clock64() - t0) / iters;
  }
}

__global__ void contention_kernel(unsigned long long* word, long long* cycles, int iters) {
  if (threadIdx.x != 0) return;
  unsigned long long seen = 0;
  const long long t0 = clock64();
  for (int i = 0; i < iters; ++i) seen += atomicAdd(word, 1ull);
  cycles[blockIdx.x] = (clock64() - t0) / iters + (seen == 1ull << 62 ? 1 : 0);
}

__global__ void __cluster_dims__(2, 1, 1) cluster_sync_kernel(long long* cycles, int iters) {
  const long long t0 = clock64();
  for (int i = 0; i < iters; ++i) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  if (threadIdx.x == 0 && blockIdx.x == 0) cycles[0] = (clock64() - t0) / iters;
}

// A grid-wide barrier the way the decode kernel builds it: one release-add per CTA on a monotonic
// counter, every CTA polls it with acquire loads. Cooperative launch; the poll is bounded.
__global__ void grid_barrier_kernel(unsigned long long* counter, long long* cycles, int iters, int* gave_up) {
  unsigned long long target = 0;
  const long long t0 = clock64();
  for (int i = 0; i < iters; ++i) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      tmb::red_release_add(counter, 1ull);
      target += gridDim.x;
      uint32_t polls = 0;
      while (tmb::ld_acquire(counter) < target) {
        if (++polls > (1u << 22)) {   // ~seconds: never reached when the grid is co-resident
          *gave_up = 1;
          break;
        }
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0 && blockIdx.x == 0) cycles[0] = (clock64() - t0) / iters;
}

struct Device {
  int sms = 0;
  double ghz = 1.0;   // SM clock while the benchmark ran, from clock64 against the global timer
};

__global__ void clock_kernel(long long* out) {
  const long long c0 = clock64();
  const unsigned long long n0 = tmb::global_timer();
  while (tmb::global_timer() - n0 < 200000ull) {   // 200 us
  }
  out[0] = clock64() - c0;
  out[1] = (long long)(tmb::global_timer() - n0);
}

int MeasureClock(Device& device) {
  long long* dev = nullptr;
  CAL_CHECK(cudaMalloc(&dev, 16));
  // under load the clock settles first: run a pipe kernel right before
  float* sink = nullptr;
  CAL_CHECK(cudaMalloc(&sink, 4));
  pipe_kernel<0><<<device.sms * 4, 256>>>(sink, 20000);
  clock_kernel<<<1, 1>>>(dev);
  long long host[2] = {0, 1};
  CAL_CHECK(cudaMemcpy(host, dev, 16, cudaMemcpyDeviceToHost));
  cudaFree(dev);
  cudaFree(sink);
  device.ghz = double(host[0]) / double(host[1]);
  return 0;
}

template <typename Launch>
double TimeMs(Launch launch, int repeats = 3) {
  Timer timer;
  launch();   // warm-up
  cudaDeviceSynchronize();
  double best = 1e30;
  for (int r = 0; r < repeats; ++r) {
    timer.start();
    launch();
    best = std::min(best, timer.stop_ms());
  }
  return best;
}

int Run(const std::string& what, double* out, int capacity) {
  Device device;
  int ordinal = 0;
  CAL_CHECK(cudaGetDevice(&ordinal));
  CAL_CHECK(cudaDeviceGetAttribute(&device.sms, cudaDevAttrMultiProcessorCount, ordinal));
  int count = 0;
  auto put = [&](double value) {
    if (count < capacity) out[count] = value;
    ++count;
  };
  float* sink = nullptr;
  CAL_CHECK(cudaMalloc(&sink, 256));
  const int blocks = device.sms * 4, threads = 256, iters = 4096;

  if (what == "clock") {
    if (int status = MeasureClock(device)) return status;
    put(device.ghz * 1e3);   // MHz under load
  } else if (what == "pipes") {
    // G(fl)op/s: fp32 FMA (2 flop), int32 multiply-add, ex2, rsqrt
    const double per_thread = double(iters) * 8 * 8;
    const double work = per_thread * blocks * threads;
    put(2.0 * work / (TimeMs([&] { pipe_kernel<0><<<blocks, threads>>>(sink, iters); }) * 1e6));
    put(2.0 * work / (TimeMs([&] { pipe_kernel<1><<<blocks, threads>>>(sink, iters); }) * 1e6));
    put(work / (TimeMs([&] { pipe_kernel<2><<<blocks, threads>>>(sink, iters / 4); }) * 1e6) / 4);
    put(work / (TimeMs([&] { pipe_kernel<3><<<blocks, threads>>>(sink, iters / 4); }) * 1e6) / 4);
  } else if (what == "tensor") {
    // mma.sync m16n8k16: 2*16*8*16 flop per warp instruction; fp16 then bf16
    const double flop = 2.0 * 16 * 8 * 16 * 8 * double(iters) * blocks * (threads / 32);
    put(flop / (TimeMs([&] { mma_kernel<false><<<blocks, threads>>>(sink, iters); }) * 1e6));
    put(flop / (TimeMs([&] { mma_kernel<true><<<blocks, threads>>>(sink, iters); }) * 1e6));
  } else if (what == "smem") {
    // GB/s of conflict-free 128-bit loads with 1, 2, 4, 8 CTAs per SM (32 KB each), then the slope of
    // time against the conflict degree (strides 1, 2, 4, 8 in 16-byte units) relative to stride 1
    CAL_CHECK(cudaFuncSetAttribute(smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768));
    const double bytes_per_block = double(iters) * 8 * 16 * threads;
    for (int per_sm : {1, 2, 4, 8}) {
      const int grid = device.sms * per_sm;
      put(bytes_per_block * grid / (TimeMs([&] { smem_kernel<<<grid, threads, 32768>>>(sink, iters, 1); }) * 1e6));
    }
    const double base = TimeMs([&] { smem_kernel<<<blocks, threads, 32768>>>(sink, iters, 1); });
    double slope = 0.0;
    for (int stride : {2, 4, 8}) {
      const double ms = TimeMs([&] { smem_kernel<<<blocks, threads, 32768>>>(sink, iters, stride); });
      slope += (ms / base - 1.0) / (stride - 1);
    }
    put(slope / 3.0);
  } else if (what == "latency") {
    // ns per dependent load: L1 (8 KB footprint, cached loads), L2 (8 MB, L1 bypassed), DRAM (2 GB)
    if (int status = MeasureClock(device)) return status;
    const size_t sizes[3] = {8u << 10, 8u << 20, size_t(2) << 30};
    for (int level = 0; level < 3; ++level) {
      const size_t words = sizes[level] / 4, stride = level == 0 ? 32 : 1024 + 32;   // words between hops
      std::vector<uint32_t> host(words, 0);
      size_t at = 0, hops = 0;
      // a cycle that visits the footprint with a large odd stride (coprime with the size)
      const size_t step = (stride | 1) * 33 % words;
      const int chase = level == 0 ? 4096 : 20000;
      const size_t needed = std::min(words, size_t(chase) + 256);   // only the part of the cycle that gets walked
      do {
        const size_t next = (at + step) % words;
        host[at] = uint32_t(next);
        at = next;
        ++hops;
      } while (at != 0 && hops < needed);
      uint32_t* dev = nullptr;
      uint32_t* result = nullptr;
      long long* cycles = nullptr;
      CAL_CHECK(cudaMalloc(&dev, sizes[level]));
      CAL_CHECK(cudaMalloc(&result, 4));
      CAL_CHECK(cudaMalloc(&cycles, 8));
      CAL_CHECK(cudaMemcpy(dev, host.data(), sizes[level], cudaMemcpyHostToDevice));
      if (level == 0) chase_l1_kernel<<<1, 1>>>(dev, chase, result, cycles);
      else chase_kernel<<<1, 1>>>(dev, chase, result, cycles);
      long long taken = 0;
      CAL_CHECK(cudaMemcpy(&taken, cycles, 8, cudaMemcpyDeviceToHost));
      put(double(taken) / chase / device.ghz);
      cudaFree(dev);
      cudaFree(result);
      cudaFree(cycles);
    }
  } else if (what == "l2_curve") {
    // pairs (footprint bytes, GB/s) of repeated reads by the whole device: L2-resident footprints run at
    // the L2 rate, larger ones fall to the DRAM rate
    const size_t footprints[] = {size_t(4) << 20, size_t(16) << 20, size_t(32) << 20, size_t(64) << 20, size_t(96) << 20,
                                 size_t(128) << 20, size_t(256) << 20, size_t(1) << 30};
    uint4* data = nullptr;
    CAL_CHECK(cudaMalloc(&data, size_t(1) << 30));
    CAL_CHECK(cudaMemset(data, 1, size_t(1) << 30));
    for (size_t bytes : footprints) {
      const int passes = int(std::max<size_t>(2, (size_t(4) << 30) / bytes));
      const double ms = TimeMs([&] { read_kernel<<<device.sms * 8, 512>>>(data, bytes / 16, passes, sink); }, 2);
      put(double(bytes));
      put(double(bytes) * passes / (ms * 1e6));
    }
    cudaFree(data);
  } else if (what == "dram") {
    // GB/s of a device-to-device copy of 2 GB (read + write bytes)
    const size_t bytes = size_t(2) << 30;
    uint4 *src = nullptr, *dst = nullptr;
    CAL_CHECK(cudaMalloc(&src, bytes));
    CAL_CHECK(cudaMalloc(&dst, bytes));
    CAL_CHECK(cudaMemset(src, 1, bytes));
    put(2.0 * bytes / (TimeMs([&] { copy_kernel<<<device.sms * 8, 512>>>(src, dst, bytes / 16); }) * 1e6));
    cudaFree(src);
    cudaFree(dst);
  } else if (what == "sync") {
    // ns: uncontended atomicAdd round trip, __threadfence, __syncthreads (256 threads), named barrier (128),
    // cluster barrier (2 CTAs)
    if (int status = MeasureClock(device)) return status;
    unsigned long long* word = nullptr;
    long long* cycles = nullptr;
    CAL_CHECK(cudaMalloc(&word, 64));
    CAL_CHECK(cudaMalloc(&cycles, 64));
    CAL_CHECK(cudaMemset(word, 0, 64));
    sync_kernel<<<1, 256>>>(word, cycles, 2000);
    long long host[4] = {};
    CAL_CHECK(cudaMemcpy(host, cycles, 32, cudaMemcpyDeviceToHost));
    for (int i = 0; i < 4; ++i) put(double(host[i]) / device.ghz);
    cluster_sync_kernel<<<2, 128>>>(cycles, 2000);
    CAL_CHECK(cudaMemcpy(host, cycles, 8, cudaMemcpyDeviceToHost));
    put(double(host[0]) / device.ghz);
    cudaFree(word);
    cudaFree(cycles);
  } else if (what == "atomic_contention" || what == "grid_barrier") {
    // pairs (CTAs, ns): one atomicAdd per CTA on one word, all at once / one grid-wide barrier
    if (int status = MeasureClock(device)) return status;
    unsigned long long* word = nullptr;
    long long* cycles = nullptr;
    int* gave_up = nullptr;
    CAL_CHECK(cudaMalloc(&word, 64));
    CAL_CHECK(cudaMalloc(&cycles, 8 * 1024));
    CAL_CHECK(cudaMalloc(&gave_up, 4));
    for (int ctas : {1, 2, 4, 8, 16, 32, 64, device.sms}) {
      CAL_CHECK(cudaMemset(word, 0, 64));
      CAL_CHECK(cudaMemset(gave_up, 0, 4));
      if (what == "atomic_contention") {
        contention_kernel<<<ctas, 32>>>(word, cycles, 1000);
        std::vector<long long> host(size_t(ctas), 0);
        CAL_CHECK(cudaMemcpy(host.data(), cycles, size_t(ctas) * 8, cudaMemcpyDeviceToHost));
        std::sort(host.begin(), host.end());
        put(ctas);
        put(double(host[host.size() / 2]) / device.ghz);
      } else {
        int iters_barrier = 500;
        void* args[] = {&word, &cycles, &iters_barrier, &gave_up};
        CAL_CHECK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(grid_barrier_kernel), dim3(unsigned(ctas)), dim3(256), args, 0,
                                              nullptr));
        long long host = 0;
        int failed = 0;
        CAL_CHECK(cudaMemcpy(&host, cycles, 8, cudaMemcpyDeviceToHost));
        CAL_CHECK(cudaMemcpy(&failed, gave_up, 4, cudaMemcpyDeviceToHost));
        if (failed) return -3;
        put(ctas);
        put(double(host) / device.ghz);
      }
    }
    cudaFree(word);
    cudaFree(cycles);
    cudaFree(gave_up);
  } else {
    cudaFree(sink);
    return -1;
  }
  CAL_CHECK(cudaDeviceSynchronize());
  cudaFree(sink);
  return count;
}

}  // namespace

extern "C" int tm_calibrate(int device, const char* what, double* out, int capacity) {
  if (!what || !out || capacity < 1) return -1;
  int previous = 0;
  if (cudaGetDevice(&previous) != cudaSuccess || cudaSetDevice(device) != cudaSuccess) return -2;
  const int status = Run(what, out, capacity);
  cudaSetDevice(previous);
  return status > capacity ? -1 : status;
}
