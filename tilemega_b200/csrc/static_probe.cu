// tm_watchdog_probe_static: the bounded-wait self test for callers that must not
// allocate device memory.
//
// Who cannot allocate: a serving process that has already handed every byte of HBM
// to its weight and KV pools (a cudaMalloc there fails, or worse, succeeds by
// evicting something), a health check that runs between decode launches and must
// not pay cudaMalloc's device-wide synchronisation, and code running under a memory
// budget enforced by its host framework. tm_plan_watchdog_probe needs a plan, and a
// plan owns cudaMalloc'd scratch; this entry point needs neither. Its scratch -- the
// arrival word the waiters poll and one record per waiter -- is a file-scope device
// array of fixed size, resident on every GPU that loads the library until the
// process exits (4.4 KB).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <mutex>

#include "../../include/tilemega_b200.h"
#include "params.h"
#include "ptx.cuh"

namespace {

constexpr int kMaxWaiters = TM_STATIC_PROBE_MAX_WAITERS;
constexpr int kRecordStride = 16;                          // words between records (12 used)
constexpr int kRecordBase = 32;                            // word 0 is the arrival counter
constexpr int kScratchWords = kRecordBase + kMaxWaiters * kRecordStride;
constexpr int kMaxDevices = 64;

// Every call uses this one array and it keeps the previous call's contents: the
// entry point clears it on the caller's stream before each launch, and two calls
// whose kernels overlap on the GPU (different streams) would race on it.
static __device__ __align__(256) unsigned long long g_probe_scratch[kScratchWords];

// CTA 0 arrives (unless told to withhold); CTAs 1..waiters each wait for that arrival
// for at most limit_ns, write what happened into their scratch record and copy it to
// the caller's output. Both roles are in ONE launch, so they are co-resident.
__global__ void static_probe_kernel(unsigned long long* scratch, int withhold, unsigned long long limit_ns,
                                    unsigned long long* records) {
  if (threadIdx.x != 0) return;
  if (blockIdx.x == 0) {
    if (!withhold) tmb::red_release_add(scratch, 1ull);
    return;
  }
  unsigned long long* record = scratch + kRecordBase + (blockIdx.x - 1) * kRecordStride;
  const unsigned long long begin = tmb::global_timer();
  unsigned long long seen = 0;
  bool gave_up = false;
  uint32_t polls = 0;
  while ((seen = tmb::ld_acquire(scratch)) < 1ull) {
    if ((++polls & 63u) == 0 && tmb::global_timer() - begin > limit_ns) {
      gave_up = true;
      break;
    }
  }
  record[tmb::kStFired] = gave_up ? 1ull : 0ull;
  record[tmb::kStSite] = gave_up ? tmb::kSiteTest : 0;
  record[tmb::kStBlock] = blockIdx.x;
  record[tmb::kStThread] = 0;
  record[tmb::kStNeed] = 1;
  record[tmb::kStValue] = seen;
  unsigned long long* out = records + size_t(blockIdx.x - 1) * 12;
  for (int i = 0; i < 12; ++i) out[i] = record[i];
}

std::mutex g_setup_mutex;
unsigned long long* g_scratch_address[kMaxDevices] = {};

}  // namespace

extern "C" int tm_watchdog_probe_static(int device, int waiters, int withhold, uint32_t limit_us,
                                        uint64_t* records_device, void* stream) {
  if (waiters < 1 || waiters > kMaxWaiters) {
    std::fprintf(stderr,
                 "tilemega_b200: tm_watchdog_probe_static: %d waiters asked, the static scratch holds records for 1..%d\n",
                 waiters, kMaxWaiters);
    return -1;
  }
  if (device < 0 || device >= kMaxDevices || !records_device || limit_us == 0 || limit_us > 1000000u) {
    std::fprintf(stderr, "tilemega_b200: tm_watchdog_probe_static: bad device, output pointer or time limit\n");
    return -1;
  }
  int previous = 0;
  cudaError_t err = cudaGetDevice(&previous);
  if (err == cudaSuccess && previous != device) err = cudaSetDevice(device);
  if (err != cudaSuccess) return int(err);
  unsigned long long* scratch = nullptr;
  {
    // First call on this device: resolve the array's device address (the symbol's
    // name is only a host-side handle). The device is current here, as it must be.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_address[device]) {
      void* address = nullptr;
      err = cudaGetSymbolAddress(&address, g_probe_scratch);
      if (err == cudaSuccess) g_scratch_address[device] = static_cast<unsigned long long*>(address);
    }
    scratch = g_scratch_address[device];
  }
  if (err == cudaSuccess) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    err = cudaMemsetAsync(scratch, 0, sizeof(unsigned long long) * kScratchWords, s);
    if (err == cudaSuccess) {
      static_probe_kernel<<<1 + waiters, 32, 0, s>>>(scratch, withhold, (unsigned long long)limit_us * 1000ull,
                                                     reinterpret_cast<unsigned long long*>(records_device));
      err = cudaGetLastError();
    }
  }
  if (previous != device) cudaSetDevice(previous);
  if (err != cudaSuccess)
    std::fprintf(stderr, "tilemega_b200: tm_watchdog_probe_static: %s\n", cudaGetErrorString(err));
  return int(err);
}
