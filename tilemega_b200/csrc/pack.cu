// Weight packing on the device: the reference's `tile_pages` recipe
// (python/tilemega/serving/weights.py:204-242) as a CUDA kernel.
//
// A row-major bf16 matrix [N][K] becomes [ceil(N/tn)][ceil(K/tk)] pages of tn x tk
// elements. Inside a page the 64-column blocks come first, then the 8-row groups, then
// the 8 rows of a group, 128 bytes each, whose eight 16-byte chunks are XOR-swizzled by
// the row: element (row, col) of a page sits at element offset
//   512*(row/8 + (tn/8)*(col/64)) + 64*(row%8) + 8*((col%64/8) ^ (row%8)) + col%8
// (weights.py:239-240). Rows and columns past the matrix are zero. The kernel walks the
// DESTINATION in 16-byte chunks, so every store is coalesced and every load is one
// aligned 16-byte chunk of a source row: pure HBM traffic, N*K*2 bytes in and out.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#include "../../include/tilemega_b200.h"

namespace {

__global__ void tile_pages_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n, long long k,
                                  long long src_pitch_chunks, int tn, int tk, long long kt, long long total_chunks) {
  const long long page_chunks = (long long)tn * tk / 8;
  const int block_chunks = tn * 8;   // chunks of one 64-column block of a page
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_chunks;
       i += (long long)gridDim.x * blockDim.x) {
    const long long page = i / page_chunks;
    const int within = int(i - page * page_chunks);
    const long long row_tile = page / kt, col_tile = page - row_tile * kt;
    const int col_block = within / block_chunks;
    const int row_in_tile = (within - col_block * block_chunks) >> 3;
    const int physical = within & 7;
    const int logical = physical ^ (row_in_tile & 7);
    const long long row = row_tile * tn + row_in_tile;
    const long long col = col_tile * tk + col_block * 64 + logical * 8;
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (row < n && col < k) value = __ldg(src + row * src_pitch_chunks + (col >> 3));
    dst[i] = value;
  }
}

}  // namespace

extern "C" int tm_pack_tile_pages(const void* src, uint64_t rows, uint64_t cols, uint64_t src_pitch, uint32_t tile_n,
                                  uint32_t tile_k, void* dst, void* stream) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  if (!src || !dst || !aligned || rows == 0 || cols == 0 || cols % 8 || src_pitch % 8 || src_pitch < cols || tile_n == 0 ||
      tile_n % 8 || tile_k == 0 || tile_k % 64) {
    std::fprintf(stderr, "tilemega_b200: tm_pack_tile_pages: needs 16-byte aligned bf16 matrices, K and the row pitch "
                         "multiples of 8, tile_n a multiple of 8 and tile_k a multiple of 64\n");
    return -1;
  }
  const long long nt = (long long)((rows + tile_n - 1) / tile_n), kt = (long long)((cols + tile_k - 1) / tile_k);
  const long long total_chunks = nt * kt * (long long)tile_n * tile_k / 8;
  int device = 0, sms = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (err != cudaSuccess) return int(err);
  const int threads = 256;
  const long long wanted = (total_chunks + threads - 1) / threads;
  const int blocks = int(wanted < (long long)sms * 16 ? wanted : (long long)sms * 16);   // a multiple of the SM count when large
  tile_pages_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), (long long)rows, (long long)cols, (long long)(src_pitch / 8),
      int(tile_n), int(tile_k), kt, total_chunks);
  return int(cudaGetLastError());
}
