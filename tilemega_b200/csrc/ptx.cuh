// Thin inline-PTX wrappers used by the persistent decode kernel (sm_100a).
// The same vocabulary the reference wraps in
// include/tilemega/Codegen/executor/Async.cuh:22-259 (mbarrier, bulk copies,
// proxy fences, gpu-scope release/acquire), minus every multicast form.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Contiguous global -> shared bulk copy, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Same, with an L2 eviction-priority hint for data that is read once per step.
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Global -> L2 prefetch of a contiguous range (no shared memory involved).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void red_release_add(unsigned long long* addr, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}

// Counter increment that both publishes this thread's earlier stores (and those ordered before it by a
// barrier) and, for the thread that finds itself last, makes the other arrivers' stores visible.
__device__ __forceinline__ unsigned atom_acq_rel_add(unsigned* addr, unsigned v) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}

__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long* addr) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(addr) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long ld_relaxed(const unsigned long long* addr) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(addr) : "memory");
  return v;
}

// System-scope strong accesses for packets that cross NVLink: a packet is one 8-byte
// word holding data and epoch together, so a reader that sees the epoch has the data
// (include/tilemega/Backend/Sm90DenseEpilogue.h:31-35 uses the same packet idea).
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* addr, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(addr), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* addr) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(addr) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Named barrier over the arithmetic warps only (the streaming warp never joins).
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// bf16 pair <-> fp32 (element 0 in the low half of the word).
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x);
  f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z);
  f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}

// Four 8x8 b16 matrices from shared memory: lane l supplies the address of row
// l%8 of matrix l/8 and receives elements 2*(l%4), 2*(l%4)+1 of row l/4 of each.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

// The transposing form: the same addressing, each 8x8 tile delivered transposed
// (what the B operand of P*V needs from row-major V[key][d]).
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}

// D[16x8] += A[16x8] * B[8x8] (k = 8), bf16 operands, fp32 accumulators, all 16 rows of A in use.
__device__ __forceinline__ void mma_bf16_m16n8k8_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(b0));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
         (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
}

// D[16x8] += A[16x16] * B[16x8], bf16 operands, fp32 accumulators. Rows 8..15 of A
// are zero here (the batch has at most 8 rows), so a1 = a3 = 0.
__device__ __forceinline__ void mma_bf16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

// Round-to-nearest-even fp32 -> bf16, returned as the fp32 value it represents.
__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ uint16_t bf16_bits(float x) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float bf16_from_bits(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

// ---------------------------------------------------------------------------
// 5th-generation tensor cores (tcgen05) and tensor memory, for the dense-batch
// GEMM stages: operands in shared memory (128-byte swizzled, K-major), the fp32
// accumulator in tensor memory, one thread issues, completion arrives on mbarriers.
// ---------------------------------------------------------------------------

// Tiled 2-D tensor copy global -> shared through a tensor map (no multicast). `x` is the
// innermost coordinate in elements and must be a multiple of 8 for 16-bit data.
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tensor_map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// The same with three coordinates (x innermost).
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tensor_map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}

// Tensor memory columns for this CTA (a power of two >= 32); the base address lands in
// shared memory. Executed by one whole warp, which also frees the columns.
__device__ __forceinline__ void tmem_alloc(uint32_t* base_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(base_in_smem)), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups
// `group_bytes` apart (1024 for densely stacked rows). `address` may point 32*j bytes into a
// swizzle row to select k-step j; the atom it lies in must start on a 1024-byte boundary.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t address, uint32_t group_bytes) {
  const uint64_t lo = uint64_t((address >> 4) & 0x3FFFu) | (uint64_t(1) << 16);            // start, leading offset (unused: 1)
  const uint64_t hi = uint64_t((group_bytes >> 4) & 0x3FFFu) | (uint64_t(1) << 14) |       // stride offset, descriptor version 1
                      (uint64_t(2) << 29);                                                  // layout: 128-byte swizzle
  return lo | (hi << 32);
}

// Instruction descriptor of kind::f16: bf16 x bf16 -> fp32, both operands K-major, M x N tile.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread; `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One arrival on `bar` once every tensor-core operation this thread issued so far is complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive fp32 columns of this thread's tensor-memory lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_load_16(uint32_t address, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(address));
  // the registers are valid only after the wait: naming them as operands of the wait keeps the
  // compiler from reading them earlier
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

}  // namespace tmb
