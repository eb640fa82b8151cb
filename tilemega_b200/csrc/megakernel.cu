// Persistent decode megakernel for sm_100a.
//
// One launch runs `nsteps` decode steps of a Llama-shaped decoder. Every CTA
// (one per SM) has one streaming warp and eight arithmetic warps:
//
//  * the streaming warp claims tasks of the current stage from a global counter
//    (one atomicAdd per chunk of about 64 KB of pages, issued one chunk ahead), posts each task id into a
//    small shared-memory FIFO and copies the task's data -- weight pages of a GEMV
//    stage, KV block groups of an attention stage -- into a shared-memory ring
//    with cp.async.bulk. It never waits for a stage boundary, only for a free ring
//    slot, so HBM keeps streaming while the arithmetic warps sit in a grid barrier
//    or stage their activations; and because tasks are claimed, not dealt, an SM
//    that streams faster simply takes more of them and every stage ends together.
//  * the arithmetic warps pop the FIFO, wait for the stage's inputs (a grid-wide
//    arrival counter with release/acquire), stage the activation rows in shared
//    memory (RMSNorm fused), and consume ring slots: ldmatrix + mma.sync (bf16 in,
//    fp32 accumulate) for the weight pages and for the attention tiles, then the
//    rounding sites of the reference's epilogues. Results do not depend on which
//    CTA ran a task, so the run-to-run bits are identical.
//
// A third kernel in this file (TMB_DENSE, batch 16..64) keeps the streaming warp and the
// stage list but runs the GEMM stages on tcgen05 tiles with accumulators in tensor memory
// (see "Dense-batch plans" below); with chunk_rows its rows may be consecutive positions
// of one sequence (chunked prefill). A fourth instantiation (TMB_FP8) reads e4m3 weight pages.
//
// Stage list per layer (reference: include/tilemega/Codegen/tasks/
// Sm90DenseProgram.cuh:903-939): qkv (RMSNorm fused) -> RoPE + KV append +
// split-KV attention (+ last-arriver merge) -> o (+residual) -> gate/up
// (RMSNorm, SwiGLU) -> down (+residual); after the last layer lm_head
// (RMSNorm, bf16 logits, argmax partials) and the argmax reduction that also
// feeds the next step's embedding. Attention tasks wait for their own KV group's QKV
// rows (a per-group counter), not for a grid barrier. A second instantiation of the
// kernel (TMB_EXTENDED) adds tensor parallelism (all-reduce packets exchanged over peer
// memory inside the o / down epilogues), a mixture-of-experts MLP (router stage,
// in-kernel top-k, chosen experts only) and the per-head QK norm.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "params.h"
#include "ptx.cuh"

#ifndef TMB_EXTENDED
#define TMB_EXTENDED 0   // 1: the translation unit with tensor parallelism, mixture of experts and QK norm
#endif
#ifndef TMB_FP8
#define TMB_FP8 0        // 1: the translation unit with the e4m3-weight instantiations of the small-batch kernel
#endif
#ifndef TMB_DENSE
#define TMB_DENSE 0      // 1: the translation unit with the dense-batch kernel (GEMM stages on tcgen05 tiles)
#endif

namespace tmb {

// ---------------------------------------------------------------------------
// shared memory map (bytes)
// ---------------------------------------------------------------------------
constexpr int kOffFull = 0;        // u64[8]  ring slot filled
constexpr int kOffEmpty = 64;      // u64[8]  ring slot released by all arithmetic warps
constexpr int kOffCtl = 128;       // int[8]: [0] abort seen, [1] last-arriver flag, [2] FIFO tail, [3] FIFO head, [4] popped task
constexpr int kOffPFull = 192;     // u64[8]  all warps wrote their partial sums of a GEMV task
constexpr int kOffTok = 256;       // int[8]
constexpr int kOffFifo = 320;      // int[kFifo] task ids claimed by the streaming warp, -1 closes a stage
constexpr int kOffBestVal = 448;   // float[8 warps][kMaxBatch]
constexpr int kOffBestIdx = 704;   // int[8 warps][kMaxBatch]
constexpr int kOffWsum = 960;      // float[kMaxBatch][8]
constexpr int kOffSc = 1216;       // routing of the current layer: int expert[8], float weight[8] (+32), mbarrier (+64)
constexpr int kOffRed = 3264;      // float[kPartialRing][8 warps][8 rows][batch]: 2 KB per sequence of the batch
// Dense-batch plans (batch > kMaxBatch) have no GEMV partial-sum area; bytes [kOffRed, kOffDenseXs) hold the
// control words of their GEMM stages instead, and the activation chunks / attention scratch start at kOffDenseXs.
constexpr int kOffDXFull = 3264;     // u64[4] activation chunk landed
constexpr int kOffDXEmpty = 3296;    // u64[4] activation chunk consumed by the tensor cores
constexpr int kOffDAccFull = 3328;   // u64[2] accumulator complete
constexpr int kOffDAccEmpty = 3344;  // u64[2] accumulator read out by its four epilogue warps
constexpr int kOffDDrain = 3360;     // u64    every tensor-core operation of the launch has completed
constexpr int kOffDTmem = 3368;      // u32    tensor memory base address
constexpr int kOffDFifo = 3392;      // int[kFifo] GEMM tasks for the issuing thread: id, first ring slot and its phase
constexpr int kOffDTok = 3520;       // int[kDenseMaxBatch]
constexpr int kOffDBestVal = 3840;   // float[8 warps][kDenseMaxBatch]
constexpr int kOffDBestIdx = 5888;   // int[8 warps][kDenseMaxBatch]
constexpr int kOffDWEmpty = 7936;    // u64[8] ring slot released by the tensor cores (one arrival: tcgen05.commit)
constexpr int kOffDenseXs = 8192;
// Features compiled into an instantiation of the kernel (template parameter X): the plain
// one (0) serves unsharded dense plans and carries neither.
constexpr int kXTp = 1;    // tensor parallelism: all-reduce epilogue, argmax exchange
constexpr int kXMoe = 2;   // mixture of experts and the per-head QK norm
constexpr int kXFp8 = 4;   // weights are e4m3 bytes with fp32 row scales (pages of 8 rows x 4096 columns)
constexpr int kFifo = 32;          // entries; the streaming warp keeps at most kFifo/2 unread

__host__ __device__ inline int xs_offset(int batch) {   // activation rows / attention scratch
  return batch > kMaxBatch ? kOffDenseXs : kOffRed + kPartialRing * 8 * 8 * 4 * batch;
}
__host__ __device__ inline int ring_offset(int xs_bytes, int batch) { return (xs_offset(batch) + xs_bytes + 1023) & ~1023; }

struct Ctx {
  const MegaParams& p;
  unsigned char* smem;
  int warp, lane, tid;
  int cta;                           // this CTA's index in its plan's grid (several plans may share one launch)
  uint32_t slot, phase;              // ring cursor
  unsigned long long bar_target;     // arrivals that complete the previous stage
  uint32_t task_seq;                 // tasks finished by this CTA (epilogue warp rotation)
  bool dead;                         // a bounded wait gave up: stop waiting, leave at the next boundary
  uint32_t q_pos;                    // FIFO entries pushed (streaming warp) / popped (arithmetic warps)
  uint32_t inst;                     // stage instances finished in this launch (index of the claim counter)
  int pending;                       // streaming thread: first task id claimed for the stage about to start
  int pending_next;                  // ... and for the stage after it (claimed a whole stage ahead)
  uint32_t gemv_seq;                 // GEMV tasks finished by this CTA (partial-sum ring cursor)
  uint32_t route_phase;              // routings published (arithmetic warps) / consumed (streaming thread), mod 2
  uint32_t dq_pos;                   // dense plans: GEMM FIFO entries pushed (streaming thread) / popped (issuing thread)
  // dense plans, streaming thread: a slot is released through one of two barriers, by the eight arithmetic
  // warps when it held keys, by one tcgen05.commit when it held a weight page. Per slot: was it filled at
  // all, did it last hold a weight page, and the parity of the next release through either barrier.
  uint32_t slot_used, slot_gemm, parity_warps, parity_mma;
  // streaming thread: where it is in the launch's sequence of weight pages, and how far ahead of
  // that it has prefetched into L2 (absolute page numbers count every GEMV stage's pages in program order)
  __device__ Ctx(const MegaParams& q, unsigned char* s, int cta_index)
      : p(q), smem(s), warp(threadIdx.x >> 5), lane(threadIdx.x & 31), tid(threadIdx.x), cta(cta_index), slot(0), phase(0),
        bar_target(q.bar_base), task_seq(0), dead(false), q_pos(0), inst(0), pending(0), pending_next(0), gemv_seq(0),
        route_phase(0), dq_pos(0), slot_used(0), slot_gemm(0), parity_warps(0), parity_mma(0) {}
  __device__ uint64_t* full(int i) const { return reinterpret_cast<uint64_t*>(smem + kOffFull) + i; }
  __device__ uint64_t* empty(int i) const { return reinterpret_cast<uint64_t*>(smem + kOffEmpty) + i; }
  __device__ uint64_t* pfull(int i) const { return reinterpret_cast<uint64_t*>(smem + kOffPFull) + i; }
  __device__ volatile int* ctl() const { return reinterpret_cast<volatile int*>(smem + kOffCtl); }
  __device__ int* tok() const { return reinterpret_cast<int*>(smem + kOffTok); }
  __device__ float* best_val() const { return reinterpret_cast<float*>(smem + kOffBestVal); }
  __device__ int* best_idx() const { return reinterpret_cast<int*>(smem + kOffBestIdx); }
  __device__ float* wsum() const { return reinterpret_cast<float*>(smem + kOffWsum); }
  __device__ float* red() const { return reinterpret_cast<float*>(smem + kOffRed); }
  __device__ volatile int* route_e() const { return reinterpret_cast<volatile int*>(smem + kOffSc); }
  __device__ volatile float* route_w() const { return reinterpret_cast<volatile float*>(smem + kOffSc + 32); }
  __device__ uint64_t* route_bar() const { return reinterpret_cast<uint64_t*>(smem + kOffSc + 64); }
  __device__ unsigned char* xs() const { return smem + xs_offset(p.batch); }
  __device__ unsigned char* ring(int i) const { return smem + ring_offset(p.xs_bytes, p.batch) + i * kSlotBytes; }
  __device__ void advance() {
    if (++slot == uint32_t(p.nslots)) { slot = 0; phase ^= 1u; }
  }
  __device__ int* fifo() const { return reinterpret_cast<int*>(smem + kOffFifo); }
};

// ---------------------------------------------------------------------------
// bounded waits: no spin in this kernel is unbounded. A wait that exceeds
// watchdog_ns records who waited for what (the 12 words the reference's
// tm_plan_watchdog reports, include/tilemega/Codegen/executor/Watchdog.cuh:13-44)
// and raises status[0]; every other wait sees status[0] and falls through, and
// every CTA leaves at its next stage boundary. Nothing traps.
// ---------------------------------------------------------------------------
static __device__ __noinline__ bool wait_give_up(const MegaParams& p, unsigned long long& t0, int site,
                                          unsigned long long need, unsigned long long value) {
  if (ld_relaxed(p.status + kStFired) != 0) return true;
  const unsigned long long now = global_timer();
  if (t0 == 0) {
    t0 = now;
    return false;
  }
  if (now - t0 <= p.watchdog_ns) return false;
  if (atomicCAS(p.status + kStFired, 0ull, 1ull) == 0ull) {
    p.status[kStSite] = site;
    p.status[kStBlock] = blockIdx.x;
    p.status[kStThread] = threadIdx.x;
    p.status[kStNeed] = need;
    p.status[kStValue] = value;
    __threadfence();
  }
  return true;
}

// Returns false when the wait was abandoned; from then on this thread waits for nothing.
// For a single waiting thread (the streaming thread).
__device__ __forceinline__ bool mbar_wait(Ctx& c, uint64_t* bar, uint32_t parity, int site) {
  if (c.dead) return false;
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 31u) == 0 && wait_give_up(c.p, t0, site, parity, polls)) {
      c.dead = true;
      return false;
    }
  }
  return true;
}

// The same for a whole warp: only lane 0 polls (thirty-two lanes spinning on one
// barrier word crowd the shared-memory pipeline that the other warps' loads and the
// streaming thread's copies go through); afterwards every lane observes the
// completed phase once itself, which is its acquire of the data behind it.
__device__ __forceinline__ bool mbar_wait_warp(Ctx& c, uint64_t* bar, uint32_t parity, int site) {
  if (c.dead) return false;
  // the common case: already there. One decision for the warp (lanes polling at
  // slightly different moments may see different answers).
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  bool ok = true;
  if (c.lane == 0) ok = mbar_wait(c, bar, parity, site);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (!ok) {
    c.dead = true;
    return false;
  }
  mbar_try_wait(bar, parity);
  return true;
}

// Arrive on the grid-wide counter: this CTA's stage outputs are in global memory.
__device__ __forceinline__ void grid_arrive(Ctx& c) {
  // dense-batch plans: the next stage reads this stage's rows with the copy engine (async proxy), so
  // every thread first orders its own ordinary stores before that proxy
  if (c.p.dense) fence_proxy_async();
  consumer_sync();
  // The CTA barrier orders every thread's stores before thread 0's release, and a release is
  // cumulative: no separate fence (one costs about half a microsecond per stage boundary).
  if (c.tid == 0) red_release_add(c.p.bar, 1ull);
  c.bar_target += (unsigned long long)c.p.grid;
}

// Wait until every CTA arrived for the previous stage. Returns false when the
// launch is being abandoned (uniform over the arithmetic warps).
__device__ __forceinline__ bool grid_wait(Ctx& c) {
  if (c.tid == 0) {
    unsigned long long t0 = 0;
    uint32_t polls = 0;
    unsigned long long seen;
    // "has a wait given up anywhere" is read while the arrivals are polled for, not after them: as a
    // dependent load behind the barrier it cost every stage boundary one more L2 round trip (a flag set
    // during this wait is seen by the next one)
    unsigned long long fired = ld_relaxed(c.p.status + kStFired);
    while ((seen = ld_acquire(c.p.bar)) < c.bar_target) {
      if ((++polls & 63u) == 0) {
        if (wait_give_up(c.p, t0, kSiteGrid, c.bar_target, seen)) {
          fired = 1;
          break;
        }
      }
    }
    c.ctl()[0] = fired != 0 ? 1 : 0;
  }
  consumer_sync();
  return c.ctl()[0] == 0;
}

// Optional stage trace (one chosen step): per CTA and stage, %globaltimer when the
// CTA started waiting for the stage's inputs, when they were there, when its
// activation rows were staged and when its last task was done. The reference's
// counterpart is the TILEMEGA_TRACE_STAGE build
// (include/tilemega/Codegen/tasks/ModelRuntime.h:758-766).
__device__ __forceinline__ void trace_mark(const Ctx& c, bool on, int stage, int what) {
  if (on && c.tid == 0) {
    c.p.trace[(size_t(c.cta) * c.p.trace_stages + stage) * 4 + what] = global_timer();
  }
}

// ---------------------------------------------------------------------------
// attention partition (identical on the streaming and the arithmetic side)
// ---------------------------------------------------------------------------
struct AttnTask {
  int b, g, c;       // row of the batch, KV head, chunk
  int sq;            // the sequence the row belongs to (= b outside prefill plans)
  int pos;           // position of the new token (= number of cached tokens)
  int ns, nch;       // slots of the sequence, chunks per KV head
  int slot0, slot1;  // slot range of this chunk
  int task0;         // first task of (b, g)
};

// Which sequence row b of the batch belongs to (its block-table row, its token row): itself, except in a
// prefill plan, whose rows are (sequence, position) pairs listed per step (`past` is then the step's first pair).
__device__ __forceinline__ int seq_of(const MegaParams& p, int past, int b) {
  return p.row_seq ? __ldg(p.row_seq + past + b) : b;
}

__device__ __forceinline__ int seq_pos(const MegaParams& p, int past, int b) {
  int pos;
  if (p.row_pos) {
    pos = __ldg(p.row_pos + past + b);   // resolved by the host at launch: position in the prompt + context_base
  } else {
    pos = past + (p.ctx_base ? __ldg(p.ctx_base + b) : 0);
  }
  return min(max(pos, 0), p.capacity - 1);
}

// The rows' positions and sequences, fetched ONCE per stage by every warp that partitions the stage: lane l
// holds rows l and l + 32 (a batch has at most 64 rows) and hands them out by shuffle. The partition below
// walks over the rows one after another; with a global load per row and step (which misses the small L1 left
// beside 227 KB of shared memory) that walk was tens of microseconds at batch 64, on the streaming warp
// before its first copy and on the arithmetic warps before their first product. Every function that takes a
// Rows must be called by all 32 lanes of a warp together.
struct Rows {
  int p0, p1, s0, s1;
};

__device__ __forceinline__ Rows load_rows(const MegaParams& p, int past) {
  const int lane = threadIdx.x & 31;
  Rows r;
  r.p0 = lane < p.batch ? seq_pos(p, past, lane) : 0;
  r.p1 = lane + 32 < p.batch ? seq_pos(p, past, lane + 32) : 0;
  r.s0 = lane < p.batch ? seq_of(p, past, lane) : 0;
  r.s1 = lane + 32 < p.batch ? seq_of(p, past, lane + 32) : 0;
  return r;
}
__device__ __forceinline__ int row_pos(const Rows& r, int b) { return __shfl_sync(0xffffffffu, b < 32 ? r.p0 : r.p1, b & 31); }
__device__ __forceinline__ int row_seq(const Rows& r, int b) { return __shfl_sync(0xffffffffu, b < 32 ? r.s0 : r.s1, b & 31); }
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
  for (int m = 16; m; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// slots-per-task and task count for one attention stage
__device__ __forceinline__ int attn_count(const MegaParams& p, const Rows& rw, int nk, int spt) {
  const int lane = threadIdx.x & 31;
  int mine = 0;
  if (lane < p.batch) mine += (rw.p0 / nk + 1 + spt - 1) / spt;
  if (lane + 32 < p.batch) mine += (rw.p1 / nk + 1 + spt - 1) / spt;
  return p.kv_heads * warp_sum(mine);
}

// How one attention stage is cut into tasks. Two regimes:
//  * little work per CTA (per == 0): a task is one chunk of `spt` slots of one (sequence, KV head);
//  * much work per CTA (per > 0): the slots of all (sequence, KV head) units, laid end to end in
//    (sequence, head, slot) order, are cut into `ntasks` <= grid RANGES of `per` slots, one claim
//    each, so every CTA streams the same number of slots whatever the sequences' lengths; a range
//    is worked through as the SEGMENTS where it meets the units, each segment a partial of its unit.
//    A segment has a fixed cost (readiness, RoPE staging, merge: about four slots' worth of time), so
//    the axis the ranges cut is slots PLUS that cost per unit: with sequences of very different
//    lengths a range over many short units would otherwise take much longer than one inside a long unit
//    (batch 64, contexts 512..8192: the slowest CTA took 242 us, the median one 195 us).
struct AttnShape {
  int spt, ntasks, per, total;
  int fixed;   // ranges are measured in slots plus `fixed` per unit: what a segment costs before its first slot
};

__device__ __forceinline__ AttnShape attn_shape(const MegaParams& p, const Rows& rw, int nk) {
  const int lane = threadIdx.x & 31;
  AttnShape sh;
  sh.total = p.kv_heads * warp_sum((lane < p.batch ? rw.p0 / nk + 1 : 0) + (lane + 32 < p.batch ? rw.p1 / nk + 1 : 0));
  const int floor_spt = max(1, p.attn_min_spt);   // a task's fixed cost wants at least this many slots
  const int per_cta = (sh.total + p.grid - 1) / p.grid;
  sh.fixed = 0;
  if (per_cta >= 2 * floor_spt) {
    sh.fixed = floor_spt;
    sh.total += p.batch * p.kv_heads * sh.fixed;       // slots plus the fixed cost of every unit
    sh.per = (sh.total + p.grid - 1) / p.grid;
    sh.spt = sh.per;
    sh.ntasks = (sh.total + sh.per - 1) / sh.per;
    return sh;
  }
  sh.per = 0;
  sh.spt = max(floor_spt, per_cta);
  sh.ntasks = attn_count(p, rw, nk, sh.spt);
  // every task owns one record of partial results: never more tasks than records
  while (sh.ntasks > p.attn_part_tasks) {
    sh.spt += 1;
    sh.ntasks = attn_count(p, rw, nk, sh.spt);
  }
  return sh;
}

__device__ __forceinline__ AttnTask attn_task(const MegaParams& p, const Rows& rw, int nk, int spt, int t) {
  AttnTask a;
  int base = 0;
  for (int b = 0;; ++b) {
    const int pos = row_pos(rw, b);
    const int ns = pos / nk + 1;
    const int nch = (ns + spt - 1) / spt;
    const int n = p.kv_heads * nch;
    if (t < base + n || b == p.batch - 1) {
      const int r = t - base;
      a.b = b;
      a.sq = row_seq(rw, b);
      a.g = r / nch;
      a.c = r % nch;
      a.pos = pos;
      a.ns = ns;
      a.nch = nch;
      const int even = (ns + nch - 1) / nch;   // the chunks of a sequence are equally long (even <= spt: none is empty)
      a.slot0 = a.c * even;
      a.slot1 = min(ns, a.slot0 + even);
      a.task0 = base + a.g * nch;
      return a;
    }
    base += n;
  }
}

// The segments of claimed task t, one after another (a chunk task has exactly one).
struct AttnWalk {
  int t, x, x1;        // task; next flattened slot and the end of the range
  int b, base, ns;     // sequence under the cursor, its first flattened slot, its slots per KV head
  bool done;
};

__device__ __forceinline__ AttnWalk attn_walk(const MegaParams& p, const Rows& rw, int nk, const AttnShape& sh, int t) {
  AttnWalk w;
  w.t = t;
  w.done = false;
  w.x = t * sh.per;
  w.x1 = min(sh.total, w.x + sh.per);
  w.b = 0;
  w.base = 0;
  w.ns = row_pos(rw, 0) / nk + 1;
  return w;
}

// Next segment of the walk into `a`; false when the task is exhausted. A unit (sequence b, head g)
// occupies flattened slots [u0, u0 + ns); the ranges that meet it are u0 / per .. (u0 + ns - 1) / per,
// and its partial records are consecutive from (first such range) + (unit index): along the
// flattened axis every new segment advances the range, the unit or both, so no two segments
// share a record and there are at most ntasks + B * Hkv of them.
__device__ __forceinline__ bool attn_next(const MegaParams& p, const Rows& rw, int nk, const AttnShape& sh, AttnWalk& w,
                                          AttnTask& a) {
  if (sh.per == 0) {
    if (w.done) return false;
    w.done = true;
    a = attn_task(p, rw, nk, sh.spt, w.t);
    return true;
  }
  // a unit occupies [u0, u0 + fixed + ns) of the axis: its fixed cost first, then its slots; the part of the
  // range inside the slots is a segment (a range that only touches a unit's fixed cost holds none of it)
  for (;;) {
    if (w.x >= w.x1) return false;
    while (w.x >= w.base + (w.ns + sh.fixed) * p.kv_heads && w.b < p.batch - 1) {
      w.base += (w.ns + sh.fixed) * p.kv_heads;
      ++w.b;
      w.ns = row_pos(rw, w.b) / nk + 1;
    }
    const int cost = w.ns + sh.fixed;
    const int g = min((w.x - w.base) / cost, p.kv_heads - 1);
    const int u0 = w.base + g * cost;
    const int lo = max(w.x, u0 + sh.fixed), hi = min(w.x1, u0 + cost);
    w.x = min(w.x1, u0 + cost);
    if (lo >= hi) continue;
    const int first = (u0 + sh.fixed) / sh.per, last = (u0 + cost - 1) / sh.per;
    a.b = w.b;
    a.sq = row_seq(rw, w.b);
    a.g = g;
    a.pos = row_pos(rw, w.b);
    a.ns = w.ns;
    a.nch = last - first + 1;
    a.c = lo / sh.per - first;
    a.slot0 = lo - (u0 + sh.fixed);
    a.slot1 = hi - (u0 + sh.fixed);
    a.task0 = first + w.b * p.kv_heads + g;
    return true;
  }
}

__device__ __forceinline__ int table_entry(const MegaParams& p, int b, int blk) {
  int e = __ldg(p.block_table + (long long)b * p.max_blocks + min(blk, p.max_blocks - 1));
  return min(max(e, 0), p.kv_max_entry);
}

// ---------------------------------------------------------------------------
// task FIFO between the streaming thread and the arithmetic warps. One 32-bit
// word per entry carries both the task id (low 20 bits; 0xFFFFF closes a stage)
// and the entry's sequence number (high 12 bits), so a reader needs exactly one
// load and no ordering between two locations.
// ---------------------------------------------------------------------------
constexpr uint32_t kFifoClose = 0xFFFFFu;

__device__ __forceinline__ uint32_t fifo_word(uint32_t pos, uint32_t value) { return ((pos + 1u) << 20) | value; }

// Streaming thread: append one entry (a task id, or -1 to close the stage).
__device__ __forceinline__ void fifo_push(Ctx& c, int value) {
  if (!c.dead) {
    volatile int* head = c.ctl() + 3;
    if (int(c.q_pos) - *head >= kFifo / 2) {
      unsigned long long t0 = 0;
      uint32_t polls = 0;
      while (int(c.q_pos) - *head >= kFifo / 2) {
        if ((++polls & 255u) == 0 && wait_give_up(c.p, t0, kSiteEmpty, c.q_pos, uint32_t(*head))) break;
      }
    }
    reinterpret_cast<volatile uint32_t*>(c.fifo())[c.q_pos & (kFifo - 1)] =
        fifo_word(c.q_pos, value < 0 ? kFifoClose : uint32_t(value));
  }
  ++c.q_pos;
}

// Arithmetic thread: next entry of the FIFO; -1 closes the stage, -2 means the
// launch is being abandoned (also treated as the end of the stage).
__device__ __forceinline__ int fifo_pop(Ctx& c) {
  const volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(c.fifo()) + (c.q_pos & (kFifo - 1));
  const uint32_t tag = (c.q_pos + 1u) & 0xFFFu;
  uint32_t word = *slot;
  if (!c.dead && (word >> 20) != tag) {
    unsigned long long t0 = 0;
    uint32_t polls = 0;
    while (((word = *slot) >> 20) != tag) {
      if ((++polls & 255u) == 0 && wait_give_up(c.p, t0, kSiteFull, c.q_pos, word)) {
        c.dead = true;
        break;
      }
    }
  }
  if (c.dead) return -2;
  ++c.q_pos;
  if (c.tid == 0) c.ctl()[3] = int(c.q_pos);
  const uint32_t value = word & kFifoClose;
  return value == kFifoClose ? -1 : int(value);
}

// The same, decided once for all arithmetic warps (stages whose tasks contain
// CTA-wide barriers must agree on every task, also while giving up).
__device__ __forceinline__ int fifo_pop_uniform(Ctx& c) {
  if (c.tid == 0) c.ctl()[4] = fifo_pop(c);
  consumer_sync();
  const int v = c.ctl()[4];
  if (c.tid != 0 && v != -2) ++c.q_pos;
  return v;
}

// ---------------------------------------------------------------------------
// streaming warp: lane 0 runs it (the other lanes only share the scattered copies
// of an attention slot, see stream_attn). A lone warp issues slowly next to eight
// busy arithmetic warps, so every instruction on this path costs ring refill rate;
// the loop is kept to a wait, a byte-count arrive and a bulk copy per slot.
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool stream_wait_empty(Ctx& c, bool weight_page = true) {
  if (c.p.dense) {
    // wait for the release that matches what the slot held, then note what it is about to hold
    const uint32_t bit = 1u << c.slot;
    bool ok = true;
    if (c.slot_used & bit) {
      if (c.slot_gemm & bit) {
        ok = mbar_wait(c, reinterpret_cast<uint64_t*>(c.smem + kOffDWEmpty) + c.slot, (c.parity_mma >> c.slot) & 1u, kSiteEmpty);
        c.parity_mma ^= bit;
      } else {
        ok = mbar_wait(c, c.empty(c.slot), (c.parity_warps >> c.slot) & 1u, kSiteEmpty);
        c.parity_warps ^= bit;
      }
    }
    c.slot_used |= bit;
    c.slot_gemm = weight_page ? (c.slot_gemm | bit) : (c.slot_gemm & ~bit);
    return ok;
  }
  return mbar_wait(c, c.empty(c.slot), c.phase ^ 1u, kSiteEmpty);
}

// Claim the next task of stage instance `inst`. The value is not needed until the
// current task's copies are issued, so the atomic's round trip overlaps them.
__device__ __forceinline__ int claim(const Ctx& c, uint32_t inst) {
  return int(atomicAdd(c.p.stage_cnt + inst, 1u));
}

// Close the stage: tell the arithmetic warps. The first task of the next stage was
// claimed a whole stage ago, so its id is here without waiting for a round trip
// (an attention stage has nothing in the ring to hide one behind); claim the first
// task of the stage after that now.
__device__ __forceinline__ void stream_close(Ctx& c) {
  fifo_push(c, -1);
  ++c.inst;
  c.pending = c.pending_next;
  c.pending_next = claim(c, c.inst + 1);
}

// Dense plans: the thread that issues the tensor-core work gets every GEMM task through a FIFO of its
// own, each entry carrying the task id (16 bits; 0xFFFF closes a stage), the ring slot the task's
// first page goes to and that slot's phase, under the entry's sequence tag.
constexpr uint32_t kDFifoClose = 0xFFFFu;

__device__ __forceinline__ void dfifo_push(Ctx& c, int value, uint32_t slot, uint32_t phase) {
  if (!c.dead) {
    volatile int* head = c.ctl() + 6;
    if (int(c.dq_pos) - *head >= kFifo / 2) {
      unsigned long long t0 = 0;
      uint32_t polls = 0;
      while (int(c.dq_pos) - *head >= kFifo / 2) {
        if ((++polls & 255u) == 0 && wait_give_up(c.p, t0, kSiteEmpty, c.dq_pos, uint32_t(*head))) break;
      }
    }
    reinterpret_cast<volatile uint32_t*>(c.smem + kOffDFifo)[c.dq_pos & (kFifo - 1)] =
        (((c.dq_pos + 1u) & 0xFFFu) << 20) | (slot << 17) | (phase << 16) | (value < 0 ? kDFifoClose : uint32_t(value));
  }
  ++c.dq_pos;
}

// One GEMV task: post its id, then copy its weight pages (consecutive from `src`) into the ring.
__device__ __forceinline__ void stream_pages(Ctx& c, const GemvGeo& geo, const unsigned char* src, int id,
                                             uint32_t page_bytes, uint64_t policy) {
  fifo_push(c, id);
  if (c.p.dense) dfifo_push(c, id, c.slot, c.phase);
  for (int pg = 0; pg < geo.pages_per_task; ++pg, src += page_bytes) {
    if (!stream_wait_empty(c)) return;
    // the last page of a padded reduction: its pad columns (whole 64-column blocks at the
    // end of the page, which no warp reads) are not copied
    const uint32_t bytes = pg + 1 == geo.pages_per_task ? uint32_t(geo.last_page_bytes) : page_bytes;
    mbar_expect_tx(c.full(c.slot), bytes);
    bulk_g2s_hint(c.ring(c.slot), src, bytes, c.full(c.slot), policy);
    c.advance();
  }
}

// task t = one row tile over the whole reduction: its pages start at page t * pages_per_task
__device__ __forceinline__ void stream_gemv_task(Ctx& c, const GemvGeo& geo, const unsigned char* weights, int t,
                                                 uint32_t page_bytes, uint64_t policy) {
  stream_pages(c, geo, weights + (size_t(t) * size_t(geo.task_pages) + size_t(geo.page0)) * page_bytes, t, page_bytes, policy);
}

__device__ __forceinline__ void stream_gemv(Ctx& c, const GemvGeo& geo, const void* weights, uint64_t policy) {
  const uint32_t page_bytes = uint32_t(geo.page_bytes);
  const unsigned char* w = static_cast<const unsigned char*>(weights);
  // Tasks are claimed in chunks of geo.claim_chunk (about 64 KB of pages): the claim for the
  // next chunk is in flight while this one is copied, and its round trip to L2 and back
  // (~1 us) must not be longer than that copying, or short tasks wait for their ids.
  const int chunk_tasks = geo.claim_chunk;
  int chunk = c.pending;
  while (chunk * chunk_tasks < geo.ntasks && !c.dead) {
    const int upcoming = claim(c, c.inst);
    for (int j = 0; j < chunk_tasks; ++j) {
      const int t = chunk * chunk_tasks + j;
      if (t < geo.ntasks) stream_gemv_task(c, geo, w, t, page_bytes, policy);
    }
    chunk = upcoming;
  }
  stream_close(c);
  if (c.p.dense) dfifo_push(c, -1, 0u, 0u);
}

// Mixture of experts, batch 1. gate/up: the chosen experts' matrices one after the other,
// task t = (expert slot t / tiles, row tile t % tiles). `stack` holds every expert packed
// by itself, experts geo.ntasks * pages_per_task pages apart.
__device__ __forceinline__ void stream_expert_gate_up(Ctx& c, const GemvGeo& geo, const void* stack,
                                                      const int (&expert)[kMaxTopK], uint64_t policy) {
  const uint32_t page_bytes = uint32_t(geo.page_bytes);
  const unsigned char* w = static_cast<const unsigned char*>(stack);
  const int total = c.p.topk * geo.ntasks;
  const int chunk_tasks = geo.claim_chunk;
  int chunk = c.pending;
  int slot = 0, tile = 0, at = 0;   // (expert slot, row tile) of task `at`: claims only grow, so no division is needed
  while (chunk * chunk_tasks < total && !c.dead) {
    const int upcoming = claim(c, c.inst);
    for (int j = 0; j < chunk_tasks; ++j) {
      const int t = chunk * chunk_tasks + j;
      if (t >= total) break;
      tile += t - at;
      at = t;
      while (tile >= geo.ntasks) {
        tile -= geo.ntasks;
        ++slot;
      }
      stream_pages(c, geo, w + (size_t(expert[slot]) * geo.ntasks + tile) * size_t(geo.pages_per_task) * page_bytes, t,
                   page_bytes, policy);
    }
    chunk = upcoming;
  }
  stream_close(c);
}

// down: a claimed task is one row tile over ALL chosen experts (their outputs are summed
// per row in rank order by one warp); it is posted as topk sub-tasks of one page each.
__device__ __forceinline__ void stream_expert_down(Ctx& c, const GemvGeo& geo, const void* stack,
                                                   const int (&expert)[kMaxTopK], uint64_t policy) {
  const uint32_t page_bytes = uint32_t(geo.page_bytes);
  const unsigned char* w = static_cast<const unsigned char*>(stack);
  int t = c.pending;
  while (t < geo.ntasks && !c.dead) {
    const int upcoming = claim(c, c.inst);
    for (int slot = 0; slot < c.p.topk; ++slot)
      stream_pages(c, geo, w + (size_t(expert[slot]) * geo.ntasks + t) * page_bytes, t * kMaxTopK + slot, page_bytes,
                   policy);   // id = tile * 8 + slot: the arithmetic warps split it with a shift and a mask
    t = upcoming;
  }
  stream_close(c);
}

// The streaming WARP (all 32 lanes; every other streaming function runs on lane 0 alone, which owns
// the ring cursor, the claims and the FIFO). A ring slot of keys and values is 2 * NB pieces of one
// KV block of one head each, scattered over the pool by the block table: lane j < 2 * NB looks up
// its own block and issues its own copy, so a slot costs the issuing side one table load, one
// address and one copy in parallel instead of 2 * NB of each in a row -- a single thread issuing
// them one after another sustains about 0.7 of the HBM rate on long contexts.
template <int D>
__device__ __forceinline__ void stream_attn(Ctx& c, const LayerPtrs& lp, int past) {
  constexpr int NK = kAttnHalfBytes / (2 * D);   // keys per slot
  constexpr int NB = NK / kKvBlock;              // KV blocks per slot
  constexpr uint32_t BLKB = kKvBlock * D * 2;    // bytes of one block of one head
  static_assert(2 * NB <= 32, "one lane per piece of a slot");
  constexpr unsigned kAll = 0xffffffffu;
  const bool lead = c.lane == 0;
  const int piece = c.lane % NB;                 // block of the slot this lane copies
  const bool is_v = c.lane >= NB;
  const unsigned char* pool = static_cast<const unsigned char*>(is_v ? lp.v_pool : lp.k_pool);
  const Rows rw = load_rows(c.p, past);
  const AttnShape sh = attn_shape(c.p, rw, NK);
  int t = __shfl_sync(kAll, c.pending, 0);
  bool dead = __shfl_sync(kAll, c.dead ? 1 : 0, 0) != 0;
  while (t < sh.ntasks && !dead) {
    int upcoming = 0;
    if (lead) {
      upcoming = claim(c, c.inst);
      fifo_push(c, t);
    }
    AttnWalk walk = attn_walk(c.p, rw, NK, sh, t);
    AttnTask a;
    while (!dead && attn_next(c.p, rw, NK, sh, walk, a)) {
      const int nblk = a.pos / kKvBlock + 1;
      // Block-table entries in windows of 32 consecutive blocks, one per lane (one coalesced load), the
      // NEXT window fetched while this one is used: a slot's entries then come out of registers by
      // shuffle. Fetched per slot, right before the copies that need them, every slot waited for an
      // L2 round trip (the small L1 beside 227 KB of shared memory does not keep the table).
      int win0 = a.slot0 * NB;
      int win = table_entry(c.p, a.sq, win0 + c.lane), ahead = table_entry(c.p, a.sq, win0 + 32 + c.lane);
      for (int s = a.slot0; s < a.slot1; ++s) {
        const int nb = min(NB, nblk - s * NB);
        if (s * NB >= win0 + 32) {   // (32 is a multiple of NB: a slot never straddles two windows)
          win0 += 32;
          win = ahead;
          ahead = table_entry(c.p, a.sq, win0 + 32 + c.lane);
        }
        const long long e = __shfl_sync(kAll, win, s * NB - win0 + min(piece, max(nb - 1, 0)));
        const long long off = (e * c.p.kv_block_stride + (long long)a.g * c.p.kv_head_stride) * 2;
        int word = -1;                           // the slot to fill, or -1: the wait gave up
        if (lead && stream_wait_empty(c, false)) {
          if (nb > 0) mbar_expect_tx(c.full(c.slot), uint32_t(nb) * 2u * BLKB);
          else mbar_arrive(c.full(c.slot));
          word = int(c.slot);
          c.advance();
        }
        word = __shfl_sync(kAll, word, 0);       // (also orders the expectation before the copies)
        if (word < 0) {
          dead = true;
          break;
        }
        if (c.lane < 2 * NB && piece < nb)
          bulk_g2s(c.ring(uint32_t(word)) + (is_v ? kAttnHalfBytes : 0) + piece * BLKB, pool + off, BLKB, c.full(uint32_t(word)));
      }
    }
    t = __shfl_sync(kAll, upcoming, 0);
    dead = __shfl_sync(kAll, (dead || c.dead) ? 1 : 0, 0) != 0;
  }
  if (lead) stream_close(c);
  __syncwarp();
}

// Lane 0's part of a layer before its attention stage: QKV pages, and the ordering of the cache rows
// the previous step appended.
__device__ __forceinline__ void stream_layer_head(Ctx& c, const LayerPtrs& lp, int si, int layer, bool& kv_ordered, uint64_t policy) {
  const MegaParams& p = c.p;
  const uint32_t norm_bytes = uint32_t(p.hidden) * 2u;
  // the RMSNorm weights are read by every CTA right after a barrier: have them in L2 by then
  bulk_prefetch_l2(lp.norm1, norm_bytes);
  bulk_prefetch_l2(lp.norm2, norm_bytes);
  stream_gemv(c, p.geo[kQkv], lp.qkv, policy);
  if (!kv_ordered) {
    // KV rows appended by the previous step were written with ordinary stores by other CTAs: take the
    // previous step's last grid barrier before any bulk (async-proxy) read of the pools
    const unsigned long long need = p.bar_base + (unsigned long long)p.bars_per_step * (unsigned long long)si * p.grid;
    unsigned long long t0 = 0, seen;
    uint32_t polls = 0;
    while ((seen = ld_acquire(p.bar)) < need) {
      if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSiteGrid, need, seen)) break;
    }
    kv_ordered = true;
  }
  if (p.chunk_rows) {
    // this layer's keys and values of ALL rows are appended (arrival 3 of the layer: norm1, QKV, append)
    const unsigned long long need =
        p.bar_base + ((unsigned long long)p.bars_per_step * (unsigned long long)si + 8ull * (unsigned long long)layer + 3ull) * p.grid;
    unsigned long long t0 = 0, seen;
    uint32_t polls = 0;
    while ((seen = ld_acquire(p.bar)) < need) {
      if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSiteGrid, need, seen)) break;
    }
  }
}

// Lane 0's part of a layer after its attention stage. False: the launch is being abandoned.
template <int X>
__device__ __forceinline__ bool stream_layer_tail(Ctx& c, const LayerPtrs& lp, uint64_t policy) {
  const MegaParams& p = c.p;
  stream_gemv(c, p.geo[kOProj], lp.o, policy);
  if ((X & kXMoe) && p.experts) {
    stream_gemv(c, p.geo[kRouter], lp.router, policy);
    for (int b = 0; b < p.batch; ++b) {   // token by token, as the arithmetic warps route them
      // the token's experts are known once the arithmetic warps have routed it
      if (!mbar_wait(c, c.route_bar(), c.route_phase, kSiteFull)) return false;
      c.route_phase ^= 1u;
      int expert[kMaxTopK];
#pragma unroll
      for (int i = 0; i < kMaxTopK; ++i) expert[i] = c.route_e()[i];
      stream_expert_gate_up(c, p.geo[kGateUp], lp.gate_up, expert, policy);
      stream_expert_down(c, p.geo[kDown], lp.down, expert, policy);
    }
  } else {
    stream_gemv(c, p.geo[kGateUp], lp.gate_up, policy);
    if (p.down_splits > 1) {
      for (int part = 0; part < p.down_splits; ++part) stream_gemv(c, p.down_part[part], lp.down, policy);
    } else {
      stream_gemv(c, p.geo[kDown], lp.down, policy);
    }
  }
  return !(c.dead || ld_relaxed(p.status + kStFired) != 0);
}

// The streaming warp. Lane 0 runs everything except the attention stages' copies, which the lanes share.
template <int D, int X>
__device__ void streamer_main(Ctx& c) {
  const MegaParams& p = c.p;
  const uint64_t policy = policy_evict_first();
  const bool lead = c.lane == 0;
  if (lead) {
    c.pending = claim(c, 0);
    c.pending_next = claim(c, 1);
  }
  for (int si = 0; si < p.nsteps; ++si) {
    const int past = __ldg(p.past + p.first_step + si);
    bool kv_ordered = si == 0;
    for (int l = 0; l < p.layers; ++l) {
      const LayerPtrs lp = p.layer[l];
      if (lead) stream_layer_head(c, lp, si, l, kv_ordered, policy);
      __syncwarp();
      // lane 0 has just taken the previous step's last barrier: every lane's copies read cache rows
      // that ordinary stores of other CTAs wrote before it (once per step; the fence is not cheap)
      if ((l == 0 && si > 0) || p.chunk_rows) fence_proxy_async();
      stream_attn<D>(c, lp, past);
      int go = 1;
      if (lead) go = stream_layer_tail<X>(c, lp, policy) ? 1 : 0;
      if (__shfl_sync(0xffffffffu, go, 0) == 0) return;
    }
    if (lead) {
      bulk_prefetch_l2(p.final_norm, uint32_t(p.hidden) * 2u);
      stream_gemv(c, p.geo[kHead], p.lm_head, policy);
    }
  }
}

// Before the CTA may retire, every bulk copy this warp issued must have landed:
// slots below the cursor were last filled in the current lap, the others in the
// previous one (a never-used barrier reports its "previous" phase complete).
__device__ __forceinline__ void streamer_drain(Ctx& c) {
  for (int i = 0; i < c.p.nslots; ++i) {
    const uint32_t parity = uint32_t(i) < c.slot ? c.phase : (c.phase ^ 1u);
    unsigned long long t0 = 0;
    uint32_t polls = 0;
    while (!mbar_try_wait(c.full(i), parity)) {
      if ((++polls & 127u) == 0) {
        // keep waiting past an abort: only the time limit ends this loop
        const unsigned long long now = global_timer();
        if (t0 == 0) t0 = now;
        else if (now - t0 > c.p.watchdog_ns) break;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// arithmetic warps: GEMV
// ---------------------------------------------------------------------------
struct GemvIo {
  const void* src;     // bf16 [B][k] activation rows (global), or embedding table when embed != 0
  const void* norm;    // bf16 [k] RMSNorm weight, or null
  int embed;           // rows are table[tok[b]] and are also copied into x
  int epilogue;
  void* out;           // kEpiStore: bf16 [B][n]; kEpiResidual: x; kEpiSwiGLU: h [B][n/2]; kEpiHead: logits
  unsigned long long* ready;   // kEpiStore: per-group counters bumped once per stored row tile (or null)
  int tiles_per_group;
  const float* partial_in;     // fp32 sums of the earlier parts of a split reduction, added before any rounding (or null)
  int ar_region;               // kEpiResidualAllReduce: which of the two packet regions (0: o, 1: down)
  uint32_t ar_epoch;           // ... and the epoch its packets carry (never 0, grows with every all-reduce)
  const float* scale;          // e4m3 weights: fp32 scale per output row, applied to the fp32 sum (or null)
};

// Where the four 32-bit words of 16-byte chunk i of an activation row go: A-fragment
// order. Inside every 64-column block, word q (columns 8m+2q, 8m+2q+1) of chunk m sits
// at block*32 + q*8 + m, so that lane (row g, q) reads its eight words of a block with
// two 128-bit loads and nothing else is fetched.
__device__ __forceinline__ void store_row_chunk(uint32_t* row, int i, const uint4& v) {
  uint32_t* dst = row + (i >> 3) * 32 + (i & 7);
  dst[0] = v.x;
  dst[8] = v.y;
  dst[16] = v.z;
  dst[24] = v.w;
}

// e4m3 weight plans multiply with f16 tensor-pipe instructions (the weights convert to f16 pairs
// exactly, one instruction per pair), so the rows are staged as f16, and in the order that path's
// fragments want: a lane (row g, q) needs, of every 16-column block m of a 128-column atom, the four
// columns 16m + 4q .. + 3 (its e4m3 word of the weight tile covers exactly those), so inside an atom
// the two words of (q, m) sit at q*16 + m*2 and a lane reads its sixteen words with four 128-bit loads.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t w) {
  const __half2 h = __floats2half2_rn(bf_lo(w), bf_hi(w));
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void store_row_chunk_f16(uint32_t* row, int i, const uint4& v) {   // v: eight bf16 values, columns 8i..8i+7
  const int r = i & 15;
  uint32_t* dst = row + (i >> 4) * 64 + ((r & 1) * 2) * 16 + (r >> 1) * 2;
  dst[0] = bf16x2_to_f16x2(v.x);
  dst[1] = bf16x2_to_f16x2(v.y);
  dst[16] = bf16x2_to_f16x2(v.z);
  dst[17] = bf16x2_to_f16x2(v.w);
}

template <bool FP8>
__device__ __forceinline__ void store_row(uint32_t* row, int i, const uint4& v) {
  if (FP8) store_row_chunk_f16(row, i, v);
  else store_row_chunk(row, i, v);
}

// Stage the stage's B activation rows in shared memory; RMSNorm fused:
// y = bf16(w * bf16(x * rsqrt(mean(x^2) + eps)))  (python/tilemega/serving/export.py:24-27).
// Rows 0..B-1 of the staging area are the rows the GEMV reads; for a normalised
// stage the raw rows go to rows B..2B-1 and the norm weights to row 2B in the same
// pass, so that their L2 round trips overlap.
// Columns [k_src, k) do not exist in the source rows (the weights are zero-padded
// there): they are staged as zeros.
template <int B, bool FP8>
__device__ __forceinline__ void stage_rows(Ctx& c, const GemvIo& io, const GemvGeo& geo) {
  const MegaParams& p = c.p;
  const int k = geo.k, k_src = geo.k_src;
  const int chunks = k >> 3, src_chunks = k_src >> 3;
  const int pitch = chunks + 1;   // rows are k + 8 elements apart, so the batch rows of a block sit on distinct banks
  // A wide batch has no room to park the raw rows next to the normalised ones: the second
  // pass reads them from global memory again (an L2 hit) and only the norm weights are kept.
  constexpr bool kWide = B > 4;
  constexpr int kNormRow = kWide ? B : 2 * B;
  uint4* xs4 = reinterpret_cast<uint4*>(c.xs());
  const uint4* nw = reinterpret_cast<const uint4*>(io.norm);
  // The chunk loop is the outer one and the loads of all B rows of a chunk are issued
  // before any is used: one L2 round trip per chunk, not one per row.
  const uint4* src[B];
#pragma unroll
  for (int b = 0; b < B; ++b) {
    if (io.embed) {
      const int tok = min(max(c.tok()[b], 0), p.vocab - 1);
      src[b] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(io.src) + size_t(tok) * geo.src_stride);
    } else {
      src[b] = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(io.src) + size_t(b) * geo.src_stride + geo.src_off);
    }
  }
  float ss[B];
#pragma unroll
  for (int b = 0; b < B; ++b) ss[b] = 0.f;
  for (int i = c.tid; i < chunks; i += kConsumerThreads) {
    uint4 v[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      v[b] = make_uint4(0u, 0u, 0u, 0u);
      if (i < src_chunks) v[b] = io.embed ? __ldg(src[b] + i) : __ldcg(src[b] + i);
    }
    if (io.norm) xs4[kNormRow * pitch + i] = i < src_chunks ? __ldg(nw + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      if (io.embed && (b % p.grid) == c.cta && i < src_chunks)
        reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.x) + size_t(b) * k_src)[i] = v[b];
      if (io.norm) {
        if (!kWide) xs4[(B + b) * pitch + i] = v[b];
        float f[8];
        unpack8(v[b], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss[b] = fmaf(f[j], f[j], ss[b]);
      } else {
        store_row<FP8>(reinterpret_cast<uint32_t*>(xs4 + b * pitch), i, v[b]);
      }
    }
  }
  if (io.norm) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float v = ss[b];
#pragma unroll
      for (int m = 16; m; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
      if (c.lane == 0) c.wsum()[b * 8 + c.warp] = v;
    }
    consumer_sync();
    float inv[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) total += c.wsum()[b * 8 + w];
      inv[b] = 1.0f / sqrtf(total / float(k_src) + p.eps);
    }
    for (int i = c.tid; i < chunks; i += kConsumerThreads) {
      uint4 raw[B];
#pragma unroll
      for (int b = 0; b < B; ++b) {
        raw[b] = make_uint4(0u, 0u, 0u, 0u);
        if (!kWide) raw[b] = xs4[(B + b) * pitch + i];    // written by this same thread above
        else if (i < src_chunks) raw[b] = io.embed ? __ldg(src[b] + i) : __ldcg(src[b] + i);
      }
      float w[8];
      unpack8(xs4[kNormRow * pitch + i], w);
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float f[8];
        unpack8(raw[b], f);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t lo = bf16_bits(w[2 * j] * bf16_round(f[2 * j] * inv[b]));
          const uint32_t hi = bf16_bits(w[2 * j + 1] * bf16_round(f[2 * j + 1] * inv[b]));
          o[j] = lo | (hi << 16);
        }
        store_row<FP8>(reinterpret_cast<uint32_t*>(xs4 + b * pitch), i, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
  }
  consumer_sync();
}

// One page = 8 weight rows x 2048 columns, 128-byte swizzled in 8x64 atoms:
// element (r, col) sits at 1024*(col/64) + 128*r + 16*((col%64/8) ^ r) + 2*(col%8)
// bytes (python/tilemega/serving/weights.py:239-240 with tn = 8). Warp w owns
// columns [256w, 256w+256) of every page.
//
// A page on the tensor pipe: D[batch row][weight row] += X * W^T with
// mma.sync m16n8k16. The 8 weight rows of the page are the B operand's 8 columns
// (an 8x64 swizzle atom of the page IS four ldmatrix tiles), the batch rows are the A
// operand's rows 0..7 (rows past the batch alias row B-1 and their outputs are never
// read; rows 8..15 are zero). The pipe converts bf16 to fp32 itself, so a page costs
// a warp 16 ldmatrix + 16 mma instead of ~140 CUDA-core instructions, at any batch
// up to 8. Four accumulator sets keep the dependent chains short.
template <int B>
__device__ __forceinline__ void gemv_page_mma(const unsigned char* page, const unsigned char* xs, int k, int col0,
                                              int warp, int lane, float (&d)[4][4]) {
  const int r = lane & 7, m = lane >> 3;                 // ldmatrix: this lane addresses row r of matrix m
  const int g = lane >> 2, q = lane & 3;                 // mma fragments: batch row g, word q
  const unsigned char* xrow = xs + (size_t(min(g, B - 1)) * (k + 8) + col0 + 256 * warp) * 2 + 32 * q;
  const uint32_t wa = smem_u32(page) + uint32_t(1024 * (4 * warp) + 128 * r);
#pragma unroll
  for (int cb = 0; cb < 4; ++cb) {
    const uint4 xlo = *reinterpret_cast<const uint4*>(xrow + 128 * cb);        // words of chunks 0..3
    const uint4 xhi = *reinterpret_cast<const uint4*>(xrow + 128 * cb + 16);   // words of chunks 4..7
    uint32_t w[4];
    ldmatrix_x4(w, wa + 1024 * cb + 16 * (m ^ r));                             // chunks 0..3 of the 8 rows
    mma_bf16_m16n8k16(d[0], xlo.x, xlo.y, w[0], w[1]);
    mma_bf16_m16n8k16(d[1], xlo.z, xlo.w, w[2], w[3]);
    ldmatrix_x4(w, wa + 1024 * cb + 16 * ((4 + m) ^ r));                       // chunks 4..7
    mma_bf16_m16n8k16(d[2], xhi.x, xhi.y, w[0], w[1]);
    mma_bf16_m16n8k16(d[3], xhi.z, xhi.w, w[2], w[3]);
  }
}

// The same page loop for e4m3 weights: a page is 8 rows x 4096 one-byte columns laid out like a
// bf16 page of 8 x 2048 (2-byte units, the same swizzle), so ldmatrix delivers to lane (g, q), per
// 16-byte chunk, the four e4m3 values W[g][16m + 4q .. + 3] in one register. Two conversions make them
// two f16 pairs; with the activations staged in the matching order (store_row_chunk_f16) they are the
// B fragments of one m16n8k16 product whose sixteen k positions are a permutation of the block's
// sixteen columns, which a sum does not mind. Per page and warp: 8 ldmatrix.x4, 64 conversions, 32 mma.
__device__ __forceinline__ void e4m3x4_to_f16x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  asm("{\n"
      " .reg .b16 a, b;\n"
      " mov.b32 {a, b}, %2;\n"
      " cvt.rn.f16x2.e4m3x2 %0, a;\n"
      " cvt.rn.f16x2.e4m3x2 %1, b;\n"
      "}\n"
      : "=r"(lo), "=r"(hi)
      : "r"(w));
}

__device__ __forceinline__ void mma_f16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

template <int B>
__device__ __forceinline__ void gemv_page_mma_e4m3(const unsigned char* page, const unsigned char* xs, int k, int col0,
                                                   int warp, int lane, float (&d)[4][4]) {
  const int r = lane & 7, m = lane >> 3;                 // ldmatrix: this lane addresses row r of matrix m
  const int g = lane >> 2, q = lane & 3;                 // mma fragments: batch row g, word q
  // this warp's 512 columns of the page are four 128-column atoms; the lane's 16 words of an atom are contiguous
  const unsigned char* xrow = xs + (size_t(min(g, B - 1)) * (k + 8) + col0 + 512 * warp) * 2 + 64 * q;
  const uint32_t wa = smem_u32(page) + uint32_t(1024 * (4 * warp) + 128 * r);
#pragma unroll
  for (int cb = 0; cb < 4; ++cb) {
    uint4 x[4];   // x[j]: the words of blocks m = 2j, 2j+1: {a0, a2} of block 2j, {a0, a2} of block 2j+1
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = *reinterpret_cast<const uint4*>(xrow + 256 * cb + 16 * j);
    uint32_t w[4], lo, hi;
    ldmatrix_x4(w, wa + 1024 * cb + 16 * (m ^ r));                             // 16-byte chunks 0..3 of the 8 rows
    e4m3x4_to_f16x2(w[0], lo, hi); mma_f16_m16n8k16(d[0], x[0].x, x[0].y, lo, hi);
    e4m3x4_to_f16x2(w[1], lo, hi); mma_f16_m16n8k16(d[1], x[0].z, x[0].w, lo, hi);
    e4m3x4_to_f16x2(w[2], lo, hi); mma_f16_m16n8k16(d[2], x[1].x, x[1].y, lo, hi);
    e4m3x4_to_f16x2(w[3], lo, hi); mma_f16_m16n8k16(d[3], x[1].z, x[1].w, lo, hi);
    ldmatrix_x4(w, wa + 1024 * cb + 16 * ((4 + m) ^ r));                       // chunks 4..7
    e4m3x4_to_f16x2(w[0], lo, hi); mma_f16_m16n8k16(d[0], x[2].x, x[2].y, lo, hi);
    e4m3x4_to_f16x2(w[1], lo, hi); mma_f16_m16n8k16(d[1], x[2].z, x[2].w, lo, hi);
    e4m3x4_to_f16x2(w[2], lo, hi); mma_f16_m16n8k16(d[2], x[3].x, x[3].y, lo, hi);
    e4m3x4_to_f16x2(w[3], lo, hi); mma_f16_m16n8k16(d[3], x[3].z, x[3].w, lo, hi);
  }
}

__device__ __forceinline__ float silu_bf16(float g) {
  // silu on a bf16 value, result rounded to bf16
  // (include/tilemega/Backend/ServingEpilogue.h:49-57).
  return bf16_round(g / (1.0f + expf(-g)));
}

// Tensor-parallel all-reduce of one tile, in two halves that are run an epilogue apart
// (include/tilemega/Backend/Sm90DenseEpilogue.h:43-86 splits it the same way). Send: the
// lane that holds the column pair (row, row + 1) of batch row b stores this rank's packet
// {two bf16 sums, epoch} into every peer's receive region. Only the tensor-parallel
// instantiation of the kernel contains these.
__device__ __forceinline__ size_t tp_slot(const MegaParams& p, int ar_region, int batch, int n, int source, int b, int row) {
  const size_t half = size_t(n) >> 1;
  return (size_t(ar_region) * p.tp_world * batch + size_t(source) * batch + b) * half + (size_t(row) >> 1);
}

__device__ __forceinline__ void tp_send(const MegaParams& p, int ar_region, uint32_t epoch, int batch, int b, int n, int row,
                                        uint32_t mine) {
  const size_t slot = tp_slot(p, ar_region, batch, n, p.tp_rank, b, row);
  const unsigned long long packet = ((unsigned long long)epoch << 32) | mine;
  for (int q = 0; q < p.tp_world; ++q)
    if (q != p.tp_rank) st_relaxed_sys(p.ar[q] + slot, packet);
}

// Finish: poll this rank's own region for the peers' packets of the same column pair and
// add the partials in ascending rank order, so the sum is bitwise the same on every rank.
__device__ __forceinline__ float2 tp_finish(const MegaParams& p, int ar_region, uint32_t epoch, int batch, int b, int n,
                                            int row, uint32_t mine) {
  float sx = 0.f, sy = 0.f;
  for (int q = 0; q < p.tp_world; ++q) {
    uint32_t bits = mine;
    if (q != p.tp_rank) {
      const unsigned long long* slot = p.ar[p.tp_rank] + tp_slot(p, ar_region, batch, n, q, b, row);
      unsigned long long seen, t0 = 0;
      uint32_t polls = 0;
      while (uint32_t((seen = ld_relaxed_sys(slot)) >> 32) != epoch) {
        if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSitePeer, epoch, seen)) break;
      }
      bits = uint32_t(seen);
    }
    sx += bf_lo(bits);
    sy += bf_hi(bits);
  }
  return make_float2(sx, sy);
}

// The lm_head winners of the ranks: CTA 0 sends this rank's (value, global index) of
// batch row b to every peer as one packet {epoch 28 bits, bf16 value, 20-bit index};
// lanes 0..tp_world-1 of the calling warp each fetch one rank's candidate. Returns the
// candidate this lane holds (lanes past tp_world: none).
static __device__ __noinline__ void tp_exchange_argmax(const MegaParams& p, int cta, unsigned long long epoch, int b, int lane,
                                                float& value, int& index) {
  if (cta == 0 && lane < p.tp_world && lane != p.tp_rank) {
    const unsigned long long packet =
        (epoch << 36) | ((unsigned long long)bf16_bits(value) << 20) | (unsigned long long)(index & 0xfffff);
    st_relaxed_sys(p.xchg[lane] + size_t(p.tp_rank) * kMaxBatch + b, packet);
  }
  if (lane < p.tp_world && lane != p.tp_rank) {
    const unsigned long long* slot = p.xchg[p.tp_rank] + size_t(lane) * kMaxBatch + b;
    unsigned long long seen, t0 = 0;
    uint32_t polls = 0;
    while (((seen = ld_relaxed_sys(slot)) >> 36) != epoch) {
      if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSitePeer, epoch, seen)) break;
    }
    value = bf16_from_bits(uint16_t(seen >> 20));
    index = int(seen & 0xfffffull);
  } else if (lane >= p.tp_world) {
    value = -INFINITY;
    index = 0x7fffffff;
  }
}

// Everything the epilogue of one GEMV task needs, kept by the warp that owns it.
// Output (batch row b, weight row r) of a task is handled by lane (b*8 + r) % 32 in
// pass (b*8 + r) / 32: one pass up to batch 4, two up to batch 8.
template <int B>
struct EpiPasses { static constexpr int value = (kTileN * B + 31) / 32; };

template <int B>
struct PendingEpilogue {
  int task;         // -1: none
  int buf;
  uint32_t lap;
  float residual[EpiPasses<B>::value];   // prefetched residual elements of this lane (kEpiResidual)
};

// A tile whose all-reduce packets are sent but whose sum is not taken yet. The owning warp
// finishes it at its NEXT epilogue, eight of the CTA's tasks later (or at the end of the
// stage): by then the peers' packets have crossed NVLink, so the wait costs nothing. Taken
// right after the send, the round trip stalls the warp on every tile, and with the short
// tiles of an 8-way sharded model the whole CTA behind it.
template <int B>
struct PendingAr {
  int task;         // -1: none
  uint32_t mine[EpiPasses<B>::value];
  float res0[EpiPasses<B>::value], res1[EpiPasses<B>::value];
};

template <int B>
__device__ __forceinline__ void tp_finish_tile(Ctx& c, const GemvGeo& geo, const GemvIo& io, PendingAr<B>& ar, int lane) {
  const MegaParams& p = c.p;
#pragma unroll
  for (int pass = 0; pass < EpiPasses<B>::value; ++pass) {
    constexpr int total = kTileN * B;
    const int live = total - 32 * pass >= 32 ? 32 : total - 32 * pass;
    if (lane < live && (lane & 1) == 0) {
      const int r = lane & 7, b = 4 * pass + (lane >> 3);
      const int row = ar.task * kTileN + r;
      const float2 sum = tp_finish(p, io.ar_region, io.ar_epoch, B, b, geo.n, row, ar.mine[pass]);
      const uint32_t pair = pack_bf16x2(bf16_round(sum.x) + ar.res0[pass], bf16_round(sum.y) + ar.res1[pass]);
      *reinterpret_cast<uint32_t*>(static_cast<__nv_bfloat16*>(io.out) + size_t(b) * geo.n + row) = pair;
    }
  }
  ar.task = -1;
}

// Epilogue of one task, run by one warp: sum the eight warps' partial sums in warp
// order, then apply the stage's rounding sites.
template <int B, int X>
__device__ __forceinline__ void gemv_epilogue(Ctx& c, const GemvGeo& geo, const GemvIo& io, const PendingEpilogue<B>& e,
                                              int lane, float (&best_val)[EpiPasses<B>::value],
                                              int (&best_idx)[EpiPasses<B>::value], PendingAr<B>& ar) {
  const MegaParams& p = c.p;
  const float* red = c.red();
  if ((X & kXTp) && io.epilogue == kEpiResidualAllReduce && ar.task >= 0) tp_finish_tile<B>(c, geo, io, ar, lane);
  mbar_wait_warp(c, c.pfull(e.buf), e.lap, kSiteFull);
#pragma unroll
  for (int pass = 0; pass < EpiPasses<B>::value; ++pass) {
    constexpr int total = kTileN * B;
    const int live = total - 32 * pass >= 32 ? 32 : total - 32 * pass;   // lanes taking part in this pass
    if (lane < live) {
      const unsigned mask = live >= 32 ? 0xffffffffu : ((1u << live) - 1u);   // exactly those lanes
      const int rt = e.task;
      const int r = lane & 7, b = 4 * pass + (lane >> 3);
      const int row = rt * kTileN + r;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) v += red[((e.buf * 8 + w) * 8 + r) * B + b];
      if (io.partial_in) v += __ldcg(io.partial_in + size_t(b) * geo.n + row);   // earlier parts of a split reduction
      if ((X & kXFp8) && io.scale && io.epilogue != kEpiPartial) v *= __ldg(io.scale + row);   // e4m3 weights: the row's scale
      const float vb = bf16_round(v);
      if (io.epilogue == kEpiPartial) {
        static_cast<float*>(io.out)[size_t(b) * geo.n + row] = v;
      } else if (io.epilogue == kEpiSwiGLU) {
        // rows 0..3 of the page are gate rows, rows 4..7 the matching up rows
        const float up = __shfl_down_sync(mask, vb, 4);
        if (r < 4) {
          __nv_bfloat16* h = static_cast<__nv_bfloat16*>(io.out);
          h[size_t(b) * (geo.n >> 1) + rt * 4 + r] = __float2bfloat16_rn(silu_bf16(vb) * up);
        }
      } else if (io.epilogue == kEpiHead) {
        // the logits buffer keeps the fp32 accumulator; the argmax below compares the
        // bf16-rounded value, as the reference's head epilogue does
        if (p.write_logits) static_cast<float*>(io.out)[size_t(b) * geo.n + row] = v;
        // ties -> smaller index (include/tilemega/Backend/Sm90DenseEpilogue.h:166-184)
        float bv = vb;
        int bi = p.head_base + row;   // this rank's head rows are a slice of the vocabulary
#pragma unroll
        for (int m = 1; m < 8; m <<= 1) {
          const float ov = __shfl_xor_sync(mask, bv, m);
          const int oi = __shfl_xor_sync(mask, bi, m);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bv > best_val[pass] || (bv == best_val[pass] && bi < best_idx[pass])) {
          best_val[pass] = bv;   // the 8 lanes of a sequence all hold its candidate
          best_idx[pass] = bi;
        }
      } else if ((X & kXTp) && io.epilogue == kEpiResidualAllReduce) {
        // Tensor parallel: every rank holds the sum over its own slice of the reduction.
        // The ranks exchange their sums rounded to bf16, two columns and the epoch per
        // 8-byte packet, stored straight into each peer's receive region; every rank
        // adds them in ascending rank order (bitwise the same x on all ranks), rounds,
        // and adds the residual (include/tilemega/Backend/Sm90DenseEpilogue.h:43-86).
        const float vb1 = __shfl_down_sync(mask, vb, 1);
        const float res1 = __shfl_down_sync(mask, e.residual[pass], 1);
        if ((r & 1) == 0) {
          ar.mine[pass] = pack_bf16x2(vb, vb1);
          ar.res0[pass] = e.residual[pass];
          ar.res1[pass] = res1;
          tp_send(p, io.ar_region, io.ar_epoch, B, b, geo.n, row, ar.mine[pass]);
        }
        ar.task = e.task;   // finished at this warp's next epilogue, or when the stage ends
      } else {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(io.out) + size_t(b) * geo.n + row;
        if (io.epilogue == kEpiResidual) {
          // bf16(float(bf16(acc)) + float(residual)) (ServingEpilogue.h:38-43)
          *out = __float2bfloat16_rn(vb + e.residual[pass]);
        } else {
          *out = __float2bfloat16_rn(v);
        }
      }
    }
  }
  if (io.ready) {
    // one more row tile of this KV-head group is in global memory: attention tasks
    // of that group wait for the group's count instead of a grid-wide barrier
    __syncwarp();
    if (lane == 0) red_release_add(io.ready + e.task / io.tiles_per_group, 1ull);   // (the release is cumulative over the warp's stores)
  }
}

template <int B, int X>
__device__ __forceinline__ void gemv_stage(Ctx& c, const GemvGeo& geo, const GemvIo& io, bool tr, int stage) {
  const MegaParams& p = c.p;
  stage_rows<B, (X & kXFp8) != 0>(c, io, geo);
  trace_mark(c, tr, stage, 2);
  // per-warp running argmax (each warp runs every eighth epilogue); merged by the caller
  float best_val[EpiPasses<B>::value];
  int best_idx[EpiPasses<B>::value];
#pragma unroll
  for (int i = 0; i < EpiPasses<B>::value; ++i) {
    best_val[i] = -INFINITY;
    best_idx[i] = 0x7fffffff;
  }
  float* red = c.red();
  uint32_t slot = c.slot, phase = c.phase, task_seq = c.task_seq, gemv_seq = c.gemv_seq;
  const int warp = c.warp, lane = c.lane;
  const uint32_t nslots = uint32_t(p.nslots);
  unsigned char* const ring0 = c.ring(0);
  const unsigned char* const xs = c.xs();
  uint64_t* const full0 = c.full(0);
  uint64_t* const empty0 = c.empty(0);
  // Warp (n mod 8) owns the epilogue of this CTA's n-th task and runs it one task
  // late, after its own pages of task n+1: by then the other warps' partial sums
  // have long arrived, so no warp ever waits for another one here, and the cost of
  // an epilogue is spread as one eighth per task instead of stalling every task.
  PendingEpilogue<B> pending;
  pending.task = -1;
  PendingAr<B> ar;
  ar.task = -1;
  for (int t = fifo_pop(c); t >= 0; t = fifo_pop(c)) {
    const int rt = t;
    float d[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) d[0][i] = d[1][i] = d[2][i] = d[3][i] = 0.f;
    const bool owner = warp == int(task_seq & 7);
    // the owner fetches the residual now, so the L2 round trip overlaps the arithmetic
    float residual[EpiPasses<B>::value];
#pragma unroll
    for (int pass = 0; pass < EpiPasses<B>::value; ++pass) {
      residual[pass] = 0.f;
      if ((io.epilogue == kEpiResidual || io.epilogue == kEpiResidualAllReduce) && owner && 32 * pass + lane < kTileN * B)
        residual[pass] = bf16_from_bits(__ldcg(reinterpret_cast<const unsigned short*>(io.out) +
                                               size_t(4 * pass + (lane >> 3)) * geo.n + rt * kTileN + (lane & 7)));
    }
    for (int pg = 0; pg < geo.pages_per_task; ++pg) {
      mbar_wait_warp(c, full0 + slot, phase, kSiteFull);
      // a warp whose 256 columns of this page lie wholly in the reduction's zero pad
      // has nothing to add (and that part of the slot was not copied)
      if (pg * geo.tile_k + (geo.tile_k >> 3) * warp < geo.k_src) {
        if constexpr ((X & kXFp8) != 0) gemv_page_mma_e4m3<B>(ring0 + slot * kSlotBytes, xs, geo.k, pg * geo.tile_k, warp, lane, d);
        else gemv_page_mma<B>(ring0 + slot * kSlotBytes, xs, geo.k, pg * geo.tile_k, warp, lane, d);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + slot);
      if (++slot == nslots) { slot = 0; phase ^= 1u; }
    }
    // lanes -> warps in a fixed order, so results are run-to-run identical. The warps
    // hand their partial sums over through a small ring of buffers guarded by mbarriers.
    const int buf = gemv_seq & (kPartialRing - 1);
    const uint32_t lap = (gemv_seq / kPartialRing) & 1u;
    // No wait before reusing buffer `buf`: its previous task lies kPartialRing tasks
    // back, and no warp can be more than the data ring (at most kMaxSlots pages, so
    // at most kMaxSlots tasks) ahead of the owner that reads it one task late.
    // lane holds D[batch row lane/4][weight rows 2*(lane%4), +1]
    if ((lane >> 2) < B) {
      float* dst = red + ((buf * 8 + warp) * 8 + 2 * (lane & 3)) * B + (lane >> 2);
      dst[0] = (d[0][0] + d[1][0]) + (d[2][0] + d[3][0]);
      dst[B] = (d[0][1] + d[1][1]) + (d[2][1] + d[3][1]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(c.pfull(buf));
    if (pending.task >= 0) {
      gemv_epilogue<B, X>(c, geo, io, pending, lane, best_val, best_idx, ar);
      pending.task = -1;
    }
    if (owner) {
      pending.task = t;
      pending.buf = buf;
      pending.lap = lap;
#pragma unroll
      for (int pass = 0; pass < EpiPasses<B>::value; ++pass) pending.residual[pass] = residual[pass];
    }
    ++task_seq;
    ++gemv_seq;
  }
  if (pending.task >= 0) gemv_epilogue<B, X>(c, geo, io, pending, lane, best_val, best_idx, ar);
  if ((X & kXTp) && ar.task >= 0) tp_finish_tile<B>(c, geo, io, ar, lane);
  c.slot = slot;
  c.phase = phase;
  c.task_seq = task_seq;
  c.gemv_seq = gemv_seq;
  if (io.epilogue == kEpiHead && (lane & 7) == 0) {
#pragma unroll
    for (int pass = 0; pass < EpiPasses<B>::value; ++pass) {
      const int b = 4 * pass + (lane >> 3);
      if (b < B) {
        c.best_val()[warp * kMaxBatch + b] = best_val[pass];
        c.best_idx()[warp * kMaxBatch + b] = best_idx[pass];
      }
    }
  }
  trace_mark(c, tr, stage, 3);
}

// ---------------------------------------------------------------------------
// arithmetic warps: mixture of experts (one token at a time)
// ---------------------------------------------------------------------------
// Top-k routing of token b, by warp 0: softmax in fp32 over the router's bf16
// logits, the k largest probabilities in descending order (ties to the smaller expert
// index), renormalised to sum 1 in fp32 (python/tilemega/moe/export.py:79-87). The result
// goes to shared memory for both the arithmetic warps and the streaming thread, and from
// CTA 0 to global memory for the host.
static __device__ __noinline__ void route_token(Ctx& c, int layer, int b) {
  const MegaParams& p = c.p;
  // probabilities of all experts in shared memory (the activation-row area is free between
  // stages), then every expert's rank by counting: rank = how many experts beat it (larger
  // probability, or equal and smaller index). The k experts of rank < k are the top-k in
  // descending order. One thread per expert does the counting: a single warp doing k
  // sequential arg-max rounds, or all the counting, issues too slowly next to nothing.
  float* prob = reinterpret_cast<float*>(c.xs());
  if (c.warp == 0) {
    constexpr int kPerLane = 8;   // experts <= 256
    const unsigned short* logits = reinterpret_cast<const unsigned short*>(p.router_logits) + size_t(b) * p.experts;
    float v[kPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = c.lane + 32 * j;
      v[j] = e < p.experts ? bf16_from_bits(__ldcg(logits + e)) : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      v[j] = c.lane + 32 * j < p.experts ? expf(v[j] - mx) : 0.f;
      sum += v[j];
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
#pragma unroll
    for (int j = 0; j < kPerLane; ++j)
      if (c.lane + 32 * j < p.experts) prob[c.lane + 32 * j] = v[j] / sum;
  }
  consumer_sync();
  if (c.tid < p.experts) {
    const float mine = prob[c.tid];
    int rank = 0;
#pragma unroll 8
    for (int o = 0; o < p.experts; ++o) {
      const float other = prob[o];   // every thread reads the same word: a broadcast
      rank += (other > mine || (other == mine && o < c.tid)) ? 1 : 0;
    }
    if (rank < p.topk) {
      c.route_e()[rank] = c.tid;
      c.route_w()[rank] = mine;
    }
  }
  consumer_sync();
  if (c.tid < kMaxTopK) {
    float total = 0.f;   // sum of the chosen probabilities, in rank order
    for (int s = 0; s < p.topk; ++s) total += c.route_w()[s];
    const int s = c.tid;
    const float w = s < p.topk ? c.route_w()[s] / total : 0.f;
    const int e = s < p.topk ? c.route_e()[s] : 0;
    __syncwarp(0xffu);   // every lane has read all weights before any is overwritten
    c.route_w()[s] = w;
    c.route_e()[s] = e;
    if (c.cta == 0 && s < p.topk) {   // [layer][token][rank]
      p.route_idx[(layer * p.batch + b) * p.topk + s] = e;
      p.route_w[(layer * p.batch + b) * p.topk + s] = w;
    }
  }
  consumer_sync();
  if (c.tid == 0) mbar_arrive(c.route_bar());   // the streaming thread may start on the experts
}

// The chosen experts' down projections and their weighted sum for ONE token (row b of the batch). Sub-task
// (row tile, expert slot s) is one page; the activation row of slot s is that expert's
// SwiGLU output. The warp that owns a row tile runs the epilogues of its topk sub-tasks
// in slot order and keeps the running sum:
//   y = bf16( sum_s fp32( bf16(W_s h_s) * w_s ) ), x += y
// (python/tilemega/moe/export.py:29-37: expert outputs in the model dtype, times the fp32
// routing weight, summed over the ranks in fp32, one rounding; then the layer's residual add).
static __device__ __noinline__ void moe_down_stage(Ctx& c, const GemvGeo& geo, bool tr, int stage, int b) {
  const MegaParams& p = c.p;
  unsigned short* const xrow = reinterpret_cast<unsigned short*>(p.x) + size_t(b) * p.hidden;   // token b's residual stream
  const int topk = p.topk;
  const int pitch_bytes = (geo.k + 8) * 2;
  {
    // rows: h[slot][k_src] -> shared memory in A-fragment order, pad columns zero
    const int chunks = geo.k >> 3, src_chunks = geo.k_src >> 3;
    for (int i = c.tid; i < chunks; i += kConsumerThreads) {
      uint4 v[kMaxTopK];   // all rows' loads in flight together: one L2 round trip, not one per row
#pragma unroll
      for (int slot = 0; slot < kMaxTopK; ++slot) {
        v[slot] = make_uint4(0u, 0u, 0u, 0u);
        if (slot < topk && i < src_chunks)
          v[slot] = __ldcg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.h) + size_t(slot) * geo.k_src) + i);
      }
#pragma unroll
      for (int slot = 0; slot < kMaxTopK; ++slot)
        if (slot < topk) store_row_chunk(reinterpret_cast<uint32_t*>(c.xs() + size_t(slot) * pitch_bytes), i, v[slot]);
    }
    consumer_sync();
  }
  trace_mark(c, tr, stage, 2);
  float* red = c.red();
  uint32_t slot = c.slot, phase = c.phase, gemv_seq = c.gemv_seq;
  const int warp = c.warp, lane = c.lane;
  const uint32_t nslots = uint32_t(p.nslots);
  unsigned char* const ring0 = c.ring(0);
  uint64_t* const full0 = c.full(0);
  uint64_t* const empty0 = c.empty(0);
  uint32_t sub_seq = 0;        // sub-tasks seen by this CTA in this stage
  uint32_t tile_seq = 0;       // row tiles completed: the owner warp rotates per tile
  int pending_task = -1, pending_buf = 0;
  uint32_t pending_lap = 0;
  float running = 0.f, residual = 0.f;
  auto epilogue = [&]() {
    mbar_wait_warp(c, c.pfull(pending_buf), pending_lap, kSiteFull);
    const int tile = pending_task / kMaxTopK, s = pending_task % kMaxTopK;
    if (lane < kTileN) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) v += red[(pending_buf * 8 + w) * 8 + lane];
      running = __fadd_rn(running, __fmul_rn(bf16_round(v), c.route_w()[s]));
      if (s == topk - 1) {
        xrow[tile * kTileN + lane] = bf16_bits(bf16_round(running) + residual);
        running = 0.f;
      }
    }
    pending_task = -1;
  };
  for (int t = fifo_pop(c); t >= 0; t = fifo_pop(c)) {
    const int tile = t / kMaxTopK, s = t % kMaxTopK;   // powers of two: no division in the loop
    const bool owner = warp == int(tile_seq & 7u);
    if (owner && s == 0 && lane < kTileN)
      residual = bf16_from_bits(__ldcg(xrow + tile * kTileN + lane));
    float d[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) d[0][i] = d[1][i] = d[2][i] = d[3][i] = 0.f;
    mbar_wait_warp(c, full0 + slot, phase, kSiteFull);
    if (256 * warp < geo.k_src)
      gemv_page_mma<1>(ring0 + slot * kSlotBytes, c.xs() + size_t(s) * pitch_bytes, geo.k, 0, warp, lane, d);
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + slot);
    if (++slot == nslots) { slot = 0; phase ^= 1u; }
    const int buf = gemv_seq & (kPartialRing - 1);
    const uint32_t lap = (gemv_seq / kPartialRing) & 1u;
    if ((lane >> 2) < 1) {   // lane q of row 0 holds weight rows 2q, 2q+1
      float* dst = red + (buf * 8 + warp) * 8 + 2 * (lane & 3);
      dst[0] = (d[0][0] + d[1][0]) + (d[2][0] + d[3][0]);
      dst[1] = (d[0][1] + d[1][1]) + (d[2][1] + d[3][1]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(c.pfull(buf));
    if (pending_task >= 0) epilogue();
    if (owner) {
      pending_task = t;
      pending_buf = buf;
      pending_lap = lap;
    }
    ++sub_seq;
    if (s == topk - 1) ++tile_seq;
    ++gemv_seq;
  }
  if (pending_task >= 0) epilogue();
  c.slot = slot;
  c.phase = phase;
  c.gemv_seq = gemv_seq;
  c.task_seq += sub_seq;
  trace_mark(c, tr, stage, 3);
}

// ---------------------------------------------------------------------------
// arithmetic warps: RoPE + KV append + split-KV decode attention
//
// KV rows are stored (in either cache layout) with their 16-byte chunks XOR-ed by
// (row position mod 8): chunk c of the row at position t sits at chunk c ^ (t & 7).
// The format is private to the plan (the reference's driver only zero-fills the
// cache). It makes the 8 rows of an ldmatrix tile land on distinct banks although a
// ring slot is filled by plain contiguous bulk copies.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int kv_swizzled(int d, int pos) { return ((((d >> 3) ^ (pos & 7))) << 3) | (d & 7); }

template <int B, int D, int GQ, int X>
__device__ void attn_stage(Ctx& c, const LayerPtrs& lp, int past, bool tr, int stage, unsigned long long qkv_stages) {
  constexpr int NK = kAttnHalfBytes / (2 * D);  // keys per slot: 64 (D=128) / 128 (D=64)
  constexpr int KW = NK / kConsumerWarps;       // keys per warp per slot: 8 / 16
  constexpr int KT = KW / 8;                    // 8-key tiles per warp per slot
  constexpr int DT = D / 8;                     // 8-column tiles of the head dimension
  constexpr int PW = D + 2;                     // floats per (chunk, head) partial: acc, m, l
  static_assert(GQ <= 8 && KW % 8 == 0, "attention slot geometry");
  const MegaParams& p = c.p;
  const int g = c.lane >> 2, q = c.lane & 3;    // mma fragments: row (query head) g, column pair q
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(c.xs());          // [GQ][D] roped q (bf16, unscaled)
  __nv_bfloat16* knew = qs + GQ * D;                                     // [D] roped new key
  __nv_bfloat16* vnew = knew + D;                                        // [D] new value
  float* scratch = reinterpret_cast<float*>(vnew + D);                   // [8 warps][GQ][PW]
  __nv_bfloat16* qkn = reinterpret_cast<__nv_bfloat16*>(scratch + kConsumerWarps * GQ * PW);   // [GQ + 1][D] normalised q, k (QK norm)
  const int qkv_width = (p.heads + 2 * p.kv_heads) * D;
  const __nv_bfloat16* cosb = static_cast<const __nv_bfloat16*>(p.rope_cos);
  const __nv_bfloat16* sinb = static_cast<const __nv_bfloat16*>(p.rope_sin);

  const Rows rw = load_rows(p, past);
  const AttnShape sh = attn_shape(p, rw, NK);
#if TMB_DENSE
  // Dense-batch plans leave a QKV reduction that ran in parts unsummed: the tasks here add the
  // parts' fp32 tiles (ascending, then one rounding to bf16 -- what a summing epilogue would have
  // stored) for the (GQ + 2) * D values of their own (sequence, KV head) while they stage them.
  const int qkv_parts = p.dense ? p.dgeo[kQkv].nsplit : 1;
  unsigned short* qraw = reinterpret_cast<unsigned short*>(qkn + (GQ + 1) * D);   // [GQ + 2][D] summed q, k, v
#else
  constexpr int qkv_parts = 1;
  unsigned short* qraw = nullptr;
#endif
  const bool summed_here = qkv_parts > 1;
  // chunk_rows plans appended every row's key and value in a stage of their own (other rows of the batch
  // may be later positions of the same sequence and read them): nothing is written to the pools here
  const bool appended = p.chunk_rows != 0;
  trace_mark(c, tr, stage, 2);
  for (int t = fifo_pop_uniform(c); t >= 0; t = fifo_pop_uniform(c)) {
    AttnWalk walk = attn_walk(p, rw, NK, sh, min(t, sh.ntasks - 1));
    AttnTask a;
    while (attn_next(p, rw, NK, sh, walk, a)) {
    const bool tail = a.slot1 == a.ns;   // this chunk holds the new token
    // the (GQ + 2) * D QKV rows of KV head a.g must be stored: their row tiles are counted per group
    if (c.tid == 0 && !c.dead) {
      // (dense-batch plans whose QKV reduction runs in parts count every part's tile)
      const unsigned long long need = qkv_stages * (unsigned long long)((GQ + 2) * D / kTileN) * (unsigned long long)qkv_parts;
      unsigned long long t0 = 0, seen;
      uint32_t polls = 0;
      while ((seen = ld_acquire(p.qkv_ready + a.g)) < need) {
        if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSiteGrid, need, seen)) break;
      }
    }
    consumer_sync();
    // ---- q (GQ heads) and the new k: RoPE with bf16 tables, each product and the
    // sum rounded to bf16 (include/tilemega/Codegen/tasks/FusedAttentionTaskBody.h:141-151)
    const unsigned short* row = reinterpret_cast<const unsigned short*>(p.qkv) + size_t(a.b) * qkv_width +
                                size_t(a.g) * (GQ + 2) * D;
#if TMB_DENSE
    if (summed_here) {
      const size_t tile_floats = size_t(kDenseTileN) * p.batch;
      const int count = tail ? (GQ + 2) * D : GQ * D;   // the key and value rows matter to the chunk with the new token only
      for (int e = c.tid; e < count; e += kConsumerThreads) {
        const int n = a.g * (GQ + 2) * D + e;          // feature index of the QKV output
        const float* src = p.gemm_part + (size_t(n >> 7) * qkv_parts * p.batch + a.b) * kDenseTileN + (n & 127);
        float v = 0.f;
#pragma unroll 4
        for (int part = 0; part < qkv_parts; ++part) v += __ldcg(src + size_t(part) * tile_floats);
        const unsigned short bits = bf16_bits(v);
        qraw[e] = bits;
        if (tail) const_cast<unsigned short*>(row)[e] = bits;   // the plan's qkv buffer holds the rows as before
      }
      consumer_sync();
    }
#endif
    auto qkv_value = [&](int idx) -> unsigned short { return summed_here ? qraw[idx] : __ldcg(row + idx); };
    long long new_off = 0;
    if (tail) {
      const long long e = table_entry(p, a.sq, a.pos / kKvBlock);
      new_off = e * p.kv_block_stride + (long long)a.g * p.kv_head_stride + (a.pos % kKvBlock) * D;
    }
    const bool qk_norm = (X & kXMoe) && lp.q_norm != nullptr;   // only the mixture-of-experts / Qwen3 instantiation carries this
    if (qk_norm) {
      // Qwen3: every query head and the key head are RMS-normalised over their own D
      // values before RoPE, y = w * bf16(x * rsqrt(mean x^2 + eps)), the product rounded
      // to bf16 (python/tilemega/serving/export.py:63-65,82-84). One warp per head.
      // (a warp with two heads -- GQ + 1 = 9 heads on 8 warps -- fetches both before it uses either:
      // one L2 round trip, not two)
      constexpr int kHeadsPerWarp = (GQ + 1 + kConsumerWarps - 1) / kConsumerWarps;
      float xv[kHeadsPerWarp][D / 32], wv[kHeadsPerWarp][D / 32];
#pragma unroll
      for (int i = 0; i < kHeadsPerWarp; ++i) {
        const int hh = c.warp + i * kConsumerWarps;
        const unsigned short* wn = reinterpret_cast<const unsigned short*>(hh < GQ ? lp.q_norm : lp.k_norm);
#pragma unroll
        for (int j = 0; j < D / 32; ++j) {
          xv[i][j] = hh < GQ + 1 ? bf16_from_bits(__ldcg(row + hh * D + c.lane + 32 * j)) : 0.f;
          wv[i][j] = hh < GQ + 1 ? bf16_from_bits(__ldg(wn + c.lane + 32 * j)) : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < kHeadsPerWarp; ++i) {
        const int hh = c.warp + i * kConsumerWarps;
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < D / 32; ++j) ss = fmaf(xv[i][j], xv[i][j], ss);
#pragma unroll
        for (int m = 16; m; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        const float inv = 1.0f / sqrtf(ss / float(D) + p.eps);
        if (hh < GQ + 1) {
#pragma unroll
          for (int j = 0; j < D / 32; ++j) qkn[hh * D + c.lane + 32 * j] = __float2bfloat16_rn(wv[i][j] * bf16_round(xv[i][j] * inv));
        }
      }
      consumer_sync();
    }
    {
      // every element's four inputs (the value, its rotation partner, cos, sin) are fetched
      // for all of this thread's elements before any is used: one L2 round trip for the
      // whole staging instead of one per element
      constexpr int kElements = (GQ + 2) * D;
      constexpr int NI = (kElements + kConsumerThreads - 1) / kConsumerThreads;
      const unsigned short* cosr = reinterpret_cast<const unsigned short*>(cosb) + size_t(a.pos) * D;
      const unsigned short* sinr = reinterpret_cast<const unsigned short*>(sinb) + size_t(a.pos) * D;
      unsigned short rv[NI], rp[NI], rc[NI], rs[NI];
#pragma unroll
      for (int it = 0; it < NI; ++it) {
        const int e = c.tid + it * kConsumerThreads;
        rv[it] = rp[it] = rc[it] = rs[it] = 0;
        if (e < kElements) {
          const int hh = e / D, d = e - hh * D;
          const int d2 = d < D / 2 ? d + D / 2 : d - D / 2;
          const bool normed = qk_norm && hh <= GQ;
          const bool roped = hh < GQ || (hh == GQ && tail);
          if (!normed && (roped || (hh == GQ + 1 && tail))) rv[it] = qkv_value(e);
          if (roped) {
            if (!normed) rp[it] = qkv_value(hh * D + d2);
            rc[it] = __ldg(cosr + d);
            rs[it] = __ldg(sinr + d);
          }
        }
      }
#pragma unroll
      for (int it = 0; it < NI; ++it) {
        const int e = c.tid + it * kConsumerThreads;
        if (e >= kElements) continue;
        const int hh = e / D, d = e - hh * D;
        const bool normed = qk_norm && hh <= GQ;
        const float xv = normed ? __bfloat162float(qkn[e]) : bf16_from_bits(rv[it]);
        if (hh == GQ + 1) {
          if (tail) {
            vnew[d] = __float2bfloat16_rn(xv);
            if (!appended) static_cast<__nv_bfloat16*>(lp.v_pool)[new_off + kv_swizzled(d, a.pos)] = __float2bfloat16_rn(xv);
          }
          continue;
        }
        if (hh == GQ && !tail) continue;
        const int d2 = d < D / 2 ? d + D / 2 : d - D / 2;
        const float xp = normed ? __bfloat162float(qkn[hh * D + d2]) : bf16_from_bits(rp[it]);
        const float cs = bf16_from_bits(rc[it]);
        const float sn = bf16_from_bits(rs[it]);
        const float rot = d < D / 2 ? -xp : xp;
        const float o = bf16_round(bf16_round(xv * cs) + bf16_round(rot * sn));
        if (hh < GQ) {
          qs[hh * D + d] = __float2bfloat16_rn(o);
        } else {
          knew[d] = __float2bfloat16_rn(o);
          if (!appended) static_cast<__nv_bfloat16*>(lp.k_pool)[new_off + kv_swizzled(d, a.pos)] = __float2bfloat16_rn(o);
        }
      }
    }
    if (tail) fence_proxy_async();
    consumer_sync();
    // A fragments of Q for S = Q K^T (m16n8k16): rows 0..GQ-1 are the query heads, the
    // other rows repeat a head and are never read. qa[s][0/1] = Q[g][16s + 2q (+8), +1].
    uint32_t qa[D / 16][2];
    {
      const uint32_t* qrow = reinterpret_cast<const uint32_t*>(qs + min(g, GQ - 1) * D);
#pragma unroll
      for (int s = 0; s < D / 16; ++s) {
        qa[s][0] = qrow[8 * s + q];
        qa[s][1] = qrow[8 * s + 4 + q];
      }
    }
    // online softmax state of this lane's row (query head g) over this warp's keys. The
    // output is kept TRANSPOSED, O^T = V^T P^T, so that all 16 rows of the tensor-pipe tile
    // carry head-dimension rows (with O = P V half of every tile would be the unused query
    // rows 8..15): oacc[mt] = O[heads 2q, 2q+1][d = 16 mt + g] and the same for d + 8.
    float m = -INFINITY, l = 0.f;
    float oacc[D / 16][4];
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) oacc[mt][0] = oacc[mt][1] = oacc[mt][2] = oacc[mt][3] = 0.f;
    for (int s = a.slot0; s < a.slot1; ++s) {
      mbar_wait_warp(c, c.full(c.slot), c.phase, kSiteFull);
      unsigned char* kbase = c.ring(c.slot);
      unsigned char* vbase = kbase + kAttnHalfBytes;
      const int nkeys = min(NK, a.pos + 1 - s * NK);
      if (tail && s == a.ns - 1) {
        // the cache row of the new token is being written this step: take it from this
        // CTA's own copy; and rows past the context may hold anything (stale ring bytes
        // where no block was copied): zero them in V, where a 0 * NaN would poison P*V
        const int r = a.pos - s * NK;
        if (c.tid < D / 8) {
          reinterpret_cast<uint4*>(kbase + size_t(r) * D * 2)[c.tid ^ (r & 7)] = reinterpret_cast<const uint4*>(knew)[c.tid];
        } else if (c.tid < D / 4) {
          reinterpret_cast<uint4*>(vbase + size_t(r) * D * 2)[(c.tid - D / 8) ^ (r & 7)] =
              reinterpret_cast<const uint4*>(vnew)[c.tid - D / 8];
        }
        for (int i = nkeys * (D / 8) + c.tid; i < NK * (D / 8); i += kConsumerThreads)
          reinterpret_cast<uint4*>(vbase)[i] = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async();   // generic writes into a slot the bulk engine refills later
        consumer_sync();
      }
      const int key0 = c.warp * KW;
      if (key0 < nkeys) {   // warp-uniform
        // ---- S = Q K^T for this warp's keys: sc[kt][0..1] = S[g][key0 + 8 kt + 2q, +1]
        float sc[KT][4];
        const int lr = c.lane & 7, lm = c.lane >> 3;   // ldmatrix: row lr of tile lm
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          sc[kt][0] = sc[kt][1] = sc[kt][2] = sc[kt][3] = 0.f;
          const uint32_t krow = smem_u32(kbase) + uint32_t((key0 + 8 * kt + lr) * D * 2);
#pragma unroll
          for (int cq = 0; cq < D / 32; ++cq) {     // four 16-byte chunks = two k-steps of 16 columns
            uint32_t kb[4];
            ldmatrix_x4(kb, krow + 16 * ((4 * cq + lm) ^ lr));
            mma_bf16_m16n8k16(sc[kt], qa[2 * cq][0], qa[2 * cq][1], kb[0], kb[1]);
            mma_bf16_m16n8k16(sc[kt], qa[2 * cq + 1][0], qa[2 * cq + 1][1], kb[2], kb[3]);
          }
        }
        // ---- online softmax in base 2 (scale log2(e)/sqrt(D)); keys past the context are masked
        float mx = m;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          const int k = key0 + 8 * kt + 2 * q;
          sc[kt][0] = k < nkeys ? sc[kt][0] * p.qk_scale_log2 : -INFINITY;
          sc[kt][1] = k + 1 < nkeys ? sc[kt][1] * p.qk_scale_log2 : -INFINITY;
          mx = fmaxf(mx, fmaxf(sc[kt][0], sc[kt][1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));   // key0 < nkeys: at least one finite score in the row
        const float alpha = ex2(m - mx);
        m = mx;
        float sum = 0.f;
        uint32_t phi[KT], plo[KT];
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          const float p0 = ex2(sc[kt][0] - mx), p1 = ex2(sc[kt][1] - mx);
          sum += p0 + p1;
          // P as a bf16 head plus a bf16 remainder: two tensor-pipe products keep ~16
          // mantissa bits of the probabilities instead of 8
          phi[kt] = pack_bf16x2(p0, p1);
          plo[kt] = pack_bf16x2(p0 - bf_lo(phi[kt]), p1 - bf_hi(phi[kt]));
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l = fmaf(l, alpha, sum);
        {
          // the rescale factors of the two heads this lane's output columns belong to
          const float alpha0 = __shfl_sync(0xffffffffu, alpha, 8 * q);
          const float alpha1 = __shfl_sync(0xffffffffu, alpha, 8 * q + 4);
#pragma unroll
          for (int mt = 0; mt < D / 16; ++mt) {
            oacc[mt][0] *= alpha0;
            oacc[mt][1] *= alpha1;
            oacc[mt][2] *= alpha0;
            oacc[mt][3] *= alpha1;
          }
        }
        // ---- O^T += V^T P^T: A = V^T by transposing loads of row-major V[key][d] (rows d,
        // columns keys), B = P^T, which is the score fragment as it stands
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
          const uint32_t vrow = smem_u32(vbase) + uint32_t((key0 + 8 * kt + lr) * D * 2);
#pragma unroll
          for (int cq = 0; cq < DT / 4; ++cq) {
            uint32_t vb[4];   // vb[j] = V[keys 2q, 2q+1][d = 8 (4 cq + j) + g]
            ldmatrix_x4_trans(vb, vrow + 16 * ((4 * cq + lm) ^ lr));
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
              mma_bf16_m16n8k8_full(oacc[2 * cq + jj], vb[2 * jj], vb[2 * jj + 1], phi[kt]);
              mma_bf16_m16n8k8_full(oacc[2 * cq + jj], vb[2 * jj], vb[2 * jj + 1], plo[kt]);
            }
          }
        }
      }
      __syncwarp();
      if (c.lane == 0) mbar_arrive(c.empty(c.slot));
      c.advance();
    }
    // ---- the warps' states meet in scratch: this lane holds columns d = 16 mt + g (+ 8) of
    // heads 2q and 2q+1, and the softmax state of head g
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      if (2 * q + hh < GQ) {
        float* dst = scratch + (c.warp * GQ + 2 * q + hh) * PW;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
          dst[16 * mt + g] = oacc[mt][hh];
          dst[16 * mt + 8 + g] = oacc[mt][2 + hh];
        }
      }
    }
    if (g < GQ && q == 0) {
      float* dst = scratch + (c.warp * GQ + g) * PW;
      dst[D] = m;
      dst[D + 1] = l;
    }
    consumer_sync();
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.attn) + size_t(a.b) * p.heads * D + size_t(a.g) * GQ * D;
    float* part = p.attn_part + size_t(a.task0 + a.c) * GQ * PW;
    for (int o = c.tid; o < GQ * D; o += kConsumerThreads) {
      const int h = o / D, d = o - h * D;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) mx = fmaxf(mx, scratch[(w * GQ + h) * PW + D]);
      const float ms = mx == -INFINITY ? 0.f : mx;
      float ls = 0.f, as = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float* src = scratch + (w * GQ + h) * PW;
        const float wgt = ex2(src[D] - ms);
        ls = fmaf(src[D + 1], wgt, ls);
        as = fmaf(src[d], wgt, as);
      }
      if (a.nch == 1) {
        out[o] = __float2bfloat16_rn(as / ls);
      } else {
        part[h * PW + d] = as;
        if (d == 0) {
          part[h * PW + D] = mx;
          part[h * PW + D + 1] = ls;
        }
      }
    }
    if (a.nch > 1) {
      // last arriver of (sequence, KV head) merges the chunks in chunk order
      // (include/tilemega/Backend/Sm90DenseAttentionBody.cuh:359-363,409-446)
      // (the CTA barrier orders every thread's partial stores before thread 0's counter
      // increment, which releases them and acquires the other chunks' -- the same pattern as
      // the grid arrival; the second barrier hands the acquired view to the other threads)
      consumer_sync();
      if (c.tid == 0) {
        unsigned* cnt = p.attn_cnt + a.b * p.kv_heads + a.g;
        const unsigned old = atom_acq_rel_add(cnt, 1u);
        const int last = old == unsigned(a.nch - 1);
        if (last) atomicExch(cnt, 0u);
        c.ctl()[1] = last;
      }
      consumer_sync();
      if (c.ctl()[1]) {
        const float* parts = p.attn_part + size_t(a.task0) * GQ * PW;
        // A thread merges NO outputs of ONE head, so the chunks' (max, sum) pairs are loaded once per
        // thread, and all of a batch of chunks' loads -- pairs and outputs -- are in flight together:
        // one L2 round trip for up to kMergeBatch chunks, where a loop over outputs paid one each.
        constexpr int TPH = kConsumerThreads / GQ;   // threads per head
        constexpr int NO = D / TPH;                  // outputs per thread: columns d0 + TPH * k
        static_assert(kConsumerThreads % GQ == 0 && D % TPH == 0, "merge mapping");
        constexpr int kMergeBatch = NO >= 4 ? 9 : 12;   // at most 54 loads per thread in flight (registers)
        const int h = c.tid / TPH, d0 = c.tid - h * TPH;
        float mx = -INFINITY, ls = 0.f, as[NO];
#pragma unroll
        for (int k = 0; k < NO; ++k) as[k] = 0.f;
        for (int c0 = 0; c0 < a.nch; c0 += kMergeBatch) {   // chunks in ascending order
          float mc[kMergeBatch], lc[kMergeBatch], ac[kMergeBatch][NO];
#pragma unroll
          for (int j = 0; j < kMergeBatch; ++j) {
            const bool live = c0 + j < a.nch;
            const float* src = parts + (size_t(live ? c0 + j : c0) * GQ + h) * PW;
            mc[j] = live ? __ldcg(src + D) : -INFINITY;
            lc[j] = live ? __ldcg(src + D + 1) : 0.f;
#pragma unroll
            for (int k = 0; k < NO; ++k) ac[j][k] = live ? __ldcg(src + d0 + TPH * k) : 0.f;
          }
          float mb = mx;
#pragma unroll
          for (int j = 0; j < kMergeBatch; ++j) mb = fmaxf(mb, mc[j]);
          const float rescale = ex2(mx - mb);   // mb is finite: chunk c0 exists and holds a valid key
          ls *= rescale;
#pragma unroll
          for (int k = 0; k < NO; ++k) as[k] *= rescale;
          mx = mb;
#pragma unroll
          for (int j = 0; j < kMergeBatch; ++j) {
            const float wgt = ex2(mc[j] - mb);
            ls = fmaf(lc[j], wgt, ls);
#pragma unroll
            for (int k = 0; k < NO; ++k) as[k] = fmaf(ac[j][k], wgt, as[k]);
          }
        }
#pragma unroll
        for (int k = 0; k < NO; ++k) out[h * D + d0 + TPH * k] = __float2bfloat16_rn(as[k] / ls);
      }
      consumer_sync();
    }
    }
    ++c.task_seq;
  }
  trace_mark(c, tr, stage, 3);
}

// ---------------------------------------------------------------------------
// arithmetic warps: one decode step after another
// ---------------------------------------------------------------------------
template <int B, int D, int GQ, int X>
__device__ void consumer_main(Ctx& c) {
  const MegaParams& p = c.p;
  for (int si = 0; si < p.nsteps; ++si) {
    const int step = p.first_step + si;
    const int past = __ldg(p.past + step);
    if (si == 0) {
      // the first step reads its token ids from the token state; later steps
      // carry them over from the argmax reduction below
      if (c.tid < B) c.tok()[c.tid] = __ldcg(p.tokens + size_t(c.tid) * p.capacity + seq_pos(p, past, c.tid));
      consumer_sync();
    }
    if (c.cta == 0 && c.tid == 0) p.step_ns[step] = global_timer();
    const bool tr = p.trace != nullptr && step == p.trace_step;
    int stage = 0;
    LayerPtrs lp = p.layer[0];
    // tensor parallel: o and down end in an all-reduce; epochs count all-reduces since the plan was made
    const int residual_kind = (X & kXTp) && p.tp_world > 1 ? kEpiResidualAllReduce : kEpiResidual;
    const unsigned long long steps_before = p.tp_steps + (unsigned long long)si;
    const uint32_t ar_epoch0 = uint32_t(steps_before * (unsigned long long)(2 * p.layers)) + 1u;
    for (int l = 0; l < p.layers; ++l) {
      // the next layer's pointer record is fetched a whole layer ahead of its use
      const LayerPtrs upcoming = p.layer[min(l + 1, p.layers - 1)];
      GemvIo io;
      // qkv: RMSNorm fused; layer 0 reads the embedding rows and seeds the residual stream
      trace_mark(c, tr, stage, 0);
      if (l > 0) {
        if (!grid_wait(c)) return;
      }
      trace_mark(c, tr, stage, 1);
      io = GemvIo{l == 0 ? p.embed : p.x, lp.norm1, l == 0, kEpiStore, p.qkv, p.qkv_ready, (GQ + 2) * D / kTileN, nullptr, 0, 0u,
                  lp.qkv_scale};
      gemv_stage<B, X>(c, p.geo[kQkv], io, tr, stage++);
      // no grid barrier here: an attention task needs the QKV rows of its own KV head
      // only, and waits for that group's row-tile count (qkv_ready)
      trace_mark(c, tr, stage, 0);
      trace_mark(c, tr, stage, 1);
      attn_stage<B, D, GQ, X>(c, lp, past, tr, stage++, (unsigned long long)(si * p.layers + l + 1));
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      io = GemvIo{p.attn, nullptr, 0, residual_kind, p.x, nullptr, 1, nullptr, 0, ar_epoch0 + uint32_t(2 * l), lp.o_scale};
      gemv_stage<B, X>(c, p.geo[kOProj], io, tr, stage++);
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      if ((X & kXMoe) && p.experts) {
        // mixture of experts: router scores, top-k, then the chosen experts only
        if constexpr ((X & kXMoe) != 0) {
          io = GemvIo{p.x, lp.norm2, 0, kEpiStore, p.router_logits, nullptr, 1, nullptr, 0, 0u};
          gemv_stage<B, X>(c, p.geo[kRouter], io, tr, stage++);
          grid_arrive(c);
          // The experts' MLP runs token by token: every token has its own experts, so their weights are
          // streamed per token (nothing is shared between tokens), each token a gate/up and a down stage
          // of the one-token form; 2 * B stages and arrivals per layer after the router's.
          for (int b = 0; b < B; ++b) {
            trace_mark(c, tr, stage, 0);
            if (!grid_wait(c)) return;         // b == 0: the router's scores; b > 0: token b-1's down stage read h
            trace_mark(c, tr, stage, 1);
            route_token(c, l, b);
            trace_mark(c, tr, stage, 1);   // the experts' inputs are there once the token is routed
            // task t = (expert slot, row tile): with one token the SwiGLU epilogue's output
            // index t * 4 + r is row `slot` of h[topk][inter]
            io = GemvIo{static_cast<const __nv_bfloat16*>(p.x) + size_t(b) * p.hidden, lp.norm2, 0, kEpiSwiGLU, p.h, nullptr, 1, nullptr, 0, 0u};
            gemv_stage<1, X>(c, p.geo[kGateUp], io, tr, stage++);
            grid_arrive(c);
            trace_mark(c, tr, stage, 0);
            if (!grid_wait(c)) return;
            trace_mark(c, tr, stage, 1);
            moe_down_stage(c, p.geo[kDown], tr, stage++, b);
            grid_arrive(c);
          }
        }
        lp = upcoming;
        continue;
      }
      io = GemvIo{p.x, lp.norm2, 0, kEpiSwiGLU, p.h, nullptr, 1, nullptr, 0, 0u, lp.gate_up_scale};
      gemv_stage<B, X>(c, p.geo[kGateUp], io, tr, stage++);
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      if (p.down_splits > 1) {
        // the reduction in parts: each part's rows fit in shared memory; the fp32 sums of the
        // parts so far wait in global memory, and only the last part rounds and adds the residual
        for (int part = 0; part < p.down_splits; ++part) {
          const bool last = part + 1 == p.down_splits;
          io = GemvIo{p.h, nullptr, 0, last ? residual_kind : int(kEpiPartial), last ? p.x : static_cast<void*>(p.down_partial),
                      nullptr, 1, part ? p.down_partial : nullptr, 1, ar_epoch0 + uint32_t(2 * l + 1), lp.down_scale};
          gemv_stage<B, X>(c, p.down_part[part], io, tr, stage++);
          grid_arrive(c);
          if (!last) {
            trace_mark(c, tr, stage, 0);
            if (!grid_wait(c)) return;
            trace_mark(c, tr, stage, 1);
          }
        }
      } else {
        io = GemvIo{p.h, nullptr, 0, residual_kind, p.x, nullptr, 1, nullptr, 1, ar_epoch0 + uint32_t(2 * l + 1), lp.down_scale};
        gemv_stage<B, X>(c, p.geo[kDown], io, tr, stage++);
        grid_arrive(c);
      }
      lp = upcoming;
    }
    trace_mark(c, tr, stage, 0);
    if (!grid_wait(c)) return;
    trace_mark(c, tr, stage, 1);
    GemvIo io{p.x, p.final_norm, 0, kEpiHead, p.logits, nullptr, 1, nullptr, 0, 0u, p.lm_head_scale};
    gemv_stage<B, X>(c, p.geo[kHead], io, tr, stage);
    consumer_sync();
    if (c.tid < B) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float v = c.best_val()[w * kMaxBatch + c.tid];
        const int i = c.best_idx()[w * kMaxBatch + c.tid];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
      p.argmax_val[size_t(c.cta) * B + c.tid] = bv;
      p.argmax_idx[size_t(c.cta) * B + c.tid] = bi;
    }
    grid_arrive(c);
    if (!grid_wait(c)) return;
    // every CTA reduces the per-CTA candidates itself: it needs the token for the
    // next step's embedding, and CTA 0 records it
    // (include/tilemega/Backend/Sm90DenseHead.cuh:48-135; ties -> smaller index)
    if (c.warp < B) {
      const int b = c.warp;
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = c.lane; g < p.grid; g += 32) {
        const float v = __ldcg(p.argmax_val + size_t(g) * B + b);
        const int i = __ldcg(p.argmax_idx + size_t(g) * B + b);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
#pragma unroll
      for (int mk = 16; mk; mk >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, mk);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, mk);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if ((X & kXTp) && p.tp_world > 1) {
        // Each rank scored a slice of the vocabulary: CTA 0 sends its winner (the compared
        // value is a bf16, the index fits 20 bits, so one packet holds both and a 28-bit
        // epoch) into every peer's block; every CTA then takes the best over the ranks in
        // ascending order, which is the whole-vocabulary argmax with ties to the smaller
        // index (include/tilemega/Backend/Sm90DenseHead.cuh:139-201).
        float ov = bv;
        int oi = bi;
        tp_exchange_argmax(p, c.cta, (steps_before + 1ull) & 0xfffffffull, b, c.lane, ov, oi);
#pragma unroll
        for (int mk = 4; mk; mk >>= 1) {   // tp_world <= 8: lanes 0..7 hold the ranks' candidates
          const float pv = __shfl_xor_sync(0xffffffffu, ov, mk);
          const int pi = __shfl_xor_sync(0xffffffffu, oi, mk);
          if (pv > ov || (pv == ov && pi < oi)) { ov = pv; oi = pi; }
        }
        bv = __shfl_sync(0xffffffffu, ov, 0);
        bi = __shfl_sync(0xffffffffu, oi, 0);
      }
      if (c.lane == 0) {
        const int pos = seq_pos(p, past, b);
        int* slot = p.tokens + size_t(b) * p.capacity + min(pos + 1, p.capacity - 1);
        int tok = min(max(bi, 0), p.vocab - 1);
        if (pos + 1 < p.prompt_len) {
          tok = __ldcg(slot);   // teacher-forced prompt position: the token state wins
        } else if (c.cta == 0 && pos + 1 < p.capacity) {
          *slot = tok;
        }
        c.tok()[b] = tok;
      }
    }
    if (c.cta == 0 && c.tid == 0) p.step_ns[step + 1] = global_timer();
    consumer_sync();
  }
}

template <int B, int D, int GQ, int X>
__device__ __forceinline__ void run_cta(const MegaParams& p, int cta) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Ctx c(p, smem, cta);
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.nslots; ++i) {
      mbar_init(c.full(i), 1);
      mbar_init(c.empty(i), kConsumerWarps);
    }
    for (int i = 0; i < kPartialRing; ++i) {
      mbar_init(c.pfull(i), kConsumerWarps);
    }
    mbar_init(c.route_bar(), 1);
    mbar_fence_init();
    for (int i = 0; i < 8; ++i) c.ctl()[i] = 0;
    for (int i = 0; i < kFifo; ++i) c.fifo()[i] = 0;   // sequence tag 0 never matches
  }
  __syncthreads();
  if (c.warp >= kConsumerWarps) {
    streamer_main<D, X>(c);   // the whole warp; lane 0 leads
    if (c.lane == 0) streamer_drain(c);
  } else {
    consumer_main<B, D, GQ, X>(c);
  }
}

template <int B, int D, int GQ, int X>
__global__ void __launch_bounds__(kThreads, 1) decode_megakernel(const __grid_constant__ MegaParams p) {
  run_cta<B, D, GQ, X>(p, int(blockIdx.x));
}

// Several rank plans of one tensor-parallel job as ONE cooperative launch on one device:
// CTAs [0, grid_0) run rank 0's plan, the next grid_1 rank 1's, and so on. The ranks wait
// for one another's packets, so they must be co-resident, which separate launches on one
// GPU cannot promise and a cooperative launch does. For boxes with fewer GPUs than ranks
// (and for tests); a rank's parameters are read from global memory here.
template <int B, int D, int GQ, int X>
__global__ void __launch_bounds__(kThreads, 1) decode_megakernel_ranks(const MegaParams* ranks, int count) {
  int base = 0, r = 0;
  while (r + 1 < count && int(blockIdx.x) >= base + ranks[r].grid) base += ranks[r++].grid;
  run_cta<B, D, GQ, X>(ranks[r], int(blockIdx.x) - base);
}

#if TMB_DENSE
// ---------------------------------------------------------------------------
// Dense-batch plans (batch 16..64): the GEMM stages on the 5th-generation tensor cores.
//
// A decode step keeps its stage list; what changes is who does the arithmetic of a GEMV
// stage. With B >= 16 rows the contraction is dense enough for a tcgen05 tile with the
// operands swapped: A = a weight page (M = 128 weight rows, K-major, 128-byte swizzled --
// exactly what the tile_pages recipe writes for tile_n = 128, so a page is still one
// contiguous 32 KB bulk copy and one ring slot), B = the activation rows of the batch
// (N = B, a 128-column chunk fetched by two tiled TMA loads through a tensor map over the
// row-major [B][K] buffer, swizzle done by the copy engine), D = fp32 [128 weight rows][B]
// in tensor memory. Roles per CTA:
//  * the streaming thread as before: it claims tasks, posts them and fills the ring with
//    weight pages (and KV slots), never waiting for a stage boundary;
//  * lane 0 of one more warp waits for the stage's inputs (the grid-wide arrival counter),
//    loads the activation chunks of each task, issues tcgen05.mma for every chunk that has
//    landed and lets tcgen05.commit release the slots and publish the accumulator;
//  * the arithmetic warps are two groups of four (a warp reads tensor-memory lanes
//    32*(warp%4)..+31): group g runs the epilogues of the CTA's tasks g, g+2, ... out of
//    accumulator g, so the next task's products overlap the previous task's epilogue. A
//    thread owns ONE weight row (output feature) for all batch rows.
// RMSNorm is a stage of its own here (rows spread over the CTAs, result in `xn`): a
// normalised row cannot stay in shared memory next to a ring when there are 64 of them.
// Attention is the same code as in the small-batch kernel.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t* dbar(const Ctx& c, int offset, int i) {
  return reinterpret_cast<uint64_t*>(c.smem + offset) + i;
}
__device__ __forceinline__ int* dtok(const Ctx& c) { return reinterpret_cast<int*>(c.smem + kOffDTok); }
__device__ __forceinline__ void group_sync(int group) { asm volatile("bar.sync %0, 128;" ::"r"(2 + group) : "memory"); }

// The issuing thread: next GEMM task of the stage. Returns the task id (or -1: stage closed,
// -2: the launch is being abandoned) and the first ring slot / phase of its pages.
__device__ __forceinline__ int dfifo_pop(Ctx& c, uint32_t& slot, uint32_t& phase) {
  const volatile uint32_t* entry = reinterpret_cast<volatile uint32_t*>(c.smem + kOffDFifo) + (c.dq_pos & (kFifo - 1));
  const uint32_t tag = (c.dq_pos + 1u) & 0xFFFu;
  uint32_t word = *entry;
  if (!c.dead && (word >> 20) != tag) {
    unsigned long long t0 = 0;
    uint32_t polls = 0;
    while (((word = *entry) >> 20) != tag) {
      if ((++polls & 255u) == 0 && wait_give_up(c.p, t0, kSiteFull, c.dq_pos, word)) {
        c.dead = true;
        break;
      }
    }
  }
  if (c.dead) return -2;
  ++c.dq_pos;
  c.ctl()[6] = int(c.dq_pos);
  slot = (word >> 17) & 7u;
  phase = (word >> 16) & 1u;
  const uint32_t value = word & kDFifoClose;
  return value == kDFifoClose ? -1 : int(value);
}

struct MmaState {
  uint32_t tmem, idesc;
  uint32_t nx;                                             // activation chunk slots in use (as many of 4 as fit 48 KB)
  uint32_t x_load_slot, x_load_phase, x_use_slot, x_use_phase;   // activation ring: next slot to fill / to consume
  uint32_t task_seq;                                       // GEMM tasks issued by this CTA (accumulator = task_seq & 1)
};

// One GEMM stage, issuing side. `arrivals`: grid-wide arrivals (counted from the start of the launch)
// after which the stage's input rows are complete in global memory.
__device__ __forceinline__ bool mma_stage(Ctx& c, MmaState& st, const DenseGeo& g, const void* tensor_map,
                                          unsigned long long arrivals) {
  const MegaParams& p = c.p;
  {
    const unsigned long long need = p.bar_base + arrivals * (unsigned long long)p.grid;
    unsigned long long t0 = 0, seen;
    uint32_t polls = 0;
    while ((seen = ld_acquire(p.bar)) < need) {
      if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSiteGrid, need, seen)) {
        c.dead = true;
        return false;
      }
    }
    fence_proxy_async();   // the rows were written with ordinary stores by other CTAs; the copy engine reads them
  }
  const uint32_t chunk_bytes = uint32_t(p.batch) * kDenseTileK * 2u;
  const uint32_t block_bytes = uint32_t(p.batch) * 128u;   // one 64-column swizzle block of the batch rows
  unsigned char* const xring = c.smem + kOffDenseXs;
  const uint32_t nx = st.nx;
  // operand descriptors differ from a slot's base descriptor by the byte offset >> 4 only (shared memory
  // addresses have 18 bits, the field 14): k-step ks of swizzle block cb lies cb * block + 32 * ks bytes in
  const uint64_t desc_hi = umma_desc_k_sw128(0u, 1024u);
  uint32_t slot = 0, phase = 0;
  for (int t = dfifo_pop(c, slot, phase); t >= 0; t = dfifo_pop(c, slot, phase)) {
    const int part = t % g.nsplit;
    const int block0 = part * g.cps * (kDenseTileK / 64);   // first 64-column block of this part of the reduction
    const uint32_t buf = st.task_seq & 1u;
    // the accumulator's previous tile (two tasks ago) must have been read out
    if (!mbar_wait(c, dbar(c, kOffDAccEmpty, buf), ((st.task_seq >> 1) & 1u) ^ 1u, kSiteEmpty)) return false;
    tcgen05_fence_after();
    const uint32_t d_tmem = st.tmem + buf * uint32_t(kDenseMaxBatch);
    int loaded = 0;
    for (int i = 0; i < g.cps; ++i) {
      // keep up to nx activation chunks of this task in flight
      while (loaded < g.cps && loaded < i + int(nx)) {
        if (!mbar_wait(c, dbar(c, kOffDXEmpty, st.x_load_slot), st.x_load_phase ^ 1u, kSiteEmpty)) return false;
        mbar_expect_tx(dbar(c, kOffDXFull, st.x_load_slot), chunk_bytes);
        tma_load_3d(xring + st.x_load_slot * chunk_bytes, tensor_map, 0, 0, block0 + 2 * loaded, dbar(c, kOffDXFull, st.x_load_slot));
        if (++st.x_load_slot == nx) { st.x_load_slot = 0; st.x_load_phase ^= 1u; }
        ++loaded;
      }
      if (!mbar_wait(c, c.full(slot), phase, kSiteFull)) return false;
      if (!mbar_wait(c, dbar(c, kOffDXFull, st.x_use_slot), st.x_use_phase, kSiteFull)) return false;
      tcgen05_fence_after();
      const uint64_t a0 = desc_hi + (smem_u32(c.ring(slot)) >> 4);
      const uint64_t b0 = desc_hi + (smem_u32(xring + st.x_use_slot * chunk_bytes) >> 4);
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_bf16(d_tmem, a0 + ((cb * (kDenseTileN * 128) + ks * 32) >> 4), b0 + ((cb * block_bytes + ks * 32) >> 4), st.idesc,
                    (i | cb | ks) != 0 ? 1u : 0u);
      }
      umma_commit(dbar(c, kOffDWEmpty, slot));                 // the weight page's slot, back to the streaming thread
      umma_commit(dbar(c, kOffDXEmpty, st.x_use_slot));
      if (++st.x_use_slot == nx) { st.x_use_slot = 0; st.x_use_phase ^= 1u; }
      if (++slot == uint32_t(p.nslots)) { slot = 0; phase ^= 1u; }
    }
    umma_commit(dbar(c, kOffDAccFull, buf));
    ++st.task_seq;
  }
  return !c.dead;
}

template <int GQ>
__device__ void mma_main_dense(Ctx& c) {
  const MegaParams& p = c.p;
  MmaState st;
  st.tmem = *reinterpret_cast<volatile uint32_t*>(c.smem + kOffDTmem);
  st.idesc = umma_idesc_bf16(kDenseTileN, p.batch);
  st.nx = uint32_t(dense_x_slots(p.batch));
  st.x_load_slot = st.x_load_phase = st.x_use_slot = st.x_use_phase = st.task_seq = 0;
  const unsigned char* maps = static_cast<const unsigned char*>(p.tmaps);
  bool alive = true;
  for (int si = 0; si < p.nsteps && alive; ++si) {
    // arrivals of a step, in program order: per layer norm1, [chunk_rows: QKV, append,] attention, o, norm2,
    // gate/up, down; then final norm, head
    const unsigned long long step0 = (unsigned long long)si * p.bars_per_step;
    const unsigned long long extra = p.chunk_rows ? 2ull : 0ull, per_layer = 6ull + extra;
    for (int l = 0; l < p.layers && alive; ++l) {
      const unsigned long long base = step0 + per_layer * l;
      alive = mma_stage(c, st, p.dgeo[kQkv], maps, base + 1) && mma_stage(c, st, p.dgeo[kOProj], maps + 128, base + 2 + extra) &&
              mma_stage(c, st, p.dgeo[kGateUp], maps, base + 4 + extra) && mma_stage(c, st, p.dgeo[kDown], maps + 256, base + 5 + extra);
    }
    if (alive) alive = mma_stage(c, st, p.dgeo[kHead], maps, step0 + per_layer * p.layers + 1);
  }
  // nothing of this CTA may still be running on the tensor cores when tensor memory is freed
  umma_commit(dbar(c, kOffDDrain, 0));
  unsigned long long t0 = 0;
  uint32_t polls = 0;
  while (!mbar_try_wait(dbar(c, kOffDDrain, 0), 0u)) {
    if ((++polls & 127u) == 0) {
      const unsigned long long now = global_timer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > p.watchdog_ns) break;
    }
  }
}

// RMSNorm stage: row b of the batch is normalised by CTA b mod grid and written to xn
// (y = bf16(w * bf16(x * rsqrt(mean x^2 + eps))), python/tilemega/serving/export.py:24-27). Layer 0
// reads the embedding row of the sequence's token and also seeds the residual stream with it.
// `parts` > 1: the projection into the residual stream that ran before this stage (o, or the previous
// layer's down) left its reduction as `parts` fp32 tiles per 128 features; the row is first completed
// here, x = bf16(bf16(sum of the parts, ascending) + x), and written back.
__device__ void norm_stage_dense(Ctx& c, const void* src, const void* weight, bool embed, int parts = 1) {
  const MegaParams& p = c.p;
  const int chunks = p.hidden >> 3;
  const uint4* nw = reinterpret_cast<const uint4*>(weight);
  const size_t tile_floats = size_t(kDenseTileN) * p.batch;
  for (int b = c.cta; b < p.batch; b += p.grid) {
    const __nv_bfloat16* row = static_cast<const __nv_bfloat16*>(src) +
                               (embed ? size_t(min(max(dtok(c)[b], 0), p.vocab - 1)) : size_t(b)) * p.hidden;
    constexpr int kHold = 4;   // hidden <= 8192: at most four 16-byte chunks per thread
    uint4 v[kHold], wv[kHold];
    float ss = 0.f;
    // Two chunks per thread at a time, and everything they need -- the row's values, the norm weights, the
    // first four parts' partial sums -- requested before anything is used: one L2 round trip for the stage's
    // loads where chunk after chunk, part group after part group and then the weights paid four or more.
#pragma unroll
    for (int j0 = 0; j0 < kHold; j0 += 2) {
      float4 x[2][4][2];
      const float4* tile0[2];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int i = c.tid + (j0 + jj) * kConsumerThreads;
        const bool live = i < chunks;
        v[j0 + jj] = wv[j0 + jj] = make_uint4(0u, 0u, 0u, 0u);
        if (live) {
          v[j0 + jj] = embed ? __ldg(reinterpret_cast<const uint4*>(row) + i) : __ldcg(reinterpret_cast<const uint4*>(row) + i);
          wv[j0 + jj] = __ldg(nw + i);
        }
        // columns 8i .. 8i+7 lie in tile i / 16 at feature 8 * (i % 16): two 16-byte loads per part
        tile0[jj] = reinterpret_cast<const float4*>(p.gemm_part + (size_t(i >> 4) * parts * p.batch + b) * kDenseTileN + ((i & 15) << 3));
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          const bool wanted = parts > 1 && live && pp < parts;
          const float4* at = tile0[jj] + size_t(wanted ? pp : 0) * (tile_floats >> 2);
          x[jj][pp][0] = wanted ? __ldcg(at) : make_float4(0.f, 0.f, 0.f, 0.f);
          x[jj][pp][1] = wanted ? __ldcg(at + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int i = c.tid + (j0 + jj) * kConsumerThreads;
        float f[8];
        unpack8(v[j0 + jj], f);
        if (parts > 1 && i < chunks) {
          float sum[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) sum[e] = 0.f;
#pragma unroll
          for (int pp = 0; pp < 4; ++pp) {   // ascending part order
            sum[0] += x[jj][pp][0].x; sum[1] += x[jj][pp][0].y; sum[2] += x[jj][pp][0].z; sum[3] += x[jj][pp][0].w;
            sum[4] += x[jj][pp][1].x; sum[5] += x[jj][pp][1].y; sum[6] += x[jj][pp][1].z; sum[7] += x[jj][pp][1].w;
          }
          for (int part = 4; part < parts; ++part) {   // (more than four parts: the rest, part by part)
            const float4* at = tile0[jj] + size_t(part) * (tile_floats >> 2);
            const float4 lo = __ldcg(at), hi = __ldcg(at + 1);
            sum[0] += lo.x; sum[1] += lo.y; sum[2] += lo.z; sum[3] += lo.w;
            sum[4] += hi.x; sum[5] += hi.y; sum[6] += hi.z; sum[7] += hi.w;
          }
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            f[2 * e] = bf16_round(bf16_round(sum[2 * e]) + f[2 * e]);
            f[2 * e + 1] = bf16_round(bf16_round(sum[2 * e + 1]) + f[2 * e + 1]);
            o[e] = uint32_t(bf16_bits(f[2 * e])) | (uint32_t(bf16_bits(f[2 * e + 1])) << 16);
          }
          v[j0 + jj] = make_uint4(o[0], o[1], o[2], o[3]);
          reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.x) + size_t(b) * p.hidden)[i] = v[j0 + jj];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
      }
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    if (c.lane == 0) c.wsum()[c.warp] = ss;
    consumer_sync();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) total += c.wsum()[w];
    const float inv = 1.0f / sqrtf(total / float(p.hidden) + p.eps);
#pragma unroll
    for (int j = 0; j < kHold; ++j) {
      const int i = c.tid + j * kConsumerThreads;
      if (i < chunks) {
        float f[8], w[8];
        unpack8(v[j], f);
        unpack8(wv[j], w);
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[e] = uint32_t(bf16_bits(w[2 * e] * bf16_round(f[2 * e] * inv))) |
                 (uint32_t(bf16_bits(w[2 * e + 1] * bf16_round(f[2 * e + 1] * inv))) << 16);
        reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.xn) + size_t(b) * p.hidden)[i] = make_uint4(o[0], o[1], o[2], o[3]);
        if (embed) reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.x) + size_t(b) * p.hidden)[i] = v[j];
      }
    }
    consumer_sync();   // wsum is reused by the next row
  }
}

// The rounding sites of one stage's epilogue on 16 batch rows (b0 .. b0+15) of ONE output feature
// `row`, held by one thread (include/tilemega/Backend/ServingEpilogue.h:38-57; Sm90DenseEpilogue.h:166-184).
__device__ __forceinline__ void dense_epilogue_16(Ctx& c, const DenseGeo& g, const GemvIo& io, const float (&v)[16], int b0,
                                                  int row, int tile) {
  const MegaParams& p = c.p;
  const int lane = c.lane, wq = c.warp & 3;
  if (io.epilogue == kEpiStore) {
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(io.out) + row;
#pragma unroll
    for (int j = 0; j < 16; ++j) out[size_t(b0 + j) * g.n] = __float2bfloat16_rn(v[j]);
  } else if (io.epilogue == kEpiResidual) {
    unsigned short* out = reinterpret_cast<unsigned short*>(io.out) + row;
    float res[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) res[j] = bf16_from_bits(__ldcg(out + size_t(b0 + j) * g.n));
#pragma unroll
    for (int j = 0; j < 16; ++j) out[size_t(b0 + j) * g.n] = bf16_bits(bf16_round(v[j]) + res[j]);
  } else if (io.epilogue == kEpiSwiGLU) {
    // rows come in units of 16 gate rows followed by their 16 up rows: lane l < 16 holds the gate of
    // feature tile*64 + wq*16 + l, lane l + 16 its up value
    __nv_bfloat16* h = static_cast<__nv_bfloat16*>(io.out) + tile * (kDenseTileN / 2) + wq * 16 + (lane & 15);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float vb = bf16_round(v[j]);
      const float up = __shfl_down_sync(0xffffffffu, vb, 16);
      if (lane < 16) h[size_t(b0 + j) * (g.n >> 1)] = __float2bfloat16_rn(silu_bf16(vb) * up);
    }
  } else {   // kEpiHead
    float* best_val = reinterpret_cast<float*>(c.smem + kOffDBestVal) + c.warp * kDenseMaxBatch;
    int* best_idx = reinterpret_cast<int*>(c.smem + kOffDBestIdx) + c.warp * kDenseMaxBatch;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (p.write_logits) static_cast<float*>(io.out)[size_t(b0 + j) * g.n + row] = v[j];
      float bv = bf16_round(v[j]);
      int bi = p.head_base + row;
#pragma unroll
      for (int m = 1; m < 32; m <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == ((b0 + j) & 31)) {   // one lane keeps the warp's running best of this batch row
        const float old = best_val[b0 + j];
        if (bv > old || (bv == old && bi < best_idx[b0 + j])) {
          best_val[b0 + j] = bv;
          best_idx[b0 + j] = bi;
        }
      }
    }
  }
}

// One GEMM stage, epilogue side. Both warp groups walk the CTA's task list; group g takes every
// second task. `seq` counts the CTA's GEMM tasks across stages (it selects the accumulator).
// `fold`: a reduction that runs in parts ends here with the parts' fp32 tiles in global memory; the
// stage that consumes the output adds them (attention staging for QKV, the next RMSNorm stage for the
// residual stream). Without it the last part to arrive adds them here -- a tail of dependent L2 round
// trips on one CTA per tile that the whole grid then waits for.
__device__ void gemm_epilogue_stage(Ctx& c, const DenseGeo& g, const GemvIo& io, uint32_t& seq, bool fold = false) {
  const MegaParams& p = c.p;
  const int group = c.warp >> 2, wq = c.warp & 3, m = wq * 32 + c.lane;
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(c.smem + kOffDTmem);
  const int nb = p.batch >> 4;   // 16-row chunks of the batch
  volatile int* last_flag = c.ctl() + (group ? 7 : 5);
  for (int t = fifo_pop(c); t >= 0; t = fifo_pop(c)) {
    // the ring cursor follows every task (the attention stages consume slots from it)
    for (int i = 0; i < g.cps; ++i) c.advance();
    const uint32_t my_seq = seq++;
    if (int(my_seq & 1u) != group) continue;
    const int tile = t / g.nsplit;
    const int row = tile * kDenseTileN + m;
    mbar_wait_warp(c, dbar(c, kOffDAccFull, group), (my_seq >> 1) & 1u, kSiteFull);
    tcgen05_fence_after();
    const uint32_t taddr = tmem + (uint32_t(wq * 32) << 16) + uint32_t(group) * uint32_t(kDenseMaxBatch);
    if (g.nsplit == 1) {
      for (int j = 0; j < nb; ++j) {
        float v[16];
        tmem_load_16(taddr + 16 * j, v);
        if (j == nb - 1) {   // the accumulator is in registers: the tensor cores may overwrite it
          tcgen05_fence_before();
          __syncwarp();
          if (c.lane == 0) mbar_arrive(dbar(c, kOffDAccEmpty, group));
        }
        dense_epilogue_16(c, g, io, v, 16 * j, row, tile);
      }
    } else {
      // this part's fp32 tile goes to global memory, laid out [batch row][weight row] so that a warp's
      // accesses are one 128-byte line each; the last part to arrive adds all parts in ascending
      // order (so the sum does not depend on arrival order) and runs the epilogue
      const size_t tile_floats = size_t(kDenseTileN) * p.batch;
      float* mine = p.gemm_part + size_t(t) * tile_floats + m;
      for (int j = 0; j < nb; ++j) {
        float v[16];
        tmem_load_16(taddr + 16 * j, v);
#pragma unroll
        for (int e = 0; e < 16; ++e) mine[size_t(16 * j + e) * kDenseTileN] = v[e];
      }
      tcgen05_fence_before();
      __syncwarp();
      if (c.lane == 0) mbar_arrive(dbar(c, kOffDAccEmpty, group));
      if (fold) {
        if (io.ready) {
          // one more part of a 128-row tile of this KV-head group is in global memory
          group_sync(group);
          if ((c.tid & 127) == 0) red_release_add(io.ready + tile / io.tiles_per_group, (unsigned long long)(kDenseTileN / kTileN));
        }
        continue;
      }
      group_sync(group);   // every thread's partial stores are ordered before the counter below
      if ((c.tid & 127) == 0) {
        const unsigned old = atom_acq_rel_add(p.gemm_cnt + tile, 1u);
        const int last = old == unsigned(g.nsplit - 1);
        if (last) atomicExch(p.gemm_cnt + tile, 0u);
        *last_flag = last;
      }
      group_sync(group);
      const bool last = *last_flag != 0;
      group_sync(group);   // everyone has read the flag before the next task may overwrite it
      if (!last) continue;
      const float* parts = p.gemm_part + size_t(tile) * g.nsplit * tile_floats + m;
      for (int j = 0; j < nb; ++j) {
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = 0.f;
        // two parts' loads in flight together (32 per thread, each a full line per warp), added in ascending order
        for (int part0 = 0; part0 < g.nsplit; part0 += 2) {
          float x[2][16];
#pragma unroll
          for (int pp = 0; pp < 2; ++pp) {
            const bool live = part0 + pp < g.nsplit;
            const float* src = parts + size_t(live ? part0 + pp : part0) * tile_floats + size_t(16 * j) * kDenseTileN;
#pragma unroll
            for (int e = 0; e < 16; ++e) x[pp][e] = live ? __ldcg(src + size_t(e) * kDenseTileN) : 0.f;
          }
#pragma unroll
          for (int pp = 0; pp < 2; ++pp) {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] += x[pp][e];
          }
        }
        dense_epilogue_16(c, g, io, v, 16 * j, row, tile);
      }
    }
    if (io.ready) {
      // one more 128-row tile of this KV-head group is in global memory (counted in 8-row units, the
      // unit the attention tasks' readiness test uses)
      group_sync(group);
      if ((c.tid & 127) == 0) red_release_add(io.ready + tile / io.tiles_per_group, (unsigned long long)(kDenseTileN / kTileN));
    }
  }
}

// chunk_rows plans: RoPE and cache append for every (row, KV head), spread over the CTAs, before any
// attention task runs. Rows of the batch may be consecutive positions of one sequence (chunked
// prefill): row i then attends to the keys and values rows j < i append in this same step, which
// therefore have to be in the pool -- behind a grid barrier -- first. Same arithmetic as the
// attention tasks' own staging (include/tilemega/Codegen/tasks/FusedAttentionTaskBody.h:141-151).
template <int GQ>
__device__ void append_stage_dense(Ctx& c, const LayerPtrs& lp, int past) {
  constexpr int D = 128;
  static_assert(kConsumerThreads == 2 * D, "one thread per key column and per value column");
  const MegaParams& p = c.p;
  const int parts = p.dgeo[kQkv].nsplit;
  const size_t tile_floats = size_t(kDenseTileN) * p.batch;
  const int qkv_width = (p.heads + 2 * p.kv_heads) * D;
  const bool is_v = c.tid >= D;
  const int d = c.tid & (D - 1);
  for (int u = c.cta; u < p.batch * p.kv_heads; u += p.grid) {
    const int b = u / p.kv_heads, g = u - b * p.kv_heads;
    const int pos = seq_pos(p, past, b);
    const long long e = table_entry(p, seq_of(p, past, b), pos / kKvBlock);
    const long long at = e * p.kv_block_stride + (long long)g * p.kv_head_stride + (pos % kKvBlock) * D + kv_swizzled(d, pos);
    const int n0 = g * (GQ + 2) * D + (GQ + (is_v ? 1 : 0)) * D;   // first feature of this head's key (value) row
    auto feature = [&](int col) -> float {
      const int n = n0 + col;
      if (parts == 1) return bf16_from_bits(__ldcg(reinterpret_cast<const unsigned short*>(p.qkv) + size_t(b) * qkv_width + n));
      const float* src = p.gemm_part + (size_t(n >> 7) * parts * p.batch + b) * kDenseTileN + (n & 127);
      float v = 0.f;
#pragma unroll 4
      for (int part = 0; part < parts; ++part) v += __ldcg(src + size_t(part) * tile_floats);
      return bf16_round(v);
    };
    const float x = feature(d);
    if (is_v) {
      static_cast<__nv_bfloat16*>(lp.v_pool)[at] = __float2bfloat16_rn(x);
    } else {
      const float xp = feature(d < D / 2 ? d + D / 2 : d - D / 2);
      const float cs = bf16_from_bits(__ldg(reinterpret_cast<const unsigned short*>(p.rope_cos) + size_t(pos) * D + d));
      const float sn = bf16_from_bits(__ldg(reinterpret_cast<const unsigned short*>(p.rope_sin) + size_t(pos) * D + d));
      const float rot = d < D / 2 ? -xp : xp;
      static_cast<__nv_bfloat16*>(lp.k_pool)[at] = __float2bfloat16_rn(bf16_round(bf16_round(x * cs) + bf16_round(rot * sn)));
    }
  }
}

template <int GQ>
__device__ void consumer_main_dense(Ctx& c) {
  const MegaParams& p = c.p;
  constexpr int D = 128;
  const int B = p.batch;
  uint32_t seq = 0;
  for (int si = 0; si < p.nsteps; ++si) {
    const int step = p.first_step + si;
    const int past = __ldg(p.past + step);
    if (si == 0 || p.row_seq) {   // (a prefill plan's rows are other (sequence, position) pairs in every step)
      if (c.tid < B) dtok(c)[c.tid] = __ldcg(p.tokens + size_t(seq_of(p, past, c.tid)) * p.capacity + seq_pos(p, past, c.tid));
      consumer_sync();
    }
    if (c.cta == 0 && c.tid == 0) p.step_ns[step] = global_timer();
    const bool tr = p.trace != nullptr && step == p.trace_step;
    int stage = 0;
    for (int l = 0; l < p.layers; ++l) {
      const LayerPtrs lp = p.layer[l];
      GemvIo io;
      // Every stage starts with the wait for the previous stage's arrivals, also where the epilogue
      // warps would be held back by their accumulators anyway: the arrival counter is one monotonic
      // count, so a CTA (one without tasks in a stage, say) must never arrive for stage n+1 before it
      // has seen every CTA's arrival for stage n.
      trace_mark(c, tr, stage, 0);
      if (l > 0 && !grid_wait(c)) return;                      // the previous layer's down projection is complete
      trace_mark(c, tr, stage, 1);
      trace_mark(c, tr, stage, 2);
      norm_stage_dense(c, l == 0 ? p.embed : p.x, lp.norm1, l == 0, l == 0 ? 1 : p.dgeo[kDown].nsplit);
      trace_mark(c, tr, stage++, 3);
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      trace_mark(c, tr, stage, 2);
      io = GemvIo{nullptr, nullptr, 0, kEpiStore, p.qkv, p.qkv_ready, (GQ + 2) * D / kDenseTileN, nullptr, 0, 0u};
      gemm_epilogue_stage(c, p.dgeo[kQkv], io, seq, true);   // parts summed by the attention tasks
      trace_mark(c, tr, stage++, 3);
      // no arrival here: an attention task waits for the QKV rows of its own KV head only
      // (chunk_rows: all of QKV, then every row's cache append, each behind a grid barrier)
      if (p.chunk_rows) {
        grid_arrive(c);
        if (!grid_wait(c)) return;
        append_stage_dense<GQ>(c, lp, past);
        grid_arrive(c);
        if (!grid_wait(c)) return;
      }
      trace_mark(c, tr, stage, 0);
      trace_mark(c, tr, stage, 1);
      attn_stage<1, D, GQ, 0>(c, lp, past, tr, stage++, (unsigned long long)(si * p.layers + l + 1));
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      trace_mark(c, tr, stage, 2);
      io = GemvIo{nullptr, nullptr, 0, kEpiResidual, p.x, nullptr, 1, nullptr, 0, 0u};
      gemm_epilogue_stage(c, p.dgeo[kOProj], io, seq, true);   // parts summed by the RMSNorm stage that follows
      trace_mark(c, tr, stage++, 3);
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;                               // the residual stream after attention is complete
      trace_mark(c, tr, stage, 1);
      trace_mark(c, tr, stage, 2);
      norm_stage_dense(c, p.x, lp.norm2, false, p.dgeo[kOProj].nsplit);
      trace_mark(c, tr, stage++, 3);
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      trace_mark(c, tr, stage, 2);
      io = GemvIo{nullptr, nullptr, 0, kEpiSwiGLU, p.h, nullptr, 1, nullptr, 0, 0u};
      gemm_epilogue_stage(c, p.dgeo[kGateUp], io, seq);
      trace_mark(c, tr, stage++, 3);
      grid_arrive(c);
      trace_mark(c, tr, stage, 0);
      if (!grid_wait(c)) return;
      trace_mark(c, tr, stage, 1);
      trace_mark(c, tr, stage, 2);
      io = GemvIo{nullptr, nullptr, 0, kEpiResidual, p.x, nullptr, 1, nullptr, 0, 0u};
      gemm_epilogue_stage(c, p.dgeo[kDown], io, seq, true);   // parts summed by the next RMSNorm stage
      trace_mark(c, tr, stage++, 3);
      grid_arrive(c);
    }
    trace_mark(c, tr, stage, 0);
    if (!grid_wait(c)) return;
    trace_mark(c, tr, stage, 1);
    trace_mark(c, tr, stage, 2);
    norm_stage_dense(c, p.x, p.final_norm, false, p.dgeo[kDown].nsplit);
    trace_mark(c, tr, stage++, 3);
    grid_arrive(c);
    trace_mark(c, tr, stage, 0);
    if (!grid_wait(c)) return;
    trace_mark(c, tr, stage, 1);
    trace_mark(c, tr, stage, 2);
    // lm_head: every warp keeps a running (value, index) per batch row
    float* best_val = reinterpret_cast<float*>(c.smem + kOffDBestVal);
    int* best_idx = reinterpret_cast<int*>(c.smem + kOffDBestIdx);
    for (int i = c.tid; i < kConsumerWarps * kDenseMaxBatch; i += kConsumerThreads) {
      best_val[i] = -INFINITY;
      best_idx[i] = 0x7fffffff;
    }
    consumer_sync();
    GemvIo io{nullptr, nullptr, 0, kEpiHead, p.logits, nullptr, 1, nullptr, 0, 0u};
    gemm_epilogue_stage(c, p.dgeo[kHead], io, seq);
    trace_mark(c, tr, stage, 3);
    consumer_sync();
    if (c.tid < B) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float v = best_val[w * kDenseMaxBatch + c.tid];
        const int i = best_idx[w * kDenseMaxBatch + c.tid];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
      p.argmax_val[size_t(c.cta) * B + c.tid] = bv;
      p.argmax_idx[size_t(c.cta) * B + c.tid] = bi;
    }
    grid_arrive(c);
    if (!grid_wait(c)) return;
    // every CTA reduces the per-CTA candidates itself (it needs the tokens for the next step's
    // embedding); CTA 0 records them (include/tilemega/Backend/Sm90DenseHead.cuh:48-135)
    for (int b = c.warp; b < B; b += kConsumerWarps) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int gi = c.lane; gi < p.grid; gi += 32) {
        const float v = __ldcg(p.argmax_val + size_t(gi) * B + b);
        const int i = __ldcg(p.argmax_idx + size_t(gi) * B + b);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
#pragma unroll
      for (int mk = 16; mk; mk >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, mk);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, mk);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (c.lane == 0) {
        const int pos = seq_pos(p, past, b), sq = seq_of(p, past, b);
        int* slot = p.tokens + size_t(sq) * p.capacity + min(pos + 1, p.capacity - 1);
        int tok = min(max(bi, 0), p.vocab - 1);
        // a prefill plan's prompt starts at its sequence's context_base: its positions are forced up to there
        const int forced_below = p.prompt_len + (p.row_pos && p.ctx_base ? __ldg(p.ctx_base + sq) : 0);
        if (pos + 1 < forced_below) {
          tok = __ldcg(slot);   // teacher-forced prompt position: the token state wins
        } else if (c.cta == 0 && pos + 1 < p.capacity) {
          *slot = tok;
        }
        dtok(c)[b] = tok;
      }
    }
    if (c.cta == 0 && c.tid == 0) p.step_ns[step + 1] = global_timer();
    consumer_sync();
  }
}

template <int GQ>
__global__ void __launch_bounds__(kDenseThreads, 1) dense_megakernel(const __grid_constant__ MegaParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Ctx c(p, smem, int(blockIdx.x));
  if (threadIdx.x == 0) {
    for (int i = 0; i < p.nslots; ++i) {
      mbar_init(c.full(i), 1);
      mbar_init(c.empty(i), kConsumerWarps);
    }
    for (int i = 0; i < kDenseXSlots; ++i) {
      mbar_init(dbar(c, kOffDXFull, i), 1);
      mbar_init(dbar(c, kOffDXEmpty, i), 1);
    }
    for (int i = 0; i < p.nslots; ++i) mbar_init(dbar(c, kOffDWEmpty, i), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(dbar(c, kOffDAccFull, i), 1);
      mbar_init(dbar(c, kOffDAccEmpty, i), 4);
    }
    mbar_init(dbar(c, kOffDDrain, 0), 1);
    mbar_fence_init();
    for (int i = 0; i < 8; ++i) c.ctl()[i] = 0;
    for (int i = 0; i < kFifo; ++i) {
      c.fifo()[i] = 0;   // sequence tag 0 never matches
      reinterpret_cast<int*>(smem + kOffDFifo)[i] = 0;
    }
  }
  const bool issuer = c.warp == kConsumerWarps + 1;
  if (issuer) tmem_alloc(reinterpret_cast<uint32_t*>(smem + kOffDTmem), kDenseTmemColumns);   // the whole warp
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (c.warp == kConsumerWarps) {
    streamer_main<128, 0>(c);   // the whole warp; lane 0 leads
    if (c.lane == 0) streamer_drain(c);
  } else if (issuer) {
    if (c.lane == 0) mma_main_dense<GQ>(c);
  } else {
    consumer_main_dense<GQ>(c);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (issuer) tmem_dealloc(*reinterpret_cast<volatile uint32_t*>(smem + kOffDTmem), kDenseTmemColumns);
}

template <int GQ>
static cudaError_t run_dense_instance(const MegaParams& p, size_t smem_bytes, cudaStream_t stream, bool prepare) {
  auto kernel = dense_megakernel<GQ>;
  if (prepare) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));
    if (err != cudaSuccess) return err;
    int resident = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kDenseThreads, smem_bytes);
    if (err != cudaSuccess) return err;
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return (resident < 1 || p.grid > sms * resident) ? cudaErrorLaunchOutOfResources : cudaSuccess;
  }
  kernel<<<p.grid, kDenseThreads, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t run_decode_dense(const MegaParams& p, cudaStream_t stream, bool prepare) {
  const size_t smem_bytes = size_t(ring_offset(p.xs_bytes, p.batch) + p.nslots * kSlotBytes);
  if (p.kv_heads <= 0 || p.heads % p.kv_heads || p.head_dim != 128 || p.batch < 16 || p.batch > kDenseMaxBatch || p.batch % 16 ||
      p.hidden > 8192 || p.tp_world > 1 || p.experts > 0 || p.qk_norm)
    return cudaErrorInvalidValue;
  const int gq = p.heads / p.kv_heads;
  if (gq == 4) return run_dense_instance<4>(p, smem_bytes, stream, prepare);
  if (gq == 8) return run_dense_instance<8>(p, smem_bytes, stream, prepare);
  return cudaErrorInvalidValue;
}
#endif   // TMB_DENSE

#if !TMB_EXTENDED && !TMB_DENSE && !TMB_FP8
// A two-CTA toy that exercises the bounded-wait path without hanging anything:
// CTA 1 waits for an arrival CTA 0 is told to withhold; the wait gives up after
// watchdog_ns, records the site and both CTAs return normally.
__global__ void watchdog_probe_kernel(MegaParams p, int withhold) {
  if (threadIdx.x != 0) return;
  if (blockIdx.x == 0) {
    if (!withhold) red_release_add(p.bar, 1ull);
    return;
  }
  unsigned long long t0 = 0, seen;
  uint32_t polls = 0;
  while ((seen = ld_acquire(p.bar)) < p.bar_base + 1) {
    if ((++polls & 63u) == 0 && wait_give_up(p, t0, kSiteTest, p.bar_base + 1, seen)) break;
  }
}

#endif

template <int B, int D, int GQ, int X>
static cudaError_t run_instance(const MegaParams& p, size_t smem_bytes, cudaStream_t stream, bool prepare) {
  auto kernel = decode_megakernel<B, D, GQ, X>;
  if (prepare) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));
    if (err != cudaSuccess) return err;
    int resident = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kThreads, smem_bytes);
    if (err != cudaSuccess) return err;
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    // liveness: every CTA of the grid must be resident at once
    // (include/tilemega/Codegen/tasks/Sm90DenseRuntime.cuh:304-308)
    return (resident < 1 || p.grid > sms * resident) ? cudaErrorLaunchOutOfResources : cudaSuccess;
  }
  kernel<<<p.grid, kThreads, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

template <int D, int GQ, int X>
static cudaError_t run_batch(const MegaParams& p, size_t smem_bytes, cudaStream_t stream, bool prepare) {
  switch (p.batch) {
    case 1: return run_instance<1, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 2: return run_instance<2, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 3: return run_instance<3, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 4: return run_instance<4, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 5: return run_instance<5, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 6: return run_instance<6, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 7: return run_instance<7, D, GQ, X>(p, smem_bytes, stream, prepare);
    case 8: return run_instance<8, D, GQ, X>(p, smem_bytes, stream, prepare);
    default: return cudaErrorInvalidValue;
  }
}

// The kernel is instantiated in two translation units (compiled side by side): the plain
// one serves unsharded dense plans and carries none of the code below; the extended one
// (TMB_EXTENDED) adds tensor parallelism, mixture of experts and the QK norm, for
// head_dim 128; a third one (TMB_DENSE) holds the dense-batch kernel.
#if (TMB_EXTENDED || TMB_FP8) && !TMB_DENSE
template <int B, int GQ, int X>
static cudaError_t run_ranks_instance(const MegaParams* ranks_dev, int count, int total_grid, size_t smem_bytes,
                                      cudaStream_t stream) {
  auto kernel = decode_megakernel_ranks<B, 128, GQ, X>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));
  if (err != cudaSuccess) return err;
  void* args[] = {static_cast<void*>(&ranks_dev), static_cast<void*>(&count)};
  // cooperative: the launch fails unless every CTA of every rank is resident at once
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(unsigned(total_grid)), dim3(kThreads), args,
                                     smem_bytes, stream);
}

// `first` is the host copy of ranks_dev[0]: all ranks of a job share one plan geometry.
template <int X>
static cudaError_t run_ranks(const MegaParams& first, const MegaParams* ranks_dev, int count, int total_grid, cudaStream_t stream) {
  const size_t smem_bytes = size_t(ring_offset(first.xs_bytes, first.batch) + first.nslots * kSlotBytes);
  if (first.kv_heads <= 0 || first.heads % first.kv_heads || first.head_dim != 128 || first.experts > 0 || first.qk_norm)
    return cudaErrorInvalidValue;
  const int gq = first.heads / first.kv_heads;
  if (gq != 4 && gq != 8) return cudaErrorInvalidValue;
  switch (first.batch) {
    case 1: return gq == 8 ? run_ranks_instance<1, 8, X>(ranks_dev, count, total_grid, smem_bytes, stream)
                           : run_ranks_instance<1, 4, X>(ranks_dev, count, total_grid, smem_bytes, stream);
    case 2: return gq == 8 ? run_ranks_instance<2, 8, X>(ranks_dev, count, total_grid, smem_bytes, stream)
                           : run_ranks_instance<2, 4, X>(ranks_dev, count, total_grid, smem_bytes, stream);
    case 3: return gq == 8 ? run_ranks_instance<3, 8, X>(ranks_dev, count, total_grid, smem_bytes, stream)
                           : run_ranks_instance<3, 4, X>(ranks_dev, count, total_grid, smem_bytes, stream);
    case 4: return gq == 8 ? run_ranks_instance<4, 8, X>(ranks_dev, count, total_grid, smem_bytes, stream)
                           : run_ranks_instance<4, 4, X>(ranks_dev, count, total_grid, smem_bytes, stream);
    default: return cudaErrorInvalidValue;   // the one-device form is built for batch 1..4
  }
}
#endif

#if TMB_DENSE
#elif TMB_FP8
cudaError_t run_decode_fp8(const MegaParams& p, cudaStream_t stream, bool prepare) {
  const size_t smem_bytes = size_t(ring_offset(p.xs_bytes, p.batch) + p.nslots * kSlotBytes);
  if (p.kv_heads <= 0 || p.heads % p.kv_heads || p.head_dim != 128 || p.experts > 0 || p.qk_norm) return cudaErrorInvalidValue;
  const int gq = p.heads / p.kv_heads;
  if (gq == 8) return run_batch<128, 8, kXFp8 | kXTp>(p, smem_bytes, stream, prepare);
  if (gq == 4) return run_batch<128, 4, kXFp8 | kXTp>(p, smem_bytes, stream, prepare);
  return cudaErrorInvalidValue;
}

cudaError_t run_decode_ranks_fp8(const MegaParams& first, const MegaParams* ranks_dev, int count, int total_grid,
                                 cudaStream_t stream) {
  return run_ranks<kXFp8 | kXTp>(first, ranks_dev, count, total_grid, stream);
}
#elif TMB_EXTENDED
cudaError_t run_decode_extended(const MegaParams& p, cudaStream_t stream, bool prepare) {
  const size_t smem_bytes = size_t(ring_offset(p.xs_bytes, p.batch) + p.nslots * kSlotBytes);
  if (p.kv_heads <= 0 || p.heads % p.kv_heads || p.head_dim != 128) return cudaErrorInvalidValue;
  const int gq = p.heads / p.kv_heads;
  if (gq != 4 && gq != 8) return cudaErrorInvalidValue;
  if (p.experts > 0 || p.qk_norm) {
    if (p.tp_world > 1) return cudaErrorInvalidValue;
    return gq == 8 ? run_batch<128, 8, kXMoe>(p, smem_bytes, stream, prepare)
                   : run_batch<128, 4, kXMoe>(p, smem_bytes, stream, prepare);
  }
  return gq == 8 ? run_batch<128, 8, kXTp>(p, smem_bytes, stream, prepare)
                 : run_batch<128, 4, kXTp>(p, smem_bytes, stream, prepare);
}

cudaError_t run_decode_ranks(const MegaParams& first, const MegaParams* ranks_dev, int count, int total_grid,
                             cudaStream_t stream) {
  return run_ranks<kXTp>(first, ranks_dev, count, total_grid, stream);
}
#else
cudaError_t run_decode_extended(const MegaParams& p, cudaStream_t stream, bool prepare);
cudaError_t run_decode_dense(const MegaParams& p, cudaStream_t stream, bool prepare);
cudaError_t run_decode_fp8(const MegaParams& p, cudaStream_t stream, bool prepare);
cudaError_t run_decode_ranks(const MegaParams& first, const MegaParams* ranks_dev, int count, int total_grid,
                             cudaStream_t stream);
cudaError_t run_decode_ranks_fp8(const MegaParams& first, const MegaParams* ranks_dev, int count, int total_grid,
                                 cudaStream_t stream);

static cudaError_t run_decode(const MegaParams& p, cudaStream_t stream, bool prepare) {
  if (p.dense) return run_decode_dense(p, stream, prepare);
  if (p.fp8) return run_decode_fp8(p, stream, prepare);
  if (p.tp_world > 1 || p.experts > 0 || p.qk_norm) return run_decode_extended(p, stream, prepare);
  const size_t smem_bytes = size_t(ring_offset(p.xs_bytes, p.batch) + p.nslots * kSlotBytes);
  if (p.kv_heads <= 0 || p.heads % p.kv_heads) return cudaErrorInvalidValue;
  const int gq = p.heads / p.kv_heads;
  if (p.head_dim == 128 && gq == 8) return run_batch<128, 8, 0>(p, smem_bytes, stream, prepare);
  if (gq != 4) return cudaErrorInvalidValue;
  if (p.head_dim == 128) return run_batch<128, 4, 0>(p, smem_bytes, stream, prepare);
  if (p.head_dim == 64) return run_batch<64, 4, 0>(p, smem_bytes, stream, prepare);
  return cudaErrorInvalidValue;
}
#endif

}  // namespace tmb

#if !TMB_EXTENDED && !TMB_DENSE && !TMB_FP8
extern "C" int tmb_smem_bytes(const tmb::MegaParams* p) {
  return tmb::ring_offset(p->xs_bytes, p->batch) + p->nslots * tmb::kSlotBytes;
}

// Once per plan: opt in to the dynamic shared memory and prove that the whole
// grid is co-resident (the kernel's grid barrier depends on it).
extern "C" int tmb_prepare_decode(const tmb::MegaParams* p) { return int(tmb::run_decode(*p, nullptr, true)); }

extern "C" int tmb_launch_decode(const tmb::MegaParams* p, void* stream) {
  return int(tmb::run_decode(*p, static_cast<cudaStream_t>(stream), false));
}

extern "C" int tmb_launch_decode_ranks(const tmb::MegaParams* first, const tmb::MegaParams* ranks_dev, int count,
                                       int total_grid, void* stream) {
  return int(first->fp8 ? tmb::run_decode_ranks_fp8(*first, ranks_dev, count, total_grid, static_cast<cudaStream_t>(stream))
                        : tmb::run_decode_ranks(*first, ranks_dev, count, total_grid, static_cast<cudaStream_t>(stream)));
}

extern "C" int tmb_launch_watchdog_probe(const tmb::MegaParams* p, int withhold, void* stream) {
  tmb::watchdog_probe_kernel<<<2, 32, 0, static_cast<cudaStream_t>(stream)>>>(*p, withhold);
  return int(cudaGetLastError());
}
#endif
