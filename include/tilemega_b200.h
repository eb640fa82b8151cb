/* C ABI of libtilemega_b200.so: the serving-plan interface of TileMega
 * (include/tilemega/Codegen/tasks/ServingAbi.h, version 1) implemented by a
 * hand-written sm_100a persistent decode kernel.
 *
 * A TileMega plan library is one compiled model: tm_plan_query takes no
 * argument. This library reads its model from the JSON sidecar
 * "<path of this .so>.plan.json" (or the file named by TILEMEGA_PLAN_JSON), so
 * one copy of the .so next to one sidecar is one plan library, loadable by the
 * reference's python/tilemega/serving/plan.py:PlanLibrary unchanged.
 *
 * Conventions (ServingAbi.h:33-55; ServingRuntime.cuh:943-977): 0 = OK,
 * -1 bad argument, -2 iteration / step-interval mismatch, -3 mode unavailable,
 * -4 plan abandoned by its watchdog; CUDA error codes are passed through as
 * positive integers. No exception crosses the boundary. The caller owns every
 * external buffer; the plan owns and frees its internal ones. Launches are
 * asynchronous on the caller's stream; synchronise before any tm_plan_read_*.
 * One host thread per plan.
 */
#ifndef TILEMEGA_B200_H_
#define TILEMEGA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ServingAbi.h:11-15 */
enum { TM_SERVING_ABI_VERSION = 1 };
enum { TM_SERVING_PREFILL = 0, TM_SERVING_DECODE = 1, TM_SERVING_FORWARD = 2 };
enum { TM_SERVING_L1 = 1, TM_SERVING_L2 = 2 };
enum { TM_BUFFER_INTERNAL = 0, TM_BUFFER_EXTERNAL = 1 };
enum { TM_DTYPE_BF16 = 0, TM_DTYPE_F32 = 1, TM_DTYPE_I32 = 2,
       /* the reference's forward runtime adds this code for token ids
        * (include/tilemega/Codegen/tasks/Sm90F3Runtime.cuh:20-22) */
       TM_DTYPE_I64 = 3,
       /* addition: fp16 elements, in the buffers of a forward plan whose sidecar says "dtype": "f16" */
       TM_DTYPE_F16 = 5,
       /* addition (the reference has no 8-bit weights): e4m3 bytes, one element per byte, in the
        * weight buffers of a plan whose sidecar says "weights": "e4m3"; each such buffer comes with an
        * fp32 buffer "<name>.scale" of one scale per output row */
       TM_DTYPE_E4M3 = 4 };

/* ServingAbi.h:17-23. All three phases are built. TM_SERVING_FORWARD (a stateless encoder pass; the reference's
 * forward runtime behind the same entry points is include/tilemega/Codegen/tasks/Sm90F3Runtime.cuh:95-200): seq =
 * the positions per sequence (128), capacity 0, ONE plan step at past 0; external buffers are the module's
 * parameters under their qualified names, "input_ids" and "token_type_ids" (TM_DTYPE_I64, [batch][seq]; with
 * "mask": true in the sidecar also "attention_mask", 0 = hidden key position) and the
 * outputs "last_hidden_state" ([batch][seq][hidden]) and "pooler_output" ([batch][hidden]); tm_plan_set_prompt_len,
 * the tracing, probe and tensor-parallel entry points refuse such a plan. TM_SERVING_DECODE: seq = 1, one sequence position per plan step
 * (past_lo..past_hi = 0..capacity-1). TM_SERVING_PREFILL: seq = the prompt length the plan was emitted for,
 * ONE plan step (past 0) that runs positions 0..seq-1 of all `batch` sequences over the same request buffers
 * a decode plan of the same model, capacity and KV layout names (tokens, RoPE tables, KV caches or pools,
 * block table) and writes the token sampled after the prompt to serving.tokens[b][seq]; its GEMM weight
 * buffers are named "prefill.<decode name>" (128 x 128 pages), so one driver-side table can hold both plans'
 * buffers (python/tilemega/serving/engine.py:49-57). */
typedef struct {
  uint32_t abi_version, phase;
  int32_t batch_lo, batch_hi, seq, past_lo, past_hi, capacity;
  int32_t grid, residency;
  uint32_t modes;
  uint32_t buffer_count;
} tm_plan_info;

/* ServingAbi.h:25-31 */
typedef struct {
  const char* name;
  uint32_t role;
  uint32_t dtype;
  uint64_t elements_constant, elements_per_batch;
  const char* pack_json;
} tm_buffer_info;

/* ---- required entry points ------------------------------------------- */

/* ServingAbi.h:33. Static description of the plan; no GPU needed. */
int tm_plan_query(tm_plan_info* out);
/* ServingAbi.h:34. Buffer table entry `index`; strings live as long as the library. */
int tm_plan_buffer(uint32_t index, tm_buffer_info* out);
/* ServingAbi.h:35. external[i] = device pointer of every TM_BUFFER_EXTERNAL
 * entry in table order, NULL for internal ones. NULL on any rejection. */
void* tm_plan_create(int batch, void* const* external, int device);
/* ServingAbi.h:36. past[s] = position decoded by step s. */
int tm_plan_set_steps(void* plan, const int32_t* past, uint32_t count);
/* ServingAbi.h:37-40. iteration = launches of this mode so far, gap-free. */
int tm_plan_launch(void* plan, uint32_t step, uint32_t mode, uint64_t iteration, void* stream);
/* ServingAbi.h:48. */
void tm_plan_destroy(void* plan);

/* ---- optional entry points the reference driver probes by name -------- */

/* ServingAbi.h:41-42. One persistent launch for steps [first, first+steps). */
int tm_plan_launch_steps(void* plan, uint32_t first_step, uint32_t steps, uint32_t mode,
                         uint64_t base_iteration, void* stream);
/* ServingAbi.h:43. Bit mask of modes that support tm_plan_launch_steps. */
unsigned tm_plan_loop_modes(void* plan);
/* ServingAbi.h:44-45. %globaltimer stamps: host[i] = start of step first+i
 * (= end of step first+i-1); count+1 stamps exist for count steps. */
int tm_plan_read_step_ns(void* plan, uint32_t first, uint32_t count, uint64_t* host);
/* ServingAbi.h:46-47. Copy table entry `index` to the host. */
int tm_plan_read_buffer(void* plan, uint32_t index, void* host, uint64_t bytes);
/* include/tilemega/Codegen/tasks/ServingRuntime.cuh:1065-1075. Returns 1 and
 * fills the 12-word record {fired, site, block, thread, waiter_stage,
 * waiter_task, producer_stage, group, row, need, value, iteration} when a
 * bounded device wait gave up; the kernel returns normally in that case. */
int tm_plan_watchdog(void* plan, uint64_t* record12);
/* python/tilemega/serving/plan.py:152-159. Positions below prompt_len keep the
 * token state the caller wrote (teacher forcing through the decode plan). */
int tm_plan_set_prompt_len(void* plan, int prompt_len);
/* plan.py:75-77; this plan never uses programmatic dependent launch. */
unsigned tm_plan_pdl_enabled(void* plan);
/* plan.py:76. Dynamic shared memory of the persistent kernel. */
uint64_t tm_plan_execution_smem(void* plan, unsigned mode);
/* ServingAbi.h:49-55. Tensor-parallel extension. A plan whose sidecar says "tp": T is
 * ONE RANK's plan (Megatron sharding: q/k/v, gate/up and lm_head by rows, o and down by
 * columns; the weight recipes carry "shard" so each rank packs its slice). tp_world()
 * returns T; tp_bytes(0) is the size of a rank's all-reduce receive region, tp_bytes(1)
 * of its argmax exchange block; the caller allocates both ZEROED on each rank's device
 * and gives bind_tp, on every rank, the T region pointers and T block pointers as they
 * are valid in the calling process (the rank's own, and its peers' through peer access
 * or CUDA IPC). bind_tp must precede the first launch; all ranks must then launch the
 * same steps. Inside the kernel the all-reduce after o and after down is fused into the
 * GEMV epilogue: packets of {two bf16 sums, epoch} are stored into the peers' regions
 * and summed in rank order (Sm90DenseEpilogue.h:43-86); lm_head winners are exchanged
 * the same way (Sm90DenseHead.cuh:139-201). */
unsigned tm_plan_tp_world(void);
unsigned long long tm_plan_tp_bytes(unsigned which);
int tm_plan_bind_tp(void* plan, int rank, void* const* ar, void* const* x);

/* ---- additions of this library (probed by name; absent in the reference) */

/* One process per GPU: allocate a zeroed region that is an allocation of its own, export
 * it as a 64-byte CUDA IPC handle, map a peer's handle, unmap it. The reference drives all ranks from one process
 * (python/tilemega/serving/tp_engine.py:47-112) and needs none of these. */
int tm_ipc_alloc(int device, uint64_t bytes, void** device_pointer);   /* zeroed, its own allocation */
int tm_ipc_free(void* device_pointer);
int tm_ipc_export(void* device_pointer, unsigned char* handle64);
int tm_ipc_open(const unsigned char* handle64, void** device_pointer);
int tm_ipc_close(void* device_pointer);

/* Several ranks of one tensor-parallel job on ONE device, as one cooperative launch:
 * plans[q] is rank q's plan (all created from this library on the same device, all bound
 * with tm_plan_bind_tp to regions in that device's memory), emitted with a "grid" small
 * enough that the ranks' grids together fit the device's SMs. Same step and iteration
 * rules as tm_plan_launch_steps, applied to every plan. The reference's driver launches
 * each rank's plan on its own GPU in turn (python/tilemega/serving/tp_engine.py:113-131);
 * ranks wait for one another's packets, and on one GPU only a single launch guarantees
 * that they run at the same time, so a box with fewer GPUs than ranks (and the one-GPU
 * test of the exchange code) goes through this entry point. Batch 1..4. */
int tm_plan_launch_steps_ranks(void* const* plans, uint32_t count, uint32_t first_step, uint32_t steps,
                               uint32_t mode, uint64_t base_iteration, void* stream);

/* Last error text of the calling thread's most recent failing call. */
const char* tm_plan_last_error(void);
/* Clear a fired watchdog so the plan can launch again (counters are rezeroed
 * by every launch). Once tm_plan_watchdog (or the probe) has reported a fired
 * wait, every launch on the plan answers -4 until this is called: the kernel's
 * other waits fall through while the record stands, so its results would be
 * garbage. Read tm_plan_watchdog after synchronising a launch. */
int tm_plan_clear_watchdog(void* plan);
/* Bounded-wait self test: a two-CTA kernel whose producer withholds its arrival
 * when `withhold` != 0; the waiter gives up after limit_us and the kernel
 * returns normally. Returns 1 if the wait gave up, 0 if it was satisfied, and
 * leaves the plan clean; `withhold` == 2 withholds too but leaves the record
 * standing, which is the state after a real abandoned launch (launches answer
 * -4 until tm_plan_clear_watchdog). */
int tm_plan_watchdog_probe(void* plan, int withhold, uint32_t limit_us, void* stream);
/* Stage trace of one step (the reference's TILEMEGA_TRACE_STAGE build,
 * include/tilemega/Codegen/tasks/ModelRuntime.h:758-766, as a run-time switch):
 * step >= 0 records, for every CTA and stage of that step, four %globaltimer
 * stamps {wait begin, inputs ready, rows staged, tasks done}; step < 0 turns it
 * off. tm_plan_read_trace(plan, NULL, 0) returns the byte size, otherwise copies
 * u64 [grid][5*layers+1][4]. A traced launch is for diagnosis, not for timing. */
int tm_plan_trace_step(void* plan, int step);
long long tm_plan_read_trace(void* plan, uint64_t* host, uint64_t bytes);
/* Algorithmic HBM bytes of one decode step: GEMV weights incl. lm_head plus
 * 4*L*Hkv*D bytes per cached token (scripts/estimate_r16_mbu.py:15-38). */
uint64_t tm_plan_step_bytes(void* plan, uint64_t cached_tokens_total);

/* The reference's `tile_pages` packing recipe (python/tilemega/serving/weights.py:204-242,
 * which runs as PyTorch indexing ops) as one kernel on the device: `src` is a row-major
 * bf16 matrix [rows][cols] whose rows are src_pitch elements apart, `dst` receives
 * ceil(rows/tile_n) * ceil(cols/tile_k) pages of tile_n*tile_k elements, zero where the
 * matrix ends. Both on the current device, 16-byte aligned; cols and src_pitch multiples
 * of 8. Asynchronous on `stream`. 0, -1 (bad argument) or a CUDA error code. */
int tm_pack_tile_pages(const void* src, uint64_t rows, uint64_t cols, uint64_t src_pitch, uint32_t tile_n,
                       uint32_t tile_k, void* dst, void* stream);

/* Microbenchmarks behind configs/targets/sm_100.json: the reference fills the "calibration"
 * block of its target descriptions with lib/Target/Calibration.cu and its siblings; this runs
 * the named benchmark on `device` and writes its numbers to out[0..capacity). `what`: "clock"
 * (SM MHz under load), "pipes" (fp32 / int32 / ex2 / rsqrt G(fl)op/s), "tensor" (mma.sync fp16,
 * bf16 GFLOP/s), "smem" (GB/s at 1, 2, 4, 8 CTAs per SM, then the bank-conflict slope),
 * "latency" (L1, L2, DRAM ns per dependent load), "l2_curve" (pairs footprint bytes, GB/s),
 * "dram" (copy GB/s), "sync" (atomic, __threadfence, __syncthreads, named barrier, cluster
 * barrier ns), "atomic_contention" and "grid_barrier" (pairs CTAs, ns). Returns the count of
 * numbers written or a negative status. Allocates and frees its own buffers; changes no
 * device setting. */
int tm_calibrate(int device, const char* what, double* out, int capacity);

/* No counterpart in the reference. The bounded-wait self test of
 * tm_plan_watchdog_probe for callers that may not allocate device memory: a
 * process whose HBM is fully committed to weight and KV pools, a health check
 * between decode launches that cannot afford cudaMalloc's device-wide
 * synchronisation, code under a framework-enforced memory budget. It needs no
 * plan and calls no allocator: its scratch (the arrival word and one record per
 * waiter) is a fixed 4.4 KB device array inside the library, present on every GPU
 * that loads it until the process exits. One producer CTA and `waiters` waiting
 * CTAs (1..TM_STATIC_PROBE_MAX_WAITERS; more is rejected with -1 and a message)
 * run in one launch on `stream`; with `withhold` != 0 the producer never arrives
 * and every waiter gives up after limit_us (1..1000000). Each waiter writes its
 * 12-word record (layout of tm_plan_watchdog; word 0 = 1 if it gave up) to
 * records_device[waiter*12 ...], a device buffer of waiters*12 u64 that the
 * caller owns; read it after synchronising the stream. Returns 0 or a CUDA error
 * code. The first call on a device resolves the scratch array's address; make
 * that call before any stream capture begins. All calls share the one array
 * (cleared on `stream` at the start of each call), so two calls whose kernels
 * could overlap on the GPU -- different streams, no ordering -- would race: run
 * them one after another. */
enum { TM_STATIC_PROBE_MAX_WAITERS = 32 };
int tm_watchdog_probe_static(int device, int waiters, int withhold, uint32_t limit_us,
                             uint64_t* records_device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TILEMEGA_B200_H_ */
