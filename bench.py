"""Decode benchmark: tokens/s and step latency of the persistent decode kernel on a
Llama-3.1-8B-shaped model (bf16, batch 1, paged KV with a shuffled block table),
with the HBM roofline of the kernel and the CPU forward timed beside it.

    python bench.py --gpus 1 --steps K --warmup W          # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W  # the reference's CPU forward

One "step" is one decode step of every sequence in the batch. The timed region is
ONE persistent launch that runs K steps; inputs (weights, KV pool, block table,
token state) are resident in HBM when it starts. `e2e` drives the same plan one
step per call through the C ABI with the token id coming from pinned host memory
and the new token read back to the host every step.

Synthetic data: seeded N(0, 0.02) weights, KV rows N(0, 0.5), a seeded context
length in [512, 8192]. Rank r > 0 of a multi-GPU run is an independent replica of
the headline workload (the 8B-shaped model at batch 1 is not tensor parallel in the
benchmark list); the job value is the sum over replicas.

    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --tp --model llama-3.1-70b

shards ONE model over the N ranks instead (tensor parallelism: column/row-sharded
weights, the all-reduce after o and down fused into the kernel's epilogues over
peer memory); the job value is then the one model's tokens/s ("strong" scaling) and
the roofline is each GPU's share of the bytes.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from tilemega_b200 import synthetic  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tok/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum per algorithmic byte of a launch, from the ncu
# capture of the same kernel on a 2-layer case of the same shapes (15.473 GB of DRAM traffic
# for 15.559 GB of algorithmic bytes; profiles/decode_megakernel_llama31_8b_b1.md). Traffic
# is proportional to the streamed weights, so the full launch's traffic is this ratio times
# its algorithmic bytes.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 0.9945


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


MODELS = {"llama-3.1-8b": synthetic.LLAMA_3_1_8B, "llama-3.2-1b": synthetic.LLAMA_3_2_1B,
          "llama-3.1-70b": synthetic.LLAMA_3_1_70B, "qwen3-30b-a3b": synthetic.QWEN3_30B_A3B}


def workload(args) -> dict:
    config = dict(MODELS[args.model])
    if args.layers:
        config["num_hidden_layers"] = args.layers
    batch = args.batch
    contexts = synthetic.seeded_contexts(batch, 512, 8192, seed=2).tolist() if args.context == 0 else [args.context] * batch
    return {"name": f"{args.model}-shaped", "config": config, "batch": batch, "contexts": contexts}


class ClockSampler:
    """Reads SM clocks and throttle reasons through NVML while the timed regions run."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples: list[tuple[int, int]] = []
        self.max_mhz = None
        self.stop = threading.Event()
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # NVML absent: report no clocks rather than fail the bench
            self.nvml = None

    def _run(self):
        nvml = self.nvml
        while not self.stop.is_set():
            try:
                mhz = int(nvml.nvmlDeviceGetClockInfo(self.handle, nvml.NVML_CLOCK_SM))
                reasons = int(nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *_):
        self.stop.set()
        if self.thread is not None:
            self.thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        seen = 0
        for _, reasons in self.samples:
            seen |= reasons
        names = [name for bit, name in self.REASONS.items() if seen & bit]
        return {"sm_mhz": int(statistics.median(mhz for mhz, _ in self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": names, "samples": len(self.samples)}


def cpu_forward_seconds_per_step(work: dict, steps: int, threads: int) -> tuple[float, str]:
    """The reference's CPU forward (the oracle port) on a bounded sample of the
    workload: 1-layer and 2-layer slices of the same shapes at the same context,
    fp32, timed per decode step; the full depth is layer_time * L + head_time."""
    from oracle.decoder_oracle import OracleDecoder, PagedKV
    torch.set_num_threads(threads)
    config, batch, contexts = work["config"], work["batch"], work["contexts"]
    layers = config["num_hidden_layers"]
    capacity = (max(contexts) + steps + 17) // 16 * 16
    two = dict(config, num_hidden_layers=min(2, layers))
    weights = synthetic.seeded_weights(two, seed=0, dtype=torch.float32)
    times = {}
    for depth in sorted({1, min(2, layers)}):
        sliced = dict(config, num_hidden_layers=depth)
        decoder = OracleDecoder(sliced, weights, torch.float32, capacity)
        kv = PagedKV(sliced, batch, capacity, torch.float32)
        kv.pool.normal_(0.0, 0.5, generator=torch.Generator().manual_seed(3))
        ids = synthetic.seeded_tokens(batch, steps + 1, config["vocab_size"], seed=4)
        decoder.forward(ids[:, :1], list(contexts), kv)  # warm-up
        begin = time.perf_counter()
        for step in range(steps):
            decoder.forward(ids[:, step + 1:step + 2], [c + step + 1 for c in contexts], kv)
        times[depth] = (time.perf_counter() - begin) / steps
    if layers >= 2:
        layer_time = max(times[2] - times[1], 1e-9)
        head_time = max(times[1] - layer_time, 0.0)
    else:
        layer_time, head_time = times[1], 0.0
    seconds = layer_time * layers + head_time
    sample = (f"fp32 oracle port, 1- and 2-layer slices + lm_head of the same shapes at context {contexts}, "
              f"{steps} decode steps each, extrapolated linearly to {layers} layers")
    return seconds, sample


def max_over_ranks(values: list[float], device=None) -> list[float]:
    """Element-wise maximum of `values` over the ranks of the default process group
    (identity without one): every reported time is the slowest rank's."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    buffer = torch.tensor(values, dtype=torch.float64, device=device)
    dist.all_reduce(buffer, op=dist.ReduceOp.MAX)
    return [float(v) for v in buffer]


def job_value(world: int, batch: int, steps: int, seconds: float) -> float:
    """Whole-job tokens per second: every replica decodes batch*steps tokens in the slowest rank's time."""
    return world * batch * steps / seconds


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    work = workload(args)
    threads = os.cpu_count() or 1
    steps = max(1, min(args.steps, 4))
    seconds, sample = cpu_forward_seconds_per_step(work, steps, threads)
    value = work["batch"] / seconds
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{work['name']} decode, batch {work['batch']}, context {work['contexts']}, "
                               "reference PyTorch CPU forward (restated in oracle/)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU implementation")
    from tilemega_b200.planbuild import emit_plan
    from tilemega_b200.serving.plan import PlanLibrary
    from tilemega_b200.serving.state import allocate_state, shuffled_block_table
    from tilemega_b200.serving.weights import TensorCheckpoint, load_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    tp = world if args.tp else 1
    if args.tp and world < 2:
        raise SystemExit("--tp shards one model over the ranks: launch at least two")

    work = workload(args)
    config, batch, contexts = work["config"], work["batch"], work["contexts"]
    steps, warmup = args.steps, max(args.warmup, 3)
    total_steps = warmup + 2 * steps + 1 + 4   # device-timed launch, the end-to-end loop, and the optional traced steps
    capacity = (max(contexts) + total_steps + 17) // 16 * 16
    max_blocks = capacity // 16
    num_blocks = batch * max_blocks + 32
    plan_dir = Path(os.environ.get("TILEMEGA_PLAN_DIR", "/tmp/tilemega_b200_plans"))
    geometry = json.loads(args.geometry) if args.geometry else None
    options = dict(batch_lo=batch, batch_hi=batch, capacity=capacity, kv_layout="paged", num_blocks=num_blocks,
                   write_logits=False, geometry=geometry, slots=args.slots, tp=tp)
    if rank == 0 or world == 1:
        so = emit_plan(config, plan_dir, **options)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        so = emit_plan(config, plan_dir, **options)
    lib = PlanLibrary(so)
    replica = 0 if tp > 1 else rank     # tensor-parallel ranks cut their slices out of ONE model and share one request
    if tp > 1 or synthetic.is_moe(config):
        # models too large to hold unpacked: every tensor is drawn on the device when its recipe asks for it
        weights = load_weights(synthetic.LazySeededCheckpoint(config, seed=replica, device=device), lib, device=device,
                               tp=(rank, world) if tp > 1 else (0, 1))
    else:
        raw = synthetic.seeded_weights(config, seed=rank, dtype=torch.bfloat16, device=device)
        weights = load_weights(TensorCheckpoint(raw, config["tie_word_embeddings"]), lib, device=device)
        keep = {tensor.data_ptr() for tensor in weights.values()}
        raw = {name: tensor for name, tensor in raw.items() if tensor.data_ptr() in keep}
    torch.cuda.empty_cache()
    table = shuffled_block_table(batch, max_blocks, num_blocks, seed=7 + replica)
    base = torch.tensor(contexts, dtype=torch.int32)
    state = allocate_state(config, batch, lib, device, block_table=table, context_base=base, tp=tp)
    state.kv_storage.normal_(0.0, 0.5)
    first = synthetic.seeded_tokens(batch, 1, config["vocab_size"], seed=11 + replica)
    for b in range(batch):
        state.tokens[b, contexts[b]] = int(first[b, 0])
    pointers = {name: tensor.data_ptr() for name, tensor in weights.items()}
    pointers.update(state.pointers)
    plan = lib.create(batch, pointers, local)
    if tp > 1:
        # each rank's receive regions, published to its peers as CUDA IPC handles
        from tilemega_b200.serving.tp_engine import exchange_handles
        regions = [lib.ipc_alloc(local, lib.tp_bytes(which)) for which in (0, 1)]
        plan.bind_tp(rank, exchange_handles(lib, regions[0]), exchange_handles(lib, regions[1]))
        torch.cuda.synchronize()
        dist.barrier()
    plan.set_prompt_len(0)
    plan.set_steps(list(range(total_steps)))   # step s decodes position context_base[b] + s
    stream = torch.cuda.current_stream()
    mode = 1 if tp > 1 else 2

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    bytes_timed = sum(plan.step_bytes(sum(c + warmup + i + 1 for c in contexts)) for i in range(steps))
    sampler = ClockSampler(local)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        plan.launch_steps(0, warmup, mode, stream.cuda_stream)
        barrier()
        begin.record(stream)
        plan.launch_steps(warmup, steps, mode, stream.cuda_stream)
        end.record(stream)
        barrier()
        device_ms = begin.elapsed_time(end)
        fired = plan.watchdog()
        if fired is not None:
            raise SystemExit(f"a bounded device wait gave up during the timed launch: {fired}")
        stamps = plan.read_step_ns(warmup, steps + 1)
        # end to end: one step per ABI call, token id from pinned host memory, new token back to the host
        host_in = torch.empty(batch, dtype=torch.int32).pin_memory()
        host_out = torch.empty(batch, dtype=torch.int32).pin_memory()
        position = [c + warmup + steps for c in contexts]
        for b in range(batch):
            host_in[b] = int(state.tokens[b, position[b]])
        barrier()
        wall = time.perf_counter()
        for i in range(steps):
            for b in range(batch):
                state.tokens[b, position[b] + i:position[b] + i + 1].copy_(host_in[b:b + 1], non_blocking=True)
            plan.launch(warmup + steps + i, mode, stream.cuda_stream)
            for b in range(batch):
                host_out[b:b + 1].copy_(state.tokens[b, position[b] + i + 1:position[b] + i + 2], non_blocking=True)
            stream.synchronize()
            host_in.copy_(host_out)
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - wall
        barrier()
    fired = plan.watchdog()
    if fired is not None:
        raise SystemExit(f"a bounded device wait gave up during the end-to-end loop: {fired}")
    if args.trace:
        # per-stage stamps of one more step (every rank of a tensor-parallel job runs it; rank 0 reports)
        import numpy as np
        from tilemega_b200.stage_trace import print_table
        plan.trace_step(warmup + 2 * steps + 2)
        plan.launch_steps(warmup + 2 * steps, 4, mode, stream.cuda_stream)
        barrier()
        stamps = np.array(plan.read_trace(), dtype=np.int64)
        grid = torch.cuda.get_device_properties(local).multi_processor_count
        per_layer = (stamps.size // 4 // grid - 1) // config["num_hidden_layers"]
        if rank == 0:
            print_table(config, stamps.reshape(grid, -1, 4), per_layer, max(contexts) + warmup + 2 * steps, batch, tp=tp)
    device_ms, e2e_seconds = max_over_ranks([device_ms, e2e_seconds], device)
    seconds = device_ms / 1e3
    replicas = 1 if tp > 1 else world
    value = job_value(replicas, batch, steps, seconds)
    achieved = bytes_timed / seconds / 1e9
    peak, peak_kind = measured_peak_gbs()
    step_us = [(stamps[i + 1] - stamps[i]) / 1e3 for i in range(steps)]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": device_ms / steps, "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak",
        "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{work['name']} decode, batch {batch}, context {contexts}, paged KV block 16, "
                               "shuffled block table", "layers": config["num_hidden_layers"],
                   "l2": "inputs larger than L2: every step streams its weights and KV rows from HBM",
                   "parallelism": f"tp{tp}" if tp > 1 else ("replicas" if world > 1 else "single"),
                   "step_latency_us_median": statistics.median(step_us),
                   "mbu_vs_nominal_8tbs": achieved / NOMINAL_HBM_GBS},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None if tp > 1 else NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_timed,
                     "traffic_source": ("not captured for the tensor-parallel run (ncu never wraps a multi-rank command)"
                                        if tp > 1 else
                                        "ncu on a 2-layer case of the same kernel, scaled by algorithmic bytes"),
                     "per": "GPU (this rank's share of the weights and KV rows)" if tp > 1 else "GPU",
                     "peak_kind": f"of {peak_kind}", "bytes_per_launch": bytes_timed},
        "e2e": {"value": job_value(replicas, batch, steps, e2e_seconds), "unit": UNIT, "h2d_bytes_per_step": 4 * batch,
                "d2h_bytes_per_step": 4 * batch},
        "gpu_launches": 1,
        "clocks": sampler.summary(),
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        seconds_cpu, sample = cpu_forward_seconds_per_step(work, 3, threads)
        line["cpu_baseline"] = {"value": batch / seconds_cpu, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": sample}
    plan.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--model", choices=sorted(MODELS), default="llama-3.1-8b",
                        help="shape of the synthetic model (the headline workload is llama-3.1-8b, batch 1)")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--context", type=int, default=0, help="0: seeded draw in [512, 8192]")
    parser.add_argument("--layers", type=int, default=0, help="override the depth (profiling a small case)")
    parser.add_argument("--geometry", default="", help="JSON overrides of the GEMV page geometry")
    parser.add_argument("--slots", type=int, default=0)
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--trace", action="store_true",
                        help="after the timed runs, stamp one more step and print the per-stage table (rank 0)")
    parser.add_argument("--tp", action="store_true",
                        help="shard one model over the ranks (tensor parallelism) instead of running replicas")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
