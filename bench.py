"""Decode benchmark: tokens/s and step latency of the persistent decode kernel, with the
HBM roofline of the kernel and the reference's CPU forward timed beside it.

    python bench.py --gpus 1 --steps K --warmup W          # this repository's CUDA path
    python bench.py --impl reference --steps K --warmup W  # the reference's CPU forward
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

One GPU: a Llama-3.1-8B-shaped model (bf16, batch 1, paged KV with a shuffled block table,
a seeded context length in [512, 8192]). N > 1 GPUs: ONE Llama-3.1-70B-shaped model at context
4096 sharded over the N ranks (tensor parallelism: column/row-sharded weights, the all-reduce
after o and down fused into the kernel's epilogues over peer memory, argmax winners exchanged
the same way); the job value is that one model's tokens/s ("strong" scaling), the roofline is
each GPU's share of the bytes, and every rank's tokens are compared. `--replicas` runs N
independent copies of the one-GPU workload instead.

One "step" is one decode step of every sequence in the batch. The timed region is ONE persistent
launch that runs K steps; inputs (weights, KV pool, block table, token state) are resident in
HBM when it starts. `e2e` drives the same plan one step per call through the C ABI with the
token id coming from pinned host memory and the new token read back to the host every step.

The reference arm and the `cpu_baseline` leg time the reference's own PyTorch module
(`Decoder.execute`, from oracle/_ref/ when oracle/build_ref.py has filled it; otherwise the
restatement in oracle/decoder_oracle.py) in fp32 on all host cores, on slices of 4 and 8 layers
of the workload's shapes at its context length, and extrapolate linearly to the full depth: the
line says so ("extrapolated", the depths, the steps really timed).

Synthetic data: seeded N(0, 0.02) weights, KV rows N(0, 0.5).
"""
from __future__ import annotations

import argparse
import json
import math
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
# dram__bytes_read.sum + dram__bytes_write.sum per algorithmic byte of a launch, from ncu captures
# of the same kernel on 2-layer cases of the same shapes (traffic is proportional to the streamed
# weights, so a full launch's traffic is this ratio times its algorithmic bytes). Keyed by
# (model, batch): a workload without a capture reports no traffic.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {("llama-3.1-8b", 1): 0.9922, ("llama-3.1-8b", 64): 1.0143}
# roofline.frac of the one-GPU headline run (profiles/decode_megakernel_llama31_8b_b1.md): the
# denominator of config.mbu_retained_vs_1gpu in a tensor-parallel line
SINGLE_GPU_FRAC = 0.791
TP_MODEL, TP_CONTEXT = "llama-3.1-70b", 4096


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


MODELS = {"llama-3.1-8b": synthetic.LLAMA_3_1_8B, "llama-3.2-1b": synthetic.LLAMA_3_2_1B,
          "llama-3.1-70b": synthetic.LLAMA_3_1_70B, "qwen3-30b-a3b": synthetic.QWEN3_30B_A3B,
          "bert-base": synthetic.BERT_BASE}   # bert-base: the encoder forward workload (run_forward)


def workload(args) -> dict:
    """What this invocation measures: one GPU (or --replicas) -> the 8B-shaped headline; several
    GPUs -> one 70B-shaped model sharded over them. --model / --context / --batch / --layers override."""
    tp = args.gpus if args.gpus > 1 and not args.replicas else 1
    model = args.model or (TP_MODEL if tp > 1 else "llama-3.1-8b")
    context = args.context if args.context is not None else (TP_CONTEXT if tp > 1 else 0)
    config = dict(MODELS[model])
    if args.layers:
        config["num_hidden_layers"] = args.layers
    batch = args.batch
    contexts = synthetic.seeded_contexts(batch, 512, 8192, seed=2).tolist() if context == 0 else [context] * batch
    label = f"{model}-shaped decode, batch {batch}, context {contexts}, paged KV block 16, shuffled block table"
    if args.weights != "bf16":
        label += f", {args.weights} weights with fp32 row scales"
    if tp > 1:
        label += f", tensor parallel over {tp} GPUs"
    return {"name": f"{model}-shaped", "model": model, "config": config, "batch": batch, "contexts": contexts, "tp": tp,
            "label": label}


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


def cpu_forward(work: dict, steps: int, threads: int, repeats: int = 3) -> dict:
    """Seconds per decode step of the reference's CPU forward, fp32, `threads` host threads.

    With oracle/_ref/ present this drives the reference's own module (`Decoder.execute`,
    python/tilemega/serving/export.py:165-172: token ids, the per-layer caches, the RoPE tables in,
    logits and the grown caches out) -- kind "reference"; otherwise the restatement in
    oracle/decoder_oracle.py -- kind "port". The full model does not fit a bounded sample (the
    8B-shaped weights are 32 GB in fp32), so slices of 4 and 8 layers of the same shapes are timed
    at the workload's context, `steps` decode steps each, `repeats` times (the median counts), and
    the full depth is head + layers * per-layer time."""
    sys.path.insert(0, str(ROOT / "oracle"))
    from build_ref import load_decoder
    torch.set_num_threads(threads)
    config, batch, contexts = work["config"], work["batch"], work["contexts"]
    layers = config["num_hidden_layers"]
    # the deeper slice is the deepest (at most 8 layers) whose fp32 weights stay under 16 GB of host memory
    shapes = dict(synthetic.parameter_shapes(dict(config, num_hidden_layers=1)))
    count = lambda names: sum(math.prod(shapes[name]) for name in names)
    per_layer_bytes = 4 * count(name for name in shapes if name.startswith("model.layers.0."))
    fixed_bytes = 4 * count(name for name in shapes if not name.startswith("model.layers."))
    deepest = max(1, min(8, layers, int((16e9 - fixed_bytes) // per_layer_bytes)))
    depths = sorted({max(1, deepest // 2), deepest})
    Decoder = None if synthetic.is_moe(config) else load_decoder()
    dim = synthetic.head_dim_of(config)
    hkv = config["num_key_value_heads"]
    context = max(contexts)
    timed = {}
    for depth in depths:
        sliced = dict(config, num_hidden_layers=depth)
        ids = synthetic.seeded_tokens(batch, steps + 2, config["vocab_size"], seed=4).long()
        if Decoder is not None:
            with torch.device("meta"):
                model = Decoder(sliced)
            model = model.to_empty(device="cpu").float().eval()
            generator = torch.Generator().manual_seed(0)
            with torch.no_grad():
                for name, parameter in model.named_parameters():
                    if parameter.ndim == 1:
                        parameter.fill_(1.0)
                    else:
                        parameter.normal_(0.0, 0.02, generator=generator)
            from tilemega_b200.serving.state import rotary_tables
            cos, sin = (table.float() for table in rotary_tables(sliced, context + steps + 2, "cpu"))
            kv = torch.Generator().manual_seed(3)
            first = tuple(torch.randn(batch, hkv, context, dim, generator=kv) * 0.5 for _ in range(2 * depth))

            def run_steps(count: int) -> None:
                caches = first
                with torch.inference_mode():
                    for step in range(count):
                        out = model.execute(ids[:, step:step + 1], caches, cos, sin)   # the module picks row `past`
                        caches = out[1:]
        else:
            from oracle.decoder_oracle import OracleDecoder, PagedKV
            weights = synthetic.seeded_weights(sliced, seed=0, dtype=torch.float32)
            capacity = (context + steps + 17) // 16 * 16
            decoder = OracleDecoder(sliced, weights, torch.float32, capacity)
            kv = PagedKV(sliced, batch, capacity, torch.float32)
            kv.pool.normal_(0.0, 0.5, generator=torch.Generator().manual_seed(3))

            def run_steps(count: int) -> None:
                for step in range(count):
                    decoder.forward(ids[:, step:step + 1].int(), [c + step for c in contexts], kv)
        run_steps(1)   # warm-up
        samples = []
        for _ in range(repeats):
            begin = time.perf_counter()
            run_steps(steps)
            samples.append((time.perf_counter() - begin) / steps)
        timed[depth] = statistics.median(samples)
        del run_steps
    if len(depths) == 2:
        per_layer = max((timed[depths[1]] - timed[depths[0]]) / (depths[1] - depths[0]), 1e-9)
        head = max(timed[depths[0]] - per_layer * depths[0], 0.0)
    else:
        per_layer, head = timed[depths[0]] / depths[0], 0.0
    kind = "reference" if Decoder is not None else "port"
    what = ("the reference's Decoder.execute (oracle/_ref)" if Decoder is not None
            else "the restatement of the reference's forward (oracle/decoder_oracle.py)")
    return {"seconds": head + per_layer * layers, "kind": kind, "depths": depths, "steps_timed": steps, "repeats": repeats,
            "extrapolated": layers not in depths,
            "sample": (f"{what}, fp32, {threads} threads: slices of {depths} layers + lm_head of the same shapes at "
                       f"context {context}, {steps} decode steps each, median of {repeats}" +
                       (f", extrapolated linearly to {layers} layers" if layers not in depths else ""))}


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
    steps = max(8, min(args.steps, 16))   # a bounded sample: the line reports what was really timed
    result = cpu_forward(work, steps, threads)
    value = work["batch"] / result["seconds"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": result["steps_timed"], "steps_requested": args.steps, "warmup": 1,
        "ms_per_step": result["seconds"] * 1e3, "higher_is_better": True,
        "scaling": "strong" if work["tp"] > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "extrapolated": result["extrapolated"], "slice_layers": result["depths"],
        "config": {"workload": work["label"], "layers": work["config"]["num_hidden_layers"],
                   "parallelism": "host cores", "arm": "reference PyTorch CPU forward"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": result["kind"], "sample": result["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_forward_reference(args) -> None:
    """Reference arm of the encoder workload: the module the reference exports for it (transformers.BertModel, fp32,
    python/tilemega/dnn/export.py:50-59) on the host cores where that package is importable, else the oracle's
    restatement of it; same metric and configuration as run_forward, a bounded sample of sequences per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle.encoder_oracle import encoder_forward
    config = dict(synthetic.BERT_BASE)
    if args.layers:
        config["num_hidden_layers"] = args.layers
    batch, seq = args.batch, 128
    threads = min(os.cpu_count() or 1, 16)
    torch.set_num_threads(threads)
    weights = synthetic.encoder_weights(config, seed=0)
    sample = min(batch, 8)
    ids, types = synthetic.encoder_inputs(config, sample, seed=1)
    kind, forward = "port", (lambda: encoder_forward(weights, config, ids, types))
    try:
        from transformers import BertConfig, BertModel
        keys = ("hidden_size", "intermediate_size", "num_attention_heads", "num_hidden_layers", "vocab_size",
                "max_position_embeddings", "type_vocab_size", "layer_norm_eps", "hidden_act")
        bert_config = BertConfig(**{key: config[key] for key in keys})
        bert_config._attn_implementation = "sdpa"
        module = BertModel(bert_config).eval()
        module.load_state_dict(weights, strict=False)
        kind = "reference"

        def forward():
            with torch.inference_mode():
                return module(input_ids=ids, token_type_ids=types)
    except ImportError:
        pass
    steps = max(3, min(args.steps, 16))
    forward()
    started = time.perf_counter()
    for _ in range(steps):
        forward()
    seconds = (time.perf_counter() - started) / steps
    value = sample / seconds
    what = "transformers.BertModel" if kind == "reference" else "the oracle's restatement of BertModel"
    line = {
        "impl": "reference", "metric": "encoder_sequences_per_s", "value": value, "unit": "seq/s", "n_gpus": args.gpus,
        "steps": steps, "steps_requested": args.steps, "warmup": 1, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"bert-base-shaped encoder forward, batch {batch} x {seq} tokens, all-ones attention mask",
                   "layers": config["num_hidden_layers"], "parallelism": "host cores", "arm": what + ", fp32, CPU"},
        "cpu_baseline": {"value": value, "unit": "seq/s", "cores": threads, "kind": kind,
                         "sample": f"{what}: {sample} sequence(s) of {seq} tokens per step, mean of {steps} steps"},
        "e2e": {"value": value, "unit": "seq/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_prefill(args) -> None:
    """Secondary workload: one prompt of `--prefill` tokens through a prefill plan (phase 0 of the plan ABI):
    ONE launch whose kernel steps take 64 (sequence, position) rows each, weights streamed once per kernel
    step, GEMM stages on tcgen05 tiles. One JSON line in the shape of the decode line; a step is one such
    kernel step (64 prompt positions)."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU implementation")
    import time

    from tilemega_b200.planbuild import PLAN_DIR, emit_plan, remove_plans
    from tilemega_b200.serving.plan import L2, PlanLibrary
    from tilemega_b200.serving.state import allocate_state, shuffled_block_table
    from tilemega_b200.serving.weights import load_weights
    config = dict(MODELS[args.model or "llama-3.1-8b"])
    if args.layers:
        config["num_hidden_layers"] = args.layers
    rows, length = 64, args.prefill
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    capacity = (length + 32) // 16 * 16
    num_blocks = capacity // 16 + 2
    plan_dir = PLAN_DIR / "bench"
    layout = dict(capacity=capacity, kv_layout="paged", num_blocks=num_blocks, write_logits=False)
    prefill_lib = PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=1, phase="prefill", seq=length, **layout))
    decode_lib = PlanLibrary(emit_plan(config, plan_dir, batch_lo=1, batch_hi=1, **layout))   # the state's description
    weights = load_weights(synthetic.LazySeededCheckpoint(config, seed=0, device=device), prefill_lib, device=device)
    table = shuffled_block_table(1, capacity // 16, num_blocks, seed=7)
    state = allocate_state(config, 1, decode_lib, device, block_table=table)
    pointers = {name: tensor.data_ptr() for name, tensor in weights.items()} | state.pointers
    plan = prefill_lib.create(1, pointers, 0)
    plan.set_steps([0])
    prompt = synthetic.seeded_tokens(1, length, config["vocab_size"], seed=3).to(torch.int32)
    host_prompt = prompt.pin_memory()
    host_token = torch.zeros(1, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream()
    chunks = -(-length // rows)

    def once() -> tuple[float, float]:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        wall = time.perf_counter()
        state.tokens[:, :length].copy_(host_prompt, non_blocking=True)
        begin.record(stream)
        plan.launch(0, L2, stream.cuda_stream)
        end.record(stream)
        host_token.copy_(state.tokens[:, length], non_blocking=True)
        stream.synchronize()
        wall = time.perf_counter() - wall
        if plan.watchdog() is not None:
            raise SystemExit(f"a bounded device wait gave up: {plan.watchdog()}")
        return begin.elapsed_time(end) / 1e3, wall

    for _ in range(max(args.warmup, 3) if length <= 1024 else 1):
        once()
    peak, peak_kind = measured_peak_gbs()
    with ClockSampler(0) as clocks:
        runs = [once() for _ in range(3)]
    device_s, wall = sorted(runs)[1]
    # algorithmic bytes: every kernel step streams the GEMM weights once; row i reads its p + 1 cached positions
    layers, hkv, dim = config["num_hidden_layers"], config["num_key_value_heads"], synthetic.head_dim_of(config)
    hidden, inter, heads, vocab = config["hidden_size"], config["intermediate_size"], config["num_attention_heads"], config["vocab_size"]
    weight_bytes = 2 * (layers * (hidden * (heads + 2 * hkv) * dim + heads * dim * hidden + 3 * hidden * inter) + vocab * hidden)
    kv_bytes = sum(position + 1 for position in range(length)) * layers * 2 * hkv * dim * 2
    total_bytes = chunks * weight_bytes + kv_bytes
    flops = float(length) * weight_bytes          # 2 flops per weight element (2 bytes) and row
    line = {
        "metric": "prefill_tokens_per_s", "value": length / device_s, "unit": UNIT, "n_gpus": 1, "steps": chunks,
        "warmup": 1 if length > 1024 else max(args.warmup, 3), "ms_per_step": device_s * 1e3 / chunks, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.model or 'llama-3.1-8b'}-shaped prefill plan, one prompt of {length} tokens, "
                               f"{rows} positions per kernel step, paged KV block 16, shuffled block table", "layers": layers,
                   "l2": "inputs (15 GB of weights per kernel step) exceed L2", "first_token": int(host_token[0]),
                   "time_to_first_token_ms": wall * 1e3},
        "roofline": {"bound": "hbm", "achieved": total_bytes / device_s / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": total_bytes / device_s / 1e9 / peak, "traffic": None, "peak_kind": "of " + peak_kind,
                     "bytes_per_launch": total_bytes, "tensor_tflops": flops / device_s / 1e12},
        "e2e": {"value": length / wall, "unit": UNIT, "h2d_bytes_per_step": length * 4 / chunks, "d2h_bytes_per_step": 4 / chunks},
        "gpu_launches": 1, "clocks": clocks.summary(),
    }
    plan.close()
    remove_plans(plan_dir)
    print(json.dumps(line), flush=True)


def run_forward(args) -> None:
    """Secondary workload: the BERT-base-shaped encoder forward (`--model bert-base --batch B`, batch x 128 tokens)
    through a forward plan (phase 2 of the plan ABI). A step is one forward pass = one graph launch of the
    encoder's kernels; `--steps` passes are timed back to back between two CUDA events. The CPU baseline is the
    oracle's fp32 forward on the host cores."""
    if int(os.environ.get("RANK", "0")) != 0:
        return   # the encoder forward does not shard: one GPU is measured, other ranks of a launcher have nothing to do
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU implementation")
    from tilemega_b200.planbuild import PLAN_DIR, emit_plan, remove_plans
    from tilemega_b200.serving.encoder import EncoderEngine
    from tilemega_b200.serving.weights import TensorCheckpoint
    config = dict(synthetic.BERT_BASE)
    if args.layers:
        config["num_hidden_layers"] = args.layers
    batch, seq, steps, warmup = args.batch, 128, args.steps, max(args.warmup, 3)
    dtype_name = args.encoder_dtype
    torch.cuda.set_device(0)
    plan_dir = PLAN_DIR / "bench"
    weights = synthetic.encoder_weights(config, seed=0)
    ids, types = synthetic.encoder_inputs(config, batch, seed=1)
    so = emit_plan(config, plan_dir, phase="forward", batch_lo=batch, dtype=dtype_name)
    engine = EncoderEngine(TensorCheckpoint(weights), so, batch)
    stream = engine.stream
    host_ids, host_types = ids.pin_memory(), types.pin_memory()
    hidden_out, pooled_out = engine.outputs()
    host_pooled = torch.zeros_like(pooled_out, device="cpu").pin_memory()
    engine(ids.cuda(), types.cuda())
    for _ in range(warmup):
        engine.launch()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    with ClockSampler(0) as clocks:
        begin.record(stream)
        for _ in range(steps):
            engine.launch()
        end.record(stream)
        stream.synchronize()
        device_s = begin.elapsed_time(end) / 1e3
        # end to end: every pass copies its ids from pinned host memory and reads the pooled rows back
        wall = time.perf_counter()
        for _ in range(steps):
            engine.tensors["input_ids"].copy_(host_ids.view(-1), non_blocking=True)
            engine.tensors["token_type_ids"].copy_(host_types.view(-1), non_blocking=True)
            engine.launch()
            host_pooled.copy_(pooled_out, non_blocking=True)
            stream.synchronize()
        wall = time.perf_counter() - wall
    if engine.plan.watchdog() is not None:
        raise SystemExit(f"a bounded device wait gave up: {engine.plan.watchdog()}")
    hidden, inter, layers = config["hidden_size"], config["intermediate_size"], config["num_hidden_layers"]
    tokens = batch * seq
    # products of the projections (2 flops per weight element and token) and of attention (QK^T and PV)
    flops = 2.0 * tokens * layers * (4 * hidden * hidden + 2 * hidden * inter) + 4.0 * batch * layers * seq * seq * hidden
    weight_bytes = 2 * layers * (4 * hidden * hidden + 2 * hidden * inter)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak_tf, peak_kind = (float(peaks["bf16_tflops"]), "measured") if peaks else (1590.0, "fallback")
    line = {
        "metric": "encoder_sequences_per_s", "value": batch * steps / device_s, "unit": "seq/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": device_s * 1e3 / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype_name, "data": "synthetic",
        "config": {"workload": f"bert-base-shaped encoder forward, batch {batch} x {seq} tokens, all-ones attention mask", "layers": layers,
                   "l2": f"weights ({weight_bytes / 1e6:.0f} MB) exceed L2" if weight_bytes > 126e6 else "weights fit L2 (small case)"},
        "roofline": {"bound": "tensor", "achieved": flops / device_s * steps / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": flops / device_s * steps / 1e12 / peak_tf, "traffic": None, "peak_kind": "of " + peak_kind + " (cuBLAS bf16 burst)",
                     "flops_per_launch": flops, "weight_gbs": weight_bytes * steps / device_s / 1e9},
        "e2e": {"value": batch * steps / wall, "unit": "seq/s", "h2d_bytes_per_step": 2 * tokens * 8,
                "d2h_bytes_per_step": pooled_out.numel() * pooled_out.element_size()},
        # per pass: embedding, pooler, and per layer QKV, attention, O-proj, add + LayerNorm, FFN up, FFN down, add + LayerNorm
        "gpu_launches": steps * (2 + 7 * layers),
        "clocks": clocks.summary(),
    }
    if not args.no_cpu:
        from oracle.encoder_oracle import encoder_forward
        threads = min(os.cpu_count() or 1, 16)
        torch.set_num_threads(threads)
        sample = min(batch, 4)
        encoder_forward(weights, config, ids[:1], types[:1])
        started = time.perf_counter()
        repeats = 3
        for _ in range(repeats):
            encoder_forward(weights, config, ids[:sample], types[:sample])
        cpu_s = (time.perf_counter() - started) / repeats
        line["cpu_baseline"] = {"value": sample / cpu_s, "unit": "seq/s", "cores": threads, "kind": "port",
                                "sample": f"the oracle's fp32 forward of {sample} sequence(s) of {seq} tokens, mean of {repeats}"}
    engine.close()
    remove_plans(plan_dir)
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU implementation")
    from tilemega_b200.planbuild import PLAN_DIR, emit_plan, remove_plans
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
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    work = workload(args)
    config, batch, contexts, tp = work["config"], work["batch"], work["contexts"], work["tp"]
    steps, warmup = args.steps, max(args.warmup, 3)
    total_steps = warmup + 2 * steps + 1 + 4   # device-timed launch, the end-to-end loop, and the optional traced steps
    capacity = (max(contexts) + total_steps + 17) // 16 * 16
    max_blocks = capacity // 16
    num_blocks = batch * max_blocks + 32
    plan_dir = PLAN_DIR / "bench"    # inside the package tree: every library this process loads is the repository's
    options = dict(batch_lo=batch, batch_hi=batch, capacity=capacity, kv_layout="paged", num_blocks=num_blocks,
                   write_logits=False, tp=tp, weights=args.weights)
    if rank == 0:
        so = emit_plan(config, plan_dir, **options)
    if world > 1:
        dist.barrier()
        so = emit_plan(config, plan_dir, **options)   # an identical plan is left alone: this only returns its path
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
    pointers = {name: tensor.data_ptr() for name, tensor in weights.items()} | state.pointers
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
            dist.barrier()
        torch.cuda.synchronize()

    def tokens_agree(first_position: int, count: int, what: str) -> None:
        """Tensor parallel: every rank must have written the same tokens (the ranks' residual
        streams are bitwise equal by construction; a difference means a broken exchange)."""
        if tp <= 1:
            return
        mine = torch.stack([state.tokens[b, contexts[b] + first_position:contexts[b] + first_position + count]
                            for b in range(batch)]).contiguous()
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        for q in range(world):
            if not torch.equal(everyone[q], everyone[0]):
                raise SystemExit(f"{what}: rank {q} generated tokens that differ from rank 0's")

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
        tokens_agree(1, warmup + steps, "timed launch")
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
    tokens_agree(warmup + steps + 1, steps, "end-to-end loop")
    peak, peak_kind = measured_peak_gbs()
    if args.trace:
        # per-stage stamps of one more step (every rank of a tensor-parallel job runs it; rank 0 reports)
        import numpy as np
        from tilemega_b200.stage_trace import print_table
        plan.trace_step(warmup + 2 * steps + 2)
        plan.launch_steps(warmup + 2 * steps, 4, mode, stream.cuda_stream)
        barrier()
        trace = np.array(plan.read_trace(), dtype=np.int64)
        grid = torch.cuda.get_device_properties(local).multi_processor_count
        per_layer = (trace.size // 4 // grid - 1) // config["num_hidden_layers"]
        if rank == 0:
            print_table(config, trace.reshape(grid, -1, 4), per_layer, sum(contexts) // len(contexts) + warmup + 2 * steps, batch, tp=tp,
                        peak=peak)
    device_ms, e2e_seconds = max_over_ranks([device_ms, e2e_seconds], device)
    seconds = device_ms / 1e3
    replicas = 1 if tp > 1 else world
    value = job_value(replicas, batch, steps, seconds)
    achieved = bytes_timed / seconds / 1e9
    step_us = [(stamps[i + 1] - stamps[i]) / 1e3 for i in range(steps)]
    ratio = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get((work["model"], batch)) if tp == 1 and args.weights == "bf16" else None
    parallelism = f"tp{tp}" if tp > 1 else ("replicas" if world > 1 else "single")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": device_ms / steps, "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak",
        "vs_baseline": None, "dtype": "bf16" if args.weights == "bf16" else f"bf16 activations, {args.weights} weights",
        "data": "synthetic",
        "config": {"workload": work["label"], "layers": config["num_hidden_layers"],
                   "l2": "inputs larger than L2: every step streams its weights and KV rows from HBM",
                   "parallelism": parallelism, "step_latency_us_median": statistics.median(step_us),
                   "mbu_vs_nominal_8tbs": achieved / NOMINAL_HBM_GBS},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": ratio * bytes_timed if ratio else None,
                     "traffic_source": ("ncu capture of the same kernel on a 2-layer case of this model and batch, scaled by "
                                        "algorithmic bytes" if ratio else
                                        "none: no ncu capture exists for this model/batch" +
                                        (" (ncu never wraps a multi-rank command)" if tp > 1 else "")),
                     "per": "GPU (this rank's share of the weights and KV rows)" if tp > 1 else "GPU",
                     "peak_kind": f"of {peak_kind}", "bytes_per_launch": bytes_timed},
        "e2e": {"value": job_value(replicas, batch, steps, e2e_seconds), "unit": UNIT, "h2d_bytes_per_step": 4 * batch,
                "d2h_bytes_per_step": 4 * batch},
        "gpu_launches": 1,
        "clocks": sampler.summary(),
    }
    if tp > 1:
        # per-GPU roofline fraction kept against the one-GPU 8B-shaped headline: the curve to read for
        # a tensor-parallel run (tokens/s at N GPUs and at one GPU belong to two different models)
        line["config"]["mbu_retained_vs_1gpu"] = achieved / peak / SINGLE_GPU_FRAC
        line["config"]["ranks_agree_on_tokens"] = True
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        result = cpu_forward(work, 8, threads, repeats=2)
        line["cpu_baseline"] = {"value": batch / result["seconds"], "unit": UNIT, "cores": threads, "kind": result["kind"],
                                "sample": result["sample"]}
    plan.close()
    if world > 1:
        dist.barrier()
    if rank == 0:
        remove_plans(plan_dir)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=4)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--model", choices=sorted(MODELS), default=None,
                        help="shape of the synthetic model (default: llama-3.1-8b on one GPU, llama-3.1-70b sharded over several)")
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--context", type=int, default=None,
                        help="0: seeded draw in [512, 8192] (the one-GPU default); several GPUs default to 4096")
    parser.add_argument("--layers", type=int, default=0, help="override the depth (profiling a small case)")
    parser.add_argument("--weights", choices=("bf16", "e4m3"), default="bf16",
                        help="e4m3: GEMV matrices as 8-bit codes with one fp32 scale per output row")
    parser.add_argument("--encoder-dtype", choices=("f16", "bf16"), default="f16",
                        help="--model bert-base: element type of the forward plan (f16: the benchmark configuration; bf16: what the reference's export runs)")
    parser.add_argument("--prefill", type=int, default=0,
                        help="secondary workload: chunked prefill of one prompt of this many tokens (one GPU)")
    parser.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    parser.add_argument("--trace", action="store_true",
                        help="after the timed runs, stamp one more step and print the per-stage table (rank 0)")
    parser.add_argument("--replicas", action="store_true",
                        help="several GPUs: independent copies of the one-GPU workload instead of one sharded model")
    parser.add_argument("--tp", action="store_true", help="accepted for compatibility: several GPUs shard one model by default")
    args = parser.parse_args()
    if args.impl == "reference" and args.model == "bert-base":
        run_forward_reference(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.model == "bert-base":
        run_forward(args)
    elif args.prefill:
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
