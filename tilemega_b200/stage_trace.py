"""Per-stage timing of one decode step of a plan, from the kernel's own stage stamps.

    python -m tilemega_b200.stage_trace --model llama-3.1-8b [--layers N] [--context C] [--batch B]

Builds a plan for a synthetic model of the given shape, runs a few steps, asks the
library to stamp one step (`tm_plan_trace_step`: per CTA and stage, %globaltimer when the
CTA started waiting for the stage's inputs, when they were there, when its activation
rows were staged and when its last task was done) and prints, per kind of stage and
averaged over the layers: the wall time of the stage (last CTA done to last CTA done), the
time its bytes take at the measured copy bandwidth, and the median CTA's wait / row
staging / task time. The reference's counterpart is its TILEMEGA_TRACE_STAGE build
(include/tilemega/Codegen/tasks/ModelRuntime.h:758-766). Needs a CUDA device.
"""
from __future__ import annotations

import argparse
import os

import torch

from . import synthetic
from .planbuild import PLAN_DIR, emit_plan, remove_plans
from .serving.plan import PlanLibrary
from .serving.state import allocate_state, shuffled_block_table
from .serving.weights import load_weights

MODELS = {"llama-3.1-8b": synthetic.LLAMA_3_1_8B, "llama-3.2-1b": synthetic.LLAMA_3_2_1B,
          "qwen3-30b-a3b": synthetic.QWEN3_30B_A3B}


# Copy bandwidth of a B200 as a plain device-to-device copy measures it (GB/s): the default
# denominator of the "ideal" column; pass the figure of the box at hand with --peak-gbs.
DEFAULT_PEAK_GBS = 6552.6


def stage_bytes(config: dict, context: int, batch: int) -> dict[str, float]:
    hidden, dim = config["hidden_size"], synthetic.head_dim_of(config)
    heads, hkv = config["num_attention_heads"], config["num_key_value_heads"]
    sizes = {"qkv": (heads + 2 * hkv) * dim * hidden * 2, "attn": 4 * hkv * dim * context * batch,
             "o": hidden * heads * dim * 2}
    if synthetic.is_moe(config):
        inter, topk = config["moe_intermediate_size"], config["num_experts_per_tok"]
        sizes.update(router=config["num_experts"] * hidden * 2, gate_up=topk * 2 * inter * hidden * 2,
                     down=topk * hidden * inter * 2)
    else:
        inter = config["intermediate_size"]
        sizes.update(gate_up=2 * inter * hidden * 2, down=hidden * inter * 2)
    return sizes


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--model", choices=sorted(MODELS), default="llama-3.1-8b")
    parser.add_argument("--layers", type=int, default=0)
    parser.add_argument("--context", type=int, default=2646)
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--attn-min-slots", type=int, default=None)
    parser.add_argument("--dump", default=None, help="also save the raw stamps, int64 [grid][stages][4], as a .npy file")
    parser.add_argument("--kv-layout", choices=("paged", "contiguous"), default="paged")
    parser.add_argument("--table", choices=("shuffled", "identity"), default="shuffled",
                        help="paged layout: pool blocks of a sequence in random order (the serving case) or in order")
    parser.add_argument("--peak-gbs", type=float, default=DEFAULT_PEAK_GBS,
                        help="measured HBM copy bandwidth the ideal stage times are computed from")
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("stage_trace needs a CUDA device")
    import numpy as np
    config = dict(MODELS[args.model])
    if args.layers:
        config["num_hidden_layers"] = args.layers
    layers, batch, context, steps = config["num_hidden_layers"], args.batch, args.context, 24
    capacity = (context + steps + 40) // 16 * 16
    device = torch.device("cuda", 0)
    num_blocks = batch * capacity // 16 + 8
    folder = PLAN_DIR / f"trace-{os.getpid()}"
    try:
        paged = args.kv_layout == "paged"
        so = emit_plan(config, folder, batch_lo=batch, batch_hi=batch, capacity=capacity, kv_layout=args.kv_layout,
                       num_blocks=num_blocks if paged else 0, write_logits=False, attn_min_slots=args.attn_min_slots)
        lib = PlanLibrary(so)
        weights = load_weights(synthetic.LazySeededCheckpoint(config, seed=0, device=device), lib, device=device)
        if paged:
            table = (shuffled_block_table(batch, capacity // 16, num_blocks, seed=7) if args.table == "shuffled"
                     else torch.arange(batch * (capacity // 16), dtype=torch.int32).reshape(batch, capacity // 16))
            state = allocate_state(config, batch, lib, device, block_table=table,
                                   context_base=torch.tensor([context] * batch, dtype=torch.int32))
            first = 0
        else:
            state = allocate_state(config, batch, lib, device)
            first = context      # a contiguous cache has no per-sequence offset: the step numbers carry the context
        state.kv_storage.normal_(0, 0.5)
        pointers = {name: tensor.data_ptr() for name, tensor in weights.items()}
        pointers.update(state.pointers)
        plan = lib.create(batch, pointers, 0)
        plan.set_prompt_len(0)
        plan.set_steps(list(range(first, first + steps)))
        stream = torch.cuda.current_stream().cuda_stream
        plan.launch_steps(0, 4, 2, stream)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        plan.launch_steps(4, 12, 2, stream)
        end.record()
        torch.cuda.synchronize()
        print(f"{args.model}, {layers} layers, batch {batch}, context {context}: "
              f"{begin.elapsed_time(end) / 12:.4f} ms/step, shared memory {plan.execution_smem()} B, "
              f"watchdog {plan.watchdog()}")
        plan.trace_step(18)
        plan.launch_steps(16, 6, 2, stream)
        torch.cuda.synchronize()
        kinds = ["qkv", "attn", "o"] + (["router"] if synthetic.is_moe(config) else []) + ["gate_up", "down"]
        stamps = np.array(plan.read_trace(), dtype=np.int64)
        # [grid][stages][4] words; the grid is one CTA per SM; a wide batch has a few more stages
        # per layer than `kinds` (its down reduction runs in parts)
        grid = torch.cuda.get_device_properties(0).multi_processor_count
        trace = stamps.reshape(grid, -1, 4)
        per_layer = (trace.shape[1] - 1) // layers
        if args.dump:
            np.save(args.dump, trace)
        plan.close()
    finally:
        remove_plans(folder)
    print_table(config, trace, per_layer, context, batch, peak=args.peak_gbs)


def print_table(config: dict, trace, per_layer: int, context: int, batch: int, tp: int = 1,
                peak: float = DEFAULT_PEAK_GBS) -> None:
    """`trace`: int64 [grid][per_layer * layers + 1][4] stage stamps of one step (one rank's)."""
    import numpy as np
    layers = config["num_hidden_layers"]
    kinds = ["qkv", "attn", "o"] + (["router"] if synthetic.is_moe(config) else []) + ["gate_up", "down"]
    if batch > 8:   # dense-batch plans: RMSNorm is a stage of its own, twice per layer
        kinds = ["norm1", "qkv", "attn", "o", "norm2", "gate_up", "down"]
    parts = per_layer - len(kinds) + 1
    if synthetic.is_moe(config) and batch > 1:   # the experts' MLP runs token by token
        kinds = kinds[:-2] + [f"{kind} tok {b}" for b in range(batch) for kind in ("gate_up", "down")]
        parts = 1
    if parts > 1:
        kinds = kinds[:-1] + [f"down part {i}" for i in range(parts)]
    start = trace[:, 0, 1].min()
    done, first_done = trace[:, :, 3].max(axis=0), trace[:, :, 3].min(axis=0)
    wall = np.diff(np.concatenate(([start], done)))
    sizes = stage_bytes(config, context + 18, batch)
    sizes = {name: value / tp for name, value in sizes.items()}
    print(f"{'stage':12s} {'wall':>7s} {'ideal':>7s} {'wait':>6s} {'rows':>6s} {'tasks':>6s} {'max':>6s} {'spread':>6s}   (us; "
          f"ideal = bytes / {peak:.0f} GB/s; medians over CTAs, means over layers 1..{layers - 1})")
    for k, kind in enumerate(kinds):
        index = [l * per_layer + k for l in range(1, layers)] or [k]
        ideal = sizes.get(kind.split(" part")[0].split(" tok")[0], 0) / peak / 1e3
        if " part" in kind:
            ideal /= parts
        print(f"{kind:12s} {wall[index].mean() / 1e3:7.2f} {ideal:7.2f} "
              f"{np.median(trace[:, index, 1] - trace[:, index, 0], axis=0).mean() / 1e3:6.2f} "
              f"{np.median(trace[:, index, 2] - trace[:, index, 1], axis=0).mean() / 1e3:6.2f} "
              f"{np.median(trace[:, index, 3] - trace[:, index, 2], axis=0).mean() / 1e3:6.2f} "
              f"{(trace[:, index, 3] - trace[:, index, 2]).max(axis=0).mean() / 1e3:6.2f} "
              f"{(done[index] - first_done[index]).mean() / 1e3:6.2f}")
    print(f"{'head':12s} {wall[-1] / 1e3:7.2f} {config['vocab_size'] * config['hidden_size'] * 2 / tp / peak / 1e3:7.2f}")
    if layers > 1:
        print(f"layer total  {wall[per_layer:per_layer * layers].sum() / (layers - 1) / 1e3:7.2f} "
              f"{sum(sizes.values()) / peak / 1e3:7.2f}")


if __name__ == "__main__":
    main()
