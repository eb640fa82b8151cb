"""One rank of the tensor-parallel GPU parity test (run under torch.distributed.run by
tests/test_gpu_tp.py; one process per GPU, gloo for the set-up and the checks).

Every rank drives its own plan through the C ABI; the ranks' kernels exchange their
partial sums over NVLink by themselves. Rank 0 compares the gathered logits and the
tokens with the CPU oracle run at the same tensor-parallel degree.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oracle.decoder_oracle import OracleDecoder, PagedKV  # noqa: E402
from tilemega_b200 import synthetic  # noqa: E402
from tilemega_b200.planbuild import emit_plan  # noqa: E402
from tilemega_b200.serving.tp_engine import TpServingEngine  # noqa: E402
from tilemega_b200.serving.weights import TensorCheckpoint  # noqa: E402

from harness import assert_parity, bf16_weights  # noqa: E402

LOGIT_TOLERANCE = 2e-2


def oracle_logits(config, weights, prompt, forced, capacity, dtype, tp):
    decoder = OracleDecoder(config, weights, dtype, capacity, tp=tp)
    kv = PagedKV(config, prompt.shape[0], capacity, dtype)
    _, logits = decoder.greedy(prompt, forced.shape[1], kv, forced=forced, head_fp32=True)
    return logits


def run_case(name: str, config: dict, batch: int, prompt_len: int, new_tokens: int, capacity: int, plan_dir: Path):
    rank, world = dist.get_rank(), dist.get_world_size()
    weights = bf16_weights(config)
    so = emit_plan(config, plan_dir / f"rank{rank}", batch_lo=batch, batch_hi=batch, capacity=capacity, tp=world)
    prompt = synthetic.seeded_tokens(batch, prompt_len, config["vocab_size"], seed=1)
    engine = TpServingEngine(TensorCheckpoint(weights, config.get("tie_word_embeddings", False)), config, so, batch,
                             prompt_len=prompt_len, max_new_tokens=new_tokens, device=rank)
    plan, state, lib = engine.plan, engine.state, engine.library
    stream = torch.cuda.current_stream().cuda_stream
    rows = config["vocab_size"] // world

    def local_logits():
        host = torch.empty(batch * rows, dtype=torch.float32)
        torch.cuda.synchronize()
        plan.read_buffer("serving.logits", host.data_ptr(), host.numel() * 4)
        return host.reshape(batch, rows)

    # step by step, every rank in lockstep, reading this rank's slice of the logits
    state.tokens.zero_()
    state.tokens[:, :prompt_len].copy_(prompt)
    plan.launch_steps(0, prompt_len, 1, stream)
    history = [local_logits()]
    for step in range(new_tokens - 1):
        plan.launch(prompt_len + step, 1, stream)
        history.append(local_logits())
    fired = plan.watchdog()
    assert fired is None, f"rank {rank}: a bounded device wait gave up: {fired}"
    tokens = state.tokens[:, prompt_len:prompt_len + new_tokens].cpu()
    gathered: list = [None] * world
    dist.all_gather_object(gathered, (torch.stack(history), tokens))
    logits = torch.cat([item[0] for item in gathered], dim=-1)   # [new][B][V]
    for q in range(world):
        assert torch.equal(gathered[q][1], tokens), f"rank {q} wrote different tokens"
    engine.close()
    # the same generation as one persistent launch per phase through the engine
    engine = TpServingEngine(TensorCheckpoint(weights, config.get("tie_word_embeddings", False)), config, so, batch,
                             prompt_len=prompt_len, max_new_tokens=new_tokens, device=rank)
    looped = engine.generate(prompt).tokens
    engine.close()
    assert torch.equal(looped, tokens), "one launch for all steps and one launch per step disagree"
    result = {}
    if rank == 0:
        exact = oracle_logits(config, weights, prompt, tokens, capacity, torch.float32, world)
        module = oracle_logits(config, weights, prompt, tokens, capacity, torch.bfloat16, world)
        ours, theirs = (logits - exact).abs(), (module - exact).abs()
        assert ours.max().item() <= 1.25 * theirs.max().item(), (name, ours.max().item(), theirs.max().item())
        assert ours.mean().item() <= 1.25 * theirs.mean().item(), (name, ours.mean().item(), theirs.mean().item())
        assert_parity(tokens, logits, exact, max(LOGIT_TOLERANCE, 1.25 * theirs.max().item()), name)
        result = {"case": name, "gpu_vs_fp32_max": ours.max().item(), "bf16_oracle_vs_fp32_max": theirs.max().item(),
                  "gpu_vs_fp32_mean": ours.mean().item(), "bf16_oracle_vs_fp32_mean": theirs.mean().item()}
        print(json.dumps(result), flush=True)
    dist.barrier()
    return result


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--plan-dir", required=True)
    parser.add_argument("--out", default="")
    args = parser.parse_args()
    dist.init_process_group("gloo")
    torch.cuda.set_device(dist.get_rank())
    plan_dir = Path(args.plan_dir)
    results = [
        # o (and, for the second case, down) reductions of 1024 columns per rank: padded to one
        # 2048-column page of which only the first half is copied
        run_case("tiny_d128 tp", synthetic.TINY_D128, 3, 13, 5, 32, plan_dir),
        run_case("tiny_gq8 tp", synthetic.TINY_GQ8, 2, 21, 6, 64, plan_dir),
    ]
    if dist.get_rank() == 0 and args.out:
        Path(args.out).write_text(json.dumps(results))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
