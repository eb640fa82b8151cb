"""Continuous batching on the GPU: requests of different lengths join and leave a two-slot batch
between steps; every request must generate exactly the tokens it generates alone (block tables,
per-slot positions and teacher forcing inside the prompt are transparent), and the pool is whole
again at the end."""
import pytest
import torch

from tilemega_b200 import synthetic
from tilemega_b200.planbuild import emit_plan
from tilemega_b200.serving.continuous import ContinuousEngine, Request
from tilemega_b200.serving.weights import TensorCheckpoint

from harness import GpuRun, bf16_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("base", ["TINY", "TINY_D128"])
def test_requests_generate_what_they_generate_alone(base, plan_dir):
    config = getattr(synthetic, base)
    capacity, slots, num_blocks = 64, 2, 4     # 3 usable blocks: fewer than slots x blocks per sequence
    weights = bf16_weights(config)
    shapes = [(5, 6), (1, 9), (20, 6), (7, 7), (3, 12)]          # (prompt length, new tokens)
    requests = []
    for number, (length, new) in enumerate(shapes):
        prompt = synthetic.seeded_tokens(1, length, config["vocab_size"], seed=20 + number)[0].tolist()
        requests.append(Request(number, prompt, new))
    # each request alone, through the static-batch path
    alone = {}
    solo = GpuRun(config, weights, 1, capacity, plan_dir)
    for request in requests:
        tokens, _ = solo.greedy(torch.tensor([request.prompt], dtype=torch.int32), request.max_new_tokens, stepwise=False)
        alone[request.id] = tokens[0].tolist()
    solo.close()
    so = emit_plan(config, plan_dir, batch_lo=slots, batch_hi=slots, capacity=capacity, kv_layout="paged",
                   num_blocks=num_blocks)
    checkpoint = TensorCheckpoint(weights, config.get("tie_word_embeddings", False))
    with ContinuousEngine(checkpoint, config, so, slots) as engine:
        for request in requests[:3]:
            engine.submit(request)
        finished = []
        for _ in range(4):                       # the last two requests arrive while the batch is running
            finished += engine.step()
        for request in requests[3:]:
            engine.submit(request)
        finished += engine.run_until_done()
        assert sorted(request.id for request in finished) == [0, 1, 2, 3, 4]
        for request in finished:
            assert request.generated == alone[request.id], (request.id, request.generated, alone[request.id])
        assert len(engine.scheduler.pool.free) == num_blocks - 1
        # fewer steps than running the requests one after another (the slots were shared)
        assert engine.steps_run < sum(length + new - 1 for length, new in shapes)
