"""Driver of a forward plan (phase 2): a stateless encoder pass through the plan ABI.

Mirrors the reference's NativeForward (python/tilemega/dnn/check.py:30-101): the plan's external buffers are the
module's parameters under their qualified names (packed from the checkpoint by their recipes), the user inputs
(`input_ids`, `token_type_ids`, int64 [batch, seq]) and the user outputs (`last_hidden_state` [batch, seq, hidden],
`pooler_output` [batch, hidden]); one call copies the inputs into their bound tensors, launches step 0 and
returns the outputs.
"""
from __future__ import annotations

import torch

from .plan import FORWARD, L2, PlanLibrary
from .weights import DTYPES, load_weights

INPUTS = ("input_ids", "token_type_ids", "attention_mask")   # the third only in a plan emitted with mask=True
OUTPUTS = ("last_hidden_state", "pooler_output")


class EncoderEngine:
    def __init__(self, checkpoint, forward_so, batch: int, device: int = 0, weights=None):
        if not torch.cuda.is_available():
            raise RuntimeError("EncoderEngine needs a CUDA device; there is no CPU path")
        torch.cuda.set_device(device)
        self.library = PlanLibrary(forward_so)
        info = self.library.info
        if info.phase != FORWARD or info.capacity or not info.batch_lo <= batch <= info.batch_hi:
            raise ValueError("the library is not a forward plan covering this batch size")
        self.batch, self.seq = batch, int(info.seq)
        where = torch.device("cuda", device)
        self.tensors = load_weights(checkpoint, self.library, device=where) if weights is None else dict(weights)
        for buffer in self.library.buffers:
            if buffer.role == 1 and buffer.name in INPUTS + OUTPUTS:
                count = buffer.elements_constant + batch * buffer.elements_per_batch
                self.tensors[buffer.name] = torch.zeros(count, dtype=DTYPES[buffer.dtype], device=where)
        external = {buffer.name for buffer in self.library.buffers if buffer.role == 1}
        if external != self.tensors.keys():
            raise ValueError("the bound tensors differ from the plan's external buffers")
        self.plan = self.library.create(batch, {name: tensor.data_ptr() for name, tensor in self.tensors.items()}, device)
        self.plan.set_steps([0])
        self.masked = "attention_mask" in self.tensors
        self.hidden = self.tensors["pooler_output"].numel() // batch
        self.stream = torch.cuda.current_stream()

    def launch(self, mode: int = L2) -> None:
        """One forward pass over the inputs already in their bound tensors (asynchronous)."""
        self.plan.launch(0, mode, self.stream.cuda_stream)

    def outputs(self) -> tuple[torch.Tensor, torch.Tensor]:
        return (self.tensors["last_hidden_state"].view(self.batch, self.seq, self.hidden),
                self.tensors["pooler_output"].view(self.batch, self.hidden))

    def __call__(self, input_ids: torch.Tensor, token_type_ids: torch.Tensor, attention_mask: torch.Tensor | None = None,
                 mode: int = L2) -> tuple[torch.Tensor, torch.Tensor]:
        if attention_mask is not None and not self.masked:
            raise ValueError("this plan was emitted without an attention_mask input")
        if self.masked and attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        given = (input_ids, token_type_ids) + ((attention_mask,) if self.masked else ())
        for name, value in zip(INPUTS, given):
            if tuple(value.shape) != (self.batch, self.seq) or value.dtype != torch.int64:
                raise ValueError(f"{name} must be int64 [{self.batch}, {self.seq}]")
            self.tensors[name].copy_(value.reshape(-1), non_blocking=True)
        self.launch(mode)
        self.stream.synchronize()
        gave_up = self.plan.watchdog()
        if gave_up is not None:
            raise RuntimeError(f"a bounded device wait gave up: {gave_up}")
        hidden, pooled = self.outputs()
        return hidden.clone(), pooled.clone()

    def close(self) -> None:
        self.plan.close()

    def __enter__(self) -> "EncoderEngine":
        return self

    def __exit__(self, *_: object) -> None:
        self.close()
