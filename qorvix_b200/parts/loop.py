"""Re-entry of the residual stream into a stretch of layers that runs several times with the same weights: at the
start of pass t the stream becomes W [x ; x0] + step[t], x0 being the embedding's output.  The sum x = residual +
pending is formed in float32; the product takes its operands in the compute type and leaves float32."""
from __future__ import annotations

import torch

from ..csrc import ops
from .linear import Linear
from .registry import register_part


class LoopEntry:
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.proj = Linear(source.get(spec.in_proj))
        self.step = source.get(spec.step, dtype=torch.float32)
        self.pass_of = {run: t for t, run in enumerate(spec.first_runs)}

    def forward(self, run: int, residual, pending, x0):
        """The stream as pass `pass_of[run]` finds it (a new float32 tensor; nothing is pending after it)."""
        T, d = residual.shape
        cat = torch.empty((T, 2 * d), device=residual.device, dtype=self.rt.dtype)
        ops.stream_concat(cat, residual, pending, x0)
        out = self.proj(cat, out_dtype=torch.float32)
        ops.add_vector(out, self.step[self.pass_of[run]])
        return out


register_part("stream", "loop_entry", LoopEntry)
