"""Mixers with a state of fixed size per request instead of a cache that grows: a matrix-memory LSTM and a
selective state space.  Both are the recurrence S = a S + b k v^T, y = S^T q per head with different gates
(csrc/recurrent.cu); the state is float32, lives in the cache manager's request slots (zeroed at
admission) and is carried from step to step, so a prompt may be cut anywhere."""
from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec
from ..csrc import ops
from .base import Mixer
from .linear import Linear
from .registry import register_part


def _fused(source, names):
    mats = [source.get(n) for n in names]
    dt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
    return torch.cat([m.to(dt) for m in mats], dim=0)


class MLSTM(Mixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dk, self.dv = spec.num_heads, spec.key_dim, spec.value_dim
        self.proj = Linear(_fused(source, [spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj]))     # [q | k | v | gate]
        self.gates = Linear(_fused(source, [spec.i_proj, spec.f_proj]))                                # [i | f], float32 out
        self.i_bias = source.get(spec.i_bias, dtype=torch.float32)
        self.f_bias = source.get(spec.f_bias, dtype=torch.float32)
        self.norm = source.get(spec.norm, dtype=torch.float32)
        self.o_proj = Linear(source.get(spec.o_proj))
        self.state_floats = ops.linear_scan_state_floats(ops.SCAN_GATED_MAX, self.H, self.dk, self.dv)

    def cache_spec(self):
        return FixedStateSpec((self.state_floats,), "float32")

    def forward(self, x, ctx, cache):
        H, dk, dv = self.H, self.dk, self.dv
        proj = self.proj(x, out_dtype=self.rt.dtype)
        gates = self.gates(x, out_dtype=torch.float32)
        T = proj.shape[0]
        y = torch.empty((T, H * dv), device=proj.device, dtype=torch.float32)
        ops.linear_scan(ops.SCAN_GATED_MAX, y, proj[:, : H * dk], proj[:, H * dk: 2 * H * dk], proj[:, 2 * H * dk: 2 * H * dk + H * dv],
                        gates[:, :H], gates[:, H:], self.i_bias, self.f_bias, None, self.spec.gate_cap, dk ** -0.5, cache.tensor,
                        ctx, H, dk, dv)
        out = torch.empty((T, H * dv), device=proj.device, dtype=self.rt.dtype)
        ops.gated_group_norm(out, y, proj[:, 2 * H * dk + H * dv:], self.norm, H, self.spec.eps, gate_first=False)
        return self.o_proj(out, out_dtype=self.rt.dtype)


class Mamba2(Mixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.P, self.N, self.G = spec.num_heads, spec.value_dim, spec.state_dim, spec.groups
        w = source.get(spec.in_proj)
        split = spec.inner + spec.conv_channels
        self.in_zx = Linear(w[:split].contiguous())                  # [z | x | B | C]
        self.in_dt = Linear(w[split:].contiguous())                  # step sizes, float32 out
        del w
        self.conv_w = source.get(spec.conv_weight, dtype=torch.float32)
        self.conv_b = source.get(spec.conv_bias, dtype=torch.float32)
        self.dt_bias = source.get(spec.dt_bias, dtype=torch.float32)
        self.a_log = source.get(spec.a_log, dtype=torch.float32)
        self.skip = source.get(spec.skip, dtype=torch.float32)
        self.norm = source.get(spec.norm, dtype=torch.float32)
        self.o_proj = Linear(source.get(spec.o_proj))
        self.scan_floats = ops.linear_scan_state_floats(ops.SCAN_DECAY, self.H, self.N, self.P)
        self.tail_floats = (spec.conv_taps - 1) * spec.conv_channels

    def cache_spec(self):
        # [the heads' states | the convolution's last inputs]
        return FixedStateSpec((self.scan_floats + self.tail_floats,), "float32")

    def forward(self, x, ctx, cache):
        s, H, P, N, G = self.spec, self.H, self.P, self.N, self.G
        inner = s.inner
        zx = self.in_zx(x, out_dtype=self.rt.dtype)
        dt = self.in_dt(x, out_dtype=torch.float32)
        T = zx.shape[0]
        conv = torch.empty((T, s.conv_channels), device=zx.device, dtype=self.rt.dtype)
        state = cache.tensor
        ops.conv_state(conv, zx[:, inner:], self.conv_w, self.conv_b, state[:, self.scan_floats:], ctx)
        y = torch.empty((T, inner), device=zx.device, dtype=torch.float32)
        ops.linear_scan(ops.SCAN_DECAY, y, conv[:, inner + G * N:], conv[:, inner: inner + G * N], conv[:, :inner], dt, None,
                        self.dt_bias, self.a_log, self.skip, 0.0, 1.0, state[:, : self.scan_floats], ctx, H, N, P, q_group=H // G)
        out = torch.empty((T, inner), device=zx.device, dtype=self.rt.dtype)
        ops.gated_group_norm(out, y, zx[:, :inner], self.norm, s.norm_groups, s.eps, gate_first=True)
        return self.o_proj(out, out_dtype=self.rt.dtype)


register_part("mixer", "mlstm", MLSTM)
register_part("mixer", "mamba2", Mamba2)
