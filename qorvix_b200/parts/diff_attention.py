"""Differential attention over the paged cache: two softmax maps per head over one set of values, the second
subtracted from the first times a number of the layer, the difference unit-normed per head.  q, k and v come from
one fused projection with float32 sums; one kernel adds the biases, norms and rotates every map of q and k and
writes k and v into the token's cache row (keys of both maps, then values); attention reads keys and values
from the pages only, so a prompt portion and a single decoded token take the same path.
"""
from __future__ import annotations

import math

import torch

from ..cache.spec import PagedRowsSpec
from ..csrc import ops
from .base import Mixer
from .linear import Linear
from .registry import build_part, register_part


class DiffAttention(Mixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.G, self.n, self.dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        if self.H % self.G:
            raise ValueError(f"num_heads {self.H} is not a multiple of num_kv_heads {self.G}")
        mats = [source.get(spec.q_proj), source.get(spec.k_proj), source.get(spec.v_proj)]
        dt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.qkv_proj = Linear(torch.cat([m.to(dt) for m in mats], dim=0))
        del mats
        self.bias = torch.cat([source.get(name + ".b", dtype=torch.float32) for name in (spec.q_proj, spec.k_proj, spec.v_proj)]).contiguous()
        self.q_weight = source.get(spec.q_norm, dtype=torch.float32)
        self.k_weight = source.get(spec.k_norm, dtype=torch.float32)
        lq1, lk1, lq2, lk2 = (source.get(name, dtype=torch.float64).cpu() for name in (spec.lam_q1, spec.lam_k1, spec.lam_q2, spec.lam_k2))
        # one number a layer, formed once on the host
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + float(spec.diff)
        self.o_proj = Linear(source.get(spec.o_proj))
        self.position = build_part("position", spec.position, source, rt)
        self.rot = int(spec.position.rotary_dim) if spec.position is not None else 0
        self.window = int(spec.window)

    def cache_spec(self):
        return PagedRowsSpec(self.G * (2 * self.n + self.dv), self.window)

    def forward(self, x, ctx, cache):
        s, H, G, n, dv = self.spec, self.H, self.G, self.n, self.dv
        T = x.shape[0]
        bt = ctx.block_tables[cache.group]
        proj = self.qkv_proj(x, out_dtype=torch.float32)
        q = torch.empty((T, H * 2 * n), device=x.device, dtype=self.rt.dtype)
        table = self.position.table() if self.position is not None else None
        ops.diff_prepare(q, proj, self.bias, self.q_weight, self.k_weight, s.eps, table, ctx, bt, cache.tensor, H, G, n, dv, self.rot,
                         cache.page_size)
        out = torch.empty((T, H * dv), device=x.device, dtype=self.rt.dtype)
        ops.diff_attention(out, q, cache.tensor, ctx, bt, H, G, n, dv, cache.page_size, self.window, s.scale, self.lam, s.eps,
                           1.0 - float(s.diff))
        return self.o_proj(out, out_dtype=self.rt.dtype)


register_part("mixer", "diff_attention", DiffAttention)
