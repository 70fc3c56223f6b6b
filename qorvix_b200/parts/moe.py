"""Routed feed-forward (mixture of experts) with an optional shared expert.  The router runs in float32;
tokens are grouped by expert on the device, the experts' products run over the grouped rows, and one
kernel forms the weighted sum in token order, adds the shared expert (scaled by its per-token gate) and,
if given, the output of the part that ran beside it (csrc/moe.cu)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward
from .registry import build_part, register_part


class RoutedFeedForward(FeedForward):
    takes_addend = True            # forward(x, ctx, add=...) returns float32 with `add` summed in

    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.router = source.get(spec.router)
        names = [spec.expert_names(e) for e in range(spec.experts)]
        self.w_gate = torch.stack([source.get(g) for g, _, _ in names]).contiguous()      # [E, ff, d]
        self.w_up = torch.stack([source.get(u) for _, u, _ in names]).to(self.w_gate.dtype).contiguous()
        self.w_down = torch.stack([source.get(dn) for _, _, dn in names]).to(self.w_gate.dtype).contiguous()   # [E, d, ff]
        # bfloat16 with rows that start on 16 bytes: the tensor-core kernel, over matrices packed in 64 x 64 tiles
        # (the rows are then dropped)
        self.tensor_cores = (rt.dtype == torch.bfloat16 and self.w_gate.dtype == torch.bfloat16 and spec.hidden_size % 8 == 0
                             and spec.expert_ff % 8 == 0)
        if self.tensor_cores:
            self.w_gate, self.w_up, self.w_down = (ops.moe_pack_experts(w) for w in (self.w_gate, self.w_up, self.w_down))
        self.shared = build_part("feed_forward", spec.shared, source, rt)
        self.shared_gate = source.get(spec.shared_gate).to(self.router.dtype).reshape(-1) if spec.shared is not None else None

    def forward(self, x, ctx, add=None, add_scale=None, scale=None):
        s = self.spec
        T, d = x.shape
        dev = x.device
        R = T * s.top
        top_idx = torch.empty((T, s.top), device=dev, dtype=torch.int32)
        top_w = torch.empty((T, s.top), device=dev, dtype=torch.float32)
        gate = torch.empty(T, device=dev, dtype=torch.float32) if self.shared is not None else None
        ops.moe_route(top_idx, top_w, gate, x, self.router, self.shared_gate)
        tc = self.tensor_cores
        tile_rows = ops.moe_tile_rows(tc)
        ints = torch.empty(3 * R + 3 * ops.moe_max_tiles(R, s.experts, tile_rows), device=dev, dtype=torch.int32)
        row_token, slot_row, scratch, tiles = ints[:R], ints[R: 2 * R], ints[2 * R: 3 * R], ints[3 * R:]
        ops.moe_group(row_token, slot_row, tiles, top_idx, scratch, s.experts, tile_rows)
        act = torch.empty((R, s.expert_ff), device=dev, dtype=x.dtype)
        y = torch.empty((R, d), device=dev, dtype=torch.float32)
        if tc:
            ops.moe_experts_tc(True, act, x, self.w_gate, self.w_up, row_token, tiles)
            ops.moe_experts_tc(False, y, act, self.w_down, None, row_token, tiles)
        else:
            ops.moe_experts(True, act, x, self.w_gate, self.w_up, row_token, tiles)
            ops.moe_experts(False, y, act, self.w_down, None, row_token, tiles)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        delta = torch.empty((T, d), device=dev, dtype=torch.float32)
        ops.moe_combine(delta, add, y, slot_row, top_w, shared, gate, mix_scale=add_scale, ff_scale=scale)
        return delta


class TableRoutedFeedForward(FeedForward):
    """Small ungated experts chosen by a table over token ids (no router), each weighted 1/top, plus an optional shared
    expert that is added as it is.  Grouping, products and the sum are the routed feed-forward's kernels."""
    takes_addend = True

    def __init__(self, spec, source, rt):
        if spec.activation != "relu2":
            raise ValueError(f"unknown activation '{spec.activation}' (known: relu2)")
        self.spec, self.rt = spec, rt
        self.table = source.get(spec.table).to(torch.int32).contiguous()
        names = [spec.expert_names(e) for e in range(spec.experts)]
        self.w_up = torch.stack([source.get(u) for u, _ in names]).contiguous()                                # [E, ff, d]
        self.w_down = torch.stack([source.get(dn) for _, dn in names]).to(self.w_up.dtype).contiguous()        # [E, d, ff]
        self.tensor_cores = (rt.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and spec.hidden_size % 8 == 0
                             and spec.expert_ff % 8 == 0)
        if self.tensor_cores:
            self.w_up, self.w_down = ops.moe_pack_experts(self.w_up), ops.moe_pack_experts(self.w_down)
        self.shared = build_part("feed_forward", spec.shared, source, rt)

    def forward(self, x, ctx, add=None, add_scale=None, scale=None):
        s = self.spec
        T, d = x.shape
        dev = x.device
        R = T * s.top
        top_idx = torch.empty((T, s.top), device=dev, dtype=torch.int32)
        top_w = torch.empty((T, s.top), device=dev, dtype=torch.float32)
        ops.moe_route_table(top_idx, top_w, self.table, ctx.token_ids, s.experts)
        tc = self.tensor_cores
        tile_rows = ops.moe_tile_rows(tc)
        ints = torch.empty(3 * R + 3 * ops.moe_max_tiles(R, s.experts, tile_rows), device=dev, dtype=torch.int32)
        row_token, slot_row, scratch, tiles = ints[:R], ints[R: 2 * R], ints[2 * R: 3 * R], ints[3 * R:]
        ops.moe_group(row_token, slot_row, tiles, top_idx, scratch, s.experts, tile_rows)
        act = torch.empty((R, s.expert_ff), device=dev, dtype=x.dtype)
        y = torch.empty((R, d), device=dev, dtype=torch.float32)
        if tc:
            ops.moe_experts_tc(2, act, x, self.w_up, None, row_token, tiles)
            ops.moe_experts_tc(0, y, act, self.w_down, None, row_token, tiles)
        else:
            ops.moe_experts(2, act, x, self.w_up, None, row_token, tiles)
            ops.moe_experts(0, y, act, self.w_down, None, row_token, tiles)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        delta = torch.empty((T, d), device=dev, dtype=torch.float32)
        ops.moe_combine(delta, add, y, slot_row, top_w, shared, None, mix_scale=add_scale, ff_scale=scale)
        return delta


register_part("feed_forward", "moe", RoutedFeedForward)
register_part("feed_forward", "table_moe", TableRoutedFeedForward)
