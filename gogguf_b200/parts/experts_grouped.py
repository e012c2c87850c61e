"""Routed experts on the tensor cores, for steps of many tokens: the (token, choice) pairs are sorted by expert
on the device, the experts' row ranges are read back (one small copy: such steps are prompts, which run eagerly),
and every expert that has rows runs its gate/up and down products through the tensor-core `Linear` on its range."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc.build import kernel
from .base import Linear, StepContext

MIN_PAIRS = 512       # below this the experts are reached through the index (nothing is read back)


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


class _Grouped:
    def __init__(self, part, gate_up: List[Linear], down: List[Linear]):
        self.part, self.gate_up, self.down = part, gate_up, down
        # (with identity outputs the pairs that chose one are filed under one more index, behind the experts)
        self.bins = part.E + (1 if getattr(part, "identity", 0) else 0)
        self._host = torch.empty(self.bins + 1, dtype=torch.int32, pin_memory=True)

    def takes(self, ctx: StepContext) -> bool:
        return (not ctx.decode and ctx.n_tokens * self.part.top >= MIN_PAIRS
                and not torch.cuda.is_current_stream_capturing())

    def run(self, h: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        p = self.part
        T, W, F, E, top = ctx.n_tokens, p.hidden, p.inter, p.E, p.top
        P = T * top
        ws = ctx.ws
        nb = self.bins
        if nb > E:
            # a choice without an expert (index -1) is sorted behind the experts; its rows get no product and are zeroed
            idx = torch.where(idx < 0, torch.full_like(idx, E), idx)
        offsets = ws.get("moe_offsets", (nb + 1,), torch.int32)
        cursor = ws.get("moe_cursor", (nb,), torch.int32)
        place = ws.get("moe_place", (P,), torch.int32)
        pair_of = ws.get("moe_pair_of", (P,), torch.int32)
        xs = ws.get("moe_rows_in", (P, W), torch.bfloat16)
        gu = ws.get("moe_gate_up", (P, 2 * F), torch.bfloat16)
        y = ws.get("moe_act_rows", (P, F), torch.bfloat16)
        out = ws.get("moe_rows_out", (P, W), torch.float32)
        kernel("moe", "gg_moe_sort")(idx.data_ptr(), P, nb, offsets.data_ptr(), place.data_ptr(), cursor.data_ptr(), _s())
        self._host.copy_(offsets, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        kernel("moe", "gg_moe_gather")(h.data_ptr(), wts.data_ptr(), place.data_ptr(), xs.data_ptr(), P, W, top,
                                       int(p.on_input), _s())
        if not p.on_input:
            kernel("moe", "gg_moe_invert")(place.data_ptr(), pair_of.data_ptr(), P, _s())
        done.synchronize()
        off = self._host.tolist()
        for e in range(E):
            n = off[e + 1] - off[e]
            if n:
                self.gate_up[e](xs[off[e]:off[e + 1]], gu[off[e]:off[e + 1]], m=n, ws=ws)
        kernel("moe", "gg_moe_glu_rows")(gu.data_ptr(), y.data_ptr(), P, F, p.limit, p.slope, p.up_offset, p.out_scale,
                                         wts.data_ptr(), 0 if p.on_input else pair_of.data_ptr(), _s())
        for e in range(E):
            n = off[e + 1] - off[e]
            if n:
                self.down[e](y[off[e]:off[e + 1]], out[off[e]:off[e + 1]], m=n, ws=ws)
        if nb > E and off[nb] > off[E]:
            out[off[E]:off[nb]].zero_()
        kernel("moe", "gg_moe_combine")(out.data_ptr(), place.data_ptr(), residual.data_ptr(), T, W, top,
                                        ctx.seq_of_token.data_ptr(), 0, _s())


def try_make(part) -> Optional[_Grouped]:
    """The sorted form for this part, or None when its matrices are outside what the tensor-core product takes."""
    E, F, W = part.E, part.inter, part.hidden
    if W % 8 or F % 8:
        return None
    gate_up = [Linear(part.w_gu[e].view(2 * F, W), part.rt) for e in range(E)]
    down = [Linear(part.w_d[e], part.rt) for e in range(E)]
    if not all(l.tensor_core for l in gate_up + down):
        return None
    return _Grouped(part, gate_up, down)
