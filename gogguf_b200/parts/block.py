"""Block arrangements: how a mixer, a feed-forward and their norms are wired around the residual."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import BlockSpec
from ..csrc import kernels as K
from .base import RowStats, Runtime, StepContext
from .registry import register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x)) (pkg/model/qwen3/model.go:198-288).
    The residual stream x is float32; the parts add their outputs into it."""

    # role -> family: what a block of this arrangement is made of (the builder builds exactly these)
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    keeps_row_stats = True      # clears RowStats.fresh itself before each write to the residual

    def __init__(self, spec: BlockSpec, parts: Dict[str, object], rt: Runtime):
        self.parts = dict(parts)
        mixer, feed_forward = parts["mixer"], parts["feed_forward"]
        mixer_norm, feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.rt = rt
        # A part may take its pre-norm into its first projection (`absorb_norm(norm) -> bool`); it then
        # gets the residual's RowStats as `h` instead of normalised rows, and the norm kernel does not run.
        self.mixer_folded = _offer_norm(mixer, mixer_norm, rt)
        self.feed_forward_folded = _offer_norm(feed_forward, feed_forward_norm, rt)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, writes_cache: bool) -> None:
        stats = ctx.shared.get("row_stats")
        if stats is None and (self.mixer_folded or self.feed_forward_folded):
            T, H = x.shape
            stats = ctx.shared["row_stats"] = RowStats(
                ctx.ws.get("residual_bf16", (T, H), torch.bfloat16),
                ctx.ws.get("residual_ssq", (T, (H + 127) // 128), torch.float32))
        h = self._input(self.mixer_folded, self.mixer_norm, x, ctx, stats)
        self.mixer.forward(h, x, ctx, cache, writes_cache)
        h = self._input(self.feed_forward_folded, self.feed_forward_norm, x, ctx, stats)
        self.feed_forward.forward(h, x, ctx)

    def _input(self, folded: bool, norm, x: torch.Tensor, ctx: StepContext, stats):
        if folded:
            h = stats.ensure(x)
        else:
            h = ctx.ws.get("block_normed", tuple(x.shape), self.rt.dtype)
            norm.forward(x, h)
        if stats is not None:
            stats.fresh = False        # the part is about to change the residual rows
        return h


@register_arrangement("parallel")
class ParallelBlock:
    """h = norm(x); x += mult * (mixer(h) + feed_forward(h)): one norm whose output both parts read, and a
    factor `residual_mult` (a parameter of the block spec, default 1) on what the block adds.  The
    feed-forward may be absent.  A part that has ``scale_output(mult) -> bool`` and accepts takes the factor
    into its own last product and adds straight into the residual stream; any other part is handed a zeroed
    float32 buffer and the block adds `mult` times that buffer itself."""

    roles = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    optional_roles = ("feed_forward",)

    def __init__(self, spec: BlockSpec, parts: Dict[str, object], rt: Runtime):
        self.parts = dict(parts)
        self.rt = rt
        self.norm, self.mixer = parts["norm"], parts["mixer"]
        self.feed_forward = parts.get("feed_forward")
        self.mult = float(spec.params.get("residual_mult", 1.0))
        self._direct = {}
        for role in ("mixer", "feed_forward"):
            part = parts.get(role)
            if part is None:
                continue
            take = getattr(part, "scale_output", None)
            self._direct[role] = self.mult == 1.0 or (take is not None and bool(take(self.mult)))

    def _run(self, role: str, x: torch.Tensor, ctx: StepContext, call) -> None:
        if self._direct[role]:
            call(x)
            return
        buf = ctx.ws.get("block_part_out", tuple(x.shape), torch.float32)
        buf.zero_()
        ctx.shared.pop("block_part_out_zeroed", None)      # (a mark other arrangements keep on this buffer)
        call(buf)
        K.residual_axpy(x, buf, self.mult)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, writes_cache: bool) -> None:
        h = ctx.ws.get("block_normed", tuple(x.shape), self.rt.dtype)
        self.norm.forward(x, h)
        self._run("mixer", x, ctx, lambda dst: self.mixer.forward(h, dst, ctx, cache, writes_cache))
        if self.feed_forward is not None:
            self._run("feed_forward", x, ctx, lambda dst: self.feed_forward.forward(h, dst, ctx))


@register_arrangement("sandwich_norm")
class SandwichNormBlock:
    """A norm on either side of each part: x += post1(mixer(pre1(x))); x += post2(feed_forward(pre2(x))).  The
    feed-forward (with its two norms) may be absent.  A part's output is collected in a zeroed float32 buffer;
    the norm after the part and the add into the residual stream are one kernel, all in float32.  The norms
    after the parts must be of the form y / rms(y) * weight (they expose `weight` and `eps`).

    A part may have a gate (roles mixer_gate, feed_forward_gate): the part's output is multiplied, element by
    element, by sigmoid(gate.logits(h) + gate.bias), h being the normed rows the part is handed, before the norm
    after the part: x += post(part(pre(x)) * gate(pre(x))).  The multiplication is done by the norm-and-add kernel."""

    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm", "feed_forward_post_norm": "norm", "mixer_gate": "gate",
             "feed_forward_gate": "gate"}
    optional_roles = ("feed_forward", "feed_forward_norm", "feed_forward_post_norm", "mixer_gate", "feed_forward_gate")
    keeps_row_stats = True      # its statistics are its own (see `forward`); it clears and sets `fresh` itself
    STATS = "sandwich_row_stats"
    ZEROED = "block_part_out_zeroed"      # ctx.shared: address of the parts' output buffer while it is known to hold zeros

    def __init__(self, spec: BlockSpec, parts: Dict[str, object], rt: Runtime):
        self.parts = dict(parts)
        self.rt = rt
        self.mixer, self.mixer_norm, self.mixer_post = parts["mixer"], parts["mixer_norm"], parts["mixer_post_norm"]
        self.feed_forward = parts.get("feed_forward")
        self.ff_norm, self.ff_post = parts.get("feed_forward_norm"), parts.get("feed_forward_post_norm")
        self.mixer_gate, self.ff_gate = parts.get("mixer_gate"), parts.get("feed_forward_gate")
        if self.ff_gate is not None and self.feed_forward is None:
            raise ValueError("sandwich_norm: a feed_forward_gate without a feed-forward")
        if self.feed_forward is not None and (self.ff_norm is None or self.ff_post is None):
            raise ValueError("sandwich_norm: a feed-forward needs feed_forward_norm and feed_forward_post_norm")
        for post in (self.mixer_post, self.ff_post):
            if post is not None and not getattr(post, "foldable", False):
                raise ValueError("sandwich_norm: the norm after a part must be y / rms(y) * weight")
        # A part may take the norm before it into its first projection (`absorb_norm(norm) -> bool`); it then reads
        # the residual's RowStats, which the norm-and-add kernel of the part before it has left behind.
        # (a gated part is handed the normed rows themselves: its gate reads them too)
        self.mixer_folded = self.mixer_gate is None and _offer_norm(self.mixer, self.mixer_norm, rt)
        self.ff_folded = (self.feed_forward is not None and self.ff_gate is None
                          and _offer_norm(self.feed_forward, self.ff_norm, rt))
        self.any_folded = self.mixer_folded or self.ff_folded

    def _part(self, x: torch.Tensor, ctx: StepContext, pre, post, call, folded: bool, stats, emit: bool,
              gate=None) -> None:
        if folded:
            h = stats.ensure(x)
        else:
            h = ctx.ws.get("block_normed", tuple(x.shape), self.rt.dtype)
            pre.forward(x, h)
        y = ctx.ws.get("block_part_out", tuple(x.shape), torch.float32)
        # the norm-and-add kernel leaves the buffer zeroed for the part that comes next; only the step's first part
        # (or one that follows a block of another make, which says so by dropping the mark) pays for a fill
        if ctx.shared.get(self.ZEROED) != y.data_ptr():
            y.zero_()
        g = gate.logits(h, ctx) if gate is not None else None
        gb = gate.bias if gate is not None else None
        call(h, y)
        if stats is not None and emit:
            K.rmsnorm_add(x, y, post.weight, post.eps, xhat=stats.xhat, ssq=stats.ssq, zero_y=True, gate=g, gate_bias=gb)
            stats.fresh = True
        else:
            K.rmsnorm_add(x, y, post.weight, post.eps, zero_y=True, gate=g, gate_bias=gb)
            if stats is not None:
                stats.fresh = False
        ctx.shared[self.ZEROED] = y.data_ptr()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, writes_cache: bool) -> None:
        # The statistics live under a key of this arrangement's own: a part's last product writes into the part's
        # output buffer here, not into the residual stream, and must not be offered the stream's statistics.
        stats = ctx.shared.get(self.STATS)
        if stats is None and self.any_folded:
            T, H = x.shape
            stats = ctx.shared[self.STATS] = RowStats(
                ctx.ws.get("residual_bf16", (T, H), torch.bfloat16),
                ctx.ws.get("residual_ssq", (T, (H + 127) // 128), torch.float32))
        # the norm-and-add after a part leaves the statistics where the part that comes next in this block reads them
        # folded; across blocks it always does (the next block may be of another make: it re-makes what is stale)
        self._part(x, ctx, self.mixer_norm, self.mixer_post,
                   lambda h, y: self.mixer.forward(h, y, ctx, cache, writes_cache), self.mixer_folded, stats,
                   emit=self.feed_forward is None or self.ff_folded, gate=self.mixer_gate)
        if self.feed_forward is not None:
            self._part(x, ctx, self.ff_norm, self.ff_post, lambda h, y: self.feed_forward.forward(h, y, ctx),
                       self.ff_folded, stats, emit=True, gate=self.ff_gate)


@register_arrangement("post_norm")
class PostNormBlock:
    """A norm on a part's output only: x += post1(mixer(x)); x += post2(feed_forward(x)).  The parts read the stream
    itself (rounded to the compute dtype; a mixer that declares ``reads_stream`` is handed the float32 rows).  A
    part's output is collected in a zeroed float32 buffer; the norm after the part and the add into the stream are
    one kernel, all in float32.  The norms expose `weight`, `eps` and, for a norm in groups, `groups`.  The
    feed-forward (with its norm) may be absent.  A `stream` part (role stream_mix, optional) runs before and after
    the block's parts on the stream as a whole."""

    roles = {"mixer": "mixer", "mixer_post_norm": "norm", "feed_forward": "feed_forward",
             "feed_forward_post_norm": "norm", "stream_mix": "stream"}
    optional_roles = ("feed_forward", "feed_forward_post_norm", "stream_mix")
    ZEROED = SandwichNormBlock.ZEROED

    def __init__(self, spec: BlockSpec, parts: Dict[str, object], rt: Runtime):
        self.parts = dict(parts)
        self.rt = rt
        self.mixer, self.mixer_post = parts["mixer"], parts["mixer_post_norm"]
        self.feed_forward, self.ff_post = parts.get("feed_forward"), parts.get("feed_forward_post_norm")
        self.stream = parts.get("stream_mix")
        if (self.feed_forward is None) != (self.ff_post is None):
            raise ValueError("post_norm: a feed-forward and feed_forward_post_norm come together")

    def _rows(self, x: torch.Tensor, ctx: StepContext, direct: bool) -> torch.Tensor:
        if direct or self.rt.dtype == torch.float32:
            return x
        h = ctx.ws.get("block_stream_rows", tuple(x.shape), self.rt.dtype)
        K.cast_rows(x, h)
        return h

    def _part(self, x: torch.Tensor, ctx: StepContext, post, call, direct: bool) -> None:
        y = ctx.ws.get("block_part_out", tuple(x.shape), torch.float32)
        if ctx.shared.get(self.ZEROED) != y.data_ptr():
            y.zero_()
        call(self._rows(x, ctx, direct), y)
        K.rmsnorm_add(x, y, post.weight, post.eps, zero_y=True, groups=int(getattr(post, "groups", 1)))
        ctx.shared[self.ZEROED] = y.data_ptr()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, writes_cache: bool) -> None:
        if self.stream is not None:
            self.stream.begin(x, ctx)
        self._part(x, ctx, self.mixer_post, lambda h, y: self.mixer.forward(h, y, ctx, cache, writes_cache),
                   bool(getattr(self.mixer, "reads_stream", False)))
        if self.feed_forward is not None:
            self._part(x, ctx, self.ff_post, lambda h, y: self.feed_forward.forward(h, y, ctx), False)
        if self.stream is not None:
            self.stream.finish(x, ctx)


def _offer_norm(part, norm, rt: Runtime) -> bool:
    absorb = getattr(part, "absorb_norm", None)
    if absorb is None or not (rt.fast and rt.fold_norms and rt.dtype == torch.bfloat16):
        return False
    if not getattr(norm, "foldable", False):
        return False
    return bool(absorb(norm))
