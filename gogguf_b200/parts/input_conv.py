"""A mixer behind a short causal convolution of its input: the inner mixer reads h + conv(h) instead of h.

    conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j)        per channel over time, inside a sequence, zeros before
                                                            its start; the last tap meets the token itself

What the convolution keeps per sequence is the last taps - 1 input rows (a `StateRequest` beside the inner mixer's
own request: the part's cache request is the pair, and it is handed the pair of views), so prompts may come in
portions and decoding goes on from them.  The sums are float32; the result is rounded to the compute dtype for the
inner mixer's first projection.

Spec parameters: hidden_size, taps, tensor (the stored [hidden_size, taps] table, named relative to this part's
prefix), residual (default True: h + conv(h); False: conv(h) alone), inner: {kind, params, prefix}.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..cache.sequence_cache import StateRequest
from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Runtime, StepContext
from .registry import MIXERS, lookup, register_mixer


def _inner(spec: PartSpec) -> Tuple[PartSpec, type]:
    m = spec["inner"]
    ps = PartSpec(kind=m["kind"], params=dict(m.get("params") or {}), prefix=m.get("prefix", ""))
    return ps, lookup(MIXERS, ps.kind, "mixer")


@register_mixer("input_conv")
class InputConvMixer:
    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        ps, mcls = _inner(spec)
        t = {ps.prefix + local: decl for local, decl in mcls.tensors(ps).items()}
        name = spec.get("tensor", "conv.weight")
        if name in t:
            raise ValueError(f"input_conv: the inner mixer also declares the tensor {name!r}")
        t[name] = TensorDecl(shape=(spec["hidden_size"], spec["taps"]), init="small_normal")
        return t

    @classmethod
    def cache_request(cls, spec: PartSpec):
        ps, mcls = _inner(spec)
        taps, W = int(spec["taps"]), int(spec["hidden_size"])
        own = StateRequest(shape=(taps - 1, W), dtype=torch.float32) if taps > 1 else None
        return (own, mcls.cache_request(ps))

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden, self.taps = int(spec["hidden_size"]), int(spec["taps"])
        if self.taps < 1:
            raise ValueError("input_conv: taps must be at least 1")
        self.keep = 1.0 if spec.get("residual", True) else 0.0
        # stored [W, taps]; kept as float32 [taps, W], a tap's weights side by side
        self.weight = rt.vector(weights[spec.get("tensor", "conv.weight")]).t().contiguous()
        ps, mcls = _inner(spec)
        own = {local: weights[ps.prefix + local] for local in mcls.tensors(ps) if ps.prefix + local in weights}
        self.inner = mcls(ps, own, rt)
        take = getattr(self.inner, "scale_output", None)
        if take is not None:
            self.scale_output = take

    @property
    def capturable(self) -> bool:
        return getattr(self.inner, "capturable", True)

    def prepare(self, ctx: StepContext) -> None:
        prep = getattr(self.inner, "prepare", None)
        if prep is not None:
            prep(ctx)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache, writes_cache: bool = True) -> None:
        if not isinstance(cache, tuple) or len(cache) != 2:
            raise ValueError("input_conv: the convolution's state and the inner mixer's cache are expected")
        if not writes_cache:
            raise ValueError("input_conv: a layer's convolution state cannot be read by another layer")
        tail, view = cache
        fed = ctx.ws.get("input_conv_out", tuple(h.shape), h.dtype)
        K.short_conv(h, fed, self.weight, tail.state if tail is not None else None, ctx.cu_seqlens, ctx.slots,
                     ctx.seq_of_token, ctx.n_tokens, ctx.n_seqs, self.keep, max_new=int(ctx.max_new))
        self.inner.forward(fed, residual, ctx, view, writes_cache)
