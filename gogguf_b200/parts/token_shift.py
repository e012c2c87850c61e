"""A mixer behind a token shift: the inner mixer reads h_t + (h_(t-1) - h_t) * mu instead of h_t.

h is the float32 stream itself (this part is handed the stream's rows, not normed ones: `reads_stream`), mu a
stored vector of the stream's width, h_(-1) = 0.  What the shift keeps per sequence is the last row it saw (a
`StateRequest` beside the inner mixer's own request: the part's cache request is the pair, and it is handed the pair
of views), so prompts may come in portions and decoding goes on from them.  The mix is float32; the result is
rounded to the compute dtype for the inner mixer's first projection.

Spec parameters: hidden_size, tensor (the stored [hidden_size] vector, named relative to this part's prefix),
inner: {kind, params, prefix}.
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


@register_mixer("token_shift")
class TokenShiftMixer:
    reads_stream = True         # handed the float32 stream rows themselves

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        ps, mcls = _inner(spec)
        t = {ps.prefix + local: decl for local, decl in mcls.tensors(ps).items()}
        name = spec.get("tensor", "shift")
        if name in t:
            raise ValueError(f"token_shift: the inner mixer also declares the tensor {name!r}")
        t[name] = TensorDecl(shape=(spec["hidden_size"],), init="unit_interval")
        return t

    @classmethod
    def cache_request(cls, spec: PartSpec):
        ps, mcls = _inner(spec)
        own = StateRequest(shape=(int(spec["hidden_size"]),), dtype=torch.float32)
        inner = mcls.cache_request(ps)
        # one flat tuple: the shift's row first, then the inner mixer's request (its members, where it is a tuple)
        return (own,) + tuple(inner) if isinstance(inner, (tuple, list)) else (own, inner)

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.rt = rt
        self.hidden = int(spec["hidden_size"])
        self.mu = rt.vector(weights[spec.get("tensor", "shift")])
        ps, mcls = _inner(spec)
        own = {local: weights[ps.prefix + local] for local in mcls.tensors(ps) if ps.prefix + local in weights}
        self.inner = mcls(ps, own, rt)
        self._inner_many = isinstance(mcls.cache_request(ps), (tuple, list))
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

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache, writes_cache: bool = True) -> None:
        if not isinstance(cache, tuple) or len(cache) < 2:
            raise ValueError("token_shift: the shift's state and the inner mixer's cache are expected")
        if not writes_cache:
            raise ValueError("token_shift: a layer's last row cannot be read by another layer")
        if x.dtype != torch.float32:
            raise ValueError("token_shift: the float32 stream rows are expected")
        last = cache[0]
        view = tuple(cache[1:]) if self._inner_many else cache[1]
        fed = ctx.ws.get("token_shift_out", tuple(x.shape), self.rt.dtype)
        K.token_shift(x, fed, self.mu, last.state, ctx.cu_seqlens, ctx.slots, ctx.seq_of_token, ctx.n_tokens, ctx.n_seqs,
                      max_new=int(ctx.max_new))
        self.inner.forward(fed, residual, ctx, view, writes_cache)
