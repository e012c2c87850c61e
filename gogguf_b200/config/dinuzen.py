"""Typed configuration of the Dinuzen decoder, read from its config.json keys.

A Dinuzen model is a list of layers that may differ from one another.  A layer norms the output of each of its two
parts, not their input, and scales it element by element:

    h_t = x_t + (x_(t-1) - x_t) * shift            (what the mixer reads; x_(-1) = 0)
    x <- x + ls1 * GN(mixer(h); norm1);   x <- x + ls2 * GN(ff(x); norm2)          (the feed-forward may be absent)
    X_(i+1) = x;   x <- sum_(j <= i+1) dwa_i[j] X_j                                 (X_0: the embedded rows)

GN is an RMS norm in `norm.groups` equal runs of the row.  The mixer is differential attention (two softmax maps
per head over shared values, q/k normed per head and map, a partial rotation in adjacent pairs with stretched
frequencies, bounded scores; a layer may read an earlier layer's keys and values), the recurrent block with a
real-gated linear recurrent unit, or Mamba-2.  The feed-forward is W_down gelu(W_up x) or routed experts (softmax
scores, a correction for the choice only, renormalised and scaled weights, identity experts, a shared expert
behind one sigmoid gate per token).  The output is the norm in groups, then a head matrix of its own.

config.json keys (every size and constant comes from here):

    architecture     "Dinuzen"
    vocab, width     vocabulary and width of the stream
    norm.eps, norm.groups
    layers[i]        type "attention": mixer {heads, kv_heads, dim, vdim, scale, softcap, diff, rot {dims, base,
                                              scaling {factor, original, fast, slow}}, kv_from}
                     type "rglru":     mixer {width, blocks, conv}
                     type "mamba2":    mixer {heads, vdim, state, groups, norm_groups, conv}
                     mlp null | {kind "dense", ff}
                              | {kind "moe", expert {ff}, router {experts, identity, top, scale}, shared {ff}}

Tensor names: ``embed``, ``final.norm``, ``head`` and per layer i ``l<i>.{norm1,norm2,ls1,ls2,shift,dwa}``;
``l<i>.mix.{q,k,v,q.norm,k.norm,lq1,lk1,lq2,lk2,o}``, ``l<i>.mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}`` or
``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}``; ``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router,correction}``,
``l<i>.mlp.e<k>.{gate,up,down}`` and ``l<i>.mlp.shared.{gate,up,down,sg}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

# the rotation has no trained limit that the design enforces: the cache bounds a sequence
MAX_POSITIONS = 1 << 22

MIXER_TYPES = ("attention", "rglru", "mamba2")


def _need(d: Any, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"dinuzen config: {where} needs {key!r}")
    return d[key]


def _pos_int(d: Any, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"dinuzen config: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _count(d: Any, key: str, where: str, default: int = 0) -> int:
    if not isinstance(d, dict) or d.get(key) is None:
        return default
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"dinuzen config: {where}.{key} must be a count, got {v!r}")
    return v


def _number(d: Any, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"dinuzen config: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "RotationConfig":
        dims = _count(d, "dims", where)
        if dims % 2:
            raise ConfigError(f"dinuzen config: {where}.dims must be even, got {dims}")
        sc = d.get("scaling") if isinstance(d, dict) else None
        scaling = None
        if sc is not None:
            scaling = tuple(_number(sc, k, where + ".scaling") for k in ("factor", "original", "fast", "slow"))
        base = _number(d, "base", where) if dims or (isinstance(d, dict) and d.get("base") is not None) else 0.0
        if dims and not base > 1.0:
            raise ConfigError(f"dinuzen config: {where}.base must be above one, got {base}")
        return cls(dims=dims, base=base, scaling=scaling)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = dict(dims=self.dims, base=self.base)
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d

    def position_spec(self) -> Optional[Dict[str, Any]]:
        if not self.dims:
            return None
        if self.scaling is None:
            return dict(kind="rope_adjacent", theta=self.base, rotary_dim=self.dims)
        f, o, fa, sl = self.scaling
        return dict(kind="rope_yarn_adjacent", theta=self.base, rotary_dim=self.dims, factor=f, original=o, fast=fa, slow=sl)


@dataclass(frozen=True)
class MixerConfig:
    # attention
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 0.0
    softcap: float = 0.0
    diff: float = 0.0
    rot: Optional[RotationConfig] = None
    kv_from: Optional[int] = None
    # rglru
    width: int = 0
    blocks: int = 0
    # mamba2 (heads and vdim above)
    state: int = 0
    groups: int = 0
    norm_groups: int = 0
    # both recurrences
    conv: int = 0

    @classmethod
    def from_dict(cls, kind: str, d: Any, where: str) -> "MixerConfig":
        if kind == "attention":
            src = d.get("kv_from") if isinstance(d, dict) else None
            if src is not None and (isinstance(src, bool) or not isinstance(src, int) or src < 0):
                raise ConfigError(f"dinuzen config: {where}.kv_from must name a layer, got {src!r}")
            cap = d.get("softcap")
            if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
                raise ConfigError(f"dinuzen config: {where}.softcap must be a number >= 0, got {cap!r}")
            heads, kv = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
            if heads % kv:
                raise ConfigError(f"dinuzen config: {where}: {heads} heads are not a multiple of {kv} kv_heads")
            rot = (RotationConfig.from_dict(d["rot"], where + ".rot") if d.get("rot") is not None
                   else RotationConfig(dims=0, base=0.0))       # no rotation where the layer names none
            dim = _pos_int(d, "dim", where)
            if rot.dims > dim:
                raise ConfigError(f"dinuzen config: {where}.rot.dims={rot.dims} exceeds dim={dim}")
            return cls(heads=heads, kv_heads=kv, dim=dim, vdim=_pos_int(d, "vdim", where),
                       scale=_number(d, "scale", where), softcap=float(cap or 0.0), diff=_number(d, "diff", where),
                       rot=rot, kv_from=src)
        if kind == "rglru":
            width, blocks = _pos_int(d, "width", where), _pos_int(d, "blocks", where)
            if width % blocks:
                raise ConfigError(f"dinuzen config: {where}: a width of {width} does not form {blocks} equal blocks")
            return cls(width=width, blocks=blocks, conv=_pos_int(d, "conv", where))
        heads, groups = _pos_int(d, "heads", where), _pos_int(d, "groups", where)
        vdim = _pos_int(d, "vdim", where)
        ng = _pos_int(d, "norm_groups", where) if d.get("norm_groups") is not None else 1
        if heads % groups:
            raise ConfigError(f"dinuzen config: {where}: {heads} heads do not form {groups} equal groups")
        if (heads * vdim) % ng:
            raise ConfigError(f"dinuzen config: {where}: {heads * vdim} outputs do not form {ng} equal norm groups")
        return cls(heads=heads, vdim=vdim, state=_pos_int(d, "state", where), groups=groups, norm_groups=ng,
                   conv=_pos_int(d, "conv", where))

    def to_dict(self, kind: str) -> Dict[str, Any]:
        if kind == "attention":
            d: Dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                                     softcap=self.softcap, diff=self.diff, rot=self.rot.to_dict())
            if self.kv_from is not None:
                d["kv_from"] = self.kv_from
            return d
        if kind == "rglru":
            return dict(width=self.width, blocks=self.blocks, conv=self.conv)
        return dict(heads=self.heads, vdim=self.vdim, state=self.state, groups=self.groups, norm_groups=self.norm_groups,
                    conv=self.conv)


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                 # "dense" or "moe"
    ff: int                   # the dense layer's, or an expert's, inner width
    experts: int = 0
    identity: int = 0
    top: int = 0
    scale: float = 1.0
    shared_ff: int = 0        # 0: no shared expert

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "FeedForwardConfig":
        kind = _need(d, "kind", where)
        if kind == "dense":
            return cls(kind="dense", ff=_pos_int(d, "ff", where))
        if kind != "moe":
            raise ConfigError(f"dinuzen config: {where}.kind={kind!r} is not known (dense, moe)")
        ex, ro = _need(d, "expert", where), _need(d, "router", where)
        experts, top = _pos_int(ro, "experts", where + ".router"), _pos_int(ro, "top", where + ".router")
        identity = _count(ro, "identity", where + ".router")
        if top > experts + identity:
            raise ConfigError(f"dinuzen config: {where}.router.top={top} exceeds its {experts + identity} outputs")
        scale = _number(ro, "scale", where + ".router") if ro.get("scale") is not None else 1.0
        sh = d.get("shared")
        return cls(kind="moe", ff=_pos_int(ex, "ff", where + ".expert"), experts=experts, identity=identity, top=top,
                   scale=scale, shared_ff=_pos_int(sh, "ff", where + ".shared") if sh is not None else 0)

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return dict(kind="dense", ff=self.ff)
        d: Dict[str, Any] = dict(kind="moe", expert=dict(ff=self.ff),
                                 router=dict(experts=self.experts, identity=self.identity, top=self.top, scale=self.scale))
        if self.shared_ff:
            d["shared"] = dict(ff=self.shared_ff)
        return d


@dataclass(frozen=True)
class DinuzenLayer:
    type: str
    mixer: MixerConfig
    mlp: Optional[FeedForwardConfig]


@register_architecture("Dinuzen", "dinuzen")
@dataclass(frozen=True)
class DinuzenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[DinuzenLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DinuzenConfig":
        raw = _need(d, "layers", "config")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("dinuzen config: 'layers' must be a non-empty list")
        layers: List[DinuzenLayer] = []
        for i, ld in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(ld, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"dinuzen config: {where}.type={kind!r} is not known ({', '.join(MIXER_TYPES)})")
            mixer = MixerConfig.from_dict(kind, _need(ld, "mixer", where), where + ".mixer")
            if mixer.kv_from is not None:
                j = mixer.kv_from
                src = layers[j] if j < i else None
                if src is None or src.type != "attention" or src.mixer.kv_from is not None:
                    raise ConfigError(f"dinuzen config: {where}.mixer.kv_from={j} must name an earlier attention layer "
                                      "with keys and values of its own")
                a, b = mixer, src.mixer
                # (the keys come rotated as layer j rotated them; this layer's own `rot` turns its queries)
                if (a.kv_heads, a.dim, a.vdim) != (b.kv_heads, b.dim, b.vdim):
                    raise ConfigError(f"dinuzen config: {where}.mixer reads the keys and values of layer {j}; kv_heads, "
                                      "dim and vdim must equal that layer's")
            mlp = ld.get("mlp")
            layers.append(DinuzenLayer(type=kind, mixer=mixer,
                                       mlp=None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp")))
        norm = _need(d, "norm", "config")
        eps = _number(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"dinuzen config: norm.eps must be > 0, got {eps}")
        groups = _pos_int(norm, "groups", "norm") if norm.get("groups") is not None else 1
        width = _pos_int(d, "width", "config")
        if width % groups:
            raise ConfigError(f"dinuzen config: a width of {width} does not form {groups} equal norm groups")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=width, norm_eps=eps, norm_groups=groups,
                   layers=tuple(layers), eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.05)))

    # ------------------------------------------------------------------ write
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": "Dinuzen", "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(l.type),
                                         "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    # ------------------------------------------------------------- derived
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def parameter_count(self) -> int:
        W = self.width
        n = 2 * self.vocab * W + W
        for i, l in enumerate(self.layers):
            m = l.mixer
            n += 3 * W + (i + 2)                       # norm1, ls1, shift, dwa
            if l.type == "attention":
                n += m.heads * 2 * m.dim * W + W * m.heads * m.vdim + 5 * m.dim
                if m.kv_from is None:
                    n += m.kv_heads * (2 * m.dim + m.vdim) * W + m.dim
            elif l.type == "rglru":
                bw = m.width // m.blocks
                n += 3 * m.width * W + m.width * (m.conv + 6) + 2 * m.blocks * bw * bw
            else:
                inner, ch = m.heads * m.vdim, m.heads * m.vdim + 2 * m.groups * m.state
                n += (2 * inner + 2 * m.groups * m.state + m.heads) * W + ch * (m.conv + 1) + 3 * m.heads + inner + W * inner
            f = l.mlp
            if f is not None:
                n += 2 * W
                if f.kind == "dense":
                    n += 2 * f.ff * W
                else:
                    n += (f.experts + f.identity) * (W + 1) + f.experts * 3 * f.ff * W
                    if f.shared_ff:
                        n += 3 * f.shared_ff * W + W
        return n

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """Bytes a token adds to the paged caches (the recurrences' states and the shifts' rows do not grow)."""
        return sum(l.mixer.kv_heads * (2 * l.mixer.dim + l.mixer.vdim) * itemsize for l in self.layers
                   if l.type == "attention" and l.mixer.kv_from is None)

    # ---------------------------------------------------------------- spec
    def _mixer(self, l: DinuzenLayer, p: str) -> Dict[str, Any]:
        W, eps, m = self.width, self.norm_eps, l.mixer
        if l.type == "attention":
            params = dict(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                          scale=m.scale, softcap=m.softcap, diff=m.diff, eps=eps, position=m.rot.position_spec())
            if m.kv_from is not None:
                # schedule entry j is layer j; its request is the pair (the shift's row, the mixer's keys and values)
                params["kv_source"] = dict(entry=m.kv_from, member=1)
            return dict(kind="diff_attention", prefix=p, params=params)
        if l.type == "rglru":
            return dict(kind="rglru", prefix=p, params=dict(hidden_size=W, width=m.width, blocks=m.blocks, taps=m.conv))
        return dict(kind="mamba2", prefix=p, params=dict(hidden_size=W, num_heads=m.heads, value_dim=m.vdim,
                                                         state_dim=m.state, groups=m.groups, norm_groups=m.norm_groups,
                                                         taps=m.conv, eps=eps))

    def _feed_forward(self, f: FeedForwardConfig, p: str) -> PartSpec:
        W = self.width
        if f.kind == "dense":
            return PartSpec(kind="gelu_mlp", prefix=p, params=dict(hidden_size=W, intermediate_size=f.ff, approximate="none",
                                                                   names=dict(up="up", down="down")))
        params: Dict[str, Any] = dict(
            hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, identity=f.identity, top_k=f.top,
            score="softmax", renormalize=True, weight_scale=f.scale, weight_on="output",
            activation=dict(kind="silu_glu"), correction=True,
            names=dict(router="router", correction="correction", expert="e{}.", gate="gate", up="up", down="down"))
        if f.shared_ff:
            params["shared"] = dict(intermediate_size=f.shared_ff, prefix="shared.", row_gate=True,
                                    names=dict(gate="gate", up="up", down="down", row_gate="sg"))
        return PartSpec(kind="routed_experts", prefix=p, params=params)

    def to_spec(self) -> ModelSpec:
        W, eps, G = self.width, self.norm_eps, self.norm_groups
        blocks: List[BlockSpec] = []
        depth = len(self.layers)

        def norm(p: str, name: str, scale: Optional[str]) -> PartSpec:
            params = dict(size=W, eps=eps, groups=G, tensor=name)
            if scale:
                params["scale_tensor"] = scale
            return PartSpec(kind="group_rmsnorm", prefix=p, params=params)

        for i, l in enumerate(self.layers):
            p = f"l{i}."
            mixer = PartSpec(kind="token_shift", prefix=p, params=dict(hidden_size=W, tensor="shift",
                                                                       inner=self._mixer(l, "mix.")))
            parts: Dict[str, PartSpec] = {
                "mixer": mixer, "mixer_post_norm": norm(p, "norm1", "ls1"),
                "stream_mix": PartSpec(kind="depth_average", prefix=p, params=dict(index=i, depth=depth, tensor="dwa"))}
            if l.mlp is not None:
                parts.update(feed_forward=self._feed_forward(l.mlp, p + "mlp."),
                             feed_forward_post_norm=norm(p, "norm2", "ls2"))
            blocks.append(BlockSpec("post_norm", parts))
        spec = ModelSpec(
            architecture="Dinuzen", vocab_size=self.vocab, hidden_size=W, max_positions=MAX_POSITIONS,
            blocks=tuple(blocks), schedule=default_schedule(len(blocks)),
            embedding=PartSpec(kind="embedding", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W, tensor="embed")),
            final_norm=PartSpec(kind="group_rmsnorm", prefix="final.", params=dict(size=W, eps=eps, groups=G, tensor="norm")),
            head=PartSpec(kind="linear_head", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W, tensor="head")),
            stop_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec
