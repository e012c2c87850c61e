"""Typed configuration of the Felolorn decoder, read from its config.json keys.

A Felolorn model is a list of layers that may differ from one another.  The embedding is multiplied by a factor.
A layer has a norm before and after each of its two parts, and a gate on each part's output:

    a = N1(x);  x += N1b( mixer(a + conv(a)) * sigmoid(G1 a + g1) )
    b = N2(x);  x += N2b( ff(b) * sigmoid(G2 b + g2) )                    (the feed-forward may be absent)

conv is a short causal convolution over time on each channel (`canon.taps` taps; the last taps - 1 inputs of a
sequence are part of its state).  The mixer is latent attention without positions (queries through a latent of
their own, a sink per head in the softmax), lightning attention (a matrix state per head with a fixed decay) or
HGRN2 (a matrix state per head whose forget gate also decides what is written).  The feed-forward is routed
experts: sigmoid scores, a correction added for the choice only, the choice restricted to the best groups of
neighbouring experts, the chosen scores as weights.  The head is the embedding table (without its factor), and
the logits are bounded by c tanh(z / c).

config.json keys (every size and constant comes from here):

    architecture     "Felolorn"
    vocab, width     vocabulary and width of the residual stream
    norm.eps         epsilon of every RMS norm
    embedding.scale  factor on the embedded rows (default 1)
    canon.taps       taps of the input convolution (absent: no convolution)
    logit_softcap    c of the bound on the logits (absent: none)
    layers[i]        type "latent_attention": mixer {heads, dim, vdim, kv_rank, q_rank, scale}
                     type "lightning":        mixer {heads, dim, vdim, decay [..]}
                     type "hgrn2":            mixer {heads, dim, vdim}
                     mlp null | {kind "moe", expert {ff}, router {experts, top, groups {count, keep}}}

Tensor names: ``embed``, ``final.norm`` and per layer i ``l<i>.norm{1,1b,2,2b}``, ``l<i>.canon1``,
``l<i>.rg{1,2}`` with ``l<i>.rg{1,2}.b``; ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}``,
``l<i>.mix.{q,k,v,g,norm,o}`` or ``l<i>.mix.{q,f,f.b,lower,v,norm,o}``; ``l<i>.mlp.router``,
``l<i>.mlp.correction`` and ``l<i>.mlp.e<k>.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .registry import ConfigError, register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

# the design has no position encoding and no trained context length: the cache bounds a sequence
MAX_POSITIONS = 1 << 22

MIXER_TYPES = ("latent_attention", "lightning", "hgrn2")


def _need(d: Any, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"felolorn config: {where} needs {key!r}")
    return d[key]


def _pos_int(d: Any, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"felolorn config: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d: Any, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"felolorn config: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class MixerConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int = 0                     # latent attention
    q_rank: int = 0
    scale: float = 0.0
    decay: Tuple[float, ...] = ()        # lightning

    @classmethod
    def from_dict(cls, kind: str, d: Any, where: str) -> "MixerConfig":
        heads, dim, vdim = _pos_int(d, "heads", where), _pos_int(d, "dim", where), _pos_int(d, "vdim", where)
        if kind == "latent_attention":
            return cls(heads=heads, dim=dim, vdim=vdim, kv_rank=_pos_int(d, "kv_rank", where),
                       q_rank=_pos_int(d, "q_rank", where), scale=_number(d, "scale", where))
        if kind == "lightning":
            decay = _need(d, "decay", where)
            if not isinstance(decay, (list, tuple)) or len(decay) != heads:
                raise ConfigError(f"felolorn config: {where}.decay must list one number per head ({heads})")
            decay = tuple(float(a) for a in decay)
            if not all(0.0 <= a <= 1.0 for a in decay):
                raise ConfigError(f"felolorn config: {where}.decay values must lie in [0, 1]")
            return cls(heads=heads, dim=dim, vdim=vdim, decay=decay)
        return cls(heads=heads, dim=dim, vdim=vdim)

    def to_dict(self, kind: str) -> Dict[str, Any]:
        d: Dict[str, Any] = dict(heads=self.heads, dim=self.dim, vdim=self.vdim)
        if kind == "latent_attention":
            d.update(kv_rank=self.kv_rank, q_rank=self.q_rank, scale=self.scale)
        elif kind == "lightning":
            d["decay"] = list(self.decay)
        return d


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int
    groups: int = 1
    keep: int = 1

    @classmethod
    def from_dict(cls, d: Any, where: str) -> "ExpertsConfig":
        kind = _need(d, "kind", where)
        if kind != "moe":
            raise ConfigError(f"felolorn config: {where}.kind={kind!r} is not known (moe)")
        ex, ro = _need(d, "expert", where), _need(d, "router", where)
        experts, top = _pos_int(ro, "experts", where + ".router"), _pos_int(ro, "top", where + ".router")
        groups = keep = 1
        gr = ro.get("groups")
        if gr is not None:
            groups = _pos_int(gr, "count", where + ".router.groups")
            keep = _pos_int(gr, "keep", where + ".router.groups")
        if experts % groups or keep > groups:
            raise ConfigError(f"felolorn config: {where}.router: {experts} experts do not form {groups} equal groups "
                              f"of which {keep} are kept")
        if top > (experts // groups) * keep:
            raise ConfigError(f"felolorn config: {where}.router.top={top} exceeds the experts of the kept groups")
        return cls(ff=_pos_int(ex, "ff", where + ".expert"), experts=experts, top=top, groups=groups, keep=keep)

    def to_dict(self) -> Dict[str, Any]:
        return dict(kind="moe", expert=dict(ff=self.ff),
                    router=dict(experts=self.experts, top=self.top, groups=dict(count=self.groups, keep=self.keep)))


@dataclass(frozen=True)
class FelolornLayer:
    type: str
    mixer: MixerConfig
    mlp: Optional[ExpertsConfig]


@register_architecture("Felolorn", "felolorn")
@dataclass(frozen=True)
class FelolornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FelolornLayer, ...]
    embedding_scale: float = 1.0
    taps: int = 0                        # 0: no input convolution
    logit_softcap: float = 0.0           # 0: none
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FelolornConfig":
        raw = _need(d, "layers", "config")
        if not isinstance(raw, (list, tuple)) or not raw:
            raise ConfigError("felolorn config: 'layers' must be a non-empty list")
        layers: List[FelolornLayer] = []
        for i, ld in enumerate(raw):
            where = f"layers[{i}]"
            kind = _need(ld, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"felolorn config: {where}.type={kind!r} is not known ({', '.join(MIXER_TYPES)})")
            mixer = MixerConfig.from_dict(kind, _need(ld, "mixer", where), where + ".mixer")
            mlp = ld.get("mlp")
            layers.append(FelolornLayer(type=kind, mixer=mixer,
                                        mlp=None if mlp is None else ExpertsConfig.from_dict(mlp, where + ".mlp")))
        eps = _number(_need(d, "norm", "config"), "eps", "norm")
        if not eps > 0:
            raise ConfigError(f"felolorn config: norm.eps must be > 0, got {eps}")
        emb = d.get("embedding")
        scale = _number(emb, "scale", "embedding") if emb is not None else 1.0
        canon = d.get("canon")
        taps = _pos_int(canon, "taps", "canon") if canon is not None else 0
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or not cap > 0):
            raise ConfigError(f"felolorn config: logit_softcap must be a positive number, got {cap!r}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"), norm_eps=eps,
                   layers=tuple(layers), embedding_scale=scale, taps=taps, logit_softcap=float(cap or 0.0),
                   eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.05)))

    # ------------------------------------------------------------------ write
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": "Felolorn", "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(l.type),
                                         "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
        if self.taps:
            d["canon"] = {"taps": self.taps}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
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
        n = self.vocab * W + W
        for l in self.layers:
            m = l.mixer
            n += 2 * W + W * W + W + W * self.taps
            if l.type == "latent_attention":
                n += (m.q_rank + m.kv_rank) * (W + 1) + m.heads * m.dim * (m.q_rank + m.kv_rank)
                n += m.heads * m.vdim * (m.kv_rank + W) + m.heads
            elif l.type == "lightning":
                n += 2 * m.heads * m.dim * W + 3 * m.heads * m.vdim * W + m.heads * m.vdim
            else:
                n += 2 * m.heads * m.dim * (W + 1) + 2 * m.heads * m.vdim * W + m.vdim
            f = l.mlp
            if f is not None:
                n += 2 * W + W * W + W + f.experts * (3 * f.ff * W + W + 1)
        return n

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        """Bytes a token adds to the paged caches (the matrix states and convolution tails do not grow)."""
        return sum(l.mixer.kv_rank * itemsize for l in self.layers if l.type == "latent_attention")

    # ---------------------------------------------------------------- spec
    def _mixer(self, l: FelolornLayer, p: str) -> Dict[str, Any]:
        W, eps, m = self.width, self.norm_eps, l.mixer
        if l.type == "latent_attention":
            return dict(kind="latent_attention", prefix=p, params=dict(
                hidden_size=W, num_heads=m.heads, nope_dim=m.dim, rope_dim=0, value_dim=m.vdim, latent_dim=m.kv_rank,
                q_latent_dim=m.q_rank, scale=m.scale, window=None, latent_norm_eps=eps, sink=True,
                names=dict(q_down="dq", q_latent_norm="dq.norm", q="uq", down="dkv", latent_norm="dkv.norm", up_k="uk",
                           up_v="uv", sink="sink", out="o")))
        if l.type == "lightning":
            return dict(kind="lightning", prefix=p, params=dict(
                hidden_size=W, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, decay=list(m.decay), eps=eps,
                names=dict(q="q", k="k", v="v", g="g", norm="norm", o="o")))
        return dict(kind="hgrn2", prefix=p, params=dict(
            hidden_size=W, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, eps=eps,
            names=dict(q="q", f="f", f_bias="f.b", lower="lower", v="v", norm="norm", o="o")))

    def to_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        blocks: List[BlockSpec] = []

        def norm(p: str, name: str) -> PartSpec:
            return PartSpec(kind="rmsnorm", prefix=p, params=dict(size=W, eps=eps, tensor=name))

        def gate(p: str, name: str) -> PartSpec:
            return PartSpec(kind="sigmoid_gate", prefix=p, params=dict(in_size=W, out_size=W,
                                                                       names=dict(weight=name, bias=name + ".b")))

        for i, l in enumerate(self.layers):
            p = f"l{i}."
            inner = self._mixer(l, "mix.")
            if self.taps:
                mixer = PartSpec(kind="input_conv", prefix=p, params=dict(hidden_size=W, taps=self.taps, tensor="canon1",
                                                                          inner=inner))
            else:
                mixer = PartSpec(kind=inner["kind"], prefix=p + inner["prefix"], params=inner["params"])
            parts: Dict[str, PartSpec] = {"mixer": mixer, "mixer_norm": norm(p, "norm1"),
                                          "mixer_post_norm": norm(p, "norm1b"), "mixer_gate": gate(p, "rg1")}
            f = l.mlp
            if f is not None:
                ff = PartSpec(kind="routed_experts", prefix=p + "mlp.", params=dict(
                    hidden_size=W, intermediate_size=f.ff, num_experts=f.experts, top_k=f.top, score="sigmoid",
                    renormalize=False, weight_on="output", activation=dict(kind="silu_glu"), correction=True,
                    groups=dict(count=f.groups, keep=f.keep),
                    names=dict(router="router", correction="correction", expert="e{}.", gate="gate", up="up",
                               down="down")))
                parts.update(feed_forward=ff, feed_forward_norm=norm(p, "norm2"),
                             feed_forward_post_norm=norm(p, "norm2b"), feed_forward_gate=gate(p, "rg2"))
            blocks.append(BlockSpec("sandwich_norm", parts))
        spec = ModelSpec(
            architecture="Felolorn", vocab_size=self.vocab, hidden_size=W, max_positions=MAX_POSITIONS,
            blocks=tuple(blocks), schedule=default_schedule(len(blocks)),
            embedding=PartSpec(kind="embedding", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W,
                                                                        tensor="embed", scale=self.embedding_scale)),
            final_norm=PartSpec(kind="rmsnorm", prefix="final.", params=dict(size=W, eps=eps, tensor="norm")),
            head=PartSpec(kind="linear_head", prefix="", params=dict(vocab_size=self.vocab, hidden_size=W,
                                                                     tied_to="embed", tensor="head",
                                                                     softcap=self.logit_softcap or None)),
            stop_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec
