"""A plain, slow restatement of the Dinuzen decoder, one function per mechanism, on the CPU.

It shares no code with the package: tensors come in as a dict of torch tensors by name, the configuration as
the parsed config.json.  Everything is computed in the dtype of `x` (float64 in the tests), one whole sequence
at a time, with explicit loops where a loop is the clearest statement.

Notation: x [n, W] is the stream of one sequence, positions 0..n-1; X_0 is the embedded sequence, X_(i+1) what
layer i leaves before the depth average.

    layer i:    h_t = x_t + (x_(t-1) - x_t) * shift                  (x_(-1) = 0; only the mixer reads h)
                x <- x + ls1 * GN(mixer(h); w1);   x <- x + ls2 * GN(ff(x); w2)      (ff may be absent)
                X_(i+1) = x;   x <- sum_(j <= i+1) dwa[j] X_j
    GN(y; w):   y cut into `norm.groups` equal runs, each divided by sqrt(mean(run^2) + eps), then times w
    mixer:      differential attention (optionally on an earlier layer's keys and values), RG-LRU, or Mamba-2
    ff:         W_down gelu(W_up x), or routed experts with identity experts and a gated shared expert
    output:     logits = head GN(x; w_final)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


# ----------------------------------------------------------------------------------------------- small pieces
def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0.0)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def mat(w: Dict[str, torch.Tensor], name: str, like: torch.Tensor) -> torch.Tensor:
    return w[name].to(like.dtype)


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_norm(y: torch.Tensor, w: Optional[torch.Tensor], groups: int, eps: float) -> torch.Tensor:
    """The last axis in `groups` equal runs, each over its own root mean square; then the weight, if any."""
    n = y.shape[-1]
    out = rms_unit(y.reshape(*y.shape[:-1], groups, n // groups), eps).reshape(y.shape)
    return out if w is None else out * w.to(y.dtype)


def causal_taps(a: torch.Tensor, c: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out_t = bias + sum_j c[:, j] a_(t - taps + 1 + j): the last column of c meets the token itself."""
    n, taps = a.shape[0], c.shape[1]
    out = bias.to(a.dtype).expand(n, -1).clone()
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += c[:, j].to(a.dtype) * a[s]
    return out


def token_shift(x: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    prev = torch.cat([torch.zeros_like(x[:1]), x[:-1]], dim=0)
    return x + (prev - x) * mu.to(x.dtype)


# ----------------------------------------------------------------------------------------------- rotation
def yarn_frequencies(rot: dict) -> Tuple[torch.Tensor, float]:
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_adjacent(v: torch.Tensor, rot: dict) -> torch.Tensor:
    """v [n, ..., d]: the pairs (2i, 2i + 1) of the first rot.dims elements turn by position * f_i."""
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(rot)
    n = v.shape[0]
    ang = torch.arange(n, dtype=torch.float64)[:, None] * f[None, :]
    shape = (n,) + (1,) * (v.dim() - 2) + (dims // 2,)
    c, s = (torch.cos(ang) * mag).to(v.dtype).reshape(shape), (torch.sin(ang) * mag).to(v.dtype).reshape(shape)
    out = v.clone()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------------------------- attention
def capped_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """q, k [n, d], v [n, dv] of one head and map; position i sees j <= i; scores bounded by cap tanh(s / cap)."""
    n = q.shape[0]
    out = torch.zeros(n, v.shape[-1], dtype=q.dtype)
    for i in range(n):
        sc = (k[: i + 1] @ q[i]) * scale
        if cap:
            sc = cap * torch.tanh(sc / cap)
        p = torch.softmax(sc, dim=0)
        out[i] = p @ v[: i + 1]
    return out


def attention_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """Keys [n, G, 2, d] as the cache holds them (normed, rotated) and values [n, G, dv]."""
    G, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    n = h.shape[0]
    k = (h @ mat(w, p + "k", h).T).reshape(n, G, 2, d)
    k = rotate_adjacent(rms_unit(k, eps) * w[p + "k.norm"].to(h.dtype), m["rot"])
    v = (h @ mat(w, p + "v", h).T).reshape(n, G, dv)
    return k, v


def differential_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, kv) -> torch.Tensor:
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    n = h.shape[0]
    k, v = kv
    q = (h @ mat(w, p + "q", h).T).reshape(n, H, 2, d)
    q = rotate_adjacent(rms_unit(q, eps) * w[p + "q.norm"].to(h.dtype), m["rot"])
    diff = float(m["diff"])
    lam = (math.exp(float((w[p + "lq1"].double() * w[p + "lk1"].double()).sum()))
           - math.exp(float((w[p + "lq2"].double() * w[p + "lk2"].double()).sum())) + diff)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a1 = capped_softmax_attention(q[:, hh, 0], k[:, g, 0], v[:, g], float(m["scale"]), float(m.get("softcap") or 0.0))
        a2 = capped_softmax_attention(q[:, hh, 1], k[:, g, 1], v[:, g], float(m["scale"]), float(m.get("softcap") or 0.0))
        heads.append(rms_unit(a1 - lam * a2, eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1) @ mat(w, p + "o", h).T


# ----------------------------------------------------------------------------------------------- RG-LRU
def rglru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    Wr, nb = int(m["width"]), int(m["blocks"])
    n = h.shape[0]
    y = gelu_tanh(h @ mat(w, p + "y", h).T + w[p + "y.b"].to(h.dtype))
    u = causal_taps(h @ mat(w, p + "x", h).T + w[p + "x.b"].to(h.dtype), w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(n, nb, Wr // nb)
    r = sigmoid(torch.einsum("boi,nbi->nbo", mat(w, p + "ra", h), ub) + w[p + "ra.b"].to(h.dtype)).reshape(n, Wr)
    i = sigmoid(torch.einsum("boi,nbi->nbo", mat(w, p + "ri", h), ub) + w[p + "ri.b"].to(h.dtype)).reshape(n, Wr)
    log_a = -8.0 * r * softplus(w[p + "lam"].to(h.dtype))
    a = torch.exp(log_a)
    S = torch.zeros(Wr, dtype=h.dtype)
    out = torch.zeros(n, Wr, dtype=h.dtype)
    for t in range(n):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ mat(w, p + "o", h).T


# ----------------------------------------------------------------------------------------------- Mamba-2
def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    H, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * P
    n = h.shape[0]
    zx = h @ mat(w, p + "in", h).T
    z, xbc, dt = zx[:, :inner], zx[:, inner:2 * inner + 2 * G * N], zx[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_taps(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(n, H, P)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + w[p + "dt_bias"].to(h.dtype))
    A = -torch.exp(w[p + "A_log"].to(h.dtype))
    D = w[p + "D"].to(h.dtype)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(n, H, P, dtype=h.dtype)
    for t in range(n):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = torch.exp(A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + D[hh] * x[t, hh]
    y = y.reshape(n, inner) * silu(z)
    y = group_norm(y, w[p + "norm"], int(m["norm_groups"]), eps)
    return y @ mat(w, p + "o", h).T


# ----------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_erf(x @ mat(w, p + "up", x).T) @ mat(w, p + "down", x).T


def gated_unit(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(x @ mat(w, p + "gate", x).T) * (x @ mat(w, p + "up", x).T)) @ mat(w, p + "down", x).T


def route(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, ro: dict):
    """Chosen outputs [n, top] (ties to the lower index) and their weights."""
    s = torch.softmax(x @ mat(w, p + "router", x).T, dim=-1)
    choice = s + w[p + "correction"].to(x.dtype)
    top = int(ro["top"])
    idx = torch.zeros(x.shape[0], top, dtype=torch.long)
    for t in range(x.shape[0]):
        order = sorted(range(choice.shape[1]), key=lambda e: (-float(choice[t, e]), e))
        idx[t] = torch.tensor(order[:top])
    picked = torch.gather(s, 1, idx)
    return idx, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20) * float(ro["scale"])


def routed_ff(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    ro = f["router"]
    E = int(ro["experts"])
    idx, wts = route(x, w, p, ro)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for c in range(idx.shape[1]):
            e = int(idx[t, c])
            ye = gated_unit(x[t:t + 1], w, f"{p}e{e}.")[0] if e < E else x[t]      # the last outputs: identity
            out[t] += wts[t, c] * ye
    if f.get("shared"):
        gate = sigmoid(x @ mat(w, p + "shared.sg", x).T)
        out = out + gate * gated_unit(x, w, p + "shared.")
    return out


# ----------------------------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [n, vocab] of one sequence; `layers_out` collects the stream after every layer."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
    x = w["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    hist = [x]
    kvs: Dict[int, tuple] = {}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        h = token_shift(x, w[p + "shift"])
        if l["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kvs[i] = attention_keys_values(h, w, p + "mix.", m, eps)
            y = differential_attention(h, w, p + "mix.", m, eps, kvs[i if src is None else int(src)])
        elif l["type"] == "rglru":
            y = rglru(h, w, p + "mix.", m)
        elif l["type"] == "mamba2":
            y = mamba2(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(l["type"])
        x = x + group_norm(y, w[p + "norm1"], groups, eps) * w[p + "ls1"].to(dtype)
        f = l.get("mlp")
        if f is not None:
            y = dense_ff(x, w, p + "mlp.") if f["kind"] == "dense" else routed_ff(x, w, p + "mlp.", f)
            x = x + group_norm(y, w[p + "norm2"], groups, eps) * w[p + "ls2"].to(dtype)
        hist.append(x)
        a = w[p + "dwa"].to(dtype)
        x = sum(a[j] * hist[j] for j in range(len(hist)))
        if layers_out is not None:
            layers_out.append(x)
    return group_norm(x, w["final.norm"], groups, eps) @ w["head"].to(dtype).T
