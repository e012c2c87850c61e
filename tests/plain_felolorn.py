"""A plain, slow restatement of the Felolorn decoder, one function per mechanism, on the CPU.

It shares no code with the package: tensors come in as a dict of torch tensors by name, the configuration as
the parsed config.json.  Everything is computed in the dtype of `x` (float64 in the tests), one whole sequence
at a time, with explicit loops where a loop is the clearest statement.

Notation: x [n, W] is the residual stream of one sequence, positions are 0..n-1.

    embedding:  x = E[token] * embedding.scale
    layer:      a = N1(x);  x <- x + N1b( mixer(a + conv(a)) * sigmoid(G1 a + g1) )
                b = N2(x);  x <- x + N2b( ff(b) * sigmoid(G2 b + g2) )          (ff may be absent)
    N(x; w):    x / sqrt(mean(x^2) + eps) * w
    conv(a)_t:  sum_j c[:, j] * a_(t - taps + 1 + j), zero before position 0 (per channel, over time)
    mixer:      latent attention with a sink, lightning attention, or HGRN2
    ff:         routed experts, chosen inside the best groups
    output:     z = E N(x; w_final);  logits = cap * tanh(z / cap)                      (z itself without a cap)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ----------------------------------------------------------------------------------------------- small pieces
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def wnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w.to(x.dtype)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def mat(w: Dict[str, torch.Tensor], name: str, like: torch.Tensor) -> torch.Tensor:
    return w[name].to(like.dtype)


# ----------------------------------------------------------------------------------------------- input convolution
def causal_taps(a: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """conv(a)_t = sum_j c[:, j] a_(t - taps + 1 + j): the last column of c meets the token itself."""
    n, taps = a.shape[0], c.shape[1]
    out = torch.zeros_like(a)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += c[:, j].to(a.dtype) * a[s]
    return out


# ----------------------------------------------------------------------------------------------- latent attention
def sink_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                           sink: torch.Tensor) -> torch.Tensor:
    """q, k [n, H, d], v [n, H, dv]; position i sees j <= i; the denominator also holds exp(sink_h)."""
    n, H, _ = q.shape
    out = torch.zeros(n, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        s0 = float(sink[h])
        for i in range(n):
            sc = (k[: i + 1, h] @ q[i, h]) * scale
            m = max(float(sc.max()), s0)
            e = torch.exp(sc - m)
            den = e.sum() + math.exp(s0 - m)
            out[i, h] = (e[:, None] * v[: i + 1, h]).sum(dim=0) / den
    return out


def latent_attention(a: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    n = a.shape[0]
    cq = wnorm(a @ mat(w, p + "dq", a).T, w[p + "dq.norm"], eps)
    q = (cq @ mat(w, p + "uq", a).T).view(n, H, d)
    c = wnorm(a @ mat(w, p + "dkv", a).T, w[p + "dkv.norm"], eps)
    k = (c @ mat(w, p + "uk", a).T).view(n, H, d)
    v = (c @ mat(w, p + "uv", a).T).view(n, H, dv)
    o = sink_softmax_attention(q, k, v, float(m["scale"]), w[p + "sink"].to(a.dtype))
    return o.reshape(n, H * dv) @ mat(w, p + "o", a).T


# ----------------------------------------------------------------------------------------------- lightning
def lightning(a: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; q, k, v through silu; all heads normed together."""
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    n = a.shape[0]
    q = silu(a @ mat(w, p + "q", a).T).view(n, H, d)
    k = silu(a @ mat(w, p + "k", a).T).view(n, H, d)
    v = silu(a @ mat(w, p + "v", a).T).view(n, H, dv)
    o = torch.zeros(n, H, dv, dtype=a.dtype)
    for h in range(H):
        S = torch.zeros(d, dv, dtype=a.dtype)
        g = float(m["decay"][h])
        for t in range(n):
            S = g * S + k[t, h][:, None] * v[t, h][None, :]
            o[t, h] = S.T @ q[t, h]
    y = wnorm(o.reshape(n, H * dv), w[p + "norm"], eps) * sigmoid(a @ mat(w, p + "g", a).T)
    return y @ mat(w, p + "o", a).T


# ----------------------------------------------------------------------------------------------- HGRN2
def hgrn2(a: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """f = l + (1 - l) sigmoid(W_f a + b); S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T; o_t = S_t^T q_t."""
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    n = a.shape[0]
    q = silu(a @ mat(w, p + "q", a).T).view(n, H, d)
    v = (a @ mat(w, p + "v", a).T).view(n, H, dv)
    low = w[p + "lower"].to(a.dtype)
    f = (low + (1.0 - low) * sigmoid(a @ mat(w, p + "f", a).T + w[p + "f.b"].to(a.dtype))).view(n, H, d)
    o = torch.zeros(n, H, dv, dtype=a.dtype)
    for h in range(H):
        S = torch.zeros(d, dv, dtype=a.dtype)
        for t in range(n):
            S = f[t, h][:, None] * S + (1.0 - f[t, h])[:, None] * v[t, h][None, :]
            o[t, h] = S.T @ q[t, h]
    o = wnorm(o, w[p + "norm"], eps)
    return o.reshape(n, H * dv) @ mat(w, p + "o", a).T


# ----------------------------------------------------------------------------------------------- routed experts
def choose_experts(s: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int) -> List[List[int]]:
    """For every token the `top` experts with the largest s + correction among the experts of the `keep` groups
    whose two largest s + correction sum highest (groups are equal runs of neighbours)."""
    n, E = s.shape
    per = E // groups
    chosen: List[List[int]] = []
    for t in range(n):
        c = [float(s[t, e]) + float(correction[e]) for e in range(E)]
        gs = []
        for g in range(groups):
            best = sorted(c[g * per:(g + 1) * per], reverse=True)[:2]
            gs.append(sum(best))
        kept = sorted(range(groups), key=lambda g: (-gs[g], g))[:keep]
        ok = [e for e in range(E) if e // per in kept]
        chosen.append(sorted(ok, key=lambda e: (-c[e], e))[:top])
    return chosen


def routed_experts(b: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    ro = f["router"]
    E, top = int(ro["experts"]), int(ro["top"])
    gr = ro.get("groups") or {}
    groups, keep = int(gr.get("count", 1)), int(gr.get("keep", gr.get("count", 1)))
    s = sigmoid(b @ mat(w, p + "router", b).T)
    chosen = choose_experts(s, w[p + "correction"].to(b.dtype), top, groups, keep)
    out = torch.zeros_like(b)
    for t in range(b.shape[0]):
        for e in chosen[t]:
            g = mat(w, f"{p}e{e}.gate", b) @ b[t]
            u = mat(w, f"{p}e{e}.up", b) @ b[t]
            out[t] += s[t, e] * (mat(w, f"{p}e{e}.down", b) @ (silu(g) * u))
    return out


# ----------------------------------------------------------------------------------------------- the model
MIXERS = {"latent_attention": latent_attention, "lightning": lightning, "hgrn2": hgrn2}


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict) -> torch.Tensor:
    L = cfg["layers"][i]
    eps = float(cfg["norm"]["eps"])
    p = f"l{i}."
    a = wnorm(x, w[p + "norm1"], eps)
    fed = a + causal_taps(a, w[p + "canon1"]) if (p + "canon1") in w else a
    y = MIXERS[L["type"]](fed, w, p + "mix.", L["mixer"], eps)
    y = y * sigmoid(a @ mat(w, p + "rg1", a).T + w[p + "rg1.b"].to(a.dtype))
    x = x + wnorm(y, w[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        b = wnorm(x, w[p + "norm2"], eps)
        y = routed_experts(b, w, p + "mlp.", L["mlp"])
        y = y * sigmoid(b @ mat(w, p + "rg2", b).T + w[p + "rg2.b"].to(b.dtype))
        x = x + wnorm(y, w[p + "norm2b"], eps)
    return x


def forward(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict, dtype=torch.float64,
            streams: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence; `streams`, if given, receives the residual stream after every layer."""
    E = w["embed"].to(dtype)
    x = E[torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i in range(len(cfg["layers"])):
        x = layer(x, w, i, cfg)
        if streams is not None:
            streams.append(x.clone())
    z = wnorm(x, w["final.norm"], float(cfg["norm"]["eps"])) @ E.T
    cap = cfg.get("logit_softcap")
    return float(cap) * torch.tanh(z / float(cap)) if cap else z
