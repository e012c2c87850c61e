"""Tiny Dinuzen configurations for the tests, model folders made from them, and the plain implementation's view of
a folder.  The configurations differ from one another in every size, in the order of their layers and in their
constants; some take values that another model may happen to make equal or one."""
from __future__ import annotations

import copy
import os
from typing import Dict, List, Optional

import torch


def rot(dims, base, scaling=None):
    d = dict(dims=dims, base=base)
    if scaling is not None:
        d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def attn(heads, kv_heads, dim, vdim, scale, softcap, diff, rotation, kv_from=None):
    d = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=softcap, diff=diff, rot=rotation)
    if kv_from is not None:
        d["kv_from"] = kv_from
    return d


def lru(width, blocks, conv):
    return dict(width=width, blocks=blocks, conv=conv)


def ssm(heads, vdim, state, groups, norm_groups, conv):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, identity, top, scale, shared=0):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top, scale=scale))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def model(vocab, width, eps, groups, layers):
    return dict(architecture="Dinuzen", vocab=vocab, width=width, norm=dict(eps=eps, groups=groups), layers=layers)


ROT_S = rot(8, 10000.0, (4.0, 64, 16.0, 2.0))
# sizes no tensor-core kernel takes; three, four and two taps; five norm groups; a layer that reads another layer's
# keys and values with another number of query heads; layers without feed-forward, without identity experts,
# without a shared expert; a rotation of a part of the head with stretched frequencies, and a whole-head one without
CASE_S = model(211, 80, 2e-6, 5, [
    layer("mamba2", ssm(3, 24, 20, 3, 2, 3), moe(40, 5, 2, 3, 2.5, 24)),
    layer("attention", attn(6, 2, 12, 20, 0.3, 15.0, 0.3, ROT_S), dense(56)),
    layer("rglru", lru(60, 3, 4), None),
    layer("attention", attn(4, 2, 12, 20, 0.45, 6.0, 0.6, ROT_S, kv_from=1), moe(24, 6, 0, 2, 0.7)),
    layer("attention", attn(3, 3, 24, 8, 0.2, 0.0, 0.8, rot(24, 500.0)), moe(16, 2, 3, 2, 1.0, 40)),
    layer("rglru", lru(24, 1, 2), dense(100)),
    layer("mamba2", ssm(4, 8, 36, 1, 4, 2), None),
])
# values that happen to be one or equal: one norm group, one head, one kv head, equal key and value sizes, no
# rotation, one tap (no convolution state), one block, one expert of which one is taken, a weight scale of one, no
# difference constant, one group of states, one norm group after the scan
CASE_ONE = model(97, 64, 1e-5, 1, [
    layer("attention", attn(1, 1, 16, 16, 1.0, 0.0, 0.0, rot(0, 0.0)), moe(48, 1, 0, 1, 1.0)),
    layer("rglru", lru(64, 1, 1), dense(64)),
    layer("mamba2", ssm(1, 16, 16, 1, 1, 1), moe(32, 3, 1, 1, 1.0, 32)),
    layer("attention", attn(1, 1, 16, 16, 0.25, 30.0, 0.5, rot(0, 0.0), kv_from=0), None),
])
# sizes the tensor-core products take: wide matrices, rows on 16-byte boundaries
CASE_W = model(523, 384, 3e-6, 2, [
    layer("attention", attn(4, 2, 64, 64, 0.125, 20.0, 0.4, rot(32, 40000.0, (3.0, 256, 16.0, 1.0))), moe(128, 6, 2, 2, 1.5, 128)),
    layer("rglru", lru(256, 4, 4), dense(512)),
    layer("mamba2", ssm(4, 64, 64, 2, 2, 4), moe(64, 8, 0, 3, 2.0, 64)),
    layer("attention", attn(8, 2, 64, 64, 0.125, 20.0, 0.4, rot(32, 40000.0, (3.0, 256, 16.0, 1.0)), kv_from=0), dense(256)),
])


def every_expert(cfg: dict) -> dict:
    """The same configuration with every router output chosen for every token.  The bfloat16 comparisons of whole
    models run on these: where the choice is among close scores, rounding alone may take another expert and change
    that token's row by far more than rounding; the choice itself is held exactly by the float32 runs and by the
    router's own test."""
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        if l["mlp"] is not None and l["mlp"]["kind"] == "moe":
            ro = l["mlp"]["router"]
            ro["top"] = ro["experts"] + ro["identity"]
    return c


CASES = {"S": (CASE_S, 3), "ONE": (CASE_ONE, 4), "W": (CASE_W, 6)}
CASES.update({"SB": (every_expert(CASE_S), 3), "ONEB": (every_expert(CASE_ONE), 4), "WB": (every_expert(CASE_W), 6)})


def write_case(tmp, tag: str, cfg: dict, seed: int, store_dtype: str = "float32", std: float = 0.12,
               norm_std: float = 0.1) -> str:
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    folder = os.path.join(str(tmp), f"dinuzen_{tag}_{store_dtype}_{std}")
    if not os.path.isdir(folder):
        write_random_model(config_from_dict(cfg), seed, folder, dtype=store_dtype, std=std, norm_std=norm_std)
    return folder


def make_folder(tmp, name: str, store_dtype: str = "float32", std: float = 0.12, norm_std: float = 0.1) -> str:
    """Write case `name` with the product's random-weights mode; returns the folder."""
    cfg, seed = CASES[name]
    return write_case(tmp, name, cfg, seed, store_dtype, std, norm_std)


def plain_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
                 dtype=torch.float64):
    import plain_dinuzen as plain
    return plain.forward(cfg, w, tokens, dtype, layers_out)


def draw_case(seed: int) -> dict:
    """A configuration nobody chose: every size, the order of the layers and the constants from a seeded generator."""
    import random
    r = random.Random(seed)
    groups = r.choice([1, 2, 3, 4])
    width = groups * r.choice([8, 12, 20]) * r.choice([1, 2, 3])
    layers, owners = [], []

    def draw_rot(dim):
        dims = r.choice([0, 2, dim // 2 // 2 * 2, dim])
        sc = None if r.random() < 0.4 else (r.choice([1.5, 2.0, 8.0]), r.choice([32, 100, 512]), r.choice([8.0, 32.0]),
                                            r.choice([0.5, 1.0, 2.0]))
        return rot(dims, r.choice([100.0, 10000.0, 1e6]), sc)

    for i in range(r.choice([1, 2, 3, 4, 5])):
        kind = r.choice(["attention", "attention", "rglru", "mamba2"])
        if kind == "attention":
            if owners and r.random() < 0.4:
                j = r.choice(owners)
                src = layers[j]["mixer"]
                G = src["kv_heads"]
                m = attn(G * r.choice([1, 2, 3]), G, src["dim"], src["vdim"], r.choice([0.1, 0.3]), r.choice([0.0, 5.0, 30.0]),
                         r.choice([0.0, 0.2, 0.7]), src["rot"], kv_from=j)
            else:
                G, dim = r.choice([1, 2, 3]), r.choice([4, 8, 20, 32, 64])
                m = attn(G * r.choice([1, 2, 4]), G, dim, r.choice([4, 8, 24, 40, 64]), r.choice([0.1, 0.3, 1.0]),
                         r.choice([0.0, 5.0, 30.0]), r.choice([0.0, 0.2, 0.7]), draw_rot(dim))
                owners.append(i)
        elif kind == "rglru":
            nb = r.choice([1, 2, 3, 5])
            m = lru(nb * r.choice([4, 8, 24, 40]), nb, r.choice([1, 2, 4, 5]))
        else:
            G = r.choice([1, 2, 3])
            H, P = G * r.choice([1, 2]), r.choice([4, 8, 24, 40])
            ng = r.choice([g for g in (1, 2, 4, H) if (H * P) % g == 0])
            m = ssm(H, P, r.choice([4, 16, 24, 72]), G, ng, r.choice([1, 2, 4]))
        u = r.random()
        if u < 0.2:
            mlp = None
        elif u < 0.45:
            mlp = dense(r.choice([8, 40, 96]))
        else:
            E, I = r.choice([1, 2, 4, 7]), r.choice([0, 0, 1, 3])
            mlp = moe(r.choice([8, 16, 40]), E, I, r.randint(1, min(E + I, 4)), r.choice([1.0, 0.5, 2.5]),
                      r.choice([0, 8, 24]))
        layers.append(layer(kind, m, mlp))
    return model(r.choice([53, 211, 641]), width, r.choice([1e-6, 1e-5, 3e-4]), groups, layers)
