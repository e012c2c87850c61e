"""Tiny Felolorn configurations for the tests, model folders made from them, and the plain implementation's view
of a folder.  The configurations differ from one another in every size, in the order of their layers and in their
constants; some take values that another model may happen to make equal or one."""
from __future__ import annotations

import copy
import os
from typing import Dict, List, Optional

import torch


def latent(heads, dim, vdim, kv_rank, q_rank, scale):
    return dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale)


def light(heads, dim, vdim, decay):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=list(decay))


def hgrn(heads, dim, vdim):
    return dict(heads=heads, dim=dim, vdim=vdim)


def moe(ff, experts, top, count=1, keep=1):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, groups=dict(count=count, keep=keep)))


def layer(kind, mixer, mlp):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def model(vocab, width, eps, scale, taps, cap, layers):
    d = dict(architecture="Felolorn", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=scale),
             layers=layers)
    if taps:
        d["canon"] = dict(taps=taps)
    if cap:
        d["logit_softcap"] = cap
    return d


# sizes no tensor-core kernel takes; four taps; three groups of which two are kept; head sizes that differ between
# queries and values; a layer without feed-forward; decays of one (nothing fades) and near zero
CASE_S = model(211, 80, 2e-6, 3.7, 4, 12.5, [
    layer("lightning", light(3, 24, 40, (0.9, 0.99, 1.0)), moe(40, 12, 2, 3, 2)),
    layer("latent_attention", latent(5, 12, 20, 44, 36, 0.21), moe(24, 6, 3, 2, 1)),
    layer("hgrn2", hgrn(2, 20, 36), None),
    layer("latent_attention", latent(3, 24, 8, 20, 52, 0.4), moe(40, 12, 2, 3, 2)),
    layer("hgrn2", hgrn(5, 8, 8), moe(16, 5, 5)),
    layer("lightning", light(1, 40, 24, (0.05,)), None),
])
# values that happen to be one or equal: one tap (no convolution state), one head, one expert of which one is taken,
# one group, a scale of one on the embedding and on the scores, equal head sizes, ranks equal to the width
CASE_ONE = model(97, 64, 1e-5, 1.0, 1, 0.0, [
    layer("latent_attention", latent(1, 16, 16, 64, 64, 1.0), moe(48, 1, 1)),
    layer("hgrn2", hgrn(1, 16, 16), moe(32, 4, 1, 4, 1)),
    layer("lightning", light(2, 16, 16, (1.0, 0.0)), None),
])
# sizes the tensor-core kernels take: wide products, head sizes of 64 and 128, latents of 128 and 64, experts whose
# rows lie on 16-byte boundaries; two taps
CASE_W = model(523, 256, 3e-6, 16.0, 2, 30.0, [
    layer("hgrn2", hgrn(2, 128, 64), moe(128, 8, 3, 4, 2)),
    layer("latent_attention", latent(4, 64, 64, 128, 64, 0.125), moe(64, 9, 2, 3, 3)),
    layer("lightning", light(4, 64, 128, (0.96, 0.99, 0.999, 0.9995)), moe(128, 8, 3, 4, 2)),
    layer("latent_attention", latent(8, 32, 32, 64, 128, 0.18), None),
])


def every_expert(cfg: dict) -> dict:
    """The same configuration with every expert chosen for every token (top = experts, every group kept).  The
    bfloat16 comparisons of whole models run on these: where the choice is among close scores, rounding alone may
    take another expert and change that token's row by far more than rounding; the choice itself is held exactly by
    the float32 runs and by the router's own test."""
    c = copy.deepcopy(cfg)
    for l in c["layers"]:
        if l["mlp"] is not None:
            ro = l["mlp"]["router"]
            ro["top"] = ro["experts"]
            ro["groups"]["keep"] = ro["groups"]["count"]
    return c


CASES = {"S": (CASE_S, 3), "ONE": (CASE_ONE, 4), "W": (CASE_W, 6)}
CASES.update({"SB": (every_expert(CASE_S), 3), "ONEB": (every_expert(CASE_ONE), 4), "WB": (every_expert(CASE_W), 6)})


def make_folder(tmp, name: str, store_dtype: str = "float32", std: float = 0.12, norm_std: float = 0.1) -> str:
    """Write case `name` with the product's random-weights mode; returns the folder."""
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import write_random_model
    cfg, seed = CASES[name]
    folder = os.path.join(str(tmp), f"felolorn_{name}_{store_dtype}_{std}")
    if not os.path.isdir(folder):
        write_random_model(config_from_dict(cfg), seed, folder, dtype=store_dtype, std=std, norm_std=norm_std)
    return folder


def plain_logits(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
                 dtype=torch.float64):
    import plain_felolorn as plain
    return plain.forward(tokens, w, cfg, dtype, layers_out)


def draw_case(seed: int) -> dict:
    """A configuration nobody chose: every size, the order of the layers and the constants from a seeded generator."""
    import random
    r = random.Random(seed)
    width = r.choice([8, 16, 24]) * r.choice([3, 5, 7, 9])

    def draw_mixer():
        kind = r.choice(["latent_attention", "lightning", "hgrn2"])
        H = r.choice([1, 2, 3, 5])
        dim, vdim = r.choice([4, 8, 20, 32, 64, 72]), r.choice([4, 8, 24, 32, 72])
        if kind == "latent_attention":
            return kind, latent(H, dim, vdim, r.choice([8, 24, 40, 64]), r.choice([8, 16, 56]), r.choice([0.05, 0.11, 0.3]))
        if kind == "lightning":
            return kind, light(H, dim, vdim, [r.choice([0.5, 0.9, 0.99, 0.999, 1.0]) for _ in range(H)])
        return kind, hgrn(H, dim, vdim)

    layers = []
    for _ in range(r.choice([1, 2, 3, 4, 5])):
        count = r.choice([1, 2, 3])
        per = r.choice([1, 2, 4])
        keep = r.randint(1, count)
        mlp = None if r.random() < 0.25 else moe(r.choice([8, 16, 40, 96]), count * per, r.randint(1, min(per * keep, 4)),
                                                  count, keep)
        kind, m = draw_mixer()
        layers.append(layer(kind, m, mlp))
    return model(r.choice([53, 211, 641, 1031]), width, r.choice([1e-6, 1e-5, 3e-4]), r.choice([1.0, 4.0, 11.3]),
                 r.choice([0, 1, 2, 3, 5]), r.choice([0.0, 8.0, 50.0]), layers)
