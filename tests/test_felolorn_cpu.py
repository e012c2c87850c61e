"""Felolorn without a GPU: the configuration and its spec, tensor names, the caches a model asks for, the plain
implementation's own consistency."""
import copy

import pytest
import torch

import plain_felolorn as plain
from felolorn_cases import CASES, draw_case


def _cfg(d):
    from gogguf_b200.config import config_from_dict
    return config_from_dict(copy.deepcopy(d))


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_round_trip_and_spec(name):
    from gogguf_b200.engine.model import expected_tensors
    d = CASES[name][0]
    cfg = _cfg(d)
    assert cfg.to_dict() == d
    spec = cfg.to_spec()
    assert len(spec.schedule) == len(spec.blocks) == len(d["layers"])
    names = set(n for n, t in expected_tensors(spec).items() if not t.optional)
    assert {"embed", "final.norm"} <= names and "head" not in names          # the head is the embedding table
    for i, l in enumerate(d["layers"]):
        p = f"l{i}."
        assert {p + "norm1", p + "norm1b", p + "rg1", p + "rg1.b"} <= names
        assert (p + "canon1" in names) == ("canon" in d)
        for n in ("norm2", "norm2b", "rg2", "rg2.b", "mlp.router", "mlp.correction"):
            assert (p + n in names) == (l["mlp"] is not None)
        own = {"latent_attention": ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "sink", "o"),
               "lightning": ("q", "k", "v", "g", "norm", "o"), "hgrn2": ("q", "f", "f.b", "lower", "v", "norm", "o")}
        assert {n[len(p) + 4:] for n in names if n.startswith(p + "mix.")} == set(own[l["type"]])
    assert cfg.parameter_count() == sum(int(torch.tensor(t.shape).prod()) for t in expected_tensors(spec).values()
                                        if not t.optional)


def test_shapes_follow_the_configuration():
    from gogguf_b200.engine.model import expected_tensors
    t = expected_tensors(_cfg(CASES["S"][0]).to_spec())
    assert t["l0.canon1"].shape == (80, 4) and t["l0.rg1"].shape == (80, 80) and t["l1.rg2.b"].shape == (80,)
    assert t["l0.mix.norm"].shape == (3 * 40,) and t["l0.mix.g"].shape == (3 * 40, 80) and t["l0.mix.k"].shape == (3 * 24, 80)
    assert t["l1.mix.dq"].shape == (36, 80) and t["l1.mix.uq"].shape == (5 * 12, 36) and t["l1.mix.dkv.norm"].shape == (44,)
    assert t["l1.mix.uv"].shape == (5 * 20, 44) and t["l1.mix.sink"].shape == (5,) and t["l1.mix.o"].shape == (80, 100)
    assert t["l2.mix.norm"].shape == (36,) and t["l2.mix.lower"].shape == (2 * 20,) and t["l2.mix.f.b"].shape == (40,)
    assert t["l1.mlp.correction"].shape == (6,) and t["l0.mlp.e11.down"].shape == (80, 40)


@pytest.mark.parametrize("bad", [
    lambda d: d["layers"][0].update(type="other"),
    lambda d: d["layers"][0]["mixer"].update(decay=[0.5]),                     # one decay per head
    lambda d: d["layers"][0]["mixer"].update(decay=[0.5, 1.5, 0.2]),
    lambda d: d["layers"][1]["mixer"].pop("kv_rank"),
    lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=5),       # 12 experts in 5 groups
    lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=4),        # more kept than there are
    lambda d: d["layers"][1]["mlp"]["router"].update(top=4),                   # beyond the kept group's experts
    lambda d: d["layers"][0]["mlp"].update(kind="dense"),
    lambda d: d["canon"].update(taps=0),
    lambda d: d.update(logit_softcap=-1.0),
    lambda d: d["norm"].update(eps=0.0),
    lambda d: d.pop("layers"),
])
def test_bad_configurations_are_refused(bad):
    from gogguf_b200.config import ConfigError
    d = copy.deepcopy(CASES["S"][0])
    bad(d)
    with pytest.raises(ConfigError):
        _cfg(d)


def test_what_a_model_asks_of_the_cache():
    from gogguf_b200.cache.sequence_cache import LatentRequest, StateRequest
    from gogguf_b200.parts import registry as R
    spec = _cfg(CASES["S"][0]).to_spec()
    reqs = [R.MIXERS[b.mixer.kind].cache_request(b.mixer) for b in spec.blocks]
    for rq, l in zip(reqs, CASES["S"][0]["layers"]):
        tail, own = rq
        assert tail == StateRequest(shape=(3, 80), dtype=torch.float32)            # taps - 1 rows of the width
        m = l["mixer"]
        if l["type"] == "latent_attention":
            assert own == LatentRequest(width=m["kv_rank"], window=None)
        else:
            assert own == StateRequest(shape=(m["heads"], m["dim"], m["vdim"]), dtype=torch.float32)
    one = _cfg(CASES["ONE"][0]).to_spec()
    assert R.MIXERS[one.blocks[0].mixer.kind].cache_request(one.blocks[0].mixer)[0] is None   # one tap keeps nothing


def _weights(d, seed=0):
    from gogguf_b200.engine.model import expected_tensors
    from gogguf_b200.weights.loader import random_tensors
    return random_tensors(expected_tensors(_cfg(d).to_spec()), seed, 0.2, 0.1, dtype=torch.float32)


@pytest.mark.parametrize("seed", range(4))
def test_plain_prefix_stands_alone(seed):
    """The logits of a position do not depend on what follows it, for drawn configurations."""
    d = draw_case(seed)
    w = _weights(d, seed)
    toks = [int(t) for t in torch.randint(0, d["vocab"], (23,), generator=torch.Generator().manual_seed(seed))]
    whole = plain.forward(toks, w, d)
    assert whole.shape == (23, d["vocab"])
    part = plain.forward(toks[:9], w, d)
    assert torch.allclose(whole[:9], part, rtol=1e-10, atol=1e-12)
    low = plain.forward(toks, w, d, torch.float32)
    assert torch.allclose(low.double(), whole, rtol=2e-3, atol=2e-3)
    cap = d.get("logit_softcap")
    if cap:
        assert float(whole.abs().max()) <= cap


def test_plain_pieces():
    a = torch.arange(12, dtype=torch.float64).view(6, 2) + 1
    c = torch.tensor([[0.5, 2.0, 3.0], [1.0, 0.0, -1.0]], dtype=torch.float64)
    y = plain.causal_taps(a, c)
    assert torch.equal(y[0], c[:, 2] * a[0])                                   # zeros before the start
    assert torch.equal(y[1], c[:, 2] * a[1] + c[:, 1] * a[0])
    assert torch.equal(y[5], c[:, 2] * a[5] + c[:, 1] * a[4] + c[:, 0] * a[3])
    # one key: the sink takes its share of the weight, and the value comes out scaled by the rest
    q = torch.ones(1, 1, 4, dtype=torch.float64)
    v = torch.tensor([[[2.0, -4.0]]], dtype=torch.float64)
    out = plain.sink_softmax_attention(q, q, v, 0.5, torch.tensor([2.0], dtype=torch.float64))
    assert torch.allclose(out[0, 0], v[0, 0] * 0.5)                           # exp(4 * 0.5) against exp(2)
    # the choice: scores with the correction, inside the kept groups; a negative choice score still beats a group left out
    s = torch.tensor([[0.9, 0.1, 0.2, 0.3, 0.8, 0.85]], dtype=torch.float64)
    corr = torch.tensor([-2.0, 0.0, 0.0, 0.4, 0.0, 0.0], dtype=torch.float64)
    assert plain.choose_experts(s, corr * 0, 2, 3, 3) == [[0, 5]]
    assert plain.choose_experts(s, corr, 2, 3, 3) == [[5, 4]]
    assert plain.choose_experts(s, corr, 2, 3, 1) == [[5, 4]]                 # groups (0,1), (2,3), (4,5): the last wins
    assert plain.choose_experts(s, corr * 0, 2, 3, 1) == [[5, 4]]             # 0.9 + 0.1 < 0.8 + 0.85
    assert plain.choose_experts(s, torch.tensor([0, 0, 0, 0, -3.0, -3.0]).double(), 2, 3, 2) == [[0, 3]]
