"""Dinuzen without a GPU: the configuration and its spec, tensor names, the caches a model asks for (a layer that
reads another layer's keys and values shares that store and nothing else), the plain implementation's own
consistency."""
import copy
import math

import pytest
import torch

import plain_dinuzen as plain
from dinuzen_cases import CASES, draw_case


def _cfg(d):
    from gogguf_b200.config import config_from_dict
    return config_from_dict(copy.deepcopy(d))


def _weights(d, seed=1, std=0.12):
    from gogguf_b200.engine.model import expected_tensors
    from gogguf_b200.weights.loader import random_tensors
    return random_tensors(expected_tensors(_cfg(d).to_spec()), seed, std, 0.1, dtype=torch.float32)


@pytest.mark.parametrize("name", sorted(CASES))
def test_config_round_trip_and_spec(name):
    from gogguf_b200.engine.model import expected_tensors
    d = CASES[name][0]
    cfg = _cfg(d)
    assert cfg.to_dict() == d
    spec = cfg.to_spec()
    assert len(spec.schedule) == len(spec.blocks) == len(d["layers"])
    names = set(n for n, t in expected_tensors(spec).items() if not t.optional)
    assert {"embed", "final.norm", "head"} <= names
    for i, l in enumerate(d["layers"]):
        p = f"l{i}."
        assert {p + "norm1", p + "ls1", p + "shift", p + "dwa"} <= names
        for n in ("norm2", "ls2"):
            assert (p + n in names) == (l["mlp"] is not None)
        m = l["mixer"]
        own = {"rglru": {"y", "y.b", "x", "x.b", "conv", "conv.b", "ra", "ra.b", "ri", "ri.b", "lam", "o"},
               "mamba2": {"in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o"},
               "attention": {"q", "q.norm", "lq1", "lk1", "lq2", "lk2", "o"}
               | (set() if m.get("kv_from") is not None else {"k", "v", "k.norm"})}
        assert {n[len(p) + 4:] for n in names if n.startswith(p + "mix.")} == own[l["type"]]
        f = l["mlp"]
        if f is not None and f["kind"] == "moe":
            assert {p + "mlp.router", p + "mlp.correction"} <= names
            assert (p + "mlp.shared.sg" in names) == ("shared" in f)
            assert (p + f"mlp.e{f['router']['experts'] - 1}.down" in names) and (p + f"mlp.e{f['router']['experts']}.down" not in names)
    assert cfg.parameter_count() == sum(int(torch.tensor(t.shape).prod()) for t in expected_tensors(spec).values()
                                        if not t.optional)


def test_shapes_follow_the_configuration():
    from gogguf_b200.engine.model import expected_tensors
    t = expected_tensors(_cfg(CASES["S"][0]).to_spec())
    assert t["l0.mix.in"].shape == (2 * 72 + 2 * 3 * 20 + 3, 80) and t["l0.mix.conv"].shape == (72 + 120, 3)
    assert t["l0.mix.norm"].shape == (72,) and t["l0.mix.A_log"].shape == (3,) and t["l0.dwa"].shape == (2,)
    assert t["l1.mix.q"].shape == (6 * 2 * 12, 80) and t["l1.mix.k"].shape == (2 * 2 * 12, 80) and t["l1.mix.v"].shape == (40, 80)
    assert t["l1.mix.q.norm"].shape == (12,) and t["l1.mix.lk2"].shape == (12,) and t["l1.mix.o"].shape == (80, 120)
    assert t["l2.mix.ra"].shape == (3, 20, 20) and t["l2.mix.ri.b"].shape == (3, 20) and t["l2.mix.conv"].shape == (60, 4)
    assert t["l3.mix.q"].shape == (4 * 2 * 12, 80) and "l3.mix.k" not in t and t["l6.dwa"].shape == (8,)
    assert t["l0.mlp.router"].shape == (7, 80) and t["l0.mlp.correction"].shape == (7,) and t["l0.mlp.shared.sg"].shape == (1, 80)
    assert t["l4.mlp.e1.gate"].shape == (16, 80) and t["l1.mlp.up"].shape == (56, 80)


@pytest.mark.parametrize("bad", [
    lambda d: d["layers"][0].update(type="other"),
    lambda d: d["layers"][1]["mixer"].update(kv_heads=4),                      # 6 heads over 4 kv heads
    lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14),                  # beyond the head
    lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7),
    lambda d: d["layers"][3]["mixer"].update(kv_from=2),                       # not an attention layer
    lambda d: d["layers"][3]["mixer"].update(kv_from=3),                       # not an earlier layer
    lambda d: d["layers"][3]["mixer"].update(vdim=24),                         # another size than its source's
    lambda d: d["layers"][2]["mixer"].update(blocks=7),
    lambda d: d["layers"][0]["mixer"].update(groups=2),
    lambda d: d["layers"][0]["mixer"].update(norm_groups=5),
    lambda d: d["layers"][0]["mlp"]["router"].update(top=8),
    lambda d: d["layers"][0]["mlp"].update(kind="other"),
    lambda d: d["norm"].update(groups=3),
    lambda d: d["norm"].pop("eps"),
    lambda d: d.pop("layers"),
])
def test_a_configuration_that_cannot_be_is_refused(bad):
    from gogguf_b200.config import ConfigError
    d = copy.deepcopy(CASES["S"][0])
    bad(d)
    with pytest.raises(ConfigError):
        _cfg(d)


def test_a_layer_that_borrows_keys_and_values_shares_that_store_and_nothing_else():
    from gogguf_b200.cache import KVRequest, SequenceCache, SharedView, StateRequest
    from gogguf_b200.engine.model import _cache_part
    spec = _cfg(CASES["S"][0]).to_spec()
    reqs = []
    for b in spec.blocks:
        ps, cls = _cache_part(b)
        reqs.append(cls.cache_request(ps))
    assert isinstance(reqs[3][1], SharedView) and reqs[3][1].entry == 1 and reqs[3][1].member == 1
    assert reqs[1][1] == KVRequest(num_kv_heads=2, head_dim=24, window=None, value_dim=20)
    assert reqs[2] == (StateRequest((80,)), StateRequest((3, 60)), StateRequest((60,)))
    cache = SequenceCache(reqs, [None] * len(reqs), max_tokens=256, dtype=torch.float32, device="cpu")
    v1, v3, v4 = cache.view(1), cache.view(3), cache.view(4)
    assert v3[1].k.data_ptr() == v1[1].k.data_ptr() and v3[1].v.data_ptr() == v1[1].v.data_ptr()
    assert v3[0].state.data_ptr() != v1[0].state.data_ptr()            # the shift's row is the layer's own
    assert v4[1].k.data_ptr() != v1[1].k.data_ptr()
    assert len(cache.groups) == 2                                        # two layers write keys: two paged stores
    a, b = cache.open(), cache.open()
    cache.plan([a, b], [70, 3]); cache.commit([a, b], [70, 3])
    cache.close(a)
    c = cache.open()
    cache.plan([c], [130]); cache.commit([c], [130])
    cache.check()
    with pytest.raises(Exception):
        SequenceCache([reqs[3]], [None], max_tokens=64, dtype=torch.float32, device="cpu")   # nothing to borrow from


def test_the_plain_implementation_is_consistent_with_itself():
    d, _ = CASES["S"]
    w = _weights(d)
    tokens = [int(t) for t in torch.randint(0, d["vocab"], (40,), generator=torch.Generator().manual_seed(5))]
    full = plain.forward(d, w, tokens)
    assert torch.isfinite(full).all()
    # a prefix stands alone: nothing looks ahead
    assert torch.allclose(plain.forward(d, w, tokens[:17]), full[:17], rtol=0, atol=1e-10)
    # float32 tracks float64
    f32 = plain.forward(d, w, tokens, torch.float32).double()
    assert float((f32 - full).abs().max() / full.abs().max()) < 2e-4


def test_facts_of_the_mechanisms():
    x = torch.randn(6, 12, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    # the norm in groups: every run has unit mean square; with one group it is the plain norm
    y = plain.group_norm(x, None, 3, 0.0).reshape(6, 3, 4)
    assert torch.allclose((y * y).mean(-1), torch.ones(6, 3, dtype=torch.float64))
    assert torch.allclose(plain.group_norm(x, None, 1, 1e-6), plain.rms_unit(x, 1e-6))
    # the shift: mu = 0 leaves the rows, mu = 1 hands every token the row before (zeros for the first)
    assert torch.equal(plain.token_shift(x, torch.zeros(12)), x)
    s = plain.token_shift(x, torch.ones(12))
    assert torch.allclose(s[1:], x[:-1]) and float(s[0].abs().max()) == 0.0
    # rotation: position 0 is the identity up to the magnitude, pairs are neighbours, the rest passes
    r = dict(dims=4, base=100.0)
    v = torch.randn(3, 2, 6, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    o = plain.rotate_adjacent(v, r)
    assert torch.allclose(o[0], v[0]) and torch.allclose(o[..., 4:], v[..., 4:])
    a = 1.0 * 100.0 ** (-2.0 / 4)                                   # pair 1 at position 1
    assert torch.allclose(o[1, 0, 2], v[1, 0, 2] * math.cos(a) - v[1, 0, 3] * math.sin(a))
    f, mag = plain.yarn_frequencies(dict(dims=8, base=10000.0, scaling=dict(factor=4.0, original=64, fast=16.0, slow=2.0)))
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0) and float(f[0]) == 1.0 and float(f[-1]) == pytest.approx(10000.0 ** -0.75 / 4)
    # attention over one key returns its value whatever the score; the bound is the identity for small scores
    q, k, val = torch.randn(1, 4, dtype=torch.float64), torch.randn(1, 4, dtype=torch.float64), torch.randn(1, 5, dtype=torch.float64)
    assert torch.allclose(plain.capped_softmax_attention(q, k, val, 0.7, 3.0), val)
    # identity experts: a router that always picks the identity output with weight one gives the input back
    W = 8
    w = {"r.router": torch.tensor([[0.0] * W, [0.0] * W]), "r.correction": torch.tensor([-5.0, 5.0]),
         "r.e0.gate": torch.randn(4, W), "r.e0.up": torch.randn(4, W), "r.e0.down": torch.randn(W, 4)}
    f = dict(kind="moe", expert=dict(ff=4), router=dict(experts=1, identity=1, top=1, scale=3.0))
    xx = torch.randn(5, W, dtype=torch.float64)
    assert torch.allclose(plain.routed_ff(xx, w, "r.", f), 3.0 * xx)
    # a recurrence with a = exp(-8 sigmoid(.) softplus(lam)): a very negative lam keeps the state
    assert float(plain.softplus(torch.tensor(-30.0, dtype=torch.float64))) < 1e-12


@pytest.mark.parametrize("seed", range(6))
def test_drawn_configurations_are_valid(seed):
    from gogguf_b200.engine.model import expected_tensors
    d = draw_case(seed)
    cfg = _cfg(d)
    assert cfg.to_dict() == d
    t = expected_tensors(cfg.to_spec())
    assert cfg.parameter_count() == sum(int(torch.tensor(x.shape).prod()) for x in t.values() if not x.optional)
