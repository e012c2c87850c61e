"""The Dinuzen decoder through the framework against the plain implementation (tests/plain_dinuzen.py): each
mechanism alone, whole prompts layer by layer, portions, decoding, unequal batches, reuse of slots, pages and states,
far keys and page borders made to stand out, the first tokens, other sizes, the entry point, the replay program."""
import math
import os

import pytest
import torch

import plain_dinuzen as plain
from dinuzen_cases import (CASES, attn, dense, draw_case, every_expert, layer, lru, make_folder, model, moe, plain_logits,
                           rot, ssm, write_case)
from helpers import random_tokens, read_folder, rel_err
from test_gpu_felolorn import close, load, run_cut

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5
DEV = "cuda:0"


def _K():
    from gogguf_b200.csrc import kernels
    return kernels


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _batch(lens):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    sot = [b for b, n in enumerate(lens) for _ in range(n)]
    return _i32(cu), _i32(sot), cu


def _gen(seed):
    return torch.Generator().manual_seed(seed)


# ----------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,lens", [(80, (37, 9, 1)), (256, (2, 130)), (24, (1, 1, 1))])
def test_token_shift_alone(dt, W, lens):
    """Whole, then continued by one token each: the row before a sequence's first row comes from its slot."""
    K = _K()
    g = _gen(W)
    mu = torch.rand(W, generator=g).to(DEV)
    slots = _i32([3, 0, 5][:len(lens)])
    state = torch.full((6, W), 7.0, device=DEV)
    state[slots.long()] = 0.0
    xs = [torch.randn(n + 1, W, generator=g, dtype=torch.float64) for n in lens]
    want = [plain.token_shift(x, mu.double().cpu()) for x in xs]
    cu, sot, _ = _batch(lens)
    x = torch.cat([x[:-1] for x in xs]).float().to(DEV)
    out = torch.empty(x.shape, dtype=dt, device=DEV)
    K.token_shift(x, out, mu, state, cu, slots, sot, x.shape[0], len(lens), max_new=max(lens))
    tol = 1e-6 if dt == torch.float32 else 1e-2
    assert rel_err(out, torch.cat([w[:-1] for w in want])) < tol
    cu1, sot1, _ = _batch([1] * len(lens))
    x1 = torch.stack([x[-1] for x in xs]).float().to(DEV)
    out1 = torch.empty(x1.shape, dtype=dt, device=DEV)
    K.token_shift(x1, out1, mu, state, cu1, slots, sot1, len(lens), len(lens), max_new=1)
    assert rel_err(out1, torch.stack([w[-1] for w in want])) < tol
    assert torch.equal(state[slots.long()], x1) and float(state[1, 0]) == 7.0          # other slots untouched


@pytest.mark.parametrize("H,groups", [(80, 5), (256, 4), (1024, 2), (100, 1), (24, 24)])
def test_norm_in_groups_of_a_parts_output_added_to_the_stream(H, groups):
    K = _K()
    g = _gen(H)
    x, y, w = torch.randn(9, H, generator=g), torch.randn(9, H, generator=g) * 3, torch.randn(H, generator=g)
    want = x.double() + plain.group_norm(y.double(), w, groups, 1e-5)
    xd, yd = x.to(DEV), y.to(DEV)
    K.rmsnorm_add(xd, yd, w.to(DEV), 1e-5, zero_y=True, groups=groups)
    assert rel_err(xd, want) < 2e-6 and float(yd.abs().max()) == 0.0
    out = torch.empty(4, H, dtype=torch.float32, device=DEV)
    K.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out, _i32([8, 0, 3, 3]), groups=groups)
    assert rel_err(out, plain.group_norm(x.double()[[8, 0, 3, 3]], w, groups, 1e-5)) < 2e-6


def test_weighted_sum_over_depth_alone():
    K = _K()
    g = _gen(1)
    T, W, L = 7, 40, 3
    hist = torch.zeros(L + 1, T, W, device=DEV)
    xs = [torch.randn(T, W, generator=g) for _ in range(L + 1)]
    cs = [torch.randn(i + 2, generator=g) for i in range(L)]
    x = xs[0].to(DEV).clone()
    K.depth_mix(hist, x, None, 0, 0)
    assert torch.equal(x.cpu(), xs[0])
    for i in range(L):
        x = xs[i + 1].to(DEV).clone()
        K.depth_mix(hist, x, cs[i].to(DEV), i + 1, i + 2)
        want = sum(cs[i][j].double() * xs[j].double() for j in range(i + 2))
        assert rel_err(x, want) < 2e-6
    assert torch.equal(hist.cpu(), torch.stack(xs))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,taps,act", [(60, 4, 0), (192, 3, 1), (64, 1, 1), (24, 2, 0), (256, 7, 1)])
def test_convolution_of_a_projections_columns_alone(dt, C, taps, act):
    """Columns of a wider buffer, with a bias on the input and one on the output; whole, then in portions, then a
    token each, from the states the portions left."""
    K = _K()
    g = _gen(C + taps)
    lens = (37, 9, 2)
    pad = 16
    w = torch.randn(C, taps, generator=g) * 0.5
    bias, in_bias = torch.randn(C, generator=g), torch.randn(C, generator=g) * 0.3
    hs = [torch.randn(n, C, generator=g).to(dt).double() for n in lens]
    want = [plain.causal_taps(h + in_bias.double(), w, bias) for h in hs]
    if act:
        want = [plain.silu(v) for v in want]
    slots = _i32([2, 0, 4])
    wt, bd, ibd = w.t().contiguous().to(DEV), bias.to(DEV), in_bias.to(DEV)

    def run(parts, state):
        n_seqs = len(parts)
        cu, sot, _ = _batch([p.shape[0] for p in parts])
        wide = torch.zeros(sum(p.shape[0] for p in parts), pad + C + 8, dtype=dt, device=DEV)
        wide[:, pad:pad + C] = torch.cat(parts).to(dt).to(DEV)
        out = torch.full((wide.shape[0], C + 8), 9.0, device=DEV)
        K.column_conv(wide[:, pad:pad + C], out[:, :C], wt, bd, ibd, state, cu, slots[:n_seqs], sot, wide.shape[0], n_seqs,
                      act=act, max_new=max(p.shape[0] for p in parts))
        assert float(out[:, C:].min()) == 9.0
        return out[:, :C].cpu()

    state = torch.zeros(6, max(taps - 1, 1), C, device=DEV) if taps > 1 else None
    tol = 3e-6
    got = run(hs, state)
    assert rel_err(got, torch.cat(want)) < tol
    if state is not None:
        state.zero_()
    a = run([h[:n - 1] for h, n in zip(hs[:2], lens)], state)          # portions of the first two, then one token each
    b = run([h[n - 1:] for h, n in zip(hs[:2], lens)], state)
    assert rel_err(a, torch.cat([v[:n - 1] for v, n in zip(want[:2], lens)])) < tol
    assert rel_err(b, torch.cat([v[n - 1:] for v, n in zip(want[:2], lens)])) < tol


@pytest.mark.parametrize("R,E,top,scale", [(7, 5, 3, 2.5), (6, 6, 2, 0.7), (5, 2, 2, 1.0), (1, 1, 1, 1.0), (12, 8, 12, 1.5), (40, 33, 4, 1.0)])
def test_choice_of_experts_with_identity_outputs_alone(R, E, top, scale):
    K = _K()
    g = _gen(R * top)
    T = 64
    z = torch.randn(T, R, generator=g) * 2
    corr = torch.randn(R, generator=g) * 0.1
    z[5] = 0.0                                       # equal scores: ties go to the lower index after the correction
    w = {"r.router": torch.eye(R), "r.correction": corr}
    idx_want, wts_want = plain.route(z.double(), w, "r.", dict(top=top, scale=scale))
    idx = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    K.moe_route(z.to(DEV), top, idx, wts, None, softmax=True, renormalize=True, correction=corr.to(DEV), n_real=E if E < R else 0,
                scale=scale)
    shown = torch.where(idx_want < E, idx_want, torch.full_like(idx_want, -1))
    assert torch.equal(idx.cpu().long(), shown)
    assert rel_err(wts, wts_want) < 1e-5
    # the identity outputs add the token's own row times their weights
    h = torch.randn(T, 24, generator=g)
    res = torch.zeros(T, 24, device=DEV)
    K.moe_identity(h.to(DEV), idx, wts, res, T, top, None)
    want = ((idx_want >= E).double() * wts_want).sum(-1, keepdim=True) * h.double()
    assert float((res.cpu().double() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("H,G,d,dv,window,cap", [(4, 1, 64, 128, 0, 20.0), (8, 2, 32, 64, 0, 0.0), (3, 3, 128, 128, 0, 30.0),
                                                  (6, 2, 64, 32, 70, 5.0), (5, 1, 32, 32, 0, 10.0), (16, 2, 64, 64, 129, 0.0)])
def test_differential_attention_on_the_tensor_cores_against_the_plain_kernel(H, G, d, dv, window, cap):
    """Both kernels on the same cache: prompts of unequal lengths, then portions that go on from the cache, then
    one token each; pages in no particular order; a window; heads that do not fill a tile evenly."""
    K = _K()
    g = _gen(H * d + dv)
    assert K.diff_attention_mma_takes(H, G, d, dv, 64)
    n_pages, ps = 40, 64
    kpool = (torch.randn(n_pages, G, ps, 2 * d, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    vpool = torch.randn(n_pages, G, ps, dv, generator=g).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(n_pages, generator=g).tolist()
    tables = [perm[0:8], perm[8:16], perm[16:24]]
    table = _i32(tables)
    done = [0, 0, 0]
    for lens in ((130, 1, 67), (65, 200, 2), (1, 1, 1), (2, 1, 3), (1, 1, 1)):
        cu, sot, cul = _batch(lens)
        T = sum(lens)
        pos = _i32([done[b] + i for b, n in enumerate(lens) for i in range(n)])
        q = torch.randn(T, H * 2 * d, generator=g).to(torch.bfloat16).to(DEV)
        a = torch.empty(T, H * dv, dtype=torch.bfloat16, device=DEV)
        b_ = torch.empty_like(a)
        K.diff_attention(q, kpool, vpool, a, pos, sot, table, ps, T, H, G, d, dv, 0.11, cap, window, 0.37, 1e-6, 0.8)
        K.diff_attention_mma(q, kpool, vpool, b_, pos, sot, cu, table, ps, T, 3, H, G, d, dv, 0.11, cap, window, 0.37, 1e-6, 0.8)
        # the same with every CTA's key tiles shared out over three CTAs and merged by the second kernel
        c_ = torch.empty_like(a)
        shares = torch.empty(K.diff_attention_partial_elems(T, H, dv, 3), device=DEV)
        K.diff_attention_mma(q, kpool, vpool, c_, pos, sot, cu, table, ps, T, 3, H, G, d, dv, 0.11, cap, window, 0.37, 1e-6, 0.8,
                             nsplit=3, partial=shares)
        assert float(((c_.float() - b_.float()).abs().max(dim=-1).values / a.float().abs().max()).max()) < 1.2e-2
        if max(lens) * (H // G) <= 16:
            # tiles of at most 16 rows (decode steps): the four warps share out every page's keys
            for ns in (1, 3):
                d_ = torch.empty_like(a)
                K.diff_attention_mma(q, kpool, vpool, d_, pos, sot, cu, table, ps, T, 3, H, G, d, dv, 0.11, cap, window, 0.37, 1e-6,
                                     0.8, nsplit=ns, partial=shares if ns > 1 else None, max_new=max(lens))
                assert float(((d_.float() - b_.float()).abs().max(dim=-1).values / a.float().abs().max()).max()) < 1.2e-2, ns
        err = (a.float() - b_.float()).abs().max(dim=-1).values / a.float().abs().max()
        assert float(err.max()) < 3e-2 and float(err.median()) < 1e-2, (float(err.max()), float(err.median()), lens)   # (an output rounds to 2^-8 of itself)
        done = [x + n for x, n in zip(done, lens)]
    # a padding row (a replayed batch smaller than its graph) gives zeros and reads nothing
    cu, sot, _ = _batch((1, 1))
    sot[1] = -1
    q = torch.randn(2, H * 2 * d, generator=g).to(torch.bfloat16).to(DEV)
    o = torch.full((2, H * dv), 5.0, dtype=torch.bfloat16, device=DEV)
    K.diff_attention_mma(q, kpool, vpool, o, _i32([done[0], 0]), sot, cu, table[:2].contiguous(), ps, 2, 2, H, G, d, dv, 0.11, cap,
                         window, 0.37, 1e-6, 0.8)
    assert float(o[1].abs().max()) == 0.0 and float(o[0].abs().max()) > 0.0


@pytest.mark.parametrize("C,lens", [(60, (200, 1, 64, 65)), (512, (129,)), (24, (63, 300))])
def test_vector_state_recurrence_in_chunks_against_row_by_row(C, lens):
    K = _K()
    g = _gen(C)
    T = sum(lens)
    cu, sot, _ = _batch(lens)
    slots = _i32([2, 0, 5, 3][:len(lens)])
    a = torch.rand(T, C, generator=g).pow(0.05).to(DEV)              # decays next to one: the state lives long
    b = torch.randn(T, C, generator=g).to(DEV)
    y = torch.randn(T, C + 8, generator=g).to(DEV)
    yb = torch.randn(C, generator=g).to(DEV)
    st0 = torch.randn(6, C, generator=g).to(DEV)
    st1, st2 = st0.clone(), st0.clone()
    o1, o2 = torch.empty(T, C, device=DEV), torch.empty(T, C, device=DEV)
    K.diag_scan(a, b, y[:, :C], yb, o1, st1, cu, slots, sot, T, len(lens))
    scratch = torch.empty(K.diag_scan_chunks_scratch(T, len(lens), C), device=DEV)
    K.diag_scan_chunks(a, b, y[:, :C], yb, o2, scratch, st2, cu, slots, sot, T, len(lens))
    assert rel_err(o2, o1) < 1e-5 and rel_err(st2, st1) < 1e-5
    assert torch.equal(st2[1], st0[1]) and torch.equal(st2[4], st0[4])          # other slots untouched


@pytest.mark.parametrize("H,G,N,P,lens", [(3, 3, 20, 24, (200, 1, 64, 65)), (4, 2, 128, 64, (129,)), (2, 1, 72, 40, (63, 300))])
def test_matrix_state_recurrence_with_step_sizes_in_chunks_against_row_by_row(H, G, N, P, lens):
    K = _K()
    g = _gen(H * N + P)
    T = sum(lens)
    cu, sot, _ = _batch(lens)
    slots = _i32([2, 0, 5, 3][:len(lens)])
    inner = H * P
    xc = torch.randn(T, inner + 2 * G * N, generator=g).to(DEV)
    xd = (torch.randn(T, H + 4, generator=g) - 2.0).to(DEV)          # small step sizes: slow decays
    dt_bias = torch.randn(H, generator=g).to(DEV) * 0.3
    neg_a = -torch.rand(H, generator=g).to(DEV)
    st0 = torch.randn(6, H, N, P, generator=g).to(DEV)
    st1, st2 = st0.clone(), st0.clone()
    r1, r2 = torch.empty(T, inner, device=DEV), torch.empty(T, inner, device=DEV)
    K.stepsize_scan(xc, inner, inner + G * N, xd, 4, r1, st1, cu, slots, sot, dt_bias, neg_a, T, len(lens), H, G, N, P)
    scratch = torch.empty(K.stepsize_scan_scratch(T, len(lens), H, N, P, 64), device=DEV)
    K.stepsize_scan(xc, inner, inner + G * N, xd, 4, r2, st2, cu, slots, sot, dt_bias, neg_a, T, len(lens), H, G, N, P,
                    chunk=64, scratch=scratch)
    assert rel_err(r2, r1) < 1e-5 and rel_err(st2, st1) < 1e-5
    assert torch.equal(st2[1], st0[1]) and torch.equal(st2[4], st0[4])


def _one_layer(kind, mixer, mlp=None, width=64, groups=2, vocab=61, eps=1e-5):
    return model(vocab, width, eps, groups, [layer(kind, mixer, mlp)])


ALONE = {
    "attention": _one_layer("attention", attn(6, 2, 12, 20, 0.3, 15.0, 0.3, rot(8, 10000.0, (4.0, 64, 16.0, 2.0)))),
    "attention_wide": _one_layer("attention", attn(4, 1, 64, 128, 0.125, 20.0, 0.5, rot(64, 1e6)), width=128),
    "attention_plain_scores": _one_layer("attention", attn(2, 2, 8, 8, 0.35, 0.0, 0.0, rot(0, 0.0))),
    "attention_long_values": _one_layer("attention", attn(2, 1, 24, 320, 0.2, 12.0, 0.1, rot(12, 3000.0))),
    "rglru": _one_layer("rglru", lru(60, 3, 4)),
    "rglru_wide": _one_layer("rglru", lru(512, 2, 4), width=128),
    "rglru_one": _one_layer("rglru", lru(40, 1, 1)),
    "mamba2": _one_layer("mamba2", ssm(3, 24, 20, 3, 2, 3)),
    "mamba2_wide": _one_layer("mamba2", ssm(4, 64, 128, 2, 4, 4), width=128),
    "mamba2_one": _one_layer("mamba2", ssm(1, 8, 8, 1, 1, 1)),
    "dense": _one_layer("rglru", lru(16, 1, 2), dense(100)),
    "experts": _one_layer("rglru", lru(16, 1, 2), moe(24, 5, 2, 3, 2.5, 40)),
    "experts_wide": _one_layer("rglru", lru(16, 1, 2), moe(64, 4, 1, 5, 1.5, 128), width=128),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_in_a_layer_of_its_own(tmp_path_factory, name, dtype):
    """A model of one layer: its mixer (or feed-forward) decides the layer's output.  Whole, cut, token by token."""
    cfg = ALONE[name]
    if dtype == "bfloat16":
        cfg = every_expert(cfg)
    folder = write_case(tmp_path_factory.getbasetemp(), "alone_" + name, cfg, 17, dtype, std=0.2)
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 140, seed=3)
    layers, layers32 = [], []
    want = plain_logits(cfg, w, tokens, layers)
    own32 = plain_logits(cfg, w, tokens, layers32, torch.float32)
    from gogguf_b200.engine import LayerTaps, StepEntry
    m, cache, st = load(folder, dtype)
    got_layers = []
    slot = cache.open()
    got = st.step([StepEntry(slot, tokens, want=list(range(len(tokens))))],
                  LayerTaps(on_layer=lambda i, rows: got_layers.append(rows.clone()))).clone()
    cache.close(slot)
    assert close(got_layers[0], layers[0], dtype, own32=layers32[0]), (rel_err(got_layers[0], layers[0]), name)
    assert close(got, want, dtype, own32=own32), (rel_err(got, want), name)
    for cuts in ([64, 2, 70], [1, 63, 1, 65], []):
        out = run_cut(st, cache, tokens if cuts else tokens[:70], cuts)
        ref = want if cuts else want[:70]
        assert close(out, ref, dtype, own32=own32[:ref.shape[0]], gauge=got[:ref.shape[0]]), (rel_err(out, ref), name, cuts)


# ----------------------------------------------------------------------------------------------- whole models
def _case(name, dtype):
    """bfloat16 runs of whole models take the configurations in which every expert is chosen (see `every_expert`)."""
    return name + "B" if dtype == "bfloat16" and name + "B" in CASES else name


@pytest.mark.parametrize("name", ["S", "ONE", "W"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_every_layer(tmp_path_factory, name, dtype):
    from gogguf_b200.engine import LayerTaps, StepEntry
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    m, cache, st = load(folder, dtype)
    for n in (1, 2, 3, 150):
        tokens = random_tokens(cfg["vocab"], n, seed=n)
        want_layers, layers32 = [], []
        want = plain_logits(cfg, w, tokens, want_layers)
        logits32 = plain_logits(cfg, w, tokens, layers32, torch.float32)
        got_layers = []
        slot = cache.open()
        got = st.step([StepEntry(slot, tokens, want=list(range(n)))],
                      LayerTaps(on_layer=lambda i, rows: got_layers.append(rows.clone()))).clone()
        cache.close(slot)
        assert len(got_layers) == len(cfg["layers"])
        for i, (a, b) in enumerate(zip(got_layers, want_layers)):
            assert close(a, b, dtype, own32=layers32[i]), (rel_err(a, b), name, n, "layer", i)
        assert close(got, want, dtype, own32=logits32), (rel_err(got, want), name, n)
    if dtype == "bfloat16":
        # the plain kernels on the same weights are the twins of the tensor-core kernels
        _, cache2, st2 = load(folder, dtype, fast=False)
        assert close(run_cut(st2, cache2, tokens, [len(tokens)]), want, dtype)


def test_sorted_form_of_the_experts_with_identity_outputs(tmp_path_factory, monkeypatch):
    """Long prompts of models with large experts sort the (token, choice) pairs by expert and run one tensor-core
    product per expert; choices of an identity output are filed behind the experts and get no product.  The
    threshold is lowered so that the test's small experts take that form."""
    from gogguf_b200.parts import experts
    monkeypatch.setattr(experts, "SORTED_FORM_MIN_WORK", 0.0)
    folder = make_folder(tmp_path_factory.getbasetemp(), "WB", "bfloat16")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 300, seed=21)
    want = plain_logits(cfg, w, tokens)
    m, cache, st = load(folder, "bfloat16")
    ff = m.blocks[0].feed_forward
    assert ff.identity == 2 and ff._grouped is not None
    got = run_cut(st, cache, tokens, [300])
    assert close(got, want, "bfloat16"), rel_err(got, want)
    monkeypatch.setattr(experts, "SORTED_FORM_MIN_WORK", 1e30)
    again = run_cut(st, cache, tokens, [300])
    assert close(again, want, "bfloat16", gauge=got), rel_err(again, want)


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("ONE", "float32"), ("W", "float32"),
                                        ("W", "bfloat16")])
def test_portions_and_decoding_equal_the_whole_prompt(tmp_path_factory, name, dtype):
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 171, seed=12)
    want = plain_logits(cfg, w, tokens)
    own32 = plain_logits(cfg, w, tokens, None, torch.float32)
    m, cache, st = load(folder, dtype)
    whole = None
    for cuts in ([171], [64, 64, 43], [2, 2, 61, 3, 100], [63, 2, 70], [130], [1, 65, 2, 2], [1, 129, 41], [1, 1, 1, 3, 160]):
        got = run_cut(st, cache, tokens, cuts)
        assert close(got, want, dtype, own32=own32, gauge=whole), (rel_err(got, want), name, cuts)
        whole = got if whole is None else whole
    # token by token from the first one, through captured graphs: the first tokens of a sequence, the shift's and the
    # convolutions' zeros before its start, states that start empty
    _, cache_g, st_g = load(folder, dtype, graphs=True)
    got = run_cut(st_g, cache_g, tokens[:90], [])
    assert close(got, want[:90], dtype, own32=own32[:90], gauge=whole[:90]), rel_err(got, want[:90])
    assert st_g.replays >= 89


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("W", "bfloat16"), ("ONE", "float32")])
def test_unequal_batches_reused_slots_pages_and_states(tmp_path_factory, name, dtype):
    """Requests of different lengths in one batch, decoded together while the short ones leave; the slots, pages,
    states, shift rows and convolution tails they give back are taken by the next batch (the cache is sized so that
    it must)."""
    from gogguf_b200.engine import StepEntry
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    m, cache, st = load(folder, dtype, max_tokens=448, graphs=True)
    got_rows, want_rows, own_rows = [], [], []
    for wave in range(3):
        reqs = [random_tokens(cfg["vocab"], n, seed=100 * wave + n) for n in (1, 65, 130, 7)]
        tails = [3, 20, 9, 40]
        full = [r + random_tokens(cfg["vocab"], t, seed=7 + t + wave) for r, t in zip(reqs, tails)]
        oracle = [plain_logits(cfg, w, f) for f in full]
        own = [plain_logits(cfg, w, f, None, torch.float32) for f in full]
        slots = [cache.open() for _ in reqs]
        out = st.step([StepEntry(s, r, want=[len(r) - 1]) for s, r in zip(slots, reqs)]).clone()
        for i, r in enumerate(reqs):
            got_rows.append(out[i]); want_rows.append(oracle[i][len(r) - 1]); own_rows.append(own[i][len(r) - 1])
        live = list(range(len(reqs)))
        for k in range(max(tails)):
            live = [i for i in live if k < tails[i]]
            out = st.step([StepEntry(slots[i], [full[i][len(reqs[i]) + k]], want=[0]) for i in live]).clone()
            for j, i in enumerate(live):
                got_rows.append(out[j]); want_rows.append(oracle[i][len(reqs[i]) + k])
                own_rows.append(own[i][len(reqs[i]) + k])
            for i in live:
                if k == tails[i] - 1:
                    cache.close(slots[i])
        cache.check()
        assert cache.live_slots == 0
    got, want = torch.stack(got_rows), torch.stack(want_rows)
    assert close(got, want, dtype, own32=torch.stack(own_rows)), rel_err(got, want)


def test_long_decoding_across_pages(tmp_path_factory):
    """A short prompt and 300 decoded tokens in float32: the sequence crosses four page borders, the states take
    every token once, the shift's row and the convolutions' tails move on by one row a step."""
    folder = make_folder(tmp_path_factory.getbasetemp(), "S", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 305, seed=77)
    want = plain_logits(cfg, w, tokens)
    own32 = plain_logits(cfg, w, tokens, None, torch.float32)
    m, cache, st = load(folder, "float32", max_tokens=512, graphs=True)
    got = run_cut(st, cache, tokens, [5])
    assert close(got, want, "float32", own32=own32), rel_err(got, want)


# ----------------------------------------------------------------------------------------------- made-up weights
MARKED, ASKING = 1, 5      # token ids: the one that is asked for, the one whose query asks


def _standout_model(tmp, kind, store):
    """A one-layer model without feed-forward whose weights make one token stand out.  The marked token's input has
    a large component along a direction that every other token's input is orthogonal to, the asking token's along
    another.  Attention: one key element of the first map of every kv head copies the marked direction, the same
    element of every head's first-map query copies the asking direction, and the scale is large: the asking token
    gives the marked one a score far above all others, wherever it lies.  The recurrences: decays next to one (a
    very negative decay parameter; a tiny step size), so that what the marked token wrote is still there."""
    from gogguf_b200.weights.loader import write_model_folder
    W, V = 64, 64
    g = _gen(31)
    embed = torch.randn(V, W, generator=g)
    a = embed[MARKED] / embed[MARKED].norm()
    for j in range(V):
        if j != MARKED:
            embed[j] -= (embed[j] @ a) * a
    mdir = embed[ASKING] / embed[ASKING].norm()
    small = lambda *s: torch.randn(*s, generator=g) * 0.02
    mid = lambda *s: torch.randn(*s, generator=g) * 0.3
    p = "l0.mix."
    w = {"embed": embed, "final.norm": torch.ones(W), "head": mid(V, W), "l0.norm1": torch.ones(W), "l0.ls1": torch.ones(W),
         "l0.shift": torch.full((W,), 0.05), "l0.dwa": torch.tensor([0.5, 0.5])}
    if kind == "attention":
        H, G, d, dv = 4, 2, 16, 24
        mx = attn(H, G, d, dv, 40.0 / math.sqrt(d), 0.0, 0.25, rot(4, 10000.0))
        q, k = small(H * 2 * d, W), small(G * 2 * d, W)
        for h in range(H):
            q[(h * 2) * d + 9] = 3.0 * mdir
        for gg in range(G):
            k[(gg * 2) * d + 9] = 3.0 * a
        w.update({p + "q": q, p + "k": k, p + "v": mid(G * dv, W), p + "q.norm": torch.ones(d), p + "k.norm": torch.ones(d),
                  p + "lq1": small(d), p + "lk1": small(d), p + "lq2": small(d), p + "lk2": small(d), p + "o": mid(W, H * dv)})
    elif kind == "rglru":
        C = 32
        mx = lru(C, 2, 3)
        x = small(C, W)
        x[7] = 3.0 * a
        w.update({p + "y": mid(C, W), p + "y.b": torch.zeros(C), p + "x": x, p + "x.b": torch.zeros(C),
                  p + "conv": torch.tensor([[0.0, 0.0, 1.0]]).repeat(C, 1), p + "conv.b": torch.zeros(C),
                  p + "ra": small(2, 16, 16), p + "ra.b": torch.zeros(2, 16), p + "ri": small(2, 16, 16),
                  p + "ri.b": torch.full((2, 16), 3.0), p + "lam": torch.full((C,), -9.0), p + "o": mid(W, C)})
    else:
        H, P, N = 2, 8, 16
        mx = ssm(H, P, N, 1, 1, 2)
        inner = H * P
        win = small(2 * inner + 2 * N + H, W)
        win[inner + 3] = 3.0 * a                              # an input channel that copies the marked direction
        win[2 * inner + 2] = 3.0 * a                          # ... written along a state row that
        win[2 * inner + N + 2] = 3.0 * mdir                   # ... the asking token reads
        w.update({p + "in": win, p + "conv": torch.tensor([[0.0, 1.0]]).repeat(inner + 2 * N, 1),
                  p + "conv.b": torch.zeros(inner + 2 * N), p + "dt_bias": torch.zeros(H), p + "A_log": torch.full((H,), -9.0),
                  p + "D": torch.zeros(H), p + "norm": torch.ones(inner), p + "o": mid(W, inner)})
    cfg = model(V, W, 1e-6, 1, [layer(kind, mx, None)])
    folder = os.path.join(str(tmp), f"standout_{kind}_{store}")
    write_model_folder(folder, cfg, {n: t.to(torch.bfloat16 if store == "bfloat16" else torch.float32) for n, t in w.items()})
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "rglru", "mamba2"])
def test_a_token_far_back_at_page_borders_and_at_the_start(tmp_path, dtype, kind):
    """The marked token stands once in a long sequence: first, second, around a page border, hundreds of tokens
    back.  The asking token at the end must see it: the same sequence without it gives another row there."""
    folder = _standout_model(tmp_path, kind, dtype)
    cfg, w = read_folder(folder)
    m, cache, st = load(folder, dtype)
    n = 330
    for marked in (0, 1, 62, 63, 64, 65, 127, 128, 200):
        tokens = [t if t not in (MARKED, ASKING) else 7 for t in random_tokens(cfg["vocab"], n, seed=marked)]
        tokens[marked], tokens[-1] = MARKED, ASKING
        without = list(tokens)
        without[marked] = 9
        want = plain_logits(cfg, w, tokens)
        moved = rel_err(plain_logits(cfg, w, without)[-1], want[-1])
        assert moved > 0.05, (kind, marked, moved)
        for cuts in ([n], [n - 1], [marked + 1, n - marked - 2], [n - 40]):
            if min(cuts) < 1:
                continue
            got = run_cut(st, cache, tokens, cuts)
            # (the marked token's own row: in bfloat16 the made-up scores, in the hundreds, round by more than the
            # distance between its two best keys, so that row is held in float32 only)
            rows = [marked, n - 1] if dtype == "float32" else [n - 1]
            assert close(got[rows], want[rows], dtype), (rel_err(got[rows], want[rows]), kind, marked, cuts)


# ----------------------------------------------------------------------------------------------- entry point, others
def test_greedy_generation_through_the_entry_point(tmp_path_factory):
    import gogguf_b200 as gg
    for name, dtype in (("S", "float32"), ("WB", "bfloat16")):
        folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype, std=0.3 if dtype == "float32" else 0.12)
        cfg, w = read_folder(folder)
        prompts = [random_tokens(cfg["vocab"], n, 30 + n) for n in (5, 1, 80)]
        engine = gg.load(folder, gg.LoadOptions(dtype=dtype, max_tokens=1024))
        ctx = engine.new_context()
        out = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[], keep_logits=True))
        rows, refs = [], []
        for p, r in zip(prompts, out):
            assert len(r.tokens) == 12 and r.prompt_tokens == len(p) and len(r.logits) == 12
            whole = plain_logits(cfg, w, list(p) + r.tokens[:-1])
            for k, row in enumerate(r.logits):
                assert int(row.argmax()) == r.tokens[k]            # greedy: the token is the best of its own row
                rows.append(row)
                refs.append(whole[len(p) - 1 + k])
        assert close(torch.stack(rows), torch.stack(refs), dtype), rel_err(torch.stack(rows), torch.stack(refs))
        # a second round in the same context reuses the slots, pages and states the first gave back; without kept
        # logits the loop runs a step ahead of the host and drops the step a finished sequence ran too far
        again = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[]))
        assert [r.tokens for r in again] == [r.tokens for r in out]
        stop = out[2].tokens[4]
        third = ctx.generate(prompts, gg.GenerateParams(max_tokens=12, stop_token_ids=[stop]))
        assert third[2].tokens == out[2].tokens[:out[2].tokens.index(stop)]
        ctx.cache.check()
        assert ctx.cache.live_slots == 0


@pytest.mark.parametrize("seed", list(range(10)))
def test_a_configuration_nobody_chose(tmp_path, seed):
    """Drawn sizes, layer orders and constants; float32 with the drawn choice of experts, bfloat16 with every expert
    chosen; whole, in portions, and a batch of two."""
    from gogguf_b200.engine import StepEntry
    for dtype in ("float32", "bfloat16"):
        cfg = draw_case(seed) if dtype == "float32" else every_expert(draw_case(seed))
        folder = write_case(tmp_path, f"drawn{seed}", cfg, seed, dtype, std=0.15)
        cfg2, w = read_folder(folder)
        tokens = random_tokens(cfg["vocab"], 97, seed=seed)
        want = plain_logits(cfg2, w, tokens)
        own32 = plain_logits(cfg2, w, tokens, None, torch.float32)
        m, cache, st = load(folder, dtype, graphs=True)
        for cuts in ([97], [3, 64, 2, 20], [90]):
            got = run_cut(st, cache, tokens, cuts)
            assert close(got, want, dtype, own32=own32), (rel_err(got, want), seed, dtype, cuts, cfg)
        other = random_tokens(cfg["vocab"], 30, seed=seed + 1)
        s1, s2 = cache.open(), cache.open()
        out = st.step([StepEntry(s1, other, want=[29]), StepEntry(s2, tokens[:66], want=[65])])
        assert close(out[1:2], want[65:66], dtype, own32=own32[65:66]), (seed, dtype)
        assert close(out[0:1], plain_logits(cfg2, w, other)[29:30], dtype,
                     own32=plain_logits(cfg2, w, other, None, torch.float32)[29:30])
        cache.close(s1); cache.close(s2)


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("W", "bfloat16")])
def test_trace_replay_through_the_program(tmp_path_factory, tmp_path, name, dtype):
    """bin/trace_run, the program a user runs: requests whole, with their last tokens one by one, and a batch of
    unequal lengths decoded together while the shorter ones end; places where nothing is wanted."""
    name = _case(name, dtype)
    from test_gpu_replay import Trace
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    lens = [150, 33, 97, 1]
    reqs = {f"r{i}": random_tokens(cfg["vocab"], n, seed=40 + i) for i, n in enumerate(lens)}
    oracle = {k: plain_logits(cfg, w, t) for k, t in reqs.items()}
    got_rows, want_rows = [], []
    tr = Trace(folder, dtype, tmp_path / "out", max_tokens=192 + 64 + 128 + 64)
    try:
        t = reqs["r0"]                                                   # the tail one by one
        cut = len(t) - 40
        assert tr.step([{"id": "d", "tokens": t[:cut], "want": []}]) is None
        for i in range(cut, len(t)):
            got = tr.step([{"id": "d", "tokens": [t[i]], "want": [0] if i % 3 else []}], end=["d"] if i == len(t) - 1 else [])
            if i % 3:
                got_rows.append(torch.from_numpy(got)); want_rows.append(oracle["r0"][i:i + 1])
        batch = ["r3", "r1", "r2", "r0"]                                 # together; the shorter ones end earlier
        pre = {k: max(1, len(reqs[k]) - 12) for k in batch}
        got = tr.step([{"id": k + "b", "tokens": reqs[k][:pre[k]], "want": [pre[k] - 1]} for k in batch],
                      end=[k + "b" for k in batch if pre[k] == len(reqs[k])])
        for j, k in enumerate(batch):
            got_rows.append(torch.from_numpy(got[j:j + 1])); want_rows.append(oracle[k][pre[k] - 1:pre[k]])
        pos = dict(pre)
        live = [k for k in batch if pre[k] < len(reqs[k])]
        while live:
            ending = [k for k in live if pos[k] + 1 == len(reqs[k])]
            got = tr.step([{"id": k + "b", "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live],
                          end=[k + "b" for k in ending])
            for j, k in enumerate(live):
                got_rows.append(torch.from_numpy(got[j:j + 1])); want_rows.append(oracle[k][pos[k]:pos[k] + 1])
                pos[k] += 1
            live = [k for k in live if k not in ending]
    finally:
        tr.close()
    assert close(torch.cat(got_rows), torch.cat(want_rows), dtype), rel_err(torch.cat(got_rows), torch.cat(want_rows))
