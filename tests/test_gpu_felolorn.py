"""The Felolorn decoder through the framework against the plain implementation (tests/plain_felolorn.py):
each mechanism alone, whole prompts layer by layer, portions, decoding, unequal batches, reuse of slots, pages and
states, far keys and page borders made to stand out, the first tokens, other sizes, the entry point, the replay
program."""
import math
import os

import pytest
import torch

import plain_felolorn as plain
from felolorn_cases import CASES, draw_case, every_expert, hgrn, latent, layer, light, make_folder, model, moe, plain_logits
from helpers import random_tokens, read_folder, rel_err

pytestmark = pytest.mark.gpu

TOL_F32 = 3e-5
TOL_BF16 = 4e-2      # as for the other architectures (tests/helpers.py): rounding alone reaches 3e-2 on single rows
DEV = "cuda:0"


def close(got, want, dtype, own32=None, few=True, gauge=None) -> bool:
    """float32: every row within TOL_F32, or within three times the distance `own32` of the plain implementation run
    in float32 from the same implementation in float64 where that is larger.  bfloat16: every row within TOL_BF16,
    except that (`few`) among 25 rows and more one in 25 may lie up to three times further out while the median
    stays below half the bound: the norms after the heads divide by the root mean square of as few as eight numbers,
    and where those nearly cancel, rounding alone moves the row; with routed experts, two choice scores closer than
    the rounding of the activations let the bfloat16 run take the other expert.  Each kernel alone, the float32 runs
    and the made-up weights hold every row.  `gauge` (bfloat16): the same rows from another run of the product (the
    prompt in one piece), itself held to the bound above; a row that rounding has moved there by d may lie up to 3 d
    out here: another cut of the prompt adds in another order, and such a row shows it as much."""
    got, want = got.double().cpu(), want.double().cpu()
    scale = want.abs().max().clamp_min(1e-30)
    rows = (got - want).abs().reshape(got.shape[0], -1).max(dim=1).values / scale
    bound = TOL_F32 if dtype == "float32" else TOL_BF16
    if own32 is not None and dtype == "float32":
        bound = max(bound, 3.0 * rel_err(own32, want))
    if gauge is not None and dtype == "bfloat16":
        g = (gauge.double().cpu() - want).abs().reshape(got.shape[0], -1).max(dim=1).values / scale
        rows = rows * (bound / torch.maximum(3.0 * g, torch.full_like(g, bound)))
    bad = int((rows >= bound).sum())
    ok = bad == 0 or (few and dtype == "bfloat16" and got.shape[0] >= 25 and bad <= got.shape[0] // 25
                      and float(rows.median()) < bound / 2 and float(rows.max()) < 3 * bound)
    if not ok:
        worst = rows.argsort(descending=True)[:8].tolist()
        print(f"close: bound {bound:.2e}, {bad} of {got.shape[0]} rows over it, median {float(rows.median()):.2e}, "
              f"worst rows {[(i, round(float(rows[i]), 5)) for i in worst]}")
    return ok


def load(folder, dtype, fast=True, max_tokens=2048, graphs=False):
    from gogguf_b200.engine import Model, Stepper
    from gogguf_b200.engine.graphs import GraphStepper
    m = Model.load(folder, dtype=dtype, fast=fast)
    cache = m.new_cache(max_tokens=max_tokens)
    return m, cache, (GraphStepper if graphs else Stepper)(m, cache)


def run_cut(st, cache, tokens, cuts):
    """One request in portions of the given sizes (the rest one token at a time); logits at every position."""
    from gogguf_b200.engine import StepEntry
    slot = cache.open()
    rows, at = [], 0
    for n in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        rows.append(st.step([StepEntry(slot, tokens[at:at + n], want=list(range(n)))]).clone())
        at += n
    cache.close(slot)
    cache.check()
    return torch.cat(rows, dim=0)


def _K():
    from gogguf_b200.csrc import kernels
    return kernels


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def _batch(lens):
    """Step tensors of a batch of sequences that bring `lens` new tokens: cu_seqlens, seq_of_token."""
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return _i32(cu), _i32([b for b, n in enumerate(lens) for _ in range(n)])


# ----------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,taps,lens", [(80, 4, (37, 9)), (64, 1, (37, 9)), (256, 2, (37, 9)), (24, 7, (37, 9)),
                                         (36, 3, (37, 9)), (50, 4, (37, 9)), (32, 9, (37, 9)),
                                         (1032, 4, (1101, 9)), (24, 5, (1030, 3)), (40, 1, (1300, 2))])
def test_input_convolution_alone(dt, W, taps, lens):
    """Two sequences in one batch; whole, then in portions down to one and two tokens with the tail carried in the
    state, in slots that were used before and hold leftovers until they are opened.  Steps of a thousand rows and
    more take the form that makes four rows a thread: a sequence's start in the middle of such a group, rows that
    do not fill the last group, channels that do not fill the last block."""
    K = _K()
    g = torch.Generator().manual_seed(W + taps)
    lens = list(lens)
    rows = [torch.randn(n, W, generator=g).to(dt) for n in lens]
    c = (0.5 * torch.randn(W, taps, generator=g)).float()
    want = torch.cat([r.double() + plain.causal_taps(r.double(), c.double()) for r in rows])
    state = torch.full((5, max(taps - 1, 1), W), 7.0, device=DEV)[:, :taps - 1] if taps > 1 else None
    slots = [3, 1]
    na, nb = lens
    for cuts in ([[na], [nb]], [[1, 2, na - 7, 4], [2, 1, 1, nb - 4]] if nb >= 9 else [[2, na - 2], [1, nb - 1]],
                 [[1] * min(na, 40) + [na - 40] * (na > 40), [1] * nb]):
        if state is not None:
            state[slots] = 0                       # what opening a slot does
        got = [[], []]
        at = [0, 0]
        for k in range(max(len(c_) for c_ in cuts)):
            live = [b for b in range(2) if k < len(cuts[b])]
            ns = [cuts[b][k] for b in live]
            h = torch.cat([rows[b][at[b]:at[b] + n] for b, n in zip(live, ns)]).to(DEV).contiguous()
            out = torch.empty_like(h)
            cu, sot = _batch(ns)
            # (steps of single tokens say so and take the launch that also moves the state on; every other time not)
            K.short_conv(h, out, c.t().contiguous().to(DEV), state, cu, _i32([slots[b] for b in live]), sot, h.shape[0], len(live),
                         max_new=max(ns) if k % 2 == 0 else 0)
            o = 0
            for b, n in zip(live, ns):
                got[b].append(out[o:o + n].cpu())
                o += n
                at[b] += n
        got = torch.cat([torch.cat(x) for x in got])
        assert rel_err(got, want) < (1e-6 if dt == torch.float32 else 8e-3), cuts
    if state is not None:
        assert torch.all(state[[0, 2, 4]] == 7.0)              # no other slot's state was touched


@pytest.mark.parametrize("H", [80, 256, 1024, 100])
def test_gated_norm_of_a_parts_output_added_to_the_stream(H):
    K = _K()
    g = torch.Generator().manual_seed(H)
    x, y, z = (torch.randn(7, H, generator=g) for _ in range(3))
    w, b = 1 + 0.2 * torch.randn(H, generator=g), torch.randn(H, generator=g)
    gated = y.double() * plain.sigmoid(z.double() + b.double())
    want = x.double() + plain.wnorm(gated, w.double(), 1e-5)
    xd, yd = x.to(DEV), y.to(DEV)
    K.rmsnorm_add(xd, yd, w.to(DEV), 1e-5, zero_y=True, gate=z.to(DEV), gate_bias=b.to(DEV))
    assert rel_err(xd, want) < 2e-6
    assert float(yd.abs().max()) == 0.0
    xd = x.to(DEV)
    K.rmsnorm_add(xd, y.to(DEV), w.to(DEV), 1e-5, gate=z.to(DEV))                       # a gate without a bias
    assert rel_err(xd, x.double() + plain.wnorm(y.double() * plain.sigmoid(z.double()), w.double(), 1e-5)) < 2e-6


def _scan_reference(kind, x, H, d, dv, consts, eps):
    """The plain functions on made-up projections: x holds the columns the product would have left."""
    n = x.shape[0]
    if kind == "lightning":
        q, k, v, g = x[:, :H * d], x[:, H * d:2 * H * d], x[:, 2 * H * d:2 * H * d + H * dv], x[:, 2 * H * d + H * dv:]
        q, k, v = (plain.silu(t) for t in (q, k, v))
        q, k, v = q.view(n, H, d), k.view(n, H, d), v.view(n, H, dv)
        o = torch.zeros(n, H, dv, dtype=x.dtype)
        for h in range(H):
            S = torch.zeros(d, dv, dtype=x.dtype)
            for t in range(n):
                S = consts["decay"][h] * S + k[t, h][:, None] * v[t, h][None, :]
                o[t, h] = S.T @ q[t, h]
        return plain.wnorm(o.reshape(n, H * dv), consts["norm"], eps) * plain.sigmoid(g)
    q, f, v = x[:, :H * d], x[:, H * d:2 * H * d], x[:, 2 * H * d:]
    q, v = plain.silu(q).view(n, H, d), v.view(n, H, dv)
    f = (consts["lower"] + (1 - consts["lower"]) * plain.sigmoid(f + consts["bias"])).view(n, H, d)
    o = torch.zeros(n, H, dv, dtype=x.dtype)
    for h in range(H):
        S = torch.zeros(d, dv, dtype=x.dtype)
        for t in range(n):
            S = f[t, h][:, None] * S + (1 - f[t, h])[:, None] * v[t, h][None, :]
            o[t, h] = S.T @ q[t, h]
    return plain.wnorm(o, consts["norm"], eps).reshape(n, H * dv)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,H,d,dv", [("lightning", 3, 24, 40), ("hgrn2", 2, 20, 36), ("lightning", 2, 128, 64),
                                         ("hgrn2", 4, 64, 128), ("hgrn2", 1, 72, 8), ("lightning", 1, 16, 16),
                                         ("lightning", 2, 8, 6), ("hgrn2", 3, 12, 10), ("hgrn2", 1, 8, 516),
                                         ("lightning", 9, 4, 460), ("hgrn2", 9, 4, 132)])
def test_matrix_state_recurrences_alone(dt, kind, H, d, dv):
    """Made-up projections of two requests through the scan and its finish against the plain loops: whole, then in
    portions and token by token from the carried state, in slots that held another sequence before.  Value sizes
    that are no multiple of four, heads of more than 512 values and rows of more than 4,096 take the finish kernel's
    plain form, more heads than a CTA has warps its loop over heads."""
    K = _K()
    g = torch.Generator().manual_seed(H * 100 + d)
    eps = 1e-5
    lens = [75, 11]
    width = 2 * H * d + (2 if kind == "lightning" else 1) * H * dv
    rows = [torch.randn(n, width, generator=g).to(dt) for n in lens]
    consts = dict(decay=([1.0, 0.97, 0.5, 0.0] * 3)[:H] if H > 1 else [0.995],
                  norm=(1 + 0.2 * torch.randn(H * dv if kind == "lightning" else dv, generator=g)).double(),
                  lower=torch.rand(H * d, generator=g).double(), bias=torch.randn(H * d, generator=g).double())
    want = torch.cat([_scan_reference(kind, r.double(), H, d, dv, consts, eps) for r in rows])
    state = torch.full((4, H, d, dv), 3.0, device=DEV)
    slots = [2, 0]
    kw = (dict(decay=torch.tensor(consts["decay"], device=DEV)) if kind == "lightning" else
          dict(forget_bias=consts["bias"].float().to(DEV), forget_lower=consts["lower"].float().to(DEV)))
    for cuts in ([[75], [11]], [[2, 9, 1, 63], [1, 8, 2]], [[70] + [1] * 5, [1] * 11]):
        state[slots] = 0
        got = [[], []]
        at = [0, 0]
        for k in range(max(len(c_) for c_ in cuts)):
            live = [b for b in range(2) if k < len(cuts[b])]
            ns = [cuts[b][k] for b in live]
            x = torch.cat([rows[b][at[b]:at[b] + n] for b, n in zip(live, ns)]).to(DEV).contiguous()
            T = x.shape[0]
            raw = torch.empty(T, H * dv, device=DEV)
            out = torch.empty(T, H * dv, device=DEV, dtype=dt)
            cu, sot = _batch(ns)
            K.gated_scan(x, 0, H * d, 2 * H * d, raw, state, cu, _i32([slots[b] for b in live]), sot, T, len(live), H, d, dv,
                         act_q=1, act_k=1 if kind == "lightning" else 0, act_v=1 if kind == "lightning" else 0, **kw)
            K.scan_finish(raw, x, 2 * H * d + H * dv, out, consts["norm"].float().to(DEV), sot, T, H, dv, eps,
                          whole=kind == "lightning", gate=1 if kind == "lightning" else 0)
            o = 0
            for b, n in zip(live, ns):
                got[b].append(out[o:o + n].cpu())
                o += n
                at[b] += n
        got = torch.cat([torch.cat(x) for x in got])
        assert rel_err(got, want) < (2e-5 if dt == torch.float32 else 1.2e-2), (kind, cuts)
    assert torch.all(state[[1, 3]] == 3.0)


def _scan_raw_reference(kind, x, H, d, dv, consts, S0):
    """o_t before the norm and the state after the last token, from the state S0 [H, d, dv], in float64."""
    n = x.shape[0]
    q = plain.silu(x[:, :H * d]).view(n, H, d)
    if kind == "lightning":
        k = plain.silu(x[:, H * d:2 * H * d]).view(n, H, d)
        v = plain.silu(x[:, 2 * H * d:2 * H * d + H * dv]).view(n, H, dv)
        g = torch.tensor(consts["decay"], dtype=x.dtype)[None, :, None].expand(n, H, d)
    else:
        g = (consts["lower"] + (1 - consts["lower"]) * plain.sigmoid(x[:, H * d:2 * H * d] + consts["bias"])).view(n, H, d)
        k = 1 - g
        v = x[:, 2 * H * d:2 * H * d + H * dv].view(n, H, dv)
    S = S0.clone()
    o = torch.zeros(n, H, dv, dtype=x.dtype)
    for t in range(n):
        S = g[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o.reshape(n, H * dv), S


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,H,d,dv,harsh", [("lightning", 3, 24, 40, False), ("hgrn2", 2, 20, 36, False),
                                               ("lightning", 2, 128, 64, False), ("hgrn2", 2, 64, 128, True),
                                               ("hgrn2", 1, 128, 128, False), ("hgrn2", 3, 96, 8, True),
                                               ("lightning", 1, 32, 128, False)])
def test_matrix_state_recurrences_in_chunks(dt, kind, H, d, dv, harsh):
    """Prompts through the form that cuts them into chunks for many CTAs, against the plain loop: portions that end
    on a chunk's border, one token past it and well inside; a second portion from the carried state; unequal
    sequences side by side with one of a single token; a padding row; forget gates that close almost entirely
    (harsh), where the products of gates inside a chunk fall below what float32 holds."""
    K = _K()
    g = torch.Generator().manual_seed(H * 1000 + d + dv)
    width = 2 * H * d + 2 * H * dv
    lens = [203, 65, 1, 130]
    rows = [(torch.randn(n, width, generator=g) * (2.0 if harsh else 1.0)).to(dt) for n in lens]
    consts = dict(decay=[1.0, 0.97, 0.5][:H] if H > 1 else [0.995],
                  lower=(torch.rand(H * d, generator=g) * (1e-3 if harsh else 1.0)).double(),
                  bias=(torch.randn(H * d, generator=g) - (6.0 if harsh else 0.0)).double())
    kw = (dict(decay=torch.tensor(consts["decay"], device=DEV), act_k=1, act_v=1) if kind == "lightning" else
          dict(forget_bias=consts["bias"].float().to(DEV), forget_lower=consts["lower"].float().to(DEV)))
    state = torch.full((6, H, d, dv), 3.0, device=DEV)
    slots = [4, 0, 5, 2]
    state[slots] = 0
    S = [torch.zeros(H, d, dv, dtype=torch.float64) for _ in lens]
    at = [0] * len(lens)
    for ns in ([64, 65, 1, 0], [129, 0, 0, 64], [10, 0, 0, 66]):
        live = [b for b, n in enumerate(ns) if n]
        x = torch.cat([rows[b][at[b]:at[b] + ns[b]] for b in live] + [torch.zeros(1, width).to(dt)]).to(DEV).contiguous()
        T = x.shape[0]
        cu = _i32([0] + list(torch.tensor([ns[b] for b in live]).cumsum(0)) + [T])
        sot = _i32([i for i, b in enumerate(live) for _ in range(ns[b])] + [-1])
        sl = _i32([slots[b] for b in live] + [1])
        raw = torch.full((T, H * dv), 7.0, device=DEV)
        n_seqs = len(live) + 1
        scratch = torch.empty(K.gated_scan_chunks_scratch(T, n_seqs, H, d, dv), device=DEV)
        K.gated_scan_chunks(x, 0, H * d, 2 * H * d, raw, scratch, state, cu, sl, sot, T, n_seqs, H, d, dv, act_q=1, **kw)
        o = 0
        for b in live:
            want, S[b] = _scan_raw_reference(kind, rows[b][at[b]:at[b] + ns[b]].double(), H, d, dv, consts, S[b])
            got = raw[o:o + ns[b]].cpu()
            # (running sums of log2 g reach hundreds where the gates close: their rounding is the looser bound)
            assert rel_err(got, want) < (1e-4 if harsh else 2e-5), (kind, ns, b)
            assert rel_err(state[slots[b]].cpu(), S[b]) < (1e-4 if harsh else 2e-5), (kind, ns, b)
            o += ns[b]
            at[b] += ns[b]
    assert torch.all(state[[1, 3]] == 3.0)


@pytest.mark.parametrize("E,top,groups,keep", [(12, 2, 3, 2), (6, 3, 2, 1), (16, 4, 4, 2), (5, 5, 1, 1), (8, 1, 8, 3),
                                               (64, 6, 8, 4), (9, 2, 3, 3)])
def test_choice_of_experts_alone(E, top, groups, keep):
    K = _K()
    g = torch.Generator().manual_seed(E * 10 + top)
    z = torch.randn(50, E, generator=g)
    z[3, :] = 0.25                                     # every score equal: the lowest indices of the first groups
    corr = torch.randn(E, generator=g)
    corr[E // 2] = -3.0                                # a choice score below zero: still better than a group left out
    idx = torch.empty(50, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(50, top, device=DEV)
    K.moe_route(z.to(DEV), top, idx, wts, None, correction=corr.to(DEV), groups=groups, keep=keep)
    s = plain.sigmoid(z.double())
    want = plain.choose_experts(s.float().double(), corr.double(), top, groups, keep)
    s32 = 1.0 / (1.0 + torch.exp(-z))                  # the kernel's own float32 scores decide ties the same way
    want = plain.choose_experts(s32.double(), corr.double(), top, groups, keep)
    assert idx.cpu().tolist() == want
    for t in range(50):
        assert torch.allclose(wts[t].cpu().double(), s[t, want[t]], rtol=1e-6)      # the scores, not renormalised
    K.moe_route(z.to(DEV), top, idx, wts, None, groups=groups, keep=keep)           # without a correction
    assert idx.cpu().tolist() == plain.choose_experts(s32.double(), 0 * corr.double(), top, groups, keep)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,dv,R,Rq", [(5, 12, 20, 44, 36), (4, 64, 64, 128, 64), (8, 32, 32, 64, 128), (1, 16, 16, 64, 64)])
def test_latent_attention_with_a_sink_alone(tmp_path, dtype, H, d, dv, R, Rq):
    """The mixer part by itself on made-up normed rows: a whole prompt (the expanded form where the sizes allow),
    portions that go on from the cache (the absorbed form) and decoding; two requests of unequal length."""
    from gogguf_b200.config.spec import PartSpec
    from gogguf_b200.engine.step import StepEntry
    W = 96
    cfg = model(64, W, 1e-5, 1.0, 0, 0.0, [layer("latent_attention", latent(H, d, dv, R, Rq, 0.3), None)])
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine.model import Model, expected_tensors
    from gogguf_b200.weights.loader import random_tensors
    spec = config_from_dict(cfg).to_spec()
    w = random_tensors(expected_tensors(spec), 5, 0.2, 0.1, dtype=torch.bfloat16)
    w["l0.mix.sink"] = torch.tensor([2.0, -1.0, 0.5, 30.0, -30.0, 0.0, 1.0, 4.0][:H]).to(torch.bfloat16)
    wd = {k: v.double() for k, v in w.items()}
    m = Model(spec, {k: v.to(DEV) for k, v in w.items()}, dtype=dtype)
    from gogguf_b200.engine import Stepper
    cache = m.new_cache(1024)
    st = Stepper(m, cache)
    toks = [random_tokens(64, n, seed=n) for n in (150, 70)]
    want = [plain.forward(t, wd, cfg) for t in toks]
    for cuts in ([150, 70], [64, 1], [100, 69], [2, 2]):
        slots = [cache.open(), cache.open()]
        got = [[], []]
        at = [0, 0]
        first = True
        while any(at[b] < len(toks[b]) for b in range(2)):
            ent, live = [], []
            for b in range(2):
                n = min(cuts[b] if first else (33 if at[b] < 120 else 1), len(toks[b]) - at[b])
                if n > 0:
                    ent.append(StepEntry(slots[b], toks[b][at[b]:at[b] + n], want=list(range(n))))
                    live.append((b, n))
            out = st.step(ent).clone()
            o = 0
            for b, n in live:
                got[b].append(out[o:o + n])
                o += n
                at[b] += n
            first = False
        for s in slots:
            cache.close(s)
        for b in range(2):
            assert close(torch.cat(got[b]), want[b], dtype), (cuts, b, rel_err(torch.cat(got[b]), want[b]))


def test_embedding_factor_and_bounded_logits():
    K = _K()
    table = torch.randn(10, 24)
    out = torch.empty(4, 24, device=DEV)
    K.embed_gather(table.to(DEV), _i32([3, 9, -1, 0]), out, 13.5)
    assert torch.equal(out.cpu()[[0, 1, 3]], table[[3, 9, 0]] * 13.5) and float(out[2].abs().max()) == 0.0
    z = torch.randn(5, 33) * 40
    zd = z.to(DEV)
    K.softcap(zd, 17.0)
    assert torch.allclose(zd.cpu().double(), 17.0 * torch.tanh(z.double() / 17.0), rtol=1e-6, atol=1e-6)


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


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("ONE", "float32"), ("W", "float32"),
                                        ("W", "bfloat16")])
def test_portions_and_decoding_equal_the_whole_prompt(tmp_path_factory, name, dtype):
    name = _case(name, dtype)
    folder = make_folder(tmp_path_factory.getbasetemp(), name, dtype)
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 171, seed=12)
    want = plain_logits(cfg, w, tokens)
    m, cache, st = load(folder, dtype)
    whole = None
    for cuts in ([171], [64, 64, 43], [2, 2, 61, 3, 100], [63, 2, 70], [130], [1, 65, 2, 2], [1, 129, 41], [1, 1, 1, 3, 160]):
        got = run_cut(st, cache, tokens, cuts)
        assert close(got, want, dtype, gauge=whole), (rel_err(got, want), name, cuts)
        whole = got if whole is None else whole
    # token by token from the first one, through captured graphs: the first tokens of a sequence, the convolution's
    # zeros before its start, states that start empty
    _, cache_g, st_g = load(folder, dtype, graphs=True)
    got = run_cut(st_g, cache_g, tokens[:90], [])
    assert close(got, want[:90], dtype, gauge=whole[:90]), rel_err(got, want[:90])
    assert st_g.replays >= 89


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("W", "bfloat16"), ("ONE", "float32")])
def test_unequal_batches_reused_slots_pages_and_states(tmp_path_factory, name, dtype):
    """Requests of different lengths in one batch, decoded together while the short ones leave; the slots, pages,
    states and convolution tails they give back are taken by the next batch (the cache is sized so that it must)."""
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
    every token once, the convolution's tail moves on by one row a step."""
    folder = make_folder(tmp_path_factory.getbasetemp(), "S", "float32")
    cfg, w = read_folder(folder)
    tokens = random_tokens(cfg["vocab"], 305, seed=77)
    want = plain_logits(cfg, w, tokens)
    m, cache, st = load(folder, "float32", max_tokens=512, graphs=True)
    got = run_cut(st, cache, tokens, [5])
    err = [(rel_err(got[i], want[i]), i) for i in range(len(tokens))]
    assert max(err)[0] < TOL_F32, max(err)


# ----------------------------------------------------------------------------------------------- made-up weights
MARKED, ASKING, PLAIN = 1, 5, 7      # token ids: the one that is asked for, the one whose query asks, a bystander


def _standout_model(tmp, kind, wide=False):
    """A one-layer model without feed-forward whose weights make one token stand out.  The marked token's input has
    a large component along a direction that every other token's input is orthogonal to, the asking token's along
    another.  Latent attention: one element of the latent copies the marked direction, one key element of every
    head copies that, and the asking token's queries are large there: the asking token gives the marked one a score
    far above all others.  Lightning (decay one) and HGRN2 (forget gates held near one by the lower bound): the
    marked token writes a large value into the state, which the asking token's query reads."""
    from gogguf_b200.weights.loader import write_model_folder
    W, V = 64, 64
    H, d, dv = (4, 64, 64) if wide else (2, 16, 24)
    R, Rq = (128, 64) if wide else (24, 16)
    g = torch.Generator().manual_seed(31)
    embed = torch.randn(V, W, generator=g)
    a = embed[MARKED] / embed[MARKED].norm()
    for j in range(V):
        if j != MARKED:
            embed[j] -= (embed[j] @ a) * a
    mdir = embed[ASKING] / embed[ASKING].norm()
    small = lambda *s: torch.randn(*s, generator=g) * 0.02
    mid = lambda *s: torch.randn(*s, generator=g) * 0.3
    p = "l0.mix."
    w = {"embed": embed, "final.norm": torch.ones(W), "l0.norm1": torch.ones(W), "l0.norm1b": torch.ones(W),
         "l0.canon1": torch.tensor([[0.0, 0.1]]).repeat(W, 1), "l0.rg1": small(W, W), "l0.rg1.b": torch.full((W,), 2.0)}
    if kind == "latent_attention":
        mx = latent(H, d, dv, R, Rq, 12.0 / math.sqrt(d))
        dq, dkv, uq, uk = mid(Rq, W), mid(R, W), small(H * d, Rq), small(H * d, R)
        dq[3], dkv[7] = 2.0 * mdir, 2.0 * a                 # latent elements that copy the two directions
        for h in range(H):
            uq[h * d + 5, 3] = 1.0                          # ... and a query / key element that copies those
            uk[h * d + 5, 7] = 1.0
        w.update({p + "dq": dq, p + "dq.norm": torch.ones(Rq), p + "uq": uq, p + "dkv": dkv, p + "dkv.norm": torch.ones(R),
                  p + "uk": uk, p + "uv": mid(H * dv, R), p + "sink": torch.zeros(H), p + "o": mid(W, H * dv)})
    elif kind == "lightning":
        mx = light(H, d, dv, [1.0] * H)
        q, k, v = small(H * d, W), small(H * d, W), small(H * dv, W)
        for h in range(H):
            q[h * d + 5], k[h * d + 5] = 0.5 * mdir, 0.5 * a
            v[h * dv:(h + 1) * dv] += torch.randn(dv, 1, generator=g) * a[None, :]
        w.update({p + "q": q, p + "k": k, p + "v": v, p + "g": small(H * dv, W), p + "norm": torch.ones(H * dv),
                  p + "o": mid(W, H * dv)})
    else:
        mx = hgrn(H, d, dv)
        q, v = small(H * d, W), small(H * dv, W)
        for h in range(H):
            q[h * d + 5] = 0.5 * mdir
            v[h * dv:(h + 1) * dv] += 3.0 * torch.randn(dv, 1, generator=g) * a[None, :]
        w.update({p + "q": q, p + "f": small(H * d, W), p + "f.b": torch.zeros(H * d), p + "lower": torch.full((H * d,), 0.998),
                  p + "v": v, p + "norm": torch.ones(dv), p + "o": mid(W, H * dv)})
    cfg = model(V, W, 1e-6, 1.0, 2, 0.0, [layer(kind, mx, None)])
    w = {k_: t.to(torch.bfloat16).contiguous() for k_, t in w.items()}       # values both compute dtypes hold exactly
    folder = os.path.join(str(tmp), f"standout_{kind}_{wide}")
    if not os.path.isdir(folder):
        write_model_folder(folder, cfg, w)
    return folder, cfg, {k_: t.float() for k_, t in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("kind", ["latent_attention", "lightning", "hgrn2"])
def test_a_token_far_back_at_page_borders_and_at_the_start(tmp_path, dtype, wide, kind):
    """The marked token sits at the first position, on either side of a page border, hundreds of positions back and
    just before the asking one; in a prompt, in a portion that goes on from the cache or state, and in decoding.
    `wide`: head sizes the tensor-core kernels take."""
    folder, cfg, w = _standout_model(tmp_path, kind, wide)
    m, cache, st = load(folder, dtype)
    n = 420
    for marked in (0, 63, 64, 127, n - 300, n - 2):
        tokens = [8 + (i * 7) % 50 for i in range(n)]
        tokens[marked], tokens[-1] = MARKED, ASKING
        want = plain_logits(cfg, w, tokens)
        unseen = list(tokens)
        unseen[marked] = PLAIN
        # the test can tell: the marked token moves the last logits by far more than the tolerance
        moved = rel_err(want[-1], plain_logits(cfg, w, unseen)[-1])
        assert moved > 0.2, (kind, marked, moved)
        for cuts in ([n], [n - 1], [marked + 1, n - marked - 2], [n - 40]):
            if min(cuts) < 1:
                continue
            got = run_cut(st, cache, tokens, cuts)
            rows = [marked, n - 1]
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
        if dtype == "float32":
            seq = list(prompts[0])
            for tok in out[0].tokens[:6]:
                assert tok == int(plain_logits(cfg, w, seq)[-1].argmax())
                seq.append(tok)
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
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.engine import StepEntry
    from gogguf_b200.engine.model import write_random_model
    for dtype in ("float32", "bfloat16"):
        cfg = draw_case(seed) if dtype == "float32" else every_expert(draw_case(seed))
        folder = os.path.join(str(tmp_path), f"drawn_{dtype}")
        write_random_model(config_from_dict(cfg), seed, folder, dtype=dtype, std=0.15, norm_std=0.1)
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
        assert close(out[0:1], plain_logits(cfg2, w, other)[29:30], dtype, own32=plain_logits(cfg2, w, other, None, torch.float32)[29:30])
        cache.close(s1); cache.close(s2)


@pytest.mark.parametrize("name,dtype", [("S", "float32"), ("S", "bfloat16"), ("W", "bfloat16"), ("ONE", "float32")])
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
        for k, t in reqs.items():                                        # whole, a few places wanted
            want = sorted({0, len(t) // 2, len(t) - 1})
            got = tr.step([{"id": k + "w", "tokens": t, "want": want}], end=[k + "w"])
            got_rows.append(torch.from_numpy(got)); want_rows.append(oracle[k][want])
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
