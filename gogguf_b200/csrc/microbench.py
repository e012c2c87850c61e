"""Kernel micro-benchmarks: python -m gogguf_b200.csrc.microbench [gemm|gemm_layer|attn|prefill_attn|sample|latent|retention|recurrence|dinuzen] [--m 1,8,64] [--ctx 2048,8192]

Times single kernels the way a decode step runs them: forty launches captured in a CUDA graph and
replayed, so that host launch cost is out of the picture and dependent launches overlap as they do
in a step.  Weights rotate over more than 400 MB so that the 126 MB L2 cannot serve them.  Prints
one line per (shape, M) with microseconds per launch and the achieved weight or cache bandwidth.
"""
from __future__ import annotations

import argparse
import math

import torch

SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gateup": (24576, 4096), "down": (4096, 12288),
          "head": (151936, 4096)}


def _time_graph(fn, reps: int = 40) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(reps):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def gemm(ms) -> None:
    from . import tcgen05_gemm as tc
    dev = "cuda:0"
    for name, (N, K) in SHAPES.items():
        nbuf = max(2, int(400e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
        for M in ms:
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            us = _time_graph(lambda i: tc.gemm_tc(x, ws[i % nbuf], out, cluster=True))
            print(f"gemm {name:7s} M={M:4d} splits={tc.splits_for(M, N, K, True):2d} {us:8.1f} us "
                  f"{N * K * 2 / us / 1e6:6.2f} TB/s", flush=True)
        del ws
        torch.cuda.empty_cache()


def gemm_layer(ms) -> None:
    """The four products of a layer as the layer runs them: q/k/v and gate-up (+ SwiGLU) with the folded norm on
    the way in, O and down adding into the residual and writing the next product's row statistics."""
    from . import tcgen05_gemm as tc
    dev = "cuda:0"
    H, QKV, I = 4096, 6144, 12288
    for M in ms:
        resid = torch.randn(M, H, device=dev)
        xh = resid.to(torch.bfloat16)
        ssq = torch.rand(M, H // 128, device=dev) * 128
        oss = torch.empty(M, H // 128, device=dev)
        oxh = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
        act = torch.randn(M, I, device=dev).to(torch.bfloat16)
        attn_out = torch.randn(M, H, device=dev).to(torch.bfloat16)
        cases = (
            ("qkv    norm in", QKV, H, lambda w, o: tc.gemm_tc_norm(xh, w, o, in_ssq=ssq, eps=1e-6),
             torch.empty(M, QKV, device=dev, dtype=torch.bfloat16)),
            ("o      add+stats", H, H, lambda w, o: tc.gemm_tc_norm(attn_out, w, o, accumulate=True, out_ssq=oss, out_xhat=oxh), resid),
            ("gateup norm in, swiglu", 2 * I, H, lambda w, o: tc.gemm_tc_norm(xh, w, o, swiglu=True, in_ssq=ssq, eps=1e-6),
             torch.empty(M, I, device=dev, dtype=torch.bfloat16)),
            ("down   add+stats", H, I, lambda w, o: tc.gemm_tc_norm(act, w, o, accumulate=True, out_ssq=oss, out_xhat=oxh), resid),
        )
        for name, N, K, fn, out in cases:
            nbuf = max(2, int(400e6 // (N * K * 2)) + 1)
            ws = [(torch.randn(N, K, device=dev) * 0.01).to(torch.bfloat16) for _ in range(nbuf)]
            us = _time_graph(lambda i: fn(ws[i % nbuf], out))
            print(f"gemm_layer {name:24s} M={M:5d} {us:8.1f} us {2.0 * M * N * K / us / 1e6:7.1f} TFLOP/s "
                  f"{N * K * 2 / us / 1e6:6.2f} TB/s", flush=True)
            del ws
            torch.cuda.empty_cache()
        tc.check_status(torch.device(dev))


def attn(ms, ctx_len: int = 2048, nq: int = 32, nkv: int = 8, d: int = 128, cluster: bool = True) -> None:
    from . import fast_attention as fa
    dev = "cuda:0"
    for B in ms:
        pages_per = (ctx_len + 63) // 64
        layers = max(2, int(400e6 // (B * pages_per * nkv * 64 * d * 2 * 2)) + 1)     # rotate over layers' pools
        kp = [torch.randn(B * pages_per, nkv, 64, d, device=dev).to(torch.bfloat16) for _ in range(layers)]
        vp = [torch.randn(B * pages_per, nkv, 64, d, device=dev).to(torch.bfloat16) for _ in range(layers)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
        pos = torch.full((B,), ctx_len - 1, dtype=torch.int32, device=dev)
        sot = torch.arange(B, dtype=torch.int32, device=dev)
        q = torch.randn(B, nq, d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        splits = fa.decode_tma_splits(B, nkv, ctx_len, cluster=cluster)
        po = torch.empty(B * nq * splits * d, device=dev) if not cluster else None
        pm = torch.empty(B * nq * splits * 2, device=dev) if not cluster else None
        us = _time_graph(lambda i: fa.attn_decode_tma(q, kp[i % layers], vp[i % layers], out, pos, sot, table, 64, B,
                                                      nq, nkv, d, 1.0 / math.sqrt(d), 0, splits, po, pm, cluster=cluster))
        nbytes = B * ctx_len * nkv * d * 2 * 2
        form = f"cluster of {splits}" if cluster else f"{splits} splits + combine"
        print(f"attn decode B={B:4d} ctx={ctx_len:6d} {form:22s} {us:8.1f} us {nbytes / us / 1e6:6.2f} TB/s", flush=True)
        del kp, vp
        torch.cuda.empty_cache()


def prefill_attn(lens, nq: int = 32, nkv: int = 8, d: int = 128) -> None:
    """One sequence of T new tokens from position 0, both prefill kernels."""
    from . import fast_attention as fa
    dev = "cuda:0"
    for T in lens:
        pages = (T + 63) // 64
        kp = torch.randn(pages, nkv, 64, d, device=dev).to(torch.bfloat16)
        vp = torch.randn(pages, nkv, 64, d, device=dev).to(torch.bfloat16)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        cl = torch.tensor([T], dtype=torch.int32, device=dev)
        sot = torch.zeros(T, dtype=torch.int32, device=dev)
        q = torch.randn(T, nq, d, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        flops = 4.0 * nq * d * (T * (T + 1) / 2)
        us = _time_graph(lambda i: fa.attn_prefill(q, kp, vp, out, cu, cl, sot, table, 64, 1, T // 64 + 1, nq, nkv, d,
                                                   1.0 / math.sqrt(d), 0), reps=10)
        print(f"attn prefill mma.sync T={T:6d} {us:9.1f} us {flops / us / 1e6:7.1f} TFLOP/s", flush=True)
        us = _time_graph(lambda i: fa.attn_prefill_tc(q, kp, vp, out, cu, cl, sot, table, 64, T, 1, T // 128 + 1, nq, nkv,
                                                      d, 1.0 / math.sqrt(d), 0), reps=10)
        print(f"attn prefill tcgen05  T={T:6d} {us:9.1f} us {flops / us / 1e6:7.1f} TFLOP/s", flush=True)


def sample(ms, V: int = 151936) -> None:
    """The sampling kernels on [batch, vocabulary] float32 logits: greedy, temperature, and the top-k chain."""
    from . import kernels as K
    dev = "cuda:0"
    for B in ms:
        logits = torch.randn(B, V, device=dev) * 3
        out = torch.empty(B, dtype=torch.int32, device=dev)
        u = torch.rand(B, dtype=torch.float64, device=dev)
        temps = torch.full((B,), 0.6, device=dev)
        for name, fn in (("greedy", lambda i: K.argmax(logits, out, B)),
                         ("temperature 0.6", lambda i: K.sample(logits, temps, u, out, B)),
                         ("temp 0.6, top-k 20, top-p 0.95", lambda i: K.sample_topk(logits, 0.6, 20, 0.95, 0.0, u, out, B)),
                         ("temp 0.6, top-k 1000, top-p 0.95", lambda i: K.sample_topk(logits, 0.6, 1000, 0.95, 0.0, u, out, B))):
            us = _time_graph(fn, reps=10)
            print(f"sample B={B:4d} V={V} {name:34s} {us:8.1f} us", flush=True)


def _peaks():
    import json
    import os
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def latent(sizes=((16, 64, 32, 64, 256, 1024, 2048), (32, 128, 64, 128, 512, 2048, 4096))) -> None:
    """The kernels of latent attention and of the routed experts alone, at layer sizes (heads, plain, rotated, value,
    latent, window, width): attention in a prompt of 2,048 tokens (tensor rate) and in decode steps (cache stream),
    the per-head products, the prep kernel, the activation, the experts through the index."""
    from . import fast_latent as FL
    from . import kernels as K
    dev = "cuda:0"
    hbm, tf, of = _peaks()
    ints = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    for H, d, r, dv, R, win, W in sizes:
        D = R + r
        tag = f"H={H} R={R} r={r} window={win}"
        # ---- a prompt of 2,048 tokens of one sequence
        T = 2048
        pages = T // 64
        pool = (torch.randn(pages, 64, D, device=dev) * 0.5).to(torch.bfloat16)
        qcat = (torch.randn(T, H, D, device=dev) * 0.2).to(torch.bfloat16)
        olat = torch.empty(T, H, R, device=dev, dtype=torch.bfloat16)
        table, cu = ints([list(range(pages))]), ints([0, T])
        pos, sot = ints(list(range(T))), ints([0] * T)
        us = _time_graph(lambda i: FL.latent_attention_mma(qcat, pool, olat, cu, pos, sot, table, 64, 1, T, H, R, r, 0.1, win), 10)
        keys = sum(min(i + 1, win) for i in range(T))
        fl = 2 * H * (2 * R + r) * keys
        print(f"latent_attention_mma prompt 2048  {tag}: {us:9.1f} us {fl / us / 1e6:7.1f} TFLOP/s {fl / us / 1e6 / tf:5.3f} of {of} bf16 peak", flush=True)
        qd = (torch.randn(T, H * (d + r) + D, device=dev) * 0.2).to(torch.bfloat16)
        kvx = (torch.randn(T, H * (d + dv), device=dev) * 0.3).to(torch.bfloat16)
        ckr = (torch.randn(T, D, device=dev) * 0.3).to(torch.bfloat16)
        avx = torch.empty(T, H, dv, device=dev, dtype=torch.bfloat16)
        us = _time_graph(lambda i: FL.latent_prompt_mma(qd, qcat, kvx, ckr, avx, cu, sot, 1, T, H, d, r, dv, R, 0.1, win, 0.5), 10)
        fl = 2 * H * (d + r + dv) * keys
        print(f"latent_prompt_mma (expanded) prompt 2048 {tag} d={d} dv={dv}: {us:9.1f} us {fl / us / 1e6:7.1f} TFLOP/s {fl / us / 1e6 / tf:5.3f} of {of} bf16 peak", flush=True)
        uk_t = (torch.randn(H, R, d, device=dev) * 0.1).to(torch.bfloat16)
        uv = (torch.randn(H, dv, R, device=dev) * 0.1).to(torch.bfloat16)
        av = torch.empty(T, H * dv, device=dev, dtype=torch.bfloat16)
        for m in (T, 8):
            us = _time_graph(lambda i: FL.headwise_gemm_mma(qd, qd.shape[1], d + r, uk_t, qcat, H * D, D, m), 10)
            fl = 2 * m * H * d * R
            by = H * d * R * 2 + m * H * (d + R) * 2
            print(f"headwise absorb M={m:5d} {tag}: {us:9.1f} us {fl / us / 1e6:7.1f} TFLOP/s {by / us / 1e3:7.1f} GB/s", flush=True)
            us = _time_graph(lambda i: FL.headwise_gemm_mma(olat, H * R, R, uv, av, H * dv, dv, m, 0.5), 10)
            fl = 2 * m * H * dv * R
            by = H * dv * R * 2 + m * H * (dv + R) * 2
            print(f"headwise expand M={m:5d} {tag}: {us:9.1f} us {fl / us / 1e6:7.1f} TFLOP/s {by / us / 1e3:7.1f} GB/s", flush=True)
        normw = torch.ones(R, device=dev)
        cos, sin = torch.ones(T, r // 2, device=dev), torch.zeros(T, r // 2, device=dev)
        us = _time_graph(lambda i: K.latent_prep(qd[:, :H * (d + r)], qd[:, H * (d + r):], normw, 1e-6, cos, sin, r, pos, sot,
                                                 table, 64, pool, qcat, T, H, d, r, R), 10)
        by = T * (H * r * 2 * 2 + D * 2 * 2)
        print(f"latent_prep T=2048 {tag}: {us:9.1f} us {by / us / 1e3:7.1f} GB/s {by / us / 1e3 / hbm:5.3f} of {of} copy bandwidth", flush=True)
        del pool, qcat, olat
        # ---- decode steps: B sequences of 2,048 cached positions each, one new token each; the pools rotate past L2
        for B in (8, 64):
            ctx = 2048
            ppseq = ctx // 64
            nrot = max(2, int(300e6 // (B * ppseq * 64 * D * 2)) + 1)
            pools = [(torch.randn(B * ppseq, 64, D, device=dev) * 0.5).to(torch.bfloat16) for _ in range(nrot)]
            q1 = (torch.randn(B, H, D, device=dev) * 0.2).to(torch.bfloat16)
            o1 = torch.empty(B, H, R, device=dev, dtype=torch.bfloat16)
            tb = ints([[b * ppseq + j for j in range(ppseq)] for b in range(B)])
            cu1, pos1, sot1 = ints(list(range(B + 1))), ints([ctx - 1] * B), ints(list(range(B)))
            S = FL.mma_splits(B, B, H, R, r, win, ctx)
            po = torch.empty(B * H, S, R, device=dev)
            pml = torch.empty(B * H, S, 2, device=dev)
            us = _time_graph(lambda i: FL.latent_attention_mma(q1, pools[i % nrot], o1, cu1, pos1, sot1, tb, 64, B, B, H, R, r, 0.1,
                                                               win, S, po, pml, max_new=1))
            by = B * min(ctx, win) * D * 2
            print(f"latent_attention_mma decode B={B:3d} splits={S:2d} {tag}: {us:9.1f} us {by / us / 1e3:7.1f} GB/s {by / us / 1e3 / hbm:5.3f} of {of} copy bandwidth", flush=True)
            del pools
            torch.cuda.empty_cache()
        # ---- feed-forward kernels
        F = 4 * W
        z = (torch.randn(2048, F, device=dev)).to(torch.bfloat16)
        us = _time_graph(lambda i: K.xielu(z, z, 0.7, 1.1, 0.5), 10)
        by = z.numel() * 4
        print(f"xielu 2048 x {F}: {us:9.1f} us {by / us / 1e3:7.1f} GB/s {by / us / 1e3 / hbm:5.3f} of {of} copy bandwidth", flush=True)
        E, top, Fe = 16, 2, W // 2
        nrot = max(2, int(300e6 // (E * 3 * Fe * W * 2)) + 1)
        gus = [(torch.randn(E, 2, Fe, W, device=dev) * 0.02).to(torch.bfloat16) for _ in range(nrot)]
        dns = [(torch.randn(E, W, Fe, device=dev) * 0.02).to(torch.bfloat16) for _ in range(nrot)]
        for B in (8, 64):
            h = torch.randn(B, W, device=dev).to(torch.bfloat16)
            idx = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(B)]).to(torch.int32)
            wts = torch.rand(B, top, device=dev)
            y = torch.empty(B * top, Fe, device=dev)
            res = torch.zeros(B, W, device=dev)
            used = len(set(idx.flatten().tolist()))
            us = _time_graph(lambda i: K.moe_gate_up(h, gus[i % nrot], idx, wts, y, B, top, True, 7.0, 1.702, 0.5))
            by = used * 2 * Fe * W * 2
            print(f"moe_gate_up B={B:3d} E={E} top={top} F={Fe} W={W}: {us:9.1f} us {by / us / 1e3:7.1f} GB/s {by / us / 1e3 / hbm:5.3f} of {of} copy bandwidth ({used} experts touched)", flush=True)
            xs = h.repeat_interleave(top, 0).contiguous()
            yb = torch.empty(B * top, Fe, device=dev, dtype=torch.bfloat16)
            rows = torch.empty(B * top, W, device=dev)
            us2 = _time_graph(lambda i: K.moe_expert_mma(xs, gus[i % nrot], idx, B * top, yb, True, 7.0, 1.702, 0.5))
            print(f"moe_expert_mma gate/up B={B:3d}: {us2:9.1f} us {by / us2 / 1e3:7.1f} GB/s {by / us2 / 1e3 / hbm:5.3f} of {of} copy bandwidth", flush=True)
            us2 = _time_graph(lambda i: K.moe_expert_mma(yb, dns[i % nrot], idx, B * top, rows, False))
            print(f"moe_expert_mma down    B={B:3d}: {us2:9.1f} us {by / 2 / us2 / 1e3:7.1f} GB/s {by / 2 / us2 / 1e3 / hbm:5.3f} of {of} copy bandwidth", flush=True)
            us = _time_graph(lambda i: K.moe_down(y, dns[i % nrot], idx, res, B, top, None))
            by = used * Fe * W * 2
            print(f"moe_down    B={B:3d} E={E} top={top} F={Fe} W={W}: {us:9.1f} us {by / us / 1e3:7.1f} GB/s {by / us / 1e3 / hbm:5.3f} of {of} copy bandwidth", flush=True)
        del gus, dns
        torch.cuda.empty_cache()


def retention(sizes=((8, 128, 128, 2048), (16, 128, 128, 4096))) -> None:
    """Retention (csrc/retention.cu) at layer sizes (heads, d, dv, width): a prompt of 2,048 tokens over many CTAs
    against the float32 multiply-add rate of the CUDA cores (the design asks for 32-bit there, so the tensor cores
    are not its roofline), decode steps against the copy bandwidth (a step reads and writes every state), and the
    norm-and-add kernel of the sandwich-norm blocks."""
    from . import kernels as K
    dev = "cuda:0"
    hbm, _, src = _peaks()
    props = torch.cuda.get_device_properties(0)
    fp32_tflops = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12      # FMA lanes x 2 x the highest SM clock
    print(f"peaks ({src}): {hbm:.0f} GB/s copy; float32 multiply-add rate {fp32_tflops:.1f} TFLOP/s (nominal, 1,965 MHz)")
    for H, d, dv, W in sizes:
        width = 2 * H * (d + dv)
        decay = torch.linspace(0.97, 0.9995, H, device=dev)
        T = 2048
        nbuf = 4
        xs = [(torch.randn(T, width, device=dev) * 0.5).to(torch.bfloat16) for _ in range(nbuf)]
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -torch.arange(16, dtype=torch.float64) / 16).to(dev)
        cos, sin = torch.empty(T, 16, device=dev), torch.empty(T, 16, device=dev)
        K.rope_tables(pos, inv, cos, sin)
        out = torch.empty(T, H * dv, device=dev, dtype=torch.bfloat16)
        state = torch.zeros(1, H, d, dv, device=dev)
        scratch = torch.empty(K.retention_chunks_scratch(T, 1, H, d, dv), device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        sot = torch.zeros(T, dtype=torch.int32, device=dev)
        us = _time_graph(lambda i: K.retention_chunks(xs[i % nbuf], out, scratch, state, cos, sin, cu, zero, sot, decay,
                                                      T, 1, H, d, dv, 32, d ** -0.5, 1e-6, 1.0), reps=10)
        C = K.RETENTION_CHUNK
        flops = 2 * T * H * (2 * d * dv + C * (d + dv) / 2)
        print(f"retention prompt  H={H} d={d} dv={dv} T={T}: {us:8.1f} us  {flops / us / 1e6:6.2f} TFLOP/s "
              f"({flops / us / 1e6 / fp32_tflops:.2f} of the float32 rate)", flush=True)
        for B in (8, 64):
            slots = 512 // B * B
            st = torch.zeros(slots, H, d, dv, device=dev)       # 512 states: 32 to 64 MB a head count, beyond L2 in turns
            x1 = (torch.randn(B, width, device=dev) * 0.5).to(torch.bfloat16)
            o1 = torch.empty(B, H * dv, device=dev, dtype=torch.bfloat16)
            raw = torch.empty(B, H * dv, device=dev)
            cu1 = torch.arange(B + 1, dtype=torch.int32, device=dev)
            sot1 = torch.arange(B, dtype=torch.int32, device=dev)
            sl = [torch.arange(k * B, (k + 1) * B, dtype=torch.int32, device=dev) for k in range(slots // B)]
            us = _time_graph(lambda i: K.retention(x1, o1, raw, st, cos, sin, cu1, sl[i % len(sl)], sot1, decay, B, B, H, d,
                                                   dv, 32, d ** -0.5, 1e-6, 1.0, 0))
            nbytes = 2 * B * H * d * dv * 4
            print(f"retention decode  H={H} d={d} dv={dv} batch {B:3d}: {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                  f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        for rows in (8, 64, 2048):
            n = max(2, int(300e6 // (rows * W * 12)) + 1) if rows >= 2048 else 2
            x = [torch.randn(rows, W, device=dev) for _ in range(n)]
            y = [torch.randn(rows, W, device=dev) for _ in range(n)]
            w = torch.ones(W, device=dev)
            xh = torch.empty(rows, W, device=dev, dtype=torch.bfloat16)
            sq = torch.empty(rows, (W + 127) // 128, device=dev)
            us = _time_graph(lambda i: K.rmsnorm_add(x[i % n], y[i % n], w, 1e-6, xhat=xh, ssq=sq))
            nbytes = rows * W * (4 + 4 + 4 + 2)
            print(f"norm-and-add      width {W} rows {rows:4d}: {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                  f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        del xs
        torch.cuda.empty_cache()


def recurrence(sizes=((8, 128, 128, 2048), (16, 128, 128, 4096))) -> None:
    """The matrix-state scan (csrc/recurrence.cu) at layer sizes (heads, d, dv, width), with a fixed decay and with
    a forget gate per channel: a prompt of 2,048 tokens against the float32 multiply-add rate of the CUDA cores
    (the state and all that enters it are 32-bit), decode steps against the copy bandwidth (a step reads and
    writes every state), then the finish kernel, the short convolution and the gated norm-and-add."""
    from . import kernels as K
    dev = "cuda:0"
    hbm, _, src = _peaks()
    props = torch.cuda.get_device_properties(0)
    fp32_tflops = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    print(f"peaks ({src}): {hbm:.0f} GB/s copy; float32 multiply-add rate {fp32_tflops:.1f} TFLOP/s (nominal, 1,965 MHz)")
    for H, d, dv, W in sizes:
        width = 2 * H * d + 2 * H * dv
        decay = torch.linspace(0.97, 0.9995, H, device=dev)
        fb, fl = torch.zeros(H * d, device=dev), torch.full((H * d,), 0.9, device=dev)
        T = 2048
        nbuf = 4
        xs = [(torch.randn(T, width, device=dev) * 0.5).to(torch.bfloat16) for _ in range(nbuf)]
        raw = torch.empty(T, H * dv, device=dev)
        out = torch.empty(T, H * dv, device=dev, dtype=torch.bfloat16)
        state = torch.zeros(1, H, d, dv, device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        sot = torch.zeros(T, dtype=torch.int32, device=dev)
        wn = torch.ones(H * dv, device=dev)
        for name, kw in (("fixed decay", dict(decay=decay, act_k=1, act_v=1)), ("forget gate", dict(forget_bias=fb, forget_lower=fl))):
            us = _time_graph(lambda i: K.gated_scan(xs[i % nbuf], 0, H * d, 2 * H * d, raw, state, cu, zero, sot, T, 1, H, d, dv,
                                                    act_q=1, **kw), reps=10)
            flops = 2 * T * H * 2 * d * dv
            print(f"scan prompt  {name} H={H} d={d} dv={dv} T={T}: {us:8.1f} us  {flops / us / 1e6:6.2f} TFLOP/s "
                  f"({flops / us / 1e6 / fp32_tflops:.2f} of the float32 rate)", flush=True)
            scratch = torch.empty(K.gated_scan_chunks_scratch(T, 1, H, d, dv), device=dev)
            us = _time_graph(lambda i: K.gated_scan_chunks(xs[i % nbuf], 0, H * d, 2 * H * d, raw, scratch, state, cu, zero, sot,
                                                           T, 1, H, d, dv, act_q=1, **kw), reps=10)
            # per chunk of 64 and head: the chunk's addition to the state, the products of q and k rows (half of
            # them below the diagonal), their product with v, the incoming state's share of the outputs
            cflops = 2 * T * H * (2 * d * dv + 32 * d + 32 * dv)
            print(f"chunked      {name} H={H} d={d} dv={dv} T={T}: {us:8.1f} us  {cflops / us / 1e6:6.2f} TFLOP/s "
                  f"({cflops / us / 1e6 / fp32_tflops:.2f} of the float32 rate; three launches)", flush=True)
            for B in (8, 64):
                slots = 512 // B * B
                st = torch.zeros(slots, H, d, dv, device=dev)       # 512 states: beyond L2 in turns
                x1 = (torch.randn(B, width, device=dev) * 0.5).to(torch.bfloat16)
                r1 = torch.empty(B, H * dv, device=dev)
                cu1 = torch.arange(B + 1, dtype=torch.int32, device=dev)
                sot1 = torch.arange(B, dtype=torch.int32, device=dev)
                sl = [torch.arange(k * B, (k + 1) * B, dtype=torch.int32, device=dev) for k in range(slots // B)]
                us = _time_graph(lambda i: K.gated_scan(x1, 0, H * d, 2 * H * d, r1, st, cu1, sl[i % len(sl)], sot1, B, B, H, d, dv,
                                                        act_q=1, **kw))
                nbytes = 2 * B * H * d * dv * 4
                print(f"scan decode  {name} H={H} d={d} dv={dv} batch {B:3d}: {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                      f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        for rows in (8, 64, 2048):
            x = xs[0][:rows]
            us = _time_graph(lambda i: K.scan_finish(raw[:rows], x, 2 * H * d + H * dv, out[:rows], wn, sot[:rows], rows, H, dv, 1e-6,
                                                     whole=True, gate=1))
            nbytes = rows * H * dv * (4 + 2 + 2)
            print(f"scan finish       heads {H} x {dv} rows {rows:4d}: {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                  f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        taps = 4
        cw = torch.randn(taps, W, device=dev) * 0.1
        for rows in (8, 64, 2048):
            n = max(2, int(300e6 // (rows * W * 4)) + 1) if rows >= 2048 else 2
            hs = [torch.randn(rows, W, device=dev).to(torch.bfloat16) for _ in range(n)]
            ho = torch.empty(rows, W, device=dev, dtype=torch.bfloat16)
            B = rows if rows < 2048 else 1
            cst = torch.zeros(B, taps - 1, W, device=dev)
            cuB = torch.arange(B + 1, dtype=torch.int32, device=dev) * (rows // B)
            sotB = torch.arange(rows, dtype=torch.int32, device=dev) // (rows // B)
            slB = torch.arange(B, dtype=torch.int32, device=dev)
            us = _time_graph(lambda i: K.short_conv(hs[i % n], ho, cw, cst, cuB, slB, sotB, rows, B, max_new=rows // B))
            nbytes = rows * W * (2 + 2)
            print(f"short conv        width {W} taps {taps} rows {rows:4d}: {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                  f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth; {'one launch' if rows == B else 'two launches'})", flush=True)
            n = max(2, int(300e6 // (rows * W * 12)) + 1) if rows >= 2048 else 2
            x = [torch.randn(rows, W, device=dev) for _ in range(n)]
            y = [torch.randn(rows, W, device=dev) for _ in range(n)]
            gt = [torch.randn(rows, W, device=dev) for _ in range(n)]
            w = torch.ones(W, device=dev)
            us = _time_graph(lambda i: K.rmsnorm_add(x[i % n], y[i % n], w, 1e-6, zero_y=True, gate=gt[i % n], gate_bias=w))
            nbytes = rows * W * (4 + 4 + 4 + 4 + 4)
            print(f"gated norm-and-add width {W} rows {rows:4d}: {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                  f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        del xs
        torch.cuda.empty_cache()


def dinuzen(sizes=((16, 4, 64, 128, 2048, 32, 64, 128, 8), (32, 8, 128, 128, 4096, 64, 64, 128, 8))) -> None:
    """The kernels the Dinuzen design added, at layer sizes (heads, kv heads, d, dv, width, state-space heads, their
    value size, state size, groups): differential attention (csrc/diff_attention.cu) on a prompt of 2,048 tokens
    against the bf16 tensor peak and in decode steps against the copy bandwidth; the two recurrences' prompt and
    decode forms; the convolution of a projection's columns, the token shift, the norm in groups with its add, the
    weighted sum over depth."""
    from . import kernels as K
    dev = "cuda:0"
    hbm, tflops, src = _peaks()
    props = torch.cuda.get_device_properties(0)
    fp32_tflops = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    print(f"peaks ({src}): {hbm:.0f} GB/s copy, {tflops:.0f} TFLOP/s bf16; float32 multiply-add rate {fp32_tflops:.1f} TFLOP/s (nominal)")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    for H, G, d, dv, W, SH, SP, SN, SG in sizes:
        T, ps = 2048, 64
        # ---- differential attention: one prompt of T tokens
        pages = T // ps
        kpool = (torch.randn(pages * 64 + 1, G, ps, 2 * d, device=dev) * 0.3).to(torch.bfloat16)
        vpool = torch.randn(pages * 64 + 1, G, ps, dv, device=dev).to(torch.bfloat16)
        q = torch.randn(T, H * 2 * d, device=dev).to(torch.bfloat16)
        o = torch.empty(T, H * dv, device=dev, dtype=torch.bfloat16)
        pos, sot, cu = i32(list(range(T))), i32([0] * T), i32([0, T])
        table = i32([list(range(pages))])
        us = _time_graph(lambda i: K.diff_attention_mma(q, kpool, vpool, o, pos, sot, cu, table, ps, T, 1, H, G, d, dv, d ** -0.5,
                                                        30.0, 0, 0.4, 1e-6, 0.7), reps=10)
        flops = 2 * H * (2 * d + 2 * dv) * (T * (T + 1) // 2)
        print(f"diff attention prompt  H={H} G={G} d={d} dv={dv} T={T}: {us:8.1f} us  {flops / us / 1e6:6.1f} TFLOP/s "
              f"({flops / us / 1e6 / tflops:.3f} of the bf16 peak)", flush=True)
        us = _time_graph(lambda i: K.diff_attention(q[:256], kpool, vpool, o[:256], pos[T - 256:], sot[:256], table, ps, 256, H, G, d,
                                                    dv, d ** -0.5, 30.0, 0, 0.4, 1e-6, 0.7), reps=3)
        print(f"   plain kernel, the last 256 rows of that prompt: {us:8.1f} us", flush=True)
        # ---- decode steps over contexts of T tokens
        for B in (8, 64):
            tb = i32([[(b * pages + j) for j in range(pages)] for b in range(B)])
            posb, sotb, cub = i32([T - 1] * B), i32(list(range(B))), i32(list(range(B + 1)))
            ns = K.diff_attention_splits(B, B, H, G, T)
            part = torch.empty(max(K.diff_attention_partial_elems(B, H, dv, ns), 1), device=dev)
            us = _time_graph(lambda i: K.diff_attention_mma(q[:B], kpool, vpool, o[:B], posb, sotb, cub, tb, ps, B, B, H, G, d, dv,
                                                            d ** -0.5, 30.0, 0, 0.4, 1e-6, 0.7, nsplit=ns, partial=part if ns > 1 else None,
                                                            max_new=1))
            nbytes = B * T * G * (2 * d + dv) * 2
            print(f"diff attention decode  batch {B:2d} ctx {T} ({ns} shares): {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s "
                  f"({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        del kpool, vpool
        # ---- the vector-state recurrence (width W)
        a = torch.rand(T, W, device=dev).pow(0.05)
        b = torch.randn(T, W, device=dev)
        y = torch.randn(T, W, device=dev).to(torch.bfloat16)
        outw = torch.empty(T, W, device=dev, dtype=torch.bfloat16)
        st = torch.zeros(64, W, device=dev)
        zero = i32([0])
        sums = torch.empty(K.diag_scan_chunks_scratch(T, 1, W), device=dev)
        us = _time_graph(lambda i: K.diag_scan_chunks(a, b, y, None, outw, sums, st, cu, zero, sot, T, 1), reps=10)
        nbytes = T * W * (2 * 8 + 2 + 2)
        print(f"vector scan prompt  W={W} T={T} (chunks): {us:8.1f} us  {nbytes / us / 1e3:7.1f} GB/s ({nbytes / us / 1e3 / hbm:.2f})", flush=True)
        us = _time_graph(lambda i: K.diag_scan(a, b, y, None, outw, st, cu, zero, sot, T, 1), reps=3)
        print(f"   row by row: {us:8.1f} us", flush=True)
        nb = W // 16
        wa = torch.randn(16, nb, nb, device=dev) * 0.05
        u = torch.randn(T, W, device=dev)
        bz, cz = torch.zeros(W, device=dev), -torch.rand(W, device=dev)
        us = _time_graph(lambda i: K.rglru_gates(u, wa, wa, bz, bz, cz, a, b, sot, T), reps=10)
        flops = 2 * T * 2 * W * nb
        print(f"gates of the unit   W={W} 16 blocks T={T}: {us:8.1f} us  {flops / us / 1e6:6.2f} TFLOP/s ({flops / us / 1e6 / fp32_tflops:.2f} of the float32 rate)", flush=True)
        for B in (8, 64):
            sotb, cub, slb = i32(list(range(B))), i32(list(range(B + 1))), i32(list(range(B)))
            us = _time_graph(lambda i: K.diag_scan(a[:B], b[:B], y[:B], None, outw[:B], st, cub, slb, sotb, B, B))
            print(f"vector scan decode  batch {B:2d}: {us:6.1f} us", flush=True)
        # ---- the matrix-state recurrence with step sizes
        inner, gn = SH * SP, SG * SN
        xc = torch.randn(T, inner + 2 * gn, device=dev) * 0.5
        xd = (torch.randn(T, SH, device=dev) - 2.0).to(torch.bfloat16)
        raw = torch.empty(T, inner, device=dev)
        sst = torch.zeros(64, SH, SN, SP, device=dev)
        dtb, na = torch.zeros(SH, device=dev), -torch.rand(SH, device=dev)
        scratch = torch.empty(K.stepsize_scan_scratch(T, 1, SH, SN, SP, 64), device=dev)
        us = _time_graph(lambda i: K.stepsize_scan(xc, inner, inner + gn, xd, 0, raw, sst, cu, zero, sot, dtb, na, T, 1, SH, SG, SN, SP,
                                                   chunk=64, scratch=scratch), reps=10)
        flops = 2 * T * SH * 2 * SN * SP
        print(f"step-size scan prompt  heads={SH} state={SN} vdim={SP} T={T} (chunks, the rows walked twice): {us:8.1f} us  "
              f"{flops / us / 1e6:6.2f} TFLOP/s ({flops / us / 1e6 / fp32_tflops:.2f} of the float32 rate)", flush=True)
        us = _time_graph(lambda i: K.stepsize_scan(xc, inner, inner + gn, xd, 0, raw, sst, cu, zero, sot, dtb, na, T, 1, SH, SG, SN, SP), reps=3)
        print(f"   row by row: {us:8.1f} us", flush=True)
        for B in (8, 64):
            sotb, cub, slb = i32(list(range(B))), i32(list(range(B + 1))), i32(list(range(B)))
            us = _time_graph(lambda i: K.stepsize_scan(xc[:B], inner, inner + gn, xd[:B], 0, raw[:B], sst, cub, slb, sotb, dtb, na, B, B,
                                                       SH, SG, SN, SP))
            nbytes = B * 2 * SH * SN * SP * 4
            print(f"step-size scan decode  batch {B:2d}: {us:6.1f} us  {nbytes / us / 1e3:7.1f} GB/s ({nbytes / us / 1e3 / hbm:.2f} of the copy bandwidth)", flush=True)
        # ---- the small kernels on T rows of width W
        x = torch.randn(T, W, device=dev)
        yy = torch.randn(T, W, device=dev)
        wv = torch.ones(W, device=dev)
        hb = torch.empty(T, W, device=dev, dtype=torch.bfloat16)
        shift_state = torch.zeros(64, W, device=dev)
        us = _time_graph(lambda i: K.rmsnorm_add(x, yy, wv, 1e-6, zero_y=False, groups=8), reps=10)
        print(f"norm in 8 groups + add  {T} x {W}: {us:6.1f} us  {T * W * 4 * 3 / us / 1e3 / hbm:.2f} of the copy bandwidth", flush=True)
        us = _time_graph(lambda i: K.token_shift(x, hb, wv, shift_state, cu, zero, sot, T, 1, max_new=T), reps=10)
        print(f"token shift             {T} x {W}: {us:6.1f} us  {T * W * 6 / us / 1e3 / hbm:.2f}", flush=True)
        hist = torch.zeros(9, T, W, device=dev)
        cf = torch.full((9,), 1.0 / 9, device=dev)
        us = _time_graph(lambda i: K.depth_mix(hist, x, cf, 8, 9), reps=10)
        print(f"sum over depth, 9 terms {T} x {W}: {us:6.1f} us  {T * W * 4 * 10 / us / 1e3 / hbm:.2f}", flush=True)
        cw = torch.randn(4, W, device=dev) * 0.3
        cst = torch.zeros(64, 3, W, device=dev)
        us = _time_graph(lambda i: K.column_conv(hb, yy, cw, wv, None, cst, cu, zero, sot, T, 1, act=1, max_new=T), reps=10)
        print(f"convolution, 4 taps     {T} x {W}: {us:6.1f} us  {T * W * 6 / us / 1e3 / hbm:.2f}", flush=True)
        for B in (8, 64):
            sotb, cub, slb = i32(list(range(B))), i32(list(range(B + 1))), i32(list(range(B)))
            t1 = _time_graph(lambda i: K.rmsnorm_add(x[:B], yy[:B], wv, 1e-6, zero_y=True, groups=8))
            t2 = _time_graph(lambda i: K.token_shift(x[:B], hb[:B], wv, shift_state, cub, slb, sotb, B, B, max_new=1))
            t3 = _time_graph(lambda i: K.depth_mix(hist[:, :B], x[:B], cf, 8, 9)) if False else 0.0
            t4 = _time_graph(lambda i: K.column_conv(hb[:B], yy[:B], cw, wv, None, cst, cub, slb, sotb, B, B, act=1, max_new=1))
            print(f"decode batch {B:2d}: norm+add {t1:5.1f} us, token shift {t2:5.1f} us, convolution {t4:5.1f} us", flush=True)
        torch.cuda.empty_cache()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "gemm_layer", "attn", "prefill_attn", "sample", "latent", "retention", "recurrence", "dinuzen"])
    ap.add_argument("--m", default="1,8,64", help="token counts (gemm), batch sizes (attn) or prompt lengths (prefill_attn)")
    ap.add_argument("--ctx", default="2048", help="attn: cached positions per sequence (comma separated)")
    ap.add_argument("--scratch", action="store_true", help="attn: splits merged by a second kernel instead of inside clusters")
    a = ap.parse_args()
    ms = [int(x) for x in a.m.split(",")]
    if a.what == "latent":
        latent()
        return
    if a.what == "retention":
        retention()
        return
    if a.what == "recurrence":
        recurrence()
        return
    if a.what == "dinuzen":
        dinuzen()
        return
    if a.what == "attn":
        for c in a.ctx.split(","):
            attn(ms, ctx_len=int(c), cluster=not a.scratch)
    else:
        {"gemm": gemm, "gemm_layer": gemm_layer, "prefill_attn": prefill_attn, "sample": sample}[a.what](ms)


if __name__ == "__main__":
    main()
