#!/usr/bin/env python3
"""Measurement: Qwen3-8B-shaped random-weight model, bfloat16, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]
                    [--shape 8b|14b|32b] [--workload] [--prefill-lengths 256,1024] [--decode-contexts 16384,32768]
    python bench.py --compare gigopel|sokirax|felolorn|dinuzen [--compare-sizes 2k,4k]   (another workload, see the end of this text)

A "step" is one decode step of a batch: every sequence goes on by one token, sampled greedily on the
device.  The timed region is exactly K steps after W warm-up steps, timed with CUDA events on the
launching stream.  One JSON line is printed:

  value        decoded tokens per second (batch * K / time), device timed, CUDA-graph replay per step
  e2e          the same through the Python entry point (Context.generate): host token ids in, host
               token ids out, every step copies its inputs from pinned host memory and reads the
               sampled ids back
  prefill      one 2,048-token prompt: tokens per second, and flops / time / measured bf16 peak
  roofline     bytes a decode step must read (every weight once + the cache of the live sequences)
               / time, against the measured HBM copy bandwidth
  points       decode tokens per second at batch 1 and 64
  config       every size, flat
  workload     (--workload) the shape's own request mix through Context.generate: prefill and decode rates
  prefill_sweep_ms  (--prefill-lengths) one prefill step per listed prompt length
  decode_by_context (--decode-contexts) decode steps of sequences that already hold that many tokens

`--compare gigopel` leaves all of the above aside and measures the Gigopel design (latent attention in a sliding
window, parallel blocks, xIELU or routed-expert feed-forwards) beside Qwen3 at equal width, depth, head count
and feed-forward parameter count (Qwen3 with full attention), random weights: one prefill step of 2,048 tokens and decode steps at batch
8 and 64 from 2,048-token contexts, for an all-dense and an all-experts Gigopel model per size.  It prints one JSON
line {"compare": "gigopel", "sizes": {...}} and per-model lines on stderr.

`--compare sokirax` does the same for the Sokirax design (norms on both sides of every part; windowed attention,
or windowed attention with sinks beside retention; gated units or routed experts with a shared unit): an all-dense
and an all-experts model per size, layers alternating between the two mixers, beside the same Qwen3.  It prints
{"compare": "sokirax", "sizes": {...}}.

`--compare felolorn` measures the Felolorn design (norms on both sides of every part, a gate on every part's
output, a short convolution before the mixer; latent attention with a query latent and sinks, lightning attention
or HGRN2; experts chosen inside the best groups): an all-experts model per size whose layers cycle through the three
mixers, beside the all-experts Sokirax model (its closest relative: the same arrangement of norms, retention,
routed experts) and the same Qwen3.  It prints {"compare": "felolorn", "sizes": {...}}.

`--compare dinuzen` measures the Dinuzen design (a norm in groups on every part's output with a layer scale, a
token shift before the mixer, a weighted sum over depth after every layer; differential attention, of which every
second layer reads the keys and values of the one before, the recurrent block with a real-gated linear recurrent
unit, Mamba-2; routed experts with identity experts and a gated shared expert): an all-experts model per size whose
layers cycle through attention, RG-LRU, Mamba-2 and attention on borrowed keys, beside the all-experts Felolorn model
(its closest relative: norms after the parts, recurrences behind short convolutions, routed experts with a
correction) and the same Qwen3.  It prints {"compare": "dinuzen", "sizes": {...}}.

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the
fallback figures of an earlier measurement on this pool.  The weights (16 GB) are far larger than
the 126 MB L2, so consecutive steps cannot be served from cache.  The reference cannot be installed
here (it is a Go program; there is no Go toolchain and no network): `--impl reference` says so.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline configuration: Qwen3-8B shape
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=12288, vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=4096, initializer_range=0.02,
)
# the layer sizes of the 14B and 32B shapes (same vocabulary and rotary base)
SHAPES = {
    "8b": {},
    "14b": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=17408),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                max_position_embeddings=8192),      # its request mix has prompts of 4,096 tokens
}
PROMPT_LEN = 2048
CONTEXT = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if k in d and d[k]:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def layer_weight_bytes(c, itemsize=2):
    qw = c["num_attention_heads"] * c["head_dim"]
    kvw = c["num_key_value_heads"] * c["head_dim"]
    h, i = c["hidden_size"], c["intermediate_size"]
    mats = (qw + 2 * kvw) * h + h * qw + 3 * h * i
    return mats * itemsize + (2 * h + 2 * c["head_dim"]) * 4      # norm weights are float32


def decode_bytes(c, layers, batch, ctx_len):
    """Bytes one decode step has to read: every weight it uses once, and the cache of the live requests."""
    h, v = c["hidden_size"], c["vocab_size"]
    w = layers * layer_weight_bytes(c) + v * h * 2 + h * 4 + batch * h * 2     # head, final norm, B embedding rows
    kv = batch * ctx_len * 2 * layers * c["num_key_value_heads"] * c["head_dim"] * 2
    return w + kv


def prefill_flops(c, layers, t):
    qw = c["num_attention_heads"] * c["head_dim"]
    kvw = c["num_key_value_heads"] * c["head_dim"]
    h, i, v = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    gemm = 2 * t * ((qw + 2 * kvw) * h + h * qw + 3 * h * i) * layers + 2 * 1 * v * h
    attn = layers * 2 * 2 * c["num_attention_heads"] * c["head_dim"] * (t * (t + 1) / 2)
    return gemm + attn


# ----------------------------------------------------------------------------- --compare gigopel
# layer sizes that resemble real models of this kind (8 layers each, so that a model is a few GB)
GIGOPEL_SIZES = {
    "2k": dict(width=2048, heads=16, dim=64, rot_dim=32, vdim=64, kv_rank=256, window=1024, ff=8192,
               experts=16, top=2, expert_ff=1024, layers=8, vocab=65536),
    "4k": dict(width=4096, heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512, window=2048, ff=16384,
               experts=32, top=4, expert_ff=2048, layers=8, vocab=65536),
}


def gigopel_config(z, kind):
    mixer = dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot_dim"], vdim=z["vdim"], kv_rank=z["kv_rank"],
                 scale=(z["dim"] + z["rot_dim"]) ** -0.5, rot=dict(base=500000.0, dims=z["rot_dim"]),
                 mask=dict(size=z["window"]))
    mlp = dict(kind="dense", ff=z["ff"]) if kind == "dense" else dict(
        kind="moe", expert=dict(ff=z["expert_ff"], limit=7.0), router=dict(experts=z["experts"], top=z["top"]))
    return dict(architecture="Gigopel", vocab=z["vocab"], width=z["width"], residual_mult=0.5, norm=dict(eps=1e-6),
                initializer_range=0.02,
                layers=[dict(type="latent_attention", mixer=mixer, mlp=mlp) for _ in range(z["layers"])])


# the same widths, depths and head counts for Sokirax; retention heads of 128 x 128, windows as Gigopel's
SOKIRAX_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=8, window=1024, ret_heads=8, ff=8192, experts=16, top=2, expert_ff=1024,
               shared_ff=1024, layers=8, vocab=65536),
    "4k": dict(width=4096, heads=32, kv_heads=8, window=2048, ret_heads=16, ff=16384, experts=32, top=4, expert_ff=2048,
               shared_ff=2048, layers=8, vocab=65536),
}


def sokirax_config(z, kind):
    """Layers alternate: attention (head size 128, stretched rotation) and attention with sinks (head size 64) beside
    retention (heads of 128 x 128, decays from 1 - 2^-5 to 1 - 2^-12)."""
    import math
    H, G, W = z["heads"], z["kv_heads"], z["width"]
    a = dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5, mask=dict(size=z["window"]),
             rot=dict(base=500000.0, dims=64, scaling=dict(factor=4.0, original=8192, fast=16.0, slow=2.0)))
    left = dict(heads=H, kv_heads=G, dim=64, vdim=64, scale=0.125, mask=dict(size=z["window"]),
                rot=dict(base=100000.0, dims=32))
    R = z["ret_heads"]
    right = dict(heads=R, dim=128, vdim=128, rot=dict(base=500000.0, dims=32),
                 decay=[1.0 - 2.0 ** (-5.0 - 7.0 * i / max(R - 1, 1)) for i in range(R)])
    p = dict(left=left, right=right, left_scale=1.0, right_scale=0.9)
    mlp = dict(kind="dense", ff=(2 * z["ff"] // 3) // 128 * 128) if kind == "dense" else dict(
        kind="moe", expert=dict(ff=z["expert_ff"]), router=dict(experts=z["experts"], top=z["top"]),
        shared=dict(ff=z["shared_ff"]))
    return dict(architecture="Sokirax", vocab=z["vocab"], width=W, norm=dict(eps=1e-6), initializer_range=0.02,
                layers=[dict(type="attention", mixer=a, mlp=mlp) if i % 2 == 0 else dict(type="parallel", mixer=p, mlp=mlp)
                        for i in range(z["layers"])])


# Felolorn at the same widths and depths: latent attention with Gigopel's head sizes and latent (no rotated part,
# no window), matrix states of 128 x 128 as Sokirax's retention, the same experts in four groups of which two are kept
FELOLORN_SIZES = {
    "2k": dict(width=2048, heads=16, dim=64, vdim=64, kv_rank=256, q_rank=512, state_heads=8, taps=4, experts=16, top=2,
               groups=4, keep=2, expert_ff=1024, layers=8, vocab=65536),
    "4k": dict(width=4096, heads=32, dim=128, vdim=128, kv_rank=512, q_rank=1024, state_heads=16, taps=4, experts=32, top=4,
               groups=4, keep=2, expert_ff=2048, layers=8, vocab=65536),
}


def felolorn_config(z):
    """Layers cycle through HGRN2, latent attention and lightning attention (heads of 128 x 128, decays from
    1 - 2^-5 to 1 - 2^-12); every layer has routed experts."""
    R = z["state_heads"]
    mixers = [
        ("hgrn2", dict(heads=R, dim=128, vdim=128)),
        ("latent_attention", dict(heads=z["heads"], dim=z["dim"], vdim=z["vdim"], kv_rank=z["kv_rank"], q_rank=z["q_rank"],
                                  scale=z["dim"] ** -0.5)),
        ("lightning", dict(heads=R, dim=128, vdim=128,
                           decay=[1.0 - 2.0 ** (-5.0 - 7.0 * i / max(R - 1, 1)) for i in range(R)])),
    ]
    mlp = dict(kind="moe", expert=dict(ff=z["expert_ff"]),
               router=dict(experts=z["experts"], top=z["top"], groups=dict(count=z["groups"], keep=z["keep"])))
    return dict(architecture="Felolorn", vocab=z["vocab"], width=z["width"], norm=dict(eps=1e-6), initializer_range=0.02,
                embedding=dict(scale=z["width"] ** 0.5), canon=dict(taps=z["taps"]), logit_softcap=30.0,
                layers=[dict(type=mixers[i % 3][0], mixer=mixers[i % 3][1], mlp=mlp) for i in range(z["layers"])])


# Dinuzen at the same widths and depths: differential attention with two maps of 64 (2k) or 128 (4k) per head over
# values of 128, a recurrent unit as wide as the stream in 16 blocks, Mamba-2 heads of 64 with states of 128, the same
# experts plus identity outputs and a shared expert
DINUZEN_SIZES = {
    "2k": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, lru_blocks=16, ssm_heads=32, ssm_vdim=64, ssm_state=128,
               ssm_groups=8, taps=4, norm_groups=8, experts=16, identity=2, top=2, expert_ff=1024, shared_ff=1024, layers=8,
               vocab=65536),
    "4k": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, lru_blocks=16, ssm_heads=64, ssm_vdim=64, ssm_state=128,
               ssm_groups=8, taps=4, norm_groups=8, experts=32, identity=4, top=4, expert_ff=2048, shared_ff=2048, layers=8,
               vocab=65536),
}


def dinuzen_config(z):
    """Layers cycle through differential attention, RG-LRU, Mamba-2 and differential attention on the keys and values
    of the attention layer three places before; every layer has routed experts."""
    W = z["width"]
    rot = dict(dims=z["dim"] // 2, base=500000.0, scaling=dict(factor=4.0, original=8192, fast=16.0, slow=2.0))
    att = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["vdim"], scale=z["dim"] ** -0.5, softcap=30.0,
               diff=0.3, rot=rot)
    mlp = dict(kind="moe", expert=dict(ff=z["expert_ff"]),
               router=dict(experts=z["experts"], identity=z["identity"], top=z["top"], scale=1.5), shared=dict(ff=z["shared_ff"]))
    layers = []
    for i in range(z["layers"]):
        k = i % 4
        if k == 0:
            layers.append(dict(type="attention", mixer=dict(att), mlp=mlp))
        elif k == 1:
            layers.append(dict(type="rglru", mixer=dict(width=W, blocks=z["lru_blocks"], conv=z["taps"]), mlp=mlp))
        elif k == 2:
            layers.append(dict(type="mamba2", mixer=dict(heads=z["ssm_heads"], vdim=z["ssm_vdim"], state=z["ssm_state"],
                                                         groups=z["ssm_groups"], norm_groups=z["ssm_groups"], conv=z["taps"]),
                               mlp=mlp))
        else:
            layers.append(dict(type="attention", mixer=dict(att, kv_from=i - 3), mlp=mlp))
    return dict(architecture="Dinuzen", vocab=z["vocab"], width=W, norm=dict(eps=1e-6, groups=z["norm_groups"]),
                initializer_range=0.02, layers=layers)


def qwen3_like(z):
    """Qwen3 at the same width, depth, head count and feed-forward parameter count (3 matrices instead of 2), with
    full attention (its cache of a 2,048-token context is read whole; Gigopel reads its window)."""
    inter = (2 * z["ff"] // 3) // 128 * 128
    return dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=z["layers"],
                hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=8, head_dim=128,
                intermediate_size=inter, vocab_size=z["vocab"], rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=True, max_position_embeddings=8192, initializer_range=0.02)


def compare_run(a):
    import torch
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.csrc import build, tcgen05_gemm
    from gogguf_b200.engine import Model, StepEntry
    from gogguf_b200.engine.graphs import GraphStepper
    from gogguf_b200.sampling import Sampler, SamplerConfig

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    pk = peaks()
    g = torch.Generator().manual_seed(0)

    def rand_tokens(V, n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    def prefill_ms(model, n):
        cache = model.new_cache(n + 64)
        st = GraphStepper(model, cache)
        times = []
        for it in range(4):
            s = cache.open()
            toks = rand_tokens(model.vocab_size, n)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            n0 = build.launch_count()
            ev0.record()
            st.step([StepEntry(s, toks, want=[n - 1])])
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1))
            launches = build.launch_count() - n0
            cache.close(s)
        return sorted(times[1:])[1], launches

    def decode_ms(model, batch, prompt_len, steps, warmup):
        room = prompt_len + warmup + steps + 8
        cache = model.new_cache(batch * (-(-room // 64) * 64))
        st = GraphStepper(model, cache)
        slots = [cache.open() for _ in range(batch)]
        chunk = max(1, 8192 // prompt_len)
        last = []
        for i in range(0, batch, chunk):
            ents = [StepEntry(s, rand_tokens(model.vocab_size, prompt_len), want=[prompt_len - 1]) for s in slots[i:i + chunk]]
            last.append(st.step(ents).clone())
        sampler = Sampler(SamplerConfig())
        rows = list(range(batch))
        pending = sampler.sample_async(torch.cat(last), rows, [0] * batch)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(warmup + steps):
            if it == warmup:
                pending.tokens()
                torch.cuda.synchronize()
                ev0.record()
            logits = st.decode_from_device(slots, pending.device_tokens, rows)
            nxt = sampler.sample_async(logits, rows, [it + 1] * batch)
            pending.tokens()
            pending = nxt
        ev1.record()
        torch.cuda.synchronize()
        tcgen05_gemm.check_status(dev)
        kernels = getattr(st, "last_graph_kernels", 0)
        for s in slots:
            cache.close(s)
        return ev0.elapsed_time(ev1) / steps, kernels

    def gig_numbers(z, kind, t):
        """Floating-point operations of a prefill step of t tokens and bytes a decode step reads, per layer stack."""
        W, H, d, r, dv, R, win = z["width"], z["heads"], z["dim"], z["rot_dim"], z["vdim"], z["kv_rank"], z["window"]
        mats = H * (d + r) * W + (R + r) * W + H * (d + dv) * R + W * H * dv
        ff_active = 2 * W * z["ff"] if kind == "dense" else z["top"] * 3 * W * z["expert_ff"] + z["experts"] * W
        keys = sum(min(i + 1, win) for i in range(t))
        attn = 2 * H * (d + r + dv) * keys                     # a whole prompt runs the expanded form: per-head keys and values
        flops = z["layers"] * (2 * t * (mats + ff_active) + attn) + 2 * z["vocab"] * W
        ff_read = 2 * W * z["ff"] if kind == "dense" else z["experts"] * 3 * W * z["expert_ff"]
        return flops, z["layers"] * (mats + ff_read) * 2 + z["vocab"] * W * 2

    def qwen_numbers(c, z, t):
        qw, kvw, h, i = c["num_attention_heads"] * 128, 8 * 128, c["hidden_size"], c["intermediate_size"]
        mats = (qw + 2 * kvw) * h + h * qw + 3 * h * i
        keys = t * (t + 1) // 2
        flops = z["layers"] * (2 * t * mats + 2 * 2 * qw * keys) + 2 * z["vocab"] * h
        return flops, z["layers"] * mats * 2 + z["vocab"] * h * 2

    def sok_numbers(z, kind, t):
        """The same two figures for a Sokirax model (per layer kind, half of the layers each), and the cache and
        state bytes a decode step reads per sequence."""
        W, H, G, R, win = z["width"], z["heads"], z["kv_heads"], z["ret_heads"], z["window"]
        att = (H * 128 + 2 * G * 128) * W + W * H * 128
        par = (H * 64 + 2 * G * 64) * W + W * H * 64 + 4 * R * 128 * W + W * R * 128
        dense_ff = (2 * z["ff"] // 3) // 128 * 128
        ff_active = 3 * W * dense_ff if kind == "dense" else (z["top"] * z["expert_ff"] + z["shared_ff"]) * 3 * W + z["experts"] * W
        ff_read = 3 * W * dense_ff if kind == "dense" else (z["experts"] * z["expert_ff"] + z["shared_ff"]) * 3 * W
        keys = sum(min(i + 1, win) for i in range(t))
        half = z["layers"] // 2
        attn = 2 * 2 * H * 128 * keys * half + (2 * 2 * H * 64 * keys + t * R * 2 * 2 * 128 * 128) * half
        flops = 2 * t * (half * (att + par) + z["layers"] * ff_active) + attn + 2 * z["vocab"] * W
        wbytes = (half * (att + par) + z["layers"] * ff_read) * 2 + z["vocab"] * W * 2
        per_seq = half * (min(t, win) * 2 * G * (128 + 64) * 2 + 2 * R * 128 * 128 * 4)
        return flops, wbytes, per_seq

    def fel_numbers(z, t):
        """The same figures for a Felolorn model whose layers cycle through HGRN2, latent attention and lightning."""
        W, H, d, dv, R, Q, S = z["width"], z["heads"], z["dim"], z["vdim"], z["kv_rank"], z["q_rank"], z["state_heads"]
        n = [len(range(k, z["layers"], 3)) for k in range(3)]
        hg = 3 * S * 128 * W + W * S * 128                     # q, f, v and the output matrix
        la = (Q + R) * W + H * d * Q + H * (d + dv) * R + W * H * dv
        li = 4 * S * 128 * W + W * S * 128                     # q, k, v, g and the output matrix
        gates = 2 * W * W
        ff_active = z["top"] * 3 * W * z["expert_ff"] + z["experts"] * W
        ff_read = z["experts"] * 3 * W * z["expert_ff"] + z["experts"] * W
        keys = t * (t + 1) // 2
        mix = n[0] * hg + n[1] * la + n[2] * li
        attn = n[1] * 2 * H * (d + dv) * keys + (n[0] + n[2]) * t * S * 2 * 2 * 128 * 128
        flops = 2 * t * (mix + z["layers"] * (gates + ff_active)) + attn + 2 * z["vocab"] * W
        wbytes = (mix + z["layers"] * (gates + ff_read)) * 2 + z["vocab"] * W * 2
        per_seq = n[1] * t * R * 2 + (n[0] + n[2]) * 2 * S * 128 * 128 * 4
        return flops, wbytes, per_seq

    def din_numbers(z, t):
        """The same figures for a Dinuzen model whose layers cycle through attention, RG-LRU, Mamba-2 and attention on
        borrowed keys and values."""
        W, H, G, d, dv = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"]
        n = [len(range(k, z["layers"], 4)) for k in range(4)]
        aq = H * 2 * d * W + W * H * dv                        # queries and the output matrix
        akv = G * (2 * d + dv) * W
        bw = W // z["lru_blocks"]
        lr = 3 * W * W + 2 * W * bw                            # y, x, the output matrix, the two gates' blocks
        inner, gn = z["ssm_heads"] * z["ssm_vdim"], z["ssm_groups"] * z["ssm_state"]
        ss = (2 * inner + 2 * gn + z["ssm_heads"]) * W + W * inner
        ff_active = (z["top"] * z["expert_ff"] + z["shared_ff"]) * 3 * W + (z["experts"] + z["identity"] + 1) * W
        ff_read = (z["experts"] * z["expert_ff"] + z["shared_ff"]) * 3 * W + (z["experts"] + z["identity"] + 1) * W
        keys = t * (t + 1) // 2
        mix = (n[0] + n[3]) * aq + n[0] * akv + n[1] * lr + n[2] * ss
        attn = (n[0] + n[3]) * 2 * H * (2 * d + 2 * dv) * keys + n[2] * t * z["ssm_heads"] * 2 * 2 * z["ssm_state"] * z["ssm_vdim"]
        flops = 2 * t * (mix + z["layers"] * ff_active) + attn + 2 * z["vocab"] * W
        wbytes = (mix + z["layers"] * ff_read) * 2 + z["vocab"] * W * 2
        per_seq = (n[0] + n[3]) * t * G * (2 * d + dv) * 2 + n[2] * 2 * inner * z["ssm_state"] * 4 + n[1] * 2 * W * 4
        return flops, wbytes, per_seq

    out = {}
    T = PROMPT_LEN
    design = a.compare
    for name in [x for x in a.compare_sizes.split(",") if x.strip()]:
        z = GIGOPEL_SIZES[name]
        if design == "dinuzen":
            zs, zf, zd = SOKIRAX_SIZES[name], FELOLORN_SIZES[name], DINUZEN_SIZES[name]
            arms = [("dinuzen_experts", dinuzen_config(zd)), ("felolorn_experts", felolorn_config(zf)),
                    ("qwen3_like", qwen3_like(z))]
        elif design == "felolorn":
            zs, zf = SOKIRAX_SIZES[name], FELOLORN_SIZES[name]
            arms = [("felolorn_experts", felolorn_config(zf)), ("sokirax_experts", sokirax_config(zs, "moe")),
                    ("qwen3_like", qwen3_like(z))]
        elif design == "sokirax":
            zs = SOKIRAX_SIZES[name]
            arms = [("sokirax_dense", sokirax_config(zs, "dense")), ("sokirax_experts", sokirax_config(zs, "moe")),
                    ("qwen3_like", qwen3_like(z))]
        else:
            arms = [("gigopel_dense", gigopel_config(z, "dense")), ("gigopel_experts", gigopel_config(z, "moe")),
                    ("qwen3_like", qwen3_like(z))]
        res = {}
        for arm, cd in arms:
            cfg = config_from_dict(cd)
            model = Model.random(cfg, seed=3, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
            torch.cuda.synchronize()
            per_seq = 0
            if arm == "qwen3_like":
                flops, wbytes = qwen_numbers(cd, z, T)
            elif arm == "dinuzen_experts":
                flops, wbytes, per_seq = din_numbers(zd, T)
            elif arm == "felolorn_experts":
                flops, wbytes, per_seq = fel_numbers(zf, T)
            elif design in ("sokirax", "felolorn"):
                flops, wbytes, per_seq = sok_numbers(zs, "dense" if arm.endswith("dense") else "moe", T)
            else:
                flops, wbytes = gig_numbers(z, "dense" if arm.endswith("dense") else "moe", T)
            pms, launches = prefill_ms(model, T)
            r = {"params_b": round(cfg.parameter_count() / 1e9, 3), "prefill_ms": round(pms, 3),
                 "prefill_tok_s": round(T / (pms / 1e3)), "prefill_tflops": round(flops / (pms / 1e3) / 1e12, 1),
                 "prefill_frac_of_bf16_peak": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 3),
                 "prefill_launches": launches}
            for b in (8, 64):
                dms, kernels = decode_ms(model, b, T, max(16, min(a.steps, 64)), max(a.warmup, 3))
                # experts: a step reads at most batch * top experts' matrices, not all of them
                rb = wbytes
                if arm in ("gigopel_experts", "sokirax_experts", "felolorn_experts", "dinuzen_experts"):
                    used = min(z["experts"], b * z["top"])
                    rb -= z["layers"] * (z["experts"] - used) * 3 * z["width"] * z["expert_ff"] * 2
                if arm == "qwen3_like":
                    rb += b * T * 2 * z["layers"] * 8 * 128 * 2
                elif design in ("sokirax", "felolorn", "dinuzen"):
                    rb += b * per_seq
                else:
                    rb += b * min(T, z["window"]) * z["layers"] * (z["kv_rank"] + z["rot_dim"]) * 2
                r[f"decode_b{b}_ms"] = round(dms, 4)
                r[f"decode_b{b}_tok_s"] = round(b / (dms / 1e3), 1)
                r[f"decode_b{b}_hbm_frac"] = round(rb / (dms / 1e3) / 1e9 / pk["hbm_gbs"], 3)
                r[f"decode_b{b}_kernels"] = kernels
            res[arm] = r
            print(f"[bench] {name} {arm}: {r}", file=sys.stderr)
            del model
            torch.cuda.empty_cache()
        out[name] = res
    print(json.dumps({"compare": design, "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), seeded token ids",
                      "prompt_len": T, "peaks": pk["source"], "sizes": out}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the 8B shape is the contract's")
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (same layer sizes); named in config")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (for short profiling runs)")
    ap.add_argument("--workload", action="store_true",
                    help="also run the shape's own request mix through the entry point (14b: 16 prompts of 128 to 2,048 "
                    "tokens and 256 new tokens each; 32b: 8 prompts of 4,096 tokens and 128 new tokens; 8b: 8 prompts "
                    "of 2,048 tokens and 64 new tokens); added to the line as workload")
    ap.add_argument("--decode-contexts", default="", help="comma separated context lengths: time decode steps of batch "
                    "--batch (and of one sequence) whose sequences already hold that many tokens (added to the line as "
                    "decode_by_context)")
    ap.add_argument("--prefill-lengths", default="", help="comma separated prompt lengths: time one prefill step of each "
                    "(printed on stderr, added to the line as prefill_sweep)")
    ap.add_argument("--compare", default="", choices=["", "gigopel", "sokirax", "felolorn", "dinuzen"],
                    help="another workload: the named design beside Qwen3 at equal size (prefill and decode), see the top")
    ap.add_argument("--compare-sizes", default="2k,4k", help="which of the comparison's layer sizes to run")
    a = ap.parse_args()

    if a.compare:
        return compare_run(a)
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "magomedcoder/gogguf is a Go program; no Go toolchain and no network here, pip cannot install it"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {a.gpus} is not built (this library runs on a single B200)")
        return 2
    if a.warmup < 3:
        a.warmup = 3

    import torch
    from gogguf_b200.config import config_from_dict
    from gogguf_b200.csrc import build
    from gogguf_b200.engine import Model, StepEntry
    from gogguf_b200.engine.graphs import GraphStepper
    from gogguf_b200.csrc import tcgen05_gemm
    from gogguf_b200.sampling import Sampler, SamplerConfig

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    base = dict(QWEN3_8B, **SHAPES[a.shape])
    if a.layers <= 0:
        a.layers = base["num_hidden_layers"]
    cdict = dict(base, num_hidden_layers=a.layers)
    long_ctx = [int(x) for x in a.decode_contexts.split(",") if x.strip()]
    longest = max(long_ctx + [int(x) for x in a.prefill_lengths.split(",") if x.strip()] + [0])
    if longest:         # the rotary tables are computed per step, so the context length is only a bound
        cdict["max_position_embeddings"] = max(cdict["max_position_embeddings"], longest + 128)
    cfg = config_from_dict(cdict)
    pk = peaks()
    t0 = time.time()
    model = Model.random(cfg, seed=2, dtype="bfloat16", device=dev, std=0.02, norm_std=0.0)
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t0:.1f} s ({cfg.parameter_count() / 1e9:.2f} B parameters)", file=sys.stderr)

    g = torch.Generator().manual_seed(0)
    V = cfg.vocab_size

    def rand_tokens(n):
        return torch.randint(0, V, (n,), generator=g).tolist()

    def decode_run(batch, steps, warmup, sampler_cfg=None, prompt_len=PROMPT_LEN):
        """Prefill `batch` prompts of `prompt_len` tokens, then time `steps` greedy decode steps on the device."""
        PROMPT_LEN = prompt_len
        room = PROMPT_LEN + warmup + steps + 8
        cache = model.new_cache(batch * (-(-room // 64) * 64))
        st = GraphStepper(model, cache)
        slots = [cache.open() for _ in range(batch)]
        chunk = max(1, 8192 // PROMPT_LEN)       # prompts per prefill step, bounds the workspace
        logits_last = []
        for i in range(0, batch, chunk):
            ents = [StepEntry(s, rand_tokens(PROMPT_LEN), want=[PROMPT_LEN - 1]) for s in slots[i:i + chunk]]
            logits_last.append(st.step(ents).clone())
        # greedy sampling on the device; each step takes its input ids from the device buffer the previous
        # step's sampling kernel wrote, and the host reads every step's ids (one step behind the device)
        sampler = Sampler(sampler_cfg if sampler_cfg is not None else SamplerConfig())
        rows = list(range(batch))
        pending = sampler.sample_async(torch.cat(logits_last), rows, [0] * batch)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clock_sampler = None
        n_launch0 = 0
        produced = []
        for it in range(warmup + steps):
            if it == warmup:
                produced.append(pending.tokens())
                torch.cuda.synchronize()
                clock_sampler = ClockSampler()
                clock_sampler.start()
                time.sleep(0.25)
                n_launch0 = build.launch_count()
                replay0 = st.replays
                ev0.record()
            logits = st.decode_from_device(slots, pending.device_tokens, rows)
            nxt_pending = sampler.sample_async(logits, rows, [it + 1] * batch)
            produced.append(pending.tokens())      # device-to-host read of the step's result, every step
            pending = nxt_pending
        ev1.record()
        torch.cuda.synchronize()
        tcgen05_gemm.check_status(dev)       # a bounded wait that ran out inside a kernel would invalidate the run
        clocks = clock_sampler.stop()
        ms = ev0.elapsed_time(ev1)
        direct = build.launch_count() - n_launch0
        launches = direct + (st.replays - replay0) * getattr(st, "last_graph_kernels", 0)
        ctx_len = PROMPT_LEN + warmup + steps // 2
        for s in slots:
            cache.close(s)
        del st, cache
        torch.cuda.empty_cache()
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "clocks": clocks,
                "launches": launches, "bytes": decode_bytes(cdict, a.layers, batch, ctx_len)}

    def e2e_run(batch, steps, warmup):
        """The same through the generation loop of the entry point: host ids in, host ids out."""
        import gogguf_b200 as gg
        engine = gg.Engine(model, gg.LoadOptions(dtype="bfloat16", max_batch=batch))
        # The prompts of the whole batch are prefilled in one step right before decoding starts, and the
        # first decode steps after that burst run at a lower clock (under the power cap) for some tens of
        # milliseconds; they are warm-up here, so that the timed steps are steady-state decoding as in
        # `decode_run`, which pauses between its prefill and its timed region.
        warmup = max(warmup, 32)
        room = PROMPT_LEN + warmup + steps + 8
        ctx = engine.new_context(max_tokens=batch * (-(-room // 64) * 64), max_batch=batch)
        prompts = [rand_tokens(PROMPT_LEN) for _ in range(batch)]
        stamps = []

        def on_token(i, t):
            if i == 0:
                stamps.append(time.perf_counter())     # the id has just arrived on the host
            return True

        ctx.generate(prompts, gg.GenerateParams(max_tokens=warmup + steps + 1, stop_token_ids=[], on_token=on_token))
        # stamps[k] is taken when token k of request 0 has reached the host; steps between stamps are decode steps
        dt = stamps[warmup + steps] - stamps[warmup]
        # bytes per decode step: the packed integer inputs (tokens, positions, slots, lengths, page tables)
        # copied from pinned host memory, and the sampled ids read back
        return {"tok_s": batch * steps / dt, "h2d": getattr(ctx.stepper, "last_h2d_bytes", None), "d2h": batch * 4,
                "warmup": warmup}

    def workload_run():
        """The request mix named for this shape, through Context.generate: host ids in, host ids out.

        Times the batch's prefill (until every request's first id is on the host) and the decoding after it."""
        import gogguf_b200 as gg
        if a.shape == "14b":
            lens = torch.randint(128, 2049, (16,), generator=torch.Generator().manual_seed(3)).tolist()
            new = 256
        elif a.shape == "32b":
            lens, new = [4096] * 8, 128
        else:
            lens, new = [PROMPT_LEN] * 8, 64
        batch = len(lens)
        engine = gg.Engine(model, gg.LoadOptions(dtype="bfloat16", max_batch=batch))
        ctx = engine.new_context(max_tokens=sum(-(-(n + new + 8) // 64) * 64 for n in lens), max_batch=batch)
        out = None
        for rep in range(2):                       # the first pass captures the graphs
            prompts = [rand_tokens(n) for n in lens]
            first = {}

            def on_token(i, t):
                if i not in first:
                    first[i] = time.perf_counter()
                return True

            torch.cuda.synchronize()
            t_start = time.perf_counter()
            res = ctx.generate(prompts, gg.GenerateParams(max_tokens=new, stop_token_ids=[], on_token=on_token))
            t_end = time.perf_counter()
            t_first = max(first.values())
            made = sum(len(r.tokens) for r in res)
            out = {"requests": batch, "prompt_tokens": sum(lens), "new_tokens": made,
                   "prefill_ms": (t_first - t_start) * 1e3, "prefill_tok_s": sum(lens) / (t_first - t_start),
                   "decode_tok_s": (made - batch) / (t_end - t_first), "decode_ms_per_step": (t_end - t_first) * 1e3 / (new - 1),
                   "total_s": t_end - t_start}
        return out

    def prefill_run(prompt_len=PROMPT_LEN):
        cache = model.new_cache(prompt_len + 64)
        st = GraphStepper(model, cache)
        times = []
        torch.cuda.synchronize()
        time.sleep(0.5)            # as before the timed decode region: start from an idle GPU, not from the previous run's heat
        for it in range(4):
            s = cache.open()
            toks = rand_tokens(prompt_len)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            ev0.record()
            st.step([StepEntry(s, toks, want=[prompt_len - 1])])
            ev1.record()
            torch.cuda.synchronize()
            times.append(ev0.elapsed_time(ev1))
            cache.close(s)
        ms = sorted(times[1:])[len(times[1:]) // 2]
        fl = prefill_flops(cdict, a.layers, prompt_len)
        return {"value": prompt_len / (ms / 1e3), "tokens": prompt_len, "ms": ms,
                "frac": fl / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), "tflops": fl / (ms / 1e3) / 1e12}

    main_run = decode_run(a.batch, a.steps, a.warmup)
    print(f"[bench] decode batch {a.batch}: {main_run['tok_s']:.1f} tok/s, {main_run['ms_per_step']:.3f} ms/step", file=sys.stderr)
    if a.no_e2e:
        e2e = {"tok_s": None, "h2d": None, "d2h": None, "warmup": None}
    else:
        e2e = e2e_run(a.batch, a.steps, a.warmup)
        print(f"[bench] e2e batch {a.batch}: {e2e['tok_s']:.1f} tok/s", file=sys.stderr)
    points, prefill = {}, None
    if not a.no_points:
        prefill = prefill_run()
        print(f"[bench] prefill: {prefill['value']:.0f} tok/s, {prefill['ms']:.2f} ms, {prefill['tflops']:.0f} TFLOP/s", file=sys.stderr)
        for b in (1, 64):
            r = decode_run(b, max(8, min(a.steps, 32)), 3)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_hbm_frac"] = r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
            print(f"[bench] decode batch {b}: {r['tok_s']:.1f} tok/s, {r['ms_per_step']:.3f} ms/step", file=sys.stderr)

    if not a.no_points:
        # the same steps with the sampling chain a chat deployment of this architecture uses, all of it on the device
        r = decode_run(a.batch, max(8, min(a.steps, 32)), 3, SamplerConfig(temp=0.6, top_k=20, top_p=0.95, seed=1))
        points[f"decode_b{a.batch}_temp0.6_top_k20_top_p0.95"] = r["tok_s"]
        print(f"[bench] decode batch {a.batch}, temp 0.6 / top-k 20 / top-p 0.95 on the device: {r['tok_s']:.1f} tok/s, "
              f"{r['ms_per_step']:.3f} ms/step", file=sys.stderr)

    sweep = {}
    for t in [int(x) for x in a.prefill_lengths.split(",") if x.strip()]:
        r = prefill_run(t)
        sweep[str(t)] = round(r["ms"], 3)
        print(f"[bench] prefill of {t} tokens: {r['ms']:.3f} ms, {r['value']:.0f} tok/s, {r['tflops']:.0f} TFLOP/s", file=sys.stderr)

    by_context = {}
    for c in long_ctx:
        for b in sorted({1, a.batch}):
            r = decode_run(b, 16, 3, prompt_len=c)
            frac = r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
            by_context[f"ctx{c}_b{b}"] = {"tok_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 3),
                                          "hbm_frac": round(frac, 3)}
            print(f"[bench] decode at context {c}, batch {b}: {r['tok_s']:.1f} tok/s, {r['ms_per_step']:.3f} ms/step, "
                  f"{frac:.3f} of the HBM roofline", file=sys.stderr)

    workload = None
    if a.workload:
        workload = workload_run()
        print(f"[bench] workload: {workload}", file=sys.stderr)

    achieved = main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"Qwen3-{a.shape.upper()} bf16 decode tok/s @ batch {a.batch} (points: batch 1/64; prefill tok/s @ 2,048 tokens)",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random weights N(0, 0.02), norm weights 1",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{a.shape.upper()} shape", "layers": a.layers, "layers_of_config": base["num_hidden_layers"],
            "hidden": cdict["hidden_size"], "q_heads": cdict["num_attention_heads"],
            "kv_heads": cdict["num_key_value_heads"], "head_dim": cdict["head_dim"],
            "intermediate": cdict["intermediate_size"], "vocab": cdict["vocab_size"],
            "rope_theta": cdict["rope_theta"], "rms_norm_eps": cdict["rms_norm_eps"], "tied": False,
            "global_batch": a.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "parallelism": "single GPU",
            "sampling": "greedy on device", "l2": "inputs>L2 (16 GB of weights per step)",
            "peaks": pk["source"],
        },
        "e2e": {"value": e2e["tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                "warmup": e2e["warmup"]},       # untimed decode steps of this arm (at least 32, see e2e_run)
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk["source"]},
    }
    if prefill is not None:
        line["prefill"] = {k: prefill[k] for k in ("value", "tokens", "ms", "frac")}
        line["points"] = points
    if sweep:
        line["prefill_sweep_ms"] = sweep
    if by_context:
        line["decode_by_context"] = by_context
    if workload is not None:
        line["workload"] = workload
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
