"""Prefill / decode throughput of the Tipetar decoder (windowed grouped-query attention with a distance bias, group-routed
experts, norms on the sublayer outputs) beside Qwen3 and Tafopel at equal width, depth, head counts and feed-forward size,
plus a per-kernel roofline table of its kernels and their counterparts (``python bench.py --windowed``).

Same rules as hybrid_bench.py, whose engine set-up, throughput loop and timing helper it uses: random weights, synthetic token
ids, device time between CUDA events after warm-up, a 256 MB write between the timed launches of the per-kernel table.
"""
from __future__ import annotations

import json
import os
import sys
import time

import hybrid_bench as hb

ROOT = hb.ROOT
VOCAB = hb.VOCAB

SIZES = {
    # name: (width, layers, heads, kv_heads, window, experts, identity, top, groups, keep)  -- head size 128; Qwen3 / Tafopel beside it: hybrid_bench.SIZES
    "w1024": (1024, 8, 16, 8, 1024, 16, 4, 2, 4, 2),
    "w2048": (2048, 8, 16, 8, 2048, 32, 8, 4, 8, 4),
}


def tipetar_config(size: str):
    from nanovllm.models.tipetar import TipetarConfig
    width, layers, heads, kv, window, experts, ident, top, groups, keep = SIZES[size]
    att = lambda src=None: {"type": "attention", "mixer": dict({"heads": heads, "kv_heads": kv, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                                                               "mask": {"size": window}}, **({"kv_from": src} if src is not None else {}))}
    moe = {"kind": "moe", "router": {"experts": experts, "identity": ident, "top": top, "scale": 2.0, "groups": {"count": groups, "keep": keep}},
           "expert": {"ff": 3 * width // (2 * top)}, "shared": {"ff": width}}
    out = [dict(att(None if i % 2 == 0 else i - 1), mlp=moe) for i in range(layers)]       # every second layer reads its predecessor's keys and values
    return TipetarConfig({"architecture": "Tipetar", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.7, "layers": out})


hb.EXTRA_KINDS["tipetar"] = tipetar_config


def kernel_table(size: str, peaks: dict):
    import torch
    from nanovllm import mixops, ops
    width, layers, H, G, window, E, ident, top, groups, keep = SIZES[size]
    d, bs, dev, bf = 128, 256, "cuda", torch.bfloat16
    hbm, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    fma = 148 * 128 * 2 * 1.9e9
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def add(name, fn, nbytes, flops, pipe="hbm"):
        t = hb.timed(fn, flush)
        peak = tc if pipe == "tensor" else fma
        roof = max(nbytes / hbm, flops / peak if flops else 0.0)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), gbs=round(nbytes / t / 1e9, 1), tflops=round(flops / t / 1e12, 2),
                         bound="hbm" if nbytes / hbm >= (flops / peak if flops else 0) else pipe, of_roofline=round(roof / t, 3)))

    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)
    from nanovllm.layers.window_attention import distance_slopes
    slopes = distance_slopes(H, dev)
    # ---- attention: prompt of 4 x 2048 tokens; decode of 64 rows at 4096 tokens, with the design's window and with none ----
    for label, S, q, k, win in (("prefill 4x2048", 4, 2048, 2048, window), ("prefill 4x2048 no window", 4, 2048, 2048, 0),
                                ("decode 64x4096", 64, 1, 4096, window), ("decode 64x4096 no window", 64, 1, 4096, 0)):
        nblk = S * (k // bs)
        cache = rn(nblk * bs, G * 2 * d)
        bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(S, -1)
        n = S * q
        qkv = rn(n, H * d)
        w = win if win else k
        if q > 1:
            cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev)
            spn = mixops.StepSpans(S, q, cu * q, cu * k, None)
            pairs = S * sum(min(i + 1, w) for i in range(q))
            keys_read = S * k
        else:
            spn = mixops.StepSpans(S, 1, None, None, torch.full((S,), k, dtype=torch.int32, device=dev))
            pairs = S * min(k, w)
            keys_read = S * min(k, w)
        flops = pairs * H * 4 * d
        nbytes = keys_read * G * 2 * d * 2 + 2 * n * H * d * 2
        add(f"window_attention {label}", lambda: mixops.window_attention(qkv, cache, bt, bs, spn, H, G, d, d, 0.088, slopes, win), nbytes, flops, "tensor")
    kv = torch.zeros(ops.kv_cache_shape(1, 64 * 16, G, bs, 128), dtype=bf, device=dev)
    kv.normal_()
    ops.bind_kv_cache(kv)
    S, q = 4, 2048
    cu = (torch.arange(0, S + 1, dtype=torch.int32, device=dev) * q).contiguous()
    qq, kk, vv = rn(S * q, H, 128), rn(S * q, G, 128), rn(S * q, G, 128)
    add("qwen3 paged_prefill 4x2048 (tcgen05)", lambda: ops.paged_prefill(0, qq, kk, vv, cu, cu, q, q, 0.088),
        S * q * (H + 2 * G + H) * 128 * 2, S * (q * (q + 1) // 2) * H * 4 * 128, "tensor")
    B, ctx = 64, 4096
    btd = torch.arange(B * (ctx // bs), dtype=torch.int32, device=dev).view(B, -1)
    cl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    qd = rn(B, H, 128)
    add("qwen3 paged_decode 64x4096", lambda: ops.paged_decode(0, qd, btd, cl, 0.088), B * ctx * G * 128 * 2 * 2, B * ctx * H * 4 * 128, "fma")
    del kv
    # ---- query / key norms + cache store, 8192 rows; Qwen3's per-head norm + rotation + store beside it ----
    n = 8192
    qkv = rn(n, (H + 2 * G) * d)
    cache = torch.zeros(n, G * 2 * d, dtype=bf, device=dev)
    sl = torch.arange(n, dtype=torch.int32, device=dev)
    wq, wk = rn(H * d), rn(G * d)
    add("qk_norm_store 8192 rows", lambda: mixops.qk_norm_store(qkv, H * d, G * d, G * d, wq, wk, sl, cache, 1e-6), n * ((2 * H + 3 * G) * d) * 2, 0)
    # ---- routed experts: 8192 tokens (prompt step) and 64 tokens (decode step); Tafopel's router and one-matrix experts beside them ----
    ff = 3 * width // (2 * top)
    w_gu, w_down, w_up1 = rn(E, 2 * ff, width), rn(E, width, ff), rn(E, ff, width)
    corr = torch.randn(E + ident, generator=g, device=dev) * 0.1
    for n in (8192, 64):
        h = rn(n, width)
        x32 = h.float()
        logits = torch.randn(n, E + ident, generator=g, device=dev)
        route = lambda: mixops.moe_route_grouped(logits, E + ident, top, corr, groups, keep, E, scale=2.0)
        idx, wgt = route()
        sr, pos, te, nt = mixops.moe_align(idx, E)
        real = int((idx >= 0).sum().item())
        inter = mixops.moe_gemm(h, sr, te, nt, w_gu, top=top, act=2, gather=True)
        out = mixops.moe_gemm(inter, sr, te, nt, w_down, out_f32=True)
        used = min(E, real)
        add(f"moe_route_grouped+align {n} tok", lambda: mixops.moe_align(route()[0], E), n * (E + ident) * 4 + n * top * 16, 0)
        add(f"moe_gemm gate|up {n} tok", lambda: mixops.moe_gemm(h, sr, te, nt, w_gu, top=top, act=2, gather=True),
            used * 2 * ff * width * 2 + real * (width + ff) * 2, 4 * real * ff * width, "tensor")
        add(f"moe_gemm down {n} tok", lambda: mixops.moe_gemm(inter, sr, te, nt, w_down, out_f32=True),
            used * ff * width * 2 + real * (ff * 2 + width * 4), 2 * real * ff * width, "tensor")
        add(f"moe_combine weighted {n} tok", lambda: mixops.moe_combine(out, pos, top, n, h, None, wgt=wgt, ident=x32), n * width * (4 * top + 2 + 4 + 4), 0)
        idx1, wgt1 = mixops.moe_route(logits, E, top)
        sr1, pos1, te1, nt1 = mixops.moe_align(idx1, E)
        add(f"tafopel moe_route+align {n} tok", lambda: mixops.moe_align(mixops.moe_route(logits, E, top)[0], E), n * (E + ident) * 4 + n * top * 16, 0)
        add(f"tafopel moe_gemm up {n} tok", lambda: mixops.moe_gemm(h, sr1, te1, nt1, w_up1, wgt=wgt1, top=top, act=1),
            min(E, n * top) * ff * width * 2 + n * top * (width + ff) * 2, 2 * n * top * ff * width, "tensor")
    # ---- row-wise ops, 8192 rows ----
    n = 8192
    x, y, w = torch.randn(n, width, device=dev), rn(n, width), rn(width)
    copy = torch.empty(n, width, dtype=bf, device=dev)
    add("add_normed 8192 rows", lambda: mixops.add_normed(x, y, w, 0.5, 1e-6, 1.0, copy), n * width * (4 + 4 + 2 + 2), 0)
    a, b = rn(n, width), rn(n, width)
    add("tafopel add_layernorm 8192 rows", lambda: mixops.add_layernorm(x, w, 1e-6, a=a, b=b), n * width * (4 + 4 + 2 + 2 + 2), 0)
    xr, res = rn(n, width), rn(n, width)
    add("qwen3 add_rmsnorm 8192 rows", lambda: ops.add_rmsnorm(xr, res, w, 1e-6), n * width * 2 * 4, 0)
    return rows


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="w1024,w2048")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=48)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-models", action="store_true")
    a = ap.parse_args(argv)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = dict(json.load(open(pk)), source="measured")
    out = {"bench": "windowed", "dtype": "bf16", "data": "synthetic token ids, random weights", "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
           "workload": {"batch": a.batch, "prompt": a.prompt, "new_tokens": a.new_tokens}, "sizes": {}}
    for size in a.sizes.split(","):
        t0 = time.time()
        entry = {"dims": dict(zip(("width", "layers", "heads", "kv_heads", "window", "experts", "identity", "top", "groups", "keep"), SIZES[size]))}
        for kind in () if a.no_models else ("tipetar", "tafopel", "qwen3"):
            entry[kind] = hb.throughput(kind, size, a.batch, a.prompt, a.new_tokens)
        if not a.no_kernels:
            entry["kernels"] = kernel_table(size, peaks)
        entry["seconds"] = round(time.time() - t0, 1)
        out["sizes"][size] = entry
        print(json.dumps({size: entry}), file=sys.stderr, flush=True)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
