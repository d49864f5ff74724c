"""Prefill / decode throughput of the Tafopel hybrid decoder beside Qwen3 at equal width, depth and feed-forward size, plus
a per-kernel roofline table of the hybrid's own kernels and their Qwen3 counterparts (``python bench.py --hybrid``).

Random weights of the given dimensions, synthetic token ids; every number is device time between CUDA events around
``ModelRunner.run`` (model + LM head + sampling), after warm-up steps, with an L2 flush (a 256 MB write) between the timed
kernel launches of the per-kernel table.  Steps are scheduled by the engine's own Scheduler: admission, chunking and
decode growth are the product's.
"""
from __future__ import annotations

import json
import os
import sys
import time
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "nano-vllm_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

VOCAB = 32768


def tafopel_config(width: int, layers: int, heads: int, kv_rank: int, experts: int, top: int) -> dict:
    rot = {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    att = lambda src=None: {"type": "latent_attention", "mixer": dict(
        {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": kv_rank, "q_rank": 3 * kv_rank // 2, "scale": 192 ** -0.5, "rot": rot},
        **({"kv_from": src} if src is not None else {}))}
    ssm = {"type": "mamba1", "mixer": {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}}
    dense = {"kind": "dense", "ff": 3 * width}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": 3 * width // (2 * top)}, "shared": {"ff": width}}
    out = []
    for i in range(layers):
        k = i % 4
        base = i - k
        layer = [att(), att(base), ssm, ssm][k]
        out.append(dict(layer, mlp=[dense, moe, moe, dense][k]))
    return {"architecture": "Tafopel", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-6}, "layers": out}


SIZES = {
    # name: (width, layers, heads, kv_rank, experts, top)   -- Qwen3 beside it: same width / layers, 3 x width feed-forward, GQA 16/8 x 128
    "w1024": (1024, 8, 16, 256, 16, 2),
    "w2048": (2048, 8, 16, 512, 32, 4),
}


EXTRA_KINDS: dict = {}          # kind -> function(size name) -> model configuration; other benches register their designs here


def make_engine(kind: str, size: str, max_seqs: int, max_tokens: int, max_len: int):
    from nanovllm.config import Config
    from nanovllm.engine.model_runner import ModelRunner
    from nanovllm.engine.scheduler import Scheduler
    from nanovllm.engine.sequence import Sequence
    if kind in EXTRA_KINDS:
        hf = EXTRA_KINDS[kind](size)
        width = hf.hidden_size
    else:
        width, layers, heads, kv_rank, experts, top = SIZES[size]
    if kind in EXTRA_KINDS:
        pass
    elif kind == "tafopel":
        from nanovllm.models.tafopel import TafopelConfig
        hf = TafopelConfig(tafopel_config(width, layers, heads, kv_rank, experts, top))
    else:
        from nanovllm.utils.synthetic import hf_config_dict
        hf = SimpleNamespace(**hf_config_dict(dict(hidden_size=width, num_hidden_layers=layers, num_attention_heads=16, num_key_value_heads=8,
                                                   head_dim=128, intermediate_size=3 * width, vocab_size=VOCAB, tie_word_embeddings=False)))
    os.environ["NANOVLLM_ALLOW_RANDOM_INIT"] = "1"
    blocks = max_seqs * (-(-max_len // 256) + 1)
    cfg = Config("/nonexistent-random-init", hf_config=hf, max_num_seqs=max_seqs, max_num_batched_tokens=max_tokens, max_model_len=max_len,
                 kvcache_block_size=256, num_kvcache_blocks=blocks)
    Sequence.block_size = 256
    runner = ModelRunner(cfg, 0, None, sample_seed=1)
    return runner, Scheduler(cfg), Sequence


def throughput(kind: str, size: str, batch: int, prompt: int, new_tokens: int, warm: int = 3):
    """Prefill tokens/s over the prompt steps and decode tokens/s over the decode steps of `batch` requests."""
    import torch
    from nanovllm.sampling_params import SamplingParams
    runner, sched, Sequence = make_engine(kind, size, batch, 8192, prompt + new_tokens + 8)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
    res = {}
    for rep in range(2):                                    # the first repetition warms up both kinds of step (and the decode graphs)
        for _ in range(batch):
            sched.add(Sequence(torch.randint(0, VOCAB, (prompt,), generator=g).tolist(), sp))
        acc = {True: [0.0, 0], False: [0.0, 0]}
        steps = 0
        while not sched.is_finished():
            seqs, is_prefill = sched.schedule()
            n = sum(s.num_scheduled_tokens for s in seqs) if is_prefill else len(seqs)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            toks = runner.run(seqs, is_prefill)
            e1.record()
            torch.cuda.synchronize()
            sched.postprocess(seqs, toks, is_prefill)
            steps += 1
            if is_prefill or steps > warm:
                acc[is_prefill][0] += e0.elapsed_time(e1)
                acc[is_prefill][1] += n
        res = {"prefill_tok_s": acc[True][1] / acc[True][0] * 1e3, "decode_tok_s": acc[False][1] / max(acc[False][0], 1e-9) * 1e3,
               "prefill_ms": acc[True][0], "decode_ms_per_step": acc[False][0] / max(acc[False][1] // batch, 1)}
    runner.exit()
    del runner, sched
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return res


def timed(fn, flush, iters=5):
    import torch
    fn()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(iters):
        flush.add_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best * 1e-3


def kernel_table(size: str, peaks: dict):
    """Per kernel: seconds, algorithmic bytes and FLOPs, and the fraction of the roofline max(bytes / HBM, FLOPs / tensor or FMA peak)."""
    import torch
    from nanovllm import mixops, ops
    width, layers, heads, R, E, top = SIZES[size]
    rd, bs, dev, bf = 64, 256, "cuda", torch.bfloat16
    hbm, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    fma = 148 * 128 * 2 * 1.9e9                      # fp32 FMA peak of the part (148 SMs x 128 lanes x 2 x clock), for the kernels that use that pipe
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    rows = []

    def add(name, fn, nbytes, flops, pipe="hbm"):
        t = timed(fn, flush)
        roof = max(nbytes / hbm, flops / (tc if pipe == "tensor" else fma) if flops else 0.0)
        rows.append(dict(kernel=name, us=round(t * 1e6, 1), gbs=round(nbytes / t / 1e9, 1), tflops=round(flops / t / 1e12, 2),
                         bound="hbm" if nbytes / hbm >= (flops / (tc if pipe == "tensor" else fma) if flops else 0) else pipe,
                         of_roofline=round(roof / t, 3)))

    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)
    # ---- latent attention: prompt of 4 x 2048 tokens; decode of 64 rows at 4096 tokens ----
    D = R + rd
    cos_sin = torch.cat([torch.ones(8192, rd // 2), torch.zeros(8192, rd // 2)], 1).to(dev)
    sink = torch.zeros(heads, device=dev)
    for label, S, q, k in (("prefill 4x2048", 4, 2048, 2048), ("decode 64x4096", 64, 1, 4096)):
        nblk = S * (k // bs)
        cache = rn(nblk * bs, D)
        bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(S, -1)
        n = S * q
        q_lat, q_raw = rn(heads, n, R), rn(n, heads, 128 + rd)
        if q > 1:
            cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev)
            spn = mixops.StepSpans(S, q, cu * q, cu * k, None)
            pairs = S * (q * (q + 1) // 2)
        else:
            spn = mixops.StepSpans(S, 1, None, None, torch.full((S,), k, dtype=torch.int32, device=dev))
            pairs = S * k
        flops = pairs * heads * 2 * (D + R)
        nbytes = S * k * D * 2 + 2 * n * heads * R * 2
        add(f"latent_attention {label}", lambda: mixops.latent_attention(q_lat, q_raw, 128, cache, bt, bs, spn, sink, cos_sin, 0.07), nbytes, flops, "tensor")
    # Qwen3 counterparts at equal head count: 16 q heads / 8 kv heads x 128
    kv = torch.zeros(ops.kv_cache_shape(1, 64 * 16, 8, bs, 128), dtype=bf, device=dev)
    kv.normal_()
    ops.bind_kv_cache(kv)
    S, q = 4, 2048
    cu = (torch.arange(0, S + 1, dtype=torch.int32, device=dev) * q).contiguous()
    qq, kk, vv = rn(S * q, 16, 128), rn(S * q, 8, 128), rn(S * q, 8, 128)
    add("qwen3 paged_prefill 4x2048 (tcgen05)", lambda: ops.paged_prefill(0, qq, kk, vv, cu, cu, q, q, 0.088),
        S * q * (16 + 16 + 16) * 128 * 2, S * (q * (q + 1) // 2) * 16 * 4 * 128, "tensor")
    B, ctx = 64, 4096
    btd = torch.arange(B * (ctx // bs), dtype=torch.int32, device=dev).view(B, -1)
    cl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    qd = rn(B, 16, 128)
    add("qwen3 paged_decode 64x4096", lambda: ops.paged_decode(0, qd, btd, cl, 0.088), B * ctx * 8 * 128 * 2 * 2, B * ctx * 16 * 4 * 128, "fma")
    del kv
    # ---- selective scan ----
    C, N, Rdt, taps = 2 * width, 16, width // 16, 4
    for label, S, q in (("prefill 4x2048", 4, 2048), ("decode 64", 64, 1)):
        n = S * q
        xz, dbc = rn(n, 2 * C), rn(n, Rdt + 2 * N)
        u, dtr = rn(n, C), rn(n, C)
        conv_state = torch.zeros(S, taps - 1, C, device=dev)
        state = torch.zeros(S, C, N, device=dev)
        slots = torch.arange(S, dtype=torch.int32, device=dev)
        cw, cb, dtb, Dv = rn(C, taps), rn(C), rn(C), rn(C)
        A = -torch.rand(C, N, device=dev) * 4 - 0.1
        if q > 1:
            cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev) * q
            spn = mixops.StepSpans(S, q, cu, cu, None)
        else:
            spn = mixops.StepSpans(S, 1, None, None, torch.full((S,), 100, dtype=torch.int32, device=dev))
        add(f"causal_conv {label}", lambda: mixops.causal_conv(xz[:, :C], cw, cb, conv_state, slots, spn), n * C * 4 + S * (taps - 1) * C * 8, 0)
        add(f"selective_scan {label}", lambda: mixops.selective_scan(u, dtr, dtb, A, dbc[:, Rdt:Rdt + N], dbc[:, Rdt + N:], Dv, xz[:, C:], state, slots, spn),
            n * C * 2 * 4 + S * C * N * 8, n * C * N * 6, "fma")
    # ---- routed experts: 8192 tokens (prompt step) and 64 tokens (decode step) ----
    ff = 3 * width // (2 * top)
    w_up, w_down = rn(E, ff, width), rn(E, width, ff)
    for n in (8192, 64):
        h = rn(n, width)
        logits = torch.randn(n, E + 1, generator=g, device=dev)
        idx, wgt = mixops.moe_route(logits, E, top)
        sr, pos, te, nt = mixops.moe_align(idx, E)
        inter = mixops.moe_gemm(h, sr, te, nt, w_up, wgt=wgt, top=top, act=1)
        out = mixops.moe_gemm(inter, sr, te, nt, w_down, out_f32=True)
        wbytes = min(E, n * top) * ff * width * 2
        add(f"moe_route+align {n} tok", lambda: mixops.moe_align(mixops.moe_route(logits, E, top)[0], E), n * (E + 1) * 4 + n * top * 16, 0)
        add(f"moe_gemm up {n} tok", lambda: mixops.moe_gemm(h, sr, te, nt, w_up, wgt=wgt, top=top, act=1), wbytes + n * top * (width + ff) * 2, 2 * n * top * ff * width, "tensor")
        add(f"moe_gemm down {n} tok", lambda: mixops.moe_gemm(inter, sr, te, nt, w_down, out_f32=True), wbytes + n * top * (ff * 2 + width * 4), 2 * n * top * ff * width, "tensor")
        add(f"moe_combine {n} tok", lambda: mixops.moe_combine(out, pos, top, n, h, logits[:, E]), n * width * (4 * top + 2 + 4), 0)
    # ---- row-wise ops, 8192 rows ----
    n = 8192
    x, a, b, w = torch.randn(n, width, device=dev), rn(n, width), rn(n, width), rn(width)
    add("add_layernorm 8192 rows", lambda: mixops.add_layernorm(x, w, 1e-6, a=a, b=b), n * width * (4 + 4 + 2 + 2 + 2), 0)
    xr, res = rn(n, width), rn(n, width)
    add("qwen3 add_rmsnorm 8192 rows", lambda: ops.add_rmsnorm(xr, res, w, 1e-6), n * width * 2 * 4, 0)
    gu = rn(n, 6 * width)
    add("ff_act gelu*up 8192 rows", lambda: mixops.ff_act(gu, mixops.FF_GELU_TANH_MUL), n * 9 * width * 2, 0)
    add("qwen3 silu_mul 8192 rows", lambda: ops.silu_mul(gu), n * 9 * width * 2, 0)
    dkv = rn(n, R + rd)
    cache = torch.zeros(n, R + rd, dtype=bf, device=dev)
    posn = torch.arange(n, dtype=torch.int64, device=dev) % 4096
    sl = torch.arange(n, dtype=torch.int32, device=dev)
    nw = rn(R)
    add("latent_store 8192 rows", lambda: mixops.latent_store(dkv, nw, cos_sin, posn, sl, cache, R, rd, 1e-6), n * (R + rd) * 4, 0)
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
    out = {"bench": "hybrid", "dtype": "bf16", "data": "synthetic token ids, random weights", "peaks": {k: peaks[k] for k in ("hbm_gbs", "bf16_tflops", "source")},
           "workload": {"batch": a.batch, "prompt": a.prompt, "new_tokens": a.new_tokens}, "sizes": {}}
    for size in a.sizes.split(","):
        t0 = time.time()
        entry = {"dims": dict(zip(("width", "layers", "heads", "kv_rank", "experts", "top"), SIZES[size]))}
        for kind in () if a.no_models else ("tafopel", "qwen3"):
            entry[kind] = throughput(kind, size, a.batch, a.prompt, a.new_tokens)
        if not a.no_kernels:
            entry["kernels"] = kernel_table(size, peaks)
        entry["seconds"] = round(time.time() - t0, 1)
        out["sizes"][size] = entry
        print(json.dumps({size: entry}), file=sys.stderr, flush=True)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
