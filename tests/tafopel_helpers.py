"""Small Tafopel configurations with random weights for the tests, written out as checkpoint directories."""
from __future__ import annotations

import json
import os

import torch


def rot(dims, base=10000.0, scaling=True):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}
    return r


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=24, kv_from=None, scale=0.2, scaling=True, base=10000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": rot(rot_dim, base, scaling)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def mamba(inner=48, state=6, dt_rank=5, conv=4):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=40, shared=24):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(layers, width=64, vocab=97, eps=1e-5):
    return {"architecture": "Tafopel", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [dict(l, mlp=mlp) for l, mlp in layers]}


def config_a():
    """mamba first, an attention layer lending its cache to a later one, every feed-forward kind, one layer without any."""
    return config([(mamba(), moe()), (latent(), dense()), (mamba(inner=40, state=9, dt_rank=3, conv=2), None),
                   (latent(heads=2, dim=24, vdim=16, q_rank=32, kv_from=1), moe(experts=3, top=1, ff=24, shared=0))])


def config_b():
    """other sizes: one head, top 3 of 8, no rotary scaling, conv of 1 and 5 taps, state of 1 and 17."""
    return config([(latent(heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=12, q_rank=8, scaling=False), moe(experts=8, top=3, ff=16, shared=8)),
                   (mamba(inner=24, state=1, dt_rank=1, conv=1), dense(40)),
                   (mamba(inner=32, state=17, dt_rank=7, conv=5), dense(24)),
                   (latent(heads=5, dim=8, rot_dim=6, vdim=4, kv_rank=136, q_rank=16, scale=0.35), None)], width=48, vocab=61)


def config_c():
    """attention only: two layers read the first layer's cache, mixed feed-forwards."""
    return config([(latent(heads=4, dim=8, rot_dim=8, vdim=8, kv_rank=24, q_rank=16), moe(4, 2, 16, 0)),
                   (latent(heads=2, dim=16, rot_dim=8, vdim=12, kv_rank=24, q_rank=8, kv_from=0), None),
                   (latent(heads=7, dim=8, rot_dim=8, vdim=8, kv_rank=24, q_rank=40, kv_from=0), dense(32))], width=40, vocab=50)


def config_d():
    """selective scan only (no paged cache at all)."""
    return config([(mamba(inner=56, state=4, dt_rank=2, conv=3), dense(48)), (mamba(inner=32, state=12, dt_rank=4, conv=7), None)],
                  width=32, vocab=40)


def config_e():
    """sizes nearer a small real model: a 192-wide latent (two column passes of the tensor-core kernel), 12 and 5 heads, a 64-wide
    recurrent state (several lanes per channel), 64 experts of which 6 are used, top == experts."""
    return config([(latent(heads=12, dim=32, rot_dim=16, vdim=48, kv_rank=192, q_rank=96, scale=0.15), dense(256)),
                   (mamba(inner=200, state=64, dt_rank=20, conv=4), moe(experts=64, top=6, ff=32, shared=64)),
                   (latent(heads=5, dim=64, rot_dim=16, vdim=32, kv_rank=192, q_rank=48, kv_from=0, scale=0.11), None),
                   (mamba(inner=384, state=24, dt_rank=8, conv=2), moe(experts=8, top=8, ff=64, shared=0))], width=160, vocab=300, eps=1e-6)


def shapes(cfg):
    W, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "head": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (W,)
        if layer["type"] == "latent_attention":
            H, d, rd, vd, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (Q, W), p + "mix.dq.norm": (Q,), p + "mix.uq": (H * (d + rd), Q), p + "mix.uk": (H * d, R),
                        p + "mix.uv": (H * vd, R), p + "mix.sink": (H,), p + "mix.o": (W, H * vd)})
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (R + rd, W), p + "mix.dkv.norm": (R,)})
        else:
            C, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            out.update({p + "mix.in": (2 * C, W), p + "mix.conv": (C, K), p + "mix.conv.b": (C,), p + "mix.x": (R + 2 * N, C),
                        p + "mix.dt": (C, R), p + "mix.dt.b": (C,), p + "mix.A_log": (C, N), p + "mix.D": (C,), p + "mix.o": (W, C)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            for k in range(mlp["router"]["experts"]):
                out[f"{p}mlp.e{k}.up"] = (mlp["expert"]["ff"], W)
                out[f"{p}mlp.e{k}.down"] = (W, mlp["expert"]["ff"])
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared"):
                s = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.up": (s, W), p + "mlp.shared.down": (W, s), p + "mlp.shared.sg": (1, W)})
    return out


def random_weights(cfg, seed=0):
    """bf16 tensors (what a checkpoint holds).  Scales keep activations O(1) and make routing and the recurrence matter."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith("norm") or name.endswith("norm1"):
            w = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            w = torch.log(0.5 + 4.0 * torch.rand(shape, generator=g))
        elif name.endswith("dt.b"):
            w = torch.log(torch.expm1(0.01 + 0.3 * torch.rand(shape, generator=g)))
        elif leaf in ("D", "sink") or name.endswith("conv.b"):
            w = torch.randn(shape, generator=g)
        elif name.endswith("mix.conv"):
            w = torch.randn(shape, generator=g) * 0.5
        elif name == "embed":
            w = torch.randn(shape, generator=g)
        else:
            w = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        W[name] = w.to(torch.bfloat16)
    return W


def write_checkpoint(path, cfg, weights):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
