"""Small Tipetar configurations with random weights for the tests, written out as checkpoint directories."""
from __future__ import annotations

import torch

from tafopel_helpers import tokens, write_checkpoint  # noqa: F401  (shared: token streams, checkpoint writer)


def attn(heads=4, kv_heads=2, dim=16, vdim=16, window=24, scale=0.25, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def moe(experts=6, identity=2, top=2, groups=(2, 1), ff=24, shared=16, scale=1.25):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "identity": identity, "top": top, "scale": scale, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def config(layers, width=64, vocab=97, eps=2e-5, mult=0.6):
    return {"architecture": "Tipetar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": [dict(l, mlp=mlp) for l, mlp in layers]}


def config_a():
    """two key/value heads, a window shorter than a page and one longer than two, a layer reading an earlier layer's keys with
    other head counts per group, a layer without feed-forward, identity experts, groups 2 keep 1 and 3 keep 2."""
    return config([(attn(), moe()),
                   (attn(heads=6, kv_heads=2, dim=16, vdim=16, window=40, kv_from=0, scale=0.2), moe(experts=7, identity=2, top=3, groups=(3, 2), ff=16, shared=0)),
                   (attn(heads=2, kv_heads=2, dim=8, vdim=24, window=9), None),
                   (attn(heads=4, kv_heads=2, dim=16, vdim=16, window=7, kv_from=0), moe(experts=4, identity=0, top=1, groups=(1, 1), ff=40, shared=8, scale=1.0))])


def config_b():
    """one head, dims that are no multiple of 16, vdim != dim, window 1 (a token sees itself only) and a window longer than
    any test sequence, top == all open experts, residual multiplier 1, odd width."""
    return config([(attn(heads=1, kv_heads=1, dim=12, vdim=20, window=1, scale=0.3), moe(experts=2, identity=2, top=2, groups=(2, 1), ff=8, shared=12, scale=2.0)),
                   (attn(heads=5, kv_heads=5, dim=8, vdim=4, window=100000, scale=0.35), moe(experts=8, identity=0, top=3, groups=(4, 2), ff=16, shared=8)),
                   (attn(heads=3, kv_heads=1, dim=20, vdim=12, window=33, scale=0.2), None)], width=44, vocab=61, mult=1.0, eps=1e-6)


def config_c():
    """sizes of the tensor-core attention path (head sizes 64 and 32, eight query heads per key/value head and one), windows
    around the 64-key tile (63, 64, 65, 130), two borrowing layers, sixteen router outputs in four groups."""
    return config([(attn(heads=8, kv_heads=1, dim=64, vdim=64, window=65, scale=0.125), moe(experts=12, identity=4, top=3, groups=(4, 2), ff=32, shared=48)),
                   (attn(heads=4, kv_heads=4, dim=32, vdim=32, window=64, scale=0.18), moe(experts=5, identity=1, top=2, groups=(1, 1), ff=24, shared=0)),
                   (attn(heads=8, kv_heads=1, dim=64, vdim=64, window=130, kv_from=0, scale=0.125), None),
                   (attn(heads=16, kv_heads=1, dim=64, vdim=64, window=63, kv_from=0, scale=0.1), moe(experts=3, identity=3, top=2, groups=(3, 2), ff=64, shared=16))],
                  width=128, vocab=211, mult=0.7)


def shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (W,), p + "mix.q": (H * d, W), p + "mix.q.norm": (H * d,), p + "mix.o": (W, H * vd)})
        if m.get("kv_from") is None:
            out.update({p + "mix.k": (G * d, W), p + "mix.v": (G * vd, W), p + "mix.k.norm": (G * d,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        r = mlp["router"]
        out[p + "norm2"] = (W,)
        for k in range(r["experts"]):
            out.update({f"{p}mlp.e{k}.gate": (mlp["expert"]["ff"], W), f"{p}mlp.e{k}.up": (mlp["expert"]["ff"], W),
                        f"{p}mlp.e{k}.down": (W, mlp["expert"]["ff"])})
        n_out = r["experts"] + r.get("identity", 0)
        out.update({p + "mlp.router": (n_out, W), p + "mlp.correction": (n_out,)})
        if mlp.get("shared"):
            s = mlp["shared"]["ff"]
            out.update({p + "mlp.shared.gate": (s, W), p + "mlp.shared.up": (s, W), p + "mlp.shared.down": (W, s)})
    return out


def random_weights(cfg, seed=0):
    """bf16 tensors (what a checkpoint holds).  Router rows are large enough that the softmax is far from uniform, and the
    corrections are of the order of the scores, so that correction, groups and identity experts all change the choice."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name.endswith(("norm1", "norm2", "final.norm")):
            w = 0.3 * torch.randn(shape, generator=g)
        elif leaf == "norm":
            w = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif leaf == "correction":
            w = 0.15 * torch.randn(shape, generator=g)
        elif leaf == "router":
            w = torch.randn(shape, generator=g) * (2.5 / shape[-1] ** 0.5)
        elif name == "embed":
            w = torch.randn(shape, generator=g)
        else:
            w = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        W[name] = w.to(torch.bfloat16)
    return W
