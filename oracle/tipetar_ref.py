"""Plain implementation of the Tipetar decoder: float64, whole sequences, no cache, no batching, one function per mechanism.
Test infrastructure only: it shares no code with the product path and is written from the design's equations.

Weights: a dict name -> tensor (any float dtype; cast to float64 here).  Linear weights are [out, in] and applied as W x.

    layer:        x <- x + m * out_norm(mixer(x), g1);  x <- x + m * out_norm(ff(x), g2)       (sublayers read x itself)
    out_norm:     y / sqrt(mean(y^2) + eps) * (1 + g)
    mixer:        windowed grouped-query attention with whole-projection query/key norms and a linear distance bias
    ff:           group-routed experts (softmax router, choice correction, identity experts, shared expert)
    output:       logits = head (out_norm-style norm of x with 'final.norm')
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def out_norm(y: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero."""
    return unit_rms(y, eps) * (1.0 + g.to(F64))


def slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F64)


def visible(n: int, window: int) -> torch.Tensor:
    """[n, n] bool: query i sees key j when 0 <= i - j < window (window 0: every j <= i)."""
    d = torch.arange(n)[:, None] - torch.arange(n)[None, :]
    ok = d >= 0
    if window:
        ok &= d < window
    return ok


def windowed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, kv_heads: int, scale: float, window: int,
                       bias: bool = True) -> torch.Tensor:
    """q [n, heads * dim], k [n, kv_heads * dim], v [n, kv_heads * vdim] -> [n, heads * vdim], one query head at a time."""
    n = q.shape[0]
    q, k, v = q.view(n, heads, -1), k.view(n, kv_heads, -1), v.view(n, kv_heads, -1)
    dist = (torch.arange(n)[:, None] - torch.arange(n)[None, :]).to(F64)
    see = visible(n, window)
    sl = slopes(heads)
    outs = []
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = (q[:, h] @ k[:, g].T) * scale
        if bias:
            s = s - sl[h] * dist
        s = torch.where(see, s, torch.full_like(s, -math.inf))
        outs.append(torch.softmax(s, -1) @ v[:, g])
    return torch.cat(outs, -1)


def attention_layer(W: dict, p: str, m: dict, x: torch.Tensor, eps: float, shared_kv: dict, index: int) -> torch.Tensor:
    w = lambda leaf: W[p + leaf].to(F64)
    q = unit_rms(x @ w("q").T, eps) * w("q.norm")                  # one statistic over all heads
    src = m.get("kv_from")
    if src is None:
        k = unit_rms(x @ w("k").T, eps) * w("k.norm")
        v = x @ w("v").T
        shared_kv[index] = (k, v)
    else:
        k, v = shared_kv[src]
    window = int((m.get("mask") or {}).get("size") or 0)
    o = windowed_attention(q, k, v, m["heads"], m["kv_heads"], m["scale"], window)
    return o @ w("o").T


def gated_expert(W: dict, p: str, x: torch.Tensor) -> torch.Tensor:
    a = x @ W[p + "gate"].to(F64).T
    return (a * torch.sigmoid(a) * (x @ W[p + "up"].to(F64).T)) @ W[p + "down"].to(F64).T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int, scale: float):
    """z [n, outputs] router logits -> (chosen outputs [n, top], weights [n, top])."""
    n, E = z.shape
    s = torch.softmax(z, -1)
    c = s + correction
    if groups > 1 and keep < groups:
        per = c.view(n, groups, E // groups)
        best = per.max(-1).values.topk(keep, -1).indices
        open_ = torch.zeros(n, groups, dtype=torch.bool).scatter_(1, best, True)
        c = torch.where(open_[:, :, None], per, torch.full_like(per, -math.inf)).reshape(n, E)
    chosen = c.topk(top, -1).indices
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def routed_ff(W: dict, p: str, mlp: dict, x: torch.Tensor) -> torch.Tensor:
    r = mlp["router"]
    real, ident = int(r["experts"]), int(r.get("identity") or 0)
    g = r.get("groups") or {}
    z = x @ W[p + "router"].to(F64).T
    chosen, wgt = route(z, W[p + "correction"].to(F64).view(-1), int(r["top"]), int(g.get("count") or 1), int(g.get("keep") or 1),
                        float(r.get("scale", 1.0)))
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, w in zip(chosen[t].tolist(), wgt[t]):
            out[t] += w * (x[t] if e >= real else gated_expert(W, f"{p}e{e}.", x[t:t + 1])[0])
    if mlp.get("shared"):
        out = out + gated_expert(W, p + "shared.", x)
    return out


def forward(cfg: dict, W: dict, tokens, taps: list | None = None) -> torch.Tensor:
    """-> logits [n, vocab] (float64) of every position of one sequence."""
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    shared_kv: dict = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + mult * out_norm(attention_layer(W, p + "mix.", layer["mixer"], x, eps, shared_kv, i), W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + mult * out_norm(routed_ff(W, p + "mlp.", layer["mlp"], x), W[p + "norm2"], eps)
        if taps is not None:
            taps.append(x.clone())
    return out_norm(x, W["final.norm"], eps) @ W["head"].to(F64).T
