"""Grouped-query attention with a sliding window and a linear distance bias, without any rotation.

    q = norm_all(W_q h) * g_q        k = norm_all(W_k h) * g_k        v = W_v h
        (norm_all: ONE root mean square over the whole projection of a token, all heads together, then a weight per column)
    s[h, i, j] = (q_i[h] . k_j[h // (H / G)]) * scale - slope[h] * (i - j),   slope[h] = 2^(-8 (h + 1) / H)
    visible j:  0 <= i - j < window        p = softmax over the visible j        out = W_o concat_h (sum_j p_j v_j)

Positions enter only through the bias and the window, so the cached keys are position-free: per token the cache holds one
row ``[k (G * dim) | v (G * vdim)]`` (keys after their norm) for every layer that owns a key/value projection.  A layer with
``kv_from`` has no key/value tensors: it reads the named layer's cache rows with its own queries, window, scale and bias.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


def distance_slopes(heads: int, device) -> torch.Tensor:
    """slope[h] = 2^(-8 (h + 1) / heads), fp32."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return torch.exp2(-8.0 * h / heads).to(torch.float32).to(device)


class BiasedWindowAttention:
    kind = "attention"

    def __init__(self, width: int, m: dict, eps: float, dtype, device):
        self.width, self.eps, self.dtype, self.device = width, eps, dtype, device
        self.heads, self.kv_heads = int(m["heads"]), int(m["kv_heads"])
        self.dim, self.vdim = int(m["dim"]), int(m["vdim"])
        self.scale = float(m["scale"])
        mask = m.get("mask") or {}
        self.window = int(mask.get("size") or 0)                  # 0: every earlier token is visible
        self.kv_from = m.get("kv_from")
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if self.vdim > 512:
            raise ValueError(f"vdim {self.vdim}: the attention kernels hold at most 512 output columns per query row")
        self.q_cols = self.heads * self.dim
        self.k_cols = 0 if self.kv_from is not None else self.kv_heads * self.dim
        self.v_cols = 0 if self.kv_from is not None else self.kv_heads * self.vdim
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_qkv = e(self.q_cols + self.k_cols + self.v_cols, width)       # [W_q ; W_k ; W_v]: one GEMM reads h once
        self.q_norm = e(self.q_cols)
        self.k_norm = e(self.k_cols) if self.kv_from is None else None
        self.w_o = e(width, self.heads * self.vdim)
        self.slopes = distance_slopes(self.heads, device)
        self.cache = None                                 # [num_blocks * block_size, G * (dim + vdim)]; the source layer's when kv_from
        self.block_size = 0

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        own = self.kv_from is None
        if leaf == "q":
            self.w_qkv[:self.q_cols].copy_(w)
        elif leaf == "k" and own:
            self.w_qkv[self.q_cols:self.q_cols + self.k_cols].copy_(w)
        elif leaf == "v" and own:
            self.w_qkv[self.q_cols + self.k_cols:].copy_(w)
        elif leaf == "q.norm":
            self.q_norm.copy_(w)
        elif leaf == "k.norm" and own:
            self.k_norm.copy_(w)
        elif leaf == "o":
            self.w_o.copy_(w)
        else:
            return False
        return True

    def weight_shapes(self, width: int) -> dict:
        out = {"q": (self.q_cols, width), "q.norm": (self.q_cols,), "o": (width, self.heads * self.vdim)}
        if self.kv_from is None:
            out.update({"k": (self.k_cols, width), "v": (self.v_cols, width), "k.norm": (self.k_cols,)})
        return out

    def cache_row_elems(self) -> int:
        """Cached elements per token (0 for a layer that borrows another layer's cache)."""
        return self.k_cols + self.v_cols

    def forward(self, h: torch.Tensor, ctx, spans: mixops.StepSpans) -> torch.Tensor:
        qkv = F.linear(h, self.w_qkv)
        mixops.qk_norm_store(qkv, self.q_cols, self.k_cols, self.v_cols, self.q_norm, self.k_norm, ctx.slot_mapping,
                             self.cache if self.kv_from is None else None, self.eps)
        o = mixops.window_attention(qkv, self.cache, ctx.block_tables, self.block_size, spans, self.heads, self.kv_heads, self.dim,
                                    self.vdim, self.scale, self.slopes, self.window)
        return F.linear(o, self.w_o)
