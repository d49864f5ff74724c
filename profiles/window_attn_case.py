"""One small case of the windowed attention kernel for an `ncu` capture: `python profiles/window_attn_case.py prefill|decode`
(16 query heads over 8 key/value heads of 128: a 4 x 2048-token prompt step with a 1024-token window, or a single-token step over
64 x 4096 cached tokens without a window)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "nano-vllm_b200"))

from nanovllm import mixops  # noqa: E402
from nanovllm.layers.window_attention import distance_slopes  # noqa: E402

H, G, d, bs, dev = 16, 8, 128, 256, "cuda"
S, q, k, win = (4, 2048, 2048, 1024) if sys.argv[1] == "prefill" else (64, 1, 4096, 0)
nblk = S * (k // bs)
cache = torch.randn(nblk * bs, G * 2 * d, device=dev).bfloat16()
bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(S, -1)
qkv = torch.randn(S * q, H * d, device=dev).bfloat16()
if q > 1:
    cu = torch.arange(0, S + 1, dtype=torch.int32, device=dev)
    sp = mixops.StepSpans(S, q, cu * q, cu * k, None)
else:
    sp = mixops.StepSpans(S, 1, None, None, torch.full((S,), k, dtype=torch.int32, device=dev))
for _ in range(4):
    o = mixops.window_attention(qkv, cache, bt, bs, sp, H, G, d, d, 0.088, distance_slopes(H, dev), win)
torch.cuda.synchronize()
print("ok", float(o.float().abs().mean()))
