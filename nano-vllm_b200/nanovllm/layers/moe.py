"""Feed-forward blocks of hybrid decoders: a gated dense block and a routed mixture of small experts.

Dense:   W_down (gelu_tanh(W_gate h) * (W_up h))
Routed:  z = W_router h (fp32), s = sigmoid(z); the `top` experts with the largest s get weight s (not renormalised);
         the weight scales the expert's INPUT:  out = sum_e expert_e(s_e h),  expert(x) = W_down relu(W_up x)^2;
         an optional shared expert of the same form runs for every token, scaled by sigmoid(W_sg h).

The routed path groups (token, choice) pairs by expert on the device and runs two grouped GEMMs over the grouped rows; the
router (and the shared gate, one more row of the same fp32 GEMM) never leave fp32.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


class GatedDenseFF:
    def __init__(self, width: int, mlp: dict, dtype, device):
        self.ff = int(mlp["ff"])
        self.w_gate_up = torch.empty(2 * self.ff, width, dtype=dtype, device=device)
        self.w_down = torch.empty(width, self.ff, dtype=dtype, device=device)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        if leaf == "gate":
            self.w_gate_up[:self.ff].copy_(w)
        elif leaf == "up":
            self.w_gate_up[self.ff:].copy_(w)
        elif leaf == "down":
            self.w_down.copy_(w)
        else:
            return False
        return True

    def forward(self, h: torch.Tensor):
        """-> (T tensor, None)"""
        return F.linear(mixops.ff_act(F.linear(h, self.w_gate_up), mixops.FF_GELU_TANH_MUL), self.w_down), None


class RoutedExpertsFF:
    def __init__(self, width: int, mlp: dict, dtype, device):
        self.experts, self.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        self.ff = int(mlp["expert"]["ff"])
        shared = mlp.get("shared")
        self.shared_ff = int(shared["ff"]) if shared else 0
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.w_up = e(self.experts, self.ff, width)
        self.w_down = e(self.experts, width, self.ff)
        self.w_router = torch.zeros(self.experts + (1 if shared else 0), width, dtype=torch.float32, device=device)  # + shared gate row
        if shared:
            self.sh_up, self.sh_down = e(self.shared_ff, width), e(width, self.shared_ff)

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        parts = leaf.split(".")
        if parts[0].startswith("e") and parts[0][1:].isdigit() and len(parts) == 2:
            k = int(parts[0][1:])
            if parts[1] == "up":
                self.w_up[k].copy_(w)
            elif parts[1] == "down":
                self.w_down[k].copy_(w)
            else:
                return False
        elif leaf == "router":
            self.w_router[:self.experts].copy_(w.float())
        elif leaf == "shared.up" and self.shared_ff:
            self.sh_up.copy_(w)
        elif leaf == "shared.down" and self.shared_ff:
            self.sh_down.copy_(w)
        elif leaf == "shared.sg" and self.shared_ff:
            self.w_router[self.experts].copy_(w.float().view(-1))
        else:
            return False
        return True

    def forward(self, h: torch.Tensor):
        """-> (None, fp32 tensor)"""
        n = h.shape[0]
        logits = F.linear(h.float(), self.w_router)
        idx, wgt = mixops.moe_route(logits, self.experts, self.top)
        sorted_rows, pos_of, tile_expert, num_tiles = mixops.moe_align(idx, self.experts)
        inter = mixops.moe_gemm(h, sorted_rows, tile_expert, num_tiles, self.w_up, wgt=wgt, top=self.top, act=1)
        rows = mixops.moe_gemm(inter, sorted_rows, tile_expert, num_tiles, self.w_down, out_f32=True)
        shared = gate = None
        if self.shared_ff:
            shared = F.linear(mixops.ff_act(F.linear(h, self.sh_up), mixops.FF_RELU2), self.sh_down)
            gate = logits[:, self.experts]
        return None, mixops.moe_combine(rows, pos_of, self.top, n, shared, gate)
