"""Mamba-1 mixer: gated selective state-space recurrence with a short causal convolution in front.

    [x | z] = W_in h                         u = silu(conv(x) + b)                  (depthwise, `taps` wide, causal)
    [dt_in | B | C] = W_x u                  dt = softplus(W_dt dt_in + b_dt)      (per channel, fp32)
    S <- exp(dt A) S + dt u B                y = S C + D u                         (A = -exp(A_log); S fp32 [inner, state])
    out = W_o (y * silu(z))

Per sequence the layer keeps S and the last taps - 1 values of x in a state slot; the slot index of every sequence of a
step arrives in ``ctx.state_slots``.  Prompt portions, single tokens and mixed batches all run the same two kernels.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import mixops


class SelectiveScanMixer:
    kind = "mamba1"

    def __init__(self, width: int, m: dict, dtype, device):
        self.width, self.dtype, self.device = width, dtype, device
        self.inner, self.nstate, self.dt_rank, self.taps = int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"])
        if self.nstate > 128:
            raise ValueError(f"state {self.nstate}: the scan kernels hold at most 128 states per channel")
        e = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        C, N, R = self.inner, self.nstate, self.dt_rank
        self.w_in = e(2 * C, width)
        self.conv_w, self.conv_b = e(C, self.taps), e(C)
        self.w_x = e(R + 2 * N, C)
        self.w_dt, self.dt_b = e(C, R), e(C)
        self.A = torch.zeros(C, N, dtype=torch.float32, device=device)      # -exp(A_log), formed once in fp32
        self.D = e(C)
        self.w_o = e(width, C)
        self.conv_state = None        # [slots, taps - 1, inner] fp32
        self.ssm_state = None         # [slots, inner, state] fp32

    def load(self, leaf: str, w: torch.Tensor) -> bool:
        named = {"in": self.w_in, "conv": self.conv_w, "conv.b": self.conv_b, "x": self.w_x, "dt": self.w_dt, "dt.b": self.dt_b,
                 "D": self.D, "o": self.w_o}
        if leaf == "A_log":
            self.A.copy_(-torch.exp(w.float()))
        elif leaf in named:
            named[leaf].copy_(w)
        else:
            return False
        return True

    def state_slot_bytes(self) -> int:
        return 4 * (max(self.taps - 1, 1) * self.inner + self.inner * self.nstate)

    def bind_state(self, num_slots: int) -> None:
        self.conv_state = torch.zeros(num_slots, max(self.taps - 1, 1), self.inner, dtype=torch.float32, device=self.device)
        self.ssm_state = torch.zeros(num_slots, self.inner, self.nstate, dtype=torch.float32, device=self.device)

    def forward(self, h: torch.Tensor, positions: torch.Tensor, ctx, spans: mixops.StepSpans) -> torch.Tensor:
        C, N, R = self.inner, self.nstate, self.dt_rank
        xz = F.linear(h, self.w_in)
        u = mixops.causal_conv(xz[:, :C], self.conv_w, self.conv_b, self.conv_state, ctx.state_slots, spans)
        dbc = F.linear(u, self.w_x)
        dt_raw = F.linear(dbc[:, :R], self.w_dt)
        y = mixops.selective_scan(u, dt_raw, self.dt_b, self.A, dbc[:, R:R + N], dbc[:, R + N:], self.D, xz[:, C:],
                                  self.ssm_state, ctx.state_slots, spans)
        return F.linear(y, self.w_o)
