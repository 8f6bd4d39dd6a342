"""A recurrent block with a real-gated linear recurrent unit (the recurrent block of Griffin): two branches of
``width`` channels, y = gelu_tanh(W_y h + b_y) and u = causal_conv(W_x h + b_x); per block of channels
r = sigmoid(Ra u + ra), i = sigmoid(Ri u + ri); a = exp(-c r softplus(lam)); s_t = a s_{t-1} + sqrt(1 - a^2) i u;
output W_o (s y).  The state per request -- s and the convolution's last taps - 1 inputs, float32 -- is one
``StateNeed`` of ``taps`` rows.  The two input projections are one product with its bias; the convolution, the gates
and the scan (which also applies y and moves the convolution's inputs on) are one kernel each."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_part

SCAN_SEGMENT_TOKENS = 32      # a prompt portion is scanned in segments of at least this many tokens, up to 32 side by side


class GatedLinearRecurrence(Mixer):
    def __init__(self, hidden_size: int, width: int, blocks: int, taps: int, gate_constant: float = 8.0):
        if width % blocks:
            raise ValueError(f"{blocks} blocks do not divide {width} channels")
        if not 1 <= taps <= 8:
            raise ValueError(f"{taps} taps: the convolution kernel takes 1 to 8")
        self.hidden_size, self.width, self.blocks, self.taps, self.gate_constant = hidden_size, width, blocks, taps, gate_constant

    def tensor_specs(self):
        C, B, h, K = self.width, self.blocks, self.hidden_size, self.taps
        bw = C // B
        return {"y": TensorSpec((C, h), "fan_in"), "y.b": TensorSpec((C,), "normal:0:0.1"),
                "x": TensorSpec((C, h), "fan_in"), "x.b": TensorSpec((C,), "normal:0:0.1"),
                "conv": TensorSpec((C, K), "normal:0:0.5"), "conv.b": TensorSpec((C,), "normal:0:0.1"),
                "ra": TensorSpec((B, bw, bw), "fan_in"), "ra.b": TensorSpec((B, bw), "normal:0:0.5"),
                "ri": TensorSpec((B, bw, bw), "fan_in"), "ri.b": TensorSpec((B, bw), "normal:0:0.5"),
                "lam": TensorSpec((C,), "uniform:-4:0"), "o": TensorSpec((h, C), "fan_in")}

    def bind(self, tensors, rt):
        self.rt = rt
        wy, wx = tensors["y"], tensors["x"]
        if wy.dtype != wx.dtype:
            wy, wx = wy.float(), wx.float()
        self.w_yx = rt.place(torch.cat([wy, wx], 0))
        self.b_yx = rt.place(torch.cat([tensors["y.b"].float(), tensors["x.b"].float()], 0).to(
            torch.float32 if rt.dtype == torch.float32 else torch.bfloat16))
        small = {n: tensors[n].float() for n in ("conv", "conv.b", "ra", "ra.b", "ri", "ri.b", "lam")}   # read as float32 by the kernels
        for n, t in small.items():
            setattr(self, "p_" + n.replace(".", "_"), t.to(rt.device).contiguous())
        self.w_o = rt.place(tensors["o"])

    def cache_need(self):
        return StateNeed((self.taps, self.width), torch.float32)

    def kernel_sources(self):
        return {"linear_recurrence"} | self.rt.product_sources(self.w_yx, self.w_o)

    def forward(self, x, ctx, cache):
        C, T = self.width, ctx.num_tokens
        yx = self.rt.linear(x, self.w_yx, self.b_yx)
        y, xb = yx[:, :C], yx[:, C:]
        u = self.rt.empty(T, C, dtype=torch.float32)
        ops.causal_conv(xb, ctx.token_row, ctx.row_q_start, ctx.state_slots, self.p_conv, self.p_conv_b, cache.state, u)
        a, b = torch.empty_like(u), torch.empty_like(u)
        ops.recurrence_gates(u, self.p_ra, self.p_ra_b, self.p_ri, self.p_ri_b, self.p_lam, self.gate_constant, a, b)
        out = self.rt.empty(T, C)
        segments = max(1, min(32, ctx.max_q_len // SCAN_SEGMENT_TOKENS))
        ops.recurrence_scan(a, b, y, xb, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, cache.state, out, segments)
        return self.rt.linear(out, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "gated_linear_recurrence", GatedLinearRecurrence)
