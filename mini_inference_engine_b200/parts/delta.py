"""The gated delta rule with a decay per head and key channel: a linear-attention mixer with a float32 state per request
and head,

    S <- diag(g_t) S;   u_t = beta_t (v_t - S^T k_t);   S <- S + k_t u_t^T;   o_t = S^T q_t,

where q, k (``num_kv_heads`` x ``dim``) and v (``num_heads`` x ``vdim``) each pass a short causal convolution over time per
channel and silu, q and k are unit vectors per head (q times dim^-1/2), beta = sigmoid(W_b h) per head, and
g = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias)) per head and key channel.  Each head's o is divided by its root
mean square, multiplied by a weight shared by the heads and by sigmoid(W_g2 W_g1 h), and projected by W_o.

Products: q|k|v|beta of the input are one, the two low-rank down-projections (a1|g1) one, and their up-projections one
block-diagonal product that leaves float32.  The convolution, activations, unit norms and decays are one kernel, the
recurrence one, the head norm and gate one.  Two states (a tuple of needs): S [heads, vdim, dim] and the
convolution's last taps - 1 inputs."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .attention import _padded_rows
from .base import Mixer, StateNeed, register_part


class ChannelDelta(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 decay_rank: int | None = None, gate_rank: int | None = None, unit_eps: float = 1e-6):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if taps < 1:
            raise ValueError("the convolution has at least one tap")
        if dim > 512:
            raise ValueError(f"key size {dim}: the recurrence kernel takes up to 512")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim = hidden_size, num_heads, num_kv_heads, dim, vdim
        self.taps, self.eps, self.unit_eps = taps, eps, unit_eps
        self.decay_rank, self.gate_rank = decay_rank, gate_rank        # None: taken from the tensors' shapes when they are bound

    def tensor_specs(self):
        H, G, D, Dv, h, K = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size, self.taps
        ra, rg = self.decay_rank or -1, self.gate_rank or -1          # a rank that the configuration does not give comes from the tensors
        da, dg = self.decay_rank or max(8, D // 4), self.gate_rank or max(8, D // 4)
        low = lambda shape, default: TensorSpec(shape, "fan_in", default)
        return {"q": TensorSpec((G * D, h), "fan_in"), "q.conv": TensorSpec((G * D, K), "normal:0:0.5"),
                "k": TensorSpec((G * D, h), "fan_in"), "k.conv": TensorSpec((G * D, K), "normal:0:0.5"),
                "v": TensorSpec((H * Dv, h), "fan_in"), "v.conv": TensorSpec((H * Dv, K), "normal:0:0.5"),
                "b": TensorSpec((H, h), "fan_in"), "A_log": TensorSpec((H,), "uniform:-3:0.5"),
                "norm": TensorSpec((Dv,), "normal:1:0.1"), "a1": low((ra, h), (da, h)), "a2": low((H * D, ra), (H * D, da)),
                "dt_bias": TensorSpec((H * D,), "uniform:-4:1"), "g1": low((rg, h), (dg, h)),
                "g2": low((H * Dv, rg), (H * Dv, dg)), "o": TensorSpec((h, H * Dv), "fan_in")}

    def bind(self, tensors, rt):
        self.rt = rt
        H, D, Dv = self.num_heads, self.dim, self.vdim
        w, _ = _padded_rows([tensors[n] for n in ("q", "k", "v", "b")])
        self.w_in = rt.place(w)
        ra, rg = tensors["a1"].shape[0], tensors["g1"].shape[0]
        if tensors["a2"].shape[1] != ra or tensors["g2"].shape[1] != rg:
            raise ValueError(f"low-rank pairs do not fit: a1 {tuple(tensors['a1'].shape)} with a2 {tuple(tensors['a2'].shape)}, "
                             f"g1 {tuple(tensors['g1'].shape)} with g2 {tuple(tensors['g2'].shape)}")
        low, self.low_rows = _padded_rows([tensors["a1"], tensors["g1"]])
        self.w_low = rt.place(low)
        a2, g2 = tensors["a2"], tensors["g2"]
        if a2.dtype != g2.dtype:
            a2, g2 = a2.float(), g2.float()
        up = torch.zeros(H * D + H * Dv, low.shape[0], dtype=a2.dtype)       # block-diagonal: a-rows read a1's outputs, gate rows g1's
        up[:H * D, :ra] = a2
        up[H * D:, ra:ra + rg] = g2
        self.w_up = rt.place(up)
        self.w_o = rt.place(tensors["o"])
        small = lambda t: t.float().to(rt.device).contiguous()               # read as float32 by the kernels
        self.conv = small(torch.cat([tensors["q.conv"].float(), tensors["k.conv"].float(), tensors["v.conv"].float()], 0))
        self.a_log, self.dt_bias, self.norm = small(tensors["A_log"]), small(tensors["dt_bias"]), small(tensors["norm"])

    def cache_need(self):
        C = 2 * self.num_kv_heads * self.dim + self.num_heads * self.vdim
        return (StateNeed((self.num_heads, self.vdim, self.dim), torch.float32), StateNeed((self.taps - 1, C), torch.float32))

    def kernel_sources(self):
        return {"delta_rule"} | self.rt.product_sources(self.w_in, self.w_low, self.w_up, self.w_o)

    def forward(self, x, ctx, cache):
        H, G, D, Dv, T = self.num_heads, self.num_kv_heads, self.dim, self.vdim, ctx.num_tokens
        state, conv_state = cache.parts[0].state, cache.parts[1].state
        proj = self.rt.linear(x, self.w_in)
        low = self.rt.linear(self.rt.linear(x, self.w_low), self.w_up, None, out_dtype=torch.float32)     # [a: H x D | gate: H x Dv]
        f32 = lambda n: self.rt.empty(T, n, dtype=torch.float32)
        qn, kn, vn, beta, decay, kq = f32(G * D), f32(G * D), f32(H * Dv), f32(H), f32(H * D), f32(G)
        ops.delta_prepare(proj, low, self.conv, conv_state, ctx.token_row, ctx.row_q_start, ctx.state_slots, self.a_log, self.dt_bias,
                          qn, kn, vn, beta, decay, kq, num_heads=H, num_kv_heads=G, dim=D, vdim=Dv, unit_eps=self.unit_eps)
        if self.taps > 1:
            ops.conv_state_update(proj, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, conv_state)
        o = f32(H * Dv)
        ops.delta_scan(qn, kn, vn, beta, decay, kq, ctx.row_q_start, ctx.row_q_len, ctx.state_slots, state, o, num_heads=H,
                       num_kv_heads=G, dim=D, vdim=Dv)
        gated = self.rt.empty(T, H * Dv)
        ops.head_norm_gate(o, low[:, H * D:], self.norm, gated, H, Dv, self.eps)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "channel_delta", ChannelDelta)
