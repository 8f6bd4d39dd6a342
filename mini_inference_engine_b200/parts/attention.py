"""Grouped-query attention over the paged cache (the mixer of Llama).

Projections q, k, v are fused into one matrix by concatenation on the output dimension, as the
reference does (inference_engine/model.py:103-107); q and k are rotated by the position part, k and
v are written to the layer's pages, and every new token attends causally to its request's
positions through the block table -- prompt portions and single decoded tokens in one kernel
(the reference has three paths: inference_engine/model.py:128-159).  ``window`` (None for Llama)
limits a query at position p to keys in (p - window, p].
"""
from __future__ import annotations

import math

import torch

from ..kernels import attention as attn_kernels
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, build_part, register_part


class Attention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position,
                 bias: bool = False, window: int | None = None, scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.bias = bias
        self.window = window
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)   # inference_engine/model.py:91
        self.position = build_part("position", position)

    def tensor_specs(self):
        H, Hkv, D, h = self.num_heads, self.num_kv_heads, self.head_dim, self.hidden_size
        specs = {"q_proj.weight": TensorSpec((H * D, h)), "k_proj.weight": TensorSpec((Hkv * D, h)),
                 "v_proj.weight": TensorSpec((Hkv * D, h)), "o_proj.weight": TensorSpec((h, H * D))}
        if self.bias:
            specs.update({"q_proj.bias": TensorSpec((H * D,), "zeros"), "k_proj.bias": TensorSpec((Hkv * D,), "zeros"),
                          "v_proj.bias": TensorSpec((Hkv * D,), "zeros")})
        specs.update(self.position.tensor_specs())       # a position encoding with tensors of its own
        return specs

    def bind(self, tensors, rt):
        self.rt = rt
        parts = [tensors[n + "_proj.weight"] for n in "qkv"]
        if len({p.dtype for p in parts}) > 1:          # mixed storage: widen to the widest
            parts = [p.float() for p in parts]
        self.w_qkv = rt.place(torch.cat(parts, 0))
        self.b_qkv = None
        if self.bias:
            self.b_qkv = rt.place(torch.cat([tensors[n + "_proj.bias"].float() for n in "qkv"], 0).to(
                torch.float32 if rt.dtype == torch.float32 else torch.bfloat16))
        self.w_o = rt.place(tensors["o_proj.weight"])
        self.position.bind({n: tensors[n] for n in self.position.tensor_specs()}, rt)

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    takes_sink = True

    def kernel_sources(self):
        import torch as _torch
        names = self.rt.product_sources(self.w_qkv, self.w_o) | self.position.kernel_sources()
        if self.rt.dtype == _torch.float32 or self.head_dim > 128:
            names.add("attention_simt")
        if self.rt.dtype != _torch.float32 and self.head_dim <= 128:
            names |= {"attention_decode", "attention_prefill_tc" if self.head_dim in (64, 128) else "attention_prefill"}
        return names

    def defers_norm(self, num_tokens: int) -> bool:
        return self.rt.defers_norm(num_tokens, self.w_qkv)

    def forward(self, x, ctx, cache, sink=None):
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        out = self.rt.empty(ctx.num_tokens, H * D)
        if getattr(self.position, "rotates_in_attention", None) and self.position.rotates_in_attention(x, self.w_qkv, ctx, cache):
            qkv = self.rt.linear(x, self.w_qkv, self.b_qkv)
            attn_kernels.attention(qkv, ctx, cache, out, H, Hkv, D, self.scale, self.window, rope=self.position.tables())
        else:
            qkv = self.position.project_rotate_and_store(x, self.w_qkv, self.b_qkv, ctx, cache, H, Hkv)
            attn_kernels.attention(qkv, ctx, cache, out, H, Hkv, D, self.scale, self.window)
        if sink is not None:
            done = self.rt.linear_into_stream(out, self.w_o, None, sink)
            if done is not None:
                return done
        return self.rt.linear(out, self.w_o)


class GatedAttention(Mixer):
    """Grouped-query softmax attention with the extras of some newer designs, each a parameter:

    * key/query size ``dim`` and value size ``vdim`` may differ (pages are as wide as the wider, tails zero);
    * ``qk_norm``: q and k are RMS-normed over their whole projection (all heads at once) with weights 'q.norm', 'k.norm';
    * rotation over the first ``rot_dims`` dims with frequencies that may be rescaled by wavelength (``rot_scaling``);
    * ``head_temp``: the score of head h is multiplied by 'temp'[h] (folded into the query);
    * ``chunk``: a query sees keys of its own block of that many positions only; ``window``: a sliding window;
    * ``gate``: the concatenated heads are multiplied by sigmoid(W_g h) before the output projection.

    q, k, v and the gate are one product; norm, rotation, temperature and the cache write one kernel; attention
    itself is the framework's paged kernels (decode and portions); the gate one more."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 rot_dims: int, rot_base: float, eps: float, rot_scaling: dict | None = None, qk_norm: bool = True,
                 head_temp: bool = True, gate: bool = True, chunk: int | None = None, window: int | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most dim {dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.dim, self.vdim = hidden_size, num_heads, num_kv_heads, dim, vdim
        self.padded = -(-max(dim, vdim) // 16) * 16          # the attention kernels take head sizes in steps of 16
        if self.padded > 256:
            raise ValueError(f"heads of {max(dim, vdim)}: the attention kernels take up to 256")
        self.scale, self.eps = float(scale), eps
        self.rot_dims, self.rot_base, self.rot_scaling = rot_dims, rot_base, rot_scaling
        self.qk_norm, self.head_temp, self.gate, self.chunk, self.window = qk_norm, head_temp, gate, chunk, window
        self.need = KVNeed(num_kv_heads, self.padded, window, chunk)

    def tensor_specs(self):
        H, G, D, Dv, h = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        specs = {"q": TensorSpec((H * D, h), "fan_in"), "k": TensorSpec((G * D, h), "fan_in"), "v": TensorSpec((G * Dv, h), "fan_in"),
                 "o": TensorSpec((h, H * Dv), "fan_in")}
        if self.gate:
            specs["g"] = TensorSpec((H * Dv, h), "fan_in")
        if self.qk_norm:
            specs.update({"q.norm": TensorSpec((H * D,), "normal:1:0.1"), "k.norm": TensorSpec((G * D,), "normal:1:0.1")})
        if self.head_temp:
            specs["temp"] = TensorSpec((H,), "uniform:0.5:2")
        return specs

    def bind(self, tensors, rt):
        from .rope import rotary_frequencies
        self.rt = rt
        parts = [tensors[n] for n in ("q", "k", "v") + (("g",) if self.gate else ())]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        self.w_in = rt.place(torch.cat(parts, 0))
        self.w_o = rt.place(tensors["o"])
        small = lambda n: tensors[n].float().to(rt.device).contiguous()        # read as float32 by the kernel
        self.q_norm = small("q.norm") if self.qk_norm else None
        self.k_norm = small("k.norm") if self.qk_norm else None
        self.temp = small("temp") if self.head_temp else None
        self.freq = rotary_frequencies(self.rot_dims, self.rot_base, self.rot_scaling).to(rt.device)

    def cache_need(self):
        return self.need

    def kernel_sources(self):
        names = self.rt.product_sources(self.w_in, self.w_o) | {"qk_norm_rope", "activation"}
        if self.rt.dtype == torch.float32 or self.padded > 128:
            names.add("attention_simt")
        else:
            names |= {"attention_decode", "attention_prefill_tc" if self.padded in (64, 128) else "attention_prefill"}
        return names

    def forward(self, x, ctx, cache):
        from ..kernels import ops
        H, G, D, Dv, DP = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.padded
        T = ctx.num_tokens
        proj = self.rt.linear(x, self.w_in)
        q = self.rt.empty(T, H, DP)
        ops.qk_norm_rope(proj, ctx.positions, ctx.slots[cache.group], self.freq, q, cache.k, cache.v, num_heads=H,
                         num_kv_heads=G, dim=D, vdim=Dv, rot=self.rot_dims, page_size=cache.page_size, eps=self.eps,
                         q_weight=self.q_norm, k_weight=self.k_norm, temp=self.temp, write_cache=cache.writes)
        heads = self.rt.empty(T, H, DP)
        attn_kernels.attention(q, ctx, cache, heads, H, G, DP, self.scale, self.need.mask(), q_stride=H * DP)
        if self.gate or DP != Dv:
            gated = self.rt.empty(T, H * Dv)
            if self.gate:
                ops.sigmoid_gate(heads, proj[:, (H + G) * D + G * Dv:], gated, H, Dv)
            else:
                gated.view(T, H, Dv).copy_(heads[:, :, :Dv])
        else:
            gated = heads.view(T, H * Dv)
        return self.rt.linear(gated, self.w_o, None, out_dtype=torch.float32)


register_part("mixer", "attention", Attention)
register_part("mixer", "gated_attention", GatedAttention)
