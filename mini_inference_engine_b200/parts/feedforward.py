"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)).  gate and up are fused into one matrix
(inference_engine/model.py:109,180-181 concatenates them on the output dimension).  In bfloat16 the
fused matrix interleaves them instead -- row 2i = gate_i, row 2i+1 = up_i -- so that the tensor-core
product can apply SwiGLU in its epilogue while both values of a pair sit side by side."""
from __future__ import annotations

import torch

from ..kernels import linear as linear_kernels
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, register_part


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate_proj.weight": TensorSpec((i, h)), "up_proj.weight": TensorSpec((i, h)),
                "down_proj.weight": TensorSpec((h, i))}

    def bind(self, tensors, rt):
        self.rt = rt
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.interleaved = rt.dtype == torch.bfloat16 and g.dtype != torch.float32
        if self.interleaved:
            self.w_gate_up = rt.place(torch.stack((g, u), 1).reshape(2 * self.intermediate_size, self.hidden_size))
        else:
            self.w_gate_up = rt.place(torch.cat([g, u], 0))
        self.w_down = rt.place(tensors["down_proj.weight"])

    takes_sink = True

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_gate_up, self.w_down)

    def defers_norm(self, num_tokens: int) -> bool:
        return self.rt.defers_norm(num_tokens, self.w_gate_up)

    def forward(self, x, ctx, sink=None):
        if self.interleaved:
            act = linear_kernels.linear_swiglu(x, self.w_gate_up, self.rt.dtype)
        else:
            gu = self.rt.linear(x, self.w_gate_up)
            act = self.rt.empty(x.shape[0], self.intermediate_size)
            ops.swiglu(gu, act)
        if sink is not None:
            done = self.rt.linear_into_stream(act, self.w_down, None, sink)
            if done is not None:
                return done
        return self.rt.linear(act, self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)


class ClampedGLU(FeedForward):
    """A gated feed-forward with clamps: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
    output W_down (g sigmoid(slope g) (u + shift)).  gate and up are one product; in bfloat16 the tensor-core
    products apply the gate to their float32 sums in the epilogue (rows interleaved, as for SwiGLU), elsewhere one
    kernel does in float32; the last product leaves float32 for the stream's sum."""

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, slope: float = 1.702, shift: float = 1.0):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit, self.slope, self.shift = float(limit), float(slope), float(shift)

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {"gate": TensorSpec((i, h), "fan_in"), "up": TensorSpec((i, h), "fan_in"), "down": TensorSpec((h, i), "fan_in")}

    def bind(self, tensors, rt):
        self.rt = rt
        g, u = tensors["gate"], tensors["up"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        # in bfloat16 the rows alternate gate_i, up_i, as for SwiGLU: the tensor-core products then apply the gate in
        # their epilogue (the same epilogue with this part's constants)
        self.interleaved = rt.dtype == torch.bfloat16 and g.dtype != torch.float32
        if self.interleaved:
            self.w_gate_up = rt.place(torch.stack((g, u), 1).reshape(2 * self.intermediate_size, self.hidden_size))
        else:
            self.w_gate_up = rt.place(torch.cat([g, u], 0))
        self.w_down = rt.place(tensors["down"])

    def kernel_sources(self):
        return {"activation"} | self.rt.product_sources(self.w_gate_up, self.w_down)

    def forward(self, x, ctx):
        if self.interleaved:
            act = linear_kernels.linear_swiglu(x, self.w_gate_up, self.rt.dtype, glu=(self.limit, self.slope, self.shift))
        else:
            gu = self.rt.linear(x, self.w_gate_up)
            act = self.rt.empty(x.shape[0], self.intermediate_size)
            ops.glu_clamped(gu, act, self.limit, self.slope, self.shift)
        return self.rt.linear(act, self.w_down, None, out_dtype=torch.float32)


register_part("feed_forward", "clamped_glu", ClampedGLU)


GROUPED_MIN_TOKENS = 32      # = kernels.linear.AUTO_MAX_TOKENS: above it the plain products are the library's too


class RoutedExperts(FeedForward):
    """A mixture of ``num_experts`` small feed-forward layers 'e<i>.up' [ff, hidden], 'e<i>.down' [hidden, ff] without
    biases, expert(h) = down act(up h).  Router logits 'router' [experts, hidden] are computed in float32; each token
    uses the ``top`` experts with the largest logits, weighted by the softmax over those logits only.

    All experts' up matrices are stacked into one and their down matrices laid side by side.  Many tokens (prompt
    portions, large batches): with the activations of the experts a token did not choose set to zero and those it chose
    multiplied by their weight, the layer is ONE wide feed-forward -- two products of the framework on the tensor cores
    and one kernel between them.  A handful of tokens (no more (token, expert) pairs than experts): every pair streams
    its own expert's rows and no others, so a decoding step reads only the experts that were chosen.  Many tokens in
    bfloat16 where a token uses at most half of the experts: the pairs are sorted by expert and both products run expert
    by expert over those rows (the library's grouped product), so no expert computes for a token that did not choose it."""

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, activation: str = "relu2"):
        if not 1 <= top <= num_experts:
            raise ValueError(f"top {top} of {num_experts} experts")
        if activation not in ops.EXPERT_ACTIVATIONS:
            raise ValueError(f"activation {activation!r}; one of {', '.join(ops.EXPERT_ACTIVATIONS)}")
        self.hidden_size, self.num_experts, self.top, self.expert_size, self.activation = hidden_size, num_experts, top, expert_size, activation

    def tensor_specs(self):
        h, F = self.hidden_size, self.expert_size
        specs = {"router": TensorSpec((self.num_experts, h), "fan_in")}
        for e in range(self.num_experts):
            specs[f"e{e}.up"] = TensorSpec((F, h), "fan_in")
            specs[f"e{e}.down"] = TensorSpec((h, F), "fan_in")
        return specs

    def bind(self, tensors, rt):
        self.rt = rt
        ups = [tensors[f"e{e}.up"] for e in range(self.num_experts)]
        downs = [tensors[f"e{e}.down"] for e in range(self.num_experts)]
        if len({t.dtype for t in ups + downs}) > 1:
            ups, downs = [t.float() for t in ups], [t.float() for t in downs]
        self.w_up = rt.place(torch.cat(ups, 0))                      # [E * F, hidden]
        self.w_down = rt.place(torch.cat(downs, 1))                  # [hidden, E * F]
        self.w_router = tensors["router"].float().to(rt.device).contiguous()      # float32: the router's product runs on CUDA cores in 32-bit
        E, F, h = self.num_experts, self.expert_size, self.hidden_size
        self.grouped = (rt.dtype == torch.bfloat16 and self.w_up.dtype == torch.bfloat16 and 2 * self.top <= E and h % 8 == 0 and F % 8 == 0
                        and hasattr(torch, "_grouped_mm") and rt.device.type == "cuda")
        if self.grouped:       # views of the stacked matrices, one [K, N] operand per expert; nothing is copied
            self.b_up = self.w_up.view(E, F, h).transpose(1, 2)
            self.b_down = torch.as_strided(self.w_down, (E, F, h), (F, 1, E * F))

    def kernel_sources(self):
        return {"moe", "gemm_simt"} | self.rt.product_sources(self.w_up, self.w_down)       # (gemm_simt: the router of a very wide model)

    def forward(self, x, ctx):
        if x.is_contiguous() and (self.hidden_size + self.num_experts) * 4 <= 200 * 1024:
            ids, wts = ops.moe_router(x, self.w_router, self.top)          # logits, top-k and weights in one kernel
        else:
            ids, wts = ops.moe_route(self.rt.linear(x, self.w_router, None, out_dtype=torch.float32), self.top)
        T = x.shape[0]
        if (T * self.top <= self.num_experts and x.is_contiguous() and (x.dtype == self.w_up.dtype or self.w_up.dtype == torch.float32)
                and ops.moe_pairs_fit(self.hidden_size, self.expert_size, self.top)):
            out = torch.empty(T, self.hidden_size, dtype=torch.float32, device=x.device)
            return ops.moe_pairs(x, self.w_up, self.w_down, ids, wts, out, self.num_experts, self.activation)
        # up to the token count that the framework's own streaming product serves, the wide form reads every expert once at
        # that kernel's rate, which the grouped product does not reach on so few rows
        if self.grouped and x.dtype == torch.bfloat16 and x.is_contiguous() and T > GROUPED_MIN_TOKENS:
            ends, place, row_weight = ops.moe_sort(ids, wts, self.num_experts)
            rows = ops.moe_gather(x, place, self.top)
            hid = ops.moe_act_rows(ops.grouped_linear(rows, self.b_up, ends), row_weight, self.activation)
            down = ops.grouped_linear(hid, self.b_down, ends)
            return ops.moe_combine(down, place, self.top, torch.empty(T, self.hidden_size, dtype=torch.float32, device=x.device))
        up = self.rt.linear(x, self.w_up)
        act = ops.moe_dense_act(up, ids, wts, torch.empty_like(up), self.num_experts, self.activation)
        return self.rt.linear(act, self.w_down, None, out_dtype=torch.float32)


register_part("feed_forward", "routed_experts", RoutedExperts)
