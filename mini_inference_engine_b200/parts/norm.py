"""RMSNorm fused with the residual sum: ``res += delta; x = res * rsqrt(mean(res^2) + eps) * w``
(inference_engine/kernels/rmsnorm.py:13-32,56-65, where the residual stays in the model dtype;
here the residual stream is float32 in both modes)."""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import Part, StreamUpdated, StreamValue, register_part


class RMSNorm(Part):
    def __init__(self, size: int, eps: float):
        self.size = size
        self.eps = eps

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), init="ones")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = rt.place(tensors["weight"])

    def kernel_sources(self):
        return {"norm"}

    def deferred_args(self):
        """Weight and eps, for a product that folds this norm into its neighbours' epilogues."""
        return self.weight, self.eps

    def __call__(self, delta, res, rows=None):
        if isinstance(delta, StreamValue):               # the block before left the stream complete
            delta = None
        if isinstance(delta, StreamUpdated):             # the part before added its output to the stream itself
            if delta.norm is self and delta.deferred is not None and rows is None:
                return delta.deferred                    # and left this norm's output, short of a factor, for the next product
            delta = None
        n_out = rows.numel() if rows is not None else res.shape[0]
        out = self.rt.empty(n_out, self.size)
        return ops.add_rmsnorm(delta, res, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)


class GroupRMSNorm(Part):
    """RMS norm with statistics per group: a row is cut into ``groups`` equal consecutive parts, each divided by
    sqrt(mean(part^2) + eps), and the whole multiplied by the weight.  It norms the stream itself (post-norm
    models): ``apply`` replaces the stream by norm(alpha * stream + coef * sum of branches), where a branch may first
    be RMS-normed over its whole row with a weight of its own (``inner_weights``), and returns the new stream in the
    activation type.  Called like the other norms (``norm(delta, res, rows)``) it adds nothing and norms a copy: the
    norm in front of the output head."""

    def __init__(self, size: int, eps: float, groups: int = 1):
        if groups < 1 or size % groups:
            raise ValueError(f"{groups} groups do not divide a width of {size}")
        self.size, self.eps, self.groups = size, eps, groups

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), init="ones")}

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = tensors["weight"].float().to(rt.device).contiguous()      # read as float32 by the kernel (16-byte loads)

    def kernel_sources(self):
        return {"norm_group"}

    def apply(self, res, deltas=(), inner_weights=(), alpha: float = 1.0, coef: float = 1.0):
        """res <- norm(alpha * res + coef * sum(branches)) in place; returns it in the activation type (``res`` itself
        where that is float32)."""
        import torch
        out = None if self.rt.dtype == torch.float32 else self.rt.empty(res.shape[0], self.size)
        ops.stream_norm(res, self.weight, self.groups, self.eps, out, alpha=alpha, deltas=deltas,
                        inner_weights=inner_weights, coef=coef)
        return res if out is None else out

    def __call__(self, delta, res, rows=None):
        if isinstance(delta, (StreamValue, StreamUpdated)):
            delta = None
        if delta is not None:
            raise ValueError("a group norm of the stream takes its branches through apply()")
        if rows is None:
            return self.apply(res)
        out = self.rt.empty(rows.numel(), self.size)
        return ops.stream_norm(res, self.weight, self.groups, self.eps, out, rows=rows)


register_part("norm", "group_rmsnorm", GroupRMSNorm)
