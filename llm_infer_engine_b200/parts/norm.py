"""RMSNorm fused with the residual add that precedes it.

y = x * rsqrt(mean(x^2) + eps) * w, all in float32, one rounding at the store
(src/rms_norm.py:32-39 of the reference). The weight is used as it is (not 1 + w), unless `weight_offset` says that
the checkpoint stores the weight's distance from a constant (1 + w for an offset of 1).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops, trace
from .base import DeferredNorm, Norm, ParamSpec, ScaledDelta, register_norm, single_delta


class RMSNorm(Norm):
    """params: size (width of a row), eps; weight_name (the tensor's name under the part's checkpoint name,
    default "weight"; "" = the part's name itself); weight_offset (default 0: the norm multiplies by
    weight_offset + the stored tensor, for checkpoints that store the weight around zero); residual_scale (default 1:
    the constant alpha of `norm_sum`, the form for blocks whose norm comes AFTER the residual sum)."""

    kind = "rmsnorm"

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight_offset = float(params.get("weight_offset", 0.0))
        self.residual_scale = float(params.get("residual_scale", 1.0))
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        init = ("ones",) if not self.weight_offset else ("uniform", -0.2, 0.2)
        return {self.weight_name: ParamSpec((self.size,), role="vector", init=tuple(self.params.get("init", init)))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].to(torch.float32).contiguous()   # bf16 -> f32 is exact
        if self.weight_offset:
            self.weight = (self.weight + self.weight_offset).contiguous()        # the sum in float32

    def weight_bytes(self) -> int:
        return self.size * 4

    def defer(self, h):
        """One-token steps of the bfloat16 engine: the next product's kernel applies this norm itself."""
        if self.runtime.dtype != torch.bfloat16 or not ops.norm_gemm_supported(h.shape[0], self.size):
            return None
        return DeferredNorm(self, h, "rmsnorm", self.weight, self.eps)

    def forward(self, h, delta, out=None, rows=None):
        n_out = h.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = torch.empty((n_out, self.size), dtype=self.runtime.dtype, device=h.device)
        trace.push("RMSNorm")
        if isinstance(delta, ScaledDelta):
            # a scaled branch output (or two): the add, the scales and the norm are one kernel
            (t1, c1), (t2, c2) = delta.terms[0], (delta.terms[1] if len(delta.terms) > 1 else (None, 0.0))
            ops.scaled_add_rmsnorm(h, t1, c1, t2, c2, delta.vector, self.weight, self.eps, out, rows)
            trace.pop()
            return out
        delta = single_delta(delta)
        if delta is not None and delta.dtype != out.dtype:
            # the fused kernel adds a branch output of the activations' type; any other is added by a kernel of its own
            if rows is not None:
                h = h.clone()
            ops.residual_add(h, delta)
            delta = None
        ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)
        trace.pop()
        return out


    def add_normed(self, h, y, bias=None, act=None):
        trace.push("RMSNorm")
        ops.branch_norm_add(h, y, bias, self.weight, self.eps, act)
        trace.pop()
        return h

    def norm_sum(self, h, y, vector=None, act=None):
        trace.push("RMSNorm")
        ops.scaled_sum_norm(h, y, vector, self.residual_scale, self.weight, self.eps, act)
        trace.pop()
        return h


register_norm("rmsnorm", RMSNorm)


class DynamicTanh(Norm):
    """y = tanh(alpha * x) * w + b, element by element: a norm that computes no mean and no variance, so nothing is
    reduced over a row. alpha is a learned scalar, w and b learned vectors; float32 arithmetic, one rounding at the
    store. The kernel adds up to two branch outputs to the stream on the way (`delta` may be a tuple).

    params: size; weight_name (default "weight"; "" = the part's own name), alpha_name (default "alpha"), bias_name
    (default "b"): the tensors' names under the part's checkpoint name."""

    kind = "dynamic_tanh"

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.size = int(params["size"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.alpha_name = str(params.get("alpha_name", "alpha"))
        self.bias_name = str(params.get("bias_name", "b"))
        self.weight = self.alpha = self.bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), role="vector", init=tuple(self.params.get("init", ("ones",)))),
                self.alpha_name: ParamSpec((), role="vector", init=("uniform", 0.3, 0.9)),
                self.bias_name: ParamSpec((self.size,), role="vector", init=("uniform", -0.1, 0.1))}

    def load(self, tensors):
        self.weight = tensors[self.weight_name].to(torch.float32).contiguous()
        self.alpha = tensors[self.alpha_name].to(torch.float32).reshape(1).contiguous()
        self.bias = tensors[self.bias_name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * 8 + 4

    def forward(self, h, delta, out=None, rows=None):
        n_out = h.shape[0] if rows is None else rows.shape[0]
        if out is None:
            out = torch.empty((n_out, self.size), dtype=self.runtime.dtype, device=h.device)
        d = [x for x in (delta if isinstance(delta, (tuple, list)) else (delta,)) if x is not None]
        if len(d) > 2:
            raise ValueError("DynamicTanh adds at most two branch outputs")
        trace.push("DyT")
        ops.add_dyt(h, d[0] if d else None, d[1] if len(d) > 1 else None, self.alpha, self.weight, self.bias, out, rows)
        trace.pop()
        return out


register_norm("dynamic_tanh", DynamicTanh)
