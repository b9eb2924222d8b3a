"""Dense gated feed-forward: down(silu(gate x) * (up x)), no bias (src/model.py:14-25 of the
reference, w1 = gate, w3 = up, w2 = down). gate and up are one GEMM over row-concatenated
weights; the activation and product are one kernel."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops, trace
from .base import DeferredBranchAdd, DeferredNorm, FeedForward, ParamSpec, register_feed_forward
from .linear import Linear


class SwiGLU(FeedForward):
    """params: hidden, intermediate; activation (on the gate: "silu", the default, or any of ops.ACTIVATIONS, e.g.
    "gelu_tanh"); names (checkpoint sub-names of gate, up, down); out_float32 (the branch output is float32 instead
    of the activations' type: for designs that round nothing between the last product and the residual sum)."""

    adds_to_residual = True
    accepts_deferred_norm = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        name = str(params.get("activation", "silu"))
        if name not in ops.ACTIVATIONS or name == "none":
            raise ValueError(f"activation {name!r} is not known ({sorted(ops.ACTIVATIONS)})")
        self.activation = ops.ACTIVATIONS[name]
        self.names = dict({"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"},
                          **(params.get("names") or {}))
        self.out_float32 = bool(params.get("out_float32", False))
        self.gate_up: Linear = None
        self.down: Linear = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {n["gate"]: ParamSpec((self.intermediate, self.hidden)),
                n["up"]: ParamSpec((self.intermediate, self.hidden)),
                n["down"]: ParamSpec((self.hidden, self.intermediate))}

    def load(self, tensors):
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        dtype = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.gate_up = Linear(torch.cat([g.to(dtype), u.to(dtype)], dim=0))
        self.down = Linear(tensors[self.names["down"]])

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    def forward(self, x, ctx, residual=None):
        trace.push("FFN")
        try:
            return self._forward(x, ctx, residual)
        finally:
            trace.pop()

    def _forward(self, x, ctx, residual):
        act = None
        if isinstance(x, DeferredNorm):
            w = self.gate_up.weight
            if x.kind == "rmsnorm" and w.dtype == torch.bfloat16 and self.intermediate % 8 == 0 \
                    and self.activation == ops.ACT_SILU:
                # one-token steps: norm, product, activation and gate in one kernel
                act = torch.empty((x.shape[0], self.intermediate), dtype=torch.bfloat16, device=w.device)
                ops.norm_gate_swiglu(x.h, x.weight, x.eps, w, act)
            else:
                x = x.apply()
        if act is None:                              # product, activation and gate in one kernel
            act = self.gate_up.swiglu(x) if self.activation == ops.ACT_SILU else self.gate_up.gated(x, self.activation)
        if act is None:
            gu = self.gate_up(x)
            act = torch.empty((x.shape[0], self.intermediate), dtype=gu.dtype, device=x.device)
            if self.activation == ops.ACT_SILU:
                ops.swiglu(gu, act)
            else:
                ops.gated_act(gu, act, self.activation)
        if residual is not None and self.down.add_into(act, residual):
            return None
        return self.down(act, out_dtype=torch.float32) if self.out_float32 else self.down(act)


register_feed_forward("swiglu", SwiGLU)


class DenseMLP(FeedForward):
    """down(act(up x + b_up)) + b_down: one up projection, a pointwise activation, one down projection.

    params: hidden, intermediate, activation ("relu2" = the square of relu, "relu", "gelu_tanh", "silu", or
    "poly_norm"), bias (bool), names (overrides of the checkpoint sub-names: up, up_bias, down, down_bias,
    poly_norm). The result is float32. A block that adds the output bias inside its own next kernel calls
    `forward(..., defer_bias=True)` and reads `down_bias` itself.

    "poly_norm" is not pointwise: a N(z) + b N(z^2) + c N(z^3) + e over a token's whole vector z of up-projections,
    N(t) = t / sqrt(mean(t^2) + eps) with `norm_eps` (a param), powers element by element, and a, b, c, e four learned
    numbers stored as one tensor; float32 arithmetic."""

    accepts_deferred_branch_add = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        name = str(params.get("activation", "relu2"))
        self.poly_norm = name == "poly_norm"
        if not self.poly_norm and name not in ops.ACTIVATIONS:
            raise ValueError(f"activation {name!r} is not known ({sorted(ops.ACTIVATIONS) + ['poly_norm']})")
        self.activation = ops.ACT_NONE if self.poly_norm else ops.ACTIVATIONS[name]
        self.norm_eps = float(params["norm_eps"]) if self.poly_norm else 0.0
        self.poly_coef = None
        self.bias = bool(params.get("bias", True))
        self.names = dict({"up": "up", "up_bias": "up.b", "down": "down", "down_bias": "down.b", "poly_norm": "act"},
                          **(params.get("names") or {}))
        self.up: Linear = None
        self.down: Linear = None
        self.up_bias = self.down_bias = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        specs = {n["up"]: ParamSpec((self.intermediate, self.hidden)),
                 n["down"]: ParamSpec((self.hidden, self.intermediate))}
        if self.bias:
            specs[n["up_bias"]] = ParamSpec((self.intermediate,), role="vector", init=("normal",))
            specs[n["down_bias"]] = ParamSpec((self.hidden,), role="vector", init=("normal",))
        if self.poly_norm:
            specs[n["poly_norm"]] = ParamSpec((4,), role="vector", init=("uniform", -1.0, 1.0))
        return specs

    def load(self, tensors):
        n = self.names
        self.up, self.down = Linear(tensors[n["up"]]), Linear(tensors[n["down"]])
        if self.bias:
            self.up_bias = tensors[n["up_bias"]].to(torch.float32).contiguous()
            self.down_bias = tensors[n["down_bias"]].to(torch.float32).contiguous()
        if self.poly_norm:
            self.poly_coef = tensors[n["poly_norm"]].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.up.nbytes() + self.down.nbytes() + (4 * (self.intermediate + self.hidden) if self.bias else 0)

    def forward(self, x, ctx, residual=None, defer_bias: bool = False):
        trace.push("FFN")
        try:
            a = None
            if isinstance(x, DeferredBranchAdd):
                if x.foldable(self.up.weight):
                    # one-token steps: the add that closes the mixer's branch, the product, bias and activation
                    a = self.up.after_branch_add(x, self.up_bias, self.activation)
                else:
                    from .gated_attention import _rounded
                    x = _rounded(x, self.runtime)
            if a is None:
                a = self.up.bias_act(x, self.up_bias, self.activation)  # product, bias and activation in one kernel
            if a is None:
                u = self.up(x)
                a = torch.empty_like(u)
                ops.bias_act(u, self.up_bias, a, self.activation)
            if self.poly_norm:
                a = ops.poly_norm(a, self.poly_coef, self.norm_eps, torch.empty_like(a))
            y = self.down(a, out_dtype=torch.float32)
            if self.down_bias is not None and not defer_bias:
                ops.bias_act(y, self.down_bias, y, ops.ACT_NONE)
            return y
        finally:
            trace.pop()


register_feed_forward("dense_mlp", DenseMLP)
