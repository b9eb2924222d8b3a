"""What some designs do to the embedded tokens before the first layer: a scale on the token embedding, a learned
vector per absolute position added to it, and a norm over the sum. Each of the three is optional.

    x_t = scale * E[token_t] + P[pos_t];    h_t = x_t / sqrt(mean(x_t^2) + eps) * w

all in float32, one kernel. Positions count from 0 in each sequence."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from .base import ParamSpec, Pointwise, register_pointwise


class EmbeddingStage(Pointwise):
    """params: size (row width), scale (default 1), positions (rows of the position table, None = no table),
    norm_eps (None = no norm), names (checkpoint names of `positions` and `norm`)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.size = int(params["size"])
        self.scale = float(params.get("scale", 1.0))
        self.positions = params.get("positions")
        self.norm_eps = params.get("norm_eps")
        self.names = dict({"positions": "positions", "norm": "norm"}, **(params.get("names") or {}))
        self.table = self.weight = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {}
        if self.positions is not None:
            specs[self.names["positions"]] = ParamSpec((int(self.positions), self.size))
        if self.norm_eps is not None:
            specs[self.names["norm"]] = ParamSpec((self.size,), role="vector", init=("ones",))
        return specs

    def load(self, tensors):
        if self.positions is not None:
            self.table = tensors[self.names["positions"]].contiguous()
        if self.norm_eps is not None:
            self.weight = tensors[self.names["norm"]].to(torch.float32).contiguous()

    def forward(self, x, ctx, rows=None):
        if rows is not None:
            raise ValueError("the embedding stage belongs after the embedding, not after the head")
        act = None
        if self.runtime.dtype != torch.float32:
            act = torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device)
        ops.scale_pos_norm(x, self.scale, self.table, ctx.tok_pos, self.weight, float(self.norm_eps or 0.0), act)
        if act is not None:
            ctx.carry["h_act"] = act          # the stream as a bfloat16 product reads it
        return x


register_pointwise("embedding_stage", EmbeddingStage)


class Scale(Pointwise):
    """x *= factor: the logits of designs that scale them (or the embedded tokens). params: factor."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.factor = float(params["factor"])

    def forward(self, x, ctx, rows=None):
        if self.factor != 1.0:
            ops.scale_rows(x, self.factor)
        return x


register_pointwise("scale", Scale)


class SoftCap(Pointwise):
    """x = cap * tanh(x / cap): logits of designs that cap them (float32). params: cap (> 0)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.cap = float(params["cap"])
        if not self.cap > 0:
            raise ValueError(f"cap must be positive, got {self.cap}")

    def forward(self, x, ctx, rows=None):
        return ops.cap_rows(x, self.cap)


register_pointwise("softcap", SoftCap)
