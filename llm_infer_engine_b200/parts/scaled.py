"""Two small parts for designs that scale what a branch returns.

`layer_scale` (pointwise): a learned number per channel. A block that has one on a branch hands the vector to the
kernel that adds the branch to the stream (`ScaledDelta`); as a pointwise part of its own it multiplies rows in place.

`mixer_sum` (mixer): several mixers side by side that read the same input; the result is the sum of their outputs,
each times a constant. Every member keeps its own cache and state: the requests of member `name` are prefixed with
`name.` and the member gets `unit.scoped(name)`. With two members the outputs travel on as a `ScaledDelta` and are
added by the next norm's kernel; with more, they are summed here.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List

import torch

from ..kernels import ops
from .base import Mixer, ParamSpec, Pointwise, ScaledDelta, build_part, register_mixer, register_pointwise


class LayerScale(Pointwise):
    """params: size; weight_name (default "" = the part's own checkpoint name)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.size = int(params["size"])
        self.weight_name = str(params.get("weight_name", ""))
        self.vector = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.size,), role="vector", init=("uniform", 0.5, 1.5))}

    def load(self, tensors):
        self.vector = tensors[self.weight_name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * 4

    def forward(self, x, ctx, rows=None):
        return ScaledDelta([(x, 1.0)], self.vector).materialize()


register_pointwise("layer_scale", LayerScale)


class MixerSum(Mixer):
    """params: members (a mapping name -> PartSpec of a mixer, in the order they run), scales (name -> constant,
    default 1). The members' tensors live under `<name>.` of this part's checkpoint name."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        members = params["members"]
        if not members:
            raise ValueError("mixer_sum needs at least one member")
        scales = params.get("scales") or {}
        self.members = {name: build_part("mixer", spec, runtime) for name, spec in members.items()}
        self.scales = {name: float(scales.get(name, 1.0)) for name in members}

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {f"{name}.{local}": ps for name, m in self.members.items() for local, ps in m.param_specs().items()}

    def load(self, tensors):
        for name, m in self.members.items():
            cut = len(name) + 1
            m.load({k[cut:]: v for k, v in tensors.items() if k.startswith(name + ".")})

    def weight_bytes(self) -> int:
        return sum(m.weight_bytes() for m in self.members.values())

    def cache_requests(self) -> List[object]:
        return [dataclasses.replace(r, name=f"{name}.{r.name}") for name, m in self.members.items()
                for r in m.cache_requests()]

    def forward(self, x, ctx, unit, owns_cache):
        outs = [(m.forward(x, ctx, unit.scoped(name), owns_cache), self.scales[name]) for name, m in self.members.items()]
        if len(outs) <= 2:
            return ScaledDelta(outs)
        total = torch.zeros(outs[0][0].shape, dtype=torch.float32, device=outs[0][0].device)
        for i in range(0, len(outs), 2):
            (t1, c1), (t2, c2) = outs[i], (outs[i + 1] if i + 1 < len(outs) else (None, 0.0))
            ops.scaled_add_rmsnorm(total, t1, c1, t2, c2, None, None, 0.0, None)
        return total


register_mixer("mixer_sum", MixerSum)
