"""A routed feed-forward (mixture of experts) with an optional shared expert.

With u [T, d] the branch input, E experts of width f, each down_e(act(gate_e u) * (up_e u)) without biases:

    z      = W_r u + b_r                       float32, whatever the engine's precision
    S_t    = the `top` experts with the largest z_t (ties: the lower index)
    a_t,e  = exp(z_t,e) / sum over e' in S_t of exp(z_t,e')        softmax over the chosen logits alone
    y_t    = sum over e in S_t of a_t,e * expert_e(u_t)  (+ shared(u_t), an expert every token uses)

The (token, choice) pairs are sorted by expert on the device into tiles (no host round trip: array sizes are upper
bounds, so a captured step replays it), the experts' two products run as ONE routed launch each over stacked weights
[E, 2 f, d] and [E, d, f] (gate and up fused with the activation), and the pairs are combined per token in the order
of the choices, in float32. A token's result does not depend on what else is in the batch.

Options: `gated` False makes an expert down_e(act(up_e u)), one product in front of the activation. `scoring`
"softmax_all" is a second rule for the router: s = softmax(z) over ALL its outputs, the `top` largest of s + c are chosen
(c a stored correction that steers the choice only), and a_t,e = s_t,e / (sum of the chosen s + 1e-20) * `weight_scale`.
"sigmoid" is a third: s = sigmoid(z) one by one, the `top` largest choose and weigh as they are (times `weight_scale`),
not normalised. `weight_on` "input" (default "output"): the weight multiplies what the expert READS, y_t = sum over e of
expert_e(a_t,e u_t), which is not the same thing under a non-linear expert; the rows are scaled while they are gathered
into the order of their experts, and the combine adds with weight one.
`identity_experts` n: the router has n more outputs than there are experts; the last n stand for experts that return
their input (their share is weight * u_t), and they hold no tensors. Prompts of a bfloat16 engine
hand the two products to the vendor library's grouped GEMM instead (as the dense layers hand theirs to its plain one):
the tokens are gathered into the order of their experts first, the offsets stay on the device.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops, trace
from .base import FeedForward, ParamSpec, build_part, register_feed_forward
from ..config.spec import PartSpec


class RoutedExperts(FeedForward):
    """params: hidden, n_experts, top, expert_ff, activation (default "silu"), router_bias (bool, default True),
    shared_ff (width of the shared expert, None = none), shared_activation (default: `activation`), gated (default
    True), scoring ("softmax_top", the default, "softmax_all" or "sigmoid"), weight_scale (default 1), weight_on
    ("output", the default, or "input"), identity_experts (default 0), names (checkpoint sub-names: router, router_bias, correction, expert (a pattern with {e}), gate, up, down,
    shared)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.n_experts, self.top = int(p["hidden"]), int(p["n_experts"]), int(p["top"])
        self.expert_ff = int(p["expert_ff"])
        if self.top <= 0 or self.n_experts <= 0:
            raise ValueError(f"top ({self.top}) and n_experts ({self.n_experts}) must be positive")
        name = str(p.get("activation", "silu"))
        if name not in ops.ACTIVATIONS or name == "none":
            raise ValueError(f"activation {name!r} is not known ({sorted(ops.ACTIVATIONS)})")
        self.activation = ops.ACTIVATIONS[name]
        self.router_bias = bool(p.get("router_bias", True))
        self.gated = bool(p.get("gated", True))
        self.scoring = str(p.get("scoring", "softmax_top"))
        if self.scoring not in ("softmax_top", "softmax_all", "sigmoid"):
            raise ValueError(f"scoring must be 'softmax_top', 'softmax_all' or 'sigmoid', got {self.scoring!r}")
        self.route_mode = {"softmax_top": ops.ROUTE_SOFTMAX_TOP, "softmax_all": ops.ROUTE_SOFTMAX_ALL,
                           "sigmoid": ops.ROUTE_SIGMOID}[self.scoring]
        self.weight_on_input = str(p.get("weight_on", "output")) == "input"
        if p.get("weight_on", "output") not in ("output", "input"):
            raise ValueError(f"weight_on must be 'output' or 'input', got {p.get('weight_on')!r}")
        if self.weight_on_input and int(p.get("identity_experts") or 0):
            raise ValueError("weights on the experts' input do not go with experts that return their input")
        self.weight_scale = float(p.get("weight_scale", 1.0))
        self.n_identity = int(p.get("identity_experts") or 0)
        self.n_outputs = self.n_experts + self.n_identity          # what the router has outputs for
        if self.top > self.n_outputs or self.n_identity < 0:
            raise ValueError(f"top ({self.top}) must not exceed the router's {self.n_outputs} outputs")
        self.names = dict({"router": "router", "router_bias": "router.b", "correction": "correction", "expert": "e{e}",
                           "gate": "gate", "up": "up", "down": "down", "shared": "shared"}, **(p.get("names") or {}))
        self.shared = None
        if p.get("shared_ff"):
            n = self.names
            self.shared = build_part("feed_forward", PartSpec("swiglu", {
                "hidden": self.hidden, "intermediate": int(p["shared_ff"]),
                "activation": str(p.get("shared_activation", name)), "out_float32": True,
                "names": {"gate": n["gate"], "up": n["up"], "down": n["down"]}}), runtime)
        self.w_router = self.b_router = self.correction = self.w_gate_up = self.w_down = None
        self._library = True          # prompts may use the vendor's grouped GEMM until it refuses a shape

    def _expert_name(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e=e)}.{self.names[which]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, f = self.names, self.hidden, self.expert_ff
        specs = {n["router"]: ParamSpec((self.n_outputs, d))}
        if self.router_bias:
            specs[n["router_bias"]] = ParamSpec((self.n_outputs,), role="vector", init=("normal",))
        if self.scoring == "softmax_all":
            specs[n["correction"]] = ParamSpec((self.n_outputs,), role="vector", init=("uniform", -0.05, 0.05))
        for e in range(self.n_experts):
            if self.gated:
                specs[self._expert_name(e, "gate")] = ParamSpec((f, d))
            specs[self._expert_name(e, "up")] = ParamSpec((f, d))
            specs[self._expert_name(e, "down")] = ParamSpec((d, f))
        if self.shared is not None:
            for local, ps in self.shared.param_specs().items():
                specs[f"{n['shared']}.{local}"] = ps
        return specs

    def load(self, tensors):
        n = self.names
        self.w_router = tensors[n["router"]].to(torch.float32).contiguous()
        self.b_router = tensors[n["router_bias"]].to(torch.float32).contiguous() if self.router_bias else None
        if self.scoring == "softmax_all":
            self.correction = tensors[n["correction"]].to(torch.float32).contiguous()
        gu, dn = [], []
        for e in range(self.n_experts):
            up = tensors[self._expert_name(e, "up")]
            gu.append(torch.cat([tensors[self._expert_name(e, "gate")], up], dim=0) if self.gated else up)
            dn.append(tensors[self._expert_name(e, "down")])
        dtype = torch.float32 if any(t.dtype == torch.float32 for t in gu + dn) else gu[0].dtype
        self.w_gate_up = torch.stack([t.to(dtype) for t in gu]).contiguous()       # [E, 2 f, d] ([E, f, d] ungated)
        self.w_down = torch.stack([t.to(dtype) for t in dn]).contiguous()          # [E, d, f]
        if self.shared is not None:
            cut = len(n["shared"]) + 1
            self.shared.load({k[cut:]: v for k, v in tensors.items() if k.startswith(n["shared"] + ".")})

    def weight_bytes(self) -> int:
        """What a one-token step of one sequence reads: the router, `top` experts and the shared expert."""
        per_expert = (3 if self.gated else 2) * self.expert_ff * self.hidden * self.w_down.element_size()
        return self.w_router.numel() * 4 + self.top * per_expert + (self.shared.weight_bytes() if self.shared else 0)

    def forward(self, x, ctx, residual=None):
        trace.push("FFN")
        try:
            T, dev = x.shape[0], x.device
            top, E = self.top, self.n_experts
            w = self.w_gate_up
            xin = x if x.dtype == w.dtype else x.to(w.dtype)
            ids = torch.empty((T, top), dtype=torch.int32, device=dev)
            weights = torch.empty((T, top), dtype=torch.float32, device=dev)
            ops.moe_route(x, self.w_router, self.b_router, ids, weights, self.route_mode, self.correction,
                          self.weight_scale)
            n_pairs = T * top
            small = n_pairs <= ops.GROUPED_SMALL_ROWS
            tile = ops.grouped_tile_rows(small)
            n_tiles = ops.moe_max_tiles(n_pairs, E, tile)
            index = torch.empty(2 * n_tiles * tile + n_tiles, dtype=torch.int32, device=dev)
            sorted_token, sorted_pair = index[:n_tiles * tile], index[n_tiles * tile:2 * n_tiles * tile]
            tile_group = index[2 * n_tiles * tile:]
            shared = None
            if self._library and ops.library_grouped_mm_ok(n_pairs, w, self.w_down):
                # prompts: each expert's rows side by side, the two products by the library's grouped GEMM
                extra = torch.empty(E + n_pairs, dtype=torch.int32, device=dev)
                group_end, pair_pos = extra[:E], extra[E:]
                ops.moe_sort(ids, E, tile, sorted_token, sorted_pair, tile_group, group_end, pair_pos)
                xs = torch.empty((n_tiles * tile, self.hidden), dtype=w.dtype, device=dev)
                if self.weight_on_input:
                    ops.moe_gather_scaled(x, sorted_token, sorted_pair, weights, xs)
                else:
                    ops.moe_gather_rows(xin, sorted_token, xs)
                try:
                    gu = ops.library_grouped_mm(xs, w, group_end)
                except RuntimeError as exc:
                    # the library refuses these sizes (it checks before it launches): this library's own routed
                    # products take them, from now on without asking again
                    if "CUDA error" in str(exc):
                        raise
                    self._library = False
                    gu = None
                if gu is not None:
                    act = torch.empty((n_tiles * tile, self.expert_ff), dtype=w.dtype, device=dev)
                    if self.gated:
                        ops.gated_act(gu, act, self.activation)
                    else:
                        ops.bias_act(gu, None, act, self.activation)
                    y = ops.library_grouped_mm(act, self.w_down, group_end)
                    return self._combine(y, weights, ids, x, ctx, pair_pos)
            ops.moe_sort(ids, E, tile, sorted_token, sorted_pair, tile_group)
            # gate and up of every pair's expert with the activation; rows stay in sorted order
            act = torch.empty((n_tiles * tile, self.expert_ff), dtype=w.dtype, device=dev)
            if self.weight_on_input:
                # every pair's row times its weight, already in sorted order (padding rows are zeros)
                xs = ops.moe_gather_scaled(x, sorted_token, sorted_pair, weights,
                                           torch.empty((n_tiles * tile, self.hidden), dtype=w.dtype, device=dev))
                ops.routed_gemm_nt(xs, None, w, act, None, tile_group, n_tiles * tile, small, dual=self.gated,
                                   act=self.activation)
            else:
                ops.routed_gemm_nt(xin, sorted_token, w, act, None, tile_group, n_tiles * tile, small, dual=self.gated,
                                   act=self.activation)
            # down: back to the order of the pairs, float32
            y = torch.empty((n_pairs, self.hidden), dtype=torch.float32, device=dev)
            ops.routed_gemm_nt(act, None, self.w_down, y, sorted_pair, tile_group, n_tiles * tile, small)
            return self._combine(y, weights, ids, x, ctx, None)
        finally:
            trace.pop()

    def _combine(self, y, weights, ids, x, ctx, pair_pos):
        """The weighted sum of the chosen experts' outputs per token (float32), with the shared expert's output and
        the share of the experts that return their input."""
        out = torch.empty((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        if not self.n_identity:
            return ops.moe_combine(y, self.top if self.weight_on_input else weights, shared, out, pair_pos)
        ops.moe_combine_identity(y, weights, ids, self.n_experts, x, out, pair_pos)
        if shared is not None:
            ops.residual_add(out, shared)
        return out


register_feed_forward("routed_experts", RoutedExperts)
