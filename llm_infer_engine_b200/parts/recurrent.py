"""Mixers that carry a fixed-size state from token to token (no cache of keys): what a sequence leaves behind is the
state alone, kept per (layer, slot) in float32 by the cache's state area and zeroed when a slot is taken.

`gated_linear_recurrence` — linear attention whose forget gate also decides what is written. With u [T, d] the input,
H heads, D gate/query channels and Dv value channels a head:

    q = silu(u Wq^T)                      f = l + (1 - l) sigmoid(u Wf^T + b)        v = u Wv^T
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T        per head, S [D, Dv] from zero; there is no key: 1 - f is it
    o_t = S_t^T q_t                                  read from the NEW state
    y   = concat_h(o_t,h / sqrt(mean(o_t,h^2) + eps) * w) Wo^T       w [Dv] shared by the heads

`l` is a learned lower bound of the gate per channel (stored as it is used, in [0, 1)).

`gated_recurrent_unit` — a real-gated linear recurrent unit behind a short causal convolution, with a second branch as
output gate. With C channels in `blocks` equal groups and K taps:

    y = act(u Wy^T + by)                  x = u Wx^T + bx
    c_t = bc + sum_j taps[:, K-1-j] x_(t-j)                          per channel, zeros before the sequence
    r = sigmoid(Ra c + bra), i = sigmoid(Ri c + bri)                 Ra, Ri block-diagonal: a square matrix per group
    a = exp(-decay * r * softplus(lam))
    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) (i_t c_t)                    S [C] from zero, the first token like any other
    out = (S (.) y) Wo^T

`decayed_linear_attention` — linear attention with a constant decay per head ("lightning" attention). With H heads,
D query/key channels and Dv value channels a head, and an activation act on all three projections:

    q = act(u Wq^T), k = act(u Wk^T), v = act(u Wv^T)
    S_t = a_h S_(t-1) + k_t v_t^T                    per head, S [D, Dv] from zero; a_h a constant of the model
    o_t = S_t^T q_t                                  read from the NEW state, no other scale
    y   = (concat_h(o_t) / sqrt(mean(concat_h(o_t)^2) + eps) * w) (.) sigmoid(u Wg^T) Wo^T     ONE norm over all heads

The state is S and the last K-1 inputs x of the convolution. Gates, decays, their logarithms and exponentials, the
state and the norm of what is read are float32 in both engines; the projections have the activation type.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.cache import StateRequest
from ..kernels import ops, trace
from .base import Mixer, ParamSpec, register_mixer
from .linear import Linear


class GatedLinearRecurrence(Mixer):
    """params: hidden, n_heads, dim (gate/query channels a head), v_dim (value channels a head), norm_eps, names
    (overrides of the checkpoint sub-names q, f, f_bias, lower, v, norm, o)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.n_heads = int(p["hidden"]), int(p["n_heads"])
        self.dim, self.v_dim = int(p["dim"]), int(p["v_dim"])
        if self.dim > 512:
            raise ValueError(f"dim ({self.dim}) exceeds what the scan kernel takes (512)")
        self.eps = float(p["norm_eps"])
        self.names = dict({"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"},
                          **(p.get("names") or {}))
        self.nq, self.nv = self.n_heads * self.dim, self.n_heads * self.v_dim
        self.proj: Linear = None
        self.o: Linear = None
        self.f_bias = self.lower = self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d = self.names, self.hidden
        return {n["q"]: ParamSpec((self.nq, d)), n["f"]: ParamSpec((self.nq, d)), n["v"]: ParamSpec((self.nv, d)),
                n["f_bias"]: ParamSpec((self.nq,), role="vector", init=("uniform", -1.0, 3.0)),
                n["lower"]: ParamSpec((self.nq,), role="vector", init=("uniform", 0.0, 0.9)),
                n["norm"]: ParamSpec((self.v_dim,), role="vector", init=("ones",)),
                n["o"]: ParamSpec((d, self.nv))}

    def load(self, tensors):
        n = self.names
        ws = [tensors[n["q"]], tensors[n["f"]], tensors[n["v"]]]
        dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0))         # [q | f | v]
        self.o = Linear(tensors[n["o"]])
        self.f_bias = tensors[n["f_bias"]].to(torch.float32).contiguous()
        self.lower = tensors[n["lower"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes() + 4 * (2 * self.nq + self.v_dim)

    def cache_requests(self):
        return [StateRequest("S", (self.n_heads, self.dim, self.v_dim))]

    def forward(self, x, ctx, unit, owns_cache):
        T, dev = x.shape[0], x.device
        trace.push("QKV_proj")
        proj = self.proj(x)                                            # [T, q | f | v]
        trace.pop()
        trace.push("Recurrence")
        q = torch.empty((T, self.nq), dtype=torch.float32, device=dev)
        f = torch.empty((T, self.nq), dtype=torch.float32, device=dev)
        ops.matrix_gates(proj, 0, self.nq, self.f_bias, self.lower, q, f)
        read = torch.empty((T, self.nv), dtype=torch.float32, device=dev)
        ops.matrix_scan(q, f, proj[:, 2 * self.nq:], unit.state["S"], ctx.cu_q, ctx.seq_slot, read, ctx.n_seqs,
                        self.n_heads, self.dim, self.v_dim, write_state=owns_cache, max_len=ctx.max_q_len)
        normed = torch.empty((T, self.nv), dtype=proj.dtype, device=dev)
        ops.head_rmsnorm(read, self.norm_w, self.eps, normed, self.v_dim)
        trace.pop()
        trace.push("Output_proj")
        y = self.o(normed, out_dtype=torch.float32)
        trace.pop()
        return y


register_mixer("gated_linear_recurrence", GatedLinearRecurrence)


class GatedRecurrentUnit(Mixer):
    """params: hidden, width (channels C), blocks (groups of the gates' block-diagonal matrices), taps (K), decay (the
    constant in the exponent, 8 in the published unit), activation (of the output-gate branch, default "gelu_tanh"),
    names (overrides of the checkpoint sub-names y, y_bias, x, x_bias, conv, conv_bias, ra, ra_bias, ri, ri_bias, lam, o)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.width = int(p["hidden"]), int(p["width"])
        self.blocks, self.taps = int(p["blocks"]), int(p["taps"])
        if self.width % self.blocks:
            raise ValueError(f"width ({self.width}) must be a multiple of blocks ({self.blocks})")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"taps ({self.taps}) must be between 1 and 16")
        self.block_width = self.width // self.blocks
        self.decay = float(p.get("decay", 8.0))
        name = str(p.get("activation", "gelu_tanh"))
        if name not in ops.ACTIVATIONS:
            raise ValueError(f"activation {name!r} is not known ({sorted(ops.ACTIVATIONS)})")
        self.activation = ops.ACTIVATIONS[name]
        self.names = dict({"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
                           "ra": "ra", "ra_bias": "ra.b", "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"},
                          **(p.get("names") or {}))
        self.proj: Linear = None
        self.o: Linear = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, C, B, bw = self.names, self.hidden, self.width, self.blocks, self.block_width
        vec = dict(role="vector", init=("normal",))
        return {n["y"]: ParamSpec((C, d)), n["y_bias"]: ParamSpec((C,), **vec),
                n["x"]: ParamSpec((C, d)), n["x_bias"]: ParamSpec((C,), **vec),
                n["conv"]: ParamSpec((C, self.taps), role="vector", init=("uniform", -0.5, 0.5)),
                n["conv_bias"]: ParamSpec((C,), **vec),
                n["ra"]: ParamSpec((B, bw, bw)), n["ra_bias"]: ParamSpec((B, bw), **vec),
                n["ri"]: ParamSpec((B, bw, bw)), n["ri_bias"]: ParamSpec((B, bw), **vec),
                n["lam"]: ParamSpec((C,), role="vector", init=("uniform", -4.0, 0.0)),
                n["o"]: ParamSpec((d, C))}

    def load(self, tensors):
        n = self.names
        wy, wx = tensors[n["y"]], tensors[n["x"]]
        dtype = torch.float32 if torch.float32 in (wy.dtype, wx.dtype) else wy.dtype
        self.proj = Linear(torch.cat([wy.to(dtype), wx.to(dtype)], dim=0))      # [y | x]
        self.o = Linear(tensors[n["o"]])
        f32 = lambda t: t.to(torch.float32).contiguous()                        # noqa: E731
        self.y_bias, self.x_bias = f32(tensors[n["y_bias"]]), f32(tensors[n["x_bias"]])
        self.conv_w, self.conv_bias = f32(tensors[n["conv"]]), f32(tensors[n["conv_bias"]])
        # per group the rows of Ra and then of Ri: one batched product gives both gates' pre-activations
        self.gate_w = torch.cat([f32(tensors[n["ra"]]), f32(tensors[n["ri"]])], dim=1).contiguous()   # [B, 2 bw, bw]
        self.ra_bias, self.ri_bias = f32(tensors[n["ra_bias"]]).reshape(-1), f32(tensors[n["ri_bias"]]).reshape(-1)
        self.lam = f32(tensors[n["lam"]])

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes() + self.gate_w.numel() * 4 + 4 * self.width * (6 + self.taps)

    def cache_requests(self):
        return [StateRequest("S", (self.width,)), StateRequest("conv", (self.taps - 1, self.width))]

    def forward(self, x, ctx, unit, owns_cache):
        T, dev, C, bw = x.shape[0], x.device, self.width, self.block_width
        trace.push("QKV_proj")
        proj = self.proj(x)                                            # [T, y | x]
        trace.pop()
        trace.push("Recurrence")
        state, conv_state = unit.state["S"], unit.state["conv"]
        u = torch.empty((T, C), dtype=torch.float32, device=dev)
        ops.causal_conv(proj, C, self.x_bias, self.conv_w, self.conv_bias, conv_state, ctx.cu_q, ctx.tok_seq,
                        ctx.seq_slot, u)
        gates = torch.empty((T, 2 * C), dtype=torch.float32, device=dev)
        ops.batched_gemm_nt(u, self.gate_w, gates, bw, 2 * bw, bw)
        ops.unit_gate_values(gates, u, self.ra_bias, self.ri_bias, self.lam, self.decay, bw)
        out = torch.empty((T, C), dtype=proj.dtype, device=dev)
        ops.unit_scan(gates, proj, 0, C, self.y_bias, self.x_bias, self.activation, state, conv_state, ctx.cu_q,
                      ctx.seq_slot, out, ctx.n_seqs, bw, write_state=owns_cache, max_len=ctx.max_q_len)
        trace.pop()
        trace.push("Output_proj")
        y = self.o(out, out_dtype=torch.float32)
        trace.pop()
        return y


register_mixer("gated_recurrent_unit", GatedRecurrentUnit)


class DecayedLinearAttention(Mixer):
    """params: hidden, n_heads, dim (query/key channels a head), v_dim (value channels a head), decay (a list of n_heads
    constants), activation (of q, k and v; default "silu"), norm_eps, names (overrides of the checkpoint sub-names q, k,
    v, gate, norm, o)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.n_heads = int(p["hidden"]), int(p["n_heads"])
        self.dim, self.v_dim = int(p["dim"]), int(p["v_dim"])
        if self.dim > 512:
            raise ValueError(f"dim ({self.dim}) exceeds what the scan kernel takes (512)")
        decay = [float(a) for a in p["decay"]]
        if len(decay) != self.n_heads:
            raise ValueError(f"decay holds {len(decay)} constants for {self.n_heads} heads")
        name = str(p.get("activation", "silu"))
        if name not in ops.ACTIVATIONS:
            raise ValueError(f"activation {name!r} is not known ({sorted(ops.ACTIVATIONS)})")
        self.activation = ops.ACTIVATIONS[name]
        self.eps = float(p["norm_eps"])
        self.names = dict({"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o"}, **(p.get("names") or {}))
        self.nq, self.nv = self.n_heads * self.dim, self.n_heads * self.v_dim
        # the constants as float32: rounded once from the configuration's double-precision numbers
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.proj: Linear = None
        self.o: Linear = None
        self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d = self.names, self.hidden
        return {n["q"]: ParamSpec((self.nq, d)), n["k"]: ParamSpec((self.nq, d)), n["v"]: ParamSpec((self.nv, d)),
                n["gate"]: ParamSpec((self.nv, d)),
                n["norm"]: ParamSpec((self.nv,), role="vector", init=("ones",)),
                n["o"]: ParamSpec((d, self.nv))}

    def load(self, tensors):
        n = self.names
        ws = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]]
        dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0))         # [q | k | v | gate]
        self.o = Linear(tensors[n["o"]])
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes() + 4 * self.nv

    def cache_requests(self):
        return [StateRequest("S", (self.n_heads, self.dim, self.v_dim))]

    def forward(self, x, ctx, unit, owns_cache):
        T, dev = x.shape[0], x.device
        trace.push("QKV_proj")
        proj = self.proj(x)                                            # [T, q | k | v | gate]
        trace.pop()
        trace.push("Recurrence")
        q = torch.empty((T, self.nq), dtype=torch.float32, device=dev)
        k = torch.empty((T, self.nq), dtype=torch.float32, device=dev)
        v = torch.empty((T, self.nv), dtype=torch.float32, device=dev)
        ops.act_columns(proj, [(0, q), (self.nq, k), (2 * self.nq, v)], self.activation)
        read = torch.empty((T, self.nv), dtype=torch.float32, device=dev)
        ops.matrix_scan(q, k, v, unit.state["S"], ctx.cu_q, ctx.seq_slot, read, ctx.n_seqs, self.n_heads, self.dim,
                        self.v_dim, write_state=owns_cache, max_len=ctx.max_q_len, head_decay=self.decay)
        normed = torch.empty((T, self.nv), dtype=proj.dtype, device=dev)
        ops.head_rmsnorm(read, self.norm_w, self.eps, normed, self.nv, gate=proj[:, 2 * self.nq + self.nv:])
        trace.pop()
        trace.push("Output_proj")
        y = self.o(normed, out_dtype=torch.float32)
        trace.pop()
        return y


register_mixer("decayed_linear_attention", DecayedLinearAttention)
