"""Gated grouped-query attention without rotation, over a window that keeps the first tokens.

With h the layer's input [T, d], H query heads of size D, G key/value heads (query head i reads key/value head
i // (H / G)), and value heads of size Dv:

    q = h Wq^T, k = h Wk^T, v = h Wv^T, g = h Wg^T                      one product over row-concatenated weights
    q <- q / sqrt(mean(q^2) + eps) * wq      over ALL H*D elements of a token's q at once (not per head);
    k <- likewise with wk over all G*D       float32, plain weights
    v <- (1 - lam) v + lam v_first           in layers that blend: v_first is what the first blending layer of
                                             the model projected for the same token; lam a learned scalar
    s_ij = scale * q_i . k_j                 no position enters the scores
    j visible to i:  j <= i and (i - j < window or j < keep_first)
    p_ij = exp(s_ij) / (1 + sum_j' exp(s_ij'))        a sink: one more key of score 0 that has no value
    o_i  = (sum_j p_ij v_j) * sigmoid(g_i)   gate on the concatenated heads, from the same input h
    y    = o Wo^T                            float32, to the norm that follows the branch

Keys are cached normalised and values blended, so a later step reads them as they are. Every constant is a
parameter; each option has an "off" value, so the part also serves designs that use only some of them.

Three more options change single scores, each off by default:

    s_ij <- c * tanh(s_ij / c)               `softcap` c, after the scale
    s_ij <- s_ij + B[bucket(i - j), head]    `distance_bias` {rows, far}: a learned table B [rows, heads]; with
                                             m = rows // 2, bucket(n) = n for n < m, else
                                             min(rows - 1, m + floor(ln(n / m) / ln(far / m) * (rows - m))): one row
                                             per distance nearby, rows evenly spaced in log(distance) up to `far`
                                             beyond, the last row for everything farther; added after the cap, unscaled
    sink = "learned"                         the sink's score is a learned number per head instead of 0

    q_i <- q_i (1 + a ln(floor((i + 1) / n) + 1))    `q_temp` {coef a, every n}: a temperature on the queries that grows
                                             with the position i, applied after the query norm (float32)
    gate = "head"                            ONE gate per head instead of one per channel: Wg has H rows and head h's
                                             output is multiplied by sigmoid(g_i)_h

Two more, also off by default: `position` (a position encoding, e.g. rotary: q and k are encoded before the scores and
keys are cached encoded; it takes the place of the query/key norm) and `weights = "sigmoid"`: no softmax, a visible
key's weight is sigmoid(s_ij + b_head) with a learned number per head, and nothing is normalised over the keys.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from ..cache.cache import KVRequest
from ..kernels import ops, trace
from .base import AttentionOptions, DeferredBranchAdd, Mixer, ParamSpec, build_part, register_mixer
from .linear import Linear

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                  "blend": "vmix", "distance_bias": "rel", "sink": "sink", "sigmoid_bias": "pb"}


RANDOM_BIAS_ROWS = 16


def distance_buckets(rows: int, far: float, longest: int) -> List[int]:
    """Row of the bias table for each distance 0, 1, 2, ... up to the first distance that reaches the last row (all
    farther ones share it) or `longest`, whichever comes first. Computed in double precision on the host."""
    half = rows // 2
    out = []
    for n in range(max(1, longest)):
        if n < half:
            b = n
        else:
            b = min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b == rows - 1:
            break
    return out


class GatedAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, head_dim, v_head_dim, scale (None = 1/sqrt(head_dim)), window (0 = every
    earlier key), keep_first, sink (bool), qk_norm_eps (None = no query/key norm), gate (bool, or "head" for one gate
    per head), q_temp (None or {coef, every}), value_blend
    (None, "first": leaves its projected values for later layers, or "blend": mixes them into its own),
    blend_key (name under which the first layer's values travel through the step), names (overrides of the
    tensors' checkpoint sub-names), position (PartSpec of a position encoding for q and k, None = none), weights
    ("softmax", the default, or "sigmoid")."""

    accepts_deferred_branch_add = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.n_heads, self.n_kv_heads = int(p["hidden"]), int(p["n_heads"]), int(p["n_kv_heads"])
        self.head_dim, self.v_head_dim = int(p["head_dim"]), int(p.get("v_head_dim") or p["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"n_heads ({self.n_heads}) must be a multiple of n_kv_heads ({self.n_kv_heads})")
        if max(self.head_dim, self.v_head_dim) > 256:
            raise ValueError(f"head sizes {self.head_dim} / {self.v_head_dim} exceed what the attention kernels take (256)")
        scale = p.get("scale")
        self.window, self.keep_first = int(p.get("window") or 0), int(p.get("keep_first") or 0)
        if not self.window:
            self.keep_first = 0
        self.learned_sink = p.get("sink") == "learned"
        self.softcap = float(p.get("softcap") or 0.0)
        self.distance_bias = p.get("distance_bias")
        if self.distance_bias is not None:
            # rows None: the table's height is whatever the checkpoint holds (a random model gets RANDOM_BIAS_ROWS)
            rows = self.distance_bias.get("rows")
            self.distance_bias = {"rows": None if rows is None else int(rows), "far": float(self.distance_bias["far"])}
        self.options = AttentionOptions(scale=float(scale) if scale is not None else self.head_dim ** -0.5,
                                        window=self.window, keep_first=self.keep_first, sink=bool(p.get("sink", False)),
                                        softcap=self.softcap)
        self.qk_norm_eps = p.get("qk_norm_eps")
        self.position = build_part("position_encoding", p["position"], runtime) if p.get("position") else None
        if self.position is not None and (self.qk_norm_eps is not None or p.get("value_blend")):
            raise ValueError("a position encoding takes the place of the query/key norm and the value blend")
        self.sigmoid = p.get("weights", "softmax") == "sigmoid"
        if p.get("weights", "softmax") not in ("softmax", "sigmoid"):
            raise ValueError(f"weights must be 'softmax' or 'sigmoid', got {p.get('weights')!r}")
        if self.sigmoid and (p.get("sink") or self.softcap or self.distance_bias is not None or self.keep_first):
            raise ValueError("sigmoid weights go with scale and window only")
        self.gate = bool(p.get("gate", False))
        self.head_gate = p.get("gate") == "head"
        temp = p.get("q_temp")
        self.temp_coef, self.temp_every = (float(temp["coef"]), int(temp["every"])) if temp else (0.0, 0)
        if temp and self.temp_every <= 0:
            raise ValueError(f"q_temp.every must be positive, got {self.temp_every}")
        if temp and self.position is not None:
            raise ValueError("a query temperature goes with the query/key norm's kernel, not with a position encoding")
        self.value_blend = p.get("value_blend")
        if self.value_blend not in (None, "first", "blend"):
            raise ValueError(f"value_blend must be None, 'first' or 'blend', got {self.value_blend!r}")
        self.blend_key = str(p.get("blend_key", "first_values"))
        self.names = dict(_DEFAULT_NAMES, **(p.get("names") or {}))
        self.nq, self.nk = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        self.nv, self.no = self.n_kv_heads * self.v_head_dim, self.n_heads * self.v_head_dim
        self.proj: Linear = None
        self.o: Linear = None
        self.q_w = self.k_w = self.lam = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d = self.names, self.hidden
        specs = {n["q"]: ParamSpec((self.nq, d)), n["k"]: ParamSpec((self.nk, d)), n["v"]: ParamSpec((self.nv, d)),
                 n["o"]: ParamSpec((d, self.no))}
        if self.gate:
            specs[n["gate"]] = ParamSpec((self.n_heads if self.head_gate else self.no, d))
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = ParamSpec((self.nq,), role="vector", init=("ones",))
            specs[n["k_norm"]] = ParamSpec((self.nk,), role="vector", init=("ones",))
        if self.distance_bias is not None:
            rows = self.distance_bias["rows"]
            specs[n["distance_bias"]] = ParamSpec((rows if rows is not None else -RANDOM_BIAS_ROWS, self.n_heads),
                                                  role="vector", init=("uniform", -1.0, 1.0))
        if self.learned_sink:
            specs[n["sink"]] = ParamSpec((self.n_heads,), role="vector", init=("uniform", -1.0, 1.0))
        if self.sigmoid:
            specs[n["sigmoid_bias"]] = ParamSpec((self.n_heads,), role="vector", init=("uniform", -6.0, -2.0))
        if self.value_blend is not None:
            # only a blending layer reads the scalar; a checkpoint may hold one for the first layer as well
            specs[n["blend"]] = ParamSpec((), role="vector", init=("uniform", 0.2, 0.8),
                                          optional=self.value_blend != "blend")
        return specs

    def load(self, tensors):
        n = self.names
        ws = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["gate"]]] if self.gate else [])
        dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0))
        self.o = Linear(tensors[n["o"]])
        if self.qk_norm_eps is not None:
            self.q_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_w = tensors[n["k_norm"]].to(torch.float32).contiguous()
        if self.value_blend == "blend":
            self.lam = tensors[n["blend"]].to(torch.float32).reshape(1).contiguous()
        extra = {}
        if self.distance_bias is not None:
            # the table by bucket becomes a table by distance: [heads, L], distances of L - 1 and more share a column
            table = tensors[n["distance_bias"]].to(torch.float32)
            rows, far = table.shape[0], self.distance_bias["far"]
            if rows < 2 or far <= rows // 2:
                raise ValueError(f"distance bias: a table of {rows} rows needs at least 2 rows and far ({far}) beyond "
                                 "half of them")
            longest = self.window if self.window else self.runtime.max_positions
            buckets = distance_buckets(rows, far, longest)
            index = torch.tensor(buckets, dtype=torch.long, device=table.device)
            extra["distance_bias"] = table[index].t().contiguous()
        if self.learned_sink:
            extra["sink_values"] = tensors[n["sink"]].to(torch.float32).contiguous()
        if self.sigmoid:
            extra["sigmoid_bias"] = tensors[n["sigmoid_bias"]].to(torch.float32).contiguous()
        if extra:
            import dataclasses
            self.options = dataclasses.replace(self.options, **extra)

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes() + (4 * (self.nq + self.nk) if self.q_w is not None else 0)

    def cache_requests(self):
        return [KVRequest(self.n_kv_heads, self.head_dim, self.window, v_head_dim=self.v_head_dim,
                          keep_first=self.keep_first)]

    def forward(self, x, ctx, unit, owns_cache, residual=None):
        kv = unit.kv
        T = x.shape[0]
        trace.push("QKV_proj")
        if isinstance(x, DeferredBranchAdd):
            # one-token steps: the add that closes the previous layer happens inside this product's kernel
            proj = self.proj.after_branch_add(x) if x.foldable(self.proj.weight) else self.proj(_rounded(x, self.runtime))
        else:
            proj = self.proj(x)                               # [T, q | k | v | gate]
        trace.pop()
        v_first = None
        if self.value_blend == "first":
            ctx.carry[self.blend_key] = proj[:, self.nq + self.nk:self.nq + self.nk + self.nv]
        elif self.value_blend == "blend":
            v_first = ctx.carry.get(self.blend_key)
            if v_first is None:
                raise RuntimeError(f"a layer blends its values with {self.blend_key!r}, but no earlier layer of this "
                                   "step has left any")
        if self.position is not None:
            trace.push("RoPE+KV_cache")
            qkv = proj if not self.gate else proj[:, :self.nq + self.nk + self.nv].contiguous()
            q = self.position.encode_and_store(qkv, ctx, kv, self.n_heads, self.n_kv_heads, self.head_dim, owns_cache,
                                               v_head_dim=self.v_head_dim)
        else:
            trace.push("QKnorm+KV_cache")
            q = torch.empty((T, self.nq), dtype=proj.dtype, device=proj.device)
            ops.qk_norm_store(proj, q, kv.k, kv.v, self.q_w, self.k_w, float(self.qk_norm_eps or 0.0), ctx.tok_pos,
                              ctx.tok_seq, ctx.seq_slot, kv.block_table, kv.page_size, self.n_heads, self.n_kv_heads,
                              self.head_dim, self.v_head_dim, owns_cache, lam=self.lam, v_first=v_first,
                              temp_coef=self.temp_coef, temp_every=self.temp_every)
        trace.pop()
        out = torch.empty((T, self.no), dtype=proj.dtype, device=proj.device)
        gate = proj[:, self.nq + self.nk + self.nv:] if self.gate else None
        trace.push("FlashDecode" if ctx.decode else "FlashAttn")
        ctx.attention(q, kv, out, self.n_heads, self.n_kv_heads, self.head_dim, self.options,
                      gate=None if self.head_gate else gate)
        if self.head_gate:
            ops.sigmoid_gate(out, gate, group=self.v_head_dim)
        trace.pop()
        trace.push("Output_proj")
        y = self.o(out, out_dtype=torch.float32)
        trace.pop()
        return y


def _rounded(pending: DeferredBranchAdd, runtime) -> torch.Tensor:
    """Does a deferred branch add in its own kernel and returns the new stream as a product reads it."""
    if runtime.dtype == torch.float32:
        return pending.apply()
    act = torch.empty(pending.shape, dtype=runtime.dtype, device=pending.h.device)
    pending.apply(act)
    return act


register_mixer("gated_attention", GatedAttention)
