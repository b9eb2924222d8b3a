"""Latent attention: keys and values are made from a small latent per token, and only the latent is cached.

With u [T, d] the branch input, H heads, per head `dim` plain and `rot` rotated query/key entries, value size
`vdim`, and a latent of `rank` numbers:

    q          = u Wq^T                          heads of [dim plain | rot rotated]
    [c' | k']  = u Wdkv^T                        rank + rot numbers per token
    c          = c' / sqrt(mean(c'^2) + eps) * w_c            float32 RMS norm, plain weight
    k_rot      = R_p k',  q_rot = R_p q[.., dim:]             rotary positions on pairs (2i, 2i+1), angle
                                                              p * base^(-2i / rot_dims), the first rot_dims entries
    per head h:  k_h = Uk_h c,  v_h = Uv_h c                  Uk [H dim, rank], Uv [H vdim, rank]
    s_ij       = scale * (q_plain,i . k_h,j + q_rot,i . k_rot,j)          j <= i, ordinary softmax
    o          = concat_h(sum_j p_ij v_h,j) * sigmoid(u Wg^T)             optional output gate
    y          = o Wo^T

Options, each off by default: `q_rank` r: the queries pass through a latent of their own, c_q = RMSnorm(u Wdq^T) w_q
(float32, eps of the layer), q = c_q Wuq^T; `rot_scaling` {factor, original, fast, slow}: YaRN's blend of the rotary
frequencies and its factor on cos and sin (`rope.yarn_frequencies`; the score scale stays as given); `window` n: token
i sees j with 0 <= i - j < n, and the cache gives pages back behind the window; `sink` "learned": the softmax's
denominator holds one more term exp(s_h) with a learned number per head (no key, no value, unscaled).

The cache holds one row [c | k_rot] per token, and the attention kernel runs on those rows directly: since
q_plain . (Uk_h c) = (Uk_h^T q_plain) . c, the queries become [Uk_h^T q_plain | q_rot] against ONE key head of size
rank + rot, the latent is its own value (the first `rank` columns of the same rows, `KVRequest.values_in_keys`), and
Uv_h is applied to the attention's output. A layer with `owns_latent = False` has no Wdkv: the block hands it the cache
unit of an earlier layer (`LayerCall.cache_of`), which it only reads.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.cache import KVRequest
from ..kernels import ops, trace
from .base import AttentionOptions, Mixer, ParamSpec, register_mixer
from .linear import Linear
from .rope import yarn_frequencies

_DEFAULT_NAMES = {"q": "q", "dkv": "dkv", "latent_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o",
                  "dq": "dq", "q_norm": "dq.norm", "uq": "uq", "sink": "sink"}


def rotation_table(rot_dims: int, base: float, positions: int, device, scaling=None) -> torch.Tensor:
    """float32 [positions, rot_dims / 2, 2] of (cos, sin) of position * base^(-2i / rot_dims); the angles are formed
    in double precision and rounded once. `scaling` {factor, original, fast, slow}: YaRN's frequencies and factor."""
    i = torch.arange(rot_dims // 2, dtype=torch.float64)
    freq = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / rot_dims)
    magnitude = 1.0
    if scaling is not None:
        freq, magnitude = yarn_frequencies(rot_dims, base, float(scaling["factor"]), float(scaling["original"]),
                                           float(scaling["fast"]), float(scaling["slow"]))
    angle = torch.arange(positions, dtype=torch.float64)[:, None] * freq[None, :]
    table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1) * magnitude
    return table.to(torch.float32).contiguous().to(device)


class LatentAttention(Mixer):
    """params: hidden, n_heads, head_dim (plain part), rot_dim, v_head_dim, kv_rank, scale, rot_base, rot_dims (how many
    of the rot_dim entries are rotated; default all), norm_eps, gate (bool), owns_latent (bool: False = reads an
    earlier layer's latent), out_float32 (bool), names; q_rank (None = queries straight from the input), rot_scaling
    (None or {factor, original, fast, slow}), window (0 = every earlier token), sink (None or "learned")."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.n_heads = int(p["hidden"]), int(p["n_heads"])
        self.dim, self.rot, self.vdim, self.rank = int(p["head_dim"]), int(p["rot_dim"]), int(p["v_head_dim"]), int(p["kv_rank"])
        self.rot_dims = int(p.get("rot_dims", self.rot))
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= self.rot:
            raise ValueError(f"rot_dims ({self.rot_dims}) must be even and at most rot_dim ({self.rot})")
        if self.rank + self.rot > 1024 or self.rot <= 0:
            raise ValueError(f"latent rows of {self.rank} + {self.rot} entries: at most 1024, and a rotated part")
        self.rot_base, self.eps = float(p["rot_base"]), float(p["norm_eps"])
        self.gate = bool(p.get("gate", False))
        self.owns_latent = bool(p.get("owns_latent", True))
        self.out_float32 = bool(p.get("out_float32", False))
        self.names = dict(_DEFAULT_NAMES, **(p.get("names") or {}))
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else 0
        self.rot_scaling = dict(p["rot_scaling"]) if p.get("rot_scaling") else None
        self.window = int(p.get("window") or 0)
        if p.get("sink") not in (None, False, "learned"):
            raise ValueError(f"sink must be None or 'learned', got {p.get('sink')!r}")
        self.learned_sink = p.get("sink") == "learned"
        self.options = AttentionOptions(scale=float(p["scale"]), window=self.window)
        self.nq = self.n_heads * (self.dim + self.rot)
        self.no = self.n_heads * self.vdim
        self.row = self.rank + self.rot
        self.table = rotation_table(max(self.rot_dims, 2), self.rot_base, runtime.max_positions, runtime.device,
                                    self.rot_scaling) if runtime.device.type == "cuda" else None
        self.uq: Linear = None
        self.q_norm_w = None
        self.proj: Linear = None
        self.o: Linear = None
        self.norm_w = self.uk_t = self.uv = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d = self.names, self.hidden
        specs = {n["uk"]: ParamSpec((self.n_heads * self.dim, self.rank)),
                 n["uv"]: ParamSpec((self.no, self.rank)), n["o"]: ParamSpec((d, self.no))}
        if self.q_rank:
            specs[n["dq"]] = ParamSpec((self.q_rank, d))
            specs[n["q_norm"]] = ParamSpec((self.q_rank,), role="vector", init=("ones",))
            specs[n["uq"]] = ParamSpec((self.nq, self.q_rank))
        else:
            specs[n["q"]] = ParamSpec((self.nq, d))
        if self.learned_sink:
            specs[n["sink"]] = ParamSpec((self.n_heads,), role="vector", init=("uniform", -1.0, 1.0))
        if self.owns_latent:
            specs[n["dkv"]] = ParamSpec((self.row, d))
            specs[n["latent_norm"]] = ParamSpec((self.rank,), role="vector", init=("ones",))
        if self.gate:
            specs[n["gate"]] = ParamSpec((self.no, d))
        return specs

    def load(self, tensors):
        n = self.names
        ws = [tensors[n["dq"] if self.q_rank else n["q"]]] + ([tensors[n["dkv"]]] if self.owns_latent else []) + \
            ([tensors[n["gate"]]] if self.gate else [])
        dtype = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0))          # rows: q (or its latent) | latent | gate
        self.q_cols = self.q_rank or self.nq                                     # columns the first part takes
        if self.q_rank:
            self.uq = Linear(tensors[n["uq"]])
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
        if self.learned_sink:
            import dataclasses
            self.options = dataclasses.replace(self.options,
                                               sink_values=tensors[n["sink"]].to(torch.float32).contiguous())
        self.o = Linear(tensors[n["o"]])
        # per head: Uk^T as [rank, dim] (the product q_plain -> latent space), Uv as [vdim, rank]
        self.uk_t = tensors[n["uk"]].to(dtype).view(self.n_heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].to(dtype).view(self.n_heads, self.vdim, self.rank).contiguous()
        if self.owns_latent:
            self.norm_w = tensors[n["latent_norm"]].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.proj.nbytes() + self.o.nbytes() + (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size() \
            + (self.uq.nbytes() if self.uq is not None else 0)

    def cache_requests(self):
        return [KVRequest(1, self.row, self.window, values_in_keys=self.rank)]

    def forward(self, x, ctx, unit, owns_cache, residual=None):
        if owns_cache != self.owns_latent:
            raise RuntimeError("a latent-attention layer that makes its own latent must own its cache unit, and one "
                               "that reads another layer's must be given that layer's unit")
        kv = unit.kv
        T, H = x.shape[0], self.n_heads
        trace.push("QKV_proj")
        proj = self.proj(x)                                       # [T, q | latent | gate]
        trace.pop()
        trace.push("Latent+KV_cache")
        q = torch.empty((T, H * self.row), dtype=proj.dtype, device=proj.device)
        q_src = None
        if self.q_rank:
            # the queries' own latent: norm of its columns (float32), then the second product
            cq = ops.rmsnorm_cols(proj, 0, self.q_rank, self.q_norm_w, self.eps,
                                  torch.empty((T, self.q_rank), dtype=proj.dtype, device=proj.device))
            q_src = self.uq(cq)
        ops.latent_prepare(proj, 0, self.q_cols, q, kv.k, self.norm_w, self.eps, self.table, self.rot_dims, ctx.tok_pos,
                           ctx.tok_seq, ctx.seq_slot, kv.block_table, kv.page_size, H, self.dim, self.rot, self.rank,
                           owns_cache, q_src=q_src)
        # the plain query parts into the latent's space: q[:, h, :rank] = q_plain[:, h] Uk_h
        ops.batched_gemm_nt(proj if q_src is None else q_src, self.uk_t, q, self.dim + self.rot, self.row, self.dim)
        trace.pop()
        lat = torch.empty((T, H * self.rank), dtype=proj.dtype, device=proj.device)
        trace.push("FlashDecode" if ctx.decode else "FlashAttn")
        ctx.attention(q, kv, lat, H, 1, self.row, self.options)
        trace.pop()
        trace.push("Output_proj")
        out = torch.empty((T, self.no), dtype=proj.dtype, device=proj.device)
        ops.batched_gemm_nt(lat, self.uv, out, self.rank, self.vdim, self.rank)
        if self.gate:
            ops.sigmoid_gate(out, proj[:, self.q_cols + (self.row if self.owns_latent else 0):])
        y = self.o(out, out_dtype=torch.float32) if self.out_float32 else self.o(out)
        trace.pop()
        return y


register_mixer("latent_attention", LatentAttention)
