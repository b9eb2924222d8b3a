"""A plain, slow restatement of the Burinex design: whole sequences, no cache, no kernels, one function per mechanism.

It shares no code with the library. `cfg` is the parsed config.json (a dict), `w` maps checkpoint names to tensors;
everything runs in the dtype of the tensors it is given (the tests use float64). Notation: T tokens, d the model
width, H heads, G key/value heads, D / Dv the query-key / value head sizes.
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softmax_with_extra(s, extra):
    """Row softmax of s [.., T, T] (masked entries are -inf) whose denominator holds one more term exp(extra)
    (extra broadcastable to s[..., :1]); the extra term has no value, so the weights sum to less than one."""
    m = torch.maximum(s.max(dim=-1, keepdim=True).values, extra)
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(extra - m))


def causal_mask(T, window=0):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    return ok


# ----------------------------------------------------------------------------------------------- mixers
def query_temperature(T, coef, every, dtype):
    """1 + coef * ln(floor((p + 1) / every) + 1) for p = 0 .. T-1."""
    p = torch.arange(T, dtype=torch.float64)
    return (1.0 + coef * torch.log(torch.floor((p + 1) / every) + 1.0)).to(dtype)


def attention(h, m, w, pre, eps):
    """Grouped-query attention, norms over the whole q and k vectors, a temperature on q that grows with the
    position, a softmax with one more term exp(0), one sigmoid gate per head."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]
    k = rms(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]
    v = h @ w[pre + "v"].T
    if m.get("q_temp") is not None:
        q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None]
    q = q.view(T, H, D).transpose(0, 1)                       # [H, T, D]
    k = k.view(T, G, D).transpose(0, 1).repeat_interleave(H // G, dim=0)
    v = v.view(T, G, Dv).transpose(0, 1).repeat_interleave(H // G, dim=0)
    s = (q @ k.transpose(1, 2)) * m["scale"]
    s = s.masked_fill(~causal_mask(T), float("-inf"))
    p = softmax_with_extra(s, torch.zeros((), dtype=h.dtype))
    o = (p @ v).transpose(0, 1)                                # [T, H, Dv]
    gate = torch.sigmoid(h @ w[pre + "g"].T)                   # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * Dv) @ w[pre + "o"].T


def rotary_table(T, rot, dtype=torch.float64):
    """cos, sin [T, dims / 2] of the interleaved rotation, with the frequency blend and magnitude of YaRN when
    `rot["scaling"]` is there."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc is not None:
        def where(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(where(sc["fast"])), 0)
        hi = min(math.ceil(where(sc["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    a = torch.arange(T, dtype=torch.float64)[:, None] * f[None, :]
    return (torch.cos(a) * mag).to(dtype), (torch.sin(a) * mag).to(dtype)


def rotate_pairs(x, cos, sin, dims):
    """x [T, .., n]: the first `dims` entries in pairs (2i, 2i+1) turned by the angle of the token's position."""
    T = x.shape[0]
    shape = [T] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = cos.view(shape), sin.view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h, m, w, pre, eps):
    """Queries through a normed latent; keys and values from a normed latent plus one rotated key part that all
    heads share; a sliding window; a learned term per head in the softmax's denominator."""
    T = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, D + R)
    ckr = h @ w[pre + "dkv"].T
    c = rms(ckr[:, :rank], eps) * w[pre + "dkv.norm"]
    kr = ckr[:, rank:]                                          # [T, R]
    cos, sin = rotary_table(T, m["rot"], h.dtype)
    dims = m["rot"]["dims"]
    q_rot = rotate_pairs(q[:, :, D:], cos, sin, dims)
    kr = rotate_pairs(kr, cos, sin, dims)
    k = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, Dv)
    s = torch.einsum("ihd,jhd->hij", q[:, :, :D], k) + torch.einsum("ihr,jr->hij", q_rot, kr)
    s = s * m["scale"]
    window = m["mask"]["size"] if m.get("mask") is not None else 0
    s = s.masked_fill(~causal_mask(T, window), float("-inf"))
    p = softmax_with_extra(s, w[pre + "sink"].to(h.dtype)[:, None, None])
    o = torch.einsum("hij,jhd->ihd", p, v)
    return o.reshape(T, H * Dv) @ w[pre + "o"].T


def lightning(h, m, w, pre, eps, state=None):
    """Linear attention with a constant decay per head: S_t = a S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[pre + "q"].T).view(T, H, D)
    k = silu(h @ w[pre + "k"].T).view(T, H, D)
    v = silu(h @ w[pre + "v"].T).view(T, H, Dv)
    a = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, Dv, dtype=h.dtype) if state is None else state
    out = []
    for t in range(T):
        S = a[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = torch.stack(out).reshape(T, H * Dv)
    o = rms(o, eps) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


# ----------------------------------------------------------------------------------------------- feed-forward
def expert(x, w, pre):
    return (silu(x @ w[pre + "gate"].T) * (x @ w[pre + "up"].T)) @ w[pre + "down"].T


def routed_experts(h, f, w, pre, margins_out=None):
    """Sigmoid router: the `top` largest scores choose, the scores themselves weigh, and the weight multiplies what
    the expert READS. A shared expert reads every token as it is. `margins_out`, a list, receives per token the gap
    between the last chosen logit and the first one left out (infinite when every expert is chosen)."""
    T = h.shape[0]
    z = h @ w[pre + "router"].T
    scores = torch.sigmoid(z)
    top = f["router"]["top"]
    val, idx = torch.topk(scores, top, dim=-1)
    if margins_out is not None:
        zs = torch.sort(z, dim=-1, descending=True).values
        margins_out.append(zs[:, top - 1] - zs[:, top] if top < z.shape[1] else torch.full((T,), float("inf")))
    out = torch.zeros_like(h)
    for t in range(T):
        for c in range(top):
            e = int(idx[t, c])
            out[t] += expert(val[t, c] * h[t], w, f"{pre}e{e}.")
    if f.get("shared") is not None:
        out = out + expert(h, w, pre + "shared.")
    return out


# ----------------------------------------------------------------------------------------------- the model
MIXERS = {"attention": attention, "latent_attention": latent_attention, "lightning": lightning}


def forward(cfg, w, tokens, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one whole sequence. `layers_out`, a list, receives the stream after every layer;
    `margins_out`, a list, every router's choice margins per token."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        y = MIXERS[layer["type"]](x, layer["mixer"], w, pre + "mix.", eps)
        x = rms(alpha * x + y * w[pre + "ls1"], eps) * w[pre + "norm1"]
        if layer.get("mlp") is not None:
            y = routed_experts(x, layer["mlp"], w, pre + "mlp.", margins_out)
            x = rms(alpha * x + y * w[pre + "ls2"], eps) * w[pre + "norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * w["final.norm"]
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
