"""A plain, slow restatement of the Ganupel design: whole sequences, no cache, no kernels, one function per
mechanism, in the precision of the tensors it is given (the tests use float64). It shares no code with the
library; the tests compare the library with it.

Notation: x [n, d] is the residual stream of one sequence of n tokens at positions 0..n-1; `w` maps checkpoint
names to tensors; `m` is a layer's `mixer` object of config.json and `f` its `mlp` object; `p` is the prefix of a
part's tensors.

    layer:    x <- x + ls1 * mixer(norm1(x));  x <- x + ls2 * ff(norm2(x))       (the second only with a feed-forward)
    norm:     x / sqrt(mean(x^2) + eps) * (1 + weight)
    output:   logits = head norm(x)
"""
import math

import torch


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_one(x, weight, eps):
    """The layers' norm: the stored weight is the distance from one."""
    return rms_unit(x, eps) * (1.0 + weight)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def rotate_half(x, positions, base, dims):
    """x [n, heads, D]: entry i < dims/2 of a head is paired with entry i + dims/2; the pair turns by the angle
    position * base^(-2i/dims); entries from `dims` on pass unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def window_visible(n, size):
    """[n, n] booleans: query i sees key j when 0 <= i - j < size (size 0: every j <= i)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size:
        ok = ok & (i - j < size)
    return ok


def sigmoid_attention(u, w, p, m):
    """Grouped-query attention with rotated queries and keys over a sliding window in which every visible key gets
    the weight sigmoid(score + a number per head): no softmax, nothing is normalised over the keys."""
    n = u.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(n)
    q = rotate_half((u @ w[p + "q"].T).view(n, H, D), pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half((u @ w[p + "k"].T).view(n, G, D), pos, m["rot"]["base"], m["rot"]["dims"])
    v = (u @ w[p + "v"].T).view(n, G, Dv)
    ok = window_visible(n, m["mask"]["size"] if m.get("mask") else 0)
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        a = torch.sigmoid(s + w[p + "pb"][h]) * ok
        heads.append(a @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def forget_gate(u, w, p):
    """HGRN2's gate with its lower bound: l + (1 - l) sigmoid(W_f u + b), per head and channel."""
    low = w[p + "lower"]
    return low + (1.0 - low) * torch.sigmoid(u @ w[p + "f"].T + w[p + "f.b"])


def gated_linear_recurrence(u, w, p, m, eps):
    """HGRN2: per head a state S [dim, vdim] from zero, S <- diag(f_t) S + (1 - f_t) v_t^T, read with q_t from the
    new state; each head's reading RMS-normed over vdim with one shared weight."""
    n = u.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(u @ w[p + "q"].T).view(n, H, D)
    v = (u @ w[p + "v"].T).view(n, H, Dv)
    f = forget_gate(u, w, p).view(n, H, D)
    S = torch.zeros(H, D, Dv, dtype=u.dtype)
    out = []
    for t in range(n):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o = torch.einsum("hdv,hd->hv", S, q[t])
        out.append(rms_unit(o, eps) * w[p + "norm"])
    return torch.stack(out).reshape(n, H * Dv) @ w[p + "o"].T


def two_mixers(u, w, p, m, eps):
    """Both mixers read the same input; their results are added with a constant each."""
    return m["left_scale"] * sigmoid_attention(u, w, p + "left.", m["left"]) + \
        m["right_scale"] * gated_linear_recurrence(u, w, p + "right.", m["right"], eps)


def causal_conv(x, taps, bias):
    """x [n, c], taps [c, k]: out_t = bias + sum_j taps[:, k-1-j] x_(t-j), zeros before the sequence."""
    n, k = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(k - 1, x.shape[1], dtype=x.dtype), x])
    out = bias.expand(n, -1).clone()
    for j in range(k):
        out = out + padded[k - 1 - j:k - 1 - j + n] * taps[:, k - 1 - j]
    return out


def block_diagonal(u, mats, bias):
    """u [n, c] cut into equal parts; part b is multiplied by mats[b] ([out, in]) and bias[b] added."""
    B, bw = mats.shape[0], mats.shape[1]
    parts = u.view(u.shape[0], B, bw)
    return (torch.einsum("nbi,boi->nbo", parts, mats) + bias).reshape(u.shape[0], B * bw)


def gated_recurrent_unit(u, w, p, m):
    """Griffin's recurrent block: a gelu branch y, and a branch that goes through a short causal convolution and a
    real-gated linear recurrence S <- a S + sqrt(1 - a^2) (i * u), a = exp(-8 r softplus(lam)), from S = 0."""
    y = gelu_tanh(u @ w[p + "y"].T + w[p + "y.b"])
    x = causal_conv(u @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    r = torch.sigmoid(block_diagonal(x, w[p + "ra"], w[p + "ra.b"]))
    i = torch.sigmoid(block_diagonal(x, w[p + "ri"], w[p + "ri.b"]))
    log_a = -8.0 * r * softplus(w[p + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * x
    S = torch.zeros(x.shape[1], dtype=u.dtype)
    states = []
    for t in range(x.shape[0]):
        S = a[t] * S + drive[t]
        states.append(S)
    return (torch.stack(states) * y) @ w[p + "o"].T


def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with N(t) = t / rms(t) over a token's vector."""
    return coef[0] * rms_unit(z, eps) + coef[1] * rms_unit(z * z, eps) + coef[2] * rms_unit(z ** 3, eps) + coef[3]


def dense_ff(u, w, p, eps):
    return poly_norm(u @ w[p + "up"].T, w[p + "act"], eps) @ w[p + "down"].T


def route(u, w, p, r):
    """Scores = softmax over all outputs of the router (identity experts included); the `top` largest of score +
    correction are chosen; the weights are the chosen scores (without the correction) over their sum, times a
    constant. Returns (chosen [n, top], weights [n, top])."""
    s = torch.softmax(u @ w[p + "router"].T, dim=-1)
    chosen = torch.topk(s + w[p + "correction"], r["top"], dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def choice_margin(u, w, p, r):
    """[n]: how far the last chosen output's choice score lies above the best one not chosen (infinite when every
    output is chosen). A token whose margin is of the size of rounding may choose otherwise in lower precision."""
    s = torch.softmax(u @ w[p + "router"].T, dim=-1) + w[p + "correction"]
    if s.shape[1] <= r["top"]:
        return torch.full((u.shape[0],), float("inf"), dtype=u.dtype)
    best = torch.topk(s, r["top"] + 1, dim=-1).values
    return best[:, -2] - best[:, -1]


def moe(u, w, p, f):
    """Experts are W_down relu(W_up u)^2; the last `identity` outputs of the router stand for experts that return
    their input."""
    r = f["router"]
    chosen, weights = route(u, w, p, r)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for c in range(r["top"]):
            e = int(chosen[t, c])
            if e >= r["experts"]:
                y = u[t]
            else:
                y = (torch.relu(u[t] @ w[f"{p}e{e}.up"].T) ** 2) @ w[f"{p}e{e}.down"].T
            out[t] = out[t] + weights[t, c] * y
    return out


def forward(w, cfg, tokens, layers_out=None, margins_out=None):
    """Logits [n, vocab] of one sequence. `layers_out`, a list, receives the stream after every layer; `margins_out`,
    a list, the routers' choice margins [n] of every layer that has a router."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        u = norm_around_one(x, w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            y = two_mixers(u, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "rglru":
            y = gated_recurrent_unit(u, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + w[p + "ls1"] * y
        f = layer.get("mlp")
        if f is not None:
            u = norm_around_one(x, w[p + "norm2"], eps)
            y = dense_ff(u, w, p + "mlp.", eps) if f["kind"] == "dense" else moe(u, w, p + "mlp.", f)
            if margins_out is not None and f["kind"] != "dense":
                margins_out.append(choice_margin(u, w, p + "mlp.", f["router"]))
            x = x + w[p + "ls2"] * y
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_around_one(x, w["final.norm"], eps) @ w["head"].T
