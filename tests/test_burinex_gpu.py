"""Burinex on the GPU against its plain restatement (tests/plain_burinex.py): each new kernel and part alone, keys at
the window's edges with one score made to stand out, state that is carried, freed and taken again, and the engine in
float32 and bfloat16 over whole prompts, token-by-token decoding, prompts in pieces down to two tokens, unequal batches
with slots and pages used again, long decoding and greedy generation through the library's own entry point."""
import json
import os

import pytest
import torch

import helpers
import plain_burinex as plain
from test_parts_gpu import DEV, DTYPES, build, kernel_plan, make_ctx

pytestmark = pytest.mark.gpu


def _moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared} if shared else None}


def _attn(heads, kv, dim, vdim, scale, temp):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
            "q_temp": {"coef": temp[0], "every": temp[1]} if temp else None}


def _latent(heads, dim, rot_dim, vdim, rank, q_rank, scale, window, base, dims, scaling):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
            "scale": scale, "mask": {"size": window} if window else None,
            "rot": {"base": base, "dims": dims, "scaling": dict(zip(("factor", "original", "fast", "slow"), scaling))
                    if scaling else None}}


# A: every layer differs. A linear-attention layer first, value heads narrower and wider than key heads, as many key
# heads as query heads, a layer without a feed-forward, a router that takes one expert, one that takes all of them, one
# without a shared expert, a window shorter than a page, a temperature that changes every 16 tokens and none at all.
TINY_A = {"architecture": "Burinex", "vocab": 211, "width": 96, "postln_alpha": 2.5, "logit_softcap": 20.0,
          "norm": {"eps": 1e-5}, "layers": [
    {"type": "lightning", "mixer": {"heads": 3, "dim": 20, "vdim": 24, "decay": [0.5, 0.9, 0.995]},
     "mlp": _moe(6, 3, 40, 56)},
    {"type": "attention", "mixer": _attn(6, 3, 32, 16, 0.2, (0.4, 16)), "mlp": None},
    {"type": "latent_attention", "mixer": _latent(4, 24, 8, 20, 40, 48, 0.15, 24, 10000.0, 8, (8.0, 64, 16.0, 2.0)),
     "mlp": _moe(4, 1, 24, None)},
    {"type": "attention", "mixer": _attn(4, 4, 20, 28, 0.3, None), "mlp": _moe(5, 5, 16, 32)}]}
# B: a width that is no multiple of 8, no cap on the logits, alpha 1, one key head, one latent head, latent rows that
# are no multiple of 16 (the plain attention kernel in both precisions), a window longer
# than a page and one of three tokens, no window, a rotation over a part of the rotated entries and without scaling, a
# temperature that changes with every token, a single linear-attention head with more channels than a warp has lanes.
TINY_B = {"architecture": "Burinex", "vocab": 97, "width": 100, "postln_alpha": 1.0, "logit_softcap": None,
          "norm": {"eps": 1e-6}, "layers": [
    {"type": "latent_attention", "mixer": _latent(2, 16, 16, 16, 48, 24, 0.2, 70, 500.0, 8, None), "mlp": _moe(3, 2, 20, 20)},
    {"type": "lightning", "mixer": {"heads": 5, "dim": 12, "vdim": 20, "decay": [0.3, 0.7, 0.9, 0.97, 1.0]}, "mlp": None},
    {"type": "latent_attention", "mixer": _latent(1, 32, 4, 8, 12, 20, 0.25, 3, 50.0, 4, (2.0, 16, 4.0, 1.0)),
     "mlp": _moe(2, 1, 12, 28)},
    {"type": "attention", "mixer": _attn(4, 1, 16, 16, 0.25, (0.3, 1)), "mlp": _moe(7, 2, 10, None)},
    {"type": "latent_attention", "mixer": _latent(3, 8, 8, 12, 20, 16, 0.3, 0, 10000.0, 8, (4.0, 32, 8.0, 0.5)),
     "mlp": None},
    {"type": "lightning", "mixer": {"heads": 1, "dim": 40, "vdim": 12, "decay": [0.98]}, "mlp": _moe(3, 3, 16, 8)}]}
# C: head sizes 64 and 128 with equal value sizes (what the fastest attention kernels take), latent rows of 128 and 256,
# wide linear-attention heads, windows of a page + 1 and of 100.
TINY_C = {"architecture": "Burinex", "vocab": 160, "width": 128, "postln_alpha": 4.0, "logit_softcap": 50.0,
          "norm": {"eps": 1e-6}, "layers": [
    {"type": "attention", "mixer": _attn(4, 2, 64, 64, 0.125, (0.25, 64)), "mlp": _moe(4, 2, 64, 64)},
    {"type": "latent_attention", "mixer": _latent(4, 64, 16, 64, 112, 64, 0.11, 100, 20000.0, 16, (3.0, 128, 16.0, 1.0)),
     "mlp": _moe(8, 2, 32, 48)},
    {"type": "lightning", "mixer": {"heads": 2, "dim": 128, "vdim": 64, "decay": [0.9, 0.999]}, "mlp": _moe(4, 1, 64, None)},
    {"type": "attention", "mixer": _attn(2, 1, 128, 128, 0.09, (0.5, 100)), "mlp": None},
    {"type": "latent_attention", "mixer": _latent(2, 32, 32, 32, 224, 32, 0.1, 65, 100000.0, 32, None),
     "mlp": _moe(4, 3, 32, 32)}]}
CFGS = {"a": TINY_A, "b": TINY_B, "c": TINY_C}
LENGTHS = {"a": [1, 5, 64, 65, 130, 300], "b": [3, 77, 200, 257], "c": [40, 129, 260]}
SHARPEN = {"a": 1.4, "b": 1.5, "c": 1.5}        # factor on what makes the attention scores
_folders, _engines = {}, {}


def folder_for(tag):
    """A model folder of random weights: wide embeddings, sharp attention scores (a few keys carry nearly all the
    weight, so one that is lost or added shows), sinks that take a share, layer scales and norm weights away from 1."""
    from llm_infer_engine_b200.weights.random_init import random_tensors
    from llm_infer_engine_b200.weights.safetensors_io import save_file
    if tag not in _folders:
        d = helpers.scratch_folder(f"llmie_burinex_{tag}_")
        tensors, _ = random_tensors(CFGS[tag], seed=51 + len(_folders), std=0.09, norm_range=(0.7, 1.3))
        g = torch.Generator().manual_seed(8)
        for name in tensors:
            t = tensors[name].float()
            if name == "embed":
                t = t * 8.0
            elif name.endswith(("mix.q.norm", "mix.uq")):
                t = t * SHARPEN[tag]
            elif name.endswith(("mix.uk", "mix.k.norm")):
                t = t * 1.5
            elif name.endswith(".sink"):
                t = torch.rand(t.shape, generator=g) * 3.0
            elif name.endswith((".o", ".down", ".uv", "mix.v")):
                t = t * 2.0
            elif name.endswith(".router"):
                t = t * 2.0
            tensors[name] = t.to(torch.bfloat16)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CFGS[tag], f)
        save_file(tensors, os.path.join(d, "model.safetensors"))
        _folders[tag] = d
    return _folders[tag]


def plain_weights(tag):
    from safetensors.torch import load_file
    return {k: v.double() for k, v in load_file(os.path.join(folder_for(tag), "model.safetensors")).items()}


def engine_for(tag, dtype, **kw):
    from llm_infer_engine_b200 import Engine
    key = (tag, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine(folder_for(tag), dtype=dtype, max_batch=kw.pop("max_batch", 8),
                               max_tokens=kw.pop("max_tokens", 64 * 48), cuda_graph=kw.pop("cuda_graph", False), **kw)
    return _engines[key]


def bound(dtype, want):
    return (3e-5 if dtype == "float32" else 0.05) * max(1.0, float(want.abs().max()))


CLOSE_CALL = 0.08          # a router's choice margin below this may fall the other way in bfloat16
_close_calls = {}


def oracle(tag, requests):
    """The plain logits of every request, and per request the tokens at which some router chooses by a margin that
    bfloat16 rounding can turn (bfloat16 comparisons count those among the positions over the bound only)."""
    w = plain_weights(tag)
    out = {}
    for rid, toks in requests.items():
        margins = []
        out[rid] = plain.forward(CFGS[tag], w, toks, margins_out=margins).float()
        close = torch.zeros(len(toks), dtype=torch.bool)
        for m in margins:
            close |= m < CLOSE_CALL
        _close_calls[(tag, rid)] = close
    return out


def compare(got, want, dtype, what, tag=None):
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        diff = (got[rid] - want[rid]).abs().max(dim=1).values
        tol_ = bound(dtype, want[rid])
        over = int((diff > tol_).sum())
        allowed = 0 if dtype == "float32" else max(1, len(diff) // 25)
        firm = diff
        if dtype != "float32" and (tag, rid) in _close_calls:
            firm = diff[~_close_calls[(tag, rid)][:len(diff)]]
        worst = float(firm.max()) if len(firm) else 0.0
        assert over <= allowed and worst <= (tol_ if dtype == "float32" else 3 * tol_), (
            f"{what}: request {rid}: {over} of {len(diff)} positions over the bound {tol_:.3e}, worst "
            f"{float(diff.max()):.3e}, first at token {int((diff > tol_).nonzero()[0])}")


def requests_for(tag):
    return {f"r{i}": helpers.random_tokens(CFGS[tag]["vocab"], n, seed=40 + i) for i, n in enumerate(LENGTHS[tag])}


def tol(dtype, scale):
    return (2e-5 if dtype == "float32" else 2e-2) * max(1.0, scale)


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [200, 202, 204, 2048, 9000])
@pytest.mark.parametrize("y_dtype", ["float32", "bfloat16"])
def test_scale_sum_and_norm_in_one_kernel(dtype, size, y_dtype):
    """h = norm(alpha h + s (.) y) w in place, and the rounded copy the next product reads."""
    norm, w = build("norm", "rmsnorm", {"size": size, "eps": 1e-5, "weight_name": "", "residual_scale": 2.5}, dtype, seed=2)
    g = torch.Generator().manual_seed(size)
    h = torch.randn(7, size, generator=g) * 3
    y = (torch.randn(7, size, generator=g) * 2).to(DTYPES[y_dtype])
    s = torch.rand(size, generator=g) + 0.5
    want = plain.rms(2.5 * h.double() + s.double() * y.double(), 1e-5) * w[""].double()
    for vector, ref in ((s.to(DEV), want), (None, plain.rms(2.5 * h.double() + y.double(), 1e-5) * w[""].double())):
        hd = h.clone().to(DEV)
        act = torch.empty(7, size, dtype=DTYPES[dtype], device=DEV)
        norm.norm_sum(hd, y.to(DEV), vector, act)
        assert float((hd.cpu().double() - ref).abs().max()) <= 2e-5 * float(ref.abs().max())
        assert float((act.float().cpu().double() - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_kernels_of_the_design(dtype):
    """A norm over a run of columns, a gate per head, the cap on the logits, activations of runs of columns, the norm
    over the concatenated heads with its gate."""
    from llm_infer_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    dt = DTYPES[dtype]
    src = (torch.randn(9, 70, generator=g) * 2).to(dt)
    w = torch.rand(24, generator=g) + 0.5
    out = ops.rmsnorm_cols(src.to(DEV), 11, 24, w.to(DEV), 1e-5, torch.empty(9, 24, dtype=dt, device=DEV))
    ref = plain.rms(src[:, 11:35].double(), 1e-5) * w.double()
    assert float((out.float().cpu().double() - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))

    o = torch.randn(9, 6 * 20, generator=g).to(dt)
    wide = torch.randn(9, 50, generator=g).to(dt)
    got = ops.sigmoid_gate(o.clone().to(DEV), wide.to(DEV)[:, 30:36], group=20).float().cpu().double()
    ref = (o.double().view(9, 6, 20) * torch.sigmoid(wide[:, 30:36].double())[:, :, None]).reshape(9, -1)
    assert float((got - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))

    x = torch.randn(5, 301, generator=g) * 40
    got = ops.cap_rows(x.clone().to(DEV), 25.0).cpu().double()
    assert float((got - 25.0 * torch.tanh(x.double() / 25.0)).abs().max()) <= 1e-4

    proj = torch.randn(13, 100, generator=g).to(dt)
    outs = [torch.empty(13, n, device=DEV) for n in (24, 24, 40)]
    ops.act_columns(proj.to(DEV), [(0, outs[0]), (24, outs[1]), (48, outs[2])], ops.ACT_SILU)
    ref = plain.silu(proj.double())
    for off, t in zip((0, 24, 48), outs):
        assert float((t.cpu().double() - ref[:, off:off + t.shape[1]]).abs().max()) <= 1e-5

    read = torch.randn(13, 60, generator=g) * 4
    wn = torch.rand(60, generator=g) + 0.5
    gate = torch.randn(13, 100, generator=g).to(dt)
    got = ops.head_rmsnorm(read.to(DEV), wn.to(DEV), 1e-5, torch.empty(13, 60, dtype=dt, device=DEV), 60,
                           gate=gate.to(DEV)[:, 40:]).float().cpu().double()
    ref = plain.rms(read.double(), 1e-5) * wn.double() * torch.sigmoid(gate[:, 40:].double())
    assert float((got - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))
    for width in (512, 2052, 4096):                      # wide rows: a block per row
        read_w = torch.randn(5, width, generator=g) * 4
        w_w = torch.rand(width, generator=g) + 0.5
        gate_w = torch.randn(5, width + 24, generator=g).to(dt)
        for gt in (gate_w.to(DEV)[:, 24:], None):
            got = ops.head_rmsnorm(read_w.to(DEV), w_w.to(DEV), 1e-5, torch.empty(5, width, dtype=dt, device=DEV), width,
                                   gate=gt).float().cpu().double()
            ref = plain.rms(read_w.double(), 1e-5) * w_w.double()
            if gt is not None:
                ref = ref * torch.sigmoid(gate_w[:, 24:].double())
            assert float((got - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))
    # a norm per head with a weight the heads share, and a gate
    got = ops.head_rmsnorm(read.to(DEV), wn[:20].contiguous().to(DEV), 1e-5, torch.empty(13, 60, dtype=dt, device=DEV),
                           20, gate=gate.to(DEV)[:, 40:]).float().cpu().double()
    ref = (plain.rms(read.double().view(13, 3, 20), 1e-5) * wn[:20].double()).reshape(13, 60) * \
        torch.sigmoid(gate[:, 40:].double())
    assert float((got - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))


def _plain_decay_scan(q, k, v, decay):
    H, D, Dv = q.shape[1], q.shape[2], v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=torch.float64)
    a = torch.tensor(decay, dtype=torch.float64)
    rows = []
    for t in range(q.shape[0]):
        S = a[:, None, None] * S + k[t].double()[:, :, None] * v[t].double()[:, None, :]
        rows.append(torch.einsum("hdv,hd->hv", S, q[t].double()).reshape(-1))
    return torch.stack(rows)


@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 24), (1, 8, 40), (2, 128, 32), (1, 300, 16), (2, 48, 136)])
def test_keyed_scan_in_pieces_and_chunks_equals_the_plain_loop(heads, dim, vdim):
    """S <- a_h S + k v^T: three sequences in pieces of unequal sizes, single tokens, and pieces long enough for the
    form that runs chunks side by side (one ending exactly at a chunk's end); decays of 1 and next to 0; the state in
    the slots, another slot's state untouched."""
    from llm_infer_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(dim + vdim)
    lens = [701, 322, 135]
    decay = [1.0, 0.05, 0.97][:heads] if heads <= 3 else None
    q = [torch.randn(n, heads, dim, generator=g) * 0.3 for n in lens]
    k = [torch.randn(n, heads, dim, generator=g) * 0.3 for n in lens]
    v = [torch.randn(n, heads, vdim, generator=g) for n in lens]
    want = [_plain_decay_scan(q[i], k[i], v[i], decay) for i in range(3)]
    state = torch.zeros(5, heads, dim, vdim, device=DEV)
    state[2] = 7.0
    slots = torch.tensor([3, 1, 4], dtype=torch.int32, device=DEV)
    a = torch.tensor(decay, dtype=torch.float32, device=DEV)
    held = [0, 0, 0]
    for pieces in ([20, 1, 5], [1, 1, 1], [279, 192, 0], [1, 1, 1], [400, 127, 128]):
        live = [i for i in range(3) if pieces[i]]
        cu = [0]
        for i in live:
            cu.append(cu[-1] + pieces[i])
        cat = lambda xs: torch.cat([xs[i][held[i]:held[i] + pieces[i]].reshape(pieces[i], -1) for i in live]).to(DEV)
        out = torch.empty(cu[-1], heads * vdim, device=DEV)
        ops.matrix_scan(cat(q), cat(k), cat(v), state, torch.tensor(cu, dtype=torch.int32, device=DEV),
                        slots[live].contiguous(), out, len(live), heads, dim, vdim, max_len=max(pieces), head_decay=a)
        ref = torch.cat([want[i][held[i]:held[i] + pieces[i]] for i in live])
        assert float((out.cpu().double() - ref).abs().max()) <= 3e-5 * max(1.0, float(ref.abs().max())), pieces
        held = [h + p for h, p in zip(held, pieces)]
    assert float((state[2] - 7.0).abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,ff,shared", [(6, 3, 40, 56), (4, 1, 24, None), (5, 5, 16, 32), (8, 2, 64, 64),
                                                   (40, 36, 16, None)])
@pytest.mark.parametrize("tokens", [1, 7, 70, 300])
def test_sigmoid_router_with_weights_on_what_the_expert_reads(dtype, experts, top, ff, shared, tokens):
    """The choice, the weights and the whole feed-forward: both tile sizes, the vendor's grouped product for long
    prompts, one expert and all experts a token, more choices than a warp has lanes."""
    from llm_infer_engine_b200.kernels import ops
    hidden = 64
    params = {"hidden": hidden, "n_experts": experts, "top": top, "expert_ff": ff, "activation": "silu",
              "router_bias": False, "scoring": "sigmoid", "weight_on": "input", "shared_ff": shared}
    part, w = build("feed_forward", "routed_experts", params, dtype, seed=experts + top, std=0.35)
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, hidden, generator=g).to(DTYPES[dtype])
    ctx = make_ctx([tokens], [0], [0], dtype)
    y = part.forward(x.to(DEV), ctx).float().cpu().double()
    wd = {k: v.double() for k, v in w.items()}
    f = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    margins = []
    want = plain.routed_experts(x.double(), f, wd, "", margins)
    clear = margins[0] > 1e-3
    assert int(clear.sum()) >= tokens * 0.8
    assert float((y - want)[clear].abs().max()) <= tol(dtype, float(want.abs().max())) * 2
    # the router alone: ids and weights
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(tokens, top, device=DEV)
    ops.moe_route(x.to(DEV), part.w_router, None, ids, wts, ops.ROUTE_SIGMOID)
    s = torch.sigmoid(x.double() @ wd["router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    assert torch.equal(ids.cpu().long()[clear], idx[clear])
    assert float((wts.cpu().double() - val)[clear].abs().max()) <= 1e-5


def test_weight_on_the_input_is_not_weight_on_the_output():
    """The two readings differ under a non-linear expert, by far more than any bound."""
    g = torch.Generator().manual_seed(3)
    w = {"router": torch.randn(4, 32, generator=g).double()}
    for e in range(4):
        w.update({f"e{e}.gate": torch.randn(16, 32, generator=g).double(), f"e{e}.up": torch.randn(16, 32, generator=g).double(),
                  f"e{e}.down": torch.randn(32, 16, generator=g).double()})
    x = torch.randn(20, 32, generator=g).double()
    f = {"router": {"experts": 4, "top": 2}, "shared": None}
    a = plain.routed_experts(x, f, w, "")
    s = torch.sigmoid(x @ w["router"].T)
    val, idx = torch.topk(s, 2, dim=-1)
    b = torch.stack([sum(val[t, c] * plain.expert(x[t], w, f"e{int(idx[t, c])}.") for c in range(2)) for t in range(20)])
    assert float((a - b).abs().max()) > 0.5


# ------------------------------------------------------------------------------------------ parts alone
def _run_mixer_in_pieces(mixer, cache, dtype, xs, want, schedule, factor=2.0):
    slots = [cache.take_slot() for _ in xs]
    held = [0] * len(xs)
    for pieces in schedule:
        live = [i for i, p in enumerate(pieces) if p > 0]
        for i in live:
            cache.reserve(slots[i], held[i] + pieces[i])
        ctx = make_ctx([pieces[i] for i in live], [held[i] for i in live], [slots[i] for i in live], dtype,
                       kernels=kernel_plan(dtype))
        x = torch.cat([xs[i][held[i]:held[i] + pieces[i]] for i in live])
        y = mixer.forward(x.to(DEV), ctx, cache.unit(0), True).float().cpu().double()
        ref = torch.cat([want[i][held[i]:held[i] + pieces[i]] for i in live])
        assert float((y - ref).abs().max()) <= tol(dtype, float(ref.abs().max())) * factor, (pieces, held)
        for i in live:
            held[i] += pieces[i]
            cache.note_appended(slots[i], held[i], device_updated=False)
    return slots


PIECES = ([100, 30], [39, 2], [1, 1], [1, 1], [0, 34])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("a", 1), ("a", 3), ("b", 3), ("c", 0), ("c", 3)])
def test_attention_with_temperature_and_a_gate_per_head(dtype, tag, layer):
    """Two sequences over prompts in pieces and single tokens, then a slot given back and taken again."""
    from llm_infer_engine_b200.cache import Cache
    cfg = CFGS[tag]
    m = cfg["layers"][layer]["mixer"]
    mixer, w = build("mixer", "gated_attention", {
        "hidden": cfg["width"], "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "v_head_dim": m["vdim"], "scale": m["scale"], "sink": True, "qk_norm_eps": 1e-5, "gate": "head",
        "q_temp": m["q_temp"]}, dtype, seed=layer + 3, std=0.25)
    w["q.norm"] = w["q.norm"] * 4.0
    mixer.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    cache = Cache([mixer.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    cache.take_slot()
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(n, cfg["width"], generator=g).to(DTYPES[dtype]) for n in (141, 68)]
    want = [plain.attention(x.double(), m, wd, "", 1e-5) for x in xs]
    slots = _run_mixer_in_pieces(mixer, cache, dtype, xs, want, PIECES)
    cache.give_back_slot(slots[1])
    xs2 = [torch.randn(70, cfg["width"], generator=g).to(DTYPES[dtype])]
    _run_mixer_in_pieces(mixer, cache, dtype, xs2, [plain.attention(xs2[0].double(), m, wd, "", 1e-5)], ([2], [67], [1]))


def test_the_temperature_changes_where_the_design_says():
    """floor((p + 1) / every): with every = 16 the factor is 1 up to position 14 and changes at 15, 31, ..."""
    t = plain.query_temperature(70, 0.4, 16, torch.float64)
    assert float(t[14]) == 1.0 and float(t[15]) == pytest.approx(1 + 0.4 * 0.6931471805599453)
    assert float(t[30]) == float(t[15]) and float(t[31]) == pytest.approx(1 + 0.4 * 1.0986122886681098)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("a", 2), ("b", 0), ("b", 2), ("b", 4), ("c", 1), ("c", 4)])
def test_latent_attention_with_its_options(dtype, tag, layer):
    """Queries through their own latent, scaled rotation, a window, a learned term in the denominator: prompts in
    pieces, single tokens that carry the window over decoded tokens, a slot used again."""
    from llm_infer_engine_b200.cache import Cache
    cfg = CFGS[tag]
    m = cfg["layers"][layer]["mixer"]
    mixer, w = build("mixer", "latent_attention", {
        "hidden": cfg["width"], "n_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
        "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"],
        "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"], "norm_eps": 1e-5,
        "window": m["mask"]["size"] if m["mask"] else 0, "sink": "learned", "out_float32": True,
        "rot_scaling": m["rot"]["scaling"]}, dtype, seed=layer + 9, std=0.25)
    w["uq"] = w["uq"] * 1.5
    mixer.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    cache = Cache([mixer.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    cache.take_slot()
    g = torch.Generator().manual_seed(12)
    xs = [torch.randn(n, cfg["width"], generator=g).to(DTYPES[dtype]) for n in (141, 68)]
    want = [plain.latent_attention(x.double(), m, wd, "", 1e-5) for x in xs]
    slots = _run_mixer_in_pieces(mixer, cache, dtype, xs, want, PIECES, factor=3.0)
    cache.give_back_slot(slots[0])
    xs2 = [torch.randn(80, cfg["width"], generator=g).to(DTYPES[dtype])]
    _run_mixer_in_pieces(mixer, cache, dtype, xs2, [plain.latent_attention(xs2[0].double(), m, wd, "", 1e-5)],
                         ([2], [67], [1]) + ([1],) * 10, factor=3.0)


def test_scaled_rotation_table_against_the_formula():
    """The table of the part against the plain one, for scalings that blend, that leave all pairs alone and that slow
    all of them down."""
    from llm_infer_engine_b200.parts.latent_attention import rotation_table
    for dims, base, sc in ((8, 10000.0, (8.0, 64, 16.0, 2.0)), (32, 100000.0, (3.0, 128, 16.0, 1.0)),
                           (4, 50.0, (2.0, 16, 4.0, 1.0)), (16, 10000.0, (40.0, 4096, 32.0, 1.0)), (8, 500.0, None)):
        rot = {"dims": dims, "base": base, "scaling": dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None}
        cos, sin = plain.rotary_table(300, rot)
        table = rotation_table(dims, base, 300, "cpu", rot["scaling"])
        assert float((table[..., 0].double() - cos).abs().max()) <= 1e-6
        assert float((table[..., 1].double() - sin).abs().max()) <= 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("a", 0), ("b", 1), ("b", 5), ("c", 2)])
def test_linear_attention_with_a_decay_per_head(dtype, tag, layer):
    """The state carried through pieces (long ones in chunks beside short ones), single tokens, and a slot given back
    and taken again, whose state must start at zero."""
    from llm_infer_engine_b200.cache import Cache
    cfg = CFGS[tag]
    m = cfg["layers"][layer]["mixer"]
    mixer, w = build("mixer", "decayed_linear_attention", {
        "hidden": cfg["width"], "n_heads": m["heads"], "dim": m["dim"], "v_dim": m["vdim"], "decay": m["decay"],
        "norm_eps": 1e-5}, dtype, seed=layer + 1, std=0.25)
    wd = {k: v.double() for k, v in w.items()}
    cache = Cache([mixer.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    cache.take_slot()
    g = torch.Generator().manual_seed(13)
    xs = [torch.randn(n, cfg["width"], generator=g).to(DTYPES[dtype]) for n in (300, 68)]
    want = [plain.lightning(x.double(), m, wd, "", 1e-5) for x in xs]
    slots = _run_mixer_in_pieces(mixer, cache, dtype, xs, want, ([130, 30], [1, 2], [1, 1], [168, 35]))
    cache.give_back_slot(slots[0])
    xs2 = [torch.randn(30, cfg["width"], generator=g).to(DTYPES[dtype])]
    _run_mixer_in_pieces(mixer, cache, dtype, xs2, [plain.lightning(xs2[0].double(), m, wd, "", 1e-5)], ([3], [27]))


# ------------------------------------------------------------------------------------------ the window's edges
def _latent_edge_case(dtype, rank, rot, n_q, window, n, q_len, probe):
    """Attention over latent rows [c | k_rot] that are keys and values at once, with a window and a learned term in the
    denominator: a sequence of n rows of which the last q_len are this step's queries; the LAST query points straight
    at row `probe`, whose latent is a marker (20 in every entry). Slots and pages were given back and taken again
    before, so the sequence's pages are out of order."""
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.parts import AttentionOptions
    row = rank + rot
    cache = Cache([[KVRequest(1, row, window, values_in_keys=rank)]], 4, 64 * 24, 1024, DTYPES[dtype], DEV)
    cache.take_slot()
    other = cache.take_slot()
    cache.reserve(other, 130)
    slot = cache.take_slot()
    cache.reserve(slot, 70)
    cache.give_back_slot(other)
    cache.reserve(slot, n)
    g = torch.Generator().manual_seed(n * 7 + probe)
    k = torch.randn(n, row, generator=g) * 0.1
    q = torch.randn(q_len, n_q, row, generator=g) * 0.1
    k[probe, :rank] = 20.0
    k[probe, rank:] = 3.0
    q[-1] = 0.0
    q[-1, :, rank:] = 3.0                                  # the score comes from the rotated part alone
    k, q = k.to(DTYPES[dtype]), q.to(DTYPES[dtype])
    kv = cache.unit(0).kv
    table = kv.block_table[slot].cpu()
    for j in range(n):
        kv.k[int(table[j // 64]), 0, j % 64] = k[j].to(DEV)
    sinks = torch.linspace(-1.0, 2.0, n_q)
    ctx = make_ctx([q_len], [n - q_len], [slot], dtype, kernels=kernel_plan(dtype))
    out = torch.empty(q_len, n_q * rank, dtype=DTYPES[dtype], device=DEV)
    ctx.attention(q.reshape(q_len, -1).to(DEV), kv, out, n_q, 1, row,
                  AttentionOptions(scale=1.0, window=window, sink_values=sinks.to(DEV)))
    ok = plain.causal_mask(n, window)[n - 1]
    s = (q[-1].double() @ k.double().T).masked_fill(~ok, float("-inf"))           # [n_q, n]
    p = plain.softmax_with_extra(s, sinks.double()[:, None])
    want = (p @ k[:, :rank].double()).reshape(-1)
    return out[-1].float().cpu(), want.float(), bool(ok[probe])


EDGES = [  # window, keys, probe, may the last query (position keys - 1) see it
    (80, 300, 220, True), (80, 300, 219, False),          # just inside and just outside the window
    (64, 257, 193, True), (64, 257, 192, False),          # the window's edge on a page's edge
    (65, 257, 192, True), (65, 257, 191, False),
    (0, 500, 3, True), (0, 700, 0, True),                 # no window: keys far back, the first token
    (1, 40, 39, True), (1, 40, 38, False), (2, 130, 128, True), (2, 130, 127, False),
    (300, 90, 0, True), (128, 129, 1, True), (128, 129, 0, False)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(64, 16, 8), (40, 8, 3), (112, 16, 4), (10, 4, 1)])
@pytest.mark.parametrize("q_len", [1, 2, 37])
def test_latent_rows_at_every_edge_stand_out(dtype, shape, q_len):
    """A probe row that the query may see puts the marker into the output (about 20); one that it may not see leaves
    the output small. Plain kernel (float32, odd sizes) and the tensor-core kernel by rows (bfloat16)."""
    rank, rot, n_q = shape
    for window, n, probe, visible in EDGES:
        if q_len > n:
            continue
        got, want, ok = _latent_edge_case(dtype, rank, rot, n_q, window, n, q_len, probe)
        assert ok == visible
        assert float((got - want).abs().max()) <= (1e-3 if dtype == "float32" else 0.3), (window, n, probe)
        assert (float(got.abs().max()) > 10) == visible, (window, n, probe, float(got.abs().max()))


# ------------------------------------------------------------------------------------------ the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_every_schedule_matches_plain(tag, dtype):
    """Whole prompts; the last tokens one by one (more of them than the longest window); unequal batches in which
    shorter requests end early and the next batch takes their slots, pages and state; prompts in pieces of 2, 7, 64
    and 100 tokens; a prompt in pieces beside sequences that go on by one token."""
    requests = requests_for(tag)
    want = oracle(tag, requests)
    engine = engine_for(tag, dtype)
    plans = {"whole": helpers.plan_whole(requests), "tail": helpers.plan_tail(requests, 120),
             "batched": helpers.plan_batched(requests, 3, 0.6), "mixed": helpers.plan_mixed(requests, 9)}
    some = {rid: toks for rid, toks in requests.items() if len(toks) <= 200}
    for chunk in (2, 7, 64, 100):
        plans[f"pieces of {chunk}"] = helpers.plan_chunked(some if chunk == 2 else requests, chunk)
    for name, steps in plans.items():
        got = helpers.run_plan_engine(engine, steps)
        compare(got, {rid: want[rid] for rid in got}, dtype, f"{tag}/{dtype}/{name}", tag)
        assert engine.cache.free_slots() == engine.cache.n_slots and engine.cache.free_pages() == engine.cache.n_pages
    if dtype == "bfloat16":
        from llm_infer_engine_b200.kernels import ops
        ops.check_tc_status("cuda")


def test_the_models_are_sharp_enough_to_show_what_a_fault_would_change():
    """The bounds above mean something only if a fault moves the logits by more than they allow. In the plain
    implementation: a window one token off, the term in the denominator left out (both kinds), the temperature left
    out, the gate per head left out, the decays a little off, the layer scales left out, alpha off, the rotation's
    scaling left out, and the router's weight on the output instead of the input each differ by several bounds."""
    for tag in ("a", "b", "c"):
        w, cfg = plain_weights(tag), CFGS[tag]
        toks = helpers.random_tokens(cfg["vocab"], max(LENGTHS[tag]), seed=47)
        right = plain.forward(cfg, w, toks)

        def gap(cfg2, w2, factor, what):
            diff = (plain.forward(cfg2, w2, toks) - right).abs().max(dim=1).values
            tol_ = bound("bfloat16", right)
            assert int((diff > tol_).sum()) > max(1, len(diff) // 25) and float(diff.max()) > factor * tol_, (
                tag, what, int((diff > tol_).sum()), float(diff.max()), tol_)

        def changed(fn):
            c = json.loads(json.dumps(cfg))
            for layer in c["layers"]:
                fn(layer)
            return c

        def window_off(layer):
            if layer["type"] == "latent_attention" and layer["mixer"]["mask"]:
                layer["mixer"]["mask"]["size"] += 1

        def no_temperature(layer):
            if layer["type"] == "attention":
                layer["mixer"]["q_temp"] = None

        def no_scaling(layer):
            if layer["type"] == "latent_attention":
                layer["mixer"]["rot"]["scaling"] = None

        def decay_off(layer):
            if layer["type"] == "lightning":
                layer["mixer"]["decay"] = [a * 0.9 for a in layer["mixer"]["decay"]]

        gap(changed(window_off), w, 2, "window")
        gap(changed(no_temperature), w, 2, "temperature")
        gap(changed(decay_off), w, 2, "decay")
        if tag != "b":
            gap(changed(no_scaling), w, 2, "rotation scaling")
        gap(cfg, {k: (v - 30 if k.endswith(".sink") else v) for k, v in w.items()}, 2, "learned sink")
        gap(cfg, {k: (v * 0 + 30 if k.endswith("mix.g") and v.shape[0] < 16 else v) for k, v in w.items()}, 2, "head gate")
        gap(cfg, {k: (v * 0 + 1 if k.endswith((".ls1", ".ls2")) else v) for k, v in w.items()}, 2, "layer scale")
        gap(dict(cfg, postln_alpha=cfg["postln_alpha"] + 1.0), w, 2, "alpha")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_and_cutting_do_not_change_a_row(dtype):
    """The logits of a position do not depend on what else is in the batch or how the prompt was cut: float32
    kernels sum in a fixed order, so there the rows are equal bit for bit."""
    tag = "a"
    requests = requests_for(tag)
    engine = engine_for(tag, dtype)
    alone = helpers.run_plan_engine(engine, helpers.plan_whole(requests))
    together = helpers.run_plan_engine(engine, helpers.plan_batched(requests, 8, 1.0))
    pieces = helpers.run_plan_engine(engine, helpers.plan_chunked(requests, 7))
    for rid in requests:
        if dtype == "float32":
            assert torch.equal(alone[rid], together[rid]), rid
            assert float((alone[rid] - pieces[rid]).abs().max()) <= 0.2 * bound(dtype, alone[rid]), rid
        else:
            # other kernels serve other batch sizes, so roundings differ, and sharp attention carries a difference on
            compare({rid: together[rid]}, {rid: alone[rid]}, dtype, "together against alone")


def test_trace_run_program_and_other_sizes_at_once(tmp_path):
    """bin/trace_run as a subprocess on the configuration with the odd sizes."""
    tag = "b"
    requests = {k: v for k, v in requests_for(tag).items() if len(v) <= 200}
    want = oracle(tag, requests)
    steps = helpers.plan_batched(requests, 4, 0.5)
    peak = max(sum(len(v) for v in requests.values()), 64)
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_trace_run(folder_for(tag), dtype, steps, peak, CFGS[tag]["vocab"])
        compare(got, want, dtype, f"trace_run/{dtype}", tag)


@pytest.mark.parametrize("dtype,gap", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_through_the_library(dtype, gap, graph):
    """generate(): admission, ragged prompts, captured one-token steps (the recurrence, the routed feed-forward's sort
    inside), slots and their state used again. Greedy tokens equal the plain implementation's; where they part the two
    candidates are a near-tie in the plain logits."""
    from llm_infer_engine_b200 import GenerationStats, generate
    tag = "a"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompts = [helpers.random_tokens(cfg["vocab"], n, seed=60 + i) for i, n in enumerate([1, 5, 42, 64, 3, 90, 2])]
    engine = engine_for(tag, dtype, max_batch=3, max_tokens=64 * 12, cuda_graph=graph)
    stats = GenerationStats()
    out = generate(engine, prompts, max_new_tokens=40, stop_ids=[], stats=stats)          # decoding crosses the window
    assert stats.batches >= 3 and [len(o) for o in out] == [40] * len(prompts)
    for p, o in zip(prompts, out):
        seq = list(p)
        for tok in o:
            row = plain.forward(cfg, w, seq)[-1]
            best = int(row.argmax())
            if tok != best:
                assert float(row[best] - row[tok]) < gap, (len(seq), tok, best)
            seq.append(tok)
    engine.cache.check()
    assert engine.cache.free_slots() == 3 and engine.cache.free_pages() == engine.cache.n_pages


def test_long_decoding_in_float32():
    """A few hundred captured one-token steps against one whole-sequence pass: the windows pass over decoded tokens
    many times and the linear attention's states are carried through every step."""
    from llm_infer_engine_b200 import generate
    tag = "b"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 4, seed=70)
    engine = engine_for(tag, "float32", max_batch=2, max_tokens=64 * 12, cuda_graph=True)
    out = generate(engine, [prompt, prompt[:1]], max_new_tokens=260, stop_ids=[])
    for p, o in zip([prompt, prompt[:1]], out):
        seq = p + o
        ref = plain.forward(cfg, w, seq[:-1])
        picks = ref[len(p) - 1:].argmax(-1).tolist()
        for i, (a, b) in enumerate(zip(o, picks)):
            if a != b:
                row = ref[len(p) - 1 + i]
                assert float(row[b] - row[a]) < 1e-4, (i, a, b)
                break


def test_command_line_generates_with_this_design(tmp_path):
    import subprocess
    import sys
    tag = "c"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 9, seed=80)
    proc = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "main.py"), "--model", folder_for(tag),
                           "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32", "--max-new-tokens", "6",
                           "--temperature", "0", "--env-file", str(tmp_path / "none")],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(x) for x in proc.stdout.split("OUTPUT")[1].split("=" * 70)[1].split()]
    seq = list(prompt)
    for tok in ids:
        row = plain.forward(cfg, w, seq)[-1]
        assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 1e-4
        seq.append(tok)
    assert len(ids) == 6
