"""Ganupel on the GPU against its plain restatement (tests/plain_ganupel.py): each new kernel and part alone, the
attention's edges with one score made to stand out, state that is carried, freed and taken again, and the engine in
float32 and bfloat16 over whole prompts, token-by-token decoding, prompts in pieces down to two tokens, unequal batches
with slots and pages used again, long decoding and greedy generation through the library's own entry point."""
import json
import os

import pytest
import torch

import helpers
import plain_ganupel as plain
from test_parts_gpu import DEV, DTYPES, build, kernel_plan, make_ctx

pytestmark = pytest.mark.gpu


def _left(heads, kv, dim, vdim, window, scale, base, dims):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": dims},
            "mask": {"size": window} if window else None}


def _moe(experts, identity, top, scale, ff):
    return {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top, "scale": scale},
            "expert": {"ff": ff}}


# A: every layer differs. Value heads narrower and wider than key heads, a rotation over a part of a head and over
# all of it, no mask, as many key heads as query heads, a single recurrent head, a layer without a feed-forward, a
# recurrent unit of one block, a router without identity outputs that takes one expert.
TINY_A = {"architecture": "Ganupel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "layers": [
    {"type": "parallel", "mixer": {"left": _left(6, 3, 32, 16, 24, 0.2, 10000.0, 16),
                                   "right": {"heads": 3, "dim": 20, "vdim": 24}, "left_scale": 0.7, "right_scale": 1.3},
     "mlp": _moe(6, 2, 3, 1.5, 40)},
    {"type": "rglru", "mixer": {"width": 64, "blocks": 4, "conv": 4}, "mlp": {"kind": "dense", "ff": 136}},
    {"type": "parallel", "mixer": {"left": _left(4, 4, 20, 28, 0, 0.3, 300.0, 20),
                                   "right": {"heads": 1, "dim": 8, "vdim": 40}, "left_scale": 1.0, "right_scale": 0.25},
     "mlp": None},
    {"type": "rglru", "mixer": {"width": 120, "blocks": 1, "conv": 2}, "mlp": _moe(4, 0, 1, 1.0, 24)}]}
# B: a width that is no multiple of 8, one key head, a window longer than a page and one of three tokens, a
# convolution of one tap, more identity outputs than experts, recurrent heads whose channels are split over lanes.
TINY_B = {"architecture": "Ganupel", "vocab": 97, "width": 100, "norm": {"eps": 1e-6}, "layers": [
    {"type": "rglru", "mixer": {"width": 100, "blocks": 5, "conv": 1}, "mlp": _moe(3, 5, 4, 2.5, 20)},
    {"type": "parallel", "mixer": {"left": _left(4, 1, 16, 16, 70, 0.25, 500.0, 8),
                                   "right": {"heads": 5, "dim": 12, "vdim": 20}, "left_scale": 0.5, "right_scale": 0.5},
     "mlp": {"kind": "dense", "ff": 60}},
    {"type": "parallel", "mixer": {"left": _left(2, 2, 24, 8, 3, 0.2, 50.0, 24),
                                   "right": {"heads": 2, "dim": 36, "vdim": 8}, "left_scale": 2.0, "right_scale": 1.0},
     "mlp": None}]}
# C: head sizes 64 and 128 with equal value sizes (what the fastest attention kernels take), wide recurrent heads.
TINY_C = {"architecture": "Ganupel", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    {"type": "parallel", "mixer": {"left": _left(4, 2, 64, 64, 100, 0.125, 100000.0, 64),
                                   "right": {"heads": 2, "dim": 64, "vdim": 64}, "left_scale": 0.8, "right_scale": 0.6},
     "mlp": {"kind": "dense", "ff": 256}},
    {"type": "rglru", "mixer": {"width": 256, "blocks": 2, "conv": 4}, "mlp": _moe(4, 4, 3, 2.0, 64)},
    {"type": "parallel", "mixer": {"left": _left(2, 1, 128, 128, 65, 0.09, 100000.0, 32),
                                   "right": {"heads": 4, "dim": 128, "vdim": 32}, "left_scale": 1.0, "right_scale": 1.0},
     "mlp": {"kind": "dense", "ff": 128}}]}
CFGS = {"a": TINY_A, "b": TINY_B, "c": TINY_C}
LENGTHS = {"a": [1, 5, 64, 65, 130, 300], "b": [3, 77, 200, 257], "c": [40, 129, 260]}
SHARPEN = {"a": 4.0, "b": 4.0, "c": 2.5}        # factor on the attention's query and key projections
_folders, _engines = {}, {}


def folder_for(tag):
    """A model folder of random weights: wide embeddings, sharp attention scores under a negative bias (a few keys carry
    nearly all the weight, so one that is lost or added shows), corrections that change the router's choice."""
    from llm_infer_engine_b200.weights.random_init import random_tensors
    from llm_infer_engine_b200.weights.safetensors_io import save_file
    if tag not in _folders:
        d = helpers.scratch_folder(f"llmie_ganupel_{tag}_")
        tensors, _ = random_tensors(CFGS[tag], seed=31 + len(_folders), std=0.09, norm_range=None)
        g = torch.Generator().manual_seed(6)
        for name in tensors:
            t = tensors[name].float()
            if name == "embed":
                t = t * 8.0
            elif name.endswith((".left.q", ".left.k")):
                t = t * SHARPEN[tag]
            elif name.endswith((".o", ".left.v", ".right.v", ".down")):
                t = t * 2.0
            elif name.endswith(".correction"):
                t = torch.randn(t.shape, generator=g) * 0.15
            elif name.endswith(".mlp.act"):
                t = torch.tensor([0.9, -0.6, 0.4, 0.1])
            elif name.endswith(".right.f.b"):
                t = t - 1.5                                          # gates that lean on their lower bound
            elif name.endswith(".mix.lam"):
                t = torch.rand(t.shape, generator=g) * 4 - 7         # long memories: a state that is lost shows
            elif name.endswith(".mix.o") and not name.endswith((".left.o", ".right.o")):
                t = t * 3.0
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


CLOSE_CALL = 0.01          # a router's choice margin below this may fall the other way in bfloat16
_close_calls = {}


def oracle(tag, requests):
    """The plain logits of every request. Beside them it notes, per request, the tokens at which some router of the
    plain model chooses by a margin that bfloat16 rounding can turn (the comparison in bfloat16 holds those tokens
    to the count of positions over the bound, not to the worst-case factor)."""
    w = plain_weights(tag)
    out = {}
    for rid, toks in requests.items():
        margins = []
        out[rid] = plain.forward(w, CFGS[tag], toks, margins_out=margins).float()
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
@pytest.mark.parametrize("size", [200, 202, 204, 2048])
@pytest.mark.parametrize("deltas", [(), ("float32",), ("bfloat16",), ("float32", "float32"), ("bfloat16", "float32")])
def test_scaled_add_and_norm_in_one_kernel(dtype, size, deltas):
    """h += s (.) (c1 d1 + c2 d2) and the norm with a weight stored around zero; all rows, and selected rows alone."""
    from llm_infer_engine_b200.parts import ScaledDelta
    norm, w = build("norm", "rmsnorm", {"size": size, "eps": 1e-5, "weight_name": "", "weight_offset": 1.0}, dtype, seed=2)
    w[""] = (w[""] - 1.0).to(torch.bfloat16).float()              # around zero
    norm.load({"": w[""].to(DEV)})
    g = torch.Generator().manual_seed(size + len(deltas))
    h = torch.randn(9, size, generator=g) * 3
    ds = [(torch.randn(9, size, generator=g).to(DTYPES[d]), c) for d, c in zip(deltas, (0.7, -1.3))]
    s = torch.rand(size, generator=g) + 0.5
    want_h = h.double()
    if ds:
        want_h = want_h + s.double() * sum(c * t.double() for t, c in ds)
    want = plain.norm_around_one(want_h, w[""].double(), 1e-5)
    delta = ScaledDelta([(t.to(DEV), c) for t, c in ds], s.to(DEV)) if ds else None
    hd = h.to(DEV)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    y_rows = norm.forward(hd, delta, rows=rows).float().cpu()
    assert torch.equal(hd.cpu(), h)                                 # selected rows leave the stream alone
    y = norm.forward(hd, delta).float().cpu()
    assert float((hd.cpu().double() - want_h).abs().max()) <= 1e-5
    assert float((y.double() - want).abs().max()) <= tol(dtype, float(want.abs().max()))
    assert float((y_rows.double() - want[[7, 0, 3]]).abs().max()) <= tol(dtype, float(want.abs().max()))
    if ds:
        assert float((delta.materialize().cpu().double() - (want_h - h.double())).abs().max()) <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,n", [(1, 20), (5, 136), (40, 1000), (300, 64), (3, 14000)])
def test_dense_feed_forward_with_normalised_powers(dtype, rows, n):
    ff, w = build("feed_forward", "dense_mlp", {"hidden": 48, "intermediate": n, "bias": False,
                                                "activation": "poly_norm", "norm_eps": 1e-5}, dtype, seed=n, std=0.3)
    w["act"] = torch.tensor([0.75, -0.5, 0.25, 0.125])
    ff.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    x = (torch.randn(rows, 48, generator=torch.Generator().manual_seed(rows)) * 1.5).to(DTYPES[dtype])
    ctx = make_ctx([rows], [0], [0], dtype)
    y = ff.forward(x.to(DEV), ctx).float().cpu().double()
    want = plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}, "", 1e-5)
    assert float((y - want).abs().max()) <= tol(dtype, float(want.abs().max())) * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,identity,top,ff", [(6, 2, 3, 40), (4, 0, 1, 24), (3, 5, 4, 20), (8, 2, 8, 64),
                                                      (40, 0, 36, 16)])
@pytest.mark.parametrize("tokens", [1, 7, 70, 300])
def test_routed_experts_with_identity_outputs(dtype, experts, identity, top, ff, tokens):
    """The router's choice and weights and the whole routed feed-forward: both tile sizes, the vendor's grouped product
    for long prompts, every output chosen, more choices than a warp has lanes, experts that return their input."""
    hidden = 64
    params = {"hidden": hidden, "n_experts": experts, "top": top, "expert_ff": ff, "activation": "relu2", "gated": False,
              "router_bias": False, "scoring": "softmax_all", "weight_scale": 1.75, "identity_experts": identity}
    part, w = build("feed_forward", "routed_experts", params, dtype, seed=experts + top, std=0.35)
    g = torch.Generator().manual_seed(tokens)
    w["correction"] = (torch.randn(experts + identity, generator=g) * 0.2).to(torch.bfloat16).float()
    part.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    x = torch.randn(tokens, hidden, generator=g).to(DTYPES[dtype])
    ctx = make_ctx([tokens], [0], [0], dtype)
    y = part.forward(x.to(DEV), ctx).float().cpu().double()
    f = {"router": {"experts": experts, "identity": identity, "top": top, "scale": 1.75}}
    wd = {k: v.double() for k, v in w.items()}
    want = plain.moe(x.double(), wd, "", f)
    # a near-tie between the last chosen and the first left out may fall the other way in bfloat16 inputs' float32
    # logits: such tokens are left out of the comparison
    s = torch.softmax(x.double() @ wd["router"].T, -1) + wd["correction"]
    top_s = torch.sort(s, -1, descending=True).values
    clear = torch.ones(tokens, dtype=torch.bool) if top == experts + identity else (top_s[:, top - 1] - top_s[:, top]) > 1e-3
    assert int(clear.sum()) >= tokens * 0.8
    assert float((y - want)[clear].abs().max()) <= tol(dtype, float(want.abs().max())) * 2


@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 24), (1, 8, 40), (2, 36, 8), (2, 128, 32), (6, 48, 64), (1, 300, 16)])
def test_matrix_scan_in_pieces_equals_the_plain_loop(heads, dim, vdim):
    """Two sequences in pieces of unequal sizes (and single tokens) through the scan kernel, state in the slots."""
    from llm_infer_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(dim)
    lens = [37, 9]
    q = [torch.randn(n, heads, dim, generator=g) for n in lens]
    f = [torch.rand(n, heads, dim, generator=g) for n in lens]
    v = [torch.randn(n, heads, vdim, generator=g) for n in lens]
    want = []
    for i in range(2):
        S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
        rows = []
        for t in range(lens[i]):
            ft = f[i][t].double()
            S = ft[:, :, None] * S + (1 - ft)[:, :, None] * v[i][t].double()[:, None, :]
            rows.append(torch.einsum("hdv,hd->hv", S, q[i][t].double()).reshape(-1))
        want.append(torch.stack(rows))
    state = torch.zeros(4, heads, dim, vdim, device=DEV)
    state[2] = 7.0                                                  # another sequence's state stays as it is
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEV)
    held = [0, 0]
    for pieces in ([20, 1], [1, 1], [16, 7]):
        cu = torch.tensor([0, pieces[0], sum(pieces)], dtype=torch.int32, device=DEV)
        cat = lambda xs: torch.cat([xs[i][held[i]:held[i] + pieces[i]].reshape(pieces[i], -1) for i in range(2)]).to(DEV)
        out = torch.empty(sum(pieces), heads * vdim, device=DEV)
        ops.matrix_scan(cat(q), cat(f), cat(v), state, cu, slots, out, 2, heads, dim, vdim)
        ref = torch.cat([want[i][held[i]:held[i] + pieces[i]] for i in range(2)])
        assert float((out.cpu().double() - ref).abs().max()) <= 2e-5 * max(1.0, float(ref.abs().max())), pieces
        held = [h + p for h, p in zip(held, pieces)]
    assert float((state[2] - 7.0).abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("heads,dim,vdim", [(2, 20, 24), (3, 64, 64), (1, 130, 40), (2, 48, 136)])
def test_matrix_scan_of_long_pieces_in_chunks(heads, dim, vdim):
    """Pieces long enough for the form that runs chunks side by side: three sequences of unequal lengths (one of them
    a single chunk, one ending exactly at a chunk's end), states handed from piece to piece and to single tokens; some
    gates sit next to 0 and next to 1, where a product of gates over a chunk is smallest and a state lives longest."""
    from llm_infer_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(dim + vdim)
    lens = [701, 322, 135]
    q = [torch.randn(n, heads, dim, generator=g) for n in lens]
    f = [torch.rand(n, heads, dim, generator=g) for n in lens]
    for x in f:
        x[:, :, 0::5] = 1 - x[:, :, 0::5] ** 4 * 0.01              # remembers for hundreds of tokens
        x[:, :, 1::7] = x[:, :, 1::7] ** 4 * 0.01                   # forgets at once
    v = [torch.randn(n, heads, vdim, generator=g) for n in lens]
    want = []
    for i in range(3):
        S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
        rows = []
        for t in range(lens[i]):
            ft = f[i][t].double()
            S = ft[:, :, None] * S + (1 - ft)[:, :, None] * v[i][t].double()[:, None, :]
            rows.append(torch.einsum("hdv,hd->hv", S, q[i][t].double()).reshape(-1))
        want.append(torch.stack(rows))
    state = torch.zeros(5, heads, dim, vdim, device=DEV)
    state[2] = 7.0
    slots = torch.tensor([3, 1, 4], dtype=torch.int32, device=DEV)
    held = [0, 0, 0]
    for pieces in ([300, 192, 5], [1, 1, 1], [400, 129, 129]):
        cu = torch.tensor([0, pieces[0], pieces[0] + pieces[1], sum(pieces)], dtype=torch.int32, device=DEV)
        cat = lambda xs: torch.cat([xs[i][held[i]:held[i] + pieces[i]].reshape(pieces[i], -1) for i in range(3)]).to(DEV)
        out = torch.empty(sum(pieces), heads * vdim, device=DEV)
        ops.matrix_scan(cat(q), cat(f), cat(v), state, cu, slots, out, 3, heads, dim, vdim, max_len=max(pieces))
        ref = torch.cat([want[i][held[i]:held[i] + pieces[i]] for i in range(3)])
        assert float((out.cpu().double() - ref).abs().max()) <= 2e-5 * max(1.0, float(ref.abs().max())), pieces
        held = [h + p for h, p in zip(held, pieces)]
    assert float((state[2] - 7.0).abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0


# ------------------------------------------------------------------------------------------ parts alone
def _run_mixer_in_pieces(mixer, cache, dtype, xs, want, schedule, unit_scope=None):
    slots = [cache.take_slot() for _ in xs]
    held = [0] * len(xs)
    for pieces in schedule:
        live = [i for i, p in enumerate(pieces) if p > 0]
        for i in live:
            cache.reserve(slots[i], held[i] + pieces[i])
        ctx = make_ctx([pieces[i] for i in live], [held[i] for i in live], [slots[i] for i in live], dtype,
                       kernels=kernel_plan(dtype))
        x = torch.cat([xs[i][held[i]:held[i] + pieces[i]] for i in live])
        y = mixer.forward(x.to(DEV), ctx, cache.unit(0), True)
        if hasattr(y, "materialize"):
            y = y.materialize()
        y = y.float().cpu().double()
        ref = torch.cat([want[i][held[i]:held[i] + pieces[i]] for i in live])
        assert float((y - ref).abs().max()) <= tol(dtype, float(ref.abs().max())) * 2, (pieces, held)
        for i in live:
            held[i] += pieces[i]
            cache.note_appended(slots[i], held[i], device_updated=False)
    return slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("a", 0), ("a", 2), ("b", 1), ("b", 2), ("c", 0), ("c", 2)])
def test_two_mixers_side_by_side_in_pieces(dtype, tag, layer):
    """The attention with rotation and sigmoid weights beside the matrix recurrence, as one mixer: two sequences over
    prompts in pieces, single tokens, and a slot that is given back and taken again (its state must start at zero)."""
    from llm_infer_engine_b200.cache import Cache
    from llm_infer_engine_b200.config import PartSpec
    cfg = CFGS[tag]
    m = cfg["layers"][layer]["mixer"]
    a, r = m["left"], m["right"]
    left = PartSpec("gated_attention", {
        "hidden": cfg["width"], "n_heads": a["heads"], "n_kv_heads": a["kv_heads"], "head_dim": a["dim"],
        "v_head_dim": a["vdim"], "scale": a["scale"], "window": a["mask"]["size"] if a["mask"] else 0,
        "weights": "sigmoid", "position": PartSpec("rope", {"rot_dim": a["rot"]["dims"], "theta": a["rot"]["base"],
                                                            "exact_angles": True})})
    right = PartSpec("gated_linear_recurrence", {"hidden": cfg["width"], "n_heads": r["heads"], "dim": r["dim"],
                                                 "v_dim": r["vdim"], "norm_eps": 1e-5})
    mixer, w = build("mixer", "mixer_sum", {"members": {"left": left, "right": right},
                                            "scales": {"left": m["left_scale"], "right": m["right_scale"]}},
                     dtype, seed=layer + 5, std=0.25)
    w["left.pb"] = torch.full_like(w["left.pb"], -2.0)
    w["right.lower"] = (w["right.lower"] - 0.5).clamp(0, 0.95)
    mixer.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    cache = Cache([mixer.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    cache.take_slot()
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(n, cfg["width"], generator=g).to(DTYPES[dtype]) for n in (140, 67)]
    want = [plain.two_mixers(x.double(), wd, "", m, 1e-5) for x in xs]
    slots = _run_mixer_in_pieces(mixer, cache, dtype, xs, want, ([100, 30], [39, 2], [1, 1], [0, 34]))
    cache.give_back_slot(slots[1])
    xs2 = [torch.randn(70, cfg["width"], generator=g).to(DTYPES[dtype])]
    _run_mixer_in_pieces(mixer, cache, dtype, xs2, [plain.two_mixers(xs2[0].double(), wd, "", m, 1e-5)], ([2], [67], [1]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,blocks,taps", [(64, 4, 4), (120, 1, 2), (100, 5, 1), (256, 2, 4), (36, 3, 7)])
def test_recurrent_unit_in_pieces(dtype, width, blocks, taps):
    """Pieces shorter than the convolution's reach, single tokens, and a slot used again."""
    from llm_infer_engine_b200.cache import Cache
    hidden = 72
    mixer, w = build("mixer", "gated_recurrent_unit", {"hidden": hidden, "width": width, "blocks": blocks, "taps": taps,
                                                       "decay": 8.0}, dtype, seed=width, std=0.25)
    g = torch.Generator().manual_seed(width + taps)
    for name in ("y.b", "x.b", "conv.b", "ra.b", "ri.b"):
        w[name] = (torch.randn(w[name].shape, generator=g) * 0.3).to(torch.bfloat16).float()
    w["conv"] = (torch.randn(width, taps, generator=g) * 0.5).to(torch.bfloat16).float()
    w["lam"] = (torch.rand(width, generator=g) * 5 - 5).to(torch.bfloat16).float()      # slow and fast channels
    mixer.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    m = {"width": width, "blocks": blocks, "conv": taps}
    cache = Cache([mixer.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    cache.take_slot()
    xs = [torch.randn(n, hidden, generator=g).to(DTYPES[dtype]) for n in (90, 41)]
    want = [plain.gated_recurrent_unit(x.double(), wd, "", m) for x in xs]
    slots = _run_mixer_in_pieces(mixer, cache, dtype, xs, want, ([1, 2], [2, 1], [50, 1], [1, 1], [36, 36]))
    cache.give_back_slot(slots[0])
    xs2 = [torch.randn(30, hidden, generator=g).to(DTYPES[dtype])]
    _run_mixer_in_pieces(mixer, cache, dtype, xs2, [plain.gated_recurrent_unit(xs2[0].double(), wd, "", m)], ([3], [27]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,blocks,taps", [(64, 4, 4), (100, 5, 3), (40, 1, 1)])
def test_recurrent_unit_over_long_pieces(dtype, width, blocks, taps):
    """Pieces long enough for the form that runs a sequence's chunks side by side, beside short ones in the same step,
    then single tokens and a second long piece that starts from the state the first one left."""
    from llm_infer_engine_b200.cache import Cache
    hidden = 56
    mixer, w = build("mixer", "gated_recurrent_unit", {"hidden": hidden, "width": width, "blocks": blocks, "taps": taps,
                                                       "decay": 8.0}, dtype, seed=width + 1, std=0.25)
    g = torch.Generator().manual_seed(width - taps)
    for name in ("y.b", "x.b", "conv.b", "ra.b", "ri.b"):
        w[name] = (torch.randn(w[name].shape, generator=g) * 0.3).to(torch.bfloat16).float()
    w["conv"] = (torch.randn(width, taps, generator=g) * 0.5).to(torch.bfloat16).float()
    w["lam"] = (torch.rand(width, generator=g) * 9 - 9).to(torch.bfloat16).float()      # some channels keep for long
    mixer.load({k: v.to(DEV, DTYPES[dtype]) for k, v in w.items()})
    wd = {k: v.double() for k, v in w.items()}
    m = {"width": width, "blocks": blocks, "conv": taps}
    cache = Cache([mixer.cache_requests()], 4, 64 * 24, 1024, DTYPES[dtype], DEV)
    cache.take_slot()
    xs = [torch.randn(n, hidden, generator=g).to(DTYPES[dtype]) for n in (520, 180, 40)]
    want = [plain.gated_recurrent_unit(x.double(), wd, "", m) for x in xs]
    _run_mixer_in_pieces(mixer, cache, dtype, xs, want, ([257, 130, 3], [1, 1, 1], [262, 49, 36]))


# ------------------------------------------------------------------------------------------ the attention's edges
def _edge_case(dtype, hd, hdv, n_q, n_kv, window, n, q_len, probe):
    """A sequence of n keys of which the last q_len are this step's queries; the LAST query points straight at key
    `probe`, whose value is a marker (50 in every entry); under a bias of -9 every other key's weight is next to
    nothing. Slots and pages were given back and taken again before, so the sequence's pages are out of order."""
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.parts import AttentionOptions
    cache = Cache([[KVRequest(n_kv, hd, window, v_head_dim=hdv)]], 4, 64 * 24, 1024, DTYPES[dtype], DEV)
    cache.take_slot()
    other = cache.take_slot()
    cache.reserve(other, 130)
    slot = cache.take_slot()
    cache.reserve(slot, 70)
    cache.give_back_slot(other)
    cache.reserve(slot, n)
    g = torch.Generator().manual_seed(n * 7 + probe)
    k = torch.randn(n, n_kv, hd, generator=g) * 0.3
    v = torch.randn(n, n_kv, hdv, generator=g) * 0.1
    q = torch.randn(q_len, n_q, hd, generator=g) * 0.3
    direction = torch.nn.functional.normalize(torch.randn(hd, generator=g), dim=0)
    k[probe] += direction * 8.0
    q[-1] = direction * 8.0
    v[probe] = 50.0
    k, v, q = (t.to(DTYPES[dtype]) for t in (k, v, q))
    kv = cache.unit(0).kv
    table = kv.block_table[slot].cpu()
    for j in range(n):
        kv.k[int(table[j // 64]), :, j % 64] = k[j].to(DEV)
        kv.v[int(table[j // 64]), :, j % 64] = v[j].to(DEV)
    bias = torch.full((n_q,), -9.0)
    ctx = make_ctx([q_len], [n - q_len], [slot], dtype, kernels=kernel_plan(dtype))
    out = torch.empty(q_len, n_q * hdv, dtype=DTYPES[dtype], device=DEV)
    ctx.attention(q.reshape(q_len, -1).to(DEV), kv, out, n_q, n_kv, hd,
                  AttentionOptions(scale=0.5, window=window, sigmoid_bias=bias.to(DEV)))
    ok = plain.window_visible(n, window)[n - 1]
    want = []
    for h in range(n_q):
        kh = k[:, h // (n_q // n_kv)].double()
        a = torch.sigmoid(q[-1, h].double() @ kh.T * 0.5 - 9.0) * ok
        want.append(a @ v[:, h // (n_q // n_kv)].double())
    return out[-1].float().cpu(), torch.cat(want).float(), bool(ok[probe])


EDGES = [  # window, keys, probe, may the last query (position keys - 1) see it
    (80, 300, 220, True), (80, 300, 219, False),          # just inside and just outside the window
    (64, 257, 193, True), (64, 257, 192, False),          # the window's edge on a page's edge
    (65, 257, 192, True), (65, 257, 191, False),
    (0, 500, 3, True), (0, 500, 255, True), (0, 700, 0, True),      # no window: keys far back, the first token
    (1, 40, 39, True), (1, 40, 38, False), (2, 130, 128, True), (2, 130, 127, False),
    (300, 90, 0, True), (128, 129, 1, True), (128, 129, 0, False)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(24, 40, 4, 2), (64, 64, 6, 1), (128, 128, 2, 2), (32, 16, 6, 3)])
@pytest.mark.parametrize("q_len", [1, 2, 37, 200])
def test_keys_at_every_edge_stand_out(dtype, shape, q_len):
    """A probe key that the query may see puts the marker into the output (about 50); one that it may not see leaves
    the output small. Plain kernel (float32, odd sizes) and the tensor-core kernels (bfloat16)."""
    hd, hdv, n_q, n_kv = shape
    for window, n, probe, visible in EDGES:
        if q_len > n:
            continue
        got, want, ok = _edge_case(dtype, hd, hdv, n_q, n_kv, window, n, q_len, probe)
        assert ok == visible
        assert float((got - want).abs().max()) <= (1e-3 if dtype == "float32" else 0.6), (window, n, probe)
        assert (float(got.abs().max()) > 25) == visible, (window, n, probe, float(got.abs().max()))


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
    implementation: a window one token off, the attention's bias left out, the gate's lower bound left out, the
    router's correction left out, the experts that return their input returning nothing, and a recurrent unit that
    forgets (lam pushed up) each differ by several bfloat16 bounds."""
    for tag in ("a", "b", "c"):
        w, cfg = plain_weights(tag), CFGS[tag]
        toks = helpers.random_tokens(cfg["vocab"], max(LENGTHS[tag]), seed=47)
        right = plain.forward(w, cfg, toks)

        def gap(cfg2, w2, factor, what):
            diff = (plain.forward(w2, cfg2, toks) - right).abs().max(dim=1).values
            tol_ = bound("bfloat16", right)
            assert int((diff > tol_).sum()) > max(1, len(diff) // 25) and float(diff.max()) > factor * tol_, (
                tag, what, int((diff > tol_).sum()), float(diff.max()), tol_)

        off = json.loads(json.dumps(cfg))
        for layer in off["layers"]:
            if layer["type"] == "parallel" and layer["mixer"]["left"]["mask"]:
                layer["mixer"]["left"]["mask"]["size"] += 1
        gap(off, w, 2, "window")
        gap(cfg, {k: (v * 0 if k.endswith(".pb") else v) for k, v in w.items()}, 3, "bias")
        gap(cfg, {k: (v * 0 if k.endswith(".lower") else v) for k, v in w.items()}, 2, "lower bound")
        gap(cfg, {k: (v * 0 if k.endswith(".correction") else v) for k, v in w.items()}, 2, "correction")
        gap(cfg, {k: (v + 6 if k.endswith(".lam") else v) for k, v in w.items()}, 2, "decay")
        if any(l["mlp"] and l["mlp"]["kind"] == "moe" and l["mlp"]["router"]["identity"] for l in cfg["layers"]):
            silent = json.loads(json.dumps(cfg))
            w2 = dict(w)
            for i, layer in enumerate(silent["layers"]):
                f = layer["mlp"]
                if f and f["kind"] == "moe" and f["router"]["identity"]:
                    # the identity outputs become experts of their own whose result is zero
                    n, extra = f["router"]["experts"], f["router"]["identity"]
                    for e in range(n, n + extra):
                        w2[f"l{i}.mlp.e{e}.up"] = torch.zeros(1, cfg["width"], dtype=torch.float64)
                        w2[f"l{i}.mlp.e{e}.down"] = torch.zeros(cfg["width"], 1, dtype=torch.float64)
                    f["router"]["experts"], f["router"]["identity"] = n + extra, 0
            gap(silent, w2, 2, "identity")


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
            assert float((alone[rid] - together[rid]).abs().max()) <= bound(dtype, alone[rid])


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
    """generate(): admission, ragged prompts, captured one-token steps (the recurrences, the routed feed-forward's sort
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
            row = plain.forward(w, cfg, seq)[-1]
            best = int(row.argmax())
            if tok != best:
                assert float(row[best] - row[tok]) < gap, (len(seq), tok, best)
            seq.append(tok)
    engine.cache.check()
    assert engine.cache.free_slots() == 3 and engine.cache.free_pages() == engine.cache.n_pages


def test_long_decoding_in_float32():
    """A few hundred captured one-token steps against one whole-sequence pass: the windows pass over decoded tokens
    many times and the recurrent states are carried through every step."""
    from llm_infer_engine_b200 import generate
    tag = "b"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 4, seed=70)
    engine = engine_for(tag, "float32", max_batch=2, max_tokens=64 * 12, cuda_graph=True)
    out = generate(engine, [prompt, prompt[:1]], max_new_tokens=260, stop_ids=[])
    for p, o in zip([prompt, prompt[:1]], out):
        seq = p + o
        ref = plain.forward(w, cfg, seq[:-1])
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
        row = plain.forward(w, cfg, seq)[-1]
        assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 1e-4
        seq.append(tok)
    assert len(ids) == 6
