"""Ganupel without a GPU: configuration and the errors that name the key, the spec and its checkpoint names, what each
layer asks of the cache, and the plain mechanisms against hand-made numbers."""
import copy
import math

import pytest
import torch

import plain_ganupel as plain

LEFT = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25, "rot": {"base": 100.0, "dims": 8},
        "mask": {"size": 5}}
CFG = {"architecture": "Ganupel", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "layers": [
    {"type": "parallel", "mixer": {"left": LEFT, "right": {"heads": 3, "dim": 4, "vdim": 6}, "left_scale": 0.5,
                                   "right_scale": 2.0},
     "mlp": {"kind": "moe", "router": {"experts": 3, "identity": 2, "top": 2, "scale": 1.5}, "expert": {"ff": 12}}},
    {"type": "rglru", "mixer": {"width": 12, "blocks": 3, "conv": 3}, "mlp": {"kind": "dense", "ff": 20}},
    {"type": "rglru", "mixer": {"width": 8, "blocks": 1, "conv": 1}, "mlp": None}]}


def test_config_reads_every_layer_and_the_registry_knows_the_name():
    from llm_infer_engine_b200.config import GanupelConfig, load_config
    from llm_infer_engine_b200.config.ganupel import DenseFF, ParallelMixers, RecurrentUnit, RoutedFF
    arch, cfg = load_config(CFG)
    assert arch.name == "Ganupel" and isinstance(cfg, GanupelConfig)
    a, b, c = cfg.layers
    assert isinstance(a.mixer, ParallelMixers) and a.mixer.left.window == 5 and a.mixer.left.rot_dims == 8
    assert a.mixer.right.vdim == 6 and a.mixer.right_scale == 2.0
    assert isinstance(a.mlp, RoutedFF) and (a.mlp.experts, a.mlp.identity, a.mlp.top, a.mlp.scale) == (3, 2, 2, 1.5)
    assert isinstance(b.mixer, RecurrentUnit) and b.mixer.taps == 3 and isinstance(b.mlp, DenseFF) and c.mlp is None
    no_mask = copy.deepcopy(CFG)
    no_mask["layers"][0]["mixer"]["left"]["mask"] = None
    assert load_config(no_mask)[1].layers[0].mixer.left.window == 0


@pytest.mark.parametrize("path,value,needle", [
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "dims"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 18, "dims"),
    (("layers", 0, "mixer", "left_scale"), None, "left_scale"),
    (("layers", 0, "mixer", "right", "vdim"), 0, "vdim"),
    (("layers", 0, "mlp", "router", "top"), 6, "top"),
    (("layers", 0, "mlp", "router", "identity"), -1, "identity"),
    (("layers", 0, "mlp", "kind"), "sparse", "kind"),
    (("layers", 1, "mixer", "blocks"), 5, "blocks"),
    (("layers", 1, "mixer", "conv"), None, "conv"),
    (("layers", 1, "type"), "attention", "type"),
    (("norm", "eps"), "tiny", "eps"),
    (("width",), None, "width")])
def test_config_errors_name_the_key(path, value, needle):
    from llm_infer_engine_b200.config import ConfigError, load_config
    bad = copy.deepcopy(CFG)
    d = bad
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(bad)
    assert needle in str(e.value)


def _model():
    from llm_infer_engine_b200.config import load_config
    from llm_infer_engine_b200.models import DecoderModel
    from llm_infer_engine_b200.parts import Runtime
    arch, cfg = load_config(CFG)
    return DecoderModel(arch.to_spec(cfg), Runtime(torch.device("cpu"), torch.float32, 256))


def test_spec_names_shapes_and_cache_requests():
    from llm_infer_engine_b200.cache import KVRequest, StateRequest
    m = _model()
    specs = m.param_specs()
    want = {"embed": (50, 24), "head": (50, 24), "final.norm": (24,), "l0.norm1": (24,), "l0.ls2": (24,),
            "l0.mix.left.q": (64, 24), "l0.mix.left.k": (32, 24), "l0.mix.left.v": (16, 24), "l0.mix.left.pb": (4,),
            "l0.mix.left.o": (24, 32), "l0.mix.right.q": (12, 24), "l0.mix.right.f.b": (12,),
            "l0.mix.right.lower": (12,), "l0.mix.right.v": (18, 24), "l0.mix.right.norm": (6,),
            "l0.mix.right.o": (24, 18), "l0.mlp.router": (5, 24), "l0.mlp.correction": (5,), "l0.mlp.e2.up": (12, 24),
            "l0.mlp.e2.down": (24, 12), "l1.mix.conv": (12, 3), "l1.mix.ra": (3, 4, 4), "l1.mix.ri.b": (3, 4),
            "l1.mix.lam": (12,), "l1.mlp.act": (4,), "l1.mlp.up": (20, 24), "l2.mix.x.b": (8,), "l2.ls1": (24,)}
    for name, shape in want.items():
        assert tuple(specs[name].shape) == shape, name
    assert not any(n.startswith(("l0.mlp.e3", "l2.mlp", "l2.norm2", "l2.ls2", "l0.mlp.e0.gate")) for n in specs)
    kv, state = m.unit_requests[0]
    assert isinstance(kv, KVRequest) and (kv.name, kv.n_kv_heads, kv.head_dim, kv.value_dim, kv.window) == \
        ("left.kv", 2, 16, 8, 5)
    assert isinstance(state, StateRequest) and (state.name, tuple(state.shape)) == ("right.S", (3, 4, 6))
    assert [(r.name, tuple(r.shape)) for r in m.unit_requests[1]] == [("S", (12,)), ("conv", (2, 12))]
    assert [(r.name, tuple(r.shape)) for r in m.unit_requests[2]] == [("S", (8,)), ("conv", (0, 8))]
    assert [l.block for l in m.spec.layers] == ["pre_norm_scaled", "pre_norm_scaled", "pre_norm_scaled_mixer"]


def test_random_weights_cover_every_tensor():
    from llm_infer_engine_b200.weights.random_init import random_tensors
    tensors, _ = random_tensors(CFG, seed=1, std=0.1, norm_range=None)
    assert set(tensors) == set(_model().param_specs())
    assert float(tensors["l0.mix.right.lower"].float().min()) >= 0 and float(tensors["l0.mix.right.lower"].float().max()) < 1


# ------------------------------------------------------------------------------------------ the plain mechanisms
def test_plain_rotation_pairs_and_leaves_the_rest():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 1, 12) + 1
    y = plain.rotate_half(x.expand(2, 1, 12), torch.tensor([0, 3]), 10.0, 4)
    assert torch.equal(y[0], x[0])                                   # position 0 turns nothing
    a0, a1 = 3 * 1.0, 3 * 10.0 ** -0.5
    assert math.isclose(float(y[1, 0, 0]), 1 * math.cos(a0) - 3 * math.sin(a0), rel_tol=1e-12)
    assert math.isclose(float(y[1, 0, 2]), 3 * math.cos(a0) + 1 * math.sin(a0), rel_tol=1e-12)
    assert math.isclose(float(y[1, 0, 1]), 2 * math.cos(a1) - 4 * math.sin(a1), rel_tol=1e-12)
    assert torch.equal(y[1, 0, 4:], x[0, 0, 4:])


def test_plain_sigmoid_attention_sums_without_normalising():
    """One head whose rotated entries are zero, keys equal: each visible key adds sigmoid(s + b) v."""
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 1, "scale": 0.5, "rot": {"base": 10.0, "dims": 2},
         "mask": {"size": 2}}
    zero = [0.0, 0.0]
    w = {"q": torch.tensor([zero, zero, [0.0, 1.0], zero]).double(), "k": torch.tensor([zero, zero, [0.0, 2.0], zero]).double(),
         "v": torch.tensor([[1.0, 0.0]]).double(), "pb": torch.tensor([-1.0]).double(), "o": torch.eye(1).double()}
    u = torch.tensor([[3.0, 1.0], [5.0, 1.0], [7.0, 1.0]]).double()
    got = plain.sigmoid_attention(u, w, "", m)
    sig = 1 / (1 + math.exp(-(0.5 * 2.0 - 1.0)))                     # every score is q.k * scale = 1 * 2 * 0.5
    assert torch.allclose(got[:, 0], torch.tensor([3 * sig, (3 + 5) * sig, (5 + 7) * sig]).double())


def test_plain_recurrences_by_hand():
    m = {"heads": 1, "dim": 1, "vdim": 2}
    w = {"q": torch.tensor([[1.0]]).double(), "f": torch.tensor([[0.0]]).double(), "f.b": torch.tensor([0.0]).double(),
         "lower": torch.tensor([0.5]).double(), "v": torch.tensor([[1.0], [2.0]]).double(),
         "norm": torch.ones(2).double(), "o": torch.eye(2).double()}
    u = torch.tensor([[1.0], [1.0]]).double()
    got = plain.gated_linear_recurrence(u, w, "", m, 0.0)
    # f = 0.5 + 0.5 * 0.5 = 0.75 ; S1 = 0.25 (1, 2) ; S2 = 0.75 S1 + 0.25 (1, 2); the read is normed, so only its
    # direction (1, 2) / rms is left
    assert torch.allclose(got, torch.tensor([[1.0, 2.0], [1.0, 2.0]]).double() / math.sqrt(2.5))
    conv = plain.causal_conv(torch.tensor([[1.0], [2.0], [4.0]]).double(), torch.tensor([[10.0, 1.0]]).double(),
                             torch.tensor([0.5]).double())
    assert conv.flatten().tolist() == [1.5, 12.5, 24.5]
    z = torch.tensor([[1.0, -2.0, 3.0]]).double()
    pn = plain.poly_norm(z, torch.tensor([1.0, 0.0, 0.0, 0.25]).double(), 0.0)
    assert torch.allclose(pn, z / math.sqrt(14 / 3) + 0.25)


def test_plain_router_chooses_by_corrected_scores_and_weighs_by_plain_ones():
    w = {"router": torch.eye(4).double(), "correction": torch.tensor([0.0, 0.0, 0.0, 10.0]).double()}
    u = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).double()
    chosen, weights = plain.route(u, w, "", {"top": 2, "scale": 3.0})
    s = torch.softmax(u[0], -1)
    assert chosen[0].tolist() == [3, 0]                              # the correction lifts the weakest to the top
    assert torch.allclose(weights[0], torch.stack([s[3], s[0]]) / (s[3] + s[0]) * 3.0)
