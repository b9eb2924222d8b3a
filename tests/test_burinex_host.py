"""Burinex without a GPU: configuration and the errors that name the key, the spec and its checkpoint names, what each
layer asks of the cache, and the plain mechanisms against hand-made numbers."""
import copy
import math

import pytest
import torch

import plain_burinex as plain

LATENT = {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "q_rank": 12, "scale": 0.3, "mask": {"size": 5},
          "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}}
CFG = {"architecture": "Burinex", "vocab": 50, "width": 24, "postln_alpha": 2.0, "logit_softcap": 10.0,
       "norm": {"eps": 1e-5}, "layers": [
    {"type": "latent_attention", "mixer": LATENT,
     "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 12}, "shared": {"ff": 20}}},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25,
                                    "q_temp": {"coef": 0.5, "every": 4}},
     "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 8}, "shared": None}},
    {"type": "lightning", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "decay": [0.5, 0.9]}, "mlp": None}]}


def test_config_reads_every_layer_and_the_registry_knows_the_name():
    from llm_infer_engine_b200.config import BurinexConfig, load_config
    from llm_infer_engine_b200.config.burinex import GatedAttention, LatentAttention, Lightning
    arch, cfg = load_config(CFG)
    assert arch.name == "Burinex" and isinstance(cfg, BurinexConfig)
    assert (cfg.alpha, cfg.logit_softcap, cfg.norm_eps) == (2.0, 10.0, 1e-5)
    a, b, c = cfg.layers
    assert isinstance(a.mixer, LatentAttention) and a.mixer.window == 5 and a.mixer.q_rank == 12
    assert a.mixer.rot_scaling.factor == 2.0 and a.mixer.rot_scaling.original == 16.0
    assert (a.mlp.experts, a.mlp.top, a.mlp.expert_ff, a.mlp.shared_ff) == (3, 2, 12, 20)
    assert isinstance(b.mixer, GatedAttention) and (b.mixer.temp_coef, b.mixer.temp_every) == (0.5, 4)
    assert b.mlp.shared_ff is None
    assert isinstance(c.mixer, Lightning) and c.mixer.decay == (0.5, 0.9) and c.mlp is None
    free = copy.deepcopy(CFG)
    free["layers"][0]["mixer"]["mask"] = None
    free["layers"][0]["mixer"]["rot"]["scaling"] = None
    free["layers"][1]["mixer"]["q_temp"] = None
    free["logit_softcap"] = None
    cfg2 = load_config(free)[1]
    assert cfg2.layers[0].mixer.window == 0 and cfg2.layers[0].mixer.rot_scaling is None
    assert cfg2.layers[1].mixer.temp_every is None and cfg2.logit_softcap is None
    assert load_config(free)[0].to_spec(cfg2).after_head is None


@pytest.mark.parametrize("path,value,needle", [
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 3, "dims"),
    (("layers", 0, "mixer", "rot", "dims"), 6, "dims"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), None, "factor"),
    (("layers", 0, "mixer", "rot", "scaling", "slow"), 0, "slow"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mlp", "router", "top"), 4, "top"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("layers", 0, "mlp", "shared", "ff"), -1, "ff"),
    (("layers", 1, "mixer", "q_temp", "every"), 0, "every"),
    (("layers", 2, "mixer", "decay"), [0.5], "decay"),
    (("layers", 2, "mixer", "decay"), [0.5, "x"], "decay"),
    (("layers", 2, "type"), "rglru", "type"),
    (("postln_alpha",), None, "postln_alpha"),
    (("logit_softcap",), -1.0, "logit_softcap"),
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
    want = {"embed": (50, 24), "head": (50, 24), "final.norm": (24,), "l0.norm1": (24,), "l0.norm2": (24,),
            "l0.ls1": (24,), "l0.ls2": (24,), "l0.mix.dq": (12, 24), "l0.mix.dq.norm": (12,), "l0.mix.uq": (36, 12),
            "l0.mix.dkv": (14, 24), "l0.mix.dkv.norm": (10,), "l0.mix.uk": (24, 10), "l0.mix.uv": (18, 10),
            "l0.mix.sink": (3,), "l0.mix.o": (24, 18), "l0.mlp.router": (3, 24), "l0.mlp.e2.gate": (12, 24),
            "l0.mlp.e2.down": (24, 12), "l0.mlp.shared.up": (20, 24), "l1.mix.q": (64, 24), "l1.mix.k": (32, 24),
            "l1.mix.v": (16, 24), "l1.mix.q.norm": (64,), "l1.mix.k.norm": (32,), "l1.mix.g": (4, 24),
            "l1.mix.o": (24, 32), "l1.mlp.e1.up": (8, 24), "l2.mix.q": (8, 24), "l2.mix.k": (8, 24),
            "l2.mix.v": (12, 24), "l2.mix.g": (12, 24), "l2.mix.norm": (12,), "l2.mix.o": (24, 12), "l2.norm1": (24,)}
    for name, shape in want.items():
        assert tuple(specs[name].shape) == shape, name
    for absent in ("l2.norm2", "l2.ls2", "l1.mlp.shared.up", "l0.mix.q", "l1.mlp.router.b", "l0.mix.g"):
        assert absent not in specs
    assert len(specs) == 3 + 4 + 9 + 1 + 9 + 3 + 4 + 7 + 1 + 6 + 2 + 6
    reqs = m.unit_requests
    assert reqs[0] == [KVRequest(1, 14, 5, values_in_keys=10)]
    assert reqs[1] == [KVRequest(2, 16, 0, v_head_dim=8)]
    assert reqs[2] == [StateRequest("S", (2, 4, 6))]
    assert [layer.block for layer in m.spec.layers] == ["post_norm_scaled", "post_norm_scaled", "post_norm_scaled_mixer"]


def test_random_weights_mode_writes_what_the_loader_reads(tmp_path):
    from llm_infer_engine_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file
    write_random_model(CFG, str(tmp_path), seed=3)
    stored = load_file(str(tmp_path / "model.safetensors"))
    specs = _model().param_specs()
    assert set(stored) == set(specs)
    assert all(tuple(stored[k].shape) == tuple(specs[k].shape) for k in specs)


def test_plain_softmax_with_one_more_term():
    s = torch.tensor([[0.0, math.log(2.0), float("-inf")]], dtype=torch.float64)
    p = plain.softmax_with_extra(s, torch.tensor(math.log(3.0), dtype=torch.float64))
    assert torch.allclose(p, torch.tensor([[1 / 6, 2 / 6, 0.0]], dtype=torch.float64))
    p0 = plain.softmax_with_extra(s, torch.tensor(0.0, dtype=torch.float64))          # a key of score 0
    assert torch.allclose(p0, torch.tensor([[1 / 4, 2 / 4, 0.0]], dtype=torch.float64))


def test_plain_window_and_temperature():
    ok = plain.causal_mask(6, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True] and ok[1].tolist() == [True, True] + [False] * 4
    assert plain.causal_mask(4)[3].all()
    t = plain.query_temperature(10, 0.5, 4, torch.float64)
    assert t[2] == 1.0 and t[3] == pytest.approx(1 + 0.5 * math.log(2)) and t[7] == pytest.approx(1 + 0.5 * math.log(3))


def test_plain_rotation_blends_frequencies():
    """dims 4, base 100, original 16: where(4) = 4 ln(16 / (8 pi)) / (2 ln 100) < 0 -> lo 0; where(1) = 0.40.. -> hi 1:
    pair 0 keeps its frequency, pair 1 has it divided by the factor; both tables times 0.1 ln(factor) + 1."""
    rot = LATENT["rot"]
    cos, sin = plain.rotary_table(7, rot)
    mag = 0.1 * math.log(2.0) + 1.0
    f = [1.0, 100.0 ** (-0.5) / 2.0]
    for p in (0, 3, 6):
        for i in range(2):
            assert float(cos[p, i]) == pytest.approx(math.cos(p * f[i]) * mag)
            assert float(sin[p, i]) == pytest.approx(math.sin(p * f[i]) * mag)
    x = torch.tensor([[1.0, 0.0, 0.0, 2.0]], dtype=torch.float64).repeat(4, 1)
    y = plain.rotate_pairs(x, cos[:4], sin[:4], 4)
    assert float(y[3, 0]) == pytest.approx(math.cos(3.0) * mag) and float(y[3, 1]) == pytest.approx(math.sin(3.0) * mag)
    assert float(y[3, 2]) == pytest.approx(-2.0 * math.sin(3 * f[1]) * mag)


def test_plain_linear_attention_by_hand():
    """One head, one channel each: S_t = a S + k v; o = S q. With act(z) = silu(z) of unit weights."""
    w = {"q": torch.ones(1, 1, dtype=torch.float64), "k": torch.ones(1, 1, dtype=torch.float64),
         "v": torch.ones(1, 1, dtype=torch.float64), "g": torch.zeros(1, 1, dtype=torch.float64),
         "norm": torch.ones(1, dtype=torch.float64), "o": torch.ones(1, 1, dtype=torch.float64)}
    h = torch.tensor([[1.0], [2.0], [-1.0]], dtype=torch.float64)
    m = {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5]}
    a = [float(plain.silu(x)) for x in h[:, 0]]
    S, reads = 0.0, []
    for x in a:
        S = 0.5 * S + x * x
        reads.append(S * x)
    y = plain.lightning(h, m, w, "", 0.0)
    # one channel: the norm leaves the sign, the gate sigmoid(0) halves
    assert [float(v) for v in y[:, 0]] == pytest.approx([0.5 * math.copysign(1.0, r) for r in reads])


def test_plain_router_scales_what_the_expert_reads():
    g = torch.Generator().manual_seed(1)
    w = {"router": torch.tensor([[5.0, 0.0], [0.0, 5.0], [-5.0, -5.0]], dtype=torch.float64)}
    for e in range(3):
        w.update({f"e{e}.gate": torch.randn(4, 2, generator=g).double(), f"e{e}.up": torch.randn(4, 2, generator=g).double(),
                  f"e{e}.down": torch.randn(2, 4, generator=g).double()})
    x = torch.tensor([[1.0, 0.2]], dtype=torch.float64)
    margins = []
    y = plain.routed_experts(x, {"router": {"experts": 3, "top": 2}, "shared": None}, w, "", margins)
    s0, s1 = 1 / (1 + math.exp(-5.0)), 1 / (1 + math.exp(-1.0))
    want = plain.expert(s0 * x[0], w, "e0.") + plain.expert(s1 * x[0], w, "e1.")
    assert torch.allclose(y[0], want) and float(margins[0][0]) == pytest.approx(1.0 + 6.0)
