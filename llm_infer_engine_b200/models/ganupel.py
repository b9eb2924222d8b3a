"""The Ganupel design as a `ModelSpec`.

x = E[token]; every layer is x += s1 (.) mixer(norm(x)) and, where it has a feed-forward, x += s2 (.) ff(norm(x)),
with norms x / sqrt(mean(x^2) + eps) * (1 + w) and learned scales s per channel; logits = head norm(x). Mixers:
"parallel" = an attention (grouped queries, rotate-half rotation of the first `rot.dims` entries of each head, a
sliding window, weights sigmoid(score + a number per head) without any normalisation over the keys) beside a gated
linear recurrence over a matrix state per head, added with a constant each; "rglru" = a real-gated linear recurrent unit
behind a short causal convolution. Feed-forwards: down(PolyNorm(up x)), or routed experts down(relu(up x)^2) under a
router that scores with a softmax over all its outputs, chooses by score + correction, and has outputs that stand
for experts returning their input. Layers are listed one by one in the configuration, each with its own sizes.
Checkpoint names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.ls1`, `l<i>.ls2`,
`l<i>.mix.left.{q,k,v,pb,o}`, `l<i>.mix.right.{q,f,f.b,lower,v,norm,o}`,
`l<i>.mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o}`, `l<i>.mlp.{up,down,act}` or
`l<i>.mlp.{router,correction,e<j>.{up,down}}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.ganupel import DenseFF, GanupelConfig, ParallelMixers
from ..config.registry import register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

NO_POSITION_LIMIT = 1 << 20       # the design has no table of positions; the engine's own limit decides
DECAY_CONSTANT = 8.0              # the recurrent unit's a = exp(-8 r softplus(lam))


def ganupel_spec(cfg: GanupelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": "", "weight_offset": 1.0})
    scale = PartSpec("layer_scale", {"size": cfg.width})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, ParallelMixers):
            a, r = m.left, m.right
            left = PartSpec("gated_attention", {
                "hidden": cfg.width, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim,
                "v_head_dim": a.vdim, "scale": a.scale, "window": a.window, "weights": "sigmoid",
                "position": PartSpec("rope", {"rot_dim": a.rot_dims, "theta": a.rot_base, "exact_angles": True})})
            right = PartSpec("gated_linear_recurrence", {"hidden": cfg.width, "n_heads": r.heads, "dim": r.dim,
                                                         "v_dim": r.vdim, "norm_eps": cfg.norm_eps})
            mixer = PartSpec("mixer_sum", {"members": {"left": left, "right": right},
                                           "scales": {"left": m.left_scale, "right": m.right_scale}})
        else:
            mixer = PartSpec("gated_recurrent_unit", {"hidden": cfg.width, "width": m.width, "blocks": m.blocks,
                                                      "taps": m.taps, "decay": DECAY_CONSTANT,
                                                      "activation": "gelu_tanh"})
        parts = {"mixer": mixer, "mixer_norm": norm, "mixer_scale": scale}
        names = {"mixer": "mix", "mixer_norm": "norm1", "mixer_scale": "ls1"}
        f = layer.mlp
        if f is not None:
            if isinstance(f, DenseFF):
                parts["feed_forward"] = PartSpec("dense_mlp", {"hidden": cfg.width, "intermediate": f.ff, "bias": False,
                                                               "activation": "poly_norm", "norm_eps": cfg.norm_eps})
            else:
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden": cfg.width, "n_experts": f.experts, "top": f.top, "expert_ff": f.expert_ff,
                    "activation": "relu2", "gated": False, "router_bias": False, "scoring": "softmax_all",
                    "weight_scale": f.scale, "identity_experts": f.identity})
            parts.update(feed_forward_norm=norm, feed_forward_scale=scale)
            names.update(feed_forward="mlp", feed_forward_norm="norm2", feed_forward_scale="ls2")
        layers.append(LayerSpec("pre_norm_scaled" if f is not None else "pre_norm_scaled_mixer", parts=parts, names=names))
        schedule.append(LayerCall(i))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT, layers=layers, schedule=schedule,
        final_norm=norm, tie_head=False, embedding_name="embed", layer_prefix="l{i}.", final_norm_name="final.norm",
        head_name="head")


register_architecture("Ganupel", GanupelConfig, ganupel_spec)
