"""The Burinex design as a `ModelSpec`.

x = E[token]; every layer is x = norm1(alpha x + s1 (.) mixer(x)) and, where it has a feed-forward,
x = norm2(alpha x + s2 (.) ff(x)): the RMS norm comes after the residual sum, alpha is one constant of the model and s a
learned scale per channel; logits = cap tanh(head norm(x) / cap). Mixers: "attention" = grouped queries without
rotation, norms over the whole query and key projections, a query temperature that grows with the position, one more
term exp(0) in the softmax's denominator, a sigmoid gate per head; "latent_attention" = queries through a normed latent,
keys and values from a cached normed latent plus one rotated key part shared by the heads (YaRN-scaled rotation), a
sliding window, a learned term per head in the denominator; "lightning" = linear attention with a constant decay per
head, silu on q, k and v, one norm over the concatenated heads, a sigmoid gate per channel. Feed-forward: routed
experts under a sigmoid router (the `top` largest scores choose and weigh, not normalised, and the weight multiplies
what the expert reads) plus a shared expert. Layers are listed one by one in the configuration, each with its own sizes.
Checkpoint names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.ls1`, `l<i>.ls2`, `l<i>.mix.{q,k,v,q.norm,k.norm,g,o}`,
`l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}`, `l<i>.mix.{q,k,v,g,norm,o}`,
`l<i>.mlp.{router,e<j>.{gate,up,down},shared.{gate,up,down}}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.burinex import BurinexConfig, GatedAttention, LatentAttention
from ..config.registry import register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

NO_POSITION_LIMIT = 1 << 20       # the design has no table of positions; the engine's own limit decides


def burinex_spec(cfg: BurinexConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": "", "residual_scale": cfg.alpha})
    scale = PartSpec("layer_scale", {"size": cfg.width})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, GatedAttention):
            mixer = PartSpec("gated_attention", {
                "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "scale": m.scale, "sink": True, "qk_norm_eps": cfg.norm_eps, "gate": "head",
                "q_temp": None if m.temp_every is None else {"coef": m.temp_coef, "every": m.temp_every}})
        elif isinstance(m, LatentAttention):
            s = m.rot_scaling
            mixer = PartSpec("latent_attention", {
                "hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "rot_base": m.rot_base,
                "rot_dims": m.rot_dims, "norm_eps": cfg.norm_eps, "window": m.window, "sink": "learned",
                "out_float32": True,
                "rot_scaling": None if s is None else {"factor": s.factor, "original": s.original, "fast": s.fast,
                                                       "slow": s.slow}})
        else:
            mixer = PartSpec("decayed_linear_attention", {
                "hidden": cfg.width, "n_heads": m.heads, "dim": m.dim, "v_dim": m.vdim, "decay": list(m.decay),
                "activation": "silu", "norm_eps": cfg.norm_eps})
        parts = {"mixer": mixer, "mixer_norm": norm, "mixer_scale": scale}
        names = {"mixer": "mix", "mixer_norm": "norm1", "mixer_scale": "ls1"}
        f = layer.mlp
        if f is not None:
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden": cfg.width, "n_experts": f.experts, "top": f.top, "expert_ff": f.expert_ff,
                "activation": "silu", "router_bias": False, "scoring": "sigmoid", "weight_on": "input",
                "shared_ff": f.shared_ff})
            parts.update(feed_forward_norm=norm, feed_forward_scale=scale)
            names.update(feed_forward="mlp", feed_forward_norm="norm2", feed_forward_scale="ls2")
        layers.append(LayerSpec("post_norm_scaled" if f is not None else "post_norm_scaled_mixer", parts=parts,
                                names=names))
        schedule.append(LayerCall(i))
    final = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT, layers=layers, schedule=schedule,
        final_norm=final, tie_head=False, embedding_name="embed", layer_prefix="l{i}.", final_norm_name="final.norm",
        head_name="head",
        after_head=None if cfg.logit_softcap is None else PartSpec("softcap", {"cap": cfg.logit_softcap}))


register_architecture("Burinex", BurinexConfig, burinex_spec)
