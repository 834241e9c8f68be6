"""The Gezozen decoder as a :class:`ModelSpec`.

Embedding row; layers that normalise after each sum (``x <- norm(alpha x + gate * sublayer(x))`` with an RMS norm
in groups and a gate per coordinate read off the sublayer's input); per layer a mixer, either two mixers side by
side (softmax attention with normed, partly rotated queries and keys, beside gated linear attention or
retention) or a gated delta rule with short convolutions, and routed experts with sigmoid scores on the experts'
inputs plus a gated shared expert (or no feed-forward); the model's norm and the head.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.rg1`` (+ ``.b``), ``l<i>.rg2``, ``l<i>.mix.*``
(``left.*`` / ``right.*`` for a pair), ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.gezozen_config import GezozenConfig, RotationConfig
from ..parts import LayerRun, ModelSpec, PartSpec
from .registry import register_architecture

DELTA_UNIT_EPS = 1e-6            # under the root where the delta rule makes queries and keys unit vectors


def _rope(rot: RotationConfig) -> PartSpec:
    scaling = None
    if rot.scaling is not None:
        factor, original, fast, slow = rot.scaling
        scaling = {"rope_type": "yarn", "factor": factor, "original": original, "fast": fast, "slow": slow}
    return PartSpec("rope", {"head_dim": rot.dims, "theta": rot.base, "scaling": scaling, "pairing": "half"})


def gezozen_spec(cfg: GezozenConfig) -> ModelSpec:
    H = cfg.hidden_size

    def norm(name: str) -> PartSpec:
        return PartSpec("group_rmsnorm", {"size": H, "eps": cfg.norm_eps, "groups": cfg.norm_groups,
                                          "weight_name": name})
    blocks, prefixes, order = [], [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "delta":
            mixer = PartSpec("linear_recurrence", {
                "hidden_size": H, "heads": m.heads, "qk_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim,
                "decay": {"kind": "head_token"}, "delta_rule": True, "conv_taps": m.conv, "qk": "unit",
                "unit_eps": DELTA_UNIT_EPS, "query_scale": m.dim ** -0.5, "norm_eps": cfg.norm_eps,
                "norm_weight": True})
        else:
            l, r = m.left, m.right
            left = PartSpec("distance_biased_attention", {
                "hidden_size": H, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "head_dim": l.dim,
                "value_dim": l.vdim, "scale": l.scale, "window": l.window, "qk_norm_eps": cfg.norm_eps,
                "qk_norm_weights": True, "distance_bias": False, "rope": _rope(l.rot), "softcap": l.softcap,
                "qkv_bias": L.type == "parallel_2"})
            if L.type == "parallel":
                right = PartSpec("linear_recurrence", {
                    "hidden_size": H, "heads": r.heads, "key_dim": r.dim, "value_dim": r.vdim,
                    "decay": {"kind": "channel", "tau": r.tau, "rank": r.rank}, "query_scale": r.dim ** -0.5,
                    "norm_eps": cfg.norm_eps, "norm_weight": True})
            else:
                right = PartSpec("linear_recurrence", {
                    "hidden_size": H, "heads": r.heads, "key_dim": r.dim, "value_dim": r.vdim,
                    "decay": {"kind": "head", "values": list(r.decay)}, "qk": "rotate", "rope": _rope(r.rot),
                    "key_scale": r.dim ** -0.5, "norm_eps": cfg.norm_eps, "norm_weight": False})
            mixer = PartSpec("mixer_pair", {"hidden_size": H, "left": left, "right": right,
                                            "left_scale": m.left_scale, "right_scale": m.right_scale})
        ffn = None
        if L.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": H, "expert_size": L.mlp.ff, "experts": L.mlp.experts, "top": L.mlp.top,
                "activation": "silu", "routing": "sigmoid", "router_bias": False, "weight_on": "input",
                "shared": {"size": L.mlp.shared_ff, "gate": True} if L.mlp.shared_ff else None})
        blocks.append(PartSpec("gated_postnorm", {
            "hidden_size": H, "alpha": cfg.alpha, "mixer": mixer, "feed_forward": ffn,
            "mixer_norm": norm("norm1"), "feed_forward_norm": norm("norm2") if ffn is not None else None,
            "mixer_gate": PartSpec("residual_gate", {"hidden_size": H, "name": "rg1"}),
            "feed_forward_gate": PartSpec("residual_gate", {"hidden_size": H, "name": "rg2"}) if ffn is not None else None,
            "mixer_prefix": "mix.", "feed_forward_prefix": "mlp.", "mixer_norm_prefix": "",
            "feed_forward_norm_prefix": "", "gate_prefix": ""}))
        prefixes.append(f"l{i}.")
        order.append(LayerRun(i))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(blocks), layer_prefixes=tuple(prefixes),
        order=tuple(order), final_norm=PartSpec("group_rmsnorm", {"size": H, "eps": cfg.norm_eps,
                                                                  "groups": cfg.norm_groups, "weight_name": ""}),
        embedding_name="embed", final_norm_prefix="final.norm", head_name="head",
        tie_word_embeddings=cfg.tie_word_embeddings, max_position_embeddings=cfg.max_position_embeddings)


register_architecture(("Gezozen", "gezozen"), GezozenConfig, gezozen_spec)
