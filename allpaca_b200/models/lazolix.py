"""The Lazolix decoder as a :class:`ModelSpec`.

Embedding row; pre-norm layers whose norms are Dynamic Tanh (``tanh(alpha x) w + b``: no mean, no
variance); the mixer reads its normed input mixed with the previous token's normed input (token shift,
a request carries its last normed row from step to step); the mixer is attention through a latent that all heads
share, without any position signal, behind a sliding window, with a learned sink in the softmax's
denominator, possibly reading the latents an earlier layer keeps; the feed-forward is dense (squared
ReLU, biases), routed (SiLU-gated experts; scores are a softmax over all experts, a correction steers the
choice only, the chosen scores are renormalised; the last router outputs may be identity experts) or
absent; after every layer the stream becomes a learned weighted sum of the embedding output and all
layers' results so far.  Final norm; the logits are products with the embedding table.

Tensor names: ``embed``, ``l<i>.norm1`` (with ``.b`` and ``.alpha``), ``l<i>.norm2``, ``l<i>.shift``,
``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.lazolix_config import LazolixConfig
from ..parts import LayerRun, ModelSpec, PartSpec
from .registry import register_architecture


def lazolix_spec(cfg: LazolixConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = PartSpec("dynamic_tanh", {"size": H, "weight_name": "", "bias_name": ".b", "alpha_name": ".alpha"})
    blocks, prefixes, order = [], [], []
    count = len(cfg.layers) + 1                  # the embedding output and every layer's result
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        window = m.window
        cache_window = cfg.cache_window(i if m.kv_from is None else m.kv_from)
        mixer = PartSpec("latent_attention", {
            "hidden_size": H, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": 0, "value_dim": m.vdim,
            "kv_rank": m.kv_rank, "q_rank": 0, "scale": m.scale, "norm_eps": cfg.norm_eps, "rope": None,
            "output_gate": False, "shares_latent": m.kv_from is not None, "window": window,
            "cache_window": cache_window, "sink": True})
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = PartSpec("dense_act", {"hidden_size": H, "intermediate_size": L.mlp.ff, "activation": "relu2",
                                         "bias": True, "names": ("up", "down")})
        elif L.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "hidden_size": H, "expert_size": L.mlp.ff, "experts": L.mlp.experts, "identity": L.mlp.identity,
                "top": L.mlp.top, "activation": "silu", "routing": "softmax_all", "router_bias": True,
                "router_bias_name": "correction"})
        order.append(LayerRun(len(blocks), m.kv_from))      # every layer is one entry of the order, at its own index
        blocks.append(PartSpec("prenorm", {
            "hidden_size": H, "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm,
            "feed_forward_norm": norm if ffn is not None else None,
            "token_shift": PartSpec("token_shift", {"hidden_size": H, "weight_name": ""}),
            "depth_average": PartSpec("depth_average", {"hidden_size": H, "index": i + 1, "count": count,
                                                        "stores_first": i == 0, "weight_name": ""}),
            "mixer_prefix": "mix.", "feed_forward_prefix": "mlp.", "mixer_norm_prefix": "norm1",
            "feed_forward_norm_prefix": "norm2", "token_shift_prefix": "shift", "depth_average_prefix": "dwa"}))
        prefixes.append(f"l{i}.")
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab_size, layers=tuple(blocks), layer_prefixes=tuple(prefixes),
        order=tuple(order), final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        head_name="head", tie_word_embeddings=True, max_position_embeddings=cfg.max_position_embeddings)


register_architecture(("Lazolix", "lazolix"), LazolixConfig, lazolix_spec)
