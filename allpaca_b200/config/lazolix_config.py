"""Typed configuration of the Lazolix decoder: a stack of pre-norm layers whose norms are Dynamic Tanh,
whose mixers (attention through a latent that all heads share, without positions, behind a sliding
window and with a softmax sink) read their input mixed with the previous token's, whose feed-forward is
dense (squared ReLU, with biases), routed (SiLU-gated experts chosen by corrected softmax scores, some of
them identity experts) or absent, and whose outputs are averaged over the depth with learned weights.

config.json gives every size and constant: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list of
``{"type", "mixer": {...}, "mlp": {...} | null}``.  A mixer may say ``kv_from: j``: it has no
down-projection to the latent and reads what layer ``j`` keeps.  What a mechanism may leave out (a
window, identity experts, the feed-forward) is None or 0.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError
from .viresun_config import _float, _int


@dataclass(frozen=True)
class LazolixMixerConfig:
    heads: int
    dim: int                    # query/key dimensions per head
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]       # mask.size
    kv_from: Optional[int]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LazolixMixerConfig":
        dim = _int(d, "dim", where)
        mask = d.get("mask") or None
        return cls(heads=_int(d, "heads", where), dim=dim,
                   vdim=_int(d, "vdim", where) if d.get("vdim") is not None else dim,
                   kv_rank=_int(d, "kv_rank", where), scale=_float(d, "scale", where),
                   window=_int(mask, "size", where + ".mask") if mask and mask.get("size") is not None else None,
                   kv_from=_int(d, "kv_from", where, minimum=0) if d.get("kv_from") is not None else None)


@dataclass(frozen=True)
class LazolixFeedForwardConfig:
    kind: str                   # "dense" | "moe"
    ff: int                     # of the dense layer, or of one expert
    experts: int = 0            # experts that have tensors
    identity: int = 0           # identity experts behind them
    top: int = 0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LazolixFeedForwardConfig":
        kind = d.get("kind", "dense")
        if kind == "dense":
            return cls(kind="dense", ff=_int(d, "ff", where))
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r} is not known (dense, moe)")
        r = d.get("router") or {}
        experts = _int(r, "experts", where + ".router", minimum=0)
        identity = _int(r, "identity", where + ".router", minimum=0) if r.get("identity") is not None else 0
        top = _int(r, "top", where + ".router")
        if top > experts + identity:
            raise ConfigError(f"{where}.router: {top} experts cannot be chosen among {experts} + {identity}")
        return cls(kind="moe", ff=_int(d.get("expert") or {}, "ff", where + ".expert"), experts=experts,
                   identity=identity, top=top)


@dataclass(frozen=True)
class LazolixLayerConfig:
    type: str                                   # "latent_attention"
    mixer: LazolixMixerConfig
    mlp: Optional[LazolixFeedForwardConfig]


@dataclass(frozen=True)
class LazolixConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[LazolixLayerConfig, ...]
    tie_word_embeddings: bool = True            # the logits are products with the embedding table
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 1 << 17      # the design sets no limit; block tables are made this wide

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LazolixConfig":
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a list with at least one entry")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind != "latent_attention":
                raise ConfigError(f"{where}.type {kind!r} is not known (latent_attention)")
            mixer = LazolixMixerConfig.from_dict(L.get("mixer") or {}, where + ".mixer")
            j = mixer.kv_from
            if j is not None:
                if j >= i or layers[j].mixer.kv_from is not None:
                    raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer that has a down-projection "
                                      f"of its own")
                if layers[j].mixer.kv_rank != mixer.kv_rank:
                    raise ConfigError(f"{where} reads what layer {j} keeps, but their kv_rank differ")
            mlp = LazolixFeedForwardConfig.from_dict(L["mlp"], where + ".mlp") if L.get("mlp") else None
            layers.append(LazolixLayerConfig(kind, mixer, mlp))
        eps = _float(d.get("norm") or {}, "eps", "norm")
        if not eps > 0:
            raise ConfigError("norm.eps must be positive")
        dtype = str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16").replace("torch.", "")
        return cls(vocab_size=_int(d, "vocab", "config"), hidden_size=_int(d, "width", "config"), norm_eps=eps,
                   layers=tuple(layers), torch_dtype=dtype,
                   max_position_embeddings=_int(d, "max_position_embeddings", "config")
                   if d.get("max_position_embeddings") is not None else 1 << 17)

    def cache_window(self, i: int) -> Optional[int]:
        """How far back the latents layer ``i`` keeps must stay readable: the largest window among the layer
        and the layers that read its latents (None as soon as one of them has no window)."""
        windows = [self.layers[i].mixer.window] + [L.mixer.window for L in self.layers if L.mixer.kv_from == i]
        return None if any(w is None for w in windows) else max(windows)
