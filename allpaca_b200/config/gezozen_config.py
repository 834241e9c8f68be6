"""Typed configuration of the Gezozen decoder: a stack of layers that normalise AFTER each sum, whose mixers
are two mixers side by side (softmax attention beside gated linear attention: ``parallel``; softmax attention
behind a sliding window beside retention: ``parallel_2``) or a gated delta rule (``delta``), and whose
feed-forwards are routed experts with a shared expert (or none).

config.json gives every size and constant: ``vocab``, ``width``, ``norm`` ``{eps, groups}``, ``postln_alpha`` and
``layers``, a list of ``{"type", "mixer": {...}, "mlp": {...} | null}``.  One size is not in config.json but in
the tensors' shapes: the inner width of the pair of products that forms the decays of gated linear attention
(``rank``; config.json may name it, and a folder of random weights written from a configuration does).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional, Tuple

from .model_config import ConfigError
from .viresun_config import _float, _int


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]]     # (factor, original, fast, slow)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str, head: int) -> "RotationConfig":
        dims = _int(d, "dims", where, minimum=2)
        if dims % 2 or dims > head:
            raise ConfigError(f"{where}.dims must be even and at most the head's {head}, got {dims}")
        sc = d.get("scaling") or None
        scaling = None
        if sc:
            w = where + ".scaling"
            scaling = (_float(sc, "factor", w), _float(sc, "original", w), _float(sc, "fast", w), _float(sc, "slow", w))
            if not (scaling[0] > 0 and scaling[1] > 0 and scaling[2] > 0 and scaling[3] > 0):
                raise ConfigError(f"{w}: factor, original, fast and slow must be positive")
        base = _float(d, "base", where)
        if not base > 1:
            raise ConfigError(f"{where}.base must exceed 1")
        return cls(base=base, dims=dims, scaling=scaling)


@dataclass(frozen=True)
class SoftmaxSideConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig
    softcap: Optional[float]
    window: Optional[int]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "SoftmaxSideConfig":
        heads = _int(d, "heads", where)
        kv = _int(d, "kv_heads", where) if d.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(d, "dim", where)
        mask = d.get("mask") or None
        cap = d.get("softcap")
        if cap is not None and not _float(d, "softcap", where) > 0:
            raise ConfigError(f"{where}.softcap must be positive")
        return cls(heads=heads, kv_heads=kv, dim=dim,
                   vdim=_int(d, "vdim", where) if d.get("vdim") is not None else dim,
                   scale=_float(d, "scale", where), rot=RotationConfig.from_dict(d.get("rot") or {}, where + ".rot", dim),
                   softcap=float(cap) if cap is not None else None,
                   window=_int(mask, "size", where + ".mask") if mask else None)


@dataclass(frozen=True)
class LinearSideConfig:
    """The recurrent side of a pair: gated linear attention (``tau``, ``rank``) or retention (``decay``, ``rot``)."""
    heads: int
    dim: int
    vdim: int
    tau: Optional[float] = None
    rank: Optional[int] = None
    decay: Optional[Tuple[float, ...]] = None
    rot: Optional[RotationConfig] = None


@dataclass(frozen=True)
class PairMixerConfig:
    left: SoftmaxSideConfig
    right: LinearSideConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "DeltaMixerConfig":
        heads = _int(d, "heads", where)
        kv = _int(d, "kv_heads", where) if d.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(d, "dim", where)
        return cls(heads=heads, kv_heads=kv, dim=dim,
                   vdim=_int(d, "vdim", where) if d.get("vdim") is not None else dim, conv=_int(d, "conv", where))


@dataclass(frozen=True)
class RoutedConfig:
    ff: int
    experts: int
    top: int
    shared_ff: Optional[int]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "RoutedConfig":
        if d.get("kind") != "moe":
            raise ConfigError(f"{where}.kind {d.get('kind')!r} is not known (moe)")
        expert, router, shared = d.get("expert") or {}, d.get("router") or {}, d.get("shared") or None
        out = cls(ff=_int(expert, "ff", where + ".expert"), experts=_int(router, "experts", where + ".router"),
                  top=_int(router, "top", where + ".router"),
                  shared_ff=_int(shared, "ff", where + ".shared") if shared else None)
        if out.top > out.experts:
            raise ConfigError(f"{where}: {out.top} of {out.experts} experts cannot be chosen")
        return out


@dataclass(frozen=True)
class GezozenLayerConfig:
    type: str                    # "parallel" | "parallel_2" | "delta"
    mixer: Any                   # PairMixerConfig | DeltaMixerConfig
    mlp: Optional[RoutedConfig]


def _linear_side(kind: str, d: Mapping[str, Any], where: str, layer: int,
                 shape_of: Optional[Callable[[str], Optional[Tuple[int, ...]]]]) -> LinearSideConfig:
    heads, dim = _int(d, "heads", where), _int(d, "dim", where)
    vdim = _int(d, "vdim", where) if d.get("vdim") is not None else dim
    if kind == "parallel":
        tau = _float(d, "tau", where)
        if not tau > 0:
            raise ConfigError(f"{where}.tau must be positive")
        rank = d.get("rank")
        if rank is None and shape_of is not None:
            shape = shape_of(f"l{layer}.mix.right.a1")
            rank = shape[0] if shape else None
        if rank is None:
            raise ConfigError(f"{where}.rank is neither in the configuration nor to be read off a tensor's shape")
        return LinearSideConfig(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=int(rank))
    decay = d.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(v, (int, float)) for v in decay):
        raise ConfigError(f"{where}.decay must list one number per head")
    return LinearSideConfig(heads=heads, dim=dim, vdim=vdim, decay=tuple(float(v) for v in decay),
                            rot=RotationConfig.from_dict(d.get("rot") or {}, where + ".rot", dim))


@dataclass(frozen=True)
class GezozenConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    norm_groups: int
    alpha: float
    layers: Tuple[GezozenLayerConfig, ...]
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    max_position_embeddings: int = 1 << 17      # the design sets no limit; block tables are made this wide

    #: ``from_dict`` takes ``shape_of`` (tensor name -> shape or None) for the one size the tensors hold
    wants_tensor_shapes = True

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shape_of=None) -> "GezozenConfig":
        norm = d.get("norm") or {}
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("layers must be a list with at least one entry")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind, m = L.get("type"), L.get("mixer") or {}
            if kind in ("parallel", "parallel_2"):
                left = SoftmaxSideConfig.from_dict(m.get("left") or {}, where + ".mixer.left")
                right = _linear_side(kind, m.get("right") or {}, where + ".mixer.right", i, shape_of)
                mixer = PairMixerConfig(left, right, _float(m, "left_scale", where + ".mixer"),
                                        _float(m, "right_scale", where + ".mixer"))
            elif kind == "delta":
                mixer = DeltaMixerConfig.from_dict(m, where + ".mixer")
            else:
                raise ConfigError(f"{where}.type {kind!r} is not known (parallel, parallel_2, delta)")
            mlp = RoutedConfig.from_dict(L["mlp"], where + ".mlp") if L.get("mlp") else None
            layers.append(GezozenLayerConfig(kind, mixer, mlp))
        eps = _float(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("norm.eps must be positive")
        width = _int(d, "width", "config")
        groups = _int(norm, "groups", "norm") if norm.get("groups") is not None else 1
        if width % groups:
            raise ConfigError(f"width {width} does not fall into {groups} equal parts")
        dtype = str(d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16").replace("torch.", "")
        return cls(vocab_size=_int(d, "vocab", "config"), hidden_size=width, norm_eps=eps, norm_groups=groups,
                   alpha=_float(d, "postln_alpha", "config") if d.get("postln_alpha") is not None else 1.0,
                   layers=tuple(layers), torch_dtype=dtype,
                   max_position_embeddings=_int(d, "max_position_embeddings", "config")
                   if d.get("max_position_embeddings") is not None else 1 << 17)
