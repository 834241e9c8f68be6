"""A plain, slow implementation of the Lazolix decoder for the tests: one function per mechanism,
whole sequences, torch on the CPU in the precision the caller chooses (float64 by default).
It shares nothing with the engine: it reads a configuration dictionary and tensors by name.

Notation: ``T`` tokens at positions ``0 .. T-1``, ``W`` the width of the residual stream, ``H`` heads.
A weight ``[out, in]`` acts as ``h @ weight.T``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


# ---- small pieces ------------------------------------------------------------------------
def dynamic_tanh(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """A norm without statistics: every entry on its own, ``tanh(alpha x) weight + bias``."""
    return torch.tanh(alpha * x) * weight + bias


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Every last-dimension vector divided by sqrt(mean of its squares + eps), times the weight."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """Row ``t`` moves towards row ``t - 1`` (as it was before any moving; zeros before row 0) by ``mix``."""
    before = torch.zeros_like(h)
    before[1:] = h[:-1]
    return h + (before - h) * mix


def depth_average(results: Sequence[torch.Tensor], a: torch.Tensor) -> torch.Tensor:
    """``sum_j a[j] results[j]`` over the embedding output and every layer's result so far."""
    assert len(results) == a.shape[0]
    out = torch.zeros_like(results[0])
    for j, r in enumerate(results):
        out = out + a[j] * r
    return out


# ---- attention through a shared latent -----------------------------------------------------
def latent_of(h: torch.Tensor, down: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """What a layer with a down-projection keeps per token: the RMS-normed latent ``[T, R]``."""
    return rms_norm(h @ down.T, weight, eps)


def windowed_sink_attention(q: torch.Tensor, latent: torch.Tensor, uk: torch.Tensor, uv: torch.Tensor, sink: torch.Tensor,
                            scale: float, window: Optional[int]) -> torch.Tensor:
    """q ``[T, H, D]``; keys ``uk c`` and values ``uv c`` of every token's latent ``c``, head by head.  Row ``i``
    sees ``j`` with ``0 <= i - j < window``; the denominator of head ``a``'s softmax also holds ``exp(sink[a])``,
    an extra logit that multiplies no value.  Row by row, head by head -> ``[T, H, E]``."""
    T, H, D = q.shape
    E = uv.shape[0] // H
    k = (latent @ uk.T).view(T, H, D)
    v = (latent @ uv.T).view(T, H, E)
    out = torch.zeros(T, H, E, dtype=q.dtype)
    for i in range(T):
        first = 0 if window is None else max(0, i - window + 1)
        for a in range(H):
            scores = (k[first:i + 1, a] @ q[i, a]) * scale
            top = torch.maximum(scores.max(), sink[a])
            e = torch.exp(scores - top)
            weights = e / (e.sum() + torch.exp(sink[a] - top))
            out[i, a] = weights @ v[first:i + 1, a]
    return out


# ---- feed-forwards -------------------------------------------------------------------------------
def dense_feed_forward(h, up, up_b, down, down_b) -> torch.Tensor:
    return (torch.relu(h @ up.T + up_b) ** 2) @ down.T + down_b


def expert(h, gate, up, down) -> torch.Tensor:
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, top: int):
    """(chosen ``[T, top]``, shares ``[T, top]``): scores are a softmax over ALL router outputs; the ``top`` with
    the largest score + correction are chosen; the shares are their scores (without the correction) over
    their sum."""
    scores = torch.softmax(h @ router.T, dim=-1)
    chosen = torch.topk(scores + correction, top, dim=-1).indices
    picked = torch.gather(scores, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def routed_feed_forward(h, w: Dict[str, torch.Tensor], p: str, experts: int, top: int) -> torch.Tensor:
    """Router outputs ``experts ..`` are identity experts: the row itself, times its share."""
    chosen, share = route(h, w[p + "router"], w[p + "correction"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t].tolist(), share[t]):
            y = h[t] if e >= experts else expert(h[t], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
            out[t] = out[t] + s * y
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            results: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of a whole sequence.  ``results`` (optional) receives the stream after every layer."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(list(tokens))]
    kept = [x]                                      # the embedding output, then every layer's result
    latents: Dict[int, torch.Tensor] = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = dynamic_tanh(x, w[p + "norm1"], w[p + "norm1.b"], w[p + "norm1.alpha"])
        h = token_shift(h, w[p + "shift"])
        if m.get("kv_from") is None:
            latents[i] = latent_of(h, w[p + "mix.dkv"], w[p + "mix.dkv.norm"], eps)
        latent = latents[i if m.get("kv_from") is None else m["kv_from"]]
        q = (h @ w[p + "mix.q"].T).view(len(tokens), m["heads"], m["dim"])
        mixed = windowed_sink_attention(q, latent, w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.sink"], m["scale"],
                                        (m.get("mask") or {}).get("size"))
        x = x + mixed.reshape(len(tokens), -1) @ w[p + "mix.o"].T
        mlp = layer.get("mlp")
        if mlp:
            h = dynamic_tanh(x, w[p + "norm2"], w[p + "norm2.b"], w[p + "norm2.alpha"])
            if mlp["kind"] == "dense":
                x = x + dense_feed_forward(h, w[p + "mlp.up"], w[p + "mlp.up.b"], w[p + "mlp.down"], w[p + "mlp.down.b"])
            else:
                x = x + routed_feed_forward(h, w, p + "mlp.", mlp["router"]["experts"], mlp["router"]["top"])
        kept.append(x)
        x = depth_average(kept, w[p + "dwa"])
        if results is not None:
            results.append(x)
    h = dynamic_tanh(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"])
    return h @ w["embed"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], count: int) -> List[int]:
    toks = list(prompt)
    for _ in range(count):
        toks.append(int(forward(config, weights, toks)[-1].argmax()))
    return toks[len(prompt):]


# ---- random weights ------------------------------------------------------------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    s = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "final.norm.alpha": ()}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, D, R = m["heads"], m["dim"], m["kv_rank"]
        E = m.get("vdim", D)
        for n in ("norm1", "norm2") if layer.get("mlp") else ("norm1",):
            s.update({p + n: (W,), p + n + ".b": (W,), p + n + ".alpha": ()})
        s.update({p + "shift": (W,), p + "dwa": (i + 2,), p + "mix.q": (H * D, W), p + "mix.uk": (H * D, R),
                  p + "mix.uv": (H * E, R), p + "mix.sink": (H,), p + "mix.o": (W, H * E)})
        if m.get("kv_from") is None:
            s.update({p + "mix.dkv": (R, W), p + "mix.dkv.norm": (R,)})
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            s.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.up.b": (mlp["ff"],), p + "mlp.down": (W, mlp["ff"]),
                      p + "mlp.down.b": (W,)})
        elif mlp:
            r, F = mlp["router"], mlp["expert"]["ff"]
            outputs = r["experts"] + r.get("identity", 0)
            s.update({p + "mlp.router": (outputs, W), p + "mlp.correction": (outputs,)})
            for e in range(r["experts"]):
                s.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
    return s


def random_tensors(config: dict, seed: int, spread: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights with which every mechanism shows in the logits: matrices of unit gain, norm weights around 1,
    mixing vectors between 0 and 1, depth weights that keep every result alive, sinks and corrections of the
    size of the numbers they sit beside.  Values are rounded to bfloat16, so that a 16-bit checkpoint of them is
    exact."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        tail = name.rsplit(".", 1)[-1]
        if tail == "alpha":
            t = 0.5 + torch.rand(shape, generator=g)
        elif tail in ("norm1", "norm2", "norm") and len(shape) == 1:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif tail == "shift":
            t = torch.rand(shape, generator=g)
        elif tail == "dwa":
            t = (1.0 + 0.5 * torch.randn(shape, generator=g)) / shape[0] ** 0.5
        elif tail == "sink":
            t = torch.randn(shape, generator=g)
        elif tail == "correction":
            t = 0.1 * torch.randn(shape, generator=g)
        elif tail == "b":
            t = 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = spread * torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float64)
    return out
