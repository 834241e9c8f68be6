"""The Gezozen decoder restated plainly: one function per mechanism, float64, token by token where the
design is a recurrence.  Nothing here is shared with the engine; tests compare the engine against it.

A model is ``(cfg, W)``: ``cfg`` the dictionary of config.json and ``W`` a dictionary of float64 tensors by
checkpoint name.  Every function takes whole sequences ``[T, ...]`` of ONE request, positions ``0 .. T-1``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64
DELTA_UNIT_EPS = 1e-6          # under the root when queries and keys of the delta rule are made unit vectors


def lin(W, name, x, bias=False):
    y = x @ W[name].T
    return y + W[name + ".b"] if bias else y


def silu(z):
    return z * torch.sigmoid(z)


def rms(x, eps):
    """x over its root mean square along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, w, groups, eps):
    """The row cut into ``groups`` equal runs, each over its own root mean square; then the weight."""
    T, n = x.shape
    return (rms(x.reshape(T, groups, n // groups), eps).reshape(T, n)) * w


def rotary_frequencies(rot) -> torch.Tensor:
    """(frequencies [dims/2], magnitude) of a rotation ``{"base", "dims", "scaling"?}``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, n0 = float(sc["factor"]), float(sc["original"])

        def index_of(turns):
            return dims * math.log(n0 / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(index_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=F64), mag


def rotate(x, rot, positions):
    """``x [T, heads, dim]``: the first ``dims`` coordinates of every head turned, coordinate i with i + dims/2."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]              # [T, dims/2]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attend(q, k, v, scale, cap=None, window=None):
    """``q [T, H, D]``, ``k [T, G, D]``, ``v [T, G, V]``: row i over the keys ``j <= i`` (with a window: the last
    ``window`` of them, itself included); scaled scores bounded by ``cap * tanh(score / cap)`` where there is a cap."""
    T, H, _ = q.shape
    G = k.shape[1]
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    seen = dist >= 0
    if window is not None:
        seen = seen & (dist < window)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, -math.inf)
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def softmax_attention(W, p, m, h, eps, biased):
    """The softmax side of a mixer pair.  ``m``: its sizes; ``p``: tensor prefix."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = lin(W, p + "q", h, biased).reshape(T, H, D)
    k = lin(W, p + "k", h, biased).reshape(T, G, D)
    v = lin(W, p + "v", h, biased).reshape(T, G, V)
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    q, k = rotate(q, m["rot"], pos), rotate(k, m["rot"], pos)
    window = int(m["mask"]["size"]) if m.get("mask") else None
    cap = float(m["softcap"]) if m.get("softcap") else None
    out = attend(q, k, v, float(m["scale"]), cap, window)
    return lin(W, p + "o", out.reshape(T, H * V))


def gated_linear_attention(W, p, m, h, eps):
    """Linear attention with a decay per key channel, read off the input through a narrow pair of products."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = lin(W, p + "q", h).reshape(T, H, D) * D ** -0.5
    k = lin(W, p + "k", h).reshape(T, H, D)
    v = lin(W, p + "v", h).reshape(T, H, V)
    z = lin(W, p + "a1", h) @ W[p + "a2"].T + W[p + "a2.b"]
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).reshape(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps) * W[p + "norm"]
    return lin(W, p + "o", o.reshape(T, H * V) * silu(lin(W, p + "g", h)))


def retention(W, p, m, h, eps):
    """Linear attention with one fixed decay per head, rotated queries and keys, nothing dividing the sum."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(T)
    q = rotate(lin(W, p + "q", h).reshape(T, H, D), m["rot"], pos)
    k = rotate(lin(W, p + "k", h).reshape(T, H, D), m["rot"], pos) * D ** -0.5
    v = lin(W, p + "v", h).reshape(T, H, V)
    decay = torch.tensor([float(d) for d in m["decay"]], dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps)
    return lin(W, p + "o", o.reshape(T, H * V) * silu(lin(W, p + "g", h)))


def short_conv(x, w):
    """``x [T, C]``, ``w [C, taps]``: every channel filtered along time, the last tap on the row itself, zeros before
    the start; then SiLU."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return silu(y)


def gated_delta(W, p, m, h, eps):
    """The gated delta rule: the state forgets by one number per head, then is corrected towards the value
    along the key; the read-out sees the correction."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = short_conv(lin(W, p + "q", h), W[p + "q.conv"]).reshape(T, G, D)
    k = short_conv(lin(W, p + "k", h), W[p + "k.conv"]).reshape(T, G, D)
    v = short_conv(lin(W, p + "v", h), W[p + "v.conv"]).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + DELTA_UNIT_EPS) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + DELTA_UNIT_EPS)
    beta = torch.sigmoid(lin(W, p + "b", h))                                       # [T, H]
    forget = torch.exp(-torch.exp(W[p + "A_log"]) * torch.nn.functional.softplus(lin(W, p + "a", h) + W[p + "dt_bias"]))
    S = torch.zeros(H, D, V, dtype=F64)
    o = torch.zeros(T, H, V, dtype=F64)
    rep = H // G
    for t in range(T):
        kt = k[t].repeat_interleave(rep, dim=0)          # [H, D]
        qt = q[t].repeat_interleave(rep, dim=0)
        S = forget[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, qt)
    o = rms(o, eps) * W[p + "norm"]
    return lin(W, p + "o", o.reshape(T, H * V) * silu(lin(W, p + "g", h)))


def expert(W, p, x):
    return lin(W, p + "down", silu(lin(W, p + "gate", x)) * lin(W, p + "up", x))


def routed_feed_forward(W, p, mlp, h):
    """Sigmoid scores, the ``top`` largest chosen, each score multiplying its expert's INPUT; a shared expert
    for every row under a gate of one number per row."""
    T = h.shape[0]
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    s = torch.sigmoid(lin(W, p + "router", h))
    out = torch.zeros_like(h)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            out[t] = out[t] + expert(W, f"{p}e{e}.", (s[t, e] * h[t])[None, :])[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(lin(W, p + "shared.sg", h)) * expert(W, p + "shared.", h)
    return out


def mixer(W, cfg, i, h):
    L = cfg["layers"][i]
    eps = float(cfg["norm"]["eps"])
    p, m = f"l{i}.mix.", L["mixer"]
    if L["type"] == "delta":
        return gated_delta(W, p, m, h, eps)
    biased = L["type"] == "parallel_2"
    left = softmax_attention(W, p + "left.", m["left"], h, eps, biased)
    if L["type"] == "parallel":
        right = gated_linear_attention(W, p + "right.", m["right"], h, eps)
    else:
        right = retention(W, p + "right.", m["right"], h, eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def layer(W, cfg, i, x):
    """Norm after the sum; every sublayer's result under a gate read off the sublayer's input."""
    n, a = cfg["norm"], float(cfg["postln_alpha"])
    eps, groups = float(n["eps"]), int(n["groups"])
    p = f"l{i}."
    gate = torch.sigmoid(lin(W, p + "rg1", x, True))
    x = group_norm(a * x + gate * mixer(W, cfg, i, x), W[p + "norm1"], groups, eps)
    mlp = cfg["layers"][i].get("mlp")
    if mlp is not None:
        gate = torch.sigmoid(lin(W, p + "rg2", x, True))
        x = group_norm(a * x + gate * routed_feed_forward(W, p + "mlp.", mlp, x), W[p + "norm2"], groups, eps)
    return x


def forward(W, cfg, tokens, streams: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one request; ``streams`` (optional) collects the stream after every layer."""
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i in range(len(cfg["layers"])):
        x = layer(W, cfg, i, x)
        if streams is not None:
            streams.append(x)
    n = cfg["norm"]
    return group_norm(x, W["final.norm"], int(n["groups"]), float(n["eps"])) @ W["head"].T


def tensor_shapes(cfg) -> Dict[str, tuple]:
    """Every tensor a model folder of this design holds, with its shape."""
    Wd, vocab = int(cfg["width"]), int(cfg["vocab"])
    out = {"embed": (vocab, Wd), "final.norm": (Wd,), "head": (vocab, Wd)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (Wd,)
        out[p + "rg1"] = (Wd, Wd)
        out[p + "rg1.b"] = (Wd,)
        if L["type"] == "delta":
            H, G, D, V, taps = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                out[p + "mix." + n] = (rows, Wd)
                out[p + "mix." + n + ".conv"] = (rows, taps)
            out.update({p + "mix.b": (H, Wd), p + "mix.a": (H, Wd), p + "mix.A_log": (H,), p + "mix.dt_bias": (H,),
                        p + "mix.norm": (V,), p + "mix.g": (H * V, Wd), p + "mix.o": (Wd, H * V)})
        else:
            l, r = m["left"], m["right"]
            H, G, D, V = (int(l[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            q = p + "mix.left."
            out.update({q + "q": (H * D, Wd), q + "k": (G * D, Wd), q + "v": (G * V, Wd), q + "q.norm": (D,),
                        q + "k.norm": (D,), q + "o": (Wd, H * V)})
            if L["type"] == "parallel_2":
                out.update({q + "q.b": (H * D,), q + "k.b": (G * D,), q + "v.b": (G * V,)})
            H, D, V = (int(r[k]) for k in ("heads", "dim", "vdim"))
            q = p + "mix.right."
            out.update({q + "q": (H * D, Wd), q + "k": (H * D, Wd), q + "v": (H * V, Wd), q + "g": (H * V, Wd),
                        q + "o": (Wd, H * V)})
            if L["type"] == "parallel":
                rank = int(r.get("rank", 16))           # config.json may leave it to the tensors' shapes
                out.update({q + "norm": (V,), q + "a1": (rank, Wd), q + "a2": (H * D, rank), q + "a2.b": (H * D,)})
        mlp = L.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (Wd,)
            out[p + "rg2"] = (Wd, Wd)
            out[p + "rg2.b"] = (Wd,)
            F = int(mlp["expert"]["ff"])
            q = p + "mlp."
            out[q + "router"] = (int(mlp["router"]["experts"]), Wd)
            for e in range(int(mlp["router"]["experts"])):
                out.update({f"{q}e{e}.gate": (F, Wd), f"{q}e{e}.up": (F, Wd), f"{q}e{e}.down": (Wd, F)})
            if mlp.get("shared"):
                F = int(mlp["shared"]["ff"])
                out.update({q + "shared.gate": (F, Wd), q + "shared.up": (F, Wd), q + "shared.down": (Wd, F),
                            q + "shared.sg": (1, Wd)})
    return out


def greedy(W, cfg, prompt, count: int) -> List[int]:
    toks = list(prompt)
    for _ in range(count):
        toks.append(int(forward(W, cfg, toks)[-1].argmax()))
    return toks[len(prompt):]


def random_tensors(cfg, seed: int) -> Dict[str, torch.Tensor]:
    """Weights with which every mechanism shows in the logits: matrices of unit gain, norm weights around 1,
    decays that neither die at once nor stay at 1, gates that are neither shut nor open.  Values are rounded to
    bfloat16, so that a 16-bit checkpoint of them is exact."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.rsplit(".", 1)[-1]
        if tail in ("norm1", "norm2", "norm") and len(shape) == 1:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif tail == "A_log":
            t = torch.log(0.05 + 0.5 * torch.rand(shape, generator=g))
        elif tail == "dt_bias":
            t = torch.randn(shape, generator=g) - 0.5
        elif name.endswith("a2.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif tail == "b" and len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).to(F64)
    return out
