"""Linear attention in its recurrent form: per head a state ``S`` of ``key_dim x value_dim`` 32-bit numbers
that a request carries from step to step,

    ``S_t = diag(a_t) S_{t-1} + k_t u_t^T``,   ``o_t = S_t^T q_t``,

with what differs between its kinds as parameters:

* the decay ``a_t`` (``decay = {"kind": ...}``): ``"head"``: one fixed number per head (``values``: a list; the
  retention of a head); ``"head_token"``: ``exp(-exp(A_log[h]) * softplus(W_a h + dt_bias[h]))``, one number per
  head and token (tensors ``a``, ``A_log``, ``dt_bias``); ``"channel"``: one number per key channel and token,
  ``sigmoid(z)^(1/tau)`` with ``z = W_a2 (W_a1 h) + b`` through a narrow pair of products (tensors ``a1``, ``a2``,
  ``a2.b``; ``tau``; the pair's inner width is ``rank``);
* ``delta_rule``: the state is corrected towards the value along the key, ``u_t = beta_t (v_t - S^T k_t)`` on
  the state already decayed, ``beta = sigmoid(W_b h)`` (tensor ``b``), and the read-out sees the correction;
  else ``u_t = v_t``;
* ``conv_taps`` ``n > 0``: Q, K and V each pass a causal convolution over the last ``n`` tokens per channel
  (tensors ``q.conv``, ``k.conv``, ``v.conv`` ``[channels, n]``, the last column on the row itself, zeros before
  the sequence's start) and SiLU; the last ``n - 1`` inputs are state too;
* ``qk``: ``"rotate"`` (with ``rope``, a ``position`` part whose ``head_dim`` is the number of rotated
  coordinates) turns queries and keys by the position; ``"unit"`` makes each a unit vector,
  ``x / sqrt(sum x^2 + unit_eps)``; None leaves them;
* ``query_scale`` and ``key_scale`` multiply queries and keys (after rotation or unit norm);
* ``qk_heads``: value head ``h`` reads query/key head ``h // (heads / qk_heads)``;
* every head's read-out is divided by its root mean square (``norm_eps``), multiplied by a weight per coordinate
  that the heads share (``norm_weight``: tensor ``norm``) or by nothing, by ``silu(W_g h)`` and by
  ``output_scale``, then projected out (tensor ``o``).

What enters the recurrence is 32-bit: the stacked projection leaves 32-bit sums; decays, gates of the write,
unit norms, the state and the read-out's norm are computed in 32-bit.  The kernels read only the step's device
tensors; a portion that starts at position 0 starts from zeros.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, LayerCache, Mixer, PartError, WeightSpec, build, register
from .linear import Linear


@register("mixer", "linear_recurrence")
class LinearRecurrence(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``qk_heads`` (``heads``), ``key_dim``, ``value_dim``, ``decay``,
    ``delta_rule`` (False), ``conv_taps`` (0), ``qk`` (None), ``rope``, ``unit_eps`` (1e-6), ``query_scale`` (1),
    ``key_scale`` (1), ``norm_eps``, ``norm_weight`` (True), ``output_scale`` (1); tensors ``q``, ``k``, ``v``,
    ``g``, ``o`` and those the parameters bring."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "heads", "key_dim", "value_dim", "decay", "norm_eps")
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.qk_heads = int(p.get("qk_heads") or self.heads)
        self.D, self.V = int(p["key_dim"]), int(p["value_dim"])
        if self.qk_heads <= 0 or self.heads % self.qk_heads:
            raise PartError(f"{self.heads} heads are not a multiple of {self.qk_heads} query/key heads")
        if not (0 < self.D <= 512 and self.V > 0):
            raise PartError(f"head sizes {self.D}/{self.V} are not ones the kernel takes (keys up to 512)")
        decay = dict(p["decay"])
        self.decay_kind = decay.get("kind")
        if self.decay_kind not in ops.recurrent.DECAY_MODES:
            raise PartError(f"decay kind {self.decay_kind!r} is not known ({', '.join(ops.recurrent.DECAY_MODES)})")
        self.decay_values = None
        self.tau, self.rank = 1.0, 0
        if self.decay_kind == "head":
            self.decay_values = [float(v) for v in decay.get("values") or ()]
            if len(self.decay_values) != self.heads:
                raise PartError(f"{len(self.decay_values)} fixed decays for {self.heads} heads")
        elif self.decay_kind == "channel":
            self.tau, self.rank = float(decay.get("tau", 1.0)), int(decay.get("rank") or 0)
            if not self.tau > 0 or self.rank <= 0:
                raise PartError("a decay per channel needs a positive tau and the rank of its pair of products")
        self.delta_rule = bool(p.get("delta_rule", False))
        self.taps = int(p.get("conv_taps") or 0)
        self.qk = p.get("qk")
        if self.qk not in ops.recurrent.QK_MODES:
            raise PartError(f"qk {self.qk!r} is not known (rotate, unit, None)")
        self.position = None
        if self.qk == "rotate":
            self.require("rope")
            self.position = build("position", p["rope"], env)
            if self.position.head_dim > self.D or self.position.pairing != 0:
                raise PartError(f"a rotation of {self.position.head_dim} coordinates in half-split pairs does not "
                                f"fit heads of {self.D}")
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        # S is linear in k and o in q: both scales meet in one factor on the read-out
        self.read_scale = float(p.get("query_scale", 1.0)) * float(p.get("key_scale", 1.0))
        if self.delta_rule and float(p.get("key_scale", 1.0)) != 1.0:
            raise PartError("the delta rule is not linear in the key: key_scale must be 1")
        self.norm_eps = float(p["norm_eps"])
        self.norm_weight = bool(p.get("norm_weight", True))
        self.output_scale = float(p.get("output_scale", 1.0))
        self.qk_size, self.v_size = self.qk_heads * self.D, self.heads * self.V
        # columns of the stacked projection: q | k | v | g | beta | decay per head
        self.cols = {"q": 0, "k": self.qk_size, "v": 2 * self.qk_size, "g": 2 * self.qk_size + self.v_size}
        total = 2 * self.qk_size + 2 * self.v_size
        if self.delta_rule:
            self.cols["b"] = total
            total += self.heads
        if self.decay_kind == "head_token":
            self.cols["a"] = total
            total += self.heads
        self.in_proj = Linear(env, total, self.hidden)
        self.out_proj = Linear(env, self.hidden, self.v_size)
        self.a1 = self.a2 = None
        if self.decay_kind == "channel":
            self.a1 = Linear(env, self.rank, self.hidden)
            self.a2 = Linear(env, self.heads * self.D, self.rank)
        self.state_floats = self.heads * self.D * self.V
        self.conv_channels = 2 * self.qk_size + self.v_size
        self.conv_floats = max(self.taps - 1, 0) * self.conv_channels
        self.norm_w = self.decay_const = self.dt_bias = self.conv_w = None

    def parts(self):
        yield self
        if self.position is not None:
            yield from self.position.parts()

    def weights(self) -> Dict[str, WeightSpec]:
        H = self.hidden
        w = {"q": WeightSpec((self.qk_size, H)), "k": WeightSpec((self.qk_size, H)),
             "v": WeightSpec((self.v_size, H)), "g": WeightSpec((self.v_size, H)),
             "o": WeightSpec((H, self.v_size))}
        if self.norm_weight:
            w["norm"] = WeightSpec((self.V,), "norm")
        if self.delta_rule:
            w["b"] = WeightSpec((self.heads, H))
        if self.decay_kind == "head_token":
            w.update({"a": WeightSpec((self.heads, H)), "A_log": WeightSpec((self.heads,), "bias"),
                      "dt_bias": WeightSpec((self.heads,), "bias")})
        if self.decay_kind == "channel":
            w.update({"a1": WeightSpec((self.rank, H)), "a2": WeightSpec((self.heads * self.D, self.rank)),
                      "a2.b": WeightSpec((self.heads * self.D,), "bias")})
        if self.taps > 0:
            w.update({"q.conv": WeightSpec((self.qk_size, self.taps), "bias"),
                      "k.conv": WeightSpec((self.qk_size, self.taps), "bias"),
                      "v.conv": WeightSpec((self.v_size, self.taps), "bias")})
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        stacked = [tensors["q"], tensors["k"], tensors["v"], tensors["g"]]
        if self.delta_rule:
            stacked.append(tensors["b"])
        if self.decay_kind == "head_token":
            stacked.append(tensors["a"])
            self.decay_const = tensors["A_log"].float().contiguous()
            self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.in_proj.load(torch.cat(stacked, dim=0))
        self.out_proj.load(tensors["o"])
        if self.decay_kind == "head":
            self.decay_const = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(self.env.device)
        if self.decay_kind == "channel":
            self.a1.load(tensors["a1"])
            self.a2.load(tensors["a2"], tensors["a2.b"].to(tensors["a2"].dtype))
        # what enters the recurrence is 32-bit whatever the engine's type
        self.norm_w = tensors["norm"].float().contiguous() if self.norm_weight else None
        if self.taps > 0:
            self.conv_w = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).float().contiguous()

    def state_bytes(self) -> int:
        return 4 * (self.state_floats + self.conv_floats)

    def forward(self, h: torch.Tensor, step, cache: LayerCache, into=None) -> torch.Tensor:
        """``into`` (optional, 32-bit ``[T, hidden]``): where the output projection leaves its sums, for a mixer
        that runs beside another one."""
        T, S = h.shape[0], step.num_seqs
        ws = self.env.workspace
        if cache.state is None:
            raise PartError("a recurrent mixer needs a state slot per request")
        proj = self.in_proj.forward(h, "linrec.proj", "float32")
        rows = cache.state.view(torch.float32)
        state = rows[:, :self.state_floats].unflatten(1, (self.heads, self.D, self.V))
        c = self.cols
        if self.taps > 0:
            conv_state = rows[:, self.state_floats:self.state_floats + self.conv_floats] \
                .unflatten(1, (self.taps - 1, self.conv_channels)) if self.taps > 1 else None
            qkv = ws.get("linrec.conv", (T, self.conv_channels), torch.float32)
            ops.causal_conv_silu(proj, 0, self.conv_w, None, conv_state, step.token_seq, step.seq_start,
                                 step.positions, step.state_slots, qkv, S)
        else:
            qkv = proj
        q, k = qkv[:, c["q"]:c["q"] + self.qk_size], qkv[:, c["k"]:c["k"] + self.qk_size]
        v = qkv[:, c["v"]:c["v"] + self.v_size]
        decay_channel = None
        if self.decay_kind == "channel":
            narrow = self.a1.forward(h, "linrec.a1", "either")
            decay_channel = self.a2.forward(narrow, "linrec.a2", "float32")
        y = ws.get("linrec.y", (T, self.v_size), torch.float32)
        ops.linear_scan(q, k, v, y, state, step.seq_start, step.positions, step.state_slots, S, self.heads,
                        self.qk_heads, self.D, self.V, self.decay_kind, decay_channel=decay_channel, tau=self.tau,
                        decay_head=proj[:, c["a"]:c["a"] + self.heads] if "a" in c else None,
                        decay_const=self.decay_const, dt_bias=self.dt_bias,
                        beta=proj[:, c["b"]:c["b"] + self.heads] if self.delta_rule else None, qk=self.qk,
                        cos_sin=self.position.rotation_for(step)[0] if self.position is not None else None,
                        unit_eps=self.unit_eps, out_scale=self.read_scale)
        gated = ws.get("linrec.gated", (T, self.v_size), self.env.dtype)
        ops.head_norm_gate(y, proj[:, c["g"]:c["g"] + self.v_size], self.norm_w, self.norm_eps, gated, self.heads,
                           self.V, out_scale=self.output_scale)
        return self.out_proj.forward(gated, "linrec.o", "delta", into=into)


@register("mixer", "mixer_pair")
class MixerPair(Mixer):
    """Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.

    Parameters: ``left``, ``right`` (:class:`PartSpec` of mixers that take ``output_scale`` as a parameter and
    ``into=`` in ``forward``), ``left_scale`` (1), ``right_scale`` (1).  Tensors: the sides' own under ``left.`` and
    ``right.``.  At most one side may keep pages; both may keep fixed-size state (the left one's first in the
    request's slot).  Each side scales its own result where that is free and leaves the sums of its output
    projection in one slice of ``[2, T, hidden]``, which whoever adds into the residual sums up."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("left", "right")
        self.sides = []
        for name in ("left", "right"):
            spec = params[name]
            scaled = dict(spec.params, output_scale=float(params.get(name + "_scale", 1.0)))
            self.sides.append((name + ".", build("mixer", type(spec)(spec.name, scaled), env)))
        if sum(1 for _, m in self.sides if m.cache_need() is not None) > 1:
            raise PartError("only one of two mixers side by side may keep pages")
        self.hidden = int(params.get("hidden_size") or self.sides[0][1].hidden)

    def parts(self):
        yield self
        for _, m in self.sides:
            yield from m.parts()

    def weights(self) -> Dict[str, WeightSpec]:
        return {prefix + n: ws for prefix, m in self.sides for n, ws in m.weights().items()}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, m in self.sides:
            m.load({n[len(prefix):]: t for n, t in tensors.items() if n.startswith(prefix)})

    def cache_need(self):
        for _, m in self.sides:
            if m.cache_need() is not None:
                return m.cache_need()
        return None

    def state_bytes(self) -> int:
        return sum(m.state_bytes() for _, m in self.sides)

    def forward(self, h: torch.Tensor, step, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        delta = self.env.workspace.get("pair.delta", (2, T, self.hidden), torch.float32)
        at = 0
        for i, (_, m) in enumerate(self.sides):
            own = m.state_bytes()
            side = cache
            if cache.state is not None:
                side = dataclasses.replace(cache, state=cache.state[:, at:at + own] if own else None)
            at += own
            m.forward(h, step, side, into=delta[i])
        return delta
