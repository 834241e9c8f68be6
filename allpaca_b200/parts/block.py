"""The pre-norm arrangement of a decoder layer.

``x -> norm -> mixer -> +x -> norm -> feed-forward -> +x``
(crates/allpaca-core/src/model.rs:8447-8696).  The residual ``x`` is 32-bit; each addition
is performed inside the norm that follows it, which reads the pending partial sums, so the
block hands its last addition to whoever runs next.
"""
from __future__ import annotations

import dataclasses
from typing import Dict

import torch

from .. import ops
from .base import Block, BuildEnv, Deferred, LayerCache, Part, PartError, build, register
from .norm import RMSNorm


@register("block", "prenorm")
class PreNormBlock(Block):
    """Parameters: ``hidden_size`` and four :class:`PartSpec`: ``mixer``, ``feed_forward``,
    ``mixer_norm``, ``feed_forward_norm`` (``feed_forward`` None: the layer is its mixer alone);
    and the weight-name prefixes ``mixer_prefix``,
    ``feed_forward_prefix``, ``mixer_norm_prefix``, ``feed_forward_norm_prefix``.

    Two optional parts of kind ``stream`` (with ``token_shift_prefix`` / ``depth_average_prefix``):
    ``token_shift``: the mixer reads its normed input mixed with the previous token's (the norm before the
    mixer must offer ``forward_shifted``; the previous row is kept in the request's state slot, behind the
    mixer's own state); ``depth_average``: what leaves the layer is a weighted sum of the results of all
    layers so far, and nothing is left pending for the next block."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "mixer", "mixer_norm")
        self.hidden = int(params["hidden_size"])
        self.mixer = build("mixer", params["mixer"], env)
        self.mixer_norm = build("norm", params["mixer_norm"], env)
        self._prefixes = {
            params.get("mixer_prefix", "mixer."): self.mixer,
            params.get("mixer_norm_prefix", "mixer_norm."): self.mixer_norm,
        }
        # a layer may have no feed-forward (``feed_forward`` None): then it has no second norm either
        self.feed_forward = self.feed_forward_norm = None
        if params.get("feed_forward") is not None:
            self.require("feed_forward_norm")
            self.feed_forward = build("feed_forward", params["feed_forward"], env)
            self.feed_forward_norm = build("norm", params["feed_forward_norm"], env)
            self._prefixes[params.get("feed_forward_prefix", "feed_forward.")] = self.feed_forward
            self._prefixes[params.get("feed_forward_norm_prefix", "feed_forward_norm.")] = self.feed_forward_norm
        self.token_shift = self.depth_average = None
        if params.get("token_shift") is not None:
            if not hasattr(self.mixer_norm, "forward_shifted"):
                raise PartError(f"the norm {params['mixer_norm'].name!r} cannot mix a row with the one before it")
            self.token_shift = build("stream", params["token_shift"], env)
            self._prefixes[params.get("token_shift_prefix", "token_shift.")] = self.token_shift
        if params.get("depth_average") is not None:
            self.depth_average = build("stream", params["depth_average"], env)
            self._prefixes[params.get("depth_average_prefix", "depth_average.")] = self.depth_average
        self.fused = False

    def sub_parts(self) -> Dict[str, Part]:
        return dict(self._prefixes)

    def state_bytes(self) -> int:
        return self.mixer.state_bytes() + (self.token_shift.state_bytes() if self.token_shift is not None else 0)

    def finalize(self) -> None:
        """In bfloat16, where both norms are RMSNorm and mixer and feed-forward can take it: the
        norms' weights are multiplied into the products that follow them.  A step of few rows then
        runs without norm kernels (the products scale their result rows by the root mean square,
        which the product before them summed up while it added into the residual); a step of many
        rows runs the norm kernels as before, without their weights."""
        if self.env.dtype != torch.bfloat16 or self.feed_forward is None:
            return
        if self.token_shift is not None or self.depth_average is not None:
            return
        if not (type(self.mixer_norm) is RMSNorm and type(self.feed_forward_norm) is RMSNorm):
            return
        if self.mixer_norm.folded or self.feed_forward_norm.folded:
            return                      # done before (weights are folded once per load)
        self.fused = False
        can = [getattr(part, "can_fold_input_norm", lambda: False)() for part in (self.mixer, self.feed_forward)]
        if not all(can):
            return
        self.mixer.fold_input_norm(self.mixer_norm.weight)
        self.feed_forward.fold_input_norm(self.feed_forward_norm.weight)
        self.mixer_norm.fold()
        self.feed_forward_norm.fold()
        self.fused = True

    def forward(self, x: torch.Tensor, delta, step, cache: LayerCache):
        T = x.shape[0]
        h = self.env.workspace.get("block.normed", (T, self.hidden), self.env.dtype)
        if self.fused and self.mixer.fused_rows_ok(T) and self.feed_forward.fused_rows_ok(T):
            if isinstance(delta, Deferred):
                inp, scale = delta.xb, ops.RowScale(delta.ss, delta.parts, self.hidden, self.mixer_norm.eps)
            else:
                self.mixer_norm.forward(x, h, delta=delta)
                inp, scale = h, None
            d = self.mixer.forward_fused(inp, scale, x, step, cache)
            scale = ops.RowScale(d.ss, d.parts, self.hidden, self.feed_forward_norm.eps)
            return self.feed_forward.forward_fused(d.xb, scale, x, step)
        if isinstance(delta, Deferred):
            delta = None                 # the block before has added into the residual itself
        if self.token_shift is not None or (self.depth_average is not None and self.depth_average.stores_first):
            if delta is not None:
                ops.residual_add(x, delta)       # both read the stream as it is, with nothing pending
                delta = None
        if self.depth_average is not None:
            self.depth_average.begin(x)
        if self.token_shift is not None:
            own = self.mixer.state_bytes()
            if cache.state is None:
                raise PartError("a block that mixes rows with the previous token's needs a state slot per request")
            previous = cache.state[:, own:own + self.token_shift.state_bytes()].view(torch.float32)
            if own > 0:
                cache = dataclasses.replace(cache, state=cache.state[:, :own])
            self.mixer_norm.forward_shifted(x, h, self.token_shift.weight, previous, step)
        else:
            self.mixer_norm.forward(x, h, delta=delta)
        delta = self.mixer.forward(h, step, cache)
        if self.feed_forward is not None:
            self.feed_forward_norm.forward(x, h, delta=delta)
            delta = self.feed_forward.forward(h, step)
        if self.depth_average is not None:
            self.depth_average.finish(x, delta)
            return None
        return delta


@register("block", "output_norm")
class OutputNormBlock(Block):
    """A layer whose norms act on what its sublayers PRODUCE, not on what they read:

    ``x <- x + m * norm1(mixer(x))``, then ``x <- x + m * norm2(feed_forward(x))``

    with one number ``m`` (``residual_mult``) for the whole layer.  Both sublayers read the
    residual stream itself (rounded to the activation type in bfloat16, as it is in 32-bit).  The
    norm, the scaling and the addition are one kernel, which also leaves the updated stream's copy
    in the activation type for the sublayer that reads it next; nothing is left pending for the
    block that follows.

    Parameters: ``hidden_size``, ``mixer``, ``feed_forward`` (None: the mixer alone), ``mixer_norm``,
    ``feed_forward_norm``, ``residual_mult`` (1.0) and the weight-name prefixes of :class:`PreNormBlock`."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "mixer", "mixer_norm")
        self.hidden = int(params["hidden_size"])
        self.mult = float(params.get("residual_mult", 1.0))
        self.mixer = build("mixer", params["mixer"], env)
        self.mixer_norm = build("norm", params["mixer_norm"], env)
        self._prefixes = {
            params.get("mixer_prefix", "mixer."): self.mixer,
            params.get("mixer_norm_prefix", "mixer_norm."): self.mixer_norm,
        }
        self.feed_forward = self.feed_forward_norm = None
        if params.get("feed_forward") is not None:
            self.require("feed_forward_norm")
            self.feed_forward = build("feed_forward", params["feed_forward"], env)
            self.feed_forward_norm = build("norm", params["feed_forward_norm"], env)
            self._prefixes[params.get("feed_forward_prefix", "feed_forward.")] = self.feed_forward
            self._prefixes[params.get("feed_forward_norm_prefix", "feed_forward_norm.")] = self.feed_forward_norm

    def sub_parts(self) -> Dict[str, Part]:
        return dict(self._prefixes)

    def forward(self, x: torch.Tensor, delta, step, cache: LayerCache):
        T = x.shape[0]
        if delta is not None and not isinstance(delta, Deferred):
            ops.residual_add(x, delta)           # what a block of another arrangement left pending
        if self.env.dtype == torch.float32:
            h = copy = None                      # the sublayers read the stream itself
        else:
            # the stream's copy in the activation type: left by the block before where that is one of this
            # kind (it was the last thing written into the buffer), else made now
            h = copy = self.env.workspace.get("block.stream_copy", (T, self.hidden), self.env.dtype)
            if step.shared.get("block.stream_copy") is not x:
                self.mixer_norm.add_normed(x, None, self.mult, copy)
        delta = self.mixer.forward(x if h is None else h, step, cache)
        self.mixer_norm.add_normed(x, delta, self.mult, copy)
        if self.feed_forward is not None:
            delta = self.feed_forward.forward(x if h is None else h, step)
            self.feed_forward_norm.add_normed(x, delta, self.mult, copy)
        step.shared["block.stream_copy"] = x     # the copy is up to date with this residual
        return None


@register("block", "gated_postnorm")
class GatedPostNormBlock(Block):
    """A layer that normalises the stream AFTER each sum, with the sublayer's result under a gate:

    ``x <- norm1(alpha * x + sigmoid(W_1 x + b_1) * mixer(x))``, then
    ``x <- norm2(alpha * x + sigmoid(W_2 x + b_2) * feed_forward(x))``.

    Both sublayers and both gates read the stream itself (rounded to the activation type in bfloat16, as it is in
    32-bit).  Gate, scaled sum and norm are one kernel, which also leaves the new stream's copy in the
    activation type for whoever reads it next; nothing is left pending for the block that follows.

    Parameters: ``hidden_size``, ``alpha`` (1.0), ``mixer``, ``feed_forward`` (None: the mixer alone),
    ``mixer_norm``, ``feed_forward_norm`` (norms that offer ``gated_sum``), ``mixer_gate``, ``feed_forward_gate``
    (``stream`` parts that give the gate's logits and hold its ``bias``; None: no gate) and the weight-name prefixes
    of :class:`PreNormBlock` plus ``gate_prefix`` (``""``)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "mixer", "mixer_norm")
        self.hidden = int(params["hidden_size"])
        self.alpha = float(params.get("alpha", 1.0))
        self.mixer = build("mixer", params["mixer"], env)
        self.mixer_norm = build("norm", params["mixer_norm"], env)
        under = [(params.get("mixer_prefix", "mixer."), self.mixer),
                 (params.get("mixer_norm_prefix", "mixer_norm."), self.mixer_norm)]
        gate_prefix = params.get("gate_prefix", "")
        self.mixer_gate = self.feed_forward_gate = None
        if params.get("mixer_gate") is not None:
            self.mixer_gate = build("stream", params["mixer_gate"], env)
            under.append((gate_prefix, self.mixer_gate))
        self.feed_forward = self.feed_forward_norm = None
        if params.get("feed_forward") is not None:
            self.require("feed_forward_norm")
            self.feed_forward = build("feed_forward", params["feed_forward"], env)
            self.feed_forward_norm = build("norm", params["feed_forward_norm"], env)
            under.append((params.get("feed_forward_prefix", "feed_forward."), self.feed_forward))
            under.append((params.get("feed_forward_norm_prefix", "feed_forward_norm."), self.feed_forward_norm))
            if params.get("feed_forward_gate") is not None:
                self.feed_forward_gate = build("stream", params["feed_forward_gate"], env)
                under.append((gate_prefix, self.feed_forward_gate))
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "gated_sum"):
                raise PartError(f"the norm {type(norm).__name__} cannot normalise a gated sum")
        # parts whose tensors lie under one prefix (the norms' and gates' names are whole names here) load as one
        self._prefixes = {}
        for prefix in dict.fromkeys(p for p, _ in under):
            members = [part for p, part in under if p == prefix]
            self._prefixes[prefix] = members[0] if len(members) == 1 else _Several(members, env)

    def sub_parts(self) -> Dict[str, Part]:
        return dict(self._prefixes)

    def _sublayer(self, x, h, copy, sub, gate, norm, *args) -> None:
        logits = gate.forward(h) if gate is not None else None
        delta = sub.forward(h, *args)
        if isinstance(delta, Deferred):
            raise PartError("a sublayer of this block must hand back its sums")
        norm.gated_sum(x, delta, logits, gate.bias if gate is not None else None, self.alpha, copy)

    def forward(self, x: torch.Tensor, delta, step, cache: LayerCache):
        T = x.shape[0]
        if delta is not None and not isinstance(delta, Deferred):
            ops.residual_add(x, delta)           # what a block of another arrangement left pending
        if self.env.dtype == torch.float32:
            h, copy = x, None                    # the sublayers read the stream itself
        else:
            h = copy = self.env.workspace.get("block.stream_copy", (T, self.hidden), self.env.dtype)
            if step.shared.get("block.stream_copy") is not x:
                ops.norm_residual(x, None, None, 0.0, 1.0, copy)         # the copy alone (the first layer's input)
        self._sublayer(x, h, copy, self.mixer, self.mixer_gate, self.mixer_norm, step, cache)
        if self.feed_forward is not None:
            self._sublayer(x, h, copy, self.feed_forward, self.feed_forward_gate, self.feed_forward_norm, step)
        step.shared["block.stream_copy"] = x     # the copy is up to date with this residual
        return None


class _Several(Part):
    """Parts of a block that share one weight-name prefix."""

    def __init__(self, members, env: BuildEnv):
        super().__init__({}, env)
        self.members = list(members)

    def parts(self):
        yield self
        for m in self.members:
            yield from m.parts()

    def weights(self):
        return {n: ws for m in self.members for n, ws in m.weights().items()}

    def load(self, tensors) -> None:
        for m in self.members:
            names = set(m.weights())
            m.load({n: t for n, t in tensors.items() if n in names})
