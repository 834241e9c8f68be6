"""SwiGLU feed-forward: ``down( silu(gate h) * (up h) )``.

``silu(z) = z / (1 + exp(-z))`` (crates/allpaca-cpu/src/kernels.rs:869-871); gate and up
are separate tensors in the checkpoint (crates/allpaca-core/src/model.rs:5664-5705) and one
matrix here whose rows alternate gate, up, gate, up ...: one product yields ``[T, 2I]`` with
each (gate, up) pair side by side.  On the tensor cores row 2i and 2i+1 of the weight are
neighbouring lanes of the accumulator, so for many rows the product's epilogue applies the
activation itself; for few rows a small kernel reads the pairs.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, FeedForward, WeightSpec, register
from .linear import Linear


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``bias`` (False: no biases, as on the
    Llama path), ``activation`` of the gate (``"silu"`` and ``"gelu_tanh"`` are applied in the
    product's epilogue on the tensor cores; others, like ``"relu"``, by a kernel of its own after the
    product; only with ``"silu"`` is the norm before folded in), ``names`` (the
    local tensor names of gate, up and down; default ``gate_proj.weight`` and so on)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "intermediate_size")
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.bias = bool(params.get("bias", False))
        self.activation = str(params.get("activation", "silu"))
        ops.routed.activation_code(self.activation)          # refuses an unknown name
        names = params.get("names") or ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
        self.gate_name, self.up_name, self.down_name = names
        if self.bias and params.get("names"):
            raise ValueError("a gated feed-forward with biases keeps the default tensor names")
        self.gate_up = Linear(env, 2 * self.inter, self.hidden)
        self.down = Linear(env, self.hidden, self.inter)

    def weights(self) -> Dict[str, WeightSpec]:
        w = {self.gate_name: WeightSpec((self.inter, self.hidden)),
             self.up_name: WeightSpec((self.inter, self.hidden)),
             self.down_name: WeightSpec((self.hidden, self.inter))}
        if self.bias:
            w.update({"gate_proj.bias": WeightSpec((self.inter,), "bias"),
                      "up_proj.bias": WeightSpec((self.inter,), "bias"),
                      "down_proj.bias": WeightSpec((self.hidden,), "bias")})
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        gate, up = tensors[self.gate_name], tensors[self.up_name]
        gu_bias = torch.stack([tensors["gate_proj.bias"], tensors["up_proj.bias"]], dim=1).reshape(-1) \
            if self.bias else None
        self.gate_up.load(torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden), gu_bias)
        self.down.load(tensors[self.down_name], tensors["down_proj.bias"] if self.bias else None)

    def can_fold_input_norm(self) -> bool:
        return self.activation == "silu" and self.gate_up.fusable() and self.down.fusable()

    def fold_input_norm(self, weight: torch.Tensor) -> None:
        """Multiply the weight of the norm before this feed-forward into its first product."""
        self.gate_up.fold_input_scale(weight)

    def fused_rows_ok(self, T: int) -> bool:
        return T <= Linear.FUSED_MAX_ROWS and self.down.residual_rows_ok(T)

    def forward_fused(self, h: torch.Tensor, scale, x: torch.Tensor, step):
        """For few rows: ``h`` with ``scale`` (an ``ops.RowScale``) stands for the normed input;
        the down projection adds into ``x`` itself.  Returns a :class:`Deferred`."""
        act = self.gate_up.forward_gated(h, "ffn.act", scale=scale)
        return self.down.forward_residual(act, x, "ffn")

    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        T = h.shape[0]
        act = None
        if self.activation in ("silu", "gelu_tanh"):
            act = self.gate_up.forward_gated(h, "ffn.act", activation=self.activation)   # the product's epilogue
        if act is None:
            gu = self.gate_up.forward(h, "ffn.gate_up", "either")
            act = self.env.workspace.get("ffn.act", (T, self.inter), self.env.dtype)
            if self.activation == "silu":
                ops.swiglu(gu, act, pairs=True)
            else:
                ops.gated_act(gu, act, self.activation, pairs=True)
        return self.down.forward(act, "ffn.down", "delta")


@register("feed_forward", "dense_act")
class DenseActivation(FeedForward):
    """A feed-forward without a gate: ``W_down act(W_up h + b_up) + b_down``.

    Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` (``"relu2"``: the square of relu;
    also ``"relu"``, ``"gelu_tanh"``, ``"silu"``), ``bias`` (True: both projections have one), ``names``
    (local tensor names of up and down, default ``("up", "down")``; a bias is ``<name>.b``).

    The first product leaves 32-bit sums; bias and activation act on those in one kernel and round once to
    the activation type; the second product's bias is added to its 32-bit sums."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "intermediate_size")
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.bias = bool(params.get("bias", True))
        self.activation = str(params.get("activation", "relu2"))
        if self.activation not in ops.stream.BIAS_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not known "
                             f"({', '.join(k for k in ops.stream.BIAS_ACTIVATIONS if k)})")
        self.up_name, self.down_name = params.get("names") or ("up", "down")
        self.up = Linear(env, self.inter, self.hidden)
        self.down = Linear(env, self.hidden, self.inter)
        self.up_bias = None

    def weights(self) -> Dict[str, WeightSpec]:
        w = {self.up_name: WeightSpec((self.inter, self.hidden)), self.down_name: WeightSpec((self.hidden, self.inter))}
        if self.bias:
            w[self.up_name + ".b"] = WeightSpec((self.inter,), "bias")
            w[self.down_name + ".b"] = WeightSpec((self.hidden,), "bias")
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.up.load(tensors[self.up_name])
        self.up_bias = tensors[self.up_name + ".b"].float().contiguous() if self.bias else None
        self.down.load(tensors[self.down_name], tensors[self.down_name + ".b"].float() if self.bias else None)

    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        T = h.shape[0]
        sums = self.up.forward(h, "ffn.up", "float32")
        act = self.env.workspace.get("ffn.act", (T, self.inter), self.env.dtype)
        ops.bias_act(sums, self.up_bias, act, self.activation)
        return self.down.forward(act, "ffn.down", "delta")
