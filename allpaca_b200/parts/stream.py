"""Parts that act on the residual stream around a layer's sublayers, for blocks that ask for them.

``token_shift``: what the mixer reads is first mixed with the PREVIOUS token's normed row,
``h_t <- h_t + (h_{t-1} - h_t) * shift`` element by element (``h_{-1} = 0``).  Between steps a
request keeps its last normed row in its state slot, 4 bytes per column.  The arithmetic lives in the
norm before the mixer (``forward_shifted``), which sees both rows anyway.

``depth_average``: the layer's result ``X_k`` (the stream after its sublayers) is kept, and what goes on
is a weighted sum of ALL results so far, ``x <- sum_{j <= k} a[j] X_j`` with ``X_0`` the embedding
output.  The results of a step's rows wait in a workspace buffer ``[count, T, hidden]``; nothing is
kept between steps.  All 32-bit.

``residual_gate``: a gate per coordinate on what a sublayer adds to the stream, read off the sublayer's input.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, Part, PartError, WeightSpec, register
from .linear import Linear


@register("stream", "token_shift")
class TokenShift(Part):
    """Parameters: ``hidden_size``, ``weight_name`` (``"weight"``); tensor: the mixing vector ``[hidden]``."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size")
        self.hidden = int(params["hidden_size"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden,), "bias")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def state_bytes(self) -> int:
        return 4 * self.hidden


@register("stream", "depth_average")
class DepthAverage(Part):
    """Parameters: ``hidden_size``, ``index`` (``k``: this layer's result is stream ``k``; the weights are
    ``k + 1`` numbers), ``count`` (streams of the whole model: every layer asks for the same buffer),
    ``stores_first`` (True for the layer that runs first: it also keeps the stream it receives as ``X_0``),
    ``weight_name`` (``"weight"``)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "index", "count")
        self.hidden, self.index, self.count = int(params["hidden_size"]), int(params["index"]), int(params["count"])
        if not (0 < self.index < self.count):
            raise PartError(f"stream {self.index} of {self.count} cannot be a layer's result")
        self.stores_first = bool(params.get("stores_first", self.index == 1))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.index + 1,), "norm")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def _streams(self, T: int) -> torch.Tensor:
        return self.env.workspace.get("stream.results", (self.count, T, self.hidden), torch.float32)

    def begin(self, x: torch.Tensor) -> None:
        """Before the first layer's sublayers: keep the stream as it arrives."""
        if self.stores_first:
            ops.stream_mix(x, None, self._streams(x.shape[0]), 0, None)

    def finish(self, x: torch.Tensor, delta) -> None:
        """``x + delta`` is this layer's result: keep it, and leave the weighted sum of all results in ``x``."""
        ops.stream_mix(x, delta, self._streams(x.shape[0]), self.index, self.weight)


@register("stream", "residual_gate")
class ResidualGate(Part):
    """A gate on what a sublayer adds to the stream: ``sigmoid(W h + b)``, one number per coordinate, read off
    the rows the sublayer itself reads.  This part forms ``W h`` (32-bit sums); the sigmoid, the bias and the
    product with the sublayer's result belong to the kernel that adds into the stream.

    Parameters: ``hidden_size``, ``name`` (the matrix's tensor name; its bias is ``<name>.b``)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "name")
        self.hidden = int(params["hidden_size"])
        self.name = str(params["name"])
        self.linear = Linear(env, self.hidden, self.hidden)
        self.bias = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.hidden, self.hidden)), self.name + ".b": WeightSpec((self.hidden,), "bias")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.linear.load(tensors[self.name])
        self.bias = tensors[self.name + ".b"].float().contiguous()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """The gate's logits without the bias, 32-bit ``[T, hidden]``."""
        return self.linear.forward(h, "stream.gate." + self.name, "float32")
