"""Norms fused with the residual addition that precedes them: RMSNorm, and Dynamic Tanh (no statistics).

``ss = sum x^2; inv = 1/sqrt(ss/n + eps); out = x * inv * w`` — eps inside the root,
weight multiplied last, no ``+1`` (crates/allpaca-cpu/src/kernels.rs:492-507; CUDA
cuda/src/kernels.cu:1152-1175).  The sum is 32-bit whatever the storage type.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, Norm, WeightSpec, register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """Parameters: ``size`` (width of a row), ``eps``, ``scalar_weight`` (False; True: the
    checkpoint holds one number for all coordinates, a tensor without dimensions), ``weight_name``
    (``"weight"``: the tensor's name behind the part's prefix; may be empty, the prefix then is
    the whole name)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("size", "eps")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.scalar_weight = bool(params.get("scalar_weight", False))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight = None
        self._kernel_weight = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec(() if self.scalar_weight else (self.size,), "norm")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        # one number for all coordinates: the kernels take it as a vector of equal entries
        self.weight = (w.reshape(1).expand(self.size) if self.scalar_weight else w).contiguous()
        self._kernel_weight = self.weight

    def fold(self) -> None:
        """The weight has been multiplied into the product that consumes this norm's output:
        from now on the kernel only divides by the root mean square."""
        self._kernel_weight = torch.ones_like(self.weight)

    @property
    def folded(self) -> bool:
        return self._kernel_weight is not self.weight

    def forward(self, x, out, delta=None, rows=None) -> None:
        ops.add_rmsnorm(x, self._kernel_weight, self.eps, out, delta=delta, rows=rows)

    def add_normed(self, x, delta, mult: float, copy=None) -> None:
        """The norm on a sublayer's output: ``x += mult * norm(delta)``; ``copy`` (optional) receives
        the updated rows in its own type."""
        ops.norm_residual(x, delta, self.weight, self.eps, mult, copy)


@register("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """A norm without statistics of the row: ``out = tanh(alpha * x) * weight + bias``, element by
    element, with one number ``alpha`` for the whole vector.  All 32-bit up to the store.

    Parameters: ``size``; ``weight_name`` (``"weight"``), ``bias_name`` (``"bias"``), ``alpha_name``
    (``"alpha"``): the tensors' names behind the part's prefix (``alpha`` is a tensor without dimensions).

    Because a row's result depends on that row alone, the norm can also hand out a row mixed with the row
    BEFORE it (:meth:`forward_shifted`) without a pass of its own."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("size")
        self.size = int(params["size"])
        self.weight_name = str(params.get("weight_name", "weight"))
        self.bias_name = str(params.get("bias_name", "bias"))
        self.alpha_name = str(params.get("alpha_name", "alpha"))
        self.weight = self.bias = None
        self.alpha = 1.0

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.size,), "norm"), self.bias_name: WeightSpec((self.size,), "bias"),
                self.alpha_name: WeightSpec((), "norm")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous()
        self.alpha = float(tensors[self.alpha_name].float().item())

    def forward(self, x, out, delta=None, rows=None) -> None:
        ops.add_dyt(x, self.weight, self.bias, self.alpha, out, delta=delta, rows=rows)

    def forward_shifted(self, x, out, shift: torch.Tensor, state: torch.Tensor, step) -> None:
        """``out_t = n_t + (n_{t-1} - n_t) * shift`` with ``n`` this norm of ``x`` (nothing pending on it) and
        ``state [slots, size]`` the requests' last normed rows, read and brought up to date."""
        ops.dyt_shift(x, self.weight, self.bias, self.alpha, shift, state, step.seq_start, step.positions,
                      step.token_seq, step.state_slots, out)


@register("norm", "group_rmsnorm")
class GroupRMSNorm(Norm):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive runs, each divided by its own
    ``sqrt(mean(run^2) + eps)``, and the whole multiplied by the weight.  All 32-bit up to the store.

    Parameters: ``size``, ``eps``, ``groups`` (1), ``weight_name`` (``"weight"``; may be empty, the prefix then is
    the whole name).

    Besides the common ``forward`` it offers :meth:`gated_sum`, the norm AFTER a sum, for blocks that normalise
    the stream itself: ``x <- norm(alpha * x + sigmoid(gate) * delta)``."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("size", "eps")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.groups = int(params.get("groups", 1))
        if self.groups <= 0 or self.size % self.groups:
            raise ValueError(f"a row of {self.size} does not fall into {self.groups} equal parts")
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.size,), "norm")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def forward(self, x, out, delta=None, rows=None) -> None:
        if delta is not None and rows is None:
            ops.residual_add(x, delta)
            delta = None
        ops.gated_postnorm(x, self.weight, self.groups, self.eps, delta=delta, rows=rows, out=out)

    def gated_sum(self, x, delta, gate, gate_bias, alpha: float, copy=None) -> None:
        """``x <- norm(alpha * x + sigmoid(gate + gate_bias) * sum(delta))`` in place on the 32-bit stream;
        ``copy`` (optional) receives the new rows in its own type."""
        ops.gated_postnorm(x, self.weight, self.groups, self.eps, alpha=alpha, delta=delta, gate=gate,
                           gate_bias=gate_bias, copy=copy)
