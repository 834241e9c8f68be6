"""A routed feed-forward: ``experts`` small gated feed-forward layers, of which every row uses
the ``top`` whose router logits are largest.

Router logits ``z = W_router h + b`` are 32-bit.  With ``S`` the set of the ``top`` largest,
expert ``e`` in ``S`` gets the share ``exp(z_e) / sum_{s in S} exp(z_s)`` and the layer returns
``sum_{e in S} share_e * expert_e(h)``.
Another routing (``"softmax_all"``): scores ``s = softmax(W_router h)`` over all experts; ``S`` holds the
``top`` largest ``s + b`` (``b`` steers the choice only); the shares are ``s_e / (sum_{s in S} s + 1e-20)``.
A third (``"sigmoid"``): scores ``s = sigmoid(W_router h)``, every expert alone; ``S`` holds the ``top`` largest
(``+ b`` where there is a bias); the shares are the chosen scores as they are.
With ``weight_on = "input"`` a share multiplies what its expert READS, not what it returns: the layer returns
``sum_{e in S} expert_e(share_e * h)`` (both first products are linear in the row, so the share multiplies their
sums before the activation).
``shared`` (``{"size", "gate"}``): one more expert of its own size that every row uses (tensors ``shared.gate``,
``shared.up``, ``shared.down``), its result multiplied by ``sigmoid(w_sg . h)``, one number per row (tensor
``shared.sg [1, hidden]``) where ``gate`` is true, and added.
The last ``identity`` outputs of the router may stand for identity experts, which have no tensors: their
result is the input ``h`` itself (times the share).
An expert is ``W_down act(W_gate h, W_up h)`` without biases, ``act`` one of the gated
activations of ``ops.gated_act`` (``clamped_sigmoid``: ``g' = min(g, limit)``,
``u' = clamp(u, -limit, limit)``, ``g' sigmoid(alpha g') (u' + shift)``).

On the device the (row, choice) pairs are grouped by expert, every expert's rows run through
its two products in tiles, and a last pass adds each row's weighted results in the order of
its choices.  Counts and tiles never leave the device, so a step can be replayed from a CUDA
graph, and a row's result does not depend on what else is in the batch.

A bfloat16 step that brings a prompt portion and many pairs takes another way: the experts'
first positions come to the host (one small copy, and the only wait on the device in the
step), the rows are gathered in grouped order, and every expert's rows run through the
tcgen05 products the dense layers use, one pair of launches per expert.  Such a step is never
recorded as a CUDA graph (only steps of one row per request are), so deciding on the host
is safe there.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, FeedForward, PartError, PartSpec, WeightSpec, build, register
from .linear import Linear


@register("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """Parameters: ``hidden_size``, ``expert_size``, ``experts``, ``top``, ``activation``
    (``"clamped_sigmoid"``), ``limit``, ``alpha`` (1.702), ``shift`` (1.0), ``router_bias`` (True),
    ``routing`` (``"top_softmax"``), ``identity`` (0: identity experts behind the ``experts`` real ones),
    ``router_bias_name`` (``"router.b"``), ``weight_on`` (``"output"``), ``shared`` (None);
    tensors ``router`` ``[experts + identity, hidden]``, the router's bias ``[experts + identity]`` and, per expert ``i``,
    ``e<i>.gate``, ``e<i>.up`` ``[expert_size, hidden]`` and ``e<i>.down`` ``[hidden, expert_size]``."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "expert_size", "experts", "top")
        p = params
        self.hidden, self.inter = int(p["hidden_size"]), int(p["expert_size"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.identity = int(p.get("identity", 0))
        self.outputs = self.experts + self.identity          # what the router chooses among
        self.routing = str(p.get("routing", "top_softmax"))
        if self.routing not in ops.routed.ROUTE_MODES:
            raise PartError(f"routing {self.routing!r} is not known ({', '.join(ops.routed.ROUTE_MODES)})")
        if self.experts < 0 or self.identity < 0 or not (0 < self.top <= self.outputs) or self.outputs > 256 \
                or self.top > 16:
            raise PartError(f"{self.top} of {self.experts} + {self.identity} experts is not a routing the kernels "
                            f"take (at most 16 of at most 256)")
        self.activation = str(p.get("activation", "clamped_sigmoid"))
        ops.routed.activation_code(self.activation)
        self.limit = float(p.get("limit", 0.0))
        self.alpha = float(p.get("alpha", 1.702))
        self.shift = float(p.get("shift", 1.0))
        self.router_bias = bool(p.get("router_bias", True))
        self.router_bias_name = str(p.get("router_bias_name", "router.b"))
        if self.activation == "clamped_sigmoid" and not self.limit > 0:
            raise PartError("the clamped activation needs a positive limit")
        self.weight_on = str(p.get("weight_on", "output"))
        if self.weight_on not in ("output", "input"):
            raise PartError(f"weight_on {self.weight_on!r} is not known (output, input)")
        if self.weight_on == "input" and self.identity:
            raise PartError("identity experts with shares on the experts' inputs are not built")
        self.shared = self.shared_gate = None
        if p.get("shared"):
            sh = dict(p["shared"])
            self.shared = build("feed_forward", PartSpec("swiglu", {
                "hidden_size": self.hidden, "intermediate_size": int(sh["size"]),
                "activation": sh.get("activation", self.activation),
                "names": ("shared.gate", "shared.up", "shared.down")}), env)
            self.shared_gated = bool(sh.get("gate", False))

    def parts(self):
        yield self
        if self.shared is not None:
            yield from self.shared.parts()

    def weights(self) -> Dict[str, WeightSpec]:
        w = {"router": WeightSpec((self.outputs, self.hidden))}
        if self.router_bias:
            w[self.router_bias_name] = WeightSpec((self.outputs,), "bias")
        for e in range(self.experts):
            w[f"e{e}.gate"] = WeightSpec((self.inter, self.hidden))
            w[f"e{e}.up"] = WeightSpec((self.inter, self.hidden))
            w[f"e{e}.down"] = WeightSpec((self.hidden, self.inter))
        if self.shared is not None:
            w.update(self.shared.weights())
            if self.shared_gated:
                w["shared.sg"] = WeightSpec((1, self.hidden))
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.router = tensors["router"].contiguous()
        if self.shared is not None:
            self.shared.load({n: tensors[n] for n in self.shared.weights()})
            self.shared_gate = tensors["shared.sg"].reshape(-1).contiguous() if self.shared_gated else None
        self.router_b = tensors[self.router_bias_name].float().contiguous() if self.router_bias else None
        # [experts, 2 F, hidden]: an expert's gate rows, then its up rows; [experts, hidden, F]
        if self.experts > 0:
            self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                        for e in range(self.experts)]).contiguous()
            self.down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).contiguous()
        else:                                            # identity experts only: nothing to multiply by
            self.gate_up = self.router.new_zeros((1, 2 * self.inter, self.hidden))
            self.down = self.router.new_zeros((1, self.hidden, self.inter))

    #: pairs from which a prompt step's experts run on the tensor cores, one product per expert
    TENSOR_CORE_MIN_PAIRS = 512

    def _per_expert_on_tensor_cores(self, h, step, pairs: int) -> bool:
        return (self.env.dtype == torch.bfloat16 and step is not None and step.max_query_len > 1
                and pairs >= self.TENSOR_CORE_MIN_PAIRS and self.gate_up.dtype == torch.bfloat16
                and self.hidden % 8 == 0 and self.inter % 8 == 0 and ops.tensor_core_gemm_available())

    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        T = h.shape[0]
        ws = self.env.workspace
        pairs = T * self.top
        on_input = self.weight_on == "input"
        chosen = ws.get("moe.chosen", (T, self.top), torch.int32)
        weight = ws.get("moe.weight", (T, self.top), torch.float32)
        ops.moe_route_rows(h, self.router, self.router_b, chosen, weight, self.routing)   # router logits in 32-bit sums
        perm = ws.get("moe.perm", (pairs,), torch.int32)
        place = ws.get("moe.place", (pairs,), torch.int32)
        tiles = ws.get("moe.tiles", (ops.moe_max_tiles(pairs, self.outputs) + 1, 3), torch.int32)
        y = ws.get("moe.act", (pairs, self.inter), self.env.dtype)
        o = ws.get("moe.out", (pairs, self.hidden), torch.float32)
        if self._per_expert_on_tensor_cores(h, step, pairs):
            offsets = ws.get("moe.offsets", (self.outputs + 1,), torch.int32)
            ops.moe_sort(chosen, perm, place, tiles, self.outputs, offsets, real=self.experts)
            first = offsets.tolist()                                   # the step waits for the device here
            rows = ws.get("moe.rows", (pairs, self.hidden), torch.bfloat16)
            ops.moe_gather(h, rows, perm, self.top)
            gu = ws.get("moe.gate_up", (pairs, 2 * self.inter), torch.bfloat16)
            for e in range(self.experts):
                a, b = first[e], first[e + 1]
                if b > a:
                    Linear.tensor_core_product(rows[a:b], self.gate_up[e], gu[a:b])
            ops.gated_act(gu, y, self.activation, False, self.limit, self.alpha, self.shift,
                          row_scale=weight.view(-1) if on_input else None, scale_index=perm if on_input else None)
            for e in range(self.experts):
                a, b = first[e], first[e + 1]
                if b > a:
                    Linear.tensor_core_product(y[a:b], self.down[e], o[a:b])
        else:
            ops.moe_sort(chosen, perm, place, tiles, self.outputs, real=self.experts)
            ops.moe_gate_up(h, self.gate_up, y, perm, self.top, tiles, self.activation, self.limit, self.alpha,
                            self.shift, experts=self.outputs, pair_scale=weight.view(-1) if on_input else None)
            ops.moe_down(y, self.down, o, tiles, experts=self.outputs)
        delta = ws.get("moe.delta", (1, T, self.hidden), torch.float32)
        if self.identity > 0:
            ops.moe_combine(o, place, weight, delta[0], chosen=chosen, real=self.experts, rows=h)
        else:
            ops.moe_combine(o, place, weight, delta[0], unweighted=on_input)
        if self.shared is not None:
            other = self.shared.forward(h, step)
            if self.shared_gate is not None:
                ops.gated_row_add(delta[0], other[0], h, self.shared_gate)
            else:
                ops.residual_add(delta[0], other)
        return delta
