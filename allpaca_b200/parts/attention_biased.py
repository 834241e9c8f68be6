"""Grouped-query attention without a rotation, whose positions enter through the scores:

* every query head and every key head is rescaled to unit mean square, ``v / sqrt(mean(v^2) + eps)``
  with ``eps = qk_norm_eps`` (None: left as projected), without a learned gain or, with
  ``qk_norm_weights``, times a weight per coordinate that all heads share (tensors ``q.norm``, ``k.norm``);
* the query at position ``p`` is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``
  (``q_temp = {"coef", "every"}``; None: no temperature);
* ``score(i, j) = (q_i . k_j) * scale - bias_h(i - j)`` with a penalty on the distance per query head
  (``distance_bias``): ``True`` or ``"log"``: ``r1[h] * ln(1 + r2[h] * d)`` with two learned numbers per
  head (tensors ``r1``, ``r2``); ``"linear"``: ``slope_h * d`` with the fixed slopes
  ``slope_h = 2^(-slope_exponent * (h + 1) / heads)`` (``slope_exponent`` 8: the slopes fall from
  ``2^(-8/heads)`` to ``2^-8``; no tensors); ``False``: none;
* the keys of a query at position ``i`` are those at ``i - window + 1 .. i`` (None: ``0 .. i``) and, with
  ``keep_first = n``, also the sequence's first ``n`` tokens, which stay visible for good at their true
  distance;
* keys and values may differ in size (``head_dim``, ``value_dim``);
* ``output_gate``: head ``h`` of the result is multiplied by ``sigmoid(g h)_h``, one number per row and
  head from the mixer's input (tensor ``g [heads, hidden]``), before the output projection;
* ``rope`` (a ``position`` part whose ``head_dim`` is the number of rotated coordinates): the first that many
  coordinates of every normed query and key head are turned by the position, coordinate ``i`` with ``i + dims/2``,
  the rest pass as they are;
* ``softcap`` ``c``: the scaled score becomes ``c * tanh(score / c)`` before bias and softmax;
* ``qkv_bias``: Q, K and V have biases (tensors ``q.b``, ``k.b``, ``v.b``), added before the norm;
* ``output_scale``: the mixer's result times a constant (carried by the values on their way into the pages, so
  that it costs nothing).

A token keeps its key and value side by side in pages ``[kv_heads, page, head_dim + value_dim]``;
with a window the cache manager takes back the pages it has passed (but those of the kept first
tokens).  Scores, softmax, gate and the weighted sum are 32-bit; the projections (the gate's among
them, stacked with Q, K and V into one product) give 32-bit sums, from which the norms are taken.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import BuildEnv, CacheNeed, LayerCache, Mixer, PartError, WeightSpec, build, register
from .linear import Linear


@register("mixer", "distance_biased_attention")
class DistanceBiasedAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``value_dim``
    (None: ``head_dim``), ``scale``, ``window``, ``keep_first``, ``qk_norm_eps``, ``qk_norm_weights``,
    ``q_temp``, ``distance_bias``, ``slope_exponent``, ``output_gate``, ``rope``, ``softcap``, ``qkv_bias``,
    ``output_scale``; tensors ``q``, ``k``, ``v``, ``o``
    (``[out, in]``) and, by the parameters, ``r1``, ``r2`` (``[num_heads]``), ``q.norm``, ``k.norm``
    (``[head_dim]``), ``g`` (``[num_heads, hidden]``)."""

    MAX_HEAD = 256

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "num_heads", "num_kv_heads", "head_dim", "scale")
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p["value_dim"]) if p.get("value_dim") is not None else self.hd
        if self.nkv <= 0 or self.nh % self.nkv:
            raise PartError(f"{self.nh} heads are not a multiple of {self.nkv} KV heads")
        if not (0 < self.hd <= self.MAX_HEAD and 0 < self.vd <= self.MAX_HEAD):
            raise PartError(f"head sizes {self.hd}/{self.vd} are not ones the kernel takes (1 to {self.MAX_HEAD})")
        self.scale = float(p["scale"])
        self.window = int(p["window"]) if p.get("window") else None
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") is not None else None
        temp = p.get("q_temp")
        self.temp_coef = float(temp["coef"]) if temp else 0.0
        self.temp_every = int(temp["every"]) if temp else 0
        if temp and self.temp_every <= 0:
            raise PartError("q_temp.every must be positive")
        bias = p.get("distance_bias", True)
        self.bias_kind = {True: "log", "log": "log", "linear": "linear", False: None, None: None}.get(bias, "?")
        if self.bias_kind == "?":
            raise PartError(f"distance_bias {bias!r} is not known (log, linear, False)")
        self.distance_bias = self.bias_kind == "log"            # the kind that has tensors
        self.slope_exponent = float(p.get("slope_exponent", 8.0))
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        if self.keep_first < 0:
            raise PartError("keep_first must not be negative")
        self.qk_norm_weights = bool(p.get("qk_norm_weights", False))
        if self.qk_norm_weights and self.qk_norm_eps is None:
            raise PartError("qk_norm_weights needs qk_norm_eps")
        self.output_gate = bool(p.get("output_gate", False))
        self.q_size, self.k_size, self.v_size = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd
        self.g_size = self.nh if self.output_gate else 0
        self.qkv = Linear(env, self.q_size + self.k_size + self.v_size + self.g_size, self.hidden)
        self.o = Linear(env, self.hidden, self.nh * self.vd)
        self.r1 = self.r2 = self.q_weight = self.k_weight = self.qkv_bias = None
        self.position = build("position", p["rope"], env) if p.get("rope") is not None else None
        if self.position is not None and (self.position.head_dim > self.hd or self.position.pairing != 0):
            raise PartError(f"a rotation of {self.position.head_dim} coordinates in half-split pairs does not fit "
                            f"heads of {self.hd}")
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.has_qkv_bias = bool(p.get("qkv_bias", False))
        self.output_scale = float(p.get("output_scale", 1.0))

    def parts(self):
        yield self
        if self.position is not None:
            yield from self.position.parts()

    def weights(self) -> Dict[str, WeightSpec]:
        w = {"q": WeightSpec((self.q_size, self.hidden)), "k": WeightSpec((self.k_size, self.hidden)),
             "v": WeightSpec((self.v_size, self.hidden)), "o": WeightSpec((self.hidden, self.nh * self.vd))}
        if self.distance_bias:
            w["r1"] = WeightSpec((self.nh,), "positive")
            w["r2"] = WeightSpec((self.nh,), "positive")
        if self.qk_norm_weights:
            w["q.norm"] = WeightSpec((self.hd,), "norm")
            w["k.norm"] = WeightSpec((self.hd,), "norm")
        if self.output_gate:
            w["g"] = WeightSpec((self.nh, self.hidden))
        if self.has_qkv_bias:
            w.update({"q.b": WeightSpec((self.q_size,), "bias"), "k.b": WeightSpec((self.k_size,), "bias"),
                      "v.b": WeightSpec((self.v_size,), "bias")})
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        stacked = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.output_gate else [])
        self.qkv.load(torch.cat(stacked, dim=0))
        self.o.load(tensors["o"])
        if self.distance_bias:
            self.r1 = tensors["r1"].float().contiguous()
            self.r2 = tensors["r2"].float().contiguous()
        elif self.bias_kind == "linear":
            # formed in 64-bit, rounded to 32-bit once
            h = torch.arange(1, self.nh + 1, dtype=torch.float64)
            self.r1 = torch.pow(torch.tensor(2.0, dtype=torch.float64), -self.slope_exponent * h / self.nh) \
                .to(torch.float32).to(self.env.device)
        if self.has_qkv_bias:
            self.qkv_bias = torch.cat([tensors["q.b"], tensors["k.b"], tensors["v.b"]]).float().contiguous()
        if self.qk_norm_weights:
            self.q_weight = tensors["q.norm"].float().contiguous()
            self.k_weight = tensors["k.norm"].float().contiguous()

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(outer=(self.nkv,), inner=(self.hd + self.vd,), window=self.window,
                         keep_first=self.keep_first)

    def forward(self, h: torch.Tensor, step, cache: LayerCache, into=None) -> torch.Tensor:
        """``into`` (optional, 32-bit ``[T, hidden]``): where the output projection leaves its sums, for a mixer
        that runs beside another one."""
        T = h.shape[0]
        ws = self.env.workspace
        qkv = self.qkv.forward(h, "battn.qkv", "float32")
        cos_sin = self.position.rotation_for(step)[0] if self.position is not None else None
        q = ws.get("battn.q", (T, self.q_size), self.env.dtype)
        table = step.block_tables[cache.group]
        ops.qk_norm_store(qkv, q, cache.pages if cache.writes else None, step.positions, step.token_seq, table,
                          self.nh, self.nkv, self.hd, self.vd, self.qk_norm_eps or 0.0,
                          normalise=self.qk_norm_eps is not None, temp_coef=self.temp_coef,
                          temp_every=self.temp_every, q_weight=self.q_weight, k_weight=self.k_weight,
                          bias=self.qkv_bias, cos_sin=cos_sin, value_scale=self.output_scale)
        gate = qkv[:, self.q_size + self.k_size + self.v_size:] if self.output_gate else None
        out = ws.get("battn.out", (T, self.nh * self.vd), self.env.dtype)
        # bfloat16: one-row sequences on the decode kernel (a step of such rows only is what a CUDA graph
        # records, and every replay is again such a step); 32-bit: one kernel for all rows, so that a
        # row has the same bits alone, in a portion and in a batch
        lens = step.host_query_lens
        single = self.env.dtype == torch.bfloat16 and (step.max_query_len == 1 or 1 in lens)
        ops.attention_window_bias(q, out, cache.pages, table, step.seq_start, step.positions, step.num_seqs,
                                  self.nh, self.nkv, self.hd, self.vd, self.scale, self.window or 0, self.r1, self.r2,
                                  single_rows=single, other_rows=step.max_query_len != 1, bias=self.bias_kind,
                                  keep_first=self.keep_first, gate=gate, softcap=self.softcap,
                                  max_context=step.max_decode_context_len or step.max_context_len)
        return self.o.forward(out, "battn.o", "delta", into=into)
