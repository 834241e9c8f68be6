"""Attention whose keys and values are projections of one small latent vector per token.

With ``h`` the mixer's input, ``H`` heads, per head ``head_dim`` unrotated and ``rot_dim`` rotated
query/key dimensions, values of ``value_dim`` and a latent of ``kv_rank``:

* queries pass through a latent of their own: ``c_q = rmsnorm(W_dq h)`` (weight ``dq.norm``),
  ``q = W_uq c_q``, head by head ``[head_dim unrotated | rot_dim rotated]``;
* ``W_dkv h`` has ``kv_rank + rot_dim`` rows: the first ``kv_rank``, RMS-normed (weight ``dkv.norm``), are
  the latent ``c``; the last ``rot_dim``, not normed, are one rotated key part all heads share;
* head ``a`` has the unrotated key ``W_uk[a] c`` and the value ``W_uv[a] c``;
  ``score = (q_unrotated . k_unrotated + q_rotated . k_rotated) * scale``, causal, ordinary softmax;
* the rotation (``rope``: ``dims``, ``theta``, ``scaling``, see :mod:`.rope`) acts on the first ``dims`` of
  the ``rot_dim`` rotated dimensions of queries and of the shared key part, never on values;
* ``output_gate``: head ``a`` of the result is multiplied by ``sigmoid(W_g h)_a`` before ``W_o``;
* ``shares_latent``: the layer has no ``W_dkv`` and reads the latent and the rotated key part another
  layer's run keeps (the model's order names that run as this run's ``cache_from``), with its own
  ``W_uk``, ``W_uv``, queries and everything else;
* ``q_rank`` 0: the queries are one projection of the input, ``q = W_q h``, with no latent of their own;
* ``window``: position ``i`` sees ``j`` with ``0 <= i - j < window`` only (``cache_window``: how far back the
  pages must stay readable, which is the largest window among this layer and the layers that read its
  latent, or None where one of them has no window; older pages go back to the pool);
* ``sink``: with ``m`` the largest scaled score of a row, the softmax of head ``a`` divides by
  ``sum_j exp(s_j - m) + exp(sink_a - m)``: a learned logit per head that takes part in the normalisation only
  (it multiplies no value, and ``scale`` does not touch it).

A token keeps ``[c | rotated key part]`` in its page and nothing per head.  The kernels never form the
per-head keys and values: since ``q . (W_uk[a] c) = (W_uk[a]^T q) . c`` and
``sum_j p_j W_uv[a] c_j = W_uv[a] sum_j p_j c_j``, queries are carried into the latent space, the
attention runs there with ONE key/value head whose value is the head of its key's record, and its
result is carried out through ``W_uv``.  Norms, angles, scores, softmax, gate and all sums are 32-bit.

That form reads little, which is what decoding wants, but a score costs ``kv_rank + rot_dim``
multiplications instead of ``head_dim + rot_dim``.  Where the latent is wide (a record of more than 128
numbers) the bfloat16 engine therefore serves sequences that bring several rows the other way round:
the records of their tokens so far are gathered from the pages, ONE product with the matrix
``[W_uk[a] | 0; 0 | I; W_uv[a] | 0]`` stacked over the heads turns them into per-head
``[key | rotated key part | value]`` rows, and a tensor-core attention kernel made for such rows runs on
those (head sizes it does not take go to the general kernel, to which they are pages of one token with
``H`` key/value heads).  The identity block copies the rotated part exactly.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import BuildEnv, CacheNeed, LayerCache, Mixer, PartError, PartSpec, WeightSpec, build, register
from .linear import Linear


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``rot_dim``, ``value_dim``, ``kv_rank``,
    ``q_rank`` (0: none), ``scale``, ``norm_eps``, ``rope`` (``{"dims", "theta", "scaling"}``), ``output_gate``,
    ``shares_latent``, ``window`` (None), ``cache_window`` (the window), ``sink`` (False); tensors ``dq``,
    ``dq.norm``, ``uq`` (or ``q`` without a query latent), ``dkv``, ``dkv.norm`` (both absent with
    ``shares_latent``), ``uk``, ``uv``, ``g`` (with ``output_gate``), ``sink`` (with ``sink``), ``o``."""

    MAX_RECORD = 640            # widest [latent | rotated part] the attention kernels take

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("hidden_size", "num_heads", "head_dim", "rot_dim", "value_dim", "kv_rank", "scale", "norm_eps")
        p = params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["num_heads"])
        self.hd, self.rot, self.vd = int(p["head_dim"]), int(p["rot_dim"]), int(p["value_dim"])
        self.R, self.Q = int(p["kv_rank"]), int(p.get("q_rank") or 0)
        self.scale, self.eps = float(p["scale"]), float(p["norm_eps"])
        self.output_gate = bool(p.get("output_gate", False))
        self.shares_latent = bool(p.get("shares_latent", False))
        if min(self.nh, self.hd, self.vd, self.R) <= 0 or self.rot < 0 or self.Q < 0:
            raise PartError("latent attention needs positive sizes")
        self.window = int(p.get("window") or 0)
        self.cache_window = int(p.get("cache_window", self.window) or 0)        # 0: every page stays
        if self.window < 0 or (self.cache_window > 0 and not (0 < self.window <= self.cache_window)):
            raise PartError("a latent attention layer's pages must stay readable as far back as its window reaches")
        self.has_sink = bool(p.get("sink", False))
        self.sink = None
        if self.R + self.rot > self.MAX_RECORD:
            raise PartError(f"a latent of {self.R} with {self.rot} rotated dimensions is wider than the "
                            f"attention kernels take ({self.MAX_RECORD})")
        rope = p.get("rope")
        self.rope = None
        self.rot_dims = 0
        if rope and self.rot > 0:
            self.rot_dims = int(rope["dims"])
            if self.rot_dims % 2 or not (0 < self.rot_dims <= self.rot):
                raise PartError(f"{self.rot_dims} rotated dimensions do not fit a rotated part of {self.rot}")
            self.rope = build("position", PartSpec("rope", {
                "head_dim": self.rot_dims, "theta": float(rope["theta"]), "scaling": rope.get("scaling"),
                "pairing": "half"}), env)
        self.kv_size = 0 if self.shares_latent else self.R + self.rot
        self.g_size = self.nh if self.output_gate else 0
        # one product for everything that reads the mixer's input: [dq (or the queries themselves) | dkv | g]
        self.q_cols = self.Q if self.Q > 0 else self.nh * (self.hd + self.rot)
        self.down = Linear(env, self.q_cols + self.kv_size + self.g_size, self.hidden)
        self.uq = Linear(env, self.nh * (self.hd + self.rot), self.Q) if self.Q > 0 else None
        self.o = Linear(env, self.hidden, self.nh * self.vd)
        self.uk = self.uv = self.q_weight = self.kv_weight = None
        # the per-head form for prompt portions (see the module's text): where the latent space is too wide for
        # the tensor-core attention kernel and the heads' own sizes are not
        rec = self.R + self.rot
        self.expands = (env.dtype == torch.bfloat16 and rec > 128 and rec % 8 == 0
                        and self.hd + self.rot <= 192 and self.vd <= 128)
        self.expand = Linear(env, self.nh * (self.hd + self.rot + self.vd), rec) if self.expands else None

    def weights(self) -> Dict[str, WeightSpec]:
        w = {"uk": WeightSpec((self.nh * self.hd, self.R)), "uv": WeightSpec((self.nh * self.vd, self.R)),
             "o": WeightSpec((self.hidden, self.nh * self.vd))}
        if self.Q > 0:
            w.update({"dq": WeightSpec((self.Q, self.hidden)), "dq.norm": WeightSpec((self.Q,), "norm"),
                      "uq": WeightSpec((self.nh * (self.hd + self.rot), self.Q))})
        else:
            w["q"] = WeightSpec((self.nh * (self.hd + self.rot), self.hidden))
        if self.has_sink:
            w["sink"] = WeightSpec((self.nh,), "bias")
        if not self.shares_latent:
            w["dkv"] = WeightSpec((self.R + self.rot, self.hidden))
            w["dkv.norm"] = WeightSpec((self.R,), "norm")
        if self.output_gate:
            w["g"] = WeightSpec((self.nh, self.hidden))
        return w

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        stacked = [tensors["dq" if self.Q > 0 else "q"]] + ([] if self.shares_latent else [tensors["dkv"]]) \
            + ([tensors["g"]] if self.output_gate else [])
        self.down.load(torch.cat(stacked, dim=0))
        if self.Q > 0:
            self.uq.load(tensors["uq"])
        if self.has_sink:
            self.sink = tensors["sink"].float().contiguous()
        self.o.load(tensors["o"])
        # per head: [head_dim, kv_rank] carries a query into the latent space as it is stored;
        # [kv_rank, value_dim] (the stored matrix transposed) carries a latent result out
        self.uk = tensors["uk"].view(self.nh, self.hd, self.R).contiguous()
        self.uv = tensors["uv"].view(self.nh, self.vd, self.R).transpose(1, 2).contiguous()
        self.q_weight = tensors["dq.norm"].float().contiguous() if self.Q > 0 else None
        if self.expands:
            uk3 = tensors["uk"].view(self.nh, self.hd, self.R)
            uv3 = tensors["uv"].view(self.nh, self.vd, self.R)
            w = torch.zeros(self.nh, self.hd + self.rot + self.vd, self.R + self.rot, dtype=uk3.dtype, device=uk3.device)
            w[:, :self.hd, :self.R] = uk3
            w[:, self.hd:self.hd + self.rot, self.R:] = torch.eye(self.rot, dtype=uk3.dtype, device=uk3.device)
            w[:, self.hd + self.rot:, :self.R] = uv3
            self.expand.load(w.view(-1, self.R + self.rot))
            self.expands = self.expand.uses_tensor_cores()
        if not self.shares_latent:
            self.kv_weight = tensors["dkv.norm"].float().contiguous()

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(outer=(), inner=(self.R + self.rot,), window=self.cache_window or None)

    def forward(self, h: torch.Tensor, step, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        ws = self.env.workspace
        dt = self.env.dtype
        if cache.writes == self.shares_latent:
            raise PartError("a latent attention layer writes pages exactly when it has a down-projection of its own")
        proj = self.down.forward(h, "lattn.down", "float32")
        cos_sin = self.rope.rotation_for(step)[0] if self.rope is not None else None
        table = step.block_tables[cache.group]
        cq = ws.get("lattn.cq", (T, self.Q), dt) if self.Q > 0 else None
        ops.latent_prepare(proj, 0, self.Q, self.q_weight, cq, self.q_cols, self.R, self.rot, self.rot_dims,
                           self.kv_weight, cache.pages if cache.writes else None, step.positions, step.token_seq,
                           table, cos_sin, self.eps)
        # the queries: through their own latent, or the first columns of the stacked product as they are
        q = self.uq.forward(cq, "lattn.q", "float32") if self.Q > 0 else proj[:, :self.q_cols]
        rec = self.R + self.rot
        gate = proj[:, self.q_cols + self.kv_size:] if self.output_gate else None
        W, sink = self.window, self.sink
        # The host's lists decide only between steps that differ in kind: a step of single rows only (what a CUDA
        # graph records, and every replay is again such a step) never reads them beyond this line
        lens = step.host_query_lens
        singles = step.max_query_len == 1 or 1 in lens
        per_head = self.expands and step.max_query_len > 1
        ov = ws.get("lattn.ov", (T, self.nh * self.vd), dt)
        if singles or not per_head:
            # in the latent space: every row, or (beside the per-head form) the sequences that bring one row
            qa = ws.get("lattn.qa", (T, self.nh * rec), dt)
            ops.head_project(q, self.uk, qa, self.nh, tail=self.rot, tail_dims=self.rot_dims, cos_sin=cos_sin)
            ol = ws.get("lattn.ol", (T, self.nh * self.R), dt)
            # sequences that bring one row: all heads together against shared key tiles on the tensor cores
            fast = dt == torch.bfloat16 and singles and ops.latent_decode_takes(rec, self.R)
            if fast:
                ops.latent_decode(qa, ol, cache.pages, table, step.seq_start, step.positions, step.num_seqs, self.nh,
                                  rec, self.R, self.scale, gate, step.max_decode_context_len or step.max_context_len, ws,
                                  window=W, sink=sink)
            others = step.max_query_len != 1 and not per_head
            if others or not fast:
                ops.attention_window_bias(qa, ol, cache.pages, table, step.seq_start, step.positions, step.num_seqs,
                                          self.nh, 1, rec, self.R, self.scale, W, None, None,
                                          single_rows="skip" if fast else (dt == torch.bfloat16 and singles),
                                          other_rows=others, bias=None, gate=gate, record=rec, value_offset=0, sink=sink)
            ops.head_project(ol, self.uv, ov, self.nh)
        if per_head:
            # the sequences that bring several rows, on per-head keys and values of all their tokens so far
            # (behind a window: from the first token that the sequence's first row still sees)
            spans = [f + n for f, n in zip(step.host_first_position, lens) if n > 1]
            kept = [n + min(f, W - 1) if W > 0 else f + n for f, n in zip(step.host_first_position, lens) if n > 1]
            total, width = sum(kept), max(spans)
            gathered = ws.get("lattn.gathered", (total, rec), dt)
            where = ws.get("lattn.where", (step.num_seqs, width), torch.int32)
            ops.latent_gather(cache.pages, table, step.seq_start, step.context_lens, step.num_seqs, gathered, where, W)
            kv = self.expand.forward(gathered, "lattn.expanded", "either")
            key = self.hd + self.rot
            qr = ws.get("lattn.qr", (T, self.nh * key), dt)
            ops.head_project(q, None, qr, self.nh, tail=self.rot, tail_dims=self.rot_dims, cos_sin=cos_sin)
            if ops.latent_prefill_takes(key, self.vd):
                ops.latent_prefill(qr, ov, kv, where, step.seq_start, step.positions, step.num_seqs, self.nh, key,
                                   self.vd, self.scale, gate, window=W, sink=sink)
            else:
                # to the general tensor-core kernel these are pages of one token with a key/value head per head
                ops.attention_window_bias(qr, ov, kv.view(total, self.nh, 1, key + self.vd), where, step.seq_start,
                                          step.positions, step.num_seqs, self.nh, self.nh, key, self.vd, self.scale, W,
                                          None, None, single_rows="skip" if singles else False, other_rows=True,
                                          bias=None, gate=gate, record=key + self.vd, value_offset=key, sink=sink)
        return self.o.forward(ov, "lattn.o", "delta")
