"""Grouped-query causal attention over the cache, as the mixer of a layer:
q, k, v projections (+ biases before the rotation, src/model/llama.rs:364-369), rotation
of q and k and the cache write in one kernel (src/model/llama.rs:370-373), attention
over the cached positions (src/model/llama.rs:374-394), output projection
(src/model/llama.rs:395).  q, k and v are one matrix after loading.

A window (not in the reference) limits each token to the last `window` positions and
gives the layer a cache group of its own kind.  With `shares_kv`, the mixer has no k
and v of its own and reads the cache of the run its schedule entry names.

Three further options, none in the reference, for designs that bring positions in without a
rotation: values of another size than keys (`v_head_dim`); queries and keys divided by their
root mean square per head, without a weight (`qk_norm_eps`); and a query temperature that grows
with the position, q <- q (1 + coef ln(floor((p + 1) / every) + 1)) (`q_temp`).  With any of them
scores, softmax and the mix of values run in 32-bit in the general attention kernel.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..cache.cache import KVSpec
from ..weights.loader import TensorRequest, WeightStore
from .base import HostBatch, Part, RunView, StepContext
from .linear import Linear
from .registry import register_mixer


@register_mixer("attention")
class Attention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale, window (None or W),
    bias (q/k/v biases), shares_kv (default False), v_head_dim (default head_dim),
    qk_norm_eps (default None: no normalisation), q_temp (default None, or {"coef", "every"}).
    tensors: q [nh*hd, E], k [nkv*hd, E], v [nkv*vd, E], o [E, nh*vd], optional q_bias, k_bias, v_bias."""

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.nh, self.nkv, self.hd = p["num_heads"], p["num_kv_heads"], p["head_dim"]
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} KV heads")
        self.scale = float(p.get("scale") or self.hd ** -0.5)
        self.window = p.get("window") or None
        self.shares_kv = bool(p.get("shares_kv", False))
        self.position = position
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.qk_norm_eps = p.get("qk_norm_eps")
        temp = p.get("q_temp") or None
        self.temp_coef, self.temp_every = (float(temp["coef"]), int(temp["every"])) if temp else (0.0, 1)
        if temp and self.temp_every <= 0:
            raise ValueError(f"attention: q_temp.every must be a positive whole number, got {temp['every']!r}")
        # normalised q and k, a query temperature or values of their own size: the exact path
        self.exact = self.vd != self.hd or self.qk_norm_eps is not None or self.temp_coef != 0.0
        if self.exact and (position is not None or self.shares_kv):
            raise ValueError("attention: qk_norm_eps, q_temp and v_head_dim go with neither a rotation nor shares_kv")

    def kv_spec(self) -> Optional[KVSpec]:
        return None if self.shares_kv else self.reads_kv_spec()

    def reads_kv_spec(self) -> KVSpec:
        """The kind of cache this mixer can read (its own, or another run's)."""
        return KVSpec(self.nkv, self.hd, self.window, None if self.vd == self.hd else self.vd)

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {}

    def tensor_requests(self) -> List[TensorRequest]:
        E, t = self.p["hidden_size"], self.spec.tensors
        names = ["q"] + ([] if self.shares_kv else ["k", "v"])
        rows = {"q": self.nh * self.hd, "k": self.nkv * self.hd, "v": self.nkv * self.vd}
        req = [TensorRequest(t[n], (rows[n], E)) for n in names]
        req.append(TensorRequest(t["o"], (E, self.nh * self.vd)))
        if self.p.get("bias"):
            req += [TensorRequest(t[n + "_bias"], (rows[n],)) for n in names]
        return req

    def load(self, store: WeightStore) -> None:
        req = {r.name: r for r in self.tensor_requests()}
        t = self.spec.tensors
        names = ["q"] + ([] if self.shares_kv else ["k", "v"])
        mats = [store.get(req[t[n]]) for n in names]
        dt = mats[0].dtype
        w = torch.cat([m.to(dt) for m in mats], dim=0) if len(mats) > 1 else mats[0]
        b = None
        if self.p.get("bias"):
            b = torch.cat([store.get(req[t[n + "_bias"]]).to(torch.float32) for n in names], dim=0)
        self.qkv = Linear(w, b, name="attn.qkv")
        self.o = Linear(store.get(req[t["o"]]), name="attn.o")

    accepts_residual = True

    # ---- planning on the host
    def plan_key(self):
        return ("attention", self.hd, self.window, self.exact)

    def plan(self, batch: HostBatch):
        """Prompts: the list of query tiles (sequence row, first query) that the prefill kernel's CTAs take."""
        if batch.decode or (self.exact and not self._exact_tiled()):
            return {}
        return {"tiles": kernels.attention_prefill_tiles(batch.qlens)}

    def _exact_tiled(self) -> bool:
        """Whether prompts of the exact path take the tiled kernel (bfloat16, keys and values of 64 or 128 entries
        both) with 32-bit attention weights; other sizes and the 32-bit mode take the general kernel."""
        return self.dtype == torch.bfloat16 and self.vd == self.hd and self.hd in (64, 128)

    def _exact_decode(self) -> bool:
        """Whether single tokens of the exact path take the CUDA-core decode kernel (32-bit weights; bfloat16, keys
        and values of one size that is a multiple of 16 up to 256)."""
        return self.dtype == torch.bfloat16 and self.vd == self.hd and self.hd % 16 == 0 and self.hd <= 256

    def graph_class(self, batch: HostBatch):
        """The decode kernel splits each sequence's pages over CTAs by a rule of the longest sequence; steps
        of one class launch the same grid and may share a captured graph."""
        if self.exact:
            # the general kernel: one block per token and head, whatever the lengths; the CUDA-core decode kernel
            # splits each sequence's pages by a rule of the longest sequence
            max_kv = min(batch.max_kv, self.window) if self.window else batch.max_kv
            return ("cuda", kernels.decode_split_class_exact(max_kv)) if self._exact_decode() else ()
        return kernels.decode_split_class(min(batch.max_kv, self.window) if self.window else batch.max_kv)

    def absorb_input_norm(self, weight: torch.Tensor) -> bool:
        """Multiplies the weight of the norm in front of this mixer into the q/k/v matrix, where
        the tensor-core product (which can apply the norm's per-token scale) will run it."""
        if not self.qkv.tensor_core():
            return False
        self.qkv.fold_input_scale(weight)
        return True

    def forward(self, h, ctx: StepContext, run: RunView, residual=None) -> Optional[torch.Tensor]:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        qkv = self.qkv(h, ctx)
        ctx.mark("qkv")
        if self.exact:
            return self._forward_exact(qkv, ctx, run, residual)
        q = qkv[:, :nh * hd]
        k = v = None
        if not self.shares_kv:
            k, v = qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
        table = ctx.tables[run.group]
        pos = self.position
        inv_freq = None if pos is None else pos.inv_freq
        rotary_dim, pairing = (0, 0) if pos is None else (pos.rotary_dim, pos.pairing)
        rope = None
        if kernels.decode_rotates(ctx, q, run.k, hd):
            rope = (k, v, inv_freq, rotary_dim, pairing)         # single tokens: the attention kernel rotates and writes
        else:
            kernels.rope_kv_write(q, k, v, nh, nkv, hd, inv_freq, rotary_dim, pairing, ctx.seq_of, ctx.pos, table,
                                  run.ring_pages, run.k if k is not None else None, run.v if k is not None else None)
        out = ctx.ws.get("attn.out", (h.shape[0], nh * hd), ctx.dtype)
        kernels.attention(q, out, nh, nkv, hd, ctx, table, run.ring_pages, run.k, run.v, self.window or 0, self.scale,
                          rope=rope, tiles=ctx.plan_of(self).get("tiles"))
        ctx.mark("attention")
        term = self.o(out, ctx, residual=residual)
        ctx.mark("o")
        return term

    def _forward_exact(self, qkv, ctx: StepContext, run: RunView, residual) -> Optional[torch.Tensor]:
        """q and k to unit root mean square, the query temperature and the cache write in one kernel, then
        attention with 32-bit scores and weights over keys of hd and values of vd entries."""
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        q, k, v = qkv[:, :nh * hd], qkv[:, nh * hd:(nh + nkv) * hd], qkv[:, (nh + nkv) * hd:]
        table = ctx.tables[run.group]
        kernels.qk_norm_kv_write(q, k, v, nh, nkv, hd, vd, self.qk_norm_eps is not None, self.qk_norm_eps or 1.0,
                                 self.temp_coef, self.temp_every, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v)
        out = ctx.ws.get("attn.out", (qkv.shape[0], nh * vd), ctx.dtype)
        tiles = ctx.plan_of(self).get("tiles")
        if not ctx.decode and tiles is not None and self._exact_tiled() and kernels.attention_prefill_supported(q, run.k, hd):
            kernels.attention_prefill(q, out, nh, nkv, hd, tiles, ctx.cu, ctx.starts, ctx.qlens, table, run.ring_pages,
                                      run.k, run.v, self.window or 0, self.scale, tc=False, exact=True)
        elif ctx.decode and self._exact_decode() and kernels.attention_decode_supported(q, run.k, hd):
            max_kv = min(ctx.max_kv, self.window) if self.window else ctx.max_kv
            splits = kernels.decode_splits_exact(q.shape[0], nh, nkv, max_kv, kernels.tc_scratch(q.device).sms)
            kernels.attention_decode(q, out, nh, nkv, hd, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v,
                                     self.window or 0, self.scale, mma=False, max_kv=max_kv, splits=splits)
        else:
            kernels.attention_generic(q, out, nh, nkv, hd, ctx.seq_of, ctx.pos, table, run.ring_pages, run.k, run.v,
                                      self.window or 0, self.scale, v_dim=vd)
        ctx.mark("attention")
        term = self.o(out, ctx, residual=residual)
        ctx.mark("o")
        return term
