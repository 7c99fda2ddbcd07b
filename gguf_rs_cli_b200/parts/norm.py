"""RMS norm: x / sqrt(mean(x^2) + eps) * w, sums in 32-bit (src/math/ops.rs:1-4,
src/gpu/rmsnorm.glsl:13-26), fused with the residual add that precedes it as the
reference's unused add_rmsnorm shader does (src/gpu/add_rmsnorm.glsl:1-32)."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorRequest, WeightStore
from .base import FUSE_MAX_TOKENS, DeferredNorm, Part, StepContext, Stream
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    """params: size, eps.  tensors: weight [size]."""

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.spec.tensors["weight"], (self.p["size"],), init="ones")]

    def load(self, store: WeightStore) -> None:
        self.weight = store.get(self.tensor_requests()[0])
        self._ones = None

    graph_class = ()

    def fold_weight(self) -> torch.Tensor:
        """The weight, for a consumer that multiplies it into the columns of its own matrix."""
        return self.weight

    def apply(self, stream: Stream, ctx: StepContext, rows: Optional[torch.Tensor] = None,
              buffer: str = "normed", absorbed: bool = False):
        """Adds the stream's pending term into x and returns the normalised rows.  With
        `rows`, only those rows are produced and x is left as it is.  absorbed: the consumer has
        this norm's weight in its matrix: it is left out here, and if the stream carries a valid
        shadow nothing is computed at all (a DeferredNorm is returned)."""
        if absorbed and rows is None and stream.pending is None and stream.xb is not None and ctx.T <= FUSE_MAX_TOKENS:
            return DeferredNorm(stream.xb, stream.ssq, stream.ssq_parts, self.p["size"], self.p["eps"])
        weight = self.weight
        if absorbed:
            if self._ones is None:
                self._ones = torch.ones_like(self.weight)
            weight = self._ones
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(buffer, (n, self.p["size"]), ctx.dtype)
        kernels.add_rmsnorm(stream.x, stream.pending, weight, self.p["eps"], out, rows=rows, write_x=rows is None)
        if rows is None:
            if stream.pending is not None:
                stream.drop_shadow()              # x has changed
            stream.pending = None
        return out


    def add_normed(self, stream: Stream, term: torch.Tensor, ctx: StepContext) -> None:
        """x += term / sqrt(mean(term^2) + eps) * w: the norm of a sublayer's result on its way into the stream
        (32-bit).  In bfloat16 mode the stream's bfloat16 copy is renewed by the same kernel; sums of squares of x
        are not kept (a deferred norm in front of the next product would need them)."""
        if stream.pending is not None:
            raise RuntimeError("rmsnorm: a term is pending on the stream")
        xb = ctx.ws.get("stream.xb", stream.x.shape, torch.bfloat16) if ctx.dtype == torch.bfloat16 else None
        kernels.norm_residual_add(stream.x, term, self.weight, self.p["eps"], xb=xb)
        stream.xb, stream.ssq, stream.ssq_parts = xb, None, 0


@register_norm("dyt")
class DynamicTanh(Part):
    """Dynamic tanh in a norm's place: tanh(alpha x) * weight + bias, no mean and no variance.
    params: size.  tensors: weight [size], bias [size], alpha [] (one scalar)."""

    def tensor_requests(self) -> List[TensorRequest]:
        t, n = self.spec.tensors, self.p["size"]
        return [TensorRequest(t["weight"], (n,), init="ones"), TensorRequest(t["bias"], (n,), init="zeros"),
                TensorRequest(t["alpha"], (), init="const:0.5")]

    def load(self, store: WeightStore) -> None:
        w, b, a = (store.get(r) for r in self.tensor_requests())
        self.weight, self.bias = w, b.to(w.dtype)
        self.alpha = float(a.float().item()) if a.device.type != "meta" else 0.0

    graph_class = ()

    def apply(self, stream: Stream, ctx: StepContext, rows: Optional[torch.Tensor] = None, buffer: str = "normed",
              absorbed: bool = False):
        """Adds the stream's pending term into x (32-bit) and returns tanh(alpha x) * weight + bias of all rows,
        or of `rows` only (x is then left as it is)."""
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(buffer, (n, self.p["size"]), ctx.dtype)
        kernels.add_dyt(stream.x, stream.pending, self.weight, self.bias, self.alpha, out, rows=rows, write_x=rows is None)
        if rows is None:
            if stream.pending is not None:
                stream.drop_shadow()
            stream.pending = None
        return out
