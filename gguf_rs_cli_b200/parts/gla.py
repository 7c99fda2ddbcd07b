"""Gated linear attention, as the mixer of a layer.

Per head the mixer keeps a matrix S [dim, vdim] per sequence (32-bit) instead of keys and values:
    S <- diag(alpha) S + k v^T;  o = S^T q
with q = W_q h dim^-1/2, k = W_k h, v = W_v h and a decay per head and key channel,
alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau).  What is read out is brought to unit root mean square per head,
multiplied by a weight of vdim entries that the heads share and by SiLU(W_g h), and projected back.  The rank of the
low-rank pair is the files' own size.  The reference has no such mixer (src/model/llama.rs has attention only).

q, k, v, g and a1 are one matrix after loading (each part starting at a multiple of 8 rows), so one product reads h
once.  Decays, their logarithms and the state are 32-bit (csrc/gla.cu).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..cache.cache import KVSpec
from ..weights.loader import TensorRequest, WeightStore
from .base import Part, RunView, StepContext
from .linear import Linear
from .registry import register_mixer


@register_mixer("gla")
class GatedLinearAttention(Part):
    """params: hidden_size, heads, dim, vdim, tau (the decay is the tau-th root of a sigmoid), eps (of the read-out's norm).
    tensors: q, k [heads*dim, E], v, g [heads*vdim, E], a1 [r, E], a2 [heads*dim, r], a2_bias [heads*dim], norm [vdim],
    o [E, heads*vdim]."""

    NAMES = ("q", "k", "v", "g", "a1", "a2", "a2_bias", "norm", "o")

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.H, self.D, self.Dv, self.tau = p["heads"], p["dim"], p["vdim"], float(p["tau"])
        if not self.tau > 0:
            raise ValueError(f"gla: tau must be positive, got {p['tau']!r}")

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"S": ((self.H, self.D, self.Dv), "float32")}

    def tensor_requests(self) -> List[TensorRequest]:
        E, t, H, D, Dv = self.p["hidden_size"], self.spec.tensors, self.H, self.D, self.Dv
        rank = max(8, (E // 16 + 7) // 8 * 8)               # what random weights get where the files' own rank is missing
        return [TensorRequest(t["q"], (H * D, E)), TensorRequest(t["k"], (H * D, E)), TensorRequest(t["v"], (H * Dv, E)),
                TensorRequest(t["g"], (H * Dv, E)), TensorRequest(t["a1"], (-1, E), init_shape=(rank, E)),
                TensorRequest(t["a2"], (H * D, -1), init_shape=(H * D, rank)),
                TensorRequest(t["a2_bias"], (H * D,), init="uniform:2:5"), TensorRequest(t["norm"], (Dv,), init="ones"),
                TensorRequest(t["o"], (E, H * Dv))]

    def load(self, store: WeightStore) -> None:
        w = {local: store.get(r) for local, r in zip(self.NAMES, self.tensor_requests())}
        if w["a1"].shape[0] != w["a2"].shape[1]:
            raise ValueError(f"gla: the low-rank pair does not fit: a1 {list(w['a1'].shape)} a2 {list(w['a2'].shape)}")
        dt = w["q"].dtype
        self.rank = w["a1"].shape[0]
        parts, self.off, rows = [], {}, 0
        for name in ("q", "k", "v", "g", "a1"):
            pad = (rows + 7) // 8 * 8 - rows
            if pad:
                parts.append(torch.zeros(pad, w[name].shape[1], dtype=dt, device=w[name].device))
            self.off[name] = rows + pad
            parts.append(w[name].to(dt))
            rows = self.off[name] + w[name].shape[0]
        pad = (rows + 7) // 8 * 8 - rows
        if pad:
            parts.append(torch.zeros(pad, w["q"].shape[1], dtype=dt, device=w["q"].device))
        self.proj = Linear(torch.cat(parts, dim=0).contiguous(), name="gla.proj")
        self.a2 = Linear(w["a2"], name="gla.a")
        self.a2_bias = w["a2_bias"].contiguous()
        self.norm_weight = w["norm"]
        self.o = Linear(w["o"], name="gla.o")

    graph_class = ()              # grids depend on the batch size only

    def forward(self, h, ctx: StepContext, run: RunView) -> torch.Tensor:
        H, D, Dv, off = self.H, self.D, self.Dv, self.off
        T = h.shape[0]
        proj = self.proj(h, ctx)
        ctx.mark("projections")
        # the decay's projection keeps 32-bit results: its sigmoid's logarithm enters the recurrence
        a = self.a2(proj[:, off["a1"]:off["a1"] + self.rank], ctx, out_dtype=torch.float32)
        read = ctx.ws.get("gla.read", (T, H * Dv), torch.float32)
        kernels.gla(proj[:, off["q"]:off["q"] + H * D], proj[:, off["k"]:off["k"] + H * D], proj[:, off["v"]:off["v"] + H * Dv],
                    a, self.a2_bias, self.tau, D ** -0.5, ctx.state(f"run{run.index}.S"), read, ctx, H, D, Dv)
        ctx.mark("recurrence")
        normed = ctx.ws.get("gla.normed", (T, H * Dv), ctx.dtype)
        kernels.gated_head_norm(read, proj[:, off["g"]:off["g"] + H * Dv], self.norm_weight, self.p["eps"], normed, H, Dv,
                                gate_function="silu")
        term = self.o(normed, ctx, out_dtype=torch.float32)
        ctx.mark("o")
        return term
