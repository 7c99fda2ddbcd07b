"""The gated delta rule with one decay per head and key channel, as the mixer of a layer.

Per head the mixer keeps a matrix S [dim, vdim] per sequence (32-bit) instead of keys and values:
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
with q and k unit vectors per head (q also times dim^-1/2), beta = sigmoid(W_b h) and
g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias)) per key channel.  q, k and v pass a short causal
convolution per channel and SiLU on their way; the convolution's last inputs are per-sequence state as
well.  What is read out is brought to unit root mean square per head, multiplied by a weight and by
sigmoid(W_g2 W_g1 h), and projected back.  The ranks of the two low-rank pairs are the files' own sizes.

q, k, v, b, a1 and g1 are one matrix after loading (each part starting at a multiple of 8 rows), so one
product reads h once.
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


def _round8(n: int) -> int:
    return (n + 7) // 8 * 8


@register_mixer("channel_delta")
class ChannelDeltaRule(Part):
    """params: hidden_size, heads, kv_heads (q and k heads; head h reads q/k head h // (heads / kv_heads)), dim,
    vdim, conv (taps of the short convolution), eps (of the read-out's norm).
    tensors: q, k [kv_heads*dim, E], v [heads*vdim, E], q_conv, k_conv, v_conv [channels, taps], b [heads, E],
    a1 [r, E], a2 [heads*dim, r], dt_bias [heads*dim], A_log [heads], g1 [s, E], g2 [heads*vdim, s], norm [vdim],
    o [E, heads*vdim]."""

    def __init__(self, spec, dtype, device, position=None):
        super().__init__(spec, dtype, device)
        p = self.p
        self.H, self.G, self.D, self.Dv, self.K = p["heads"], p["kv_heads"], p["dim"], p["vdim"], p["conv"]
        if self.H % self.G:
            raise ValueError(f"channel_delta: {self.H} heads are not a multiple of {self.G} q/k heads")
        if not 1 <= self.K <= 16:
            raise ValueError(f"channel_delta: a convolution of {self.K} taps is not supported (1..16)")
        self.conv_channels = 2 * self.G * self.D + self.H * self.Dv

    def kv_spec(self) -> Optional[KVSpec]:
        return None

    def state_spec(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        spec = {"S": ((self.H, self.D, self.Dv), "float32")}
        if self.K > 1:
            spec["conv"] = ((self.K - 1, self.conv_channels), "float32")
        return spec

    def tensor_requests(self) -> List[TensorRequest]:
        E, t = self.p["hidden_size"], self.spec.tensors
        H, G, D, Dv, K = self.H, self.G, self.D, self.Dv, self.K
        rank = max(8, _round8(E // 8))                 # what random weights get where the files' own rank is missing
        return [TensorRequest(t["q"], (G * D, E)), TensorRequest(t["k"], (G * D, E)), TensorRequest(t["v"], (H * Dv, E)),
                TensorRequest(t["q_conv"], (G * D, K), init="uniform:-0.6:0.6"),
                TensorRequest(t["k_conv"], (G * D, K), init="uniform:-0.6:0.6"),
                TensorRequest(t["v_conv"], (H * Dv, K), init="uniform:-0.6:0.6"),
                TensorRequest(t["b"], (H, E)),
                TensorRequest(t["a1"], (-1, E), init_shape=(rank, E)), TensorRequest(t["a2"], (H * D, -1), init_shape=(H * D, rank)),
                TensorRequest(t["dt_bias"], (H * D,), init="uniform:-4:-1"), TensorRequest(t["A_log"], (H,), init="uniform:-1:1"),
                TensorRequest(t["g1"], (-1, E), init_shape=(rank, E)), TensorRequest(t["g2"], (H * Dv, -1), init_shape=(H * Dv, rank)),
                TensorRequest(t["norm"], (Dv,), init="ones"), TensorRequest(t["o"], (E, H * Dv))]

    def load(self, store: WeightStore) -> None:
        w = {local: store.get(r) for local, r in zip(
            ["q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a1", "a2", "dt_bias", "A_log", "g1", "g2", "norm", "o"],
            self.tensor_requests())}
        if w["a1"].shape[0] != w["a2"].shape[1] or w["g1"].shape[0] != w["g2"].shape[1]:
            raise ValueError(f"channel_delta: the low-rank pairs do not fit: a1 {list(w['a1'].shape)} a2 {list(w['a2'].shape)} "
                             f"g1 {list(w['g1'].shape)} g2 {list(w['g2'].shape)}")
        dt = w["q"].dtype
        self.ra, self.rg = w["a1"].shape[0], w["g1"].shape[0]
        # one matrix: q, k, v (contiguous: the convolution runs over all their channels at once), then b, a1, g1,
        # each from a multiple of 8 rows on (zero rows between), so that every slice of the result is aligned
        parts, self.off, rows = [], {}, 0
        for name in ("q", "k", "v"):
            parts.append(w[name].to(dt))
            rows += w[name].shape[0]
        for name in ("b", "a1", "g1"):
            pad = _round8(rows) - rows
            if pad:
                parts.append(torch.zeros(pad, parts[0].shape[1], dtype=dt, device=parts[0].device))
            self.off[name] = rows + pad
            parts.append(w[name].to(dt))
            rows = self.off[name] + w[name].shape[0]
        pad = _round8(rows) - rows
        if pad:
            parts.append(torch.zeros(pad, parts[0].shape[1], dtype=dt, device=parts[0].device))
        self.proj = Linear(torch.cat(parts, dim=0).contiguous(), name="delta.proj")
        self.taps = torch.cat([w["q_conv"], w["k_conv"], w["v_conv"]], dim=0).to(dt).contiguous()
        self.taps_t = self.taps.t().contiguous() if dt == torch.bfloat16 else None      # tap by tap, for 16-byte loads
        self.a2 = Linear(w["a2"], name="delta.a")
        self.g2 = Linear(w["g2"], name="delta.gate")
        self.dt_bias, self.a_log = w["dt_bias"].to(dt).contiguous(), w["A_log"].to(dt).contiguous()
        self.norm_weight = w["norm"]
        self.o = Linear(w["o"], name="delta.o")

    accepts_residual = True
    graph_class = ()              # grids depend on the batch size only

    def forward(self, h, ctx: StepContext, run: RunView, residual=None) -> Optional[torch.Tensor]:
        H, G, D, Dv = self.H, self.G, self.D, self.Dv
        T, C = h.shape[0], self.conv_channels
        proj = self.proj(h, ctx)
        ctx.mark("projections")
        conv = ctx.ws.get("delta.conv", (T, C), ctx.dtype)
        carried = ctx.state(f"run{run.index}.conv") if self.K > 1 else None
        kernels.short_conv_silu(proj[:, :C], self.taps, carried, ctx, conv, taps_t=self.taps_t)
        a = self.a2(proj[:, self.off["a1"]:self.off["a1"] + self.ra], ctx)
        gate = self.g2(proj[:, self.off["g1"]:self.off["g1"] + self.rg], ctx)
        ctx.mark("conv_gates")
        read = ctx.ws.get("delta.read", (T, H * Dv), torch.float32)
        kernels.delta_rule(conv[:, :G * D], conv[:, G * D:2 * G * D], conv[:, 2 * G * D:], proj[:, self.off["b"]:self.off["b"] + H],
                           a, self.dt_bias, self.a_log, ctx.state(f"run{run.index}.S"), read, ctx, H, G, D, Dv, D ** -0.5)
        ctx.mark("recurrence")
        normed = ctx.ws.get("delta.normed", (T, H * Dv), ctx.dtype)
        kernels.gated_head_norm(read, gate, self.norm_weight, self.p["eps"], normed, H, Dv)
        term = self.o(normed, ctx, residual=residual)
        ctx.mark("o")
        return term
