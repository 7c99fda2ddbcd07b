"""A plain, slow implementation of the Debonex design, one function per mechanism, written
from the design's equations with torch on the CPU.  It is the oracle of the tests and
shares no code with the package: whole sequences, no cache, loops over heads and tokens.

Notation.  h [n, E] are a sequence's rows in front of a mixer, positions 0..n-1.
W are stored [out, in] and applied as h W^T.  `w` is a dict of tensors by the names of
the model folder; `p` a prefix such as "l3.mix.".
"""
import math

import torch


def lin(x, w):
    return x @ w.to(x.dtype).T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x, weight, bias, alpha):
    """Dynamic tanh: tanh(alpha x) * weight + bias; no statistics of x."""
    return torch.tanh(alpha.to(x.dtype) * x) * weight.to(x.dtype) + bias.to(x.dtype)


def dense_ff(h, gate, up, down):
    return lin(gelu_tanh(lin(h, gate)) * lin(h, up), down)


def causal_conv_silu(x, taps):
    """x [n, C], taps [C, K] with the last column on the current row; rows before the first are zero."""
    n, C = x.shape
    K = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(n):
        for j in range(K):
            src = t - (K - 1 - j)
            if src >= 0:
                out[t] += x[src] * taps[:, j].to(x.dtype)
    return silu(out)


def delta_recurrence(q, k, v, beta, decay, S=None):
    """One head.  q, k [n, D] (unit vectors, q already scaled), v [n, Dv], beta [n], decay [n, D]; S [D, Dv] or None
    (zeros).  Per token: S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; out = S^T q.  Returns (out, S)."""
    n, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype) if S is None else S.clone()
    out = torch.zeros(n, v.shape[1], dtype=q.dtype)
    for t in range(n):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out, S


def channel_delta(h, w, p, m, eps):
    """The gated delta rule with one decay per head and key channel.  m: the layer's mixer sizes."""
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(lin(h, w[p + "q"]), w[p + "q.conv"]).reshape(n, G, D)
    k = causal_conv_silu(lin(h, w[p + "k"]), w[p + "k.conv"]).reshape(n, G, D)
    v = causal_conv_silu(lin(h, w[p + "v"]), w[p + "v.conv"]).reshape(n, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(h, w[p + "b"]))                                       # [n, H]
    a = lin(lin(h, w[p + "a1"]), w[p + "a2"]) + w[p + "dt_bias"].to(h.dtype)       # [n, H*D]
    rate = torch.exp(w[p + "A_log"].to(h.dtype))                                   # [H]
    decay = torch.exp(-rate[None, :, None] * softplus(a).reshape(n, H, D))         # [n, H, D]
    gate = torch.sigmoid(lin(lin(h, w[p + "g1"]), w[p + "g2"])).reshape(n, H, Dv)
    out = torch.zeros(n, H, Dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd], _ = delta_recurrence(q[:, g], k[:, g], v[:, hd], beta[:, hd], decay[:, hd])
    out = rms_unit(out, eps) * w[p + "norm"].to(h.dtype) * gate
    return lin(out.reshape(n, H * Dv), w[p + "o"])


def rotate_interleaved(x, pos, dims, base):
    """x [n, heads, d]: the first `dims` entries of every head are rotated, pair (2i, 2i+1) by pos * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = (pos.to(torch.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :])
    # the product is taken in the working precision, as a 32-bit implementation would take it
    if x.dtype == torch.float32:
        ang = (pos.to(torch.float32)[:, None] * (float(base) ** (-2.0 * i / dims)).to(torch.float32)[None, :])
    cs, sn = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
    return out


def causal_softmax_mix(scores, values):
    """scores [n, n] (query, key); values [n, d]: softmax over keys j <= i, then the mix of values."""
    n = scores.shape[0]
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = scores.masked_fill(~mask, float("-inf"))
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return (e / e.sum(-1, keepdim=True)) @ values


def latent_attention(h, w, p, m, eps):
    """Keys and values of all heads come from one latent row per position and one rotated key part that
    all heads share."""
    n = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    q = lin(h, w[p + "q"]).reshape(n, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_interleaved(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    dkv = lin(h, w[p + "dkv"])
    c = rms_unit(dkv[:, :C], eps) * w[p + "dkv.norm"].to(h.dtype)
    k_rot = rotate_interleaved(dkv[:, None, C:], pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]      # [n, R]
    k_plain = lin(c, w[p + "uk"]).reshape(n, H, D)
    v = lin(c, w[p + "uv"]).reshape(n, H, Dv)
    out = torch.zeros(n, H, Dv, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = causal_softmax_mix(s, v[:, hd])
    return lin(out.reshape(n, H * Dv), w[p + "o"])


def normed_attention(h, w, p, m, eps):
    """Grouped-query attention without rotation: q and k are brought to unit root mean square per head, and
    the query at position t is multiplied by 1 + coef * ln(floor((t + 1) / every) + 1)."""
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit(lin(h, w[p + "q"]).reshape(n, H, D), eps)
    k = rms_unit(lin(h, w[p + "k"]).reshape(n, G, D), eps)
    v = lin(h, w[p + "v"]).reshape(n, G, Dv)
    qt = m.get("q_temp")
    if qt:
        t = torch.arange(n)
        temp = 1.0 + qt["coef"] * torch.log(torch.floor((t + 1) / qt["every"]) + 1.0)
        q = q * temp.to(h.dtype)[:, None, None]
    out = torch.zeros(n, H, Dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = causal_softmax_mix((q[:, hd] @ k[:, g].T) * m["scale"], v[:, g])
    return lin(out.reshape(n, H * Dv), w[p + "o"])


MIXERS = {"channel_delta": channel_delta, "latent_attention": latent_attention, "attention": normed_attention}


def norm_of(w, name, x):
    return dyt(x, w[name], w[name + ".b"], w[name + ".alpha"])


def forward(cfg, w, tokens, dtype=torch.float32, layers_out=None):
    """Logits [n, vocab] of one sequence.  layers_out: a list that receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](norm_of(w, p + "norm1", x), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + dense_ff(norm_of(w, p + "norm2", x), w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(norm_of(w, "final.norm", x), w["head"]) * cfg["logit_scale"]
