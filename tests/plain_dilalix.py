"""A plain, slow implementation of the Dilalix design, one function per mechanism, written from the
design's equations with torch on the CPU.  It is the oracle of the tests and shares no code with the
package: whole sequences, no cache, loops over heads and tokens.

Notation.  x [n, E] is a sequence's residual stream, positions 0..n-1; a sublayer reads x itself and its
result is normed before it is added: x <- x + rms(sub(x)) w.  W are stored [out, in] and applied as
h W^T.  `w` is a dict of tensors by the names of the model folder; `p` a prefix such as "l3.mix.".
"""
import math

import torch


def lin(x, w):
    return x @ w.to(x.dtype).T


def rms(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(x.dtype)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


# ------------------------------------------------------------------ attention
def rotate_half(x, base, dims):
    """x [n, heads, D]; the first `dims` entries of each head: entry i pairs with entry i + dims/2, the pair
    (a, b) at position t becomes (a cos - b sin, b cos + a sin) of the angle t base^(-2i/dims)."""
    n, half = x.shape[0], dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = torch.arange(n, dtype=x.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j: a window of `size` positions that ends at
    i, and the first `keep_first` positions of the sequence for ever."""
    return j <= i and (i - j < size or j < keep_first)


def windowed_softmax_attention(q, k, v, scale, size, keep_first):
    """q [n, H, D], k [n, G, D], v [n, G, Dv] -> [n, H, Dv]; head h reads key/value head h // (H/G)."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=q.dtype)
    for i in range(n):
        js = [j for j in range(i + 1) if visible(i, j, size, keep_first)]
        for h in range(H):
            g = h // (H // G)
            a = torch.softmax(k[js, g] @ q[i, h] * scale, dim=0)
            out[i, h] = a @ v[js, g]
    return out


def attention(h, w, p, m, eps, v_first=None):
    """The attention mixer.  m: the layer's mixer sizes.  v_first None: this layer does not mix values (or is the
    first that does); else the first such layer's values [n, G, Dv].  Returns (result [n, E], this layer's values
    before mixing)."""
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(lin(h, w[p + "q"]).reshape(n, H, D), w[p + "q.norm"], eps)
    k = rms(lin(h, w[p + "k"]).reshape(n, G, D), w[p + "k.norm"], eps)
    q = rotate_half(q, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half(k, m["rot"]["base"], m["rot"]["dims"])
    v = lin(h, w[p + "v"]).reshape(n, G, Dv)
    raw = v
    if v_first is not None:
        lam = w[p + "vmix"].to(h.dtype)
        v = (1.0 - lam) * v + lam * v_first
    o = windowed_softmax_attention(q, k, v, m["scale"], m["mask"]["size"], m["mask"]["keep_first"])
    o = o.reshape(n, H * Dv) * torch.sigmoid(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"]), raw


# ------------------------------------------------------- gated linear attention
def decayed_outer_recurrence(q, k, v, alpha, S=None):
    """One head.  q, k, alpha [n, D], v [n, Dv]; S [D, Dv] or None (zeros).  Per token: S <- diag(alpha) S + k v^T;
    out = S^T q.  Returns (out, S)."""
    n, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=q.dtype) if S is None else S.clone()
    out = torch.zeros(n, v.shape[1], dtype=q.dtype)
    for t in range(n):
        S = alpha[t][:, None] * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out, S


def gla(h, w, p, m, eps):
    n = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = lin(h, w[p + "q"]).reshape(n, H, D) * D ** -0.5
    k = lin(h, w[p + "k"]).reshape(n, H, D)
    v = lin(h, w[p + "v"]).reshape(n, H, Dv)
    z = lin(lin(h, w[p + "a1"]), w[p + "a2"]) + w[p + "a2.b"].to(h.dtype)
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).reshape(n, H, D)
    o = torch.stack([decayed_outer_recurrence(q[:, i], k[:, i], v[:, i], alpha[:, i])[0] for i in range(H)], dim=1)
    o = rms(o, w[p + "norm"], eps).reshape(n, H * Dv) * silu(lin(h, w[p + "g"]))
    return lin(o, w[p + "o"])


# ---------------------------------------------------------------- feed-forward
def dense_ff(h, w, p):
    return lin(gelu_erf(lin(h, w[p + "up"])), w[p + "down"])


def expert(h, w, p, limit):
    g = torch.clamp(lin(h, w[p + "gate"]), max=limit)
    u = torch.clamp(lin(h, w[p + "up"]), min=-limit, max=limit)
    return lin(g * torch.sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def route(scores, top, n_groups, keep):
    """scores [experts] of one token -> the chosen experts (indices), largest score first.  The experts form
    n_groups equal groups of neighbours; a group's mark is the sum of its two largest scores (of its one score if
    it has but one expert); only experts of the `keep` groups with the largest marks can be chosen."""
    n = scores.numel()
    size = n // n_groups
    marks = []
    for g in range(n_groups):
        part = sorted(scores[g * size:(g + 1) * size].tolist(), reverse=True)
        marks.append(sum(part[:2]))
    kept = sorted(range(n_groups), key=lambda g: (-marks[g], g))[:keep]
    allowed = [e for e in range(n) if e // size in kept]
    return sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]


def moe_ff(h, w, p, mlp, chosen=None, scores_out=None):
    """chosen: per token the experts to use in place of the router's choice (a caller that follows another
    implementation through a near tie); scores_out: a list that receives the scores [n, experts]."""
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    scores = torch.sigmoid(lin(h, w[p + "router"]))
    if scores_out is not None:
        scores_out.append(scores)
    for t in range(h.shape[0]):
        picked = route(scores[t], r["top"], groups["count"], groups["keep"]) if chosen is None else list(chosen[t])
        s = scores[t][picked]
        weights = s / (s.sum() + 1e-20) * r["scale"]
        for e, a in zip(picked, weights):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


# ------------------------------------------------------------------- the model
def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None, routes=None, scores_out=None):
    """Logits [n, vocab] of one sequence.  layers_out: a list that receives the residual stream after each layer.
    routes {layer: experts per token} replaces the routers' choices; scores_out {layer: scores} receives theirs."""
    eps = cfg["norm"]["eps"]
    w = {k: v.to(dtype) for k, v in w.items()}
    x = w["embed"][torch.tensor(tokens)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            y, raw = attention(x, w, p, m, eps, v_first if m.get("v_mix") else None)
            if m.get("v_mix") and v_first is None:
                v_first = raw
        elif layer["type"] == "gla":
            y = gla(x, w, p, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms(y, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = dense_ff(x, w, f"l{i}.mlp.")
            else:
                got = []
                y = moe_ff(x, w, f"l{i}.mlp.", mlp, None if routes is None else routes.get(i), got)
                if scores_out is not None:
                    scores_out[i] = got[0]
            x = x + rms(y, w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(rms(x, w["final.norm"], eps), w["head"])
