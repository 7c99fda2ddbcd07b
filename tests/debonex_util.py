"""Small Debonex configurations with weights of the tests' own making, as the plain implementation's dict
and as an engine of the package.

The configurations differ from each other in every size and constant, and avoid coincidences that would hide
a fault: heads and q/k heads differ, key and value sizes differ, the two low-rank pairs have different ranks,
fewer dimensions are rotated than the rotated part holds, one layer has no feed-forward, the query
temperature changes every few positions.  Scales are chosen so that attention is peaked.
"""
import copy
import functools

import torch

from tests import plain_debonex as P

SMALL = {
    "architecture": "Debonex", "vocab": 211, "width": 72, "embedding": {"scale": 2.0}, "logit_scale": 0.25,
    "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 24, "vdim": 40, "scale": 0.5,
                                        "q_temp": {"coef": 0.7, "every": 5}}, "mlp": {"kind": "dense", "ff": 136}},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 3}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "rot_dim": 24, "rot": {"base": 100.0, "dims": 16},
                                               "kv_rank": 40, "vdim": 20, "scale": 0.4}, "mlp": {"kind": "dense", "ff": 100}},
        {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 24, "conv": 2},
         "mlp": {"kind": "dense", "ff": 80}},
    ],
}
SMALL_RANKS = {1: (12, 20), 3: (8, 5)}          # layer -> ranks of the decay pair and of the gate pair

# Sizes that reach the tensor-core products (multiples of 8), the tiled attention kernels (keys and values of 64
# entries per head, in both attention mixers) and the delta rule's shapes with several lanes per column; a query
# temperature that is absent; as many q/k heads as heads.
WIDE = {
    "architecture": "Debonex", "vocab": 520, "width": 256, "embedding": {"scale": 1.5}, "logit_scale": 2.0,
    "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 32, "rot_dim": 32, "rot": {"base": 5000.0, "dims": 32},
                                               "kv_rank": 192, "vdim": 64, "scale": 0.25}, "mlp": {"kind": "dense", "ff": 360}},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 4, "dim": 128, "vdim": 64, "conv": 4},
         "mlp": {"kind": "dense", "ff": 256}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.5, "q_temp": None},
         "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 48, "vdim": 136, "conv": 1},
         "mlp": {"kind": "dense", "ff": 64}},
    ],
}
WIDE_RANKS = {1: (32, 16), 3: (16, 24)}

CONFIGS = {"small": (SMALL, SMALL_RANKS), "wide": (WIDE, WIDE_RANKS)}


def config(name):
    return copy.deepcopy(CONFIGS[name][0])


def make_weights(cfg, ranks, seed=0, slow_decay=False, gain=1.4):
    """name -> float32 tensor holding bfloat16 values.  Projections N(0, 1/in), so that rows stay of order one;
    norms near the identity with noise; decays between fast and slow (slow_decay: all slow, so that the first
    tokens still show at the end of a long sequence)."""
    g = torch.Generator().manual_seed(seed)
    E, w = cfg["width"], {}

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def norm(name):
        w[name] = 1.0 + 0.2 * torch.randn(E, generator=g)
        w[name + ".b"] = 0.1 * torch.randn(E, generator=g)
        w[name + ".alpha"] = torch.tensor(0.4 + 0.4 * float(torch.rand((), generator=g)))

    w["embed"] = torch.randn(cfg["vocab"], E, generator=g) * 0.7
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        norm(f"l{i}.norm1")
        if layer["type"] == "channel_delta":
            H, G, D, Dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = ranks[i]
            w[p + "q"], w[p + "k"], w[p + "v"] = mat(G * D, E, gain), mat(G * D, E, gain), mat(H * Dv, E, gain)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                w[p + n + ".conv"] = torch.rand(c, K, generator=g) * 1.2 - 0.4
            w[p + "b"] = mat(H, E, gain)
            w[p + "a1"], w[p + "a2"] = mat(ra, E), mat(H * D, ra, gain)
            w[p + "dt_bias"] = torch.rand(H * D, generator=g) * (1.0 if slow_decay else 4.0) - (7.0 if slow_decay else 4.0)
            w[p + "A_log"] = torch.rand(H, generator=g) * 2.0 - (3.0 if slow_decay else 1.5)
            w[p + "g1"], w[p + "g2"] = mat(rg, E), mat(H * Dv, rg, gain)
            w[p + "norm"] = 1.0 + 0.2 * torch.randn(Dv, generator=g)
            w[p + "o"] = mat(E, H * Dv)
        elif layer["type"] == "latent_attention":
            H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "q"], w[p + "dkv"] = mat(H * (D + R), E, gain), mat(C + R, E, gain)
            w[p + "dkv.norm"] = 1.0 + 0.2 * torch.randn(C, generator=g)
            w[p + "uk"], w[p + "uv"], w[p + "o"] = mat(H * D, C, gain), mat(H * Dv, C), mat(E, H * Dv)
        else:
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "o"] = mat(H * D, E), mat(G * D, E), mat(G * Dv, E), mat(E, H * Dv)
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            norm(f"l{i}.norm2")
            w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"] = mat(F, E, 1.5), mat(F, E), mat(E, F)
    norm("final.norm")
    w["head"] = mat(cfg["vocab"], E)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def weights(name, seed=0, slow_decay=False):
    cfg, ranks = CONFIGS[name]
    return make_weights(cfg, ranks, seed, slow_decay)


def build(cfg, w, dtype):
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.weights import TensorSource
    return _build(copy.deepcopy(cfg), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="test weights"),
                  dtype, "cuda:0")


@functools.lru_cache(maxsize=None)
def llm(name, dtype, seed=0, slow_decay=False):
    return build(CONFIGS[name][0], weights(name, seed, slow_decay), dtype)


def new_engine(name, dtype, n_tokens=2048, n_slots=8, **kw):
    from gguf_rs_cli_b200.engine.step import Engine
    return Engine(llm(name, dtype, **kw).model, n_tokens=n_tokens, n_slots=n_slots)


def tokens_of(name, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, CONFIGS[name][0]["vocab"], (n,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name, n, seed, slow_decay=False):
    return P.forward(CONFIGS[name][0], weights(name, 0, slow_decay), tokens_of(name, n, seed), dtype=torch.float64).float()
