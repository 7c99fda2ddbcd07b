"""Small Dilalix configurations with weights of the tests' own making, as the plain implementation's dict and as an
engine of the package.

The configurations differ from each other in every size and constant, and avoid coincidences that would hide a
fault: heads and key/value heads differ, key and value sizes differ, fewer entries are rotated than a head holds, the
window is shorter than a page in one and longer in the other, more first positions are kept than the window holds in
one, a layer has no feed-forward, one mixture has no shared expert and a single group, one attention layer mixes no
values.  Scales are chosen so that attention is peaked and decays are slow.
"""
import copy
import functools

import torch

from tests import plain_dilalix as P

SMALL = {
    "architecture": "Dilalix", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "gla", "mixer": {"heads": 3, "dim": 24, "vdim": 40, "tau": 7.0}, "mlp": {"kind": "dense", "ff": 136}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 40, "scale": 0.3, "v_mix": True,
                                        "mask": {"size": 13, "keep_first": 5}, "rot": {"base": 100.0, "dims": 16}},
         "mlp": {"kind": "moe", "expert": {"ff": 20, "limit": 1.2},
                 "router": {"experts": 12, "top": 3, "scale": 2.5, "groups": {"count": 3, "keep": 2}},
                 "shared": {"ff": 28, "limit": 0.8}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.4, "v_mix": False,
                                        "mask": {"size": 30, "keep_first": 0}, "rot": {"base": 50.0, "dims": 16}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 40, "scale": 0.25, "v_mix": True,
                                        "mask": {"size": 7, "keep_first": 9}, "rot": {"base": 1000.0, "dims": 8}},
         "mlp": {"kind": "dense", "ff": 100}},
    ],
}
SMALL_RANKS = {0: 12}

# Sizes that reach the tensor-core products (multiples of 8) and the tiled attention kernels (keys and values of 64
# entries); more than a page of kept first positions; a mixture with one group, one chosen expert and no shared one.
WIDE = {
    "architecture": "Dilalix", "vocab": 520, "width": 256, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.2, "v_mix": True,
                                        "mask": {"size": 70, "keep_first": 70}, "rot": {"base": 5000.0, "dims": 64}},
         "mlp": {"kind": "moe", "expert": {"ff": 64, "limit": 3.0}, "router": {"experts": 4, "top": 1, "scale": 1.0}}},
        {"type": "gla", "mixer": {"heads": 2, "dim": 128, "vdim": 64, "tau": 16.0}, "mlp": {"kind": "dense", "ff": 360}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.2, "v_mix": True,
                                        "mask": {"size": 100, "keep_first": 3}, "rot": {"base": 5000.0, "dims": 32}},
         "mlp": {"kind": "moe", "expert": {"ff": 48, "limit": 2.0},
                 "router": {"experts": 8, "top": 4, "scale": 1.5, "groups": {"count": 4, "keep": 2}},
                 "shared": {"ff": 96, "limit": 1.5}}},
        {"type": "gla", "mixer": {"heads": 4, "dim": 48, "vdim": 136, "tau": 4.0}, "mlp": None},
    ],
}
WIDE_RANKS = {1: 32, 3: 16}



def without_experts(cfg):
    """The same model with a dense feed-forward in every mixture's place: nothing in it decides between near ties, so
    bfloat16 results stay within rounding of the plain ones however long the sequence."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer.get("mlp") and layer["mlp"]["kind"] == "moe":
            layer["mlp"] = {"kind": "dense", "ff": 8 * layer["mlp"]["expert"]["ff"]}
    return cfg


CONFIGS = {"small": (SMALL, SMALL_RANKS), "wide": (WIDE, WIDE_RANKS),
           "small-dense": (without_experts(SMALL), SMALL_RANKS), "wide-dense": (without_experts(WIDE), WIDE_RANKS)}


def scenario(name, dtype):
    """The configuration a scenario of many steps runs in: in bfloat16 the one without routed experts (a router's
    choice between two close scores may fall otherwise than in the plain model, and through kept first positions and
    recurrent states every later token would see it); 32-bit runs keep the experts."""
    return name if dtype == "float32" else name + "-dense"


def config(name):
    return copy.deepcopy(CONFIGS[name][0])


def make_weights(cfg, ranks, seed=0, gain=1.3):
    """name -> float32 tensor holding bfloat16 values.  Projections N(0, gain^2/in), so that rows stay of order one;
    norms near the identity with noise; decays slow (biases of 2 to 6 in front of the sigmoid), so that the first tokens
    still show at the end of a long sequence; router rows large enough for clear choices."""
    g = torch.Generator().manual_seed(seed)
    E, w = cfg["width"], {}

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def vec(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)

    w["embed"] = torch.randn(cfg["vocab"], E, generator=g) * 0.7
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        w[f"l{i}.norm1"] = vec(E)
        if layer["type"] == "gla":
            H, D, Dv, r = m["heads"], m["dim"], m["vdim"], ranks[i]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = mat(H * D, E, gain), mat(H * D, E, gain), mat(H * Dv, E, gain), mat(H * Dv, E, gain)
            w[p + "a1"], w[p + "a2"] = mat(r, E), mat(H * D, r, gain)
            w[p + "a2.b"] = torch.rand(H * D, generator=g) * 4.0 + 2.0
            w[p + "norm"], w[p + "o"] = vec(Dv), mat(E, H * Dv)
        else:
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = mat(H * D, E, gain), mat(G * D, E, gain), mat(G * Dv, E, gain), mat(H * Dv, E, gain)
            w[p + "q.norm"], w[p + "k.norm"] = vec(D) * 1.3, vec(D) * 1.3
            w[p + "vmix"] = torch.tensor(0.2 + 0.5 * float(torch.rand((), generator=g)))
            w[p + "o"] = mat(E, H * Dv)
        mlp = layer.get("mlp")
        if mlp:
            q = f"l{i}.mlp."
            w[f"l{i}.norm2"] = vec(E)
            if mlp["kind"] == "dense":
                w[q + "up"], w[q + "down"] = mat(mlp["ff"], E, 1.5), mat(E, mlp["ff"])
            else:
                F = mlp["expert"]["ff"]
                w[q + "router"] = mat(mlp["router"]["experts"], E, 3.0)
                for e in range(mlp["router"]["experts"]):
                    w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = mat(F, E, 2.0), mat(F, E, 2.0), mat(E, F)
                if mlp.get("shared"):
                    Fs = mlp["shared"]["ff"]
                    w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = mat(Fs, E, 2.0), mat(Fs, E, 2.0), mat(E, Fs)
    w["final.norm"] = vec(E)
    w["head"] = mat(cfg["vocab"], E)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def weights(name, seed=0):
    cfg, ranks = CONFIGS[name]
    return make_weights(cfg, ranks, seed)


def build(cfg, w, dtype):
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.weights import TensorSource
    return _build(copy.deepcopy(cfg), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="test weights"),
                  dtype, "cuda:0")


@functools.lru_cache(maxsize=None)
def llm(name, dtype, seed=0):
    return build(CONFIGS[name][0], weights(name, seed), dtype)


def new_engine(name, dtype, n_tokens=2048, n_slots=8, **kw):
    from gguf_rs_cli_b200.engine.step import Engine
    return Engine(llm(name, dtype).model, n_tokens=n_tokens, n_slots=n_slots, **kw)


def tokens_of(name, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, CONFIGS[name][0]["vocab"], (n,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name, n, seed):
    return P.forward(CONFIGS[name][0], weights(name), tokens_of(name, n, seed), dtype=torch.float64).float()
