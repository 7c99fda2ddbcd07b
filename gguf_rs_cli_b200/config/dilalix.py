"""Typed configuration of the Dilalix design and its description as parts.

A Dilalix model is a list of layers that norm what a sublayer gives, not what it reads:
x <- x + rms(mixer(x)) w1, then x <- x + rms(ff(x)) w2.  A layer's mixer is either `attention` (grouped-query
attention with an RMS norm per head on q and k, a rotation of the heads' first entries in halves, a window behind
which the sequence's first positions stay visible, values mixed with those of the first such layer, and a sigmoid
gate on the heads' results) or `gla` (gated linear attention: a matrix per head that decays per key channel).  Its
feed-forward is dense (up, exact GELU, down), a mixture of routed experts with an optional shared one, or absent.
config.json gives every size and every constant; ranks of low-rank pairs are the tensors' own sizes.  The
reference knows one architecture only (src/model/config.rs:20-47) and has none of these parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .debonex import NO_POSITION_LIMIT, _get
from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, Run

MIXER_TYPES = ("attention", "gla")


@dataclass(frozen=True)
class DilalixLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]            # None: the layer has no feed-forward


@dataclass(frozen=True)
class DilalixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[DilalixLayer] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "DilalixConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {list(MIXER_TYPES)}")
            out.append(DilalixLayer(kind, _read_mixer(kind, entry.get("mixer"), where + ".mixer"),
                                    _read_mlp(entry.get("mlp"), where + ".mlp")))
        return cls(vocab=_get(raw, "vocab", "the top level"), width=_get(raw, "width", "the top level"),
                   norm_eps=_get(raw.get("norm"), "eps", "'norm'", float), layers=out)


def _read_mixer(kind: str, raw, where: str) -> Dict[str, Any]:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    m: Dict[str, Any] = {k: _get(raw, k, where) for k in ("heads", "dim")}
    m["vdim"] = _get(raw, "vdim", where) if raw.get("vdim") is not None else m["dim"]
    if kind == "gla":
        m["tau"] = _get(raw, "tau", where, float)
        return m
    m["kv_heads"] = _get(raw, "kv_heads", where) if raw.get("kv_heads") is not None else m["heads"]
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    m["scale"] = _get(raw, "scale", where, float) if raw.get("scale") is not None else m["dim"] ** -0.5
    m["v_mix"] = bool(raw.get("v_mix", False))
    m["mask"] = m["rot"] = None
    if raw.get("mask") is not None:
        mask = raw["mask"]
        keep = mask.get("keep_first") if isinstance(mask, dict) else None
        m["mask"] = {"size": _get(mask, "size", where + ".mask"),
                     "keep_first": _get(mask, "keep_first", where + ".mask", positive=False) if keep is not None else 0}
        if m["mask"]["keep_first"] < 0:
            raise ConfigError(f"config.json: {where}.mask.keep_first must not be negative")
    if raw.get("rot") is not None:
        m["rot"] = {"base": _get(raw["rot"], "base", where + ".rot", float), "dims": _get(raw["rot"], "dims", where + ".rot")}
        if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims {m['rot']['dims']} must be even and at most dim {m['dim']}")
    return m


def _read_unit(raw, where: str) -> Dict[str, Any]:
    return {"ff": _get(raw, "ff", where), "limit": _get(raw, "limit", where, float)}


def _read_mlp(raw, where: str) -> Optional[Dict[str, Any]]:
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, dict) else raw
    if kind == "dense":
        return {"kind": "dense", "ff": _get(raw, "ff", where)}
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (dense, moe)")
    r = raw.get("router")
    out = {"kind": "moe", "expert": _read_unit(raw.get("expert"), where + ".expert"),
           "experts": _get(r, "experts", where + ".router"), "top": _get(r, "top", where + ".router"),
           "scale": _get(r, "scale", where + ".router", float) if isinstance(r, dict) and r.get("scale") is not None else 1.0,
           "groups": 1, "keep": 1, "shared": None}
    groups = r.get("groups")
    if groups is not None:
        out["groups"], out["keep"] = _get(groups, "count", where + ".router.groups"), _get(groups, "keep", where + ".router.groups")
    if raw.get("shared") is not None:
        out["shared"] = _read_unit(raw["shared"], where + ".shared")
    if out["experts"] % out["groups"] or out["keep"] > out["groups"]:
        raise ConfigError(f"config.json: {where}.router: {out['experts']} experts do not form {out['groups']} equal groups "
                          f"of which {out['keep']} are kept")
    if out["top"] > out["keep"] * (out["experts"] // out["groups"]):
        raise ConfigError(f"config.json: {where}.router: {out['top']} experts cannot be chosen from {out['keep']} groups of "
                          f"{out['experts'] // out['groups']}")
    return out


def build_dilalix_spec(cfg: DilalixConfig) -> ModelSpec:
    E, layers = cfg.width, []

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(size=E, eps=cfg.norm_eps), {"weight": name})

    first_mixing = next((i for i, l in enumerate(cfg.layers) if l.type == "attention" and l.mixer["v_mix"]), None)
    for i, layer in enumerate(cfg.layers):
        p, m, position = f"l{i}.mix.", layer.mixer, None
        if layer.type == "attention":
            if m["rot"] is not None:
                position = PartSpec("rope", dict(head_dim=m["dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"],
                                                 pairing="half", scaling=None))
            mask = m["mask"] or {"size": None, "keep_first": 0}
            # the first layer that mixes values gives them, the later ones take them; all of them must agree in size
            role = None if not m["v_mix"] else "gives" if i == first_mixing else "takes"
            if role == "takes":
                f = cfg.layers[first_mixing].mixer
                if (f["kv_heads"], f["vdim"]) != (m["kv_heads"], m["vdim"]):
                    raise ConfigError(f"config.json: layers[{i}] mixes its values with those of layers[{first_mixing}], whose "
                                      f"kv_heads and vdim differ")
            mixer = PartSpec("attention", dict(hidden_size=E, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                               v_head_dim=m["vdim"], scale=m["scale"], window=mask["size"],
                                               keep_first=mask["keep_first"], bias=False, head_norm_eps=cfg.norm_eps,
                                               out_gate=True, v_mix=role, v_mix_optional=not m["v_mix"]),
                             {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "g": p + "g", "q_norm": p + "q.norm",
                              "k_norm": p + "k.norm", "v_mix": p + "vmix"})
        else:
            mixer = PartSpec("gla", dict(hidden_size=E, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], tau=m["tau"],
                                         eps=cfg.norm_eps),
                             {n: p + n for n in ("q", "k", "v", "g", "o", "norm", "a1", "a2")} | {"a2_bias": p + "a2.b"})
        norms, ff, q = {"mixer": norm(f"l{i}.norm1")}, None, f"l{i}.mlp."
        mlp = layer.mlp
        if mlp is not None:
            norms["feed_forward"] = norm(f"l{i}.norm2")
            if mlp["kind"] == "dense":
                ff = PartSpec("mlp", dict(hidden_size=E, intermediate_size=mlp["ff"], activation="gelu"),
                              {"up": q + "up", "down": q + "down"})
            else:
                shared = mlp["shared"]
                ff = PartSpec("moe", dict(hidden_size=E, experts=mlp["experts"], top=mlp["top"], groups=mlp["groups"],
                                          keep=mlp["keep"], scale=mlp["scale"], expert_ff=mlp["expert"]["ff"],
                                          limit=mlp["expert"]["limit"], shared_ff=shared["ff"] if shared else None,
                                          shared_limit=shared["limit"] if shared else None),
                              {"router": q + "router", "experts": q + "e", "shared": q + "shared"})
        layers.append(LayerSpec(block="outnorm", mixer=mixer, feed_forward=ff, norms=norms, position=position))
    spec = ModelSpec(
        architecture="Dilalix", vocab_size=cfg.vocab, hidden_size=E,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab, hidden_size=E), {"weight": "embed"}),
        layers=layers, schedule=[Run(i) for i in range(len(layers))], final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=E, tied_to=None, tied=False), {"weight": "head"}),
        max_position=NO_POSITION_LIMIT)
    spec.validate()
    return spec


register_architecture("Dilalix", DilalixConfig, build_dilalix_spec, "dilalix")
