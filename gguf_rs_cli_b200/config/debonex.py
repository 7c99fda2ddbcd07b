"""Typed configuration of the Debonex design and its description as parts.

A Debonex model is a list of pre-norm layers, each with one of three mixers (`channel_delta`: a gated
delta rule with a decay per key channel; `latent_attention`: attention over one cached latent row per
position; `attention`: grouped-query attention with normalised q and k and a query temperature, without a
rotation) and an optional dense gated feed-forward with GELU's tanh form.  Norms are dynamic tanh.  The
embedding and the logits carry a constant factor each.  config.json gives every size and every constant;
ranks of low-rank pairs are the tensors' own sizes.  The reference knows one architecture only
(src/model/config.rs:20-47) and has none of these mixers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, Run

NO_POSITION_LIMIT = 1 << 30          # the design names no longest sequence: the cache's size is the limit


def _get(raw: Dict[str, Any], key: str, where: str, kind=int, positive: bool = True):
    if not isinstance(raw, dict) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json: missing key '{key}' in {where}")
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' in {where} must be a number, got {v!r}")
    if kind is int:
        if int(v) != v:
            raise ConfigError(f"config.json: '{key}' in {where} must be a whole number, got {v!r}")
        v = int(v)
    else:
        v = float(v)
    if positive and not v > 0:
        raise ConfigError(f"config.json: '{key}' in {where} must be positive, got {v!r}")
    return v


def _factor(raw, key: str, where: str) -> float:
    """A constant factor; a configuration that does not name it has none (1)."""
    if not isinstance(raw, dict) or raw.get(key) is None:
        return 1.0
    return _get(raw, key, where, float, positive=False)


MIXER_TYPES = ("channel_delta", "latent_attention", "attention")


@dataclass(frozen=True)
class DebonexLayer:
    type: str
    mixer: Dict[str, Any]
    ff: Optional[int]               # size of the feed-forward's hidden layer, None: the layer has none


@dataclass(frozen=True)
class DebonexConfig:
    vocab: int
    width: int
    embedding_scale: float
    logit_scale: float
    norm_eps: float
    layers: List[DebonexLayer] = field(default_factory=list)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "DebonexConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {list(MIXER_TYPES)}")
            out.append(DebonexLayer(kind, _read_mixer(kind, entry.get("mixer"), where + ".mixer"), _read_mlp(entry.get("mlp"), where + ".mlp")))
        return cls(vocab=_get(raw, "vocab", "the top level"), width=_get(raw, "width", "the top level"),
                   embedding_scale=_factor(raw.get("embedding"), "scale", "'embedding'"),
                   logit_scale=_factor(raw, "logit_scale", "the top level"),
                   norm_eps=_get(raw.get("norm"), "eps", "'norm'", float), layers=out)


def _read_mlp(raw, where: str) -> Optional[int]:
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") != "dense":
        raise ConfigError(f"config.json: {where}.kind {raw.get('kind') if isinstance(raw, dict) else raw!r} is not supported (dense)")
    return _get(raw, "ff", where)


def _read_mixer(kind: str, raw, where: str) -> Dict[str, Any]:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    m: Dict[str, Any] = {k: _get(raw, k, where) for k in ("heads", "dim", "vdim")}
    if kind == "channel_delta":
        m["kv_heads"], m["conv"] = _get(raw, "kv_heads", where), _get(raw, "conv", where)
        if m["conv"] > 16:
            raise ConfigError(f"config.json: {where}.conv {m['conv']} exceeds the 16 taps that are supported")
    elif kind == "attention":
        m["kv_heads"], m["scale"] = _get(raw, "kv_heads", where), _get(raw, "scale", where, float)
        m["q_temp"] = None
        if raw.get("q_temp") is not None:
            m["q_temp"] = {"coef": _get(raw["q_temp"], "coef", where + ".q_temp", float, positive=False),
                           "every": _get(raw["q_temp"], "every", where + ".q_temp")}
    else:
        m["kv_rank"], m["rot_dim"], m["scale"] = _get(raw, "kv_rank", where), _get(raw, "rot_dim", where), _get(raw, "scale", where, float)
        rot = raw.get("rot")
        m["rot"] = {"base": _get(rot, "base", where + ".rot", float), "dims": _get(rot, "dims", where + ".rot")}
        if m["rot_dim"] % 2 or m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
            raise ConfigError(f"config.json: {where}: rot_dim {m['rot_dim']} and rot.dims {m['rot']['dims']} must be even, "
                              f"rot.dims at most rot_dim")
    if "kv_heads" in m and m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    return m


def build_debonex_spec(cfg: DebonexConfig) -> ModelSpec:
    E, layers = cfg.width, []

    def norm(name: str) -> PartSpec:
        return PartSpec("dyt", dict(size=E), {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})

    for i, layer in enumerate(cfg.layers):
        p, m, position = f"l{i}.mix.", layer.mixer, None
        if layer.type == "channel_delta":
            mixer = PartSpec("channel_delta", dict(hidden_size=E, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"],
                                                   vdim=m["vdim"], conv=m["conv"], eps=cfg.norm_eps),
                             {n: p + n for n in ("q", "k", "v", "b", "a1", "a2", "dt_bias", "A_log", "g1", "g2", "norm", "o")}
                             | {n + "_conv": p + n + ".conv" for n in ("q", "k", "v")})
        elif layer.type == "latent_attention":
            position = PartSpec("rope", dict(head_dim=m["rot_dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"],
                                             pairing="interleaved", scaling=None))
            mixer = PartSpec("latent_attention", dict(hidden_size=E, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                                                      vdim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], eps=cfg.norm_eps),
                             {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                              "o": p + "o"})
        else:
            mixer = PartSpec("attention", dict(hidden_size=E, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                                               head_dim=m["dim"], v_head_dim=m["vdim"], scale=m["scale"], window=None,
                                               bias=False, qk_norm_eps=cfg.norm_eps, q_temp=m["q_temp"]),
                             {n: p + n for n in ("q", "k", "v", "o")})
        norms, ff = {"mixer": norm(f"l{i}.norm1")}, None
        if layer.ff is not None:
            norms["feed_forward"] = norm(f"l{i}.norm2")
            ff = PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=layer.ff, activation="gelu_tanh"),
                          {n: f"l{i}.mlp.{n}" for n in ("gate", "up", "down")})
        layers.append(LayerSpec(block="prenorm", mixer=mixer, feed_forward=ff, norms=norms, position=position))
    spec = ModelSpec(
        architecture="Debonex", vocab_size=cfg.vocab, hidden_size=E,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab, hidden_size=E, scale=cfg.embedding_scale), {"weight": "embed"}),
        layers=layers, schedule=[Run(i) for i in range(len(layers))], final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=E, tied_to=None, tied=False,
                                      logit_scale=cfg.logit_scale), {"weight": "head"}),
        max_position=NO_POSITION_LIMIT)
    spec.validate()
    return spec


register_architecture("Debonex", DebonexConfig, build_debonex_spec, "debonex")
