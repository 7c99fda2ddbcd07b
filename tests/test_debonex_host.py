"""Debonex without a device: the configuration reader and what it refuses, the model as parts and tensor
names, random weights, and the plain implementation against closed forms and against itself."""
import copy
import math

import pytest
import torch

from tests import plain_debonex as P
from tests.debonex_util import CONFIGS, config, weights


def test_config_reads_every_size_and_constant():
    from gguf_rs_cli_b200.config import load_config
    arch, cfg = load_config(config("small"))
    assert arch.name == "Debonex" and (cfg.vocab, cfg.width) == (211, 72)
    assert (cfg.embedding_scale, cfg.logit_scale, cfg.norm_eps) == (2.0, 0.25, 1e-6)
    assert [l.type for l in cfg.layers] == ["attention", "channel_delta", "latent_attention", "channel_delta"]
    assert cfg.layers[1].ff is None and cfg.layers[0].ff == 136
    assert cfg.layers[0].mixer["q_temp"] == {"coef": 0.7, "every": 5}
    assert cfg.layers[2].mixer["rot"] == {"base": 100.0, "dims": 16}
    spec = arch.build_spec(cfg)
    assert spec.layers[1].feed_forward is None and set(spec.layers[1].norms) == {"mixer"}
    assert spec.layers[2].position.params["pairing"] == "interleaved" and spec.layers[2].position.params["rotary_dim"] == 16
    assert spec.layers[0].mixer.params["v_head_dim"] == 40 and spec.layers[0].mixer.params["qk_norm_eps"] == 1e-6
    assert spec.embedding.params["scale"] == 2.0 and spec.head.params["logit_scale"] == 0.25
    assert spec.layers[0].feed_forward.params["activation"] == "gelu_tanh"


def test_config_without_factors_has_none():
    from gguf_rs_cli_b200.config import load_config
    raw = config("small")
    del raw["embedding"], raw["logit_scale"]
    raw["layers"][0]["mixer"].pop("q_temp")
    raw["layers"][3].pop("mlp")
    _, cfg = load_config(raw)
    assert (cfg.embedding_scale, cfg.logit_scale) == (1.0, 1.0)
    assert cfg.layers[0].mixer["q_temp"] is None and cfg.layers[3].ff is None


@pytest.mark.parametrize("path,value,match", [
    (("layers", 0, "type"), "conv_mixer", "not one of"),
    (("layers", 1, "mixer", "kv_heads"), 3, "not a multiple"),
    (("layers", 1, "mixer", "conv"), 40, "16 taps"),
    (("layers", 2, "mixer", "rot", "dims"), 30, "rot.dims"),
    (("layers", 2, "mixer", "kv_rank"), None, "missing key 'kv_rank'"),
    (("layers", 0, "mlp", "kind"), "experts", "not supported"),
    (("layers", 0, "mixer", "q_temp", "every"), 0, "must be positive"),
    (("norm", "eps"), 0.0, "must be positive"),
    (("vocab",), 2.5, "whole number"),
    (("layers",), [], "at least one layer"),
])
def test_config_errors_name_the_key(path, value, match):
    from gguf_rs_cli_b200.config import ConfigError, load_config
    raw = config("small")
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        load_config(raw)


def test_tensor_names_shapes_and_ranks_left_to_the_file():
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.models.decoder import tensor_requests
    from gguf_rs_cli_b200.weights.loader import TensorSource, WeightError, WeightStore, shape_matches
    for name in CONFIGS:
        arch, cfg = load_config(config(name))
        reqs = tensor_requests(arch.build_spec(cfg))
        w = weights(name)
        assert {r.name for r in reqs} == set(w)
        assert all(shape_matches(tuple(r.shape), tuple(w[r.name].shape)) for r in reqs)
        store = WeightStore(TensorSource(tensors=w), torch.float32, "cpu")
        store.check(reqs)
        bad = dict(w)
        bad["l1.mix.a2"] = torch.zeros(7, 3)
        del bad["final.norm.alpha"]
        bad["l9.extra"] = torch.zeros(1)
        with pytest.raises(WeightError) as e:
            WeightStore(TensorSource(tensors=bad), torch.float32, "cpu").check(reqs)
        assert "final.norm.alpha" in e.value.missing and "l9.extra" in e.value.unexpected
        assert [n for n, _, _ in e.value.wrong_shape] == ["l1.mix.a2"]


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from gguf_rs_cli_b200.weights import write_random_model
    from gguf_rs_cli_b200.weights.loader import TensorSource
    folder = write_random_model(str(tmp_path / "m"), config("small"), seed=3)
    src = TensorSource.from_folder(folder)
    assert src.shape("l1.mix.a1")[1] == 72 and src.shape("l1.mix.a2")[1] == src.shape("l1.mix.a1")[0]
    assert src.shape("l0.norm1.alpha") == () and float(src.get("l0.norm1.alpha")) == 0.5
    assert float(src.get("l1.mix.dt_bias").float().max()) <= -1.0
    assert "l1.norm2" not in src.names() and "l0.norm2" in src.names()


def test_cache_layout_of_the_three_mixers():
    from gguf_rs_cli_b200.cache.cache import Cache, KVSpec
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.models.decoder import Decoder
    arch, cfg = load_config(config("small"))
    layout = Decoder(arch.build_spec(cfg), torch.float32, "meta").cache_layout()
    assert layout.kv == {0: KVSpec(4, 24, None, 40), 2: KVSpec(1, 64, None, 0)}
    assert layout.states == {"run1.S": ((4, 24, 40), "float32"), "run1.conv": ((2, 2 * 2 * 24 + 4 * 40), "float32"),
                             "run3.S": ((2, 40, 24), "float32"), "run3.conv": ((1, 2 * 40 + 2 * 24), "float32")}
    cache = Cache(layout, n_slots=3, n_tokens=256)
    a, b = cache.open(), cache.open()
    cache.reserve([a, b], [70, 3])
    cache.advance([a, b], [70, 3])
    assert [len(g.tables[a]) for g in cache.groups] == [2, 2]
    cache.close(a)
    cache.check()


# ------------------------------------------------------------ the plain implementation
def test_plain_dyt_gelu_and_temperature_by_hand():
    x = torch.tensor([[0.5, -2.0]])
    got = P.dyt(x, torch.tensor([2.0, 1.0]), torch.tensor([0.1, -0.1]), torch.tensor(0.5))
    assert torch.allclose(got, torch.tensor([[2 * math.tanh(0.25) + 0.1, math.tanh(-1.0) - 0.1]]))
    z = torch.tensor([1.0])
    assert abs(float(P.gelu_tanh(z)) - 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715))) < 1e-7
    # the temperature is 1 until position every - 2 and grows at every - 1, where floor((p + 1) / every) first is 1
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "q_temp": {"coef": 0.5, "every": 3}}
    eye = torch.eye(2)
    w = {"q": eye, "k": eye, "v": eye, "o": eye}
    h = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [1.0, -1.0]])
    got = P.normed_attention(h, w, "", m, 1e-12)
    t2 = 1 + 0.5 * math.log(2.0)
    q2 = torch.tensor([1.0, 1.0]) * t2                       # unit root mean square already
    k = torch.stack([torch.tensor([2 ** 0.5, 0.0]), torch.tensor([0.0, 2 ** 0.5]), torch.tensor([1.0, 1.0])])
    p = torch.softmax(k @ q2, 0)
    assert torch.allclose(got[2], p @ h[:3], atol=1e-6)
    assert torch.allclose(got[0], h[0]) and not torch.allclose(got[2], torch.softmax(k @ (q2 / t2), 0) @ h[:3], atol=1e-3)


def test_plain_delta_rule_first_steps_by_hand():
    """One head, dim 2, vdim 1, no convolution taps but the current one, first two tokens worked out."""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "conv": 1}
    w = {"q": torch.tensor([[1.0, 0.0], [0.0, 1.0]]), "k": torch.tensor([[0.0, 1.0], [1.0, 0.0]]), "v": torch.tensor([[1.0, 1.0]]),
         "q.conv": torch.ones(2, 1), "k.conv": torch.ones(2, 1), "v.conv": torch.ones(1, 1), "b": torch.zeros(1, 2),
         "a1": torch.zeros(1, 2), "a2": torch.zeros(2, 1), "dt_bias": torch.tensor([0.0, 1.0]), "A_log": torch.tensor([0.5]),
         "g1": torch.zeros(1, 2), "g2": torch.zeros(1, 1), "norm": torch.ones(1), "o": torch.ones(1, 1)}
    h = torch.tensor([[1.0, 2.0], [0.5, -1.0]], dtype=torch.float64)
    got = P.channel_delta(h, {k: v.double() for k, v in w.items()}, "", m, 1e-12)
    silu = lambda z: z / (1 + math.exp(-z))
    unit = lambda a, b: (a / math.sqrt(a * a + b * b + 1e-6), b / math.sqrt(a * a + b * b + 1e-6))
    decay = [math.exp(-math.exp(0.5) * math.log1p(math.exp(z))) for z in (0.0, 1.0)]
    S, outs = [0.0, 0.0], []
    for x0, x1 in h.tolist():
        q = unit(silu(x0), silu(x1))
        q = (q[0] / math.sqrt(2), q[1] / math.sqrt(2))
        k = unit(silu(x1), silu(x0))
        v = silu(x0 + x1)
        S = [decay[0] * S[0], decay[1] * S[1]]
        u = 0.5 * (v - (S[0] * k[0] + S[1] * k[1]))
        S = [S[0] + k[0] * u, S[1] + k[1] * u]
        outs.append(S[0] * q[0] + S[1] * q[1])
    # one value per head: the norm leaves its sign, the gate sigmoid(0) halves it
    want = torch.tensor([[0.5 * o / math.sqrt(o * o + 1e-12)] for o in outs], dtype=torch.float64)
    assert torch.allclose(got, want, atol=1e-9)


def test_plain_latent_attention_equals_its_absorbed_form():
    """The scores and values through the latent's space (what the package computes) equal the per-head keys
    and values of the plain form."""
    cfg, w = config("small"), weights("small")
    m, p, eps = cfg["layers"][2]["mixer"], "l2.mix.", cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(5)
    n = 19
    h = torch.randn(n, cfg["width"], generator=g, dtype=torch.float64)
    wd = {k: v.double() for k, v in w.items()}
    want = P.latent_attention(h, wd, p, m, eps)
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    q = P.lin(h, wd[p + "q"]).reshape(n, H, D + R)
    dkv = P.lin(h, wd[p + "dkv"])
    c = P.rms_unit(dkv[:, :C], eps) * wd[p + "dkv.norm"]
    k_rot = P.rotate_interleaved(dkv[:, None, C:], pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    q_rot = P.rotate_interleaved(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    out = torch.zeros(n, H, Dv, dtype=torch.float64)
    for hd in range(H):
        q_lat = q[:, hd, :D] @ wd[p + "uk"][hd * D:(hd + 1) * D]                       # [n, C]
        s = (q_lat @ c.T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = P.causal_softmax_mix(s, c) @ wd[p + "uv"][hd * Dv:(hd + 1) * Dv].T
    assert torch.allclose(P.lin(out.reshape(n, H * Dv), wd[p + "o"]), want, atol=1e-10)


def test_plain_model_is_causal_and_sensitive():
    """A later token changes nothing earlier; and the things the tests are to catch do change the logits:
    the first token (through slow decays) at the end of a long sequence, the temperature, the rotation."""
    cfg, w = config("small"), weights("small", 0, True)
    toks = [(7 * i + 3) % cfg["vocab"] for i in range(150)]
    full = P.forward(cfg, w, toks, dtype=torch.float64)
    assert torch.allclose(P.forward(cfg, w, toks[:60], dtype=torch.float64), full[:60], atol=1e-9)
    scale = float(full[-1].abs().max())
    other = P.forward(cfg, w, [toks[0] + 1] + toks[1:], dtype=torch.float64)
    assert float((other[-1] - full[-1]).abs().max()) > 1e-3 * scale
    for change in ("temp", "rot"):
        c2 = copy.deepcopy(cfg)
        if change == "temp":
            c2["layers"][0]["mixer"]["q_temp"] = None
        else:
            c2["layers"][2]["mixer"]["rot"]["base"] = 90.0
        assert float((P.forward(c2, w, toks, dtype=torch.float64)[-1] - full[-1]).abs().max()) > 1e-2 * scale, change
