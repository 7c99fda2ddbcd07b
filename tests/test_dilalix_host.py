"""Dilalix without a device: the configuration reader and what it refuses, the model as parts and tensor names, the
cache of a window that keeps the first positions, random weights, and the plain implementation against closed forms
and against itself."""
import math

import pytest
import torch

from tests import plain_dilalix as P
from tests.dilalix_util import CONFIGS, config, weights


def test_config_reads_every_size_and_constant():
    from gguf_rs_cli_b200.config import load_config
    arch, cfg = load_config(config("small"))
    assert arch.name == "Dilalix" and (cfg.vocab, cfg.width, cfg.norm_eps) == (211, 72, 1e-5)
    assert [l.type for l in cfg.layers] == ["gla", "attention", "attention", "attention"]
    assert cfg.layers[2].mlp is None and cfg.layers[0].mlp == {"kind": "dense", "ff": 136}
    assert cfg.layers[1].mixer["mask"] == {"size": 13, "keep_first": 5} and cfg.layers[1].mixer["rot"] == {"base": 100.0, "dims": 16}
    assert cfg.layers[1].mlp["groups"] == 3 and cfg.layers[1].mlp["keep"] == 2 and cfg.layers[1].mlp["shared"] == {"ff": 28, "limit": 0.8}
    spec = arch.build_spec(cfg)
    assert all(l.block == "outnorm" for l in spec.layers)
    assert spec.layers[2].feed_forward is None and set(spec.layers[2].norms) == {"mixer"}
    a = spec.layers[1].mixer.params
    assert (a["window"], a["keep_first"], a["v_head_dim"], a["scale"], a["head_norm_eps"], a["out_gate"]) == (13, 5, 40, 0.3, 1e-5, True)
    # the first layer that mixes values gives them, later ones take them, one in between does neither
    assert [l.mixer.params.get("v_mix") for l in spec.layers] == [None, "gives", None, "takes"]
    assert spec.layers[1].position.params["pairing"] == "half" and spec.layers[1].position.params["rotary_dim"] == 16
    assert spec.layers[0].mixer.kind == "gla" and spec.layers[0].mixer.params["tau"] == 7.0
    assert spec.layers[0].feed_forward.kind == "mlp" and spec.layers[0].feed_forward.params["activation"] == "gelu"
    m = spec.layers[1].feed_forward.params
    assert (m["experts"], m["top"], m["groups"], m["keep"], m["scale"], m["expert_ff"], m["limit"], m["shared_ff"], m["shared_limit"]) == \
        (12, 3, 3, 2, 2.5, 20, 1.2, 28, 0.8)


def test_config_defaults_and_refusals():
    from gguf_rs_cli_b200.config import ConfigError, load_config
    raw = config("wide")
    _, cfg = load_config(raw)
    assert cfg.layers[0].mlp["groups"] == 1 and cfg.layers[0].mlp["keep"] == 1 and cfg.layers[0].mlp["shared"] is None
    for path, value, text in [(("layers", 0, "type"), "conv", "type"), (("layers", 0, "mixer", "heads"), 7, "kv_heads"),
                              (("layers", 0, "mixer", "rot", "dims"), 66, "rot.dims"), (("layers", 1, "mlp", "kind"), "glu", "kind"),
                              (("layers", 2, "mlp", "router", "top"), 5, "chosen"), (("layers", 2, "mlp", "router", "experts"), 9, "groups"),
                              (("layers", 2, "mixer", "vdim"), 32, "mixes its values")]:
        bad = config("wide")
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            arch, c = load_config(bad)
            arch.build_spec(c)
    bad = config("wide")
    del bad["layers"][1]["mixer"]["tau"]
    with pytest.raises(ConfigError, match="tau"):
        load_config(bad)


def test_tensor_names_and_shapes():
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.models.decoder import tensor_requests
    for name in CONFIGS:
        arch, cfg = load_config(config(name))
        reqs = {r.name: r for r in tensor_requests(arch.build_spec(cfg))}
        w = weights(name)
        assert set(reqs) == set(w)
        for n, r in reqs.items():
            assert len(r.shape) == w[n].dim() and all(a in (-1, b) for a, b in zip(r.shape, w[n].shape)), n
    assert reqs["l2.mix.vmix"].shape == () and reqs["l3.mix.a1"].shape == (-1, 256)


def test_random_weights_folder_round_trip(tmp_path):
    from gguf_rs_cli_b200.weights import write_random_model
    from gguf_rs_cli_b200.weights.safetensors_io import SafetensorsFile
    write_random_model(str(tmp_path), config("small"), seed=3)
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    names = set(f.names())
    assert "l1.mlp.e11.down" in names and "l1.mlp.shared.gate" in names and "l0.mix.a2.b" in names and "l2.mlp.up" not in names
    assert f.shape("l1.mix.vmix") == () and "l2.mix.vmix" not in names        # a layer that mixes nothing writes no scalar


# ------------------------------------------------------------------- the cache
def test_cache_keeps_the_first_pages_in_front_of_the_ring():
    from gguf_rs_cli_b200.cache.cache import Cache, CacheLayout, KVSpec
    layout = CacheLayout(kv={0: KVSpec(2, 16, window=40, keep_first=70), 1: KVSpec(2, 16, window=40), 2: KVSpec(2, 16)})
    c = Cache(layout, n_slots=3, n_tokens=4096, max_len=2048, max_step_tokens=32)
    kept, ring, full = (c.groups[c.group_of_run[r][0]] for r in (0, 1, 2))
    assert (kept.head_pages, kept.ring_pages) == (2, 3) and (ring.head_pages, ring.ring_pages) == (0, 3) and full.ring_pages == 32
    s = c.open()
    for n in (32, 32, 32, 32, 32, 32, 32, 32, 32, 32, 32, 32):
        c.reserve([s], [n])
        c.advance([s], [n])
        c.check()
    assert len(kept.tables[s]) == 5 and len(ring.tables[s]) == 3 and len(full.tables[s]) == 6
    first = list(kept.tables[s])
    for _ in range(20):
        c.reserve([s], [32])
        c.advance([s], [32])
    assert kept.tables[s] == first                       # the ring goes round, the table stays
    c.close(s)
    c.check()
    assert kept.pool.held_count == 0
    # a sequence too short for the ring never wraps: the kept pages take what the table has
    small = Cache(CacheLayout(kv={0: KVSpec(1, 8, window=10, keep_first=200)}), n_slots=1, n_tokens=128, max_len=128)
    g = small.groups[0]
    assert g.head_pages + g.ring_pages == 2 and g.head_pages == 1


def table_entry(pos, ring, head):
    pg = pos // 64
    return pg if pg < head else head + (pg - head) % ring


def test_positions_of_a_window_never_share_a_table_entry():
    """The rule the kernels use (first `head` entries for ever, the ring behind them): whatever a step of up to 32
    tokens can still see lies in entries of its own."""
    window, keep, step = 40, 70, 32
    head, ring = 2, 3
    for p in range(0, 900):
        lo = max(0, p - step + 1 - window + 1)
        seen = list(range(0, min(keep, lo))) + list(range(lo, p + 1))
        pages = {}
        for j in seen:
            e = table_entry(j, ring, head)
            assert pages.setdefault(e, j // 64) == j // 64, (p, j)


# ------------------------------------------------- the plain implementation itself
def test_visible_is_a_window_and_the_first_positions():
    assert [j for j in range(12) if P.visible(11, j, 3, 2)] == [0, 1, 9, 10, 11]
    assert [j for j in range(12) if P.visible(3, j, 3, 2)] == [0, 1, 2, 3]
    assert [j for j in range(12) if P.visible(11, j, 3, 0)] == [9, 10, 11]
    assert [j for j in range(12) if P.visible(5, j, 100, 0)] == [0, 1, 2, 3, 4, 5]


def test_rotation_in_halves_is_a_complex_rotation():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 2, 10, generator=g, dtype=torch.float64)
    y = P.rotate_half(x, 100.0, 6)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    for t in (1, 8):
        for i in range(3):
            a = t * 100.0 ** (-2.0 * i / 6)
            z = complex(x[t, 1, i], x[t, 1, i + 3]) * complex(math.cos(a), math.sin(a))
            assert abs(z.real - float(y[t, 1, i])) < 1e-12 and abs(z.imag - float(y[t, 1, i + 3])) < 1e-12
    # a score depends on the distance only
    q, k = torch.randn(1, 1, 6, generator=g, dtype=torch.float64), torch.randn(1, 1, 6, generator=g, dtype=torch.float64)
    def score(i, j):
        return float((P.rotate_half(q.expand(i + 1, 1, 6), 50.0, 6)[i] * P.rotate_half(k.expand(j + 1, 1, 6), 50.0, 6)[j]).sum())
    assert abs(score(9, 4) - score(25, 20)) < 1e-12


def test_recurrence_is_a_decayed_sum_of_outer_products():
    g = torch.Generator().manual_seed(1)
    n, D, Dv = 6, 3, 2
    q, k, a = (torch.randn(n, D, generator=g, dtype=torch.float64) for _ in range(3))
    a, v = torch.sigmoid(a), torch.randn(n, Dv, generator=g, dtype=torch.float64)
    out, S = P.decayed_outer_recurrence(q, k, v, a)
    for t in range(n):
        want = torch.zeros(Dv, dtype=torch.float64)
        for s in range(t + 1):
            decay = torch.ones(D, dtype=torch.float64)
            for u in range(s + 1, t + 1):
                decay = decay * a[u]
            want += (q[t] * decay * k[s]).sum() * v[s]
        assert torch.allclose(out[t], want)
    # carried over a cut
    o1, S1 = P.decayed_outer_recurrence(q[:4], k[:4], v[:4], a[:4])
    o2, S2 = P.decayed_outer_recurrence(q[4:], k[4:], v[4:], a[4:], S1)
    assert torch.allclose(torch.cat([o1, o2]), out) and torch.allclose(S2, S)


def test_route_keeps_groups_by_their_two_best():
    s = torch.tensor([0.9, 0.1, 0.1, 0.1,   0.5, 0.6, 0.1, 0.1,   0.45, 0.45, 0.45, 0.45])
    # marks 1.0, 1.1, 0.9: with one group kept, the second; its two best and then its next
    assert P.route(s, 3, 3, 1) == [5, 4, 6]
    assert P.route(s, 3, 3, 2) == [0, 5, 4]              # groups 1 and 0
    assert P.route(s, 2, 1, 1) == [0, 5]                 # one group: plain top-k
    assert P.route(s, 1, 12, 12) == [0]                  # groups of one expert


def test_expert_clamps_and_feed_forwards():
    h = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    w = {"x.gate": torch.tensor([[3.0, 0.0], [0.0, 1.0]]), "x.up": torch.tensor([[0.0, -2.0], [5.0, 0.0]]), "x.down": torch.eye(2),
         "y.up": torch.tensor([[0.5, 0.0]]), "y.down": torch.tensor([[2.0], [0.0]])}
    got = P.expert(h, w, "x.", 1.5)
    g0, g1 = 1.5, -2.0                                   # min(3, 1.5); min(-2, 1.5): only the top is cut
    u0, u1 = 1.5, 1.5                                    # clamp(4), clamp(5)
    want = [g0 / (1 + math.exp(-1.702 * g0)) * (u0 + 1), g1 / (1 + math.exp(-1.702 * g1)) * (u1 + 1)]
    assert torch.allclose(got, torch.tensor([want], dtype=torch.float64))
    z = 0.5
    assert torch.allclose(P.dense_ff(h, w, "y."), torch.tensor([[2 * 0.5 * z * (1 + math.erf(z / math.sqrt(2))), 0.0]], dtype=torch.float64))


def test_every_mechanism_moves_the_logits():
    """Leaving a mechanism out of the plain model changes its logits by far more than rounding: the tests that
    compare the package with it would see the same omission in the package."""
    cfg, w = config("small"), weights("small")
    toks = torch.randint(0, cfg["vocab"], (60,), generator=torch.Generator().manual_seed(5)).tolist()
    base = P.forward(cfg, w, toks)
    ref = float(base.abs().max())

    def moved(change_cfg=None, change_w=None):
        c, ww = config("small"), dict(w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(ww)
        return float((P.forward(c, ww, toks) - base).abs().max()) / ref

    assert moved(lambda c: c["layers"][1]["mixer"]["mask"].update(keep_first=0)) > 0.02          # the kept first positions
    assert moved(lambda c: c["layers"][3]["mixer"]["mask"].update(size=8)) > 0.02                # a window one longer
    assert moved(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8)) > 0.02                 # the rotated width
    assert moved(lambda c: c["layers"][3]["mixer"].update(v_mix=False)) > 0.02                   # mixed values
    assert moved(lambda c: c["layers"][0]["mixer"].update(tau=3.0)) > 0.02                       # the decay's root
    assert moved(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=3)) > 0.02      # the groups
    assert moved(lambda c: c["layers"][1]["mlp"]["expert"].update(limit=5.0)) > 0.02             # the clamp
    assert moved(lambda c: c["layers"][1]["mlp"].update(shared=None)) > 0.02                     # the shared expert
    assert moved(None, lambda ww: ww.update({"l1.mix.q.norm": torch.ones(24)})) > 0.02           # the heads' norm weight
    assert moved(None, lambda ww: ww.update({"l1.mix.g": torch.zeros_like(ww["l1.mix.g"])})) > 0.02     # the gate
