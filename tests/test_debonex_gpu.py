"""Debonex in the package against the plain implementation (tests/plain_debonex.py), in 32-bit and in
bfloat16: every mechanism alone, whole prompts against token-by-token decoding, prompts cut into portions
down to two tokens, unequal batches against each request alone, slots and pages that are used again, keys
far back and at page borders, the first tokens of a sequence, long decoding, and greedy generation through
the package's entry point."""
import copy

import pytest
import torch

from tests import plain_debonex as P
from tests.debonex_util import CONFIGS, build, config, llm, make_weights, new_engine, plain_logits, tokens_of, weights
from tests.gpu_util import TOL

pytestmark = pytest.mark.gpu


def assert_close(got, want, dtype, what=""):
    """32-bit: the largest error against the largest value of the compared block, 1e-4 (the sharp test: a key left
    out, a state not carried or a wrong edge moves results by far more).  bfloat16: rounding of the intermediates
    moves single values of these small, peaked models by a few percent, so the root mean square of the error is held
    to 5% of the block's and the largest error to 10% of the largest value."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err, ref = float((got - want).abs().max()), max(float(want.abs().max()), 1e-6)
    if dtype == "float32":
        assert err <= TOL[dtype] * ref, f"{what}: max error {err:.3e} against max |ref| {ref:.3e} ({dtype})"
        return
    rms_err, rms_ref = float((got - want).pow(2).mean().sqrt()), max(float(want.pow(2).mean().sqrt()), 1e-6)
    assert rms_err <= 5e-2 * rms_ref and err <= 1e-1 * ref, \
        f"{what}: rms error {rms_err:.3e} of {rms_ref:.3e}, max error {err:.3e} of {ref:.3e} ({dtype})"
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = ["small", "wide"]


def entry(slot, tokens, want):
    from gguf_rs_cli_b200.engine.step import Entry
    return Entry(slot, tokens, want)


def tdtype(name):
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def plan_for(eng, lens):
    slots = [eng.open() for _ in lens]
    ctx, _, _ = eng.plan([entry(s, [1] * n, ()) for s, n in zip(slots, lens)])
    return ctx, slots


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_embedding_norm_feed_forward_head_alone(name, dtype):
    from gguf_rs_cli_b200.parts.base import Stream
    cfg, w, model = config(name), weights(name), llm(name, dtype).model
    eng = new_engine(name, dtype)
    ctx, _ = plan_for(eng, [9, 4])
    toks = tokens_of(name, 13, 1)
    x = model.embedding.forward(torch.tensor(toks, dtype=torch.int32, device=DEV), ctx)
    want_x = w["embed"][toks] * cfg["embedding"]["scale"]
    assert torch.allclose(x.cpu(), want_x, atol=1e-6)
    g = torch.Generator().manual_seed(2)
    pend = (torch.randn(13, cfg["width"], generator=g) * 0.3).to(tdtype(dtype))
    stream = Stream(x.clone())
    stream.pending = pend.to(DEV)
    got = model.layers[0].norms["mixer"].apply(stream, ctx)
    assert_close(got, P.norm_of(w, "l0.norm1", want_x + pend.float()), dtype, "dynamic tanh")
    assert stream.pending is None and torch.allclose(stream.x.cpu(), want_x + pend.float(), atol=1e-6)
    h = torch.randn(13, cfg["width"], generator=g).to(tdtype(dtype))
    got = model.layers[0].feed_forward.forward(h.to(DEV), ctx)
    assert_close(got, P.dense_ff(h.float(), w["l0.mlp.gate"], w["l0.mlp.up"], w["l0.mlp.down"]), dtype, "feed-forward")
    rows = torch.tensor([12, 3], dtype=torch.int32, device=DEV)
    hf = model.final_norm.apply(stream, ctx, rows=rows, buffer="t.final")
    logits = model.head.forward(hf, ctx)
    want = P.lin(P.norm_of(w, "final.norm", (want_x + pend.float())[[12, 3]]), w["head"]) * cfg["logit_scale"]
    assert logits.dtype == torch.float32
    assert_close(logits, want, dtype, "head")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_mixer_alone_in_an_unequal_batch(name, dtype):
    cfg, w, model = config(name), weights(name), llm(name, dtype).model
    eng = new_engine(name, dtype)
    lens = [70, 5, 1]
    ctx, _ = plan_for(eng, lens)
    g = torch.Generator().manual_seed(3)
    h = torch.randn(sum(lens), cfg["width"], generator=g).to(tdtype(dtype))
    for i, layer in enumerate(cfg["layers"]):
        got = model.layers[i].mixer.forward(h.to(DEV), ctx, eng.runs[i])
        want, t0 = [], 0
        for n in lens:
            want.append(P.MIXERS[layer["type"]](h[t0:t0 + n].float(), w, f"l{i}.mix.", layer["mixer"], cfg["norm"]["eps"]))
            t0 += n
        assert_close(got, torch.cat(want), dtype, f"{name} layer {i} ({layer['type']})")


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_carries_its_inputs_over_cuts(taps, wide):
    """The convolution kernel alone: a sequence fed in pieces of 1, 2, 3 and more rows gives what it gives whole,
    beside a second sequence in the same step.  wide: bfloat16 rows of 40 channels, which the kernel of 16-byte
    accesses takes; else 32-bit rows of 37."""
    from gguf_rs_cli_b200 import kernels
    from gguf_rs_cli_b200.engine.step import Engine
    eng = new_engine("small", "float32")
    g = torch.Generator().manual_seed(taps)
    C, n = (40, 23) if wide else (37, 23)
    x = torch.randn(2, n, C, generator=g)
    w = torch.randn(C, taps, generator=g)
    if wide:
        x, w = x.to(torch.bfloat16), w.to(torch.bfloat16)
    state = torch.zeros(eng.cache.n_slots, max(taps - 1, 1), C, device=DEV) if taps > 1 else None
    slots = [eng.open(), eng.open()]
    fed, got = [0, 0], [[], []]
    for cut_a, cut_b in [(1, 2), (2, 1), (3, 9), (1, 1), (16, 10)]:
        ctx, _, _ = eng.plan([entry(slots[0], [1] * cut_a, ()), entry(slots[1], [1] * cut_b, ())])
        rows = torch.cat([x[0, fed[0]:fed[0] + cut_a], x[1, fed[1]:fed[1] + cut_b]]).to(DEV)
        out = torch.empty_like(rows)
        kernels.short_conv_silu(rows, w.to(DEV), state, ctx, out, taps_t=w.t().contiguous().to(DEV) if wide else None)
        eng.cache.advance(slots, [cut_a, cut_b])
        got[0].append(out[:cut_a].float().cpu())
        got[1].append(out[cut_a:].float().cpu())
        fed = [fed[0] + cut_a, fed[1] + cut_b]
    assert fed == [n, n]
    for b in range(2):
        want = P.causal_conv_silu(x[b].float(), w.float())
        assert torch.allclose(torch.cat(got[b]), want, atol=2e-2 * float(want.abs().max()) if wide else 1e-5)


@pytest.mark.parametrize("D,Dv,H,G", [(8, 5, 2, 1), (24, 40, 4, 2), (300, 36, 2, 2), (600, 20, 1, 1), (1100, 12, 1, 1)])
def test_delta_rule_kernel_at_every_shape_of_its_walk(D, Dv, H, G):
    """The recurrence alone in 32-bit, at key sizes that take 8, 16, 32 and 64 rows a lane, sizes that are no multiple
    of four, fewer q/k heads than heads; two sequences in a step, then both continued from their states."""
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "float32")
    g = torch.Generator().manual_seed(D)
    lens = [[9, 4], [1, 3]]
    n = [sum(x) for x in zip(*lens)]
    raw = {b: dict(q=torch.randn(n[b], G * D, generator=g), k=torch.randn(n[b], G * D, generator=g),
                   v=torch.randn(n[b], H * Dv, generator=g), beta=torch.randn(n[b], H, generator=g),
                   a=torch.randn(n[b], H * D, generator=g) * 2) for b in range(2)}
    dt_bias, a_log = torch.rand(H * D, generator=g) * 4 - 5, torch.rand(H, generator=g) * 2 - 1.5
    want = []
    for b in range(2):
        r = raw[b]
        q, k = r["q"].reshape(-1, G, D), r["k"].reshape(-1, G, D)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        decay = torch.exp(-torch.exp(a_log)[None, :, None] * P.softplus(r["a"] + dt_bias).reshape(-1, H, D))
        beta = torch.sigmoid(r["beta"])
        want.append(torch.stack([P.delta_recurrence(q[:, h // (H // G)], k[:, h // (H // G)], r["v"].reshape(-1, H, Dv)[:, h],
                                                    beta[:, h], decay[:, h])[0] for h in range(H)], dim=1).reshape(-1, H * Dv))
    state = torch.zeros(eng.cache.n_slots, H, D, Dv, device=DEV)
    slots, fed, got = [eng.open(), eng.open()], [0, 0], [[], []]
    for cut in lens:
        ctx, _, _ = eng.plan([entry(s, [1] * c, ()) for s, c in zip(slots, cut)])
        rows = {name: torch.cat([raw[b][name][fed[b]:fed[b] + cut[b]] for b in range(2)]).to(DEV) for name in ("q", "k", "v", "beta", "a")}
        qkv = torch.cat([rows["q"], rows["k"], rows["v"]], dim=1).contiguous()
        out = torch.empty(sum(cut), H * Dv, device=DEV)
        kernels.delta_rule(qkv[:, :G * D], qkv[:, G * D:2 * G * D], qkv[:, 2 * G * D:], rows["beta"], rows["a"], dt_bias.to(DEV),
                           a_log.to(DEV), state, out, ctx, H, G, D, Dv, D ** -0.5)
        eng.cache.advance(slots, cut)
        got[0].append(out[:cut[0]].cpu())
        got[1].append(out[cut[0]:].cpu())
        fed = [fed[0] + cut[0], fed[1] + cut[1]]
    for b in range(2):
        assert_close(torch.cat(got[b]), want[b], "float32", f"delta rule D={D} sequence {b}")


# ------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_request_alone(name, dtype):
    eng = new_engine(name, dtype)
    for n, seed in [(1, 1), (2, 2), (5, 3), (64, 4), (65, 5), (131, 6)]:
        s = eng.open()
        got = eng.step([entry(s, tokens_of(name, n, seed), range(n))])
        eng.close(s)
        assert_close(got, plain_logits(name, n, seed), dtype, f"{name} whole n={n}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(name, dtype):
    """Decoding from an empty sequence: the convolution's zeros before the start, the empty state, the temperature's
    first change, and a page border on the way."""
    eng = new_engine(name, dtype)
    n, seed = 70, 8
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    s = eng.open()
    for i in range(n):
        got = eng.step([entry(s, [toks[i]], [0])])
        assert_close(got[0], want[i], dtype, f"{name} position {i} decoded alone")
    eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_in_portions(name, dtype):
    eng = new_engine(name, dtype)
    n, seed = 150, 9
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    for cuts in ([2, 3, 59, 1, 64, 21], [63, 2, 2, 83], [64, 64, 22], [1, 2, 147]):
        assert sum(cuts) == n
        s, at = eng.open(), 0
        for c in cuts:
            got = eng.step([entry(s, toks[at:at + c], range(c))])
            assert_close(got, want[at:at + c], dtype, f"{name} portion {at}..{at + c} of {cuts}")
            at += c
        eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_slots_and_pages_used_again(name, dtype):
    """Batches one after another in an engine with few slots and pages: what a finished request held (pages of keys,
    the recurrent state, the convolution's inputs) goes to the next one, which must not see it."""
    eng = new_engine(name, dtype, n_tokens=64 * 7, n_slots=4)
    decode, seed = 6, 100
    for lens in ([5, 9, 13, 70], [1, 7, 20, 33], [64, 65, 2], [129, 3]):
        reqs = []
        for n in lens:
            seed += 1
            total = n + decode
            reqs.append(dict(toks=tokens_of(name, total, seed), want=plain_logits(name, total, seed), n=n,
                             keep=decode - (seed % 3), slot=eng.open(), fed=0))
        got = eng.step([entry(r["slot"], r["toks"][:r["n"]], [r["n"] - 1]) for r in reqs])
        for i, r in enumerate(reqs):
            assert_close(got[i], r["want"][r["n"] - 1], dtype, f"{name} prompt of {r['n']} in batch {lens}")
            r["fed"] = r["n"]
        live = list(reqs)
        for step in range(decode):
            live = [r for r in live if r["fed"] < r["n"] + r["keep"]]
            for r in reqs:
                if r not in live and r["slot"] is not None:
                    eng.close(r["slot"])
                    r["slot"] = None
            if not live:
                break
            got = eng.step([entry(r["slot"], [r["toks"][r["fed"]]], [0]) for r in live])
            for i, r in enumerate(live):
                assert_close(got[i], r["want"][r["fed"]], dtype, f"{name} step {step} of prompt {r['n']}")
                r["fed"] += 1
        for r in reqs:
            if r["slot"] is not None:
                eng.close(r["slot"])
        eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_with_slow_decays(dtype):
    """A short prompt and 300 tokens one by one: with slow decays the state still holds the first tokens, and keys
    of the first page are still looked at from the fifth."""
    name = "small"
    eng = new_engine(name, dtype, slow_decay=True)
    n, seed = 310, 12
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed, True)
    s = eng.open()
    eng.step([entry(s, toks[:10], [])])
    for i in range(10, n):
        got = eng.step([entry(s, [toks[i]], [0])])
        if i % 7 == 0 or i in (63, 64, 65, 127, 128, 129, 255, 256, 257) or i > n - 5:
            assert_close(got[0], want[i], dtype, f"position {i} of a long decode")
    eng.close(s)


# ------------------------------------------------------------ keys far back
def far_key_case(kind, n, far):
    """An attention layer whose last query matches the key at position `far` as well as its own and no other: q and k
    read the first half of a row with the same matrix, v reads the second half; the two rows agree in the first
    half only, and the scale lets these two scores stand out.  Half of the last row's result is then the far
    position's value.  Returns (config, weights, rows in front of the mixer)."""
    cfg = config("small")
    cfg["layers"] = [cfg["layers"][0]]
    m = cfg["layers"][0]["mixer"]
    m.update(heads=2, kv_heads=2, dim=24, vdim=40, scale=1.5, q_temp={"coef": 0.3, "every": 50})
    w = make_weights(cfg, {}, seed=far)
    half = cfg["width"] // 2
    w["l0.mix.q"][:, half:] = 0
    w["l0.mix.k"] = w["l0.mix.q"].clone()
    w["l0.mix.v"][:, :half] = 0
    g = torch.Generator().manual_seed(n + far)
    h = torch.randn(n, cfg["width"], generator=g).to(torch.bfloat16).float()
    h[far, :half] = h[n - 1, :half]
    return cfg, w, h


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 2, 63, 64, 65, 127, 128, 250])
def test_a_far_key_that_stands_out_in_prompt_and_decode(far, dtype):
    n = 300
    cfg, w, h = far_key_case("attention", n, far)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    want = P.normed_attention(h, w, "l0.mix.", m, eps)
    # the case is what it claims: without the far key the last row would be another
    keep = [i for i in range(n) if i != far]
    assert float((P.normed_attention(h[keep], w, "l0.mix.", m, eps)[-1] - want[-1]).abs().max()) > 0.2 * float(want[-1].abs().max())
    from gguf_rs_cli_b200.engine.step import Engine
    model = build(cfg, w, dtype).model
    eng = Engine(model, n_tokens=1024, n_slots=2)
    hd = h.to(tdtype(dtype)).to(DEV)
    # in a prompt
    s = eng.open()
    ctx, _, _ = eng.plan([entry(s, [1] * n, ())])
    got = model.layers[0].mixer.forward(hd, ctx, eng.runs[0])
    assert_close(got, want, dtype, f"far key {far} in a prompt")
    eng.close(s)
    # decoded: all but the last row as a prompt, the last one alone
    s = eng.open()
    ctx, _, _ = eng.plan([entry(s, [1] * (n - 1), ())])
    model.layers[0].mixer.forward(hd[:n - 1], ctx, eng.runs[0])
    eng.cache.advance([s], [n - 1])
    ctx, _, _ = eng.plan([entry(s, [1], ())])
    got = model.layers[0].mixer.forward(hd[n - 1:], ctx, eng.runs[0])
    assert_close(got, want[n - 1:], dtype, f"far key {far} seen from a decoded token")
    eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,heads,kv_heads", [(48, 4, 2), (80, 2, 2), (128, 8, 1), (256, 2, 1)])
def test_attention_layer_with_keys_and_values_of_one_size(hd, heads, kv_heads, dtype):
    """The normalised attention alone where keys and values have one size: in bfloat16 single tokens then take the
    CUDA-core decode kernel (any multiple of 16 up to 256) and prompts of 128 the tiled one; 140 rows as a prompt,
    then 70 more one by one over the page border at 192, with page splits in the longer of two sequences."""
    from gguf_rs_cli_b200.engine.step import Engine
    cfg = config("small")
    cfg["layers"] = [cfg["layers"][0]]
    cfg["layers"][0]["mixer"].update(heads=heads, kv_heads=kv_heads, dim=hd, vdim=hd, scale=2.0 / hd ** 0.5,
                                     q_temp={"coef": 0.4, "every": 64})
    w = make_weights(cfg, {}, seed=hd)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    model = build(cfg, w, dtype).model
    eng = Engine(model, n_tokens=2048, n_slots=2)
    g = torch.Generator().manual_seed(hd)
    n, n0 = 210, 140
    h = torch.randn(n, cfg["width"], generator=g).to(torch.bfloat16).float()
    want = P.normed_attention(h, w, "l0.mix.", m, eps)
    hd_ = h.to(tdtype(dtype)).to(DEV)
    a, b = eng.open(), eng.open()
    ctx, _, _ = eng.plan([entry(a, [1] * n0, ()), entry(b, [1] * 3, ())])
    got = model.layers[0].mixer.forward(torch.cat([hd_[:n0], hd_[:3]]), ctx, eng.runs[0])
    assert_close(got[:n0], want[:n0], dtype, f"prompt, heads of {hd}")
    assert_close(got[n0:], want[:3], dtype, f"short prompt beside it, heads of {hd}")
    eng.cache.advance([a, b], [n0, 3])
    for t in range(n0, n):
        ctx, _, _ = eng.plan([entry(a, [1], ()), entry(b, [1], ())])
        got = model.layers[0].mixer.forward(torch.stack([hd_[t], hd_[3 + t - n0]]), ctx, eng.runs[0])
        eng.cache.advance([a, b], [1, 1])
        assert_close(got[:1], want[t:t + 1], dtype, f"row {t} alone, heads of {hd}")
        assert_close(got[1:], want[3 + t - n0:4 + t - n0], dtype, f"row {3 + t - n0} of the short sequence, heads of {hd}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_and_delta_rule_over_page_borders(dtype):
    """The two other mixers alone over 200 rows, whole and with the last 72 rows one by one (over the borders at
    128 and 192), with slow decays."""
    name = "small"
    cfg, w = config(name), weights(name, 0, True)
    model = llm(name, dtype, slow_decay=True).model
    from gguf_rs_cli_b200.engine.step import Engine
    eng = Engine(model, n_tokens=1024, n_slots=2)
    n = 200
    g = torch.Generator().manual_seed(77)
    h = torch.randn(n, cfg["width"], generator=g).to(torch.bfloat16).float()
    hd = h.to(tdtype(dtype)).to(DEV)
    for i in (1, 2, 3):
        layer = cfg["layers"][i]
        want = P.MIXERS[layer["type"]](h, w, f"l{i}.mix.", layer["mixer"], cfg["norm"]["eps"])
        s = eng.open()
        ctx, _, _ = eng.plan([entry(s, [1] * 128, ())])
        got = model.layers[i].mixer.forward(hd[:128], ctx, eng.runs[i])
        assert_close(got, want[:128], dtype, f"layer {i} prompt")
        eng.cache.advance([s], [128])
        for t in range(128, n):
            ctx, _, _ = eng.plan([entry(s, [1], ())])
            got = model.layers[i].mixer.forward(hd[t:t + 1], ctx, eng.runs[i])
            eng.cache.advance([s], [1])
            assert_close(got, want[t:t + 1], dtype, f"layer {i} ({layer['type']}) row {t} alone")
        eng.close(s)


def test_fast_attention_paths_agree_with_the_general_kernel():
    """In bfloat16, with keys and values of 64 entries per head, prompts of both attention mixers take the tiled
    kernel (32-bit weights as three bfloat16 terms; the latent mixer over per-head keys and values of the step's own)
    and single tokens take the CUDA-core decode kernel (plain attention) or the kernel that serves all heads from one
    pass over the latent rows (latent attention).  The general kernel on the same
    rows gives the same up to the rounding of bfloat16 intermediates, for sequences that end at a page's edge,
    inside a page, and, where the path allows it, with cached positions in front."""
    name, dtype = "wide", "bfloat16"
    cfg, model = config(name), llm(name, dtype).model
    eng = new_engine(name, dtype)
    g = torch.Generator().manual_seed(5)

    def both(layer, h, ctx, switch):
        mixer = model.layers[layer].mixer
        fast = mixer.forward(h, ctx, eng.runs[layer]).float().clone()
        setattr(mixer, switch, lambda: False)
        try:
            ctx2 = ctx if switch != "_tiled" else eng.plan([entry(s, [1] * n, ()) for s, n in zip(ctx.host["slots"], ctx.host["qlens"])])[0]
            general = mixer.forward(h, ctx2, eng.runs[layer]).float().clone()
        finally:
            delattr(mixer, switch)
        return fast, general

    assert model.layers[0].mixer._tiled() and model.layers[0].mixer._fast_decode()
    assert model.layers[2].mixer._exact_tiled() and model.layers[2].mixer._exact_decode()
    for layer, switch, steps in ((0, "_tiled", [[130, 64, 3]]), (2, "_exact_tiled", [[130, 64, 3], [70, 1, 129]])):
        slots = [eng.open() for _ in range(3)]
        for lens in steps:
            h = torch.randn(sum(lens), cfg["width"], generator=g).to(torch.bfloat16).to(DEV)
            ctx, _, _ = eng.plan([entry(s, [1] * n, ()) for s, n in zip(slots, lens)])
            if layer == 0:
                assert "pages" in ctx.plan_of(model.layers[0].mixer)
            fast, general = both(layer, h, ctx, switch)
            eng.cache.advance(slots, lens)
            assert float((fast - general).abs().max()) <= 2 ** -5 * float(general.abs().max()), (layer, lens)
        # single tokens: the CUDA-core decode kernel (attention), the kernel that serves all heads from one pass (latent)
        h = torch.randn(3, cfg["width"], generator=g).to(torch.bfloat16).to(DEV)
        ctx, _, _ = eng.plan([entry(s, [1], ()) for s in slots])
        fast, general = both(layer, h, ctx, "_exact_decode" if layer == 2 else "_fast_decode")
        assert float((fast - general).abs().max()) <= 2 ** -6 * float(general.abs().max()), layer
        if layer == 0:
            # the same without the tensor-core kernel: the CUDA-core kernel of one pass for all heads
            from gguf_rs_cli_b200 import native
            native.library().gb_latent_decode_set_mma(0)
            try:
                plain = model.layers[0].mixer.forward(h, ctx, eng.runs[0]).float().clone()
            finally:
                native.library().gb_latent_decode_set_mma(1)
            assert float((plain - general).abs().max()) <= 2 ** -6 * float(general.abs().max())
        for s_ in slots:
            eng.close(s_)


# ------------------------------------------------------------ generation
def plain_greedy(name, prompt, max_tokens):
    cfg, w = CONFIGS[name][0], weights(name)
    seq, out = list(prompt), []
    for _ in range(max_tokens):
        tok = int(P.forward(cfg, w, seq, dtype=torch.float64)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out


def test_greedy_generation_float32_equals_plain():
    from gguf_rs_cli_b200.api import generate
    prompts = [tokens_of("small", n, 50 + n) for n in (5, 1, 13, 66)]
    got = generate(llm("small", "float32"), prompts, max_tokens=10, temperature=0.0, stop_token_ids=[])
    assert got == [plain_greedy("small", p, 10) for p in prompts]
    # more requests than the batch holds: one batch after another through the same slots
    got2 = generate(llm("small", "float32"), prompts, max_tokens=10, temperature=0.0, stop_token_ids=[], max_batch=2)
    assert got2 == got


def test_bfloat16_greedy_follows_plain_until_a_near_tie():
    from gguf_rs_cli_b200.api import generate
    cfg, w = CONFIGS["wide"][0], weights("wide")
    prompts = [tokens_of("wide", n, 80 + n) for n in (3, 40)]
    got = generate(llm("wide", "bfloat16"), prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = P.forward(cfg, w, seq)[-1]
            assert float(logits[tok]) >= float(logits.max()) - TOL["bfloat16"] * float(logits.abs().max()), f"token {tok} at length {len(seq)}"
            seq.append(tok)


def test_command_line_with_random_weights(tmp_path, capsys):
    import json
    from gguf_rs_cli_b200.cli import main
    path = tmp_path / "config.json"
    path.write_text(json.dumps(config("small")))
    assert main(["--random", str(path), "-p", "1,2,3", "-p", "9", "-n", "5", "-t", "0", "--no-eos"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and all(len(l.split(",")) == 5 for l in lines)


def test_trace_replay_of_a_model_folder(tmp_path):
    """bin/trace_run on a Debonex folder: whole, then one by one, then two requests together."""
    import json
    import os
    from gguf_rs_cli_b200.weights import write_safetensors
    from tests.test_trace_run_gpu import Replay, close
    cfg, w = config("small"), weights("small")
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(folder / "model.safetensors"), [(n, t.to(torch.bfloat16)) for n, t in w.items()])
    a, b = tokens_of("small", 40, 1), tokens_of("small", 9, 2)
    wa, wb = plain_logits("small", 40, 1), plain_logits("small", 9, 2)
    for dtype in DTYPES:
        r = Replay(str(folder), dtype, str(tmp_path / f"out_{dtype}"), max_tokens=49)
        close(r.step([("a", a, range(40))], end=["a"]), wa, dtype, "whole")
        close(r.step([("a", a[:30], [29]), ("b", b[:5], [0, 4])]), torch.stack([wa[29], wb[0], wb[4]]), dtype, "two prompts")
        for i in range(4):
            close(r.step([("a", [a[30 + i]], [0]), ("b", [b[5 + i]], [0])], end=["b"] if i == 3 else []),
                  torch.stack([wa[30 + i], wb[5 + i]]), dtype, f"two requests, step {i}")
        close(r.step([("a", [a[34]], [0])], end=["a"]), wa[34], dtype, "the longer one alone")
        r.finish()
