"""Dilalix in the package against the plain implementation (tests/plain_dilalix.py), in 32-bit and in bfloat16: every
mechanism alone, whole prompts against token-by-token decoding, prompts cut into portions down to two tokens, unequal
batches against each request alone, slots and pages that are used again, keys far back, at page borders and just
inside and outside the window and the kept first positions, the first tokens of a sequence, long decoding through a
ring of pages that goes round, and greedy generation through the package's entry point."""
import copy

import pytest
import torch

from tests import plain_dilalix as P
from tests.dilalix_util import CONFIGS, build, config, llm, new_engine, plain_logits, scenario, tokens_of, weights
from tests.gpu_util import TOL

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = ["small", "wide"]


def assert_close(got, want, dtype, what="", tally=None):
    """32-bit: the largest error against the largest value of the compared block, 1e-4 (the sharp test: a key left
    out, a state not carried or a wrong edge moves results by far more).  bfloat16, row by row: the root mean square of a
    row's error is held to 8% of the block's root mean square.  A router's choice is discrete: where two scores are
    closer than bfloat16's rounding of the rows in front of them, another expert is taken and that token's row is far
    off, in a correct implementation too.  So one row in ten may fail (none of a block of fewer than eight rows);
    rows compared one at a time are counted in `tally` and judged together by settle()."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err, ref = float((got - want).abs().max()), max(float(want.abs().max()), 1e-6)
    if dtype == "float32":
        assert err <= TOL[dtype] * ref, f"{what}: max error {err:.3e} against max |ref| {ref:.3e} ({dtype})"
        return
    g2, w2 = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
    rms_ref = max(float(w2.pow(2).mean().sqrt()), 1e-6)
    bad = ((g2 - w2).pow(2).mean(-1).sqrt() > 8e-2 * rms_ref).tolist()
    if tally is not None:
        tally.extend(bad)
        return
    allowed = len(bad) // 10 if len(bad) >= 8 else 0
    assert sum(bad) <= allowed, f"{what}: {sum(bad)} of {len(bad)} rows are off by more than 8% of {rms_ref:.3e} (max error {err:.3e}, {dtype})"


def settle(tally, what=""):
    assert sum(tally) <= max(1, len(tally) // 10), f"{what}: {sum(tally)} of {len(tally)} rows were off"


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
@pytest.mark.parametrize("y_dtype", DTYPES)
@pytest.mark.parametrize("E", [5, 72, 1000])
def test_norm_of_a_result_into_the_stream(E, y_dtype):
    from gguf_rs_cli_b200 import kernels
    g = torch.Generator().manual_seed(E)
    x, y, w = torch.randn(7, E, generator=g), (torch.randn(7, E, generator=g) * 3).to(tdtype(y_dtype)), torch.randn(E, generator=g)
    xd, xb = x.to(DEV), torch.empty(7, E, dtype=torch.bfloat16, device=DEV)
    kernels.norm_residual_add(xd, y.to(DEV), w.to(DEV), 1e-3, xb=xb)
    want = x + P.rms(y.float(), w, 1e-3)
    assert torch.allclose(xd.cpu(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(xb.cpu(), xd.cpu().to(torch.bfloat16))
    kernels.norm_residual_add(xd, None, None, 1.0, xb=xb.zero_())          # the copy alone
    assert torch.equal(xb.cpu(), xd.cpu().to(torch.bfloat16)) and torch.allclose(xd.cpu(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("act", ["gelu", "silu", "gelu_tanh"])
def test_activation_of_a_whole_buffer(act):
    from gguf_rs_cli_b200 import kernels
    z = torch.randn(37, 50, generator=torch.Generator().manual_seed(3)) * 3
    want = {"gelu": P.gelu_erf, "silu": P.silu,
            "gelu_tanh": lambda v: 0.5 * v * (1 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))}[act](z.double())
    got = kernels.unary_act_(z.clone().to(DEV), act)
    assert torch.allclose(got.cpu().double(), want, rtol=1e-5, atol=1e-6)
    got = kernels.unary_act_(z.to(torch.bfloat16).to(DEV), act)
    assert float((got.float().cpu().double() - want).abs().max()) <= 4e-2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_mixer_alone_in_an_unequal_batch(name, dtype):
    cfg, w, model = config(name), weights(name), llm(name, dtype).model
    eng = new_engine(name, dtype)
    lens = [70, 5, 1]
    ctx, _ = plan_for(eng, lens)
    g = torch.Generator().manual_seed(3)
    h = torch.randn(sum(lens), cfg["width"], generator=g).to(tdtype(dtype))
    first = None
    for i, layer in enumerate(cfg["layers"]):
        got = model.layers[i].mixer.forward(h.to(DEV), ctx, eng.runs[i])
        want, raws, t0 = [], [], 0
        for b, n in enumerate(lens):
            rows = h[t0:t0 + n].float()
            if layer["type"] == "gla":
                want.append(P.gla(rows, w, f"l{i}.mix.", layer["mixer"], cfg["norm"]["eps"]))
            else:
                takes = layer["mixer"]["v_mix"] and first is not None
                y, raw = P.attention(rows, w, f"l{i}.mix.", layer["mixer"], cfg["norm"]["eps"], first[b] if takes else None)
                want.append(y)
                raws.append(raw)
            t0 += n
        if layer["type"] == "attention" and layer["mixer"]["v_mix"] and first is None:
            first = raws
        assert_close(got, torch.cat(want), dtype, f"{name} layer {i} ({layer['type']})")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_feed_forward_alone(name, dtype):
    cfg, w, model = config(name), weights(name), llm(name, dtype).model
    eng = new_engine(name, dtype)
    ctx, _ = plan_for(eng, [40, 3])
    h = torch.randn(43, cfg["width"], generator=torch.Generator().manual_seed(4)).to(tdtype(dtype))
    for i, layer in enumerate(cfg["layers"]):
        mlp = layer.get("mlp")
        if mlp is None:
            assert model.layers[i].feed_forward is None
            continue
        got = model.layers[i].feed_forward.forward(h.to(DEV), ctx)
        want = P.dense_ff(h.float(), w, f"l{i}.mlp.") if mlp["kind"] == "dense" else P.moe_ff(h.float(), w, f"l{i}.mlp.", mlp)
        assert_close(got, want, dtype, f"{name} layer {i} feed-forward ({mlp['kind']})")


@pytest.mark.parametrize("E,groups,keep,top", [(12, 3, 2, 3), (8, 2, 1, 4), (16, 1, 1, 5), (6, 6, 2, 2), (64, 8, 3, 8), (5, 1, 1, 5), (96, 4, 4, 1)])
def test_router_choice_alone(E, groups, keep, top):
    from gguf_rs_cli_b200 import kernels
    T = 50
    z = torch.randn(T, E, generator=torch.Generator().manual_seed(E + top)) * 2
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.moe_route(z.to(DEV), groups, keep, top, 1.75, ids, wts)
    s = torch.sigmoid(z.double())
    for t in range(T):
        chosen = P.route(s[t], top, groups, keep)
        assert ids[t].tolist() == chosen, f"token {t}"
        want = s[t][chosen] / (s[t][chosen].sum() + 1e-20) * 1.75
        assert torch.allclose(wts[t].cpu().double(), want, rtol=1e-5)


@pytest.mark.parametrize("T,K,F,N,E,top,skew", [(70, 72, 24, 72, 12, 3, False), (300, 256, 48, 200, 8, 4, True), (17, 64, 8, 64, 5, 1, False)])
def test_grouped_experts_agree_with_token_by_token(T, K, F, N, E, top, skew):
    """The tiled kernels of many tokens against the kernels that take every (token, choice) pair for itself and against
    the plain expert, also when one expert gets most pairs (several tiles) and others none."""
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "bfloat16")
    ctx, _ = plan_for(eng, [1])
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, K, generator=g).to(torch.bfloat16)
    wg, wu = (torch.randn(E, F, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16), (torch.randn(E, F, K, generator=g) / K ** 0.5 * 2).to(torch.bfloat16)
    wd = (torch.randn(E, N, F, generator=g) / F ** 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if skew:
        ids[: T - 20, 0] = 2
        for t in range(T - 20):                                      # a token names no expert twice
            for r in range(1, top):
                if ids[t, r] == 2:
                    ids[t, r] = (3 + r) % E if (3 + r) % E != 2 else 0
        ids[ids == 5] = 6 if not (ids == 6).any() else 5
    wts = torch.rand(T, top, generator=g) + 0.1
    limit = 1.5
    want = torch.zeros(T, N, dtype=torch.float64)
    for t in range(T):
        for r in range(top):
            e = int(ids[t, r])
            w = {"x.gate": wg[e].float(), "x.up": wu[e].float(), "x.down": wd[e].float()}
            want[t] += float(wts[t, r]) * P.expert(h[t:t + 1].double(), w, "x.", limit)[0]
    base = torch.randn(T, N, generator=g)
    hd, idd, wtd = h.to(DEV), ids.to(DEV), wts.to(DEV)
    out = base.clone().to(DEV)
    kernels.moe_grouped(hd, idd, wtd, wg.to(DEV), wu.to(DEV), wd.to(DEV), limit, out, ctx, accumulate=True)
    y = torch.empty(T, top, F, dtype=torch.bfloat16, device=DEV)
    one = base.clone().to(DEV)
    kernels.moe_gate_up(hd, idd, wg.to(DEV), wu.to(DEV), limit, y)
    kernels.moe_down(y, idd, wtd, wd.to(DEV), one, accumulate=True)
    assert_close(one - base.to(DEV), want.float(), "bfloat16", "token by token")
    assert_close(out - base.to(DEV), want.float(), "bfloat16", "tiled")
    assert float((out - one).abs().max()) <= 2e-2 * float(want.abs().max())
    fresh = torch.full((T, N), 9.0, device=DEV)
    kernels.moe_grouped(hd, idd, wtd, wg.to(DEV), wu.to(DEV), wd.to(DEV), limit, fresh, ctx, accumulate=False)
    assert torch.equal(fresh, out - base.to(DEV)) or float((fresh - (out - base.to(DEV))).abs().max()) < 1e-5
    # expert by expert as ordinary products (the path of very many tokens)
    each = base.clone().to(DEV)
    kernels.moe_by_expert(hd, idd, wtd, wg.to(DEV), wu.to(DEV), wd.to(DEV), limit, each, ctx, accumulate=True)
    assert_close(each - base.to(DEV), want.float(), "bfloat16", "expert by expert")
    assert float((each - one).abs().max()) <= 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("D,Dv,H,cuts", [(8, 4, 1, None), (24, 40, 3, None), (64, 64, 2, None), (100, 36, 2, None), (128, 128, 1, None),
                                         (200, 8, 1, None), (24, 40, 3, [(300, 2), (257, 400), (1, 129), (130, 157)]),
                                         (128, 64, 2, [(640, 3), (1, 600), (47, 85)])])
def test_gla_kernel_at_every_shape_of_its_walk(D, Dv, H, cuts):
    """The recurrence kernels alone: two sequences fed in unequal pieces give what the plain walk gives whole; the
    state is carried in the slots' rows.  With pieces of more than 256 tokens the segments of a sequence are walked side
    by side, beside a sequence that brings a few tokens, from states that earlier steps left."""
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "float32", n_tokens=4096)
    g = torch.Generator().manual_seed(D + Dv)
    cuts = cuts or [(1, 2), (2, 1), (3, 17), (1, 1), (30, 16)]
    n, tau = max(sum(a for a, _ in cuts), sum(b for _, b in cuts)), 5.0
    q, k, a = (torch.randn(2, n, H * D, generator=g) for _ in range(3))
    v, bias = torch.randn(2, n, H * Dv, generator=g), torch.rand(H * D, generator=g) * 4 + 1
    alpha = torch.sigmoid((a + bias).double()) ** (1.0 / tau)
    want = [torch.stack([P.decayed_outer_recurrence(q[b, :, i * D:(i + 1) * D].double() * D ** -0.5, k[b, :, i * D:(i + 1) * D].double(),
                                                    v[b, :, i * Dv:(i + 1) * Dv].double(), alpha[b, :, i * D:(i + 1) * D])[0]
                         for i in range(H)], dim=1).reshape(n, H * Dv) for b in range(2)]
    state = torch.zeros(eng.cache.n_slots, H, D, Dv, device=DEV)
    state[:] = 7.0                                                   # slots of other sequences are not touched
    slots = [eng.open(), eng.open()]
    for s in slots:
        state[s] = 0.0
    fed, got = [0, 0], [[], []]
    for cut_a, cut_b in cuts:
        ctx, _, _ = eng.plan([entry(slots[0], [1] * cut_a, ()), entry(slots[1], [1] * cut_b, ())])
        rows = [torch.cat([t[0, fed[0]:fed[0] + cut_a], t[1, fed[1]:fed[1] + cut_b]]) for t in (q, k, v, a)]
        buf = torch.cat(rows[:3], dim=1).to(DEV)                     # q, k, v as column slices of one buffer
        out = torch.empty(cut_a + cut_b, H * Dv, device=DEV)
        kernels.gla(buf[:, :H * D], buf[:, H * D:2 * H * D], buf[:, 2 * H * D:], rows[3].to(DEV), bias.to(DEV), tau, D ** -0.5,
                    state, out, ctx, H, D, Dv)
        eng.cache.advance(slots, [cut_a, cut_b])
        got[0].append(out[:cut_a].cpu())
        got[1].append(out[cut_a:].cpu())
        fed = [fed[0] + cut_a, fed[1] + cut_b]
    for b in range(2):
        assert_close(torch.cat(got[b]), want[b][:fed[b]].float(), "float32", f"gla D={D} sequence {b}")
    others = [s for s in range(eng.cache.n_slots) if s not in slots]
    assert bool((state[others] == 7.0).all())


def near_tie(scores, mine, theirs, n_groups, margin=0.05):
    """Whether two choices of experts differ by a near tie only: the experts that one has and the other has not have
    scores within the margin of each other, or they lie in groups whose marks (the sum of a group's two largest scores)
    are within the margin."""
    only_mine, only_theirs = sorted(set(mine) - set(theirs)), sorted(set(theirs) - set(mine))
    if len(only_mine) != len(only_theirs):
        return False
    size = scores.numel() // n_groups
    mark = [sum(sorted(scores[g * size:(g + 1) * size].tolist(), reverse=True)[:2]) for g in range(n_groups)]
    a, b = sorted(float(scores[e]) for e in only_mine), sorted(float(scores[e]) for e in only_theirs)
    if all(abs(x - y) < margin for x, y in zip(a, b)):
        return True
    ga, gb = {e // size for e in only_mine} - {e // size for e in theirs}, {e // size for e in only_theirs} - {e // size for e in mine}
    return bool(ga) and bool(gb) and all(abs(mark[x] - mark[y]) < margin for x in ga for y in gb)


# ------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_request_alone(name, dtype):
    """Whole prompts with the routed experts in the model.  bfloat16: where the package's router chose otherwise than
    the plain one, the two scores must be a near tie, the plain model then follows the package's choice, and such
    tokens are few."""
    eng, model = new_engine(name, dtype), llm(name, dtype).model
    taken = {}
    for i, layer in enumerate(model.layers):
        ff = layer.feed_forward
        if ff is not None and ff.spec.kind == "moe":
            def wrapped(h, ctx, x32=None, orig=ff.forward, i=i, top=ff.top):
                out = orig(h, ctx, x32=x32)
                taken[i] = ctx.ws.get("moe.ids", (h.shape[0], top), torch.int32).cpu().tolist()
                return out
            ff.forward = wrapped
    try:
        for n, seed in [(1, 1), (2, 2), (5, 3), (64, 4), (65, 5), (131, 6)]:
            s = eng.open()
            got = eng.step([entry(s, tokens_of(name, n, seed), range(n))])
            eng.close(s)
            want = plain_logits(name, n, seed)
            if dtype == "bfloat16":
                scores, own = {}, {}
                P.forward(CONFIGS[name][0], weights(name), tokens_of(name, n, seed), scores_out=scores)
                differ = 0
                for i, sc in scores.items():
                    r = CONFIGS[name][0]["layers"][i]["mlp"]["router"]
                    groups = r.get("groups") or {"count": 1, "keep": 1}
                    for t in range(n):
                        mine = P.route(sc[t], r["top"], groups["count"], groups["keep"])
                        if sorted(mine) != sorted(taken[i][t]):
                            differ += 1
                            assert near_tie(sc[t], mine, taken[i][t], groups["count"]), f"{name} n={n} layer {i} token {t}: {mine} against {taken[i][t]}"
                assert differ <= max(1, n // 20), f"{name} n={n}: {differ} choices differ"
                if differ:
                    want = P.forward(CONFIGS[name][0], weights(name), tokens_of(name, n, seed), routes=taken).float()
            assert_close(got, want, dtype, f"{name} whole n={n}")
    finally:
        for layer in model.layers:
            if layer.feed_forward is not None:
                layer.feed_forward.__dict__.pop("forward", None)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(name, dtype):
    """Decoding from an empty sequence: the empty state, windows that are not yet full, the kept first positions while
    the window still holds them, and a page border on the way."""
    name = scenario(name, dtype)
    eng = new_engine(name, dtype)
    n, seed = 80, 8
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    s, tally = eng.open(), []
    for i in range(n):
        got = eng.step([entry(s, [toks[i]], [0])])
        assert_close(got[0], want[i], dtype, f"{name} position {i} decoded alone", tally)
    eng.close(s)
    settle(tally, f"{name} decoded from the first")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_in_portions(name, dtype):
    name = scenario(name, dtype)
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
    the recurrent state) goes to the next one, which must not see it."""
    name = scenario(name, dtype)
    eng = new_engine(name, dtype, n_tokens=64 * 7, n_slots=4)
    decode, seed, tally = 6, 100, []
    for lens in ([5, 9, 13, 70], [1, 7, 20, 33], [64, 65, 2], [129, 3]):
        reqs = []
        for n in lens:
            seed += 1
            total = n + decode
            reqs.append(dict(toks=tokens_of(name, total, seed), want=plain_logits(name, total, seed), n=n,
                             keep=decode - (seed % 3), slot=eng.open(), fed=0))
        got = eng.step([entry(r["slot"], r["toks"][:r["n"]], [r["n"] - 1]) for r in reqs])
        for i, r in enumerate(reqs):
            assert_close(got[i], r["want"][r["n"] - 1], dtype, f"{name} prompt of {r['n']} in batch {lens}", tally)
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
                assert_close(got[i], r["want"][r["fed"]], dtype, f"{name} step {step} of prompt {r['n']}", tally)
                r["fed"] += 1
        for r in reqs:
            if r["slot"] is not None:
                eng.close(r["slot"])
        eng.cache.check()
    settle(tally, f"{name} unequal batches")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_through_a_ring_that_goes_round(name, dtype):
    """A cache sized for steps of at most 16 tokens: the windowed layers keep a few pages that are written again and
    again, in front of them the pages of the kept first positions.  A prompt in portions of 16, then 200 tokens one by
    one; the recurrent state still holds the first tokens at the end."""
    name = scenario(name, dtype)
    eng = new_engine(name, dtype, n_tokens=1024, n_slots=2, max_step_tokens=16)
    assert any(g.ring_pages + g.head_pages < 8 for g in eng.cache.groups)
    n_prompt, n = 160, 360
    toks, want = tokens_of(name, n, 21), plain_logits(name, n, 21)
    s, tally = eng.open(), []
    for at in range(0, n_prompt, 16):
        got = eng.step([entry(s, toks[at:at + 16], [0, 15])])
        assert_close(got, want[[at, at + 15]], dtype, f"{name} portion at {at}", tally)
    for i in range(n_prompt, n):
        got = eng.step([entry(s, [toks[i]], [0])])
        if i % 7 == 0 or i > n - 20:
            assert_close(got[0], want[i], dtype, f"{name} position {i}", tally)
    eng.close(s)
    eng.cache.check()
    settle(tally, f"{name} long decoding")


@pytest.mark.parametrize("kind", ["gla", "attention", "bare"])
def test_models_of_one_kind_of_layer(kind):
    """A model whose layers are all gated linear attention keeps no keys at all (a cache without page groups); one of
    attention alone keeps no fixed-size state of a mixer; `bare` has one attention layer with nothing optional: no window,
    no rotation, no mixing of values, as many key/value heads as heads, values as wide as keys, no feed-forward."""
    from gguf_rs_cli_b200.engine.step import Engine
    cfg = copy.deepcopy(CONFIGS["small"][0])
    if kind == "gla":
        cfg["layers"] = [cfg["layers"][0], copy.deepcopy(cfg["layers"][0])]
        cfg["layers"][1]["mixer"]["tau"], cfg["layers"][1]["mlp"] = 2.5, None
        ranks = {0: 12, 1: 5}
    elif kind == "attention":
        cfg["layers"], ranks = cfg["layers"][1:], {}
    else:
        cfg["layers"], ranks = [{"type": "attention", "mixer": {"heads": 3, "dim": 24}, "mlp": None}], {}
    from tests.dilalix_util import make_weights
    w = make_weights(cfg, ranks, seed=4) if kind != "bare" else make_weights(
        {**cfg, "layers": [{"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 24, "vdim": 24}, "mlp": None}]}, ranks, seed=4)
    if kind == "bare":
        del w["l0.mix.vmix"]
    n = 90
    toks = torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(9)).tolist()
    plain_cfg = cfg if kind != "bare" else {**cfg, "layers": [{"type": "attention", "mlp": None, "mixer": {
        "heads": 3, "kv_heads": 3, "dim": 24, "vdim": 24, "scale": 24 ** -0.5, "v_mix": False, "mask": {"size": 10 ** 9, "keep_first": 0},
        "rot": {"base": 1.0, "dims": 0}}}]}
    want = P.forward(plain_cfg, w, toks).float()
    model = build(cfg, w, "float32").model
    eng = Engine(model, n_tokens=512, n_slots=2)
    assert (len(eng.cache.groups) == 0) == (kind == "gla")
    s = eng.open()
    got = [eng.step([entry(s, toks[:70], range(70))])]
    got += [eng.step([entry(s, [toks[i]], [0])]).clone() for i in range(70, n)]
    eng.close(s)
    assert_close(torch.cat(got), want, "float32", f"a model of {kind} layers")


# ------------------------------------------------- keys that stand out at every edge
SPIKE = {
    "architecture": "Dilalix", "vocab": 2048, "width": 48, "norm": {"eps": 1e-6},
    "layers": [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 16, "scale": 1.5, "v_mix": False,
                                               "mask": {"size": 70, "keep_first": 67}, "rot": {"base": 1e6, "dims": 4}}, "mlp": None}],
}


def spike_weights(cfg):
    """Token t + 1024 is the partner of token t: its query is the key of t (the query projection is the key projection
    behind an orthogonal map S of the rows, and the partner's row is S^T times the row of t).  A partner's score with
    its token's key is 1.5 * 24 (unit root mean square, 24 entries); all other scores are a few units."""
    g = torch.Generator().manual_seed(7)
    E, m = cfg["width"], cfg["layers"][0]["mixer"]
    k = torch.randn(m["dim"], E, generator=g) / E ** 0.5
    S, _ = torch.linalg.qr(torch.randn(E, E, generator=g))
    base = torch.randn(1024, E, generator=g)
    w = {"embed": torch.cat([base, base @ S]), "l0.norm1": torch.ones(E), "final.norm": torch.ones(E),
         "head": torch.randn(cfg["vocab"], E, generator=g) / E ** 0.5, "l0.mix.k": k, "l0.mix.q": torch.cat([k @ S, k @ S]),
         "l0.mix.v": torch.randn(m["vdim"], E, generator=g) / E ** 0.5 * 3, "l0.mix.g": torch.zeros(2 * m["vdim"], E),
         "l0.mix.o": torch.randn(E, 2 * m["vdim"], generator=g) / 6, "l0.mix.q.norm": torch.ones(m["dim"]),
         "l0.mix.k.norm": torch.ones(m["dim"]), "l0.mix.vmix": torch.tensor(0.0)}
    return {n: t.to(torch.bfloat16).float() for n, t in w.items()}


@pytest.mark.parametrize("dims", [(24, 16), (64, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_that_stand_out_at_every_edge_in_prompt_and_decode(dtype, dims):
    """All tokens differ; for chosen pairs (i, j) position i holds the partner of the token at position j, whose key
    then takes all of i's attention if and only if i may see j.  Pairs: j just inside and just outside the window, the last kept
    position and the first one that is not kept, across page borders, and hundreds of positions back."""
    cfg = copy.deepcopy(SPIKE)
    # keys and values of 64 entries reach the tiled kernel of prompts and the decode kernel in bfloat16
    cfg["layers"][0]["mixer"]["dim"], cfg["layers"][0]["mixer"]["vdim"] = dims
    cfg["layers"][0]["mixer"]["scale"] = 36.0 / dims[0]
    size, keep = cfg["layers"][0]["mixer"]["mask"]["size"], cfg["layers"][0]["mixer"]["mask"]["keep_first"]
    w = spike_weights(cfg)
    n = 700
    toks = torch.randperm(1024, generator=torch.Generator().manual_seed(1))[:n].tolist()
    pairs = [(200, 200 - size + 1), (210, 210 - size), (300, keep - 1), (310, keep), (320, 0), (330, 63), (340, 64),
             (64 + size - 1, 64), (64 + size + 3, 65), (128, 127), (650, 3), (660, 660 - size + 1), (670, 670 - size), (699, 66), (690, 68)]
    for i, j in pairs:
        toks[i] = toks[j] + 1024
    want = P.forward(cfg, w, toks).float()
    # the pairs do decide the logits: a window one longer, or one more kept position, moves them far
    longer, keeps_more = copy.deepcopy(cfg), copy.deepcopy(cfg)
    longer["layers"][0]["mixer"]["mask"]["size"] = size + 1
    keeps_more["layers"][0]["mixer"]["mask"]["keep_first"] = keep + 1
    top = float(want.abs().max())
    assert float((P.forward(longer, w, toks[:211]).float()[210] - want[210]).abs().max()) > 0.3 * top
    assert float((P.forward(keeps_more, w, toks[:311]).float()[310] - want[310]).abs().max()) > 0.3 * top
    rows = sorted({i for i, _ in pairs})
    model = build(cfg, w, dtype).model
    from gguf_rs_cli_b200.engine.step import Engine
    for max_step, cuts in [(None, [n]), (None, [190, 12, 2, 96, 400]), (64, [64] * 10 + [60])]:
        eng = Engine(model, n_tokens=2048, n_slots=2, max_step_tokens=max_step)
        s, at = eng.open(), 0
        for c in cuts:
            wanted = [r - at for r in rows if at <= r < at + c]
            got = eng.step([entry(s, toks[at:at + c], wanted)])
            if wanted:
                assert_close(got, want[[at + x for x in wanted]], dtype, f"portion {at}..{at + c} of {cuts}")
            at += c
        eng.close(s)
    # decoded one by one from position 180 on, in a cache whose ring goes round
    eng = Engine(model, n_tokens=2048, n_slots=2, max_step_tokens=32)
    s = eng.open()
    for at in range(0, 160, 32):
        eng.step([entry(s, toks[at:at + 32], [])])
    eng.step([entry(s, toks[160:180], [])])
    for i in range(180, n):
        got = eng.step([entry(s, [toks[i]], [0])])
        if i in rows:
            assert_close(got[0], want[i], dtype, f"position {i} decoded alone")
    eng.close(s)


@pytest.mark.parametrize("hd,window,keep", [(64, 70, 70), (128, 40, 5), (64, 200, 0), (128, 64, 64)])
def test_fast_attention_paths_agree_with_the_general_kernel(hd, window, keep):
    """One attention layer in bfloat16, fed the same rows twice: with the tiled kernel of prompts and the decode kernel
    of single tokens, and with the general kernel in their place.  Prompts in portions, then single tokens, two
    sequences of unequal lengths, in a cache whose ring goes round."""
    from gguf_rs_cli_b200.engine.step import Engine
    from gguf_rs_cli_b200.parts.attention import Attention
    cfg = {"architecture": "Dilalix", "vocab": 32, "width": 128, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mlp": None,
                       "mixer": {"heads": 4, "kv_heads": 2, "dim": hd, "vdim": hd, "scale": 3.0 / hd, "v_mix": False,
                                 "mask": {"size": window, "keep_first": keep}, "rot": {"base": 100.0, "dims": hd // 2}}}]}
    g = torch.Generator().manual_seed(hd + window)
    E = cfg["width"]
    w = {"embed": torch.randn(32, E, generator=g), "l0.norm1": torch.ones(E), "final.norm": torch.ones(E), "head": torch.randn(32, E, generator=g),
         "l0.mix.q": torch.randn(4 * hd, E, generator=g) / E ** 0.5, "l0.mix.k": torch.randn(2 * hd, E, generator=g) / E ** 0.5,
         "l0.mix.v": torch.randn(2 * hd, E, generator=g) / E ** 0.5, "l0.mix.g": torch.randn(4 * hd, E, generator=g) / E ** 0.5,
         "l0.mix.o": torch.randn(E, 4 * hd, generator=g) / (4 * hd) ** 0.5, "l0.mix.q.norm": torch.ones(hd) * 2, "l0.mix.k.norm": torch.ones(hd) * 2,
         "l0.mix.vmix": torch.tensor(0.0)}
    model = build(cfg, w, "bfloat16").model
    mixer = model.layers[0].mixer
    assert mixer._exact_tiled() and mixer._exact_decode()
    steps = [(48, 33), (48, 1), (48, 48), (48, 7), (40, 48)] + [(1, 1)] * 40
    rows = [torch.randn(a + b, E, generator=g).to(torch.bfloat16).to(DEV) for a, b in steps]
    results = []
    for fast in (True, False):
        eng = Engine(model, n_tokens=2048, n_slots=2, max_step_tokens=48)
        slots = [eng.open(), eng.open()]
        if not fast:
            mixer._exact_tiled = mixer._exact_decode = lambda: False
        outs = []
        for (a, b), h in zip(steps, rows):
            ctx, _, _ = eng.plan([entry(slots[0], [1] * a, ()), entry(slots[1], [1] * b, ())])
            outs.append(mixer.forward(h, ctx, eng.runs[0]).float().clone())
            eng.cache.advance(slots, [a, b])
        results.append(torch.cat(outs))
        if not fast:
            del mixer.__dict__["_exact_tiled"], mixer.__dict__["_exact_decode"]
    ref = float(results[1].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 2e-2 * ref, f"{float((results[0] - results[1]).abs().max())} of {ref}"


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
    cfg, w = CONFIGS["wide-dense"][0], weights("wide-dense")
    prompts = [tokens_of("wide", n, 80 + n) for n in (3, 40)]
    got = generate(llm("wide-dense", "bfloat16"), prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    off = []
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = P.forward(cfg, w, seq)[-1]
            off.append(float(logits[tok]) < float(logits.max()) - 0.1 * float(logits.abs().max()))
            seq.append(tok)
    settle(off, "greedy tokens that the plain model ranks far below its best")


def test_decode_steps_run_as_captured_graphs():
    """The generation loop captures decode steps of this design as of the others: every part declares its class."""
    assert llm("wide", "bfloat16").model.capturable and llm("small", "float32").model.capturable


def test_command_line_with_random_weights(tmp_path, capsys):
    import json
    from gguf_rs_cli_b200.cli import main
    path = tmp_path / "config.json"
    path.write_text(json.dumps(config("small")))
    assert main(["--random", str(path), "-p", "1,2,3", "-p", "9", "-n", "5", "-t", "0", "--no-eos"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and all(len(l.split(",")) == 5 for l in lines)


def test_trace_replay_of_a_model_folder(tmp_path):
    """bin/trace_run on a Dilalix folder: whole, then two requests together, then one by one."""
    import json
    from gguf_rs_cli_b200.weights import write_safetensors
    from tests.test_trace_run_gpu import Replay
    for dtype in DTYPES:
        name = scenario("small", dtype)
        cfg, w, V = config(name), weights(name), config(name)["vocab"]
        folder = tmp_path / f"model_{dtype}"
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(cfg))
        write_safetensors(str(folder / "model.safetensors"), [(n, t.to(torch.bfloat16)) for n, t in w.items()])
        a, b = tokens_of(name, 40, 1), tokens_of(name, 9, 2)
        wa, wb = plain_logits(name, 40, 1), plain_logits(name, 9, 2)
        r = Replay(str(folder), dtype, str(tmp_path / f"out_{dtype}"), max_tokens=49)

        def close(got, want, what):
            assert_close(torch.from_numpy(got.copy()).reshape(-1, V), want.reshape(-1, V), dtype, what)

        close(r.step([("a", a, range(40))], end=["a"]), wa, "whole")
        close(r.step([("a", a[:30], [29]), ("b", b[:5], [0, 4])]), torch.stack([wa[29], wb[0], wb[4]]), "two prompts")
        for i in range(4):
            close(r.step([("a", [a[30 + i]], [0]), ("b", [b[5 + i]], [0])], end=["b"] if i == 3 else []),
                  torch.stack([wa[30 + i], wb[5 + i]]), f"two requests, step {i}")
        close(r.step([("a", [a[34]], [0])], end=["a"]), wa[34], "the longer one alone")
        r.finish()
