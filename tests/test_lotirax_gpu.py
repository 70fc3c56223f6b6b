"""The Lotirax parts and the whole decoder against the plain implementation (tests/plain_lotirax.py): each mechanism
alone in portions and token by token, windows' edges, one far key among hundreds, then whole models under every way of
cutting, batching and reusing pages and slots, in float32 and bfloat16, and greedy generation through the scheduler."""
import pytest
import torch

import lotirax_helpers as lh
import plain_lotirax as plain
from qorvix_b200 import LLM, ModelRunner, SamplingParams, StepEntry
from qorvix_b200.cache import CacheManager
from qorvix_b200.config import lookup_architecture
from qorvix_b200.engine.batch import BatchBuilder
from qorvix_b200.parts import LoopSpec, Runtime, build_part
from qorvix_b200.weights import TensorSource

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]
CUTS = (33, 2, 1, 40, 1, 13, 2, 3)          # 95 tokens: page edges (16, 32, ...) fall inside portions and between them
EPS = 2e-5


def close(got, want, dtype, what="", loose=1.0):
    bound = (1e-4 if dtype in (torch.float32, "float32") else 3e-2 * loose) * max(1.0, float(want.abs().max()))
    err = (got.double().cpu() - want).abs().amax(dim=-1)
    bad = torch.nonzero(err > bound)
    assert not bad.numel(), f"{what}: {bad.numel()} of {err.numel()} rows off, first {int(bad[0])} (err {float(err.max()):.3e}, allowed {bound:.3e})"


def close_model(got, want, dtype, what=""):
    """Whole models.  float32: every row within 1e-4 of the largest logit.  bfloat16: rows are measured by their root
    mean square error against the logits' root mean square: the typical row within 2 %, few beyond 8 %, none beyond
    40 %; a wrong key or another request's page moves rows by far more in these sharpened models."""
    if dtype in (torch.float32, "float32"):
        return close(got, want, dtype, what)
    d = got.double().cpu() - want
    rel = d.pow(2).mean(dim=-1).sqrt() / want.pow(2).mean().sqrt()
    over = int((rel > 0.08).sum())
    assert float(rel.median()) < 0.02 and over <= max(1, rel.numel() // 30) and float(rel.max()) < 0.4, \
        f"{what}: median {float(rel.median()):.3e}, {over} of {rel.numel()} rows over 8 %, worst {float(rel.max()):.3e} at row {int(rel.argmax())}"


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def layer_spec(layer, width=72, vocab=211):
    """The framework's own spec builder for one layer of a configuration."""
    arch = lookup_architecture("Lotirax")
    return arch.build_spec(arch.config_from_dict(lh.config([layer], width=width, vocab=vocab, eps=EPS))).layers[0]


def run_in_portions(part, cache, x, cuts, dtype, rid="r", tokens=None):
    """Feeds x [T, width] through a mixer in the given portions of one request; returns the outputs."""
    builder = BatchBuilder(DEV)
    if not cache.has(rid):
        cache.admit(rid)
    outs, i = [], 0
    for n in cuts:
        assert cache.reserve(rid, n)
        segs = [dict(tokens=tokens[i:i + n] if tokens else [0] * n, pos0=cache.length(rid), slot=cache.slot(rid), want=[], first=i == 0)]
        tables = {g: [cache.block_table(rid, g)] for g in cache.paged_groups()}
        ctx = builder.build(segs, tables, cache.scratch_page)
        outs.append(part.forward(x[i:i + n].to(dtype).to(DEV), ctx, cache.layer_view(0)))
        cache.commit(rid, n)
        i += n
    return torch.cat(outs).float()


def mixer_setup(layer, dtype, width=72, seed=1, tweak=None, max_tokens=256):
    spec = layer_spec(lh.layer(layer, None), width).mixer
    w = lh.mixer_weights(layer["mixer"], width, torch.Generator().manual_seed(seed))
    if tweak:
        tweak(w)
    src = TensorSource(tensors={f"l0.mix.{k}": v.to(torch.bfloat16) for k, v in w.items()}, device=DEV, compute_dtype=dtype)
    part = build_part("mixer", spec, src, Runtime(DEV, dtype, 512))
    cache = CacheManager([(part.cache_spec(), None)], max_tokens=max_tokens, page_size=16, max_requests=2, device=DEV, dtype=dtype)
    return part, cache, {k: v.double() for k, v in w.items()}


MIXER_CASES = [lh.attn(), lh.attn(heads=3, kv_heads=3, dim=20, vdim=12, window=9, rot_dims=20, scaling=None),
               lh.attn(heads=2, kv_heads=1, dim=16, vdim=56, window=40, rot_dims=4),
               lh.attn(heads=6, kv_heads=2, dim=8, vdim=8, window=0, rot_dims=8, diff=0.6),
               lh.attn(heads=1, kv_heads=1, dim=36, vdim=24, window=17, rot_dims=0),
               lh.attn(heads=5, kv_heads=5, dim=12, vdim=28, window=64, rot_dims=12, scaling={"factor": 8.0, "original": 16, "fast": 4.0, "slow": 0.5}),
               lh.attn(heads=4, kv_heads=2, dim=32, vdim=64, window=33, rot_dims=32), lh.attn(heads=8, kv_heads=2, dim=64, vdim=128, window=0, rot_dims=32),
               lh.attn(heads=4, kv_heads=4, dim=16, vdim=32, window=48, rot_dims=16), lh.attn(heads=2, kv_heads=2, dim=40, vdim=88, window=20, rot_dims=40),
               lh.attn(heads=3, kv_heads=1, dim=7, vdim=70, window=5, rot_dims=6),
               lh.attn(heads=34, kv_heads=2, dim=8, vdim=8, window=30, rot_dims=8),      # 17 query heads a key/value head: no shared tile
               lh.attn(heads=4, kv_heads=2, dim=72, vdim=136, window=50, rot_dims=36),   # the widest tiles: maps of up to 128, values of up to 256
               lh.attn(heads=2, kv_heads=1, dim=128, vdim=256, window=0, rot_dims=128, scaling=None),
               lh.attn(heads=2, kv_heads=2, dim=96, vdim=64, window=19, rot_dims=64), lh.attn(heads=3, kv_heads=3, dim=24, vdim=200, window=35, rot_dims=24)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(MIXER_CASES)))
def test_differential_attention_alone_in_portions_and_token_by_token(case, dtype, monkeypatch):
    layer = MIXER_CASES[case]
    served = count_calls(monkeypatch, "diff_attention_tc")
    part, cache, w = mixer_setup(layer, dtype)
    x = rnd(95, 72, seed=case + 5).to(torch.bfloat16).float()
    want = plain.differential_attention(x.double(), w, layer["mixer"], EPS)
    close(run_in_portions(part, cache, x, CUTS, dtype), want, dtype, "portions", loose=2.0)
    # the same request again after another took and left its slot, one token at a time after a short start: a cache
    # row that the first run left behind would show
    cache.release("r")
    cache.admit("filler"); cache.release("filler")
    close(run_in_portions(part, cache, x[:60], (5,) + (1,) * 55, dtype, rid="again"), want[:60], dtype, "token by token", loose=2.0)
    cache.check_invariants()
    m = layer["mixer"]
    fits = dtype == torch.bfloat16 and m["dim"] % 8 == 0 and m["vdim"] % 8 == 0
    assert (served["diff_attention_tc"] > 0) == fits, "the tensor-core kernel serves bfloat16 sizes in multiples of 8, and only those"


def count_calls(monkeypatch, name):
    from qorvix_b200.csrc import ops
    calls = {name: 0}
    fn = getattr(ops, name)

    def counted(*a, **kw):
        res = fn(*a, **kw)
        calls[name] += 1 if res else 0
        return res
    monkeypatch.setattr(ops, name, counted)
    return calls


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=24, vdim=40, rot_dims=16), dict(heads=4, kv_heads=2, dim=32, vdim=64, rot_dims=32)])
@pytest.mark.parametrize("window", [1, 2, 5, 16, 17, 32, 40])
def test_window_edges_in_portions_and_in_decoding(window, sizes, dtype):
    """Keys just inside and just outside a window; pages the window has passed go back to the pool."""
    layer = lh.attn(window=window, sharp=4.0, **sizes)
    part, cache, w = mixer_setup(layer, dtype)
    x = rnd(95, 72, seed=3).to(torch.bfloat16).float()
    want = plain.differential_attention(x.double(), w, layer["mixer"], EPS)
    close(run_in_portions(part, cache, x, CUTS, dtype), want, dtype, f"window {window}", loose=2.0)
    if window <= 17:
        assert cache.free_pages() >= cache.num_pages - 3
    cache.release("r")
    close(run_in_portions(part, cache, x[:80], (3,) + (1,) * 77, dtype, rid="t"), want[:80], dtype, f"window {window}, token by token", loose=2.0)
    # one token wider or narrower is another function: the oracle itself tells them apart
    other = plain.differential_attention(x.double(), w, dict(layer["mixer"], mask={"size": window + 1}), EPS)
    assert float((other - want).abs().max()) > 0.05 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,sees", [(0, True), (300, True), (198, True), (197, False)])
@pytest.mark.parametrize("sizes", [dict(heads=2, kv_heads=1, dim=24, vdim=40, rot_dims=8), dict(heads=4, kv_heads=2, dim=32, vdim=64, rot_dims=16)])
def test_one_far_key_among_hundreds(sizes, window, sees, dtype):
    """A key far back is made to stand out in map 1 of every head: input 70 feeds only one unrotated entry of every key's
    first map and is set at position 3 alone; input 71 feeds the same entry of every query's first map and is set from
    position 200 on.  Position 200 sees key 3 exactly when the window reaches 198 keys; the outputs must follow."""
    layer = lh.attn(window=window, sharp=3.0, **sizes)
    n, H, G = sizes["dim"], sizes["heads"], sizes["kv_heads"]
    e = n - 2                                              # an entry that is not rotated

    def tweak(w):
        for mat, heads in (("k", G), ("q", H)):
            col = 70 if mat == "k" else 71
            w[mat][:, col] = 0.0
            for h in range(heads):
                w[mat][h * 2 * n + e] = 0.0
                w[mat][h * 2 * n + e, col] = 1.0
                w[mat + ".b"][h * 2 * n + e] = 0.0

    part, cache, w = mixer_setup(layer, dtype, seed=4, tweak=tweak, max_tokens=320)
    x = rnd(230, 72, seed=8)
    x[:, 70:] = 0.0
    x[3, 70] = 8.0
    x[200:, 71] = 8.0
    x = x.to(torch.bfloat16).float()
    want = plain.differential_attention(x.double(), w, layer["mixer"], EPS)
    got = run_in_portions(part, cache, x, (150, 41, 2, 7, 2) + (1,) * 28, dtype)
    close(got, want, dtype, "far key", loose=2.0)
    blind = x.clone()
    blind[3, 70] = 0.0                                      # what not seeing that key would give
    lost = plain.differential_attention(blind.double(), w, layer["mixer"], EPS)
    gap = (want[200:] - lost[200:]).abs().amax(dim=-1)
    if sees:
        assert float(gap[0]) > 0.05 * float(want.abs().max())
    if window == 197:
        assert float(gap.max()) < 1e-9
    if window == 198:                                       # seen by position 200 alone
        assert float(gap[1:].max()) < 1e-9


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("f", [lh.moe(), lh.moe(experts=3, top=1, ff=16, shared=0), lh.moe(experts=4, top=4, ff=40, shared=8),
                               lh.moe(experts=37, top=2, ff=8, shared=24), lh.moe(experts=6, top=2, ff=32, shared=16)])
def test_table_experts_alone(f, dtype):
    width, vocab = 72, 211
    spec = layer_spec(lh.layer(lh.attn(), f), width, vocab).feed_forward
    w = lh.mlp_weights(f, width, vocab, torch.Generator().manual_seed(2))
    src = TensorSource(tensors={f"l0.mlp.{k}": (v if v.dtype == torch.int32 else v.to(torch.bfloat16)) for k, v in w.items()}, device=DEV,
                       compute_dtype=dtype)
    part = build_part("feed_forward", spec, src, Runtime(DEV, dtype, 64))
    toks = [int(t) for t in torch.randint(0, vocab, (70,), generator=torch.Generator().manual_seed(5))]
    x = rnd(70, width, seed=6).to(torch.bfloat16).float()
    want = plain.table_experts(x.double(), toks, lh.as_float64(w), f)
    add = rnd(70, width, seed=7).to(dtype)
    s_mix, s_ff = (1 + 0.3 * rnd(width, seed=8)).to(DEV), (1 + 0.3 * rnd(width, seed=9)).to(DEV)
    builder = BatchBuilder(DEV)
    for lo, hi in ((0, 70), (0, 1), (1, 3), (3, 40)):           # batches of other sizes group the rows otherwise
        ctx = builder.build([dict(tokens=toks[lo:hi], pos0=lo, slot=0, want=[], first=lo == 0)], {}, 0)
        xs, ad = x[lo:hi].to(dtype).to(DEV), add[lo:hi].to(DEV).contiguous()
        got = part.forward(xs, ctx, add=ad)
        assert got.dtype == torch.float32
        close(got.cpu() - add[lo:hi].float(), want[lo:hi], dtype, f"rows {lo}:{hi}")
        got = part.forward(xs, ctx, add=ad, add_scale=s_mix, scale=s_ff)
        close(got.cpu(), add[lo:hi].double() * s_mix.double().cpu() + want[lo:hi] * s_ff.double().cpu(), dtype, f"scaled rows {lo}:{hi}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_re_entry_alone(dtype):
    width, passes = 40, 3
    w_in, step = (rnd(width, 2 * width, seed=1) * 0.1).to(torch.bfloat16), (0.3 * rnd(passes, width, seed=2)).to(torch.bfloat16)
    src = TensorSource(tensors={"loop.in": w_in, "loop.step": step}, device=DEV, compute_dtype=dtype)
    part = build_part("stream", LoopSpec((2, 5, 9), "loop.in", "loop.step", width), src, Runtime(DEV, dtype, 64))
    x, delta, x0 = rnd(7, width, seed=3), rnd(7, width, seed=4), rnd(7, width, seed=5).to(torch.bfloat16).float()
    for t, run in enumerate((2, 5, 9)):
        for pending in (None, delta.to(DEV), delta.to(dtype).to(DEV)):
            got = part.forward(run, x.to(DEV), pending, x0.to(DEV))
            xs = x.double() + (pending.double().cpu() if pending is not None else 0)
            want = torch.cat([xs, x0.double()], dim=1) @ w_in.double().T + step[t].double()
            assert got.dtype == torch.float32
            close(got, want, dtype, f"pass {t}")


# ---------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module")
def models():
    out = {}
    for name, cfg in (("A", lh.CONFIG_A), ("B", lh.CONFIG_B), ("C", lh.CONFIG_C), ("D", lh.CONFIG_D)):
        d = lh.make_model_dir(cfg, seed=11 + len(out))
        out[name] = (d, cfg, lh.as_float64(lh.model_weights(cfg, seed=11 + len(out))), {})
    return out


def plain_logits(model, toks):
    _, cfg, weights, memo = model
    key = tuple(toks)
    if key not in memo:
        memo[key] = plain.forward(cfg, weights, list(toks))
    return memo[key]


def tokens(vocab, n, seed):
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed))]


def runner(model, dtype, max_tokens=256, **kw):
    return ModelRunner(model[0], dtype=dtype, max_tokens=max_tokens, page_size=16, max_requests=kw.pop("max_requests", 4), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts_and_the_stream_after_every_run(models, name, dtype):
    m = models[name]
    r = runner(m, dtype, use_graphs=False)          # the tap copies to the host, which a captured step cannot
    for n, seed in ((1, 1), (2, 2), (17, 3), (64, 4), (97, 5)):
        toks = tokens(m[1]["vocab"], n, seed)
        taps = []
        r.model.stream_tap = lambda run, res, pend: taps.append((res + pend.float()).double().cpu())
        out = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        r.model.stream_tap = None
        close_model(out, plain_logits(m, toks), dtype, f"whole n={n}")
        streams = []
        plain.forward(m[1], m[2], toks, streams)
        assert len(taps) == len(streams)
        for run, (got, want) in enumerate(zip(taps, streams)):
            close(got, want, dtype, f"stream after run {run}, n={n}", loose=3.0)
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("graphs", [True, False])
def test_prefill_then_long_decode(models, name, dtype, graphs):
    m = models[name]
    toks = tokens(m[1]["vocab"], 130, 21)
    want = plain_logits(m, toks)
    r = runner(m, dtype, use_graphs=graphs)
    outs = [r.step([StepEntry("d", toks[:30], [29])])]
    for t in toks[30:]:
        outs.append(r.step([StepEntry("d", [t], [0])]))
    close_model(torch.cat(outs), want[29:], dtype, "decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_many_sizes(models, name, dtype):
    m = models[name]
    toks = tokens(m[1]["vocab"], 120, 31)
    want = plain_logits(m, toks)
    r = runner(m, dtype)
    for cuts in ((2,) * 10 + (100,), (31, 1, 2, 16, 3, 47, 2, 18), (1, 15, 16, 17, 63, 8), (7,) * 17 + (1,)):
        assert sum(cuts) == 120
        outs, i = [], 0
        for n in cuts:
            outs.append(r.step([StepEntry("p", toks[i:i + n], list(range(n)))]))
            i += n
        r.release("p")
        close_model(torch.cat(outs), want, dtype, f"cuts {cuts[:4]}..")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Four requests of unequal length advance in unequal portions beside one another in a pool that holds little more
    than they need; two end early and two new ones take their slots and pages.  Every row equals the request alone."""
    m = models[name]
    V = m[1]["vocab"]
    reqs = {"a": tokens(V, 90, 41), "b": tokens(V, 33, 42), "c": tokens(V, 61, 43), "d": tokens(V, 5, 44),
            "e": tokens(V, 70, 45), "f": tokens(V, 18, 46)}
    plan = [{"a": 40, "b": 2, "c": 17, "d": 5}, {"a": 1, "b": 30, "c": 1}, {"a": 16, "b": 1, "c": 3, "e": 2}, {"a": 1, "c": 31, "e": 37, "f": 1},
            {"a": 32, "c": 1, "e": 1, "f": 16}, {"c": 1, "e": 30, "f": 1}, {"c": 7}]
    r = runner(m, dtype, max_tokens=288)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step.items():
            entries.append(StepEntry(k, reqs[k][at[k]: at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = r.step(entries, end=end)
        row = 0
        for k, n in step.items():
            got[k].append(out[row: row + n])
            row += n
        r.cache.check_invariants()
    for k, toks in reqs.items():
        assert at[k] == len(toks)
        close_model(torch.cat(got[k]), plain_logits(m, toks), dtype, f"request {k}")
    assert r.cache.free_slots() == 4 and not r.cache.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_do_not_depend_on_the_batch(models, dtype):
    """A request's logits with three others in the step equal its logits alone: bit for bit in float32 (every sum has a
    fixed order), to rounding in bfloat16."""
    m = models["A"]
    V = m[1]["vocab"]
    toks = tokens(V, 50, 51)
    r = runner(m, dtype)
    alone = torch.cat([r.step([StepEntry("x", toks[:20], list(range(20)))]), r.step([StepEntry("x", toks[20:], list(range(30)))], end=["x"])])
    others = [StepEntry(k, tokens(V, n, 60 + n), []) for k, n in (("o1", 3), ("o2", 1), ("o3", 37))]
    first = r.step(others[:2] + [StepEntry("x", toks[:20], list(range(20)))] + others[2:])
    rest = r.step([StepEntry("o1", [1], []), StepEntry("x", toks[20:], list(range(30))), StepEntry("o2", [2, 3], [])])
    both = torch.cat([first, rest])
    if dtype == "float32":
        assert torch.equal(both, alone)
    else:
        close_model(both, alone.double().cpu(), dtype, "beside others")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_greedy_generation_through_the_scheduler(models, name, dtype):
    m = models[name]
    V = m[1]["vocab"]
    prompts = [tokens(V, n, 70 + n) for n in (9, 40, 3)]
    llm = LLM(str(m[0]), dtype=dtype, max_tokens=512, max_concurrent=2, max_batch_tokens=32)       # portions of prompts beside decoding; a third request waits for a slot
    results = llm.generate(prompts, SamplingParams.greedy_params(max_new_tokens=10))
    slack = 1e-3 if dtype == "float32" else 0.05
    for p, res in zip(prompts, results):
        assert len(res.tokens) == 10
        seq = list(p)
        for i, tok in enumerate(res.tokens):
            # along the engine's own continuation, every token must be the plain implementation's best or within
            # rounding of it (a near tie may fall either way)
            full = plain_logits(m, seq)[-1]
            assert float(full[tok]) >= float(full.max()) - slack * float(full.abs().max()), f"token {i} of a prompt of {len(p)}: {tok}, plain {int(full.argmax())}"
            seq.append(tok)
