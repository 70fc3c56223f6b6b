"""The Deganex parts and the whole decoder against the plain implementation (tests/plain_deganex.py): each
mechanism alone in portions, then whole models under every way of cutting, batching and reusing pages and slots,
in float32 and bfloat16, and greedy generation through the scheduler."""
import pytest
import torch

import deganex_helpers as dh
import plain_deganex as plain
from qorvix_b200 import LLM, ModelRunner, SamplingParams, StepEntry
from qorvix_b200.cache import CacheManager
from qorvix_b200.config import load_config, lookup_architecture
from qorvix_b200.engine.batch import BatchBuilder
from qorvix_b200.parts import Runtime, build_part
from qorvix_b200.weights import TensorSource

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]
NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
CUTS = (33, 2, 1, 40, 1, 13, 2, 3)          # 95 tokens: page edges (16, 32, ...) fall inside portions and between them


def close(got, want, dtype, what="", loose=1.0):
    bound = (1e-4 if dtype in (torch.float32, "float32") else 3e-2 * loose) * max(1.0, float(want.abs().max()))
    err = (got.double().cpu() - want).abs().amax(dim=-1)
    bad = torch.nonzero(err > bound)
    assert not bad.numel(), f"{what}: {bad.numel()} of {err.numel()} rows off, first {int(bad[0])} (err {float(err.max()):.3e}, allowed {bound:.3e})"


def close_model(got, want, dtype, what=""):
    """Whole models.  float32: every row within 1e-4 of the largest logit.  bfloat16: rounding in a deep, sharpened model
    moves single rows by percents (a near tie in a router flips an expert), so rows are measured by their root mean
    square error against the logits' root mean square: the typical row within 2 %, none beyond 15 %; a wrong key, a
    stale state or another request's slot moves rows by 30 % and more in these models."""
    if dtype in (torch.float32, "float32"):
        return close(got, want, dtype, what)
    d = got.double().cpu() - want
    rel = d.pow(2).mean(dim=-1).sqrt() / want.pow(2).mean().sqrt()
    over = int((rel > 0.08).sum())
    assert float(rel.median()) < 0.02 and over <= max(1, rel.numel() // 30) and float(rel.max()) < 0.4, \
        f"{what}: median {float(rel.median()):.3e}, {over} of {rel.numel()} rows over 8 %, worst {float(rel.max()):.3e} at row {int(rel.argmax())}"


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def part_spec(layer, width, eps):
    """The framework's own spec builder for one layer of a configuration."""
    cfg = load_config_dict(dh.config([layer], width=width, eps=eps))
    return lookup_architecture("Deganex").build_spec(cfg).layers[0]


def load_config_dict(raw):
    return lookup_architecture("Deganex").config_from_dict(raw)


def run_in_portions(part, cache, x, cuts, dtype, is_mixer=True, rid="r", first_call=True):
    """Feeds x [T, width] through a part in the given portions of one request; returns the outputs."""
    builder = BatchBuilder(DEV)
    if not cache.has(rid):
        cache.admit(rid)
    outs, i = [], 0
    for n in cuts:
        assert cache.reserve(rid, n)
        segs = [dict(tokens=[0] * n, pos0=cache.length(rid), slot=cache.slot(rid), want=[], first=i == 0)]
        tables = {g: [cache.block_table(rid, g)] for g in cache.paged_groups()}
        ctx = builder.build(segs, tables, cache.scratch_page)
        xi = x[i:i + n].to(dtype).to(DEV)
        outs.append(part.forward(xi, ctx, cache.layer_view(0)) if is_mixer else part.forward(xi, ctx))
        cache.commit(rid, n)
        i += n
    return torch.cat(outs).float()


def mixer_setup(layer, dtype, width=72, eps=2e-5, seed=1, sharp=1.0, window=0, tweak=None):
    import dataclasses
    spec = part_spec(dh.layer(layer, None), width, eps).mixer
    if window:
        spec = dataclasses.replace(spec, window=window)
    w = dh.mixer_weights(layer["type"], layer["mixer"], width, torch.Generator().manual_seed(seed), sharp)
    if tweak:
        tweak(w)
    src = TensorSource(tensors={f"l0.mix.{k}": v.to(torch.bfloat16) for k, v in w.items()}, device=DEV, compute_dtype=dtype)
    part = build_part("mixer", spec, src, Runtime(DEV, dtype, 512))
    cache = CacheManager([(part.cache_spec(), None)], max_tokens=256, page_size=16, max_requests=2, device=DEV, dtype=dtype)
    return part, cache, {k: v.double() for k, v in w.items()}


MIXER_CASES = [dh.attn(), dh.attn(heads=1, dim=8, rot_dim=16, vdim=36, kv_rank=24, scale=0.3, base=10000.0),
               dh.attn(heads=5, dim=16, rot_dim=4, vdim=7, kv_rank=33, scale=0.4),
               dh.attn(heads=3, dim=24, rot_dim=16, vdim=40, kv_rank=128), dh.attn(heads=5, dim=16, rot_dim=32, vdim=9, kv_rank=192, scale=0.15),
               dh.attn(heads=16, dim=8, rot_dim=16, vdim=8, kv_rank=64),           # sizes the tensor-core kernels take
               dh.mlstm(), dh.mlstm(heads=1, dim=33, vdim=16, gate_cap=3.0), dh.mlstm(heads=2, dim=7, vdim=70, gate_cap=15.0),
               dh.mamba(), dh.mamba(heads=2, vdim=40, state=12, groups=2, conv=2, norm_groups=1),
               dh.mamba(heads=4, vdim=16, state=36, groups=1, conv=5, norm_groups=2),
               dh.mlstm(heads=2, dim=136, vdim=24, gate_cap=6.0), dh.mamba(heads=2, vdim=40, state=160, groups=1, conv=4, norm_groups=1),   # key sizes of 129..256: 16-column tiles
               dh.mlstm(heads=1, dim=264, vdim=8, gate_cap=6.0)]                                     # beyond 256: the state stays in shared memory


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(MIXER_CASES)))
def test_each_mixer_alone_in_portions_and_token_by_token(case, dtype, monkeypatch):
    layer = MIXER_CASES[case]
    served = count_calls(monkeypatch, "latent_attention_tc")
    sharp = 3.0 if layer["type"] == "latent_attention" else 1.0          # peaked attention: one lost key shows
    part, cache, w = mixer_setup(layer, dtype, sharp=sharp)
    x = rnd(95, 72, seed=case + 5).to(torch.bfloat16).float()
    want = plain.MIXERS[layer["type"]](x.double(), w, layer["mixer"], 2e-5)
    close(run_in_portions(part, cache, x, CUTS, dtype), want, dtype, "portions", loose=2.0)
    # the same request again in the other slot, one token at a time after a short start: a state or cache row
    # that the first run left behind, or a slot that was not cleared, would show
    cache.release("r")
    cache.admit("filler"); cache.release("filler")
    close(run_in_portions(part, cache, x[:60], (5,) + (1,) * 55, dtype, rid="again"), want[:60], dtype, "token by token", loose=2.0)
    cache.check_invariants()
    m = layer["mixer"]
    if layer["type"] == "latent_attention" and dtype == torch.bfloat16 and m["kv_rank"] % 64 == 0 and m["rot_dim"] % 16 == 0 and m["dim"] % 8 == 0:
        assert served["latent_attention_tc"] > 0, "the tensor-core kernels were meant to serve these sizes"


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
@pytest.mark.parametrize("rank", [40, 64])
@pytest.mark.parametrize("window", [1, 5, 16, 17, 40])
def test_latent_attention_window_edges(window, rank, dtype):
    """Keys just inside and just outside a window, in portions and single tokens; pages the window has passed go back."""
    layer = dh.attn(kv_rank=rank, rot_dim=8 if rank == 40 else 16)
    part, cache, w = mixer_setup(layer, dtype, sharp=3.0, window=window)
    x = rnd(95, 72, seed=3).to(torch.bfloat16).float()
    want = plain.latent_attention(x.double(), w, layer["mixer"], 2e-5, window=window)
    close(run_in_portions(part, cache, x, CUTS, dtype), want, dtype, f"window {window}", loose=2.0)
    if window <= 17:
        assert cache.free_pages() >= cache.num_pages - 3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank,dr", [(32, 4), (64, 16)])
def test_latent_attention_finds_one_far_key(rank, dr, dtype):
    """One key far back among hundreds is made to stand out: input 70 feeds only a barely rotated entry of the shared
    key part and is set at position 3 alone; input 71 feeds the same entry of every head's query and is set from
    position 200 on.  Those queries must then return position 3's value row, through portions and single tokens."""
    m = dh.attn(heads=2, dim=16, rot_dim=dr, vdim=24, kv_rank=rank, scale=1.0, base=1e12 ** (dr / 4))
    H, dn = 2, 16

    def tweak(w):
        w["dkv"][rank + 2] = 0.0
        w["dkv"][rank + 2, 70] = 1.0
        w["q"][:, 71] = 0.0
        for h in range(H):
            w["q"][h * (dn + dr) + dn + 2, 71] = 1.0

    part, cache, w = mixer_setup(m, dtype, seed=4, tweak=tweak)
    x = rnd(230, 72, seed=8)
    x[:, 70:] = 0.0
    x[3, 70] = 8.0
    x[200:, 71] = 4.0
    x = x.to(torch.bfloat16).float()
    want = plain.latent_attention(x.double(), w, m["mixer"], 2e-5)
    got = run_in_portions(part, cache, x, (190, 2, 8) + (1,) * 30, dtype)
    close(got, want, dtype, "far key", loose=2.0)
    blind = x.clone()
    blind[3, 70] = 0.0                                          # what not seeing that key would give
    lost = plain.latent_attention(blind.double(), w, m["mixer"], 2e-5)
    assert float((want[200:] - lost[200:]).abs().amax(dim=-1).min()) > 0.05 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("f", [dh.moe(), dh.moe(experts=3, top=1, ff=16, shared=0), dh.moe(experts=4, top=4, ff=40, shared=8),
                               dh.moe(experts=37, top=2, ff=8, shared=24)])
def test_routed_feed_forward_alone(f, dtype):
    width = 72
    spec = part_spec(dh.layer(dh.mlstm(), f), width, 1e-5).feed_forward
    w = dh.moe_weights(f, width, torch.Generator().manual_seed(2))
    src = TensorSource(tensors={f"l0.mlp.{k}": v.to(torch.bfloat16) for k, v in w.items()}, device=DEV, compute_dtype=dtype)
    part = build_part("feed_forward", spec, src, Runtime(DEV, dtype, 64))
    x = rnd(70, width, seed=6).to(torch.bfloat16).float()
    want = plain.moe(x.double(), {k: v.double() for k, v in w.items()}, f)
    add = rnd(70, width, seed=7).to(dtype)
    for lo, hi in ((0, 70), (0, 1), (1, 3), (3, 40)):           # batches of other sizes group the rows otherwise
        got = part.forward(x[lo:hi].to(dtype).to(DEV), None, add=add[lo:hi].to(DEV).contiguous())
        assert got.dtype == torch.float32
        close(got.cpu() - add[lo:hi].float(), want[lo:hi], dtype, f"rows {lo}:{hi}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_bigram_embedding_alone(dtype):
    from qorvix_b200.parts import BigramEmbeddingSpec
    vocab, width, buckets = 50, 24, 11
    emb, pair = rnd(vocab, width, seed=1).to(torch.bfloat16), rnd(buckets + 1, width, seed=2).to(torch.bfloat16)
    src = TensorSource(tensors={"e": emb, "p": pair}, device=DEV, compute_dtype=dtype)
    mul_prev, mul_cur = (5, 3) if dtype == torch.float32 else (-7, 100003)       # also a negative and a large multiplier
    part = build_part("embedding", BigramEmbeddingSpec(vocab, width, "e", "p", buckets, mul_prev, mul_cur), src, Runtime(DEV, dtype, 64))
    cache = CacheManager([(part.cache_spec(), None)], max_tokens=64, page_size=16, max_requests=2, device=DEV, dtype=dtype)
    toks = [int(t) for t in torch.randint(0, vocab, (40,), generator=torch.Generator().manual_seed(3))]
    want = plain.embed_bigram(toks, emb.double(), pair.double(), buckets, mul_prev, mul_cur)
    builder = BatchBuilder(DEV)
    for rid in ("a", "b", "c"):                                  # 'c' takes the slot 'a' gave back: its first token is a first token
        cache.admit(rid)
        outs, i = [], 0
        for n in (1, 2, 7, 1, 1, 28):
            cache.reserve(rid, n)
            ctx = builder.build([dict(tokens=toks[i:i + n], pos0=i, slot=cache.slot(rid), want=[], first=i == 0)], {}, cache.scratch_page)
            out = torch.empty((n, width), device=DEV, dtype=torch.float32)
            part.forward(out, ctx, cache.layer_view(0))
            outs.append(out)
            cache.commit(rid, n)
            i += n
        assert torch.equal(torch.cat(outs).double().cpu(), want)
        if rid != "b":
            cache.release(rid)


# ---------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module")
def models():
    out = {}
    for name, cfg, sharp in (("A", dh.CONFIG_A, 2.5), ("B", dh.CONFIG_B, 2.0), ("C", dh.CONFIG_C, 2.0)):
        d = dh.make_model_dir(cfg, seed=11 + len(out), sharp=sharp)
        cfg_read, weights = plain.read_model_dir(d)
        out[name] = (d, cfg_read, weights, {})
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_layers(models, name, dtype):
    m = models[name]
    r = runner(m, dtype)
    for n, seed in ((1, 1), (2, 2), (17, 3), (64, 4), (97, 5)):
        toks = tokens(m[1]["vocab"], n, seed)
        out = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        close_model(out, plain_logits(m, toks), dtype, f"whole n={n}")
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
def test_float32_and_bfloat16_do_not_depend_on_the_batch(models, dtype):
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
@pytest.mark.parametrize("name", ["A", "B", "C"])
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
