"""End-to-end parity of the engine (through the C ABI) against the CPU oracle on BASELINE
configuration 0: tiny random-init Llama decoder (seed 0), 4 concurrent sequences with prompt lengths
17/33/64/129, page size 16, greedy continuous-batch decode of 32 tokens each.

The scenarios mirror the reference's own tests: tests/continuous.rs (Exact == batch-1, admit-on-retire
with 5 requests / max_batch 2, cancel semantics, zero budget), tests/streaming.rs (max tokens,
determinism, stop token excluded, empty prompt error), tests/paged.rs and the unit tests of
src/primitives/paged_kv_cache.rs (block accounting, seeded prefixes, truncate, reset)."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, engine
    from oracle import oracle as orc

    ctx = _lib.Context(0)
    weights = H.tiny_weights()
    model = H.build_engine_model(engine, ctx, weights=weights)
    omodel = H.build_oracle_model(orc, weights=weights)
    yield ctx, engine, orc, model, omodel
    model.free()
    ctx.close()


def logits_close(got_bf16, ref_f32):
    """End-to-end logits of a whole decoder.  Every op is checked at 2e-3 / bit-exact in
    test_gpu_kernels.py; chained through two layers, a 1-ulp difference in any bf16 activation
    (2^-8 relative) is amplified by every later rounding, so two faithful bf16 implementations sit
    about 1e-3 rms apart on the logits and a few e-3 apart at the worst of thousands of entries (one
    bf16 ulp of a logit near 1 is 3.9e-3..7.8e-3).  Gate: rms <= 2e-3 and worst entry <= 1e-2."""
    got = H.bf16_to_f32_np(got_bf16)
    err = got - ref_f32
    rms, worst = float(np.sqrt(np.mean(err * err))), float(np.abs(err).max())
    return bool(np.isfinite(got).all() and rms <= 2e-3 and worst <= 1e-2), worst


def undecidable(ref_f32_row, top, other):
    """A greedy step whose two candidates are closer than what the parity bound can resolve: both
    logits may move by 2e-3 and each is then rounded to bf16 (ties go to the lower index)."""
    ulp = 2.0 ** (np.floor(np.log2(max(abs(float(ref_f32_row[top])), 1e-30))) - 7)
    return float(ref_f32_row[top] - ref_f32_row[other]) <= 2 * 2e-3 + ulp


def test_prefill_logits_match_oracle(env):
    ctx, eng, orc, model, omodel = env
    prompts = H.config0_prompts()
    pool = eng.BlockPool(ctx, model, 16, 64, 4, 16)
    caches = [eng.PagedKvCache(pool) for _ in prompts]
    logits, am = model.step(list(zip(prompts, caches)))
    ocs = [orc.Cache(2, block_size=16) for _ in prompts]
    ref, ref_f32 = omodel.forward([(p, c, 0) for p, c in zip(prompts, ocs)])
    ok, err = logits_close(logits, ref_f32)
    assert ok, f"prefill logits max-abs {err}"
    assert [c.offset() for c in caches] == [17, 33, 64, 129]
    assert [c.blocks() for c in caches] == [1, 2, 4, 8]
    assert [c.reserved_tokens() for c in caches] == [32, 48, 64, 144]
    # KV written to the pages equals what the reference's cache would hold
    for c, oc in zip(caches, ocs):
        for layer in range(2):
            k, v = c.gather(layer, 2, 64)
            ok_, ov_ = oc.gather(layer)
            ok_ = ok_.reshape(-1, 2, 64).transpose(1, 0, 2)
            ov_ = ov_.reshape(-1, 2, 64).transpose(1, 0, 2)
            for got_, ref_ in ((k, ok_), (v, ov_)):
                g32, r32 = H.bf16_to_f32_np(got_), H.bf16_to_f32_np(ref_)
                # layer 0 sees identical inputs; layer 1 inherits the 1-ulp differences of layer 0
                err = np.abs(g32 - r32)
                assert np.sqrt(np.mean(err * err)) <= 2e-3 and err.max() <= 2e-2
                assert (got_ != ref_).mean() < 0.5  # differences are isolated 1-ulp roundings, not a shift
    # one decode step over all four (decode_logits_per_seq)
    feed = [[int(a)] for a in am]
    logits2, am2 = model.step(list(zip(feed, caches)))
    ref2, ref2_f32 = omodel.forward([(f, c, c.offset()) for f, c in zip(feed, ocs)])
    ok, err = logits_close(logits2, ref2_f32)
    assert ok, f"decode logits max-abs {err}"
    for c in caches:
        c.free()
    pool.free()


def test_config0_teacher_forced_greedy(env):
    """Feed the ORACLE's greedy streams through the engine and compare the argmax at all 4 x 32
    steps.  Random-init logits over 1024 tokens put the top two candidates within one bf16 ulp at
    roughly one step in ten, so the oracle's per-step top-2 margin is printed, and a disagreement is
    accepted only where that margin is below what the numeric parity bound can resolve."""
    ctx, eng, orc, model, omodel = env
    prompts = H.config0_prompts()
    ref = omodel.generate_continuous(prompts, [32] * 4)
    pool = eng.BlockPool(ctx, model, 16, 64, 4, 16)
    caches = [eng.PagedKvCache(pool) for _ in prompts]
    ocs = [orc.Cache(2, block_size=16) for _ in prompts]
    feed = [p for p in prompts]
    mism, tight, min_margin = [], 0, 1e9
    for step in range(32):
        _, am = model.step(list(zip(feed, caches)), want_logits=False)
        lg, lf = omodel.forward([(f, c, c.offset()) for f, c in zip(feed, ocs)])
        for si in range(4):
            want = ref["tokens"][si][step]
            order = np.argsort(-lf[si])
            margin = float(lf[si][order[0]] - lf[si][order[1]])
            min_margin = min(min_margin, margin)
            tight += undecidable(lf[si], order[0], order[1])
            if int(am[si]) != want:
                mism.append((si, step, int(am[si]), want, float(lf[si][want] - lf[si][int(am[si])])))
                assert undecidable(lf[si], want, int(am[si])), f"decidable step disagrees: {mism[-1]}"
        feed = [[t[step]] for t in ref["tokens"]]
    print(f"[config0 teacher-forced] 128 steps, {tight} within the undecidable margin, min top-2 f32 margin "
          f"{min_margin:.2e}, disagreements (seq, step, engine, oracle, oracle f32 margin): {mism}")
    assert len(mism) <= 4
    for c in caches:
        c.free()
    pool.free()


@pytest.mark.parametrize("mode", ["exact", "throughput", "chunked"])
def test_config0_greedy_identity_and_block_tables(env, mode):
    ctx, eng, orc, model, omodel = env
    prompts = H.config0_prompts()
    ref = omodel.generate_continuous(prompts, [32] * 4, max_batch=8, block_size=16)
    reqs = [eng.BatchRequest(p.tolist(), 32) for p in prompts]
    cfg = eng.ContinuousConfig(max_batch=8, block_size=16, exactness=eng.EXACT if mode == "exact" else eng.THROUGHPUT,
                               prefill_chunk_tokens=48 if mode == "chunked" else 0)
    events = []
    outs, stats = eng.generate_continuous(model, reqs, cfg, on_event=lambda i, e: events.append((i,) + e), return_stats=True)
    got = [o.tokens for o in outs]
    # Streams must be identical up to the first step the parity bound cannot decide (see
    # test_config0_teacher_forced_greedy for the per-step margins); at that step the engine's token
    # must be the oracle's runner-up within the undecidable margin.
    identical = 0
    for si, (g, r) in enumerate(zip(got, ref["tokens"])):
        if g == r:
            identical += 1
            continue
        k = next(j for j in range(32) if g[j] != r[j])
        oc = orc.Cache(2, block_size=16)
        _, lf = omodel.forward([(prompts[si], oc, 0)])
        for t in r[:k]:
            _, lf = omodel.forward([([t], oc, oc.offset())])
        assert undecidable(lf[0], r[k], g[k]), (
            f"sequence {si} diverges at step {k} ({g[k]} vs {r[k]}) with an oracle f32 margin of "
            f"{float(lf[0][r[k]] - lf[0][g[k]]):.3e}: that step is decidable")
    print(f"[config0/{mode}] sequences identical to the oracle for all 32 tokens: {identical}/4")
    assert identical >= 2
    assert [o.finish_reason for o in outs] == [eng.MAX_TOKENS] * 4
    assert all(len(t) == 32 for t in got)
    if mode != "chunked":  # chunking staggers the sequences, so fewer blocks are live at once
        assert stats["peak_live_blocks"] == 22  # fill-order ids 0..21 of the reference's allocator
    if mode != "chunked":
        # same event order as the reference loop: (request, kind, step/generated); token ids are
        # compared above
        exp = [(r, "token" if k == 0 else "done", b) for r, k, a, b in ref["events"]]
        assert [(e[0], e[1], e[3]) for e in events] == exp
    else:
        # chunking interleaves requests differently but every request sees Token* then one Done
        for r in range(4):
            mine = [e for e in events if e[0] == r]
            assert [e[1] for e in mine] == ["token"] * 32 + ["done"]
            assert [e[3] for e in mine[:-1]] == list(range(32))


def test_block_ids_match_reference_rules(env):
    """Block ids are handed out when a block fills, in lane order: prompts 17/33/64/129 then 31 decode
    steps give seq0 [0,15,19], seq1 [1,2,16,20], seq2 [3,4,5,6,18], seq3 [7..14,17,21]."""
    ctx, eng, orc, model, omodel = env
    prompts = H.config0_prompts()
    pool = eng.BlockPool(ctx, model, 16, 64, 4, 16)
    caches = [eng.PagedKvCache(pool) for _ in prompts]
    feed = []
    for p, c in zip(prompts, caches):  # admission order: one prefill each
        _, am = model.step([(p, c)], want_logits=False)
        feed.append([int(am[0])])
    for _ in range(31):
        _, am = model.step(list(zip(feed, caches)), want_logits=False)
        feed = [[int(a)] for a in am]
    assert [c.block_ids() for c in caches] == [[0, 15, 19], [1, 2, 16, 20], [3, 4, 5, 6, 18], [7, 8, 9, 10, 11, 12, 13, 14, 17, 21]]
    assert [c.offset() for c in caches] == [48, 64, 95, 160]
    st = pool.stats()
    assert st["live_blocks"] == 22 and st["peak_live_blocks"] == 22 and st["reserved_tokens"] == 22 * 16
    ref = omodel.generate_continuous(prompts, [32] * 4)
    assert [c.block_ids() for c in caches] == ref["block_ids"]
    for c in caches:
        c.free()
    assert pool.stats()["live_blocks"] == 0
    pool.free()


def test_admit_on_retire_matches_batch1(env):
    """5 requests through 2 slots with budgets 4,8,6,10,12 (tests/continuous.rs:123-149): every row
    equals its batch-1 generate() run, and the event stream equals the reference loop's."""
    ctx, eng, orc, model, omodel = env
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 1024, size=n).astype(np.int32) for n in (9, 21, 16, 40, 5)]
    budgets = [4, 8, 6, 10, 12]
    reqs = [eng.BatchRequest(p.tolist(), b) for p, b in zip(prompts, budgets)]
    events = []
    outs = eng.generate_continuous(model, reqs, eng.ContinuousConfig(max_batch=2, block_size=16, exactness=eng.EXACT),
                                   on_event=lambda i, e: events.append((i,) + e))
    for p, b, o in zip(prompts, budgets, outs):
        single = eng.generate(model, p.tolist(), b)
        assert o.tokens == single.tokens and len(o.tokens) == b and o.finish_reason == eng.MAX_TOKENS
    ref = omodel.generate_continuous(prompts, budgets, max_batch=2)
    assert [o.tokens for o in outs] == ref["tokens"]
    assert events == [(r, "token" if k == 0 else "done", a, b) for r, k, a, b in ref["events"]]
    # determinism (tests/streaming.rs:118-130)
    outs2 = eng.generate_continuous(model, reqs, eng.ContinuousConfig(max_batch=2, block_size=16, exactness=eng.THROUGHPUT))
    assert [o.tokens for o in outs2] == [o.tokens for o in outs]


def test_stop_token_excluded_and_zero_budget(env):
    ctx, eng, orc, model, omodel = env
    prompts = H.config0_prompts()[:2]
    base = eng.generate(model, prompts[0].tolist(), 12)
    stop = base.tokens[5]
    first = base.tokens.index(stop)
    out = eng.generate(model, prompts[0].tolist(), 12, stop_tokens=[stop])
    assert out.tokens == base.tokens[:first] and out.finish_reason == eng.STOP_TOKEN
    oref = omodel.generate(prompts[0], 12, stop=[stop])
    assert out.tokens == oref["tokens"] and oref["reason"] == 0
    events = []
    reqs = [eng.BatchRequest(prompts[0].tolist(), 0), eng.BatchRequest(prompts[1].tolist(), 3, stop_tokens=[stop])]
    outs = eng.generate_continuous(model, reqs, eng.ContinuousConfig(), on_event=lambda i, e: events.append((i,) + e))
    assert outs[0].tokens == [] and outs[0].finish_reason == eng.MAX_TOKENS  # zero budget: Done{MaxTokens, 0}, no prefill
    assert events[0] == (0, "done", eng.MAX_TOKENS, 0)
    ref = omodel.generate_continuous(prompts, [0, 3], stops=[[], [stop]])
    assert [o.tokens for o in outs] == ref["tokens"] and [o.finish_reason for o in outs] == ref["reasons"]


def test_errors_and_cancel(env):
    ctx, eng, orc, model, omodel = env
    from mlx_llm_b200._lib import B2Error

    prompts = H.config0_prompts()
    with pytest.raises(B2Error) as e:
        eng.generate_continuous(model, [], eng.ContinuousConfig())
    assert e.value.code == -7
    with pytest.raises(B2Error):
        eng.generate_continuous(model, [eng.BatchRequest([], 4)], eng.ContinuousConfig())
    with pytest.raises(B2Error):
        eng.generate_continuous(model, [eng.BatchRequest([1, 2], 4)], eng.ContinuousConfig(max_batch=0))
    with pytest.raises(B2Error):
        eng.generate_continuous(model, [eng.BatchRequest([1, 2], 4)], eng.ContinuousConfig(block_size=0))
    with pytest.raises(B2Error):
        eng.generate(model, [], 4)
    with pytest.raises(B2Error) as e:  # non-greedy sampling is not on the device path
        eng.generate_continuous(model, [eng.BatchRequest([1, 2], 4, sampling=eng.SamplingParams(temperature=0.8))], eng.ContinuousConfig())
    assert e.value.code == -5
    # pre-set cancel is a typed error (continuous.rs:138-140)
    flag = eng.CancelFlag()
    flag.cancel()
    with pytest.raises(B2Error) as e:
        eng.generate_continuous(model, [eng.BatchRequest(prompts[0].tolist(), 4)], eng.ContinuousConfig(), cancel=flag)
    assert e.value.code == -6
    # mid-stream cancel: 6 requests, 2 slots; every request gets exactly one Done (continuous.rs:198-214)
    flag = eng.CancelFlag()
    events = []

    def on_event(i, e):
        events.append((i,) + e)
        if sum(1 for x in events if x[1] == "token") >= 7:
            flag.cancel()

    reqs = [eng.BatchRequest(prompts[i % 4].tolist(), 0 if i == 5 else 20) for i in range(6)]
    outs = eng.generate_continuous(model, reqs, eng.ContinuousConfig(max_batch=2), cancel=flag, on_event=on_event)
    dones = [e for e in events if e[1] == "done"]
    assert sorted(d[0] for d in dones) == list(range(6))
    assert [o.finish_reason for o in outs[:5]] == [eng.CANCELLED] * 5
    assert outs[5].finish_reason == eng.MAX_TOKENS and outs[5].tokens == []  # zero-budget request keeps MaxTokens
    assert sum(len(o.tokens) for o in outs) <= 9  # stops within one step of the flag
    # single-sequence loop: mid-stream cancel keeps the partial output (stream.rs:9-12)
    flag = eng.CancelFlag()
    seen = []

    def on_ev(e):
        seen.append(e)
        if len(seen) == 3:
            flag.cancel()

    out = eng.generate(model, prompts[1].tolist(), 20, cancel=flag, on_event=on_ev)
    assert out.finish_reason == eng.CANCELLED and len(out.tokens) == 3 and seen[-1] == ("done", eng.CANCELLED, 3)


def test_seeded_prefix_truncate_reset(env):
    """Copy-on-write prefix sharing, truncate and reset on real pages (paged_kv_cache.rs:642-787,
    scaled to 16-token blocks)."""
    ctx, eng, orc, model, omodel = env
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 1024, size=40).astype(np.int32)
    pool = eng.BlockPool(ctx, model, 16, 32, 4, 8)
    a = eng.PagedKvCache(pool)
    la, _ = model.step([(ids, a)])
    assert (a.offset(), a.blocks(), a.reserved_tokens()) == (40, 2, 48)
    assert pool.live_blocks() == 2 and pool.shared_blocks() == 0
    shared = a.shareable_prefix_blocks(40)
    assert shared == a.block_ids()[:2] and a.shareable_prefix_blocks(15) == []
    b = eng.PagedKvCache.new_seeded(pool, shared)
    assert b.offset() == 32 and pool.live_blocks() == 2 and pool.shared_blocks() == 2
    lb, _ = model.step([(ids[32:], b)])  # recompute only the suffix
    assert np.array_equal(lb, la), "seeded prefix + suffix must reproduce the cold run"
    assert pool.shared_blocks() == 2, "divergence touches only the private tail"
    for layer in range(2):
        ka, va = a.gather(layer, 2, 64)
        kb, vb = b.gather(layer, 2, 64)
        assert np.array_equal(ka, kb) and np.array_equal(va, vb)
    # truncate B into the shared second block: B must get a private copy, A stays intact
    ka_before = a.gather(0, 2, 64)[0].copy()
    b.truncate(20)
    assert (b.offset(), b.blocks()) == (20, 1) and pool.shared_blocks() == 1
    lb2, _ = model.step([(ids[20:], b)])
    assert np.array_equal(lb2, la)
    assert np.array_equal(a.gather(0, 2, 64)[0], ka_before)
    b.free()
    assert pool.shared_blocks() == 0 and pool.live_blocks() == 2
    # truncate within the tail / onto a boundary / no-op / negative (paged_kv_cache.rs:743-768)
    a.truncate(36)
    assert (a.offset(), a.blocks()) == (36, 2)
    a.truncate(20)
    assert (a.offset(), a.blocks()) == (20, 1) and pool.live_blocks() == 1
    a.truncate(16)
    assert (a.offset(), a.blocks(), a.reserved_tokens()) == (16, 1, 16)
    a.truncate(100)
    assert a.offset() == 16
    from mlx_llm_b200._lib import B2Error
    with pytest.raises(B2Error):
        a.truncate(-1)
    la2, _ = model.step([(ids[16:], a)])  # rollback then replay gives the same logits
    assert np.array_equal(la2, la)
    with pytest.raises(B2Error):
        a.retain_sequences([1])
    a.retain_sequences([0])
    assert a.offset() == 40
    a.reset()
    assert a.offset() == 0 and a.batch_size() == 0 and pool.live_blocks() == 0
    a.retain_sequences([])
    a.free()
    st = pool.stats()
    assert st["free_pages"] == st["total_pages"]
    pool.free()


def test_pool_exhaustion_is_an_error_not_a_fault(env):
    ctx, eng, orc, model, omodel = env
    from mlx_llm_b200._lib import B2Error

    pool = eng.BlockPool(ctx, model, 16, 2, 1, 8)
    c = eng.PagedKvCache(pool)
    with pytest.raises(B2Error) as e:
        model.step([(np.arange(40, dtype=np.int32), c)])
    assert e.value.code == -8
    with pytest.raises(B2Error):
        eng.PagedKvCache(pool)  # no free block-table row
    c.free()
    pool.free()


def test_quantize_on_load_q4_q8(env):
    """Quantize-on-load (CausalLm::from_weights_with with a QuantSpec): generation through the Q4/Q8
    projections equals the oracle run on the same quantized weights.  intermediate_size 688 is not a
    multiple of the group size, so this uses a 640-wide variant of the tiny model."""
    ctx, eng, orc, model, omodel = env
    cfg = dict(H.CONFIG0, inter=640)
    weights = H.tiny_weights(cfg, seed=7)
    prompts = H.config0_prompts(seed=9)[:3]
    for bits in (4, 8):
        qm = H.build_engine_model(eng, ctx, cfg, weights, quant=eng.QuantSpec(64, bits))
        assert qm.is_quantized()
        om = H.build_oracle_model(orc, cfg, weights, quant_bits=bits)
        pool = eng.BlockPool(ctx, qm, 16, 64, 4, 16)
        caches = [eng.PagedKvCache(pool) for _ in prompts]
        logits, _ = qm.step(list(zip(prompts, caches)))
        ocs = [orc.Cache(2, block_size=16) for _ in prompts]
        _, ref_f32 = om.forward([(p, c, 0) for p, c in zip(prompts, ocs)])
        ok, err = logits_close(logits, ref_f32)
        assert ok, f"Q{bits} logits max-abs {err}"
        for c in caches:
            c.free()
        pool.free()
        qm.free()
    from mlx_llm_b200._lib import B2Error
    with pytest.raises(B2Error):  # group size must divide the input dimension (688 % 64 != 0)
        H.build_engine_model(eng, ctx, H.CONFIG0, H.tiny_weights(), quant=eng.QuantSpec(64, 4))


def test_seeded_then_truncated_before_any_step(env):
    """A seeded cache truncated into its shared block BEFORE any forward: two block-table writes for one
    (row, index) are pending at once, and the private copy must win, or the sequence would append into a page its
    donor still reads.  Then a seeded cache freed before its first step, whose row goes to a new cache."""
    ctx, eng, orc, model, omodel = env
    rng = np.random.default_rng(15)
    ids = rng.integers(0, 1024, size=40).astype(np.int32)
    pool = eng.BlockPool(ctx, model, 16, 32, 2, 8)
    a = eng.PagedKvCache(pool)
    la, _ = model.step([(ids, a)])
    donor = [a.gather(l, 2, 64) for l in range(2)]
    b = eng.PagedKvCache.new_seeded(pool, a.shareable_prefix_blocks(40))
    b.truncate(20)                      # no step in between: (row, 1) -> shared page, then -> private copy
    other = rng.integers(0, 1024, size=20).astype(np.int32)
    model.step([(other, b)])            # overwrites positions 20..39 of b's private copy
    for l in range(2):
        k, v = a.gather(l, 2, 64)
        assert np.array_equal(k, donor[l][0]) and np.array_equal(v, donor[l][1]), "the donor's pages were written"
    b.truncate(20)
    lb, _ = model.step([(ids[20:], b)])
    assert np.array_equal(lb, la)
    b.free()
    c = eng.PagedKvCache.new_seeded(pool, a.shareable_prefix_blocks(40))   # takes the row b had
    c.free()                                                                # freed before its first step
    d = eng.PagedKvCache(pool)                                              # same row again, cold
    ld, _ = model.step([(ids, d)])
    assert np.array_equal(ld, la)
    for l in range(2):
        k, v = a.gather(l, 2, 64)
        assert np.array_equal(k, donor[l][0]) and np.array_equal(v, donor[l][1])
    for x in (a, d):
        x.free()
    pool.free()


@pytest.mark.parametrize("mode", ["exact", "chunked"])
def test_staggered_arrivals_are_all_served(env, mode):
    """Requests that arrive later than the lanes drain (arrival_s extension): the loop must idle until the next
    arrival instead of ending, in the reference's schedule as well as in the chunked one."""
    ctx, eng, orc, model, omodel = env
    prompts = H.config0_prompts()[:3]
    reqs = [eng.BatchRequest(p.tolist(), 4, arrival_s=0.05 + 0.15 * i) for i, p in enumerate(prompts)]  # none at t = 0
    events = []
    cfg = eng.ContinuousConfig(max_batch=2, block_size=16, exactness=eng.EXACT, prefill_chunk_tokens=32 if mode == "chunked" else 0)
    outs = eng.generate_continuous(model, reqs, cfg, on_event=lambda i, e: events.append((i,) + e))
    assert [o.finish_reason for o in outs] == [eng.MAX_TOKENS] * 3 and all(len(o.tokens) == 4 for o in outs)
    assert sorted(e[0] for e in events if e[1] == "done") == [0, 1, 2]
    for p, o in zip(prompts, outs):
        assert o.tokens == eng.generate(model, p.tolist(), 4).tokens


def test_duplicate_cache_in_a_large_step_is_rejected(env):
    ctx, eng, orc, model, omodel = env
    from mlx_llm_b200._lib import B2Error

    pool = eng.BlockPool(ctx, model, 16, 200, 80, 2)
    caches = [eng.PagedKvCache(pool) for _ in range(70)]
    seqs = [([1, 2, 3], c) for c in caches] + [([4], caches[68])]
    with pytest.raises(B2Error) as e:
        model.step(seqs)
    assert e.value.code == -7 and all(c.offset() == 0 for c in caches)
    model.step([([1, 2, 3], c) for c in caches])   # the pool is still consistent
    assert all(c.offset() == 3 for c in caches)
    for c in caches:
        c.free()
    pool.free()


# ---- configuration 0 as BASELINE words it: fp32 -----------------------------------------------------------------------
CONFIG0_F32 = dict(H.CONFIG0, f32_mode=1)


@pytest.fixture(scope="module")
def env32():
    """The tiny decoder with f32 weights, activations, pages and logits on both sides.  Engine and oracle then run
    the same arithmetic in the same order (see csrc/engine_step_f32.cu), so the stated targets hold strictly."""
    from mlx_llm_b200 import _lib, engine
    from oracle import oracle as orc

    ctx = _lib.Context(0)
    weights = H.tiny_weights()
    model = H.build_engine_model(engine, ctx, CONFIG0_F32, weights=weights)
    omodel = H.build_oracle_model(orc, CONFIG0_F32, weights=weights)
    yield ctx, engine, orc, model, omodel
    model.free()
    ctx.close()


def test_config0_f32_logits_and_pages_strict(env32):
    ctx, eng, orc, model, omodel = env32
    assert model.config().compute_f32 == 1 and not model.is_quantized()
    prompts = H.config0_prompts()
    pool = eng.BlockPool(ctx, model, 16, 64, 4, 16)
    caches = [eng.PagedKvCache(pool) for _ in prompts]
    ocs = [orc.Cache(2, block_size=16) for _ in prompts]
    feed, worst = prompts, 0.0
    for step in range(6):   # one ragged prefill, then five decode steps over all four sequences
        logits, am = model.step(list(zip(feed, caches)))
        assert logits.dtype == np.float32
        _, ref = omodel.forward([(f, c, c.offset()) for f, c in zip(feed, ocs)])
        err = float(np.abs(logits - ref).max())
        worst = max(worst, err)
        assert err <= 2e-3, f"step {step}: logits max-abs {err}"
        assert am.tolist() == [int(np.argmax(r)) for r in ref]
        feed = [[int(a)] for a in am]
    print(f"[config0 f32] worst logits max-abs over 6 steps: {worst:.3e}")
    assert worst <= 1e-4   # in practice the two sides differ by the last bits of exp() only
    for c, oc in zip(caches, ocs):
        for layer in range(2):
            k, v = c.gather_f32(layer, 2, 64)
            ok_, ov_ = oc.gather(layer)
            ok_ = ok_.view(np.float32).reshape(-1, 2, 64).transpose(1, 0, 2)
            ov_ = ov_.view(np.float32).reshape(-1, 2, 64).transpose(1, 0, 2)
            assert np.abs(k - ok_).max() <= 1e-5 and np.abs(v - ov_).max() <= 1e-5
            if layer == 0:
                assert np.array_equal(v, ov_)   # before any exp(): the same multiplies and adds in the same order
    from mlx_llm_b200._lib import B2Error
    with pytest.raises(B2Error):
        caches[0].gather(0, 2, 64)   # bf16 view of f32 pages
    for c in caches:
        c.free()
    pool.free()


@pytest.mark.parametrize("mode", ["exact", "throughput", "chunked"])
def test_config0_f32_greedy_streams_identical(env32, mode):
    """The stated target: greedy token streams identical to the reference loop's for all 32 tokens of all four
    sequences (tests/continuous.rs:92-118), in every schedule."""
    ctx, eng, orc, model, omodel = env32
    prompts = H.config0_prompts()
    ref = omodel.generate_continuous(prompts, [32] * 4, max_batch=8, block_size=16)
    reqs = [eng.BatchRequest(p.tolist(), 32) for p in prompts]
    cfg = eng.ContinuousConfig(max_batch=8, block_size=16, exactness=eng.EXACT if mode == "exact" else eng.THROUGHPUT,
                               prefill_chunk_tokens=48 if mode == "chunked" else 0)
    events = []
    outs, stats = eng.generate_continuous(model, reqs, cfg, on_event=lambda i, e: events.append((i,) + e), return_stats=True)
    identical = sum(o.tokens == r for o, r in zip(outs, ref["tokens"]))
    assert identical == 4, [next((j for j in range(32) if o.tokens[j] != r[j]), None) for o, r in zip(outs, ref["tokens"])]
    assert [o.finish_reason for o in outs] == [eng.MAX_TOKENS] * 4
    if mode != "chunked":
        assert stats["peak_live_blocks"] == 22
        assert events == [(r, "token" if k == 0 else "done", a, b) for r, k, a, b in ref["events"]]
    for p, o in zip(prompts[:2], outs[:2]):   # and equal to the single-sequence loop (generate)
        assert eng.generate(model, p.tolist(), 32).tokens == o.tokens


def test_config0_f32_streams_match_committed_fixture(env32):
    """The committed golden fixture (tests/golden/config0.json, written by tests/golden/gen_config0.py from the CPU
    oracle): all four greedy streams of the f32 engine, 32 tokens each, and the block-id table of the run."""
    import json
    import os

    ctx, eng, orc, model, omodel = env32
    with open(os.path.join(os.path.dirname(__file__), "golden", "config0.json")) as f:
        g = json.load(f)
    if g["weights_crc"] != H.weights_crc(H.tiny_weights()):
        pytest.skip("this platform's libm draws different Box-Muller weights than the fixture's")
    reqs = [eng.BatchRequest(p, 32) for p in g["prompts"]]
    outs = eng.generate_continuous(model, reqs, eng.ContinuousConfig(max_batch=8, block_size=16, exactness=eng.THROUGHPUT))
    assert [o.tokens for o in outs] == g["tokens_f32"]


def test_f32_model_limits(env32):
    ctx, eng, orc, model, omodel = env32
    from mlx_llm_b200._lib import B2Error

    with pytest.raises(B2Error) as e:   # no quantize-on-load on the f32 path
        H.build_engine_model(eng, ctx, dict(CONFIG0_F32, inter=640), H.tiny_weights(dict(H.CONFIG0, inter=640)), quant=eng.QuantSpec(64, 4))
    assert e.value.code == -5
    with pytest.raises(B2Error):
        eng.CausalLm.synthetic(ctx, H.engine_config(eng, CONFIG0_F32), seed=0)


def test_nvtx_ranges_do_not_change_a_step(env):
    """With NVTX ranges on (no tool attached: the calls are no-ops) a step gives the same logits and launches."""
    ctx, eng, model = env[0], env[1], env[3]
    prompts = H.config0_prompts()
    outs = []
    for on in (False, True):
        ctx.nvtx(on)
        pool = eng.BlockPool(ctx, model, 16, 32, 4, 16)
        caches = [eng.PagedKvCache(pool) for _ in range(2)]
        n0 = ctx.launch_count()
        logits, am = model.step([(prompts[0], caches[0]), (prompts[1], caches[1])])
        outs.append((logits.copy(), am.copy(), ctx.launch_count() - n0))
        for c in caches:
            c.free()
        pool.free()
    ctx.nvtx(False)
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1]) and outs[0][2] == outs[1][2]

