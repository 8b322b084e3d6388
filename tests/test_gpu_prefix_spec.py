"""Shared-prefix KV reuse and prompt-lookup speculative decoding on the paged cache, through the C ABI.

Scenarios follow the reference's own suites (tests/prefix.rs:72-117, tests/speculative.rs:47-108), which need a real
snapshot; here the tiny random-init decoder of configuration 0 stands in.  The f32 model is the strict case: reuse
and speculation must not change a single token, and every counter must equal the CPU restatement of the policy
(oracle/policies.py).  On the bf16 model a reused prefix was computed by a forward of another shape, whose f32 sums
may round differently (the reference documents the same for its verify forward, src/decode/speculative.rs:15-26): there
the counters are exact and the streams must agree up to the first near-tie."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

CONFIG0_F32 = dict(H.CONFIG0, f32_mode=1)


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, engine
    from oracle import oracle as orc
    from oracle import policies

    ctx = _lib.Context(0)
    weights = H.tiny_weights()
    m32 = H.build_engine_model(engine, ctx, CONFIG0_F32, weights=weights)
    m16 = H.build_engine_model(engine, ctx, H.CONFIG0, weights=weights)
    o32 = H.build_oracle_model(orc, CONFIG0_F32, weights=weights)
    yield ctx, engine, orc, policies, m32, m16, o32
    m32.free()
    m16.free()
    ctx.close()


def repetitive_prompt(rng, period=7, reps=6):
    base = rng.integers(0, 1024, size=period).tolist()
    return base * reps


def test_cache_fork_shares_whole_blocks_and_copies_the_partial_one(env):
    ctx, eng, orc, pol, m32, m16, o32 = env
    rng = np.random.default_rng(21)
    ids = rng.integers(0, 1024, size=45).astype(np.int32)
    pool = eng.BlockPool(ctx, m16, 16, 32, 4, 8)
    a = eng.PagedKvCache(pool)
    la, _ = m16.step([(ids, a)])
    for keep in (32, 37, 16, 5, 45):
        b = a.fork(keep)
        assert (b.offset(), b.blocks()) == (keep, keep // 16)
        assert pool.shared_blocks() == keep // 16
        lb, _ = m16.step([(ids[keep:], b)]) if keep < 45 else (None, None)
        if keep < 45:
            assert np.array_equal(lb, la), keep            # the fork continues exactly like the cold run
        kb, vb = b.gather(0, 2, 64)
        ka, va = a.gather(0, 2, 64)
        assert np.array_equal(kb[:, :keep], ka[:, :keep]) and np.array_equal(vb[:, :keep], va[:, :keep])
        b.free()
        assert pool.shared_blocks() == 0
    from mlx_llm_b200._lib import B2Error
    with pytest.raises(B2Error):
        a.fork(46)
    a.free()
    st = pool.stats()
    assert st["free_pages"] == st["total_pages"] and st["live_blocks"] == 0
    pool.free()


def test_prefix_reuse_f32_is_token_exact_and_counted(env):
    """run_suite of tests/prefix.rs:72-117: two prompts sharing a system prefix, then the first prompt again."""
    ctx, eng, orc, pol, m32, m16, o32 = env
    rng = np.random.default_rng(22)
    sys_p = rng.integers(0, 1024, size=37).tolist()
    q1, q2 = rng.integers(0, 1024, size=9).tolist(), rng.integers(0, 1024, size=14).tolist()
    q2[0] = (q1[0] + 1) % 1024                        # the questions diverge right after the prefix
    p1, p2 = sys_p + q1, sys_p + q2
    base1, base2 = eng.generate(m32, p1, 24).tokens, eng.generate(m32, p2, 24).tokens
    assert base1 == o32.generate(p1, 24)["tokens"] and base2 == o32.generate(p2, 24)["tokens"]   # the cold runs are the oracle's
    pc, sim = eng.PrefixCache(ctx, m32, 16, max_pages=64, max_blocks_per_seq=16), pol.PrefixPolicy(16)

    def run(prompt, base):
        reused = sim.lookup(prompt)
        out = eng.generate_cached(m32, prompt, len(base), pc)
        assert out.tokens == base and out.finish_reason == eng.MAX_TOKENS
        sim.store(prompt + out.tokens, len(prompt) + len(out.tokens) - 1)
        assert pc.stats() == sim.stats and len(pc) == len(sim.entries)
        return reused

    assert run(p1, base1) == 0
    assert pc.stats()["hits"] == 0 and pc.stats()["computed_prefill_tokens"] == len(p1)
    assert run(p2, base2) == len(sys_p)               # the whole system span is reused, not a page multiple of it
    assert pc.stats()["hits"] == 1 and pc.stats()["computed_prefill_tokens"] == len(p1) + len(q2)
    assert run(p1, base1) == len(p1) - 1              # whole-prompt reuse recomputes the last prompt token only
    assert pc.stats()["hits"] == 2 and pc.stats()["reused_prefix_tokens"] == len(sys_p) + len(p1) - 1
    # a conversation that grows: every turn reuses everything before it
    turn = p1 + base1 + rng.integers(0, 1024, size=5).tolist()
    cold = eng.generate(m32, turn, 8).tokens
    assert run(turn, cold) == len(p1) + len(base1) - 1
    # events and the stop token, as in the plain loop
    events = []
    stop = cold[3]
    out = eng.generate_cached(m32, turn, 8, pc, stop_tokens=[stop], on_event=events.append)
    assert out.tokens == cold[:cold.index(stop)] and out.finish_reason == eng.STOP_TOKEN and events[-1] == ("done", eng.STOP_TOKEN, len(out.tokens))
    pc.free()


def test_prefix_cache_eviction_and_errors(env):
    ctx, eng, orc, pol, m32, m16, o32 = env
    from mlx_llm_b200._lib import B2Error

    rng = np.random.default_rng(23)
    prompts = [rng.integers(0, 1024, size=n).tolist() for n in (20, 33, 18, 40)]
    cold = [eng.generate(m32, p, 6).tokens for p in prompts]
    # capacity 1: only the last sequence survives; capacity 0 keeps nothing
    for cap in (1, 0):
        pc, sim = eng.PrefixCache(ctx, m32, cap, max_pages=32, max_blocks_per_seq=8), pol.PrefixPolicy(cap)
        for p, c in list(zip(prompts, cold)) + [(prompts[3], cold[3]), (prompts[0], cold[0])]:
            sim.lookup(p)
            out = eng.generate_cached(m32, p, 6, pc)
            assert out.tokens == c
            sim.store(p + out.tokens, len(p) + len(out.tokens) - 1)
            assert pc.stats() == sim.stats and len(pc) == len(sim.entries) == min(cap, 1)
        pc.free()
    # a pool too small for every stored sequence: the least recently used ones make room, results stay exact
    pc = eng.PrefixCache(ctx, m32, 8, max_pages=7, max_blocks_per_seq=4)
    for _ in range(2):
        for p, c in zip(prompts, cold):
            assert eng.generate_cached(m32, p, 6, pc).tokens == c
    assert 1 <= len(pc) <= 3
    with pytest.raises(B2Error):
        eng.generate_cached(m32, [], 4, pc)
    flag = eng.CancelFlag()
    flag.cancel()
    with pytest.raises(B2Error) as e:
        eng.generate_cached(m32, prompts[0], 4, pc, cancel=flag)
    assert e.value.code == -6
    with pytest.raises(B2Error):
        eng.generate_cached(m16, prompts[0], 4, pc)   # the cache belongs to another model
    pc.free()


def test_prefix_reuse_bf16_counts_and_tracks(env):
    ctx, eng, orc, pol, m32, m16, o32 = env
    rng = np.random.default_rng(24)
    sys_p = rng.integers(0, 1024, size=48).tolist()
    pc, sim = eng.PrefixCache(ctx, m16, 4, max_pages=64, max_blocks_per_seq=16), pol.PrefixPolicy(4)
    same = 0
    for i in range(4):
        p = sys_p + rng.integers(0, 1024, size=6 + i).tolist()
        cold = eng.generate(m16, p, 16).tokens
        sim.lookup(p)
        out = eng.generate_cached(m16, p, 16, pc)
        sim.store(p + out.tokens, len(p) + len(out.tokens) - 1)
        assert pc.stats() == sim.stats
        cp = next((j for j in range(16) if out.tokens[j] != cold[j]), 16)
        assert cp >= 1
        same += cp == 16
    print(f"[prefix reuse, bf16] {same}/4 cached streams identical to their cold runs for all 16 tokens")
    assert pc.stats()["hits"] == 3 and pc.stats()["reused_prefix_tokens"] >= 3 * 48
    pc.free()


def test_prompt_lookup_f32_equals_oracle_and_plain_greedy(env):
    ctx, eng, orc, pol, m32, m16, o32 = env
    rng = np.random.default_rng(25)
    prompts = [H.config0_prompts()[0].tolist(), repetitive_prompt(rng), rng.integers(0, 1024, size=30).tolist()]
    total_accepted = 0
    for p in prompts:
        base = eng.generate(m32, p, 40).tokens
        # the exactness gate (tests/speculative.rs:52-66): no drafts -> the plain loop, one forward per token
        out0, st0 = eng.generate_prompt_lookup(m32, p, 40, eng.SpeculativeConfig(3, 0))
        assert out0.tokens == base and st0 == dict(forwards=40, proposed=0, accepted=0)
        for spec in (eng.SpeculativeConfig(3, 4), eng.SpeculativeConfig(2, 7), eng.SpeculativeConfig(1, 1)):
            events = []
            out, st = eng.generate_prompt_lookup(m32, p, 40, spec, on_event=events.append)
            ref_tokens, ref_finish, ref_st = pol.generate_prompt_lookup(o32, orc.Cache(2, block_size=16), p, 40, spec.max_ngram, spec.num_draft)
            assert out.tokens == ref_tokens == base and out.finish_reason == ref_finish == eng.MAX_TOKENS
            assert st == ref_st
            assert [e[1] for e in events[:-1]] == base and [e[2] for e in events[:-1]] == list(range(40)) and events[-1] == ("done", eng.MAX_TOKENS, 40)
            assert st["forwards"] <= 40 and st["forwards"] == 40 - st["accepted"]
            total_accepted += st["accepted"]
    assert total_accepted > 0, "a greedy random-init decoder repeats itself: some drafts must be accepted"
    # stop token inside an accepted run, zero budget, errors
    p = prompts[1]
    base = eng.generate(m32, p, 40).tokens
    stop = base[17]
    out, st = eng.generate_prompt_lookup(m32, p, 40, eng.SpeculativeConfig(3, 4), stop_tokens=[stop])
    ref_tokens, ref_finish, ref_st = pol.generate_prompt_lookup(o32, orc.Cache(2, block_size=16), p, 40, 3, 4, stop=(stop,))
    assert out.tokens == ref_tokens == base[:base.index(stop)] and out.finish_reason == eng.STOP_TOKEN and st == ref_st
    out, st = eng.generate_prompt_lookup(m32, p, 0)
    assert out.tokens == [] and st["forwards"] == 0
    from mlx_llm_b200._lib import B2Error
    with pytest.raises(B2Error):
        eng.generate_prompt_lookup(m32, [], 4)
    with pytest.raises(B2Error):
        eng.generate_prompt_lookup(m32, p, 4, eng.SpeculativeConfig(0, 4))


def test_prompt_lookup_bf16_tracks_plain_greedy(env):
    """tests/speculative.rs:68-96 on the bf16 model: fewer forwards than tokens when drafts are accepted, and the
    stream tracks the non-speculative one (it may leave it only at a near-tie of the multi-token verify forward)."""
    ctx, eng, orc, pol, m32, m16, o32 = env
    p = H.config0_prompts()[0].tolist()   # this prompt sends the tiny decoder into a repeating stream
    base = eng.generate(m16, p, 48).tokens
    out0, st0 = eng.generate_prompt_lookup(m16, p, 48, eng.SpeculativeConfig(3, 0))
    assert out0.tokens == base and st0["forwards"] == 48
    out, st = eng.generate_prompt_lookup(m16, p, 48, eng.SpeculativeConfig(3, 4))
    cp = next((j for j in range(48) if out.tokens[j] != base[j]), 48)
    print(f"[prompt lookup, bf16] 48 tokens in {st['forwards']} forwards, {st['accepted']}/{st['proposed']} drafts accepted, "
          f"tracks the plain loop for {cp}/48 tokens")
    assert len(out.tokens) == 48 and cp >= 1 and st["forwards"] == 48 - st["accepted"] + 0
    assert st["accepted"] > 0 and st["forwards"] < 48 + 1
