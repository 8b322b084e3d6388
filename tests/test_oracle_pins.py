"""Pins of the CPU oracle against everything the reference's own tests fix for this path (no GPU).

Each test names the reference test it restates.  The reference ships no stored numeric goldens for
logits or tokens (its token-level tests need real checkpoints that are not available), so the token
streams of configuration 0 are pinned by a committed fixture generated from this oracle
(tests/golden/gen_config0.py)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests import helpers as H

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "config0.json")


def rows(h, s, d, base):
    """Token-major [s, h*d] bf16 rows of sequential values (small integers are exact in bf16)."""
    n = h * s * d
    a = (base + np.arange(n, dtype=np.float32)).reshape(h, s, d).transpose(1, 0, 2).reshape(s, h * d)
    return orc.f32_to_bf16(a)


def vals(x):
    return orc.bf16_to_f32(x)


# ---- sampler.rs ------------------------------------------------------------------------------------
def test_splitmix64_known_answers():  # sampler.rs:300-305
    r = orc.SplitMix64(0)
    assert r.next_u64() == 0xE220A8397B1DCDAF
    assert r.next_u64() == 0x6E789E6AA1B965F4
    assert [int(x) for x in H.splitmix_stream(0, 2)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4]


def test_next_f32_unit_interval():  # sampler.rs:307-314
    r = orc.SplitMix64(42)
    xs = [r.next_f32() for _ in range(1000)]
    assert all(0.0 <= x < 1.0 for x in xs)
    assert np.allclose(xs, H.splitmix_f32(42, 1000))


def test_argmax_first_maximum_wins():  # sampler.rs:318-334
    assert orc.argmax_bf16(orc.f32_to_bf16(np.array([0.1, 5.0, 0.2, -1.0], np.float32))) == 1
    assert orc.argmax_bf16(orc.f32_to_bf16(np.array([0.1, 5.0, 0.2, 9.9, 3.0], np.float32))) == 3
    assert orc.argmax_bf16(orc.f32_to_bf16(np.array([1.0, 5.0, 5.0, 2.0], np.float32))) == 1


# ---- rope.rs ---------------------------------------------------------------------------------------
def test_standard_inv_freq_formula():  # rope.rs:400-408
    inv = orc.rope_inv_freq(8, 10000.0)
    assert inv.size == 4 and abs(inv[0] - 1.0) < 1e-6
    assert abs(inv[1] - 1.0 / np.float32(10000.0) ** np.float32(2.0 / 8.0)) < 1e-6


def test_llama3_unit_factor_equals_standard_and_scales_low_frequencies():  # rope.rs:411-428
    std = orc.rope_inv_freq(128, 500000.0)
    assert np.abs(std - orc.rope_inv_freq(128, 500000.0, 1, 1.0, 1.0, 4.0, 8192.0)).max() < 1e-6
    l3 = orc.rope_inv_freq(128, 500000.0, 1, 8.0, 1.0, 4.0, 8192.0)
    assert l3[-1] < std[-1] and abs(l3[-1] - std[-1] / 8.0) < 1e-9
    assert np.array_equal(l3[:20], std[:20])  # short wavelengths pass through unchanged


def test_rope_position_zero_identity_and_norm():  # rope.rs:465-476, :505-525
    inv = orc.rope_inv_freq(8, 10000.0)
    x = orc.f32_to_bf16(np.arange(1, 9, dtype=np.float32).reshape(1, 1, 8))
    cos, sin = orc.rope_cos_sin(inv, [0])
    assert np.array_equal(orc.apply_rope(x, cos, sin), x)
    inv4 = orc.rope_inv_freq(4, 10000.0)
    xs = np.array([1.0, 0.5, -0.5, 2.0, 0.3, 1.0, -1.0, 0.7, 2.0, -0.2, 0.1, 0.9], np.float32).reshape(3, 1, 4)
    cos, sin = orc.rope_cos_sin(inv4, [0, 1, 2])
    y = vals(orc.apply_rope(orc.f32_to_bf16(xs), cos, sin))
    for p in range(3):  # rotation preserves the norm (bf16 rounding allowed for)
        assert abs(np.linalg.norm(vals(orc.f32_to_bf16(xs))[p]) - np.linalg.norm(y[p])) < 2e-2


def test_rope_rotates_pairs_like_the_closed_form():
    inv = orc.rope_inv_freq(64, 10000.0)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 2, 64)).astype(np.float32)
    pos = np.array([0, 1, 7, 100, 4095], np.int32)
    cos, sin = orc.rope_cos_sin(inv, pos)
    y = vals(orc.apply_rope(orc.f32_to_bf16(x), cos, sin))
    xb = vals(orc.f32_to_bf16(x))
    ang = pos[:, None].astype(np.float32) * inv[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    exp = np.concatenate([xb[..., :32] * c - xb[..., 32:] * s, xb[..., 32:] * c + xb[..., :32] * s], -1)
    assert np.abs(y - exp).max() < 0.05  # three bf16 roundings on values up to ~4


# ---- paged_kv_cache.rs -----------------------------------------------------------------------------
def test_single_step_under_block_stays_in_tail():  # :593-601
    c = orc.Cache(1, block_size=4)
    k = rows(2, 3, 2, 0.0)
    ka, _ = c.update(0, k, k)
    assert ka.shape == (3, 4) and c.offset() == 3
    assert c.paged_stats()["blocks"] == 0 and c.pool.stats()["live_blocks"] == 0


def test_crossing_block_boundary_freezes_and_gather_preserves_order():  # :604-619
    c = orc.Cache(1, block_size=2)
    g0, _ = c.update(0, rows(1, 2, 1, 0.0), rows(1, 2, 1, 0.0))
    assert vals(g0).ravel().tolist() == [0.0, 1.0]
    assert c.paged_stats()["blocks"] == 1 and c.paged_stats()["tail_len"] == 0
    g1, _ = c.update(0, rows(1, 3, 1, 2.0), rows(1, 3, 1, 2.0))
    assert c.offset() == 5 and c.paged_stats()["blocks"] == 2 and c.paged_stats()["tail_len"] == 1
    assert vals(g1).ravel().tolist() == [0.0, 1.0, 2.0, 3.0, 4.0]


def test_matches_contiguous_cache_step_by_step():  # :622-639
    paged, contig = orc.Cache(2, block_size=4), orc.Cache(2)
    off = 0.0
    for step in (5, 1, 1, 4, 1):
        for layer in range(2):
            k, v = rows(2, step, 3, off + layer * 100.0), rows(2, step, 3, off + 50.0 + layer * 100.0)
            pk, pv = paged.update(layer, k, v)
            ck, cv = contig.update(layer, k, v)
            assert np.array_equal(pk, ck) and np.array_equal(pv, cv), (step, layer)
        off += step * 6
    assert paged.offset() == contig.offset() == 12


def test_seeded_prefix_then_freeze_matches_contiguous():  # :642-670
    pool = orc.Pool(2)
    a = orc.Cache(2, pool)
    for layer in range(2):
        a.update(layer, rows(1, 4, 1, layer * 100.0), rows(1, 4, 1, layer * 100.0))
    shared = a.shareable_prefix_blocks(4)
    assert len(shared) == 2
    b, contig = orc.Cache(2, pool, seeded=shared), orc.Cache(2)
    for layer in range(2):
        prefix, suffix = rows(1, 4, 1, layer * 100.0), rows(1, 3, 1, layer * 100.0 + 4.0)
        contig.update(layer, prefix, prefix)
        ck, cv = contig.update(layer, suffix, suffix)
        bk, bv = b.update(layer, suffix, suffix)
        assert np.array_equal(bk, ck) and np.array_equal(bv, cv)
    assert b.offset() == 7 and b.paged_stats()["blocks"] == 3


def test_reserved_tokens_tracks_blocks_not_max_context():  # :673-682
    c = orc.Cache(1, block_size=16)
    c.update(0, rows(1, 20, 1, 0.0), rows(1, 20, 1, 0.0))
    st = c.paged_stats()
    assert st["blocks"] == 1 and st["tail_len"] == 4 and st["reserved_tokens"] == 32


def test_shared_prefix_blocks_are_refcounted_not_copied():  # :685-713
    pool = orc.Pool(2)
    a = orc.Cache(1, pool)
    a.update(0, rows(1, 4, 1, 0.0), rows(1, 4, 1, 0.0))
    assert pool.stats()["live_blocks"] == 2 and pool.stats()["shared_blocks"] == 0
    shared = a.shareable_prefix_blocks(4)
    b = orc.Cache(1, pool, seeded=shared)
    assert b.offset() == 4 and pool.stats()["live_blocks"] == 2 and pool.stats()["shared_blocks"] == 2
    b.update(0, rows(1, 1, 1, 99.0), rows(1, 1, 1, 99.0))
    assert pool.stats()["shared_blocks"] == 2
    assert vals(b.gather(0)[0]).ravel().tolist() == [0.0, 1.0, 2.0, 3.0, 99.0]
    b.free()
    assert pool.stats()["shared_blocks"] == 0 and pool.stats()["live_blocks"] == 2


def test_unshared_blocks_hold_no_bytes_until_shared():  # :716-740
    pool = orc.Pool(2)
    a = orc.Cache(1, pool)
    a.update(0, rows(1, 6, 1, 0.0), rows(1, 6, 1, 0.0))
    ids = a.block_ids()
    assert len(ids) == 3 and not any(pool.is_materialized(i) for i in ids)
    shared = a.shareable_prefix_blocks(4)
    assert len(shared) == 2 and all(pool.is_materialized(i) for i in shared) and not pool.is_materialized(ids[2])


def test_truncate_within_tail_and_across_blocks():  # :743-768
    c = orc.Cache(1, block_size=4)
    c.update(0, rows(1, 10, 1, 0.0), rows(1, 10, 1, 0.0))
    assert c.offset() == 10
    c.truncate(9)
    assert c.offset() == 9 and vals(c.gather(0)[0]).ravel().tolist() == [float(i) for i in range(9)]
    c.truncate(5)
    assert c.offset() == 5 and vals(c.gather(0)[0]).ravel().tolist() == [float(i) for i in range(5)]
    assert c.pool.stats()["live_blocks"] == 1
    c.truncate(4)
    assert c.offset() == 4 and vals(c.gather(0)[0]).ravel().tolist() == [0.0, 1.0, 2.0, 3.0]
    c.truncate(100)
    assert c.offset() == 4
    with pytest.raises(ValueError):
        c.truncate(-1)


def test_reset_frees_blocks_and_batched_update_is_rejected():  # :771-787
    pool = orc.Pool(2)
    c = orc.Cache(1, pool)
    c.update(0, rows(1, 4, 1, 0.0), rows(1, 4, 1, 0.0))
    assert pool.stats()["live_blocks"] == 2
    c.reset()
    assert pool.stats()["live_blocks"] == 0 and c.offset() == 0
    with pytest.raises(ValueError):
        c.update(0, rows(2, 1, 2, 0.0), rows(2, 1, 2, 0.0), batch=2)
    with pytest.raises(ValueError):
        c.retain_sequences([1])
    c.retain_sequences([0])
    c.retain_sequences([])


def test_contiguous_cache_concat_truncate_reset():  # kv_cache.rs:193-313
    c = orc.Cache(2)
    assert c.offset() == 0
    c.update(0, rows(2, 3, 2, 0.0), rows(2, 3, 2, 0.0))
    k, _ = c.update(0, rows(2, 2, 2, 100.0), rows(2, 2, 2, 100.0))
    assert k.shape == (5, 4) and c.offset() == 5
    c.truncate(2)
    assert c.offset() == 2
    c.reset()
    assert c.offset() == 0


# ---- attention.rs -----------------------------------------------------------------------------------
def test_native_gqa_equals_repeat_kv():  # attention.rs:329-367
    for nh, nkv, s, hd in [(8, 2, 1, 64), (32, 8, 1, 128), (8, 2, 16, 64), (6, 3, 5, 64), (4, 4, 7, 64)]:
        q = H.lcg_randf(nh * s * hd, 1).reshape(nh, s, hd)
        k = H.lcg_randf(nkv * s * hd, 2).reshape(nkv, s, hd)
        v = H.lcg_randf(nkv * s * hd, 3).reshape(nkv, s, hd)
        g = nh // nkv
        scale = float(1.0 / np.sqrt(np.float32(hd)))
        for causal in (False, True):
            a = orc.host_attn_gqa(q, k, v, scale, causal)
            b = orc.host_attn_gqa(q, np.repeat(k, g, 0), np.repeat(v, g, 0), scale, causal)
            assert np.abs(a - b).max() < 1e-4


def test_host_attention_against_numpy_softmax():  # attention.rs:373-405 restated twice
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((4, 3, 16)), rng.standard_normal((2, 7, 16)), rng.standard_normal((2, 7, 16))
    out = orc.host_attn_gqa(q, k, v, 0.25, True)
    for h in range(4):
        for i in range(3):
            j = 7 - 3 + i + 1
            s = (k[h // 2, :j] @ q[h, i]) * 0.25
            p = np.exp(s - s.max())
            assert np.abs(out[h, i] - (p / p.sum()) @ v[h // 2, :j]).max() < 1e-5


def test_paged_attention_equals_contiguous_host_attention():
    case = H.make_paged_case(3, [40, 17], 4, 2, 64, 16, q_lens=[5, 1])
    out = orc.paged_attention(case["q"], case["kpool"], case["vpool"], case["block_tables"], case["cu_seqlens"], case["ctx_lens"],
                              case["scale"])
    kp, vp = vals(case["kpool"]), vals(case["vpool"])
    t0 = 0
    for s, (ctx, qn) in enumerate(zip([40, 17], [5, 1])):
        k = np.stack([kp[case["block_tables"][s, j // 16], :, j % 16] for j in range(ctx)], 1)  # [hkv, ctx, hd]
        v = np.stack([vp[case["block_tables"][s, j // 16], :, j % 16] for j in range(ctx)], 1)
        q = vals(case["q"][t0:t0 + qn]).transpose(1, 0, 2)
        ref = orc.host_attn_gqa(q, k, v, case["scale"], True).transpose(1, 0, 2)
        assert np.abs(out[t0:t0 + qn] - ref).max() < 1e-5
        t0 += qn
    fast = orc.paged_attention(case["q"][5:], case["kpool"], case["vpool"], case["block_tables"][1:], None, case["ctx_lens"][1:],
                               case["scale"], fast_decode=True)
    assert np.abs(fast - out[5:]).max() < 1e-4


# ---- quant.rs ---------------------------------------------------------------------------------------
def test_quantize_dequantize_roundtrip_q8():  # quant.rs:91-107
    w = ((np.arange(128, dtype=np.float32) / 128.0) - 0.5).reshape(2, 64)
    wb = orc.f32_to_bf16(w)
    p, s, b = orc.quantize(wb, 64, 8)
    assert p.shape == (2, 16) and s.shape == (2, 1)
    assert np.abs(vals(orc.dequantize(p, s, b, 64, 64, 8)) - vals(wb)).max() < 0.01


def test_quantized_matmul_approximates_linear_q8():  # quant.rs:110-125
    w = np.array([((i * 7 % 13) / 13.0) - 0.5 for i in range(256)], np.float32).reshape(4, 64)
    x = ((np.arange(64, dtype=np.float32) / 64.0) - 0.5).reshape(1, 64)
    wb, xb = orc.f32_to_bf16(w), orc.f32_to_bf16(x)
    p, s, b = orc.quantize(wb, 64, 8)
    dense, _ = orc.linear(xb, wb)
    q, _ = orc.qmm(xb, p, s, b, 64, 8)
    assert np.abs(dense - q).max() < 0.05


@pytest.mark.parametrize("bits", [4, 8])
def test_pack_layout_lowest_bits_first(bits):
    """Element j of a row lives in word j*bits/32 at bit offset (j*bits) mod 32."""
    per = 32 // bits
    codes = (np.arange(128) * 7 % (1 << bits)).astype(np.uint32).reshape(1, 128)
    packed = np.zeros((1, 128 // per), np.uint32)
    for j in range(128):
        packed[0, j // per] |= codes[0, j] << np.uint32((j % per) * bits)
    assert np.array_equal(orc.unpack_codes(packed, 128, bits), codes.astype(np.uint8))
    s = orc.f32_to_bf16(np.array([[0.5, 0.25]], np.float32))
    b = orc.f32_to_bf16(np.array([[-1.0, 2.0]], np.float32))
    w = vals(orc.dequantize(packed, s, b, 128, 64, bits))
    exp = np.concatenate([codes[0, :64] * 0.5 - 1.0, codes[0, 64:] * 0.25 + 2.0]).astype(np.float32)
    assert np.array_equal(w[0], vals(orc.f32_to_bf16(exp)))


def test_quantize_codes_reconstruct_within_half_a_step():
    rng = np.random.default_rng(1)
    wb = orc.f32_to_bf16(rng.standard_normal((8, 256)).astype(np.float32) * 0.02)
    for bits in (4, 8):
        p, s, b = orc.quantize(wb, 64, bits)
        back = vals(orc.dequantize(p, s, b, 256, 64, bits))
        step = np.abs(vals(s)).repeat(64, 1)
        # Half a step in the interior.  The published encoder re-fits the scale so that the larger-
        # magnitude edge lands exactly on a code, which can push the opposite edge up to one step past
        # the last code (clamped); the bf16 rounding of the stored scale adds up to code * 2^-9 steps.
        err = np.abs(back - vals(wb)) / step
        assert err.max() <= 1.6 and np.median(err) <= 0.3


# ---- synthetic generator -------------------------------------------------------------------------------
def test_synthetic_generator_is_a_pure_function_of_seed_and_index():
    a, b = orc.synth_codes(5, 1000), orc.synth_codes(5, 2000)
    assert np.array_equal(a, b[:1000]) and not np.array_equal(a, orc.synth_codes(6, 1000))
    n = vals(orc.synth_dense(9, 200000, 1.0))
    assert abs(n.mean()) < 0.01 and abs(n.std() - 1.0) < 0.01
    s, bz = orc.synth_scales_biases(1, 2, 10000, 0.02 / 7.5, 8.0)
    assert (vals(s) >= 0).all() and abs(np.mean(vals(bz) + 8 * vals(s))) < 1e-4


# ---- continuous.rs / stream.rs on configuration 0 ------------------------------------------------------
@pytest.fixture(scope="module")
def tiny():
    return H.build_oracle_model(orc), H.config0_prompts()


def test_config0_block_id_table(tiny):
    """Fill-order block ids derived from paged_kv_cache.rs:315-340 + continuous.rs:157-181."""
    m, prompts = tiny
    out = m.generate_continuous(prompts, [32] * 4)
    assert out["block_ids"] == [[0, 15, 19], [1, 2, 16, 20], [3, 4, 5, 6, 18], [7, 8, 9, 10, 11, 12, 13, 14, 17, 21]]
    assert out["pool"]["peak_live_blocks"] == 22 and out["pool"]["live_blocks"] == 0
    assert all(len(t) == 32 for t in out["tokens"]) and out["reasons"] == [1] * 4


def test_config0_exact_equals_throughput_equals_batch1(tiny):  # tests/continuous.rs:92-118
    m, prompts = tiny
    a = m.generate_continuous(prompts, [32] * 4)
    b = m.generate_continuous(prompts, [32] * 4, throughput=True)
    assert a["tokens"] == b["tokens"] and a["events"] == b["events"]
    for p, t in zip(prompts, a["tokens"]):
        assert m.generate(p, 32)["tokens"] == t
        assert m.generate(p, 32, paged_block=16)["tokens"] == t  # paged == contiguous (tests/paged.rs:68-95)


def test_config0_golden_fixture(tiny):
    m, prompts = tiny
    with open(GOLDEN) as f:
        g = json.load(f)
    w = H.tiny_weights()
    if g["weights_crc"] != H.weights_crc(w):
        pytest.skip("this platform's libm draws different Box-Muller weights than the fixture's")
    assert [p.tolist() for p in prompts] == g["prompts"]
    out = m.generate_continuous(prompts, [32] * 4)
    assert out["tokens"] == g["tokens"] and out["block_ids"] == g["block_ids"]
    m32 = H.build_oracle_model(orc, cfg=dict(H.CONFIG0, f32_mode=1), weights=w)
    assert m32.generate_continuous(prompts, [32] * 4)["tokens"] == g["tokens_f32"]
    m32.free()


def test_admit_on_retire_and_event_order(tiny):  # tests/continuous.rs:123-149
    m, prompts = tiny
    rng = np.random.default_rng(3)
    ps = [rng.integers(0, 1024, size=n).astype(np.int32) for n in (9, 21, 16, 40, 5)]
    budgets = [4, 8, 6, 10, 12]
    out = m.generate_continuous(ps, budgets, max_batch=2)
    assert [len(t) for t in out["tokens"]] == budgets
    for p, b, t in zip(ps, budgets, out["tokens"]):
        assert m.generate(p, b)["tokens"] == t
    for r in range(5):  # Token{step 0..} then exactly one Done, per request
        ev = [e for e in out["events"] if e[0] == r]
        assert [e[1] for e in ev] == [0] * budgets[r] + [1] and [e[3] for e in ev[:-1]] == list(range(budgets[r]))
    first_seen = []
    for e in out["events"]:
        if e[0] not in first_seen:
            first_seen.append(e[0])
    assert first_seen == [0, 1, 2, 3, 4]


def test_cancel_zero_budget_stop_token_and_errors(tiny):  # tests/continuous.rs:243-375, tests/streaming.rs:94-217
    m, prompts = tiny
    assert m.generate_continuous([], []) == {"error": -7}
    assert m.generate_continuous([prompts[0], []], [4, 4]) == {"error": -7}
    assert m.generate_continuous(prompts, [4] * 4, max_batch=0) == {"error": -7}
    assert m.generate_continuous(prompts, [4] * 4, cancel_after_steps=0) == {"error": -6}
    out = m.generate_continuous([prompts[i % 4] for i in range(6)], [20, 20, 20, 20, 20, 0], max_batch=2, cancel_after_steps=3)
    dones = [e for e in out["events"] if e[1] == 1]
    assert sorted(d[0] for d in dones) == list(range(6))
    assert out["reasons"][:5] == [2] * 5 and out["reasons"][5] == 1 and out["tokens"][5] == []
    z = m.generate_continuous(prompts[:2], [0, 3])
    assert z["tokens"][0] == [] and z["reasons"][0] == 1 and z["events"][0] == [0, 1, 1, 0]
    base = m.generate(prompts[0], 12)
    stop = base["tokens"][5]
    first = base["tokens"].index(stop)
    st = m.generate(prompts[0], 12, stop=[stop])
    assert st["tokens"] == base["tokens"][:first] and st["reason"] == 0 and st["events"][-1] == [0, 1, 0, first]
    c = m.generate(prompts[1], 20, cancel_after_tokens=3)
    assert c["reason"] == 2 and len(c["tokens"]) == 3
