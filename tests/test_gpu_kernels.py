"""Parity of every kernel-level C-ABI entry point against the CPU oracle.

Integer outputs (unpacked codes, packer metadata, KV slots, argmax) and bf16 outputs whose
arithmetic has no reduction (dequantized weights, RoPE, KV append, residual add) must be bit-exact.
Outputs behind an f32 reduction are compared on the unrounded f32 accumulation with max-abs <= 2e-3
(matmuls); a bf16 result must be a bf16 number that a value within 2e-3 of the reference rounds to
(helpers.close_bf16_out), or lie within one bf16 ulp of the oracle's (RMSNorm, SwiGLU)."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, kernels
    from oracle import oracle as orc

    ctx = _lib.Context(0)
    yield ctx, kernels, orc
    ctx.close()


def quant_case(orc, seed, n, k, bits, literal_cfg2=True):
    """BASELINE configuration 2 recipe: uniform codes, scales |N(0,0.02)|/7.5, biases -8*scale + N(0,1e-3)."""
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 2**32, size=(n, k * bits // 32), dtype=np.uint32)
    s = np.abs(rng.standard_normal((n, k // 64)).astype(np.float32) * 0.02) / 7.5
    scales = H.f32_to_bf16_np(s)
    biases = H.f32_to_bf16_np(-8.0 * H.bf16_to_f32_np(scales) + rng.standard_normal((n, k // 64)).astype(np.float32) * 1e-3)
    return packed, scales, biases


@pytest.mark.parametrize("bits", [4, 8])
def test_unpack_and_dequantize_bit_exact(env, bits):
    ctx, K, orc = env
    n, k = 96, 512
    packed, scales, biases = quant_case(orc, 1, n, k, bits)
    dp, ds, db = ctx.buf(packed), ctx.buf(scales), ctx.buf(biases)
    codes = ctx.empty((n, k), np.uint8)
    K.unpack_codes(ctx, dp, n, k, bits, codes)
    w = ctx.empty((n, k), np.uint16)
    K.dequantize(ctx, dp, ds, db, n, k, bits, w)
    ctx.sync()
    assert np.array_equal(codes.download(), orc.unpack_codes(packed, k, bits))
    assert np.array_equal(w.download(), orc.dequantize(packed, scales, biases, k, 64, bits))


@pytest.mark.parametrize("bits", [4, 8])
def test_quantize_matches_oracle_and_roundtrips(env, bits):
    ctx, K, orc = env
    rng = np.random.default_rng(2)
    n, k = 64, 256
    w = H.f32_to_bf16_np(rng.standard_normal((n, k)).astype(np.float32) * 0.02)
    w[0, :64] = H.f32_to_bf16_np(np.linspace(-0.5, 0.5, 64, dtype=np.float32))  # the reference's ramp (quant.rs:91-107)
    w[1, :64] = 0  # constant group: scale floor
    dw = ctx.buf(w)
    dp, ds, db = ctx.empty((n, k * bits // 32), np.uint32), ctx.empty((n, k // 64), np.uint16), ctx.empty((n, k // 64), np.uint16)
    K.quantize(ctx, dw, n, k, bits, dp, ds, db)
    ctx.sync()
    ep, es, eb = orc.quantize(w, 64, bits)
    assert np.array_equal(dp.download(), ep)
    assert np.array_equal(ds.download(), es)
    assert np.array_equal(db.download(), eb)
    back = H.bf16_to_f32_np(orc.dequantize(ep, es, eb, k, 64, bits))
    if bits == 8:  # the reference's own bound: 8-bit affine round trip error < 0.01 (quant.rs:91-107)
        assert np.abs(back - H.bf16_to_f32_np(w)).max() < 0.01


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 8, 33, 130])
def test_qmm_vs_oracle(env, bits, m):
    ctx, K, orc = env
    n, k = 320, 512
    packed, scales, biases = quant_case(orc, 3, n, k, bits)
    rng = np.random.default_rng(4)
    x = H.f32_to_bf16_np(rng.standard_normal((m, k)).astype(np.float32))
    dp, ds, db, dx = ctx.buf(packed), ctx.buf(scales), ctx.buf(biases), ctx.buf(x)
    yb, yf = ctx.empty((m, n), np.uint16), ctx.empty((m, n), np.float32)
    K.qmm(ctx, dx, dp, ds, db, m, n, k, bits, yb, yf)
    ctx.sync()
    rf, rb = orc.qmm(x, packed, scales, biases, 64, bits)
    assert np.abs(yf.download() - rf).max() <= 2e-3
    assert H.close_bf16_out(yb.download(), rf)[0]


def test_qmm_reference_small_case(env):
    """The reference's own quantized-matmul check (quant.rs:110-125): [4, 64] Q8 weight, one row of x,
    quantized result within 0.05 of the dense linear."""
    ctx, K, orc = env
    w = np.array([((i * 7 % 13) / 13.0) - 0.5 for i in range(4 * 64)], np.float32).reshape(4, 64)
    x = np.array([(i / 64.0) - 0.5 for i in range(64)], np.float32).reshape(1, 64)
    wb, xb = H.f32_to_bf16_np(w), H.f32_to_bf16_np(x)
    dw = ctx.buf(wb)
    dp, ds, db = ctx.empty((4, 16), np.uint32), ctx.empty((4, 1), np.uint16), ctx.empty((4, 1), np.uint16)
    K.quantize(ctx, dw, 4, 64, 8, dp, ds, db)
    y = ctx.empty((1, 4), np.float32)
    K.qmm(ctx, ctx.buf(xb), dp, ds, db, 1, 4, 64, 8, None, y)
    ctx.sync()
    dense = H.bf16_to_f32_np(xb) @ H.bf16_to_f32_np(wb).T
    assert np.abs(y.download() - dense).max() < 0.05


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (17, 688, 256), (129, 256, 688), (64, 1024, 256), (5, 130, 72)])
def test_linear_vs_oracle(env, m, n, k):
    ctx, K, orc = env
    rng = np.random.default_rng(5)
    x = H.f32_to_bf16_np(rng.standard_normal((m, k)).astype(np.float32))
    w = H.f32_to_bf16_np(rng.standard_normal((n, k)).astype(np.float32) * 0.05)
    yb, yf = ctx.empty((m, n), np.uint16), ctx.empty((m, n), np.float32)
    K.linear(ctx, ctx.buf(x), ctx.buf(w), m, n, k, yb, yf)
    ctx.sync()
    rf, rb = orc.linear(x, w)
    assert np.abs(yf.download() - rf).max() <= 2e-3
    assert H.close_bf16_out(yb.download(), rf)[0]


def test_linear_exact_small_ints(env):
    """linear_matches_manual_matmul (nn.rs:130-139): small integers are exact in bf16/f32."""
    ctx, K, _ = env
    x = np.arange(16, dtype=np.float32).reshape(2, 8) - 4
    w = (np.arange(24, dtype=np.float32).reshape(3, 8) % 5) - 2
    y = ctx.empty((2, 3), np.float32)
    K.linear(ctx, ctx.buf(H.f32_to_bf16_np(x)), ctx.buf(H.f32_to_bf16_np(w)), 2, 3, 8, None, y)
    ctx.sync()
    assert np.array_equal(y.download(), x @ w.T)


@pytest.mark.parametrize("rows,dim", [(3, 256), (2, 4096), (5, 64), (1, 100)])
def test_rms_norm(env, rows, dim):
    ctx, K, orc = env
    rng = np.random.default_rng(6)
    x = H.f32_to_bf16_np(rng.standard_normal((rows, dim)).astype(np.float32) * 3)
    w = H.f32_to_bf16_np(1 + 0.1 * rng.standard_normal(dim).astype(np.float32))
    out = ctx.empty((rows, dim), np.uint16)
    K.rms_norm(ctx, ctx.buf(x), ctx.buf(w), 1e-5, rows, dim, out)
    ctx.sync()
    d = H.bf16_ulp_diff(out.download(), orc.rms_norm(x, w, 1e-5))
    assert d.max() <= 1 and (d > 0).mean() < 0.02


def test_swiglu_add_embed(env):
    ctx, K, orc = env
    rng = np.random.default_rng(7)
    n = 5000
    g = H.f32_to_bf16_np(rng.standard_normal(n).astype(np.float32) * 3)
    u = H.f32_to_bf16_np(rng.standard_normal(n).astype(np.float32))
    out = ctx.empty((n,), np.uint16)
    K.swiglu(ctx, ctx.buf(g), ctx.buf(u), n, out)
    ctx.sync()
    d = H.bf16_ulp_diff(out.download(), orc.swiglu(g, u))
    assert d.max() <= 1 and (d > 0).mean() < 0.01  # expf differs from libm by an ulp now and then
    K.add(ctx, ctx.buf(g), ctx.buf(u), n, out)
    ctx.sync()
    assert np.array_equal(out.download(), orc.add_bf16(g, u))
    table = H.f32_to_bf16_np(rng.standard_normal((50, 72)).astype(np.float32))
    ids = np.array([3, 49, 0, 7, 7], np.int32)
    e = ctx.empty((5, 72), np.uint16)
    K.embed(ctx, ctx.buf(table), ctx.buf(ids), 5, 72, 50, e)
    ctx.sync()
    assert np.array_equal(e.download(), table[ids])


def test_argmax_ties_lowest_index(env):
    ctx, K, orc = env
    rng = np.random.default_rng(8)
    vocab = 128256
    logits = H.f32_to_bf16_np(rng.standard_normal((4, vocab)).astype(np.float32))
    big = H.f32_to_bf16_np(np.array([9.0], np.float32))[0]
    logits[0, [77777, 500, 120000]] = big   # three-way tie -> 500
    logits[1, [vocab - 1]] = big
    logits[2, [0, 1]] = big
    logits[3, :] = H.f32_to_bf16_np(np.array([-np.inf], np.float32))[0]  # all -inf -> 0 (host scan semantics)
    out = ctx.empty((4,), np.int32)
    K.argmax(ctx, ctx.buf(logits), 4, vocab, out)
    ctx.sync()
    got = out.download()
    assert got.tolist() == [500, vocab - 1, 0, 0]
    assert got.tolist() == [orc.argmax_bf16(logits[i]) for i in range(4)]
    # the reference's own cases (sampler.rs:318-334)
    small = H.f32_to_bf16_np(np.array([[0.1, 5.0, 0.2, 9.9, 3.0], [1.0, 5.0, 5.0, 2.0, 0.0]], np.float32))
    o2 = ctx.empty((2,), np.int32)
    K.argmax(ctx, ctx.buf(small), 2, 5, o2)
    ctx.sync()
    assert o2.download().tolist() == [3, 1]


@pytest.mark.parametrize("kind,theta,hd", [(0, 10000.0, 64), (1, 500000.0, 128), (0, 1000000.0, 128)])
def test_rope_tables_match_oracle(env, kind, theta, hd):
    _, K, orc = env
    inv = K.rope_inv_freq(hd, theta, kind, 8.0, 1.0, 4.0, 8192.0)
    assert np.array_equal(inv, orc.rope_inv_freq(hd, theta, kind, 8.0, 1.0, 4.0, 8192.0))
    cos, sin = K.rope_tables(inv, 300)
    oc, os_ = orc.rope_cos_sin(inv, np.arange(300, dtype=np.int32))
    assert np.array_equal(cos, oc[:, : hd // 2]) and np.array_equal(sin, os_[:, : hd // 2])


@pytest.mark.parametrize("hq,hkv,hd,qk_norm", [(4, 2, 64, False), (32, 8, 128, False), (8, 2, 128, True)])
def test_rope_kv_append_bit_exact(env, hq, hkv, hd, qk_norm):
    ctx, K, orc = env
    rng = np.random.default_rng(9)
    T, page, pages = 37, 16, 12
    qkv = H.f32_to_bf16_np(rng.standard_normal((T, (hq + 2 * hkv) * hd)).astype(np.float32))
    positions = rng.integers(0, 5000, size=T).astype(np.int32)
    slots = rng.permutation(pages * page)[:T].astype(np.int32)
    slots[5] = -1  # skipped cache write
    inv = K.rope_inv_freq(hd, 500000.0, 1, 8.0, 1.0, 4.0, 8192.0)
    cos, sin = K.rope_tables(inv, 5000)
    qn = H.f32_to_bf16_np(1 + 0.1 * rng.standard_normal(hd).astype(np.float32)) if qk_norm else None
    kn = H.f32_to_bf16_np(1 + 0.1 * rng.standard_normal(hd).astype(np.float32)) if qk_norm else None
    kp = ctx.buf(np.zeros((pages, hkv, page, hd), np.uint16))
    vp = ctx.buf(np.zeros((pages, hkv, page, hd), np.uint16))
    qo = ctx.empty((T, hq, hd), np.uint16)
    K.rope_kv_append(ctx, ctx.buf(qkv), T, hq, hkv, hd, ctx.buf(positions), ctx.buf(slots), ctx.buf(cos), ctx.buf(sin),
                     ctx.buf(qn) if qk_norm else None, ctx.buf(kn) if qk_norm else None, 1e-6, page, kp, vp, qo)
    ctx.sync()
    q = qkv[:, : hq * hd].reshape(T, hq, hd)
    k = qkv[:, hq * hd:(hq + hkv) * hd].reshape(T, hkv, hd)
    v = qkv[:, (hq + hkv) * hd:].reshape(T, hkv, hd)
    if qk_norm:
        q = orc.rms_norm(q, qn, 1e-6)
        k = orc.rms_norm(k, kn, 1e-6)
    oc, os_ = orc.rope_cos_sin(inv, positions)
    rq, rk = orc.apply_rope(q, oc, os_), orc.apply_rope(k, oc, os_)
    got_q, got_k, got_v = qo.download(), kp.download(), vp.download()
    exp_k, exp_v = np.zeros_like(got_k), np.zeros_like(got_v)
    for t in range(T):
        if slots[t] < 0:
            continue
        exp_k[slots[t] // page, :, slots[t] % page, :] = rk[t]
        exp_v[slots[t] // page, :, slots[t] % page, :] = v[t]
    assert np.array_equal(got_v, exp_v)
    if qk_norm:  # the norm's f32 reduction order differs: allow one ulp on a few elements
        assert H.bf16_ulp_diff(got_q, rq).max() <= 2 and H.bf16_ulp_diff(got_k, exp_k).max() <= 2
    else:
        assert np.array_equal(got_q, rq)
        assert np.array_equal(got_k, exp_k)


def test_rope_analytic_properties(env):
    """The reference's analytic RoPE checks (rope.rs:400-428): inv_freq[0] == 1, formula for index 1,
    llama3 with factor 1 equals standard, lowest frequency divided by the factor."""
    _, K, _ = env
    std8 = K.rope_inv_freq(8, 10000.0)
    assert abs(std8[0] - 1.0) < 1e-6 and abs(std8[1] - 1.0 / np.float32(10000.0) ** np.float32(0.25)) < 1e-6
    std = K.rope_inv_freq(128, 500000.0)
    assert np.abs(std - K.rope_inv_freq(128, 500000.0, 1, 1.0, 1.0, 4.0, 8192.0)).max() < 1e-6
    l3 = K.rope_inv_freq(128, 500000.0, 1, 8.0, 1.0, 4.0, 8192.0)
    assert l3[-1] < std[-1] and abs(l3[-1] - std[-1] / 8.0) < 1e-9


def test_batch_metadata_bit_exact(env):
    ctx, K, _ = env
    from oracle import batch_meta as bm

    rng = np.random.default_rng(10)
    page, max_blocks, slots = 16, 40, 12
    pool = bm.PagePool(300, page)
    seqs = [bm.SeqPages(pool, s) for s in rng.permutation(slots)[:9]]
    bt_ref = np.zeros((slots, max_blocks), np.int32)
    bt_dev = ctx.buf(bt_ref)
    for step in range(4):
        q_len, want = [], []
        for i, s in enumerate(seqs):
            if step == 0:
                n = int(rng.integers(1, 200))
            else:
                n = 1 if i % 3 else int(rng.integers(2, 90))
            q_len.append(n)
            want.append(int(i % 4 != 1))
        upd = []
        for s, n in zip(seqs, q_len):
            upd += s.reserve(n)
        args = ([s.slot for s in seqs], q_len, [s.len for s in seqs], want)
        exp = bm.build_batch_metadata(*args, bt_ref, upd, 64, 64, page)
        W, P = len(exp["dec_work_seq"]) + 3, len(exp["pf_seq"]) + 2
        got = K.build_batch_metadata(ctx, *args, upd, 64, 64, page, max_blocks, W, P, bt_dev)
        for k in exp:
            assert np.array_equal(got[k], exp[k]), (step, k)
        assert np.array_equal(bt_dev.download(), bt_ref)
        for s, n in zip(seqs, q_len):
            s.commit(n)


@pytest.mark.parametrize("hq,hkv,hd", [(8, 2, 64), (32, 8, 128), (4, 4, 128), (9, 3, 64)])
def test_prefill_attention_vs_oracle(env, hq, hkv, hd):
    """Ragged prefill: cold prompts, chunks behind a cached prefix and single-token rows, including the
    reference's chunked shapes (attention.rs:550-573: 16 new on 16, 64 on 64, 40 on 40, 16 behind 64)."""
    ctx, K, orc = env
    q_lens = [16, 64, 40, 16, 1, 130, 7]
    ctx_lens = [16, 64, 40, 80, 33, 130, 300]
    case = H.make_paged_case(11, ctx_lens, hq, hkv, hd, 16, q_lens=q_lens)
    kp, vp, bt, q = ctx.buf(case["kpool"]), ctx.buf(case["vpool"]), ctx.buf(case["block_tables"]), ctx.buf(case["q"])
    out = ctx.empty(case["q"].shape, np.uint16)
    K.paged_attn_prefill(ctx, q, kp, vp, bt, case["max_blocks"], case["cu_seqlens"], case["ctx_lens"], hq, hkv, hd, 16, case["scale"], out)
    ctx.sync()
    ref = orc.paged_attention(case["q"], case["kpool"], case["vpool"], case["block_tables"], case["cu_seqlens"], case["ctx_lens"],
                              case["scale"])
    ok, err = H.close_bf16_out(out.download(), ref)
    assert ok, f"max-abs {err}"


def test_attention_reference_shapes_f64_host(env):
    """The reference's safe-path gate (attention.rs:457-480): LCG inputs, contiguous K/V laid into pages,
    relative error against the f64 host loop below 2e-3 (bf16 inputs here)."""
    ctx, K, orc = env
    for nh, nkv, ql, kl, hd in [(8, 2, 1, 64, 64), (32, 8, 1, 256, 128), (8, 2, 8, 8, 64), (8, 2, 8, 256, 64), (8, 2, 8, 8, 128),
                                (4, 4, 4, 64, 128)]:
        scale = 1.0 / np.sqrt(np.float32(hd))
        q = H.bf16_to_f32_np(H.f32_to_bf16_np(H.lcg_randf(nh * ql * hd, 1).reshape(nh, ql, hd)))
        k = H.bf16_to_f32_np(H.f32_to_bf16_np(H.lcg_randf(nkv * kl * hd, 2).reshape(nkv, kl, hd)))
        v = H.bf16_to_f32_np(H.f32_to_bf16_np(H.lcg_randf(nkv * kl * hd, 3).reshape(nkv, kl, hd)))
        host = orc.host_attn_gqa(q, k, v, float(scale), True)
        pages = (kl + 15) // 16
        kp = np.zeros((pages, nkv, 16, hd), np.float32)
        vp = np.zeros_like(kp)
        for j in range(kl):
            kp[j // 16, :, j % 16] = k[:, j]
            vp[j // 16, :, j % 16] = v[:, j]
        bt = np.arange(pages, dtype=np.int32).reshape(1, pages)
        qt = H.f32_to_bf16_np(np.ascontiguousarray(q.transpose(1, 0, 2)))  # [ql, nh, hd]
        out = ctx.empty(qt.shape, np.uint16)
        K.paged_attn_prefill(ctx, ctx.buf(qt), ctx.buf(H.f32_to_bf16_np(kp)), ctx.buf(H.f32_to_bf16_np(vp)), ctx.buf(bt), pages,
                             np.array([0, ql], np.int32), np.array([kl], np.int32), nh, nkv, hd, 16, float(scale), out)
        ctx.sync()
        # the reference's gate: max |got - host| / max |host| < 2e-3, applied to the value BEFORE the bf16 output
        # rounding (close_bf16_out accepts exactly the bf16 numbers such a value can round to)
        tol = 2e-3 * float(np.abs(host).max())
        ok, err = H.close_bf16_out(out.download().transpose(1, 0, 2), host, tol)
        assert ok, (nh, nkv, ql, kl, hd, err / float(np.abs(host).max()))


@pytest.mark.parametrize("hq,hkv,page", [(8, 2, 16), (4, 1, 32)])
def test_prefill_attention_long_contexts_hd128(env, hq, hkv, page):
    """head_dim 128 takes the tcgen05 kernel: many 128-key tiles per work item (ring phases wrap), chunks that end
    inside a tile, several 128-query work items per sequence, contexts that are not multiples of the page."""
    ctx, K, orc = env
    q_lens = [300, 128, 129, 5, 512]
    ctx_lens = [1500, 128, 700, 1031, 2048]
    case = H.make_paged_case(21, ctx_lens, hq, hkv, 128, page, q_lens=q_lens)
    kp, vp, bt, q = ctx.buf(case["kpool"]), ctx.buf(case["vpool"]), ctx.buf(case["block_tables"]), ctx.buf(case["q"])
    out = ctx.empty(case["q"].shape, np.uint16)
    K.paged_attn_prefill(ctx, q, kp, vp, bt, case["max_blocks"], case["cu_seqlens"], case["ctx_lens"], hq, hkv, 128, page, case["scale"], out)
    ctx.sync()
    ref = orc.paged_attention(case["q"], case["kpool"], case["vpool"], case["block_tables"], case["cu_seqlens"], case["ctx_lens"],
                              case["scale"])
    ok, err = H.close_bf16_out(out.download(), ref)
    assert ok, f"max-abs {err}"


def test_prefill_attention_key_split_hd128(env):
    """Few (work item, head) pairs and a long context: the launch splits every work item's key tiles over several CTAs
    and a second kernel adds the partial results up.  The 704-token sequence starts 64 tokens into a key tile, so some
    splits begin on a tile that half of the query rows do not see at all (their partial is empty)."""
    ctx, K, orc = env
    hq, hkv, hd, page = 2, 1, 128, 16
    q_lens = [300, 640]
    ctx_lens = [8192 + 37, 64 + 640]
    case = H.make_paged_case(23, ctx_lens, hq, hkv, hd, page, q_lens=q_lens)
    kp, vp, bt, q = ctx.buf(case["kpool"]), ctx.buf(case["vpool"]), ctx.buf(case["block_tables"]), ctx.buf(case["q"])
    out = ctx.empty(case["q"].shape, np.uint16)
    n0 = ctx.launch_count()
    K.paged_attn_prefill(ctx, q, kp, vp, bt, case["max_blocks"], case["cu_seqlens"], case["ctx_lens"], hq, hkv, hd, page, case["scale"], out)
    ctx.sync()
    assert ctx.launch_count() - n0 == 2, "expected the split kernel and its merge"
    ref = orc.paged_attention(case["q"], case["kpool"], case["vpool"], case["block_tables"], case["cu_seqlens"], case["ctx_lens"],
                              case["scale"])
    ok, err = H.close_bf16_out(out.download(), ref)
    assert ok, f"max-abs {err}"


def test_prefill_attention_rising_scores_hd128(env):
    """Scores that keep growing along the context force the running maximum up by more than the lazy-rescale
    threshold several times (the accumulator in TMEM is rescaled in place), and a peaked softmax exercises the
    two-part P."""
    ctx, K, orc = env
    hq, hkv, hd, page = 4, 2, 128, 16
    case = H.make_paged_case(22, [900], hq, hkv, hd, page, q_lens=[200])
    # keys in logical order get a growing component along one direction that every query shares
    kpool = H.bf16_to_f32_np(case["kpool"]).copy()
    qf = H.bf16_to_f32_np(case["q"]).copy()
    qf[:, :, 0] = 6.0
    for pos in range(900):
        pg, slot = case["block_tables"][0, pos // page], pos % page
        kpool[pg, :, slot, 0] = 0.04 * pos  # score contribution 6 * 0.04 * pos / sqrt(128): ~19 units over the context
    case["kpool"], case["q"] = H.f32_to_bf16_np(kpool), H.f32_to_bf16_np(qf)
    kp, vp, bt, q = ctx.buf(case["kpool"]), ctx.buf(case["vpool"]), ctx.buf(case["block_tables"]), ctx.buf(case["q"])
    out = ctx.empty(case["q"].shape, np.uint16)
    K.paged_attn_prefill(ctx, q, kp, vp, bt, case["max_blocks"], case["cu_seqlens"], case["ctx_lens"], hq, hkv, hd, page, case["scale"], out)
    ctx.sync()
    ref = orc.paged_attention(case["q"], case["kpool"], case["vpool"], case["block_tables"], case["cu_seqlens"], case["ctx_lens"],
                              case["scale"])
    ok, err = H.close_bf16_out(out.download(), ref)
    assert ok, f"max-abs {err}"
