"""b2_paged_attn_decode_static: the decode-attention entry point that allocates nothing.

Its split-K scratch is a fixed array inside the library's device image, so the checks are: same bits
as b2_paged_attn_decode on the same inputs, also when two calls follow each other on the stream with
no host synchronisation in between (the second reuses the array the first just used), also when
other kernels of the library ran before in this process, and a clean refusal of batches that the
array cannot hold.  The file name sorts last so the default collection order runs it after every
other GPU test; it makes no assumption about that and passes alone too."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _cudart():
    for name in ("libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so"):
        try:
            return C.CDLL(name)
        except OSError:
            continue
    pytest.fail("libcudart not found")


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, kernels
    from oracle import oracle as orc

    ctx = _lib.Context(0)
    rt = _cudart()
    yield ctx, kernels, orc, _lib, rt
    ctx.close()


def _upload(ctx, case):
    return dict(kp=ctx.buf(case["kpool"]), vp=ctx.buf(case["vpool"]), bt=ctx.buf(case["block_tables"]),
                cl=ctx.buf(case["ctx_lens"]), q=ctx.buf(case["q"]))


def _free(bufs):
    for b in bufs.values():
        b.free()


def _existing(ctx, kernels, case, d, chunk):
    o = ctx.empty(case["q"].shape, np.uint16)
    kernels.paged_attn_decode(ctx, d["q"], d["kp"], d["vp"], d["bt"], d["cl"], case["ctx_lens"].size, case["hq"], case["hkv"],
                              case["hd"], case["page"], case["scale"], o, case["max_blocks"], chunk)
    ctx.sync()
    out = o.download()
    o.free()
    return out


def _static(_lib, stream, case, d, chunk, out_buf):
    p = _lib.ptr
    return _lib.load().b2_paged_attn_decode_static(
        C.c_void_p(stream), p(d["q"]), p(d["kp"]), p(d["vp"]), p(d["bt"]), C.c_int32(case["max_blocks"]), p(d["cl"]),
        C.c_int32(case["ctx_lens"].size), C.c_int32(case["hq"]), C.c_int32(case["hkv"]), C.c_int32(case["hd"]),
        C.c_int32(case["page"]), C.c_float(case["scale"]), C.c_int32(chunk), p(out_buf))


@pytest.mark.parametrize("use_stream", [False, True])
def test_static_matches_existing_entry_point_twice_in_a_row(env, use_stream):
    ctx, kernels, orc, _lib, rt = env
    case_a = H.make_paged_case(41, [1, 17, 300, 700, 1500, 2049], 32, 8, 128, 16)
    case_b = H.make_paged_case(42, [5, 64, 129, 1000], 8, 2, 64, 16)
    da, db = _upload(ctx, case_a), _upload(ctx, case_b)
    want_a = _existing(ctx, kernels, case_a, da, 256)
    want_b = _existing(ctx, kernels, case_b, db, 64)

    stream = C.c_void_p(0)
    if use_stream:
        assert rt.cudaStreamCreateWithFlags(C.byref(stream), C.c_uint(1)) == 0  # cudaStreamNonBlocking
    s = stream.value or 0
    oa, ob, oa2 = (ctx.empty(case_a["q"].shape, np.uint16), ctx.empty(case_b["q"].shape, np.uint16),
                   ctx.empty(case_a["q"].shape, np.uint16))
    # three calls back to back on one stream, no host synchronisation between them
    _lib.check(_static(_lib, s, case_a, da, 256, oa))
    _lib.check(_static(_lib, s, case_b, db, 64, ob))
    _lib.check(_static(_lib, s, case_a, da, 256, oa2))
    assert rt.cudaStreamSynchronize(stream) == 0
    assert rt.cudaDeviceSynchronize() == 0
    got_a, got_b, got_a2 = oa.download(), ob.download(), oa2.download()
    if use_stream:
        assert rt.cudaStreamDestroy(stream) == 0
    assert np.array_equal(got_a, want_a)
    assert np.array_equal(got_b, want_b)
    assert np.array_equal(got_a2, want_a)
    # and the result is the oracle's, to the decode kernel's own tolerance
    ref = orc.paged_attention(case_a["q"], case_a["kpool"], case_a["vpool"], case_a["block_tables"], case_a["cu_seqlens"],
                              case_a["ctx_lens"], case_a["scale"])
    ok, err = H.close_bf16_out(got_a, ref, 2e-3)
    assert ok, f"max-abs {err}"
    for b in (oa, ob, oa2):
        b.free()
    _free(da)
    _free(db)


def test_static_default_chunk_and_empty_batch(env):
    ctx, kernels, orc, _lib, rt = env
    case = H.make_paged_case(43, [33, 511, 512, 513, 1200], 16, 4, 128, 32)
    d = _upload(ctx, case)
    want = _existing(ctx, kernels, case, d, 512)
    o = ctx.empty(case["q"].shape, np.uint16)
    _lib.check(_static(_lib, 0, case, d, 0, o))  # 0 -> 512
    assert rt.cudaDeviceSynchronize() == 0
    assert np.array_equal(o.download(), want)
    empty = dict(case)
    empty["ctx_lens"] = np.zeros(0, np.int32)
    _lib.check(_static(_lib, 0, empty, d, 0, o))
    o.free()
    _free(d)


def test_static_rejects_what_the_array_cannot_hold(env):
    ctx, kernels, orc, _lib, rt = env
    case = H.make_paged_case(44, [100, 200], 32, 8, 128, 16)
    d = _upload(ctx, case)
    o = ctx.empty(case["q"].shape, np.uint16)
    big = dict(case)
    big["max_blocks"] = 1024                       # 16 K tokens per table row
    big["ctx_lens"] = np.zeros(64, np.int32)       # 64 rows x 32 chunks x 16640 B > 16 MiB; only the size is read
    rc = _static(_lib, 0, big, d, 512, o)
    assert rc == -7
    msg = _lib.load().b2_last_error().decode()
    assert str(16 << 20) in msg and "scratch" in msg
    # within the limit again: 31 rows are accepted by the size check (launch itself needs real tables, so only
    # the arithmetic is probed here through a rejected neighbour)
    big["ctx_lens"] = np.zeros(32, np.int32)
    assert _static(_lib, 0, big, d, 512, o) == -7
    # bad arguments are refused before anything is launched
    bad = dict(case)
    bad["hd"] = 96
    assert _static(_lib, 0, bad, d, 256, o) == -5
    assert _static(_lib, 0, case, d, 4096, o) == -7
    assert rt.cudaDeviceSynchronize() == 0
    # the library still works afterwards
    want = _existing(ctx, kernels, case, d, 256)
    _lib.check(_static(_lib, 0, case, d, 256, o))
    assert rt.cudaDeviceSynchronize() == 0
    assert np.array_equal(o.download(), want)
    o.free()
    _free(d)
