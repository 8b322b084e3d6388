"""The tensor-parallel reduction over peer memory (b2_tp_peer_*), protocol and arithmetic, on ONE GPU: the ranks
of a group live in one process, their regions are used directly, and the whole group's reduction runs as a single
cooperative launch (kernels that wait on one another are never separate launches on one device).  Checked
bit-exactly against numpy: x = bf16(x + bf16(sum over ranks, in rank order, of the f32 partial sums))."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _lib_check(rc):
    from mlx_llm_b200 import _lib

    _lib.check(rc)


def _upload(lib, ctx, dev_ptr, arr):
    arr = np.ascontiguousarray(arr)
    _lib_check(lib.b2_memcpy_h2d(ctx.h, C.c_void_p(dev_ptr), arr.ctypes.data_as(C.c_void_p), C.c_size_t(arr.nbytes)))


def _download(lib, ctx, dev_ptr, shape, dtype):
    out = np.empty(shape, dtype)
    _lib_check(lib.b2_memcpy_d2h(ctx.h, out.ctypes.data_as(C.c_void_p), C.c_void_p(dev_ptr), C.c_size_t(out.nbytes)))
    return out


@pytest.mark.parametrize("world,hidden,cap", [(2, 256, 64), (4, 1024, 700), (8, 5120, 300), (1, 128, 8)])
def test_peer_reduce_residual_matches_numpy(world, hidden, cap):
    from mlx_llm_b200 import _lib, engine as eng

    lib = _lib.load()
    ctx = _lib.Context(0)
    groups = [eng.TpGroup(ctx, None, r, world) for r in range(world)]
    for g in groups:
        g.peer_alloc(cap, hidden)
    eng.TpGroup.peer_attach_local(groups)
    bufs = [g.peer_buffers() for g in groups]
    assert all(b[2] == cap and b[3] == hidden for b in bufs)
    rng = np.random.default_rng(world * 1000 + hidden)
    x = H.f32_to_bf16_np(rng.standard_normal((cap, hidden)).astype(np.float32))
    for rows in (cap, 1, max(1, cap // 3), cap):  # consecutive reductions reuse the regions and the flags
        parts = [(rng.standard_normal((rows, hidden)) * 3).astype(np.float32) for _ in range(world)]
        for r in range(world):
            _upload(lib, ctx, bufs[r][0], parts[r])
            _upload(lib, ctx, bufs[r][1], x)
        eng.TpGroup.peer_reduce_residual_local(groups, rows)
        ctx.sync()
        acc = parts[0].copy()
        for r in range(1, world):
            acc = acc + parts[r]
        want = x.copy()
        y = H.bf16_to_f32_np(H.f32_to_bf16_np(acc))
        want[:rows] = H.f32_to_bf16_np(H.bf16_to_f32_np(x[:rows]) + y)
        for r in range(world):
            got = _download(lib, ctx, bufs[r][1], (cap, hidden), np.uint16)
            assert np.array_equal(got, want), (world, rows, r)
        x = want
    for g in groups:
        g.free()
    ctx.close()


def test_peer_reduce_argument_errors():
    from mlx_llm_b200 import _lib, engine as eng

    ctx = _lib.Context(0)
    g = eng.TpGroup(ctx, None, 0, 2)
    with pytest.raises(_lib.B2Error):
        g.peer_buffers()                      # nothing attached
    with pytest.raises(_lib.B2Error):
        g.peer_alloc(16, 100)                 # hidden not a multiple of 4 x world
    g.peer_alloc(16, 128)
    with pytest.raises(_lib.B2Error):
        g.peer_alloc(16, 128)                 # one region per group
    with pytest.raises(_lib.B2Error):
        g.peer_attach([b"\0" * 64])           # one handle per rank
    with pytest.raises(_lib.B2Error):
        buf = ctx.buf(np.zeros(8, np.float32))
        g.all_reduce_f32(buf, 8)              # created without an NCCL id
    g.free()
    ctx.close()
