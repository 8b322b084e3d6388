"""Parity of the tcgen05 / TMEM projection kernel (taken for more than 64 tokens when the output width
is a multiple of 128 and K a multiple of 64) against the CPU oracle, and against the warp-level
kernel on the same inputs.  Same bounds as test_gpu_kernels.py: unrounded f32 accumulation within
2e-3, bf16 output within that plus its own rounding."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from mlx_llm_b200 import _lib, kernels
    from oracle import oracle as orc

    ctx = _lib.Context(0)
    yield ctx, kernels, orc, _lib
    ctx.close()


def quant_case(seed, n, k, bits):
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 2**32, size=(n, k * bits // 32), dtype=np.uint32)
    s = np.abs(rng.standard_normal((n, k // 64)).astype(np.float32) * 0.02) / 7.5
    scales = H.f32_to_bf16_np(s)
    biases = H.f32_to_bf16_np(-8.0 * H.bf16_to_f32_np(scales) + rng.standard_normal((n, k // 64)).astype(np.float32) * 1e-3)
    return packed, scales, biases


@pytest.mark.parametrize("bits", [4, 8, 0])
@pytest.mark.parametrize("m,n,k", [(33, 256, 2048), (48, 384, 512), (64, 640, 1024), (65, 128, 64), (100, 256, 512), (256, 128, 4096), (300, 384, 1024), (700, 256, 2048),
                                   # more 256-token blocks than CTA pairs: several pieces per pair, two-block pieces,
                                   # a ragged last block, and an output width that is an odd multiple of 128
                                   (700, 20480, 256), (530, 19072, 128), (1100, 9984, 192)])
def test_tc_gemm_vs_oracle(env, bits, m, n, k):
    ctx, K, orc, _lib = env
    rng = np.random.default_rng(m + n + k)
    x = H.f32_to_bf16_np(rng.standard_normal((m, k)).astype(np.float32))
    dx = ctx.buf(x)
    yb, yf = ctx.empty((m, n), np.uint16), ctx.empty((m, n), np.float32)
    if bits:
        packed, scales, biases = quant_case(1, n, k, bits)
        K.qmm(ctx, dx, ctx.buf(packed), ctx.buf(scales), ctx.buf(biases), m, n, k, bits, yb, yf)
        rf, _ = orc.qmm(x, packed, scales, biases, 64, bits)
    else:
        w = H.f32_to_bf16_np(rng.standard_normal((n, k)).astype(np.float32) * 0.03)
        K.linear(ctx, dx, ctx.buf(w), m, n, k, yb, yf)
        rf, _ = orc.linear(x, w)
    ctx.sync()
    got = yf.download()
    assert np.isfinite(got).all()
    assert np.abs(got - rf).max() <= 2e-3, f"max-abs {np.abs(got - rf).max()}"
    assert H.close_bf16_out(yb.download(), rf)[0]


def test_tc_matches_warp_level_kernel(env):
    """Both projection kernels dequantise to the same bf16 weights and accumulate in f32: their
    unrounded outputs agree to f32 summation-order noise."""
    ctx, K, orc, _lib = env
    m, n, k = 512, 512, 4096
    rng = np.random.default_rng(0)
    x = H.f32_to_bf16_np(rng.standard_normal((m, k)).astype(np.float32))
    packed, scales, biases = quant_case(2, n, k, 4)
    dx, dp, ds, db = ctx.buf(x), ctx.buf(packed), ctx.buf(scales), ctx.buf(biases)
    outs = []
    for use_tc in (1, 0):
        _lib.check(_lib.load().b2_ctx_set_tensor_path(ctx.h, use_tc))
        y = ctx.empty((m, n), np.float32)
        K.qmm(ctx, dx, dp, ds, db, m, n, k, 4, None, y)
        ctx.sync()
        outs.append(y.download())
    _lib.check(_lib.load().b2_ctx_set_tensor_path(ctx.h, 1))
    assert np.abs(outs[0] - outs[1]).max() <= 1e-4


@pytest.mark.parametrize("bits", [4, 8, 0])
@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (5, 256, 512), (8, 1024, 4096), (9, 128, 1024), (16, 384, 2048), (17, 256, 4096),
                                   (32, 512, 1024), (3, 128, 14336)])
def test_stream_gemm_vs_oracle(env, bits, m, n, k):
    """Up to 32 tokens with N a multiple of 128 and K of 256 take the weight-streaming kernel: the token-tile counts
    8, 16 and 32 wide, one and several K ranges, ragged token counts (from 33 tokens on the tcgen05 kernel takes every
    shape its tiling fits, see test_tc_gemm_vs_oracle)."""
    ctx, K, orc, _lib = env
    rng = np.random.default_rng(7 * m + n + k)
    x = H.f32_to_bf16_np(rng.standard_normal((m, k)).astype(np.float32))
    dx = ctx.buf(x)
    yb, yf = ctx.empty((m, n), np.uint16), ctx.empty((m, n), np.float32)
    if bits:
        packed, scales, biases = quant_case(3, n, k, bits)
        K.qmm(ctx, dx, ctx.buf(packed), ctx.buf(scales), ctx.buf(biases), m, n, k, bits, yb, yf)
        rf, _ = orc.qmm(x, packed, scales, biases, 64, bits)
    else:
        w = H.f32_to_bf16_np(rng.standard_normal((n, k)).astype(np.float32) * 0.03)
        K.linear(ctx, dx, ctx.buf(w), m, n, k, yb, yf)
        rf, _ = orc.linear(x, w)
    ctx.sync()
    got = yf.download()
    assert np.isfinite(got).all()
    assert np.abs(got - rf).max() <= 2e-3, f"max-abs {np.abs(got - rf).max()}"
    assert H.close_bf16_out(yb.download(), rf)[0]


def test_stream_matches_tile_kernel(env):
    """Same bf16 weights, f32 accumulation: the streaming kernel and the tile kernel agree to summation-order noise."""
    ctx, K, orc, _lib = env
    m, n, k = 7, 512, 4096
    rng = np.random.default_rng(1)
    x = H.f32_to_bf16_np(rng.standard_normal((m, k)).astype(np.float32))
    packed, scales, biases = quant_case(4, n, k, 4)
    dx, dp, ds, db = ctx.buf(x), ctx.buf(packed), ctx.buf(scales), ctx.buf(biases)
    outs = []
    for fast in (1, 0):
        _lib.check(_lib.load().b2_ctx_set_tensor_path(ctx.h, fast))
        y = ctx.empty((m, n), np.float32)
        K.qmm(ctx, dx, dp, ds, db, m, n, k, 4, None, y)
        ctx.sync()
        outs.append(y.download())
    _lib.check(_lib.load().b2_ctx_set_tensor_path(ctx.h, 1))
    assert np.abs(outs[0] - outs[1]).max() <= 1e-4
