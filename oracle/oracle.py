"""ctypes loader for the CPU oracle — TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the CPU-baseline leg of bench.py import this module.  The product
package never does.  Arrays are numpy; bf16 tensors travel as uint16.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

c_i32p = C.POINTER(C.c_int32)
c_i64p = C.POINTER(C.c_int64)
c_u16p = C.POINTER(C.c_uint16)
c_u32p = C.POINTER(C.c_uint32)
c_u8p = C.POINTER(C.c_uint8)
c_f32p = C.POINTER(C.c_float)


def build(force=False):
    """Compile oracle/_build/liboracle.so with the Makefile beside this file."""
    srcs = [os.path.join(_HERE, f) for f in os.listdir(_HERE) if f.endswith((".cpp", ".h"))]
    if not force and os.path.exists(_SO) and all(os.path.getmtime(_SO) >= os.path.getmtime(s) for s in srcs):
        return _SO
    subprocess.check_call(["make", "-C", _HERE], stdout=subprocess.DEVNULL)
    return _SO


class ModelCfg(C.Structure):
    _fields_ = [
        ("layers", C.c_int32), ("hidden", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("inter", C.c_int32), ("vocab", C.c_int32),
        ("eps", C.c_float), ("theta", C.c_float), ("rope_kind", C.c_int32),
        ("rope_factor", C.c_float), ("rope_low", C.c_float), ("rope_high", C.c_float), ("rope_orig", C.c_float),
        ("qk_norm", C.c_int32), ("quant_bits", C.c_int32), ("group", C.c_int32), ("f32_mode", C.c_int32),
        ("sum_order", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.orc_splitmix64_next.restype = C.c_uint64
        _lib.orc_splitmix64_next_f32.restype = C.c_float
        _lib.orc_argmax_bf16.restype = C.c_int32
        _lib.orc_argmax_f32.restype = C.c_int32
        _lib.orc_synth_tensor_seed.restype = C.c_uint64
        _lib.orc_synth_tensor_seed.argtypes = [C.c_uint64, C.c_int, C.c_int]
        for name in ("orc_model_new", "orc_pool_new", "orc_cache_new_paged", "orc_cache_new_seeded", "orc_cache_new_contiguous"):
            getattr(_lib, name).restype = C.c_void_p
        _lib.orc_cache_gather.restype = C.c_int64
        _lib.orc_cache_offset.restype = C.c_int32
    return _lib


def use_host_cores():
    """Give the OpenMP loops every core this process may run on (launchers such as torch.distributed.run export
    OMP_NUM_THREADS=1 to their children) and return the thread count they will really use."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().orc_set_threads(int(n))
    return int(lib().orc_max_threads())


def threads():
    return int(lib().orc_max_threads())


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---- scalar helpers ------------------------------------------------------------------------------
class SplitMix64:
    def __init__(self, seed):
        self.state = C.c_uint64(seed)

    def next_u64(self):
        return int(lib().orc_splitmix64_next(C.byref(self.state)))

    def next_f32(self):
        return float(lib().orc_splitmix64_next_f32(C.byref(self.state)))


def f32_to_bf16(x):
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x, c_f32p), _p(out, c_u16p), C.c_int64(x.size))
    return out


def bf16_to_f32(x):
    x = _c(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x, c_u16p), _p(out, c_f32p), C.c_int64(x.size))
    return out


# ---- leaves ---------------------------------------------------------------------------------------
def rope_inv_freq(head_dim, theta, kind=0, factor=1.0, low=1.0, high=4.0, orig=8192.0):
    out = np.empty(head_dim // 2, np.float32)
    lib().orc_rope_inv_freq(head_dim, C.c_float(theta), kind, C.c_float(factor), C.c_float(low), C.c_float(high),
                            C.c_float(orig), _p(out, c_f32p))
    return out


def rope_cos_sin(inv_freq, positions):
    inv_freq = _c(inv_freq, np.float32)
    positions = _c(positions, np.int32)
    half = inv_freq.size
    cos = np.empty((positions.size, 2 * half), np.uint16)
    sin = np.empty_like(cos)
    lib().orc_rope_cos_sin(_p(inv_freq, c_f32p), half, _p(positions, c_i32p), positions.size, _p(cos, c_u16p), _p(sin, c_u16p))
    return cos, sin


def apply_rope(x_bf16, cos, sin):
    """x [n, heads, hd] bf16 -> rotated copy."""
    x = _c(x_bf16, np.uint16).copy()
    n, heads, hd = x.shape
    lib().orc_apply_rope(_p(x, c_u16p), _p(_c(cos, np.uint16), c_u16p), _p(_c(sin, np.uint16), c_u16p), n, heads, hd)
    return x


def rms_norm(x_bf16, w_bf16, eps):
    x = _c(x_bf16, np.uint16)
    w = _c(w_bf16, np.uint16)
    out = np.empty_like(x)
    rows = x.size // x.shape[-1]
    lib().orc_rms_norm(_p(x, c_u16p), _p(w, c_u16p), C.c_float(eps), rows, x.shape[-1], _p(out, c_u16p))
    return out


def swiglu(gate, up):
    g = _c(gate, np.uint16)
    u = _c(up, np.uint16)
    out = np.empty_like(g)
    lib().orc_swiglu(_p(g, c_u16p), _p(u, c_u16p), C.c_int64(g.size), _p(out, c_u16p))
    return out


def add_bf16(a, b):
    a = _c(a, np.uint16)
    b = _c(b, np.uint16)
    out = np.empty_like(a)
    lib().orc_add_bf16(_p(a, c_u16p), _p(b, c_u16p), C.c_int64(a.size), _p(out, c_u16p))
    return out


def linear(x_bf16, w_bf16):
    """Returns (f32 accumulations, bf16-rounded)."""
    x = _c(x_bf16, np.uint16)
    w = _c(w_bf16, np.uint16)
    m, k = x.shape
    n = w.shape[0]
    of = np.empty((m, n), np.float32)
    ob = np.empty((m, n), np.uint16)
    lib().orc_linear(_p(x, c_u16p), _p(w, c_u16p), m, n, k, _p(of, c_f32p), _p(ob, c_u16p))
    return of, ob


def argmax_bf16(logits):
    l = _c(logits, np.uint16)
    return int(lib().orc_argmax_bf16(_p(l, c_u16p), l.size))


def unpack_codes(packed, in_dim, bits):
    packed = _c(packed, np.uint32)
    rows = packed.shape[0]
    out = np.empty((rows, in_dim), np.uint8)
    lib().orc_unpack_codes(_p(packed, c_u32p), C.c_int64(rows), C.c_int64(in_dim), bits, _p(out, c_u8p))
    return out


def dequantize(packed, scales, biases, in_dim, group, bits):
    packed = _c(packed, np.uint32)
    rows = packed.shape[0]
    out = np.empty((rows, in_dim), np.uint16)
    lib().orc_dequantize(_p(packed, c_u32p), _p(_c(scales, np.uint16), c_u16p), _p(_c(biases, np.uint16), c_u16p),
                         C.c_int64(rows), C.c_int64(in_dim), group, bits, _p(out, c_u16p))
    return out


def quantize(w_bf16, group, bits):
    w = _c(w_bf16, np.uint16)
    rows, in_dim = w.shape
    packed = np.empty((rows, in_dim * bits // 32), np.uint32)
    scales = np.empty((rows, in_dim // group), np.uint16)
    biases = np.empty_like(scales)
    lib().orc_quantize(_p(w, c_u16p), C.c_int64(rows), C.c_int64(in_dim), group, bits, _p(packed, c_u32p),
                       _p(scales, c_u16p), _p(biases, c_u16p))
    return packed, scales, biases


def qmm(x_bf16, packed, scales, biases, group, bits):
    x = _c(x_bf16, np.uint16)
    packed = _c(packed, np.uint32)
    m, k = x.shape
    n = packed.shape[0]
    of = np.empty((m, n), np.float32)
    ob = np.empty((m, n), np.uint16)
    lib().orc_qmm(_p(x, c_u16p), _p(packed, c_u32p), _p(_c(scales, np.uint16), c_u16p), _p(_c(biases, np.uint16), c_u16p),
                  m, n, k, group, bits, _p(of, c_f32p), _p(ob, c_u16p))
    return of, ob


def host_attn_gqa(q, k, v, scale, causal):
    """q [h, ql, hd], k/v [hkv, kl, hd] f32 -> [h, ql, hd] f32 (f64 accumulate)."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    h, ql, hd = q.shape
    hkv, kl, _ = k.shape
    out = np.empty_like(q)
    lib().orc_host_attn_gqa(_p(q, c_f32p), _p(k, c_f32p), _p(v, c_f32p), h, hkv, ql, kl, hd, C.c_float(scale), int(causal),
                            _p(out, c_f32p))
    return out


def paged_attention(q, kpool, vpool, block_tables, cu_seqlens, ctx_lens, scale, fast_decode=False):
    """q [T, hq, hd] bf16; pools [pages, hkv, page, hd] bf16; returns [T, hq, hd] f32."""
    q = _c(q, np.uint16)
    kpool = _c(kpool, np.uint16)
    vpool = _c(vpool, np.uint16)
    bt = _c(block_tables, np.int32)
    ctx = _c(ctx_lens, np.int32)
    cu = _c(cu_seqlens if cu_seqlens is not None else np.arange(ctx.size + 1), np.int32)
    T, hq, hd = q.shape
    _, hkv, page, _ = kpool.shape
    out = np.empty((T, hq, hd), np.float32)
    if fast_decode:
        assert T == ctx.size
        lib().orc_paged_attention_decode_f32(_p(q, c_u16p), _p(kpool, c_u16p), _p(vpool, c_u16p), _p(bt, c_i32p), bt.shape[1],
                                             _p(ctx, c_i32p), ctx.size, hq, hkv, hd, page, C.c_float(scale), _p(out, c_f32p))
    else:
        lib().orc_paged_attention(_p(q, c_u16p), _p(kpool, c_u16p), _p(vpool, c_u16p), _p(bt, c_i32p), bt.shape[1],
                                  _p(cu, c_i32p), _p(ctx, c_i32p), ctx.size, hq, hkv, hd, page, C.c_float(scale),
                                  _p(out, c_f32p))
    return out


def synth_codes(seed, n_words):
    out = np.empty(n_words, np.uint32)
    lib().orc_synth_codes(C.c_uint64(seed), C.c_int64(n_words), _p(out, c_u32p))
    return out


def synth_scales_biases(seed_scale, seed_bias, n, mul, mid):
    s = np.empty(n, np.uint16)
    b = np.empty(n, np.uint16)
    lib().orc_synth_scales_biases(C.c_uint64(seed_scale), C.c_uint64(seed_bias), C.c_int64(n), C.c_float(mul), C.c_float(mid),
                                  _p(s, c_u16p), _p(b, c_u16p))
    return s, b


def synth_dense(seed, n, std):
    out = np.empty(n, np.uint16)
    lib().orc_synth_dense(C.c_uint64(seed), C.c_int64(n), C.c_float(std), _p(out, c_u16p))
    return out


def synth_tensor_seed(seed, layer, which):
    return int(lib().orc_synth_tensor_seed(C.c_uint64(seed), layer, which))


# ---- caches ---------------------------------------------------------------------------------------
class Pool:
    def __init__(self, block_size):
        self.h = C.c_void_p(lib().orc_pool_new(block_size))
        self.block_size = block_size

    def stats(self):
        out = np.zeros(4, np.int64)
        lib().orc_pool_stats(self.h, _p(out, c_i64p))
        return dict(live_blocks=int(out[0]), shared_blocks=int(out[1]), peak_live_blocks=int(out[2]), reserved_tokens=int(out[3]))

    def is_materialized(self, bid):
        return bool(lib().orc_pool_is_materialized(self.h, C.c_int64(bid)))


class Cache:
    """Paged (pool given) or contiguous (pool None) oracle cache.  Rows are token-major
    [step, n_kv*hd] bf16."""

    def __init__(self, layers, pool=None, block_size=None, seeded=None):
        self.layers = layers
        self.pool = pool
        if pool is None and block_size is not None:
            self.pool = pool = Pool(block_size)
        if pool is None:
            self.h = C.c_void_p(lib().orc_cache_new_contiguous(layers))
        elif seeded is not None:
            ids = _c(seeded, np.int64)
            self.h = C.c_void_p(lib().orc_cache_new_seeded(pool.h, layers, _p(ids, c_i64p), ids.size))
        else:
            self.h = C.c_void_p(lib().orc_cache_new_paged(pool.h, layers))
        self.row = None

    def free(self):
        if self.h:
            lib().orc_cache_free(self.h)
            self.h = None

    def update(self, layer, k, v, batch=1):
        k = _c(k, np.uint16)
        v = _c(v, np.uint16)
        step, row = k.shape
        self.row = row
        rc = lib().orc_cache_update(self.h, layer, _p(k, c_u16p), _p(v, c_u16p), step, row, batch)
        if rc != 0:
            raise ValueError("PagedKvCache is single-sequence (batch 1)")
        return self.gather(layer)

    def gather(self, layer):
        n = lib().orc_cache_gather(self.h, layer, None, None)
        k = np.empty(n, np.uint16)
        v = np.empty(n, np.uint16)
        lib().orc_cache_gather(self.h, layer, _p(k, c_u16p), _p(v, c_u16p))
        if self.row:
            k = k.reshape(-1, self.row)
            v = v.reshape(-1, self.row)
        return k, v

    def offset(self):
        return int(lib().orc_cache_offset(self.h))

    def truncate(self, n):
        if lib().orc_cache_truncate(self.h, n) != 0:
            raise ValueError("truncate: negative len")

    def reset(self):
        lib().orc_cache_reset(self.h)

    def retain_sequences(self, keep):
        keep = _c(keep, np.int32)
        if lib().orc_cache_retain_sequences(self.h, _p(keep, c_i32p), keep.size) != 0:
            raise ValueError("retain_sequences expects [] or [0]")

    def paged_stats(self):
        out = np.zeros(4, np.int64)
        lib().orc_cache_paged_stats(self.h, _p(out, c_i64p))
        return dict(blocks=int(out[0]), tail_len=int(out[1]), reserved_tokens=int(out[2]), batch_size=int(out[3]))

    def block_ids(self):
        out = np.zeros(4096, np.int64)
        n = lib().orc_cache_block_ids(self.h, _p(out, c_i64p), out.size)
        return [int(x) for x in out[:n]]

    def shareable_prefix_blocks(self, tokens):
        out = np.zeros(4096, np.int64)
        n = lib().orc_cache_shareable_prefix_blocks(self.h, C.c_int64(tokens), _p(out, c_i64p), out.size)
        return [int(x) for x in out[:n]]


# ---- model -----------------------------------------------------------------------------------------
WHICH = dict(q=0, k=1, v=2, o=3, gate=4, up=5, down=6, embed=7, lm_head=8)
NORMS = dict(input_ln=0, post_ln=1, q_norm=2, k_norm=3, norm=4)


class Model:
    def __init__(self, **cfg):
        self.cfg = ModelCfg(**cfg)
        self.h = C.c_void_p(lib().orc_model_new(C.byref(self.cfg)))

    def free(self):
        if self.h:
            lib().orc_model_free(self.h)
            self.h = None

    def set_dense(self, layer, which, data_f32):
        d = _c(data_f32, np.float32)
        lib().orc_model_set_dense(self.h, layer, WHICH[which], _p(d, c_f32p))

    def set_quantized(self, layer, which, packed, scales, biases, bits, group=64):
        lib().orc_model_set_quantized(self.h, layer, WHICH[which], _p(_c(packed, np.uint32), c_u32p),
                                      _p(_c(scales, np.uint16), c_u16p), _p(_c(biases, np.uint16), c_u16p), bits, group)

    def quantize_projection(self, layer, which, bits, group=64):
        lib().orc_model_quantize_projection(self.h, layer, WHICH[which], bits, group)

    def set_norm(self, layer, which, data_f32):
        d = _c(data_f32, np.float32)
        lib().orc_model_set_norm(self.h, layer, NORMS[which], _p(d, c_f32p), d.size)

    def fill_synthetic(self, seed):
        lib().orc_model_fill_synthetic(self.h, C.c_uint64(seed))

    def forward(self, seqs):
        """seqs: list of (ids, Cache, offset) -> (logits [B, vocab] f32 holding bf16-rounded values,
        unrounded f32 accumulations)."""
        ids = np.concatenate([_c(s[0], np.int32) for s in seqs])
        n = np.array([len(s[0]) for s in seqs], np.int32)
        offs = np.array([s[2] for s in seqs], np.int32)
        arr = (C.c_void_p * len(seqs))(*[s[1].h for s in seqs])
        lg = np.empty((len(seqs), self.cfg.vocab), np.float32)
        lgf = np.empty_like(lg)
        lib().orc_model_forward(self.h, len(seqs), _p(ids, c_i32p), _p(n, c_i32p), arr, _p(offs, c_i32p), _p(lg, c_f32p),
                                _p(lgf, c_f32p))
        return lg, lgf

    def generate(self, prompt, max_new, stop=(), cancel_after_tokens=-1, paged_block=None):
        prompt = _c(prompt, np.int32)
        stop = _c(list(stop), np.int32)
        toks = np.zeros(max(max_new, 1), np.int32)
        n = C.c_int(0)
        reason = C.c_int(0)
        ev = np.zeros((max_new + 2, 4), np.int32)
        nev = C.c_int(0)
        rc = lib().orc_generate(self.h, _p(prompt, c_i32p), prompt.size, max_new, _p(stop, c_i32p), stop.size,
                                cancel_after_tokens, 1 if paged_block else 0, paged_block or 16, _p(toks, c_i32p), C.byref(n),
                                C.byref(reason), _p(ev, c_i32p), ev.shape[0], C.byref(nev))
        if rc != 0:
            raise RuntimeError(f"orc_generate rc={rc}")
        return dict(tokens=toks[: n.value].tolist(), reason=reason.value, events=ev[: nev.value].tolist())

    def generate_continuous(self, prompts, max_new, stops=None, max_batch=8, block_size=16, throughput=False, cancel_after_steps=-1):
        n_req = len(prompts)
        stops = stops or [[] for _ in prompts]
        pcat = np.concatenate([_c(p, np.int32) for p in prompts]) if n_req else np.zeros(0, np.int32)
        plen = np.array([len(p) for p in prompts], np.int32)
        mnew = _c(max_new, np.int32)
        scat = np.concatenate([_c(s, np.int32) for s in stops] + [np.zeros(0, np.int32)])
        nstop = np.array([len(s) for s in stops], np.int32)
        stride = int(max(1, mnew.max() if n_req else 1))
        toks = np.zeros((max(n_req, 1), stride), np.int32)
        ntok = np.zeros(max(n_req, 1), np.int32)
        reasons = np.zeros(max(n_req, 1), np.int32)
        cap = int(mnew.sum() + 2 * n_req + 8) if n_req else 8
        ev = np.zeros((cap, 4), np.int32)
        nev = C.c_int(0)
        bstride = 4096
        bids = np.zeros((max(n_req, 1), bstride), np.int64)
        nb = np.zeros(max(n_req, 1), np.int32)
        pstats = np.zeros(4, np.int64)
        rc = lib().orc_generate_continuous(self.h, n_req, _p(pcat, c_i32p), _p(plen, c_i32p), _p(mnew, c_i32p), _p(scat, c_i32p),
                                           _p(nstop, c_i32p), max_batch, block_size, int(throughput), cancel_after_steps,
                                           _p(toks, c_i32p), stride, _p(ntok, c_i32p), _p(reasons, c_i32p), _p(ev, c_i32p), cap,
                                           C.byref(nev), _p(bids, c_i64p), bstride, _p(nb, c_i32p), _p(pstats, c_i64p), None)
        if rc != 0:
            return dict(error=rc)
        return dict(
            tokens=[toks[i, : ntok[i]].tolist() for i in range(n_req)],
            reasons=reasons[:n_req].tolist(),
            events=ev[: nev.value].tolist(),
            block_ids=[bids[i, : nb[i]].tolist() for i in range(n_req)],
            pool=dict(live_blocks=int(pstats[0]), shared_blocks=int(pstats[1]), peak_live_blocks=int(pstats[2]),
                      reserved_tokens=int(pstats[3])),
        )
