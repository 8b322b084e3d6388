"""Host-side mirror of the reference's engine API over the C ABI.

Names and argument meaning follow SceneWorks/mlx-llm so that tests read like the reference's own:
Weights (src/primitives/weights.rs), QuantSpec (src/primitives/projection.rs:15-32), ModelConfig
(src/config.rs), CausalLm (src/models/llama.rs), BlockPool / PagedKvCache (src/primitives/
paged_kv_cache.rs), BatchRequest (src/decode/batch.rs:47-59), ContinuousConfig / BatchExactness /
generate_continuous (src/decode/continuous.rs), generate / StreamEvent / FinishReason
(src/decode/stream.rs).  Everything numerical happens inside libb200llm.so.
"""
import ctypes as C
import json
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from ._lib import B2Error, Context, check, load, ptr

# FinishReason (src/decode/stream.rs:31-46)
STOP_TOKEN, MAX_TOKENS, CANCELLED, STOPPED = 0, 1, 2, 3
# BatchExactness (src/decode/continuous.rs:51-63)
EXACT, THROUGHPUT = 0, 1
DTYPES = {np.dtype(np.float32): 0, np.dtype(np.float16): 2, np.dtype(np.uint32): 3, np.dtype(np.int32): 4}


class CModelConfig(C.Structure):
    _fields_ = [
        ("num_layers", C.c_int32), ("hidden_size", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("intermediate_size", C.c_int32), ("vocab_size", C.c_int32),
        ("rms_norm_eps", C.c_float), ("rope_theta", C.c_float), ("rope_kind", C.c_int32),
        ("rope_factor", C.c_float), ("rope_low_freq_factor", C.c_float), ("rope_high_freq_factor", C.c_float),
        ("rope_original_context", C.c_float),
        ("qk_norm", C.c_int32), ("quant_bits", C.c_int32), ("quant_group", C.c_int32), ("tie_word_embeddings", C.c_int32),
        ("compute_f32", C.c_int32),
    ]


class CQuantSpec(C.Structure):
    _fields_ = [("group_size", C.c_int32), ("bits", C.c_int32)]


class CSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int32), ("repetition_penalty", C.c_float),
                ("repetition_context", C.c_int32)]


class CRequest(C.Structure):
    _fields_ = [("prompt_ids", C.POINTER(C.c_int32)), ("n_prompt", C.c_int32), ("sampling", CSampling), ("seed", C.c_uint64),
                ("has_seed", C.c_int32), ("max_new_tokens", C.c_int32), ("stop_tokens", C.POINTER(C.c_int32)), ("n_stop", C.c_int32),
                ("arrival_s", C.c_double)]


class CGenOutput(C.Structure):
    _fields_ = [("tokens", C.POINTER(C.c_int32)), ("capacity", C.c_int32), ("n_tokens", C.c_int32), ("finish_reason", C.c_int32)]


class CContinuousConfig(C.Structure):
    _fields_ = [("max_batch", C.c_int32), ("block_size", C.c_int32), ("exactness", C.c_int32), ("prefill_chunk_tokens", C.c_int32),
                ("max_pages", C.c_int64), ("max_blocks_per_seq", C.c_int32)]


class CRunStats(C.Structure):
    _fields_ = [("steps", C.c_int64), ("decode_tokens", C.c_int64), ("prefill_tokens", C.c_int64), ("kernel_launches", C.c_int64),
                ("device_ms", C.c_double), ("wall_ms", C.c_double), ("peak_live_blocks", C.c_int64), ("peak_concurrent", C.c_int64),
                ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64)]


class CPoolStats(C.Structure):
    _fields_ = [("live_blocks", C.c_int64), ("shared_blocks", C.c_int64), ("peak_live_blocks", C.c_int64),
                ("reserved_tokens", C.c_int64), ("free_pages", C.c_int64), ("total_pages", C.c_int64)]


EVENT_CB = C.CFUNCTYPE(None, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32)


@dataclass
class QuantSpec:
    group_size: int = 64
    bits: int = 4

    @staticmethod
    def q4():
        return QuantSpec(64, 4)

    @staticmethod
    def q8():
        return QuantSpec(64, 8)


def model_config_from_json(text):
    """ModelConfig::from_json (src/config.rs:315-502), Llama / Qwen3 subset."""
    if not isinstance(text, str):
        text = json.dumps(text)
    c = CModelConfig()
    check(load().b2_model_config_from_json(text.encode(), C.byref(c)))
    return c


def model_config(**kw):
    c = CModelConfig(rms_norm_eps=1e-5, rope_theta=500000.0, rope_factor=1.0, rope_low_freq_factor=1.0, rope_high_freq_factor=4.0,
                     rope_original_context=8192.0)
    for k, v in kw.items():
        setattr(c, k, v)
    return c


class Weights:
    """Name -> tensor map (src/primitives/weights.rs:17-96)."""

    def __init__(self, handle=None):
        self.h = handle or C.c_void_p()
        if handle is None:
            check(load().b2_weights_new(C.byref(self.h)))

    @classmethod
    def from_dir(cls, path):
        h = C.c_void_p()
        check(load().b2_weights_from_dir(str(path).encode(), C.byref(h)))
        return cls(h)

    from_file = from_dir

    def add(self, name, arr, bf16=False):
        arr = np.ascontiguousarray(arr)
        dt = 1 if bf16 else DTYPES[arr.dtype]
        shape = (C.c_int64 * arr.ndim)(*arr.shape)
        check(load().b2_weights_add(self.h, name.encode(), dt, shape, arr.ndim, arr.ctypes.data_as(C.c_void_p)))

    def contains(self, name):
        return bool(load().b2_weights_contains(self.h, name.encode()))

    def free(self):
        if self.h:
            load().b2_weights_free(self.h)
            self.h = C.c_void_p()


class CausalLm:
    """CausalLm (src/models/llama.rs:33-330)."""

    def __init__(self, ctx, handle):
        self.ctx, self.h = ctx, handle

    @classmethod
    def from_weights(cls, ctx, weights, prefix, config, quant: Optional[QuantSpec] = None, tp=None):
        h = C.c_void_p()
        q = C.byref(CQuantSpec(quant.group_size, quant.bits)) if quant else None
        check(load().b2_model_from_weights_tp(ctx.h, weights.h, (prefix or "").encode(), C.byref(config), q,
                                              tp.h if tp is not None else None, C.byref(h)))
        return cls(ctx, h)

    from_weights_with = from_weights

    @classmethod
    def synthetic(cls, ctx, config, seed=0, tp=None):
        h = C.c_void_p()
        check(load().b2_model_synthetic_tp(ctx.h, C.byref(config), C.c_uint64(seed), tp.h if tp is not None else None, C.byref(h)))
        return cls(ctx, h)

    def config(self):
        c = CModelConfig()
        check(load().b2_model_get_config(self.h, C.byref(c)))
        return c

    def is_quantized(self):
        return bool(load().b2_model_is_quantized(self.h))

    def weight_bytes(self):
        lib = load()
        lib.b2_model_weight_bytes.restype = C.c_int64
        return int(lib.b2_model_weight_bytes(self.h))

    def new_paged_cache(self, block_size, max_pages=4096, max_blocks=None):
        pool = BlockPool(self.ctx, self, block_size, max_pages, 1, max_blocks or max_pages)
        return PagedKvCache(pool)

    def step(self, seqs, want_logits=True):
        """One ragged forward.  seqs: list of (ids, PagedKvCache).  Returns (logits [n, vocab]: bf16 as uint16, or
        float32 for an f32 model; argmax int32 [n]).  Covers decode_logits / decode_logits_per_seq / Decode::step."""
        ids = np.concatenate([np.ascontiguousarray(s[0], np.int32) for s in seqs])
        n = np.array([len(s[0]) for s in seqs], np.int32)
        arr = (C.c_void_p * len(seqs))(*[s[1].h for s in seqs])
        cfg = self.config()
        vocab = cfg.vocab_size
        logits = np.empty((len(seqs), vocab), np.float32 if cfg.compute_f32 else np.uint16) if want_logits else None
        am = np.empty(len(seqs), np.int32)
        check(load().b2_model_step(self.h, ids.ctypes.data_as(C.c_void_p), n.ctypes.data_as(C.c_void_p), len(seqs), arr,
                                   logits.ctypes.data_as(C.c_void_p) if want_logits else None, am.ctypes.data_as(C.c_void_p)))
        return logits, am

    def free(self):
        if self.h:
            load().b2_model_free(self.h)
            self.h = C.c_void_p()


def step_local_group(models, seqs_per_rank, want_logits=True):
    """One forward of every emulated rank of a group attached with TpGroup.peer_attach_local (b2_model_step_local_group).
    seqs_per_rank[r] is rank r's list of (ids, PagedKvCache) -- the same ids on every rank, each rank's own caches.
    Returns (logits [n, B, vocab] bf16 as uint16 or None, argmax [n, B])."""
    n, B = len(models), len(seqs_per_rank[0])
    ids = np.concatenate([np.ascontiguousarray(s[0], np.int32) for s in seqs_per_rank[0]])
    ntok = np.array([len(s[0]) for s in seqs_per_rank[0]], np.int32)
    marr = (C.c_void_p * n)(*[m.h for m in models])
    carr = (C.c_void_p * (n * B))(*[s[1].h for seqs in seqs_per_rank for s in seqs])
    vocab = models[0].config().vocab_size
    logits = np.empty((n, B, vocab), np.uint16) if want_logits else None
    am = np.empty((n, B), np.int32)
    check(load().b2_model_step_local_group(marr, n, ids.ctypes.data_as(C.c_void_p), ntok.ctypes.data_as(C.c_void_p), B, carr,
                                           logits.ctypes.data_as(C.c_void_p) if want_logits else None, am.ctypes.data_as(C.c_void_p)))
    return logits, am


def write_snapshot(ctx, weights, config_json, out_dir, quant: Optional[QuantSpec] = None):
    """write_snapshot (src/snapshot.rs:86-148): dense tensors -> out_dir/{model.safetensors, config.json}, the
    projections re-quantized to MLX Q4/Q8 triplets when `quant` is given.  Returns the number of tensors written."""
    n = C.c_int32(0)
    q = C.byref(CQuantSpec(quant.group_size, quant.bits)) if quant else None
    cfg = config_json if isinstance(config_json, str) else json.dumps(config_json)
    check(load().b2_write_snapshot(ctx.h, weights.h, cfg.encode(), q, str(out_dir).encode(), C.byref(n)))
    return n.value


class TpGroup:
    """Tensor-parallel group of one rank per GPU (b2_tp_group_*): rank 0 draws the id with
    TpGroup.unique_id(), the caller distributes those 128 bytes, every rank constructs its group."""

    @staticmethod
    def unique_id():
        buf = (C.c_uint8 * 128)()
        check(load().b2_tp_unique_id(buf))
        return bytes(buf)

    def __init__(self, ctx, unique_id, rank, world):
        self.h = C.c_void_p()
        self.rank, self.world = rank, world
        idbuf = (C.c_uint8 * 128).from_buffer_copy(unique_id) if unique_id is not None else None
        check(load().b2_tp_group_create(ctx.h, idbuf, int(rank), int(world), C.byref(self.h)))

    def all_reduce_f32(self, buf, n):
        check(load().b2_tp_all_reduce_f32(self.h, ptr(buf), C.c_int64(n)))

    # ---- reductions over peer memory (b2_tp_peer_*) ----
    def peer_alloc(self, max_tokens, hidden):
        """Allocates this rank's region and returns its 64-byte handle; gather every rank's handle (rank
        order) and pass them to peer_attach."""
        buf = (C.c_uint8 * 64)()
        check(load().b2_tp_peer_alloc(self.h, int(max_tokens), int(hidden), buf))
        return bytes(buf)

    def peer_attach(self, handles):
        blob = b"".join(handles)
        arr = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        check(load().b2_tp_peer_attach(self.h, arr, len(handles)))

    def enable_peer(self, max_tokens, hidden, all_gather):
        """alloc + attach; `all_gather(bytes) -> list of every rank's bytes in rank order` is the caller's
        channel.  Returns False (and leaves the group on NCCL) when a region cannot be mapped."""
        from ._lib import B2Error

        handles = all_gather(self.peer_alloc(max_tokens, hidden))
        try:
            self.peer_attach(handles)
        except B2Error:
            return False
        return True

    def peer_buffers(self):
        """(slots pointer, slot stride in floats, x pointer, max_tokens, hidden) of this rank's region."""
        slots, x = C.c_void_p(), C.c_void_p()
        stride = C.c_int64()
        cap, hidden = C.c_int32(), C.c_int32()
        check(load().b2_tp_peer_buffers(self.h, C.byref(slots), C.byref(stride), C.byref(x), C.byref(cap), C.byref(hidden)))
        return slots.value, stride.value, x.value, cap.value, hidden.value

    def peer_projection(self, x, m, in_dim, w, scales=None, biases=None, bits=0):
        check(load().b2_tp_peer_projection(self.h, ptr(x), int(m), int(in_dim), ptr(w), ptr(scales) if scales is not None else None,
                                           ptr(biases) if biases is not None else None, int(bits)))

    def peer_set_push(self, push):
        check(load().b2_tp_peer_set_push(self.h, 1 if push else 0))

    def peer_reduce_residual(self, rows):
        check(load().b2_tp_peer_reduce_residual(self.h, int(rows)))

    @staticmethod
    def peer_attach_local(groups):
        arr = (C.c_void_p * len(groups))(*[g.h for g in groups])
        check(load().b2_tp_peer_attach_local(arr, len(groups)))

    @staticmethod
    def peer_reduce_residual_local(groups, rows):
        arr = (C.c_void_p * len(groups))(*[g.h for g in groups])
        check(load().b2_tp_peer_reduce_residual_local(arr, len(groups), int(rows)))

    def free(self):
        if self.h:
            check(load().b2_tp_group_free(self.h))
            self.h = C.c_void_p()


class BlockPool:
    """BlockPool (src/primitives/paged_kv_cache.rs:72-160) with bounded physical pages."""

    def __init__(self, ctx, model, block_size, max_pages=1024, max_seqs=8, max_blocks_per_seq=None):
        self.h = C.c_void_p()
        self.block_size = block_size
        check(load().b2_pool_new(ctx.h, model.h, int(block_size), C.c_int64(max_pages), int(max_seqs),
                                 int(max_blocks_per_seq or max_pages), C.byref(self.h)))

    def stats(self):
        s = CPoolStats()
        check(load().b2_pool_stats(self.h, C.byref(s)))
        return {k: int(getattr(s, k)) for k, _ in CPoolStats._fields_}

    def live_blocks(self):
        return self.stats()["live_blocks"]

    def shared_blocks(self):
        return self.stats()["shared_blocks"]

    def peak_live_blocks(self):
        return self.stats()["peak_live_blocks"]

    def reserved_tokens(self):
        return self.stats()["reserved_tokens"]

    def free(self):
        if self.h:
            check(load().b2_pool_free(self.h))
            self.h = C.c_void_p()


class PagedKvCache:
    """PagedKvCache + impl KvCache (src/primitives/paged_kv_cache.rs:168-516)."""

    def __init__(self, pool, seeded=None):
        self.pool = pool
        self.h = C.c_void_p()
        if seeded is None:
            check(load().b2_cache_new(pool.h, C.byref(self.h)))
        else:
            ids = np.ascontiguousarray(seeded, np.int64)
            check(load().b2_cache_new_seeded(pool.h, ids.ctypes.data_as(C.c_void_p), ids.size, C.byref(self.h)))

    @classmethod
    def with_pool(cls, pool):
        return cls(pool)

    @classmethod
    def new_seeded(cls, pool, shared_block_ids):
        return cls(pool, seeded=shared_block_ids)

    def offset(self):
        return int(load().b2_cache_offset(self.h))

    def batch_size(self):
        return int(load().b2_cache_batch_size(self.h))

    def num_layers(self):
        return int(load().b2_cache_num_layers(self.h))

    def blocks(self):
        lib = load()
        lib.b2_cache_blocks.restype = C.c_int64
        return int(lib.b2_cache_blocks(self.h))

    def reserved_tokens(self):
        lib = load()
        lib.b2_cache_reserved_tokens.restype = C.c_int64
        return int(lib.b2_cache_reserved_tokens(self.h))

    def block_ids(self):
        out = np.zeros(8192, np.int64)
        n = load().b2_cache_block_ids(self.h, out.ctypes.data_as(C.c_void_p), out.size)
        return [int(x) for x in out[:n]]

    def truncate(self, n):
        check(load().b2_cache_truncate(self.h, int(n)))

    def reset(self):
        check(load().b2_cache_reset(self.h))

    def retain_sequences(self, keep):
        keep = np.ascontiguousarray(keep, np.int32)
        check(load().b2_cache_retain_sequences(self.h, keep.ctypes.data_as(C.c_void_p), keep.size))

    def shareable_prefix_blocks(self, tokens):
        out = np.zeros(8192, np.int64)
        n = load().b2_cache_shareable_prefix_blocks(self.h, C.c_int64(tokens), out.ctypes.data_as(C.c_void_p), out.size)
        return [int(x) for x in out[:n]]

    def gather(self, layer, n_kv_heads, head_dim):
        """K and V of a layer as [n_kv_heads, len, head_dim] bf16 (uint16) host arrays."""
        n = self.offset()
        k = np.empty((n_kv_heads, n, head_dim), np.uint16)
        v = np.empty_like(k)
        check(load().b2_cache_gather(self.h, int(layer), k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))
        return k, v

    def fork(self, length):
        """A new cache holding the first `length` positions: whole blocks shared, a partial last block copied."""
        c = PagedKvCache.__new__(PagedKvCache)
        c.pool, c.h = self.pool, C.c_void_p()
        check(load().b2_cache_fork(self.h, int(length), C.byref(c.h)))
        return c

    def gather_f32(self, layer, n_kv_heads, head_dim):
        """The same for a pool of an f32 model: float32 arrays."""
        n = self.offset()
        k = np.empty((n_kv_heads, n, head_dim), np.float32)
        v = np.empty_like(k)
        check(load().b2_cache_gather_f32(self.h, int(layer), k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))
        return k, v

    def free(self):
        if self.h:
            load().b2_cache_free(self.h)
            self.h = C.c_void_p()


@dataclass
class SamplingParams:  # src/primitives/sampler.rs:64-90
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    repetition_context: int = 0


@dataclass
class BatchRequest:  # src/decode/batch.rs:47-59 (+ arrival_s extension)
    prompt_ids: List[int]
    max_new_tokens: int = 256
    stop_tokens: List[int] = field(default_factory=list)
    sampling: SamplingParams = field(default_factory=SamplingParams)
    seed: Optional[int] = None
    arrival_s: float = 0.0


@dataclass
class ContinuousConfig:  # src/decode/continuous.rs:67-85 (+ chunking / bounded-pool extensions)
    max_batch: int = 8
    block_size: int = 16
    exactness: int = EXACT
    prefill_chunk_tokens: int = 0
    max_pages: int = 0
    max_blocks_per_seq: int = 0


@dataclass
class GenerationOutput:  # src/decode/stream.rs:91-98
    tokens: List[int]
    finish_reason: int


class CancelFlag:
    """Cross-thread cancel flag (src/decode/cancel.rs): an int32 the engine polls once per step."""

    def __init__(self):
        self.v = C.c_int32(0)

    def cancel(self):
        self.v.value = 1

    def is_cancelled(self):
        return self.v.value != 0


def _c_requests(requests):
    keep = []
    arr = (CRequest * len(requests))()
    for i, r in enumerate(requests):
        p = np.ascontiguousarray(r.prompt_ids, np.int32)
        s = np.ascontiguousarray(r.stop_tokens, np.int32)
        keep += [p, s]
        arr[i].prompt_ids = p.ctypes.data_as(C.POINTER(C.c_int32))
        arr[i].n_prompt = p.size
        sp = r.sampling
        arr[i].sampling = CSampling(sp.temperature, sp.top_p, sp.top_k, sp.repetition_penalty, sp.repetition_context)
        arr[i].seed = r.seed or 0
        arr[i].has_seed = r.seed is not None
        arr[i].max_new_tokens = r.max_new_tokens
        arr[i].stop_tokens = s.ctypes.data_as(C.POINTER(C.c_int32))
        arr[i].n_stop = s.size
        arr[i].arrival_s = r.arrival_s
    return arr, keep


def generate_continuous(model, requests, config: ContinuousConfig, cancel: Optional[CancelFlag] = None, on_event=None,
                        return_stats=False):
    """generate_continuous (src/decode/continuous.rs:117-229).  on_event(request_index, event) with
    event = ("token", id, step) or ("done", reason, generated)."""
    n = len(requests)
    arr, keep = _c_requests(requests)
    outs = (CGenOutput * max(n, 1))()
    bufs = []
    for i, r in enumerate(requests):
        b = np.zeros(max(r.max_new_tokens, 1), np.int32)
        bufs.append(b)
        outs[i].tokens = b.ctypes.data_as(C.POINTER(C.c_int32))
        outs[i].capacity = b.size
    err = []

    def _cb(_user, req, kind, a, b):
        try:
            if on_event:
                on_event(req, ("token", a, b) if kind == 0 else ("done", a, b))
        except Exception as e:  # never unwind through C
            err.append(e)

    cb = EVENT_CB(_cb)
    cfg = CContinuousConfig(config.max_batch, config.block_size, config.exactness, config.prefill_chunk_tokens, config.max_pages,
                            config.max_blocks_per_seq)
    stats = CRunStats()
    check(load().b2_generate_continuous(model.h, arr, n, C.byref(cfg), C.byref(cancel.v) if cancel else None, cb, None, outs,
                                        C.byref(stats)))
    if err:
        raise err[0]
    res = [GenerationOutput(bufs[i][: outs[i].n_tokens].tolist(), int(outs[i].finish_reason)) for i in range(n)]
    if return_stats:
        return res, {k: getattr(stats, k) for k, _ in CRunStats._fields_}
    return res


def generate(model, prompt_ids, max_new_tokens=256, stop_tokens=(), cancel: Optional[CancelFlag] = None, on_event=None):
    """generate (src/decode/stream.rs:113-121): on_event(event) with the same event tuples."""
    req = BatchRequest(list(prompt_ids), max_new_tokens, list(stop_tokens))
    arr, keep = _c_requests([req])
    buf = np.zeros(max(max_new_tokens, 1), np.int32)
    out = CGenOutput(buf.ctypes.data_as(C.POINTER(C.c_int32)), buf.size, 0, 0)
    err = []

    def _cb(_user, _req, kind, a, b):
        try:
            if on_event:
                on_event(("token", a, b) if kind == 0 else ("done", a, b))
        except Exception as e:
            err.append(e)

    cb = EVENT_CB(_cb)
    check(load().b2_generate(model.h, C.byref(arr[0]), C.byref(cancel.v) if cancel else None, cb, None, C.byref(out)))
    if err:
        raise err[0]
    return GenerationOutput(buf[: out.n_tokens].tolist(), int(out.finish_reason))


class CSpeculativeConfig(C.Structure):
    _fields_ = [("max_ngram", C.c_int32), ("num_draft", C.c_int32)]


class CSpeculativeStats(C.Structure):
    _fields_ = [("forwards", C.c_int64), ("proposed", C.c_int64), ("accepted", C.c_int64)]


class CPrefixStats(C.Structure):
    _fields_ = [("lookups", C.c_int64), ("hits", C.c_int64), ("reused_prefix_tokens", C.c_int64), ("computed_prefill_tokens", C.c_int64)]


@dataclass
class SpeculativeConfig:  # src/decode/speculative.rs:45-60
    max_ngram: int = 3
    num_draft: int = 4


def _single(fn_name, model, prompt_ids, max_new_tokens, stop_tokens, cancel, on_event, *extra):
    """Shared driver of the single-sequence loops: builds the request, the output buffer and the callback."""
    req = BatchRequest(list(prompt_ids), max_new_tokens, list(stop_tokens))
    arr, keep = _c_requests([req])
    buf = np.zeros(max(max_new_tokens, 1), np.int32)
    out = CGenOutput(buf.ctypes.data_as(C.POINTER(C.c_int32)), buf.size, 0, 0)
    err = []

    def _cb(_user, _req, kind, a, b):
        try:
            if on_event:
                on_event(("token", a, b) if kind == 0 else ("done", a, b))
        except Exception as e:
            err.append(e)

    cb = EVENT_CB(_cb)
    cancel_p = C.byref(cancel.v) if cancel else None
    yield arr, cancel_p, cb, out
    if err:
        raise err[0]
    yield GenerationOutput(buf[: out.n_tokens].tolist(), int(out.finish_reason))


def generate_prompt_lookup(model, prompt_ids, max_new_tokens=256, spec: Optional[SpeculativeConfig] = None, stop_tokens=(),
                           cancel: Optional[CancelFlag] = None, on_event=None):
    """generate_prompt_lookup (src/decode/speculative.rs:73-171).  Returns (GenerationOutput, stats dict)."""
    spec = spec or SpeculativeConfig()
    g = _single("b2_generate_prompt_lookup", model, prompt_ids, max_new_tokens, stop_tokens, cancel, on_event)
    arr, cancel_p, cb, out = next(g)
    cs, st = CSpeculativeConfig(spec.max_ngram, spec.num_draft), CSpeculativeStats()
    check(load().b2_generate_prompt_lookup(model.h, C.byref(arr[0]), C.byref(cs), cancel_p, cb, None, C.byref(out), C.byref(st)))
    return next(g), dict(forwards=int(st.forwards), proposed=int(st.proposed), accepted=int(st.accepted))


def ngram_propose(history, max_ngram, k):
    h = np.ascontiguousarray(history, np.int32)
    out = np.zeros(max(k, 1), np.int32)
    n = C.c_int32(0)
    check(load().b2_ngram_propose(h.ctypes.data_as(C.c_void_p), int(h.size), int(max_ngram), int(k), out.ctypes.data_as(C.c_void_p), C.byref(n)))
    return out[: n.value].tolist()


class PrefixCache:
    """PrefixCache (src/decode/prefix.rs:56-131) over a page pool of its own."""

    def __init__(self, ctx, model, capacity, max_pages=1024, max_blocks_per_seq=256):
        self.h = C.c_void_p()
        check(load().b2_prefix_cache_new(ctx.h, model.h, int(capacity), C.c_int64(max_pages), int(max_blocks_per_seq), C.byref(self.h)))

    def stats(self):
        s = CPrefixStats()
        check(load().b2_prefix_cache_stats(self.h, C.byref(s)))
        return {k: int(getattr(s, k)) for k, _ in CPrefixStats._fields_}

    def __len__(self):
        return int(load().b2_prefix_cache_len(self.h))

    def free(self):
        if self.h:
            check(load().b2_prefix_cache_free(self.h))
            self.h = C.c_void_p()


def generate_cached(model, prompt_ids, max_new_tokens, prefix_cache: PrefixCache, stop_tokens=(), cancel: Optional[CancelFlag] = None,
                    on_event=None):
    """generate_cached (src/decode/prefix.rs:144-188)."""
    g = _single("b2_generate_cached", model, prompt_ids, max_new_tokens, stop_tokens, cancel, on_event)
    arr, cancel_p, cb, out = next(g)
    check(load().b2_generate_cached(model.h, C.byref(arr[0]), cancel_p, cb, None, prefix_cache.h, C.byref(out)))
    return next(g)


class CProfile(C.Structure):
    _fields_ = [("ms", C.c_double * 8), ("launches", C.c_int64 * 8), ("gemm_flops", C.c_double), ("gemm_weight_bytes", C.c_double),
                ("attn_decode_bytes", C.c_double), ("attn_prefill_flops", C.c_double)]


PROFILE_CLASSES = ["gemm", "attn_decode", "attn_prefill", "rope_kv", "elementwise", "meta_copies", "collective"]


def profile_enable(ctx, on=True):
    check(load().b2_profile_enable(ctx.h, int(bool(on))))


def profile_read(ctx):
    p = CProfile()
    check(load().b2_profile_read(ctx.h, C.byref(p)))
    out = {"ms": {k: p.ms[i] for i, k in enumerate(PROFILE_CLASSES)}, "launches": {k: int(p.launches[i]) for i, k in enumerate(PROFILE_CLASSES)}}
    for k in ("gemm_flops", "gemm_weight_bytes", "attn_decode_bytes", "attn_prefill_flops"):
        out[k] = getattr(p, k)
    return out


class ContinuousEngine:
    """generate_continuous one iteration at a time (b2_continuous_*): step(k) runs up to k iterations
    of the loop and returns (done, cumulative stats)."""

    def __init__(self, model, requests, config: ContinuousConfig, cancel: Optional[CancelFlag] = None, on_event=None):
        self.requests = requests
        self._arr, self._keep = _c_requests(requests)
        self._err = []

        def _cb(_user, req, kind, a, b):
            try:
                if on_event:
                    on_event(req, ("token", a, b) if kind == 0 else ("done", a, b))
            except Exception as e:
                self._err.append(e)

        self._cb = EVENT_CB(_cb) if on_event else C.cast(None, EVENT_CB)
        self._cancel = cancel
        cfg = CContinuousConfig(config.max_batch, config.block_size, config.exactness, config.prefill_chunk_tokens, config.max_pages,
                                config.max_blocks_per_seq)
        self.h = C.c_void_p()
        check(load().b2_continuous_new(model.h, self._arr, len(requests), C.byref(cfg), C.byref(cancel.v) if cancel else None, self._cb,
                                       None, C.byref(self.h)))

    def step(self, max_steps=1):
        done = C.c_int32(0)
        stats = CRunStats()
        check(load().b2_continuous_step(self.h, int(max_steps), C.byref(done), C.byref(stats)))
        if self._err:
            raise self._err[0]
        return bool(done.value), {k: getattr(stats, k) for k, _ in CRunStats._fields_}

    def finish(self):
        n = len(self.requests)
        outs = (CGenOutput * max(n, 1))()
        bufs = []
        for i, r in enumerate(self.requests):
            b = np.zeros(max(r.max_new_tokens, 1), np.int32)
            bufs.append(b)
            outs[i].tokens = b.ctypes.data_as(C.POINTER(C.c_int32))
            outs[i].capacity = b.size
        stats = CRunStats()
        check(load().b2_continuous_finish(self.h, outs, C.byref(stats)))
        return [GenerationOutput(bufs[i][: outs[i].n_tokens].tolist(), int(outs[i].finish_reason)) for i in range(n)], \
            {k: getattr(stats, k) for k, _ in CRunStats._fields_}

    def free(self):
        if self.h:
            load().b2_continuous_free(self.h)
            self.h = C.c_void_p()


class ServingEngine:
    """The continuous-batching loop opened for submissions (b2_continuous_open / _submit / _halt / _result): requests
    join between iterations, each can be halted on its own.  One thread drives it.  on_event(request_id, event) with
    event = ("token", id, step) or ("done", reason, generated) is called from step()."""

    def __init__(self, model, config: ContinuousConfig, on_event=None):
        self._err = []

        def _cb(_user, req, kind, a, b):
            try:
                if on_event:
                    on_event(req, ("token", a, b) if kind == 0 else ("done", a, b))
            except Exception as e:  # a Python exception must not unwind through the C frame
                self._err.append(e)

        self._cb = EVENT_CB(_cb)
        cfg = CContinuousConfig(config.max_batch, config.block_size, config.exactness, config.prefill_chunk_tokens, config.max_pages,
                                config.max_blocks_per_seq)
        self.h = C.c_void_p()
        check(load().b2_continuous_open(model.h, C.byref(cfg), self._cb, None, C.byref(self.h)))

    def submit(self, request: BatchRequest) -> int:
        arr, _keep = _c_requests([request])  # the engine copies the prompt and the stop tokens
        rid = C.c_int32(-1)
        check(load().b2_continuous_submit(self.h, arr, C.byref(rid)))
        return rid.value

    def halt(self, request_id, reason=2):
        check(load().b2_continuous_halt(self.h, int(request_id), int(reason)))

    def result(self, request_id, capacity=4096):
        buf = np.zeros(max(capacity, 1), np.int32)
        n, fin = C.c_int32(0), C.c_int32(-1)
        check(load().b2_continuous_result(self.h, int(request_id), buf.ctypes.data_as(C.POINTER(C.c_int32)), buf.size, C.byref(n), C.byref(fin)))
        return GenerationOutput([int(t) for t in buf[:min(n.value, buf.size)]], fin.value)

    def step(self, max_steps=1):
        """Runs up to max_steps iterations; returns True when the engine is idle (nothing admitted, nothing waiting)."""
        done = C.c_int32(0)
        check(load().b2_continuous_step(self.h, int(max_steps), C.byref(done), None))
        if self._err:
            raise self._err.pop(0)
        return bool(done.value)

    def free(self):
        if self.h:
            load().b2_continuous_free(self.h)
            self.h = C.c_void_p()

