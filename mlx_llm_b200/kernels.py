"""Kernel-level entry points of the C ABI as Python callables (device buffers in, device buffers
out).  Used by the parity tests and the microbenchmarks; the engine API lives in engine.py."""
import ctypes as C

import numpy as np

from ._lib import Context, DevBuf, check, load, ptr


def paged_attn_decode(ctx, q, k_pool, v_pool, block_tables, ctx_lens, num_seqs, hq, hkv, head_dim, page_size, scale,
                      out, max_blocks, chunk_tokens=0):
    check(load().b2_paged_attn_decode(ctx.h, ptr(q), ptr(k_pool), ptr(v_pool), ptr(block_tables), int(max_blocks), ptr(ctx_lens),
                                      int(num_seqs), int(hq), int(hkv), int(head_dim), int(page_size), C.c_float(scale),
                                      int(chunk_tokens), ptr(out)))


def paged_attn_decode_host(ctx, q_host, k_pool, v_pool, block_tables, ctx_lens, num_seqs, hq, hkv, head_dim, page_size, scale,
                           out_host, max_blocks, chunk_tokens=0):
    check(load().b2_paged_attn_decode_host(ctx.h, ptr(q_host), ptr(k_pool), ptr(v_pool), ptr(block_tables), int(max_blocks),
                                           ptr(ctx_lens), int(num_seqs), int(hq), int(hkv), int(head_dim), int(page_size),
                                           C.c_float(scale), int(chunk_tokens), ptr(out_host)))
