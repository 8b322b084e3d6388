"""Kernel-level entry points of the C ABI as Python callables (device buffers in, device buffers
out).  Used by the parity tests and the microbenchmarks; the engine API lives in engine.py."""
import ctypes as C

import numpy as np

from ._lib import check, load, ptr


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


def paged_attn_prefill(ctx, q, k_pool, v_pool, block_tables, max_blocks, cu_seqlens, ctx_lens, hq, hkv, head_dim, page_size,
                       scale, out):
    cu = np.ascontiguousarray(cu_seqlens, np.int32)
    cl = np.ascontiguousarray(ctx_lens, np.int32)
    check(load().b2_paged_attn_prefill(ctx.h, ptr(q), ptr(k_pool), ptr(v_pool), ptr(block_tables), int(max_blocks), ptr(cu), ptr(cl),
                                       int(cl.size), int(hq), int(hkv), int(head_dim), int(page_size), C.c_float(scale), ptr(out)))


def quantize(ctx, w, out_dim, in_dim, bits, packed, scales, biases, group=64):
    check(load().b2_quantize(ctx.h, ptr(w), C.c_int64(out_dim), C.c_int64(in_dim), int(group), int(bits), ptr(packed), ptr(scales),
                             ptr(biases)))


def dequantize(ctx, packed, scales, biases, out_dim, in_dim, bits, w, group=64):
    check(load().b2_dequantize(ctx.h, ptr(packed), ptr(scales), ptr(biases), C.c_int64(out_dim), C.c_int64(in_dim), int(group),
                               int(bits), ptr(w)))


def unpack_codes(ctx, packed, out_dim, in_dim, bits, codes):
    check(load().b2_unpack_codes(ctx.h, ptr(packed), C.c_int64(out_dim), C.c_int64(in_dim), int(bits), ptr(codes)))


def qmm(ctx, x, packed, scales, biases, m, out_dim, in_dim, bits, y_bf16=None, y_f32=None, group=64):
    check(load().b2_qmm(ctx.h, ptr(x), ptr(packed), ptr(scales), ptr(biases), int(m), int(out_dim), int(in_dim), int(group),
                        int(bits), ptr(y_bf16), ptr(y_f32)))


def qmm_residual(ctx, x, packed, scales, biases, m, out_dim, in_dim, bits, h, group=64):
    check(load().b2_qmm_residual(ctx.h, ptr(x), ptr(packed), ptr(scales), ptr(biases), int(m), int(out_dim), int(in_dim), int(group),
                                 int(bits), ptr(h)))


def qmm_host(ctx, x_host, packed, scales, biases, m, out_dim, in_dim, bits, y_host, group=64):
    check(load().b2_qmm_host(ctx.h, ptr(x_host), ptr(packed), ptr(scales), ptr(biases), int(m), int(out_dim), int(in_dim), int(group),
                             int(bits), ptr(y_host)))


def linear(ctx, x, w, m, out_dim, in_dim, y_bf16=None, y_f32=None):
    check(load().b2_linear(ctx.h, ptr(x), ptr(w), int(m), int(out_dim), int(in_dim), ptr(y_bf16), ptr(y_f32)))


def rms_norm(ctx, x, w, eps, rows, dim, out):
    check(load().b2_rms_norm(ctx.h, ptr(x), ptr(w), C.c_float(eps), int(rows), int(dim), ptr(out)))


def swiglu(ctx, gate, up, n, out):
    check(load().b2_swiglu(ctx.h, ptr(gate), ptr(up), C.c_int64(n), ptr(out)))


def add(ctx, a, b, n, out):
    check(load().b2_add(ctx.h, ptr(a), ptr(b), C.c_int64(n), ptr(out)))


def embed(ctx, table, ids, n, dim, vocab, out):
    check(load().b2_embed(ctx.h, ptr(table), ptr(ids), int(n), int(dim), int(vocab), ptr(out)))


def argmax(ctx, logits, rows, vocab, out):
    check(load().b2_argmax(ctx.h, ptr(logits), int(rows), int(vocab), ptr(out)))


def rope_inv_freq(head_dim, theta, kind=0, factor=1.0, low=1.0, high=4.0, orig=8192.0):
    out = np.empty(head_dim // 2, np.float32)
    check(load().b2_rope_inv_freq(int(head_dim), C.c_float(theta), int(kind), C.c_float(factor), C.c_float(low), C.c_float(high),
                                  C.c_float(orig), ptr(out)))
    return out


def rope_tables(inv_freq, n_pos):
    inv = np.ascontiguousarray(inv_freq, np.float32)
    cos = np.empty((n_pos, inv.size), np.uint16)
    sin = np.empty_like(cos)
    check(load().b2_rope_tables(ptr(inv), int(inv.size), int(n_pos), ptr(cos), ptr(sin)))
    return cos, sin


def rope_kv_append(ctx, qkv, T, hq, hkv, head_dim, positions, slot_mapping, cos, sin, q_norm, k_norm, eps, page_size, k_pool,
                   v_pool, q_out):
    check(load().b2_rope_kv_append(ctx.h, ptr(qkv), int(T), int(hq), int(hkv), int(head_dim), ptr(positions), ptr(slot_mapping),
                                   ptr(cos), ptr(sin), ptr(q_norm), ptr(k_norm), C.c_float(eps), int(page_size), ptr(k_pool),
                                   ptr(v_pool), ptr(q_out)))


META_FIELDS = ["cu_seqlens", "context_lens", "positions", "token_seq", "slot_mapping", "logit_rows", "logit_seq", "dec_ctx",
               "dec_qrow", "dec_slot", "dec_work_off", "dec_work_seq", "dec_work_chunk", "pf_seq", "pf_qstart", "counts"]


def meta_layout(B, T, W, P):
    sizes = [B + 1, B, T, T, T, B, B, B, B, B, B + 1, W, W, P, P, 8]
    off, out = 0, {}
    for name, n in zip(META_FIELDS, sizes):
        out[name] = (off, n)
        off += n
    return out, off


def build_batch_metadata(ctx, seq_slot, q_len, ctx_before, want_logits, upd, chunk_tokens, q_tile, page_size, max_blocks,
                         max_dec_work, max_pf_work, block_tables_dev):
    """Runs the packer; returns a dict of numpy arrays trimmed to their valid lengths."""
    seq_slot = np.ascontiguousarray(seq_slot, np.int32)
    q_len = np.ascontiguousarray(q_len, np.int32)
    ctx_before = np.ascontiguousarray(ctx_before, np.int32)
    want_logits = np.ascontiguousarray(want_logits, np.int32)
    us = np.ascontiguousarray([u[0] for u in upd], np.int32)
    ui = np.ascontiguousarray([u[1] for u in upd], np.int32)
    up = np.ascontiguousarray([u[2] for u in upd], np.int32)
    B, T = int(seq_slot.size), int(q_len.sum())
    lay, total = meta_layout(B, T, max_dec_work, max_pf_work)
    lib = load()
    lib.b2_batch_metadata_elems.restype = C.c_int64
    assert lib.b2_batch_metadata_elems(B, T, max_dec_work, max_pf_work) == total
    out = ctx.empty((total,), np.int32)
    check(lib.b2_memset(ctx.h, ptr(out), 0xFF, C.c_size_t(total * 4)))
    check(lib.b2_build_batch_metadata(ctx.h, ptr(seq_slot), ptr(q_len), ptr(ctx_before), ptr(want_logits), B, ptr(us), ptr(ui), ptr(up),
                                      int(us.size), int(chunk_tokens), int(q_tile), int(page_size), int(max_blocks),
                                      int(max_dec_work), int(max_pf_work), ptr(block_tables_dev), ptr(out)))
    ctx.sync()
    flat = out.download()
    out.free()
    res = {k: flat[o:o + n].copy() for k, (o, n) in lay.items()}
    n_logits, n_dec, n_dw, n_pw = (int(x) for x in res["counts"][:4])
    res["logit_rows"], res["logit_seq"] = res["logit_rows"][:n_logits], res["logit_seq"][:n_logits]
    for k in ("dec_ctx", "dec_qrow", "dec_slot"):
        res[k] = res[k][:n_dec]
    res["dec_work_off"] = res["dec_work_off"][: n_dec + 1]
    res["dec_work_seq"], res["dec_work_chunk"] = res["dec_work_seq"][:n_dw], res["dec_work_chunk"][:n_dw]
    res["pf_seq"], res["pf_qstart"] = res["pf_seq"][:n_pw], res["pf_qstart"][:n_pw]
    res["counts"] = res["counts"][:6]
    return res
