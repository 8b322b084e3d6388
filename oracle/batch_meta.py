"""CPU oracle (TEST INFRASTRUCTURE ONLY) of this build's own scheduling policy.

The reference never packs a ragged batch (src/decode/continuous.rs:254-301 runs whole-prompt batch-1
prefills and per-sequence decode forwards), so there is nothing in it to restate for these arrays.
What is restated here, in plain integer numpy, is the policy the GPU packer and the host page
allocator of this library implement, so the device outputs can be compared bit for bit:

 * physical pages come from a stack that hands out page 0 first and reuses the most recently freed
   page first; a sequence takes a page when the first token of a block arrives, in batch order;
 * per step: cu_seqlens, context lengths, per-token position / owning sequence / KV slot
   (page * page_size + offset), rows that sample, the compact decode arrays with their split-K work
   list (chunks of `chunk_tokens` positions), and the prefill query-tile list.
"""
import numpy as np


class PagePool:
    def __init__(self, max_pages, page_size):
        self.page_size = page_size
        self.free = list(range(max_pages - 1, -1, -1))  # pop() hands out page 0 first
        self.ref = [0] * max_pages

    def alloc(self):
        p = self.free.pop()
        self.ref[p] = 1
        return p

    def unref(self, p):
        self.ref[p] -= 1
        if self.ref[p] == 0:
            self.free.append(p)


class SeqPages:
    """Pages of one sequence (one block-table row)."""

    def __init__(self, pool, slot):
        self.pool, self.slot, self.len, self.pages = pool, slot, 0, []

    def reserve(self, n):
        """Pages for n more tokens; returns the block-table updates (slot, index, page)."""
        bs = self.pool.page_size
        need = (self.len + n + bs - 1) // bs
        upd = []
        while len(self.pages) < need:
            p = self.pool.alloc()
            upd.append((self.slot, len(self.pages), p))
            self.pages.append(p)
        return upd

    def commit(self, n):
        self.len += n

    def free(self):
        for p in self.pages:
            self.pool.unref(p)
        self.pages = []
        self.len = 0


def build_batch_metadata(seq_slot, q_len, ctx_before, want_logits, block_tables, upd, chunk_tokens, q_tile, page_size):
    """block_tables [slots, max_blocks] is updated in place with `upd` first.  Returns the same dict of
    arrays the GPU packer produces."""
    seq_slot = np.asarray(seq_slot, np.int32)
    q_len = np.asarray(q_len, np.int32)
    ctx_before = np.asarray(ctx_before, np.int32)
    want_logits = np.asarray(want_logits, np.int32)
    for s, i, p in upd:
        block_tables[s, i] = p
    B = seq_slot.size
    cu = np.zeros(B + 1, np.int32)
    cu[1:] = np.cumsum(q_len)
    T = int(cu[-1])
    ctx = (ctx_before + q_len).astype(np.int32)
    positions = np.zeros(T, np.int32)
    token_seq = np.zeros(T, np.int32)
    slot_mapping = np.zeros(T, np.int32)
    for i in range(B):
        for j in range(q_len[i]):
            t = cu[i] + j
            pos = ctx_before[i] + j
            positions[t] = pos
            token_seq[t] = i
            slot_mapping[t] = block_tables[seq_slot[i], pos // page_size] * page_size + pos % page_size
    chunk_tiles = chunk_tokens // 16
    logit_rows, logit_seq = [], []
    dec_ctx, dec_qrow, dec_slot, dec_off, dec_ws, dec_wc = [], [], [], [], [], []
    pf_seq, pf_q = [], []
    for i in range(B):
        if q_len[i] > 0 and want_logits[i]:
            logit_rows.append(cu[i] + q_len[i] - 1)
            logit_seq.append(i)
        if q_len[i] == 1:
            d = len(dec_ctx)
            dec_ctx.append(ctx[i])
            dec_qrow.append(cu[i])
            dec_slot.append(seq_slot[i])
            dec_off.append(len(dec_ws))
            tiles = (ctx[i] + 15) // 16
            for c in range((tiles + chunk_tiles - 1) // chunk_tiles):
                dec_ws.append(d)
                dec_wc.append(c)
        elif q_len[i] > 1:
            for s in range(0, q_len[i], q_tile):
                pf_seq.append(i)
                pf_q.append(s)
    dec_off.append(len(dec_ws))
    a = lambda x: np.asarray(x, np.int32)
    return dict(cu_seqlens=cu, context_lens=ctx, positions=positions, token_seq=token_seq, slot_mapping=slot_mapping,
                logit_rows=a(logit_rows), logit_seq=a(logit_seq), dec_ctx=a(dec_ctx), dec_qrow=a(dec_qrow), dec_slot=a(dec_slot),
                dec_work_off=a(dec_off), dec_work_seq=a(dec_ws), dec_work_chunk=a(dec_wc), pf_seq=a(pf_seq), pf_qstart=a(pf_q),
                counts=a([len(logit_rows), len(dec_ctx), len(dec_ws), len(pf_seq), 0, T]))
