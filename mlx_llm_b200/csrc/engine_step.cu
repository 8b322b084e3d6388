// One decoder forward over a ragged batch (decode tokens and prefill chunks of many sequences).
//
// Replaces CausalLm::decode_logits / decode_logits_per_seq (src/models/llama.rs:351-370, :530-558):
// embed -> per layer [RMSNorm -> fused QKV projection -> (q/k norm) RoPE + KV append -> paged
// attention -> o_proj + residual -> RMSNorm -> gate|up projection -> SwiGLU -> down_proj + residual]
// -> last-token gather + final RMSNorm -> lm_head -> greedy argmax.  One host->device copy of the
// step descriptors before, one device->host copy of the sampled ids (or logits) after.
#include <algorithm>
#include <cstring>

#include "engine.h"

int32_t b2_cache_reserve(b2_cache* c, int n);
void b2_cache_commit(b2_cache* c, int n);
int32_t b2_model_ensure_rope(b2_model* m, int positions);

namespace {

template <typename T>
int32_t regrow(T*& p, size_t elems) {
    if (p) B2_CUDA(cudaFree(p));
    p = nullptr;
    B2_CUDA(cudaMalloc((void**)&p, elems * sizeof(T)));
    return B2_OK;
}

int32_t ensure_workspace(b2_model* m, int T, int B, int W, int P, size_t stage_ints) {
    Workspace& w = m->ws;
    const b2_model_config& c = m->cfg;
    const bool grow_t = T > w.t_cap, grow_b = B > w.b_cap, grow_w = W > w.w_cap, grow_p = P > w.p_cap;
    if (grow_t || grow_b || grow_w || grow_p) B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
    // reductions over peer memory write x on every rank: x then lives in the group's exported region
    const bool peer = m->tp && m->tp->world > 1 && m->tp->peer_ready && m->tp->peer_hidden == c.hidden_size;
    if (peer) {
        B2_REQUIRE(T <= m->tp->peer_cap_rows, B2_ERR_UNSUPPORTED,
                   "a step of " + std::to_string(T) + " tokens exceeds the peer regions' " + std::to_string(m->tp->peer_cap_rows));
        if (!w.x_in_peer_region) {
            B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
            if (w.x) cudaFree(w.x);
            w.x = b2_tp_peer_x(m->tp);
            w.x_in_peer_region = true;
        }
    }
    if (grow_t) {
        const size_t t = (size_t)std::max(T, 64) * 5 / 4;
        const size_t qkv_w = (size_t)(m->hq_l + 2 * m->hkv_l) * c.head_dim;
        if (!w.x_in_peer_region) B2_CHECK(regrow(w.x, t * c.hidden_size));
        B2_CHECK(regrow(w.xn, t * c.hidden_size));
        B2_CHECK(regrow(w.qkv, t * qkv_w));
        B2_CHECK(regrow(w.q, t * m->hq_l * c.head_dim));
        B2_CHECK(regrow(w.attn, t * m->hq_l * c.head_dim));
        B2_CHECK(regrow(w.gu, t * 2 * m->inter_l));
        B2_CHECK(regrow(w.act, t * m->inter_l));
        if (m->tp && m->tp->world > 1) B2_CHECK(regrow(w.tp_part, t * c.hidden_size));
        B2_CHECK(regrow(w.ids, t));
        w.t_cap = (int)t;
    }
    if (grow_b) {
        const size_t b = (size_t)std::max(B, 16) * 5 / 4;
        B2_CHECK(regrow(w.last, b * c.hidden_size));
        B2_CHECK(regrow(w.logits, b * c.vocab_size));
        B2_CHECK(regrow(w.argmax, b));
        if (w.argmax_host) cudaFreeHost(w.argmax_host);
        B2_CUDA(cudaHostAlloc((void**)&w.argmax_host, b * 4, cudaHostAllocDefault));
        w.b_cap = (int)b;
    }
    if (grow_w) w.w_cap = std::max(W, 256) * 5 / 4;
    if (grow_p) w.p_cap = std::max(P, 64) * 5 / 4;
    if (grow_t || grow_b || grow_w || grow_p) {
        B2_CHECK(regrow(w.meta, (size_t)b2_batch_metadata_elems(w.b_cap, w.t_cap, w.w_cap, w.p_cap)));
        const size_t sb = b2_decode_attn_scratch_bytes(w.w_cap, m->hq_l, c.head_dim);
        if (w.attn_scratch) cudaFree(w.attn_scratch);
        B2_CUDA(cudaMalloc((void**)&w.attn_scratch, sb));
        w.attn_scratch_bytes = sb;
    }
    if (stage_ints > w.stage_cap) {
        B2_CUDA(cudaStreamSynchronize(m->ctx->stream));
        const size_t n = stage_ints * 5 / 4 + 1024;
        B2_CHECK(regrow(w.stage_dev, n));
        if (w.stage_host) cudaFreeHost(w.stage_host);
        B2_CUDA(cudaHostAlloc((void**)&w.stage_host, n * 4, cudaHostAllocDefault));
        w.stage_cap = n;
    }
    return B2_OK;
}

int32_t gemm(b2_model* m, const Proj& p, const uint16_t* x, int M, int ldx, uint16_t* out, int ldo, const uint16_t* res, int x_rows_cap) {
    GemmParams g{};
    g.x_rows_cap = x_rows_cap;
    g.x = x;
    g.w = p.w;
    g.scales = p.scales;
    g.biases = p.biases;
    g.sbt = p.sbt;
    g.bits = p.bits;
    g.group = 64;
    g.M = M;
    g.N = p.N;
    g.K = p.K;
    g.ldx = ldx;
    g.ldo = ldo;
    g.ldres = ldo;
    g.epilogue = res ? EPI_BF16_RESADD : EPI_BF16;
    g.out = out;
    g.res = res;
    return b2_gemm_launch(m->ctx, g);
}

// x += proj(a) where every tensor-parallel rank holds a slice of the input dimension: f32 partial
// products, a sum over the ranks, then the residual add with the fused epilogue's roundings.
int32_t gemm_reduce_residual(b2_model* m, const Proj& p, const uint16_t* a, int M, int lda, uint16_t* x, int H, int x_rows_cap) {
    b2_ctx* ctx = m->ctx;
    GemmParams g{};
    g.x_rows_cap = x_rows_cap;
    g.x = a;
    g.w = p.w;
    g.scales = p.scales;
    g.biases = p.biases;
    g.sbt = p.sbt;
    g.bits = p.bits;
    g.group = 64;
    g.M = M;
    g.N = p.N;
    g.K = p.K;
    g.ldx = lda;
    g.ldo = H;
    g.ldres = H;
    g.epilogue = EPI_F32;
    b2_prof_mark(ctx, B2_CLS_GEMM);
    if (m->ws.x_in_peer_region) {  // the epilogue stores each column range into its owner's memory; one kernel sums + adds the residual
        b2_tp_peer_scatter(m->tp, g);
        B2_CHECK(b2_gemm_launch(ctx, g));
        b2_prof_mark(ctx, B2_CLS_COLLECTIVE);
        return b2_tp_peer_reduce_residual_launch(m->tp, M);
    }
    g.out_f32 = m->ws.tp_part;
    B2_CHECK(b2_gemm_launch(ctx, g));
    b2_prof_mark(ctx, B2_CLS_COLLECTIVE);
    B2_CHECK(b2_tp_all_reduce_sum_f32(m->tp, m->ws.tp_part, (size_t)M * H));
    b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
    return b2_residual_add_f32_launch(ctx, m->ws.tp_part, (int64_t)M * H, x);
}

int pick_chunk_tiles(long dec_ctx_sum, int hkv, int sm_count) {
    // enough (chunk, kv head) CTAs for ~8 per SM, chunks between 128 and 1024 tokens
    long target = (long)sm_count * 8;
    long tok = dec_ctx_sum * hkv / std::max(1l, target);
    int chunk = 128;
    while (chunk < 1024 && chunk < tok) chunk *= 2;
    return chunk / 16;
}

// The bf16 layers of one step: embedding, every decoder layer, the sampled rows' final norm, lm_head and argmax.
int32_t forward_bf16_layers(b2_model* m, b2_pool* pool, const BatchMetaOut& mo, const BatchMetaIn& in, const int32_t* ids_dev, int T, int n_dec,
                            long dec_ctx_sum, int W, int P, double pf_flops, int pf_max_ctx, int chunk_tiles, int q_tile, int n_logits, const int32_t* logit_rows) {
    b2_ctx* ctx = m->ctx;
    const b2_model_config& c = m->cfg;
    Workspace& w = m->ws;
    const int H = c.hidden_size, hq = m->hq_l, hkv = m->hkv_l, hd = c.head_dim, I = m->inter_l;  // this rank's heads / columns
    const bool tp = m->tp && m->tp->world > 1;
    const int qkv_w = (hq + 2 * hkv) * hd;
    const float scale_log2 = powf((float)hd, -0.5f) * 1.4426950408889634f;  // attn_scale, config.rs:597-598
    b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
    B2_CHECK(b2_embed_launch(ctx, m->embed, ids_dev, T, H, c.vocab_size, w.x));
    for (int l = 0; l < c.num_layers; l++) {
        const LayerW& L = m->layers[l];
        b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
        B2_CHECK(b2_rms_norm_launch(ctx, w.x, L.input_ln, c.rms_norm_eps, T, H, H, nullptr, w.xn));
        b2_prof_mark(ctx, B2_CLS_GEMM);
        B2_CHECK(gemm(m, L.qkv, w.xn, T, H, w.qkv, qkv_w, nullptr, w.t_cap));
        RopeKvParams rp{};
        rp.qkv = w.qkv;
        rp.ld = qkv_w;
        rp.positions = mo.positions;
        rp.slot_mapping = mo.slot_mapping;
        rp.cos_table = m->cos_tab;
        rp.sin_table = m->sin_tab;
        rp.q_norm = L.q_norm;
        rp.k_norm = L.k_norm;
        rp.eps = c.rms_norm_eps;
        rp.T = T;
        rp.hq = hq;
        rp.hkv = hkv;
        rp.hd = hd;
        rp.page_size = pool->block_size;
        rp.k_pool = pool->k_layer(l);
        rp.v_pool = pool->v_layer(l);
        rp.q_out = w.q;
        b2_prof_mark(ctx, B2_CLS_ROPE_KV);
        B2_CHECK(b2_rope_kv_launch(ctx, rp));
        if (n_dec > 0) {
            DecodeAttnParams dp{};
            dp.q = w.q;
            dp.k_pool = pool->k_layer(l);
            dp.v_pool = pool->v_layer(l);
            dp.block_tables = pool->block_tables;
            dp.max_blocks = pool->max_blocks;
            dp.bt_rows = mo.dec_slot;
            dp.q_rows = mo.dec_qrow;
            dp.ctx_lens = mo.dec_ctx;
            dp.work_seq = mo.dec_work_seq;
            dp.work_chunk = mo.dec_work_chunk;
            dp.seq_work_off = mo.dec_work_off;
            dp.n_work = mo.counts + 2;
            dp.chunk_tiles = chunk_tiles;
            dp.hq = hq;
            dp.hkv = hkv;
            dp.page_tiles = pool->block_size / 16;
            dp.scale_log2 = scale_log2;
            dp.part_o = w.attn_scratch;
            dp.part_ml = w.attn_scratch + (size_t)w.w_cap * hq * hd;
            dp.out = w.attn;
            dp.num_seqs = n_dec;
            B2_CHECK(b2_decode_attn_counters(ctx, n_dec, hkv, &dp.merge_counters));
            b2_prof_mark(ctx, B2_CLS_ATTN_DECODE);
            B2_CHECK(b2_decode_attn_launch(ctx, dp, hd, W, n_dec));
            ctx->attn_decode_bytes += (double)dec_ctx_sum * hkv * hd * 2 * 2;
        }
        if (P > 0) {
            PrefillAttnParams pp{};
            pp.q = w.q;
            pp.k_pool = pool->k_layer(l);
            pp.v_pool = pool->v_layer(l);
            pp.block_tables = pool->block_tables;
            pp.max_blocks = pool->max_blocks;
            pp.seq_slot = in.seq_slot;
            pp.cu_seqlens = mo.cu_seqlens;
            pp.context_lens = mo.context_lens;
            pp.pf_seq = mo.pf_seq;
            pp.pf_qstart = mo.pf_qstart;
            pp.n_work = mo.counts + 3;
            pp.hq = hq;
            pp.hkv = hkv;
            pp.page_tiles = pool->block_size / 16;
            pp.scale_log2 = scale_log2;
            pp.out = w.attn;
            pp.q_tile = q_tile;
            pp.q_rows = w.t_cap;
            pp.pool_rows = (int64_t)pool->max_pages * hkv * pool->block_size;
            pp.max_ctx = pf_max_ctx;
            b2_prof_mark(ctx, B2_CLS_ATTN_PREFILL);
            B2_CHECK(b2_prefill_attn_launch(ctx, pp, hd, P));
            ctx->attn_prefill_flops += pf_flops;
        }
        if (tp) {
            B2_CHECK(gemm_reduce_residual(m, L.o, w.attn, T, hq * hd, w.x, H, w.t_cap));
        } else {
            b2_prof_mark(ctx, B2_CLS_GEMM);
            B2_CHECK(gemm(m, L.o, w.attn, T, hq * hd, w.x, H, w.x, w.t_cap));  // h = x + o_proj(attn)
        }
        b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
        B2_CHECK(b2_rms_norm_launch(ctx, w.x, L.post_ln, c.rms_norm_eps, T, H, H, nullptr, w.xn));
        b2_prof_mark(ctx, B2_CLS_GEMM);
        B2_CHECK(gemm(m, L.gu, w.xn, T, H, w.gu, 2 * I, nullptr, w.t_cap));
        b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
        B2_CHECK(b2_swiglu_launch(ctx, w.gu, T, I, w.act));
        if (tp) {
            B2_CHECK(gemm_reduce_residual(m, L.down, w.act, T, I, w.x, H, w.t_cap));
        } else {
            b2_prof_mark(ctx, B2_CLS_GEMM);
            B2_CHECK(gemm(m, L.down, w.act, T, I, w.x, H, w.x, w.t_cap));  // x = h + down(...)
        }
    }
    if (n_logits > 0) {
        b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
        B2_CHECK(b2_rms_norm_launch(ctx, w.x, m->norm, c.rms_norm_eps, n_logits, H, H, logit_rows, w.last));
        Proj head;
        head.bits = 0;
        head.N = c.vocab_size;
        head.K = H;
        head.w = m->lm_head;
        b2_prof_mark(ctx, B2_CLS_GEMM);
        B2_CHECK(gemm(m, head, w.last, n_logits, H, w.logits, c.vocab_size, nullptr, w.b_cap));
        b2_prof_mark(ctx, B2_CLS_ELEMENTWISE);
        B2_CHECK(b2_argmax_launch(ctx, w.logits, n_logits, c.vocab_size, w.argmax));
    }
    return B2_OK;
}

}  // namespace

int32_t b2_engine_forward(b2_model* m, std::vector<SeqStep>& seqs, void* logits_out, int32_t* argmax_out) {
    b2_ctx* ctx = m->ctx;
    const b2_model_config& c = m->cfg;
    const int B = (int)seqs.size();
    if (B == 0) return B2_OK;
    B2_CUDA(cudaSetDevice(ctx->device));
    b2_pool* pool = seqs[0].cache->pool;
    int T = 0, max_pos = 0, n_logits = 0, n_dec = 0;
    long dec_ctx_sum = 0;
    const bool all_positions = seqs[0].all_positions;
    B2_REQUIRE(!all_positions || B == 1, B2_ERR_MSG, "forward: logits of every position are available for a step of one sequence");
    for (auto& s : seqs) {
        B2_REQUIRE(s.cache && s.cache->pool == pool, B2_ERR_MSG, "forward: all caches of a step must share one pool");
        B2_REQUIRE(s.n > 0, B2_ERR_MSG, "forward: a sequence contributes no token");
        T += s.n;
        max_pos = std::max(max_pos, s.cache->len + s.n);
        n_logits += s.want_logits ? 1 : 0;
        if (s.n == 1) {
            n_dec++;
            dec_ctx_sum += s.cache->len + 1;
        }
    }
    {  // a cache may appear once per step: stamp each with the number of this step
        const uint64_t stamp = ++pool->step_stamp;
        for (auto& s : seqs) {
            B2_REQUIRE(s.cache->step_stamp != stamp, B2_ERR_MSG, "forward: a cache appears twice in one step");
            s.cache->step_stamp = stamp;
        }
    }
    ctx->pdl_consumers = T >= ctx->pdl_min_tokens;  // (see b2_launch_pdl)
    B2_CHECK(b2_model_ensure_rope(m, max_pos));
    // pages for the new tokens (host allocator), then the step descriptors
    for (auto& s : seqs) B2_CHECK(b2_cache_reserve(s.cache, s.n));
    const int chunk_tiles = pick_chunk_tiles(dec_ctx_sum, m->hkv_l, ctx->sm_count);
    const int q_tile = b2_prefill_q_tile(ctx, c.head_dim);
    int W = 0, P = 0;
    double pf_flops = 0;  // 4*hd*hq flops per (query, visible key) pair
    int pf_max_ctx = 0;   // longest context among the sequences that prefill in this step
    for (auto& s : seqs) {
        if (s.n > 1) pf_max_ctx = std::max(pf_max_ctx, s.cache->len + s.n);
        if (s.n > 1) pf_flops += 4.0 * c.head_dim * m->hq_l * ((double)s.n * s.cache->len + 0.5 * (double)s.n * (s.n + 1));
        if (s.n == 1) {
            const int tiles = (s.cache->len + 1 + 15) / 16;
            W += (tiles + chunk_tiles - 1) / chunk_tiles;
        } else {
            P += (s.n + q_tile - 1) / q_tile;
        }
    }
    if (all_positions) n_logits = T;  // rows 0..T-1 of the step, in order
    const int U = (int)pool->upd_slot.size();
    const size_t stage_ints = 4 * (size_t)B + 3 * (size_t)U + (size_t)T;
    B2_CHECK(ensure_workspace(m, T, std::max(B, n_logits), W, P, stage_ints));
    Workspace& w = m->ws;
    int32_t* sh = w.stage_host;
    for (int i = 0; i < B; i++) {
        sh[i] = seqs[i].cache->slot;
        sh[B + i] = seqs[i].n;
        sh[2 * B + i] = seqs[i].cache->len;
        sh[3 * B + i] = seqs[i].want_logits ? 1 : 0;
    }
    if (U) {
        memcpy(sh + 4 * B, pool->upd_slot.data(), (size_t)U * 4);
        memcpy(sh + 4 * B + U, pool->upd_index.data(), (size_t)U * 4);
        memcpy(sh + 4 * B + 2 * U, pool->upd_page.data(), (size_t)U * 4);
    }
    {
        int32_t* ids = sh + 4 * B + 3 * U;
        for (auto& s : seqs) {
            memcpy(ids, s.ids, (size_t)s.n * 4);
            ids += s.n;
        }
    }
    cudaStream_t st = ctx->stream;
    B2_CUDA(cudaEventRecord(m->ev0, st));
    b2_prof_mark(ctx, B2_CLS_META);
    B2_CUDA(cudaMemcpyAsync(w.stage_dev, sh, stage_ints * 4, cudaMemcpyHostToDevice, st));
    m->h2d_bytes += (int64_t)stage_ints * 4;
    pool->upd_slot.clear();
    pool->upd_index.clear();
    pool->upd_page.clear();

    BatchMetaIn in{};
    const int32_t* d = w.stage_dev;
    in.seq_slot = d;
    in.q_len = d + B;
    in.ctx_before = d + 2 * B;
    in.want_logits = d + 3 * B;
    in.upd_slot = d + 4 * B;
    in.upd_index = d + 4 * B + U;
    in.upd_page = d + 4 * B + 2 * U;
    const int32_t* ids_dev = d + 4 * B + 3 * U;
    in.B = B;
    in.T = T;
    in.U = U;
    in.chunk_tiles = chunk_tiles;
    in.q_tile = q_tile;
    in.page_size = pool->block_size;
    in.max_blocks = pool->max_blocks;
    BatchMetaOut mo{};
    mo.block_tables = pool->block_tables;
    b2_batch_meta_carve(w.meta, B, T, W, P, mo);
    B2_CHECK(b2_batch_meta_launch(ctx, in, mo));

    float* logits_f32_dev = nullptr;
    if (m->f32) {
        B2_CHECK(b2_forward_f32(m, pool, mo, in.seq_slot, ids_dev, T, B, n_logits, all_positions ? nullptr : mo.logit_rows, max_pos, &logits_f32_dev));
    } else {
        B2_CHECK(forward_bf16_layers(m, pool, mo, in, ids_dev, T, n_dec, dec_ctx_sum, W, P, pf_flops, pf_max_ctx, chunk_tiles, q_tile, n_logits,
                                     all_positions ? nullptr : mo.logit_rows));
    }
    if (n_logits > 0) {
        b2_prof_mark(ctx, B2_CLS_META);
        B2_CUDA(cudaMemcpyAsync(w.argmax_host, w.argmax, (size_t)n_logits * 4, cudaMemcpyDeviceToHost, st));
        m->d2h_bytes += (int64_t)n_logits * 4;
        if (logits_out) {
            const size_t bytes = (size_t)n_logits * c.vocab_size * (m->f32 ? 4 : 2);
            if (bytes > w.logits_host_cap) {
                B2_CUDA(cudaStreamSynchronize(st));
                if (w.logits_host) cudaFreeHost(w.logits_host);
                B2_CUDA(cudaHostAlloc((void**)&w.logits_host, bytes, cudaHostAllocDefault));
                w.logits_host_cap = bytes;
            }
            B2_CUDA(cudaMemcpyAsync(w.logits_host, m->f32 ? (const void*)logits_f32_dev : (const void*)w.logits, bytes, cudaMemcpyDeviceToHost, st));
            m->d2h_bytes += (int64_t)bytes;
        }
    }
    // the error word a bounded device-side wait raises travels back with the sampled ids
    B2_CUDA(cudaMemcpyAsync(ctx->err_host, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    m->d2h_bytes += (int64_t)sizeof(int);
    b2_prof_mark(ctx, -1);
    B2_CUDA(cudaEventRecord(m->ev1, st));
    B2_CUDA(cudaStreamSynchronize(st));
    B2_CUDA(cudaGetLastError());
    b2_prof_collect(ctx);
    float ms = 0.f;
    B2_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    m->device_ms += ms;
    if (ctx->err_host[0] != 0) {
        // the step's hidden state is incomplete: nothing is sampled and the caches do not advance (their pages
        // stay reserved and are reused by the next step or released with the cache)
        const int code = ctx->err_host[0];
        ctx->err_host[0] = 0;
        B2_CUDA(cudaMemsetAsync(ctx->dev_err, 0, sizeof(int), st));
        return b2_fail(B2_ERR_TIMEOUT, "forward: a bounded device-side wait ran out (code " + std::to_string(code) +
                                           "): the step was abandoned, no token was sampled and no cache advanced");
    }
    if (n_logits > 0) {
        if (argmax_out) memcpy(argmax_out, w.argmax_host, (size_t)n_logits * 4);
        if (logits_out) memcpy(logits_out, w.logits_host, (size_t)n_logits * c.vocab_size * (m->f32 ? 4 : 2));
    }
    for (auto& s : seqs) b2_cache_commit(s.cache, s.n);
    return B2_OK;
}

extern "C" int32_t b2_model_step(b2_model* m, const int32_t* ids_host, const int32_t* n_tokens, int32_t num_seqs, b2_cache** caches,
                                 void* logits_host, int32_t* argmax_host) {
    B2_REQUIRE(m && ids_host && n_tokens && caches, B2_ERR_MSG, "b2_model_step: null argument");
    std::vector<SeqStep> seqs;
    const int32_t* cur = ids_host;
    for (int i = 0; i < num_seqs; i++) {
        B2_REQUIRE(caches[i], B2_ERR_MSG, "b2_model_step: null cache");
        seqs.push_back(SeqStep{caches[i], cur, n_tokens[i], true});
        cur += n_tokens[i];
    }
    return b2_engine_forward(m, seqs, logits_host, argmax_host);
}
