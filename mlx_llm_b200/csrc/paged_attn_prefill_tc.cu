// Chunked-prefill paged attention on the 5th-generation tensor cores (tcgen05 + TMEM), head_dim 128.
//
// Same contract as the warp-level kernel in paged_attn_prefill.cu (it replaces the whole-prompt prefill
// attention of the reference: src/decode/continuous.rs:255 -> src/models/llama.rs:837-852 ->
// src/primitives/attention.rs:68-102, bottom-right aligned causal mask attention.rs:31-39); this one takes
// over for head_dim 128, where a long context makes the chunk's attention the largest item of a step.
//
// CTA = (128-query tile of one sequence's chunk, one q head), flash-attention over 128-key tiles:
//   warp 8      TMA: lane 0 the Q tile once; then per key tile 16 boxes of 16 keys x 64 dims for K and 16
//               for V, a pair of boxes per lane (16 lanes), each located through the block table (a page
//               holds 16 keys of one kv head contiguously); boxes past the context are filled from a page
//               of zeros; three K / V stages
//   warp 9      one thread issues tcgen05.mma: S = Q K^T (M 128 queries, N 128 keys, 8 steps of K = 16
//               over head_dim) into one of two S buffers in TMEM, and O += P V (N = head_dim, 8 steps
//               over the keys, V read as an MN-major operand straight from the page layout) with P taken
//               from TMEM as the A operand; P enters twice, as its bf16 head and its bf16 remainder, so the
//               product keeps ~16 mantissa bits
//   warps 0-7   softmax, thread = (query row = TMEM lane, half of the key tile): reads its 64 scores once,
//               agrees on the row maximum with the row's other thread through shared memory, then exp2, row
//               sum, and P written back with tcgen05.st OVER the scores it came from: the thread's 64 f32
//               columns become 32 columns of bf16 pairs (head) + 32 columns (remainder).
//               The running maximum is raised only when a tile exceeds it by more than 2^8 ("lazy
//               rescale"): P stays within bf16/f32 range, the final division by the row sum makes the
//               result independent of the reference point, and the O accumulator in TMEM is touched
//               (tcgen05.ld / st, after the previous P V has completed) only on those rare tiles.
// The tensor pipe executes one thread's MMAs in issue order, which is all the ordering the S/P buffers need:
// S(j+2) is issued after P(j) V(j) and so overwrites buffer j & 1 only once P(j) has been consumed, while the
// softmax of tile j+1 runs on the other buffer.  No P tile in shared memory: the room goes to a third K/V
// stage.  Every mbarrier wait is bounded.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int QT = 128, KT = 128, HD = 128;
constexpr int kSoftmaxWarps = 8, kTmaWarp = 8, kMmaWarp = 9, kThreads = 320;
constexpr int HALF_BYTES = 128 * 128;            // 128 rows x 64 bf16: one 128B-swizzled block
constexpr int TILE_BYTES = 2 * HALF_BYTES;       // 128 x 128 bf16
constexpr int NS = 3;                            // K / V stages
constexpr int OFF_Q = 0, OFF_K = TILE_BYTES, OFF_V = OFF_K + NS * TILE_BYTES;
constexpr int OFF_BAR = OFF_V + NS * TILE_BYTES; // 224 KB of operands, then 256 B of barriers
constexpr int OFF_X = OFF_BAR + 256;             // row-maximum / row-sum exchange between the two softmax groups
constexpr int SMEM_BYTES = OFF_X + 2048;         // dynamic shared memory must start 1024-byte aligned (checked)
constexpr uint32_t kSpinLimit = 64;
constexpr float kRescaleThreshold = 8.0f;        // log2 units

__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(addr), "r"(bytes) : "memory");
}
// Bounded wait; false when the limit (about 2 s) ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity) {
    long long start = 0;
    while (true) {
        for (uint32_t i = 0; i < kSpinLimit; i++) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}\n"
                : "=r"(ok)
                : "r"(addr), "r"(parity)
                : "memory");
            if (ok) return true;
        }
        const long long now = clock64();
        if (start == 0) start = now;
        if (now - start > 4000000000ll) return false;
    }
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D += A B with A (128 rows x 16 bf16 = 8 columns of bf16 pairs per lane) read from tensor memory
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32_nowait(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
        "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
        "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tc_st16_nowait(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
        "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
        "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
        "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(mbar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(mbar)
        : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart (SBO), descriptor version 1.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand, 128-byte swizzle: 64 contiguous MN elements per 128-byte row, one row per K index,
// 8-row groups 1024 B apart (SBO), the next 64 MN elements 2 KB further (LBO): a V box holds 16 keys as
// [head_dim half][key][64 dims], and every 16-key MMA step starts its own descriptor at its own box.
constexpr int V_BOX_BYTES = 4096;
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | ((uint64_t)((V_BOX_BYTES / 2) >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// f32 accumulate, bf16 x bf16, M = 128, N = 128; bit 16 set = B is MN-major
constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescQK | (1u << 16);

struct TcPrefillExtra {
    int* err;
    int oob_row;  // marks a 16-key box past the context: it is filled from a page of zeros
    int q_box;    // rows per Q box: 128, or the largest power of two that the q tensor's row count allows
    int page_shift;  // log2 of the page size in keys
    // Split over keys (grid.z > 1): CTA z of a work item takes key tiles [z * per, (z + 1) * per) of the item's tiles,
    // per = ceil(tiles / splits), and leaves its unnormalised output, reference maximum and row sum in part_o / part_ml
    // for the merge kernel; with one split the kernel writes the attention output itself.
    int splits;
    float* part_o;   // [work item][q head][split][128 rows][128 dims]
    float* part_ml;  // [work item][q head][split][128 rows][2]: maximum (log2 domain), row sum
};

__global__ void __launch_bounds__(kThreads, 1)
    paged_attn_prefill_tc_kernel(const PrefillAttnParams p, const TcPrefillExtra ex, const __grid_constant__ CUtensorMap map_q,
                                 const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                 const __grid_constant__ CUtensorMap map_zero, const __grid_constant__ CUtensorMap map_zero_v) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // lets a dependent launch (the o_proj kernel, launched with programmatic stream serialisation) set itself up and
    // fetch its first weights now; it still waits for this grid to complete before it reads the attention output
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();
    const int w = blockIdx.x;
    if (w >= *p.n_work) return;
    const uint32_t raw = smem_u32(smem_raw);
    if (raw & 1023u) {  // the swizzled operand layouts need this alignment; every thread sees the same value
        if (threadIdx.x == 0) atomicExch(ex.err, 7);
        return;
    }
    const uint32_t base = raw;
    const uint32_t bar = base + OFF_BAR;
    const uint32_t q_full = bar;
    auto k_full = [&](int s) { return bar + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar + 8u * (4 + s); };
    auto v_full = [&](int s) { return bar + 8u * (7 + s); };
    auto v_empty = [&](int s) { return bar + 8u * (10 + s); };
    auto s_ready = [&](int s) { return bar + 8u * (13 + s); };
    auto p_ready = [&](int s) { return bar + 8u * (15 + s); };  // all softmax warps have written P over S buffer s
    auto x_ready = [&](int s) { return bar + 8u * (17 + s); };  // both softmax groups have published their maxima
    // P V of tile j completes a phase of pv_done(j & 1).  Two barriers, because a softmax warp looks at them only
    // now and then: when it waits for tile t, P V of t - 2 is known to be complete (S(t) could not exist otherwise)
    // and P V of t + 2 cannot have been issued, so on barrier t & 1 the awaited phase is the current or the last one.
    auto pv_done = [&](int s) { return bar + 8u * (19 + s); };
    const uint32_t l_ready = bar + 8u * 21;
    const uint32_t slot_addr = bar + 8u * 22;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (slot_addr - raw));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y, kvh = head / (p.hq / p.hkv);
    const int b = p.pf_seq[w], q_start = p.pf_qstart[w];
    const int tok0 = p.cu_seqlens[b], qn = p.cu_seqlens[b + 1] - tok0;
    const int ctx = p.context_lens[b], ctx_before = ctx - qn;
    const int rows = min(QT, qn - q_start);
    const int page_size = p.page_tiles * 16;
    const int last_q_pos = ctx_before + q_start + rows - 1;
    const int all_tiles = last_q_pos / KT + 1;
    // this CTA's key tiles: global tile j0 + j for j < n_tiles (every index below is local; only key positions and
    // page look-ups add j0)
    const int tiles_per = (all_tiles + ex.splits - 1) / ex.splits;
    const int j0 = (int)blockIdx.z * tiles_per;
    const int n_tiles = min(tiles_per, all_tiles - j0);
    if (n_tiles <= 0) return;  // the merge kernel computes the same ranges and skips this split

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < NS; s++) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(s_ready(s), 1);
            mbar_init(p_ready(s), kSoftmaxWarps);
            mbar_init(x_ready(s), kSoftmaxWarps);
        }
        mbar_init(l_ready, kSoftmaxWarps);
        mbar_init(pv_done(0), 1);
        mbar_init(pv_done(1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot_addr), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 256u;
    bool alive = true;

    if (warp == kTmaWarp) {
        // Lane 0 loads the Q tile.  Then 24 lanes share each key tile, one copy apiece: lanes 0-15 the 16-key x 64-dim
        // boxes of K (box s = lane % 8, head_dim half = lane / 8), lanes 16-23 the 16-key boxes of V (both halves in
        // one rank-3 box), each looking up its own page one tile ahead.  Issuing a copy occupies its thread for ~100
        // cycles whoever issues it; spread over lanes the copies overlap, from one thread they did not.
        const int32_t* bt = p.block_tables + (size_t)p.seq_slot[b] * p.max_blocks;
        if (lane == 0) {
            // the Q tile in as few boxes as the q tensor's height allows (a box is never taller than the tensor and
            // never starts outside it; rows of the tile that stay unwritten belong to queries whose results are dropped)
            const int q_boxes = (rows + ex.q_box - 1) / ex.q_box;
            const uint32_t q_box_bytes = (uint32_t)ex.q_box * 128u;
            mbar_expect_tx(q_full, (uint32_t)q_boxes * 2u * q_box_bytes);
            for (int qb = 0; qb < q_boxes; qb++) {
                tma_load_2d(base + OFF_Q + qb * q_box_bytes, &map_q, head * HD, tok0 + q_start + qb * ex.q_box, q_full);
                tma_load_2d(base + OFF_Q + HALF_BYTES + qb * q_box_bytes, &map_q, head * HD + 64, tok0 + q_start + qb * ex.q_box, q_full);
            }
        }
        if (lane < 24) {
            const int sub = lane & 7, khalf = (lane >> 3) & 1;
            const bool is_v = lane >= 16;
            const unsigned grp = is_v ? 0xff0000u : 0xffffu;
            const CUtensorMap* map_kv = is_v ? &map_v : &map_k;
            const uint32_t dst0 = base + (is_v ? (uint32_t)OFF_V + (uint32_t)sub * V_BOX_BYTES : (uint32_t)OFF_K + (uint32_t)sub * 2048u);
            // page of this lane's box; the index is clamped to the block-table row so the load is unconditional
            auto page_of = [&](int j) {
                const int blk = ((j0 + j) * KT + sub * 16) >> ex.page_shift;
                return __ldg(bt + (blk < p.max_blocks ? blk : p.max_blocks - 1));
            };
            int pg = page_of(0);
            int st = 0;
            uint32_t par = 0;  // stage of tile j and the parity of its use of that stage
            for (int j = 0; j < n_tiles; j++) {
                const int pg_next = j + 1 < n_tiles ? page_of(j + 1) : 0;
                // row of the box in the pool's (page, kv head, slot) order; self-checks: never past the block-table
                // row, never outside the pool; a box past the context is filled from a page of zeros
                const int key0 = (j0 + j) * KT + sub * 16;
                int row = ex.oob_row;
                if (key0 < ctx) {
                    const long rr = (((long)pg * p.hkv + kvh) << ex.page_shift) + (key0 & (page_size - 1));
                    if ((key0 >> ex.page_shift) >= p.max_blocks)
                        atomicExch(ex.err, 5);
                    else if (rr < 0 || rr + 16 > p.pool_rows)
                        atomicExch(ex.err, 6);
                    else
                        row = (int)rr;
                }
                pg = pg_next;
                const uint32_t full = is_v ? v_full(st) : k_full(st);
                // the verdict is taken by the eight lanes of the tile together, so none is left behind at the __syncwarp
                if (!__all_sync(grp, mbar_wait(is_v ? v_empty(st) : k_empty(st), par ^ 1u))) {
                    alive = false;
                    break;
                }
                if ((lane & 15) == 0) mbar_expect_tx(full, TILE_BYTES);
                __syncwarp(grp);
                const bool past = row == ex.oob_row;
                const uint32_t dst = dst0 + (uint32_t)st * TILE_BYTES;
                if (is_v) {  // both head_dim halves of the 16 keys in one box
                    tma_load_3d(dst, past ? &map_zero_v : map_kv, 0, past ? 0 : row, 0, full);
                } else {
                    tma_load_2d(dst + (uint32_t)khalf * HALF_BYTES, past ? &map_zero : map_kv, khalf * 64, past ? 0 : row, full);
                }
                if (++st == NS) st = 0, par ^= 1u;
            }
            if (!alive && (lane & 15) == 0) atomicExch(ex.err, 2);
        }
        __syncwarp();
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            // Descriptors are linear in the address (14 bits of address >> 4, no carry inside 227 KB), so the loop
            // adds offsets instead of rebuilding them: this thread's instruction count per tile sets how soon the next
            // MMAs are queued.
            uint64_t dq[HD / 16];
#pragma unroll
            for (int k = 0; k < HD / 16; k++) dq[k] = desc_kmajor(base + OFF_Q + (uint32_t)(k >> 2) * HALF_BYTES + (uint32_t)(k & 3) * 32);
            const uint64_t dk0 = desc_kmajor(base + OFF_K), dv0 = desc_mnmajor(base + OFF_V);
            // S[j & 1] = Q K_j^T; `kst` is the K stage of tile j
            auto issue_qk = [&](int j, int kst) {
                const uint64_t dk = dk0 + (uint64_t)((uint32_t)kst * (TILE_BYTES >> 4));
                const uint32_t ts = tmem_base + (uint32_t)(j & 1) * 128u;
#pragma unroll
                for (int k = 0; k < HD / 16; k++)
                    tc_mma(ts, dq[k], dk + (uint64_t)((uint32_t)(k >> 2) * (HALF_BYTES >> 4) + (uint32_t)(k & 3) * 2), kIdescQK, k > 0 ? 1u : 0u);
                tc_commit(s_ready(j & 1));
                tc_commit(k_empty(kst));
            };
            alive = mbar_wait(q_full, 0) && mbar_wait(k_full(0), 0);
            if (alive) {
                tc_fence_after();
                issue_qk(0, 0);
            }
            if (alive && n_tiles > 1) {
                alive = mbar_wait(k_full(1), 0);
                if (alive) {
                    tc_fence_after();
                    issue_qk(1, 1);
                }
            }
            int vst = 0, kst = 2 % NS;  // V stage of tile j, K stage of tile j + 2
            uint32_t vpar = 0, kpar = (2 / NS) & 1u;
            for (int j = 0; j < n_tiles && alive; j++) {
                const int sb = j & 1;
                alive = mbar_wait(v_full(vst), vpar) && mbar_wait(p_ready(sb), (uint32_t)(j >> 1) & 1u);
                if (!alive) break;
                tc_fence_after();
                const uint64_t dvs = dv0 + (uint64_t)((uint32_t)vst * (TILE_BYTES >> 4));
                const uint32_t tP = tmem_base + (uint32_t)sb * 128u;
#pragma unroll
                for (int k = 0; k < KT / 16; k++) {  // O += P_hi V + P_lo V, 16 keys per step
                    // keys 0-63 of the tile: head in columns 0-31 of the buffer, remainder in 32-63; keys 64-127: 64-95, 96-127
                    const uint32_t ta = tP + (uint32_t)(k >> 2) * 64u + (uint32_t)(k & 3) * 8u;
                    const uint64_t dv = dvs + (uint64_t)((uint32_t)k * (V_BOX_BYTES >> 4));
                    tc_mma_ts(tmem_o, ta, dv, kIdescPV, (j > 0 || k > 0) ? 1u : 0u);
                    tc_mma_ts(tmem_o, ta + 32u, dv, kIdescPV, 1u);
                }
                tc_commit(pv_done(sb));
                tc_commit(v_empty(vst));
                if (++vst == NS) vst = 0, vpar ^= 1u;
                if (j + 2 < n_tiles) {
                    // S(j+2) goes over P(j): issued after the MMAs above, which the tensor pipe completes first
                    alive = mbar_wait(k_full(kst), kpar);
                    if (!alive) break;
                    tc_fence_after();
                    issue_qk(j + 2, kst);
                    if (++kst == NS) kst = 0, kpar ^= 1u;
                }
            }
            if (!alive) atomicExch(ex.err, 3);
        }
        __syncwarp();
    } else {
        // ---------------- softmax: thread = (query row = TMEM lane, half of the key tile) ----------------
        // warps 0-3 take keys 0-63 of every tile, warps 4-7 keys 64-127 (a warp reaches the TMEM lanes
        // 32 * (warp % 4) ..); the two threads of a row agree on the row maximum through shared memory
        const int wg = warp >> 2, r = tid & 127;
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        const bool row_ok = r < rows;
        // last key this row may see; rows past the chunk see the whole context (their result is dropped)
        const int kvis = row_ok ? min(ctx_before + q_start + r, ctx - 1) : ctx - 1;
        float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's half of the row sum
        volatile float* xb = reinterpret_cast<volatile float*>(smem_raw + OFF_X);  // [2 tiles in flight][2 groups][128 rows]
        for (int j = 0; j < n_tiles && alive; j++) {
            const int st = j & 1;
            const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)st * 128u + (uint32_t)wg * 64u;
            if (!__all_sync(0xffffffffu, mbar_wait(s_ready(st), (uint32_t)(j >> 1) & 1u))) {
                alive = false;
                break;
            }
            tc_fence_after();
            const int key_base = (j0 + j) * KT + wg * 64;
            const bool need_mask = key_base + 63 > kvis;
            // this thread's 64 scores (log2 domain, masked), their maximum, then the maximum of the whole row
            uint32_t v0[32], v1[32];
            tc_ld32_nowait(s_addr, v0);
            tc_ld32_nowait(s_addr + 32u, v1);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            // raw scores: the scale is positive, so the maximum can be taken first and scaled once, and the
            // exponent below is one fused multiply-add per score.  Masking (diagonal tiles only) writes -inf.
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (key_base + i > kvis) v0[i] = 0xff800000u;
                    if (key_base + 32 + i > kvis) v1[i] = 0xff800000u;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                mx0 = fmaxf(mx0, __uint_as_float(v0[i]));
                mx1 = fmaxf(mx1, __uint_as_float(v0[i + 1]));
                mx2 = fmaxf(mx2, __uint_as_float(v1[i]));
                mx3 = fmaxf(mx3, __uint_as_float(v1[i + 1]));
            }
            float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
            xb[(st * 2 + wg) * 128 + r] = mx;
            __syncwarp();
            if (lane == 0) mbar_arrive(x_ready(st));  // (release: the maxima above are visible to whoever sees the phase complete)
            if (!__all_sync(0xffffffffu, mbar_wait(x_ready(st), (uint32_t)(j >> 1) & 1u))) {
                alive = false;
                break;
            }
            mx = fmaxf(mx, xb[(st * 2 + (wg ^ 1)) * 128 + r]);
            // raise the reference point only when this tile exceeds it by more than the threshold
            float alpha = 1.f;
            bool rescale = false;
            if (j == 0) {
                // key 0 is visible to every row, so the first tile of the whole range gives a finite maximum; a later
                // split may begin on a tile that a row does not see at all: it starts from a finite floor instead, so
                // that exp2(-inf - m) is 0 and not NaN, and is rescaled away by the first tile the row does see
                m_run = fmaxf(mx, -1e30f);
            } else if (mx > m_run + kRescaleThreshold) {
                alpha = exp2f(m_run - mx);
                m_run = mx;
                rescale = true;
            }
            if (__any_sync(0xffffffffu, rescale)) {  // this group rescales its half of the head dimension
                // O belongs to the previous tile's P V until it has completed (P V of this tile cannot have been
                // issued yet: it waits for this warp's arrival below)
                if (!__all_sync(0xffffffffu, mbar_wait(pv_done((j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u))) {
                    alive = false;
                    break;
                }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 2; c++) {
                    const uint32_t o_addr = tmem_o + lane_addr + (uint32_t)wg * 64u + (uint32_t)c * 32u;
                    uint32_t v[32];
                    tc_ld32(o_addr, v);
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tc_st32(o_addr, v);
                }
            }
            l_run *= alpha;
            // P = exp2(scale * s - m), row sum; bf16 head and remainder as pairs of consecutive keys, over the scores'
            // own columns.  The head is the upper 16 bits of the f32 (truncated, not rounded: the remainder carries what
            // is cut off, and truncating the remainder leaves a relative error below 2^-15), so the split costs integer
            // and add instructions only -- conversions share the exp2 unit's narrow issue rate.
            // Columns of this thread's 64: head of keys 0-31 in 0-15, of keys 32-63 in 16-31, remainders in 32-47 and
            // 48-63 (a column holds two consecutive keys); the first half is on its way while the second is computed.
            const float neg_m = -m_run, sc = p.scale_log2;
            float l0 = 0.f, l1 = 0.f;
            {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float a0 = fast_exp2(fmaf(__uint_as_float(v0[2 * i]), sc, neg_m)), a1 = fast_exp2(fmaf(__uint_as_float(v0[2 * i + 1]), sc, neg_m));
                    l0 += a0;
                    l1 += a1;
                    const uint32_t u0 = __float_as_uint(a0), u1 = __float_as_uint(a1);
                    hi[i] = __byte_perm(u0, u1, 0x7632);
                    lo[i] = __byte_perm(__float_as_uint(a0 - __uint_as_float(u0 & 0xffff0000u)), __float_as_uint(a1 - __uint_as_float(u1 & 0xffff0000u)), 0x7632);
                }
                tc_st16_nowait(s_addr, hi);
                tc_st16_nowait(s_addr + 32u, lo);
            }
            {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float a0 = fast_exp2(fmaf(__uint_as_float(v1[2 * i]), sc, neg_m)), a1 = fast_exp2(fmaf(__uint_as_float(v1[2 * i + 1]), sc, neg_m));
                    l0 += a0;
                    l1 += a1;
                    const uint32_t u0 = __float_as_uint(a0), u1 = __float_as_uint(a1);
                    hi[i] = __byte_perm(u0, u1, 0x7632);
                    lo[i] = __byte_perm(__float_as_uint(a0 - __uint_as_float(u0 & 0xffff0000u)), __float_as_uint(a1 - __uint_as_float(u1 & 0xffff0000u)), 0x7632);
                }
                tc_st16_nowait(s_addr + 16u, hi);
                tc_st16_nowait(s_addr + 48u, lo);
            }
            l_run += l0 + l1;
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready(st));
        }
        // ---------------- output: O / l, each group its half of the head dimension ----------------
        if (alive && !__all_sync(0xffffffffu, mbar_wait(pv_done((n_tiles - 1) & 1), (uint32_t)((n_tiles - 1) >> 1) & 1u))) alive = false;
        // the row sum is the two halves' sums (slot of the tile parity that is not in use any more)
        if (alive) {
            const int slot = n_tiles & 1;
            xb[(slot * 2 + wg) * 128 + r] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(l_ready);
            if (!__all_sync(0xffffffffu, mbar_wait(l_ready, 0))) alive = false;
            l_run += xb[(slot * 2 + (wg ^ 1)) * 128 + r];
        }
        if (alive && ex.splits > 1) {
            tc_fence_after();
            const size_t slot = (((size_t)w * p.hq + head) * ex.splits + blockIdx.z) * QT + r;
            float* dst = ex.part_o + slot * HD + wg * 64;
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tc_ld32(tmem_o + lane_addr + (uint32_t)wg * 64u + (uint32_t)c * 32u, v);
                if (row_ok) {
#pragma unroll
                    for (int g = 0; g < 8; g++)
                        *reinterpret_cast<uint4*>(dst + c * 32 + g * 4) = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                }
            }
            if (row_ok && wg == 0) {
                ex.part_ml[slot * 2] = m_run;
                ex.part_ml[slot * 2 + 1] = l_run;
            }
        } else if (alive) {
            tc_fence_after();
            const float inv = 1.0f / l_run;
            uint16_t* dst = p.out + ((size_t)(tok0 + q_start + (row_ok ? r : 0)) * p.hq + head) * HD + wg * 64;
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[32];
                tc_ld32(tmem_o + lane_addr + (uint32_t)wg * 64u + (uint32_t)c * 32u, v);
                if (row_ok && tok0 + q_start + r < p.q_rows) {
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        uint4 o4;
                        o4.x = pack_bf2(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
                        o4.y = pack_bf2(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
                        o4.z = pack_bf2(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
                        o4.w = pack_bf2(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = o4;
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(ex.err, 4);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// Sum of the key splits of one (work item, q head): out = sum_z 2^(m_z - M) O_z / sum_z 2^(m_z - M) l_z with M the
// largest m_z, the splits taken in index order.  One warp per query row at a time, a lane per four head dimensions.
__global__ void __launch_bounds__(128) paged_attn_prefill_merge_kernel(const PrefillAttnParams p, const TcPrefillExtra ex) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();
    const int w = blockIdx.x, head = blockIdx.y;
    if (w >= *p.n_work) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = p.pf_seq[w], q_start = p.pf_qstart[w];
    const int tok0 = p.cu_seqlens[b], qn = p.cu_seqlens[b + 1] - tok0;
    const int ctx_before = p.context_lens[b] - qn;
    const int rows = min(QT, qn - q_start);
    const int all_tiles = (ctx_before + q_start + rows - 1) / KT + 1;
    const int tiles_per = (all_tiles + ex.splits - 1) / ex.splits;
    const int used = (all_tiles + tiles_per - 1) / tiles_per;  // splits that had tiles
    const size_t slot0 = ((size_t)w * p.hq + head) * ex.splits * QT;
    for (int r = warp; r < rows; r += 4) {
        if (tok0 + q_start + r >= p.q_rows) break;
        float M = -INFINITY;
        for (int z = 0; z < used; z++) M = fmaxf(M, ex.part_ml[(slot0 + (size_t)z * QT + r) * 2]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
        for (int z = 0; z < used; z++) {
            const size_t s = slot0 + (size_t)z * QT + r;
            const float wz = exp2f(ex.part_ml[s * 2] - M);
            const float4 o = *reinterpret_cast<const float4*>(ex.part_o + s * HD + lane * 4);
            acc.x = fmaf(wz, o.x, acc.x), acc.y = fmaf(wz, o.y, acc.y), acc.z = fmaf(wz, o.z, acc.z), acc.w = fmaf(wz, o.w, acc.w);
            L = fmaf(wz, ex.part_ml[s * 2 + 1], L);
        }
        const float inv = 1.0f / L;
        uint2 o2;
        o2.x = pack_bf2(acc.x * inv, acc.y * inv);
        o2.y = pack_bf2(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(p.out + ((size_t)(tok0 + q_start + r) * p.hq + head) * HD + lane * 4) = o2;
    }
}

// ---- tensor maps -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}
struct MapEntry {
    const void* ptr;
    uint64_t rows, cols, ld;
    uint32_t box_rows;
    int device;
    CUtensorMap map;
};
// bf16 matrix [rows, cols] with row stride ld elements; box = 64 columns x box_rows, 128-byte swizzle, zero fill
int32_t get_map(b2_ctx* ctx, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, CUtensorMap* out) {
    static thread_local std::vector<MapEntry> cache;
    for (auto& e : cache)
        if (e.ptr == ptr && e.rows == rows && e.cols == cols && e.ld == ld && e.box_rows == box_rows && e.device == ctx->device) {
            *out = e.map;
            return B2_OK;
        }
    EncodeTiledFn fn = encode_fn();
    B2_REQUIRE(fn != nullptr, B2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    B2_REQUIRE(((uintptr_t)ptr & 15) == 0 && (ld * 2) % 16 == 0, B2_ERR_UNSUPPORTED, "tcgen05 attention: operand must be 16-byte aligned");
    if (cache.size() >= 1024) cache.clear();
    MapEntry e{ptr, rows, cols, ld, box_rows, ctx->device, {}};
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B2_REQUIRE(r == CUDA_SUCCESS, B2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    cache.push_back(e);
    *out = e.map;
    return B2_OK;
}

// V rows [rows, 128] bf16 seen as (64 dims, rows, 2 halves): one box = 16 rows with both halves, stored as
// [half][row][64 dims] (128-byte swizzle), which is the MN-major operand layout of a 16-key MMA step.
int32_t get_map_v(b2_ctx* ctx, const void* ptr, uint64_t rows, CUtensorMap* out) {
    static thread_local std::vector<MapEntry> cache;
    for (auto& e : cache)
        if (e.ptr == ptr && e.rows == rows && e.device == ctx->device) {
            *out = e.map;
            return B2_OK;
        }
    EncodeTiledFn fn = encode_fn();
    B2_REQUIRE(fn != nullptr, B2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    B2_REQUIRE(((uintptr_t)ptr & 15) == 0, B2_ERR_UNSUPPORTED, "tcgen05 attention: operand must be 16-byte aligned");
    if (cache.size() >= 1024) cache.clear();
    MapEntry e{ptr, rows, HD, HD, 16, ctx->device, {}};
    const cuuint64_t dims[3] = {64, rows, 2};
    const cuuint64_t strides[2] = {HD * 2, 128};
    const cuuint32_t box[3] = {64, 16, 2};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B2_REQUIRE(r == CUDA_SUCCESS, B2_ERR_CUDA, "cuTensorMapEncodeTiled (V, rank 3) failed with code " + std::to_string((int)r));
    cache.push_back(e);
    *out = e.map;
    return B2_OK;
}

}  // namespace

bool b2_prefill_attn_tc_eligible(const PrefillAttnParams& p, int head_dim) {
    // pages of 16, 32, 64 ... keys: the loader shifts instead of dividing
    return head_dim == 128 && p.page_tiles > 0 && (p.page_tiles & (p.page_tiles - 1)) == 0 && p.pool_rows > 0 && p.q_rows > 0 && ((uintptr_t)p.q & 15) == 0 && ((uintptr_t)p.k_pool & 15) == 0 &&
           ((uintptr_t)p.v_pool & 15) == 0;
}

// The work list (pf_seq / pf_qstart) must have been built with 128-query tiles.
int32_t b2_prefill_attn_tc_launch(b2_ctx* ctx, const PrefillAttnParams& p, int grid_work) {
    if (grid_work <= 0) return B2_OK;
    B2_SMEM_ONCE(ctx, paged_attn_prefill_tc_kernel, SMEM_BYTES);
    if (!ctx->dev_err) {
        B2_CUDA(cudaMalloc((void**)&ctx->dev_err, 16));
        B2_CUDA(cudaMemsetAsync(ctx->dev_err, 0, 16, ctx->stream));
    }
    // a page of zeros for the 16-key boxes that lie past a sequence's context
    static thread_local void* zero_page[16] = {};
    void*& zp = zero_page[ctx->device & 15];
    if (!zp) {
        B2_CUDA(cudaMalloc(&zp, 16 * HD * 2));
        B2_CUDA(cudaMemsetAsync(zp, 0, 16 * HD * 2, ctx->stream));
    }
    CUtensorMap mq, mk, mv, mz, mzv;
    B2_CHECK(get_map(ctx, zp, 16, HD, HD, 16, &mz));
    B2_CHECK(get_map_v(ctx, zp, 16, &mzv));
    // a box is never taller than the tensor it reads
    int q_box = QT;
    while (q_box > p.q_rows) q_box >>= 1;
    B2_CHECK(get_map(ctx, p.q, (uint64_t)p.q_rows, (uint64_t)p.hq * HD, (uint64_t)p.hq * HD, (uint32_t)q_box, &mq));
    B2_CHECK(get_map(ctx, p.k_pool, (uint64_t)p.pool_rows, HD, HD, 16, &mk));
    B2_CHECK(get_map_v(ctx, p.v_pool, (uint64_t)p.pool_rows, &mv));
    int page_shift = 4;
    while ((16 << (page_shift - 4)) < p.page_tiles * 16) page_shift++;
    TcPrefillExtra ex{ctx->dev_err, -1, q_box, page_shift, 1, nullptr, nullptr};
    // A CTA fills an SM (224 KB of operands), so the grid is (work items x q heads) CTAs at one per SM.  When that is
    // well short of the machine and the contexts are long -- a 512-token chunk of a 32K-token prompt on one rank of
    // a tensor-parallel group: 4 x 8 CTAs looping over up to 256 key tiles each -- the keys are split as well, up to
    // what fills the SMs once and leaves every split at least four tiles.
    const int base_ctas = grid_work * p.hq;
    const int max_tiles = (p.max_ctx + KT - 1) / KT;
    int splits = 1;
    if (p.max_ctx > 0 && base_ctas * 2 <= ctx->sm_count) {
        splits = ctx->sm_count / base_ctas;
        if (splits > max_tiles / 4) splits = max_tiles / 4;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    if (splits > 1) {
        const size_t slots = (size_t)grid_work * p.hq * splits * QT;
        const size_t bytes = slots * (HD + 2) * sizeof(float);
        if (bytes > ctx->pf_part_bytes) {
            B2_CUDA(cudaStreamSynchronize(ctx->stream));
            if (ctx->pf_part) B2_CUDA(cudaFree(ctx->pf_part));
            ctx->pf_part = nullptr;
            B2_CUDA(cudaMalloc((void**)&ctx->pf_part, bytes + (bytes >> 2)));
            ctx->pf_part_bytes = bytes + (bytes >> 2);
        }
        ex.splits = splits;
        ex.part_o = ctx->pf_part;
        ex.part_ml = ctx->pf_part + slots * HD;
    }
    dim3 grid(grid_work, p.hq, splits);
    B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, paged_attn_prefill_tc_kernel, grid, dim3(kThreads), (size_t)SMEM_BYTES, ctx->stream, p, ex, mq, mk, mv, mz, mzv));
    B2_LAUNCHED(ctx);
    if (splits > 1) {
        B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, paged_attn_prefill_merge_kernel, dim3(grid_work, p.hq), dim3(128), 0, ctx->stream, p, ex));
        B2_LAUNCHED(ctx);
    }
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
