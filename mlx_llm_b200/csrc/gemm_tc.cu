// Large-M projection GEMM on the 5th-generation tensor cores, CTA-pair form (tcgen05 cta_group::2).
//
//   y[M, N] = x[M, K] . W[N, K]^T,   W dense bf16 or MLX-format group-64 affine Q4 / Q8
//
// Same contract as the warp-level tile kernel in gemm.cu (it replaces primitives::nn::linear,
// src/primitives/nn.rs:26-33, and QuantizedLinear::forward, src/primitives/quant.rs:56-70); this one
// takes over once a step carries enough tokens for the tensor pipe to be the bound (prefill chunks
// packed with decode tokens).
//
// Why pairs.  With W as the UMMA A operand a CTA dequantises 128 feature rows per 64-wide K slab; the
// only way to spread that cost (and the L2 -> SM traffic of the activation tile, which every feature
// tile re-reads) over more math is more tokens per slab.  A cluster of two CTAs issues one
// 256-feature x N-token MMA whose B operand is split between the two CTAs' shared memories, so each CTA
// holds 128 features x up to 512 tokens of f32 accumulator (all 512 TMEM columns) while loading only
// half of the tokens: one dequantised weight element feeds up to 512 MACs, and the activation bytes
// per MAC are a quarter of a 128 x 256 single-CTA tile.
//
// Work split.  The output is cut into blocks of 256 tokens of one 256-feature tile; every CTA pair takes one
// contiguous run of blocks, equal to within one, and walks it in "pieces" of one or two consecutive blocks of a
// tile (two blocks = all 512 TMEM columns, eight MMAs per 64-wide K slab).  When the blocks alone cannot occupy the
// 74 pairs (down_proj at a few hundred tokens) K is split as well: pieces then write f32 partial sums and a second
// kernel adds the K ranges in range order and applies the epilogue.
//
// Roles per CTA (608 threads):
//   warps 0-15  weight producers, four groups of four warps, group g converting every 4th K slab (thread = feature
//               row): packed codes prefetched into registers, dequantised (w = bf16(code*scale+bias), one
//               rounding), stored in the 128B-swizzled K-major UMMA layout, generic->async proxy fence, one
//               mbarrier arrive per warp on the LEADER CTA's "full" barrier (a remote arrive from the second CTA);
//               afterwards the piece's epilogue: tcgen05.ld 32 lanes x 32 columns, then bf16 / residual-add /
//               f32 / partial-sum stores (the residual rows are fetched a column group ahead)
//   warp 16     one thread drives TMA (tiled bulk-tensor loads, cta_group::2 form, each CTA fetching its own
//               rows): this CTA's half of the token rows of every stage (one 128-row box, or 32-row boxes for
//               short blocks), plus the W tile when the weights are dense bf16; completion bytes land on the
//               leader's "full" barrier
//   warps 17-18 leader CTA only, one thread each issues tcgen05.mma.cta_group::2 and releases stages / publishes
//               the accumulator with tcgen05.commit arriving on both CTAs' barriers: a two-block piece (two
//               instructions per K=16 step) belongs to the first; a one-block piece is shared, even K slabs into
//               TMEM columns 0-255 by the first, odd slabs into 256-511 by the second, added by the epilogue
// An MMA of the pair occupies the tensor pipe for max(93, N/2) cycles (128.6 at N = 256) whatever the accumulator
// pattern; what keeps the kernel under that rate is the turn-around of a ring stage (commit, both CTAs see it free,
// dequantise / TMA, remote arrive, issue), which shared memory does not let the ring hide.
// Every mbarrier wait is bounded: on expiry the kernel raises an error word, stops producing and
// falls through to the common exit, where the TMEM columns are freed.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr int TM = 128;          // features per CTA (half of the UMMA M = 256)
constexpr int PAIR_F = 2 * TM;   // features per CTA pair
constexpr int TN_MAX = 512;      // tokens per piece (all TMEM columns)
constexpr int TK = 64;           // K per slab (one 128-byte swizzled row, one quant group)
constexpr int GROUPS = 4;        // producer groups (4 warps each); group g dequantises every 4th K slab
constexpr int MAX_STAGES = 6;
constexpr int RING_BYTES = 192 * 1024;  // 4 stages of (A + 2 units) for two-block pieces, 6 of (A + 1 unit) otherwise
constexpr int BOX_BIG = 128, BOX_SMALL = 32;  // token rows per TMA box (one big box, or up to two small ones)
constexpr int A_BYTES = TM * TK * 2, UNIT_BYTES = 128 * TK * 2;  // unit: 128 token rows x 64 K, one MMA instruction's B half
constexpr int kProducerWarps = 16, kProducerThreads = kProducerWarps * 32;
// warps: 16 producers (which also run the epilogue), one for TMA, two MMA issuers (the second shares the slabs of
// one-block pieces)
constexpr int kDequantWarps = kProducerWarps;
constexpr int kTmaWarp = kProducerWarps, kMmaWarp = kProducerWarps + 1, kThreads = kProducerThreads + 96;
constexpr int SMEM_BYTES = RING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit = 64;  // try_wait attempts between two looks at the clock

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_local(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}
// arrive on a barrier anywhere in the cluster (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(addr), "r"(bytes) : "memory");
}
// Bounded wait on a barrier of this CTA (cluster-scope acquire: the arrivals come from both CTAs and
// from the tensor core's commit); false when the limit ran out.
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
        if (now - start > 4000000000ll) return false;  // ~2 s: give up instead of hanging
    }
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// arrive (once the MMAs issued so far have completed) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void tc_commit_pair(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(mbar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
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
// 2-D tiled TMA load, CTA-pair form, one destination CTA: the box lands in THIS CTA's shared memory, the
// completion bytes on `mbar`, a shared::cluster address that may name the peer CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(mbar)
        : "memory");
}

// K-major, 128-byte swizzle, rows of 128 B, 8-row groups 1024 B apart (SBO = 64 x 16 B), LBO unused (1),
// descriptor version 1 (bit 46), layout type 2 = SWIZZLE_128B (bits 61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor: f32 accumulate (bit 4), bf16 x bf16 (bits 7, 10), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24 (M = 256 across the pair)
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(PAIR_F >> 4) << 24);
}

__device__ __forceinline__ uint32_t sub_bf2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t fma_bf2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// 32-byte read-only global load (32-byte aligned address) that leaves no copy in L1: every code is read once, and
// keeping the lines out of L1 measured 2-6 % on every shape
__device__ __forceinline__ void ldg256(const uint4* p, uint4& a, uint4& b) {
    asm("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
        : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
        : "l"(p));
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 8 nibbles -> 8 bf16 in natural order (see gemm.cu for the derivation; bit-identical result)
__device__ __forceinline__ void dequant8_q4(uint32_t w, uint32_t s2, uint32_t b2, uint32_t (&out)[4]) {
    const uint32_t magic = 0x43004300u;
    uint32_t r0 = (w & 0x000f000fu) | magic, r1 = ((w >> 4) & 0x000f000fu) | magic;
    uint32_t r2 = ((w >> 8) & 0x000f000fu) | magic, r3 = ((w >> 12) & 0x000f000fu) | magic;
    r0 = fma_bf2(sub_bf2(r0, magic), s2, b2);
    r1 = fma_bf2(sub_bf2(r1, magic), s2, b2);
    r2 = fma_bf2(sub_bf2(r2, magic), s2, b2);
    r3 = fma_bf2(sub_bf2(r3, magic), s2, b2);
    out[0] = prmt(r0, r1, 0x5410u);
    out[1] = prmt(r2, r3, 0x5410u);
    out[2] = prmt(r0, r1, 0x7632u);
    out[3] = prmt(r2, r3, 0x7632u);
}
__device__ __forceinline__ void dequant4_q8(uint32_t w, float s, float b, uint32_t (&out)[2]) {
    const float c0 = (float)(w & 0xffu), c1 = (float)((w >> 8) & 0xffu), c2 = (float)((w >> 16) & 0xffu), c3 = (float)(w >> 24);
    out[0] = pack_bf2(__fmaf_rn(c0, s, b), __fmaf_rn(c1, s, b));
    out[1] = pack_bf2(__fmaf_rn(c2, s, b), __fmaf_rn(c3, s, b));
}

// The output is cut into blocks of 256 tokens of one 256-feature tile (block index = tile * blocks_per_tile
// + token block).  A tcgen05.mma of the pair costs the same for any N up to 256, so a block is the unit
// of cost; every pair gets a contiguous run of blocks, equal to within one.
struct PairPlan {
    int n_pairs;          // CTA pairs launched
    int block_tokens;     // tokens per block: a multiple of 16, at most 256 (the last block of a tile may hold fewer)
    int blocks_per_tile;  // ceil(M / block_tokens)
    int total_blocks;     // ceil(N / 256) * blocks_per_tile
    int splits;           // K ranges per block (> 1 only when the blocks alone cannot occupy the pairs)
    float* partial;       // [splits, M, N] f32 partial sums when splits > 1
    int* err;             // device error word
};

// One piece: one or two consecutive token blocks of 256-feature tile `fp`.
struct Piece {
    int fp, t0, cnt;  // cnt tokens starting at t0
    int n0, n1;       // UMMA N of the two instructions (n1 == 0 for a single block); multiples of 16
    int blocks;       // 1 or 2
    int k0, nk;       // first K slab and number of K slabs
    int split;        // index of the K range
};
// Ring geometry of a piece: two-block pieces use 4 stages of 48 KB (A slab + two B units), one-block pieces
// 4 stages of 32 KB.
// (Four stages also for one-block pieces, although six of their 32 KB stages would fit: measured 5-13 % faster on
// every shape whose pieces are single blocks.  Each producer group then always meets the same stage.)
__device__ __forceinline__ int ring_stages(const Piece& pc) { return 4; }
__device__ __forceinline__ uint32_t ring_stage_bytes(const Piece& pc) { return pc.blocks == 2 ? 48u * 1024u : 32u * 1024u; }
// Phase bookkeeping: bit s of `par` is the parity of the next use of stage s.  After a piece with KT slabs on
// NS stages, stage s has been used ceil((KT - s) / NS) more times.
__device__ __forceinline__ uint32_t ring_advance(uint32_t par, int KT, int NS) {
    for (int st = 0; st < NS; st++) {
        const int uses = KT > st ? (KT - st + NS - 1) / NS : 0;
        par ^= (uint32_t)(uses & 1) << st;
    }
    return par;
}
// Work units are numbered block-major: unit = block * splits + K range.  Without split-K two consecutive
// token blocks of a tile are taken together when the pair owns both.
__device__ __forceinline__ Piece piece_at(int unit, int unit_end, int bpt, int bs, int M, int KT, int splits) {
    Piece pc;
    const int blk = unit / splits;
    pc.split = unit - blk * splits;
    pc.k0 = (int)((long)pc.split * KT / splits);
    pc.nk = (int)((long)(pc.split + 1) * KT / splits) - pc.k0;
    pc.fp = blk / bpt;
    const int tb = blk % bpt;
    pc.blocks = (splits == 1 && tb + 1 < bpt && unit + 1 < unit_end) ? 2 : 1;
    pc.t0 = tb * bs;
    int cnt = M - pc.t0;
    if (cnt > bs * pc.blocks) cnt = bs * pc.blocks;
    pc.cnt = cnt;
    const int padded = (cnt + 15) & ~15;
    pc.n0 = padded < bs ? padded : bs;
    pc.n1 = padded - pc.n0;
    return pc;
}

template <int WK, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_tc_pair_kernel(const GemmParams p, const PairPlan plan, const __grid_constant__ CUtensorMap map_x,
                        const __grid_constant__ CUtensorMap map_x_small, const __grid_constant__ CUtensorMap map_w) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // operand ring: stage s at base + s * stage bytes, A slab first
    const uint32_t bar = base + RING_BYTES;
    auto full = [&](int s) { return bar + 8u * s; };                  // used in the leader CTA only
    auto empty = [&](int s) { return bar + 8u * (MAX_STAGES + s); };  // one per CTA, armed by the leader's commit
    const uint32_t accum_full = bar + 8u * (2 * MAX_STAGES);          // one per CTA
    const uint32_t accum_empty = accum_full + 8u;                     // leader only
    const uint32_t slot_addr = accum_empty + 8u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (slot_addr - raw));
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int M = p.M, N = p.N, K = p.K;
    const int KT = K / TK;
    const int bpt = plan.blocks_per_tile, bs = plan.block_tokens;
    const int splits = plan.splits;
    const int total_units = plan.total_blocks * splits;
    const int blk_begin = (int)((long)pair * total_units / plan.n_pairs);  // first work unit of this pair
    const int blk_end = (int)((long)(pair + 1) * total_units / plan.n_pairs);
    // arrivals per stage on the leader's "full" barrier: the four warps that fill the A slab in each CTA
    // (quantised weights only) plus the leader's TMA thread (arrive.expect_tx for both CTAs' bytes)
    constexpr uint32_t kFullCount = (WK != 0 ? 2 * (kDequantWarps / GROUPS) : 0) + 1;
    const uint32_t leader_accum_empty = map_to_cta(accum_empty, 0);

    if (tid == 0) {
        for (int s = 0; s < MAX_STAGES; s++) {
            mbar_init(full(s), kFullCount);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum_full, 2);  // one commit from each MMA issuer
        mbar_init(accum_empty, 2 * kProducerWarps);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot_addr), "r"(TN_MAX) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anyone arrives remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // All CTAs of this grid are resident from the start (one per SM), so the kernel after it in the stream may be
    // scheduled into whatever frees up as pairs finish; it waits for this grid's completion before it reads anything.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    if (warp < kProducerWarps) {
        // Four groups of four warps; group g dequantises every 4th K slab, one thread per feature row (64
        // codes, one scale and one bias per slab).  While one group waits for its slot or for its barrier
        // arrive to travel to the leader CTA, the other three keep dequantising.
        static_assert(kDequantWarps == 4 * GROUPS, "four warps per producer group");
        constexpr bool dequantises = true;
        const int grp = warp >> 2, row = tid & 127;
        const int groups = K / 64;
        const int lane_grp = warp & 3, col_grp = warp >> 2;
        const uint32_t leader_full0 = leader ? full(0) : map_to_cta(full(0), 0);
        uint32_t it_global = 0;  // K slabs issued before this piece (all roles count the same)
        uint32_t par = 0;        // per-stage phase parities (all roles keep the same)
        uint32_t n_piece = 0;
        bool alive = true;
        for (int blk = blk_begin; blk < blk_end && alive; n_piece++) {
            const Piece pc = piece_at(blk, blk_end, bpt, bs, M, KT, splits);
            blk += pc.blocks;
            const int NS = ring_stages(pc);
            const uint32_t SB = ring_stage_bytes(pc);
            if (WK != 0 && dequantises) {
                const int gn = pc.fp * PAIR_F + (int)rank * TM + row;
                const bool row_ok = gn < N;  // rows past N contribute exact zeros
                const uint4* wq = reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(p.w) + (size_t)(row_ok ? gn : 0) * (K * WK / 32));
                const uint16_t* sc_row = p.scales + (size_t)(row_ok ? gn : 0) * groups;
                const uint16_t* bi_row = p.biases + (size_t)(row_ok ? gn : 0) * groups;
                const uint32_t* sbt_col = p.sbt ? p.sbt + (row_ok ? gn : 0) : nullptr;
                constexpr int NQ = WK == 4 ? 2 : 4;  // 16-byte loads per 64 codes
                // Codes, scale and bias of the next DEPTH slabs of this group wait in registers (DEPTH * GROUPS slabs
                // ahead of the one being dequantised): the loads come from DRAM or a busy L2, and with a single slab
                // in flight per thread the group's period was that latency, not the arithmetic.
                constexpr int DEPTH = 1;
                uint4 q[DEPTH][NQ];
                uint32_t sb[DEPTH];
                auto load_codes = [&](int d, int kb) {
                    // 32 bytes per instruction (sm_100 has 256-bit global loads): a row's 32 or 64 bytes of codes lie in one
                    // 128-byte line of their own, and every load instruction of a warp costs the load unit one tag look-up
                    // per line it touches, so half as many instructions is half of that cost
#pragma unroll
                    for (int i = 0; i < NQ; i += 2) {
                        if (row_ok)
                            ldg256(wq + kb * NQ + i, q[d][i], q[d][i + 1]);
                        else
                            q[d][i] = q[d][i + 1] = make_uint4(0, 0, 0, 0);
                    }
                    // scale and bias: one coalesced 4-byte load where the caller supplies the transposed table (a warp's 32
                    // rows read one 128-byte line), two 2-byte loads that each touch 32 lines where it does not
                    if (!row_ok)
                        sb[d] = 0u;
                    else if (sbt_col)
                        sb[d] = __ldg(sbt_col + (size_t)kb * N);
                    else
                        sb[d] = (uint32_t)__ldg(sc_row + kb) | ((uint32_t)__ldg(bi_row + kb) << 16);
                };
                // first K slab of this piece that belongs to this group
                int kb0 = (int)((grp + GROUPS - (it_global % GROUPS)) % GROUPS);  // slab index within the piece
#pragma unroll
                for (int d = 0; d < DEPTH; d++)
                    if (kb0 + d * GROUPS < pc.nk) load_codes(d, pc.k0 + kb0 + d * GROUPS);
                const uint32_t sw = (uint32_t)(row & 7);
                for (; kb0 < pc.nk && alive; kb0 += GROUPS * DEPTH) {
#pragma unroll
                  for (int d = 0; d < DEPTH; d++) {
                    const int kb = kb0 + d * GROUPS;
                    if (kb >= pc.nk) break;
                    const int st = kb % NS;
                    const uint32_t ph = ((par >> st) ^ (uint32_t)(kb / NS)) & 1u;
                    const uint32_t sA = base + st * SB + row * 128;
                    uint4 cd[NQ];
#pragma unroll
                    for (int i = 0; i < NQ; i++) cd[i] = q[d][i];
                    const uint32_t csc = sb[d] & 0xffffu, cbi = sb[d] >> 16;
                    if (kb + GROUPS * DEPTH < pc.nk) load_codes(d, pc.k0 + kb + GROUPS * DEPTH);
                    // the verdict is taken warp-wide so that no lane leaves the others at the __syncwarp below
                    if (!__all_sync(0xffffffffu, mbar_wait(empty(st), ph ^ 1u))) {
                        alive = false;
                        break;
                    }
                    if (WK == 4) {
                        const uint32_t s2 = csc * 0x10001u, b2 = cbi * 0x10001u;
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const uint32_t w4[4] = {cd[i].x, cd[i].y, cd[i].z, cd[i].w};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint32_t o[4];
                                dequant8_q4(w4[j], s2, b2, o);
                                sts128(sA + ((((uint32_t)(i * 4 + j)) ^ sw) << 4), o[0], o[1], o[2], o[3]);
                            }
                        }
                    } else {
                        const float sf = __uint_as_float(csc << 16), bf = __uint_as_float(cbi << 16);
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            uint32_t lo[2], hi[2];
                            dequant4_q8(cd[i].x, sf, bf, lo);
                            dequant4_q8(cd[i].y, sf, bf, hi);
                            sts128(sA + ((((uint32_t)(i * 2)) ^ sw) << 4), lo[0], lo[1], hi[0], hi[1]);
                            dequant4_q8(cd[i].z, sf, bf, lo);
                            dequant4_q8(cd[i].w, sf, bf, hi);
                            sts128(sA + ((((uint32_t)(i * 2 + 1)) ^ sw) << 4), lo[0], lo[1], hi[0], hi[1]);
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (leader)
                            mbar_arrive_local(leader_full0 + 8u * st);
                        else
                            mbar_arrive_cluster(leader_full0 + 8u * st);
                    }
                  }
                }
                // the first lines of the next piece's weight rows start their way into L2 while this piece drains
                if (blk < blk_end) {
                    const Piece nx = piece_at(blk, blk_end, bpt, bs, M, KT, splits);
                    const int gx = nx.fp * PAIR_F + (int)rank * TM + row;
                    if (gx < N && (nx.fp != pc.fp || nx.k0 != pc.k0) && nx.k0 * (NQ * 16) + grp * 128 < K * WK / 8) {
                        const uint8_t* line = reinterpret_cast<const uint8_t*>(p.w) + ((size_t)gx * (K * WK / 32) + (size_t)nx.k0 * (NQ * 4)) * 4 + grp * 128;
                        asm volatile("prefetch.global.L2 [%0];\n" ::"l"(line));
                    }
                }
            }
            it_global += (uint32_t)pc.nk;
            par = ring_advance(par, pc.nk, NS);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            // ---------------- epilogue of this piece ----------------
            // (the residual it reads and the buffers it writes belong to earlier kernels until they have completed)
            if (n_piece == 0) asm volatile("griddepcontrol.wait;\n" ::: "memory");
            // The residual rows of a 32-token column group are fetched a group ahead, all 32 in flight at once and the
            // first group before the accumulator is waited for: in place (out == res) the compiler must otherwise order
            // every load behind the store before it, and each load would pay the whole trip to L2.
            const int f = pc.fp * PAIR_F + (int)rank * TM + lane_grp * 32 + lane;
            // 32-column groups of the piece: those of the first block (TMEM columns from 0), then those of the second
            // (columns from 256, tokens from t0 + block size)
            const int cnt0 = pc.cnt < bs ? pc.cnt : bs, cnt1 = pc.cnt - cnt0;
            const int grp0 = (cnt0 + 31) >> 5, grps = grp0 + ((cnt1 + 31) >> 5);
            uint32_t r2[16];
            auto load_res = [&](int g) {
                if (EPI == EPI_BF16_RESADD && splits == 1 && f < N && g < grps) {
                    const int tg = g < grp0 ? pc.t0 + g * 32 : pc.t0 + bs + (g - grp0) * 32;
                    const int left = g < grp0 ? cnt0 - g * 32 : cnt1 - (g - grp0) * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const uint32_t lo = i < left ? p.res[(size_t)(tg + i) * p.ldres + f] : 0u;
                        const uint32_t hi = i + 1 < left ? p.res[(size_t)(tg + i + 1) * p.ldres + f] : 0u;
                        r2[i >> 1] = lo | (hi << 16);
                    }
                }
            };
            load_res(col_grp);
            bool ok = mbar_wait(accum_full, n_piece & 1u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                alive = false;
                break;
            }
            tc_fence_after();
#pragma unroll 1
            for (int g = col_grp; g < grps; g += kProducerWarps / 4) {
                const int col = g < grp0 ? g * 32 : 256 + (g - grp0) * 32;
                const int tg = g < grp0 ? pc.t0 + g * 32 : pc.t0 + bs + (g - grp0) * 32;
                const int left = g < grp0 ? cnt0 - g * 32 : cnt1 - (g - grp0) * 32;
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)col, v);
                if (pc.n1 == 0 && pc.nk > 1) {  // one block: the sums of the odd K slabs sit 256 columns further
                    uint32_t w[32];
                    tc_ld32(tmem_base + ((uint32_t)(lane_grp * 32) << 16) + 256u + (uint32_t)col, w);
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(w[i]));
                }
                if (f < N) {
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (i >= left) break;
                        const int t = tg + i;
                        const float a = __uint_as_float(v[i]);
                        if (splits > 1) {
                            plan.partial[((size_t)pc.split * M + t) * N + f] = a;
                        } else if (EPI == EPI_F32) {
                            *gemm_f32_dst(p, t, f) = a;
                        } else if (EPI == EPI_BF16) {
                            p.out[(size_t)t * p.ldo + f] = f2bf(a);
                        } else {
                            const uint32_t rr = r2[i >> 1];
                            p.out[(size_t)t * p.ldo + f] = f2bf(((i & 1) ? bfhi(rr) : bflo(rr)) + rbf(a));
                        }
                    }
                }
                load_res(g + kProducerWarps / 4);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_accum_empty);  // this warp's TMEM reads of the piece are done
        }
        if (!alive) {
            *abort_flag = 1;
            atomicExch(plan.err, 1);
        }
    } else if (warp == kTmaWarp) {
        if (lane == 0) {
            uint32_t par = 0, n_piece = 0;
            int prev_blocks = 0;
            bool alive = true;
            const uint32_t leader_full0 = map_to_cta(full(0), 0);
            // Launched with programmatic stream serialisation: everything up to here (barriers, TMEM, and the producers'
            // first weight slabs, which no earlier kernel writes) may overlap the tail of the kernel before; the
            // activations are that kernel's output.
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
            for (int blk = blk_begin; blk < blk_end && alive; n_piece++) {
                const Piece pc = piece_at(blk, blk_end, bpt, bs, M, KT, splits);
                blk += pc.blocks;
                const int NS = ring_stages(pc);
                const uint32_t SB = ring_stage_bytes(pc);
                if (prev_blocks != 0 && prev_blocks != pc.blocks) {
                    // the ring is carved differently for this piece: every MMA of the previous one must be done
                    if (!mbar_wait(accum_full, (n_piece - 1) & 1u)) {
                        alive = false;
                        break;
                    }
                }
                prev_blocks = pc.blocks;
                const int h0 = pc.n0 >> 1, h1 = pc.n1 >> 1;  // token rows this CTA holds per MMA instruction
                // one 128-row box, or one or two 32-row boxes when the CTA holds at most 64 rows
                const bool big0 = h0 > 2 * BOX_SMALL, big1 = h1 > 2 * BOX_SMALL;
                const int nb0 = big0 ? 1 : (h0 + BOX_SMALL - 1) / BOX_SMALL, nb1 = big1 ? 1 : (h1 + BOX_SMALL - 1) / BOX_SMALL;
                const uint32_t bb0 = (uint32_t)(big0 ? BOX_BIG : BOX_SMALL) * 128u, bb1 = (uint32_t)(big1 ? BOX_BIG : BOX_SMALL) * 128u;
                const CUtensorMap* m0 = big0 ? &map_x : &map_x_small;
                const CUtensorMap* m1 = big1 ? &map_x : &map_x_small;
                const int y0 = pc.t0 + (int)rank * h0, y1 = pc.t0 + bs + (int)rank * h1;
                const uint32_t tx = 2u * ((uint32_t)nb0 * bb0 + (uint32_t)nb1 * bb1 + (WK == 0 ? (uint32_t)A_BYTES : 0u));
                for (int kb = 0; kb < pc.nk; kb++) {
                    const int st = kb % NS;
                    const uint32_t ph = ((par >> st) ^ (uint32_t)(kb / NS)) & 1u;
                    if (!mbar_wait(empty(st), ph ^ 1u)) {
                        alive = false;
                        break;
                    }
                    const uint32_t sA = base + st * SB, sB = sA + A_BYTES;
                    const uint32_t fb = leader_full0 + 8u * st;
                    if (leader) mbar_expect_tx(full(st), tx);
                    const int kx = (pc.k0 + kb) * TK;
                    for (int b = 0; b < nb0; b++) tma_load_2d_pair(sB + b * bb0, m0, kx, y0 + b * BOX_SMALL, fb);
                    for (int b = 0; b < nb1; b++) tma_load_2d_pair(sB + UNIT_BYTES + b * bb1, m1, kx, y1 + b * BOX_SMALL, fb);
                    if (WK == 0) tma_load_2d_pair(sA, &map_w, kx, pc.fp * PAIR_F + (int)rank * TM, fb);
                }
                par = ring_advance(par, pc.nk, NS);
            }
            if (!alive) {
                *abort_flag = 1;
                atomicExch(plan.err, 1);
            }
        }
        __syncwarp();
    } else {
        // ---------------- MMA issuers (leader CTA) ----------------
        // Issuing an MMA occupies its thread (~90 cycles, ~170 when it accumulates into the previous MMA's columns), and
        // with the barrier round trips around each slab one thread cannot keep the tensor pipe fed when a slab carries
        // only four MMAs.  So a one-block piece is shared: issuer 0 takes the even K slabs and accumulates in TMEM
        // columns 0-255, issuer 1 the odd slabs in columns 256-511, and the epilogue adds the two.  A two-block piece
        // (eight MMAs per slab, alternating between its two accumulators) stays with issuer 0; issuer 1 only keeps the
        // ring's phases and gives its arrival on accum_full.
        const int issuer = warp - kMmaWarp;
        if (leader && lane == 0) {
            uint32_t par = 0, n_piece = 0;
            bool alive = true;
            for (int blk = blk_begin; blk < blk_end && alive; n_piece++) {
                const Piece pc = piece_at(blk, blk_end, bpt, bs, M, KT, splits);
                blk += pc.blocks;
                const int NS = ring_stages(pc);
                const uint32_t SB = ring_stage_bytes(pc);
                if (n_piece > 0) {
                    // both CTAs' epilogue warps have drained the previous accumulator (this also keeps issuer 1 from
                    // running a piece ahead and arriving twice in one phase of accum_full)
                    if (!mbar_wait(accum_empty, (n_piece - 1) & 1u)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                }
                const uint32_t id0 = umma_idesc(pc.n0), id1 = umma_idesc(pc.n1 > 0 ? pc.n1 : 16);
                const bool two = pc.n1 > 0;
                // descriptors advance by whole stages (SB >> 4) and by 32 bytes (2) per K=16 step; the stage
                // index and its phase are carried, not recomputed, to keep this thread's instruction count low
                const uint64_t dA0 = umma_desc(base), dB0 = umma_desc(base + A_BYTES), dB1 = umma_desc(base + A_BYTES + UNIT_BYTES);
                const uint64_t dstep = (uint64_t)(SB >> 4);
                if (two) {
                    if (issuer == 0) {
                        int st = 0;
                        uint32_t flip = 0;  // toggles each time the stage index wraps
                        uint64_t dA = dA0, dB = dB0, dC = dB1;
                        for (int kb = 0; kb < pc.nk; kb++) {
                            const uint32_t ph = ((par >> st) ^ flip) & 1u;
                            if (!mbar_wait(full(st), ph)) {
                                alive = false;
                                break;
                            }
                            tc_fence_after();
#pragma unroll
                            for (int k = 0; k < TK / 16; k++) {
                                const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                                tc_mma_pair(tmem_base, dA + 2 * k, dB + 2 * k, id0, acc);
                                tc_mma_pair(tmem_base + 256u, dA + 2 * k, dC + 2 * k, id1, acc);
                            }
                            tc_commit_pair(empty(st));
                            st++;
                            dA += dstep, dB += dstep, dC += dstep;
                            if (st == NS) st = 0, flip ^= 1u, dA = dA0, dB = dB0, dC = dB1;
                        }
                    }
                } else {
                    // slabs issuer, issuer + 2, ...: stage (kb mod NS), phase flipped once per turn of the ring
                    const uint32_t td = tmem_base + (uint32_t)issuer * 256u;
                    int st = issuer % NS;
                    uint32_t flip = 0;
                    for (int kb = issuer; kb < pc.nk; kb += 2) {
                        const uint32_t ph = ((par >> st) ^ flip) & 1u;
                        if (!mbar_wait(full(st), ph)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after();
                        const uint64_t dA = dA0 + (uint64_t)st * dstep, dB = dB0 + (uint64_t)st * dstep;
#pragma unroll
                        for (int k = 0; k < TK / 16; k++) tc_mma_pair(td, dA + 2 * k, dB + 2 * k, id0, (kb > issuer || k > 0) ? 1u : 0u);
                        tc_commit_pair(empty(st));
                        st += 2;
                        if (st >= NS) st -= NS, flip ^= 1u;
                    }
                }
                par = ring_advance(par, pc.nk, NS);
                if (alive) tc_commit_pair(accum_full);
            }
            if (!alive) {
                *abort_flag = 1;
                atomicExch(plan.err, 1);
            }
        }
        __syncwarp();
    }

    // common exit: nobody leaves while the peer may still signal this CTA's barriers or read its operands
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TN_MAX) : "memory");
    }
}

// out = epilogue(sum over K ranges of partial)
// four features per thread (N, the output / residual strides and their base addresses allow 16- and 8-byte accesses)
template <int EPI>
__global__ void splitk_reduce4_kernel(const GemmParams p, const float* __restrict__ partial, int splits) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    pdl_wait();  // (launched with programmatic stream serialisation behind the kernel that writes the partial sums)
    const size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)p.M * p.N;
    const size_t i = q * 4;
    if (i >= total) return;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int z = 0; z < splits; z++) {  // same additions in the same order as the one-feature kernel
        const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + (size_t)z * total + i));
        a.x += v.x, a.y += v.y, a.z += v.z, a.w += v.w;
    }
    const int t = (int)(i / p.N), f = (int)(i % p.N);
    if (EPI == EPI_F32) {
        *reinterpret_cast<float4*>(gemm_f32_dst(p, t, f)) = a;
    } else if (EPI == EPI_BF16) {
        uint2 o;
        o.x = pack_bf2(a.x, a.y);
        o.y = pack_bf2(a.z, a.w);
        *reinterpret_cast<uint2*>(p.out + (size_t)t * p.ldo + f) = o;
    } else {
        const uint2 r = *reinterpret_cast<const uint2*>(p.res + (size_t)t * p.ldres + f);
        uint2 o;
        o.x = pack_bf2(bflo(r.x) + rbf(a.x), bfhi(r.x) + rbf(a.y));
        o.y = pack_bf2(bflo(r.y) + rbf(a.z), bfhi(r.y) + rbf(a.w));
        *reinterpret_cast<uint2*>(p.out + (size_t)t * p.ldo + f) = o;
    }
}

template <int EPI>
__global__ void splitk_reduce_kernel(const GemmParams p, const float* __restrict__ partial, int splits) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)p.M * p.N;
    if (i >= total) return;
    float a = 0.f;
    for (int z = 0; z < splits; z++) a += partial[(size_t)z * total + i];
    const int t = (int)(i / p.N), f = (int)(i % p.N);
    if (EPI == EPI_F32)
        *gemm_f32_dst(p, t, f) = a;
    else if (EPI == EPI_BF16)
        p.out[(size_t)t * p.ldo + f] = f2bf(a);
    else
        p.out[(size_t)t * p.ldo + f] = f2bf(bf2f(p.res[(size_t)t * p.ldres + f]) + rbf(a));
}

// ---- TMA tensor maps (encoded on the host through the driver entry point; cached) -------------------
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
    uint64_t rows, k, ld, box_rows;
    int device;
    CUtensorMap map;
};
// bf16 matrix [rows, k] with row stride ld elements; box = 64 (k) x box_rows, 128-byte swizzle, zero fill
int32_t get_map(b2_ctx* ctx, const void* ptr, uint64_t rows, uint64_t k, uint64_t ld, uint32_t box_rows, const CUtensorMap** out) {
    static thread_local std::vector<MapEntry> cache;
    for (auto& e : cache)
        if (e.ptr == ptr && e.rows == rows && e.k == k && e.ld == ld && e.box_rows == box_rows && e.device == ctx->device) {
            *out = &e.map;
            return B2_OK;
        }
    EncodeTiledFn fn = encode_fn();
    B2_REQUIRE(fn != nullptr, B2_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    B2_REQUIRE(((uintptr_t)ptr & 15) == 0 && (ld * 2) % 16 == 0, B2_ERR_UNSUPPORTED, "tcgen05 gemm: operand must be 16-byte aligned");
    if (cache.size() >= 256) cache.clear();
    MapEntry e{ptr, rows, k, ld, box_rows, ctx->device, {}};
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    B2_REQUIRE(r == CUDA_SUCCESS, B2_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    cache.push_back(e);
    *out = &cache.back().map;
    return B2_OK;
}

__global__ void sbt_build_kernel(const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases, int N, int G, uint32_t* __restrict__ sbt) {
    // 32 x 32 tiles through shared memory: coalesced reads along the groups of a row, coalesced writes along the rows
    __shared__ uint32_t tile[32][33];
    const int g0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int n = n0 + r, g = g0 + threadIdx.x;
        if (n < N && g < G) tile[r][threadIdx.x] = (uint32_t)scales[(size_t)n * G + g] | ((uint32_t)biases[(size_t)n * G + g] << 16);
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int g = g0 + r, n = n0 + threadIdx.x;
        if (n < N && g < G) sbt[(size_t)g * N + n] = tile[threadIdx.x][r];
    }
}

template <int WK, int EPI>
int32_t launch_pair(b2_ctx* ctx, const GemmParams& p, int* err) {
    B2_SMEM_ONCE(ctx, (gemm_tc_pair_kernel<WK, EPI>), SMEM_BYTES);
    PairPlan plan{};
    plan.block_tokens = 256;
    plan.blocks_per_tile = (p.M + plan.block_tokens - 1) / plan.block_tokens;
    plan.total_blocks = ((p.N + PAIR_F - 1) / PAIR_F) * plan.blocks_per_tile;
    const int max_pairs = ctx->sm_count / 2;
    // Split K only when the blocks cannot occupy the pairs (down_proj at a few hundred tokens).  Cost model in K
    // slabs, fitted to measurements: a piece costs its slabs plus about 16 (prologue, first fill, epilogue), the
    // reduction pass about 20.
    const int KT = p.K / TK;
    int best = 1;
    if (plan.total_blocks * 10 <= max_pairs * 7) {
        long best_cost = (long)((plan.total_blocks + max_pairs - 1) / max_pairs) * (KT + 16);
        for (int sp = 2; sp <= 4 && sp * 16 <= KT; sp++) {
            const int units = plan.total_blocks * sp;
            const long cost = (long)((units + max_pairs - 1) / max_pairs) * (KT / sp + 16) + 20;
            if (cost < best_cost) best_cost = cost, best = sp;
        }
    }
    plan.splits = best;
    plan.partial = nullptr;
    if (best > 1) {
        const size_t bytes = (size_t)best * p.M * p.N * sizeof(float);
        if (bytes > ctx->tc_partial_bytes) {
            B2_CUDA(cudaStreamSynchronize(ctx->stream));
            if (ctx->tc_partial) B2_CUDA(cudaFree(ctx->tc_partial));
            ctx->tc_partial = nullptr;
            B2_CUDA(cudaMalloc((void**)&ctx->tc_partial, bytes + (bytes >> 2)));
            ctx->tc_partial_bytes = bytes + (bytes >> 2);
        }
        plan.partial = ctx->tc_partial;
    }
    const int units = plan.total_blocks * best;
    plan.n_pairs = units < max_pairs ? units : max_pairs;
    plan.err = err;
    const CUtensorMap *mx = nullptr, *ms = nullptr, *mw = nullptr;
    const uint64_t x_rows = p.x_rows_cap > p.M ? (uint64_t)p.x_rows_cap : (uint64_t)p.M;
    B2_CHECK(get_map(ctx, p.x, x_rows, (uint64_t)p.K, (uint64_t)p.ldx, BOX_BIG, &mx));
    CUtensorMap map_x = *mx;  // copied before the next lookup may move the cache
    B2_CHECK(get_map(ctx, p.x, x_rows, (uint64_t)p.K, (uint64_t)p.ldx, BOX_SMALL, &ms));
    CUtensorMap map_s = *ms, map_w = *ms;
    if (WK == 0) {
        B2_CHECK(get_map(ctx, p.w, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, TM, &mw));
        map_w = *mw;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * plan.n_pairs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // with split K the pair kernel only writes partial sums: the residual variant's extra registers buy nothing there
    if (best > 1 && EPI == EPI_BF16_RESADD) {
        B2_SMEM_ONCE(ctx, (gemm_tc_pair_kernel<WK, EPI_BF16>), SMEM_BYTES);
        B2_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<WK, EPI_BF16>, p, plan, map_x, map_s, map_w));
    } else {
        B2_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<WK, EPI>, p, plan, map_x, map_s, map_w));
    }
    B2_LAUNCHED(ctx);
    if (best > 1) {
        const size_t total = (size_t)p.M * p.N;
        const bool vec4 = p.N % 4 == 0 && p.ldo % 4 == 0 && (EPI != EPI_BF16_RESADD || (p.ldres % 4 == 0 && ((uintptr_t)p.res & 7) == 0)) &&
                          (EPI == EPI_F32 ? (((uintptr_t)p.out_f32 & 15) == 0 && p.f32_chunk % 4 == 0) : ((uintptr_t)p.out & 7) == 0);
        if (vec4)
            B2_CUDA(b2_launch_pdl(ctx->pdl_consumers, splitk_reduce4_kernel<EPI>, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, ctx->stream, p,
                                  (const float*)plan.partial, best));
        else
            splitk_reduce_kernel<EPI><<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(p, plan.partial, best);
        B2_LAUNCHED(ctx);
    }
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

template <int WK>
int32_t dispatch_pair(b2_ctx* ctx, const GemmParams& p, int* err) {
    switch (p.epilogue) {
        case EPI_BF16: return launch_pair<WK, EPI_BF16>(ctx, p, err);
        case EPI_BF16_RESADD: return launch_pair<WK, EPI_BF16_RESADD>(ctx, p, err);
        case EPI_F32: return launch_pair<WK, EPI_F32>(ctx, p, err);
    }
    return b2_fail(B2_ERR_MSG, "gemm: bad epilogue");
}

}  // namespace

int32_t b2_gemm_build_sbt(b2_ctx* ctx, const uint16_t* scales_dev, const uint16_t* biases_dev, int N, int G, uint32_t* sbt_dev) {
    sbt_build_kernel<<<dim3((unsigned)((G + 31) / 32), (unsigned)((N + 31) / 32)), dim3(32, 8), 0, ctx->stream>>>(scales_dev, biases_dev, N, G, sbt_dev);
    B2_LAUNCHED(ctx);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

bool b2_gemm_tc_eligible(const GemmParams& p) {
    return p.M > 32 && p.N % TM == 0 && p.K % TK == 0 && p.ldx % 8 == 0 && ((uintptr_t)p.x & 15) == 0 &&
           ((uintptr_t)p.w & (p.bits ? 31 : 15)) == 0 && (p.bits == 0 || p.bits == 4 || p.bits == 8);
}

int32_t b2_gemm_tc_launch(b2_ctx* ctx, const GemmParams& p) {
    if (!ctx->dev_err) {
        B2_CUDA(cudaMalloc((void**)&ctx->dev_err, 16));
        B2_CUDA(cudaMemsetAsync(ctx->dev_err, 0, 16, ctx->stream));
    }
    if (p.bits == 0) return dispatch_pair<0>(ctx, p, ctx->dev_err);
    if (p.bits == 4) return dispatch_pair<4>(ctx, p, ctx->dev_err);
    return dispatch_pair<8>(ctx, p, ctx->dev_err);
}
