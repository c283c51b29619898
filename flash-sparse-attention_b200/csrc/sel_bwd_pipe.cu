// Selected-attention backward, pipelined kernel for head_dim 128 and blocks of <= 64 keys
// (the shapes of the benchmark configurations); other shapes use the unpipelined kernel in
// sel_bwd.cu.  Same math and same outputs: per tile of <= 128 (head, token) rows of one KV block
//     S = Q K^T, dP = dO V^T | P = exp2(S c - lse), dS = scale P (dP - delta) | dQ = dS K,
//     dK^T += Q^T dS, dV^T += dO^T P
// Warp roles (768 threads in six warpgroups whose register budgets are rebalanced with setmaxnreg; one CTA per SM,
// persistent over a round-robin run schedule):
//   warps 0..7   gather Q and dO rows with 16-byte async copies (two stages);
//   warp 8       issues S and dP (tcgen05, fp32 in TMEM, two buffers);
//   warp 9       issues dQ, dK^T, dV^T;
//   warp 10      prepares, up to four tiles ahead, the token of every tile row (the gather warps then run without
//                any global load of their own: a plain load issued behind a burst of async copies waits for it);
//   warp 11      loads the K/V block of every run of tiles by TMA;
//   warps 12..15 the accumulator drain, one row / one head-dim index per thread: for every tile the dQ partial from TMEM
//                through a swizzled staging area to global memory by TMA store (input dtype, tile order: the load/store
//                unit is left to the row gathers); at the end of a segment (the tiles of one block inside one
//                scheduling run) the finished dK^T / dV^T accumulators from TMEM to registers (freeing them for the next
//                segment at once) and on to the segment's own fp32 slab while the next segment computes; a second kernel
//                sums the slabs of a block in segment order, so dK and dV do not depend on the order in which CTAs
//                finish (no atomics);
//   warps 16..23 two groups, one row per thread, each on half of the 64 key columns of every tile: P / dS to swizzled smem
//                and nothing else -- they are the critical path of a tile (the exp2 and the dS arithmetic between two
//                MMA phases), so both groups shorten the same tile instead of alternating tiles.
#include "sel_launch.cuh"

namespace fsa {

template <typename ET>
struct SelBwdPipeParams {
    const ET* q;   int64_t q_sn, q_sh;
    const ET* d_o; int64_t do_sn, do_sh;
    const float* lse;
    const float* delta;
    SelShape s;
    SelIndex ix;
    float scale, scale_log2;
    int run;
    SelBounds bd;      // visible K/V rows per token
    ET* dq_part;       // [max_tiles * 128, D] (written through dqmap)
    float* slabs;      // [segments][2 (dK, dV)][64 keys][D] fp32: the partial sums of every segment of tiles
    int no_dq;         // 1: dQ is computed elsewhere (range attention: the query-tile-major dQ kernel); only dK / dV here
};

namespace bwdpipe {
constexpr int D = 128, KT = 64;
constexpr int kKVStages = 1;                     // (a second K/V stage and the dQ staging area compete for the same 32 KB)
constexpr int kThreads = 768, kLoaders = 256;
constexpr int kWLoad = kLoaders / 32, kWMma1 = kWLoad, kWMma2 = kWLoad + 1, kWFlush = kWLoad + 4, kWGroups = kWLoad + 8;
// registers per thread of each role (multiples of 8); 32 * sum over warps <= 768 * 80 = the CTA's allocation
constexpr int kRegLoad = 40, kRegMma = 48, kRegFlush = 96, kRegGroup = 128;
static_assert(8 * kRegLoad + 4 * kRegMma + 4 * kRegFlush + 8 * kRegGroup <= 24 * 80, "register budget");
constexpr int kKV = 2 * KT * D * 2;              // K then V: 32 KB
constexpr int kQD = 2 * kTileRows * D * 2;       // Q then dO: 64 KB
constexpr int kPS = 2 * kTileRows * KT * 2;      // P then dS: 32 KB
constexpr int kDQ = kTileRows * D * 2;           // dQ staging: 32 KB, 8 KB per TMEM lane quarter
constexpr int kTail = 2560;
constexpr int kBytes = kKVStages * kKV + 2 * kQD + kPS + kDQ + kTail;
constexpr int cS = 0, cDP = 64;                  // + 128 * buffer
constexpr int cDQ = 256, cDK = 384, cDV = 448;
constexpr uint32_t kCols = 512;
static_assert(kBytes <= 227 * 1024, "smem budget");
}  // namespace bwdpipe

// Optional cycle accounting per role (debug builds only, -DFSA_TIMING): a table [gridDim.x][64] of accumulated
// clock64() deltas, read back with fsa_debug_read_bwd_timing.
#ifdef FSA_TIMING
__device__ unsigned long long g_bwd_timing[512 * 64];
#define BT_DECL unsigned long long _t0 = clock64(), _acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define BT_TOC(i) do { unsigned long long _t1 = clock64(); _acc[i] += _t1 - _t0; _t0 = _t1; } while (0)
#define BT_DUMP(base, n) do { for (int _i = 0; _i < (n); ++_i) g_bwd_timing[blockIdx.x * 64 + (base) + _i] = _acc[_i]; } while (0)
// Event trace of eight consecutive tiles of CTA 0 (absolute clock64() values), [tile][16 events].
__device__ unsigned long long g_bwd_trace[8 * 16];
constexpr int kTraceTile0 = 200;
#define BT_EV(k, ev, who) do { if (blockIdx.x == 0 && (k) >= kTraceTile0 && (k) < kTraceTile0 + 8 && (who)) \
        g_bwd_trace[((k) - kTraceTile0) * 16 + (ev)] = clock64(); } while (0)
#else
#define BT_DECL
#define BT_TOC(i)
#define BT_DUMP(base, n)
#define BT_EV(k, ev, who)
#endif

template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

__device__ __forceinline__ float ex2_approx_b(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename ET>
__global__ void __launch_bounds__(bwdpipe::kThreads, 1) sel_bwd_pipe(const SelBwdPipeParams<ET> p,
                                                                     const __grid_constant__ CUtensorMap kmap,
                                                                     const __grid_constant__ CUtensorMap vmap,
                                                                     const __grid_constant__ CUtensorMap dqmap) {
    using namespace bwdpipe;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sKV = smem;
    uint8_t* sQD = sKV + kKVStages * kKV;
    uint8_t* sP = sQD + 2 * kQD;
    uint8_t* sDS = sP + kTileRows * KT * 2;
    uint8_t* sDQ = sP + kPS;
    uint8_t* tail = sDQ + kDQ;
    int (*s_tok)[kTileRows] = reinterpret_cast<int (*)[kTileRows]>(tail);                // [4][128] token of every tile row, -1 padding
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 2048);
    uint64_t* qd_full = bars;            // [2]
    uint64_t* qd_empty = bars + 2;       // [2]
    uint64_t* kv_full = bars + 4;        // [2]
    uint64_t* kv_empty = bars + 6;       // [2]
    uint64_t* sdp_full = bars + 10;      // [2]
    uint64_t* sdp_empty = bars + 12;     // [2]
    uint64_t* pds_full = bars + 14;
    uint64_t* pds_empty = bars + 15;
    uint64_t* dq_full = bars + 16;
    uint64_t* dq_empty = bars + 17;
    uint64_t* acc_full = bars + 18;
    uint64_t* acc_empty = bars + 19;
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 20);
    uint64_t* off_full = bars + 26;      // [4] ring of prepared tiles: tokens, kv head and new-block flag are valid
    uint64_t* off_empty = bars + 30;     // [4] ... have been read by the eight gather warps and the S/dP issuer
    int* s_h = reinterpret_cast<int*>(bars + 34);    // [4] kv head of the prepared tile
    int* s_nb = s_h + 4;                             // [4] 1: the tile starts a new K/V block

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const SelShape& s = p.s;
    int* status = p.ix.header;
    if (smem_u32(smem) & 1023u) {
        if (tid == 0) atomicMax(status, (int)kStatusBadIndex);
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&qd_full[i], kLoaders); mbar_init(&qd_empty[i], 1);
            mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1);
            mbar_init(&sdp_full[i], 1); mbar_init(&sdp_empty[i], 256);
        }
        mbar_init(pds_full, 256); mbar_init(pds_empty, 1);
        mbar_init(dq_full, 1); mbar_init(dq_empty, 128);
        mbar_init(acc_full, 1); mbar_init(acc_empty, 128);
        for (int i = 0; i < 4; ++i) { mbar_init(&off_full[i], 1); mbar_init(&off_empty[i], kWLoad + 1); }
        mbar_init_fence();
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        tma_prefetch_desc(&dqmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const TileSchedule sched(p.ix.header[1], p.run);
    const int nloc = sched.nloc;
    const int key_lim = min(KT, s.BK);

    if (warp < kWLoad) {
        // ------------------------------------------------------------------ gather warps
        // Thread t copies 16-byte chunk t % 16 of the rows t / 16 + 16 i (a half-warp covers one 256-byte row) of Q and
        // dO.  Tokens come from the prepared ring; the head part of every row offset is a thread constant.
        reg_dec<kRegLoad>();
        const int t = tid;
        bool ok = true;
        constexpr int CPR = D / 8, RSTEP = kLoaders / CPR, NIT = kTileRows / RSTEP;   // 16 chunks per row, 8 rows per thread
        const int cchunk = t % CPR, rbase = t / CPR;
        const uint32_t slab_off = (uint32_t)(cchunk >> 3) * (kTileRows * 128);
        int gq[NIT], gd[NIT];                   // (head-in-group * head stride) / 8 of this thread's rows
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
            const int g = (rbase + it * RSTEP) / s.TPT;
            gq[it] = (int)((g * p.q_sh) >> 3);
            gd[it] = (int)((g * p.do_sh) >> 3);
        }
        const int qsn8 = (int)(p.q_sn >> 3), dsn8 = (int)(p.do_sn >> 3);
        const ET* qc = p.q + cchunk * 8;
        const ET* dc = p.d_o + cchunk * 8;
        BT_DECL;
        for (int k = 0; k < nloc && ok; ++k) {
            const int st = k & 1, slot = k & 3;
            BT_TOC(0);
            ok = mbar_wait(&off_full[slot], (k >> 2) & 1, status) && ok;
            BT_TOC(2);
            const int hq0 = (int)(((long long)s_h[slot] * s.G * p.q_sh) >> 3), hd0 = (int)(((long long)s_h[slot] * s.G * p.do_sh) >> 3);
            int tok[NIT];
#pragma unroll
            for (int it = 0; it < NIT; ++it) tok[it] = s_tok[slot][rbase + it * RSTEP];
            __syncwarp();
            if (lane == 0) mbar_arrive(&off_empty[slot]);
            BT_TOC(3);
            ok = mbar_wait(&qd_empty[st], ((k >> 1) & 1) ^ 1, status) && ok;
            BT_EV(k, 0, t == 0);
            BT_TOC(1);
            const uint32_t dq_ = smem_u32(sQD + st * kQD) + slab_off;
            const uint32_t dd_ = dq_ + kTileRows * D * 2;
#pragma unroll
            for (int it = 0; it < NIT; ++it) {
                const int r = rbase + it * RSTEP;
                const bool valid = tok[it] >= 0;
                const int tk = valid ? tok[it] : 0;
                const uint32_t so = sw128_chunk_off(r, cchunk & 7);
                cp_async16(dq_ + so, qc + ((long long)(tk * qsn8 + hq0 + gq[it]) << 3), valid);
                cp_async16(dd_ + so, dc + ((long long)(tk * dsn8 + hd0 + gd[it]) << 3), valid);
            }
            cp_async_mbar_arrive_noinc(&qd_full[st]);
            BT_EV(k, 1, t == 0);
            BT_TOC(4);
        }
        if (t == 0) BT_DUMP(0, 5);
    } else if (warp >= kWFlush && warp < kWFlush + 4) {
        // ------------------------------------------------------------------ accumulator drain: dQ per tile, dK / dV per segment
        // Walks the CTA's tiles in order.  Per tile: wait for its dQ product, move it TMEM -> registers -> swizzled staging
        // (this warp's 32 rows) -> TMA store.  At the last tile of a segment: wait for the segment's last products, pull
        // dK^T / dV^T (lane = head-dim index, columns = keys) into registers, release the TMEM accumulators, store them to
        // the segment's slab.
        reg_inc<kRegFlush>();
        const int quarter = warp & 3;
        const int d_idx = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        uint8_t* my_stage = sDQ + quarter * (32 * 256);
        bool ok = true;
        int nflush = 0;
        BT_DECL;
        // key ids of the CTA's tiles, fetched two tiles ahead
        int hg0 = -1, hg1 = -1, hg2 = -1;
        if (nloc > 0) hg1 = load_tile(p.ix, sched.tile(0)).hg;
        if (nloc > 1) hg2 = load_tile(p.ix, sched.tile(1)).hg;
        int seg_first = 0;                 // local index of the first tile of the running segment
        for (int k = 0; k < nloc && ok; ++k) {
            const int prev_hg = hg0;
            hg0 = hg1; hg1 = hg2;
            if (k + 2 < nloc) hg2 = load_tile(p.ix, sched.tile(k + 2)).hg;
            if (hg0 != prev_hg || (k % sched.run) == 0) seg_first = k;
            const bool last_of_seg = (k + 1 >= nloc) || (hg1 != hg0) || ((k + 1) % sched.run) == 0;
            const int j = sched.tile(k);
            // ---- dQ partial of this tile
            BT_TOC(0);
            if (!p.no_dq) {
            ok = mbar_wait(dq_full, k & 1, status) && ok;
            BT_EV(k, 13, warp == kWFlush && lane == 0);
            BT_TOC(1);
            tc_fence_after();
            if (lane == 0) bulk_wait_read0();          // the store of the previous tile has read this warp's staging rows
            __syncwarp();
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tbase + lane_off + cDQ + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 u;
                    u.x = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
                    u.y = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
                    u.z = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
                    u.w = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
                    const int chunk = (c0 >> 3) + q4;
                    *reinterpret_cast<uint4*>(my_stage + (chunk >> 3) * (32 * 128) + sw128_chunk_off(lane, chunk & 7)) = u;
                }
            }
            tc_fence_before();
            mbar_arrive(dq_empty);
            BT_EV(k, 14, warp == kWFlush && lane == 0);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int b = 0; b < D / 64; ++b)
                    tma_store_2d(&dqmap, b * 64, j * kTileRows + quarter * 32, smem_u32(my_stage + b * (32 * 128)));
                bulk_commit();
            }
            }
            BT_TOC(2);
            if (!last_of_seg) continue;
            // ---- dK^T / dV^T of the finished segment
            const int j0 = sched.tile(seg_first);
            const TileInfo ti = load_tile(p.ix, j0);
            // segments of a key are numbered by the scheduling run they fall into
            const int seg = ti.seg0 + j0 / sched.run - __ldg(p.ix.tile_aux + j0).x / sched.run;
            float* slab = p.slabs + (int64_t)seg * (2 * KT * D) + d_idx;
            ok = mbar_wait(acc_full, nflush & 1, status) && ok;
            BT_TOC(3);
            tc_fence_after();
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                uint32_t v[KT];
#pragma unroll
                for (int c0 = 0; c0 < KT; c0 += 32)
                    tmem_ld32(tbase + lane_off + (which == 0 ? cDK : cDV) + c0, *reinterpret_cast<uint32_t (*)[32]>(&v[c0]));
                tmem_ld_wait();
                if (which == 1) {
                    // both accumulators are in registers now: the next segment may overwrite them
                    tc_fence_before();
                    mbar_arrive(acc_empty);
                    ++nflush;
                }
                float* dst = slab + which * (KT * D);
#pragma unroll
                for (int key = 0; key < KT; ++key) dst[key * D] = __uint_as_float(v[key]);
            }
            BT_TOC(4);
        }
        if (lane == 0) bulk_wait0();
        if (warp == kWFlush && lane == 0) BT_DUMP(8, 5);
    } else if (warp < kWFlush) {
      reg_dec<kRegMma>();
      if (warp == kWMma1) {
        // ------------------------------------------------------------------ MMA issuer 1: S and dP
        const bool leader = elect_one();
        constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, KT, false, false);
        constexpr uint32_t hi_1024 = umma_desc_hi(1024);
        const uint32_t qd_lo = umma_desc_lo(smem_u32(sQD), 16);
        const uint32_t kv_lo = umma_desc_lo(smem_u32(sKV), 16);
        int kvn = -1;
        bool ok = true;
        BT_DECL;
        for (int k = 0; k < nloc && ok; ++k) {
            const int st = k & 1;
            BT_TOC(0);
            ok = mbar_wait(&off_full[k & 3], (k >> 2) & 1, status) && ok;
            BT_TOC(1);
            const int new_block = s_nb[k & 3];
            __syncwarp();
            if (lane == 0) mbar_arrive(&off_empty[k & 3]);
            if (new_block != 0) {
                ++kvn;
                ok = mbar_wait(&kv_full[kvn % kKVStages], (kvn / kKVStages) & 1, status) && ok;
            }
            BT_TOC(2);
            ok = mbar_wait(&qd_full[st], (k >> 1) & 1, status) && ok;
            BT_EV(k, 2, lane == 0);
            BT_TOC(3);
            fence_async_smem();
            ok = mbar_wait(&sdp_empty[st], ((k >> 1) & 1) ^ 1, status) && ok;
            BT_EV(k, 3, lane == 0);
            BT_TOC(4);
            tc_fence_after();
            const uint32_t aq = qd_lo + (uint32_t)(st * (kQD >> 4));
            const uint32_t ad = aq + (uint32_t)((kTileRows * D * 2) >> 4);
            const uint32_t bk = kv_lo + (uint32_t)((kvn % kKVStages) * (kKV >> 4));
            const uint32_t bv = bk + (uint32_t)((KT * D * 2) >> 4);
            const uint32_t dS_ = tbase + cS + st * 128, dP_ = tbase + cDP + st * 128;
            if (leader) {
                constexpr int kSlabA = (kTileRows * 128) >> 4, kSlabB = (KT * 128) >> 4;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(dS_, umma_desc_pack(aq + (ks >> 2) * kSlabA + (ks & 3) * 2, hi_1024),
                            umma_desc_pack(bk + (ks >> 2) * kSlabB + (ks & 3) * 2, hi_1024), idesc_s, ks > 0);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    umma_ss(dP_, umma_desc_pack(ad + (ks >> 2) * kSlabA + (ks & 3) * 2, hi_1024),
                            umma_desc_pack(bv + (ks >> 2) * kSlabB + (ks & 3) * 2, hi_1024), idesc_s, ks > 0);
                umma_commit(&sdp_full[st]);
            }
            __syncwarp();
            BT_EV(k, 4, lane == 0);
            BT_TOC(5);
        }
        if (lane == 0) BT_DUMP(16, 6);
      } else if (warp == kWMma2) {
        // ------------------------------------------------------------------ MMA issuer 2: dQ, dK^T, dV^T
        const bool leader = elect_one();
        constexpr uint32_t idesc_dq = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);     // dS (K-major) x K (MN-major)
        constexpr uint32_t idesc_dk = umma_idesc(ElemTraits<ET>::kIsBF16, 128, KT, true, true);     // Q^T / dO^T x dS / P
        constexpr uint32_t hi_1024 = umma_desc_hi(1024);
        const uint32_t ds_k_lo = umma_desc_lo(smem_u32(sDS), 16);                       // dS as K-major A
        const uint32_t ds_mn_lo = umma_desc_lo(smem_u32(sDS), 8192);                    // dS as MN-major B (one slab)
        const uint32_t p_mn_lo = umma_desc_lo(smem_u32(sP), 8192);
        const uint32_t k_mn_lo = umma_desc_lo(smem_u32(sKV), KT * 128);                 // K as MN-major B: slabs KT*128 apart
        const uint32_t qd_mn_lo = umma_desc_lo(smem_u32(sQD), kTileRows * 128);         // Q / dO as MN-major A
        int kvn = -1, blk = -1;
        bool ok = true;
        int hg0 = -1, hg1 = -1, hg2 = -1;
        if (nloc > 0) hg1 = load_tile(p.ix, sched.tile(0)).hg;
        if (nloc > 1) hg2 = load_tile(p.ix, sched.tile(1)).hg;
        BT_DECL;
        for (int k = 0; k < nloc && ok; ++k) {
            const int st = k & 1;
            const int prev_hg = hg0;
            hg0 = hg1; hg1 = hg2;
            if (k + 2 < nloc) hg2 = load_tile(p.ix, sched.tile(k + 2)).hg;
            // a segment ends where the block changes or the scheduling run ends
            const bool first_of_block = hg0 != prev_hg || (k % sched.run) == 0;
            const bool last_of_block = (k + 1 >= nloc) || (hg1 != hg0) || ((k + 1) % sched.run) == 0;
            if (first_of_block) { ++kvn; ++blk; }
            BT_TOC(0);
            ok = mbar_wait(pds_full, k & 1, status) && ok;
            BT_EV(k, 9, lane == 0);
            BT_TOC(1);
            BT_TOC(2);
            ok = mbar_wait(&qd_full[st], (k >> 1) & 1, status) && ok;     // already complete: acquire only
            ok = mbar_wait(&kv_full[kvn % kKVStages], (kvn / kKVStages) & 1, status) && ok;
            BT_TOC(3);
            if (first_of_block && blk > 0) ok = mbar_wait(acc_empty, (blk - 1) & 1, status) && ok;
            BT_TOC(4);
            fence_async_smem();
            tc_fence_after();
            const uint32_t bk = k_mn_lo + (uint32_t)((kvn % kKVStages) * (kKV >> 4));
            const uint32_t aq = qd_mn_lo + (uint32_t)(st * (kQD >> 4));
            const uint32_t ad = aq + (uint32_t)((kTileRows * D * 2) >> 4);
            // dK^T / dV^T first: they are the last readers of the Q / dO stage, which goes back to the gather warps as
            // soon as they are done; dQ (which reads dS and K only) follows
            if (leader) {
#pragma unroll
                for (int ks = 0; ks < kTileRows / 16; ++ks) {
                    const uint32_t acc = (!first_of_block || ks > 0) ? 1u : 0u;
                    umma_ss(tbase + cDK, umma_desc_pack(aq + ks * (2048 >> 4), hi_1024),
                            umma_desc_pack(ds_mn_lo + ks * (2048 >> 4), hi_1024), idesc_dk, acc);
                    umma_ss(tbase + cDV, umma_desc_pack(ad + ks * (2048 >> 4), hi_1024),
                            umma_desc_pack(p_mn_lo + ks * (2048 >> 4), hi_1024), idesc_dk, acc);
                }
                umma_commit(&qd_empty[st]);
                if (last_of_block) umma_commit(acc_full);
            }
            __syncwarp();
            BT_EV(k, 10, lane == 0);
            if (!p.no_dq) {
                ok = mbar_wait(dq_empty, (k & 1) ^ 1, status) && ok;
                BT_EV(k, 11, lane == 0);
                tc_fence_after();
            }
            if (leader) {
                if (!p.no_dq) {
#pragma unroll
                    for (int ks = 0; ks < KT / 16; ++ks)
                        umma_ss(tbase + cDQ, umma_desc_pack(ds_k_lo + ks * 2, hi_1024), umma_desc_pack(bk + ks * (2048 >> 4), hi_1024),
                                idesc_dq, ks > 0);
                }
                umma_commit(pds_empty);
                if (!p.no_dq) umma_commit(dq_full);
                if (last_of_block) umma_commit(&kv_empty[kvn % kKVStages]);
            }
            __syncwarp();
            BT_EV(k, 12, lane == 0);
            BT_TOC(5);
        }
        if (lane == 0) BT_DUMP(24, 6);
      } else if (warp == kWMma2 + 1) {
        // ------------------------------------------------------------------ tile preparation (tokens of the rows)
        // lane l owns rows l, l + 32, l + 64, l + 96; records and entries are fetched three tiles ahead
        bool ok = true;
        int gg[4], ee[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            gg[i] = r / s.TPT;
            ee[i] = r - gg[i] * s.TPT;
        }
        struct Pre { int h, hg; uint32_t e[4]; };
        auto fetch = [&](int k, Pre& m) {
            const int j = sched.tile(k);
            const TileInfo ti = load_tile(p.ix, j);
            m.h = ti.h; m.hg = ti.hg;
#pragma unroll
            for (int i = 0; i < 4; ++i) m.e[i] = gg[i] < s.G ? __ldg(p.ix.entries + (int64_t)j * s.TPT + ee[i]) : 0xFFFFFFFFu;
        };
        Pre m1{0, -1, {0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu}}, m2 = m1, m3 = m1;
        if (nloc > 0) fetch(0, m1);
        if (nloc > 1) fetch(1, m2);
        if (nloc > 2) fetch(2, m3);
        int prev_hg = -1;
        for (int k = 0; k < nloc && ok; ++k) {
            const int slot = k & 3;
            const Pre cur = m1;
            m1 = m2; m2 = m3;
            if (k + 3 < nloc) fetch(k + 3, m3);
            ok = mbar_wait(&off_empty[slot], ((k >> 2) & 1) ^ 1, status) && ok;
#pragma unroll
            for (int i = 0; i < 4; ++i) s_tok[slot][lane + 32 * i] = cur.e[i] != 0xFFFFFFFFu ? (int)(cur.e[i] >> kSlotBits) : -1;
            if (lane == 0) {
                s_h[slot] = cur.h;
                s_nb[slot] = (cur.hg != prev_hg || (k % sched.run) == 0) ? 1 : 0;
            }
            prev_hg = cur.hg;
            __syncwarp();
            if (lane == 0) mbar_arrive(&off_full[slot]);
        }
      } else {
        // ------------------------------------------------------------------ K/V blocks by TMA
        bool ok = true;
        int kvn = -1, prev_hg = -1;
        TileInfo t1{0, 0, 0, -1, 0}, t2 = t1;
        if (nloc > 0) t1 = load_tile(p.ix, sched.tile(0));
        if (nloc > 1) t2 = load_tile(p.ix, sched.tile(1));
        for (int k = 0; k < nloc && ok; ++k) {
            const TileInfo cur = t1;
            t1 = t2;
            if (k + 2 < nloc) t2 = load_tile(p.ix, sched.tile(k + 2));
            if (cur.hg == prev_hg && (k % sched.run) != 0) continue;     // (every segment loads its K/V block)
            prev_hg = cur.hg;
            ++kvn;
            if (lane == 0) {
                const int ks = kvn % kKVStages;
                ok = mbar_wait(&kv_empty[ks], ((kvn / kKVStages) & 1) ^ 1, status) && ok;
                mbar_expect_tx(&kv_full[ks], (uint32_t)kKV);
                uint8_t* dK = sKV + ks * kKV;
                uint8_t* dV = dK + KT * D * 2;
#pragma unroll
                for (int b = 0; b < D / 64; ++b) {
                    tma_load_2d(smem_u32(dK + b * KT * 128), &kmap, cur.h * D + b * 64, cur.row0, &kv_full[ks]);
                    tma_load_2d(smem_u32(dV + b * KT * 128), &vmap, cur.h * D + b * 64, cur.row0, &kv_full[ks]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
      }
    } else {
        // ------------------------------------------------------------------ P / dS
        // Both groups work on every tile, each on its 32 of the 64 key columns: the P / dS step sits on the tile's
        // critical path (between the two MMA phases), so its latency counts, not only its throughput.
        reg_inc<kRegGroup>();
        const int sb = (warp - kWGroups) >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const int g = r / s.TPT;
        const int e = r - g * s.TPT;
        const bool row_exists = g < s.G;
        constexpr int HC = KT / 2;              // columns of this group
        const int cb = sb * HC;
        bool ok = true;
        // software pipeline over the tiles: entries two tiles ahead, lse / delta one ahead
        uint32_t entB = 0xFFFFFFFFu;            // entry of tile k + 2
        uint32_t entA = 0xFFFFFFFFu;            // entry of tile k + 1 (after rotation)
        int row0A = 0, row0B = 0, hA = 0, hB = 0;
        float lseA = 0.f, deltaA = 0.f;
        int cloA = 0, chiA = 0;
        auto fetch_ent = [&](int j, uint32_t& ent, int& row0, int& h) {
            TileInfo ti = load_tile(p.ix, j);
            row0 = ti.row0; h = ti.h;
            ent = 0xFFFFFFFFu;
            if (row_exists) ent = __ldg(p.ix.entries + (int64_t)j * s.TPT + e);
        };
        auto fetch_stats = [&](uint32_t ent, int h, int row0, float& lse_, float& delta_, int& c_lo, int& c_hi) {
            // padding rows: their Q and dO rows are zero, so they add nothing to dK / dV whatever P is, and their dQ
            // rows are never read: they count as fully visible with lse = delta = 0 (finite values everywhere)
            lse_ = 0.f; delta_ = 0.f; c_lo = 0; c_hi = key_lim;
            if (ent != 0xFFFFFFFFu) {
                const int tok_ = (int)(ent >> kSlotBits);
                const int64_t idx = (int64_t)(h * s.G + g) * s.N + tok_;
                lse_ = __ldg(p.lse + idx);
                delta_ = __ldg(p.delta + idx) * p.scale;
                visible_cols(p.bd, tok_, row0, key_lim, c_lo, c_hi);
            }
        };
        if (nloc > 0) {
            fetch_ent(sched.tile(0), entA, row0A, hA);
            fetch_stats(entA, hA, row0A, lseA, deltaA, cloA, chiA);
        }
        if (nloc > 1) fetch_ent(sched.tile(1), entB, row0B, hB);
        BT_DECL;
        for (int k = 0; k < nloc && ok; ++k) {
            const int st = k & 1;
            const float lse_r = lseA, delta_s = deltaA;
            const int c_lo = cloA, c_hi = chiA;
            // rotate the prefetch registers
            entA = entB; row0A = row0B; hA = hB;
            if (k + 1 < nloc) fetch_stats(entA, hA, row0A, lseA, deltaA, cloA, chiA);
            if (k + 2 < nloc) fetch_ent(sched.tile(k + 2), entB, row0B, hB);
            BT_TOC(0);
            ok = mbar_wait(&sdp_full[st], (k >> 1) & 1, status) && ok;
            BT_EV(k, 5, sb == 0 && quarter == 0 && lane == 0);
            BT_TOC(1);
            tc_fence_after();
            uint32_t pp[HC / 2], dd[HC / 2];
            // most tiles are fully visible to all their rows (only a token's own block is cut by causality)
            const bool all_visible = __all_sync(0xffffffffu, c_lo == 0 && c_hi == KT);
            {
                uint32_t sv[32], dv[32];
                tmem_ld32(tbase + lane_off + cS + st * 128 + cb, sv);
                tmem_ld32(tbase + lane_off + cDP + st * 128 + cb, dv);
                tmem_ld_wait();
                if (all_visible) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2_approx_b(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse_r));
                        const float p1 = ex2_approx_b(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -lse_r));
                        const float d0 = p0 * fmaf(__uint_as_float(dv[i]), p.scale, -delta_s);
                        const float d1 = p1 * fmaf(__uint_as_float(dv[i + 1]), p.scale, -delta_s);
                        pp[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
                        dd[i >> 1] = ElemTraits<ET>::pack2(d0, d1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = (cb + i >= c_lo && cb + i < c_hi) ? ex2_approx_b(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse_r)) : 0.f;
                        const float p1 = (cb + i + 1 >= c_lo && cb + i + 1 < c_hi) ? ex2_approx_b(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -lse_r)) : 0.f;
                        const float d0 = p0 * fmaf(__uint_as_float(dv[i]), p.scale, -delta_s);
                        const float d1 = p1 * fmaf(__uint_as_float(dv[i + 1]), p.scale, -delta_s);
                        pp[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
                        dd[i >> 1] = ElemTraits<ET>::pack2(d0, d1);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&sdp_empty[st]);
            BT_EV(k, 6, sb == 0 && quarter == 0 && lane == 0);
            BT_TOC(2);
            ok = mbar_wait(pds_empty, (k & 1) ^ 1, status) && ok;
            BT_EV(k, 7, sb == 0 && quarter == 0 && lane == 0);
            BT_TOC(3);
#pragma unroll
            for (int c4 = 0; c4 < HC / 8; ++c4) {
                const uint32_t off = sw128_chunk_off(r, sb * (HC / 8) + c4);
                *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[c4 * 4], pp[c4 * 4 + 1], pp[c4 * 4 + 2], pp[c4 * 4 + 3]);
                *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[c4 * 4], dd[c4 * 4 + 1], dd[c4 * 4 + 2], dd[c4 * 4 + 3]);
            }
            fence_async_smem();
            mbar_arrive(pds_full);
            BT_EV(k, 8, sb == 0 && quarter == 0 && lane == 0);
            BT_TOC(4);
            BT_TOC(6);
        }
        if (quarter == 0 && lane == 0) BT_DUMP(32 + sb * 8, 7);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, bwdpipe::kCols);
}

template <typename ET>
static cudaError_t launch_pipe(const SelBwdArgs& a, const SelShape& s, const SelIndex& ix, const CUtensorMap& kmap,
                               const CUtensorMap& vmap, const CUtensorMap& dqmap, int num_sms, bool no_dq, cudaStream_t stream) {
    SelBwdPipeParams<ET> p;
    p.q = (const ET*)a.q; p.q_sn = a.q_sn; p.q_sh = a.q_sh;
    p.d_o = (const ET*)a.d_o; p.do_sn = a.do_sn; p.do_sh = a.do_sh;
    p.lse = a.lse; p.delta = a.delta;
    p.s = s; p.ix = ix;
    p.scale = a.sm_scale; p.scale_log2 = a.sm_scale * 1.4426950408889634f;
    p.run = s.RB;                      // (long runs: few segments per block)
    p.bd = a.bd;
    p.dq_part = (ET*)a.dq_part; p.slabs = a.slabs;
    p.no_dq = no_dq ? 1 : 0;
    auto kern = sel_bwd_pipe<ET>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bwdpipe::kBytes);
    if (e != cudaSuccess) return e;
    prof_begin(2, stream);
    kern<<<num_sms, bwdpipe::kThreads, bwdpipe::kBytes, stream>>>(p, kmap, vmap, dqmap);
    prof_end(2, stream);
    return cudaGetLastError();
}

#ifdef FSA_TIMING
}  // namespace fsa
extern "C" int fsa_debug_read_bwd_timing(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, fsa::g_bwd_timing, (size_t)n * sizeof(unsigned long long));
}
extern "C" int fsa_debug_read_bwd_trace(unsigned long long* host) {
    return (int)cudaMemcpyFromSymbol(host, fsa::g_bwd_trace, sizeof(fsa::g_bwd_trace));
}
namespace fsa {
#endif

cudaError_t launch_sel_bwd_pipe(int dtype, const SelBwdArgs& a, const SelShape& s, const SelIndex& ix,
                                const CUtensorMap& kmap, const CUtensorMap& vmap, const CUtensorMap& dqmap, int num_sms,
                                bool no_dq, cudaStream_t stream) {
    return dtype == kBF16 ? launch_pipe<__nv_bfloat16>(a, s, ix, kmap, vmap, dqmap, num_sms, no_dq, stream)
                          : launch_pipe<__half>(a, s, ix, kmap, vmap, dqmap, num_sms, no_dq, stream);
}

}  // namespace fsa
