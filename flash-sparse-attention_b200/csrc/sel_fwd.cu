// Selected-attention forward for sm_100a.
//
// Main kernel (replaces forward_kernel_opt and the qk_kernel pre-pass of the reference,
// fsa/ops/FSA_topk_sparse_attention.py:285-566): KV blocks are the outer loop.  A persistent
// CTA owns a contiguous range of tiles; a tile is <= 128 rows = (query head of the group,
// selecting token).  Warp-specialised:
//   warps 0..3  gather the query rows by token id with 16-byte async copies into a ring of swizzled Q stages
//               (TMA gather4 was measured at ~70 cycles per 512-byte instruction: too slow);
//   warp 4      one elected thread issues tcgen05.mma S = Q K^T into one of two TMEM S buffers;
//   warp 5      one elected thread issues O = P V (P read from TMEM, V MN-major from smem) into one
//               of two TMEM O buffers; two issuing warps keep the two streams from blocking each other;
//   warps 6..13 two softmax groups, each owning every other tile: one thread per row, row
//               max / exp2 / row sum from TMEM, P written back to TMEM over S (16-bit), then the
//               epilogue: O / l rounded to the input dtype, staged in swizzled smem and written
//               with TMA tile stores (one per warp and 64-column slab);
//   warp 14     prepares the tokens of the tile rows up to four tiles ahead (the gather warps then issue
//               no global load of their own);
//   warp 15     loads the K/V blocks by tiled TMA (128-byte swizzle, double-buffered).
// Partial rows are stored in TILE ORDER (contiguous 128-row slabs); their (m, l) statistics go to
// ml[(query head, token, slot)] so that the merge reads a token's pairs as one line.  No atomics, no
// cross-block state.
//
// Reduce kernel (replaces reduce_kernel, :139-281): one warp per (token, head) looks up the
// <= T partial rows through the `pos` map and merges them:  M = max m_s,
// w_s = exp2(m_s - M),  o = sum w_s O_s / sum w_s l_s,  lse = M + log2 sum w_s l_s  (log2 units;
// O_s is the unnormalised partial, l_s its row sum).
#include <type_traits>

#include "sel_launch.cuh"
#include <cstdlib>

namespace fsa {

template <typename ET>
struct SelFwdParams {
    SelShape s;
    SelIndex ix;
    float scale_log2;        // softmax scale * log2(e)
    int run;                 // tiles per scheduling run (see TileSchedule)
    SelBounds bd;            // visible K/V rows per token
    int dbg;                 // debug builds only: bit 0 skip Q copies, bit 1 skip partial stores
    ET* opart;               // [max_tiles * 128, D]  unnormalised partial outputs, tile order
    float2* ml;              // [Hq, N, T] (fits in max_tiles * 128 pairs): row max in log2 units, row sum
};

__host__ __device__ constexpr uint32_t tmem_cols_pow2(int c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : c <= 256 ? 256 : 512; }

template <int D, int BK>
struct SelFwdCfg {
    static constexpr int kQ = kTileRows * D * 2;
    static constexpr int kKV = 2 * BK * D * 2;         // K then V
    static constexpr int kOS = kTileRows * D * 2;      // output staging per softmax warpgroup (input dtype)
    static constexpr int kTail = 2560;                 // barriers, TMEM slot, row-offset table
    static constexpr int kMax = 227 * 1024;
    static constexpr int NKV = (2 * kQ + 2 * kKV + 2 * kOS + kTail <= kMax) ? 2 : 1;    // K/V stages
    static constexpr int NQ = (3 * kQ + NKV * kKV + 2 * kOS + kTail <= kMax) ? 3 : 2;   // Q stages
    static constexpr int kBytes = NQ * kQ + NKV * kKV + 2 * kOS + kTail;
    static constexpr int NS = (4 * BK + 2 * D <= 512) ? 4 : 2;   // S buffers (BK columns each); two per softmax group when they fit
    static constexpr int cS = 0;
    static constexpr int cO = NS * BK;                 // two O buffers of D columns, one per softmax group
    static constexpr uint32_t kCols = tmem_cols_pow2(NS * BK + 2 * D);
};

// warps: 0..3 gather loaders | 4 issues S = Q K^T | 5 issues O = P V | 6..9 softmax group 0 | 10..13 softmax group 1
// (any four consecutive warps cover the four TMEM lane quarters, warp % 4) | 14 prepares the tokens of the tile rows up
// to four tiles ahead | 15 loads the K/V blocks by TMA.  The gather warps issue no global load of their own: a plain
// load issued behind a burst of async copies waits for the burst.
constexpr int kFwdThreads = 512;
constexpr int kFwdLoaders = 128;
constexpr int kFwdRing = 4;

// Optional cycle accounting per role (debug builds only): FSA_TIMING defines a global table
// [gridDim.x][32] of accumulated clock64() deltas.
#ifdef FSA_TIMING
__device__ unsigned long long g_fwd_timing[512 * 32];
#define T_DECL unsigned long long _t0 = 0, _acc[12] = {0,0,0,0,0,0,0,0,0,0,0,0}
#define T_TIC _t0 = clock64()
#define T_TOC(i) do { unsigned long long _t1 = clock64(); _acc[i] += _t1 - _t0; _t0 = _t1; } while (0)
#define T_DUMP(base, n) do { for (int _i = 0; _i < (n); ++_i) g_fwd_timing[blockIdx.x * 32 + (base) + _i] = _acc[_i]; } while (0)
#define TR(role, k, ev) do { if (blockIdx.x == 3 && (k) >= 64 && (k) < 96) g_fwd_trace[((role) * 32 + ((k) - 64)) * 4 + (ev)] = clock64(); } while (0)
__device__ long long g_fwd_trace[6 * 32 * 4];
#else
#define TR(role, k, ev)
#define T_DECL
#define T_TIC
#define T_TOC(i)
#define T_DUMP(base, n)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int BK, typename ET>
__global__ void __launch_bounds__(kFwdThreads, 1) sel_fwd_main(const SelFwdParams<ET> p, const ET* __restrict__ q, int64_t q_sn,
                                                               int64_t q_sh, const __grid_constant__ CUtensorMap kmap,
                                                               const __grid_constant__ CUtensorMap vmap,
                                                               const __grid_constant__ CUtensorMap omap) {
    using C = SelFwdCfg<D, BK>;
    static_assert(C::NS * BK + 2 * D <= 512, "TMEM budget");
    static_assert(C::kBytes <= 227 * 1024, "smem budget");
    // The kernel uses no static shared memory: the dynamic region starts 1024-byte aligned, which
    // the swizzled tiles need, and every byte of the 227 KB is budgeted (checked below).
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + C::NQ * C::kQ;
    uint8_t* sOS = sKV + C::NKV * C::kKV;
    uint8_t* tail = sOS + 2 * C::kOS;
    int (*s_tok)[kTileRows] = reinterpret_cast<int (*)[kTileRows]>(tail);   // [4][128] token of every tile row (-1: padding)
    uint64_t* bars = reinterpret_cast<uint64_t*>(tail + kFwdRing * kTileRows * 4);
    uint64_t* q_full = bars;                 // [NQ]
    uint64_t* q_empty = q_full + C::NQ;      // [NQ]
    uint64_t* kv_full = q_empty + C::NQ;     // [NKV]
    uint64_t* kv_empty = kv_full + C::NKV;   // [NKV]
    uint64_t* s_full = kv_empty + C::NKV;    // [NS]
    uint64_t* s_empty = s_full + C::NS;      // [NS]
    uint64_t* p_full = s_empty + C::NS;      // [NS]
    uint64_t* o_full = p_full + C::NS;       // [2]
    uint64_t* o_empty = o_full + 2;          // [2]
    uint64_t* off_full = o_empty + 2;        // [4] ring of prepared tiles: tokens, kv head, new-block flag are valid
    uint64_t* off_empty = off_full + kFwdRing;   // [4] ... have been read by the gather warps and the S issuer
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(off_empty + kFwdRing);
    int* s_h = reinterpret_cast<int*>(off_empty + kFwdRing) + 2;   // [4] kv head of the prepared tile
    int* s_nb = s_h + kFwdRing;                                    // [4] 1: the tile starts a new K/V block
    static_assert(kFwdRing * kTileRows * 4 + (2 * C::NQ + 2 * C::NKV + 3 * C::NS + 4 + 2 * kFwdRing) * 8 + 8 + 8 * kFwdRing <= C::kTail,
                  "tail budget");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const SelShape& s = p.s;
    int* status = p.ix.header;
    if (smem_u32(smem) & 1023u) {   // never expected; the tiles would be mis-swizzled
        if (tid == 0) atomicMax(status, (int)kStatusBadIndex);
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < C::NQ; ++i) { mbar_init(&q_full[i], kFwdLoaders); mbar_init(&q_empty[i], 1); }
        for (int i = 0; i < kFwdRing; ++i) { mbar_init(&off_full[i], 1); mbar_init(&off_empty[i], kFwdLoaders / 32 + 1); }
        for (int i = 0; i < C::NKV; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
        for (int i = 0; i < C::NS; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 1); mbar_init(&p_full[i], 128); }
        for (int i = 0; i < 2; ++i) { mbar_init(&o_full[i], 1); mbar_init(&o_empty[i], 128); }
        mbar_init_fence();
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        tma_prefetch_desc(&omap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, C::kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;

    const TileSchedule sched(p.ix.header[1], p.run);
    const int nloc = sched.nloc;

    if (warp < 4) {
        // ------------------------------------------------------------------ gather warps (128 threads)
        // Thread t copies 16-byte chunk (t % CPR) of the rows t / CPR, t / CPR + RSTEP, ... (a half-warp covers one
        // 256-byte row).  Tokens come from the prepared ring; the head part of a row offset is a thread constant.
        T_DECL;
        const int t = tid;
        bool ok = true;
        constexpr int CPR = D / 8;                         // 16-byte chunks per row
        constexpr int RSTEP = kFwdLoaders / CPR;           // rows advanced per iteration
        constexpr int NIT = kTileRows / RSTEP;
        const int cchunk = t % CPR, rbase = t / CPR;
        const uint32_t slab_off = (uint32_t)(cchunk >> 3) * (kTileRows * 128);
        int gq[NIT];                                       // (head-in-group * head stride) / 8 of this thread's rows
#pragma unroll
        for (int it = 0; it < NIT; ++it) gq[it] = (int)((((rbase + it * RSTEP) / s.TPT) * q_sh) >> 3);
        const int qsn8 = (int)(q_sn >> 3);
        const ET* qc = q + cchunk * 8;
        for (int k = 0; k < nloc && ok; ++k) {
            const int qs = k % C::NQ, slot = k % kFwdRing;
            T_TIC;
            // the Q stage is free once the S MMA of the tile that used it is done
            ok = mbar_wait(&q_empty[qs], ((k / C::NQ) & 1) ^ 1, status) && ok;
            T_TOC(1);
            if (t == 0) TR(0, k, 0);
            ok = mbar_wait(&off_full[slot], (k / kFwdRing) & 1, status) && ok;
            const int hq0 = (int)(((long long)s_h[slot] * s.G * q_sh) >> 3);
            int tok[NIT];
#pragma unroll
            for (int it = 0; it < NIT; ++it) tok[it] = s_tok[slot][rbase + it * RSTEP];
            __syncwarp();
            if (lane == 0) mbar_arrive(&off_empty[slot]);
            T_TOC(2);
            const uint32_t dstq = smem_u32(sQ + qs * C::kQ) + slab_off;
#ifdef FSA_TIMING
            if (!(p.dbg & 1))
#endif
            {
#pragma unroll
                for (int it = 0; it < NIT; ++it) {
                    const int r = rbase + it * RSTEP;
                    const bool valid = tok[it] >= 0;
                    const int tk = valid ? tok[it] : 0;
                    cp_async16(dstq + sw128_chunk_off(r, cchunk & 7), qc + ((long long)(tk * qsn8 + hq0 + gq[it]) << 3), valid);
                }
            }
            // arrives on q_full when this thread's copies have landed; nobody waits here, so the
            // loader never holds a finished tile back behind a later wait
            cp_async_mbar_arrive_noinc(&q_full[qs]);
            T_TOC(3);
            if (t == 0) TR(0, k, 1);
        }
        if (t == 0) T_DUMP(0, 5);
    } else if (warp == 14) {
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
            const int slot = k % kFwdRing;
            const Pre cur = m1;
            m1 = m2; m2 = m3;
            if (k + 3 < nloc) fetch(k + 3, m3);
            ok = mbar_wait(&off_empty[slot], ((k / kFwdRing) & 1) ^ 1, status) && ok;
#pragma unroll
            for (int i = 0; i < 4; ++i) s_tok[slot][lane + 32 * i] = cur.e[i] != 0xFFFFFFFFu ? (int)(cur.e[i] >> kSlotBits) : -1;
            if (lane == 0) {
                s_h[slot] = cur.h;
                s_nb[slot] = cur.hg != prev_hg ? 1 : 0;
            }
            prev_hg = cur.hg;
            __syncwarp();
            if (lane == 0) mbar_arrive(&off_full[slot]);
        }
    } else if (warp == 15) {
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
            if (cur.hg == prev_hg) continue;
            prev_hg = cur.hg;
            ++kvn;
            if (lane == 0) {
                const int ks = kvn % C::NKV;
                ok = mbar_wait(&kv_empty[ks], ((kvn / C::NKV) & 1) ^ 1, status) && ok;
                mbar_expect_tx(&kv_full[ks], (uint32_t)C::kKV);
                uint8_t* dK = sKV + ks * C::kKV;
                uint8_t* dV = dK + BK * D * 2;
#pragma unroll
                for (int b = 0; b < D / 64; ++b) {
                    tma_load_2d(smem_u32(dK + b * BK * 128), &kmap, cur.h * D + b * 64, cur.row0, &kv_full[ks]);
                    tma_load_2d(smem_u32(dV + b * BK * 128), &vmap, cur.h * D + b * 64, cur.row0, &kv_full[ks]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------------ MMA issuer 1: S = Q K^T
        // The whole warp walks the loop (uniform control flow); one elected lane issues.  S and P V
        // are issued by different warps so that neither waits behind the other's barriers.
        const bool leader = elect_one();
        constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, BK, false, false);
        // descriptor words: constant high word (SBO 1024, version, swizzle), low words of the bases
        constexpr uint32_t hi_1024 = umma_desc_hi(1024);
        const uint32_t q_lo = umma_desc_lo(smem_u32(sQ), 16);
        const uint32_t k_lo = umma_desc_lo(smem_u32(sKV), 16);
        int kvn = -1;
        bool ok = true;
        T_DECL;
        for (int k = 0; k < nloc && ok; ++k) {
            const int qs = k % C::NQ, sbuf = k % C::NS;
            T_TIC;
            // "does this tile start a new K/V block": published by the loader with the Q stage
            ok = mbar_wait(&off_full[k % kFwdRing], (k / kFwdRing) & 1, status) && ok;
            const int new_block = s_nb[k % kFwdRing];
            __syncwarp();
            if (lane == 0) mbar_arrive(&off_empty[k % kFwdRing]);
            if (new_block != 0) {
                ++kvn;
                ok = mbar_wait(&kv_full[kvn % C::NKV], (kvn / C::NKV) & 1, status) && ok;
            }
            T_TOC(1);
            if (lane == 0) TR(1, k, 0);
            ok = mbar_wait(&q_full[qs], (k / C::NQ) & 1, status) && ok;
            fence_async_smem();   // the Q rows were written by cp.async (generic proxy)
            T_TOC(2);
            if (lane == 0) TR(1, k, 1);
            ok = mbar_wait(&s_empty[sbuf], ((k / C::NS) & 1) ^ 1, status) && ok;
            T_TOC(3);
            if (lane == 0) TR(1, k, 2);
            tc_fence_after();
            const uint32_t a_lo = q_lo + (uint32_t)(qs * (C::kQ >> 4));
            const uint32_t b_lo = k_lo + (uint32_t)((kvn % C::NKV) * (C::kKV >> 4));
            const uint32_t d_s = tbase + C::cS + sbuf * BK;
            if (leader) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    // k-step ks: 64-column slab ks / 4, 32-byte step (ks % 4) inside the 128-byte swizzle row
                    constexpr int kSlabA = (kTileRows * 128) >> 4, kSlabB = (BK * 128) >> 4;
                    umma_ss(d_s, umma_desc_pack(a_lo + (ks >> 2) * kSlabA + (ks & 3) * 2, hi_1024),
                            umma_desc_pack(b_lo + (ks >> 2) * kSlabB + (ks & 3) * 2, hi_1024), idesc_s, ks > 0);
                }
                umma_commit(&q_empty[qs]);
                umma_commit(&s_full[sbuf]);
            }
            __syncwarp();
            T_TOC(4);
            if (lane == 0) TR(1, k, 3);
        }
        if (lane == 0) T_DUMP(8, 5);
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer 2: O = P V
        const bool leader = elect_one();
        constexpr uint32_t idesc_o = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);
        constexpr uint32_t hi_1024 = umma_desc_hi(1024);
        const uint32_t v_lo = umma_desc_lo(smem_u32(sKV + BK * D * 2), BK * 128);   // MN-major: LBO = slab stride
        int kvn = -1;
        bool ok = true;
        T_DECL;
        // block ids of the CTA's tiles, fetched two tiles ahead (needed to know when a K/V stage is done)
        int hg0 = -1, hg1 = -1, hg2 = -1;
        if (nloc > 0) hg1 = load_tile(p.ix, sched.tile(0)).hg;
        if (nloc > 1) hg2 = load_tile(p.ix, sched.tile(1)).hg;
        for (int k = 0; k < nloc && ok; ++k) {
            const int sb = k & 1, sbuf = k % C::NS;
            const int prev_hg = hg0;
            hg0 = hg1; hg1 = hg2;
            if (k + 2 < nloc) hg2 = load_tile(p.ix, sched.tile(k + 2)).hg;
            if (hg0 != prev_hg) ++kvn;
            const bool last_of_block = (k + 1 >= nloc) || (hg1 != hg0);
            const int kv_cur = kvn % C::NKV;
            T_TIC;
            ok = mbar_wait(&p_full[sbuf], (k / C::NS) & 1, status) && ok;
            T_TOC(5);
            if (lane == 0) TR(2, k, 0);
            ok = mbar_wait(&o_empty[sb], ((k >> 1) & 1) ^ 1, status) && ok;
            T_TOC(6);
            if (lane == 0) TR(2, k, 1);
            tc_fence_after();
            const uint32_t b_lo = v_lo + (uint32_t)(kv_cur * (C::kKV >> 4));
            const uint32_t d_o = tbase + C::cO + sb * D, a_p = tbase + C::cS + sbuf * BK;
            if (leader) {
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks)
                    umma_ts(d_o, a_p + ks * 8, umma_desc_pack(b_lo + ks * (2048 >> 4), hi_1024), idesc_o, ks > 0);
                umma_commit(&o_full[sb]);
                umma_commit(&s_empty[sbuf]);
                if (last_of_block) umma_commit(&kv_empty[kv_cur]);
            }
            __syncwarp();
            T_TOC(7);
            if (lane == 0) TR(2, k, 2);
        }
#ifdef FSA_TIMING
        if (lane == 0) for (int i = 5; i < 8; ++i) g_fwd_timing[blockIdx.x * 32 + 8 + i] = _acc[i];
#endif
    } else {
        // ------------------------------------------------------------------ softmax + epilogue
        // Group sb (warps 6..9 / 10..13) owns the CTA's tiles with odd / even local index, hence TMEM
        // buffers S[sb], O[sb] and its own staging area.  One row per thread.
        const int sb = (warp - 6) >> 2;
        const int quarter = warp & 3;                 // TMEM lane quarter this warp may access
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const int g = r / s.TPT;
        const int e = r - g * s.TPT;
        // this warp's 32 staged rows: D/64 slabs of 32 rows x 128 bytes, 128-byte swizzle
        uint8_t* my_os = sOS + sb * C::kOS + quarter * (32 * D * 2);
        // the (m, l) pairs of a (head, token) complete a 128-byte line over T tiles far apart in time: keep those lines in
        // L2; the partial rows are written once and read once by the merge: let them leave first
        const uint64_t pol_ml = l2_policy_evict_last(), pol_part = l2_policy_evict_first();
        const uint32_t tS0 = tbase + lane_off + C::cS;
        const uint32_t tO = tbase + lane_off + C::cO + sb * D;
        bool ok = true;
        T_DECL;
        // software pipeline over this group's tiles: the entry of this thread's row is fetched two
        // own tiles ahead, the visible-column bounds (which may need the token's row limits) one ahead
        const bool row_exists = g < s.G;
        uint32_t entA = 0xFFFFFFFFu, entB = 0xFFFFFFFFu;
        int row0A = 0, row0B = 0, cloA = 0, chiA = BK, hA = 0, hB = 0;
        // tile indices of this group's tiles k, k + 2, k + 4 without a division per tile: a cursor (run index, offset
        // in the run) that advances by two
        int cq = sb / sched.run, cr = sb % sched.run;
        auto cursor_next = [&]() {
            const int j = (cq * sched.grid + sched.cta) * sched.run + cr;
            cr += 2;
            while (cr >= sched.run) { cr -= sched.run; ++cq; }
            return j;
        };
        int jA = 0, jB = 0;
        auto fetch_ent = [&](int j, uint32_t& ent, int& row0, int& h) {
            const TileInfo ti = load_tile(p.ix, j);
            row0 = ti.row0; h = ti.h;
            ent = 0xFFFFFFFFu;
            if (row_exists) ent = __ldg(p.ix.entries + (int64_t)j * s.TPT + e);
        };
        // statistics go to ml[(head, token, slot)]: the merge kernel reads a token's T pairs as one contiguous line
        auto ml_index = [&](uint32_t ent, int h) {
            return ((int64_t)(h * s.G + g) * s.N + (int64_t)(ent >> kSlotBits)) * s.T + (int)(ent & ((1u << kSlotBits) - 1));
        };
        auto fetch_bounds = [&](uint32_t ent, int row0, int& c_lo, int& c_hi) {
            c_lo = 0; c_hi = BK;   // padding rows: anything finite
            if (ent != 0xFFFFFFFFu) visible_cols(p.bd, (int)(ent >> kSlotBits), row0, BK, c_lo, c_hi);
        };
        bool have_prev = false, prev_valid = false;
        int prev_j = 0, prev_u = 0;
        float prev_m = 0.f, prev_l = 0.f;
        int64_t prev_mli = 0;
        // O / l -> staging -> TMA store, for the tile (prev_j) whose softmax ran one iteration ago
        auto epilogue = [&]() {
            T_TIC;
            ok = mbar_wait(&o_full[sb], prev_u & 1, status) && ok;
            T_TOC(3);
            if (quarter == 2 && lane == 0) TR(3, prev_u * 2 + sb, 2);
            tc_fence_after();
            if (lane == 0) bulk_wait_read0();   // previous store of this warp has read its staging rows
            __syncwarp();
            T_TOC(4);
            // (two TMEM loads in flight per wait, 64 columns per round trip, measured 5 % slower than one)
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tO + c0, v);
                tmem_ld_wait();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    // unnormalised O (its row sum l travels in the statistics): rounding to a floating-point
                    // format is scale-free, so dividing first would not make the partial more accurate
                    uint4 x;
                    x.x = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
                    x.y = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
                    x.z = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
                    x.w = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
                    const int chunk = (c0 >> 3) + q4;     // 16-byte chunk of the row
                    *reinterpret_cast<uint4*>(my_os + (chunk >> 3) * (32 * 128) + sw128_chunk_off(lane, chunk & 7)) = x;
                }
            }
            tc_fence_before();
            mbar_arrive(&o_empty[sb]);
            if (prev_valid) st_float2_hint(p.ml + prev_mli, prev_m, prev_l, pol_ml);
            fence_async_smem();
            __syncwarp();
#ifdef FSA_TIMING
            if (!(p.dbg & 2))
#endif
            if (lane == 0) {
#pragma unroll
                for (int b = 0; b < D / 64; ++b)
                    tma_store_2d_hint(&omap, b * 64, prev_j * kTileRows + quarter * 32, smem_u32(my_os + b * (32 * 128)), pol_part);
                bulk_commit();
            }
            T_TOC(5);
            if (quarter == 2 && lane == 0) TR(3, prev_u * 2 + sb, 3);
        };
        if (sb < nloc) {
            jA = cursor_next();
            fetch_ent(jA, entA, row0A, hA);
            fetch_bounds(entA, row0A, cloA, chiA);
        }
        if (sb + 2 < nloc) {
            jB = cursor_next();
            fetch_ent(jB, entB, row0B, hB);
        }
        for (int k = sb; k < nloc && ok; k += 2) {
            const int j = jA;
            const int u = k >> 1;                     // use count of this group's O buffer
            const int sbuf = k % C::NS;
            const uint32_t tS = tS0 + sbuf * BK;
            const bool row_valid = entA != 0xFFFFFFFFu;
            const int c_lo = cloA, c_hi = chiA;            // visible key columns of this row
            const int64_t mli = row_valid ? ml_index(entA, hA) : 0;
            entA = entB; row0A = row0B; hA = hB; jA = jB;
            T_TIC;
            if (k + 2 < nloc) fetch_bounds(entA, row0A, cloA, chiA);
            if (k + 4 < nloc) {
                jB = cursor_next();
                fetch_ent(jB, entB, row0B, hB);
            }
            T_TOC(0);
            ok = mbar_wait(&s_full[sbuf], (k / C::NS) & 1, status) && ok;
            T_TOC(1);
            if (quarter == 2 && lane == 0) TR(3, k, 0);
            tc_fence_after();
            float m, l;
            if constexpr (BK <= 64) {
                // whole row in registers: one TMEM read
                uint32_t v[BK];
                {
                    uint32_t (&v0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[0]);
                    tmem_ld32(tS, v0);
                    if constexpr (BK == 64) {
                        uint32_t (&v1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&v[32]);
                        tmem_ld32(tS + 32, v1);
                    }
                    tmem_ld_wait();
                }
                if (c_lo > 0 || c_hi < BK) {
#pragma unroll
                    for (int i = 0; i < BK; ++i)
                        if (i < c_lo || i >= c_hi) v[i] = 0xff800000u;   // -inf: exp2 gives exactly 0
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < BK; i += 4) {
                    mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
                    mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
                    mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
                    mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
                }
                m = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
                float ls[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[BK / 2];
#pragma unroll
                for (int i = 0; i < BK; i += 4) {
                    float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), p.scale_log2, -m));
                    float p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m));
                    float p2 = ex2_approx(fmaf(__uint_as_float(v[i + 2]), p.scale_log2, -m));
                    float p3 = ex2_approx(fmaf(__uint_as_float(v[i + 3]), p.scale_log2, -m));
                    ls[0] += p0; ls[1] += p1; ls[2] += p2; ls[3] += p3;
                    pk[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
                    pk[(i >> 1) + 1] = ElemTraits<ET>::pack2(p2, p3);
                }
                l = (ls[0] + ls[1]) + (ls[2] + ls[3]);
                if constexpr (BK == 64) {
                    tmem_st32(tS, *reinterpret_cast<uint32_t (*)[32]>(&pk[0]));
                } else {
                    tmem_st16(tS, *reinterpret_cast<uint32_t (*)[16]>(&pk[0]));
                }
            } else {
                float mx = -INFINITY;
#pragma unroll
                for (int c0 = 0; c0 < BK; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tS + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c0 + i >= c_lo && c0 + i < c_hi) mx = fmaxf(mx, __uint_as_float(v[i]));
                }
                m = mx * p.scale_log2;
                l = 0.f;
#pragma unroll
                for (int c0 = 0; c0 < BK; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tS + c0, v);
                    tmem_ld_wait();
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float p0 = (c0 + i >= c_lo && c0 + i < c_hi) ? ex2_approx(fmaf(__uint_as_float(v[i]), p.scale_log2, -m)) : 0.f;
                        float p1 = (c0 + i + 1 >= c_lo && c0 + i + 1 < c_hi) ? ex2_approx(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m)) : 0.f;
                        l += p0 + p1;
                        pk[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
                    }
                    tmem_st16(tS + (c0 >> 1), pk);
                }
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&p_full[sbuf]);
            T_TOC(2);
            if (quarter == 2 && lane == 0) TR(3, k, 1);

            // the epilogue of this group's previous tile runs now: its P V has had a whole softmax
            // to finish, so the wait below is normally free
            if (have_prev) epilogue();
            have_prev = true;
            prev_j = j; prev_u = u; prev_m = m; prev_l = l; prev_valid = row_valid; prev_mli = mli;
        }
        if (have_prev && ok) epilogue();
        if (lane == 0) bulk_wait0();
        if (warp == 6 && lane == 0) T_DUMP(16, 6);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, C::kCols);
}

// ------------------------------------------------------------------------------------------
// Unpipelined variant (one tile at a time, 128 threads) for the shapes whose tiles do not fit
// the staged layout above (head_dim 256, 256-key blocks).  Same partial layout.
template <int D, int BK>
struct SelFwdSimpleSmem {
    static constexpr int kK = BK * D * 2;
    static constexpr int kQ = kTileRows * D * 2;
    static constexpr int kBytes = 2 * kK + kQ + 1024;
};

template <int D, int BK, typename ET>
__global__ void __launch_bounds__(128, 1) sel_fwd_simple(const SelFwdParams<ET> p, const ET* __restrict__ q, int64_t q_sn,
                                                        int64_t q_sh, const __grid_constant__ CUtensorMap kmap,
                                                        const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = smem;
    uint8_t* sV = sK + SelFwdSimpleSmem<D, BK>::kK;
    uint8_t* sQ = sV + SelFwdSimpleSmem<D, BK>::kK;
    __shared__ uint64_t bar_kv, bar_s, bar_o;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t s_ent[kTileRows];

    constexpr uint32_t kCols = tmem_cols_pow2(BK + D);
    const int tid = threadIdx.x, warp = tid >> 5;
    const SelShape& s = p.s;
    int* status = p.ix.header;
    if (tid == 0) {
        mbar_init(&bar_kv, 1);
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o, 1);
        mbar_init_fence();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const uint32_t tS = tbase, tO = tbase + BK;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const int total = p.ix.header[1];
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int begin = min(total, (int)blockIdx.x * per);
    const int end = min(total, begin + per);
    constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, BK, false, false);
    constexpr uint32_t idesc_o = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);
    TileWalker w(p.ix, s);
    uint32_t kv_loads = 0;
    bool ok = true;
    int it = 0;
    for (int item = begin; item < end && ok; ++item, ++it) {
        const bool new_kv = w.seek(item);
        if (tid < s.TPT) s_ent[tid] = tid < w.ne ? p.ix.entries[w.ebase + tid] : 0u;
        if (new_kv && tid == 0) {
            mbar_expect_tx(&bar_kv, (uint32_t)(2 * BK * D * 2));
#pragma unroll
            for (int b = 0; b < D / 64; ++b) {
                tma_load_2d(smem_u32(sK + b * BK * 128), &kmap, w.h * D + b * 64, w.row0, &bar_kv);
                tma_load_2d(smem_u32(sV + b * BK * 128), &vmap, w.h * D + b * 64, w.row0, &bar_kv);
            }
        }
        __syncthreads();
        {
            constexpr int CPR = D / 8;
#pragma unroll 4
            for (int i = tid; i < kTileRows * CPR; i += 128) {
                int r = i / CPR, c = i % CPR;
                int g = r / s.TPT, e = r - g * s.TPT;
                bool valid = g < s.G && e < w.ne;
                int64_t n = valid ? (s_ent[e] >> kSlotBits) : 0;
                const ET* src = q + n * q_sn + (int64_t)(w.h * s.G + (valid ? g : 0)) * q_sh + c * 8;
                uint32_t dst = smem_u32(sQ + (c >> 3) * (kTileRows * 128)) + sw128_chunk_off(r, c & 7);
                cp_async16(dst, src, valid);
            }
            cp_async_commit();
            cp_async_wait<0>();
            fence_async_smem();
        }
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            if (new_kv) ok = mbar_wait(&bar_kv, kv_loads & 1, status);
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a = smem_u32(sQ + (ks >> 2) * (kTileRows * 128)) + (ks & 3) * 32;
                uint32_t b = smem_u32(sK + (ks >> 2) * (BK * 128)) + (ks & 3) * 32;
                umma_ss(tS, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(b, 16, 1024), idesc_s, ks > 0);
            }
            umma_commit(&bar_s);
        }
        if (new_kv) ++kv_loads;
        ok = mbar_wait(&bar_s, it & 1, status) && ok;
        tc_fence_after();
        const int r = tid;
        const int g = r / s.TPT, e = r - g * s.TPT;
        const bool row_valid = g < s.G && e < w.ne;
        const int tok = row_valid ? (int)(s_ent[e] >> kSlotBits) : 0;
        int c_lo = 0, c_hi = BK;
        if (row_valid) visible_cols(p.bd, tok, w.row0, BK, c_lo, c_hi);
        float mx = -INFINITY;
#pragma unroll 2
        for (int c0 = 0; c0 < BK; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tS + lane_off + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (c0 + i >= c_lo && c0 + i < c_hi) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
        const float m = mx * p.scale_log2;
        float l = 0.f;
#pragma unroll 2
        for (int c0 = 0; c0 < BK; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tS + lane_off + c0, v);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float p0 = (c0 + i >= c_lo && c0 + i < c_hi) ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -m)) : 0.f;
                float p1 = (c0 + i + 1 >= c_lo && c0 + i + 1 < c_hi) ? exp2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m)) : 0.f;
                l += p0 + p1;
                pk[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
            }
            tmem_st16(tS + lane_off + (c0 >> 1), pk);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
                uint32_t b = smem_u32(sV) + ks * 2048;
                umma_ts(tO, tS + ks * 8, umma_desc_sw128(b, BK * 128, 1024), idesc_o, ks > 0);
            }
            umma_commit(&bar_o);
        }
        ok = mbar_wait(&bar_o, it & 1, status) && ok;
        tc_fence_after();
        {
            const int64_t grow = (int64_t)item * kTileRows + r;
            if (row_valid) {
                const uint32_t ent = s_ent[r - (r / s.TPT) * s.TPT];
                p.ml[((int64_t)(w.h * s.G + r / s.TPT) * s.N + (int64_t)(ent >> kSlotBits)) * s.T + (int)(ent & ((1u << kSlotBits) - 1))] =
                    make_float2(m, l);
            }
            uint4* dst = reinterpret_cast<uint4*>(p.opart + grow * D);
#pragma unroll 2
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tO + lane_off + c0, v);
                tmem_ld_wait();
                if (row_valid) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 u;
                        u.x = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
                        u.y = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
                        u.z = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
                        u.w = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
                        dst[(c0 >> 3) + q4] = u;
                    }
                }
            }
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, kCols);
}

// ------------------------------------------------------------------------------------------
template <int D, typename ET>
__global__ void __launch_bounds__(256) sel_fwd_reduce(const ET* __restrict__ opart, const float2* __restrict__ ml,
                                                      const int* __restrict__ pos, SelShape s, ET* __restrict__ o,
                                                      int64_t o_sn, int64_t o_sh, float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // n * Hq + hq
    if (row >= s.N * s.Hq) return;
    const int n = (int)(row / s.Hq), hq = (int)(row % s.Hq);   // (a 32-bit division here measured 50 % SLOWER end to end:
                                                               // the kernel is sensitive to how its warps' loads interleave)
    const int h = hq / s.G, g = hq - h * s.G;
    const int* prow = pos + ((int64_t)h * s.N + n) * s.T;
    const float2* mlrow = ml + ((int64_t)hq * s.N + n) * s.T;      // this row's statistics, one pair per slot
    constexpr int V = D / 32;   // elements per lane
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    float L, M;
    if (s.T <= 16) {
        // Up to 16 slots (with 32 rows in flight the kernel measured slower: registers, occupancy): the row loads depend only on the positions, so they are issued together with
        // the load of the statistics (one round trip less, all rows in flight per warp); weights are applied afterwards.
        int ps = lane < s.T ? __ldg(prow + lane) : -1;
        long long pr = -1;
        float m0 = -INFINITY, l0 = 0.f;
        if (ps >= 0) {
            pr = (long long)(ps / s.TPT) * kTileRows + g * s.TPT + ps % s.TPT;
            float2 v = mlrow[lane];
            m0 = v.x; l0 = v.y;
        }
        auto body = [&](auto nt_tag) {
            constexpr int NT = decltype(nt_tag)::value;
            uint4 u[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const long long prj = __shfl_sync(0xffffffffu, pr, j);
                u[j] = prj >= 0 ? ld_row_vec<V, ET>(opart + prj * D + lane * V) : make_uint4(0u, 0u, 0u, 0u);
            }
            M = m0;
#pragma unroll
            for (int o_ = 16; o_; o_ >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o_));
            const float w0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M);
            L = w0 * l0;
#pragma unroll
            for (int o_ = 16; o_; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);
#pragma unroll
            for (int j = 0; j < NT; ++j) fma_row_vec<V, ET>(acc, u[j], __shfl_sync(0xffffffffu, w0, j));
        };
        body(std::integral_constant<int, 16>{});
    } else {
        // lane handles slots lane and lane + 32: partial row index and statistics
        int64_t pr0 = -1, pr1 = -1;
        float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
        if (lane < s.T) {
            int ps = __ldg(prow + lane);
            if (ps >= 0) {
                pr0 = (int64_t)(ps / s.TPT) * kTileRows + g * s.TPT + ps % s.TPT;
                float2 v = mlrow[lane];
                m0 = v.x; l0 = v.y;
            }
        }
        if (lane + 32 < s.T) {
            int ps = __ldg(prow + lane + 32);
            if (ps >= 0) {
                pr1 = (int64_t)(ps / s.TPT) * kTileRows + g * s.TPT + ps % s.TPT;
                float2 v = mlrow[lane + 32];
                m1 = v.x; l1 = v.y;
            }
        }
        M = fmaxf(m0, m1);
#pragma unroll
        for (int o_ = 16; o_; o_ >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o_));
        float w0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M);
        float w1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - M);
        L = w0 * l0 + w1 * l1;
#pragma unroll
        for (int o_ = 16; o_; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);
        for (int sl0 = 0; sl0 < s.T; sl0 += 8) {
            uint4 u[8];
            float w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int sl = sl0 + j;
                w[j] = __shfl_sync(0xffffffffu, sl < 32 ? w0 : w1, sl & 31);
                const long long pr = __shfl_sync(0xffffffffu, (long long)(sl < 32 ? pr0 : pr1), sl & 31);
                if (sl >= s.T) w[j] = 0.f;
                u[j] = w[j] != 0.f ? ld_row_vec<V, ET>(opart + pr * D + lane * V) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) fma_row_vec<V, ET>(acc, u[j], w[j]);
        }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    ET* dst = o + (int64_t)n * o_sn + (int64_t)hq * o_sh + lane * V;
    if constexpr (V == 2) {
        *reinterpret_cast<uint32_t*>(dst) = ElemTraits<ET>::pack2(acc[0] * inv, acc[1] * inv);
    } else if constexpr (V == 4) {
        uint2 u;
        u.x = ElemTraits<ET>::pack2(acc[0] * inv, acc[1] * inv);
        u.y = ElemTraits<ET>::pack2(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2*>(dst) = u;
    } else {
        uint4 u;
        u.x = ElemTraits<ET>::pack2(acc[0] * inv, acc[1] * inv);
        u.y = ElemTraits<ET>::pack2(acc[2] * inv, acc[3] * inv);
        u.z = ElemTraits<ET>::pack2(acc[4] * inv, acc[5] * inv);
        u.w = ElemTraits<ET>::pack2(acc[6] * inv, acc[7] * inv);
        *reinterpret_cast<uint4*>(dst) = u;
    }
    if (lane == 0) lse[(int64_t)hq * s.N + n] = L > 0.f ? M + log2f(L) : -INFINITY;
}

// ------------------------------------------------------------------------------------------
template <int D, int BK, typename ET>
static cudaError_t launch_sel_fwd(const SelFwdArgs& a, const SelShape& s, const SelIndex& ix, int num_sms,
                                  cudaStream_t stream) {
    SelFwdParams<ET> p;
    p.s = s; p.ix = ix;
    p.scale_log2 = a.sm_scale * 1.4426950408889634f;
    p.opart = (ET*)a.opart; p.ml = a.ml;
    p.run = a.run > 0 ? a.run : 8;
    p.bd = a.bd;
    p.dbg = 0;
#ifdef FSA_TIMING
    { const char* v = getenv("FSA_DBG"); p.dbg = v ? atoi(v) : 0; }
#endif
    cudaError_t e;
    constexpr bool kPipelined = (D <= 128 && BK <= 128);
    // the gather warps of the pipelined kernel address rows by 32-bit offsets in units of 8 elements
    const bool offsets_fit = ((s.N * a.q_sn + (int64_t)s.Hq * a.q_sh) >> 3) < 0x7fffffffll;
    if (kPipelined && a.omap && offsets_fit) {
        if constexpr (kPipelined) {
            auto kern = sel_fwd_main<D, BK, ET>;
            constexpr int smem = SelFwdCfg<D, BK>::kBytes;
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e;
            prof_begin(0, stream);
            kern<<<num_sms, kFwdThreads, smem, stream>>>(p, (const ET*)a.q, a.q_sn, a.q_sh, *a.kmap, *a.vmap, *a.omap);
            prof_end(0, stream);
        }
    } else {
        auto kern = sel_fwd_simple<D, BK, ET>;
        constexpr int smem = SelFwdSimpleSmem<D, BK>::kBytes;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        constexpr int tmem_per_cta = (int)tmem_cols_pow2(BK + D);
        int per_sm = 512 / tmem_per_cta;
        int by_smem = (227 * 1024) / (smem + 2048);
        if (by_smem < per_sm) per_sm = by_smem;
        if (per_sm < 1) per_sm = 1;
        prof_begin(0, stream);
        kern<<<num_sms * per_sm, 128, smem, stream>>>(p, (const ET*)a.q, a.q_sn, a.q_sh, *a.kmap, *a.vmap);
        prof_end(0, stream);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    int64_t rows = s.N * s.Hq;
    if (rows > 0) {
        unsigned grid = (unsigned)((rows + 7) / 8);
        prof_begin(1, stream);
        sel_fwd_reduce<D, ET><<<grid, 256, 0, stream>>>((const ET*)a.opart, a.ml, ix.pos, s, (ET*)a.o, a.o_sn, a.o_sh, a.lse);
        prof_end(1, stream);
    }
    return cudaGetLastError();
}

template <typename ET>
static cudaError_t dispatch_typed(const SelFwdArgs& a, const SelShape& s, const SelIndex& ix, int num_sms, cudaStream_t stream) {
#define FSA_CASE(DD, BB) \
    if (s.D == DD && s.BK == BB) return launch_sel_fwd<DD, BB, ET>(a, s, ix, num_sms, stream);
    FSA_CASE(64, 32) FSA_CASE(64, 64) FSA_CASE(64, 128) FSA_CASE(64, 256)
    FSA_CASE(128, 32) FSA_CASE(128, 64) FSA_CASE(128, 128) FSA_CASE(128, 256)
    FSA_CASE(256, 32) FSA_CASE(256, 64) FSA_CASE(256, 128)
#undef FSA_CASE
    return cudaErrorInvalidValue;
}

cudaError_t dispatch_sel_fwd(int dtype, const SelFwdArgs& a, const SelShape& s, const SelIndex& ix, int num_sms,
                             cudaStream_t stream) {
    if (dtype == kBF16) return dispatch_typed<__nv_bfloat16>(a, s, ix, num_sms, stream);
    return dispatch_typed<__half>(a, s, ix, num_sms, stream);
}

}  // namespace fsa

#ifdef FSA_TIMING
extern "C" int fsa_debug_read_fwd_trace(long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, fsa::g_fwd_trace, (size_t)n * sizeof(long long));
}
extern "C" int fsa_debug_read_fwd_timing(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, fsa::g_fwd_timing, (size_t)n * sizeof(unsigned long long));
}
#endif
