// Range attention forward, query-tile-major ("dense") kernel for sm_100a: every token attends one contiguous range of
// K/V rows, as in the compressed branch (replaces the forward of CompressedAttention,
// nsa_ref/ops/compressed_attention.py:762-829, kernel :33-190) and in the sliding-window branch (replaces the
// flash_attn_varlen_func call of fsa/module/fsa.py:149-159).
//
// One CTA = one tile of <= 128 rows = (query head of a GQA group, TPT consecutive tokens of one sequence) x one KV head.
// The rows of the tile see neighbouring ranges, so the CTA walks the 64-row K/V tiles from the lowest row any of its rows
// sees to the highest, keeps the output accumulator in TMEM across them (online softmax) and writes o and lse once: no
// partial rows, no merge kernel, no index.  Two CTAs share an SM (96 KB of shared memory and 256 TMEM columns each), so
// the softmax of one overlaps the MMAs of the other.
//   warp 0      TMA producer: the Q tile once (3-D box: column, token, head -> head-major rows), K and V tiles through two
//               rings of two stages (K is released by the S product, V by the P V product, so K runs a tile ahead);
//   warp 1      one elected thread issues S(j+1) = Q K^T before the softmax of tile j is done, then O (+)= P(j) V(j);
//   warps 2..5  one row per thread: scaled logits from TMEM, per-row range mask, running max / sum, P -> TMEM (input dtype,
//               over S).  The reference max of a row is only raised when a tile exceeds it by more than 2^8 (the final
//               o = O / l does not depend on the reference); then the warp waits for the previous P V product and
//               rescales its 32 accumulator rows in TMEM.  Epilogue: o = O / l through swizzled staging (the Q tile's
//               memory) and a 3-D TMA store, or plain stores for the last, partial tile of a sequence; lse = m + log2 l.
#include "../../include/fsa_sm100.h"
#include <climits>

#include "sel_launch.cuh"

namespace fsa {

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int box_rows);
int make_tile_map_3d_box(CUtensorMap* map, const void* base, int dtype, int64_t d0, int64_t d1, int64_t d2, int64_t stride1,
                         int64_t stride2, int box1, int box2);
int ensure_context();
int device_sm_count(int* out);

struct RangeDenseParams {
    const int32_t* cu_q;    // [B + 1]
    const int32_t* cu_k;    // [B + 1] first K/V row of every sequence
    const int32_t* kv_lo;   // [N] lowest visible K/V row of every token, or null (the sequence's first row)
    const int32_t* kv_hi;   // [N] highest visible K/V row, lower than kv_lo when the token sees nothing
    int64_t N, Nk;
    int B, Hq, Hk, G, TPT;
    float scale_log2;
    void* o;  int64_t o_sn, o_sh;     // [N, Hq, D]
    float* lse;                       // [Hq, N] log2 units
    int* status;
};

constexpr int kRdThreads = 192;
constexpr int kRdBK = 64;
constexpr float kRdLazy = 8.0f;       // raise a row's reference max only when exceeded by more than this (log2 units)

__device__ __forceinline__ float rd_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, typename ET>
__global__ void __launch_bounds__(kRdThreads, 2) range_fwd_dense(const RangeDenseParams p, const __grid_constant__ CUtensorMap qmap,
                                                                const __grid_constant__ CUtensorMap kmap,
                                                                const __grid_constant__ CUtensorMap vmap,
                                                                const __grid_constant__ CUtensorMap omap) {
    constexpr int BK = kRdBK;
    constexpr int kQ = kTileRows * D * 2;            // Q tile, later the output staging
    constexpr int kKt = BK * D * 2;                  // one K (or V) tile
    constexpr int KH = D / 64;
    constexpr uint32_t kCols = (2 * BK + D) <= 128 ? 128 : 256;
    constexpr int cS = 0, cO = 2 * BK;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kQ;
    uint8_t* sV = sK + 2 * kKt;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kKt);
    uint64_t* q_full = bars;            // [1]
    uint64_t* k_full = bars + 1;        // [2]
    uint64_t* k_empty = bars + 3;       // [2]
    uint64_t* v_full = bars + 5;        // [2]
    uint64_t* v_empty = bars + 7;       // [2]
    uint64_t* s_full = bars + 9;        // [2]
    uint64_t* p_full = bars + 11;       // [2]
    uint64_t* pv_done = bars + 13;      // [1]
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 14);
    int* s_meta = reinterpret_cast<int*>(bars + 15);     // [0] sequence, [1] first token, [2] tokens, [3] first K/V row, [4] K/V tiles

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int* status = p.status;
    const int h = blockIdx.y;
    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 128);
        }
        mbar_init(pv_done, 1);
        mbar_init_fence();
        tma_prefetch_desc(&qmap);
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        tma_prefetch_desc(&omap);
    }
    if (warp == 0) {
        // which tile is this: the heaviest (last) tiles of the list start first
        const int total = count_seq_tiles(p.cu_q, p.B, p.TPT, lane);
        int seq, tok0, ne;
        find_seq_tile(p.cu_q, p.B, p.TPT, total - 1 - (int)blockIdx.x, lane, seq, tok0, ne);
        // lowest and highest K/V row any token of the tile sees
        int lo = INT_MAX, hi = -1;
        if (seq >= 0) {
            const int k0 = __ldg(p.cu_k + seq);
            for (int e = lane; e < ne; e += 32) {
                const int l = p.kv_lo ? __ldg(p.kv_lo + tok0 + e) : k0;
                const int u = __ldg(p.kv_hi + tok0 + e);
                if (u >= l) { lo = min(lo, l); hi = max(hi, u); }
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, d));
            hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, d));
        }
        if (lane == 0) {
            lo = max(lo, 0);
            hi = min(hi, (int)p.Nk - 1);
            s_meta[0] = seq; s_meta[1] = tok0; s_meta[2] = ne; s_meta[3] = lo;
            s_meta[4] = hi >= lo ? (hi - lo) / BK + 1 : 0;
        }
        tmem_alloc(&tmem_slot, kCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const int seq = s_meta[0], tok0 = s_meta[1], ne = s_meta[2], row_lo = s_meta[3], nblk = s_meta[4];

    if (seq >= 0) {
        if (warp == 0) {
            // ------------------------------------------------------------------ TMA producer
            bool ok = true;
            if (lane == 0 && nblk > 0) {
                mbar_expect_tx(q_full, (uint32_t)(KH * 128 * p.TPT * p.G));
#pragma unroll
                for (int b = 0; b < KH; ++b) tma_load_3d(smem_u32(sQ + b * (kTileRows * 128)), &qmap, b * 64, tok0, h * p.G, q_full);
            }
            // K tile j and V tile j are loaded in the order the MMA warp needs them: K(0), K(1), V(0), K(2), V(1), ...
            for (int step = 0; step < nblk + 1 && ok; ++step) {
                if (lane == 0) {
                    const int jk = step, jv = step - 1;
                    if (jk < nblk) {
                        const int st = jk & 1;
                        ok = mbar_wait(&k_empty[st], ((jk >> 1) & 1) ^ 1, status) && ok;
                        mbar_expect_tx(&k_full[st], (uint32_t)kKt);
#pragma unroll
                        for (int b = 0; b < KH; ++b)
                            tma_load_2d(smem_u32(sK + st * kKt + b * (BK * 128)), &kmap, h * D + b * 64, row_lo + jk * BK, &k_full[st]);
                    }
                    if (jv >= 0) {
                        const int st = jv & 1;
                        ok = mbar_wait(&v_empty[st], ((jv >> 1) & 1) ^ 1, status) && ok;
                        mbar_expect_tx(&v_full[st], (uint32_t)kKt);
#pragma unroll
                        for (int b = 0; b < KH; ++b)
                            tma_load_2d(smem_u32(sV + st * kKt + b * (BK * 128)), &vmap, h * D + b * 64, row_lo + jv * BK, &v_full[st]);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer
            const bool leader = elect_one();
            constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, BK, false, false);
            constexpr uint32_t idesc_o = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);
            constexpr uint32_t hi_1024 = umma_desc_hi(1024);
            const uint32_t q_lo = umma_desc_lo(smem_u32(sQ), 16);
            const uint32_t k_lo = umma_desc_lo(smem_u32(sK), 16);
            const uint32_t v_lo = umma_desc_lo(smem_u32(sV), BK * 128);     // MN-major: LBO = slab stride
            bool ok = true;
            auto issue_s = [&](int j) {
                const int st = j & 1;
                ok = mbar_wait(&k_full[st], (j >> 1) & 1, status) && ok;
                tc_fence_after();
                if (leader) {
                    constexpr int kSlabA = (kTileRows * 128) >> 4, kSlabB = (BK * 128) >> 4;
                    const uint32_t b_lo = k_lo + (uint32_t)(st * (kKt >> 4));
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks)
                        umma_ss(tbase + cS + st * BK, umma_desc_pack(q_lo + (ks >> 2) * kSlabA + (ks & 3) * 2, hi_1024),
                                umma_desc_pack(b_lo + (ks >> 2) * kSlabB + (ks & 3) * 2, hi_1024), idesc_s, ks > 0);
                    umma_commit(&k_empty[st]);
                    umma_commit(&s_full[st]);
                }
                __syncwarp();
            };
            if (nblk > 0) {
                ok = mbar_wait(q_full, 0, status) && ok;
                issue_s(0);
            }
            for (int j = 0; j < nblk && ok; ++j) {
                const int st = j & 1;
                // S(j + 1) overwrites the buffer P(j - 1) was read from by the product issued one iteration ago (in order)
                if (j + 1 < nblk) issue_s(j + 1);
                ok = mbar_wait(&p_full[st], (j >> 1) & 1, status) && ok;
                ok = mbar_wait(&v_full[st], (j >> 1) & 1, status) && ok;
                tc_fence_after();
                if (leader) {
                    const uint32_t b_lo = v_lo + (uint32_t)(st * (kKt >> 4));
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks)
                        umma_ts(tbase + cO, tbase + cS + st * BK + ks * 8, umma_desc_pack(b_lo + ks * (2048 >> 4), hi_1024), idesc_o,
                                (j > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(&v_empty[st]);
                    umma_commit(pv_done);
                }
                __syncwarp();
            }
        } else {
            // ------------------------------------------------------------------ softmax and epilogue: one row per thread
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane;
            const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
            const int g = r / p.TPT, e = r - g * p.TPT;
            const bool row_valid = g < p.G && e < ne;
            const int tok = tok0 + e;
            int lo_r = 0, hi_r = -1;
            if (row_valid) {
                lo_r = p.kv_lo ? __ldg(p.kv_lo + tok) : __ldg(p.cu_k + seq);
                hi_r = min(__ldg(p.kv_hi + tok), (int)p.Nk - 1);     // rows past the end of K/V do not exist
            }
            float m_ref = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < nblk && ok; ++j) {
                const int st = j & 1;
                const int R0 = row_lo + j * BK;
                const int c_lo = max(0, lo_r - R0), c_hi = min(BK, hi_r - R0 + 1);      // visible columns [c_lo, c_hi)
                ok = mbar_wait(&s_full[st], (j >> 1) & 1, status) && ok;
                tc_fence_after();
                uint32_t v[BK];
                tmem_ld32(tbase + lane_off + cS + st * BK, *reinterpret_cast<uint32_t (*)[32]>(&v[0]));
                tmem_ld32(tbase + lane_off + cS + st * BK + 32, *reinterpret_cast<uint32_t (*)[32]>(&v[32]));
                tmem_ld_wait();
                if (c_lo > 0 || c_hi < BK) {
#pragma unroll
                    for (int i = 0; i < BK; ++i)
                        if (i < c_lo || i >= c_hi) v[i] = 0xff800000u;      // -inf: exp2 gives exactly 0
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < BK; i += 4) {
                    mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
                    mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
                    mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
                    mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
                }
                const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
                // raise the reference only when this tile exceeds it by a lot; the first finite maximum sets it
                float alpha = 1.f;
                const bool raise = m_blk > m_ref + kRdLazy;     // false when m_blk is -inf; true when m_ref is -inf and m_blk finite
                if (raise) {
                    alpha = m_ref == -INFINITY ? 0.f : rd_ex2(m_ref - m_blk);
                    m_ref = m_blk;
                }
                // accumulator rows already hold products (j > 0): rescale them when any row of the warp changes reference
                const bool scale_acc = __any_sync(0xffffffffu, raise && j > 0);
                if (scale_acc) {
                    ok = mbar_wait(pv_done, (j - 1) & 1, status) && ok;
                    tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < D; c0 += 32) {
                        uint32_t a[32];
                        tmem_ld32(tbase + lane_off + cO + c0, a);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * alpha);
                        tmem_st32(tbase + lane_off + cO + c0, a);
                    }
                }
                l_run *= alpha;
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;     // all columns masked so far: every p is exp2(-inf) = 0
                float ls[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[BK / 2];
#pragma unroll
                for (int i = 0; i < BK; i += 4) {
                    const float p0 = rd_ex2(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_use));
                    const float p1 = rd_ex2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_use));
                    const float p2 = rd_ex2(fmaf(__uint_as_float(v[i + 2]), p.scale_log2, -m_use));
                    const float p3 = rd_ex2(fmaf(__uint_as_float(v[i + 3]), p.scale_log2, -m_use));
                    ls[0] += p0; ls[1] += p1; ls[2] += p2; ls[3] += p3;
                    pk[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
                    pk[(i >> 1) + 1] = ElemTraits<ET>::pack2(p2, p3);
                }
                l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
                tmem_st32(tbase + lane_off + cS + st * BK, *reinterpret_cast<uint32_t (*)[32]>(&pk[0]));
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(&p_full[st]);
            }
            // ---- epilogue
            if (nblk > 0) {
                ok = mbar_wait(pv_done, (nblk - 1) & 1, status) && ok;
                tc_fence_after();
            }
            const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
            if (row_valid && ok) p.lse[(int64_t)(h * p.G + g) * p.N + tok] = l_run > 0.f ? m_ref + log2f(l_run) : -INFINITY;
            const bool full_tile = ne == p.TPT && p.G * p.TPT == kTileRows;      // whole box inside the sequence, every row staged
            uint8_t* my_stage = sQ + quarter * (32 * 128);     // per 64-column slab: rows of this warp at (slab base) + 32 * 128 * quarter
            ET* orow = reinterpret_cast<ET*>(p.o) + (int64_t)tok * p.o_sn + (int64_t)(h * p.G + g) * p.o_sh;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t a[32];
                if (nblk > 0) {
                    tmem_ld32(tbase + lane_off + cO + c0, a);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) a[i] = 0u;
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 x;
                    x.x = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 0]) * inv_l, __uint_as_float(a[q4 * 8 + 1]) * inv_l);
                    x.y = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 2]) * inv_l, __uint_as_float(a[q4 * 8 + 3]) * inv_l);
                    x.z = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 4]) * inv_l, __uint_as_float(a[q4 * 8 + 5]) * inv_l);
                    x.w = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 6]) * inv_l, __uint_as_float(a[q4 * 8 + 7]) * inv_l);
                    const int chunk = (c0 >> 3) + q4;
                    if (full_tile) {
                        *reinterpret_cast<uint4*>(sQ + (chunk >> 3) * (kTileRows * 128) + sw128_chunk_off(r, chunk & 7)) = x;
                    } else if (row_valid && ok) {
                        *reinterpret_cast<uint4*>(orow + chunk * 8) = x;
                    }
                }
            }
            (void)my_stage;
            if (full_tile) {
                // all four warps have staged their rows: one 3-D store per 64-column slab
                fence_async_smem();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0 && ok) {
#pragma unroll
                    for (int b = 0; b < KH; ++b) tma_store_3d(&omap, b * 64, tok0, h * p.G, smem_u32(sQ + b * (kTileRows * 128)));
                    bulk_commit();
                    bulk_wait_read0();     // the staging memory has been read; the global writes complete on their own
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, kCols);
}

template <int D, typename ET>
static cudaError_t launch_rd(const RangeDenseParams& p, const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                             const CUtensorMap& omap, int max_tiles, cudaStream_t stream) {
    constexpr int smem = kTileRows * D * 2 + 4 * kRdBK * D * 2 + 256;
    auto kern = range_fwd_dense<D, ET>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    prof_begin(FSA_KERNEL_RANGE_DENSE, stream);
    kern<<<dim3((unsigned)max_tiles, (unsigned)p.Hk), kRdThreads, smem, stream>>>(p, qmap, kmap, vmap, omap);
    prof_end(FSA_KERNEL_RANGE_DENSE, stream);
    return cudaGetLastError();
}


// ------------------------------------------------------------------------------------------------ dQ, query-tile-major
// dQ of range attention with the same tiling as the forward above: per K/V tile S = Q K^T and dP = dO V^T, then
// P = exp2(S c - lse), dS = scale P (dP - delta) to swizzled shared memory, dQ (+)= dS K accumulated in TMEM over the
// tiles and written once.  (In the reference: the dQ part of _backward_kernel, nsa_ref/ops/compressed_attention.py:
// 193-760, and of flash-attn's backward for the sliding window.)  With it the block-major backward kernel computes
// only dK and dV and no partial dQ row is written or merged.  One CTA per SM, 352 threads:
//   warp 0      TMA producer: Q and dO tiles of every item, (K, V) tiles through a four-stage ring (a stage comes free only
//               when the tile's dQ product is done, and the next load needs a microsecond to land);
//   warp 1      one elected thread issues S and dP (two TMEM buffers: they run a tile ahead of the row threads);
//   warp 10     one elected thread issues dQ (a second issuer: see the MMA section);
//   warps 2..9  two groups of 128 row threads, each on 32 of the 64 key columns: dS to one of two shared-memory buffers;
//               epilogue: each group rounds 64 of the dQ columns, stages them (the Q tile's memory) and stores its slab by
//               3-D TMA (plain stores for the last, partial tile of a sequence).
struct RangeDqParams {
    const int32_t* cu_q;
    const int32_t* cu_k;
    const int32_t* kv_lo;
    const int32_t* kv_hi;
    int64_t N, Nk;
    int B, Hq, Hk, G, TPT;
    float scale, scale_log2;
    const float* lse;       // [Hq, N] log2 units
    const float* delta;     // [Hq, N] sum_d o dO
    void* dq;               // [N, Hq, D] contiguous
    int* status;
};

constexpr int kDqThreads = 352;     // producer, S/dP issuer, 8 row warps, dQ issuer
constexpr int kDqStages = 4;

// One work item of the dQ kernel: a tile of tokens x one KV head.
struct DqItem {
    int seq, tok0, ne, row_lo, nblk, h;
};

// Work item w of the list (heaviest tiles first).  Warp-collective: all 32 lanes call it and get the same answer.
__device__ __forceinline__ DqItem dq_item(const RangeDqParams& p, int ntiles, int w, int lane) {
    DqItem m;
    m.h = w % p.Hk;
    const int want = ntiles - 1 - w / p.Hk;
    m.row_lo = 0; m.nblk = 0;
    find_seq_tile(p.cu_q, p.B, p.TPT, want, lane, m.seq, m.tok0, m.ne);
    if (m.seq < 0) return m;
    int lo = INT_MAX, hi = -1;
    const int k0 = __ldg(p.cu_k + m.seq);
    for (int e = lane; e < m.ne; e += 32) {
        const int l = p.kv_lo ? __ldg(p.kv_lo + m.tok0 + e) : k0;
        const int u = __ldg(p.kv_hi + m.tok0 + e);
        if (u >= l) { lo = min(lo, l); hi = max(hi, u); }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, d));
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, d));
    }
    lo = max(lo, 0);
    hi = min(hi, (int)p.Nk - 1);
    m.row_lo = lo;
    m.nblk = hi >= lo ? (hi - lo) / kRdBK + 1 : 0;
    return m;
}

template <typename ET>
__global__ void __launch_bounds__(kDqThreads, 1) range_bwd_dq_dense(const RangeDqParams p, const __grid_constant__ CUtensorMap qmap,
                                                                   const __grid_constant__ CUtensorMap domap,
                                                                   const __grid_constant__ CUtensorMap kmap,
                                                                   const __grid_constant__ CUtensorMap vmap,
                                                                   const __grid_constant__ CUtensorMap dqmap) {
    constexpr int D = 128, BK = kRdBK, KH = D / 64;
    constexpr int kQ = kTileRows * D * 2;            // Q tile, same for dO
    constexpr int kKt = BK * D * 2;
    constexpr int kDS = kTileRows * BK * 2;          // one dS buffer; the two together stage a dQ tile in the epilogue
    constexpr uint32_t kCols = 512;
    constexpr int cDQ = 256;                         // S(b) at 128 b, dP(b) at 128 b + 64
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sDO = sQ + kQ;
    uint8_t* sKV = sDO + kQ;                         // stage: K then V
    uint8_t* sDS = sKV + kDqStages * 2 * kKt;        // two buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + 2 * kDS);
    uint64_t* qd_full = bars;           // Q and dO tiles of an item have landed
    uint64_t* qd_empty = bars + 1;      // ... have been read by the item's last S / dP products
    uint64_t* kv_full = bars + 2;                        // [stages]
    uint64_t* kv_empty = kv_full + kDqStages;            // [stages] the dQ product of the tile is done
    uint64_t* sdp_full = kv_empty + kDqStages;           // [2]
    uint64_t* sdp_free = sdp_full + 2;                   // [2] the 256 row threads have read S and dP
    uint64_t* ds_full = sdp_free + 2;                    // [2] ... have written dS
    uint64_t* ds_empty = ds_full + 2;                    // [2] the dQ product has read dS
    uint64_t* dq_free = ds_empty + 2;                    // the 256 row threads have read an item's dQ accumulator
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(dq_free + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int* status = p.status;
    if (tid == 0) {
        mbar_init(qd_full, 1); mbar_init(qd_empty, 1);
        for (int i = 0; i < kDqStages; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sdp_full[i], 1); mbar_init(&sdp_free[i], 256);
            mbar_init(&ds_full[i], 256); mbar_init(&ds_empty[i], 1);
        }
        mbar_init(dq_free, 256);
        mbar_init_fence();
        tma_prefetch_desc(&qmap);
        tma_prefetch_desc(&domap);
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
        tma_prefetch_desc(&dqmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const int ntiles = count_seq_tiles(p.cu_q, p.B, p.TPT, lane);
    const int nitems = ntiles * p.Hk;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        bool ok = true;
        int kvc = 0, qi = 0;           // K/V tiles and non-empty items so far
        for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
            const DqItem m = dq_item(p, ntiles, w, lane);
            if (m.nblk == 0) continue;
            if (lane == 0) {
                ok = mbar_wait(qd_empty, (qi & 1) ^ 1, status) && ok;
                mbar_expect_tx(qd_full, (uint32_t)(2 * KH * 128 * p.TPT * p.G));
#pragma unroll
                for (int b = 0; b < KH; ++b) {
                    tma_load_3d(smem_u32(sQ + b * (kTileRows * 128)), &qmap, b * 64, m.tok0, m.h * p.G, qd_full);
                    tma_load_3d(smem_u32(sDO + b * (kTileRows * 128)), &domap, b * 64, m.tok0, m.h * p.G, qd_full);
                }
            }
            ++qi;
            for (int j = 0; j < m.nblk && ok; ++j, ++kvc) {
                if (lane == 0) {
                    const int st = kvc % kDqStages;
                    ok = mbar_wait(&kv_empty[st], ((kvc / kDqStages) & 1) ^ 1, status) && ok;
                    mbar_expect_tx(&kv_full[st], (uint32_t)(2 * kKt));
                    uint8_t* dK = sKV + st * 2 * kKt;
                    uint8_t* dV = dK + kKt;
#pragma unroll
                    for (int b = 0; b < KH; ++b) {
                        tma_load_2d(smem_u32(dK + b * (BK * 128)), &kmap, m.h * D + b * 64, m.row_lo + j * BK, &kv_full[st]);
                        tma_load_2d(smem_u32(dV + b * (BK * 128)), &vmap, m.h * D + b * 64, m.row_lo + j * BK, &kv_full[st]);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
    } else if (warp == 1 || warp == kDqThreads / 32 - 1) {
        // ------------------------------------------------------------------ MMA issuers
        // Two warps: the k-steps of one accumulator follow one another at ~100 cycles each, and a single issuing thread also
        // waits on barriers between products; with dQ on a warp of its own its chain overlaps the S / dP chains of the next
        // tile (measured: 20 % faster).  Warp 1 issues S and dP, the last warp issues dQ.  The K/V tiles of all items form one sequence
        // c = 0, 1, ...; S / dP run ahead of dQ as far as their two TMEM buffers and the K/V ring allow, also across the
        // boundary between two items (the next item's Q / dO are loaded as soon as this item's last S / dP are done).
        const bool leader = elect_one();
        constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, BK, false, false);
        constexpr uint32_t idesc_dq = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);     // dS (K-major) x K (MN-major)
        constexpr uint32_t hi_1024 = umma_desc_hi(1024);
        constexpr int kSlabA = (kTileRows * 128) >> 4, kSlabB = (BK * 128) >> 4;
        const uint32_t q_lo = umma_desc_lo(smem_u32(sQ), 16), do_lo = umma_desc_lo(smem_u32(sDO), 16);
        const uint32_t kv_lo_ = umma_desc_lo(smem_u32(sKV), 16);
        const uint32_t ds_lo = umma_desc_lo(smem_u32(sDS), 16);
        const uint32_t k_mn_lo = umma_desc_lo(smem_u32(sKV), BK * 128);
        bool ok = true;
        int c = 0, qi = 0;
        for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
            const DqItem m = dq_item(p, ntiles, w, lane);
            if (m.nblk == 0) continue;
            if (warp == 1) {
                ok = mbar_wait(qd_full, qi & 1, status) && ok;
                for (int j = 0; j < m.nblk && ok; ++j, ++c) {
                    const int b = c & 1, st = c % kDqStages;
                    ok = mbar_wait(&kv_full[st], (c / kDqStages) & 1, status) && ok;
                    ok = mbar_wait(&sdp_free[b], ((c >> 1) & 1) ^ 1, status) && ok;     // S / dP of tile c - 2 have been read
                    tc_fence_after();
                    if (leader) {
                        const uint32_t k_lo = kv_lo_ + (uint32_t)(st * ((2 * kKt) >> 4));
                        const uint32_t v_lo = k_lo + (uint32_t)(kKt >> 4);
#pragma unroll
                        for (int ks = 0; ks < D / 16; ++ks)
                            umma_ss(tbase + b * 128, umma_desc_pack(q_lo + (ks >> 2) * kSlabA + (ks & 3) * 2, hi_1024),
                                    umma_desc_pack(k_lo + (ks >> 2) * kSlabB + (ks & 3) * 2, hi_1024), idesc_s, ks > 0);
#pragma unroll
                        for (int ks = 0; ks < D / 16; ++ks)
                            umma_ss(tbase + b * 128 + BK, umma_desc_pack(do_lo + (ks >> 2) * kSlabA + (ks & 3) * 2, hi_1024),
                                    umma_desc_pack(v_lo + (ks >> 2) * kSlabB + (ks & 3) * 2, hi_1024), idesc_s, ks > 0);
                        umma_commit(&sdp_full[b]);
                        if (j + 1 == m.nblk) umma_commit(qd_empty);          // every S / dP of this item has been issued
                    }
                    __syncwarp();
                }
            } else {
                for (int j = 0; j < m.nblk && ok; ++j, ++c) {
                    const int b = c & 1, st = c % kDqStages;
                    ok = mbar_wait(&ds_full[b], (c >> 1) & 1, status) && ok;      // (implies S / dP of the tile are done with K and V)
                    if (j == 0 && qi > 0) ok = mbar_wait(dq_free, (qi - 1) & 1, status) && ok;     // the previous item's dQ has been read
                    fence_async_smem();
                    tc_fence_after();
                    if (leader) {
                        const uint32_t a_lo = ds_lo + (uint32_t)(b * (kDS >> 4));
                        const uint32_t b_lo = k_mn_lo + (uint32_t)(st * ((2 * kKt) >> 4));
#pragma unroll
                        for (int ks = 0; ks < BK / 16; ++ks)
                            umma_ss(tbase + cDQ, umma_desc_pack(a_lo + ks * 2, hi_1024), umma_desc_pack(b_lo + ks * (2048 >> 4), hi_1024),
                                    idesc_dq, (j > 0 || ks > 0) ? 1u : 0u);
                        umma_commit(&kv_empty[st]);
                        umma_commit(&ds_empty[b]);
                    }
                    __syncwarp();
                }
            }
            ++qi;
        }
    } else {
        // ------------------------------------------------------------------ dS and the epilogue: one row, half the columns
        const int sb = (warp - 2) >> 2;               // column half of this group
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const int g = r / p.TPT, e = r - g * p.TPT;
        constexpr int HC = BK / 2;
        const int cb = sb * HC;
        bool ok = true;
        int c = 0, qi = 0;
        for (int w = blockIdx.x; w < nitems && ok; w += gridDim.x) {
            const DqItem m = dq_item(p, ntiles, w, lane);
            const bool row_valid = g < p.G && e < m.ne;
            const int tok = m.tok0 + e;
            int lo_r = 0, hi_r = -1;
            float lse_r = 0.f, delta_s = 0.f;
            if (row_valid) {
                lo_r = p.kv_lo ? __ldg(p.kv_lo + tok) : __ldg(p.cu_k + m.seq);
                hi_r = min(__ldg(p.kv_hi + tok), (int)p.Nk - 1);     // rows past the end of K/V do not exist
                const int64_t idx = (int64_t)(m.h * p.G + g) * p.N + tok;
                lse_r = __ldg(p.lse + idx);
                delta_s = __ldg(p.delta + idx) * p.scale;
                if (!(lse_r > -INFINITY)) hi_r = lo_r - 1;      // a row that saw nothing in the forward sees nothing here
            }
            for (int j = 0; j < m.nblk && ok; ++j, ++c) {
                const int b = c & 1;
                const int R0 = m.row_lo + j * BK;
                const int c_lo = max(0, lo_r - R0), c_hi = min(BK, hi_r - R0 + 1);
                ok = mbar_wait(&sdp_full[b], (c >> 1) & 1, status) && ok;
                tc_fence_after();
                uint32_t dd[HC / 2];
                const bool all_visible = __all_sync(0xffffffffu, c_lo == 0 && c_hi == BK);
                {
                    uint32_t sv[32], dv[32];
                    tmem_ld32(tbase + lane_off + b * 128 + cb, sv);
                    tmem_ld32(tbase + lane_off + b * 128 + BK + cb, dv);
                    tmem_ld_wait();
                    tc_fence_before();
                    mbar_arrive(&sdp_free[b]);       // both rows are in registers: the buffer may take tile c + 2
                    if (all_visible) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = rd_ex2(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse_r));
                            const float p1 = rd_ex2(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -lse_r));
                            dd[i >> 1] = ElemTraits<ET>::pack2(p0 * fmaf(__uint_as_float(dv[i]), p.scale, -delta_s),
                                                               p1 * fmaf(__uint_as_float(dv[i + 1]), p.scale, -delta_s));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = (cb + i >= c_lo && cb + i < c_hi) ? rd_ex2(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse_r)) : 0.f;
                            const float p1 = (cb + i + 1 >= c_lo && cb + i + 1 < c_hi) ? rd_ex2(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -lse_r)) : 0.f;
                            const float d0 = p0 > 0.f ? p0 * fmaf(__uint_as_float(dv[i]), p.scale, -delta_s) : 0.f;
                            const float d1 = p1 > 0.f ? p1 * fmaf(__uint_as_float(dv[i + 1]), p.scale, -delta_s) : 0.f;
                            dd[i >> 1] = ElemTraits<ET>::pack2(d0, d1);
                        }
                    }
                }
                ok = mbar_wait(&ds_empty[b], ((c >> 1) & 1) ^ 1, status) && ok;      // the dQ product of tile c - 2 has read this buffer
                uint8_t* ds = sDS + b * kDS;
#pragma unroll
                for (int c4 = 0; c4 < HC / 8; ++c4)
                    *reinterpret_cast<uint4*>(ds + sw128_chunk_off(r, sb * (HC / 8) + c4)) =
                        make_uint4(dd[c4 * 4], dd[c4 * 4 + 1], dd[c4 * 4 + 2], dd[c4 * 4 + 3]);
                fence_async_smem();
                mbar_arrive(&ds_full[b]);
            }
            // ---- epilogue of the item: this group's 64 of the 128 dQ columns
            const bool full_tile = m.ne == p.TPT && p.G * p.TPT == kTileRows && m.nblk > 0;
            if (m.nblk > 0) {
                ok = mbar_wait(&ds_empty[(c - 1) & 1], ((c - 1) >> 1) & 1, status) && ok;      // the item's last dQ product is done
                tc_fence_after();
            }
            ET* drow = reinterpret_cast<ET*>(p.dq) + ((int64_t)tok * p.Hq + (m.h * p.G + g)) * D + sb * 64;
            uint8_t* stage = sDS + sb * kDS;            // (both dS buffers are free: every dQ product of the item is done)
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t a[32];
                if (m.nblk > 0) {
                    tmem_ld32(tbase + lane_off + cDQ + sb * 64 + c0, a);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) a[i] = 0u;
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 x;
                    x.x = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 0]), __uint_as_float(a[q4 * 8 + 1]));
                    x.y = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 2]), __uint_as_float(a[q4 * 8 + 3]));
                    x.z = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 4]), __uint_as_float(a[q4 * 8 + 5]));
                    x.w = ElemTraits<ET>::pack2(__uint_as_float(a[q4 * 8 + 6]), __uint_as_float(a[q4 * 8 + 7]));
                    const int chunk = (c0 >> 3) + q4;       // 16-byte chunk inside this group's 128-byte half row
                    if (full_tile) {
                        *reinterpret_cast<uint4*>(stage + sw128_chunk_off(r, chunk)) = x;
                    } else if (row_valid && ok) {
                        *reinterpret_cast<uint4*>(drow + chunk * 8) = x;
                    }
                }
            }
            if (m.nblk > 0) {
                tc_fence_before();
                mbar_arrive(dq_free);            // the accumulator may take the next item
                ++qi;
            }
            if (full_tile) {
                fence_async_smem();
                if (sb == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
                else asm volatile("bar.sync 2, 128;" ::: "memory");
                if (quarter == 0 && lane == 0) {
                    if (ok) tma_store_3d(&dqmap, sb * 64, m.tok0, m.h * p.G, smem_u32(stage));
                    bulk_commit();
                    bulk_wait_read0();           // the staging memory is a dS buffer again in the next item
                }
                asm volatile("bar.sync 3, 256;" ::: "memory");
            }
        }
        (void)qi;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, kCols);
}

// dQ of a range-attention backward (head_dim 128).  q / dO strided, dq contiguous [N, Hq, 128].
cudaError_t launch_range_bwd_dq(int dtype, const SelBwdArgs& a, const SelShape& s, const CUtensorMap& kmap, const CUtensorMap& vmap,
                                int* status, cudaStream_t stream) {
    CUtensorMap qmap, domap, dqmap;
    if (make_tile_map_3d_box(&qmap, a.q, dtype, 128, s.N, s.Hq, a.q_sn, a.q_sh, s.TPT, s.G)) return cudaErrorInvalidValue;
    if (make_tile_map_3d_box(&domap, a.d_o, dtype, 128, s.N, s.Hq, a.do_sn, a.do_sh, s.TPT, s.G)) return cudaErrorInvalidValue;
    if (make_tile_map_3d_box(&dqmap, a.dq, dtype, 128, s.N, s.Hq, (int64_t)s.Hq * 128, 128, s.TPT, s.G)) return cudaErrorInvalidValue;
    RangeDqParams p;
    p.cu_q = a.cu; p.cu_k = a.bd.cu_k ? a.bd.cu_k : a.cu; p.kv_lo = a.bd.kv_lo; p.kv_hi = a.bd.kv_hi;
    p.N = s.N; p.Nk = s.Nk; p.B = s.B; p.Hq = s.Hq; p.Hk = s.Hk; p.G = s.G; p.TPT = s.TPT;
    p.scale = a.sm_scale; p.scale_log2 = a.sm_scale * 1.4426950408889634f;
    p.lse = a.lse; p.delta = a.delta; p.dq = a.dq; p.status = status;
    constexpr int smem = 2 * kTileRows * 128 * 2 + kDqStages * 2 * kRdBK * 128 * 2 + 2 * kTileRows * kRdBK * 2 + 256;
    const int64_t max_items = ((s.N + s.TPT - 1) / s.TPT + s.B) * (int64_t)s.Hk;
    int sms = 0;
    if (device_sm_count(&sms) != 0 || sms <= 0) return cudaErrorInvalidValue;
    const unsigned grid = (unsigned)(max_items < sms ? max_items : sms);
    cudaError_t e;
    if (dtype == kBF16) {
        auto kern = range_bwd_dq_dense<__nv_bfloat16>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        prof_begin(FSA_KERNEL_SEL_BWD_DQ_REDUCE, stream);
        kern<<<grid, kDqThreads, smem, stream>>>(p, qmap, domap, kmap, vmap, dqmap);
        prof_end(FSA_KERNEL_SEL_BWD_DQ_REDUCE, stream);
    } else {
        auto kern = range_bwd_dq_dense<__half>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        prof_begin(FSA_KERNEL_SEL_BWD_DQ_REDUCE, stream);
        kern<<<grid, kDqThreads, smem, stream>>>(p, qmap, domap, kmap, vmap, dqmap);
        prof_end(FSA_KERNEL_SEL_BWD_DQ_REDUCE, stream);
    }
    return cudaGetLastError();
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_range_attn_fwd_dense(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q,
                                        const int32_t* cu_seqlens_k, const int32_t* kv_lo, const int32_t* kv_hi, int64_t N, int64_t Nk,
                                        int B, int Hq, int Hk, int D, int dtype, int64_t q_sn, int64_t q_sh, int64_t k_sn, int64_t v_sn,
                                        float sm_scale, void* o, int64_t o_sn, int64_t o_sh, float* lse, int32_t* status, void* stream_) {
    if (N < 0 || Nk < 0 || B < 0 || Hq <= 0 || Hk <= 0 || Hq % Hk != 0) return FSA_ERR_BAD_ARG;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (D != 64 && D != 128) return FSA_ERR_UNSUPPORTED;
    const int G = Hq / Hk;
    if (G > 32) return FSA_ERR_UNSUPPORTED;
    if (!(sm_scale > 0.f)) return FSA_ERR_BAD_ARG;
    if (N == 0 || B == 0) return FSA_OK;
    if (!q || !k || !v || !cu_seqlens_q || !cu_seqlens_k || !kv_hi || !o || !lse || Nk == 0) return FSA_ERR_BAD_ARG;
    if (((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) || ((uintptr_t)o & 15)) return FSA_ERR_BAD_ARG;
    if ((q_sn % 8) || (q_sh % 8) || (k_sn % 8) || (v_sn % 8) || (o_sn % 8) || (o_sh % 8)) return FSA_ERR_BAD_ARG;
    if (k_sn < (int64_t)Hk * D || v_sn < (int64_t)Hk * D) return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    int rc = ensure_context();
    if (rc) return rc;
    const int TPT = (kTileRows / G) & ~3;
    CUtensorMap qmap, kmap, vmap, omap;
    if ((rc = make_tile_map_3d_box(&qmap, q, dtype, D, N, Hq, q_sn, q_sh, TPT, G))) return rc;
    if ((rc = make_tile_map_3d_box(&omap, o, dtype, D, N, Hq, o_sn, o_sh, TPT, G))) return rc;
    if ((rc = make_tile_map(&kmap, k, dtype, Nk, (int64_t)Hk * D, k_sn, 64))) return rc;
    if ((rc = make_tile_map(&vmap, v, dtype, Nk, (int64_t)Hk * D, v_sn, 64))) return rc;
    RangeDenseParams p;
    p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k; p.kv_lo = kv_lo; p.kv_hi = kv_hi;
    p.N = N; p.Nk = Nk; p.B = B; p.Hq = Hq; p.Hk = Hk; p.G = G; p.TPT = TPT;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.o = o; p.o_sn = o_sn; p.o_sh = o_sh; p.lse = lse; p.status = status;
    const int max_tiles = (int)((N + TPT - 1) / TPT) + B;
    cudaStream_t stream = (cudaStream_t)stream_;
    cudaError_t e;
    if (dtype == FSA_DTYPE_BF16)
        e = D == 128 ? launch_rd<128, __nv_bfloat16>(p, qmap, kmap, vmap, omap, max_tiles, stream)
                     : launch_rd<64, __nv_bfloat16>(p, qmap, kmap, vmap, omap, max_tiles, stream);
    else
        e = D == 128 ? launch_rd<128, __half>(p, qmap, kmap, vmap, omap, max_tiles, stream)
                     : launch_rd<64, __half>(p, qmap, kmap, vmap, omap, max_tiles, stream);
    return e == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}
