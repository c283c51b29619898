// Selected-attention backward for sm_100a.
//
// One KV-major kernel does all five products of the backward (the reference runs S and dP
// twice: once in backward_dkdv, fsa/ops/FSA_topk_sparse_attention.py:1548-1712, once in
// dq_compute_kernel, :1120-1247).  For a resident 64-key tile of K and V and a tile of <= 128
// gathered (token, head) rows:
//     S  = Q K^T            dP = dO V^T                       (tcgen05, fp32 in TMEM)
//     P  = exp2(S*scale*log2e - lse)     dS = scale * P * (dP - delta)      (one row per thread)
//     dQ_part = dS K        dK^T += Q^T dS      dV^T += dO^T P
// dK^T / dV^T stay in TMEM while the CTA walks the tiles of the block (all G heads of the group
// accumulate into the same tile; the reference stages [G, N, Hk, d] and sums, :1793-1855) and are
// flushed with fp32 reductions into an accumulator when the block changes.  dQ partials go to a
// per-(token, head, slot) buffer and are summed by a bandwidth-bound kernel (dq_reduce_kernel,
// :1251-1321).  delta = sum_d O*dO is backward_sum_o_do (nsa_ref/ops/topk_sparse_attention.py:198-230).
//
// Blocks larger than 64 keys are walked as BK/64 independent 64-key sub-tiles (the backward has
// no per-block softmax state); a 32-key block is a 64-key tile whose upper half is masked.
#include "sel_launch.cuh"

namespace fsa {

constexpr int kKT = 64;   // keys per backward tile

template <typename ET>
struct SelBwdParams {
    const ET* q;  int64_t q_sn, q_sh;
    const ET* d_o; int64_t do_sn, do_sh;
    const float* lse;      // [Hq, N] log2 units
    const float* delta;    // [Hq, N]
    SelShape s;
    SelIndex ix;
    int nsub;              // 64-key sub-tiles per block
    SelBounds bd;          // visible K/V rows per token
    float scale, scale_log2;
    ET* dq_part;           // [max_tiles * nsub * 128, D] partial dQ rows in tile order (input dtype)
    float* dk_acc;         // [N, Hk, D] fp32, zero-initialised
    float* dv_acc;
};

template <int D>
struct SelBwdCfg {
    static constexpr int DM = D < 128 ? 128 : D;              // rows of dK^T / dV^T handled by the MMA
    static constexpr int kSlabsQ = DM / 64;                   // 64-column slabs of the Q / dO tiles (zero slab for D = 64)
    static constexpr int kK = kKT * D * 2;
    static constexpr int kQ = kTileRows * DM * 2;
    static constexpr int kP = kTileRows * kKT * 2;
    static constexpr int kBytes = 2 * kK + 2 * kQ + 2 * kP + 1024;
    static constexpr int cS = 0, cDP = kKT, cDQ = 0;
    static constexpr int cDK = (2 * kKT > D) ? 2 * kKT : D;
    static constexpr int cDV = cDK + (DM / 128) * kKT;
    static constexpr int kColsUsed = cDV + (DM / 128) * kKT;
    static constexpr uint32_t kCols = kColsUsed <= 256 ? 256 : 512;
};

template <int D, typename ET>
__global__ void __launch_bounds__(128, 1) sel_bwd_main(const SelBwdParams<ET> p, const __grid_constant__ CUtensorMap kmap,
                                                      const __grid_constant__ CUtensorMap vmap) {
    using C = SelBwdCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = smem;
    uint8_t* sV = sK + C::kK;
    uint8_t* sQ = sV + C::kK;
    uint8_t* sDO = sQ + C::kQ;
    uint8_t* sP = sDO + C::kQ;
    uint8_t* sDS = sP + C::kP;
    __shared__ uint64_t bar_kv, bar_a, bar_b;
    __shared__ uint32_t tmem_slot;
    __shared__ uint32_t s_ent[kTileRows];

    const int tid = threadIdx.x, warp = tid >> 5;
    const SelShape& s = p.s;
    int* status = p.ix.header;

    if (tid == 0) {
        mbar_init(&bar_kv, 1);
        mbar_init(&bar_a, 1);
        mbar_init(&bar_b, 1);
        mbar_init_fence();
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, C::kCols);
    if constexpr (D < 128) {
        // zero slab that pads the M dimension of dK^T / dV^T to 128
        for (int i = tid; i < kTileRows * 128 / 16; i += 128) {
            *reinterpret_cast<uint4*>(sQ + kTileRows * 128 + i * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(sDO + kTileRows * 128 + i * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

    const int total = p.ix.header[1] * p.nsub;
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int begin = blockIdx.x * per;
    const int end = min(total, begin + per);

    constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, kKT, false, false);   // Q K^T, dO V^T
    constexpr uint32_t idesc_dq = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);     // dS K
    constexpr uint32_t idesc_dk = umma_idesc(ElemTraits<ET>::kIsBF16, 128, kKT, true, true);    // Q^T dS, dO^T P

    int hg = -1, sub = -1, hg_tiles = 0, hg_first = 0;
    int cur_h = 0, cur_row0 = 0;       // of the accumulators held in TMEM
    bool have_acc = false;
    uint32_t kv_loads = 0;
    bool ok = true;
    int it = 0;

    // dK^T / dV^T accumulators -> global fp32 (thread = d index, registers = keys)
    auto flush = [&]() {
        const int key_lim = min(kKT, s.BK);
#pragma unroll
        for (int mh = 0; mh < C::DM / 128; ++mh) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                float* acc = which == 0 ? p.dk_acc : p.dv_acc;
                const uint32_t col = (which == 0 ? C::cDK : C::cDV) + mh * kKT;
#pragma unroll
                for (int c0 = 0; c0 < kKT; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(tbase + lane_off + col + c0, v);
                    tmem_ld_wait();
                    const int d = mh * 128 + tid;
                    if (d < D) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            int key = c0 + i;
                            int64_t row = (int64_t)cur_row0 + key;
                            if (key < key_lim && row < s.Nk)
                                atomicAdd(acc + (row * s.Hk + cur_h) * D + d, __uint_as_float(v[i]));
                        }
                    }
                }
            }
        }
    };

    for (int item = begin; item < end && ok; ++item, ++it) {
        bool new_kv = false;
        {
            int tl = item / p.nsub;
            if (hg < 0 || tl < hg_first || tl >= hg_first + hg_tiles) {
                hg = load_tile(p.ix, tl).hg;     // items of one key span [first tile, first tile + tiles) * nsub
                const int2 ax = __ldg(p.ix.tile_aux + tl);
                hg_first = ax.x;
                hg_tiles = ax.y;
                sub = -1;
            }
        }
        const int local = item - hg_first * p.nsub;
        const int nsub_i = local / hg_tiles;
        const int tile = local - nsub_i * hg_tiles;
        if (nsub_i != sub) { sub = nsub_i; new_kv = true; }
        const TileInfo ti = load_tile(p.ix, hg_first + tile);
        const int h = ti.h;
        const int row0 = ti.row0 + sub * kKT;
        const int ne = ti.ne;
        const int64_t ebase = (int64_t)(hg_first + tile) * s.TPT;

        // ---- stage 1
        if (new_kv && have_acc) {
            tc_fence_after();
            flush();
            tc_fence_before();
            have_acc = false;
        }
        if (tid < s.TPT) s_ent[tid] = tid < ne ? p.ix.entries[ebase + tid] : 0xFFFFFFFFu;
        if (new_kv && tid == 0) {
            mbar_expect_tx(&bar_kv, (uint32_t)(2 * kKT * D * 2));
#pragma unroll
            for (int b = 0; b < D / 64; ++b) {
                tma_load_2d(smem_u32(sK + b * kKT * 128), &kmap, h * D + b * 64, row0, &bar_kv);
                tma_load_2d(smem_u32(sV + b * kKT * 128), &vmap, h * D + b * 64, row0, &bar_kv);
            }
        }
        __syncthreads();

        // ---- stage 2: gather Q and dO rows
        {
            constexpr int CPR = D / 8;
#pragma unroll 4
            for (int i = tid; i < kTileRows * CPR; i += 128) {
                int r = i / CPR, c = i % CPR;
                int g = r / s.TPT, e = r - g * s.TPT;      // head-major rows, as in the forward
                bool valid = g < s.G && e < ne;
                uint32_t ent = valid ? s_ent[e] : 0u;
                int64_t n = ent >> kSlotBits;
                int hq = h * s.G + (valid ? g : 0);
                uint32_t off = (uint32_t)((c >> 3) * (kTileRows * 128)) + sw128_chunk_off(r, c & 7);
                cp_async16(smem_u32(sQ) + off, p.q + n * p.q_sn + (int64_t)hq * p.q_sh + c * 8, valid);
                cp_async16(smem_u32(sDO) + off, p.d_o + n * p.do_sn + (int64_t)hq * p.do_sh + c * 8, valid);
            }
            cp_async_commit();
        }
        const int r = tid;
        const int g_row = r / s.TPT;
        const int e = r - g_row * s.TPT;
        const bool row_valid = g_row < s.G && e < ne;
        const uint32_t ent = row_valid ? s_ent[e] : 0u;
        const int tok = (int)(ent >> kSlotBits);
        const int hq_row = h * s.G + (row_valid ? g_row : 0);
        float lse_r = 0.f, delta_r = 0.f;
        if (row_valid) {
            lse_r = __ldg(p.lse + (int64_t)hq_row * s.N + tok);
            delta_r = __ldg(p.delta + (int64_t)hq_row * s.N + tok);
        }
        cp_async_wait<0>();
        fence_async_smem();
        tc_fence_before();
        __syncthreads();

        // ---- stage 3: S = Q K^T, dP = dO V^T
        if (tid == 0) {
            if (new_kv) ok = mbar_wait(&bar_kv, kv_loads & 1, status);
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a = smem_u32(sQ + (ks >> 2) * (kTileRows * 128)) + (ks & 3) * 32;
                uint32_t b = smem_u32(sK + (ks >> 2) * (kKT * 128)) + (ks & 3) * 32;
                umma_ss(tbase + C::cS, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(b, 16, 1024), idesc_s, ks > 0);
            }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a = smem_u32(sDO + (ks >> 2) * (kTileRows * 128)) + (ks & 3) * 32;
                uint32_t b = smem_u32(sV + (ks >> 2) * (kKT * 128)) + (ks & 3) * 32;
                umma_ss(tbase + C::cDP, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(b, 16, 1024), idesc_s, ks > 0);
            }
            umma_commit(&bar_a);
        }
        if (new_kv) ++kv_loads;
        ok = mbar_wait(&bar_a, it & 1, status) && ok;
        tc_fence_after();

        // ---- stage 4: P and dS rows -> smem (K-major rows of 64 keys)
        {
            int c_lo = 0, c_hi = 0;   // may be empty: nothing visible
            if (row_valid) visible_cols(p.bd, tok, row0, min(kKT, s.BK), c_lo, c_hi);
#pragma unroll
            for (int c0 = 0; c0 < kKT; c0 += 32) {
                uint32_t sv[32], dv[32];
                tmem_ld32(tbase + lane_off + C::cS + c0, sv);
                tmem_ld32(tbase + lane_off + C::cDP + c0, dv);
                tmem_ld_wait();
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t pp[4], dd[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        int i = ch * 8 + j * 2;
                        float p0 = (c0 + i >= c_lo && c0 + i < c_hi) ? exp2f(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse_r)) : 0.f;
                        float p1 = (c0 + i + 1 >= c_lo && c0 + i + 1 < c_hi) ? exp2f(fmaf(__uint_as_float(sv[i + 1]), p.scale_log2, -lse_r)) : 0.f;
                        float d0 = p0 * (__uint_as_float(dv[i]) - delta_r) * p.scale;
                        float d1 = p1 * (__uint_as_float(dv[i + 1]) - delta_r) * p.scale;
                        pp[j] = ElemTraits<ET>::pack2(p0, p1);
                        dd[j] = ElemTraits<ET>::pack2(d0, d1);
                    }
                    uint32_t off = sw128_chunk_off(r, (c0 >> 3) + ch);
                    *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[0], pp[1], pp[2], pp[3]);
                    *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dd[0], dd[1], dd[2], dd[3]);
                }
            }
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();

        // ---- stage 5: dQ = dS K ; dK^T += Q^T dS ; dV^T += dO^T P
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < kKT / 16; ++ks) {
                uint32_t a = smem_u32(sDS) + ks * 32;
                uint32_t b = smem_u32(sK) + ks * 2048;
                umma_ss(tbase + C::cDQ, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(b, kKT * 128, 1024), idesc_dq, ks > 0);
            }
#pragma unroll
            for (int mh = 0; mh < C::DM / 128; ++mh) {
#pragma unroll
                for (int ks = 0; ks < kTileRows / 16; ++ks) {
                    uint32_t acc = (have_acc || ks > 0) ? 1u : 0u;
                    uint32_t aq = smem_u32(sQ) + mh * 2 * (kTileRows * 128) + ks * 2048;
                    uint32_t ad = smem_u32(sDO) + mh * 2 * (kTileRows * 128) + ks * 2048;
                    uint32_t bs = smem_u32(sDS) + ks * 2048;
                    uint32_t bp = smem_u32(sP) + ks * 2048;
                    umma_ss(tbase + C::cDK + mh * kKT, umma_desc_sw128(aq, kTileRows * 128, 1024),
                            umma_desc_sw128(bs, 8192, 1024), idesc_dk, acc);
                    umma_ss(tbase + C::cDV + mh * kKT, umma_desc_sw128(ad, kTileRows * 128, 1024),
                            umma_desc_sw128(bp, 8192, 1024), idesc_dk, acc);
                }
            }
            umma_commit(&bar_b);
        }
        have_acc = true;
        cur_h = h;
        cur_row0 = row0;
        ok = mbar_wait(&bar_b, it & 1, status) && ok;
        tc_fence_after();

        // ---- stage 6: dQ partial -> global
        {
            const int64_t prow = ((int64_t)(hg_first + tile) * p.nsub + sub) * kTileRows + r;
            uint4* dst = reinterpret_cast<uint4*>(p.dq_part + prow * D);
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tbase + lane_off + C::cDQ + c0, v);
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
    if (have_acc) {
        tc_fence_after();
        flush();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, C::kCols);
}

// delta[hq, n] = sum_d o[n, hq, d] * do[n, hq, d].  D / 8 threads per row (16 bytes of o and of dO each), two rows per
// thread in flight, few registers: the kernel is a pure stream and wants every warp slot of the SM.
template <typename ET>
__global__ void __launch_bounds__(256) sel_bwd_delta(const ET* __restrict__ o, int64_t o_sn, int64_t o_sh,
                                                     const ET* __restrict__ d_o, int64_t do_sn, int64_t do_sh,
                                                     int64_t N, int Hq, int D, float* __restrict__ delta) {
    const int tpr = D >> 3;                                  // threads per row: 8, 16 or 32 (a power of two)
    const int rpc = 256 / tpr;                               // rows per pass of the CTA
    const int part = threadIdx.x & (tpr - 1), rloc = threadIdx.x / tpr;
    const int64_t rows = N * Hq;
    const int64_t row0 = (int64_t)blockIdx.x * (2 * rpc) + rloc;
    uint4 a[2], b[2];
    int64_t nn[2];
    int hh[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int64_t r = row0 + (int64_t)j * rpc;
        a[j] = b[j] = make_uint4(0u, 0u, 0u, 0u);
        nn[j] = 0; hh[j] = 0;
        if (r < rows) {
            // (N * Hq fits in 32 bits for every problem the index build accepts: a 32-bit division, not a 64-bit one)
            const uint32_t n32 = (uint32_t)r / (uint32_t)Hq;
            nn[j] = n32;
            hh[j] = (int)((uint32_t)r - n32 * (uint32_t)Hq);
            a[j] = *reinterpret_cast<const uint4*>(o + nn[j] * o_sn + (int64_t)hh[j] * o_sh + part * 8);
            b[j] = *reinterpret_cast<const uint4*>(d_o + nn[j] * do_sn + (int64_t)hh[j] * do_sh + part * 8);
        }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const uint32_t* ua = &a[j].x;
        const uint32_t* ub = &b[j].x;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 x = ElemTraits<ET>::unpack2(ua[i]);
            float2 y = ElemTraits<ET>::unpack2(ub[i]);
            acc = fmaf(x.x, y.x, acc);
            acc = fmaf(x.y, y.y, acc);
        }
        for (int o_ = tpr >> 1; o_; o_ >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o_);
        if (part == 0 && row0 + (int64_t)j * rpc < rows) delta[(int64_t)hh[j] * N + nn[j]] = acc;
    }
}

// dq[n, hq, :] = sum over usable slots (and sub-tiles) of the partial rows, looked up through
// the `pos` map; one warp per (n, hq)
template <int D, typename ET>
__global__ void __launch_bounds__(256) sel_bwd_dq_reduce(const ET* __restrict__ dq_part, const int* __restrict__ pos, SelShape s,
                                                         int nsub, ET* __restrict__ dq) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= s.N * s.Hq) return;
    // 32-bit division when the row index allows it (a 64-bit one costs about as much as the rest of the prologue)
    const bool small = s.N * s.Hq <= 0x7fffffffll;
    const int n = small ? (int)((unsigned)row / (unsigned)s.Hq) : (int)(row / s.Hq);
    const int hq = (int)(row - (int64_t)n * s.Hq);
    const int h = hq / s.G, g = hq - h * s.G;
    const int* prow = pos + ((int64_t)h * s.N + n) * s.T;
    long long pr0 = -1, pr1 = -1;    // partial row of slot lane / lane + 32 (sub-tile 0)
    if (lane < s.T) {
        int ps = __ldg(prow + lane);
        if (ps >= 0) pr0 = ((long long)(ps / s.TPT) * nsub) * kTileRows + g * s.TPT + ps % s.TPT;
    }
    if (lane + 32 < s.T) {
        int ps = __ldg(prow + lane + 32);
        if (ps >= 0) pr1 = ((long long)(ps / s.TPT) * nsub) * kTileRows + g * s.TPT + ps % s.TPT;
    }
    constexpr int V = D / 32;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    // eight partial rows in flight per warp: all loads of a batch are issued before the first is used
    for (int u_ = 0; u_ < nsub; ++u_) {
        for (int sl0 = 0; sl0 < s.T; sl0 += 8) {
            uint4 x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int sl = sl0 + j;
                const long long pr = __shfl_sync(0xffffffffu, sl < 32 ? pr0 : pr1, sl & 31);
                x[j] = (sl < s.T && pr >= 0) ? ld_row_vec<V, ET>(dq_part + (pr + (long long)u_ * kTileRows) * D + lane * V)
                                             : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) fma_row_vec<V, ET>(acc, x[j], 1.f);
        }
    }
    ET* dst = dq + row * D + lane * V;
    if constexpr (V == 2) {
        *reinterpret_cast<uint32_t*>(dst) = ElemTraits<ET>::pack2(acc[0], acc[1]);
    } else if constexpr (V == 4) {
        uint2 w;
        w.x = ElemTraits<ET>::pack2(acc[0], acc[1]);
        w.y = ElemTraits<ET>::pack2(acc[2], acc[3]);
        *reinterpret_cast<uint2*>(dst) = w;
    } else {
        uint4 w;
        w.x = ElemTraits<ET>::pack2(acc[0], acc[1]);
        w.y = ElemTraits<ET>::pack2(acc[2], acc[3]);
        w.z = ElemTraits<ET>::pack2(acc[4], acc[5]);
        w.w = ElemTraits<ET>::pack2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(dst) = w;
    }
}

// dk / dv of one (kv head, block): the sum, in segment order, of the slabs the pipelined kernel wrote for the block's
// segments, rounded to the output dtype (replaces the `.sum(0)` over the group's copies of the reference,
// fsa/ops/FSA_topk_sparse_attention.py:1854-1855).  Thread = head-dim index; blocks nobody selected keep the zeros
// the caller put there.
template <typename ET>
__global__ void __launch_bounds__(256) sel_bwd_dkdv_reduce(const float* __restrict__ slabs, SelShape s, SelIndex ix,
                                                           ET* __restrict__ dk, ET* __restrict__ dv) {
    constexpr int D = 128, KT = 64;
    const int hg = blockIdx.x;
    if (ix.key_cnt[hg] == 0) return;
    const int h = hg / s.NBmax, gb = hg - h * s.NBmax;
    const int row0 = ix.row0[gb];
    const int seg0 = ix.key_seg[hg], nseg = ix.key_seg[hg + 1] - seg0;
    const int nkeys = min(KT, ix.nrow[gb]);     // rows past the end of the sequence belong to the next sequence's block
    // a warp per K/V row (32 lanes x 16 bytes = the row's 128 floats); the CTA's 8 warps walk the block's rows of dK, then dV,
    // four rows in flight per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float4* base = reinterpret_cast<const float4*>(slabs + (int64_t)seg0 * (2 * KT * D)) + lane;
    constexpr int kSegStride = 2 * KT * D / 4, kRowStride = D / 4;       // in float4
    for (int r0 = warp * 4; r0 < 2 * KT; r0 += 32) {
        float4 acc[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sg = 0; sg < nseg; ++sg) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = r0 + j;                        // row of the slab: which * 64 + key
                v[j] = (r & (KT - 1)) < nkeys ? __ldcs(base + (int64_t)sg * kSegStride + r * kRowStride) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) { acc[j].x += v[j].x; acc[j].y += v[j].y; acc[j].z += v[j].z; acc[j].w += v[j].w; }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = r0 + j, key = r & (KT - 1);
            if (key < nkeys) {
                ET* dst = (r < KT ? dk : dv) + ((int64_t)(row0 + key) * s.Hk + h) * D + lane * 4;
                uint2 w;
                w.x = ElemTraits<ET>::pack2(acc[j].x, acc[j].y);
                w.y = ElemTraits<ET>::pack2(acc[j].z, acc[j].w);
                *reinterpret_cast<uint2*>(dst) = w;
            }
        }
    }
}

// fp32 accumulators -> output dtype
template <typename ET>
__global__ void __launch_bounds__(256) sel_bwd_convert(const float* __restrict__ a, const float* __restrict__ b,
                                                       ET* __restrict__ oa, ET* __restrict__ ob, int64_t n4) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    float4 x = reinterpret_cast<const float4*>(a)[i];
    float4 y = reinterpret_cast<const float4*>(b)[i];
    uint2 u, w;
    u.x = ElemTraits<ET>::pack2(x.x, x.y); u.y = ElemTraits<ET>::pack2(x.z, x.w);
    w.x = ElemTraits<ET>::pack2(y.x, y.y); w.y = ElemTraits<ET>::pack2(y.z, y.w);
    reinterpret_cast<uint2*>(oa)[i] = u;
    reinterpret_cast<uint2*>(ob)[i] = w;
}

template <int D, typename ET>
static cudaError_t launch_sel_bwd(const SelBwdArgs& a, const SelShape& s, const SelIndex& ix, const CUtensorMap& kmap,
                                  const CUtensorMap& vmap, int num_sms, cudaStream_t stream) {
    const int nsub = s.BK > kKT ? s.BK / kKT : 1;
    const int64_t rows = s.N * s.Hq;
    const int64_t kv_elems = s.Nk * s.Hk * (int64_t)D;
    // the gather warps of the pipelined kernel address rows by 32-bit offsets in units of 8 elements
    const bool offsets_fit = ((s.N * a.q_sn + (int64_t)s.Hq * a.q_sh) >> 3) < 0x7fffffffll &&
                             ((s.N * a.do_sn + (int64_t)s.Hq * a.do_sh) >> 3) < 0x7fffffffll;
    const bool pipelined = D == 128 && s.BK <= kKT && a.dqmap && offsets_fit;
    cudaError_t e;
    if (pipelined) {
        // dk / dv rows of blocks that nobody selected stay zero
        e = cudaMemsetAsync(a.dk, 0, kv_elems * sizeof(ET), stream);
        if (e != cudaSuccess) return e;
        e = cudaMemsetAsync(a.dv, 0, kv_elems * sizeof(ET), stream);
    } else {
        e = cudaMemsetAsync(a.dk_acc, 0, kv_elems * 4 * 2, stream);   // dk_acc and dv_acc are adjacent
    }
    if (e != cudaSuccess) return e;
    if (rows > 0) {
        const int64_t rows_per_cta = 2 * (256 / (D / 8));
        unsigned grid = (unsigned)((rows + rows_per_cta - 1) / rows_per_cta);
        sel_bwd_delta<ET><<<grid, 256, 0, stream>>>((const ET*)a.o, a.o_sn, a.o_sh, (const ET*)a.d_o, a.do_sn, a.do_sh,
                                                    s.N, s.Hq, D, a.delta);
    }
    SelBwdParams<ET> p;
    p.q = (const ET*)a.q; p.q_sn = a.q_sn; p.q_sh = a.q_sh;
    p.d_o = (const ET*)a.d_o; p.do_sn = a.do_sn; p.do_sh = a.do_sh;
    p.lse = a.lse; p.delta = a.delta;
    p.s = s; p.ix = ix; p.nsub = nsub; p.bd = a.bd;
    p.scale = a.sm_scale; p.scale_log2 = a.sm_scale * 1.4426950408889634f;
    p.dq_part = (ET*)a.dq_part; p.dk_acc = a.dk_acc; p.dv_acc = a.dv_acc;
    // range attention (every token sees one contiguous range): dQ by the query-tile-major kernel, no partial dQ rows
    const bool dq_dense = pipelined && a.bd.kv_hi != nullptr && s.G <= 32;
    if (pipelined) {
        const int dt = ElemTraits<ET>::kIsBF16 ? (int)kBF16 : (int)kFP16;
        if (dq_dense && rows > 0) {
            e = launch_range_bwd_dq(dt, a, s, kmap, vmap, ix.header, stream);
            if (e != cudaSuccess) return e;
        }
        e = launch_sel_bwd_pipe(dt, a, s, ix, kmap, vmap, *a.dqmap, num_sms, dq_dense, stream);
        if (e != cudaSuccess) return e;
    } else {
        auto kern = sel_bwd_main<D, ET>;
        constexpr int smem = SelBwdCfg<D>::kBytes;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        int per_sm = (int)(512 / SelBwdCfg<D>::kCols);
        int by_smem = (227 * 1024) / (smem + 2048);
        if (by_smem < per_sm) per_sm = by_smem;
        if (per_sm < 1) per_sm = 1;
        prof_begin(2, stream);
        kern<<<num_sms * per_sm, 128, smem, stream>>>(p, kmap, vmap);
        prof_end(2, stream);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    if (rows > 0 && !dq_dense) {
        unsigned grid = (unsigned)((rows + 7) / 8);
        prof_begin(3, stream);
        sel_bwd_dq_reduce<D, ET><<<grid, 256, 0, stream>>>((const ET*)a.dq_part, ix.pos, s, nsub, (ET*)a.dq);
        prof_end(3, stream);
    }
    if (kv_elems > 0) {
        if (pipelined) {
            if constexpr (D == 128)
                sel_bwd_dkdv_reduce<ET><<<(unsigned)(s.Hk * s.NBmax), 256, 0, stream>>>(a.slabs, s, ix, (ET*)a.dk, (ET*)a.dv);
        } else {
            int64_t n4 = kv_elems / 4;
            sel_bwd_convert<ET><<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(a.dk_acc, a.dv_acc, (ET*)a.dk, (ET*)a.dv, n4);
        }
    }
    return cudaGetLastError();
}

cudaError_t dispatch_sel_bwd(int dtype, const SelBwdArgs& a, const SelShape& s, const SelIndex& ix,
                             const CUtensorMap& kmap, const CUtensorMap& vmap, int num_sms, cudaStream_t stream) {
#define FSA_CASE(DD)                                                                                    \
    if (s.D == DD)                                                                                      \
        return dtype == kBF16 ? launch_sel_bwd<DD, __nv_bfloat16>(a, s, ix, kmap, vmap, num_sms, stream) \
                              : launch_sel_bwd<DD, __half>(a, s, ix, kmap, vmap, num_sms, stream);
    FSA_CASE(64) FSA_CASE(128) FSA_CASE(256)
#undef FSA_CASE
    return cudaErrorInvalidValue;
}

}  // namespace fsa
