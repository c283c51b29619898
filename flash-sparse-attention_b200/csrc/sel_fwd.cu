// Selected-attention forward for sm_100a.
//
// Main kernel (replaces forward_kernel_opt and the qk_kernel pre-pass of the reference,
// fsa/ops/FSA_topk_sparse_attention.py:285-566): KV blocks are the outer loop.  A CTA owns a
// contiguous range of tiles; a tile is <= 128 rows = (selecting token, query head of the
// group).  K and V of the block arrive by TMA (128-byte swizzle) and stay resident while the
// CTA walks the block's tiles; the query rows are gathered by token id with 16-byte async
// copies into the same swizzled layout.  S = Q K^T and O = P V run on tcgen05 with TMEM
// accumulators; each thread owns one row of S, so row max / row sum need no shuffles.  The
// kernel writes, per (token, head, slot), an unnormalised partial O (fp32) and the pair
// (m, l) = (row max in log2 units, sum of exp2(s - m)).  No atomics, no cross-block state.
//
// Reduce kernel (replaces reduce_kernel, :139-281): one warp per (token, head) merges the
// <= T partials with 128-bit loads:  M = max m_s, w_s = exp2(m_s - M),
// o = sum w_s O_s / sum w_s l_s,  lse = M + log2 sum w_s l_s   (log2 units, as the reference).
#include "sel_launch.cuh"

namespace fsa {

template <typename ET>
struct SelFwdParams {
    const ET* q;
    int64_t q_sn, q_sh;      // element strides of q[N, Hq, D]
    SelShape s;
    SelIndex ix;
    float scale_log2;        // softmax scale * log2(e)
    float* opart;            // [N, Hq, T, D] fp32
    float2* ml;              // [N, Hq, T]
};

template <int D, int BK>
struct SelFwdSmem {
    static constexpr int kK = BK * D * 2;
    static constexpr int kV = BK * D * 2;
    static constexpr int kQ = kTileRows * D * 2;
    static constexpr int kBytes = kK + kV + kQ + 1024;   // + alignment slack
};

__host__ __device__ constexpr uint32_t tmem_cols_pow2(int c) { return c <= 32 ? 32 : c <= 64 ? 64 : c <= 128 ? 128 : c <= 256 ? 256 : 512; }

template <int D, int BK, typename ET>
__global__ void __launch_bounds__(128, 1) sel_fwd_main(const SelFwdParams<ET> p, const __grid_constant__ CUtensorMap kmap,
                                                      const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = smem;
    uint8_t* sV = sK + SelFwdSmem<D, BK>::kK;
    uint8_t* sQ = sV + SelFwdSmem<D, BK>::kV;
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
        tma_prefetch_desc(&kmap);
        tma_prefetch_desc(&vmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, kCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const uint32_t tS = tbase;            // S (fp32, BK cols); P (packed 16-bit, BK/2 cols) aliases it
    const uint32_t tO = tbase + BK;       // O (fp32, D cols)
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

    const int HG = s.Hk * s.NBmax;
    const int total = p.ix.header[1];
    const int per = (total + gridDim.x - 1) / gridDim.x;
    const int begin = blockIdx.x * per;
    const int end = min(total, begin + per);

    constexpr uint32_t idesc_s = umma_idesc(ElemTraits<ET>::kIsBF16, 128, BK, false, false);
    constexpr uint32_t idesc_o = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);

    int hg = -1, hg_end = 0, hg_begin = 0;
    uint32_t kv_loads = 0;
    bool ok = true;
    int it = 0;
    for (int item = begin; item < end && ok; ++item, ++it) {
        bool new_kv = false;
        if (hg < 0 || item >= hg_end) {
            hg = upper_seg(p.ix.tile_off, HG, item);
            hg_begin = p.ix.tile_off[hg];
            hg_end = p.ix.tile_off[hg + 1];
            new_kv = true;
        }
        const int h = hg / s.NBmax;
        const int gb = hg - h * s.NBmax;
        const int row0 = p.ix.row0[gb];
        const int cnt = p.ix.counts[hg];
        const int e0 = (item - hg_begin) * s.TPT;
        const int ne = min(s.TPT, cnt - e0);
        const int64_t ebase = (int64_t)p.ix.blk_off[hg] + e0;

        // ---- stage 1: entries -> smem; K/V tile by TMA when the block changes
        if (tid < s.TPT) s_ent[tid] = tid < ne ? p.ix.entries[ebase + tid] : 0xFFFFFFFFu;
        if (new_kv && tid == 0) {
            mbar_expect_tx(&bar_kv, (uint32_t)(2 * BK * D * 2));
#pragma unroll
            for (int b = 0; b < D / 64; ++b) {
                tma_load_2d(smem_u32(sK + b * BK * 128), &kmap, h * D + b * 64, row0, &bar_kv);
                tma_load_2d(smem_u32(sV + b * BK * 128), &vmap, h * D + b * 64, row0, &bar_kv);
            }
        }
        __syncthreads();

        // ---- stage 2: gather Q rows (row r = entry r / G, head r % G)
        {
            constexpr int CPR = D / 8;   // 16-byte chunks per row
#pragma unroll 4
            for (int i = tid; i < kTileRows * CPR; i += 128) {
                int r = i / CPR, c = i % CPR;
                int e = r / s.G, g = r - e * s.G;
                bool valid = e < ne;
                uint32_t ent = valid ? s_ent[e] : 0u;
                int64_t n = ent >> kSlotBits;
                const ET* src = p.q + n * p.q_sn + (int64_t)(h * s.G + g) * p.q_sh + c * 8;
                uint32_t dst = smem_u32(sQ + (c >> 3) * (kTileRows * 128)) + sw128_chunk_off(r, c & 7);
                cp_async16(dst, src, valid);
            }
            cp_async_commit();
            cp_async_wait<0>();
            fence_async_smem();
        }
        tc_fence_before();
        __syncthreads();

        // ---- stage 3: S = Q K^T
        if (tid == 0) {
            if (new_kv) {
                ok = mbar_wait(&bar_kv, kv_loads & 1, status);
            }
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

        // ---- stage 4: row softmax statistics, P -> TMEM
        const int r = tid;
        const int e = r / s.G;
        const bool row_valid = e < ne;
        const uint32_t ent = row_valid ? s_ent[e] : 0u;
        const int tok = (int)(ent >> kSlotBits);
        const int slot = (int)(ent & (kMaxTopk - 1));
        const int nvis = row_valid ? min(BK, tok - row0 + 1) : BK;   // causal: key row0 + j <= tok
        float mx = -INFINITY;
#pragma unroll
        for (int c0 = 0; c0 < BK; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tS + lane_off + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (c0 + i < nvis) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
        const float m = mx * p.scale_log2;
        float l = 0.f;
#pragma unroll
        for (int c0 = 0; c0 < BK; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tS + lane_off + c0, v);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float p0 = (c0 + i < nvis) ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -m)) : 0.f;
                float p1 = (c0 + i + 1 < nvis) ? exp2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m)) : 0.f;
                l += p0 + p1;
                pk[i >> 1] = ElemTraits<ET>::pack2(p0, p1);
            }
            tmem_st16(tS + lane_off + (c0 >> 1), pk);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncthreads();

        // ---- stage 5: O = P V   (P from TMEM, V MN-major from smem)
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

        // ---- stage 6: partial O and (m, l) -> global, indexed by (token, head, slot)
        {
            const int hq = h * s.G + (r - e * s.G);
            const int64_t prow = ((int64_t)tok * s.Hq + hq) * s.T + slot;
            if (row_valid) p.ml[prow] = make_float2(m, l);
            float4* dst = reinterpret_cast<float4*>(p.opart + prow * D);
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tO + lane_off + c0, v);
                tmem_ld_wait();
                if (row_valid) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dst[(c0 >> 2) + i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                         __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                }
            }
        }
        tc_fence_before();
        // make every thread see the same `ok` so the loop exits together
        ok = __syncthreads_and(ok);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, kCols);
}

// ------------------------------------------------------------------------------------------
template <int D, typename ET>
__global__ void __launch_bounds__(256) sel_fwd_reduce(const float* __restrict__ opart, const float2* __restrict__ ml,
                                                      const int* __restrict__ topk_idx, const int* __restrict__ cu,
                                                      SelShape s, ET* __restrict__ o, int64_t o_sn, int64_t o_sh,
                                                      float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // n * Hq + hq
    if (row >= s.N * s.Hq) return;
    const int n = (int)(row / s.Hq), hq = (int)(row % s.Hq);
    const int h = hq / s.G;
    const int* idrow = topk_idx + ((int64_t)h * s.N + n) * s.T;
    // lane handles slots lane and lane + 32
    float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
    int r0;
    if (lane < s.T && entry_block(cu, s.B, s.BK, n, __ldg(idrow + lane), &r0) >= 0) {
        float2 v = ml[row * s.T + lane];
        m0 = v.x; l0 = v.y;
    }
    if (lane + 32 < s.T && entry_block(cu, s.B, s.BK, n, __ldg(idrow + lane + 32), &r0) >= 0) {
        float2 v = ml[row * s.T + lane + 32];
        m1 = v.x; l1 = v.y;
    }
    float M = fmaxf(m0, m1);
#pragma unroll
    for (int o_ = 16; o_; o_ >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o_));
    float w0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M);
    float w1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - M);
    float L = w0 * l0 + w1 * l1;
#pragma unroll
    for (int o_ = 16; o_; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);

    constexpr int V = D / 32;   // floats per lane
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    const float* base = opart + row * s.T * D + lane * V;
    for (int sl = 0; sl < s.T; ++sl) {
        float w = __shfl_sync(0xffffffffu, sl < 32 ? w0 : w1, sl & 31);
        if (w == 0.f) continue;
        const float* src = base + (int64_t)sl * D;
        if constexpr (V == 4) {
            float4 x = *reinterpret_cast<const float4*>(src);
            acc[0] = fmaf(w, x.x, acc[0]); acc[1] = fmaf(w, x.y, acc[1]);
            acc[2] = fmaf(w, x.z, acc[2]); acc[3] = fmaf(w, x.w, acc[3]);
        } else if constexpr (V == 2) {
            float2 x = *reinterpret_cast<const float2*>(src);
            acc[0] = fmaf(w, x.x, acc[0]); acc[1] = fmaf(w, x.y, acc[1]);
        } else {
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                float4 x = *reinterpret_cast<const float4*>(src + i);
                acc[i] = fmaf(w, x.x, acc[i]); acc[i + 1] = fmaf(w, x.y, acc[i + 1]);
                acc[i + 2] = fmaf(w, x.z, acc[i + 2]); acc[i + 3] = fmaf(w, x.w, acc[i + 3]);
            }
        }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    ET* dst = o + (int64_t)n * o_sn + (int64_t)hq * o_sh + lane * V;
    if constexpr (V == 2) {
        *reinterpret_cast<uint32_t*>(dst) = ElemTraits<ET>::pack2(acc[0] * inv, acc[1] * inv);
    } else {
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            uint2 u;
            u.x = ElemTraits<ET>::pack2(acc[i] * inv, acc[i + 1] * inv);
            u.y = ElemTraits<ET>::pack2(acc[i + 2] * inv, acc[i + 3] * inv);
            *reinterpret_cast<uint2*>(dst + i) = u;
        }
    }
    if (lane == 0) lse[(int64_t)hq * s.N + n] = L > 0.f ? M + log2f(L) : -INFINITY;
}

// ------------------------------------------------------------------------------------------
template <int D, int BK, typename ET>
cudaError_t launch_sel_fwd(const SelFwdParams<ET>& p, const CUtensorMap& kmap, const CUtensorMap& vmap,
                           const int* topk_idx, const int* cu, ET* o, int64_t o_sn, int64_t o_sh, float* lse,
                           int num_sms, cudaStream_t stream) {
    auto kern = sel_fwd_main<D, BK, ET>;
    constexpr int smem = SelFwdSmem<D, BK>::kBytes;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    constexpr int tmem_per_cta = (int)tmem_cols_pow2(BK + D);
    int by_tmem = 512 / tmem_per_cta;
    int by_smem = (227 * 1024) / (smem + 2048);
    int per_sm = by_tmem < by_smem ? by_tmem : by_smem;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    prof_begin(0, stream);
    kern<<<num_sms * per_sm, 128, smem, stream>>>(p, kmap, vmap);
    prof_end(0, stream);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    int64_t rows = p.s.N * p.s.Hq;
    if (rows > 0) {
        unsigned grid = (unsigned)((rows + 7) / 8);
        prof_begin(1, stream);
        sel_fwd_reduce<D, ET><<<grid, 256, 0, stream>>>(p.opart, p.ml, topk_idx, cu, p.s, o, o_sn, o_sh, lse);
        prof_end(1, stream);
    }
    return cudaGetLastError();
}

template <typename ET>
static cudaError_t dispatch_typed(const void* q, int64_t q_sn, int64_t q_sh, const SelShape& s, const SelIndex& ix,
                                  float sm_scale, float* opart, float2* ml, const CUtensorMap& kmap,
                                  const CUtensorMap& vmap, const int* topk_idx, const int* cu, void* o, int64_t o_sn,
                                  int64_t o_sh, float* lse, int num_sms, cudaStream_t stream) {
    SelFwdParams<ET> p;
    p.q = (const ET*)q; p.q_sn = q_sn; p.q_sh = q_sh;
    p.s = s; p.ix = ix;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.opart = opart; p.ml = ml;
#define FSA_CASE(DD, BB)                                                                                         \
    if (s.D == DD && s.BK == BB)                                                                                 \
        return launch_sel_fwd<DD, BB, ET>(p, kmap, vmap, topk_idx, cu, (ET*)o, o_sn, o_sh, lse, num_sms, stream);
    FSA_CASE(64, 32) FSA_CASE(64, 64) FSA_CASE(64, 128) FSA_CASE(64, 256)
    FSA_CASE(128, 32) FSA_CASE(128, 64) FSA_CASE(128, 128) FSA_CASE(128, 256)
    FSA_CASE(256, 32) FSA_CASE(256, 64) FSA_CASE(256, 128)
#undef FSA_CASE
    return cudaErrorInvalidValue;
}

cudaError_t dispatch_sel_fwd(int dtype, const void* q, int64_t q_sn, int64_t q_sh, const SelShape& s,
                             const SelIndex& ix, float sm_scale, float* opart, float2* ml, const CUtensorMap& kmap,
                             const CUtensorMap& vmap, const int* topk_idx, const int* cu, void* o, int64_t o_sn,
                             int64_t o_sh, float* lse, int num_sms, cudaStream_t stream) {
    if (dtype == kBF16)
        return dispatch_typed<__nv_bfloat16>(q, q_sn, q_sh, s, ix, sm_scale, opart, ml, kmap, vmap, topk_idx, cu, o, o_sn,
                                             o_sh, lse, num_sms, stream);
    return dispatch_typed<__half>(q, q_sn, q_sh, s, ix, sm_scale, opart, ml, kmap, vmap, topk_idx, cu, o, o_sn, o_sh, lse,
                                  num_sms, stream);
}

}  // namespace fsa
