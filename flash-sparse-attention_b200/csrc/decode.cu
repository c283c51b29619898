// One-step NSA decode kernels: bandwidth-bound attention of ONE query token per sequence over
// ranges of K/V cache rows, split into chunks so that a small batch still fills the GPU, with
// partial (o, m, l) results merged by log-sum-exp.  The same merge combines the partials of
// different GPUs when the KV sequence is sharded.
//
// Replaces forward_kernel_decode / score_kernel_decode of the reference
// (fsa_preview/ops/compressed_attention_decode.py:361-592), its reuse of the prefill kernel for the
// selected branch (fsa_preview/ops/selected_attention_decode.py:8-42) and the flash-attn call for the
// window (fsa_preview/module/fsa_decode.py:175-185).  Semantics: the decoded token is the LAST token
// of its sequence and gets exactly what the prefill path computes for that row.
#include "../../include/fsa_sm100.h"
#include "sm100_prims.cuh"

namespace fsa {

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int box_rows);

// Set (atomicMax) by a decode kernel whose bounded wait ran out; read with fsa_decode_read_status.
static __device__ int g_decode_status;

struct DecodeParams {
    const void* q;          // [B, Hq, D]
    const void* k;          // [rows, Hk, D] (row stride kv_sn elements, head stride D)
    const void* v;
    int64_t kv_sn;
    const int* rng_lo;      // [B, Hk, R] first row of range r (global), or -1
    const int* rng_hi;      // [B, Hk, R] one past the last row
    int B, Hq, Hk, R, chunk, nchunk;   // P = R * nchunk partials per (b, head)
    float scale_log2;
    float* o_part;          // [B, Hq, P, D]
    float2* ml;             // [B, Hq, P]
    float* scores;          // optional [B, Hk, scores_ld]: scaled logits (log2 units) of the group's FIRST head, range 0 only
    int64_t scores_ld;
    int nst;                // pipeline stages of the TMA kernel
    int rpp, NP;            // ranges per partial (one online softmax over rpp consecutive ranges), partial groups = ceil(R / rpp)
};

// m16n8k16 tensor-core step on register fragments (the legacy warp-level path: this kernel is bound by HBM, the
// tensor work is a few percent of a step; what matters is that the per-key instruction count stays far below the
// issue budget of a memory-bound SM, which scalar FMAs do not manage for GQA groups of 4 and more).
template <typename ET>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (ElemTraits<ET>::kIsBF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// The same partial attention with the K/V rows of the chunk streamed by TMA: a producer warp keeps `nst` stages of
// 64 keys (K and V, 128-byte swizzled 64-column halves) in flight on full/empty mbarriers, so the bytes in flight per
// SM do not depend on registers or occupancy; the four consumer warps each take 16 keys of a stage, read their MMA
// fragments with ldmatrix (transposed for V) and keep the online softmax in registers.  Every wait is bounded.
constexpr int kDecKT = 64;
template <int D, bool HI, typename ET>
__global__ void __launch_bounds__(160) decode_partial_tma(const DecodeParams p, const __grid_constant__ CUtensorMap kmap,
                                                          const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ __align__(1024) unsigned char dsm_raw[];
    constexpr int HALF_BYTES = 64 * 128;                 // one 64-column half of 64 rows
    constexpr int KV_BYTES = (D / 64) * HALF_BYTES;
    constexpr int STAGE_BYTES = 2 * KV_BYTES;
    constexpr int NK = D / 16;                           // k-steps of Q K^T
    constexpr int NO = D / 8;                            // 8-column output tiles of P V
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(dsm_raw) + 1023) & ~uintptr_t(1023));
    const int nst = p.nst;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + (size_t)nst * STAGE_BYTES);
    uint64_t* empty = full + 4;
    float* smm = reinterpret_cast<float*>(empty + 4);    // [4][16]
    float* sll = smm + 64;
    float* so = reinterpret_cast<float*>(base);          // [4][G][D], aliases stage 0 after the loop

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const int G = p.Hq / p.Hk;
    const int c = blockIdx.x % p.nchunk;
    const int pr = (blockIdx.x / p.nchunk) % p.NP;
    const int h = (blockIdx.x / (p.nchunk * p.NP)) % p.Hk;
    const int b = blockIdx.x / (p.nchunk * p.NP * p.Hk);
    const int P = p.NP * p.nchunk, pidx = pr * p.nchunk + c;
    const int j0 = pr * p.rpp, j1 = min(p.R, j0 + p.rpp);
    const int* rlo = p.rng_lo + ((int64_t)b * p.Hk + h) * p.R;
    const int* rhi = p.rng_hi + ((int64_t)b * p.Hk + h) * p.R;
    // rows [lo, lo + n) of range j that fall into this CTA's chunk
    auto bounds = [&](int j, int& lo, int& n) {
        const int lo_r = rlo[j], hi_r = rhi[j];
        lo = lo_r + c * p.chunk;
        n = lo_r < 0 ? 0 : max(min(hi_r, lo + p.chunk) - lo, 0);
    };
    const int64_t pbase = ((int64_t)b * p.Hq + h * G) * P + pidx;
    int total = 0;
    for (int j = j0; j < j1; ++j) {
        int lo, n;
        bounds(j, lo, n);
        total += n;
    }
    if (total == 0) {
        if (tid < G) p.ml[pbase + (int64_t)tid * P] = make_float2(-INFINITY, 0.f);
        return;
    }
    if (tid == 0) {
        for (int s = 0; s < nst; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 4); }
        mbar_init_fence();
    }
    __syncthreads();
    const uint32_t sbase = smem_u32(base);
    float acc[NO][4];
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    if (warp == 4) {
        if (elect_one()) {
            int it = 0;
            bool ok = true;
            for (int j = j0; j < j1 && ok; ++j) {
                int lo, n;
                bounds(j, lo, n);
                for (int i = 0; i * kDecKT < n; ++i, ++it) {
                    const int s = it % nst;
                    if (it >= nst && !mbar_wait(&empty[s], ((it / nst) - 1) & 1, &g_decode_status)) { ok = false; break; }
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    const uint32_t kb = sbase + s * STAGE_BYTES;
#pragma unroll
                    for (int hf = 0; hf < D / 64; ++hf) {
                        tma_load_2d(kb + hf * HALF_BYTES, &kmap, h * D + hf * 64, lo + i * kDecKT, &full[s]);
                        tma_load_2d(kb + KV_BYTES + hf * HALF_BYTES, &vmap, h * D + hf * 64, lo + i * kDecKT, &full[s]);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        uint32_t qf[NK][2], qh[NK][2];
        {
            const ET* q = (const ET*)p.q + ((int64_t)b * p.Hq + h * G) * D;
#pragma unroll
            for (int kk = 0; kk < NK; ++kk) {
                qf[kk][0] = gid < G ? *reinterpret_cast<const uint32_t*>(q + gid * D + kk * 16 + tig * 2) : 0u;
                qf[kk][1] = gid < G ? *reinterpret_cast<const uint32_t*>(q + gid * D + kk * 16 + 8 + tig * 2) : 0u;
                qh[kk][0] = (HI && gid + 8 < G) ? *reinterpret_cast<const uint32_t*>(q + (gid + 8) * D + kk * 16 + tig * 2) : 0u;
                qh[kk][1] = (HI && gid + 8 < G) ? *reinterpret_cast<const uint32_t*>(q + (gid + 8) * D + kk * 16 + 8 + tig * 2) : 0u;
            }
        }
#pragma unroll
        for (int i = 0; i < NO; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        const bool want_scores = p.scores != nullptr && p.rpp == 1 && pr == 0 && gid == 0;
        const int lrow = lane & 7, lmat = lane >> 3;
        int it = 0;
        bool ok_wait = true;
        for (int j = j0; j < j1 && ok_wait; ++j) {
        int lo, n;
        bounds(j, lo, n);
        float* srow = want_scores ? p.scores + ((int64_t)b * p.Hk + h) * p.scores_ld + c * p.chunk : nullptr;
        for (int i = 0; i * kDecKT < n; ++i, ++it) {
            const int s = it % nst;
            if (!mbar_wait(&full[s], (it / nst) & 1, &g_decode_status)) { ok_wait = false; break; }
            const int k0 = i * kDecKT + warp * 16;               // first key of this warp's tile
            if (k0 < n) {
                const uint32_t kb = sbase + s * STAGE_BYTES, vb = kb + KV_BYTES;
                float sc[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
                    const int row = warp * 16 + nt * 8 + lrow;
#pragma unroll
                    for (int c0 = 0; c0 < D / 8; c0 += 4) {
                        const int cg = c0 + lmat;
                        uint32_t r0, r1, r2, r3;
                        ldsm_x4(kb + (cg >> 3) * HALF_BYTES + row * 128 + (((cg & 7) ^ (row & 7)) << 4), r0, r1, r2, r3);
                        mma16816<ET>(sc[nt], qf[c0 / 2][0], qh[c0 / 2][0], qf[c0 / 2][1], qh[c0 / 2][1], r0, r1);
                        mma16816<ET>(sc[nt], qf[c0 / 2 + 1][0], qh[c0 / 2 + 1][0], qf[c0 / 2 + 1][1], qh[c0 / 2 + 1][1], r2, r3);
                    }
                }
                float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = k0 + nt * 8 + tig * 2 + e;
                        const bool ok = key < n;
                        sc[nt][e] = ok ? sc[nt][e] * p.scale_log2 : -INFINITY;
                        sc[nt][2 + e] = ok ? sc[nt][2 + e] * p.scale_log2 : -INFINITY;
                        if (want_scores && ok) srow[key] = sc[nt][e];
                        tmax0 = fmaxf(tmax0, sc[nt][e]);
                        tmax1 = fmaxf(tmax1, sc[nt][2 + e]);
                    }
                tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
                tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
                if (HI) {
                    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
                    tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
                }
                const float mn0 = fmaxf(m0, tmax0), mn1 = HI ? fmaxf(m1, tmax1) : m1;
                if (__any_sync(0xffffffffu, mn0 > m0 || (HI && mn1 > m1))) {
                    const float a0 = exp2f(m0 - mn0), a1 = HI ? exp2f(m1 - mn1) : 1.f;
                    l0 *= a0;
                    l1 *= a1;
#pragma unroll
                    for (int t = 0; t < NO; ++t) {
                        acc[t][0] *= a0; acc[t][1] *= a0;
                        if (HI) { acc[t][2] *= a1; acc[t][3] *= a1; }
                    }
                    m0 = mn0;
                    m1 = mn1;
                }
                uint32_t pa[4];
                {
                    float e00 = exp2f(sc[0][0] - m0), e01 = exp2f(sc[0][1] - m0), e10 = exp2f(sc[1][0] - m0), e11 = exp2f(sc[1][1] - m0);
                    l0 += e00 + e01 + e10 + e11;
                    pa[0] = ElemTraits<ET>::pack2(e00, e01);
                    pa[2] = ElemTraits<ET>::pack2(e10, e11);
                    if (HI) {
                        float f00 = exp2f(sc[0][2] - m1), f01 = exp2f(sc[0][3] - m1), f10 = exp2f(sc[1][2] - m1), f11 = exp2f(sc[1][3] - m1);
                        l1 += f00 + f01 + f10 + f11;
                        pa[1] = ElemTraits<ET>::pack2(f00, f01);
                        pa[3] = ElemTraits<ET>::pack2(f10, f11);
                    } else {
                        pa[1] = pa[3] = 0u;
                    }
                }
                {
                    const int row = warp * 16 + (lmat & 1) * 8 + lrow;
#pragma unroll
                    for (int c0 = 0; c0 < D / 8; c0 += 2) {
                        const int cg = c0 + (lmat >> 1);
                        uint32_t r0, r1, r2, r3;
                        ldsm_x4_trans(vb + (cg >> 3) * HALF_BYTES + row * 128 + (((cg & 7) ^ (row & 7)) << 4), r0, r1, r2, r3);
                        mma16816<ET>(acc[c0], pa[0], pa[1], pa[2], pa[3], r0, r1);
                        mma16816<ET>(acc[c0 + 1], pa[0], pa[1], pa[2], pa[3], r2, r3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
    __syncthreads();                                     // every stage has been consumed: stage memory is free
    if (warp < 4) {
#pragma unroll
        for (int half = 0; half < (HI ? 2 : 1); ++half) {
            const int g = gid + half * 8;
            if (g < G) {
                float* dst = so + ((size_t)warp * G + g) * D;
#pragma unroll
                for (int t = 0; t < NO; ++t)
                    *reinterpret_cast<float2*>(dst + t * 8 + tig * 2) = make_float2(acc[t][half * 2], acc[t][half * 2 + 1]);
                if (tig == 0) {
                    smm[warp * 16 + g] = half ? m1 : m0;
                    sll[warp * 16 + g] = half ? l1 : l0;
                }
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < G * D; i += 160) {
        const int g = i / D;
        const float M = fmaxf(fmaxf(smm[g], smm[16 + g]), fmaxf(smm[32 + g], smm[48 + g]));
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = smm[w * 16 + g];
            if (mw > -INFINITY) o += exp2f(mw - M) * so[(size_t)w * G * D + i];
        }
        p.o_part[(pbase + (int64_t)g * P) * D + (i - g * D)] = o;
    }
    if (tid < G) {
        const int g = tid;
        const float M = fmaxf(fmaxf(smm[g], smm[16 + g]), fmaxf(smm[32 + g], smm[48 + g]));
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = smm[w * 16 + g];
            if (mw > -INFINITY) L += exp2f(mw - M) * sll[w * 16 + g];
        }
        p.ml[pbase + (int64_t)g * P] = make_float2(M, L);
    }
}

// o[row, :] = sum_p exp2(m_p - M) o_p / sum_p exp2(m_p - M) l_p ; lse = M + log2(...).  One warp per row; a lane owns 4
// consecutive columns per 128-column slab and keeps several 128-bit loads in flight.
template <typename OT>
__device__ __forceinline__ void store4(OT* dst, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
    uint2 u = make_uint2(ElemTraits<__nv_bfloat16>::pack2(v.x, v.y), ElemTraits<__nv_bfloat16>::pack2(v.z, v.w));
    *reinterpret_cast<uint2*>(dst) = u;
}
template <> __device__ __forceinline__ void store4<__half>(__half* dst, float4 v) {
    uint2 u = make_uint2(ElemTraits<__half>::pack2(v.x, v.y), ElemTraits<__half>::pack2(v.z, v.w));
    *reinterpret_cast<uint2*>(dst) = u;
}

template <typename OT>
__global__ void __launch_bounds__(256) lse_merge_kernel(const float* __restrict__ o_part, const float2* __restrict__ ml, int64_t rows, int P,
                                                        int PS, int D, OT* __restrict__ o, float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float2* mlr = ml + row * PS;
    float M = -INFINITY;
    for (int i = lane; i < P; i += 32) {
        float2 v = mlr[i];
        if (v.y > 0.f) M = fmaxf(M, v.x);
    }
#pragma unroll
    for (int o_ = 16; o_; o_ >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o_));
    float L = 0.f;
    for (int i = lane; i < P; i += 32) {
        float2 v = mlr[i];
        if (v.y > 0.f) L += exp2f(v.x - M) * v.y;
    }
#pragma unroll
    for (int o_ = 16; o_; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const float* src = o_part + row * PS * D;
    for (int d = lane * 4; d < D; d += 128) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int i = 0;
        for (; i + 4 <= P; i += 4) {
            float4 x[4];
            float w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 v = mlr[i + j];
                w[j] = v.y > 0.f ? exp2f(v.x - M) : 0.f;
                x[j] = v.y > 0.f ? *reinterpret_cast<const float4*>(src + (int64_t)(i + j) * D + d) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc.x = fmaf(w[j], x[j].x, acc.x); acc.y = fmaf(w[j], x[j].y, acc.y);
                acc.z = fmaf(w[j], x[j].z, acc.z); acc.w = fmaf(w[j], x[j].w, acc.w);
            }
        }
        for (; i < P; ++i) {
            const float2 v = mlr[i];
            if (v.y > 0.f) {
                const float w = exp2f(v.x - M);
                const float4 x = *reinterpret_cast<const float4*>(src + (int64_t)i * D + d);
                acc.x = fmaf(w, x.x, acc.x); acc.y = fmaf(w, x.y, acc.y); acc.z = fmaf(w, x.z, acc.z); acc.w = fmaf(w, x.w, acc.w);
            }
        }
        store4<OT>(o + row * D + d, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
    }
    if (lane == 0 && lse) lse[row] = L > 0.f ? M + log2f(L) : -INFINITY;
}

// Last kernel of a one-GPU decode step: merges the selected-block partials [0, ns) and the window partials [ns, ns + nw)
// of every (sequence, query head) row and mixes the three branches with the sequence's gates, out = g0 o_cmp + g1 o_sel
// + g2 o_win.  o_sel and o_win are rounded to the output type before the mix, as the separate merge + gate_mix kernels do.
// One warp per row; a lane owns 4 consecutive columns per 128-column slab.
template <typename ET>
__global__ void __launch_bounds__(256) decode_finish_kernel(const float* __restrict__ o_part, const float2* __restrict__ ml, int64_t rows,
                                                            int ns, int nw, int PS, int D, int Hq, const ET* __restrict__ o_cmp,
                                                            const ET* __restrict__ gate, ET* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t b = row / Hq;
    const float g0 = (float)gate[b * 3], g1 = (float)gate[b * 3 + 1], g2 = (float)gate[b * 3 + 2];
    const float2* mlr = ml + row * PS;
    const float* src = o_part + row * PS * D;
    float M[2], inv[2];
#pragma unroll
    for (int seg = 0; seg < 2; ++seg) {
        const int p0 = seg ? ns : 0, pn = seg ? nw : ns;
        float m = -INFINITY;
        for (int i = lane; i < pn; i += 32) {
            float2 v = mlr[p0 + i];
            if (v.y > 0.f) m = fmaxf(m, v.x);
        }
#pragma unroll
        for (int o_ = 16; o_; o_ >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o_));
        float L = 0.f;
        for (int i = lane; i < pn; i += 32) {
            float2 v = mlr[p0 + i];
            if (v.y > 0.f) L += exp2f(v.x - m) * v.y;
        }
#pragma unroll
        for (int o_ = 16; o_; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);
        M[seg] = m;
        inv[seg] = L > 0.f ? 1.f / L : 0.f;
    }
    for (int d = lane * 4; d < D; d += 128) {
        float4 acc[2];
#pragma unroll
        for (int seg = 0; seg < 2; ++seg) {
            const int p0 = seg ? ns : 0, pn = seg ? nw : ns;
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int i = 0; i < pn; ++i) {
                const float2 v = mlr[p0 + i];
                if (v.y > 0.f) {
                    const float w = exp2f(v.x - M[seg]);
                    const float4 x = *reinterpret_cast<const float4*>(src + (int64_t)(p0 + i) * D + d);
                    a.x = fmaf(w, x.x, a.x); a.y = fmaf(w, x.y, a.y); a.z = fmaf(w, x.z, a.z); a.w = fmaf(w, x.w, a.w);
                }
            }
            // round to the output type as the unfused path does
            const uint32_t lo = ElemTraits<ET>::pack2(a.x * inv[seg], a.y * inv[seg]), hi = ElemTraits<ET>::pack2(a.z * inv[seg], a.w * inv[seg]);
            const float2 f0 = ElemTraits<ET>::unpack2(lo), f1 = ElemTraits<ET>::unpack2(hi);
            acc[seg] = make_float4(f0.x, f0.y, f1.x, f1.y);
        }
        const uint2 cu_ = *reinterpret_cast<const uint2*>(o_cmp + row * D + d);
        const float2 c0 = ElemTraits<ET>::unpack2(cu_.x), c1 = ElemTraits<ET>::unpack2(cu_.y);
        uint2 o;
        o.x = ElemTraits<ET>::pack2(g0 * c0.x + g1 * acc[0].x + g2 * acc[1].x, g0 * c0.y + g1 * acc[0].y + g2 * acc[1].y);
        o.y = ElemTraits<ET>::pack2(g0 * c1.x + g1 * acc[0].z + g2 * acc[1].z, g0 * c1.y + g1 * acc[0].w + g2 * acc[1].w);
        *reinterpret_cast<uint2*>(out + row * D + d) = o;
    }
}

// Top-k block ids of the decoded token of every sequence from its compressed-branch logits.
// Same rule as select_topk_kernel (select_topk.cu) for the single row t = seq_len - 1.
struct DecodeTopkParams {
    const float* scores;     // [B, Hk, ld] scaled logits (log2 units) of the group's first head
    int64_t ld;
    int shard_len;           // compressed index c lives in shard c / shard_len at column c % shard_len
    int64_t shard_stride;    // elements between the score buffers of consecutive shards
    const float* lse;        // [B, Hq]
    const int* seq_len;      // [B] tokens in the sequence including the decoded one
    const int* ncmp;         // [B] compressed tokens visible
    int B, Hk, Hq, G;
    int ks, stride, BK, init_blocks, local_blocks, T;
    int nw;
    float w[16];
    int max_blocks;
    int32_t* out;            // [B, Hk, T]
};

__global__ void __launch_bounds__(256) decode_topk_kernel(const DecodeTopkParams p) {
    extern __shared__ float tsm[];
    float* bs = tsm;                                         // [max_blocks] bf16-rounded block scores
    int* sel = reinterpret_cast<int*>(bs + p.max_blocks);    // [64] winners in selection order
    __shared__ float wbest[8];
    __shared__ int wbi[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x / p.Hk, h = blockIdx.x % p.Hk;
    const int t = p.seq_len[b] - 1;
    const int ncmp = p.ncmp[b];
    const float lse = p.lse[(int64_t)b * p.Hq + h * p.G];
    const float* row = p.scores + ((int64_t)b * p.Hk + h) * p.ld;
    const int bq = t / p.BK;
    const int nb = t >= 0 ? min(bq + 1, p.max_blocks) : 0;
    const int bstride = p.BK / p.stride, pad = p.ks / p.stride - 1;
    // probabilities of the compressed tokens the candidate blocks can touch, staged in shared memory with coalesced
    // loads (eight in flight per thread); then every block sums its few neighbours
    float* pv = reinterpret_cast<float*>(sel + 64);
    const int cmax = min(ncmp, nb * bstride + p.nw);
    for (int c0 = 0; c0 < cmax; c0 += 2048) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * 256 + tid;
            v[j] = c < cmax ? row[(int64_t)(c / p.shard_len) * p.shard_stride + c % p.shard_len] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * 256 + tid;
            if (c < cmax) pv[c] = exp2f(v[j] - lse);
        }
    }
    __syncthreads();
    for (int blk = tid; blk < nb; blk += 256) {
        float s = 0.f;
        for (int o = 0; o < p.nw; ++o) {
            int c = blk * bstride - pad + o;
            float v = (c >= 0 && c < cmax) ? pv[c] : 0.f;
            s += v * p.w[o];
        }
        if (blk < p.init_blocks || (bq >= blk && bq < blk + p.local_blocks)) s = INFINITY;
        bs[blk] = __bfloat162float(__float2bfloat16(s));
    }
    __syncthreads();
    const int nsel = min(p.T, nb);
    for (int r = 0; r < nsel; ++r) {
        float best = -INFINITY; int bi = 0x7fffffff;
        for (int blk = tid; blk < nb; blk += 256) {
            float v = bs[blk];
            if (v > best || (v == best && blk < bi)) { best = v; bi = blk; }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { wbest[warp] = best; wbi[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
#pragma unroll
            for (int w = 1; w < 8; ++w)
                if (wbest[w] > best || (wbest[w] == best && wbi[w] < bi)) { best = wbest[w]; bi = wbi[w]; }
            sel[r] = bi;
            bs[bi] = -INFINITY;      // taken (a block whose score is -inf can only win once nothing else is left)
        }
        __syncthreads();
    }
    int32_t* out = p.out + ((int64_t)b * p.Hk + h) * p.T;
    for (int i = tid; i < p.T; i += 256)
        if (i >= nsel) out[i] = -1;
    for (int i = tid; i < nsel; i += 256) {
        int v = sel[i], rank = 0;
        for (int j = 0; j < nsel; ++j) rank += sel[j] < v;
        out[rank] = v;
    }
}

// Row ranges of the selected blocks and of the sliding window of the decoded token (t = seq_len - 1),
// clipped to the tokens [shard_lo, shard_hi) that this GPU stores.  Token `tok` of sequence b sits in cache
// row seq_row0[b] + tok - shard_lo.  Ranges 0..T-1: block ids of topk_idx; ranges T..T+NW-1: the window
// [max(0, t - window), t] cut into pieces of `piece` rows.
__global__ void decode_ranges_kernel(const int32_t* __restrict__ topk_idx, const int* __restrict__ seq_len, const int* __restrict__ seq_row0,
                                     int B, int Hk, int T, int BK, int window, int piece, int NW, int shard_lo, int shard_hi,
                                     int* __restrict__ lo_out, int* __restrict__ hi_out) {
    const int R = T + NW;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * Hk * R) return;
    const int r = i % R, h = (i / R) % Hk, b = i / (R * Hk);
    const int len = seq_len[b], t = len - 1;
    int a = 0, e = 0;
    if (len > 0) {
        if (r < T) {
            const int id = topk_idx[((int64_t)b * Hk + h) * T + r];
            if (id >= 0 && id <= t / BK) { a = id * BK; e = min(a + BK, len); }
        } else {
            const int w0 = max(0, t - window);
            a = w0 + (r - T) * piece;
            e = min(a + piece, len);
        }
    }
    a = max(a, shard_lo);
    e = min(e, shard_hi);
    if (a < e) {
        lo_out[i] = seq_row0[b] + a - shard_lo;
        hi_out[i] = seq_row0[b] + e - shard_lo;
    } else {
        lo_out[i] = -1;
        hi_out[i] = -1;
    }
}

// Visible compressed tokens of the decoded row and the cache rows of this GPU's share of them.
__global__ void decode_cmp_ranges_kernel(const int* __restrict__ seq_len, const int* __restrict__ cmp_row0, int B, int Hk, int ks, int stride,
                                         int cmp_lo, int cmp_hi, int* __restrict__ num_cmp, int* __restrict__ lo_out, int* __restrict__ hi_out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * Hk) return;
    const int b = i / Hk;
    const int len = seq_len[b];
    const int n = len >= ks ? (len - ks) / stride + 1 : 0;
    if (i % Hk == 0) num_cmp[b] = n;
    const int e = min(n, cmp_hi) - cmp_lo;
    lo_out[i] = e > 0 ? cmp_row0[b] : -1;
    hi_out[i] = e > 0 ? cmp_row0[b] + e : -1;
}

template <int D, bool HI, typename ET>
static cudaError_t launch_partial_tma(DecodeParams p, const CUtensorMap& kmap, const CUtensorMap& vmap, cudaStream_t stream) {
    constexpr int STAGE_BYTES = 2 * (D / 64) * 64 * 128;
    p.nst = min(max((p.chunk + kDecKT - 1) / kDecKT * p.rpp, 1), 3);
    const size_t smem = (size_t)p.nst * STAGE_BYTES + 1024 /* alignment slack */ + 1024 /* barriers, statistics */;
    auto kern = decode_partial_tma<D, HI, ET>;
    static int attr_dev_mask = 0;                          // the attribute is per device; set it once for each
    int dev = 0;
    cudaGetDevice(&dev);
    if (!(attr_dev_mask >> (dev & 31) & 1)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * STAGE_BYTES + 2048);
        if (e != cudaSuccess) return e;
        attr_dev_mask |= 1 << (dev & 31);
    }
    kern<<<(unsigned)((int64_t)p.B * p.Hk * p.NP * p.nchunk), 160, smem, stream>>>(p, kmap, vmap);
    return cudaGetLastError();
}

template <int D, typename ET>
static cudaError_t dispatch_g(int G, const DecodeParams& p, const CUtensorMap* kmap, const CUtensorMap* vmap, cudaStream_t stream) {
    if (G < 1 || G > 16) return cudaErrorInvalidValue;
    return G > 8 ? launch_partial_tma<D, true, ET>(p, *kmap, *vmap, stream) : launch_partial_tma<D, false, ET>(p, *kmap, *vmap, stream);
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_decode_attn_partial(const void* q, const void* k, const void* v, int64_t kv_rows, int64_t kv_stride_n, const int32_t* rng_lo,
                                       const int32_t* rng_hi, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                       int num_ranges, int ranges_per_partial, int chunk, int num_chunks, int dtype, float sm_scale, float* o_part,
                                       float* ml, float* scores, int64_t scores_ld, void* stream) {
    if (!q || !k || !v || !rng_lo || !rng_hi || !o_part || !ml) return FSA_ERR_BAD_ARG;
    if (batch <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || num_ranges <= 0 || chunk <= 0 || num_chunks <= 0)
        return FSA_ERR_BAD_ARG;
    if ((kv_stride_n % 8) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15)) return FSA_ERR_BAD_ARG;
    const int G = num_q_heads / num_kv_heads;
    DecodeParams p;
    p.q = q; p.k = k; p.v = v; p.kv_sn = kv_stride_n; p.rng_lo = rng_lo; p.rng_hi = rng_hi;
    p.B = batch; p.Hq = num_q_heads; p.Hk = num_kv_heads; p.R = num_ranges; p.chunk = chunk; p.nchunk = num_chunks;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.o_part = o_part; p.ml = (float2*)ml; p.scores = scores; p.scores_ld = scores_ld; p.nst = 1;
    if (ranges_per_partial < 1 || (ranges_per_partial > 1 && num_chunks != 1)) return FSA_ERR_BAD_ARG;
    p.rpp = ranges_per_partial;
    p.NP = (num_ranges + ranges_per_partial - 1) / ranges_per_partial;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (head_dim != 128 && head_dim != 64) return FSA_ERR_UNSUPPORTED;
    (void)cudaGetLastError();
    // K/V rows are streamed by TMA (tensor maps over [kv_rows, Hk * D])
    CUtensorMap kmap, vmap;
    if (kv_rows <= 0) return FSA_ERR_BAD_ARG;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return FSA_ERR_CUDA;   // binds the context
        int rc = make_tile_map(&kmap, k, dtype, kv_rows, (int64_t)num_kv_heads * head_dim, kv_stride_n, kDecKT);
        if (rc) return rc;
        rc = make_tile_map(&vmap, v, dtype, kv_rows, (int64_t)num_kv_heads * head_dim, kv_stride_n, kDecKT);
        if (rc) return rc;
    }
    const CUtensorMap *km = &kmap, *vm = &vmap;
    cudaError_t e = cudaErrorInvalidValue;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == FSA_DTYPE_BF16) {
        if (head_dim == 128) e = dispatch_g<128, __nv_bfloat16>(G, p, km, vm, st);
        else e = dispatch_g<64, __nv_bfloat16>(G, p, km, vm, st);
    } else {
        if (head_dim == 128) e = dispatch_g<128, __half>(G, p, km, vm, st);
        else e = dispatch_g<64, __half>(G, p, km, vm, st);
    }
    if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
    return e == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_lse_merge(const float* o_part, const float* ml, int64_t rows, int num_partials, int part_stride, int head_dim, int out_dtype,
                             void* o, float* lse, void* stream) {
    if (!o_part || !ml || !o || rows < 0 || num_partials <= 0 || part_stride < num_partials || head_dim <= 0 || head_dim % 4) return FSA_ERR_BAD_ARG;
    if (((uintptr_t)o_part & 15) || ((uintptr_t)o & 7)) return FSA_ERR_BAD_ARG;
    if (rows == 0) return FSA_OK;
    (void)cudaGetLastError();
    unsigned grid = (unsigned)((rows + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == FSA_DTYPE_BF16)
        lse_merge_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(o_part, (const float2*)ml, rows, num_partials, part_stride, head_dim, (__nv_bfloat16*)o, lse);
    else if (out_dtype == FSA_DTYPE_FP16)
        lse_merge_kernel<__half><<<grid, 256, 0, st>>>(o_part, (const float2*)ml, rows, num_partials, part_stride, head_dim, (__half*)o, lse);
    else if (out_dtype == 2)
        lse_merge_kernel<float><<<grid, 256, 0, st>>>(o_part, (const float2*)ml, rows, num_partials, part_stride, head_dim, (float*)o, lse);
    else
        return FSA_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_decode_select_topk(const float* scores, int64_t scores_ld, int shard_len, int64_t shard_stride, const float* lse, const int32_t* seq_len,
                                      const int32_t* num_cmp, int batch, int num_q_heads, int num_kv_heads, int kernel_size,
                                      int kernel_stride, int block_size, int init_blocks, int local_blocks, int topk, int max_blocks,
                                      int32_t* topk_idx, void* stream) {
    if (!scores || !lse || !seq_len || !num_cmp || !topk_idx) return FSA_ERR_BAD_ARG;
    if (batch <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || topk <= 0 || topk > 64 || max_blocks <= 0) return FSA_ERR_BAD_ARG;
    if (kernel_size % kernel_stride || block_size % kernel_stride) return FSA_ERR_UNSUPPORTED;
    DecodeTopkParams p;
    if (shard_len <= 0) return FSA_ERR_BAD_ARG;
    p.scores = scores; p.ld = scores_ld; p.shard_len = shard_len; p.shard_stride = shard_stride; p.lse = lse; p.seq_len = seq_len; p.ncmp = num_cmp;
    p.B = batch; p.Hk = num_kv_heads; p.Hq = num_q_heads; p.G = num_q_heads / num_kv_heads;
    p.ks = kernel_size; p.stride = kernel_stride; p.BK = block_size; p.init_blocks = init_blocks; p.local_blocks = local_blocks;
    p.T = topk; p.max_blocks = max_blocks;
    const int a = kernel_size / kernel_stride, bb = block_size / kernel_stride;
    p.nw = a + bb - 1;
    if (p.nw > 16) return FSA_ERR_UNSUPPORTED;
    for (int i = 0; i < 16; ++i) p.w[i] = 0.f;
    for (int i = 0; i < a; ++i)
        for (int j = 0; j < bb; ++j) p.w[i + j] += 1.f;
    p.out = topk_idx;
    // block scores, winners, probabilities of the compressed tokens those blocks can touch
    const int max_cmp_touched = max_blocks * (block_size / kernel_stride) + (kernel_size / kernel_stride + block_size / kernel_stride - 1);
    size_t smem = (size_t)(max_blocks + 64 + max_cmp_touched) * sizeof(float);
    if (smem > 200 * 1024) return FSA_ERR_UNSUPPORTED;
    (void)cudaGetLastError();
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(decode_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return FSA_ERR_CUDA;
    }
    decode_topk_kernel<<<(unsigned)(batch * num_kv_heads), 256, smem, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_decode_ranges(const int32_t* topk_idx, const int32_t* seq_len, const int32_t* seq_row0, int batch, int num_kv_heads,
                                 int topk, int block_size, int window, int piece, int num_window_pieces, int shard_lo, int shard_hi,
                                 int32_t* rng_lo, int32_t* rng_hi, void* stream) {
    if (!seq_len || !seq_row0 || !rng_lo || !rng_hi || (topk > 0 && !topk_idx)) return FSA_ERR_BAD_ARG;
    if (batch <= 0 || num_kv_heads <= 0 || topk < 0 || num_window_pieces < 0 || topk + num_window_pieces == 0 || block_size <= 0 || piece <= 0)
        return FSA_ERR_BAD_ARG;
    if ((int64_t)piece * num_window_pieces < (int64_t)window + 1 && num_window_pieces > 0) return FSA_ERR_BAD_ARG;
    const int total = batch * num_kv_heads * (topk + num_window_pieces);
    (void)cudaGetLastError();
    decode_ranges_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(topk_idx, seq_len, seq_row0, batch, num_kv_heads, topk,
                                                                             block_size, window, piece, num_window_pieces, shard_lo,
                                                                             shard_hi, rng_lo, rng_hi);
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_decode_cmp_ranges(const int32_t* seq_len, const int32_t* cmp_row0, int batch, int num_kv_heads, int kernel_size,
                                     int kernel_stride, int cmp_lo, int cmp_hi, int32_t* num_cmp, int32_t* rng_lo, int32_t* rng_hi,
                                     void* stream) {
    if (!seq_len || !cmp_row0 || !num_cmp || !rng_lo || !rng_hi || batch <= 0 || num_kv_heads <= 0 || kernel_size <= 0 || kernel_stride <= 0)
        return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    const int total = batch * num_kv_heads;
    decode_cmp_ranges_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(seq_len, cmp_row0, batch, num_kv_heads, kernel_size,
                                                                                 kernel_stride, cmp_lo, cmp_hi, num_cmp, rng_lo, rng_hi);
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_decode_read_status(int* status_out) {
    if (!status_out) return FSA_ERR_BAD_ARG;
    return cudaMemcpyFromSymbol(status_out, g_decode_status, sizeof(int)) == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_decode_finish(const float* o_part, const float* ml, int64_t rows, int num_sel_partials, int num_win_partials,
                                 int part_stride, int head_dim, int num_q_heads, int dtype, const void* o_cmp, const void* gate,
                                 void* out, void* stream) {
    if (!o_part || !ml || !o_cmp || !gate || !out || rows < 0 || num_sel_partials < 0 || num_win_partials < 0 || num_q_heads <= 0)
        return FSA_ERR_BAD_ARG;
    if (part_stride < num_sel_partials + num_win_partials || head_dim <= 0 || head_dim % 4 || ((uintptr_t)o_part & 15)) return FSA_ERR_BAD_ARG;
    if (rows == 0) return FSA_OK;
    (void)cudaGetLastError();
    unsigned grid = (unsigned)((rows + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == FSA_DTYPE_BF16)
        decode_finish_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(o_part, (const float2*)ml, rows, num_sel_partials, num_win_partials, part_stride,
                                                                 head_dim, num_q_heads, (const __nv_bfloat16*)o_cmp, (const __nv_bfloat16*)gate,
                                                                 (__nv_bfloat16*)out);
    else if (dtype == FSA_DTYPE_FP16)
        decode_finish_kernel<__half><<<grid, 256, 0, st>>>(o_part, (const float2*)ml, rows, num_sel_partials, num_win_partials, part_stride, head_dim,
                                                          num_q_heads, (const __half*)o_cmp, (const __half*)gate, (__half*)out);
    else
        return FSA_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}
