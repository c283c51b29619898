// Bandwidth-bound pieces around the three attention branches: rotary embedding and the gate mix.
#include "../../include/fsa_sm100.h"
#include "sel_common.cuh"

namespace fsa {

// Half-split ("non-interleaved") rotary embedding, positions restarting at every sequence:
//   (x1, x2) = halves of x;  out = (x1 cos - x2 sin, x1 sin + x2 cos)
// cos / sin tables are [table_len, d/2] in the activation dtype (the reference rounds them to
// it first, nsa_ref/module/rope.py:124) and row p holds position start + p * stride, so the
// row index is the token's position inside its sequence.  conj = 1 applies the inverse
// rotation (the backward).  One thread per 8 output pairs.
template <typename ET>
__global__ void __launch_bounds__(256) rope_kernel(const ET* __restrict__ x, int64_t x_sn, int64_t x_sh, const ET* __restrict__ cs,
                                                   const ET* __restrict__ sn, const int* __restrict__ cu, int B, int64_t N, int H,
                                                   int D, int conj, ET* __restrict__ out) {
    const int half = D / 2, vec = half / 8;           // 16-byte vectors per half row
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= N * H * vec) return;
    const int v = (int)(gid % vec);
    const int h = (int)((gid / vec) % H);
    const int n = (int)(gid / ((int64_t)vec * H));
    const int b = find_seq(cu, B, n);
    const int pos = n - __ldg(cu + b);
    const ET* xr = x + (int64_t)n * x_sn + (int64_t)h * x_sh;
    uint4 a = *reinterpret_cast<const uint4*>(xr + v * 8);
    uint4 c = *reinterpret_cast<const uint4*>(xr + half + v * 8);
    uint4 co = *reinterpret_cast<const uint4*>(cs + (int64_t)pos * half + v * 8);
    uint4 si = *reinterpret_cast<const uint4*>(sn + (int64_t)pos * half + v * 8);
    const uint32_t *pa = &a.x, *pc = &c.x, *pco = &co.x, *psi = &si.x;
    uint4 o1, o2;
    uint32_t *q1 = &o1.x, *q2 = &o2.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 x1 = ElemTraits<ET>::unpack2(pa[i]), x2 = ElemTraits<ET>::unpack2(pc[i]);
        float2 cc = ElemTraits<ET>::unpack2(pco[i]), ss = ElemTraits<ET>::unpack2(psi[i]);
        if (conj) { ss.x = -ss.x; ss.y = -ss.y; }
        q1[i] = ElemTraits<ET>::pack2(x1.x * cc.x - x2.x * ss.x, x1.y * cc.y - x2.y * ss.y);
        q2[i] = ElemTraits<ET>::pack2(x1.x * ss.x + x2.x * cc.x, x1.y * ss.y + x2.y * cc.y);
    }
    ET* orow = out + ((int64_t)n * H + h) * D;
    *reinterpret_cast<uint4*>(orow + v * 8) = o1;
    *reinterpret_cast<uint4*>(orow + half + v * 8) = o2;
}

// 16-byte streaming load / store (the rows are used once: keep them out of the way of L2-resident data)
__device__ __forceinline__ uint4 ld_stream16(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) { __stcs(reinterpret_cast<uint4*>(p), v); }

// out[n, :] = g[n,0] a[n, :] + g[n,1] b[n, :] + g[n,2] c[n, :]   (rows of HD = heads * head_dim elements).
// Two 16-byte vectors per thread, all six loads issued before the arithmetic.
template <typename ET>
__global__ void __launch_bounds__(256) gate_mix_fwd_kernel(const ET* __restrict__ g, const ET* __restrict__ a,
                                                           const ET* __restrict__ b, const ET* __restrict__ c, int64_t N, int HD,
                                                           ET* __restrict__ out) {
    const int vec = HD / 8;
    const int64_t total = N * vec;
    const int64_t base = (int64_t)blockIdx.x * (blockDim.x * 2) + threadIdx.x;
    uint4 va[2], vb[2], vc[2];
    float gg[2][3];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int64_t gid = base + u * blockDim.x;
        if (gid < total) {
            va[u] = ld_stream16(reinterpret_cast<const uint4*>(a) + gid);
            vb[u] = ld_stream16(reinterpret_cast<const uint4*>(b) + gid);
            vc[u] = ld_stream16(reinterpret_cast<const uint4*>(c) + gid);
            const int64_t n = gid / vec;
            gg[u][0] = (float)g[n * 3]; gg[u][1] = (float)g[n * 3 + 1]; gg[u][2] = (float)g[n * 3 + 2];
        }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int64_t gid = base + u * blockDim.x;
        if (gid >= total) continue;
        const uint32_t *pa = &va[u].x, *pb = &vb[u].x, *pc = &vc[u].x;
        uint4 o;
        uint32_t* po = &o.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 x = ElemTraits<ET>::unpack2(pa[i]), y = ElemTraits<ET>::unpack2(pb[i]), z = ElemTraits<ET>::unpack2(pc[i]);
            po[i] = ElemTraits<ET>::pack2(gg[u][0] * x.x + gg[u][1] * y.x + gg[u][2] * z.x, gg[u][0] * x.y + gg[u][1] * y.y + gg[u][2] * z.y);
        }
        st_stream16(reinterpret_cast<uint4*>(out) + gid, o);
    }
}

// da = g0 do, db = g1 do, dc = g2 do, dg[n, i] = sum over the row of do * branch_i.  One warp per token; two 16-byte
// vectors of every input per lane and iteration (eight loads in flight).
template <typename ET>
__global__ void __launch_bounds__(256) gate_mix_bwd_kernel(const ET* __restrict__ g, const ET* __restrict__ a,
                                                           const ET* __restrict__ b, const ET* __restrict__ c,
                                                           const ET* __restrict__ d_o, int64_t N, int HD, ET* __restrict__ da,
                                                           ET* __restrict__ db, ET* __restrict__ dc, float* __restrict__ dg) {
    const int lane = threadIdx.x & 31;
    const int64_t n = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    const float g0 = (float)g[n * 3], g1 = (float)g[n * 3 + 1], g2 = (float)g[n * 3 + 2];
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    const int vec = HD / 8;
    for (int v0 = lane; v0 < vec; v0 += 64) {
        uint4 vd[2], va[2], vb[2], vc[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = v0 + 32 * u;
            if (v < vec) {
                const int64_t idx = n * vec + v;
                vd[u] = ld_stream16(reinterpret_cast<const uint4*>(d_o) + idx);
                va[u] = ld_stream16(reinterpret_cast<const uint4*>(a) + idx);
                vb[u] = ld_stream16(reinterpret_cast<const uint4*>(b) + idx);
                vc[u] = ld_stream16(reinterpret_cast<const uint4*>(c) + idx);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = v0 + 32 * u;
            if (v >= vec) continue;
            const int64_t idx = n * vec + v;
            const uint32_t *pd = &vd[u].x, *pa = &va[u].x, *pb = &vb[u].x, *pc = &vc[u].x;
            uint4 oa, ob, oc;
            uint32_t *qa = &oa.x, *qb = &ob.x, *qc = &oc.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 d = ElemTraits<ET>::unpack2(pd[i]);
                float2 x = ElemTraits<ET>::unpack2(pa[i]), y = ElemTraits<ET>::unpack2(pb[i]), z = ElemTraits<ET>::unpack2(pc[i]);
                s0 += d.x * x.x + d.y * x.y;
                s1 += d.x * y.x + d.y * y.y;
                s2 += d.x * z.x + d.y * z.y;
                qa[i] = ElemTraits<ET>::pack2(g0 * d.x, g0 * d.y);
                qb[i] = ElemTraits<ET>::pack2(g1 * d.x, g1 * d.y);
                qc[i] = ElemTraits<ET>::pack2(g2 * d.x, g2 * d.y);
            }
            st_stream16(reinterpret_cast<uint4*>(da) + idx, oa);
            st_stream16(reinterpret_cast<uint4*>(db) + idx, ob);
            st_stream16(reinterpret_cast<uint4*>(dc) + idx, oc);
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) { dg[n * 3] = s0; dg[n * 3 + 1] = s1; dg[n * 3 + 2] = s2; }
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_rope(const void* x, int64_t x_sn, int64_t x_sh, const void* cos_tab, const void* sin_tab,
                        const int32_t* cu_seqlens, int batch, int64_t total, int heads, int head_dim, int dtype, int conj,
                        void* out, void* stream) {
    if (!x || !cos_tab || !sin_tab || !cu_seqlens || !out) return total == 0 ? FSA_OK : FSA_ERR_BAD_ARG;
    if (head_dim % 16 || (x_sn % 8) || (x_sh % 8) || ((uintptr_t)x & 15) || ((uintptr_t)out & 15)) return FSA_ERR_BAD_ARG;
    if (total == 0) return FSA_OK;
    (void)cudaGetLastError();
    int64_t threads = total * heads * (head_dim / 16);
    unsigned grid = (unsigned)((threads + 255) / 256);
    if (dtype == FSA_DTYPE_BF16)
        rope_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, x_sn, x_sh, (const __nv_bfloat16*)cos_tab,
                                                                           (const __nv_bfloat16*)sin_tab, cu_seqlens, batch, total, heads,
                                                                           head_dim, conj, (__nv_bfloat16*)out);
    else if (dtype == FSA_DTYPE_FP16)
        rope_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)x, x_sn, x_sh, (const __half*)cos_tab, (const __half*)sin_tab,
                                                                    cu_seqlens, batch, total, heads, head_dim, conj, (__half*)out);
    else
        return FSA_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_gate_mix_fwd(const void* gate, const void* a, const void* b, const void* c, int64_t total, int row_elems, int dtype,
                                void* out, void* stream) {
    if (total == 0) return FSA_OK;
    if (!gate || !a || !b || !c || !out || row_elems % 8) return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    int64_t threads = total * (row_elems / 8);
    unsigned grid = (unsigned)((threads + 511) / 512);   // two vectors per thread
    if (dtype == FSA_DTYPE_BF16)
        gate_mix_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)a,
                                                                                   (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, total,
                                                                                   row_elems, (__nv_bfloat16*)out);
    else if (dtype == FSA_DTYPE_FP16)
        gate_mix_fwd_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)gate, (const __half*)a, (const __half*)b,
                                                                            (const __half*)c, total, row_elems, (__half*)out);
    else
        return FSA_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_gate_mix_bwd(const void* gate, const void* a, const void* b, const void* c, const void* d_out, int64_t total,
                                int row_elems, int dtype, void* da, void* db, void* dc, float* dgate, void* stream) {
    if (total == 0) return FSA_OK;
    if (!gate || !a || !b || !c || !d_out || !da || !db || !dc || !dgate || row_elems % 8) return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    unsigned grid = (unsigned)((total + 7) / 8);
    if (dtype == FSA_DTYPE_BF16)
        gate_mix_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)gate, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c,
            (const __nv_bfloat16*)d_out, total, row_elems, (__nv_bfloat16*)da, (__nv_bfloat16*)db, (__nv_bfloat16*)dc, dgate);
    else if (dtype == FSA_DTYPE_FP16)
        gate_mix_bwd_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half*)gate, (const __half*)a, (const __half*)b,
                                                                            (const __half*)c, (const __half*)d_out, total, row_elems,
                                                                            (__half*)da, (__half*)db, (__half*)dc, dgate);
    else
        return FSA_ERR_BAD_ARG;
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}
