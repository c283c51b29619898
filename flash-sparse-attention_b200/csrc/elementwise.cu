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


// ------------------------------------------------------------------------------------------------ gate projection + mix
// The layer's gate path in one kernel each way (fsa/module/fsa.py:162-171: gate = sigmoid(Linear(hidden, 3)(x)), then the
// mix of the three branch outputs): z = x Wg^T rounded to the activation dtype as the Linear would, g = sigmoid(z) rounded
// again, out = g0 a + g1 b + g2 c.  One warp per token; Wg (3 rows) sits in shared memory.
__device__ __forceinline__ float round_to(float v, __nv_bfloat16) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float round_to(float v, __half) { return __half2float(__float2half_rn(v)); }

template <typename ET>
__device__ __forceinline__ void dot8x3(const uint4& xv, const uint4& w0, const uint4& w1, const uint4& w2, float& a0, float& a1, float& a2) {
    const uint32_t *px = &xv.x, *p0 = &w0.x, *p1 = &w1.x, *p2 = &w2.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = ElemTraits<ET>::unpack2(px[i]);
        const float2 u = ElemTraits<ET>::unpack2(p0[i]), v = ElemTraits<ET>::unpack2(p1[i]), w = ElemTraits<ET>::unpack2(p2[i]);
        a0 = fmaf(x.x, u.x, fmaf(x.y, u.y, a0));
        a1 = fmaf(x.x, v.x, fmaf(x.y, v.y, a1));
        a2 = fmaf(x.x, w.x, fmaf(x.y, w.y, a2));
    }
}

template <typename ET>
__global__ void __launch_bounds__(256) gate_proj_mix_fwd_kernel(const ET* __restrict__ x, int64_t x_sn, const ET* __restrict__ wg,
                                                                const ET* __restrict__ a, const ET* __restrict__ b,
                                                                const ET* __restrict__ c, int64_t N, int hidden, int HD,
                                                                ET* __restrict__ out, ET* __restrict__ gate) {
    extern __shared__ __align__(16) uint8_t gsm[];
    uint4* sw = reinterpret_cast<uint4*>(gsm);                 // [3][hidden / 8]
    const int hv = hidden / 8, vec = HD / 8;
    for (int i = threadIdx.x; i < 3 * hv; i += blockDim.x) sw[i] = reinterpret_cast<const uint4*>(wg)[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int64_t n = (int64_t)blockIdx.x * nw + warp; n < N; n += (int64_t)gridDim.x * nw) {
        float z0 = 0.f, z1 = 0.f, z2 = 0.f;
        const uint4* xr = reinterpret_cast<const uint4*>(x + n * x_sn);
        for (int v = lane; v < hv; v += 32) dot8x3<ET>(__ldg(xr + v), sw[v], sw[hv + v], sw[2 * hv + v], z0, z1, z2);
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            z0 += __shfl_xor_sync(0xffffffffu, z0, o);
            z1 += __shfl_xor_sync(0xffffffffu, z1, o);
            z2 += __shfl_xor_sync(0xffffffffu, z2, o);
        }
        const float g0 = round_to(1.f / (1.f + __expf(-round_to(z0, ET()))), ET());
        const float g1 = round_to(1.f / (1.f + __expf(-round_to(z1, ET()))), ET());
        const float g2 = round_to(1.f / (1.f + __expf(-round_to(z2, ET()))), ET());
        if (lane == 0) { gate[n * 3] = (ET)g0; gate[n * 3 + 1] = (ET)g1; gate[n * 3 + 2] = (ET)g2; }
        for (int v0 = lane; v0 < vec; v0 += 64) {
            uint4 va[2], vb[2], vc[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = v0 + 32 * u;
                if (v < vec) {
                    const int64_t idx = n * vec + v;
                    va[u] = ld_stream16(reinterpret_cast<const uint4*>(a) + idx);
                    vb[u] = ld_stream16(reinterpret_cast<const uint4*>(b) + idx);
                    vc[u] = ld_stream16(reinterpret_cast<const uint4*>(c) + idx);
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = v0 + 32 * u;
                if (v >= vec) continue;
                const uint32_t *pa = &va[u].x, *pb = &vb[u].x, *pc = &vc[u].x;
                uint4 o;
                uint32_t* po = &o.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 p = ElemTraits<ET>::unpack2(pa[i]), q = ElemTraits<ET>::unpack2(pb[i]), r = ElemTraits<ET>::unpack2(pc[i]);
                    po[i] = ElemTraits<ET>::pack2(g0 * p.x + g1 * q.x + g2 * r.x, g0 * p.y + g1 * q.y + g2 * r.y);
                }
                st_stream16(reinterpret_cast<uint4*>(out) + n * vec + v, o);
            }
        }
    }
}

// Backward, per token: da = g0 do, db = g1 do, dc = g2 do; dg_j = sum(do * branch_j) rounded; dz_j = dg_j g_j (1 - g_j)
// rounded (the sigmoid's backward in the activation dtype); dx[n, :] = sum_j dz_j Wg[j, :]; dz kept in fp32 for dWg.
template <typename ET>
__global__ void __launch_bounds__(256) gate_proj_mix_bwd_kernel(const ET* __restrict__ gate, const ET* __restrict__ wg,
                                                                const ET* __restrict__ a, const ET* __restrict__ b,
                                                                const ET* __restrict__ c, const ET* __restrict__ d_o, int64_t N,
                                                                int hidden, int HD, ET* __restrict__ da, ET* __restrict__ db,
                                                                ET* __restrict__ dc, ET* __restrict__ dx, float* __restrict__ dz) {
    extern __shared__ __align__(16) uint8_t gsm[];
    uint4* sw = reinterpret_cast<uint4*>(gsm);
    const int hv = hidden / 8, vec = HD / 8;
    for (int i = threadIdx.x; i < 3 * hv; i += blockDim.x) sw[i] = reinterpret_cast<const uint4*>(wg)[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int64_t n = (int64_t)blockIdx.x * nw + warp; n < N; n += (int64_t)gridDim.x * nw) {
        const float g0 = (float)gate[n * 3], g1 = (float)gate[n * 3 + 1], g2 = (float)gate[n * 3 + 2];
        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
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
                    float2 p = ElemTraits<ET>::unpack2(pa[i]), q = ElemTraits<ET>::unpack2(pb[i]), r = ElemTraits<ET>::unpack2(pc[i]);
                    s0 += d.x * p.x + d.y * p.y;
                    s1 += d.x * q.x + d.y * q.y;
                    s2 += d.x * r.x + d.y * r.y;
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
        const float z0 = round_to(round_to(s0, ET()) * g0 * (1.f - g0), ET());
        const float z1 = round_to(round_to(s1, ET()) * g1 * (1.f - g1), ET());
        const float z2 = round_to(round_to(s2, ET()) * g2 * (1.f - g2), ET());
        if (lane == 0) { dz[n * 3] = z0; dz[n * 3 + 1] = z1; dz[n * 3 + 2] = z2; }
        uint4* xr = reinterpret_cast<uint4*>(dx + n * (int64_t)hidden);
        for (int v = lane; v < hv; v += 32) {
            const uint4 w0 = sw[v], w1 = sw[hv + v], w2 = sw[2 * hv + v];
            const uint32_t *p0 = &w0.x, *p1 = &w1.x, *p2 = &w2.x;
            uint4 o;
            uint32_t* po = &o.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 u = ElemTraits<ET>::unpack2(p0[i]), vv = ElemTraits<ET>::unpack2(p1[i]), w = ElemTraits<ET>::unpack2(p2[i]);
                po[i] = ElemTraits<ET>::pack2(z0 * u.x + z1 * vv.x + z2 * w.x, z0 * u.y + z1 * vv.y + z2 * w.y);
            }
            st_stream16(xr + v, o);
        }
    }
}

// dWg[j, col] = sum_n dz[n, j] x[n, col]: thread = 8 columns, CTA row = a chunk of tokens; partial[chunk][3][hidden] fp32.
template <typename ET>
__global__ void __launch_bounds__(256) gate_dw_partial_kernel(const ET* __restrict__ x, int64_t x_sn, const float* __restrict__ dz,
                                                              int64_t N, int hidden, int chunk_tokens, float* __restrict__ partial) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;         // 16-byte column vector
    if (v >= hidden / 8) return;
    const int64_t n0 = (int64_t)blockIdx.y * chunk_tokens, n1 = n0 + chunk_tokens < N ? n0 + chunk_tokens : N;
    float acc[3][8];
#pragma unroll
    for (int j = 0; j < 3; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
    for (int64_t n = n0; n < n1; ++n) {
        const uint4 xv = ld_stream16(reinterpret_cast<const uint4*>(x + n * x_sn) + v);
        const float z0 = __ldg(dz + n * 3), z1 = __ldg(dz + n * 3 + 1), z2 = __ldg(dz + n * 3 + 2);
        const uint32_t* px = &xv.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = ElemTraits<ET>::unpack2(px[i]);
            acc[0][2 * i] = fmaf(z0, f.x, acc[0][2 * i]); acc[0][2 * i + 1] = fmaf(z0, f.y, acc[0][2 * i + 1]);
            acc[1][2 * i] = fmaf(z1, f.x, acc[1][2 * i]); acc[1][2 * i + 1] = fmaf(z1, f.y, acc[1][2 * i + 1]);
            acc[2][2 * i] = fmaf(z2, f.x, acc[2][2 * i]); acc[2][2 * i + 1] = fmaf(z2, f.y, acc[2][2 * i + 1]);
        }
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        float* dst = partial + ((int64_t)blockIdx.y * 3 + j) * hidden + v * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
    }
}

// the chunks' partial sums added in chunk order (deterministic) and rounded
template <typename ET>
__global__ void __launch_bounds__(256) gate_dw_reduce_kernel(const float* __restrict__ partial, int chunks, int hidden, ET* __restrict__ dwg) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 3 * hidden) return;
    float s = 0.f;
    for (int c = 0; c < chunks; ++c) s += partial[(int64_t)c * 3 * hidden + i];
    dwg[i] = (ET)s;
}

constexpr int kGateChunks = 256;

template <typename ET>
static int run_gate_fwd(const void* x, int64_t x_sn, const void* wg, const void* a, const void* b, const void* c, int64_t N, int hidden,
                        int HD, void* out, void* gate, cudaStream_t stream) {
    const int smem = 3 * hidden * 2;
    auto kern = gate_proj_mix_fwd_kernel<ET>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FSA_ERR_CUDA;
    const int64_t want = (N + 7) / 8;
    const unsigned grid = (unsigned)(want < 148 * 8 ? want : 148 * 8);
    kern<<<grid, 256, smem, stream>>>((const ET*)x, x_sn, (const ET*)wg, (const ET*)a, (const ET*)b, (const ET*)c, N, hidden, HD,
                                      (ET*)out, (ET*)gate);
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

template <typename ET>
static int run_gate_bwd(const void* x, int64_t x_sn, const void* wg, const void* gate, const void* a, const void* b, const void* c,
                        const void* d_o, int64_t N, int hidden, int HD, void* da, void* db, void* dc, void* dx, void* dwg, float* dz,
                        float* partial, cudaStream_t stream) {
    const int smem = 3 * hidden * 2;
    auto kern = gate_proj_mix_bwd_kernel<ET>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FSA_ERR_CUDA;
    const int64_t want = (N + 7) / 8;
    const unsigned grid = (unsigned)(want < 148 * 8 ? want : 148 * 8);
    kern<<<grid, 256, smem, stream>>>((const ET*)gate, (const ET*)wg, (const ET*)a, (const ET*)b, (const ET*)c, (const ET*)d_o, N, hidden,
                                      HD, (ET*)da, (ET*)db, (ET*)dc, (ET*)dx, dz);
    const int chunk_tokens = (int)((N + kGateChunks - 1) / kGateChunks);
    const int chunks = (int)((N + chunk_tokens - 1) / chunk_tokens);
    gate_dw_partial_kernel<ET><<<dim3((unsigned)((hidden / 8 + 255) / 256), (unsigned)chunks), 256, 0, stream>>>((const ET*)x, x_sn, dz, N, hidden,
                                                                                                          chunk_tokens, partial);
    gate_dw_reduce_kernel<ET><<<(unsigned)((3 * hidden + 255) / 256), 256, 0, stream>>>(partial, chunks, hidden, (ET*)dwg);
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
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

extern "C" int64_t fsa_gate_proj_mix_scratch_bytes(int64_t total, int hidden) {
    return (total * 3 + 3) / 4 * 16 + (int64_t)kGateChunks * 3 * hidden * 4;
}

extern "C" int fsa_gate_proj_mix_fwd(const void* x, int64_t x_stride_n, const void* w_gate, const void* a, const void* b, const void* c,
                                     int64_t total, int hidden, int row_elems, int dtype, void* out, void* gate, void* stream) {
    if (total == 0) return FSA_OK;
    if (!x || !w_gate || !a || !b || !c || !out || !gate || hidden <= 0 || hidden % 8 || row_elems % 8 || x_stride_n % 8) return FSA_ERR_BAD_ARG;
    if (hidden > 16384) return FSA_ERR_UNSUPPORTED;      // the three weight rows live in shared memory
    if (((uintptr_t)x & 15) || ((uintptr_t)w_gate & 15) || ((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)c & 15) || ((uintptr_t)out & 15))
        return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    if (dtype == FSA_DTYPE_BF16) return run_gate_fwd<__nv_bfloat16>(x, x_stride_n, w_gate, a, b, c, total, hidden, row_elems, out, gate, (cudaStream_t)stream);
    if (dtype == FSA_DTYPE_FP16) return run_gate_fwd<__half>(x, x_stride_n, w_gate, a, b, c, total, hidden, row_elems, out, gate, (cudaStream_t)stream);
    return FSA_ERR_BAD_ARG;
}

extern "C" int fsa_gate_proj_mix_bwd(const void* x, int64_t x_stride_n, const void* w_gate, const void* gate, const void* a, const void* b,
                                     const void* c, const void* d_out, int64_t total, int hidden, int row_elems, int dtype, void* da, void* db,
                                     void* dc, void* dx, void* dw_gate, float* scratch, int64_t scratch_bytes, void* stream) {
    if (total == 0) return FSA_OK;
    if (!x || !w_gate || !gate || !a || !b || !c || !d_out || !da || !db || !dc || !dx || !dw_gate || !scratch) return FSA_ERR_BAD_ARG;
    if (hidden <= 0 || hidden % 8 || row_elems % 8 || x_stride_n % 8) return FSA_ERR_BAD_ARG;
    if (hidden > 16384) return FSA_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w_gate & 15) || ((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)c & 15) || ((uintptr_t)d_out & 15) ||
        ((uintptr_t)da & 15) || ((uintptr_t)db & 15) || ((uintptr_t)dc & 15) || ((uintptr_t)dx & 15) || ((uintptr_t)scratch & 15))
        return FSA_ERR_BAD_ARG;
    if (scratch_bytes < fsa_gate_proj_mix_scratch_bytes(total, hidden)) return FSA_ERR_WORKSPACE;
    float* dz = scratch;
    float* partial = scratch + (total * 3 + 3) / 4 * 4;
    (void)cudaGetLastError();
    if (dtype == FSA_DTYPE_BF16)
        return run_gate_bwd<__nv_bfloat16>(x, x_stride_n, w_gate, gate, a, b, c, d_out, total, hidden, row_elems, da, db, dc, dx, dw_gate, dz, partial, (cudaStream_t)stream);
    if (dtype == FSA_DTYPE_FP16)
        return run_gate_bwd<__half>(x, x_stride_n, w_gate, gate, a, b, c, d_out, total, hidden, row_elems, da, db, dc, dx, dw_gate, dz, partial, (cudaStream_t)stream);
    return FSA_ERR_BAD_ARG;
}
