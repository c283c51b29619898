// K/V compression by a strided linear projection (backward), two tcgen05 GEMM kernels without atomics.
//
// Replaces linear_compress_bwd_kernel of the reference (nsa_ref/ops/linear_compress.py:135-292, launched at :401-470),
// which scatters both gradients with fp32 tl.atomic_add (:275, :292).  With
//     y[c, h, :] = sum_{k < ks} x[s_b + c * stride + k, h, :] @ W[h, k * d : (k + 1) * d, :]
// the gradients are
//     dx[s_b + t, h, :]          = sum_{j < ks / stride} dy[m - j, h, :] @ W[h, (p + j * stride) * d : ..., :]^T      t = m * stride + p
//     dW[h, k * d + a, :]        = sum_b sum_c x[s_b + c * stride + k, h, a] * dy[y_b + c, h, :]
//
// dx: a token belongs to ks / stride windows, and tokens with the same phase p = t mod stride meet the same slices of W.
// One CTA = 128 consecutive m of one sequence x one head x a group of phases; per phase it runs the GEMM
// [128, (ks / stride) * d] x [(ks / stride) * d, d] whose left operand is dy shifted by j rows (TMA; rows outside the
// sequence's windows are out of the map's bounds and read as zero) and writes the rows m * stride + p once, in the
// activation dtype, from an fp32 accumulator in TMEM (two accumulators: the stores of a phase overlap the next phase).
//
// dW: one CTA = one head x one window offset k (two offsets when d = 64): M = input feature, N = output feature, the
// reduction runs over every window of every sequence in 128-window tiles.  Both operands are "MN-major" (the window index
// is the row of both tiles), gathered with 16-byte async copies (rows of x are stride tokens apart; windows past the end
// of a sequence are zero-filled), so no tensor map per sequence is needed and the whole gradient is one launch.
#include "../../include/fsa_sm100.h"
#include "sm100_prims.cuh"

namespace fsa {

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int box_rows);

// ------------------------------------------------------------------------------------------------ dx
struct LcDxParams {
    int n_cmp;          // windows of this sequence
    int L;              // tokens of this sequence
    int H, ks, stride;
    int phases;         // phases per CTA
    void* dx;           // first row of this sequence, [L, H, D] contiguous
    int* status;
};

constexpr int kLcDxStages = 4;

template <int D, typename ET>
__global__ void __launch_bounds__(192) linear_compress_dx_kernel(const LcDxParams p, const __grid_constant__ CUtensorMap ymap,
                                                                const __grid_constant__ CUtensorMap wmap) {
    constexpr int kA = 128 * 128, kB = D * 128;           // one stage: 128 rows of dy x 64 columns, D rows of W x 64 columns
    constexpr int KH = D / 64;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;
    uint8_t* sB = sA + kLcDxStages * kA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + kLcDxStages * kB);
    uint64_t* full = bars;                      // [stages]
    uint64_t* empty = bars + kLcDxStages;       // [stages]
    uint64_t* acc_full = bars + 2 * kLcDxStages;        // [2]
    uint64_t* acc_empty = bars + 2 * kLcDxStages + 2;   // [2]
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 2 * kLcDxStages + 4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.x * 128, h = blockIdx.y, p0 = blockIdx.z * p.phases;
    const int J = p.ks / p.stride;
    const int per_phase = J * KH;
    int* status = p.status;
    if (tid == 0) {
        for (int i = 0; i < kLcDxStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 128); }
        mbar_init_fence();
        tma_prefetch_desc(&ymap);
        tma_prefetch_desc(&wmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 2 * D);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    if (warp == 0) {
        // ---- producer: (dy shifted by j, W slice of offset p + j * stride), 64 reduction columns per stage
        bool ok = true;
        int i = 0;
        for (int pi = 0; pi < p.phases && ok; ++pi) {
            for (int q = 0; q < per_phase && ok; ++q, ++i) {
                const int st = i % kLcDxStages;
                if (lane == 0) {
                    ok = mbar_wait(&empty[st], ((i / kLcDxStages) & 1) ^ 1, status) && ok;
                    mbar_expect_tx(&full[st], (uint32_t)(kA + kB));
                    const int j = q / KH, kh = q % KH;
                    const int k = p0 + pi + j * p.stride;
                    tma_load_2d(smem_u32(sA + st * kA), &ymap, h * D + kh * 64, m0 - j, &full[st]);
#pragma unroll
                    for (int nh = 0; nh < KH; ++nh)
                        tma_load_2d(smem_u32(sB + st * kB + nh * (64 * 128)), &wmap, kh * 64, (h * p.ks + k) * D + nh * 64, &full[st]);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        const bool leader = elect_one();
        constexpr uint32_t idesc = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, false);
        bool ok = true;
        int i = 0;
        for (int pi = 0; pi < p.phases && ok; ++pi) {
            const int buf = pi & 1;
            ok = mbar_wait(&acc_empty[buf], ((pi >> 1) & 1) ^ 1, status) && ok;
            tc_fence_after();
            for (int q = 0; q < per_phase && ok; ++q, ++i) {
                const int st = i % kLcDxStages;
                ok = mbar_wait(&full[st], (i / kLcDxStages) & 1, status) && ok;
                tc_fence_after();
                if (leader) {
#pragma unroll
                    for (int k16 = 0; k16 < 4; ++k16) {
                        const uint64_t ad = umma_desc_sw128(smem_u32(sA + st * kA) + k16 * 32, 16, 1024);
                        const uint64_t bd = umma_desc_sw128(smem_u32(sB + st * kB) + k16 * 32, 16, 1024);
                        umma_ss(tbase + buf * D, ad, bd, idesc, (q > 0 || k16 > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[st]);
                    if (q == per_phase - 1) umma_commit(&acc_full[buf]);
                }
                __syncwarp();
            }
        }
    } else {
        // ---- epilogue: thread = one m (TMEM lane quarter = warp % 4), one row of dx per phase
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        for (int pi = 0; pi < p.phases && ok; ++pi) {
            const int buf = pi & 1;
            ok = mbar_wait(&acc_full[buf], (pi >> 1) & 1, status) && ok;
            tc_fence_after();
            const int64_t t = (int64_t)(m0 + r) * p.stride + p0 + pi;
            const bool valid = ok && t < p.L;
            ET* dst = reinterpret_cast<ET*>(p.dx) + (t * p.H + h) * D;
#pragma unroll
            for (int cc = 0; cc < D; cc += 32) {
                uint32_t v[32];
                tmem_ld32(tbase + lane_off + buf * D + cc, v);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 u;
                        u.x = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
                        u.y = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
                        u.z = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
                        u.w = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
                        *reinterpret_cast<uint4*>(dst + cc + q4 * 8) = u;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, 2 * D);
}

template <int D, typename ET>
static cudaError_t launch_dx(const LcDxParams& p, const CUtensorMap& ymap, const CUtensorMap& wmap, cudaStream_t stream) {
    constexpr int smem = kLcDxStages * (128 * 128 + D * 128) + 256;
    auto kern = linear_compress_dx_kernel<D, ET>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const int m_rows = (p.L + p.stride - 1) / p.stride;
    kern<<<dim3((unsigned)((m_rows + 127) / 128), (unsigned)p.H, (unsigned)(p.stride / p.phases)), 192, smem, stream>>>(p, ymap, wmap);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ dW
template <typename ET>
struct LcDwParams {
    const ET* x;  int64_t x_sn;     // [N, H, D], token stride in elements
    const ET* dy;                   // [sum n_b, H, D] contiguous
    const int32_t* cu;              // [batch + 1] token offsets
    int batch, H, ks, stride;
    ET* dw;                         // [H, ks * D, D]
    int* status;
};

constexpr int kLcDwStages = 3;

template <int D, typename ET>
__global__ void __launch_bounds__(256) linear_compress_dw_kernel(const LcDwParams<ET> p) {
    constexpr int KPC = 128 / D;                  // window offsets per CTA (M = 128 input features in all)
    constexpr int KH = D / 64;                    // 64-column slabs of a dy row
    constexpr int kSlab = 128 * 128;              // 128 windows x 64 elements
    constexpr int kX = 2 * kSlab, kY = KH * kSlab, kStage = kX + kY;
    constexpr int CY = D / 8;                     // 16-byte chunks of a dy row
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kLcDwStages * kStage);
    uint64_t* full = bars;                        // [stages] 128 arrivals (one per producer thread, when its copies landed)
    uint64_t* empty = bars + kLcDwStages;         // [stages]
    uint64_t* acc_full = bars + 2 * kLcDwStages;
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 2 * kLcDwStages + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k0 = blockIdx.x * KPC, h = blockIdx.y;
    int* status = p.status;
    if (tid == 0) {
        for (int i = 0; i < kLcDwStages; ++i) { mbar_init(&full[i], 128); mbar_init(&empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_init_fence();
    }
    if (warp == 4) tmem_alloc(&tmem_slot, D < 32 ? 32 : D);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    // tiles of 128 windows over all sequences
    int nitems = 0;
    for (int b = 0; b < p.batch; ++b) {
        const int L = __ldg(p.cu + b + 1) - __ldg(p.cu + b);
        const int n = L >= p.ks ? (L - p.ks) / p.stride + 1 : 0;
        nitems += (n + 127) / 128;
    }
    if (warp < 4) {
        // ---- producers: thread t copies 16-byte chunk t % 16 of the rows t / 16 + 8 i of the x tile (a half-warp covers the
        // 256 bytes of one window: both 64-feature halves of offset k0 when d = 128, offsets k0 and k0 + 1 when d = 64),
        // and chunk t % CY of the rows t / CY + (128 / CY) i of the dy tile
        const int xc = tid & 15, xr0 = tid >> 4;
        const int yc = tid % CY, yr0 = tid / CY;
        constexpr int YSTEP = 128 / CY, YIT = 128 / YSTEP;
        // column of x this thread reads, and the window offset it belongs to
        const int x_k = KPC == 1 ? k0 : k0 + (xc >> 3);
        const int x_col = h * D + (KPC == 1 ? xc * 8 : (xc & 7) * 8);
        const uint32_t x_slab = (uint32_t)(xc >> 3) * kSlab;
        const uint32_t y_slab = (uint32_t)(yc >> 3) * kSlab;
        bool ok = true;
        int i = 0;
        int64_t y0 = 0;
        for (int b = 0; b < p.batch && ok; ++b) {
            const int s_b = __ldg(p.cu + b);
            const int L = __ldg(p.cu + b + 1) - s_b;
            const int n = L >= p.ks ? (L - p.ks) / p.stride + 1 : 0;
            for (int c0 = 0; c0 < n && ok; c0 += 128, ++i) {
                const int st = i % kLcDwStages;
                ok = mbar_wait(&empty[st], ((i / kLcDwStages) & 1) ^ 1, status) && ok;
                const uint32_t sx = smem_u32(smem + st * kStage) + x_slab;
                const uint32_t sy = smem_u32(smem + st * kStage + kX) + y_slab;
#pragma unroll
                for (int it = 0; it < 16; ++it) {
                    const int r = xr0 + it * 8;
                    const bool valid = c0 + r < n;
                    const int64_t row = valid ? (int64_t)s_b + (int64_t)(c0 + r) * p.stride + x_k : 0;
                    cp_async16(sx + sw128_chunk_off(r, xc & 7), p.x + row * p.x_sn + x_col, valid);
                }
#pragma unroll
                for (int it = 0; it < YIT; ++it) {
                    const int r = yr0 + it * YSTEP;
                    const bool valid = c0 + r < n;
                    const int64_t row = valid ? y0 + c0 + r : 0;
                    cp_async16(sy + sw128_chunk_off(r, yc & 7), p.dy + (row * p.H + h) * D + yc * 8, valid);
                }
                cp_async_mbar_arrive_noinc(&full[st]);
            }
            y0 += n;
        }
    } else {
        if (warp == 4) {
            // ---- MMA issuer: dW^T tile (+)= x_tile^T dy_tile, 16 windows per instruction
            const bool leader = elect_one();
            constexpr uint32_t idesc = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, true, true);
            constexpr uint32_t hi_1024 = umma_desc_hi(1024);
            bool ok = true;
            for (int i = 0; i < nitems && ok; ++i) {
                const int st = i % kLcDwStages;
                ok = mbar_wait(&full[st], (i / kLcDwStages) & 1, status) && ok;
                fence_async_smem();
                tc_fence_after();
                if (leader) {
                    const uint32_t a_lo = umma_desc_lo(smem_u32(smem + st * kStage), kSlab);
                    const uint32_t b_lo = umma_desc_lo(smem_u32(smem + st * kStage + kX), kSlab);
#pragma unroll
                    for (int ks16 = 0; ks16 < 8; ++ks16)
                        umma_ss(tbase, umma_desc_pack(a_lo + ks16 * (2048 >> 4), hi_1024), umma_desc_pack(b_lo + ks16 * (2048 >> 4), hi_1024),
                                idesc, (i > 0 || ks16 > 0) ? 1u : 0u);
                    umma_commit(&empty[st]);
                    if (i == nitems - 1) umma_commit(acc_full);
                }
                __syncwarp();
            }
        }
        // ---- epilogue (warps 4..7): thread = one row of dW (TMEM lane = input feature, or offset and feature when d = 64)
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        if (nitems > 0) {
            ok = mbar_wait(acc_full, 0, status);
            tc_fence_after();
        }
        ET* dst = p.dw + ((int64_t)(h * p.ks + k0) * D + r) * D;
#pragma unroll
        for (int cc = 0; cc < D; cc += 32) {
            uint32_t v[32];
            if (nitems > 0) {
                tmem_ld32(tbase + lane_off + cc, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0u;
            }
            if (ok) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 u;
                    u.x = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
                    u.y = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
                    u.z = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
                    u.w = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
                    *reinterpret_cast<uint4*>(dst + cc + q4 * 8) = u;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tbase, D < 32 ? 32 : D);
}

template <int D, typename ET>
static cudaError_t launch_dw(const LcDwParams<ET>& p, cudaStream_t stream) {
    constexpr int smem = kLcDwStages * (2 + D / 64) * 128 * 128 + 256;
    auto kern = linear_compress_dw_kernel<D, ET>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<dim3((unsigned)(p.ks / (128 / D)), (unsigned)p.H), 256, smem, stream>>>(p);
    return cudaGetLastError();
}

template <typename ET>
static int run_bwd(const void* x, int64_t x_stride_n, const void* w, const void* dy, const int32_t* cu_dev, const int32_t* seqlens_host,
                   int batch, int H, int D, int ks, int stride, int dtype, void* dx, void* dw, int32_t* status, cudaStream_t stream) {
    if (dx) {
        CUtensorMap wmap;
        int rc = make_tile_map(&wmap, w, dtype, (int64_t)H * ks * D, D, D, 64);
        if (rc) return rc;
        int64_t tok0 = 0, y0 = 0;
        const int64_t row_bytes = (int64_t)H * D * 2;
        for (int b = 0; b < batch; ++b) {
            const int L = seqlens_host[b];
            if (L < 0) return FSA_ERR_BAD_ARG;
            const int n = L >= ks ? (L - ks) / stride + 1 : 0;
            char* dx_b = (char*)dx + tok0 * row_bytes;
            if (n == 0) {
                // no window covers this sequence: its gradient is zero
                if (L > 0 && cudaMemsetAsync(dx_b, 0, (size_t)(L * row_bytes), stream) != cudaSuccess) return FSA_ERR_CUDA;
            } else {
                CUtensorMap ymap;
                rc = make_tile_map(&ymap, (const char*)dy + y0 * row_bytes, dtype, n, (int64_t)H * D, (int64_t)H * D, 128);
                if (rc) return rc;
                LcDxParams p;
                p.n_cmp = n; p.L = L; p.H = H; p.ks = ks; p.stride = stride; p.phases = stride < 4 ? stride : 4;
                p.dx = dx_b; p.status = status;
                const cudaError_t e = D == 128 ? launch_dx<128, ET>(p, ymap, wmap, stream) : launch_dx<64, ET>(p, ymap, wmap, stream);
                if (e != cudaSuccess) return FSA_ERR_CUDA;
            }
            tok0 += L;
            y0 += n;
        }
    }
    if (dw) {
        LcDwParams<ET> p;
        p.x = (const ET*)x; p.x_sn = x_stride_n; p.dy = (const ET*)dy; p.cu = cu_dev;
        p.batch = batch; p.H = H; p.ks = ks; p.stride = stride; p.dw = (ET*)dw; p.status = status;
        const cudaError_t e = D == 128 ? launch_dw<128, ET>(p, stream) : launch_dw<64, ET>(p, stream);
        if (e != cudaSuccess) return FSA_ERR_CUDA;
    }
    return FSA_OK;
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_linear_compress_bwd(const void* x, int64_t x_stride_n, const void* w, const void* dy, const int32_t* cu_seqlens,
                                       const int32_t* seqlens_host, int batch, int num_heads, int head_dim, int kernel_size,
                                       int kernel_stride, int dtype, void* dx, void* dw, int32_t* status, void* stream_) {
    if (!x || !w || !cu_seqlens || !seqlens_host || batch < 0 || num_heads <= 0 || kernel_size <= 0 || kernel_stride <= 0)
        return FSA_ERR_BAD_ARG;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (head_dim != 64 && head_dim != 128) return FSA_ERR_UNSUPPORTED;
    if (kernel_size % kernel_stride != 0 || (kernel_stride & (kernel_stride - 1)) != 0 || (kernel_size & 1)) return FSA_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)dy & 15) || ((uintptr_t)dx & 15) || ((uintptr_t)dw & 15) || (x_stride_n % 8))
        return FSA_ERR_BAD_ARG;
    if (x_stride_n < (int64_t)num_heads * head_dim) return FSA_ERR_BAD_ARG;
    int64_t total_y = 0;
    for (int b = 0; b < batch; ++b)
        if (seqlens_host[b] >= kernel_size) total_y += (seqlens_host[b] - kernel_size) / kernel_stride + 1;
    if (total_y > 0 && !dy) return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return FSA_ERR_CUDA;   // binds the context
    cudaStream_t stream = (cudaStream_t)stream_;
    return dtype == FSA_DTYPE_BF16
               ? run_bwd<__nv_bfloat16>(x, x_stride_n, w, dy, cu_seqlens, seqlens_host, batch, num_heads, head_dim, kernel_size,
                                        kernel_stride, dtype, dx, dw, status, stream)
               : run_bwd<__half>(x, x_stride_n, w, dy, cu_seqlens, seqlens_host, batch, num_heads, head_dim, kernel_size,
                                 kernel_stride, dtype, dx, dw, status, stream);
}
