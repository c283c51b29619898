// K/V compression by a strided linear projection (forward), as a tcgen05 GEMM that reads the overlapping token windows
// in place.
//
// Replaces linear_compress_fwd_kernel of the reference (nsa_ref/ops/linear_compress.py:28-131, launched at :334-398):
//     y[c, h, :] = sum_{k < ks} x[s_b + c * stride + k, h, :] @ W[h, k * d : (k + 1) * d, :]      c < n_b
//     n_b = floor((L_b - ks) / stride) + 1, or 0 when L_b < ks                                     (:334-337)
// and the bias of the intra-block position embedding, bias[h, :] = sum_{k, d'} pe[h, k, d'] W[h, k * d + d', :], which the
// reference adds to the rounded product in the activation dtype (:497-501).
//
// Per head this is the GEMM [n_b, ks * d] x [ks * d, d] whose left operand is never materialised: a 3-D tensor map over
// the sequence's rows of x -- dims (column, window c, offset k), strides (1, stride * row, row): overlapping -- lets TMA
// fetch the 64-column slab (k, half of d) of 128 consecutive windows straight into a swizzled K-major tile; windows
// past n_b are out of the map's bounds and read as zero.  One CTA = 128 windows of one sequence x one head; a producer
// warp streams (A slab, W slab) stages through a four-stage mbarrier ring, one elected thread issues the MMAs (M = 128,
// N = d, fp32 in TMEM), four warps round the accumulator to the activation dtype, add the bias and store the rows.
// There is one launch per sequence (the map's base is the sequence's first row).
#include "../../include/fsa_sm100.h"
#include "sm100_prims.cuh"

namespace fsa {

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int box_rows);
int make_tile_map_3d(CUtensorMap* map, const void* base, int dtype, int64_t d0, int64_t d1, int64_t d2, int64_t stride1,
                     int64_t stride2, int box1);

struct LcParams {
    int n_cmp;        // windows of this sequence
    int y_row0;       // first output row of this sequence
    int H, ks;
    const void* bias; // [H, D] activation dtype, or null
    void* y;          // [sum n_b, H, D]
    int* status;
};

constexpr int kLcStages = 4;

template <int D, typename ET>
__global__ void __launch_bounds__(192) linear_compress_fwd_kernel(const LcParams p, const __grid_constant__ CUtensorMap amap,
                                                                 const __grid_constant__ CUtensorMap wmap) {
    constexpr int kA = 128 * 128, kB = 64 * D * 2;        // one stage: 128 windows x 64 columns, 64 weight rows x D columns
    constexpr int kSlabsPerK = D / 64;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sA = smem;
    uint8_t* sB = sA + kLcStages * kA;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + kLcStages * kB);
    uint64_t* full = bars;                  // [stages]
    uint64_t* empty = bars + kLcStages;     // [stages]
    uint64_t* acc_full = bars + 2 * kLcStages;
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 2 * kLcStages + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c0 = blockIdx.x * 128, h = blockIdx.y;
    const int nslab = p.ks * kSlabsPerK;
    int* status = p.status;
    if (tid == 0) {
        for (int i = 0; i < kLcStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_init_fence();
        tma_prefetch_desc(&amap);
        tma_prefetch_desc(&wmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, D);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    if (warp == 0) {
        // ---- producer
        bool ok = true;
        for (int i = 0; i < nslab && ok; ++i) {
            const int st = i % kLcStages;
            if (lane == 0) {
                ok = mbar_wait(&empty[st], ((i / kLcStages) & 1) ^ 1, status) && ok;
                mbar_expect_tx(&full[st], (uint32_t)(kA + kB));
                const int k = i / kSlabsPerK, dh = i % kSlabsPerK;
                tma_load_3d(smem_u32(sA + st * kA), &amap, h * D + dh * 64, c0, k, &full[st]);
#pragma unroll
                for (int nh = 0; nh < D / 64; ++nh)
                    tma_load_2d(smem_u32(sB + st * kB + nh * (64 * 128)), &wmap, nh * 64, (h * p.ks * D) + i * 64, &full[st]);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        const bool leader = elect_one();
        constexpr uint32_t idesc = umma_idesc(ElemTraits<ET>::kIsBF16, 128, D, false, true);
        bool ok = true;
        for (int i = 0; i < nslab && ok; ++i) {
            const int st = i % kLcStages;
            ok = mbar_wait(&full[st], (i / kLcStages) & 1, status) && ok;
            tc_fence_after();
            if (leader) {
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16) {
                    const uint64_t ad = umma_desc_sw128(smem_u32(sA + st * kA) + k16 * 32, 16, 1024);
                    const uint64_t bd = umma_desc_sw128(smem_u32(sB + st * kB) + k16 * 2048, 64 * 128, 1024);
                    umma_ss(tbase, ad, bd, idesc, (i > 0 || k16 > 0) ? 1u : 0u);
                }
                umma_commit(&empty[st]);
                if (i == nslab - 1) umma_commit(acc_full);
            }
            __syncwarp();
        }
    } else {
        // ---- epilogue: thread = one window (TMEM lane quarter = warp % 4)
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const bool ok = mbar_wait(acc_full, 0, status);
        tc_fence_after();
        const bool valid = ok && c0 + r < p.n_cmp;
        ET* dst = reinterpret_cast<ET*>(p.y) + ((int64_t)(p.y_row0 + c0 + r) * p.H + h) * D;
        const ET* bias = p.bias ? reinterpret_cast<const ET*>(p.bias) + (int64_t)h * D : nullptr;
#pragma unroll
        for (int cc = 0; cc < D; cc += 32) {
            uint32_t v[32];
            tmem_ld32(tbase + lane_off + cc, v);
            tmem_ld_wait();
            if (valid) {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // the product rounded to the activation dtype, then the bias added in that dtype
                        uint32_t pk = ElemTraits<ET>::pack2(__uint_as_float(v[q4 * 8 + 2 * j]), __uint_as_float(v[q4 * 8 + 2 * j + 1]));
                        if (bias) {
                            const float2 a = ElemTraits<ET>::unpack2(pk);
                            const float2 bb = ElemTraits<ET>::unpack2(*reinterpret_cast<const uint32_t*>(bias + cc + q4 * 8 + 2 * j));
                            pk = ElemTraits<ET>::pack2(a.x + bb.x, a.y + bb.y);
                        }
                        w[j] = pk;
                    }
                    *reinterpret_cast<uint4*>(dst + cc + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, D);
}

template <int D, typename ET>
static cudaError_t launch_lc(const LcParams& p, const CUtensorMap& amap, const CUtensorMap& wmap, cudaStream_t stream) {
    constexpr int smem = kLcStages * (128 * 128 + 64 * D * 2) + 256;
    auto kern = linear_compress_fwd_kernel<D, ET>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kern<<<dim3((unsigned)((p.n_cmp + 127) / 128), (unsigned)p.H), 192, smem, stream>>>(p, amap, wmap);
    return cudaGetLastError();
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_linear_compress_fwd(const void* x, int64_t x_stride_n, const void* w, const void* bias, const int32_t* seqlens_host,
                                       int batch, int num_heads, int head_dim, int kernel_size, int kernel_stride, int dtype, void* y,
                                       int32_t* status, void* stream_) {
    if (!x || !w || !seqlens_host || batch < 0 || num_heads <= 0 || kernel_size <= 0 || kernel_stride <= 0) return FSA_ERR_BAD_ARG;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (head_dim != 64 && head_dim != 128) return FSA_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || (bias && ((uintptr_t)bias & 15)) || (x_stride_n % 8)) return FSA_ERR_BAD_ARG;
    if (x_stride_n < (int64_t)num_heads * head_dim) return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return FSA_ERR_CUDA;   // binds the context
    CUtensorMap wmap;
    int rc = make_tile_map(&wmap, w, dtype, (int64_t)num_heads * kernel_size * head_dim, head_dim, head_dim, 64);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    int64_t tok0 = 0;
    int y_row0 = 0;
    for (int b = 0; b < batch; ++b) {
        const int L = seqlens_host[b];
        if (L < 0) return FSA_ERR_BAD_ARG;
        const int n = L >= kernel_size ? (L - kernel_size) / kernel_stride + 1 : 0;
        if (n > 0) {
            if (!y || ((uintptr_t)y & 15)) return FSA_ERR_BAD_ARG;
            CUtensorMap amap;
            const char* base = (const char*)x + tok0 * x_stride_n * 2;
            rc = make_tile_map_3d(&amap, base, dtype, (int64_t)num_heads * head_dim, n, kernel_size, (int64_t)kernel_stride * x_stride_n,
                                  x_stride_n, 128);
            if (rc) return rc;
            LcParams p;
            p.n_cmp = n; p.y_row0 = y_row0; p.H = num_heads; p.ks = kernel_size; p.bias = bias; p.y = y; p.status = status;
            cudaError_t e;
            if (dtype == FSA_DTYPE_BF16)
                e = head_dim == 128 ? launch_lc<128, __nv_bfloat16>(p, amap, wmap, stream) : launch_lc<64, __nv_bfloat16>(p, amap, wmap, stream);
            else
                e = head_dim == 128 ? launch_lc<128, __half>(p, amap, wmap, stream) : launch_lc<64, __half>(p, amap, wmap, stream);
            if (e != cudaSuccess) return FSA_ERR_CUDA;
        }
        tok0 += L;
        y_row0 += n;
    }
    return FSA_OK;
}
