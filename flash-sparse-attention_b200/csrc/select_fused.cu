// Fused top-k block selection: q.k^T, probabilities, block scores and the top-k ids in one kernel, without any
// score tensor in global memory.
//
// Replaces score_kernel + _transform_score_kernel + the torch topk / sort / mask tail of the reference
// (nsa_ref/ops/compressed_attention.py:833-1158 and :1274-1315, the per-KV-head path the layer uses; the reference's
// own unfinished fusion is fsa/ops/fused_score_kernels.py:15-145).  The reference materialises the probabilities
// [1, N, max_cmp] fp32 per KV head and the block scores [1, N, max_blocks] fp32; here nothing larger than the ids
// [Hk, N, T] leaves the chip.
//
// One CTA (128 threads) = 128 consecutive query tokens of one sequence x one KV head (the FIRST query head of the group
// scores for the whole group, :897-912 with the slicing at :1280-1283).  The Q tile is loaded once by TMA; the
// compressed keys of the sequence stream through a two-stage TMA ring in tiles of 128 keys; S = Q K^T (M = N = 128,
// tcgen05, fp32 in one of two TMEM buffers) for tile kt + 1 is issued before tile kt is evaluated.  One thread owns one
// query row:
//   p[c]  = exp2(s[c] * scale * log2e - lse)   for visible c (t >= c * stride + ks - 1), else 0              (:897-912)
//   bs[b] = sum_o w[o] * p[b * BS - (A - 1) + o], added in ascending o, out-of-range terms 0                  (:1046-1067)
//           A = ks / stride, BS = block_size / stride, w = histogram of i + j, i < A, j < BS                  (:1105-1115)
//   bs[b] = +inf for b < init_blocks and for b <= t / block_size < b + local_blocks                           (:1068-1075)
//   bs rounded to bf16                                                                                         (:1307-1308)
// and keeps the best min(T, causal blocks) of its row in registers, ordered by (score descending, block ascending):
// blocks arrive in ascending order, so a candidate only enters when it is strictly greater than the current worst
// and bubbles up while strictly greater -- ties go to the lower block index (the reference leaves the tie order to
// torch.topk).  Ascending ids, -1 tail (:1309-1313).
//
// Accumulation order of q.k: the tensor core's (products of 16-bit inputs are exact in fp32; the sums are not
// associative), so a score can differ from another implementation's in its last bits, and an id can differ where two
// block scores are equal after bf16 rounding up to that difference.
#include "../../include/fsa_sm100.h"
#include "sel_common.cuh"

namespace fsa {

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int box_rows);

struct SelFusedParams {
    const float* lse;        // [Hq, N] log2 units (compressed branch)
    const int* cu_q;         // [B + 1]
    const int* cu_k;         // [B + 1] compressed rows
    int64_t N;
    int B, Hk, G;
    float scale_log2;
    int ks, stride, BK, init_blocks, local_blocks, max_blocks, T_out;
    int32_t* out;            // [Hk, N, T_out]
    int* status;             // device status word or null
};

constexpr int kSfRows = 128, kSfKeys = 128;

template <int A, int BS>
struct TapWeights {
    // w[o] = #{(i, j): i < A, j < BS, i + j = o}
    __host__ __device__ static constexpr float w(int o) {
        int lo = o - (BS - 1) > 0 ? o - (BS - 1) : 0;
        int hi = o < A - 1 ? o : A - 1;
        return (float)(hi - lo + 1);
    }
};

template <int D, typename ET, int A, int BS, int TL>
__global__ void __launch_bounds__(128) select_topk_fused_kernel(const SelFusedParams p, const __grid_constant__ CUtensorMap qmap,
                                                               const __grid_constant__ CUtensorMap kmap) {
    constexpr int kQ = kSfRows * D * 2, kK = kSfKeys * D * 2;
    constexpr int PAD = A - 1, NWT = A + BS - 1;
    static_assert(32 % BS == 0, "a group of 32 key columns holds whole blocks");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + kQ;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sK + 2 * kK);
    uint64_t* q_full = bars;          // [1]
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* s_full = bars + 3;      // [2]
    uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 5);

    const int tid = threadIdx.x, warp = tid >> 5;
    // which (sequence, query tile) is this CTA's (every warp finds it, 32 sequences per step)
    int b, n0, ne;
    find_seq_tile(p.cu_q, p.B, kSfRows, (int)blockIdx.x, tid & 31, b, n0, ne);
    if (b < 0) return;
    const int h = blockIdx.y;
    const int L = __ldg(p.cu_q + b + 1) - __ldg(p.cu_q + b);
    const int tok0 = n0 - __ldg(p.cu_q + b);
    const int kbase = __ldg(p.cu_k + b), ncmp = __ldg(p.cu_k + b + 1) - kbase;
    const int t_last = min(L, tok0 + kSfRows) - 1;
    const int nkt = ((t_last / p.BK + 1) * BS + kSfKeys - 1) / kSfKeys;     // key tiles that hold a causal block of the tile
    const bool have_keys = ncmp > 0;       // a sequence shorter than the compression window has none: every probability is 0
    int* status = p.status;

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&s_full[i], 1); }
        mbar_init_fence();
        tma_prefetch_desc(&qmap);
        tma_prefetch_desc(&kmap);
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = tmem_slot;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

    auto load_k = [&](int kt) {
        const int buf = kt & 1;
        mbar_expect_tx(&k_full[buf], (uint32_t)kK);
#pragma unroll
        for (int sl = 0; sl < D / 64; ++sl)
            tma_load_2d(smem_u32(sK + buf * kK + sl * kSfKeys * 128), &kmap, h * D + sl * 64, kbase + kt * kSfKeys, &k_full[buf]);
    };
    constexpr uint32_t idesc = umma_idesc(ElemTraits<ET>::kIsBF16, 128, kSfKeys, false, false);
    auto issue_mma = [&](int kt) {
        const int buf = kt & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t a = smem_u32(sQ + (ks >> 2) * (kSfRows * 128)) + (ks & 3) * 32;
            const uint32_t bb = smem_u32(sK + buf * kK + (ks >> 2) * (kSfKeys * 128)) + (ks & 3) * 32;
            umma_ss(tbase + buf * kSfKeys, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(bb, 16, 1024), idesc, ks > 0);
        }
        umma_commit(&s_full[buf]);
    };

    bool ok = true;
    if (tid == 0 && have_keys) {
        mbar_expect_tx(q_full, (uint32_t)kQ);
#pragma unroll
        for (int sl = 0; sl < D / 64; ++sl)
            tma_load_2d(smem_u32(sQ + sl * kSfRows * 128), &qmap, (h * p.G) * D + sl * 64, n0, q_full);
        load_k(0);
        if (nkt > 1) load_k(1);
        ok = mbar_wait(q_full, 0, status) && ok;
        ok = mbar_wait(&k_full[0], 0, status) && ok;
        tc_fence_after();
        issue_mma(0);
    }

    // this thread's row
    const int t = tok0 + tid;
    const bool valid = t < L;
    const int nvis = (valid && t >= p.ks - 1) ? min((t - (p.ks - 1)) / p.stride + 1, ncmp) : 0;
    const int bq = t / p.BK;
    const int nb = valid ? min(bq + 1, p.max_blocks) : 0;          // causal candidate blocks
    const float lse = nvis > 0 ? __ldg(p.lse + (int64_t)(h * p.G) * p.N + n0 + tid) : 0.f;
    const int nb_warp = __reduce_max_sync(0xffffffffu, nb);       // the TMEM loads below are warp-wide: uniform trip counts
    float best_s[TL];
    int best_i[TL];
#pragma unroll
    for (int i = 0; i < TL; ++i) { best_s[i] = -1.f; best_i[i] = -1; }     // scores are >= 0
    float carry[PAD > 0 ? PAD : 1];
#pragma unroll
    for (int i = 0; i < (PAD > 0 ? PAD : 1); ++i) carry[i] = 0.f;

    for (int kt = 0; kt < nkt; ++kt) {
        const int buf = kt & 1;
        // S(kt) done: its K stage is free; S(kt + 1) can be issued at once (its TMEM buffer was read in iteration kt - 1,
        // before the barrier that ended it)
        if (have_keys) ok = mbar_wait(&s_full[buf], (kt >> 1) & 1, status) && ok;
        tc_fence_after();
        if (tid == 0 && have_keys) {
            if (kt + 1 < nkt) {
                ok = mbar_wait(&k_full[buf ^ 1], ((kt + 1) >> 1) & 1, status) && ok;
                tc_fence_after();
                issue_mma(kt + 1);
            }
            if (kt + 2 < nkt) load_k(kt + 2);
        }
        __syncwarp();
#pragma unroll 1
        for (int c32 = 0; c32 < kSfKeys / 32; ++c32) {
            const int c0 = kt * kSfKeys + c32 * 32;      // first compressed token of this group of columns
            if (c0 - PAD >= nb_warp * BS) break;         // no causal block of any row of this warp is left
            uint32_t v[32];
            if (have_keys) {
                tmem_ld32(tbase + lane_off + buf * kSfKeys + c32 * 32, v);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
            float pv[PAD + 32];
#pragma unroll
            for (int i = 0; i < PAD; ++i) pv[i] = carry[i];
#pragma unroll
            for (int i = 0; i < 32; ++i)
                pv[PAD + i] = (c0 + i < nvis) ? exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -lse)) : 0.f;
#pragma unroll
            for (int i = 0; i < PAD; ++i) carry[i] = pv[32 + i];
#pragma unroll
            for (int j = 0; j < 32 / BS; ++j) {
                const int blk = c0 / BS + j;
                if (blk < nb) {
                    float sc = 0.f;
#pragma unroll
                    for (int o = 0; o < NWT; ++o) sc = __fadd_rn(sc, __fmul_rn(pv[j * BS + o], TapWeights<A, BS>::w(o)));   // (no fused multiply-add: the order and rounding of the sum are part of the result)
                    if (blk < p.init_blocks || (bq >= blk && bq < blk + p.local_blocks)) sc = INFINITY;
                    sc = __bfloat162float(__float2bfloat16(sc));
                    if (sc > best_s[TL - 1]) {
                        best_s[TL - 1] = sc; best_i[TL - 1] = blk;
#pragma unroll
                        for (int i = TL - 1; i > 0; --i) {
                            if (best_s[i] > best_s[i - 1]) {
                                const float ts = best_s[i]; best_s[i] = best_s[i - 1]; best_s[i - 1] = ts;
                                const int ti = best_i[i]; best_i[i] = best_i[i - 1]; best_i[i - 1] = ti;
                            }
                        }
                    }
                }
            }
        }
        tc_fence_before();
        ok = __syncthreads_and(ok);
        if (!ok) break;
    }

    if (valid) {
        // the first min(T_out, nb) entries are the selection; ascending ids, -1 tail
        const int nsel = min(p.T_out, nb);
#pragma unroll
        for (int i = 0; i < TL; ++i)
            if (i >= nsel) best_i[i] = 0x7fffffff;
#pragma unroll
        for (int pass = 0; pass < TL; ++pass) {
#pragma unroll
            for (int i = pass & 1; i + 1 < TL; i += 2) {
                if (best_i[i] > best_i[i + 1]) { const int ti = best_i[i]; best_i[i] = best_i[i + 1]; best_i[i + 1] = ti; }
            }
        }
        int32_t* out = p.out + ((int64_t)h * p.N + n0 + tid) * p.T_out;
#pragma unroll
        for (int i = 0; i < TL; ++i)
            if (i < p.T_out) out[i] = best_i[i] == 0x7fffffff ? -1 : best_i[i];
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, 256);
}

template <int D, typename ET, int A, int BS>
static cudaError_t launch_tl(const SelFusedParams& p, const CUtensorMap& qmap, const CUtensorMap& kmap, int64_t n_items, cudaStream_t stream) {
    constexpr int smem = kSfRows * D * 2 + 2 * kSfKeys * D * 2 + 64;
    const dim3 grid((unsigned)n_items, (unsigned)p.Hk);
    cudaError_t e;
    if (p.T_out <= 16) {
        auto kern = select_topk_fused_kernel<D, ET, A, BS, 16>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        kern<<<grid, 128, smem, stream>>>(p, qmap, kmap);
    } else {
        auto kern = select_topk_fused_kernel<D, ET, A, BS, 32>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        kern<<<grid, 128, smem, stream>>>(p, qmap, kmap);
    }
    return cudaGetLastError();
}

template <int D, typename ET>
static cudaError_t launch_ab(int A, int BS, const SelFusedParams& p, const CUtensorMap& qmap, const CUtensorMap& kmap, int64_t n_items,
                             cudaStream_t stream) {
#define FSA_AB(a, b) if (A == a && BS == b) return launch_tl<D, ET, a, b>(p, qmap, kmap, n_items, stream);
    FSA_AB(2, 4) FSA_AB(2, 2) FSA_AB(2, 8) FSA_AB(1, 4) FSA_AB(4, 4) FSA_AB(4, 8)
#undef FSA_AB
    return cudaErrorInvalidValue;
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_select_topk_fused(const void* q, int64_t q_stride_n, const void* cmp_k, int64_t k_stride_n, const float* lse,
                                     const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int64_t total_tokens,
                                     int64_t total_cmp, int batch, int num_q_heads, int num_kv_heads, int head_dim, int dtype,
                                     float sm_scale, int kernel_size, int kernel_stride, int block_size, int init_blocks,
                                     int local_blocks, int max_blocks, int topk_out, int32_t* topk_idx, int32_t* status, void* stream_) {
    if (!q || !lse || !cu_seqlens_q || !cu_seqlens_k || !topk_idx) return FSA_ERR_BAD_ARG;
    if (total_tokens < 0 || total_cmp < 0 || batch < 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) return FSA_ERR_BAD_ARG;
    if (kernel_size <= 0 || kernel_stride <= 0 || block_size <= 0 || max_blocks <= 0 || topk_out <= 0) return FSA_ERR_BAD_ARG;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (kernel_size % kernel_stride || block_size % kernel_stride) return FSA_ERR_UNSUPPORTED;
    if (topk_out > 32 || (head_dim != 64 && head_dim != 128) || num_kv_heads > 65535) return FSA_ERR_UNSUPPORTED;
    if (((uintptr_t)q & 15) || (q_stride_n % 8) || (total_cmp > 0 && (!cmp_k || ((uintptr_t)cmp_k & 15) || (k_stride_n % 8)))) return FSA_ERR_BAD_ARG;
    if (q_stride_n < (int64_t)num_q_heads * head_dim || (total_cmp > 0 && k_stride_n < (int64_t)num_kv_heads * head_dim)) return FSA_ERR_BAD_ARG;
    if (total_tokens == 0 || batch == 0) return FSA_OK;
    const int A = kernel_size / kernel_stride, BS = block_size / kernel_stride;
    (void)cudaGetLastError();
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return FSA_ERR_CUDA;   // binds the context
    CUtensorMap qmap, kmap;
    int rc = make_tile_map(&qmap, q, dtype, total_tokens, (int64_t)num_q_heads * head_dim, q_stride_n, kSfRows);
    if (rc) return rc;
    // a batch without any compressed token still needs a valid map: it is never loaded from
    const void* kptr = total_cmp > 0 ? cmp_k : q;
    const int64_t krows = total_cmp > 0 ? total_cmp : 1, kstride = total_cmp > 0 ? k_stride_n : q_stride_n;
    rc = make_tile_map(&kmap, kptr, dtype, krows, (int64_t)num_kv_heads * head_dim, kstride, kSfKeys);
    if (rc) return rc;
    SelFusedParams p;
    p.lse = lse; p.cu_q = cu_seqlens_q; p.cu_k = cu_seqlens_k; p.N = total_tokens; p.B = batch; p.Hk = num_kv_heads;
    p.G = num_q_heads / num_kv_heads; p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.ks = kernel_size; p.stride = kernel_stride; p.BK = block_size; p.init_blocks = init_blocks; p.local_blocks = local_blocks;
    p.max_blocks = max_blocks; p.T_out = topk_out; p.out = topk_idx; p.status = status;
    const int64_t n_items = total_tokens / kSfRows + batch;     // >= sum of ceil(L / 128)
    cudaError_t e;
    cudaStream_t st = (cudaStream_t)stream_;
    if (dtype == FSA_DTYPE_BF16)
        e = head_dim == 128 ? launch_ab<128, __nv_bfloat16>(A, BS, p, qmap, kmap, n_items, st) : launch_ab<64, __nv_bfloat16>(A, BS, p, qmap, kmap, n_items, st);
    else
        e = head_dim == 128 ? launch_ab<128, __half>(A, BS, p, qmap, kmap, n_items, st) : launch_ab<64, __half>(A, BS, p, qmap, kmap, n_items, st);
    if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
    return e == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}
