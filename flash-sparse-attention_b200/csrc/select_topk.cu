// Top-k block selection from the compressed-attention scores.
//
// Replaces score_kernel + _transform_score_kernel + the torch topk / sort / mask tail of the
// reference (nsa_ref/ops/compressed_attention.py:833-1158 and :1274-1315, the per-KV-head path the
// layer uses).  Input: the raw dot products q.k of the FIRST query head of every GQA group against
// the compressed keys of one sequence (a plain library GEMM makes them), and that head's lse.
// One warp per (kv head, token):
//   p[c]   = exp2(qk[c] * scale * log2e - lse)        for visible c (t >= c*stride + ks - 1), else 0   (:897-912)
//   bs[b]  = sum_o w[o] * p[b * (BK/stride) - (ks/stride - 1) + o], out-of-range terms 0              (:1046-1067)
//            w = histogram of i + j, i < ks/stride, j < BK/stride                                      (:1105-1115)
//   bs[b]  = +inf for b < init_blocks and for b <= t/BK < b + local_blocks                             (:1068-1075)
//   bs     rounded to bf16                                                                             (:1307-1308)
//   top min(T, #causal blocks) by (score descending, block index ascending); ascending output; -1 tail (:1309-1313)
// The reference's tie order is whatever torch.topk does; here it is stated: lower block index wins.
// Blocks after the token's own block only ever tie at score 0 with higher indices, so they are never
// preferred over a causal block; the reference masks them to -1 afterwards, which is the same result.
#include "../../include/fsa_sm100.h"
#include "sm100_prims.cuh"

namespace fsa {

constexpr int kMaxW = 16;

struct TopkParams {
    const float* qk;      // [Hk, L, ld]
    int64_t ld;
    const float* lse;     // [Hq, N] log2 units
    int64_t N;
    int seq_start, L, ncmp, Hk, G;
    float scale_log2;
    int ks, stride, BK, init_blocks, local_blocks, max_blocks, T_out;
    int nw;               // number of weights
    float w[kMaxW];
    int32_t* out;         // [Hk, N, T_out]
    int smem_p;           // floats of p per warp (ncmp rounded up)
};

__global__ void __launch_bounds__(128) select_topk_kernel(const TopkParams p) {
    extern __shared__ float smem_f[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* ps = smem_f + (size_t)warp * (p.smem_p + p.max_blocks + 64);
    float* bs = ps + p.smem_p;
    int* sel = reinterpret_cast<int*>(bs + p.max_blocks);
    const int64_t wid = (int64_t)blockIdx.x * 4 + warp;
    if (wid >= (int64_t)p.Hk * p.L) return;
    const int h = (int)(wid / p.L), t = (int)(wid % p.L);
    const int n = p.seq_start + t;
    const float lse = p.lse[(int64_t)(h * p.G) * p.N + n];
    // visible compressed keys: c * stride + ks - 1 <= t
    int nvis = t >= p.ks - 1 ? (t - (p.ks - 1)) / p.stride + 1 : 0;
    nvis = min(nvis, p.ncmp);
    const float* row = p.qk + ((int64_t)h * p.L + t) * p.ld;
    const int bq = t / p.BK;                 // the token's own block
    const int nb = min(bq + 1, p.max_blocks);   // causal candidates
    const int bstride = p.BK / p.stride, pad = p.ks / p.stride - 1;
    // probabilities of the compressed keys the candidate blocks can touch; eight loads in flight per lane, none past
    // the visible keys
    const int cmax = min(p.ncmp, nb * bstride + p.nw);
    for (int c0 = 0; c0 < cmax; c0 += 256) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * 32 + lane;
            v[j] = c < nvis ? row[c] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * 32 + lane;
            if (c < cmax) ps[c] = c < nvis ? exp2f(fmaf(v[j], p.scale_log2, -lse)) : 0.f;
        }
    }
    __syncwarp();
    for (int b = lane; b < nb; b += 32) {
        float s = 0.f;
        for (int o = 0; o < p.nw; ++o) {
            int c = b * bstride - pad + o;
            float v = (c >= 0 && c < cmax) ? ps[c] : 0.f;
            s += v * p.w[o];
        }
        if (b < p.init_blocks || (bq >= b && bq < b + p.local_blocks)) s = INFINITY;
        bs[b] = __bfloat162float(__float2bfloat16(s));
    }
    __syncwarp();
    const int nsel = min(p.T_out, nb);
    for (int r = 0; r < nsel; ++r) {
        // lane-local best (score descending, index ascending), then warp argmax
        float best = -INFINITY; int bi = 0x7fffffff;
        for (int b = lane; b < nb; b += 32) {
            float v = bs[b];
            if (v > best || (v == best && b < bi)) { best = v; bi = b; }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { sel[r] = bi; bs[bi] = -INFINITY; }   // scores are >= 0 or +inf: -inf marks "taken"
        __syncwarp();
    }
    // ascending order by rank counting (indices are distinct), -1 tail
    int32_t* out = p.out + ((int64_t)h * p.N + n) * p.T_out;
    for (int i = lane; i < p.T_out; i += 32) {
        if (i >= nsel) { out[i] = -1; }
    }
    for (int i = lane; i < nsel; i += 32) {
        int v = sel[i], rank = 0;
        for (int j = 0; j < nsel; ++j) rank += sel[j] < v;
        out[rank] = v;
    }
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_select_topk_seq(const float* qk, int64_t ld, const float* lse, int64_t total_tokens, int seq_start, int seq_len,
                                   int num_cmp, int num_kv_heads, int group, float sm_scale, int kernel_size, int kernel_stride,
                                   int block_size, int init_blocks, int local_blocks, int max_blocks, int topk_out,
                                   int32_t* topk_idx, void* stream_) {
    if (!qk || !lse || !topk_idx) return FSA_ERR_BAD_ARG;
    if (seq_len < 0 || num_cmp < 0 || num_kv_heads <= 0 || group <= 0 || kernel_size <= 0 || kernel_stride <= 0 || block_size <= 0)
        return FSA_ERR_BAD_ARG;
    if (kernel_size % kernel_stride || block_size % kernel_stride) return FSA_ERR_UNSUPPORTED;
    if (topk_out <= 0 || topk_out > 64 || max_blocks <= 0) return FSA_ERR_UNSUPPORTED;
    if (seq_len == 0) return FSA_OK;
    TopkParams p;
    p.qk = qk; p.ld = ld; p.lse = lse; p.N = total_tokens;
    p.seq_start = seq_start; p.L = seq_len; p.ncmp = num_cmp; p.Hk = num_kv_heads; p.G = group;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.ks = kernel_size; p.stride = kernel_stride; p.BK = block_size;
    p.init_blocks = init_blocks; p.local_blocks = local_blocks; p.max_blocks = max_blocks; p.T_out = topk_out;
    const int a = kernel_size / kernel_stride, b = block_size / kernel_stride;
    p.nw = a + b - 1;
    if (p.nw > kMaxW) return FSA_ERR_UNSUPPORTED;
    for (int i = 0; i < kMaxW; ++i) p.w[i] = 0.f;
    for (int i = 0; i < a; ++i)
        for (int j = 0; j < b; ++j) p.w[i + j] += 1.f;
    p.out = topk_idx;
    p.smem_p = (num_cmp + 31) / 32 * 32 + 32;
    size_t smem = (size_t)4 * (p.smem_p + max_blocks + 64) * sizeof(float);
    if (smem > 200 * 1024) return FSA_ERR_UNSUPPORTED;
    (void)cudaGetLastError();
    cudaError_t e = cudaFuncSetAttribute(select_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return FSA_ERR_CUDA;
    int64_t warps = (int64_t)num_kv_heads * seq_len;
    select_topk_kernel<<<(unsigned)((warps + 3) / 4), 128, smem, (cudaStream_t)stream_>>>(p);
    return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}
