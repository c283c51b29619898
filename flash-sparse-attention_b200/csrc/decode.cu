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
};

template <int D, int G, typename ET>
__global__ void __launch_bounds__(128) decode_partial_kernel(const DecodeParams p) {
    extern __shared__ float dsm[];
    float* sq = dsm;                       // [G][D]
    float* ss = sq + G * D;                // [G][chunk]
    float* so = ss + G * p.chunk;          // [G][D] reduction buffer
    const int tid = threadIdx.x;
    const int c = blockIdx.x % p.nchunk;
    const int r = (blockIdx.x / p.nchunk) % p.R;
    const int h = (blockIdx.x / (p.nchunk * p.R)) % p.Hk;
    const int b = blockIdx.x / (p.nchunk * p.R * p.Hk);
    const int P = p.R * p.nchunk, pidx = r * p.nchunk + c;
    const int lo_r = p.rng_lo[((int64_t)b * p.Hk + h) * p.R + r];
    const int hi_r = p.rng_hi[((int64_t)b * p.Hk + h) * p.R + r];
    const int lo = lo_r + c * p.chunk;
    const int hi = min(hi_r, lo + p.chunk);
    const int64_t pbase = ((int64_t)b * p.Hq + h * G) * P + pidx;     // + g * P
    if (lo_r < 0 || lo >= hi) {
        if (tid < G) p.ml[pbase + (int64_t)tid * P] = make_float2(-INFINITY, 0.f);
        return;
    }
    const int n = hi - lo;
    const ET* q = (const ET*)p.q + ((int64_t)b * p.Hq + h * G) * D;
    for (int i = tid; i < G * D; i += 128) { sq[i] = (float)q[i]; so[i] = 0.f; }
    __syncthreads();
    constexpr int TPK = D / 8;             // threads per key row (16-byte loads)
    constexpr int KPI = 128 / TPK;         // keys per iteration
    const int part = tid % TPK, kg = tid / TPK;
    // ---- scores
    for (int k0 = 0; k0 < n; k0 += KPI) {
        const int key = k0 + kg;
        float acc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) acc[g] = 0.f;
        if (key < n) {
            uint4 u = *reinterpret_cast<const uint4*>((const ET*)p.k + (int64_t)(lo + key) * p.kv_sn + h * D + part * 8);
            const uint32_t* pu = &u.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 x = ElemTraits<ET>::unpack2(pu[i]);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] += x.x * sq[g * D + part * 8 + 2 * i] + x.y * sq[g * D + part * 8 + 2 * i + 1];
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int o = TPK / 2; o; o >>= 1) acc[g] += __shfl_xor_sync(0xffffffffu, acc[g], o);
            if (part == 0 && key < n) ss[g * p.chunk + key] = acc[g] * p.scale_log2;
        }
    }
    __syncthreads();
    if (p.scores && r == 0)
        for (int i = tid; i < n; i += 128) p.scores[((int64_t)b * p.Hk + h) * p.scores_ld + (lo - lo_r) + i] = ss[i];
    // ---- per-head max and sum (warp g handles head g, g + 4, ...)
    __shared__ float sm_m[32], sm_l[32];
    for (int g = tid >> 5; g < G; g += 4) {
        const int lane = tid & 31;
        float m = -INFINITY;
        for (int i = lane; i < n; i += 32) m = fmaxf(m, ss[g * p.chunk + i]);
#pragma unroll
        for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int i = lane; i < n; i += 32) {
            float e = exp2f(ss[g * p.chunk + i] - m);
            ss[g * p.chunk + i] = e;
            l += e;
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) { sm_m[g] = m; sm_l[g] = l; }
    }
    __syncthreads();
    // ---- o = sum_key p[key] v[key]
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    for (int k0 = 0; k0 < n; k0 += KPI) {
        const int key = k0 + kg;
        if (key < n) {
            uint4 u = *reinterpret_cast<const uint4*>((const ET*)p.v + (int64_t)(lo + key) * p.kv_sn + h * D + part * 8);
            const uint32_t* pu = &u.x;
            float x[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 t2 = ElemTraits<ET>::unpack2(pu[i]);
                x[2 * i] = t2.x; x[2 * i + 1] = t2.y;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float w = ss[g * p.chunk + key];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(w, x[i], acc[g][i]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&so[g * D + part * 8 + i], acc[g][i]);
    __syncthreads();
    for (int i = tid; i < G * D; i += 128) {
        const int g = i / D;
        p.o_part[(pbase + (int64_t)g * P) * D + (i - g * D)] = so[i];
    }
    if (tid < G) p.ml[pbase + (int64_t)tid * P] = make_float2(sm_m[tid], sm_l[tid]);
}

// o[row, :] = sum_p exp2(m_p - M) o_p / sum_p exp2(m_p - M) l_p ; lse = M + log2(...).  One warp per row.
template <typename OT>
__global__ void __launch_bounds__(256) lse_merge_kernel(const float* __restrict__ o_part, const float2* __restrict__ ml, int64_t rows, int P,
                                                        int PS, int D, OT* __restrict__ o, float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float M = -INFINITY;
    for (int i = lane; i < P; i += 32) M = fmaxf(M, ml[row * PS + i].x);
#pragma unroll
    for (int o_ = 16; o_; o_ >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o_));
    float L = 0.f;
    for (int i = lane; i < P; i += 32) {
        float2 v = ml[row * PS + i];
        if (v.y > 0.f) L += exp2f(v.x - M) * v.y;
    }
#pragma unroll
    for (int o_ = 16; o_; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int i = 0; i < P; ++i) {
            float2 v = ml[row * PS + i];
            if (v.y > 0.f) acc += exp2f(v.x - M) * o_part[(row * PS + i) * D + d];
        }
        o[row * D + d] = (OT)(acc * inv);
    }
    if (lane == 0 && lse) lse[row] = L > 0.f ? M + log2f(L) : -INFINITY;
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

__global__ void __launch_bounds__(128) decode_topk_kernel(const DecodeTopkParams p) {
    extern __shared__ float tsm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* bs = tsm + (size_t)warp * (p.max_blocks + 64);
    int* sel = reinterpret_cast<int*>(bs + p.max_blocks);
    const int wid = blockIdx.x * 4 + warp;
    if (wid >= p.B * p.Hk) return;
    const int b = wid / p.Hk, h = wid % p.Hk;
    const int t = p.seq_len[b] - 1;
    const int ncmp = p.ncmp[b];
    const float lse = p.lse[(int64_t)b * p.Hq + h * p.G];
    const float* row = p.scores + ((int64_t)b * p.Hk + h) * p.ld;
    const int bq = t / p.BK;
    const int nb = min(bq + 1, p.max_blocks);
    const int bstride = p.BK / p.stride, pad = p.ks / p.stride - 1;
    for (int blk = lane; blk < nb; blk += 32) {
        float s = 0.f;
        for (int o = 0; o < p.nw; ++o) {
            int c = blk * bstride - pad + o;
            float v = (c >= 0 && c < ncmp) ? exp2f(row[(int64_t)(c / p.shard_len) * p.shard_stride + c % p.shard_len] - lse) : 0.f;
            s += v * p.w[o];
        }
        if (blk < p.init_blocks || (bq >= blk && bq < blk + p.local_blocks)) s = INFINITY;
        bs[blk] = __bfloat162float(__float2bfloat16(s));
    }
    __syncwarp();
    const int nsel = min(p.T, nb);
    for (int r = 0; r < nsel; ++r) {
        float best = -INFINITY; int bi = 0x7fffffff;
        for (int blk = lane; blk < nb; blk += 32) {
            float v = bs[blk];
            if (v > best || (v == best && blk < bi)) { best = v; bi = blk; }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { sel[r] = bi; bs[bi] = -INFINITY; }
        __syncwarp();
    }
    int32_t* out = p.out + ((int64_t)b * p.Hk + h) * p.T;
    for (int i = lane; i < p.T; i += 32)
        if (i >= nsel) out[i] = -1;
    for (int i = lane; i < nsel; i += 32) {
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

template <int D, int G, typename ET>
static cudaError_t launch_partial(const DecodeParams& p, cudaStream_t stream) {
    size_t smem = (size_t)(2 * G * D + G * p.chunk) * sizeof(float);
    auto kern = decode_partial_kernel<D, G, ET>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)((int64_t)p.B * p.Hk * p.R * p.nchunk), 128, smem, stream>>>(p);
    return cudaGetLastError();
}

template <int D, typename ET>
static cudaError_t dispatch_g(int G, const DecodeParams& p, cudaStream_t stream) {
    switch (G) {
        case 1: return launch_partial<D, 1, ET>(p, stream);
        case 2: return launch_partial<D, 2, ET>(p, stream);
        case 4: return launch_partial<D, 4, ET>(p, stream);
        case 8: return launch_partial<D, 8, ET>(p, stream);
        case 16: return launch_partial<D, 16, ET>(p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace fsa

using namespace fsa;

extern "C" int fsa_decode_attn_partial(const void* q, const void* k, const void* v, int64_t kv_stride_n, const int32_t* rng_lo,
                                       const int32_t* rng_hi, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                                       int num_ranges, int chunk, int num_chunks, int dtype, float sm_scale, float* o_part,
                                       float* ml, float* scores, int64_t scores_ld, void* stream) {
    if (!q || !k || !v || !rng_lo || !rng_hi || !o_part || !ml) return FSA_ERR_BAD_ARG;
    if (batch <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || num_ranges <= 0 || chunk <= 0 || num_chunks <= 0)
        return FSA_ERR_BAD_ARG;
    if (chunk > 1024 || (kv_stride_n % 8) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15)) return FSA_ERR_BAD_ARG;
    const int G = num_q_heads / num_kv_heads;
    DecodeParams p;
    p.q = q; p.k = k; p.v = v; p.kv_sn = kv_stride_n; p.rng_lo = rng_lo; p.rng_hi = rng_hi;
    p.B = batch; p.Hq = num_q_heads; p.Hk = num_kv_heads; p.R = num_ranges; p.chunk = chunk; p.nchunk = num_chunks;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.o_part = o_part; p.ml = (float2*)ml; p.scores = scores; p.scores_ld = scores_ld;
    (void)cudaGetLastError();
    cudaError_t e = cudaErrorInvalidValue;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == FSA_DTYPE_BF16) {
        if (head_dim == 128) e = dispatch_g<128, __nv_bfloat16>(G, p, st);
        else if (head_dim == 64) e = dispatch_g<64, __nv_bfloat16>(G, p, st);
        else return FSA_ERR_UNSUPPORTED;
    } else if (dtype == FSA_DTYPE_FP16) {
        if (head_dim == 128) e = dispatch_g<128, __half>(G, p, st);
        else if (head_dim == 64) e = dispatch_g<64, __half>(G, p, st);
        else return FSA_ERR_UNSUPPORTED;
    } else {
        return FSA_ERR_BAD_ARG;
    }
    if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
    return e == cudaSuccess ? FSA_OK : FSA_ERR_CUDA;
}

extern "C" int fsa_lse_merge(const float* o_part, const float* ml, int64_t rows, int num_partials, int part_stride, int head_dim, int out_dtype,
                             void* o, float* lse, void* stream) {
    if (!o_part || !ml || !o || rows < 0 || num_partials <= 0 || part_stride < num_partials || head_dim <= 0) return FSA_ERR_BAD_ARG;
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
    size_t smem = (size_t)4 * (max_blocks + 64) * sizeof(float);
    if (smem > 200 * 1024) return FSA_ERR_UNSUPPORTED;
    (void)cudaGetLastError();
    cudaError_t e = cudaFuncSetAttribute(decode_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return FSA_ERR_CUDA;
    decode_topk_kernel<<<(unsigned)((batch * num_kv_heads + 3) / 4), 128, smem, (cudaStream_t)stream>>>(p);
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
