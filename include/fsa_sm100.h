/* C ABI of libfsa_sm100.so: hand-written sm_100a (B200) kernels for Native-Sparse-Attention's
 * selected (top-k block-sparse) attention and the pieces next to it.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host or _out;
 *   - tensors are described by raw pointers, sizes and element strides; the innermost
 *     (head_dim) stride is always 1;
 *   - `dtype`: 0 = bfloat16, 1 = float16 (the type of q/k/v/o/do/dq/dk/dv);
 *   - every entry point enqueues its work on `stream` (a cudaStream_t) and returns without
 *     synchronising; it never allocates device memory: workspaces are caller-owned and their
 *     sizes come from the *_bytes queries;
 *   - return value: 0 on success, negative FSA_ERR_* otherwise; nothing throws, nothing traps.
 *     Device-side problems (a bounded wait that ran out) are recorded in a status word inside
 *     the index workspace and read back with fsa_read_status().
 *
 * Each entry point names the reference interface it replaces (path:line inside the
 * Relaxed-System-Lab/Flash-Sparse-Attention tree).
 */
#ifndef FSA_SM100_H_
#define FSA_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSA_OK 0
#define FSA_ERR_BAD_ARG (-1)        /* null pointer, negative size, misaligned pointer/stride */
#define FSA_ERR_UNSUPPORTED (-2)    /* shape outside the compiled kernels (head_dim, block size, top-k, group) */
#define FSA_ERR_WORKSPACE (-3)      /* workspace smaller than the matching *_bytes query */
#define FSA_ERR_CUDA (-4)           /* a CUDA runtime/driver call failed; see fsa_last_cuda_error() */
#define FSA_ERR_DEVICE_STATUS (-5)  /* fsa_read_status(): a kernel recorded a failure */
#define FSA_ERR_STATIC_LIMIT (-6)   /* fsa_sel_fwd_static(): the problem does not fit the built-in scratch array */

#define FSA_DTYPE_BF16 0
#define FSA_DTYPE_FP16 1

/* Library version and a human-readable string for an error code.  No reference counterpart (the reference raises
 * Python exceptions). */
int fsa_version(void);
const char* fsa_error_string(int code);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread.  No reference
 * counterpart (diagnostics). */
int fsa_last_cuda_error(void);
/* Source line inside the library's API file of that failing call.  No reference counterpart (diagnostics). */
int fsa_last_cuda_error_line(void);

/* Optional kernel timing for benchmarks (off by default; no counterpart in the reference, which
 * times whole operators with CUDA events, utils.py:6-27).  When enabled, the library brackets each
 * named kernel with its own CUDA events on the launching stream (a ring of 64 launches per kernel,
 * restarted by every fsa_profile_enable call); fsa_profile_read() waits for those launches and
 * returns the sum of their durations in milliseconds and how many there were. */
#define FSA_KERNEL_SEL_FWD_MAIN 0
#define FSA_KERNEL_SEL_FWD_REDUCE 1
#define FSA_KERNEL_SEL_BWD_MAIN 2
#define FSA_KERNEL_SEL_BWD_DQ_REDUCE 3
#define FSA_KERNEL_SEL_INDEX 4            /* the index build of a forward (several small kernels) */
#define FSA_KERNEL_RANGE_DENSE 5
int fsa_profile_enable(int on);
int fsa_profile_read(int kernel_id, float* ms_sum_out, int* launches_out);

/* ---------------------------------------------------------------------------------------------
 * Selected attention (fsa/ops/FSA_topk_sparse_attention.py)
 * ------------------------------------------------------------------------------------------- */

/* Size of the index workspace: the inversion "KV block -> (token, slot) entries" that the
 * reference rebuilds with block_to_token / index_mapping / bincount in the forward
 * (FSA_topk_sparse_attention.py:60-135, 622-668, 951-1020) and again with reorder_topk_idx in the
 * backward (nsa_ref/ops/topk_sparse_attention.py:412-476).  The forward fills it; the backward
 * reuses it, so the caller keeps it alive between the two. */
int fsa_sel_index_bytes(int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads, int topk,
                        int block_size, int64_t* bytes_out);

/* Size of the transient forward scratch (per-tile partial outputs in the input dtype and fp32
 * softmax statistics; the reference's o_tiles / l_ij / acc_o_scales buffers, :959-988). */
int fsa_sel_fwd_scratch_bytes(int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads, int head_dim, int topk,
                              int block_size, int64_t* bytes_out);

/* Forward.  Replaces _topk_sparse_attention_fwd_opt (FSA_topk_sparse_attention.py:569-618) as called
 * by FSATopkSparseAttention.forward (:1889-1932).
 *   q [N, Hq, D], k/v [N, Hk, D], o [N, Hq, D] in `dtype`; head stride of k and v must be D;
 *   topk_idx [Hk, N, T] int32 contiguous: block ids local to each sequence, usable ids first,
 *   -1 padding; cu_seqlens [B+1] int32; lse_out [Hq, N] fp32, log2 units (:178 of nsa_ref's kernel). */
int fsa_sel_fwd(const void* q, const void* k, const void* v, const int32_t* topk_idx, const int32_t* cu_seqlens,
                int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads, int head_dim, int topk,
                int block_size, int dtype, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                int64_t v_stride_n, float sm_scale, void* o, int64_t o_stride_n, int64_t o_stride_h, float* lse,
                void* index_ws, int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream);

/* Forward for callers that cannot allocate device memory.  (No counterpart in the reference, whose
 * forward allocates its scratch tensors with torch on every call.)
 *
 * Who needs it: a host program that gave the whole GPU to its own arena at start-up, or one that
 * must not risk the device-wide synchronisation or a late out-of-memory failure of an allocation
 * while it is serving.  Such a caller has no workspace to hand to fsa_sel_fwd, so here the index
 * workspace and the partial-result scratch live in a fixed array of FSA_SEL_STATIC_SCRATCH_BYTES
 * inside the library; every GPU that loads the library holds that array until the process exits.
 *
 * Same inputs, outputs and results as fsa_sel_fwd.  Differences:
 *   - problems whose index workspace plus forward scratch (the two *_bytes queries above, each rounded
 *     up to 1 KiB) exceed FSA_SEL_STATIC_SCRATCH_BYTES are refused with FSA_ERR_STATIC_LIMIT;
 *   - the first call on each device looks up the array's device address (one runtime query, with that
 *     device current); make that first call before any stream capture begins;
 *   - no cudaMalloc / cudaFree or any other allocating call is made, on the first call or later;
 *   - all calls on a device share the one array, and it keeps what the previous call left: the words
 *     that must start at zero are cleared on `stream` by the call itself, but two calls that may
 *     overlap on the GPU (different streams, no ordering between them) race on the array and must be
 *     serialised by the caller;
 *   - device-side failures (a bounded wait that ran out) are recorded in a status word inside the array:
 *     read it with fsa_read_status(NULL, stream, &status), which allocates nothing either;
 *   - there is no workspace to keep for a backward pass: fsa_sel_bwd needs the caller-owned index
 *     workspace of fsa_sel_fwd. */
#define FSA_SEL_STATIC_SCRATCH_BYTES (64u << 20)
int fsa_sel_fwd_static(const void* q, const void* k, const void* v, const int32_t* topk_idx, const int32_t* cu_seqlens,
                       int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads, int head_dim, int topk,
                       int block_size, int dtype, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t v_stride_n, float sm_scale, void* o, int64_t o_stride_n, int64_t o_stride_h, float* lse,
                       void* stream);

/* Size of the transient backward scratch (dQ partials, fp32 dK/dV accumulators, delta): the reference's dq buffer
 * [1, nb-1, max_valid, d] (fsa/ops/FSA_topk_sparse_attention.py:1408-1420), its dk / dv [G, N, Hk, d] staging (:1799-1806)
 * and delta (:1745). */
int fsa_sel_bwd_scratch_bytes(int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                              int topk, int block_size, int64_t* bytes_out);

/* Backward.  Replaces _topk_sparse_attention_bwd_opt (FSA_topk_sparse_attention.py:1715-1884):
 * backward_sum_o_do, backward_dkdv, dq_compute_kernel, dq_reduce_kernel.  `index_ws` is the
 * workspace the forward filled for the same topk_idx / cu_seqlens.
 *   o, d_o, dq [N, Hq, D]; dk, dv [N, Hk, D] contiguous; lse [Hq, N] from the forward. */
int fsa_sel_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                const int32_t* topk_idx, const int32_t* cu_seqlens, int64_t total_tokens, int batch, int num_q_heads,
                int num_kv_heads, int head_dim, int topk, int block_size, int dtype, int64_t q_stride_n,
                int64_t q_stride_h, int64_t k_stride_n, int64_t v_stride_n, int64_t o_stride_n, int64_t o_stride_h,
                int64_t do_stride_n, int64_t do_stride_h, float sm_scale, void* dq, void* dk, void* dv,
                void* index_ws, int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Range attention: the compressed branch and the sliding-window branch
 * ------------------------------------------------------------------------------------------- */

/* Attention in which token n attends the K/V rows kv_lo[n] .. kv_hi[n] (global row ids of k / v, which may
 * have their own packing cu_seqlens_k; nothing when kv_hi[n] < kv_lo[n]; kv_lo may be null = from the start of
 * the sequence).  It runs on the selected-attention kernels: every token "selects" the block_size-row
 * blocks its range touches (at most max_blocks <= 64 of them), rows outside the range are masked.
 *   compressed branch  - replaces CompressedAttention forward/backward and their kernels
 *       (nsa_ref/ops/compressed_attention.py:28-156, 160-545, 762-829): k/v are the compressed tokens,
 *       kv_hi[n] = cu_k[b] + floor((t_local - kernel_size + 1) / kernel_stride), or -1 when t_local < kernel_size - 1
 *       (the mask `t >= c * stride + kernel_size - 1`, :77-80); such rows get o = 0, lse = -inf (:548-553);
 *   sliding window     - replaces flash_attn_varlen_func(causal=True, window_size=(W, -1)) as called in
 *       fsa/module/fsa.py:149-159: kv_lo[n] = max(cu[b], n - W), kv_hi[n] = n.
 * Tensors, strides, dtype, lse (log2 units), workspaces and return codes are as for fsa_sel_fwd / fsa_sel_bwd;
 * fsa_range_attn_bytes returns the three workspace sizes (any out pointer may be null).
 * fsa_range_attn_bwd at head_dim 128 computes dq with a query-tile-major kernel (accumulator in TMEM over the K/V tiles a
 * tile of tokens sees, written once) and dk / dv with the block-major kernel; other head sizes use the block-major kernel
 * for all three. */
int fsa_range_attn_bytes(int64_t total_tokens, int64_t total_kv_rows, int batch, int num_q_heads, int num_kv_heads,
                         int head_dim, int max_blocks, int block_size, int64_t* index_bytes_out,
                         int64_t* fwd_scratch_bytes_out, int64_t* bwd_scratch_bytes_out);
int fsa_range_attn_fwd(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q,
                       const int32_t* cu_seqlens_k, const int32_t* kv_lo, const int32_t* kv_hi, int64_t total_tokens,
                       int64_t total_kv_rows, int batch, int num_q_heads, int num_kv_heads, int head_dim, int max_blocks,
                       int block_size, int dtype, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t v_stride_n, float sm_scale, void* o, int64_t o_stride_n, int64_t o_stride_h, float* lse,
                       void* index_ws, int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream);
int fsa_range_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                       const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* kv_lo,
                       const int32_t* kv_hi, int64_t total_tokens, int64_t total_kv_rows, int batch, int num_q_heads,
                       int num_kv_heads, int head_dim, int max_blocks, int block_size, int dtype, int64_t q_stride_n,
                       int64_t q_stride_h, int64_t k_stride_n, int64_t v_stride_n, int64_t o_stride_n,
                       int64_t o_stride_h, int64_t do_stride_n, int64_t do_stride_h, float sm_scale, void* dq, void* dk,
                       void* dv, void* index_ws, int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes,
                       void* stream);

/* Range attention forward without partial rows: one CTA per tile of consecutive query tokens walks the K/V rows its
 * tokens see and keeps the output accumulator in TMEM (online softmax); o and lse are written once, no index and no
 * scratch are needed.  Same arguments and results as fsa_range_attn_fwd (it replaces the same reference code: the
 * forward of CompressedAttention, nsa_ref/ops/compressed_attention.py:33-190, :762-829, and the sliding-window
 * flash_attn_varlen_func call of fsa/module/fsa.py:149-159).  head_dim 64 or 128, GQA group <= 32.  status: a device int
 * (zeroed by the caller) that receives a non-zero code if a bounded wait ran out, or NULL.
 * fsa_range_attn_bwd needs the tile index that fsa_range_attn_fwd leaves in index_ws; after this forward, build it
 * with fsa_range_attn_index (same max_blocks / block_size as the backward call). */
int fsa_range_attn_fwd_dense(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q,
                             const int32_t* cu_seqlens_k, const int32_t* kv_lo, const int32_t* kv_hi, int64_t total_tokens,
                             int64_t total_kv_rows, int batch, int num_q_heads, int num_kv_heads, int head_dim, int dtype,
                             int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n, int64_t v_stride_n, float sm_scale,
                             void* o, int64_t o_stride_n, int64_t o_stride_h, float* lse, int32_t* status, void* stream);
int fsa_range_attn_index(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* kv_lo, const int32_t* kv_hi,
                         int64_t total_tokens, int64_t total_kv_rows, int batch, int num_q_heads, int num_kv_heads,
                         int max_blocks, int block_size, void* index_ws, int64_t index_ws_bytes, void* stream);

/* K/V compression forward: y[c, h, :] = sum_k x[s_b + c * stride + k, h, :] @ W[h, k*d:(k+1)*d, :] (+ bias[h, :]) for the
 * n_b = floor((L_b - kernel_size) / stride) + 1 windows of every sequence (0 when L_b < kernel_size).  Replaces
 * linear_compress_fwd_kernel (nsa_ref/ops/linear_compress.py:28-131, :334-398) and the bias add of :497-501; the token
 * windows are read in place through a strided tensor map (no unfolded copy).
 *   x [N, H, D] (row stride x_stride_n, head stride D), w [H, kernel_size * D, D] contiguous, bias [H, D] or NULL (added
 *   to the rounded product in the activation dtype, as the reference does), seqlens_host [batch] HOST array of sequence
 *   lengths, y [sum n_b, H, D] contiguous.  head_dim 64 or 128.  One launch per sequence.
 *   status: a device int (zeroed by the caller) that receives a non-zero code if a bounded wait ran out, or NULL. */
int fsa_linear_compress_fwd(const void* x, int64_t x_stride_n, const void* w, const void* bias, const int32_t* seqlens_host,
                            int batch, int num_heads, int head_dim, int kernel_size, int kernel_stride, int dtype, void* y,
                            int32_t* status, void* stream);

/* K/V compression backward without atomics: dx and dW of fsa_linear_compress_fwd from dy.  Replaces
 * linear_compress_bwd_kernel (nsa_ref/ops/linear_compress.py:135-292, launched at :401-470), which scatters both
 * gradients with fp32 tl.atomic_add (:275, :292); here every dx row and every dW row is written once from an fp32
 * accumulator, so the result does not depend on scheduling.
 *   x, w as in the forward; dy [sum n_b, H, D] contiguous; cu_seqlens [batch + 1] DEVICE token offsets and
 *   seqlens_host [batch] the same lengths on the HOST (dx runs one launch per sequence, dW a single launch over all
 *   sequences); dx [N, H, D] contiguous or NULL, dw [H, kernel_size * D, D] contiguous or NULL (a NULL gradient is not
 *   computed).  head_dim 64 or 128, kernel_stride a power of two dividing kernel_size.  The gradient of the bias is
 *   the column sum of dy and is left to the caller. */
int fsa_linear_compress_bwd(const void* x, int64_t x_stride_n, const void* w, const void* dy, const int32_t* cu_seqlens,
                            const int32_t* seqlens_host, int batch, int num_heads, int head_dim, int kernel_size,
                            int kernel_stride, int dtype, void* dx, void* dw, int32_t* status, void* stream);

/* Fused top-k block selection for a varlen batch: q.k^T on the tensor cores, probabilities, block scores and the ids
 * in one kernel; no score tensor is written to memory.  Replaces _get_attention_score / score_kernel, transform_score /
 * _transform_score_kernel and the topk + sort + mask tail (nsa_ref/ops/compressed_attention.py:833-1158, :1274-1315;
 * per-KV-head path) -- the fusion the reference sketches in fsa/ops/fused_score_kernels.py:15-145.
 *   q [N, Hq, D] (row stride q_stride_n, head stride D; the first head of every GQA group is used), cmp_k [Nc, Hk, D]
 *   compressed keys (row stride k_stride_n, head stride D), lse [Hq, N] of the compressed branch (log2 units),
 *   cu_seqlens_q / cu_seqlens_k [B + 1]; topk_idx [Hk, N, topk_out] int32: ascending sequence-local block ids, -1 padded.
 *   Scores are rounded to bf16 as in the reference; ties go to the lower block index.  topk_out = min(topk, max_blocks)
 *   <= 32, max_blocks = ceil(max_seqlen / block_size); head_dim 64 or 128; (kernel_size / stride, block_size / stride)
 *   in {(2,2), (2,4), (2,8), (1,4), (4,4), (4,8)}, else FSA_ERR_UNSUPPORTED (use fsa_select_topk_seq).
 *   status: a device int (zeroed by the caller) that receives a non-zero code if a bounded wait ran out, or NULL. */
int fsa_select_topk_fused(const void* q, int64_t q_stride_n, const void* cmp_k, int64_t k_stride_n, const float* lse,
                          const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int64_t total_tokens, int64_t total_cmp,
                          int batch, int num_q_heads, int num_kv_heads, int head_dim, int dtype, float sm_scale,
                          int kernel_size, int kernel_stride, int block_size, int init_blocks, int local_blocks,
                          int max_blocks, int topk_out, int32_t* topk_idx, int32_t* status, void* stream);

/* Top-k block selection for one sequence.  Replaces _get_attention_score / score_kernel, transform_score /
 * _transform_score_kernel and the topk + sort + mask tail (nsa_ref/ops/compressed_attention.py:833-1158,
 * :1274-1315; per-KV-head path).
 *   qk [Hk, seq_len, ld] fp32: raw dot products of the FIRST query head of each GQA group with the num_cmp
 *   compressed keys of this sequence (a library GEMM); lse [Hq, total_tokens] of the compressed branch (log2);
 *   topk_idx [Hk, total_tokens, topk_out] int32 receives, for the tokens of this sequence, ascending
 *   sequence-local block ids, -1 padded.  Scores are rounded to bf16 as in the reference; ties go to the lower
 *   block index (the reference leaves tie order to torch.topk).  topk_out = min(topk, max_blocks),
 *   max_blocks = ceil(max_seqlen / block_size). */
int fsa_select_topk_seq(const float* qk, int64_t ld, const float* lse, int64_t total_tokens, int seq_start, int seq_len,
                        int num_cmp, int num_kv_heads, int group, float sm_scale, int kernel_size, int kernel_stride,
                        int block_size, int init_blocks, int local_blocks, int max_blocks, int topk_out,
                        int32_t* topk_idx, void* stream);

/* Rotary embedding, half-split layout, positions restarting per sequence.  Replaces the flash-attn
 * apply_rotary_emb call of RotaryEmbedding.forward (nsa_ref/module/rope.py:126-134).  x [total, heads, head_dim]
 * with element strides; cos_tab / sin_tab [table_len, head_dim / 2] in the activation dtype, row p = position
 * start + p * stride (the caller builds the table that way, rope.py:130); out is contiguous.  conj != 0
 * applies the inverse rotation (backward). */
int fsa_rope(const void* x, int64_t x_stride_n, int64_t x_stride_h, const void* cos_tab, const void* sin_tab,
             const int32_t* cu_seqlens, int batch, int64_t total, int heads, int head_dim, int dtype, int conj, void* out,
             void* stream);

/* Gate mix of the three branches (fsa/module/fsa.py:162-167): out = g0 a + g1 b + g2 c with gate [total, 3]
 * (already through the sigmoid) and a, b, c, out contiguous [total, row_elems].  The backward also returns
 * dgate [total, 3] fp32 = row sums of d_out * branch. */
int fsa_gate_mix_fwd(const void* gate, const void* a, const void* b, const void* c, int64_t total, int row_elems, int dtype,
                     void* out, void* stream);
int fsa_gate_mix_bwd(const void* gate, const void* a, const void* b, const void* c, const void* d_out, int64_t total,
                     int row_elems, int dtype, void* da, void* db, void* dc, float* dgate, void* stream);

/* The layer's gate path fused (fsa/module/fsa.py:162-171): gate = sigmoid(x @ w_gate^T) with w_gate [3, hidden] (the
 * Linear's product and the sigmoid each rounded to the activation dtype, as the separate modules round), then
 * out = g0 a + g1 b + g2 c.  x [N, hidden] (row stride x_stride_n), a / b / c / out [N, row_elems] contiguous,
 * gate [N, 3] (written: the backward needs it).  hidden <= 16384.
 * Backward: da, db, dc = g_i d_out; dx [N, hidden] contiguous = the gate path's part of dL/dx; dw_gate [3, hidden];
 * scratch: fsa_gate_proj_mix_scratch_bytes(N, hidden) bytes.  No atomics: dw_gate is summed over token chunks in order. */
int64_t fsa_gate_proj_mix_scratch_bytes(int64_t total, int hidden);
int fsa_gate_proj_mix_fwd(const void* x, int64_t x_stride_n, const void* w_gate, const void* a, const void* b, const void* c,
                          int64_t total, int hidden, int row_elems, int dtype, void* out, void* gate, void* stream);
int fsa_gate_proj_mix_bwd(const void* x, int64_t x_stride_n, const void* w_gate, const void* gate, const void* a, const void* b,
                          const void* c, const void* d_out, int64_t total, int hidden, int row_elems, int dtype, void* da, void* db,
                          void* dc, void* dx, void* dw_gate, float* scratch, int64_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One-step decode (fsa_preview)
 * ------------------------------------------------------------------------------------------- */

/* Partial attention of one query token per sequence over ranges of K/V cache rows.  Replaces
 * forward_kernel_decode and score_kernel_decode (fsa_preview/ops/compressed_attention_decode.py:361-592),
 * _topk_sparse_attention_decode (fsa_preview/ops/selected_attention_decode.py:8-42) and the window call
 * (fsa_preview/module/fsa_decode.py:175-185).
 *   q [B, Hq, D]; k, v [kv_rows, Hk, D] with row stride kv_stride_n (kv_rows bounds the TMA tensor map); rng_lo / rng_hi [B, Hk, R]: range r of
 *   (sequence, kv head) covers the rows [lo, hi) (lo = -1: empty).  Every range is cut into num_chunks chunks
 *   of `chunk` rows (chunk * num_chunks >= the longest range); with ranges_per_partial = n > 1 (num_chunks must
 *   be 1) n consecutive ranges share one softmax and one partial, P = ceil(R / n) * num_chunks; partial
 *   (b, head, (r / n) * num_chunks + c) receives
 *   o_part [B, Hq, P, D] fp32 (unnormalised) and ml [B, Hq, P, 2] = (max logit in log2 units, sum of exp2).
 *   scores (optional) [B, Hk, scores_ld]: the scaled log2 logits of each group's FIRST head over range 0,
 *   the input of fsa_decode_select_topk. */
int fsa_decode_attn_partial(const void* q, const void* k, const void* v, int64_t kv_rows, int64_t kv_stride_n, const int32_t* rng_lo,
                            const int32_t* rng_hi, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                            int num_ranges, int ranges_per_partial, int chunk, int num_chunks, int dtype, float sm_scale,
                            float* o_part, float* ml,
                            float* scores, int64_t scores_ld, void* stream);

/* Device status word of the decode kernels: 0, or 1 after a bounded wait ran out (the step's results are then
 * invalid).  Synchronises with the device.  No reference counterpart. */
int fsa_decode_read_status(int* status_out);

/* Log-sum-exp merge of P partials per row: o = sum w_p o_p / sum w_p l_p, w_p = exp2(m_p - max m), lse = max m +
 * log2 sum w_p l_p: the online-softmax merge of the reference's reduce kernel (fsa/ops/FSA_topk_sparse_attention.py:
 * 139-281) as a stand-alone operator.  Used inside one GPU (chunks, blocks) and across GPUs (after an all-gather of the
 * partials; the reference has no multi-GPU path).  Row r reads partials o_part[(r * part_stride + p) * head_dim ...] and
 * ml[(r * part_stride + p) * 2 ...], p < num_partials, so a sub-range of a wider partial buffer can be merged in
 * place (offset the pointers).  out_dtype: 0 bf16, 1 fp16, 2 fp32; lse may be null. */
int fsa_lse_merge(const float* o_part, const float* ml, int64_t rows, int num_partials, int part_stride, int head_dim,
                  int out_dtype, void* o, float* lse, void* stream);

/* Last kernel of a one-GPU decode step: LSE-merges the selected-block partials [0, num_sel_partials) and the window
 * partials [num_sel_partials, + num_win_partials) of every row (rows = batch * num_q_heads, partial stride part_stride)
 * and mixes the three branches with the sequence's gates [batch, 3] (after the sigmoid, activation dtype):
 * out = g0 o_cmp + g1 o_sel + g2 o_win, all [rows, head_dim] in the activation dtype.  Replaces the two merges and the
 * gate mix of fsa_preview/module/fsa_decode.py:188-193 by one launch. */
int fsa_decode_finish(const float* o_part, const float* ml, int64_t rows, int num_sel_partials, int num_win_partials,
                      int part_stride, int head_dim, int num_q_heads, int dtype, const void* o_cmp, const void* gate, void* out,
                      void* stream);

/* Top-k block ids for the decoded token of every sequence, from the scores buffer of the compressed branch
 * and its merged lse [B, Hq].  Same scoring, bf16 rounding and tie rule as fsa_select_topk_seq, evaluated at
 * t = seq_len[b] - 1 (the reference evaluates the "local blocks" rule at t = 0,
 * fsa_preview/ops/compressed_attention_decode.py:329-355, which does not match its own prefill).
 * When the compressed cache is sharded over GPUs the gathered score buffers stay shard-major: compressed token c
 * is read at scores[(c / shard_len) * shard_stride + row * scores_ld + c % shard_len] (one GPU: shard_len >= num_cmp).
 * topk_idx [B, Hk, topk]: ascending block ids, -1 padded. */
int fsa_decode_select_topk(const float* scores, int64_t scores_ld, int shard_len, int64_t shard_stride, const float* lse, const int32_t* seq_len,
                           const int32_t* num_cmp, int batch, int num_q_heads, int num_kv_heads, int kernel_size,
                           int kernel_stride, int block_size, int init_blocks, int local_blocks, int topk, int max_blocks,
                           int32_t* topk_idx, void* stream);

/* Visible compressed tokens of the decoded row, num_cmp[b] = floor((seq_len - kernel_size) / kernel_stride) + 1 (0 when
 * the sequence is shorter than a window; fsa_preview/module/fsa_decode.py:87-91), and this GPU's rows of them: compressed
 * tokens [cmp_lo, cmp_hi) are stored from row cmp_row0[b] on.  rng_lo / rng_hi [B, Hk, 1]. */
int fsa_decode_cmp_ranges(const int32_t* seq_len, const int32_t* cmp_row0, int batch, int num_kv_heads, int kernel_size,
                          int kernel_stride, int cmp_lo, int cmp_hi, int32_t* num_cmp, int32_t* rng_lo, int32_t* rng_hi,
                          void* stream);

/* Cache-row ranges of the selected blocks (ranges 0..topk-1, from topk_idx [B, Hk, topk]) and of the sliding window
 * [max(0, t - window), t] cut into num_window_pieces pieces of `piece` rows (ranges topk..), for t = seq_len[b] - 1,
 * clipped to the tokens [shard_lo, shard_hi) this GPU stores; token tok of sequence b is cache row
 * seq_row0[b] + tok - shard_lo.  Output rng_lo / rng_hi [B, Hk, topk + num_window_pieces] feed fsa_decode_attn_partial.
 * Host-side arithmetic of the reference: fsa_preview/module/fsa_decode.py:160-185. */
int fsa_decode_ranges(const int32_t* topk_idx, const int32_t* seq_len, const int32_t* seq_row0, int batch, int num_kv_heads,
                      int topk, int block_size, int window, int piece, int num_window_pieces, int shard_lo, int shard_hi,
                      int32_t* rng_lo, int32_t* rng_hi, void* stream);

/* Copy the device status word of an index workspace to the host (synchronises `stream`).  No reference counterpart
 * (the reference's kernels have no bounded waits to report).  index_ws = NULL reads the status word of the built-in
 * array that fsa_sel_fwd_static works in (on the current device; nothing is allocated).
 * *status_out: 0 ok, 1 a bounded wait ran out, 2 an out-of-table index was skipped.
 * Returns FSA_ERR_DEVICE_STATUS when the word is non-zero. */
int fsa_read_status(const void* index_ws, void* stream, int* status_out);

/* Debug/inspection: launch one thread that waits on a barrier nothing will ever signal.  Like every wait of the library
 * it gives up after its bound (0.2 s), records status 1 in the int at status_ws (a zeroed device word, e.g. the start of
 * an index workspace) and returns: fsa_read_status(status_ws, ...) then reports FSA_ERR_DEVICE_STATUS.  Exists so that the
 * failure path of the status plumbing can be tested without hanging or faulting a GPU.  No reference counterpart. */
int fsa_debug_wait_timeout(void* status_ws, void* stream);

/* Debug/inspection: geometry of the index workspace for a problem: the upper bound on tiles the workspace is sized
 * for, the entries per tile tpt = (128 / group) & ~3, and nbmax = total_tokens / block_size + batch + 1, the bound on
 * global block ids.  No reference counterpart (host arithmetic only). */
int fsa_sel_index_geometry(int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads, int topk, int block_size,
                           int64_t* max_tiles_out, int* tpt_out, int* nbmax_out);

/* Debug/inspection: copy the "(kv head, block) -> entries" tile list built by the forward to host arrays (what the
 * reference keeps as valid_lens / valid_start_indices / the flat token list,
 * fsa/ops/FSA_topk_sparse_attention.py:60-135).  Sizes from fsa_sel_index_geometry:
 *   tile_rec_host [4 * max_tiles]: per tile {first K/V row of its block, entries | kv head << 8, key = kv head * nbmax +
 *   global block id, first dK/dV segment of the key};
 *   entries_host [max_tiles * tpt]: entry e of tile j at j * tpt + e, (token << 6) | slot, 0xFFFFFFFF padding;
 *   key_tile_host [Hk * nbmax + 1]: first tile of every key;
 *   header_host [64]: [0] status, [1] tiles, [2] entries, [3] segments.  Any pointer may be NULL. */
int fsa_sel_index_dump(const void* index_ws, int64_t total_tokens, int batch, int num_q_heads, int num_kv_heads,
                       int topk, int block_size, void* stream, int32_t* tile_rec_host, uint32_t* entries_host,
                       int32_t* key_tile_host, int32_t* header_host);

#ifdef __cplusplus
}
#endif
#endif /* FSA_SM100_H_ */
