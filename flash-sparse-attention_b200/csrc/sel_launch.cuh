// Host-side launch interfaces of the selected-attention kernels (defined in sel_index.cu,
// sel_fwd.cu, sel_bwd.cu; called from fsa_api.cu).
#pragma once
#include "sel_common.cuh"

namespace fsa {

// Optional per-kernel timing (off by default): library-owned CUDA events bracket a kernel on
// the stream it is launched on.  Ids are the FSA_KERNEL_* constants of the public header.
void prof_begin(int kernel_id, cudaStream_t stream);
void prof_end(int kernel_id, cudaStream_t stream);

// warps per CTA of the index kernels (their per-warp histograms must fit in shared memory); 0: too many blocks
int sel_index_warps(const SelShape& s);

cudaError_t sel_build_index(const int* topk_idx, const int* cu, const SelBounds& bd, const SelShape& s, const SelIndex& ix,
                            void* ws, cudaStream_t stream);

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

struct SelFwdArgs {
    const void* q;            // used by the unpipelined kernel (arbitrary strides)
    int64_t q_sn, q_sh;
    float sm_scale;
    int run;                  // tiles per scheduling run; 0 = default
    void* opart;              // [max_tiles * 128, D] input dtype
    float2* ml;               // [Hq, N, T] statistics (capacity max_tiles * 128 pairs)
    void* o;
    int64_t o_sn, o_sh;
    float* lse;
    const CUtensorMap* qmap;  // [N, Hq*D] box {64,1} for gather4; null when q's head stride != D
    const CUtensorMap* kmap;  // [N, Hk*D] box {64, BK}
    const CUtensorMap* vmap;
    const CUtensorMap* omap;  // [max_tiles * 128, D] box {64, 32} for the partial stores
    SelBounds bd;             // visible K/V rows per token (all null: causal rule of selected attention)
};

cudaError_t dispatch_sel_fwd(int dtype, const SelFwdArgs& a, const SelShape& s, const SelIndex& ix, int num_sms,
                             cudaStream_t stream);

struct SelBwdArgs {
    const void *q, *d_o, *o;
    int64_t q_sn, q_sh, do_sn, do_sh, o_sn, o_sh;
    const float* lse;
    const int* topk_idx;
    const int* cu;
    float sm_scale;
    int run;           // tiles per scheduling run; 0 = default
    // scratch
    float* delta;      // [Hq, N]
    void* dq_part;     // [max_tiles * nsub * 128, D] input dtype
    const CUtensorMap* dqmap;   // over dq_part, box {64, 32}: partial stores of the pipelined kernel (null: not built)
    float* dk_acc;     // [N, Hk, D]; dv_acc follows immediately (unpipelined kernel: fp32 accumulators)
    float* dv_acc;
    float* slabs;      // [segments][2][64][D] fp32 (pipelined kernel: per-segment partial dK / dV); shares memory with dk_acc
    // outputs (contiguous)
    void *dq, *dk, *dv;
    SelBounds bd;      // visible K/V rows per token (all null: causal rule of selected attention)
};

// pipelined main kernel for head_dim 128, block size <= 64 (sel_bwd_pipe.cu)
cudaError_t launch_sel_bwd_pipe(int dtype, const SelBwdArgs& a, const SelShape& s, const SelIndex& ix,
                                const CUtensorMap& kmap, const CUtensorMap& vmap, const CUtensorMap& dqmap, int num_sms,
                                bool no_dq, cudaStream_t stream);

// dQ of a range-attention backward as one query-tile-major kernel (range_dense.cu; head_dim 128): the accumulator stays
// in TMEM across the K/V tiles a tile of tokens sees, so the block-major kernel above runs with no_dq
cudaError_t launch_range_bwd_dq(int dtype, const SelBwdArgs& a, const SelShape& s, const CUtensorMap& kmap, const CUtensorMap& vmap,
                                int* status, cudaStream_t stream);

cudaError_t dispatch_sel_bwd(int dtype, const SelBwdArgs& a, const SelShape& s, const SelIndex& ix,
                             const CUtensorMap& kmap, const CUtensorMap& vmap, int num_sms, cudaStream_t stream);

}  // namespace fsa
