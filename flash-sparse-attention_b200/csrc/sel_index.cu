// Index inversion for selected attention: from topk_idx[Hk, N, T] (token -> KV blocks) build
// the CSR "KV block -> (token, slot) entries" and the per-block tile offsets the persistent
// kernels walk.  Replaces the reference's block_to_token / index_mapping kernels, its
// bincount + boolean-mask compaction (fsa/ops/FSA_topk_sparse_attention.py:60-135, 622-668,
// 951-1020) and, for the backward, reorder_topk_idx (nsa_ref/ops/topk_sparse_attention.py:412-476):
// one structure serves forward and backward, its size is O(N*Hk*T), and no step syncs with the host.
#include "sel_launch.cuh"

namespace fsa {

template <bool FILL>
__global__ void __launch_bounds__(256) sel_index_pass(const int* __restrict__ topk_idx, const int* __restrict__ cu,
                                                      SelShape s, SelIndex ix) {
    int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)s.Hk * s.N;
    bool active = gid < total;
    int h = active ? (int)(gid / s.N) : 0;
    int n = active ? (int)(gid % s.N) : 0;
    const int* row = topk_idx + ((int64_t)h * s.N + n) * s.T;
    unsigned lane = threadIdx.x & 31;
    unsigned lt = (1u << lane) - 1;
    for (int sl = 0; sl < s.T; ++sl) {
        int id = active ? __ldg(row + sl) : -1;
        int r0 = 0;
        int gb = active ? entry_block(cu, s.B, s.BK, n, id, &r0) : -1;
        int key = gb < 0 ? -1 : h * s.NBmax + gb;
        unsigned m = __match_any_sync(0xffffffffu, key);
        if (key >= 0) {
            int leader = __ffs(m) - 1;
            int cnt = __popc(m);
            if (!FILL) {
                if ((int)lane == leader) {
                    atomicAdd(ix.counts + key, cnt);
                    ix.row0[gb] = r0;
                }
            } else {
                int base = 0;
                if ((int)lane == leader) base = atomicAdd(ix.cursor + key, cnt);
                base = __shfl_sync(m, base, leader);
                int rank = __popc(m & lt);
                ix.entries[(int64_t)ix.blk_off[key] + base + rank] = ((uint32_t)n << kSlotBits) | (uint32_t)sl;
            }
        }
    }
}

// Single-CTA exclusive scans of counts and of ceil(counts / TPT).
__global__ void __launch_bounds__(1024) sel_index_scan(SelShape s, SelIndex ix) {
    __shared__ int wsum_a[32], wsum_b[32];
    __shared__ int carry_a, carry_b;
    int HG = s.Hk * s.NBmax;
    int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { carry_a = 0; carry_b = 0; }
    __syncthreads();
    for (int base = 0; base < HG; base += 1024) {
        int i = base + tid;
        int a = i < HG ? ix.counts[i] : 0;
        int b = (a + s.TPT - 1) / s.TPT;
        int sa = a, sb = b;
        for (int o = 1; o < 32; o <<= 1) {
            int ta = __shfl_up_sync(0xffffffffu, sa, o);
            int tb = __shfl_up_sync(0xffffffffu, sb, o);
            if (lane >= o) { sa += ta; sb += tb; }
        }
        if (lane == 31) { wsum_a[warp] = sa; wsum_b[warp] = sb; }
        __syncthreads();
        if (warp == 0) {
            int va = wsum_a[lane], vb = wsum_b[lane];
            for (int o = 1; o < 32; o <<= 1) {
                int ta = __shfl_up_sync(0xffffffffu, va, o);
                int tb = __shfl_up_sync(0xffffffffu, vb, o);
                if (lane >= o) { va += ta; vb += tb; }
            }
            wsum_a[lane] = va; wsum_b[lane] = vb;
        }
        __syncthreads();
        int pa = carry_a + (warp ? wsum_a[warp - 1] : 0);
        int pb = carry_b + (warp ? wsum_b[warp - 1] : 0);
        if (i < HG) {
            ix.blk_off[i] = pa + sa - a;
            ix.tile_off[i] = pb + sb - b;
        }
        __syncthreads();
        if (tid == 1023) { carry_a = pa + sa; carry_b = pb + sb; }
        __syncthreads();
    }
    if (tid == 0) {
        ix.blk_off[HG] = carry_a;
        ix.tile_off[HG] = carry_b;
        ix.header[1] = carry_b;
        ix.header[2] = carry_a;
    }
}

cudaError_t sel_build_index(const int* topk_idx, const int* cu, const SelShape& s, const SelIndex& ix, void* ws,
                            cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(ws, 0, sel_index_zero_bytes(s), stream);
    if (e != cudaSuccess) return e;
    int64_t total = (int64_t)s.Hk * s.N;
    if (total == 0) return cudaSuccess;
    unsigned grid = (unsigned)((total + 255) / 256);
    sel_index_pass<false><<<grid, 256, 0, stream>>>(topk_idx, cu, s, ix);
    sel_index_scan<<<1, 1024, 0, stream>>>(s, ix);
    sel_index_pass<true><<<grid, 256, 0, stream>>>(topk_idx, cu, s, ix);
    return cudaGetLastError();
}

}  // namespace fsa
