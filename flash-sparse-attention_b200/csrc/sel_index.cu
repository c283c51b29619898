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
                                                      SelBounds bd, SelShape s, SelIndex ix) {
    int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)s.Hk * s.N;
    bool active = gid < total;
    const bool small = total <= 0x7fffffffll;
    int h = active ? (small ? (int)((unsigned)gid / (unsigned)s.N) : (int)(gid / s.N)) : 0;
    int n = active ? (int)(gid - (int64_t)h * s.N) : 0;
    const int* row = topk_idx + ((int64_t)h * s.N + n) * s.T;
    unsigned lane = threadIdx.x & 31;
    unsigned lt = (1u << lane) - 1;
    TokenCtx tc{0, 0, 0, 0, -1};
    if (active) tc = token_ctx(cu, bd, s.B, s.BK, n);
    const bool list = bd.kv_hi == nullptr;
    for (int sl = 0; sl < s.T; ++sl) {
        int r0 = 0;
        int gb = active ? entry_block_ctx(tc, bd, s.BK, n, sl, list ? __ldg(row + sl) : 0, &r0) : -1;
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
                const int ps = ix.tile_off[key] * s.TPT + base + rank;
                ix.entries[ps] = ((uint32_t)n << kSlotBits) | (uint32_t)sl;
                ix.pos[((int64_t)h * s.N + n) * s.T + sl] = ps;
            }
        } else if (FILL && active) {
            ix.pos[((int64_t)h * s.N + n) * s.T + sl] = -1;
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
        if (i < HG) ix.tile_off[i] = pb + sb - b;
        __syncthreads();
        if (tid == 1023) { carry_a = pa + sa; carry_b = pb + sb; }
        __syncthreads();
    }
    if (tid == 0) {
        ix.tile_off[HG] = carry_b;
        ix.header[1] = carry_b;
        ix.header[2] = carry_a;
    }
}

// Tile records and the padding of the tile-ordered entry list: one warp per hg.
__global__ void __launch_bounds__(256) sel_index_tiles(SelShape s, SelIndex ix) {
    const int lane = threadIdx.x & 31;
    const int hg = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (hg >= s.Hk * s.NBmax) return;
    const int cnt = ix.counts[hg];
    if (cnt == 0) return;
    const int t0 = ix.tile_off[hg], nt = ix.tile_off[hg + 1] - t0;
    const int h = hg / s.NBmax;
    const int row0 = ix.row0[hg - h * s.NBmax];
    for (int t = lane; t < nt; t += 32) ix.tile_rec[t0 + t] = make_int4(h, row0, min(s.TPT, cnt - t * s.TPT), hg);
    // unused slots of the last tile
    const int used = cnt - (nt - 1) * s.TPT;
    for (int e = used + lane; e < s.TPT; e += 32) ix.entries[(int64_t)(t0 + nt - 1) * s.TPT + e] = 0xFFFFFFFFu;
}

cudaError_t sel_build_index(const int* topk_idx, const int* cu, const SelBounds& bd, const SelShape& s, const SelIndex& ix,
                            void* ws, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(ws, 0, sel_index_zero_bytes(s), stream);
    if (e != cudaSuccess) return e;
    int64_t total = (int64_t)s.Hk * s.N;
    if (total == 0) return cudaSuccess;
    unsigned grid = (unsigned)((total + 255) / 256);
    sel_index_pass<false><<<grid, 256, 0, stream>>>(topk_idx, cu, bd, s, ix);
    sel_index_scan<<<1, 1024, 0, stream>>>(s, ix);
    sel_index_tiles<<<(unsigned)((s.Hk * s.NBmax + 7) / 8), 256, 0, stream>>>(s, ix);
    sel_index_pass<true><<<grid, 256, 0, stream>>>(topk_idx, cu, bd, s, ix);
    return cudaGetLastError();
}

}  // namespace fsa
