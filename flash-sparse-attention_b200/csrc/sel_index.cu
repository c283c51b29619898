// Index inversion for selected attention: from topk_idx[Hk, N, T] (token -> KV blocks) build the CSR
// "KV block -> (token, slot) entries", cut into the tiles the persistent kernels walk, and the inverse map `pos`.
// Replaces the reference's block_to_token / index_mapping kernels, its bincount + boolean-mask compaction
// (fsa/ops/FSA_topk_sparse_attention.py:60-135, 622-668, 951-1020) and, for the backward, reorder_topk_idx
// (nsa_ref/ops/topk_sparse_attention.py:412-476): one structure serves forward and backward, its size is O(N*Hk*T),
// and no step syncs with the host.
//
// The build is a counting sort without global atomics, so the same input always gives the same list (the backward's
// dK / dV sums depend on the order of the entries):
//   1. count   one CTA per (kv head, chunk of C tokens): its warps take contiguous token ranges of the chunk and count
//              the entries per block into private shared-memory histograms; the chunk's totals go to chunk_cnt;
//   2. keys    one thread per (kv head, block): exclusive prefix of chunk_cnt over the chunks (every chunk's first
//              position inside the key) and the key's total;
//   3. scan    one CTA: first tile and first segment of every key;
//   4. tiles   one warp per key: tile records, padding of the last tile;
//   5. fill    the CTAs of step 1 again: the same counting pass gives every warp its first position inside each key,
//              a second pass over the same tokens writes entries and positions.
// Entries of a key are in ascending order of (chunk, warp range, 32-token group, slot): ascending token groups.
#include "sel_launch.cuh"

namespace fsa {

constexpr int kIdxMaxWarps = 8;     // (8 warps x 512-token chunks keep four CTAs resident per SM: the kernels are latency-bound)
constexpr int kIdxMaxSlots = 16;   // top-k lists up to this length are held in registers

// Count (FILL = false: hw[gb] += entries) or place (FILL = true: hw[gb] is this warp's next position in the
// tile-ordered entry list) the entries of this warp's share of the chunk [n0, n1).
template <bool FILL>
__device__ __forceinline__ void chunk_pass(const int* __restrict__ topk_idx, const int* __restrict__ cu, const SelBounds& bd,
                                           const SelShape& s, const SelIndex& ix, int h, int c, int n0, int n1, int* hw, int warp,
                                           int nwarps, int lane) {
    const int ngroups = (n1 - n0 + 31) >> 5;
    const int gpw = (ngroups + nwarps - 1) / nwarps;
    const int g_lo = warp * gpw, g_hi = min(ngroups, g_lo + gpw);
    const bool list = bd.kv_hi == nullptr;
    const bool in_regs = list && s.T <= kIdxMaxSlots && (s.T & 3) == 0 && (reinterpret_cast<uintptr_t>(topk_idx) & 15) == 0;
    const unsigned lt = (1u << lane) - 1;
    for (int g = g_lo; g < g_hi; ++g) {
        const int n = n0 + g * 32 + lane;
        const bool active = n < n1;
        TokenCtx tc{0, 0, 0, 0, -1, 0};
        if (active) tc = token_ctx(cu, bd, s.B, s.BK, n);
        const int* row = topk_idx + ((int64_t)h * s.N + n) * s.T;
        int ids[kIdxMaxSlots];
        if (in_regs && active) {
            // the whole list in one round trip (rows are 16-byte aligned: T is a multiple of 4)
#pragma unroll
            for (int i = 0; i < kIdxMaxSlots / 4; ++i) {
                if (i * 4 < s.T) {
                    const int4 v = __ldg(reinterpret_cast<const int4*>(row) + i);
                    ids[i * 4] = v.x; ids[i * 4 + 1] = v.y; ids[i * 4 + 2] = v.z; ids[i * 4 + 3] = v.w;
                }
            }
        }
#pragma unroll 1
        for (int sl0 = 0; sl0 < s.T; sl0 += kIdxMaxSlots) {
#pragma unroll
            for (int j = 0; j < kIdxMaxSlots; ++j) {
                const int sl = sl0 + j;
                if (sl >= s.T) break;
                int r0 = 0;
                const int id = !active ? -1 : in_regs ? ids[j] : list ? __ldg(row + sl) : 0;
                int gb = active ? entry_block_ctx(tc, bd, s.BK, n, sl, id, &r0) : -1;
                if (gb >= s.NBmax) {   // only a malformed range can do this: skip the entry, record it
                    atomicMax(ix.header, (int)kStatusBadIndex);
                    gb = -1;
                }
                __syncwarp();
                const unsigned m = __match_any_sync(0xffffffffu, gb);
                const int leader = __ffs(m) - 1;
                if (!FILL) {
                    if (gb >= 0 && lane == leader) {
                        hw[gb] += __popc(m);
                    }
                } else {
                    int base = 0;
                    if (gb >= 0 && lane == leader) {
                        base = hw[gb];
                        hw[gb] = base + __popc(m);
                    }
                    base = __shfl_sync(m, base, leader);
                    if (active) {
                        int ps = -1;
                        if (gb >= 0) {
                            ps = base + __popc(m & lt);
                            ix.entries[ps] = ((uint32_t)n << kSlotBits) | (uint32_t)sl;
                        }
                        if (in_regs) ids[j] = ps;      // the slot's id is used up: keep its position, written as whole rows below
                        else ix.pos[((int64_t)h * s.N + n) * s.T + sl] = ps;
                    }
                }
                __syncwarp();
            }
        }
        if (FILL && in_regs && active) {
            int4* prow = reinterpret_cast<int4*>(ix.pos + ((int64_t)h * s.N + n) * s.T);
#pragma unroll
            for (int i = 0; i < kIdxMaxSlots / 4; ++i)
                if (i * 4 < s.T) prow[i] = make_int4(ids[i * 4], ids[i * 4 + 1], ids[i * 4 + 2], ids[i * 4 + 3]);
        }
    }
}

// Step 1 (FILL = false) and step 5 (FILL = true).
template <bool FILL>
__global__ void __launch_bounds__(kIdxMaxWarps * 32) sel_index_chunk(const int* __restrict__ topk_idx, const int* __restrict__ cu,
                                                                     SelBounds bd, SelShape s, SelIndex ix) {
    extern __shared__ int sm[];   // [nwarps][NBmax]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthreads = blockDim.x, nwarps = nthreads >> 5;
    const int c = blockIdx.x, h = blockIdx.y;
    const int n0 = (int)min((int64_t)c * s.C, s.N), n1 = (int)min((int64_t)(c + 1) * s.C, s.N);
    int* cc = ix.chunk_cnt + ((int64_t)h * s.NC + c) * s.NBmax;
    int* wo = ix.warp_off + ((int64_t)h * s.NC + c) * nwarps * s.NBmax;
    if (!FILL) {
        for (int i = tid; i < nwarps * s.NBmax; i += nthreads) sm[i] = 0;
        __syncthreads();
        chunk_pass<false>(topk_idx, cu, bd, s, ix, h, c, n0, n1, sm + warp * s.NBmax, warp, nwarps, lane);
        __syncthreads();
        for (int gb = tid; gb < s.NBmax; gb += nthreads) {
            int run = 0;
            for (int i = 0; i < nwarps; ++i) {
                const int v = sm[i * s.NBmax + gb];
                wo[i * s.NBmax + gb] = run;        // this warp's first position inside the key, relative to the chunk
                run += v;
            }
            cc[gb] = run;
        }
    } else {
        // every warp's first position in the tile-ordered entry list: first entry of the key (step 3) + the chunk's first
        // position inside the key (step 2) + the warp's inside the chunk (step 1)
        const int* kt = ix.key_tile + (int64_t)h * s.NBmax;
        for (int gb = tid; gb < s.NBmax; gb += nthreads) {
            const int base = kt[gb] * s.TPT + cc[gb];
            for (int i = 0; i < nwarps; ++i) sm[i * s.NBmax + gb] = base + wo[i * s.NBmax + gb];
        }
        __syncthreads();
        chunk_pass<true>(topk_idx, cu, bd, s, ix, h, c, n0, n1, sm + warp * s.NBmax, warp, nwarps, lane);
    }
}

// Step 2: per key, exclusive prefix of the chunks' counts and the total (thread per key; eight loads in flight).
__global__ void __launch_bounds__(64) sel_index_keys(SelShape s, SelIndex ix) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= s.Hk * s.NBmax) return;
    const int h = k / s.NBmax, gb = k - h * s.NBmax;
    int* p = ix.chunk_cnt + (int64_t)h * s.NC * s.NBmax + gb;
    int run = 0;
    for (int c0 = 0; c0 < s.NC; c0 += 8) {
        int v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = c0 + j < s.NC ? p[(int64_t)(c0 + j) * s.NBmax] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (c0 + j < s.NC) p[(int64_t)(c0 + j) * s.NBmax] = run;
            run += v[j];
        }
    }
    ix.key_cnt[k] = run;
}

// Step 3: exclusive scans over the keys (a single CTA): first tile, then -- it depends on the first tile -- first segment.
// A key with tiles [t0, t0 + nt) is cut by the backward's schedule at every multiple of RB.
__global__ void __launch_bounds__(1024) sel_index_scan(SelShape s, SelIndex ix) {
    __shared__ int wsum_a[32], wsum_b[32], wsum_c[32];
    __shared__ int carry_a, carry_b, carry_c;
    const int HG = s.Hk * s.NBmax;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { carry_a = 0; carry_b = 0; carry_c = 0; }
    __syncthreads();
    for (int base = 0; base < HG; base += 1024) {
        const int i = base + tid;
        const int a = i < HG ? ix.key_cnt[i] : 0;
        const int b = (a + s.TPT - 1) / s.TPT;
        int sa = a, sb = b;
        for (int o = 1; o < 32; o <<= 1) {
            const int ta = __shfl_up_sync(0xffffffffu, sa, o), tb = __shfl_up_sync(0xffffffffu, sb, o);
            if (lane >= o) { sa += ta; sb += tb; }
        }
        if (lane == 31) { wsum_a[warp] = sa; wsum_b[warp] = sb; }
        __syncthreads();
        if (warp == 0) {
            int va = wsum_a[lane], vb = wsum_b[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const int ta = __shfl_up_sync(0xffffffffu, va, o), tb = __shfl_up_sync(0xffffffffu, vb, o);
                if (lane >= o) { va += ta; vb += tb; }
            }
            wsum_a[lane] = va; wsum_b[lane] = vb;
        }
        __syncthreads();
        const int pa = carry_a + (warp ? wsum_a[warp - 1] : 0);
        const int t0 = carry_b + (warp ? wsum_b[warp - 1] : 0) + sb - b;     // first tile of this key
        if (i < HG) ix.key_tile[i] = t0;
        const int cseg = b > 0 ? (t0 + b - 1) / s.RB - t0 / s.RB + 1 : 0;
        int sc = cseg;
        for (int o = 1; o < 32; o <<= 1) {
            const int tc = __shfl_up_sync(0xffffffffu, sc, o);
            if (lane >= o) sc += tc;
        }
        if (lane == 31) wsum_c[warp] = sc;
        __syncthreads();
        if (warp == 0) {
            int vc = wsum_c[lane];
            for (int o = 1; o < 32; o <<= 1) {
                const int tc = __shfl_up_sync(0xffffffffu, vc, o);
                if (lane >= o) vc += tc;
            }
            wsum_c[lane] = vc;
        }
        __syncthreads();
        const int pc = carry_c + (warp ? wsum_c[warp - 1] : 0);
        if (i < HG) ix.key_seg[i] = pc + sc - cseg;
        __syncthreads();
        if (tid == 1023) { carry_a = pa + sa; carry_b = t0 + b; carry_c = pc + sc; }
        __syncthreads();
    }
    if (tid == 0) {
        ix.key_tile[HG] = carry_b;
        ix.key_seg[HG] = carry_c;
        ix.header[1] = carry_b;
        ix.header[2] = carry_a;
        ix.header[3] = carry_c;
    }
}

// Step 4: tile records and the padding of the tile-ordered entry list: one warp per key.  The block's first K/V row
// and its row count follow from the block id: gb = cu_k[b] / BK + b + j for block j of sequence b.
__global__ void __launch_bounds__(256) sel_index_tiles(const int* __restrict__ cu, SelBounds bd, SelShape s, SelIndex ix) {
    const int lane = threadIdx.x & 31;
    const int hg = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (hg >= s.Hk * s.NBmax) return;
    const int cnt = ix.key_cnt[hg];
    if (cnt == 0) return;
    const int t0 = ix.key_tile[hg], nt = (cnt + s.TPT - 1) / s.TPT;
    const int h = hg / s.NBmax, gb = hg - h * s.NBmax;
    const int* ck = bd.cu_k ? bd.cu_k : cu;
    int lo = 0, hi = s.B;   // largest b with cu_k[b] / BK + b <= gb
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(ck + mid) / s.BK + mid <= gb) lo = mid; else hi = mid;
    }
    const int k0 = __ldg(ck + lo), k1 = __ldg(ck + lo + 1);
    const int row0 = k0 + (gb - (k0 / s.BK + lo)) * s.BK;
    if (lane == 0) {
        ix.row0[gb] = row0;                     // (the same values from every kv head)
        ix.nrow[gb] = min(s.BK, k1 - row0);
    }
    const int seg0 = ix.key_seg[hg];
    for (int t = lane; t < nt; t += 32) {
        ix.tile_rec[t0 + t] = make_int4(row0, min(s.TPT, cnt - t * s.TPT) | (h << 8), hg, seg0);
        ix.tile_aux[t0 + t] = make_int2(t0, nt);
    }
    // unused slots of the last tile
    const int used = cnt - (nt - 1) * s.TPT;
    for (int e = used + lane; e < s.TPT; e += 32) ix.entries[(int64_t)(t0 + nt - 1) * s.TPT + e] = 0xFFFFFFFFu;
}

// warps per CTA of the chunk kernels so that the per-warp histograms fit in shared memory; 0: the problem does not fit
int sel_index_warps(const SelShape& s) {
    const int64_t ints = (200 * 1024) / 4;
    int64_t nw = ints / (s.NBmax > 0 ? s.NBmax : 1);
    if (nw < 1) return 0;
    if (nw > kIdxMaxWarps) nw = kIdxMaxWarps;
    const int64_t groups = (s.C + 31) / 32;    // no more warps than 32-token groups in a chunk
    if (nw > groups) nw = groups;
    return (int)nw;
}

cudaError_t sel_build_index(const int* topk_idx, const int* cu, const SelBounds& bd, const SelShape& s, const SelIndex& ix,
                            void* ws, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(ws, 0, sel_index_zero_bytes(s), stream);
    if (e != cudaSuccess) return e;
    if ((int64_t)s.Hk * s.N == 0) return cudaSuccess;
    const int nw = s.IW;
    if (nw == 0) return cudaErrorInvalidValue;
    const int smem = nw * s.NBmax * 4;
    e = cudaFuncSetAttribute(sel_index_chunk<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(sel_index_chunk<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    const dim3 grid((unsigned)s.NC, (unsigned)s.Hk);
    const int HG = s.Hk * s.NBmax;
    sel_index_chunk<false><<<grid, nw * 32, smem, stream>>>(topk_idx, cu, bd, s, ix);
    sel_index_keys<<<(unsigned)((HG + 63) / 64), 64, 0, stream>>>(s, ix);
    sel_index_scan<<<1, 1024, 0, stream>>>(s, ix);
    sel_index_tiles<<<(unsigned)((HG + 7) / 8), 256, 0, stream>>>(cu, bd, s, ix);
    sel_index_chunk<true><<<grid, nw * 32, smem, stream>>>(topk_idx, cu, bd, s, ix);
    return cudaGetLastError();
}

}  // namespace fsa
