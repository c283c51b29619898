// Shared definitions of the selected-attention kernels: problem description, the index
// workspace that inverts "token -> selected KV blocks" into "KV block -> selecting tokens",
// and the partial-result buffers.
//
// Vocabulary
//   entry      one (token, slot) pair: token n selected a KV block in slot s of its top-k list
//   gb         global KV-block id.  For sequence b starting at row c_b, local block j:
//                  gb = c_b / BK + b + j      (unique, ascending, < N/BK + B + 1)
//   hg         kv_head * NBmax + gb, the key of the block->entries CSR
//   tile       up to TPT = 128 / G consecutive entries of one hg; each entry contributes its G
//              query heads, so a tile is <= 128 rows of the MMA
#pragma once
#include <stdint.h>
#include "sm100_prims.cuh"

namespace fsa {

constexpr int kTileRows = 128;
constexpr int kSlotBits = 6;               // entries are packed as (token << 6) | slot
constexpr int kMaxTopk = 1 << kSlotBits;   // 64
constexpr int64_t kMaxTokens = (int64_t)1 << (31 - kSlotBits);

enum DType : int { kBF16 = 0, kFP16 = 1 };

struct SelShape {
    int64_t N;       // total packed tokens
    int B;           // sequences
    int Hq, Hk, G;   // heads, G = Hq / Hk
    int D;           // head dim
    int T;           // top-k slots
    int BK;          // KV block size
    int NBmax;       // bound on gb: N / BK + B + 1
    int TPT;         // entries per tile = 128 / G
};

// Index workspace (kept by the caller between forward and backward).  All int32.
struct SelIndex {
    int* header;     // [64]: [0] status, [1] total tiles
    int* counts;     // [Hk * NBmax]   entries per hg
    int* cursor;     // [Hk * NBmax]   fill cursors (scratch)
    int* row0;       // [NBmax]        first global K/V row of block gb
    int* blk_off;    // [Hk * NBmax + 1] exclusive scan of counts
    int* tile_off;   // [Hk * NBmax + 1] exclusive scan of ceil(counts / TPT)
    uint32_t* entries;  // [Hk * N * T]  packed entries grouped by hg
};

__host__ __device__ inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

inline int64_t sel_index_bytes(const SelShape& s) {
    int64_t HG = (int64_t)s.Hk * s.NBmax;
    int64_t b = 0;
    b += align_up(64 * 4, 256);
    b += align_up(HG * 4, 256) * 2;
    b += align_up((int64_t)s.NBmax * 4, 256);
    b += align_up((HG + 1) * 4, 256) * 2;
    b += align_up((int64_t)s.Hk * s.N * s.T * 4, 256);
    return b;
}

inline SelIndex sel_index_carve(void* ws, const SelShape& s) {
    int64_t HG = (int64_t)s.Hk * s.NBmax;
    char* p = (char*)ws;
    SelIndex ix;
    ix.header = (int*)p;   p += align_up(64 * 4, 256);
    ix.counts = (int*)p;   p += align_up(HG * 4, 256);
    ix.cursor = (int*)p;   p += align_up(HG * 4, 256);
    ix.row0 = (int*)p;     p += align_up((int64_t)s.NBmax * 4, 256);
    ix.blk_off = (int*)p;  p += align_up((HG + 1) * 4, 256);
    ix.tile_off = (int*)p; p += align_up((HG + 1) * 4, 256);
    ix.entries = (uint32_t*)p;
    return ix;
}
// bytes from the start of the workspace that must be zero before the index build
inline int64_t sel_index_zero_bytes(const SelShape& s) {
    int64_t HG = (int64_t)s.Hk * s.NBmax;
    return align_up(64 * 4, 256) + align_up(HG * 4, 256) * 2;
}

// sequence of token n: largest b with cu[b] <= n
__device__ __forceinline__ int find_seq(const int* __restrict__ cu, int B, int n) {
    int lo = 0, hi = B;   // invariant: cu[lo] <= n < cu[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (__ldg(cu + mid) <= n) lo = mid; else hi = mid;
    }
    return lo;
}

// A slot is usable when 0 <= id <= t_local / BK (nsa_ref/ops/topk_sparse_attention.py:116-119).
__device__ __forceinline__ int entry_block(const int* __restrict__ cu, int B, int BK, int n, int id, int* row0_out) {
    int b = find_seq(cu, B, n);
    int c = __ldg(cu + b);
    int t_local = n - c;
    if (id < 0 || id > t_local / BK) return -1;
    *row0_out = c + id * BK;
    return c / BK + b + id;
}

// largest i in [0, n) with off[i] <= x  (off ascending, off[0] = 0)
__device__ __forceinline__ int upper_seg(const int* __restrict__ off, int n, int x) {
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (off[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

}  // namespace fsa
