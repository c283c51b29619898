// Shared definitions of the selected-attention kernels: problem description, the index
// workspace that inverts "token -> selected KV blocks" into "KV block -> selecting tokens",
// and the partial-result buffers.
//
// Vocabulary
//   entry      one (token, slot) pair: token n selected a KV block in slot s of its top-k list
//   gb         global KV-block id.  For sequence b starting at row c_b, local block j:
//                  gb = c_b / BK + b + j      (unique, ascending, < N/BK + B + 1)
//   key        hg = kv_head * NBmax + gb, the key of the block->entries CSR; the entries of a key are in ascending
//              order of their 32-token group (a deterministic order: no atomics decide it)
//   chunk      C consecutive query tokens: the unit of work of the index build (one CTA per (kv head, chunk))
//   tile       up to TPT = (128 / G) & ~3 consecutive entries of one key; each entry contributes its G
//              query heads, so a tile is <= 128 rows of the MMA.  Rows are head-major inside a tile:
//              row r = g * TPT + e (head g of the group, e-th entry of the tile), so that four
//              consecutive rows are four tokens of one head
//   segment    the tiles of one key that one CTA of the backward walks in a row (its static schedule deals runs of
//              RB consecutive tiles): every segment owns one slab of partial dK / dV sums
//   pos        for every (kv head, token, slot): first tile of the key * TPT + rank of the entry inside its
//              key, or -1 for an unusable slot.  Partial results live in tile order
//              (row = (pos / TPT) * 128 + g * TPT + pos % TPT), which the merge kernels look up here.
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
    int64_t N;       // total packed (query) tokens
    int64_t Nk;      // rows of K / V (= N for selected attention; compressed tokens for the compressed branch)
    int B;           // sequences
    int Hq, Hk, G;   // heads, G = Hq / Hk
    int D;           // head dim
    int T;           // top-k slots
    int BK;          // KV block size
    int NBmax;       // bound on gb: N / BK + B + 1
    int TPT;         // entries per tile = (128 / G) & ~3
    int C;           // query tokens per chunk of the index build
    int NC;          // chunks = ceil(N / C)
    int RB;          // tiles per scheduling run of the backward kernel (fixes the segments)
    int IW;          // warps per CTA of the index build
};

// Index workspace (kept by the caller between forward and backward).  All int32.
// Which K/V rows a token may attend.  Selected attention: kv_lo = kv_hi = null, the rule is the
// causal one (rows <= the token's own row) and the blocks come from topk_idx.  Range mode
// (compressed and sliding-window branches): every token attends the K/V rows [kv_lo[n], kv_hi[n]]
// (global row ids, empty when hi < lo) and "selects" every block that range touches.
struct SelBounds {
    const int* cu_k;     // [B+1] sequence starts in K/V rows (null: same as the query cu_seqlens)
    const int* kv_lo;    // [N] or null
    const int* kv_hi;    // [N] or null
};

struct SelIndex {
    int* header;     // [64]: [0] status, [1] total tiles, [2] total entries, [3] total segments
    int* chunk_cnt;  // [Hk * NC * NBmax]  entries of (kv head, chunk, block); then their exclusive prefix over the chunks
    int* warp_off;   // [Hk * NC * IW * NBmax]  first position, inside the chunk's share of the key, of every warp of the count kernel
    int* key_cnt;    // [Hk * NBmax]       entries per key
    int* key_tile;   // [Hk * NBmax + 1]   first tile of every key (exclusive scan of ceil(count / TPT))
    int* key_seg;    // [Hk * NBmax + 1]   first segment of every key
    int* row0;       // [NBmax]            first global K/V row of block gb
    int* nrow;       // [NBmax]            K/V rows of block gb (the last block of a sequence may be short)
    int4* tile_rec;  // [max_tiles]   per tile {first K/V row of the block, entries | kv head << 8, key, first segment of the key}
    int2* tile_aux;  // [max_tiles]   per tile {first tile of its key, tiles of its key}
    uint32_t* entries;  // [max_tiles * TPT]  packed entries in TILE ORDER: entry e of tile j at j * TPT + e,
                        //                    0xFFFFFFFF where a tile is not full
    int* pos;        // [Hk * N * T]  tile-order position of every (head, token, slot), -1 if unusable
};

__host__ __device__ inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// upper bound on the number of tiles (known on the host without a sync)
inline int64_t sel_max_tiles(const SelShape& s) {
    return ((int64_t)s.Hk * s.N * s.T + s.TPT - 1) / s.TPT + (int64_t)s.Hk * s.NBmax;
}
// upper bound on the number of segments: one per key plus one per scheduling run that cuts a key
inline int64_t sel_max_segments(const SelShape& s) {
    return (int64_t)s.Hk * s.NBmax + sel_max_tiles(s) / s.RB + 1;
}

inline int64_t sel_index_bytes(const SelShape& s) {
    const int64_t HG = (int64_t)s.Hk * s.NBmax;
    int64_t b = 0;
    b += align_up(64 * 4, 256);
    b += align_up(HG * s.NC * 4, 256);
    b += align_up(HG * s.NC * s.IW * 4, 256);
    b += align_up(HG * 4, 256);
    b += align_up((HG + 1) * 4, 256) * 2;
    b += align_up((int64_t)s.NBmax * 4, 256) * 2;
    b += align_up(sel_max_tiles(s) * 16, 256);
    b += align_up(sel_max_tiles(s) * 8, 256);
    b += align_up(sel_max_tiles(s) * s.TPT * 4, 256);
    b += align_up((int64_t)s.Hk * s.N * s.T * 4, 256);
    return b;
}

inline SelIndex sel_index_carve(void* ws, const SelShape& s) {
    const int64_t HG = (int64_t)s.Hk * s.NBmax;
    char* p = (char*)ws;
    SelIndex ix;
    ix.header = (int*)p;    p += align_up(64 * 4, 256);
    ix.chunk_cnt = (int*)p; p += align_up(HG * s.NC * 4, 256);
    ix.warp_off = (int*)p;  p += align_up(HG * s.NC * s.IW * 4, 256);
    ix.key_cnt = (int*)p;   p += align_up(HG * 4, 256);
    ix.key_tile = (int*)p;  p += align_up((HG + 1) * 4, 256);
    ix.key_seg = (int*)p;   p += align_up((HG + 1) * 4, 256);
    ix.row0 = (int*)p;      p += align_up((int64_t)s.NBmax * 4, 256);
    ix.nrow = (int*)p;      p += align_up((int64_t)s.NBmax * 4, 256);
    ix.tile_rec = (int4*)p; p += align_up(sel_max_tiles(s) * 16, 256);
    ix.tile_aux = (int2*)p; p += align_up(sel_max_tiles(s) * 8, 256);
    ix.entries = (uint32_t*)p; p += align_up(sel_max_tiles(s) * s.TPT * 4, 256);
    ix.pos = (int*)p;
    return ix;
}
// bytes from the start of the workspace that must be zero before the index build (the header: every other word is
// written before it is read)
inline int64_t sel_index_zero_bytes(const SelShape&) { return align_up(64 * 4, 256); }

// sequence of token n: largest b with cu[b] <= n
__device__ __forceinline__ int find_seq(const int* __restrict__ cu, int B, int n) {
    int lo = 0, hi = B;   // invariant: cu[lo] <= n < cu[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (__ldg(cu + mid) <= n) lo = mid; else hi = mid;
    }
    return lo;
}

// Block of slot `sl` of token n, or -1.  List mode: a slot is usable when 0 <= id <= t_local / BK
// (nsa_ref/ops/topk_sparse_attention.py:116-119).  Range mode: slot sl is the sl-th block touched by
// [kv_lo[n], kv_hi[n]].
__device__ __forceinline__ int entry_block(const int* __restrict__ cu, const SelBounds& bd, int B, int BK, int n, int sl,
                                           const int* __restrict__ idrow, int* row0_out) {
    const int b = find_seq(cu, B, n);
    const int c = __ldg(cu + b);
    const int ck = bd.cu_k ? __ldg(bd.cu_k + b) : c;
    int id;
    if (bd.kv_hi) {
        const int lo = bd.kv_lo ? __ldg(bd.kv_lo + n) : ck, hi = __ldg(bd.kv_hi + n);
        if (hi < lo) return -1;
        id = (lo - ck) / BK + sl;
        if (id > (hi - ck) / BK) return -1;
    } else {
        id = __ldg(idrow + sl);
        if (id < 0 || id > (n - c) / BK) return -1;
    }
    *row0_out = ck + id * BK;
    return ck / BK + b + id;
}

// The same, with everything that depends only on the token looked up once (one binary search per token instead of
// one per slot).
struct TokenCtx {
    int c, ck, kb, lo, hi;    // sequence start (q rows), K/V start, global id of block 0, visible range (range mode)
    int ke;                   // K/V end of the sequence
};
__device__ __forceinline__ TokenCtx token_ctx(const int* __restrict__ cu, const SelBounds& bd, int B, int BK, int n) {
    TokenCtx t;
    const int b = find_seq(cu, B, n);
    t.c = __ldg(cu + b);
    t.ck = bd.cu_k ? __ldg(bd.cu_k + b) : t.c;
    t.ke = bd.cu_k ? __ldg(bd.cu_k + b + 1) : __ldg(cu + b + 1);
    t.kb = t.ck / BK + b;
    t.lo = t.ck; t.hi = -1;
    if (bd.kv_hi) {
        t.hi = __ldg(bd.kv_hi + n);
        if (bd.kv_lo) t.lo = __ldg(bd.kv_lo + n);
    }
    return t;
}
__device__ __forceinline__ int entry_block_ctx(const TokenCtx& t, const SelBounds& bd, int BK, int n, int sl, int id_list,
                                               int* row0_out) {
    int id;
    if (bd.kv_hi) {
        if (t.hi < t.lo) return -1;
        id = (t.lo - t.ck) / BK + sl;
        if (id > (t.hi - t.ck) / BK) return -1;
    } else {
        id = id_list;
        if (id < 0 || id > (n - t.c) / BK) return -1;
    }
    *row0_out = t.ck + id * BK;
    return t.kb + id;
}

// Visible key columns [c_lo, c_hi) of a tile row whose block starts at K/V row `row0` and holds
// `klim` keys: list mode is causal (rows <= tok); range mode uses the per-token bounds.
__device__ __forceinline__ void visible_cols(const SelBounds& bd, int tok, int row0, int klim, int& c_lo, int& c_hi) {
    int lo = row0, hi = tok;
    if (bd.kv_hi) {
        hi = __ldg(bd.kv_hi + tok);
        if (bd.kv_lo) lo = __ldg(bd.kv_lo + tok);
    }
    c_lo = max(0, lo - row0);
    c_hi = min(klim, hi - row0 + 1);
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

// Static tile schedule of a persistent grid: runs of `run` consecutive tiles are dealt to the
// CTAs round-robin, so the whole grid advances through the tile list together (neighbouring
// blocks of one kv head: their query rows stay in L2) while a CTA still reuses a resident K/V
// block across the tiles of a run.
struct TileSchedule {
    int total, grid, cta, run, nloc;
    __device__ TileSchedule(int total_, int run_) : total(total_), grid((int)gridDim.x), cta((int)blockIdx.x), run(run_) {
        const int NR = (total + run - 1) / run;                    // runs in the list
        const int mine = cta < NR ? (NR - cta + grid - 1) / grid : 0;
        nloc = mine * run;
        if (mine > 0 && (NR - 1) % grid == cta) nloc -= NR * run - total;   // the last run may be short
    }
    __device__ __forceinline__ int tile(int k) const { return ((k / run) * grid + cta) * run + (k % run); }
};

// Query-tile-major kernels cut every sequence into tiles of TPT consecutive tokens.  Both helpers are warp-collective (every lane calls them and gets the same
// answer) and walk the sequences 32 at a time, so that a packed batch of thousands of short sequences costs B / 32 steps.
__device__ __forceinline__ int count_seq_tiles(const int32_t* __restrict__ cu_q, int B, int TPT, int lane) {
    int total = 0;
    for (int b0 = 0; b0 < B; b0 += 32) {
        const int b = b0 + lane;
        int nt = b < B ? (__ldg(cu_q + b + 1) - __ldg(cu_q + b) + TPT - 1) / TPT : 0;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) nt += __shfl_xor_sync(0xffffffffu, nt, d);
        total += nt;
    }
    return total;
}
// tile `want` of the list: its sequence (-1 if there is no such tile), first token and number of tokens
__device__ __forceinline__ void find_seq_tile(const int32_t* __restrict__ cu_q, int B, int TPT, int want, int lane, int& seq, int& tok0,
                                             int& ne) {
    seq = -1; tok0 = 0; ne = 0;
    if (want < 0) return;
    int acc = 0;
    for (int b0 = 0; b0 < B; b0 += 32) {
        const int b = b0 + lane;
        const int s0 = b < B ? __ldg(cu_q + b) : 0, L = b < B ? __ldg(cu_q + b + 1) - s0 : 0;
        const int nt = (L + TPT - 1) / TPT;
        int incl = nt;                                   // inclusive prefix over the 32 sequences
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        const unsigned hit = __ballot_sync(0xffffffffu, want < acc + incl);
        if (hit) {
            const int src = __ffs(hit) - 1;              // first sequence whose tiles reach past `want`
            const int first = acc + __shfl_sync(0xffffffffu, incl - nt, src);
            const int s_src = __shfl_sync(0xffffffffu, s0, src), L_src = __shfl_sync(0xffffffffu, L, src);
            seq = b0 + src;
            tok0 = s_src + (want - first) * TPT;
            ne = min(TPT, s_src + L_src - tok0);
            return;
        }
        acc += __shfl_sync(0xffffffffu, incl, 31);
    }
}

// One tile of the list, read from its record: no searching, and the address depends only on the
// tile index, so records and entries can be prefetched any number of tiles ahead.
struct TileInfo {
    int h, row0, ne, hg, seg0;   // kv head, first K/V row of the block, entries, key, first segment of the key
};
__device__ __forceinline__ TileInfo load_tile(const SelIndex& ix, int tile) {
    int4 r = __ldg(ix.tile_rec + tile);
    return TileInfo{r.y >> 8, r.x, r.y & 255, r.z, r.w};
}

// Sequential walker used by the unpipelined kernels.
struct TileWalker {
    const SelIndex& ix;
    const SelShape& s;
    int hg = -1;
    int h = 0, row0 = 0, ne = 0;
    int64_t ebase = 0;
    __device__ TileWalker(const SelIndex& ix_, const SelShape& s_) : ix(ix_), s(s_) {}
    // returns true when the tile belongs to a different block than the previous one
    __device__ __forceinline__ bool seek(int item) {
        TileInfo t = load_tile(ix, item);
        bool nb = t.hg != hg;
        hg = t.hg; h = t.h; row0 = t.row0; ne = t.ne;
        ebase = (int64_t)item * s.TPT;
        return nb;
    }
};

// One lane's share of a partial row: V = D / 32 elements (4, 8 or 16 bytes), as raw words.
template <int V, typename ET>
__device__ __forceinline__ uint4 ld_row_vec(const ET* src) {
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (V == 2) u.x = *reinterpret_cast<const uint32_t*>(src);
    else if constexpr (V == 4) { uint2 t = *reinterpret_cast<const uint2*>(src); u.x = t.x; u.y = t.y; }
    else u = *reinterpret_cast<const uint4*>(src);
    return u;
}
template <int V, typename ET>
__device__ __forceinline__ void fma_row_vec(float (&acc)[V], const uint4& u, float w) {
    const uint32_t* uu = &u.x;
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
        float2 x = ElemTraits<ET>::unpack2(uu[i]);
        acc[2 * i] = fmaf(w, x.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(w, x.y, acc[2 * i + 1]);
    }
}

}  // namespace fsa
