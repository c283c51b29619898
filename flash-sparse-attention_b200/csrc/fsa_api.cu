// extern "C" entry points of libfsa_sm100.so (declared in include/fsa_sm100.h): argument
// checks, workspace carving, TMA tensor-map encoding and kernel dispatch.  No torch types,
// no allocation, no synchronisation on the compute paths.
#include "../../include/fsa_sm100.h"
#include "sel_common.cuh"
#include "sel_launch.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace fsa {

static thread_local int g_last_cuda_error = 0;
static thread_local int g_last_cuda_line = 0;

static int cuda_fail_at(cudaError_t e, int line) {
    g_last_cuda_error = (int)e;
    g_last_cuda_line = line;
    return FSA_ERR_CUDA;
}
#define cuda_fail(e) cuda_fail_at((e), __LINE__)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess) fn = (EncodeTiledFn)p;
    });
    return fn;
}

// 2-D map over a [rows, cols] 16-bit matrix with row stride `row_stride` elements; box = 64 x box_rows,
// 128-byte swizzle.  Rows past the end read as zero.
int make_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t rows, int64_t cols, int64_t row_stride,
                  int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return cuda_fail(cudaErrorNotSupported);
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)(rows > 0 ? rows : 1)};
    cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1, 1};
    CUresult r = fn(map, dtype == FSA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail_at(cudaErrorInvalidValue, -(int)r - 100000);   // driver error code, negated
    return FSA_OK;
}

// 3-D map over 16-bit elements: dims {d0 (contiguous), d1, d2}, strides of d1 and d2 in ELEMENTS (multiples of 8; they may
// overlap), box {64, box1, 1}, 128-byte swizzle.  Coordinates past a dimension read as zero.
int make_tile_map_3d(CUtensorMap* map, const void* base, int dtype, int64_t d0, int64_t d1, int64_t d2, int64_t stride1,
                     int64_t stride2, int box1) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return cuda_fail(cudaErrorNotSupported);
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)(d1 > 0 ? d1 : 1), (cuuint64_t)(d2 > 0 ? d2 : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)stride1 * 2, (cuuint64_t)stride2 * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box1, 1};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = fn(map, dtype == FSA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail_at(cudaErrorInvalidValue, -(int)r - 100000);   // driver error code, negated
    return FSA_OK;
}

// The same with a box of box2 entries along the third dimension (box {64, box1, box2}).
int make_tile_map_3d_box(CUtensorMap* map, const void* base, int dtype, int64_t d0, int64_t d1, int64_t d2, int64_t stride1,
                         int64_t stride2, int box1, int box2) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return cuda_fail(cudaErrorNotSupported);
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)(d1 > 0 ? d1 : 1), (cuuint64_t)(d2 > 0 ? d2 : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)stride1 * 2, (cuuint64_t)stride2 * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box1, (cuuint32_t)box2};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = fn(map, dtype == FSA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail_at(cudaErrorInvalidValue, -(int)r - 100000);   // driver error code, negated
    return FSA_OK;
}

int device_sm_count(int* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    static int cache[64];
    if (dev >= 0 && dev < 64 && cache[dev] > 0) { *out = cache[dev]; return FSA_OK; }
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev >= 0 && dev < 64) cache[dev] = n;
    *out = n;
    return FSA_OK;
}

// ---- optional kernel timing: a ring of event pairs per kernel id
constexpr int kProfKernels = 16;
constexpr int kProfRing = 64;
static bool g_prof_on = false;
static cudaEvent_t g_prof_ev[kProfKernels][kProfRing][2];
static bool g_prof_made[kProfKernels];
static int g_prof_count[kProfKernels];

void prof_begin(int id, cudaStream_t stream) {
    if (!g_prof_on || id < 0 || id >= kProfKernels) return;
    if (!g_prof_made[id]) {
        for (int i = 0; i < kProfRing; ++i)
            if (cudaEventCreate(&g_prof_ev[id][i][0]) != cudaSuccess || cudaEventCreate(&g_prof_ev[id][i][1]) != cudaSuccess) return;
        g_prof_made[id] = true;
    }
    cudaEventRecord(g_prof_ev[id][g_prof_count[id] % kProfRing][0], stream);
}
void prof_end(int id, cudaStream_t stream) {
    if (!g_prof_on || id < 0 || id >= kProfKernels || !g_prof_made[id]) return;
    cudaEventRecord(g_prof_ev[id][g_prof_count[id] % kProfRing][1], stream);
    ++g_prof_count[id];
}

// Tensor-map encoding is a driver call and needs the primary context bound to the calling
// thread; a thread that has only ever been handed device pointers (an autograd worker) may not
// have one yet.  cudaSetDevice on the current device binds it.
int ensure_context() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaSetDevice(dev);
    if (e != cudaSuccess) return cuda_fail(e);
    return FSA_OK;
}

// Tuning knobs read from the environment (0 / unset = built-in default).
static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

static int make_shape(int64_t N, int B, int Hq, int Hk, int D, int T, int BK, SelShape* s, int64_t Nk = -1) {
    if (Nk < 0) Nk = N;
    if (N < 0 || B < 0 || Hq <= 0 || Hk <= 0 || T <= 0 || BK <= 0) return FSA_ERR_BAD_ARG;
    if (Hq % Hk != 0) return FSA_ERR_BAD_ARG;
    int G = Hq / Hk;
    if (G > 32) return FSA_ERR_UNSUPPORTED;   // a tile needs >= 4 tokens per head row group
    if (T > kMaxTopk || N >= kMaxTokens || Nk >= kMaxTokens) return FSA_ERR_UNSUPPORTED;
    if (!(BK == 32 || BK == 64 || BK == 128 || BK == 256)) return FSA_ERR_UNSUPPORTED;
    if (D != 0 && !(D == 64 || D == 128 || D == 256)) return FSA_ERR_UNSUPPORTED;
    s->N = N; s->Nk = Nk; s->B = B; s->Hq = Hq; s->Hk = Hk; s->G = G; s->D = D; s->T = T; s->BK = BK;
    s->NBmax = (int)(Nk / BK) + B + 1;
    s->TPT = (kTileRows / G) & ~3;
    // chunk of the index build: at least 512 tokens, at most 512 chunks
    int64_t C = 512;
    while (C * 512 < N) C *= 2;
    s->C = (int)C;
    s->NC = (int)((N + C - 1) / C);
    if (s->NC < 1) s->NC = 1;
    // tiles per scheduling run of the backward (FSA_SEL_RUN overrides; read once)
    static const int env_run = env_int("FSA_SEL_RUN", 0);
    s->RB = env_run > 0 ? env_run : 32;
    if ((int64_t)s->Hk * s->NBmax >= ((int64_t)1 << 30)) return FSA_ERR_UNSUPPORTED;
    if ((int64_t)s->Hk * s->NBmax * s->NC >= ((int64_t)1 << 31)) return FSA_ERR_UNSUPPORTED;
    if (Hk > 65535) return FSA_ERR_UNSUPPORTED;
    s->IW = sel_index_warps(*s);
    if (s->IW == 0) return FSA_ERR_UNSUPPORTED;                                           // a sequence of millions of blocks
    if ((int64_t)s->Hk * s->NBmax * s->NC * s->IW >= ((int64_t)1 << 31)) return FSA_ERR_UNSUPPORTED;
    if (sel_max_tiles(*s) * kTileRows >= ((int64_t)1 << 31)) return FSA_ERR_UNSUPPORTED;  // partial rows are 32-bit
    return FSA_OK;
}

static int bwd_nsub(int BK) { return BK > 64 ? BK / 64 : 1; }
static int64_t bwd_dq_part_bytes(const SelShape& s) {
    return align_up(sel_max_tiles(s) * bwd_nsub(s.BK) * kTileRows * (int64_t)s.D * 2, 1024);
}
// fp32 dK / dV accumulators (unpipelined kernel) or per-segment slabs (pipelined kernel): the same region
static int64_t bwd_dkdv_bytes(const SelShape& s) {
    const int64_t acc = align_up(2 * s.Nk * s.Hk * (int64_t)s.D * 4, 256);
    const int64_t slabs = align_up(sel_max_segments(s) * 2 * 64 * (int64_t)s.D * 4, 256);
    return acc > slabs ? acc : slabs;
}
static int64_t bwd_scratch_bytes(const SelShape& s) {
    return align_up(s.N * s.Hq * 4, 1024) + bwd_dq_part_bytes(s) + bwd_dkdv_bytes(s);
}

static int64_t fwd_scratch_bytes(const SelShape& s) {
    int64_t rows = sel_max_tiles(s) * kTileRows;
    return align_up(rows * s.D * 2, 1024) + align_up(rows * 8, 256);
}

}  // namespace fsa

using namespace fsa;

extern "C" {

int fsa_version(void) { return 100; }

const char* fsa_error_string(int code) {
    switch (code) {
        case FSA_OK: return "ok";
        case FSA_ERR_BAD_ARG: return "bad argument (null/misaligned pointer, bad size or stride)";
        case FSA_ERR_UNSUPPORTED: return "shape not supported by the compiled sm_100a kernels";
        case FSA_ERR_WORKSPACE: return "workspace too small";
        case FSA_ERR_CUDA: return "CUDA call failed";
        case FSA_ERR_DEVICE_STATUS: return "a kernel recorded a device-side failure";
        case FSA_ERR_STATIC_LIMIT: return "problem needs more scratch than the library's built-in static buffer holds";
        default: return "unknown error";
    }
}

int fsa_last_cuda_error(void) { return g_last_cuda_error; }
int fsa_last_cuda_error_line(void) { return g_last_cuda_line; }

int fsa_profile_enable(int on) {
    g_prof_on = on != 0;
    for (int i = 0; i < kProfKernels; ++i) g_prof_count[i] = 0;
    return FSA_OK;
}

int fsa_profile_read(int kernel_id, float* ms_sum_out, int* launches_out) {
    if (!ms_sum_out || !launches_out || kernel_id < 0 || kernel_id >= kProfKernels) return FSA_ERR_BAD_ARG;
    *ms_sum_out = 0.f;
    *launches_out = 0;
    if (!g_prof_made[kernel_id]) return FSA_OK;
    int n = g_prof_count[kernel_id] < kProfRing ? g_prof_count[kernel_id] : kProfRing;
    for (int i = 0; i < n; ++i) {
        cudaError_t e = cudaEventSynchronize(g_prof_ev[kernel_id][i][1]);
        if (e != cudaSuccess) return cuda_fail(e);
        float ms = 0.f;
        e = cudaEventElapsedTime(&ms, g_prof_ev[kernel_id][i][0], g_prof_ev[kernel_id][i][1]);
        if (e != cudaSuccess) return cuda_fail(e);
        *ms_sum_out += ms;
    }
    *launches_out = n;
    return FSA_OK;
}

int fsa_sel_index_bytes(int64_t N, int B, int Hq, int Hk, int T, int BK, int64_t* bytes_out) {
    if (!bytes_out) return FSA_ERR_BAD_ARG;
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, 0, T, BK, &s);
    if (rc) return rc;
    *bytes_out = sel_index_bytes(s);
    return FSA_OK;
}

int fsa_sel_fwd_scratch_bytes(int64_t N, int B, int Hq, int Hk, int D, int T, int BK, int64_t* bytes_out) {
    if (!bytes_out) return FSA_ERR_BAD_ARG;
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, D, T, BK, &s);
    if (rc) return rc;
    *bytes_out = fwd_scratch_bytes(s);
    return FSA_OK;
}

}  // extern "C"

static int sel_fwd_impl(const SelBounds& bd, int64_t Nk, const void* q, const void* k, const void* v, const int32_t* topk_idx,
                        const int32_t* cu_seqlens, int64_t N, int B, int Hq, int Hk, int D, int T, int BK, int dtype, int64_t q_sn, int64_t q_sh,
                int64_t k_sn, int64_t v_sn, float sm_scale, void* o, int64_t o_sn, int64_t o_sh, float* lse,
                void* index_ws, int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    (void)cudaGetLastError();   // drop any stale error another library left on this thread
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, D, T, BK, &s, Nk);
    if (rc) return rc;
    if ((rc = ensure_context()) != FSA_OK) return rc;
    if (D == 0) return FSA_ERR_BAD_ARG;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (!(sm_scale > 0.f)) return FSA_ERR_BAD_ARG;
    if (N == 0) return FSA_OK;
    if (!q || !k || !v || (!topk_idx && !bd.kv_hi) || !cu_seqlens || !o || !lse || !index_ws || !scratch) return FSA_ERR_BAD_ARG;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(scratch) || !aligned16(index_ws))
        return FSA_ERR_BAD_ARG;
    if ((q_sn % 8) || (q_sh % 8) || (k_sn % 8) || (v_sn % 8) || (o_sn % 8) || (o_sh % 8)) return FSA_ERR_BAD_ARG;
    if (k_sn < (int64_t)Hk * D || v_sn < (int64_t)Hk * D) return FSA_ERR_BAD_ARG;
    if (BK == 256 && D == 256) return FSA_ERR_UNSUPPORTED;
    if (index_ws_bytes < sel_index_bytes(s)) return FSA_ERR_WORKSPACE;
    if (scratch_bytes < fwd_scratch_bytes(s)) return FSA_ERR_WORKSPACE;

    SelIndex ix = sel_index_carve(index_ws, s);
    prof_begin(FSA_KERNEL_SEL_INDEX, stream);
    cudaError_t e = sel_build_index(topk_idx, cu_seqlens, bd, s, ix, index_ws, stream);
    prof_end(FSA_KERNEL_SEL_INDEX, stream);
    if (e != cudaSuccess) return cuda_fail(e);

    CUtensorMap kmap, vmap, omap;
    rc = make_tile_map(&kmap, k, dtype, Nk, (int64_t)Hk * D, k_sn, BK);
    if (rc) return rc;
    rc = make_tile_map(&vmap, v, dtype, Nk, (int64_t)Hk * D, v_sn, BK);
    if (rc) return rc;
    const int64_t prow = sel_max_tiles(s) * kTileRows;
    SelFwdArgs a;
    a.q = q; a.q_sn = q_sn; a.q_sh = q_sh; a.sm_scale = sm_scale;
    static const int env_run = env_int("FSA_SEL_RUN", 0);
    a.run = env_run;
    a.opart = scratch;
    a.ml = (float2*)((char*)scratch + align_up(prow * D * 2, 1024));
    a.o = o; a.o_sn = o_sn; a.o_sh = o_sh; a.lse = lse;
    a.kmap = &kmap; a.vmap = &vmap; a.qmap = nullptr; a.omap = nullptr;
    a.bd = bd;
    if (D <= 128 && BK <= 128) {
        rc = make_tile_map(&omap, scratch, dtype, prow, D, D, 32);
        if (rc) return rc;
        a.omap = &omap;
    }
    int sms = 0;
    rc = device_sm_count(&sms);
    if (rc) return rc;
    e = dispatch_sel_fwd(dtype, a, s, ix, sms, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    return FSA_OK;
}


extern "C" {

int fsa_sel_fwd(const void* q, const void* k, const void* v, const int32_t* topk_idx, const int32_t* cu_seqlens,
                int64_t N, int B, int Hq, int Hk, int D, int T, int BK, int dtype, int64_t q_sn, int64_t q_sh,
                int64_t k_sn, int64_t v_sn, float sm_scale, void* o, int64_t o_sn, int64_t o_sh, float* lse,
                void* index_ws, int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream_) {
    if (!topk_idx) return FSA_ERR_BAD_ARG;
    return sel_fwd_impl(SelBounds{nullptr, nullptr, nullptr}, N, q, k, v, topk_idx, cu_seqlens, N, B, Hq, Hk, D, T, BK, dtype, q_sn,
                        q_sh, k_sn, v_sn, sm_scale, o, o_sn, o_sh, lse, index_ws, index_ws_bytes, scratch, scratch_bytes, stream_);
}

int fsa_range_attn_fwd(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                       const int32_t* kv_lo, const int32_t* kv_hi, int64_t N, int64_t Nk, int B, int Hq, int Hk, int D,
                       int max_blocks, int BK, int dtype, int64_t q_sn, int64_t q_sh, int64_t k_sn, int64_t v_sn,
                       float sm_scale, void* o, int64_t o_sn, int64_t o_sh, float* lse, void* index_ws,
                       int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream_) {
    if (!kv_hi || !cu_seqlens_k) return FSA_ERR_BAD_ARG;
    return sel_fwd_impl(SelBounds{cu_seqlens_k, kv_lo, kv_hi}, Nk, q, k, v, nullptr, cu_seqlens_q, N, B, Hq, Hk, D, max_blocks, BK,
                        dtype, q_sn, q_sh, k_sn, v_sn, sm_scale, o, o_sn, o_sh, lse, index_ws, index_ws_bytes, scratch,
                        scratch_bytes, stream_);
}

int fsa_sel_bwd_scratch_bytes(int64_t N, int B, int Hq, int Hk, int D, int T, int BK, int64_t* bytes_out) {
    if (!bytes_out) return FSA_ERR_BAD_ARG;
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, D, T, BK, &s);
    if (rc) return rc;
    *bytes_out = bwd_scratch_bytes(s);
    return FSA_OK;
}

}  // extern "C"

static int sel_bwd_impl(const SelBounds& bd, int64_t Nk, const void* q, const void* k, const void* v, const void* o, const float* lse,
                        const void* d_o, const int32_t* topk_idx, const int32_t* cu_seqlens, int64_t N, int B, int Hq, int Hk, int D, int T,
                int BK, int dtype, int64_t q_sn, int64_t q_sh, int64_t k_sn, int64_t v_sn, int64_t o_sn, int64_t o_sh,
                int64_t do_sn, int64_t do_sh, float sm_scale, void* dq, void* dk, void* dv, void* index_ws,
                int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    (void)cudaGetLastError();   // drop any stale error another library left on this thread
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, D, T, BK, &s, Nk);
    if (rc) return rc;
    if ((rc = ensure_context()) != FSA_OK) return rc;
    if (D == 0) return FSA_ERR_BAD_ARG;
    if (dtype != FSA_DTYPE_BF16 && dtype != FSA_DTYPE_FP16) return FSA_ERR_BAD_ARG;
    if (!(sm_scale > 0.f)) return FSA_ERR_BAD_ARG;
    if (N == 0) return FSA_OK;
    if (!q || !k || !v || !o || !lse || !d_o || !cu_seqlens || !dq || !dk || !dv || !index_ws || !scratch)
        return FSA_ERR_BAD_ARG;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o) || !aligned16(dq) ||
        !aligned16(dk) || !aligned16(dv) || !aligned16(scratch) || !aligned16(index_ws))
        return FSA_ERR_BAD_ARG;
    if ((q_sn % 8) || (q_sh % 8) || (k_sn % 8) || (v_sn % 8) || (o_sn % 8) || (o_sh % 8) || (do_sn % 8) || (do_sh % 8))
        return FSA_ERR_BAD_ARG;
    if (k_sn < (int64_t)Hk * D || v_sn < (int64_t)Hk * D) return FSA_ERR_BAD_ARG;
    if (index_ws_bytes < sel_index_bytes(s)) return FSA_ERR_WORKSPACE;
    if (scratch_bytes < bwd_scratch_bytes(s)) return FSA_ERR_WORKSPACE;

    SelIndex ix = sel_index_carve(index_ws, s);
    CUtensorMap kmap, vmap;
    rc = make_tile_map(&kmap, k, dtype, Nk, (int64_t)Hk * D, k_sn, 64);
    if (rc) return rc;
    rc = make_tile_map(&vmap, v, dtype, Nk, (int64_t)Hk * D, v_sn, 64);
    if (rc) return rc;
    int sms = 0;
    rc = device_sm_count(&sms);
    if (rc) return rc;

    SelBwdArgs a;
    a.q = q; a.d_o = d_o; a.o = o;
    a.q_sn = q_sn; a.q_sh = q_sh; a.do_sn = do_sn; a.do_sh = do_sh; a.o_sn = o_sn; a.o_sh = o_sh;
    a.lse = lse; a.topk_idx = topk_idx; a.cu = cu_seqlens; a.sm_scale = sm_scale;
    a.run = s.RB;
    char* sp = (char*)scratch;
    a.delta = (float*)sp;   sp += align_up(N * Hq * 4, 1024);
    a.dq_part = (void*)sp;  sp += bwd_dq_part_bytes(s);
    CUtensorMap dqmap;
    a.dqmap = nullptr;
    if (D == 128 && BK <= 64) {
        rc = make_tile_map(&dqmap, a.dq_part, dtype, sel_max_tiles(s) * kTileRows, D, D, 32);
        if (rc) return rc;
        a.dqmap = &dqmap;
    }
    a.dk_acc = (float*)sp;
    a.dv_acc = a.dk_acc + Nk * Hk * (int64_t)D;
    a.slabs = (float*)sp;
    a.bd = bd;
    a.dq = dq; a.dk = dk; a.dv = dv;
    cudaError_t e = dispatch_sel_bwd(dtype, a, s, ix, kmap, vmap, sms, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    return FSA_OK;
}


extern "C" {

int fsa_sel_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                const int32_t* topk_idx, const int32_t* cu_seqlens, int64_t N, int B, int Hq, int Hk, int D, int T,
                int BK, int dtype, int64_t q_sn, int64_t q_sh, int64_t k_sn, int64_t v_sn, int64_t o_sn, int64_t o_sh,
                int64_t do_sn, int64_t do_sh, float sm_scale, void* dq, void* dk, void* dv, void* index_ws,
                int64_t index_ws_bytes, void* scratch, int64_t scratch_bytes, void* stream_) {
    return sel_bwd_impl(SelBounds{nullptr, nullptr, nullptr}, N, q, k, v, o, lse, d_o, topk_idx, cu_seqlens, N, B, Hq, Hk, D, T, BK,
                        dtype, q_sn, q_sh, k_sn, v_sn, o_sn, o_sh, do_sn, do_sh, sm_scale, dq, dk, dv, index_ws, index_ws_bytes,
                        scratch, scratch_bytes, stream_);
}

int fsa_range_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                       const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* kv_lo, const int32_t* kv_hi,
                       int64_t N, int64_t Nk, int B, int Hq, int Hk, int D, int max_blocks, int BK, int dtype, int64_t q_sn,
                       int64_t q_sh, int64_t k_sn, int64_t v_sn, int64_t o_sn, int64_t o_sh, int64_t do_sn, int64_t do_sh,
                       float sm_scale, void* dq, void* dk, void* dv, void* index_ws, int64_t index_ws_bytes, void* scratch,
                       int64_t scratch_bytes, void* stream_) {
    if (!kv_hi || !cu_seqlens_k) return FSA_ERR_BAD_ARG;
    return sel_bwd_impl(SelBounds{cu_seqlens_k, kv_lo, kv_hi}, Nk, q, k, v, o, lse, d_o, nullptr, cu_seqlens_q, N, B, Hq, Hk, D,
                        max_blocks, BK, dtype, q_sn, q_sh, k_sn, v_sn, o_sn, o_sh, do_sn, do_sh, sm_scale, dq, dk, dv, index_ws,
                        index_ws_bytes, scratch, scratch_bytes, stream_);
}

int fsa_range_attn_index(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* kv_lo, const int32_t* kv_hi,
                         int64_t N, int64_t Nk, int B, int Hq, int Hk, int max_blocks, int BK, void* index_ws,
                         int64_t index_ws_bytes, void* stream_) {
    if (!kv_hi || !cu_seqlens_k || !cu_seqlens_q) return FSA_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    (void)cudaGetLastError();
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, 0, max_blocks, BK, &s, Nk);
    if (rc) return rc;
    if (N == 0) return FSA_OK;
    if (!index_ws || !aligned16(index_ws)) return FSA_ERR_BAD_ARG;
    if (index_ws_bytes < sel_index_bytes(s)) return FSA_ERR_WORKSPACE;
    SelIndex ix = sel_index_carve(index_ws, s);
    prof_begin(FSA_KERNEL_SEL_INDEX, stream);
    cudaError_t e = sel_build_index(nullptr, cu_seqlens_q, SelBounds{cu_seqlens_k, kv_lo, kv_hi}, s, ix, index_ws, stream);
    prof_end(FSA_KERNEL_SEL_INDEX, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    return FSA_OK;
}

int fsa_range_attn_bytes(int64_t N, int64_t Nk, int B, int Hq, int Hk, int D, int max_blocks, int BK, int64_t* index_bytes_out,
                         int64_t* fwd_scratch_bytes_out, int64_t* bwd_scratch_bytes_out) {
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, D, max_blocks, BK, &s, Nk);
    if (rc) return rc;
    if (index_bytes_out) *index_bytes_out = sel_index_bytes(s);
    if (fwd_scratch_bytes_out) *fwd_scratch_bytes_out = fwd_scratch_bytes(s);
    if (bwd_scratch_bytes_out) *bwd_scratch_bytes_out = bwd_scratch_bytes(s);
    return FSA_OK;
}

static int sel_static_base(void** out);

int fsa_read_status(const void* index_ws, void* stream_, int* status_out) {
    if (!status_out) return FSA_ERR_BAD_ARG;
    if (!index_ws) {
        // the status word of fsa_sel_fwd_static lives at the start of the library's built-in array
        void* base = nullptr;
        int rc = sel_static_base(&base);
        if (rc) return rc;
        index_ws = base;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    int st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, index_ws, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return cuda_fail(e);
    *status_out = st;
    return st == 0 ? FSA_OK : FSA_ERR_DEVICE_STATUS;
}

int fsa_sel_index_geometry(int64_t N, int B, int Hq, int Hk, int T, int BK, int64_t* max_tiles_out, int* tpt_out,
                           int* nbmax_out) {
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, 0, T, BK, &s);
    if (rc) return rc;
    if (max_tiles_out) *max_tiles_out = sel_max_tiles(s);
    if (tpt_out) *tpt_out = s.TPT;
    if (nbmax_out) *nbmax_out = s.NBmax;
    return FSA_OK;
}

int fsa_sel_index_dump(const void* index_ws, int64_t N, int B, int Hq, int Hk, int T, int BK, void* stream_,
                       int32_t* tile_rec_host, uint32_t* entries_host, int32_t* key_tile_host, int32_t* header_host) {
    cudaStream_t stream = (cudaStream_t)stream_;
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, 0, T, BK, &s);
    if (rc) return rc;
    if (!index_ws) return FSA_ERR_BAD_ARG;
    SelIndex ix = sel_index_carve(const_cast<void*>(index_ws), s);
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return cuda_fail(e);
    const int64_t mt = sel_max_tiles(s), HG = (int64_t)s.Hk * s.NBmax;
    if (tile_rec_host && (e = cudaMemcpy(tile_rec_host, ix.tile_rec, mt * 16, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail(e);
    if (entries_host && (e = cudaMemcpy(entries_host, ix.entries, mt * s.TPT * 4, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail(e);
    if (key_tile_host && (e = cudaMemcpy(key_tile_host, ix.key_tile, (HG + 1) * 4, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail(e);
    if (header_host && (e = cudaMemcpy(header_host, ix.header, 64 * 4, cudaMemcpyDeviceToHost)) != cudaSuccess) return cuda_fail(e);
    return FSA_OK;
}

// A bounded wait that runs out, on purpose and harmlessly: one thread waits on an mbarrier that nothing arrives on, gives
// up after FSA_WAIT_NS like every wait of the library does, records kStatusWaitTimeout in the status word and returns.
// Lets a test walk the failure path of the status plumbing without hanging or faulting anything.
static __global__ void wait_timeout_probe_kernel(int* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
        if (mbar_wait(&bar, 0, status)) atomicMax(status, 99);   // cannot happen: nobody arrives
    }
}

int fsa_debug_wait_timeout(void* status_ws, void* stream_) {
    if (!status_ws || ((uintptr_t)status_ws & 3)) return FSA_ERR_BAD_ARG;
    (void)cudaGetLastError();
    wait_timeout_probe_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>((int*)status_ws);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FSA_OK : cuda_fail(e);
}

// ---------------------------------------------------------------------------------------------
// Forward without any caller-provided workspace.
//
// Some host programs may not allocate device memory once they are running: they handed the whole
// GPU to their own arena at start-up, or they cannot afford the device-wide synchronisation and
// the late out-of-memory failure that an allocation can bring in the middle of serving.  For them
// the index workspace and the partial-result scratch of the forward live in this fixed array,
// which every GPU that loads the library carries until the process exits.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_sel_static_scratch[FSA_SEL_STATIC_SCRATCH_BYTES];

// Device address of the array on each device (index = CUDA device ordinal).  In host code the
// array's name is only a handle for the runtime, never a pointer a kernel may use.
static void* g_sel_static_ptr[64];
static std::mutex g_sel_static_mutex;

static int sel_static_base(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 64) return FSA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_sel_static_mutex);
    if (!g_sel_static_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_sel_static_scratch);   // address on the current device
        if (e != cudaSuccess) return cuda_fail(e);
        if (!p || ((uintptr_t)p & 255)) return FSA_ERR_BAD_ARG;
        g_sel_static_ptr[dev] = p;
    }
    *out = g_sel_static_ptr[dev];
    return FSA_OK;
}

int fsa_sel_fwd_static(const void* q, const void* k, const void* v, const int32_t* topk_idx, const int32_t* cu_seqlens,
                       int64_t N, int B, int Hq, int Hk, int D, int T, int BK, int dtype, int64_t q_sn, int64_t q_sh,
                       int64_t k_sn, int64_t v_sn, float sm_scale, void* o, int64_t o_sn, int64_t o_sh, float* lse,
                       void* stream_) {
    SelShape s;
    int rc = make_shape(N, B, Hq, Hk, D, T, BK, &s);
    if (rc) return rc;
    if (D == 0) return FSA_ERR_BAD_ARG;
    // layout inside the static array: [index workspace | forward scratch]; the array is 256-byte aligned and the
    // index workspace is rounded up to 1 KiB, so both regions start 256-byte aligned (all the kernels need)
    const int64_t index_bytes = align_up(sel_index_bytes(s), 1024);
    const int64_t scratch_bytes = fwd_scratch_bytes(s);
    if (index_bytes + scratch_bytes > (int64_t)FSA_SEL_STATIC_SCRATCH_BYTES) return FSA_ERR_STATIC_LIMIT;
    void* base = nullptr;
    rc = sel_static_base(&base);
    if (rc) return rc;
    // The array keeps the previous call's contents.  Everything that must start from zero (status word,
    // per-block counters and cursors) is cleared by the index build on `stream`; every other word is
    // written before it is read.
    return fsa_sel_fwd(q, k, v, topk_idx, cu_seqlens, N, B, Hq, Hk, D, T, BK, dtype, q_sn, q_sh, k_sn, v_sn, sm_scale, o, o_sn,
                       o_sh, lse, base, index_bytes, (char*)base + index_bytes, scratch_bytes, stream_);
}

}  // extern "C"
