// The C ABI of the library (declared in include/prism_b200.h): argument checks, tensor-map construction, kernel
// selection and launches.  One translation unit: the kernels are header-only templates included below.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "../../include/prism_b200.h"
#include "common.cuh"
#include "quant.cuh"
#include "quant_pipe.cuh"
#include "w8a8_gemm.cuh"
#include "w8a8_groups.cuh"
#include "w8a8_g32.cuh"
#include "w4a8_gemm.cuh"
#include "w4a8_few.cuh"
#include "w4a8_gemv.cuh"
#include "w8a8_gemv.cuh"
#include "mxfp4_gemm.cuh"
#include "mxfp4_gemv.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return PB_CUDA_ERROR;
}
#define PB_CUDA(call)                                 \
    do {                                              \
        cudaError_t e__ = (call);                     \
        if (e__ != cudaSuccess) return cuda_fail(e__); \
    } while (0)

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// ------------------------------------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// Programmatic dependent launch for the few-row chain (pb_set_pdl): while on, the small producers (rows_q8, swiglu_q8,
// fold) and the few-row tensor-core GEMMs are launched as programmatic dependents
// of the kernel before them on the stream; each begins with pdl_trigger and reads another kernel's output, or writes
// global memory, only after pdl_wait.  Off: plain launches (the two instructions are no-ops then).  The one-row
// CUDA-core GEMM stays a plain launch: as a programmatic dependent (first weights requested before the wait) the
// one-row pass measured 0.42 ms per four layers against 0.33.
std::atomic<int> g_pdl{0};

template <class... KA, class... A>
cudaError_t launch_dep(void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl.load(std::memory_order_relaxed) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<A>(args)...);
}

struct MapKey {
    const void* ptr;
    uint64_t inner, outer, stride;
    uint32_t box_inner, box_outer, kind;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && inner == o.inner && outer == o.outer && stride == o.stride && box_inner == o.box_inner &&
               box_outer == o.box_outer && kind == o.kind;
    }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        auto mix = [&](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
        mix(k.inner); mix(k.outer); mix(k.stride); mix(k.box_inner); mix(k.box_outer); mix(k.kind);
        return h;
    }
};

// A 2-D row-major matrix [outer, inner] of 1-byte (kind 0, 128-byte swizzle) or 4-byte (kind 1 fp32 / kind 3 uint32,
// no swizzle) elements,
// loaded in boxes of [box_outer, box_inner].  Maps are cached by (pointer, shape, box) and passed to kernels by value,
// so a captured CUDA graph keeps the maps of its capture.
int tensor_map(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t stride_bytes,
               uint32_t box_inner, uint32_t box_outer, uint32_t kind) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    MapKey key{ptr, inner, outer, stride_bytes, box_inner, box_outer, kind};
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return PB_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return PB_CUDA_ERROR;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    // kinds: 0 bytes with the 128-byte swizzle, 1 fp32, 3 32-bit words, 4 fp32 with the 128-byte swizzle
    const CUtensorMapDataType dt = kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : (kind == 1 || kind == 4) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    CUresult r = fn(out, dt, 2,
                    const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    (kind == 0 || kind == 4) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return PB_CUDA_ERROR;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return PB_OK;
}

// An int8 matrix [rows, K] (K a multiple of 128) as {128 bytes, rows, K / 128 chunks}: a box of {128, box_rows, 2} is
// 256 bytes of K for box_rows rows, laid down as two 128-byte-swizzled tiles one after the other.
int tensor_map_kchunks(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t K, uint32_t box_rows) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    MapKey key{ptr, K, rows, K, 128, box_rows, 100};
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return PB_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return PB_CUDA_ERROR;
    cuuint64_t dims[3] = {128, rows, K / 128};
    cuuint64_t strides[2] = {K, 128};
    cuuint32_t box[3] = {128, box_rows, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return PB_CUDA_ERROR;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return PB_OK;
}

// Per-device state.  One process may drive several GPUs (one context each): the SM count, a kernel's opt-in to more
// than 48 KB of dynamic shared memory (cudaFuncSetAttribute applies to the current device only) and the occupancy
// answers are therefore kept per device ordinal, looked up with the device current at the call.
constexpr int kMaxDevices = 64;

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return dev;
}

int sm_count() {
    static int n[kMaxDevices] = {};
    const int dev = current_device();
    if (!n[dev]) {
        int v = 0;
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        n[dev] = v > 0 ? v : 148;
    }
    return n[dev];
}

// Opt a kernel in to `bytes` of dynamic shared memory on the current device, once per (device, kernel).
int set_smem_raw(const void* fn, int bytes) {
    struct Key {
        const void* fn;
        int dev;
        bool operator==(const Key& o) const { return fn == o.fn && dev == o.dev; }
    };
    struct Hash {
        size_t operator()(const Key& k) const { return (size_t)k.fn * 31 + (size_t)k.dev; }
    };
    static std::mutex mu;
    static std::unordered_map<Key, int, Hash> done;
    const Key key{fn, current_device()};
    std::lock_guard<std::mutex> lock(mu);
    auto it = done.find(key);
    if (it != done.end() && it->second >= bytes) return PB_OK;
    PB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done[key] = bytes;
    return PB_OK;
}

template <typename Kernel>
int set_smem(Kernel k, int bytes) {
    return set_smem_raw((const void*)k, bytes);
}

// Failure injection from the host (pb_test_drop_loads): the many-rows W8A8 kernel's producers request no tiles.
int g_drop_loads = 0;

// ------------------------------------------------------------------------------------------------- W8A8 launches
// How the many-rows kernel adds into the fp32 residual.  PRISM_B200_ADD = regs: read, add, write through registers;
// tma (default, measured fastest): 32 x 32 boxes reduced by the copy engine; red: per-row-segment reductions at the
// memory side.
int add_mode() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_ADD");
        v = !e ? 1 : (e[0] == 'r' && e[2] == 'g') ? 0 : (e[0] == 't') ? 1 : 2;
    }
    return v;
}

// PRISM_B200_BN192=0: never use 128 x 192 tiles (comparison runs).
bool wide192_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_BN192");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// PRISM_B200_TAIL=0: never split the last wave of tiles (comparison runs).
bool tail_split_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_TAIL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

template <int BN, int EPI>
int launch_tile(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, void* out, long ldo,
                const int* n_rows, int M, int N, int K, cudaStream_t st, int split = 1, void* workspace = nullptr,
                int* counters = nullptr, const w8a8::RowBlocks* blocks = nullptr, float* souts = nullptr, int gbn = 0,
                long workspace_bytes = 0, int n_counters = 0) {
    using C = w8a8::TileCfg<BN>;
    CUtensorMap ta, tw;
    int rc;
    if ((rc = tensor_map(&ta, a, K, M, K, w8a8::BK, w8a8::BM, 0))) return rc;
    if ((rc = tensor_map(&tw, w, K, N, K, w8a8::BK, BN, 0))) return rc;
    auto kern = w8a8::w8a8_tile_kernel<BN, EPI>;
    constexpr int smem = EPI == w8a8::EPI_ADD ? C::SMEM_ADD : C::SMEM;
    static_assert(smem <= 232448, "tile kernel shared memory");
    if ((rc = set_smem(kern, smem))) return rc;
    // the coalesced epilogue moves 32-bit words: bf16 outputs need an even row stride and a 4-byte aligned base
    int word_ok = EPI == w8a8::EPI_BF16 ? (((uintptr_t)out & 3) == 0 && ldo % 2 == 0) : 1;
    // K splits.  split > 1 from the caller: every tile is split (few tiles, long K).  split == 1 with a workspace at
    // hand: the LAST wave of tiles, when it is a partial one, is split over the SMs it would leave idle (exact: the
    // slices' int32 sums meet in the workspace) - 320 tiles on 148 SMs take 2.2 waves instead of 3.
    const int KB = (K + 127) / 128;
    const int tiles = ((M + 127) / 128) * ((N + BN - 1) / BN);
    const int sms = sm_count();
    int full_tiles = split > 1 ? 0 : tiles;
    // (measured: a gain of 3-8 % for K = 17408, a loss for K = 5120, where a tile's main loop is shorter than the trip of
    // its slices through the workspace: long K only)
    if (split == 1 && workspace && counters && tail_split_enabled() && tiles > sms && KB >= 96) {
        const int tail = tiles % sms;
        if (tail > 0 && tail * 5 <= sms * 3) {                     // a last wave less than 60 % full
            int s = sms / tail;
            if (s > 8) s = 8;
            if (s > KB / 8) s = KB / 8;                            // at least eight K blocks per slice
            if (s > 1 && (long)tail * s * 128 * BN * 4 <= workspace_bytes && tail <= n_counters) {
                const int per = (KB + s - 1) / s;
                split = (KB + per - 1) / per;
                full_tiles = tiles - tail;
            }
        }
    }
    // residual add: 32 x 32 fp32 boxes added into out by the copy engine (bit 1 of word_ok), when out can be a tensor map
    CUtensorMap tout = ta;
    const bool whole_tiles = full_tiles > 0;
    if (EPI == w8a8::EPI_ADD && whole_tiles && add_mode() == 1 && ((uintptr_t)out & 15) == 0 && ldo % 4 == 0) {
        if ((rc = tensor_map(&tout, out, N, M, (uint64_t)ldo * 4, 32, 32, 4))) return rc;
        word_ok |= 2;
    } else if (EPI == w8a8::EPI_ADD && whole_tiles && add_mode() == 2) {
        word_ok |= 4;
    }
    if (g_drop_loads) word_ok |= 16;                               // failure injection (pb_test_drop_loads)
    // weight tiles fastest when the activations are the larger operand, do not fit in L2 and the weights do
    if ((long)M * K > (long)N * K && (long)M * K > (64l << 20) && (long)N * K <= (100l << 20)) word_ok |= 8;
    const int kbs = (KB + split - 1) / split;
    const int units = full_tiles + (tiles - full_tiles) * split;
    const int grid = units < sms ? units : sms;
    w8a8::RowBlocks rb{};
    if (blocks) rb = *blocks;
    kern<<<grid, w8a8::TileWarps<EPI>::THREADS, smem, st>>>(ta, tw, tout, a_s, w_s, out, ldo, n_rows, M, N, K, word_ok,
                                                           split, kbs, (int32_t*)workspace, counters, rb, souts, gbn,
                                                           full_tiles);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// The CTA-pair kernel (clusters of two): 256 x 256 tiles.  Opt-in with PRISM_B200_PAIR=1: under the 1 kW power cap it
// sustains the same rate as the single-CTA tile kernel and is a little slower in short bursts.
bool pair_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_PAIR");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// PRISM_B200_MXFP4_NARROW=1: the 128 x 128 MXFP4 kernel for every shape (comparison runs).
bool mxfp4_narrow_only() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_MXFP4_NARROW");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// PRISM_B200_W4A8_TILE=1 keeps the many-rows W4A8 kernel for every batch (comparison runs).
bool w4a8_tile_only() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_W4A8_TILE");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// PRISM_B200_W4A8_STAGED=1: the few-rows Q4_K kernel that stages the expanded operand in shared memory (comparison runs).
bool w4a8_few_staged() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_W4A8_STAGED");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

template <int EPI>
int launch_pair(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, void* out, long ldo,
                const int* n_rows, int M, int N, int K, cudaStream_t st) {
    CUtensorMap ta, tw;
    int rc;
    if ((rc = tensor_map(&ta, a, K, M, K, w8a8::BK, w8a8::BM, 0))) return rc;
    if ((rc = tensor_map(&tw, w, K, N, K, w8a8::BK, w8a8::BM, 0))) return rc;
    auto kern = w8a8::w8a8_pair_kernel<EPI>;
    if ((rc = set_smem(kern, w8a8::PAIR_SMEM))) return rc;
    const int word_ok = EPI == w8a8::EPI_BF16 ? (((uintptr_t)out & 3) == 0 && ldo % 2 == 0) : 1;
    const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
    int pairs = sm_count() / 2;
    if (pairs > tiles) pairs = tiles;
    // the kernel carries its cluster shape (2 x 1 x 1) at compile time: an even grid is all a launch needs
    kern<<<2 * pairs, 192, w8a8::PAIR_SMEM, st>>>(ta, tw, a_s, w_s, out, ldo, n_rows, M, N, K, word_ok);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

template <int NB, bool GROUPED, int RW = 0>
int launch_swap(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, w8a8::SwapArgs p, int split,
                cudaStream_t st) {
    using C = w8a8::SwapCfg<NB, GROUPED>;
    constexpr int RCTA = RW ? 2 * RW : NB;                         // activation rows per CTA
    CUtensorMap tw, tx, tsw, tsa;
    int rc;
    // per-32 groups in one K slice: PRISM_B200_WROWS = 64 / 32 gives every CTA fewer weight rows (more CTAs when the
    // 128-row tiles are fewer than the SMs; the group order, and so every bit, stays the same).  Measured on B200 at 16
    // rows: 5120 x 5120 takes 46 us with 32-row tiles against 25.6 us with 128-row ones (the time goes with the number
    // of K stages a CTA walks through, not with its bytes), so 128 stays the default.
    int wrows = w8a8::BM;
    if (GROUPED && split == 1) {
        static const int forced = [] { const char* e = getenv("PRISM_B200_WROWS"); return e ? atoi(e) : 0; }();
        if (forced == 32 || forced == 64) wrows = forced;
    }
    p.wrows = wrows;
    if ((rc = tensor_map(&tw, w, p.K, p.N, p.K, w8a8::BK, wrows, 0))) return rc;
    if ((rc = tensor_map(&tx, a, p.K, p.M, p.K, w8a8::BK, NB, 0))) return rc;
    if (GROUPED) {
        const uint64_t G = p.K / 32;
        if ((rc = tensor_map(&tsw, w_s, G, p.N, G * 4, 4, w8a8::BM, 1))) return rc;
        if ((rc = tensor_map(&tsa, a_s, G, p.M, G * 4, 4, NB, 1))) return rc;
    } else {
        tsw = tw;
        tsa = tx;
    }
    auto kern = w8a8::w8a8_swap_kernel<NB, GROUPED, RW>;
    if ((rc = set_smem(kern, C::smem_bytes(C::STAGES_DEEP)))) return rc;
    dim3 grid((p.N + wrows - 1) / wrows, split, (p.M + RCTA - 1) / RCTA);
    // a grid no larger than the SM count gets one CTA per SM and the deepest pipeline; a larger one two CTAs per SM
    // (per-32 groups: the accumulator slots fill the SM's tensor memory, so one CTA per SM at any grid size)
    p.stages = (GROUPED || (long)grid.x * grid.y * grid.z <= sm_count()) ? C::STAGES_DEEP : C::STAGES;
    const int smem = C::smem_bytes(p.stages);
    if (p.pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(C::THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        PB_CUDA(cudaLaunchKernelEx(&cfg, kern, tw, tx, tsw, tsa, p));
        return PB_OK;
    }
    kern<<<grid, C::THREADS, smem, st>>>(tw, tx, tsw, tsa, p);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// Per-32 groups, up to 16 rows, one K slice, fewer weight tiles than SMs: how many activation rows a CTA owns (16, 8 or
// 4).  Fewer rows per CTA = more CTAs on one weight tile, i.e. the per-group fp32 arithmetic (what bounds this kernel:
// ncu shows the fp32 pipe saturated on the SMs in use) spread over more SMs; the smallest count whose grid still
// fits the SMs at once.  PRISM_B200_GROWS forces 16 / 8 / 4.
int grouped_rows_per_cta(int M, int N) {
    static const int forced = [] { const char* e = getenv("PRISM_B200_GROWS"); return e ? atoi(e) : 0; }();
    if (forced == 16 || forced == 8 || forced == 4) return forced;
    const long tiles = (N + 127) / 128, cap = sm_count();     // one wave: a CTA takes a whole SM
    for (int r : {4, 8})
        if (M > r && tiles * ((M + r - 1) / r) <= cap) return r;
    return 16;
}

// Per-32 groups, one K slice (w8a8_g32.cuh): NB = 16 with row blocks of 16, 8 or 4 per CTA, or NB = 32 (more than 16 rows).
template <int NB, int RW>
int launch_g32(const int8_t* a, const int8_t* w, w8a8::SwapArgs p, cudaStream_t st) {
    using C = w8a8::G32<NB>;
    constexpr int RCTA = 2 * RW;
    CUtensorMap tw, tx;
    int rc;
    if ((rc = tensor_map_kchunks(&tw, w, p.N, p.K, w8a8::BM))) return rc;
    if ((rc = tensor_map_kchunks(&tx, a, p.M, p.K, NB))) return rc;
    p.stages = C::stages_for(p.K, RCTA);
    const int smem = C::smem_bytes(p.K, RCTA, p.stages);
    auto kern = w8a8::w8a8_g32_kernel<NB, RW>;
    if ((rc = set_smem(kern, 232448))) return rc;
    dim3 grid((p.N + w8a8::BM - 1) / w8a8::BM, 1, (p.M + RCTA - 1) / RCTA);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 1 : 0;
    PB_CUDA(cudaLaunchKernelEx(&cfg, kern, tw, tx, p));
    return PB_OK;
}

// Can w8a8_g32_kernel take the call?  One K slice, a direct store, and room for at least three stages beside the
// activation scales (K up to about 80 k at 16 rows, 40 k at 32).  PRISM_B200_G32=0 keeps the older kernel (comparisons).
int g32_rows(const w8a8::SwapArgs& p, int split) {
    static const bool on = [] { const char* e = getenv("PRISM_B200_G32"); return !(e && e[0] == '0'); }();
    if (!on || split != 1 || p.mode != w8a8::MODE_DIRECT || p.wrows != 0 || p.K % 128 != 0 ||
        !(p.epi == w8a8::EPI_BF16 || p.epi == w8a8::EPI_ADD || p.epi == w8a8::EPI_F32))
        return 0;
    // more than 16 rows: row blocks of 16 while they all fit one wave (the per-group fp32 chain, which bounds the kernel,
    // then spreads over more SMs: 20 against 31 us on 5120 x 5120 at 32 rows), blocks of 32 beyond that (half the
    // re-reads of the weights from L2: 31.6 against 37.8 us at 64 rows)
    const long blocks16 = (long)((p.N + 127) / 128) * ((p.M + 15) / 16);
    if (p.M > 16 && blocks16 > sm_count() && w8a8::G32<32>::stages_for(p.K, 32) >= 3) return 32;
    return w8a8::G32<16>::stages_for(p.K, 16) >= 3 ? 16 : 0;
}

template <bool GROUPED>
int launch_swap_nb(int nb, const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, w8a8::SwapArgs p,
                   int split, cudaStream_t st) {
    if constexpr (GROUPED) if (const int rows = g32_rows(p, split)) {
        if (rows == 32) return launch_g32<32, 16>(a, w, p, st);
        const int r = p.M <= 16 ? grouped_rows_per_cta(p.M, p.N) : 16;
        if (r == 4) return launch_g32<16, 2>(a, w, p, st);
        if (r == 8) return launch_g32<16, 4>(a, w, p, st);
        return launch_g32<16, 8>(a, w, p, st);
    }
    if constexpr (GROUPED) if (nb == 16 && split == 1) {
        const int r = grouped_rows_per_cta(p.M, p.N);
        if (r == 4) return launch_swap<16, GROUPED, 2>(a, a_s, w, w_s, p, split, st);
        if (r == 8) return launch_swap<16, GROUPED, 4>(a, a_s, w, w_s, p, split, st);
    }
    switch (nb) {
        case 16: return launch_swap<16, GROUPED>(a, a_s, w, w_s, p, split, st);
        case 32: return launch_swap<32, GROUPED>(a, a_s, w, w_s, p, split, st);
        default: return launch_swap<64, GROUPED>(a, a_s, w, w_s, p, split, st);
    }
}


// Scale groups of gk = 32 * gblocks inputs (w8a8_groups.cuh): any gk that is neither 32 nor K.
template <int NB>
int launch_groups(const int8_t* a, const int8_t* w, w8a8::SwapArgs p, cudaStream_t st) {
    using C = w8a8::GroupsCfg<NB>;
    CUtensorMap tw, tx;
    int rc;
    if ((rc = tensor_map(&tw, w, p.K, p.N, p.K, w8a8::BK, w8a8::BM, 0))) return rc;
    if ((rc = tensor_map(&tx, a, p.K, p.M, p.K, w8a8::BK, NB, 0))) return rc;
    auto kern = w8a8::w8a8_groups_kernel<NB>;
    if ((rc = set_smem(kern, C::SMEM))) return rc;
    dim3 grid((p.N + 127) / 128, 1, (p.M + NB - 1) / NB);
    kern<<<grid, C::THREADS, C::SMEM, st>>>(tw, tx, p);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

template <int KIND>
int launch_w4a8(const int8_t* xq, const float* a, const int8_t* xs, int Ma, const void* wq, const void* wsc,
                const void* wmn, const float* wd, const float* wdm, void* out, long ldo, const int* n_rows, int M,
                int N, int K, int epi, cudaStream_t st) {
    using C = w4a8::Cfg<KIND>;
    w4a8::Maps m;
    int rc;
    const uint64_t NSB = K / 256;
    if ((rc = tensor_map(&m.x, xq, K, M, K, 128, 128, 0))) return rc;
    if (KIND == w4a8::KIND_Q4K) {
        if ((rc = tensor_map(&m.wq, wq, K / 2, N, K / 2, 128, 64, 0))) return rc;
        if ((rc = tensor_map(&m.xs, xs, (uint64_t)Ma * 4, NSB, (uint64_t)Ma * 16, 256, 1, 3))) return rc;
        if ((rc = tensor_map(&m.sc, wsc, (uint64_t)N * 2, NSB, (uint64_t)N * 8, 128, 1, 3))) return rc;
        if ((rc = tensor_map(&m.mn, wmn, (uint64_t)N * 2, NSB, (uint64_t)N * 8, 128, 1, 3))) return rc;
        if ((rc = tensor_map(&m.dm, wdm, N, NSB, (uint64_t)N * 4, 64, 1, 1))) return rc;
    } else {
        if ((rc = tensor_map(&m.wq, wq, K, N, K, 128, 64, 0))) return rc;
        if ((rc = tensor_map(&m.sc, wsc, (uint64_t)N * 4, NSB, (uint64_t)N * 16, 256, 1, 3))) return rc;
        m.xs = m.x;
        m.mn = m.x;
        m.dm = m.x;
    }
    if ((rc = tensor_map(&m.d, wd, N, NSB, (uint64_t)N * 4, 64, 1, 1))) return rc;
    auto kern = w4a8::w4a8_kernel<KIND>;
    if ((rc = set_smem(kern, C::SMEM))) return rc;
    w4a8::Args p{a, out, ldo, n_rows, M, N, K, Ma, epi, nullptr, nullptr, nullptr, nullptr, 1, K / 256, nullptr, nullptr};
    const int grid = ((M + 127) / 128) * ((N + 63) / 64);
    kern<<<grid, w4a8::THREADS, C::SMEM, st>>>(m, p);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// Few activation rows (w4a8_few.cuh): weight tiles of 128 (Q4_K) or 64 (Q6_K) rows against 16 activation rows.
template <int KIND>
int launch_w4a8_few(const int8_t* xq, const float* a, const int8_t* xs, int Ma, const void* wq, const void* wsc,
                    const void* wmn, const float* wd, const float* wdm, void* out, long ldo, const int* n_rows, int M,
                    int N, int K, int epi, cudaStream_t st, int split = 1, float* ws = nullptr, int* counters = nullptr) {
    using C = w4a8::FewCfg<KIND>;
    w4a8::FewMaps m;
    int rc;
    const uint64_t NSB = K / 256;
    if ((rc = tensor_map(&m.x, xq, K, M, K, 128, w4a8::FEW_NB, 0))) return rc;
    if (KIND == w4a8::KIND_Q4K) {
        if ((rc = tensor_map(&m.wq, wq, K / 2, N, K / 2, 128, 128, 0))) return rc;
        if ((rc = tensor_map(&m.xs, xs, (uint64_t)Ma * 4, NSB, (uint64_t)Ma * 16, w4a8::FEW_NB * 4, 1, 3))) return rc;
        if ((rc = tensor_map(&m.sc, wsc, (uint64_t)N * 2, NSB, (uint64_t)N * 8, 256, 1, 3))) return rc;
        if ((rc = tensor_map(&m.mn, wmn, (uint64_t)N * 2, NSB, (uint64_t)N * 8, 256, 1, 3))) return rc;
        if ((rc = tensor_map(&m.dm, wdm, N, NSB, (uint64_t)N * 4, 128, 1, 1))) return rc;
    } else {
        if ((rc = tensor_map(&m.wq, wq, K, N, K, 128, 64, 0))) return rc;
        if ((rc = tensor_map(&m.sc, wsc, (uint64_t)N * 4, NSB, (uint64_t)N * 16, 256, 1, 3))) return rc;
        m.xs = m.x;
        m.mn = m.x;
        m.dm = m.x;
    }
    if ((rc = tensor_map(&m.d, wd, N, NSB, (uint64_t)N * 4, C::TILE_N, 1, 1))) return rc;
    const int nsb = K / 256;
    if (split > nsb) split = nsb;
    const int sps = (nsb + split - 1) / split;
    split = (nsb + sps - 1) / sps;                                    // no empty slice
    w4a8::Args p{a, out, ldo, n_rows, M, N, K, Ma, epi, (const uint8_t*)wsc, (const uint8_t*)wmn, wd, wdm, split, sps, ws,
                 counters};
    // the row tiles of one weight tile are neighbours in launch order: the weights of all but the first come from L2
    dim3 grid((M + w4a8::FEW_NB - 1) / w4a8::FEW_NB, (N + C::TILE_N - 1) / C::TILE_N);
    if (KIND == w4a8::KIND_Q4K && !w4a8_few_staged()) {
        // Q4_K: the expanded operand goes through tensor memory
        if ((rc = set_smem(w4a8::w4a8_few_q4k_tm_kernel<false>, w4a8::TmCfg::SMEM))) return rc;
        if ((rc = set_smem(w4a8::w4a8_few_q4k_tm_kernel<true>, w4a8::TmCfg::SMEM))) return rc;
        grid.z = split;
        if (split > 1) w4a8::w4a8_few_q4k_tm_kernel<true><<<grid, w4a8::FEW_THREADS, w4a8::TmCfg::SMEM, st>>>(m, p);
        else w4a8::w4a8_few_q4k_tm_kernel<false><<<grid, w4a8::FEW_THREADS, w4a8::TmCfg::SMEM, st>>>(m, p);
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    auto kern = w4a8::w4a8_few_kernel<KIND>;
    if ((rc = set_smem(kern, C::SMEM))) return rc;
    if (KIND == w4a8::KIND_Q6K) grid.z = split;
    else p.split = 1;
    kern<<<grid, w4a8::FEW_THREADS, C::SMEM, st>>>(m, p);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// One to four activation rows: integer dot products on the CUDA cores (w4a8_gemv.cuh).
template <int MR>
int launch_w4a8_gemv(int kind, const w4a8::GemvArgs& p, cudaStream_t st) {
    constexpr int R = w4a8::GEMV_R;
    const int grid = (p.N + 4 * R - 1) / (4 * R);                  // eight weight rows per CTA
    auto split_k = kind == 0 ? w4a8::w4a8_gemv_q4k_kernel<MR, R, true> : w4a8::w4a8_gemv_q6k_kernel<MR, R, true>;
    auto whole_k = kind == 0 ? w4a8::w4a8_gemv_q4k_kernel<MR, R, false> : w4a8::w4a8_gemv_q6k_kernel<MR, R, false>;
    // few rows: two to four warps per CTA share the rows' super-blocks (exact: the chain runs in order afterwards);
    // the most warps with which the whole grid is resident at once (a second, short wave would double the time)
    const size_t smem = (size_t)(p.K >> 8) * 4 * R * MR * sizeof(float);
    if (grid < 8 * sm_count() && smem <= 48 * 1024) {
        static int resident_dev[kMaxDevices][2][5] = {};           // [device][kind][warps] CTAs per SM, 0 = not asked yet
        int (&resident)[2][5] = resident_dev[current_device()];
        int kw = 2;
        for (int k = 4; k >= 2; --k) {
            if (!resident[kind][k]) {
                int nb = 0;
                PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, split_k, 32 * k, 16 * 1024));
                resident[kind][k] = nb > 0 ? nb : 1;
            }
            if ((long)grid <= (long)resident[kind][k] * sm_count()) {
                kw = k;
                break;
            }
        }
        split_k<<<grid, 32 * kw, smem, st>>>(p);
    } else {
        whole_k<<<grid, 32, 0, st>>>(p);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

template <int MR>
int launch_mxfp4_gemv(const mxfp4::GemvArgs& p, cudaStream_t st) {
    const int grid = (p.N + 7) / 8;                                // eight weight rows per CTA
    if (grid < 8 * sm_count()) {
        // few rows: the most warps per CTA with which the whole grid is resident at once
        static int resident_dev[kMaxDevices][5] = {};
        int (&resident)[5] = resident_dev[current_device()];
        int kw = 2;
        for (int k = 4; k >= 2; --k) {
            if (!resident[k]) {
                int nb = 0;
                PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, mxfp4::mxfp4_gemv_kernel<MR, true>, 32 * k, 1024));
                resident[k] = nb > 0 ? nb : 1;
            }
            if ((long)grid <= (long)resident[k] * sm_count()) {
                kw = k;
                break;
            }
        }
        mxfp4::mxfp4_gemv_kernel<MR, true><<<grid, 32 * kw, (size_t)kw * 8 * MR * sizeof(float), st>>>(p);
    } else {
        mxfp4::mxfp4_gemv_kernel<MR, false><<<grid, 32, 0, st>>>(p);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

template <int MR>
int launch_w8a8_gemv(const w8a8::GemvArgs& p, cudaStream_t st) {
    const int grid = (p.N + 7) / 8;                                // eight weight rows per CTA
    if (grid < 8 * sm_count()) {
        // few rows: the most warps per CTA with which the whole grid is resident at once
        static int resident_dev[kMaxDevices][5] = {};
        int (&resident)[5] = resident_dev[current_device()];
        int kw = 2;
        for (int k = 4; k >= 2; --k) {
            if (!resident[k]) {
                int nb = 0;
                PB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, w8a8::w8a8_gemv_kernel<MR, true>, 32 * k, 2048));
                resident[k] = nb > 0 ? nb : 1;
            }
            if ((long)grid <= (long)resident[k] * sm_count()) {
                kw = k;
                break;
            }
        }
        w8a8::w8a8_gemv_kernel<MR, true><<<grid, 32 * kw, (size_t)kw * 8 * MR * sizeof(int), st>>>(p);
    } else {
        w8a8::w8a8_gemv_kernel<MR, false><<<grid, 32, 0, st>>>(p);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// PRISM_B200_W8A8_NO_GEMV=1 keeps the tensor-core kernel for one to eight rows (comparison runs).
bool w8a8_no_gemv() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_W8A8_NO_GEMV");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// PRISM_B200_W4A8_NO_GEMV=1 keeps the tensor-core kernels for one to four rows (comparison runs).
bool w4a8_no_gemv() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_W4A8_NO_GEMV");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// Row-pipelined quantizers (quant_pipe.cuh): persistent CTAs, rows staged in shared memory by bulk copies.
template <int KIND, int VPT, bool BF16>
int launch_pipe_v(bool full, const quant::PipeArgs& p, int grid, int threads, int smem, cudaStream_t st) {
    int rc;
    if (full) {
        auto k = quant::row_pipe_kernel<KIND, VPT, BF16, true, 576>;
        if ((rc = set_smem(k, 200 * 1024))) return rc;
        k<<<grid, threads, smem, st>>>(p);
    } else {
        auto k = quant::row_pipe_kernel<KIND, VPT, BF16, false, 576>;
        if ((rc = set_smem(k, 200 * 1024))) return rc;
        k<<<grid, threads, smem, st>>>(p);
    }
    return PB_OK;
}

template <int KIND, bool BF16>
int launch_pipe(bool full, quant::PipeArgs p, cudaStream_t st) {
    const int nvec = p.K / 8;
    // two CTAs per SM: about 100 KB of row ring each
    int stages = (100 * 1024) / p.row_bytes;
    int per_sm = 2;
    if (stages < 2) {                                             // very long rows: one CTA per SM
        stages = (199 * 1024) / p.row_bytes;
        per_sm = 1;
    }
    if (stages < 2) return PB_UNSUPPORTED_SHAPE;
    if (stages > 8) stages = 8;
    p.stages = stages;
    const int smem = stages * p.row_bytes + 128;
    int grid = sm_count() * per_sm;
    if (grid > p.T) grid = p.T;
    // vectors of 8 inputs per thread, then just enough threads (whole warps) to cover the row
    const int vpt = (nvec + 575) / 576;
    const int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
    int rc;
    switch (vpt) {
        case 1: rc = launch_pipe_v<KIND, 1, BF16>(full, p, grid, threads, smem, st); break;
        case 2: rc = launch_pipe_v<KIND, 2, BF16>(full, p, grid, threads, smem, st); break;
        case 3: rc = launch_pipe_v<KIND, 3, BF16>(full, p, grid, threads, smem, st); break;
        case 4: rc = launch_pipe_v<KIND, 4, BF16>(full, p, grid, threads, smem, st); break;
        case 5: rc = launch_pipe_v<KIND, 5, BF16>(full, p, grid, threads, smem, st); break;
        case 6: rc = launch_pipe_v<KIND, 6, BF16>(full, p, grid, threads, smem, st); break;
        case 7: rc = launch_pipe_v<KIND, 7, BF16>(full, p, grid, threads, smem, st); break;
        case 8: rc = launch_pipe_v<KIND, 8, BF16>(full, p, grid, threads, smem, st); break;
        default: return PB_UNSUPPORTED_SHAPE;
    }
    if (rc) return rc;
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

constexpr int kPipeMinRows = 256;      // below this one CTA per row is as good (too few rows to pipeline)

// activation rows per CTA = the MMA's N: tcgen05.mma with M = 128 takes N = 16, 32, ... 256 (N = 8 needs M = 64)
int pick_nb(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }

bool div_full() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PRISM_B200_QUANT_DIV");
        v = (e && e[0] == 'f') ? 1 : 0;   // "full": div.full.f32 instead of the IEEE division
    }
    return v == 1;
}

template <int VPT>
void launch_rows(bool bf16, bool full, int threads, const void* x, long ldx, const float* inv_s, int8_t* q, float* s,
                        const int* n_rows, int T, int K, int mode, float* amax, const tpx::Sync& sy, cudaStream_t st) {
    if (bf16) {
        if (full) (void)(launch_dep(quant::rows_q8_kernel<VPT, true, true>, dim3(T), dim3(threads), 0, st, x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy));
        else (void)(launch_dep(quant::rows_q8_kernel<VPT, true, false>, dim3(T), dim3(threads), 0, st, x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy));
    } else {
        if (full) (void)(launch_dep(quant::rows_q8_kernel<VPT, false, true>, dim3(T), dim3(threads), 0, st, x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy));
        else (void)(launch_dep(quant::rows_q8_kernel<VPT, false, false>, dim3(T), dim3(threads), 0, st, x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy));
    }
}


}  // namespace

// ------------------------------------------------------------------------------------------------- static scratch
// Scratch of pb_w8a8_gemm_static: the split-K workspace and its per-tile counters live in the library's own device
// image instead of in memory the caller allocates.  Every GPU that loads the library holds these bytes until the
// process exits.  In host code the array's name is only a handle for the runtime: the device address is looked up
// with cudaGetSymbolAddress, once per device, and that address is what the kernel receives.
#define PB_STATIC_WS_BYTES (16l << 20)
#define PB_STATIC_COUNTERS 4096
static __device__ __align__(256) unsigned char g_static_scratch[PB_STATIC_WS_BYTES + PB_STATIC_COUNTERS * 4];

namespace {
void* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_scratch_mu;

// The device address of g_static_scratch on the current device (set-up on the first call per device).
int static_scratch(void** out) {
    int dev = -1;
    PB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return PB_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        PB_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        if (!ptr) return PB_CUDA_ERROR;
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return PB_OK;
}
}  // namespace

extern "C" {

int pb_version(void) { return 1; }

const char* pb_status_string(int s) {
    switch (s) {
        case PB_OK: return "ok";
        case PB_BAD_ARGUMENT: return "bad argument (null or misaligned pointer, negative size, unknown enum)";
        case PB_UNSUPPORTED_SHAPE: return "unsupported shape";
        case PB_CUDA_ERROR: return "a CUDA call failed";
        case PB_DEVICE_TIMEOUT: return "a kernel gave up a bounded wait";
        case PB_TOO_LARGE: return "size beyond a stated maximum";
    }
    return "unknown status";
}

int pb_last_cuda_error(void) { return g_last_cuda_error; }

int pb_device_status(int* code, unsigned* where, int reset) {
    int c = 0;
    unsigned w = 0;
    PB_CUDA(cudaDeviceSynchronize());
    PB_CUDA(cudaMemcpyFromSymbol(&c, g_pb_device_status, sizeof(int)));
    PB_CUDA(cudaMemcpyFromSymbol(&w, g_pb_device_status_where, sizeof(unsigned)));
    if (code) *code = c;
    if (where) *where = w;
    if (reset && (c || w)) {
        int z = 0;
        unsigned zw = 0;
        PB_CUDA(cudaMemcpyToSymbol(g_pb_device_status, &z, sizeof(int)));
        PB_CUDA(cudaMemcpyToSymbol(g_pb_device_status_where, &zw, sizeof(unsigned)));
    }
    return PB_OK;
}

int pb_set_wait_limit_ns(unsigned long long ns) {
    if (ns == 0) ns = PB_WAIT_NS;
    PB_CUDA(cudaMemcpyToSymbol(g_pb_wait_ns, &ns, sizeof(ns)));
    return PB_OK;
}

int pb_set_pdl(int on) { return g_pdl.exchange(on ? 1 : 0); }

int pb_test_drop_loads(int on) {
    g_drop_loads = on ? 1 : 0;
    return PB_OK;
}

// Weight rows per tile of the many-rows kernel.
int tile_bn(int M, int N) {
    if (N <= 128) return 128;
    const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    return tiles256 * 2 <= sm_count() ? 128 : 256;
}

long pb_w8a8_workspace_bytes(int M, int N, int split) {
    if (M <= 0 || N <= 0 || split <= 1) return 0;
    if (M > 64) {                                       // tile kernel: int32 [tiles][split][128][BN]
        const int bn = tile_bn(M, N);
        const long tiles = (long)((M + 127) / 128) * ((N + bn - 1) / bn);
        return tiles * split * 128 * bn * 4;
    }
    const int nb = pick_nb(M);
    const long tiles = (long)((N + 127) / 128) * ((M + nb - 1) / nb);
    return (long)split * tiles * nb * 128 * 4;
}

int pb_w8a8_counters(int M, int N) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) return ((M + 127) / 128) * ((N + tile_bn(M, N) - 1) / tile_bn(M, N));
    const int nb = pick_nb(M);
    return ((N + 127) / 128) * ((M + nb - 1) / nb);
}

int pb_w8a8_gemm(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, void* out, long ldo,
                 const int* n_rows, int M, int N, int K, int gk, int epi, int split, long slot_stride,
                 void* workspace, long workspace_bytes, int* counters, int n_counters, int pdl, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!a || !w || !out || !n_rows || M <= 0 || N <= 0 || K <= 0 || split < 1) return PB_BAD_ARGUMENT;
    if (epi != PB_EPI_BF16 && epi != PB_EPI_ADD && epi != PB_EPI_I32 && epi != PB_EPI_F32) return PB_BAD_ARGUMENT;
    const int pdl_asked = pdl;                                     // the caller's own request keeps a row off the CUDA-core kernel
    if (g_pdl.load(std::memory_order_relaxed) && M <= 64) pdl = 1;
    if (epi == PB_EPI_F32 && (gk != 32 || M > 64)) return PB_UNSUPPORTED_SHAPE;
    if (epi != PB_EPI_I32 && (!a_s || !w_s)) return PB_BAD_ARGUMENT;
    if (!aligned16(a) || !aligned16(w)) return PB_BAD_ARGUMENT;
    if (K % 16) return PB_UNSUPPORTED_SHAPE;
    if (ldo < N) return PB_BAD_ARGUMENT;
    const int KB = (K + 127) / 128;
    if (gk == 32) {
        // Q8_0's own scale per 32 inputs: fp32 partial sums per group, added in group order (no K split, no int32 out)
        if (epi == PB_EPI_I32) return PB_UNSUPPORTED_SHAPE;
        if (K % 128 || !aligned16(a_s) || !aligned16(w_s)) return PB_UNSUPPORTED_SHAPE;
        if (split > 1 && M > 64) return PB_UNSUPPORTED_SHAPE;
        if (split > KB) split = KB;
        const int kbs = (KB + split - 1) / split;
        split = (KB + kbs - 1) / kbs;
        w8a8::SwapArgs p{a_s, w_s, out, ldo, 0, (int32_t*)workspace, counters, n_rows, M, N, K, kbs, epi,
                         split == 1 ? w8a8::MODE_DIRECT : w8a8::MODE_WS, pdl != 0, 0};
        if (split > 1) {
            // fp32 slice sums are added in slice order by the tile's last CTA: deterministic, within fp32 rounding of
            // the unsplit group order (one bf16 step at most after the store)
            if (!workspace || !counters) return PB_BAD_ARGUMENT;
            if (workspace_bytes < pb_w8a8_workspace_bytes(M, N, split) || n_counters < pb_w8a8_counters(M, N))
                return PB_TOO_LARGE;
        }
        return launch_swap_nb<true>(pick_nb(M), a, a_s, w, w_s, p, split, st);
    }
    if (gk != K) {
        // any other group size (a multiple of 32 that divides K): one accumulator slot per group, fp32 sums in group
        // order.  No K split, no int32 output.
        if (gk <= 0 || gk % 32 || K % gk || K % 128 || epi == PB_EPI_I32 || epi == PB_EPI_F32) return PB_UNSUPPORTED_SHAPE;
        if (split > 1) return PB_UNSUPPORTED_SHAPE;
        w8a8::SwapArgs p{a_s, w_s, out, ldo, 0, nullptr, nullptr, n_rows, M, N, K, KB, epi, w8a8::MODE_DIRECT, 0, 0, gk / 32};
        const int nb = pick_nb(M);
        if (nb == 16) return launch_groups<16>(a, w, p, st);
        if (nb == 32) return launch_groups<32>(a, w, p, st);
        return launch_groups<64>(a, w, p, st);
    }
    if (M <= PB_W8A8_GEMV_ROWS && (N + 7) / 8 < 8 * sm_count() && split == 1 && !pdl_asked && K % 256 == 0 &&
        (epi == PB_EPI_BF16 || epi == PB_EPI_ADD) && !w8a8_no_gemv()) {
        // one row against a matrix of few rows, no K split asked for: the CUDA-core kernel (the same bits: exact
        // integer sums, the same two multiplies).  Measured at one row: qkv 9.8 / o 7.6 / down 18.4 µs against the
        // tensor-core kernel's 12.4 / 10.9 / 20.7 with its fold; level on the 34816-row gate|up; behind from two rows
        // on (its dp4a work grows with the rows: 61 µs at four rows of gate|up against 31).
        w8a8::GemvArgs g{a, a_s, w, w_s, out, ldo, n_rows, M, N, K, epi};
        return launch_w8a8_gemv<1>(g, st);
    }
    if (M >= 512 && N >= 256 && pair_enabled() && split == 1) {
        if (epi == PB_EPI_I32) return launch_pair<w8a8::EPI_I32>(a, a_s, w, w_s, out, ldo, n_rows, M, N, K, st);
        if (epi == PB_EPI_BF16) return launch_pair<w8a8::EPI_BF16>(a, a_s, w, w_s, out, ldo, n_rows, M, N, K, st);
        return launch_pair<w8a8::EPI_ADD>(a, a_s, w, w_s, out, ldo, n_rows, M, N, K, st);
    }
    if (M > 64) {
        // many rows: K splits (few tiles only: callers pick them, w8a8.pick_split) add their int32 partial sums in a
        // workspace, exactly; the last CTA of a tile runs the epilogue
        if (split > KB) split = KB;
        if (split > 1) {
            const int kbs = (KB + split - 1) / split;
            split = (KB + kbs - 1) / kbs;
        }
        if (split > 1) {
            if (!workspace || !counters) return PB_BAD_ARGUMENT;
            if (workspace_bytes < pb_w8a8_workspace_bytes(M, N, split) || n_counters < pb_w8a8_counters(M, N))
                return PB_TOO_LARGE;
        }
        // tile width: 128 x 256, 128 x 128 when those would leave more than half of the SMs without a tile, or (one K
        // slice only) 128 x 192 when that needs fewer tile-widths of waves: 5120 columns at 2048 rows are 320 tiles
        // of 256 = 3 waves x 256, but 432 tiles of 192 = 3 waves x 192
        int bn = (N <= 128 || tile_bn(M, N) == 128) ? 128 : 256;
        if (bn == 256 && split == 1 && wide192_enabled()) {
            const long mt = (M + 127) / 128, sms = sm_count();
            const long w256 = (mt * ((N + 255) / 256) + sms - 1) / sms * 256 * 100;
            const long w192 = (mt * ((N + 191) / 192) + sms - 1) / sms * 192 * 107;     // its operand traffic per MMA is higher
            if (w192 < w256) bn = 192;
        }
#define PB_TILE(BN_, EPI_) launch_tile<BN_, w8a8::EPI_>(a, a_s, w, w_s, out, ldo, n_rows, M, N, K, st, split, workspace, counters, nullptr, nullptr, 0, workspace_bytes, n_counters)
        if (epi == PB_EPI_I32) return bn == 128 ? PB_TILE(128, EPI_I32) : bn == 192 ? PB_TILE(192, EPI_I32) : PB_TILE(256, EPI_I32);
        if (epi == PB_EPI_BF16) return bn == 128 ? PB_TILE(128, EPI_BF16) : bn == 192 ? PB_TILE(192, EPI_BF16) : PB_TILE(256, EPI_BF16);
        return bn == 128 ? PB_TILE(128, EPI_ADD) : bn == 192 ? PB_TILE(192, EPI_ADD) : PB_TILE(256, EPI_ADD);
#undef PB_TILE
    }
    // few rows: operands swapped, K split over blockIdx.y
    if (split > KB) split = KB;
    int kbs = (KB + split - 1) / split;
    split = (KB + kbs - 1) / kbs;                       // every slice non-empty
    const int nb = pick_nb(M);
    w8a8::SwapArgs p{a_s, w_s, out, ldo, slot_stride, (int32_t*)workspace, counters, n_rows, M, N, K, kbs, epi, 0, pdl != 0, 0};
    if (epi == PB_EPI_I32) {
        p.mode = w8a8::MODE_SLOTS;
        if (split > 1 && slot_stride < (long)M * N) return PB_BAD_ARGUMENT;
    } else if (split == 1) {
        p.mode = w8a8::MODE_DIRECT;
    } else {
        p.mode = w8a8::MODE_WS;
        if (!workspace || !counters) return PB_BAD_ARGUMENT;
        if (workspace_bytes < pb_w8a8_workspace_bytes(M, N, split) || n_counters < pb_w8a8_counters(M, N))
            return PB_TOO_LARGE;
    }
    return launch_swap_nb<false>(nb, a, a_s, w, w_s, p, split, st);
}

int pb_w8a8_gemm_swiglu(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, int8_t* q, long ldq, float* s,
                        const int* n_rows, int M, int N, int K, int bn, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!a || !a_s || !w || !w_s || !q || !s || !n_rows || M <= 0 || N <= 0 || K <= 0) return PB_BAD_ARGUMENT;
    if (bn != 64 && bn != 128) return PB_UNSUPPORTED_SHAPE;
    if (N % bn || K % 16 || ldq < N / 2) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(a) || !aligned16(w)) return PB_BAD_ARGUMENT;
    // 128 x 256 tiles (two or four interleave tiles each), or 128 x 128 when those would leave most SMs idle
    const bool narrow = N <= 128 || tile_bn(M, N) == 128;
    return narrow ? launch_tile<128, w8a8::EPI_SWIGLU>(a, a_s, w, w_s, q, ldq, n_rows, M, N, K, st, 1, nullptr, nullptr, nullptr, s, bn)
                  : launch_tile<256, w8a8::EPI_SWIGLU>(a, a_s, w, w_s, q, ldq, n_rows, M, N, K, st, 1, nullptr, nullptr, nullptr, s, bn);
}

int pb_w8a8_gemm_scatter(const int8_t* a, const int8_t* w, void* const* blocks, int n_blocks, int block_rows, long ldo,
                         const int* n_rows, int M, int N, int K, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!a || !w || !blocks || !n_rows || M <= 0 || N <= 0 || K <= 0) return PB_BAD_ARGUMENT;
    if (n_blocks < 1 || n_blocks > 8 || block_rows <= 0 || (long)n_blocks * block_rows < M) return PB_BAD_ARGUMENT;
    if (block_rows % 128) return PB_UNSUPPORTED_SHAPE;             // a tile lies in one block
    if (M <= 64) return PB_UNSUPPORTED_SHAPE;                      // the many-rows kernel only
    if (!aligned16(a) || !aligned16(w) || ldo < N) return PB_BAD_ARGUMENT;
    if (K % 16) return PB_UNSUPPORTED_SHAPE;
    w8a8::RowBlocks rb{};
    for (int i = 0; i < n_blocks; ++i) {
        if (!blocks[i] || !aligned16(blocks[i])) return PB_BAD_ARGUMENT;
        rb.base[i] = blocks[i];
    }
    rb.rows = block_rows;
    const bool narrow = N <= 128 || tile_bn(M, N) == 128;
    return narrow ? launch_tile<128, w8a8::EPI_I32>(a, nullptr, w, nullptr, blocks[0], ldo, n_rows, M, N, K, st, 1, nullptr, nullptr, &rb)
                  : launch_tile<256, w8a8::EPI_I32>(a, nullptr, w, nullptr, blocks[0], ldo, n_rows, M, N, K, st, 1, nullptr, nullptr, &rb);
}

// Device memory that other processes' GPUs can store into (CUDA IPC; peer access over NVLink).
int pb_peer_alloc(long bytes, void** ptr, void* handle64) {
    if (bytes <= 0 || !ptr || !handle64) return PB_BAD_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    PB_CUDA(cudaMalloc(&p, (size_t)bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        PB_CUDA(e);
    }
    memcpy(handle64, &h, 64);
    *ptr = p;
    return PB_OK;
}

int pb_peer_open(const void* handle64, void** ptr) {
    if (!handle64 || !ptr) return PB_BAD_ARGUMENT;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    PB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return PB_OK;
}

int pb_peer_close(void* ptr) {
    if (!ptr) return PB_BAD_ARGUMENT;
    PB_CUDA(cudaIpcCloseMemHandle(ptr));
    return PB_OK;
}

int pb_peer_free(void* ptr) {
    if (!ptr) return PB_BAD_ARGUMENT;
    PB_CUDA(cudaFree(ptr));
    return PB_OK;
}

int pb_fold(float* h, long ldh, const int32_t* slots, long slot_stride, int S, const float* a_s, const float* w_s,
            const int* n_rows, int rows, int N, void* stream) {
    if (!h || !slots || !a_s || !w_s || !n_rows || rows <= 0 || N <= 0 || S < 1 || ldh < N) return PB_BAD_ARGUMENT;
    if ((N % 4 == 0) && (!aligned16(h) || !aligned16(slots) || !aligned16(w_s) || (ldh % 4) || (slot_stride % 4)))
        return PB_BAD_ARGUMENT;
    dim3 grid(((N + 3) / 4 + 255) / 256, rows);
    PB_CUDA(launch_dep(quant::fold_kernel, grid, dim3(256), 0, (cudaStream_t)stream, h, ldh, slots, slot_stride, S, a_s, w_s, n_rows, N));
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

// pb_sync (the C struct) -> the kernels' view; world <= 1 when there is none
static int to_sync(const pb_sync* in, tpx::Sync* out, bool need_others) {
    memset(out, 0, sizeof(*out));
    out->world = 1;
    if (!in) return PB_OK;
    if (in->world < 2 || in->world > tpx::MAX_RANKS || in->rank < 0 || in->rank >= in->world || !in->epoch) return PB_BAD_ARGUMENT;
    out->epoch = in->epoch;
    for (int r = 0; r < in->world; ++r) {
        if (!in->bufs[r] || ((uintptr_t)in->bufs[r] & 7)) return PB_BAD_ARGUMENT;
        out->bufs[r] = (unsigned long long*)in->bufs[r];
    }
    for (int r = 0; r + 1 < in->world; ++r) {
        if (need_others && (!in->others[r] || !aligned16(in->others[r]))) return PB_BAD_ARGUMENT;
        out->others[r] = (const int32_t*)in->others[r];
    }
    out->off = in->off;
    out->rank = in->rank;
    out->world = in->world;
    return PB_OK;
}

static int quant_rows_impl(const void* x, int x_fp32, long ldx, const float* inv_s, int8_t* q, float* s, const int* n_rows,
                           int T, int K, int gk, int mode, float* amax, const tpx::Sync& sy, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!x || !q || !s || !n_rows || T <= 0 || K <= 0 || gk <= 0 || K % gk) return PB_BAD_ARGUMENT;
    if (mode < 0 || mode > 3 || ((mode == 1 || mode == 2) && !amax) || ldx < K) return PB_BAD_ARGUMENT;
    if (mode == 3 && (sy.world < 2 || gk != K)) return PB_BAD_ARGUMENT;
    const bool bf16 = !x_fp32, full = div_full();
    if (gk != K) {
        if (inv_s || mode != 0 || ldx != K) return PB_UNSUPPORTED_SHAPE;
        if (gk != 32 && gk != 64 && gk != 128 && gk != 256) return PB_UNSUPPORTED_SHAPE;
        if (!aligned16(x) || ((uintptr_t)q & 7)) return PB_BAD_ARGUMENT;
        dim3 grid((K / 8 + 255) / 256, T);
        if (bf16) {
            if (full) quant::quant_groups_kernel<true, true><<<grid, 256, 0, st>>>(x, q, s, n_rows, K, gk);
            else quant::quant_groups_kernel<true, false><<<grid, 256, 0, st>>>(x, q, s, n_rows, K, gk);
        } else {
            if (full) quant::quant_groups_kernel<false, true><<<grid, 256, 0, st>>>(x, q, s, n_rows, K, gk);
            else quant::quant_groups_kernel<false, false><<<grid, 256, 0, st>>>(x, q, s, n_rows, K, gk);
        }
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    const bool fast = K % 8 == 0 && K <= 65536 && aligned16(x) && (ldx * (bf16 ? 2 : 4)) % 16 == 0 && !((uintptr_t)q & 7) && (!inv_s || aligned16(inv_s));
    if (!fast) {
        if (bf16) {
            if (full) quant::rows_q8_generic_kernel<true, true><<<T, 256, 0, st>>>(x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy);
            else quant::rows_q8_generic_kernel<true, false><<<T, 256, 0, st>>>(x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy);
        } else {
            if (full) quant::rows_q8_generic_kernel<false, true><<<T, 256, 0, st>>>(x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy);
            else quant::rows_q8_generic_kernel<false, false><<<T, 256, 0, st>>>(x, ldx, inv_s, q, s, n_rows, K, mode, amax, sy);
        }
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    if (T >= kPipeMinRows && K <= 32768 && mode != 3) {        // (the in-kernel exchange lives in the one-CTA-per-row kernels)
        quant::PipeArgs pa{x, ldx, inv_s, q, s, n_rows, amax, T, K, mode, K * (bf16 ? 2 : 4), 0};
        const int rc = bf16 ? launch_pipe<quant::PIPE_ROWS, true>(full, pa, st)
                            : launch_pipe<quant::PIPE_ROWS, false>(full, pa, st);
        if (rc != PB_UNSUPPORTED_SHAPE) return rc;
    }
    // 4 vectors of 8 inputs per thread (8 beyond 32768 / 2 inputs), as many threads as the row needs
    const int nvec = K / 8;
    const int vpt = nvec <= 4096 ? 4 : 8;
    const int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
    if (vpt == 4) launch_rows<4>(bf16, full, threads, x, ldx, inv_s, q, s, n_rows, T, K, mode, amax, sy, st);
    else launch_rows<8>(bf16, full, threads, x, ldx, inv_s, q, s, n_rows, T, K, mode, amax, sy, st);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_quant_rows(const void* x, int x_fp32, long ldx, const float* inv_s, int8_t* q, float* s, const int* n_rows,
                  int T, int K, int gk, int mode, float* amax, void* stream) {
    if (mode == 3) return PB_BAD_ARGUMENT;                         // pb_quant_rows_exchange
    tpx::Sync sy;
    to_sync(nullptr, &sy, false);
    return quant_rows_impl(x, x_fp32, ldx, inv_s, q, s, n_rows, T, K, gk, mode, amax, sy, stream);
}

int pb_quant_rows_exchange(const void* x, int x_fp32, long ldx, const float* inv_s, int8_t* q, float* s, const int* n_rows,
                           int T, int K, const pb_sync* sync, void* stream) {
    tpx::Sync sy;
    int rc = to_sync(sync, &sy, false);
    if (rc) return rc;
    if (!sync) return PB_BAD_ARGUMENT;
    return quant_rows_impl(x, x_fp32, ldx, inv_s, q, s, n_rows, T, K, K, 3, nullptr, sy, stream);
}

static int norm_q8_impl(float* h, const float* w, int8_t* q, float* s, const int* rows, const int* n_rows, int T, int HID,
                        float eps, const int32_t* parts, long part_stride, int n_parts, const float* psa, const float* psw,
                        const tpx::Sync& sy, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!h || !w || !q || !s || !n_rows || T <= 0 || HID <= 0 || n_parts < 0) return PB_BAD_ARGUMENT;
    if (n_parts > 0 && (!parts || !psa || !psw || rows)) return PB_BAD_ARGUMENT;
    if (HID % 8 || HID > 65536) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(h) || !aligned16(w) || ((uintptr_t)q & 7) || (n_parts > 0 && (!aligned16(parts) || !aligned16(psw) || part_stride % 4)))
        return PB_BAD_ARGUMENT;
    const bool full = div_full();
    const int nvec = HID / 8;
    const int vpt = nvec <= 2048 ? 4 : 8;
    const int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
    if (vpt == 4) {
        if (full) quant::norm_q8_kernel<4, true><<<T, threads, 0, st>>>(h, w, q, s, rows, n_rows, HID, eps, parts, part_stride, n_parts, psa, psw, sy);
        else quant::norm_q8_kernel<4, false><<<T, threads, 0, st>>>(h, w, q, s, rows, n_rows, HID, eps, parts, part_stride, n_parts, psa, psw, sy);
    } else {
        if (full) quant::norm_q8_kernel<8, true><<<T, threads, 0, st>>>(h, w, q, s, rows, n_rows, HID, eps, parts, part_stride, n_parts, psa, psw, sy);
        else quant::norm_q8_kernel<8, false><<<T, threads, 0, st>>>(h, w, q, s, rows, n_rows, HID, eps, parts, part_stride, n_parts, psa, psw, sy);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_norm_q8(float* h, const float* w, int8_t* q, float* s, const int* rows, const int* n_rows, int T, int HID,
               float eps, const int32_t* parts, long part_stride, int n_parts, const float* psa, const float* psw,
               void* stream) {
    tpx::Sync sy;
    to_sync(nullptr, &sy, false);
    return norm_q8_impl(h, w, q, s, rows, n_rows, T, HID, eps, parts, part_stride, n_parts, psa, psw, sy, stream);
}

int pb_norm_q8_sync(float* h, const float* w, int8_t* q, float* s, const int* n_rows, int T, int HID, float eps,
                    const int32_t* parts, long part_stride, int n_parts, const float* psa, const float* psw,
                    const pb_sync* sync, void* stream) {
    tpx::Sync sy;
    int rc = to_sync(sync, &sy, true);
    if (rc) return rc;
    if (!sync || n_parts <= 0) return PB_BAD_ARGUMENT;
    return norm_q8_impl(h, w, q, s, nullptr, n_rows, T, HID, eps, parts, part_stride, n_parts, psa, psw, sy, stream);
}

static int gated_norm_q8_impl(const float* o, const void* proj, long P, long z_off, const float* w, const float* inv_s, int8_t* q,
                              float* s, const int* n_rows, int T, int HV, int D, float eps, int mode, float* amax,
                              const tpx::Sync& sy, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!o || !proj || !w || !inv_s || !q || !s || !n_rows || T <= 0 || HV <= 0) return PB_BAD_ARGUMENT;
    if (mode < 0 || mode > 3 || ((mode == 1 || mode == 2) && !amax) || (mode == 3 && sy.world < 2)) return PB_BAD_ARGUMENT;
    if (D != 64 && D != 128 && D != 256) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(o) || !aligned16(w) || !aligned16(inv_s) || ((uintptr_t)q & 7) || !aligned16(proj) || (P * 2) % 16 ||
        (z_off * 2) % 16)
        return PB_BAD_ARGUMENT;
    const bool full = div_full();
    const int nvec = HV * D / 8;
    if (nvec > 4 * 1024) return PB_UNSUPPORTED_SHAPE;
    // whole warps, and a head's lanes never straddle two of a thread's vectors: blockDim is a multiple of 32 >= D / 8
    const int vpt = nvec <= 1024 ? 1 : nvec <= 2048 ? 2 : 4;
    const int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
    const __nv_bfloat16* pj = (const __nv_bfloat16*)proj;
#define PB_GN(V, F) quant::gated_norm_q8_kernel<V, F><<<T, threads, 0, st>>>(o, pj, P, z_off, w, inv_s, q, s, n_rows, HV, D, eps, mode, amax, sy)
    if (vpt == 1) { if (full) PB_GN(1, true); else PB_GN(1, false); }
    else if (vpt == 2) { if (full) PB_GN(2, true); else PB_GN(2, false); }
    else { if (full) PB_GN(4, true); else PB_GN(4, false); }
#undef PB_GN
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_gated_norm_q8(const float* o, const void* proj, long P, long z_off, const float* w, const float* inv_s, int8_t* q,
                     float* s, const int* n_rows, int T, int HV, int D, float eps, int mode, float* amax, void* stream) {
    if (mode == 3) return PB_BAD_ARGUMENT;
    tpx::Sync sy;
    to_sync(nullptr, &sy, false);
    return gated_norm_q8_impl(o, proj, P, z_off, w, inv_s, q, s, n_rows, T, HV, D, eps, mode, amax, sy, stream);
}

int pb_gated_norm_q8_exchange(const float* o, const void* proj, long P, long z_off, const float* w, const float* inv_s,
                              int8_t* q, float* s, const int* n_rows, int T, int HV, int D, float eps, const pb_sync* sync,
                              void* stream) {
    tpx::Sync sy;
    int rc = to_sync(sync, &sy, false);
    if (rc) return rc;
    if (!sync) return PB_BAD_ARGUMENT;
    return gated_norm_q8_impl(o, proj, P, z_off, w, inv_s, q, s, n_rows, T, HV, D, eps, 3, nullptr, sy, stream);
}

int pb_head_quant(const float* h, const float* w, int8_t* q, float* s, const int* n_rows, int B, int HID, float eps,
                  void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!h || !w || !q || !s || !n_rows || B <= 0 || HID <= 0) return PB_BAD_ARGUMENT;
    if (HID % 32 || HID > 65536 || !aligned16(h) || !aligned16(w) || ((uintptr_t)q & 7)) return PB_UNSUPPORTED_SHAPE;
    const bool full = div_full();
    const int nvec = HID / 8;
    const int vpt = nvec <= 2048 ? 4 : 8;
    const int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
    if (vpt == 4) {
        if (full) quant::head_quant_kernel<4, true><<<B, threads, 0, st>>>(h, w, q, s, n_rows, HID, eps);
        else quant::head_quant_kernel<4, false><<<B, threads, 0, st>>>(h, w, q, s, n_rows, HID, eps);
    } else {
        if (full) quant::head_quant_kernel<8, true><<<B, threads, 0, st>>>(h, w, q, s, n_rows, HID, eps);
        else quant::head_quant_kernel<8, false><<<B, threads, 0, st>>>(h, w, q, s, n_rows, HID, eps);
    }
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

static int swiglu_q8_impl(const void* gu, const float* inv_s, int8_t* q, float* s, const int* n_rows, int T, int FF, int mode,
                          float* amax, const tpx::Sync& sy, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!gu || !q || !s || !n_rows || T <= 0 || FF <= 0) return PB_BAD_ARGUMENT;
    if (mode < 0 || mode > 3 || ((mode == 1 || mode == 2) && !amax) || (mode == 3 && sy.world < 2)) return PB_BAD_ARGUMENT;
    if (FF % 8 || FF > 32768 || !aligned16(gu) || ((uintptr_t)q & 7)) return PB_UNSUPPORTED_SHAPE;
    const bool full = div_full();
    if (T >= kPipeMinRows && mode != 3) {
        quant::PipeArgs pa{gu, 2l * FF, inv_s, q, s, n_rows, amax, T, FF, mode, 4 * FF, 0};
        const int rc = launch_pipe<quant::PIPE_SWIGLU, true>(full, pa, st);
        if (rc != PB_UNSUPPORTED_SHAPE) return rc;
    }
    const int nvec = FF / 8;
    const int threads = ((nvec + 3) / 4 + 31) / 32 * 32;          // 4 vectors of 8 outputs per thread
    const __nv_bfloat16* g = (const __nv_bfloat16*)gu;
    if (full) PB_CUDA(launch_dep(quant::swiglu_q8_kernel<4, true>, dim3(T), dim3(threads), 0, st, g, inv_s, q, s, n_rows, FF, mode, amax, sy));
    else PB_CUDA(launch_dep(quant::swiglu_q8_kernel<4, false>, dim3(T), dim3(threads), 0, st, g, inv_s, q, s, n_rows, FF, mode, amax, sy));
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_swiglu_q8(const void* gu, const float* inv_s, int8_t* q, float* s, const int* n_rows, int T, int FF, int mode,
                 float* amax, void* stream) {
    if (mode == 3) return PB_BAD_ARGUMENT;
    tpx::Sync sy;
    to_sync(nullptr, &sy, false);
    return swiglu_q8_impl(gu, inv_s, q, s, n_rows, T, FF, mode, amax, sy, stream);
}

int pb_swiglu_q8_exchange(const void* gu, const float* inv_s, int8_t* q, float* s, const int* n_rows, int T, int FF,
                          const pb_sync* sync, void* stream) {
    tpx::Sync sy;
    int rc = to_sync(sync, &sy, false);
    if (rc) return rc;
    if (!sync) return PB_BAD_ARGUMENT;
    return swiglu_q8_impl(gu, inv_s, q, s, n_rows, T, FF, 3, nullptr, sy, stream);
}

int pb_fold_sync(float* h, long ldh, const int32_t* slots, long slot_stride, int S, const float* a_s, const float* w_s,
                 const int* n_rows, int rows, int N, const pb_sync* sync, void* stream) {
    if (!h || !slots || !a_s || !w_s || !n_rows || rows <= 0 || N <= 0 || S < 1 || ldh < N || !sync) return PB_BAD_ARGUMENT;
    if (N % 4) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(h) || !aligned16(slots) || !aligned16(w_s) || (ldh % 4) || (slot_stride % 4)) return PB_BAD_ARGUMENT;
    tpx::Sync sy;
    // no `others`: a handshake only - every slot is already in this rank's memory (the other ranks' kernels stored
    // them there), and the flags say that those kernels have ended
    int rc = to_sync(sync, &sy, sync->others[0] != nullptr);
    if (rc) return rc;
    dim3 grid((N / 4 + 255) / 256, rows);
    cudaStream_t st = (cudaStream_t)stream;
    if ((long)grid.x * grid.y > 256) {
        // many blocks: one small kernel does the handshake (a system-scope wait and fence in each of thousands of blocks
        // measured slower than NCCL's barrier), the fold after it finds the flags already checked
        tpx::handshake_kernel<<<1, 32, 0, st>>>(sy);
        PB_CUDA(cudaGetLastError());
        if (!sync->others[0]) {
            quant::fold_kernel<<<grid, 256, 0, st>>>(h, ldh, slots, slot_stride, S, a_s, w_s, n_rows, N);
            PB_CUDA(cudaGetLastError());
            return PB_OK;
        }
        for (int r = 0; r < tpx::MAX_RANKS; ++r) sy.bufs[r] = nullptr;
    }
    quant::fold_sync_kernel<<<grid, 256, 0, st>>>(h, ldh, slots, slot_stride, S, a_s, w_s, n_rows, N, sy);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_handshake(const pb_sync* sync, void* stream) {
    if (!sync) return PB_BAD_ARGUMENT;
    tpx::Sync sy;
    int rc = to_sync(sync, &sy, false);
    if (rc) return rc;
    if (sy.world < 2) return PB_OK;
    tpx::handshake_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(sy);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_push(const void* src, void* const* dsts, int n, long nbytes, void* stream) {
    if (!src || !dsts || n < 0 || n > tpx::MAX_RANKS - 1 || nbytes < 0 || nbytes % 16 || !aligned16(src)) return PB_BAD_ARGUMENT;
    if (n == 0 || nbytes == 0) return PB_OK;
    tpx::PushArgs a{};
    a.src = (const uint4*)src;
    a.n16 = nbytes / 16;
    a.n = n;
    for (int d = 0; d < n; ++d) {
        if (!dsts[d] || !aligned16(dsts[d])) return PB_BAD_ARGUMENT;
        a.dst[d] = (uint4*)dsts[d];
    }
    long blocks = (a.n16 + 255) / 256;
    const long cap = 4l * sm_count();
    if (blocks > cap) blocks = cap;
    tpx::push_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_quant_g(const void* x, int x_fp32, int8_t* q, float* a, int8_t* xs, const int* n_rows, int T, int Ma, int K,
               void* stream) {
    if (!x || !q || !a || !xs || !n_rows || T <= 0 || K <= 0 || Ma < T) return PB_BAD_ARGUMENT;
    if (K % 256 || !aligned16(x) || ((uintptr_t)q & 7)) return PB_UNSUPPORTED_SHAPE;
    dim3 grid((K / 256 + 7) / 8, T);
    if (x_fp32) quant::quant_g_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(x, q, a, xs, n_rows, Ma, K);
    else quant::quant_g_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(x, q, a, xs, n_rows, Ma, K);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_swiglu_g(const void* gu, int8_t* q, float* a, int8_t* xs, const int* n_rows, int T, int Ma, int FF, void* stream) {
    if (!gu || !q || !a || !xs || !n_rows || T <= 0 || FF <= 0 || Ma < T) return PB_BAD_ARGUMENT;
    if (FF % 256 || !aligned16(gu) || ((uintptr_t)q & 7)) return PB_UNSUPPORTED_SHAPE;
    dim3 grid((FF / 256 + 7) / 8, T);
    quant::swiglu_g_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, q, a, xs, n_rows, Ma, FF);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_norm_g(const float* h, const float* w, int8_t* q, float* a, int8_t* xs, const int* n_rows, int T, int Ma, int HID,
              float eps, void* stream) {
    if (!h || !w || !q || !a || !xs || !n_rows || T <= 0 || HID <= 0 || Ma < T) return PB_BAD_ARGUMENT;
    if (HID % 256 || HID > 8192 || !aligned16(h) || !aligned16(w) || ((uintptr_t)q & 7)) return PB_UNSUPPORTED_SHAPE;
    quant::norm_g_kernel<<<T, HID / 8, 0, (cudaStream_t)stream>>>(h, w, q, a, xs, n_rows, Ma, HID, eps);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_gated_norm_g(const float* o, const void* proj, long P, long z_off, const float* w, int8_t* q, float* a, int8_t* xs,
                    const int* n_rows, int T, int Ma, int HV, int D, float eps, void* stream) {
    if (!o || !proj || !w || !q || !a || !xs || !n_rows || T <= 0 || HV <= 0 || Ma < T) return PB_BAD_ARGUMENT;
    if ((D != 64 && D != 128 && D != 256) || (HV * D) % 256) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(o) || !aligned16(w) || !aligned16(proj) || (P * 2) % 16 || (z_off * 2) % 16 || ((uintptr_t)q & 7))
        return PB_BAD_ARGUMENT;
    dim3 grid((HV * D / 256 + 7) / 8, T);
    quant::gated_norm_g_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(o, (const __nv_bfloat16*)proj, P, z_off, w, q, a, xs,
                                                                       n_rows, Ma, HV, D, eps);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

long pb_w4a8_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0) return 0;
    return (long)((N + 127) / 128) * (K / 256) * 16 * 128 * 4;
}

int pb_w4a8_counters(int M, int N) { return (M <= 0 || M > 16 || N <= 0) ? 0 : (N + 63) / 64; }

int pb_w4a8_gemm(const int8_t* xq, const float* a, const int8_t* xs, int Ma, int kind, const void* wq,
                 const void* wsc, const void* wmn, const float* wd, const float* wdm, void* out, long ldo,
                 const int* n_rows, int M, int N, int K, int epi, int split, void* workspace, long workspace_bytes,
                 int* counters, int n_counters, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!xq || !a || !wq || !wsc || !wd || !out || !n_rows || M <= 0 || N <= 0 || K <= 0 || Ma < M) return PB_BAD_ARGUMENT;
    if (kind != 0 && kind != 1) return PB_BAD_ARGUMENT;
    if (kind == 0 && (!xs || !wmn || !wdm)) return PB_BAD_ARGUMENT;
    if (epi != PB_EPI_BF16 && epi != PB_EPI_ADD) return PB_BAD_ARGUMENT;
    if (K % 256 || N % 4 || ldo < N) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(xq) || !aligned16(wq) || !aligned16(wsc) || !aligned16(wd) || (kind == 0 && (!aligned16(xs) ||
        !aligned16(wmn) || !aligned16(wdm)))) return PB_BAD_ARGUMENT;
    // one or two rows, or up to eight against a matrix of few rows: the CUDA-core kernel (measured: from three rows on
    // a 34816-row matrix the tensor-core kernel below is level or ahead)
    if ((M <= 2 || (M <= 8 && (N + 7) / 8 < 8 * sm_count())) && !w4a8_tile_only() && !w4a8_no_gemv()) {
        w4a8::GemvArgs g{xq, a, xs, (const uint8_t*)wq, (const uint8_t*)wsc, (const uint8_t*)wmn, wd, wdm, out, ldo, n_rows, M, N,
                         K, Ma, epi};
        if (M == 1) return launch_w4a8_gemv<1>(kind, g, st);
        if (M == 2) return launch_w4a8_gemv<2>(kind, g, st);
        if (M <= 4) return launch_w4a8_gemv<4>(kind, g, st);
        return launch_w4a8_gemv<8>(kind, g, st);
    }
    if (M <= 32 && !w4a8_tile_only()) {                            // measured: the many-rows kernel is faster from 64 rows
        if (kind == 0) {
            // K split (exact): Q4_K through tensor memory, one tile of 16 rows
            if (split > 1 && M <= 16 && !w4a8_few_staged()) {
                if (!workspace || !counters) return PB_BAD_ARGUMENT;
                if (workspace_bytes < pb_w4a8_workspace_bytes(M, N, K) || n_counters < pb_w4a8_counters(M, N)) return PB_TOO_LARGE;
            } else {
                split = 1;
            }
            return launch_w4a8_few<w4a8::KIND_Q4K>(xq, a, xs, Ma, wq, wsc, wmn, wd, wdm, out, ldo, n_rows, M, N, K, epi, st,
                                                   split, (float*)workspace, counters);
        }
        if (split > 1 && M <= 16) {
            if (!workspace || !counters) return PB_BAD_ARGUMENT;
            if (workspace_bytes < pb_w4a8_workspace_bytes(M, N, K) || n_counters < pb_w4a8_counters(M, N)) return PB_TOO_LARGE;
        } else {
            split = 1;
        }
        return launch_w4a8_few<w4a8::KIND_Q6K>(xq, a, xs, Ma, wq, wsc, wmn, wd, wdm, out, ldo, n_rows, M, N, K, epi, st,
                                               split, (float*)workspace, counters);
    }
    if (kind == 0)
        return launch_w4a8<w4a8::KIND_Q4K>(xq, a, xs, Ma, wq, wsc, wmn, wd, wdm, out, ldo, n_rows, M, N, K, epi, st);
    return launch_w4a8<w4a8::KIND_Q6K>(xq, a, xs, Ma, wq, wsc, wmn, wd, wdm, out, ldo, n_rows, M, N, K, epi, st);
}

long pb_w8a8_static_scratch_bytes(void) { return PB_STATIC_WS_BYTES; }

int pb_w8a8_gemm_static(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, void* out, long ldo,
                        const int* n_rows, int M, int N, int K, int epi, int split, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!a || !w || !out || !n_rows || !a_s || !w_s || M <= 0 || N <= 0 || K <= 0 || split < 1) return PB_BAD_ARGUMENT;
    if (epi != PB_EPI_BF16 && epi != PB_EPI_ADD) return PB_BAD_ARGUMENT;
    if (!aligned16(a) || !aligned16(w) || ldo < N) return PB_BAD_ARGUMENT;
    if (K % 16 || M > 64) return PB_UNSUPPORTED_SHAPE;
    const int KB = (K + 127) / 128;
    if (split > KB) split = KB;
    const int kbs = (KB + split - 1) / split;
    split = (KB + kbs - 1) / kbs;
    // sizes beyond the static array are refused, never truncated
    if (split > 1 && (pb_w8a8_workspace_bytes(M, N, split) > PB_STATIC_WS_BYTES || pb_w8a8_counters(M, N) > PB_STATIC_COUNTERS))
        return PB_TOO_LARGE;
    void* scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc) return rc;
    int32_t* ws = (int32_t*)scratch;
    int* counters = (int*)((unsigned char*)scratch + PB_STATIC_WS_BYTES);
    w8a8::SwapArgs p{a_s, w_s, out, ldo, 0, ws, counters, n_rows, M, N, K, kbs, epi,
                     split == 1 ? w8a8::MODE_DIRECT : w8a8::MODE_WS, 0, 0};
    if (split > 1) {
        // the counters must start at zero; the array keeps whatever an earlier call (or an aborted one) left
        PB_CUDA(cudaMemsetAsync(counters, 0, (size_t)pb_w8a8_counters(M, N) * sizeof(int), st));
    }
    return launch_swap_nb<false>(pick_nb(M), a, a_s, w, w_s, p, split, st);
}

long pb_mxfp4_sf_bytes(int rows, int K) {
    if (rows <= 0 || K <= 0 || K % 128) return 0;
    return (long)((rows + 127) / 128) * (K / 128) * 512;
}

int pb_mxfp4_prepare_sf(const void* s, void* dst, int rows, int K, void* stream) {
    if (!s || !dst || rows <= 0 || K <= 0) return PB_BAD_ARGUMENT;
    if (K % 128 || ((uintptr_t)dst & 15)) return PB_UNSUPPORTED_SHAPE;
    const long threads = (long)((rows + 127) / 128) * (K / 128) * 128;
    mxfp4::sf_tile_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)s, (uint8_t*)dst, rows, K);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_mxfp4_quant(const void* x, int x_fp32, const float* inv, void* q, void* s, int n, int K, void* stream) {
    if (!x || !q || !s || n <= 0 || K <= 0) return PB_BAD_ARGUMENT;
    if (K % 32 || !aligned16(x) || ((uintptr_t)q & 3)) return PB_UNSUPPORTED_SHAPE;
    dim3 grid((K / 8 + 255) / 256, n);
    if (x_fp32) mxfp4::mxfp4_quant_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(x, inv, (uint8_t*)q, (uint8_t*)s, n, K);
    else mxfp4::mxfp4_quant_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(x, inv, (uint8_t*)q, (uint8_t*)s, n, K);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_mxfp4_gemm(const void* aq, const void* a_sf, const void* bq, const void* b_sf, void* out, long ldo, int M,
                  int N, int K, int epi, void* stream) {
    return pb_mxfp4_gemm_split(aq, a_sf, bq, b_sf, out, ldo, M, N, K, epi, 1, nullptr, 0, nullptr, 0, stream);
}

long pb_mxfp4_workspace_bytes(int M, int N, int split) {
    if (M <= 0 || N <= 0 || split <= 1) return 0;
    return (long)((M + 127) / 128) * ((N + 127) / 128) * split * 128 * 128 * 4;
}

int pb_mxfp4_counters(int M, int N) {
    if (M <= 0 || N <= 0) return 0;
    return ((M + 127) / 128) * ((N + 127) / 128);
}

int pb_mxfp4_gemm_split(const void* aq, const void* a_sf, const void* bq, const void* b_sf, void* out, long ldo, int M,
                        int N, int K, int epi, int split, void* workspace, long workspace_bytes, int* counters,
                        int n_counters, void* stream) {
    if (!aq || !a_sf || !bq || !b_sf || !out || M <= 0 || N <= 0 || K <= 0 || ldo < N) return PB_BAD_ARGUMENT;
    if (epi != 0 && epi != 1) return PB_BAD_ARGUMENT;
    if (K % 256) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(aq) || !aligned16(bq) || !aligned16(a_sf) || !aligned16(b_sf)) return PB_BAD_ARGUMENT;
    if (split < 1) return PB_BAD_ARGUMENT;
    const int KB = K / 256;
    if (split > KB) split = KB;
    int kbs = (KB + split - 1) / split;
    split = (KB + kbs - 1) / kbs;                                  // every slice non-empty
    if (split > 1) {
        if (!workspace || !counters) return PB_BAD_ARGUMENT;
        if (workspace_bytes < pb_mxfp4_workspace_bytes(M, N, split) || n_counters < pb_mxfp4_counters(M, N))
            return PB_TOO_LARGE;
    }
    CUtensorMap ta, tb;
    int rc;
    if ((rc = tensor_map(&ta, aq, K / 2, M, K / 2, 128, 128, 0))) return rc;
    if ((rc = tensor_map(&tb, bq, K / 2, N, K / 2, 128, 128, 0))) return rc;
    mxfp4::GemmArgs p{(const uint8_t*)a_sf, (const uint8_t*)b_sf, out, ldo, M, N, K, epi, split, kbs, (float*)workspace, counters};
    // 128 x 256 tiles when there are enough of them to fill the SMs (the same K order either way: one accumulator
    // over all of K, so a row's bits do not depend on the choice)
    const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    if (N > 128 && tiles256 >= sm_count() && !mxfp4_narrow_only() && split == 1) {
        CUtensorMap tb2;
        if ((rc = tensor_map(&tb2, bq, K / 2, N, K / 2, 128, 256, 0))) return rc;
        if ((rc = set_smem(mxfp4::mxfp4_gemm256_kernel, mxfp4::SMEM2))) return rc;
        const int grid2 = tiles256 < sm_count() ? (int)tiles256 : sm_count();
        // the epilogue hands 32 x 64-byte boxes to the copy engine when out can be described by a tensor map
        CUtensorMap tout = ta;
        int by_engine = 0;
        const int esz = epi == 0 ? 2 : 4;
        if (((uintptr_t)out & 15) == 0 && (ldo * esz) % 16 == 0) {
            if (epi == 0) rc = tensor_map(&tout, out, (uint64_t)N / 2, M, (uint64_t)ldo * 2, 16, 32, 3);   // bf16 pairs as words
            else rc = tensor_map(&tout, out, N, M, (uint64_t)ldo * 4, 16, 32, 1);
            if (rc) return rc;
            by_engine = (epi == 1 || N % 2 == 0) ? 1 : 0;
        }
        mxfp4::mxfp4_gemm256_kernel<<<grid2, mxfp4::THREADS2, mxfp4::SMEM2, (cudaStream_t)stream>>>(ta, tb2, tout, p, by_engine);
        PB_CUDA(cudaGetLastError());
        return PB_OK;
    }
    if ((rc = set_smem(mxfp4::mxfp4_gemm_kernel, mxfp4::SMEM))) return rc;
    const int tiles = ((M + 127) / 128) * ((N + 127) / 128) * split;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    mxfp4::mxfp4_gemm_kernel<<<grid, 192, mxfp4::SMEM, (cudaStream_t)stream>>>(ta, tb, p);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_mxfp4_gemv(const void* aq, const void* a_s, const void* bq, const void* b_s, void* out, long ldo, int M, int N,
                  int K, int epi, void* stream) {
    if (!aq || !a_s || !bq || !b_s || !out || M <= 0 || N <= 0 || K <= 0 || ldo < N) return PB_BAD_ARGUMENT;
    if (epi != 0 && epi != 1) return PB_BAD_ARGUMENT;
    if (M > 4 || K % 256) return PB_UNSUPPORTED_SHAPE;
    if (!aligned16(aq) || !aligned16(bq)) return PB_BAD_ARGUMENT;
    mxfp4::GemvArgs p{(const uint8_t*)aq, (const uint8_t*)a_s, (const uint8_t*)bq, (const uint8_t*)b_s, out, ldo, M, N, K, epi};
    cudaStream_t st = (cudaStream_t)stream;
    if (M == 1) return launch_mxfp4_gemv<1>(p, st);
    if (M == 2) return launch_mxfp4_gemv<2>(p, st);
    return launch_mxfp4_gemv<4>(p, st);
}

int pb_int8_peak_probe(int iters, int pattern, int mma_n, unsigned long long* cycles, void* stream) {
    if (iters <= 0 || mma_n < 16 || mma_n > 256 || mma_n % 16) return PB_BAD_ARGUMENT;
    const int smem = (128 + 256) * 128 + 1024;
    int rc = set_smem(w8a8::int8_peak_kernel, smem);
    if (rc) return rc;
    w8a8::int8_peak_kernel<<<sm_count(), 128, smem, (cudaStream_t)stream>>>(iters, pattern, mma_n, cycles);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_l2_prefetch(const void* const* ptrs, const long* nbytes, int n, int ctas, void* stream) {
    if (!ptrs || !nbytes || n < 1 || n > 8 || ctas < 1 || ctas > 1024) return PB_BAD_ARGUMENT;
    PrefetchRanges r{};
    r.n = n;
    for (int i = 0; i < n; ++i) {
        if (!ptrs[i] || nbytes[i] < 0 || !aligned16(ptrs[i])) return PB_BAD_ARGUMENT;
        r.ptr[i] = (const char*)ptrs[i];
        r.bytes[i] = nbytes[i] & ~15l;                             // whole 16-byte units (the tail is at most 15 bytes)
    }
    l2_prefetch_kernel<<<ctas, 128, 0, (cudaStream_t)stream>>>(r);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

int pb_mxf4_peak_probe(int iters, int pattern, unsigned long long* cycles, void* stream) {
    if (iters <= 0) return PB_BAD_ARGUMENT;
    const int smem = (128 + 256) * 128 + 512 + 1024;
    int rc = set_smem(mxfp4::mxf4_peak_kernel, smem);
    if (rc) return rc;
    mxfp4::mxf4_peak_kernel<<<sm_count(), 128, smem, (cudaStream_t)stream>>>(iters, pattern, cycles);
    PB_CUDA(cudaGetLastError());
    return PB_OK;
}

}  // extern "C"
