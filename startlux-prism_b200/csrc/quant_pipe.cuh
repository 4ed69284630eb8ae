// Row-pipelined activation quantizers: persistent CTAs stream whole input rows into a shared-memory ring with bulk
// asynchronous copies (cp.async.bulk, completion counted on an mbarrier), so the next rows are in flight while the
// current row is reduced and rounded.  Bytes in flight per SM no longer depend on how many threads are resident, which
// is what held the one-CTA-per-row kernels at about 40 % of the HBM rate.
//
//   PIPE_ROWS    x bf16 or fp32 [T, K] (row stride ldx) (* inv_s[k]) -> int8 [T, K] + one scale per row (rows_q8)
//   PIPE_SWIGLU  gu bf16 [T, 2 FF] -> silu(gate) * up (* inv_s) -> int8 [T, FF] + one scale per row (swiglu_q8)
// Same rounding contract as quant.cuh (IEEE division semantics through the reciprocal fast path of quant8).
#pragma once
#include "common.cuh"
#include "quant.cuh"

namespace quant {

constexpr int PIPE_ROWS = 0, PIPE_SWIGLU = 1;
constexpr int PIPE_THREADS = 256;

struct PipeArgs {
    const void* x;
    long ldx;              // elements between input rows
    const float* inv_s;
    int8_t* q;
    float* s;
    const int* n_rows;
    float* amax_io;
    int T, K, mode;        // K: output columns (FF for SwiGLU)
    int row_bytes;         // input bytes per row (2 FF bf16 for SwiGLU)
    int stages;
};

// silu(g) * u with the approximate full-range division (2 ulp): the reference's expression g / (1 + exp(-g)) * u
// (kernels/quant.py:256) as its Triton `/` evaluates it.
__device__ __forceinline__ float swiglu_fast(float g, float u) {
    return __fmul_rn(fdiv<true>(g, 1.0f + __expf(-g)), u);
}

template <int KIND, int VPT, bool BF16, bool FULL>
__global__ void __launch_bounds__(PIPE_THREADS, 1)
row_pipe_kernel(const PipeArgs p) {
    extern __shared__ uint8_t pipe_smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)pipe_smem_raw + 127) & ~(uintptr_t)127);
    __shared__ uint64_t full[8];
    __shared__ float red[32];
    __shared__ int abort_flag;
    const int live = min(*p.n_rows, p.T);
    const int nvec = p.K >> 3;
    const int my_rows = live > (int)blockIdx.x ? (live - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(&full[s]), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    auto issue = [&](int i) {                    // thread 0: bulk copy of this CTA's i-th row into slot i % stages
        const long t = (long)blockIdx.x + (long)i * gridDim.x;
        const int s = i % p.stages;
        const uint32_t bar = smem_u32(&full[s]);
        mbar_expect_tx(bar, (uint32_t)p.row_bytes);
        const uint8_t* src = (const uint8_t*)p.x + t * p.ldx * (BF16 ? 2 : 4);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     : : "r"(smem_u32(smem + (long)s * p.row_bytes)), "l"(src), "r"((uint32_t)p.row_bytes), "r"(bar)
                     : "memory");
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < p.stages - 1 && i < my_rows; ++i) issue(i);

    for (int i = 0; i < my_rows; ++i) {
        const long t = (long)blockIdx.x + (long)i * gridDim.x;
        const int s = i % p.stages;
        // the slot of row i + stages - 1 was read by every thread in iteration i - 1 (the block barriers below)
        if (threadIdx.x == 0 && i + p.stages - 1 < my_rows) issue(i + p.stages - 1);
        if (!mbar_wait(smem_u32(&full[s]), (uint32_t)((i / p.stages) & 1), &abort_flag, 0xF00 + s)) break;
        const uint8_t* row = smem + (long)s * p.row_bytes;
        float v[VPT][8];
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = threadIdx.x + j * PIPE_THREADS;
            if (c < nvec) {
                if (KIND == PIPE_SWIGLU) {
                    const uint4 g4 = *(const uint4*)(row + (long)c * 16);
                    const uint4 u4 = *(const uint4*)(row + (long)p.K * 2 + (long)c * 16);
                    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[j][2 * e] = swiglu_fast(__uint_as_float(gw[e] << 16), __uint_as_float(uw[e] << 16));
                        v[j][2 * e + 1] = swiglu_fast(__uint_as_float(gw[e] & 0xffff0000u),
                                                      __uint_as_float(uw[e] & 0xffff0000u));
                    }
                } else if (BF16) {
                    const uint4 u = *(const uint4*)(row + (long)c * 16);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[j][2 * e] = __uint_as_float(w[e] << 16);
                        v[j][2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                    }
                } else {
                    const float4 a = *(const float4*)(row + (long)c * 32), b = *(const float4*)(row + (long)c * 32 + 16);
                    v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
                    v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
                }
                if (p.inv_s) {
                    const float4 a = __ldg((const float4*)(p.inv_s + c * 8)), b = __ldg((const float4*)(p.inv_s + c * 8 + 4));
                    v[j][0] = __fmul_rn(v[j][0], a.x); v[j][1] = __fmul_rn(v[j][1], a.y);
                    v[j][2] = __fmul_rn(v[j][2], a.z); v[j][3] = __fmul_rn(v[j][3], a.w);
                    v[j][4] = __fmul_rn(v[j][4], b.x); v[j][5] = __fmul_rn(v[j][5], b.y);
                    v[j][6] = __fmul_rn(v[j][6], b.z); v[j][7] = __fmul_rn(v[j][7], b.w);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[j][e]));
            }
        }
        amax = block_max(amax, red);             // two block barriers: every thread is done with slot s after them
        if (p.mode == MODE_STORE_AMAX && threadIdx.x == 0) p.amax_io[t] = amax;
        if (p.mode == MODE_USE_AMAX) amax = fmaxf(p.amax_io[t], amax);
        const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
        const float rcp = __fdiv_rn(1.0f, scale);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int c = threadIdx.x + j * PIPE_THREADS;
            if (c < nvec) *(uint2*)(p.q + t * p.K + (long)c * 8) = quant8<FULL>(v[j], scale, rcp);
        }
        if (threadIdx.x == 0) p.s[t] = scale;
    }
    // armed copies of rows this CTA never reached (abort only) must land before the shared memory is released
    if (abort_flag && threadIdx.x == 0) {
        unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
    }
}

}  // namespace quant
