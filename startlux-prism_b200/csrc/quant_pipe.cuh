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

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&v)[8]) {
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
    v[4] = __uint_as_float(u.z << 16); v[5] = __uint_as_float(u.z & 0xffff0000u);
    v[6] = __uint_as_float(u.w << 16); v[7] = __uint_as_float(u.w & 0xffff0000u);
}

// max |x| over 8 packed bf16 values, exact (a maximum of bf16 values is one of them): two values per instruction
__device__ __forceinline__ __nv_bfloat162 absmax_bf16x8(const uint4& u, __nv_bfloat162 m) {
    m = __hmax2(m, __habs2(*(const __nv_bfloat162*)&u.x));
    m = __hmax2(m, __habs2(*(const __nv_bfloat162*)&u.y));
    m = __hmax2(m, __habs2(*(const __nv_bfloat162*)&u.z));
    m = __hmax2(m, __habs2(*(const __nv_bfloat162*)&u.w));
    return m;
}

// The block size is chosen at launch so that blockDim.x * VPT just covers the row's vectors (a fixed size left up to
// a quarter of the threads without a vector); MAXT bounds it for the register allocation.
template <int KIND, int VPT, bool BF16, bool FULL, int MAXT>
__global__ void __launch_bounds__(MAXT, 1)
row_pipe_kernel(const PipeArgs p) {
    const int THREADS = blockDim.x;
    extern __shared__ uint8_t pipe_smem_raw[];
    const uint32_t smem = (smem_u32(pipe_smem_raw) + 127u) & ~127u;
    __shared__ uint64_t full[8];
    __shared__ float red[32];
    __shared__ int abort_flag;
    const int live = min(*p.n_rows, p.T);
    const int nvec = p.K >> 3;
    const int my_rows = live > (int)blockIdx.x ? (live - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    // a bf16 row without smoothing keeps its packed words in registers: the maximum is taken on packed pairs and the
    // values are widened only for the rounding
    constexpr bool PACKED = KIND == PIPE_ROWS && BF16;

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
                     : : "r"(smem + (uint32_t)(s * p.row_bytes)), "l"(src), "r"((uint32_t)p.row_bytes), "r"(bar)
                     : "memory");
    };
    if (threadIdx.x == 0)
        for (int i = 0; i < p.stages - 1 && i < my_rows; ++i) issue(i);

    const bool smooth = p.inv_s != nullptr;
    for (int i = 0; i < my_rows; ++i) {
        const long t = (long)blockIdx.x + (long)i * gridDim.x;
        const int s = i % p.stages;
        // the slot of row i + stages - 1 was read by every thread in iteration i - 1 (the block barriers below)
        if (threadIdx.x == 0 && i + p.stages - 1 < my_rows) issue(i + p.stages - 1);
        if (!mbar_wait(smem_u32(&full[s]), (uint32_t)((i / p.stages) & 1), &abort_flag, 0xF00 + s)) break;
        const uint32_t row = smem + (uint32_t)(s * p.row_bytes) + threadIdx.x * (BF16 ? 16u : 32u);
        float v[VPT][8];
        uint4 raw[PACKED ? VPT : 1];
        float amax = 0.0f;
        if (PACKED && !smooth) {
            __nv_bfloat162 m2 = __float2bfloat162_rn(0.0f);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (threadIdx.x + j * THREADS < nvec) {
                    raw[j] = lds128(row + j * THREADS * 16);
                    m2 = absmax_bf16x8(raw[j], m2);
                }
            }
            amax = fmaxf(__low2float(m2), __high2float(m2));
        } else {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int c = threadIdx.x + j * THREADS;
                if (c < nvec) {
                    if (KIND == PIPE_SWIGLU) {
                        float g[8], u[8];
                        unpack_bf16x8(lds128(row + j * THREADS * 16), g);
                        unpack_bf16x8(lds128(row + (uint32_t)p.K * 2 + j * THREADS * 16), u);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[j][e] = swiglu_fast(g[e], u[e]);
                    } else if (BF16) {
                        unpack_bf16x8(lds128(row + j * THREADS * 16), v[j]);
                    } else {
                        const uint4 a = lds128(row + j * THREADS * 32), b = lds128(row + j * THREADS * 32 + 16);
                        v[j][0] = __uint_as_float(a.x); v[j][1] = __uint_as_float(a.y);
                        v[j][2] = __uint_as_float(a.z); v[j][3] = __uint_as_float(a.w);
                        v[j][4] = __uint_as_float(b.x); v[j][5] = __uint_as_float(b.y);
                        v[j][6] = __uint_as_float(b.z); v[j][7] = __uint_as_float(b.w);
                    }
                    if (smooth) {
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
        }
        amax = block_max(amax, red);             // two block barriers: every thread is done with slot s after them
        if (p.mode == MODE_STORE_AMAX && threadIdx.x == 0) p.amax_io[t] = amax;
        if (p.mode == MODE_USE_AMAX) amax = fmaxf(p.amax_io[t], amax);
        const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
        const float rcp = __fdiv_rn(1.0f, scale);
        int8_t* qrow = p.q + t * p.K + threadIdx.x * 8;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            if (threadIdx.x + j * THREADS < nvec) {
                if (PACKED && !smooth) unpack_bf16x8(raw[j], v[j]);
                *(uint2*)(qrow + j * THREADS * 8) = quant8<FULL>(v[j], scale, rcp);
            }
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
