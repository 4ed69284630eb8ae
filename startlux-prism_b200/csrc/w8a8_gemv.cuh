// W8A8 (one scale per row, gk == K) for one to eight activation rows on the CUDA cores: at these row counts the
// projection is a stream of int8 weights from HBM and the tensor core's 128-row tile is 94-99 % padding.  The integer
// dot products are exact in any order (dp4a, int32), the epilogue is the tile kernels' (float(acc) * a_s) * w_s with
// the same roundings: bit-identical to them.
//
// Geometry of the W4A8 CUDA-core kernel (w4a8_gemv.cuh): eight lanes share a weight row, a lane takes 32 of every 256
// inputs (two 16-byte loads), two rows per lane group, eight rows per warp; weights are loaded for PD steps of 256
// inputs at a time, all requests before the first use; the lanes' int32 sums are added once, at the end.  Matrices of
// few rows: KW warps of a CTA take every KW-th step of the same rows and their sums meet in shared memory (exact).
#pragma once
#include "common.cuh"
#include "w4a8_gemv.cuh"

namespace w8a8 {

struct GemvArgs {
    const int8_t* a;        // int8 [M, K]
    const float* a_s;       // fp32 [M]
    const int8_t* w;        // int8 [N, K]
    const float* w_s;       // fp32 [N]
    void* out;
    long ldo;
    const int* n_rows;
    int M, N, K, epi;       // epi 0: bf16 store, 1: fp32 add
};

constexpr int GV_R = 2, GV_PD = 4;

template <int MR, bool SPLIT>
__global__ void __launch_bounds__(SPLIT ? 128 : 32)
w8a8_gemv_kernel(const GemvArgs p) {
    constexpr int R = GV_R, PD = GV_PD, NV = R * MR;
    extern __shared__ int gv8_part[];                              // SPLIT: [warp][4 * NV] partial sums
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int KW = SPLIT ? (int)(blockDim.x >> 5) : 1;
    const int g = lane & 7;
    const long n0 = ((long)blockIdx.x * 4 + (lane >> 3)) * R;
    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    if (live <= 0) return;
    const int steps = p.K >> 8;
    const int8_t* wrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const long nn = n0 + r < p.N ? n0 + r : p.N - 1;           // rows past N read the last row and store nothing
        wrow[r] = p.w + nn * p.K + g * 32;
    }
    int acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0;
    uint4 ring[PD][R][2];
    for (int b0 = warp; b0 < steps; b0 += PD * KW) {
#pragma unroll
        for (int j = 0; j < PD; ++j)
            if (b0 + j * KW < steps) {
                const long b = b0 + j * KW;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    ring[j][r][0] = w4a8::ldg_stream(wrow[r] + b * 256);
                    ring[j][r][1] = w4a8::ldg_stream(wrow[r] + b * 256 + 16);
                }
            }
#pragma unroll
        for (int j = 0; j < PD; ++j) {
            const int b = b0 + j * KW;
            if (b < steps) {
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const int mm = m < p.M ? m : p.M - 1;
                    const uint4* xp = (const uint4*)(p.a + (long)mm * p.K + b * 256 + g * 32);
                    const uint4 x0 = __ldg(xp), x1 = __ldg(xp + 1);
#pragma unroll
                    for (int r = 0; r < R; ++r)
                        acc[r * MR + m] += w4a8::dot32(ring[j][r][0], ring[j][r][1], x0, x1);
                }
            }
        }
    }
    // the eight lanes of a row (exact): every (row, activation row) pair's sum ends in one lane
    w4a8::reduce8<NV>(acc, lane);
    constexpr int NF = NV >= 8 ? NV / 8 : 1;                       // pairs a lane ends up with
    const int base = w4a8::reduce8_index<NV>(lane);
    const bool owner = w4a8::reduce8_owner<NV>(lane);
    if (SPLIT) {
        if (owner) {
#pragma unroll
            for (int i = 0; i < NF; ++i) {
                const int v = base + i;
                gv8_part[warp * (4 * NV) + ((lane >> 3) * R + v / MR) * MR + v % MR] = acc[i];
            }
        }
        __syncthreads();
        const int t = threadIdx.x;
        if (t >= 4 * NV) return;
        int tot = gv8_part[t];
        for (int w = 1; w < KW; ++w) tot += gv8_part[w * (4 * NV) + t];
        const long n = (long)blockIdx.x * 4 * R + t / MR;
        const int m = t % MR;
        if (n < p.N && m < live) {
            const float v = scale2(tot, p.a_s[m], p.w_s[n]);
            if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(v);
            else {
                float* o = (float*)p.out + (long)m * p.ldo + n;
                *o = __fadd_rn(*o, v);
            }
        }
    } else if (owner) {
#pragma unroll
        for (int i = 0; i < NF; ++i) {
            const int v = base + i, m = v % MR;
            const long n = n0 + v / MR;
            if (n < p.N && m < live) {
                const float f = scale2(acc[i], p.a_s[m], p.w_s[n]);
                if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(f);
                else {
                    float* o = (float*)p.out + (long)m * p.ldo + n;
                    *o = __fadd_rn(*o, f);
                }
            }
        }
    }
}

}  // namespace w8a8
