// MXFP4 for one to four activation rows, on the CUDA cores.  The products of two e2m1 values are small integers (the
// grid doubled is 0, 1, 2, 3, 4, 6, 8, 12), so a 32-input block's dot product is an exact integer (dp4a on the doubled
// values, a quarter of it is the true sum) and only the block scale 2^(ea + ew - 254) and the sum over the blocks are
// floating point: one fp32 multiply-add per block, each lane over its own blocks in K order, the eight lanes of a row
// added at the end (a fixed order: deterministic).  The result differs from the tensor-core kernels' only in the
// order of the fp32 additions.
//
// Geometry as in the W4A8 CUDA-core kernel: eight lanes share a weight row, a lane takes one 32-input block (16 bytes)
// of every 256 inputs, two rows per lane group, eight rows per warp; weights and their scale bytes are loaded for PD
// steps at a time, all requests before the first use.  Matrices of few rows: KW warps of a CTA take every KW-th step of
// the same rows and their partial sums are added in warp order through shared memory.
// Code -> doubled magnitude by byte permute from an 8-entry table (two registers), sign masks by the permute's sign
// replication, the combined sign of a product applied by splitting the weight magnitudes into the products that count
// positive and those that count negative (two dp4a per four inputs); a negative zero (code 8) is a zero either way.
#pragma once
#include "common.cuh"

namespace mxfp4 {

struct GemvArgs {
    const uint8_t* aq;      // activation codes [M, K/2]
    const uint8_t* as;      // activation scales [M, K/32] (row-major, not the tiled order)
    const uint8_t* wq;      // weight codes [N, K/2]
    const uint8_t* ws;      // weight scales [N, K/32]
    void* out;
    long ldo;
    int M, N, K, epi;
};

constexpr int GV_R = 2, GV_PD = 4;

__device__ __forceinline__ uint4 gv_ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t gv_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;                                                      // selector bit 3 of a nibble: replicate the byte's top bit
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// eight codes of a word -> doubled magnitudes (two words of four bytes, element order) and sign masks (0xff / 0x00)
__device__ __forceinline__ void gv_decode(uint32_t w, uint32_t& m0, uint32_t& m1, uint32_t& s0, uint32_t& s1) {
    m0 = gv_prmt(0x03020100u, 0x0C080604u, w & 0x7777u);
    m1 = gv_prmt(0x03020100u, 0x0C080604u, (w >> 16) & 0x7777u);
    const uint32_t e = w << 4;                                       // even codes' sign bits at their bytes' top
    s0 = gv_prmt(e, w, 0xD9C8u);
    s1 = gv_prmt(e, w, 0xFBEAu);
}

// 2^(ea + ew - 254) / 4 as a float (the dot product is of doubled values); exact for every exponent a float holds
__device__ __forceinline__ float gv_scale(int ea, int ew) {
    const int e = ea + ew - 256 + 127;                               // biased exponent
    if (e >= 1 && e <= 254) return __uint_as_float((uint32_t)e << 23);
    return ldexpf(1.0f, e - 127);
}

template <int MR, bool SPLIT>
__global__ void __launch_bounds__(SPLIT ? 128 : 32)
mxfp4_gemv_kernel(const GemvArgs p) {
    constexpr int R = GV_R, PD = GV_PD;
    extern __shared__ float gv_part[];                             // SPLIT: [warp][4 * R * MR] partial sums
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int KW = SPLIT ? (int)(blockDim.x >> 5) : 1;
    const int g = lane & 7;
    const long n0 = ((long)blockIdx.x * 4 + (lane >> 3)) * R;
    const int steps = p.K >> 8, SB = p.K >> 5;                     // 256-input steps; scale bytes per row
    const uint8_t* wrow[R];
    const uint8_t* srow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const long nn = n0 + r < p.N ? n0 + r : p.N - 1;           // rows past N read the last row and store nothing
        wrow[r] = p.wq + nn * (p.K >> 1) + g * 16;
        srow[r] = p.ws + nn * SB + g;
    }
    float y[R][MR];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MR; ++m) y[r][m] = 0.0f;
    uint4 ring[PD][R];
    int sc[PD][R];
    for (int b0 = warp; b0 < steps; b0 += PD * KW) {
#pragma unroll
        for (int j = 0; j < PD; ++j)
            if (b0 + j * KW < steps) {
                const long b = b0 + j * KW;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    ring[j][r] = gv_ldg_stream(wrow[r] + b * 128);
                    sc[j][r] = srow[r][b * 8];
                }
            }
#pragma unroll
        for (int j = 0; j < PD; ++j) {
            const int b = b0 + j * KW;
            if (b < steps) {
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const int mm = m < p.M ? m : p.M - 1;
                    const uint4 x = __ldg((const uint4*)(p.aq + (long)mm * (p.K >> 1) + b * 128 + g * 16));
                    const int ea = p.as[(long)mm * SB + b * 8 + g];
                    uint32_t xm[8], xs[8];
                    gv_decode(x.x, xm[0], xm[1], xs[0], xs[1]);
                    gv_decode(x.y, xm[2], xm[3], xs[2], xs[3]);
                    gv_decode(x.z, xm[4], xm[5], xs[4], xs[5]);
                    gv_decode(x.w, xm[6], xm[7], xs[6], xs[7]);
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t ww[4] = {ring[j][r].x, ring[j][r].y, ring[j][r].z, ring[j][r].w};
                        unsigned pos = 0, neg = 0;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t wm0, wm1, ws0, ws1;
                            gv_decode(ww[q], wm0, wm1, ws0, ws1);
                            const uint32_t n0m = ws0 ^ xs[2 * q], n1m = ws1 ^ xs[2 * q + 1];   // products that count negative
                            pos = __dp4a(wm0 & ~n0m, xm[2 * q], pos);
                            neg = __dp4a(wm0 & n0m, xm[2 * q], neg);
                            pos = __dp4a(wm1 & ~n1m, xm[2 * q + 1], pos);
                            neg = __dp4a(wm1 & n1m, xm[2 * q + 1], neg);
                        }
                        y[r][m] = __fmaf_rn(__int2float_rn((int)pos - (int)neg), gv_scale(ea, sc[j][r]), y[r][m]);
                    }
                }
            }
        }
    }
    // the eight lanes of a row: a fixed butterfly
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MR; ++m)
#pragma unroll
            for (int o = 4; o >= 1; o >>= 1) y[r][m] = __fadd_rn(y[r][m], __shfl_xor_sync(0xffffffffu, y[r][m], o));
    if (SPLIT) {
        if (g == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int m = 0; m < MR; ++m) gv_part[warp * (4 * R * MR) + ((lane >> 3) * R + r) * MR + m] = y[r][m];
        }
        __syncthreads();
        const int t = threadIdx.x;
        if (t >= 4 * R * MR) return;
        float tot = gv_part[t];
        for (int w = 1; w < KW; ++w) tot = __fadd_rn(tot, gv_part[w * (4 * R * MR) + t]);
        const long n = (long)blockIdx.x * 4 * R + t / MR;
        const int m = t % MR;
        if (n < p.N && m < p.M) {
            if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(tot);
            else {
                float* o = (float*)p.out + (long)m * p.ldo + n;
                *o = __fadd_rn(*o, tot);
            }
        }
    } else if (g == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                const long n = n0 + r;
                if (n < p.N && m < p.M) {
                    if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(y[r][m]);
                    else {
                        float* o = (float*)p.out + (long)m * p.ldo + n;
                        *o = __fadd_rn(*o, y[r][m]);
                    }
                }
            }
    }
}

}  // namespace mxfp4
