// W4A8 for one to four activation rows (the decode step's usual batch): no tensor core - at these row counts the MMA
// would be 3 % used and the hand-offs between its stages are what the time goes to - but integer dot products on the
// CUDA cores, straight from the packed weights in global memory.  Same arithmetic as the other W4A8 kernels
// (kernels/w4a8.py:14-24): exact integers inside a 256-input super-block, then per super-block, in order,
//   Q4_K  t = d * float(acc); t = fma(-dmin, float(mins), t); y = fma(a, t, y)
//   Q6_K  y = fma(a, d * float(acc), y)
//
// Eight lanes share a weight row's super-block, 32 inputs each, and take R = 2 rows at a time, so a warp covers eight
// rows and a warp instruction reads whole 128-byte lines:
//   Q4_K  a lane's share of a row is one 32-input sub-block = 16 packed bytes (byte t = q[t] | q[t + 16] << 4): four
//         words, split into low and high nibbles, eight dp4a against the activations' 32 bytes (held in registers for
//         both rows), times the sub-block's 6-bit scale;
//   Q6_K  32 int8 values = two 16-input sub-blocks with an int8 scale each: eight dp4a, two multiplies.
// The R x M partial sums are then added over the eight lanes by a halving exchange (each step a lane keeps half of its
// values and sends the other half: R x M - 1 shuffles instead of 3 R x M), which leaves every (row, activation row)
// pair's exact integer in one lane; that lane owns the pair's fp32 chain.  Q4_K's mins term needs no exchange: the
// owner forms it from the row's eight 6-bit mins and the activation row's eight group sums with four dp4a (the sums
// are stored as S & 63 and S >> 6, both inside int8).
// Everything that comes from HBM once - the weights, their sub-block scales and mins, the super-block's d and dmin -
// is loaded for PD super-blocks at a time into registers (about 150 bytes per lane and super-block), all requests
// issued before the first use; the PD super-blocks are then worked through while other warps' requests are in flight.
// (A rolling register prefetch, one super-block consumed and one requested per step, measured at a third of the HBM
// rate: a wait for the oldest request also waits for the younger ones that share its scoreboard.)  Activations, their
// group sums and scales are small and stay in L1.  A CTA is one warp: eight rows, so that even a 5120-row projection
// spreads evenly over the SMs; for matrices of few rows a CTA is two to four warps on the same eight rows, each
// taking every KW-th super-block: its terms of the chain meet in shared memory and are added in order by one thread
// per output, so the bits do not depend on the split.
#pragma once
#include "common.cuh"

namespace w4a8 {

struct GemvArgs {
    const int8_t* xq;        // int8 [M, K]
    const float* a;          // fp32 [K/256, Ma]
    const int8_t* xs;        // int8 [K/256, Ma, 16] (Q4_K)
    const uint8_t* wq;       // Q4_K: uint8 [N, K/2]; Q6_K: int8 [N, K]
    const uint8_t* sc;       // Q4_K: uint8 [K/256, N, 8]; Q6_K: int8 [K/256, N, 16]
    const uint8_t* mn;       // Q4_K: uint8 [K/256, N, 8]
    const float* d;          // fp32 [K/256, N]
    const float* dm;         // fp32 [K/256, N] (Q4_K)
    void* out;
    long ldo;
    const int* n_rows;
    int M, N, K, Ma, epi;
};

constexpr int GEMV_R = 2;                // weight rows per eight-lane group: a warp covers 4 x R rows
constexpr int GEMV_PD = 4;               // super-blocks per load batch

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Sum v[0..NV) (NV = 1, 2, 4, 8 or 16) over the eight lanes that differ in bits 2, 1, 0.  While more than one value is left a
// step halves them (the lane whose bit is set keeps the upper half); after that the steps are plain butterflies.  On
// return v[0] (and v[1] for sixteen values) hold the totals of the original indices reduce8_index<NV>(lane) (+ 1).
template <int NV>
__device__ __forceinline__ void reduce8(int (&v)[NV], int lane) {
    int n = NV;
#pragma unroll
    for (int msk = 4; msk >= 1; msk >>= 1) {
        if (NV > 1 && n > 1) {
            n >>= 1;
            const bool up = (lane & msk) != 0;
#pragma unroll
            for (int i = 0; i < (NV + 1) / 2; ++i) {
                if (i < n) {
                    const int send = up ? v[i] : v[i + n];
                    const int keep = up ? v[i + n] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, msk);
                }
            }
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], msk);
        }
    }
}

template <int NV>
__device__ __forceinline__ int reduce8_index(int lane) {
    static_assert(NV == 1 || NV == 2 || NV == 4 || NV == 8 || NV == 16, "a power of two up to sixteen values");
    int base = (lane & 4) ? NV / 2 : 0;
    if (NV >= 4) base += (lane & 2) ? NV / 4 : 0;
    if (NV >= 8) base += (lane & 1) ? NV / 8 : 0;
    return base;
}

template <int NV>
__device__ __forceinline__ bool reduce8_owner(int lane) {
    // with fewer than eight values the butterfly steps leave copies: the lane with the low bits clear stores
    return NV >= 8 ? true : (lane & (8 / (NV >= 8 ? 8 : NV) - 1)) == 0;
}

__device__ __forceinline__ int dot32(const uint4& w0, const uint4& w1, const uint4& x0, const uint4& x1) {
    int d = __dp4a((int)w0.x, (int)x0.x, 0);
    d = __dp4a((int)w0.y, (int)x0.y, d);
    d = __dp4a((int)w0.z, (int)x0.z, d);
    d = __dp4a((int)w0.w, (int)x0.w, d);
    d = __dp4a((int)w1.x, (int)x1.x, d);
    d = __dp4a((int)w1.y, (int)x1.y, d);
    d = __dp4a((int)w1.z, (int)x1.z, d);
    d = __dp4a((int)w1.w, (int)x1.w, d);
    return d;
}

__device__ __forceinline__ void gemv_store(const GemvArgs& p, float y, long n, int m, int live, bool owner) {
    if (owner && n < p.N && m < live) {
        if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(y);
        else {
            float* o = (float*)p.out + (long)m * p.ldo + n;
            *o = __fadd_rn(*o, y);
        }
    }
}

// SPLIT: the CTA's KW warps took every KW-th super-block of the same rows and left each super-block's term t_b in shared
// memory; one thread per (row, activation row) pair now runs the chain y = fma(a_b, t_b, y) over all b in order - the
// unsplit kernel's operations on the same values.
template <int MR, int R>
__device__ __forceinline__ void gemv_chain(const GemvArgs& p, const float* terms, int NSB, int live) {
    constexpr int NV = R * MR;
    __syncthreads();
    const int t = threadIdx.x;
    if (t >= 4 * NV) return;
    const int m = t % MR, mm = m < p.M ? m : p.M - 1;
    float y = 0.0f;
    for (int b = 0; b < NSB; ++b) y = __fmaf_rn(__ldg(p.a + (long)b * p.Ma + mm), terms[b * (4 * NV) + t], y);
    gemv_store(p, y, (long)blockIdx.x * 4 * R + t / MR, m, live, true);
}

template <int MR, int R, bool SPLIT>
__global__ void __launch_bounds__(SPLIT ? 128 : 32)
w4a8_gemv_q4k_kernel(const GemvArgs p) {
    constexpr int NV = R * MR, PD = GEMV_PD, NF = NV >= 8 ? NV / 8 : 1;   // NF: (row, activation row) pairs per lane
    extern __shared__ float gemv_terms[];                          // SPLIT: [K / 256][4 * R * MR] chain terms
    const int KW = SPLIT ? (int)(blockDim.x >> 5) : 1;             // warps sharing the CTA's rows
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane & 7;                                        // sub-block of the super-block
    const long n0 = ((long)blockIdx.x * 4 + (lane >> 3)) * R;
    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    if (live <= 0) return;
    const int NSB = p.K >> 8;
    // the (row, activation row) pairs whose fp32 chains this lane owns: NF consecutive activation rows of one row
    const int mine = reduce8_index<NV>(lane), r_o = mine / MR, m_o = mine % MR;
    const long row_o = n0 + r_o < p.N ? n0 + r_o : p.N - 1;        // rows past N read the last row and store nothing
    const uint8_t* wrow[R];
    const uint8_t* scrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const long nn = n0 + r < p.N ? n0 + r : p.N - 1;
        wrow[r] = p.wq + nn * (p.K >> 1) + g * 16;
        scrow[r] = p.sc + nn * 8 + g;
    }
    const long sb_stride = (long)p.N * 8;
    uint4 ring[PD][R];
    int sc[PD][R];
    uint2 mn[PD];
    float dv[PD], dmv[PD];
    float y[NF];
#pragma unroll
    for (int i = 0; i < NF; ++i) y[i] = 0.0f;
    for (int b0 = warp; b0 < NSB; b0 += PD * KW) {
#pragma unroll
        for (int j = 0; j < PD; ++j)
            if (b0 + j * KW < NSB) {
                const long b = b0 + j * KW;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    ring[j][r] = ldg_stream(wrow[r] + b * 128);
                    sc[j][r] = scrow[r][b * sb_stride];
                }
                mn[j] = __ldg((const uint2*)(p.mn + (b * p.N + row_o) * 8));
                dv[j] = __ldg(p.d + b * p.N + row_o);
                dmv[j] = __ldg(p.dm + b * p.N + row_o);
            }
#pragma unroll
        for (int j = 0; j < PD; ++j) {
            const int b = b0 + j * KW;
            if (b < NSB) {
                uint4 w[R];
                int scb[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    w[r] = ring[j][r];
                    scb[r] = sc[j][r];
                }
                const uint2 mnb = mn[j];
                const float dvb = dv[j], ndm = -dmv[j];
                uint4 x0[MR], x1[MR];
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const int mm = m < p.M ? m : p.M - 1;
                    const uint4* xp = (const uint4*)(p.xq + (long)mm * p.K + b * 256 + g * 32);
                    x0[m] = __ldg(xp);                             // inputs 0..15 and 16..31 of the sub-block
                    x1[m] = __ldg(xp + 1);
                }
                int v[NV];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint4 lo = {w[r].x & 0x0F0F0F0Fu, w[r].y & 0x0F0F0F0Fu, w[r].z & 0x0F0F0F0Fu, w[r].w & 0x0F0F0F0Fu};
                    const uint4 hi = {(w[r].x >> 4) & 0x0F0F0F0Fu, (w[r].y >> 4) & 0x0F0F0F0Fu, (w[r].z >> 4) & 0x0F0F0F0Fu,
                                      (w[r].w >> 4) & 0x0F0F0F0Fu};
#pragma unroll
                    for (int m = 0; m < MR; ++m) v[r * MR + m] = scb[r] * dot32(lo, hi, x0[m], x1[m]);
                }
                reduce8<NV>(v, lane);
#pragma unroll
                for (int i = 0; i < NF; ++i) {                     // this lane's pairs: the same row, consecutive m
                    const int mi = m_o + i < p.M ? m_o + i : p.M - 1;
                    const uint4 s = __ldg((const uint4*)(p.xs + ((long)b * p.Ma + mi) * 16));
                    const int mins = __dp4a((int)mnb.x, (int)s.x, __dp4a((int)mnb.y, (int)s.y, 0)) +
                                     64 * __dp4a((int)mnb.x, (int)s.z, __dp4a((int)mnb.y, (int)s.w, 0));
                    float t = __fmul_rn(dvb, __int2float_rn(v[i]));
                    t = __fmaf_rn(ndm, __int2float_rn(mins), t);
                    if (!SPLIT) y[i] = __fmaf_rn(__ldg(p.a + (long)b * p.Ma + mi), t, y[i]);
                    else if (reduce8_owner<NV>(lane)) gemv_terms[b * (4 * NV) + ((lane >> 3) * R + r_o) * MR + m_o + i] = t;
                }
            }
        }
    }
    if (!SPLIT) {
#pragma unroll
        for (int i = 0; i < NF; ++i) gemv_store(p, y[i], n0 + r_o, m_o + i, live, reduce8_owner<NV>(lane));
    } else {
        gemv_chain<MR, R>(p, gemv_terms, NSB, live);
    }
}

template <int MR, int R, bool SPLIT>
__global__ void __launch_bounds__(SPLIT ? 128 : 32)
w4a8_gemv_q6k_kernel(const GemvArgs p) {
    constexpr int NV = R * MR, PD = GEMV_PD, NF = NV >= 8 ? NV / 8 : 1;   // NF: (row, activation row) pairs per lane
    extern __shared__ float gemv_terms[];                          // SPLIT: [K / 256][4 * R * MR] chain terms
    const int KW = SPLIT ? (int)(blockDim.x >> 5) : 1;             // warps sharing the CTA's rows
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane & 7;                                        // 32 of the super-block's 256 inputs
    const long n0 = ((long)blockIdx.x * 4 + (lane >> 3)) * R;
    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    if (live <= 0) return;
    const int NSB = p.K >> 8;
    const int mine = reduce8_index<NV>(lane), r_o = mine / MR, m_o = mine % MR;
    const long row_o = n0 + r_o < p.N ? n0 + r_o : p.N - 1;
    const uint8_t* wrow[R];
    const uint8_t* scrow[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const long nn = n0 + r < p.N ? n0 + r : p.N - 1;
        wrow[r] = p.wq + nn * p.K + g * 32;
        scrow[r] = p.sc + nn * 16 + 2 * g;
    }
    const long sb_stride = (long)p.N * 16;
    uint4 ring[PD][R][2];
    short sc[PD][R];                                               // two int8 sub-block scales
    float dv[PD];
    float y[NF];
#pragma unroll
    for (int i = 0; i < NF; ++i) y[i] = 0.0f;
    for (int b0 = warp; b0 < NSB; b0 += PD * KW) {
#pragma unroll
        for (int j = 0; j < PD; ++j)
            if (b0 + j * KW < NSB) {
                const long b = b0 + j * KW;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    ring[j][r][0] = ldg_stream(wrow[r] + b * 256);
                    ring[j][r][1] = ldg_stream(wrow[r] + b * 256 + 16);
                    sc[j][r] = *(const short*)(scrow[r] + b * sb_stride);
                }
                dv[j] = __ldg(p.d + b * p.N + row_o);
            }
#pragma unroll
        for (int j = 0; j < PD; ++j) {
            const int b = b0 + j * KW;
            if (b < NSB) {
                uint4 w0[R], w1[R];
                short scb[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    w0[r] = ring[j][r][0];
                    w1[r] = ring[j][r][1];
                    scb[r] = sc[j][r];
                }
                const float dvb = dv[j];
                uint4 x0[MR], x1[MR];
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    const int mm = m < p.M ? m : p.M - 1;
                    const uint4* xp = (const uint4*)(p.xq + (long)mm * p.K + b * 256 + g * 32);
                    x0[m] = __ldg(xp);
                    x1[m] = __ldg(xp + 1);
                }
                int v[NV];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int sc0 = (int)(int8_t)(scb[r] & 0xff), sc1 = (int)(int8_t)((scb[r] >> 8) & 0xff);
#pragma unroll
                    for (int m = 0; m < MR; ++m) {
                        int d0 = __dp4a((int)w0[r].x, (int)x0[m].x, 0);
                        d0 = __dp4a((int)w0[r].y, (int)x0[m].y, d0);
                        d0 = __dp4a((int)w0[r].z, (int)x0[m].z, d0);
                        d0 = __dp4a((int)w0[r].w, (int)x0[m].w, d0);
                        int d1 = __dp4a((int)w1[r].x, (int)x1[m].x, 0);
                        d1 = __dp4a((int)w1[r].y, (int)x1[m].y, d1);
                        d1 = __dp4a((int)w1[r].z, (int)x1[m].z, d1);
                        d1 = __dp4a((int)w1[r].w, (int)x1[m].w, d1);
                        v[r * MR + m] = sc0 * d0 + sc1 * d1;
                    }
                }
                reduce8<NV>(v, lane);
#pragma unroll
                for (int i = 0; i < NF; ++i) {
                    const int mi = m_o + i < p.M ? m_o + i : p.M - 1;
                    const float t = __fmul_rn(dvb, __int2float_rn(v[i]));
                    if (!SPLIT) y[i] = __fmaf_rn(__ldg(p.a + (long)b * p.Ma + mi), t, y[i]);
                    else if (reduce8_owner<NV>(lane)) gemv_terms[b * (4 * NV) + ((lane >> 3) * R + r_o) * MR + m_o + i] = t;
                }
            }
        }
    }
    if (!SPLIT) {
#pragma unroll
        for (int i = 0; i < NF; ++i) gemv_store(p, y[i], n0 + r_o, m_o + i, live, reduce8_owner<NV>(lane));
    } else {
        gemv_chain<MR, R>(p, gemv_terms, NSB, live);
    }
}

}  // namespace w4a8
