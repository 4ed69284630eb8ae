// Producers of quantized GEMM inputs and the deferred residual add.  All HBM-bound: one pass over the input with
// 128-bit loads, the row kept in registers between the maximum and the rounding, 128-bit stores of the int8 values.
//
//   rows_q8    x bf16/fp32 [T, K] (* inv_s[k]) -> int8 [T, K] + one fp32 scale per row   (kernels/quant.py:287-309)
//   quant_rows the same with one scale per group of gk inputs                             (kernels/w8a8.py:101-112)
//   swiglu_q8  gu bf16 [T, 2 FF] -> silu(gate) * up (* inv_s) -> int8 [T, FF] + scale      (kernels/quant.py:249-284)
//   quant_g    x -> int8 + one scale per 256 inputs + split sums of each 32 (W4A8)         (kernels/quant.py:314-330)
//   fold       h += (float(sum of int32 slots) * a_s[row]) * w_s[col]                      (kernels/quant.py:128-141)
//
// Rounding contract: scale = max(amax, 1e-10) / 127 and q = rint(y / scale) with IEEE divisions (__fdiv_rn), half to
// even.  PB_DIV_FULL selects the approximate full-range division (div.full.f32) for both instead.
#pragma once
#include "common.cuh"
#include "tp_sync.cuh"

namespace quant {

constexpr int MODE_PLAIN = 0;      // the row's own maximum
constexpr int MODE_STORE_AMAX = 1; // also store the row's maximum (tensor parallel, before the max all-reduce)
constexpr int MODE_USE_AMAX = 2;   // quantize with max(amax[t], own) (after it)
constexpr int MODE_EXCHANGE = 3;   // the ranks exchange their row maxima inside this launch (tp_sync.cuh; kernels/quant.py:190-212)

template <bool FULL>
__device__ __forceinline__ float fdiv(float a, float b) {
    if (FULL) {
        float r;
        asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
        return r;
    }
    return __fdiv_rn(a, b);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide maximum for up to 1024 threads; `red` is a 32-float shared array.
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : 0.0f;
    r = warp_max(r);
    __syncthreads();
    return r;
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)d << 24);
}

// Loads 8 consecutive inputs as fp32 (bf16: one 128-bit load; fp32: two).
template <bool BF16>
__device__ __forceinline__ void load8(const void* x, long idx, float (&v)[8]) {
    if (BF16) {
        const uint4 u = __ldg((const uint4*)((const __nv_bfloat16*)x + idx));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
        const float4 a = __ldg((const float4*)((const float*)x + idx));
        const float4 b = __ldg((const float4*)((const float*)x + idx + 4));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

// q = rint(v / scale) for 8 values, bit-identical to the IEEE division but far cheaper.  t = fma(v, r, 1.5 * 2^23)
// holds rint(v * r) (computed from the exact product, half to even) in its low mantissa bits, so the int8 value is the
// low byte of t: no conversion instruction.  r is taken twice, a little below and a little above 1 / scale
// (rcp * (1 -+ 2^-22); rcp itself is within 2^-24 of 1 / scale): the true quotient and its fp32 rounding both lie
// between v * r_lo and v * r_hi, rint is monotonic, so when both give the same integer that integer is
// rint(v / scale).  The (rare: about one vector in two thousand) vectors where they differ take the exact division.
template <bool FULL>
__device__ __forceinline__ uint2 quant8(const float (&v)[8], float scale, float rcp) {
    if (FULL) {
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __float2int_rn(fdiv<true>(v[i], scale));
        return make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
    }
    const float magic = 12582912.0f;
    const float r_lo = __fmul_rn(rcp, 0.99999976158142089844f);  // 1 - 2^-22
    const float r_hi = __fmul_rn(rcp, 1.00000023841857910156f);  // 1 + 2^-22
    uint32_t t[8];
    uint32_t differ = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        t[i] = __float_as_uint(__fmaf_rn(v[i], r_lo, magic));
        differ |= t[i] ^ __float_as_uint(__fmaf_rn(v[i], r_hi, magic));
    }
    if (differ) {                                               // rare: one branch per 8 values
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __float2int_rn(__fdiv_rn(v[i], scale));
        return make_uint2(pack4(q[0], q[1], q[2], q[3]), pack4(q[4], q[5], q[6], q[7]));
    }
    return make_uint2(__byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410),
                      __byte_perm(__byte_perm(t[4], t[5], 0x0040), __byte_perm(t[6], t[7], 0x0040), 0x5410));
}

// ------------------------------------------------------------------------------------------------- rows_q8
// One CTA per row, VPT vectors of 8 inputs per thread held in registers (K <= 8 * VPT * blockDim).
template <int VPT, bool BF16, bool FULL>
__global__ void __launch_bounds__(1024)
rows_q8_kernel(const void* __restrict__ x, long ldx, const float* __restrict__ inv_s, int8_t* __restrict__ q,
               float* __restrict__ s, const int* __restrict__ n_rows, int K, int mode, float* __restrict__ amax_io,
               const tpx::Sync sync) {
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const long t = blockIdx.x;
    if (t >= *n_rows) return;
    const int nvec = K >> 3;
    float v[VPT][8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nvec) {
            load8<BF16>(x, t * ldx + (long)c * 8, v[i]);
            if (inv_s) {
                const float4 a = __ldg((const float4*)(inv_s + c * 8)), b = __ldg((const float4*)(inv_s + c * 8 + 4));
                v[i][0] = __fmul_rn(v[i][0], a.x); v[i][1] = __fmul_rn(v[i][1], a.y);
                v[i][2] = __fmul_rn(v[i][2], a.z); v[i][3] = __fmul_rn(v[i][3], a.w);
                v[i][4] = __fmul_rn(v[i][4], b.x); v[i][5] = __fmul_rn(v[i][5], b.y);
                v[i][6] = __fmul_rn(v[i][6], b.z); v[i][7] = __fmul_rn(v[i][7], b.w);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
        }
    }
    amax = block_max(amax, red);
    if (mode == MODE_STORE_AMAX && threadIdx.x == 0) amax_io[t] = amax;
    if (mode == MODE_USE_AMAX) amax = fmaxf(amax_io[t], amax);
    if (mode == MODE_EXCHANGE) amax = tpx::exchange_amax(amax, t, sync);
    const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
    const float rcp = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nvec) *(uint2*)(q + t * K + (long)c * 8) = quant8<FULL>(v[i], scale, rcp);
    }
    if (threadIdx.x == 0) s[t] = scale;
}

// Any K (no alignment assumed), two passes over the row (the second hits L2): the fallback for odd shapes.
template <bool BF16, bool FULL>
__global__ void __launch_bounds__(256)
rows_q8_generic_kernel(const void* __restrict__ x, long ldx, const float* __restrict__ inv_s,
                       int8_t* __restrict__ q, float* __restrict__ s, const int* __restrict__ n_rows, int K, int mode,
                       float* __restrict__ amax_io, const tpx::Sync sync) {
    __shared__ float red[32];
    const long t = blockIdx.x;
    if (t >= *n_rows) return;
    auto val = [&](int k) {
        float y = BF16 ? __bfloat162float(((const __nv_bfloat16*)x)[t * ldx + k]) : ((const float*)x)[t * ldx + k];
        return inv_s ? __fmul_rn(y, inv_s[k]) : y;
    };
    float amax = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(val(k)));
    amax = block_max(amax, red);
    if (mode == MODE_STORE_AMAX && threadIdx.x == 0) amax_io[t] = amax;
    if (mode == MODE_USE_AMAX) amax = fmaxf(amax_io[t], amax);
    if (mode == MODE_EXCHANGE) amax = tpx::exchange_amax(amax, t, sync);
    const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
    for (int k = threadIdx.x; k < K; k += blockDim.x) q[t * K + k] = (int8_t)__float2int_rn(fdiv<FULL>(val(k), scale));
    if (threadIdx.x == 0) s[t] = scale;
}

// ------------------------------------------------------------------------------------------------- quant_rows (groups)
// One scale per gk inputs (gk = 32, 64, 128 or 256): a thread holds 8 inputs, gk / 8 neighbouring lanes share a group.
template <bool BF16, bool FULL>
__global__ void __launch_bounds__(256)
quant_groups_kernel(const void* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ s,
                    const int* __restrict__ n_rows, int K, int gk) {
    const long t = blockIdx.y;
    if (t >= *n_rows) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;      // vector of 8 inputs
    const bool in = c < (K >> 3);
    float v[8];
    float amax = 0.0f;
    if (in) {
        load8<BF16>(x, t * K + (long)c * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    }
    for (int o = 1; o < (gk >> 3); o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
    if (in) {
        *(uint2*)(q + t * K + (long)c * 8) = quant8<FULL>(v, scale, __fdiv_rn(1.0f, scale));
        if ((c & ((gk >> 3) - 1)) == 0) s[t * (K / gk) + c / (gk >> 3)] = scale;
    }
}

// ------------------------------------------------------------------------------------------------- swiglu_q8
// y = g / (1 + exp(-g)) * u * inv_s[c] (the reference's expression order, kernels/quant.py:256; the division is the
// approximate full-range one a Triton `/` lowers to), then rows_q8's rounding.  The same expression as the
// row-pipelined kernel (quant_pipe.cuh): a row's bits do not depend on which kernel quantizes it.
__device__ __forceinline__ float swiglu(float g, float u) { return __fmul_rn(fdiv<true>(g, 1.0f + __expf(-g)), u); }

template <int VPT, bool FULL>
__global__ void __launch_bounds__(1024)
swiglu_q8_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ inv_s, int8_t* __restrict__ q,
                 float* __restrict__ s, const int* __restrict__ n_rows, int FF, int mode, float* __restrict__ amax_io,
                 const tpx::Sync sync) {
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const long t = blockIdx.x;
    if (t >= *n_rows) return;
    const int nvec = FF >> 3;
    const __nv_bfloat16* row = gu + t * 2 * FF;
    float v[VPT][8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nvec) {
            float g[8], u[8];
            load8<true>(row, (long)c * 8, g);
            load8<true>(row + FF, (long)c * 8, u);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float y = swiglu(g[j], u[j]);
                if (inv_s) y = __fmul_rn(y, __ldg(inv_s + c * 8 + j));
                v[i][j] = y;
                amax = fmaxf(amax, fabsf(y));
            }
        }
    }
    amax = block_max(amax, red);
    if (mode == MODE_STORE_AMAX && threadIdx.x == 0) amax_io[t] = amax;
    if (mode == MODE_USE_AMAX) amax = fmaxf(amax_io[t], amax);
    if (mode == MODE_EXCHANGE) amax = tpx::exchange_amax(amax, t, sync);
    const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
    const float rcp = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nvec) *(uint2*)(q + t * FF + (long)c * 8) = quant8<FULL>(v[i], scale, rcp);
    }
    if (threadIdx.x == 0) s[t] = scale;
}

// ------------------------------------------------------------------------------------------------- norm_q8
// RMSNorm fused with the per-token quantizer, with the deferred residual add of a split-K projection finished first
// (the reference's _norm_q8_kernel, kernels/quant.py:145-171):
//   h[r, :] = add_rn(h, mul_rn(mul_rn(float(sum_p parts[p, r, :]), psa[r]), psw[:]))   (n_parts > 0; stored back)
//   y = (h * rsqrt(sum(h * h) / HID + eps)) * w;  scale = max(|y|max, 1e-10) / 127;  q = rint(y / scale)
// One CTA per output row i (input row rows[i] when gathering); the row stays in registers between the three passes.
// The sum of squares is added in a fixed order (lane-strided partial sums, then a warp and a block tree): the
// reference's Triton reduction leaves its order to the compiler, so this step is pinned by tolerance, not by bits.
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    __syncthreads();
    return r;
}

template <int VPT, bool FULL>
__global__ void __launch_bounds__(1024)
norm_q8_kernel(float* __restrict__ h, const float* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ s,
               const int* __restrict__ rows, const int* __restrict__ n_rows, int HID, float eps,
               const int32_t* __restrict__ parts, long part_stride, int n_parts, const float* __restrict__ psa,
               const float* __restrict__ psw, const tpx::Sync sync) {
    __shared__ float red[32];
    const long i = blockIdx.x;
    if (i >= *n_rows) return;
    const long r = rows ? (long)rows[i] : i;
    // tensor parallel, shortest passes: the deferred add's slots are every rank's (read over NVLink after the handshake)
    if (n_parts > 0) tpx::arrive_and_wait(sync, blockIdx.x == 0);
    const int nvec = HID >> 3;
    float v[VPT][8];
    float ss = 0.0f;
    const float sa = n_parts > 0 ? psa[r] : 0.0f;                 // read before this row's new scale is written
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nvec) {
            float* hp = h + r * HID + (long)c * 8;
            const float4 a = *(const float4*)hp, b = *(const float4*)(hp + 4);
            v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
            v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
            if (n_parts > 0) {
                int tot[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int pidx = 0; pidx < n_parts; ++pidx) {
                    const int4* pp = (const int4*)(parts + pidx * part_stride + r * HID + (long)c * 8);
                    const int4 x0 = __ldcs(pp), x1 = __ldcs(pp + 1);
                    tot[0] += x0.x; tot[1] += x0.y; tot[2] += x0.z; tot[3] += x0.w;
                    tot[4] += x1.x; tot[5] += x1.y; tot[6] += x1.z; tot[7] += x1.w;
                }
                for (int o = 0; o + 1 < sync.world; ++o)
                    for (int pidx = 0; pidx < n_parts; ++pidx) {
                        const int32_t* pp = sync.others[o] + pidx * part_stride + r * HID + (long)c * 8;
                        const int4 x0 = tpx::ld_peer4(pp), x1 = tpx::ld_peer4(pp + 4);
                        tot[0] += x0.x; tot[1] += x0.y; tot[2] += x0.z; tot[3] += x0.w;
                        tot[4] += x1.x; tot[5] += x1.y; tot[6] += x1.z; tot[7] += x1.w;
                    }
                const float4 w0 = __ldg((const float4*)(psw + c * 8)), w1 = __ldg((const float4*)(psw + c * 8 + 4));
                const float sw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j][e] = __fadd_rn(v[j][e], scale2(tot[e], sa, sw[e]));
                *(float4*)hp = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
                *(float4*)(hp + 4) = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = __fmaf_rn(v[j][e], v[j][e], ss);
        }
    }
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)HID), eps));
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nvec) {
            const float4 w0 = __ldg((const float4*)(w + c * 8)), w1 = __ldg((const float4*)(w + c * 8 + 4));
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[j][e] = __fmul_rn(__fmul_rn(v[j][e], rinv), ww[e]);
                amax = fmaxf(amax, fabsf(v[j][e]));
            }
        }
    }
    amax = block_max(amax, red);
    const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
    const float rcp = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nvec) *(uint2*)(q + i * HID + (long)c * 8) = quant8<FULL>(v[j], scale, rcp);
    }
    if (threadIdx.x == 0) s[i] = scale;
}

// ------------------------------------------------------------------------------------------------- gated_norm_q8
// The gated RMSNorm of the linear-attention output fused with the per-token quantizer (the reference's
// _gated_norm_q8_kernel, kernels/quant.py:215-246): per token, for every value head h (HV heads of D values):
//   y[h, d] = ((o[h, d] * rsqrt(sum_d o[h, :]^2 / D + eps)) * w[d]) * silu(z[h, d]) * inv_s[h, d]
// then scale = max(|y|max over the whole row, 1e-10) / 127 and q = rint(y / scale) (modes 1 / 2 as rows_q8).
// o fp32 [T, HV * D]; z bf16 at proj + t * P + z_off; one CTA per token, a thread owns 8 consecutive values, so the D / 8
// neighbouring lanes of a head reduce its sum of squares with shuffles (D = 64, 128 or 256).  The sum's order is this
// kernel's own (the reference's is its compiler's): pinned by tolerance, like norm_q8.
template <int VPT, bool FULL>
__global__ void __launch_bounds__(1024)
gated_norm_q8_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ proj, long P, long z_off,
                     const float* __restrict__ w, const float* __restrict__ inv_s, int8_t* __restrict__ q,
                     float* __restrict__ s, const int* __restrict__ n_rows, int HV, int D, float eps, int mode,
                     float* __restrict__ amax_io, const tpx::Sync sync) {
    __shared__ float red[32];
    const long t = blockIdx.x;
    if (t >= *n_rows) return;
    const int nvec = (HV * D) >> 3, lanes = D >> 3;                // lanes of one head (8, 16 or 32)
    float v[VPT][8];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        const bool on = c < nvec;
        float ss = 0.0f;
        if (on) {
            const float* op = o + t * HV * D + (long)c * 8;
            const float4 a = __ldg((const float4*)op), b = __ldg((const float4*)(op + 4));
            v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
            v[j][4] = b.x; v[j][5] = b.y; v[j][6] = b.z; v[j][7] = b.w;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = __fmaf_rn(v[j][e], v[j][e], ss);
        }
        // every lane takes part in the shuffles (whole heads are on or off together: nvec is a multiple of lanes)
        for (int off = lanes >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if (on) {
            const float rinv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)D), eps));
            const int d0 = (c * 8) % D;
            float z[8];
            load8<true>(proj, t * P + z_off + (long)c * 8, z);
            const float4 w0 = __ldg((const float4*)(w + d0)), w1 = __ldg((const float4*)(w + d0 + 4));
            const float4 i0 = __ldg((const float4*)(inv_s + c * 8)), i1 = __ldg((const float4*)(inv_s + c * 8 + 4));
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            const float iv[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float g = fdiv<true>(z[e], 1.0f + __expf(-z[e]));
                float y = __fmul_rn(__fmul_rn(__fmul_rn(v[j][e], rinv), ww[e]), g);
                y = __fmul_rn(y, iv[e]);
                v[j][e] = y;
                amax = fmaxf(amax, fabsf(y));
            }
        }
    }
    amax = block_max(amax, red);
    if (mode == MODE_STORE_AMAX && threadIdx.x == 0) amax_io[t] = amax;
    if (mode == MODE_USE_AMAX) amax = fmaxf(amax_io[t], amax);
    if (mode == MODE_EXCHANGE) amax = tpx::exchange_amax(amax, t, sync);
    const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
    const float rcp = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nvec) *(uint2*)(q + t * HV * D + (long)c * 8) = quant8<FULL>(v[j], scale, rcp);
    }
    if (threadIdx.x == 0) s[t] = scale;
}

// ------------------------------------------------------------------------------------------------- head_quant
// The final RMSNorm of a residual row, then int8 per group of 32 inputs (the reference's _head_quant_kernel,
// kernels/decode.py:113-133): one CTA per row, the row in registers; a group of 32 is four neighbouring lanes.
template <int VPT, bool FULL>
__global__ void __launch_bounds__(1024)
head_quant_kernel(const float* __restrict__ h, const float* __restrict__ w, int8_t* __restrict__ q,
                  float* __restrict__ s, const int* __restrict__ n_rows, int HID, float eps) {
    __shared__ float red[32];
    const long r = blockIdx.x;
    if (r >= *n_rows) return;
    const int nvec = HID >> 3;
    float v[VPT][8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nvec) {
            load8<false>(h, r * HID + (long)c * 8, v[j]);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = __fmaf_rn(v[j][e], v[j][e], ss);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j][e] = 0.0f;
        }
    }
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)HID), eps));
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        const bool on = c < nvec;
        float amax = 0.0f;
        if (on) {
            const float4 w0 = __ldg((const float4*)(w + c * 8)), w1 = __ldg((const float4*)(w + c * 8 + 4));
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[j][e] = __fmul_rn(__fmul_rn(v[j][e], rinv), ww[e]);
                amax = fmaxf(amax, fabsf(v[j][e]));
            }
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float scale = fdiv<FULL>(fmaxf(amax, 1e-10f), 127.0f);
        if (on) {
            *(uint2*)(q + r * HID + (long)c * 8) = quant8<FULL>(v[j], scale, __fdiv_rn(1.0f, scale));
            if ((c & 3) == 0) s[r * (HID >> 5) + (c >> 2)] = scale;
        }
    }
}

// ------------------------------------------------------------------------------------------------- quant_g (W4A8)
// One warp per 256 inputs of a row: lane l holds inputs 8 l .. 8 l + 7, so 4 neighbouring lanes make a group of 32.
// Writes q int8 [T, K], a fp32 [K/256, Ma] and xs int8 [K/256, Ma, 16] (eight S & 63 then eight S >> 6), IEEE division
// (the reference's _store_g, kernels/quant.py:315-330).
__device__ __forceinline__ void store_g_warp(const float (&v)[8], int8_t* __restrict__ q, float* __restrict__ a,
                                             int8_t* __restrict__ xs, long t, int b, int lane, int Ma, int K) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = warp_max(amax);
    const float scale = __fdiv_rn(fmaxf(amax, 1e-10f), 127.0f);
    int qi[8], S = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        qi[j] = __float2int_rn(__fdiv_rn(v[j], scale));
        S += qi[j];
    }
    *(uint2*)(q + t * K + (long)b * 256 + lane * 8) =
        make_uint2(pack4(qi[0], qi[1], qi[2], qi[3]), pack4(qi[4], qi[5], qi[6], qi[7]));
    S += __shfl_xor_sync(0xffffffffu, S, 1);
    S += __shfl_xor_sync(0xffffffffu, S, 2);
    if (lane == 0) a[(long)b * Ma + t] = scale;
    if ((lane & 3) == 0) {
        int8_t* o = xs + ((long)b * Ma + t) * 16 + (lane >> 2);
        o[0] = (int8_t)(S & 63);
        o[8] = (int8_t)(S >> 6);
    }
}

template <bool BF16>
__global__ void __launch_bounds__(256)
quant_g_kernel(const void* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ a, int8_t* __restrict__ xs,
               const int* __restrict__ n_rows, int Ma, int K) {
    const long t = blockIdx.y;
    if (t >= *n_rows) return;
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);     // super-block
    if (b >= (K >> 8)) return;
    float v[8];
    load8<BF16>(x, t * K + (long)b * 256 + lane * 8, v);
    store_g_warp(v, q, a, xs, t, b, lane, Ma, K);
}

// SwiGLU + the per-256 quantizer (the reference's _swiglu_g_kernel, kernels/quant.py:371-381): gu bf16 [T, 2 FF]
// (gate columns then up columns) -> the W4A8 activation triple of silu(gate) * up.  Nothing row-wide: a warp per 256.
__global__ void __launch_bounds__(256)
swiglu_g_kernel(const __nv_bfloat16* __restrict__ gu, int8_t* __restrict__ q, float* __restrict__ a,
                int8_t* __restrict__ xs, const int* __restrict__ n_rows, int Ma, int FF) {
    const long t = blockIdx.y;
    if (t >= *n_rows) return;
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= (FF >> 8)) return;
    float g[8], u[8], v[8];
    load8<true>(gu, t * 2 * FF + (long)b * 256 + lane * 8, g);
    load8<true>(gu, t * 2 * FF + FF + (long)b * 256 + lane * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(fdiv<true>(g[e], 1.0f + __expf(-g[e])), u[e]);
    store_g_warp(v, q, a, xs, t, b, lane, Ma, FF);
}

// RMSNorm + the per-256 quantizer (the reference's _norm_g_kernel, kernels/quant.py:333-345): one CTA per row, a warp
// per 256 inputs (HID / 256 warps), the row's sum of squares through the block.
__global__ void __launch_bounds__(1024)
norm_g_kernel(const float* __restrict__ h, const float* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ a,
              int8_t* __restrict__ xs, const int* __restrict__ n_rows, int Ma, int HID, float eps) {
    __shared__ float red[32];
    const long t = blockIdx.x;
    if (t >= *n_rows) return;
    const int lane = threadIdx.x & 31, b = threadIdx.x >> 5;
    float v[8];
    load8<false>(h, t * HID + (long)b * 256 + lane * 8, v);
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = __fmaf_rn(v[e], v[e], ss);
    ss = block_sum(ss, red);
    const float rinv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)HID), eps));
    const float4 w0 = __ldg((const float4*)(w + b * 256 + lane * 8)), w1 = __ldg((const float4*)(w + b * 256 + lane * 8 + 4));
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(__fmul_rn(v[e], rinv), ww[e]);
    store_g_warp(v, q, a, xs, t, b, lane, Ma, HID);
}

// Gated RMSNorm + the per-256 quantizer (the reference's _gated_norm_g_kernel, kernels/quant.py:348-368): a warp per
// 256 values = 256 / D heads (D = 64, 128 or 256), the head's sum of squares over its D / 8 lanes.
__global__ void __launch_bounds__(256)
gated_norm_g_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ proj, long P, long z_off,
                    const float* __restrict__ w, int8_t* __restrict__ q, float* __restrict__ a, int8_t* __restrict__ xs,
                    const int* __restrict__ n_rows, int Ma, int HV, int D, float eps) {
    const long t = blockIdx.y;
    if (t >= *n_rows) return;
    const int lane = threadIdx.x & 31, K = HV * D;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= (K >> 8)) return;
    const int c = b * 32 + lane;                                   // vector of 8 values in the row
    float v[8], z[8];
    load8<false>(o, t * K + (long)c * 8, v);
    load8<true>(proj, t * P + z_off + (long)c * 8, z);
    float ss = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) ss = __fmaf_rn(v[e], v[e], ss);
    for (int off = D >> 4; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float rinv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float)D), eps));
    const int d0 = (c * 8) % D;
    const float4 w0 = __ldg((const float4*)(w + d0)), w1 = __ldg((const float4*)(w + d0 + 4));
    const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e)
        v[e] = __fmul_rn(__fmul_rn(__fmul_rn(v[e], rinv), ww[e]), fdiv<true>(z[e], 1.0f + __expf(-z[e])));
    store_g_warp(v, q, a, xs, t, b, lane, Ma, K);
}

// ------------------------------------------------------------------------------------------------- fold
// h[r, c] = add_rn(h, mul_rn(mul_rn(float(sum_p slots[p, r, c]), a_s[r]), w_s[c])); 4 columns per thread.
__global__ void __launch_bounds__(256)
fold_kernel(float* __restrict__ h, long ldh, const int32_t* __restrict__ slots, long slot_stride, int S,
            const float* __restrict__ a_s, const float* __restrict__ w_s, const int* __restrict__ n_rows, int N) {
    pdl_trigger();
    pdl_wait();
    const long r = blockIdx.y;
    if (r >= *n_rows) return;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= N) return;
    const float sa = a_s[r];
    if (c + 4 <= N && (N & 3) == 0 && (ldh & 3) == 0) {
        int4 tot = __ldcs((const int4*)(slots + r * N + c));
        for (int p = 1; p < S; ++p) {
            const int4 v = __ldcs((const int4*)(slots + p * slot_stride + r * N + c));
            tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
        }
        const float4 sw = __ldg((const float4*)(w_s + c));
        float4 o = *(float4*)(h + r * ldh + c);
        o.x = __fadd_rn(o.x, scale2(tot.x, sa, sw.x));
        o.y = __fadd_rn(o.y, scale2(tot.y, sa, sw.y));
        o.z = __fadd_rn(o.z, scale2(tot.z, sa, sw.z));
        o.w = __fadd_rn(o.w, scale2(tot.w, sa, sw.w));
        *(float4*)(h + r * ldh + c) = o;
    } else {
        for (int j = c; j < N && j < c + 4; ++j) {
            int tot = 0;
            for (int p = 0; p < S; ++p) tot += slots[p * slot_stride + r * N + j];
            h[r * ldh + j] = __fadd_rn(h[r * ldh + j], scale2(tot, sa, w_s[j]));
        }
    }
}

// The same fold over every rank's slots (the fused all-reduce of the shortest tensor-parallel passes,
// kernels/quant.py:128-141 with NR > 1): after the handshake the other ranks' slots are read over NVLink, uncached, and
// added to this rank's - integer sums, exact in any order - before the one scaling.  N % 4 == 0.
__global__ void __launch_bounds__(256)
fold_sync_kernel(float* __restrict__ h, long ldh, const int32_t* __restrict__ slots, long slot_stride, int S,
                 const float* __restrict__ a_s, const float* __restrict__ w_s, const int* __restrict__ n_rows, int N,
                 const tpx::Sync sync) {
    const long r = blockIdx.y;
    if (r >= *n_rows) return;                       // whole block: the live count is the same on every rank
    tpx::arrive_and_wait(sync, blockIdx.x == 0 && blockIdx.y == 0);
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= N) return;
    const float sa = a_s[r];
    int4 tot = __ldcs((const int4*)(slots + r * N + c));
    for (int p = 1; p < S; ++p) {
        const int4 v = __ldcs((const int4*)(slots + p * slot_stride + r * N + c));
        tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
    }
    for (int o = 0; o + 1 < sync.world; ++o)
        for (int p = 0; p < S && sync.others[o]; ++p) {
            const int4 v = tpx::ld_peer4(sync.others[o] + p * slot_stride + r * N + c);
            tot.x += v.x; tot.y += v.y; tot.z += v.z; tot.w += v.w;
        }
    const float4 sw = __ldg((const float4*)(w_s + c));
    float4 o4 = *(float4*)(h + r * ldh + c);
    o4.x = __fadd_rn(o4.x, scale2(tot.x, sa, sw.x));
    o4.y = __fadd_rn(o4.y, scale2(tot.y, sa, sw.y));
    o4.z = __fadd_rn(o4.z, scale2(tot.z, sa, sw.z));
    o4.w = __fadd_rn(o4.w, scale2(tot.w, sa, sw.w));
    *(float4*)(h + r * ldh + c) = o4;
}

}  // namespace quant
