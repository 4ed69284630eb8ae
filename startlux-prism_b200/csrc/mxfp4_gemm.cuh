// MXFP4 projections on the sm_100a tensor cores: e2m1 values (two per byte, low nibble = even k) with one UE8M0
// scale per 32 inputs on both operands, fp32 accumulation (tcgen05.mma kind::mxf4.block_scale, K = 64 per
// instruction, scale factors read from tensor memory).
//
//   mxfp4_quant_kernel    x bf16 / fp32 [n, K] (* inv[k]) -> packed codes [n, K/2] + scale bytes [n, K/32]
//                         (the reference's _quant_kernel / _code, kernels/mxfp4.py:106-171)
//   sf_tile_kernel        scale bytes [rows, K/32] -> the tensor core's tiled order: blocks of 128 rows x 4 scales
//                         (512 bytes: 32 x 16 bytes, byte (r % 32) * 16 + (r / 32) * 4 + k) - what the reference
//                         delegates to CUTLASS (csrc/mxfp4_gemm.cu:66-72,130-153)
//   mxfp4_gemm_kernel     out = deq(A) deq(W)^T: bf16 store or fp32 add (kernels/mxfp4.py:260-289, csrc/mxfp4_gemm.cu)
//
// The K loop runs whole 256-input blocks in ascending order for every M, so an output element has the same bits
// whatever batch it is computed in (the reference's batch-invariance rule, kernels/mxfp4.py:244-246).
#pragma once
#include "common.cuh"

namespace mxfp4 {

// ------------------------------------------------------------------------------------------------- quantizer
// Block exponent e = clamp(ceil(log2(max(amax, 1e-30) / 6)), -127, 127), evaluated exactly from the float's fields:
// amax = 1.f x 2^(E - 127) is at most 6 x 2^e = 1.5 x 2^(e + 2)  <=>  e = E - 129 when 1.f <= 1.5, else E - 128.
__device__ __forceinline__ int block_exponent(float amax) {
    amax = fmaxf(amax, 1e-30f);
    const uint32_t b = __float_as_uint(amax);
    const int E = (int)((b >> 23) & 0xff);
    int e = ((b & 0x7fffffu) <= 0x400000u) ? E - 129 : E - 128;
    return e < -127 ? -127 : (e > 127 ? 127 : e);
}

// 2^(-e) for e in [-127, 127] (2^-127 is subnormal)
__device__ __forceinline__ float pow2_neg(int e) {
    return e == 127 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(127 - e) << 23);
}

// magnitude code by strict thresholds, sign bit whenever v < 0 (kernels/mxfp4.py:106-117)
__device__ __forceinline__ uint32_t e2m1_code(float v, float inv_scale) {
    const float a = __fmul_rn(fabsf(v), inv_scale);
    uint32_t c = 0;
    c = a > 0.25f ? 1u : c;
    c = a > 0.75f ? 2u : c;
    c = a > 1.25f ? 3u : c;
    c = a > 1.75f ? 4u : c;
    c = a > 2.5f ? 5u : c;
    c = a > 3.5f ? 6u : c;
    c = a > 5.0f ? 7u : c;
    return v < 0.0f ? (c | 8u) : c;
}

// One thread per 8 inputs, four neighbouring lanes per 32-input block.
template <bool BF16>
__global__ void __launch_bounds__(256)
mxfp4_quant_kernel(const void* __restrict__ x, const float* __restrict__ inv, uint8_t* __restrict__ q,
                   uint8_t* __restrict__ s, int n, int K) {
    const long row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;            // vector of 8 inputs
    if (row >= n) return;
    const bool in = c < (K >> 3);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    if (in) {
        if (BF16) {
            const uint4 u = __ldg((const uint4*)((const __nv_bfloat16*)x + row * K + (long)c * 8));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
            const float4 a = __ldg((const float4*)((const float*)x + row * K + (long)c * 8));
            const float4 b = __ldg((const float4*)((const float*)x + row * K + (long)c * 8 + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        if (inv) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], __ldg(inv + c * 8 + j));
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const int e = block_exponent(amax);
    const float is = pow2_neg(e);
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) packed |= e2m1_code(v[j], is) << (4 * j);
    if (in) {
        *(uint32_t*)(q + row * (K >> 1) + (long)c * 4) = packed;
        if ((c & 3) == 0) s[row * (K >> 5) + (c >> 2)] = (uint8_t)(e + 127);
    }
}

// ------------------------------------------------------------------------------------------------- scale tiling
// dst block (rb, ka) at ((rb * KA + ka) * 512): rows rb * 128 .. + 127, scales ka * 4 .. + 3.  Rows past `rows` get 0.
__global__ void __launch_bounds__(256)
sf_tile_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int rows, int K) {
    const int KA = K >> 7, G = K >> 5;
    const long total = (long)((rows + 127) / 128) * KA * 128;       // one thread per (block, row): 4 bytes
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int r_in = (int)(i & 127);
    const long blk = i >> 7;
    const int ka = (int)(blk % KA);
    const long rb = blk / KA;
    const long r = rb * 128 + r_in;
    uint32_t v = 0;
    if (r < rows) {
        const uint8_t* p = src + r * G + ka * 4;
        v = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    }
    *(uint32_t*)(dst + blk * 512 + (r_in & 31) * 16 + (r_in >> 5) * 4) = v;
}

// ------------------------------------------------------------------------------------------------- GEMM
constexpr int BM = 128, BN = 128;
constexpr int KB_BYTES = 128;                  // 256 e2m1 inputs per pipeline stage (one 128-byte swizzle row)
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * KB_BYTES, B_BYTES = BN * KB_BYTES, SF_BYTES = 1024;   // 2 scale blocks per operand
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;
constexpr int TMEM_COLS = 512;                 // 2 x 128 accumulator columns + 2 x 16 scale columns
constexpr int SF_COL0 = 256;

struct AuxM {
    uint64_t full[8], empty[8], tfull[2], tempty[2];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256 + 4 * 32 * 33 * 4;

// tcgen05.mma kind::mxf4 with block scales: e2m1 x e2m1, UE8M0 scale per 32 inputs, fp32 accumulate.
//   bits [4,6) B scale-factor id, [7,10) A format (1 = e2m1), [10,13) B format, [17,23) N >> 3, bit 23 scale format
//   (1 = UE8M0), [24,29) M >> 4, [29,31) A scale-factor id (the byte pair of the 32-bit scale word: 0 or 2).
__device__ __forceinline__ uint32_t idesc_mxf4(int m, int n, uint32_t a_sf, uint32_t b_sf) {
    return (b_sf << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) |
           ((uint32_t)(m >> 4) << 24) | (a_sf << 29);
}

__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        : : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 tensor-memory columns, replicated in the four lane quarters.
__device__ __forceinline__ void tmem_cp_sf(uint32_t dst_tmem, uint32_t smem_addr) {
    uint64_t d = 0;                                   // no swizzle, 8-row groups 128 bytes apart, one 16-byte K chunk
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(d) : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 : : "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

struct GemmArgs {
    const uint8_t* sfa;     // tiled activation scales
    const uint8_t* sfb;     // tiled weight scales
    void* out;
    long ldo;
    int M, N, K, epi;
    // K split of the 128 x 128 kernel (few rows, few tiles): slice z of a tile covers K blocks [z * kbs, (z + 1) * kbs);
    // the slices' fp32 accumulators meet in ws [tile][slice][128][128] and the CTA that finishes a tile last adds them
    // in slice order (deterministic; the sum's rounding differs from the unsplit order within fp32)
    int split, kbs;
    float* ws;
    int* counters;
};

__global__ void __launch_bounds__(192, 1)
mxfp4_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const GemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    AuxM* aux = (AuxM*)(smem + STAGES * STAGE_BYTES);
    uint32_t* stage_buf = (uint32_t*)(smem + STAGES * STAGE_BYTES + 256);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
    const int num_tiles = num_m * num_n, KB = p.K / 256, KA = p.K / 128;
    const int num_units = num_tiles * p.split;                        // (tile, K slice)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&aux->tfull[b]), 1);
            mbar_init(smem_u32(&aux->tempty[b]), 4);
        }
        aux->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&aux->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    volatile int* abort_flag = &aux->abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const int t = u / p.split, z = u - t * p.split;
                const int mt = t % num_m, nt = t / num_m;
                const int kb_end = (z + 1) * p.kbs < KB ? (z + 1) * p.kbs : KB;
                for (int kb = z * p.kbs; kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0xE00 + stage)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&aux->full[stage]);
                    mbar_expect_tx(bar, STAGE_BYTES);
                    const uint32_t st = smem_u32(smem + stage * STAGE_BYTES);
                    tma_load_2d(st, &tm_a, kb * KB_BYTES, mt * BM, bar);
                    tma_load_2d(st + A_BYTES, &tm_b, kb * KB_BYTES, nt * BN, bar);
                    bulk_load(st + A_BYTES + B_BYTES, p.sfa + ((long)mt * KA + kb * 2) * 512, SF_BYTES, bar);
                    bulk_load(st + A_BYTES + B_BYTES + SF_BYTES, p.sfb + ((long)nt * KA + kb * 2) * 512, SF_BYTES, bar);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                unsigned long long t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 2000000ull) {
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0, buf = 0, sfp = 0;
            uint32_t phase = 0, bphase = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const int z = u % p.split;
                const int kb_begin = z * p.kbs, kb_end = (z + 1) * p.kbs < KB ? (z + 1) * p.kbs : KB;
                if (!mbar_wait(smem_u32(&aux->tempty[buf]), bphase ^ 1, abort_flag, 0xE10 + buf)) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0xE20 + stage)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + stage * STAGE_BYTES);
                    const uint32_t sf_smem = st + A_BYTES + B_BYTES;
                    const uint32_t sfa_t = tmem_base + SF_COL0 + sfp * 16, sfb_t = sfa_t + 8;
                    tmem_cp_sf(sfa_t, sf_smem);
                    tmem_cp_sf(sfa_t + 4, sf_smem + 512);
                    tmem_cp_sf(sfb_t, sf_smem + SF_BYTES);
                    tmem_cp_sf(sfb_t + 4, sf_smem + SF_BYTES + 512);
                    const uint64_t ad = umma_desc_k128(st), bd = umma_desc_k128(st + A_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {                 // K = 64 inputs = 32 bytes per instruction
                        const uint32_t sf_id = (k & 1) * 2;
                        umma_mxf4(d, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32),
                                  idesc_mxf4(BM, BN, sf_id, sf_id), sfa_t + (k >> 1) * 4, sfb_t + (k >> 1) * 4,
                                  (kb > kb_begin || k) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&aux->empty[stage]));
                    sfp ^= 1;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&aux->tfull[buf]));
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else {
        const int q = warp & 3;
        uint32_t* stg = stage_buf + q * (32 * 33);
        int buf = 0;
        uint32_t bphase = 0;
        for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
            const int t = u / p.split, z = u - t * p.split;
            const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN;
            if (!mbar_wait(smem_u32(&aux->tfull[buf]), bphase, abort_flag, 0xE30 + buf)) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            const int rows_here = p.M - (m0 + q * 32);
            const bool word_ok = p.epi != 0 || ((((uintptr_t)p.out & 3) == 0) && (p.ldo % 2 == 0));
            const int cpw = p.epi == 0 ? 2 : 1;
            float* ws_tile = p.ws + (long)t * p.split * (BM * BN);
            if (p.split > 1) {
                // this slice's accumulator -> workspace (live rows only), then the tile's last CTA adds the slices
                float* mine = ws_tile + (long)z * (BM * BN) + (long)(q * 32) * BN;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    if (n0 + c0 >= p.N) break;
                    uint32_t r[32];
                    tmem_ld32(lane_addr + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = r[j];
                    __syncwarp();
                    for (int rr = 0; rr < 32 && rr < rows_here; ++rr)
                        __stcg(mine + rr * BN + c0 + lane, __uint_as_float(stg[rr * 33 + lane]));
                    __syncwarp();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->tempty[buf]));
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) aux->is_last = (atomicAdd(p.counters + t, 1) == p.split - 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!aux->is_last) continue;
                __threadfence();
                if (threadIdx.x == 64) p.counters[t] = 0;
                // the slices in order, eight rows' loads in flight at a time; a lane owns four consecutive columns
                const int col = n0 + lane * 4;
                const bool vec = col + 4 <= p.N && (p.ldo & 3) == 0 && ((uintptr_t)p.out & 15) == 0;
#pragma unroll 1
                for (int rr0 = 0; rr0 < 32 && rr0 < rows_here; rr0 += 8) {
                    float4 acc[8];
                    const float* src = ws_tile + (long)(q * 32 + rr0) * BN + lane * 4;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (rr0 + j < rows_here) acc[j] = __ldcg((const float4*)(src + j * BN));
                    for (int zz = 1; zz < p.split; ++zz) {
                        float4 v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (rr0 + j < rows_here) v[j] = __ldcg((const float4*)(src + (long)zz * (BM * BN) + j * BN));
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (rr0 + j < rows_here) {
                                acc[j].x = __fadd_rn(acc[j].x, v[j].x);
                                acc[j].y = __fadd_rn(acc[j].y, v[j].y);
                                acc[j].z = __fadd_rn(acc[j].z, v[j].z);
                                acc[j].w = __fadd_rn(acc[j].w, v[j].w);
                            }
                    }
                    float4 old[8];
                    if (p.epi != 0 && vec) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (rr0 + j < rows_here)
                                old[j] = __ldcg((const float4*)((float*)p.out + (long)(m0 + q * 32 + rr0 + j) * p.ldo + col));
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (rr0 + j >= rows_here) continue;
                        const long off = (long)(m0 + q * 32 + rr0 + j) * p.ldo + col;
                        const float a4[4] = {acc[j].x, acc[j].y, acc[j].z, acc[j].w};
                        if (p.epi == 0) {
                            if (vec) {
                                __nv_bfloat162 b0 = __floats2bfloat162_rn(a4[0], a4[1]), b1 = __floats2bfloat162_rn(a4[2], a4[3]);
                                *(uint2*)((__nv_bfloat16*)p.out + off) = make_uint2(*(uint32_t*)&b0, *(uint32_t*)&b1);
                            } else {
                                for (int e = 0; e < 4; ++e)
                                    if (col + e < p.N) ((__nv_bfloat16*)p.out)[off + e] = __float2bfloat16_rn(a4[e]);
                            }
                        } else if (vec) {
                            float4 o = old[j];
                            o.x = __fadd_rn(o.x, a4[0]);
                            o.y = __fadd_rn(o.y, a4[1]);
                            o.z = __fadd_rn(o.z, a4[2]);
                            o.w = __fadd_rn(o.w, a4[3]);
                            *(float4*)((float*)p.out + off) = o;
                        } else {
                            for (int e = 0; e < 4; ++e)
                                if (col + e < p.N) ((float*)p.out)[off + e] = __fadd_rn(((float*)p.out)[off + e], a4[e]);
                        }
                    }
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32 * cpw) {
                if (n0 + c0 >= p.N) break;
                uint32_t r[32];
                tmem_ld32(lane_addr + c0, r);
                tmem_ld_wait();
                if (p.epi == 0) {
                    uint32_t r2[32];
                    tmem_ld32(lane_addr + c0 + 32, r2);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                        __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(r2[2 * j]), __uint_as_float(r2[2 * j + 1]));
                        stg[lane * 33 + j] = *(uint32_t*)&b0;
                        stg[lane * 33 + 16 + j] = *(uint32_t*)&b1;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = r[j];
                }
                __syncwarp();
                const int col = n0 + c0 + lane * cpw;
                if (p.epi == 0) {
                    for (int rr = 0; rr < 32 && rr < rows_here; ++rr) {
                        const long off = (long)(m0 + q * 32 + rr) * p.ldo + col;
                        const uint32_t v = stg[rr * 33 + lane];
                        if (word_ok && col + 2 <= p.N) {
                            *(uint32_t*)((__nv_bfloat16*)p.out + off) = v;
                        } else {
                            if (col < p.N) ((uint16_t*)p.out)[off] = (uint16_t)(v & 0xffff);
                            if (col + 1 < p.N) ((uint16_t*)p.out)[off + 1] = (uint16_t)(v >> 16);
                        }
                    }
                } else if (col < p.N) {
                    float* base = (float*)p.out + (long)(m0 + q * 32) * p.ldo + col;
                    float o[32];
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr)
                        if (rr < rows_here) o[rr] = __ldcg(base + (long)rr * p.ldo);
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr)
                        if (rr < rows_here) base[(long)rr * p.ldo] = __fadd_rn(o[rr], __uint_as_float(stg[rr * 33 + lane]));
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->tempty[buf]));
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------- GEMM, 128 x 256 tiles
// The 128 x 128 kernel above needs 32 KB of operands per four MMAs (256 cycles at the fp4 rate): shared memory is
// written by the bulk copies and read by the tensor core at 128 bytes per cycle each, and that, not the tensor pipe,
// bounds it (ncu: tensor pipe 29 % busy).  A 128 x 256 tile needs 48 KB per four MMAs of twice the work.  Tensor
// memory then has room for ONE accumulator (256 columns; the scale factors need 48 more), so a tile's epilogue does
// not overlap the next tile's MMAs: eight epilogue warps keep it short.
//   tensor memory: accumulator columns 0..255 | scale factors from column 256: two alternating sets of
//                  (A: 2 K blocks x 4 columns, B: 2 K blocks x 8 columns)
//   stage: A 16 KB | B 32 KB | scales of A 1 KB | scales of B 2 KB (weight rows 0-127: K blocks 0, 1; rows 128-255: 0, 1)
constexpr int BN2 = 256;
constexpr int STAGES2 = 4;
constexpr int B2_BYTES = BN2 * KB_BYTES;
constexpr int STAGE2_BYTES = A_BYTES + B2_BYTES + SF_BYTES + 2 * SF_BYTES;
constexpr int EPI2_WARPS = 8;
constexpr int THREADS2 = 96 + 32 * EPI2_WARPS;                         // producer, MMA issuer, scale-factor copier, epilogue
constexpr int STG2_WORDS = 32 * 17;                                   // per warp: 32 rows x 16 words (+1: no conflicts)
constexpr int SMEM2 = STAGES2 * STAGE2_BYTES + 1024 + 256 + EPI2_WARPS * STG2_WORDS * 4;
static_assert(SMEM2 <= 232448, "shared memory");

__global__ void __launch_bounds__(THREADS2, 1)
mxfp4_gemm256_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_out, const GemmArgs p, int out_by_copy_engine) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    AuxM* aux = (AuxM*)(smem + STAGES2 * STAGE2_BYTES);
    uint32_t* stage_buf = (uint32_t*)(smem + STAGES2 * STAGE2_BYTES + 256);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN2 - 1) / BN2;
    const int num_tiles = num_m * num_n, KB = p.K / 256, KA = p.K / 128;
    const int n_blocks = (p.N + 127) / 128;                           // 128-row blocks of the tiled weight scales

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 1);
        }
        mbar_init(smem_u32(&aux->tfull[0]), 1);
        mbar_init(smem_u32(&aux->tempty[0]), EPI2_WARPS);
        mbar_init(smem_u32(&aux->full[4]), 1);                         // scale-factor set 0 / 1 copied into tensor memory
        mbar_init(smem_u32(&aux->full[5]), 1);
        aux->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&aux->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    volatile int* abort_flag = &aux->abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int mt = t % num_m, nt = t / num_m;
                const bool second = 2 * nt + 1 < n_blocks;            // the tile's weight rows 128-255 exist
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0x1700 + stage)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&aux->full[stage]);
                    mbar_expect_tx(bar, STAGE2_BYTES - (second ? 0 : SF_BYTES));
                    const uint32_t st = smem_u32(smem + stage * STAGE2_BYTES);
                    tma_load_2d(st, &tm_a, kb * KB_BYTES, mt * BM, bar);
                    tma_load_2d(st + A_BYTES, &tm_b, kb * KB_BYTES, nt * BN2, bar);
                    const uint32_t sf = st + A_BYTES + B2_BYTES;
                    bulk_load(sf, p.sfa + ((long)mt * KA + kb * 2) * 512, SF_BYTES, bar);
                    bulk_load(sf + SF_BYTES, p.sfb + ((long)(2 * nt) * KA + kb * 2) * 512, SF_BYTES, bar);
                    if (second)
                        bulk_load(sf + 2 * SF_BYTES, p.sfb + ((long)(2 * nt + 1) * KA + kb * 2) * 512, SF_BYTES, bar);
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                unsigned long long t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 2000000ull) {
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // MMA issuer.  The scale factors' copies into tensor memory are another thread's (warp 2): one thread doing
            // both issued twelve asynchronous instructions per K block, about 700 cycles against 570 of MMA time.
            int stage = 0;
            uint32_t phase = 0, tphase = 0;
            long kbt = 0;                                             // K blocks issued so far, over all tiles
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                // one accumulator: the previous tile must be drained
                if (!mbar_wait(smem_u32(&aux->tempty[0]), tphase ^ 1, abort_flag, 0x1710)) break;
                tc_fence_after();
                for (int kb = 0; kb < KB; ++kb, ++kbt) {
                    const int sfp = (int)(kbt & 1);
                    if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x1720 + stage) ||
                        !mbar_wait(smem_u32(&aux->full[4 + sfp]), (uint32_t)(kbt >> 1) & 1, abort_flag, 0x1740 + sfp)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + stage * STAGE2_BYTES);
                    const uint32_t sfa_t = tmem_base + 256 + sfp * 24, sfb_t = sfa_t + 8;
                    const uint64_t ad = umma_desc_k128(st), bd = umma_desc_k128(st + A_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {                 // K = 64 inputs = 32 bytes per instruction
                        const uint32_t sf_id = (k & 1) * 2;
                        umma_mxf4(tmem_base, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32),
                                  idesc_mxf4(BM, BN2, sf_id, sf_id), sfa_t + (k >> 1) * 4, sfb_t + (k >> 1) * 8,
                                  (kb | k) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&aux->empty[stage]));
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&aux->tfull[0]));
                tphase ^= 1;
            }
        }
    } else if (warp == 2) {
        if (lane == 0) {
            // Scale factors: shared memory -> tensor memory (two alternating sets), one K block ahead of its MMAs.  A
            // set is rewritten only after the MMAs of the K block two before have completed (that block's `empty`).
            int stage = 0;
            uint32_t phase = 0;
            long kbt = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                for (int kb = 0; kb < KB; ++kb, ++kbt) {
                    const int sfp = (int)(kbt & 1);
                    if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x1750 + stage)) {
                        ok = false;
                        break;
                    }
                    if (kbt >= 2) {
                        const long prev = kbt - 2;
                        if (!mbar_wait(smem_u32(&aux->empty[prev % STAGES2]), (uint32_t)(prev / STAGES2) & 1, abort_flag,
                                       0x1760 + sfp)) {
                            ok = false;
                            break;
                        }
                    }
                    tc_fence_after();
                    const uint32_t sf_smem = smem_u32(smem + stage * STAGE2_BYTES) + A_BYTES + B2_BYTES;
                    const uint32_t sfa_t = tmem_base + 256 + sfp * 24, sfb_t = sfa_t + 8;
                    tmem_cp_sf(sfa_t, sf_smem);                               // A rows, K block 0
                    tmem_cp_sf(sfa_t + 4, sf_smem + 512);                     // A rows, K block 1
                    tmem_cp_sf(sfb_t, sf_smem + SF_BYTES);                    // B rows 0-127, K block 0
                    tmem_cp_sf(sfb_t + 4, sf_smem + 2 * SF_BYTES);            // B rows 128-255, K block 0
                    tmem_cp_sf(sfb_t + 8, sf_smem + SF_BYTES + 512);          // B rows 0-127, K block 1
                    tmem_cp_sf(sfb_t + 12, sf_smem + 2 * SF_BYTES + 512);     // B rows 128-255, K block 1
                    tc_commit(smem_u32(&aux->full[4 + sfp]));
                    if (++stage == STAGES2) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else {
        const int q = warp & 3, half = (warp - 3) >> 2;
        uint32_t* stg = stage_buf + (warp - 3) * STG2_WORDS;
        uint32_t tphase = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const int m0 = (t % num_m) * BM, n0 = (t / num_m) * BN2;
            if (!mbar_wait(smem_u32(&aux->tfull[0]), tphase, abort_flag, 0x1730)) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            const int rows_here = p.M - (m0 + q * 32);
            const bool word_ok = p.epi != 0 || ((((uintptr_t)p.out & 3) == 0) && (p.ldo % 2 == 0));
            const int cstep = p.epi == 0 ? 32 : 16;                   // columns per chunk: 16 words either way
            if (out_by_copy_engine) {
                // 32 rows x 64 bytes per chunk, parked densely in shared memory and handed to the copy engine: a plain
                // tile store (bf16) or an add into the fp32 residual (one round-to-nearest add per element; the tensor
                // map ends at row M and column N, so nothing outside is touched).  No load, no store loop.
                if (m0 + q * 32 < p.M) {
#pragma unroll 1
                    for (int c0 = half * (BN2 / 2); c0 < (half + 1) * (BN2 / 2); c0 += cstep) {
                        if (n0 + c0 >= p.N) break;
                        uint32_t wv[16];
                        if (p.epi == 0) {
                            uint32_t r[32];
                            tmem_ld32(lane_addr + c0, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                __nv_bfloat162 b0 =
                                    __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                                wv[j] = *(uint32_t*)&b0;
                            }
                        } else {
                            tmem_ld16(lane_addr + c0, wv);
                            tmem_ld_wait();
                        }
                        // the engine must be done reading the box (the previous chunk) before it is rewritten
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        __syncwarp();
                        uint4* dst = (uint4*)(stg + lane * 16);
#pragma unroll
                        for (int v = 0; v < 4; ++v) dst[v] = make_uint4(wv[4 * v], wv[4 * v + 1], wv[4 * v + 2], wv[4 * v + 3]);
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (p.epi == 0)
                                // (the bf16 output is described as 32-bit words: two columns per element)
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                                             : : "l"(&tm_out), "r"((n0 + c0) >> 1), "r"(m0 + q * 32), "r"(smem_u32(stg)) : "memory");
                            else
                                asm volatile(
                                    "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                                    : : "l"(&tm_out), "r"(n0 + c0), "r"(m0 + q * 32), "r"(smem_u32(stg)) : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = half * (BN2 / 2); c0 < (half + 1) * (BN2 / 2); c0 += cstep) {
                    if (n0 + c0 >= p.N) break;
                    if (p.epi == 0) {
                        uint32_t r[32];
                        tmem_ld32(lane_addr + c0, r);
                        tmem_ld_wait();
    #pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                            stg[lane * 17 + j] = *(uint32_t*)&b0;
                        }
                    } else {
                        uint32_t r[16];
                        tmem_ld16(lane_addr + c0, r);
                        tmem_ld_wait();
    #pragma unroll
                        for (int j = 0; j < 16; ++j) stg[lane * 17 + j] = r[j];
                    }
                    __syncwarp();
                    // half a warp per row: lanes 0-15 row rr, lanes 16-31 row rr + 1; 16 words = 64 contiguous bytes
                    const int w = lane & 15, rsel = lane >> 4;
                    if (p.epi == 0) {
                        const int col = n0 + c0 + 2 * w;
                        for (int rr = rsel; rr < 32 && rr < rows_here; rr += 2) {
                            const long off = (long)(m0 + q * 32 + rr) * p.ldo + col;
                            const uint32_t v = stg[rr * 17 + w];
                            if (word_ok && col + 2 <= p.N) {
                                *(uint32_t*)((__nv_bfloat16*)p.out + off) = v;
                            } else {
                                if (col < p.N) ((uint16_t*)p.out)[off] = (uint16_t)(v & 0xffff);
                                if (col + 1 < p.N) ((uint16_t*)p.out)[off + 1] = (uint16_t)(v >> 16);
                            }
                        }
                    } else {
                        const int col = n0 + c0 + w;
                        if (col < p.N) {
                            float* base = (float*)p.out + (long)(m0 + q * 32) * p.ldo + col;
                            float o[16];
    #pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (rsel + 2 * i < rows_here) o[i] = __ldcg(base + (long)(rsel + 2 * i) * p.ldo);
    #pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (rsel + 2 * i < rows_here)
                                    base[(long)(rsel + 2 * i) * p.ldo] =
                                        __fadd_rn(o[i], __uint_as_float(stg[(rsel + 2 * i) * 17 + w]));
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->tempty[0]));
            tphase ^= 1;
        }
        if (out_by_copy_engine && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ================================================================================================= peak probe
// The FP4 tensor-core rate with no operand traffic: every CTA fills one stage of shared memory once (pattern 0: zeros,
// 1: pseudo-random e2m1 codes), copies unit scale factors (UE8M0 127 = 1.0) into tensor memory, and its MMA thread
// issues `iters` batches of four 128 x 256 x 64 block-scaled MMAs on it.  ops = 2 * 128 * 256 * 256 * iters per SM.
// The ceiling the MXFP4 GEMMs are quoted against (the method of the reference's bench/csrc/mma_peak.cu, on tcgen05
// kind::mxf4).
__global__ void __launch_bounds__(128, 1) mxf4_peak_kernel(int iters, int pattern, unsigned long long* cycles) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    constexpr int OPER = (128 + 256) * 128;                    // A 128 rows + B 256 rows, 128 bytes of K each
    for (int i = threadIdx.x; i < OPER / 4; i += blockDim.x) {
        uint32_t v = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        v ^= v >> 13;
        v *= 0x9E3779B1u;
        ((uint32_t*)smem)[i] = pattern ? (v ^ (v >> 15)) : 0u;
    }
    for (int i = threadIdx.x; i < 512 / 4; i += blockDim.x) ((uint32_t*)(smem + OPER))[i] = 0x7f7f7f7fu;   // scales 1.0
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t sf = smem_u32(smem + OPER);
        const uint32_t sfa_t = tmem_base + 256, sfb_t = sfa_t + 8;
        for (int c = 0; c < 6; ++c) tmem_cp_sf(sfa_t + 4 * c, sf);         // A: 2 K blocks; B: 2 x 2 (rows 0-127, 128-255)
        const uint64_t ad = umma_desc_k128(smem_u32(smem)), bd = umma_desc_k128(smem_u32(smem + 128 * 128));
        const long long c0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t sf_id = (k & 1) * 2;
                umma_mxf4(tmem_base, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32),
                          idesc_mxf4(128, 256, sf_id, sf_id), sfa_t + (k >> 1) * 4, sfb_t + (k >> 1) * 8, (it | k) ? 1u : 0u);
            }
        }
        tc_commit(smem_u32(&done));
        mbar_wait(smem_u32(&done), 0, &abort_flag, 0x1a00);
        if (cycles) cycles[blockIdx.x] = (unsigned long long)(clock64() - c0);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace mxfp4
