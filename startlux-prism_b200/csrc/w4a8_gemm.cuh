// W4A8 GEMM on llama.cpp k-quant weights (Q4_K, Q6_K) with int8 activations scaled per 256 inputs, on the sm_100a
// tensor cores.  Arithmetic of the reference (kernels/w4a8.py:14-24), per 256-input super-block b in increasing b:
//   Q4_K  acc  = sum_g sc[n, g] * (xq . q)_g          mins = sum_g mn[n, g] * S[m, g]            (int32, exact)
//         t = d[n, b] * float(acc); t = fma(-dmin[n, b], float(mins), t); y = fma(a[m, b], t, y)
//   Q6_K  acc  = sum_h sc[n, h] * (xq . q)_h (16-input sub-blocks);  y = fma(a[m, b], d[n, b] * float(acc), y)
// then bf16(y) or out + y.
//
// The tensor core cannot scale per sub-block, so the integer scale is folded into the weights in shared memory, as two
// int8 planes whose weighted sum is exact (the scheme of the reference's Hopper kernel, csrc/w4a8_wgmma.cu:4-16,
// 201-217):
//   Q4_K  sc = s0 + 8 s1 (3 bits each):   plane0 = s0 * q, plane1 = s1 * q  (0..105)     acc = P0 + 8 P1
//   Q6_K  p = sc * q (13 bits signed):    plane0 = p & 63, plane1 = p >> 6  (-64..63)    acc = P0 + 64 P1
// and Q4_K's mins are one more K = 32 MMA per super-block: A = the activation group sums (eight S & 63, eight S >> 6,
// as the quantizer stores them), B = the 6-bit mins placed against the low or the high parts: mins = MLO + 64 MHI.
//
// One CTA per 128 x 64 output tile; warps: 0 TMA producer, 1 MMA issuer, 2-5 expanders (packed weights -> int8 planes
// in the 128-byte-swizzled operand layout), 6-13 epilogue (two per tensor-memory lane quarter: 32 columns each).  Per
// super-block the MMAs fill one of two accumulator sets in tensor memory while the epilogue warps drain the other
// (the floating-point step per 256 inputs).
#pragma once
#include "common.cuh"

namespace w4a8 {

constexpr int BM = 128, BN = 64;
constexpr int KIND_Q4K = 0, KIND_Q6K = 1;
constexpr int THREADS = 15 * 32;               // producer, MMA issuer, 4 expanders, 8 epilogue warps, second MMA issuer

template <int KIND>
struct Cfg {
    static constexpr int A_BYTES = 2 * BM * 128;                         // two 128-byte K blocks of int8 activations
    static constexpr int WQ_BYTES = KIND == KIND_Q4K ? BN * 128 : BN * 256;
    static constexpr int XS_BYTES = KIND == KIND_Q4K ? BM * 16 : 0;
    static constexpr int SC_BYTES = KIND == KIND_Q4K ? BN * 8 : BN * 16;
    static constexpr int MN_BYTES = KIND == KIND_Q4K ? BN * 8 : 0;
    static constexpr int OFF_WQ = A_BYTES;
    static constexpr int OFF_XS = OFF_WQ + WQ_BYTES;
    static constexpr int OFF_SC = OFF_XS + XS_BYTES;
    static constexpr int OFF_MN = OFF_SC + SC_BYTES;
    static constexpr int TX_BYTES = OFF_MN + MN_BYTES;
    static constexpr int STAGE_BYTES = (TX_BYTES + 1023) / 1024 * 1024;
    static constexpr int STAGES = 3;
    static constexpr int BX_BYTES = 2 * 128 * 128;                       // expanded planes: two K blocks x 128 rows
    static constexpr int BM_BYTES = KIND == KIND_Q4K ? 128 * 16 : 0;     // mins operand (one 16-byte K chunk per row)
    static constexpr int EXP_BYTES = BX_BYTES + 2048;
    static constexpr int OFF_EXP = STAGES * STAGE_BYTES;
    static constexpr int OFF_ZERO = OFF_EXP + 2 * EXP_BYTES;             // 2 KB of zeros: the second K chunk of the
    static constexpr int OFF_SCL = OFF_ZERO + 2048;                      //   K = 32 mins operands
    static constexpr int SCL_SLOTS = 8;                                  // ring of per-super-block weight scales
    static constexpr int SCL_BYTES = 512;                                //   (fp32 d[64], then dmin[64])
    static constexpr int OFF_AUX = OFF_SCL + SCL_SLOTS * SCL_BYTES;
    static constexpr int SET_COLS = KIND == KIND_Q4K ? 256 : 128;        // P0 | P1 (| MLO | MHI), 64 columns each
    static constexpr int TMEM_COLS = 2 * SET_COLS;
    static constexpr int SMEM = OFF_AUX + 1024 + 512;
};

struct Aux4 {
    uint64_t full[4], empty[4];
    uint64_t exp_full[2], exp_empty[2];
    uint64_t acc_full[2], acc_empty[2];
    uint64_t sfull[8], sempty[8];
    uint32_t tmem_base;
    int abort_flag;
};

struct Maps {
    CUtensorMap x, wq, xs, sc, mn, d, dm;
};

struct Args {
    const float* a;          // activation scales fp32 [K/256, Ma]
    void* out;
    long ldo;
    const int* n_rows;
    int M, N, K, Ma, epi;
    const uint8_t* sc;       // few-rows Q4_K kernel: the per-row scales read straight from global memory
    const uint8_t* mn;
    const float* d;
    const float* dm;
    // few-rows Q4_K kernel, K split over blockIdx.z: the slices leave their per-super-block terms t_b (exact, the same
    // three roundings) in ws [tile][K/256][16][128]; the tile's last CTA runs the chain y = fma(a_b, t_b, y) in b order
    int split, sb_per_split;
    float* ws;
    int* counters;
};

// K-major operand without swizzle: 8-row x 16-byte core matrices, `sbo` bytes between 8-row groups, `lbo` bytes
// between the two 16-byte K chunks of a K = 32 step.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// Q4_K: 32 packed inputs (16 bytes: low nibbles = inputs 0..15, high nibbles = inputs 16..31) times the 6-bit
// sub-block scale, split s0 + 8 s1, into chunks 2j and 2j + 1 of rows n (plane 0) and 64 + n (plane 1).  A byte
// holds at most 15 * 7 = 105, so one 32-bit multiply scales four values with no carry between bytes.
__device__ __forceinline__ void expand_q4(uint8_t* bx, int n, int j, uint4 w, uint32_t sc) {
    const uint32_t s0 = sc & 7, s1 = sc >> 3;
    const uint32_t lo[4] = {w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu};
    const uint32_t hi[4] = {(w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu,
                            (w.w >> 4) & 0x0F0F0F0Fu};
    *(uint4*)(bx + swz(n, 2 * j)) = make_uint4(lo[0] * s0, lo[1] * s0, lo[2] * s0, lo[3] * s0);
    *(uint4*)(bx + swz(n, 2 * j + 1)) = make_uint4(hi[0] * s0, hi[1] * s0, hi[2] * s0, hi[3] * s0);
    *(uint4*)(bx + swz(64 + n, 2 * j)) = make_uint4(lo[0] * s1, lo[1] * s1, lo[2] * s1, lo[3] * s1);
    *(uint4*)(bx + swz(64 + n, 2 * j + 1)) = make_uint4(hi[0] * s1, hi[1] * s1, hi[2] * s1, hi[3] * s1);
}

// Q6_K: four int8 values q (-32..31) of one sub-block -> the bytes (sc * q) & 63 and (sc * q) >> 6.  u = q + 32 is
// unsigned, two of them sit in 16-bit fields, and u * sc + (4096 - 32 sc) = sc * q + 4096 lies in [0, 8160]: one
// multiply-add per pair, no borrow between the fields.
__device__ __forceinline__ void split_q6(uint32_t w, int sc, uint32_t kc, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = (w ^ 0x20202020u) & 0x3F3F3F3Fu;
    const uint32_t re = (u & 0x00FF00FFu) * (uint32_t)sc + kc;           // values 0 and 2 (+ 4096 each)
    const uint32_t ro = ((u >> 8) & 0x00FF00FFu) * (uint32_t)sc + kc;    // values 1 and 3
    lo = (re & 0x003F003Fu) | ((ro & 0x003F003Fu) << 8);
    const uint32_t he = (((re >> 6) & 0x03FF03FFu) + 0x00C000C0u) & 0x00FF00FFu;   // (p >> 6) as int8: biased - 64
    const uint32_t ho = (((ro >> 6) & 0x03FF03FFu) + 0x00C000C0u) & 0x00FF00FFu;
    hi = he | (ho << 8);
}

template <int KIND>
__global__ void __launch_bounds__(THREADS, 1)
w4a8_kernel(const __grid_constant__ Maps maps, const Args p) {
    using C = Cfg<KIND>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Aux4* aux = (Aux4*)(smem + C::OFF_AUX);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    const int num_m = (p.M + BM - 1) / BM;
    const int m0 = (blockIdx.x % num_m) * BM, n0 = (blockIdx.x / num_m) * BN;
    if (m0 >= live) return;
    const int NSB = p.K / 256;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 1 + 4);                  // MMA commit, expander warps
        }
        for (int i = 0; i < C::SCL_SLOTS; ++i) {
            mbar_init(smem_u32(&aux->sfull[i]), 1);
            mbar_init(smem_u32(&aux->sempty[i]), 8);                     // the 8 epilogue warps
        }
        for (int e = 0; e < 2; ++e) {
            mbar_init(smem_u32(&aux->exp_full[e]), 4);
            mbar_init(smem_u32(&aux->exp_empty[e]), 1);
            mbar_init(smem_u32(&aux->acc_full[e]), 1);
            mbar_init(smem_u32(&aux->acc_empty[e]), 8);
        }
        aux->abort_flag = 0;
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < 2048 / 16; i += THREADS) *(uint4*)(smem + C::OFF_ZERO + i * 16) = make_uint4(0, 0, 0, 0);
    if (warp == 1) {
        tmem_alloc(smem_u32(&aux->tmem_base), C::TMEM_COLS);
        tmem_relinquish();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    volatile int* abort_flag = &aux->abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int b = 0; b < NSB && ok; ++b) {
                if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0xA00 + stage)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&aux->full[stage]);
                mbar_expect_tx(bar, C::TX_BYTES);
                const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
                tma_load_2d(st, &maps.x, b * 256, m0, bar);
                tma_load_2d(st + BM * 128, &maps.x, b * 256 + 128, m0, bar);
                if (KIND == KIND_Q4K) {
                    tma_load_2d(st + C::OFF_WQ, &maps.wq, b * 128, n0, bar);
                    tma_load_2d(st + C::OFF_XS, &maps.xs, m0 * 4, b, bar);
                    tma_load_2d(st + C::OFF_XS + 1024, &maps.xs, m0 * 4 + 256, b, bar);
                    tma_load_2d(st + C::OFF_SC, &maps.sc, n0 * 2, b, bar);
                    tma_load_2d(st + C::OFF_MN, &maps.mn, n0 * 2, b, bar);
                } else {
                    tma_load_2d(st + C::OFF_WQ, &maps.wq, b * 256, n0, bar);
                    tma_load_2d(st + C::OFF_WQ + BN * 128, &maps.wq, b * 256 + 128, n0, bar);
                    tma_load_2d(st + C::OFF_SC, &maps.sc, n0 * 4, b, bar);
                }
                // the super-block's weight scales go to their own, deeper ring: the epilogue reads them long after
                // the operand stage has been handed back
                const int slot = b & (C::SCL_SLOTS - 1);
                if (!mbar_wait(smem_u32(&aux->sempty[slot]), ((b / C::SCL_SLOTS) & 1) ^ 1, abort_flag, 0xA40 + slot)) {
                    ok = false;
                    break;
                }
                const uint32_t sbar = smem_u32(&aux->sfull[slot]);
                mbar_expect_tx(sbar, KIND == KIND_Q4K ? 512 : 256);
                const uint32_t sdst = smem_u32(smem + C::OFF_SCL + slot * C::SCL_BYTES);
                tma_load_2d(sdst, &maps.d, n0, b, sbar);
                if (KIND == KIND_Q4K) tma_load_2d(sdst + 256, &maps.dm, n0, b, sbar);
                if (++stage == C::STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok) {                                       // let armed copies land before the CTA can exit
                unsigned long long t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 2000000ull) {
                }
            }
        }
    } else if (warp == 1 || warp == 14) {
        // ------------------------------------------------------------------ MMA issuers
        // Two threads take alternate super-blocks (warp 1 the even ones, warp 14 the odd ones): one thread's iteration -
        // three barrier waits, nine MMAs, three commits - takes about 1,000 cycles (cycle stamps on a B200) against 580
        // of MMA time.  Super-block b uses accumulator set and operand buffer b & 1, so each thread owns one of each and
        // every set is started (accumulate = 0) and committed by the thread that issues all of its MMAs.
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(BM, 128);
            const int e = warp == 1 ? 0 : 1;
            for (int b = e; b < NSB; b += 2) {
                const int stage = b % C::STAGES;
                const uint32_t phase = (uint32_t)(b / C::STAGES) & 1, eph = (b >> 1) & 1;
                if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0xB00 + stage)) break;
                if (!mbar_wait(smem_u32(&aux->exp_full[e]), eph, abort_flag, 0xB10 + e)) break;
                if (!mbar_wait(smem_u32(&aux->acc_empty[e]), eph ^ 1, abort_flag, 0xB20 + e)) break;
                tc_fence_after();
                const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
                const uint32_t ex = smem_u32(smem + C::OFF_EXP + e * C::EXP_BYTES);
                const uint32_t d = tmem_base + e * C::SET_COLS;
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
                    const uint64_t ad = umma_desc_k128(st + kb * BM * 128);
                    const uint64_t bd = umma_desc_k128(ex + kb * 128 * 128);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_i8(d, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc,
                                (kb | k) ? 1u : 0u);
                }
                if (KIND == KIND_Q4K) {
                    const uint32_t zero = smem_u32(smem + C::OFF_ZERO);
                    const uint32_t xa = st + C::OFF_XS, mb = ex + C::BX_BYTES;
                    umma_i8(d + 128, umma_desc_plain(xa, zero - xa, 128), umma_desc_plain(mb, zero - mb, 128), idesc, 0u);
                }
                tc_commit(smem_u32(&aux->empty[stage]));
                tc_commit(smem_u32(&aux->exp_empty[e]));
                tc_commit(smem_u32(&aux->acc_full[e]));
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ expanders: packed weights -> int8 planes
        const int t = threadIdx.x - 64;
        const int n = t & 63, h = t >> 6;                                // weight row in the tile, K half
        int stage = 0;
        uint32_t phase = 0;
        for (int b = 0; b < NSB; ++b) {
            const int e = b & 1;
            const uint32_t eph = (b >> 1) & 1;
            if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0xC00 + stage)) break;
            if (!mbar_wait(smem_u32(&aux->exp_empty[e]), eph ^ 1, abort_flag, 0xC10 + e)) break;
            const uint8_t* st = smem + stage * C::STAGE_BYTES;
            uint8_t* ex = smem + C::OFF_EXP + e * C::EXP_BYTES;
            uint8_t* bx = ex + h * 128 * 128;
            if (KIND == KIND_Q4K) {
                const uint8_t* wq = st + C::OFF_WQ;                      // 64 rows x 128 bytes, 128-byte swizzle
                const uint2 sc8 = *(const uint2*)(st + C::OFF_SC + n * 8);
                const uint32_t scw = h == 0 ? sc8.x : sc8.y;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 w = *(const uint4*)(wq + swz(n, h * 4 + j));
                    expand_q4(bx, n, j, w, (scw >> (8 * j)) & 0xff);
                }
                const uint2 mn8 = *(const uint2*)(st + C::OFF_MN + n * 8);
                uint8_t* bm = ex + C::BX_BYTES;
                if (h == 0) *(uint4*)(bm + n * 16) = make_uint4(mn8.x, mn8.y, 0, 0);
                else *(uint4*)(bm + (64 + n) * 16) = make_uint4(0, 0, mn8.x, mn8.y);
            } else {
                const uint8_t* wq = st + C::OFF_WQ + h * BN * 128;       // this K half: 64 rows x 128 bytes, swizzled
                const uint2 sc8 = *(const uint2*)(st + C::OFF_SC + n * 16 + h * 8);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int sc = (int)(int8_t)(((i < 4 ? sc8.x : sc8.y) >> (8 * (i & 3))) & 0xff);
                    const uint32_t kc = (uint32_t)(4096 - 32 * sc) * 0x00010001u;
                    const uint4 w = *(const uint4*)(wq + swz(n, i));
                    uint4 lo, hi;
                    split_q6(w.x, sc, kc, lo.x, hi.x);
                    split_q6(w.y, sc, kc, lo.y, hi.y);
                    split_q6(w.z, sc, kc, lo.z, hi.z);
                    split_q6(w.w, sc, kc, lo.w, hi.w);
                    *(uint4*)(bx + swz(n, i)) = lo;
                    *(uint4*)(bx + swz(64 + n, i)) = hi;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&aux->exp_full[e]));
                mbar_arrive(smem_u32(&aux->empty[stage]));
            }
            if (++stage == C::STAGES) {
                stage = 0;
                phase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: 8 warps, 32 rows x 32 columns each
        const int q = warp & 3, ch = (warp - 6) >> 2;
        const int ml = q * 32 + lane;                                    // row in the tile
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + ch * 32;
        // two output columns per instruction (packed fp32 multiply and fused multiply-add: each half rounds like its
        // scalar twin, and the reference's definition has these fmas, so nothing is contracted that was not one)
        float2 y2[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) y2[j] = make_float2(0.0f, 0.0f);
        bool ok = true;
        // this row's activation scale of the coming super-block: loaded one super-block ahead (an L2 round trip)
        float am_next = (NSB > 0 && m0 + ml < p.Ma) ? __ldg(p.a + m0 + ml) : 0.0f;
        for (int b = 0; b < NSB; ++b) {
            const int e = b & 1;
            const uint32_t eph = (b >> 1) & 1;
            const int slot = b & (C::SCL_SLOTS - 1);
            const float2* dv = (const float2*)(smem + C::OFF_SCL + slot * C::SCL_BYTES) + ch * 16;
            const float2* dmv = dv + 32;
            const float am = am_next;
            if (b + 1 < NSB && m0 + ml < p.Ma) am_next = __ldg(p.a + (long)(b + 1) * p.Ma + m0 + ml);
            const float2 am2 = make_float2(am, am);
            if (!mbar_wait(smem_u32(&aux->acc_full[e]), eph, abort_flag, 0xD00 + e) ||
                !mbar_wait(smem_u32(&aux->sfull[slot]), (b / C::SCL_SLOTS) & 1, abort_flag, 0xD20 + slot)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t set = lane_base + e * C::SET_COLS;
#pragma unroll
            for (int c = 0; c < 32; c += 16) {
                uint32_t p0[16], p1[16];
                tmem_ld16(set + c, p0);
                tmem_ld16(set + 64 + c, p1);
                if (KIND == KIND_Q4K) {
                    uint32_t l0[16], l1[16];
                    tmem_ld16(set + 128 + c, l0);
                    tmem_ld16(set + 192 + c, l1);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float2 fa = make_float2(__int2float_rn((int)p0[j] + 8 * (int)p1[j]),
                                                      __int2float_rn((int)p0[j + 1] + 8 * (int)p1[j + 1]));
                        const float2 fm = make_float2(__int2float_rn((int)l0[j] + 64 * (int)l1[j]),
                                                      __int2float_rn((int)l0[j + 1] + 64 * (int)l1[j + 1]));
                        const float2 d2 = dv[(c + j) >> 1], dm2 = dmv[(c + j) >> 1];
                        float2 t = __fmul2_rn(d2, fa);
                        t = __ffma2_rn(make_float2(-dm2.x, -dm2.y), fm, t);
                        y2[(c + j) >> 1] = __ffma2_rn(am2, t, y2[(c + j) >> 1]);
                    }
                } else {
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float2 fa = make_float2(__int2float_rn((int)p0[j] + 64 * (int)p1[j]),
                                                      __int2float_rn((int)p0[j + 1] + 64 * (int)p1[j + 1]));
                        y2[(c + j) >> 1] = __ffma2_rn(am2, __fmul2_rn(dv[(c + j) >> 1], fa), y2[(c + j) >> 1]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&aux->acc_empty[e]));
                mbar_arrive(smem_u32(&aux->sempty[slot]));
            }
        }
        float y[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            y[2 * j] = y2[j].x;
            y[2 * j + 1] = y2[j].y;
        }
        if (ok) {
            // every MMA has completed (the last accumulator set was full): the expanded-operand buffers are free and
            // serve as the transpose staging of the coalesced store (32 rows x 33 words per warp)
            uint32_t* stg = (uint32_t*)(smem + C::OFF_EXP) + (warp - 6) * (32 * 33);
            const int rows_here = live - (m0 + q * 32);
            const int ncol0 = n0 + ch * 32;
            if (p.epi == 0) {
                const bool word_ok = (((uintptr_t)p.out & 3) == 0) && (p.ldo % 2 == 0);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
                    stg[lane * 33 + j] = *(uint32_t*)&b2;
                }
                __syncwarp();
                __nv_bfloat16* o = (__nv_bfloat16*)p.out;
                for (int rr = 0; rr < 32 && rr < rows_here; ++rr) {
                    const long off = (long)(m0 + q * 32 + rr) * p.ldo + ncol0;
                    if (lane < 16) {
                        const uint32_t v = stg[rr * 33 + lane];
                        const int col = ncol0 + 2 * lane;
                        if (word_ok && col + 2 <= p.N) {
                            *(uint32_t*)(o + off + 2 * lane) = v;
                        } else {
                            if (col < p.N) ((uint16_t*)o)[off + 2 * lane] = (uint16_t)(v & 0xffff);
                            if (col + 1 < p.N) ((uint16_t*)o)[off + 2 * lane + 1] = (uint16_t)(v >> 16);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __float_as_uint(y[j]);
                __syncwarp();
                if (ncol0 + lane < p.N) {
                    float* base = (float*)p.out + (long)(m0 + q * 32) * p.ldo + ncol0 + lane;
                    float o[32];
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr)
                        if (rr < rows_here) o[rr] = __ldcg(base + (long)rr * p.ldo);
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr)
                        if (rr < rows_here) base[(long)rr * p.ldo] = __fadd_rn(o[rr], __uint_as_float(stg[rr * 33 + lane]));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace w4a8
