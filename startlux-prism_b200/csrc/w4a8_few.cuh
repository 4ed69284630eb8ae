// W4A8 for few activation rows (decode, M <= 64 in tiles of 16 rows): the operands of w4a8_gemm.cuh swapped, so that
// the packed weights - the bytes that bound this shape - fill the tensor core's 128-row operand and nothing is padded.
// Same arithmetic, bit for bit (kernels/w4a8.py:14-24; the integer part is exact, the fp32 step per 256 inputs is the
// same three roundings in the same order).
//
//   Q4_K  tile = 128 weight rows.  The expanders only split nibbles (no scale is folded in): every 32-input sub-block
//         is one K = 32 MMA of its own, 128 x 16, written to its own 16 accumulator columns.  The thread that owns a
//         weight row (one tensor-memory lane) then applies that row's eight 6-bit scales with integer multiplies,
//         acc = sum_g sc[g] * D[g], and takes the mins from the activation group sums with dot-product instructions,
//         mins = sum_g mn[g] * S[m, g] - no second plane, no extra MMA.
//   Q6_K  tile = 64 weight rows as two int8 planes of sc * q (p & 63 and p >> 6, the scheme of w4a8_gemm.cuh): lanes
//         0-63 hold P0, lanes 64-127 hold P1; the upper epilogue warps hand P1 to the lower ones through shared memory:
//         acc = P0 + 64 P1.
//
// Warps: 0 TMA producer, 1 MMA issuer, 2-9 expanders, 10-17 epilogue (two per tensor-memory lane quarter, eight
// activation rows each).  Four accumulator sets in tensor memory, so the MMAs of a super-block never wait for the
// floating-point step of the one two before it.  The per-super-block scales (weight scales and
// mins, d, dmin, the activation group sums) travel in their own ring of 8 slots, because the epilogue reads them long
// after the operand stage went back to the producer.
#pragma once
#include "common.cuh"
#include "w4a8_gemm.cuh"

namespace w4a8 {

constexpr int FEW_NB = 16;                       // activation rows per CTA = the MMA's N
constexpr int FEW_THREADS = 18 * 32;
constexpr int FEW_SETS = 4;                      // accumulator sets in tensor memory

template <int KIND>
struct FewCfg {
    static constexpr int TILE_N = KIND == KIND_Q4K ? 128 : 64;           // weight rows per CTA
    static constexpr int WQ_BYTES = KIND == KIND_Q4K ? 128 * 128 : 2 * 64 * 128;
    static constexpr int X_BYTES = 2 * FEW_NB * 128;                     // two 128-byte K blocks of int8 activations
    static constexpr int OFF_X = WQ_BYTES;
    static constexpr int TX_BYTES = WQ_BYTES + X_BYTES;
    static constexpr int STAGE_BYTES = (TX_BYTES + 1023) / 1024 * 1024;
    static constexpr int STAGES = 4;
    static constexpr int EXP_BYTES = 2 * 128 * 128;                      // expanded operand: two K blocks x 128 rows
    static constexpr int OFF_EXP = STAGES * STAGE_BYTES;
    // scale ring slot
    static constexpr int SC_BYTES = KIND == KIND_Q4K ? 128 * 8 : 64 * 16;
    static constexpr int MN_BYTES = KIND == KIND_Q4K ? 128 * 8 : 0;
    static constexpr int D_BYTES = TILE_N * 4;
    static constexpr int DM_BYTES = KIND == KIND_Q4K ? TILE_N * 4 : 0;
    static constexpr int XS_BYTES = KIND == KIND_Q4K ? FEW_NB * 16 : 0;
    static constexpr int SOFF_MN = SC_BYTES;
    static constexpr int SOFF_D = SOFF_MN + MN_BYTES;
    static constexpr int SOFF_DM = SOFF_D + D_BYTES;
    static constexpr int SOFF_XS = SOFF_DM + DM_BYTES;
    static constexpr int SCL_TX = SOFF_XS + XS_BYTES;
    static constexpr int SCL_BYTES = (SCL_TX + 127) / 128 * 128;
    static constexpr int SCL_SLOTS = 8;
    static constexpr int OFF_SCL = OFF_EXP + 2 * EXP_BYTES;
    static constexpr int XCHG_PITCH = 20;                                // words per row: 16 values, conflict-free 16-byte reads
    static constexpr int XCHG_BYTES = KIND == KIND_Q6K ? 64 * XCHG_PITCH * 4 : 0;
    static constexpr int OFF_XCHG = OFF_SCL + SCL_SLOTS * SCL_BYTES;
    static constexpr int OFF_AUX = OFF_XCHG + FEW_SETS * XCHG_BYTES;
    static constexpr int SET_COLS = KIND == KIND_Q4K ? 8 * FEW_NB : 32;  // accumulator columns per super-block
    static constexpr int TMEM_COLS = FEW_SETS * SET_COLS;
    static constexpr int SMEM = OFF_AUX + 512 + 1024;
};

struct AuxFew {
    uint64_t full[4], empty[4];
    uint64_t exp_full[2];
    uint64_t acc_full[FEW_SETS], acc_empty[FEW_SETS];
    uint64_t xfull[FEW_SETS * 2];
    uint64_t sfull[8], sempty[8];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};

struct FewMaps {
    CUtensorMap x, wq, xs, sc, mn, d, dm;
};

template <int KIND>
__global__ void __launch_bounds__(FEW_THREADS, 1)
w4a8_few_kernel(const __grid_constant__ FewMaps maps, const Args p) {
    using C = FewCfg<KIND>;
    constexpr int NB = FEW_NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    AuxFew* aux = (AuxFew*)(smem + C::OFF_AUX);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    const int m0 = blockIdx.x * NB, n0 = blockIdx.y * C::TILE_N;
    if (m0 >= live) return;                                              // whole CTA, before any barrier or allocation
    // this CTA's super-blocks: [b0, b0 + NSB) of the row's NSBT (K split over blockIdx.z: Q6_K only, see TmCfg's kernel)
    const int NSBT = p.K / 256;
    const bool split = KIND == KIND_Q6K && p.split > 1;
    const int b0 = split ? (int)blockIdx.z * p.sb_per_split : 0;
    const int NSB = split ? (b0 + p.sb_per_split < NSBT ? p.sb_per_split : NSBT - b0) : NSBT;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 8 + 8);                  // expander warps (weights), epilogue warps (the MMAs that
                                                                         //   read the activations have completed)
        }
        for (int i = 0; i < C::SCL_SLOTS; ++i) {
            mbar_init(smem_u32(&aux->sfull[i]), 1);
            mbar_init(smem_u32(&aux->sempty[i]), KIND == KIND_Q4K ? 8 : 4);
        }
        for (int e = 0; e < 2; ++e) mbar_init(smem_u32(&aux->exp_full[e]), 8);
        for (int a = 0; a < FEW_SETS; ++a) {
            mbar_init(smem_u32(&aux->acc_full[a]), 1);
            mbar_init(smem_u32(&aux->acc_empty[a]), 8);
            mbar_init(smem_u32(&aux->xfull[2 * a]), 2);
            mbar_init(smem_u32(&aux->xfull[2 * a + 1]), 2);
        }
        aux->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&aux->tmem_base), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    volatile int* abort_flag = &aux->abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // weights are read once - unless more row tiles (their CTAs are neighbours in launch order) want them from L2
            const uint64_t pol_w = gridDim.x == 1 ? policy_evict_first() : policy_evict_last();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int b = 0; b < NSB && ok; ++b) {
                if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0xE00 + stage)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&aux->full[stage]);
                mbar_expect_tx(bar, C::TX_BYTES);
                const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
                if (KIND == KIND_Q4K) {
                    tma_load_2d_hint(st, &maps.wq, (b0 + b) * 128, n0, bar, pol_w);
                } else {
                    tma_load_2d_hint(st, &maps.wq, (b0 + b) * 256, n0, bar, pol_w);
                    tma_load_2d_hint(st + 64 * 128, &maps.wq, (b0 + b) * 256 + 128, n0, bar, pol_w);
                }
                tma_load_2d(st + C::OFF_X, &maps.x, (b0 + b) * 256, m0, bar);
                tma_load_2d(st + C::OFF_X + NB * 128, &maps.x, (b0 + b) * 256 + 128, m0, bar);
                const int slot = b & (C::SCL_SLOTS - 1);
                if (!mbar_wait(smem_u32(&aux->sempty[slot]), ((b / C::SCL_SLOTS) & 1) ^ 1, abort_flag, 0xE40 + slot)) {
                    ok = false;
                    break;
                }
                const uint32_t sbar = smem_u32(&aux->sfull[slot]);
                mbar_expect_tx(sbar, C::SCL_TX);
                const uint32_t sdst = smem_u32(smem + C::OFF_SCL + slot * C::SCL_BYTES);
                if (KIND == KIND_Q4K) {
                    tma_load_2d(sdst, &maps.sc, n0 * 2, b0 + b, sbar);
                    tma_load_2d(sdst + C::SOFF_MN, &maps.mn, n0 * 2, b0 + b, sbar);
                    tma_load_2d(sdst + C::SOFF_D, &maps.d, n0, b0 + b, sbar);
                    tma_load_2d(sdst + C::SOFF_DM, &maps.dm, n0, b0 + b, sbar);
                    tma_load_2d(sdst + C::SOFF_XS, &maps.xs, m0 * 4, b0 + b, sbar);
                } else {
                    tma_load_2d(sdst, &maps.sc, n0 * 4, b0 + b, sbar);
                    tma_load_2d(sdst + C::SOFF_D, &maps.d, n0, b0 + b, sbar);
                }
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
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(128, NB);
            int stage = 0;
            uint32_t phase = 0;
            // An mbarrier test keeps this thread waiting about 200 cycles for its answer, and this thread's instruction
            // stream is what bounds the kernel: the tests of the NEXT super-block's barriers are issued before the
            // current MMAs and read after them, and one commit per super-block tells everybody (epilogue: accumulators
            // ready; expanders: operand buffer free; producer, through the epilogue warps: stage free).
            bool r_acc = true;                                           // fresh accumulator sets are free
            bool r_full = NSB > 0 && mbar_test(smem_u32(&aux->full[0]), 0);
            bool r_exp = NSB > 0 && mbar_test(smem_u32(&aux->exp_full[0]), 0);
            for (int b = 0; b < NSB; ++b) {
                const int e = b & 1, a = b & (FEW_SETS - 1);
                const uint32_t eph = (b >> 1) & 1, aph = (b / FEW_SETS) & 1;
                if (!r_acc && !mbar_wait(smem_u32(&aux->acc_empty[a]), aph ^ 1, abort_flag, 0xF20 + a)) break;
                if (!r_full && !mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0xF00 + stage)) break;
                if (!r_exp && !mbar_wait(smem_u32(&aux->exp_full[e]), eph, abort_flag, 0xF10 + e)) break;
                const int nstage = stage + 1 == C::STAGES ? 0 : stage + 1;
                const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
                const int ne = e ^ 1, na = (b + 1) & (FEW_SETS - 1);
                const uint32_t neph = ((b + 1) >> 1) & 1, naph = ((b + 1) / FEW_SETS) & 1;
                r_acc = mbar_test(smem_u32(&aux->acc_empty[na]), naph ^ 1);
                r_full = mbar_test(smem_u32(&aux->full[nstage]), nphase);
                r_exp = mbar_test(smem_u32(&aux->exp_full[ne]), neph);
                tc_fence_after();
                const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
                const uint32_t ex = smem_u32(smem + C::OFF_EXP + e * C::EXP_BYTES);
                const uint32_t d = tmem_base + a * C::SET_COLS;
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
                    const uint64_t ad = umma_desc_k128(ex + kb * 128 * 128);
                    const uint64_t bd = umma_desc_k128(st + C::OFF_X + kb * NB * 128);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (KIND == KIND_Q4K)                            // sub-block kb * 4 + k gets its own columns
                            umma_i8(d + (kb * 4 + k) * NB, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32),
                                    idesc, 0u);
                        else
                            umma_i8(d, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc,
                                    (kb | k) ? 1u : 0u);
                    }
                }
                tc_commit(smem_u32(&aux->acc_full[a]));
                stage = nstage;
                phase = nphase;
            }
        }
    } else if (warp < 10) {
        // ------------------------------------------------------------------ expanders: packed weights -> int8 operand
        const int t = threadIdx.x - 64;
        int stage = 0;
        uint32_t phase = 0;
        for (int b = 0; b < NSB; ++b) {
            const int e = b & 1;
            if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x1000 + stage)) break;
            // buffer e was last read by the MMAs of super-block b - 2: their commit completed that accumulator set
            if (b >= 2 && !mbar_wait(smem_u32(&aux->acc_full[(b - 2) & (FEW_SETS - 1)]), ((b - 2) / FEW_SETS) & 1, abort_flag,
                                     0x1010 + e)) break;
            const uint8_t* st = smem + stage * C::STAGE_BYTES;
            uint8_t* ex = smem + C::OFF_EXP + e * C::EXP_BYTES;
            if (KIND == KIND_Q4K) {
                const int n = t & 127, h = t >> 7;                       // weight row, K half (= 128-byte K block)
                uint8_t* bx = ex + h * 128 * 128;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 w = *(const uint4*)(st + swz(n, h * 4 + j));
                    *(uint4*)(bx + swz(n, 2 * j)) =
                        make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu);
                    *(uint4*)(bx + swz(n, 2 * j + 1)) = make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu,
                                                                   (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
                }
            } else {
                const int n = t & 63, h = (t >> 6) & 1, part = t >> 7;   // weight row, K half, four of its eight sub-blocks
                const uint8_t* wq = st + h * 64 * 128;
                uint8_t* bx = ex + h * 128 * 128;
                // the sub-block scales of this row: the scale ring's slot of super-block b (it was requested right
                // after this stage, and is waited for here)
                const int slot = b & (C::SCL_SLOTS - 1);
                if (!mbar_wait(smem_u32(&aux->sfull[slot]), (b / C::SCL_SLOTS) & 1, abort_flag, 0x1020 + slot)) break;
                const uint32_t scq = *(const uint32_t*)(smem + C::OFF_SCL + slot * C::SCL_BYTES + n * 16 + h * 8 + part * 4);
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const int i = part * 4 + ii;
                    const int sc = (int)(int8_t)((scq >> (8 * ii)) & 0xff);
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
        // ------------------------------------------------------------------ epilogue: one weight row, eight rows of x per thread
        const int q = warp & 3, hsel = (warp - 10) >> 2;
        const int c0 = hsel * 8;                                         // this warp's activation rows: m0 + c0 .. + 7
        const int nl = q * 32 + lane;                                    // tensor-memory lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool rows_live = m0 + c0 < live;                           // warp-uniform
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = 0.0f;
        bool ok = true;
        // lane l carries the activation scale of row m0 + (l & 15) of the coming super-block
        const int ml = m0 + (lane & 15);
        float am_next = (NSB > 0 && ml < p.Ma) ? __ldg(p.a + (long)b0 * p.Ma + ml) : 0.0f;
        if (KIND == KIND_Q4K) {
            const int n = n0 + nl;
            for (int b = 0; b < NSB; ++b) {
                const int a = b & (FEW_SETS - 1);
                const uint32_t aph = (b / FEW_SETS) & 1;
                const int slot = b & (C::SCL_SLOTS - 1);
                const float am_l = am_next;
                if (b + 1 < NSB && ml < p.Ma) am_next = __ldg(p.a + (long)(b0 + b + 1) * p.Ma + ml);
                if (!mbar_wait(smem_u32(&aux->sfull[slot]), (b / C::SCL_SLOTS) & 1, abort_flag, 0x1120 + slot) ||
                    !mbar_wait(smem_u32(&aux->acc_full[a]), aph, abort_flag, 0x1100 + a)) {
                    ok = false;
                    break;
                }
                if (lane == 0) mbar_arrive(smem_u32(&aux->empty[b % C::STAGES]));   // the MMAs are done with the stage
                tc_fence_after();
                if (rows_live) {
                    const uint8_t* sl = smem + C::OFF_SCL + slot * C::SCL_BYTES;
                    const uint2 sc8 = *(const uint2*)(sl + nl * 8);
                    const uint2 mn8 = *(const uint2*)(sl + C::SOFF_MN + nl * 8);
                    const float dv = *(const float*)(sl + C::SOFF_D + nl * 4);
                    const float ndm = -*(const float*)(sl + C::SOFF_DM + nl * 4);
                    int scg[8];
#pragma unroll
                    for (int g = 0; g < 8; ++g) scg[g] = (int)(((g < 4 ? sc8.x : sc8.y) >> (8 * (g & 3))) & 0xff);
                    const uint32_t set = lane_base + a * C::SET_COLS;
                    uint32_t r[8][8];
#pragma unroll
                    for (int g = 0; g < 8; ++g) tmem_ld8(set + g * NB + c0, r[g]);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        int acc = scg[0] * (int)r[0][j];
#pragma unroll
                        for (int g = 1; g < 8; ++g) acc += scg[g] * (int)r[g][j];
                        const uint4 s16 = *(const uint4*)(sl + C::SOFF_XS + (c0 + j) * 16);   // eight S & 63, eight S >> 6
                        const int mlo = __dp4a((int)mn8.x, (int)s16.x, __dp4a((int)mn8.y, (int)s16.y, 0));
                        const int mhi = __dp4a((int)mn8.x, (int)s16.z, __dp4a((int)mn8.y, (int)s16.w, 0));
                        const int mins = mlo + 64 * mhi;
                        const float am = __shfl_sync(0xffffffffu, am_l, c0 + j);
                        float t = __fmul_rn(dv, __int2float_rn(acc));
                        t = __fmaf_rn(ndm, __int2float_rn(mins), t);
                        y[j] = __fmaf_rn(am, t, y[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&aux->acc_empty[a]));
                    mbar_arrive(smem_u32(&aux->sempty[slot]));
                }
            }
            if (ok && n < p.N) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int m = m0 + c0 + j;
                    if (m < live) {
                        if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(y[j]);
                        else {
                            float* o = (float*)p.out + (long)m * p.ldo + n;
                            *o = __fadd_rn(*o, y[j]);
                        }
                    }
                }
            }
        } else {
            const bool upper = q >= 2;                                   // lanes 64-127: plane 1 of weight row nl - 64
            const int row = nl & 63;
            const int n = n0 + row;
            const int tile = blockIdx.y * gridDim.x + blockIdx.x;
            float* ws_tile = split ? p.ws + (long)tile * NSBT * NB * 64 : nullptr;
            for (int b = 0; b < NSB; ++b) {
                const int a = b & (FEW_SETS - 1);
                const uint32_t aph = (b / FEW_SETS) & 1;
                const int slot = b & (C::SCL_SLOTS - 1);
                const float am_l = am_next;
                if (b + 1 < NSB && ml < p.Ma) am_next = __ldg(p.a + (long)(b0 + b + 1) * p.Ma + ml);
                if (!mbar_wait(smem_u32(&aux->acc_full[a]), aph, abort_flag, 0x1200 + a)) {
                    ok = false;
                    break;
                }
                if (lane == 0) mbar_arrive(smem_u32(&aux->empty[b % C::STAGES]));   // the MMAs are done with the stage
                tc_fence_after();
                uint32_t pv[8];
                if (rows_live) {
                    tmem_ld8(lane_base + a * C::SET_COLS + c0, pv);
                    tmem_ld_wait();
                }
                uint32_t* xr = (uint32_t*)(smem + C::OFF_XCHG + a * C::XCHG_BYTES) + row * C::XCHG_PITCH + c0;
                if (upper) {
                    if (rows_live) {
                        *(uint4*)xr = make_uint4(pv[0], pv[1], pv[2], pv[3]);
                        *(uint4*)(xr + 4) = make_uint4(pv[4], pv[5], pv[6], pv[7]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(smem_u32(&aux->xfull[2 * a + hsel]));
                        mbar_arrive(smem_u32(&aux->acc_empty[a]));
                    }
                } else {
                    if (!mbar_wait(smem_u32(&aux->sfull[slot]), (b / C::SCL_SLOTS) & 1, abort_flag, 0x1220 + slot) ||
                        !mbar_wait(smem_u32(&aux->xfull[2 * a + hsel]), aph, abort_flag, 0x1230 + a)) {
                        ok = false;
                        break;
                    }
                    if (rows_live) {
                        const float dv = *(const float*)(smem + C::OFF_SCL + slot * C::SCL_BYTES + C::SOFF_D + row * 4);
                        const uint4 h0 = *(const uint4*)xr, h1 = *(const uint4*)(xr + 4);
                        const uint32_t h8[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int acc = (int)pv[j] + 64 * (int)h8[j];
                            const float am = __shfl_sync(0xffffffffu, am_l, c0 + j);
                            const float tb = __fmul_rn(dv, __int2float_rn(acc));
                            if (split) ws_tile[((long)(b0 + b) * NB + c0 + j) * 64 + row] = tb;   // the chain runs later
                            else y[j] = __fmaf_rn(am, tb, y[j]);
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(smem_u32(&aux->acc_empty[a]));
                        mbar_arrive(smem_u32(&aux->sempty[slot]));
                    }
                }
            }
            if (split) {
                // the hand-over of TmCfg's kernel: slices' terms in the workspace, the tile's last CTA runs the chain
                __threadfence();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (threadIdx.x == 320) {
                    const int old = ok ? atomicAdd(p.counters + tile, 1) : -1;
                    aux->is_last = (old == p.split - 1);
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (!aux->is_last) ok = false;
                else {
                    __threadfence();
                    if (rows_live && !upper) {
                        for (int b = 0; b < NSBT; ++b) {
                            const float am_l = ml < p.Ma ? __ldg(p.a + (long)b * p.Ma + ml) : 0.0f;
                            float tv[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) tv[j] = __ldcg(ws_tile + ((long)b * NB + c0 + j) * 64 + row);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                y[j] = __fmaf_rn(__shfl_sync(0xffffffffu, am_l, c0 + j), tv[j], y[j]);
                        }
                    }
                    if (threadIdx.x == 320) p.counters[tile] = 0;
                }
            }
            if (ok && !upper && n < p.N) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int m = m0 + c0 + j;
                    if (m < live) {
                        if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(y[j]);
                        else {
                            float* o = (float*)p.out + (long)m * p.ldo + n;
                            *o = __fadd_rn(*o, y[j]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ================================================================================================ Q4_K, operand in tensor memory
// The same Q4_K arithmetic with the expanded weights handed to the tensor core through TENSOR memory instead of shared
// memory (tcgen05.mma with its A operand in tensor memory): an expander thread owns a weight row (= lane), splits its
// nibbles in registers and stores them with tcgen05.st.  Shared memory then only carries the packed bytes (written once
// by the bulk copy, read once by the expanders) - a third of the traffic of the staged version, which was what bounded
// it - and the 32 KB operand buffers become eight more stages of packed weights in flight.
//   tensor memory: 3 accumulator sets x 128 columns | 2 operand buffers x 64 columns (256 inputs x 8 bit per lane)
//   shared memory: 8 stages x 16 KB packed weights | 8 slots x 5 KB (activations 4 KB, their group sums)
// One thread issues every bulk copy, and each copy costs it about 150 cycles: the per-row scales (sc, mn, d, dmin)
// are therefore not copied into shared memory at all - the epilogue thread of a weight row reads its own 24 bytes per
// super-block straight from global memory, one super-block ahead (a warp's reads are contiguous).
struct TmCfg {
    static constexpr int W_BYTES = 128 * 128;
    static constexpr int W_STAGES = 8;
    static constexpr int SOFF_XS = 2 * FEW_NB * 128;                     // after the two activation K blocks
    static constexpr int SCL_TX = SOFF_XS + FEW_NB * 16;
    static constexpr int SCL_BYTES = 5120;
    static constexpr int SCL_SLOTS = 8;
    static constexpr int OFF_SCL = W_STAGES * W_BYTES;
    static constexpr int OFF_AUX = OFF_SCL + SCL_SLOTS * SCL_BYTES;
    static constexpr int SMEM = OFF_AUX + 512 + 1024;
    static constexpr int D_SETS = 3, SET_COLS = 8 * FEW_NB;
    static constexpr int A_BUFS = 2, A_COLS = 64, A_COL0 = D_SETS * SET_COLS;
    static constexpr int TMEM_COLS = 512;
};
static_assert(TmCfg::SCL_TX <= TmCfg::SCL_BYTES, "scale slot");
static_assert(TmCfg::A_COL0 + TmCfg::A_BUFS * TmCfg::A_COLS <= 512, "tensor memory");

struct AuxTm {
    uint64_t wfull[8], wempty[8];
    uint64_t sfull[8], sempty[8];
    uint64_t afull[2];
    uint64_t acc_full[3], acc_empty[3];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};

// SPLIT: K split over blockIdx.z (two instantiations: the unsplit one keeps its registers for the fp32 chain).
template <bool SPLIT>
__global__ void __launch_bounds__(FEW_THREADS, 1)
w4a8_few_q4k_tm_kernel(const __grid_constant__ FewMaps maps, const Args p) {
    using C = TmCfg;
    constexpr int NB = FEW_NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    AuxTm* aux = (AuxTm*)(smem + C::OFF_AUX);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    const int m0 = blockIdx.x * NB, n0 = blockIdx.y * 128;
    if (m0 >= live) return;                                              // whole CTA, before any barrier or allocation
    // this CTA's super-blocks: [b0, b0 + NSB) of the row's NSBT (all of them without a K split)
    const int NSBT = p.K / 256;
    const int b0 = SPLIT ? (int)blockIdx.z * p.sb_per_split : 0;
    const int NSB = SPLIT ? (b0 + p.sb_per_split < NSBT ? p.sb_per_split : NSBT - b0) : NSBT;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::W_STAGES; ++s) {
            mbar_init(smem_u32(&aux->wfull[s]), 1);
            mbar_init(smem_u32(&aux->wempty[s]), 8);                     // the expander warps
        }
        for (int i = 0; i < C::SCL_SLOTS; ++i) {
            mbar_init(smem_u32(&aux->sfull[i]), 1);
            mbar_init(smem_u32(&aux->sempty[i]), 8);                     // the epilogue warps (the MMAs that read the
        }                                                                //   slot's activations have completed by then)
        for (int e = 0; e < C::A_BUFS; ++e) mbar_init(smem_u32(&aux->afull[e]), 8);
        for (int a = 0; a < C::D_SETS; ++a) {
            mbar_init(smem_u32(&aux->acc_full[a]), 1);
            mbar_init(smem_u32(&aux->acc_empty[a]), 8);
        }
        aux->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&aux->tmem_base), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    volatile int* abort_flag = &aux->abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint64_t pol_w = gridDim.x == 1 ? policy_evict_first() : policy_evict_last();
            bool ok = true;
            for (int b = 0; b < NSB && ok; ++b) {
                const int ws = b & (C::W_STAGES - 1), slot = b & (C::SCL_SLOTS - 1);
                const uint32_t ph = (b >> 3) & 1;
                if (!mbar_wait(smem_u32(&aux->wempty[ws]), ph ^ 1, abort_flag, 0x1300 + ws)) {
                    ok = false;
                    break;
                }
                const uint32_t wbar = smem_u32(&aux->wfull[ws]);
                mbar_expect_tx(wbar, C::W_BYTES);
                tma_load_2d_hint(smem_u32(smem + ws * C::W_BYTES), &maps.wq, (b0 + b) * 128, n0, wbar, pol_w);
                if (!mbar_wait(smem_u32(&aux->sempty[slot]), ph ^ 1, abort_flag, 0x1340 + slot)) {
                    ok = false;
                    break;
                }
                const uint32_t sbar = smem_u32(&aux->sfull[slot]);
                mbar_expect_tx(sbar, C::SCL_TX);
                const uint32_t sdst = smem_u32(smem + C::OFF_SCL + slot * C::SCL_BYTES);
                tma_load_2d(sdst, &maps.x, (b0 + b) * 256, m0, sbar);
                tma_load_2d(sdst + NB * 128, &maps.x, (b0 + b) * 256 + 128, m0, sbar);
                tma_load_2d(sdst + C::SOFF_XS, &maps.xs, m0 * 4, b0 + b, sbar);
            }
            if (!ok) {                                       // let armed copies land before the CTA can exit
                unsigned long long t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 2000000ull) {
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(128, NB);
            int a = 0;
            uint32_t aph = 0;
            bool r_acc = true;                                           // fresh accumulator sets are free
            bool r_a = NSB > 0 && mbar_test(smem_u32(&aux->afull[0]), 0);
            bool r_s = NSB > 0 && mbar_test(smem_u32(&aux->sfull[0]), 0);
            for (int b = 0; b < NSB; ++b) {
                const int e = b & 1, slot = b & (C::SCL_SLOTS - 1);
                const uint32_t eph = (b >> 1) & 1, sph = (b >> 3) & 1;
                if (!r_acc && !mbar_wait(smem_u32(&aux->acc_empty[a]), aph ^ 1, abort_flag, 0x1420 + a)) break;
                if (!r_s && !mbar_wait(smem_u32(&aux->sfull[slot]), sph, abort_flag, 0x1400 + slot)) break;
                if (!r_a && !mbar_wait(smem_u32(&aux->afull[e]), eph, abort_flag, 0x1410 + e)) break;
                // the next super-block's barriers are tested before this one's MMAs are issued (the answers take time)
                const int na = a + 1 == C::D_SETS ? 0 : a + 1;
                const uint32_t naph = na == 0 ? aph ^ 1 : aph;
                r_acc = mbar_test(smem_u32(&aux->acc_empty[na]), naph ^ 1);
                r_s = mbar_test(smem_u32(&aux->sfull[(b + 1) & (C::SCL_SLOTS - 1)]), ((b + 1) >> 3) & 1);
                r_a = mbar_test(smem_u32(&aux->afull[e ^ 1]), ((b + 1) >> 1) & 1);
                tc_fence_after();
                const uint32_t xs = smem_u32(smem + C::OFF_SCL + slot * C::SCL_BYTES);
                const uint32_t d = tmem_base + a * C::SET_COLS;
                const uint32_t at = tmem_base + C::A_COL0 + e * C::A_COLS;
#pragma unroll
                for (int g = 0; g < 8; ++g) {                            // sub-block g: 8 operand columns -> its own 16 columns
                    const uint64_t bd = umma_desc_advance(umma_desc_k128(xs + (g >> 2) * NB * 128), (g & 3) * 32);
                    umma_i8_ts(d + g * NB, at + g * 8, bd, idesc, 0u);
                }
                tc_commit(smem_u32(&aux->acc_full[a]));
                a = na;
                aph = naph;
            }
        }
    } else if (warp < 10) {
        // ------------------------------------------------------------------ expanders: packed weights -> tensor memory
        const int q = warp & 3, kh = (warp - 2) >> 2;                    // lane quarter, K half of the super-block
        const int n = q * 32 + lane;                                     // weight row in the tile = tensor-memory lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + C::A_COL0 + kh * 32;
        for (int b = 0; b < NSB; ++b) {
            const int ws = b & (C::W_STAGES - 1), e = b & 1;
            if (!mbar_wait(smem_u32(&aux->wfull[ws]), (b >> 3) & 1, abort_flag, 0x1500 + ws)) break;
            // operand buffer e was last read by the MMAs of super-block b - 2: their commit completed that set's barrier
            if (b >= 2 && !mbar_wait(smem_u32(&aux->acc_full[(b - 2) % C::D_SETS]), ((b - 2) / C::D_SETS) & 1, abort_flag,
                                     0x1510 + e)) break;
            tc_fence_after();
            const uint8_t* st = smem + ws * C::W_BYTES;
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 w = *(const uint4*)(st + swz(n, kh * 4 + j));
                // inputs 0..15 are the low nibbles, 16..31 the high nibbles: four values per 32-bit column
                r[8 * j + 0] = w.x & 0x0F0F0F0Fu;
                r[8 * j + 1] = w.y & 0x0F0F0F0Fu;
                r[8 * j + 2] = w.z & 0x0F0F0F0Fu;
                r[8 * j + 3] = w.w & 0x0F0F0F0Fu;
                r[8 * j + 4] = (w.x >> 4) & 0x0F0F0F0Fu;
                r[8 * j + 5] = (w.y >> 4) & 0x0F0F0F0Fu;
                r[8 * j + 6] = (w.z >> 4) & 0x0F0F0F0Fu;
                r[8 * j + 7] = (w.w >> 4) & 0x0F0F0F0Fu;
            }
            tmem_st32(lane_base + e * C::A_COLS, r);                     // this K half: 128 inputs = 32 columns
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&aux->afull[e]));
                mbar_arrive(smem_u32(&aux->wempty[ws]));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: one weight row, eight rows of x per thread
        const int q = warp & 3, hsel = (warp - 10) >> 2;
        const int c0 = hsel * 8;
        const int nl = q * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool rows_live = m0 + c0 < live;                           // warp-uniform
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = 0.0f;
        bool ok = true;
        const int ml = m0 + (lane & 15);                                 // lane l carries the scale of activation row m0 + (l & 15)
        float am_next = (NSB > 0 && ml < p.Ma) ? __ldg(p.a + (long)b0 * p.Ma + ml) : 0.0f;
        const int n = n0 + nl;
        // this weight row's scales, one super-block ahead: sc, mn uint8 [K/256, N, 8]; d, dmin fp32 [K/256, N]
        const long nn = n < p.N ? n : 0;
        const uint2* scp = (const uint2*)p.sc + (long)b0 * p.N + nn;
        const uint2* mnp = (const uint2*)p.mn + (long)b0 * p.N + nn;
        const float* dp = p.d + (long)b0 * p.N + nn;
        const float* dmp = p.dm + (long)b0 * p.N + nn;
        uint2 sc_next = make_uint2(0, 0), mn_next = make_uint2(0, 0);
        float d_next = 0.0f, dm_next = 0.0f;
        if (NSB > 0) {
            sc_next = __ldg(scp);
            mn_next = __ldg(mnp);
            d_next = __ldg(dp);
            dm_next = __ldg(dmp);
        }
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        float* ws_tile = SPLIT ? p.ws + (long)tile * NSBT * NB * 128 : nullptr;
        int a = 0;
        uint32_t aph = 0;
        for (int b = 0; b < NSB; ++b) {
            const int slot = b & (C::SCL_SLOTS - 1);
            const float am_l = am_next;
            const uint2 sc8 = sc_next, mn8 = mn_next;
            const float dv = d_next, ndm = -dm_next;
            if (b + 1 < NSB) {
                if (ml < p.Ma) am_next = __ldg(p.a + (long)(b0 + b + 1) * p.Ma + ml);
                sc_next = __ldg(scp + (long)(b + 1) * p.N);
                mn_next = __ldg(mnp + (long)(b + 1) * p.N);
                d_next = __ldg(dp + (long)(b + 1) * p.N);
                dm_next = __ldg(dmp + (long)(b + 1) * p.N);
            }
            if (!mbar_wait(smem_u32(&aux->sfull[slot]), (b >> 3) & 1, abort_flag, 0x1620 + slot) ||
                !mbar_wait(smem_u32(&aux->acc_full[a]), aph, abort_flag, 0x1600 + a)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (rows_live) {
                const uint8_t* sl = smem + C::OFF_SCL + slot * C::SCL_BYTES;
                int scg[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) scg[g] = (int)(((g < 4 ? sc8.x : sc8.y) >> (8 * (g & 3))) & 0xff);
                const uint32_t set = lane_base + a * C::SET_COLS;
                uint32_t r[8][8];
#pragma unroll
                for (int g = 0; g < 8; ++g) tmem_ld8(set + g * NB + c0, r[g]);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int acc = scg[0] * (int)r[0][j];
#pragma unroll
                    for (int g = 1; g < 8; ++g) acc += scg[g] * (int)r[g][j];
                    const uint4 s16 = *(const uint4*)(sl + C::SOFF_XS + (c0 + j) * 16);       // eight S & 63, eight S >> 6
                    const int mlo = __dp4a((int)mn8.x, (int)s16.x, __dp4a((int)mn8.y, (int)s16.y, 0));
                    const int mhi = __dp4a((int)mn8.x, (int)s16.z, __dp4a((int)mn8.y, (int)s16.w, 0));
                    const int mins = mlo + 64 * mhi;
                    const float am = SPLIT ? 0.0f : __shfl_sync(0xffffffffu, am_l, c0 + j);
                    float t = __fmul_rn(dv, __int2float_rn(acc));
                    t = __fmaf_rn(ndm, __int2float_rn(mins), t);
                    if (SPLIT) ws_tile[((long)(b0 + b) * NB + c0 + j) * 128 + nl] = t;   // the chain runs later
                    else y[j] = __fmaf_rn(am, t, y[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&aux->acc_empty[a]));
                mbar_arrive(smem_u32(&aux->sempty[slot]));
            }
            if (++a == C::D_SETS) {
                a = 0;
                aph ^= 1;
            }
        }
        if (SPLIT) {
            // every epilogue thread takes part in the hand-over (the abort path too: it then reports not-last)
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (threadIdx.x == 320) {
                const int old = ok ? atomicAdd(p.counters + tile, 1) : -1;
                aux->is_last = (old == p.split - 1);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (!aux->is_last) ok = false;                               // another CTA finishes this tile
            else {
                __threadfence();
                if (rows_live) {
                    // the reference's chain, in super-block order, over every slice's terms (read from L2)
                    for (int b = 0; b < NSBT; ++b) {
                        const float am_l = ml < p.Ma ? __ldg(p.a + (long)b * p.Ma + ml) : 0.0f;
                        float tv[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) tv[j] = __ldcg(ws_tile + ((long)b * NB + c0 + j) * 128 + nl);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            y[j] = __fmaf_rn(__shfl_sync(0xffffffffu, am_l, c0 + j), tv[j], y[j]);
                    }
                }
                if (threadIdx.x == 320) p.counters[tile] = 0;
            }
        }
        if (ok && n < p.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int m = m0 + c0 + j;
                if (m < live) {
                    if (p.epi == 0) ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(y[j]);
                    else {
                        float* o = (float*)p.out + (long)m * p.ldo + n;
                        *o = __fadd_rn(*o, y[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace w4a8
