// W8A8 with any scale group along K (gk a multiple of 32 that divides K, other than 32 and K, which have their own
// kernels): the arithmetic of the reference's Triton kernel for a general GK (kernels/w8a8.py:64-76) - per group an
// exact int32 dot product, then acc = add_rn(acc, mul_rn(mul_rn(float(acci), sa[m, g]), sw[n, g])) for g ascending.
// The consumer of the fused SwiGLU epilogue's output (one activation scale per BN / 2 columns) is such a product.
//
// Structure of the operand-swapped few-rows kernel (weight tile of 128 rows = the MMA's M, NB activation rows = its N,
// TMA-staged 128-byte K blocks).  Every scale group owns one slot of a ring of int32 accumulators in tensor memory:
// the MMA thread accumulates the group's K = 32 steps into the slot, commits it, and moves to the next slot while the
// four epilogue warps scale the finished one (thread = weight row, fp32 sums of its NB rows in registers).  Stages
// are handed back by the MMA's own commit, slots by the epilogue warps.
#pragma once
#include "w8a8_gemm.cuh"

namespace w8a8 {

template <int NB>
struct GroupsCfg {
    static constexpr int W_BYTES = BM * BK;
    static constexpr int X_BYTES = NB * BK;
    static constexpr int STAGE_BYTES = (W_BYTES + X_BYTES + 1023) / 1024 * 1024;
    static constexpr int STAGES = (108 * 1024 / STAGE_BYTES) > 8 ? 8 : (108 * 1024 / STAGE_BYTES);
    static constexpr int RING = 4;
    static constexpr int ACC_COLS = RING * NB;
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : 256;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + (int)sizeof(Aux);
    static constexpr int THREADS = 64 + 128;
};

// p.gblocks: 32-input blocks per scale group (gk / 32); p.a_s fp32 [M, K / gk], p.w_s fp32 [N, K / gk].
template <int NB>
__global__ void __launch_bounds__(GroupsCfg<NB>::THREADS, 1)
w8a8_groups_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const SwapArgs p) {
    using C = GroupsCfg<NB>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    Aux* aux = (Aux*)(smem + C::STAGES * C::STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    const int n0 = blockIdx.x * BM, m0 = blockIdx.z * NB;
    if (m0 >= live) return;                                    // whole CTA, before any barrier or allocation
    const int nkb = p.K / BK;                                  // K % 128 == 0 (checked by the host)
    const int gb = p.gblocks;
    const int G = (p.K >> 5) / gb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 1);
        }
        for (int b = 0; b < C::RING; ++b) {
            mbar_init(smem_u32(&aux->tfull[b]), 1);
            mbar_init(smem_u32(&aux->tempty[b]), 4);
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
        if (lane == 0) {
            tma_prefetch_desc(&tm_w);
            tma_prefetch_desc(&tm_x);
            const uint64_t pol_w = policy_evict_first();
            uint32_t armed_parity[8];
            uint32_t armed_mask = 0;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0x1600 + stage)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&aux->full[stage]);
                mbar_expect_tx(bar, C::W_BYTES + C::X_BYTES);
                uint8_t* st = smem + stage * C::STAGE_BYTES;
                tma_load_2d_hint(smem_u32(st), &tm_w, kb * BK, n0, bar, pol_w);
                tma_load_2d(smem_u32(st + C::W_BYTES), &tm_x, kb * BK, m0, bar);
                armed_parity[stage] = phase;
                armed_mask |= 1u << stage;
                if (++stage == C::STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok) drain_armed(aux, C::STAGES, armed_parity, armed_mask);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(BM, NB);
            int stage = 0, ring = 0, in_group = 0;
            uint32_t phase = 0, rphase = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x1700 + stage)) break;
                tc_fence_after();
                uint8_t* st = smem + stage * C::STAGE_BYTES;
                const uint64_t ad = umma_desc_k128(smem_u32(st));
                const uint64_t bd = umma_desc_k128(smem_u32(st + C::W_BYTES));
#pragma unroll
                for (int k = 0; k < BK / 32; ++k) {
                    if (in_group == 0) {
                        // a new group: its slot must have been read out (a fresh barrier passes at once)
                        if (!mbar_wait(smem_u32(&aux->tempty[ring]), rphase ^ 1, abort_flag, 0x1800 + ring)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                    }
                    umma_i8(tmem_base + ring * NB, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc,
                            in_group ? 1u : 0u);
                    if (++in_group == gb) {
                        tc_commit(smem_u32(&aux->tfull[ring]));
                        in_group = 0;
                        if (++ring == C::RING) {
                            ring = 0;
                            rphase ^= 1;
                        }
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&aux->empty[stage]));
                if (++stage == C::STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else {
        const int q = warp & 3;
        const int nl = q * 32 + lane;
        const int n = n0 + nl;
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        float acc[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j) acc[j] = 0.0f;
        const float* swp = p.w_s + (long)(n < p.N ? n : 0) * G;
        // the row's scales go to L2 now: the loads below, one group ahead of their use, then meet an L2 hit and not a
        // scattered DRAM read per group
        for (int off = 0; off < G * 4; off += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)swp + off));
        asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)swp + G * 4 - 4));
        float sw_next = __ldg(swp);
        int ring = 0;
        uint32_t rphase = 0;
        bool ok = true;
        for (int g = 0; g < G; ++g) {
            const float sw = sw_next;
            if (g + 1 < G) sw_next = __ldg(swp + g + 1);
            if (!mbar_wait(smem_u32(&aux->tfull[ring]), rphase, abort_flag, 0x1900 + ring)) {
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < NB; c += 8) {
                if (m0 + c >= live) break;
                uint32_t r[8];
                tmem_ld8(lane_base + ring * NB + c, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float sa = (m0 + c + j < live) ? __ldg(p.a_s + (long)(m0 + c + j) * G + g) : 0.0f;
                    acc[c + j] = __fadd_rn(acc[c + j], scale2((int)r[j], sa, sw));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->tempty[ring]));
            if (++ring == C::RING) {
                ring = 0;
                rphase ^= 1;
            }
        }
        if (ok) swap_store<NB>(p, n, m0, live, acc);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace w8a8
