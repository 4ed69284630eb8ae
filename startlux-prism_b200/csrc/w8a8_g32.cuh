// W8A8 with one scale per 32 inputs on both operands (Q8_0 weights against per-32 activation scales), few rows:
// out[m, n] = sum over groups g, in ascending order, of mul_rn(mul_rn(float(sum_g), a_s[m, g]), w_s[n, g])
// (the reference's decode kernel, kernels/decode.py:118-163: an fp32 chain per output element, so K cannot be split
// between CTAs without changing bits).  The operands are swapped: 128 weight rows own the tensor-memory lanes, up to
// 16 activation rows are the MMA's N; every group is one tcgen05.mma (K = 32) into its own 16 columns.
//
// What bounds this kernel was measured with cycle stamps inside it and with single-thread probes on a B200:
//   * one thread issues a 128 x 16 x 32 MMA every 45-50 cycles whatever N is (the tensor core reads the 4 KB A tile
//     from shared memory each time): 160 MMAs per 128 weight rows of K = 5120 are 7-8 k cycles, the floor of a tile;
//   * a loop iteration of the producer or of the MMA thread costs 300-500 cycles beyond its copies and MMAs, so a
//     stage carries 256 bytes of K (two 128-byte swizzle rows per operand row, one 3-D tensor-map box per operand)
//     and there are half as many iterations;
//   * the epilogue's fp32 chain (convert, two rounded multiplies, one add per group and element) is about 600 cycles
//     of the fp32 pipe per 512 bytes of K and 8 rows a warp; it reads the activation scales, loaded once into shared
//     memory, and never waits on a pipeline stage: the stages go back to the producer when their MMAs have completed.
// Roles: warp 0 = TMA producer (one thread), warps 1 and 2 = MMA issuers (one thread each; warp 1 owns the tensor
// memory), warps 3..10 = epilogue: two warps per lane quarter, each with RW of the CTA's 2 * RW activation rows.
// Up to 16 rows: NB = 16 and a CTA owns 16, 8 or 4 of them; more rows: NB = 32, row blocks of 32 in grid.z (each block
// re-reads the weights from L2).
#pragma once
#include "w8a8_gemm.cuh"

namespace w8a8 {

template <int NB_>
struct G32 {
    static constexpr int NB = NB_;                        // MMA N: activation rows per CTA (zero-filled past M): 16 or 32
    static constexpr int KS = 256;                        // bytes of K per stage
    static constexpr int W_BYTES = BM * KS;               // 32 KB: [2][128 rows][128 bytes], 128-byte swizzle
    static constexpr int X_BYTES = NB * KS;               // [2][NB rows][128 bytes]
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int SLOT_COLS = 256;                 // an accumulator slot: 16 columns per group and row ...
    static constexpr int SLOT_QUADS = SLOT_COLS / (4 * NB);   // ... = 4 quads of 16 rows, 2 quads of 32 (a quad = 4 groups = 128 bytes of K)
    static constexpr int SLOT_STAGES = SLOT_QUADS / 2;    // stages per slot: 2 or 1
    static constexpr int RING = 2;                        // 512 columns: one CTA per SM
    static constexpr int TMEM_COLS = 512;
    static constexpr int EPI_WARPS = 8;
    static constexpr int MMA_WARPS = 2;                   // stages alternate between two issuing threads
    static constexpr int FIRST_EPI_WARP = 1 + MMA_WARPS;
    static constexpr int THREADS = 32 * (FIRST_EPI_WARP + EPI_WARPS);
    static constexpr int MAX_STAGES = 5;
    // activation scales in shared memory: [rows][quads rounded up to a multiple of four] float4
    __host__ __device__ static constexpr int padded_quads(int K) { return (K / 128 + 3) / 4 * 4; }
    __host__ __device__ static constexpr int sa_bytes(int K, int rows) { return rows * padded_quads(K) * 16; }
    static constexpr int smem_bytes(int K, int rows, int stages) {
        return 1024 + stages * STAGE_BYTES + sa_bytes(K, rows) + (int)sizeof(Aux);
    }
    static constexpr int stages_for(int K, int rows) {
        const int room = 232448 - 1024 - (int)sizeof(Aux) - sa_bytes(K, rows);
        return room / STAGE_BYTES > MAX_STAGES ? MAX_STAGES : room / STAGE_BYTES;
    }
};

// 3-D tiled load: c0 = byte inside the 128-byte chunk (0), c1 = row, c2 = 128-byte chunk of K.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        : : "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;"
        : : "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy) : "memory");
}

// Packed fp32 pairs with the rounding written out (an operation with an explicit rounding mode is never contracted
// into a fused multiply-add): two rows of one output column per instruction.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ float2 unpack2(f32x2 v) {
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(v));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {          // never directly on a packed product (see add_quad)
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
// Two int32 group sums as a packed pair of floats: |sum| < 2^19, so the sum added to the bit pattern of 1.5 * 2^23
// minus that constant is exactly float(sum) (two integer adds and one packed add instead of two conversions).
__device__ __forceinline__ f32x2 pair_of(uint32_t a, uint32_t b) {
    f32x2 biased;
    asm("mov.b64 %0, {%1, %2};" : "=l"(biased) : "r"(0x4B400000u + a), "r"(0x4B400000u + b));
    return add2(biased, pack2(-12582912.0f, -12582912.0f));
}

// One quad (four groups, 128 bytes of K) of RW activation rows added to the rows' fp32 sums in group order.
// r[g][j]: int32 sum of group g and row j; sa: the quad's activation scales as row pairs, float2 [RW / 2 pairs at
// `stride` float4s apart][4 groups] = (row 2i, row 2i + 1) per group; sw4: this thread's weight row's four scales.
// plain: acc = add_rn(acc, mul_rn(mul_rn(float(sum), sa), sw)); fuse (the vocabulary head, whose reference kernel
// leaves the roundings to its compiler, kernels/decode.py:157): acc = fma_rn(mul_rn(float(sum), sa), sw, acc).
template <int RW>
__device__ __forceinline__ void add_quad(f32x2* acc, const uint32_t (&r)[4][RW], const float4* sa, int stride,
                                         const float4 sw4, bool fuse) {
    const f32x2 w[4] = {pack2(sw4.x, sw4.x), pack2(sw4.y, sw4.y), pack2(sw4.z, sw4.z), pack2(sw4.w, sw4.w)};
#pragma unroll
    for (int i = 0; i < RW / 2; ++i) {
        const float4 s01 = sa[i * stride], s23 = sa[i * stride + 1];     // groups 0,1 and 2,3 of rows (2i, 2i + 1)
        const f32x2 s[4] = {pack2(s01.x, s01.y), pack2(s01.z, s01.w), pack2(s23.x, s23.y), pack2(s23.z, s23.w)};
        f32x2 a = acc[i];
        if (fuse) {
#pragma unroll
            for (int g = 0; g < 4; ++g) a = fma2(mul2(pair_of(r[g][2 * i], r[g][2 * i + 1]), s[g]), w[g], a);
        } else {
            // the adds stay scalar: the assembler contracts a packed multiply followed by a packed add into a fused
            // multiply-add even with the roundings written out (measured: a few results in a thousand change)
            float2 f = unpack2(a);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float2 t = unpack2(mul2(mul2(pair_of(r[g][2 * i], r[g][2 * i + 1]), s[g]), w[g]));
                f.x = __fadd_rn(f.x, t.x);
                f.y = __fadd_rn(f.y, t.y);
            }
            a = pack2(f.x, f.y);
        }
        acc[i] = a;
    }
}

// tm_w: weights [N, K] as {128, N, K / 128} with box {128, 128, 2}; tm_x: activations [M, K] the same way with box
// {128, NB, 2}.  p: a_s [M, K / 32], w_s [N, K / 32], out, ldo, n_rows, M, N, K (a multiple of 128), epi (bf16, fp32 add
// or fp32), pdl, stages.  Grid (N / 128 tiles, 1, row blocks of 2 * RW).
template <int NB, int RW>
__global__ void __launch_bounds__(G32<NB>::THREADS, 1)
w8a8_g32_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const SwapArgs p) {
    using C = G32<NB>;
    constexpr int RCTA = 2 * RW;                               // activation rows this CTA owns (<= NB)
    constexpr int RC = RW < 8 ? RW : 8;                        // rows per tensor-memory load
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    const int NST = p.stages;
    const int KC = p.K / BK;                                   // quads = 128-byte chunks of K
    const int QP = C::padded_quads(p.K);
    float4* sa = (float4*)(smem + NST * C::STAGE_BYTES);       // float2 [RCTA / 2 row pairs][QP quads][4 groups]
    Aux* aux = (Aux*)((uint8_t*)sa + C::sa_bytes(p.K, RCTA));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    const int n0 = blockIdx.x * BM, m0 = blockIdx.z * RCTA;
    if (m0 >= live) return;                                    // whole CTA, before any barrier or allocation
    const int nst = (KC + 1) / 2;                              // stages of K this CTA walks through
    const int nslots = (KC + C::SLOT_QUADS - 1) / C::SLOT_QUADS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 1);            // the MMA's commit hands a stage back
        }
        for (int b = 0; b < C::RING; ++b) {
            mbar_init(smem_u32(&aux->tfull[b]), C::SLOT_STAGES);   // one commit per stage of the slot (= per issuing thread)
            mbar_init(smem_u32(&aux->tempty[b]), C::EPI_WARPS);
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
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_w);
            tma_prefetch_desc(&tm_x);
            const uint64_t pol_w = policy_evict_first();       // weights are read once
            // programmatic dependent launch: the first stages' weights are requested before the wait for the kernel
            // that produces the activations, their activation tiles after it
            const int pre = p.pdl ? (nst < NST ? nst : NST) : 0;
            for (int i = 0; i < pre; ++i) {
                const uint32_t bar = smem_u32(&aux->full[i]);
                mbar_expect_tx(bar, C::STAGE_BYTES);
                tma_load_3d_hint(smem_u32(smem + i * C::STAGE_BYTES), &tm_w, 0, n0, 2 * i, bar, pol_w);
            }
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < pre; ++i)
                tma_load_3d(smem_u32(smem + i * C::STAGE_BYTES + C::W_BYTES), &tm_x, 0, m0, 2 * i,
                            smem_u32(&aux->full[i]));
            int stage = pre == NST ? 0 : pre;
            uint32_t phase = pre == NST ? 1 : 0;
            int issued = pre;
            bool ok = true;
            for (int i = pre; i < nst; ++i) {
                if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0x2500 + stage)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&aux->full[stage]);
                uint8_t* st = smem + stage * C::STAGE_BYTES;
                mbar_expect_tx(bar, C::STAGE_BYTES);
                tma_load_3d_hint(smem_u32(st), &tm_w, 0, n0, 2 * i, bar, pol_w);
                tma_load_3d(smem_u32(st + C::W_BYTES), &tm_x, 0, m0, 2 * i, bar);
                issued = i + 1;
                if (++stage == NST) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok) {
                // after an abort every copy still in flight gets a bounded time to land before the CTA may exit
                const unsigned long long t0 = global_timer_ns();
                const unsigned long long limit = *(volatile unsigned long long*)&g_pb_wait_ns;
                for (int j = issued > NST ? issued - NST : 0; j < issued; ++j)
                    while (!mbar_test(smem_u32(&aux->full[j % NST]), (uint32_t)(j / NST) & 1))
                        if (global_timer_ns() - t0 > limit) break;
            }
        }
    } else if (warp < C::FIRST_EPI_WARP) {
        if (lane == 0) {
            // Stage i belongs to issuing thread i % 2: a thread's loop iteration (two barrier waits, eight MMAs, two
            // commits) takes about 1,500 cycles, twice what the tensor core needs for the stage.  An accumulator slot
            // is two consecutive stages, one of each thread (16 rows), or one stage (32 rows); every stage's thread
            // commits its MMAs to the slot's barrier.
            const int t = warp - 1;
            const uint32_t idesc = umma_idesc_i8(BM, NB);
            int stage = t % NST;
            uint32_t phase = (uint32_t)(t / NST) & 1;
            for (int i = t; i < nst; i += C::MMA_WARPS) {
                const int slot = i / C::SLOT_STAGES, ring = slot & 1, sub = i % C::SLOT_STAGES;
                // the slot must have been drained (a fresh barrier passes at once)
                if (!mbar_wait(smem_u32(&aux->tempty[ring]), ((uint32_t)(slot >> 1) & 1) ^ 1, abort_flag, 0x2600 + ring)) break;
                if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x2700 + stage)) break;
                tc_fence_after();
                const uint32_t st = smem_u32(smem + stage * C::STAGE_BYTES);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (2 * i + c >= KC) break;                // K / 128 odd: the last stage's second chunk is fill
                    const uint64_t ad = umma_desc_k128(st + c * (BM * BK));
                    const uint64_t bd = umma_desc_k128(st + C::W_BYTES + c * (NB * BK));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_i8(tmem_base + ring * C::SLOT_COLS + ((sub * 2 + c) * 4 + k) * NB,
                                umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc, 0u);
                }
                tc_commit(smem_u32(&aux->empty[stage]));       // the stage is free once these MMAs have read it
                tc_commit(smem_u32(&aux->tfull[ring]));
                // a last slot of one stage where slots have two: its barrier still expects the other thread's arrival
                if (C::SLOT_STAGES == 2 && sub == 0 && i + 1 == nst) tc_commit(smem_u32(&aux->tfull[ring]));
                stage += C::MMA_WARPS;
                if (stage >= NST) {
                    stage -= NST;
                    phase ^= 1;
                }
            }
        }
    } else {
        const int q = warp & 3;                                // this warp's tensor-memory lane quarter
        const int h = (warp - C::FIRST_EPI_WARP) >> 2;         // which half of the CTA's rows
        const int nl = q * 32 + lane;                          // this thread's weight row inside the tile
        const int n = n0 + nl;
        const int j0 = h * RW;
        const int G = p.K >> 5;
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // before any global read or write of this warp
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        // this thread's weight row: one float4 of group scales per quad.  The whole row goes to L2 now (rows are K / 8
        // bytes apart: a scattered read whose DRAM latency must not be met once per slot); the loads run a slot ahead.
        const float4* swp = (const float4*)(p.w_s + (long)(n < p.N ? n : 0) * G);
        for (int off = h * 128; off < KC * 16; off += 256) asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)swp + off));
        if (h == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"((const char*)swp + KC * 16 - 16));
        float4 sw_ahead[C::SLOT_QUADS];
#pragma unroll
        for (int b = 0; b < C::SLOT_QUADS; ++b) sw_ahead[b] = b < KC ? __ldg(swp + b) : make_float4(0.f, 0.f, 0.f, 0.f);
        // the CTA's activation scales: a_s rows m0 .. m0 + RCTA - 1, one float4 per quad, read once
        {
            const int e = threadIdx.x - 32 * C::FIRST_EPI_WARP;
            float* saf = (float*)sa;
            for (int idx = e; idx < RCTA * KC; idx += 32 * C::EPI_WARPS) {
                const int row = idx / KC, qd = idx - row * KC;
                const int m = m0 + row;
                const float4 v = m < live ? __ldg((const float4*)(p.a_s + (long)m * G) + qd)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                float* dst = saf + (((row >> 1) * QP + qd) * 4) * 2 + (row & 1);
                dst[0] = v.x;
                dst[2] = v.y;
                dst[4] = v.z;
                dst[6] = v.w;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * C::EPI_WARPS) : "memory");
        }
        f32x2 acc[RW / 2];                                     // rows (j0 + 2i, j0 + 2i + 1)
#pragma unroll
        for (int j = 0; j < RW / 2; ++j) acc[j] = pack2(0.0f, 0.0f);
        const bool fuse = p.epi == EPI_F32;
        const bool mine = m0 + j0 < live;                      // warp-uniform: does this warp hold live rows?
        int ring = 0;
        uint32_t rphase = 0;
        bool ok = true;
        for (int slot = 0; slot < nslots; ++slot) {
            const int nq = KC - slot * C::SLOT_QUADS < C::SLOT_QUADS ? KC - slot * C::SLOT_QUADS : C::SLOT_QUADS;
            float4 sw4[C::SLOT_QUADS];
#pragma unroll
            for (int b = 0; b < C::SLOT_QUADS; ++b) {
                sw4[b] = sw_ahead[b];
                const int qd = (slot + 1) * C::SLOT_QUADS + b;
                if (qd < KC) sw_ahead[b] = __ldg(swp + qd);
            }
            if (!mbar_wait(smem_u32(&aux->tfull[ring]), rphase, abort_flag, 0x2800 + ring)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (mine) {
#pragma unroll
                for (int c = 0; c < RW; c += RC) {             // RC rows at a time
                    if (m0 + j0 + c >= live) break;
                    const float4* sa_slot = sa + (((j0 + c) >> 1) * QP + slot * C::SLOT_QUADS) * 2;
#pragma unroll
                    for (int b0 = 0; b0 < C::SLOT_QUADS; b0 += 2) {
                        if (b0 >= nq) break;
                        uint32_t r[2][4][RC];                  // two quads' loads in flight before each wait
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            if (b0 + u < nq) {
#pragma unroll
                                for (int g = 0; g < 4; ++g)
                                    tmem_ldn(lane_base + ring * C::SLOT_COLS + ((b0 + u) * 4 + g) * NB + j0 + c, r[u][g]);
                            }
                        tmem_ld_wait();
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            if (b0 + u < nq)
                                add_quad<RC>(acc + c / 2, r[u], sa_slot + (b0 + u) * 2, QP * 2, sw4[b0 + u], fuse);
                    }
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
        if (ok && mine) {
            float v[RW];
#pragma unroll
            for (int j = 0; j < RW / 2; ++j) {
                const float2 a = unpack2(acc[j]);
                v[2 * j] = a.x;
                v[2 * j + 1] = a.y;
            }
            swap_store<RW>(p, n, m0 + j0, live, v);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

}  // namespace w8a8
