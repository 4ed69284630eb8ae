// W8A8 GEMMs on the sm_100a tensor cores: int8 x int8 -> int32 in tensor memory (tcgen05.mma kind::i8), operand
// tiles staged in shared memory by TMA (128-byte swizzle, K-major), warp-specialised: one TMA thread, one MMA thread,
// four epilogue warps that read the accumulators with tcgen05.ld.
//
// Numerics (the reference's contract, kernels/w8a8.py:14-17,76,85; csrc/w8a8_gemm.cu:334-339,370-371): the integer
// sum over K (or over one scale group) is exact; then v = mul_rn(mul_rn(float(acc), s_a[m]), s_w[n]); epilogue 1 adds
// with add_rn.  No fused multiply-add anywhere in an epilogue, so every tile shape and K split gives the same bits.
//
// Two kernels:
//   w8a8_tile_kernel  many rows (prefill): the activation tile is the MMA's M operand (128 rows), the weight tile its
//                     N operand (BN rows); persistent over output tiles, two accumulator buffers in tensor memory so
//                     a tile's epilogue overlaps the next tile's main loop.  One scale group (gk == K).
//   w8a8_swap_kernel  few rows (decode) and per-32 scale groups: operands swapped, the weight tile (128 rows) is the
//                     MMA's M operand so every tensor-memory lane holds an output column, the activation rows (8..64)
//                     are its N.  Splits K over blockIdx.y: int32 partial sums go to the caller's slots (deferred
//                     residual add), or to a workspace where the last CTA of a tile adds them (exact) and runs the
//                     epilogue.  With GROUPED each K = 32 step writes its own accumulator columns and the epilogue
//                     warps scale and add them in fp32 in group order (Q8_0's own per-32 scales, kernels/w8a8.py:64-76).
#pragma once
#include "common.cuh"

namespace w8a8 {

constexpr int BM = 128;        // MMA M: rows of the operand that owns the tensor-memory lanes
constexpr int BK = 128;        // bytes (= int8 values) of K per pipeline stage: one 128-byte swizzle row
constexpr int EPI_BF16 = 0;    // out bf16 [M, N] = v
constexpr int EPI_ADD = 1;     // out fp32 [M, N] = add_rn(out, v)
constexpr int EPI_SWIGLU = 2;  // out int8 [M, N / 2] = per-tile quantized silu(gate) * up, one scale per row and tile
constexpr int EPI_I32 = 3;     // out int32 [M, N] = acc (no scales)
constexpr int EPI_F32 = 4;     // out fp32 [M, N] = v (the vocabulary head's logits; per-32 groups, few rows)

struct Aux {                   // shared-memory control block placed after the stages
    uint64_t full[12];
    uint64_t empty[12];
    uint64_t tfull[8];
    uint64_t tempty[8];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
    int pad;
};

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
    return (uint8_t*)(((uintptr_t)p + 1023) & ~(uintptr_t)1023);
}

// After an abort the producer gives every armed stage a bounded time to land before the CTA may exit (shared memory
// must not be handed to another CTA with a bulk copy still writing into it).
__device__ __forceinline__ void drain_armed(Aux* aux, int stages, const uint32_t* armed_parity, uint32_t armed_mask) {
    unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = *(volatile unsigned long long*)&g_pb_wait_ns;
    for (int s = 0; s < stages; ++s) {
        if (!(armed_mask >> s & 1)) continue;
        while (!mbar_test(smem_u32(&aux->full[s]), armed_parity[s])) {
            if (global_timer_ns() - t0 > limit) return;
        }
    }
}

// ------------------------------------------------------------------------------------------------- epilogue stores
template <int EPI>
__device__ __forceinline__ void store_row32(void* out, long ldo, long row, int col0, int ncols_ok, bool vec_ok,
                                            const uint32_t (&r)[32], float sa, const float* sw) {
    // One thread: 32 consecutive columns [col0, col0 + 32) of one output row; ncols_ok = columns inside N.
    if (EPI == EPI_BF16) {
        __nv_bfloat16* p = (__nv_bfloat16*)out + row * ldo + col0;
        if (vec_ok && ncols_ok == 32) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x0 = scale2((int)r[v * 8 + 2 * j], sa, sw[v * 8 + 2 * j]);
                    float x1 = scale2((int)r[v * 8 + 2 * j + 1], sa, sw[v * 8 + 2 * j + 1]);
                    __nv_bfloat162 b = __floats2bfloat162_rn(x0, x1);
                    w[j] = *(uint32_t*)&b;
                }
                *(uint4*)(p + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols_ok) p[j] = __float2bfloat16_rn(scale2((int)r[j], sa, sw[j]));
        }
    } else if (EPI == EPI_ADD) {
        float* p = (float*)out + row * ldo + col0;
        if (vec_ok && ncols_ok == 32) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                float4 o = *(float4*)(p + v * 4);
                o.x = __fadd_rn(o.x, scale2((int)r[v * 4 + 0], sa, sw[v * 4 + 0]));
                o.y = __fadd_rn(o.y, scale2((int)r[v * 4 + 1], sa, sw[v * 4 + 1]));
                o.z = __fadd_rn(o.z, scale2((int)r[v * 4 + 2], sa, sw[v * 4 + 2]));
                o.w = __fadd_rn(o.w, scale2((int)r[v * 4 + 3], sa, sw[v * 4 + 3]));
                *(float4*)(p + v * 4) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols_ok) p[j] = __fadd_rn(p[j], scale2((int)r[j], sa, sw[j]));
        }
    } else {
        int32_t* p = (int32_t*)out + row * ldo + col0;
        if (vec_ok && ncols_ok == 32) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
                *(uint4*)(p + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols_ok) p[j] = (int32_t)r[j];
        }
    }
}

// ================================================================================================= tile kernel
// The epilogue of one 128 x BN accumulator (one lane quarter per warp, thread = row): scale, then store.
template <int BN, int EPI>
__device__ __forceinline__ void drain_accumulator(void* __restrict__ out, long ldo, int N, int live, int m0, int n0,
                                                  int q, int lane, uint32_t lane_addr, uint32_t* stg,
                                                  const float* swb, float sa, bool word_ok) {
    const int row = m0 + q * 32 + lane;
    const bool rok = row < live;
    if (word_ok) {
        // coalesced path: every thread scales its row's values and parks them in shared memory (row-major,
        // 33-word pitch: conflict-free both ways); then each warp instruction moves one row's 32 consecutive
        // words (128 bytes) to or from global memory.
        constexpr int CPW = (EPI == EPI_BF16) ? 2 : 1;            // output columns per 32-bit word
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32 * CPW) {
            if (n0 + c0 >= N) break;
            uint32_t r[32];
            tmem_ld32(lane_addr + c0, r);
            tmem_ld_wait();
            if (EPI == EPI_BF16) {
                uint32_t r2[32];
                tmem_ld32(lane_addr + c0 + 32, r2);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(scale2((int)r[2 * j], sa, swb[c0 + 2 * j]),
                                                              scale2((int)r[2 * j + 1], sa, swb[c0 + 2 * j + 1]));
                    stg[lane * 33 + j] = *(uint32_t*)&b2;
                }
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(
                        scale2((int)r2[2 * j], sa, swb[c0 + 32 + 2 * j]),
                        scale2((int)r2[2 * j + 1], sa, swb[c0 + 32 + 2 * j + 1]));
                    stg[lane * 33 + 16 + j] = *(uint32_t*)&b2;
                }
            } else if (EPI == EPI_ADD) {
#pragma unroll
                for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __float_as_uint(scale2((int)r[j], sa, swb[c0 + j]));
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = r[j];
            }
            __syncwarp();
            const int col = n0 + c0 + lane * CPW;                 // first column of this lane's word
            const int rows_here = live - (m0 + q * 32);           // live rows among this warp's 32
            if (col + CPW <= N) {
                if (EPI == EPI_ADD) {
                    // all 32 rows' loads are issued before the first add: one round trip per chunk, not 32
                    float* base = (float*)out + (long)(m0 + q * 32) * ldo + col;
                    float o[32];
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr)
                        if (rr < rows_here) o[rr] = __ldcg(base + (long)rr * ldo);
#pragma unroll
                    for (int rr = 0; rr < 32; ++rr)
                        if (rr < rows_here)
                            base[(long)rr * ldo] = __fadd_rn(o[rr], __uint_as_float(stg[rr * 33 + lane]));
                } else {
#pragma unroll 8
                    for (int rr = 0; rr < 32; ++rr) {
                        if (rr < rows_here) {
                            const long off = (long)(m0 + q * 32 + rr) * ldo + col;
                            const uint32_t v = stg[rr * 33 + lane];
                            if (EPI == EPI_BF16)
                                *(uint32_t*)((__nv_bfloat16*)out + off) = v;
                            else
                                ((uint32_t*)out)[off] = v;
                        }
                    }
                }
            } else if (EPI == EPI_BF16 && col < N) {              // odd N: the word's first column only
                for (int rr = 0; rr < 32 && rr < rows_here; ++rr)
                    ((uint16_t*)out)[(long)(m0 + q * 32 + rr) * ldo + col] = (uint16_t)(stg[rr * 33 + lane] & 0xffff);
            }
            __syncwarp();
        }
    } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(lane_addr + c * 32, r);
            tmem_ld_wait();
            const int col0 = n0 + c * 32;
            const int nok = N - col0 >= 32 ? 32 : (N - col0 > 0 ? N - col0 : 0);
            if (rok && nok > 0) store_row32<EPI>(out, ldo, row, col0, nok, false, r, sa, swb + c * 32);
        }
    }
}

// The residual-add epilogue of columns [c_begin, c_end) of one accumulator, for one warp: out += v with every
// global access a full 128-byte row segment.  The loads of the next 32-column chunk are in flight while the current
// one is scaled, transposed through shared memory (32 x 32 words, XOR-swizzled: conflict-free both ways) and stored.
__device__ __forceinline__ void drain_add(float* __restrict__ out, long ldo, int N, int live, int m0, int n0, int q,
                                          int lane, uint32_t lane_addr, uint32_t* stg, const float* swb, float sa,
                                          int c_begin, int c_end) {
    const int rows_here = live - (m0 + q * 32);
    float* base = out + (long)(m0 + q * 32) * ldo + n0 + lane;
    float o_next[32];
    auto load_chunk = [&](int c0) {
        if (n0 + c0 + lane < N) {
#pragma unroll
            for (int rr = 0; rr < 32; ++rr)
                if (rr < rows_here) o_next[rr] = __ldcg(base + (long)rr * ldo + c0);
        }
    };
    if (n0 + c_begin < N) load_chunk(c_begin);
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        if (n0 + c0 >= N) break;
        float o[32];
#pragma unroll
        for (int rr = 0; rr < 32; ++rr) o[rr] = o_next[rr];
        if (c0 + 32 < c_end && n0 + c0 + 32 < N) load_chunk(c0 + 32);
        uint32_t r[32];
        tmem_ld32(lane_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) stg[lane * 32 + (j ^ lane)] = __float_as_uint(scale2((int)r[j], sa, swb[c0 + j]));
        __syncwarp();
        if (n0 + c0 + lane < N) {
#pragma unroll
            for (int rr = 0; rr < 32; ++rr)
                if (rr < rows_here)
                    base[(long)rr * ldo + c0] = __fadd_rn(o[rr], __uint_as_float(stg[rr * 32 + (lane ^ rr)]));
        }
        __syncwarp();
    }
}

// The residual add without a round trip through the SM: every warp scales 32 x 32 accumulator values into a
// shared-memory box (row-major, 128-byte swizzle: conflict-free 16-byte stores) and the copy engine adds the box into
// out (cp.reduce.async.bulk.tensor .add on fp32: one IEEE round-to-nearest add per element, each element touched
// once, so the result does not depend on any order).  Rows past the live count hold -0.0f, which changes no value it is
// added to.  A warp rewrites its box only after the engine has read the previous one (the wait sits after the
// next chunk's values are already scaled in registers).
// Note: the memory-side adder flushes subnormal inputs and results to zero (as fp32 atomics do); out values in the
// normal range - any real residual stream - get the same bits as __fadd_rn.
__device__ __forceinline__ void drain_add_tma(const CUtensorMap* tm_out, int N, int live, int m0, int n0, int q, int lane,
                                              uint32_t lane_addr, uint32_t* box, const float* swb, float sa,
                                              int c_begin, int c_end) {
    const int row0 = m0 + q * 32;
    if (row0 >= live) return;                                       // warp-uniform: no live row in this quarter
    const bool rok = row0 + lane < live;
    const uint64_t pol = policy_evict_first();
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        if (n0 + c0 >= N) break;
        uint32_t r[32];
        tmem_ld32(lane_addr + c0, r);
        tmem_ld_wait();
        float4 o[8];
#pragma unroll
        for (int v = 0; v < 8; ++v) {
            o[v].x = rok ? scale2((int)r[4 * v + 0], sa, swb[c0 + 4 * v + 0]) : -0.0f;
            o[v].y = rok ? scale2((int)r[4 * v + 1], sa, swb[c0 + 4 * v + 1]) : -0.0f;
            o[v].z = rok ? scale2((int)r[4 * v + 2], sa, swb[c0 + 4 * v + 2]) : -0.0f;
            o[v].w = rok ? scale2((int)r[4 * v + 3], sa, swb[c0 + 4 * v + 3]) : -0.0f;
        }
        // the engine must be done READING the box (the previous chunk's reduction) before it is rewritten
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        const uint32_t base = smem_u32(box) + lane * 128;
#pragma unroll
        for (int v = 0; v < 8; ++v)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};"
                         : : "r"(base + (uint32_t)((v ^ (lane & 7)) << 4)), "f"(o[v].x), "f"(o[v].y), "f"(o[v].z), "f"(o[v].w)
                         : "memory");
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            // evict-first: the residual stream passes through L2 once and must not push out the operands
            asm volatile(
                "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;"
                : : "l"(tm_out), "r"(n0 + c0), "r"(row0), "r"(smem_u32(box)), "l"(pol) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}

// The residual add as fire-and-forget reductions: no load, nothing to wait for.  Each warp instruction adds one row
// segment of 32 consecutive fp32 values (128 bytes) at the memory side (red.global.add.f32: one round-to-nearest add per
// element, every element touched once).  Same note on subnormals as drain_add_tma.
__device__ __forceinline__ void drain_add_red(float* __restrict__ out, long ldo, int N, int live, int m0, int n0, int q,
                                              int lane, uint32_t lane_addr, uint32_t* stg, const float* swb, float sa,
                                              int c_begin, int c_end) {
    const int rows_here = live - (m0 + q * 32);
    if (rows_here <= 0) return;
    float* base = out + (long)(m0 + q * 32) * ldo + n0 + lane;
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        if (n0 + c0 >= N) break;
        uint32_t r[32];
        tmem_ld32(lane_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) stg[lane * 32 + (j ^ lane)] = __float_as_uint(scale2((int)r[j], sa, swb[c0 + j]));
        __syncwarp();
        if (n0 + c0 + lane < N) {
#pragma unroll
            for (int rr = 0; rr < 32; ++rr)
                if (rr < rows_here)
                    asm volatile("red.global.add.f32 [%0], %1;"
                                 : : "l"(base + (long)rr * ldo + c0), "f"(__uint_as_float(stg[rr * 32 + (lane ^ rr)]))
                                 : "memory");
        }
        __syncwarp();
    }
}

// The fused SwiGLU epilogue (the reference's EPI 2, kernels/w8a8.py:86-98) of one 128 x BN accumulator.  The weight
// rows are interleaved in tiles of `gbn` rows (w8a8.interleave_gate_up): gbn / 2 gate rows, then the matching up rows.
// For every such tile the thread (= output row) computes act = silu(gate) * up from the scaled fp32 values, takes the
// maximum over the tile's gbn / 2 columns, and stores them as int8 with one scale per (row, tile):
//   scale = max(amax, 1e-10) / 127, q = rint(act / scale)   (IEEE divisions)
// q int8 [M, N / 2] with row stride ldq, scales fp32 [M, N / gbn].  HB = gbn / 2 is 32 or 64.
template <int BN, int HB>
__device__ __forceinline__ void drain_swiglu(int8_t* __restrict__ qout, long ldq, float* __restrict__ souts, int N, int live,
                                             int m0, int n0, int q, int lane, uint32_t lane_addr, const float* swb,
                                             float sa) {
    constexpr int GBN = 2 * HB;
    const int row = m0 + q * 32 + lane;
    const bool rok = row < live;
    const int tiles_n = N / GBN;
    const bool vec_ok = (((uintptr_t)qout & 15) == 0) && (ldq % 16 == 0);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += GBN) {
        if (n0 + c0 >= N) break;
        float act[HB];
        float amax = 0.0f;
#pragma unroll
        for (int h = 0; h < HB; h += 32) {
            uint32_t rg[32], ru[32];
            tmem_ld32(lane_addr + c0 + h, rg);
            tmem_ld32(lane_addr + c0 + HB + h, ru);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float g = scale2((int)rg[j], sa, swb[c0 + h + j]);
                const float u = scale2((int)ru[j], sa, swb[c0 + HB + h + j]);
                const float a = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, __expf(-g))), u);
                act[h + j] = a;
                amax = fmaxf(amax, fabsf(a));
            }
        }
        if (!rok) continue;
        const float scale = __fdiv_rn(fmaxf(amax, 1e-10f), 127.0f);
        const int tile = (n0 + c0) / GBN;
        souts[(long)row * tiles_n + tile] = scale;
        int8_t* dst = qout + (long)row * ldq + (long)tile * HB;
#pragma unroll
        for (int v = 0; v < HB; v += 16) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t word = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int qi = __float2int_rn(__fdiv_rn(act[v + 4 * k + b], scale));
                    word |= ((uint32_t)qi & 0xffu) << (8 * b);
                }
                w[k] = word;
            }
            if (vec_ok) {
                *(uint4*)(dst + v) = make_uint4(w[0], w[1], w[2], w[3]);
            } else {
#pragma unroll
                for (int k = 0; k < 16; ++k) dst[v + k] = (int8_t)((w[k >> 2] >> (8 * (k & 3))) & 0xff);
            }
        }
    }
}

// Split-K in the tile kernel: the last CTA to finish a tile (a counter per tile) adds the K slices' int32 partial
// accumulators ws[slice][128][BN] (exact, so the order is free) and runs the epilogue for rows [r_begin, r_begin + 32)
// and columns [c_begin, c_end) of the tile.  Lane = column: every load and store is a full row segment.
template <int BN, int EPI>
__device__ __forceinline__ void reduce_store(void* __restrict__ out, long ldo, int N, int live, int m0, int n0, int q,
                                             int lane, const int32_t* __restrict__ ws_tile, long slice_stride, int split,
                                             const float* swb, float sa_lane, int c_begin, int c_end) {
    // Lane = four consecutive columns: a warp instruction moves 512 contiguous bytes of one workspace row; eight rows
    // are in flight together (the workspace is read from L2: latency, not bandwidth, is what this loop has to hide).
    const int rows_here = live - (m0 + q * 32);
    const bool vec_ok = (ldo % 4 == 0) && (((uintptr_t)out & 15) == 0);
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end; c0 += 128) {
        const int cl = c0 + lane * 4;                                // column inside the tile
        const bool mine = cl < c_end;                                // a 64-column range uses half of the lanes
        const int col = mine ? n0 + cl : N;
        const float4 sw4 = mine ? *(const float4*)(swb + cl) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int r0 = 0; r0 < 32; r0 += 8) {
            if (r0 >= rows_here) break;
            int4 tot[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) tot[i] = make_int4(0, 0, 0, 0);
            const int4* src = (const int4*)(ws_tile + (long)(q * 32 + r0) * BN + cl);
            for (int sl = 0; sl < split && mine; ++sl) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int4 v = __ldcg(src + (sl * slice_stride + (long)i * BN) / 4);
                    tot[i].x += v.x; tot[i].y += v.y; tot[i].z += v.z; tot[i].w += v.w;
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float sa = __shfl_sync(0xffffffffu, sa_lane, r0 + i);
                if (r0 + i >= rows_here || col >= N) continue;
                const long off = (long)(m0 + q * 32 + r0 + i) * ldo + col;
                const int t4[4] = {tot[i].x, tot[i].y, tot[i].z, tot[i].w};
                const float w4[4] = {sw4.x, sw4.y, sw4.z, sw4.w};
                if (vec_ok && col + 4 <= N && (EPI != EPI_BF16 || (off % 4) == 0)) {
                    if (EPI == EPI_BF16) {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(scale2(t4[0], sa, w4[0]), scale2(t4[1], sa, w4[1]));
                        __nv_bfloat162 hi = __floats2bfloat162_rn(scale2(t4[2], sa, w4[2]), scale2(t4[3], sa, w4[3]));
                        *(uint2*)((__nv_bfloat16*)out + off) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
                    } else if (EPI == EPI_ADD) {
                        float4 o = *(float4*)((float*)out + off);
                        o.x = __fadd_rn(o.x, scale2(t4[0], sa, w4[0]));
                        o.y = __fadd_rn(o.y, scale2(t4[1], sa, w4[1]));
                        o.z = __fadd_rn(o.z, scale2(t4[2], sa, w4[2]));
                        o.w = __fadd_rn(o.w, scale2(t4[3], sa, w4[3]));
                        *(float4*)((float*)out + off) = o;
                    } else {
                        *(int4*)((int32_t*)out + off) = tot[i];
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (col + j >= N) break;
                        if (EPI == EPI_BF16) ((__nv_bfloat16*)out)[off + j] = __float2bfloat16_rn(scale2(t4[j], sa, w4[j]));
                        else if (EPI == EPI_ADD) ((float*)out)[off + j] = __fadd_rn(((float*)out)[off + j], scale2(t4[j], sa, w4[j]));
                        else ((int32_t*)out)[off + j] = t4[j];
                    }
                }
            }
        }
    }
}

template <int BN>
struct TileCfg {
    static constexpr int STAGES = (BN >= 192) ? 4 : 6;
    static constexpr int A_BYTES = BM * BK;
    static constexpr int W_BYTES = BN * BK;
    static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
    static constexpr int ACC_COLS = 2 * BN;                            // two accumulator buffers
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128
                                   : ACC_COLS <= 256 ? 256 : 512;
    // + control block + scale stash + per-warp staging: (2 stashes, 4 x 33-word-pitch buffers) or, for the residual
    // add, (1 stash, 8 x 32-word-pitch buffers)
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + (int)sizeof(Aux) + 2 * BN * 4 + 4 * 32 * 33 * 4;
    // (the residual add's boxes are copy-engine sources with the 128-byte swizzle: 1024-byte aligned)
    static constexpr int SMEM_ADD = 1024 + (STAGES * STAGE_BYTES + (int)sizeof(Aux) + BN * 4 + 1023) / 1024 * 1024 + 8 * 32 * 32 * 4;
};

// Row blocks of an int32 output that live in different buffers (a row-parallel projection on several GPUs: the rows
// another GPU will fold go straight into that GPU's memory, peer stores over NVLink, as each tile is drained).  Block
// o covers output rows [o * rows, (o + 1) * rows) and starts at base[o]; rows is a multiple of the tile height, so a
// tile never straddles two blocks.  rows == 0: one buffer (`out`).
struct RowBlocks {
    void* base[8];
    int rows;
};

// A work unit of the persistent tile kernel: a whole tile, or one K slice of a tile.  The first `full` tiles are whole
// (K unsplit); each later tile is `split` units, one per K slice, neighbours in the unit order so that they finish
// together.  full == 0: every tile is split (few tiles, long K); full == all tiles: nothing is split; in between: only
// the last, partial wave of tiles is split over the SMs that would otherwise idle through it.
struct Unit {
    int t, z, kb0, kb1, split;
};
__device__ __forceinline__ Unit unit_of(int u, int full, int split, int kb_per_split, int KB) {
    if (u < full) return Unit{u, 0, 0, KB, 1};
    const int v = u - full, t = full + v / split, z = v % split;
    const int kb0 = z * kb_per_split;
    const int kb1 = kb0 + kb_per_split < KB ? kb0 + kb_per_split : KB;
    return Unit{t, z, kb0, kb1, split};
}

// Epilogue warps: four (one per tensor-memory lane quarter), eight for the residual add (two per quarter, half the
// columns each: its global round trips are what the main loop must hide).
template <int EPI>
struct TileWarps {
    static constexpr int EPI_WARPS = EPI == EPI_ADD ? 8 : 4;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
};

template <int BN, int EPI>
__global__ void __launch_bounds__(TileWarps<EPI>::THREADS, 1)
w8a8_tile_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                 const __grid_constant__ CUtensorMap tm_out, const float* __restrict__ a_s, const float* __restrict__ w_s, void* __restrict__ out, long ldo,
                 const int* __restrict__ n_rows, int M, int N, int K, int word_ok, int split, int kb_per_split,
                 int32_t* __restrict__ ws, int* __restrict__ counters, const __grid_constant__ RowBlocks rb,
                 float* __restrict__ souts, int gbn, int full_tiles) {
    using C = TileCfg<BN>;
    using W = TileWarps<EPI>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    Aux* aux = (Aux*)(smem + C::STAGES * C::STAGE_BYTES);
    float* sw_stash = (float*)(aux + 1);
    uint32_t* stage_buf = (uint32_t*)(sw_stash + (EPI == EPI_ADD ? 1 : 2) * BN);   // per-warp transpose staging
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *n_rows;
    live = live < M ? live : M;
    const int num_m = (live + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    const int num_tiles = num_m * num_n, KB = (K + BK - 1) / BK;
    // work units: whole tiles first, then (tile, K slice) for the rest (unit_of)
    const int full = full_tiles < num_tiles ? full_tiles : num_tiles;
    const int num_units = full + (num_tiles - full) * split;
    // Tile order.  Row tiles fastest: a weight panel is read once and the activations come back from L2 for every
    // panel - right while the activations fit in L2.  Weight tiles fastest (bit 3 of word_ok): a group of row tiles
    // is read once and the weights come back from L2 - right when the activations are the larger operand and the
    // weights fit (down projection at many rows).
    const bool n_fastest = (word_ok & 8) != 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&aux->tfull[b]), 1);
            mbar_init(smem_u32(&aux->tempty[b]), W::EPI_WARPS);
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
        // ------------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            tma_prefetch_desc(&tm_a);
            tma_prefetch_desc(&tm_w);
            const uint64_t pol_keep = policy_evict_last();
            uint32_t armed_parity[C::STAGES];
            uint32_t armed_mask = 0;
            int stage = 0;
            uint32_t phase = 0;
            // bit 4 of word_ok (failure injection from the host, pb_test_drop_loads): this producer requests nothing, so
            // the MMA thread's bounded wait for the first stage expires and the CTA leaves through its abort path
            bool ok = !(word_ok & 16);
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const Unit un = unit_of(u, full, split, kb_per_split, KB);
                const int t = un.t;
                const int m0 = (n_fastest ? t / num_n : t % num_m) * BM, n0 = (n_fastest ? t % num_n : t / num_m) * BN;
                for (int kb = un.kb0; kb < un.kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0x100 + stage)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&aux->full[stage]);
                    mbar_expect_tx(bar, C::STAGE_BYTES);
                    uint8_t* st = smem + stage * C::STAGE_BYTES;
                    if (EPI == EPI_ADD) {                     // keep the operands in L2 against the residual stream
                        tma_load_2d_hint(smem_u32(st), &tm_a, kb * BK, m0, bar, pol_keep);
                        tma_load_2d_hint(smem_u32(st + C::A_BYTES), &tm_w, kb * BK, n0, bar, pol_keep);
                    } else {
                        tma_load_2d(smem_u32(st), &tm_a, kb * BK, m0, bar);
                        tma_load_2d(smem_u32(st + C::A_BYTES), &tm_w, kb * BK, n0, bar);
                    }
                    armed_parity[stage] = phase;
                    armed_mask |= 1u << stage;
                    if (++stage == C::STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok && armed_mask) drain_armed(aux, C::STAGES, armed_parity, armed_mask);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one thread)
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(BM, BN);
            int stage = 0, buf = 0;
            uint32_t phase = 0, bphase = 0;
            bool ok = true;
            // An mbarrier test costs this thread about 200 cycles before its answer can be used, as much as issuing
            // two MMAs.  So the test of the NEXT stage's barrier is issued before the current stage's MMAs and its
            // answer read after them: the thread stays ahead of the tensor core (512 cycles per stage).
            bool ready = mbar_test(smem_u32(&aux->full[0]), 0);
            for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                const Unit un = unit_of(u, full, split, kb_per_split, KB);
                const int kb_begin = un.kb0, kb_end = un.kb1;
                if (!mbar_wait(smem_u32(&aux->tempty[buf]), bphase ^ 1, abort_flag, 0x200 + buf)) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!ready && !mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x300 + stage)) {
                        ok = false;
                        break;
                    }
                    const int nstage = stage + 1 == C::STAGES ? 0 : stage + 1;
                    const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
                    const bool ready_next = mbar_test(smem_u32(&aux->full[nstage]), nphase);
                    tc_fence_after();
                    uint8_t* st = smem + stage * C::STAGE_BYTES;
                    const uint64_t ad = umma_desc_k128(smem_u32(st));
                    const uint64_t bd = umma_desc_k128(smem_u32(st + C::A_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        umma_i8(d, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc,
                                ((kb - kb_begin) | k) ? 1u : 0u);
                    tc_commit(smem_u32(&aux->empty[stage]));
                    stage = nstage;
                    phase = nphase;
                    ready = ready_next;
                }
                if (!ok) break;
                tc_commit(smem_u32(&aux->tfull[buf]));
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (one lane quarter per warp)
        constexpr int ET = 32 * W::EPI_WARPS;                    // epilogue threads
        const int q = warp & 3, et = threadIdx.x - 64;
        const int half = (warp - 2) >> 2;                        // EPI_ADD: which half of the columns
        int buf = 0;
        uint32_t bphase = 0;
        for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
            const Unit un = unit_of(u, full, split, kb_per_split, KB);
            const int t = un.t, z = un.z;
            const int m0 = (n_fastest ? t / num_n : t % num_m) * BM, n0 = (n_fastest ? t % num_n : t / num_m) * BN;
            float* swb = sw_stash + (EPI == EPI_ADD ? 0 : buf * BN);
            void* out_t = out;
            if (EPI == EPI_I32 && rb.rows > 0) {
                // this tile's row block: its buffer, moved back by the block's first row so that the global row
                // index addresses it
                const int o = m0 / rb.rows;
                out_t = (int32_t*)rb.base[o] - (long)o * rb.rows * ldo;
            }
            if (EPI == EPI_ADD) {
                // one scale stash: everyone must be done with the previous tile's before it is rewritten
                asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
            }
            if (EPI != EPI_I32)
                for (int i = et; i < BN; i += ET) swb[i] = (n0 + i < N) ? w_s[n0 + i] : 0.0f;
            if (EPI == EPI_ADD && !(word_ok & 6)) {
                // (register path only: the memory-side adds need no early copy in L2, it measured as a loss there)
                // the residual rows this CTA adds into one tile from now: pulled into L2 while that tile's main loop
                // runs (the first tile's are requested as its main loop starts)
                const int tn = (u == (int)blockIdx.x) ? u : u + (int)gridDim.x;
                for (int pass = 0; pass < 2; ++pass) {
                    const int uu = pass == 0 ? tn : tn + (int)gridDim.x;
                    if (pass == 1 && u != (int)blockIdx.x) break;
                    if (uu >= num_units) break;
                    const int tt = unit_of(uu, full, split, kb_per_split, KB).t;
                    const int pm0 = (n_fastest ? tt / num_n : tt % num_m) * BM, pn0 = (n_fastest ? tt % num_n : tt / num_m) * BN;
                    for (int line = et; line < BM * (BN / 32); line += ET) {
                        const int pr = pm0 + line / (BN / 32), pc = pn0 + (line % (BN / 32)) * 32;
                        if (pr < live && pc < N)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"((const float*)out + (long)pr * ldo + pc));
                    }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
            if (!mbar_wait(smem_u32(&aux->tfull[buf]), bphase, abort_flag, 0x400 + buf)) break;
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const bool rok = row < live;
            const float sa = (rok && EPI != EPI_I32) ? a_s[row] : 0.0f;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            if (un.split > 1) {
                // this slice's int32 accumulator -> workspace (the four warps of the first column half do it all)
                int32_t* ws_tile = ws + (long)(t - full) * split * (BM * BN);
                if (half == 0) {
                    uint32_t* stg = stage_buf + q * (32 * 33);
                    drain_accumulator<BN, EPI_I32>(ws_tile + (long)z * (BM * BN), BN, BN, BM, 0, 0, q, lane, lane_addr,
                                                   stg, swb, 0.0f, true);
                }
                // the accumulator buffer is free again: the next unit's MMAs may start while this tile is reduced
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&aux->tempty[buf]));
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
                if (et == 0) {
                    const int old = atomicAdd(counters + (t - full), 1);
                    aux->is_last = (old == split - 1);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
                if (aux->is_last) {
                    __threadfence();
                    const int cb = EPI == EPI_ADD ? half * (BN / 2) : 0, ce = EPI == EPI_ADD ? (half + 1) * (BN / 2) : BN;
                    reduce_store<BN, EPI>(out_t, ldo, N, live, m0, n0, q, lane, ws_tile, (long)BM * BN, split, swb, sa, cb,
                                          ce);
                    if (et == 0) counters[t - full] = 0;
                }
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
                continue;
            }
            if (EPI == EPI_ADD && (word_ok & 2)) {
                uint32_t* box = (uint32_t*)(((uintptr_t)stage_buf + 1023) & ~(uintptr_t)1023) + (warp - 2) * (32 * 32);
                drain_add_tma(&tm_out, N, live, m0, n0, q, lane, lane_addr, box, swb, sa, half * (BN / 2),
                              (half + 1) * (BN / 2));
            } else if (EPI == EPI_ADD && (word_ok & 4)) {
                uint32_t* stg = stage_buf + (warp - 2) * (32 * 32);
                drain_add_red((float*)out, ldo, N, live, m0, n0, q, lane, lane_addr, stg, swb, sa, half * (BN / 2),
                              (half + 1) * (BN / 2));
            } else if (EPI == EPI_ADD) {
                uint32_t* stg = stage_buf + (warp - 2) * (32 * 32);
                drain_add((float*)out, ldo, N, live, m0, n0, q, lane, lane_addr, stg, swb, sa, half * (BN / 2),
                          (half + 1) * (BN / 2));
            } else if (EPI == EPI_SWIGLU) {
                if (gbn == 128) drain_swiglu<BN, 64>((int8_t*)out, ldo, souts, N, live, m0, n0, q, lane, lane_addr, swb, sa);
                else drain_swiglu<BN, 32>((int8_t*)out, ldo, souts, N, live, m0, n0, q, lane, lane_addr, swb, sa);
            } else {
                uint32_t* stg = stage_buf + q * (32 * 33);
                drain_accumulator<BN, EPI>(out_t, ldo, N, live, m0, n0, q, lane, lane_addr, stg, swb, sa, (word_ok & 1) != 0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&aux->tempty[buf]));
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
        // reductions still in flight read this CTA's shared memory: they complete before the CTA ends
        if (EPI == EPI_ADD && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (EPI == EPI_I32 && rb.rows > 0) __threadfence_system();   // stores into other GPUs' memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}


// ================================================================================================= pair kernel
// The tile kernel on CTA pairs (clusters of two, tcgen05 cta_group::2): a pair owns a 256 x 256 output tile; each CTA
// loads its own 128 activation rows and its own 128 of the 256 weight rows per K block (32 KB instead of the single-CTA
// kernel's 48 KB for the same tensor work, and half the weight tile's shared-memory reads), the leader (cluster rank
// 0) issues 256 x 256 x 32 MMAs that write 128 accumulator lanes in each CTA, and each CTA's epilogue warps drain their
// own lanes.  Barriers: `full` lives in the leader and counts both CTAs' bytes; `empty` and `tfull` exist in both CTAs
// and are each committed to by the leader; `tempty` lives in the leader and takes one arrival per epilogue warp of
// both CTAs.  No multicast anywhere.
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = 2 * BM * BK;                     // 16 KB of A + 16 KB of B per CTA
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + (int)sizeof(Aux) + 2 * PAIR_BN * 4 + 4 * 32 * 33 * 4;

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
w8a8_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                 const float* __restrict__ a_s, const float* __restrict__ w_s, void* __restrict__ out, long ldo,
                 const int* __restrict__ n_rows, int M, int N, int K, int word_ok) {
    constexpr int BN = PAIR_BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    Aux* aux = (Aux*)(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
    float* sw_stash = (float*)(aux + 1);
    uint32_t* stage_buf = (uint32_t*)(sw_stash + 2 * BN);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;

    int live = *n_rows;
    live = live < M ? live : M;
    const int num_m = (live + 2 * BM - 1) / (2 * BM), num_n = (N + BN - 1) / BN;
    const int num_tiles = num_m * num_n, KB = (K + BK - 1) / BK;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);                // used in the leader only
            mbar_init(smem_u32(&aux->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&aux->tfull[b]), 1);
            mbar_init(smem_u32(&aux->tempty[b]), 8);              // used in the leader only: 4 warps of each CTA
        }
        aux->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&aux->tmem_base), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                            // both CTAs' barriers exist before any remote use
    tc_fence_after();
    const uint32_t tmem_base = aux->tmem_base;
    volatile int* abort_flag = &aux->abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one thread per CTA)
        if (lane == 0) {
            tma_prefetch_desc(&tm_a);
            tma_prefetch_desc(&tm_w);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += npairs) {
                const int m0 = (t % num_m) * 2 * BM + (int)rank * BM, n0 = (t / num_m) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0x1100 + stage)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = map_to_cta(smem_u32(&aux->full[stage]), 0);
                    if (leader) mbar_expect_tx(smem_u32(&aux->full[stage]), 2 * PAIR_STAGE_BYTES);
                    uint8_t* st = smem + stage * PAIR_STAGE_BYTES;
                    tma_load_2d_pair(smem_u32(st), &tm_a, kb * BK, m0, bar);
                    tma_load_2d_pair(smem_u32(st + BM * BK), &tm_w, kb * BK, n0, bar);
                    if (++stage == PAIR_STAGES) {
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
        // ------------------------------------------------------------------ MMA issuer (the leader's one thread)
        if (leader && lane == 0) {
            const uint32_t idesc = umma_idesc_i8(2 * BM, BN);
            int stage = 0, buf = 0;
            uint32_t phase = 0, bphase = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += npairs) {
                if (!mbar_wait(smem_u32(&aux->tempty[buf]), bphase ^ 1, abort_flag, 0x1200 + buf)) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * BN;
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x1300 + stage)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint8_t* st = smem + stage * PAIR_STAGE_BYTES;
                    const uint64_t ad = umma_desc_k128(smem_u32(st));
                    const uint64_t bd = umma_desc_k128(smem_u32(st + BM * BK));
#pragma unroll
                    for (int k = 0; k < BK / 32; ++k)
                        umma_i8_pair(d, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc,
                                     (kb | k) ? 1u : 0u);
                    const uint32_t eb = smem_u32(&aux->empty[stage]);
                    tc_commit_pair(eb);                           // this CTA's producer may refill the stage ...
                    tc_commit_pair(map_to_cta(eb, 1));            // ... and the peer's
                    if (++stage == PAIR_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                const uint32_t fb = smem_u32(&aux->tfull[buf]);
                tc_commit_pair(fb);
                tc_commit_pair(map_to_cta(fb, 1));
                buf ^= 1;
                if (buf == 0) bphase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps per CTA, own lanes)
        const int q = warp & 3, et = threadIdx.x - 64;
        int buf = 0;
        uint32_t bphase = 0;
        for (int t = pair; t < num_tiles; t += npairs) {
            const int m0 = (t % num_m) * 2 * BM + (int)rank * BM, n0 = (t / num_m) * BN;
            float* swb = sw_stash + buf * BN;
            if (EPI != EPI_I32)
                for (int i = et; i < BN; i += 128) swb[i] = (n0 + i < N) ? w_s[n0 + i] : 0.0f;
            if (EPI == EPI_ADD) {
                const int tn = (t == pair) ? t : t + npairs;
                for (int pass = 0; pass < 2; ++pass) {
                    const int tt = pass == 0 ? tn : tn + npairs;
                    if (pass == 1 && t != pair) break;
                    if (tt >= num_tiles) break;
                    const int pm0 = (tt % num_m) * 2 * BM + (int)rank * BM, pn0 = (tt / num_m) * BN;
                    for (int line = et; line < BM * (BN / 32); line += 128) {
                        const int pr = pm0 + line / (BN / 32), pc = pn0 + (line % (BN / 32)) * 32;
                        if (pr < live && pc < N)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"((const float*)out + (long)pr * ldo + pc));
                    }
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!mbar_wait(smem_u32(&aux->tfull[buf]), bphase, abort_flag, 0x1400 + buf)) break;
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const float sa = (row < live && EPI != EPI_I32) ? a_s[row] : 0.0f;
            uint32_t* stg = stage_buf + q * (32 * 33);
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            drain_accumulator<BN, EPI>(out, ldo, N, live, m0, n0, q, lane, lane_addr, stg, swb, sa, word_ok != 0);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&aux->tempty[buf]), 0));
            buf ^= 1;
            if (buf == 0) bphase ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                            // no CTA leaves while its peer may still signal it
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// ================================================================================================= swapped kernel
// MODE_DIRECT: the CTA owns all of K (split = 1): scales + store (bf16 / fp32 add / int32).
// MODE_SLOTS:  int32 partial sums of K slice z into slots[z] (int32 [S, rows, N]); the caller folds them later.
// MODE_WS:     int32 partial sums into a workspace; the last CTA to finish a tile (a counter per tile) adds the
//              slices and runs the epilogue.  Counters return to zero.
constexpr int MODE_DIRECT = 0, MODE_SLOTS = 1, MODE_WS = 2;

template <int NB, bool GROUPED>
struct SwapCfg {
    static constexpr int W_BYTES = BM * BK;                      // 16 KB
    static constexpr int X_BYTES = NB * BK;
    static constexpr int SW_BYTES = 0;                           // weight group scales: read by their thread, not staged
    static constexpr int SA_BYTES = GROUPED ? NB * 16 : 0;       // 4 fp32 group scales per activation row
    static constexpr int STAGE_BYTES_RAW = W_BYTES + X_BYTES + SW_BYTES + SA_BYTES;
    static constexpr int STAGE_BYTES = (STAGE_BYTES_RAW + 1023) / 1024 * 1024;
    // about 110 KB per CTA, so that two CTAs share an SM, when the grid has more CTAs than SMs; otherwise one CTA per
    // SM with all the shared memory (bytes in flight per SM are what hides the DRAM latency)
    static constexpr int STAGES = (108 * 1024 / STAGE_BYTES) > 8 ? 8 : (108 * 1024 / STAGE_BYTES);
    static constexpr int STAGES_DEEP = (212 * 1024 / STAGE_BYTES) > 12 ? 12 : (212 * 1024 / STAGE_BYTES);
    // per-32 groups: an accumulator slot takes SUPER K stages (4 groups of NB columns each) and the epilogue warps drain
    // a whole slot per hand-off: one barrier round trip and one tensor-memory load latency per SUPER stages instead of
    // per stage (that chain of latencies, about 1,000 cycles per stage, was the kernel's whole time).  Two slots: the
    // MMAs of the next fill while the epilogue drains this one.  512 columns: one CTA per SM.
    static constexpr int SUPER = GROUPED ? (NB == 16 ? 4 : NB == 32 ? 2 : 1) : 1;
    static constexpr int BATCH_COLS = GROUPED ? SUPER * 4 * NB : NB;
    static constexpr int RING = GROUPED ? 2 : 1;
    static constexpr int ACC_COLS = BATCH_COLS * RING;
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128
                                   : ACC_COLS <= 256 ? 256 : 512;
    static constexpr int smem_bytes(int stages) { return stages * STAGE_BYTES + 1024 + (int)sizeof(Aux); }
    // per-32 groups keep the epilogue warps busy after every stage: two warps per lane quarter from 16 rows up
    static constexpr int EPI_WARPS = (GROUPED && NB >= 16) ? 8 : 4;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
};

struct SwapArgs {
    const float* a_s;       // [M] (gk == K) or [M, K/32] (GROUPED; read through tm_sa)
    const float* w_s;       // [N] (gk == K) or [N, K/32] (GROUPED: each thread reads its row)
    void* out;              // bf16 / fp32 / int32 [M, N]; MODE_SLOTS: slots base
    long ldo;               // row stride of out (elements)
    long slot_stride;       // MODE_SLOTS: elements between slots
    int32_t* ws;            // MODE_WS: split * tiles * NB * 128 int32
    int* counters;          // MODE_WS: one per (n tile, m tile)
    const int* n_rows;
    int M, N, K;
    int kb_per_split;       // 128-byte K blocks per blockIdx.y
    int epi;                // EPI_BF16 / EPI_ADD / EPI_I32
    int mode;
    int pdl;                // launched as a programmatic dependent: weights may stream before the wait
    int stages;             // pipeline depth (shared-memory stages per CTA)
    int gblocks;            // w8a8_groups_kernel: 32-input blocks per scale group (gk / 32)
    int wrows;              // per-32 groups, one K slice: weight rows per CTA (32, 64 or 128; 0 = 128).  Fewer rows =
                            // more CTAs when N / 128 tiles leave SMs idle; the MMA still spans 128 lanes, the spare
                            // lanes' sums are never read
};

template <int NB>
__device__ __forceinline__ void swap_store(const SwapArgs& p, int n, int m0, int live, const float (&v)[NB]) {
    // thread = output column n; v[j] = value of row m0 + j.  A warp's 32 lanes write 32 consecutive columns.
    if (n >= p.N) return;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int m = m0 + j;
        if (m < live) {
            if (p.epi == EPI_BF16)
                ((__nv_bfloat16*)p.out)[(long)m * p.ldo + n] = __float2bfloat16_rn(v[j]);
            else if (p.epi == EPI_F32)
                ((float*)p.out)[(long)m * p.ldo + n] = v[j];
            else {
                float* o = (float*)p.out + (long)m * p.ldo + n;
                *o = __fadd_rn(*o, v[j]);
            }
        }
    }
}

// One K stage's four scale groups of CH (2, 4 or 8) activation rows (c .. c + CH - 1 of this warp's rows), added to the rows' fp32 sums
// in ascending group order.  r[g][j]: the int32 sum of group g and row c + j; sa4[row * stride]: the row's four
// activation scales of this stage; sw4: this thread's weight row's four scales.
//   plain: (float(sum) * sa) * sw, each product rounded (two rows per packed multiply), then a scalar add_rn.  The adds
//          stay scalar on purpose: the assembler contracts a packed multiply followed by a packed add into one fused
//          multiply-add (measured: 15 % of results change), which would break the reference's two-rounding contract.
//   fuse:  the vocabulary head - the reference's kernel writes `acc += (ai * sa) * sw` without explicit roundings
//          (kernels/decode.py:157) and its compiler fuses the second multiply with the add: one rounded product, then
//          a fused multiply-add, per group.
// Two int32 group sums as floats.  A sum of 32 products of int8 values is below 2^19 in magnitude, so adding it to the
// bit pattern of 1.5 * 2^23 and subtracting that constant gives exactly float(sum): one integer add each and one packed
// fp32 add for the pair, instead of two conversions on the slower conversion unit.
__device__ __forceinline__ float2 float2_of(uint32_t a, uint32_t b) {
    return __fadd2_rn(make_float2(__uint_as_float(0x4B400000u + a), __uint_as_float(0x4B400000u + b)),
                      make_float2(-12582912.0f, -12582912.0f));
}

template <int CH>
__device__ __forceinline__ void add_stage_groups(float2* acc, int c, const uint32_t (&r)[4][CH], const float4* sa4,
                                                 int stride, const float4 sw4, bool fuse) {
    const float2 w0 = make_float2(sw4.x, sw4.x), w1 = make_float2(sw4.y, sw4.y), w2 = make_float2(sw4.z, sw4.z),
                 w3 = make_float2(sw4.w, sw4.w);
    if (fuse) {
        // two rows per instruction: one packed multiply and one packed fused multiply-add per group (each lane
        // rounded as the scalar operation: the bits of fma(float(sum) * sa, sw, acc))
#pragma unroll
        for (int j = 0; j < CH; j += 2) {
            const float4 s0 = sa4[(c + j) * stride], s1 = sa4[(c + j + 1) * stride];
            float2 a = acc[(c + j) >> 1];
            a = __ffma2_rn(__fmul2_rn(float2_of(r[0][j], r[0][j + 1]),
                                      make_float2(s0.x, s1.x)), w0, a);
            a = __ffma2_rn(__fmul2_rn(float2_of(r[1][j], r[1][j + 1]),
                                      make_float2(s0.y, s1.y)), w1, a);
            a = __ffma2_rn(__fmul2_rn(float2_of(r[2][j], r[2][j + 1]),
                                      make_float2(s0.z, s1.z)), w2, a);
            a = __ffma2_rn(__fmul2_rn(float2_of(r[3][j], r[3][j + 1]),
                                      make_float2(s0.w, s1.w)), w3, a);
            acc[(c + j) >> 1] = a;
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < CH; j += 2) {
        const float4 s0 = sa4[(c + j) * stride], s1 = sa4[(c + j + 1) * stride];
        float2 a = acc[(c + j) >> 1];
        float2 t;
        t = __fmul2_rn(__fmul2_rn(float2_of(r[0][j], r[0][j + 1]),
                                  make_float2(s0.x, s1.x)), w0);
        a.x = __fadd_rn(a.x, t.x); a.y = __fadd_rn(a.y, t.y);
        t = __fmul2_rn(__fmul2_rn(float2_of(r[1][j], r[1][j + 1]),
                                  make_float2(s0.y, s1.y)), w1);
        a.x = __fadd_rn(a.x, t.x); a.y = __fadd_rn(a.y, t.y);
        t = __fmul2_rn(__fmul2_rn(float2_of(r[2][j], r[2][j + 1]),
                                  make_float2(s0.z, s1.z)), w2);
        a.x = __fadd_rn(a.x, t.x); a.y = __fadd_rn(a.y, t.y);
        t = __fmul2_rn(__fmul2_rn(float2_of(r[3][j], r[3][j + 1]),
                                  make_float2(s0.w, s1.w)), w3);
        a.x = __fadd_rn(a.x, t.x); a.y = __fadd_rn(a.y, t.y);
        acc[(c + j) >> 1] = a;
    }
}

// RW > 0 (per-32 groups, NB = 16 only): the CTA owns 2 * RW activation rows (4 or 8) instead of NB - the MMA still spans
// NB rows (its minimum), the epilogue warps take RW rows each.  More CTAs share one weight tile (re-read from L2), so
// the per-group fp32 arithmetic of a short batch spreads over more SMs when the weight tiles are fewer than the SMs.
template <int NB, bool GROUPED, int RW = 0>
__global__ void __launch_bounds__(SwapCfg<NB, GROUPED>::THREADS, 1)
w8a8_swap_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                 const __grid_constant__ CUtensorMap tm_sw, const __grid_constant__ CUtensorMap tm_sa,
                 const SwapArgs p) {
    using C = SwapCfg<NB, GROUPED>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    const int NST = p.stages;                                  // pipeline depth chosen by the host (2 .. 12)
    Aux* aux = (Aux*)(smem + NST * C::STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int live = *p.n_rows;
    live = live < p.M ? live : p.M;
    const int WR = (GROUPED && p.wrows > 0) ? p.wrows : BM;     // weight rows this CTA owns
    constexpr int RCTA = RW ? 2 * RW : NB;                     // activation rows this CTA owns
    const int n0 = blockIdx.x * WR, m0 = blockIdx.z * RCTA, z = blockIdx.y;
    if (m0 >= live) return;                                    // whole CTA, before any barrier or allocation
    const int KB = (p.K + BK - 1) / BK;
    const int kb0 = z * p.kb_per_split;
    int kb1 = kb0 + p.kb_per_split;
    kb1 = kb1 < KB ? kb1 : KB;
    const int nkb = kb1 > kb0 ? kb1 - kb0 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(smem_u32(&aux->full[s]), 1);
            mbar_init(smem_u32(&aux->empty[s]), GROUPED ? C::EPI_WARPS : 1);   // the MMA's commit, or (per-32 groups) the epilogue warps
        }
        for (int b = 0; b < C::RING; ++b) {
            mbar_init(smem_u32(&aux->tfull[b]), 1);
            mbar_init(smem_u32(&aux->tempty[b]), C::EPI_WARPS);
        }
        aux->abort_flag = 0;
        aux->is_last = 0;
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
    if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel may begin its set-up

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_w);
            tma_prefetch_desc(&tm_x);
            const uint64_t pol_w = policy_evict_first();       // weights are read once
            uint32_t armed_parity[12];
            uint32_t armed_mask = 0;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // Programmatic dependent launch: this grid may start while the kernel before it (the producer of the
            // activations) still runs.  The weights do not depend on it: the first stages' weight tiles are requested
            // at once, the activation tiles after the wait.
            const int pre = p.pdl ? (nkb < NST ? nkb : NST) : 0;
            const uint32_t stage_tx = C::STAGE_BYTES_RAW - C::W_BYTES + WR * BK;   // bytes a stage's copies deliver
            for (int i = 0; i < pre; ++i) {
                const uint32_t bar = smem_u32(&aux->full[i]);
                mbar_expect_tx(bar, stage_tx);
                uint8_t* st = smem + i * C::STAGE_BYTES;
                tma_load_2d_hint(smem_u32(st), &tm_w, (kb0 + i) * BK, n0, bar, pol_w);
                armed_parity[i] = 0;
                armed_mask |= 1u << i;
            }
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < pre; ++i) {
                const uint32_t bar = smem_u32(&aux->full[i]);
                uint8_t* st = smem + i * C::STAGE_BYTES;
                tma_load_2d(smem_u32(st + C::W_BYTES), &tm_x, (kb0 + i) * BK, m0, bar);
                if (GROUPED)
                    tma_load_2d(smem_u32(st + C::W_BYTES + C::X_BYTES), &tm_sa, (kb0 + i) * 4, m0, bar);
            }
            if (pre == NST) phase = 1;
            else stage = pre;
            for (int i = pre; i < nkb; ++i) {
                if (!mbar_wait(smem_u32(&aux->empty[stage]), phase ^ 1, abort_flag, 0x500 + stage)) {
                    ok = false;
                    break;
                }
                const uint32_t bar = smem_u32(&aux->full[stage]);
                mbar_expect_tx(bar, stage_tx);
                uint8_t* st = smem + stage * C::STAGE_BYTES;
                const int kb = kb0 + i;
                tma_load_2d_hint(smem_u32(st), &tm_w, kb * BK, n0, bar, pol_w);
                tma_load_2d(smem_u32(st + C::W_BYTES), &tm_x, kb * BK, m0, bar);
                if (GROUPED) tma_load_2d(smem_u32(st + C::W_BYTES + C::X_BYTES), &tm_sa, kb * 4, m0, bar);
                armed_parity[stage] = phase;
                armed_mask |= 1u << stage;
                if (++stage == NST) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (!ok) drain_armed(aux, NST, armed_parity, armed_mask);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(BM, NB);
            int stage = 0, ring = 0;
            uint32_t phase = 0, rphase = 0;
            bool ok = true;
            // An mbarrier test keeps this thread waiting about 200 cycles for its answer: the tests of the NEXT stage's
            // barriers are issued before the current stage's MMAs, their answers read after them.
            bool ready = nkb > 0 && mbar_test(smem_u32(&aux->full[0]), 0);
            int sub = 0;                                             // per-32 groups: K stage inside the accumulator slot
            for (int i = 0; i < nkb && ok; ++i) {
                // a new slot must have been drained (a fresh barrier passes at once)
                if (GROUPED && sub == 0 &&
                    !mbar_wait(smem_u32(&aux->tempty[ring]), rphase ^ 1, abort_flag, 0x600 + ring)) {
                    ok = false;
                    break;
                }
                if (!ready && !mbar_wait(smem_u32(&aux->full[stage]), phase, abort_flag, 0x700 + stage)) {
                    ok = false;
                    break;
                }
                const int nstage = stage + 1 == NST ? 0 : stage + 1;
                const uint32_t nphase = nstage == 0 ? phase ^ 1 : phase;
                const bool ready_next = mbar_test(smem_u32(&aux->full[nstage]), nphase);
                tc_fence_after();
                uint8_t* st = smem + stage * C::STAGE_BYTES;
                const uint64_t ad = umma_desc_k128(smem_u32(st));
                const uint64_t bd = umma_desc_k128(smem_u32(st + C::W_BYTES));
#pragma unroll
                for (int k = 0; k < BK / 32; ++k) {
                    if (GROUPED)
                        umma_i8(tmem_base + ring * C::BATCH_COLS + (sub * 4 + k) * NB, umma_desc_advance(ad, k * 32),
                                umma_desc_advance(bd, k * 32), idesc, 0u);
                    else
                        umma_i8(tmem_base, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc,
                                (i | k) ? 1u : 0u);
                }
                if (GROUPED) {
                    // the epilogue warps hand the stages back themselves (they read the stages' scales after these MMAs
                    // have completed): one commit per slot
                    if (++sub == C::SUPER || i + 1 == nkb) {
                        tc_commit(smem_u32(&aux->tfull[ring]));
                        sub = 0;
                        if (++ring == C::RING) {
                            ring = 0;
                            rphase ^= 1;
                        }
                    }
                } else {
                    tc_commit(smem_u32(&aux->empty[stage]));
                }
                stage = nstage;
                phase = nphase;
                ready = ready_next;
            }
            if (!GROUPED && ok) tc_commit(smem_u32(&aux->tfull[0]));
        }
    } else {
        const int q = warp & 3;
        const int nl = q * 32 + lane;                          // this thread's weight row inside the tile
        if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");   // before any global read or write of this warp
        const int n = nl < WR ? n0 + nl : p.N;                 // lanes past this CTA's rows own no output column
        const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
        if (GROUPED) {
            const bool active = q * 32 < WR;                   // warp-uniform: does this lane quarter hold weight rows?
            // NH activation rows per warp: all NB with four epilogue warps, half of them with eight (two per lane quarter)
            constexpr int NH = RW ? RW : (C::EPI_WARPS == 8 ? NB / 2 : NB);
            constexpr int CH = NH < 8 ? NH : 8;                     // rows per tensor-memory load
            const int j0 = C::EPI_WARPS == 8 ? ((warp - 2) >> 2) * NH : 0;
            float2 acc[NH / 2];                                     // rows (j0 + 2i, j0 + 2i + 1)
#pragma unroll
            for (int j = 0; j < NH / 2; ++j) acc[j] = make_float2(0.0f, 0.0f);
            int stage = 0, ring = 0;
            uint32_t phase = 0, rphase = 0;
            bool ok = true;
            // this thread's weight row: four group scales (16 bytes) per stage, read straight from global memory (a
            // tensor-map box of 128 rows x 16 bytes costs the TMA unit a request per row)
            const float4* swp = (const float4*)(p.w_s + (long)(n < p.N ? n : 0) * (p.K >> 5)) + kb0;
            // The row's scales of this CTA's whole K range go to L2 now (16 bytes per stage, rows K / 8 bytes apart: a
            // scattered read whose DRAM latency, met once per slot, was the kernel's whole time), and the loads below run
            // AHEAD stages in front of their use, so that what they meet is an L2 hit with several slots to land.
            if (active) {
                const int part = C::EPI_WARPS == 8 ? (warp - 2) >> 2 : 0, parts = C::EPI_WARPS == 8 ? 2 : 1;
                const char* row = (const char*)swp;
                for (int off = part * 128; off < nkb * 16; off += parts * 128)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(row + off));
                if (part == 0 && nkb > 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(row + nkb * 16 - 16));
            }
            constexpr int AHEAD = C::SUPER > 4 ? C::SUPER : 4;
            float4 sw_ahead[AHEAD];
#pragma unroll
            for (int sidx = 0; sidx < AHEAD; ++sidx)
                sw_ahead[sidx] = sidx < nkb ? __ldg(swp + sidx) : make_float4(0.f, 0.f, 0.f, 0.f);
            const bool fuse = p.epi == EPI_F32;
            for (int i0 = 0; i0 < nkb && ok; i0 += C::SUPER) {
                const int ns = nkb - i0 < C::SUPER ? nkb - i0 : C::SUPER;      // K stages in this slot
                float4 sw4[C::SUPER];
#pragma unroll
                for (int sidx = 0; sidx < C::SUPER; ++sidx) sw4[sidx] = sw_ahead[sidx];
#pragma unroll
                for (int sidx = 0; sidx + C::SUPER < AHEAD; ++sidx) sw_ahead[sidx] = sw_ahead[sidx + C::SUPER];
#pragma unroll
                for (int sidx = 0; sidx < C::SUPER; ++sidx)
                    if (i0 + AHEAD + sidx < nkb) sw_ahead[AHEAD - C::SUPER + sidx] = __ldg(swp + i0 + AHEAD + sidx);
                if (!mbar_wait(smem_u32(&aux->tfull[ring]), rphase, abort_flag, 0x800 + ring)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                // the stages' scales landed with their operands: their full barriers have completed (the MMAs ran after
                // them); testing them here orders this thread's reads after the bulk copies' writes
                const float4* sa4[C::SUPER];
#pragma unroll
                for (int sidx = 0; sidx < C::SUPER; ++sidx) {
                    int st = stage + sidx;
                    uint32_t ph = phase;
                    if (st >= NST) {
                        st -= NST;
                        ph ^= 1;
                    }
                    sa4[sidx] = (const float4*)(smem + st * C::STAGE_BYTES + C::W_BYTES + C::X_BYTES) + j0;
                    if (sidx < ns && ok && !mbar_wait(smem_u32(&aux->full[st]), ph, abort_flag, 0x880 + st)) ok = false;
                }
                if (!ok) break;
#pragma unroll
                for (int c = 0; c < NH; c += CH) {
                    if (!active || m0 + j0 + c >= live) break;     // no weight rows here, or these rows are not live
                    // two stages' loads (eight of them) are in flight before each wait
                    constexpr int LB = C::SUPER >= 2 ? 2 : 1;
#pragma unroll
                    for (int s0 = 0; s0 < C::SUPER; s0 += LB) {
                        if (s0 >= ns) break;
                        uint32_t r[LB][4][CH];
#pragma unroll
                        for (int u = 0; u < LB; ++u)
                            if (s0 + u < ns) {
#pragma unroll
                                for (int g = 0; g < 4; ++g)
                                    tmem_ldn(lane_base + ring * C::BATCH_COLS + ((s0 + u) * 4 + g) * NB + j0 + c, r[u][g]);
                            }
                        tmem_ld_wait();
#pragma unroll
                        for (int u = 0; u < LB; ++u)
                            if (s0 + u < ns) add_stage_groups<CH>(acc, c, r[u], sa4[s0 + u], 1, sw4[s0 + u], fuse);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&aux->tempty[ring]));
                    for (int sidx = 0; sidx < ns; ++sidx) {
                        const int st = stage + sidx >= NST ? stage + sidx - NST : stage + sidx;
                        mbar_arrive(smem_u32(&aux->empty[st]));
                    }
                }
                if (++ring == C::RING) {
                    ring = 0;
                    rphase ^= 1;
                }
                stage += ns;
                if (stage >= NST) {
                    stage -= NST;
                    phase ^= 1;
                }
            }
            float v[NH];
#pragma unroll
            for (int j = 0; j < NH / 2; ++j) {
                v[2 * j] = acc[j].x;
                v[2 * j + 1] = acc[j].y;
            }
            if (p.mode == MODE_WS) {
                // K split over blockIdx.y: every slice has added its own groups in order from zero; the last CTA of
                // the tile adds the slices' fp32 sums in slice order (deterministic, but not the unsplit order: results
                // agree with it to fp32 rounding, i.e. within one bf16 step after the store)
                constexpr int ET = 32 * C::EPI_WARPS;
                uint32_t got = ok ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\t"
                    "setp.ne.u32 p, %1, 0;\n\t"
                    "bar.red.and.pred q, 1, %2, p;\n\t"
                    "selp.u32 %0, 1, 0, q;\n\t}"
                    : "=r"(got) : "r"(got), "n"(ET) : "memory");
                if (got) {
                    const int tile = blockIdx.z * gridDim.x + blockIdx.x;
                    const long tile_elems = (long)NB * BM;
                    float* ws = (float*)p.ws;
                    float* mine = ws + ((long)z * gridDim.x * gridDim.z + tile) * tile_elems;
#pragma unroll
                    for (int j = 0; j < NH; ++j) mine[(j0 + j) * BM + nl] = v[j];
                    __threadfence();
                    asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
                    if (threadIdx.x == 64) {
                        const int old = atomicAdd(p.counters + tile, 1);
                        aux->is_last = (old == (int)gridDim.y - 1);
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
                    if (aux->is_last) {
                        __threadfence();
#pragma unroll
                        for (int j = 0; j < NH; ++j) v[j] = 0.0f;
                        for (int sl = 0; sl < (int)gridDim.y; ++sl) {
                            const float* src = ws + ((long)sl * gridDim.x * gridDim.z + tile) * tile_elems + nl;
#pragma unroll
                            for (int j = 0; j < NH; ++j) {
                                const float part = __ldcg(src + (j0 + j) * BM);
                                v[j] = sl == 0 ? part : __fadd_rn(v[j], part);
                            }
                        }
                        swap_store<NH>(p, n, m0 + j0, live, v);
                        if (threadIdx.x == 64) p.counters[tile] = 0;
                    }
                }
            } else if (ok) {
                swap_store<NH>(p, n, m0 + j0, live, v);
            }
        } else {
            // every epilogue thread takes the same branch: the barrier-wide AND of the wait's outcome
            uint32_t got = (nkb > 0 && mbar_wait(smem_u32(&aux->tfull[0]), 0, abort_flag, 0x900)) ? 1u : 0u;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.u32 p, %1, 0;\n\t"
                "bar.red.and.pred q, 1, 128, p;\n\t"
                "selp.u32 %0, 1, 0, q;\n\t}"
                : "=r"(got) : "r"(got) : "memory");
            if (got) {
                tc_fence_after();
                int32_t acc[NB];
#pragma unroll
                for (int c = 0; c < NB; c += 8) {
                    uint32_t r[8];
                    tmem_ld8(lane_base + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[c + j] = (int32_t)r[j];
                }
                if (p.mode == MODE_SLOTS || (p.mode == MODE_DIRECT && p.epi == EPI_I32)) {
                    int32_t* o = (int32_t*)p.out + (p.mode == MODE_SLOTS ? (long)z * p.slot_stride : 0);
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < NB; ++j)
                            if (m0 + j < live) o[(long)(m0 + j) * p.ldo + n] = acc[j];
                    }
                } else if (p.mode == MODE_DIRECT) {
                    const float sw = n < p.N ? p.w_s[n] : 0.0f;
                    float v[NB];
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
                        const float sa = (m0 + j < live) ? __ldg(p.a_s + m0 + j) : 0.0f;
                        v[j] = scale2(acc[j], sa, sw);
                    }
                    swap_store<NB>(p, n, m0, live, v);
                } else {
                    // workspace: ws[z][tile][j][128]; the last CTA of the tile adds the slices in slice order
                    const int tile = blockIdx.z * gridDim.x + blockIdx.x;
                    const long tile_elems = (long)NB * BM;
                    int32_t* mine = p.ws + ((long)z * gridDim.x * gridDim.z + tile) * tile_elems;
#pragma unroll
                    for (int j = 0; j < NB; ++j) mine[j * BM + nl] = acc[j];
                    __threadfence();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (threadIdx.x == 64) {
                        const int old = atomicAdd(p.counters + tile, 1);
                        aux->is_last = (old == (int)gridDim.y - 1);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (aux->is_last) {
                        __threadfence();
                        const float sw = n < p.N ? p.w_s[n] : 0.0f;
                        int32_t tot[NB];
#pragma unroll
                        for (int j = 0; j < NB; ++j) tot[j] = 0;
                        for (int s = 0; s < (int)gridDim.y; ++s) {
                            const int32_t* src = p.ws + ((long)s * gridDim.x * gridDim.z + tile) * tile_elems + nl;
#pragma unroll
                            for (int j = 0; j < NB; ++j) tot[j] += __ldcg(src + j * BM);
                        }
                        float v[NB];
#pragma unroll
                        for (int j = 0; j < NB; ++j) {
                            const float sa = (m0 + j < live) ? __ldg(p.a_s + m0 + j) : 0.0f;
                            v[j] = scale2(tot[j], sa, sw);
                        }
                        swap_store<NB>(p, n, m0, live, v);
                        if (threadIdx.x == 64) p.counters[tile] = 0;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ================================================================================================= peak probe
// The tensor core's int8 rate with no operand traffic at all: every CTA fills one stage of shared memory once
// (pattern 0: zeros, 1: pseudo-random bytes) and its MMA thread issues `iters` batches of four 128 x 256 x 32 MMAs
// on it.  What a GEMM kernel can reach at most on this GPU at the clock the power cap allows: the roofline's measured
// denominator (the method of the reference's bench/csrc/mma_peak.cu, on tcgen05).
__global__ void __launch_bounds__(128, 1) int8_peak_kernel(int iters, int pattern, int mma_n, unsigned long long* cycles) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = align1024(smem_raw);
    __shared__ uint64_t done;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 4; i += blockDim.x) {
        uint32_t v = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        v ^= v >> 13;
        v *= 0x9E3779B1u;
        ((uint32_t*)smem)[i] = pattern ? (v ^ (v >> 15)) : 0u;
    }
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&done), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_slot), 256);
        tmem_relinquish();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = umma_idesc_i8(128, mma_n);
        const uint64_t ad = umma_desc_k128(smem_u32(smem)), bd = umma_desc_k128(smem_u32(smem + 128 * 128));
        const long long c0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                umma_i8(tmem_base, umma_desc_advance(ad, k * 32), umma_desc_advance(bd, k * 32), idesc, (it | k) ? 1u : 0u);
        }
        tc_commit(smem_u32(&done));
        mbar_wait(smem_u32(&done), 0, &abort_flag, 0x1500);
        if (cycles) cycles[blockIdx.x] = (unsigned long long)(clock64() - c0);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 256);
}

}  // namespace w8a8
