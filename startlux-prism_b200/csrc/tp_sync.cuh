// Cross-GPU exchanges inside a kernel, for the shortest tensor-parallel passes (a few rows: decode): what the
// reference does with its mode-3 producers and _tp_sync (kernels/quant.py:55-125, :190-212), on plain peer memory
// (CUDA IPC mappings: loads and stores over NVLink from registers; no TMA, no multicast, no library call).
//
//   exchange_amax  a row's maximum over every rank inside the producer's one launch.  This rank's maximum and the pass
//                  number travel as ONE 64-bit word (number above the float's bits: written and read whole, so the data
//                  is its own flag) into word (off + t) * world + rank of every other rank's buffer; then every other
//                  rank's word for the row is read from this rank's buffer until it carries this pass's number.
//   arrive_and_wait  a flag handshake before a consumer reads what the other ranks' earlier kernels wrote: the grid's
//                  first block stores the pass number into this rank's flag of the step on every other rank (a release
//                  store, system scope); every block waits until every other rank's flag has reached it (relaxed loads,
//                  then one acquire fence).  The first block signals before it waits, so nobody waits for a signal that
//                  cannot come.
// Every wait is bounded by the device's wait limit (g_pb_wait_ns): on expiry the kernel records PB_DEVICE_TIMEOUT and
// goes on with what it has (the result is then wrong, the status word says so, the context survives).  The reference's
// waits spin without a bound.
// Up to 8 ranks (the reference's argument lists stop at 4).
#pragma once
#include "common.cuh"

namespace tpx {

constexpr int MAX_RANKS = 8;

struct Sync {
    const long long* epoch;                  // device int64 [1]: the pass number, the same on every rank
    unsigned long long* bufs[MAX_RANKS];     // every rank's word / flag buffer as mapped on this GPU, in rank order
    const int32_t* others[MAX_RANKS - 1];    // fold: the other ranks' int32 slots as mapped here (world - 1 entries)
    long off;                                // words: first row of this exchange; flags: this step's channel
    int rank, world;                         // world <= 1: no exchange
};

__device__ __forceinline__ unsigned long long ld_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Spins (bounded) until the word at p satisfies the test: tagged (its high half equals e) or reached (its value is at
// least e).  Returns the word; *ok = false when the bound ran out.
template <bool TAGGED>
__device__ __forceinline__ unsigned long long wait_word(const unsigned long long* p, unsigned long long e, bool* ok,
                                                        unsigned where) {
    unsigned long long v = ld_sys(p);
    auto good = [&](unsigned long long w) { return TAGGED ? (w >> 32) == e : w >= e; };
    if (good(v)) return v;
    const unsigned long long t0 = global_timer_ns();
    const unsigned long long limit = *(volatile unsigned long long*)&g_pb_wait_ns;
    for (unsigned it = 1;; ++it) {
        v = ld_sys(p);
        if (good(v)) return v;
        if ((it & 0x3f) == 0 && global_timer_ns() - t0 > limit) {
            pb_report(PB_DEVICE_TIMEOUT, where);
            *ok = false;
            return v;
        }
    }
}

// Called by every thread of the block with the block's maximum of row t; returns the maximum over all ranks.
__device__ __forceinline__ float exchange_amax(float amax, long t, const Sync& s) {
    __shared__ float xch;
    if (s.world <= 1) return amax;
    if (threadIdx.x == 0) {
        const unsigned long long e = (unsigned long long)(*s.epoch) & 0xffffffffull;
        const unsigned long long word = (e << 32) | (unsigned long long)__float_as_uint(amax);
        const long slot = (s.off + t) * s.world;
        for (int q = 0; q < s.world; ++q)
            if (q != s.rank) st_sys(s.bufs[q] + slot + s.rank, word);
        bool ok = true;
        for (int q = 0; q < s.world && ok; ++q) {
            if (q == s.rank) continue;
            const unsigned long long v = wait_word<true>(s.bufs[s.rank] + slot + q, e, &ok, 0x2000 + q);
            if (ok) amax = fmaxf(amax, __uint_as_float((unsigned)(v & 0xffffffffull)));
        }
        xch = amax;
    }
    __syncthreads();
    return xch;
}

// Called by every thread of every block before the first read of another rank's data.
__device__ __forceinline__ void arrive_and_wait(const Sync& s, bool first_block) {
    if (s.world <= 1 || !s.bufs[s.rank]) return;              // no flags: the handshake was a kernel of its own
    if (threadIdx.x == 0) {
        const unsigned long long e = (unsigned long long)(*s.epoch);
        const long chan = s.off * s.world;
        if (first_block)
            for (int q = 0; q < s.world; ++q)
                if (q != s.rank) st_release_sys(s.bufs[q] + chan + s.rank, e);
        bool ok = true;
        for (int q = 0; q < s.world && ok; ++q)
            if (q != s.rank) wait_word<false>(s.bufs[s.rank] + chan + q, e, &ok, 0x2100 + q);
        fence_sys();
    }
    __syncthreads();
}

// The handshake as a kernel of its own (one block): for consumers with thousands of blocks, where a system-scope wait
// and fence in every block costs more than one extra launch.  Kernels after it on the stream start after it has ended.
__global__ void __launch_bounds__(32) handshake_kernel(const Sync s) { arrive_and_wait(s, true); }

// One block of this rank's memory stored into the same place of up to seven other ranks' buffers (an all-gather's
// send side: plain 16-byte loads here, 16-byte stores over NVLink there; the receivers learn of it by a handshake).
struct PushArgs {
    const uint4* src;
    uint4* dst[MAX_RANKS - 1];
    long n16;                                // 16-byte units
    int n;                                   // destinations
};
__global__ void __launch_bounds__(256) push_kernel(const PushArgs a) {
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n16; i += stride) {
        const uint4 v = a.src[i];
        for (int d = 0; d < a.n; ++d) a.dst[d][i] = v;
    }
}

// Four consecutive int32 sums of another rank's slots, read past this GPU's caches (the data changes between passes).
__device__ __forceinline__ int4 ld_peer4(const int32_t* p) {
    int4 v;
    asm volatile("ld.volatile.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

}  // namespace tpx
