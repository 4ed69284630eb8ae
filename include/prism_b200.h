/* prism_b200 - C ABI of the B200 (sm_100a) quantized linear-layer kernels.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream (as void*, a cudaStream_t), launches on that
 * stream, never synchronizes, never allocates, and returns a status (0 = ok, see PB_* below).  The live row count
 * `n_rows` is a device int32 read by the kernels, so one captured CUDA graph serves any live count; rows at or past it
 * are left untouched.  Each declaration names the interface of the reference (StartLux-Prism) it stands in for.
 */
#ifndef PRISM_B200_H
#define PRISM_B200_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PB_OK 0
#define PB_BAD_ARGUMENT 1      /* null / misaligned pointer, negative size, unknown enum value */
#define PB_UNSUPPORTED_SHAPE 2 /* a size the kernels do not take (see each function) */
#define PB_CUDA_ERROR 3        /* a CUDA call failed: pb_last_cuda_error() has the code */
#define PB_DEVICE_TIMEOUT 4    /* a kernel gave up a bounded wait (read with pb_device_status) */
#define PB_TOO_LARGE 5         /* beyond a stated maximum */

#define PB_EPI_BF16 0 /* out bf16 [M, N] = v */
#define PB_EPI_ADD 1  /* out fp32 [M, N] = add_rn(out, v) */
#define PB_EPI_SWIGLU 2 /* pb_w8a8_gemm_swiglu only */
#define PB_EPI_I32 3  /* out int32 = the raw integer sums */
#define PB_EPI_F32 4  /* out fp32 [M, N] (gk == 32, M <= 64: the vocabulary head's logits, kernels/decode.py:136-160): per
                         group acc = fma(float(acc_g) * a_s, w_s, acc), the reference kernel's compiled arithmetic */

#define PB_W8A8_GEMV_ROWS 1 /* pb_w8a8_gemm, gk == K, split == 1, no pdl: this many rows against a matrix of fewer than
                               9,472 rows run on the CUDA cores (the same bits) */

#define PB_MODE_PLAIN 0
#define PB_MODE_STORE_AMAX 1
#define PB_MODE_USE_AMAX 2

int pb_version(void);
const char* pb_status_string(int status);
int pb_last_cuda_error(void);

/* Reads (and with reset != 0 clears) the current device's status word, which a kernel sets when a bounded wait
 * expires.  Synchronizes the device: for tests and error paths, not for the hot path. */
int pb_device_status(int* code, unsigned* where, int reset);

/* Programmatic dependent launch for the few-row chain.  While on (process-wide), pb_quant_rows with one scale per row,
 * pb_swiglu_q8, pb_fold and pb_w8a8_gemm at 2 <= M <= 64 launch their kernel as a programmatic dependent of the kernel
 * before it on the stream: it may begin (set-up, weight reads) before that kernel has ended, and reads the kernel's
 * output or writes global memory only after it has.  Works inside stream capture (the graph keeps the edges).
 * Callers' own kernels launched between these calls need no change.  Returns the previous setting.
 * The reference has no counterpart: its few-row path is a CUDA graph of plain launches (engine/decoder.py). */
int pb_set_pdl(int on);

/* Every device-side wait (an mbarrier a copy or an MMA completes, a flag or word another GPU writes) is bounded: when
 * the bound runs out the kernel records PB_DEVICE_TIMEOUT with a code for the place, every role of the CTA leaves its
 * loop, copies already requested are given the same bound to land, tensor memory is freed and the kernel returns - no
 * trap, the context stays usable.  The reference's waits are unbounded spins (kernels/quant.py:105-108, :204-206).
 *   pb_set_wait_limit_ns  the bound on the current device (default 4 s; 0 restores it).  Synchronous.
 *   pb_test_drop_loads    failure injection for tests, on the host: while on, the many-rows W8A8 kernel's producers
 *                         request no tiles, so its consumers' waits run out.  Results of such launches are undefined.
 * After a PB_DEVICE_TIMEOUT the split-K counters of the launch that gave up may be left non-zero: zero them (and the
 * status word, pb_device_status) before the workspace is used again. */
int pb_set_wait_limit_ns(unsigned long long ns);
int pb_test_drop_loads(int on);

/* Bytes of workspace and number of int32 counters pb_w8a8_gemm needs for a split-K product whose splits are added
 * inside the kernel (epi 0 / 1 with split > 1).  Stands in for kernels/cuda_ext.py:22-23,139-143 (_workspace). */
long pb_w8a8_workspace_bytes(int M, int N, int split);
int pb_w8a8_counters(int M, int N);

/* W8A8 GEMM.  Replaces torch.ops.startlux_prism.w8a8_gemm / w8a8_gemm_sk / w8a8_wgmma (csrc/w8a8_gemm.cu:794-800,
 * csrc/w8a8_wgmma.cu:709-713) and the Triton kernel behind kernels/w8a8.py:183-231 (gemm) and :234-261 (gemm_i32).
 *   a int8 [M, K], w int8 [N, K] (both K-contiguous, 16-byte aligned, K % 16 == 0);
 *   gk == K: a_s fp32 [M], w_s fp32 [N];  gk == 32: a_s fp32 [M, K/32], w_s fp32 [N, K/32] (K % 128 == 0);
 *   any other gk that is a multiple of 32 and divides K (K % 128 == 0): a_s fp32 [M, K/gk], w_s fp32 [N, K/gk], the
 *   groups' scaled sums added in fp32 in group order (kernels/w8a8.py:64-76); epi 0 / 1, split == 1;
 *   epi PB_EPI_BF16 / PB_EPI_ADD: out [M, N] with row stride ldo elements;
 *   epi PB_EPI_I32: out = slots int32 [split, rows, N] (ldo = N, slot_stride = rows * N elements): split z's sums.
 *   split > 1 with epi 0 / 1 (gk == K, M <= 64): the splits are added inside the kernel through `workspace`
 *   (pb_w8a8_workspace_bytes) and `counters` (pb_w8a8_counters, zero before the first call; left zero).
 *   split == 1 with a workspace and counters given (gk == K, M > 64): when the tiles' last wave would fill less than
 *   60 % of the SMs, that wave's tiles are split along K over the idle SMs (exact, as above; up to 148 x 128 KB of
 *   workspace and 148 counters are used); without a workspace the last wave runs unsplit.
 *   split > 1 with gk == 32 (M <= 64, epi 0 / 1, same workspace): each K slice adds its groups in order, the slices'
 *   fp32 sums are added in slice order: deterministic, within one bf16 step of the unsplit (reference) order.
 *   pdl != 0 (few rows only; ignored otherwise): launch as a programmatic dependent of the kernel before it on the
 *   stream (csrc/w8a8_gemm.cu:273-296): the weights start streaming while that kernel still runs; activations,
 *   scales and every output are touched only after it has completed.  n_rows must not be written by that kernel.
 * The result bits do not depend on split, on the kernel chosen or on M (batch invariance). */
int pb_w8a8_gemm(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, void* out, long ldo,
                 const int* n_rows, int M, int N, int K, int gk, int epi, int split, long slot_stride,
                 void* workspace, long workspace_bytes, int* counters, int n_counters, int pdl, void* stream);

/* The gate|up projection with the SwiGLU and the next projection's activation quantization fused into its epilogue.
 * Replaces the Triton kernel's EPI 2 (kernels/w8a8.py:9-11,86-98): w int8 [N = 2 FF, K] holds, per tile of bn rows,
 * bn / 2 gate rows and then the matching bn / 2 up rows (w8a8.interleave_gate_up, kernels/w8a8.py:289-294), w_s fp32
 * [N] in the same order, one scale group over K (a_s fp32 [M]).  For every row and tile:
 *   act = silu(gate) * up of the scaled fp32 sums; s[m, tile] = max(|act|max, 1e-10) / 127; q = rint(act / s)
 * q int8 [M, FF] (row stride ldq), s fp32 [M, N / bn]: the input of a down projection with gk = bn / 2.  bn 64 or 128. */
int pb_w8a8_gemm_swiglu(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, int8_t* q, long ldq, float* s,
                        const int* n_rows, int M, int N, int K, int bn, void* stream);

/* The int32 partial sums of a row-parallel projection on several GPUs, stored where they will be folded: output rows
 * [o * block_rows, (o + 1) * block_rows) go to blocks[o] (int32 [block_rows, N], row stride ldo), which may be another
 * GPU's memory (pb_peer_open): the tile kernel's epilogue stores over NVLink as each tile is drained, so the exchange
 * of tp.out_proj (tp.py:159-180: gemm_i32, then an int32 all-reduce) overlaps the GEMM and moves half the bytes (each
 * sum travels once, to the rank that folds it).  The receiving rank adds the ranks' blocks with pb_fold (S = ranks),
 * after a barrier over the ranks.  M > 64, block_rows % 128 == 0, n_blocks <= 8, n_blocks * block_rows >= M. */
int pb_w8a8_gemm_scatter(const int8_t* a, const int8_t* w, void* const* blocks, int n_blocks, int block_rows, long ldo,
                         const int* n_rows, int M, int N, int K, void* stream);

/* Device memory other processes can map: pb_peer_alloc allocates (zeroed) and writes a 64-byte handle to pass to the
 * other ranks (any host channel); pb_peer_open maps another rank's handle on the current device with peer access
 * enabled (the role of the reference's symmetric-memory rendezvous, tp.py:381-403); pb_peer_close / pb_peer_free undo. */
int pb_peer_alloc(long bytes, void** ptr, void* handle64);
int pb_peer_open(const void* handle64, void** ptr);
int pb_peer_close(void* ptr);
int pb_peer_free(void* ptr);

/* Deferred residual add.  Replaces quant.fold / _fold_kernel (kernels/quant.py:128-141, :434-457):
 * h[r, c] = add_rn(h[r, c], mul_rn(mul_rn(float(sum_p slots[p, r, c]), a_s[r]), w_s[c])).  N % 4 == 0, 16-byte aligned. */
int pb_fold(float* h, long ldh, const int32_t* slots, long slot_stride, int S, const float* a_s, const float* w_s,
            const int* n_rows, int rows, int N, void* stream);

/* Per-token activation quantization.  Replaces quant.rows_q8 (kernels/quant.py:287-309, :481-486; gk == K, optional
 * SmoothQuant factors inv_s [K], tensor-parallel modes 1 / 2 with amax [rows]) and w8a8.quant_rows
 * (kernels/w8a8.py:101-112, :264-271; gk in {32, 64, 128, 256}).  x bf16 (x_fp32 = 0) or fp32 [T, K] with row
 * stride ldx elements (a column slice of a wider buffer when ldx > K; gk == K only). */
int pb_quant_rows(const void* x, int x_fp32, long ldx, const float* inv_s, int8_t* q, float* s, const int* n_rows,
                  int T, int K, int gk, int mode, float* amax, void* stream);


/* Exchanges between the GPUs of a tensor-parallel group INSIDE a kernel, for passes of a few rows (decode), where a
 * collective call per exchange costs more than the work between them.  Replaces the reference's quant.Sync / mode 3 /
 * _tp_sync / _ll_amax / _fold_parts over symmetric memory (kernels/quant.py:55-141, :190-212; tp.py:358-432); up to 8
 * ranks (the reference: 4).  Buffers are device memory every rank has mapped (pb_peer_alloc / pb_peer_open):
 *   epoch   device int64 [1], the pass number: the same on every rank, incremented once per pass before its kernels
 *   bufs    every rank's 64-bit word buffer as mapped on this GPU, in rank order (bufs[rank] is this rank's own)
 *   off     row maxima: the first word row of this exchange (a step's rows are (off + t) * world + rank);
 *           flag handshakes: the step's channel (its flags are off * world + rank)
 *   others  folds only: the other ranks' int32 slot buffers as mapped here (world - 1 entries), laid out as the own
 * pb_quant_rows_exchange / pb_swiglu_q8_exchange / pb_gated_norm_q8_exchange: the producers' mode 3 - every row's
 * maximum over all ranks travels as one word (pass number above the float's bits) per row and rank; fewer than 256
 * rows per call.  pb_fold_sync / pb_norm_q8_sync: the deferred add over EVERY rank's slots, read over NVLink after a
 * flag handshake (the grid's first block signals, every block waits) - the int32 all-reduce disappears.  pb_fold_sync
 * with no `others` is the handshake alone: the slots the other ranks' kernels stored into THIS rank's memory
 * (pb_w8a8_gemm_scatter) are folded once every rank has signalled that its kernel ended - no barrier collective.
 * Each wait is bounded (pb_set_wait_limit_ns): a rank that never arrives yields PB_DEVICE_TIMEOUT in the status word,
 * not a hang.  Peer traffic is plain loads and stores; no TMA and no multicast touches another GPU's memory. */
typedef struct pb_sync {
    const long long* epoch;
    void* bufs[8];
    const void* others[7];
    long off;
    int rank, world;
} pb_sync;
int pb_quant_rows_exchange(const void* x, int x_fp32, long ldx, const float* inv_s, int8_t* q, float* s, const int* n_rows,
                           int T, int K, const pb_sync* sync, void* stream);
int pb_swiglu_q8_exchange(const void* gu, const float* inv_s, int8_t* q, float* s, const int* n_rows, int T, int FF,
                          const pb_sync* sync, void* stream);
int pb_gated_norm_q8_exchange(const float* o, const void* proj, long P, long z_off, const float* w, const float* inv_s,
                              int8_t* q, float* s, const int* n_rows, int T, int HV, int D, float eps, const pb_sync* sync,
                              void* stream);
int pb_fold_sync(float* h, long ldh, const int32_t* slots, long slot_stride, int S, const float* a_s, const float* w_s,
                 const int* n_rows, int rows, int N, const pb_sync* sync, void* stream);
int pb_norm_q8_sync(float* h, const float* w, int8_t* q, float* s, const int* n_rows, int T, int HID, float eps,
                    const int32_t* parts, long part_stride, int n_parts, const float* psa, const float* psw,
                    const pb_sync* sync, void* stream);

/* The send side of an all-gather between the ranks' peer-mapped buffers, and the handshake that tells the receivers:
 * pb_push stores nbytes (a multiple of 16) from src into each of dsts[0..n) (the same block of the other ranks'
 * buffers as mapped on this GPU: plain stores over NVLink, no TMA, no multicast); pb_handshake then signals this
 * rank's flag of the step on every other rank and waits (bounded: PB_DEVICE_TIMEOUT in the status word) until every
 * other rank has signalled, so that what follows on the stream may read what the others pushed.  The reference
 * gathers with NCCL (tp.py:435-439). */
int pb_push(const void* src, void* const* dsts, int n, long nbytes, void* stream);
int pb_handshake(const pb_sync* sync, void* stream);

/* RMSNorm + per-token quantization, with a deferred residual add finished first.  Replaces quant.norm_q8 /
 * _norm_q8_kernel (kernels/quant.py:145-171, :418-431): for output row i (input row rows[i] when rows != NULL, else i):
 *   h = add_rn(h, mul_rn(mul_rn(float(sum_p parts[p]), psa[r]), psw[c]))  (n_parts > 0; stored back into h)
 *   y = h * rsqrt(sum(h * h) / HID + eps) * w;  s[i] = max(|y|max, 1e-10) / 127;  q[i] = rint(y / s[i]).
 * h fp32 [rows, HID] contiguous, w fp32 [HID] (the norm weight over the SmoothQuant factors), HID % 8 == 0.  The
 * sum of squares is added in this library's fixed order (the reference's Triton reduction has no defined order). */
int pb_norm_q8(float* h, const float* w, int8_t* q, float* s, const int* rows, const int* n_rows, int T, int HID,
               float eps, const int32_t* parts, long part_stride, int n_parts, const float* psa, const float* psw,
               void* stream);

/* Gated RMSNorm of the linear-attention output + per-token quantization.  Replaces quant.gated_norm_q8 /
 * _gated_norm_q8_kernel (kernels/quant.py:215-246, :460-470), modes 0 / 1 / 2 (mode 3, the in-kernel cross-rank
 * exchange: pb_gated_norm_q8_exchange).  o fp32 [T, HV * D]; z = bf16 proj[t * P + z_off + ...]; w fp32 [D];
 * inv_s fp32 [HV * D]; D in {64, 128, 256}.  y = ((o * rsqrt(mean_D(o^2) + eps)) * w) * silu(z) * inv_s per head,
 * s[t] = max(|y|max, 1e-10) / 127, q = rint(y / s[t]). */
int pb_gated_norm_q8(const float* o, const void* proj, long P, long z_off, const float* w, const float* inv_s, int8_t* q,
                     float* s, const int* n_rows, int T, int HV, int D, float eps, int mode, float* amax, void* stream);

/* Final RMSNorm of a residual row, then int8 per 32 inputs: the vocabulary head's activations.  Replaces head_quant /
 * _head_quant_kernel (kernels/decode.py:113-133): y = h * rsqrt(sum(h * h) / HID + eps) * w;
 * s[r, g] = max(|y_g|max, 1e-10) / 127, q = rint(y / s).  h fp32 [B, HID], q int8 [B, HID], s fp32 [B, HID / 32];
 * HID % 32 == 0.  (The head GEMM itself is pb_w8a8_gemm with gk = 32 and PB_EPI_F32.) */
int pb_head_quant(const float* h, const float* w, int8_t* q, float* s, const int* n_rows, int B, int HID, float eps,
                  void* stream);

/* SwiGLU + per-token quantization.  Replaces quant.swiglu_q8 (kernels/quant.py:249-284, :473-478):
 * gu bf16 [T, 2 FF] -> q int8 [T, FF], s fp32 [T].  FF % 8 == 0. */
int pb_swiglu_q8(const void* gu, const float* inv_s, int8_t* q, float* s, const int* n_rows, int T, int FF,
                 int mode, float* amax, void* stream);

/* W4A8 activation quantization (one scale per 256 inputs + split sums of each 32).  Replaces quant.rows_g / _store_g
 * (kernels/quant.py:314-330, :381-411): q int8 [T, K], a fp32 [K/256, Ma], xs int8 [K/256, Ma, 16].  K % 256 == 0. */
int pb_quant_g(const void* x, int x_fp32, int8_t* q, float* a, int8_t* xs, const int* n_rows, int T, int Ma, int K,
               void* stream);

/* The W4A8 twins of the fused producers: the same values, quantized per 256 inputs with the group sums (the
 * reference's swiglu_g, norm_g, gated_norm_g; kernels/quant.py:333-381, :397-411).  Outputs as pb_quant_g.
 * FF, HID, HV * D multiples of 256; D in {64, 128, 256}; HID <= 8192. */
int pb_swiglu_g(const void* gu, int8_t* q, float* a, int8_t* xs, const int* n_rows, int T, int Ma, int FF, void* stream);
int pb_norm_g(const float* h, const float* w, int8_t* q, float* a, int8_t* xs, const int* n_rows, int T, int Ma, int HID,
              float eps, void* stream);
int pb_gated_norm_g(const float* o, const void* proj, long P, long z_off, const float* w, int8_t* q, float* a, int8_t* xs,
                    const int* n_rows, int T, int Ma, int HV, int D, float eps, void* stream);

/* W4A8 GEMM on k-quant weights.  Replaces torch.ops.startlux_prism.w4a8_gemm / w4a8_wgmma (csrc/w4a8_gemm.cu:963-969,
 * csrc/w4a8_wgmma.cu:744-748) behind kernels/w4a8.py:353-366 (gemm).  Operands in the repacked layout of
 * kernels/w4a8.py:44-94: kind 0 (Q4_K): wq uint8 [N, K/2], wsc / wmn uint8 [K/256, N, 8], wd / wdm fp32 [K/256, N];
 * kind 1 (Q6_K): wq int8 [N, K], wsc int8 [K/256, N, 16], wd fp32 [K/256, N] (wmn, wdm, xs unused).  Activations as
 * pb_quant_g writes them: xq int8 [M, K], a fp32 [K/256, Ma], xs int8 [K/256, Ma, 16].  out bf16 (epi 0) or fp32 +=
 * (epi 1), row stride ldo.  K % 256 == 0, N % 4 == 0, 16-byte aligned operands.  Bit-identical to the reference's
 * gemm_ref (kernels/w4a8.py:177-199) for every M (batch invariance).
 * split > 1 (Q4_K, M <= 16 only; ignored otherwise): K is split over CTAs; the slices leave the per-super-block terms
 * of the reference's chain in `workspace` (pb_w4a8_workspace_bytes) and the last CTA of a tile (counters: one int per
 * tile, zero on entry and on return) runs the chain in super-block order - the same bits as split == 1. */
int pb_w4a8_gemm(const int8_t* xq, const float* a, const int8_t* xs, int Ma, int kind, const void* wq,
                 const void* wsc, const void* wmn, const float* wd, const float* wdm, void* out, long ldo,
                 const int* n_rows, int M, int N, int K, int epi, int split, void* workspace, long workspace_bytes,
                 int* counters, int n_counters, void* stream);
long pb_w4a8_workspace_bytes(int M, int N, int K);
int pb_w4a8_counters(int M, int N);

/* MXFP4.  Replace the reference's ctypes ABI (csrc/mxfp4_gemm.cu:121-168: mxfp4_sfa_bytes / mxfp4_sfb_bytes,
 * mxfp4_prepare_sfa / mxfp4_prepare_sfb, mxfp4_gemm) and its Triton kernels (kernels/mxfp4.py:119-185 quantize_act,
 * :260-317 gemm).  Formats (kernels/mxfp4.py:3-5): codes uint8 [rows, K/2] (two e2m1 per byte, low nibble first),
 * scales uint8 [rows, K/32] (UE8M0: 2^(s - 127)).
 *   pb_mxfp4_quant       x bf16 / fp32 [n, K] (times inv [K] when given) -> q, s.  K % 32 == 0.
 *   pb_mxfp4_sf_bytes    bytes of the tensor core's tiled scale layout for a [rows, K] operand (K % 128 == 0)
 *   pb_mxfp4_prepare_sf  s [rows, K/32] -> that layout (weights: once at load; activations: per call, as the reference)
 *   pb_mxfp4_gemm        out [M, N] = deq(A) deq(B)^T, fp32 accumulation: bf16 store (epi 0) or fp32 out += (epi 1);
 *                        a_sf / b_sf are the tiled scales.  K % 256 == 0.  M is a host integer (the reference's n_rows). */
long pb_mxfp4_sf_bytes(int rows, int K);
int pb_mxfp4_prepare_sf(const void* s, void* dst, int rows, int K, void* stream);
int pb_mxfp4_quant(const void* x, int x_fp32, const float* inv, void* q, void* s, int n, int K, void* stream);
int pb_mxfp4_gemm(const void* aq, const void* a_sf, const void* bq, const void* b_sf, void* out, long ldo, int M,
                  int N, int K, int epi, void* stream);

/* The same with K split over `split` CTAs per 128 x 128 tile (few rows, few tiles: the HBM-bound decode shapes): the
 * slices' fp32 accumulators meet in `workspace` and the CTA that finishes a tile last adds them in slice order
 * (deterministic for a given split; within fp32 rounding of the unsplit sum).  counters: zeroed int32, left zeroed. */
/* One to four activation rows on the CUDA cores (exact integer dot products per 32-input block, one fp32 multiply-add
 * per block): a_s / b_s are the plain row-major scale bytes [rows, K/32], not the tiled order.  The result differs from
 * pb_mxfp4_gemm's only in the order of the fp32 additions; no counterpart in the reference (its decode path pads the
 * tensor-core GEMM, kernels/mxfp4.py:292-317).  K % 256 == 0, M <= 4. */
int pb_mxfp4_gemv(const void* aq, const void* a_s, const void* bq, const void* b_s, void* out, long ldo, int M, int N,
                  int K, int epi, void* stream);

long pb_mxfp4_workspace_bytes(int M, int N, int split);
int pb_mxfp4_counters(int M, int N);
int pb_mxfp4_gemm_split(const void* aq, const void* a_sf, const void* bq, const void* b_sf, void* out, long ldo, int M,
                        int N, int K, int epi, int split, void* workspace, long workspace_bytes, int* counters,
                        int n_counters, void* stream);

/* Weight prefetch into L2: the bytes of up to eight ranges (16-byte aligned starts) are requested from the copy
 * engine in 4 KB bulk prefetches by ctas x 128 threads, on `stream` (a side stream: the point is to overlap a
 * latency-bound kernel).  Replaces torch.ops.startlux_prism.l2_prefetch (csrc/l2_prefetch.cu:12-49, kernels/cuda_ext.py:171-173),
 * which the reference measured as a loss on its GPUs and keeps off by default; off by default here too. */
int pb_l2_prefetch(const void* const* ptrs, const long* nbytes, int n, int ctas, void* stream);

/* Measurement aid: the int8 tensor-core rate with shared-memory-resident operands and no loads (one CTA per SM, `iters`
 * batches of four 128 x mma_n x 32 MMAs each, mma_n a multiple of 16 up to 256; pattern 0 = zero operands, 1 =
 * pseudo-random bytes).  ops = 2 * 128 * mma_n * 128 * iters per SM.  Counterpart of the reference's bench/csrc/mma_peak.cu.  cycles (device, one per SM) may be NULL. */
int pb_int8_peak_probe(int iters, int pattern, int mma_n, unsigned long long* cycles, void* stream);

/* The same for the FP4 tensor-core rate: `iters` batches of four 128 x 256 x 64 tcgen05 kind::mxf4.block_scale MMAs
 * per SM on shared-memory-resident operands with unit scales.  ops = 2 * 128 * 256 * 256 * iters per SM. */
int pb_mxf4_peak_probe(int iters, int pattern, unsigned long long* cycles, void* stream);

/* pb_w8a8_gemm for callers that cannot allocate device memory.  No counterpart in the reference (its stream-K
 * workspace is always a torch allocation, kernels/cuda_ext.py:139-143).
 * Some hosts of this library have no allocator to offer: a plugin loaded into a process whose memory pool is owned by
 * another runtime, a replay thread that may only launch, a code path that runs while a stream is being captured (where
 * cudaMalloc is illegal).  For them the few-rows split-K GEMM (M <= 64, gk == K, epi 0 / 1) keeps its scratch - the
 * int32 partial sums of the K splits and the per-tile arrival counters - in a fixed array inside the library's device
 * image: pb_w8a8_static_scratch_bytes() = 16 MiB of partial sums plus 4,096 counters, resident on every GPU that loads
 * the library until the process exits.  Same arguments and result bits as pb_w8a8_gemm; a product whose scratch
 * (pb_w8a8_workspace_bytes / pb_w8a8_counters) exceeds the array returns PB_TOO_LARGE and launches nothing.
 * The call makes no cudaMalloc / cudaFree and calls no allocating library routine.  The first call on each device
 * looks up the array's device address (cudaGetSymbolAddress, with that device current) and should therefore come
 * before any stream capture on that device.  All calls on a device share the one array: the counters are cleared on
 * the stream before each launch, but two calls that overlap on the GPU (different streams) race on it - serialize
 * them. */
long pb_w8a8_static_scratch_bytes(void);
int pb_w8a8_gemm_static(const int8_t* a, const float* a_s, const int8_t* w, const float* w_s, void* out, long ldo,
                        const int* n_rows, int M, int N, int K, int epi, int split, void* stream);

#ifdef __cplusplus
}
#endif
#endif
