/*
 * C ABI of libavefp4: block-scaled FP4 (NVFP4 / MXFP4) GEMM  D = A * B^T  and the
 * bf16 -> FP4 activation quantise for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host binding talks to.  Plain pointers and sizes only; all
 * pointers are device pointers unless stated otherwise; every call enqueues work on
 * `stream` (a cudaStream_t passed as void*) of the current device and returns
 * without synchronising, so calls are safe inside CUDA graph capture.  No entry
 * point below allocates or frees device memory except ave_fp4_init.
 *
 * Return value: 0 on success; negative = argument error; positive = cudaError_t.
 * ave_fp4_last_error() gives the message of the calling thread's last failure.
 *
 * Reference interfaces these entry points stand in for (paths inside
 * causalflow-ai/avelang):
 *   - the operator  gemm_pipeline_transposed_b(A, B, out=None)
 *     python/avelang_kernels/amdgpu_gemm.py:458-494  (A (M,K), B (N,K), K contiguous,
 *     D = A * B^T, fp32 accumulate, bf16 out);
 *   - the launch convention of the NVIDIA backend: raw data_ptr() pointers, current
 *     device, current raw stream, errors raised as RuntimeError
 *     python/avelang/backends/nvidia/driver.py:68-81,120-131,284-311 and
 *     python/avelang/backends/driver.py:24-32.
 *
 * Storage convention of a quantised (R,K) operand:
 *   packed : uint8 (R, K/2) row-major; byte j = element 2j in bits 3:0, 2j+1 in bits 7:4;
 *            a nibble is E2M1 (sign, 2 exponent bits, 1 mantissa bit).
 *   scales : uint8; one per 16 (NVFP4, E4M3) or 32 (MXFP4, E8M0) consecutive K elements.
 *            AVE_FP4_SF_ROW_MAJOR : (R, K/blk) row-major.
 *            AVE_FP4_SF_TILED     : 128x4 tiles of 512 bytes, tile (rb, cb) at
 *                                   (rb * ceil(K/blk/4) + cb) * 512, scale (r, c) inside a tile at
 *                                   (r % 32) * 16 + (r / 32) * 4 + c; rows padded to 128 and scale
 *                                   columns to 4 with zero bytes.  The GEMM consumes this layout.
 *   global : one fp32 in device memory (NVFP4 only): value = nibble * scale * global.
 */
#ifndef AVE_FP4_H_
#define AVE_FP4_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AVE_FP4_FMT_NVFP4 0
#define AVE_FP4_FMT_MXFP4 1

#define AVE_FP4_SF_ROW_MAJOR 0
#define AVE_FP4_SF_TILED 1

/* Kernel variants for ave_fp4_gemm (0 lets the library choose by shape). */
#define AVE_FP4_GEMM_AUTO 0
#define AVE_FP4_GEMM_1CTA_N128 1 /* 128x128 tile, two accumulator buffers */
#define AVE_FP4_GEMM_1CTA_N256 2 /* 128x256 tile */
#define AVE_FP4_GEMM_2CTA_N256 3 /* CTA pair, 256x256 tile */
#define AVE_FP4_GEMM_2CTA_N128 4 /* CTA pair, 256x128 tile, two accumulator buffers */
#define AVE_FP4_GEMM_2CTA_N192 5 /* CTA pair, 256x192 tile, two accumulator buffers */
#define AVE_FP4_GEMM_SKINNY 10   /* M <= 64 (chosen by default up to M = 32): operands swapped, stream-K over all SMs */
#define AVE_FP4_GEMM_SKINNY_TILED_W 11 /* as 10, with b_packed in the tile-major layout of ave_fp4_pack_weight_tiles */

/*
 * Flag, OR-ed into `variant`: the weight operand (b_packed, b_scales) is not written by any work queued
 * earlier on `stream`.  The decode kernel is then launched with programmatic stream serialisation: it
 * starts streaming weights while the previous kernel in the stream is still finishing and waits for it
 * only before touching activations, scales, scratch or output.  Ignored by the tiled kernels.
 */
#define AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS 0x100

/* Error codes returned as negative values. */
#define AVE_FP4_ERR_ARG 1
#define AVE_FP4_ERR_NOT_INIT 2
#define AVE_FP4_ERR_WORKSPACE 3
#define AVE_FP4_ERR_DEVICE 4

/*
 * One-time set-up for `device` (idempotent, thread-safe): checks that the device is
 * sm_100, resolves the driver's tensor-map encoder, opts the kernels into large
 * dynamic shared memory and allocates the 4-byte device status word.
 * Replaces the load_binary / launcher-build step of the reference
 * (python/avelang/backends/nvidia/driver.c:51-113, driver.py:182-336).
 */
int ave_fp4_init(int device);

/* Message for the last non-zero return value on this thread (never NULL). */
const char* ave_fp4_last_error(void);

/* Bytes of the scale array of a (rows, k) operand in the given format and layout. */
int64_t ave_fp4_sf_bytes(int64_t rows, int64_t k, int fmt, int sf_layout);

/*
 * Bytes of zero-initialised scratch ave_fp4_gemm needs for this shape on `device`
 * (0 for shapes served by the tiled kernels).  The scratch must be all zero before
 * its first use; the kernel leaves it reusable for the next call on the same stream,
 * also for a call of a different shape (what has to be zero between calls sits in a
 * prefix whose size does not depend on the shape, for N up to 524288).
 */
int64_t ave_fp4_workspace_bytes(int64_t m, int64_t n, int64_t k, int fmt, int variant, int device);

/*
 * max |x| of a (rows, k) bf16 matrix with row stride ldx (elements) -> *amax_f32
 * (device fp32; the call zeroes it first).  k % 8 == 0, rows 16-byte aligned.
 */
int ave_fp4_amax(const void* x_bf16, int64_t rows, int64_t k, int64_t ldx, void* amax_f32, void* stream);

/*
 * Quantise a (rows, k) bf16 matrix (row stride ldx elements, k % 32 == 0).
 *   NVFP4: if amax_f32 != NULL the tensor scale is amax / 2688 (1 if amax == 0) and is
 *          written to *global_scale; if amax_f32 == NULL the value already in
 *          *global_scale is used (static scale).
 *   MXFP4: amax_f32 and global_scale are ignored (may be NULL).
 * No counterpart in the reference (it has no quantise operator); semantics are those
 * of the CPU oracle.
 */
int ave_fp4_quantize(const void* x_bf16, int64_t rows, int64_t k, int64_t ldx, int fmt, const void* amax_f32,
                     void* global_scale, void* packed, void* scales, int sf_layout, void* stream);

/*
 * NVFP4 quantise with the tensor scale taken from the data (amax / 2688), in one call: for inputs of up
 * to 2^20 elements (decode activations) one 8-CTA cluster launch does amax and quantise together (up to 8192
 * blocks of 16 elements, e.g. 16 x 8192, with one block per thread kept in registers across the exchange of the
 * maxima -- the shortest dependent chain, which is what the decode GEMM queued behind it waits for); above
 * that it is ave_fp4_amax + ave_fp4_quantize and needs `amax_scratch` (4 bytes of device memory).
 * Results are identical to the two-call form.
 */
int ave_fp4_quantize_nvfp4_dynamic(const void* x_bf16, int64_t rows, int64_t k, int64_t ldx, void* global_scale,
                                   void* packed, void* scales, int sf_layout, void* amax_scratch, void* stream);

/* Row-major (rows, cols) scale bytes -> tiled layout (for weights quantised elsewhere). */
int ave_fp4_sf_to_tiled(const void* sf_row_major, int64_t rows, int64_t cols, void* sf_tiled, void* stream);

/*
 * Offline weight packing for the decode path: packed E2M1 weights (n, k/2) row-major ->
 * tile-major, 16 KB tiles of 128 rows x 128 bytes ordered [row block][K block], zero padded,
 * ave_fp4_weight_tiles_bytes(n, k) bytes in total.  With this layout the skinny kernel reads
 * each weight row block as one contiguous HBM stream.  No counterpart in the reference.
 */
int64_t ave_fp4_weight_tiles_bytes(int64_t n, int64_t k);
int ave_fp4_pack_weight_tiles(const void* packed_row_major, int64_t n, int64_t k, void* packed_tiles, void* stream);

/*
 * D (m, n) bf16, row stride ldd elements  =  A (m, k) * B (n, k)^T, fp32 accumulation,
 * result scaled by (*a_global_scale) * (*b_global_scale) (NULL = 1) and rounded to
 * bf16 (nearest even).  Scales in AVE_FP4_SF_TILED layout.
 * Requirements: k % 32 == 0, n % 8 == 0, ldd % 8 == 0 (anything else is rejected with a negative return
 * code before a launch: the write-out moves 8-column chunks), all pointers 16-byte aligned.
 * Stands in for the kernel launch of gemm_pipeline_transposed_b
 * (python/avelang_kernels/amdgpu_gemm.py:488-494).
 */
int ave_fp4_gemm(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                 const void* b_scales, const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k,
                 int64_t ldd, int fmt, int variant, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Fused epilogue of ave_fp4_gemm_epilogue: D = act(gsA * gsB * (A * B^T) + bias), evaluated in fp32 and
 * rounded to bf16 once.  The reference operator has no epilogue (its write-out is
 * python/avelang_kernels/amdgpu_gemm.py:293-329); this is the linear layer a caller builds around it.
 */
#define AVE_FP4_ACT_NONE 0
#define AVE_FP4_ACT_RELU 1      /* max(x, 0) */
#define AVE_FP4_ACT_GELU 2      /* 0.5 x (1 + erf(x / sqrt 2)) */
#define AVE_FP4_ACT_GELU_TANH 3 /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) */
#define AVE_FP4_ACT_SILU 4      /* x / (1 + exp(-x)) */

typedef struct ave_fp4_epilogue {
    const void* bias_bf16; /* device, n bf16 values, one per output column, 16-byte aligned; NULL = no bias */
    int32_t activation;    /* AVE_FP4_ACT_* */
    /*
     * quantize_out != 0: the bf16-rounded result is also emitted as an FP4 operand of the GEMM's own format
     * (`fmt`), scale blocks along N, i.e. ready to be the A operand of the next layer's GEMM -- bit-identical
     * to running ave_fp4_quantize on the bf16 result (static tensor scale for NVFP4).  d_bf16 may then be NULL,
     * in which case only the quantised result is written.  Needs n % 16 == 0 (NVFP4) or n % 32 == 0 (MXFP4) and
     * a tiled kernel (AVE_FP4_GEMM_AUTO picks one for any M).
     */
    int32_t quantize_out;
    void* q_packed;              /* (m, n/2) bytes, row-major, 16-byte aligned */
    void* q_scales;              /* ave_fp4_sf_bytes(m, n, fmt, q_sf_layout) bytes */
    const void* q_global_scale;  /* NVFP4: device fp32 tensor scale of the result (read, not written); MXFP4: unused */
    int32_t q_sf_layout;         /* AVE_FP4_SF_ROW_MAJOR or AVE_FP4_SF_TILED */
    int32_t reserved;            /* must be 0 */
} ave_fp4_epilogue;

/* ave_fp4_gemm with the fused epilogue above (bias and activation: all kernel variants; quantised result: the tiled
 * kernels; epilogue == NULL is ave_fp4_gemm). */
int ave_fp4_gemm_epilogue(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                          const void* b_scales, const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k,
                          int64_t ldd, int fmt, int variant, void* workspace, int64_t workspace_bytes, void* stream,
                          const ave_fp4_epilogue* epilogue);

/*
 * Decode-shaped linear layer on unquantised activations (M <= 32), in one call that allocates nothing:
 *   D (m, n) bf16 = act(quantise(X) * B^T + bias),  X (m, k) bf16 with row stride ldx elements.
 * X is quantised to the GEMM's format into the caller's scratch exactly as ave_fp4_quantize /
 * ave_fp4_quantize_nvfp4_dynamic would (NVFP4: tensor scale amax / 2688 taken from X; up to 8192 blocks of 16
 * elements, e.g. 16 x 8192, by one 8-CTA cluster launch with one block per thread, amax and quantise together), and the
 * decode GEMM is chained behind it with programmatic dependent launch, so its CTAs start and stream weights while
 * the quantise still runs.  D is bit-identical to ave_fp4_quantize* followed by ave_fp4_gemm (decode variant).
 * (Quantising inside the GEMM kernel itself was built and measured and is not shipped: every CTA needs all of X,
 * and the exact-division quantise costs about ten instructions per element, so doing it redundantly per CTA, or
 * exchanging the bytes between CTAs through memory with its ~3 us loaded latency, was slower than this chain.)
 * `workspace`: ave_fp4_linear_decode_workspace_bytes(...) bytes, 256-byte aligned, all zero before its first use;
 * the call leaves it reusable for the next call on the same stream (calls that may overlap on the GPU need
 * separate workspaces).  After the call it holds the quantised activations (layout private).
 * `flags`: AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS (as for ave_fp4_gemm) and/or AVE_FP4_LINEAR_FLAG_TILE_MAJOR_WEIGHTS
 * (b_packed in the layout of ave_fp4_pack_weight_tiles).  `epilogue`: NULL, or bias and activation (no quantize_out).
 * Stands in for the prologue + launch of gemm_pipeline_transposed_b (python/avelang_kernels/amdgpu_gemm.py:392-401,
 * 488-494) when the activations arrive unquantised; the reference has no quantise step of its own.
 */
#define AVE_FP4_LINEAR_FLAG_TILE_MAJOR_WEIGHTS 0x200
int64_t ave_fp4_linear_decode_workspace_bytes(int64_t m, int64_t n, int64_t k, int fmt, int device);
int ave_fp4_linear_decode(const void* x_bf16, int64_t ldx, const void* b_packed, const void* b_scales,
                          const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k, int64_t ldd, int fmt,
                          int flags, void* workspace, int64_t workspace_bytes, void* stream,
                          const ave_fp4_epilogue* epilogue);

/*
 * The reference operator itself on sm_100a: D (m, n) bf16 = A (m, k) bf16 * B (n, k)^T bf16, fp32 accumulation in
 * tensor memory (tcgen05.mma kind::f16), bf16 output rounded to nearest even (the reference's MI300 kernel
 * truncates, python/avelang_kernels/amdgpu_gemm.py:322-328).  K % 8 == 0, ldd % 8 == 0, 16-byte aligned pointers;
 * M and N need not be tile multiples (the reference requires M, N % 128 and K % 64, amdgpu_gemm.py:471-476).
 * Stands in for the launch in gemm_pipeline_transposed_b, python/avelang_kernels/amdgpu_gemm.py:488-494.
 * variant: AVE_FP4_GEMM_AUTO / AVE_FP4_GEMM_2CTA_N256 (256x256 tiles, CTA pairs) or AVE_FP4_GEMM_1CTA_N128.
 */
int ave_bf16_gemm(const void* a_bf16, const void* b_bf16, void* d_bf16, int64_t m, int64_t n, int64_t k, int64_t ldd,
                  int variant, void* stream);

/*
 * GEMM fused with the all-gather of its output (N-sharded weights on one NVLink/NVSwitch box).
 * As ave_fp4_gemm (tiled kernels, M > 64), and in addition every output tile is stored to
 * peer_d[0 .. n_peers-1]: device pointers, valid on THIS GPU, to the same (m, n) block inside each
 * other GPU's result buffer (peer-mapped memory, e.g. CUDA IPC / symmetric memory; same ldd).
 * The stores are plain peer stores issued by the epilogue, so the exchange overlaps the remaining
 * tiles' math.  The caller synchronises the ranks afterwards (all kernels done) before any rank
 * reads its gathered buffer.  `peer_d` is a host array read during the call.  No counterpart in
 * the reference, which has no multi-GPU code.
 */
int ave_fp4_gemm_allgather(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                           const void* b_scales, const void* b_global_scale, void* d_bf16, void* const* peer_d, int n_peers,
                           int64_t m, int64_t n, int64_t k, int64_t ldd, int fmt, int variant, void* stream);

/*
 * GEMM fused with the all-gather of its QUANTISED output: for an N-sharded layer whose consumer is another FP4
 * GEMM, the ranks gather the next layer's operand (0.5 byte per element + one scale byte per block) instead of
 * the bf16 matrix (2 bytes per element), about 3.5 times fewer bytes over NVLink.  As ave_fp4_gemm_epilogue with
 * quantize_out (bias and activation allowed, tiled kernels, M > 64, d_bf16 not written): this rank's (m, n) result
 * is quantised in the epilogue, blocks along N, as columns [col0, col0 + n) of a gathered (m, n_total) operand.
 * epilogue->q_packed / q_scales point at the BASE of this rank's copy of that operand ((m, n_total / 2) bytes and
 * ave_fp4_sf_bytes(m, n_total, fmt, q_sf_layout) scale bytes); peer_q_packed[i] / peer_q_scales[i] are device
 * pointers, valid on THIS GPU, to the bases of the other ranks' copies (peer-mapped memory), to which the
 * epilogue stores the same bytes at the same offsets with plain peer stores (no TMA, no multicast).  NVFP4 needs
 * a static tensor scale of the result (epilogue->q_global_scale), the same on every rank.  n, col0 and n_total must
 * be multiples of 64.  The caller synchronises the ranks afterwards (all kernels done) before any rank reads its
 * copy; padding rows of a tiled scale layout are written by every rank for its own columns.  The bytes are those of
 * ave_fp4_quantize applied to the bf16-rounded unsharded result.  No counterpart in the reference.
 */
int ave_fp4_gemm_allgather_quantized(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                                     const void* b_scales, const void* b_global_scale, int64_t m, int64_t n, int64_t k, int fmt,
                                     int variant, const ave_fp4_epilogue* epilogue, int64_t n_total, int64_t col0,
                                     void* const* peer_q_packed, void* const* peer_q_scales, int n_peers, void* stream);

/*
 * K-sharded GEMM + reduce-scatter in two calls (row-parallel linear layer on one NVLink/NVSwitch box).  No counterpart
 * in the reference, which has no multi-GPU code.
 *
 * ave_fp4_gemm_partials: this rank holds the K-slices A (m, k) and B (n, k) of the full operands; the fp32 product
 * (tensor scales applied, no rounding) is scattered by the epilogue's own stores: rows [j*m/world, (j+1)*m/world)
 * go, row stride n, to slab_dst[j] -- a device pointer valid on THIS GPU to the (m/world, n) fp32 slab this rank owns
 * inside rank j's staging buffer (peer-mapped memory for j != this rank, plain stores over NVLink; `slab_dst` is a host
 * array read during the call).  m % (32 * world) == 0; 256x256 CTA-pair tiles.  The tile schedule visits the owners' rows
 * in turn, starting with owner `first_owner`: give every rank a different one (e.g. rank + 1 mod world), so that at any
 * moment the ranks store to different destination GPUs and no NVLink ingress is the target of all of them.
 *
 * ave_fp4_reduce_partials: after every rank's partials have landed (the caller synchronises the ranks), the owner sums
 * its `world` slabs (fp32 (rows, n), back to back, in slab order -- deterministic), applies the optional bias and
 * activation, and rounds to bf16 once.
 */
int ave_fp4_gemm_partials(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                          const void* b_scales, const void* b_global_scale, void* const* slab_dst, int world, int first_owner,
                          int64_t m, int64_t n, int64_t k, int fmt, void* stream);
int ave_fp4_reduce_partials(const void* slabs_f32, int world, int64_t rows, int64_t n, void* d_bf16, int64_t ldd,
                            const ave_fp4_epilogue* epilogue, void* stream);

/*
 * Decode GEMM (M <= 16, N <= 65536) that allocates nothing and needs no caller workspace.
 * It has no counterpart in the reference.  It exists for hosts that cannot call cudaMalloc:
 * a plugin living inside another runtime's memory pool, or a serving loop that must not risk
 * the device-wide stall an allocation can cause.  The stream-K scratch of the skinny kernel is
 * a fixed array inside the library instead (about 2.56 MiB, held by every GPU that loads the
 * library until the process exits).  Same arguments and result as ave_fp4_gemm with the skinny
 * variant; shapes beyond the limits are rejected with an error, not served some other way.
 * The first call on a device looks the array's device address up, so make that first call
 * outside any stream capture.  All calls on one device share the array: calls that may overlap
 * on the GPU (different streams) race on it and must be serialised by the caller.
 */
int ave_fp4_gemm_decode_noalloc(const void* a_packed, const void* a_scales, const void* a_global_scale,
                                const void* b_packed, const void* b_scales, const void* b_global_scale, void* d_bf16,
                                int64_t m, int64_t n, int64_t k, int64_t ldd, int fmt, void* stream);

/*
 * Synchronises `stream`, reads and clears the device status word of the current
 * device.  Returns 0 if every kernel since the last check ran to completion, or the
 * positive status code a kernel recorded when one of its bounded waits expired
 * (101 producer, 102 MMA issuer, 103 epilogue, 104 self-test).  Not capturable.
 */
int ave_fp4_check(void* stream);

/*
 * Failure-path self-test: launches a one-warp kernel whose only barrier wait can never complete; the
 * bounded wait expires after `timeout_us` (1 us .. 100 ms), the kernel records status 104 and returns
 * normally.  The next ave_fp4_check then reports 104.  Nothing faults, traps or hangs.
 */
int ave_fp4_selftest_wait_timeout(int64_t timeout_us, void* stream);

/*
 * Profiling aid (no counterpart in the reference, whose only tracing is event timing in
 * benchmark/gemm/bench_amdgpu_gemm.py:43-52).  While a device buffer is set, the GEMM
 * kernels make CTA 0 record clock64() stamps: with cap = bytes / 96, record r of role q
 * (0 = TMA producer, 1 = MMA issuer, per K block or load burst; 2 = first epilogue warp, per tile or segment) is four
 * int64 at buffer[(q * cap + r) * 4]: {before wait, after wait, after issue / drain, aux}.
 * Pass NULL to switch it off (the default).
 */
int ave_fp4_set_trace(void* buffer, int64_t bytes);

/* Number of SMs the library sees on the current device (after ave_fp4_init). */
int ave_fp4_sm_count(void);

#ifdef __cplusplus
}
#endif

#endif /* AVE_FP4_H_ */
