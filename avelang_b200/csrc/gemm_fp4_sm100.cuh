// Block-scaled FP4 GEMM  D[M,N] (bf16) = alpha * A[M,K] * B[N,K]^T  for sm_100a.
//
// Counterpart of the reference operator kernel
// python/avelang_kernels/amdgpu_gemm.py:349-455 (one 128x128 tile per workgroup,
// LDS-staged MFMA loop, bf16 truncating store) re-designed for Blackwell:
//
//   * persistent CTAs (optionally 2-CTA pairs), static tile schedule with grouped raster;
//   * warp 0: TMA producer -- packed E2M1 tiles (128-byte swizzle, 256 K-elements per
//     row chunk) and 128x4 scale-factor tiles into a STAGES-deep shared-memory ring;
//   * warp 1: one thread issues tcgen05.cp (scale factors smem -> TMEM) and
//     tcgen05.mma kind::mxf4nvf4 / kind::mxf4 block-scaled, fp32 accumulators in TMEM;
//   * warps 2-9: epilogue -- each warp drains 32 TMEM lanes x BLOCK_N/2 columns into
//     registers (tcgen05.ld, * alpha, round-to-nearest-even bf16) and hands the
//     accumulator back at once, so the next tile's MMAs start while the bf16 rows
//     are still being written out through a swizzled shared-memory transpose as
//     full 128-byte lines (predicated at the matrix edges).
//
// Operand convention (python/avelang_kernels/amdgpu_gemm.py:458-494): A is (M,K),
// B is (N,K), both K-contiguous; D = A * B^T.
#pragma once

#include <cuda_bf16.h>

#include "quantize_fp4.cuh"
#include "sm100_ptx.cuh"

namespace avefp4 {

// 256-bit store (one whole 32-byte sector per lane), streaming.
__device__ __forceinline__ void st_global_v8_cs(void* ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}

enum GemmStatus : int {
    kStatusOk = 0,
    kStatusTimeoutProducer = 101,
    kStatusTimeoutMma = 102,
    kStatusTimeoutEpilogue = 103,
    kStatusTimeoutSelfTest = 104,
};

// Exercises the failure path every kernel here relies on, without any fault: one warp waits on a
// barrier that nobody will ever arrive on, the bounded wait gives up after `timeout_ns`, the kernel
// records a status code and returns normally.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long timeout_ns) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
    }
    __syncwarp();
    if (!mbar_wait(b, 0, timeout_ns)) {
        if (threadIdx.x == 0) atomicCAS(status, 0, kStatusTimeoutSelfTest);
    }
}

struct GemmParams {
    int m, n, k;
    int tiles_m, tiles_n;      // in units of (128 * CTA_GROUP) x BLOCK_N
    int sf_k_atoms;            // 128x4 scale tiles along K: ceil(K / SF_VEC / 4)
    const float* a_gs;         // device fp32 scalars (NVFP4 tensor scales) or nullptr
    const float* b_gs;
    __nv_bfloat16* d;          // output, row stride ldd elements
    int ldd;
    int n_peers;               // fused all-gather: the same tile is also stored to these buffers,
    __nv_bfloat16* peer_d[7];  // which live in other GPUs' memory (peer-mapped), same layout as d
    int* status;               // device status word, written on a wait timeout
    long long* trace;          // optional clock64() stamps of CTA 0 (profiling aid), or nullptr
    int trace_cap;             // records per role; record r of role q at trace[(q * trace_cap + r) * 4 ..+3]
    const __nv_bfloat16* bias; // fused epilogue: n values added to every output row after the tensor scales, or nullptr
    int act;                   // fused epilogue: kActNone / kActRelu / kActGelu / kActGeluTanh / kActSilu
    // quantising epilogue (kEpiQuant): the bf16-rounded result is also emitted as an FP4 operand of the
    // kernel's own format, blocks along N, ready to be the A operand of the next GEMM
    uint8_t* q_packed;         // (m, n/2) bytes, row-major
    uint8_t* q_sf;             // scale bytes, layout q_tiled
    const float* q_gs;         // NVFP4: device fp32 tensor scale of the result (static)
    int q_tiled;               // 1: 128x4 tiled scale layout (padding written as zero), 0: row-major (m, n/blk)
    // The quantised result may be a column block of a wider operand (the N-sharded layer gathers its quantised output):
    int q_ld;                  // bytes per row of the packed operand q_packed points into (n/2 when it is just this result)
    int q_sf_cols;             // scale columns per row of that operand (n/blk when it is just this result)
    int q_sf_col0;             // scale column of this result's column 0 inside it (a multiple of 4)
    int q_n_peers;             // fused all-gather of the quantised result: the same bytes are also stored to the copies of
    uint8_t* q_peer_packed[7]; // the operand in other GPUs' memory (peer-mapped; same layout, same offsets)
    uint8_t* q_peer_sf[7];
    // fp32 partial result for a K-sharded GEMM (kEpiPartial): rows [j * rs_rows, (j + 1) * rs_rows) go, row stride n,
    // to rs_dst[j] -- the slab this rank owns inside rank j's staging buffer (peer-mapped for j != this rank)
    float* rs_dst[8];
    int rs_rows;               // rows per owner, a multiple of 32
    int rs_world;
    int tm_perm_w;             // tile-row order of the schedule, see decode_tile: owners visited in turn (0 = off)
    int tm_first;              // first owner (tm_perm_w > 0) or cyclic shift of the tile rows (tm_perm_w = 0)
    int band;                  // tile rows per band of the schedule (decode_tile), >= 1
    int pdl;                   // 1: launched with programmatic stream serialisation -- the grid may be scheduled while the
                               //    previous kernel in the stream still runs; it touches global memory only after that
                               //    kernel has finished (griddepcontrol.wait), so only launch and set-up are overlapped
};

// Activations of the fused epilogue, evaluated in fp32 on (scaled accumulator + bias) before the bf16 rounding.
enum Activation : int { kActNone = 0, kActRelu = 1, kActGelu = 2, kActGeluTanh = 3, kActSilu = 4 };

// The epilogue warps have about 60 issue slots per element before they fall behind the tensor pipe, and a
// call to a division or erff subroutine per element costs far more (silu with an IEEE division ran the 8192^3
// GEMM at 2.5x its time).  So: sigmoid-type functions are x / (1 + e^-y) with ex2.approx and the approximate
// division (a few ulp of fp32, far inside the bf16 rounding), and erf is Abramowitz & Stegun 7.1.26
// (|error| < 1.5e-7), arranged so that negative inputs need no 1 + erf cancellation.
__device__ __forceinline__ float sigmoid_mul(float x, float y) { return __fdividef(x, 1.0f + __expf(-y)); }   // x * sigmoid(y)

template <int ACT>
__device__ __forceinline__ float activate(float x) {
    if constexpr (ACT == kActRelu) {
        return fmaxf(x, 0.0f);
    } else if constexpr (ACT == kActGelu) {
        const float z = fabsf(x) * 0.70710678118654752f;
        const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
        float poly = fmaf(1.061405429f, t, -1.453152027f);
        poly = fmaf(poly, t, 1.421413741f);
        poly = fmaf(poly, t, -0.284496736f);
        poly = fmaf(poly, t, 0.254829592f);
        const float e = poly * t * __expf(-z * z);          // erfc(z), z >= 0
        return (x >= 0.0f) ? x * fmaf(-0.5f, e, 1.0f) : 0.5f * x * e;
    } else if constexpr (ACT == kActGeluTanh) {
        // 0.5 (1 + tanh u) = sigmoid(2u)
        return sigmoid_mul(x, 1.59576912160573071f * (x + 0.044715f * x * x * x));
    } else if constexpr (ACT == kActSilu) {
        return sigmoid_mul(x, x);
    } else {
        return x;
    }
}

__device__ __forceinline__ float activate_rt(float x, int act) {
    switch (act) {
        case kActRelu: return activate<kActRelu>(x);
        case kActGelu: return activate<kActGelu>(x);
        case kActGeluTanh: return activate<kActGeluTanh>(x);
        case kActSilu: return activate<kActSilu>(x);
        default: return x;
    }
}

// fp32 accumulator columns (two per 32-bit word after the call) -> act(acc * alpha + bias[col]) as bf16 pairs.
template <int ACT, int NCOLS>
__device__ __forceinline__ void convert_bias_act(uint32_t (&packed)[NCOLS], float alpha, const __nv_bfloat16* bias, int col0, int n) {
#pragma unroll
    for (int i = 0; i < NCOLS / 2; ++i) {
        float b0 = 0.0f, b1 = 0.0f;
        const int col = col0 + 2 * i;
        if (bias != nullptr && col < n) {
            const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(bias + col));
            b0 = __uint_as_float(w << 16);
            b1 = __uint_as_float(w & 0xffff0000u);
        }
        const float lo = activate<ACT>(fmaf(__uint_as_float(packed[2 * i]), alpha, b0));
        const float hi = activate<ACT>(fmaf(__uint_as_float(packed[2 * i + 1]), alpha, b1));
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        packed[i] = *reinterpret_cast<uint32_t*>(&h);
    }
}

template <int CTA_GROUP, int BLOCK_N, int SF_VEC, int STAGES, int ACC_STAGES>
struct GemmConfig {
    static constexpr int kBlockM = 128;                 // rows of A per CTA
    static constexpr bool kDense = (SF_VEC == 0);       // SF_VEC 0: dense bf16 operands, no scale factors
    static constexpr int kBlockK = kDense ? 64 : 256;   // K elements per stage = 128 bytes
    static constexpr int kBnCta = BLOCK_N / CTA_GROUP;  // rows of B loaded by one CTA
    static constexpr int kNb = (BLOCK_N + 127) / 128;   // 128-row scale tiles covering BLOCK_N columns
    static constexpr int kSfK = kDense ? 0 : kBlockK / (kDense ? 1 : SF_VEC) / 4;   // scale tiles along K per stage (4 NVFP4, 2 MXFP4)
    static constexpr int kABytes = kBlockM * 128;
    static constexpr int kBBytes = kBnCta * 128;
    static constexpr int kSfaBytes = kSfK * 512;
    static constexpr int kSfbBytes = kNb * kSfK * 512;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr uint32_t kTxBytes = static_cast<uint32_t>(kStageBytes) * CTA_GROUP;
    static constexpr int kEpiWarps = 8;                 // two warps per TMEM lane quadrant
    static constexpr int kEpiGroups = BLOCK_N / 64;     // 64-column (128-byte) output groups per tile row
    static constexpr int kEpiGroups0 = (kEpiGroups + 1) / 2;  // groups drained by the first warp of a quadrant
    static constexpr int kEpiGroups1 = kEpiGroups / 2;        // ... and by the second
    static constexpr int kEpiCols = kEpiGroups0 * 64;   // most accumulator columns one warp holds
    static constexpr int kEpiBufBytes = 32 * 128;       // 32 rows x 64 bf16, one per epilogue warp
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufBytes;
    static constexpr int kOffA = 0;
    static constexpr int kOffB = kOffA + STAGES * kABytes;
    static constexpr int kOffSfa = kOffB + STAGES * kBBytes;
    static constexpr int kOffSfb = kOffSfa + STAGES * kSfaBytes;
    static constexpr int kOffEpi = kOffSfb + STAGES * kSfbBytes;
    // staging of the quantising epilogue's scale tiles: per column half two 512-byte tile images (double-buffered)
    static constexpr int kSfStageBytes = kDense ? 0 : 2 * 2 * 512;
    static constexpr int kOffSfStage = kOffEpi + kEpiBytes;
    static constexpr int kOffBar = kOffSfStage + kSfStageBytes;
    static constexpr int kNumBars = 2 * STAGES + 2 * ACC_STAGES;
    static constexpr int kOffTmemPtr = kOffBar + kNumBars * 8;
    static constexpr int kSmemBytes = kOffTmemPtr + 16 + 1024;  // + slack for 1024-byte alignment
    static constexpr int kTmemAcc = 0;
    static constexpr int kTmemSfa = ACC_STAGES * BLOCK_N;
    static constexpr int kTmemSfb = kTmemSfa + kSfK * 4;
    static constexpr int kTmemUsed = kTmemSfb + kSfK * kNb * 4;
    static constexpr int kTmemCols = kTmemUsed <= 32 ? 32 : kTmemUsed <= 64 ? 64 : kTmemUsed <= 128 ? 128 : kTmemUsed <= 256 ? 256 : 512;
    static constexpr int kThreads = 64 + 32 * kEpiWarps;
    static_assert(BLOCK_N % 64 == 0 && BLOCK_N >= 128 && BLOCK_N <= 256, "BLOCK_N must be 128, 192 or 256");
    static_assert((BLOCK_N / CTA_GROUP) % 8 == 0, "each CTA's B tile must be whole 8-row swizzle groups");
    static_assert(kTmemUsed <= 512, "tensor memory budget");
    static_assert(kOffB % 1024 == 0 && kOffSfa % 1024 == 0 && kOffEpi % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// Tile index -> (tile_m, tile_n): bands of `kGroup` tile rows (chosen by the host: 16 for FP4 operands, 8 for dense
// bf16), M fastest inside a band, so concurrently running CTAs share a few A panels and a few B panels in L2.
// K-sharded GEMMs scatter their tile rows to different owner GPUs, so the order of the tile rows decides where the
// stores go at any moment.  With `perm_w` owners of tiles_m / perm_w tile rows each, consecutive positions of the schedule
// visit the owners in turn, starting with owner `first` (position p -> owner (first + p mod w) mod w, its row p / w): every
// rank sends to every owner all the time, NVLink traffic is spread over the whole kernel and no GPU's ingress is the target
// of all ranks at once.  perm_w = 0: tile rows are only shifted cyclically by `first` (0 = the plain order).
__device__ __forceinline__ void decode_tile(int t, int tiles_m, int tiles_n, int perm_w, int first, int& tm, int& tn, int kGroup) {
    const int band = kGroup * tiles_n;
    const int g = t / band;
    const int first_row = g * kGroup;
    const int gm = min(tiles_m - first_row, kGroup);
    const int r = t - g * band;
    const int pos = first_row + r % gm;
    if (perm_w > 0) {
        const int per_owner = tiles_m / perm_w;
        int owner = first + pos % perm_w;
        if (owner >= perm_w) owner -= perm_w;
        tm = owner * per_owner + pos / perm_w;
    } else {
        tm = pos + first;
        if (tm >= tiles_m) tm -= tiles_m;
    }
    tn = r / gm;
}

// EPI selects the epilogue at compile time, so that the plain kernel keeps its register allocation:
// kEpiPlain: D = bf16(alpha * acc); kEpiBiasAct: D = bf16(act(alpha * acc + bias)).
// kEpiQuant: kEpiBiasAct, then the bf16 values are quantised exactly as quantize_fp4_kernel would quantise them
// (same device functions), so the packed nibbles and scale bytes equal those of the two-kernel sequence; the
// bf16 matrix itself is written only if p.d is not null.
// kEpiPartial: alpha * acc is written as fp32 (no rounding) to the slab of the rank that owns the row: the
// first half of a K-sharded GEMM + reduce-scatter, with the scatter done by the epilogue's own (peer) stores.
enum EpilogueKind : int { kEpiPlain = 0, kEpiBiasAct = 1, kEpiQuant = 2, kEpiPartial = 3 };

template <int CTA_GROUP, int BLOCK_N, int SF_VEC, int STAGES, int ACC_STAGES, int EPI = kEpiPlain>
__global__ void __launch_bounds__(320, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
                const GemmParams p) {
    using Cfg = GemmConfig<CTA_GROUP, BLOCK_N, SF_VEC, STAGES, ACC_STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    // Warp-uniform values go through a shuffle broadcast so that the compiler keeps them, and
    // the addresses and descriptors derived from them, in uniform registers: the TMA and tcgen05
    // instructions read their operands from there, and the issue loops below stay cheap.
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CTA_GROUP == 2) ? __shfl_sync(0xffffffffu, cluster_ctarank(), 0) : 0u;
    const bool is_leader = (cta_rank == 0);
    const int cluster_id = blockIdx.x / CTA_GROUP;
    const int num_clusters = gridDim.x / CTA_GROUP;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_kb = (p.k + Cfg::kBlockK - 1) / Cfg::kBlockK;

    const uint32_t bar_full = smem_base + Cfg::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_tfull = bar_empty + STAGES * 8;
    const uint32_t bar_tempty = bar_tfull + ACC_STAGES * 8;
    const uint32_t tmem_ptr_smem = smem_base + Cfg::kOffTmemPtr;
    volatile uint32_t* tmem_ptr_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::kOffTmemPtr);

    if (threadIdx.x == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&tm_sfa);
        prefetch_tensormap(&tm_sfb);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(bar_tfull + a * 8, 1);
            mbar_init(bar_tempty + a * 8, Cfg::kEpiWarps * CTA_GROUP);
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<CTA_GROUP>(tmem_ptr_smem, Cfg::kTmemCols);
        tmem_relinquish<CTA_GROUP>();
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_ptr_gen, 0);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp walks the loop (so loop state is warp-uniform); one elected lane issues.
        {
            const bool issuer = elect_one_sync();
            if (p.pdl) {
                if (issuer) pdl_launch_dependents();   // the next kernel may be scheduled as soon as SMs free up
                pdl_wait_prior_grid();                 // operands may come from the previous kernel
            }
            const uint32_t full0 = (CTA_GROUP == 2) ? mapa_shared(bar_full, 0) : bar_full;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const bool tr = (p.trace != nullptr) && (blockIdx.x == 0);
            int rec = 0;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
                int tm, tn;
                decode_tile(t, p.tiles_m, p.tiles_n, p.tm_perm_w, p.tm_first, tm, tn, p.band);
                const int row_a = (tm * CTA_GROUP + static_cast<int>(cta_rank)) * Cfg::kBlockM;
                const int row_b = tn * BLOCK_N + static_cast<int>(cta_rank) * Cfg::kBnCta;
                const int sfa_atom0 = (row_a / 128) * p.sf_k_atoms;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const long long t0 = tr ? clock64() : 0;
                    if (!mbar_wait(bar_empty + stage * 8, phase ^ 1u)) {
                        if (issuer) atomicCAS(p.status, 0, kStatusTimeoutProducer);
                        ok = false;
                        break;
                    }
                    const long long t1 = tr ? clock64() : 0;
                    const uint32_t full = full0 + stage * 8;
                    if (issuer) {
                        if (is_leader) mbar_arrive_expect_tx(bar_full + stage * 8, Cfg::kTxBytes);
                        tma_load_2d<CTA_GROUP, 2>(smem_base + Cfg::kOffA + stage * Cfg::kABytes, &tm_a, full, kb * 128, row_a);
                        tma_load_2d<CTA_GROUP, 2>(smem_base + Cfg::kOffB + stage * Cfg::kBBytes, &tm_b, full, kb * 128, row_b);
                        if constexpr (!Cfg::kDense) {
                            tma_load_2d<CTA_GROUP, 2>(smem_base + Cfg::kOffSfa + stage * Cfg::kSfaBytes, &tm_sfa, full, 0,
                                                   sfa_atom0 + kb * Cfg::kSfK);
#pragma unroll
                            for (int nb = 0; nb < Cfg::kNb; ++nb) {
                                tma_load_2d<CTA_GROUP, 2>(smem_base + Cfg::kOffSfb + stage * Cfg::kSfbBytes + nb * Cfg::kSfK * 512,
                                                       &tm_sfb, full, 0,
                                                       ((tn * BLOCK_N) / 128 + nb) * p.sf_k_atoms + kb * Cfg::kSfK);
                            }
                        }
                        if (tr && rec < p.trace_cap) {
                            long long* r = p.trace + (0ll * p.trace_cap + rec) * 4;
                            r[0] = t0; r[1] = t1; r[2] = clock64(); r[3] = stage;
                        }
                    }
                    ++rec;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (ok) {
                // Drain: wait until every stage this CTA filled has been consumed, so no
                // copy is in flight and no peer signal is outstanding when the CTA exits.
                for (int i = 0; i < STAGES; ++i) {
                    if (!mbar_wait(bar_empty + stage * 8, phase ^ 1u)) {
                        if (issuer) atomicCAS(p.status, 0, kStatusTimeoutProducer);
                        break;
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        if (is_leader) {
            constexpr int kMmaM = 128 * CTA_GROUP;
            constexpr bool kUe8m0 = (SF_VEC == 32);
            const bool issuer = elect_one_sync();
            int stage = 0;
            uint32_t phase = 0;
            int tile_iter = 0;
            bool ok = true;
            const bool tr = (p.trace != nullptr) && (blockIdx.x == 0);
            int rec = 0;
            for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++tile_iter) {
                const int acc = tile_iter % ACC_STAGES;
                const uint32_t acc_phase = static_cast<uint32_t>(tile_iter / ACC_STAGES) & 1u;
                const long long ta = tr ? clock64() : 0;
                if (!mbar_wait(bar_tempty + acc * 8, acc_phase ^ 1u)) {
                    if (issuer) atomicCAS(p.status, 0, kStatusTimeoutMma);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + Cfg::kTmemAcc + acc * BLOCK_N;
                // A tile that starts inside a 128-row scale tile (BLOCK_N = 192, odd tiles) reads its
                // B scales from a column offset: 32 rows of B per TMEM column.
                uint32_t sfb_shift = 0;
                if constexpr (BLOCK_N % 128 != 0) {
                    int tm, tn;
                    decode_tile(t, p.tiles_m, p.tiles_n, p.tm_perm_w, p.tm_first, tm, tn, p.band);
                    sfb_shift = static_cast<uint32_t>(((tn * BLOCK_N) % 128) / 32);
                }
                for (int kb = 0; kb < num_kb; ++kb) {
                    const long long t0 = tr ? (kb == 0 ? ta : clock64()) : 0;
                    if (!mbar_wait(bar_full + stage * 8, phase)) {
                        if (issuer) atomicCAS(p.status, 0, kStatusTimeoutMma);
                        ok = false;
                        break;
                    }
                    const long long t1 = tr ? clock64() : 0;
                    tcgen05_fence_after();
                    const uint32_t sfa_s = smem_base + Cfg::kOffSfa + stage * Cfg::kSfaBytes;
                    const uint32_t sfb_s = smem_base + Cfg::kOffSfb + stage * Cfg::kSfbBytes;
                    const uint64_t sfa_desc = make_desc_sf(sfa_s);
                    const uint64_t sfb_desc = make_desc_sf(sfb_s);
                    const uint64_t a_desc = make_desc_k_sw128(smem_base + Cfg::kOffA + stage * Cfg::kABytes);
                    const uint64_t b_desc = make_desc_k_sw128(smem_base + Cfg::kOffB + stage * Cfg::kBBytes);
                    const uint32_t accum0 = (kb > 0) ? 1u : 0u;
                    if (issuer) {
#pragma unroll
                        for (int j = 0; j < Cfg::kSfK; ++j) {
                            // descriptor start address is in 16-byte units: one 512-byte scale tile = 32
                            tmem_cp_sf<CTA_GROUP>(tmem_base + Cfg::kTmemSfa + j * 4, sfa_desc + static_cast<uint64_t>(j * 32));
#pragma unroll
                            for (int nb = 0; nb < Cfg::kNb; ++nb)
                                tmem_cp_sf<CTA_GROUP>(tmem_base + Cfg::kTmemSfb + (j * Cfg::kNb + nb) * 4,
                                                      sfb_desc + static_cast<uint64_t>((nb * Cfg::kSfK + j) * 32));
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            // one MMA K step = 32 bytes along the swizzled 128-byte row = 2 address units
                            if constexpr (Cfg::kDense) {
                                mma_bf16<CTA_GROUP>(d_tmem, a_desc + static_cast<uint64_t>(j * 2), b_desc + static_cast<uint64_t>(j * 2),
                                                    make_idesc_bf16(kMmaM, BLOCK_N), (j > 0) ? 1u : accum0);
                            } else {
                                constexpr bool nv = (SF_VEC == 16);
                                const int sf_tile = nv ? j : (j >> 1);
                                const int sf_id = nv ? 0 : 2 * (j & 1);
                                const uint32_t idesc = make_idesc_fp4(kMmaM, BLOCK_N, kUe8m0, sf_id);
                                mma_fp4_block_scaled<CTA_GROUP, (Cfg::kDense ? 16 : SF_VEC)>(
                                    d_tmem, a_desc + static_cast<uint64_t>(j * 2), b_desc + static_cast<uint64_t>(j * 2), idesc,
                                    tmem_base + Cfg::kTmemSfa + sf_tile * 4,
                                    tmem_base + Cfg::kTmemSfb + sf_tile * Cfg::kNb * 4 + sfb_shift,
                                    (j > 0) ? 1u : accum0);
                            }
                        }
                        tcgen05_commit<CTA_GROUP>(bar_empty + stage * 8);
                        if (tr && rec < p.trace_cap) {
                            long long* r = p.trace + (1ll * p.trace_cap + rec) * 4;
                            r[0] = t0; r[1] = t1; r[2] = clock64(); r[3] = kb;
                        }
                    }
                    ++rec;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok && issuer) tcgen05_commit<CTA_GROUP>(bar_tfull + acc * 8);
                __syncwarp();
            }
        }
    } else {
        // --------------------------------------------------------------- epilogue
        const int quad = warp & 3;             // TMEM lane quadrant this warp may access
        const int half = (warp - 2) >> 2;      // which half of the accumulator columns
        const uint32_t sbuf = smem_base + Cfg::kOffEpi + (warp - 2) * Cfg::kEpiBufBytes;
        // everything this role reads (tensor scales, bias) or writes may be touched by the previous kernel
        if (p.pdl) pdl_wait_prior_grid();
        float alpha = 1.0f;
        if (p.a_gs) alpha *= __ldg(p.a_gs);
        if (p.b_gs) alpha *= __ldg(p.b_gs);
        // constants of the quantising epilogue (the divisions a / 6 / gs are done with reciprocals, see quantize_block)
        float q_gs = 1.0f;
        if (EPI == kEpiQuant && SF_VEC == 16 && p.q_gs != nullptr) q_gs = __ldg(p.q_gs);
        const bool q_gs_plain = divisor_is_plain(q_gs);
        const float q_gs_recip = __frcp_rn(q_gs);
        const float sixth = __frcp_rn(6.0f);
        const uint32_t tempty0 = (CTA_GROUP == 2) ? mapa_shared(bar_tempty, 0) : bar_tempty;
        const int my_groups = (half == 0) ? Cfg::kEpiGroups0 : Cfg::kEpiGroups1;   // warp-uniform
        const int my_col = (half == 0) ? 0 : Cfg::kEpiGroups0 * 64;
        int tile_iter = 0;
        int sf_stage_parity = 0;     // which of the two scale-tile images of this column half is written next
        for (int t = cluster_id; t < num_tiles; t += num_clusters, ++tile_iter) {
            int tm, tn;
            decode_tile(t, p.tiles_m, p.tiles_n, p.tm_perm_w, p.tm_first, tm, tn, p.band);
            const int acc = tile_iter % ACC_STAGES;
            const uint32_t acc_phase = static_cast<uint32_t>(tile_iter / ACC_STAGES) & 1u;
            const bool tr = (p.trace != nullptr) && (blockIdx.x == 0) && (warp == 2) && (lane == 0) && (tile_iter < p.trace_cap);
            const long long te0 = tr ? clock64() : 0;
            if (!mbar_wait(bar_tfull + acc * 8, acc_phase)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
                break;
            }
            const long long te1 = tr ? clock64() : 0;
            tcgen05_fence_after();
            const int row0 = (tm * CTA_GROUP + static_cast<int>(cta_rank)) * Cfg::kBlockM + quad * 32;
            const int col0 = tn * BLOCK_N + my_col;
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + Cfg::kTmemAcc + acc * BLOCK_N + my_col;
            // ---- drain: all of this warp's accumulator columns go to registers with the loads in
            // flight together (one round trip), then the accumulator is handed back at once
            uint32_t packed[Cfg::kEpiCols];
#pragma unroll
            for (int c = 0; c < Cfg::kEpiGroups0; ++c)
                if (c < my_groups) tmem_ld_32x32b_x64(t_acc + c * 64, &packed[c * 64]);
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CTA_GROUP == 2) mbar_arrive_cluster(tempty0 + acc * 8);
                else mbar_arrive(bar_tempty + acc * 8);
            }
            // fp32 -> bf16 pairs in place: word i takes columns 2i and 2i+1
            if constexpr (EPI == kEpiPartial) {
#pragma unroll
                for (int i = 0; i < Cfg::kEpiCols; ++i) packed[i] = __float_as_uint(__uint_as_float(packed[i]) * alpha);
            } else if constexpr (EPI == kEpiPlain) {
#pragma unroll
                for (int i = 0; i < Cfg::kEpiCols / 2; ++i) {
                    const float lo = __uint_as_float(packed[2 * i]) * alpha;
                    const float hi = __uint_as_float(packed[2 * i + 1]) * alpha;
                    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                    packed[i] = *reinterpret_cast<uint32_t*>(&h);
                }
            } else {
                switch (p.act) {   // warp-uniform
                    case kActRelu: convert_bias_act<kActRelu>(packed, alpha, p.bias, col0, p.n); break;
                    case kActGelu: convert_bias_act<kActGelu>(packed, alpha, p.bias, col0, p.n); break;
                    case kActGeluTanh: convert_bias_act<kActGeluTanh>(packed, alpha, p.bias, col0, p.n); break;
                    case kActSilu: convert_bias_act<kActSilu>(packed, alpha, p.bias, col0, p.n); break;
                    default: convert_bias_act<kActNone>(packed, alpha, p.bias, col0, p.n); break;
                }
            }
            if constexpr (EPI == kEpiQuant && !Cfg::kDense) {
                constexpr int QFMT = (SF_VEC == 16) ? kFmtNvfp4 : kFmtMxfp4;
                constexpr int BLK = SF_VEC;                 // elements per scale block
                constexpr int NB = 64 / BLK;                // blocks per 64-column group (4 or 2)
                const int row = row0 + lane;
                const int sf_cols = p.q_sf_cols;              // of the whole operand this result is a column block of
                const int k_atoms = (sf_cols + 3) / 4;
                const int sf_cols_here = p.n / BLK;           // scale columns this GEMM produces
                // the zero padding up to a multiple of 4 scale columns belongs to the block that ends the operand;
                // a block with a neighbour to its right must not write past its own columns
                const int sf_cols_limit = (p.q_sf_col0 + sf_cols_here == sf_cols) ? k_atoms * 4 - p.q_sf_col0 : sf_cols_here;
                const int rows_pad = ((p.m + 127) / 128) * 128;
                // Whole 128-byte rows of packed output: with 256-column tiles, no bf16 output (the staging buffers are
                // free) and the tile inside N, the two warps of a lane quadrant (column halves) put their 64 bytes per row
                // side by side in one 4 KB staging buffer and then write 32 rows x 128 bytes as whole lines, eight lanes per
                // row -- to this GPU and to the peers, where a 128-byte store uses NVLink four times better than 32-byte ones.
                // The conditions depend on the tile and the launch only, so both warps agree.
                const bool line_rows = (BLOCK_N == 256) && (p.d == nullptr) && (tn * BLOCK_N + BLOCK_N <= p.n) &&
                                       (((p.q_ld | static_cast<int>(reinterpret_cast<uintptr_t>(p.q_packed))) & 15) == 0);
                const uint32_t qbuf = smem_base + Cfg::kOffEpi + (((warp - 2) & 3) + 4 * (tile_iter & 1)) * Cfg::kEpiBufBytes;
#pragma unroll
                for (int g = 0; g < Cfg::kEpiGroups0; ++g) {
                    if (g >= my_groups) break;
                    const int colg = col0 + g * 64;
                    uint32_t codes = 0;
                    uint32_t w[8];
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        uint32_t code = quantize_block<QFMT>(&packed[g * 32 + b * (BLK / 2)], q_gs, q_gs_plain, q_gs_recip, sixth,
                                                             &w[b * (BLK / 8)]);
                        if (colg + b * BLK >= p.n || row >= p.m) code = 0;   // padding of the scale layout is zero
                        codes |= code << (8 * b);
                    }
                    const size_t pk_off = static_cast<size_t>(row) * p.q_ld + colg / 2;
                    if (line_rows) {
                        // lane = row; 16-byte chunk q of the 128-byte row lives at chunk q ^ (row & 7)
                        const int q0 = (half * Cfg::kEpiGroups0 + g) * 2;
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(qbuf + lane * 128 + ((q0 ^ (lane & 7)) << 4)),
                                     "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(qbuf + lane * 128 + (((q0 + 1) ^ (lane & 7)) << 4)),
                                     "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
                    } else if (row < p.m) {
                        if (colg + 64 <= p.n && ((p.q_ld | static_cast<int>(reinterpret_cast<uintptr_t>(p.q_packed))) & 31) == 0) {
                            // whole group, rows 32-byte aligned: the row's 32 bytes as one 256-bit store, i.e. one whole
                            // sector per lane (the form that also goes to the peers; the host admits peers only for such
                            // shapes -- over NVLink a store of part of a sector costs as much as a whole one)
                            st_global_v8_cs(p.q_packed + pk_off, w);
                            for (int pi = 0; pi < p.q_n_peers; ++pi) st_global_v8_cs(p.q_peer_packed[pi] + pk_off, w);
                        } else {
                            uint8_t* dst = p.q_packed + pk_off;
#pragma unroll
                            for (int h = 0; h < 4; ++h)     // 16 columns = 8 bytes each; N % 16 == 0
                                if (colg + h * 16 < p.n) *reinterpret_cast<uint2*>(dst + h * 8) = make_uint2(w[2 * h], w[2 * h + 1]);
                        }
                    }
                    const int c = colg / BLK;           // first scale column of the group (multiple of NB) in this result
                    const int cg = p.q_sf_col0 + c;     // ... and in the operand it is a block of
                    if (p.q_tiled) {
                        if (row < rows_pad && c < sf_cols_limit) {
                            const long long so = sf_tiled_offset(row, cg, k_atoms);
                            if constexpr (NB == 4) {
                                // One 64-column group of the CTA's 128 rows is exactly one 512-byte scale tile, spread
                                // over the four quadrant warps (16-byte slot l holds rows l, l+32, l+64, l+96).  The warps
                                // put their 4 bytes per row into a tile image in shared memory and the first of them
                                // writes the image as 512 contiguous bytes -- four whole lines -- to this GPU and the
                                // peers, instead of 128 scattered 4-byte stores.  (All four warps take this branch
                                // together: the conditions above depend on the tile and the group only.)
                                const uint32_t img = smem_base + Cfg::kOffSfStage + (half * 2 + (sf_stage_parity & 1)) * 512;
                                asm volatile("st.shared.b32 [%0], %1;" ::"r"(img + lane * 16 + quad * 4), "r"(codes) : "memory");
                                if (half == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
                                else asm volatile("bar.sync 4, 128;" ::: "memory");
                                if (quad == 0) {
                                    uint32_t v0, v1, v2, v3;
                                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(img + lane * 16) : "memory");
                                    const long long tile_off = sf_tiled_offset(row0 - quad * 32, cg, k_atoms) + lane * 16;
                                    *reinterpret_cast<uint4*>(p.q_sf + tile_off) = make_uint4(v0, v1, v2, v3);
                                    for (int pi = 0; pi < p.q_n_peers; ++pi)
                                        __stcs(reinterpret_cast<uint4*>(p.q_peer_sf[pi] + tile_off), make_uint4(v0, v1, v2, v3));
                                }
                                ++sf_stage_parity;
                            } else {
                                // MXFP4: a group carries two scale columns, so with 256-column tiles the two groups of a
                                // column half make one scale tile; staged like the NVFP4 one and written after the second
                                // group, when both groups lie inside this result's columns and the result starts on a tile
                                // boundary of the operand it is a block of (conditions of the tile and the launch alone)
                                const bool staged = (BLOCK_N == 256) && (col0 / BLK + 4 <= sf_cols_limit) && ((p.q_sf_col0 & 3) == 0);
                                if (staged) {
                                    const uint32_t img = smem_base + Cfg::kOffSfStage + (half * 2 + (sf_stage_parity & 1)) * 512;
                                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(img + lane * 16 + quad * 4 + (g & 1) * 2),
                                                 "h"(static_cast<uint16_t>(codes)) : "memory");
                                    if (g == 1) {
                                        if (half == 0) asm volatile("bar.sync 3, 128;" ::: "memory");
                                        else asm volatile("bar.sync 4, 128;" ::: "memory");
                                        if (quad == 0) {
                                            uint32_t v0, v1, v2, v3;
                                            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(img + lane * 16) : "memory");
                                            const long long tile_off = sf_tiled_offset(row0 - quad * 32, cg - 2, k_atoms) + lane * 16;
                                            *reinterpret_cast<uint4*>(p.q_sf + tile_off) = make_uint4(v0, v1, v2, v3);
                                            for (int pi = 0; pi < p.q_n_peers; ++pi)
                                                __stcs(reinterpret_cast<uint4*>(p.q_peer_sf[pi] + tile_off), make_uint4(v0, v1, v2, v3));
                                        }
                                        ++sf_stage_parity;
                                    }
                                } else {
                                    *reinterpret_cast<uint16_t*>(p.q_sf + so) = static_cast<uint16_t>(codes);
                                    for (int pi = 0; pi < p.q_n_peers; ++pi)
                                        __stcs(reinterpret_cast<unsigned short*>(p.q_peer_sf[pi] + so), static_cast<unsigned short>(codes));
                                }
                            }
                        }
                    } else if (row < p.m) {
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (c + b < sf_cols_here) {
                                const size_t so = static_cast<size_t>(row) * sf_cols + cg + b;
                                p.q_sf[so] = static_cast<uint8_t>(codes >> (8 * b));
                                for (int pi = 0; pi < p.q_n_peers; ++pi) p.q_peer_sf[pi][so] = static_cast<uint8_t>(codes >> (8 * b));
                            }
                    }
                }
                if (line_rows) {
                    // both column halves of this quadrant have staged their 64 bytes per row (one named barrier per quadrant;
                    // the buffer alternates with the tile, so the next tile's staging cannot overtake this read-out)
                    switch (quad) {
                        case 0: asm volatile("bar.sync 5, 64;" ::: "memory"); break;
                        case 1: asm volatile("bar.sync 6, 64;" ::: "memory"); break;
                        case 2: asm volatile("bar.sync 7, 64;" ::: "memory"); break;
                        default: asm volatile("bar.sync 8, 64;" ::: "memory"); break;
                    }
                    // each of the two warps writes 16 of the 32 rows: eight lanes per 128-byte row, four rows per instruction
                    const int q = lane & 7;
                    const size_t col_off = static_cast<size_t>(tn) * (BLOCK_N / 2) + q * 16;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = half * 16 + i * 4 + (lane >> 3);
                        uint32_t v0, v1, v2, v3;
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                     : "r"(qbuf + r * 128 + ((q ^ (r & 7)) << 4)) : "memory");
                        const int grow = row0 + r;
                        if (grow < p.m) {
                            const size_t off = static_cast<size_t>(grow) * p.q_ld + col_off;
                            *reinterpret_cast<uint4*>(p.q_packed + off) = make_uint4(v0, v1, v2, v3);
                            for (int pi = 0; pi < p.q_n_peers; ++pi)
                                __stcs(reinterpret_cast<uint4*>(p.q_peer_packed[pi] + off), make_uint4(v0, v1, v2, v3));
                        }
                    }
                }
            }
            const long long te2 = tr ? clock64() : 0;
            // ---- write out: 32 rows x 64 columns at a time through a swizzled transpose, so
            // that every global store instruction writes four complete 128-byte lines
            // A 128-byte row piece is 64 bf16 columns, or 32 fp32 columns of a partial result.
            constexpr int kPieceCols = (EPI == kEpiPartial) ? 32 : 64;
            constexpr int kPieces0 = Cfg::kEpiCols / kPieceCols;
            const int my_pieces = my_groups * (64 / kPieceCols);
            // partial results: all 32 rows of this warp belong to one owner (rs_rows is a multiple of 32)
            float* rs_base = nullptr;
            if constexpr (EPI == kEpiPartial) {
                const int owner = min(row0 / p.rs_rows, p.rs_world - 1);
                rs_base = p.rs_dst[owner] - static_cast<size_t>(owner) * p.rs_rows * p.n;
            }
#pragma unroll
            for (int g = 0; g < kPieces0; ++g) {
                if (g >= my_pieces) break;
                if (EPI == kEpiQuant && p.d == nullptr) break;   // quantised result only
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    // lane = row; 16-byte chunk q of the row lives at chunk q ^ (row & 7)
                    const uint32_t addr = sbuf + lane * 128 + ((q ^ (lane & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[g * 32 + 4 * q]),
                                 "r"(packed[g * 32 + 4 * q + 1]), "r"(packed[g * 32 + 4 * q + 2]),
                                 "r"(packed[g * 32 + 4 * q + 3])
                                 : "memory");
                }
                __syncwarp();
                const int q = lane & 7;
                const int col = col0 + g * kPieceCols + q * (kPieceCols / 8);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = i * 4 + (lane >> 3);
                    const uint32_t addr = sbuf + r * 128 + ((q ^ (r & 7)) << 4);
                    uint32_t w0, w1, w2, w3;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(addr) : "memory");
                    const int row = row0 + r;
                    if (row < p.m && col < p.n) {
                        if constexpr (EPI == kEpiPartial) {
                            __stcs(reinterpret_cast<uint4*>(rs_base + static_cast<size_t>(row) * p.n + col), make_uint4(w0, w1, w2, w3));
                        } else {
                            // streaming store: the output is not re-read here and should not push the
                            // operands (which other CTAs still need) out of L2
                            const size_t off = static_cast<size_t>(row) * p.ldd + col;
                            __stcs(reinterpret_cast<uint4*>(p.d + off), make_uint4(w0, w1, w2, w3));
                            // fused all-gather: push the same 128-byte lines straight into every peer's copy
                            // over NVLink (plain peer stores), so the exchange overlaps the next tiles' math
                            for (int pi = 0; pi < p.n_peers; ++pi)
                                __stcs(reinterpret_cast<uint4*>(p.peer_d[pi] + off), make_uint4(w0, w1, w2, w3));
                        }
                    }
                }
            }
            if (tr) {
                long long* r = p.trace + (2ll * p.trace_cap + tile_iter) * 4;
                r[0] = te0; r[1] = te1; r[2] = te2; r[3] = clock64();
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) cluster_sync_all();
    if (warp == 1) tmem_dealloc<CTA_GROUP>(tmem_base, Cfg::kTmemCols);
}

// Second half of the K-sharded GEMM + reduce-scatter: D (rows, n) bf16 = act(sum over r of slab r + bias), slabs
// fp32 (rows, n) back to back, summed in slab order so that the result does not depend on arrival order.
// A thread takes 8 consecutive columns: two 128-bit loads per slab, one 128-bit store.
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ slabs, int world, long long rows, long long n, __nv_bfloat16* __restrict__ d,
                       long long ldd, const __nv_bfloat16* __restrict__ bias, int act) {
    const long long groups_per_row = n / 8;
    const long long total = rows * groups_per_row;
    const long long slab_elems = rows * n;
    for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < total;
         g += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = g / groups_per_row;
        const long long c = (g - r * groups_per_row) * 8;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int w = 0; w < world; ++w) {
            const float4* src = reinterpret_cast<const float4*>(slabs + w * slab_elems + r * n + c);
            const float4 lo = __ldcs(src), hi = __ldcs(src + 1);
            acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
            acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
        }
        if (bias != nullptr) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias + c));
            const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] += __uint_as_float(bw[i] << 16);
                acc[2 * i + 1] += __uint_as_float(bw[i] & 0xffff0000u);
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(activate_rt(acc[2 * i], act), activate_rt(acc[2 * i + 1], act));
            o[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(d + r * ldd + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace avefp4
