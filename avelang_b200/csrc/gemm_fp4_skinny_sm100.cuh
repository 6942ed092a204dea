// Skinny (decode-shaped) block-scaled FP4 GEMM for sm_100a:
//   D[M,N] (bf16) = alpha * X[M,K] * W[N,K]^T   with M <= MP <= 64.
//
// The weight matrix streams from HBM once, so the kernel is bandwidth-bound.  The
// operands are swapped on the tensor core: 128 weight rows sit on the MMA M axis
// (TMEM lanes) and the few activation rows on the MMA N axis (TMEM columns), so a
// 128 x MP x 64 tcgen05.mma does the work without padding M up to 128.
//
// Work is split so that every SM pulls the same number of bytes, in two phases.  With T weight
// tiles and G persistent CTAs, the first T mod G tiles are split stream-K style: their (tile, K block)
// units are cut into min(G, units) equal contiguous ranges, one per CTA.  A range that covers only part of a
// tile's K writes an fp32 partial to scratch memory; the CTA that completes a tile last (per-tile
// arrival counter) adds the partials in a fixed order and writes the bf16 result, so the output is
// deterministic and nobody waits on another CTA.  After its range every CTA computes floor(T / G)
// whole tiles of its own.  The stream-K part comes first, so its partial-sum round trips run under
// the following tiles' loads, and the kernel ends with a plain whole-tile write-out.
//
// Plays the role of python/avelang_kernels/amdgpu_gemm.py:349-455 for the shapes
// the reference tile (128x128) cannot fill.
#pragma once

#include <cuda_bf16.h>

#include <type_traits>

#include "gemm_fp4_sm100.cuh"

namespace avefp4 {

struct SkinnyParams {
    int m, n, k;
    int tiles_n;          // ceil(N / 128)
    int w_sf_k_atoms;     // scale tiles along K
    int ldd;              // row stride of D in elements
    int pdl;              // 1: launched with programmatic stream serialisation; weights may be read before the
                          //    previous kernel in the stream has finished, everything else waits for it
    int burst;            // K blocks whose loads are issued together (1 .. min(8, STAGES))
    int w_tile_major;     // 0: W packed row-major (N, K/2); 1: 16 KB tiles [N/128][K/256][128 rows][128 B]
    int no_streamk;       // 1: whole tiles only, tile t on CTA t mod G (the schedule the stream-K split is measured against)
    const float* x_gs;    // device fp32 tensor scales or nullptr
    const float* w_gs;
    __nv_bfloat16* d;
    float* partials;      // gridDim.x * 2 * MP * 128 fp32
    int* counters;        // 4 * tiles_n ints, zero on entry, zero again on exit
    int* status;
    long long* trace;     // optional clock64() stamps of CTA 0 (same record layout as the tiled kernel)
    int trace_cap;
    const __nv_bfloat16* bias;  // fused epilogue: n values (one per weight row), or nullptr
    int act;                    // fused epilogue activation (Activation enum of the tiled kernel)
};

template <int MP, int SF_VEC, int STAGES>
struct SkinnyConfig {
    static constexpr int kBlockK = 256;
    static constexpr int kSfK = kBlockK / SF_VEC / 4;
    static constexpr int kWBytes = 128 * 128;
    static constexpr int kXBytes = MP * 128;
    static constexpr int kSfBytes = kSfK * 512;
    static constexpr int kStageBytes = kWBytes + kXBytes + 2 * kSfBytes;
    static constexpr int kAccStages = 2;
    static constexpr int kOffW = 0;
    static constexpr int kOffX = kOffW + STAGES * kWBytes;
    static constexpr int kOffSfw = kOffX + STAGES * kXBytes;
    static constexpr int kOffSfx = kOffSfw + STAGES * kSfBytes;
    static constexpr int kOffBar = kOffSfx + STAGES * kSfBytes;
    static constexpr int kNumBars = 2 * STAGES + 2 * kAccStages;
    static constexpr int kOffTmemPtr = kOffBar + kNumBars * 8;
    static constexpr int kOffFlag = kOffTmemPtr + 8;
    static constexpr int kSmemBytes = kOffFlag + 8 + 1024;
    static constexpr int kTmemSfw = kAccStages * MP;
    static constexpr int kTmemSfx = kTmemSfw + kSfK * 4;
    static constexpr int kTmemUsed = kTmemSfx + kSfK * 4;
    static constexpr int kTmemCols = kTmemUsed <= 32 ? 32 : kTmemUsed <= 64 ? 64 : kTmemUsed <= 128 ? 128 : kTmemUsed <= 256 ? 256 : 512;
    static_assert(MP % 16 == 0 && MP >= 16 && MP <= 128, "MP must be a multiple of 16 up to 128");
    static_assert(kTmemUsed <= 512, "tensor memory budget");
    static_assert((MP * 128) % 1024 == 0, "activation tile must keep 1024-byte alignment of later stages");
    static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// CTA whose unit range [floor(i*U/G), floor((i+1)*U/G)) holds unit u.
__device__ __forceinline__ int skinny_cta_of(long long u, long long units, long long ctas) {
    return static_cast<int>(((u + 1) * ctas - 1) / units);
}

template <int MP, int SF_VEC, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_fp4_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_sfw, const __grid_constant__ CUtensorMap tm_sfx,
                       const SkinnyParams p) {
    using Cfg = SkinnyConfig<MP, SF_VEC, STAGES>;
    constexpr int ACC = Cfg::kAccStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    // warp-uniform values via a shuffle broadcast: keeps issue-loop state in uniform registers
    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const int num_kb = (p.k + Cfg::kBlockK - 1) / Cfg::kBlockK;
    const long long ctas = gridDim.x;
    // whole tiles per CTA (second phase); tiles 0 .. sk_tiles-1 are split stream-K
    const int whole_tiles = p.no_streamk ? (p.tiles_n - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x)
                                         : p.tiles_n / static_cast<int>(gridDim.x);
    const int sk_tiles = p.no_streamk ? 0 : p.tiles_n - whole_tiles * static_cast<int>(gridDim.x);
    const long long units = static_cast<long long>(sk_tiles) * num_kb;           // stream-K units, cut into equal ranges
    // Only min(G, units) CTAs take part in the stream-K phase, so that every one of them owns at least one unit:
    // the finish test below counts one contribution from every CTA between the first and the last owner of a tile.
    // (With more CTAs than units -- many tiles, short K -- the other CTAs go straight to their whole tiles.)
    const long long sk_ctas = units < ctas ? units : ctas;
    const bool in_sk = static_cast<long long>(blockIdx.x) < sk_ctas;
    const long long u_begin = in_sk ? (static_cast<long long>(blockIdx.x) * units) / sk_ctas : 0;
    const long long u_end = in_sk ? (static_cast<long long>(blockIdx.x + 1) * units) / sk_ctas : 0;
    const int first_whole = sk_tiles + static_cast<int>(blockIdx.x);              // then tiles first_whole + j * G

    const uint32_t bar_full = smem_base + Cfg::kOffBar;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_tfull = bar_empty + STAGES * 8;
    const uint32_t bar_tempty = bar_tfull + ACC * 8;
    const uint32_t tmem_ptr_smem = smem_base + Cfg::kOffTmemPtr;
    volatile uint32_t* tmem_ptr_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + Cfg::kOffTmemPtr);

    // Set-up.  Warp 0 initialises the barriers and goes straight on to issue loads (it only
    // arrives at the set-up barrier); the other warps wait there for the barriers and for the
    // tensor-memory allocation made by warp 1.  This takes the set-up off the critical path of
    // the first weight tiles, which matters for a kernel that runs for ~20 us.
    if (warp == 0) {
        if (elect_one_sync()) {
            prefetch_tensormap(&tm_w);
            prefetch_tensormap(&tm_x);
            prefetch_tensormap(&tm_sfw);
            prefetch_tensormap(&tm_sfx);
            for (int s = 0; s < STAGES; ++s) {
                mbar_init(bar_full + s * 8, 1);
                mbar_init(bar_empty + s * 8, 1);
            }
            for (int a = 0; a < ACC; ++a) {
                mbar_init(bar_tfull + a * 8, 1);
                mbar_init(bar_tempty + a * 8, 4);
            }
            fence_mbar_init();
        }
        __syncwarp();
        asm volatile("bar.arrive 1, 192;" ::: "memory");
    } else {
        if (warp == 1) {
            tmem_alloc<1>(tmem_ptr_smem, Cfg::kTmemCols);
            tmem_relinquish<1>();
        }
        tcgen05_fence_before();
        asm volatile("bar.sync 1, 192;" ::: "memory");
        tcgen05_fence_after();
    }
    const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_ptr_gen, 0);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        // the whole warp walks the loop (warp-uniform state); one elected lane issues
        {
            const bool issuer = elect_one_sync();
            if (issuer) pdl_launch_dependents();
            bool prior_done = (p.pdl == 0);
            // Loads are issued in bursts of kBurst consecutive K blocks: the weight tiles of a
            // burst are neighbouring 128-byte pieces of the same 128 rows, so DRAM sees
            // 512 contiguous bytes per row and page visit instead of 128.
            constexpr int kBurst = (STAGES < 8) ? STAGES : 8;   // upper bound; p.burst is the size used
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const bool tr = (p.trace != nullptr) && (blockIdx.x == 0);
            int rec = 0;
            // (tile, K block) of the next unit, advanced incrementally (no division in the loop)
            int tile = static_cast<int>(u_begin / num_kb);
            int kb = static_cast<int>(u_begin - static_cast<long long>(tile) * num_kb);
            int left_sk = static_cast<int>(u_end - u_begin);               // units left in the stream-K range
            if (left_sk == 0) { tile = first_whole; kb = 0; }
            int left = left_sk + whole_tiles * num_kb;
            const int tile_step = static_cast<int>(gridDim.x);
            // next unit after (t, k): inside the stream-K range the next K block or tile; after its last unit the
            // first whole tile; among the whole tiles every gridDim.x-th tile
            auto advance = [&](int& t, int& k, int& lsk) {
                if (lsk > 0 && --lsk == 0) { t = first_whole; k = 0; return; }
                if (++k == num_kb) { k = 0; t += (lsk > 0) ? 1 : tile_step; }
            };
            while (left > 0 && ok) {
                const long long t0 = tr ? clock64() : 0;
                // the first burst fills the whole ring (every slot is free): all of these weight loads are in flight
                // before the producer waits for the previous kernel's activations
                const int want = (rec == 0) ? STAGES : p.burst;
                const int g = left < want ? left : want;
                // slots are released in order, so a free last slot means the whole burst is free
                const int last = stage + g - 1;
                const int last_stage = last >= STAGES ? last - STAGES : last;
                const uint32_t last_phase = last >= STAGES ? (phase ^ 1u) : phase;
                if (!mbar_wait(bar_empty + last_stage * 8, last_phase ^ 1u)) {
                    if (issuer) atomicCAS(p.status, 0, kStatusTimeoutProducer);
                    ok = false;
                    break;
                }
                const long long t1 = tr ? clock64() : 0;
                if (issuer) {
                    // weight tiles first: neighbouring K blocks of the same rows go out back to back
                    int s = stage, t = tile, k = kb, lsk = left_sk;
#pragma unroll
                    for (int i = 0; i < kBurst; ++i) {
                        if (i < g) {
                            mbar_arrive_expect_tx(bar_full + s * 8, Cfg::kStageBytes);
                            if (p.w_tile_major)
                                tma_load_2d<1, 1>(smem_base + Cfg::kOffW + s * Cfg::kWBytes, &tm_w, bar_full + s * 8, 0,
                                               (t * num_kb + k) * 128);
                            else
                                tma_load_2d<1, 1>(smem_base + Cfg::kOffW + s * Cfg::kWBytes, &tm_w, bar_full + s * 8, k * 128,
                                               t * 128);
                            tma_load_2d<1, 1>(smem_base + Cfg::kOffSfw + s * Cfg::kSfBytes, &tm_sfw, bar_full + s * 8, 0,
                                           t * p.w_sf_k_atoms + k * Cfg::kSfK);
                            if (++s == STAGES) s = 0;
                            advance(t, k, lsk);
                        }
                    }
                    // the activations (and their scales) may come from the previous kernel: wait for it
                    // once, after the first weight tiles are already on their way
                    if (!prior_done) {
                        pdl_wait_prior_grid();
                        prior_done = true;
                    }
                    s = stage; t = tile; k = kb; lsk = left_sk;
#pragma unroll
                    for (int i = 0; i < kBurst; ++i) {
                        if (i < g) {
                            const uint32_t full = bar_full + s * 8;
                            tma_load_2d<1, 2>(smem_base + Cfg::kOffX + s * Cfg::kXBytes, &tm_x, full, k * 128, 0);
                            tma_load_2d<1, 2>(smem_base + Cfg::kOffSfx + s * Cfg::kSfBytes, &tm_sfx, full, 0, k * Cfg::kSfK);
                            if (++s == STAGES) s = 0;
                            advance(t, k, lsk);
                        }
                    }
                    if (tr && rec < p.trace_cap) {
                        long long* r = p.trace + (0ll * p.trace_cap + rec) * 4;
                        r[0] = t0; r[1] = t1; r[2] = clock64(); r[3] = g;
                    }
                }
                ++rec;
                left -= g;
                stage += g;
                if (stage >= STAGES) { stage -= STAGES; phase ^= 1u; }
                for (int i = 0; i < g; ++i) advance(tile, kb, left_sk);
            }
            if (ok) {
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
        {
            constexpr bool kUe8m0 = (SF_VEC == 32);
            const bool issuer = elect_one_sync();
            int stage = 0;
            uint32_t phase = 0;
            int seg = 0;
            bool ok = true;
            const bool tr = (p.trace != nullptr) && (blockIdx.x == 0);
            int rec = 0;
            const int num_segs_whole = whole_tiles;
            long long u = u_begin;
            for (int done_whole = 0; (u < u_end || done_whole < num_segs_whole) && ok; ++seg) {
                // segment = K blocks [kb0, kb1) of one tile: first the stream-K range, then the whole tiles
                int kb0 = 0, kb1 = num_kb;
                if (u < u_end) {
                    kb0 = static_cast<int>(u % num_kb);
                    const long long left = u_end - u;
                    kb1 = (left < num_kb - kb0) ? kb0 + static_cast<int>(left) : num_kb;
                    u += kb1 - kb0;
                } else {
                    ++done_whole;
                }
                const int acc = seg % ACC;
                const uint32_t acc_phase = static_cast<uint32_t>(seg / ACC) & 1u;
                if (!mbar_wait(bar_tempty + acc * 8, acc_phase ^ 1u)) {
                    if (issuer) atomicCAS(p.status, 0, kStatusTimeoutMma);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * MP;
                for (int kb = kb0; kb < kb1; ++kb) {
                    const long long t0 = tr ? clock64() : 0;
                    if (!mbar_wait(bar_full + stage * 8, phase)) {
                        if (issuer) atomicCAS(p.status, 0, kStatusTimeoutMma);
                        ok = false;
                        break;
                    }
                    const long long t1 = tr ? clock64() : 0;
                    tcgen05_fence_after();
                    const uint64_t sfw_desc = make_desc_sf(smem_base + Cfg::kOffSfw + stage * Cfg::kSfBytes);
                    const uint64_t sfx_desc = make_desc_sf(smem_base + Cfg::kOffSfx + stage * Cfg::kSfBytes);
                    const uint64_t w_desc = make_desc_k_sw128(smem_base + Cfg::kOffW + stage * Cfg::kWBytes);
                    const uint64_t x_desc = make_desc_k_sw128(smem_base + Cfg::kOffX + stage * Cfg::kXBytes);
                    const uint32_t accum0 = (kb > kb0) ? 1u : 0u;
                    if (issuer) {
#pragma unroll
                        for (int j = 0; j < Cfg::kSfK; ++j) {
                            // descriptor start address is in 16-byte units: one 512-byte scale tile = 32
                            tmem_cp_sf<1>(tmem_base + Cfg::kTmemSfw + j * 4, sfw_desc + static_cast<uint64_t>(j * 32));
                            tmem_cp_sf<1>(tmem_base + Cfg::kTmemSfx + j * 4, sfx_desc + static_cast<uint64_t>(j * 32));
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            constexpr bool nv = (SF_VEC == 16);
                            const int sf_tile = nv ? j : (j >> 1);
                            const int sf_id = nv ? 0 : 2 * (j & 1);
                            const uint32_t idesc = make_idesc_fp4(128, MP, kUe8m0, sf_id);
                            mma_fp4_block_scaled<1, SF_VEC>(d_tmem, w_desc + static_cast<uint64_t>(j * 2),
                                                            x_desc + static_cast<uint64_t>(j * 2), idesc,
                                                            tmem_base + Cfg::kTmemSfw + sf_tile * 4,
                                                            tmem_base + Cfg::kTmemSfx + sf_tile * 4, (j > 0) ? 1u : accum0);
                        }
                        tcgen05_commit<1>(bar_empty + stage * 8);
                        if (tr && rec < p.trace_cap) {
                            long long* r = p.trace + (1ll * p.trace_cap + rec) * 4;
                            r[0] = t0; r[1] = t1; r[2] = clock64(); r[3] = kb;
                        }
                    }
                    ++rec;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok && issuer) tcgen05_commit<1>(bar_tfull + acc * 8);
                __syncwarp();
            }
        }
    } else {
        // --------------------------------------------------------------- epilogue
        const int quad = warp & 3;
        const int n_local = quad * 32 + lane;
        // everything this role reads (tensor scales) or writes (output, scratch) may be touched by the
        // previous kernel in the stream
        if (p.pdl) pdl_wait_prior_grid();
        float alpha = 1.0f;
        if (p.x_gs) alpha *= __ldcg(p.x_gs);
        if (p.w_gs) alpha *= __ldcg(p.w_gs);
        int seg = 0;
        bool ok = true;
        long long u = u_begin;
        for (int done_whole = 0; (u < u_end || done_whole < whole_tiles) && ok; ++seg) {
            int tile, kb0 = 0, kb1 = num_kb;
            if (u < u_end) {
                tile = static_cast<int>(u / num_kb);
                kb0 = static_cast<int>(u - static_cast<long long>(tile) * num_kb);
                const long long left = u_end - u;
                kb1 = (left < num_kb - kb0) ? kb0 + static_cast<int>(left) : num_kb;
                u += kb1 - kb0;
            } else {
                tile = first_whole + done_whole * static_cast<int>(gridDim.x);
                ++done_whole;
            }
            const int acc = seg % ACC;
            const uint32_t acc_phase = static_cast<uint32_t>(seg / ACC) & 1u;
            const bool tr = (p.trace != nullptr) && (blockIdx.x == 0) && (warp == 2) && (lane == 0) && (seg < p.trace_cap);
            const long long te0 = tr ? clock64() : 0;
            if (!mbar_wait(bar_tfull + acc * 8, acc_phase)) {
                if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
                ok = false;
                break;
            }
            const long long te1 = tr ? clock64() : 0;
            tcgen05_fence_after();
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * MP;
            uint32_t v[MP];
#pragma unroll
            for (int c = 0; c < MP / 16; ++c)
                tmem_ld_32x32b_x16(t_acc + c * 16, reinterpret_cast<uint32_t(&)[16]>(v[c * 16]));
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + acc * 8);

            const long long te2 = tr ? clock64() : 0;
            const int n = tile * 128 + n_local;
            const bool whole = (kb0 == 0 && kb1 == num_kb);
            // `v` ends up holding the complete fp32 sums of this thread's weight row when `final_here` is set:
            // at once for a whole tile, or after the last contributor has added up the partials.
            bool final_here = whole;
            if (!whole) {
                const int slot = (kb0 == 0) ? 1 : 0;
                float* mine = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (MP * 128);
#pragma unroll
                for (int m = 0; m < MP; ++m) __stcg(mine + m * 128 + n_local, __uint_as_float(v[m]));
                // Each warp owns 32 weight rows of the tile and settles them on its own
                // (counter per tile and warp quadrant), so no barrier between warps is needed.
                __threadfence();
                __syncwarp();
                int f = -1;
                if (lane == 0) {
                    const int c0 = skinny_cta_of(static_cast<long long>(tile) * num_kb, units, sk_ctas);
                    const int c1 = skinny_cta_of(static_cast<long long>(tile + 1) * num_kb - 1, units, sk_ctas);
                    const int old = atomicAdd(p.counters + tile * 4 + quad, 1);
                    if (old == c1 - c0) {
                        p.counters[tile * 4 + quad] = 0;
                        f = c0 | (c1 << 16);
                    }
                }
                f = __shfl_sync(0xffffffffu, f, 0);
                if (f >= 0) {
                    __threadfence();
                    const int c0 = f & 0xffff, c1 = f >> 16;
#pragma unroll
                    for (int m = 0; m < MP; ++m) v[m] = 0u;   // +0.0f
                    for (int c = c0; c <= c1; ++c) {
                        const float* src = p.partials + (static_cast<size_t>(c) * 2 + (c == c0 ? 1 : 0)) * (MP * 128);
#pragma unroll
                        for (int m = 0; m < MP; ++m) v[m] = __float_as_uint(__uint_as_float(v[m]) + __ldcg(src + m * 128 + n_local));
                    }
                    final_here = true;
                }
            }
            // One write-out for both cases, and the epilogue choice made outside the unrolled loops: the plain
            // path stays a compact run of multiply-convert-store (the unrolled code of this kernel is large enough
            // for instruction fetch to show up in a ~20 us kernel).
            if (final_here && n < p.n) {
                __nv_bfloat16* dst = p.d + n;
                if (p.bias == nullptr && p.act == kActNone) {
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < p.m) dst[static_cast<size_t>(m) * p.ldd] = __float2bfloat16_rn(__uint_as_float(v[m]) * alpha);
                } else {
                    const float b = (p.bias != nullptr) ? __bfloat162float(p.bias[n]) : 0.0f;
                    auto store_act = [&](auto act_tag) {
                        constexpr int ACT = decltype(act_tag)::value;
#pragma unroll
                        for (int m = 0; m < MP; ++m)
                            if (m < p.m)
                                dst[static_cast<size_t>(m) * p.ldd] = __float2bfloat16_rn(activate<ACT>(fmaf(__uint_as_float(v[m]), alpha, b)));
                    };
                    switch (p.act) {
                        case kActRelu: store_act(std::integral_constant<int, kActRelu>{}); break;
                        case kActGelu: store_act(std::integral_constant<int, kActGelu>{}); break;
                        case kActGeluTanh: store_act(std::integral_constant<int, kActGeluTanh>{}); break;
                        case kActSilu: store_act(std::integral_constant<int, kActSilu>{}); break;
                        default: store_act(std::integral_constant<int, kActNone>{}); break;
                    }
                }
            }
            if (tr) {
                long long* r = p.trace + (2ll * p.trace_cap + seg) * 4;
                r[0] = te0; r[1] = te1; r[2] = te2; r[3] = clock64();
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
}

}  // namespace avefp4
