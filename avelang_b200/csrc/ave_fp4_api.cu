// Host side of libavefp4: argument checks, tensor-map encoding, kernel selection and
// launch behind the C ABI declared in include/ave_fp4.h.
//
// Launch conventions follow the reference's NVIDIA backend
// (python/avelang/backends/nvidia/driver.py:284-311): raw device pointers, the
// caller's stream, no synchronisation, errors reported to the caller (there as a
// Python RuntimeError, here as a return code plus ave_fp4_last_error()).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/ave_fp4.h"
#include "gemm_fp4_skinny_sm100.cuh"
#include "gemm_fp4_sm100.cuh"
#include "quantize_fp4.cuh"

namespace {

using namespace avefp4;

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int fail_cuda(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof(g_err), "ave-lang Error [CUDA]: %s: %s", what, cudaGetErrorString(e));
    return static_cast<int>(e);
}

#define AVE_CUDA(call)                                         \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return fail_cuda(e__, #call);  \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxDevices = 64;

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    int* status = nullptr;
    long long* trace = nullptr;  // optional profiling buffer set by ave_fp4_set_trace
    int trace_cap = 0;
    // resident 256-thread blocks per SM of the streaming kernels: their grids are exactly one wave
    int occ_amax = 1;
    int occ_quant[2][2] = {{1, 1}, {1, 1}};   // [format][tiled]
    int occ_reduce = 1;
};

std::mutex g_mutex;
DeviceState g_dev[kMaxDevices];
EncodeTiledFn g_encode = nullptr;

// ----------------------------------------------------------------------------------
// Kernel table.  One entry per instantiation so that attributes are set once at init.
template <int CG, int BN, int VEC, int ST, int ACC>
cudaError_t prepare_gemm() {
    using Cfg = GemmConfig<CG, BN, VEC, ST, ACC>;
    cudaError_t e = cudaFuncSetAttribute(gemm_fp4_kernel<CG, BN, VEC, ST, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if constexpr (VEC != 0) {   // the dense bf16 operator has no fused epilogue
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_fp4_kernel<CG, BN, VEC, ST, ACC, kEpiBiasAct>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_fp4_kernel<CG, BN, VEC, ST, ACC, kEpiQuant>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::kSmemBytes);
        if (e == cudaSuccess && CG == 2 && BN == 256)   // K-sharded partial results: the 256x256 CTA-pair tile only
            e = cudaFuncSetAttribute(gemm_fp4_kernel<CG, BN, VEC, ST, ACC, kEpiPartial>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::kSmemBytes);
    }
    return e;
}

template <int MP, int VEC, int ST>
cudaError_t prepare_skinny() {
    using Cfg = SkinnyConfig<MP, VEC, ST>;
    return cudaFuncSetAttribute(gemm_fp4_skinny_kernel<MP, VEC, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg::kSmemBytes);
}

// Stage counts per tile shape (shared-memory budget 227 KB per CTA).
constexpr int kSt1N128 = 5, kSt1N256 = 3, kSt2N256 = 5, kSt2N128 = 6, kSt2N192 = 5;
constexpr int kStDense2N256 = 6, kStDense1N128 = 6;   // dense bf16: 32 KB per stage
constexpr int kStSkinny16 = 8, kStSkinny32 = 8, kStSkinny64 = 7;

// Pipeline-depth tuning aid: the NVFP4 256x256 CTA-pair tile with 3 and 4 stages (plain epilogue only), chosen with
// AVE_FP4_GEMM_STAGES; the depth used otherwise is kSt2N256.
int tuning_stages_2n256() {
    static const int v = [] { const char* e = getenv("AVE_FP4_GEMM_STAGES"); return e ? atoi(e) : 0; }();
    return v;
}

template <int ST>
cudaError_t prepare_gemm_plain_2n256() {
    return cudaFuncSetAttribute(gemm_fp4_kernel<2, 256, 16, ST, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GemmConfig<2, 256, 16, ST, 1>::kSmemBytes);
}

cudaError_t prepare_all() {
    cudaError_t e;
#define PREP(x) if ((e = (x)) != cudaSuccess) return e;
    PREP((prepare_gemm_plain_2n256<3>()));
    PREP((prepare_gemm_plain_2n256<4>()));
    PREP((prepare_gemm<1, 128, 16, kSt1N128, 2>()));
    PREP((prepare_gemm<1, 128, 32, kSt1N128, 2>()));
    PREP((prepare_gemm<1, 256, 16, kSt1N256, 1>()));
    PREP((prepare_gemm<1, 256, 32, kSt1N256, 1>()));
    PREP((prepare_gemm<2, 256, 16, kSt2N256, 1>()));
    PREP((prepare_gemm<2, 256, 32, kSt2N256, 1>()));
    PREP((prepare_gemm<2, 192, 16, kSt2N192, 2>()));
    PREP((prepare_gemm<2, 192, 32, kSt2N192, 2>()));
    PREP((prepare_gemm<2, 128, 16, kSt2N128, 2>()));
    PREP((prepare_gemm<2, 128, 32, kSt2N128, 2>()));
    PREP((prepare_gemm<2, 256, 0, kStDense2N256, 2>()));
    PREP((prepare_gemm<1, 128, 0, kStDense1N128, 2>()));
    PREP((prepare_skinny<16, 16, kStSkinny16>()));
    PREP((prepare_skinny<16, 32, kStSkinny16>()));
    PREP((prepare_skinny<32, 16, kStSkinny32>()));
    PREP((prepare_skinny<32, 32, kStSkinny32>()));
    PREP((prepare_skinny<64, 16, kStSkinny64>()));
    PREP((prepare_skinny<64, 32, kStSkinny64>()));
#undef PREP
    return cudaSuccess;
}

int current_state(DeviceState** out) {
    int dev = -1;
    AVE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices || !g_dev[dev].ready)
        return fail(-AVE_FP4_ERR_NOT_INIT, "ave_fp4_init(%d) has not been called for the current device", dev);
    *out = &g_dev[dev];
    return 0;
}

// ----------------------------------------------------------------------------------
// Tensor maps.
// L2 fetch granularity of TMA loads (256 bytes unless AVE_FP4_L2_PROMOTION = 64 | 128 | 0 overrides it for tuning).
CUtensorMapL2promotion l2_promotion() {
    static const CUtensorMapL2promotion chosen = [] {
        if (const char* e = getenv("AVE_FP4_L2_PROMOTION")) {
            const int v = atoi(e);
            if (v == 0) return CU_TENSOR_MAP_L2_PROMOTION_NONE;
            if (v == 64) return CU_TENSOR_MAP_L2_PROMOTION_L2_64B;
            if (v == 128) return CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
        }
        return CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    }();
    return chosen;
}

// A tensor map depends only on the address and the geometry, never on the memory's contents, and a serving loop
// calls with the same few operands over and over (the weights of each layer, a handful of activation buffers).
// Each host thread therefore keeps the maps it encoded last in a small direct-mapped cache: a hit replaces the
// driver call (four per GEMM launch) by a 128-byte copy.
struct TensorMapKey {
    const void* base;
    uint64_t inner, outer, stride;
    uint32_t box_inner, box_outer;
    int dt, swz, promo;
    bool operator==(const TensorMapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride && box_inner == o.box_inner &&
               box_outer == o.box_outer && dt == o.dt && swz == o.swz && promo == o.promo;
    }
};
struct TensorMapSlot {
    bool valid = false;
    TensorMapKey key{};
    CUtensorMap map;
};
constexpr int kTensorMapSlots = 256;
thread_local TensorMapSlot g_tm_cache[kTensorMapSlots];

int encode_2d(CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
              uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz,
              const char* what) {
    const CUtensorMapL2promotion promo = l2_promotion();
    const TensorMapKey key{base, inner, outer, outer_stride_bytes, box_inner, box_outer, static_cast<int>(dt),
                           static_cast<int>(swz), static_cast<int>(promo)};
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h = (h ^ (h >> 17) ^ (outer * 0x9E3779B97F4A7C15ull) ^ (static_cast<uint64_t>(box_outer) << 7) ^ inner) * 0xD6E8FEB86659FD93ull;
    TensorMapSlot& slot = g_tm_cache[(h >> 40) % kTensorMapSlots];
    if (slot.valid && slot.key == key) {
        memcpy(tm, &slot.map, sizeof(CUtensorMap));
        return 0;
    }
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {outer_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swz, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(-AVE_FP4_ERR_ARG,
                    "tensor map for %s rejected (CUresult %d): base %p dims (%llu,%llu) stride %llu box (%u,%u)", what,
                    static_cast<int>(r), base, static_cast<unsigned long long>(inner),
                    static_cast<unsigned long long>(outer), static_cast<unsigned long long>(outer_stride_bytes),
                    box_inner, box_outer);
    slot.key = key;
    memcpy(&slot.map, tm, sizeof(CUtensorMap));
    slot.valid = true;
    return 0;
}

// packed E2M1 operand (rows, k/2 bytes): box = 128 bytes x box_rows, 128-byte swizzle
int encode_packed(CUtensorMap* tm, const void* p, int64_t rows, int64_t k, uint32_t box_rows, const char* what) {
    return encode_2d(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, p, static_cast<uint64_t>(k / 2), static_cast<uint64_t>(rows),
                     static_cast<uint64_t>(k / 2), 128, box_rows, CU_TENSOR_MAP_SWIZZLE_128B, what);
}

// tiled scale factors: one 512-byte tile per row of a (tiles, 128 x u32) matrix
int encode_sf(CUtensorMap* tm, const void* p, int64_t rows, int64_t k, int vec, uint32_t box_tiles, const char* what) {
    const int64_t k_atoms = (k / vec + 3) / 4;
    const int64_t tiles = ((rows + 127) / 128) * k_atoms;
    return encode_2d(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, p, 128, static_cast<uint64_t>(tiles), 512, 128, box_tiles,
                     CU_TENSOR_MAP_SWIZZLE_NONE, what);
}

constexpr int64_t kFusedSmallElems = 1 << 20;  // up to here amax + quantise run as one 8-CTA cluster launch

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The tiled kernels are launched with programmatic stream serialisation (their launch and set-up run under the tail of
// the previous kernel in the stream; they wait for it on the device before touching memory): +2 % on back-to-back
// 8192^3 launches.  The profiling stamps want launches that do not overlap; AVE_FP4_GEMM_PDL=0 switches it off for A/B timing.
// Tile rows per band of the persistent schedule (decode_tile).  FP4: 16 (at 8192^3 the CTA-pair tiles run 2 % faster than
// with 8, config 3's 57344 columns 6.7 %, 16384^3 1.9 %; 32 and more lose 10-25 % at 16384^3); dense bf16, whose operand
// rows are four times as long, and the K-sharded schedule keep 8.  AVE_FP4_GEMM_BAND overrides (tuning aid).
int gemm_band(int by_default) {
    static const int v = [] { const char* e = getenv("AVE_FP4_GEMM_BAND"); return e ? atoi(e) : 0; }();
    return v > 0 ? v : by_default;
}

int tiled_pdl(const DeviceState& ds) {
    static const bool pdl_off = [] { const char* e = getenv("AVE_FP4_GEMM_PDL"); return e != nullptr && e[0] == '0'; }();
    return (ds.trace == nullptr && !pdl_off) ? 1 : 0;
}

// ----------------------------------------------------------------------------------
// Where a quantised result goes when it is one column block of a wider operand that all ranks gather
// (ave_fp4_gemm_allgather_quantized); null = the result is an operand of its own.
struct QuantGather {
    int64_t n_total;            // columns of the gathered operand
    int64_t col0;               // first column of this rank's block in it
    void* const* peer_packed;   // the operand's packed bytes / scales in the other ranks' memory (base addresses)
    void* const* peer_sf;
    int n_peers;
};

template <int CG, int BN, int VEC, int ST, int ACC, bool PLAIN_ONLY = false>
int launch_gemm(const DeviceState& ds, const void* a, const void* sfa, const float* ags, const void* b, const void* sfb,
                const float* bgs, void* d, int64_t m, int64_t n, int64_t k, int64_t ldd, cudaStream_t stream,
                void* const* peers = nullptr, int n_peers = 0, const ave_fp4_epilogue* epi = nullptr,
                void* const* slabs = nullptr, int rs_world = 0, int first_owner = 0, const QuantGather* qg = nullptr) {
    using Cfg = GemmConfig<CG, BN, VEC, ST, ACC>;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
    int rc;
    if ((rc = encode_packed(&tm_a, a, m, k, 128, "A"))) return rc;
    if ((rc = encode_packed(&tm_b, b, n, k, Cfg::kBnCta, "B"))) return rc;
    if ((rc = encode_sf(&tm_sfa, sfa, m, k, VEC, Cfg::kSfK, "A scales"))) return rc;
    if ((rc = encode_sf(&tm_sfb, sfb, n, k, VEC, Cfg::kSfK, "B scales"))) return rc;

    GemmParams p;
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.tiles_m = static_cast<int>((m + 128 * CG - 1) / (128 * CG));
    p.tiles_n = static_cast<int>((n + BN - 1) / BN);
    p.sf_k_atoms = static_cast<int>((k / VEC + 3) / 4);
    p.a_gs = ags;
    p.b_gs = bgs;
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = static_cast<int>(ldd);
    p.n_peers = n_peers;
    for (int i = 0; i < 7; ++i) p.peer_d[i] = (i < n_peers) ? static_cast<__nv_bfloat16*>(peers[i]) : nullptr;
    p.status = ds.status;
    p.trace = ds.trace;
    p.trace_cap = ds.trace_cap;
    p.bias = epi ? static_cast<const __nv_bfloat16*>(epi->bias_bf16) : nullptr;
    p.act = epi ? epi->activation : 0;
    const bool quant = epi && epi->quantize_out;
    p.q_packed = quant ? static_cast<uint8_t*>(epi->q_packed) : nullptr;
    p.q_sf = quant ? static_cast<uint8_t*>(epi->q_scales) : nullptr;
    p.q_gs = quant ? static_cast<const float*>(epi->q_global_scale) : nullptr;
    p.q_tiled = (quant && epi->q_sf_layout == AVE_FP4_SF_TILED) ? 1 : 0;
    {
        const int64_t blk = (VEC == 0) ? 16 : VEC;
        const int64_t q_n = qg ? qg->n_total : n;
        const int64_t q_c0 = qg ? qg->col0 : 0;
        p.q_ld = static_cast<int>(q_n / 2);
        p.q_sf_cols = static_cast<int>(q_n / blk);
        p.q_sf_col0 = static_cast<int>(q_c0 / blk);
        if (quant) p.q_packed += q_c0 / 2;      // this rank's column block; the scale offset is applied per scale column
        p.q_n_peers = (quant && qg) ? qg->n_peers : 0;
        for (int i = 0; i < 7; ++i) {
            p.q_peer_packed[i] = (i < p.q_n_peers) ? static_cast<uint8_t*>(qg->peer_packed[i]) + q_c0 / 2 : nullptr;
            p.q_peer_sf[i] = (i < p.q_n_peers) ? static_cast<uint8_t*>(qg->peer_sf[i]) : nullptr;
        }
    }
    p.pdl = tiled_pdl(ds);
    p.band = gemm_band(rs_world > 0 ? 8 : 16);
    p.rs_world = rs_world;
    p.rs_rows = rs_world > 0 ? static_cast<int>(m / rs_world) : 0;
    for (int i = 0; i < 8; ++i) p.rs_dst[i] = (i < rs_world) ? static_cast<float*>(slabs[i]) : nullptr;
    // K-sharded partials: visit the owners' tile rows in turn, starting with first_owner; when the owners' row ranges are not
    // whole tile rows, only start the schedule at the tile row that holds first_owner's first row
    p.tm_perm_w = 0;
    p.tm_first = 0;
    if (rs_world > 1) {
        if (p.tiles_m % rs_world == 0 && p.rs_rows % (128 * CG) == 0) {
            p.tm_perm_w = rs_world;
            p.tm_first = first_owner;
        } else {
            p.tm_first = static_cast<int>((static_cast<int64_t>(first_owner) * p.rs_rows / (128 * CG)) % p.tiles_m);
        }
    }

    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    long long clusters = ds.sm_count / CG;
    if (tiles < clusters) clusters = tiles;

    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * CG), 1, 1);
    cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 2 : 1;
    if constexpr (PLAIN_ONLY) {
        if (rs_world > 0 || quant || p.bias != nullptr || p.act != 0)
            return fail(-AVE_FP4_ERR_ARG, "this tuning instantiation has the plain epilogue only");
        AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<CG, BN, VEC, ST, ACC>, tm_a, tm_b, tm_sfa, tm_sfb, p));
    } else if (rs_world > 0) {
        if constexpr (CG == 2 && BN == 256)
            AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<CG, BN, VEC, ST, ACC, kEpiPartial>, tm_a, tm_b, tm_sfa, tm_sfb, p));
        else
            return fail(-AVE_FP4_ERR_ARG, "partial results are served by the 256x256 CTA-pair kernel only");
    } else if (quant)
        AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<CG, BN, VEC, ST, ACC, kEpiQuant>, tm_a, tm_b, tm_sfa, tm_sfb, p));
    else if (p.bias != nullptr || p.act != 0)
        AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<CG, BN, VEC, ST, ACC, kEpiBiasAct>, tm_a, tm_b, tm_sfa, tm_sfb, p));
    else
        AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<CG, BN, VEC, ST, ACC>, tm_a, tm_b, tm_sfa, tm_sfb, p));
    return 0;
}

// Dense bf16 operands (the reference operator's own data type): same kernel, no scale factors.
template <int CG, int BN, int ST, int ACC>
int launch_dense(const DeviceState& ds, const void* a, const void* b, void* d, int64_t m, int64_t n, int64_t k, int64_t ldd,
                 cudaStream_t stream) {
    using Cfg = GemmConfig<CG, BN, 0, ST, ACC>;
    CUtensorMap tm_a, tm_b;
    int rc;
    // bf16 rows seen as bytes: K * 2 bytes per row, 128-byte (64-element) boxes, 128-byte swizzle
    if ((rc = encode_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a, static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(m),
                        static_cast<uint64_t>(k) * 2, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B, "A")))
        return rc;
    if ((rc = encode_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, b, static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(n),
                        static_cast<uint64_t>(k) * 2, 128, Cfg::kBnCta, CU_TENSOR_MAP_SWIZZLE_128B, "B")))
        return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.tiles_m = static_cast<int>((m + 128 * CG - 1) / (128 * CG));
    p.tiles_n = static_cast<int>((n + BN - 1) / BN);
    p.d = static_cast<__nv_bfloat16*>(d);
    p.ldd = static_cast<int>(ldd);
    p.status = ds.status;
    p.trace = ds.trace;
    p.trace_cap = ds.trace_cap;
    p.pdl = tiled_pdl(ds);
    p.band = gemm_band(8);
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
    long long clusters = ds.sm_count / CG;
    if (tiles < clusters) clusters = tiles;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * CG), 1, 1);
    cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = p.pdl ? 2 : 1;
    // the scale-factor tensor maps are unused in dense mode; pass copies of the operand maps
    AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_kernel<CG, BN, 0, ST, ACC>, tm_a, tm_b, tm_a, tm_b, p));
    return 0;
}

// Load-burst size of the decode kernel: 4 K blocks (512 contiguous bytes per weight row and DRAM page visit), also with
// the 7-stage ring of the 64-row form (27.0 us with 4, 27.8 with 3 at 64 x 28672 x 8192); AVE_FP4_SKINNY_BURST overrides it.
int skinny_burst(int stages) {
    static const int env_burst = [] { const char* e = getenv("AVE_FP4_SKINNY_BURST"); return e ? atoi(e) : 4; }();
    int b = env_burst;
    const int cap = stages < 8 ? stages : 8;
    if (b < 1) b = 1;
    if (b > cap) b = cap;
    return b;
}

int skinny_mp(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : 64; }

// Scratch of the decode kernel: [header 256 B][arrival counters][stream-K partials].  Everything that has to be zero
// between launches (the header words and the counters) sits in a prefix whose size does not depend on the shape
// (up to 4096 weight tiles, N = 524288), so one zero-initialised buffer can serve calls of different shapes one
// after the other: what a call leaves behind in the partials never lands where another shape keeps a counter.
constexpr int64_t kSkinnyHdrBytes = 256;
constexpr int64_t kSkinnyCounterRegion = 64 * 1024;

int64_t skinny_counter_bytes(int64_t n) {
    const int64_t tiles_n = (n + 127) / 128;
    return ((tiles_n * 4 * 4 + 255) / 256) * 256;
}

int64_t skinny_counter_region(int64_t n) {
    const int64_t used = skinny_counter_bytes(n);
    return used > kSkinnyCounterRegion ? used : kSkinnyCounterRegion;
}

int64_t skinny_workspace_bytes(int64_t m, int64_t n, int sm_count) {
    return kSkinnyHdrBytes + skinny_counter_region(n) + static_cast<int64_t>(sm_count) * 2 * skinny_mp(m) * 128 * 4;
}

// Scratch of ave_fp4_linear_decode: the decode kernel's scratch, then the quantised activations the quantise kernel
// writes and the GEMM reads (packed bytes of up to MP rows and their tiled scales), then two floats (tensor scale, amax).
struct FusedScratch {
    int64_t packed, sf, gs, total;
};

FusedScratch fused_scratch_layout(int64_t m, int64_t n, int64_t k, int vec, int sm_count) {
    auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
    FusedScratch f;
    f.packed = up(skinny_workspace_bytes(m, n, sm_count));
    f.sf = f.packed + up(static_cast<int64_t>(skinny_mp(m)) * (k / 2));
    f.gs = f.sf + up(((k / vec + 3) / 4) * 512);
    f.total = f.gs + 256;
    return f;
}

template <int MP, int VEC, int ST>
int launch_skinny(const DeviceState& ds, const void* x, const void* sfx, const float* xgs, const void* w, const void* sfw,
                  const float* wgs, void* d, int64_t m, int64_t n, int64_t k, int64_t ldd, void* workspace,
                  bool w_tile_major, cudaStream_t stream, bool pdl = false, const ave_fp4_epilogue* epi = nullptr) {
    using Cfg = SkinnyConfig<MP, VEC, ST>;
    CUtensorMap tm_w, tm_x, tm_sfw, tm_sfx;
    int rc;
    if (w_tile_major) {
        // tile-major weights: every 128-byte row piece of every 16 KB tile is one row of a (tiles*128, 128) matrix
        const uint64_t tile_rows = static_cast<uint64_t>((n + 127) / 128) * static_cast<uint64_t>((k + 255) / 256) * 128;
        if ((rc = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, 128, tile_rows, 128, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B,
                            "B (tile-major)")))
            return rc;
    } else if ((rc = encode_packed(&tm_w, w, n, k, 128, "B"))) {
        return rc;
    }
    if ((rc = encode_packed(&tm_x, x, m, k, MP, "A"))) return rc;
    if ((rc = encode_sf(&tm_sfw, sfw, n, k, VEC, Cfg::kSfK, "B scales"))) return rc;
    if ((rc = encode_sf(&tm_sfx, sfx, m, k, VEC, Cfg::kSfK, "A scales"))) return rc;

    SkinnyParams p;
    p.m = static_cast<int>(m);
    p.n = static_cast<int>(n);
    p.k = static_cast<int>(k);
    p.tiles_n = static_cast<int>((n + 127) / 128);
    p.w_sf_k_atoms = static_cast<int>((k / VEC + 3) / 4);
    p.ldd = static_cast<int>(ldd);
    p.w_tile_major = w_tile_major ? 1 : 0;
    p.pdl = pdl ? 1 : 0;
    p.burst = skinny_burst(ST);
    // AVE_FP4_SKINNY_STREAMK=0: whole tiles only (tuning aid: the schedule the two-phase stream-K split is measured against)
    static const bool no_streamk = [] { const char* e = getenv("AVE_FP4_SKINNY_STREAMK"); return e != nullptr && e[0] == '0'; }();
    p.no_streamk = no_streamk ? 1 : 0;
    p.x_gs = xgs;
    p.w_gs = wgs;
    p.d = static_cast<__nv_bfloat16*>(d);
    char* ws = static_cast<char*>(workspace);
    p.counters = reinterpret_cast<int*>(ws + kSkinnyHdrBytes);
    p.partials = reinterpret_cast<float*>(ws + kSkinnyHdrBytes + skinny_counter_region(n));
    p.status = ds.status;
    p.trace = ds.trace;
    p.trace_cap = ds.trace_cap;
    p.bias = epi ? static_cast<const __nv_bfloat16*>(epi->bias_bf16) : nullptr;
    p.act = epi ? epi->activation : 0;

    const long long units = no_streamk ? static_cast<long long>(p.tiles_n) : static_cast<long long>(p.tiles_n) * ((k + 255) / 256);
    long long grid = ds.sm_count;
    if (units < grid) grid = units;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    AVE_CUDA(cudaLaunchKernelEx(&cfg, gemm_fp4_skinny_kernel<MP, VEC, ST>, tm_w, tm_x, tm_sfw, tm_sfx, p));
    return 0;
}

int resolve_variant(int variant, int64_t m, int64_t n) {
    variant &= ~AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS;
    if (variant == AVE_FP4_GEMM_SKINNY_TILED_W) return AVE_FP4_GEMM_SKINNY;
    if (variant != AVE_FP4_GEMM_AUTO) return variant;
    // Decode kernel up to 32 rows.  From 33 rows on the 128x128 tiles are as fast or faster even for weight-streaming
    // shapes (measured at 64 rows: 28.1 vs 30.9 us for 28672 x 8192, 13.7 vs 20.8 us for 8192 x 8192): the stream-K
    // partial sums grow with the row count (64 rows: 32 KB per partial tile) while a 128-row tile costs the same for any M.
    if (m <= 32) return AVE_FP4_GEMM_SKINNY;
    // Tiled kernels: estimate the time of each tile shape as (waves of tiles over the SMs) x (tile work) /
    // (how well that shape feeds the tensor pipe, measured at 8192^3), and take the smallest.  Large problems
    // get 256x256 CTA-pair tiles; problems with few tiles get smaller tiles so that more SMs have work.
    // eff = TFLOP/s of the shape relative to the 256x256 CTA-pair tile, measured at 8192^3 with every tile shape
    // (5783 / 5368 / 4951 / 4826 / 4394 TFLOP/s; tensor pipe active 85 / 79 / 72 / 69 / 61 %; the same order and
    // ratios at 8192 x 7168 x 8192).
    struct Cand { int variant; int cta_m, bn, group; double eff; };
    static const Cand cands[] = {
        {AVE_FP4_GEMM_2CTA_N256, 256, 256, 2, 1.00},
        {AVE_FP4_GEMM_2CTA_N192, 256, 192, 2, 0.93},
        {AVE_FP4_GEMM_2CTA_N128, 256, 128, 2, 0.86},
        {AVE_FP4_GEMM_1CTA_N256, 128, 256, 1, 0.83},
        {AVE_FP4_GEMM_1CTA_N128, 128, 128, 1, 0.76},
    };
    int sms = 148;
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_dev[dev].ready) sms = g_dev[dev].sm_count;
    int best = AVE_FP4_GEMM_2CTA_N256;
    double best_t = 0.0;
    for (const Cand& c : cands) {
        const double tiles = static_cast<double>((m + c.cta_m - 1) / c.cta_m) * static_cast<double>((n + c.bn - 1) / c.bn);
        const double slots = static_cast<double>(sms / c.group);
        const double waves = static_cast<double>(static_cast<long long>((tiles + slots - 1) / slots));
        const double t = waves * (static_cast<double>(c.cta_m) * c.bn / c.group) / c.eff;   // per-SM work per wave
        if (best_t == 0.0 || t < best_t) {
            best_t = t;
            best = c.variant;
        }
    }
    return best;
}

// ------------------------------------------------------------------------------------
// Decode GEMM for callers that cannot allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc around a GEMM: a plugin that runs inside
// another runtime's memory pool has no allocator of its own to ask, and a serving loop that
// must never stall cannot afford the implicit device-wide synchronisation cudaMalloc/cudaFree
// may cause.  For them the stream-K scratch of the skinny kernel lives in this fixed array,
// which every GPU that loads the library holds (about 2.56 MiB) until the process exits.
constexpr int kNoAllocMaxM = 16;          // one MMA-N step of activation rows
constexpr int kNoAllocMaxN = 65536;       // 512 weight tiles
constexpr int kNoAllocMaxCtas = 160;      // persistent CTAs (one per SM)
constexpr size_t kNoAllocCounterBytes = kSkinnyHdrBytes + kSkinnyCounterRegion;                    // header + counters, 64.25 KiB
constexpr size_t kNoAllocPartialBytes = static_cast<size_t>(kNoAllocMaxCtas) * 2 * 16 * 128 * 4;  // 2.5 MiB
static_assert((kNoAllocMaxN / 128) * 4 * sizeof(int) <= static_cast<size_t>(kSkinnyCounterRegion), "counters of the largest N must fit");
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocCounterBytes + kNoAllocPartialBytes];

// Device address of the array per device.  The array's name is only a host-side handle for the
// symbol, so the address the kernel needs is looked up with cudaGetSymbolAddress, once per
// device, while that device is current.
void* g_noalloc_ptr[kMaxDevices] = {};

int noalloc_scratch_for_current_device(void** out) {
    int dev = -1;
    AVE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(-AVE_FP4_ERR_ARG, "device %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        AVE_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        if (ptr == nullptr) return fail(-AVE_FP4_ERR_DEVICE, "cudaGetSymbolAddress returned a null scratch address");
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int ave_fp4_gemm_decode_noalloc(const void* a_packed, const void* a_scales, const void* a_global_scale,
                                           const void* b_packed, const void* b_scales, const void* b_global_scale,
                                           void* d_bf16, int64_t m, int64_t n, int64_t k, int64_t ldd, int fmt,
                                           void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (fmt != AVE_FP4_FMT_NVFP4 && fmt != AVE_FP4_FMT_MXFP4) return fail(-AVE_FP4_ERR_ARG, "unknown format %d", fmt);
    if (m < 0 || n < 0 || m > kNoAllocMaxM || n > kNoAllocMaxN)
        return fail(-AVE_FP4_ERR_ARG,
                    "ave_fp4_gemm_decode_noalloc: the built-in scratch serves M <= %d and N <= %d, got M = %lld, N = %lld; "
                    "use ave_fp4_gemm with a caller-provided workspace for larger shapes",
                    kNoAllocMaxM, kNoAllocMaxN, static_cast<long long>(m), static_cast<long long>(n));
    if (ds->sm_count > kNoAllocMaxCtas)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_decode_noalloc: the built-in scratch serves at most %d SMs, this device has %d",
                    kNoAllocMaxCtas, ds->sm_count);
    if (m == 0 || n == 0) return 0;
    if (k <= 0 || k % 32 != 0 || k > 0x7fffffff)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_decode_noalloc: K must be a positive multiple of 32, got %lld", static_cast<long long>(k));
    if (n % 8 != 0 || ldd < n || ldd % 8 != 0)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_decode_noalloc: N and ldd must be multiples of 8 and ldd >= N");
    if (!a_packed || !a_scales || !b_packed || !b_scales || !d_bf16 || !aligned16(a_packed) || !aligned16(a_scales) ||
        !aligned16(b_packed) || !aligned16(b_scales) || !aligned16(d_bf16))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_decode_noalloc: null or misaligned (16-byte) pointer");
    void* scratch = nullptr;
    if ((rc = noalloc_scratch_for_current_device(&scratch))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left: the arrival counters must start at zero.
    AVE_CUDA(cudaMemsetAsync(scratch, 0, kSkinnyHdrBytes + skinny_counter_bytes(n), s));
    const float* ags = static_cast<const float*>(a_global_scale);
    const float* bgs = static_cast<const float*>(b_global_scale);
    if (fmt == AVE_FP4_FMT_NVFP4)
        return launch_skinny<16, 16, kStSkinny16>(*ds, a_packed, a_scales, ags, b_packed, b_scales, bgs, d_bf16, m, n, k, ldd,
                                                  scratch, false, s);
    return launch_skinny<16, 32, kStSkinny16>(*ds, a_packed, a_scales, ags, b_packed, b_scales, bgs, d_bf16, m, n, k, ldd,
                                              scratch, false, s);
}

// ====================================================================================
extern "C" {

const char* ave_fp4_last_error(void) { return g_err; }

int ave_fp4_init(int device) {
    if (device < 0 || device >= kMaxDevices) return fail(-AVE_FP4_ERR_ARG, "device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_dev[device].ready) return 0;
    int prev = -1;
    AVE_CUDA(cudaGetDevice(&prev));
    // whatever happens below, the caller gets its current device back, and a status word that was
    // allocated but not handed over is freed
    struct Restore {
        int prev;
        int* status;
        ~Restore() {
            if (status != nullptr) cudaFree(status);
            cudaSetDevice(prev);
        }
    } restore{prev, nullptr};
    AVE_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    AVE_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(-AVE_FP4_ERR_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                    prop.minor);
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        AVE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (fn == nullptr || q != cudaDriverEntryPointSuccess)
            return fail(-AVE_FP4_ERR_DEVICE, "driver does not export cuTensorMapEncodeTiled");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    AVE_CUDA(prepare_all());
    AVE_CUDA(cudaMalloc(&restore.status, sizeof(int)));
    AVE_CUDA(cudaMemset(restore.status, 0, sizeof(int)));
    g_dev[device].status = restore.status;
    restore.status = nullptr;
    g_dev[device].sm_count = prop.multiProcessorCount;
    {
        DeviceState& d = g_dev[device];
        auto occ = [](auto kernel, int threads = 256) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, 0) != cudaSuccess || n < 1) n = 1;
            return n;
        };
        d.occ_amax = occ(amax_bf16_kernel);
        d.occ_quant[0][0] = occ(quantize_fp4_kernel<kFmtNvfp4, false>, kQuantThreads);
        d.occ_quant[0][1] = occ(quantize_fp4_kernel<kFmtNvfp4, true>, kQuantThreads);
        d.occ_quant[1][0] = occ(quantize_fp4_kernel<kFmtMxfp4, false>, kQuantThreads);
        d.occ_quant[1][1] = occ(quantize_fp4_kernel<kFmtMxfp4, true>, kQuantThreads);
        d.occ_reduce = occ(reduce_partials_kernel);
    }
    g_dev[device].ready = true;
    return 0;
}

int ave_fp4_sm_count(void) {
    DeviceState* ds = nullptr;
    if (current_state(&ds)) return 0;
    return ds->sm_count;
}

int64_t ave_fp4_sf_bytes(int64_t rows, int64_t k, int fmt, int sf_layout) {
    const int64_t blk = (fmt == AVE_FP4_FMT_NVFP4) ? 16 : 32;
    const int64_t cols = k / blk;
    if (sf_layout == AVE_FP4_SF_ROW_MAJOR) return rows * cols;
    return ((rows + 127) / 128) * ((cols + 3) / 4) * 512;
}

int64_t ave_fp4_workspace_bytes(int64_t m, int64_t n, int64_t k, int fmt, int variant, int device) {
    (void)k;
    (void)fmt;
    if (resolve_variant(variant, m, n) != AVE_FP4_GEMM_SKINNY) return 0;
    if (device < 0 || device >= kMaxDevices || !g_dev[device].ready) return -AVE_FP4_ERR_NOT_INIT;
    return skinny_workspace_bytes(m, n, g_dev[device].sm_count);
}

int ave_fp4_amax(const void* x_bf16, int64_t rows, int64_t k, int64_t ldx, void* amax_f32, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (!x_bf16 || !amax_f32 || rows < 0 || k < 0 || k % 8 != 0 || ldx % 8 != 0 || !aligned16(x_bf16))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_amax: need k %% 8 == 0, ldx %% 8 == 0 and a 16-byte aligned input");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    AVE_CUDA(cudaMemsetAsync(amax_f32, 0, 4, s));
    const long long groups = rows * (k / 8);
    if (groups == 0) return 0;
    long long blocks = (groups + 255) / 256;
    const long long cap = static_cast<long long>(ds->sm_count) * ds->occ_amax;   // one full wave
    if (blocks > cap) blocks = cap;
    amax_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x_bf16), rows, k, ldx,
                                                                   static_cast<unsigned int*>(amax_f32));
    AVE_CUDA(cudaGetLastError());
    return 0;
}

int ave_fp4_quantize(const void* x_bf16, int64_t rows, int64_t k, int64_t ldx, int fmt, const void* amax_f32,
                     void* global_scale, void* packed, void* scales, int sf_layout, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (fmt != AVE_FP4_FMT_NVFP4 && fmt != AVE_FP4_FMT_MXFP4) return fail(-AVE_FP4_ERR_ARG, "unknown format %d", fmt);
    if (sf_layout != AVE_FP4_SF_ROW_MAJOR && sf_layout != AVE_FP4_SF_TILED)
        return fail(-AVE_FP4_ERR_ARG, "unknown scale layout %d", sf_layout);
    if (rows < 0 || k < 0 || k % 32 != 0 || ldx % 8 != 0 || ldx < k)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize: need k %% 32 == 0 and ldx %% 8 == 0, ldx >= k (k=%lld ldx=%lld)",
                    static_cast<long long>(k), static_cast<long long>(ldx));
    if (rows == 0 || k == 0) return 0;
    if (!x_bf16 || !packed || !scales || !aligned16(x_bf16) || !aligned16(packed))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize: null or misaligned pointer");
    if (fmt == AVE_FP4_FMT_NVFP4 && !global_scale)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize: NVFP4 needs a global_scale pointer");
    if (sf_layout == AVE_FP4_SF_TILED && (reinterpret_cast<uintptr_t>(scales) & 3u))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize: tiled scales must be 4-byte aligned");
    if (reinterpret_cast<uintptr_t>(scales) & 1u) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize: scales must be 2-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool tiled = (sf_layout == AVE_FP4_SF_TILED);
    const long long rows_pad = tiled ? ((rows + 127) / 128) * 128 : rows;
    const long long items = rows_pad * ((k + 1023) / 1024);  // one warp step each
    constexpr int kWarps = kQuantThreads / 32;
    long long blocks = (items + kWarps - 1) / kWarps;
    const long long cap = static_cast<long long>(ds->sm_count) * ds->occ_quant[fmt == AVE_FP4_FMT_NVFP4 ? 0 : 1][tiled ? 1 : 0];
    if (blocks > cap) blocks = cap;   // one full wave of resident blocks; each walks the items with a grid stride
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(x_bf16);
    const unsigned int* amax = static_cast<const unsigned int*>(amax_f32);
    float* gs = static_cast<float*>(global_scale);
    uint8_t* pk = static_cast<uint8_t*>(packed);
    uint8_t* sf = static_cast<uint8_t*>(scales);
    // launched with programmatic stream serialisation: the launch overlaps the tail of the previous kernel (the amax
    // pass, or the GEMM before it); the kernel waits for that kernel on the device before its first access
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
    cfg.blockDim = dim3(kQuantThreads, 1, 1);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    long long rows_ll = rows, k_ll = k, ldx_ll = ldx;
    const unsigned int* no_amax = nullptr;
    float* no_gs = nullptr;
    if (fmt == AVE_FP4_FMT_NVFP4) {
        if (tiled) AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_fp4_kernel<kFmtNvfp4, true>, x, rows_ll, k_ll, ldx_ll, amax, gs, pk, sf));
        else AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_fp4_kernel<kFmtNvfp4, false>, x, rows_ll, k_ll, ldx_ll, amax, gs, pk, sf));
    } else {
        if (tiled) AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_fp4_kernel<kFmtMxfp4, true>, x, rows_ll, k_ll, ldx_ll, no_amax, no_gs, pk, sf));
        else AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_fp4_kernel<kFmtMxfp4, false>, x, rows_ll, k_ll, ldx_ll, no_amax, no_gs, pk, sf));
    }
    return 0;
}

int ave_fp4_quantize_nvfp4_dynamic(const void* x_bf16, int64_t rows, int64_t k, int64_t ldx, void* global_scale,
                                   void* packed, void* scales, int sf_layout, void* amax_scratch, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (rows < 0 || k < 0 || k % 32 != 0 || ldx % 8 != 0 || ldx < k)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize_nvfp4_dynamic: need k %% 32 == 0 and ldx %% 8 == 0, ldx >= k");
    if (rows == 0 || k == 0) return 0;
    if (!global_scale) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize_nvfp4_dynamic: global_scale is NULL");
    if (rows * k <= kFusedSmallElems) {
        if (sf_layout != AVE_FP4_SF_ROW_MAJOR && sf_layout != AVE_FP4_SF_TILED)
            return fail(-AVE_FP4_ERR_ARG, "unknown scale layout %d", sf_layout);
        if (!x_bf16 || !packed || !scales || !aligned16(x_bf16) || !aligned16(packed))
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize_nvfp4_dynamic: null or misaligned pointer");
        if (sf_layout == AVE_FP4_SF_TILED && (reinterpret_cast<uintptr_t>(scales) & 3u))
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize_nvfp4_dynamic: tiled scales must be 4-byte aligned");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(x_bf16);
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(kFusedClusterCtas, 1, 1);
        cfg.blockDim = dim3(kFusedThreads, 1, 1);
        const bool decode_sized = rows * (k / 16) <= kDecodeQuantBlocks;   // one 16-element block per thread
        if (decode_sized) cfg.blockDim = dim3(kDecodeQuantThreads, 1, 1);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits for its predecessor itself
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        long long rows_ll = rows, k_ll = k, ldx_ll = ldx;
        float* gs = static_cast<float*>(global_scale);
        uint8_t* pk = static_cast<uint8_t*>(packed);
        uint8_t* sf = static_cast<uint8_t*>(scales);
        if (decode_sized) {
            int rows_i = static_cast<int>(rows), k_i = static_cast<int>(k);
            if (sf_layout == AVE_FP4_SF_TILED)
                AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_nvfp4_decode_kernel<true>, x, rows_i, k_i, ldx_ll, gs, pk, sf));
            else
                AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_nvfp4_decode_kernel<false>, x, rows_i, k_i, ldx_ll, gs, pk, sf));
            return 0;
        }
        if (sf_layout == AVE_FP4_SF_TILED)
            AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_nvfp4_fused_small_kernel<true>, x, rows_ll, k_ll, ldx_ll, gs, pk, sf));
        else
            AVE_CUDA(cudaLaunchKernelEx(&cfg, quantize_nvfp4_fused_small_kernel<false>, x, rows_ll, k_ll, ldx_ll, gs, pk, sf));
        return 0;
    }
    if (!amax_scratch) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_quantize_nvfp4_dynamic: amax_scratch (4 bytes) is needed above %lld elements",
                                   static_cast<long long>(kFusedSmallElems));
    if ((rc = ave_fp4_amax(x_bf16, rows, k, ldx, amax_scratch, stream))) return rc;
    return ave_fp4_quantize(x_bf16, rows, k, ldx, AVE_FP4_FMT_NVFP4, amax_scratch, global_scale, packed, scales, sf_layout, stream);
}

int ave_fp4_sf_to_tiled(const void* sf_row_major, int64_t rows, int64_t cols, void* sf_tiled, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (rows < 0 || cols < 0) return fail(-AVE_FP4_ERR_ARG, "negative size");
    if (rows == 0 || cols == 0) return 0;
    if (!sf_row_major || !sf_tiled || (reinterpret_cast<uintptr_t>(sf_tiled) & 3u))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_sf_to_tiled: null or misaligned pointer");
    const long long total = ((rows + 127) / 128) * 128 * ((cols + 3) / 4);
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(ds->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    sf_to_tiled_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(sf_row_major), rows, cols, static_cast<uint8_t*>(sf_tiled));
    AVE_CUDA(cudaGetLastError());
    return 0;
}

int64_t ave_fp4_weight_tiles_bytes(int64_t n, int64_t k) { return ((n + 127) / 128) * ((k + 255) / 256) * 16384; }

int ave_fp4_pack_weight_tiles(const void* packed_row_major, int64_t n, int64_t k, void* packed_tiles, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (n < 0 || k < 0 || k % 32 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_pack_weight_tiles: K must be a multiple of 32");
    if (n == 0 || k == 0) return 0;
    if (!packed_row_major || !packed_tiles || !aligned16(packed_row_major) || !aligned16(packed_tiles))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_pack_weight_tiles: null or misaligned pointer");
    const long long total = ave_fp4_weight_tiles_bytes(n, k) / 16;
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(ds->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    pack_weight_tiles_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed_row_major), n, k / 2, static_cast<uint8_t*>(packed_tiles));
    AVE_CUDA(cudaGetLastError());
    return 0;
}

static int gemm_entry(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                      const void* b_scales, const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k,
                      int64_t ldd, int fmt, int variant, void* workspace, int64_t workspace_bytes, void* stream,
                      void* const* peers, int n_peers, const ave_fp4_epilogue* epi = nullptr, void* const* slabs = nullptr,
                      int rs_world = 0, int first_owner = 0, const QuantGather* qg = nullptr) {
    // shape and pointer rules first (they need no device), then the per-device state
    if (fmt != AVE_FP4_FMT_NVFP4 && fmt != AVE_FP4_FMT_MXFP4) return fail(-AVE_FP4_ERR_ARG, "unknown format %d", fmt);
    if (m < 0 || n < 0 || k < 0 || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: size out of range");
    if (m == 0 || n == 0) {
        DeviceState* ds0 = nullptr;
        return current_state(&ds0);
    }
    if (k == 0 || k % 32 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: K must be a positive multiple of 32, got %lld", static_cast<long long>(k));
    // the write-out moves 16-byte (8-column) chunks and the bias is read the same way
    if (n % 8 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: N must be a multiple of 8, got %lld", static_cast<long long>(n));
    if (ldd < n || ldd % 8 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: ldd must be >= N and a multiple of 8, got %lld", static_cast<long long>(ldd));
    const bool quant_out = epi && epi->quantize_out;
    if (!a_packed || !a_scales || !b_packed || !b_scales || (!d_bf16 && !quant_out && rs_world == 0) || !aligned16(a_packed) || !aligned16(a_scales) ||
        !aligned16(b_packed) || !aligned16(b_scales) || !aligned16(d_bf16))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: null or misaligned (16-byte) pointer");
    if (epi) {
        if (epi->activation < AVE_FP4_ACT_NONE || epi->activation > AVE_FP4_ACT_SILU || epi->reserved != 0)
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_epilogue: unknown activation %d (or reserved field not 0)", epi->activation);
        if (epi->bias_bf16 && !aligned16(epi->bias_bf16)) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_epilogue: bias must be 16-byte aligned");
        if (quant_out) {
            const int blk = (fmt == AVE_FP4_FMT_NVFP4) ? 16 : 32;
            if (n % blk != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_epilogue: a quantised result needs N %% %d == 0, got %lld", blk, static_cast<long long>(n));
            if (!epi->q_packed || !epi->q_scales || !aligned16(epi->q_packed) || !aligned16(epi->q_scales))
                return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_epilogue: q_packed / q_scales null or misaligned (16-byte)");
            if (fmt == AVE_FP4_FMT_NVFP4 && !epi->q_global_scale) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_epilogue: NVFP4 result needs q_global_scale");
            if (epi->q_sf_layout != AVE_FP4_SF_ROW_MAJOR && epi->q_sf_layout != AVE_FP4_SF_TILED)
                return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_epilogue: unknown q_sf_layout %d", epi->q_sf_layout);
        }
    }
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    const float* ags = static_cast<const float*>(a_global_scale);
    const float* bgs = static_cast<const float*>(b_global_scale);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int v = resolve_variant(variant, m, n);
    if (quant_out && v == AVE_FP4_GEMM_SKINNY && (variant & ~AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS) == AVE_FP4_GEMM_AUTO)
        v = AVE_FP4_GEMM_1CTA_N128;   // the quantising epilogue lives in the tiled kernels
    const bool nv = (fmt == AVE_FP4_FMT_NVFP4);

#define GEMM_ARGS *ds, a_packed, a_scales, ags, b_packed, b_scales, bgs, d_bf16, m, n, k, ldd, s, peers, n_peers, epi, slabs, rs_world, first_owner, qg
    switch (v) {
        case AVE_FP4_GEMM_1CTA_N128:
            return nv ? launch_gemm<1, 128, 16, kSt1N128, 2>(GEMM_ARGS) : launch_gemm<1, 128, 32, kSt1N128, 2>(GEMM_ARGS);
        case AVE_FP4_GEMM_1CTA_N256:
            return nv ? launch_gemm<1, 256, 16, kSt1N256, 1>(GEMM_ARGS) : launch_gemm<1, 256, 32, kSt1N256, 1>(GEMM_ARGS);
        case AVE_FP4_GEMM_2CTA_N256:
            if (nv && epi == nullptr && rs_world == 0 && tuning_stages_2n256() == 3) return launch_gemm<2, 256, 16, 3, 1, true>(GEMM_ARGS);
            if (nv && epi == nullptr && rs_world == 0 && tuning_stages_2n256() == 4) return launch_gemm<2, 256, 16, 4, 1, true>(GEMM_ARGS);
            return nv ? launch_gemm<2, 256, 16, kSt2N256, 1>(GEMM_ARGS) : launch_gemm<2, 256, 32, kSt2N256, 1>(GEMM_ARGS);
        case AVE_FP4_GEMM_2CTA_N128:
            return nv ? launch_gemm<2, 128, 16, kSt2N128, 2>(GEMM_ARGS) : launch_gemm<2, 128, 32, kSt2N128, 2>(GEMM_ARGS);
        case AVE_FP4_GEMM_2CTA_N192:
            return nv ? launch_gemm<2, 192, 16, kSt2N192, 2>(GEMM_ARGS) : launch_gemm<2, 192, 32, kSt2N192, 2>(GEMM_ARGS);
        case AVE_FP4_GEMM_SKINNY: {
            if (n_peers > 0) return fail(-AVE_FP4_ERR_ARG, "the fused all-gather is served by the tiled kernels only (M > 64)");
            if (epi && epi->quantize_out) return fail(-AVE_FP4_ERR_ARG, "the quantising epilogue is served by the tiled kernels only");
            if (m > 64) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: the skinny variant needs M <= 64, got %lld", static_cast<long long>(m));
            const int64_t need = skinny_workspace_bytes(m, n, ds->sm_count);
            if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
                return fail(-AVE_FP4_ERR_WORKSPACE, "ave_fp4_gemm: workspace of %lld bytes (256-byte aligned, zero-initialised) required, got %lld",
                            static_cast<long long>(need), static_cast<long long>(workspace ? workspace_bytes : 0));
#define SKINNY_ARGS *ds, a_packed, a_scales, ags, b_packed, b_scales, bgs, d_bf16, m, n, k, ldd, workspace, \
    (variant & ~AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS) == AVE_FP4_GEMM_SKINNY_TILED_W, s, (variant & AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS) != 0, epi
            const int mp = skinny_mp(m);
            if (mp == 16) return nv ? launch_skinny<16, 16, kStSkinny16>(SKINNY_ARGS) : launch_skinny<16, 32, kStSkinny16>(SKINNY_ARGS);
            if (mp == 32) return nv ? launch_skinny<32, 16, kStSkinny32>(SKINNY_ARGS) : launch_skinny<32, 32, kStSkinny32>(SKINNY_ARGS);
            return nv ? launch_skinny<64, 16, kStSkinny64>(SKINNY_ARGS) : launch_skinny<64, 32, kStSkinny64>(SKINNY_ARGS);
#undef SKINNY_ARGS
        }
        default:
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm: unknown variant %d", variant);
    }
#undef GEMM_ARGS
}

int64_t ave_fp4_linear_decode_workspace_bytes(int64_t m, int64_t n, int64_t k, int fmt, int device) {
    if (device < 0 || device >= kMaxDevices || !g_dev[device].ready) return -AVE_FP4_ERR_NOT_INIT;
    if (m < 0 || n < 0 || k < 0 || m > 32) return -AVE_FP4_ERR_ARG;
    return fused_scratch_layout(m, n, k, fmt == AVE_FP4_FMT_NVFP4 ? 16 : 32, g_dev[device].sm_count).total;
}

int ave_fp4_linear_decode(const void* x_bf16, int64_t ldx, const void* b_packed, const void* b_scales,
                          const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k, int64_t ldd, int fmt,
                          int flags, void* workspace, int64_t workspace_bytes, void* stream, const ave_fp4_epilogue* epilogue) {
    if (fmt != AVE_FP4_FMT_NVFP4 && fmt != AVE_FP4_FMT_MXFP4) return fail(-AVE_FP4_ERR_ARG, "unknown format %d", fmt);
    if (m < 0 || n < 0 || k < 0 || n > 0x7fffffff || k > 0x7fffffff) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: size out of range");
    if (m > 32)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode serves M <= 32 (got %lld); quantise with ave_fp4_quantize and call ave_fp4_gemm for more rows",
                    static_cast<long long>(m));
    if (flags & ~(AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS | AVE_FP4_LINEAR_FLAG_TILE_MAJOR_WEIGHTS))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: unknown flag bits 0x%x", flags);
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (m == 0 || n == 0) return 0;
    if (k == 0 || k % 32 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: K must be a positive multiple of 32, got %lld", static_cast<long long>(k));
    if (n % 8 != 0 || ldd < n || ldd % 8 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: N and ldd must be multiples of 8 and ldd >= N");
    if (ldx < k || ldx % 8 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: ldx must be >= K and a multiple of 8, got %lld", static_cast<long long>(ldx));
    if (!x_bf16 || !b_packed || !b_scales || !d_bf16 || !aligned16(x_bf16) || !aligned16(b_packed) || !aligned16(b_scales) || !aligned16(d_bf16))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: null or misaligned (16-byte) pointer");
    if (epilogue) {
        if (epilogue->activation < AVE_FP4_ACT_NONE || epilogue->activation > AVE_FP4_ACT_SILU || epilogue->reserved != 0 || epilogue->quantize_out)
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: the epilogue takes a bias and an activation only");
        if (epilogue->bias_bf16 && !aligned16(epilogue->bias_bf16)) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_linear_decode: bias must be 16-byte aligned");
    }
    const bool nv = (fmt == AVE_FP4_FMT_NVFP4);
    const int64_t need = fused_scratch_layout(m, n, k, nv ? 16 : 32, ds->sm_count).total;
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return fail(-AVE_FP4_ERR_WORKSPACE, "ave_fp4_linear_decode: workspace of %lld bytes (256-byte aligned, zero-initialised) required, got %lld",
                    static_cast<long long>(need), static_cast<long long>(workspace ? workspace_bytes : 0));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float* bgs = static_cast<const float*>(b_global_scale);
    const bool tile_major = (flags & AVE_FP4_LINEAR_FLAG_TILE_MAJOR_WEIGHTS) != 0;
    const bool pdl = (flags & AVE_FP4_GEMM_FLAG_STATIC_WEIGHTS) != 0;
    const int mp = skinny_mp(m);
    // quantise into the scratch (one launch: amax and quantise together for NVFP4), then the decode GEMM, chained by
    // programmatic dependent launch: the GEMM's CTAs start and stream weights while the quantise still runs
    const FusedScratch fq = fused_scratch_layout(m, n, k, nv ? 16 : 32, ds->sm_count);
    char* ws = static_cast<char*>(workspace);
    void* xq = ws + fq.packed;
    void* xsf = ws + fq.sf;
    float* xgs = nv ? reinterpret_cast<float*>(ws + fq.gs) : nullptr;
    if (nv) {
        if ((rc = ave_fp4_quantize_nvfp4_dynamic(x_bf16, m, k, ldx, xgs, xq, xsf, AVE_FP4_SF_TILED, xgs + 1, stream))) return rc;
    } else {
        if ((rc = ave_fp4_quantize(x_bf16, m, k, ldx, fmt, nullptr, nullptr, xq, xsf, AVE_FP4_SF_TILED, stream))) return rc;
    }
#define CHAIN_ARGS *ds, xq, xsf, xgs, b_packed, b_scales, bgs, d_bf16, m, n, k, ldd, workspace, tile_major, s, pdl, epilogue
    if (mp == 16) return nv ? launch_skinny<16, 16, kStSkinny16>(CHAIN_ARGS) : launch_skinny<16, 32, kStSkinny16>(CHAIN_ARGS);
    return nv ? launch_skinny<32, 16, kStSkinny32>(CHAIN_ARGS) : launch_skinny<32, 32, kStSkinny32>(CHAIN_ARGS);
#undef CHAIN_ARGS
}

int ave_fp4_set_trace(void* buffer, int64_t bytes) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (buffer == nullptr || bytes < 3 * 4 * 8) {
        ds->trace = nullptr;
        ds->trace_cap = 0;
        return 0;
    }
    if (reinterpret_cast<uintptr_t>(buffer) & 7u) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_set_trace: buffer must be 8-byte aligned");
    ds->trace = static_cast<long long*>(buffer);
    ds->trace_cap = static_cast<int>(bytes / (3 * 4 * 8));
    return 0;
}

int ave_fp4_gemm(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                 const void* b_scales, const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k,
                 int64_t ldd, int fmt, int variant, void* workspace, int64_t workspace_bytes, void* stream) {
    return gemm_entry(a_packed, a_scales, a_global_scale, b_packed, b_scales, b_global_scale, d_bf16, m, n, k, ldd, fmt,
                      variant, workspace, workspace_bytes, stream, nullptr, 0);
}

int ave_fp4_gemm_epilogue(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                          const void* b_scales, const void* b_global_scale, void* d_bf16, int64_t m, int64_t n, int64_t k,
                          int64_t ldd, int fmt, int variant, void* workspace, int64_t workspace_bytes, void* stream,
                          const ave_fp4_epilogue* epilogue) {
    return gemm_entry(a_packed, a_scales, a_global_scale, b_packed, b_scales, b_global_scale, d_bf16, m, n, k, ldd, fmt,
                      variant, workspace, workspace_bytes, stream, nullptr, 0, epilogue);
}

int ave_fp4_gemm_partials(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                          const void* b_scales, const void* b_global_scale, void* const* slab_dst, int world, int first_owner,
                          int64_t m, int64_t n, int64_t k, int fmt, void* stream) {
    if (first_owner < 0 || first_owner >= world) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_partials: first_owner %d out of range", first_owner);
    if (world < 1 || world > 8) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_partials: world must be 1..8, got %d", world);
    if (slab_dst == nullptr) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_partials: slab_dst is NULL");
    if (m <= 0 || m % (static_cast<int64_t>(world) * 32) != 0)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_partials: M must be a positive multiple of 32 * world, got %lld", static_cast<long long>(m));
    for (int i = 0; i < world; ++i)
        if (!slab_dst[i] || !aligned16(slab_dst[i])) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_partials: slab pointer %d is null or misaligned", i);
    return gemm_entry(a_packed, a_scales, a_global_scale, b_packed, b_scales, b_global_scale, nullptr, m, n, k, n, fmt,
                      AVE_FP4_GEMM_2CTA_N256, nullptr, 0, stream, nullptr, 0, nullptr, slab_dst, world, first_owner);
}

int ave_fp4_reduce_partials(const void* slabs_f32, int world, int64_t rows, int64_t n, void* d_bf16, int64_t ldd,
                            const ave_fp4_epilogue* epilogue, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (world < 1 || world > 8) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_reduce_partials: world must be 1..8, got %d", world);
    if (rows < 0 || n < 0 || n % 8 != 0 || ldd < n || ldd % 8 != 0)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_reduce_partials: N and ldd must be multiples of 8 and ldd >= N");
    if (rows == 0 || n == 0) return 0;
    if (!slabs_f32 || !d_bf16 || !aligned16(slabs_f32) || !aligned16(d_bf16))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_reduce_partials: null or misaligned (16-byte) pointer");
    const __nv_bfloat16* bias = nullptr;
    int act = 0;
    if (epilogue) {
        if (epilogue->activation < AVE_FP4_ACT_NONE || epilogue->activation > AVE_FP4_ACT_SILU || epilogue->reserved != 0 || epilogue->quantize_out)
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_reduce_partials: epilogue takes a bias and an activation only");
        if (epilogue->bias_bf16 && !aligned16(epilogue->bias_bf16)) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_reduce_partials: bias must be 16-byte aligned");
        bias = static_cast<const __nv_bfloat16*>(epilogue->bias_bf16);
        act = epilogue->activation;
    }
    const long long groups = rows * (n / 8);
    long long blocks = (groups + 255) / 256;
    const long long cap = static_cast<long long>(ds->sm_count) * ds->occ_reduce;
    if (blocks > cap) blocks = cap;
    reduce_partials_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(slabs_f32), world, rows, n, static_cast<__nv_bfloat16*>(d_bf16), ldd, bias, act);
    AVE_CUDA(cudaGetLastError());
    return 0;
}

int ave_fp4_gemm_allgather(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                           const void* b_scales, const void* b_global_scale, void* d_bf16, void* const* peer_d, int n_peers,
                           int64_t m, int64_t n, int64_t k, int64_t ldd, int fmt, int variant, void* stream) {
    if (n_peers < 0 || n_peers > 7) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather: 0..7 peers supported, got %d", n_peers);
    if (n_peers > 0 && peer_d == nullptr) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather: peer_d is NULL");
    for (int i = 0; i < n_peers; ++i)
        if (!peer_d[i] || !aligned16(peer_d[i])) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather: peer pointer %d is null or misaligned", i);
    if (variant == AVE_FP4_GEMM_AUTO) variant = AVE_FP4_GEMM_2CTA_N256;
    return gemm_entry(a_packed, a_scales, a_global_scale, b_packed, b_scales, b_global_scale, d_bf16, m, n, k, ldd, fmt,
                      variant, nullptr, 0, stream, peer_d, n_peers);
}

int ave_fp4_gemm_allgather_quantized(const void* a_packed, const void* a_scales, const void* a_global_scale, const void* b_packed,
                                     const void* b_scales, const void* b_global_scale, int64_t m, int64_t n, int64_t k, int fmt,
                                     int variant, const ave_fp4_epilogue* epilogue, int64_t n_total, int64_t col0,
                                     void* const* peer_q_packed, void* const* peer_q_scales, int n_peers, void* stream) {
    if (fmt != AVE_FP4_FMT_NVFP4 && fmt != AVE_FP4_FMT_MXFP4) return fail(-AVE_FP4_ERR_ARG, "unknown format %d", fmt);
    if (epilogue == nullptr || !epilogue->quantize_out)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather_quantized: the epilogue must ask for the quantised result (quantize_out)");
    if (n_peers < 0 || n_peers > 7) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather_quantized: 0..7 peers supported, got %d", n_peers);
    if (n_peers > 0 && (peer_q_packed == nullptr || peer_q_scales == nullptr))
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather_quantized: peer pointer arrays are NULL");
    for (int i = 0; i < n_peers; ++i)
        if (!peer_q_packed[i] || !peer_q_scales[i] || (reinterpret_cast<uintptr_t>(peer_q_packed[i]) & 31u) || !aligned16(peer_q_scales[i]))
            return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather_quantized: peer pointer %d is null or misaligned (packed: 32 bytes, scales: 16)", i);
    if (reinterpret_cast<uintptr_t>(epilogue->q_packed) & 31u)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather_quantized: q_packed must be 32-byte aligned");
    // every rank's block is whole 64-column groups (32 packed bytes, 4 NVFP4 / 2 MXFP4 scale columns of one tile row)
    if (n <= 0 || n % 64 != 0 || col0 < 0 || col0 % 64 != 0 || n_total % 64 != 0 || col0 + n > n_total)
        return fail(-AVE_FP4_ERR_ARG,
                    "ave_fp4_gemm_allgather_quantized: N, col0 and n_total must be multiples of 64 with col0 + N <= n_total "
                    "(got N = %lld, col0 = %lld, n_total = %lld)", static_cast<long long>(n), static_cast<long long>(col0),
                    static_cast<long long>(n_total));
    if (m <= 64) return fail(-AVE_FP4_ERR_ARG, "ave_fp4_gemm_allgather_quantized is served by the tiled kernels only (M > 64)");
    if (variant == AVE_FP4_GEMM_AUTO) variant = AVE_FP4_GEMM_2CTA_N256;
    QuantGather qg{n_total, col0, peer_q_packed, peer_q_scales, n_peers};
    return gemm_entry(a_packed, a_scales, a_global_scale, b_packed, b_scales, b_global_scale, nullptr, m, n, k, n, fmt, variant,
                      nullptr, 0, stream, nullptr, 0, epilogue, nullptr, 0, 0, &qg);
}

int ave_bf16_gemm(const void* a_bf16, const void* b_bf16, void* d_bf16, int64_t m, int64_t n, int64_t k, int64_t ldd,
                  int variant, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (m < 0 || n < 0 || k < 0 || m > 0x7fffffff || n > 0x7fffffff || k > 0x3fffffff)
        return fail(-AVE_FP4_ERR_ARG, "ave_bf16_gemm: size out of range");
    if (m == 0 || n == 0) return 0;
    if (k == 0 || k % 8 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_bf16_gemm: K must be a positive multiple of 8, got %lld", static_cast<long long>(k));
    if (ldd < n || ldd % 8 != 0) return fail(-AVE_FP4_ERR_ARG, "ave_bf16_gemm: ldd must be >= N and a multiple of 8, got %lld", static_cast<long long>(ldd));
    if (!a_bf16 || !b_bf16 || !d_bf16 || !aligned16(a_bf16) || !aligned16(b_bf16) || !aligned16(d_bf16))
        return fail(-AVE_FP4_ERR_ARG, "ave_bf16_gemm: null or misaligned (16-byte) pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (variant) {
        case AVE_FP4_GEMM_AUTO:
        case AVE_FP4_GEMM_2CTA_N256:
            return launch_dense<2, 256, kStDense2N256, 2>(*ds, a_bf16, b_bf16, d_bf16, m, n, k, ldd, s);
        case AVE_FP4_GEMM_1CTA_N128:
            return launch_dense<1, 128, kStDense1N128, 2>(*ds, a_bf16, b_bf16, d_bf16, m, n, k, ldd, s);
        default:
            return fail(-AVE_FP4_ERR_ARG, "ave_bf16_gemm: variant %d is not built for bf16 operands", variant);
    }
}

int ave_fp4_selftest_wait_timeout(int64_t timeout_us, void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    if (timeout_us < 1 || timeout_us > 100000)
        return fail(-AVE_FP4_ERR_ARG, "ave_fp4_selftest_wait_timeout: timeout must be 1 us .. 100 ms, got %lld us", static_cast<long long>(timeout_us));
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ds->status, static_cast<unsigned long long>(timeout_us) * 1000ull);
    AVE_CUDA(cudaGetLastError());
    return 0;
}

int ave_fp4_check(void* stream) {
    DeviceState* ds = nullptr;
    int rc = current_state(&ds);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    AVE_CUDA(cudaStreamSynchronize(s));
    int status = 0;
    AVE_CUDA(cudaMemcpy(&status, ds->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != 0) {
        AVE_CUDA(cudaMemset(ds->status, 0, sizeof(int)));
        return fail(status, "ave-lang Error [CUDA]: a kernel gave up waiting (status %d: 101 producer, 102 MMA issuer, 103 epilogue, 104 self-test)", status);
    }
    return 0;
}

}  // extern "C"
