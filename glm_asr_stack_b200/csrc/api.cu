// C-ABI entry points of libglmasr_fp4 (declared in include/glmasr_fp4.h): argument checks,
// TMA descriptor construction, the one-time weight-scale pre-pack cache, private workspaces,
// tile-shape selection and launches.  No torch types, no cuBLAS.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <unordered_map>
#include <vector>

#include "../../include/glmasr_fp4.h"
#include "elementwise.cuh"
#include "gemm_simt.cuh"
#include "gemm_umma.cuh"
#include "runtime.cuh"

namespace glmasr {

// ------------------------------------------------------------------------------------------
// private state
// ------------------------------------------------------------------------------------------
static cudaStream_t g_stream = nullptr;
static int *g_status = nullptr;
static long long g_launches = 0;
// Per-device facts and one-time set-up (the large shared-memory opt-in is an attribute of the kernel ON a
// device): indexed by the current device, so a process that drives several GPUs sets each one up.
static constexpr int kMaxDevices = 64;
static int g_num_sms[kMaxDevices] = {0};
static bool g_umma_ready[kMaxDevices] = {false};
static bool g_pair16_ready[kMaxDevices] = {false};
static bool g_pair_ready[kMaxDevices] = {false};

static int current_device() {
    int dev = 0;
    GLMASR_CUDA_CHECK(cudaGetDevice(&dev));
    GLMASR_CHECK(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
    return dev;
}

// optional per-launch timing of the GEMM kernel (CUDA events on the launching stream)
static bool g_profile = false;
struct TimedLaunch {
    cudaEvent_t start, stop;
    double flops;
    double bytes;
};
static std::vector<TimedLaunch> g_timed;

static constexpr int kSlots = 56;   // (35..37: mel.cu, 38..47: encoder.cu) 0..12, 24..25, 30..31 used here, 13..23 and 26..29 by the decode step (decoder_step.cu),
                                    // 32..33 by the prefill attention (prefill_attention_umma.cu)
static void *g_ws[kSlots] = {nullptr};
static size_t g_ws_bytes[kSlots] = {0};

struct PrepackedScales {
    uint8_t *tiled;   // [ceil(N/128)][ceil(K/64)][512]
    int N, K;
};
static std::unordered_map<const void *, PrepackedScales> g_prepack;

cudaStream_t current_stream() { return g_stream; }
void note_launches(int n) { g_launches += n; }

int *device_status_word() {
    if (g_status == nullptr) {
        GLMASR_CUDA_CHECK(cudaMalloc(&g_status, 4 * sizeof(int)));
        GLMASR_CUDA_CHECK(cudaMemset(g_status, 0, 4 * sizeof(int)));
    }
    return g_status;
}

// 0: never, 1: everywhere except the chunked host-buffer call, 2: everywhere
static int g_pdl_mode = -1;
static bool g_pdl_suppressed = false;      // set while the chunked host-buffer call enqueues its kernels
bool pdl_enabled() {
    if (g_pdl_mode < 0) {
        const char *e = getenv("GLMASR_PDL");
        g_pdl_mode = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
    }
    return g_pdl_mode == 2 || (g_pdl_mode == 1 && !g_pdl_suppressed);
}

void *workspace_slot(int slot, size_t bytes) {
    if (bytes > g_ws_bytes[slot]) {
        if (g_ws[slot]) {
            GLMASR_CUDA_CHECK(cudaStreamSynchronize(g_stream));
            GLMASR_CUDA_CHECK(cudaFree(g_ws[slot]));
        }
        const size_t want = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
        GLMASR_CUDA_CHECK(cudaMalloc(&g_ws[slot], want));
        g_ws_bytes[slot] = want;
    }
    return g_ws[slot];
}
void *workspace(size_t bytes) { return workspace_slot(0, bytes); }
// Same, zero-filled whenever it is (re)allocated; users keep it zero between their launches.
static void *workspace_slot_zeroed(int slot, size_t bytes) {
    const size_t before = g_ws_bytes[slot];
    void *ptr = workspace_slot(slot, bytes);
    if (g_ws_bytes[slot] != before) GLMASR_CUDA_CHECK(cudaMemsetAsync(ptr, 0, g_ws_bytes[slot], g_stream));
    return ptr;
}

static void clear_tmap_cache();

// W4A16: bf16 copies of FP4 weights kept on the device.  The reference's fallback dequantises a weight to bf16 on
// every call (Infer-engine/cuda/kernels.cu:1297-1318) because it has one scratch buffer for all of them; with
// 180 GB per GPU the copy of a weight that takes this route (1.5 GB for the k|v and gate|up projections of 28 layers)
// is made on first use and kept, keyed like the re-tiled scales by the weight's scale pointer and dropped by
// glmasr_fp4_forget / the cleanup hooks.  Same values as the reference's: bf16(lut * e4m3(scale) * global).
// GLMASR_W4A16_RESIDENT_MB bounds the total (default 4096; 0: off).
struct ResidentBf16 {
    __nv_bfloat16 *w;
    const void *packed;
    int N, K;
    float global;
    size_t bytes;
};
static std::unordered_map<const void *, ResidentBf16> g_resident;
static size_t g_resident_bytes = 0;

static size_t resident_budget_bytes() {
    static long long v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_W4A16_RESIDENT_MB");
        v = (e && e[0]) ? atoll(e) : 4096;
        if (v < 0) v = 0;
    }
    return (size_t)v << 20;
}

static void drop_resident(const void *w_scales) {
    auto it = g_resident.find(w_scales);
    if (it == g_resident.end()) return;
    cudaFree(it->second.w);
    g_resident_bytes -= it->second.bytes;
    g_resident.erase(it);
}


void free_all_private_state() {
    cudaDeviceSynchronize();
    encoder_forget_all();          // its tables live in workspace slots
    for (int i = 0; i < kSlots; ++i) {
        if (g_ws[i]) cudaFree(g_ws[i]);
        g_ws[i] = nullptr;
        g_ws_bytes[i] = 0;
    }
    for (auto &kv : g_prepack) cudaFree(kv.second.tiled);
    g_prepack.clear();
    for (auto &kv : g_resident) cudaFree(kv.second.w);
    g_resident.clear();
    g_resident_bytes = 0;
    tail_forget_scales(nullptr);
    clear_tmap_cache();
    if (g_status) cudaFree(g_status);
    g_status = nullptr;
}

enum Slot : int {
    WS_XQ = 0,        // quantised activations (packed e2m1)
    WS_XSF = 1,       // their scales, 128x4-tiled
    WS_XSF_ROW = 2,   // row-major scales (SIMT path)
    WS_LOGITS = 3,    // lm_head logits
    WS_TOKENS = 4,    // lm_head arg-max result
    WS_TMP = 5,       // SIMT-path epilogue staging
    WS_L_QKV = 6, WS_L_H1 = 7, WS_L_ACT = 8, WS_L_IN = 9, WS_L_OUT = 10,
    WS_WDEQ = 11,
    WS_DBG = 12,      // cycle counters of timing experiments
    WS_L_ACTQ = 24, WS_L_ACTSF = 25,
    WS_PARTIAL = 30, WS_COUNTERS = 31,   // split-K partial accumulators and per-tile arrival counters   // layer path: quantised SiLU-gate output handed to the down projection
};

static int num_sms() {
    const int dev = current_device();
    if (g_num_sms[dev] == 0)
        GLMASR_CUDA_CHECK(cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev));
    return g_num_sms[dev];
}

// rows from which W4A16 dequantises each weight once instead of inside the GEMM
static int w4a16_dequant_once_rows() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_W4A16_DEQUANT_ONCE_ROWS");
        v = (e && e[0]) ? atoi(e) : 1024;
        if (v < 1) v = 1;
    }
    return v;
}

#ifdef GLMASR_EXPERIMENTS
static int g_debug_override = -1;           // glmasr_debug_set_flags: timing experiments from the host language
static int debug_flags() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_DEBUG_FLAGS");
        v = (e && e[0]) ? atoi(e) : 0;
    }
    return g_debug_override >= 0 ? g_debug_override : v;
}
#else
static int debug_flags() { return 0; }
#endif

// GLMASR_FORCE_NB=1/2: 128-row weight sub-tiles per CTA tile of the single-CTA kernel (comparison runs); 0 = per shape
static int forced_nb() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_FORCE_NB");
        v = (e && e[0]) ? (atoi(e) == 1 ? 1 : 2) : 0;
    }
    return v;
}

// GLMASR_PAIR_KERNEL=0 keeps W4A4 on the single-CTA kernel (comparison runs)
static bool use_pair_kernel() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_PAIR_KERNEL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

static bool no_tma_store() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_NO_TMA_STORE");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// GLMASR_NO_FUSED_ACT_QUANT=1: the layer path writes the bf16 activation and quantises it with the
// stand-alone kernel (for A/B comparisons against the quantising epilogue)
static bool no_fused_act_quant() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_NO_FUSED_ACT_QUANT");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// GLMASR_SPLIT_K=n: split-K factor of the small-M W4A4 GEMMs (0 = chosen per shape); unset or 1: no split
static int split_k_override() {
    static int v = -2;
    if (v == -2) {
        const char *e = getenv("GLMASR_SPLIT_K");
        v = (e && e[0]) ? atoi(e) : -1;
    }
    return v;
}

// GLMASR_PAIR16=0: SiLU-gate epilogues stay on the eight-epilogue-warp pair kernel (comparison runs)
// GLMASR_BF16_PAIR=0: bf16 GEMMs never take the CTA-pair kernel.
static bool use_pair_bf16() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_BF16_PAIR");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}
// GLMASR_SPLIT_TAIL=0: the pair kernel's last, partly filled tile round is not cut into half tiles.
static bool split_tail_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_SPLIT_TAIL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}
static bool use_pair16_kernel() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_PAIR16");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

static bool force_simt() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_FP4_FORCE_SIMT");
        v = (e && e[0] && strcmp(e, "0") != 0) ? 1 : 0;
    }
    return v == 1;
}

// ------------------------------------------------------------------------------------------
// TMA descriptors
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        GLMASR_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        GLMASR_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled not available");
        fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D row-major tensor [rows, inner] of `elem_bytes`-byte elements, row pitch `pitch_bytes`;
// boxes of box_rows x box_inner elements.  Encoding a descriptor is a driver call of several
// microseconds and a decode step needs ~900 of them over the same few buffers, so encoded
// descriptors are cached by their full parameter tuple.
struct TmapKey {
    const void *base;
    uint64_t inner, rows, pitch;
    uint32_t box_inner, box_rows;
    int dt, swizzle;
    bool operator==(const TmapKey &o) const {
        return base == o.base && inner == o.inner && rows == o.rows && pitch == o.pitch && box_inner == o.box_inner &&
               box_rows == o.box_rows && dt == o.dt && swizzle == o.swizzle;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey &k) const {
        uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull;
        h ^= (k.inner + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= (k.rows * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2));
        h ^= (k.pitch + ((uint64_t)k.box_inner << 32) + ((uint64_t)k.box_rows << 16) + (uint64_t)(k.dt * 4 + k.swizzle) + (h << 6));
        return (size_t)h;
    }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
static void clear_tmap_cache() { g_tmaps.clear(); }

static bool make_tmap(CUtensorMap *tm, const void *base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner,
                      uint64_t rows, uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, bool swizzle128,
                      bool swizzle64 = false) {
    if (((uintptr_t)base & 15) != 0 || (pitch_bytes & 15) != 0) return false;
    (void)elem_bytes;
    const TmapKey key = {base, inner, rows, pitch_bytes, box_inner, box_rows, (int)dt, swizzle128 ? 1 : (swizzle64 ? 2 : 0)};
    auto it = g_tmaps.find(key);
    if (it != g_tmaps.end()) {
        *tm = it->second;
        return true;
    }
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode_fn()(tm, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                              : (swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (g_tmaps.size() > 16384) g_tmaps.clear();
    g_tmaps.emplace(key, *tm);
    return true;
}

bool make_bf16_tmap_sw128(CUtensorMap *tm, const void *base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                          uint32_t box_inner, uint32_t box_rows) {
    return make_tmap(tm, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, inner, rows, pitch_bytes, box_inner, box_rows, true);
}

// ------------------------------------------------------------------------------------------
// weight-scale pre-pack cache
// ------------------------------------------------------------------------------------------
static size_t tiled_sf_bytes(int rows, int K) {
    return (size_t)((rows + 127) / 128) * (size_t)((K + 63) / 64) * 512;
}

static const uint8_t *prepacked_scales(const uint8_t *w_scales, int N, int K) {
    auto it = g_prepack.find(w_scales);
    if (it != g_prepack.end() && it->second.N == N && it->second.K == K) return it->second.tiled;
    if (it != g_prepack.end()) {
        GLMASR_CUDA_CHECK(cudaStreamSynchronize(g_stream));
        cudaFree(it->second.tiled);
        g_prepack.erase(it);
    }
    PrepackedScales ps;
    ps.N = N;
    ps.K = K;
    const size_t bytes = tiled_sf_bytes(N, K);
    GLMASR_CUDA_CHECK(cudaMalloc(&ps.tiled, bytes));
    GLMASR_CUDA_CHECK(cudaMemsetAsync(ps.tiled, 0, bytes, g_stream));
    launch_swizzle_scales(ps.tiled, w_scales, N, K / 16, g_stream);
    ++g_launches;
    GLMASR_CUDA_CHECK(cudaGetLastError());
    g_prepack[w_scales] = ps;
    return ps.tiled;
}

// ------------------------------------------------------------------------------------------
// the fused linear
// ------------------------------------------------------------------------------------------
struct FusedArgs {
    int mode;                       // GEMM_W4A4 / GEMM_W4A16 / GEMM_BF16
    __nv_bfloat16 *out;
    int ldo;
    const __nv_bfloat16 *x;
    int ldx;
    const glmasr_fp4_weight *w;     // FP4 modes
    const __nv_bfloat16 *w_bf16[kMaxSegments];   // BF16 mode: one bf16 [N_s, K] tensor per segment
    int n_bf16[kMaxSegments];
    int num_w;
    __nv_bfloat16 *weight_scratch;  // W4A16, large M: caller scratch for the dequantised weight (may be NULL)
    float input_scale;
    const __nv_bfloat16 *pre;
    __nv_bfloat16 *prequant_scratch;
    int epi;
    const __nv_bfloat16 *residual;
    const __nv_bfloat16 *bias;
    int M, K;
    // W4A4 only.  xq / xq_sf: the activation is already quantised (e2m1 bytes [M, K/2] + tiled
    // scales), x is ignored.  q_out / q_out_sf: EPI_SILU_GATE writes its result quantised with
    // q_out_input_scale for the next GEMM instead of bf16 to out (pair kernel only).
    const uint8_t *xq, *xq_sf;
    uint8_t *q_out, *q_out_sf;
    float q_out_input_scale;
};

static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

static bool tensor_core_eligible(const FusedArgs &a) {
    if (force_simt()) return false;
    // operand tiles are 128 bytes of K per step: 256 e2m1 elements, 64 bf16; W4A16 stages raw weights 256 at a time
    if (a.K % (a.mode == GEMM_BF16 ? 64 : 256) != 0) return false;
    if (!aligned16(a.x) || !aligned16(a.out) || (a.ldx % 8) != 0) return false;
    if (a.mode == GEMM_BF16) {
        for (int i = 0; i < a.num_w; ++i)
            if (!aligned16(a.w_bf16[i])) return false;
        return true;
    }
    for (int i = 0; i < a.num_w; ++i) {
        if (a.w[i].w_scales == nullptr) return false;
        if (!aligned16(a.w[i].w_packed) || !aligned16(a.w[i].w_scales)) return false;
    }
    return true;
}

static int total_out_cols(const FusedArgs &a) {
    if (a.epi == EPI_SILU_GATE) return a.mode == GEMM_BF16 ? a.n_bf16[0] : a.w[0].N;
    int n = 0;
    for (int i = 0; i < a.num_w; ++i) n += a.mode == GEMM_BF16 ? a.n_bf16[i] : a.w[i].N;
    return n;
}

// SIMT route: same results, any shape.
static int run_simt(const FusedArgs &a) {
    const uint8_t *xq = nullptr, *xs = nullptr;
    const __nv_bfloat16 *x = a.x;
    int ldx = a.ldx;
    if (a.mode == GEMM_W4A4) {
        uint8_t *q = (uint8_t *)workspace_slot(WS_XQ, (size_t)a.M * a.K / 2);
        uint8_t *s = (uint8_t *)workspace_slot(WS_XSF_ROW, (size_t)a.M * a.K / 16);
        launch_quantize_act(q, s, nullptr, a.x, a.pre, a.input_scale, a.M, a.K, a.ldx, g_stream);
        ++g_launches;
        xq = q;
        xs = s;
    } else if (a.pre != nullptr) {
        GLMASR_CHECK(a.prequant_scratch != nullptr && a.ldx == a.K, "pre_quant_scale needs prequant_scratch and a dense x");
        launch_prequant(a.prequant_scratch, a.x, a.pre, a.M, a.K, g_stream);
        ++g_launches;
        x = a.prequant_scratch;
        ldx = a.K;
    }
    __nv_bfloat16 *dst = a.out;
    int ldo = a.ldo;
    const int n0 = a.mode == GEMM_BF16 ? a.n_bf16[0] : a.w[0].N;
    if (a.epi == EPI_SILU_GATE) {
        dst = (__nv_bfloat16 *)workspace_slot(WS_TMP, (size_t)a.M * 2 * n0 * 2);
        ldo = 2 * n0;
    } else if (a.epi == EPI_RESIDUAL) {
        dst = (__nv_bfloat16 *)workspace_slot(WS_TMP, (size_t)a.M * a.ldo * 2);
    }
    int col = 0;
    for (int i = 0; i < a.num_w; ++i) {
        SimtGemmArgs g;
        memset(&g, 0, sizeof(g));
        g.mode = a.mode == GEMM_W4A4 ? 0 : (a.mode == GEMM_W4A16 ? 1 : 2);
        g.x_packed = xq;
        g.x_scales = xs;
        g.x = x;
        g.ldx = ldx;
        g.M = a.M;
        g.K = a.K;
        g.out = dst;
        g.ldo = ldo;
        g.col0 = col;
        g.bias = a.bias;
        if (a.mode == GEMM_BF16) {
            g.w_bf16 = a.w_bf16[i];
            g.N = a.n_bf16[i];
            g.alpha = 1.0f;
        } else {
            g.w_packed = a.w[i].w_packed;
            g.w_scales = a.w[i].w_scales;
            g.N = a.w[i].N;
            g.alpha = a.mode == GEMM_W4A4 ? a.input_scale * a.w[i].w_global_scale : a.w[i].w_global_scale;
        }
        if (launch_simt_gemm(g, g_stream) != cudaSuccess) return -1;
        ++g_launches;
        col += g.N;
    }
    if (a.epi == EPI_SILU_GATE) {
        GLMASR_CHECK(a.ldo == n0, "SIMT SiLU path needs a dense output");
        launch_silu_split(a.out, dst, a.M, n0, g_stream);
        ++g_launches;
    } else if (a.epi == EPI_RESIDUAL) {
        GLMASR_CHECK(a.ldo == total_out_cols(a), "SIMT residual path needs a dense output");
        launch_residual_add(a.out, dst, a.residual, (long long)a.M * a.ldo, g_stream);
        ++g_launches;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Row count that picks the W4A16 route while a larger call is being served in row chunks, so that
// every chunk takes the route (and gives the bytes) of the whole call.
static int g_route_rows = 0;

// The resident bf16 copy of one FP4 weight [N, K]; nullptr when it cannot be kept (no scale tensor to key it by,
// budget spent, allocation refused).
static const __nv_bfloat16 *resident_bf16_weight(const glmasr_fp4_weight &w, int K) {
    if (w.w_scales == nullptr || w.w_packed == nullptr || w.N <= 0 || K <= 0) return nullptr;
    auto it = g_resident.find(w.w_scales);
    if (it != g_resident.end()) {
        const ResidentBf16 &r = it->second;
        if (r.packed == w.w_packed && r.N == w.N && r.K == K && r.global == w.w_global_scale) return r.w;
        cudaStreamSynchronize(g_stream);
        drop_resident(w.w_scales);          // the key now names another tensor
    }
    const size_t bytes = (size_t)w.N * K * sizeof(__nv_bfloat16);
    if (g_resident_bytes + bytes > resident_budget_bytes()) return nullptr;
    ResidentBf16 r = {nullptr, w.w_packed, w.N, K, w.w_global_scale, bytes};
    if (cudaMalloc(&r.w, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    launch_dequant(r.w, w.w_packed, w.w_scales, w.w_global_scale, w.N, K, g_stream);
    ++g_launches;
    g_resident[w.w_scales] = r;
    g_resident_bytes += bytes;
    return r.w;
}

static int run_fused(const FusedArgs &a) {
    if (a.M <= 0 || a.K <= 0) return -1;
    if (a.mode != GEMM_BF16) {
        if (a.num_w < 1 || a.num_w > kMaxSegments) return -1;
        for (int i = 0; i < a.num_w; ++i)
            if (a.w[i].N <= 0 || a.w[i].w_packed == nullptr) return -1;
        if (a.K % 16 != 0) return -1;
        if (a.epi == EPI_SILU_GATE && (a.num_w != 2 || a.w[0].N != a.w[1].N)) return -1;
        if (a.epi == EPI_RESIDUAL && (a.num_w != 1 || a.residual == nullptr)) return -1;
    }
    if (!tensor_core_eligible(a)) {
        if (a.xq != nullptr || a.q_out != nullptr) return -1;   // quantised hand-over exists on the tensor-core path only
        return run_simt(a);
    }

    // W4A16 on resident bf16 copies of the weights (made on first use, within the budget): the bf16 GEMM streams
    // them at the rate of the memory system, where the in-kernel dequant of a decode-sized call is a chain of
    // small dependent stages (gate|up at 256 rows: 43 us against ~12)
    if (a.mode == GEMM_W4A16 && resident_budget_bytes() > 0) {
        const __nv_bfloat16 *wb[kMaxSegments];
        bool all = true;
        for (int i = 0; i < a.num_w && all; ++i) {
            wb[i] = resident_bf16_weight(a.w[i], a.K);
            all = wb[i] != nullptr;
        }
        if (all) {
            FusedArgs b = a;
            b.mode = GEMM_BF16;
            for (int i = 0; i < a.num_w; ++i) {
                b.w_bf16[i] = wb[i];
                b.n_bf16[i] = a.w[i].N;
            }
            b.w = nullptr;
            return run_fused(b);
        }
    }

    // W4A16 with many rows: the in-kernel dequant (repeated for every 128-row tile) becomes the
    // bottleneck, so do what the reference does -- dequantise each weight once to bf16
    // (Infer-engine/cuda/kernels.cu:1316) -- and run the bf16 GEMM on the result.
    if (a.mode == GEMM_W4A16 && (a.M > g_route_rows ? a.M : g_route_rows) >= w4a16_dequant_once_rows()) {
        size_t elems = 0;
        for (int i = 0; i < a.num_w; ++i) elems += (size_t)a.w[i].N * a.K;
        __nv_bfloat16 *wd = (a.weight_scratch != nullptr && a.num_w == 1)
                                ? a.weight_scratch
                                : (__nv_bfloat16 *)workspace_slot(WS_WDEQ, elems * 2);
        FusedArgs b = a;
        b.mode = GEMM_BF16;
        size_t off = 0;
        for (int i = 0; i < a.num_w; ++i) {
            launch_dequant(wd + off, a.w[i].w_packed, a.w[i].w_scales, a.w[i].w_global_scale, a.w[i].N, a.K, g_stream);
            ++g_launches;
            b.w_bf16[i] = wd + off;
            b.n_bf16[i] = a.w[i].N;
            off += (size_t)a.w[i].N * a.K;
        }
        b.w = nullptr;
        return run_fused(b);
    }

    const int dev = current_device();
    if (!g_umma_ready[dev]) {
        GLMASR_CUDA_CHECK(umma_gemm_init());
        g_umma_ready[dev] = true;
    }

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = a.M;
    p.K = a.K;
    p.out = a.out;
    p.ldo = a.ldo;
    p.residual = a.residual;
    p.bias = a.bias;
    p.epi = a.epi;
    p.status = device_status_word();
    p.debug = debug_flags();
#ifdef GLMASR_EXPERIMENTS
    p.dbg_cycles = (p.debug & 64) ? (unsigned long long *)workspace_slot(WS_DBG, 148 * 16 * 8 * 4) : nullptr;
#endif
    p.num_m_tiles = (a.M + 127) / 128;
    p.n_out = total_out_cols(a);
    // W4A4 weights and their re-tiled scales are read-only for every kernel that signals its dependents early:
    // the only writer, the one-time scale re-tiling, is launched as an ordinary kernel and therefore completes
    // before anything behind it starts.  So the producer may fetch them ahead of the dependency wait.
    p.early_weights = (a.mode == GEMM_W4A4 && pdl_enabled()) ? 1 : 0;

    // operand A
    const __nv_bfloat16 *x = a.x;
    int ldx = a.ldx;
    if (a.mode == GEMM_W4A4) {
        const uint8_t *xq = a.xq, *xsf = a.xq_sf;
        if (xq == nullptr) {
            uint8_t *q = (uint8_t *)workspace_slot(WS_XQ, (size_t)a.M * a.K / 2);
            uint8_t *sf = (uint8_t *)workspace_slot(WS_XSF, tiled_sf_bytes(a.M, a.K));
            launch_quantize_act(q, nullptr, sf, a.x, a.pre, a.input_scale, a.M, a.K, a.ldx, g_stream);
            ++g_launches;
            xq = q, xsf = sf;
        }
        if (!make_tmap(&p.tm_a, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.K / 2, (uint64_t)a.M,
                       (uint64_t)a.K / 2, 128, 128, true))
            return -1;
        p.sfa = xsf;
        p.num_k_blocks = a.K / 256;
        p.sf_k_chunks = a.K / 64;
        if (!make_tmap(&p.tm_sfa, xsf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, 128,
                       (uint64_t)((a.M + 127) / 128) * (uint64_t)(a.K / 64), 512, 128, 4, false))
            return -1;
    } else {
        if (a.pre != nullptr) {
            if (a.prequant_scratch == nullptr || a.ldx != a.K) return -1;
            launch_prequant(a.prequant_scratch, a.x, a.pre, a.M, a.K, g_stream);
            ++g_launches;
            x = a.prequant_scratch;
            ldx = a.K;
        }
        if (!make_tmap(&p.tm_a, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K, (uint64_t)a.M,
                       (uint64_t)ldx * 2, 64, 128, true))
            return -1;
        p.num_k_blocks = a.K / 64;
    }

    // operand B
    int subtiles = 0;
    if (a.mode == GEMM_BF16) {
        p.num_segs = a.num_w;
        for (int i = 0; i < a.num_w; ++i) {
            p.seg_rows[i] = a.n_bf16[i];
            p.seg_subtiles[i] = (a.n_bf16[i] + 127) / 128;
            subtiles += p.seg_subtiles[i];
            p.alpha[i] = 1.0f;
            if (!make_tmap(&p.tm_b[i], a.w_bf16[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)a.K,
                           (uint64_t)a.n_bf16[i], (uint64_t)a.K * 2, 64, 128, true))
                return -1;
        }
    } else {
        p.num_segs = a.num_w;
        for (int i = 0; i < a.num_w; ++i) {
            const glmasr_fp4_weight &w = a.w[i];
            p.seg_rows[i] = w.N;
            p.seg_subtiles[i] = (w.N + 127) / 128;
            subtiles += p.seg_subtiles[i];
            p.alpha[i] = a.mode == GEMM_W4A4 ? a.input_scale * w.w_global_scale : w.w_global_scale;
            if (!make_tmap(&p.tm_b[i], w.w_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.K / 2, (uint64_t)w.N,
                           (uint64_t)a.K / 2, 128, 128, true))
                return -1;
            if (a.mode == GEMM_W4A4) {
                p.sfb[i] = prepacked_scales(w.w_scales, w.N, a.K);
                if (!make_tmap(&p.tm_sfb[i], p.sfb[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, 128,
                               (uint64_t)((w.N + 127) / 128) * (uint64_t)(a.K / 64), 512, 128, 4, false))
                    return -1;
            } else {
                if (!make_tmap(&p.tm_bs[i], w.w_scales, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.K / 16,
                               (uint64_t)w.N, (uint64_t)a.K / 16, 16, 128, false))
                    return -1;
            }
        }
    }

    // W4A4 with enough 256 x 256 tiles for every CTA pair: the cta_group::2 kernel
    // (a bias together with a residual stays on the single-CTA kernel, whose epilogue rounds bf16(acc) + bias before
    // the residual is added, as residual_add_bias does: Infer-engine/cuda/kernels.cu:763-782)
    // The bf16 GEMM takes the same kernel on bf16 operands (GLMASR_BF16_PAIR=0: always the single-CTA kernel).
    const bool pair_bf16 = a.mode == GEMM_BF16 && use_pair_bf16();
    if ((a.mode == GEMM_W4A4 || pair_bf16) && use_pair_kernel() && (pair_bf16 || !(a.bias != nullptr && a.epi == EPI_RESIDUAL))) {
        const int n_tiles = a.epi == EPI_SILU_GATE ? p.seg_subtiles[0] : (subtiles + 1) / 2;
        const int m_pairs = (p.num_m_tiles + 1) / 2;
        const int pairs = num_sms() / 2;
        if (m_pairs * n_tiles >= pairs && a.M >= 512) {
            if (!g_pair_ready[dev]) {
                GLMASR_CUDA_CHECK(umma_gemm_pair_init());
                g_pair_ready[dev] = true;
            }
            p.num_n_tiles = n_tiles;
            p.split_tail = (!pair_bf16 && a.epi != EPI_SILU_GATE && split_tail_enabled()) ? 1 : 0;
            for (int i = 0; i < p.num_segs && p.split_tail; ++i)
                if (!make_tmap(&p.tm_b_half[i], a.w[i].w_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)a.K / 2,
                               (uint64_t)a.w[i].N, (uint64_t)a.K / 2, 128, 64, true))
                    p.split_tail = 0;
            // epilogue through shared memory + bulk tensor stores when the output can be described to TMA
            bool tma_ok = aligned16(a.out) && (a.ldo % 8) == 0 && !no_tma_store();
            for (int i = 0; i < p.num_segs && a.epi != EPI_SILU_GATE; ++i)
                if (i + 1 < p.num_segs && (p.seg_rows[i] % 8) != 0) tma_ok = false;   // segment column offsets stay 16-byte aligned
            // SiLU-gate epilogues run on the sixteen-epilogue-warp variant (32 x 32 output boxes)
            const bool wide = !pair_bf16 && a.epi == EPI_SILU_GATE && use_pair16_kernel();
            if (tma_ok && a.q_out == nullptr)
                tma_ok = wide ? make_tmap(&p.tm_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)p.n_out, (uint64_t)a.M,
                                          (uint64_t)a.ldo * 2, 32, 32, false, true)
                              : make_tmap(&p.tm_out, a.out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)p.n_out, (uint64_t)a.M,
                                          (uint64_t)a.ldo * 2, 64, 32, true);
            p.tma_store = tma_ok ? 1 : 0;
            if (a.q_out != nullptr) {
                if (a.epi != EPI_SILU_GATE || (p.seg_rows[0] % 64) != 0 || !(a.q_out_input_scale > 0.0f)) return -1;
                p.q_packed = a.q_out;
                p.q_sf = a.q_out_sf;
                p.q_inv_in = 1.0f / a.q_out_input_scale;
                p.q_ld = p.seg_rows[0] / 2;
                p.q_sf_chunks = p.seg_rows[0] / 64;
                // the sixteen-warp variant stores the codes through TMA: [M, q_ld] bytes, 32-row x 16-byte boxes
                p.tma_store = (wide && !no_tma_store() && aligned16(a.q_out) && (p.q_ld % 16) == 0 &&
                               make_tmap(&p.tm_out, a.q_out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)p.q_ld, (uint64_t)a.M,
                                         (uint64_t)p.q_ld, 16, 32, false))
                                  ? 1
                                  : 0;
            }
            TimedLaunch tl;
            if (g_profile) {
                cudaEventCreate(&tl.start);
                cudaEventCreate(&tl.stop);
                int n_rows = 0;
                for (int i = 0; i < p.num_segs; ++i) n_rows += p.seg_rows[i];
                tl.flops = 2.0 * a.M * (double)n_rows * a.K;
                tl.bytes = (double)n_rows * a.K * 0.5625 + (double)a.M * a.K * 0.5625 + 2.0 * a.M * p.n_out +
                           (a.epi == EPI_RESIDUAL ? 2.0 * a.M * p.n_out : 0.0);
                if (a.q_out != nullptr) tl.bytes -= (2.0 - 0.5625) * a.M * p.n_out;   // e2m1 + scales instead of bf16
                if (pair_bf16) tl.bytes += ((double)n_rows * a.K + (double)a.M * a.K) * (2.0 - 0.5625);   // bf16 operands
                cudaEventRecord(tl.start, g_stream);
            }
            if (wide) {
                if (!g_pair16_ready[dev]) {
                    GLMASR_CUDA_CHECK(umma_gemm_pair16_init());
                    g_pair16_ready[dev] = true;
                }
                if (launch_umma_gemm_pair16(p, pairs, g_stream) != cudaSuccess) return -1;
            } else if ((pair_bf16 ? launch_umma_gemm_pair_bf16(p, pairs, g_stream) : launch_umma_gemm_pair(p, pairs, g_stream)) != cudaSuccess) {
                return -1;
            }
            ++g_launches;
            if (g_profile) {
                cudaEventRecord(tl.stop, g_stream);
                g_timed.push_back(tl);
            }
            return 0;
        }
    }

    if (a.q_out != nullptr) {               // quantising SiLU-gate epilogue of the single-CTA kernel (two sub-tiles per tile)
        if (a.epi != EPI_SILU_GATE || (p.seg_rows[0] % 64) != 0 || !(a.q_out_input_scale > 0.0f)) return -1;
        p.q_packed = a.q_out;
        p.q_sf = a.q_out_sf;
        p.q_inv_in = 1.0f / a.q_out_input_scale;
        p.q_ld = p.seg_rows[0] / 2;
        p.q_sf_chunks = p.seg_rows[0] / 64;
    }

    // tile shape: two weight sub-tiles per CTA tile when that still fills the machine
    int nb;
    if (a.epi == EPI_SILU_GATE) {
        nb = 2;
        p.num_n_tiles = p.seg_subtiles[0];
    } else {
        const int tiles2 = p.num_m_tiles * ((subtiles + 1) / 2);
        nb = (subtiles >= 2 && tiles2 >= num_sms()) ? 2 : 1;
        if (forced_nb() != 0) nb = forced_nb();
        p.num_n_tiles = (subtiles + nb - 1) / nb;
    }
    const int total_tiles = p.num_m_tiles * p.num_n_tiles;
    // Few tiles (decode: M <= 256): K can be split so that every SM streams a share of the weights
    // (GLMASR_SPLIT_K=n, or 0 for a per-shape choice).  Off unless asked for: at these sizes a launch is
    // bound by its fixed latency (set-up, first loads, epilogue), not by the K loop, and the partials'
    // round trip through L2 plus the last CTA's reduction cost more than the shorter loop saves
    // (decode step 3.12 ms unsplit, 3.34 / 3.38 / 3.44 ms with 2 / 3 / per-shape splits).
    int split = 1;
    if (a.mode == GEMM_W4A4 && total_tiles * 2 <= num_sms() && split_k_override() >= 0) {
        const int forced = split_k_override();
        if (forced == 0) {
            split = num_sms() / total_tiles;
            if (split > 4) split = 4;
            if (split > p.num_k_blocks / 2) split = p.num_k_blocks / 2;     // at least two K blocks per CTA
        } else {
            split = forced > p.num_k_blocks ? p.num_k_blocks : forced;
        }
        if (split < 1) split = 1;
    }
    if (split > 1) {
        p.split_k = split;
        p.partial = (float *)workspace_slot(WS_PARTIAL, (size_t)total_tiles * split * 128 * (128 * nb) * sizeof(float));
        p.tile_counters = (int *)workspace_slot_zeroed(WS_COUNTERS, (size_t)total_tiles * sizeof(int));
    }
    const int work = total_tiles * split;
    const int ctas = work < num_sms() ? work : num_sms();
    TimedLaunch tl;
    if (g_profile) {
        cudaEventCreate(&tl.start);
        cudaEventCreate(&tl.stop);
        int n_rows = 0;
        for (int i = 0; i < p.num_segs; ++i) n_rows += p.seg_rows[i];
        tl.flops = 2.0 * a.M * (double)n_rows * a.K;
        // algorithmic bytes of this launch: operands as stored + output (+ residual read)
        const double wbytes = a.mode == GEMM_BF16 ? 2.0 * n_rows * a.K : (double)n_rows * a.K / 2 + (double)n_rows * a.K / 16;
        const double xbytes = a.mode == GEMM_W4A4 ? (double)a.M * a.K / 2 + (double)a.M * a.K / 16 : 2.0 * a.M * a.K;
        tl.bytes = wbytes + xbytes + 2.0 * a.M * p.n_out + (a.epi == EPI_RESIDUAL ? 2.0 * a.M * p.n_out : 0.0);
        cudaEventRecord(tl.start, g_stream);
    }
    if (launch_umma_gemm(a.mode, nb, p, ctas, g_stream) != cudaSuccess) return -1;
    ++g_launches;
    if (g_profile) {
        cudaEventRecord(tl.stop, g_stream);
        g_timed.push_back(tl);
    }
    return 0;
}

size_t tiled_scale_bytes(int rows, int K) { return tiled_sf_bytes(rows, K); }

bool make_u8_tmap_sw128(CUtensorMap *tm, const void *base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_inner, uint32_t box_rows) {
    return make_tmap(tm, base, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, inner, rows, pitch_bytes, box_inner, box_rows, true);
}

// Event bracket around a launch made outside this file, recorded like the GEMM launches above when
// glmasr_profile_enable is on (no-ops otherwise).
static TimedLaunch g_open_bracket;
void profile_bracket_begin(double flops, double bytes) {
    if (!g_profile) return;
    cudaEventCreate(&g_open_bracket.start);
    cudaEventCreate(&g_open_bracket.stop);
    g_open_bracket.flops = flops;
    g_open_bracket.bytes = bytes;
    cudaEventRecord(g_open_bracket.start, g_stream);
}
void profile_bracket_end() {
    if (!g_profile) return;
    cudaEventRecord(g_open_bracket.stop, g_stream);
    g_timed.push_back(g_open_bracket);
}

// W4A4 GEMM whose activation has already been quantised (e2m1 bytes [M, K/2] + tiled scales) by
// a producer kernel of this library.  Tensor-core path only; -1 when the shape cannot take it.
int fp4_linear_w4a4_prequantized(uint16_t *out, int ldo, const uint8_t *xq, const uint8_t *xq_sf,
                                 const glmasr_fp4_weight *weights, int num_weights, float input_scale, int epilogue,
                                 const uint16_t *residual, int M, int K, uint8_t *q_out, uint8_t *q_out_sf,
                                 float q_out_input_scale) {
    if ((out == nullptr && q_out == nullptr) || xq == nullptr || xq_sf == nullptr || weights == nullptr || !(input_scale > 0.0f))
        return -1;
    for (int i = 0; i < num_weights && i < kMaxSegments; ++i)
        if (weights[i].w_scales == nullptr) return -1;
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = GEMM_W4A4;
    a.out = (__nv_bfloat16 *)out;
    a.ldo = ldo;
    a.ldx = K;
    a.xq = xq;
    a.xq_sf = xq_sf;
    a.w = weights;
    a.num_w = num_weights;
    a.input_scale = input_scale;
    a.epi = epilogue;
    a.residual = (const __nv_bfloat16 *)residual;
    a.M = M;
    a.K = K;
    a.q_out = q_out;
    a.q_out_sf = q_out_sf;
    a.q_out_input_scale = q_out_input_scale;
    if (ldo < total_out_cols(a)) return -1;
    return run_fused(a);
}

// gate|up as one W4A16 GEMM (the arithmetic of the reference's fused pair, Infer-engine/cuda/decoder.cu:923-978)
// whose SiLU-gate epilogue writes the quantised operand of a following W4A4 GEMM (e2m1 bytes [M, N/2] + tiled
// scales, quantiser input scale q_out_input_scale) instead of the bf16 activation: the same bytes as
// silu_mul_split_packed followed by the activation quantiser.  Tensor-core path only; -1 when the shape cannot take it.
int fp4_linear_w4a16_silu_quantized(uint8_t *q_out, uint8_t *q_out_sf, float q_out_input_scale, const uint16_t *x, int ldx,
                                    const glmasr_fp4_weight *gate_up, int M, int K) {
    if (q_out == nullptr || q_out_sf == nullptr || x == nullptr || gate_up == nullptr || !(q_out_input_scale > 0.0f)) return -1;
    if (gate_up[0].w_scales == nullptr || gate_up[1].w_scales == nullptr || gate_up[0].N != gate_up[1].N || ldx < K) return -1;
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = GEMM_W4A16;
    a.out = nullptr;                 // the epilogue writes q_out only
    a.ldo = gate_up[0].N;
    a.x = (const __nv_bfloat16 *)x;
    a.ldx = ldx;
    a.w = gate_up;
    a.num_w = 2;
    a.epi = EPI_SILU_GATE;
    a.M = M;
    a.K = K;
    a.q_out = q_out;
    a.q_out_sf = q_out_sf;
    a.q_out_input_scale = q_out_input_scale;
    return run_fused(a);
}

// bf16 GEMM with the epilogues of the audio encoder: out[M, sum N_i] = epilogue(x[M, K] * concat_i(w_i[N_i, K])^T)
// for up to three weight tensors that share the input (q | k | v without copying them together), bias indexed by
// output column.  epi: EPI_STORE (+ bias), EPI_GELU (bias, tanh-GELU), EPI_RESIDUAL (bf16(bf16(acc) + bias) + residual,
// residual row pitch ldo).  x row pitch ldx, out row pitch ldo.  Returns 0, or -1 when the shape cannot run on
// the tensor-core path (K % 64, 16-byte alignment).
int bf16_linear_ex(uint16_t *out, int ldo, const uint16_t *x, int ldx, const uint16_t *const *w, const int *n, int num_w,
                   const uint16_t *bias, int epi, const uint16_t *residual, int M, int K) {
    if (out == nullptr || x == nullptr || w == nullptr || n == nullptr || num_w < 1 || num_w > kMaxSegments || M <= 0 || K <= 0)
        return -1;
    if (epi == EPI_RESIDUAL && residual == nullptr) return -1;
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = GEMM_BF16;
    a.out = (__nv_bfloat16 *)out;
    a.ldo = ldo;
    a.x = (const __nv_bfloat16 *)x;
    a.ldx = ldx;
    for (int i = 0; i < num_w; ++i) {
        if (w[i] == nullptr || n[i] <= 0) return -1;
        a.w_bf16[i] = (const __nv_bfloat16 *)w[i];
        a.n_bf16[i] = n[i];
    }
    a.num_w = num_w;
    a.epi = epi;
    a.bias = (const __nv_bfloat16 *)bias;
    a.residual = (const __nv_bfloat16 *)residual;
    a.M = M;
    a.K = K;
    if (ldo < total_out_cols(a) || ldx < K) return -1;
    if (!tensor_core_eligible(a)) return -1;
    return run_fused(a);
}

}  // namespace glmasr

using namespace glmasr;

// ============================================================================================
// 1. reference symbols
// ============================================================================================
extern "C" void fp4_dequant_to_bf16(uint16_t *out, const uint8_t *packed_w, const uint8_t *block_scales,
                                    float global_scale, int rows, int cols) {
    launch_dequant((__nv_bfloat16 *)out, packed_w, block_scales, global_scale, rows, cols, g_stream);
    ++g_launches;
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

extern "C" void fp4_linear(void *handle, uint16_t *out, uint16_t *weight_scratch, uint16_t *prequant_scratch,
                           const uint16_t *x, const uint8_t *w_packed, const uint8_t *w_scales, float w_global_scale,
                           const uint16_t *pre_quant_scale, const uint16_t *bias, int M, int N, int K) {
    (void)handle;
    if (M <= 0 || N <= 0 || K <= 0) return;   // the reference launches empty grids here
    glmasr_fp4_weight w = {w_packed, w_scales, w_global_scale, N};
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = GEMM_W4A16;
    a.out = (__nv_bfloat16 *)out;
    a.ldo = N;
    a.x = (const __nv_bfloat16 *)x;
    a.ldx = K;
    a.w = &w;
    a.num_w = 1;
    a.pre = (const __nv_bfloat16 *)pre_quant_scale;
    a.prequant_scratch = (__nv_bfloat16 *)prequant_scratch;
    a.weight_scratch = (__nv_bfloat16 *)weight_scratch;
    a.epi = EPI_STORE;
    a.bias = (const __nv_bfloat16 *)bias;
    a.M = M;
    a.K = K;
    GLMASR_CHECK(run_fused(a) == 0, "fp4_linear failed (M=%d N=%d K=%d)", M, N, K);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

extern "C" int nvfp4_cutlass_available(void) { return 1; }

extern "C" int nvfp4_linear(void *handle, uint16_t *out, uint16_t *dequant_buf, const uint16_t *x,
                            const uint8_t *w_packed, const uint8_t *w_scales, float input_scale, float w_global_scale,
                            const uint16_t *pre_quant_scale, const uint16_t *bias, int M, int N, int K) {
    (void)handle;
    (void)dequant_buf;
    (void)bias;
    if (M <= 0 || N <= 0 || K <= 0) return -1;
    if (w_scales == nullptr) return -1;
    if ((K % 16) != 0) return -1;
    if (!(input_scale > 0.0f)) return -1;
    glmasr_fp4_weight w = {w_packed, w_scales, w_global_scale, N};
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = GEMM_W4A4;
    a.out = (__nv_bfloat16 *)out;
    a.ldo = N;
    a.x = (const __nv_bfloat16 *)x;
    a.ldx = K;
    a.w = &w;
    a.num_w = 1;
    a.input_scale = input_scale;
    a.pre = (const __nv_bfloat16 *)pre_quant_scale;
    a.epi = EPI_STORE;
    a.M = M;
    a.K = K;
    return run_fused(a);
}

extern "C" void bf16_linear(void *handle, uint16_t *out, const uint16_t *x, const uint16_t *w, const uint16_t *bias,
                            int M, int N, int K) {
    (void)handle;
    if (M <= 0 || N <= 0 || K <= 0) return;
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = GEMM_BF16;
    a.out = (__nv_bfloat16 *)out;
    a.ldo = N;
    a.x = (const __nv_bfloat16 *)x;
    a.ldx = K;
    a.w_bf16[0] = (const __nv_bfloat16 *)w;
    a.n_bf16[0] = N;
    a.num_w = 1;
    a.epi = EPI_STORE;
    a.bias = (const __nv_bfloat16 *)bias;
    a.M = M;
    a.K = K;
    GLMASR_CHECK(run_fused(a) == 0, "bf16_linear failed (M=%d N=%d K=%d)", M, N, K);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:71-75, Infer-engine/cuda/kernels.cu:1211-1250: bf16 linear + bias + tanh-GELU.
extern "C" void bf16_linear_gelu(void *handle, uint16_t *out, const uint16_t *x, const uint16_t *w, const uint16_t *bias,
                                 int M, int N, int K) {
    (void)handle;
    if (M <= 0 || N <= 0 || K <= 0) return;
    const uint16_t *ws[1] = {w};
    const int ns[1] = {N};
    GLMASR_CHECK(bf16_linear_ex(out, N, x, K, ws, ns, 1, bias, EPI_GELU, nullptr, M, K) == 0,
                 "bf16_linear_gelu: unsupported shape or alignment (M=%d N=%d K=%d)", M, N, K);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

extern "C" void silu_mul_split_packed(uint16_t *out, const uint16_t *packed_gate_up, int M, int N) {
    launch_silu_split((__nv_bfloat16 *)out, (const __nv_bfloat16 *)packed_gate_up, M, N, g_stream);
    ++g_launches;
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

extern "C" void silu_elementwise_mul(uint16_t *gate, const uint16_t *up, int n) {
    launch_silu_mul((__nv_bfloat16 *)gate, (const __nv_bfloat16 *)up, n, g_stream);
    ++g_launches;
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

extern "C" void residual_add(uint16_t *out, const uint16_t *a, const uint16_t *b, int n) {
    launch_residual_add((__nv_bfloat16 *)out, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, n, g_stream);
    ++g_launches;
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

extern "C" void lm_head_argmax_batched(void *handle, const uint16_t *hidden, const uint16_t *lm_weight, int rows,
                                       int dim, int vocab_size, int *out_tokens_host) {
    if (rows <= 0) return;
    uint16_t *logits = (uint16_t *)workspace_slot(WS_LOGITS, (size_t)rows * vocab_size * 2);
    int *tokens = (int *)workspace_slot(WS_TOKENS, (size_t)rows * sizeof(int));
    bf16_linear(handle, logits, hidden, lm_weight, nullptr, rows, vocab_size, dim);
    launch_argmax_rows((const __nv_bfloat16 *)logits, tokens, rows, vocab_size, g_stream);
    ++g_launches;
    GLMASR_CUDA_CHECK(cudaGetLastError());
    GLMASR_CUDA_CHECK(cudaMemcpyAsync(out_tokens_host, tokens, (size_t)rows * sizeof(int), cudaMemcpyDeviceToHost, g_stream));
    GLMASR_CUDA_CHECK(cudaStreamSynchronize(g_stream));
}

extern "C" void lm_head_cleanup(void) {
    GLMASR_CUDA_CHECK(cudaStreamSynchronize(g_stream));
    for (int s : {(int)WS_LOGITS, (int)WS_TOKENS}) {
        if (g_ws[s]) GLMASR_CUDA_CHECK(cudaFree(g_ws[s]));
        g_ws[s] = nullptr;
        g_ws_bytes[s] = 0;
    }
}

// ============================================================================================
// 2. additive entry points
// ============================================================================================
extern "C" int glmasr_fp4_linear_fused(int mode, uint16_t *out, int ldo, const uint16_t *x, int ldx,
                                       const glmasr_fp4_weight *weights, int num_weights, float input_scale,
                                       const uint16_t *pre_quant_scale, uint16_t *prequant_scratch, int epilogue,
                                       const uint16_t *residual, int M, int K) {
    if (mode != GLMASR_MODE_W4A4 && mode != GLMASR_MODE_W4A16) return -1;
    if (out == nullptr || x == nullptr || weights == nullptr) return -1;
    if (epilogue < 0 || epilogue > 2) return -1;
    if (mode == GLMASR_MODE_W4A4) {
        if (!(input_scale > 0.0f)) return -1;
        for (int i = 0; i < num_weights && i < kMaxSegments; ++i)
            if (weights[i].w_scales == nullptr) return -1;
    }
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    a.mode = mode == GLMASR_MODE_W4A4 ? GEMM_W4A4 : GEMM_W4A16;
    a.out = (__nv_bfloat16 *)out;
    a.ldo = ldo;
    a.x = (const __nv_bfloat16 *)x;
    a.ldx = ldx;
    a.w = weights;
    a.num_w = num_weights;
    a.input_scale = input_scale;
    a.pre = (const __nv_bfloat16 *)pre_quant_scale;
    a.prequant_scratch = (__nv_bfloat16 *)prequant_scratch;
    a.epi = epilogue;
    a.residual = (const __nv_bfloat16 *)residual;
    a.M = M;
    a.K = K;
    if (ldo < total_out_cols(a) || ldx < K) return -1;
    return run_fused(a);
}

extern "C" int glmasr_fp4_prepack(const uint8_t *w_scales, int N, int K) {
    if (w_scales == nullptr || N <= 0 || K <= 0 || (K % 16) != 0) return -1;
    return prepacked_scales(w_scales, N, K) != nullptr ? 0 : -1;
}

extern "C" void glmasr_fp4_forget(const void *w_scales) {
    cudaStreamSynchronize(g_stream);
    tail_forget_scales(w_scales);
    drop_resident(w_scales);
    auto it = g_prepack.find(w_scales);
    if (it == g_prepack.end()) return;
    cudaFree(it->second.tiled);
    g_prepack.erase(it);
}

extern "C" int glmasr_quantize_bf16_to_fp4(uint8_t *packed_out, uint8_t *scale_out, const uint16_t *x,
                                           const uint16_t *pre_quant_scale, float input_scale, int M, int K) {
    if (M <= 0 || K <= 0 || (K % 16) != 0 || !(input_scale > 0.0f)) return -1;
    if (packed_out == nullptr || scale_out == nullptr || x == nullptr) return -1;
    if (!aligned16(x) || ((uintptr_t)packed_out & 7) != 0) return -1;
    launch_quantize_act(packed_out, scale_out, nullptr, (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)pre_quant_scale,
                        input_scale, M, K, K, g_stream);
    ++g_launches;
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int glmasr_swizzle_rowwise_scales(uint8_t *dst, const uint8_t *src, int rows, int cols) {
    if (dst == nullptr || src == nullptr || rows <= 0 || cols <= 0) return -1;
    const size_t bytes = (size_t)((rows + 127) / 128 * 128) * (size_t)((cols + 3) / 4 * 4);
    if (cudaMemsetAsync(dst, 0, bytes, g_stream) != cudaSuccess) return -1;
    launch_swizzle_scales(dst, src, rows, cols, g_stream);
    ++g_launches;
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

extern "C" int glmasr_argmax_rows(const uint16_t *logits, int *out_tokens, int rows, int vocab) {
    if (logits == nullptr || out_tokens == nullptr || rows <= 0 || vocab <= 0) return -1;
    launch_argmax_rows((const __nv_bfloat16 *)logits, out_tokens, rows, vocab, g_stream);
    ++g_launches;
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// True when gate|up (K = H, 2 x F columns, SiLU-gate) at M rows runs on the CTA-pair kernel, whose
// epilogue can emit the down projection's quantised operand.  Mirrors the selection in run_fused.
static bool silu_quant_fusable(int M, int H, int F) {
    if (force_simt() || !use_pair_kernel() || no_fused_act_quant()) return false;
    if (M < 512 || (H % 256) != 0 || (F % 256) != 0) return false;
    const int m_pairs = ((M + 127) / 128 + 1) / 2;
    return m_pairs * ((F + 127) / 128) >= num_sms() / 2;
}

static int layer_proj_device(int mode, uint16_t *hidden_out, const uint16_t *hidden_in, const glmasr_layer_weights *lw,
                             int M) {
    const int H = lw->hidden, F = lw->ffn;
    const int nqkv = lw->q.N + lw->k.N + lw->v.N;
    if (lw->q.N != H || lw->o.N != H || lw->down.N != H || lw->gate.N != F || lw->up.N != F) return -1;
    uint16_t *qkv = (uint16_t *)workspace_slot(WS_L_QKV, (size_t)M * nqkv * 2);
    uint16_t *h1 = (uint16_t *)workspace_slot(WS_L_H1, (size_t)M * H * 2);
    uint16_t *act = (uint16_t *)workspace_slot(WS_L_ACT, (size_t)M * F * 2);
    const glmasr_fp4_weight qkvw[3] = {lw->q, lw->k, lw->v};
    const glmasr_fp4_weight gu[2] = {lw->gate, lw->up};
    int rc = glmasr_fp4_linear_fused(mode, qkv, nqkv, hidden_in, H, qkvw, 3, lw->in_qkv, nullptr, nullptr,
                                     GLMASR_EPI_STORE, nullptr, M, H);
    if (rc != 0) return rc;
    // attention stand-in: the q slice of the fused output (row pitch nqkv) feeds o_proj
    rc = glmasr_fp4_linear_fused(mode, h1, H, qkv, nqkv, &lw->o, 1, lw->in_o, nullptr, nullptr, GLMASR_EPI_RESIDUAL,
                                 hidden_in, M, H);
    if (rc != 0) return rc;
    if (mode == GLMASR_MODE_W4A4 && silu_quant_fusable(M, H, F) && lw->in_down > 0.0f && lw->gate.w_scales != nullptr &&
        lw->up.w_scales != nullptr && lw->down.w_scales != nullptr && lw->in_gate_up > 0.0f) {
        // gate|up's SiLU-gate epilogue quantises its result for the down projection (the same bytes
        // the stand-alone quantiser would produce from the bf16 activation), so the bf16
        // intermediate is never written and the separate quantiser launch is gone
        uint8_t *aq = (uint8_t *)workspace_slot(WS_L_ACTQ, (size_t)M * F / 2);
        uint8_t *asf = (uint8_t *)workspace_slot(WS_L_ACTSF, tiled_sf_bytes(M, F));
        FusedArgs g;
        memset(&g, 0, sizeof(g));
        g.mode = GEMM_W4A4;
        g.out = (__nv_bfloat16 *)act;
        g.ldo = F;
        g.x = (const __nv_bfloat16 *)h1;
        g.ldx = H;
        g.w = gu;
        g.num_w = 2;
        g.input_scale = lw->in_gate_up;
        g.epi = EPI_SILU_GATE;
        g.M = M;
        g.K = H;
        g.q_out = aq;
        g.q_out_sf = asf;
        g.q_out_input_scale = lw->in_down;
        rc = run_fused(g);
        if (rc != 0) return rc;
        FusedArgs d;
        memset(&d, 0, sizeof(d));
        d.mode = GEMM_W4A4;
        d.out = (__nv_bfloat16 *)hidden_out;
        d.ldo = H;
        d.ldx = F;
        d.xq = aq;
        d.xq_sf = asf;
        d.w = &lw->down;
        d.num_w = 1;
        d.input_scale = lw->in_down;
        d.epi = EPI_RESIDUAL;
        d.residual = (const __nv_bfloat16 *)h1;
        d.M = M;
        d.K = F;
        return run_fused(d);
    }
    rc = glmasr_fp4_linear_fused(mode, act, F, h1, H, gu, 2, lw->in_gate_up, nullptr, nullptr, GLMASR_EPI_SILU_GATE,
                                 nullptr, M, H);
    if (rc != 0) return rc;
    return glmasr_fp4_linear_fused(mode, hidden_out, H, act, F, &lw->down, 1, lw->in_down, nullptr, nullptr,
                                   GLMASR_EPI_RESIDUAL, h1, M, F);
}

extern "C" int glmasr_fp4_layer_proj(int mode, uint16_t *hidden_out, const uint16_t *hidden_in,
                                     const glmasr_layer_weights *lw, int M) {
    if (hidden_out == nullptr || hidden_in == nullptr || lw == nullptr || M <= 0) return -1;
    return layer_proj_device(mode, hidden_out, hidden_in, lw, M);
}

// Host-buffer call: the rows are independent, so the call is cut into row chunks and the three
// legs of consecutive chunks overlap -- chunk i+1 crosses PCIe host->device while chunk i is
// computed and chunk i-1 goes device->host (the link is full duplex).  Same bytes as one pass.
static cudaStream_t g_copy_in = nullptr, g_copy_out = nullptr;
static constexpr int kMaxHostChunks = 16;
static cudaEvent_t g_ev_in[kMaxHostChunks], g_ev_done[kMaxHostChunks];

static int host_chunks(int M) {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("GLMASR_HOST_CHUNKS");
        v = (e && e[0]) ? atoi(e) : 8;
        if (v < 1) v = 1;
        if (v > kMaxHostChunks) v = kMaxHostChunks;
    }
    return M >= 2048 ? v : 1;
}

extern "C" int glmasr_fp4_layer_proj_host(int mode, uint16_t *hidden_out_host, const uint16_t *hidden_in_host,
                                          const glmasr_layer_weights *lw, int M) {
    if (hidden_out_host == nullptr || hidden_in_host == nullptr || lw == nullptr || M <= 0) return -1;
    const size_t row_bytes = (size_t)lw->hidden * 2;
    const size_t bytes = (size_t)M * row_bytes;
    uint8_t *din = (uint8_t *)workspace_slot(WS_L_IN, bytes);
    uint8_t *dout = (uint8_t *)workspace_slot(WS_L_OUT, bytes);
    const int chunks = host_chunks(M);
    if (chunks == 1) {
        if (cudaMemcpyAsync(din, hidden_in_host, bytes, cudaMemcpyHostToDevice, g_stream) != cudaSuccess) return -1;
        const int rc = layer_proj_device(mode, (uint16_t *)dout, (const uint16_t *)din, lw, M);
        if (rc != 0) return rc;
        if (cudaMemcpyAsync(hidden_out_host, dout, bytes, cudaMemcpyDeviceToHost, g_stream) != cudaSuccess) return -1;
        return cudaStreamSynchronize(g_stream) == cudaSuccess ? 0 : -1;
    }
    if (g_copy_in == nullptr) {
        if (cudaStreamCreateWithFlags(&g_copy_in, cudaStreamNonBlocking) != cudaSuccess) return -1;
        if (cudaStreamCreateWithFlags(&g_copy_out, cudaStreamNonBlocking) != cudaSuccess) return -1;
        for (int i = 0; i < kMaxHostChunks; ++i) {
            if (cudaEventCreateWithFlags(&g_ev_in[i], cudaEventDisableTiming) != cudaSuccess) return -1;
            if (cudaEventCreateWithFlags(&g_ev_done[i], cudaEventDisableTiming) != cudaSuccess) return -1;
        }
    }
    // whole 256-row tile pairs per chunk
    int rows_per = ((M + chunks - 1) / chunks + 255) / 256 * 256;
    // everything queued so far on the compute stream (it may still use the staging buffers) comes first
    if (cudaEventRecord(g_ev_done[0], g_stream) != cudaSuccess) return -1;
    if (cudaStreamWaitEvent(g_copy_in, g_ev_done[0], 0) != cudaSuccess) return -1;
    int n = 0;
    for (int r0 = 0; r0 < M; r0 += rows_per, ++n) {
        const int rows = M - r0 < rows_per ? M - r0 : rows_per;
        const size_t off = (size_t)r0 * row_bytes;
        if (cudaMemcpyAsync(din + off, (const uint8_t *)hidden_in_host + off, (size_t)rows * row_bytes,
                            cudaMemcpyHostToDevice, g_copy_in) != cudaSuccess)
            return -1;
        if (cudaEventRecord(g_ev_in[n], g_copy_in) != cudaSuccess) return -1;
    }
    n = 0;
    for (int r0 = 0; r0 < M; r0 += rows_per, ++n) {
        const int rows = M - r0 < rows_per ? M - r0 : rows_per;
        const size_t off = (size_t)r0 * row_bytes;
        if (cudaStreamWaitEvent(g_stream, g_ev_in[n], 0) != cudaSuccess) return -1;
        g_route_rows = M;
        g_pdl_suppressed = true;    // kernels of one chunk overlapping the next chunk's copy-in wait measured slower
        const int rc = layer_proj_device(mode, (uint16_t *)(dout + off), (const uint16_t *)(din + off), lw, rows);
        g_pdl_suppressed = false;
        g_route_rows = 0;
        if (rc != 0) return rc;
        if (cudaEventRecord(g_ev_done[n], g_stream) != cudaSuccess) return -1;
        if (cudaStreamWaitEvent(g_copy_out, g_ev_done[n], 0) != cudaSuccess) return -1;
        if (cudaMemcpyAsync((uint8_t *)hidden_out_host + off, dout + off, (size_t)rows * row_bytes,
                            cudaMemcpyDeviceToHost, g_copy_out) != cudaSuccess)
            return -1;
    }
    if (cudaStreamSynchronize(g_copy_out) != cudaSuccess) return -1;
    return cudaStreamSynchronize(g_stream) == cudaSuccess ? 0 : -1;
}

// ============================================================================================
// W4A4 linear that allocates nothing
// ============================================================================================
// Scratch of the no-allocation entry point: quantised activations, their tiled scales and the
// re-tiled weight scales.  Lives in the library image, so every GPU that loads the library
// holds these bytes until the process exits.
static constexpr int kNoAllocMaxM = 512;                        // rows of x
static constexpr int kNoAllocMaxK = 8192;                       // reduction length
static constexpr long long kNoAllocMaxWeight = 32ll << 20;      // ceil128(N) * K elements
static constexpr size_t kNoAllocXq = (size_t)kNoAllocMaxM * kNoAllocMaxK / 2;                    // 2 MiB
static constexpr size_t kNoAllocXsf = (size_t)(kNoAllocMaxM / 128) * (kNoAllocMaxK / 64) * 512;  // 256 KiB
static constexpr size_t kNoAllocWsf = (size_t)(kNoAllocMaxWeight / 16);                          // 2 MiB
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocXq + kNoAllocXsf + kNoAllocWsf];
// Status word of this entry point's kernels (a bounded wait that ran out records its code here).  It cannot
// share the library's ordinary status word, which is allocated on first use; glmasr_fp4_status reads both.
static __device__ int g_noalloc_status[4];

static uint8_t *g_noalloc_ptr[kMaxDevices] = {nullptr};
static int *g_noalloc_status_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device.  The array's name is only a
// host-side handle; the address a kernel can use comes from cudaGetSymbolAddress, once per device.
static uint8_t *noalloc_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (g_noalloc_ptr[dev] == nullptr) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) {
            fprintf(stderr, "glmasr_nvfp4_linear_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            return nullptr;
        }
        void *sptr = nullptr;
        const cudaError_t e2 = cudaGetSymbolAddress(&sptr, g_noalloc_status);
        if (e2 != cudaSuccess) {
            fprintf(stderr, "glmasr_nvfp4_linear_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e2));
            return nullptr;
        }
        if (!g_umma_ready[dev]) {           // the kernels' shared-memory opt-in is per device
            if (umma_gemm_init() != cudaSuccess) return nullptr;
            g_umma_ready[dev] = true;
        }
        (void)num_sms();
        (void)encode_fn();
        g_noalloc_status_ptr[dev] = (int *)sptr;
        g_noalloc_ptr[dev] = (uint8_t *)ptr;
    }
    return g_noalloc_ptr[dev];
}

extern "C" int glmasr_nvfp4_linear_noalloc(uint16_t *out, const uint16_t *x, const uint8_t *w_packed,
                                           const uint8_t *w_scales, float input_scale, float w_global_scale,
                                           int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || out == nullptr || x == nullptr || w_packed == nullptr || w_scales == nullptr)
        return -1;
    if (!(input_scale > 0.0f)) return -1;
    const long long n_pad = ((long long)N + 127) / 128 * 128;
    if (M > kNoAllocMaxM || K > kNoAllocMaxK || n_pad * K > kNoAllocMaxWeight) {
        fprintf(stderr,
                "glmasr_nvfp4_linear_noalloc: M=%d N=%d K=%d exceeds the built-in scratch "
                "(M <= %d, K <= %d, ceil128(N)*K <= %lld); use nvfp4_linear instead\n",
                M, N, K, kNoAllocMaxM, kNoAllocMaxK, kNoAllocMaxWeight);
        return -1;
    }
    if (K % 256 != 0 || !aligned16(x) || !aligned16(out) || !aligned16(w_packed) || !aligned16(w_scales) || (N % 8) != 0) {
        fprintf(stderr, "glmasr_nvfp4_linear_noalloc: needs K %% 256 == 0, N %% 8 == 0 and 16-byte aligned pointers\n");
        return -1;
    }
    uint8_t *scratch = noalloc_scratch_for_current_device();
    if (scratch == nullptr) return -1;
    uint8_t *xq = scratch;
    uint8_t *xsf = scratch + kNoAllocXq;
    uint8_t *wsf = scratch + kNoAllocXq + kNoAllocXsf;

    // the re-tiled weight scales must be zero where no real scale lands (rows past N)
    if (cudaMemsetAsync(wsf, 0, tiled_sf_bytes(N, K), g_stream) != cudaSuccess) return -1;
    launch_swizzle_scales(wsf, w_scales, N, K / 16, g_stream);
    ++g_launches;
    launch_quantize_act(xq, nullptr, xsf, (const __nv_bfloat16 *)x, nullptr, input_scale, M, K, K, g_stream);
    ++g_launches;

    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = M;
    p.K = K;
    p.out = (__nv_bfloat16 *)out;
    p.ldo = N;
    p.epi = EPI_STORE;
    p.status = g_noalloc_status_ptr[current_device()];
    p.num_m_tiles = (M + 127) / 128;
    p.n_out = N;
    p.num_segs = 1;
    p.seg_rows[0] = N;
    p.seg_subtiles[0] = (N + 127) / 128;
    p.alpha[0] = input_scale * w_global_scale;
    p.sfa = xsf;
    p.sfb[0] = wsf;
    p.num_k_blocks = K / 256;
    p.sf_k_chunks = K / 64;
    if (!make_tmap(&p.tm_a, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, 128, 128, true))
        return -1;
    if (!make_tmap(&p.tm_b[0], w_packed, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, 128,
                   128, true))
        return -1;
    const int subtiles = p.seg_subtiles[0];
    const int tiles2 = p.num_m_tiles * ((subtiles + 1) / 2);
    const int nb = (subtiles >= 2 && tiles2 >= num_sms()) ? 2 : 1;
    p.num_n_tiles = (subtiles + nb - 1) / nb;
    const int total_tiles = p.num_m_tiles * p.num_n_tiles;
    const int ctas = total_tiles < num_sms() ? total_tiles : num_sms();
    if (launch_umma_gemm(GEMM_W4A4, nb, p, ctas, g_stream) != cudaSuccess) return -1;
    ++g_launches;
    return 0;
}

extern "C" int glmasr_fp4_status(void) {
    int host[4] = {0, 0, 0, 0};
    if (cudaStreamSynchronize(g_stream) != cudaSuccess) return -1;
    int code = 0;
    if (g_status != nullptr) {
        if (cudaMemcpy(host, g_status, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
        if (host[0] != 0) cudaMemset(g_status, 0, sizeof(host));
        code = host[0];
    }
    // the no-allocation entry point reports through a word inside the library image
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_noalloc_status_ptr[dev] != nullptr) {
        if (cudaMemcpy(host, g_noalloc_status_ptr[dev], sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
        if (host[0] != 0) cudaMemset(g_noalloc_status_ptr[dev], 0, sizeof(host));
        if (code == 0) code = host[0];
    }
    return code;
}

extern "C" long long glmasr_launch_count(void) { return g_launches; }

#ifdef GLMASR_EXPERIMENTS
// experiment builds only: switch the kernels' experiment flags (wrong results by design; -1 = back to the environment's)
extern "C" void glmasr_debug_set_flags(int flags) { g_debug_override = flags; }

// experiment builds only: copy the per-CTA cycle counters of the last instrumented GEMM launch
extern "C" int glmasr_debug_cycles(unsigned long long *host_out, int max_ctas) {
    if (g_ws[WS_DBG] == nullptr) return 0;
    cudaStreamSynchronize(g_stream);
    const int n = max_ctas < 148 ? max_ctas : 148;
    if (cudaMemcpy(host_out, g_ws[WS_DBG], (size_t)n * 16 * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return n;
}
#endif

extern "C" void glmasr_profile_enable(int on) {
    g_profile = on != 0;
    if (!g_profile) {
        for (auto &t : g_timed) {
            cudaEventDestroy(t.start);
            cudaEventDestroy(t.stop);
        }
        g_timed.clear();
    }
}

extern "C" int glmasr_profile_read(int max_entries, double *ms, double *flops, double *bytes) {
    if (cudaStreamSynchronize(g_stream) != cudaSuccess) return -1;
    int n = 0;
    for (auto &t : g_timed) {
        if (n < max_entries) {
            float f = 0.0f;
            cudaEventElapsedTime(&f, t.start, t.stop);
            ms[n] = f;
            flops[n] = t.flops;
            bytes[n] = t.bytes;
            ++n;
        }
        cudaEventDestroy(t.start);
        cudaEventDestroy(t.stop);
    }
    g_timed.clear();
    return n;
}

extern "C" void glmasr_set_stream(void *cuda_stream) { g_stream = (cudaStream_t)cuda_stream; }

extern "C" void glmasr_fp4_cleanup(void) { free_all_private_state(); }
