// Parameters and launcher of the tcgen05 GEMM behind every FP4 linear (see gemm_umma.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glmasr {

enum GemmMode : int {
    GEMM_W4A4 = 0,   // e2m1 weights x e2m1 activations, block-scaled MMA (reference nvfp4_linear semantics)
    GEMM_W4A16 = 1,  // e2m1 weights dequantised in-kernel x bf16 activations (reference fp4_linear semantics)
    GEMM_BF16 = 2,   // bf16 weights x bf16 activations (reference bf16_linear semantics, e.g. lm_head)
};

enum EpilogueMode : int {
    EPI_STORE = 0,      // out[m, n] = bf16(acc * alpha_seg (+ bias[n]))
    EPI_SILU_GATE = 1,  // segments 0/1 = gate/up: out[m, n] = bf16(silu(bf16(g)) * bf16(u))
    EPI_RESIDUAL = 2,   // out[m, n] = bf16(float(bf16(acc * alpha)) + float(residual[m, n])); with a bias:
                        // bf16(float(bf16(float(bf16(acc * alpha)) + bias[n])) + float(residual[m, n]))
    EPI_GELU = 3,       // out[m, n] = bf16(gelu_tanh(acc * alpha_seg + bias[n]))   (single-CTA kernel only)
};

static constexpr int kMaxSegments = 3;

// Timing experiments (per-role cycle counters, branches that leave work out and therefore give wrong
// results) exist only in a library built with -DGLMASR_EXPERIMENTS (`make EXPERIMENTS=1`).  In the
// default build every test below is the constant false and the compiler removes the branches.
#ifdef GLMASR_EXPERIMENTS
#define GLMASR_EXP(p, bits) ((((p).debug) & (bits)) != 0)
#else
#define GLMASR_EXP(p, bits) false
#endif

// One launch computes out[M, sum N_s] = x[M, K] * concat_s(W_s[N_s, K])^T for up to three
// weight tensors that share the input (q|k|v, gate|up), each with its own per-tensor scale.
struct alignas(64) GemmParams {
    CUtensorMap tm_a;                   // activations, 128-row x 128-byte boxes, 128B swizzle
    CUtensorMap tm_b[kMaxSegments];     // weights (packed e2m1 bytes, or bf16), same box
    CUtensorMap tm_bs[kMaxSegments];    // W4A16: row-major e4m3 scales [N_s, K/16], 128-row x 16-byte boxes
    CUtensorMap tm_sfa;                 // W4A4 pair kernel: tiled activation scales as [chunks, 128 x u32], 4-chunk boxes
    CUtensorMap tm_sfb[kMaxSegments];   // W4A4 pair kernel: tiled weight scales, same view
    CUtensorMap tm_out;                 // pair kernel: output as [M, n_out] bf16, 32-row x 64-column boxes, 128B swizzle
    int tma_store;                      // 1: the epilogue stages tiles in shared memory and stores them through tm_out
    const uint8_t *sfa;                 // W4A4: activation scales, 128x4-tiled
    const uint8_t *sfb[kMaxSegments];   // W4A4: weight scales, 128x4-tiled
    float alpha[kMaxSegments];          // applied to the fp32 accumulator of that segment
    int seg_rows[kMaxSegments];         // N_s
    int seg_subtiles[kMaxSegments];     // ceil(N_s / 128)
    int num_segs;
    int M, K;
    int n_out;                          // output columns
    int ldo;                            // output (and residual) row pitch in elements
    __nv_bfloat16 *out;
    const __nv_bfloat16 *residual;
    const __nv_bfloat16 *bias;
    int epi;
    // EPI_SILU_GATE only, optional: emit the activation already quantised for the next W4A4 GEMM
    // (e2m1 bytes [M, q_ld] + 128x4-tiled e4m3 scales with q_sf_chunks 512-byte chunks per row
    // tile) instead of bf16.  Same bytes as the stand-alone quantiser run on the bf16 result.
    uint8_t *q_packed;
    uint8_t *q_sf;
    float q_inv_in;                     // 1 / input_scale of the consuming GEMM
    int q_ld;                           // bytes per packed row (= columns / 2)
    int q_sf_chunks;                    // ceil(columns / 64)
    // Split-K (single-CTA kernel, W4A4): every tile is computed by split_k CTAs over disjoint K ranges.
    // Each writes its raw fp32 partial to `partial`; the CTA that finishes last (per-tile counter) adds
    // the partials in split order and runs the epilogue, so the result does not depend on arrival order
    // and no CTA ever waits for another.  split_k <= 1: off.
    // 1: weights and their scales are not written by any kernel still running when this one starts, so the
    // producer may load them before it waits for the preceding kernels (programmatic dependent launch)
    int early_weights;
    int split_k;
    float *partial;                     // [tiles][split_k][128 x BN] fp32, column-quad major
    int *tile_counters;                 // [tiles], zero between launches (the last CTA resets its tile's)
    int num_m_tiles, num_n_tiles;
    // Pair kernel, store / residual epilogues: when the last round of 256 x 256 tiles would occupy at most half of
    // the CTA pairs, each of its tiles is computed as two 256 x 128 halves by two pairs (N = 128 MMAs).
    int split_tail;
    CUtensorMap tm_b_half[kMaxSegments];    // split_tail: the weights again, as 64-row x 128-byte boxes
    int num_k_blocks;                   // K steps of 128 operand bytes per row (W4A4: 256 elements, else 64)
    int sf_k_chunks;                    // W4A4: 512-byte scale chunks per 128-row tile along K (= ceil(K/64))
    int *status;
    int debug;                          // experiment builds only (GLMASR_DEBUG_FLAGS); ignored otherwise
    unsigned long long *dbg_cycles;     // debug & 64: per-CTA cycle counters [gridDim.x][16]
};

// W4A4 on CTA pairs (cta_group::2): 256 x 256 tiles, one cluster of two CTAs per tile.
cudaError_t launch_umma_gemm_pair(const GemmParams &p, int num_pairs, cudaStream_t st);
cudaError_t umma_gemm_pair_init();
// The same kernel on bf16 operands (kind::f16, no scale factors): tm_a / tm_b are the bf16 views, num_k_blocks = K / 64.
cudaError_t launch_umma_gemm_pair_bf16(const GemmParams &p, int num_pairs, cudaStream_t st);
// Same pipeline with sixteen epilogue warps, for the SiLU-gate epilogues (gemm_umma3.cu); tm_out must be
// a 32-row x 32-column, 64B-swizzled view of the output when tma_store is set.
cudaError_t launch_umma_gemm_pair16(const GemmParams &p, int num_pairs, cudaStream_t st);
cudaError_t umma_gemm_pair16_init();

// nb = 128-row weight sub-tiles per CTA tile (1 or 2).  Returns cudaSuccess or the launch error.
cudaError_t launch_umma_gemm(int mode, int nb, const GemmParams &p, int num_ctas, cudaStream_t st);
// Opt in to the large dynamic shared memory carve-out once per process.
cudaError_t umma_gemm_init();
int umma_gemm_threads(int mode, int nb);
int umma_gemm_smem_bytes(int mode, int nb);

}  // namespace glmasr
