// The resident part of a decoder layer at decode batch sizes (M <= 256 rows), as ONE co-resident kernel:
// o projection + residual -> RMSNorm + activation quantiser -> gate|up + SiLU-gate + quantiser ->
// down + residual -> (next layer's) RMSNorm + quantiser -> (next layer's) q|k|v.  See decode_tail.cu.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glmasr {

enum : int { TAIL_GEMM = 0, TAIL_NORM = 1 };
enum : int {
    TAIL_EPI_STORE = 0,       // out[m, n] = bf16(acc * alpha_seg)
    TAIL_EPI_RESIDUAL = 1,    // out[m, n] = bf16(float(bf16(acc * alpha)) + float(out[m, n]))   (in place)
    TAIL_EPI_SILU_QUANT = 2,  // segments 0 / 1 = gate / up; silu(bf16(g)) * bf16(u), rounded to bf16, quantised in
                              // 16-column blocks into the next GEMM's operand (e2m1 bytes + 128x4-tiled scales)
};

constexpr int kTailMaxPhases = 6;
constexpr int kTailMaxGemms = 4;
constexpr int kTailMaxNorms = 2;
constexpr int kTailMaxSegs = 3;
constexpr int kTailCounterStride = 32;   // unsigned ints between the arrival counters of two phases (one 128-byte line each)
constexpr int kTailCounterBytes = kTailMaxPhases * kTailCounterStride * 4;
constexpr int kTailMaxRunUnits = 3;     // 32-column units per run of one CTA (bounded by the shared-memory stage layout)

// One W4A4 GEMM phase: out[M, sum N_s] = xq[M, K] * concat_s(W_s[N_s, K])^T over up to three weight tensors.
struct alignas(64) TailGemm {
    CUtensorMap tm_a;                    // quantised activations: bytes [M, K/2], 128-row x 128-byte boxes, 128B swizzle
    CUtensorMap tm_w[kTailMaxSegs];      // packed e2m1 weights: bytes [N_s, K/2], 32-row x 128-byte boxes, 128B swizzle
    const uint8_t *sfa;                  // activation scales, 128x4-tiled
    const uint8_t *sfb[kTailMaxSegs];    // weight scales re-tiled per CTA of this phase (tail_tiled_scales)
    float alpha[kTailMaxSegs];           // input_scale * per-tensor weight scale
    int seg_units[kTailMaxSegs];         // N_s / 32
    int num_segs;
    int K;                               // multiple of 256
    int cpm;                             // CTAs per row tile that share this phase's columns (<= grid / num_m_tiles)
    int epi;
    int res_local;                       // TAIL_EPI_RESIDUAL: out was last written by an earlier launch, or earlier in this one
                                         // by the very threads that now read it (same columns, same cpm): no acquire needed
    int ldo;                             // row pitch of out, elements
    __nv_bfloat16 *out;
    uint8_t *q_packed;                   // TAIL_EPI_SILU_QUANT: bytes [M, q_ld]
    uint8_t *q_sf;                       //                      tiled scales, q_sf_chunks 512-byte chunks per 128 rows
    float q_inv_in;                      //                      1 / input_scale of the consuming GEMM
    int q_ld;
    int q_sf_chunks;
};

// RMSNorm (reference arithmetic and summation order) + activation quantiser over the rows of x [M, dim].
struct TailNorm {
    const __nv_bfloat16 *x;
    const __nv_bfloat16 *weight;
    uint8_t *q_packed;                   // bytes [M, dim / 2]
    uint8_t *q_sf;                       // tiled scales, dim / 64 chunks per 128 rows
    float eps;
    float inv_in;
    int dim;                             // multiple of 64, at most 4096
};

struct alignas(64) TailParams {
    TailGemm g[kTailMaxGemms];
    TailNorm n[kTailMaxNorms];
    int kind[kTailMaxPhases];            // TAIL_GEMM / TAIL_NORM, in execution order
    int index[kTailMaxPhases];           // which g[] / n[]
    int num_phases;
    int M;
    int num_m_tiles;
    unsigned int *counter;               // kTailCounterBytes: one grid-wide arrival counter per phase, see decode_tail.cu
    unsigned int base;                   // their value when this launch starts (every launch adds the grid size to each)
    int *status;
    int debug;                           // experiment builds only (timing experiments that leave work out)
    unsigned long long *dbg;             // experiment builds only: cycle counters [grid][kTailMaxPhases][16]
};

// CTAs per row tile that share a phase of `units` 32-column units per row tile (one of the two tensors for
// TAIL_EPI_SILU_QUANT) on `grid` CTAs over `num_m_tiles` row tiles, subject to at most kTailMaxRunUnits units per
// run of a CTA.  0: the phase cannot be split that way.
int tail_choose_cpm(int units, int K, bool silu, int grid, int num_m_tiles);
int tail_grid_size();                    // CTAs of a launch on the current device (one per SM)
// The scales [N, K/16] of one weight tensor of a GEMM phase, re-tiled for that phase's split over cpm = grid /
// num_m_tiles CTAs per row tile: total_units = 32-column units of the whole phase (of one of the two tensors for
// TAIL_EPI_SILU_QUANT), seg_first = this tensor's first unit among them.  Built once and cached; nullptr if the
// shape is not covered.  tail_forget_scales(ptr) drops the copies made from one scale tensor (nullptr: all).
const uint8_t *tail_tiled_scales(const uint8_t *w_scales, int N, int K, int cpm, int total_units, int seg_first, cudaStream_t st);
void tail_forget_scales(const void *w_scales);
// Cooperative launch (all CTAs co-resident).  Advances nothing on the host: the caller adds tail_grid_size() to
// `base` for the next launch on the same counters.
cudaError_t launch_decode_tail(const TailParams &p, cudaStream_t st);

}  // namespace glmasr
