// HBM-bound element-wise kernels of the FP4 linear path: whole-weight dequant, pre-quant
// scaling, the bf16 -> FP4 activation quantiser (with the scale swizzle fused in), the scale
// swizzle itself, SiLU-gate, residual add and the batched row arg-max.
//
// Each is bit-exact with the reference kernel it replaces (same fp32 operation order, same
// converters); they differ in that each thread moves 16-32 bytes instead of one element.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdlib.h>

#include "elementwise.cuh"
#include "fp4_format.cuh"
#include "runtime.cuh"

namespace glmasr {

static inline int blocks_for(long long work, int threads) { return (int)((work + threads - 1) / threads); }

// --------------------------------------------------------------------------------------------
// fp4_dequant_to_bf16 (reference: Infer-engine/cuda/kernels.cu:188-246)
//   out[r,c] = bf16( (lut[nibble] * e4m3(scales[r, c/16])) * global )
// One thread per 16-element scale block: 8 packed bytes in, 32 bytes out.
// --------------------------------------------------------------------------------------------
__global__ void dequant_blocks_kernel(__nv_bfloat16 *__restrict__ out, const uint8_t *__restrict__ packed,
                                      const uint8_t *__restrict__ scales, float global, int rows, int cols) {
    const int blocks_per_row = cols >> 4;
    const long long total = (long long)rows * blocks_per_row;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int r = (int)(i / blocks_per_row);
    const int b = (int)(i % blocks_per_row);
    const uint2 w = *reinterpret_cast<const uint2 *>(packed + (size_t)r * (cols >> 1) + (size_t)b * 8);
    const float s = scales ? e4m3_to_float_ref(scales[(size_t)r * blocks_per_row + b]) : 1.0f;
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t word = j < 4 ? w.x : w.y;
        const uint32_t byte = (word >> ((j & 3) * 8)) & 0xFFu;
        const float v0 = (e2m1_to_float(byte & 0xFu) * s) * global;
        const float v1 = (e2m1_to_float(byte >> 4) * s) * global;
        const __nv_bfloat162 p = __floats2bfloat162_rn(v0, v1);
        o[j] = *reinterpret_cast<const uint32_t *>(&p);
    }
    uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)r * cols + (size_t)b * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// Any column count (packed row pitch (cols+1)/2, scale row pitch (cols+15)/16), one element per thread.
__global__ void dequant_generic_kernel(__nv_bfloat16 *__restrict__ out, const uint8_t *__restrict__ packed,
                                       const uint8_t *__restrict__ scales, float global, int rows, int cols) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * cols) return;
    const int r = (int)(idx / cols), c = (int)(idx % cols);
    const uint8_t byte = packed[(size_t)r * ((cols + 1) / 2) + c / 2];
    const uint32_t nib = (c & 1) ? (byte >> 4) : (byte & 0xFu);
    const float s = scales ? e4m3_to_float_ref(scales[(size_t)r * ((cols + 15) / 16) + c / 16]) : 1.0f;
    out[idx] = __float2bfloat16((e2m1_to_float(nib) * s) * global);
}

void launch_dequant(__nv_bfloat16 *out, const uint8_t *packed, const uint8_t *scales, float global, int rows,
                    int cols, cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return;
    const bool aligned = (cols % 16 == 0) && (((uintptr_t)packed & 7) == 0) && (((uintptr_t)out & 15) == 0);
    if (aligned) {
        const long long total = (long long)rows * (cols / 16);
        dequant_blocks_kernel<<<blocks_for(total, 256), 256, 0, st>>>(out, packed, scales, global, rows, cols);
    } else {
        dequant_generic_kernel<<<blocks_for((long long)rows * cols, 256), 256, 0, st>>>(out, packed, scales, global,
                                                                                         rows, cols);
    }
}

// --------------------------------------------------------------------------------------------
// apply_prequant (reference: Infer-engine/cuda/kernels.cu:1280-1295): out = bf16(x[m,k]*pre[k])
// --------------------------------------------------------------------------------------------
__global__ void prequant_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ x,
                                const __nv_bfloat16 *__restrict__ pre, long long total, int K) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int k = (int)(idx % K);
    out[idx] = __float2bfloat16(__bfloat162float(x[idx]) * __bfloat162float(pre[k]));
}

void launch_prequant(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *pre, int M, int K,
                     cudaStream_t st) {
    const long long total = (long long)M * K;
    if (total <= 0) return;
    prequant_kernel<<<blocks_for(total, 256), 256, 0, st>>>(out, x, pre, total, K);
}

// --------------------------------------------------------------------------------------------
// Activation quantiser (reference: Infer-engine/cuda/nvfp4_cutlass.cu:35-87) with the scale
// swizzle (:89-111) fused in.  One thread per 16-element block of one row.
//   amax = max |x*pre| ; scale = (inv_in*amax)/6 ; s8 = e4m3(scale) ; os = inv_in/float(s8)
//   q = e2m1((x*pre)*os) ; byte = lo | hi<<4
// scale_rowmajor (optional) receives the reference's plain [M, K/16] layout; scale_swizzled
// (optional) receives the 128x4-tiled layout the tensor core reads, rows padded to 128.
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ size_t swizzled_sf_index(int r, int c, int col_tiles) {
    const int ty = r >> 7, rem = r & 127;
    return ((((size_t)ty * col_tiles + (c >> 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4 + (c & 3);
}

__global__ void quantize_act_kernel(uint8_t *__restrict__ packed_out, uint8_t *__restrict__ scale_rowmajor,
                                    uint8_t *__restrict__ scale_swizzled, const __nv_bfloat16 *__restrict__ x,
                                    const __nv_bfloat16 *__restrict__ pre, float inv_in, int M, int K, int ldx) {
    pdl_launch_dependents();
    pdl_wait();
    const int blocks_per_row = K >> 4;
    const long long total = (long long)M * blocks_per_row;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int r = (int)(i / blocks_per_row);
    const int b = (int)(i % blocks_per_row);
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)r * ldx + (size_t)b * 16);
    const uint4 a0 = src[0], a1 = src[1];
    const uint32_t w[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    float v[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[2 * j] = __uint_as_float(w[j] << 16);
        v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
    if (pre) {
        const uint4 *ps = reinterpret_cast<const uint4 *>(pre + (size_t)b * 16);
        const uint4 p0 = ps[0], p1 = ps[1];
        const uint32_t pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[2 * j] = v[2 * j] * __uint_as_float(pw[j] << 16);
            v[2 * j + 1] = v[2 * j + 1] * __uint_as_float(pw[j] & 0xFFFF0000u);
        }
    }
    uint32_t lo, hi;
    const uint32_t s8 = quantize_block16(v, inv_in, lo, hi);
    *reinterpret_cast<uint2 *>(packed_out + (size_t)r * (K >> 1) + (size_t)b * 8) = make_uint2(lo, hi);
    if (scale_rowmajor) scale_rowmajor[(size_t)r * blocks_per_row + b] = (uint8_t)s8;
    if (scale_swizzled) scale_swizzled[swizzled_sf_index(r, b, (blocks_per_row + 3) >> 2)] = (uint8_t)s8;
}

// The same quantiser for the common prefill case (no pre-scale, K a multiple of 2048, thousands of rows): a warp
// takes 2048 consecutive elements of a row, reads them once with coalesced 16-byte loads into a private strip of
// shared memory (128-byte lines 144 bytes apart: conflict-free both ways), and every lane then quantises line
// `lane`, i.e. four consecutive blocks: 32 contiguous output bytes and one aligned 4-byte group of scales per lane
// instead of four 8-byte and four 1-byte stores.  Same bytes as quantize_act_kernel.
constexpr int kQuantStrip = 32 * 144;
__global__ void __launch_bounds__(256) quantize_act_strip_kernel(uint8_t *__restrict__ packed_out, uint8_t *__restrict__ scale_rowmajor,
                                                                uint8_t *__restrict__ scale_swizzled,
                                                                const __nv_bfloat16 *__restrict__ x, float inv_in, int M, int K,
                                                                int ldx) {
    __shared__ __align__(16) uint8_t strips[8 * kQuantStrip];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int segs = K >> 11;                                   // 2048-element segments per row
    const long long unit = (long long)blockIdx.x * 8 + wib;
    if (unit >= (long long)M * segs) return;
    const int r = (int)(unit / segs), seg = (int)(unit % segs);
    uint8_t *rs = strips + wib * kQuantStrip;
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)r * ldx + (size_t)seg * 2048);
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = src[k * 32 + lane];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int byte = 512 * k + 16 * lane;
            *reinterpret_cast<uint4 *>(rs + byte + (byte >> 7) * 16) = v[k];
        }
    }
    __syncwarp();
    const int blocks_per_row = K >> 4;
    const int b0 = seg * 128 + 4 * lane;                        // first of this lane's four blocks
    const uint8_t *line = rs + lane * 144;
    uint32_t packed[8], sfw = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float v[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 xv = *reinterpret_cast<const uint4 *>(line + (2 * k + h) * 16);
            const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * h + 2 * j] = __uint_as_float(xs[j] << 16);
                v[8 * h + 2 * j + 1] = __uint_as_float(xs[j] & 0xFFFF0000u);
            }
        }
        const uint32_t s8 = quantize_block16(v, inv_in, packed[2 * k], packed[2 * k + 1]);
        sfw |= (s8 & 0xFFu) << (8 * k);
    }
    uint4 *dst = reinterpret_cast<uint4 *>(packed_out + (size_t)r * (K >> 1) + (size_t)b0 * 8);
    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    if (scale_rowmajor) *reinterpret_cast<uint32_t *>(scale_rowmajor + (size_t)r * blocks_per_row + b0) = sfw;
    if (scale_swizzled) *reinterpret_cast<uint32_t *>(scale_swizzled + swizzled_sf_index(r, b0, (blocks_per_row + 3) >> 2)) = sfw;
}

void launch_quantize_act(uint8_t *packed_out, uint8_t *scale_rowmajor, uint8_t *scale_swizzled,
                         const __nv_bfloat16 *x, const __nv_bfloat16 *pre, float input_scale, int M, int K,
                         int ldx, cudaStream_t st) {
    const long long total = (long long)M * (K / 16);
    if (total <= 0) return;
    static int strip = -1;
    if (strip < 0) {
        const char *e = getenv("GLMASR_QUANT_STRIP");
        strip = (e && e[0] == '0') ? 0 : 1;
    }
    if (strip && pre == nullptr && M >= 1024 && (K % 2048) == 0 && (ldx % 8) == 0 &&
        (((uintptr_t)x | (uintptr_t)packed_out) & 15) == 0 && (((uintptr_t)scale_rowmajor | (uintptr_t)scale_swizzled) & 3) == 0) {
        const long long units = (long long)M * (K / 2048);
        launch_chained(quantize_act_strip_kernel, dim3(blocks_for(units, 8)), dim3(256), 0, st, packed_out, scale_rowmajor,
                       scale_swizzled, x, 1.0f / input_scale, M, K, ldx);
        return;
    }
    GLMASR_PREFER_MAX_SMEM(quantize_act_kernel);
    launch_chained(quantize_act_kernel, dim3(blocks_for(total, 256)), dim3(256), 0, st, packed_out, scale_rowmajor, scale_swizzled, x, pre,
                                                                1.0f / input_scale, M, K, ldx);
}

// --------------------------------------------------------------------------------------------
// Scale swizzle (reference: Infer-engine/cuda/nvfp4_cutlass.cu:89-111): row-major [rows, cols]
// -> 128x4 tiles.  dst must be zero-filled beforehand where padding matters.
// --------------------------------------------------------------------------------------------
__global__ void swizzle_scales_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, int rows,
                                      int cols, int col_tiles) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * cols) return;
    const int r = (int)(idx / cols), c = (int)(idx % cols);
    dst[swizzled_sf_index(r, c, col_tiles)] = src[idx];
}

void launch_swizzle_scales(uint8_t *dst, const uint8_t *src, int rows, int cols, cudaStream_t st) {
    const long long total = (long long)rows * cols;
    if (total <= 0) return;
    // deliberately an ordinary launch without early dependent signalling: the GEMMs fetch re-tiled weight
    // scales before their dependency wait, which is only safe because this writer ends before they start
    swizzle_scales_kernel<<<blocks_for(total, 256), 256, 0, st>>>(dst, src, rows, cols, (cols + 3) / 4);
}

// --------------------------------------------------------------------------------------------
// SiLU-gate (reference: Infer-engine/cuda/kernels.cu:1252-1273 and :405-421)
//   out = bf16( (g * (1/(1+expf(-g)))) * u )
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_gate(float g, float u) {
    const float sig = __fdiv_rn(1.0f, 1.0f + expf(-g));
    return (g * sig) * u;
}

__global__ void silu_split_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ packed,
                                  int M, int N) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * N) return;
    const int m = (int)(idx / N), n = (int)(idx % N);
    const __nv_bfloat16 *row = packed + (size_t)m * (2 * (size_t)N);
    out[idx] = __float2bfloat16(silu_gate(__bfloat162float(row[n]), __bfloat162float(row[N + n])));
}

void launch_silu_split(__nv_bfloat16 *out, const __nv_bfloat16 *packed, int M, int N, cudaStream_t st) {
    const long long total = (long long)M * N;
    if (total <= 0) return;
    silu_split_kernel<<<blocks_for(total, 256), 256, 0, st>>>(out, packed, M, N);
}

__global__ void silu_mul_kernel(__nv_bfloat16 *__restrict__ gate, const __nv_bfloat16 *__restrict__ up, long long n) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    gate[idx] = __float2bfloat16(silu_gate(__bfloat162float(gate[idx]), __bfloat162float(up[idx])));
}

void launch_silu_mul(__nv_bfloat16 *gate, const __nv_bfloat16 *up, long long n, cudaStream_t st) {
    if (n <= 0) return;
    silu_mul_kernel<<<blocks_for(n, 256), 256, 0, st>>>(gate, up, n);
}

// --------------------------------------------------------------------------------------------
// residual_add (reference: Infer-engine/cuda/kernels.cu:741-761): out = bf16(float(a)+float(b))
// --------------------------------------------------------------------------------------------
__global__ void residual_add_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *a, const __nv_bfloat16 *b, long long n) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    out[idx] = __float2bfloat16(__bfloat162float(a[idx]) + __bfloat162float(b[idx]));
}

void launch_residual_add(__nv_bfloat16 *out, const __nv_bfloat16 *a, const __nv_bfloat16 *b, long long n,
                         cudaStream_t st) {
    if (n <= 0) return;
    residual_add_kernel<<<blocks_for(n, 256), 256, 0, st>>>(out, a, b, n);
}

// --------------------------------------------------------------------------------------------
// Batched row arg-max over bf16 logits (reference: Infer-engine/cuda/kernels.cu:1387-1426).
// The reference's result on ties follows from its 256-thread layout: thread t keeps the first
// maximum of its strided slice (indices t, t+256, ...), then a strict-> tree reduce merges slot
// t+off into slot t for off = 128..1, the lower slot keeping ties.  Two tied threads meet at
// the step given by their lowest differing bit and the one with that bit clear survives, so
// the winner among maximal elements is the one with the smallest bit-reversed (index mod 256),
// then the smallest index.  Values must exceed -1e20 to win, otherwise index 0 is returned.
// The same total order is used here with 16-byte loads.
// --------------------------------------------------------------------------------------------
__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bi) {
    if (v > bv) return true;
    if (!(v == bv)) return false;
    const unsigned t = __brev((unsigned)(i & 255)), bt = __brev((unsigned)(bi & 255));
    return t < bt || (t == bt && i < bi);
}

__global__ void argmax_rows_kernel(const __nv_bfloat16 *__restrict__ logits, int *__restrict__ out_tokens, int rows,
                                   int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sh_val[256];
    __shared__ int sh_idx[256];
    const int row = blockIdx.x, tid = threadIdx.x;
    if (row >= rows) return;
    const __nv_bfloat16 *p = logits + (size_t)row * (size_t)vocab;
    float bv = -1e20f;
    int bi = -1;  // -1: nothing beat the floor yet
    auto consider = [&](float v, int i) {
        if (bi < 0) {
            if (v > bv) { bv = v; bi = i; }
        } else if (argmax_better(v, i, bv, bi)) {
            bv = v;
            bi = i;
        }
    };
    const bool vec_ok = (((uintptr_t)p & 15) == 0);
    const int nvec = vec_ok ? vocab / 8 : 0;
    // four 16-byte loads in flight per thread: a row is read once from HBM and one load at a time leaves the
    // memory system idle (the order of the comparisons does not matter: argmax_better is a total order)
    auto consider8 = [&](const uint4 &q, int c) {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            consider(__uint_as_float(w[j] << 16), c * 8 + 2 * j);
            consider(__uint_as_float(w[j] & 0xFFFF0000u), c * 8 + 2 * j + 1);
        }
    };
    int c = tid;
    for (; c + 768 < nvec; c += 1024) {
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) q[u] = reinterpret_cast<const uint4 *>(p)[c + 256 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u) consider8(q[u], c + 256 * u);
    }
    for (; c < nvec; c += 256) consider8(reinterpret_cast<const uint4 *>(p)[c], c);
    for (int v = nvec * 8 + tid; v < vocab; v += 256) consider(__bfloat162float(p[v]), v);
    sh_val[tid] = bv;
    sh_idx[tid] = bi;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) {
        if (tid < off) {
            const float ov = sh_val[tid + off];
            const int oi = sh_idx[tid + off];
            const int mi = sh_idx[tid];
            bool take;
            if (oi < 0) take = false;
            else if (mi < 0) take = true;
            else take = argmax_better(ov, oi, sh_val[tid], mi);
            if (take) {
                sh_val[tid] = ov;
                sh_idx[tid] = oi;
            }
        }
        __syncthreads();
    }
    if (tid == 0) out_tokens[row] = sh_idx[0] < 0 ? 0 : sh_idx[0];
}

// The same arg-max with a row cut into `parts` column ranges, one CTA each (a few hundred rows of a 59264-wide
// vocabulary are otherwise one or two CTAs per SM, each waiting on a handful of loads at a time).  A CTA leaves its
// range's winner in `partial`; the CTA that arrives last at the row's counter merges the parts and resets the counter.
// argmax_better is a total order, so the result is the one-CTA kernel's.
struct ArgmaxPart {
    float val;
    int idx;
};

__global__ void __launch_bounds__(256) argmax_rows_parts_kernel(const __nv_bfloat16 *__restrict__ logits, int *__restrict__ out_tokens,
                                                               int rows, int vocab, int parts, ArgmaxPart *partial,
                                                               unsigned int *counters) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sh_val[256];
    __shared__ int sh_idx[256];
    __shared__ int sh_last;
    const int row = blockIdx.x / parts, part = blockIdx.x - row * parts, tid = threadIdx.x;
    if (row >= rows) return;
    const __nv_bfloat16 *p = logits + (size_t)row * (size_t)vocab;
    // ranges in whole 16-byte vectors; the last part also takes the columns past the last whole vector
    const int nvec = vocab / 8;
    const int per = (nvec + parts - 1) / parts;
    const int v0 = min(nvec, part * per), v1 = min(nvec, v0 + per);
    float bv = -1e20f;
    int bi = -1;
    auto consider = [&](float v, int i) {
        if (bi < 0) {
            if (v > bv) { bv = v; bi = i; }
        } else if (argmax_better(v, i, bv, bi)) {
            bv = v;
            bi = i;
        }
    };
    auto consider8 = [&](const uint4 &q, int c) {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            consider(__uint_as_float(w[j] << 16), c * 8 + 2 * j);
            consider(__uint_as_float(w[j] & 0xFFFF0000u), c * 8 + 2 * j + 1);
        }
    };
    // eight loads in flight per thread (a range of a 59264-wide row is seven or eight vectors per thread: one batch)
    for (int c = v0 + tid; c < v1; c += 2048) {
        uint4 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (c + 256 * u < v1) q[u] = reinterpret_cast<const uint4 *>(p)[c + 256 * u];
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (c + 256 * u < v1) consider8(q[u], c + 256 * u);
    }
    if (part == parts - 1)
        for (int v = nvec * 8 + tid; v < vocab; v += 256) consider(__bfloat162float(p[v]), v);
    auto merge = [&](float ov, int oi) {          // fold (ov, oi) into this thread's slot of the shared arrays
        const int mi = sh_idx[tid];
        bool take;
        if (oi < 0) take = false;
        else if (mi < 0) take = true;
        else take = argmax_better(ov, oi, sh_val[tid], mi);
        if (take) {
            sh_val[tid] = ov;
            sh_idx[tid] = oi;
        }
    };
    auto reduce_block = [&]() {
        __syncthreads();
        for (int off = 128; off > 0; off >>= 1) {
            if (tid < off) merge(sh_val[tid + off], sh_idx[tid + off]);
            __syncthreads();
        }
    };
    sh_val[tid] = bv;
    sh_idx[tid] = bi;
    reduce_block();
    if (tid == 0) {
        partial[(size_t)row * parts + part] = ArgmaxPart{sh_val[0], sh_idx[0]};
        __threadfence();
        const unsigned int old = atomicAdd(counters + row, 1u);
        sh_last = (old == (unsigned int)parts - 1u) ? 1 : 0;
        if (sh_last) counters[row] = 0u;          // ready for the next launch
    }
    __syncthreads();
    if (!sh_last) return;
    __threadfence();
    sh_val[tid] = -1e20f;
    sh_idx[tid] = -1;
    for (int q = tid; q < parts; q += 256) {
        const int2 raw = __ldcg(reinterpret_cast<const int2 *>(partial + (size_t)row * parts + q));
        merge(__int_as_float(raw.x), raw.y);
    }
    reduce_block();
    if (tid == 0) out_tokens[row] = sh_idx[0] < 0 ? 0 : sh_idx[0];
}

void launch_argmax_rows(const __nv_bfloat16 *logits, int *out_tokens, int rows, int vocab, cudaStream_t st) {
    if (rows <= 0) return;
    // enough CTAs for every SM to hold several; narrow rows stay on the one-CTA kernel
    const int parts = (vocab >= 16384 && (((uintptr_t)logits & 15) == 0) && (vocab % 8) == 0) ? 4 : 1;
    if (parts > 1) {
        constexpr int kArgmaxSlot = 53;
        static void *zeroed = nullptr;
        static int zeroed_rows = 0;
        const size_t part_bytes = ((size_t)rows * parts * sizeof(ArgmaxPart) + 255) & ~(size_t)255;
        uint8_t *ws = (uint8_t *)workspace_slot(kArgmaxSlot, part_bytes + (size_t)rows * sizeof(unsigned int));
        if (ws != zeroed || rows != zeroed_rows) {  // a fresh allocation or another layout: every counter starts at zero
            GLMASR_CUDA_CHECK(cudaMemsetAsync(ws, 0, part_bytes + (size_t)rows * sizeof(unsigned int), st));
            zeroed = ws;
            zeroed_rows = rows;
        }
        launch_chained(argmax_rows_parts_kernel, dim3(rows * parts), dim3(256), 0, st, logits, out_tokens, rows, vocab, parts,
                       reinterpret_cast<ArgmaxPart *>(ws), reinterpret_cast<unsigned int *>(ws + part_bytes));
        return;
    }
    GLMASR_PREFER_MAX_SMEM(argmax_rows_kernel);
    launch_chained(argmax_rows_kernel, dim3(rows), dim3(256), 0, st, logits, out_tokens, rows, vocab);
}

}  // namespace glmasr
