// Audio encoder and adapter (reference: encoder_forward_packed, Infer-engine/cuda/encoder.cu:1974-2188; the
// convolution front end and the projector, Infer-engine/src/engine.c:1111-1160, 1561-1601): 32 pre-norm
// Whisper-style layers at d = 1280, 20 heads of 64, FFN 5120, partial rotary embedding on the first 32
// dims of every head, no attention mask; a two-convolution front end (k = 3, stride 1 then 2, each
// followed by tanh-GELU) and a 4-frame-concatenating two-layer projector to the decoder width.
//
// Everything heavy is a GEMM on the library's tcgen05 bf16 kernel with its epilogues:
//   q | k | v      one GEMM over the three weight tensors (no copy), bias per column (k has none)
//   o, fc2         epilogue bf16(bf16(acc) + bias) + residual, in place on the residual stream
//   fc1, adapter   epilogue bias + tanh-GELU
//   conv1, conv2   the convolution as ONE GEMM with K = 3 * in_channels on a time-major im2col of the
//                  input (the reference issues three accumulating GEMMs per convolution with a bf16
//                  round-trip of the partial sums, plus strided-copy and weight-slice kernels per tap)
// between them LayerNorm (one warp per row, the reference's summation order), the rotary embedding
// (table in the reference's own float arithmetic) and non-causal attention over each window's own
// frames (prefill_attention.cu, head_dim 64).  Weights are found by the checkpoint's names once per
// WeightStore; re-packed convolution weights and the fused q|k|v bias live in private memory until
// encoder_cleanup / glmasr_fp4_cleanup.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../../include/glmasr_engine_types.h"
#include "../../include/glmasr_fp4.h"
#include "decoder_ops.cuh"
#include "gemm_umma.cuh"
#include "runtime.cuh"

namespace glmasr {

int bf16_linear_ex(uint16_t *out, int ldo, const uint16_t *x, int ldx, const uint16_t *const *w, const int *n, int num_w,
                   const uint16_t *bias, int epi, const uint16_t *residual, int M, int K);   // api.cu

// private workspace slots of this file
enum : int { WS_E_NORM = 38, WS_E_QKV = 39, WS_E_FFN = 40, WS_E_POS = 41, WS_E_META = 42, WS_E_COL = 43, WS_E_CONV1 = 44,
             WS_E_TMP = 45, WS_E_PROJ = 46, WS_E_ROPE = 47 };

// --------------------------------------------------------------------------------------------
// LayerNorm (reference: layernorm_kernel, Infer-engine/cuda/kernels.cu:299-345): one warp per row; lane i
// adds x[i], x[i + 32], ... in that order, a shuffle-down tree, lane 0's total broadcast; the variance is a
// second pass over (x - mean)^2; out = bf16(((x - mean) * inv_std) * w + b).  Eight rows per CTA.  out may
// alias x (a warp has its whole row in shared memory before it writes any of it).
// --------------------------------------------------------------------------------------------
template <int MAXE>
__global__ void __launch_bounds__(256) layernorm_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *weight,
                                                        const __nv_bfloat16 *bias, float eps, int rows, int dim) {
    // Rows move between global and shared memory in 16-byte pieces (dim % 8 == 0, 16-byte aligned rows); the
    // arithmetic reads the warp's row from shared memory in the reference's lane-strided order.  weight and bias
    // are staged once per CTA.
    extern __shared__ __align__(16) uint8_t ln_smem[];
    __nv_bfloat16 *w_s = reinterpret_cast<__nv_bfloat16 *>(ln_smem);
    __nv_bfloat16 *b_s = w_s + dim;
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, row = blockIdx.x * 8 + wib;
    __nv_bfloat16 *row_s = b_s + dim + (size_t)wib * dim;
    const int vecs = dim >> 3;
    for (int i = threadIdx.x; i < vecs; i += 256) {
        reinterpret_cast<uint4 *>(w_s)[i] = reinterpret_cast<const uint4 *>(weight)[i];
        reinterpret_cast<uint4 *>(b_s)[i] = bias != nullptr ? reinterpret_cast<const uint4 *>(bias)[i] : make_uint4(0u, 0u, 0u, 0u);
    }
    pdl_wait();
    if (row < rows) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * dim);
        for (int i = lane; i < vecs; i += 32) reinterpret_cast<uint4 *>(row_s)[i] = xr[i];
    }
    __syncthreads();
    if (row >= rows) return;
    // three passes over the row in shared memory (kept out of registers: eight CTAs per SM stay resident)
    float sum = 0.0f;
#pragma unroll 8
    for (int j = 0; j < MAXE; ++j) {
        const int i = lane + 32 * j;
        if (i < dim) sum += __bfloat162float(row_s[i]);
    }
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xFFFFFFFFu, sum, off);
    sum = __shfl_sync(0xFFFFFFFFu, sum, 0);
    const float mean = sum / dim;
    float sum_sq = 0.0f;
#pragma unroll 8
    for (int j = 0; j < MAXE; ++j) {
        const int i = lane + 32 * j;
        if (i < dim) {
            const float d = __bfloat162float(row_s[i]) - mean;
            sum_sq += d * d;
        }
    }
    for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
    sum_sq = __shfl_sync(0xFFFFFFFFu, sum_sq, 0);
    const float inv_std = 1.0f / sqrtf(sum_sq / dim + eps);
#pragma unroll 8
    for (int j = 0; j < MAXE; ++j) {
        const int i = lane + 32 * j;
        if (i < dim) {
            const float val = (__bfloat162float(row_s[i]) - mean) * inv_std;
            row_s[i] = __float2bfloat16(val * __bfloat162float(w_s[i]) + __bfloat162float(b_s[i]));
        }
    }
    __syncwarp();
    uint4 *orow = reinterpret_cast<uint4 *>(out + (size_t)row * dim);
    for (int i = lane; i < vecs; i += 32) orow[i] = reinterpret_cast<const uint4 *>(row_s)[i];
}

// any width (three passes over global memory), same arithmetic; in place is fine here too: a lane reads and writes
// only its own elements, and the warp-wide reductions separate the passes
__global__ void layernorm_generic_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *weight,
                                         const __nv_bfloat16 *bias, float eps, int rows, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const __nv_bfloat16 *xr = x + (size_t)row * dim;
    float sum = 0.0f;
    for (int i = lane; i < dim; i += 32) sum += __bfloat162float(xr[i]);
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_down_sync(0xFFFFFFFFu, sum, off);
    sum = __shfl_sync(0xFFFFFFFFu, sum, 0);
    const float mean = sum / dim;
    float sum_sq = 0.0f;
    for (int i = lane; i < dim; i += 32) {
        const float d = __bfloat162float(xr[i]) - mean;
        sum_sq += d * d;
    }
    for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
    sum_sq = __shfl_sync(0xFFFFFFFFu, sum_sq, 0);
    const float inv_std = 1.0f / sqrtf(sum_sq / dim + eps);
    __nv_bfloat16 *orow = out + (size_t)row * dim;
    __syncwarp();
    for (int i = lane; i < dim; i += 32) {
        const float val = (__bfloat162float(xr[i]) - mean) * inv_std;
        const float b = bias != nullptr ? __bfloat162float(bias[i]) : 0.0f;
        orow[i] = __float2bfloat16(val * __bfloat162float(weight[i]) + b);
    }
}

void launch_layernorm(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *weight, const __nv_bfloat16 *bias,
                      float eps, int rows, int dim, cudaStream_t st) {
    if (rows <= 0) return;
    const dim3 grid((rows + 7) / 8);
    const bool vec = (dim % 8) == 0 && (((uintptr_t)out | (uintptr_t)x | (uintptr_t)weight | (uintptr_t)bias) & 15) == 0;
    if (dim <= 32 * 40 && vec)       // the row fits the registers of a warp (the encoder's 1280)
        launch_chained(layernorm_kernel<40>, grid, dim3(256), (size_t)dim * 2 * 10, st, out, x, weight, bias, eps, rows, dim);
    else
        launch_chained(layernorm_generic_kernel, grid, dim3(256), (size_t)0, st, out, x, weight, bias, eps, rows, dim);
    note_launches(1);
}

// --------------------------------------------------------------------------------------------
// Rotary embedding of the encoder (reference: encoder_rope_fast, Infer-engine/cuda/encoder.cu:1572-1668):
// the first rot_dim = 32 dims of every 64-dim head, pairs (d, d + 16), angle pos * 10000^(-2d/32) with the
// cos / sin table computed on the HOST in float exactly as the reference does (powf, cosf, sinf of the float
// product), dims 32..63 untouched.  q and k rotated in one launch, in place, any row pitch.
// --------------------------------------------------------------------------------------------
static constexpr int kRotHalf = 16, kRopeTablePos = 3072;

__global__ void encoder_rope_kernel(__nv_bfloat16 *q, __nv_bfloat16 *k, const float *__restrict__ cos_t,
                                    const float *__restrict__ sin_t, const int *__restrict__ row_pos, int total_rows,
                                    int num_heads, int head_dim, int q_stride, int k_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_rows * num_heads * kRotHalf) return;
    const int d = idx % kRotHalf, rh = idx / kRotHalf;
    const int head = rh % num_heads, row = rh / num_heads;
    const int pos = row_pos[row];
    const float c = cos_t[pos * kRotHalf + d], s = sin_t[pos * kRotHalf + d];
    if (q != nullptr) {
        __nv_bfloat16 *p = q + (size_t)row * q_stride + head * head_dim;
        const float a = __bfloat162float(p[d]), b = __bfloat162float(p[d + kRotHalf]);
        p[d] = __float2bfloat16(a * c - b * s);
        p[d + kRotHalf] = __float2bfloat16(b * c + a * s);
    }
    if (k != nullptr) {
        __nv_bfloat16 *p = k + (size_t)row * k_stride + head * head_dim;
        const float a = __bfloat162float(p[d]), b = __bfloat162float(p[d + kRotHalf]);
        p[d] = __float2bfloat16(a * c - b * s);
        p[d + kRotHalf] = __float2bfloat16(b * c + a * s);
    }
}

// Same values, 16 bytes per access: a thread takes dims d0..d0+7 (d0 = 0 or 8) of one head of one row and their
// partners d0+16..d0+23, for q and k.  Needs 16-byte aligned rows and heads (strides and head_dim multiples of 8).
__global__ void __launch_bounds__(256) encoder_rope_vec_kernel(__nv_bfloat16 *q, __nv_bfloat16 *k, const float *__restrict__ cos_t,
                                                               const float *__restrict__ sin_t, const int *__restrict__ row_pos,
                                                               int total_rows, int num_heads, int head_dim, int q_stride, int k_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_rows * num_heads * 2) return;
    const int d0 = (idx & 1) * 8, rh = idx >> 1;
    const int head = rh % num_heads, row = rh / num_heads;
    const int pos = row_pos[row];
    float c[8], s[8];
    {
        const float4 *cp = reinterpret_cast<const float4 *>(cos_t + pos * kRotHalf + d0);
        const float4 *sp = reinterpret_cast<const float4 *>(sin_t + pos * kRotHalf + d0);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        c[0] = c0.x, c[1] = c0.y, c[2] = c0.z, c[3] = c0.w, c[4] = c1.x, c[5] = c1.y, c[6] = c1.z, c[7] = c1.w;
        s[0] = s0.x, s[1] = s0.y, s[2] = s0.z, s[3] = s0.w, s[4] = s1.x, s[5] = s1.y, s[6] = s1.z, s[7] = s1.w;
    }
    auto rotate = [&](__nv_bfloat16 *base) {
        uint4 *pa = reinterpret_cast<uint4 *>(base + d0), *pb = reinterpret_cast<uint4 *>(base + d0 + kRotHalf);
        const uint4 va = *pa, vb = *pb;
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t oa[4], ob[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a0 = __uint_as_float(wa[i] << 16), a1 = __uint_as_float(wa[i] & 0xFFFF0000u);
            const float b0 = __uint_as_float(wb[i] << 16), b1 = __uint_as_float(wb[i] & 0xFFFF0000u);
            const __nv_bfloat162 ra = __floats2bfloat162_rn(a0 * c[2 * i] - b0 * s[2 * i], a1 * c[2 * i + 1] - b1 * s[2 * i + 1]);
            const __nv_bfloat162 rb = __floats2bfloat162_rn(b0 * c[2 * i] + a0 * s[2 * i], b1 * c[2 * i + 1] + a1 * s[2 * i + 1]);
            oa[i] = *reinterpret_cast<const uint32_t *>(&ra);
            ob[i] = *reinterpret_cast<const uint32_t *>(&rb);
        }
        *pa = make_uint4(oa[0], oa[1], oa[2], oa[3]);
        *pb = make_uint4(ob[0], ob[1], ob[2], ob[3]);
    };
    if (q != nullptr) rotate(q + (size_t)row * q_stride + head * head_dim);
    if (k != nullptr) rotate(k + (size_t)row * k_stride + head * head_dim);
}

static float *g_rope_dev = nullptr;          // lives in a workspace slot: dropped by encoder_forget_all before the slots are freed
static const float *rope_tables(cudaStream_t st) {
    float *&dev = g_rope_dev;
    if (dev == nullptr) {
        std::vector<float> h((size_t)2 * kRopeTablePos * kRotHalf);
        for (int pos = 0; pos < kRopeTablePos; ++pos)
            for (int d = 0; d < kRotHalf; ++d) {
                const float inv_freq = powf(10000.0f, -(2.0f * d) / 32.0f);       // encoder.cu:1583-1587
                const float theta = pos * inv_freq;
                h[(size_t)pos * kRotHalf + d] = cosf(theta);
                h[(size_t)kRopeTablePos * kRotHalf + (size_t)pos * kRotHalf + d] = sinf(theta);
            }
        dev = (float *)workspace_slot(WS_E_ROPE, h.size() * sizeof(float));
        GLMASR_CUDA_CHECK(cudaMemcpyAsync(dev, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice, st));
        GLMASR_CUDA_CHECK(cudaStreamSynchronize(st));            // the host vector goes away
    }
    return dev;
}

void launch_encoder_rope(__nv_bfloat16 *q, __nv_bfloat16 *k, const int *d_row_pos, int total_rows, int num_heads, int head_dim,
                         int q_stride, int k_stride, cudaStream_t st) {
    if (total_rows <= 0) return;
    const float *tab = rope_tables(st);
    const bool vec = (head_dim % 8) == 0 && (q_stride % 8) == 0 && (k_stride % 8) == 0 && (((uintptr_t)q | (uintptr_t)k) & 15) == 0;
    if (vec) {
        const int work = total_rows * num_heads * 2;
        launch_chained(encoder_rope_vec_kernel, dim3((work + 255) / 256), dim3(256), (size_t)0, st, q, k, tab,
                       tab + (size_t)kRopeTablePos * kRotHalf, d_row_pos, total_rows, num_heads, head_dim, q_stride, k_stride);
    } else {
        const int work = total_rows * num_heads * kRotHalf;
        launch_chained(encoder_rope_kernel, dim3((work + 255) / 256), dim3(256), (size_t)0, st, q, k, tab,
                       tab + (size_t)kRopeTablePos * kRotHalf, d_row_pos, total_rows, num_heads, head_dim, q_stride, k_stride);
    }
    note_launches(1);
}

// --------------------------------------------------------------------------------------------
// small element-wise kernels with reference names
// --------------------------------------------------------------------------------------------
__global__ void gelu_kernel(__nv_bfloat16 *x, long long n) {          // kernels.cu:364-372
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = __bfloat162float(x[i]);
    x[i] = __float2bfloat16(0.5f * v * (1.0f + tanhf(0.79788456f * (v + 0.044715f * v * v * v))));
}

// x[i] = bf16(float(x[i]) + bias[i % N])   (add_bias_2d / add_bias, kernels.cu:832-842, 1541-1549)
__global__ void add_bias_cols_kernel(__nv_bfloat16 *x, const __nv_bfloat16 *bias, long long total, int N) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    x[i] = __float2bfloat16(__bfloat162float(x[i]) + __bfloat162float(bias[i % N]));
}

__global__ void residual_add_bias_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *a, const __nv_bfloat16 *b,
                                         const __nv_bfloat16 *bias, long long total, int N) {     // kernels.cu:763-782
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float av = __bfloat162float(a[i]);
    if (bias != nullptr) av += __bfloat162float(bias[i % N]);
    av = __bfloat162float(__float2bfloat16(av));
    out[i] = __float2bfloat16(av + __bfloat162float(b[i]));
}

// out[c, r] = in[r, c]   (kernels.cu:1631-1650), 32 x 32 tiles through shared memory
__global__ void transpose_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *in, int rows, int cols) {
    __shared__ __nv_bfloat16 tile[32][33];
    pdl_launch_dependents();
    pdl_wait();
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8)
        if (r0 + j < rows && c0 + threadIdx.x < cols) tile[j][threadIdx.x] = in[(size_t)(r0 + j) * cols + c0 + threadIdx.x];
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8)
        if (c0 + j < cols && r0 + threadIdx.x < rows) out[(size_t)(c0 + j) * rows + r0 + threadIdx.x] = tile[threadIdx.x][j];
}

// --------------------------------------------------------------------------------------------
// convolution as a GEMM: time-major im2col.  Row t of the result holds the kernel_size input frames
// t * stride - padding + k (zeros outside), each as in_ch contiguous channels: column k * in_ch + c.
// The matching weight matrix is w2[oc, k * in_ch + c] = w[oc, c, k].
// --------------------------------------------------------------------------------------------
// input time-major [windows][in_len_stride rows][in_ch]; 8 channels (16 bytes) per thread
__global__ void im2col_time_major_kernel(__nv_bfloat16 *__restrict__ col, const __nv_bfloat16 *__restrict__ in, int in_ch,
                                         long long in_window_stride, const int *__restrict__ in_lens, int out_len_max,
                                         int kernel_size, int stride, int padding) {
    pdl_launch_dependents();
    pdl_wait();
    const int w = blockIdx.z, t = blockIdx.y;
    const int in_len = in_lens[w];
    const int out_len = (in_len + 2 * padding - kernel_size) / stride + 1;
    if (t >= out_len) return;
    const int chunks = kernel_size * in_ch / 8;
    const int K = kernel_size * in_ch;
    uint4 *dst = reinterpret_cast<uint4 *>(col + ((size_t)w * out_len_max + t) * K);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += gridDim.x * blockDim.x) {
        const int k = (i * 8) / in_ch, c = (i * 8) % in_ch;
        const int src_t = t * stride - padding + k;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (src_t >= 0 && src_t < in_len)
            v = *reinterpret_cast<const uint4 *>(in + (size_t)w * in_window_stride + (size_t)src_t * in_ch + c);
        dst[i] = v;
    }
}

// input channel-major [in_ch, in_len] (the reference's conv1d_forward layout)
__global__ void im2col_channel_major_kernel(__nv_bfloat16 *__restrict__ col, const __nv_bfloat16 *__restrict__ in, int in_ch,
                                            int in_len, int out_len, int kernel_size, int stride, int padding) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = (long long)out_len * kernel_size * in_ch;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int K = kernel_size * in_ch;
    const int t = (int)(i / K), kc = (int)(i % K);
    const int k = kc / in_ch, c = kc % in_ch;
    const int src_t = t * stride - padding + k;
    col[i] = (src_t >= 0 && src_t < in_len) ? in[(size_t)c * in_len + src_t] : __float2bfloat16(0.0f);
}

__global__ void repack_conv_weight_kernel(__nv_bfloat16 *__restrict__ w2, const __nv_bfloat16 *__restrict__ w, int out_ch,
                                          int in_ch, int kernel_size) {
    const long long total = (long long)out_ch * in_ch * kernel_size;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int K = kernel_size * in_ch;
    const int oc = (int)(i / K), kc = (int)(i % K);
    const int k = kc / in_ch, c = kc % in_ch;
    w2[i] = w[((size_t)oc * in_ch + c) * kernel_size + k];
}

// row r of sequence s -> position r - offset[s]  (reference: encoder_fill_row_positions_kernel)
__global__ void fill_row_positions_kernel(int *row_pos, const int *seq_offsets, const int *seq_lens, int num_seqs) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    if (s >= num_seqs) return;
    const int len = seq_lens[s], off = seq_offsets[s];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < len; i += gridDim.x * blockDim.x) row_pos[off + i] = i;
}

// --------------------------------------------------------------------------------------------
// weights by name, once per store
// --------------------------------------------------------------------------------------------
struct EncLayerRef {
    const uint16_t *ln1_w, *ln1_b, *ln2_w, *ln2_b;
    const uint16_t *q_w, *k_w, *v_w, *o_w, *fc1_w, *fc2_w;
    const uint16_t *q_b, *v_b, *o_b, *fc1_b, *fc2_b;
    uint16_t *qkv_bias;            // [3 hidden]: q bias | zeros | v bias (private copy), or NULL when there is none
};
struct EncoderRefs {
    const glmasr_WeightStore *ws = nullptr;
    uint64_t fingerprint = 0;
    int count = -1;
    std::vector<EncLayerRef> layers;
    const uint16_t *norm_w = nullptr, *norm_b = nullptr;
    uint16_t *bias_arena = nullptr;
};
static EncoderRefs g_enc;

static const glmasr_Tensor *find_t(const glmasr_WeightStore *ws, const char *name) {
    for (int i = 0; i < ws->count; ++i)
        if (ws->names[i] != nullptr && strcmp(ws->names[i], name) == 0) return &ws->tensors[i];
    return nullptr;
}
static const uint16_t *need_bf16(const glmasr_WeightStore *ws, const char *name, bool required) {
    const glmasr_Tensor *t = find_t(ws, name);
    if (t == nullptr) {
        if (required) {
            fprintf(stderr, "Weight not found: %s\n", name);
            exit(1);
        }
        return nullptr;
    }
    GLMASR_CHECK(t->dtype == GLMASR_DTYPE_BF16, "encoder weight %s is not bf16 (dtype %d)", name, t->dtype);
    return (const uint16_t *)t->data;
}
static uint64_t store_print(const glmasr_WeightStore *ws) {
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < ws->count; ++i) {
        h = (h ^ (uint64_t)(uintptr_t)ws->tensors[i].data) * 1099511628211ull;
        h = (h ^ (uint64_t)ws->tensors[i].nbytes) * 1099511628211ull;
    }
    return h;
}

static void drop_encoder_refs() {
    if (g_enc.bias_arena != nullptr) {
        cudaDeviceSynchronize();
        cudaFree(g_enc.bias_arena);
    }
    g_enc = EncoderRefs();
}

static const EncoderRefs &encoder_refs(const glmasr_WeightStore *ws, int layers, int hidden, cudaStream_t st) {
    const uint64_t fp = store_print(ws);
    if (g_enc.ws == ws && g_enc.count == ws->count && g_enc.fingerprint == fp && (int)g_enc.layers.size() == layers) return g_enc;
    drop_encoder_refs();
    g_enc.ws = ws;
    g_enc.count = ws->count;
    g_enc.fingerprint = fp;
    g_enc.layers.resize(layers);
    GLMASR_CUDA_CHECK(cudaMalloc(&g_enc.bias_arena, (size_t)layers * 3 * hidden * sizeof(uint16_t)));
    GLMASR_CUDA_CHECK(cudaMemsetAsync(g_enc.bias_arena, 0, (size_t)layers * 3 * hidden * sizeof(uint16_t), st));
    char n[256];
    for (int l = 0; l < layers; ++l) {
        EncLayerRef &L = g_enc.layers[l];
        auto get = [&](const char *suffix, bool required) {
            snprintf(n, sizeof(n), "audio_tower.layers.%d.%s", l, suffix);
            return need_bf16(ws, n, required);
        };
        L.ln1_w = get("input_layernorm.weight", true);
        L.ln1_b = get("input_layernorm.bias", false);
        L.ln2_w = get("post_attention_layernorm.weight", true);
        L.ln2_b = get("post_attention_layernorm.bias", false);
        L.q_w = get("self_attn.q_proj.weight", true);
        L.q_b = get("self_attn.q_proj.bias", false);
        L.k_w = get("self_attn.k_proj.weight", true);
        L.v_w = get("self_attn.v_proj.weight", true);
        L.v_b = get("self_attn.v_proj.bias", false);
        L.o_w = get("self_attn.o_proj.weight", true);
        L.o_b = get("self_attn.o_proj.bias", false);
        L.fc1_w = get("mlp.fc1.weight", true);
        L.fc1_b = get("mlp.fc1.bias", false);
        L.fc2_w = get("mlp.fc2.weight", true);
        L.fc2_b = get("mlp.fc2.bias", false);
        L.qkv_bias = nullptr;
        if (L.q_b != nullptr || L.v_b != nullptr) {
            L.qkv_bias = g_enc.bias_arena + (size_t)l * 3 * hidden;
            if (L.q_b) GLMASR_CUDA_CHECK(cudaMemcpyAsync(L.qkv_bias, L.q_b, (size_t)hidden * 2, cudaMemcpyDeviceToDevice, st));
            if (L.v_b) GLMASR_CUDA_CHECK(cudaMemcpyAsync(L.qkv_bias + 2 * hidden, L.v_b, (size_t)hidden * 2, cudaMemcpyDeviceToDevice, st));
        }
    }
    g_enc.norm_w = need_bf16(ws, "audio_tower.norm.weight", true);
    g_enc.norm_b = need_bf16(ws, "audio_tower.norm.bias", false);
    return g_enc;
}

// re-packed convolution weights [out_ch, kernel_size * in_ch], cached by the original's device pointer
struct ConvPack {
    const void *src;
    uint16_t *packed;
    int out_ch, in_ch, ks;
};
static std::vector<ConvPack> g_conv_packs;

static const uint16_t *packed_conv_weight(const uint16_t *w, int out_ch, int in_ch, int ks, cudaStream_t st) {
    for (const ConvPack &p : g_conv_packs)
        if (p.src == w && p.out_ch == out_ch && p.in_ch == in_ch && p.ks == ks) return p.packed;
    ConvPack p = {w, nullptr, out_ch, in_ch, ks};
    const long long total = (long long)out_ch * in_ch * ks;
    GLMASR_CUDA_CHECK(cudaMalloc(&p.packed, (size_t)total * sizeof(uint16_t)));
    repack_conv_weight_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((__nv_bfloat16 *)p.packed, (const __nv_bfloat16 *)w,
                                                                             out_ch, in_ch, ks);
    note_launches(1);
    g_conv_packs.push_back(p);
    return p.packed;
}

static void drop_conv_packs() {
    if (!g_conv_packs.empty()) cudaDeviceSynchronize();
    for (ConvPack &p : g_conv_packs) cudaFree(p.packed);
    g_conv_packs.clear();
}

void encoder_forget_all() {
    drop_encoder_refs();
    drop_conv_packs();
    g_rope_dev = nullptr;
}

static int gemm(uint16_t *out, int ldo, const uint16_t *x, int ldx, const uint16_t *w, int N, const uint16_t *bias, int epi,
                const uint16_t *residual, int M, int K) {
    const uint16_t *ws[1] = {w};
    const int ns[1] = {N};
    return bf16_linear_ex(out, ldo, x, ldx, ws, ns, 1, bias, epi, residual, M, K);
}

// The 32 layers and the final norm, in place on hidden [total_rows, H]; d_meta = device {offsets[num_seqs], lens[num_seqs]}.
static void encoder_layers(const glmasr_WeightStore *ws, const glmasr_ModelConfig *cfg, uint16_t *hidden, int total_rows,
                           int num_seqs, const int *d_offsets, const int *d_lens, int max_seq_len, cudaStream_t st) {
    const int H = cfg->enc_hidden, L = cfg->enc_layers, NH = cfg->enc_heads, HD = cfg->enc_head_dim, F = cfg->enc_ffn;
    GLMASR_CHECK(NH * HD == H, "encoder: heads * head_dim != hidden");
    GLMASR_CHECK(HD == 64, "encoder attention is built for head_dim 64 (got %d)", HD);
    const EncoderRefs &R = encoder_refs(ws, L, H, st);
    const int M = total_rows;
    uint16_t *nrm = (uint16_t *)workspace_slot(WS_E_NORM, (size_t)M * H * 2);
    uint16_t *qkv = (uint16_t *)workspace_slot(WS_E_QKV, (size_t)M * 3 * H * 2);
    uint16_t *ffn = (uint16_t *)workspace_slot(WS_E_FFN, (size_t)M * F * 2);
    int *row_pos = (int *)workspace_slot(WS_E_POS, (size_t)M * sizeof(int));
    launch_chained(fill_row_positions_kernel, dim3(8, num_seqs), dim3(256), (size_t)0, st, row_pos, d_offsets, d_lens, num_seqs);
    note_launches(1);
    for (int l = 0; l < L; ++l) {
        const EncLayerRef &W = R.layers[l];
        launch_layernorm((__nv_bfloat16 *)nrm, (const __nv_bfloat16 *)hidden, (const __nv_bfloat16 *)W.ln1_w,
                         (const __nv_bfloat16 *)W.ln1_b, 1e-5f, M, H, st);
        const uint16_t *w3[3] = {W.q_w, W.k_w, W.v_w};
        const int n3[3] = {H, H, H};
        GLMASR_CHECK(bf16_linear_ex(qkv, 3 * H, nrm, H, w3, n3, 3, W.qkv_bias, EPI_STORE, nullptr, M, H) == 0,
                     "encoder q|k|v projection failed (rows %d)", M);
        launch_encoder_rope((__nv_bfloat16 *)qkv, (__nv_bfloat16 *)qkv + H, row_pos, M, NH, HD, 3 * H, 3 * H, st);
        const bool ok = launch_prefill_attention((__nv_bfloat16 *)nrm, H, (const __nv_bfloat16 *)qkv, 3 * H,
                                                 (const __nv_bfloat16 *)qkv + H, 3 * H, (const __nv_bfloat16 *)qkv + 2 * H, 3 * H,
                                                 d_offsets, d_lens, num_seqs, max_seq_len, M, NH, NH, HD, false, st);
        GLMASR_CHECK(ok, "encoder attention: unsupported layout");
        note_launches(1);
        GLMASR_CHECK(gemm(hidden, H, nrm, H, W.o_w, H, W.o_b, EPI_RESIDUAL, hidden, M, H) == 0, "encoder o projection failed");
        launch_layernorm((__nv_bfloat16 *)nrm, (const __nv_bfloat16 *)hidden, (const __nv_bfloat16 *)W.ln2_w,
                         (const __nv_bfloat16 *)W.ln2_b, 1e-5f, M, H, st);
        GLMASR_CHECK(gemm(ffn, F, nrm, H, W.fc1_w, F, W.fc1_b, EPI_GELU, nullptr, M, H) == 0, "encoder fc1 failed");
        GLMASR_CHECK(gemm(hidden, H, ffn, F, W.fc2_w, H, W.fc2_b, EPI_RESIDUAL, hidden, M, F) == 0, "encoder fc2 failed");
    }
    launch_layernorm((__nv_bfloat16 *)hidden, (const __nv_bfloat16 *)hidden, (const __nv_bfloat16 *)R.norm_w,
                     (const __nv_bfloat16 *)R.norm_b, 1e-5f, M, H, st);
}

}  // namespace glmasr

using namespace glmasr;

// ============================================================================================
// reference-named entry points
// ============================================================================================
// Infer-engine/include/cuda_kernels.h:26-28, Infer-engine/cuda/kernels.cu:299-356.
extern "C" void layernorm(uint16_t *out, const uint16_t *x, const uint16_t *weight, const uint16_t *bias, float eps, int rows,
                          int dim) {
    launch_layernorm((__nv_bfloat16 *)out, (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)weight, (const __nv_bfloat16 *)bias,
                     eps, rows, dim, current_stream());
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:30, Infer-engine/cuda/kernels.cu:364-381.
extern "C" void gelu_inplace(uint16_t *x, int n) {
    if (n <= 0) return;
    launch_chained(gelu_kernel, dim3((n + 255) / 256), dim3(256), (size_t)0, current_stream(), (__nv_bfloat16 *)x, (long long)n);
    note_launches(1);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:47-51, Infer-engine/cuda/kernels.cu:763-795.
extern "C" void residual_add_bias(uint16_t *out, const uint16_t *a, const uint16_t *b, const uint16_t *bias, int M, int N) {
    const long long total = (long long)M * N;
    if (total <= 0) return;
    launch_chained(residual_add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), (size_t)0, current_stream(),
                   (__nv_bfloat16 *)out, (const __nv_bfloat16 *)a, (const __nv_bfloat16 *)b, (const __nv_bfloat16 *)bias, total, N);
    note_launches(1);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:53-54, Infer-engine/cuda/kernels.cu:801-826: [seq, dim] -> [seq / 4, 4 dim].  Four
// consecutive rows of a row-major matrix ARE one row of the result, so this is a copy of the first 4 * (seq / 4) rows.
extern "C" void concat_4frames(uint16_t *out, const uint16_t *in, int seq_len, int dim) {
    const int groups = seq_len / 4;
    if (groups <= 0 || out == in) return;
    GLMASR_CUDA_CHECK(cudaMemcpyAsync(out, in, (size_t)groups * 4 * dim * sizeof(uint16_t), cudaMemcpyDeviceToDevice, current_stream()));
}

// Infer-engine/include/cuda_kernels.h:61-62, Infer-engine/cuda/kernels.cu:1631-1660.
extern "C" void transpose_2d(uint16_t *out, const uint16_t *in, int rows, int cols) {
    if (rows <= 0 || cols <= 0) return;
    launch_chained(transpose_kernel, dim3((cols + 31) / 32, (rows + 31) / 32), dim3(32, 8), (size_t)0, current_stream(),
                   (__nv_bfloat16 *)out, (const __nv_bfloat16 *)in, rows, cols);
    note_launches(1);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:56-59, Infer-engine/cuda/kernels.cu:1561-1629: input [in_ch, seq_len], weight
// [out_ch, in_ch, kernel_size], out [out_ch, out_len], all channel-major bf16, bias per output channel.  One GEMM over
// K = kernel_size * in_ch (fp32 accumulation across the taps; the reference rounds the partial sums to bf16 between
// its per-tap GEMMs), bias added to the bf16 result as the reference does.
extern "C" void conv1d_forward(uint16_t *out, const uint16_t *input, const uint16_t *weight, const uint16_t *bias, int in_ch,
                               int out_ch, int seq_len, int kernel_size, int stride, int padding) {
    cudaStream_t st = current_stream();
    const int out_len = (seq_len + 2 * padding - kernel_size) / stride + 1;
    if (out_len <= 0) return;
    const int K = kernel_size * in_ch;
    uint16_t *col = (uint16_t *)workspace_slot(WS_E_COL, (size_t)out_len * K * 2);
    uint16_t *tmp = (uint16_t *)workspace_slot(WS_E_TMP, (size_t)out_len * out_ch * 2);
    const long long total = (long long)out_len * K;
    launch_chained(im2col_channel_major_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), (size_t)0, st,
                   (__nv_bfloat16 *)col, (const __nv_bfloat16 *)input, in_ch, seq_len, out_len, kernel_size, stride, padding);
    note_launches(1);
    const uint16_t *w2 = packed_conv_weight(weight, out_ch, in_ch, kernel_size, st);
    GLMASR_CHECK(gemm(tmp, out_ch, col, K, w2, out_ch, nullptr, EPI_STORE, nullptr, out_len, K) == 0,
                 "conv1d_forward: unsupported shape (in_ch %d, out_ch %d, kernel %d)", in_ch, out_ch, kernel_size);
    if (bias != nullptr) {
        // add_bias_2d (kernels.cu:1541-1549) adds bias[channel] to the bf16 GEMM result and rounds again; on the
        // time-major buffer the channel is the column
        const long long n = (long long)out_len * out_ch;
        launch_chained(add_bias_cols_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, st, (__nv_bfloat16 *)tmp,
                       (const __nv_bfloat16 *)bias, n, out_ch);
        note_launches(1);
    }
    transpose_2d(out, tmp, out_len, out_ch);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:34-36, Infer-engine/cuda/kernels.cu:427-484: partial rotary embedding of one dense
// sequence, q and k [seq_len, num_heads, head_dim] in place, positions 0 .. seq_len - 1.  partial_factor * head_dim
// must be 32 (the encoder's value), the only case the table covers.
extern "C" void rope_encoder(uint16_t *q, uint16_t *k, int seq_len, int num_heads, int head_dim, float partial_factor) {
    if (seq_len <= 0) return;
    GLMASR_CHECK((int)(head_dim * partial_factor) == 2 * kRotHalf && seq_len <= kRopeTablePos,
                 "rope_encoder: only rot_dim 32 and up to %d positions are supported", kRopeTablePos);
    cudaStream_t st = current_stream();
    int *pos = (int *)workspace_slot(WS_E_POS, (size_t)seq_len * sizeof(int));
    int *meta = (int *)workspace_slot(WS_E_META, 2 * sizeof(int));
    const int h_meta[2] = {0, seq_len};
    GLMASR_CUDA_CHECK(cudaMemcpyAsync(meta, h_meta, sizeof(h_meta), cudaMemcpyHostToDevice, st));
    launch_chained(fill_row_positions_kernel, dim3(8, 1), dim3(256), (size_t)0, st, pos, (const int *)meta, (const int *)meta + 1, 1);
    note_launches(1);
    launch_encoder_rope((__nv_bfloat16 *)q, (__nv_bfloat16 *)k, pos, seq_len, num_heads, head_dim, num_heads * head_dim,
                        num_heads * head_dim, st);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:104-111, Infer-engine/cuda/encoder.cu:2441-2462: the encoder stack in place on
// hidden [total_rows, enc_hidden]; sequence s owns rows [seq_offsets[s], + seq_lens[s]) (host arrays).  handle is unused.
extern "C" void encoder_forward_packed(void *handle, const void *ws_v, uint16_t *hidden, int total_rows, int num_seqs,
                                       const int *seq_lens, const int *seq_offsets, const void *cfg_v) {
    (void)handle;
    if (total_rows <= 0 || num_seqs <= 0) return;
    GLMASR_CHECK(ws_v != nullptr && hidden != nullptr && seq_lens != nullptr && seq_offsets != nullptr && cfg_v != nullptr,
                 "encoder_forward_packed received a null argument");
    cudaStream_t st = current_stream();
    int max_len = 0;
    std::vector<int> meta((size_t)2 * num_seqs);
    for (int i = 0; i < num_seqs; ++i) {
        GLMASR_CHECK(seq_lens[i] >= 0 && seq_offsets[i] >= 0 && seq_offsets[i] + seq_lens[i] <= total_rows,
                     "encoder_forward_packed: sequence %d outside the batch", i);
        GLMASR_CHECK(seq_lens[i] <= kRopeTablePos, "encoder_forward_packed: sequence %d longer than %d frames", i, kRopeTablePos);
        meta[i] = seq_offsets[i];
        meta[num_seqs + i] = seq_lens[i];
        if (seq_lens[i] > max_len) max_len = seq_lens[i];
    }
    int *d_meta = (int *)workspace_slot(WS_E_META, meta.size() * sizeof(int));
    GLMASR_CUDA_CHECK(cudaMemcpyAsync(d_meta, meta.data(), meta.size() * sizeof(int), cudaMemcpyHostToDevice, st));
    // pageable host memory: the copy has been staged when the call returns
    encoder_layers((const glmasr_WeightStore *)ws_v, (const glmasr_ModelConfig *)cfg_v, hidden, total_rows, num_seqs, d_meta,
                   d_meta + num_seqs, max_len, st);
    GLMASR_CUDA_CHECK(cudaGetLastError());
}

// Infer-engine/include/cuda_kernels.h:101-103, Infer-engine/cuda/encoder.cu:2427-2439.
extern "C" void encoder_forward(void *handle, const void *ws, uint16_t *hidden, int seq_len, const void *cfg) {
    const int off = 0;
    encoder_forward_packed(handle, ws, hidden, seq_len, 1, &seq_len, &off, cfg);
}

// Infer-engine/include/cuda_kernels.h:121, Infer-engine/cuda/encoder.cu:2421-2423.
extern "C" void encoder_cleanup(void) { encoder_forget_all(); }

// Whole audio path after the log-mel features, for a batch of windows: convolution front end, encoder, projector
// (Infer-engine/src/engine.c:1111-1160 per window; :1561-1601 batched).  mel: TIME-MAJOR features as
// glmasr_mel_spectrogram_batched(time_major = 1) writes them, window i at mel + i * mel_stride holding
// [n_frames_host[i], num_mel_bins]; out: window i's audio embeddings at out + i * out_stride as
// [tokens_i, dec_hidden], tokens_i = ((n_i + 1) / 2) / 4 = out_tokens_host[i] (frames after the stride-2 convolution,
// grouped by four; trailing frames that do not fill a group are dropped as in the reference).  Returns 0 or -1.
extern "C" int glmasr_audio_encode_batched(const void *ws_v, const void *cfg_v, const uint16_t *mel, long long mel_stride,
                                           const int *n_frames_host, int num_windows, uint16_t *out, long long out_stride,
                                           int *out_tokens_host) {
    if (num_windows <= 0) return 0;
    if (ws_v == nullptr || cfg_v == nullptr || mel == nullptr || n_frames_host == nullptr || out == nullptr) return -1;
    const glmasr_WeightStore *ws = (const glmasr_WeightStore *)ws_v;
    const glmasr_ModelConfig *cfg = (const glmasr_ModelConfig *)cfg_v;
    const int H = cfg->enc_hidden, MELS = cfg->num_mel_bins, W = num_windows, D = cfg->dec_hidden, PM = cfg->proj_mid;
    if ((MELS % 8) != 0 || (H % 8) != 0 || H <= 0 || D <= 0 || PM <= 0) return -1;
    cudaStream_t st = current_stream();
    int t1_max = 0;
    std::vector<int> meta((size_t)4 * W);             // conv1 lens | conv2 lens | encoder offsets | (spare)
    for (int i = 0; i < W; ++i) {
        const int n = n_frames_host[i];
        if (n <= 0 || n > cfg->max_audio_frames || n > kRopeTablePos) return -1;
        meta[i] = n;                                   // conv1: k 3, stride 1, padding 1 keeps the length
        meta[W + i] = (n + 2 - 3) / 2 + 1;             // conv2: k 3, stride 2, padding 1
        if (n > t1_max) t1_max = n;
    }
    const int t2_max = (t1_max + 2 - 3) / 2 + 1;
    const int rows_enc = t2_max / 4 * 4 == t2_max ? t2_max : (t2_max + 3) / 4 * 4;      // whole groups of four per window
    for (int i = 0; i < W; ++i) meta[2 * W + i] = i * rows_enc;
    int *d_meta = (int *)workspace_slot(WS_E_META, meta.size() * sizeof(int));
    if (cudaMemcpyAsync(d_meta, meta.data(), meta.size() * sizeof(int), cudaMemcpyHostToDevice, st) != cudaSuccess) return -1;
    const int *d_len1 = d_meta, *d_len2 = d_meta + W, *d_off = d_meta + 2 * W;

    const uint16_t *c1w = need_bf16(ws, "audio_tower.conv1.weight", true), *c1b = need_bf16(ws, "audio_tower.conv1.bias", false);
    const uint16_t *c2w = need_bf16(ws, "audio_tower.conv2.weight", true), *c2b = need_bf16(ws, "audio_tower.conv2.bias", false);
    const uint16_t *p1w = need_bf16(ws, "multi_modal_projector.linear_1.weight", true);
    const uint16_t *p1b = need_bf16(ws, "multi_modal_projector.linear_1.bias", false);
    const uint16_t *p2w = need_bf16(ws, "multi_modal_projector.linear_2.weight", true);
    const uint16_t *p2b = need_bf16(ws, "multi_modal_projector.linear_2.bias", false);
    const uint16_t *c1p = packed_conv_weight(c1w, H, MELS, 3, st);
    const uint16_t *c2p = packed_conv_weight(c2w, H, H, 3, st);

    // conv1 + GELU: [W * t1_max, 3 MELS] x [H, 3 MELS]^T -> [W][t1_max][H]
    const int K1 = 3 * MELS, K2 = 3 * H;
    uint16_t *col = (uint16_t *)workspace_slot(WS_E_COL, (size_t)W * (size_t)((size_t)t1_max * K1 > (size_t)t2_max * K2 ? (size_t)t1_max * K1 : (size_t)t2_max * K2) * 2);
    uint16_t *c1 = (uint16_t *)workspace_slot(WS_E_CONV1, (size_t)W * t1_max * H * 2);
    launch_chained(im2col_time_major_kernel, dim3(1, t1_max, W), dim3(64), (size_t)0, st, (__nv_bfloat16 *)col,
                   (const __nv_bfloat16 *)mel, MELS, mel_stride, d_len1, t1_max, 3, 1, 1);
    note_launches(1);
    if (gemm(c1, H, col, K1, c1p, H, c1b, EPI_GELU, nullptr, W * t1_max, K1) != 0) return -1;
    // conv2 + GELU: [W * t2_max, 3 H] x [H, 3 H]^T -> the encoder's hidden state [W][rows_enc][H]
    uint16_t *hid = (uint16_t *)workspace_slot(WS_E_TMP, (size_t)W * rows_enc * H * 2);
    launch_chained(im2col_time_major_kernel, dim3(2, t2_max, W), dim3(256), (size_t)0, st, (__nv_bfloat16 *)col,
                   (const __nv_bfloat16 *)c1, H, (long long)t1_max * H, d_len1, t2_max, 3, 2, 1);
    note_launches(1);
    if (rows_enc == t2_max) {
        if (gemm(hid, H, col, K2, c2p, H, c2b, EPI_GELU, nullptr, W * t2_max, K2) != 0) return -1;
    } else {
        for (int i = 0; i < W; ++i)
            if (gemm(hid + (size_t)i * rows_enc * H, H, col + (size_t)i * t2_max * K2, K2, c2p, H, c2b, EPI_GELU, nullptr, t2_max, K2) != 0)
                return -1;
    }
    int max_len2 = 0;
    for (int i = 0; i < W; ++i) max_len2 = meta[W + i] > max_len2 ? meta[W + i] : max_len2;
    encoder_layers(ws, cfg, hid, W * rows_enc, W, d_off, d_len2, max_len2, st);
    // projector on groups of four frames: [W * rows_enc / 4, 4 H] is the same memory
    const int groups = W * (rows_enc / 4);
    uint16_t *p1 = (uint16_t *)workspace_slot(WS_E_PROJ, (size_t)groups * PM * 2);
    uint16_t *p2 = (uint16_t *)workspace_slot(WS_E_FFN, (size_t)groups * D * 2);
    if (gemm(p1, PM, hid, 4 * H, p1w, PM, p1b, EPI_GELU, nullptr, groups, 4 * H) != 0) return -1;
    if (gemm(p2, D, p1, PM, p2w, D, p2b, EPI_STORE, nullptr, groups, PM) != 0) return -1;
    for (int i = 0; i < W; ++i) {
        const int tokens = meta[W + i] / 4;
        if (out_tokens_host != nullptr) out_tokens_host[i] = tokens;
        if (tokens > 0 &&
            cudaMemcpyAsync(out + (size_t)i * out_stride, p2 + (size_t)i * (rows_enc / 4) * D, (size_t)tokens * D * 2,
                            cudaMemcpyDeviceToDevice, st) != cudaSuccess)
            return -1;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
