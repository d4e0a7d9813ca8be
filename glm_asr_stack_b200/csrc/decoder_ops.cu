// Step-resident glue kernels of the batched decode step (bf16, HBM-bound).  They are not FP4
// work, but the decode step cannot run without them and the paged attention decides its time:
// 256 sequences x ~325 tokens x 28 layers of K and V are 4.8 GB per step against 0.83 GB of
// FP4 weights.
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "decoder_ops.cuh"
#include "fp4_format.cuh"
#include "runtime.cuh"

namespace glmasr {

// --------------------------------------------------------------------------------------------
// RMSNorm (reference: Infer-engine/cuda/kernels.cu:252-295): out = (x / sqrt(mean(x^2)+eps)) * w.
// The reference uses one warp per row: lane l adds x[l]^2, x[l+32]^2, ... in order, then a
// shfl_down tree.  Here a 256-thread block stages the row in shared memory with 16-byte loads,
// warp 0 repeats exactly that summation order from shared memory (so the result is bit-equal),
// and all threads normalise.
// --------------------------------------------------------------------------------------------
__global__ void rmsnorm_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ x,
                               const __nv_bfloat16 *__restrict__ weight, float eps, int rows, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __nv_bfloat16 row_s[];
    __shared__ float rms_s;
    const int row = blockIdx.x;
    if (row >= rows) return;
    const __nv_bfloat16 *xr = x + (size_t)row * dim;
    __nv_bfloat16 *orow = out + (size_t)row * dim;
    const bool vec = (dim % 8 == 0) && (((uintptr_t)xr & 15) == 0) && (((uintptr_t)orow & 15) == 0) &&
                     (((uintptr_t)weight & 15) == 0);
    if (vec) {
        for (int i = threadIdx.x; i < dim / 8; i += blockDim.x)
            reinterpret_cast<uint4 *>(row_s)[i] = reinterpret_cast<const uint4 *>(xr)[i];
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) row_s[i] = xr[i];
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float sum_sq = 0.0f;
        for (int i = threadIdx.x; i < dim; i += 32) {
            const float v = __bfloat162float(row_s[i]);
            sum_sq += v * v;
        }
        for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
        if (threadIdx.x == 0) rms_s = sqrtf(sum_sq / dim + eps);
    }
    __syncthreads();
    const float rms = rms_s;
    if (vec) {
        for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
            const uint4 xv = reinterpret_cast<const uint4 *>(row_s)[i];
            const uint4 wv = reinterpret_cast<const uint4 *>(weight)[i];
            const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float a0 = __fdiv_rn(__uint_as_float(xs[j] << 16), rms) * __uint_as_float(ws[j] << 16);
                const float a1 = __fdiv_rn(__uint_as_float(xs[j] & 0xFFFF0000u), rms) * __uint_as_float(ws[j] & 0xFFFF0000u);
                const __nv_bfloat162 b = __floats2bfloat162_rn(a0, a1);
                o[j] = *reinterpret_cast<const uint32_t *>(&b);
            }
            reinterpret_cast<uint4 *>(orow)[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x)
            orow[i] = __float2bfloat16(__fdiv_rn(__bfloat162float(row_s[i]), rms) * __bfloat162float(weight[i]));
    }
}

void launch_rmsnorm(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *weight, float eps, int rows,
                    int dim, cudaStream_t st) {
    if (rows <= 0 || dim <= 0) return;
    GLMASR_PREFER_MAX_SMEM(rmsnorm_kernel);
    launch_chained(rmsnorm_kernel, dim3(rows), dim3(256), (size_t)dim * sizeof(__nv_bfloat16), st, out, x, weight, eps, rows, dim);
}

// --------------------------------------------------------------------------------------------
// RoPE for one new token per sequence (reference: rope_batched_single_token_kernel,
// Infer-engine/cuda/decoder.cu:605-632): rotate-half, theta 10000, full head_dim, position =
// positions[seq]; same float expressions, so bit-equal.
// --------------------------------------------------------------------------------------------
__global__ void rope_single_token_kernel(__nv_bfloat16 *tensor, int ld, int col0, const int *__restrict__ positions,
                                         int num_seqs, int n_heads, int head_dim) {
    pdl_launch_dependents();
    pdl_wait();
    const int half_dim = head_dim / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= num_seqs * n_heads * half_dim) return;
    const int seq = idx / (n_heads * half_dim);
    const int head = (idx / half_dim) % n_heads;
    const int d = idx % half_dim;
    const int pos = positions[seq];
    const float inv_freq = 1.0f / powf(10000.0f, (2.0f * d) / head_dim);
    const float theta = pos * inv_freq;
    const float cos_t = cosf(theta);
    const float sin_t = sinf(theta);
    __nv_bfloat16 *base = tensor + (size_t)seq * ld + col0 + head * head_dim;
    const float v0 = __bfloat162float(base[d]);
    const float v1 = __bfloat162float(base[d + half_dim]);
    base[d] = __float2bfloat16(v0 * cos_t - v1 * sin_t);
    base[d + half_dim] = __float2bfloat16(v0 * sin_t + v1 * cos_t);
}

void launch_rope_single_token(__nv_bfloat16 *tensor, int ld, int col0, const int *positions, int num_seqs, int n_heads,
                              int head_dim, cudaStream_t st) {
    const int total = num_seqs * n_heads * (head_dim / 2);
    if (total <= 0) return;
    GLMASR_PREFER_MAX_SMEM(rope_single_token_kernel);
    launch_chained(rope_single_token_kernel, dim3((total + 255) / 256), dim3(256), 0, st, tensor, ld, col0, positions, num_seqs, n_heads, head_dim);
}

// --------------------------------------------------------------------------------------------
// The decode step's three launches between the q|k|v projection and attention as one: RoPE on
// the new token's q heads (in place), RoPE on its k heads, and the K / V rows written to the
// paged cache (reference: rope_batched_single_token_kernel, decoder.cu:605-632, twice, then
// reshape_and_cache, paged_kv.cu:70-97).  One CTA per sequence; the 64 (cos, sin) pairs of the
// position are computed once with the reference's float expressions and shared by all heads,
// so every value is bit-equal to the three separate kernels.  The rotated k is also written back
// in place, as the separate kernels leave it.
// --------------------------------------------------------------------------------------------
// 1 / 10000^(2 d / head_dim) for d < head_dim / 2, computed once per head_dim on the device with the
// reference's own float expression (so that every later use has the same bits as computing it in place)
static __device__ float g_inv_freq[512];
static int g_inv_freq_dim = 0;

__global__ void rope_inv_freq_kernel(int head_dim) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d < head_dim / 2) g_inv_freq[d] = 1.0f / powf(10000.0f, (2.0f * d) / head_dim);
}

// cos / sin of every row's position, [rows][head_dim] floats (cos for d < head_dim / 2, then sin): the values the
// kernel below computes per launch, for callers that run it once per layer on the same positions.
__global__ void rope_angles_kernel(float *__restrict__ table, const int *__restrict__ positions, int rows, int head_dim) {
    pdl_launch_dependents();
    pdl_wait();
    const int half_dim = head_dim / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * half_dim) return;
    const int row = idx / half_dim, d = idx - row * half_dim;
    const float theta = positions[row] * g_inv_freq[d];
    table[(size_t)row * head_dim + d] = cosf(theta);
    table[(size_t)row * head_dim + half_dim + d] = sinf(theta);
}

__global__ void rope_qk_cache_kernel(__nv_bfloat16 *qkv, int ld, int k_col, int v_col, const int *__restrict__ positions,
                                     const int64_t *__restrict__ slot_mapping, __nv_bfloat16 *__restrict__ key_cache,
                                     __nv_bfloat16 *__restrict__ value_cache, int q_heads, int kv_heads, int head_dim,
                                     const float *__restrict__ angles) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float cs[];            // [half_dim] cos, [half_dim] sin
    const int seq = blockIdx.x;
    const int half_dim = head_dim / 2;
    if (angles != nullptr) {                 // computed once for all layers (rope_angles_kernel: the same expressions)
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) cs[d] = angles[(size_t)seq * head_dim + d];
    } else {
        const int pos = positions[seq];
        for (int d = threadIdx.x; d < half_dim; d += blockDim.x) {
            const float theta = pos * g_inv_freq[d];
            cs[d] = cosf(theta);
            cs[half_dim + d] = sinf(theta);
        }
    }
    __syncthreads();
    __nv_bfloat16 *row = qkv + (size_t)seq * ld;
    const int64_t slot = slot_mapping[seq];
    const size_t row_elems = (size_t)kv_heads * head_dim;
    __nv_bfloat16 *kdst = key_cache + (size_t)slot * row_elems;
    __nv_bfloat16 *vdst = value_cache + (size_t)slot * row_elems;
    // one task = 8 consecutive dims d of one head and their partners d + half_dim: two 16-byte loads,
    // eight rotations, two 16-byte stores (and two more into the cache for a k head)
    const int cpt = half_dim / 8;
    const int tasks = (q_heads + kv_heads) * cpt;
    for (int t = threadIdx.x; t < tasks; t += blockDim.x) {
        const int head_all = t / cpt, c = t - head_all * cpt;
        const bool is_k = head_all >= q_heads;
        const int head = is_k ? head_all - q_heads : head_all;
        __nv_bfloat16 *base = row + (is_k ? k_col : 0) + head * head_dim;
        const uint4 lo4 = *reinterpret_cast<const uint4 *>(base + 8 * c);
        const uint4 hi4 = *reinterpret_cast<const uint4 *>(base + half_dim + 8 * c);
        const uint32_t lo[4] = {lo4.x, lo4.y, lo4.z, lo4.w}, hi[4] = {hi4.x, hi4.y, hi4.z, hi4.w};
        uint32_t o_lo[4], o_hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float r0[2], r1[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int d = 8 * c + 2 * j + e;
                const float v0 = __uint_as_float(e ? (lo[j] & 0xFFFF0000u) : (lo[j] << 16));
                const float v1 = __uint_as_float(e ? (hi[j] & 0xFFFF0000u) : (hi[j] << 16));
                const float cos_t = cs[d], sin_t = cs[half_dim + d];
                r0[e] = v0 * cos_t - v1 * sin_t;
                r1[e] = v0 * sin_t + v1 * cos_t;
            }
            const __nv_bfloat162 a = __floats2bfloat162_rn(r0[0], r0[1]);
            const __nv_bfloat162 b = __floats2bfloat162_rn(r1[0], r1[1]);
            o_lo[j] = *reinterpret_cast<const uint32_t *>(&a);
            o_hi[j] = *reinterpret_cast<const uint32_t *>(&b);
        }
        const uint4 out_lo = make_uint4(o_lo[0], o_lo[1], o_lo[2], o_lo[3]);
        const uint4 out_hi = make_uint4(o_hi[0], o_hi[1], o_hi[2], o_hi[3]);
        *reinterpret_cast<uint4 *>(base + 8 * c) = out_lo;
        *reinterpret_cast<uint4 *>(base + half_dim + 8 * c) = out_hi;
        if (is_k) {
            *reinterpret_cast<uint4 *>(kdst + head * head_dim + 8 * c) = out_lo;
            *reinterpret_cast<uint4 *>(kdst + head * head_dim + half_dim + 8 * c) = out_hi;
        }
    }
    // V row: 16 bytes per thread (the launcher checks the alignment)
    const int chunks = (int)(row_elems / 8);
    for (int c = threadIdx.x; c < chunks; c += blockDim.x)
        reinterpret_cast<uint4 *>(vdst)[c] = reinterpret_cast<const uint4 *>(row + v_col)[c];
}

static void ensure_inv_freq(int head_dim, cudaStream_t st) {
    if (g_inv_freq_dim != head_dim) {
        // ordinary launch: it completes before the kernels behind it start
        rope_inv_freq_kernel<<<(head_dim / 2 + 127) / 128, 128, 0, st>>>(head_dim);
        g_inv_freq_dim = head_dim;
    }
}

bool launch_rope_angles(float *table, const int *positions, int rows, int head_dim, cudaStream_t st) {
    if (rows <= 0) return true;
    if (table == nullptr || positions == nullptr || (head_dim % 2) != 0 || head_dim > 1024) return false;
    ensure_inv_freq(head_dim, st);
    const int total = rows * (head_dim / 2);
    launch_chained(rope_angles_kernel, dim3((total + 255) / 256), dim3(256), (size_t)0, st, table, positions, rows, head_dim);
    return true;
}

bool launch_rope_qk_cache(__nv_bfloat16 *qkv, int ld, int k_col, int v_col, const int *positions,
                          const int64_t *slot_mapping, __nv_bfloat16 *key_cache, __nv_bfloat16 *value_cache, int num_seqs,
                          int q_heads, int kv_heads, int head_dim, cudaStream_t st, const float *angles) {
    const int row_elems = kv_heads * head_dim;
    if (num_seqs <= 0) return true;
    if ((head_dim % 16) != 0 || head_dim > 1024 || (row_elems % 8) != 0 || (ld % 8) != 0 || (v_col % 8) != 0 || (k_col % 8) != 0 ||
        (((uintptr_t)qkv | (uintptr_t)value_cache | (uintptr_t)key_cache) & 15) != 0)
        return false;
    ensure_inv_freq(head_dim, st);
    GLMASR_PREFER_MAX_SMEM(rope_qk_cache_kernel);
    launch_chained(rope_qk_cache_kernel, dim3(num_seqs), dim3(256), (size_t)head_dim * sizeof(float), st, qkv, ld, k_col, v_col, positions, slot_mapping,
                                                                             key_cache, value_cache, q_heads, kv_heads,
                                                                             head_dim, angles);
    return true;
}

// 16 bf16-representable floats as 32 contiguous bytes (dst 16-byte aligned)
__device__ __forceinline__ void store_bf16x16(__nv_bfloat16 *dst, const float (&v)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&b);
    }
    reinterpret_cast<uint4 *>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4 *>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// --------------------------------------------------------------------------------------------
// RMSNorm whose result goes straight into the next W4A4 GEMM: same normalisation as rmsnorm_kernel
// (bit-equal bf16 values), then the activation quantiser on 16-element blocks of that bf16 row
// (quantize_block16) with the scales written in the 128x4-tiled layout.  One CTA per row.
// --------------------------------------------------------------------------------------------
__global__ void rmsnorm_quant_kernel(uint8_t *__restrict__ q_packed, uint8_t *__restrict__ q_sf, int sf_chunks,
                                     const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ weight,
                                     float eps, float inv_in, int rows, int dim, __nv_bfloat16 *__restrict__ normed_out) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __nv_bfloat16 row_s[];
    __shared__ float rms_s;
    const int row = blockIdx.x;
    if (row >= rows) return;
    const __nv_bfloat16 *xr = x + (size_t)row * dim;
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x)
        reinterpret_cast<uint4 *>(row_s)[i] = reinterpret_cast<const uint4 *>(xr)[i];
    __syncthreads();
    if (threadIdx.x < 32) {
        float sum_sq = 0.0f;
        for (int i = threadIdx.x; i < dim; i += 32) {
            const float v = __bfloat162float(row_s[i]);
            sum_sq += v * v;
        }
        for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
        if (threadIdx.x == 0) rms_s = sqrtf(sum_sq / dim + eps);
    }
    __syncthreads();
    const float rms = rms_s;
    for (int b = threadIdx.x; b < dim / 16; b += blockDim.x) {
        float v[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 xv = reinterpret_cast<const uint4 *>(row_s)[2 * b + h];
            const uint4 wv = reinterpret_cast<const uint4 *>(weight)[2 * b + h];
            const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float a0 = __fdiv_rn(__uint_as_float(xs[j] << 16), rms) * __uint_as_float(ws[j] << 16);
                const float a1 = __fdiv_rn(__uint_as_float(xs[j] & 0xFFFF0000u), rms) * __uint_as_float(ws[j] & 0xFFFF0000u);
                v[8 * h + 2 * j] = __bfloat162float(__float2bfloat16(a0));
                v[8 * h + 2 * j + 1] = __bfloat162float(__float2bfloat16(a1));
            }
        }
        if (normed_out != nullptr) store_bf16x16(normed_out + (size_t)row * dim + (size_t)b * 16, v);
        uint32_t lo, hi;
        const uint32_t sf = quantize_block16(v, inv_in, lo, hi);
        *reinterpret_cast<uint2 *>(q_packed + (size_t)row * (dim / 2) + (size_t)b * 8) = make_uint2(lo, hi);
        const int rem = row & 127;
        q_sf[((((size_t)(row >> 7) * sf_chunks + (b >> 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4 + (b & 3)] = (uint8_t)sf;
    }
}

// Same results, one WARP per row, for batches of thousands of rows (prefill), where the CTA-per-row
// kernel above is a chain of load -> one-warp reduction -> quantise with little to overlap it.  A warp
// reads its row once, coalesced, into a private strip of shared memory (128-byte lines 144 bytes apart,
// so that every access pattern below is free of avoidable bank conflicts).  Lane i then adds x[i],
// x[i + 32], ... in that order -- the summation order of the kernel above and of the reference's rmsnorm
// -- and the shuffle tree and the arithmetic after it give the same values (the division by the row's
// rms through ExactRowDivider).  For the quantiser a lane takes line `lane` of the strip: four
// consecutive 16-element blocks, i.e. 32 contiguous output bytes and one 4-byte group of scales.
// dim = 2048 * P.
constexpr int kNormStrip = 32 * 144;      // bytes of shared memory per 2048 elements
template <int P>
__global__ void __launch_bounds__(256) rmsnorm_quant_warp_kernel(uint8_t *__restrict__ q_packed, uint8_t *__restrict__ q_sf,
                                                                int sf_chunks, const __nv_bfloat16 *__restrict__ x,
                                                                const __nv_bfloat16 *__restrict__ weight, float eps,
                                                                float inv_in, int rows, __nv_bfloat16 *__restrict__ normed_out) {
    extern __shared__ __align__(16) uint8_t strips[];
    constexpr int dim = 2048 * P;
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int row = blockIdx.x * 8 + wib;
    if (row >= rows) return;
    uint8_t *rs = strips + wib * (P * kNormStrip);
    {
        const uint4 *xr4 = reinterpret_cast<const uint4 *>(x + (size_t)row * dim);
        uint4 v[8 * P];
#pragma unroll
        for (int k = 0; k < 8 * P; ++k) v[k] = xr4[k * 32 + lane];
#pragma unroll
        for (int k = 0; k < 8 * P; ++k) {
            const int byte = 512 * k + 16 * lane;
            *reinterpret_cast<uint4 *>(rs + byte + (byte >> 7) * 16) = v[k];
        }
    }
    __syncwarp();
    float sum_sq = 0.0f;
    {
        const uint8_t *ri = rs + 2 * lane;
#pragma unroll
        for (int t = 0; t < 64 * P; ++t) {
            const uint32_t h = *reinterpret_cast<const uint16_t *>(ri + 64 * t + 16 * (t >> 1));
            const float v = __uint_as_float(h << 16);
            sum_sq += v * v;
        }
    }
    for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
    const float rms = __shfl_sync(0xFFFFFFFFu, sqrtf(sum_sq / dim + eps), 0);
    const ExactRowDivider by_rms(rms);
    const int rem = row & 127;
#pragma unroll
    for (int pass = 0; pass < P; ++pass) {
        const int b0 = pass * 128 + 4 * lane;            // first of this lane's four blocks
        const uint8_t *line = rs + pass * kNormStrip + lane * 144;
        uint32_t packed[8], sfw = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float v[16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 xv = *reinterpret_cast<const uint4 *>(line + (2 * k + h) * 16);
                const uint4 wv = reinterpret_cast<const uint4 *>(weight)[2 * (b0 + k) + h];
                const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // x / rms * w rounded to bf16, two elements per operation
                    float q0, q1, a0, a1;
                    by_rms.pair(__uint_as_float(xs[j] << 16), __uint_as_float(xs[j] & 0xFFFF0000u), q0, q1);
                    unpack_f32x2(mul_f32x2(pack_f32x2(q0, q1), pack_f32x2(__uint_as_float(ws[j] << 16), __uint_as_float(ws[j] & 0xFFFF0000u))),
                                 a0, a1);
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(a0, a1);
                    const uint32_t bw = *reinterpret_cast<const uint32_t *>(&b2);
                    v[8 * h + 2 * j] = __uint_as_float(bw << 16);
                    v[8 * h + 2 * j + 1] = __uint_as_float(bw & 0xFFFF0000u);
                }
            }
            if (normed_out != nullptr) store_bf16x16(normed_out + (size_t)row * dim + (size_t)(b0 + k) * 16, v);
            const uint32_t sf = quantize_block16(v, inv_in, packed[2 * k], packed[2 * k + 1]);
            sfw |= (sf & 0xFFu) << (8 * k);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(q_packed + (size_t)row * (dim / 2) + (size_t)b0 * 8);
        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        *reinterpret_cast<uint32_t *>(q_sf + ((((size_t)(row >> 7) * sf_chunks + (b0 >> 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4) = sfw;
    }
}

bool launch_rmsnorm_quant(uint8_t *q_packed, uint8_t *q_sf, const __nv_bfloat16 *x, const __nv_bfloat16 *weight, float eps,
                          float input_scale, int rows, int dim, cudaStream_t st, __nv_bfloat16 *normed_out) {
    if (rows <= 0) return true;
    if ((dim % 64) != 0 || (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)q_packed | (uintptr_t)normed_out) & 15) != 0 ||
        !(input_scale > 0.0f))
        return false;
    if (rows >= 2048 && (dim == 2048 || dim == 4096)) {
        const dim3 grid((rows + 7) / 8);
        if (dim == 2048) {
            launch_chained(rmsnorm_quant_warp_kernel<1>, grid, dim3(256), (size_t)(8 * kNormStrip), st, q_packed, q_sf, dim / 64, x,
                           weight, eps, 1.0f / input_scale, rows, normed_out);
        } else {
            static bool configured = false;
            if (!configured) {
                cudaFuncSetAttribute(rmsnorm_quant_warp_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * kNormStrip);
                configured = true;
            }
            launch_chained(rmsnorm_quant_warp_kernel<2>, grid, dim3(256), (size_t)(16 * kNormStrip), st, q_packed, q_sf, dim / 64, x,
                           weight, eps, 1.0f / input_scale, rows, normed_out);
        }
        return true;
    }
    GLMASR_PREFER_MAX_SMEM(rmsnorm_quant_kernel);
    launch_chained(rmsnorm_quant_kernel, dim3(rows), dim3(128), (size_t)dim * sizeof(__nv_bfloat16), st, q_packed, q_sf, dim / 64, x, weight, eps,
                   1.0f / input_scale, rows, dim, normed_out);
    return true;
}

// --------------------------------------------------------------------------------------------
// reshape_and_cache (reference: Infer-engine/cuda/paged_kv.cu:70-97): scatter each token's K and
// V rows to slot = block * block_size + offset of the paged cache
// [block][token][kv_head][dim].  16 bytes per thread.
// --------------------------------------------------------------------------------------------
__global__ void reshape_and_cache_kernel(__nv_bfloat16 *__restrict__ key_cache, __nv_bfloat16 *__restrict__ value_cache,
                                         const __nv_bfloat16 *__restrict__ key, int ldk,
                                         const __nv_bfloat16 *__restrict__ value, int ldv,
                                         const int64_t *__restrict__ slot_mapping, int num_tokens, int row_elems) {
    pdl_launch_dependents();
    pdl_wait();
    const int chunks = row_elems / 8;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= num_tokens * chunks) return;
    const int tok = idx / chunks, c = idx % chunks;
    const int64_t slot = slot_mapping[tok];
    const size_t dst = (size_t)slot * row_elems + (size_t)c * 8;
    *reinterpret_cast<uint4 *>(key_cache + dst) = *reinterpret_cast<const uint4 *>(key + (size_t)tok * ldk + c * 8);
    *reinterpret_cast<uint4 *>(value_cache + dst) = *reinterpret_cast<const uint4 *>(value + (size_t)tok * ldv + c * 8);
}

__global__ void reshape_and_cache_scalar_kernel(__nv_bfloat16 *key_cache, __nv_bfloat16 *value_cache,
                                                const __nv_bfloat16 *key, int ldk, const __nv_bfloat16 *value, int ldv,
                                                const int64_t *slot_mapping, int num_tokens, int row_elems) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= num_tokens * row_elems) return;
    const int tok = idx / row_elems, c = idx % row_elems;
    const size_t dst = (size_t)slot_mapping[tok] * row_elems + c;
    key_cache[dst] = key[(size_t)tok * ldk + c];
    value_cache[dst] = value[(size_t)tok * ldv + c];
}

void launch_reshape_and_cache(__nv_bfloat16 *key_cache, __nv_bfloat16 *value_cache, const __nv_bfloat16 *key, int ldk,
                              const __nv_bfloat16 *value, int ldv, const int64_t *slot_mapping, int num_tokens,
                              int num_kv_heads, int head_dim, int block_size, cudaStream_t st) {
    (void)block_size;   // slot * row_elems already is ((block*block_size + offset) * kv_heads + head) * dim
    const int row_elems = num_kv_heads * head_dim;
    if (num_tokens <= 0 || row_elems <= 0) return;
    const bool vec = (row_elems % 8 == 0) && (ldk % 8 == 0) && (ldv % 8 == 0) && (((uintptr_t)key & 15) == 0) &&
                     (((uintptr_t)value & 15) == 0) && (((uintptr_t)key_cache & 15) == 0) &&
                     (((uintptr_t)value_cache & 15) == 0);
    if (vec) {
        const int total = num_tokens * (row_elems / 8);
        GLMASR_PREFER_MAX_SMEM(reshape_and_cache_kernel);
        launch_chained(reshape_and_cache_kernel, dim3((total + 255) / 256), dim3(256), 0, st, key_cache, value_cache, key, ldk, value, ldv,
                                                                      slot_mapping, num_tokens, row_elems);
    } else {
        const int total = num_tokens * row_elems;
        reshape_and_cache_scalar_kernel<<<(total + 255) / 256, 256, 0, st>>>(key_cache, value_cache, key, ldk, value,
                                                                             ldv, slot_mapping, num_tokens, row_elems);
    }
}

}  // namespace glmasr

namespace glmasr {

// --------------------------------------------------------------------------------------------
// Paged GQA decode attention, head_dim 128 (reference: paged_decode_attention and its
// gqa4_h128 warp kernel, Infer-engine/cuda/paged_kv.cu:321-422, 440-519):
//   out[seq, h, :] = softmax_t( q[seq, h, :] . K[t, kv(h), :] / sqrt(128) ) V[t, kv(h), :]
// over the seq_lens[seq] cached tokens found through the block table; a negative block id masks
// its tokens; seq_len <= 0 gives zeros; the final division adds 1e-9 to the sum as the
// reference does.
//
// One CTA per (kv head, sequence); warp g handles query head kv*G + g, so all G warps read the
// same K/V rows (one HBM read, the rest L1 hits).  A lane owns 4 consecutive dims (8-byte loads,
// 256 contiguous bytes per warp per row).  Tokens are taken 8 at a time: 8 independent dot
// products and shuffle reductions in flight, one online-softmax update per 8 tokens (the
// reference updates per token; the result differs only by fp32 rounding).
// --------------------------------------------------------------------------------------------
static constexpr int kAttnTokens = 8;

__global__ void __launch_bounds__(256) paged_decode_attention_h128_kernel(
    __nv_bfloat16 *__restrict__ out, int ldo, const __nv_bfloat16 *__restrict__ query, int ldq,
    const __nv_bfloat16 *__restrict__ key_cache, const __nv_bfloat16 *__restrict__ value_cache,
    const int *__restrict__ block_tables, const int *__restrict__ seq_lens, int num_q_heads, int num_kv_heads,
    int group, int block_size, int max_blocks_per_seq, float scale) {
    const int kv_head = blockIdx.x;
    const int seq = blockIdx.y;
    const int g = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (g >= group) return;
    const int q_head = kv_head * group + g;
    const int seq_len = seq_lens[seq];
    __nv_bfloat16 *out_ptr = out + (size_t)seq * ldo + (size_t)q_head * 128 + lane * 4;
    if (seq_len <= 0) {
        *reinterpret_cast<uint2 *>(out_ptr) = make_uint2(0u, 0u);
        return;
    }
    const uint2 qraw = *reinterpret_cast<const uint2 *>(query + (size_t)seq * ldq + (size_t)q_head * 128 + lane * 4);
    const float q0 = __uint_as_float(qraw.x << 16), q1 = __uint_as_float(qraw.x & 0xFFFF0000u);
    const float q2 = __uint_as_float(qraw.y << 16), q3 = __uint_as_float(qraw.y & 0xFFFF0000u);
    const int *bt = block_tables + (size_t)seq * max_blocks_per_seq;
    const size_t row_elems = (size_t)num_kv_heads * 128;
    const size_t head_off = (size_t)kv_head * 128 + lane * 4;

    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    float run_max = -INFINITY, run_sum = 0.f;

    for (int t0 = 0; t0 < seq_len; t0 += kAttnTokens) {
        uint2 kr[kAttnTokens], vr[kAttnTokens];
        bool valid[kAttnTokens];
#pragma unroll
        for (int j = 0; j < kAttnTokens; ++j) {
            const int t = t0 + j;
            int blk = -1;
            if (t < seq_len) blk = bt[t / block_size];
            valid[j] = blk >= 0;
            kr[j] = make_uint2(0u, 0u);
            vr[j] = make_uint2(0u, 0u);
            if (valid[j]) {
                const size_t base = ((size_t)blk * block_size + (size_t)(t % block_size)) * row_elems + head_off;
                kr[j] = *reinterpret_cast<const uint2 *>(key_cache + base);
                vr[j] = *reinterpret_cast<const uint2 *>(value_cache + base);
            }
        }
        float s[kAttnTokens];
#pragma unroll
        for (int j = 0; j < kAttnTokens; ++j) {
            s[j] = q0 * __uint_as_float(kr[j].x << 16) + q1 * __uint_as_float(kr[j].x & 0xFFFF0000u) +
                   q2 * __uint_as_float(kr[j].y << 16) + q3 * __uint_as_float(kr[j].y & 0xFFFF0000u);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int j = 0; j < kAttnTokens; ++j) s[j] += __shfl_xor_sync(0xFFFFFFFFu, s[j], off);
        }
        float cmax = run_max;
#pragma unroll
        for (int j = 0; j < kAttnTokens; ++j) {
            s[j] = valid[j] ? s[j] * scale : -INFINITY;
            cmax = fmaxf(cmax, s[j]);
        }
        if (cmax == -INFINITY) continue;          // nothing valid yet
        const float corr = (run_max == -INFINITY) ? 0.f : expf(run_max - cmax);
        acc0 *= corr; acc1 *= corr; acc2 *= corr; acc3 *= corr;
        run_sum *= corr;
#pragma unroll
        for (int j = 0; j < kAttnTokens; ++j) {
            const float pj = valid[j] ? expf(s[j] - cmax) : 0.f;
            run_sum += pj;
            acc0 += pj * __uint_as_float(vr[j].x << 16);
            acc1 += pj * __uint_as_float(vr[j].x & 0xFFFF0000u);
            acc2 += pj * __uint_as_float(vr[j].y << 16);
            acc3 += pj * __uint_as_float(vr[j].y & 0xFFFF0000u);
        }
        run_max = cmax;
    }
    const float inv = 1.0f / (run_sum + 1e-9f);
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc0 * inv, acc1 * inv);
    const __nv_bfloat162 o23 = __floats2bfloat162_rn(acc2 * inv, acc3 * inv);
    *reinterpret_cast<uint2 *>(out_ptr) =
        make_uint2(*reinterpret_cast<const uint32_t *>(&o01), *reinterpret_cast<const uint32_t *>(&o23));
}

bool launch_paged_decode_attention(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *query, int ldq,
                                   const __nv_bfloat16 *key_cache, const __nv_bfloat16 *value_cache,
                                   const int *block_tables, const int *seq_lens, int num_seqs, int num_q_heads,
                                   int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                   cudaStream_t st) {
    if (head_dim != 128 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return false;
    const int group = num_q_heads / num_kv_heads;
    if (group > 8 || (ldq % 4) != 0 || (ldo % 4) != 0) return false;
    if (num_seqs <= 0) return true;
    // default: the tensor-core flash-decoding kernel; GLMASR_ATTN_SCALAR=1 keeps the scalar one (comparison runs)
    static int scalar = -1;
    if (scalar < 0) {
        const char *e = getenv("GLMASR_ATTN_SCALAR");
        scalar = (e && e[0] == '1') ? 1 : 0;
    }
    if (!scalar && launch_paged_decode_attention_mma(out, ldo, query, ldq, key_cache, value_cache, block_tables, seq_lens,
                                                     num_seqs, num_q_heads, num_kv_heads, head_dim, block_size,
                                                     max_blocks_per_seq, st))
        return true;
    const float scale = 1.0f / sqrtf((float)head_dim);
    dim3 grid(num_kv_heads, num_seqs);
    paged_decode_attention_h128_kernel<<<grid, 32 * group, 0, st>>>(out, ldo, query, ldq, key_cache, value_cache,
                                                                    block_tables, seq_lens, num_q_heads, num_kv_heads,
                                                                    group, block_size, max_blocks_per_seq, scale);
    return true;
}

// --------------------------------------------------------------------------------------------
// embedding_lookup (reference: Infer-engine/cuda/kernels.cu:712-736) and row gather / scatter
// --------------------------------------------------------------------------------------------
__global__ void embedding_lookup_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ table,
                                        const int *__restrict__ ids, int n, int dim) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    if (i >= n) return;
    const __nv_bfloat16 *row = table + (size_t)ids[i] * dim;
    __nv_bfloat16 *orow = out + (size_t)i * dim;
    if (dim % 8 == 0 && (((uintptr_t)row & 15) == 0) && (((uintptr_t)orow & 15) == 0)) {
        for (int d = threadIdx.x; d < dim / 8; d += blockDim.x)
            reinterpret_cast<uint4 *>(orow)[d] = reinterpret_cast<const uint4 *>(row)[d];
    } else {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) orow[d] = row[d];
    }
}

void launch_embedding_lookup(__nv_bfloat16 *out, const __nv_bfloat16 *table, const int *ids, int n, int dim,
                             cudaStream_t st) {
    if (n <= 0) return;
    GLMASR_PREFER_MAX_SMEM(embedding_lookup_kernel);
    launch_chained(embedding_lookup_kernel, dim3(n), dim3(256), 0, st, out, table, ids, n, dim);
}

__global__ void gather_rows_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *const *__restrict__ src_rows,
                                   int n, int dim) {
    const int i = blockIdx.x;
    if (i >= n) return;
    const __nv_bfloat16 *row = src_rows[i];
    for (int d = threadIdx.x; d < dim; d += blockDim.x) out[(size_t)i * dim + d] = row[d];
}
__global__ void scatter_rows_kernel(__nv_bfloat16 *const *__restrict__ dst_rows, const __nv_bfloat16 *__restrict__ in,
                                    int n, int dim) {
    const int i = blockIdx.x;
    if (i >= n) return;
    __nv_bfloat16 *row = dst_rows[i];
    for (int d = threadIdx.x; d < dim; d += blockDim.x) row[d] = in[(size_t)i * dim + d];
}
void launch_gather_rows(__nv_bfloat16 *out, const __nv_bfloat16 *const *src_rows, int n, int dim, cudaStream_t st) {
    if (n > 0) gather_rows_kernel<<<n, 256, 0, st>>>(out, src_rows, n, dim);
}
void launch_scatter_rows(__nv_bfloat16 *const *dst_rows, const __nv_bfloat16 *in, int n, int dim, cudaStream_t st) {
    if (n > 0) scatter_rows_kernel<<<n, 256, 0, st>>>(dst_rows, in, n, dim);
}

__global__ void gather_block_tables_kernel(int *__restrict__ dst, const int *__restrict__ tables,
                                           const int *__restrict__ rows, int n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    if (i >= n) return;
    const int *src = tables + (size_t)rows[i] * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x) dst[(size_t)i * width + d] = src[d];
}
void launch_gather_block_tables(int *dst, const int *tables, const int *rows, int n, int width, cudaStream_t st) {
    GLMASR_PREFER_MAX_SMEM(gather_block_tables_kernel);
    if (n > 0) launch_chained(gather_block_tables_kernel, dim3(n), dim3(128), 0, st, dst, tables, rows, n, width);
}

}  // namespace glmasr
