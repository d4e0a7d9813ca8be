// Device helpers for the stored FP4 format of the GLM-ASR Infer-engine checkpoints:
// e2m1 nibbles (two per byte, even k in the low nibble), one e4m3 scale byte per 16 K-elements,
// one fp32 per-tensor scale.  Restates Infer-engine/cuda/kernels.cu:96-120 of the reference.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "ptx.cuh"

namespace glmasr {

// e2m1 nibble -> float (reference fp4_lut, kernels.cu:96-99), computed without a table:
// magnitude code c = e1 e0 m;  c<2 -> c*0.5, else 2^(e-1) * (1 + m/2).
__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
    const uint32_t c = nib & 7u;
    // fp32 bits of {0, .5, 1, 1.5, 2, 3, 4, 6}: for c >= 2 this is (c << 22) + 0x3F000000
    uint32_t bits = (c << 22) + 0x3F000000u;
    bits = (c == 0u) ? 0u : ((c == 1u) ? 0x3F000000u : bits);
    bits |= (nib & 8u) << 28;
    return __uint_as_float(bits);
}

// e4m3 byte -> float exactly as the reference decodes it (kernels.cu:103-120): no NaN pattern,
// 0x7F -> 480, subnormals m/8 * 2^-6, sign bit honoured.
__device__ __forceinline__ float e4m3_to_float_ref(uint32_t b) {
    // (b & 0x7F) << 20 read as fp32 is value * 2^-120, subnormals included (fp32 keeps them).
    const float mag = __uint_as_float((b & 0x7Fu) << 20) * 1.329227995784916e36f;  // * 2^120
    return (b & 0x80u) ? -mag : mag;
}

// x / 6 rounded as the IEEE division (the quantiser's first division) in four multiply-adds: the correctly rounded
// reciprocal of 6 as r_hi + r_lo, q0 = x * (r_hi + r_lo) within one unit of the quotient, the exact residual
// x - 6 q0 from a fused multiply-add, and q0 + e * r_hi (Markstein; 6's significand is not all ones).  x outside
// [2^-60, 2^60] takes the ordinary division.
__device__ __forceinline__ float div6_exact(float x) {
    const float r_hi = 0.16666667163372040f;                        // RN(1 / 6)
    const float r_lo = -4.967053879312289e-09f;                     // fma(-6, r_hi, 1) * r_hi
    if (x >= 8.6736174e-19f && x <= 1.1529215e18f) {
        const float q0 = fmaf(x, r_hi, x * r_lo);
        const float e = fmaf(-q0, 6.0f, x);
        return fmaf(e, r_hi, q0);
    }
    return __fdiv_rn(x, 6.0f);
}

// One 16-element block of the activation quantiser (reference: Infer-engine/cuda/nvfp4_cutlass.cu:35-87):
//   amax = max |v| ; scale = (inv_in * amax) / 6 ; s8 = e4m3(scale) ; os = inv_in / float(s8)
//   q_j = e2m1(v_j * os), even j in the low nibble.
// Returns the e4m3 scale byte; lo / hi receive the 8 packed bytes.  Used by the stand-alone
// quantiser and by GEMM epilogues that emit the next GEMM's operand directly, so both produce
// the same bytes.
__device__ __forceinline__ uint32_t quantize_block16(const float (&v)[16], float inv_in, uint32_t &lo, uint32_t &hi) {
    // (three-input maximum, exact division by 6 in four multiply-adds, two products per multiply: the same bits
    // as the plain expressions above in about two thirds of the instructions)
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j += 2) amax = max3(amax, fabsf(v[j]), fabsf(v[j + 1]));
    const float scale = amax > 0.0f ? div6_exact(inv_in * amax) : 0.0f;
    const __nv_fp8_e4m3 s8(scale);
    const float scale_rounded = scale > 0.0f ? (float)s8 : 0.0f;
    const float os = scale_rounded > 0.0f ? __fdiv_rn(inv_in, scale_rounded) : 0.0f;
    const unsigned long long os2 = pack_f32x2(os, os);
    lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float x0, x1;
        unpack_f32x2(mul_f32x2(pack_f32x2(v[2 * j], v[2 * j + 1]), os2), x0, x1);
        const uint32_t q = __nv_cvt_float2_to_fp4x2(make_float2(x0, x1), __NV_E2M1,
                                                    cudaRoundNearest) & 0xFFu;
        if (j < 4) lo |= q << (8 * j);
        else hi |= q << (8 * (j - 4));
    }
    return (uint32_t)s8.__x;
}

// Same block quantiser with the second division looked up: os = inv_in / float(s8) takes one of 127 values
// per launch, so a kernel can fill os_table[s8] once (fill_os_table, IEEE divisions) and index it afterwards.
// Same bytes as quantize_block16.
__device__ __forceinline__ void fill_os_table(float *os_table, float inv_in, int tid, int nthreads) {
    for (int b = tid; b < 128; b += nthreads) {
        __nv_fp8_e4m3 s8;
        s8.__x = (__nv_fp8_storage_t)b;
        const float sr = (float)s8;
        os_table[b] = (b != 0 && b != 0x7F && sr > 0.0f) ? __fdiv_rn(inv_in, sr) : 0.0f;
    }
}

__device__ __forceinline__ uint32_t quantize_block16_lut(const float (&v)[16], float inv_in, const float *os_table, uint32_t &lo,
                                                         uint32_t &hi) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    const float scale = amax > 0.0f ? __fdiv_rn(inv_in * amax, 6.0f) : 0.0f;
    const __nv_fp8_e4m3 s8(scale);
    const uint32_t code = scale > 0.0f ? (uint32_t)s8.__x : 0u;      // scale == 0 -> os = 0 whatever the byte
    const float os = os_table[code & 0x7Fu];
    lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t q = __nv_cvt_float2_to_fp4x2(make_float2(v[2 * j] * os, v[2 * j + 1] * os), __NV_E2M1,
                                                    cudaRoundNearest) & 0xFFu;
        if (j < 4) lo |= q << (8 * j);
        else hi |= q << (8 * (j - 4));
    }
    return (uint32_t)s8.__x;
}


// quantize_block16_lut on values that are already bf16-rounded floats, with the packed multiply, the three-input
// maximum and div6_exact: the same bytes in about half the instructions.  pack_f32x2 / mul_f32x2 / max3: ptx.cuh.
__device__ __forceinline__ uint32_t quantize_block16_fast(const float (&v)[16], float inv_in, const float *os_table, uint32_t &lo,
                                                          uint32_t &hi) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; j += 2) amax = max3(amax, fabsf(v[j]), fabsf(v[j + 1]));
    const float scale = amax > 0.0f ? div6_exact(inv_in * amax) : 0.0f;
    const __nv_fp8_e4m3 s8(scale);
    const uint32_t code = scale > 0.0f ? (uint32_t)s8.__x : 0u;
    const float os = os_table[code & 0x7Fu];
    const unsigned long long os2 = pack_f32x2(os, os);
    lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float x0, x1;
        unpack_f32x2(mul_f32x2(pack_f32x2(v[2 * j], v[2 * j + 1]), os2), x0, x1);
        const uint32_t q = __nv_cvt_float2_to_fp4x2(make_float2(x0, x1), __NV_E2M1, cudaRoundNearest) & 0xFFu;
        if (j < 4) lo |= q << (8 * j);
        else hi |= q << (8 * (j - 4));
    }
    return (uint32_t)s8.__x;
}

// x / d for many x and one divisor d, each quotient rounded exactly as the IEEE division the reference's
// rmsnorm performs (x[i] / rms).  The correctly rounded reciprocal is taken once per divisor, kept as
// r_hi + r_lo, and every quotient then costs four multiply-adds: q0 = x * (r_hi + r_lo) lies within one
// unit in the last place of x / d, the residual e = x - q0 * d is exact in a fused multiply-add, and
// q0 + e * r_hi rounds to the correctly rounded quotient (Markstein's theorem; it needs r_hi = RN(1 / d)
// and a divisor whose significand is not all ones).  Operands outside the range where every intermediate
// is a normal number, zeros, infinities and NaNs take the ordinary division.
struct ExactRowDivider {
    float d, r_hi, r_lo, fast_min;
    __device__ __forceinline__ explicit ExactRowDivider(float divisor) : d(divisor) {
        r_hi = __frcp_rn(d);
        r_lo = fmaf(-d, r_hi, 1.0f) * r_hi;
        const bool ok = d > 9.094947e-13f && d < 1.0995116e12f &&                  // 2^-40 < d < 2^40
                        (__float_as_uint(d) & 0x007FFFFFu) != 0x007FFFFFu;
        fast_min = ok ? 8.6736174e-19f : __int_as_float(0x7FC00000);               // 2^-60, or NaN: never fast
    }
    __device__ __forceinline__ float operator()(float x) const {
        const float ax = fabsf(x);
        if (ax >= fast_min && ax <= 1.1529215e18f) {                               // 2^-60 .. 2^60
            const float q0 = fmaf(x, r_hi, x * r_lo);
            const float e = fmaf(-q0, d, x);
            return fmaf(e, r_hi, q0);
        }
        return __fdiv_rn(x, d);
    }
    // Two quotients with the packed forms of the same four operations (same bits as two calls of operator()).
    __device__ __forceinline__ void pair(float x0, float x1, float &o0, float &o1) const {
        const float a0 = fabsf(x0), a1 = fabsf(x1);
        if (fminf(a0, a1) >= fast_min && fmaxf(a0, a1) <= 1.1529215e18f) {
            const unsigned long long x2 = pack_f32x2(x0, x1), rh2 = pack_f32x2(r_hi, r_hi);
            const unsigned long long q0 = fma_f32x2(x2, rh2, mul_f32x2(x2, pack_f32x2(r_lo, r_lo)));
            const unsigned long long e = fma_f32x2(q0, pack_f32x2(-d, -d), x2);
            unpack_f32x2(fma_f32x2(e, rh2, q0), o0, o1);
        } else {
            o0 = (*this)(x0);
            o1 = (*this)(x1);
        }
    }
};

}  // namespace glmasr
