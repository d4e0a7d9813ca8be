// Plain SIMT GEMMs for shapes the tensor-core path does not take (K not a multiple of 256,
// missing block scales, unaligned pointers).  Same arithmetic as the tcgen05 kernels, one
// output element per thread; correctness path for odd shapes, not a performance path.
#include <cuda_bf16.h>
#include <stdint.h>

#include "fp4_format.cuh"
#include "gemm_simt.cuh"

namespace glmasr {

__device__ __forceinline__ float w_elem(const uint8_t *packed, const uint8_t *scales, int n, int k, int K) {
    const uint8_t byte = packed[(size_t)n * (K / 2) + k / 2];
    const uint32_t nib = (k & 1) ? (byte >> 4) : (byte & 0xFu);
    const float s = scales ? e4m3_to_float_ref(scales[(size_t)n * (K / 16) + k / 16]) : 1.0f;
    return e2m1_to_float(nib) * s;
}

// mode 0: x given as packed e2m1 + row-major e4m3 scales (W4A4); mode 1: bf16 x (W4A16);
// mode 2: bf16 x and bf16 w.
__global__ void simt_gemm_kernel(SimtGemmArgs a) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)a.M * a.N) return;
    const int m = (int)(idx / a.N), n = (int)(idx % a.N);
    float acc = 0.0f;
    for (int k = 0; k < a.K; ++k) {
        float xv, wv;
        if (a.mode == 0) xv = w_elem(a.x_packed, a.x_scales, m, k, a.K);
        else xv = __bfloat162float(a.x[(size_t)m * a.ldx + k]);
        if (a.mode == 2) wv = __bfloat162float(a.w_bf16[(size_t)n * a.K + k]);
        else wv = w_elem(a.w_packed, a.w_scales, n, k, a.K);
        acc = fmaf(xv, wv, acc);
    }
    float v = acc * a.alpha;
    if (a.bias) v += __bfloat162float(a.bias[n]);
    a.out[(size_t)m * a.ldo + a.col0 + n] = __float2bfloat16(v);
}

cudaError_t launch_simt_gemm(const SimtGemmArgs &a, cudaStream_t st) {
    const long long total = (long long)a.M * a.N;
    if (total <= 0) return cudaSuccess;
    simt_gemm_kernel<<<(int)((total + 127) / 128), 128, 0, st>>>(a);
    return cudaGetLastError();
}

}  // namespace glmasr
