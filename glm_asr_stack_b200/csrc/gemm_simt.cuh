// SIMT GEMM for odd shapes (see gemm_simt.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glmasr {

struct SimtGemmArgs {
    int mode;                      // 0 = W4A4 (quantised x), 1 = W4A16, 2 = bf16 x bf16
    const uint8_t *x_packed;       // mode 0: [M, K/2]
    const uint8_t *x_scales;       // mode 0: [M, K/16] row-major
    const __nv_bfloat16 *x;        // modes 1, 2
    int ldx;
    const uint8_t *w_packed;
    const uint8_t *w_scales;
    const __nv_bfloat16 *w_bf16;   // mode 2
    const __nv_bfloat16 *bias;
    float alpha;
    __nv_bfloat16 *out;
    int ldo, col0;
    int M, N, K;
};

cudaError_t launch_simt_gemm(const SimtGemmArgs &a, cudaStream_t st);

}  // namespace glmasr
