// Launchers of the element-wise kernels (see elementwise.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glmasr {

void launch_dequant(__nv_bfloat16 *out, const uint8_t *packed, const uint8_t *scales, float global, int rows,
                    int cols, cudaStream_t st);
void launch_prequant(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *pre, int M, int K,
                     cudaStream_t st);
void launch_quantize_act(uint8_t *packed_out, uint8_t *scale_rowmajor, uint8_t *scale_swizzled,
                         const __nv_bfloat16 *x, const __nv_bfloat16 *pre, float input_scale, int M, int K,
                         int ldx, cudaStream_t st);
void launch_swizzle_scales(uint8_t *dst, const uint8_t *src, int rows, int cols, cudaStream_t st);
void launch_silu_split(__nv_bfloat16 *out, const __nv_bfloat16 *packed, int M, int N, cudaStream_t st);
void launch_silu_mul(__nv_bfloat16 *gate, const __nv_bfloat16 *up, long long n, cudaStream_t st);
void launch_residual_add(__nv_bfloat16 *out, const __nv_bfloat16 *a, const __nv_bfloat16 *b, long long n,
                         cudaStream_t st);
void launch_argmax_rows(const __nv_bfloat16 *logits, int *out_tokens, int rows, int vocab, cudaStream_t st);

}  // namespace glmasr
