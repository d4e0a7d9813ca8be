/*
 * Host-side wrappers around NVIDIA's own e2m1 / e4m3 converters (cuda_fp4.h,
 * cuda_fp8.h).  These are the constructors the reference's activation quantiser
 * calls (Infer-engine/cuda/nvfp4_cutlass.cu:68,79-80); both are host-callable,
 * so the oracle's encoders can be checked bit-for-bit without a GPU.
 * TEST INFRASTRUCTURE ONLY.
 *
 * Build: nvcc -O2 -shared -Xcompiler -fPIC -o libnv_cvt_host.so nv_cvt_host.cu
 */
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <stdint.h>

extern "C" void nv_e4m3_encode(const float *in, uint8_t *out, int n)
{
    for (int i = 0; i < n; i++) {
        __nv_fp8_e4m3 v(in[i]);
        out[i] = v.__x;
    }
}

extern "C" void nv_e4m3_decode(const uint8_t *in, float *out, int n)
{
    for (int i = 0; i < n; i++) {
        __nv_fp8_e4m3 v;
        v.__x = in[i];
        out[i] = (float)v;
    }
}

extern "C" void nv_e2m1_encode(const float *in, uint8_t *out, int n)
{
    for (int i = 0; i < n; i++) {
        __nv_fp4_e2m1 v(in[i]);
        out[i] = v.__x;
    }
}
