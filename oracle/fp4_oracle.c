/*
 * CPU oracle for the GLM-ASR Infer-engine FP4-weight linear path, plain C.
 *
 * TEST INFRASTRUCTURE ONLY: linked by nothing in the product library.  It is a
 * second, independent restatement (the first is fp4_oracle.py) of the same
 * reference arithmetic, so the two can be checked against each other and
 * against the golden fixtures.  Each function cites the reference file:line it
 * follows (paths inside the reference project).  Parity pinning: see the
 * header of fp4_oracle.py.
 *
 * Build: gcc -O2 -fPIC -shared -ffp-contract=off -o libfp4_oracle.so fp4_oracle.c -lm
 * (-ffp-contract=off keeps float32 products and sums separate, as the
 * reference kernels compute them.)
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <string.h>

/* ---- bf16 <-> f32 (round to nearest even, as __float2bfloat16) ---- */
static inline float bf16_to_f32(uint16_t b)
{
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if (f != f) return 0x7FFF;
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* Infer-engine/cuda/kernels.cu:96-99 */
static const float kE2M1[16] = {
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* Infer-engine/cuda/kernels.cu:103-120: every pattern is a number (0x7F -> 480). */
float oracle_e4m3_decode(uint8_t x)
{
    int sign = (x >> 7) & 1;
    int e = (x >> 3) & 0x0F;
    int m = x & 7;
    float v;
    if (e == 0) {
        v = ((float)m / 8.0f) * 0.015625f;
    } else {
        v = (8.0f + (float)m) / 8.0f;
        v *= ldexpf(1.0f, e - 7);
    }
    return sign ? -v : v;
}

/*
 * __nv_fp8_e4m3(float): round to nearest even, saturate to +-448, NaN -> 0x7F
 * (constructor used at Infer-engine/cuda/nvfp4_cutlass.cu:68).
 * Bit-twiddled independently of the table search used by the numpy oracle.
 */
uint8_t oracle_e4m3_encode(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7F;                 /* NaN */
    float af;
    memcpy(&af, &a, 4);
    if (af >= 464.0f) return sign | 0x7E;             /* would round past 448 */
    if (af < 0.0009765625f) return sign;              /* < 2^-10 -> 0 (tie at 2^-10 -> even 0 handled below) */
    /* quantum: 2^-9 for subnormals (|x| < 2^-6), else 2^(e-3) */
    int e;
    (void)frexpf(af, &e);                             /* af = m * 2^e, m in [0.5,1) => exponent = e-1 */
    int ex = e - 1;
    if (ex < -6) ex = -6;
    float q = ldexpf(1.0f, ex - 3);
    float n = af / q;                                 /* exact: power-of-two scaling */
    float r = nearbyintf(n);                          /* RNE in the default rounding mode */
    float v = r * q;
    if (v > 448.0f) v = 448.0f;
    /* re-encode v (exactly representable) */
    if (v == 0.0f) return sign;
    int e2;
    float m2 = frexpf(v, &e2);                        /* v = m2*2^e2, m2 in [0.5,1) */
    int exp_unb = e2 - 1;
    if (exp_unb < -6) {                               /* subnormal: v = mant/8 * 2^-6 */
        int mant = (int)(v * 512.0f);
        return sign | (uint8_t)mant;
    }
    int mant = (int)((m2 * 2.0f - 1.0f) * 8.0f);
    return sign | (uint8_t)(((exp_unb + 7) << 3) | mant);
}

/* __nv_fp4_e2m1(float): RNE, saturate to +-6 (Infer-engine/cuda/nvfp4_cutlass.cu:79-80). */
uint8_t oracle_e2m1_encode(float f)
{
    uint8_t sign = signbit(f) ? 8 : 0;
    float a = fabsf(f);
    uint8_t c;
    if (a != a) return 7;
    /* midpoints between {0,.5,1,1.5,2,3,4,6}; ties go to the even code */
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return sign | c;
}

/* Infer-engine/cuda/kernels.cu:188-232 */
void oracle_fp4_dequant_to_bf16(uint16_t *out, const uint8_t *packed_w, const uint8_t *block_scales,
                                float global_scale, int rows, int cols)
{
    int prow = (cols + 1) / 2, srow = (cols + 15) / 16;
    for (int r = 0; r < rows; r++) {
        for (int c = 0; c < cols; c++) {
            uint8_t byte = packed_w[(size_t)r * prow + c / 2];
            uint8_t nib = (c & 1) ? (byte >> 4) & 0x0F : byte & 0x0F;
            float s = block_scales ? oracle_e4m3_decode(block_scales[(size_t)r * srow + c / 16]) : 1.0f;
            float v = kE2M1[nib] * s;
            v = v * global_scale;
            out[(size_t)r * cols + c] = f32_to_bf16(v);
        }
    }
}

/* Infer-engine/cuda/nvfp4_cutlass.cu:35-87 (rows < M only; pad rows get scale 0 in the reference). */
void oracle_quantize_bf16_to_fp4(uint8_t *packed_out, uint8_t *scale_out, const uint16_t *x,
                                 const uint16_t *pre, float input_scale, int M, int K)
{
    float inv_in = 1.0f / input_scale;
    for (int m = 0; m < M; m++) {
        for (int b = 0; b < K / 16; b++) {
            float v[16], amax = 0.0f;
            for (int i = 0; i < 16; i++) {
                int k = b * 16 + i;
                float p = pre ? bf16_to_f32(pre[k]) : 1.0f;
                v[i] = bf16_to_f32(x[(size_t)m * K + k]) * p;
                if (fabsf(v[i]) > amax) amax = fabsf(v[i]);
            }
            float scale = amax > 0.0f ? (inv_in * amax / 6.0f) : 0.0f;
            uint8_t sb = oracle_e4m3_encode(scale);
            float sr = scale > 0.0f ? oracle_e4m3_decode(sb) : 0.0f;
            float os = sr > 0.0f ? inv_in / sr : 0.0f;
            scale_out[(size_t)m * (K / 16) + b] = sb;
            for (int i = 0; i < 8; i++) {
                uint8_t q0 = oracle_e2m1_encode(v[2 * i] * os);
                uint8_t q1 = oracle_e2m1_encode(v[2 * i + 1] * os);
                packed_out[(size_t)m * (K / 2) + b * 8 + i] = (uint8_t)((q0 & 0x0F) | ((q1 & 0x0F) << 4));
            }
        }
    }
}

/* Infer-engine/cuda/nvfp4_cutlass.cu:101-109 */
size_t oracle_swizzled_scale_index(int r, int c, int col_tiles)
{
    int ty = r / 128, rem = r % 128;
    return ((((size_t)ty * col_tiles + c / 4) * 32 + rem % 32) * 4 + rem / 32) * 4 + c % 4;
}

/*
 * Infer-engine/cuda/kernels.cu:1297-1318 (fp4_linear): optional pre-quant scaling
 * rounded to bf16, whole-weight dequant rounded to bf16, fp32-accumulate GEMM
 * (k ascending here; cuBLAS leaves the order unspecified), bf16 out.
 * w_bf16 is caller scratch of N*K elements (the reference's weight_scratch).
 */
void oracle_fp4_linear(uint16_t *out, uint16_t *w_bf16, const uint16_t *x, const uint8_t *w_packed,
                       const uint8_t *w_scales, float global, const uint16_t *pre, int M, int N, int K)
{
    oracle_fp4_dequant_to_bf16(w_bf16, w_packed, w_scales, global, N, K);
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) {
                float xv = bf16_to_f32(x[(size_t)m * K + k]);
                if (pre) xv = bf16_to_f32(f32_to_bf16(xv * bf16_to_f32(pre[k])));
                acc += xv * bf16_to_f32(w_bf16[(size_t)n * K + k]);
            }
            out[(size_t)m * N + n] = f32_to_bf16(acc);
        }
    }
}

/* Infer-engine/cuda/kernels.cu:1252-1264 */
void oracle_silu_mul_split_packed(uint16_t *out, const uint16_t *packed, int M, int N)
{
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float g = bf16_to_f32(packed[(size_t)m * 2 * N + n]);
            float u = bf16_to_f32(packed[(size_t)m * 2 * N + N + n]);
            float sig = 1.0f / (1.0f + expf(-g));
            out[(size_t)m * N + n] = f32_to_bf16((g * sig) * u);
        }
}

/* Infer-engine/cuda/kernels.cu:741-752 */
void oracle_residual_add(uint16_t *out, const uint16_t *a, const uint16_t *b, int n)
{
    for (int i = 0; i < n; i++) out[i] = f32_to_bf16(bf16_to_f32(a[i]) + bf16_to_f32(b[i]));
}
