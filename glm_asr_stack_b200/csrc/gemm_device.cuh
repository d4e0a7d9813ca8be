// Device helpers shared by the tcgen05 GEMM kernels: mapping of an output tile to the weight
// tensors of a fused projection, shared-memory access by 32-bit address, the W4A16 in-kernel
// dequant, and the epilogue's row-chunk loads / stores.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "fp4_format.cuh"
#include "gemm_umma.cuh"

namespace glmasr {

struct SubTile {
    int seg;        // weight tensor
    int row0;       // first weight row of the 128-row sub-tile (may lie past the tensor: zero-filled)
    int col0;       // first output column
    int ncols;      // valid output columns (0..128)
};

__device__ __forceinline__ SubTile resolve_subtile(const GemmParams &p, int n_tile, int h, int nb) {
    SubTile t;
    if (p.epi == EPI_SILU_GATE) {
        t.seg = h;
        t.row0 = n_tile * 128;
        t.col0 = n_tile * 128;
        t.ncols = min(128, p.seg_rows[0] - t.row0);
        return t;
    }
    int g = n_tile * nb + h;
    int seg = 0, col = 0;
    while (seg < p.num_segs - 1 && g >= p.seg_subtiles[seg]) {
        g -= p.seg_subtiles[seg];
        col += p.seg_rows[seg];
        ++seg;
    }
    t.seg = seg;
    t.row0 = g * 128;
    t.col0 = col + g * 128;
    t.ncols = max(0, min(128, p.seg_rows[seg] - t.row0));
    return t;
}

// ---- shared-memory access by 32-bit shared address ---------------------------------------
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- W4A16 dequant: 8 e2m1 nibbles (one 32-bit word) times one block scale -> 8 bf16 ------
// e2m1x2 -> f16x2 is a hardware conversion; an f16 pattern shifted right by 3 reads as a bf16
// of value v * 2^-112 (zero stays zero), so one bf16x2 multiply by (scale * 2^112) yields the
// exact product lut*scale (6 significant bits) as bf16.
__device__ __forceinline__ uint32_t e2m1x2_to_scaled_bf16x2(uint32_t byte, __nv_bfloat162 s2) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
    const uint32_t hb = (uint32_t)h.x | ((uint32_t)h.y << 16);
    const uint32_t t = ((hb >> 3) & 0x0FFF0FFFu) | (hb & 0x80008000u);
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&t), s2);
    return *reinterpret_cast<const uint32_t *>(&r);
}
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __nv_bfloat162 s2) {
    uint4 o;
    o.x = e2m1x2_to_scaled_bf16x2(w & 0xFFu, s2);
    o.y = e2m1x2_to_scaled_bf16x2((w >> 8) & 0xFFu, s2);
    o.z = e2m1x2_to_scaled_bf16x2((w >> 16) & 0xFFu, s2);
    o.w = e2m1x2_to_scaled_bf16x2(w >> 24, s2);
    return o;
}
__device__ __forceinline__ __nv_bfloat162 block_scale_bf16x2(uint32_t scale_byte) {
    // e4m3 decoded as the reference does (no NaN pattern), times 2^112; exact in bf16.
    const float s = e4m3_to_float_ref(scale_byte) * 5.192296858534828e33f;  // 2^112
    return __floats2bfloat162_rn(s, s);
}

// ---- epilogue helpers ----------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

__device__ __forceinline__ void store_row_chunk(__nv_bfloat16 *dst, const float (&v)[32], int nvalid) {
    if (nvalid >= 32 && (((uintptr_t)dst & 15) == 0)) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&b);
        }
        if (((uintptr_t)dst & 31) == 0) {
            // 32-byte stores: every store fills a whole 32-byte L2 sector
#pragma unroll
            for (int i = 0; i < 2; ++i)
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * i),
                             "r"(w[8 * i]), "r"(w[8 * i + 1]), "r"(w[8 * i + 2]), "r"(w[8 * i + 3]), "r"(w[8 * i + 4]),
                             "r"(w[8 * i + 5]), "r"(w[8 * i + 6]), "r"(w[8 * i + 7])
                             : "memory");
        } else {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
            for (int i = 0; i < 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < nvalid) dst[i] = __float2bfloat16(v[i]);
    }
}

__device__ __forceinline__ void load_row_chunk(const __nv_bfloat16 *src, float (&v)[32], int nvalid) {
    if (nvalid >= 32 && (((uintptr_t)src & 15) == 0)) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 q = s4[i];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = i < nvalid ? __bfloat162float(src[i]) : 0.0f;
    }
}

// ---- compact forms for kernels whose epilogue must stay small in the instruction cache ------------
// 32 bf16 values of one row chunk, packed two per register.
struct Packed16 {
    uint32_t w[16];
};

__device__ __forceinline__ Packed16 pack_bf16(const float (&v)[32]) {
    Packed16 pk;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        pk.w[i] = *reinterpret_cast<const uint32_t *>(&b);
    }
    return pk;
}

__device__ __forceinline__ void unpack_bf16(const Packed16 &pk, float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        v[2 * i] = __uint_as_float(pk.w[i] << 16);
        v[2 * i + 1] = __uint_as_float(pk.w[i] & 0xFFFF0000u);
    }
}

// Rare paths (row tails, unaligned pointers), kept out of line on purpose.
static __device__ __noinline__ void store_packed_any(__nv_bfloat16 *dst, Packed16 pk, int nvalid) {
    uint16_t *d = reinterpret_cast<uint16_t *>(dst);
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
        if (i < nvalid) d[i] = (uint16_t)(pk.w[i >> 1] >> ((i & 1) * 16));
}

static __device__ __noinline__ Packed16 load_packed_any(const __nv_bfloat16 *src, int nvalid) {
    const uint16_t *s16 = reinterpret_cast<const uint16_t *>(src);
    Packed16 pk;
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {
        const uint32_t lo = 2 * i < nvalid ? s16[2 * i] : 0u;
        const uint32_t hi = 2 * i + 1 < nvalid ? s16[2 * i + 1] : 0u;
        pk.w[i] = lo | (hi << 16);
    }
    return pk;
}

// Row chunk to global memory: 32-byte stores when the chunk is whole and 32-byte aligned.
__device__ __forceinline__ void store_packed(__nv_bfloat16 *dst, const Packed16 &pk, int nvalid) {
    if (nvalid >= 32 && (((uintptr_t)dst & 31) == 0)) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * i),
                         "r"(pk.w[8 * i]), "r"(pk.w[8 * i + 1]), "r"(pk.w[8 * i + 2]), "r"(pk.w[8 * i + 3]),
                         "r"(pk.w[8 * i + 4]), "r"(pk.w[8 * i + 5]), "r"(pk.w[8 * i + 6]), "r"(pk.w[8 * i + 7])
                         : "memory");
    } else {
        store_packed_any(dst, pk, nvalid);
    }
}

__device__ __forceinline__ Packed16 load_packed(const __nv_bfloat16 *src, int nvalid) {
    if (nvalid >= 32 && (((uintptr_t)src & 15) == 0)) {
        Packed16 pk;
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 q = s4[i];
            pk.w[4 * i] = q.x, pk.w[4 * i + 1] = q.y, pk.w[4 * i + 2] = q.z, pk.w[4 * i + 3] = q.w;
        }
        return pk;
    }
    return load_packed_any(src, nvalid);
}

__device__ __forceinline__ float gelu_tanh(float v) {
    // 0.5 v (1 + tanh(0.79788456 (v + 0.044715 v^3))) as in the reference (Infer-engine/cuda/kernels.cu:364-372,
    // 844-856), with the hardware tanh (relative error ~2^-11, below the bf16 output's resolution)
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.79788456f * (v + 0.044715f * v * v * v)));
    return 0.5f * v * (1.0f + t);
}

__device__ __forceinline__ float silu_gate(float g, float u) {
    // (g * sigmoid(g)) * u as in the reference SiLU-gate (Infer-engine/cuda/kernels.cu:1259-1263), with the
    // hardware exponential and reciprocal: the fused epilogue is compared with the reference within the bf16
    // tolerance anyway (its inputs come from a differently ordered accumulation), and the exact expf + IEEE
    // division made the epilogue slower than the tile's MMAs.  Six instructions: the flush-to-zero forms of
    // ex2 / rcp need no range fix-up code around them, and a flushed exp(-g) (g > 87) or a flushed 1 / (1 + e)
    // (e > 2^126, g < -87) gives the same product as the unflushed one to the last bit of a bf16.
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return (g * r) * u;
}


// ---- the same arithmetic two values at a time (same bits; about two thirds of the instructions) ----------
// bf16(a0 * s), bf16(a1 * s) back as floats: one packed multiply, one two-input conversion, two unpack operations
__device__ __forceinline__ void scale_round_bf16_x2(float a0, float a1, unsigned long long s2, float &o0, float &o1) {
    float x0, x1;
    unpack_f32x2(mul_f32x2(pack_f32x2(a0, a1), s2), x0, x1);
    const __nv_bfloat162 b = __floats2bfloat162_rn(x0, x1);
    const uint32_t w = *reinterpret_cast<const uint32_t *>(&b);
    o0 = __uint_as_float(w << 16);
    o1 = __uint_as_float(w & 0xFFFF0000u);
}
// bf16-rounded pair as floats, and the packed word (low half = first value)
__device__ __forceinline__ uint32_t round_bf16_x2(float x0, float x1, float &o0, float &o1) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(x0, x1);
    const uint32_t w = *reinterpret_cast<const uint32_t *>(&b);
    o0 = __uint_as_float(w << 16);
    o1 = __uint_as_float(w & 0xFFFF0000u);
    return w;
}
__device__ __forceinline__ void silu_gate_x2(float g0, float g1, float u0, float u1, float &v0, float &v1) {
    const unsigned long long g2 = pack_f32x2(g0, g1);
    float t0, t1, e0, e1, d0, d1, r0, r1;
    unpack_f32x2(mul_f32x2(g2, pack_f32x2(-1.4426950408889634f, -1.4426950408889634f)), t0, t1);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(t0));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(t1));
    unpack_f32x2(add_f32x2(pack_f32x2(e0, e1), pack_f32x2(1.0f, 1.0f)), d0, d1);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d1));
    unpack_f32x2(mul_f32x2(mul_f32x2(g2, pack_f32x2(r0, r1)), pack_f32x2(u0, u1)), v0, v1);
}

// cycle accounting of experiment builds: T0 opens an interval, ACC closes it into a counter
#ifdef GLMASR_EXPERIMENTS
#define DBG_T0() long long _t0 = dbg ? clock64() : 0
#define DBG_ACC(slot) do { if (dbg) { long long _t1 = clock64(); dbg_acc[slot] += (unsigned long long)(_t1 - _t0); _t0 = _t1; } } while (0)
#else
#define DBG_T0() do { } while (0)
#define DBG_ACC(slot) do { } while (0)
#endif

}  // namespace glmasr
