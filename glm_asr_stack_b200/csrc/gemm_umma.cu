// tcgen05 GEMM for the FP4 linear path on sm_100a.
//
//   out[M, N] = epilogue( x[M, K] * W[N, K]^T )
//
// One persistent CTA per SM walks 128 x (128*NB) output tiles.  Warp roles:
//   warp 0      TMA producer: activation tile, weight tile(s), and (W4A4) the 128x4-tiled scale
//               chunks, into a ring of shared-memory stages guarded by full/empty mbarriers
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits stages
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator, apply the per-tensor scale and the
//               fused SiLU-gate / residual, 16-byte bf16 stores
//   warps 6+    (W4A16 only) dequantise packed e2m1 weights + e4m3 scales from a raw ring into
//               the 128B-swizzled bf16 operand tile the MMA reads
//
// Tokens sit on the 128 TMEM lanes (operand A), weight rows on the accumulator columns
// (operand B), so an epilogue thread owns one output row and writes contiguous bf16.
//
// Three arithmetic modes share the skeleton:
//   W4A4   kind::mxf4nvf4 block-scaled MMA; both operands packed e2m1 (256 K-elements per
//          128-byte row), scales copied shared -> tensor memory with tcgen05.cp
//          (semantics of the reference nvfp4_linear, Infer-engine/cuda/nvfp4_cutlass.cu:118-270)
//   W4A16  kind::f16 MMA on bf16 activations and weights dequantised on the fly; lut*e4m3 is
//          exact in bf16, the fp32 per-tensor scale is applied to the accumulator
//          (semantics of the reference fp4_linear, Infer-engine/cuda/kernels.cu:1297-1318,
//          without materialising the bf16 weight)
//   BF16   kind::f16 MMA on bf16 weights (reference bf16_linear, kernels.cu:1147-1193)
//
// Every mbarrier wait is bounded (ptx.cuh); on a time-out the CTA records a code in the
// status word, stops issuing work, frees its tensor memory and returns.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "fp4_format.cuh"
#include "gemm_umma.cuh"
#include "ptx.cuh"

namespace glmasr {

constexpr int next_pow2_cols(int n) { return n <= 32 ? 32 : n <= 64 ? 64 : n <= 128 ? 128 : n <= 256 ? 256 : 512; }

template <int MODE, int NB>
struct Cfg {
    static constexpr int BN = 128 * NB;
    static constexpr int A_BYTES = 128 * 128;
    static constexpr int SUB_BYTES = 128 * 128;           // one 128-row operand sub-tile
    static constexpr int B_BYTES = NB * SUB_BYTES;
    static constexpr int SF_CHUNK = 512;                  // scales of 128 rows x 4 K-blocks
    static constexpr int SF_TILE = 4 * SF_CHUNK;          // one 128-row tile x 256 K-elements
    static constexpr int SF_BYTES = MODE == GEMM_W4A4 ? (1 + NB) * SF_TILE : 0;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_BYTES;
    static constexpr int RAW_SUB = SUB_BYTES + 128 * 16;  // packed 128x128 B + scales 128x16 B
    static constexpr int RAW_STAGES = MODE == GEMM_W4A16 ? 2 : 0;
    static constexpr int RAW_STAGE_BYTES = MODE == GEMM_W4A16 ? NB * RAW_SUB : 0;
    static constexpr int STAGES = MODE == GEMM_W4A16 ? (NB == 2 ? 3 : 4) : (NB == 2 ? 4 : 6);
    static constexpr int NUM_ACC = (MODE == GEMM_W4A4 && NB == 2) ? 1 : 2;
    static constexpr int DQ_WARPS = MODE == GEMM_W4A16 ? 4 * NB : 0;
    static constexpr int THREADS = (6 + DQ_WARPS) * 32;
    static constexpr int SFA_COL = NUM_ACC * BN;          // tensor-memory column of the A scales
    static constexpr int SFB_COL = SFA_COL + 16;
    static constexpr int TMEM_NEEDED = NUM_ACC * BN + (MODE == GEMM_W4A4 ? 16 + 16 * NB : 0);
    static constexpr int TMEM_COLS = next_pow2_cols(TMEM_NEEDED);
    static constexpr int BAR_BYTES = 1024;
    static constexpr int SMEM_BYTES = 1024 + BAR_BYTES + STAGES * STAGE_BYTES + RAW_STAGES * RAW_STAGE_BYTES;
    // bytes the producer announces per stage
    static constexpr int TX_BYTES = MODE == GEMM_W4A16 ? A_BYTES : STAGE_BYTES;
    static_assert(TMEM_NEEDED <= 512, "tensor memory budget");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

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
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
        for (int i = 0; i < 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
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

__device__ __forceinline__ float silu_gate(float g, float u) {
    // same operation order as the reference SiLU-gate (Infer-engine/cuda/kernels.cu:1259-1263)
    const float sig = __fdiv_rn(1.0f, 1.0f + expf(-g));
    return (g * sig) * u;
}

// ---------------------------------------------------------------------------------------------
template <int MODE, int NB>
__global__ void __launch_bounds__(Cfg<MODE, NB>::THREADS, 1) umma_gemm_kernel(const __grid_constant__ GemmParams p) {
    using C = Cfg<MODE, NB>;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_raw = smem_u32(smem_dyn);
    const uint32_t smem_base = (smem_raw + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_dyn + (smem_base - smem_raw);

    // barrier block
    const uint32_t bar = smem_base;
    auto full_bar = [&](int s) { return bar + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar + 8u * (uint32_t)(C::STAGES + s); };
    auto tfull_bar = [&](int a) { return bar + 8u * (uint32_t)(2 * C::STAGES + a); };
    auto tempty_bar = [&](int a) { return bar + 8u * (uint32_t)(2 * C::STAGES + C::NUM_ACC + a); };
    auto rfull_bar = [&](int r) { return bar + 8u * (uint32_t)(2 * C::STAGES + 2 * C::NUM_ACC + r); };
    auto rempty_bar = [&](int r) { return bar + 8u * (uint32_t)(2 * C::STAGES + 2 * C::NUM_ACC + 2 + r); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + 512);
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem_gen + 520);
    const uint32_t tiles = smem_base + C::BAR_BYTES;
    const uint32_t raw_tiles = tiles + C::STAGES * C::STAGE_BYTES;
    auto stage_base = [&](int s) { return tiles + (uint32_t)s * C::STAGE_BYTES; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_bar(s), 1 + C::DQ_WARPS);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < C::NUM_ACC; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        for (int r = 0; r < C::RAW_STAGES; ++r) {
            mbar_init(rfull_bar(r), 1);
            mbar_init(rempty_bar(r), C::DQ_WARPS);
        }
        *abort_word = 0;
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_a);
        for (int s = 0; s < p.num_segs; ++s) tma_prefetch_desc(&p.tm_b[s]);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void *)tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = p.num_m_tiles * p.num_n_tiles;
    const int nkb = p.num_k_blocks;

    if (warp == 0) {
        // ================================ TMA producer ================================
        if (lane == 0) {
            uint32_t it = 0, raw_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int m_tile = tile % p.num_m_tiles;
                const int n_tile = tile / p.num_m_tiles;
                SubTile st[NB];
#pragma unroll
                for (int h = 0; h < NB; ++h) st[h] = resolve_subtile(p, n_tile, h, NB);
                for (int kb = 0; kb < nkb; ++kb) {
                    if constexpr (MODE == GEMM_W4A16) {
                        if ((kb & 3) == 0) {
                            const int r = raw_it & 1;
                            const uint32_t rph = (raw_it >> 1) & 1u;
                            if (!mbar_wait(rempty_bar(r), rph ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                            mbar_expect_tx(rfull_bar(r), C::RAW_STAGE_BYTES);
                            const uint32_t rb = raw_tiles + (uint32_t)r * C::RAW_STAGE_BYTES;
#pragma unroll
                            for (int h = 0; h < NB; ++h) {
                                tma_load_2d(rb + h * C::RAW_SUB, &p.tm_b[st[h].seg], rfull_bar(r), (kb >> 2) * 128, st[h].row0);
                                tma_load_2d(rb + h * C::RAW_SUB + C::SUB_BYTES, &p.tm_bs[st[h].seg], rfull_bar(r),
                                            (kb >> 2) * 16, st[h].row0);
                            }
                            ++raw_it;
                        }
                    }
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), C::TX_BYTES);
                    const uint32_t sb = stage_base(s);
                    // innermost coordinate in elements of the tensor map: bytes for packed e2m1, bf16 otherwise
                    const int kx = MODE == GEMM_W4A4 ? kb * 128 : kb * 64;
                    tma_load_2d(sb, &p.tm_a, full_bar(s), kx, m_tile * 128);
                    if constexpr (MODE != GEMM_W4A16) {
#pragma unroll
                        for (int h = 0; h < NB; ++h)
                            tma_load_2d(sb + C::A_BYTES + h * C::SUB_BYTES, &p.tm_b[st[h].seg], full_bar(s), kx, st[h].row0);
                    }
                    if constexpr (MODE == GEMM_W4A4) {
                        const uint32_t sf = sb + C::A_BYTES + C::B_BYTES;
                        bulk_load_1d(sf, p.sfa + ((size_t)m_tile * p.sf_k_chunks + (size_t)kb * 4) * C::SF_CHUNK, C::SF_TILE,
                                     full_bar(s));
#pragma unroll
                        for (int h = 0; h < NB; ++h) {
                            // a sub-tile past the end of its tensor reads tile 0 (any valid memory: its columns are never stored)
                            const int rt = st[h].ncols > 0 ? (st[h].row0 >> 7) : 0;
                            bulk_load_1d(sf + (1 + h) * C::SF_TILE,
                                         p.sfb[st[h].seg] + ((size_t)rt * p.sf_k_chunks + (size_t)kb * 4) * C::SF_CHUNK,
                                         C::SF_TILE, full_bar(s));
                        }
                    }
                    ++it;
                }
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ==================================
        if (lane == 0) {
            constexpr uint32_t idesc = MODE == GEMM_W4A4 ? idesc_nvfp4(128, C::BN) : idesc_bf16(128, C::BN);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const int acc = acc_it % C::NUM_ACC;
                const uint32_t aph = (acc_it / C::NUM_ACC) & 1u;
                if (!mbar_wait(tempty_bar(acc), aph ^ 1u, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * C::BN);
                for (int kb = 0; kb < nkb; ++kb) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = stage_base(s);
                    const uint32_t b_addr = a_addr + C::A_BYTES;
                    if constexpr (MODE == GEMM_W4A4) {
                        const uint32_t sf = a_addr + C::A_BYTES + C::B_BYTES;
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            tmem_cp_32x128b_warpx4(tmem_base + C::SFA_COL + 4 * c, smem_desc_sf_chunk(sf + c * C::SF_CHUNK));
#pragma unroll
                        for (int h = 0; h < NB; ++h)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                tmem_cp_32x128b_warpx4(tmem_base + C::SFB_COL + c * 4 * NB + 4 * h,
                                                       smem_desc_sf_chunk(sf + (1 + h) * C::SF_TILE + c * C::SF_CHUNK));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t adesc = smem_desc_sw128(a_addr + k * 32);
                        const uint64_t bdesc = smem_desc_sw128(b_addr + k * 32);
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (MODE == GEMM_W4A4)
                            umma_nvfp4(d_tmem, adesc, bdesc, idesc, accumulate, tmem_base + C::SFA_COL + 4 * k,
                                       tmem_base + C::SFB_COL + 4 * NB * k);
                        else
                            umma_bf16(d_tmem, adesc, bdesc, idesc, accumulate);
                    }
                    umma_commit(empty_bar(s));   // frees the stage once these MMAs have read it
                    ++it;
                }
                if (!ok) break;
                umma_commit(tfull_bar(acc));     // accumulator complete
                ++acc_it;
            }
        }
    } else if (warp < 6) {
        // ================================ epilogue =====================================
        const int quad = warp & 3;               // TMEM lane quadrant this warp may read
        uint32_t acc_it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int m_tile = tile % p.num_m_tiles;
            const int n_tile = tile / p.num_m_tiles;
            const int acc = acc_it % C::NUM_ACC;
            const uint32_t aph = (acc_it / C::NUM_ACC) & 1u;
            bool ok = mbar_wait(tfull_bar(acc), aph, abort_word, ST_TIMEOUT_EPILOGUE);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = m_tile * 128 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C::BN);
            __nv_bfloat16 *out_row = p.out + (size_t)row * p.ldo;

            if (p.epi == EPI_SILU_GATE) {
                if constexpr (NB == 2) {
                    const SubTile sg = resolve_subtile(p, n_tile, 0, NB);
                    const float ag = p.alpha[0], au = p.alpha[1];
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        uint32_t rg[32], ru[32];
                        tmem_ld_x32(t_row + ch * 32, rg);
                        tmem_ld_x32(t_row + 128 + ch * 32, ru);
                        tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = bf16_round(__uint_as_float(rg[i]) * ag);
                            const float u = bf16_round(__uint_as_float(ru[i]) * au);
                            v[i] = silu_gate(g, u);
                        }
                        const int nvalid = sg.ncols - ch * 32;
                        if (row_ok && nvalid > 0) store_row_chunk(out_row + sg.col0 + ch * 32, v, nvalid);
                    }
                }
            } else {
#pragma unroll
                for (int h = 0; h < NB; ++h) {
                    const SubTile st = resolve_subtile(p, n_tile, h, NB);
                    const float alpha = p.alpha[st.seg];
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        uint32_t r[32];
                        tmem_ld_x32(t_row + h * 128 + ch * 32, r);
                        tmem_ld_wait();
                        const int nvalid = st.ncols - ch * 32;
                        if (!(row_ok && nvalid > 0)) continue;
                        const int col = st.col0 + ch * 32;
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
                        if (p.bias != nullptr) {
                            float b[32];
                            load_row_chunk(p.bias + col, b, nvalid);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += b[i];
                        }
                        if (p.epi == EPI_RESIDUAL) {
                            float res[32];
                            load_row_chunk(p.residual + (size_t)row * p.ldo + col, res, nvalid);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = bf16_round(v[i]) + res[i];
                        }
                        store_row_chunk(out_row + col, v, nvalid);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            ++acc_it;
        }
    } else {
        // ================================ W4A16 dequant warps ============================
        if constexpr (MODE == GEMM_W4A16) {
            const int dq = warp - 6;
            const int h = dq >> 2;                       // weight sub-tile
            const int r = (dq & 3) * 32 + lane;          // row within the sub-tile
            const uint32_t sw = (uint32_t)(r & 7);
            uint32_t it = 0, raw_it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < nkb; ++kb) {
                    const int j = kb & 3;
                    const int rr = raw_it & 1;
                    if (j == 0) {
                        const uint32_t rph = (raw_it >> 1) & 1u;
                        ok = mbar_wait(rfull_bar(rr), rph, abort_word, ST_TIMEOUT_DEQUANT);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                        if (!ok) break;
                    }
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, abort_word, ST_TIMEOUT_DEQUANT);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    const uint32_t raw = raw_tiles + (uint32_t)rr * C::RAW_STAGE_BYTES + (uint32_t)h * C::RAW_SUB;
                    const uint32_t prow = raw + (uint32_t)r * 128;
                    const uint4 q0 = lds128(prow + ((((uint32_t)(2 * j)) ^ sw) << 4));
                    const uint4 q1 = lds128(prow + ((((uint32_t)(2 * j + 1)) ^ sw) << 4));
                    const uint32_t sc = lds32(raw + C::SUB_BYTES + (uint32_t)r * 16 + 4 * j);
                    const uint32_t dst = stage_base(s) + C::A_BYTES + (uint32_t)h * C::SUB_BYTES + (uint32_t)r * 128;
                    const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                    for (int cc = 0; cc < 8; ++cc) {
                        const __nv_bfloat162 s2 = block_scale_bf16x2((sc >> (8 * (cc >> 1))) & 0xFFu);
                        sts128(dst + ((((uint32_t)cc) ^ sw) << 4), dequant_word(words[cc], s2));
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(full_bar(s));
                        if (j == 3) mbar_arrive(rempty_bar(rr));
                    }
                    if (j == 3) ++raw_it;
                    ++it;
                }
            }
        }
    }

    // ================================ teardown ==========================================
    tc_fence_before();
    __syncthreads();
    if (*abort_word != 0) {
        // give copies that may still be in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
    }
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
template <int MODE, int NB>
static cudaError_t launch_one(const GemmParams &p, int num_ctas, cudaStream_t st) {
    using C = Cfg<MODE, NB>;
    umma_gemm_kernel<MODE, NB><<<num_ctas, C::THREADS, C::SMEM_BYTES, st>>>(p);
    return cudaGetLastError();
}

template <int MODE, int NB>
static cudaError_t init_one() {
    return cudaFuncSetAttribute(umma_gemm_kernel<MODE, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Cfg<MODE, NB>::SMEM_BYTES);
}

cudaError_t umma_gemm_init() {
    cudaError_t e;
    if ((e = init_one<GEMM_W4A4, 1>()) != cudaSuccess) return e;
    if ((e = init_one<GEMM_W4A4, 2>()) != cudaSuccess) return e;
    if ((e = init_one<GEMM_W4A16, 1>()) != cudaSuccess) return e;
    if ((e = init_one<GEMM_W4A16, 2>()) != cudaSuccess) return e;
    if ((e = init_one<GEMM_BF16, 1>()) != cudaSuccess) return e;
    if ((e = init_one<GEMM_BF16, 2>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_umma_gemm(int mode, int nb, const GemmParams &p, int num_ctas, cudaStream_t st) {
    if (mode == GEMM_W4A4) return nb == 2 ? launch_one<GEMM_W4A4, 2>(p, num_ctas, st) : launch_one<GEMM_W4A4, 1>(p, num_ctas, st);
    if (mode == GEMM_W4A16) return nb == 2 ? launch_one<GEMM_W4A16, 2>(p, num_ctas, st) : launch_one<GEMM_W4A16, 1>(p, num_ctas, st);
    return nb == 2 ? launch_one<GEMM_BF16, 2>(p, num_ctas, st) : launch_one<GEMM_BF16, 1>(p, num_ctas, st);
}

int umma_gemm_threads(int mode, int nb) {
    if (mode == GEMM_W4A16) return nb == 2 ? Cfg<GEMM_W4A16, 2>::THREADS : Cfg<GEMM_W4A16, 1>::THREADS;
    return 192;
}

int umma_gemm_smem_bytes(int mode, int nb) {
    if (mode == GEMM_W4A4) return nb == 2 ? Cfg<GEMM_W4A4, 2>::SMEM_BYTES : Cfg<GEMM_W4A4, 1>::SMEM_BYTES;
    if (mode == GEMM_W4A16) return nb == 2 ? Cfg<GEMM_W4A16, 2>::SMEM_BYTES : Cfg<GEMM_W4A16, 1>::SMEM_BYTES;
    return nb == 2 ? Cfg<GEMM_BF16, 2>::SMEM_BYTES : Cfg<GEMM_BF16, 1>::SMEM_BYTES;
}

}  // namespace glmasr
