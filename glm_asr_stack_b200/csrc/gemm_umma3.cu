// W4A4 GEMM on CTA pairs, SiLU-gate epilogues only, with SIXTEEN epilogue warps per CTA.
// Pipeline, barrier protocol and tile geometry: gemm_umma_pair.cuh (shared with gemm_umma2.cu); what
// differs is the epilogue.  With the activation quantiser folded in, the SiLU-gate epilogue of eight
// warps (two per sub-partition, ~0.25 instructions per clock each) takes longer than a tile's MMAs and
// the kernel runs at the epilogue's pace.  Here every warp owns 32 rows x 32 outputs, works on 16
// outputs at a time (96 registers per thread) and four warps share a sub-partition, so the
// arithmetic of one warp hides the tensor-memory and MUFU latencies of the others.
//   warp 0: producer (activations + their scales); warp 1: MMA issuer; warps 2..17: epilogue,
//   lane quarter = warp % 4, output slice = (warp - 2) / 4; warp 18: producer (weights + scales).
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "fp4_format.cuh"
#include "gemm_device.cuh"
#include "gemm_umma.cuh"
#include "gemm_umma_pair.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

// 32 rows x 32 bf16 (64B-swizzled) of output staging per epilogue warp; barriers and flags in the first KB of
// the barrier block, the quantiser look-up table in the second
using Pair16Cfg = PairCfgT<16, 32 * 64, 2048>;

__global__ void __launch_bounds__(640, 1) umma_gemm_pair16_kernel(const __grid_constant__ GemmParams p) {
    using C = Pair16Cfg;
    extern __shared__ uint8_t smem_dyn[];
    PairCtx<C> ctx = pair_setup_begin<C>(p, smem_dyn);
    float *os_table = reinterpret_cast<float *>(ctx.smem_gen + 1024);
    if (p.q_packed != nullptr) fill_os_table(os_table, p.q_inv_in, (int)threadIdx.x, (int)blockDim.x);
    pair_setup_finish<C>(p, ctx);

    const int warp = ctx.warp, lane = ctx.lane;
    if (warp == 0 || warp == C::PRODUCER_B_WARP) {
        pair_producer<C>(p, ctx);
    } else if (warp == 1) {
        pair_mma_issuer<C>(p, ctx);
    } else {
        // ================================ epilogue (both CTAs) ==========================
        const uint32_t rank = ctx.rank, tmem_base = ctx.tmem_base, tiles = ctx.tiles;
        const int pair = ctx.pair, num_pairs = ctx.num_pairs, num_m_pairs = ctx.num_m_pairs, total_tiles = ctx.total_tiles;
        volatile int *abort_word = ctx.abort_word;
        auto tfull_bar = [&](int a) { return ctx.tfull_bar(a); };
        auto tempty_bar = [&](int a) { return ctx.tempty_bar(a); };
        const uint32_t tovl_bar = ctx.tovl_bar();
        const bool dbg = GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr;
        unsigned long long dbg_acc[4] = {0, 0, 0, 0};
        (void)dbg_acc;
        const int quad = warp & 3;               // tensor-memory lane quarter this warp may read
        const int slice = (warp - 2) >> 2;       // outputs [32 slice, +32) of the tile's 128
        const uint32_t tempty0 = mapa_shared(tempty_bar(0), 0);      // tempty[a] = tempty0 + 8 a
        const uint32_t tovl0 = mapa_shared(tovl_bar, 0);
        // bf16 output staging: 32 rows x 64 bytes per warp, 16-byte chunks at (chunk ^ (row / 2 % 4)): the
        // layout a 64B-swizzled TMA store reads back
        const uint32_t out_stage = tiles + C::STAGES * C::STAGE_BYTES + (uint32_t)(warp - 2) * C::OUT_STAGE_BYTES;
        const bool store_leader = elect_one();
        uint32_t acc_it = 0;
        for (int tile = pair; tile < total_tiles; tile += num_pairs) {
            const int m_tile = (tile % num_m_pairs) * 2 + (int)rank;
            const int n_tile = tile / num_m_pairs;
            const int acc = acc_it & 1;
            const uint32_t aph = (acc_it >> 1) & 1u;
            DBG_T0();
            bool ok = mbar_wait(tfull_bar(acc), aph, abort_word, ST_TIMEOUT_EPILOGUE);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            DBG_ACC(0);
            tc_fence_after();
            const int row = m_tile * 128 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C::ACC_STRIDE);
            __nv_bfloat16 *out_row = p.out + (size_t)row * p.ldo;
            // gate columns [32 slice, +32) pair with up columns [128 + 32 slice, +32).  The shared physical
            // columns [192, 256) are up columns of slices 2, 3 in accumulator 0 and gate columns of slices
            // 0, 1 in accumulator 1: those warps read them first and release them at once.
            const bool kept_is_gate = acc == 1;
            const bool owns_shared = kept_is_gate ? slice < 2 : slice >= 2;
            const SubTile sg = resolve_subtile(p, n_tile, 0, 2);
            const float ag = p.alpha[0], au = p.alpha[1];
            const uint32_t g_col = t_row + slice * 32, u_col = t_row + 128 + slice * 32;
            uint32_t kept[16];                   // the owner's 32 shared values: scaled, bf16-rounded, packed
            if (owns_shared) {
                uint32_t k0[32];
                tmem_ld_x32(kept_is_gate ? g_col : u_col, k0);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tovl0);
                const float sk = kept_is_gate ? ag : au;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(k0[2 * i]) * sk, __uint_as_float(k0[2 * i + 1]) * sk);
                    kept[i] = *reinterpret_cast<const uint32_t *>(&b2);
                }
            }
            const int nvalid_w = sg.ncols - slice * 32;           // valid outputs of this warp
            const bool box_tma = p.tma_store && p.q_packed == nullptr && nvalid_w >= 32;
            // quantised output: the warp's 32 rows x 16 bytes of codes also leave through a bulk tensor store (tm_out
            // then describes the code matrix), because 32 scattered 16-byte stores per instruction cost more
            // load/store-unit time than the whole quantiser
            const bool q_tma = p.tma_store && p.q_packed != nullptr && nvalid_w >= 32;
            if (box_tma || q_tma) {              // the previous store of this warp must have finished reading the buffer
                if (store_leader) bulk_wait_read_all();
                __syncwarp();
            }
            uint32_t q_first_lo = 0, q_first_hi = 0, sf_first = 0;       // quantised first half, stored with the second
#pragma unroll 1
            for (int it = 0; it < 2; ++it) {     // 16 outputs per pass
                // two values per multiply / conversion (scale_round_bf16_x2, silu_gate_x2: the same bits as the scalar
                // forms): this epilogue shares its issue slots with the MMA and producer warps
                float g[16], u[16];
                const unsigned long long ag2 = pack_f32x2(ag, ag), au2 = pack_f32x2(au, au);
                if (!owns_shared) {
                    uint32_t a[16], b[16];
                    tmem_ld_x16(g_col + it * 16, a);
                    tmem_ld_x16(u_col + it * 16, b);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        scale_round_bf16_x2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1]), ag2, g[2 * i], g[2 * i + 1]);
                        scale_round_bf16_x2(__uint_as_float(b[2 * i]), __uint_as_float(b[2 * i + 1]), au2, u[2 * i], u[2 * i + 1]);
                    }
                } else {
                    uint32_t a[16];
                    tmem_ld_x16((kept_is_gate ? u_col : g_col) + it * 16, a);
                    tmem_ld_wait();
                    const unsigned long long sa2 = kept_is_gate ? au2 : ag2;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t kw = it == 0 ? kept[i] : kept[8 + i];
                        const float k_lo = __uint_as_float(kw << 16), k_hi = __uint_as_float(kw & 0xFFFF0000u);
                        float x_lo, x_hi;
                        scale_round_bf16_x2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1]), sa2, x_lo, x_hi);
                        g[2 * i] = kept_is_gate ? k_lo : x_lo;
                        g[2 * i + 1] = kept_is_gate ? k_hi : x_hi;
                        u[2 * i] = kept_is_gate ? x_lo : k_lo;
                        u[2 * i + 1] = kept_is_gate ? x_hi : k_hi;
                    }
                }
                if (it == 1) {                   // every column of this warp is in registers: hand the accumulator back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * (uint32_t)acc);
                    DBG_ACC(1);
                }
                float v[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) silu_gate_x2(g[2 * i], g[2 * i + 1], u[2 * i], u[2 * i + 1], v[2 * i], v[2 * i + 1]);
                const int c0 = slice * 32 + it * 16;
                const int col = sg.col0 + c0;
                const int nvalid = sg.ncols - c0;
                if (p.q_packed != nullptr) {
                    // the next GEMM's operand: quantise the bf16-rounded products of this 16-column block
#pragma unroll
                    for (int i = 0; i < 8; ++i) round_bf16_x2(v[2 * i], v[2 * i + 1], v[2 * i], v[2 * i + 1]);
                    uint32_t qlo, qhi, sf;
                    if (GLMASR_EXP(p, 8)) {           // timing experiment: no quantiser arithmetic (wrong results)
                        qlo = __float_as_uint(v[0]), qhi = __float_as_uint(v[9]), sf = __float_as_uint(v[3]) & 0x7Fu;
                    } else {
                        sf = quantize_block16_fast(v, p.q_inv_in, os_table, qlo, qhi);
                    }
                    if (it == 0) {
                        q_first_lo = qlo, q_first_hi = qhi, sf_first = sf;
                    } else if (q_tma) {
                        sts128(out_stage + (uint32_t)lane * 16, make_uint4(q_first_lo, q_first_hi, qlo, qhi));
                        if (row_ok && !GLMASR_EXP(p, 4 | 16)) {
                            const int col0 = col - 16;
                            uint8_t *sfp = p.q_sf + ((size_t)m_tile * p.q_sf_chunks + (col0 >> 6)) * 512 + lane * 16 + quad * 4 +
                                           ((col0 >> 4) & 3);
                            *reinterpret_cast<uint16_t *>(sfp) = (uint16_t)(sf_first | (sf << 8));
                        }
                    } else if (row_ok && nvalid >= 16 && !GLMASR_EXP(p, 4)) {
                        // both halves at once: 16 bytes of codes and the two scale bytes of this warp's 32 outputs
                        const int col0 = col - 16;
                        *reinterpret_cast<uint4 *>(p.q_packed + (size_t)row * p.q_ld + (col0 >> 1)) =
                            make_uint4(q_first_lo, q_first_hi, qlo, qhi);
                        // tiled scale layout: chunk (row tile, col / 64), byte (row % 32) * 16 + (row / 32 % 4) * 4 + block
                        uint8_t *sfp = p.q_sf + ((size_t)m_tile * p.q_sf_chunks + (col0 >> 6)) * 512 + lane * 16 + quad * 4 +
                                       ((col0 >> 4) & 3);
                        *reinterpret_cast<uint16_t *>(sfp) = (uint16_t)(sf_first | (sf << 8));
                    }
                    continue;
                }
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                    w[i] = *reinterpret_cast<const uint32_t *>(&b2);
                }
                if (box_tma) {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        sts128(out_stage + (uint32_t)lane * 64 + ((((uint32_t)(it * 2 + j)) ^ (((uint32_t)lane >> 1) & 3u)) << 4),
                               make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]));
                } else if (row_ok && nvalid > 0 && !GLMASR_EXP(p, 4)) {
                    Packed16 pk;
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk.w[i] = i < 8 ? w[i] : 0u;
                    if (nvalid >= 16 && (((uintptr_t)(out_row + col)) & 15) == 0) {
                        uint4 *d4 = reinterpret_cast<uint4 *>(out_row + col);
                        d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    } else {
                        store_packed_any(out_row + col, pk, nvalid < 16 ? nvalid : 16);
                    }
                }
            }
            if ((box_tma || q_tma) && !GLMASR_EXP(p, 4)) {
                fence_proxy_async_smem();
                __syncwarp();
                if (store_leader) {
                    // bf16 output: x in elements of the [M, n_out] view; codes: x in bytes of the [M, q_ld] view
                    const int x = q_tma ? ((sg.col0 + slice * 32) >> 1) : (sg.col0 + slice * 32);
                    tma_store_2d(&p.tm_out, out_stage, x, m_tile * 128 + quad * 32);
                    bulk_commit_group();
                }
            }
            DBG_ACC(2);
            ++acc_it;
        }
        if (store_leader) bulk_wait_all();      // this warp's bulk stores are complete before the CTA exits
        __syncwarp();
        if (dbg && warp == 2 && lane == 0 && rank == 0)
            for (int i = 0; i < 3; ++i) p.dbg_cycles[pair * 16 + 8 + i] = dbg_acc[i];
    }

    pair_teardown<C>(p, ctx);
}

cudaError_t umma_gemm_pair16_init() {
    return cudaFuncSetAttribute(umma_gemm_pair16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Pair16Cfg::SMEM_BYTES);
}

cudaError_t launch_umma_gemm_pair16(const GemmParams &p, int num_pairs, cudaStream_t st) {
    return pair_launch<Pair16Cfg>(umma_gemm_pair16_kernel, p, num_pairs, st);
}

}  // namespace glmasr
