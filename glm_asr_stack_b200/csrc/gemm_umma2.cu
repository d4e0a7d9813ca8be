// W4A4 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a, eight epilogue warps per CTA: plain, bias,
// residual and SiLU-gate epilogues (the latter optionally emitting the next GEMM's quantised operand).
// Pipeline, barrier protocol and tile geometry: gemm_umma_pair.cuh.  This file is the epilogue:
//   warp 0: producer (activations + their scales); warp 1: MMA issuer; warps 2..9: epilogue, TMEM lane
//   quarter = warp % 4, column half = (warp - 2) / 4; warp 10: producer (weights + their scales).
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "fp4_format.cuh"
#include "gemm_device.cuh"
#include "gemm_umma.cuh"
#include <type_traits>

#include "gemm_umma_pair.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

// 32 rows x 64 bf16 (128B-swizzled) of output staging per epilogue warp; 1 KB of barriers and flags
using PairCfg = PairCfgT<8, 32 * 128, 1024>;
using PairCfgBf16 = PairCfgT<8, 32 * 128, 1024, false>;

template <bool BF16>
__global__ void __launch_bounds__(PairCfg::THREADS, 1) umma_gemm_pair_kernel(const __grid_constant__ GemmParams p) {
    using C = typename std::conditional<BF16, PairCfgBf16, PairCfg>::type;
    extern __shared__ uint8_t smem_dyn[];
    PairCtx<C> ctx = pair_setup_begin<C>(p, smem_dyn);
    pair_setup_finish<C>(p, ctx);

    const int warp = ctx.warp, lane = ctx.lane;
    if (warp == 0 || warp == C::PRODUCER_B_WARP) {
        pair_producer<C, BF16>(p, ctx);
    } else if (warp == 1) {
        pair_mma_issuer<C, BF16>(p, ctx);
    } else {
        // ================================ epilogue (both CTAs) ==========================
        const uint32_t rank = ctx.rank, tmem_base = ctx.tmem_base, tiles = ctx.tiles;
        const int pair = ctx.pair, num_pairs = ctx.num_pairs, num_m_pairs = ctx.num_m_pairs;
        volatile int *abort_word = ctx.abort_word;
        auto tfull_bar = [&](int a) { return ctx.tfull_bar(a); };
        auto tempty_bar = [&](int a) { return ctx.tempty_bar(a); };
        const uint32_t tovl_bar = ctx.tovl_bar();
        const bool dbg = GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr;
        unsigned long long dbg_acc[4] = {0, 0, 0, 0};
        (void)dbg_acc;
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;       // warps 2..9 only: the second producer took its own branch above
        const uint32_t tempty0 = mapa_shared(tempty_bar(0), 0);      // tempty[a] = tempty0 + 8 a
        const uint32_t tovl0 = mapa_shared(tovl_bar, 0);
        // output staging: each lane writes its row's 16-byte chunks at (chunk ^ (row & 7)), the layout a
        // 128B-swizzled TMA store reads back, so the warp's 32 x 64 tile leaves as one bulk store
        const uint32_t out_stage = tiles + C::STAGES * C::STAGE_BYTES + (uint32_t)(warp - 2) * C::OUT_STAGE_BYTES;
        const bool store_leader = elect_one();
        auto stage_packed = [&](const Packed16 &pk, int hch) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                sts128(out_stage + (uint32_t)lane * 128 + ((((uint32_t)(hch * 4 + j)) ^ ((uint32_t)lane & 7u)) << 4),
                       make_uint4(pk.w[4 * j], pk.w[4 * j + 1], pk.w[4 * j + 2], pk.w[4 * j + 3]));
        };
        auto stage_begin = [&]() {          // the previous store of this warp must have finished reading the buffer
            if (store_leader) bulk_wait_read_all();
            __syncwarp();
        };
        auto stage_flush = [&](int col, int row0) {
            fence_proxy_async_smem();
            __syncwarp();
            if (store_leader) {
                tma_store_2d(&p.tm_out, out_stage, col, row0);
                bulk_commit_group();
            }
        };
        uint32_t acc_it = 0;
        for (int w = pair; w < ctx.total_items; w += num_pairs) {
            int tile, part;
            ctx.resolve(w, tile, part);
            const int m_tile = (tile % num_m_pairs) * 2 + (int)rank;
            const int n_tile = tile / num_m_pairs;
            const int acc = acc_it & 1;
            // This warp's columns.  Whole tile: 128-column sub-tile `half`, two 64-column boxes.  Half tile (the
            // accumulator's first 128 columns hold sub-tile `part`): columns [64 half, 64 half + 64) of it, one box.
            const int boxes = part < 0 ? 2 : 1;
            const int w_tcol = part < 0 ? half * 128 : half * 64;      // first tensor-memory column within the accumulator
            const uint32_t aph = (acc_it >> 1) & 1u;
            // The residual does not depend on the accumulator, and a load issued when its value is needed waits
            // behind the operand ring's traffic (about 3000 cycles here), so both 64-column boxes are requested
            // before the wait for the tile's MMAs: the first straight into the staging buffer (idle between tiles;
            // the sum is formed in place there), the second into registers.  A warp reads a box (32 rows x 128
            // bytes) by whole lines, copy j of lane l being chunk l & 7 of row 4 j + (l >> 3), and the chunks reach
            // their row's lane through the staging buffer: with one row per lane every load would touch 32 lines.
            const bool owns_pre = (half == 1 - acc);
            const int first_box_pre = (owns_pre && acc == 0 && part < 0) ? 1 : 0;
            SubTile st_pre = resolve_subtile(p, n_tile, part < 0 ? half : part, 2);
            if (part >= 0) {
                st_pre.col0 += half * 64;
                st_pre.ncols = max(0, min(64, st_pre.ncols - half * 64));
            }
            const bool res_lines = p.epi == EPI_RESIDUAL && p.tma_store && st_pre.ncols >= 64 * boxes && (p.ldo & 7) == 0 &&
                                   (((uintptr_t)p.residual) & 15) == 0;
            uint4 res_c[8];
            if (res_lines) {
                const int r0 = m_tile * 128 + quad * 32 + (lane >> 3);
                const __nv_bfloat16 *src = p.residual + (size_t)min(r0, p.M - 1) * p.ldo + st_pre.col0 + (lane & 7) * 8;
                stage_begin();      // the previous tile's last store has read the buffer
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t rb = (uint32_t)(4 * j) + ((uint32_t)lane >> 3);
                    const bool in = r0 + 4 * j < p.M;
                    cp_async16_zfill(out_stage + rb * 128 + ((((uint32_t)lane & 7u) ^ (rb & 7u)) << 4),
                                     src + first_box_pre * 64 + (in ? (size_t)(4 * j) * p.ldo : 0), in);
                }
                cp_async_commit();
                if (boxes == 2) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        res_c[j] = (r0 + 4 * j < p.M) ? *reinterpret_cast<const uint4 *>(src + (first_box_pre ^ 1) * 64 + (size_t)(4 * j) * p.ldo)
                                                      : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            auto stage_res_lines = [&]() {      // registers -> staging buffer, in the layout stage_packed uses
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t rb = (uint32_t)(4 * j) + ((uint32_t)lane >> 3);
                    sts128(out_stage + rb * 128 + ((((uint32_t)lane & 7u) ^ (rb & 7u)) << 4), res_c[j]);
                }
                __syncwarp();
            };
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
            // the shared physical columns [192, 256) are tile columns [192, 256) of acc0 (second half)
            // and tile columns [0, 64) of acc1 (first half): that half's warps drain them first
            const bool owns_shared = (half == 1 - acc);
            auto release_shared = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tovl0);
            };
            auto release_acc = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(tempty0 + 8u * (uint32_t)acc);
                DBG_ACC(1);
            };

            // The epilogue is written for a small instruction footprint: every warp runs the same
            // loop bodies (one 32-column chunk, or one pair of chunks, per iteration; addresses at run
            // time) instead of separately unrolled code per accumulator, per half and per owner.  With
            // each path unrolled the kernel's code was several times the instruction cache, and
            // fetching it, not the arithmetic, set the time of a tile's epilogue.
            if (p.epi == EPI_SILU_GATE) {
                // gate columns [64*half, +64) pair with up columns [128 + 64*half, +64)
                const SubTile sg = resolve_subtile(p, n_tile, 0, 2);
                const float ag = p.alpha[0], au = p.alpha[1];
                const uint32_t g_col = t_row + half * 64, u_col = t_row + 128 + half * 64;
                const bool box_tma = p.tma_store && p.q_packed == nullptr && (sg.ncols - half * 64) >= 64;
                // The owner's chunks in the shared columns (its up columns in accumulator 0, its gate
                // columns in accumulator 1) are read first, scaled, rounded and kept packed.
                const bool kept_is_gate = acc == 1;
                Packed16 kept[2];
                if (owns_shared) {
                    uint32_t k0[32], k1[32];
                    const uint32_t c = kept_is_gate ? g_col : u_col;
                    tmem_ld_x32(c, k0);
                    tmem_ld_x32(c + 32, k1);
                    tmem_ld_wait();
                    release_shared();
                    const float sk = kept_is_gate ? ag : au;
                    float f[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(k0[i]) * sk;
                    kept[0] = pack_bf16(f);
#pragma unroll
                    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(k1[i]) * sk;
                    kept[1] = pack_bf16(f);
                }
                if (box_tma) stage_begin();
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    float g[32], u[32];
                    if (!owns_shared) {
                        uint32_t a[32], b[32];
                        tmem_ld_x32(g_col + ch * 32, a);
                        tmem_ld_x32(u_col + ch * 32, b);
                        tmem_ld_wait();
                        if (ch == 1) release_acc();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            g[i] = bf16_round(__uint_as_float(a[i]) * ag);
                            u[i] = bf16_round(__uint_as_float(b[i]) * au);
                        }
                    } else {
                        uint32_t a[32];
                        tmem_ld_x32((kept_is_gate ? u_col : g_col) + ch * 32, a);
                        tmem_ld_wait();
                        if (ch == 1) release_acc();
                        Packed16 k;
#pragma unroll
                        for (int i = 0; i < 16; ++i) k.w[i] = ch == 0 ? kept[0].w[i] : kept[1].w[i];
                        float fk[32];
                        unpack_bf16(k, fk);
                        const float sa = kept_is_gate ? au : ag;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float x = bf16_round(__uint_as_float(a[i]) * sa);
                            g[i] = kept_is_gate ? fk[i] : x;
                            u[i] = kept_is_gate ? x : fk[i];
                        }
                    }
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = silu_gate(g[i], u[i]);
                    const int c0 = half * 64 + ch * 32;
                    const int nvalid = sg.ncols - c0;
                    if (p.q_packed != nullptr) {
                        // the next GEMM's operand: quantise the bf16-rounded products in 16-column blocks
                        uint32_t q[4], sf = 0;
#pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            float blk[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) blk[j] = bf16_round(v[16 * b + j]);
                            sf |= quantize_block16(blk, p.q_inv_in, q[2 * b], q[2 * b + 1]) << (8 * b);
                        }
                        if (row_ok && nvalid >= 32) {
                            const int col = sg.col0 + c0;
                            *reinterpret_cast<uint4 *>(p.q_packed + (size_t)row * p.q_ld + (col >> 1)) =
                                make_uint4(q[0], q[1], q[2], q[3]);
                            // tiled scale layout: chunk (row tile, col / 64), byte (row % 32) * 16 + (row / 32 % 4) * 4 + block
                            uint8_t *sfp = p.q_sf + ((size_t)m_tile * p.q_sf_chunks + (col >> 6)) * 512 + lane * 16 +
                                           quad * 4 + ((col >> 4) & 3);
                            *reinterpret_cast<uint16_t *>(sfp) = (uint16_t)sf;
                        }
                        continue;
                    }
                    const Packed16 pk = pack_bf16(v);
                    if (box_tma) stage_packed(pk, ch);
                    else if (row_ok && nvalid > 0 && !GLMASR_EXP(p, 4)) store_packed(out_row + sg.col0 + c0, pk, nvalid);
                }
                if (box_tma && !GLMASR_EXP(p, 4)) stage_flush(sg.col0 + half * 64, m_tile * 128 + quad * 32);
            } else {
                const SubTile st = st_pre;          // this warp's columns (128, or 64 of a half tile)
                const float alpha = p.alpha[st.seg];
                // the owner's shared columns are its chunks 2, 3 (accumulator 0) or 0, 1 (accumulator 1):
                // that 64-column box goes first (a half tile has one box per warp; the owners signal all the same)
                const int first_box = first_box_pre;
#pragma unroll 1
                for (int k = 0; k < boxes; ++k) {
                    const int bx = k ^ first_box;
                    uint32_t r[2][32];
                    tmem_ld_x32(t_row + w_tcol + bx * 64, r[0]);
                    tmem_ld_x32(t_row + w_tcol + bx * 64 + 32, r[1]);
                    tmem_ld_wait();
                    if (k == 0 && owns_shared) release_shared();
                    if (k == boxes - 1) release_acc();
                    const bool box_tma = p.tma_store && (st.ncols - bx * 64) >= 64;
                    if (res_lines && k == 0) {          // the buffer already holds this box's residual
                        cp_async_wait<0>();
                        __syncwarp();
                    } else if (box_tma) {
                        stage_begin();
                        if (res_lines) stage_res_lines();
                    }
#pragma unroll
                    for (int hc = 0; hc < 2; ++hc) {
                        const int c0 = bx * 64 + hc * 32;
                        const int nvalid = st.ncols - c0;
                        const int col = st.col0 + c0;
                        const bool live = row_ok && nvalid > 0;
                        float v[32];
                        const unsigned long long alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(r[hc][2 * i]), __uint_as_float(r[hc][2 * i + 1])), alpha2),
                                         v[2 * i], v[2 * i + 1]);
                        if (p.bias != nullptr && nvalid > 0) {
                            float b[32];
                            unpack_bf16(load_packed(p.bias + col, nvalid), b);
                            // With a residual the reference adds the bias to the linear's bf16 OUTPUT and rounds again
                            // before the residual (residual_add_bias, Infer-engine/cuda/kernels.cu:763-782).  Only the
                            // bf16 instance takes that combination (the host keeps it off the FP4 instance).
                            if (BF16 && p.epi == EPI_RESIDUAL) {
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] = bf16_round(v[i]) + b[i];
                            } else {
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] += b[i];
                            }
                        }
                        if constexpr (BF16) {
                            if (p.epi == EPI_GELU) {
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
                            }
                        }
                        if (p.epi == EPI_RESIDUAL && live) {
                            // bf16(acc) + residual, two values per conversion and per addition
                            Packed16 rs;
                            if (res_lines) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint4 q = lds128(out_stage + (uint32_t)lane * 128 + ((((uint32_t)(hc * 4 + j)) ^ ((uint32_t)lane & 7u)) << 4));
                                    rs.w[4 * j] = q.x, rs.w[4 * j + 1] = q.y, rs.w[4 * j + 2] = q.z, rs.w[4 * j + 3] = q.w;
                                }
                            } else {
                                rs = load_packed(p.residual + (size_t)row * p.ldo + col, nvalid);
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                float x0, x1;
                                round_bf16_x2(v[2 * i], v[2 * i + 1], x0, x1);
                                const uint32_t rw = rs.w[i];
                                unpack_f32x2(add_f32x2(pack_f32x2(x0, x1),
                                                       pack_f32x2(__uint_as_float(rw << 16), __uint_as_float(rw & 0xFFFF0000u))),
                                             v[2 * i], v[2 * i + 1]);
                            }
                        }
                        const Packed16 pk = pack_bf16(v);
                        if (box_tma) stage_packed(pk, hc);
                        else if (live && !GLMASR_EXP(p, 4)) store_packed(out_row + col, pk, nvalid);
                    }
                    if (box_tma && !GLMASR_EXP(p, 4)) stage_flush(st.col0 + bx * 64, m_tile * 128 + quad * 32);
                }
            }
            DBG_ACC(2);
            ++acc_it;
        }
        cp_async_wait<0>();                     // (a copy requested before a wait that gave up)
        if (store_leader) bulk_wait_all();      // this warp's bulk stores are complete before the CTA exits
        __syncwarp();
        if (dbg && warp == 2 && lane == 0 && rank == 0)
            for (int i = 0; i < 3; ++i) p.dbg_cycles[pair * 16 + 8 + i] = dbg_acc[i];
    }

    pair_teardown<C>(p, ctx);
}

cudaError_t umma_gemm_pair_init() {
    const cudaError_t e = cudaFuncSetAttribute(umma_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(umma_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfgBf16::SMEM_BYTES);
}

cudaError_t launch_umma_gemm_pair(const GemmParams &p, int num_pairs, cudaStream_t st) {
    return pair_launch<PairCfg>(umma_gemm_pair_kernel<false>, p, num_pairs, st);
}

cudaError_t launch_umma_gemm_pair_bf16(const GemmParams &p, int num_pairs, cudaStream_t st) {
    return pair_launch<PairCfgBf16>(umma_gemm_pair_kernel<true>, p, num_pairs, st);
}

}  // namespace glmasr
