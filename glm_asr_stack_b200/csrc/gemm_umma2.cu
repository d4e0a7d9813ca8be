// W4A4 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// Two CTAs of a cluster compute one 256 x 256 output tile with M = 256 block-scaled MMAs.
// CTA r of the pair holds token rows [128 r, 128 r + 128) of the tile in its 128 TMEM lanes and
// loads only its own operands: its 128 activation rows and HALF of the weight tile (128 of the 256
// weight rows); the tensor cores of both SMs read the two weight halves from both shared
// memories.  Per 256-k stage a CTA therefore writes 32 KB of operands into shared memory for
// 128 x 256 x 256 multiply-adds instead of 48 KB in the single-CTA kernel, which is what that
// kernel is limited by.  Scale factors: each CTA loads the scales of its own rows and of all 256
// weight rows (each CTA needs every column's scales) and both copy them to their tensor memory.
//
// Synchronisation (all waits bounded):
//   full[s]    in CTA 0 only; CTA 0's producer announces the bytes of both CTAs, every load of
//              either CTA credits that barrier
//   empty[s]   in each CTA; the MMA thread (CTA 0) commits to both after the stage's MMAs
//   tfull[a]   in each CTA, one per accumulator; committed to both when a tile's last MMA is issued
//   tempty[a]  in CTA 0; the epilogue warps of both CTAs arrive on it once accumulator a has
//              been drained into registers
//   tovl       in CTA 0; the epilogue warps that own the 64 tensor-memory columns shared by the two
//              accumulators arrive on it as soon as those columns are drained
// No cluster-wide broadcast load is used: every TMA load has exactly one destination CTA.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include "fp4_format.cuh"
#include "gemm_device.cuh"
#include "gemm_umma.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

struct PairCfg {
    static constexpr int BN = 256;
    static constexpr int A_BYTES = 128 * 128;             // this CTA's 128 rows x 256 k of packed e2m1
    static constexpr int B_BYTES = 128 * 128;             // this CTA's half of the weight tile
    static constexpr int SF_CHUNK = 512;
    static constexpr int SF_TILE = 4 * SF_CHUNK;          // 128 rows x 256 k of scales
    static constexpr int SFA_BYTES = SF_TILE;
    static constexpr int SFB_BYTES = 2 * SF_TILE;         // all 256 weight rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;   // 38912
    static constexpr int STAGES = 5;
    static constexpr int EPI_WARPS = 8;
    // warp 0: producer of the activation tile and its scales; warp 1: MMA issuer; warps 2..9: epilogue;
    // warp 10: producer of the weight half-tile and the weight scales.  Two producer warps halve the
    // time between a stage being freed and its last load being issued (each TMA issue costs ~60 cycles).
    static constexpr int PRODUCER_B_WARP = 2 + EPI_WARPS;
    static constexpr int THREADS = (3 + EPI_WARPS) * 32;
    // Two accumulators that share 64 columns: acc0 = columns [0, 256), acc1 = [192, 448).  A tile's
    // MMAs may start as soon as the previous tile's epilogue has drained the 64 shared columns
    // (which it does first), instead of the whole accumulator.
    static constexpr int ACC_STRIDE = 192;
    static constexpr int OVL_LO = 192, OVL_HI = 256;      // shared physical columns
    static constexpr int SFA_COL = 448;
    static constexpr int SFB_COL = SFA_COL + 16;          // 464 .. 495
    static constexpr int TMEM_COLS = 512;
    static constexpr int BAR_BYTES = 1024;
    static constexpr int OUT_STAGE_BYTES = 32 * 128;      // per epilogue warp: 32 rows x 64 bf16, 128B-swizzled
    static constexpr int SMEM_BYTES = 1024 + BAR_BYTES + STAGES * STAGE_BYTES + EPI_WARPS * OUT_STAGE_BYTES;
    static constexpr uint32_t TX_BYTES_PAIR = 2 * STAGE_BYTES;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

__global__ void __launch_bounds__(PairCfg::THREADS, 1) umma_gemm_pair_kernel(const __grid_constant__ GemmParams p) {
    using C = PairCfg;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_raw = smem_u32(smem_dyn);
    const uint32_t smem_base = (smem_raw + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_dyn + (smem_base - smem_raw);

    const uint32_t bar = smem_base;
    auto full_bar = [&](int s) { return bar + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar + 8u * (uint32_t)(C::STAGES + s); };
    // One "accumulator full" barrier per accumulator: with a single shared one, an epilogue warp still
    // storing tile t-1 could miss phase t altogether (tile t+1 needs only the early releases), see the
    // barrier back at its old parity and wait for a tile that cannot start without that warp.
    auto tfull_bar = [&](int a) { return bar + 8u * (uint32_t)(2 * C::STAGES + a); };
    auto tempty_bar = [&](int a) { return bar + 8u * (uint32_t)(2 * C::STAGES + 2 + a); };
    const uint32_t tovl_bar = bar + 8u * (uint32_t)(2 * C::STAGES + 4);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + 512);
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem_gen + 520);
    const uint32_t tiles = smem_base + C::BAR_BYTES;
    auto stage_base = [&](int s) { return tiles + (uint32_t)s * C::STAGE_BYTES; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = peer
    const uint32_t peer = rank ^ 1u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar(0), 1);
        mbar_init(tfull_bar(1), 1);
        mbar_init(tempty_bar(0), 2 * C::EPI_WARPS);
        mbar_init(tempty_bar(1), 2 * C::EPI_WARPS);
        mbar_init(tovl_bar, C::EPI_WARPS);                 // 4 warps of each CTA own the shared columns
        *abort_word = 0;
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_a);
        tma_prefetch_desc(&p.tm_sfa);
        for (int s = 0; s < p.num_segs; ++s) {
            tma_prefetch_desc(&p.tm_b[s]);
            tma_prefetch_desc(&p.tm_sfb[s]);
        }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32((const void *)tmem_slot), C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                // both CTAs' barriers exist before any remote signal
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                 // set-up above touched no global memory; everything below may

    const int num_pairs = gridDim.x >> 1;
    const int pair = blockIdx.x >> 1;
    const int num_m_pairs = (p.num_m_tiles + 1) >> 1;
    const int total_tiles = num_m_pairs * p.num_n_tiles;
    const int nkb = p.num_k_blocks;
    const bool dbg = (p.debug & 64) != 0 && p.dbg_cycles != nullptr;
    unsigned long long dbg_acc[4] = {0, 0, 0, 0};

    if (warp == 0 || warp == C::PRODUCER_B_WARP) {
        // ================================ TMA producers (both CTAs) ======================
        // debug & 256 (timing experiments): warp 0 issues everything and the second producer idles
        const bool solo = (p.debug & 256) != 0;
        const bool do_a = warp == 0, do_b = solo ? warp == 0 : warp == C::PRODUCER_B_WARP;
        const bool leader_lane = elect_one();
        const uint32_t full0 = mapa_shared(full_bar(0), 0);      // CTA 0's full[0]; full[s] = full0 + 8 s
        uint32_t it = 0;
        bool ok = !(solo && warp == C::PRODUCER_B_WARP);
        for (int tile = pair; ok && tile < total_tiles; tile += num_pairs) {
            const int m_tile = (tile % num_m_pairs) * 2 + (int)rank;     // this CTA's 128-row tile
            const int n_tile = tile / num_m_pairs;
            const SubTile mine = resolve_subtile(p, n_tile, (int)rank, 2);      // the weight half this CTA loads
            const SubTile st0 = resolve_subtile(p, n_tile, 0, 2);
            const SubTile st1 = resolve_subtile(p, n_tile, 1, 2);
            const int sfa_row = m_tile * p.sf_k_chunks;
            const int sfb_row0 = (st0.row0 >> 7) * p.sf_k_chunks;
            const int sfb_row1 = (st1.row0 >> 7) * p.sf_k_chunks;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1u;
                DBG_T0();
                if (!mbar_wait_warp(empty_bar(s), ph ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                DBG_ACC(0);
                const uint32_t sb = stage_base(s);
                const uint32_t fb = full0 + 8u * (uint32_t)s;
                const uint32_t sf = sb + C::A_BYTES + C::B_BYTES;
                const bool no_sf = (p.debug & 2) != 0;      // timing experiment: no scale-factor traffic (wrong results)
                if ((p.debug & 8) && it >= (uint32_t)C::STAGES) {
                    // timing experiment: operands stay resident in shared memory after the first round of the
                    // ring, so the k-loop runs at the rate the tensor pipe (and the MMA issue) allows
                    if (leader_lane && do_a && rank == 0) mbar_arrive(full_bar(s));
                    ++it;
                    continue;
                }
                if (leader_lane) {
                    if (do_a) {
                        if (rank == 0) mbar_expect_tx(full_bar(s), no_sf ? 2u * (C::A_BYTES + C::B_BYTES) : C::TX_BYTES_PAIR);
                        tma_load_2d_pair(sb, &p.tm_a, fb, kb * 128, m_tile * 128);
                        if (!no_sf) tma_load_2d_pair(sf, &p.tm_sfa, fb, 0, sfa_row + kb * 4);
                    }
                    if (do_b) {
                        tma_load_2d_pair(sb + C::A_BYTES, &p.tm_b[mine.seg], fb, kb * 128, mine.row0);
                        if (!no_sf) {
                            tma_load_2d_pair(sf + C::SF_TILE, &p.tm_sfb[st0.seg], fb, 0, sfb_row0 + kb * 4);
                            tma_load_2d_pair(sf + 2 * C::SF_TILE, &p.tm_sfb[st1.seg], fb, 0, sfb_row1 + kb * 4);
                        }
                    }
                }
                ++it;
                DBG_ACC(1);
            }
        }
        if (dbg && leader_lane && rank == 0 && warp == 0) { p.dbg_cycles[pair * 16 + 0] = dbg_acc[0]; p.dbg_cycles[pair * 16 + 1] = dbg_acc[1]; }
    } else if (warp == 1) {
        // ================================ MMA issuer (CTA 0 only) ========================
        if (rank == 0) {
            const bool leader_lane = elect_one();
            constexpr uint32_t idesc = idesc_nvfp4(256, C::BN);
            const uint32_t empty0_peer = mapa_shared(empty_bar(0), 1);
            const uint32_t tfull0_peer = mapa_shared(tfull_bar(0), 1);
            uint32_t it = 0, acc_it = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < total_tiles; tile += num_pairs) {
                const int acc = acc_it & 1;
                const uint32_t aph = (acc_it >> 1) & 1u;
                DBG_T0();
                // this accumulator's previous tile (two tiles ago) fully drained ...
                if (!mbar_wait_warp(tempty_bar(acc), aph ^ 1u, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                // ... and the shared columns drained by the previous tile's epilogue
                if (acc_it > 0 && !mbar_wait_warp(tovl_bar, (acc_it - 1) & 1u, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                DBG_ACC(0);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * C::ACC_STRIDE);
                for (int kb = 0; kb < nkb; ++kb) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1u;
                    if (!mbar_wait_warp(full_bar(s), ph, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                    DBG_ACC(1);
                    tc_fence_after();
                    const uint32_t a_addr = stage_base(s);
                    const uint32_t b_addr = a_addr + C::A_BYTES;
                    const uint32_t sfa_t = tmem_base + C::SFA_COL;
                    const uint32_t sfb_t = tmem_base + C::SFB_COL;
                    const uint64_t adesc0 = smem_desc_sw128(a_addr);
                    const uint64_t bdesc0 = smem_desc_sw128(b_addr);
                    if (leader_lane) {
                        const uint64_t sfdesc0 = smem_desc_sf_chunk(a_addr + C::A_BYTES + C::B_BYTES);
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            tmem_cp_32x128b_warpx4_pair(sfa_t + 4 * c, sfdesc0 + (uint64_t)((c * C::SF_CHUNK) >> 4));
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                tmem_cp_32x128b_warpx4_pair(sfb_t + c * 8 + 4 * h,
                                                            sfdesc0 + (uint64_t)(((1 + h) * C::SF_TILE + c * C::SF_CHUNK) >> 4));
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                            umma_nvfp4_pair(d_tmem, adesc0 + (uint64_t)((k * 32) >> 4), bdesc0 + (uint64_t)((k * 32) >> 4),
                                            idesc, accumulate, sfa_t + 4 * k, sfb_t + 8 * k);
                        }
                        umma_commit_pair(empty_bar(s));                       // frees the stage in this CTA ...
                        umma_commit_pair(empty0_peer + 8u * (uint32_t)s);     // ... and in the peer
                    }
                    ++it;
                    DBG_ACC(2);
                }
                if (!ok) break;
                if (leader_lane) {
                    umma_commit_pair(tfull_bar(acc));
                    umma_commit_pair(tfull0_peer + 8u * (uint32_t)acc);
                }
                ++acc_it;
            }
            if (dbg && leader_lane) for (int i = 0; i < 3; ++i) p.dbg_cycles[pair * 16 + 4 + i] = dbg_acc[i];
        }
    } else {
        // ================================ epilogue (both CTAs) ==========================
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
                    else if (row_ok && nvalid > 0 && !(p.debug & 4)) store_packed(out_row + sg.col0 + c0, pk, nvalid);
                }
                if (box_tma && !(p.debug & 4)) stage_flush(sg.col0 + half * 64, m_tile * 128 + quad * 32);
            } else {
                const SubTile st = resolve_subtile(p, n_tile, half, 2);
                const float alpha = p.alpha[st.seg];
                // the owner's shared columns are its chunks 2, 3 (accumulator 0) or 0, 1 (accumulator 1):
                // that 64-column box goes first
                const int first_box = (owns_shared && acc == 0) ? 1 : 0;
#pragma unroll 1
                for (int k = 0; k < 2; ++k) {
                    const int bx = k ^ first_box;
                    uint32_t r[2][32];
                    tmem_ld_x32(t_row + half * 128 + bx * 64, r[0]);
                    tmem_ld_x32(t_row + half * 128 + bx * 64 + 32, r[1]);
                    tmem_ld_wait();
                    if (k == 1) release_acc();
                    else if (owns_shared) release_shared();
                    const bool box_tma = p.tma_store && (st.ncols - bx * 64) >= 64;
                    if (box_tma) stage_begin();
#pragma unroll
                    for (int hc = 0; hc < 2; ++hc) {
                        const int c0 = bx * 64 + hc * 32;
                        const int nvalid = st.ncols - c0;
                        const int col = st.col0 + c0;
                        const bool live = row_ok && nvalid > 0;
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[hc][i]) * alpha;
                        if (p.bias != nullptr && nvalid > 0) {
                            float b[32];
                            unpack_bf16(load_packed(p.bias + col, nvalid), b);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += b[i];
                        }
                        if (p.epi == EPI_RESIDUAL && live) {
                            float res[32];
                            unpack_bf16(load_packed(p.residual + (size_t)row * p.ldo + col, nvalid), res);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = bf16_round(v[i]) + res[i];
                        }
                        const Packed16 pk = pack_bf16(v);
                        if (box_tma) stage_packed(pk, hc);
                        else if (live && !(p.debug & 4)) store_packed(out_row + col, pk, nvalid);
                    }
                    if (box_tma && !(p.debug & 4)) stage_flush(st.col0 + bx * 64, m_tile * 128 + quad * 32);
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

    // ================================ teardown ==========================================
    tc_fence_before();
    __syncthreads();
    if (*abort_word != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
    }
    cluster_sync_all();        // neither CTA frees shared / tensor memory while the other may still use it
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

cudaError_t umma_gemm_pair_init() {
    return cudaFuncSetAttribute(umma_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM_BYTES);
}

cudaError_t launch_umma_gemm_pair(const GemmParams &p, int num_pairs, cudaStream_t st) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * num_pairs, 1, 1);
    cfg.blockDim = dim3(PairCfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = PairCfg::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, umma_gemm_pair_kernel, p);
}

}  // namespace glmasr
