// W4A4 GEMM on CTA pairs, SiLU-gate epilogues only, with SIXTEEN epilogue warps per CTA.
// Same pipeline as gemm_umma2.cu (two producer warps, one MMA warp, cta_group::2 MMAs on 256 x 256
// tiles, two accumulators overlapping in 64 tensor-memory columns); what differs is the epilogue.
// With the activation quantiser folded in, the SiLU-gate epilogue of eight warps (two per
// sub-partition, ~0.25 instructions per clock each) takes longer than a tile's MMAs and the
// kernel runs at the epilogue's pace.  Here every warp owns 32 rows x 32 outputs, works on 16
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
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

struct Pair16Cfg {
    static constexpr int BN = 256;
    static constexpr int A_BYTES = 128 * 128;             // this CTA's 128 rows x 256 k of packed e2m1
    static constexpr int B_BYTES = 128 * 128;             // this CTA's half of the weight tile
    static constexpr int SF_CHUNK = 512;
    static constexpr int SF_TILE = 4 * SF_CHUNK;          // 128 rows x 256 k of scales
    static constexpr int SFA_BYTES = SF_TILE;
    static constexpr int SFB_BYTES = 2 * SF_TILE;         // all 256 weight rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;   // 38912
    static constexpr int STAGES = 5;
    static constexpr int EPI_WARPS = 16;
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
    static constexpr int BAR_BYTES = 2048;                // barriers and flags (first KB), quantiser look-up table (second KB)
    static constexpr int OUT_STAGE_BYTES = 32 * 64;       // per epilogue warp: 32 rows x 32 bf16, 64B-swizzled
    static constexpr int SMEM_BYTES = 1024 + BAR_BYTES + STAGES * STAGE_BYTES + EPI_WARPS * OUT_STAGE_BYTES;
    static constexpr uint32_t TX_BYTES_PAIR = 2 * STAGE_BYTES;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

__global__ void __launch_bounds__(640, 1) umma_gemm_pair16_kernel(const __grid_constant__ GemmParams p) {
    using C = Pair16Cfg;
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
    float *os_table = reinterpret_cast<float *>(smem_gen + 1024);
    if (p.q_packed != nullptr) fill_os_table(os_table, p.q_inv_in, (int)threadIdx.x, (int)blockDim.x);
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
                float g[16], u[16];
                if (!owns_shared) {
                    uint32_t a[16], b[16];
                    tmem_ld_x16(g_col + it * 16, a);
                    tmem_ld_x16(u_col + it * 16, b);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        g[i] = bf16_round(__uint_as_float(a[i]) * ag);
                        u[i] = bf16_round(__uint_as_float(b[i]) * au);
                    }
                } else {
                    uint32_t a[16];
                    tmem_ld_x16((kept_is_gate ? u_col : g_col) + it * 16, a);
                    tmem_ld_wait();
                    const float sa = kept_is_gate ? au : ag;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t kw = it == 0 ? kept[i] : kept[8 + i];
                        const float k_lo = __uint_as_float(kw << 16), k_hi = __uint_as_float(kw & 0xFFFF0000u);
                        const float x_lo = bf16_round(__uint_as_float(a[2 * i]) * sa);
                        const float x_hi = bf16_round(__uint_as_float(a[2 * i + 1]) * sa);
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
                for (int i = 0; i < 16; ++i) v[i] = silu_gate(g[i], u[i]);
                const int c0 = slice * 32 + it * 16;
                const int col = sg.col0 + c0;
                const int nvalid = sg.ncols - c0;
                if (p.q_packed != nullptr) {
                    // the next GEMM's operand: quantise the bf16-rounded products of this 16-column block
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = bf16_round(v[i]);
                    uint32_t qlo, qhi, sf;
                    if (p.debug & 8) {           // timing experiment: no quantiser arithmetic (wrong results)
                        qlo = __float_as_uint(v[0]), qhi = __float_as_uint(v[9]), sf = __float_as_uint(v[3]) & 0x7Fu;
                    } else {
                        sf = quantize_block16_lut(v, p.q_inv_in, os_table, qlo, qhi);
                    }
                    if (it == 0) {
                        q_first_lo = qlo, q_first_hi = qhi, sf_first = sf;
                    } else if (q_tma) {
                        sts128(out_stage + (uint32_t)lane * 16, make_uint4(q_first_lo, q_first_hi, qlo, qhi));
                        if (row_ok && !(p.debug & (4 | 16))) {
                            const int col0 = col - 16;
                            uint8_t *sfp = p.q_sf + ((size_t)m_tile * p.q_sf_chunks + (col0 >> 6)) * 512 + lane * 16 + quad * 4 +
                                           ((col0 >> 4) & 3);
                            *reinterpret_cast<uint16_t *>(sfp) = (uint16_t)(sf_first | (sf << 8));
                        }
                    } else if (row_ok && nvalid >= 16 && !(p.debug & 4)) {
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
                } else if (row_ok && nvalid > 0 && !(p.debug & 4)) {
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
            if ((box_tma || q_tma) && !(p.debug & 4)) {
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

cudaError_t umma_gemm_pair16_init() {
    return cudaFuncSetAttribute(umma_gemm_pair16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Pair16Cfg::SMEM_BYTES);
}

cudaError_t launch_umma_gemm_pair16(const GemmParams &p, int num_pairs, cudaStream_t st) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * num_pairs, 1, 1);
    cfg.blockDim = dim3(Pair16Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Pair16Cfg::SMEM_BYTES;
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
    return cudaLaunchKernelEx(&cfg, umma_gemm_pair16_kernel, p);
}

}  // namespace glmasr
