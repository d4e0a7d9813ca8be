// The pipeline shared by the two CTA-pair W4A4 GEMM kernels (gemm_umma2.cu: eight epilogue warps,
// every epilogue mode; gemm_umma3.cu: sixteen epilogue warps, SiLU-gate epilogues): configuration,
// barrier layout, set-up, the two TMA producer warps, the MMA issuer and the teardown.  A kernel
// supplies only its epilogue.  One copy of the barrier protocol: a fix lands in both kernels.
//
// Two CTAs of a cluster compute one 256 x 256 output tile with M = 256 block-scaled MMAs
// (tcgen05 cta_group::2).  CTA r of the pair holds token rows [128 r, 128 r + 128) of the tile in its
// 128 TMEM lanes and loads only its own operands: its 128 activation rows and HALF of the weight tile
// (128 of the 256 weight rows); the tensor cores of both SMs read the two weight halves from both
// shared memories.  Per 256-k stage a CTA therefore writes 32 KB of operands into shared memory for
// 128 x 256 x 256 multiply-adds instead of 48 KB in the single-CTA kernel.  Scale factors: each CTA
// loads the scales of its own rows and of all 256 weight rows and both copy them to their tensor memory.
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
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

#include "gemm_device.cuh"
#include "gemm_umma.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

// SCALES_ = false: bf16 operands.  A stage then has no scale-factor part (32 KB, six stages) and the two accumulators
// take 256 tensor-memory columns each without sharing any (nothing else needs columns), so a tile's MMAs wait only
// for the epilogue of the tile before the previous one.
template <int EPI_WARPS_, int OUT_STAGE_BYTES_, int BAR_BYTES_, bool SCALES_ = true>
struct PairCfgT {
    static constexpr int BN = 256;
    static constexpr int A_BYTES = 128 * 128;             // this CTA's 128 rows x 256 k of packed e2m1
    static constexpr int B_BYTES = 128 * 128;             // this CTA's half of the weight tile
    static constexpr int SF_CHUNK = 512;
    static constexpr int SF_TILE = 4 * SF_CHUNK;          // 128 rows x 256 k of scales
    static constexpr int SFA_BYTES = SCALES_ ? SF_TILE : 0;
    static constexpr int SFB_BYTES = SCALES_ ? 2 * SF_TILE : 0;         // all 256 weight rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;   // 38912 (32768 without scales)
    static constexpr int STAGES = SCALES_ ? 5 : 6;
    static constexpr int EPI_WARPS = EPI_WARPS_;
    // warp 0: producer of the activation tile and its scales; warp 1: MMA issuer; warps 2 .. 1 + EPI_WARPS:
    // epilogue; the last warp: producer of the weight half-tile and the weight scales.  Two producer warps
    // halve the time between a stage being freed and its last load being issued (each TMA issue costs
    // ~60 cycles).
    static constexpr int PRODUCER_B_WARP = 2 + EPI_WARPS;
    static constexpr int THREADS = (3 + EPI_WARPS) * 32;
    // Two accumulators that share 64 columns: acc0 = columns [0, 256), acc1 = [192, 448).  A tile's
    // MMAs may start as soon as the previous tile's epilogue has drained the 64 shared columns
    // (which it does first), instead of the whole accumulator.
    static constexpr int ACC_STRIDE = SCALES_ ? 192 : 256;
    static constexpr int OVL_LO = 192, OVL_HI = 256;      // shared physical columns
    static constexpr int SFA_COL = 448;
    static constexpr int SFB_COL = SFA_COL + 16;          // 464 .. 495
    static constexpr int TMEM_COLS = 512;
    static constexpr int BAR_BYTES = BAR_BYTES_;          // barriers and flags in the first KB
    static constexpr int OUT_STAGE_BYTES = OUT_STAGE_BYTES_;   // per epilogue warp
    static constexpr int SMEM_BYTES = 1024 + BAR_BYTES + STAGES * STAGE_BYTES + EPI_WARPS * OUT_STAGE_BYTES;
    static constexpr uint32_t TX_BYTES_PAIR = 2 * STAGE_BYTES;
    // a 256 x 128 half tile: 64 weight rows per CTA and one weight-scale tile
    static constexpr uint32_t TX_BYTES_PAIR_HALF = 2 * (STAGE_BYTES - B_BYTES / 2 - SF_TILE);
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// Per-thread view of the CTA's shared-memory layout and of its place in the grid.
template <class C>
struct PairCtx {
    uint32_t bar;                 // shared address of the barrier block
    uint32_t tiles;               // shared address of stage 0
    uint8_t *smem_gen;            // generic pointer to the 1024-aligned base
    volatile int *abort_word;
    uint32_t tmem_base;
    uint32_t rank;                // 0 = leader CTA (issues the MMAs), 1 = peer
    int warp, lane;
    int num_pairs, pair, num_m_pairs, total_tiles, nkb;
    // Work items of the grid, taken round-robin by the pairs: items [0, split_from) are whole tiles; from there on
    // two consecutive items are the column halves of one tile (GemmParams::split_tail).
    int split_from, total_items;
    // item -> tile and part (-1: the whole 256 x 256 tile; 0 / 1: its columns [0, 128) / [128, 256))
    __device__ __forceinline__ void resolve(int w, int &tile, int &part) const {
        if (w < split_from) {
            tile = w;
            part = -1;
        } else {
            const int j = w - split_from;
            tile = split_from + (j >> 1);
            part = j & 1;
        }
    }

    __device__ __forceinline__ uint32_t full_bar(int s) const { return bar + 8u * (uint32_t)s; }
    __device__ __forceinline__ uint32_t empty_bar(int s) const { return bar + 8u * (uint32_t)(C::STAGES + s); }
    // One "accumulator full" barrier per accumulator: with a single shared one, an epilogue warp still
    // storing tile t-1 could miss phase t altogether (tile t+1 needs only the early releases), see the
    // barrier back at its old parity and wait for a tile that cannot start without that warp.
    __device__ __forceinline__ uint32_t tfull_bar(int a) const { return bar + 8u * (uint32_t)(2 * C::STAGES + a); }
    __device__ __forceinline__ uint32_t tempty_bar(int a) const { return bar + 8u * (uint32_t)(2 * C::STAGES + 2 + a); }
    __device__ __forceinline__ uint32_t tovl_bar() const { return bar + 8u * (uint32_t)(2 * C::STAGES + 4); }
    __device__ __forceinline__ uint32_t stage_base(int s) const { return tiles + (uint32_t)s * C::STAGE_BYTES; }
    __device__ __forceinline__ uint32_t out_stage_base() const { return tiles + C::STAGES * C::STAGE_BYTES; }
};

// Barrier initialisation, tensor-memory allocation and descriptor prefetch.  Touches no global memory.
// The caller may do further set-up of its own, then calls pair_setup_finish().
template <class C>
__device__ __forceinline__ PairCtx<C> pair_setup_begin(const GemmParams &p, uint8_t *smem_dyn) {
    PairCtx<C> c;
    const uint32_t smem_raw = smem_u32(smem_dyn);
    const uint32_t smem_base = (smem_raw + 1023u) & ~1023u;
    c.smem_gen = smem_dyn + (smem_base - smem_raw);
    c.bar = smem_base;
    c.tiles = smem_base + C::BAR_BYTES;
    c.abort_word = reinterpret_cast<volatile int *>(c.smem_gen + 520);
    c.warp = threadIdx.x >> 5;
    c.lane = threadIdx.x & 31;
    pdl_launch_dependents();
    c.rank = cluster_ctarank();
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(c.full_bar(s), 1);
            mbar_init(c.empty_bar(s), 1);
        }
        mbar_init(c.tfull_bar(0), 1);
        mbar_init(c.tfull_bar(1), 1);
        mbar_init(c.tempty_bar(0), 2 * C::EPI_WARPS);
        mbar_init(c.tempty_bar(1), 2 * C::EPI_WARPS);
        mbar_init(c.tovl_bar(), C::EPI_WARPS);             // half of each CTA's epilogue warps own the shared columns
        *c.abort_word = 0;
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_a);
        tma_prefetch_desc(&p.tm_sfa);
        for (int s = 0; s < p.num_segs; ++s) {
            if (p.split_tail) tma_prefetch_desc(&p.tm_b_half[s]);
            tma_prefetch_desc(&p.tm_b[s]);
            tma_prefetch_desc(&p.tm_sfb[s]);
        }
    }
    if (c.warp == 1) {
        tmem_alloc_pair(smem_u32((const void *)(c.smem_gen + 512)), C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    return c;
}

template <class C>
__device__ __forceinline__ void pair_setup_finish(const GemmParams &p, PairCtx<C> &c) {
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                // both CTAs' barriers exist before any remote signal
    tc_fence_after();
    c.tmem_base = *reinterpret_cast<volatile uint32_t *>(c.smem_gen + 512);
    pdl_wait();                 // set-up touched no global memory; everything after this may
    c.num_pairs = gridDim.x >> 1;
    c.pair = blockIdx.x >> 1;
    c.num_m_pairs = (p.num_m_tiles + 1) >> 1;
    c.total_tiles = c.num_m_pairs * p.num_n_tiles;
    c.nkb = p.num_k_blocks;
    const int last_round = c.total_tiles % c.num_pairs;
    const bool split = p.split_tail != 0 && last_round > 0 && 2 * last_round <= c.num_pairs;
    c.split_from = split ? c.total_tiles - last_round : c.total_tiles;
    c.total_items = split ? c.total_tiles + last_round : c.total_tiles;
}

// Warps 0 and C::PRODUCER_B_WARP of both CTAs.  BF16: the operands are bf16 (64 elements per 128-byte row, kind::f16
// MMAs) and there are no scale factors; a stage keeps its layout and leaves the scale-factor part unused.
template <class C, bool BF16 = false>
__device__ __forceinline__ void pair_producer(const GemmParams &p, const PairCtx<C> &c) {
    const bool dbg = GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr;
    unsigned long long dbg_acc[4] = {0, 0, 0, 0};
    (void)dbg_acc;
    // experiment 256: warp 0 issues everything and the second producer idles
    const bool solo = GLMASR_EXP(p, 256);
    const bool do_a = c.warp == 0, do_b = solo ? c.warp == 0 : c.warp == C::PRODUCER_B_WARP;
    const bool leader_lane = elect_one();
    constexpr int KX = BF16 ? 64 : 128;                        // elements of the operand maps per 128-byte row (bf16 / packed e2m1 bytes)
    const uint32_t full0 = mapa_shared(c.full_bar(0), 0);      // CTA 0's full[0]; full[s] = full0 + 8 s
    const int rank = (int)c.rank;
    uint32_t it = 0;
    bool ok = !(solo && c.warp == C::PRODUCER_B_WARP);
    for (int w = c.pair; ok && w < c.total_items; w += c.num_pairs) {
        int tile, part;
        c.resolve(w, tile, part);
        const int m_tile = (tile % c.num_m_pairs) * 2 + rank;     // this CTA's 128-row tile
        const int n_tile = tile / c.num_m_pairs;
        // whole tile: this CTA loads weight sub-tile `rank`; half tile: rows [64 rank, 64 rank + 64) of sub-tile
        // `part`, through the 64-row view of the weights
        const SubTile mine = resolve_subtile(p, n_tile, part < 0 ? rank : part, 2);
        const int b_row = part < 0 ? mine.row0 : mine.row0 + 64 * rank;
        const SubTile st0 = part < 0 ? resolve_subtile(p, n_tile, 0, 2) : mine;
        const SubTile st1 = resolve_subtile(p, n_tile, 1, 2);
        const int sfa_row = m_tile * p.sf_k_chunks;
        const int sfb_row0 = (st0.row0 >> 7) * p.sf_k_chunks;
        const int sfb_row1 = (st1.row0 >> 7) * p.sf_k_chunks;
        for (int kb = 0; kb < c.nkb; ++kb) {
            const int s = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1u;
            DBG_T0();
            if (!mbar_wait_warp(c.empty_bar(s), ph ^ 1u, c.abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
            DBG_ACC(0);
            const uint32_t sb = c.stage_base(s);
            const uint32_t fb = full0 + 8u * (uint32_t)s;
            const uint32_t sf = sb + C::A_BYTES + C::B_BYTES;
            const bool no_sf = BF16 || GLMASR_EXP(p, 2);      // (experiment 2: no scale-factor traffic, wrong results)
            if (GLMASR_EXP(p, 8) && it >= (uint32_t)C::STAGES) {
                // experiment: operands stay resident in shared memory after the first round of the ring
                if (leader_lane && do_a && rank == 0) mbar_arrive(c.full_bar(s));
                ++it;
                continue;
            }
            if (leader_lane) {
                if (do_a) {
                    if (rank == 0)
                        mbar_expect_tx(c.full_bar(s), no_sf ? 2u * (C::A_BYTES + (part < 0 ? C::B_BYTES : C::B_BYTES / 2))
                                                            : (part < 0 ? C::TX_BYTES_PAIR : C::TX_BYTES_PAIR_HALF));
                    tma_load_2d_pair(sb, &p.tm_a, fb, kb * KX, m_tile * 128);
                    if (!no_sf) tma_load_2d_pair(sf, &p.tm_sfa, fb, 0, sfa_row + kb * 4);
                }
                if (do_b) {
                    tma_load_2d_pair(sb + C::A_BYTES, part < 0 ? &p.tm_b[mine.seg] : &p.tm_b_half[mine.seg], fb, kb * KX, b_row);
                    if (!no_sf) {
                        tma_load_2d_pair(sf + C::SF_TILE, &p.tm_sfb[st0.seg], fb, 0, sfb_row0 + kb * 4);
                        if (part < 0) tma_load_2d_pair(sf + 2 * C::SF_TILE, &p.tm_sfb[st1.seg], fb, 0, sfb_row1 + kb * 4);
                    }
                }
            }
            ++it;
            DBG_ACC(1);
        }
    }
    if (dbg && leader_lane && rank == 0 && c.warp == 0) {
        p.dbg_cycles[c.pair * 16 + 0] = dbg_acc[0];
        p.dbg_cycles[c.pair * 16 + 1] = dbg_acc[1];
    }
}

// Warp 1.  Only the leader CTA issues; the peer's warp 1 falls through to the teardown.
template <class C, bool BF16 = false>
__device__ __forceinline__ void pair_mma_issuer(const GemmParams &p, const PairCtx<C> &c) {
    if (c.rank != 0) return;
    const bool dbg = GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr;
    unsigned long long dbg_acc[4] = {0, 0, 0, 0};
    (void)dbg_acc;
    const bool leader_lane = elect_one();
    constexpr uint32_t idesc_whole = BF16 ? idesc_bf16(256, C::BN) : idesc_nvfp4(256, C::BN);
    constexpr uint32_t idesc_half = BF16 ? idesc_bf16(256, C::BN / 2) : idesc_nvfp4(256, C::BN / 2);
    const uint32_t empty0_peer = mapa_shared(c.empty_bar(0), 1);
    const uint32_t tfull0_peer = mapa_shared(c.tfull_bar(0), 1);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    for (int w = c.pair; ok && w < c.total_items; w += c.num_pairs) {
        int tile, part;
        c.resolve(w, tile, part);
        const uint32_t idesc = part < 0 ? idesc_whole : idesc_half;   // a half tile fills the first 128 columns of its accumulator
        const int acc = acc_it & 1;
        const uint32_t aph = (acc_it >> 1) & 1u;
        DBG_T0();
        // this accumulator's previous tile (two tiles ago) fully drained ...
        if (!mbar_wait_warp(c.tempty_bar(acc), aph ^ 1u, c.abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
        // ... and the shared columns drained by the previous tile's epilogue
        if (C::ACC_STRIDE < C::BN && acc_it > 0 &&
            !mbar_wait_warp(c.tovl_bar(), (acc_it - 1) & 1u, c.abort_word, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
        }
        DBG_ACC(0);
        tc_fence_after();
        const uint32_t d_tmem = c.tmem_base + (uint32_t)(acc * C::ACC_STRIDE);
        for (int kb = 0; kb < c.nkb; ++kb) {
            const int s = it % C::STAGES;
            const uint32_t ph = (it / C::STAGES) & 1u;
            if (!mbar_wait_warp(c.full_bar(s), ph, c.abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
            DBG_ACC(1);
            tc_fence_after();
            const uint32_t a_addr = c.stage_base(s);
            const uint32_t b_addr = a_addr + C::A_BYTES;
            const uint32_t sfa_t = c.tmem_base + C::SFA_COL;
            const uint32_t sfb_t = c.tmem_base + C::SFB_COL;
            const uint64_t adesc0 = smem_desc_sw128(a_addr);
            const uint64_t bdesc0 = smem_desc_sw128(b_addr);
            if (leader_lane) {
                const uint64_t sfdesc0 = smem_desc_sf_chunk(a_addr + C::A_BYTES + C::B_BYTES);
                if (!BF16 && !(GLMASR_EXP(p, 32) && it > 0)) {        // (experiment 32: scale factors copied once, wrong results)
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch)
                        tmem_cp_32x128b_warpx4_pair(sfa_t + 4 * ch, sfdesc0 + (uint64_t)((ch * C::SF_CHUNK) >> 4));
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        if (h == 0 || part < 0) {
#pragma unroll
                            for (int ch = 0; ch < 4; ++ch)
                                tmem_cp_32x128b_warpx4_pair(sfb_t + ch * 8 + 4 * h,
                                                            sfdesc0 + (uint64_t)(((1 + h) * C::SF_TILE + ch * C::SF_CHUNK) >> 4));
                        }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                    if constexpr (BF16)
                        umma_bf16_pair(d_tmem, adesc0 + (uint64_t)((k * 32) >> 4), bdesc0 + (uint64_t)((k * 32) >> 4), idesc, accumulate);
                    else
                        umma_nvfp4_pair(d_tmem, adesc0 + (uint64_t)((k * 32) >> 4), bdesc0 + (uint64_t)((k * 32) >> 4), idesc,
                                        accumulate, sfa_t + 4 * k, sfb_t + 8 * k);
                }
                umma_commit_pair(c.empty_bar(s));                       // frees the stage in this CTA ...
                umma_commit_pair(empty0_peer + 8u * (uint32_t)s);       // ... and in the peer
            }
            ++it;
            DBG_ACC(2);
        }
        if (!ok) break;
        if (leader_lane) {
            umma_commit_pair(c.tfull_bar(acc));
            umma_commit_pair(tfull0_peer + 8u * (uint32_t)acc);
        }
        ++acc_it;
    }
    if (dbg && leader_lane)
        for (int i = 0; i < 3; ++i) p.dbg_cycles[c.pair * 16 + 4 + i] = dbg_acc[i];
}

template <class C>
__device__ __forceinline__ void pair_teardown(const GemmParams &p, const PairCtx<C> &c) {
    tc_fence_before();
    __syncthreads();
    if (*c.abort_word != 0) {
        // give copies that may still be in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, *c.abort_word);
    }
    cluster_sync_all();        // neither CTA frees shared / tensor memory while the other may still use it
    if (c.warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(c.tmem_base, C::TMEM_COLS);
    }
}

// Clusters of two CTAs, chained to the preceding kernel by programmatic dependent launch.
template <class C, class Kernel>
inline cudaError_t pair_launch(Kernel kernel, const GemmParams &p, int num_pairs, cudaStream_t st) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * num_pairs, 1, 1);
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
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
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace glmasr
