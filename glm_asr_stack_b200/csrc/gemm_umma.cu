// tcgen05 GEMM for the FP4 linear path on sm_100a.
//
//   out[M, N] = epilogue( x[M, K] * W[N, K]^T )
//
// One persistent CTA per SM walks 128 x (128*NB) output tiles.  Warp roles:
//   warp 0      TMA producer: activation tile, weight tile(s), and (W4A4) the 128x4-tiled scale
//               chunks, into a ring of shared-memory stages guarded by full/empty mbarriers
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits stages
//   warps 2-9   epilogue: tcgen05.ld the fp32 accumulator (two warps per TMEM lane quadrant, half
//               the columns each), apply the per-tensor scale and the fused SiLU-gate / residual,
//               16-byte bf16 stores
//   warps 10+   (W4A16 only) dequantise packed e2m1 weights + e4m3 scales from a raw ring into
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
#include "gemm_device.cuh"
#include "gemm_umma.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

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
    // epilogue warps: one or two per TMEM lane quadrant (each then takes half the columns); the
    // W4A16 variant keeps four because its dequant warps need the register budget
    static constexpr int EPI_WARPS = MODE == GEMM_W4A16 ? 4 : 8;
    static constexpr int FIRST_DQ_WARP = 2 + EPI_WARPS;
    static constexpr int DQ_WARPS = MODE == GEMM_W4A16 ? 4 * NB : 0;
    static constexpr int THREADS = (2 + EPI_WARPS + DQ_WARPS) * 32;
    // With a single accumulator the epilogue first drains its columns into registers and hands the
    // accumulator back to the MMA warp, then converts and stores while the next tile is computed.
    static constexpr bool EARLY_RELEASE = NUM_ACC == 1;
    // scale factors of one stage: 16 columns for A, 16 per weight sub-tile for B; two such sets are
    // alternated stage by stage so that the copy for the next stage does not wait for the MMAs
    // still reading the current one
    static constexpr int SF_SET_COLS = 16 + 16 * NB;
    static constexpr int SF_SETS = 2;
    static constexpr int SFA_COL = NUM_ACC * BN;          // tensor-memory column of the A scales (set 0)
    static constexpr int SFB_COL = SFA_COL + 16;
    static constexpr int TMEM_NEEDED = NUM_ACC * BN + (MODE == GEMM_W4A4 ? SF_SETS * SF_SET_COLS : 0);
    static constexpr int TMEM_COLS = next_pow2_cols(TMEM_NEEDED);
    static constexpr int BAR_BYTES = 1024;
    static constexpr int SMEM_BYTES = 1024 + BAR_BYTES + STAGES * STAGE_BYTES + RAW_STAGES * RAW_STAGE_BYTES;
    // bytes the producer announces per stage
    static constexpr int TX_BYTES = MODE == GEMM_W4A16 ? A_BYTES : STAGE_BYTES;
    static_assert(TMEM_NEEDED <= 512, "tensor memory budget");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

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
    const long long t_start = (GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr) ? clock64() : 0;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_bar(s), 1 + C::DQ_WARPS);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < C::NUM_ACC; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), C::EPI_WARPS);
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
    // Set-up above touched no global memory.  Everything below may, so every warp waits for the preceding
    // kernels here -- except the producer, which first starts the WEIGHT loads of its first stages (weights
    // and their re-tiled scales are written by no kernel of a chain; p.early_weights is cleared by the host
    // when that is not true) and waits before its first activation load.
    const bool early_b = MODE != GEMM_W4A16 && p.early_weights != 0;
    if (warp != 0 || !early_b) pdl_wait();
    const long long t_setup = (GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr) ? clock64() : 0;

    const int total_tiles = p.num_m_tiles * p.num_n_tiles;
    const int nkb = p.num_k_blocks;
    // split-K: work item w = tile * S + split covers K blocks [split * nkb / S, (split + 1) * nkb / S)
    const int S = (MODE == GEMM_W4A4 && p.split_k > 1) ? p.split_k : 1;
    const int total_work = total_tiles * S;
    const bool dbg = GLMASR_EXP(p, 64) && p.dbg_cycles != nullptr;
    unsigned long long dbg_acc[4] = {0, 0, 0, 0};
    (void)dbg_acc;

    if (warp == 0) {
        // ================================ TMA producer ================================
        // The whole warp walks the loop (uniform control flow and addresses); one elected lane issues.
        const bool leader = elect_one();
        uint32_t it = 0, raw_it = 0;
        bool ok = true;
        // weight tiles (and their scales) of stage `s` for K block kb of a tile
        auto load_weights = [&](int s, int kb, const SubTile (&st)[NB], const uint8_t *const (&sfb_src)[NB]) {
            const uint32_t sb = stage_base(s);
            const int kx = MODE == GEMM_W4A4 ? kb * 128 : kb * 64;
#pragma unroll
            for (int h = 0; h < NB; ++h)
                tma_load_2d(sb + C::A_BYTES + h * C::SUB_BYTES, &p.tm_b[st[h].seg], full_bar(s), kx, st[h].row0);
            if (MODE == GEMM_W4A4 && !GLMASR_EXP(p, 2)) {
                const uint32_t sf = sb + C::A_BYTES + C::B_BYTES;
#pragma unroll
                for (int h = 0; h < NB; ++h)
                    bulk_load_1d(sf + (1 + h) * C::SF_TILE, sfb_src[h] + (size_t)kb * C::SF_TILE, C::SF_TILE, full_bar(s));
            }
        };
        int preloaded = 0;          // stages of the first work item whose weight loads were issued before the wait
        if (early_b) {
            if ((int)blockIdx.x < total_work) {
                const int tile = (int)blockIdx.x / S, split = (int)blockIdx.x - tile * S;
                const int kb0 = split * nkb / S, kb1 = (split + 1) * nkb / S;
                const int n_tile = tile / p.num_m_tiles;
                SubTile st[NB];
                const uint8_t *sfb_src[NB];
#pragma unroll
                for (int h = 0; h < NB; ++h) {
                    st[h] = resolve_subtile(p, n_tile, h, NB);
                    sfb_src[h] = nullptr;
                    if constexpr (MODE == GEMM_W4A4) {
                        const int rt = st[h].ncols > 0 ? (st[h].row0 >> 7) : 0;
                        sfb_src[h] = p.sfb[st[h].seg] + (size_t)rt * p.sf_k_chunks * C::SF_CHUNK;
                    }
                }
                preloaded = kb1 - kb0 < C::STAGES ? kb1 - kb0 : C::STAGES;
                if (GLMASR_EXP(p, 8)) preloaded = 0;
                for (int i = 0; i < preloaded; ++i) {
                    if (leader) {
                        mbar_expect_tx(full_bar(i), GLMASR_EXP(p, 2) ? (uint32_t)(C::A_BYTES + C::B_BYTES) : (uint32_t)C::TX_BYTES);
                        load_weights(i, kb0 + i, st, sfb_src);
                    }
                }
            }
            pdl_wait();
        }
        for (int work = blockIdx.x; ok && work < total_work; work += gridDim.x) {
            const int tile = work / S, split = work - tile * S;
            const int kb0 = split * nkb / S, kb1 = (split + 1) * nkb / S;
            const int m_tile = tile % p.num_m_tiles;
            const int n_tile = tile / p.num_m_tiles;
            SubTile st[NB];
#pragma unroll
            for (int h = 0; h < NB; ++h) st[h] = resolve_subtile(p, n_tile, h, NB);
            const uint8_t *sfa_src = nullptr;
            const uint8_t *sfb_src[NB];
            if constexpr (MODE == GEMM_W4A4) {
                sfa_src = p.sfa + (size_t)m_tile * p.sf_k_chunks * C::SF_CHUNK;
#pragma unroll
                for (int h = 0; h < NB; ++h) {
                    // a sub-tile past the end of its tensor reads tile 0 (any valid memory: its columns are never stored)
                    const int rt = st[h].ncols > 0 ? (st[h].row0 >> 7) : 0;
                    sfb_src[h] = p.sfb[st[h].seg] + (size_t)rt * p.sf_k_chunks * C::SF_CHUNK;
                }
            }
            for (int kb = kb0; kb < kb1; ++kb) {
                if constexpr (MODE == GEMM_W4A16) {
                    if ((kb & 3) == 0) {
                        const int r = raw_it & 1;
                        const uint32_t rph = (raw_it >> 1) & 1u;
                        if (!mbar_wait_warp(rempty_bar(r), rph ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                        const uint32_t rb = raw_tiles + (uint32_t)r * C::RAW_STAGE_BYTES;
                        if (leader) {
                            mbar_expect_tx(rfull_bar(r), C::RAW_STAGE_BYTES);
#pragma unroll
                            for (int h = 0; h < NB; ++h) {
                                tma_load_2d(rb + h * C::RAW_SUB, &p.tm_b[st[h].seg], rfull_bar(r), (kb >> 2) * 128, st[h].row0);
                                tma_load_2d(rb + h * C::RAW_SUB + C::SUB_BYTES, &p.tm_bs[st[h].seg], rfull_bar(r),
                                            (kb >> 2) * 16, st[h].row0);
                            }
                        }
                        ++raw_it;
                    }
                }
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1u;
                DBG_T0();
                if (!mbar_wait_warp(empty_bar(s), ph ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                DBG_ACC(0);
                if (GLMASR_EXP(p, 8) && it >= (uint32_t)C::STAGES) {   // experiment: no memory traffic
                    if (leader) mbar_arrive(full_bar(s));
                    ++it;
                    continue;
                }
                const uint32_t sb = stage_base(s);
                // innermost coordinate in elements of the tensor map: bytes for packed e2m1, bf16 otherwise
                const int kx = MODE == GEMM_W4A4 ? kb * 128 : kb * 64;
                // the first stages of the first work item already have their byte count announced and their
                // weights on the way
                const bool have_weights = work == (int)blockIdx.x && kb - kb0 < preloaded;
                if (leader) {
                    if (!have_weights)
                        mbar_expect_tx(full_bar(s), GLMASR_EXP(p, 2) ? (uint32_t)(C::A_BYTES + C::B_BYTES) : (uint32_t)C::TX_BYTES);
                    tma_load_2d(sb, &p.tm_a, full_bar(s), kx, m_tile * 128);
                    if (MODE == GEMM_W4A4 && !GLMASR_EXP(p, 2))
                        bulk_load_1d(sb + C::A_BYTES + C::B_BYTES, sfa_src + (size_t)kb * C::SF_TILE, C::SF_TILE, full_bar(s));
                    if constexpr (MODE != GEMM_W4A16) {
                        if (!have_weights) load_weights(s, kb, st, sfb_src);
                    }
                }
                ++it;
                DBG_ACC(1);
            }
        }
        if (dbg && leader) { p.dbg_cycles[blockIdx.x * 16 + 0] = dbg_acc[0]; p.dbg_cycles[blockIdx.x * 16 + 1] = dbg_acc[1]; }
    } else if (warp == 1) {
        // ================================ MMA issuer ==================================
        // Warp-uniform loop; the elected lane issues tcgen05.cp / tcgen05.mma / tcgen05.commit.
        const bool leader = elect_one();
        constexpr uint32_t idesc = MODE == GEMM_W4A4 ? idesc_nvfp4(128, C::BN) : idesc_bf16(128, C::BN);
        uint32_t it = 0, acc_it = 0;
        bool ok = true;
        for (int work = blockIdx.x; ok && work < total_work; work += gridDim.x) {
            const int split = work % S;
            const int kb0 = split * nkb / S, kb1 = (split + 1) * nkb / S;
            const int acc = acc_it % C::NUM_ACC;
            const uint32_t aph = (acc_it / C::NUM_ACC) & 1u;
            DBG_T0();
            if (!mbar_wait_warp(tempty_bar(acc), aph ^ 1u, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
            DBG_ACC(0);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(acc * C::BN);
            for (int kb = kb0; kb < kb1; ++kb) {
                const int s = it % C::STAGES;
                const uint32_t ph = (it / C::STAGES) & 1u;
                if (!mbar_wait_warp(full_bar(s), ph, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                DBG_ACC(1);
                tc_fence_after();
                const uint32_t a_addr = stage_base(s);
                const uint32_t b_addr = a_addr + C::A_BYTES;
                const uint32_t sf_set = (GLMASR_EXP(p, 32) ? 0u : (it & 1u)) * C::SF_SET_COLS;
                const uint32_t sfa_t = tmem_base + C::SFA_COL + sf_set;
                const uint32_t sfb_t = tmem_base + C::SFB_COL + sf_set;
                // descriptors differ from stage to stage only in their 14-bit start-address field
                const uint64_t adesc0 = smem_desc_sw128(a_addr);
                const uint64_t bdesc0 = smem_desc_sw128(b_addr);
                if (leader) {
                    if (MODE == GEMM_W4A4 && !(GLMASR_EXP(p, 1) && it > 1)) {
                        const uint64_t sfdesc0 = smem_desc_sf_chunk(a_addr + C::A_BYTES + C::B_BYTES);
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            tmem_cp_32x128b_warpx4(sfa_t + 4 * c, sfdesc0 + (uint64_t)((c * C::SF_CHUNK) >> 4));
#pragma unroll
                        for (int h = 0; h < NB; ++h)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                tmem_cp_32x128b_warpx4(sfb_t + c * 4 * NB + 4 * h,
                                                       sfdesc0 + (uint64_t)(((1 + h) * C::SF_TILE + c * C::SF_CHUNK) >> 4));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (GLMASR_EXP(p, 16) && k > 0) break;   // experiment: a quarter of the MMAs
                        const uint64_t adesc = adesc0 + (uint64_t)((k * 32) >> 4);
                        const uint64_t bdesc = bdesc0 + (uint64_t)((k * 32) >> 4);
                        const uint32_t accumulate = (kb > kb0 || k > 0) ? 1u : 0u;
                        if constexpr (MODE == GEMM_W4A4)
                            umma_nvfp4(d_tmem, adesc, bdesc, idesc, accumulate, sfa_t + 4 * k, sfb_t + 4 * NB * k);
                        else
                            umma_bf16(d_tmem, adesc, bdesc, idesc, accumulate);
                    }
                    umma_commit(empty_bar(s));   // frees the stage once these MMAs have read it
                }
                ++it;
                DBG_ACC(2);
            }
            if (!ok) break;
            if (leader) umma_commit(tfull_bar(acc));     // accumulator complete
            ++acc_it;
        }
        if (dbg && leader) for (int i = 0; i < 3; ++i) p.dbg_cycles[blockIdx.x * 16 + 4 + i] = dbg_acc[i];
    } else if (warp < C::FIRST_DQ_WARP) {
        // ================================ epilogue =====================================
        const int quad = warp & 3;               // TMEM lane quadrant this warp may read
        const int half = (warp - 2) >> 2;        // which half of the accumulator columns
        constexpr int HC = C::BN / (C::EPI_WARPS / 4);   // columns per warp
        constexpr int NCH = HC / 32;             // 32-column groups per warp
        uint32_t acc_it = 0;
        for (int work = blockIdx.x; work < total_work; work += gridDim.x) {
            const int tile = work / S, split = work - tile * S;
            const int m_tile = tile % p.num_m_tiles;
            const int n_tile = tile / p.num_m_tiles;
            const int acc = acc_it % C::NUM_ACC;
            const uint32_t aph = (acc_it / C::NUM_ACC) & 1u;
            DBG_T0();
            bool ok = mbar_wait(tfull_bar(acc), aph, abort_word, ST_TIMEOUT_EPILOGUE);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            DBG_ACC(0);
            tc_fence_after();
            const int row = m_tile * 128 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * C::BN);
            __nv_bfloat16 *out_row = p.out + (size_t)row * p.ldo;
            auto release_acc = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
                DBG_ACC(1);
            };

            // ---- split-K: dump the raw partial; the CTA that arrives last reduces and finishes the tile ----
            bool from_partials = false;
            if constexpr (MODE == GEMM_W4A4) {
                if (S > 1) {
                    const int rowt = quad * 32 + lane;
                    float4 *mine = reinterpret_cast<float4 *>(p.partial + ((size_t)tile * S + split) * (size_t)(128 * C::BN));
#pragma unroll 1
                    for (int ch = 0; ch < NCH; ++ch) {
                        uint32_t r[32];
                        tmem_ld_x32(t_row + half * HC + ch * 32, r);
                        tmem_ld_wait();
                        const int c4 = (half * HC + ch * 32) >> 2;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            __stcg(mine + (size_t)(c4 + j) * 128 + rowt,
                                   make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                    }
                    release_acc();
                    __threadfence();
                    volatile int *flag = reinterpret_cast<volatile int *>(smem_gen + 528) + (acc_it & 1u);
                    asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
                    if (warp == 2 && lane == 0) {
                        const int old = atomicAdd(p.tile_counters + tile, 1);
                        if (old == S - 1) p.tile_counters[tile] = 0;          // ready for the next launch
                        *flag = old;
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
                    if (*flag != S - 1) {
                        DBG_ACC(2);
                        ++acc_it;
                        continue;
                    }
                    __threadfence();
                    from_partials = true;
                }
            }
            // 32 columns of this lane's row, from tile column col0: the sum of the splits' partials in split order
            auto load_sum = [&](int col0, uint32_t (&r)[32]) {
                const int rowt = quad * 32 + lane;
                float4 a[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp = 0; sp < S; ++sp) {
                    const float4 *ps = reinterpret_cast<const float4 *>(p.partial + ((size_t)tile * S + sp) * (size_t)(128 * C::BN));
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 v = __ldcg(ps + (size_t)((col0 >> 2) + j) * 128 + rowt);
                        a[j].x += v.x, a[j].y += v.y, a[j].z += v.z, a[j].w += v.w;
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    r[4 * j] = __float_as_uint(a[j].x), r[4 * j + 1] = __float_as_uint(a[j].y);
                    r[4 * j + 2] = __float_as_uint(a[j].z), r[4 * j + 3] = __float_as_uint(a[j].w);
                }
            };

            if (p.epi == EPI_SILU_GATE) {
                if constexpr (NB == 2) {
                    // gate columns [GC*half, +GC) pair with up columns [128 + GC*half, +GC)
                    constexpr int GC = 128 / (C::EPI_WARPS / 4);
                    constexpr int GCH = GC / 32;
                    const SubTile sg = resolve_subtile(p, n_tile, 0, NB);
                    const float ag = p.alpha[0], au = p.alpha[1];
                    auto finish_gate = [&](const uint32_t (&rg)[32], const uint32_t (&ru)[32], int ch) {
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = bf16_round(__uint_as_float(rg[i]) * ag);
                            const float u = bf16_round(__uint_as_float(ru[i]) * au);
                            v[i] = silu_gate(g, u);
                        }
                        const int c0 = half * GC + ch * 32;
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
                                *reinterpret_cast<uint4 *>(p.q_packed + (size_t)row * p.q_ld + (col >> 1)) = make_uint4(q[0], q[1], q[2], q[3]);
                                uint8_t *sfp = p.q_sf + ((size_t)m_tile * p.q_sf_chunks + (col >> 6)) * 512 + lane * 16 + quad * 4 +
                                               ((col >> 4) & 3);
                                *reinterpret_cast<uint16_t *>(sfp) = (uint16_t)sf;
                            }
                            return;
                        }
                        if (row_ok && nvalid > 0 && !GLMASR_EXP(p, 4)) store_row_chunk(out_row + sg.col0 + c0, v, nvalid);
                    };
                    if (from_partials) {
#pragma unroll 1
                        for (int ch = 0; ch < GCH; ++ch) {
                            uint32_t rg[32], ru[32];
                            load_sum(half * GC + ch * 32, rg);
                            load_sum(128 + half * GC + ch * 32, ru);
                            finish_gate(rg, ru, ch);
                        }
                    } else if constexpr (C::EARLY_RELEASE) {
                        uint32_t rg[GCH][32], ru[GCH][32];
#pragma unroll
                        for (int ch = 0; ch < GCH; ++ch) {
                            tmem_ld_x32(t_row + half * GC + ch * 32, rg[ch]);
                            tmem_ld_x32(t_row + 128 + half * GC + ch * 32, ru[ch]);
                        }
                        tmem_ld_wait();
                        release_acc();
#pragma unroll
                        for (int ch = 0; ch < GCH; ++ch) finish_gate(rg[ch], ru[ch], ch);
                    } else {
#pragma unroll 1
                        for (int ch = 0; ch < GCH; ++ch) {
                            uint32_t rg[32], ru[32];
                            tmem_ld_x32(t_row + half * GC + ch * 32, rg);
                            tmem_ld_x32(t_row + 128 + half * GC + ch * 32, ru);
                            tmem_ld_wait();
                            finish_gate(rg, ru, ch);
                        }
                        release_acc();
                    }
                }
            } else {
                // plain / bias / residual: this warp's columns [half*HC, +HC) of the tile.  They lie in one weight
                // sub-tile when there are two epilogue warps per lane quadrant, and span both sub-tiles of a
                // 256-column tile when there is one (the W4A16 variant): the sub-tile is resolved per 32-column chunk.
                SubTile st = resolve_subtile(p, n_tile, (half * HC) / 128, NB);
                int st_sub = (half * HC) / 128;
                auto finish_chunk = [&](const uint32_t (&r)[32], int ch) {
                    const int tile_col = half * HC + ch * 32;
                    if (tile_col / 128 != st_sub) {
                        st_sub = tile_col / 128;
                        st = resolve_subtile(p, n_tile, st_sub, NB);
                    }
                    const float alpha = p.alpha[st.seg];
                    const int c0 = tile_col % 128;
                    const int nvalid = st.ncols - c0;
                    if (!(row_ok && nvalid > 0)) return;
                    const int col = st.col0 + c0;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
                    if (p.epi == EPI_RESIDUAL) {
                        // the reference adds to the linear's bf16 OUTPUT: bf16(acc) (+ bias, rounded again:
                        // residual_add_bias, Infer-engine/cuda/kernels.cu:763-782), then the residual
                        if (p.bias != nullptr) {
                            float b[32];
                            load_row_chunk(p.bias + col, b, nvalid);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = bf16_round(v[i]) + b[i];
                        }
                        float res[32];
                        load_row_chunk(p.residual + (size_t)row * p.ldo + col, res, nvalid);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = bf16_round(v[i]) + res[i];
                    } else {
                        if (p.bias != nullptr) {
                            float b[32];
                            load_row_chunk(p.bias + col, b, nvalid);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += b[i];
                        }
                        if (p.epi == EPI_GELU) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
                        }
                    }
                    if (!GLMASR_EXP(p, 4)) store_row_chunk(out_row + col, v, nvalid);
                };
                if (from_partials) {
#pragma unroll 1
                    for (int ch = 0; ch < NCH; ++ch) {
                        uint32_t r[32];
                        load_sum(half * HC + ch * 32, r);
                        finish_chunk(r, ch);
                    }
                } else if constexpr (C::EARLY_RELEASE) {
                    uint32_t r[NCH][32];
#pragma unroll
                    for (int ch = 0; ch < NCH; ++ch) tmem_ld_x32(t_row + half * HC + ch * 32, r[ch]);
                    tmem_ld_wait();
                    release_acc();
#pragma unroll
                    for (int ch = 0; ch < NCH; ++ch) finish_chunk(r[ch], ch);
                } else {
#pragma unroll 1
                    for (int ch = 0; ch < NCH; ++ch) {
                        uint32_t r[32];
                        tmem_ld_x32(t_row + half * HC + ch * 32, r);
                        tmem_ld_wait();
                        finish_chunk(r, ch);
                    }
                    release_acc();
                }
            }
            DBG_ACC(2);
            ++acc_it;
        }
        if (dbg && warp == 2 && lane == 0)
            for (int i = 0; i < 3; ++i) p.dbg_cycles[blockIdx.x * 16 + 8 + i] = dbg_acc[i];
    } else {
        // ================================ W4A16 dequant warps ============================
        if constexpr (MODE == GEMM_W4A16) {
            const int dq = warp - C::FIRST_DQ_WARP;
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
    const long long t_roles = dbg ? clock64() : 0;
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
        if (dbg && lane == 0) {
            // kernel timeline of this CTA: set-up, role loops (this warp), teardown
            p.dbg_cycles[blockIdx.x * 16 + 12] = (unsigned long long)(t_setup - t_start);
            p.dbg_cycles[blockIdx.x * 16 + 13] = (unsigned long long)(t_roles - t_setup);
            p.dbg_cycles[blockIdx.x * 16 + 14] = (unsigned long long)(clock64() - t_roles);
        }
    }
}

// ---------------------------------------------------------------------------------------------
template <int MODE, int NB>
static cudaError_t launch_one(const GemmParams &p, int num_ctas, cudaStream_t st) {
    using C = Cfg<MODE, NB>;
    return launch_chained(umma_gemm_kernel<MODE, NB>, dim3(num_ctas), dim3(C::THREADS), (size_t)C::SMEM_BYTES, st, p);
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
    return Cfg<GEMM_W4A4, 2>::THREADS;
}

int umma_gemm_smem_bytes(int mode, int nb) {
    if (mode == GEMM_W4A4) return nb == 2 ? Cfg<GEMM_W4A4, 2>::SMEM_BYTES : Cfg<GEMM_W4A4, 1>::SMEM_BYTES;
    if (mode == GEMM_W4A16) return nb == 2 ? Cfg<GEMM_W4A16, 2>::SMEM_BYTES : Cfg<GEMM_W4A16, 1>::SMEM_BYTES;
    return nb == 2 ? Cfg<GEMM_BF16, 2>::SMEM_BYTES : Cfg<GEMM_BF16, 1>::SMEM_BYTES;
}

}  // namespace glmasr
