// Decode-sized layer tail as one co-resident kernel (sm_100a).
//
// At M <= 256 rows every projection of a decoder layer is a few microseconds of work, and run as one launch per
// operation the step is a chain of ~8 dependent launches per layer whose fixed costs (launch, tensor-memory
// allocation, barrier set-up, first-byte latency of the weight stream, tear-down) exceed the work.  This kernel
// keeps one CTA per SM alive through a PROGRAM of phases
//
//     o + residual | RMSNorm + quantiser | gate|up + SiLU-gate + quantiser | down + residual |
//     RMSNorm + quantiser (next layer) | q|k|v (next layer)
//
// with tensor memory, the mbarrier ring and the TMA descriptors set up once.  Phases are separated by grid-wide
// arrival counters in global memory, one per phase (every CTA adds one to a phase's counter when it has finished
// the phase; the consumers of the next phase poll it with acquire loads, bounded like every wait of this
// library), which needs all CTAs co-resident: the launch is cooperative.
//
// GEMM phases (block-scaled e2m1 x e2m1, semantics of the reference nvfp4_linear,
// Infer-engine/cuda/nvfp4_cutlass.cu:118-270, on an activation the producing phase has already quantised):
//   * a row tile (128 tokens = the 128 TMEM lanes) is shared by grid / num_m_tiles CTAs; each takes a contiguous
//     range of 32-column units of the output, so that all SMs stream a share of the weights whatever N is
//     (N = 2048 at M = 256: 64 units over 74 CTAs per row tile, against 32 CTAs of 128 x 128 tiles);
//   * a CTA's range is at most two RUNS (a run = consecutive units of one weight tensor: gate and up, or the
//     two sides of a q|k / k|v boundary); each run is one tcgen05.mma of N = 32 * units per 64 K-elements;
//   * every CTA of a row tile reads that tile's whole activation operand from L2, so the traffic of a phase grows
//     with the number of CTAs that take part; the host picks that number per phase (TailGemm::cpm, fewer and wider
//     shares where the activation operand dominates, as in the down projection with K = 6144);
//   * the operand ring is one pool of shared memory cut into stages per phase and work item (Geo): a share of one
//     32-column unit gets eight 24 KB stages, gate|up with 3 + 3 units four 46 KB ones;
//   * the weight tiles and weight scales of a phase do not depend on the phase before it: the producer warp issues
//     them for the first ring stages BEFORE it waits for the grid counter, so the weight stream of phase p+1
//     overlaps the counter's latency;
//   * scale factors: the MMA reads the scales of a run's units from consecutive tensor-memory columns starting at a
//     4-column boundary, so the weight scales are re-tiled once per weight and grid partition
//     (tail_retile_scales_kernel): CTA j owns 512-byte chunks [K/64][32 rows][4 unit slots][4 K-blocks] holding
//     exactly its units, in order, from slot 0 (one tcgen05.cp per chunk).
// Norm phases: row r is taken by CTA r % grid, four warps per row, with the reference's summation order
// (Infer-engine/cuda/kernels.cu:252-295) and the activation quantiser of nvfp4_cutlass.cu:35-87 behind it, i.e. the
// same bytes as rmsnorm_quant_kernel.
//
// Data written by one phase and read by the next crosses CTAs through global memory (L2): the writing CTA's warps
// meet at a barrier, one thread fences at gpu scope and adds the CTA's arrival; readers acquire the counter,
// fence generic -> async proxy and only then issue TMA loads; generic reads of such data use ld.global.cg.
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <stdint.h>

#include <map>

#include "decode_tail.cuh"
#include "fp4_format.cuh"
#include "gemm_device.cuh"
#include "gemm_umma.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

namespace {

// cycle accounting of experiment builds: per CTA, phase and role, where the time goes
#ifdef GLMASR_EXPERIMENTS
#define TAIL_T0() long long _t0 = clock64()
#define TAIL_ACC(ph, slot)                                                                                      \
    do {                                                                                                        \
        const long long _t1 = clock64();                                                                        \
        if (P.dbg != nullptr && lane == 0)                                                                      \
            P.dbg[((size_t)blockIdx.x * kTailMaxPhases + (ph)) * 16 + (slot)] += (unsigned long long)(_t1 - _t0); \
        _t0 = _t1;                                                                                              \
    } while (0)
#else
#define TAIL_T0() do { } while (0)
#define TAIL_ACC(ph, slot) do { } while (0)
#endif

constexpr int MAX_STAGES = 8;                            // mbarrier pairs of the operand ring
constexpr int A_BYTES = 128 * 128;                       // 128 rows x 256 K-elements, packed
constexpr int SF_TILE = 2048;                            // scales of 128 rows x 256 K-elements (4 chunks of 512 B)
constexpr int SF_CHUNK = 512;
constexpr int UNIT_BYTES = 32 * 128;                     // 32 weight rows x 256 K-elements
constexpr int OFF_ASF = A_BYTES;
constexpr int OFF_W = OFF_ASF + SF_TILE;                 // weight units of the runs, then one scale tile per run
constexpr int BAR_BYTES = 2048;                          // mbarriers, a few status words, the quantiser's look-up table
constexpr int NORM_ROW_BYTES = 8192;                     // one row of up to 4096 bf16
constexpr int OFF_OS_TABLE = 1024;                       // 128 floats in the second half of the barrier block
constexpr int OFF_TILES = BAR_BYTES;
constexpr int POOL_BYTES = 208 * 1024;                   // operand ring: cut into stages phase by phase (Geo below)
constexpr int OFF_NORM = OFF_TILES + POOL_BYTES;
constexpr int SMEM_BYTES = 1024 + OFF_NORM + 2 * NORM_ROW_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = (2 + EPI_WARPS) * 32;
constexpr int ACC_RUN1 = 128;                            // tensor-memory column of the second run's accumulator
constexpr int SF_BASE = 2 * ACC_RUN1;
static_assert(32 * kTailMaxRunUnits <= ACC_RUN1, "a run's accumulator must fit before the next one");
constexpr int SF_SET_COLS = 16 + 2 * 16;                 // A and each run: 4 columns per 64 K-elements, 4 such steps per stage
constexpr int TMEM_COLS = 512;
static_assert(OFF_W % 1024 == 0 && UNIT_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(SF_BASE + 2 * SF_SET_COLS <= TMEM_COLS, "tensor memory budget");
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
static_assert(OFF_W + 2 * (kTailMaxRunUnits * UNIT_BYTES + SF_TILE) <= POOL_BYTES / 2, "at least two stages for the widest work item");

struct Run {
    int seg;        // weight tensor
    int unit0;      // first 32-row unit inside that tensor
    int units;      // 1..kTailMaxRunUnits
    int col0;       // output column of the run's first element
};
struct Work {
    int m_tile;
    int nruns;      // 0: this CTA has nothing to do in the phase
    Run r[2];
};

// How one CTA's share of a phase lies in a ring stage: A tile, A scales, the runs' weight units, one scale tile per
// run; the pool holds as many such stages as fit (at most MAX_STAGES), so narrow work items get a deeper ring.
struct Geo {
    int off_w[2], off_sf[2];
    int stage_bytes, ns;
    uint32_t tx;                // bytes one stage receives
};

__device__ __forceinline__ Work resolve_work(const TailGemm &g, int num_m_tiles, int cta) {
    Work w;
    w.nruns = 0;
    w.m_tile = 0;
    const int cpm = g.cpm;
    const int m_tile = cta / cpm;
    if (m_tile >= num_m_tiles) return w;
    w.m_tile = m_tile;
    const int j = cta - m_tile * cpm;
    int total = 0;
    if (g.epi == TAIL_EPI_SILU_QUANT) total = g.seg_units[0];
    else
        for (int s = 0; s < g.num_segs; ++s) total += g.seg_units[s];
    const int u0 = (int)(((long long)j * total) / cpm), u1 = (int)(((long long)(j + 1) * total) / cpm);
    if (u1 <= u0) return w;
    if (g.epi == TAIL_EPI_SILU_QUANT) {
        w.nruns = 2;
        w.r[0] = {0, u0, u1 - u0, u0 * 32};
        w.r[1] = {1, u0, u1 - u0, u0 * 32};
        return w;
    }
    int s = 0, first = 0;
    while (s + 1 < g.num_segs && u0 >= first + g.seg_units[s]) first += g.seg_units[s++];
    const int end0 = u1 < first + g.seg_units[s] ? u1 : first + g.seg_units[s];
    w.nruns = 1;
    w.r[0] = {s, u0 - first, end0 - u0, u0 * 32};
    if (end0 < u1) {
        w.nruns = 2;
        w.r[1] = {s + 1, 0, u1 - end0, end0 * 32};
    }
    return w;
}

__device__ __forceinline__ Geo stage_geometry(const Work &w) {
    Geo G;
    int off = OFF_W;
    G.tx = A_BYTES + SF_TILE;
    G.off_w[1] = G.off_sf[1] = 0;
    for (int r = 0; r < w.nruns; ++r) {
        G.off_w[r] = off;
        off += w.r[r].units * UNIT_BYTES;
        G.tx += (uint32_t)(w.r[r].units * UNIT_BYTES + SF_TILE);
    }
    for (int r = 0; r < w.nruns; ++r) {
        G.off_sf[r] = off;
        off += SF_TILE;
    }
    G.stage_bytes = (off + 1023) & ~1023;
    const int fit = POOL_BYTES / G.stage_bytes;
    G.ns = fit < MAX_STAGES ? fit : MAX_STAGES;
    return G;
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait until the grid counter has reached `target` (wrap-safe).  False: the limit ran out, this CTA
// aborted, or the status word says that another CTA (or an earlier launch on the same counter) gave up -- the
// counter will then never reach the target, and the first to time out tells the others through that word.
__device__ __forceinline__ bool grid_wait(const unsigned int *counter, unsigned int target, volatile int *abort_word,
                                          int *status) {
    if ((int)(ld_acquire_gpu(counter) - target) >= 0) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
            if ((int)(ld_acquire_gpu(counter) - target) >= 0) return true;
        if (*abort_word != 0) return false;
        if (status != nullptr && *reinterpret_cast<volatile int *>(status) != 0) {
            *abort_word = ST_TIMEOUT_GRID;
            return false;
        }
        if (clock64() - t0 > kWaitLimitCycles) {
            *abort_word = ST_TIMEOUT_GRID;
            if (status != nullptr) atomicCAS(status, 0, ST_TIMEOUT_GRID);
            return false;
        }
    }
}

// Barrier over `nthreads` threads (named barrier `id`) that also ANDs a predicate, so that a failed bounded wait
// becomes a verdict every participant agrees on.
__device__ __forceinline__ bool named_bar_and(int id, int nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %3, 0;\n\t"
        "bar.red.and.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ uint4 ldcg_u4(const void *p) { return __ldcg(reinterpret_cast<const uint4 *>(p)); }

}  // namespace

__global__ void __launch_bounds__(THREADS, 1) decode_tail_kernel(const __grid_constant__ TailParams P) {
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_raw = smem_u32(smem_dyn);
    const uint32_t smem_base = (smem_raw + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_dyn + (smem_base - smem_raw);

    const uint32_t bar = smem_base;
    auto full_bar = [&](int s) { return bar + 8u * (uint32_t)s; };
    auto empty_bar = [&](int s) { return bar + 8u * (uint32_t)(MAX_STAGES + s); };
    const uint32_t tfull_bar = bar + 8u * (uint32_t)(2 * MAX_STAGES);
    const uint32_t tempty_bar = bar + 8u * (uint32_t)(2 * MAX_STAGES + 1);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + 512);
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem_gen + 520);
    volatile float *rms_slot = reinterpret_cast<volatile float *>(smem_gen + 528);      // two floats
    const uint32_t pool = smem_base + OFF_TILES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int grid = (int)gridDim.x;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        mbar_init(tempty_bar, EPI_WARPS);
        *abort_word = 0;
        fence_mbar_init();
        for (int ph = 0; ph < P.num_phases; ++ph) {
            if (P.kind[ph] != TAIL_GEMM) continue;
            const TailGemm &g = P.g[P.index[ph]];
            tma_prefetch_desc(&g.tm_a);
            for (int s = 0; s < g.num_segs; ++s) tma_prefetch_desc(&g.tm_w[s]);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void *)tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    // the quantising epilogue's second division (inv_in / scale, one of 127 values) looked up: one table per launch
    // (a program has at most one SiLU-gate phase)
    float *os_table = reinterpret_cast<float *>(smem_gen + OFF_OS_TABLE);
    if (warp >= 2) {
        for (int ph = 0; ph < P.num_phases; ++ph)
            if (P.kind[ph] == TAIL_GEMM && P.g[P.index[ph]].epi == TAIL_EPI_SILU_QUANT)
                fill_os_table(os_table, P.g[P.index[ph]].q_inv_in, (int)threadIdx.x - 64, EPI_WARPS * 32);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Every phase has its own arrival counter (a CTA that has nothing to do in a phase arrives at once and runs
    // ahead, so one shared count would not say which phase the arrivals belong to).  The counters only grow:
    // a launch finds them at P.base and every CTA adds one to each.
    auto phase_counter = [&](int ph) { return P.counter + ph * kTailCounterStride; };
    const unsigned int phase_target = P.base + (unsigned int)grid;

    if (warp == 0) {
        // ================================ TMA producer ================================
        const bool leader = elect_one();
        uint32_t fills = 0;          // bit s: parity of the number of times stage s has been filled
        int prev_ns = 0;
        bool ok = true, waited = false;
        for (int ph = 0; ok && ph < P.num_phases; ++ph) {
            if (P.kind[ph] != TAIL_GEMM) continue;
            const TailGemm &g = P.g[P.index[ph]];
            const Work w = resolve_work(g, P.num_m_tiles, (int)blockIdx.x);
            if (w.nruns == 0) continue;
            const Geo G = stage_geometry(w);
            const int nkb = g.K >> 8;
            const int sf_k_chunks = g.K >> 6;
            const int cta_in_tile = (int)blockIdx.x - w.m_tile * g.cpm;
            // per-run state in scalars: the two loops below are the producer's hot path, and indexing the run arrays
            // with a run-time index would put them in local memory
            const bool two = w.nruns > 1;
            const int units0 = w.r[0].units, units1 = two ? w.r[1].units : 0;
            const int row00 = w.r[0].unit0 * 32, row01 = two ? w.r[1].unit0 * 32 : 0;
            const CUtensorMap *tm0 = &g.tm_w[w.r[0].seg], *tm1 = &g.tm_w[two ? w.r[1].seg : 0];
            const uint8_t *sf0 = g.sfb[w.r[0].seg] + (size_t)cta_in_tile * sf_k_chunks * SF_CHUNK;
            const uint8_t *sf1 = g.sfb[two ? w.r[1].seg : 0] + (size_t)cta_in_tile * sf_k_chunks * SF_CHUNK;
            const int off_w0 = G.off_w[0], off_w1 = G.off_w[1], off_sf0 = G.off_sf[0], off_sf1 = G.off_sf[1];
            auto issue_weights = [&](int s, int kb) {
                const uint32_t sb = pool + (uint32_t)(s * G.stage_bytes);
                const uint32_t fb = full_bar(s);
#pragma unroll
                for (int u = 0; u < kTailMaxRunUnits; ++u)
                    if (u < units0) tma_load_2d(sb + off_w0 + u * UNIT_BYTES, tm0, fb, kb * 128, row00 + u * 32);
                bulk_load_1d(sb + off_sf0, sf0 + (size_t)kb * SF_TILE, SF_TILE, fb);
                if (two) {
#pragma unroll
                    for (int u = 0; u < kTailMaxRunUnits; ++u)
                        if (u < units1) tma_load_2d(sb + off_w1 + u * UNIT_BYTES, tm1, fb, kb * 128, row01 + u * 32);
                    bulk_load_1d(sb + off_sf1, sf1 + (size_t)kb * SF_TILE, SF_TILE, fb);
                }
            };
            const CUtensorMap *tma = &g.tm_a;
            const uint8_t *sfa = g.sfa + (size_t)w.m_tile * sf_k_chunks * SF_CHUNK;
            const int a_row = w.m_tile * 128;
            auto issue_acts = [&](int s, int kb) {
                const uint32_t sb = pool + (uint32_t)(s * G.stage_bytes);
                tma_load_2d(sb, tma, full_bar(s), kb * 128, a_row);
                bulk_load_1d(sb + OFF_ASF, sfa + (size_t)kb * SF_TILE, SF_TILE, full_bar(s));
            };
            TAIL_T0();
            // the stages of this phase lie differently in the pool: everything the previous phase put there must
            // have been consumed first (the wait is the one that would precede the next fill of each stage)
            for (int s = 0; ok && s < prev_ns; ++s)
                if (!mbar_wait_warp(empty_bar(s), ((fills >> s) & 1u) ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) ok = false;
            if (!ok) break;
            TAIL_ACC(ph, 0);     // producer: drain
            prev_ns = G.ns;
            // weights of the first ring stages go out before the hand-over of the previous phase is awaited
            const int pre = nkb < G.ns ? nkb : G.ns;
            for (int i = 0; i < pre; ++i) {
                if (leader) {
                    mbar_expect_tx(full_bar(i), G.tx);
                    issue_weights(i, i);
                }
                fills ^= 1u << i;
            }
            TAIL_ACC(ph, 1);     // producer: early weight issue
            if (!waited) {
                pdl_wait();
                waited = true;
            }
            if (ph > 0) {
                bool got = true;
                if (lane == 0) got = grid_wait(phase_counter(ph - 1), phase_target, abort_word, P.status);
                got = __shfl_sync(0xFFFFFFFFu, got, 0);
                if (!got) { ok = false; break; }
                fence_proxy_async_all();
            }
            TAIL_ACC(ph, 2);     // producer: hand-over wait
            for (int i = 0; i < pre; ++i)
                if (leader) issue_acts(i, i);
            TAIL_ACC(ph, 3);     // producer: first activation issues
            for (int kb = pre; kb < nkb; ++kb) {
                const int s = kb % G.ns;
                if (!mbar_wait_warp(empty_bar(s), ((fills >> s) & 1u) ^ 1u, abort_word, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                TAIL_ACC(ph, 4); // producer: waiting for a free stage
                if (GLMASR_EXP(P, 1)) {                 // experiment: no memory traffic after the first ring round
                    if (leader) mbar_arrive(full_bar(s));
                } else if (leader) {
                    const bool no_w = GLMASR_EXP(P, 8), no_a = GLMASR_EXP(P, 16);   // experiments: one operand only
                    mbar_expect_tx(full_bar(s), no_w ? (uint32_t)(A_BYTES + SF_TILE) : (no_a ? G.tx - A_BYTES - SF_TILE : G.tx));
                    if (!no_w) issue_weights(s, kb);
                    if (!no_a) issue_acts(s, kb);
                }
                TAIL_ACC(ph, 5); // producer: issuing a stage
                fills ^= 1u << s;
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ==================================
        const bool leader = elect_one();
        uint32_t uses = 0;           // bit s: parity of the number of times stage s has been consumed
        uint32_t it = 0, acc_it = 0;
        bool ok = true;
        for (int ph = 0; ok && ph < P.num_phases; ++ph) {
            if (P.kind[ph] != TAIL_GEMM) continue;
            const TailGemm &g = P.g[P.index[ph]];
            const Work w = resolve_work(g, P.num_m_tiles, (int)blockIdx.x);
            if (w.nruns == 0) continue;
            const Geo G = stage_geometry(w);
            const int nkb = g.K >> 8;
            const bool two = w.nruns > 1;
            const uint32_t idesc0 = idesc_nvfp4(128, 32 * w.r[0].units);
            const uint32_t idesc1 = idesc_nvfp4(128, 32 * (two ? w.r[1].units : 1));
            // descriptors of stage 0; a stage adds its byte offset to the start-address field (no carry: every
            // shared-memory address is below 2^18)
            const uint64_t adesc_base = smem_desc_sw128(pool);
            const uint64_t b0desc_base = smem_desc_sw128(pool + (uint32_t)G.off_w[0]);
            const uint64_t b1desc_base = smem_desc_sw128(pool + (uint32_t)G.off_w[1]);
            const uint64_t sfa_base = smem_desc_sf_chunk(pool + OFF_ASF);
            const uint64_t sfb0_base = smem_desc_sf_chunk(pool + (uint32_t)G.off_sf[0]);
            const uint64_t sfb1_base = smem_desc_sf_chunk(pool + (uint32_t)G.off_sf[1]);
            const uint32_t stage_step = (uint32_t)G.stage_bytes >> 4;
            TAIL_T0();
            if (!mbar_wait_warp(tempty_bar, (acc_it & 1u) ^ 1u, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after();
            TAIL_ACC(ph, 6);     // MMA: accumulator free
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % G.ns;
                if (!mbar_wait_warp(full_bar(s), (uses >> s) & 1u, abort_word, ST_TIMEOUT_MMA)) { ok = false; break; }
                if (kb == 0) TAIL_ACC(ph, 7); else TAIL_ACC(ph, 8);   // MMA: waiting for the first / a later stage
                uses ^= 1u << s;
                tc_fence_after();
                const uint64_t soff = (uint64_t)((uint32_t)s * stage_step);
                const uint32_t set = tmem_base + SF_BASE + (it & 1u) * SF_SET_COLS;
                if (leader) {
                    if (!(GLMASR_EXP(P, 4) && kb > 0)) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) tmem_cp_32x128b_warpx4(set + 4 * c, sfa_base + soff + (uint64_t)((c * SF_CHUNK) >> 4));
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            tmem_cp_32x128b_warpx4(set + 16 + 4 * c, sfb0_base + soff + (uint64_t)((c * SF_CHUNK) >> 4));
                        if (two) {
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                tmem_cp_32x128b_warpx4(set + 32 + 4 * c, sfb1_base + soff + (uint64_t)((c * SF_CHUNK) >> 4));
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (GLMASR_EXP(P, 2) && k > 0) break;    // experiment: a quarter of the MMAs
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        const uint64_t koff = soff + (uint64_t)((k * 32) >> 4);
                        umma_nvfp4(tmem_base, adesc_base + koff, b0desc_base + koff, idesc0, accumulate, set + 4 * k, set + 16 + 4 * k);
                        if (two)
                            umma_nvfp4(tmem_base + ACC_RUN1, adesc_base + koff, b1desc_base + koff, idesc1, accumulate, set + 4 * k,
                                       set + 32 + 4 * k);
                    }
                    umma_commit(empty_bar(s));
                }
                TAIL_ACC(ph, 9); // MMA: issuing a stage
                ++it;
            }
            if (!ok) break;
            if (leader) umma_commit(tfull_bar);
            ++acc_it;
        }
    } else {
        // ================================ epilogue / norm warps ==========================
        const int ew = warp - 2;                 // 0..7
        const int quad = warp & 3;               // TMEM lane quadrant this warp may read
        const int half = ew >> 2;                // which of the two warps sharing the quadrant; also the norm group
        const int gtid = (ew & 3) * 32 + lane;   // thread index inside the norm group (128 threads)
        uint32_t acc_it = 0;
        bool alive = true;
        pdl_wait();
        for (int ph = 0; ph < P.num_phases; ++ph) {
#ifdef GLMASR_EXPERIMENTS
            long long _t0 = clock64();
#endif
            if (P.kind[ph] == TAIL_GEMM) {
                const TailGemm &g = P.g[P.index[ph]];
                const Work w = resolve_work(g, P.num_m_tiles, (int)blockIdx.x);
                if (w.nruns != 0 && alive) {
                    bool ok = true;
                    // a residual written earlier in this launch by OTHER threads: acquire their arrival first
                    if (g.epi == TAIL_EPI_RESIDUAL && ph > 0 && !g.res_local) {
                        if (lane == 0) ok = grid_wait(phase_counter(ph - 1), phase_target, abort_word, P.status);
                        ok = __all_sync(0xFFFFFFFFu, ok);
                    }
                    // the residual can be fetched while the accumulator is still being computed: the chunk this warp
                    // will finish first, 64 bytes of the thread's row
                    uint4 res_pre[4];
                    const bool pre_res = ok && g.epi == TAIL_EPI_RESIDUAL && (w.m_tile * 128 + quad * 32 + lane) < P.M && half < w.r[0].units + (w.nruns > 1 ? w.r[1].units : 0);
                    if (pre_res) {
                        const int ci0 = half;                                  // first chunk of this warp
                        const int r0 = ci0 < w.r[0].units ? 0 : 1;
                        const int j0 = r0 == 0 ? ci0 : ci0 - w.r[0].units;
                        const __nv_bfloat16 *src = g.out + (size_t)(w.m_tile * 128 + quad * 32 + lane) * g.ldo + w.r[r0].col0 + 32 * j0;
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) res_pre[q4] = ldcg_u4(src + 8 * q4);
                    }
                    ok = ok && mbar_wait(tfull_bar, acc_it & 1u, abort_word, ST_TIMEOUT_EPILOGUE);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (ew == 0) TAIL_ACC(ph, 10);   // epilogue: waiting for the accumulator
                    if (ok) {
                        tc_fence_after();
                        const int row = w.m_tile * 128 + quad * 32 + lane;
                        const bool row_ok = row < P.M;
                        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
                        if (g.epi == TAIL_EPI_SILU_QUANT) {
                            const float ag = g.alpha[0], au = g.alpha[1];
                            for (int j = half; j < w.r[0].units; j += 2) {
                                uint32_t rg[32], ru[32];
                                tmem_ld_x32(t_row + 32 * j, rg);
                                tmem_ld_x32(t_row + ACC_RUN1 + 32 * j, ru);
                                tmem_ld_wait();
                                uint32_t q[4], sf = 0;
                                const unsigned long long ag2 = pack_f32x2(ag, ag), au2 = pack_f32x2(au, au);
#pragma unroll
                                for (int b = 0; b < 2; ++b) {
                                    float blk[16];
#pragma unroll
                                    for (int i = 0; i < 8; ++i) {      // two values at a time: the same bits as the scalar forms
                                        float g0, g1, u0, u1, v0, v1;
                                        scale_round_bf16_x2(__uint_as_float(rg[16 * b + 2 * i]), __uint_as_float(rg[16 * b + 2 * i + 1]), ag2, g0, g1);
                                        scale_round_bf16_x2(__uint_as_float(ru[16 * b + 2 * i]), __uint_as_float(ru[16 * b + 2 * i + 1]), au2, u0, u1);
                                        silu_gate_x2(g0, g1, u0, u1, v0, v1);
                                        round_bf16_x2(v0, v1, blk[2 * i], blk[2 * i + 1]);
                                    }
                                    sf |= quantize_block16_fast(blk, g.q_inv_in, os_table, q[2 * b], q[2 * b + 1]) << (8 * b);
                                }
                                if (row_ok) {
                                    const int col = w.r[0].col0 + 32 * j;
                                    *reinterpret_cast<uint4 *>(g.q_packed + (size_t)row * g.q_ld + (col >> 1)) = make_uint4(q[0], q[1], q[2], q[3]);
                                    uint8_t *sfp = g.q_sf + ((size_t)w.m_tile * g.q_sf_chunks + (col >> 6)) * 512 + lane * 16 + quad * 4 +
                                                   ((col >> 4) & 3);
                                    *reinterpret_cast<uint16_t *>(sfp) = (uint16_t)sf;
                                }
                            }
                        } else {
                            int ci = 0;
                            for (int r = 0; r < w.nruns; ++r) {
                                const float alpha = g.alpha[w.r[r].seg];
                                for (int j = 0; j < w.r[r].units; ++j, ++ci) {
                                    if ((ci & 1) != half) continue;
                                    uint32_t rr[32];
                                    tmem_ld_x32(t_row + (uint32_t)(r * ACC_RUN1 + 32 * j), rr);
                                    tmem_ld_wait();
                                    if (!row_ok) continue;
                                    __nv_bfloat16 *dst = g.out + (size_t)row * g.ldo + w.r[r].col0 + 32 * j;
                                    float v[32];
#pragma unroll
                                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]) * alpha;
                                    if (g.epi == TAIL_EPI_RESIDUAL) {
#pragma unroll
                                        for (int q4 = 0; q4 < 4; ++q4) {
                                            const uint4 rv = (pre_res && ci == half) ? res_pre[q4] : ldcg_u4(dst + 8 * q4);
                                            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                                            for (int i = 0; i < 4; ++i) {
                                                v[8 * q4 + 2 * i] = bf16_round(v[8 * q4 + 2 * i]) + __uint_as_float(rw[i] << 16);
                                                v[8 * q4 + 2 * i + 1] = bf16_round(v[8 * q4 + 2 * i + 1]) + __uint_as_float(rw[i] & 0xFFFF0000u);
                                            }
                                        }
                                    }
#pragma unroll
                                    for (int q4 = 0; q4 < 4; ++q4) {
                                        uint32_t o[4];
#pragma unroll
                                        for (int i = 0; i < 4; ++i) {
                                            const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * q4 + 2 * i], v[8 * q4 + 2 * i + 1]);
                                            o[i] = *reinterpret_cast<const uint32_t *>(&b2);
                                        }
                                        *reinterpret_cast<uint4 *>(dst + 8 * q4) = make_uint4(o[0], o[1], o[2], o[3]);
                                    }
                                }
                            }
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar);
                        ++acc_it;
                    } else {
                        alive = false;
                    }
                }
            } else {
                const TailNorm &nm = P.n[P.index[ph]];
                const int row = (int)blockIdx.x + half * grid;
                const bool has_row = row < P.M;
                uint8_t *rowbuf = smem_gen + OFF_NORM + half * NORM_ROW_BYTES;
                bool ok = alive;
                // one thread of the group acquires the previous phase's hand-over; the group barrier passes it on
                if (ok && ph > 0 && gtid == 0) ok = grid_wait(phase_counter(ph - 1), phase_target, abort_word, P.status);
                ok = named_bar_and(2 + half, 128, ok);
                if (ew == 0) TAIL_ACC(ph, 10);       // norm: waiting for the hand-over
                if (ok && has_row) {
                    const uint4 *xr = reinterpret_cast<const uint4 *>(nm.x + (size_t)row * nm.dim);
                    for (int i = gtid; i < nm.dim / 8; i += 128) reinterpret_cast<uint4 *>(rowbuf)[i] = __ldcg(xr + i);
                }
                ok = named_bar_and(2 + half, 128, ok);
                if (ok && has_row && gtid < 32) {
                    // lane i adds x[i], x[i + 32], ... in that order (the reference's summation order); dim % 64 == 0
                    const uint16_t *rs = reinterpret_cast<const uint16_t *>(rowbuf) + gtid;
                    float sum_sq = 0.0f;
                    for (int t = 0; t < nm.dim / 32; t += 8) {
                        uint32_t h[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) h[u] = rs[(t + u) * 32];
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float v = __uint_as_float(h[u] << 16);
                            sum_sq += v * v;
                        }
                    }
                    for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
                    if (gtid == 0) rms_slot[half] = sqrtf(sum_sq / nm.dim + nm.eps);
                }
                ok = named_bar_and(2 + half, 128, ok);
                if (ok && has_row) {
                    const float rms = rms_slot[half];
                    const ExactRowDivider by_rms(rms);       // same quotients as x / rms, without sixteen IEEE divisions
                    const int sf_chunks = nm.dim / 64;
                    const int rem = row & 127;
                    for (int b = gtid; b < nm.dim / 16; b += 128) {
                        float v[16];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint4 xv = reinterpret_cast<const uint4 *>(rowbuf)[2 * b + h];
                            const uint4 wv = reinterpret_cast<const uint4 *>(nm.weight)[2 * b + h];
                            const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float a0 = by_rms(__uint_as_float(xs[j] << 16)) * __uint_as_float(ws[j] << 16);
                                const float a1 = by_rms(__uint_as_float(xs[j] & 0xFFFF0000u)) * __uint_as_float(ws[j] & 0xFFFF0000u);
                                v[8 * h + 2 * j] = bf16_round(a0);
                                v[8 * h + 2 * j + 1] = bf16_round(a1);
                            }
                        }
                        uint32_t lo, hi;
                        const uint32_t sf = quantize_block16(v, nm.inv_in, lo, hi);
                        *reinterpret_cast<uint2 *>(nm.q_packed + (size_t)row * (nm.dim / 2) + (size_t)b * 8) = make_uint2(lo, hi);
                        nm.q_sf[((((size_t)(row >> 7) * sf_chunks + (b >> 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4 + (b & 3)] = (uint8_t)sf;
                    }
                }
                if (!ok) alive = false;
            }
            // ---- end of the phase: everything this CTA wrote becomes visible, then the CTA arrives ----
            if (ew == 0) TAIL_ACC(ph, 11);           // epilogue / norm: the work itself
            alive = named_bar_and(1, EPI_WARPS * 32, alive);
            if (!alive) break;          // the verdict is the same in all epilogue threads
            if (ew == 0) TAIL_ACC(ph, 12);           // fence + CTA barrier
            if (ew == 0 && lane == 0) {
                __threadfence();
                atomicAdd(phase_counter(ph), 1u);
            }
            if (ew == 0) TAIL_ACC(ph, 13);           // gpu-scope fence + arrival
#ifdef GLMASR_EXPERIMENTS
            if (ew == 0 && lane == 0 && P.dbg != nullptr) P.dbg[((size_t)blockIdx.x * kTailMaxPhases + ph) * 16 + 15] = (unsigned long long)clock64();
#endif
        }
    }

    // ================================ teardown ==========================================
    tc_fence_before();
    __syncthreads();
    if (*abort_word != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);     // let copies still in flight land
        if (threadIdx.x == 0 && P.status != nullptr) atomicCAS(P.status, 0, *abort_word);
    }
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Weight scales [N, K/16] (row-major e4m3, as stored) -> the per-CTA chunks of a GEMM phase whose units are split
// over `cpm` CTAs per row tile: CTA j takes units [j * total / cpm, (j + 1) * total / cpm) of the phase's `total`
// units, of which this tensor holds [seg_first, seg_first + seg_units).  One 32-bit word per thread.
__global__ void tail_retile_scales_kernel(uint32_t *__restrict__ dst, const uint8_t *__restrict__ src, int k16, int cpm,
                                          int total, int seg_first, int seg_units) {
    const int k64s = k16 >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)cpm * k64s * 128) return;
    const int slot = (int)(idx & 3), row = (int)((idx >> 2) & 31);
    const int k64 = (int)((idx >> 7) % k64s), j = (int)((idx >> 7) / k64s);
    const int u0 = (int)(((long long)j * total) / cpm), u1 = (int)(((long long)(j + 1) * total) / cpm);
    const int lo = u0 > seg_first ? u0 : seg_first;
    const int hi = u1 < seg_first + seg_units ? u1 : seg_first + seg_units;
    uint32_t v = 0;
    if (lo + slot < hi)
        v = *reinterpret_cast<const uint32_t *>(src + ((size_t)(lo + slot - seg_first) * 32 + row) * k16 + (size_t)k64 * 4);
    dst[idx] = v;
}

namespace {
struct TailScaleKey {
    const void *src;
    int N, K, cpm, total, seg_first;
    bool operator<(const TailScaleKey &o) const {
        if (src != o.src) return src < o.src;
        if (N != o.N) return N < o.N;
        if (K != o.K) return K < o.K;
        if (cpm != o.cpm) return cpm < o.cpm;
        if (total != o.total) return total < o.total;
        return seg_first < o.seg_first;
    }
};
std::map<TailScaleKey, uint8_t *> g_tail_scales;
}  // namespace

const uint8_t *tail_tiled_scales(const uint8_t *w_scales, int N, int K, int cpm, int total_units, int seg_first, cudaStream_t st) {
    if (w_scales == nullptr || (N % 32) != 0 || (K % 256) != 0 || cpm <= 0 || (((uintptr_t)w_scales) & 3) != 0) return nullptr;
    const TailScaleKey key = {w_scales, N, K, cpm, total_units, seg_first};
    auto it = g_tail_scales.find(key);
    if (it != g_tail_scales.end()) return it->second;
    uint8_t *dst = nullptr;
    const size_t words = (size_t)cpm * (K / 64) * 128;
    if (cudaMalloc(&dst, words * 4) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    tail_retile_scales_kernel<<<(unsigned)((words + 255) / 256), 256, 0, st>>>((uint32_t *)dst, w_scales, K / 16, cpm, total_units,
                                                                               seg_first, N / 32);
    note_launches(1);
    g_tail_scales[key] = dst;
    return dst;
}

void tail_forget_scales(const void *w_scales) {
    for (auto it = g_tail_scales.begin(); it != g_tail_scales.end();) {
        if (w_scales == nullptr || it->first.src == w_scales) {
            cudaFree(it->second);
            it = g_tail_scales.erase(it);
        } else {
            ++it;
        }
    }
}

int tail_choose_cpm(int units, int K, bool silu, int grid, int num_m_tiles) {
    (void)K;
    (void)silu;
    const int max_cpm = num_m_tiles > 0 ? grid / num_m_tiles : 0;
    if (max_cpm <= 0 || units <= 0) return 0;
    // Every available CTA takes part.  Fewer, wider shares cut the L2 traffic of the activation operand (every
    // CTA of a row tile reads all of it) but were slower on B200 at every phase of the 2048 / 6144 decoder
    // (down projection, 256 rows: 14.1 us with 74 CTAs per row tile, 15.9 with 32, 16.8 with 22): a phase is
    // bound by its per-stage hand-overs and fixed latencies, not by that traffic.
    return (units + max_cpm - 1) / max_cpm <= kTailMaxRunUnits ? max_cpm : 0;
}

static int g_tail_grid[64] = {0};
static bool g_tail_ready[64] = {false};
static int g_tail_pdl_ok = -1;           // can the cooperative launch carry the programmatic-serialization attribute

int tail_grid_size() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 0;
    if (g_tail_grid[dev] == 0) {
        int sms = 0, coop = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        g_tail_grid[dev] = coop ? sms : -1;
    }
    return g_tail_grid[dev] > 0 ? g_tail_grid[dev] : 0;
}

cudaError_t launch_decode_tail(const TailParams &p, cudaStream_t st) {
    int dev = 0;
    cudaGetDevice(&dev);
    const int grid = tail_grid_size();
    if (grid <= 0) return cudaErrorNotSupported;
    if (!g_tail_ready[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decode_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_tail_kernel, THREADS, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) return cudaErrorCooperativeLaunchTooLarge;
        g_tail_ready[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (pdl_enabled() && g_tail_pdl_ok != 0) {
        cfg.numAttrs = 2;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_tail_kernel, p);
        if (e == cudaSuccess) {
            g_tail_pdl_ok = 1;
            return e;
        }
        if (g_tail_pdl_ok == 1) return e;
        (void)cudaGetLastError();           // the combination is not accepted here: cooperative only from now on
        g_tail_pdl_ok = 0;
    }
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_tail_kernel, p);
}

}  // namespace glmasr
