// Variable-length GQA self-attention for batched prefill on the tcgen05 tensor cores (head_dim 128).
// Same arithmetic as prefill_attention.cu (the attention step of decoder_prefill_paged_batched,
// Infer-engine/cuda/decoder.cu:1401-1441, and the plug-in entry flash_fwd_vllm_gqa_launch,
// Infer-engine/cuda/flash_fwd_vllm.h:21-30): per sequence softmax(Q K^T / sqrt(d) [+ causal mask]) V.
//
// Persistent CTAs (two per SM) take work items = 128 queries of one (sequence, q head), longest first; the
// keys of an item are walked in steps of 64:
//   warp 0      TMA producer: Q once per item (two 128-row x 64-dim boxes), then per step the K tile (two 64-row
//               boxes) and the V^T tile (128 dims x 64 keys) into two-stage rings, 128-byte swizzle;
//   warp 1      MMA issuer: S_j = Q K_j^T (M 128, N 64, K 128) into one of two TMEM score buffers, and
//               O += P_j V_j (M 128, N 128, K 64) into the TMEM output accumulator; S_{j+1} is issued
//               before P_j V_j so that the soft-max of step j+1 never waits for the second product;
//   warps 2-5   soft-max: thread = query row (TMEM lane).  tcgen05.ld the 64 scores, mask, running
//               maximum and sum in registers, P rounded to bf16 into shared memory in the K-major
//               swizzled layout the second MMA reads.  The accumulator is rescaled (tcgen05.ld / st)
//               only when a row's maximum grew by more than 2^8 since the value P is expressed
//               against -- the final division by the row sum uses the same reference value, so the
//               result is that of the ordinary online soft-max up to rounding.
// 112 KB of shared memory and 256 TMEM columns per CTA: two CTAs per SM, one's soft-max under the
// other's MMAs.  V is consumed as V^T (keys contiguous) so that both products take K-major
// operands: transpose_v_kernel writes V^T for every kv head into a private workspace first, each
// sequence starting at a multiple of 64 columns and zero-filled to the next multiple (10 MB per
// layer at 10000 tokens, a few microseconds).
// Every wait is bounded (status ST_TIMEOUT_ATTENTION); nothing here loads with cluster-wide delivery.
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include <vector>

#include "decoder_ops.cuh"
#include "fp4_format.cuh"
#include "ptx.cuh"
#include "runtime.cuh"

namespace glmasr {

namespace {

constexpr int QT = 128;                       // queries per CTA
constexpr int KT = 64;                        // keys per step
constexpr int P_BYTES = 128 * 128;            // P: 128 queries x 64 keys, bf16
constexpr int TMEM_COLS = 256;                // S0 [0,64), S1 [64,128), O [128,128 + head_dim)
constexpr int THREADS = 192;
constexpr float kRescaleThreshold = 8.0f;     // log2 units

// Shared-memory layout for one head_dim (64: the audio encoder, 128: the decoder).  Rows of Q and K are cut
// into 64-dim boxes of 128 bytes (the widest box the 128-byte swizzle takes).
template <int HD>
struct Geo {
    static_assert(HD == 64 || HD == 128, "head_dim 64 or 128");
    static constexpr int NB = HD / 64;                 // 64-dim boxes per Q / K row
    static constexpr int Q_BYTES = NB * 128 * 128;
    static constexpr int K_BYTES = NB * KT * 128;
    static constexpr int V_BYTES = HD * 128;           // V^T: head_dim dims x 64 keys
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = OFF_Q + Q_BYTES;
    static constexpr int OFF_V = OFF_K + 2 * K_BYTES;
    static constexpr int OFF_P = OFF_V + 2 * V_BYTES;
    static constexpr int OFF_BAR = OFF_P + P_BYTES;    // tiles (112 KB / 64 KB), then barriers
    static constexpr int OFF_OS_TABLE = OFF_BAR + 256; // 128 floats: the quantiser's second division, one entry per scale byte
    static constexpr int SMEM_BYTES = OFF_OS_TABLE + 512;
};

enum : int { B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 3, B_VFULL = 5, B_VEMPTY = 7, B_SFULL = 9, B_SFREE = 11, B_PFULL = 13,
             B_PVDONE = 14, B_QEMPTY = 15, B_OFREE = 16 };

struct AttnParams {
    CUtensorMap tm_q, tm_k, tm_vt;
    __nv_bfloat16 *out;
    const int *seq_offsets;
    const int *seq_lens;          // NULL: seq_offsets is cumulative (num_seqs + 1 entries)
    int *status;
    const int *vt_col;            // first V^T column of every sequence (written by transpose_v_kernel)
    unsigned long long *dbg;      // experiment builds (-DGLMASR_EXPERIMENTS): 8 cycle sums per CTA (soft-max warp 2), else NULL
    int dbg_no_store;             // experiment builds: leave the result stores out
    int ldo, num_q_heads, num_seqs, group, q_tiles, total_items, causal;
    float scale_log2;             // log2(e) / sqrt(head_dim)
    // optional: the result quantised for the next projection (activation quantiser on the bf16 values)
    uint8_t *q_packed;            // [rows, q_ld] e2m1 pairs; NULL = bf16 output to `out`
    uint8_t *q_sf;                // 128x4-tiled e4m3 scales, q_sf_chunks 64-column chunks per row
    int q_ld, q_sf_chunks;
    float q_inv_in;
};

__device__ __forceinline__ int seq_len_of(const int *offs, const int *lens, int s) {
    return lens != nullptr ? lens[s] : offs[s + 1] - offs[s];
}
// First V^T column of sequence `seq`: the lengths before it, each rounded up to 64.
__device__ __forceinline__ int padded_column_of(const int *offs, const int *lens, int seq, int lane) {
    int col = 0;
    for (int s = lane; s < seq; s += 32) col += (seq_len_of(offs, lens, s) + 63) & ~63;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) col += __shfl_xor_sync(0xFFFFFFFFu, col, d);
    return col;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&b);
}

// vt[(h * HD + d) * vt_cols + col(seq) + t] = v[(off(seq) + t) * ldv + h * HD + d], zero for t >= len
// up to the next multiple of 64.  grid = (64-token tiles, kv heads, sequences).
template <int HD>
__global__ void __launch_bounds__(256) transpose_v_kernel(__nv_bfloat16 *__restrict__ vt, int vt_cols,
                                                         const __nv_bfloat16 *__restrict__ v, int ldv,
                                                         const int *__restrict__ seq_offsets,
                                                         const int *__restrict__ seq_lens, int *__restrict__ vt_col,
                                                         int *status) {
    __shared__ uint32_t tile[64][HD / 2 + 1];  // [token][dim pair], odd pitch
    __shared__ int s_col;
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * 64;
    const int off = seq_offsets[seq];
    const int len = seq_len_of(seq_offsets, seq_lens, seq);
    if (t0 >= len) return;
    if (threadIdx.x < 32) {
        const int col = padded_column_of(seq_offsets, seq_lens, seq, threadIdx.x);
        if (threadIdx.x == 0) {
            s_col = col;
            if (blockIdx.x == 0 && blockIdx.y == 0) vt_col[seq] = col;
        }
    }
    constexpr int CH = HD / 8;                  // 16-byte chunks (8 dims) per token row
#pragma unroll
    for (int i = 0; i < 64 * CH / 256; ++i) {
        const int idx = threadIdx.x + i * 256;
        const int r = idx / CH, c = idx % CH;          // token row, 16-byte chunk (8 dims)
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (t0 + r < len) val = *reinterpret_cast<const uint4 *>(v + (size_t)(off + t0 + r) * ldv + (size_t)h * HD + c * 8);
        tile[r][c * 4 + 0] = val.x;
        tile[r][c * 4 + 1] = val.y;
        tile[r][c * 4 + 2] = val.z;
        tile[r][c * 4 + 3] = val.w;
    }
    __syncthreads();
    const int col = s_col;
    if (col + t0 + 64 > vt_cols) {              // the workspace was sized from the caller's token count
        if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, 0, ST_BAD_LAYOUT);
        return;
    }
#pragma unroll
    for (int i = 0; i < HD * 8 / 256; ++i) {
        const int idx = threadIdx.x + i * 256;
        const int d = idx >> 3, c = idx & 7;           // dim row, 16-byte chunk (8 tokens)
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t a = tile[c * 8 + 2 * e][d >> 1], b = tile[c * 8 + 2 * e + 1][d >> 1];
            const uint32_t lo = (d & 1) ? (a >> 16) : (a & 0xFFFFu);
            const uint32_t hi = (d & 1) ? (b >> 16) : (b & 0xFFFFu);
            w[e] = lo | (hi << 16);
        }
        *reinterpret_cast<uint4 *>(vt + (size_t)(h * HD + d) * vt_cols + col + t0 + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Work item = (128-query tile, sequence, q head).  Items are numbered with the last (longest, when causal)
// query tiles first; CTA c takes items c, c + gridDim.x, ...  Every role walks the same item list and keeps
// running counters for its ring stages and barrier phases, so the producer and the MMA issuer run ahead into
// the next item while the soft-max warps still write the current one's result.
struct ItemInfo {
    int head, seq, q0, off, len, n;
};
__device__ __forceinline__ bool decode_item(const AttnParams &p, int item, ItemInfo &it) {
    const int per_tile = p.num_q_heads * p.num_seqs;
    const int x = item % per_tile;
    it.q0 = (p.q_tiles - 1 - item / per_tile) * QT;
    it.head = x % p.num_q_heads;
    it.seq = x / p.num_q_heads;
    it.off = p.seq_offsets[it.seq];
    it.len = seq_len_of(p.seq_offsets, p.seq_lens, it.seq);
    if (it.q0 >= it.len) return false;
    const int kv_end = p.causal ? min(it.len, it.q0 + QT) : it.len;
    it.n = (kv_end + KT - 1) / KT;              // key steps of this tile (>= 1)
    return true;
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 2) prefill_attention_umma_kernel(const __grid_constant__ AttnParams p) {
    using G = Geo<HD>;
    constexpr int OFF_Q = G::OFF_Q, OFF_K = G::OFF_K, OFF_V = G::OFF_V, OFF_P = G::OFF_P, OFF_BAR = G::OFF_BAR;
    constexpr int OFF_OS_TABLE = G::OFF_OS_TABLE, Q_BYTES = G::Q_BYTES, K_BYTES = G::K_BYTES, V_BYTES = G::V_BYTES;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if ((sbase & 1023u) != 0) {                 // the swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, ST_BAD_LAYOUT);
        return;
    }
    auto bar = [&](int i) { return sbase + OFF_BAR + 8u * (uint32_t)i; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + OFF_BAR + 192);
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem + OFF_BAR + 200);

    if (threadIdx.x == 0) {
        mbar_init(bar(B_QFULL), 1);
        mbar_init(bar(B_QEMPTY), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(B_KFULL + s), 1);
            mbar_init(bar(B_KEMPTY + s), 1);
            mbar_init(bar(B_VFULL + s), 1);
            mbar_init(bar(B_VEMPTY + s), 1);
            mbar_init(bar(B_SFULL + s), 1);
            mbar_init(bar(B_SFREE + s), 128);
        }
        mbar_init(bar(B_PFULL), 128);
        mbar_init(bar(B_PVDONE), 1);
        mbar_init(bar(B_OFREE), 128);
        *abort_word = 0;
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_q);
        tma_prefetch_desc(&p.tm_k);
        tma_prefetch_desc(&p.tm_vt);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void *)tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    float *os_table = reinterpret_cast<float *>(smem + OFF_OS_TABLE);
    if (p.q_packed != nullptr) fill_os_table(os_table, p.q_inv_in, (int)threadIdx.x, (int)blockDim.x);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                 // nothing above touched global memory

    if (warp == 0) {
        // ================================ TMA producer ================================
        const bool leader = elect_one();
        uint32_t kv = 0, qi = 0;                // key steps loaded, items started
        bool ok = true;
        for (int item = blockIdx.x; ok && item < p.total_items; item += gridDim.x) {
            ItemInfo it;
            if (!decode_item(p, item, it)) continue;
            const int kv_head = it.head / p.group;
            const int col = p.vt_col[it.seq];
            if (!mbar_wait_warp(bar(B_QEMPTY), (qi & 1u) ^ 1u, abort_word, ST_TIMEOUT_ATTENTION)) break;
            if (leader) {
                mbar_expect_tx(bar(B_QFULL), Q_BYTES);
#pragma unroll
                for (int b = 0; b < G::NB; ++b)
                    tma_load_2d(sbase + OFF_Q + b * (Q_BYTES / G::NB), &p.tm_q, bar(B_QFULL), it.head * HD + 64 * b, it.off + it.q0);
            }
            ++qi;
            for (int j = 0; j < it.n; ++j, ++kv) {
                const int s = (int)(kv & 1u);
                const uint32_t ph = (kv >> 1) & 1u;
                if (!mbar_wait_warp(bar(B_KEMPTY + s), ph ^ 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                if (leader) {
                    const uint32_t dst = sbase + OFF_K + (uint32_t)s * K_BYTES;
                    mbar_expect_tx(bar(B_KFULL + s), K_BYTES);
#pragma unroll
                    for (int b = 0; b < G::NB; ++b)
                        tma_load_2d(dst + b * (K_BYTES / G::NB), &p.tm_k, bar(B_KFULL + s), kv_head * HD + 64 * b, it.off + j * KT);
                }
                if (!mbar_wait_warp(bar(B_VEMPTY + s), ph ^ 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                if (leader) {
                    mbar_expect_tx(bar(B_VFULL + s), V_BYTES);
                    tma_load_2d(sbase + OFF_V + (uint32_t)s * V_BYTES, &p.tm_vt, bar(B_VFULL + s), col + j * KT, kv_head * HD);
                }
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ==================================
        const bool leader = elect_one();
        constexpr uint32_t idesc_s = idesc_bf16(128, KT);
        constexpr uint32_t idesc_o = idesc_bf16(128, HD);
        const uint32_t t_o = tmem_base + 128;
        uint32_t ks = 0, kp = 0, qi = 0;        // S products issued, P V products issued, items started
        bool ok = true;
        for (int item = blockIdx.x; ok && item < p.total_items; item += gridDim.x) {
            ItemInfo it;
            if (!decode_item(p, item, it)) continue;
            if (!mbar_wait_warp(bar(B_QFULL), qi & 1u, abort_word, ST_TIMEOUT_ATTENTION)) break;
            for (int j = 0; j <= it.n; ++j) {
                if (j < it.n) {
                    const int s = (int)(ks & 1u);
                    const uint32_t ph = (ks >> 1) & 1u;
                    if (!mbar_wait_warp(bar(B_KFULL + s), ph, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                    // the score buffer is free once the soft-max of the step two before has loaded it
                    if (!mbar_wait_warp(bar(B_SFREE + s), ph ^ 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                    tc_fence_after();
                    if (leader) {
                        const uint32_t kaddr = sbase + OFF_K + (uint32_t)s * K_BYTES;
#pragma unroll
                        for (int k = 0; k < HD / 16; ++k) {
                            const uint64_t adesc = smem_desc_sw128(sbase + OFF_Q + (uint32_t)(k >> 2) * (Q_BYTES / G::NB)) + (uint64_t)(((k & 3) * 32) >> 4);
                            const uint64_t bdesc = smem_desc_sw128(kaddr + (uint32_t)(k >> 2) * (K_BYTES / G::NB)) + (uint64_t)(((k & 3) * 32) >> 4);
                            umma_bf16(tmem_base + (uint32_t)s * KT, adesc, bdesc, idesc_s, k > 0 ? 1u : 0u);
                        }
                        umma_commit(bar(B_KEMPTY + s));
                        umma_commit(bar(B_SFULL + s));
                        if (j == it.n - 1) umma_commit(bar(B_QEMPTY));      // last product that reads this Q tile
                    }
                    ++ks;
                }
                if (j >= 1) {
                    const int s = (int)(kp & 1u);
                    const uint32_t ph = (kp >> 1) & 1u;
                    if (!mbar_wait_warp(bar(B_VFULL + s), ph, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                    if (!mbar_wait_warp(bar(B_PFULL), kp & 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                    // the first product of an item overwrites the accumulator the previous item's result is read from
                    if (j == 1 && !mbar_wait_warp(bar(B_OFREE), (qi & 1u) ^ 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                    tc_fence_after();
                    if (leader) {
                        const uint64_t adesc0 = smem_desc_sw128(sbase + OFF_P);
                        const uint64_t bdesc0 = smem_desc_sw128(sbase + OFF_V + (uint32_t)s * V_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_bf16(t_o, adesc0 + (uint64_t)((k * 32) >> 4), bdesc0 + (uint64_t)((k * 32) >> 4), idesc_o,
                                      (j > 1 || k > 0) ? 1u : 0u);
                        umma_commit(bar(B_VEMPTY + s));
                        umma_commit(bar(B_PVDONE));
                    }
                    ++kp;
                }
            }
            ++qi;
        }
    } else {
        // ================================ soft-max ====================================
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may access
        const int row = quad * 32 + lane;               // query row of the tile = TMEM lane
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t p_row = sbase + OFF_P + (uint32_t)row * 128u;
        const float scale = p.scale_log2;
        uint32_t sc = 0, pv = 0;                        // key steps consumed, P V products of earlier items
        bool ok = true;
#ifdef GLMASR_EXPERIMENTS
        const bool dbg = p.dbg != nullptr && warp == 2 && lane == 0;
        unsigned long long dsum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tl = dbg ? clock64() : 0;
        const long long t_begin = tl;
#define ATT_DBG(i)                                   \
    if (dbg) {                                       \
        const long long t_ = clock64();              \
        dsum[i] += (unsigned long long)(t_ - tl);    \
        tl = t_;                                     \
    }
#define ATT_STORES_ON (!p.dbg_no_store)
#else
#define ATT_DBG(i) do { } while (0)
#define ATT_STORES_ON true
#endif
        for (int item = blockIdx.x; ok && item < p.total_items; item += gridDim.x) {
            ItemInfo it;
            if (!decode_item(p, item, it)) continue;
            ATT_DBG(7);
            const int n = it.n, len = it.len, head = it.head, off = it.off;
            const int row_g = it.q0 + row;                  // position within the sequence
            const int visible = p.causal ? min(len, row_g + 1) : len;     // keys [0, visible) count for this row
            float m = -INFINITY, l = 0.0f;
            for (int j = 0; j < n; ++j, ++sc) {
                const int b = (int)(sc & 1u);
                if (!mbar_wait_warp(bar(B_SFULL + b), (sc >> 1) & 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                ATT_DBG(1);
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld_x32(t_row + (uint32_t)b * KT, sr[0]);
                tmem_ld_x32(t_row + (uint32_t)b * KT + 32, sr[1]);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(bar(B_SFREE + b));
                const int lim = visible - j * KT;           // columns [0, lim) of this step are visible
                if (lim < KT) {
#pragma unroll
                    for (int c = 0; c < KT; ++c)
                        if (c >= lim) sr[c >> 5][c & 31] = 0xFF800000u;      // -inf
                }
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < KT; c += 2) mx = max3(mx, __uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1]));
                const float m_new = fmaxf(m, mx * scale);
                float alpha = 1.0f;
                if (j == 0) {
                    m = m_new;
                } else if (m_new - m > kRescaleThreshold) {
                    alpha = ex2(m - m_new);
                    m = m_new;
                }
                const bool rescale = __any_sync(0xFFFFFFFFu, alpha != 1.0f);
                const float neg_m = -m;
                // two scores per multiply-add and per addition; the row sum is kept as two partial sums
                const unsigned long long scale2 = pack_f32x2(scale, scale), neg_m2 = pack_f32x2(neg_m, neg_m);
                unsigned long long sum2 = pack_f32x2(0.0f, 0.0f);
                uint32_t pk[32];
#pragma unroll
                for (int c = 0; c < KT; c += 2) {
                    float t0, t1;
                    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[c >> 5][(c & 31) + 1])),
                                           scale2, neg_m2),
                                 t0, t1);
                    const float p0 = ex2(t0), p1 = ex2(t1);
                    sum2 = add_f32x2(sum2, pack_f32x2(p0, p1));
                    pk[c >> 1] = pack2(p0, p1);
                }
                float sum_lo, sum_hi;
                unpack_f32x2(sum2, sum_lo, sum_hi);
                l = l * alpha + (sum_lo + sum_hi);
                ATT_DBG(2);
                if (j >= 1) {
                    // P V of the previous step has to be complete before P is overwritten or O rescaled
                    if (!mbar_wait_warp(bar(B_PVDONE), (pv + (uint32_t)j - 1u) & 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
                    tc_fence_after();
                    if (rescale) {
#pragma unroll 1
                        for (int ch = 0; ch < HD / 32; ++ch) {
                            uint32_t o[32];
                            tmem_ld_x32(t_row + 128 + (uint32_t)ch * 32, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                            tmem_st_x32(t_row + 128 + (uint32_t)ch * 32, o);
                        }
                        tmem_st_wait();
                    }
                }
                ATT_DBG(3);
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    const uint32_t dst = p_row + (uint32_t)((ch ^ (row & 7)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * ch]), "r"(pk[4 * ch + 1]),
                                 "r"(pk[4 * ch + 2]), "r"(pk[4 * ch + 3])
                                 : "memory");
                }
                fence_proxy_async_smem();
                tc_fence_before();
                mbar_arrive(bar(B_PFULL));
                ATT_DBG(4);
            }
            if (!ok) break;
            if (!mbar_wait_warp(bar(B_PVDONE), (pv + (uint32_t)n - 1u) & 1u, abort_word, ST_TIMEOUT_ATTENTION)) { ok = false; break; }
            ATT_DBG(5);
            pv += (uint32_t)n;
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const size_t grow = (size_t)(off + row_g);                 // row of the token in q / k / v / out
            // The result leaves through the warp's own 32 rows of the P tile (free once the last P V has
            // completed; the next item's P is written by the same warp after this), so that global stores
            // cover whole 128-byte (bf16) or 64-byte (quantised) row segments instead of 16 bytes per row.
            const int wrow0 = quad * 32;                               // first tile row of this warp
            const uint32_t stage = sbase + OFF_P + (uint32_t)wrow0 * 128u;
            if (HD != 128 || p.q_packed == nullptr) {
#pragma unroll 1
                for (int half = 0; half < HD / 64; ++half) {
#pragma unroll
                    for (int c2 = 0; c2 < 2; ++c2) {
                        uint32_t o[32];
                        tmem_ld_x32(t_row + 128 + (uint32_t)(half * 64 + c2 * 32), o);
                        tmem_ld_wait();
                        if (half == HD / 64 - 1 && c2 == 1) {           // the accumulator may be overwritten by the next item
                            tc_fence_before();
                            mbar_arrive(bar(B_OFREE));
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t w0 = pack2(__uint_as_float(o[8 * e + 0]) * inv, __uint_as_float(o[8 * e + 1]) * inv);
                            const uint32_t w1 = pack2(__uint_as_float(o[8 * e + 2]) * inv, __uint_as_float(o[8 * e + 3]) * inv);
                            const uint32_t w2 = pack2(__uint_as_float(o[8 * e + 4]) * inv, __uint_as_float(o[8 * e + 5]) * inv);
                            const uint32_t w3 = pack2(__uint_as_float(o[8 * e + 6]) * inv, __uint_as_float(o[8 * e + 7]) * inv);
                            const uint32_t dst = stage + (uint32_t)lane * 128u + (uint32_t)(((c2 * 4 + e) ^ (lane & 7)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                        }
                    }
                    __syncwarp();
                    if (ATT_STORES_ON) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = i * 4 + (lane >> 3), c = lane & 7;       // row of the warp, 16-byte chunk
                            uint4 w;
                            const uint32_t src = stage + (uint32_t)r * 128u + (uint32_t)((c ^ (r & 7)) << 4);
                            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(src));
                            const int rg = it.q0 + wrow0 + r;
                            if (rg < len)
                                *reinterpret_cast<uint4 *>(p.out + (size_t)(off + rg) * p.ldo + (size_t)head * HD + half * 64 + c * 8) = w;
                        }
                    }
                    __syncwarp();
                }
            } else if constexpr (HD == 128) {
                // a row of one head is eight 16-element blocks of the quantiser: 64 packed bytes, 8 scale bytes
                uint32_t sf_lo = 0u, sf_hi = 0u;
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t o[32];
                    tmem_ld_x32(t_row + 128 + (uint32_t)ch * 32, o);
                    tmem_ld_wait();
                    if (ch == 3) {
                        tc_fence_before();
                        mbar_arrive(bar(B_OFREE));
                    }
                    uint32_t pk[4];
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        float v[16];
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            v[e] = __bfloat162float(__float2bfloat16(__uint_as_float(o[16 * hb + e]) * inv));
                        const uint32_t sf = quantize_block16_lut(v, p.q_inv_in, os_table, pk[2 * hb], pk[2 * hb + 1]);
                        const uint32_t byte = (sf & 0xFFu) << (8 * (2 * (ch & 1) + hb));
                        if (ch < 2) sf_lo |= byte;
                        else sf_hi |= byte;
                    }
                    // 64 staged bytes per row; the chunk position is swizzled by the row pair
                    const uint32_t dst = stage + (uint32_t)lane * 64u + (uint32_t)((ch ^ ((lane >> 1) & 3)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = i * 8 + (lane >> 2), c = lane & 3;
                    uint4 w;
                    const uint32_t src = stage + (uint32_t)r * 64u + (uint32_t)((c ^ ((r >> 1) & 3)) << 4);
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(src));
                    const int rg = it.q0 + wrow0 + r;
                    if (rg < len) *reinterpret_cast<uint4 *>(p.q_packed + (size_t)(off + rg) * p.q_ld + (size_t)head * 64 + c * 16) = w;
                }
                __syncwarp();
                if (row_g < len) {
                    const int rem = (int)(grow & 127);
                    uint8_t *sf0 = p.q_sf + ((((grow >> 7) * p.q_sf_chunks + (size_t)(head * 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4;
                    *reinterpret_cast<uint32_t *>(sf0) = sf_lo;
                    *reinterpret_cast<uint32_t *>(sf0 + 512) = sf_hi;           // next 64-column chunk
                }
            }
            ATT_DBG(6);
        }
#ifdef GLMASR_EXPERIMENTS
        if (dbg) {
            dsum[0] = (unsigned long long)(clock64() - t_begin);
            for (int i = 0; i < 8; ++i) p.dbg[(size_t)blockIdx.x * 8 + i] = dsum[i];
        }
#endif
#undef ATT_DBG
#undef ATT_STORES_ON
    }

    // ================================ teardown ==========================================
    tc_fence_before();
    __syncthreads();
    if (*abort_word != 0) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);      // let copies in flight land
        if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
    }
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace

static bool umma_attention_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("GLMASR_ATTN_UMMA");
        on = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// Same contract as launch_prefill_attention; false when the shape is outside what this kernel covers
// (the caller then uses the warp-level kernel).
bool launch_prefill_attention_umma(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *q, int ldq, const __nv_bfloat16 *k,
                                   int ldk, const __nv_bfloat16 *v, int ldv, const int *seq_offsets, const int *seq_lens,
                                   int num_seqs, int max_seq_len, int total_tokens, int num_q_heads, int num_kv_heads,
                                   int head_dim, bool causal, cudaStream_t st, uint8_t *q_packed, uint8_t *q_sf,
                                   float q_input_scale) {
    if (!umma_attention_enabled()) return false;
    if (q_packed != nullptr && (q_sf == nullptr || !(q_input_scale > 0.0f) || (((uintptr_t)q_packed) & 15) != 0 ||
                                (((uintptr_t)q_sf) & 3) != 0 || (num_q_heads % 2) != 0))
        return false;
    if ((head_dim != 128 && head_dim != 64) || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0 || total_tokens <= 0) return false;
    if (head_dim != 128 && q_packed != nullptr) return false;          // the quantising epilogue exists for head_dim 128 only
    const int HD = head_dim;
    if ((ldq % 8) != 0 || (ldo % 8) != 0 || (ldk % 8) != 0 || (ldv % 8) != 0) return false;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) != 0) return false;
    if (ldq < num_q_heads * HD || ldk < num_kv_heads * HD) return false;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(prefill_attention_umma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<128>::SMEM_BYTES) !=
                cudaSuccess ||
            cudaFuncSetAttribute(prefill_attention_umma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<64>::SMEM_BYTES) !=
                cudaSuccess)
            return false;
        cudaFuncSetAttribute(prefill_attention_umma_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(prefill_attention_umma_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             (int)cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    const int vt_cols = (total_tokens + 64 * num_seqs + 63) & ~63;
    __nv_bfloat16 *vt = (__nv_bfloat16 *)workspace_slot(WS_ATTN_VT, (size_t)num_kv_heads * HD * (size_t)vt_cols * 2);
    AttnParams p;
    memset(&p, 0, sizeof(p));
    if (!make_bf16_tmap_sw128(&p.tm_q, q, (uint64_t)num_q_heads * HD, (uint64_t)total_tokens, (uint64_t)ldq * 2, 64, 128)) return false;
    if (!make_bf16_tmap_sw128(&p.tm_k, k, (uint64_t)num_kv_heads * HD, (uint64_t)total_tokens, (uint64_t)ldk * 2, 64, KT)) return false;
    if (!make_bf16_tmap_sw128(&p.tm_vt, vt, (uint64_t)vt_cols, (uint64_t)num_kv_heads * HD, (uint64_t)vt_cols * 2, 64, HD)) return false;
    p.out = out;
    p.seq_offsets = seq_offsets;
    p.seq_lens = seq_lens;
    p.status = device_status_word();
    p.ldo = ldo;
    p.num_q_heads = num_q_heads;
    p.group = num_q_heads / num_kv_heads;
    p.q_tiles = (max_seq_len + QT - 1) / QT;
    p.num_seqs = num_seqs;
    p.total_items = p.q_tiles * num_q_heads * num_seqs;
    int *vt_col = (int *)workspace_slot(WS_ATTN_VT_COL, (size_t)num_seqs * sizeof(int));
    p.vt_col = vt_col;
    p.causal = causal ? 1 : 0;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)head_dim);
    p.q_packed = q_packed;
    p.q_sf = q_sf;
    p.q_ld = num_q_heads * 64;
    p.q_sf_chunks = num_q_heads * 2;
    p.q_inv_in = q_packed != nullptr ? 1.0f / q_input_scale : 0.0f;

    const dim3 tgrid((max_seq_len + 63) / 64, num_kv_heads, num_seqs);
    if (HD == 128)
        launch_chained(transpose_v_kernel<128>, tgrid, dim3(256), (size_t)0, st, vt, vt_cols, v, ldv, seq_offsets, seq_lens, vt_col, p.status);
    else
        launch_chained(transpose_v_kernel<64>, tgrid, dim3(256), (size_t)0, st, vt, vt_cols, v, ldv, seq_offsets, seq_lens, vt_col, p.status);
    note_launches(1);
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
    }
    const dim3 grid(p.total_items < 2 * num_sms ? p.total_items : 2 * num_sms, 1, 1);
#ifdef GLMASR_EXPERIMENTS
    static int debug = -1;
    if (debug < 0) {
        const char *e = getenv("GLMASR_ATTN_DEBUG");
        debug = (e != nullptr && e[0] >= '1' && e[0] <= '2') ? e[0] - '0' : 0;
    }
    p.dbg_no_store = debug == 2 ? 1 : 0;
    if (debug) {
        p.dbg = (unsigned long long *)workspace_slot(WS_ATTN_DEBUG, (size_t)grid.x * 8 * sizeof(unsigned long long));
        cudaMemsetAsync(p.dbg, 0, (size_t)grid.x * 8 * sizeof(unsigned long long), st);
    }
#endif
    if (HD == 128)
        launch_chained(prefill_attention_umma_kernel<128>, grid, dim3(THREADS), (size_t)Geo<128>::SMEM_BYTES, st, p);
    else
        launch_chained(prefill_attention_umma_kernel<64>, grid, dim3(THREADS), (size_t)Geo<64>::SMEM_BYTES, st, p);
#ifdef GLMASR_EXPERIMENTS
    if (debug) {
        // timing experiment: where the soft-max warps of every CTA spent their cycles (averages over the CTAs)
        std::vector<unsigned long long> h((size_t)grid.x * 8);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), p.dbg, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
        double avg[8] = {0};
        for (unsigned c = 0; c < grid.x; ++c)
            for (int i = 0; i < 8; ++i) avg[i] += (double)h[(size_t)c * 8 + i] / grid.x;
        fprintf(stderr, "attention cycles per CTA: loop %.0f | wait S %.0f, soft-max %.0f, wait PV+rescale %.0f, write P %.0f, "
                        "last PV %.0f, result %.0f, item set-up %.0f\n",
                avg[0], avg[1], avg[2], avg[3], avg[4], avg[5], avg[6], avg[7]);
    }
#endif
    return true;
}

}  // namespace glmasr
