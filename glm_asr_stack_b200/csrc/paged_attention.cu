// Paged GQA decode attention, head_dim 128, as a flash-decoding kernel (reference semantics:
// paged_decode_attention, Infer-engine/cuda/paged_kv.cu:321-422, 440-519).
//
// The batched decode step reads ~170 MB of K and V per layer (4.8 GB per step) and only ~1 k
// flops per 512 bytes, so the kernel has to be HBM-bound; a scalar warp-per-head loop (the
// reference's design) is instruction-bound at ~1/10 of the bandwidth.  Here:
//   * one CTA per (kv head, sequence), four warps; warp w takes the 16-token tiles w, w+4, ... of the
//     context and keeps its own online-softmax state; the four partial results are merged through
//     shared memory at the end;
//   * each tile's K and V rows (16 x 256 B each) are brought to shared memory with 16-byte cp.async
//     into a 2-deep per-warp ring (64 KB per CTA, so three CTAs share an SM: measured faster than a deeper ring with two) (rows past the sequence or in masked pages are zero-filled), with
//     the 16-byte chunks XOR-swizzled by row so that ldmatrix is bank-conflict free;
//   * S = Q K^T and O += P V run on mma.sync m16n8k16 (bf16 in, fp32 accumulate): the G <= 8 query
//     heads of the group are rows 0..G-1 of the 16-row A operand.  Four query rows are far below the
//     64/128-row minimum of tcgen05, so the warp-level MMA is the right tool here.
// Result differences to the reference (token-serial fp32 loop): P is rounded to bf16 before the
// PV product and the summation order differs; both are far inside the bf16 output tolerance.
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

#include "decoder_ops.cuh"
#include "fp4_format.cuh"
#include "runtime.cuh"

namespace glmasr {

static constexpr int kTile = 16;                       // tokens per tile
static constexpr int kRowBytes = 256;                  // one K or V row of one kv head (128 bf16)
static constexpr int kTileBytes = kTile * kRowBytes;   // 4 KB
static constexpr int kStages = 2;
static constexpr int kWarps = 4;
static constexpr int kWarpSmem = kStages * 2 * kTileBytes;          // K and V rings of one warp: 16 KB
static constexpr int kAttnSmem = kWarps * kWarpSmem;                // 64 KB


__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&b);
}

// swizzled byte offset of 16-byte chunk c (0..15) of row r (0..15) inside a 4 KB tile
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * kRowBytes + ((c ^ (r & 7)) << 4)); }

// PAGE_ALIGNED: block_size is a multiple of the 16-token tile, so a tile lies in one page: one block-table
// lookup and one division per tile instead of one per row, and row addresses by pointer increments.
template <bool PAGE_ALIGNED>
__global__ void __launch_bounds__(kWarps * 32) paged_decode_attention_mma_kernel(
    __nv_bfloat16 *__restrict__ out, int ldo, const __nv_bfloat16 *__restrict__ query, int ldq,
    const __nv_bfloat16 *__restrict__ key_cache, const __nv_bfloat16 *__restrict__ value_cache,
    const int *__restrict__ block_tables, const int *__restrict__ seq_lens, int num_kv_heads, int group,
    int block_size, int max_blocks_per_seq, float scale, uint8_t *__restrict__ q_packed, uint8_t *__restrict__ q_sf,
    int q_sf_chunks, float q_inv_in) {
    extern __shared__ __align__(1024) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int kv_head = blockIdx.x;
    const int seq = blockIdx.y;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;            // MMA row / column group of this lane (query head when < group)
    const int tq = lane & 3;
    const int seq_len = seq_lens[seq];
    const int q_head0 = kv_head * group;

    if (seq_len <= 0) {                 // reference: zeros
        if (q_packed != nullptr) {      // zeros quantise to zero codes and zero scales
            const int hidden = num_kv_heads * group * 128;
            for (int i = threadIdx.x; i < group * 64; i += blockDim.x)
                q_packed[(size_t)seq * (hidden / 2) + (size_t)q_head0 * 64 + i] = 0;
            for (int b = threadIdx.x; b < group * 8; b += blockDim.x) {
                const int kb = q_head0 * 8 + b, rem = seq & 127;
                q_sf[((((size_t)(seq >> 7) * q_sf_chunks + (kb >> 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4 + (kb & 3)] = 0;
            }
            return;
        }
        for (int i = threadIdx.x; i < group * 128; i += blockDim.x)
            out[(size_t)seq * ldo + (size_t)q_head0 * 128 + i] = __float2bfloat16(0.0f);
        return;
    }

    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t ring = smem_base + (uint32_t)warp * kWarpSmem;
    const int *bt = block_tables + (size_t)seq * max_blocks_per_seq;
    const size_t row_elems = (size_t)num_kv_heads * 128;
    const size_t head_off = (size_t)kv_head * 128;
    const int num_tiles = (seq_len + kTile - 1) / kTile;
    const int my_tiles = num_tiles > warp ? (num_tiles - warp + kWarps - 1) / kWarps : 0;

    // ---- producer: this warp's tile i (global tile index warp + 4 i) into ring slot i % kStages ----
    auto load_tile = [&](int i) {
        const int tile = warp + kWarps * i;
        const uint32_t kdst = ring + (uint32_t)(i % kStages) * (2 * kTileBytes);
        const uint32_t vdst = kdst + kTileBytes;
        const int c = lane & 15;                        // 16-byte chunk of the row
        if (PAGE_ALIGNED) {
            const int t0 = tile * kTile;
            const int page = t0 / block_size;
            const int blk = bt[page];
            const bool page_ok = blk >= 0;
            const int r0 = lane >> 4;
            size_t off = page_ok ? ((size_t)blk * block_size + (size_t)(t0 - page * block_size) + r0) * row_elems + head_off + c * 8 : 0;
            const int rows_left = seq_len - t0;         // rows r < rows_left exist
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = j * 2 + r0;
                const bool valid = page_ok && r < rows_left;
                const size_t o = valid ? off : 0;
                cp_async16_zfill(kdst + tile_off(r, c), key_cache + o, valid);
                cp_async16_zfill(vdst + tile_off(r, c), value_cache + o, valid);
                off += 2 * row_elems;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int r = j * 2 + (lane >> 4);          // row of the tile
                const int t = tile * kTile + r;
                int blk = -1;
                if (t < seq_len) blk = bt[t / block_size];
                const bool valid = blk >= 0;
                const size_t base = valid ? ((size_t)blk * block_size + (size_t)(t % block_size)) * row_elems + head_off + c * 8 : 0;
                cp_async16_zfill(kdst + tile_off(r, c), key_cache + base, valid);
                cp_async16_zfill(vdst + tile_off(r, c), value_cache + base, valid);
            }
        }
    };

    float acc[16][4];                   // O accumulators: 16 dim-tiles of 8; [.][0..1] are rows g (valid), [2..3] rows g+8 (unused)
#pragma unroll
    for (int n = 0; n < 16; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    float run_max = -INFINITY, run_sum = 0.0f;

#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if (i < my_tiles) load_tile(i);
        cp_async_commit();
    }

    // ---- Q fragments (loaded while the first K / V tiles are on their way): rows = query heads of the group (lanes with g >= group hold zeros) ----
    uint32_t qa[8][2];
    {
        const __nv_bfloat16 *qp = query + (size_t)seq * ldq + (size_t)(q_head0 + g) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = 0u;
            qa[ks][1] = 0u;
            if (g < group) {
                qa[ks][0] = *reinterpret_cast<const uint32_t *>(qp + ks * 16 + tq * 2);
                qa[ks][1] = *reinterpret_cast<const uint32_t *>(qp + ks * 16 + 8 + tq * 2);
            }
        }
    }


    for (int i = 0; i < my_tiles; ++i) {
        if (i + kStages - 1 < my_tiles) load_tile(i + kStages - 1);
        cp_async_commit();
        cp_async_wait<kStages - 1>();        // this warp's tile i has landed (groups complete in order)
        __syncwarp();

        const int t0 = (warp + kWarps * i) * kTile;
        const uint32_t kbase = ring + (uint32_t)(i % kStages) * (2 * kTileBytes);
        const uint32_t vbase = kbase + kTileBytes;

        // ---- S = Q K^T for 16 tokens: two 8-token column tiles ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t kb[4];
            ldmatrix_x4(kbase + tile_off((lane & 7) + 8 * (lane >> 4), 2 * ks + ((lane >> 3) & 1)), kb);
            mma_bf16_16816(s0, qa[ks][0], 0u, qa[ks][1], 0u, kb[0], kb[1]);
            mma_bf16_16816(s1, qa[ks][0], 0u, qa[ks][1], 0u, kb[2], kb[3]);
        }
        // this lane holds, for query head g, the scores of tokens t0 + {2tq, 2tq+1, 8+2tq, 9+2tq}
        float sc[4] = {s0[0], s0[1], s1[0], s1[1]};
        float tmax = -INFINITY;
        const bool tile_page_ok = PAGE_ALIGNED ? bt[t0 / block_size] >= 0 : true;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int t = t0 + (e >> 1) * 8 + tq * 2 + (e & 1);
            const bool ok = PAGE_ALIGNED ? (tile_page_ok && t < seq_len) : (t < seq_len && bt[t / block_size] >= 0);
            sc[e] = ok ? sc[e] * scale : -INFINITY;
            tmax = fmaxf(tmax, sc[e]);
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, 2));
        const float m_new = fmaxf(run_max, tmax);
        const float corr = (run_max == -INFINITY) ? 0.0f : __expf(run_max - m_new);
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) p[e] = (sc[e] == -INFINITY) ? 0.0f : __expf(sc[e] - m_new);
        run_sum = run_sum * corr + ((p[0] + p[1]) + (p[2] + p[3]));
        run_max = m_new;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            acc[n][0] *= corr;
            acc[n][1] *= corr;
        }
        // ---- O += P V ----
        const uint32_t pa0 = pack_bf16x2(p[0], p[1]);
        const uint32_t pa2 = pack_bf16x2(p[2], p[3]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vbase + tile_off((lane & 7) + 8 * ((lane >> 3) & 1), 2 * j + (lane >> 4)), vb);
            mma_bf16_16816(acc[2 * j], pa0, 0u, pa2, 0u, vb[0], vb[1]);
            mma_bf16_16816(acc[2 * j + 1], pa0, 0u, pa2, 0u, vb[2], vb[3]);
        }
        __syncwarp();                        // every lane is done with this slot before it is refilled
    }
    cp_async_wait<0>();

    // ---- merge the four warps' partial results ----
    run_sum += __shfl_xor_sync(0xFFFFFFFFu, run_sum, 1);
    run_sum += __shfl_xor_sync(0xFFFFFFFFu, run_sum, 2);
    __syncthreads();                         // rings are dead: reuse shared memory for the partials
    float *part = reinterpret_cast<float *>(smem);              // [warp][head][130]: max, sum, 128 accumulators
    constexpr int kPart = 130;
    if (g < group) {
        float *mine = part + ((size_t)warp * 8 + g) * kPart;
        if (tq == 0) {
            mine[0] = run_max;
            mine[1] = run_sum;
        }
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            mine[2 + n * 8 + tq * 2] = acc[n][0];
            mine[2 + n * 8 + tq * 2 + 1] = acc[n][1];
        }
    }
    __syncthreads();
    if (q_packed != nullptr) {
        // the o projection's operand directly: 16-element blocks of the bf16-rounded result through the
        // activation quantiser (same bytes as the bf16 output followed by the stand-alone quantiser)
        const int hidden = num_kv_heads * group * 128;
        for (int task = threadIdx.x; task < group * 8; task += blockDim.x) {
            const int h = task >> 3, b = task & 7;
            float m = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) m = fmaxf(m, part[((size_t)w * 8 + h) * kPart]);
            float e[kWarps], den = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float *pw = part + ((size_t)w * 8 + h) * kPart;
                e[w] = (pw[0] == -INFINITY) ? 0.0f : __expf(pw[0] - m);
                den += e[w] * pw[1];
            }
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float num = 0.0f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) num += e[w] * part[((size_t)w * 8 + h) * kPart + 2 + b * 16 + j];
                v[j] = __bfloat162float(__float2bfloat16(num / (den + 1e-9f)));
            }
            uint32_t lo, hi;
            const uint32_t sf = quantize_block16(v, q_inv_in, lo, hi);
            const int col = (q_head0 + h) * 128 + b * 16;
            *reinterpret_cast<uint2 *>(q_packed + (size_t)seq * (hidden / 2) + (col >> 1)) = make_uint2(lo, hi);
            const int kb = col >> 4, rem = seq & 127;
            q_sf[((((size_t)(seq >> 7) * q_sf_chunks + (kb >> 2)) * 32 + (rem & 31)) * 4 + (rem >> 5)) * 4 + (kb & 3)] = (uint8_t)sf;
        }
        return;
    }
    for (int idx = threadIdx.x; idx < group * 128; idx += blockDim.x) {
        const int h = idx >> 7, d = idx & 127;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, part[((size_t)w * 8 + h) * kPart]);
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float *pw = part + ((size_t)w * 8 + h) * kPart;
            const float e = (pw[0] == -INFINITY) ? 0.0f : __expf(pw[0] - m);
            num += e * pw[2 + d];
            den += e * pw[1];
        }
        out[(size_t)seq * ldo + (size_t)(q_head0 + h) * 128 + d] = __float2bfloat16(num / (den + 1e-9f));
    }
}

bool launch_paged_decode_attention_mma(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *query, int ldq,
                                       const __nv_bfloat16 *key_cache, const __nv_bfloat16 *value_cache,
                                       const int *block_tables, const int *seq_lens, int num_seqs, int num_q_heads,
                                       int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                       cudaStream_t st, uint8_t *q_packed, uint8_t *q_sf, float q_input_scale) {
    if (head_dim != 128 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return false;
    const int group = num_q_heads / num_kv_heads;
    if (group > 8 || (ldq % 2) != 0) return false;
    if ((((uintptr_t)key_cache | (uintptr_t)value_cache) & 15) != 0 || (((uintptr_t)query) & 3) != 0) return false;
    if (num_seqs <= 0) return true;
    if (q_packed != nullptr && (q_sf == nullptr || !(q_input_scale > 0.0f) || (((uintptr_t)q_packed) & 7) != 0)) return false;
    const int q_sf_chunks = num_q_heads * head_dim / 64;
    const float q_inv_in = q_packed != nullptr ? 1.0f / q_input_scale : 0.0f;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(paged_decode_attention_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kAttnSmem) != cudaSuccess ||
            cudaFuncSetAttribute(paged_decode_attention_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kAttnSmem) != cudaSuccess)
            return false;
        configured = true;
    }
    GLMASR_PREFER_MAX_SMEM(paged_decode_attention_mma_kernel<true>);
    GLMASR_PREFER_MAX_SMEM(paged_decode_attention_mma_kernel<false>);
    const float scale = 1.0f / sqrtf((float)head_dim);
    dim3 grid(num_kv_heads, num_seqs);
    if (block_size % kTile == 0)
        launch_chained(paged_decode_attention_mma_kernel<true>, grid, dim3(kWarps * 32), (size_t)kAttnSmem, st, out, ldo, query,
                       ldq, key_cache, value_cache, block_tables, seq_lens, num_kv_heads, group, block_size,
                       max_blocks_per_seq, scale, q_packed, q_sf, q_sf_chunks, q_inv_in);
    else
        launch_chained(paged_decode_attention_mma_kernel<false>, grid, dim3(kWarps * 32), (size_t)kAttnSmem, st, out, ldo, query,
                       ldq, key_cache, value_cache, block_tables, seq_lens, num_kv_heads, group, block_size,
                       max_blocks_per_seq, scale, q_packed, q_sf, q_sf_chunks, q_inv_in);
    return true;
}

}  // namespace glmasr
