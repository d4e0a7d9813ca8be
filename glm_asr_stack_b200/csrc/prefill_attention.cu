// Variable-length GQA self-attention, head_dim 128 (causal, batched prefill) or 64 (non-causal, the audio
// encoder's attention, Infer-engine/cuda/encoder.cu:1870-1970): the kernel is a template on the head dimension.
// Head_dim 128 is the attention
// step of decoder_prefill_paged_batched, Infer-engine/cuda/decoder.cu:1401-1441: per sequence
// softmax(Q K^T / sqrt(d) + causal mask) V over the sequence's own new tokens, q heads sharing
// kv head q / group).  The reference reaches it through a compiled plug-in
// (flash_fwd_vllm_gqa_launch) or a per-sequence path that materialises the scores; the arithmetic is the
// same, here as one flash-attention kernel:
//   * grid = (64-query tiles, q heads, sequences); 4 warps, warp w owns query rows 16 w .. 16 w + 15;
//   * K and V tiles of 64 tokens are staged with 16-byte cp.async into a double buffer, chunks
//     XOR-swizzled by row so that ldmatrix is bank-conflict free;
//   * S = Q K^T and O += P V on mma.sync m16n8k16 (bf16 in, fp32 accumulate), online softmax in
//     fp32 registers, P rounded to bf16 for the second product.
// This warp-level kernel serves the shapes and alignments the tcgen05 kernel
// (prefill_attention_umma.cu) does not take; launch_prefill_attention tries that one first.
#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

#include "decoder_ops.cuh"
#include "runtime.cuh"

namespace glmasr {

namespace {

constexpr int kQTile = 64;                 // queries per CTA
constexpr int kKTile = 64;                 // keys per step
template <int HD>
struct AttnCfg {
    static constexpr int kRowBytes = HD * 2;                       // one K / V row of a head
    static constexpr int kChunks = HD / 8;                         // 16-byte chunks per row
    static constexpr int kTileBytes = kKTile * kRowBytes;          // 16 KB (head_dim 128) / 8 KB (64)
    static constexpr int kSmem = 2 * 2 * kTileBytes;               // K and V, double-buffered
    static constexpr int kKSteps = HD / 16;                        // k steps of the S product, dim-tile pairs of PV
    static constexpr int kDimTiles = HD / 8;                       // 8-column accumulator tiles of O
};

__device__ __forceinline__ void cp16(uint32_t dst, const void *src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&b);
}
// swizzled byte offset of 16-byte chunk c of row r inside a tile (rows of 16 or 8 chunks)
template <int HD>
__device__ __forceinline__ uint32_t toff(int r, int c) { return (uint32_t)(r * AttnCfg<HD>::kRowBytes + ((c ^ (r & 7)) << 4)); }

template <int HD>
__global__ void __launch_bounds__(128) prefill_attention_kernel(__nv_bfloat16 *__restrict__ out, int ldo,
                                                               const __nv_bfloat16 *__restrict__ q, int ldq,
                                                               const __nv_bfloat16 *__restrict__ k, int ldk,
                                                               const __nv_bfloat16 *__restrict__ v, int ldv,
                                                               const int *__restrict__ seq_offsets,
                                                               const int *__restrict__ seq_lens, int group, float scale,
                                                               int causal) {
    using C = AttnCfg<HD>;
    constexpr int kTileBytes = C::kTileBytes;
    extern __shared__ __align__(1024) uint8_t smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, head = blockIdx.y, q0 = blockIdx.x * kQTile;
    // seq_lens == NULL: seq_offsets is a cumulative table of num_seqs + 1 entries (cu_seqlens)
    const int off = seq_offsets[seq];
    const int len = seq_lens != nullptr ? seq_lens[seq] : seq_offsets[seq + 1] - off;
    if (q0 >= len) return;
    const int kv_head = head / group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);

    const int kv_end = causal ? min(len, q0 + kQTile) : len;      // causal: keys up to the tile's last query
    const int nt = (kv_end + kKTile - 1) / kKTile;

    auto load_tile = [&](int t) {
        const uint32_t kdst = sbase + (uint32_t)(t & 1) * (2 * kTileBytes);
        const uint32_t vdst = kdst + kTileBytes;
        constexpr int kRowsPerPass = 128 / C::kChunks;   // 8 (head_dim 128) or 16 (64) rows per pass
        const int c = threadIdx.x % C::kChunks;
        const int r0 = threadIdx.x / C::kChunks;
#pragma unroll
        for (int j = 0; j < kKTile / kRowsPerPass; ++j) {
            const int r = j * kRowsPerPass + r0;
            const int tok = t * kKTile + r;
            const bool valid = tok < len;
            const size_t row = (size_t)(off + (valid ? tok : 0));
            cp16(kdst + toff<HD>(r, c), k + row * ldk + (size_t)kv_head * HD + c * 8, valid);
            cp16(vdst + toff<HD>(r, c), v + row * ldv + (size_t)kv_head * HD + c * 8, valid);
        }
    };

    load_tile(0);
    cp_commit();

    // Q fragments of this warp's 16 rows (rows past the sequence read zeros)
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    uint32_t qa[C::kKSteps][4];
    {
        const __nv_bfloat16 *qa_p = q + (size_t)(off + row_a) * ldq + (size_t)head * HD;
        const __nv_bfloat16 *qb_p = q + (size_t)(off + row_b) * ldq + (size_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < C::kKSteps; ++ks) {
            qa[ks][0] = row_a < len ? *reinterpret_cast<const uint32_t *>(qa_p + ks * 16 + tq * 2) : 0u;
            qa[ks][1] = row_b < len ? *reinterpret_cast<const uint32_t *>(qb_p + ks * 16 + tq * 2) : 0u;
            qa[ks][2] = row_a < len ? *reinterpret_cast<const uint32_t *>(qa_p + ks * 16 + 8 + tq * 2) : 0u;
            qa[ks][3] = row_b < len ? *reinterpret_cast<const uint32_t *>(qb_p + ks * 16 + 8 + tq * 2) : 0u;
        }
    }

    float acc[C::kDimTiles][4];
#pragma unroll
    for (int n = 0; n < C::kDimTiles; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;      // running max / partial sum of rows a, b

    for (int t = 0; t < nt; ++t) {
        if (t + 1 < nt) {
            load_tile(t + 1);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const uint32_t kbase = sbase + (uint32_t)(t & 1) * (2 * kTileBytes);
        const uint32_t vbase = kbase + kTileBytes;
        const int t0 = t * kKTile;
        // a warp whose rows all lie before this key tile has nothing to add (causal)
        const bool warp_live = !causal || t0 <= q0 + warp * 16 + 15;
        if (warp_live) {
            // ---- S = Q K^T: 16 rows x 64 keys = 8 column tiles of 8 ----
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < C::kKSteps; ++ks) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {           // 16 keys per ldmatrix.x4
                    uint32_t kb[4];
                    ldsm4(kbase + toff<HD>(jj * 16 + (lane & 7) + 8 * (lane >> 4), 2 * ks + ((lane >> 3) & 1)), kb);
                    mma16816(s[2 * jj], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
                    mma16816(s[2 * jj + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[2], kb[3]);
                }
            }
            // ---- scale, mask, online softmax (rows a = g and b = g + 8 of the warp's 16) ----
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = t0 + j * 8 + tq * 2 + e;
                    const bool ok_a = key < len && (!causal || key <= row_a);
                    const bool ok_b = key < len && (!causal || key <= row_b);
                    s[j][e] = ok_a ? s[j][e] * scale : -INFINITY;
                    s[j][2 + e] = ok_b ? s[j][2 + e] * scale : -INFINITY;
                    mx_a = fmaxf(mx_a, s[j][e]);
                    mx_b = fmaxf(mx_b, s[j][2 + e]);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xFFFFFFFFu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xFFFFFFFFu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float corr_a = (m_a == -INFINITY) ? 0.0f : __expf(m_a - mn_a);
            const float corr_b = (m_b == -INFINITY) ? 0.0f : __expf(m_b - mn_b);
            float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pa = (s[j][e] == -INFINITY) ? 0.0f : __expf(s[j][e] - mn_a);
                    const float pb = (s[j][2 + e] == -INFINITY) ? 0.0f : __expf(s[j][2 + e] - mn_b);
                    s[j][e] = pa;
                    s[j][2 + e] = pb;
                    sum_a += pa;
                    sum_b += pb;
                }
            }
            l_a = l_a * corr_a + sum_a;
            l_b = l_b * corr_b + sum_b;
            m_a = mn_a;
            m_b = mn_b;
#pragma unroll
            for (int n = 0; n < C::kDimTiles; ++n) {
                acc[n][0] *= corr_a;
                acc[n][1] *= corr_a;
                acc[n][2] *= corr_b;
                acc[n][3] *= corr_b;
            }
            // ---- O += P V: 4 key steps of 16, head_dim / 8 dim tiles of 8 ----
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t pa0 = pack2(s[2 * kk][0], s[2 * kk][1]);
                const uint32_t pa1 = pack2(s[2 * kk][2], s[2 * kk][3]);
                const uint32_t pa2 = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                const uint32_t pa3 = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int j = 0; j < C::kKSteps; ++j) {
                    uint32_t vb[4];
                    ldsm4t(vbase + toff<HD>(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * j + (lane >> 4)), vb);
                    mma16816(acc[2 * j], pa0, pa1, pa2, pa3, vb[0], vb[1]);
                    mma16816(acc[2 * j + 1], pa0, pa1, pa2, pa3, vb[2], vb[3]);
                }
            }
        }
        __syncthreads();                     // the buffer is refilled two iterations later
    }

    // ---- normalise and store ----
    l_a += __shfl_xor_sync(0xFFFFFFFFu, l_a, 1);
    l_a += __shfl_xor_sync(0xFFFFFFFFu, l_a, 2);
    l_b += __shfl_xor_sync(0xFFFFFFFFu, l_b, 1);
    l_b += __shfl_xor_sync(0xFFFFFFFFu, l_b, 2);
    const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f;
    const float inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
    if (row_a < len) {
        __nv_bfloat16 *o = out + (size_t)(off + row_a) * ldo + (size_t)head * HD + tq * 2;
#pragma unroll
        for (int n = 0; n < C::kDimTiles; ++n) *reinterpret_cast<uint32_t *>(o + n * 8) = pack2(acc[n][0] * inv_a, acc[n][1] * inv_a);
    }
    if (row_b < len) {
        __nv_bfloat16 *o = out + (size_t)(off + row_b) * ldo + (size_t)head * HD + tq * 2;
#pragma unroll
        for (int n = 0; n < C::kDimTiles; ++n) *reinterpret_cast<uint32_t *>(o + n * 8) = pack2(acc[n][2] * inv_b, acc[n][3] * inv_b);
    }
}

}  // namespace

bool launch_prefill_attention(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *q, int ldq, const __nv_bfloat16 *k,
                              int ldk, const __nv_bfloat16 *v, int ldv, const int *seq_offsets, const int *seq_lens,
                              int num_seqs, int max_seq_len, int total_tokens, int num_q_heads, int num_kv_heads,
                              int head_dim, bool causal, cudaStream_t st, uint8_t *q_packed, uint8_t *q_sf,
                              float q_input_scale) {
    if (num_seqs > 0 && max_seq_len > 0 &&
        launch_prefill_attention_umma(out, ldo, q, ldq, k, ldk, v, ldv, seq_offsets, seq_lens, num_seqs, max_seq_len,
                                      total_tokens, num_q_heads, num_kv_heads, head_dim, causal, st, q_packed, q_sf,
                                      q_input_scale))
        return true;
    if (q_packed != nullptr) return false;      // only the tcgen05 kernel quantises its output
    if ((head_dim != 128 && head_dim != 64) || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) return false;
    if ((ldq % 2) != 0 || (ldo % 2) != 0 || (ldk % 8) != 0 || (ldv % 8) != 0) return false;
    if ((((uintptr_t)k | (uintptr_t)v) & 15) != 0 || (((uintptr_t)q | (uintptr_t)out) & 3) != 0) return false;
    if (num_seqs <= 0 || max_seq_len <= 0) return true;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(prefill_attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnCfg<128>::kSmem) !=
            cudaSuccess)
            return false;
        configured = true;
    }
    const dim3 grid((max_seq_len + kQTile - 1) / kQTile, num_q_heads, num_seqs);
    const float scale = 1.0f / sqrtf((float)head_dim);
    if (head_dim == 128) {
        GLMASR_PREFER_MAX_SMEM(prefill_attention_kernel<128>);
        launch_chained(prefill_attention_kernel<128>, grid, dim3(128), (size_t)AttnCfg<128>::kSmem, st, out, ldo, q, ldq, k, ldk, v,
                       ldv, seq_offsets, seq_lens, num_q_heads / num_kv_heads, scale, causal ? 1 : 0);
    } else {
        GLMASR_PREFER_MAX_SMEM(prefill_attention_kernel<64>);
        launch_chained(prefill_attention_kernel<64>, grid, dim3(128), (size_t)AttnCfg<64>::kSmem, st, out, ldo, q, ldq, k, ldk, v,
                       ldv, seq_offsets, seq_lens, num_q_heads / num_kv_heads, scale, causal ? 1 : 0);
    }
    return true;
}

}  // namespace glmasr
