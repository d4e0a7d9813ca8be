// Launchers of the decoder's step-resident glue kernels (decoder_ops.cu): RMSNorm, rotate-half
// RoPE for one new token per sequence, paged-KV write, paged GQA decode attention, embedding
// gather, row gather/scatter.  All take explicit row pitches so that they can read q / k / v
// straight out of the fused q|k|v projection output.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace glmasr {

void launch_rmsnorm(__nv_bfloat16 *out, const __nv_bfloat16 *x, const __nv_bfloat16 *weight, float eps, int rows,
                    int dim, cudaStream_t st);
// In place on `tensor` rows of pitch `ld`: heads [0, n_heads) of head_dim at column offset col0.
void launch_rope_single_token(__nv_bfloat16 *tensor, int ld, int col0, const int *positions, int num_seqs, int n_heads,
                              int head_dim, cudaStream_t st);
// RoPE on q (columns [0, q_heads*head_dim)) and k (at k_col) of the new token's q|k|v row, in place, and the
// K / V rows into the paged cache: the three launches between the projection and attention as one.
// Returns false when the layout is not supported (alignment).
// angles (optional): the rows' cos / sin as launch_rope_angles wrote them, so that 28 layers share one evaluation.
bool launch_rope_qk_cache(__nv_bfloat16 *qkv, int ld, int k_col, int v_col, const int *positions,
                          const int64_t *slot_mapping, __nv_bfloat16 *key_cache, __nv_bfloat16 *value_cache, int num_seqs,
                          int q_heads, int kv_heads, int head_dim, cudaStream_t st, const float *angles = nullptr);
// table[rows][head_dim] floats: cos(pos * inv_freq[d]) for d < head_dim / 2, then the sines (the kernel's own expressions).
bool launch_rope_angles(float *table, const int *positions, int rows, int head_dim, cudaStream_t st);
// RMSNorm + activation quantiser for the next W4A4 GEMM: e2m1 bytes [rows, dim/2] and 128x4-tiled scales.
// normed_out (optional, dense [rows, dim], 16-byte aligned): the bf16 result of the norm as well, for consumers
// that take bf16.
bool launch_rmsnorm_quant(uint8_t *q_packed, uint8_t *q_sf, const __nv_bfloat16 *x, const __nv_bfloat16 *weight, float eps,
                          float input_scale, int rows, int dim, cudaStream_t st, __nv_bfloat16 *normed_out = nullptr);
void launch_reshape_and_cache(__nv_bfloat16 *key_cache, __nv_bfloat16 *value_cache, const __nv_bfloat16 *key, int ldk,
                              const __nv_bfloat16 *value, int ldv, const int64_t *slot_mapping, int num_tokens,
                              int num_kv_heads, int head_dim, int block_size, cudaStream_t st);
// Returns false when the shape is not supported (head_dim != 128 or q heads not a multiple of kv heads, group > 8).
bool launch_paged_decode_attention(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *query, int ldq,
                                   const __nv_bfloat16 *key_cache, const __nv_bfloat16 *value_cache,
                                   const int *block_tables, const int *seq_lens, int num_seqs, int num_q_heads,
                                   int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                   cudaStream_t st);
// Flash-decoding variant (paged_attention.cu): cp.async-staged tiles + warp-level tensor-core MMA.
// With q_packed / q_sf the result is written as the quantised operand of the next W4A4 GEMM (e2m1 bytes
// [num_seqs, hidden / 2] + 128x4-tiled scales, quantiser input scale q_input_scale) instead of bf16 to out.
bool launch_paged_decode_attention_mma(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *query, int ldq,
                                       const __nv_bfloat16 *key_cache, const __nv_bfloat16 *value_cache,
                                       const int *block_tables, const int *seq_lens, int num_seqs, int num_q_heads,
                                       int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                                       cudaStream_t st, uint8_t *q_packed = nullptr, uint8_t *q_sf = nullptr,
                                       float q_input_scale = 0.0f);
// Variable-length GQA self-attention of a prefill batch (prefill_attention.cu): sequence s owns rows
// [seq_offsets[s], +seq_lens[s]) of q / k / v / out (device arrays; seq_lens == NULL: seq_offsets is a
// cumulative table of num_seqs + 1 entries); head_dim 128.  total_tokens = rows of q / k / v (the sequences
// lie inside them and do not overlap).  The caller accounts for one launch; a second one (the V transposition
// of the tcgen05 path) is noted by the launcher itself.  With q_packed / q_sf the result is written as the
// next projection's quantised operand (packed e2m1 [rows, q_heads * 64] + 128x4-tiled scales) instead of bf16;
// false if that form is not available for the shape.
bool launch_prefill_attention(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *q, int ldq, const __nv_bfloat16 *k,
                              int ldk, const __nv_bfloat16 *v, int ldv, const int *seq_offsets, const int *seq_lens,
                              int num_seqs, int max_seq_len, int total_tokens, int num_q_heads, int num_kv_heads,
                              int head_dim, bool causal, cudaStream_t st, uint8_t *q_packed = nullptr,
                              uint8_t *q_sf = nullptr, float q_input_scale = 0.0f);
// The tcgen05 kernel behind it (prefill_attention_umma.cu); false = shape or alignment not covered.
bool launch_prefill_attention_umma(__nv_bfloat16 *out, int ldo, const __nv_bfloat16 *q, int ldq, const __nv_bfloat16 *k,
                                   int ldk, const __nv_bfloat16 *v, int ldv, const int *seq_offsets, const int *seq_lens,
                                   int num_seqs, int max_seq_len, int total_tokens, int num_q_heads, int num_kv_heads,
                                   int head_dim, bool causal, cudaStream_t st, uint8_t *q_packed = nullptr,
                                   uint8_t *q_sf = nullptr, float q_input_scale = 0.0f);
void launch_embedding_lookup(__nv_bfloat16 *out, const __nv_bfloat16 *table, const int *ids, int n, int dim,
                             cudaStream_t st);
// out[i, :] = src_rows[i][:]  /  dst_rows[i][:] = in[i, :]   (device arrays of row pointers)
void launch_gather_rows(__nv_bfloat16 *out, const __nv_bfloat16 *const *src_rows, int n, int dim, cudaStream_t st);
void launch_scatter_rows(__nv_bfloat16 *const *dst_rows, const __nv_bfloat16 *in, int n, int dim, cudaStream_t st);
// dst[i, :] = tables[rows[i], :]  (int32 block tables)
void launch_gather_block_tables(int *dst, const int *tables, const int *rows, int n, int width, cudaStream_t st);

}  // namespace glmasr
