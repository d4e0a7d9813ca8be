/*
 * libglmasr_fp4 -- B200 (sm_100a) drop-in for the FP4-weight linear path of the GLM-ASR
 * Infer-engine.  Plain C ABI: bf16 tensors are uint16_t*, handles are void*, every pointer
 * is a DEVICE pointer unless the parameter name ends in _host.
 *
 * Section 1 re-exports, with unchanged names, argument order and error behaviour, the
 * symbols the engine's decoder links for this path; each declaration cites the reference
 * interface it replaces (paths inside the reference project).  Section 2 is additive.
 *
 * Threading/stream contract (same as the reference): one host thread, launches go to the
 * legacy default stream unless glmasr_set_stream() was called, not re-entrant.
 * Error contract: the void entry points print to stderr and exit(1) on a CUDA error
 * (reference: Infer-engine/include/types.h:182-199); the int entry points return 0 on
 * success and -1 on bad arguments or a launch failure.
 *
 * FP4 storage format (reference: Infer-engine/cuda/kernels.cu:96-120, 200-231):
 *   w_packed  uint8 [N, K/2]   two e2m1 nibbles per byte, even k in bits 0-3
 *   w_scales  uint8 [N, K/16]  one e4m3 scale per 16 consecutive k, row-major
 *   w_global_scale  fp32 per tensor;   weight = lut[nibble] * e4m3(scale) * global
 */
#ifndef GLMASR_FP4_H
#define GLMASR_FP4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ======================= 1. reference symbols (drop-in) ======================= */

/* Infer-engine/include/cuda_kernels.h:17-21, Infer-engine/cuda/kernels.cu:234-246.
 * out[r,c] = bf16(lut[nibble] * e4m3(block_scales[r, c/16]) * global_scale);
 * block_scales == NULL means scale 1.  Bit-exact with the reference. */
void fp4_dequant_to_bf16(uint16_t *out, const uint8_t *packed_w, const uint8_t *block_scales,
                         float global_scale, int rows, int cols);

/* Infer-engine/include/cuda_kernels.h:80-89, Infer-engine/cuda/kernels.cu:1297-1318.
 * W4A16: out[M,N] = bf16(x[M,K] * dequant(W)[N,K]^T (+ bias)), fp32 accumulation.
 * The reference materialises the bf16 weight in weight_scratch on every call.  Here, below
 * 1024 rows (decode), the weight is dequantised inside the GEMM and weight_scratch is left
 * untouched; from 1024 rows (prefill) it is dequantised once per call into weight_scratch
 * (a private workspace if NULL), exactly like the reference, and a bf16 GEMM follows.
 * prequant_scratch ([M,K] bf16) is written only when pre_quant_scale != NULL, as in the
 * reference.  handle is ignored (no cuBLAS). */
void fp4_linear(void *handle, uint16_t *out, uint16_t *weight_scratch, uint16_t *prequant_scratch,
                const uint16_t *x, const uint8_t *w_packed, const uint8_t *w_scales,
                float w_global_scale, const uint16_t *pre_quant_scale, const uint16_t *bias,
                int M, int N, int K);

/* Infer-engine/include/cuda_kernels.h:91, Infer-engine/cuda/nvfp4_cutlass.cu:113-116. Returns 1. */
int nvfp4_cutlass_available(void);

/* Infer-engine/include/cuda_kernels.h:93-101, Infer-engine/cuda/nvfp4_cutlass.cu:118-270.
 * W4A4: activations are quantised to e2m1 with one e4m3 scale per 16 k exactly as the
 * reference quantiser does, then a block-scaled FP4 x FP4 product with fp32 accumulation,
 * alpha = input_scale * w_global_scale, bf16 out.  Returns -1 (nothing launched) when
 * M, N or K <= 0, w_scales == NULL, K % 16 != 0 or input_scale <= 0.  bias is ignored, as
 * in the reference.  dequant_buf is NOT used: temporaries live in a private workspace
 * (the reference carves them from dequant_buf + N*K and can overrun it). */
int nvfp4_linear(void *handle, uint16_t *out, uint16_t *dequant_buf, const uint16_t *x,
                 const uint8_t *w_packed, const uint8_t *w_scales, float input_scale,
                 float w_global_scale, const uint16_t *pre_quant_scale, const uint16_t *bias,
                 int M, int N, int K);

/* Infer-engine/include/cuda_kernels.h:66-70, Infer-engine/cuda/kernels.cu:1147-1193.
 * out[M,N] = bf16(x[M,K] * w[N,K]^T (+ bias)), bf16 weights (the reference lm_head). */
void bf16_linear(void *handle, uint16_t *out, const uint16_t *x, const uint16_t *w,
                 const uint16_t *bias, int M, int N, int K);

/* Infer-engine/include/cuda_kernels.h:76-78, Infer-engine/cuda/kernels.cu:1252-1273.
 * out[m,n] = bf16((g*sigmoid(g))*u), g = packed[m,n], u = packed[m,N+n]. */
void silu_mul_split_packed(uint16_t *out, const uint16_t *packed_gate_up, int M, int N);

/* Infer-engine/include/cuda_kernels.h:32, Infer-engine/cuda/kernels.cu:405-421. In place on gate. */
void silu_elementwise_mul(uint16_t *gate, const uint16_t *up, int n);

/* Infer-engine/include/cuda_kernels.h:45-46, Infer-engine/cuda/kernels.cu:741-761. */
void residual_add(uint16_t *out, const uint16_t *a, const uint16_t *b, int n);

/* Infer-engine/include/cuda_kernels.h:176-180, Infer-engine/cuda/kernels.cu:1443-1459.
 * bf16 lm_head projection + row arg-max (reference tie-break), tokens copied to the HOST
 * array out_tokens_host before returning. */
void lm_head_argmax_batched(void *handle, const uint16_t *hidden, const uint16_t *lm_weight,
                            int rows, int dim, int vocab_size, int *out_tokens_host);

/* Infer-engine/include/cuda_kernels.h:182, Infer-engine/cuda/kernels.cu:1461-1475. */
void lm_head_cleanup(void);

/* ---- decode step and its glue (layout of the structs: include/glmasr_engine_types.h) ---- */

/* Infer-engine/include/cuda_kernels.h:23-24, Infer-engine/cuda/kernels.cu:252-295.  Bit-exact
 * (same summation order as the reference's one-warp-per-row kernel); out may alias x. */
void rmsnorm(uint16_t *out, const uint16_t *x, const uint16_t *weight, float eps, int rows, int dim);

/* Infer-engine/include/cuda_kernels.h:42-43, Infer-engine/cuda/kernels.cu:712-736. */
void embedding_lookup(uint16_t *out, const uint16_t *table, const int *ids, int n, int dim);

/* Infer-engine/cuda/paged_kv.cu:424-438 (kernel :70-97): scatter K/V rows [num_tokens, kv_heads*head_dim]
 * to slot_mapping[token] = block * block_size + offset of the paged cache. */
void reshape_and_cache(uint16_t *key_cache, uint16_t *value_cache, const uint16_t *key, const uint16_t *value,
                       const int64_t *slot_mapping, int num_tokens, int num_kv_heads, int head_dim,
                       int block_size);

/* Infer-engine/cuda/paged_kv.cu:440-519 (kernels :99-422): paged GQA decode attention, one query
 * token per sequence, scale 1/sqrt(head_dim), seq_lens counts the tokens to attend to.
 * head_dim must be 128 and q heads a multiple (<= 8x) of kv heads, otherwise exit(1). */
void paged_decode_attention(uint16_t *out, const uint16_t *query, const uint16_t *key_cache,
                            const uint16_t *value_cache, const int *block_tables, const int *seq_lens,
                            int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                            int max_blocks_per_seq);

/* Infer-engine/include/cuda_kernels.h:164-170, Infer-engine/cuda/decoder.cu:1849-2173.
 * ws: WeightStore*, cfg: ModelConfig*, pool: KVPool*, bts: BlockTable[num_seqs]; handle and
 * dequant_buf are ignored.  Arithmetic per projection as in the reference: without
 * GLMASR_USE_CUTLASS_NVFP4 every FP4 projection is W4A16 (fp4_linear); with it q, o and down are W4A4
 * (nvfp4_linear) while the same-input pairs k|v and gate|up stay W4A16 (the reference's fused pair,
 * Infer-engine/cuda/decoder.cu:923-978, always dequantises), unless a pair carries a pre_quant_scale and is
 * therefore run one projection at a time.  GLMASR_NVFP4_PAIRS=1 (additive, not in the reference) runs the
 * pairs in W4A4 too. */
void decoder_decode_step_batched(void *handle, const void *ws, uint16_t **query_ptrs, void *pool, void *bts,
                                 int *d_seq_lens, int *h_seq_lens, int num_seqs, int *seq_indices,
                                 uint16_t *dequant_buf, const void *cfg);

/* Infer-engine/include/safetensors.h:6-7, Infer-engine/src/safetensors.c:57-193.  ws: WeightStore*.
 * safetensors_load fills the store with every tensor of the file whose dtype the engine knows (BF16, F32,
 * F16, U8, F8_E4M3), in header order: name, dtype tag, shape (<= 4 dims), byte count, device pointer; at most
 * 2048 entries; "__metadata__" and other dtypes are skipped.  Returns 0, or -1 (message on stderr) when the
 * file cannot be read or device memory runs out.  Unlike the reference, which allocates every tensor on its
 * own, the tensors of one file live at 256-byte aligned offsets of ONE device allocation, filled through two
 * pinned staging buffers in 64 MiB copies; so a store filled here must be released with this library's
 * safetensors_free (which also accepts stores whose tensors were allocated one by one), and single tensors
 * must not be passed to cudaFree. */
int safetensors_load(const char *path, void *ws);
void safetensors_free(void *ws);

/* Infer-engine/include/cuda_kernels.h:12-14, Infer-engine/cuda/mel.cu:253-294.  Log-mel features of one 16 kHz
 * window: pcm float [num_samples] and mel_filters_transposed float [201, 128] on the device; mel_out bf16
 * [128, n_frames] (mel-major) with n_frames = clamp(ceil(num_samples / 160), 1, 3000) returned in *out_frames
 * (host).  Periodic Hann window, 400-point DFT, power, filterbank, log10(p + 1e-10), clamp to (maximum - 8),
 * (v + 4) / 4.  The maximum is taken over the WHOLE window; the reference's second reduction pass
 * (mel.cu:195-206) lets only one warp's share through, which is treated as a defect and not reproduced. */
void mel_spectrogram(const float *pcm, int num_samples, const float *mel_filters_transposed, uint16_t *mel_out,
                     int *out_frames);
/* Infer-engine/cuda/mel.cu:86-109.  Nothing to release here beyond what glmasr_fp4_cleanup frees. */
void mel_cleanup(void);

/* ---- audio encoder (bf16) ---- */

/* Infer-engine/include/cuda_kernels.h:26-28, Infer-engine/cuda/kernels.cu:299-356.  out = bf16(((x - mean) / sqrt(var
 * + eps)) * weight + bias) per row, the reference's summation order; bias may be NULL; out may alias x. */
void layernorm(uint16_t *out, const uint16_t *x, const uint16_t *weight, const uint16_t *bias, float eps, int rows, int dim);
/* Infer-engine/include/cuda_kernels.h:30, Infer-engine/cuda/kernels.cu:364-381: tanh-GELU in place. */
void gelu_inplace(uint16_t *x, int n);
/* Infer-engine/include/cuda_kernels.h:34-36, Infer-engine/cuda/kernels.cu:427-484: the encoder's partial rotary
 * embedding of q and k [seq_len, num_heads, head_dim] in place (rot_dim = head_dim * partial_factor = 32 only). */
void rope_encoder(uint16_t *q, uint16_t *k, int seq_len, int num_heads, int head_dim, float partial_factor);
/* Infer-engine/include/cuda_kernels.h:47-51, Infer-engine/cuda/kernels.cu:763-795: out = bf16(bf16(a + bias[col]) + b). */
void residual_add_bias(uint16_t *out, const uint16_t *a, const uint16_t *b, const uint16_t *bias, int M, int N);
/* Infer-engine/include/cuda_kernels.h:53-54, Infer-engine/cuda/kernels.cu:801-826: [seq, dim] -> [seq / 4, 4 dim]. */
void concat_4frames(uint16_t *out, const uint16_t *in, int seq_len, int dim);
/* Infer-engine/include/cuda_kernels.h:56-59, Infer-engine/cuda/kernels.cu:1561-1629: input [in_ch, seq_len], weight
 * [out_ch, in_ch, kernel_size], out [out_ch, out_len] bf16, bias per output channel.  One GEMM with K = kernel_size
 * * in_ch (the reference: one accumulating GEMM per tap, partial sums rounded to bf16 in between). */
void conv1d_forward(uint16_t *out, const uint16_t *input, const uint16_t *weight, const uint16_t *bias, int in_ch, int out_ch,
                    int seq_len, int kernel_size, int stride, int padding);
/* Infer-engine/include/cuda_kernels.h:61-62, Infer-engine/cuda/kernels.cu:1631-1660: out[c, r] = in[r, c]. */
void transpose_2d(uint16_t *out, const uint16_t *in, int rows, int cols);
/* Infer-engine/include/cuda_kernels.h:71-75, Infer-engine/cuda/kernels.cu:1211-1250: bf16 linear + bias + tanh-GELU
 * in one tcgen05 GEMM (K % 64 == 0, 16-byte aligned pointers; otherwise exit(1)). */
void bf16_linear_gelu(void *handle, uint16_t *out, const uint16_t *x, const uint16_t *w, const uint16_t *bias, int M, int N,
                      int K);
/* Infer-engine/include/cuda_kernels.h:101-111, Infer-engine/cuda/encoder.cu:1974-2188, 2427-2462: the encoder stack
 * (enc_layers pre-norm layers: LayerNorm, q|k|v, partial rotary embedding, non-causal attention over the sequence's
 * own frames, o + bias + residual, LayerNorm, fc1 + bias + GELU, fc2 + bias + residual; final LayerNorm) in place on
 * hidden [total_rows, enc_hidden]; sequence s owns rows [seq_offsets[s], + seq_lens[s]) (host arrays).  ws:
 * WeightStore*, cfg: ModelConfig* (enc_head_dim must be 64); handle is unused. */
void encoder_forward(void *handle, const void *ws, uint16_t *hidden, int seq_len, const void *cfg);
void encoder_forward_packed(void *handle, const void *ws, uint16_t *hidden, int total_rows, int num_seqs, const int *seq_lens,
                            const int *seq_offsets, const void *cfg);
/* Infer-engine/include/cuda_kernels.h:121, Infer-engine/cuda/encoder.cu:2421-2423: drop what the encoder cached
 * about a WeightStore (call before freeing the store). */
void encoder_cleanup(void);

/* ======================= 2. additive entry points ======================= */

/* The whole audio path after the log-mel features for a batch of windows (Infer-engine/src/engine.c:1111-1160,
 * 1561-1601): convolution front end (k 3 stride 1, k 3 stride 2, tanh-GELU after each), encoder stack, projector
 * (four frames concatenated, linear + GELU, linear).  mel: TIME-MAJOR features as glmasr_mel_spectrogram_batched
 * (time_major = 1) writes them, window i at mel + i * mel_stride holding [n_frames_host[i], num_mel_bins]; out:
 * window i's audio embeddings at out + i * out_stride as [tokens_i, dec_hidden], tokens_i = ((n_i + 1) / 2) / 4 =
 * out_tokens_host[i] (may be NULL).  Returns 0 or -1. */
int glmasr_audio_encode_batched(const void *ws, const void *cfg, const uint16_t *mel, long long mel_stride,
                                const int *n_frames_host, int num_windows, uint16_t *out, long long out_stride,
                                int *out_tokens_host);

/* mel_spectrogram for a batch of windows in two launches: window i reads pcm + i * pcm_stride (floats,
 * num_samples_host[i] of them) and writes mel_out + i * out_stride (bf16 elements) as [128, n_frames_i]
 * (time_major = 0, the reference's layout) or [n_frames_i, 128] (time_major = 1, rows = frames: what the
 * encoder's convolution-as-GEMM reads); out_frames_host[i] = n_frames_i (may be NULL).  num_windows <= 4096.
 * Returns 0 or -1. */
int glmasr_mel_spectrogram_batched(const float *pcm, long long pcm_stride, const int *num_samples_host, int num_windows,
                                   const float *mel_filters_transposed, uint16_t *mel_out, long long out_stride,
                                   int time_major, int *out_frames_host);

/* The header pass of safetensors_load on its own: names, dtype tags, shapes and byte counts exactly as the load
 * would set them, with every tensor's OFFSET inside the one device allocation stored in `data`, and that
 * allocation's size in *arena_bytes.  No device memory is touched and no CUDA call is made.  The names are
 * malloc'd; release them with glmasr_safetensors_release_index.  Returns 0 or -1. */
int glmasr_safetensors_inspect(const char *path, void *ws, size_t *arena_bytes);
void glmasr_safetensors_release_index(void *ws);

/* Batched variable-length prefill, in place on hidden [total_tokens, dec_hidden]
 * (Infer-engine/cuda/decoder.cu:1219-1557; include/cuda_kernels.h): sequence s owns rows
 * [seq_offsets[s], seq_offsets[s]+seq_lens[s]) (host arrays) and the blocks of bts[s]; writes every
 * layer's K / V rows to the paged pool.  ws / pool / bts / cfg are the engine's WeightStore, KVPool,
 * BlockTable[] and ModelConfig (layouts in glmasr_engine_types.h); handle and dequant_buf are unused. */
void decoder_prefill_paged_batched(void *handle, const void *ws, uint16_t *hidden, int total_tokens, int num_seqs,
                                   const int *seq_lens, const int *seq_offsets, void *pool, void *bts,
                                   uint16_t *dequant_buf, const void *cfg);
/* The attention plug-in's entry points (Infer-engine/cuda/flash_fwd_vllm.h:21-30) served by this library:
 * variable-length GQA self-attention, head_dim 128, q / k / v rows of sequence s at
 * [d_cu_seqlens[s], d_cu_seqlens[s+1]) with the given row strides (elements), out dense
 * [total_seqlen, q_heads*head_dim].  Returns 1 on success, 0 otherwise, like the plug-in.  With 16-byte aligned
 * pointers and row strides that are multiples of 8 elements it runs on the tcgen05 tensor cores (TMA-staged tiles,
 * accumulators in tensor memory; total_seqlen must cover every row the table points at); other layouts run on a
 * warp-level MMA kernel with the same results up to rounding. */
int flash_fwd_vllm_gqa_available(void);
int flash_fwd_vllm_gqa_launch(void *q, void *k, void *v, void *out, int total_seqlen, int max_seqlen, int q_heads,
                              int kv_heads, int head_dim, int q_row_stride, int k_row_stride, int v_row_stride,
                              int num_seqs, int *d_cu_seqlens, int is_causal);
/* Rotate-half RoPE (theta 10000) of one new token per sequence, in place on [num_seqs, n_heads*head_dim],
 * position = positions[seq] (the reference's rope_batched_single_token_kernel,
 * Infer-engine/cuda/decoder.cu:605-632, which has no host entry point of its own). */
void glmasr_rope_single_token(uint16_t *tensor, const int *positions, int num_seqs, int n_heads, int head_dim);
/* The three launches between the q|k|v projection and attention of a decode step as one: RoPE on the q
 * heads (columns [0, q_heads*head_dim)) and the k heads (at k_col) of every sequence's new-token row of
 * qkv [num_seqs, ld], in place, and the K / V rows written to slot_mapping[seq] of the paged cache
 * (Infer-engine/cuda/decoder.cu:605-632 twice + cuda/paged_kv.cu:70-97; same bytes).  Returns -1 for an
 * unsupported layout (ld, v_col, kv_heads*head_dim multiples of 8; 16-byte aligned pointers). */
int glmasr_rope_qk_cache(uint16_t *qkv, int ld, int k_col, int v_col, const int *positions,
                         const int64_t *slot_mapping, uint16_t *key_cache, uint16_t *value_cache, int num_seqs,
                         int q_heads, int kv_heads, int head_dim);
/* rmsnorm (Infer-engine/cuda/kernels.cu rmsnorm_kernel) followed by the activation quantiser
 * (cuda/nvfp4_cutlass.cu:35-87) in one launch: packed_out [rows, dim/2] e2m1 bytes and the scales in the
 * 128x4-tiled layout (ceil(rows/128) * dim/64 * 512 bytes), the same bytes as rmsnorm then
 * glmasr_quantize_bf16_to_fp4 + glmasr_swizzle_rowwise_scales.  dim % 64 == 0.  Returns -1 otherwise. */
int glmasr_rmsnorm_quant(uint8_t *packed_out, uint8_t *tiled_scale_out, const uint16_t *x, const uint16_t *weight,
                         float eps, float input_scale, int rows, int dim);
/* Forget the per-layer pointer table built from a WeightStore (call before freeing the store).  Also drops
 * the cached values of GLMASR_USE_CUTLASS_NVFP4 and GLMASR_NVFP4_PAIRS: they are read again on next use. */
void glmasr_decoder_forget_weights(void);

#define GLMASR_MODE_W4A4  0   /* nvfp4_linear arithmetic */
#define GLMASR_MODE_W4A16 1   /* fp4_linear arithmetic   */

#define GLMASR_EPI_STORE     0  /* out = bf16(acc*alpha)                                         */
#define GLMASR_EPI_SILU_GATE 1  /* weights = {gate, up}: out[M,N] = silu_mul_split_packed fused   */
#define GLMASR_EPI_RESIDUAL  2  /* one weight: out = residual_add(bf16(acc*alpha), residual) fused */

typedef struct {
    const uint8_t *w_packed;   /* [N, K/2] */
    const uint8_t *w_scales;   /* [N, K/16] */
    float w_global_scale;      /* the tensor's weight_scale_2 */
    int N;
} glmasr_fp4_weight;

/* Up to three FP4 weights that share one input (q|k|v, gate|up) in ONE GEMM, each with its
 * own per-tensor scale, replacing linear_proj + linear_proj_pair_same_input
 * (Infer-engine/cuda/decoder.cu:861-978) and, through the epilogue modes, the separate
 * silu_mul_split_packed / residual_add passes.  Output columns are the weights'
 * concatenated rows (EPI_STORE, EPI_RESIDUAL) or N of the gate (EPI_SILU_GATE).
 * x has row pitch ldx elements, out and residual row pitch ldo.  input_scale is used by
 * W4A4 only.  prequant_scratch ([M,K] bf16) is needed for W4A16 with pre_quant_scale.
 * Returns 0, or -1 on invalid arguments. */
int glmasr_fp4_linear_fused(int mode, uint16_t *out, int ldo, const uint16_t *x, int ldx,
                            const glmasr_fp4_weight *weights, int num_weights, float input_scale,
                            const uint16_t *pre_quant_scale, uint16_t *prequant_scratch,
                            int epilogue, const uint16_t *residual, int M, int K);

/* W4A4 linear on an activation that is ALREADY quantised: xq = e2m1 bytes [M, K/2], xq_sf = its e4m3 block
 * scales in the 128x4-tiled layout, exactly as glmasr_rmsnorm_quant (or a quantising epilogue of this library)
 * writes them; up to three same-input weight tensors side by side as in glmasr_fp4_linear_fused.  No reference
 * counterpart: the reference re-quantises the bf16 activation inside every nvfp4_linear call
 * (Infer-engine/cuda/nvfp4_cutlass.cu:155-166).
 *   resident = 0  the library's regular GEMM kernels.
 *   resident = 1  one phase of the co-resident layer-tail kernel the decode step uses at M <= 256 (every SM takes a
 *                 share of the output columns).  GLMASR_EPI_RESIDUAL then adds in place (residual == out) and
 *                 GLMASR_EPI_SILU_GATE writes only the quantised product (q_out / q_out_sf, required).
 * q_out / q_out_sf / q_out_input_scale (GLMASR_EPI_SILU_GATE): the SiLU-gate product quantised for a following
 * W4A4 GEMM, e2m1 bytes [M, N/2] + tiled scales.  Both settings produce the same bytes.  Returns 0, or -1 when the
 * shape is not covered (K % 256, N % 32, M > 256 for resident = 1, missing scales). */
int glmasr_fp4_linear_quantized(int resident, uint16_t *out, int ldo, const uint8_t *xq, const uint8_t *xq_sf,
                                const glmasr_fp4_weight *weights, int num_weights, float input_scale, int epilogue,
                                const uint16_t *residual, int M, int K, uint8_t *q_out, uint8_t *q_out_sf,
                                float q_out_input_scale);

/* One-time re-tiling of a weight's e4m3 scales into the 128x4 tile order the tensor core
 * reads (what Infer-engine/cuda/nvfp4_cutlass.cu:184-188 redoes on every call; the slot of
 * the declared-but-undefined swizzle_weight_scale, Infer-engine/cuda/kernels.cuh:24).
 * Cached by device pointer; nvfp4_linear / glmasr_fp4_linear_fused call it on first use. */
int glmasr_fp4_prepack(const uint8_t *w_scales, int N, int K);
/* Drop cached state for a weight whose memory is about to be freed (safetensors_free). */
void glmasr_fp4_forget(const void *w_scales);

/* The reference activation quantiser as a stand-alone call
 * (Infer-engine/cuda/nvfp4_cutlass.cu:35-87): packed_out [M,K/2], scale_out [M,K/16] row-major. */
int glmasr_quantize_bf16_to_fp4(uint8_t *packed_out, uint8_t *scale_out, const uint16_t *x,
                                const uint16_t *pre_quant_scale, float input_scale, int M, int K);
/* Infer-engine/cuda/nvfp4_cutlass.cu:89-111 into dst of ceil128(rows)*ceil4(cols) bytes (zero-filled here). */
int glmasr_swizzle_rowwise_scales(uint8_t *dst, const uint8_t *src, int rows, int cols);

/* Row arg-max over bf16 logits [rows, vocab] with the reference tie-break
 * (Infer-engine/cuda/kernels.cu:1387-1426); out_tokens is a device array. */
int glmasr_argmax_rows(const uint16_t *logits, int *out_tokens, int rows, int vocab);

/* The FP4 projections of one decoder layer in the order the reference drivers call them
 * (Infer-engine/cuda/decoder.cu:1375-1391, 1443-1533): q|k|v, o + residual, gate|up with
 * SiLU-gate, down + residual.  Attention itself is not part of this path: the q slice of the
 * fused q|k|v output stands in for the attention output.  hidden_in/out are [M, hidden]. */
typedef struct {
    glmasr_fp4_weight q, k, v, o, gate, up, down;
    float in_qkv, in_o, in_gate_up, in_down;   /* per-projection input_scale (W4A4) */
    int hidden, ffn;
} glmasr_layer_weights;
int glmasr_fp4_layer_proj(int mode, uint16_t *hidden_out, const uint16_t *hidden_in,
                          const glmasr_layer_weights *lw, int M);
/* Same, with HOST (preferably pinned) hidden_in_host / hidden_out_host: copies in, runs,
 * copies out and synchronises -- the end-to-end call the benchmark times. */
int glmasr_fp4_layer_proj_host(int mode, uint16_t *hidden_out_host, const uint16_t *hidden_in_host,
                               const glmasr_layer_weights *lw, int M);

/* The part of a decoder layer that follows attention, at decode batch sizes (M <= 256), as ONE launch of a
 * co-resident kernel (one CTA per SM, phases separated by a grid-wide counter; no reference counterpart -- the
 * reference runs these as ~10 launches, Infer-engine/cuda/decoder.cu:2050-2160):
 *     o projection + residual | RMSNorm + activation quantiser | gate|up + SiLU-gate + quantiser | down + residual
 * and, when `next` is given, | RMSNorm + quantiser | q|k|v of the FOLLOWING layer into next_qkv [M, H + 2 KV].
 * Every projection is W4A4.  hidden [M, H] is updated in place.  attn_q / attn_sf: the attention output already
 * quantised with input scale lw->in_o (e2m1 bytes [M, H/2] + 128x4-tiled scales).  norm_q / norm_sf ([M, H/2],
 * tiled scales for K = H) and act_q / act_sf ([M, F/2], K = F) are scratch the phases hand over through; after the
 * call they hold the last quantised norm output and the quantised SiLU-gate product.  max_phases > 0 stops the
 * program after that many phases (for tests).  Same bytes as glmasr_fp4_linear_quantized / glmasr_rmsnorm_quant
 * run one after the other.  Returns 0, or -1 when a shape is not covered (then nothing was launched). */
int glmasr_decode_layer_tail(uint16_t *hidden, int M, const uint8_t *attn_q, const uint8_t *attn_sf,
                             const glmasr_layer_weights *lw, const uint16_t *post_attention_norm,
                             const glmasr_layer_weights *next, const uint16_t *next_input_norm, uint16_t *next_qkv,
                             uint8_t *norm_q, uint8_t *norm_sf, uint8_t *act_q, uint8_t *act_sf, int max_phases);

/* W4A4 linear (nvfp4_linear arithmetic, no pre_quant_scale, no bias) for callers that must not
 * allocate device memory.  No counterpart in the reference.  The engine sizes its paged-KV pool
 * from whatever device memory is still free after warm-up, so a decode-loop call that grows a
 * workspace later can fail or stall the loop on cudaMalloc's implicit synchronisation; this
 * entry point instead keeps its temporaries (quantised activations, their scales, the re-tiled
 * weight scales) in a fixed 4.25 MiB array inside the library image, resident on every GPU that
 * loads the library until the process exits.
 * Limits: M <= 512, K <= 8192, K % 256 == 0, N % 8 == 0, ceil128(N) * K <= 32 Mi, 16-byte aligned
 * pointers; anything else returns -1 with a message on stderr (use nvfp4_linear then).
 * The first call on each device looks up the array's device address and opts the kernels in to
 * large shared memory, and it may be the call that makes the CUDA runtime load the module holding the
 * array and the kernels onto that device: make it once per device during warm-up -- before the KV pool
 * takes the remaining memory and before any stream capture begins.
 * A bounded wait that runs out inside these kernels is reported by glmasr_fp4_status() like any other
 * (through a status word that also lives in the library image).
 * All calls share the one array and it keeps the previous call's contents (the part that must
 * start at zero is cleared on every call), so two calls whose GPU work overlaps -- different
 * streams, different host threads -- race; issue them in stream order. */
int glmasr_nvfp4_linear_noalloc(uint16_t *out, const uint16_t *x, const uint8_t *w_packed,
                                const uint8_t *w_scales, float input_scale, float w_global_scale,
                                int M, int N, int K);

/* Synchronise and return the first device-side status code recorded since the last call
 * (0 = none; 1..6 = a bounded wait inside a kernel ran out, 7 = a layout a kernel cannot work with),
 * then clear it. */
int glmasr_fp4_status(void);
/* Number of kernels this library has launched since load (for launch accounting). */
long long glmasr_launch_count(void);
/* Per-launch timing of the tensor-core GEMM kernel with CUDA events recorded on the launching
 * stream.  While enabled, every GEMM launch is bracketed; glmasr_profile_read synchronises,
 * returns up to max_entries (duration ms, algorithmic flops, algorithmic bytes) triples in
 * launch order and clears the list.  Off by default. */
void glmasr_profile_enable(int on);
int glmasr_profile_read(int max_entries, double *ms, double *flops, double *bytes);
/* Route all launches to the given cudaStream_t (NULL = legacy default stream). */
void glmasr_set_stream(void *cuda_stream);
/* Free every private workspace / cache (decoder_cleanup_all / lm_head_cleanup analogue). */
void glmasr_fp4_cleanup(void);

#ifdef __cplusplus
}
#endif
#endif /* GLMASR_FP4_H */
