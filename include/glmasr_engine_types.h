/*
 * Layout-compatible declarations of the engine structures that cross the decoder entry points
 * (decoder_decode_step_batched and the paged-KV helpers).  A drop-in has to agree with the
 * engine on the byte layout of these structs, so field order and types follow
 *   Infer-engine/include/types.h:8-35   (dtype tags, Tensor)
 *   Infer-engine/include/types.h:37-72  (ModelConfig)
 *   Infer-engine/include/types.h:88-95  (WeightStore)
 *   Infer-engine/include/kv_pool.h:27-56 (KVPool, BlockTable)
 * exactly.  When building inside the engine tree, include the engine's own headers instead.
 */
#ifndef GLMASR_ENGINE_TYPES_H
#define GLMASR_ENGINE_TYPES_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLMASR_DTYPE_FP32  0
#define GLMASR_DTYPE_BF16  1
#define GLMASR_DTYPE_FP16  2
#define GLMASR_DTYPE_UINT8 3   /* packed FP4, two values per byte */
#define GLMASR_DTYPE_FP8   4   /* e4m3 block scales */

#define GLMASR_MAX_DIMS    4
#define GLMASR_MAX_WEIGHTS 2048

typedef struct {
    void   *data;                       /* device memory */
    int     dtype;
    int     ndim;
    int64_t shape[GLMASR_MAX_DIMS];
    size_t  nbytes;
} glmasr_Tensor;

typedef struct {
    int enc_hidden, enc_layers, enc_heads, enc_head_dim, enc_ffn, num_mel_bins, max_audio_frames;
    int proj_mid;
    int dec_hidden, dec_layers, dec_heads, dec_kv_heads, dec_head_dim, dec_ffn, vocab_size;
    int max_position_embeddings;
    int audio_token_id;
    int eos_ids[4];
    int pad_token_id;
    int max_new_tokens;
} glmasr_ModelConfig;

typedef struct {
    char         *names[GLMASR_MAX_WEIGHTS];
    glmasr_Tensor tensors[GLMASR_MAX_WEIGHTS];
    int           count;
} glmasr_WeightStore;

typedef struct {
    void  *k_cache;             /* [layers][num_blocks][block_size][kv_heads][head_dim] bf16 */
    void  *v_cache;
    int   *d_block_tables;      /* device [max_seqs, max_blocks_per_seq] int32 */
    int    max_seqs;
    int    max_blocks_per_seq;
    int   *free_stack;          /* host LIFO of free block ids */
    int    free_top;
    int    num_blocks;
    int    block_size;
    int    num_layers;
    int    kv_heads;
    int    head_dim;
    int    kv_head_stride;      /* kv_heads * head_dim */
    int    block_stride;        /* block_size * kv_head_stride */
    int    layer_stride;        /* num_blocks * block_stride (elements) */
    size_t per_layer_bytes;
} glmasr_KVPool;

typedef struct {
    int *d_table;               /* row of pool->d_block_tables */
    int  max_blocks;
    int  num_blocks;
    int *h_table;               /* host mirror */
    int  seq_idx;
} glmasr_BlockTable;

#ifdef __cplusplus
}
#endif
#endif /* GLMASR_ENGINE_TYPES_H */
