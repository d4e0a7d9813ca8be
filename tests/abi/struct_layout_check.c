/* Compile-time proof that include/glmasr_engine_types.h lays its structures out exactly as the
 * engine's own headers do (Infer-engine/include/types.h:8-95, Infer-engine/include/kv_pool.h:27-56):
 * sizeof of every struct and offsetof of every field, as _Static_assert.  Compiling this file IS the
 * test (tests/test_abi.py runs gcc on it with -I<reference>/Infer-engine/include); nothing is linked
 * or executed.  Test infrastructure only. */
#include <stddef.h>

#include "types.h"    /* the reference's */
#include "kv_pool.h"  /* the reference's */
#include "glmasr_engine_types.h"

#define SAME_SIZE(ours, theirs) _Static_assert(sizeof(ours) == sizeof(theirs), "sizeof " #ours " != sizeof " #theirs)
#define SAME_FIELD(ours, theirs, f)                                                                  \
    _Static_assert(offsetof(ours, f) == offsetof(theirs, f), "offsetof " #ours "." #f " differs");   \
    _Static_assert(sizeof(((ours *)0)->f) == sizeof(((theirs *)0)->f), "sizeof " #ours "." #f " differs")

/* dtype tags and limits */
_Static_assert(GLMASR_DTYPE_FP32 == DTYPE_FP32 && GLMASR_DTYPE_BF16 == DTYPE_BF16 && GLMASR_DTYPE_FP16 == DTYPE_FP16 &&
                   GLMASR_DTYPE_UINT8 == DTYPE_UINT8 && GLMASR_DTYPE_FP8 == DTYPE_FP8,
               "dtype tags differ");
_Static_assert(GLMASR_MAX_DIMS == MAX_DIMS && GLMASR_MAX_WEIGHTS == MAX_WEIGHTS, "limits differ");

SAME_SIZE(glmasr_Tensor, Tensor);
SAME_FIELD(glmasr_Tensor, Tensor, data);
SAME_FIELD(glmasr_Tensor, Tensor, dtype);
SAME_FIELD(glmasr_Tensor, Tensor, ndim);
SAME_FIELD(glmasr_Tensor, Tensor, shape);
SAME_FIELD(glmasr_Tensor, Tensor, nbytes);

SAME_SIZE(glmasr_ModelConfig, ModelConfig);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, enc_hidden);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, enc_layers);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, enc_heads);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, enc_head_dim);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, enc_ffn);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, num_mel_bins);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, max_audio_frames);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, proj_mid);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, dec_hidden);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, dec_layers);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, dec_heads);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, dec_kv_heads);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, dec_head_dim);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, dec_ffn);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, vocab_size);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, max_position_embeddings);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, audio_token_id);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, eos_ids);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, pad_token_id);
SAME_FIELD(glmasr_ModelConfig, ModelConfig, max_new_tokens);

SAME_SIZE(glmasr_WeightStore, WeightStore);
SAME_FIELD(glmasr_WeightStore, WeightStore, names);
SAME_FIELD(glmasr_WeightStore, WeightStore, tensors);
SAME_FIELD(glmasr_WeightStore, WeightStore, count);

SAME_SIZE(glmasr_KVPool, KVPool);
SAME_FIELD(glmasr_KVPool, KVPool, k_cache);
SAME_FIELD(glmasr_KVPool, KVPool, v_cache);
SAME_FIELD(glmasr_KVPool, KVPool, d_block_tables);
SAME_FIELD(glmasr_KVPool, KVPool, max_seqs);
SAME_FIELD(glmasr_KVPool, KVPool, max_blocks_per_seq);
SAME_FIELD(glmasr_KVPool, KVPool, free_stack);
SAME_FIELD(glmasr_KVPool, KVPool, free_top);
SAME_FIELD(glmasr_KVPool, KVPool, num_blocks);
SAME_FIELD(glmasr_KVPool, KVPool, block_size);
SAME_FIELD(glmasr_KVPool, KVPool, num_layers);
SAME_FIELD(glmasr_KVPool, KVPool, kv_heads);
SAME_FIELD(glmasr_KVPool, KVPool, head_dim);
SAME_FIELD(glmasr_KVPool, KVPool, kv_head_stride);
SAME_FIELD(glmasr_KVPool, KVPool, block_stride);
SAME_FIELD(glmasr_KVPool, KVPool, layer_stride);
SAME_FIELD(glmasr_KVPool, KVPool, per_layer_bytes);

SAME_SIZE(glmasr_BlockTable, BlockTable);
SAME_FIELD(glmasr_BlockTable, BlockTable, d_table);
SAME_FIELD(glmasr_BlockTable, BlockTable, max_blocks);
SAME_FIELD(glmasr_BlockTable, BlockTable, num_blocks);
SAME_FIELD(glmasr_BlockTable, BlockTable, h_table);
SAME_FIELD(glmasr_BlockTable, BlockTable, seq_idx);

int glmasr_struct_layout_check(void) { return 0; }
