"""The window -> tokens flow (glm_asr_stack_b200/pipeline.py: log-mel, audio encoder, prompt assembly, batched prefill,
greedy decode in waves) on a small random model: shapes and ranges, run-to-run determinism, independence of a
wave from what ran before it (the KV pool and every workspace are reused), and the prompt-length arithmetic the
engine uses (Infer-engine/src/engine.c:576-607).  The numerics of every stage are covered by the stage's own tests."""
import numpy as np
import pytest

from glm_asr_stack_b200 import pipeline


def test_prompt_length_arithmetic():
    assert pipeline.feature_frames(480000) == 3000 and pipeline.feature_frames(1) == 1 and pipeline.feature_frames(0) == 1
    assert pipeline.feature_frames(10 ** 7) == 3000
    assert pipeline.audio_tokens(3000) == 375 and pipeline.audio_tokens(1) == 0 and pipeline.audio_tokens(8) == 1
    for f in (1, 7, 8, 9, 1001, 2993, 3000):
        p = pipeline.padded_feature_frames(f)
        assert f <= p <= 3000 and (((p + 1) // 2) % 4 == 0 or p == 3000)
    assert len(pipeline.PROMPT_HEAD) + len(pipeline.PROMPT_TAIL) == 19            # 8 specials + 11 instruction ids


@pytest.mark.gpu
def test_pipeline_waves_are_deterministic_and_independent():
    import torch

    from glm_asr_stack_b200 import ops, synth, workloads
    model = workloads.build_decoder(layers=2, hidden=256, ffn=512, heads=2, kv_heads=1, head_dim=128, vocab=59264)
    workloads.add_audio_tower(model.ws, model.cfg, layers=2, hidden=256, heads=4, head_dim=64, ffn=512, proj_mid=512)
    import os
    os.environ["GLMASR_USE_CUTLASS_NVFP4"] = "1"
    os.environ["GLMASR_NVFP4_PAIRS"] = "1"
    from glm_asr_stack_b200 import _lib
    _lib.load().glmasr_decoder_forget_weights()
    filt = synth.mel_filterbank()
    lens = [480000, 160000, 480000, 33333, 480000, 480000]
    pcm = torch.zeros((len(lens), pipeline.SAMPLES_PER_WINDOW), dtype=torch.float32).pin_memory()
    for i, n in enumerate(lens):
        pcm[i, :n] = pipeline.synthetic_window(i)[:n].cpu()
    pipe = pipeline.AsrPipeline(model, filt, max_seqs=4, max_batched_tokens=800, new_tokens=6)
    assert pipe.prefill_group == 2
    a = pipe.transcribe(pcm, lens).clone()
    assert ops.status() == 0
    assert a.shape == (6, 6) and a.dtype == torch.int32
    assert int(a.min()) >= 0 and int(a.max()) < 59264
    b = pipe.transcribe(pcm, lens).clone()
    assert torch.equal(a, b)                                   # same work, same kernels, same tokens
    # the second wave (windows 4, 5) on a pipeline that has not run the first: same tokens
    c = pipe.transcribe(pcm[4:6], lens[4:6]).clone()
    assert torch.equal(c, a[4:6])
    # windows are independent: different audio gives different tokens somewhere
    assert not torch.equal(a[0], a[2]) or not torch.equal(a[0], a[4])
    os.environ.pop("GLMASR_NVFP4_PAIRS", None)
    os.environ.pop("GLMASR_USE_CUTLASS_NVFP4", None)
    _lib.load().glmasr_decoder_forget_weights()
