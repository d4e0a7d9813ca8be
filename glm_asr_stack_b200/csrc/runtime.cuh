// Library-private runtime state shared by the translation units: the stream every launch
// goes to (legacy default stream unless the host sets another one), the device status word
// the kernels report bounded-wait failures through, and error helpers that follow the
// reference's conventions (Infer-engine/include/types.h:182-199: print and exit(1) for the
// void entry points; nvfp4_linear instead returns -1, Infer-engine/cuda/nvfp4_cutlass.cu:262-269).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

namespace glmasr {

cudaStream_t current_stream();
int *device_status_word();          // device pointer, 4 ints, zero-initialised; allocated on first use
void *workspace(size_t bytes);      // grow-only private device workspace (slot 0)
void *workspace_slot(int slot, size_t bytes);
// Slots owned outside api.cu / decoder_step.cu (those two number their own, 0..31).
enum : int { WS_ATTN_VT = 32, WS_ATTN_VT_COL = 33, WS_ATTN_DEBUG = 34 };
void free_all_private_state();
void tail_forget_scales(const void *w_scales);   // decode_tail.cu: per-CTA re-tiled weight scales (nullptr: all)
void encoder_forget_all();         // encoder.cu: per-store weight table, re-packed convolution weights, rotary table
void note_launches(int n);          // launch accounting for kernels started outside api.cu
size_t tiled_scale_bytes(int rows, int K);   // bytes of the 128x4-tiled scale layout for [rows, K]
// Cached TMA descriptor of a row-major bf16 matrix [rows, inner] (row pitch in bytes, a multiple of 16; base
// 16-byte aligned) cut into box_rows x box_inner boxes with the 128-byte swizzle.  False if it cannot be encoded.
bool make_bf16_tmap_sw128(CUtensorMap *tm, const void *base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                          uint32_t box_inner, uint32_t box_rows);

// Same for a byte matrix (packed e2m1 operands): inner = bytes per row.
bool make_u8_tmap_sw128(CUtensorMap *tm, const void *base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_inner, uint32_t box_rows);
// CUDA-event bracket around launches made outside api.cu; recorded only while profiling is enabled.
void profile_bracket_begin(double flops, double bytes);
void profile_bracket_end();

// Ask once for the largest shared-memory carve-out for `kernel`.  The GEMM kernels need almost all
// of an SM's shared memory; a small kernel launched between two of them with the default
// preference makes the SM switch its L1 / shared split back and forth, which costs microseconds per
// launch in a chain of 5-15 us kernels.  None of the glue kernels depends on L1 capacity.
#define GLMASR_PREFER_MAX_SMEM(kernel)                                                                     \
    do {                                                                                                   \
        static bool done_ = false;                                                                         \
        if (!done_) {                                                                                      \
            cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,                   \
                                 (int)cudaSharedmemCarveoutMaxShared);                                     \
            done_ = true;                                                                                  \
        }                                                                                                  \
    } while (0)

// ---- programmatic dependent launch -------------------------------------------------------------
// A chain of 5-40 us kernels on one stream pays a few microseconds per kernel boundary (launch
// latency, block scheduling, set-up code).  Kernels launched through launch_chained() may become
// resident while their predecessor is still draining: each of them calls pdl_launch_dependents()
// first thing and pdl_wait() before it touches global memory, and pdl_wait() returns only when
// every preceding kernel of the stream has completed and its writes are visible, so data
// dependencies are exactly those of an ordinary stream.  GLMASR_PDL=0 turns the attribute off.
bool pdl_enabled();

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

#define GLMASR_CUDA_CHECK(call)                                                              \
    do {                                                                                     \
        cudaError_t _e = (call);                                                             \
        if (_e != cudaSuccess) {                                                             \
            fprintf(stderr, "CUDA error [%s:%d]: %s\n", __FILE__, __LINE__, cudaGetErrorString(_e)); \
            exit(1);                                                                         \
        }                                                                                    \
    } while (0)

#define GLMASR_CHECK(cond, ...)                                         \
    do {                                                                \
        if (!(cond)) {                                                  \
            fprintf(stderr, "ERROR [%s:%d]: ", __FILE__, __LINE__);     \
            fprintf(stderr, __VA_ARGS__);                               \
            fprintf(stderr, "\n");                                      \
            exit(1);                                                    \
        }                                                               \
    } while (0)

}  // namespace glmasr
