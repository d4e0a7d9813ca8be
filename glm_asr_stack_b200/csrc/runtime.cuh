// Library-private runtime state shared by the translation units: the stream every launch
// goes to (legacy default stream unless the host sets another one), the device status word
// the kernels report bounded-wait failures through, and error helpers that follow the
// reference's conventions (Infer-engine/include/types.h:182-199: print and exit(1) for the
// void entry points; nvfp4_linear instead returns -1, Infer-engine/cuda/nvfp4_cutlass.cu:262-269).
#pragma once
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

namespace glmasr {

cudaStream_t current_stream();
int *device_status_word();          // device pointer, 4 ints, zero-initialised; allocated on first use
void *workspace(size_t bytes);      // grow-only private device workspace (slot 0)
void *workspace_slot(int slot, size_t bytes);
void free_all_private_state();
void note_launches(int n);          // launch accounting for kernels started outside api.cu
size_t tiled_scale_bytes(int rows, int K);   // bytes of the 128x4-tiled scale layout for [rows, K]

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
