// Log-mel front end (reference: mel_spectrogram, Infer-engine/cuda/mel.cu:111-294), batched over windows.
//
// Per 16 kHz window: n_frames = clamp(ceil(samples / 160), 1, 3000) frames of 400 samples centred on
// f * 160 (zero outside the signal), periodic Hann window, 400-point real DFT (bins 0..200), power, the
// 201 x 128 mel filterbank (given transposed, as the engine loads it), log10(p + 1e-10), clamp to
// (window maximum - 8), (v + 4) / 4, bf16.
//
// The reference runs five launches and a cuFFT call per window, one window at a time.  Here a whole batch
// of windows is two launches:
//   mel_power_kernel      grid (frame tiles, windows): a CTA stages the tile's samples in shared memory,
//                         applies the window, evaluates the DFT directly against a 400-entry twiddle table
//                         (thread = frequency bin, 8 frames per pass in registers; N = 400 is not a power of
//                         two and a tile's 32 x 201 outputs need only 5 M multiply-adds), then the power
//                         spectrum times the filterbank in the reference's summation order, log10, the fp32
//                         result to scratch and the tile's maximum to the window's maximum (atomic);
//   mel_normalize_kernel  clamp, affine map, bf16, written mel-major [128, n_frames] like the reference or
//                         time-major [n_frames, 128] (what the encoder's convolution-as-GEMM reads).
// The window maximum is the maximum over the WHOLE window.  The reference's second reduction pass
// (final_max_kernel, mel.cu:195-206) reduces inside each warp but lets thread 0 alone write, so it returns
// the maximum of one eighth of the block maxima; that is a defect, not a definition, and is not reproduced.
// fp32 throughout, like the reference; results agree with it to the rounding of a different DFT
// factorisation (compared within one bf16 unit in the tests).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../../include/glmasr_fp4.h"
#include "runtime.cuh"

namespace glmasr {

constexpr int kFft = 400, kHop = 160, kMels = 128, kBins = 201, kMaxFrames = 3000;
constexpr int kTileFrames = 32;                                    // frames per CTA
constexpr int kTileSamples = (kTileFrames - 1) * kHop + kFft;      // 5360
constexpr int kMelThreads = 256;

enum : int { WS_MEL_LOG = 35, WS_MEL_MAX = 36 };                   // private workspace slots of this file

struct MelSmem {
    float xw[kFft][kTileFrames];          // windowed frames, tap-major: 8 consecutive frames are two 16-byte loads
    float2 tw[kFft];                      // (cos, sin)(2 pi j / 400)
    float hann[kFft];
    float power[kTileFrames][kBins + 3];  // first the tile's raw samples (kTileSamples floats), then the power spectrum
    float red[kMelThreads / 32];
};
static_assert(kTileSamples <= kTileFrames * (kBins + 3), "the raw samples of a tile are staged in the power array");

__device__ __forceinline__ void atomic_max_float(float *addr, float v) {
    // the cell starts as 0xFFFFFFFF: below every float in both orders used here
    if (v >= 0.0f) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

__global__ void __launch_bounds__(kMelThreads) mel_power_kernel(const float *__restrict__ pcm, long long pcm_stride,
                                                                const int *__restrict__ num_samples,
                                                                const float *__restrict__ filters_t,
                                                                float *__restrict__ logmel, float *__restrict__ win_max) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    MelSmem &s = *reinterpret_cast<MelSmem *>(smem_raw);
    pdl_launch_dependents();
    pdl_wait();
    const int w = blockIdx.y, tid = threadIdx.x;
    const int ns = num_samples[w];
    int n_frames = (ns + kHop - 1) / kHop;
    n_frames = n_frames < 1 ? 1 : (n_frames > kMaxFrames ? kMaxFrames : n_frames);
    const int f0 = blockIdx.x * kTileFrames;
    if (f0 >= n_frames) return;
    const float *x = pcm + (size_t)w * (size_t)pcm_stride;

    // twiddles, the window, and the tile's samples (coalesced; zero outside the signal)
    float *raw = &s.power[0][0];
    const int s0 = f0 * kHop - kFft / 2;                 // first sample of the tile
    for (int j = tid; j < kFft; j += kMelThreads) {
        float sn, cs;
        sincospif((float)j * (2.0f / kFft), &sn, &cs);
        s.tw[j] = make_float2(cs, sn);
        // periodic Hann window as the reference evaluates it (mel.cu:118: the argument in double, cosf of its float)
        s.hann[j] = 0.5f * (1.0f - cosf((float)(2.0 * 3.14159265358979323846 * j / kFft)));
    }
    for (int i = tid; i < kTileSamples; i += kMelThreads) {
        const int idx = s0 + i;
        raw[i] = (idx >= 0 && idx < ns) ? x[idx] : 0.0f;
    }
    __syncthreads();
    for (int i = tid; i < kFft * kTileFrames; i += kMelThreads) {
        const int t = i / kTileFrames, f = i - t * kTileFrames;
        s.xw[t][f] = (f0 + f < n_frames) ? raw[f * kHop + t] * s.hann[t] : 0.0f;
    }
    __syncthreads();

    // DFT: thread = bin k, eight frames per pass
    if (tid < kBins) {
        const int k = tid;
#pragma unroll 1
        for (int fg = 0; fg < kTileFrames; fg += 8) {
            float re[8], im[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) re[i] = im[i] = 0.0f;
            int j = 0;                                   // (k * t) mod 400
#pragma unroll 4
            for (int t = 0; t < kFft; ++t) {
                const float2 c = s.tw[j];
                const float4 a = *reinterpret_cast<const float4 *>(&s.xw[t][fg]);
                const float4 b = *reinterpret_cast<const float4 *>(&s.xw[t][fg + 4]);
                // the sign of the imaginary part does not matter for the power
#define GLMASR_MEL_ACC(i, xval) re[i] = fmaf(xval, c.x, re[i]), im[i] = fmaf(xval, c.y, im[i])
                GLMASR_MEL_ACC(0, a.x); GLMASR_MEL_ACC(1, a.y); GLMASR_MEL_ACC(2, a.z); GLMASR_MEL_ACC(3, a.w);
                GLMASR_MEL_ACC(4, b.x); GLMASR_MEL_ACC(5, b.y); GLMASR_MEL_ACC(6, b.z); GLMASR_MEL_ACC(7, b.w);
#undef GLMASR_MEL_ACC
                j += k;
                if (j >= kFft) j -= kFft;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) s.power[fg + i][k] = re[i] * re[i] + im[i] * im[i];
        }
    }
    __syncthreads();

    // filterbank, log10, tile maximum: thread = mel bin m (two frame phases)
    const int m = tid & (kMels - 1), phase = tid >> 7;
    float tmax = -FLT_MAX;
    for (int f = phase; f < kTileFrames && f0 + f < n_frames; f += kMelThreads / kMels) {
        float p = 0.0f;
#pragma unroll 4
        for (int k = 0; k < kBins; ++k) p += s.power[f][k] * filters_t[k * kMels + m];      // mel.cu:141-149
        const float v = log10f(p + 1e-10f);
        logmel[((size_t)w * kMaxFrames + (size_t)(f0 + f)) * kMels + m] = v;
        tmax = fmaxf(tmax, v);
    }
    for (int off = 16; off > 0; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xFFFFFFFFu, tmax, off));
    if ((tid & 31) == 0) s.red[tid >> 5] = tmax;
    __syncthreads();
    if (tid == 0) {
        float v = s.red[0];
        for (int i = 1; i < kMelThreads / 32; ++i) v = fmaxf(v, s.red[i]);
        if (v > -FLT_MAX) atomic_max_float(win_max + w, v);
    }
}

// out = bf16((max(v, vmax - 8) + 4) / 4)   (mel.cu:217-233).  grid (frame tiles of 32, windows), block (32, 8).
__global__ void mel_normalize_kernel(const float *__restrict__ logmel, const float *__restrict__ win_max,
                                     const int *__restrict__ num_samples, __nv_bfloat16 *__restrict__ out,
                                     long long out_stride, int time_major) {
    __shared__ float tile[32][kMels + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int w = blockIdx.y;
    const int ns = num_samples[w];
    int n_frames = (ns + kHop - 1) / kHop;
    n_frames = n_frames < 1 ? 1 : (n_frames > kMaxFrames ? kMaxFrames : n_frames);
    const int f0 = blockIdx.x * 32;
    if (f0 >= n_frames) return;
    const float floor_v = win_max[w] - 8.0f;
    __nv_bfloat16 *o = out + (size_t)w * (size_t)out_stride;
    const int tx = threadIdx.x, ty = threadIdx.y;
    for (int f = ty; f < 32; f += 8) {
        if (f0 + f >= n_frames) break;
        const float *src = logmel + ((size_t)w * kMaxFrames + (size_t)(f0 + f)) * kMels;
        for (int m = tx; m < kMels; m += 32) {
            const float v = (fmaxf(src[m], floor_v) + 4.0f) / 4.0f;
            if (time_major) o[(size_t)(f0 + f) * kMels + m] = __float2bfloat16(v);
            else tile[f][m] = v;
        }
    }
    if (time_major) return;
    __syncthreads();
    // mel-major [128, n_frames]: consecutive threads write consecutive frames of one mel row
    for (int m = ty; m < kMels; m += 8)
        if (f0 + tx < n_frames) o[(size_t)m * n_frames + f0 + tx] = __float2bfloat16(tile[tx][m]);
}

static int g_mel_smem_ready = 0;

// d_num_samples: device array [num_windows].  Returns false on a bad argument.
bool launch_mel_batched(const float *pcm, long long pcm_stride, const int *d_num_samples, int num_windows, int max_frames,
                        const float *filters_t, __nv_bfloat16 *out, long long out_stride, int time_major, cudaStream_t st) {
    if (num_windows <= 0) return true;
    if (pcm == nullptr || d_num_samples == nullptr || filters_t == nullptr || out == nullptr) return false;
    if (!g_mel_smem_ready) {
        if (cudaFuncSetAttribute(mel_power_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(MelSmem)) != cudaSuccess)
            return false;
        g_mel_smem_ready = 1;
    }
    float *logmel = (float *)workspace_slot(WS_MEL_LOG, (size_t)num_windows * kMaxFrames * kMels * sizeof(float));
    float *win_max = (float *)workspace_slot(WS_MEL_MAX, (size_t)num_windows * sizeof(float));
    if (cudaMemsetAsync(win_max, 0xFF, (size_t)num_windows * sizeof(float), st) != cudaSuccess) return false;
    const int tiles = (max_frames + kTileFrames - 1) / kTileFrames;
    // only the two launches' own results decide: an error some earlier call of the process left behind is not ours
    const cudaError_t e1 = launch_chained(mel_power_kernel, dim3(tiles, num_windows), dim3(kMelThreads), sizeof(MelSmem), st, pcm,
                                          pcm_stride, d_num_samples, filters_t, logmel, win_max);
    const cudaError_t e2 = launch_chained(mel_normalize_kernel, dim3((max_frames + 31) / 32, num_windows), dim3(32, 8), (size_t)0, st,
                                          (const float *)logmel, (const float *)win_max, d_num_samples, out, out_stride, time_major);
    note_launches(2);
    return e1 == cudaSuccess && e2 == cudaSuccess;
}

static int frames_for(int ns) {
    int n = (ns + kHop - 1) / kHop;
    return n < 1 ? 1 : (n > kMaxFrames ? kMaxFrames : n);
}

}  // namespace glmasr

using namespace glmasr;

enum : int { WS_MEL_NS = 37 };

// Infer-engine/include/cuda_kernels.h:12-14, Infer-engine/cuda/mel.cu:253-294: one window, output mel-major
// [128, n_frames] bf16, *out_frames (host) = n_frames.
extern "C" void mel_spectrogram(const float *pcm, int num_samples, const float *mel_filters_transposed, uint16_t *mel_out,
                                int *out_frames) {
    cudaStream_t st = current_stream();
    int *d_ns = (int *)workspace_slot(WS_MEL_NS, 4096 * sizeof(int));
    GLMASR_CUDA_CHECK(cudaMemcpyAsync(d_ns, &num_samples, sizeof(int), cudaMemcpyHostToDevice, st));
    const int n = frames_for(num_samples);
    if (out_frames != nullptr) *out_frames = n;
    // an empty clip has no samples to point at: nothing is read from pcm then, any valid pointer will do
    if (pcm == nullptr && num_samples <= 0) pcm = mel_filters_transposed;
    GLMASR_CHECK(launch_mel_batched(pcm, 0, d_ns, 1, n, mel_filters_transposed, (__nv_bfloat16 *)mel_out, 0, 0, st),
                 "mel_spectrogram: bad arguments (pcm %p, %d samples, filters %p, out %p)", (const void *)pcm, num_samples,
                 (const void *)mel_filters_transposed, (void *)mel_out);
}

// Infer-engine/cuda/mel.cu:86-109: the reference frees its FFT plan and buffers; here the buffers are private
// workspace slots released by glmasr_fp4_cleanup, so there is nothing to do.
extern "C" void mel_cleanup(void) {}

extern "C" int glmasr_mel_spectrogram_batched(const float *pcm, long long pcm_stride, const int *num_samples_host,
                                              int num_windows, const float *mel_filters_transposed, uint16_t *mel_out,
                                              long long out_stride, int time_major, int *out_frames_host) {
    if (num_windows <= 0) return 0;
    if (num_windows > 4096 || pcm == nullptr || num_samples_host == nullptr || mel_filters_transposed == nullptr || mel_out == nullptr)
        return -1;
    cudaStream_t st = current_stream();
    int *d_ns = (int *)workspace_slot(WS_MEL_NS, 4096 * sizeof(int));
    int max_frames = 1;
    for (int i = 0; i < num_windows; ++i) {
        if (num_samples_host[i] < 0) return -1;
        const int n = frames_for(num_samples_host[i]);
        if (out_frames_host != nullptr) out_frames_host[i] = n;
        if (n > max_frames) max_frames = n;
    }
    if (cudaMemcpyAsync(d_ns, num_samples_host, (size_t)num_windows * sizeof(int), cudaMemcpyHostToDevice, st) != cudaSuccess) return -1;
    // the copy above reads pageable host memory: it has been staged when the call returns
    return launch_mel_batched(pcm, pcm_stride, d_ns, num_windows, max_frames, mel_filters_transposed, (__nv_bfloat16 *)mel_out,
                              out_stride, time_major, st)
               ? 0
               : -1;
}
