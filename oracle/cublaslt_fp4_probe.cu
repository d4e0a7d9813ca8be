// Yardstick for the W4A4 GEMM: NVIDIA's own block-scaled FP4 GEMM (cuBLASLt, e2m1 operands with one
// ue4m3 scale per 16 elements, fp32 accumulation, bf16 out) timed ALONE -- descriptors, heuristic and
// operands prepared outside the timed region -- on the shapes the benchmark runs and on 8192^3.
// It is the library call the reference's nvfp4_linear makes (Infer-engine/cuda/nvfp4_cutlass.cu:192-249)
// without that function's per-call quantiser, scale re-tiling, memsets and descriptor churn, so it is
// both "the kernel to beat" and a measured stand-in for the FP4 tensor peak of the GPU it runs on.
//
// MEASUREMENT INFRASTRUCTURE ONLY: built by oracle/Makefile into libcublaslt_fp4_probe.so, loaded by
// bench.py's yardstick leg and nothing else.  The product library does not link cuBLAS.
#include <cublasLt.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <algorithm>
#include <vector>

namespace {

struct Buffers {
    std::vector<uint8_t *> w, ws;      // rotating weight sets: packed e2m1 [N, K/2], tiled ue4m3 scales
    std::vector<uint8_t *> x, xs;      // rotating activation sets
    __nv_bfloat16 *out = nullptr;
    void *workspace = nullptr;
    ~Buffers() {
        for (auto p : w) cudaFree(p);
        for (auto p : ws) cudaFree(p);
        for (auto p : x) cudaFree(p);
        for (auto p : xs) cudaFree(p);
        cudaFree(out);
        cudaFree(workspace);
    }
};

__global__ void fill_bytes(uint8_t *p, size_t n, uint32_t seed, int scales) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + seed;
        h ^= h >> 15;
        h *= 2246822519u;
        h ^= h >> 13;
        // scales: e4m3 codes of 0.5 .. 1.75 (finite, non-zero); operands: any byte is a valid pair of e2m1 codes
        p[i] = scales ? (uint8_t)(0x30 + (h & 0x0F)) : (uint8_t)(h >> 8);
    }
}

size_t tiled_scale_bytes(int rows, int K) { return (size_t)((rows + 127) / 128 * 128) * (size_t)((K / 16 + 3) / 4 * 4); }

}  // namespace

// Times `iters` back-to-back cublasLtMatmul calls of out[M, N] = x[M, K] * w[N, K]^T after `warmup` untimed
// ones, rotating over `sets` operand sets so that no call finds its operands in L2, for each of up to
// `max_algos` heuristic results; *best_ms = the fastest algorithm's mean time per call, *first_ms = the
// first heuristic result's (what a caller that takes the top suggestion gets).  Returns 0, or -1 with a
// message on stderr.
extern "C" int cublaslt_fp4_gemm_time(int M, int N, int K, int iters, int warmup, int sets, int max_algos, double *best_ms,
                                      double *first_ms) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % 32) != 0 || iters <= 0 || sets <= 0 || best_ms == nullptr) return -1;
    const int Mp = (M + 15) / 16 * 16;
    cublasLtHandle_t lt = nullptr;
    if (cublasLtCreate(&lt) != CUBLAS_STATUS_SUCCESS) {
        fprintf(stderr, "cublaslt_fp4_probe: cublasLtCreate failed\n");
        return -1;
    }
    Buffers b;
    const size_t wbytes = (size_t)N * K / 2, xbytes = (size_t)Mp * K / 2;
    const size_t wsb = tiled_scale_bytes(N, K), xsb = tiled_scale_bytes(Mp, K);
    const size_t wsp = 64ull << 20;
    bool ok = true;
    for (int s = 0; s < sets && ok; ++s) {
        uint8_t *p[4] = {nullptr, nullptr, nullptr, nullptr};
        ok = cudaMalloc(&p[0], wbytes) == cudaSuccess && cudaMalloc(&p[1], wsb) == cudaSuccess &&
             cudaMalloc(&p[2], xbytes) == cudaSuccess && cudaMalloc(&p[3], xsb) == cudaSuccess;
        b.w.push_back(p[0]), b.ws.push_back(p[1]), b.x.push_back(p[2]), b.xs.push_back(p[3]);
        if (!ok) break;
        fill_bytes<<<1024, 256>>>(p[0], wbytes, 11u + s, 0);
        fill_bytes<<<256, 256>>>(p[1], wsb, 23u + s, 1);
        fill_bytes<<<1024, 256>>>(p[2], xbytes, 37u + s, 0);
        fill_bytes<<<256, 256>>>(p[3], xsb, 41u + s, 1);
    }
    ok = ok && cudaMalloc(&b.out, (size_t)Mp * N * sizeof(__nv_bfloat16)) == cudaSuccess &&
         cudaMalloc(&b.workspace, wsp) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    if (!ok) {
        fprintf(stderr, "cublaslt_fp4_probe: allocation failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        cublasLtDestroy(lt);
        return -1;
    }

    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasLtMatmulPreference_t pref = nullptr;
    const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    const cublasLtMatmulMatrixScale_t vec16 = CUBLASLT_MATMUL_MATRIX_SCALE_VEC16_UE4M3;
    int rc = -1;
    std::vector<cublasLtMatmulHeuristicResult_t> res((size_t)std::max(1, max_algos));
    int found = 0;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    do {
        if (cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_MODE, &vec16, sizeof(vec16)) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_MODE, &vec16, sizeof(vec16)) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatrixLayoutCreate(&la, CUDA_R_4F_E2M1, K, N, K) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatrixLayoutCreate(&lb, CUDA_R_4F_E2M1, K, Mp, K) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatrixLayoutCreate(&lc, CUDA_R_16BF, N, Mp, N) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulPreferenceCreate(&pref) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &wsp, sizeof(wsp)) != CUBLAS_STATUS_SUCCESS) break;
        const uint8_t *as = b.ws[0], *bs = b.xs[0];
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, &as, sizeof(as)) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, &bs, sizeof(bs)) != CUBLAS_STATUS_SUCCESS) break;
        if (cublasLtMatmulAlgoGetHeuristic(lt, op, la, lb, lc, lc, pref, (int)res.size(), res.data(), &found) != CUBLAS_STATUS_SUCCESS || found == 0) {
            fprintf(stderr, "cublaslt_fp4_probe: no algorithm for M=%d N=%d K=%d\n", M, N, K);
            break;
        }
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        const float alpha = 1.0f / 64.0f, beta = 0.0f;
        double best = 1e30, first = -1.0;
        for (int a = 0; a < found; ++a) {
            if (res[a].state != CUBLAS_STATUS_SUCCESS) continue;
            bool fail = false;
            auto call = [&](int i) {
                const int s = i % sets;
                const uint8_t *as2 = b.ws[s], *bs2 = b.xs[s];
                cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, &as2, sizeof(as2));
                cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, &bs2, sizeof(bs2));
                if (cublasLtMatmul(lt, op, &alpha, b.w[s], la, b.x[s], lb, &beta, b.out, lc, b.out, lc, &res[a].algo, b.workspace,
                                   wsp, 0) != CUBLAS_STATUS_SUCCESS)
                    fail = true;
            };
            for (int i = 0; i < warmup && !fail; ++i) call(i);
            if (fail || cudaDeviceSynchronize() != cudaSuccess) continue;
            cudaEventRecord(e0, 0);
            for (int i = 0; i < iters && !fail; ++i) call(i);
            cudaEventRecord(e1, 0);
            if (cudaEventSynchronize(e1) != cudaSuccess || fail) continue;
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, e0, e1);
            const double per = (double)ms / iters;
            if (first < 0.0) first = per;
            best = std::min(best, per);
        }
        if (best < 1e29) {
            *best_ms = best;
            if (first_ms != nullptr) *first_ms = first;
            rc = 0;
        }
    } while (false);
    if (rc != 0) fprintf(stderr, "cublaslt_fp4_probe: failed for M=%d N=%d K=%d (%s)\n", M, N, K, cudaGetErrorString(cudaGetLastError()));
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (pref) cublasLtMatmulPreferenceDestroy(pref);
    if (la) cublasLtMatrixLayoutDestroy(la);
    if (lb) cublasLtMatrixLayoutDestroy(lb);
    if (lc) cublasLtMatrixLayoutDestroy(lc);
    if (op) cublasLtMatmulDescDestroy(op);
    cublasLtDestroy(lt);
    return rc;
}
