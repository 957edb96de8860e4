// Stand-alone check of the grouped GEMM library without Python: numerics against a CPU loop that accumulates in fp32,
// and throughput against cuBLAS on the same problem.
//
// Counterpart of the reference's C++ harness (mix_moe/csrc/test.cpp: cpuF16F16Gemm oracle :215-226, max-error check
// :229-279, cuBLAS GemmEx timing loop :306-352, comparison with tolerance :59-70), which needs MPI + NVSHMEM, pickled
// fixtures at absolute paths and no longer compiles against its own kernels. This one links only the library, cudart
// and cuBLAS and generates its inputs:
//
//   ccf_selftest [rows_per_group=1000] [groups=4] [k=512] [n=1024] [iters=10]
//
// rows_per_group need not be a multiple of the tile height: the ragged last tile of every group is part of the check.
// Exit status 0 = all variants within tolerance and no status word set.
#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "gemm_args.h"

extern "C" int ccf_gemm_launch(const CcfGemmLaunch* L, void* stream);

#define CK(call)                                                                               \
  do {                                                                                         \
    cudaError_t e_ = (call);                                                                   \
    if (e_ != cudaSuccess) {                                                                   \
      fprintf(stderr, "%s:%d %s: %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(e_));    \
      return 2;                                                                                \
    }                                                                                          \
  } while (0)

static float bf(const __nv_bfloat16 v) { return __bfloat162float(v); }

static unsigned lcg(unsigned& s) { return s = s * 1664525u + 1013904223u; }
static float unit(unsigned& s) { return (static_cast<int>(lcg(s) >> 8) & 0xffff) / 32768.f - 1.f; }

int main(int argc, char** argv) {
  const int rows_per = argc > 1 ? atoi(argv[1]) : 1000;
  const int groups = argc > 2 ? atoi(argv[2]) : 4;
  const int k = argc > 3 ? atoi(argv[3]) : 512;
  const int n = argc > 4 ? atoi(argv[4]) : 1024;
  const int iters = argc > 5 ? atoi(argv[5]) : 10;
  if (rows_per < 1 || groups < 1 || groups > CCF_MAX_GROUPS || k < 64 || k % 8 || n < 32 || n % 32) {
    fprintf(stderr, "need rows_per_group >= 1, 1 <= groups <= %d, k >= 64 and k %% 8 == 0, n %% 32 == 0\n", CCF_MAX_GROUPS);
    return 2;
  }
  // every group starts on a multiple of 128 rows, as the layer's plan lays them out
  const int padded = (rows_per + 127) / 128 * 128;
  const long long rows = static_cast<long long>(padded) * groups;
  std::vector<__nv_bfloat16> ha(rows * k), hb(static_cast<size_t>(groups) * n * k), hc(rows * n);
  unsigned seed = 12345u;
  for (auto& v : ha) v = __float2bfloat16(unit(seed));
  for (auto& v : hb) v = __float2bfloat16(unit(seed) * 0.05f);
  std::vector<int> hbase(groups), hrows(groups);
  for (int g = 0; g < groups; ++g) { hbase[g] = g * padded; hrows[g] = rows_per; }

  __nv_bfloat16 *da, *db, *dc, *dref;
  int *dbase, *drows, *dsched, *dstatus;
  char* dflush;
  const size_t flush_bytes = 256u << 20;
  CK(cudaMalloc(&da, ha.size() * 2));
  CK(cudaMalloc(&db, hb.size() * 2));
  CK(cudaMalloc(&dc, hc.size() * 2));
  CK(cudaMalloc(&dref, hc.size() * 2));
  CK(cudaMalloc(&dbase, groups * 4));
  CK(cudaMalloc(&drows, groups * 4));
  CK(cudaMalloc(&dsched, 8 * 4));
  CK(cudaMalloc(&dstatus, 2 * 4));
  CK(cudaMalloc(&dflush, flush_bytes));
  CK(cudaMemcpy(da, ha.data(), ha.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(db, hb.data(), hb.size() * 2, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(dbase, hbase.data(), groups * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(drows, hrows.data(), groups * 4, cudaMemcpyHostToDevice));
  CK(cudaMemset(dsched, 0, 8 * 4));
  CK(cudaMemset(dstatus, 0, 2 * 4));

  CcfGemmLaunch L;
  memset(&L, 0, sizeof(L));
  L.args.group_base = dbase;
  L.args.group_rows = drows;
  L.args.out0 = dc;
  L.args.sched = dsched;
  L.args.status = dstatus;
  L.args.wait_limit_ns = 2000000000ull;
  L.args.ld_out = n;
  L.args.n = n;
  L.args.k = k;
  L.args.num_groups = groups;
  L.args.kseg = 1;
  L.args.b_group_rows = n;
  L.args.world = 1;
  L.args.total_index = -1;
  L.a0 = da;
  L.b0 = db;
  L.a_rows = rows;
  L.a_cols = k;
  L.b_rows = static_cast<long long>(groups) * n;
  L.b_cols = k;
  L.a_major = 0;
  L.b_major = 0;
  L.epi = CCF_EPI_STORE;
  L.device = -1;

  // CPU oracle on a sample of rows of every group (first, last valid, and a stride through the middle)
  std::vector<int> sample;
  for (int g = 0; g < groups; ++g) {
    sample.push_back(g * padded);
    sample.push_back(g * padded + rows_per - 1);
    for (int r = 7; r < rows_per; r += 97) sample.push_back(g * padded + r);
  }
  int failures = 0;
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  const double flops = 2.0 * rows_per * groups * static_cast<double>(k) * n;
  for (int two_cta = 0; two_cta <= 1; ++two_cta) {
    L.two_cta = two_cta;
    CK(cudaMemset(dc, 0xff, hc.size() * 2));
    int rc = ccf_gemm_launch(&L, nullptr);
    if (rc != 0) {
      fprintf(stderr, "ccf_gemm_launch(two_cta=%d) returned %d\n", two_cta, rc);
      return 2;
    }
    CK(cudaDeviceSynchronize());
    int st[2];
    CK(cudaMemcpy(st, dstatus, 8, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(hc.data(), dc, hc.size() * 2, cudaMemcpyDeviceToHost));
    double max_err = 0, max_ref = 0;
    for (int r : sample) {
      const int g = r / padded;
      for (int j = 0; j < n; ++j) {
        float acc = 0.f;
        const __nv_bfloat16* arow = &ha[static_cast<size_t>(r) * k];
        const __nv_bfloat16* brow = &hb[(static_cast<size_t>(g) * n + j) * k];
        for (int i = 0; i < k; ++i) acc += bf(arow[i]) * bf(brow[i]);
        const double err = fabs(static_cast<double>(bf(hc[static_cast<size_t>(r) * n + j])) - acc);
        if (err > max_err) max_err = err;
        if (fabs(acc) > max_ref) max_ref = fabs(acc);
      }
    }
    // bf16 output rounding is 2^-9 relative; allow 1 % of the largest reference magnitude
    const bool ok = st[0] == 0 && st[1] == 0 && max_err <= 0.01 * max_ref + 1e-6;
    if (!ok) ++failures;
    // timing: L2 flushed between launches
    float ms_sum = 0.f;
    for (int it = 0; it < iters + 2; ++it) {
      CK(cudaMemsetAsync(dflush, it, flush_bytes, nullptr));
      CK(cudaEventRecord(e0, nullptr));
      rc = ccf_gemm_launch(&L, nullptr);
      CK(cudaEventRecord(e1, nullptr));
      CK(cudaEventSynchronize(e1));
      if (rc != 0) return 2;
      float ms;
      CK(cudaEventElapsedTime(&ms, e0, e1));
      if (it >= 2) ms_sum += ms;
    }
    const double ms = ms_sum / iters;
    printf("{\"variant\": \"%s\", \"rows_per_group\": %d, \"groups\": %d, \"k\": %d, \"n\": %d, \"max_abs_err\": %.5g, "
           "\"max_ref\": %.5g, \"status\": [%d, %d], \"ok\": %s, \"ms\": %.4f, \"tflops\": %.1f}\n",
           two_cta ? "cta_pair_256x256" : "one_cta_128x256", rows_per, groups, k, n, max_err, max_ref, st[0], st[1],
           ok ? "true" : "false", ms, flops / ms / 1e9);
  }

  // cuBLAS on the same problem: one GEMM per group, C_g[rows, n] = A_g[rows, k] B_g[n, k]^T (column-major view: C^T = B A^T)
  cublasHandle_t h;
  if (cublasCreate(&h) != CUBLAS_STATUS_SUCCESS) {
    fprintf(stderr, "cublasCreate failed\n");
    return 2;
  }
  const float one = 1.f, zero = 0.f;
  float ms_sum = 0.f;
  for (int it = 0; it < iters + 2; ++it) {
    CK(cudaMemsetAsync(dflush, it, flush_bytes, nullptr));
    CK(cudaEventRecord(e0, nullptr));
    for (int g = 0; g < groups; ++g) {
      cublasStatus_t s = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, n, rows_per, k, &one,
                                      db + static_cast<size_t>(g) * n * k, CUDA_R_16BF, k,
                                      da + static_cast<size_t>(g) * padded * k, CUDA_R_16BF, k, &zero,
                                      dref + static_cast<size_t>(g) * padded * n, CUDA_R_16BF, n, CUBLAS_COMPUTE_32F,
                                      CUBLAS_GEMM_DEFAULT);
      if (s != CUBLAS_STATUS_SUCCESS) {
        fprintf(stderr, "cublasGemmEx failed: %d\n", static_cast<int>(s));
        return 2;
      }
    }
    CK(cudaEventRecord(e1, nullptr));
    CK(cudaEventSynchronize(e1));
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    if (it >= 2) ms_sum += ms;
  }
  {
    // the library result against cuBLAS on every valid element
    std::vector<__nv_bfloat16> href(hc.size());
    CK(cudaMemcpy(href.data(), dref, href.size() * 2, cudaMemcpyDeviceToHost));
    double max_diff = 0;
    for (int g = 0; g < groups; ++g)
      for (int r = 0; r < rows_per; ++r)
        for (int j = 0; j < n; ++j) {
          const size_t o = (static_cast<size_t>(g) * padded + r) * n + j;
          const double d = fabs(static_cast<double>(bf(hc[o])) - bf(href[o]));
          if (d > max_diff) max_diff = d;
        }
    const double ms = ms_sum / iters;
    printf("{\"variant\": \"cublas_per_group\", \"ms\": %.4f, \"tflops\": %.1f, \"max_abs_diff_vs_library\": %.5g}\n", ms,
           flops / ms / 1e9, max_diff);
  }
  cublasDestroy(h);
  cudaFree(da); cudaFree(db); cudaFree(dc); cudaFree(dref); cudaFree(dbase); cudaFree(drows); cudaFree(dsched);
  cudaFree(dstatus); cudaFree(dflush);
  return failures ? 1 : 0;
}
