// LayerNorm forward and backward for 2-byte activations, one warp per row, fp32 statistics.
//
// The transformer blocks around the MoE layers (the reference's example models are stock GPT-2 / BERT / Transformer-XL,
// mix_moe/mix_moe/examples/models/moe_gpt.py, moe_bert.py, transformer-xl/mem_transformer_mix_moe.py) normalise a
// [tokens, d_model] matrix twice per block. Both passes are bound by reading and writing that matrix once; the
// backward also reduces the weight and bias gradients over all rows, which is done here with per-thread partial sums
// over the rows a warp visits, one shared-memory reduction per block and one fp32 atomic per column and block.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dispatch.cuh"   // pack2 / unpack2

namespace ccf {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;

// kV = 16-byte pieces of a row per lane (row length <= 256 * kV elements)
template <int kV>
__global__ void __launch_bounds__(kLnThreads) layernorm_fwd_kernel(const void* __restrict__ x, const void* __restrict__ gamma,
                                                                    const void* __restrict__ beta, void* __restrict__ y,
                                                                    float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                    int rows, int d, float eps, int fp16) {
  const int row = blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int vecs = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x) + static_cast<size_t>(row) * vecs;
  float f[kV][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kV; ++i) {
    const int v = lane + 32 * i;
    uint4 r = make_uint4(0, 0, 0, 0);
    if (v < vecs) r = __ldg(xr + v);
    const uint32_t q[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2(q[j], fp16);
      f[i][2 * j] = t.x;
      f[i][2 * j + 1] = t.y;
      sum += t.x + t.y;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const float mean = sum / d;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < kV; ++i) {
    if (lane + 32 * i < vecs) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = f[i][j] - mean;
        var = fmaf(c, c, var);
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) var += __shfl_xor_sync(0xffffffffu, var, off);
  const float rstd = rsqrtf(var / d + eps);
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  uint4* yr = reinterpret_cast<uint4*>(y) + static_cast<size_t>(row) * vecs;
  const uint4* gv = reinterpret_cast<const uint4*>(gamma);
  const uint4* bv = reinterpret_cast<const uint4*>(beta);
#pragma unroll
  for (int i = 0; i < kV; ++i) {
    const int v = lane + 32 * i;
    if (v >= vecs) continue;
    const uint4 g = __ldg(gv + v);
    const uint4 b = beta != nullptr ? __ldg(bv + v) : make_uint4(0, 0, 0, 0);
    const uint32_t gq[4] = {g.x, g.y, g.z, g.w}, bq[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gf = unpack2(gq[j], fp16), bf = unpack2(bq[j], fp16);
      o[j] = pack2((f[i][2 * j] - mean) * rstd * gf.x + bf.x, (f[i][2 * j + 1] - mean) * rstd * gf.y + bf.y, fp16);
    }
    yr[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Backward. With xh = (x - mean) * rstd and g = dy * gamma:
//   dx = rstd * (g - mean_row(g) - xh * mean_row(g * xh)),   dgamma = sum_rows dy * xh,   dbeta = sum_rows dy.
// Warps stride over the rows; every thread keeps the dgamma / dbeta partial sums of its own columns in registers.
template <int kV>
__global__ void __launch_bounds__(kLnThreads) layernorm_bwd_kernel(const void* __restrict__ x, const void* __restrict__ dy,
                                                                    const void* __restrict__ gamma,
                                                                    const float* __restrict__ mean_in,
                                                                    const float* __restrict__ rstd_in, void* __restrict__ dx,
                                                                    float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                                    int rows, int d, int fp16) {
  extern __shared__ float lred[];   // [2][256 * kV]: dgamma and dbeta partial sums of the block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vecs = d >> 3;
  float pg[kV][8], pb[kV][8];
  const uint4* gv = reinterpret_cast<const uint4*>(gamma);
#pragma unroll
  for (int i = 0; i < kV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { pg[i][j] = 0.f; pb[i][j] = 0.f; }
  }
  const int warps_total = gridDim.x * kLnWarps;
  for (int row = blockIdx.x * kLnWarps + warp; row < rows; row += warps_total) {
    const uint4* xr = reinterpret_cast<const uint4*>(x) + static_cast<size_t>(row) * vecs;
    const uint4* dr = reinterpret_cast<const uint4*>(dy) + static_cast<size_t>(row) * vecs;
    const float mean = mean_in[row], rstd = rstd_in[row];
    // the row stays packed in registers between the two passes (statistics, then dx); gamma is re-read (cached)
    uint4 xv[kV], dv[kV];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kV; ++i) {
      const int v = lane + 32 * i;
      xv[i] = make_uint4(0, 0, 0, 0);
      dv[i] = make_uint4(0, 0, 0, 0);
      uint4 gq4 = make_uint4(0, 0, 0, 0);
      if (v < vecs) { xv[i] = __ldg(xr + v); dv[i] = __ldg(dr + v); gq4 = __ldg(gv + v); }
      const uint32_t xq[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, dq[4] = {dv[i].x, dv[i].y, dv[i].z, dv[i].w};
      const uint32_t gq[4] = {gq4.x, gq4.y, gq4.z, gq4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = unpack2(xq[j], fp16), df = unpack2(dq[j], fp16), gf = unpack2(gq[j], fp16);
        const bool on = v < vecs;
        const float h0 = on ? (xf.x - mean) * rstd : 0.f, h1 = on ? (xf.y - mean) * rstd : 0.f;
        pg[i][2 * j] = fmaf(df.x, h0, pg[i][2 * j]);
        pg[i][2 * j + 1] = fmaf(df.y, h1, pg[i][2 * j + 1]);
        pb[i][2 * j] += df.x;
        pb[i][2 * j + 1] += df.y;
        const float g0 = df.x * gf.x, g1 = df.y * gf.y;
        s1 += g0 + g1;
        s2 = fmaf(g0, h0, fmaf(g1, h1, s2));
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, off);
      s2 += __shfl_xor_sync(0xffffffffu, s2, off);
    }
    const float m1 = s1 / d, m2 = s2 / d;
    uint4* outr = reinterpret_cast<uint4*>(dx) + static_cast<size_t>(row) * vecs;
#pragma unroll
    for (int i = 0; i < kV; ++i) {
      const int v = lane + 32 * i;
      if (v >= vecs) continue;
      const uint4 gq4 = __ldg(gv + v);
      const uint32_t xq[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, dq[4] = {dv[i].x, dv[i].y, dv[i].z, dv[i].w};
      const uint32_t gq[4] = {gq4.x, gq4.y, gq4.z, gq4.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = unpack2(xq[j], fp16), df = unpack2(dq[j], fp16), gf = unpack2(gq[j], fp16);
        const float h0 = (xf.x - mean) * rstd, h1 = (xf.y - mean) * rstd;
        o[j] = pack2(rstd * (df.x * gf.x - m1 - h0 * m2), rstd * (df.y * gf.y - m1 - h1 * m2), fp16);
      }
      outr[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  // block reduction of the column sums: warp after warp adds its partials into shared memory, then one atomic per column
  float* sg = lred;
  float* sb = lred + 256 * kV;
  for (int i = threadIdx.x; i < 2 * 256 * kV; i += kLnThreads) lred[i] = 0.f;
  __syncthreads();
  for (int w = 0; w < kLnWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < kV; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // column c0 + j is stored at [j][vector index]: consecutive lanes hit consecutive banks
          sg[j * 32 * kV + lane + 32 * i] += pg[i][j];
          sb[j * 32 * kV + lane + 32 * i] += pb[i][j];
        }
      }
    }
    __syncthreads();
  }
  for (int s = threadIdx.x; s < 256 * kV; s += kLnThreads) {
    const int j = s / (32 * kV), v = s % (32 * kV);
    const int c = v * 8 + j;
    if (c < d) {
      atomicAdd(dgamma + c, sg[s]);
      if (dbeta != nullptr) atomicAdd(dbeta + c, sb[s]);
    }
  }
}

template <int kV>
static int launch_ln(bool fwd, const void* x, const void* dy, const void* gamma, const void* beta, void* out, float* mean,
                     float* rstd, float* dgamma, float* dbeta, int rows, int d, float eps, int fp16, cudaStream_t st) {
  if (fwd) {
    const int blocks = (rows + kLnWarps - 1) / kLnWarps;
    layernorm_fwd_kernel<kV><<<blocks, kLnThreads, 0, st>>>(x, gamma, beta, out, mean, rstd, rows, d, eps, fp16);
  } else {
    int blocks = (rows + kLnWarps - 1) / kLnWarps;
    if (blocks > 148 * 2) blocks = 148 * 2;
    const int smem = 2 * 256 * kV * static_cast<int>(sizeof(float));
    layernorm_bwd_kernel<kV><<<blocks, kLnThreads, smem, st>>>(x, dy, gamma, mean, rstd, out, dgamma, dbeta, rows, d, fp16);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // namespace ccf

extern "C" {

// Largest row length the kernels take (8 pieces of 16 bytes per lane).
int ccf_layernorm_max_d() { return 2048; }

// y = (x - mean) * rstd * gamma + beta over the last dimension of x [rows, d] (2-byte elements, gamma / beta of the same
// type, beta may be null); mean and rstd [rows] fp32 are written for the backward pass. d % 8 == 0, d <= 2048.
int ccf_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows,
                      int d, float eps, int fp16, void* stream) {
  using namespace ccf;
  if (rows < 1 || d < 8 || d % 8 != 0 || d > 2048) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (d <= 512) return launch_ln<2>(true, x, nullptr, gamma, beta, y, mean, rstd, nullptr, nullptr, rows, d, eps, fp16, st);
  if (d <= 1024) return launch_ln<4>(true, x, nullptr, gamma, beta, y, mean, rstd, nullptr, nullptr, rows, d, eps, fp16, st);
  return launch_ln<8>(true, x, nullptr, gamma, beta, y, mean, rstd, nullptr, nullptr, rows, d, eps, fp16, st);
}

// dx [rows, d] is written; dgamma and dbeta [d] (fp32, zero on entry; dbeta may be null) are accumulated into.
int ccf_layernorm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx,
                      float* dgamma, float* dbeta, int rows, int d, int fp16, void* stream) {
  using namespace ccf;
  if (rows < 1 || d < 8 || d % 8 != 0 || d > 2048) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (d <= 512) return launch_ln<2>(false, x, dy, gamma, nullptr, dx, const_cast<float*>(mean), const_cast<float*>(rstd), dgamma, dbeta, rows, d, 0.f, fp16, st);
  if (d <= 1024) return launch_ln<4>(false, x, dy, gamma, nullptr, dx, const_cast<float*>(mean), const_cast<float*>(rstd), dgamma, dbeta, rows, d, 0.f, fp16, st);
  return launch_ln<8>(false, x, dy, gamma, nullptr, dx, const_cast<float*>(mean), const_cast<float*>(rstd), dgamma, dbeta, rows, d, 0.f, fp16, st);
}

}  // extern "C"
