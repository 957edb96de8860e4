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
  // the row stays packed (8 registers per 16-byte piece instead of 16 floats): more warps fit on an SM
  uint4 xv[kV];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kV; ++i) {
    const int v = lane + 32 * i;
    xv[i] = make_uint4(0, 0, 0, 0);
    if (v < vecs) xv[i] = __ldg(xr + v);
    const uint32_t q[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2(q[j], fp16);
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
      const uint32_t q[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack2(q[j], fp16);
        const float c0 = t.x - mean, c1 = t.y - mean;
        var = fmaf(c0, c0, fmaf(c1, c1, var));
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
    const uint32_t xq[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, gq[4] = {g.x, g.y, g.z, g.w}, bq[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = unpack2(xq[j], fp16), gf = unpack2(gq[j], fp16), bf = unpack2(bq[j], fp16);
      o[j] = pack2((xf.x - mean) * rstd * gf.x + bf.x, (xf.y - mean) * rstd * gf.y + bf.y, fp16);
    }
    yr[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Backward, two kernels. With xh = (x - mean) * rstd and g = dy * gamma:
//   dx = rstd * (g - mean_row(g) - xh * mean_row(g * xh))        one warp per row, like the forward pass
//   dgamma = sum_rows dy * xh,   dbeta = sum_rows dy              a column reduction over all rows
// Keeping both in one kernel meant a whole row's dgamma / dbeta partial sums in registers (255 per thread, one block
// per SM); reading x and dy a second time for the column reduction costs less than that occupancy did.
template <int kV>
__global__ void __launch_bounds__(kLnThreads) layernorm_bwd_dx_kernel(const void* __restrict__ x, const void* __restrict__ dy,
                                                                       const void* __restrict__ gamma,
                                                                       const float* __restrict__ mean_in,
                                                                       const float* __restrict__ rstd_in,
                                                                       void* __restrict__ dx, int rows, int d, int fp16) {
  const int row = blockIdx.x * kLnWarps + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int vecs = d >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x) + static_cast<size_t>(row) * vecs;
  const uint4* dr = reinterpret_cast<const uint4*>(dy) + static_cast<size_t>(row) * vecs;
  const uint4* gv = reinterpret_cast<const uint4*>(gamma);
  const float mean = mean_in[row], rstd = rstd_in[row];
  uint4 xv[kV], dv[kV];   // dv is overwritten with g = dy * gamma, packed again
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < kV; ++i) {
    const int v = lane + 32 * i;
    xv[i] = make_uint4(0, 0, 0, 0);
    dv[i] = make_uint4(0, 0, 0, 0);
    uint4 g4 = make_uint4(0, 0, 0, 0);
    if (v < vecs) { xv[i] = __ldg(xr + v); dv[i] = __ldg(dr + v); g4 = __ldg(gv + v); }
    const uint32_t xq[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, dq[4] = {dv[i].x, dv[i].y, dv[i].z, dv[i].w};
    const uint32_t gq[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = unpack2(xq[j], fp16), df = unpack2(dq[j], fp16), gf = unpack2(gq[j], fp16);
      const bool on = v < vecs;
      const float h0 = on ? (xf.x - mean) * rstd : 0.f, h1 = on ? (xf.y - mean) * rstd : 0.f;
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
    const uint4 g4 = __ldg(gv + v);
    const uint32_t xq[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w}, dq[4] = {dv[i].x, dv[i].y, dv[i].z, dv[i].w};
    const uint32_t gq[4] = {g4.x, g4.y, g4.z, g4.w};
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

// Block (cx, ry): columns [128 cx, 128 cx + 128) (16 lanes x 16 bytes), rows ry * kLnParamRows ... (16 row lanes, four
// rows in flight per thread). Partial sums meet in shared memory, then one fp32 atomic per column and block.
constexpr int kLnParamRows = 512;
__global__ void __launch_bounds__(256) layernorm_bwd_param_kernel(const void* __restrict__ x, const void* __restrict__ dy,
                                                                  const float* __restrict__ mean_in,
                                                                  const float* __restrict__ rstd_in,
                                                                  float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                                  int rows, int d, int fp16) {
  __shared__ float red[2][16][128];
  const int cx = threadIdx.x & 15, ry = threadIdx.x >> 4;
  const int col = blockIdx.x * 128 + cx * 8;
  const int r_begin = blockIdx.y * kLnParamRows, r_end = min(rows, r_begin + kLnParamRows);
  float pg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, pb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < d) {
    const uint16_t* xb = reinterpret_cast<const uint16_t*>(x) + col;
    const uint16_t* db = reinterpret_cast<const uint16_t*>(dy) + col;
    for (int r = r_begin + ry; r < r_end; r += 64) {
      uint4 xv[4], dv[4];
      float mu[4], rs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 16 * u;
        const bool on = rr < r_end;
        xv[u] = on ? __ldg(reinterpret_cast<const uint4*>(xb + static_cast<size_t>(rr) * d)) : make_uint4(0, 0, 0, 0);
        dv[u] = on ? __ldg(reinterpret_cast<const uint4*>(db + static_cast<size_t>(rr) * d)) : make_uint4(0, 0, 0, 0);
        mu[u] = on ? mean_in[rr] : 0.f;
        rs[u] = on ? rstd_in[rr] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t xq[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w}, dq[4] = {dv[u].x, dv[u].y, dv[u].z, dv[u].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 xf = unpack2(xq[q], fp16), df = unpack2(dq[q], fp16);
          pg[2 * q] = fmaf(df.x, (xf.x - mu[u]) * rs[u], pg[2 * q]);
          pg[2 * q + 1] = fmaf(df.y, (xf.y - mu[u]) * rs[u], pg[2 * q + 1]);
          pb[2 * q] += df.x;
          pb[2 * q + 1] += df.y;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    red[0][ry][cx * 8 + i] = pg[i];
    red[1][ry][cx * 8 + i] = pb[i];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c < d) {
      float sg = 0.f, sb = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) { sg += red[0][i][threadIdx.x]; sb += red[1][i][threadIdx.x]; }
      atomicAdd(dgamma + c, sg);
      if (dbeta != nullptr) atomicAdd(dbeta + c, sb);
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
    const int blocks = (rows + kLnWarps - 1) / kLnWarps;
    layernorm_bwd_dx_kernel<kV><<<blocks, kLnThreads, 0, st>>>(x, dy, gamma, mean, rstd, out, rows, d, fp16);
    dim3 grid((d + 127) / 128, (rows + kLnParamRows - 1) / kLnParamRows);
    layernorm_bwd_param_kernel<<<grid, 256, 0, st>>>(x, dy, mean, rstd, dgamma, dbeta, rows, d, fp16);
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
