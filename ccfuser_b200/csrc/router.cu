// Router in one kernel: logits = x Wg^T (+ bias) on the tensor cores, then top-k and the softmax over the k selected
// logits in the epilogue, where the TMEM register layout already gives every thread one complete token row.
//
// Replaces nn.Linear + torch.topk + softmax of the reference gate (mix_moe/mix_moe/gates/naive_gate.py:31-38): the
// [T, E] logits never go to memory (unless asked for, in fp32, for an auxiliary loss) and the selection runs on fp32
// accumulators instead of logits rounded to half precision.
//
// Shape of the problem: T x d times d x E with E <= 256, i.e. a skinny GEMM that is bound by reading x once. One CTA
// per 128 token rows, 6 warps: warp 0 = TMA producer (x tile 128 x 64 and the matching 64-deep slice of all router
// rows per stage), warp 1 = MMA issuer (tcgen05.mma M128 x N x K16, N = E rounded up to 32, accumulator in TMEM),
// warps 2..5 = epilogue, one per TMEM lane quarter. Router rows beyond E are zero-filled by TMA and masked out of the
// selection. Every wait is bounded and reports through the status word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "gemm_common.cuh"

namespace ccf {

constexpr int kRtThreads = 192;
constexpr int kRtMaxStages = 8;
constexpr int kRtABytes = BM * BK * 2;   // 128 rows x 128 bytes
constexpr int kRtMaxK = 8;

// Running top-kRtMaxK selection, best first. A candidate enters only if it is strictly greater than the current last
// entry (or that entry is still empty, id -1) and bubbles up past strictly smaller or empty ones, so among equal logits
// the lower expert id stays in front (candidates are offered in ascending id order) and a row of -inf logits still
// yields the ids 0, 1, ... rather than none. Host-callable so that the rule can be tested without a GPU.
__host__ __device__ __forceinline__ void topk_offer(float (&tv)[kRtMaxK], int (&ti)[kRtMaxK], float v, int e) {
  if (v > tv[kRtMaxK - 1] || ti[kRtMaxK - 1] < 0) {
    tv[kRtMaxK - 1] = v;
    ti[kRtMaxK - 1] = e;
#pragma unroll
    for (int j = kRtMaxK - 1; j > 0; --j) {
      if (tv[j] > tv[j - 1] || ti[j - 1] < 0) {
        const float fv = tv[j]; tv[j] = tv[j - 1]; tv[j - 1] = fv;
        const int iv = ti[j]; ti[j] = ti[j - 1]; ti[j - 1] = iv;
      }
    }
  }
}

// softmax over the first k selected logits -> idx[k], w[k]; `poison` (the row held a NaN logit) makes the weights NaN
__host__ __device__ __forceinline__ void topk_finish(const float (&tv)[kRtMaxK], const int (&ti)[kRtMaxK], int k, int* idx,
                                                     float* w, bool poison = false) {
  float ex[kRtMaxK];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kRtMaxK; ++j) {
    ex[j] = (j < k) ? expf(tv[j] - tv[0]) : 0.f;
    sum += ex[j];
  }
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < kRtMaxK; ++j) {
    if (j < k) {
      idx[j] = ti[j];
      w[j] = poison ? NAN : ex[j] * inv;
    }
  }
}

struct __align__(16) RouterCtrl {
  uint64_t full[kRtMaxStages];
  uint64_t empty[kRtMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_word;
  float bias[256];
};

struct RouterArgs {
  const void* bias;        // [E] in the operand type, or null
  int* idx;                // [T, k] out
  float* w;                // [T, k] out
  float* logits;           // optional [T, E] fp32 out
  int* status;
  unsigned long long wait_limit_ns;
  int tokens, d, e, n_pad, k, fp16, stages, tmem_cols;
};

__global__ void __launch_bounds__(kRtThreads, 1)
router_topk_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ RouterArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = kRtABytes + a.n_pad * 128;
  RouterCtrl* ctrl = reinterpret_cast<RouterCtrl*>(smem + a.stages * stage_bytes);
  const uint32_t smem_base = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_word = &ctrl->abort_word;
  const uint64_t limit = fail_fast_limit(a.status, a.wait_limit_ns);
  const int row0 = blockIdx.x * BM;
  const int kblocks = (a.d + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctrl->acc_full), 1);
    ctrl->abort_word = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmX);
    prefetch_tensormap(&tmW);
  }
  for (int e = threadIdx.x; e < 256; e += kRtThreads) {
    float b = 0.f;
    if (a.bias != nullptr && e < a.e)
      b = a.fp16 ? __half2float(reinterpret_cast<const __half*>(a.bias)[e])
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[e]);
    ctrl->bias[e] = b;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), static_cast<uint32_t>(a.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  if (warp == 0) {
    // ======================= TMA producer =======================
    int stage = 0, phase = 0;
    for (int kb = 0; kb < kblocks; ++kb) {
      if (!mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_word, limit)) {
        report_status(a.status, CCF_ERR_MBAR_TIMEOUT, 0x40);
        break;
      }
      if (lane == 0) {
        const uint32_t fullb = smem_u32(&ctrl->full[stage]);
        const uint32_t sa = smem_base + stage * stage_bytes;
        mbar_arrive_expect_tx(fullb, static_cast<uint32_t>(stage_bytes));
        tma_load_2d(sa, &tmX, fullb, kb * BK, row0);            // rows past T and columns past d read as zero
        tma_load_2d(sa + kRtABytes, &tmW, fullb, kb * BK, 0);   // all router rows (box of n_pad rows)
      }
      __syncwarp();
      if (++stage == a.stages) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1) {
    // ======================= MMA issuer =======================
    const uint32_t idesc = make_idesc(BM, a.n_pad, a.fp16, MAJ_K, MAJ_K);
    int stage = 0, phase = 0;
    for (int kb = 0; kb < kblocks; ++kb) {
      if (!mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_word, limit)) {
        report_status(a.status, CCF_ERR_MBAR_TIMEOUT, 0x41);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t sa = smem_base + stage * stage_bytes;
        const uint32_t sb = sa + kRtABytes;
#pragma unroll
        for (int k = 0; k < BK / UK; ++k)
          umma_f16(tmem_base, make_smem_desc(sa + k * 32, 16, 1024), make_smem_desc(sb + k * 32, 16, 1024), idesc,
                   (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(smem_u32(&ctrl->empty[stage]));
        if (kb == kblocks - 1) umma_commit(smem_u32(&ctrl->acc_full));
      }
      __syncwarp();
      if (++stage == a.stages) { stage = 0; phase ^= 1; }
    }
  } else {
    // ======================= epilogue: one token row per thread =======================
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    const int row = row0 + q * 32 + lane;
    if (mbar_wait(smem_u32(&ctrl->acc_full), 0, abort_word, limit)) {
      tc_fence_after();
      // running top-8 in registers, best first; a candidate enters only if it is strictly greater than the current
      // last entry and bubbles up past strictly smaller ones, so equal logits keep the lower expert id first
      float tv[kRtMaxK];
      int ti[kRtMaxK];
#pragma unroll
      for (int j = 0; j < kRtMaxK; ++j) { tv[j] = -INFINITY; ti[j] = -1; }
      bool has_nan = false;   // a NaN logit is ranked as -inf and turns the row's weights into NaN
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      for (int c = 0; c < a.n_pad; c += 32) {
        uint32_t racc[32];
        tmem_ld32(t_row + c, racc);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int e = c + i;
          float v = __uint_as_float(racc[i]) + ctrl->bias[e];
          if (a.logits != nullptr && row < a.tokens && e < a.e) a.logits[static_cast<size_t>(row) * a.e + e] = v;
          if (e < a.e) {
            if (v != v) { has_nan = true; v = -INFINITY; }
            topk_offer(tv, ti, v, e);
          }
        }
      }
      if (row < a.tokens)
        topk_finish(tv, ti, a.k, a.idx + static_cast<size_t>(row) * a.k, a.w + static_cast<size_t>(row) * a.k, has_nan);
    } else {
      report_status(a.status, CCF_ERR_MBAR_TIMEOUT, 0x42);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (ctrl->abort_word) {
    // give copies still in flight time to land before shared memory and TMEM go away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(a.tmem_cols));
  }
}


// ---------------------------------------------------------------------------------------------------
// Backward of the router without a GEMM. The gradient of the logits is non-zero only in the k selected columns,
//   g[t, j] = w[t, j] * (dw[t, j] - sum_i w[t, i] dw[t, i])          (softmax over the selected logits),
// so   dx[t, :]  = sum_j g[t, j] * Wg[idx[t, j], :]                  (k rows of the small router matrix per token)
// and  dWg[e, :] = sum over the slots routed to e of g * x[t, :],   db[e] = sum of those g.
// Both are bound by reading or writing one [T, d] matrix once; the dense [T, E] gradient is never formed. A slot whose
// id lies outside [0, E) (masked token) contributes nothing.
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float slot_grad(const float* w, const float* dw, size_t base, int K, int j) {
  float dot = 0.f;
  for (int i = 0; i < K; ++i) dot += w[base + i] * dw[base + i];
  return w[base + j] * (dw[base + j] - dot);
}

// one warp per token; every lane owns 16-byte pieces of the row
__global__ void __launch_bounds__(256) router_bwd_dx_kernel(const int* __restrict__ idx, const float* __restrict__ w,
                                                            const float* __restrict__ dw, const void* __restrict__ wg,
                                                            void* __restrict__ dx, int T, int d, int E, int K, int fp16) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const size_t base = static_cast<size_t>(t) * K;
  int e_j[kRtMaxK];
  float g_j[kRtMaxK];
#pragma unroll
  for (int j = 0; j < kRtMaxK; ++j) {
    e_j[j] = -1;
    g_j[j] = 0.f;
    if (j < K) {
      const int e = idx[base + j];
      if (e >= 0 && e < E) { e_j[j] = e; g_j[j] = slot_grad(w, dw, base, K, j); }
    }
  }
  const int vecs = d >> 3;
  const uint4* wv = reinterpret_cast<const uint4*>(wg);
  uint4* out = reinterpret_cast<uint4*>(dx) + static_cast<size_t>(t) * vecs;
  for (int v = lane; v < vecs; v += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < kRtMaxK; ++j) {
      if (e_j[j] < 0) continue;
      const uint4 r = __ldg(wv + static_cast<size_t>(e_j[j]) * vecs + v);
      const uint32_t q[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2(q[i], fp16);
        acc[2 * i] = fmaf(g_j[j], f.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(g_j[j], f.y, acc[2 * i + 1]);
      }
    }
    out[v] = make_uint4(pack2(acc[0], acc[1], fp16), pack2(acc[2], acc[3], fp16), pack2(acc[4], acc[5], fp16),
                        pack2(acc[6], acc[7], fp16));
  }
}

// Block (cx, ty, ez): columns [256 cx, 256 cx + 256), tokens ty, ty + gridDim.y, ... (one warp each), experts
// [64 ez, 64 ez + 64). Partial sums are kept in shared memory (64 x 256 fp32) and added to the fp32 result at the end,
// so the global atomics number E x d per block, not one per slot.
constexpr int kRtBwdCols = 256, kRtBwdExperts = 64;
__global__ void __launch_bounds__(256) router_bwd_dw_kernel(const int* __restrict__ idx, const float* __restrict__ w,
                                                            const float* __restrict__ dw, const void* __restrict__ x,
                                                            float* __restrict__ dwg, float* __restrict__ db, int T, int d,
                                                            int E, int K, int fp16) {
  extern __shared__ float racc[];   // [kRtBwdExperts][kRtBwdCols] + [kRtBwdExperts]
  float* bacc = racc + kRtBwdExperts * kRtBwdCols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = blockIdx.x * kRtBwdCols + lane * 8;
  const int e0 = blockIdx.z * kRtBwdExperts;
  for (int i = threadIdx.x; i < kRtBwdExperts * kRtBwdCols + kRtBwdExperts; i += blockDim.x) racc[i] = 0.f;
  __syncthreads();
  const int warps_total = gridDim.y * (blockDim.x >> 5);
  for (int t = blockIdx.y * (blockDim.x >> 5) + warp; t < T; t += warps_total) {
    const size_t base = static_cast<size_t>(t) * K;
    bool any = false;
    for (int j = 0; j < K; ++j) {
      const int e = idx[base + j] - e0;
      any |= (e >= 0 && e < kRtBwdExperts && e + e0 < E);
    }
    if (!any) continue;
    float xf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (col0 < d) {
      const uint4 r = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) +
                                                           static_cast<size_t>(t) * d + col0));
      const uint32_t q[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2(q[i], fp16);
        xf[2 * i] = f.x;
        xf[2 * i + 1] = f.y;
      }
    }
    for (int j = 0; j < K; ++j) {
      const int e = idx[base + j] - e0;
      if (e < 0 || e >= kRtBwdExperts || e + e0 >= E) continue;
      const float g = slot_grad(w, dw, base, K, j);
      if (col0 < d) {
        // element i of this lane's 8 columns lives at [e][32 i + lane]: the 32 lanes of an atomic hit 32 banks
        float* row = racc + e * kRtBwdCols + lane;
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(row + 32 * i, g * xf[i]);
      }
      if (blockIdx.x == 0 && lane == 0 && db != nullptr) atomicAdd(bacc + e, g);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kRtBwdExperts * kRtBwdCols; i += blockDim.x) {
    const int e = i / kRtBwdCols + e0, within = i % kRtBwdCols;
    const int c = blockIdx.x * kRtBwdCols + (within & 31) * 8 + (within >> 5);
    const float v = racc[i];
    if (e < E && c < d && v != 0.f) atomicAdd(dwg + static_cast<size_t>(e) * d + c, v);
  }
  if (blockIdx.x == 0 && db != nullptr && threadIdx.x < kRtBwdExperts && e0 + threadIdx.x < E) {
    const float v = bacc[threadIdx.x];
    if (v != 0.f) atomicAdd(db + e0 + threadIdx.x, v);
  }
}

}  // namespace ccf

extern "C" {

// The epilogue's selection rule on host memory (fp32 logits [tokens, e] -> idx, w), for tests without a GPU.
int ccf_router_select_host(const float* logits, int tokens, int e, int k, int* idx, float* w) {
  using namespace ccf;
  if (e < 1 || e > 256 || k < 1 || k > kRtMaxK || k > e) return -2;
  for (int t = 0; t < tokens; ++t) {
    float tv[kRtMaxK];
    int ti[kRtMaxK];
    for (int j = 0; j < kRtMaxK; ++j) { tv[j] = -INFINITY; ti[j] = -1; }
    bool has_nan = false;
    for (int i = 0; i < e; ++i) {
      float v = logits[static_cast<size_t>(t) * e + i];
      if (v != v) { has_nan = true; v = -INFINITY; }
      topk_offer(tv, ti, v, i);
    }
    topk_finish(tv, ti, k, idx + static_cast<size_t>(t) * k, w + static_cast<size_t>(t) * k, has_nan);
  }
  return 0;
}

// x [tokens, d] and wg [e, d] are 2-byte row-major operands of the same type (fp16 = 1: half, 0: bf16), bias [e] of
// that type or null. idx [tokens, k] int32 and w [tokens, k] fp32 are written; logits_f32 [tokens, e] only if not null.
// Limits: e <= 256, k <= min(8, e), d a multiple of 8 and at least 64. Returns 0, or a negative host-side error.
int ccf_router_topk(const void* x, const void* wg, const void* bias, int tokens, int d, int e, int k, int fp16, int* idx,
                    float* w, float* logits_f32, int* status, unsigned long long wait_limit_ns, int device,
                    void* stream_v) {
  using namespace ccf;
  if (tokens < 1 || e < 1 || e > 256 || k < 1 || k > kRtMaxK || k > e || d < 64 || d % 8 != 0) return -2;
  if (device >= 0 && cudaSetDevice(device) != cudaSuccess) return -7;
  RouterArgs a;
  a.bias = bias; a.idx = idx; a.w = w; a.logits = logits_f32; a.status = status; a.wait_limit_ns = wait_limit_ns;
  a.tokens = tokens; a.d = d; a.e = e; a.k = k; a.fp16 = fp16;
  a.n_pad = (e + 31) / 32 * 32;
  a.tmem_cols = 32;
  while (a.tmem_cols < a.n_pad) a.tmem_cols *= 2;
  const int stage_bytes = kRtABytes + a.n_pad * 128;
  a.stages = 200 * 1024 / stage_bytes;
  if (a.stages > kRtMaxStages) a.stages = kRtMaxStages;
  const int kblocks = (d + BK - 1) / BK;
  if (a.stages > kblocks) a.stages = kblocks;
  if (a.stages < 1) return -3;
  const int smem_bytes = 1024 + a.stages * stage_bytes + static_cast<int>(sizeof(RouterCtrl));
  CUtensorMap tmx, tmw;
  int rc;
  if ((rc = make_tmap(&tmx, x, tokens, d, 64, BM, fp16))) return rc;
  if ((rc = make_tmap(&tmw, wg, e, d, 64, a.n_pad, fp16))) return rc;
  static bool configured[64] = {};   // per device: the attribute belongs to the (function, device) pair
  int cur = 0;
  cudaGetDevice(&cur);
  if (!configured[cur & 63]) {
    cudaError_t err = cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (err != cudaSuccess) return -static_cast<int>(err);
    configured[cur & 63] = true;
  }
  const int grid = (tokens + BM - 1) / BM;
  router_topk_kernel<<<grid, kRtThreads, smem_bytes, reinterpret_cast<cudaStream_t>(stream_v)>>>(tmx, tmw, a);
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -static_cast<int>(err);
}

// Backward of the router for the k selected columns (see the kernels above). idx [tokens, k], w and dw [tokens, k] fp32
// (dw = gradient arriving for the weights); wg [e, d] and x [tokens, d] in the operand type. dx [tokens, d] (operand
// type) is written when not null; dwg [e, d] and db [e] (fp32, zero on entry; db may be null) are accumulated into
// when dwg is not null. Limits as in ccf_router_topk.
int ccf_router_bwd(const int* idx, const float* w, const float* dw, const void* wg, const void* x, void* dx, float* dwg,
                   float* db, int tokens, int d, int e, int k, int fp16, void* stream_v) {
  using namespace ccf;
  if (tokens < 1 || e < 1 || e > 256 || k < 1 || k > kRtMaxK || d < 8 || d % 8 != 0) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_v);
  if (dx != nullptr) {
    const int threads = 256, blocks = (tokens * 32 + threads - 1) / threads;
    router_bwd_dx_kernel<<<blocks, threads, 0, st>>>(idx, w, dw, wg, dx, tokens, d, e, k, fp16);
  }
  if (dwg != nullptr) {
    const int smem = (kRtBwdExperts * kRtBwdCols + kRtBwdExperts) * static_cast<int>(sizeof(float));
    static bool configured[64] = {};
    int cur = 0;
    cudaGetDevice(&cur);
    if (!configured[cur & 63]) {
      cudaError_t err = cudaFuncSetAttribute(router_bwd_dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (err != cudaSuccess) return -static_cast<int>(err);
      configured[cur & 63] = true;
    }
    const int cx = (d + kRtBwdCols - 1) / kRtBwdCols, ez = (e + kRtBwdExperts - 1) / kRtBwdExperts;
    int ty = (tokens + 63) / 64;                 // at least 64 tokens (8 per warp) per block
    const int cap = (4 * 148 + cx * ez - 1) / (cx * ez);
    if (ty > cap) ty = cap;
    if (ty < 1) ty = 1;
    router_bwd_dw_kernel<<<dim3(cx, ty, ez), 256, smem, st>>>(idx, w, dw, x, dwg, db, tokens, d, e, k, fp16);
  }
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : -static_cast<int>(err);
}

}  // extern "C"
