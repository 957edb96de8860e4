// Routing, planning, dispatch, combine-reduce and bias-gradient kernels of the fused MoE layer.
// Everything here is bandwidth- or latency-bound glue around the tcgen05 GEMMs in gemm.cu; nothing
// involves the host (the reference plans on the CPU in Python, mix_moe/mix_moe/transformer.py:150-250,
// after a count all-gather and two device-to-host copies, mix_moe/mix_moe/functions.py:83-105).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "dispatch.cuh"
#include "gemm_args.h"
#include "sm100.cuh"

namespace ccf {

// ---------------------------------------------------------------------------------------------------
// gate: top-k over E logits + softmax over the k selected values, one warp per token
// (mix_moe/mix_moe/gates/naive_gate.py:31-38). Ties go to the lower expert id. A NaN logit never wins a comparison, so
// it is ranked as -inf (the ids written stay inside [0, E) whatever the row holds) and the row's k weights are NaN: a
// diverged router shows up in the layer's output instead of as an index out of range.
// ---------------------------------------------------------------------------------------------------
template <int kMaxPerLane>
__global__ void topk_softmax_kernel(const void* logits, int fp16, int is_f32, int T, int E, int K, int* idx_out,
                                    float* w_out) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  float v[kMaxPerLane];
  bool has_nan = false;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = i * 32 + lane;
    float x = -INFINITY;
    if (e < E) {
      if (is_f32) x = reinterpret_cast<const float*>(logits)[static_cast<size_t>(warp) * E + e];
      else if (fp16) x = __half2float(reinterpret_cast<const __half*>(logits)[static_cast<size_t>(warp) * E + e]);
      else x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[static_cast<size_t>(warp) * E + e]);
      if (x != x) { has_nan = true; x = -INFINITY; }
    }
    v[i] = x;
  }
  has_nan = __any_sync(0xffffffffu, has_nan);
  // entries already taken: a bit per register so that a row of -inf (or NaN) still yields K distinct ids
  unsigned taken = 0u;
  float sel_v[8];
  int sel_i[8];
  for (int j = 0; j < K; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < E && !((taken >> i) & 1u) && (v[i] > best || (v[i] == best && e < bi))) { best = v[i]; bi = e; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    sel_v[j] = best;
    sel_i[j] = bi;
    // remove the winner
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
  }
  if (lane == 0) {
    const float mx = sel_v[0];
    float sum = 0.f;
    for (int j = 0; j < K; ++j) { sel_v[j] = __expf(sel_v[j] - mx); sum += sel_v[j]; }
    for (int j = 0; j < K; ++j) {
      idx_out[static_cast<size_t>(warp) * K + j] = sel_i[j];
      w_out[static_cast<size_t>(warp) * K + j] = has_nan ? __int_as_float(0x7fc00000) : sel_v[j] / sum;
    }
  }
}

// dlogits[t, idx_j] = w_j * (dw_j - sum_i w_i dw_i), zero elsewhere. One thread per token.
__global__ void topk_softmax_bwd_kernel(const int* idx, const float* w, const float* dw, int T, int E, int K,
                                        void* dlogits, int fp16, int is_f32) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float dot = 0.f;
  for (int j = 0; j < K; ++j) dot += w[static_cast<size_t>(t) * K + j] * dw[static_cast<size_t>(t) * K + j];
  for (int j = 0; j < K; ++j) {
    const float g = w[static_cast<size_t>(t) * K + j] * (dw[static_cast<size_t>(t) * K + j] - dot);
    const int e = idx[static_cast<size_t>(t) * K + j];
    if (e < 0 || e >= E) continue;   // an id outside the table (masked slot) has no logit to receive a gradient
    const size_t o = static_cast<size_t>(t) * E + e;
    if (is_f32) reinterpret_cast<float*>(dlogits)[o] = g;
    else if (fp16) reinterpret_cast<__half*>(dlogits)[o] = __float2half(g);
    else reinterpret_cast<__nv_bfloat16*>(dlogits)[o] = __float2bfloat16(g);
  }
}

// ---------------------------------------------------------------------------------------------------
// deterministic position of every slot inside its expert (prefix count in slot order), counts, capacity
// (replaces expert_count_kernel + assign_pos_kernel, mix_moe/csrc/cuda/local_exchange.cu:6-70)
// ---------------------------------------------------------------------------------------------------
constexpr int kRouteBlock = 1024;

__global__ void __launch_bounds__(kRouteBlock)
route_hist_kernel(const int* __restrict__ expert, int S, int E, int cap, int* pos, int* block_hist, int* block_off,
                  int* count_raw, int* count_kept, int* ticket, int* order_off, int first_expert) {
  __shared__ int wh[32][CCF_MAX_GROUPS];
  __shared__ int is_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = gridDim.x;
  for (int i = tid; i < 32 * CCF_MAX_GROUPS; i += kRouteBlock) (&wh[0][0])[i] = 0;
  __syncthreads();
  const int s = blockIdx.x * kRouteBlock + tid;
  int e = (s < S) ? expert[s] : -1;
  if (e < 0 || e >= E) e = -1;
  const unsigned m = __match_any_sync(0xffffffffu, e);
  const int rank = __popc(m & ((1u << lane) - 1u));
  if (e >= 0 && rank == 0) wh[warp][e] = __popc(m);
  __syncthreads();
  if (tid < E) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = wh[w][tid];
      wh[w][tid] = run;
      run += c;
    }
    block_hist[blockIdx.x * E + tid] = run;
  }
  __syncthreads();
  if (s < S) pos[s] = (e >= 0) ? wh[warp][e] + rank : 0x3fffffff;
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = (atomicAdd(ticket, 1) == nb - 1);
  __syncthreads();
  if (is_last) {
    __threadfence();
    if (tid < E) {
      int run = 0;
      for (int b = 0; b < nb; ++b) {
        const int c = __ldcg(block_hist + b * E + tid);
        block_off[b * E + tid] = run;
        run += c;
      }
      count_raw[tid] = run;
      count_kept[tid] = min(run, cap);
    }
    __syncthreads();
    if (tid == 0) {
      *ticket = 0;
      if (order_off != nullptr) {
        // destination order of this rank's kept rows: experts starting with this rank's own (first_expert), then the
        // next owner's, ... so that local rows are pushed first and every source starts with a different owner
        int run = 0;
        for (int k = 0; k < E; ++k) {
          const int e = (first_expert + k) % E;
          order_off[e] = run;
          run += count_kept[e];
        }
        order_off[E] = run;  // kept rows in total
      }
    }
  }
}

__global__ void route_pos_kernel(const int* __restrict__ expert, int S, int E, const int* __restrict__ block_off,
                                 int* pos, int cap, const int* __restrict__ order_off, int* sorted_slot, int* slot_row) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const int e = expert[s];
  int p = pos[s];
  if (e >= 0 && e < E) {
    p += block_off[(s / kRouteBlock) * E + e];
    pos[s] = p;
  }
  if (sorted_slot != nullptr) {
    if (e >= 0 && e < E && p < cap) sorted_slot[order_off[e] + p] = s;   // inverse of the destination order
    else if (slot_row != nullptr) slot_row[s] = -1;                       // dropped slots are never dispatched
  }
}

// ---------------------------------------------------------------------------------------------------
// count exchange + plan. One CTA. Every rank writes its kept counts into every rank's table (peer
// stores + release flag carrying the step epoch), waits (bounded) for all rows of its own table, then
// computes the row layout of every owner's receive buffer:
//   rows of expert e start at base[e] (multiple of 128) on owner e / E_loc,
//   rows sent by source r start at base[e] + sum_{r' < r} count[r'][e].
// Replaces the NCCL all-gather + .cpu() + Python block planner of the reference
// (mix_moe/csrc/cuda/global_exchange.cpp:139-177, mix_moe/mix_moe/transformer.py:150-250).
// ---------------------------------------------------------------------------------------------------
using PlanArgs = ::CcfPlanArgs;   // gemm_args.h

__device__ __forceinline__ void plan_body(const PlanArgs& a, const int epoch) {
  __shared__ int rows[CCF_MAX_GROUPS];
  __shared__ int myoff[CCF_MAX_GROUPS];
  __shared__ int base[CCF_MAX_GROUPS];
  __shared__ int failed;
  const int tid = threadIdx.x;
  if (tid == 0) failed = 0;
  // 1. publish my counts
  for (int i = tid; i < a.world * a.e_total; i += blockDim.x) {
    const int p = i / a.e_total, e = i - p * a.e_total;
    a.peer_table[p][a.my_rank * a.e_total + e] = a.count_kept[e];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < a.world) st_release_sys(a.peer_flag[tid] + a.my_rank, epoch);
  // 2. wait for everyone's counts (my own table, local memory)
  if (tid < a.world) {
    if (!wait_flag_ge(a.peer_flag[a.my_rank] + tid, epoch, fail_fast_limit(a.status, a.wait_limit_ns))) {
      report_status(a.status, CCF_ERR_FLAG_TIMEOUT, 0x800000 | tid);
      failed = 1;
    }
  }
  __syncthreads();
  if (failed) {
    for (int e = tid; e < a.e_total; e += blockDim.x) a.dst_base[e] = 0;
    for (int e = tid; e < a.e_loc; e += blockDim.x) {
      a.group_base[e] = 0;
      a.group_rows[e] = 0;
      if (a.local_begin != nullptr) { a.local_begin[e] = 0; a.local_rows[e] = 0; }
    }
    if (tid < a.world) a.sent_rows[tid] = 0;
    return;
  }
  // 3. plan
  const int* table = a.peer_table[a.my_rank];
  for (int e = tid; e < a.e_total; e += blockDim.x) {
    int tot = 0, off = 0;
    for (int r = 0; r < a.world; ++r) {
      const int c = ld_relaxed_sys(table + r * a.e_total + e);
      if (a.table_copy) a.table_copy[r * a.e_total + e] = c;
      if (r < a.my_rank) off += c;
      tot += c;
    }
    rows[e] = tot;
    myoff[e] = off;
  }
  __syncthreads();
  if (tid < a.world) {
    int run = 0, sent = 0;
    for (int i = 0; i < a.e_loc; ++i) {
      const int e = tid * a.e_loc + i;
      base[e] = run;
      run += (rows[e] + 127) & ~127;
      // rows of mine that fit into the owner's buffer: the rest is rejected by the dispatch role and must not be
      // waited for (source and owner derive the same limit from the same table)
      const int first = run - ((rows[e] + 127) & ~127) + myoff[e];
      sent += max(0, min(a.count_kept[e], a.max_rows - first));
    }
    a.sent_rows[tid] = sent;
    if (run > a.max_rows) report_status(a.status, CCF_ERR_OVERFLOW, tid);
  }
  __syncthreads();
  for (int e = tid; e < a.e_total; e += blockDim.x) a.dst_base[e] = base[e] + myoff[e];
  for (int i = tid; i < a.e_loc; i += blockDim.x) {
    const int e = a.my_rank * a.e_loc + i;
    a.group_base[i] = base[e];
    a.group_rows[i] = min(rows[e], max(0, a.max_rows - base[e]));
    if (a.local_begin != nullptr) {
      a.local_begin[i] = myoff[e];
      a.local_rows[i] = max(0, min(a.count_kept[e], a.max_rows - (base[e] + myoff[e])));
    }
  }
}

__global__ void __launch_bounds__(256) plan_kernel(const __grid_constant__ PlanArgs a) { plan_body(a, a.epoch); }

// Same, with the call's epoch taken from a counter in device memory (previous value + 1, written back at the end)
// instead of a launch argument: a captured CUDA graph replays with fixed arguments, so a host-side epoch would
// repeat and the wait for the peers' counts would be satisfied by the previous call's flags.
__global__ void __launch_bounds__(256) plan_kernel_dev_epoch(const __grid_constant__ PlanArgs a, int* epoch_counter) {
  __shared__ int epoch;
  if (threadIdx.x == 0) epoch = *epoch_counter + 1;
  __syncthreads();
  plan_body(a, epoch);
  __syncthreads();
  if (threadIdx.x == 0) *epoch_counter = epoch;
}

// ---------------------------------------------------------------------------------------------------
// stand-alone dispatch kernel (the same role also runs inside the fused GEMM kernel)
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dispatch_kernel(const __grid_constant__ CcfDispatchArgs a, int* status,
                                                       int* done_ctas) {
  if (a.backward) dispatch_rows<8, true>(a, status); else dispatch_rows<8, false>(a, status);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_ctas, 1) == static_cast<int>(gridDim.x) - 1) {
      *a.work_counter = 0;
      *done_ctas = 0;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// combine: wait until every owner has stored all rows of this rank (and finished its kernel), then
// sum the top-k slots of each token. Counters are monotonic; `cum` holds the value already consumed.
// ---------------------------------------------------------------------------------------------------
__global__ void combine_wait_kernel(const int* done, int* cum, const int* sent_rows, int n_tiles, int world,
                                    unsigned long long limit_ns, int* status) {
  const int o = threadIdx.x;
  if (o >= world) return;
  const int target = cum[o] + sent_rows[o] * n_tiles + 1;
  if (!wait_flag_ge(done + o, target, fail_fast_limit(status, limit_ns)))
    report_status(status, CCF_ERR_FLAG_TIMEOUT, 0x400000 | o);
  cum[o] = target;
}

// y[t, :] = sum_j keep(t, j) * comb[t * k + j, :]; one thread per 16-byte piece of an output row, fp32 accumulate.
// (A warp per token made the kernel latency-bound for small batches: d / 256 dependent iterations per warp.)
__global__ void combine_reduce_kernel(const void* comb, const int* slot_row, void* y, int T, int K, int d, int fp16) {
  const int vecs = d >> 3;
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<long long>(T) * vecs) return;
  const int t = static_cast<int>(gid / vecs), v = static_cast<int>(gid - static_cast<long long>(t) * vecs);
  const uint4* c = reinterpret_cast<const uint4*>(comb);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < K; ++j) {
    const int s = t * K + j;
    if (__ldg(slot_row + s) < 0) continue;
    const uint4 x = c[static_cast<size_t>(s) * vecs + v];
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = unpack2(w[q], fp16);
      acc[2 * q] += f.x;
      acc[2 * q + 1] += f.y;
    }
  }
  uint4 o;
  o.x = pack2(acc[0], acc[1], fp16);
  o.y = pack2(acc[2], acc[3], fp16);
  o.z = pack2(acc[4], acc[5], fp16);
  o.w = pack2(acc[6], acc[7], fp16);
  reinterpret_cast<uint4*>(y)[static_cast<size_t>(t) * vecs + v] = o;
}

// ---------------------------------------------------------------------------------------------------
// bias gradients: out[g, n] = sum over the rows of group g of x[r, n]. Block = 128 columns (16 lanes x 16 bytes) x 16
// row lanes, four rows in flight per thread: the kernel streams the matrix once and has to keep enough loads in
// flight to do so at the memory rate.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) colsum_grouped_kernel(const void* x, long long ld, int n, const int* group_base,
                                                             const int* group_rows, void* out, int fp16) {
  __shared__ float red[16][128];
  const int g = blockIdx.y;
  const int cx = threadIdx.x & 15, ry = threadIdx.x >> 4;
  const int col = blockIdx.x * 128 + cx * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < n) {
    const int r0 = group_base[g], nr = group_rows[g];
    const uint16_t* base = reinterpret_cast<const uint16_t*>(x) + static_cast<size_t>(r0) * ld + col;
    for (int r = ry; r < nr; r += 64) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 16 * u;
        v[u] = rr < nr ? __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(rr) * ld)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack2(w[q], fp16);
          acc[2 * q] += f.x;
          acc[2 * q + 1] += f.y;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[ry][cx * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < 128) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c < n) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) s += red[i][threadIdx.x];
      if (fp16) reinterpret_cast<__half*>(out)[static_cast<size_t>(g) * n + c] = __float2half(s);
      else reinterpret_cast<__nv_bfloat16*>(out)[static_cast<size_t>(g) * n + c] = __float2bfloat16(s);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// SGD step on 2-byte parameters: p -= lr * (g + wd * p), 16-byte vectors, fp32 arithmetic. With 64 experts per GPU
// the optimizer streams ~150 GB per step; one pass with full-width accesses keeps it at the HBM rate.
// ---------------------------------------------------------------------------------------------------
// blocks [0, nb) of one tensor: block lb takes every nb-th group of 256 vectors; the odd elements at the end go to
// the first threads of block 0
__device__ __forceinline__ void sgd_range(void* p, const void* g, long long n, float lr, float wd, int fp16, int lb, int nb) {
  const long long nvec = n >> 3;
  uint4* pv = reinterpret_cast<uint4*>(p);
  const uint4* gv = reinterpret_cast<const uint4*>(g);
  for (long long i = static_cast<long long>(lb) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(nb) * blockDim.x) {
    const uint4 a = pv[i];
    const uint4 b = __ldg(gv + i);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 pf = unpack2(aw[q], fp16), gf = unpack2(bw[q], fp16);
      o[q] = pack2(pf.x - lr * (gf.x + wd * pf.x), pf.y - lr * (gf.y + wd * pf.y), fp16);
    }
    pv[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // tail (n not a multiple of 8)
  const long long t = (nvec << 3) + threadIdx.x;
  if (lb == 0 && threadIdx.x < 8 && t < n) {
    if (fp16) {
      __half* ph = reinterpret_cast<__half*>(p);
      const float pf = __half2float(ph[t]), gf = __half2float(reinterpret_cast<const __half*>(g)[t]);
      ph[t] = __float2half(pf - lr * (gf + wd * pf));
    } else {
      __nv_bfloat16* pb = reinterpret_cast<__nv_bfloat16*>(p);
      const float pf = __bfloat162float(pb[t]), gf = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[t]);
      pb[t] = __float2bfloat16(pf - lr * (gf + wd * pf));
    }
  }
}

__global__ void __launch_bounds__(256) sgd_step_kernel(void* p, const void* g, long long n, float lr, float wd, int fp16) {
  sgd_range(p, g, n, lr, wd, fp16, blockIdx.x, gridDim.x);
}

// The same step over up to CCF_SGD_MULTI tensors in one launch. A transformer has hundreds of small parameter tensors
// (biases, LayerNorm weights, routers): one launch each costs more in launch gaps than in memory traffic.
__global__ void __launch_bounds__(256) sgd_multi_kernel(const __grid_constant__ CcfSgdMulti a) {
  const int b = blockIdx.x;
  int lo = 0, hi = a.count;  // largest t with first_block[t] <= b
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (a.first_block[mid] <= b) lo = mid; else hi = mid;
  }
  sgd_range(a.p[lo], a.g[lo], a.n[lo], a.lr, a.wd, a.fp16, b - a.first_block[lo], a.first_block[lo + 1] - a.first_block[lo]);
}

// ---------------------------------------------------------------------------------------------------
// On-stream barrier of the ranks of a group: everything this rank issued before it on the stream is complete and
// visible at system scope before any rank passes. One warp; rank r stores the call's epoch into element r of every
// rank's flag array and waits (bounded) until its own array holds the epoch in every element. Not on the layer's hot
// path (tile counters and completion counters order the data there); meant for set-up, tear-down and for users who
// recycle buffers themselves. Stands in for nvshmemx_barrier_all_on_stream (mix_moe/csrc/mix_moe.h:271,336,420,467).
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) flag_barrier_kernel(const __grid_constant__ CcfBarrierArgs a) {
  const int tid = threadIdx.x;
  __threadfence_system();
  if (tid < a.world) st_release_sys(a.peer_flag[tid] + a.my_rank, a.epoch);
  if (tid < a.world) {
    if (!wait_flag_ge(a.peer_flag[a.my_rank] + tid, a.epoch, fail_fast_limit(a.status, a.wait_limit_ns)))
      report_status(a.status, CCF_ERR_FLAG_TIMEOUT, 0x900000 | tid);
  }
}

// A wait that nothing satisfies unless `flag` already holds `target`: used to exercise the timeout path.
__global__ void wait_probe_kernel(const int* flag, int target, unsigned long long limit_ns, int* status) {
  if (!wait_flag_ge(flag, target, limit_ns)) report_status(status, CCF_ERR_FLAG_TIMEOUT, 0x123);
}

}  // namespace ccf

// ---------------------------------------------------------------------------------------------------
// C entry points
// ---------------------------------------------------------------------------------------------------
extern "C" {

static int last_err() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

int ccf_topk_softmax(const void* logits, int fp16, int is_f32, int T, int E, int K, int* idx, float* w, void* stream) {
  if (E > 256 || K > 8 || K < 1 || K > E) return -2;
  if (T == 0) return 0;
  const int threads = 256, blocks = (T * 32 + threads - 1) / threads;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (E <= 64) ccf::topk_softmax_kernel<2><<<blocks, threads, 0, st>>>(logits, fp16, is_f32, T, E, K, idx, w);
  else if (E <= 128) ccf::topk_softmax_kernel<4><<<blocks, threads, 0, st>>>(logits, fp16, is_f32, T, E, K, idx, w);
  else ccf::topk_softmax_kernel<8><<<blocks, threads, 0, st>>>(logits, fp16, is_f32, T, E, K, idx, w);
  return last_err();
}

int ccf_topk_softmax_bwd(const int* idx, const float* w, const float* dw, int T, int E, int K, void* dlogits, int fp16,
                         int is_f32, void* stream) {
  if (T == 0) return 0;
  ccf::topk_softmax_bwd_kernel<<<(T + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      idx, w, dw, T, E, K, dlogits, fp16, is_f32);
  return last_err();
}

// scratch: block_hist [nb*E] + block_off [nb*E] ints, ticket 1 int (zero before the first call)
static int route_impl(const int* expert, int S, int E, int cap, int* pos, int* block_hist, int* block_off,
                      int* count_raw, int* count_kept, int* ticket, int* order_off, int* sorted_slot, int* slot_row,
                      int first_expert, void* stream) {
  if (E > CCF_MAX_GROUPS) return -2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (S == 0) {
    // a call without tokens on this rank still takes part in the count exchange: its counts are zero, not stale
    cudaMemsetAsync(count_raw, 0, sizeof(int) * E, st);
    cudaMemsetAsync(count_kept, 0, sizeof(int) * E, st);
    if (order_off != nullptr) cudaMemsetAsync(order_off, 0, sizeof(int) * (E + 1), st);
    return last_err();
  }
  const int nb = (S + ccf::kRouteBlock - 1) / ccf::kRouteBlock;
  ccf::route_hist_kernel<<<nb, ccf::kRouteBlock, 0, st>>>(expert, S, E, cap, pos, block_hist, block_off, count_raw,
                                                          count_kept, ticket, order_off, first_expert);
  ccf::route_pos_kernel<<<(S + 255) / 256, 256, 0, st>>>(expert, S, E, block_off, pos, cap, order_off, sorted_slot,
                                                         slot_row);
  return last_err();
}

int ccf_route(const int* expert, int S, int E, int cap, int* pos, int* block_hist, int* block_off, int* count_raw,
              int* count_kept, int* ticket, void* stream) {
  return route_impl(expert, S, E, cap, pos, block_hist, block_off, count_raw, count_kept, ticket, nullptr, nullptr,
                    nullptr, 0, stream);
}

// Same, and also the destination order of the kept slots: order_off [E + 1] (order_off[E] = kept rows in total),
// sorted_slot [S] (slot id at each position of that order), slot_row [S] set to -1 for dropped slots.
int ccf_route_ordered(const int* expert, int S, int E, int cap, int* pos, int* block_hist, int* block_off,
                      int* count_raw, int* count_kept, int* ticket, int* order_off, int* sorted_slot, int* slot_row,
                      int first_expert, void* stream) {
  return route_impl(expert, S, E, cap, pos, block_hist, block_off, count_raw, count_kept, ticket, order_off,
                    sorted_slot, slot_row, first_expert, stream);
}

int ccf_sizeof_plan_args() { return static_cast<int>(sizeof(ccf::PlanArgs)); }

int ccf_plan(const ccf::PlanArgs* a, void* stream) {
  if (a->e_total > CCF_MAX_GROUPS || a->world > CCF_MAX_RANKS) return -2;
  ccf::plan_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  return last_err();
}

// epoch_counter: one int in device memory, equal on every rank of the group, advanced by one per call
int ccf_plan_dev_epoch(const ccf::PlanArgs* a, int* epoch_counter, void* stream) {
  if (a->e_total > CCF_MAX_GROUPS || a->world > CCF_MAX_RANKS || epoch_counter == nullptr) return -2;
  ccf::plan_kernel_dev_epoch<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a, epoch_counter);
  return last_err();
}

int ccf_dispatch(const CcfDispatchArgs* a, int* status, int* done_ctas, int grid, void* stream) {
  if (a->d % 8 != 0) return -2;
  if (grid <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    grid = sms * 2;
  }
  ccf::dispatch_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a, status, done_ctas);
  return last_err();
}

int ccf_combine_wait(const int* done, int* cum, const int* sent_rows, int n_tiles, int world,
                     unsigned long long limit_ns, int* status, void* stream) {
  ccf::combine_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(done, cum, sent_rows, n_tiles, world,
                                                                                 limit_ns, status);
  return last_err();
}

int ccf_combine_reduce(const void* comb, const int* slot_row, void* y, int T, int K, int d, int fp16, void* stream) {
  if (d % 8 != 0) return -2;
  if (T == 0) return 0;
  const long long pieces = static_cast<long long>(T) * (d >> 3);
  const int threads = 256;
  const long long blocks = (pieces + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return -2;
  ccf::combine_reduce_kernel<<<static_cast<unsigned>(blocks), threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      comb, slot_row, y, T, K, d, fp16);
  return last_err();
}

int ccf_colsum_grouped(const void* x, long long ld, int n, int groups, const int* group_base, const int* group_rows,
                       void* out, int fp16, void* stream) {
  if (n % 8 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;   // 16-byte loads
  dim3 grid((n + 127) / 128, groups);
  ccf::colsum_grouped_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, ld, n, group_base,
                                                                                        group_rows, out, fp16);
  return last_err();
}

int ccf_sgd_step(void* p, const void* g, long long n, float lr, float wd, int fp16, void* stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15) return -2;
  long long blocks = ((n >> 3) + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ccf::sgd_step_kernel<<<static_cast<int>(blocks), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p, g, n, lr, wd, fp16);
  return last_err();
}

int ccf_sizeof_sgd_multi() { return static_cast<int>(sizeof(CcfSgdMulti)); }

// a->first_block must be filled: first_block[0] = 0, non-decreasing, at least one block per tensor
int ccf_sgd_multi(const CcfSgdMulti* a, void* stream) {
  if (a->count < 1 || a->count > CCF_SGD_MULTI) return -2;
  uintptr_t bits = 0;
  for (int t = 0; t < a->count; ++t) {
    bits |= reinterpret_cast<uintptr_t>(a->p[t]) | reinterpret_cast<uintptr_t>(a->g[t]);
    if (a->n[t] <= 0 || a->first_block[t + 1] <= a->first_block[t]) return -3;
  }
  if ((bits & 15) || a->first_block[0] != 0) return -2;
  ccf::sgd_multi_kernel<<<a->first_block[a->count], 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  return last_err();
}

int ccf_sizeof_barrier_args() { return static_cast<int>(sizeof(CcfBarrierArgs)); }

int ccf_flag_barrier(const CcfBarrierArgs* a, void* stream) {
  if (a->world < 1 || a->world > CCF_MAX_RANKS || a->my_rank < 0 || a->my_rank >= a->world) return -2;
  ccf::flag_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*a);
  return last_err();
}

int ccf_wait_probe(const int* flag, int target, unsigned long long limit_ns, int* status, void* stream) {
  ccf::wait_probe_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, target, limit_ns, status);
  return last_err();
}

// ---- symmetric memory: plain device allocations shared through CUDA IPC ------------------------------
// The allocator stands in for nvshmem_malloc of the reference (mix_moe/csrc/mix_moe.h:75-77): every rank
// allocates the same size, exports a handle, and maps every peer's allocation, which gives the
// peer_base[rank] table the kernels index (the role of NVSHMEM's peer_heap_base).
int ccf_symm_alloc(unsigned long long bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return -static_cast<int>(e);
  e = cudaMemset(*ptr, 0, bytes);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
int ccf_symm_free(void* ptr) { return -static_cast<int>(cudaFree(ptr)); }
int ccf_symm_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
int ccf_symm_get_handle(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return -static_cast<int>(e);
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
int ccf_symm_open_handle(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
int ccf_symm_close_handle(void* ptr) { return -static_cast<int>(cudaIpcCloseMemHandle(ptr)); }

const char* ccf_error_string(int neg_code) { return cudaGetErrorString(static_cast<cudaError_t>(-neg_code)); }

}  // extern "C"
