// Dispatch role: push routed token rows straight into the expert input buffers of their owner GPUs
// (peer stores over NVLink, plain 16-byte vector stores, never TMA multicast) and bump the arrival
// counter of the 128-row tile each row lands in. The same device function is used by the stand-alone
// dispatch kernel and by the first CTAs of the fused dispatch+GEMM kernel.
//
// Replaces _local_scatter_kernel + nvshmemx_get16_nbi_block of the reference
// (mix_moe/csrc/cuda/mix_moe_kernel.cu:18-33, mix_moe/csrc/cuda/mix_gemm.cu:304-307): the reference sorts
// rows locally and lets the owner pull 64-row blocks after a global barrier; here the source pushes
// and the owner's GEMM starts tile by tile as the counters fill, with no barrier.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "gemm_args.h"
#include "sm100.cuh"

namespace ccf {

// First hard error wins the status word; an overflow (rows dropped because a receive buffer is full) is only a note
// and is recorded in the second word so that it can neither hide nor be hidden by a time-out.
__device__ __forceinline__ void report_status(int* status, int code, int detail) {
  if (!status) return;
  if (code == CCF_ERR_OVERFLOW) atomicAdd(status + 1, 1);
  else atomicCAS(status, 0, (detail << 8) | code);
}

// Once a time-out (or any other hard error) is on record, later waits give up after a millisecond instead of their
// full limit, so one lost peer costs one limit, not one limit per kernel. An overflow is not a reason to hurry.
__device__ __forceinline__ unsigned long long fail_fast_limit(const int* status, unsigned long long limit_ns) {
  if (status != nullptr) {
    const int code = *reinterpret_cast<const volatile int*>(status) & 0xff;
    if (code == CCF_ERR_MBAR_TIMEOUT || code == CCF_ERR_FLAG_TIMEOUT) return 1000000ull;
  }
  return limit_ns;
}

__device__ __forceinline__ float2 unpack2(uint32_t u, int fp16) {
  if (fp16) {
    __half2 h = *reinterpret_cast<__half2*>(&u);
    return __half22float2(h);
  }
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(b);
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int fp16) {
  if (fp16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One warp works on chunks of kChunk consecutive positions of the destination order (rows of this rank's own experts
// first, then the next owner's, ...; inside an expert in position order), claimed from a shared counter. Consecutive
// positions land on consecutive rows of one receive buffer, so tiles fill up one after the other: the owner's GEMM can
// start on its first tiles while later rows are still being pushed, and all sources start with a different owner.
// Claiming is dynamic on purpose: only warps that are running push rows. With a static assignment a CTA that cannot
// start yet (its SM is held by another kernel, e.g. a collective of the data-parallel all-reduce that itself waits for
// a peer) would hold back rows that other GPUs wait for. The next claim is issued before the current chunk is
// processed so the atomic's round trip is off the critical path.
// Not inlined, and one instantiation per direction: the role keeps kChunk rows' worth of pointers and data in registers
// (the backward form twice as much), which must not be added to the register budget of the GEMM roles it shares a
// kernel with (168 registers per thread at 320 threads).
template <int kChunk, bool kBackward>
__device__ __noinline__ void dispatch_rows(const CcfDispatchArgs& a, int* status) {
  static_assert(kChunk <= 16, "one lane per row of a chunk; rows of a chunk are held in registers");
  // Scalars used inside the copy loops are read once: `a` arrives by reference, so the compiler must assume that the
  // row stores below may alias it and would otherwise reload them after every store.
  const int e_total = a.e_total;
  const int fp16 = a.fp16, top_k = a.top_k, my_rank = a.my_rank, experts_per_rank = a.experts_per_rank;
  const int capacity = a.capacity, max_rows = a.max_rows, total_index = a.total_index;
  float* const dgate = a.dgate;
  const void* const saved_comb = a.saved_comb;
  const void* const x_rows = a.x;
  const int kept = a.order_off[e_total];   // rows to push
  const int lane = threadIdx.x & 31;
  const int vecs = a.d >> 3;  // 16-byte vectors per row
  const int n_chunks = (kept + kChunk - 1) / kChunk;
  int c_next = 0;
  if (lane == 0) c_next = atomicAdd(a.work_counter, 1);
  for (;;) {
    const int c = __shfl_sync(0xffffffffu, c_next, 0);
    if (c >= n_chunks) break;
    if (lane == 0) c_next = atomicAdd(a.work_counter, 1);
    const int i0 = c * kChunk;
    const int ns = min(kChunk, kept - i0);
    // lane i plans the row at position i0 + i of the destination order
    int my_row = -1, my_owner = 0, my_slot = 0;
    float my_gate = 0.f;
    if (lane < ns) {
      const int s = a.sorted_slot[i0 + lane];
      my_slot = s;
      const int e = a.slot_expert[s];
      const int p = a.slot_pos[s];
      my_gate = a.slot_gate[s];
      my_owner = e / experts_per_rank;
      my_row = a.dst_base[e] + p;
      if (my_row < 0 || my_row >= max_rows || my_owner >= CCF_MAX_RANKS || p >= capacity) {
        // beyond the owner's buffer: dropped on both sides (the plan did not count it)
        if (p < capacity) report_status(status, CCF_ERR_OVERFLOW, s & 0xffffff);
        my_row = -1;
      }
      if (a.slot_row) a.slot_row[s] = my_row;
      if (my_row >= 0) {
        a.peer_row_src[my_owner][my_row] = (my_rank << 24) | s;
        a.peer_row_gate[my_owner][my_row] = my_gate;
      } else if (kBackward && dgate) {
        dgate[s] = 0.f;
      }
    }
    // Source and destination of the chunk's rows (null = dropped or past the end). All kChunk rows are
    // copied together, one 16-byte column at a time, so kChunk independent loads are in flight per lane
    // (one row at a time made the copy latency-bound: ~2 us per row and warp).
    const uint4* src[kChunk];
    uint4* dst[kChunk];
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      const int row = __shfl_sync(0xffffffffu, my_row, i);
      const int owner = __shfl_sync(0xffffffffu, my_owner, i);
      const bool on = i < ns && row >= 0;
      const int t = __shfl_sync(0xffffffffu, my_slot, i) / top_k;
      src[i] = on ? reinterpret_cast<const uint4*>(x_rows) + static_cast<size_t>(t) * vecs : nullptr;
      dst[i] = on ? reinterpret_cast<uint4*>(a.peer_recv[owner]) + static_cast<size_t>(row) * vecs : nullptr;
    }
    if constexpr (!kBackward) {
      // kU column steps at a time, so that kChunk * kU = 8 loads are in flight per lane whatever the chunk size: with
      // few rows to push (small chunks, see dispatch_role) the copy of a row is then a few memory latencies, not d / 256
      constexpr int kU = 8 / kChunk > 0 ? 8 / kChunk : 1;
      for (int v0 = lane; v0 < vecs; v0 += 32 * kU) {
        uint4 r[kChunk][kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int v = v0 + 32 * u;
#pragma unroll
          for (int i = 0; i < kChunk; ++i)
            if (src[i] && v < vecs) r[i][u] = __ldg(src[i] + v);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int v = v0 + 32 * u;
#pragma unroll
          for (int i = 0; i < kChunk; ++i)
            if (dst[i] && v < vecs) dst[i][v] = r[i][u];
        }
      }
    } else {
      // rows of the backward pass carry g * dy; the gate gradient is <dy, saved scaled output> / g
      float dot[kChunk], g[kChunk];
      int slot[kChunk];
      const uint4* sv[kChunk];
#pragma unroll
      for (int i = 0; i < kChunk; ++i) {
        dot[i] = 0.f;
        g[i] = __shfl_sync(0xffffffffu, my_gate, i);
        slot[i] = __shfl_sync(0xffffffffu, my_slot, i);
        sv[i] = (src[i] && saved_comb)
                    ? reinterpret_cast<const uint4*>(saved_comb) + static_cast<size_t>(slot[i]) * vecs
                    : nullptr;
      }
      for (int v = lane; v < vecs; v += 32) {
        uint4 xr[kChunk], cr[kChunk];
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
          if (src[i]) xr[i] = __ldg(src[i] + v);
          cr[i] = sv[i] ? __ldg(sv[i] + v) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < kChunk; ++i) {
          if (!dst[i]) continue;
          const uint32_t xi[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
          const uint32_t ci[4] = {cr[i].x, cr[i].y, cr[i].z, cr[i].w};
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 xf = unpack2(xi[q], fp16);
            const float2 cf = unpack2(ci[q], fp16);
            dot[i] += xf.x * cf.x + xf.y * cf.y;
            o[q] = pack2(xf.x * g[i], xf.y * g[i], fp16);
          }
          dst[i][v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
#pragma unroll
      for (int i = 0; i < kChunk; ++i) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot[i] += __shfl_xor_sync(0xffffffffu, dot[i], off);
        if (lane == 0 && dst[i] && dgate) dgate[slot[i]] = (g[i] != 0.f) ? dot[i] / g[i] : 0.f;
      }
    }
    // The counters move with release semantics at system scope after a warp barrier: the barrier orders the other
    // lanes' row stores before this lane's release, which makes them visible before the counter value.
    __syncwarp();
    // Rows that stay on this GPU only need device scope (the consumer is a CTA of this GPU); a system-scope
    // release costs several microseconds more per chunk.
    const bool sent = lane < ns && my_row >= 0;
    const bool all_local = __all_sync(0xffffffffu, !sent || my_owner == my_rank);
    // rows of a chunk mostly share one tile: one counter update per distinct (owner, tile)
    const int key = sent ? ((my_owner << 24) | (my_row >> 7)) : -1;
    const unsigned same_tile = __match_any_sync(0xffffffffu, key);
    if (sent && lane == __ffs(same_tile) - 1) {
      int* flag = a.peer_tile_flags[my_owner] + (my_row >> 7);
      if (all_local) red_release_gpu_add(flag, __popc(same_tile)); else red_release_sys_add(flag, __popc(same_tile));
    }
    if (total_index >= 0) {
      // one add per distinct owner of the chunk to that owner's count of all arrived rows
      const unsigned same = __match_any_sync(0xffffffffu, sent ? my_owner : -1);
      if (sent && lane == __ffs(same) - 1) {
        int* tot = a.peer_tile_flags[my_owner] + total_index;
        if (all_local) red_release_gpu_add(tot, __popc(same)); else red_release_sys_add(tot, __popc(same));
      }
    }
  }
}

}  // namespace ccf
