// ccf_route_noalloc: the routing-plan kernels with their scratch memory inside the library.
// See no_alloc.h for who this is for, the size limits and the rules of use.
#include <cuda_runtime.h>

#include "no_alloc.h"

namespace {

constexpr int kBlock = 1024;
constexpr int kMaxDevices = 64;

// Scratch shared by every call on this device: [block_hist | block_off | ticket]. In host code this name is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) int g_route_scratch[CCF_NOALLOC_SCRATCH_INTS];

// Per-block histogram and in-block positions; the last block to finish scans the histograms.
__global__ void __launch_bounds__(kBlock)
noalloc_hist_kernel(const int* __restrict__ expert, int S, int E, int cap, int* pos, int* block_hist, int* block_off,
                    int* count_raw, int* count_kept, int* ticket) {
  __shared__ int wh[32][CCF_NOALLOC_MAX_EXPERTS];
  __shared__ int is_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = gridDim.x;
  for (int i = tid; i < 32 * CCF_NOALLOC_MAX_EXPERTS; i += kBlock) (&wh[0][0])[i] = 0;
  __syncthreads();
  const int s = blockIdx.x * kBlock + tid;
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
  }
}

__global__ void noalloc_pos_kernel(const int* __restrict__ expert, int S, int E, const int* __restrict__ block_off,
                                   int* pos) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const int e = expert[s];
  if (e >= 0 && e < E) pos[s] += block_off[(s / kBlock) * E + e];
}

// device address of g_route_scratch, looked up once per device
int* g_scratch_addr[kMaxDevices] = {nullptr};

int* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_route_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // leave no sticky error behind
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<int*>(p);
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int ccf_route_noalloc(const int* expert, int S, int E, int cap, int* pos, int* count_raw, int* count_kept,
                                 void* stream) {
  if (S < 0 || S > CCF_NOALLOC_MAX_SLOTS || E < 1 || E > CCF_NOALLOC_MAX_EXPERTS) return CCF_NOALLOC_ERR_SIZE;
  if (!count_raw || !count_kept || (S > 0 && (!expert || !pos))) return CCF_NOALLOC_ERR_ARG;
  int* scratch = scratch_for_current_device();
  if (!scratch) return CCF_NOALLOC_ERR_SETUP;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* block_hist = scratch;
  int* block_off = scratch + CCF_NOALLOC_MAX_BLOCKS * CCF_NOALLOC_MAX_EXPERTS;
  int* ticket = scratch + 2 * CCF_NOALLOC_MAX_BLOCKS * CCF_NOALLOC_MAX_EXPERTS;
  if (S == 0) {
    // nothing routed: the counts are all zero
    if (cudaMemsetAsync(count_raw, 0, sizeof(int) * E, st) != cudaSuccess) return CCF_NOALLOC_ERR_LAUNCH;
    if (cudaMemsetAsync(count_kept, 0, sizeof(int) * E, st) != cudaSuccess) return CCF_NOALLOC_ERR_LAUNCH;
    return 0;
  }
  // the ticket must start at zero whatever an earlier call left in the shared array
  if (cudaMemsetAsync(ticket, 0, sizeof(int), st) != cudaSuccess) return CCF_NOALLOC_ERR_LAUNCH;
  const int nb = (S + kBlock - 1) / kBlock;
  noalloc_hist_kernel<<<nb, kBlock, 0, st>>>(expert, S, E, cap, pos, block_hist, block_off, count_raw, count_kept,
                                             ticket);
  noalloc_pos_kernel<<<(S + 255) / 256, 256, 0, st>>>(expert, S, E, block_off, pos);
  return cudaGetLastError() == cudaSuccess ? 0 : CCF_NOALLOC_ERR_LAUNCH;
}

extern "C" const char* ccf_route_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case CCF_NOALLOC_ERR_SIZE:
      return "ccf_route_noalloc: S must be in [0, 65536] and E in [1, 256] (fixed scratch array); use ccf_route with "
             "caller-provided scratch for larger problems";
    case CCF_NOALLOC_ERR_ARG: return "ccf_route_noalloc: null input or output pointer";
    case CCF_NOALLOC_ERR_SETUP: return "ccf_route_noalloc: cudaGetSymbolAddress failed for the scratch array on the current device";
    case CCF_NOALLOC_ERR_LAUNCH: return "ccf_route_noalloc: the CUDA runtime refused a memset or a kernel launch";
    default: return "ccf_route_noalloc: unknown error code";
  }
}
