// Pieces shared by the one-CTA (gemm.cu) and two-CTA (gemm2.cu) grouped GEMM kernels: tile geometry, epilogue
// arithmetic, staged row I/O, the per-tile epilogue and the optional trace.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "dispatch.cuh"
#include "gemm_args.h"
#include "sm100.cuh"

namespace ccf {

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int kEpiWarps = 8;            // two per TMEM lane quarter, each takes half of the columns
// Two more warps per CTA exist only for the dispatch role: with them the row push runs next to the MMA and epilogue warps
// (which start on the tiles made of this rank's own rows) instead of in front of the epilogue.
constexpr int kCommWarps = 2;
constexpr int kThreads = 64 + 32 * kEpiWarps + 32 * kCommWarps;
constexpr int kTmemCols = 512;
constexpr int MAJ_K = 0, MAJ_MN = 1;
constexpr int kEpiStageBytes = 2048;  // per epilogue warp: 32 rows x 64 bytes, XOR-swizzled

// Host: tensor map of a 2-D row-major view [rows, cols] of 2-byte elements with box {box_cols, box_rows} and 128-byte
// swizzle (defined in gemm.cu). Returns 0 or a negative error code.
int make_tmap(CUtensorMap* m, const void* base, long long rows, long long cols, int box_cols, int box_rows, int fp16);

struct Tile {
  int g;           // group (expert)
  int row0;        // row-grouped: first A/C row; k-grouped: first output row inside the group (m0)
  int n0;          // first output column (for SWIGLU: first *output* column, 128 per tile)
  int rows_valid;  // valid rows of the tile
  int kblocks;     // 64-deep reduction steps
  int krow0;       // k-grouped: first reduction row
};

// ---------------------------------------------------------------------------------------------------
// epilogue math
// ---------------------------------------------------------------------------------------------------
// erf as an odd polynomial: erf(z) ~= z * P(z^2) on |z| <= 3 (degree 8 in z^2, fitted minimax-style; |error| <= 2.6e-5
// in fp32 Horner form, erf(3) = 1 - 2.2e-5 beyond the clamp), far below bf16 / fp16 resolution. No MUFU operation and
// no branch: libm's erff and the exp/rcp-based forms kept the SFU pipe busy for ~4 k cycles per 128x256 tile.
__device__ __forceinline__ float erf_poly(float z) {
  z = fminf(fmaxf(z, -3.f), 3.f);
  const float u = z * z;
  float p = 4.074189994e-08f;
  p = fmaf(p, u, -1.944814854e-06f);
  p = fmaf(p, u, 4.106040073e-05f);
  p = fmaf(p, u, -5.110358431e-04f);
  p = fmaf(p, u, 4.235422620e-03f);
  p = fmaf(p, u, -2.510284860e-02f);
  p = fmaf(p, u, 1.110793178e-01f);
  p = fmaf(p, u, -3.753148649e-01f);
  p = fmaf(p, u, 1.128268424e+00f);
  return p * z;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // branch-free, 1 ulp: keeps the element loops interleavable
  return y;
}
__device__ __forceinline__ float gelu_f(float x) {
  const float hx = 0.5f * x;
  return fmaf(hx, erf_poly(x * 0.70710678118654752f), hx);
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float cdf = fmaf(0.5f, erf_poly(x * 0.70710678118654752f), 0.5f);
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return fmaf(x, pdf, cdf);
}
// The activation switch sits outside the element loop: with a branch per element the compiler cannot
// interleave the 32 independent dependency chains and the epilogue ran ~200 clocks per element.
__device__ __forceinline__ void act32(float (&f)[32], int act) {
  if (act == CCF_ACT_GELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = gelu_f(f[i]);
  } else if (act == CCF_ACT_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = fmaxf(f[i], 0.f);
  }
}
// f[i] *= act'(pz[i])
__device__ __forceinline__ void act_grad32(float (&f)[32], const float (&pz)[32], int act) {
  if (act == CCF_ACT_GELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] *= gelu_grad_f(pz[i]);
  } else if (act == CCF_ACT_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = pz[i] > 0.f ? f[i] : 0.f;
  }
}

// 32 consecutive 2-byte elements -> floats (64 bytes, 16-byte aligned)
__device__ __forceinline__ void load32(const void* p, float (&f)[32], int fp16) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v = __ldg(q + i);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack2(w[j], fp16);
      f[i * 8 + j * 2] = t.x;
      f[i * 8 + j * 2 + 1] = t.y;
    }
  }
}

__device__ __forceinline__ void store32(void* p, const float (&f)[32], int fp16) {
  uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 v;
    v.x = pack2(f[i * 8 + 0], f[i * 8 + 1], fp16);
    v.y = pack2(f[i * 8 + 2], f[i * 8 + 3], fp16);
    v.z = pack2(f[i * 8 + 4], f[i * 8 + 5], fp16);
    v.w = pack2(f[i * 8 + 6], f[i * 8 + 7], fp16);
    q[i] = v;
  }
}

__device__ __forceinline__ void store32_f32(float* p, const float (&f)[32]) {
  float4* q = reinterpret_cast<float4*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = make_float4(f[i * 4], f[i * 4 + 1], f[i * 4 + 2], f[i * 4 + 3]);
}

// 32 bias values as raw 16-byte words (same address for every lane: a broadcast load), applied later so that the
// load latency of chunk c+1 hides behind the math of chunk c
__device__ __forceinline__ void load_bias_raw(const void* bias, size_t elem_off, uint4 (&raw)[4]) {
  const uint4* q = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(bias) + elem_off);
#pragma unroll
  for (int i = 0; i < 4; ++i) raw[i] = __ldg(q + i);
}
__device__ __forceinline__ void add_bias_raw(float (&f)[32], const uint4 (&raw)[4], int fp16) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack2(w[j], fp16);
      f[i * 8 + j * 2] += t.x;
      f[i * 8 + j * 2 + 1] += t.y;
    }
  }
}

__device__ __forceinline__ void acc_to_float(const uint32_t (&r)[32], float (&f)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
}


// ---------------------------------------------------------------------------------------------------
// Epilogue row I/O through a per-warp shared-memory staging buffer (32 rows x 64 bytes, XOR-swizzled).
// In the TMEM register layout every lane owns one row, so a direct vector store writes 16 bytes to 32
// different rows per instruction: 4096 partial-sector requests per 128x256 tile and output, which capped
// the tensor pipe at ~46 % for two-output epilogues. Staged, each instruction moves 8 rows x 64 contiguous
// bytes (full 32-byte sectors). Lane l owns row l; `row_ptr` is the global address of this lane's
// 64-byte segment (0 = skip the row).
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t stage_off(int row, int piece) {
  return static_cast<uint32_t>(row * 64 + ((piece ^ ((row >> 1) & 3)) << 4));
}

__device__ __forceinline__ void staged_store64(uint32_t stage, int lane, const uint32_t (&w)[16],
                                               unsigned long long row_ptr) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + stage_off(lane, j)), "r"(w[4 * j]),
                 "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), piece = lane & 3;
    const unsigned long long p = __shfl_sync(0xffffffffu, row_ptr, row);
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(stage + stage_off(row, piece))
                 : "memory");
    if (p != 0ull) *reinterpret_cast<uint4*>(p + piece * 16) = v;
  }
  __syncwarp();
}

__device__ __forceinline__ void pack32(const float (&f)[32], uint32_t (&w)[16], int fp16) {
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = pack2(f[2 * i], f[2 * i + 1], fp16);
}
__device__ __forceinline__ void unpack32(const uint32_t (&w)[16], float (&f)[32], int fp16) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 t = unpack2(w[i], fp16);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
// byte address of element (row, col) of a 2-byte matrix with leading dimension ld
__device__ __forceinline__ unsigned long long addr2(const void* base, long long row, long long ld, int col) {
  return reinterpret_cast<unsigned long long>(base) + static_cast<unsigned long long>((row * ld + col) * 2);
}

// Optional per-tile trace: slot `ev` of tile number `seq` of this CTA gets the SM clock (clock64).
__device__ __forceinline__ void trace_ev(const CcfGemmArgs& a, int seq, int ev) {
  if (a.trace != nullptr && seq < a.trace_tiles)
    a.trace[(static_cast<size_t>(blockIdx.x) * a.trace_tiles + seq) * 8 + ev] = clock64();
}


// ---------------------------------------------------------------------------------------------------
// Epilogue of one accumulator tile for one epilogue warp: lane l owns tile row q*32 + l, the warp covers
// n_chunks chunks of 32 columns starting at chunk `half * n_chunks`. Shared by the one-CTA and the two-CTA kernels.
//   row_base     first output row of this CTA's 128 accumulator rows (group offset included for k-grouped mode)
//   rows_valid   rows of this CTA's part that hold data
//   rows_store   rows of this CTA's part that may be written at all (rows in [rows_valid, rows_store) get zeros)
// Returns where the row went (COMBINE) so that the caller can report completion after releasing the accumulator.
// ---------------------------------------------------------------------------------------------------
struct CombineDest {
  int rank;
  bool ok;
};

// In-place SGD epilogue (STORE with sgd_lr != 0): the weights under the tile are read before they are rewritten. One
// 32-column chunk of a warp's 32 rows is 2 KB, so a warp that asked for it only when it needed it kept 16 KB per SM in
// flight and the kernel ran at the latency of a DRAM read per chunk. sgd_prefetch_l2 asks L2 for this lane's row of the
// tile part as soon as the tile is known (before its accumulator is complete); sgd_fetch_lin reads one chunk in the layout
// of the staged accesses (row 8 i + lane / 4, piece lane % 4) into registers one chunk ahead of its use. Measured on the
// 64-expert GPT-MoE step: asking for the NEXT tile's weights instead, or reading two chunks ahead, was slower than this.
__device__ __forceinline__ void sgd_prefetch_l2(const CcfGemmArgs& args, long long row_base, int n0, int rows_valid, int q,
                                                int half, int lane) {
  const int r_in_tile = q * 32 + lane;
  if (r_in_tile >= rows_valid) return;
  const int n_chunks = args.bn == 128 ? 2 : 4;
  const int n = n0 + half * n_chunks * 32;
  if (n >= args.n) return;
  const char* p = reinterpret_cast<const char*>(args.out0) + (static_cast<size_t>(row_base + r_in_tile) * args.ld_out + n) * 2;
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
  if (n_chunks == 4 && n + 64 < args.n) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + 128));
}
// Staged accesses for rows that lie one after the other in memory (every epilogue but COMBINE: row r of the warp's 32
// rows is at base + r * stride, the first rows_ok of them exist). The addresses are computed, not shuffled from the lane
// that owns the row: eight shuffles fewer per staged access, 15 % of the time of a launch that is bound by its epilogue.
__device__ __forceinline__ void sgd_fetch_lin(unsigned long long base, unsigned long long stride, int rows_ok, int lane,
                                              uint4 (&v)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), piece = lane & 3;
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_ok) v[i] = *reinterpret_cast<const uint4*>(base + row * stride + piece * 16);
  }
}
__device__ __forceinline__ void staged_load64_lin(uint32_t stage, int lane, uint32_t (&w)[16], unsigned long long base,
                                                  unsigned long long stride, int rows_ok) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), piece = lane & 3;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_ok) v = __ldg(reinterpret_cast<const uint4*>(base + row * stride + piece * 16));
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + stage_off(row, piece)), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3])
                 : "r"(stage + stage_off(lane, j))
                 : "memory");
  }
  __syncwarp();
}
__device__ __forceinline__ void staged_store64_lin(uint32_t stage, int lane, const uint32_t (&w)[16], unsigned long long base,
                                                   unsigned long long stride, int rows_ok) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + stage_off(lane, j)), "r"(w[4 * j]),
                 "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), piece = lane & 3;
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(stage + stage_off(row, piece))
                 : "memory");
    if (row < rows_ok) *reinterpret_cast<uint4*>(base + row * stride + piece * 16) = v;
  }
  __syncwarp();
}
// the chunk fetched by sgd_fetch, transposed through the warp's staging area into one row per lane
__device__ __forceinline__ void sgd_unstage(uint32_t stage, int lane, const uint4 (&v)[4], uint32_t (&w)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), piece = lane & 3;
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + stage_off(row, piece)), "r"(v[i].x), "r"(v[i].y),
                 "r"(v[i].z), "r"(v[i].w)
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3])
                 : "r"(stage + stage_off(lane, j))
                 : "memory");
  }
  __syncwarp();
}

template <int kEpi>
__device__ __forceinline__ CombineDest epilogue_tile(const CcfGemmArgs& args, const Tile& ti, long long row_base,
                                                     int rows_valid, int rows_store, bool have_acc, uint32_t t_row,
                                                     uint32_t stage, int q, int half, int lane) {
  const int fp16 = args.fp16;
  const int r_in_tile = q * 32 + lane;
  const bool valid = r_in_tile < rows_valid;
  const long long orow = row_base + r_in_tile;

  // COMBINE: where this row goes
  int c_rank = 0, c_slot = 0;
  float c_gate = 1.f;
  bool c_ok = false;
  if constexpr (kEpi == CCF_EPI_COMBINE) {
    if (valid) {
      const int packed = args.row_src[orow];
      c_rank = (packed >> 24) & 0xff;
      c_slot = packed & 0xffffff;
      c_gate = args.row_gate ? args.row_gate[orow] : 1.f;
      c_ok = c_rank < args.world && c_slot < args.max_slots;
      if (!c_ok) report_status(args.status, CCF_ERR_BOUNDS, static_cast<int>(orow) & 0xffffff);
    }
  }

  // chunks of 32 accumulator columns; this warp takes n_chunks of them starting at chunk0
  // 32-column chunks per warp: half of a 256-column tile (or of the 128 output columns of a SwiGLU tile, or of a
  // 128-column narrow tile)
  const int n_chunks = (kEpi == CCF_EPI_SWIGLU || args.bn == 128) ? 2 : 4;
  const int chunk0 = half * n_chunks;
  uint32_t racc[32];  // one buffer: the next chunk is requested right after this one is copied out to f[]
  if (have_acc) tmem_ld32(t_row + chunk0 * 32, racc);
  constexpr bool kBias0Prefetch = (kEpi == CCF_EPI_STORE || kEpi == CCF_EPI_BIAS_ACT || kEpi == CCF_EPI_COMBINE);
  uint4 bcur[4], bnext[4];
  const bool has_b0 = kBias0Prefetch && args.bias0 != nullptr;
  if (has_b0 && ti.n0 + chunk0 * 32 < args.n)
    load_bias_raw(args.bias0, static_cast<size_t>(ti.g) * args.n + ti.n0 + chunk0 * 32, bnext);
  // in-place SGD never carries a bias (the host refuses the combination): the bias registers hold the weights' chunks
  const bool sgd = kEpi == CCF_EPI_STORE && args.sgd_lr != 0.f && !args.out_fp32;
  // every epilogue but COMBINE: the warp's 32 rows follow each other in the output and auxiliary matrices; the first
  // lin_rows of them hold data, the first lin_rows_store may be written (zeros beyond the data)
  const unsigned long long lin_stride = static_cast<unsigned long long>(args.ld_out) * 2ull;
  const int lin_rows = min(32, max(0, rows_valid - q * 32));
  const int lin_rows_store = min(32, max(0, rows_store - q * 32));
  auto lin_of = [&](const void* p) { return addr2(p, row_base + q * 32, args.ld_out, 0); };
  const unsigned long long lin_base = lin_of(args.out0);
  if (sgd) sgd_fetch_lin(lin_base + (ti.n0 + chunk0 * 32) * 2ull, lin_stride, ti.n0 + chunk0 * 32 < args.n ? lin_rows : 0, lane, bnext);
  // not unrolled: the body is large and every launch pays for fetching the kernel's code once per SM
#pragma unroll 1
  for (int c = 0; c < n_chunks; ++c) {
    const int cg = chunk0 + c;
    const int n = ti.n0 + cg * 32;
    float f[32];
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) bcur[i] = bnext[i];
    if (has_b0 && c + 1 < n_chunks && n + 32 < args.n)
      load_bias_raw(args.bias0, static_cast<size_t>(ti.g) * args.n + n + 32, bnext);
    if (sgd && c + 1 < n_chunks)
      sgd_fetch_lin(lin_base + (n + 32) * 2ull, lin_stride, n + 32 < args.n ? lin_rows : 0, lane, bnext);
    if (have_acc) {
      tmem_ld_wait();
      acc_to_float(racc, f);
      if constexpr (kEpi != CCF_EPI_SWIGLU) {
        // next chunk's TMEM load overlaps this chunk's math and stores
        if (c + 1 < n_chunks) tmem_ld32(t_row + (cg + 1) * 32, racc);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) f[i] = 0.f;
    }
    if constexpr (kEpi == CCF_EPI_SWIGLU) {
      // f = gate pre-activation (accumulator columns cg*32..), u = up pre-activation (+128)
      float u[32];
      if (have_acc) {
        tmem_ld32(t_row + 128 + cg * 32, racc);
        tmem_ld_wait();
        acc_to_float(racc, u);
        if (c + 1 < n_chunks) tmem_ld32(t_row + (cg + 1) * 32, racc);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) u[i] = 0.f;
      }
      if (n < args.n) {
        if (args.bias1) {
          float b[32];
          load32(reinterpret_cast<const uint16_t*>(args.bias1) + static_cast<size_t>(ti.g) * args.n + n, b, fp16);
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] += b[i];
        }
        if (args.bias0) {
          float b[32];
          load32(reinterpret_cast<const uint16_t*>(args.bias0) + static_cast<size_t>(ti.g) * args.n + n, b, fp16);
#pragma unroll
          for (int i = 0; i < 32; ++i) u[i] += b[i];
        }
        if (!valid) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { f[i] = 0.f; u[i] = 0.f; }
        }
        if (args.out1) {
          pack32(f, w, fp16);
          staged_store64_lin(stage, lane, w, lin_of(args.out1) + n * 2ull, lin_stride, lin_rows_store);
        }
        if (args.out2) {
          pack32(u, w, fp16);
          staged_store64_lin(stage, lane, w, lin_of(args.out2) + n * 2ull, lin_stride, lin_rows_store);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float sg = fast_rcp(1.f + __expf(-f[i]));
          f[i] = f[i] * sg * u[i];
        }
        pack32(f, w, fp16);
        staged_store64_lin(stage, lane, w, lin_of(args.out0) + n * 2ull, lin_stride, lin_rows_store);
      }
    } else if (n < args.n) {  // column edge: chunks beyond the matrix are skipped
      if constexpr (kEpi == CCF_EPI_STORE) {
        if (has_b0) add_bias_raw(f, bcur, fp16);
        if (args.out_fp32) {
          if (valid) store32_f32(reinterpret_cast<float*>(args.out0) + orow * args.ld_out + n, f);
        } else if (sgd) {
          // the accumulator is a weight gradient and out0 the weights themselves: plain SGD applied here saves writing
          // the gradient, and the optimizer's pass that would read it and the weights again
          sgd_unstage(stage, lane, bcur, w);
          const float lr = args.sgd_lr, wd = args.sgd_wd;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 p = unpack2(w[j], fp16);
            w[j] = pack2(p.x - lr * fmaf(wd, p.x, f[2 * j]), p.y - lr * fmaf(wd, p.y, f[2 * j + 1]), fp16);
          }
          staged_store64_lin(stage, lane, w, lin_base + n * 2ull, lin_stride, lin_rows);
        } else {
          pack32(f, w, fp16);
          staged_store64_lin(stage, lane, w, lin_base + n * 2ull, lin_stride, lin_rows);
        }
      } else if constexpr (kEpi == CCF_EPI_BIAS_ACT) {
        if (has_b0) add_bias_raw(f, bcur, fp16);
        if (!valid) {
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = 0.f;
        }
        if (args.out1) {
          pack32(f, w, fp16);
          staged_store64_lin(stage, lane, w, lin_of(args.out1) + n * 2ull, lin_stride, lin_rows_store);
        }
        act32(f, args.act);  // rows beyond the group hold zeros: act(0) = 0 for every supported activation
        pack32(f, w, fp16);
        staged_store64_lin(stage, lane, w, lin_of(args.out0) + n * 2ull, lin_stride, lin_rows_store);
      } else if constexpr (kEpi == CCF_EPI_COMBINE) {
        if (has_b0) add_bias_raw(f, bcur, fp16);
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] *= c_gate;
        pack32(f, w, fp16);
        // peer stores over NVLink (or local when c_rank is this rank), 64 contiguous bytes per row
        staged_store64(stage, lane, w, c_ok ? addr2(args.peer_comb[c_rank], c_slot, args.ld_out, n) : 0ull);
      } else if constexpr (kEpi == CCF_EPI_DACT) {
        staged_load64_lin(stage, lane, w, lin_of(args.aux0) + n * 2ull, lin_stride, lin_rows);
        {
          float pz[32];
          unpack32(w, pz, fp16);
          act_grad32(f, pz, args.act);
          if (!valid) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = 0.f;
          }
        }
        pack32(f, w, fp16);
        staged_store64_lin(stage, lane, w, lin_of(args.out0) + n * 2ull, lin_stride, lin_rows_store);
      } else if constexpr (kEpi == CCF_EPI_DSWIGLU) {
        uint32_t wu[16];
        staged_load64_lin(stage, lane, w, lin_of(args.aux0) + n * 2ull, lin_stride, lin_rows);
        staged_load64_lin(stage, lane, wu, lin_of(args.aux1) + n * 2ull, lin_stride, lin_rows);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 gp = unpack2(w[j], fp16), up = unpack2(wu[j], fp16);
          const float a0 = valid ? f[2 * j] : 0.f, a1 = valid ? f[2 * j + 1] : 0.f;
          const float s0 = fast_rcp(1.f + __expf(-gp.x)), s1 = fast_rcp(1.f + __expf(-gp.y));
          w[j] = pack2(a0 * up.x * (s0 * (1.f + gp.x * (1.f - s0))), a1 * up.y * (s1 * (1.f + gp.y * (1.f - s1))), fp16);
          wu[j] = pack2(a0 * gp.x * s0, a1 * gp.y * s1, fp16);
        }
        staged_store64_lin(stage, lane, w, lin_of(args.out0) + n * 2ull, lin_stride, lin_rows_store);
        staged_store64_lin(stage, lane, wu, lin_of(args.out1) + n * 2ull, lin_stride, lin_rows_store);
      }
    }
  }
  CombineDest cd;
  cd.rank = c_rank;
  cd.ok = c_ok;
  return cd;
}

// COMBINE: tell every source rank how many of its rows (for this half column tile) are now in its buffer
__device__ __forceinline__ void combine_signal(const CcfGemmArgs& args, const CombineDest& cd, int lane) {
  __threadfence_system();
  __syncwarp();
  for (int s = 0; s < args.world; ++s) {
    const unsigned m = __ballot_sync(0xffffffffu, cd.ok && cd.rank == s);
    if (m != 0u && lane == 0) red_release_sys_add(args.peer_done[s], __popc(m));
  }
}

// The dispatch role as the epilogue warps of a GEMM kernel run it before their first accumulator is due. Only the
// kernels whose A operand is the receive buffer carry it: the forward ones (bias + activation, SwiGLU) push x rows, the
// backward ones (activation derivative) push g * dy rows; every other epilogue compiles to nothing here.
// `comm_warp`: the caller is one of the CTA's dedicated dispatch warps (else an epilogue warp); args.comm_warps says
// which of the two kinds carries the role in this launch.
template <int kEpi>
__device__ __forceinline__ void dispatch_role(const CcfGemmArgs& args, bool comm_warp) {
  if (comm_warp != (args.comm_warps != 0)) return;
  if constexpr (kEpi == CCF_EPI_BIAS_ACT || kEpi == CCF_EPI_SWIGLU) {
    if (static_cast<int>(blockIdx.x) < args.n_comm_ctas) {
      // A chunk is pushed by one warp from start to end. With only a few thousand rows in all (the latency-bound
      // serving shapes) chunks of two rows spread them over sixteen times as many warps, and the first tile's rows are
      // complete after microseconds instead of tens of them.
      if (args.disp.order_off[args.disp.e_total] <= 4096) dispatch_rows<2, false>(args.disp, args.status);
      else dispatch_rows<8, false>(args.disp, args.status);
    }
  } else if constexpr (kEpi == CCF_EPI_DACT || kEpi == CCF_EPI_DSWIGLU) {
    if (static_cast<int>(blockIdx.x) < args.n_comm_ctas) dispatch_rows<8, true>(args.disp, args.status);
  }
}

// two-CTA kernels (gemm2.cu), selected by the same key as the one-CTA ones
int launch_pair_by_key(int key, const CUtensorMap* tm, const CcfGemmArgs& a, int grid, cudaStream_t stream);

}  // namespace ccf
