// Grouped GEMM for sm_100a: TMA (local memory, no multicast) -> 128B-swizzled shared memory ->
// tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld epilogue. One persistent CTA per SM,
// 10 warps: warp 0 = tile scheduler + TMA producer, warp 1 = MMA issuer (one elected thread),
// warps 2..9 = epilogue (two per TMEM lane quarter, each taking half of the tile's columns). Tiles are 128 x 256 x 64, four shared-memory
// stages, two TMEM accumulator stages (2 x 256 columns) so the epilogue of a tile overlaps the
// main loop of the next one.
//
// The kernel replaces the reference's wmma tile GEMM and its callers (mix_moe/csrc/cuda/mix_gemm.cu:22-244
// myHGEMMAlignedV5, :282-436 moe_first_mm, :439-555 moe_second_mm, :780-974 the wgrad block-gather GEMM)
// with fp32 accumulation (the reference accumulates in fp16, mix_gemm.cu:43).
//
//   row-grouped mode   C[rows of group g, N] = A[rows of g, K] * B_g       (forward and dgrad GEMMs)
//   k-grouped mode     C_g[M, N] = sum over rows r of group g  A[r, M]^T B[r, N]   (wgrad)
//
// Operand majors: A and B may each be K-major (reduction index contiguous) or MN-major; weights are
// read in their [expert, out, in] layout for x W^T (K-major) and for dy W (MN-major), activations are
// read MN-major for wgrad, so nothing is ever transposed in memory.
//
// Fusion with the collectives:
//   * A tiles may be gated on per-tile arrival counters that remote dispatch roles increment
//     (args.tile_flags); the TMA producer polls its own GPU's memory with a bounded acquire loop.
//   * The first args.n_comm_ctas CTAs run the dispatch role (dispatch.cuh) before joining the tile loop,
//     so the all-to-all dispatch and the first GEMM are one kernel.
//   * EPI_COMBINE stores each output row, scaled by its gate weight, directly into the combine buffer of
//     the rank the token came from and bumps that rank's completion counter.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "gemm_common.cuh"

namespace ccf {

constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSchedSlots = 4;

struct __align__(16) Ctrl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sched_full[kSchedSlots];
  uint64_t sched_empty[kSchedSlots];
  uint32_t tmem_base;
  int abort_word;
  int total_tiles;
  int n_tiles;
  int total_rows;   // valid rows over all groups (row-grouped mode)
  int pad;
  int sched_tile[kSchedSlots];
  int mt_prefix[CCF_MAX_GROUPS + 1];
};

constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kEpiWarps * kEpiStageBytes + static_cast<int>(sizeof(Ctrl));

template <bool kKGroup, int kEpi>
__device__ __forceinline__ Tile decode_tile(int t, const CcfGemmArgs& a, const Ctrl* c) {
  Tile ti;
  const int bn_out = (kEpi == CCF_EPI_SWIGLU) ? BN / 2 : (a.bn == 128 ? 128 : BN);
  if constexpr (!kKGroup) {
    const int nt = c->n_tiles;
    int lo = 0, hi = a.num_groups;  // largest g with nt * mt_prefix[g] <= t
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (nt * c->mt_prefix[mid] <= t) lo = mid; else hi = mid;
    }
    ti.g = lo;
    const int mt_g = c->mt_prefix[lo + 1] - c->mt_prefix[lo];
    const int local = t - nt * c->mt_prefix[lo];
    const int j = local / mt_g, i = local - j * mt_g;
    const int rows = a.group_rows[lo];
    ti.row0 = a.group_base[lo] + i * BM;
    ti.rows_valid = min(BM, rows - i * BM);
    ti.n0 = j * bn_out;
    ti.kblocks = a.kseg * ((a.k + BK - 1) / BK);
    ti.krow0 = 0;
  } else {
    const int mt = a.m_per_group / BM;
    const int tpg = mt * c->n_tiles;
    ti.g = t / tpg;
    const int local = t - ti.g * tpg;
    const int j = local / mt, i = local - j * mt;
    ti.row0 = i * BM;
    ti.rows_valid = BM;
    ti.n0 = j * BN;
    ti.kblocks = (a.group_rows[ti.g] + BK - 1) / BK;
    ti.krow0 = a.group_base[ti.g];
  }
  return ti;
}

// ---------------------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------------------
template <int kAMajor, int kBMajor, int kEpi, bool kKGroup>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                    const __grid_constant__ CcfGemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + kStages * kStageBytes + kEpiWarps * kEpiStageBytes);
  const uint32_t smem_base = smem_u32(smem);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_word = &ctrl->abort_word;
  const uint64_t limit = fail_fast_limit(args.status, args.wait_limit_ns);
  const int bn_run = (!kKGroup && kBMajor == MAJ_K && kEpi != CCF_EPI_SWIGLU && args.bn == 128) ? 128 : BN;   // MMA N
  const int bn_out = (kEpi == CCF_EPI_SWIGLU) ? BN / 2 : bn_run;

  // ---- set-up ------------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctrl->acc_full[s]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[s]), kEpiWarps);
    }
    for (int s = 0; s < kSchedSlots; ++s) {
      mbar_init(smem_u32(&ctrl->sched_full[s]), 1);
      mbar_init(smem_u32(&ctrl->sched_empty[s]), 1 + kEpiWarps);
    }
    ctrl->abort_word = 0;
    const int nt = (args.n + bn_out - 1) / bn_out;
    ctrl->n_tiles = nt;
    if constexpr (!kKGroup) {
      int acc = 0;
      for (int g = 0; g < args.num_groups; ++g) {
        ctrl->mt_prefix[g] = acc;
        acc += (args.group_rows[g] + BM - 1) / BM;
      }
      ctrl->mt_prefix[args.num_groups] = acc;
      ctrl->total_tiles = acc * nt;
      int rows = 0;
      for (int g = 0; g < args.num_groups; ++g) rows += args.group_rows[g];
      ctrl->total_rows = rows;
    } else {
      ctrl->total_tiles = args.num_groups * (args.m_per_group / BM) * nt;
    }
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmA0);
    prefetch_tensormap(&tmB0);
    if (args.kseg > 1 || kEpi == CCF_EPI_SWIGLU) {
      prefetch_tensormap(&tmA1);
      prefetch_tensormap(&tmB1);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->total_tiles;

  // ---- dispatch role (fused all-to-all dispatch) -----------------------------------------------------
  // Run by the epilogue warps before their first accumulator is due (see below); the producer and MMA warps go
  // straight to the tile loop and start on tiles whose rows have already landed.
  // (trace: the last recorded tile slot of every CTA holds {0: kernel start, 1: this CTA's dispatch part finished})
  if (threadIdx.x == 0 && args.trace != nullptr) trace_ev(args, args.trace_tiles - 1, 0);

  if (warp == 0) {
    // ======================= tile scheduler + TMA producer =======================
    int stage = 0, phase = 0, ss = 0, sphase = 0;
    bool ok = true;
    // The index of the next tile is requested one tile ahead, so the latency of the global atomic is
    // hidden behind the loads of the current tile (lane 0 holds it until the next iteration).
    int t_next = 0, seq = 0;
    bool all_in = false;  // every row of this rank has arrived: no further flag reads
    if (lane == 0) t_next = atomicAdd(args.sched, 1);
    while (ok) {
      if (!mbar_wait(smem_u32(&ctrl->sched_empty[ss]), sphase ^ 1, abort_word, limit)) {
        report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 1);
        break;
      }
      int t = __shfl_sync(0xffffffffu, t_next, 0);
      if (t >= total_tiles) t = -1;
      if (lane == 0) {
        ctrl->sched_tile[ss] = t;
        mbar_arrive(smem_u32(&ctrl->sched_full[ss]));
        if (t >= 0) t_next = atomicAdd(args.sched, 1);
      }
      if (++ss == kSchedSlots) { ss = 0; sphase ^= 1; }
      if (t < 0) break;
      const Tile ti = decode_tile<kKGroup, kEpi>(t, args, ctrl);
      if (lane == 0) trace_ev(args, seq, 0);
      if constexpr (!kKGroup) {
        if (args.tile_flags != nullptr && !all_in) {
          // rows of this tile are pushed by other GPUs; wait until all of them have landed. The count of all
          // arrived rows is read alongside: once it is complete, later tiles skip the flag read and its latency.
          int state = 1;
          if (lane == 0) {
            int total = 0;
            if (args.total_index >= 0) total = ld_acquire_sys(args.tile_flags + args.total_index);
            if (!wait_flag_ge(args.tile_flags + (ti.row0 >> 7), ti.rows_valid, limit)) state = 0;
            else if (args.total_index >= 0 && total >= ctrl->total_rows) state = 2;
          }
          state = __shfl_sync(0xffffffffu, state, 0);
          if (state == 0) {
            report_status(args.status, CCF_ERR_FLAG_TIMEOUT, ti.row0 >> 7);
            *abort_word = 1;
            break;
          }
          all_in = state == 2;
          fence_proxy_async();  // generic-proxy peer stores -> async-proxy (TMA) reads
        }
      }
      if (lane == 0) trace_ev(args, seq, 1);
      const int kb_per_seg = kKGroup ? ti.kblocks : (args.k + BK - 1) / BK;
      for (int kb = 0; kb < ti.kblocks; ++kb) {
        if (!mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_word, limit)) {
          report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 2);
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t fullb = smem_u32(&ctrl->full[stage]);
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          mbar_arrive_expect_tx(fullb, kABytes + bn_run * BK * 2);
          const int seg = kKGroup ? 0 : kb / kb_per_seg;
          const int kk = kKGroup ? 0 : (kb - seg * kb_per_seg) * BK;
          const CUtensorMap* ma = seg ? &tmA1 : &tmA0;
          const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
          // A operand
          if constexpr (kAMajor == MAJ_K) {
            tma_load_2d(sa, ma, fullb, kk, ti.row0);
          } else {
            const int r = ti.krow0 + kb * BK;
            tma_load_2d(sa, ma, fullb, ti.row0, r);
            tma_load_2d(sa + 8192, ma, fullb, ti.row0 + 64, r);
          }
          // B operand
          if constexpr (kBMajor == MAJ_K) {
            if constexpr (kEpi == CCF_EPI_SWIGLU) {
              const int brow = ti.g * args.b_group_rows + ti.n0;
              tma_load_2d(sb, &tmB1, fullb, kk, brow);          // gate rows -> accumulator columns [0,128)
              tma_load_2d(sb + 16384, &tmB0, fullb, kk, brow);  // up rows   -> accumulator columns [128,256)
            } else {
              tma_load_2d(sb, mb, fullb, kk, ti.g * args.b_group_rows + ti.n0);
            }
          } else {
            const int r = kKGroup ? ti.krow0 + kb * BK : ti.g * args.b_group_rows + kk;
#pragma unroll
            for (int i = 0; i < 4; ++i) tma_load_2d(sb + i * 8192, mb, fullb, ti.n0 + 64 * i, r);
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (lane == 0) trace_ev(args, seq, 2);
      ++seq;
    }
  } else if (warp == 1) {
    // ======================= MMA issuer =======================
    const uint32_t idesc = make_idesc(BM, bn_run, args.fp16, kAMajor, kBMajor);
    int stage = 0, phase = 0, ss = 0, sphase = 0, as = 0, aphase = 0, seq = -1;
    bool ok = true;
    while (ok) {
      ++seq;
      if (!mbar_wait(smem_u32(&ctrl->sched_full[ss]), sphase, abort_word, limit)) {
        report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 3);
        break;
      }
      const int t = ctrl->sched_tile[ss];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->sched_empty[ss]));
      if (++ss == kSchedSlots) { ss = 0; sphase ^= 1; }
      if (t < 0) break;
      const Tile ti = decode_tile<kKGroup, kEpi>(t, args, ctrl);
      if (ti.kblocks == 0) continue;  // empty group: the epilogue writes zeros
      if (!mbar_wait(smem_u32(&ctrl->acc_empty[as]), aphase ^ 1, abort_word, limit)) {
        report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 4);
        break;
      }
      tc_fence_after();
      if (lane == 0) trace_ev(args, seq, 3);
      const uint32_t d_tmem = tmem_base + as * BN;
      for (int kb = 0; kb < ti.kblocks; ++kb) {
        if (!mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_word, limit)) {
          report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 5);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          if (kb == 0) trace_ev(args, seq, 4);
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = (kAMajor == MAJ_K) ? make_smem_desc(sa + k * 32, 16, 1024)
                                                   : make_smem_desc(sa + k * 2048, 8192, 1024);
            const uint64_t db = (kBMajor == MAJ_K) ? make_smem_desc(sb + k * 32, 16, 1024)
                                                   : make_smem_desc(sb + k * 2048, 8192, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&ctrl->empty[stage]));
          if (kb == ti.kblocks - 1) {
            umma_commit(smem_u32(&ctrl->acc_full[as]));
            trace_ev(args, seq, 5);
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (++as == 2) { as = 0; aphase ^= 1; }
    }
  } else if (warp >= 2 + kEpiWarps) {
    // ======================= dispatch warps =======================
    dispatch_role<kEpi>(args, true);
    if (warp == 2 + kEpiWarps && lane == 0 && args.trace != nullptr && args.comm_warps) trace_ev(args, args.trace_tiles - 1, 1);
  } else {
    // ======================= epilogue (warps 2..9) =======================
    const int q = warp & 3;               // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;     // which half of the tile's columns this warp handles
    dispatch_role<kEpi>(args, false);
    if (warp == 2 && lane == 0 && args.trace != nullptr && !args.comm_warps) trace_ev(args, args.trace_tiles - 1, 1);
    int ss = 0, sphase = 0, as = 0, aphase = 0, seq = -1;
    while (true) {
      ++seq;
      if (!mbar_wait(smem_u32(&ctrl->sched_full[ss]), sphase, abort_word, limit)) {
        report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 6);
        break;
      }
      const int t = ctrl->sched_tile[ss];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->sched_empty[ss]));
      if (++ss == kSchedSlots) { ss = 0; sphase ^= 1; }
      if (t < 0) break;
      const Tile ti = decode_tile<kKGroup, kEpi>(t, args, ctrl);
      if constexpr (kEpi == CCF_EPI_STORE) {
        // SGD in the epilogue: ask L2 for the weights under this tile while its accumulator is still being filled
        if (args.sgd_lr != 0.f && !args.out_fp32)
          sgd_prefetch_l2(args, (kKGroup ? static_cast<long long>(ti.g) * args.m_per_group : 0ll) + ti.row0, ti.n0,
                          ti.rows_valid, q, half, lane);
      }
      const bool have_acc = ti.kblocks > 0;
      if (have_acc) {
        if (!mbar_wait(smem_u32(&ctrl->acc_full[as]), aphase, abort_word, limit)) {
          report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 7);
          break;
        }
        tc_fence_after();
      }
      if (warp == 2 && lane == 0) trace_ev(args, seq, 6);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * BN;
      const uint32_t stage = smem_base + kStages * kStageBytes + (warp - 2) * kEpiStageBytes;
      long long row_base;
      if constexpr (kKGroup) row_base = static_cast<long long>(ti.g) * args.m_per_group + ti.row0;
      else row_base = ti.row0;
      const CombineDest cd = epilogue_tile<kEpi>(args, ti, row_base, ti.rows_valid, BM, have_acc, t_row, stage, q, half, lane);
      if (warp == 2 && lane == 0) trace_ev(args, seq, 7);
      if (have_acc) {
        // all TMEM reads of this accumulator stage are complete: hand it back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty[as]));
        if (++as == 2) { as = 0; aphase ^= 1; }
      }
      if constexpr (kEpi == CCF_EPI_COMBINE) combine_signal(args, cd, lane);
      (void)cd;
    }
  }

  // ---- tear-down -----------------------------------------------------------------------------------
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
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(args.sched + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      // last CTA: every tile of this rank is finished
      if constexpr (kEpi == CCF_EPI_COMBINE) {
        if (args.send_finish) {
          __threadfence_system();
          for (int s = 0; s < args.world; ++s) red_release_sys_add(args.peer_done[s], 1);
        }
      }
      args.sched[0] = 0;
      args.sched[1] = 0;
      args.sched[2] = 0;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major view [rows, cols] of 2-byte elements, box = {box_cols, box_rows}, 128-byte swizzle.
// A tensor map is a pure function of (address, extents, box, type), so encoded maps are kept in a small direct-mapped
// cache: a layer launches the same few operands every step, and in the latency-bound regime four driver calls per
// launch cost as much as a small kernel.
namespace {
struct TmapKey {
  const void* base;
  long long rows, cols;
  int box_cols, box_rows, fp16;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_cols == o.box_cols && box_rows == o.box_rows &&
           fp16 == o.fp16;
  }
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kTmapCacheSize = 512;
TmapEntry g_tmap_cache[kTmapCacheSize];
std::mutex g_tmap_mutex;
size_t tmap_hash(const TmapKey& k) {
  size_t h = reinterpret_cast<size_t>(k.base) >> 8;
  h = h * 1000003u ^ static_cast<size_t>(k.rows);
  h = h * 1000003u ^ static_cast<size_t>(k.cols);
  h = h * 1000003u ^ static_cast<size_t>((k.box_cols << 12) ^ (k.box_rows << 1) ^ k.fp16);
  return h % kTmapCacheSize;
}
}  // namespace

int make_tmap(CUtensorMap* m, const void* base, long long rows, long long cols, int box_cols, int box_rows,
                     int fp16) {
  const TmapKey key = {base, rows, cols, box_cols, box_rows, fp16};
  const size_t slot = tmap_hash(key);
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    const TmapEntry& e = g_tmap_cache[slot];
    if (e.valid && e.key == key) {
      *m = e.map;
      return 0;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstr[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -static_cast<int>(r) - 1000;
  {
    std::lock_guard<std::mutex> lock(g_tmap_mutex);
    TmapEntry& e = g_tmap_cache[slot];
    e.key = key;
    e.map = *m;
    e.valid = true;
  }
  return 0;
}

template <int A, int B, int E, bool KG>
static int launch_variant(const CUtensorMap* tm, const CcfGemmArgs& args, int grid, cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<A, B, E, KG>;
  // the attribute belongs to the (function, device) pair: set it once per device this process launches on
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured[dev & 63] = true;
  }
  kern<<<grid, kThreads, kSmemBytes, stream>>>(tm[0], tm[1], tm[2], tm[3], args);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // namespace ccf

extern "C" {

int ccf_gemm_smem_bytes() { return ccf::kSmemBytes; }

// sizes of the argument blocks, so the Python mirror of the structures can be checked at load time
int ccf_sizeof_gemm_args() { return static_cast<int>(sizeof(CcfGemmArgs)); }
int ccf_sizeof_dispatch_args() { return static_cast<int>(sizeof(CcfDispatchArgs)); }
int ccf_sizeof_gemm_launch() { return static_cast<int>(sizeof(CcfGemmLaunch)); }

// Returns 0 on success, a negative number on a host-side error (bad combination, encode or launch failure).
int ccf_gemm_launch(const CcfGemmLaunch* L, void* stream_v) {
  using namespace ccf;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  const CcfGemmArgs& a = L->args;
  // Tensor maps are encoded through the driver API, which needs a context bound to the calling thread;
  // a framework worker thread (autograd) may not have touched the runtime yet.
  if (L->device >= 0 && cudaSetDevice(L->device) != cudaSuccess) return -7;
  if (a.num_groups < 1 || a.num_groups > CCF_MAX_GROUPS) return -2;
  if (a.n % 32 != 0) return -3;
  if (L->kgroup && (a.m_per_group % BM != 0)) return -4;
  if (!L->kgroup && (a.k % 8 != 0)) return -5;
  if (a.n_comm_ctas > 0) {
    // the dispatch role is compiled into the kernels that read the receive buffer, in the direction of their pass
    const bool fwd = L->epi == CCF_EPI_BIAS_ACT || L->epi == CCF_EPI_SWIGLU;
    const bool bwd = L->epi == CCF_EPI_DACT || L->epi == CCF_EPI_DSWIGLU;
    if (!(fwd && a.disp.backward == 0) && !(bwd && a.disp.backward == 1)) return -9;
  }
  CUtensorMap tm[4];
  const int fp16 = a.fp16;
  const int a_box_rows = (L->a_major == MAJ_K) ? BM : BK;
  const bool pair = L->two_cta != 0;
  if (pair && L->kgroup && (a.m_per_group % (2 * BM) != 0)) return -8;
  if (a.bn != 0 && a.bn != BN) {
    // the narrow tile exists in the one-CTA kernel for row-grouped launches with a K-major B operand
    if (a.bn != 128 || pair || L->kgroup || L->b_major != MAJ_K || L->epi == CCF_EPI_SWIGLU) return -10;
  }
  int b_box_rows = (L->b_major == MAJ_K) ? (a.bn == 128 ? 128 : BN) : BK;
  if (L->epi == CCF_EPI_SWIGLU || (pair && L->b_major == MAJ_K)) b_box_rows = BN / 2;  // a pair member loads half of B
  int rc;
  if ((rc = make_tmap(&tm[0], L->a0, L->a_rows, L->a_cols, 64, a_box_rows, fp16))) return rc;
  if ((rc = make_tmap(&tm[1], L->a1 ? L->a1 : L->a0, L->a_rows, L->a_cols, 64, a_box_rows, fp16))) return rc;
  if ((rc = make_tmap(&tm[2], L->b0, L->b_rows, L->b_cols, 64, b_box_rows, fp16))) return rc;
  if ((rc = make_tmap(&tm[3], L->b1 ? L->b1 : L->b0, L->b_rows, L->b_cols, 64, b_box_rows, fp16))) return rc;
  int grid = L->grid;
  if (grid <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    grid = sms;
  }
  const int key = (L->a_major << 12) | (L->b_major << 8) | (L->epi << 4) | (L->kgroup ? 1 : 0);
  if (pair) return launch_pair_by_key(key, tm, a, grid, stream);
  switch (key) {
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_STORE << 4):
      return launch_variant<MAJ_K, MAJ_K, CCF_EPI_STORE, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_BIAS_ACT << 4):
      return launch_variant<MAJ_K, MAJ_K, CCF_EPI_BIAS_ACT, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_SWIGLU << 4):
      return launch_variant<MAJ_K, MAJ_K, CCF_EPI_SWIGLU, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_COMBINE << 4):
      return launch_variant<MAJ_K, MAJ_K, CCF_EPI_COMBINE, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_STORE << 4):
      return launch_variant<MAJ_K, MAJ_MN, CCF_EPI_STORE, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_DACT << 4):
      return launch_variant<MAJ_K, MAJ_MN, CCF_EPI_DACT, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_DSWIGLU << 4):
      return launch_variant<MAJ_K, MAJ_MN, CCF_EPI_DSWIGLU, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_COMBINE << 4):
      return launch_variant<MAJ_K, MAJ_MN, CCF_EPI_COMBINE, false>(tm, a, grid, stream);
    case (MAJ_MN << 12) | (MAJ_MN << 8) | (CCF_EPI_STORE << 4) | 1:
      return launch_variant<MAJ_MN, MAJ_MN, CCF_EPI_STORE, true>(tm, a, grid, stream);
    default:
      return -6;
  }
}

}  // extern "C"
