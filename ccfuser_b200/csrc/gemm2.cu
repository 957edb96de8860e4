// Two-CTA variant of the grouped GEMM (tcgen05 cta_group::2): a cluster of two CTAs on neighbouring SMs computes one
// 256 x 256 tile. Each CTA loads its own 128 rows of A and its own 128-column half of B with plain (non-multicast) TMA
// loads, the leader CTA issues one M = 256 MMA that reads both CTAs' shared memory and writes both CTAs' TMEM, and each
// CTA runs the epilogue for its own 128 rows. Compared with the one-CTA kernel (gemm.cu) the B operand crosses the
// L2 -> SM fabric once per pair instead of once per CTA: 64 KB instead of 96 KB per 128x256x64 worth of MMA work, and
// six 32 KB pipeline stages fit where four 48 KB stages did.
//
// Same modes, operand majors, epilogues, dispatch role and arrival-counter gating as gemm.cu; tiles are assigned
// statically (tile = pair index + k * number of pairs) because both CTAs of a pair must walk the same sequence.
// No TMA load in this file uses cluster multicast, and the stage hand-back uses two plain tcgen05.commit arrivals
// (one per CTA) rather than a multicast commit.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <string.h>

#include "gemm_common.cuh"

namespace ccf {

constexpr int k2Stages = 6;
constexpr int k2ABytes = BM * BK * 2;          // this CTA's 128 rows of A
constexpr int k2BBytes = (BN / 2) * BK * 2;    // this CTA's 128-column half of B
constexpr int k2StageBytes = k2ABytes + k2BBytes;
constexpr int PM = 2 * BM;                     // rows of a pair tile

struct __align__(16) Ctrl2 {
  uint64_t full[k2Stages];     // used on the leader: both CTAs' TMA loads complete on it
  uint64_t empty[k2Stages];    // one per CTA: the leader's MMA thread commits to both
  uint64_t acc_full[2];        // one per CTA
  uint64_t acc_empty[2];       // used on the leader: 2 * kEpiWarps arrivals (local + remote)
  uint32_t tmem_base;
  int abort_word;
  int total_tiles;
  int n_tiles;
  int total_rows;
  int tiles_a;                          // pair tiles (x n-tiles) of phase A: made only of rows this rank pushed itself
  int mt_prefix[CCF_MAX_GROUPS + 1];    // phase B (all other pair tiles), prefix over groups
  int mta_prefix[CCF_MAX_GROUPS + 1];   // phase A, prefix over groups
  short a0[CCF_MAX_GROUPS];             // first phase-A pair tile of each group
  short na[CCF_MAX_GROUPS];             // number of phase-A pair tiles of each group
};

constexpr int k2SmemBytes = 1024 + k2Stages * k2StageBytes + kEpiWarps * kEpiStageBytes + static_cast<int>(sizeof(Ctrl2));

// ---- cluster / cta_group::2 primitives -------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_word,
                                                  uint64_t limit_ns) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*abort_word) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_word = 1;
        return false;
      }
    }
  }
  return true;
}
// arrive on a barrier given by its shared::cluster address (own CTA or the peer)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory, completion bytes counted on a barrier of the pair (shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// one arrival on the barrier at `cluster_addr` when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

struct PairTile {
  int g;
  int row0;        // first row of the pair tile (row-grouped) / first output row inside the group (k-grouped)
  int n0;
  int rows_pair;   // valid rows of the 256-row pair tile
  int kblocks;
  int krow0;
};

template <bool kKGroup, int kEpi>
__host__ __device__ __forceinline__ PairTile decode_pair_tile(int t, const CcfGemmArgs& a, const Ctrl2* c) {
  PairTile ti;
  constexpr int bn_out = (kEpi == CCF_EPI_SWIGLU) ? BN / 2 : BN;
  if constexpr (!kKGroup) {
    // Phase A first: the pair tiles that hold only rows pushed by this rank itself (they arrive first, without
    // crossing NVLink); then phase B, every other pair tile. Inside a phase: group-major, column tile, row tile.
    const int nt = c->n_tiles;
    const bool phase_a = t < c->tiles_a;
    const int* pre = phase_a ? c->mta_prefix : c->mt_prefix;
    const int tt = phase_a ? t : t - c->tiles_a;
    int lo = 0, hi = a.num_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (nt * pre[mid] <= tt) lo = mid; else hi = mid;
    }
    ti.g = lo;
    const int mt_g = pre[lo + 1] - pre[lo];
    const int local = tt - nt * pre[lo];
    const int j = local / mt_g;
    int i = local - j * mt_g;
    if (phase_a) i += c->a0[lo];
    else if (i >= c->a0[lo]) i += c->na[lo];
    ti.row0 = a.group_base[lo] + i * PM;
    ti.rows_pair = min(PM, a.group_rows[lo] - i * PM);
    ti.n0 = j * bn_out;
    ti.kblocks = a.kseg * ((a.k + BK - 1) / BK);
    ti.krow0 = 0;
  } else {
    const int mt = a.m_per_group / PM;
    const int tpg = mt * c->n_tiles;
    ti.g = t / tpg;
    const int local = t - ti.g * tpg;
    const int j = local / mt, i = local - j * mt;
    ti.row0 = i * PM;
    ti.rows_pair = PM;
    ti.n0 = j * BN;
    ti.kblocks = (a.group_rows[ti.g] + BK - 1) / BK;
    ti.krow0 = a.group_base[ti.g];
  }
  return ti;
}

// Tile tables of one launch, computed by one thread of every CTA at start-up (host-callable so that the tile order can
// be checked exhaustively without a GPU): number of column tiles; pair tiles per group, split into phase A (tiles that
// hold only rows this rank pushed itself) and phase B (the rest) with their prefix sums; total tiles and total rows.
template <bool kKGroup, int kEpi>
__host__ __device__ __forceinline__ void pair_tile_tables(const CcfGemmArgs& args, Ctrl2* ctrl) {
  constexpr int bn_out = (kEpi == CCF_EPI_SWIGLU) ? BN / 2 : BN;
  const int nt = (args.n + bn_out - 1) / bn_out;
  ctrl->n_tiles = nt;
  if constexpr (!kKGroup) {
    int acc_a = 0, acc_b = 0, rows = 0;
    for (int g = 0; g < args.num_groups; ++g) {
      const int gr = args.group_rows[g];
      const int mt = (gr + PM - 1) / PM;
      int a0 = 0, na = 0;
      if (args.local_begin != nullptr && args.tile_flags != nullptr) {
        const int lb = args.local_begin[g], le = min(gr, lb + args.local_rows[g]);
        a0 = (lb + PM - 1) / PM;
        // a tile is local-only when it lies inside [lb, le); the last tile of the group also counts when le == gr
        int a1 = (le == gr) ? mt : le / PM;
        na = max(0, a1 - a0);
        if (na == 0) a0 = 0;
      }
      ctrl->a0[g] = static_cast<short>(a0);
      ctrl->na[g] = static_cast<short>(na);
      ctrl->mta_prefix[g] = acc_a;
      ctrl->mt_prefix[g] = acc_b;
      acc_a += na;
      acc_b += mt - na;
      rows += gr;
    }
    ctrl->mta_prefix[args.num_groups] = acc_a;
    ctrl->mt_prefix[args.num_groups] = acc_b;
    ctrl->tiles_a = acc_a * nt;
    ctrl->total_tiles = (acc_a + acc_b) * nt;
    ctrl->total_rows = rows;
  } else {
    ctrl->total_tiles = args.num_groups * (args.m_per_group / PM) * nt;
  }
}

template <int kAMajor, int kBMajor, int kEpi, bool kKGroup>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                         const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                         const __grid_constant__ CcfGemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctrl2* ctrl = reinterpret_cast<Ctrl2*>(smem + k2Stages * k2StageBytes + kEpiWarps * kEpiStageBytes);
  const uint32_t smem_base = smem_u32(smem);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();   // 0 = leader (issues the MMAs), 1 = peer
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  const int n_pairs = static_cast<int>(gridDim.x) >> 1;
  volatile int* abort_word = &ctrl->abort_word;
  const uint64_t limit = fail_fast_limit(args.status, args.wait_limit_ns);

  // ---- set-up ------------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctrl->acc_full[s]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[s]), 2 * kEpiWarps);
    }
    ctrl->abort_word = 0;
    pair_tile_tables<kKGroup, kEpi>(args, ctrl);
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
    tmem_alloc_pair(smem_u32(&ctrl->tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->total_tiles;

  // ---- dispatch role (fused all-to-all dispatch) -----------------------------------------------------
  // Run by the epilogue warps before their first accumulator is due (see below); the producer and MMA warps go
  // straight to the tile loop and start on tiles whose rows have already landed.
  // (trace: the last recorded tile slot of every CTA holds {0: kernel start, 1: this CTA's dispatch part finished})
  if (threadIdx.x == 0 && args.trace != nullptr) trace_ev(args, args.trace_tiles - 1, 0);

  if (warp == 0) {
    // ======================= TMA producer (both CTAs) =======================
    int stage = 0, phase = 0, seq = 0;
    bool all_in = false, ok = true;
    for (int t = pair; t < total_tiles && ok; t += n_pairs, ++seq) {
      const PairTile ti = decode_pair_tile<kKGroup, kEpi>(t, args, ctrl);
      const int my_rows = kKGroup ? BM : max(0, min(BM, ti.rows_pair - static_cast<int>(cta) * BM));
      const int my_row0 = ti.row0 + static_cast<int>(cta) * BM;
      if (lane == 0) trace_ev(args, seq, 0);
      if constexpr (!kKGroup) {
        if (args.tile_flags != nullptr && !all_in && my_rows > 0) {
          int state = 1;
          if (lane == 0) {
            int total = 0;
            if (args.total_index >= 0) total = ld_acquire_sys(args.tile_flags + args.total_index);
            if (!wait_flag_ge(args.tile_flags + (my_row0 >> 7), my_rows, limit)) state = 0;
            else if (args.total_index >= 0 && total >= ctrl->total_rows) state = 2;
          }
          state = __shfl_sync(0xffffffffu, state, 0);
          if (state == 0) {
            report_status(args.status, CCF_ERR_FLAG_TIMEOUT, my_row0 >> 7);
            *abort_word = 1;
            break;
          }
          all_in = state == 2;
          fence_proxy_async();
        }
      }
      if (lane == 0) trace_ev(args, seq, 1);
      const int kb_per_seg = kKGroup ? ti.kblocks : (args.k + BK - 1) / BK;
      for (int kb = 0; kb < ti.kblocks; ++kb) {
        if (!mbar_wait_cluster(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_word, limit)) {
          report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 0x22);
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t full_leader = map_to_cta(smem_u32(&ctrl->full[stage]), 0);
          const uint32_t sa = smem_base + stage * k2StageBytes;
          const uint32_t sb = sa + k2ABytes;
          if (cta == 0) mbar_arrive_expect_tx(smem_u32(&ctrl->full[stage]), 2 * k2StageBytes);
          const int seg = kKGroup ? 0 : kb / kb_per_seg;
          const int kk = kKGroup ? 0 : (kb - seg * kb_per_seg) * BK;
          const CUtensorMap* ma = seg ? &tmA1 : &tmA0;
          const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
          // A: this CTA's 128 rows
          if constexpr (kAMajor == MAJ_K) {
            tma_load_2d_pair(sa, ma, full_leader, kk, my_row0);
          } else {
            const int r = ti.krow0 + kb * BK;
            tma_load_2d_pair(sa, ma, full_leader, my_row0, r);
            tma_load_2d_pair(sa + 8192, ma, full_leader, my_row0 + 64, r);
          }
          // B: this CTA's half of the 256 columns
          const int nh = static_cast<int>(cta) * (BN / 2);
          if constexpr (kBMajor == MAJ_K) {
            if constexpr (kEpi == CCF_EPI_SWIGLU) {
              // leader loads the gate rows (accumulator columns [0,128)), the peer the up rows ([128,256))
              tma_load_2d_pair(sb, cta == 0 ? &tmB1 : &tmB0, full_leader, kk, ti.g * args.b_group_rows + ti.n0);
            } else {
              tma_load_2d_pair(sb, mb, full_leader, kk, ti.g * args.b_group_rows + ti.n0 + nh);
            }
          } else {
            const int r = kKGroup ? ti.krow0 + kb * BK : ti.g * args.b_group_rows + kk;
            tma_load_2d_pair(sb, mb, full_leader, ti.n0 + nh, r);
            tma_load_2d_pair(sb + 8192, mb, full_leader, ti.n0 + nh + 64, r);
          }
        }
        __syncwarp();
        if (++stage == k2Stages) { stage = 0; phase ^= 1; }
      }
      if (lane == 0) trace_ev(args, seq, 2);
    }
  } else if (warp == 1) {
    // ======================= MMA issuer (leader CTA only) =======================
    if (cta == 0) {
      const uint32_t idesc = make_idesc(PM, BN, args.fp16, kAMajor, kBMajor);
      int stage = 0, phase = 0, as = 0, aphase = 0, seq = 0;
      bool ok = true;
      for (int t = pair; t < total_tiles && ok; t += n_pairs, ++seq) {
        const PairTile ti = decode_pair_tile<kKGroup, kEpi>(t, args, ctrl);
        if (ti.kblocks == 0) continue;
        if (!mbar_wait_cluster(smem_u32(&ctrl->acc_empty[as]), aphase ^ 1, abort_word, limit)) {
          report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 0x24);
          break;
        }
        tc_fence_after();
        if (lane == 0) trace_ev(args, seq, 3);
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = 0; kb < ti.kblocks; ++kb) {
          if (!mbar_wait_cluster(smem_u32(&ctrl->full[stage]), phase, abort_word, limit)) {
            report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 0x25);
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            if (kb == 0) trace_ev(args, seq, 4);
            const uint32_t sa = smem_base + stage * k2StageBytes;
            const uint32_t sb = sa + k2ABytes;
#pragma unroll
            for (int k = 0; k < BK / UK; ++k) {
              const uint64_t da = (kAMajor == MAJ_K) ? make_smem_desc(sa + k * 32, 16, 1024)
                                                     : make_smem_desc(sa + k * 2048, 8192, 1024);
              const uint64_t db = (kBMajor == MAJ_K) ? make_smem_desc(sb + k * 32, 16, 1024)
                                                     : make_smem_desc(sb + k * 2048, 8192, 1024);
              umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            // hand the stage back to both producers
            const uint32_t e0 = smem_u32(&ctrl->empty[stage]);
            umma_commit_pair(map_to_cta(e0, 0));
            umma_commit_pair(map_to_cta(e0, 1));
            if (kb == ti.kblocks - 1) {
              const uint32_t f0 = smem_u32(&ctrl->acc_full[as]);
              umma_commit_pair(map_to_cta(f0, 0));
              umma_commit_pair(map_to_cta(f0, 1));
              trace_ev(args, seq, 5);
            }
          }
          __syncwarp();
          if (++stage == k2Stages) { stage = 0; phase ^= 1; }
        }
        if (++as == 2) { as = 0; aphase ^= 1; }
      }
    }
  } else if (warp >= 2 + kEpiWarps) {
    // ======================= dispatch warps =======================
    dispatch_role<kEpi>(args, true);
    if (warp == 2 + kEpiWarps && lane == 0 && args.trace != nullptr && args.comm_warps) trace_ev(args, args.trace_tiles - 1, 1);
  } else {
    // ======================= epilogue (warps 2..9, both CTAs) =======================
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    dispatch_role<kEpi>(args, false);
    if (warp == 2 && lane == 0 && args.trace != nullptr && !args.comm_warps) trace_ev(args, args.trace_tiles - 1, 1);
    int as = 0, aphase = 0, seq = 0;
    for (int t = pair; t < total_tiles; t += n_pairs, ++seq) {
      const PairTile ti = decode_pair_tile<kKGroup, kEpi>(t, args, ctrl);
      if constexpr (kEpi == CCF_EPI_STORE) {
        // SGD in the epilogue: ask L2 for the weights under this tile while its accumulator is still being filled
        if (args.sgd_lr != 0.f && !args.out_fp32)
          sgd_prefetch_l2(args, (kKGroup ? static_cast<long long>(ti.g) * args.m_per_group : 0ll) + ti.row0 + static_cast<int>(cta) * BM,
                          ti.n0, kKGroup ? BM : max(0, min(BM, ti.rows_pair - static_cast<int>(cta) * BM)), q, half, lane);
      }
      const bool have_acc = ti.kblocks > 0;
      if (have_acc) {
        if (!mbar_wait_cluster(smem_u32(&ctrl->acc_full[as]), aphase, abort_word, limit)) {
          report_status(args.status, CCF_ERR_MBAR_TIMEOUT, 0x27);
          break;
        }
        tc_fence_after();
      }
      if (warp == 2 && lane == 0) trace_ev(args, seq, 6);
      const int my_rows = kKGroup ? BM : max(0, min(BM, ti.rows_pair - static_cast<int>(cta) * BM));
      const int rows_store = my_rows > 0 ? BM : 0;   // an empty second half may belong to the next group: never written
      Tile tt;
      tt.g = ti.g;
      tt.row0 = ti.row0 + static_cast<int>(cta) * BM;
      tt.n0 = ti.n0;
      tt.rows_valid = my_rows;
      tt.kblocks = ti.kblocks;
      tt.krow0 = ti.krow0;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + as * BN;
      const uint32_t stage = smem_base + k2Stages * k2StageBytes + (warp - 2) * kEpiStageBytes;
      long long row_base;
      if constexpr (kKGroup) row_base = static_cast<long long>(ti.g) * args.m_per_group + tt.row0;
      else row_base = tt.row0;
      const CombineDest cd = epilogue_tile<kEpi>(args, tt, row_base, my_rows, rows_store, have_acc, t_row, stage, q, half, lane);
      if (warp == 2 && lane == 0) trace_ev(args, seq, 7);
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctrl->acc_empty[as]), 0));
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
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 50000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();   // neither CTA frees TMEM or leaves while the other may still use the pair's resources
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(args.sched + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
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

template <int A, int B, int E, bool KG>
static int launch_pair_variant(const CUtensorMap* tm, const CcfGemmArgs& args, int grid, cudaStream_t stream) {
  auto kern = grouped_gemm_pair_kernel<A, B, E, KG>;
  // the attribute belongs to the (function, device) pair: set it once per device this process launches on
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, k2SmemBytes);
    if (e != cudaSuccess) return -static_cast<int>(e);
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid & ~1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = k2SmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm[0], tm[1], tm[2], tm[3], args);
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

// Called by ccf_gemm_launch (gemm.cu) when the two-CTA kernel is requested. `key` encodes (A-major, B-major, epilogue,
// k-grouped) exactly as there. Returns -6 for a combination that has no two-CTA instantiation.
int launch_pair_by_key(int key, const CUtensorMap* tm, const CcfGemmArgs& a, int grid, cudaStream_t stream) {
  switch (key) {
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_STORE << 4):
      return launch_pair_variant<MAJ_K, MAJ_K, CCF_EPI_STORE, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_BIAS_ACT << 4):
      return launch_pair_variant<MAJ_K, MAJ_K, CCF_EPI_BIAS_ACT, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_SWIGLU << 4):
      return launch_pair_variant<MAJ_K, MAJ_K, CCF_EPI_SWIGLU, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_K << 8) | (CCF_EPI_COMBINE << 4):
      return launch_pair_variant<MAJ_K, MAJ_K, CCF_EPI_COMBINE, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_STORE << 4):
      return launch_pair_variant<MAJ_K, MAJ_MN, CCF_EPI_STORE, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_DACT << 4):
      return launch_pair_variant<MAJ_K, MAJ_MN, CCF_EPI_DACT, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_DSWIGLU << 4):
      return launch_pair_variant<MAJ_K, MAJ_MN, CCF_EPI_DSWIGLU, false>(tm, a, grid, stream);
    case (MAJ_K << 12) | (MAJ_MN << 8) | (CCF_EPI_COMBINE << 4):
      return launch_pair_variant<MAJ_K, MAJ_MN, CCF_EPI_COMBINE, false>(tm, a, grid, stream);
    case (MAJ_MN << 12) | (MAJ_MN << 8) | (CCF_EPI_STORE << 4) | 1:
      return launch_pair_variant<MAJ_MN, MAJ_MN, CCF_EPI_STORE, true>(tm, a, grid, stream);
    default:
      return -6;
  }
}

}  // namespace ccf

// The tile sequence of a row-grouped launch of the CTA-pair kernel, computed on the host with the kernel's own
// functions: for tile t in launch order, out[5 t ...] = {group, first row, first column, valid rows, phase (0 = A)}.
// Host arrays in, nothing touches a device. Returns the number of tiles (only the first `cap` are written).
extern "C" int ccf_debug_pair_tile_order(const int* group_base, const int* group_rows, const int* local_begin,
                                         const int* local_rows, int num_groups, int n, int k, int gated, int swiglu,
                                         int* out, int cap) {
  using namespace ccf;
  if (num_groups < 1 || num_groups > CCF_MAX_GROUPS) return -2;
  static const int dummy_flags = 0;
  CcfGemmArgs a;
  memset(&a, 0, sizeof(a));
  a.group_base = group_base;
  a.group_rows = group_rows;
  a.local_begin = local_begin;
  a.local_rows = local_rows;
  a.tile_flags = gated ? &dummy_flags : nullptr;
  a.num_groups = num_groups;
  a.n = n;
  a.k = k;
  a.kseg = 1;
  Ctrl2* c = new Ctrl2;
  int total;
  if (swiglu) {
    pair_tile_tables<false, CCF_EPI_SWIGLU>(a, c);
    total = c->total_tiles;
    for (int t = 0; t < total && t < cap; ++t) {
      const PairTile ti = decode_pair_tile<false, CCF_EPI_SWIGLU>(t, a, c);
      const int rec[5] = {ti.g, ti.row0, ti.n0, ti.rows_pair, t < c->tiles_a ? 0 : 1};
      memcpy(out + 5 * t, rec, sizeof(rec));
    }
  } else {
    pair_tile_tables<false, CCF_EPI_STORE>(a, c);
    total = c->total_tiles;
    for (int t = 0; t < total && t < cap; ++t) {
      const PairTile ti = decode_pair_tile<false, CCF_EPI_STORE>(t, a, c);
      const int rec[5] = {ti.g, ti.row0, ti.n0, ti.rows_pair, t < c->tiles_a ? 0 : 1};
      memcpy(out + 5 * t, rec, sizeof(rec));
    }
  }
  delete c;
  return total;
}
