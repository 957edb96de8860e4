// Native runtime of one fused MoE layer (see runtime.h): ccf_layer_forward / ccf_layer_backward issue, in order and on
// one stream, exactly the launches that ops/fused.py issues call by call from Python: routing, count exchange + plan,
// dispatch fused with GEMM-1, GEMM-2 fused with combine, wait + reduce; and for backward the dy dispatch fused with
// dgrad-2, both weight-gradient GEMMs, the bias-gradient column sums and dgrad-1 fused with combine.
// tests/test_native_runtime.py compares the GEMM launch blocks built here with the ones the Python path builds.
#include <cuda_runtime.h>
#include <string.h>

#include "runtime.h"

extern "C" {
int ccf_gemm_launch(const CcfGemmLaunch* L, void* stream);
int ccf_route_ordered(const int* expert, int S, int E, int cap, int* pos, int* block_hist, int* block_off,
                      int* count_raw, int* count_kept, int* ticket, int* order_off, int* sorted_slot, int* slot_row,
                      int first_expert, void* stream);
int ccf_plan(const CcfPlanArgs* a, void* stream);
int ccf_plan_dev_epoch(const CcfPlanArgs* a, int* epoch_counter, void* stream);
int ccf_combine_wait(const int* done, int* cum, const int* sent_rows, int n_tiles, int world,
                     unsigned long long limit_ns, int* status, void* stream);
int ccf_combine_reduce(const void* comb, const int* slot_row, void* y, int T, int K, int d, int fp16, void* stream);
int ccf_colsum_grouped(const void* x, long long ld, int n, int groups, const int* group_base, const int* group_rows,
                       void* out, int fp16, void* stream);
}

namespace {

constexpr int kMajK = 0, kMajMN = 1;

struct Dry {
  CcfGemmLaunch* out;
  int cap;
  int n;
};

// completion-counter increments per row of a COMBINE GEMM with n columns (two epilogue warps per 256-column tile)
int combine_units(int n, int bn) { return 2 * ((n + bn - 1) / bn); }

// fields every launch of this layer shares
CcfGemmLaunch base_launch(const CcfLayer* L) {
  CcfGemmLaunch g;
  memset(&g, 0, sizeof(g));
  g.args.group_base = L->group_base;
  g.args.group_rows = L->group_rows;
  g.args.sched = L->sched;
  g.args.status = L->status;
  g.args.wait_limit_ns = L->wait_limit_ns;
  g.args.num_groups = L->e_loc;
  g.args.kseg = 1;
  g.args.fp16 = L->fp16;
  g.args.world = 1;
  g.args.total_index = -1;
  g.args.comm_warps = L->comm_warps;
  g.device = L->device;
  g.two_cta = L->two_cta;
  return g;
}

void set_a(CcfGemmLaunch& g, const void* a0, long long rows, long long cols, int major) {
  g.a0 = a0;
  g.a_rows = rows;
  g.a_cols = cols;
  g.a_major = major;
}
void set_b(CcfGemmLaunch& g, const void* b0, long long rows, long long cols, int major) {
  g.b0 = b0;
  g.b_rows = rows;
  g.b_cols = cols;
  g.b_major = major;
}

// the dispatch role's arguments (forward: x rows into the owners' xrecv; backward: g * dy rows into their grecv)
void set_dispatch(CcfGemmLaunch& g, const CcfLayer* L, const void* src, const int* idx, const float* gate_w, int tokens,
                  int capacity, int backward, float* dgate) {
  CcfDispatchArgs& a = g.args.disp;
  a.x = src;
  a.slot_expert = idx;
  a.slot_pos = L->slot_pos;
  a.dst_base = L->dst_base;
  a.slot_gate = gate_w;
  a.saved_comb = backward ? L->comb : nullptr;
  a.dgate = dgate;
  a.slot_row = L->slot_row;
  a.sorted_slot = L->sorted_slot;
  a.order_off = L->order_off;
  for (int r = 0; r < L->world; ++r) {
    a.peer_recv[r] = backward ? L->peer_grecv[r] : L->peer_xrecv[r];
    a.peer_row_src[r] = L->peer_row_src[r];
    a.peer_row_gate[r] = L->peer_row_gate[r];
    a.peer_tile_flags[r] = L->peer_tile_flags[r];
  }
  a.work_counter = L->sched + 2;
  a.tokens = tokens;
  a.top_k = L->top_k;
  a.d = L->d_model;
  a.capacity = capacity;
  a.experts_per_rank = L->e_loc;
  a.my_rank = L->rank;
  a.backward = backward;
  a.fp16 = L->fp16;
  a.max_rows = L->max_rows;
  a.total_index = L->max_rows / 128;
  a.e_total = L->e_total;
  // the GEMM side of the same kernel: tiles gated on the arrival counters, local-source tiles first
  g.args.tile_flags = L->tile_flags;
  g.args.local_begin = L->local_begin;
  g.args.local_rows = L->local_rows;
  g.args.n_comm_ctas = L->n_comm_ctas;
  g.args.total_index = L->max_rows / 128;
}

void set_combine(CcfGemmLaunch& g, const CcfLayer* L, void* const* peer_comb, const float* row_gate) {
  g.args.row_src = L->row_src;
  g.args.row_gate = row_gate;
  for (int r = 0; r < L->world; ++r) {
    g.args.peer_comb[r] = peer_comb[r];
    g.args.peer_done[r] = L->peer_done[r];
  }
  g.args.world = L->world;
  g.args.send_finish = 1;
  g.args.max_slots = L->max_slots;
}

int issue(CcfGemmLaunch& g, Dry* dry, void* stream) {
  // the pair kernel needs 256-row output tiles in k-grouped mode
  if (g.kgroup && g.args.m_per_group % 256 != 0) g.two_cta = 0;
  if (g.args.ld_out == 0) g.args.ld_out = g.args.n;
  if (dry != nullptr) {
    if (dry->n < dry->cap) dry->out[dry->n] = g;
    ++dry->n;
    return 0;
  }
  return ccf_gemm_launch(&g, stream);
}

int wait_and_reduce(const CcfLayer* L, const void* comb, void* out, int tokens, int bn, Dry* dry, void* stream) {
  if (dry != nullptr) return 0;
  int rc = ccf_combine_wait(L->done, L->done_cum, L->sent_rows, combine_units(L->d_model, bn), L->world, L->wait_limit_ns,
                            L->status, stream);
  if (rc) return rc;
  return ccf_combine_reduce(comb, L->slot_row, out, tokens, L->top_k, L->d_model, L->fp16, stream);
}

int zero_tile_flags(const CcfLayer* L, Dry* dry, void* stream) {
  if (dry != nullptr) return 0;
  cudaError_t e = cudaMemsetAsync(L->tile_flags, 0, sizeof(int) * (L->max_rows / 128 + 1),
                                  reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

}  // namespace

extern "C" {

int ccf_sizeof_layer() { return static_cast<int>(sizeof(CcfLayer)); }
int ccf_sizeof_layer_grads() { return static_cast<int>(sizeof(CcfLayerGrads)); }

int ccf_layer_forward(const CcfLayer* L, const void* x, const int* idx, const float* gate_w, void* y, int tokens,
                      int capacity, int save_pre, int epoch, void* stream, CcfGemmLaunch* dry_gemms, int dry_cap,
                      int* dry_count) {
  if (L == nullptr || L->world < 1 || L->world > CCF_MAX_RANKS || L->e_total > CCF_MAX_GROUPS) return -2;
  Dry dry_state = {dry_gemms, dry_cap, 0};
  Dry* dry = dry_gemms != nullptr ? &dry_state : nullptr;
  const int d = L->d_model, f = L->d_ffn, e_loc = L->e_loc;
  int rc = 0;
  // An expert that receives about one 256-row pair tile's worth of rows fills most second tiles with padding: such
  // calls run on 128-row tiles (one-CTA kernel).
  const long long rows_per_expert = static_cast<long long>(tokens) * L->top_k * L->world / (L->e_total > 0 ? L->e_total : 1);
  const int row_two_cta = rows_per_expert > L->small_rows ? L->two_cta : 0;
  // GEMM-2 on the one-CTA kernel with so few tiles that most SMs would idle: 128-column tiles (twice as many)
  int gemm2_bn = 256;
  if (row_two_cta == 0) {
    const long long tiles = static_cast<long long>(e_loc) * ((rows_per_expert + 127) / 128 > 0 ? (rows_per_expert + 127) / 128 : 1) *
                            ((d + 255) / 256);
    if (tiles < 148) gemm2_bn = 128;
  }
  if (dry == nullptr) {
    if (L->device >= 0 && cudaSetDevice(L->device) != cudaSuccess) return -7;
    // 1. positions, kept counts, destination order of this rank's slots
    rc = ccf_route_ordered(idx, tokens * L->top_k, L->e_total, capacity, L->slot_pos, L->block_hist, L->block_off,
                           L->count_raw, L->count_kept, L->ticket, L->order_off, L->sorted_slot, L->slot_row,
                           L->rank * e_loc, stream);
    if (rc) return rc;
    // 2. count exchange with all ranks + row layout
    CcfPlanArgs p;
    memset(&p, 0, sizeof(p));
    p.count_kept = L->count_kept;
    for (int r = 0; r < L->world; ++r) {
      p.peer_table[r] = L->peer_cnt_table[r];
      p.peer_flag[r] = L->peer_cnt_flag[r];
    }
    p.dst_base = L->dst_base;
    p.group_base = L->group_base;
    p.group_rows = L->group_rows;
    p.sent_rows = L->sent_rows;
    p.table_copy = L->table_copy;
    p.local_begin = L->local_begin;
    p.local_rows = L->local_rows;
    p.status = L->status;
    p.wait_limit_ns = L->wait_limit_ns;
    p.world = L->world;
    p.my_rank = L->rank;
    p.e_total = L->e_total;
    p.e_loc = e_loc;
    p.epoch = epoch;
    p.max_rows = L->max_rows;
    rc = epoch >= 0 ? ccf_plan(&p, stream) : ccf_plan_dev_epoch(&p, L->epoch_dev, stream);
    if (rc) return rc;
  }
  // 3. dispatch + GEMM-1 (+ bias + activation)
  {
    CcfGemmLaunch g = base_launch(L);
    set_a(g, L->xrecv, L->max_rows, d, kMajK);
    set_b(g, L->w1, static_cast<long long>(e_loc) * f, d, kMajK);
    g.args.n = f;
    g.args.k = d;
    g.args.b_group_rows = f;
    g.args.out0 = L->h_act;
    g.args.out1 = save_pre ? L->h_pre : nullptr;
    g.args.bias0 = L->b1;
    if (L->swiglu) {
      g.epi = CCF_EPI_SWIGLU;
      g.b1 = L->wg;
      g.args.out2 = save_pre ? L->h_pre2 : nullptr;
      g.args.bias1 = L->bg;
    } else {
      g.epi = CCF_EPI_BIAS_ACT;
      g.args.act = L->act;
    }
    set_dispatch(g, L, x, idx, gate_w, tokens, capacity, 0, nullptr);
    g.two_cta = row_two_cta;
    if ((rc = issue(g, dry, stream))) return rc;
    if ((rc = zero_tile_flags(L, dry, stream))) return rc;
  }
  // 4. GEMM-2 + combine into the source ranks
  {
    CcfGemmLaunch g = base_launch(L);
    set_a(g, L->h_act, L->max_rows, f, kMajK);
    set_b(g, L->w2, static_cast<long long>(e_loc) * d, f, kMajK);
    g.epi = CCF_EPI_COMBINE;
    g.args.n = d;
    g.args.k = f;
    g.args.b_group_rows = d;
    g.args.bias0 = L->b2;
    g.args.ld_out = d;
    set_combine(g, L, L->peer_comb, L->row_gate);
    g.two_cta = row_two_cta;
    g.args.bn = gemm2_bn;
    if ((rc = issue(g, dry, stream))) return rc;
  }
  // 5. wait for every owner, sum the k slots of each token
  rc = wait_and_reduce(L, L->comb, y, tokens, gemm2_bn, dry, stream);
  if (dry_count != nullptr) *dry_count = dry_state.n;
  return rc;
}

int ccf_layer_backward(const CcfLayer* L, const void* dy, const int* idx, const float* gate_w, const CcfLayerGrads* G,
                       int tokens, int capacity, void* stream, CcfGemmLaunch* dry_gemms, int dry_cap, int* dry_count) {
  if (L == nullptr || G == nullptr || L->world < 1 || L->world > CCF_MAX_RANKS) return -2;
  Dry dry_state = {dry_gemms, dry_cap, 0};
  Dry* dry = dry_gemms != nullptr ? &dry_state : nullptr;
  const int d = L->d_model, f = L->d_ffn, e_loc = L->e_loc;
  int rc = 0;
  if (dry == nullptr && L->device >= 0 && cudaSetDevice(L->device) != cudaSuccess) return -7;
  // With few rows per expert the weight-gradient reduction is only a handful of k-blocks and the per-tile latency chain
  // decides: there the one-CTA kernel is faster than CTA pairs.
  const long long rows_per_expert = static_cast<long long>(tokens) * L->top_k * L->world / (L->e_total > 0 ? L->e_total : 1);
  const int wgrad_two_cta = rows_per_expert > 512 ? L->two_cta : 0;
  const int row_two_cta = rows_per_expert > L->small_rows ? L->two_cta : 0;
  // In-place SGD (sgd_lr != 0), matrix by matrix: a weight whose gradient pointer is null is updated by its weight-gradient
  // GEMM. w2 may be at any group size (dgrad-2 above it is its last reader). w1 / wg only on a single rank: dgrad-1 reads
  // them and, with peers, has to stay the last owner-side kernel of the pass.
  const bool sgd2 = G->sgd_lr != 0.f && G->dw2 == nullptr;
  const bool sgd = G->sgd_lr != 0.f && G->dw1 == nullptr;     // w1 (and wg) in place: dgrad-1 moves in front of wgrad-1
  if (sgd && L->world != 1) return -2;
  if (sgd && L->swiglu && G->dwg != nullptr) return -2;
  // 1 + 2. push g * dy rows + dgrad-2 with the activation derivative
  {
    CcfGemmLaunch g = base_launch(L);
    set_a(g, L->grecv, L->max_rows, d, kMajK);
    set_b(g, L->w2, static_cast<long long>(e_loc) * d, f, kMajMN);
    g.args.n = f;
    g.args.k = d;
    g.args.b_group_rows = d;
    g.args.out0 = G->dh;
    g.args.aux0 = L->h_pre;
    if (L->swiglu) {
      g.epi = CCF_EPI_DSWIGLU;
      g.args.out1 = G->dh2;
      g.args.aux1 = L->h_pre2;
    } else {
      g.epi = CCF_EPI_DACT;
      g.args.act = L->act;
    }
    set_dispatch(g, L, dy, idx, gate_w, tokens, capacity, 1, G->dgate);
    g.two_cta = row_two_cta;
    if ((rc = issue(g, dry, stream))) return rc;
    if ((rc = zero_tile_flags(L, dry, stream))) return rc;
  }
  // 3. wgrad-2: dW2[e] = (g dy)^T h_act  [d, f]
  {
    CcfGemmLaunch g = base_launch(L);
    set_a(g, L->grecv, L->max_rows, d, kMajMN);
    set_b(g, L->h_act, L->max_rows, f, kMajMN);
    g.epi = CCF_EPI_STORE;
    g.kgroup = 1;
    g.args.n = f;
    g.args.m_per_group = d;
    g.args.out0 = sgd2 ? const_cast<void*>(L->w2) : G->dw2;   // dgrad-2 above was the last reader of the old w2
    g.args.sgd_lr = sgd2 ? G->sgd_lr : 0.f;
    g.args.sgd_wd = sgd2 ? G->sgd_wd : 0.f;
    g.args.ld_out = f;
    g.two_cta = wgrad_two_cta;
    if ((rc = issue(g, dry, stream))) return rc;
  }
  if (G->db2 != nullptr && dry == nullptr) {
    if ((rc = ccf_colsum_grouped(L->grecv, d, d, e_loc, L->group_base, L->group_rows, G->db2, L->fp16, stream))) return rc;
  }
  // 4. wgrad-1: dW1[e] = dh^T x_e  [f, d]  (SwiGLU: gate projection from dh, up projection from dh2)
  auto wgrad1 = [&](const void* a0, void* out) {
    CcfGemmLaunch g = base_launch(L);
    set_a(g, a0, L->max_rows, f, kMajMN);
    set_b(g, L->xrecv, L->max_rows, d, kMajMN);
    g.epi = CCF_EPI_STORE;
    g.kgroup = 1;
    g.args.n = d;
    g.args.m_per_group = f;
    g.args.out0 = out;
    g.args.sgd_lr = sgd ? G->sgd_lr : 0.f;
    g.args.sgd_wd = sgd ? G->sgd_wd : 0.f;
    g.args.ld_out = d;
    g.two_cta = wgrad_two_cta;
    return issue(g, dry, stream);
  };
  // 5. dgrad-1 + combine: dx rows go back to the ranks the tokens came from. Issued after the weight gradients (its
  // finish token then tells the sources that every buffer of this call is free), except when those update w1 / wg in
  // place: then it must read them first.
  auto dgrad1 = [&]() {
    CcfGemmLaunch g = base_launch(L);
    set_a(g, G->dh, L->max_rows, f, kMajK);
    g.epi = CCF_EPI_COMBINE;
    g.args.n = d;
    g.args.k = f;
    g.args.b_group_rows = f;
    g.args.ld_out = d;
    if (L->swiglu) {
      g.a1 = G->dh2;
      set_b(g, L->wg, static_cast<long long>(e_loc) * f, d, kMajMN);
      g.b1 = L->w1;
      g.args.kseg = 2;
    } else {
      set_b(g, L->w1, static_cast<long long>(e_loc) * f, d, kMajMN);
    }
    set_combine(g, L, L->peer_gcomb, nullptr);
    g.two_cta = row_two_cta;
    return issue(g, dry, stream);
  };
  if (sgd && (rc = dgrad1())) return rc;
  if (L->swiglu) {
    if ((rc = wgrad1(G->dh, sgd ? const_cast<void*>(L->wg) : G->dwg))) return rc;
    if ((rc = wgrad1(G->dh2, sgd ? const_cast<void*>(L->w1) : G->dw1))) return rc;
    if (dry == nullptr) {
      if (G->db1 != nullptr &&
          (rc = ccf_colsum_grouped(G->dh2, f, f, e_loc, L->group_base, L->group_rows, G->db1, L->fp16, stream)))
        return rc;
      if (G->dbg != nullptr &&
          (rc = ccf_colsum_grouped(G->dh, f, f, e_loc, L->group_base, L->group_rows, G->dbg, L->fp16, stream)))
        return rc;
    }
  } else {
    if ((rc = wgrad1(G->dh, sgd ? const_cast<void*>(L->w1) : G->dw1))) return rc;
    if (dry == nullptr && G->db1 != nullptr &&
        (rc = ccf_colsum_grouped(G->dh, f, f, e_loc, L->group_base, L->group_rows, G->db1, L->fp16, stream)))
      return rc;
  }
  if (!sgd && (rc = dgrad1())) return rc;
  rc = wait_and_reduce(L, L->gcomb, G->dx, tokens, 256, dry, stream);
  if (dry_count != nullptr) *dry_count = dry_state.n;
  return rc;
}

}  // extern "C"
