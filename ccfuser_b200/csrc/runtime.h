// Native runtime of one fused MoE layer: the whole forward (or backward) of a layer is one C call that issues the
// routing, planning, fused GEMM and reduce launches in order on a stream. It plays the part of the reference's
// `_MixMOE` object (mix_moe/csrc/mix_moe.h:30-603: first/second_gemm_forward/backward), without owning memory: the
// description below holds the addresses of buffers that the Python side allocates once per layer and per
// expert-parallel group (symmetric ones with their peer mappings).
#pragma once
#include "gemm_args.h"

struct CcfLayer {
  // this rank's expert parameters, [E_local, out, in] / [E_local, out]; null where the layer has none
  const void* w1;
  const void* b1;
  const void* wg;   // SwiGLU gate projection
  const void* bg;
  const void* w2;
  const void* b2;
  // per-layer buffers of this rank
  void* xrecv;      // [max_rows, d] rows received in forward (symmetric)
  void* comb;       // [max_slots, d] scaled expert outputs returned to this rank (symmetric)
  void* h_act;      // [max_rows, f]
  void* h_pre;      // [max_rows, f] pre-activation (SwiGLU: gate pre-activation)
  void* h_pre2;     // [max_rows, f] SwiGLU: up pre-activation
  int* slot_pos;
  int* slot_row;
  int* sorted_slot;
  int* order_off;
  int* local_begin;
  int* local_rows;
  int* count_raw;
  int* count_kept;
  int* dst_base;
  int* group_base;
  int* group_rows;
  int* sent_rows;
  int* table_copy;
  // buffers shared by the layers of one expert-parallel group
  void* grecv;      // [max_rows, d] rows received in backward (symmetric)
  void* gcomb;      // [max_slots, d] input-gradient rows returned to this rank (symmetric)
  int* row_src;
  float* row_gate;
  int* tile_flags;  // [max_rows / 128 + 1]
  int* done;        // [CCF_MAX_RANKS] completion counters written by the owners
  int* done_cum;    // [CCF_MAX_RANKS] values already consumed
  int* block_hist;
  int* block_off;
  int* ticket;
  int* sched;       // scheduler words of the device's workspace (8 ints)
  int* status;      // status words of the device's workspace (2 ints)
  int* epoch_dev;   // device-side call epoch (used when a call passes epoch < 0)
  // the same buffers on every rank of the group, as mapped into this process
  void* peer_xrecv[CCF_MAX_RANKS];
  void* peer_comb[CCF_MAX_RANKS];
  void* peer_grecv[CCF_MAX_RANKS];
  void* peer_gcomb[CCF_MAX_RANKS];
  int* peer_row_src[CCF_MAX_RANKS];
  float* peer_row_gate[CCF_MAX_RANKS];
  int* peer_tile_flags[CCF_MAX_RANKS];
  int* peer_cnt_table[CCF_MAX_RANKS];
  int* peer_cnt_flag[CCF_MAX_RANKS];
  int* peer_done[CCF_MAX_RANKS];   // this rank's element of every rank's `done` array
  unsigned long long wait_limit_ns;
  int d_model, d_ffn, e_total, e_loc, top_k, world, rank;
  int act;          // CcfAct of a non-gated FFN
  int swiglu;       // 1: SwiGLU FFN (wg / bg / h_pre2 in use)
  int fp16;
  int max_rows, max_slots;
  int n_comm_ctas;  // CTAs whose epilogue warps run the dispatch role
  int two_cta;      // default GEMM kernel: 1 = CTA pairs
  int device;       // CUDA device (-1: leave the calling thread's device alone)
  int pad0;
  int comm_warps;   // 1: dedicated dispatch warps carry the row push, 0: the epilogue warps do
  int small_rows;   // calls that expect at most this many rows per expert use the one-CTA kernel (128-row tiles)
};

// Per-call tensors of the backward pass (all allocated by the caller; null where the layer has no such parameter).
struct CcfLayerGrads {
  float* dgate;     // [tokens * top_k], zero on entry (dropped slots keep 0)
  void* dh;         // [max_rows, f] scratch: gradient of the (gate) pre-activation
  void* dh2;        // [max_rows, f] scratch, SwiGLU: gradient of the up pre-activation
  void* dw1;
  void* db1;
  void* dwg;
  void* dbg;
  void* dw2;
  void* db2;
  void* dx;         // [tokens, d]
  // Non-zero sgd_lr (single-rank layers only): the weight-gradient GEMMs apply plain SGD to w1 / wg / w2 in their
  // epilogue (w -= lr * (dw + wd * w)) instead of writing dw1 / dwg / dw2, and the input-gradient GEMM that still needs
  // the old w1 / wg runs before them.
  float sgd_lr;
  float sgd_wd;
};

extern "C" {
int ccf_sizeof_layer();
int ccf_sizeof_layer_grads();
// `epoch` >= 0: the call's epoch as kept by the host; < 0: take it from L->epoch_dev (CUDA-graph replay).
// `dry_gemms` non-null: nothing is launched; the GEMM launch blocks the call would issue are written there
// (at most `dry_cap`) and their number to *dry_count. Returns 0 or the first negative error of a launcher.
int ccf_layer_forward(const CcfLayer* L, const void* x, const int* idx, const float* gate_w, void* y, int tokens,
                      int capacity, int save_pre, int epoch, void* stream, CcfGemmLaunch* dry_gemms, int dry_cap,
                      int* dry_count);
int ccf_layer_backward(const CcfLayer* L, const void* dy, const int* idx, const float* gate_w, const CcfLayerGrads* G,
                       int tokens, int capacity, void* stream, CcfGemmLaunch* dry_gemms, int dry_cap, int* dry_count);
}
