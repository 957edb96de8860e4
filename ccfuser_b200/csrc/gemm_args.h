// Argument blocks shared by the host launchers and the kernels. Plain C structs: the Python side fills
// them through ctypes, so every field has a fixed width and the layout has no hidden padding surprises
// (pointers first, then 64-bit, then 32-bit fields).
#pragma once
#include <stdint.h>

#define CCF_MAX_RANKS 8
#define CCF_MAX_GROUPS 256

// Epilogues of the grouped GEMM kernel
enum CcfEpilogue {
  CCF_EPI_STORE = 0,     // out0 = acc (+ bias0)
  CCF_EPI_BIAS_ACT = 1,  // out1 = acc + bias0 (pre-activation, optional), out0 = act(acc + bias0)
  CCF_EPI_SWIGLU = 2,    // B tile = [128 gate rows | 128 up rows]; out1 = g, out2 = u, out0 = silu(g) * u
  CCF_EPI_COMBINE = 3,   // (acc + bias0) * row_gate -> row `slot` of the source rank's combine buffer (peer store)
  CCF_EPI_DACT = 4,      // out0 = acc * act'(aux0)
  CCF_EPI_DSWIGLU = 5    // out0 = acc * aux1 * silu'(aux0) (d gate), out1 = acc * silu(aux0) (d up)
};

enum CcfAct { CCF_ACT_NONE = 0, CCF_ACT_GELU = 1, CCF_ACT_RELU = 2 };

// status word values (low 8 bits = code, upper bits = detail such as a tile index)
enum CcfStatus {
  CCF_OK = 0,
  CCF_ERR_MBAR_TIMEOUT = 1,   // a pipeline barrier inside one CTA never completed
  CCF_ERR_FLAG_TIMEOUT = 2,   // a peer's arrival flag / counter never reached its target
  CCF_ERR_BOUNDS = 3,         // an index failed a debug bounds check; the access was skipped
  CCF_ERR_OVERFLOW = 4        // more rows routed to a rank than its receive buffer holds
};

// Rows pushed by the dispatch role. All peer_* pointers are addresses in *this* process' address space
// (own memory for this rank, IPC mappings for the others).
struct CcfDispatchArgs {
  const void* x;            // [T, D] rows to send (2-byte elements)
  const int* slot_expert;   // [S] expert id of each slot, S = T * top_k
  const int* slot_pos;      // [S] position of the slot inside (this rank, expert)
  const int* dst_base;      // [E_total] first destination row of this rank's rows of expert e on its owner
  const float* slot_gate;   // [S] gate weight of the slot
  const void* saved_comb;   // backward only: [S, D] scaled expert outputs saved by the forward pass
  float* dgate;             // backward only: [S] gradient of the gate weight
  int* slot_row;            // [S] out: destination row (dropped slots are set to -1 by the routing kernels)
  const int* sorted_slot;   // [S] slot ids in destination order (own experts first, then the next owner's, ...)
  const int* order_off;     // [E_total + 1]; order_off[E_total] = number of kept rows = length of sorted_slot in use
  void* peer_recv[CCF_MAX_RANKS];      // receive buffer [R, D] of every rank
  int* peer_row_src[CCF_MAX_RANKS];    // [R] packed (source rank << 24 | slot)
  float* peer_row_gate[CCF_MAX_RANKS]; // [R]
  int* peer_tile_flags[CCF_MAX_RANKS]; // [R / 128] rows arrived per 128-row tile
  int* work_counter;        // chunk claim counter (zero before launch; the kernel's last CTA restores zero)
  int tokens;
  int top_k;
  int d;                    // row length in elements (multiple of 8)
  int capacity;
  int experts_per_rank;
  int my_rank;
  int backward;             // 1: rows are scaled by the gate weight and dgate is produced
  int fp16;                 // 1: fp16 rows, 0: bf16 rows
  int max_rows;             // rows of a receive buffer (bounds check)
  int total_index;          // element of peer_tile_flags[] that counts all rows arrived on that rank (-1 = none)
  int e_total;              // number of experts over all ranks
  int pad0;
};

struct CcfGemmArgs {
  // grouping
  const int* group_base;    // [G] first row of each group (multiple of 128)
  const int* group_rows;    // [G] valid rows of each group
  const int* tile_flags;    // optional [R / 128] arrival counters gating the A tiles (row-grouped only)
  const int* local_begin;   // optional [G] offset of the rows pushed by this rank itself inside each group
  const int* local_rows;    // optional [G] their number; tiles made only of such rows are scheduled first
  // epilogue operands
  void* out0;
  void* out1;
  void* out2;
  const void* bias0;        // [G, N]
  const void* bias1;        // [G, N] (swiglu gate bias)
  const void* aux0;         // [R, N] saved pre-activation (DACT / DSWIGLU: gate pre-activation)
  const void* aux1;         // [R, N] DSWIGLU: up pre-activation
  const int* row_src;       // [R] COMBINE: packed (source rank << 24 | slot)
  const float* row_gate;    // [R] COMBINE: gate weight (null = 1)
  void* peer_comb[CCF_MAX_RANKS];   // COMBINE: combine buffer [S, N] of every rank
  int* peer_done[CCF_MAX_RANKS];    // COMBINE: this rank's completion counter on every rank
  int* sched;               // {tile counter, finished CTAs, spare, spare}; zero before the first launch
  int* status;              // error word (first error wins)
  long long* trace;         // optional [grid, trace_tiles, 8] clock stamps per tile and role (null = off)
  unsigned long long wait_limit_ns;
  long long ld_out;         // leading dimension (elements) of out0/out1/out2/aux0/aux1
  int n;                    // output columns
  int k;                    // reduction length per k segment (row-grouped)
  int num_groups;
  int m_per_group;          // k-grouped: output rows per group
  int kseg;                 // 1 or 2 reduction segments (second one uses the *1 tensor maps)
  int b_group_rows;         // rows of one group inside B's 2-D view
  int act;                  // CcfAct
  int fp16;                 // operand/output element type: 1 fp16, 0 bf16
  int out_fp32;             // EPI_STORE: write fp32
  int world;                // COMBINE: number of ranks
  int send_finish;          // COMBINE: the last CTA adds 1 to every rank's completion counter
  int n_comm_ctas;          // CTAs that run the dispatch role before taking GEMM tiles (0 = none)
  int max_slots;            // COMBINE: rows of a combine buffer (bounds check)
  int trace_tiles;          // tiles per CTA recorded in `trace`
  int total_index;          // element of tile_flags that counts all arrived rows (-1 = none); lets late tiles skip their flag
  float sgd_lr;             // EPI_STORE, non-zero: out0 holds parameters and is updated in place, out0 -= lr * (acc + wd * out0)
  int comm_warps;           // 1: the CTA's two dedicated warps run the dispatch role; 0: its epilogue warps do, before their first tile
  float sgd_wd;             // weight decay of that update
  int bn;                   // one-CTA kernel, row-grouped, K-major B: output tile width, 256 (or 0) / 128. The narrow tile doubles
                            // the number of tiles of a launch that would otherwise leave most SMs idle
  int pad3;
  CcfDispatchArgs disp;
};

// One launch of the grouped GEMM as the host entry point ccf_gemm_launch takes it: the kernel arguments plus the 2-D
// views of the operands, from which the tensor maps are encoded.
struct CcfGemmLaunch {
  CcfGemmArgs args;
  const void* a0;
  const void* a1;
  const void* b0;
  const void* b1;
  long long a_rows, a_cols;  // 2-D views, cols contiguous
  long long b_rows, b_cols;
  int a_major, b_major;      // 0 = K-major, 1 = MN-major
  int epi;                   // CcfEpilogue
  int kgroup;                // 1 = k-grouped (wgrad)
  int grid;                  // 0 = one CTA per SM
  int device;                // CUDA device of the operands; made current for the calling thread (-1 = leave)
  int two_cta;               // 1 = 256x256 tiles on CTA pairs (tcgen05 cta_group::2), 0 = 128x256 tiles per CTA
  int pad0;
};

// Arguments of the count exchange + planning kernel (ccf_plan).
struct CcfPlanArgs {
  const int* count_kept;               // [E_total] this rank's kept rows per expert
  int* peer_table[CCF_MAX_RANKS];      // count table [W, E_total] of every rank
  int* peer_flag[CCF_MAX_RANKS];       // epoch flags [W] of every rank
  int* dst_base;                       // out [E_total]
  int* group_base;                     // out [E_loc]
  int* group_rows;                     // out [E_loc]
  int* sent_rows;                      // out [W] kept rows this rank sends to each owner
  int* table_copy;                     // out [W, E_total] snapshot of the table (routing statistics)
  int* local_begin;                    // out [E_loc] offset of this rank's own rows inside each local expert (optional)
  int* local_rows;                     // out [E_loc] number of those rows
  int* status;
  unsigned long long wait_limit_ns;
  int world, my_rank, e_total, e_loc, epoch, max_rows;
};

// Arguments of the on-stream barrier over the ranks of a group (ccf_flag_barrier).
struct CcfBarrierArgs {
  int* peer_flag[CCF_MAX_RANKS];   // barrier flags [W] of every rank; rank r writes element r everywhere
  int* status;
  unsigned long long wait_limit_ns;
  int world, my_rank, epoch, pad0;
};

// One launch of the SGD step over several parameter tensors (ccf_sgd_multi): tensor t is updated by the blocks
// [first_block[t], first_block[t + 1]).
#define CCF_SGD_MULTI 48
struct CcfSgdMulti {
  void* p[CCF_SGD_MULTI];
  const void* g[CCF_SGD_MULTI];
  long long n[CCF_SGD_MULTI];
  int first_block[CCF_SGD_MULTI + 1];
  int count;
  float lr, wd;
  int fp16;
};
