// Parameter blocks of the fused compute + collective kernels (host- and device-visible).
#pragma once
#include <stdint.h>

#include "status.h"

namespace b200 {

constexpr int kMaxRanks = 8;

struct FusedArParams {
  // problem: partial[T, H] = A[T, K] . W[H, K]^T on every rank; rows are owned in contiguous
  // chunks of rows_per_rank.
  int T, H, K;
  int tp, rank, rows_per_rank;
  // symmetric buffers, one pointer per rank (index = rank that OWNS the memory)
  void* recv[kMaxRanks];          // [tp (source)][rows_per_rank_cap][H] 16-bit partial rows
  uint32_t* counters[kMaxRanks];  // [2 (parity)][num_row_blocks_cap] arrivals per 128-row block
  uint32_t* flags[kMaxRanks];     // [tp] epoch written by each source when its pushes are complete
  void* out[kMaxRanks];           // [T_cap, H] normalised hidden states (all-gathered result)
  int rows_cap;                   // rows_per_rank_cap (stride of recv's source dimension)
  int rb_cap;                     // num_row_blocks_cap
  // local tensors
  void* residual;                 // [rows_per_rank, H] this rank's shard of the residual stream (in/out)
  const void* norm_weight;        // [H]
  float eps;
  int add_residual;               // 0: residual_out = reduced sum (first use), 1: residual += sum
  int rows_per_gap;               // rows an epilogue warp may reduce between two tiles (set by the launcher)
  int ksplit;                     // K is cut into this many ranges, each a work unit of its own (set by the launcher)
  int slot_rows;                  // rows between two (source, K-range) slots of recv: rows_cap / ksplit, multiple of 8
  uint32_t* local_sync;           // [4] local scratch: [0] CTAs done, [1] last finished epoch (the call's
                                  // epoch is that + 1; its low bit selects the counter set)
  long long wait_cycles;          // budget of every flag wait
  StatusWord* status;
};

// Row scatter of a GEMM's output (gemm_pair_tcgen05.cu, gemm_streamk_tcgen05.cu): output row r belongs to rank
// r / rows_per_rank and is stored into that rank's receive slot for this source, over NVLink when the owner is a
// peer.  tp == 0 switches the scatter off.  When the last CTA of the launch has finished, flag[d][src_rank] on every
// rank d is set to the call's epoch (local_sync[1] + 1, kept in device memory so that graph replays advance it).
struct RowScatter {
  int tp, src_rank, rows_per_rank, rows_cap;
  void* recv[kMaxRanks];          // [tp (source)][rows_cap][ld] 16-bit rows, indexed by the OWNING rank
  uint32_t* flag[kMaxRanks];      // [tp] push epoch per source, indexed by the owning rank
  uint32_t* local_sync;           // [0] CTA ticket, [1] last finished push epoch
};

// Reduce + residual + RMSNorm + all-gather over the slots a RowScatter GEMM filled (comm_ar_norm.cu).
struct ArNormParams {
  int T, H, tp, rank, rows_per_rank, rows_cap;
  void* recv[kMaxRanks];          // as in RowScatter
  uint32_t* flag1[kMaxRanks];     // [tp] push epochs (written by the GEMMs)
  uint32_t* flag2[kMaxRanks];     // [tp] gather epochs (written by this kernel)
  void* out[kMaxRanks];           // [T_cap, H] normalised rows on every rank
  void* out_mc;                   // the same buffers as ONE NVLink multicast address (multimem.st reaches every
                                  // rank's copy through the switch), or null: one peer store per rank
  void* residual;                 // [rows_per_rank, H] this rank's shard of the residual stream (in/out)
  const void* norm_weight;        // [H]
  float eps;
  int add_residual;
  uint32_t* local_sync;           // [2] CTA ticket, [3] last finished epoch of this kernel
  long long wait_cycles;
  StatusWord* status;
};

// All-reduce + residual + RMSNorm through the switch (comm_nvls_ar_norm.cu).  `*_mc` are addresses inside ONE
// multicast mapping of a symmetric buffer; `flag_local` is this rank's own copy of the two flag words.
struct NvlsArNormParams {
  int T, H, tp, rank, rows_per_rank;
  const void* partial_mc;         // [T_cap, H] the GEMM outputs of all ranks behind one address (multimem.ld_reduce)
  void* out_mc;                   // [T_cap, H] normalised rows, written on every rank (multimem.st)
  uint32_t* flag_mc;              // [2] arrival counters (multimem.red.add)
  const uint32_t* flag_local;     // [2] this rank's copy of them (polled)
  void* residual;                 // [rows_per_rank, H] this rank's shard of the residual stream (in/out)
  const void* norm_weight;        // [H]
  float eps;
  int add_residual;
  uint32_t* local_sync;           // [0] CTA ticket, [1] number of finished calls
  long long wait_cycles;
  StatusWord* status;
};

// All-gather -> GEMM (comm_ag_gemm.cu): C[tp*R, N] = concat_r(X_r[R, K]) . W[N, K]^T.
struct AgGemmParams {
  int rows_per_rank, N, K, tp, rank, ldc;
  void* x_shard[kMaxRanks];        // [rows_per_rank, K] 16-bit, contiguous (symmetric)
  uint32_t* xready[kMaxRanks];     // [tp] epoch written by each source: "my shard may be pulled"
  uint32_t* done[kMaxRanks];       // [1] pulls completed on the owner's shard (monotonic counter)
  void* gathered;                  // local [tp*rows_per_rank, K]
  uint32_t* ready;                 // local [tp*rows_per_rank/128] epoch per landed row block
  uint32_t* sync;                  // local [3]: last finished epoch, CTAs-left counter, pulls expected so far
  long long wait_cycles;
  StatusWord* status;
};

// Expert-parallel all-to-all (comm_moe_a2a.cu).  Pointer arrays are indexed by the rank that OWNS the memory.
struct MoeA2aParams {
  int ep, rank, experts_per_rank, H, topk, T, cap, quant;   // cap: tokens one source may send to one destination
  void* recv_x[kMaxRanks];          // [ep*cap][H] 16-bit rows, or e4m3 rows when quant
  float* recv_scale[kMaxRanks];     // [ep*cap][H/128] (quant only)
  int* recv_ids[kMaxRanks];         // [ep*cap][topk] local expert ids of the token, -1 = not on this rank / empty slot
  float* recv_w[kMaxRanks];         // [ep*cap][topk] routing weights (0 where the id is -1)
  int* recv_src[kMaxRanks];         // [ep*cap] token index at the source
  uint32_t* recv_count[kMaxRanks];  // [ep] rows pushed by each source
  uint32_t* disp_flag[kMaxRanks];   // [ep] dispatch epoch per source
  void* comb_x[kMaxRanks];          // [ep (rank that computed)][cap][H] 16-bit partial sums
  uint32_t* comb_flag[kMaxRanks];   // [ep] combine epoch per source
  uint32_t* local_sync;             // [0] ticket, [1] dispatch epoch, [2] combine epoch, [8+r] send counters
  long long wait_cycles;
  StatusWord* status;
};

// Stand-alone all-reduce over peer memory (comm_allreduce.cu).  Pointer arrays are indexed by the rank that OWNS
// the memory.
struct CustomArParams {
  int tp, rank;
  long long n_bytes;                // payload, multiple of 16
  long long cap_bytes;              // stride of one (parity, source) slot of recv and of one parity half of gather
  void* recv[kMaxRanks];            // [2 parity][tp source][cap_bytes] pushed inputs (one-shot) or segments (two-shot)
  void* gather[kMaxRanks];          // [2 parity][cap_bytes] reduced segments written by their owners (two-shot)
  uint32_t* flag1[kMaxRanks];       // [tp source][max_ctas] epoch per pushing CTA
  uint32_t* flag2[kMaxRanks];       // [tp source][max_ctas] epoch per CTA after its reduced segment is out
  int max_ctas;
  uint32_t* local_sync;             // [0] ticket, [1] last finished epoch
  long long wait_cycles;
  StatusWord* status;
};

// Cross-rank RMSNorm over a hidden dimension that is split across ranks (comm_allreduce.cu): the per-token sums of
// squares travel as 4-byte values whose arrival is their own flag (-0.0 = "not yet written").
struct ReduceRmsParams {
  int tp, rank, T, n_tensors;       // up to two tensors (q and k) per launch
  const void* x[2];
  const void* w[2];
  void* out[2];
  int H[2];                         // local width of each tensor (multiple of 8)
  int ld[2];                        // row pitch of x / out in elements
  float eps;
  float* slots[kMaxRanks];          // [3 buffers][2 tensors][tp source][t_cap]
  int t_cap;
  uint32_t* local_sync;             // [0] ticket, [1] calls finished, [2 + b] tokens of the last call that used buffer b
  long long wait_cycles;
  StatusWord* status;
};

}  // namespace b200
