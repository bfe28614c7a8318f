// Host-callable launchers of every CUDA kernel in this library.  The .cu files are
// free of torch headers; bindings.cpp adapts torch tensors to these entry points.
// dtype codes: 0 = bf16, 1 = fp16, 2 = fp32.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "status.h"
#include "comm_params.h"

namespace b200 {

struct DecodeParams {
  void* out;                 // [T, Hq, D] (T dtype)
  float* part_out;           // [splits, T, Hq, D]
  float* part_lse;           // [splits, T, Hq]
  const void* q;             // [T, Hq, D] with token stride q_stride (elements)
  const void* kv_cache;
  const float* kv_scales;    // kinds 1, 2
  const int* block_table;    // [B, max_blocks]
  const int* seq_lens;       // [B]
  const int* query_start_loc;  // [B+1] or null (one token per sequence)
  const float* sinks;        // [Hq] or null
  const float* alibi_slopes; // [Hq] or null: score += slope * (kv position - query position)
  float* lse_out;            // [Hq, T] or null (natural-log LSE of the final result)
  int64_t q_stride;
  int num_q_heads, num_kv_heads, block_size, max_blocks, num_splits, total_tokens;
  int64_t num_blocks;
  float scale, softcap, k_scale, v_scale;
  int window;                // <=0: none
  int causal;
  StatusWord* status;
};

struct PrefillParams {
  void* out;                     // [T, Hq, DV]
  float* lse_out;                // [Hq, T] or null
  const int* block_table;        // [B, max_blocks] (paged) or null
  const int* seq_lens;           // [B] kv length (paged) ; contiguous: derived from kv_start_loc
  const int* query_start_loc;    // [B+1]
  const int* kv_start_loc;       // [B+1] (contiguous mode) or null
  const float* sinks;            // [Hq] or null
  const float* alibi_slopes;     // [Hq] or null
  int num_q_heads, num_kv_heads, gp;  // gp: heads packed per tile (divides 128)
  int block_size, max_blocks;
  int64_t num_blocks;
  int total_q;
  float scale, softcap;
  int window, causal, paged;
  StatusWord* status;
};

struct MlaDecodeParams {
  void* out;                   // [T, H, 512]
  float* lse_out;              // [H, T] or null
  float* part_out;             // [splits, T, H, 512]
  float* part_lse;             // [splits, T, H]
  const void* q;               // [T, H, 576], token stride q_stride (elements)
  const void* cache;           // latent cache (bf16 576 rows or 656-byte fp8 records)
  const int* block_table;      // [B, max_blocks]
  const int* seq_lens;         // [B]
  const int* query_start_loc;  // [B+1] or null (one token per sequence)
  const int* topk_indices;     // [T, topk] per-request positions (-1 = none) or null (dense)
  int64_t q_stride;
  int num_heads, block_size, max_blocks, num_splits, total_tokens, batch, topk;
  int64_t num_blocks;
  float scale;
  StatusWord* status;
};

// ---- gemm_tcgen05.cu
void gemm_tn(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
             int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int force_bn, int epi);
// gemm_streamk_tcgen05.cu: swap-AB CTA-pair stream-K for skinny problems (scratch supplied by the caller)
size_t gemm_streamk_workspace_bytes(int sms);
int gemm_streamk_max_tiles();
int gemm_tn_streamk(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                    int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int epi,
                    float* ws, int* counters, int sms, const struct RowScatter* scatter = nullptr);
void gemm_tn_pair(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                  int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int epi,
                  const struct RowScatter* scatter = nullptr);
// ---- comm_ar_norm.cu
int ar_norm_gather(const ArNormParams& p, int dtype, cudaStream_t stream);
int nvls_ar_norm(const NvlsArNormParams& p, int dtype, cudaStream_t stream);
// ---- gemm_splitk_tcgen05.cu
int gemm_splitk_choice(int M, int N, int K, int sms);
void gemm_tn_splitk(const void* A, const void* W, void* C, const void* bias, const void* residual, int M, int N, int K,
                    int lda, int ldw, int ldc, int ldr, int dtype, cudaStream_t stream, void* status, int epi,
                    int splits);
// ---- norm.cu
void rms_norm(void* out, void* x, void* residual, const void* weight, float eps, int tokens, int hidden,
              int64_t x_stride, int64_t out_stride, int dtype, int mode, cudaStream_t stream);
void head_rms_norm(void* x, const void* weight, float eps, int tokens, int heads, int head_dim, int64_t token_stride,
                   int dtype, cudaStream_t stream);
void rms_norm_quant(void* out_q, float* scale_out, const float* scale_in, const void* x, void* residual,
                    const void* weight, float eps, int tokens, int hidden, int dtype, int qmode, int group, int ue8m0,
                    float scale_ub, cudaStream_t stream);
// ---- rope_cache.cu
void rope_and_cache(const int64_t* positions, void* q, void* k, const void* v, const float* cos_sin, int rot,
                    int head_dim, int num_q, int num_kv, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                    int is_neox, int rot_offset, int inverse, void* kv_cache, float* kv_scales,
                    const int64_t* slot_mapping, int block_size, int64_t num_slots, int cache_kind, float k_scale,
                    float v_scale, int tokens, int dtype, void* status, cudaStream_t stream);
void copy_blocks(void* cache, const int64_t* pairs, int num_pairs, int64_t block_bytes, cudaStream_t stream);
void concat_and_cache_mla(const void* kv_c, const void* k_pe, void* cache, const int64_t* slot_mapping, int tokens,
                          int rank, int rope, int64_t kvc_stride, int64_t kpe_stride, int64_t num_slots,
                          int fp8_record, int dtype, void* status, cudaStream_t stream);
void indexer_k_quant_and_cache(const void* k, void* cache, const int64_t* slot_mapping, int tokens, int head_dim,
                               int block_size, int64_t num_slots, int64_t k_stride, int ue8m0, int dtype, void* status,
                               cudaStream_t stream, int kind = 0);
// ---- activation.cu
void act_and_mul(void* out, const void* x, int tokens, int d, int64_t x_stride, int64_t out_stride, int act, float p0,
                 float p1, int dtype, cudaStream_t stream);
void activation(void* out, const void* x, int64_t n, int act, float p0, int dtype, cudaStream_t stream);
void act_and_mul_quant(void* out_q, float* scale_out, const float* scale_in, const void* x, int tokens, int d, int act,
                       float p0, float p1, int group, int ue8m0, int dtype, cudaStream_t stream);
// ---- attention
int paged_attention_decode(const DecodeParams& p, int head_dim, int kv_kind, int dtype, int batch, int max_q_len,
                           cudaStream_t stream);
int attention_prefill(const PrefillParams& p, const void* q, int64_t q_stride, const void* k_src, const void* v_src,
                      int64_t k_tok_stride, int64_t v_tok_stride, int64_t total_kv, int dqk, int dv, int dtype,
                      int batch, int max_q_len, cudaStream_t stream);
// attn_prefill_pingpong.cu: two query tiles per CTA, P and O resident in TMEM
int attention_prefill_pp(const PrefillParams& p, const void* q, int64_t q_stride, const void* k_src, const void* v_src,
                      int64_t k_tok_stride, int64_t v_tok_stride, int64_t total_kv, int dqk, int dv, int dtype,
                      int batch, int max_q_len, cudaStream_t stream);
// ---- sampling.cu
void argmax(int64_t* out, const void* logits, int rows, int vocab, int64_t stride, int dtype, cudaStream_t stream);
void sample(int64_t* out, const void* logits, int rows, int vocab, int64_t stride, const float* temperature,
            const int* top_k, const float* top_p, const float* min_p, const float* uniform, int dtype,
            cudaStream_t stream);
void apply_penalties(void* logits, const int* prompt_mask, const int* output_counts, const float* rep,
                     const float* presence, const float* frequency, int rows, int vocab, int64_t stride, int dtype,
                     cudaStream_t stream);
void advance_step(int64_t* input_ids, int64_t* positions, int* seq_lens, int64_t* slot_mapping, const int64_t* sampled,
                  const int* block_table, int max_blocks, int block_size, int batch, int64_t* token_log, int log_col,
                  int log_stride, cudaStream_t stream);
void embedding(void* out, const void* table, const int64_t* ids, int tokens, int hidden, int64_t vocab,
               int64_t vocab_start, int dtype, cudaStream_t stream);

// ---- moe.cu / gemm_grouped_tcgen05.cu
void topk_gating(float* weights, int* ids, const void* gating, const float* bias, int tokens, int experts, int topk,
                 int mode, int renorm, float scale, int dtype, cudaStream_t stream);
void grouped_topk(float* weights, int* ids, const void* gating, const float* bias, int tokens, int experts, int topk,
                  int n_group, int topk_group, int sigmoid, int renorm, float scale, int dtype, cudaStream_t stream);
void moe_align(int* sorted_ids, int* block_expert, int* total_padded, int* inv_pos, const int* topk_ids,
               const int* expert_map, int numel, int experts, int block, int max_padded, cudaStream_t stream);
void moe_gather(void* out, const void* x, const int* sorted_ids, const int* total_padded, int max_padded, int numel,
                int topk, int hidden, int dtype, cudaStream_t stream);
void moe_combine(void* out, const void* y, const float* weights, const int* inv_pos, const void* shared, int tokens,
                 int topk, int hidden, int dtype, cudaStream_t stream);
void moe_sum(void* out, const void* in, int tokens, int topk, int hidden, int dtype, cudaStream_t stream);
void gemm_grouped(const void* A, int max_rows, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                  const int* block_expert, const int* total_padded, int epi, int dtype, cudaStream_t stream,
                  void* status);
// ---- quant.cu / gemm_fp8_blockscale.cu
void per_token_group_quant(void* q, float* scales, const void* x, int64_t rows, int K, int group, int int8, int ue8m0,
                           int col_major, float eps, int dtype, cudaStream_t stream);
void scaled_fp8_quant(void* q, float* scale, const void* x, int64_t rows, int K, int mode, float scale_ub, int dtype,
                      cudaStream_t stream);
void scaled_int8_quant(void* q, float* scale, int* azp, const void* x, int64_t rows, int K, int mode, int dtype,
                       cudaStream_t stream);
void merge_attn_states(void* out, float* out_lse, const void* p_out, const float* p_lse, const void* s_out,
                       const float* s_lse, int tokens, int heads, int D, int dtype, cudaStream_t stream);
void gemm_fp8_blockscale(const void* A, int M, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                         const float* a_scale, const float* w_scale, const int* block_expert,
                         const int* total_padded, int grouped, int out_dtype, cudaStream_t stream, void* status);
// ---- gemm_scaled_mm.cu
void gemm_scaled_mm(const void* A, int M, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                    const float* a_scale, int a_per_row, const float* w_scale, int w_per_col, const int* azp,
                    const int* azp_adj, const void* bias, const int* block_expert, const int* total_padded,
                    int grouped, int kind, int out_dtype, cudaStream_t stream, void* status);
// ---- gemm_wna16_tcgen05.cu
int gemm_wna16_token_tile(int M);
int gemm_wna16_splits(int M, int N, int K, int bn);
void gemm_wna16(const void* A, int M, int lda, const void* Q, const void* scales, const void* zeros, int E, int N,
                int K, int group, int bits, void* C, int ldc, const void* bias, float* partial, int splits,
                const int* block_expert, const int* total_padded, int grouped, int token_tile, int epi, int dtype,
                cudaStream_t stream, void* status);
// ---- small_gemm.cu
int small_gemm(void* C, const void* A, const void* W, const void* bias, int M, int N, int K, int lda, int ldw, int ldc,
               int dtype, int out_kind, cudaStream_t stream);
// ---- fused_misc.cu
int qkv_norm_rope_insert(void* qkv, int64_t row_stride, const void* q_w, const void* k_w, const void* iq_w,
                         const void* ik_w, const float* cos_sin, const int64_t* positions, const int64_t* slot_mapping,
                         void* q_out, void* iq_out, void* kv_cache, void* idx_cache, int tokens, int insert_tokens, int hq,
                         int hk, int niq, int has_ik, int insert_v, int rot, int is_neox, int gemma, int idx_fp8,
                         int block_size, int64_t num_slots, float eps, int dtype, cudaStream_t stream);
int fused_qk_norm_rope(void* qkv, const void* q_weight, const void* k_weight, const float* cos_sin,
                       const int64_t* positions, int tokens, int hq, int hk, int hv, int head_dim, int rot, int is_neox,
                       float eps, int gemma, int dtype, cudaStream_t stream);
void mla_rope_and_cache(void* q_pe, void* k_pe, const void* kv_c, void* cache, const float* cos_sin,
                        const int64_t* positions, const int64_t* slots, int tokens, int heads, int64_t q_tok_stride,
                        int64_t kpe_stride, int64_t kvc_stride, int is_neox, int64_t num_slots, int dtype,
                        cudaStream_t stream);
void concat_mla_q(void* out, const void* nope, const void* pe, int64_t rows, int64_t nope_stride, int64_t pe_stride,
                  int dtype, cudaStream_t stream);
void permute_cols(void* out, const void* a, const int* perm, int64_t rows, int cols, int64_t lda, int dtype,
                  cudaStream_t stream);
void gather_mla_cache(void* dst, const void* cache, const int* block_table, const int* cu_seq_lens,
                      const int* seq_starts, int batch, int max_blocks, int block_size, int max_total, int records,
                      int dtype, cudaStream_t stream);
void gather_indexer_k(void* dst_k, float* dst_s, const void* cache, const int* block_table, const int* cu_seq_lens,
                      int batch, int max_blocks, int block_size, int max_total, cudaStream_t stream);
// ---- mamba_scan.cu
struct ScanParams {
  const void* u; const void* delta; const void* z; void* out;
  const float* A;                 // [dim, dstate]
  const void* B; const void* C;   // [(batch,) groups, dstate, tokens]
  const float* D;                 // [dim] or null
  const float* delta_bias;        // [dim] or null
  float* state;                   // [slots, dim, dstate] fp32
  const int* query_start_loc;     // [batch+1] or null (dense layout)
  const int* cache_indices;       // [batch] or null (slot = b)
  const uint8_t* has_initial_state;  // [batch] or null (no initial state)
  int batch, dim, dstate, groups, seqlen, total_tokens, softplus, pad_slot;
};
int selective_scan_fwd(const ScanParams& p, int dtype, cudaStream_t stream);
// ---- mhc.cu
struct MhcParams {
  const void* residual;   // [T, M, H] (input streams)
  void* residual_out;     // fused: new streams [T, M, H] (a different buffer than residual)
  const void* y;          // fused: sub-layer output [T, H]
  const float* post_in;   // fused: [T, M]
  const float* comb_in;   // fused: [T, M, M]
  const float* fn;        // [mix, M*H]
  const float* scale;     // [3] (head: [1])
  const float* base;      // [mix]
  float* post_out;        // [T, M]
  float* comb_out;        // [T, M, M]
  void* x_out;            // [T, H]
  int T, M, H, iters, head;
  float rms_eps, pre_eps, sinkhorn_eps, post_mult;
};
int mhc_pre(const MhcParams& p, int fused, int dtype, cudaStream_t stream);
void mhc_post(void* out, const void* y, const void* res, const float* post, const float* comb, int tokens, int M, int H,
              int dtype, cudaStream_t stream);
// ---- p2p_copy.cu
void p2p_copy(void* dst, const void* src, size_t nbytes, int ctas, int mode, void* status, cudaStream_t stream);
// ---- comm_ag_gemm.cu
int ag_gemm_copiers(int tp, int rows_per_rank);
int ag_gemm(const AgGemmParams& p, const void* W, int ldw, void* C, const void* bias, int dtype, cudaStream_t stream);
// ---- comm_moe_a2a.cu
void moe_a2a_dispatch(const MoeA2aParams& p, const void* x, const int* topk_ids, const float* topk_w, int dtype,
                      cudaStream_t stream);
void moe_a2a_combine(const MoeA2aParams& p, const void* y, void* out, const int* topk_ids, const void* shared_out,
                     int dtype, cudaStream_t stream);
void gather_rows(void* dst, const void* src, const int* idx, const int* count, int max_rows, int limit, int row_bytes,
                 int div, cudaStream_t stream);
// ---- v4_cache.cu
void v4_qnorm_rope_kv_insert(const void* q_in, int64_t q_stride_t, int64_t q_stride_h, const void* kv, int64_t kv_stride,
                             void* q_out, void* cache, int64_t block_stride, const int64_t* slot_mapping,
                             const int64_t* positions, const float* cos_sin, int tokens, int insert_tokens, int hq,
                             int hq_pad, int block_size, float eps, cudaStream_t stream);
void v4_gather_dequant(void* dst, const void* cache, int64_t block_stride, const int64_t* slots, int n, int block_size,
                       cudaStream_t stream);
void v4_inv_rope(void* out, const void* o, int64_t o_stride_t, int64_t o_stride_h, const int64_t* positions,
                 const float* cos_sin, int tokens, int heads, int hpg, int dtype, cudaStream_t stream);
void v4_indexer_q(void* q8, float* w_out, const void* q, int64_t q_stride_t, int64_t q_stride_h, const void* weights,
                  int64_t w_stride, const int64_t* positions, const float* cos_sin, int tokens, int heads, int rot,
                  float softmax_scale, float head_scale, int dtype, cudaStream_t stream);
// ---- gdn.cu
int gdn_recurrent(void* out, float* state, const void* q, const void* k, const void* v, const float* g, const float* beta,
                  const int* query_start_loc, const int* state_idx, int batch, int hq, int hv, int dk, int dv,
                  int64_t q_stride, int64_t k_stride, int64_t v_stride, float scale, int l2norm,
                  const int* has_initial, int dtype, cudaStream_t stream);
// ---- causal_conv1d.cu (depthwise causal convolution over ragged batches with a per-sequence carry)
int causal_conv1d(void* out, const void* x, int64_t x_stride, const void* w, const void* bias, void* state,
                  const int* query_start_loc, const int* state_idx, const int* has_init, int batch, int tokens,
                  int channels, int K, int silu, int dtype, cudaStream_t stream);
// ---- tq_cache.cu (TurboQuant KV cache, head_dim 128)
int tq_slot_bytes(int kbits, int vbits);
int tq_store(void* cache, const void* k, const void* v, int64_t k_stride, int64_t v_stride, const int64_t* slot_mapping,
             int tokens, int heads, int64_t num_slots, int kbits, int vbits, int nc, int dtype, cudaStream_t stream);
int tq_dequant(void* k_out, void* v_out, const void* cache, const int64_t* slots, int rows, int heads, int kbits, int vbits,
               int nc, int dtype, cudaStream_t stream);
int tq_decode(void* out, float* part_out, float* part_lse, const void* q, int64_t q_stride, const void* cache,
              const int* block_table, int max_blocks, const int* seq_lens, int batch, int hq, int hkv, int block_size,
              int64_t num_blocks, int splits, float scale, int kbits, int vbits, int nc, int dtype, cudaStream_t stream);
// ---- comm_allreduce.cu
int custom_allreduce(const CustomArParams& p, const void* in, void* out, int dtype, int mode, cudaStream_t stream);
int reduce_rms(const ReduceRmsParams& p, int dtype, cudaStream_t stream);
// ---- mla_decode.cu
// impl: 0 = choose (tcgen05 kernel for dense 16-bit caches from 64 heads per rank up), 1 = mma.sync kernel,
// 2 = tcgen05 kernel or fail.  Returns 0, or -1 when impl 2 was asked for and that kernel does not serve the call.
int mla_decode(const MlaDecodeParams& p, int fp8_records, int dtype, cudaStream_t stream, int impl = 1);
// ---- mla_decode_tcgen05.cu: 0 = launched, -1 = not served
int mla_decode_tc(const MlaDecodeParams& p, int dtype, cudaStream_t stream);
// ---- indexer.cu
void indexer_logits(float* logits, int64_t logits_stride, const void* q, const float* w, const void* cache,
                    const int* block_table, int max_blocks, const int* seq_lens, const int* query_start_loc,
                    int tokens, int batch, int heads, int block_size, int64_t num_blocks, int max_len, void* status,
                    cudaStream_t stream, int kind = 0);   // kind 1: int8 queries and keys
// ---- indexer_tcgen05.cu: returns -1 when the shapes are not served (caller falls back to indexer_logits)
int indexer_logits_tc(float* logits, int64_t logits_stride, const void* q, const float* w, const void* cache,
                      const int* block_table, int max_blocks, const int* seq_lens, const int* query_start_loc,
                      int tokens, int batch, int heads, int block_size, int64_t num_blocks, int max_len,
                      int max_query_len, void* status, cudaStream_t stream, int kind);
void topk_per_row(int* out, const float* x, int64_t stride, const int* row_len, int rows, int cols, int k,
                  cudaStream_t stream);
// ---- comm_gemm_ar_norm.cu (FusedArParams: comm_params.h)
struct FusedArParams;
int gemm_ar_norm(const FusedArParams& p, const void* A, int lda, const void* W, int ldw, int dtype,
                 cudaStream_t stream);

}  // namespace b200
