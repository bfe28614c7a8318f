// torch.ops.b200.* : adapts torch tensors to the torch-free launchers in ops.h.
// Every op writes into caller-provided tensors (no allocation here), so the ops can
// be captured in CUDA graphs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <cstdlib>
#include <cstring>
#include <tuple>

#include "comm_params.h"
#include "ops.h"

namespace {

using at::Tensor;
using c10::optional;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline int dtype_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return 0;
    case at::kHalf: return 1;
    case at::kFloat: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
inline int dtype16(const Tensor& t) {
  const int c = dtype_code(t);
  TORCH_CHECK(c < 2, "expected a bf16 / fp16 tensor");
  return c;
}
template <typename T = void>
inline T* ptr(const optional<Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

// One status word per device, zero-initialised on first use.
Tensor& status_tensor(int device) {
  static std::vector<Tensor> words(64);
  if (!words[device].defined())
    words[device] = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  return words[device];
}
inline void* status_ptr(const Tensor& any) { return status_tensor(any.get_device()).data_ptr(); }

Tensor get_status(int64_t device) { return status_tensor((int)device); }

// ------------------------------------------------------------------ GEMM
// Scratch of the stream-K GEMM (partial tiles + arrival counters): allocated once per device, stream-ordered use.
struct StkScratch {
  float* ws;
  int* counters;
  int sms;
};
static StkScratch stk_scratch(const Tensor& like) {
  // leaked on purpose: destroying CUDA tensors from static destructors can outlive the allocator
  static Tensor* ws = new Tensor[64];
  static Tensor* counters = new Tensor[64];
  static int sms_k[64] = {};
  const int dev = like.get_device();
  TORCH_CHECK(dev >= 0 && dev < 64);
  if (sms_k[dev] == 0) cudaDeviceGetAttribute(&sms_k[dev], cudaDevAttrMultiProcessorCount, dev);
  if (!ws[dev].defined()) {
    ws[dev] = torch::empty({(int64_t)(b200::gemm_streamk_workspace_bytes(sms_k[dev]) / 4)},
                           like.options().dtype(at::kFloat));
    counters[dev] = torch::zeros({2 * (int64_t)b200::gemm_streamk_max_tiles()}, like.options().dtype(at::kInt));
  }
  return {ws[dev].data_ptr<float>(), counters[dev].data_ptr<int>(), sms_k[dev]};
}

void gemm(Tensor& out, const Tensor& a, const Tensor& w, const optional<Tensor>& bias,
          const optional<Tensor>& residual, int64_t force_bn, int64_t epi) {
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm expects 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1, "inner dims must be contiguous");
  const int M = a.size(0), K = a.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == M && out.size(1) == (epi == 1 ? N / 2 : N), "gemm shape mismatch");
  TORCH_CHECK(epi == 0 || (!residual.has_value() && N % 16 == 0), "gated epilogue: no residual, N % 16 == 0");
  TORCH_CHECK(K % 8 == 0 && a.stride(0) % 8 == 0 && w.stride(0) % 8 == 0 && out.stride(0) % 8 == 0,
              "gemm: K and row pitches must be multiples of 8 elements");
  TORCH_CHECK(a.scalar_type() == w.scalar_type() && a.scalar_type() == out.scalar_type(), "gemm dtype mismatch");
  int ldr = 0;
  if (residual.has_value()) {
    TORCH_CHECK(residual->stride(1) == 1 && residual->size(0) == M && residual->size(1) == N);
    ldr = residual->stride(0);
  }
  const c10::cuda::CUDAGuard guard(a.device());
  // CTA-pair (cta_group::2) kernel for large problems: at least one 256 x 256 tile per pair of SMs.
  static const bool pair_default = [] {
    const char* e = std::getenv("B200_GEMM_PAIR");
    return e == nullptr || std::atoi(e) != 0;
  }();
  const int64_t pair_tiles = ((M + 255) / 256) * (int64_t)((N + 255) / 256);
  // (a full 256-token decode batch against a wide weight, e.g. gate_up, already gives every CTA pair a tile)
  if (force_bn == 512 || (force_bn == 0 && pair_default && ((M >= 512 && pair_tiles >= 64) ||
                                                             (M >= 256 && pair_tiles >= 96)))) {
    b200::gemm_tn_pair(a.data_ptr(), w.data_ptr(), out.data_ptr(), ptr(bias), ptr(residual), M, N, K, a.stride(0),
                       w.stride(0), out.stride(0), ldr, dtype16(a), cur_stream(), status_ptr(a), (int)epi);
    return;
  }
  // stream-K over CTA pairs for skinny problems: decode batches and narrow tensor-parallel shards (force_bn 2000
  // pins it).  Its scratch (partial tiles + arrival counters) is allocated once per device and stream-ordered
  // use is assumed, like every other op of this library.
  static const bool streamk_default = [] {
    const char* e = std::getenv("B200_GEMM_STREAMK");
    return e == nullptr || std::atoi(e) != 0;
  }();
  {
    StkScratch sk = stk_scratch(a);
    const int64_t tiles = ((M + 255) / 256) * (int64_t)((N + 255) / 256);
    // measured inside replayed graphs: with up to 64 tokens the partial tiles are small and streaming over all SMs
    // wins; at 256 tokens the 128 KB partials make the fix-up cost more than the balanced stream saves
    if (force_bn == 2000 || (force_bn == 0 && streamk_default && M <= 64 && K >= 1024 && tiles <= 2 * sk.sms)) {
      const int rc = b200::gemm_tn_streamk(a.data_ptr(), w.data_ptr(), out.data_ptr(), ptr(bias), ptr(residual), M, N,
                                           K, a.stride(0), w.stride(0), out.stride(0), ldr, dtype16(a), cur_stream(),
                                           status_ptr(a), (int)epi, sk.ws, sk.counters, sk.sms);
      if (rc == 0) return;
      TORCH_CHECK(force_bn != 2000, "gemm: shape outside the stream-K kernel's scratch");
    }
  }
  // cluster split-K for medium M with too few tiles to cover the GPU (force_bn 1002 / 1004 pins the split count)
  static const bool splitk_default = [] {
    const char* e = std::getenv("B200_GEMM_SPLITK");
    return e == nullptr || std::atoi(e) != 0;
  }();
  static int sms = 0;
  if (sms == 0) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, a.get_device());
  int splits = 1;
  if (force_bn == 1002 || force_bn == 1004) splits = (int)force_bn - 1000;
  else if (force_bn == 0 && splitk_default && M > 64 && M <= 1024) splits = b200::gemm_splitk_choice(M, N, K, sms);
  if (splits > 1) {
    b200::gemm_tn_splitk(a.data_ptr(), w.data_ptr(), out.data_ptr(), ptr(bias), ptr(residual), M, N, K, a.stride(0),
                         w.stride(0), out.stride(0), ldr, dtype16(a), cur_stream(), status_ptr(a), (int)epi, splits);
    return;
  }
  b200::gemm_tn(a.data_ptr(), w.data_ptr(), out.data_ptr(), ptr(bias), ptr(residual), M, N, K, a.stride(0),
                w.stride(0), out.stride(0), ldr, dtype16(a), cur_stream(), status_ptr(a), (int)force_bn, (int)epi);
}

// ------------------------------------------------------------------ norms
void rms_norm(Tensor& out, const Tensor& x, const Tensor& weight, double eps, bool gemma) {
  const int hidden = x.size(-1);
  const int tokens = x.numel() / hidden;
  const c10::cuda::CUDAGuard guard(x.device());
  b200::rms_norm(out.data_ptr(), x.data_ptr(), nullptr, weight.data_ptr(), (float)eps, tokens, hidden,
                 x.dim() >= 2 ? x.stride(-2) : hidden, out.dim() >= 2 ? out.stride(-2) : hidden, dtype16(x),
                 gemma ? 1 : 0, cur_stream());
}
void fused_add_rms_norm(Tensor& x, Tensor& residual, const Tensor& weight, double eps, bool gemma) {
  const int hidden = x.size(-1);
  const int tokens = x.numel() / hidden;
  TORCH_CHECK(residual.is_contiguous(), "residual must be contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  b200::rms_norm(x.data_ptr(), x.data_ptr(), residual.data_ptr(), weight.data_ptr(), (float)eps, tokens, hidden,
                 x.dim() >= 2 ? x.stride(-2) : hidden, x.dim() >= 2 ? x.stride(-2) : hidden, dtype16(x),
                 gemma ? 1 : 0, cur_stream());
}
void head_rms_norm(Tensor& x, const Tensor& weight, double eps, int64_t heads, int64_t head_dim) {
  // x: [T, >= heads*head_dim] view whose first heads*head_dim columns are normalised per head
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(head_dim % 32 == 0 && head_dim <= 256);
  b200::head_rms_norm(x.data_ptr(), weight.data_ptr(), (float)eps, x.size(0), heads, head_dim, x.stride(0), dtype16(x),
                      cur_stream());
}
void rms_norm_quant(Tensor& out_q, const optional<Tensor>& scale_out, const optional<Tensor>& scale_in,
                    const Tensor& x, const optional<Tensor>& residual, const Tensor& weight, double eps, int64_t qmode,
                    int64_t group, bool ue8m0, double scale_ub) {
  const int hidden = x.size(-1);
  const int tokens = x.numel() / hidden;
  TORCH_CHECK(x.is_contiguous() && out_q.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  b200::rms_norm_quant(out_q.data_ptr(), ptr<float>(scale_out), ptr<float>(scale_in), x.data_ptr(), ptr(residual),
                       weight.data_ptr(), (float)eps, tokens, hidden, dtype16(x), qmode, group, ue8m0, (float)scale_ub,
                       cur_stream());
}

// ------------------------------------------------------------------ rope / cache
void rope_and_cache(const optional<Tensor>& positions, const optional<Tensor>& q, const optional<Tensor>& k,
                    const optional<Tensor>& v, const optional<Tensor>& cos_sin, int64_t head_dim, int64_t num_q,
                    int64_t num_kv, bool is_neox, int64_t rot_offset, bool inverse, const optional<Tensor>& kv_cache,
                    const optional<Tensor>& kv_scales, const optional<Tensor>& slot_mapping, int64_t cache_kind,
                    double k_scale, double v_scale) {
  const Tensor& any = q.has_value() ? *q : *k;
  const int tokens = any.size(0);
  int rot = 0;
  if (cos_sin.has_value()) {
    TORCH_CHECK(cos_sin->scalar_type() == at::kFloat && cos_sin->is_contiguous(), "cos_sin cache must be f32");
    rot = cos_sin->size(-1);
  }
  int block_size = 0;
  int64_t num_slots = 0;
  if (kv_cache.has_value()) {
    TORCH_CHECK(kv_cache->dim() == 5 && kv_cache->is_contiguous(), "kv cache must be [nb,2,bs,Hkv,D] contiguous");
    block_size = kv_cache->size(2);
    num_slots = kv_cache->size(0) * block_size;
    TORCH_CHECK(slot_mapping.has_value() && slot_mapping->scalar_type() == at::kLong);
  }
  if (positions.has_value()) TORCH_CHECK(positions->scalar_type() == at::kLong);
  TORCH_CHECK(head_dim <= 576);
  const c10::cuda::CUDAGuard guard(any.device());
  b200::rope_and_cache(ptr<int64_t>(positions), ptr(q), ptr(k), ptr(v), ptr<float>(cos_sin), rot, head_dim,
                       q.has_value() ? num_q : 0, num_kv, q.has_value() ? q->stride(0) : 0,
                       k.has_value() ? k->stride(0) : 0, v.has_value() ? v->stride(0) : 0, is_neox, rot_offset, inverse,
                       ptr(kv_cache), ptr<float>(kv_scales), ptr<int64_t>(slot_mapping), block_size, num_slots,
                       cache_kind, (float)k_scale, (float)v_scale, tokens, dtype16(any), status_ptr(any), cur_stream());
}
void copy_blocks(Tensor& cache, const Tensor& pairs) {
  TORCH_CHECK(pairs.scalar_type() == at::kLong && pairs.is_contiguous() && cache.is_contiguous());
  const int64_t block_bytes = cache.stride(0) * cache.element_size();
  TORCH_CHECK(block_bytes % 16 == 0);
  const c10::cuda::CUDAGuard guard(cache.device());
  b200::copy_blocks(cache.data_ptr(), pairs.data_ptr<int64_t>(), pairs.size(0), block_bytes, cur_stream());
}
void concat_and_cache_mla(const Tensor& kv_c, const Tensor& k_pe, Tensor& cache, const Tensor& slot_mapping) {
  const bool rec = cache.scalar_type() == at::kByte;
  const int rank = kv_c.size(-1), rope = k_pe.size(-1);
  if (rec) TORCH_CHECK(rank == 512 && rope == 64 && cache.size(-1) == 656, "fp8_ds_mla needs 512+64 and 656-byte records");
  const int64_t num_slots = cache.size(0) * cache.size(1);
  const c10::cuda::CUDAGuard guard(kv_c.device());
  b200::concat_and_cache_mla(kv_c.data_ptr(), k_pe.data_ptr(), cache.data_ptr(), slot_mapping.data_ptr<int64_t>(),
                             kv_c.size(0), rank, rope, kv_c.stride(0), k_pe.stride(0), num_slots, rec, dtype16(kv_c),
                             status_ptr(kv_c), cur_stream());
}
void indexer_k_quant_and_cache(const Tensor& k, Tensor& cache, const Tensor& slot_mapping, int64_t block_size,
                               bool ue8m0, bool int8) {
  const int hd = k.size(-1);
  TORCH_CHECK(hd % 32 == 0 && hd <= 128 && cache.scalar_type() == at::kByte);
  const int64_t num_slots = cache.size(0) * block_size;
  const c10::cuda::CUDAGuard guard(k.device());
  b200::indexer_k_quant_and_cache(k.data_ptr(), cache.data_ptr(), slot_mapping.data_ptr<int64_t>(), k.size(0), hd,
                                  block_size, num_slots, k.stride(0), ue8m0, dtype16(k), status_ptr(k), cur_stream(), int8 ? 1 : 0);
}

// ------------------------------------------------------------------ activations
void act_and_mul(Tensor& out, const Tensor& x, int64_t act, double p0, double p1) {
  const int d = x.size(-1) / 2;
  const int tokens = x.numel() / x.size(-1);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::act_and_mul(out.data_ptr(), x.data_ptr(), tokens, d, x.dim() >= 2 ? x.stride(-2) : 2 * d,
                    out.dim() >= 2 ? out.stride(-2) : d, act, (float)p0, (float)p1, dtype16(x), cur_stream());
}
void activation(Tensor& out, const Tensor& x, int64_t act, double p0) {
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  b200::activation(out.data_ptr(), x.data_ptr(), x.numel(), act, (float)p0, dtype16(x), cur_stream());
}
void act_and_mul_quant(Tensor& out_q, const optional<Tensor>& scale_out, const optional<Tensor>& scale_in,
                       const Tensor& x, int64_t act, double p0, double p1, int64_t group, bool ue8m0) {
  TORCH_CHECK(x.is_contiguous() && out_q.is_contiguous());
  const int d = x.size(-1) / 2;
  const int tokens = x.numel() / x.size(-1);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::act_and_mul_quant(out_q.data_ptr(), ptr<float>(scale_out), ptr<float>(scale_in), x.data_ptr(), tokens, d, act,
                          (float)p0, (float)p1, group, ue8m0, dtype16(x), cur_stream());
}

// ------------------------------------------------------------------ attention
int64_t kv_kind_of(const Tensor& cache, bool has_scales) {
  if (cache.scalar_type() == at::kChar) return 1;
  if (cache.scalar_type() == at::kFloat8_e4m3fn) return has_scales ? 2 : 3;
  return 0;
}

void paged_attention_decode(Tensor& out, const Tensor& q, const Tensor& kv_cache, const optional<Tensor>& kv_scales,
                            const Tensor& block_table, const Tensor& seq_lens,
                            const optional<Tensor>& query_start_loc, double scale, int64_t window, double softcap,
                            const optional<Tensor>& sinks, const optional<Tensor>& lse_out,
                            const optional<Tensor>& workspace, int64_t num_splits, int64_t batch, int64_t max_q_len,
                            double k_scale, double v_scale, bool causal, const optional<Tensor>& alibi_slopes) {
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2), "q must be [T, Hq, D] with packed heads");
  TORCH_CHECK(kv_cache.dim() == 5 && kv_cache.is_contiguous());
  TORCH_CHECK(block_table.scalar_type() == at::kInt && seq_lens.scalar_type() == at::kInt);
  TORCH_CHECK(out.is_contiguous());
  b200::DecodeParams p{};
  const int T = q.size(0), Hq = q.size(1), D = q.size(2);
  p.out = out.data_ptr();
  p.q = q.data_ptr();
  p.q_stride = q.stride(0);
  p.kv_cache = kv_cache.data_ptr();
  p.kv_scales = ptr<float>(kv_scales);
  p.block_table = block_table.data_ptr<int>();
  p.seq_lens = seq_lens.data_ptr<int>();
  p.query_start_loc = ptr<int>(query_start_loc);
  p.sinks = ptr<float>(sinks);
  p.alibi_slopes = ptr<float>(alibi_slopes);
  p.lse_out = ptr<float>(lse_out);
  p.num_q_heads = Hq;
  p.num_kv_heads = kv_cache.size(3);
  p.block_size = kv_cache.size(2);
  p.max_blocks = block_table.size(1);
  p.num_blocks = kv_cache.size(0);
  p.num_splits = std::max<int64_t>(1, num_splits);
  p.total_tokens = T;
  p.scale = (float)scale;
  p.softcap = (float)softcap;
  p.k_scale = (float)k_scale;
  p.v_scale = (float)v_scale;
  p.window = (int)window;
  p.causal = causal;
  TORCH_CHECK(p.block_size % 16 == 0, "block_size must be a multiple of 16");
  if (p.num_splits > 1) {
    TORCH_CHECK(workspace.has_value(), "split-KV decode needs a workspace");
    const int64_t need = p.num_splits * (int64_t)T * Hq * (D + 1);
    TORCH_CHECK(workspace->scalar_type() == at::kFloat && workspace->numel() >= need, "decode workspace too small");
    p.part_out = workspace->data_ptr<float>();
    p.part_lse = p.part_out + p.num_splits * (int64_t)T * Hq * D;
  }
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(q));
  const c10::cuda::CUDAGuard guard(q.device());
  const int rc = b200::paged_attention_decode(p, D, kv_kind_of(kv_cache, kv_scales.has_value()), dtype16(q), batch,
                                              max_q_len, cur_stream());
  TORCH_CHECK(rc == 0, "paged_attention_decode: unsupported head_dim ", D);
}

void attention_prefill(Tensor& out, const Tensor& q, const Tensor& k_src, const optional<Tensor>& v_src,
                       const optional<Tensor>& block_table, const optional<Tensor>& seq_lens,
                       const Tensor& query_start_loc, const optional<Tensor>& kv_start_loc, double scale,
                       int64_t window, double softcap, const optional<Tensor>& sinks,
                       const optional<Tensor>& lse_out, int64_t batch, int64_t max_q_len, bool causal,
                       const optional<Tensor>& alibi_slopes) {
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2));
  b200::PrefillParams p{};
  p.alibi_slopes = ptr<float>(alibi_slopes);
  const int T = q.size(0), Hq = q.size(1), DQK = q.size(2);
  const bool paged = block_table.has_value();
  int Hkv, DV;
  int64_t total_kv = 0, ks = 0, vs = 0;
  const void* kptr = k_src.data_ptr();
  const void* vptr = nullptr;
  if (paged) {
    TORCH_CHECK(k_src.dim() == 5 && k_src.is_contiguous(), "paged mode expects the [nb,2,bs,Hkv,D] cache");
    TORCH_CHECK(k_src.scalar_type() == q.scalar_type(), "tcgen05 prefill needs a 16-bit cache of the query dtype");
    Hkv = k_src.size(3);
    DV = k_src.size(4);
    p.block_size = k_src.size(2);
    p.num_blocks = k_src.size(0);
    p.max_blocks = block_table->size(1);
    p.block_table = block_table->data_ptr<int>();
    p.seq_lens = seq_lens->data_ptr<int>();
    TORCH_CHECK(p.block_size % 16 == 0 && (128 % p.block_size == 0 || p.block_size % 128 == 0),
                "block_size must be 16/32/64 or a multiple of 128");
    vptr = kptr;
  } else {
    TORCH_CHECK(v_src.has_value() && kv_start_loc.has_value());
    TORCH_CHECK(k_src.dim() == 3 && k_src.stride(2) == 1 && k_src.stride(1) == k_src.size(2));
    TORCH_CHECK(v_src->dim() == 3 && v_src->stride(2) == 1 && v_src->stride(1) == v_src->size(2));
    Hkv = k_src.size(1);
    DV = v_src->size(2);
    total_kv = k_src.size(0);
    ks = k_src.stride(0);
    vs = v_src->stride(0);
    vptr = v_src->data_ptr();
    p.kv_start_loc = kv_start_loc->data_ptr<int>();
  }
  p.out = out.data_ptr();
  p.lse_out = ptr<float>(lse_out);
  p.query_start_loc = query_start_loc.data_ptr<int>();
  p.sinks = ptr<float>(sinks);
  p.num_q_heads = Hq;
  p.num_kv_heads = Hkv;
  const int g = Hq / Hkv;
  p.gp = (128 % g == 0) ? g : 1;
  p.total_q = T;
  p.scale = (float)scale;
  p.softcap = (float)softcap;
  p.window = (int)window;
  p.causal = causal;
  p.paged = paged;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(q));
  TORCH_CHECK(out.is_contiguous() && out.size(-1) == DV);
  TORCH_CHECK(q.stride(0) % 8 == 0, "q token stride must be a multiple of 8 elements");
  const c10::cuda::CUDAGuard guard(q.device());
  // B200_ATTN_PREFILL_SINGLE=1 selects the one-tile-per-CTA kernel (P through shared memory)
  static const bool single_tile = [] {
    const char* e = std::getenv("B200_ATTN_PREFILL_SINGLE");
    return e != nullptr && std::atoi(e) != 0;
  }();
  const int rc = single_tile
                     ? b200::attention_prefill(p, q.data_ptr(), q.stride(0), kptr, vptr, ks, vs, total_kv, DQK, DV,
                                               dtype16(q), batch, max_q_len, cur_stream())
                     : b200::attention_prefill_pp(p, q.data_ptr(), q.stride(0), kptr, vptr, ks, vs, total_kv, DQK, DV,
                                                  dtype16(q), batch, max_q_len, cur_stream());
  TORCH_CHECK(rc == 0, "attention_prefill: unsupported head dims ", DQK, "/", DV);
}

// ------------------------------------------------------------------ sampling
void argmax(Tensor& out, const Tensor& logits) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && out.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(logits.device());
  b200::argmax(out.data_ptr<int64_t>(), logits.data_ptr(), logits.size(0), logits.size(1), logits.stride(0),
               dtype_code(logits), cur_stream());
}
void sample(Tensor& out, const Tensor& logits, const Tensor& temperature, const optional<Tensor>& top_k,
            const optional<Tensor>& top_p, const optional<Tensor>& min_p, const Tensor& uniform) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && out.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(logits.device());
  b200::sample(out.data_ptr<int64_t>(), logits.data_ptr(), logits.size(0), logits.size(1), logits.stride(0),
               temperature.data_ptr<float>(), ptr<int>(top_k), ptr<float>(top_p), ptr<float>(min_p),
               uniform.data_ptr<float>(), dtype_code(logits), cur_stream());
}
void apply_penalties(Tensor& logits, const optional<Tensor>& prompt_mask, const optional<Tensor>& output_counts,
                     const optional<Tensor>& rep, const optional<Tensor>& presence,
                     const optional<Tensor>& frequency) {
  const c10::cuda::CUDAGuard guard(logits.device());
  b200::apply_penalties(logits.data_ptr(), ptr<int>(prompt_mask), ptr<int>(output_counts), ptr<float>(rep),
                        ptr<float>(presence), ptr<float>(frequency), logits.size(0), logits.size(1), logits.stride(0),
                        dtype_code(logits), cur_stream());
}
void advance_step(Tensor& input_ids, Tensor& positions, Tensor& seq_lens, Tensor& slot_mapping, const Tensor& sampled,
                  const Tensor& block_table, int64_t block_size, int64_t batch, const optional<Tensor>& token_log,
                  int64_t log_col) {
  const c10::cuda::CUDAGuard guard(input_ids.device());
  b200::advance_step(input_ids.data_ptr<int64_t>(), positions.data_ptr<int64_t>(), seq_lens.data_ptr<int>(),
                     slot_mapping.data_ptr<int64_t>(), sampled.data_ptr<int64_t>(), block_table.data_ptr<int>(),
                     block_table.size(1), block_size, batch, ptr<int64_t>(token_log), log_col,
                     token_log.has_value() ? token_log->stride(0) : 0, cur_stream());
}
void embedding(Tensor& out, const Tensor& table, const Tensor& ids, int64_t vocab_start) {
  TORCH_CHECK(table.is_contiguous() && out.is_contiguous() && ids.scalar_type() == at::kLong);
  TORCH_CHECK(table.size(1) % 8 == 0);
  const c10::cuda::CUDAGuard guard(table.device());
  b200::embedding(out.data_ptr(), table.data_ptr(), ids.data_ptr<int64_t>(), ids.numel(), table.size(1), table.size(0),
                  vocab_start, dtype16(table), cur_stream());
}


// ------------------------------------------------------------------ MoE
void topk_gating(Tensor& weights, Tensor& ids, const Tensor& gating, const optional<Tensor>& bias, int64_t mode,
                 bool renorm, double scale) {
  TORCH_CHECK(gating.dim() == 2 && gating.is_contiguous() && gating.size(1) <= 1024 && ids.size(1) <= 32);
  TORCH_CHECK(weights.scalar_type() == at::kFloat && ids.scalar_type() == at::kInt);
  const c10::cuda::CUDAGuard guard(gating.device());
  b200::topk_gating(weights.data_ptr<float>(), ids.data_ptr<int>(), gating.data_ptr(), ptr<float>(bias),
                    gating.size(0), gating.size(1), ids.size(1), mode, renorm, (float)scale, dtype_code(gating),
                    cur_stream());
}
void grouped_topk(Tensor& weights, Tensor& ids, const Tensor& gating, const optional<Tensor>& bias, int64_t n_group,
                  int64_t topk_group, bool sigmoid, bool renorm, double scale) {
  TORCH_CHECK(gating.dim() == 2 && gating.is_contiguous() && gating.size(1) <= 1024 && ids.size(1) <= 32);
  TORCH_CHECK(n_group <= 32 && gating.size(1) % n_group == 0);
  const c10::cuda::CUDAGuard guard(gating.device());
  b200::grouped_topk(weights.data_ptr<float>(), ids.data_ptr<int>(), gating.data_ptr(), ptr<float>(bias),
                     gating.size(0), gating.size(1), ids.size(1), n_group, topk_group, sigmoid, renorm, (float)scale,
                     dtype_code(gating), cur_stream());
}
void moe_align(Tensor& sorted_ids, Tensor& block_expert, Tensor& total_padded, const optional<Tensor>& inv_pos,
               const Tensor& topk_ids, const optional<Tensor>& expert_map, int64_t experts, int64_t block) {
  TORCH_CHECK(topk_ids.scalar_type() == at::kInt && topk_ids.is_contiguous());
  TORCH_CHECK(sorted_ids.numel() % block == 0 && block_expert.numel() >= sorted_ids.numel() / block);
  const c10::cuda::CUDAGuard guard(topk_ids.device());
  b200::moe_align(sorted_ids.data_ptr<int>(), block_expert.data_ptr<int>(), total_padded.data_ptr<int>(),
                  ptr<int>(inv_pos), topk_ids.data_ptr<int>(), ptr<int>(expert_map), topk_ids.numel(), experts, block,
                  sorted_ids.numel(), cur_stream());
}
void moe_gather(Tensor& out, const Tensor& x, const Tensor& sorted_ids, const Tensor& total_padded, int64_t topk) {
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && x.size(1) % 8 == 0);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::moe_gather(out.data_ptr(), x.data_ptr(), sorted_ids.data_ptr<int>(), total_padded.data_ptr<int>(),
                   out.size(0), x.size(0) * topk, topk, x.size(1), dtype16(x), cur_stream());
}
void moe_combine(Tensor& out, const Tensor& y, const Tensor& weights, const Tensor& inv_pos,
                 const optional<Tensor>& shared) {
  TORCH_CHECK(y.is_contiguous() && out.is_contiguous() && weights.scalar_type() == at::kFloat);
  const c10::cuda::CUDAGuard guard(y.device());
  b200::moe_combine(out.data_ptr(), y.data_ptr(), weights.data_ptr<float>(), inv_pos.data_ptr<int>(), ptr(shared),
                    out.size(0), weights.size(1), out.size(1), dtype16(y), cur_stream());
}
void moe_sum(Tensor& out, const Tensor& in) {
  TORCH_CHECK(in.dim() == 3 && in.is_contiguous() && out.is_contiguous());
  const c10::cuda::CUDAGuard guard(in.device());
  b200::moe_sum(out.data_ptr(), in.data_ptr(), in.size(0), in.size(1), in.size(2), dtype16(in), cur_stream());
}
void gemm_grouped(Tensor& out, const Tensor& a, const Tensor& w, const Tensor& block_expert,
                  const Tensor& total_padded, int64_t epi) {
  TORCH_CHECK(a.dim() == 2 && w.dim() == 3 && a.stride(1) == 1 && w.is_contiguous() && out.stride(1) == 1);
  TORCH_CHECK(a.size(0) % 128 == 0 && a.size(1) == w.size(2) && a.size(1) % 8 == 0 && a.stride(0) % 8 == 0);
  TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == (epi == 1 ? w.size(1) / 2 : w.size(1)));
  const c10::cuda::CUDAGuard guard(a.device());
  b200::gemm_grouped(a.data_ptr(), a.size(0), a.stride(0), w.data_ptr(), w.size(0), w.size(1), w.size(2),
                     out.data_ptr(), out.stride(0), block_expert.data_ptr<int>(), total_padded.data_ptr<int>(), epi,
                     dtype16(a), cur_stream(), status_ptr(a));
}

// ------------------------------------------------------------------ quantisation
void per_token_group_quant(Tensor& q, Tensor& scales, const Tensor& x, int64_t group, bool ue8m0, bool col_major,
                           double eps) {
  TORCH_CHECK(x.is_contiguous() && q.is_contiguous() && (group == 64 || group == 128 || group == 256));
  const int K = x.size(-1);
  TORCH_CHECK(K % group == 0);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::per_token_group_quant(q.data_ptr(), scales.data_ptr<float>(), x.data_ptr(), x.numel() / K, K, group,
                              q.scalar_type() == at::kChar, ue8m0, col_major, (float)eps, dtype16(x), cur_stream());
}
void scaled_fp8_quant(Tensor& q, Tensor& scale, const Tensor& x, int64_t mode, double scale_ub) {
  TORCH_CHECK(x.is_contiguous() && q.is_contiguous());
  const int K = x.size(-1);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::scaled_fp8_quant(q.data_ptr(), scale.data_ptr<float>(), x.data_ptr(), x.numel() / K, K, mode, (float)scale_ub,
                         dtype16(x), cur_stream());
}
void scaled_int8_quant(Tensor& q, Tensor& scale, const optional<Tensor>& azp, const Tensor& x, int64_t mode) {
  TORCH_CHECK(x.is_contiguous() && q.is_contiguous());
  const int K = x.size(-1);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::scaled_int8_quant(q.data_ptr(), scale.data_ptr<float>(), ptr<int>(azp), x.data_ptr(), x.numel() / K, K, mode,
                          dtype16(x), cur_stream());
}
void merge_attn_states(Tensor& out, const optional<Tensor>& out_lse, const Tensor& p_out, const Tensor& p_lse,
                       const Tensor& s_out, const Tensor& s_lse) {
  TORCH_CHECK(p_out.is_contiguous() && s_out.is_contiguous() && out.is_contiguous() && p_out.size(2) % 8 == 0);
  TORCH_CHECK(p_lse.is_contiguous() && s_lse.is_contiguous());
  const c10::cuda::CUDAGuard guard(p_out.device());
  b200::merge_attn_states(out.data_ptr(), ptr<float>(out_lse), p_out.data_ptr(), p_lse.data_ptr<float>(),
                          s_out.data_ptr(), s_lse.data_ptr<float>(), p_out.size(0), p_out.size(1), p_out.size(2),
                          dtype16(p_out), cur_stream());
}
void gemm_fp8_blockscale(Tensor& out, const Tensor& a, const Tensor& a_scale, const Tensor& w, const Tensor& w_scale,
                         const optional<Tensor>& block_expert, const optional<Tensor>& total_padded) {
  const bool grouped = w.dim() == 3;
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && w.is_contiguous() && a_scale.is_contiguous() && w_scale.is_contiguous());
  TORCH_CHECK(a.element_size() == 1 && w.element_size() == 1 && a.size(1) % 128 == 0 && a.stride(0) % 16 == 0);
  const int M = a.size(0), K = a.size(1);
  const int E = grouped ? w.size(0) : 1, N = grouped ? w.size(1) : w.size(0);
  TORCH_CHECK(w.size(-1) == K && out.size(0) == M && out.size(1) == N && out.stride(1) == 1);
  TORCH_CHECK(a_scale.size(-1) == K / 128 && w_scale.size(-1) == K / 128 && w_scale.size(-2) == (N + 127) / 128);
  if (grouped) TORCH_CHECK(block_expert.has_value() && total_padded.has_value() && M % 128 == 0);
  const c10::cuda::CUDAGuard guard(a.device());
  b200::gemm_fp8_blockscale(a.data_ptr(), M, a.stride(0), w.data_ptr(), E, N, K, out.data_ptr(), out.stride(0),
                            a_scale.data_ptr<float>(), w_scale.data_ptr<float>(), ptr<int>(block_expert),
                            ptr<int>(total_padded), grouped, dtype16(out), cur_stream(), status_ptr(a));
}

// kind is taken from the operand dtype: int8 -> kind::i8, anything else one byte wide -> e4m3
void scaled_mm(Tensor& out, const Tensor& a, const Tensor& w, const Tensor& a_scale, const Tensor& w_scale,
               const optional<Tensor>& azp, const optional<Tensor>& azp_adj, const optional<Tensor>& bias,
               const optional<Tensor>& block_expert, const optional<Tensor>& total_padded) {
  const bool grouped = w.dim() == 3;
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && w.is_contiguous() && a_scale.is_contiguous() && w_scale.is_contiguous());
  TORCH_CHECK(a.element_size() == 1 && w.element_size() == 1 && a.size(1) % 16 == 0 && a.stride(0) % 16 == 0);
  TORCH_CHECK(a_scale.scalar_type() == at::kFloat && w_scale.scalar_type() == at::kFloat);
  const int M = a.size(0), K = a.size(1);
  const int E = grouped ? w.size(0) : 1, N = grouped ? w.size(1) : w.size(0);
  TORCH_CHECK(w.size(-1) == K && out.size(0) == M && out.size(1) == N && out.stride(1) == 1);
  const int a_per_row = a_scale.numel() > 1;
  TORCH_CHECK(!a_per_row || a_scale.numel() == M, "a_scale must have 1 or M entries");
  const int w_per_col = w_scale.numel() > E;
  TORCH_CHECK(w_per_col ? w_scale.numel() == (int64_t)E * N : w_scale.numel() == E, "w_scale must be per tensor or per channel");
  if (azp.has_value()) TORCH_CHECK(azp->numel() == M && azp->scalar_type() == at::kInt && azp_adj.has_value());
  if (azp_adj.has_value()) TORCH_CHECK(azp_adj->numel() == N && azp_adj->scalar_type() == at::kInt && !grouped);
  if (bias.has_value()) TORCH_CHECK(bias->numel() == N && bias->scalar_type() == out.scalar_type() && !grouped);
  if (grouped) TORCH_CHECK(block_expert.has_value() && total_padded.has_value() && M % 128 == 0);
  const c10::cuda::CUDAGuard guard(a.device());
  b200::gemm_scaled_mm(a.data_ptr(), M, a.stride(0), w.data_ptr(), E, N, K, out.data_ptr(), out.stride(0),
                       a_scale.data_ptr<float>(), a_per_row, w_scale.data_ptr<float>(), w_per_col, ptr<int>(azp),
                       ptr<int>(azp_adj), bias.has_value() ? bias->data_ptr() : nullptr, ptr<int>(block_expert),
                       ptr<int>(total_padded), grouped, a.scalar_type() == at::kChar ? 0 : 1, dtype16(out),
                       cur_stream(), status_ptr(a));
}

// Weight-only quantised GEMM; q [(E,) N, K*bits/8] uint8, scales / zeros [(E,) K/group, N] in a's dtype.
void wna16_gemm(Tensor& out, const Tensor& a, const Tensor& q, const Tensor& scales, const optional<Tensor>& zeros,
                int64_t bits, int64_t group, const optional<Tensor>& bias, const optional<Tensor>& block_expert,
                const optional<Tensor>& total_padded, int64_t token_tile, int64_t epi) {
  const bool grouped = q.dim() == 3;
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && a.stride(0) % 8 == 0 && q.is_contiguous() && scales.is_contiguous());
  TORCH_CHECK(bits == 4 || bits == 8);
  const int M = a.size(0), K = a.size(1);
  const int E = grouped ? q.size(0) : 1, N = q.size(-2);
  TORCH_CHECK(q.size(-1) * 8 == K * bits && K % 64 == 0 && group >= 32 && K % group == 0 && group % 32 == 0);
  TORCH_CHECK(scales.scalar_type() == a.scalar_type() && scales.size(-1) == N && scales.size(-2) == K / group);
  if (zeros.has_value()) TORCH_CHECK(zeros->scalar_type() == a.scalar_type() && zeros->sizes() == scales.sizes() && zeros->is_contiguous());
  TORCH_CHECK(out.size(0) == M && out.size(1) == (epi == 1 ? N / 2 : N) && out.stride(1) == 1);
  if (bias.has_value()) TORCH_CHECK(bias->numel() == N && bias->scalar_type() == a.scalar_type());
  const c10::cuda::CUDAGuard guard(a.device());
  int bn = token_tile > 0 ? (int)token_tile : b200::gemm_wna16_token_tile(M);
  if (grouped) TORCH_CHECK(block_expert.has_value() && total_padded.has_value() && token_tile > 0 && M % bn == 0);
  int splits = (grouped || epi != 0) ? 1 : b200::gemm_wna16_splits(M, N, K, bn);
  Tensor partial;
  if (splits > 1) partial = at::empty({splits, M, N}, a.options().dtype(at::kFloat));
  b200::gemm_wna16(a.data_ptr(), M, a.stride(0), q.data_ptr(), scales.data_ptr(),
                   zeros.has_value() ? zeros->data_ptr() : nullptr, E, N, K, group, bits, out.data_ptr(), out.stride(0),
                   bias.has_value() ? bias->data_ptr() : nullptr, splits > 1 ? partial.data_ptr<float>() : nullptr,
                   splits, ptr<int>(block_expert), ptr<int>(total_padded), grouped, bn, epi, dtype16(a), cur_stream(),
                   status_ptr(a));
}

// ------------------------------------------------------------------ MLA
void mla_decode(Tensor& out, const Tensor& q, const Tensor& cache, const Tensor& block_table, const Tensor& seq_lens,
                const optional<Tensor>& query_start_loc, const optional<Tensor>& topk_indices, double scale,
                const optional<Tensor>& lse_out, const optional<Tensor>& workspace, int64_t num_splits, int64_t impl) {
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 576 && q.stride(2) == 1 && q.stride(1) == 576);
  TORCH_CHECK(cache.is_contiguous() && cache.dim() == 3 && out.is_contiguous() && out.size(2) == 512);
  const bool rec = cache.scalar_type() == at::kByte;
  TORCH_CHECK(rec ? cache.size(2) == 656 : (cache.size(2) == 576 && cache.scalar_type() == q.scalar_type()));
  b200::MlaDecodeParams p{};
  p.out = out.data_ptr();
  p.lse_out = ptr<float>(lse_out);
  p.q = q.data_ptr();
  p.q_stride = q.stride(0);
  p.cache = cache.data_ptr();
  p.block_table = block_table.data_ptr<int>();
  p.seq_lens = seq_lens.data_ptr<int>();
  p.query_start_loc = ptr<int>(query_start_loc);
  p.topk_indices = ptr<int>(topk_indices);
  p.topk = topk_indices.has_value() ? topk_indices->size(1) : 0;
  p.num_heads = q.size(1);
  p.block_size = cache.size(1);
  p.num_blocks = cache.size(0);
  p.max_blocks = block_table.size(1);
  p.num_splits = std::max<int64_t>(1, num_splits);
  p.total_tokens = q.size(0);
  p.batch = seq_lens.size(0);
  p.scale = (float)scale;
  if (p.num_splits > 1) {
    const int64_t need = p.num_splits * (int64_t)p.total_tokens * p.num_heads * 513;
    TORCH_CHECK(workspace.has_value() && workspace->numel() >= need, "mla_decode workspace too small");
    p.part_out = workspace->data_ptr<float>();
    p.part_lse = p.part_out + p.num_splits * (int64_t)p.total_tokens * p.num_heads * 512;
  }
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(q));
  const c10::cuda::CUDAGuard guard(q.device());
  const int rc = b200::mla_decode(p, rec, dtype16(q), cur_stream(), (int)impl);
  TORCH_CHECK(rc == 0, "mla_decode: the tcgen05 kernel was asked for (impl = 2) but does not serve this call");
}

// ------------------------------------------------------------------ DSA indexer
void indexer_logits(Tensor& logits, const Tensor& q, const Tensor& w, const Tensor& cache, const Tensor& block_table,
                    const Tensor& seq_lens, const Tensor& query_start_loc, int64_t block_size, int64_t max_len,
                    bool int8, int64_t max_query_len, int64_t impl) {
  // impl: 0 = tcgen05 kernel when it serves the shapes (8-bit operands, heads a multiple of 32), 1 = mma.sync kernel,
  // 2 = tcgen05 kernel or an error
  const bool bf16 = q.scalar_type() == at::kBFloat16;      // unquantised indexer: bf16 queries, bf16 key cache
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.is_contiguous() && (q.element_size() == 1 || bf16));
  TORCH_CHECK(q.size(1) % 16 == 0 && q.size(1) <= 64 && w.is_contiguous() && w.scalar_type() == at::kFloat);
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.stride(1) == 1 && logits.size(1) >= max_len);
  TORCH_CHECK(cache.is_contiguous() && cache.scalar_type() == at::kByte);
  const c10::cuda::CUDAGuard guard(q.device());
  if (impl != 1 && !bf16) {
    const int rc = b200::indexer_logits_tc(logits.data_ptr<float>(), logits.stride(0), q.data_ptr(), w.data_ptr<float>(),
                                           cache.data_ptr(), block_table.data_ptr<int>(), block_table.size(1),
                                           seq_lens.data_ptr<int>(), query_start_loc.data_ptr<int>(), q.size(0),
                                           seq_lens.size(0), q.size(1), block_size, cache.size(0), max_len,
                                           max_query_len, status_ptr(q), cur_stream(), int8 ? 1 : 0);
    if (rc == 0) return;
    TORCH_CHECK(impl != 2, "indexer_logits: shapes not served by the tcgen05 kernel");
  }
  b200::indexer_logits(logits.data_ptr<float>(), logits.stride(0), q.data_ptr(), w.data_ptr<float>(), cache.data_ptr(),
                       block_table.data_ptr<int>(), block_table.size(1), seq_lens.data_ptr<int>(),
                       query_start_loc.data_ptr<int>(), q.size(0), seq_lens.size(0), q.size(1), block_size,
                       cache.size(0), max_len, status_ptr(q), cur_stream(), bf16 ? 2 : (int8 ? 1 : 0));
}
void topk_per_row(Tensor& out, const Tensor& x, const optional<Tensor>& row_len, int64_t cols) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kFloat && out.is_contiguous());
  TORCH_CHECK(out.scalar_type() == at::kInt && out.size(0) == x.size(0));
  const c10::cuda::CUDAGuard guard(x.device());
  b200::topk_per_row(out.data_ptr<int>(), x.data_ptr<float>(), x.stride(0), ptr<int>(row_len), x.size(0), cols,
                     out.size(1), cur_stream());
}

// ------------------------------------------------------------------ symmetric (peer-mapped) memory
// A plain cudaMalloc allocation whose IPC handle can be opened by the other ranks of the node.
std::tuple<Tensor, Tensor> symm_alloc(int64_t nbytes, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  void* p = nullptr;
  TORCH_CHECK(cudaMalloc(&p, (size_t)nbytes) == cudaSuccess, "symm_alloc: cudaMalloc of ", nbytes, " bytes failed");
  TORCH_CHECK(cudaMemset(p, 0, (size_t)nbytes) == cudaSuccess);
  cudaIpcMemHandle_t h;
  TORCH_CHECK(cudaIpcGetMemHandle(&h, p) == cudaSuccess, "cudaIpcGetMemHandle failed");
  Tensor handle = torch::empty({(int64_t)sizeof(h)}, torch::kUInt8);
  std::memcpy(handle.data_ptr(), &h, sizeof(h));
  Tensor buf = torch::from_blob(p, {nbytes}, [](void* q) { cudaFree(q); },
                                torch::dtype(torch::kUInt8).device(torch::kCUDA, (c10::DeviceIndex)device));
  return {buf, handle};
}
int64_t symm_open(const Tensor& handle, int64_t device) {
  const c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaIpcMemHandle_t h;
  TORCH_CHECK(handle.numel() == (int64_t)sizeof(h));
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  TORCH_CHECK(e == cudaSuccess, "cudaIpcOpenMemHandle failed: ", cudaGetErrorString(e));
  return reinterpret_cast<int64_t>(p);
}
void symm_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

// x [T, K_local], w [H, K_local]; ptrs: CPU int64 [4, tp] = recv / counters / flags / out base per rank.
void gemm_ar_norm(const Tensor& x, const Tensor& w, Tensor& residual, const Tensor& norm_weight, double eps,
                  const Tensor& ptrs, int64_t tp, int64_t rank, int64_t rows_per_rank, int64_t rows_cap,
                  int64_t rb_cap, Tensor& local_sync, bool add_residual, int64_t wait_cycles) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && x.size(1) == w.size(1));
  TORCH_CHECK(tp >= 1 && tp <= b200::kMaxRanks && ptrs.dim() == 2 && ptrs.size(0) == 4 && ptrs.size(1) >= tp);
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong && residual.is_contiguous());
  TORCH_CHECK(x.size(1) % 8 == 0 && x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0);
  b200::FusedArParams p{};
  p.T = x.size(0); p.H = w.size(0); p.K = x.size(1);
  p.tp = tp; p.rank = rank; p.rows_per_rank = rows_per_rank;
  p.rows_cap = rows_cap; p.rb_cap = rb_cap;
  TORCH_CHECK(rows_per_rank <= rows_cap && (p.T + 127) / 128 <= rb_cap, "fused all-reduce workspace too small");
  const int64_t* pp = ptrs.data_ptr<int64_t>();
  const int64_t st = ptrs.stride(0);
  for (int r = 0; r < tp; ++r) {
    p.recv[r] = reinterpret_cast<void*>(pp[0 * st + r]);
    p.counters[r] = reinterpret_cast<uint32_t*>(pp[1 * st + r]);
    p.flags[r] = reinterpret_cast<uint32_t*>(pp[2 * st + r]);
    p.out[r] = reinterpret_cast<void*>(pp[3 * st + r]);
  }
  p.residual = residual.data_ptr();
  p.norm_weight = norm_weight.data_ptr();
  p.eps = (float)eps;
  p.add_residual = add_residual;
  p.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(x));
  const c10::cuda::CUDAGuard guard(x.device());
  const int rc = b200::gemm_ar_norm(p, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), dtype16(x), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_ar_norm: hidden size ", p.H, " not supported");
}

// Row-parallel GEMM whose output rows go straight into the owning rank's receive slot (NVLink peer stores from the
// GEMM epilogue).  ptrs: CPU int64 [>= 2, tp] = recv / flag1 base per rank; local_sync: int32 [4] on the device.
void gemm_row_scatter(const Tensor& x, const Tensor& w, const Tensor& ptrs, int64_t tp, int64_t rank,
                      int64_t rows_per_rank, int64_t rows_cap, Tensor& local_sync) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && x.size(1) == w.size(1));
  TORCH_CHECK(tp >= 1 && tp <= b200::kMaxRanks && ptrs.dim() == 2 && ptrs.size(0) >= 2 && ptrs.size(1) >= tp);
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong);
  TORCH_CHECK(x.size(1) % 8 == 0 && x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0 && w.size(0) % 8 == 0);
  const int M = x.size(0), N = w.size(0), K = x.size(1);
  TORCH_CHECK(rows_per_rank >= 1 && rows_per_rank <= rows_cap && rows_per_rank * tp >= M,
              "gemm_row_scatter: receive slots too small");
  b200::RowScatter sc{};
  sc.tp = tp; sc.src_rank = rank; sc.rows_per_rank = rows_per_rank; sc.rows_cap = rows_cap;
  const int64_t* pp = ptrs.data_ptr<int64_t>();
  const int64_t st = ptrs.stride(0);
  for (int r = 0; r < tp; ++r) {
    sc.recv[r] = reinterpret_cast<void*>(pp[0 * st + r]);
    sc.flag[r] = reinterpret_cast<uint32_t*>(pp[1 * st + r]);
  }
  sc.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  const c10::cuda::CUDAGuard guard(x.device());
  if (M <= 64) {   // few tokens: stream over all SMs; otherwise CTA-pair tiles
    StkScratch sk = stk_scratch(x);
    const int rc = b200::gemm_tn_streamk(x.data_ptr(), w.data_ptr(), nullptr, nullptr, nullptr, M, N, K, x.stride(0),
                                         w.stride(0), N, 0, dtype16(x), cur_stream(), status_ptr(x), 0, sk.ws,
                                         sk.counters, sk.sms, &sc);
    if (rc == 0) return;
  }
  b200::gemm_tn_pair(x.data_ptr(), w.data_ptr(), nullptr, nullptr, nullptr, M, N, K, x.stride(0), w.stride(0), N, 0,
                     dtype16(x), cur_stream(), status_ptr(x), 0, &sc);
}

// Reduce + residual + RMSNorm + all-gather over the slots filled by gemm_row_scatter.
// ptrs: CPU int64 [4, tp] = recv / flag1 / flag2 / out base per rank.
void ar_norm_gather(Tensor& residual, const Tensor& norm_weight, double eps, const Tensor& ptrs, int64_t T, int64_t H,
                    int64_t tp, int64_t rank, int64_t rows_per_rank, int64_t rows_cap, Tensor& local_sync,
                    bool add_residual, int64_t wait_cycles, int64_t out_multicast_ptr) {
  TORCH_CHECK(tp >= 1 && tp <= b200::kMaxRanks && ptrs.dim() == 2 && ptrs.size(0) == 4 && ptrs.size(1) >= tp);
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong && residual.is_contiguous());
  TORCH_CHECK(residual.size(-1) == H && norm_weight.numel() == H && residual.size(0) >= rows_per_rank);
  b200::ArNormParams p{};
  p.T = T; p.H = H; p.tp = tp; p.rank = rank; p.rows_per_rank = rows_per_rank; p.rows_cap = rows_cap;
  const int64_t* pp = ptrs.data_ptr<int64_t>();
  const int64_t st = ptrs.stride(0);
  for (int r = 0; r < tp; ++r) {
    p.recv[r] = reinterpret_cast<void*>(pp[0 * st + r]);
    p.flag1[r] = reinterpret_cast<uint32_t*>(pp[1 * st + r]);
    p.flag2[r] = reinterpret_cast<uint32_t*>(pp[2 * st + r]);
    p.out[r] = reinterpret_cast<void*>(pp[3 * st + r]);
  }
  p.out_mc = reinterpret_cast<void*>(out_multicast_ptr);
  p.residual = residual.data_ptr();
  p.norm_weight = norm_weight.data_ptr();
  p.eps = (float)eps;
  p.add_residual = add_residual;
  p.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(residual));
  const c10::cuda::CUDAGuard guard(residual.device());
  const int rc = b200::ar_norm_gather(p, dtype16(residual), cur_stream());
  TORCH_CHECK(rc == 0, "ar_norm_gather: hidden size ", H, " / dtype not supported");
}

// All-reduce + residual + RMSNorm through the NVSwitch.  The four addresses lie inside one multicast-mapped symmetric
// buffer (flag_local: this rank's own copy of the flag words).
void nvls_ar_norm(Tensor& residual, const Tensor& norm_weight, double eps, int64_t partial_mc, int64_t out_mc,
                  int64_t flag_mc, int64_t flag_local, int64_t T, int64_t H, int64_t tp, int64_t rank,
                  int64_t rows_per_rank, Tensor& local_sync, bool add_residual, int64_t wait_cycles) {
  TORCH_CHECK(tp >= 2 && tp <= b200::kMaxRanks && residual.is_contiguous() && residual.is_cuda());
  TORCH_CHECK(residual.size(-1) == H && norm_weight.numel() == H && residual.size(0) >= rows_per_rank);
  TORCH_CHECK(partial_mc != 0 && out_mc != 0 && flag_mc != 0 && flag_local != 0 && (partial_mc & 15) == 0 &&
              (out_mc & 15) == 0, "nvls_ar_norm needs a multicast mapping");
  TORCH_CHECK(local_sync.is_cuda() && local_sync.scalar_type() == at::kInt && local_sync.numel() >= 2);
  b200::NvlsArNormParams p{};
  p.T = T; p.H = H; p.tp = tp; p.rank = rank; p.rows_per_rank = rows_per_rank;
  p.partial_mc = reinterpret_cast<const void*>(partial_mc);
  p.out_mc = reinterpret_cast<void*>(out_mc);
  p.flag_mc = reinterpret_cast<uint32_t*>(flag_mc);
  p.flag_local = reinterpret_cast<const uint32_t*>(flag_local);
  p.residual = residual.data_ptr();
  p.norm_weight = norm_weight.data_ptr();
  p.eps = (float)eps;
  p.add_residual = add_residual;
  p.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(residual));
  const c10::cuda::CUDAGuard guard(residual.device());
  const int rc = b200::nvls_ar_norm(p, dtype16(residual), cur_stream());
  TORCH_CHECK(rc == 0, "nvls_ar_norm: hidden size ", H, " / dtype not supported");
}

// A tensor over the same storage that does not keep it alive: CUDA-graph wrappers hold their captured outputs this
// way so that the graph's memory pool, not Python references, owns the buffers (upstream's ``weak_ref_tensor``).
Tensor weak_ref_tensor(const Tensor& t) {
  TORCH_CHECK(t.is_cuda(), "weak_ref_tensor expects a CUDA tensor");
  return torch::from_blob(t.data_ptr(), t.sizes(), t.strides(), t.options());
}

// ------------------------------------------------------------------ small / fused kernels
void small_gemm(Tensor& out, const Tensor& a, const Tensor& w, const optional<Tensor>& bias) {
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.stride(1) == 1 && w.stride(1) == 1 && a.size(1) == w.size(1));
  TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == w.size(0) && out.stride(1) == 1 && w.scalar_type() == a.scalar_type());
  const bool f32 = out.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || out.scalar_type() == a.scalar_type());
  if (bias.has_value()) TORCH_CHECK(bias->numel() == w.size(0) && bias->scalar_type() == a.scalar_type());
  const c10::cuda::CUDAGuard guard(a.device());
  const int rc = b200::small_gemm(out.data_ptr(), a.data_ptr(), w.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr,
                                  a.size(0), w.size(0), a.size(1), a.stride(0), w.stride(0), out.stride(0), dtype16(a),
                                  f32 ? 1 : 0, cur_stream());
  TORCH_CHECK(rc == 0, "small_gemm: needs M <= 32, K % 32 == 0 and 16-byte aligned rows (rc=", rc, ")");
}

void fused_qk_norm_rope(Tensor& qkv, const Tensor& q_weight, const Tensor& k_weight, const Tensor& cos_sin,
                        const Tensor& positions, int64_t hq, int64_t hk, int64_t hv, int64_t head_dim, bool is_neox,
                        double eps, bool gemma) {
  TORCH_CHECK(qkv.dim() == 2 && qkv.is_contiguous() && qkv.size(1) == (hq + hk + hv) * head_dim);
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && positions.scalar_type() == at::kLong);
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int rc = b200::fused_qk_norm_rope(qkv.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(),
                                          cos_sin.data_ptr<float>(), positions.data_ptr<int64_t>(), qkv.size(0), hq, hk,
                                          hv, head_dim, cos_sin.size(1), is_neox, (float)eps, gemma, dtype16(qkv),
                                          cur_stream());
  TORCH_CHECK(rc == 0, "fused_qk_norm_rope: unsupported head_dim / rotary_dim");
}

// qkv [T, (hq + 2 hk + niq + has_ik) * 128]; kv_cache [blocks, 2, block_size, hk, 128]; idx_cache [slots, 128]
void qkv_norm_rope_insert(Tensor& qkv, Tensor& q_out, const optional<Tensor>& iq_out, const optional<Tensor>& kv_cache,
                          const optional<Tensor>& idx_cache, const optional<Tensor>& q_w, const optional<Tensor>& k_w,
                          const optional<Tensor>& iq_w, const optional<Tensor>& ik_w, const Tensor& cos_sin,
                          const Tensor& positions, const Tensor& slot_mapping, int64_t hq, int64_t hk, int64_t niq,
                          bool has_ik, bool is_neox, double eps, bool gemma) {
  const int64_t width = (hq + 2 * hk + niq + (has_ik ? 1 : 0)) * 128;
  TORCH_CHECK(qkv.dim() == 2 && qkv.stride(1) == 1 && qkv.size(1) == width && qkv.stride(0) % 4 == 0);
  TORCH_CHECK(q_out.is_contiguous() && q_out.numel() == qkv.size(0) * hq * 128 && q_out.scalar_type() == qkv.scalar_type());
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && positions.scalar_type() == at::kLong &&
              slot_mapping.scalar_type() == at::kLong && positions.numel() >= qkv.size(0) &&
              slot_mapping.numel() <= qkv.size(0));
  bool idx_fp8 = false;
  if (niq > 0) {
    TORCH_CHECK(iq_out.has_value() && iq_out->is_contiguous() && iq_out->numel() == qkv.size(0) * niq * 128);
    idx_fp8 = iq_out->element_size() == 1;
  }
  int64_t block_size = 1, num_slots = 0;
  if (kv_cache.has_value()) {
    TORCH_CHECK(kv_cache->dim() == 5 && kv_cache->is_contiguous() && kv_cache->size(1) == 2 && kv_cache->size(3) == hk &&
                kv_cache->size(4) == 128 && kv_cache->scalar_type() == qkv.scalar_type());
    block_size = kv_cache->size(2);
    num_slots = kv_cache->size(0) * block_size;
  }
  if (has_ik && idx_cache.has_value()) {
    TORCH_CHECK(idx_cache->is_contiguous() && idx_cache->size(-1) == 128 && (idx_cache->element_size() == 1) == idx_fp8);
    const int64_t n = idx_cache->numel() / 128;
    num_slots = kv_cache.has_value() ? std::min(num_slots, n) : n;
  }
  auto wp = [&](const optional<Tensor>& w) -> const void* {
    if (!w.has_value()) return nullptr;
    TORCH_CHECK(w->numel() == 128 && w->scalar_type() == qkv.scalar_type() && w->is_contiguous());
    return w->data_ptr();
  };
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int rc = b200::qkv_norm_rope_insert(
      qkv.data_ptr(), qkv.stride(0), wp(q_w), wp(k_w), wp(iq_w), wp(ik_w), cos_sin.data_ptr<float>(),
      positions.data_ptr<int64_t>(), slot_mapping.data_ptr<int64_t>(), q_out.data_ptr(),
      iq_out.has_value() ? iq_out->data_ptr() : nullptr, kv_cache.has_value() ? kv_cache->data_ptr() : nullptr,
      has_ik && idx_cache.has_value() ? idx_cache->data_ptr() : nullptr, (int)qkv.size(0), (int)slot_mapping.numel(),
      (int)hq, (int)hk, (int)niq, has_ik ? 1 : 0, kv_cache.has_value() ? 1 : 0, (int)cos_sin.size(1), is_neox, gemma,
      idx_fp8, (int)block_size, num_slots, (float)eps, dtype16(qkv), cur_stream());
  TORCH_CHECK(rc == 0, "qkv_norm_rope_insert: unsupported rotary width");
}

void mla_rope_and_cache(Tensor& q_pe, Tensor& k_pe, const Tensor& kv_c, Tensor& cache, const Tensor& cos_sin,
                        const Tensor& positions, const Tensor& slot_mapping, bool is_neox) {
  TORCH_CHECK(q_pe.dim() == 3 && q_pe.size(2) == 64 && q_pe.stride(2) == 1 && q_pe.stride(1) == 64);
  TORCH_CHECK(k_pe.size(-1) == 64 && k_pe.stride(-1) == 1 && kv_c.size(-1) == 512 && kv_c.stride(-1) == 1);
  TORCH_CHECK(cache.is_contiguous() && cache.size(-1) == 576 && cache.scalar_type() == q_pe.scalar_type());
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.size(1) == 64 && cos_sin.is_contiguous());
  const c10::cuda::CUDAGuard guard(q_pe.device());
  b200::mla_rope_and_cache(q_pe.data_ptr(), k_pe.data_ptr(), kv_c.data_ptr(), cache.data_ptr(), cos_sin.data_ptr<float>(),
                           positions.data_ptr<int64_t>(), slot_mapping.data_ptr<int64_t>(), q_pe.size(0), q_pe.size(1),
                           q_pe.stride(0), k_pe.stride(0), kv_c.stride(0), is_neox, cache.numel() / 576, dtype16(q_pe),
                           cur_stream());
}

void concat_mla_q(Tensor& out, const Tensor& nope, const Tensor& pe) {
  TORCH_CHECK(out.is_contiguous() && out.size(-1) == 576 && nope.size(-1) == 512 && pe.size(-1) == 64);
  TORCH_CHECK(nope.dim() == 3 && pe.dim() == 3 && nope.stride(2) == 1 && pe.stride(2) == 1);
  TORCH_CHECK(nope.stride(0) == nope.size(1) * nope.stride(1) && pe.stride(0) == pe.size(1) * pe.stride(1));
  const c10::cuda::CUDAGuard guard(out.device());
  b200::concat_mla_q(out.data_ptr(), nope.data_ptr(), pe.data_ptr(), nope.size(0) * nope.size(1), nope.stride(1),
                     pe.stride(1), dtype16(out), cur_stream());
}

void permute_cols(Tensor& out, const Tensor& a, const Tensor& perm) {
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && out.is_contiguous() && perm.scalar_type() == at::kInt);
  TORCH_CHECK(out.size(0) == a.size(0) && out.size(1) == perm.numel());
  const c10::cuda::CUDAGuard guard(a.device());
  b200::permute_cols(out.data_ptr(), a.data_ptr(), perm.data_ptr<int>(), a.size(0), perm.numel(), a.stride(0),
                     dtype16(a), cur_stream());
}

void gather_mla_cache(Tensor& dst, const Tensor& cache, const Tensor& block_table, const Tensor& cu_seq_lens,
                      const optional<Tensor>& seq_starts) {
  TORCH_CHECK(dst.is_contiguous() && dst.size(1) == 576 && cache.is_contiguous() && cache.dim() == 3);
  const bool rec = cache.scalar_type() == at::kByte;
  TORCH_CHECK(rec ? cache.size(2) == 656 : (cache.size(2) == 576 && cache.scalar_type() == dst.scalar_type()));
  const c10::cuda::CUDAGuard guard(dst.device());
  b200::gather_mla_cache(dst.data_ptr(), cache.data_ptr(), block_table.data_ptr<int>(), cu_seq_lens.data_ptr<int>(),
                         ptr<int>(seq_starts), cu_seq_lens.numel() - 1, block_table.size(1), cache.size(1), dst.size(0),
                         rec, dtype16(dst), cur_stream());
}

void gather_indexer_k(Tensor& dst_k, Tensor& dst_s, const Tensor& cache, const Tensor& block_table,
                      const Tensor& cu_seq_lens, int64_t block_size) {
  TORCH_CHECK(dst_k.is_contiguous() && dst_k.size(1) == 128 && dst_k.element_size() == 1 && dst_s.scalar_type() == at::kFloat);
  TORCH_CHECK(cache.is_contiguous() && cache.scalar_type() == at::kByte);
  const c10::cuda::CUDAGuard guard(dst_k.device());
  b200::gather_indexer_k(dst_k.data_ptr(), dst_s.data_ptr<float>(), cache.data_ptr(), block_table.data_ptr<int>(),
                         cu_seq_lens.data_ptr<int>(), cu_seq_lens.numel() - 1, block_table.size(1), block_size,
                         dst_k.size(0), cur_stream());
}

// u / delta / z / out: [dim, tokens] with query_start_loc, or [batch, dim, L]; B / C: [groups, dstate, tokens] or
// [batch, groups, dstate, L]; state fp32 [slots, dim, dstate].
void selective_scan(Tensor& out, const Tensor& u, const Tensor& delta, const Tensor& A, const Tensor& B, const Tensor& C,
                    const optional<Tensor>& D, const optional<Tensor>& z, const optional<Tensor>& delta_bias,
                    bool delta_softplus, Tensor& state, const optional<Tensor>& query_start_loc,
                    const optional<Tensor>& cache_indices, const optional<Tensor>& has_initial_state, int64_t pad_slot) {
  TORCH_CHECK(u.is_contiguous() && delta.is_contiguous() && B.is_contiguous() && C.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(A.scalar_type() == at::kFloat && A.is_contiguous() && state.scalar_type() == at::kFloat && state.is_contiguous());
  const bool varlen = query_start_loc.has_value();
  b200::ScanParams p{};
  p.u = u.data_ptr(); p.delta = delta.data_ptr(); p.out = out.data_ptr();
  p.z = z.has_value() ? z->data_ptr() : nullptr;
  p.A = A.data_ptr<float>(); p.B = B.data_ptr(); p.C = C.data_ptr();
  p.D = ptr<float>(D); p.delta_bias = ptr<float>(delta_bias);
  p.state = state.data_ptr<float>();
  p.query_start_loc = ptr<int>(query_start_loc);
  p.cache_indices = ptr<int>(cache_indices);
  p.has_initial_state = has_initial_state.has_value() ? has_initial_state->data_ptr<uint8_t>() : nullptr;
  p.dim = A.size(0); p.dstate = A.size(1);
  if (varlen) {
    TORCH_CHECK(u.dim() == 2 && B.dim() == 3);
    p.batch = query_start_loc->numel() - 1; p.total_tokens = u.size(1); p.seqlen = 0; p.groups = B.size(0);
  } else {
    TORCH_CHECK(u.dim() == 3 && B.dim() == 4);
    p.batch = u.size(0); p.seqlen = u.size(2); p.total_tokens = 0; p.groups = B.size(1);
  }
  p.softplus = delta_softplus; p.pad_slot = pad_slot;
  const int dt = u.scalar_type() == at::kFloat ? 2 : dtype16(u);
  const c10::cuda::CUDAGuard guard(u.device());
  TORCH_CHECK(b200::selective_scan_fwd(p, dt, cur_stream()) == 0, "selective_scan: unsupported dstate / dim");
}

// mHC pre (optionally fused with the previous sub-layer's post).  residual [T, M, H]; fn fp32 [mix, M*H].
void mhc_pre(Tensor& x_out, const optional<Tensor>& post_out, const optional<Tensor>& comb_out, const Tensor& residual,
             const optional<Tensor>& residual_out, const optional<Tensor>& y, const optional<Tensor>& post_in,
             const optional<Tensor>& comb_in, const Tensor& fn, const Tensor& scale, const Tensor& base, double rms_eps,
             double pre_eps, double sinkhorn_eps, double post_mult, int64_t iters, bool head) {
  TORCH_CHECK(residual.dim() == 3 && residual.is_contiguous() && fn.scalar_type() == at::kFloat && fn.is_contiguous());
  b200::MhcParams p{};
  p.T = residual.size(0); p.M = residual.size(1); p.H = residual.size(2);
  const int nmix = head ? p.M : 2 * p.M + p.M * p.M;
  TORCH_CHECK(fn.size(0) == nmix && fn.size(1) == (int64_t)p.M * p.H && base.numel() == nmix && scale.numel() >= (head ? 1 : 3));
  TORCH_CHECK(scale.scalar_type() == at::kFloat && base.scalar_type() == at::kFloat && x_out.is_contiguous());
  const bool fused = y.has_value();
  if (fused) TORCH_CHECK(residual_out.has_value() && post_in.has_value() && comb_in.has_value() && y->is_contiguous() &&
                         residual_out->is_contiguous() && residual_out->data_ptr() != residual.data_ptr());
  if (!head) TORCH_CHECK(post_out.has_value() && comb_out.has_value());
  p.residual = residual.data_ptr();
  p.residual_out = fused ? residual_out->data_ptr() : nullptr;
  p.y = fused ? y->data_ptr() : nullptr;
  p.post_in = ptr<float>(post_in); p.comb_in = ptr<float>(comb_in);
  p.fn = fn.data_ptr<float>(); p.scale = scale.data_ptr<float>(); p.base = base.data_ptr<float>();
  p.post_out = ptr<float>(post_out); p.comb_out = ptr<float>(comb_out);
  p.x_out = x_out.data_ptr();
  p.iters = iters; p.head = head;
  p.rms_eps = rms_eps; p.pre_eps = pre_eps; p.sinkhorn_eps = sinkhorn_eps; p.post_mult = post_mult;
  const c10::cuda::CUDAGuard guard(residual.device());
  TORCH_CHECK(b200::mhc_pre(p, fused, dtype16(residual), cur_stream()) == 0, "mhc_pre: unsupported stream count");
}

void mhc_post(Tensor& out, const Tensor& y, const Tensor& residual, const Tensor& post, const Tensor& comb) {
  TORCH_CHECK(residual.dim() == 3 && residual.is_contiguous() && y.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(post.scalar_type() == at::kFloat && comb.scalar_type() == at::kFloat && residual.size(1) <= 4);
  const c10::cuda::CUDAGuard guard(residual.device());
  b200::mhc_post(out.data_ptr(), y.data_ptr(), residual.data_ptr(), post.data_ptr<float>(), comb.data_ptr<float>(),
                 residual.size(0), residual.size(1), residual.size(2), dtype16(residual), cur_stream());
}

// copy `src` (a local tensor) to the raw device address `dst_ptr` (typically a peer-mapped buffer)
void p2p_copy(int64_t dst_ptr, const Tensor& src, int64_t ctas, int64_t mode) {
  TORCH_CHECK(src.is_contiguous() && ctas >= 1 && ctas <= 1024);
  const size_t n = (size_t)src.numel() * src.element_size();
  TORCH_CHECK(n % (mode == 0 ? 16 : 16384) == 0, "p2p_copy: size granularity");
  const c10::cuda::CUDAGuard guard(src.device());
  b200::p2p_copy(reinterpret_cast<void*>(dst_ptr), src.data_ptr(), n, (int)ctas, (int)mode, status_ptr(src), cur_stream());
}

// DeepSeek-V4 records: q [T, Hq, 512] bf16 (any token / head pitch), kv [T, 512] bf16, q_out [T, Hq_pad, 512],
// cache uint8 [blocks, block_stride >= block_size * 584], cos_sin fp32 [max_pos, 64]
void v4_qnorm_rope_kv_insert(Tensor& q_out, Tensor& cache, const Tensor& q, const Tensor& kv, const Tensor& slot_mapping,
                             const Tensor& positions, const Tensor& cos_sin, double eps, int64_t block_size) {
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 512 && q.stride(2) == 1 && q.scalar_type() == at::kBFloat16);
  TORCH_CHECK(kv.dim() == 2 && kv.size(1) == 512 && kv.stride(1) == 1 && kv.scalar_type() == at::kBFloat16 &&
              kv.size(0) == q.size(0));
  TORCH_CHECK(q_out.dim() == 3 && q_out.is_contiguous() && q_out.size(0) == q.size(0) && q_out.size(1) >= q.size(1) &&
              q_out.size(2) == 512 && q_out.scalar_type() == at::kBFloat16);
  TORCH_CHECK(q.stride(0) % 8 == 0 && q.stride(1) % 8 == 0 && kv.stride(0) % 8 == 0, "rows must be 16-byte aligned");
  TORCH_CHECK(cache.dim() == 2 && cache.element_size() == 1 && cache.stride(1) == 1 &&
              cache.stride(0) >= block_size * 584 && cache.stride(0) % 16 == 0 && block_size % 2 == 0);
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong && positions.scalar_type() == at::kLong &&
              slot_mapping.is_contiguous() && positions.is_contiguous() && positions.numel() >= q.size(0) &&
              slot_mapping.numel() <= q.size(0));
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.dim() == 2 && cos_sin.size(1) == 64 && cos_sin.is_contiguous());
  const c10::cuda::CUDAGuard guard(q.device());
  b200::v4_qnorm_rope_kv_insert(q.data_ptr(), q.stride(0), q.stride(1), kv.data_ptr(), kv.stride(0), q_out.data_ptr(),
                                cache.data_ptr(), cache.stride(0), slot_mapping.data_ptr<int64_t>(),
                                positions.data_ptr<int64_t>(), cos_sin.data_ptr<float>(), (int)q.size(0),
                                (int)slot_mapping.numel(), (int)q.size(1), (int)q_out.size(1), (int)block_size,
                                (float)eps, cur_stream());
}

void v4_gather_dequant(Tensor& dst, const Tensor& cache, const Tensor& slots, int64_t block_size) {
  TORCH_CHECK(dst.dim() == 2 && dst.size(1) == 512 && dst.is_contiguous() && dst.scalar_type() == at::kBFloat16);
  TORCH_CHECK(cache.dim() == 2 && cache.element_size() == 1 && cache.stride(1) == 1 && cache.stride(0) >= block_size * 584);
  TORCH_CHECK(slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() == dst.size(0));
  const c10::cuda::CUDAGuard guard(dst.device());
  b200::v4_gather_dequant(dst.data_ptr(), cache.data_ptr(), cache.stride(0), slots.data_ptr<int64_t>(), (int)dst.size(0),
                          (int)block_size, cur_stream());
}

// q, k [T, Hq, 128], v [T, Hv, 128], g / beta f32 [T, Hv], state f32 [slots, Hv, 128, 128] (in / out)
void gdn_recurrent(Tensor& out, Tensor& state, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g,
                   const Tensor& beta, const Tensor& query_start_loc, const optional<Tensor>& state_idx,
                   const optional<Tensor>& has_initial, double scale, bool l2norm) {
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1);
  TORCH_CHECK(q.stride(1) == q.size(2) && k.stride(1) == k.size(2) && v.stride(1) == v.size(2) && k.sizes() == q.sizes());
  const int64_t T = q.size(0), hq = q.size(1), hv = v.size(1);
  TORCH_CHECK(v.size(0) == T && out.is_contiguous() && out.sizes() == v.sizes() && out.scalar_type() == q.scalar_type());
  TORCH_CHECK(g.is_contiguous() && beta.is_contiguous() && g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat &&
              g.numel() == T * hv && beta.numel() == T * hv);
  TORCH_CHECK(state.is_contiguous() && state.scalar_type() == at::kFloat && state.dim() == 4 && state.size(1) == hv);
  TORCH_CHECK(query_start_loc.scalar_type() == at::kInt && query_start_loc.is_contiguous());
  const int64_t B = query_start_loc.numel() - 1;
  if (state_idx.has_value()) TORCH_CHECK(state_idx->scalar_type() == at::kInt && state_idx->numel() >= B);
  if (has_initial.has_value()) TORCH_CHECK(has_initial->scalar_type() == at::kInt && has_initial->numel() >= B);
  const c10::cuda::CUDAGuard guard(q.device());
  const int rc = b200::gdn_recurrent(out.data_ptr(), state.data_ptr<float>(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                     g.data_ptr<float>(), beta.data_ptr<float>(), query_start_loc.data_ptr<int>(),
                                     state_idx.has_value() ? state_idx->data_ptr<int>() : nullptr, (int)B, (int)hq, (int)hv,
                                     (int)q.size(2), (int)v.size(2), q.stride(0), k.stride(0), v.stride(0), (float)scale,
                                     l2norm, has_initial.has_value() ? has_initial->data_ptr<int>() : nullptr,
                                     dtype16(q), cur_stream());
  TORCH_CHECK(rc == 0, "gdn_recurrent: head sizes must be 128 and value heads a multiple of q/k heads");
}

// x [T, C] (row pitch free), w [C, K], state [slots, K-1, C] (in / out), all of one dtype (bf16 / fp16 / fp32)
void causal_conv1d(Tensor& out, const Tensor& x, const Tensor& w, const optional<Tensor>& bias,
                   const optional<Tensor>& state, const Tensor& query_start_loc, const optional<Tensor>& state_idx,
                   const optional<Tensor>& has_initial, bool silu) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.is_contiguous() && out.sizes() == x.sizes() &&
              out.scalar_type() == x.scalar_type());
  const int64_t T = x.size(0), C = x.size(1), K = w.size(1);
  TORCH_CHECK(w.dim() == 2 && w.size(0) == C && w.is_contiguous() && w.scalar_type() == x.scalar_type());
  if (bias.has_value()) TORCH_CHECK(bias->is_contiguous() && bias->numel() == C && bias->scalar_type() == x.scalar_type());
  TORCH_CHECK(query_start_loc.scalar_type() == at::kInt && query_start_loc.is_contiguous());
  const int64_t B = query_start_loc.numel() - 1;
  if (state.has_value()) {
    TORCH_CHECK(state_idx.has_value(), "a carry needs state indices");
    TORCH_CHECK(state->is_contiguous() && state->dim() == 3 && state->size(1) == K - 1 && state->size(2) == C &&
                state->scalar_type() == x.scalar_type());
  }
  if (state_idx.has_value()) TORCH_CHECK(state_idx->scalar_type() == at::kInt && state_idx->numel() >= B);
  if (has_initial.has_value()) TORCH_CHECK(has_initial->scalar_type() == at::kInt && has_initial->numel() >= B);
  const c10::cuda::CUDAGuard guard(x.device());
  const int rc = b200::causal_conv1d(out.data_ptr(), x.data_ptr(), x.stride(0), w.data_ptr(),
                                     bias.has_value() ? bias->data_ptr() : nullptr,
                                     state.has_value() ? state->data_ptr() : nullptr, query_start_loc.data_ptr<int>(),
                                     state_idx.has_value() ? state_idx->data_ptr<int>() : nullptr,
                                     has_initial.has_value() ? has_initial->data_ptr<int>() : nullptr, (int)B, (int)T,
                                     (int)C, (int)K, silu ? 1 : 0, dtype_code(x), cur_stream());
  TORCH_CHECK(rc == 0, "causal_conv1d: kernel width must be 2..8");
}

// TurboQuant cache: uint8 [blocks, block_size, kv_heads, slot_bytes]; k, v [T, kv_heads * 128] (any row pitch)
int64_t tq_slot_bytes(int64_t kbits, int64_t vbits) { return b200::tq_slot_bytes((int)kbits, (int)vbits); }

void tq_store(Tensor& cache, const Tensor& k, const Tensor& v, const Tensor& slot_mapping, int64_t kbits, int64_t vbits,
              bool nc) {
  TORCH_CHECK(cache.dim() == 4 && cache.is_contiguous() && cache.element_size() == 1 &&
              cache.size(3) == b200::tq_slot_bytes((int)kbits, (int)vbits));
  const int64_t heads = cache.size(2);
  TORCH_CHECK(k.dim() == 2 && v.dim() == 2 && k.size(1) == heads * 128 && v.size(1) == heads * 128 && k.stride(1) == 1 &&
              v.stride(1) == 1 && k.stride(0) % 4 == 0 && v.stride(0) % 4 == 0 && k.scalar_type() == v.scalar_type());
  TORCH_CHECK(slot_mapping.scalar_type() == at::kLong && slot_mapping.is_contiguous() && slot_mapping.numel() <= k.size(0));
  const c10::cuda::CUDAGuard guard(k.device());
  const int rc = b200::tq_store(cache.data_ptr(), k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0),
                                slot_mapping.data_ptr<int64_t>(), (int)slot_mapping.numel(), (int)heads,
                                cache.size(0) * cache.size(1), (int)kbits, (int)vbits, nc, dtype16(k), cur_stream());
  TORCH_CHECK(rc == 0, "tq_store: unsupported bit widths");
}

void tq_dequant(Tensor& k_out, Tensor& v_out, const Tensor& cache, const Tensor& slots, int64_t kbits, int64_t vbits,
                bool nc) {
  TORCH_CHECK(cache.dim() == 4 && cache.is_contiguous() && cache.size(3) == b200::tq_slot_bytes((int)kbits, (int)vbits));
  const int64_t heads = cache.size(2), rows = slots.numel();
  TORCH_CHECK(k_out.is_contiguous() && v_out.is_contiguous() && k_out.numel() == rows * heads * 128 &&
              v_out.numel() == k_out.numel() && k_out.scalar_type() == v_out.scalar_type());
  TORCH_CHECK(slots.scalar_type() == at::kLong && slots.is_contiguous());
  const c10::cuda::CUDAGuard guard(cache.device());
  const int rc = b200::tq_dequant(k_out.data_ptr(), v_out.data_ptr(), cache.data_ptr(), slots.data_ptr<int64_t>(),
                                  (int)rows, (int)heads, (int)kbits, (int)vbits, nc, dtype16(k_out), cur_stream());
  TORCH_CHECK(rc == 0, "tq_dequant: unsupported bit widths");
}

// q [B, Hq, 128] (one query token per sequence); workspace f32 [splits * B * Hq * 129] when splits > 1
void tq_decode(Tensor& out, const Tensor& q, const Tensor& cache, const Tensor& block_table, const Tensor& seq_lens,
               const optional<Tensor>& workspace, double scale, int64_t splits, int64_t kbits, int64_t vbits, bool nc) {
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.stride(2) == 1 && q.stride(1) == 128 && q.stride(0) % 4 == 0);
  TORCH_CHECK(out.is_contiguous() && out.sizes() == q.sizes() && out.scalar_type() == q.scalar_type());
  TORCH_CHECK(cache.dim() == 4 && cache.is_contiguous() && cache.size(3) == b200::tq_slot_bytes((int)kbits, (int)vbits));
  TORCH_CHECK(block_table.dim() == 2 && block_table.is_contiguous() && block_table.scalar_type() == at::kInt &&
              block_table.size(0) >= q.size(0) && seq_lens.scalar_type() == at::kInt && seq_lens.numel() >= q.size(0));
  const int64_t B = q.size(0), hq = q.size(1), hkv = cache.size(2);
  TORCH_CHECK(hq % hkv == 0 && splits >= 1);
  float* part = nullptr;
  if (splits > 1) {
    TORCH_CHECK(workspace.has_value() && workspace->scalar_type() == at::kFloat && workspace->is_contiguous() &&
                workspace->numel() >= splits * B * hq * 129);
    part = workspace->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(q.device());
  const int rc = b200::tq_decode(out.data_ptr(), part, part ? part + splits * B * hq * 128 : nullptr, q.data_ptr(),
                                 q.stride(0), cache.data_ptr(), block_table.data_ptr<int>(), (int)block_table.size(1),
                                 seq_lens.data_ptr<int>(), (int)B, (int)hq, (int)hkv, (int)cache.size(1), cache.size(0),
                                 (int)splits, (float)scale, (int)kbits, (int)vbits, nc, dtype16(q), cur_stream());
  TORCH_CHECK(rc == 0, "tq_decode: unsupported format or GQA group (1, 2, 4, 8)");
}

// o [T, H, 512] -> out [G, T, (H / G) * 512] with the rope dims rotated back
void v4_inv_rope(Tensor& out, const Tensor& o, const Tensor& positions, const Tensor& cos_sin, int64_t n_groups) {
  TORCH_CHECK(o.dim() == 3 && o.size(2) == 512 && o.stride(2) == 1 && o.stride(0) % 8 == 0 && o.stride(1) % 8 == 0);
  TORCH_CHECK(n_groups >= 1 && o.size(1) % n_groups == 0 && out.is_contiguous() && out.numel() == o.numel() &&
              out.scalar_type() == o.scalar_type());
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() >= o.size(0));
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.dim() == 2 && cos_sin.size(1) == 64 && cos_sin.is_contiguous());
  const c10::cuda::CUDAGuard guard(o.device());
  b200::v4_inv_rope(out.data_ptr(), o.data_ptr(), o.stride(0), o.stride(1), positions.data_ptr<int64_t>(),
                    cos_sin.data_ptr<float>(), (int)o.size(0), (int)o.size(1), (int)(o.size(1) / n_groups), dtype16(o),
                    cur_stream());
}

// q [T, H, 128] -> q8 int8 [T, H, 128], w_out f32 [T, H] = weights * q_scale * softmax_scale * head_scale
void v4_indexer_q(Tensor& q8, Tensor& w_out, const Tensor& q, const Tensor& weights, const Tensor& positions,
                  const Tensor& cos_sin, double softmax_scale, double head_scale) {
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.stride(2) == 1 && q.stride(0) % 4 == 0 && q.stride(1) % 4 == 0);
  TORCH_CHECK(q8.is_contiguous() && q8.element_size() == 1 && q8.numel() == q.numel());
  TORCH_CHECK(w_out.is_contiguous() && w_out.scalar_type() == at::kFloat && w_out.numel() == q.size(0) * q.size(1));
  TORCH_CHECK(weights.dim() == 2 && weights.size(0) == q.size(0) && weights.size(1) == q.size(1) &&
              weights.stride(1) == 1 && weights.scalar_type() == q.scalar_type());
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() >= q.size(0));
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.dim() == 2 && cos_sin.is_contiguous() &&
              cos_sin.size(1) % 4 == 0 && cos_sin.size(1) <= 128);
  const c10::cuda::CUDAGuard guard(q.device());
  b200::v4_indexer_q(q8.data_ptr(), w_out.data_ptr<float>(), q.data_ptr(), q.stride(0), q.stride(1), weights.data_ptr(),
                     weights.stride(0), positions.data_ptr<int64_t>(), cos_sin.data_ptr<float>(), (int)q.size(0),
                     (int)q.size(1), (int)cos_sin.size(1), (float)softmax_scale, (float)head_scale, dtype16(q),
                     cur_stream());
}

// ptrs: int64 CPU tensor [4, tp] = recv, gather, flag1, flag2 (per owning rank)
void custom_allreduce(Tensor& out, const Tensor& inp, const Tensor& ptrs, int64_t tp, int64_t rank, int64_t cap_bytes,
                      int64_t max_ctas, Tensor& local_sync, int64_t mode, int64_t wait_cycles) {
  TORCH_CHECK(inp.is_contiguous() && out.is_contiguous() && inp.scalar_type() == out.scalar_type() &&
              inp.numel() == out.numel());
  TORCH_CHECK(tp >= 1 && tp <= b200::kMaxRanks && ptrs.dim() == 2 && ptrs.size(0) == 4 && ptrs.size(1) >= tp);
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong && local_sync.numel() >= 2);
  b200::CustomArParams p{};
  p.tp = tp; p.rank = rank; p.n_bytes = (long long)inp.numel() * inp.element_size(); p.cap_bytes = cap_bytes;
  p.max_ctas = max_ctas;
  const int64_t* pp = ptrs.data_ptr<int64_t>();
  const int64_t st = ptrs.stride(0);
  for (int r = 0; r < tp; ++r) {
    p.recv[r] = reinterpret_cast<void*>(pp[0 * st + r]);
    p.gather[r] = reinterpret_cast<void*>(pp[1 * st + r]);
    p.flag1[r] = reinterpret_cast<uint32_t*>(pp[2 * st + r]);
    p.flag2[r] = reinterpret_cast<uint32_t*>(pp[3 * st + r]);
  }
  p.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(inp));
  const int dt = inp.scalar_type() == at::kBFloat16 ? 0 : inp.scalar_type() == at::kHalf ? 1
               : inp.scalar_type() == at::kFloat ? 2 : -1;
  const c10::cuda::CUDAGuard guard(inp.device());
  const int rc = b200::custom_allreduce(p, inp.data_ptr(), out.data_ptr(), dt, (int)mode, cur_stream());
  TORCH_CHECK(rc == 0, "custom_allreduce: payload must be bf16/fp16/fp32, a multiple of 16 bytes and fit the buffers");
}

// slots_ptrs: int64 CPU tensor [tp]; x / w / out: one or two tensors (q and k) normalised over the hidden
// dimension of ALL ranks
void reduce_rms(Tensor& out0, const Tensor& x0, const Tensor& w0, const optional<Tensor>& out1,
                const optional<Tensor>& x1, const optional<Tensor>& w1, double eps, const Tensor& slots_ptrs,
                int64_t tp, int64_t rank, int64_t t_cap, Tensor& local_sync, int64_t wait_cycles) {
  TORCH_CHECK(x0.dim() == 2 && x0.stride(1) == 1 && out0.dim() == 2 && out0.stride(1) == 1 &&
              out0.stride(0) == x0.stride(0) && w0.numel() == x0.size(1) && w0.scalar_type() == x0.scalar_type());
  TORCH_CHECK(tp >= 1 && tp <= b200::kMaxRanks && !slots_ptrs.is_cuda() && slots_ptrs.numel() >= tp &&
              local_sync.numel() >= 5);
  b200::ReduceRmsParams p{};
  p.tp = tp; p.rank = rank; p.T = x0.size(0); p.n_tensors = x1.has_value() ? 2 : 1;
  p.x[0] = x0.data_ptr(); p.w[0] = w0.data_ptr(); p.out[0] = out0.data_ptr(); p.H[0] = x0.size(1); p.ld[0] = x0.stride(0);
  if (x1.has_value()) {
    TORCH_CHECK(out1.has_value() && w1.has_value() && x1->dim() == 2 && x1->size(0) == x0.size(0) && x1->stride(1) == 1 &&
                out1->stride(0) == x1->stride(0) && out1->stride(1) == 1 && w1->numel() == x1->size(1) &&
                x1->scalar_type() == x0.scalar_type() && w1->scalar_type() == x0.scalar_type());
    p.x[1] = x1->data_ptr(); p.w[1] = w1->data_ptr(); p.out[1] = out1->data_ptr(); p.H[1] = x1->size(1);
    p.ld[1] = x1->stride(0);
  }
  p.eps = (float)eps;
  const int64_t* pp = slots_ptrs.data_ptr<int64_t>();
  for (int r = 0; r < tp; ++r) p.slots[r] = reinterpret_cast<float*>(pp[r]);
  p.t_cap = t_cap;
  p.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(x0));
  const c10::cuda::CUDAGuard guard(x0.device());
  const int rc = b200::reduce_rms(p, dtype16(x0), cur_stream());
  TORCH_CHECK(rc == 0, "reduce_rms: widths and pitches must be multiples of 8 and T must fit the slot arrays");
}

// ptrs: int64 CPU tensor [3, tp] = x_shard, xready, done (per owning rank)
void ag_gemm(Tensor& out, const Tensor& w, const optional<Tensor>& bias, const Tensor& ptrs, Tensor& gathered,
             Tensor& ready, Tensor& sync, int64_t tp, int64_t rank, int64_t rows_per_rank, int64_t wait_cycles) {
  TORCH_CHECK(w.dim() == 2 && w.stride(1) == 1 && w.stride(0) % 8 == 0 && out.dim() == 2 && out.stride(1) == 1);
  TORCH_CHECK(tp >= 1 && tp <= b200::kMaxRanks && ptrs.dim() == 2 && ptrs.size(0) == 3 && ptrs.size(1) >= tp);
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong && gathered.is_contiguous());
  b200::AgGemmParams p{};
  p.rows_per_rank = rows_per_rank; p.N = w.size(0); p.K = w.size(1); p.tp = tp; p.rank = rank; p.ldc = out.stride(0);
  TORCH_CHECK(out.size(0) == tp * rows_per_rank && out.size(1) == p.N && gathered.numel() >= tp * rows_per_rank * p.K);
  TORCH_CHECK(ready.numel() >= tp * rows_per_rank / 128 && sync.numel() >= 3 && rows_per_rank % 128 == 0 && p.K % 64 == 0);
  const int64_t* pp = ptrs.data_ptr<int64_t>();
  const int64_t st = ptrs.stride(0);
  for (int r = 0; r < tp; ++r) {
    p.x_shard[r] = reinterpret_cast<void*>(pp[0 * st + r]);
    p.xready[r] = reinterpret_cast<uint32_t*>(pp[1 * st + r]);
    p.done[r] = reinterpret_cast<uint32_t*>(pp[2 * st + r]);
  }
  p.gathered = gathered.data_ptr();
  p.ready = reinterpret_cast<uint32_t*>(ready.data_ptr());
  p.sync = reinterpret_cast<uint32_t*>(sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(w));
  if (bias.has_value()) TORCH_CHECK(bias->numel() == p.N && bias->scalar_type() == w.scalar_type());
  const c10::cuda::CUDAGuard guard(w.device());
  const int rc = b200::ag_gemm(p, w.data_ptr(), w.stride(0), out.data_ptr(), bias.has_value() ? bias->data_ptr() : nullptr,
                               dtype16(w), cur_stream());
  TORCH_CHECK(rc == 0, "ag_gemm: rows per rank must be a multiple of 128");
}

// ptrs: int64 CPU tensor [9, ep] = recv_x, recv_scale, recv_ids, recv_src, recv_count, disp_flag, comb_x, comb_flag,
// recv_w
static b200::MoeA2aParams a2a_params(const Tensor& ptrs, int64_t ep, int64_t rank, int64_t experts_per_rank, int64_t H,
                                     int64_t topk, int64_t T, int64_t cap, bool quant, Tensor& local_sync,
                                     int64_t wait_cycles, const Tensor& any) {
  TORCH_CHECK(ep >= 1 && ep <= b200::kMaxRanks && ptrs.dim() == 2 && ptrs.size(0) == 9 && ptrs.size(1) >= ep);
  TORCH_CHECK(!ptrs.is_cuda() && ptrs.scalar_type() == at::kLong && H % 8 == 0 && (!quant || H % 128 == 0));
  TORCH_CHECK(local_sync.numel() >= 8 + ep && local_sync.element_size() == 4);
  b200::MoeA2aParams p{};
  p.ep = ep; p.rank = rank; p.experts_per_rank = experts_per_rank; p.H = H; p.topk = topk; p.T = T; p.cap = cap;
  p.quant = quant;
  const int64_t* pp = ptrs.data_ptr<int64_t>();
  const int64_t st = ptrs.stride(0);
  for (int r = 0; r < ep; ++r) {
    p.recv_x[r] = reinterpret_cast<void*>(pp[0 * st + r]);
    p.recv_scale[r] = reinterpret_cast<float*>(pp[1 * st + r]);
    p.recv_ids[r] = reinterpret_cast<int*>(pp[2 * st + r]);
    p.recv_src[r] = reinterpret_cast<int*>(pp[3 * st + r]);
    p.recv_count[r] = reinterpret_cast<uint32_t*>(pp[4 * st + r]);
    p.disp_flag[r] = reinterpret_cast<uint32_t*>(pp[5 * st + r]);
    p.comb_x[r] = reinterpret_cast<void*>(pp[6 * st + r]);
    p.comb_flag[r] = reinterpret_cast<uint32_t*>(pp[7 * st + r]);
    p.recv_w[r] = reinterpret_cast<float*>(pp[8 * st + r]);
  }
  p.local_sync = reinterpret_cast<uint32_t*>(local_sync.data_ptr());
  p.wait_cycles = wait_cycles;
  p.status = reinterpret_cast<b200::StatusWord*>(status_ptr(any));
  return p;
}

void moe_a2a_dispatch(const Tensor& x, const Tensor& topk_ids, const Tensor& topk_w, const Tensor& ptrs, int64_t ep,
                      int64_t rank, int64_t experts_per_rank, int64_t cap, bool quant, Tensor& local_sync,
                      int64_t wait_cycles) {
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && topk_ids.is_contiguous() && topk_ids.scalar_type() == at::kInt);
  TORCH_CHECK(topk_ids.size(0) == x.size(0) && topk_w.is_contiguous() && topk_w.scalar_type() == at::kFloat &&
              topk_w.sizes() == topk_ids.sizes() && x.size(0) <= cap);
  auto p = a2a_params(ptrs, ep, rank, experts_per_rank, x.size(1), topk_ids.size(1), x.size(0), cap, quant, local_sync,
                      wait_cycles, x);
  const c10::cuda::CUDAGuard guard(x.device());
  b200::moe_a2a_dispatch(p, x.data_ptr(), topk_ids.data_ptr<int>(), topk_w.data_ptr<float>(), dtype16(x), cur_stream());
}

// y [ep*cap, H]: weighted partial sums of the received tokens, one row per receive slot
void moe_a2a_combine(Tensor& out, const Tensor& y, const Tensor& topk_ids, const optional<Tensor>& shared_out,
                     const Tensor& ptrs, int64_t ep, int64_t rank, int64_t experts_per_rank, int64_t cap,
                     Tensor& local_sync, int64_t wait_cycles) {
  TORCH_CHECK(y.dim() == 2 && y.is_contiguous() && y.size(0) == ep * cap && out.is_contiguous() && out.size(1) == y.size(1));
  TORCH_CHECK(topk_ids.is_contiguous() && topk_ids.scalar_type() == at::kInt && topk_ids.size(0) == out.size(0) &&
              out.scalar_type() == y.scalar_type() && out.size(0) <= cap);
  if (shared_out.has_value()) TORCH_CHECK(shared_out->is_contiguous() && shared_out->sizes() == out.sizes());
  auto p = a2a_params(ptrs, ep, rank, experts_per_rank, y.size(1), topk_ids.size(1), out.size(0), cap, false,
                      local_sync, wait_cycles, y);
  const c10::cuda::CUDAGuard guard(y.device());
  b200::moe_a2a_combine(p, y.data_ptr(), out.data_ptr(), topk_ids.data_ptr<int>(),
                        shared_out.has_value() ? shared_out->data_ptr() : nullptr, dtype16(y), cur_stream());
}

// dst[i] = src[idx[i] / div] for i < count[0] (rows of any dtype whose byte width is a multiple of 16)
void gather_rows(Tensor& dst, const Tensor& src, const Tensor& idx, const Tensor& count, int64_t div) {
  TORCH_CHECK(dst.is_contiguous() && src.is_contiguous() && dst.dim() == 2 && src.dim() == 2);
  const int64_t row_bytes = src.size(1) * src.element_size();
  TORCH_CHECK(row_bytes % 16 == 0 && dst.size(1) * dst.element_size() == row_bytes && idx.numel() >= dst.size(0));
  const c10::cuda::CUDAGuard guard(src.device());
  b200::gather_rows(dst.data_ptr(), src.data_ptr(), idx.data_ptr<int>(), count.data_ptr<int>(), dst.size(0),
                    src.size(0), row_bytes, (int)div, cur_stream());
}

}  // namespace

TORCH_LIBRARY(b200, m) {
  m.def("moe_a2a_dispatch(Tensor x, Tensor topk_ids, Tensor topk_w, Tensor ptrs, int ep, int rank, int experts_per_rank, int cap, bool quant, Tensor(a!) local_sync, int wait_cycles) -> ()", &moe_a2a_dispatch);
  m.def("moe_a2a_combine(Tensor(a!) out, Tensor y, Tensor topk_ids, Tensor? shared_out, Tensor ptrs, int ep, int rank, int experts_per_rank, int cap, Tensor(b!) local_sync, int wait_cycles) -> ()", &moe_a2a_combine);
  m.def("v4_qnorm_rope_kv_insert(Tensor(a!) q_out, Tensor(b!) cache, Tensor q, Tensor kv, Tensor slot_mapping, Tensor positions, Tensor cos_sin, float eps, int block_size) -> ()", &v4_qnorm_rope_kv_insert);
  m.def("v4_gather_dequant(Tensor(a!) dst, Tensor cache, Tensor slots, int block_size) -> ()", &v4_gather_dequant);
  m.def("causal_conv1d(Tensor(a!) out, Tensor x, Tensor w, Tensor? bias, Tensor(b!)? state, Tensor query_start_loc, Tensor? state_idx, Tensor? has_initial, bool silu) -> ()", &causal_conv1d);
  m.def("gdn_recurrent(Tensor(a!) out, Tensor(b!) state, Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor query_start_loc, Tensor? state_idx, Tensor? has_initial, float scale, bool l2norm) -> ()", &gdn_recurrent);
  m.def("tq_slot_bytes(int kbits, int vbits) -> int", &tq_slot_bytes);
  m.def("tq_store(Tensor(a!) cache, Tensor k, Tensor v, Tensor slot_mapping, int kbits, int vbits, bool nc) -> ()", &tq_store);
  m.def("tq_dequant(Tensor(a!) k_out, Tensor(b!) v_out, Tensor cache, Tensor slots, int kbits, int vbits, bool nc) -> ()", &tq_dequant);
  m.def("tq_decode(Tensor(a!) out, Tensor q, Tensor cache, Tensor block_table, Tensor seq_lens, Tensor? workspace, float scale, int splits, int kbits, int vbits, bool nc) -> ()", &tq_decode);
  m.def("v4_inv_rope(Tensor(a!) out, Tensor o, Tensor positions, Tensor cos_sin, int n_groups) -> ()", &v4_inv_rope);
  m.def("v4_indexer_q(Tensor(a!) q8, Tensor(b!) w_out, Tensor q, Tensor weights, Tensor positions, Tensor cos_sin, float softmax_scale, float head_scale) -> ()", &v4_indexer_q);
  m.def("custom_allreduce(Tensor(a!) out, Tensor inp, Tensor ptrs, int tp, int rank, int cap_bytes, int max_ctas, Tensor(b!) local_sync, int mode, int wait_cycles) -> ()", &custom_allreduce);
  m.def("reduce_rms(Tensor(a!) out0, Tensor x0, Tensor w0, Tensor(b!)? out1, Tensor? x1, Tensor? w1, float eps, Tensor slots_ptrs, int tp, int rank, int t_cap, Tensor(c!) local_sync, int wait_cycles) -> ()", &reduce_rms);
  m.def("ag_gemm(Tensor(a!) out, Tensor w, Tensor? bias, Tensor ptrs, Tensor(b!) gathered, Tensor(c!) ready, Tensor(d!) sync, int tp, int rank, int rows_per_rank, int wait_cycles) -> ()", &ag_gemm);
  m.def("mhc_pre(Tensor(a!) x_out, Tensor(b!)? post_out, Tensor(c!)? comb_out, Tensor residual, Tensor(d!)? residual_out, Tensor? y, Tensor? post_in, Tensor? comb_in, Tensor fn, Tensor scale, Tensor base, float rms_eps, float pre_eps, float sinkhorn_eps, float post_mult, int iters, bool head) -> ()", &mhc_pre);
  m.def("mhc_post(Tensor(a!) out, Tensor y, Tensor residual, Tensor post, Tensor comb) -> ()", &mhc_post);
  m.def("small_gemm(Tensor(a!) out, Tensor a, Tensor w, Tensor? bias) -> ()", &small_gemm);
  m.def("qkv_norm_rope_insert(Tensor(a!) qkv, Tensor(b!) q_out, Tensor(c!)? iq_out, Tensor(d!)? kv_cache, Tensor(e!)? idx_cache, Tensor? q_w, Tensor? k_w, Tensor? iq_w, Tensor? ik_w, Tensor cos_sin, Tensor positions, Tensor slot_mapping, int hq, int hk, int niq, bool has_ik, bool is_neox, float eps, bool gemma) -> ()", &qkv_norm_rope_insert);
  m.def("fused_qk_norm_rope(Tensor(a!) qkv, Tensor q_weight, Tensor k_weight, Tensor cos_sin, Tensor positions, int hq, int hk, int hv, int head_dim, bool is_neox, float eps, bool gemma) -> ()", &fused_qk_norm_rope);
  m.def("mla_rope_and_cache(Tensor(a!) q_pe, Tensor(b!) k_pe, Tensor kv_c, Tensor(c!) cache, Tensor cos_sin, Tensor positions, Tensor slot_mapping, bool is_neox) -> ()", &mla_rope_and_cache);
  m.def("concat_mla_q(Tensor(a!) out, Tensor nope, Tensor pe) -> ()", &concat_mla_q);
  m.def("permute_cols(Tensor(a!) out, Tensor a, Tensor perm) -> ()", &permute_cols);
  m.def("gather_mla_cache(Tensor(a!) dst, Tensor cache, Tensor block_table, Tensor cu_seq_lens, Tensor? seq_starts) -> ()", &gather_mla_cache);
  m.def("gather_indexer_k(Tensor(a!) dst_k, Tensor(b!) dst_s, Tensor cache, Tensor block_table, Tensor cu_seq_lens, int block_size) -> ()", &gather_indexer_k);
  m.def("selective_scan(Tensor(a!) out, Tensor u, Tensor delta, Tensor A, Tensor B, Tensor C, Tensor? D, Tensor? z, Tensor? delta_bias, bool delta_softplus, Tensor(b!) state, Tensor? query_start_loc, Tensor? cache_indices, Tensor? has_initial_state, int pad_slot) -> ()", &selective_scan);
  m.def("p2p_copy(int dst_ptr, Tensor src, int ctas, int mode) -> ()", &p2p_copy);
  m.def("gather_rows(Tensor(a!) dst, Tensor src, Tensor idx, Tensor count, int div) -> ()", &gather_rows);
  m.def("get_status(int device) -> Tensor", &get_status);
  m.def("topk_gating(Tensor(a!) weights, Tensor(b!) ids, Tensor gating, Tensor? bias, int mode, bool renorm, float scale) -> ()", &topk_gating);
  m.def("grouped_topk(Tensor(a!) weights, Tensor(b!) ids, Tensor gating, Tensor? bias, int n_group, int topk_group, bool sigmoid, bool renorm, float scale) -> ()", &grouped_topk);
  m.def("moe_align(Tensor(a!) sorted_ids, Tensor(b!) block_expert, Tensor(c!) total_padded, Tensor(d!)? inv_pos, Tensor topk_ids, Tensor? expert_map, int experts, int block) -> ()", &moe_align);
  m.def("moe_gather(Tensor(a!) out, Tensor x, Tensor sorted_ids, Tensor total_padded, int topk) -> ()", &moe_gather);
  m.def("moe_combine(Tensor(a!) out, Tensor y, Tensor weights, Tensor inv_pos, Tensor? shared) -> ()", &moe_combine);
  m.def("moe_sum(Tensor(a!) out, Tensor inp) -> ()", &moe_sum);
  m.def("gemm_grouped(Tensor(a!) out, Tensor a, Tensor w, Tensor block_expert, Tensor total_padded, int epi) -> ()", &gemm_grouped);
  m.def("per_token_group_quant(Tensor(a!) q, Tensor(b!) scales, Tensor x, int group, bool ue8m0, bool col_major, float eps) -> ()", &per_token_group_quant);
  m.def("scaled_fp8_quant(Tensor(a!) q, Tensor(b!) scale, Tensor x, int mode, float scale_ub) -> ()", &scaled_fp8_quant);
  m.def("scaled_int8_quant(Tensor(a!) q, Tensor(b!) scale, Tensor(c!)? azp, Tensor x, int mode) -> ()", &scaled_int8_quant);
  m.def("merge_attn_states(Tensor(a!) out, Tensor(b!)? out_lse, Tensor p_out, Tensor p_lse, Tensor s_out, Tensor s_lse) -> ()", &merge_attn_states);
  m.def("gemm_fp8_blockscale(Tensor(a!) out, Tensor a, Tensor a_scale, Tensor w, Tensor w_scale, Tensor? block_expert, Tensor? total_padded) -> ()", &gemm_fp8_blockscale);
  m.def("scaled_mm(Tensor(a!) out, Tensor a, Tensor w, Tensor a_scale, Tensor w_scale, Tensor? azp, Tensor? azp_adj, Tensor? bias, Tensor? block_expert, Tensor? total_padded) -> ()", &scaled_mm);
  m.def("wna16_gemm(Tensor(a!) out, Tensor a, Tensor q, Tensor scales, Tensor? zeros, int bits, int group, Tensor? bias, Tensor? block_expert, Tensor? total_padded, int token_tile, int epi) -> ()", &wna16_gemm);
  m.def("mla_decode(Tensor(a!) out, Tensor q, Tensor cache, Tensor block_table, Tensor seq_lens, Tensor? query_start_loc, Tensor? topk_indices, float scale, Tensor(b!)? lse_out, Tensor(c!)? workspace, int num_splits, int impl=1) -> ()", &mla_decode);
  m.def("indexer_logits(Tensor(a!) logits, Tensor q, Tensor w, Tensor cache, Tensor block_table, Tensor seq_lens, Tensor query_start_loc, int block_size, int max_len, bool int8, int max_query_len, int impl) -> ()", &indexer_logits);
  m.def("topk_per_row(Tensor(a!) out, Tensor x, Tensor? row_len, int cols) -> ()", &topk_per_row);
  m.def("symm_alloc(int nbytes, int device) -> (Tensor, Tensor)", &symm_alloc);
  m.def("symm_open(Tensor handle, int device) -> int", &symm_open);
  m.def("symm_close(int ptr) -> ()", &symm_close);
  m.def(
      "gemm_row_scatter(Tensor x, Tensor w, Tensor ptrs, int tp, int rank, int rows_per_rank, int rows_cap, "
      "Tensor(a!) local_sync) -> ()",
      &gemm_row_scatter);
  m.def(
      "ar_norm_gather(Tensor(a!) residual, Tensor norm_weight, float eps, Tensor ptrs, int T, int H, int tp, int rank, "
      "int rows_per_rank, int rows_cap, Tensor(b!) local_sync, bool add_residual, int wait_cycles, "
      "int out_multicast_ptr=0) -> ()",
      &ar_norm_gather);
  m.def(
      "nvls_ar_norm(Tensor(a!) residual, Tensor norm_weight, float eps, int partial_mc, int out_mc, int flag_mc, "
      "int flag_local, int T, int H, int tp, int rank, int rows_per_rank, Tensor(b!) local_sync, bool add_residual, "
      "int wait_cycles) -> ()",
      &nvls_ar_norm);
  m.def(
      "gemm_ar_norm(Tensor x, Tensor w, Tensor(a!) residual, Tensor norm_weight, float eps, Tensor ptrs, int tp, "
      "int rank, int rows_per_rank, int rows_cap, int rb_cap, Tensor(b!) local_sync, bool add_residual, "
      "int wait_cycles) -> ()",
      &gemm_ar_norm);
  m.def("gemm(Tensor(a!) out, Tensor a, Tensor w, Tensor? bias, Tensor? residual, int force_bn, int epi) -> ()", &gemm);
  m.def("rms_norm(Tensor(a!) out, Tensor x, Tensor weight, float eps, bool gemma) -> ()", &rms_norm);
  m.def("fused_add_rms_norm(Tensor(a!) x, Tensor(b!) residual, Tensor weight, float eps, bool gemma) -> ()",
        &fused_add_rms_norm);
  m.def("head_rms_norm(Tensor(a!) x, Tensor weight, float eps, int heads, int head_dim) -> ()", &head_rms_norm);
  m.def(
      "rms_norm_quant(Tensor(a!) out_q, Tensor(b!)? scale_out, Tensor? scale_in, Tensor x, Tensor(c!)? residual, "
      "Tensor weight, float eps, int qmode, int group, bool ue8m0, float scale_ub) -> ()",
      &rms_norm_quant);
  m.def(
      "rope_and_cache(Tensor? positions, Tensor(a!)? q, Tensor(b!)? k, Tensor? v, Tensor? cos_sin, int head_dim, "
      "int num_q, int num_kv, bool is_neox, int rot_offset, bool inverse, Tensor(c!)? kv_cache, "
      "Tensor(d!)? kv_scales, Tensor? slot_mapping, int cache_kind, float k_scale, float v_scale) -> ()",
      &rope_and_cache);
  m.def("copy_blocks(Tensor(a!) cache, Tensor pairs) -> ()", &copy_blocks);
  m.def("concat_and_cache_mla(Tensor kv_c, Tensor k_pe, Tensor(a!) cache, Tensor slot_mapping) -> ()",
        &concat_and_cache_mla);
  m.def(
      "indexer_k_quant_and_cache(Tensor k, Tensor(a!) cache, Tensor slot_mapping, int block_size, bool ue8m0, bool int8) -> ()",
      &indexer_k_quant_and_cache);
  m.def("act_and_mul(Tensor(a!) out, Tensor x, int act, float p0, float p1) -> ()", &act_and_mul);
  m.def("activation(Tensor(a!) out, Tensor x, int act, float p0) -> ()", &activation);
  m.def(
      "act_and_mul_quant(Tensor(a!) out_q, Tensor(b!)? scale_out, Tensor? scale_in, Tensor x, int act, float p0, "
      "float p1, int group, bool ue8m0) -> ()",
      &act_and_mul_quant);
  m.def(
      "paged_attention_decode(Tensor(a!) out, Tensor q, Tensor kv_cache, Tensor? kv_scales, Tensor block_table, "
      "Tensor seq_lens, Tensor? query_start_loc, float scale, int window, float softcap, Tensor? sinks, "
      "Tensor(b!)? lse_out, Tensor(c!)? workspace, int num_splits, int batch, int max_q_len, float k_scale, "
      "float v_scale, bool causal, Tensor? alibi_slopes=None) -> ()",
      &paged_attention_decode);
  m.def(
      "attention_prefill(Tensor(a!) out, Tensor q, Tensor k_src, Tensor? v_src, Tensor? block_table, "
      "Tensor? seq_lens, Tensor query_start_loc, Tensor? kv_start_loc, float scale, int window, float softcap, "
      "Tensor? sinks, Tensor(b!)? lse_out, int batch, int max_q_len, bool causal, Tensor? alibi_slopes=None) -> ()",
      &attention_prefill);
  m.def("argmax(Tensor(a!) out, Tensor logits) -> ()", &argmax);
  m.def(
      "sample(Tensor(a!) out, Tensor logits, Tensor temperature, Tensor? top_k, Tensor? top_p, Tensor? min_p, "
      "Tensor uniform) -> ()",
      &sample);
  m.def(
      "apply_penalties(Tensor(a!) logits, Tensor? prompt_mask, Tensor? output_counts, Tensor? rep, Tensor? presence, "
      "Tensor? frequency) -> ()",
      &apply_penalties);
  m.def(
      "advance_step(Tensor(a!) input_ids, Tensor(b!) positions, Tensor(c!) seq_lens, Tensor(d!) slot_mapping, "
      "Tensor sampled, Tensor block_table, int block_size, int batch, Tensor(e!)? token_log, int log_col) -> ()",
      &advance_step);
  m.def("embedding(Tensor(a!) out, Tensor table, Tensor ids, int vocab_start) -> ()", &embedding);
  m.def("weak_ref_tensor(Tensor input) -> Tensor", &weak_ref_tensor);
}
