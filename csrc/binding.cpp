// Python bindings (torch extension `bee2bee_b200._C`).  The only torch-facing translation
// unit: it validates tensors, picks the current CUDA stream and calls the C launchers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gemm_tc.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "peer.h"

using at::Tensor;
using OptT = c10::optional<Tensor>;

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check(int err, const char* what) {
  if (err != 0) {
    const char* msg = err > 0 ? cudaGetErrorString(static_cast<cudaError_t>(err)) : "invalid argument";
    TORCH_CHECK(false, what, " failed: code ", err, " (", msg, ")");
  }
}
template <typename T>
inline T* ptr_or_null(const OptT& t) {
  return (t.has_value() && t->defined()) ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}
template <typename T>
inline T* as_ptr(int64_t addr) { return reinterpret_cast<T*>(static_cast<uintptr_t>(addr)); }

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name,
              " must be a contiguous CUDA bf16 tensor");
}

// ---------------------------------------------------------------------- GEMM
// out[t, n] = epi(X[t,:] . W[n,:]).  Handoff pointers are raw device addresses (0 = unused)
// because they may live in IPC-mapped peer memory.
void gemm(const Tensor& w, const Tensor& x, int64_t out_ptr, int64_t ld_out, int64_t epi, int64_t bn,
          int64_t splitk, int64_t residual_ptr, int64_t ld_res, const OptT& bias, const OptT& rstd,
          bool norm_from_x, double eps, int64_t act_gelu, bool out_fp32,
          // qkv epilogue
          const OptT& q_out, const OptT& k_cache, const OptT& v_cache, const OptT& positions, const OptT& slots,
          int64_t n_q_heads, int64_t n_kv_heads, int64_t head_dim, double rope_theta, double q_scale,
          // handoff
          int64_t wait_flag, int64_t wait_epoch, int64_t signal_flag, int64_t signal_epoch, int64_t done_counter,
          int64_t free_flag, int64_t bump_epoch, int64_t ack_flag, int64_t dbg, const OptT& w_scale,
          const OptT& sfa, const OptT& sfb, int64_t mc, int64_t pf_tiles, int64_t stages, int64_t free_lag, int64_t out2_ptr,
          // fused MX quantisation of the output / RMSNorm statistics (raw addresses, 0 = off)
          int64_t q_out8, int64_t q_sf, int64_t ld_q, int64_t q_bn, int64_t sumsq_out, int64_t zero_buf, int64_t sumsq) {
  const bool fp8 = w.scalar_type() == at::kFloat8_e4m3fn;
  if (fp8) {
    TORCH_CHECK(x.scalar_type() == at::kFloat8_e4m3fn && w.is_cuda() && x.is_cuda() && w.is_contiguous() &&
                x.is_contiguous(), "fp8 gemm: w and x must be contiguous CUDA float8_e4m3fn");
    const bool mx = sfa.has_value();
    TORCH_CHECK(mx == sfb.has_value(), "MX fp8 gemm needs both sfa and sfb");
    if (mx) {
      const int64_t nkc = w.size(1) / 128, chunk = bn > 128 ? 1024 : 512;
      TORCH_CHECK(w.size(1) % 128 == 0 && bn >= 32, "MX fp8 gemm: K must be a multiple of 128 and bn >= 32");
      TORCH_CHECK(sfa->scalar_type() == at::kByte && sfa->is_contiguous() && sfa->numel() >= (w.size(0) / 128) * nkc * 512,
                  "MX fp8 gemm: sfa too small");
      TORCH_CHECK(sfb->scalar_type() == at::kByte && sfb->is_contiguous() &&
                      sfb->numel() >= ((x.size(0) + bn - 1) / bn) * nkc * chunk, "MX fp8 gemm: sfb too small");
    } else {
      TORCH_CHECK(w_scale.has_value() && w_scale->scalar_type() == at::kFloat, "fp8 gemm needs per-row w_scale (fp32)");
    }
  } else {
    check_bf16(w, "w");
    check_bf16(x, "x");
  }
  TORCH_CHECK(w.dim() == 2 && x.dim() == 2 && w.size(1) == x.size(1), "gemm: shape mismatch");
  c10::cuda::CUDAGuard guard(w.device());
  b2b::GemmParams p{};
  p.m_tok = static_cast<int>(x.size(0));
  p.n_out = static_cast<int>(w.size(0));
  p.k = static_cast<int>(w.size(1));
  p.splitk = static_cast<int8_t>(splitk);
  p.epi = static_cast<int8_t>(epi);
  p.out_fp32 = out_fp32 ? 1 : 0;
  p.act_gelu = static_cast<int8_t>(act_gelu);   // 0 / 1: see GemmParams; 2: squared relu (EPI_GELU)
  p.fp8 = fp8 ? 1 : 0;
  p.stages = static_cast<int8_t>(stages);
  p.mc = static_cast<int8_t>(mc);      // experimental TMA-multicast cluster (0/1 = off)
  p.w_scale = ptr_or_null<const float>(w_scale);
  p.sfa = fp8 ? ptr_or_null<const uint8_t>(sfa) : nullptr;
  p.sfb = fp8 ? ptr_or_null<const uint8_t>(sfb) : nullptr;
  p.out = as_ptr<void>(out_ptr);
  p.ld_out = static_cast<int>(ld_out);
  p.out2 = as_ptr<void>(out2_ptr);
  p.q_out8 = as_ptr<uint8_t>(q_out8);
  p.q_sf = as_ptr<uint8_t>(q_sf);
  p.ld_q = static_cast<int>(ld_q);
  p.q_bn = static_cast<int16_t>(q_bn > 0 ? q_bn : 32);
  p.sumsq_out = as_ptr<float>(sumsq_out);
  p.zero_buf = as_ptr<float>(zero_buf);
  p.sumsq = as_ptr<const float>(sumsq);
  TORCH_CHECK(!p.q_out8 || (p.q_sf && p.sfa && p.ld_q % 128 == 0 && (epi == b2b::EPI_RESIDUAL || epi == b2b::EPI_GLU)),
              "fused output quantisation: MX GEMMs with residual / GLU epilogues, scale-factor buffer, row stride multiple of 128");
  p.residual = as_ptr<const __nv_bfloat16>(residual_ptr);
  p.ld_res = static_cast<int>(ld_res);
  p.bias = ptr_or_null<const float>(bias);
  p.rstd = ptr_or_null<const float>(rstd);
  TORCH_CHECK(!(fp8 && norm_from_x), "fp8 gemm: pass the combined activation scale through rstd");
  p.norm_src = norm_from_x ? reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()) : nullptr;
  p.eps = static_cast<float>(eps);
  p.q_out = ptr_or_null<__nv_bfloat16>(q_out);
  p.k_cache = ptr_or_null<__nv_bfloat16>(k_cache);
  p.v_cache = ptr_or_null<__nv_bfloat16>(v_cache);
  p.positions = ptr_or_null<const int>(positions);
  p.slots = ptr_or_null<const int>(slots);
  p.n_q_heads = static_cast<int16_t>(n_q_heads);
  p.n_kv_heads = static_cast<int16_t>(n_kv_heads);
  p.head_dim = static_cast<int16_t>(head_dim);
  p.rope_theta = static_cast<float>(rope_theta);
  p.q_scale = static_cast<float>(q_scale);
  p.wait_flag = as_ptr<const uint32_t>(wait_flag);
  p.wait_epoch = as_ptr<const uint32_t>(wait_epoch);
  p.signal_flag = as_ptr<uint32_t>(signal_flag);
  p.signal_epoch = as_ptr<uint32_t>(signal_epoch);
  p.done_counter = as_ptr<uint32_t>(done_counter);
  p.free_flag = as_ptr<const uint32_t>(free_flag);
  p.bump_epoch = as_ptr<uint32_t>(bump_epoch);
  p.ack_flag = as_ptr<uint32_t>(ack_flag);
  p.free_lag = static_cast<uint8_t>(free_lag);
  p.dbg = as_ptr<unsigned long long>(dbg);
  if (p.epi == b2b::EPI_QKV_ROPE) {
    TORCH_CHECK(p.q_out && p.k_cache && p.v_cache && p.slots, "qkv epilogue needs q_out/k_cache/v_cache/slots");
    TORCH_CHECK(p.rope_theta <= 0.f || p.positions, "rope needs positions");
    TORCH_CHECK((p.n_q_heads * p.head_dim) % 128 == 0 && (p.n_kv_heads * p.head_dim) % 128 == 0,
                "q/kv widths must be multiples of 128");
    TORCH_CHECK(p.n_out == (p.n_q_heads + 2 * p.n_kv_heads) * p.head_dim, "qkv rows mismatch");
  }
  if (p.epi == b2b::EPI_RESIDUAL) TORCH_CHECK(p.residual != nullptr, "residual epilogue needs residual");
  if (p.epi == b2b::EPI_GLU) TORCH_CHECK(p.out != nullptr || (p.q_out8 != nullptr && p.sfa != nullptr), "GLU epilogue needs an output");
  if (p.signal_flag || p.bump_epoch) TORCH_CHECK(p.done_counter != nullptr, "handoff needs done_counter");
  check(b2b::launch_gemm_tc(p, w.data_ptr(), x.data_ptr(), static_cast<int>(bn), cur_stream()), "gemm_tc");
}

// Bounded handoff waits (call once per device after peer_alloc'ing the abort word): limit_ms == 0 restores "trap".
void set_wait_policy(int64_t abort_word, double limit_ms) {
  const auto ns = static_cast<unsigned long long>(limit_ms * 1e6);
  check(b2b::set_wait_policy_gemm(as_ptr<uint32_t>(abort_word), ns), "set_wait_policy(gemm)");
  check(b2b::set_wait_policy_elementwise(as_ptr<uint32_t>(abort_word), ns), "set_wait_policy(elementwise)");
}

void set_pdl(bool on) { b2b::g_pdl_mode = on ? 1 : 0; }
bool get_pdl() { return b2b::pdl_enabled(); }

int64_t gemm_max_splitk(int64_t bn, int64_t epi, int64_t stages) {
  return b2b::gemm_tc_max_splitk(static_cast<int>(bn), static_cast<int>(epi), static_cast<int>(stages));
}

void init_kernels(int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  check(b2b::gemm_tc_init(), "gemm_tc_init");
  check(b2b::attention_init(), "attention_init");
}

// ----------------------------------------------------------------- elementwise
void rmsnorm(const Tensor& x, const Tensor& gamma, const OptT& residual, const OptT& out, const OptT& rstd_out,
             double eps, bool gemma_plus_one) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int h = static_cast<int>(x.size(-1));
  const int tokens = static_cast<int>(x.numel() / h);
  check(b2b::launch_rmsnorm(x.data_ptr(), gamma.data_ptr(), ptr_or_null<void>(residual), ptr_or_null<void>(out),
                            ptr_or_null<float>(rstd_out), tokens, h, static_cast<float>(eps), gemma_plus_one ? 1 : 0,
                            cur_stream()),
        "rmsnorm");
}

void layernorm(const Tensor& x, const Tensor& gamma, const Tensor& beta, const Tensor& out, double eps) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int h = static_cast<int>(x.size(-1));
  check(b2b::launch_layernorm(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                              static_cast<int>(x.numel() / h), h, static_cast<float>(eps), cur_stream()),
        "layernorm");
}

void embed(int64_t ids_ptr, const Tensor& table, const OptT& pos_table, const OptT& positions, const Tensor& out,
           double scale, int64_t tok_flag, int64_t tok_epoch, int64_t pf_flag, int64_t pf_need) {
  check_bf16(table, "table");
  c10::cuda::CUDAGuard guard(table.device());
  const int h = static_cast<int>(table.size(1));
  check(b2b::launch_embed(as_ptr<const int>(ids_ptr), table.data_ptr(), ptr_or_null<void>(pos_table),
                          ptr_or_null<const int>(positions), out.data_ptr(), static_cast<int>(out.numel() / h), h,
                          static_cast<int>(table.size(0)), static_cast<float>(scale), as_ptr<const uint32_t>(tok_flag),
                          as_ptr<const uint32_t>(tok_epoch), as_ptr<const uint32_t>(pf_flag), as_ptr<const uint32_t>(pf_need),
                          cur_stream()),
        "embed");
}

void kv_append(const Tensor& qkv, const Tensor& q_out, const Tensor& k_cache, const Tensor& v_cache,
               const Tensor& slots, int64_t q_dim, int64_t kv_dim, double q_scale) {
  check_bf16(qkv, "qkv");
  c10::cuda::CUDAGuard guard(qkv.device());
  check(b2b::launch_kv_append(qkv.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                              reinterpret_cast<const int*>(slots.data_ptr()), static_cast<int>(qkv.size(0)),
                              static_cast<int>(q_dim), static_cast<int>(kv_dim), static_cast<float>(q_scale),
                              cur_stream()),
        "kv_append");
}

void add(const Tensor& a, const Tensor& b, const Tensor& out) {
  check_bf16(a, "a");
  c10::cuda::CUDAGuard guard(a.device());
  check(b2b::launch_add(a.data_ptr(), b.data_ptr(), out.data_ptr(), static_cast<size_t>(a.numel()), cur_stream()),
        "add");
}

void quant_fp8_rows(const Tensor& x, const Tensor& q, const Tensor& scale_out, double eps, bool with_rms) {
  check_bf16(x, "x");
  TORCH_CHECK(q.scalar_type() == at::kFloat8_e4m3fn && q.is_contiguous() && scale_out.scalar_type() == at::kFloat,
              "quant_fp8_rows: q must be float8_e4m3fn, scale fp32");
  c10::cuda::CUDAGuard guard(x.device());
  const int h = static_cast<int>(x.size(-1));
  check(b2b::launch_quant_fp8_rows(x.data_ptr(), q.data_ptr(), reinterpret_cast<float*>(scale_out.data_ptr()),
                                   static_cast<int>(x.numel() / h), h, static_cast<float>(eps), with_rms ? 1 : 0,
                                   cur_stream()),
        "quant_fp8_rows");
}

void quant_mxfp8_rows(const Tensor& x, const Tensor& q, const Tensor& sf, int64_t bn, double eps, int64_t with_rms,
                      const OptT& sumsq_out) {
  check_bf16(x, "x");
  TORCH_CHECK(q.scalar_type() == at::kFloat8_e4m3fn && q.is_contiguous() && sf.scalar_type() == at::kByte &&
                  sf.is_contiguous(), "quant_mxfp8_rows: q must be float8_e4m3fn, sf uint8");
  c10::cuda::CUDAGuard guard(x.device());
  const int h = static_cast<int>(x.size(-1));
  const int tokens = static_cast<int>(x.numel() / h);
  TORCH_CHECK(sf.numel() >= ((tokens + bn - 1) / bn) * (h / 128) * (bn > 128 ? 1024 : 512), "quant_mxfp8_rows: sf too small");
  check(b2b::launch_quant_mxfp8_rows(x.data_ptr(), q.data_ptr(), sf.data_ptr(), tokens, h, static_cast<int>(bn),
                                     static_cast<float>(eps), static_cast<int>(with_rms), ptr_or_null<float>(sumsq_out),
                                     cur_stream()),
        "quant_mxfp8_rows");
}

void flag_wait(int64_t flag, int64_t epoch, int64_t delta) {
  check(b2b::launch_flag_wait(as_ptr<const uint32_t>(flag), as_ptr<const uint32_t>(epoch),
                              static_cast<uint32_t>(delta), cur_stream()),
        "flag_wait");
}
void decode_advance(const Tensor& positions, const Tensor& kv_len, const Tensor& slots, const Tensor& q_len,
                    const Tensor& block_table) {
  c10::cuda::CUDAGuard guard(positions.device());
  check(b2b::launch_decode_advance(reinterpret_cast<int*>(positions.data_ptr()), reinterpret_cast<int*>(kv_len.data_ptr()),
                                   reinterpret_cast<int*>(slots.data_ptr()),
                                   reinterpret_cast<const int*>(q_len.data_ptr()),
                                   reinterpret_cast<const int*>(block_table.data_ptr()),
                                   static_cast<int>(block_table.size(1)), static_cast<int>(positions.numel()),
                                   cur_stream()),
        "decode_advance");
}
void flag_signal(int64_t flag, int64_t epoch, int64_t bump_epoch, int64_t ack_flag) {
  check(b2b::launch_flag_signal(as_ptr<uint32_t>(flag), as_ptr<uint32_t>(epoch), as_ptr<uint32_t>(bump_epoch),
                                as_ptr<uint32_t>(ack_flag), cur_stream()),
        "flag_signal");
}

// -------------------------------------------------------------------- attention
// query-chunk length from which the tensor-core prefill kernel is used (0 = never); env B2B_ATTN_TC_MIN_Q
static int64_t g_attn_tc_min_q = [] {
  const char* e = std::getenv("B2B_ATTN_TC_MIN_Q");
  return e ? static_cast<int64_t>(std::atoi(e)) : static_cast<int64_t>(2);
}();
void set_attn_tc_min_q(int64_t v) { g_attn_tc_min_q = v; }
int64_t get_attn_tc_min_q() { return g_attn_tc_min_q; }

void attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& out,
               const Tensor& block_table, const Tensor& q_start, const Tensor& q_len, const Tensor& kv_len,
               const OptT& ws, int64_t max_q, int64_t n_q, int64_t n_kv, int64_t head_dim, int64_t window,
               double softcap, int64_t splits, int64_t use_tc, int64_t fq_out, int64_t fq_sf, int64_t fq_bn) {
  check_bf16(q, "q");
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(block_table.scalar_type() == at::kInt && q_len.scalar_type() == at::kInt, "int32 metadata expected");
  const int seqs = static_cast<int>(q_len.size(0));
  // use_tc: -1 = by query-chunk length (prefill chunks), 1 = force the tcgen05 kernel (decode: one-token query blocks,
  // the GQA group stacked into the MMA rows), 0 = force the CUDA-core kernel (split-KV decode of few sequences)
  const bool want_tc = use_tc < 0 ? (max_q >= g_attn_tc_min_q && g_attn_tc_min_q > 0) : (use_tc > 0 && g_attn_tc_min_q > 0);
  if (want_tc && splits > 1 && max_q == 1) {
    TORCH_CHECK(ws.has_value(), "split-KV needs a workspace");
    const int64_t R = b2b::attn_rows(static_cast<int>(n_q / n_kv), 1);
    TORCH_CHECK(ws->numel() >= seqs * n_kv * splits * R * (head_dim + 2), "attention workspace too small");
  }
  if (want_tc &&
      b2b::attention_tc_supported(static_cast<int>(n_q), static_cast<int>(n_kv), static_cast<int>(head_dim))) {
    // prefill chunk: tcgen05 flash attention
    check(b2b::launch_attention_tc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                   reinterpret_cast<const int*>(block_table.data_ptr()),
                                   reinterpret_cast<const int*>(q_start.data_ptr()),
                                   reinterpret_cast<const int*>(q_len.data_ptr()),
                                   reinterpret_cast<const int*>(kv_len.data_ptr()), seqs, static_cast<int>(max_q),
                                   static_cast<int>(block_table.size(1)), static_cast<int>(q.size(0)),
                                   static_cast<int>(k_cache.size(0)), static_cast<int>(n_q), static_cast<int>(n_kv),
                                   static_cast<int>(head_dim), static_cast<int>(window), static_cast<float>(softcap),
                                   static_cast<int>(splits), ptr_or_null<float>(ws), as_ptr<void>(fq_out), as_ptr<void>(fq_sf),
                                   static_cast<int>(fq_bn), cur_stream()),
          "attention_tc");
    return;
  }
  TORCH_CHECK(fq_out == 0, "fused output quantisation needs the tcgen05 attention kernel");
  if (splits > 1) {
    TORCH_CHECK(ws.has_value(), "split-KV needs a workspace");
    const int64_t R = b2b::attn_rows(static_cast<int>(n_q / n_kv), 1);
    TORCH_CHECK(ws->numel() >= seqs * n_kv * splits * R * (head_dim + 2), "attention workspace too small");
  }
  check(b2b::launch_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                              reinterpret_cast<const int*>(block_table.data_ptr()),
                              reinterpret_cast<const int*>(q_start.data_ptr()),
                              reinterpret_cast<const int*>(q_len.data_ptr()),
                              reinterpret_cast<const int*>(kv_len.data_ptr()), ptr_or_null<float>(ws), seqs,
                              static_cast<int>(max_q), static_cast<int>(block_table.size(1)), static_cast<int>(n_q),
                              static_cast<int>(n_kv), static_cast<int>(head_dim), static_cast<int>(window),
                              static_cast<float>(softcap), static_cast<int>(splits), cur_stream()),
        "attention");
}

// ---------------------------------------------------------------------- sampler
void sample(const Tensor& logits, const OptT& seen, const Tensor& out_tokens, int64_t peer_tokens,
            int64_t history, const OptT& hist_pos, int64_t hist_stride, int64_t vocab, double softcap,
            const OptT& temperature, const OptT& top_p,
            const OptT& rep_penalty, const OptT& seeds, const OptT& step, int64_t signal_flag, int64_t signal_epoch,
            int64_t done_counter, int64_t row_map) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.stride(1) == 1, "logits: fp32");
  c10::cuda::CUDAGuard guard(logits.device());
  int* hp = ptr_or_null<int>(hist_pos);
  check(b2b::launch_sample(reinterpret_cast<const float*>(logits.data_ptr()), ptr_or_null<uint32_t>(seen),
                           reinterpret_cast<int*>(out_tokens.data_ptr()), as_ptr<int>(peer_tokens),
                           as_ptr<int>(history), hp, hp, static_cast<int>(hist_stride),
                           static_cast<int>(logits.size(0)), static_cast<int>(vocab > 0 ? vocab : logits.size(1)),
                           static_cast<int>(logits.stride(0)), static_cast<float>(softcap),
                           ptr_or_null<const float>(temperature), ptr_or_null<const float>(top_p),
                           ptr_or_null<const float>(rep_penalty), ptr_or_null<const uint32_t>(seeds),
                           ptr_or_null<const uint32_t>(step), as_ptr<uint32_t>(signal_flag),
                           as_ptr<uint32_t>(signal_epoch), as_ptr<uint32_t>(done_counter), as_ptr<const int>(row_map),
                           cur_stream()),
        "sample");
}

void set_decode_state(const Tensor& positions, const Tensor& kv_len, const Tensor& q_len, int64_t row_map, int64_t kvlen,
                      int64_t n) {
  c10::cuda::CUDAGuard guard(positions.device());
  check(b2b::launch_set_decode_state(reinterpret_cast<int*>(positions.data_ptr()), reinterpret_cast<int*>(kv_len.data_ptr()),
                                     reinterpret_cast<int*>(q_len.data_ptr()), as_ptr<const int>(row_map),
                                     as_ptr<const int>(kvlen), static_cast<int>(n), cur_stream()),
        "set_decode_state");
}

// history / cursors / out / waits are raw addresses: the ring may be peer memory, the rest mapped pinned host memory
void fetch_window(int64_t history, int64_t hist_stride, int64_t cursors, int64_t rows, int64_t width, int64_t out,
                  int64_t waits, int64_t n_waits, int64_t status) {
  check(b2b::launch_fetch_window(as_ptr<const int>(history), static_cast<int>(hist_stride), as_ptr<const int>(cursors),
                                 static_cast<int>(rows), static_cast<int>(width), as_ptr<int>(out),
                                 as_ptr<const b2b::FlagWait>(waits), static_cast<int>(n_waits), as_ptr<int>(status),
                                 cur_stream()),
        "fetch_window");
}

void mark_seen(const Tensor& ids, const Tensor& seq_of, const Tensor& seen, int64_t vocab) {
  c10::cuda::CUDAGuard guard(ids.device());
  check(b2b::launch_mark_seen(reinterpret_cast<const int*>(ids.data_ptr()),
                              reinterpret_cast<const int*>(seq_of.data_ptr()),
                              reinterpret_cast<uint32_t*>(seen.data_ptr()), static_cast<int>(ids.numel()),
                              static_cast<int>(vocab), cur_stream()),
        "mark_seen");
}

// ------------------------------------------------------------------ peer memory
int64_t peer_alloc(int64_t bytes) {
  void* p = nullptr;
  check(b2b::peer_alloc(static_cast<size_t>(bytes), &p), "peer_alloc");
  return static_cast<int64_t>(reinterpret_cast<uintptr_t>(p));
}
void peer_free(int64_t p) { check(b2b::peer_free(as_ptr<void>(p)), "peer_free"); }
py::bytes ipc_export(int64_t p) {
  char h[64];
  check(b2b::ipc_export(as_ptr<void>(p), h), "cudaIpcGetMemHandle");
  return py::bytes(h, 64);
}
int64_t ipc_import(const std::string& handle) {
  TORCH_CHECK(handle.size() == 64, "IPC handle must be 64 bytes");
  void* p = nullptr;
  check(b2b::ipc_import(handle.data(), &p), "cudaIpcOpenMemHandle");
  return static_cast<int64_t>(reinterpret_cast<uintptr_t>(p));
}
void ipc_close(int64_t p) { check(b2b::ipc_close(as_ptr<void>(p)), "cudaIpcCloseMemHandle"); }
void enable_peer_access(int64_t dev, int64_t peer) {
  check(b2b::enable_peer_access(static_cast<int>(dev), static_cast<int>(peer)), "cudaDeviceEnablePeerAccess");
}
bool can_access_peer(int64_t dev, int64_t peer) {
  return b2b::can_access_peer(static_cast<int>(dev), static_cast<int>(peer)) != 0;
}
void memcpy_peer(int64_t dst, int64_t dst_dev, int64_t src, int64_t src_dev, int64_t bytes) {
  check(b2b::memcpy_peer_async(as_ptr<void>(dst), static_cast<int>(dst_dev), as_ptr<const void>(src),
                               static_cast<int>(src_dev), static_cast<size_t>(bytes), cur_stream()),
        "cudaMemcpyPeerAsync");
}
std::pair<int64_t, int64_t> host_ring_alloc(int64_t bytes) {
  void *h = nullptr, *d = nullptr;
  check(b2b::host_ring_alloc(static_cast<size_t>(bytes), &h, &d), "cudaHostAlloc");
  return {static_cast<int64_t>(reinterpret_cast<uintptr_t>(h)), static_cast<int64_t>(reinterpret_cast<uintptr_t>(d))};
}
void host_ring_free(int64_t h) { check(b2b::host_ring_free(as_ptr<void>(h)), "cudaFreeHost"); }

// View raw (possibly peer-mapped or host-mapped) memory as a tensor; no ownership.
Tensor tensor_from_ptr(int64_t p, std::vector<int64_t> sizes, const std::string& dtype, int64_t device) {
  at::ScalarType st = dtype == "bf16" ? at::kBFloat16 : dtype == "f32" ? at::kFloat : dtype == "i32" ? at::kInt
                      : dtype == "u8" ? at::kByte : at::kLong;
  auto opts = at::TensorOptions().dtype(st);
  opts = device >= 0 ? opts.device(at::kCUDA, static_cast<c10::DeviceIndex>(device)) : opts.device(at::kCPU);
  return at::from_blob(as_ptr<void>(p), sizes, opts);
}

}  // namespace

// ------------------------------------------------------------------ hybrid graphs (streams, sigmoid attention, delta rule)
namespace {
inline const int* ip(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kInt, "expected an int32 tensor");
  return reinterpret_cast<const int*>(t.data_ptr());
}
inline const float* fp(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kFloat, "expected a float32 tensor");
  return reinterpret_cast<const float*>(t.data_ptr());
}
inline const float* fp_or_null(const OptT& t) { return (t.has_value() && t->defined()) ? fp(*t) : nullptr; }
inline int is_f32(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16, "expected float32 or bfloat16");
  return t.scalar_type() == at::kFloat ? 1 : 0;
}

void hyb_embed(const Tensor& ids, const Tensor& positions, const Tensor& q_start, const Tensor& q_len,
               const Tensor& seq_slot, const Tensor& prev_tok, const Tensor& table, const OptT& pair, int64_t buckets,
               int64_t mul_prev, int64_t mul_cur, double scale, const Tensor& streams, int64_t n_seqs, int64_t max_q) {
  c10::cuda::CUDAGuard guard(table.device());
  const bool has_pair = pair.has_value() && pair->defined();
  TORCH_CHECK(!has_pair || pair->scalar_type() == table.scalar_type(), "pair table dtype");
  check(b2b::launch_hyb_embed(ip(ids), ip(positions), ip(q_start), ip(q_len), ip(seq_slot), ip(prev_tok), table.data_ptr(),
                              has_pair ? pair->data_ptr() : nullptr, static_cast<int>(buckets), mul_prev, mul_cur,
                              static_cast<float>(scale), const_cast<float*>(fp(streams)), static_cast<int>(streams.size(1)),
                              static_cast<int>(streams.size(2)), static_cast<int>(table.size(0)), static_cast<int>(n_seqs),
                              static_cast<int>(max_q), is_f32(table), cur_stream()),
        "hyb_embed");
}

void hyb_commit_prev(const Tensor& ids, const Tensor& q_start, const Tensor& q_len, const Tensor& seq_slot,
                     const Tensor& prev_tok, int64_t n_seqs) {
  c10::cuda::CUDAGuard guard(prev_tok.device());
  check(b2b::launch_hyb_commit_prev(ip(ids), ip(q_start), ip(q_len), ip(seq_slot), const_cast<int*>(ip(prev_tok)),
                                    static_cast<int>(n_seqs), cur_stream()),
        "hyb_commit_prev");
}

// streams [T, ns, W] fp32.  rows (optional): gathered mode, output row i <- token rows[i], streams are not written.
void hc_step(const Tensor& streams, const Tensor& q_start, const Tensor& q_len, const OptT& rows, int64_t n_rows,
             int64_t n_seqs, int64_t max_q, const OptT& y, const OptT& mix, const OptT& outw, double mult, const OptT& inw,
             const OptT& gamma, double eps, const OptT& h) {
  c10::cuda::CUDAGuard guard(streams.device());
  const bool has_h = h.has_value() && h->defined();
  const bool has_y = y.has_value() && y->defined();
  TORCH_CHECK(has_h == (gamma.has_value() && gamma->defined()), "hc_step: h and gamma come together");
  check(b2b::launch_hc_step(const_cast<float*>(fp(streams)), ip(q_start), ip(q_len),
                            (rows.has_value() && rows->defined()) ? ip(*rows) : nullptr, static_cast<int>(n_rows),
                            static_cast<int>(n_seqs), static_cast<int>(max_q), fp_or_null(y),
                            has_y ? static_cast<int>(y->stride(0)) : 0, fp_or_null(mix), fp_or_null(outw),
                            static_cast<float>(mult), fp_or_null(inw), fp_or_null(gamma), static_cast<float>(eps),
                            has_h ? h->data_ptr() : nullptr, has_h ? static_cast<int>(h->stride(0)) : 0,
                            static_cast<int>(streams.size(1)), static_cast<int>(streams.size(2)),
                            has_h ? is_f32(*h) : 1, cur_stream()),
        "hc_step");
}

void act_cols(const Tensor& in, int64_t off, const Tensor& out, int64_t n, int64_t act, int64_t T, double p0, double p1) {
  c10::cuda::CUDAGuard guard(in.device());
  check(b2b::launch_act_cols(fp(in), static_cast<int>(in.stride(0)), static_cast<int>(off), out.data_ptr(),
                             static_cast<int>(out.stride(0)), static_cast<int>(n), static_cast<int>(act),
                             static_cast<float>(p0), static_cast<float>(p1), static_cast<int>(T), is_f32(out),
                             cur_stream()),
        "act_cols");
}

void attn_prep(const Tensor& proj, const Tensor& qn, const Tensor& kn, const Tensor& slots, const Tensor& q_out,
               const Tensor& k_cache, const Tensor& v_cache, int64_t T, int64_t H, int64_t G, int64_t D, int64_t V,
               double eps) {
  c10::cuda::CUDAGuard guard(proj.device());
  TORCH_CHECK(k_cache.scalar_type() == v_cache.scalar_type(), "cache dtypes");
  check(b2b::launch_attn_prep(fp(proj), static_cast<int>(proj.stride(0)), fp(qn), fp(kn), ip(slots),
                              const_cast<float*>(fp(q_out)), k_cache.data_ptr(), v_cache.data_ptr(), static_cast<int>(T),
                              static_cast<int>(H), static_cast<int>(G), static_cast<int>(D), static_cast<int>(V),
                              static_cast<float>(eps), is_f32(k_cache), cur_stream()),
        "attn_prep");
}

void sig_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& gate, int64_t gate_off,
                   const Tensor& pb, const Tensor& out, const Tensor& block_table, const Tensor& q_start,
                   const Tensor& q_len, const Tensor& kv_len, int64_t n_seqs, int64_t max_q, int64_t H, int64_t G,
                   int64_t D, int64_t V, int64_t chunk, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(k_cache.scalar_type() == out.scalar_type() && v_cache.scalar_type() == out.scalar_type(),
              "sig_attention: cache and output dtypes must match");
  check(b2b::launch_sig_attention(fp(q), k_cache.data_ptr(), v_cache.data_ptr(), fp(gate),
                                  static_cast<int>(gate.stride(0)), static_cast<int>(gate_off), fp(pb), out.data_ptr(),
                                  static_cast<int>(out.stride(0)), ip(block_table),
                                  static_cast<int>(block_table.stride(0)), ip(q_start), ip(q_len), ip(kv_len),
                                  static_cast<int>(n_seqs), static_cast<int>(max_q), static_cast<int>(H),
                                  static_cast<int>(G), static_cast<int>(D), static_cast<int>(V), static_cast<int>(chunk),
                                  static_cast<float>(scale), is_f32(out), cur_stream()),
        "sig_attention");
}

void delta_scan(const Tensor& proj, int64_t off_r, int64_t off_k, int64_t off_v, int64_t off_a, const Tensor& lora,
                const Tensor& w0, const Tensor& a_bias, const Tensor& state, const Tensor& out, const Tensor& q_start,
                const Tensor& q_len, const Tensor& kv_len, const Tensor& seq_slot, int64_t n_seqs, int64_t max_q, int64_t H,
                int64_t dk, int64_t dv) {
  c10::cuda::CUDAGuard guard(proj.device());
  check(b2b::launch_delta_scan(fp(proj), static_cast<int>(proj.stride(0)), static_cast<int>(off_r),
                               static_cast<int>(off_k), static_cast<int>(off_v), static_cast<int>(off_a), fp(lora),
                               static_cast<int>(lora.stride(0)), fp(w0), fp(a_bias), const_cast<float*>(fp(state)),
                               const_cast<float*>(fp(out)), static_cast<int>(out.stride(0)), ip(q_start), ip(q_len),
                               ip(kv_len), ip(seq_slot), static_cast<int>(n_seqs), static_cast<int>(max_q),
                               static_cast<int>(H), static_cast<int>(dk), static_cast<int>(dv), cur_stream()),
        "delta_scan");
}

void delta_post(const Tensor& o, const Tensor& gate, int64_t off_g, const Tensor& weight, const Tensor& out, int64_t T,
                int64_t H, int64_t dv, double eps) {
  c10::cuda::CUDAGuard guard(o.device());
  check(b2b::launch_delta_post(fp(o), static_cast<int>(o.stride(0)), fp(gate), static_cast<int>(gate.stride(0)),
                               static_cast<int>(off_g), fp(weight), out.data_ptr(), static_cast<int>(out.stride(0)),
                               static_cast<int>(T), static_cast<int>(H), static_cast<int>(dv), static_cast<float>(eps),
                               is_f32(out), cur_stream()),
        "delta_post");
}

// ---- one residual stream with layer scale, softmax attention with distinct key / value widths, linear recurrences
// x [T, W] fp32.  Up to three terms (y, w, norm) join the residual; h (optional) receives the normed operand rows.
void ls_join(const Tensor& x, const Tensor& q_start, const Tensor& q_len, const OptT& rows, int64_t n_rows, int64_t n_seqs,
             int64_t max_q, const OptT& y0, const OptT& w0, int64_t norm0, const OptT& y1, const OptT& w1, int64_t norm1,
             const OptT& y2, const OptT& w2, int64_t norm2, double eps, const OptT& gamma, int64_t plus_one,
             const OptT& h, const OptT& gamma2, const OptT& h2, int64_t replace) {
  c10::cuda::CUDAGuard guard(x.device());
  const bool has_h = h.has_value() && h->defined();
  const bool has_g = gamma.has_value() && gamma->defined();
  const bool has_h2 = h2.has_value() && h2->defined();
  TORCH_CHECK(has_h || !has_g, "ls_join: a norm weight needs an operand to write");
  TORCH_CHECK(!has_h2 || (has_h && has_g && gamma2.has_value() && gamma2->defined() && gamma2->numel() == x.size(-1) &&
                          h2->scalar_type() == h->scalar_type()),
              "ls_join: the second operand needs the first one and a weight vector of its own");
  auto ld = [](const OptT& t) { return (t.has_value() && t->defined()) ? static_cast<int>(t->stride(0)) : 0; };
  const int W = static_cast<int>(x.size(-1));
  check(b2b::launch_ls_join(const_cast<float*>(fp(x)), ip(q_start), ip(q_len),
                            (rows.has_value() && rows->defined()) ? ip(*rows) : nullptr, static_cast<int>(n_rows),
                            static_cast<int>(n_seqs), static_cast<int>(max_q), fp_or_null(y0), ld(y0), fp_or_null(w0),
                            static_cast<int>(norm0), fp_or_null(y1), ld(y1), fp_or_null(w1), static_cast<int>(norm1),
                            fp_or_null(y2), ld(y2), fp_or_null(w2), static_cast<int>(norm2), static_cast<float>(eps),
                            fp_or_null(gamma), (has_g && gamma->numel() > 1) ? 1 : 0, static_cast<int>(plus_one),
                            has_h ? h->data_ptr() : nullptr, has_h ? static_cast<int>(h->stride(0)) : 0, W,
                            has_h ? is_f32(*h) : 1, has_h2 ? fp(*gamma2) : nullptr, has_h2 ? h2->data_ptr() : nullptr,
                            has_h2 ? static_cast<int>(h2->stride(0)) : 0, static_cast<int>(replace), cur_stream()),
        "ls_join");
}

void rot_attn_prep(const Tensor& proj, int64_t off_q, int64_t off_k, int64_t off_v, const Tensor& qn, const Tensor& kn,
                   const Tensor& freq, int64_t rdims, double amp, const Tensor& positions, const Tensor& slots,
                   const Tensor& q_out, const Tensor& k_cache, const Tensor& v_cache, int64_t T, int64_t H, int64_t G,
                   int64_t D, int64_t V, double eps) {
  c10::cuda::CUDAGuard guard(proj.device());
  TORCH_CHECK(k_cache.scalar_type() == v_cache.scalar_type(), "cache dtypes");
  TORCH_CHECK(rdims == 0 || freq.numel() >= rdims / 2, "rot_attn_prep: frequency table too short");
  check(b2b::launch_rot_attn_prep(fp(proj), static_cast<int>(proj.stride(0)), static_cast<int>(off_q),
                                  static_cast<int>(off_k), static_cast<int>(off_v), fp(qn), fp(kn), fp(freq),
                                  static_cast<int>(rdims), static_cast<float>(amp), ip(positions), ip(slots),
                                  const_cast<float*>(fp(q_out)), k_cache.data_ptr(), v_cache.data_ptr(),
                                  static_cast<int>(T), static_cast<int>(H), static_cast<int>(G), static_cast<int>(D),
                                  static_cast<int>(V), static_cast<float>(eps), is_f32(k_cache), cur_stream()),
        "rot_attn_prep");
}

void softmax_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& out,
                       const Tensor& block_table, const Tensor& q_start, const Tensor& q_len, const Tensor& kv_len,
                       int64_t n_seqs, int64_t max_q, int64_t H, int64_t G, int64_t D, int64_t V, int64_t window,
                       double scale, double softcap, int64_t keep_first, const OptT& sink) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(!(sink.has_value() && sink->defined()) || sink->numel() >= H, "softmax_attention: one sink per head");
  TORCH_CHECK(k_cache.scalar_type() == out.scalar_type() && v_cache.scalar_type() == out.scalar_type(),
              "softmax_attention: cache and output dtypes must match");
  check(b2b::launch_softmax_attention(fp(q), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                      static_cast<int>(out.stride(0)), ip(block_table),
                                      static_cast<int>(block_table.stride(0)), ip(q_start), ip(q_len), ip(kv_len),
                                      static_cast<int>(n_seqs), static_cast<int>(max_q), static_cast<int>(H),
                                      static_cast<int>(G), static_cast<int>(D), static_cast<int>(V),
                                      static_cast<int>(window), static_cast<float>(scale),
                                      static_cast<int>(v_cache.stride(1)), is_f32(out), static_cast<float>(softcap),
                                      static_cast<int>(keep_first), fp_or_null(sink), cur_stream()),
        "softmax_attention");
}

void short_conv(const Tensor& x, int64_t off, const Tensor& w, const Tensor& tail, const Tensor& y, const Tensor& q_start,
                const Tensor& q_len, const Tensor& kv_len, const Tensor& seq_slot, int64_t n_seqs, int64_t max_q) {
  c10::cuda::CUDAGuard guard(x.device());
  check(b2b::launch_short_conv(fp(x), static_cast<int>(x.stride(0)), static_cast<int>(off), fp(w),
                               const_cast<float*>(fp(tail)), const_cast<float*>(fp(y)), static_cast<int>(y.stride(0)),
                               ip(q_start), ip(q_len), ip(kv_len), ip(seq_slot), static_cast<int>(n_seqs),
                               static_cast<int>(max_q), static_cast<int>(w.size(0)), static_cast<int>(w.size(1)),
                               cur_stream()),
        "short_conv");
}

void mlstm_gates(const Tensor& proj, int64_t off_q, int64_t off_k, int64_t off_i, int64_t off_f, const Tensor& bi,
                 const Tensor& bf, double cap, double qscale, const Tensor& nstate, const Tensor& mstate,
                 const Tensor& aux, const Tensor& q_start, const Tensor& q_len, const Tensor& kv_len,
                 const Tensor& seq_slot, int64_t n_seqs, int64_t H, int64_t dk) {
  c10::cuda::CUDAGuard guard(proj.device());
  check(b2b::launch_mlstm_gates(fp(proj), static_cast<int>(proj.stride(0)), static_cast<int>(off_q),
                                static_cast<int>(off_k), static_cast<int>(off_i), static_cast<int>(off_f), fp(bi), fp(bf),
                                static_cast<float>(cap), static_cast<float>(qscale), const_cast<float*>(fp(nstate)),
                                const_cast<float*>(fp(mstate)), const_cast<float*>(fp(aux)), ip(q_start), ip(q_len),
                                ip(kv_len), ip(seq_slot), static_cast<int>(n_seqs), static_cast<int>(H),
                                static_cast<int>(dk), cur_stream()),
        "mlstm_gates");
}

void lin_scan(int64_t mode, const Tensor& qk, int64_t off_q, int64_t off_k, const Tensor& v, int64_t off_v, const OptT& z,
              int64_t off_z, const OptT& zbias, const OptT& hparam, const OptT& beta, int64_t off_b, const OptT& aux,
              double qscale, double inv_tau, const Tensor& state, const Tensor& out, const Tensor& q_start,
              const Tensor& q_len, const Tensor& kv_len, const Tensor& seq_slot, int64_t n_seqs, int64_t max_q, int64_t H,
              int64_t G, int64_t dk, int64_t dv) {
  c10::cuda::CUDAGuard guard(qk.device());
  auto ld = [](const OptT& t) { return (t.has_value() && t->defined()) ? static_cast<int>(t->stride(0)) : 0; };
  TORCH_CHECK(mode == 2 ? fp_or_null(aux) != nullptr : (fp_or_null(z) != nullptr && fp_or_null(zbias) != nullptr),
              "lin_scan: missing gate inputs for this mode");
  TORCH_CHECK(mode != 1 || (fp_or_null(hparam) != nullptr && fp_or_null(beta) != nullptr), "lin_scan: delta rule inputs");
  check(b2b::launch_lin_scan(static_cast<int>(mode), fp(qk), static_cast<int>(qk.stride(0)), static_cast<int>(off_q),
                             static_cast<int>(off_k), fp(v), static_cast<int>(v.stride(0)), static_cast<int>(off_v),
                             fp_or_null(z), ld(z), static_cast<int>(off_z), fp_or_null(zbias), fp_or_null(hparam),
                             fp_or_null(beta), ld(beta), static_cast<int>(off_b), fp_or_null(aux),
                             static_cast<float>(qscale), static_cast<float>(inv_tau), const_cast<float*>(fp(state)),
                             const_cast<float*>(fp(out)), static_cast<int>(out.stride(0)), ip(q_start), ip(q_len),
                             ip(kv_len), ip(seq_slot), static_cast<int>(n_seqs), static_cast<int>(max_q),
                             static_cast<int>(H), static_cast<int>(G), static_cast<int>(dk), static_cast<int>(dv),
                             cur_stream()),
        "lin_scan");
}

void scan_post(const Tensor& o, const Tensor& gate, int64_t off_g, const Tensor& weight, int64_t act, const OptT& aux,
               const Tensor& out, int64_t T, int64_t H, int64_t dv, double eps) {
  c10::cuda::CUDAGuard guard(o.device());
  TORCH_CHECK(weight.numel() == dv || weight.numel() == H * dv, "scan_post: weight is [dv] or [H * dv]");
  check(b2b::launch_scan_post(fp(o), static_cast<int>(o.stride(0)), fp(gate), static_cast<int>(gate.stride(0)),
                              static_cast<int>(off_g), fp(weight), (weight.numel() == dv && H > 1) ? 1 : 0,
                              static_cast<int>(act), fp_or_null(aux), out.data_ptr(), static_cast<int>(out.stride(0)),
                              static_cast<int>(T), static_cast<int>(H), static_cast<int>(dv), static_cast<float>(eps),
                              is_f32(out), cur_stream()),
        "scan_post");
}

// ---- post-norm layers, latent attention prep, router, gated columns (csrc/postnorm.cu)
void post_norm_join(const Tensor& x, const OptT& rows, int64_t n_rows, const OptT& y, const OptT& gate, int64_t off_g,
                    const OptT& gbias, const OptT& idw, double alpha, const Tensor& w, int64_t groups, double eps,
                    const Tensor& h) {
  c10::cuda::CUDAGuard guard(x.device());
  const bool has_gate = gate.has_value() && gate->defined();
  TORCH_CHECK(!has_gate || (gbias.has_value() && gbias->defined()), "post_norm_join: the gate comes with its bias");
  auto ld = [](const OptT& t) { return (t.has_value() && t->defined()) ? static_cast<int>(t->stride(0)) : 0; };
  check(b2b::launch_post_norm_join(const_cast<float*>(fp(x)), (rows.has_value() && rows->defined()) ? ip(*rows) : nullptr,
                                   static_cast<int>(n_rows), fp_or_null(y), ld(y), fp_or_null(gate), ld(gate),
                                   static_cast<int>(off_g), fp_or_null(gbias), fp_or_null(idw), static_cast<float>(alpha),
                                   fp(w), static_cast<int>(groups), static_cast<float>(eps), h.data_ptr(),
                                   static_cast<int>(h.stride(0)), static_cast<int>(x.size(-1)), is_f32(h), cur_stream()),
        "post_norm_join");
}

void latent_prep(const Tensor& proj, int64_t off_q, int64_t q_rank, int64_t off_kv, int64_t C, int64_t R, const Tensor& wq,
                 const Tensor& wc, const Tensor& freq, int64_t rdims, const Tensor& positions, const Tensor& slots,
                 const Tensor& cq, const Tensor& k_cache, double eps, int64_t T, double amp, const OptT& freq_lo) {
  c10::cuda::CUDAGuard guard(proj.device());
  TORCH_CHECK(cq.scalar_type() == k_cache.scalar_type(), "latent_prep: operand and cache dtypes must match");
  TORCH_CHECK(k_cache.size(-1) == R + C && k_cache.is_contiguous(), "latent_prep: cache rows are [rotary | latent]");
  TORCH_CHECK(rdims == 0 || freq.numel() >= rdims / 2, "latent_prep: frequency table too short");
  TORCH_CHECK(!(freq_lo.has_value() && freq_lo->defined()) || freq_lo->numel() >= rdims / 2, "latent_prep: low parts too short");
  check(b2b::launch_latent_prep(fp(proj), static_cast<int>(proj.stride(0)), static_cast<int>(off_q),
                                static_cast<int>(q_rank), static_cast<int>(off_kv), static_cast<int>(C),
                                static_cast<int>(R), fp(wq), fp(wc), fp(freq), static_cast<int>(rdims), ip(positions),
                                ip(slots), cq.data_ptr(), static_cast<int>(cq.stride(0)), k_cache.data_ptr(),
                                static_cast<float>(eps), static_cast<int>(T), is_f32(cq), static_cast<float>(amp),
                                fp_or_null(freq_lo), cur_stream()),
        "latent_prep");
}

void rot_heads(const Tensor& src, int64_t off, const Tensor& dst, int64_t H, int64_t Dh, const Tensor& freq, int64_t rdims,
               const Tensor& positions, const OptT& slots, int64_t T, int64_t roff, double amp, const OptT& freq_lo) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(rdims == 0 || freq.numel() >= rdims / 2, "rot_heads: frequency table too short");
  TORCH_CHECK(!(freq_lo.has_value() && freq_lo->defined()) || freq_lo->numel() >= rdims / 2, "rot_heads: low parts too short");
  TORCH_CHECK(dst.is_contiguous() && dst.size(-1) == H * Dh, "rot_heads: dense [T, H * Dh] output");
  check(b2b::launch_rot_heads(fp(src), static_cast<int>(src.stride(0)), static_cast<int>(off), const_cast<float*>(fp(dst)),
                              static_cast<int>(H), static_cast<int>(Dh), fp(freq), static_cast<int>(rdims), ip(positions),
                              (slots.has_value() && slots->defined()) ? ip(*slots) : nullptr, static_cast<int>(T),
                              static_cast<int>(roff), static_cast<float>(amp), fp_or_null(freq_lo), cur_stream()),
        "rot_heads");
}

void moe_route(const Tensor& proj, int64_t off, const OptT& corr, int64_t E, int64_t n_real, int64_t count, int64_t keep,
               int64_t top, double scale, const Tensor& wt, const Tensor& idw, const OptT& sel_idx, const OptT& sel_w,
               int64_t T) {
  c10::cuda::CUDAGuard guard(proj.device());
  const bool has_sel = sel_idx.has_value() && sel_idx->defined();
  TORCH_CHECK(!(corr.has_value() && corr->defined()) || corr->numel() == E, "moe_route: one correction per router output");
  check(b2b::launch_moe_route(fp(proj), static_cast<int>(proj.stride(0)), static_cast<int>(off), fp_or_null(corr),
                              static_cast<int>(E), static_cast<int>(n_real), static_cast<int>(count),
                              static_cast<int>(keep), static_cast<int>(top), static_cast<float>(scale),
                              const_cast<float*>(fp(wt)), static_cast<int>(wt.stride(0)), const_cast<float*>(fp(idw)),
                              has_sel ? const_cast<int*>(ip(*sel_idx)) : nullptr,
                              const_cast<float*>(fp_or_null(sel_w)), static_cast<int>(T), cur_stream()),
        "moe_route");
}

void gated_cols(const Tensor& in, int64_t off_a, int64_t off_b, const OptT& wt, int64_t per, const Tensor& out, int64_t n,
                int64_t act, int64_t T, int64_t both, int64_t lead) {
  c10::cuda::CUDAGuard guard(in.device());
  const bool has_wt = wt.has_value() && wt->defined();
  check(b2b::launch_gated_cols(fp(in), static_cast<int>(in.stride(0)), static_cast<int>(off_a), static_cast<int>(off_b),
                               fp_or_null(wt), has_wt ? static_cast<int>(wt->stride(0)) : 0,
                               static_cast<int>(per > 0 ? per : 1), out.data_ptr(), static_cast<int>(out.stride(0)),
                               static_cast<int>(n), static_cast<int>(act), static_cast<int>(T), is_f32(out),
                               static_cast<int>(both), static_cast<int>(lead), cur_stream()),
        "gated_cols");
}

// a [T, >= H * C] per-head latent rows, U [H, V, C]; out [T, >= H * V] = sigmoid(gate[:, off_g + h V + v]) * (U[h] a[t, h])
void head_up_gate(const Tensor& a, const Tensor& U, const OptT& gate, int64_t off_g, const Tensor& out, int64_t T, int64_t H,
                  int64_t V, int64_t C) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.scalar_type() == U.scalar_type() && a.scalar_type() == out.scalar_type(), "head_up_gate: operand dtypes must match");
  TORCH_CHECK(U.is_contiguous() && U.numel() == H * V * C, "head_up_gate: U is a dense [H, V, C]");
  TORCH_CHECK(a.size(-1) >= H * C && out.size(-1) >= H * V, "head_up_gate: rows too short");
  const bool has_g = gate.has_value() && gate->defined();
  check(b2b::launch_head_up_gate(a.data_ptr(), static_cast<int>(a.stride(0)), U.data_ptr(), fp_or_null(gate),
                                 has_g ? static_cast<int>(gate->stride(0)) : 0, static_cast<int>(off_g), out.data_ptr(),
                                 static_cast<int>(out.stride(0)), static_cast<int>(T), static_cast<int>(H),
                                 static_cast<int>(V), static_cast<int>(C), is_f32(out), cur_stream()),
        "head_up_gate");
}
}  // namespace


PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "bee2bee_b200 native sm_100a kernels + NVLink peer-memory runtime";
  m.def("gemm", &gemm);
  m.def("gemm_max_splitk", &gemm_max_splitk);
  m.def("init_kernels", &init_kernels);
  m.def("set_pdl", &set_pdl);
  m.def("get_pdl", &get_pdl);
  m.def("rmsnorm", &rmsnorm);
  m.def("layernorm", &layernorm);
  m.def("embed", &embed);
  m.def("kv_append", &kv_append);
  m.def("add", &add);
  m.def("quant_fp8_rows", &quant_fp8_rows);
  m.def("quant_mxfp8_rows", &quant_mxfp8_rows);
  m.def("flag_wait", &flag_wait);
  m.def("flag_signal", &flag_signal);
  m.def("decode_advance", &decode_advance);
  m.def("attention", &attention);
  m.def("set_attn_tc_min_q", &set_attn_tc_min_q);
  m.def("get_attn_tc_min_q", &get_attn_tc_min_q);
  m.def("sample", &sample);
  m.def("mark_seen", &mark_seen);
  m.def("set_decode_state", &set_decode_state);
  m.def("fetch_window", &fetch_window);
  m.def("set_wait_policy", &set_wait_policy);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_free", &peer_free);
  m.def("ipc_export", &ipc_export);
  m.def("ipc_import", &ipc_import);
  m.def("ipc_close", &ipc_close);
  m.def("enable_peer_access", &enable_peer_access);
  m.def("can_access_peer", &can_access_peer);
  m.def("memcpy_peer", &memcpy_peer);
  m.def("host_ring_alloc", &host_ring_alloc);
  m.def("host_ring_free", &host_ring_free);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("hyb_embed", &hyb_embed);
  m.def("hyb_commit_prev", &hyb_commit_prev);
  m.def("hc_step", &hc_step);
  m.def("act_cols", &act_cols);
  m.def("attn_prep", &attn_prep);
  m.def("sig_attention", &sig_attention);
  m.def("delta_scan", &delta_scan);
  m.def("delta_post", &delta_post);
  m.def("ls_join", &ls_join);
  m.def("rot_attn_prep", &rot_attn_prep);
  m.def("softmax_attention", &softmax_attention);
  m.def("short_conv", &short_conv);
  m.def("mlstm_gates", &mlstm_gates);
  m.def("lin_scan", &lin_scan);
  m.def("scan_post", &scan_post);
  m.def("post_norm_join", &post_norm_join);
  m.def("latent_prep", &latent_prep);
  m.def("rot_heads", &rot_heads);
  m.def("moe_route", &moe_route);
  m.def("gated_cols", &gated_cols);
  m.def("head_up_gate", &head_up_gate);
}
