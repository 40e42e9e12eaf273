// C launcher API of the hand-written sm_100a kernels (no torch dependency: every .cu
// compiles in seconds with plain nvcc; csrc/binding.cpp is the only torch-facing file).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace b2b {

// elementwise.cu
int launch_rmsnorm(const void* x, const void* gamma, const void* residual, void* out, float* rstd_out, int tokens,
                   int h, float eps, int gemma_plus_one, cudaStream_t s);
int launch_layernorm(const void* x, const void* gamma, const void* beta, void* out, int tokens, int h, float eps,
                     cudaStream_t s);
int launch_embed(const int* ids, const void* table, const void* pos_table, const int* positions, void* out, int tokens,
                 int h, int vocab, float scale, const uint32_t* tok_flag, const uint32_t* tok_epoch, const uint32_t* pf_flag,
                 const uint32_t* pf_need, cudaStream_t s);
int launch_kv_append(const void* qkv, void* q_out, void* k_cache, void* v_cache, const int* slots, int tokens,
                     int q_dim, int kv_dim, float q_scale, cudaStream_t s);
int launch_add(const void* a, const void* b, void* out, size_t n, cudaStream_t s);
int launch_quant_fp8_rows(const void* x, void* q, float* scale_out, int tokens, int h, float eps, int with_rms,
                          cudaStream_t s);
int launch_quant_mxfp8_rows(const void* x, void* q, void* sf, int tokens, int h, int bn, float eps, int with_rms,
                            float* sumsq_out, cudaStream_t s);
int launch_flag_wait(const uint32_t* flag, const uint32_t* epoch, uint32_t delta, cudaStream_t s);
int launch_decode_advance(int* positions, int* kv_len, int* slots, const int* q_len, const int* block_table,
                          int max_pages, int n, cudaStream_t s);
int launch_flag_signal(uint32_t* flag, uint32_t* epoch, uint32_t* bump_epoch, uint32_t* ack_flag, cudaStream_t s);

// attention.cu
int launch_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                     const int* q_start, const int* q_len, const int* kv_len, float* ws, int seqs, int max_q,
                     int max_pages, int n_q, int n_kv, int head_dim, int window, float softcap, int splits,
                     cudaStream_t s);
int attn_rows(int G, int QB);
// attention_tc.cu: tcgen05 flash-attention forward for prefill chunks
bool attention_tc_supported(int n_q, int n_kv, int head_dim);
int launch_attention_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                        const int* q_start, const int* q_len, const int* kv_len, int seqs, int max_q, int max_pages,
                        int n_tokens, int n_pages, int n_q, int n_kv, int head_dim, int window, float softcap,
                        int splits, float* ws, void* q_out8, void* q_sf, int q_bn, cudaStream_t s);
// merge pass of split-KV decode (shared by the CUDA-core and the tcgen05 kernels)
int launch_attention_merge(void* out, const int* q_start, const float* ws, int seqs, int n_q, int n_kv, int head_dim,
                           int splits, cudaStream_t s);
int attention_init();

// sampler.cu
int launch_sample(const float* logits, uint32_t* seen, int* out_tokens, int* peer_tokens, int* history,
                  const int* hist_pos, int* hist_pos_out, int hist_stride, int batch, int vocab, int ld, float softcap,
                  const float* temperature, const float* top_p, const float* rep_penalty, const uint32_t* seeds,
                  const uint32_t* step, uint32_t* signal_flag, uint32_t* signal_epoch, uint32_t* done_counter,
                  const int* row_map, cudaStream_t s);
int launch_set_decode_state(int* positions, int* kv_len, int* q_len, const int* row_map, const int* kvlen, int n,
                            cudaStream_t s);
// token-window read-back: wait for up to `n_waits` (flag, target) pairs, then out[b, j] = history[b, (cursor[b] + j) % stride]
struct FlagWait { const uint32_t* flag; uint32_t target; uint32_t pad; };
int launch_fetch_window(const int* history, int hist_stride, const int* cursors, int rows, int width, int* out,
                        const FlagWait* waits, int n_waits, int* status, cudaStream_t s);
int launch_mark_seen(const int* ids, const int* seq_of, uint32_t* seen, int n, int vocab, cudaStream_t s);

// hybrid.cu: residual streams with hyper-connections, hashed token-pair embedding, sigmoid attention inside position
// blocks over the paged cache, generalized delta-rule recurrence (fp32 state per sequence slot).  f32 != 0: operands of
// matrix products and caches are float instead of bf16.
int launch_hyb_embed(const int* ids, const int* positions, const int* q_start, const int* q_len, const int* seq_slot,
                     const int* prev_tok, const void* table, const void* pair, int buckets, long long mul_prev,
                     long long mul_cur, float scale, float* streams, int ns, int W, int vocab, int n_seqs, int max_q,
                     int f32, cudaStream_t s);
int launch_hyb_commit_prev(const int* ids, const int* q_start, const int* q_len, const int* seq_slot, int* prev_tok,
                           int n_seqs, cudaStream_t s);
int launch_hc_step(float* streams, const int* q_start, const int* q_len, const int* rows, int n_rows, int n_seqs,
                   int max_q, const float* y, int ld_y, const float* mix, const float* outw, float mult,
                   const float* inw, const float* gamma, float eps, void* h, int ld_h, int ns, int W, int f32,
                   cudaStream_t s);
int launch_act_cols(const float* in, int ld_in, int off, void* out, int ld_out, int n, int act, float p0, float p1, int T,
                    int f32, cudaStream_t s);
int launch_attn_prep(const float* proj, int ld, const float* qn, const float* kn, const int* slots, float* q_out,
                     void* k_cache, void* v_cache, int T, int H, int G, int D, int V, float eps, int f32,
                     cudaStream_t s);
int launch_sig_attention(const float* q, const void* k_cache, const void* v_cache, const float* gate, int ld_gate,
                         int gate_off, const float* pb, void* out, int ld_out, const int* block_table, int max_pages,
                         const int* q_start, const int* q_len, const int* kv_len, int n_seqs, int max_q, int H, int G,
                         int D, int V, int chunk, float scale, int f32, cudaStream_t s);
int launch_delta_scan(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lora, int ld_l,
                      const float* w0, const float* a_bias, float* state, float* out, int ld_out, const int* q_start,
                      const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int max_q, int H, int dk, int dv,
                      cudaStream_t s);
int launch_delta_post(const float* o, int ld_o, const float* gate, int ld_g, int off_g, const float* weight, void* out,
                      int ld_out, int T, int H, int dv, float eps, int f32, cudaStream_t s);

// seqmix.cu: one residual stream with layer scale (parallel blocks), softmax attention with a norm over the whole q / k
// projection, rotary positions from a frequency table and key width != value width over the paged cache, short causal
// convolutions with a per-slot tail, gated linear recurrences (diag-gated linear attention, delta rule with a decay per
// key channel, mLSTM matrix memory) with an fp32 state per sequence slot.  f32 as above.
int launch_ls_join(float* x, const int* q_start, const int* q_len, const int* rows, int n_rows, int n_seqs, int max_q,
                   const float* y0, int ld0, const float* w0, int norm0, const float* y1, int ld1, const float* w1,
                   int norm1, const float* y2, int ld2, const float* w2, int norm2, float eps, const float* gamma,
                   int gstride, int plus_one, void* h, int ld_h, int W, int f32, const float* gamma2, void* h2, int ld_h2,
                   int replace, cudaStream_t s);
int launch_rot_attn_prep(const float* proj, int ld, int off_q, int off_k, int off_v, const float* qn, const float* kn,
                         const float* freq, int rdims, float amp, const int* positions, const int* slots, float* q_out,
                         void* k_cache, void* v_cache, int T, int H, int G, int D, int V, float eps, int f32,
                         cudaStream_t s);
int launch_softmax_attention(const float* q, const void* k_cache, const void* v_cache, void* out, int ld_out,
                             const int* block_table, int max_pages, const int* q_start, const int* q_len,
                             const int* kv_len, int n_seqs, int max_q, int H, int G, int D, int V, int window,
                             float scale, int ldv, int f32, float softcap, int keep_first, const float* sink,
                             cudaStream_t s);
int launch_short_conv(const float* x, int ld_x, int off, const float* w, float* tail, float* y, int ld_y,
                      const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs,
                      int max_q, int C, int taps, cudaStream_t s);
int launch_mlstm_gates(const float* proj, int ld, int off_q, int off_k, int off_i, int off_f, const float* bi,
                       const float* bf_, float cap, float qscale, float* nstate, float* mstate, float* aux,
                       const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs, int H,
                       int dk, cudaStream_t s);
// mode: 0 diag-gated linear attention, 1 delta rule with channel decay, 2 mLSTM matrix memory, 3 HGRN2 (forget gate with a
// lower bound, its complement is the write strength; hparam = the bound [H * dk], z = the gate projection, no keys)
int launch_lin_scan(int mode, const float* qk, int ld_qk, int off_q, int off_k, const float* v, int ld_v, int off_v,
                    const float* z, int ld_z, int off_z, const float* zbias, const float* hparam, const float* beta,
                    int ld_b, int off_b, const float* aux, float qscale, float inv_tau, float* state, float* out,
                    int ld_out, const int* q_start, const int* q_len, const int* kv_len, const int* seq_slot, int n_seqs,
                    int max_q, int H, int G, int dk, int dv, cudaStream_t s);
int launch_scan_post(const float* o, int ld_o, const float* gate, int ld_g, int off_g, const float* weight, int wshared,
                     int act, const float* aux, void* out, int ld_out, int T, int H, int dv, float eps, int f32,
                     cudaStream_t s);

// postnorm.cu: post-norm layers (grouped RMS norm behind the residual addition, scaled skip, sigmoid-gated sublayer results), latent
// attention prep (normed query latent; cache row = [rotated shared key part | normed latent]), rotary positions on the first
// channels of every head (-> dense query rows), softmax router (selection-only correction, group-limited top-k, identity experts),
// act(a) * b over column blocks or per-expert weights.  freq_lo (optional): low parts of the rotary frequencies (frequency =
// freq + freq_lo in double-float form), so that angles at far positions keep their last bits.  ldv of launch_softmax_attention: row stride of the value view
// (0 = a cache of its own) so that values can be a slice of the key rows.
int launch_post_norm_join(float* x, const int* rows, int n_rows, const float* y, int ld_y, const float* gate, int ld_g,
                          int off_g, const float* gbias, const float* idw, float alpha, const float* w, int groups,
                          float eps, void* h, int ld_h, int W, int f32, cudaStream_t s);
int launch_latent_prep(const float* proj, int ld, int off_q, int q_rank, int off_kv, int C, int R, const float* wq,
                       const float* wc, const float* freq, int rdims, const int* positions, const int* slots, void* cq,
                       int ld_cq, void* k_cache, float eps, int T, int f32, float amp, const float* freq_lo,
                       cudaStream_t s);
int launch_rot_heads(const float* src, int ld, int off, float* dst, int H, int Dh, const float* freq, int rdims,
                     const int* positions, const int* slots, int T, int roff, float amp, const float* freq_lo,
                     cudaStream_t s);
int launch_moe_route(const float* proj, int ld, int off, const float* corr, int E, int n_real, int count, int keep,
                     int top, float scale, float* wt, int ld_wt, float* idw, int* sel_idx, float* sel_w, int T,
                     cudaStream_t s);
int launch_gated_cols(const float* in, int ld_in, int off_a, int off_b, const float* wt, int ld_wt, int per, void* out,
                      int ld_out, int n, int act, int T, int f32, int both, int lead, cudaStream_t s);
// out[t, h, :] = gate * U[h] a[t, h, :]: one [V, C] matrix per head (operands bf16, or float when f32), sigmoid gate from fp32 rows
int launch_head_up_gate(const void* a, int ld_a, const void* U, const float* gate, int ld_g, int off_g, void* out,
                        int ld_out, int T, int H, int V, int C, int f32, cudaStream_t s);

// bounded handoff waits: device abort word + time limit for the waits of each translation unit (0 / null = trap policy)
int set_wait_policy_gemm(uint32_t* abort_word, unsigned long long limit_ns);
int set_wait_policy_elementwise(uint32_t* abort_word, unsigned long long limit_ns);

// gemm_tc.cu
int gemm_tc_max_splitk(int bn, int epi, int stages);
int gemm_tc_init();

}  // namespace b2b
