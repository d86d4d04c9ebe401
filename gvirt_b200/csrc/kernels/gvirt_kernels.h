// C ABI of libgvirt_kernels.so — every hand-written sm_100a kernel launcher.
//
// Calling convention: integers are `long long`, scalars `float`, tensors raw device
// pointers (bf16 unless stated), `stream` a cudaStream_t. Return value 0 = launched,
// negative = GV_E* (see common.cuh); gv_last_error() describes the last CUDA failure.
// No launcher allocates or frees device memory; scratch buffers are arguments.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// ---- support
const char* gv_last_error();
int gv_abi_version();
// Turns programmatic dependent launch on (non-zero, default unless GVIRT_DISABLE_PDL is set) or off
// for every later launch of this library in the process.
int gv_set_pdl(long long on);
int gv_status_read(unsigned int* host_out, void* stream);  // synchronises `stream`
int gv_status_reset(void* stream);
void* gv_status_ptr();

// ---- GEMM (tcgen05 / TMEM / TMA):  out[M,N] = x[M,K] . w[N,K]^T (+ bias[N])
int gv_gemm_bf16(const void* x, const void* w, const void* bias, void* out, long long M,
                 long long N, long long K, long long ldx, long long ldw, long long ldo,
                 long long force_splitk, void* stream);
// Per-shape split-K override of the weight-major path (see tools/gemm_sweep.py).
int gv_gemm_set_splitk(long long N, long long K, long long bn, long long splitk);
// Gate/up GEMM with SwiGLU epilogue over block-interleaved weights (see gemm_bf16.cu).
int gv_gemm_bf16_swiglu(const void* x, const void* w, void* out, long long M, long long N, long long K,
                        long long ldx, long long ldw, long long ldo, long long force_splitk,
                        void* stream);

// ---- normalisation: kind 0 RMS, 1 LayerNorm, 2 L2
int gv_norm(long long kind, const void* x, void* residual, const void* w, const void* b, void* out,
            void* var_out, const void* var_in, float var_in_scale, long long rows, long long cols,
            long long cnt, long long ldx, long long ldr, long long ldo, float eps, void* stream);

// ---- RoPE (+bias, +qk-norm, +q scale) and paged KV write
int gv_rope_kvwrite(void* qkv, const void* bias, const void* q_norm_w, const void* k_norm_w,
                    const void* cos_sin, const void* positions, const void* slot_mapping,
                    void* k_cache, void* v_cache, void* q_out, long long tokens, long long nq,
                    long long nkv, long long hd, long long rot_dim, long long ld, float q_scale,
                    float eps, long long max_pos, long long num_slots, long long mrope_mode,
                    long long sec0, long long sec1, long long sec2, long long interleaved,
                    void* stream);

// ---- elementwise / layout
int gv_silu_and_mul(const void* x, void* out, long long rows, long long d, long long ldx,
                    long long ldo, const void* num, float clamp, long long interleaved, void* stream);
int gv_binary(long long mode, const void* a, const void* b, void* out, long long rows,
              long long cols, long long lda, long long ldb, long long ldo, float scale,
              void* stream);
int gv_cast(long long to_f32, const void* in, void* out, long long n, void* stream);
// In-place causal row softmax of x [rows, cols] bf16 (leading dimension ldx): row m over its
// first min(calc_len + m, cols) entries, zeros behind them. cols and ldx multiples of 8.
int gv_causal_softmax(void* x, long long rows, long long cols, long long ldx, long long calc_len,
                      void* stream);
int gv_embed(const void* ids, const void* table, void* out, long long tokens, long long hidden,
             long long vstart, long long vend, void* stream);
int gv_gather_rows(const void* src, const void* idx, void* out, long long n, long long cols,
                   long long lds, long long src_rows, void* stream);
int gv_transpose12(const void* in, void* out, long long B, long long S, long long C, void* stream);
int gv_pack_fields(void* const* fields, const long long* widths, long long nfields, void* packed,
                   long long npackets, long long pack, void* stream);

// ---- paged attention
int gv_paged_attention_decode(const void* q, const void* k_cache, const void* v_cache,
                              const void* block_tables, const void* seq_lens, void* out,
                              void* part_o, void* part_lse, long long batch, long long nq,
                              long long nkv, long long head_dim, long long block_size,
                              long long max_blocks, long long nsplit, float scale,
                              long long num_blocks, void* stream);
// tile / ring shape of the decode kernel: 0 = 32 tok x 2, 1 = 16 x 2, 2 = 16 x 3, 3 = 16 x 4, 4 = 32 x 3
void gv_set_decode_variant(long long v);
int gv_paged_attention_prefill(const void* q, const void* k_cache, const void* v_cache,
                               const void* block_tables, const void* q_start,
                               const void* cached_lens, void* out, long long batch,
                               long long max_q_len, long long nq, long long nkv,
                               long long head_dim, long long block_size, long long max_blocks,
                               float scale, long long num_blocks, void* stream);

// In-kernel split merge (one launch): `counters` = batch * nkv int32, zero before the first call.
int gv_paged_attention_decode_merged(const void* q, const void* k_cache, const void* v_cache,
                                     const void* block_tables, const void* seq_lens, void* out,
                                     void* part_o, void* part_lse, void* counters, long long batch,
                                     long long nq, long long nkv, long long head_dim,
                                     long long block_size, long long max_blocks, long long nsplit,
                                     float scale, long long num_blocks, void* stream);
// Softmax warp groups of that kernel: 1 = one thread per query row, 2 (default) = two per row.
void gv_set_prefill_tc_warpgroups(long long wg);
// tcgen05 / TMEM / TMA flash attention for head_dim 128 (attention_prefill_tc.cu).
int gv_paged_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache,
                                  const void* block_tables, const void* q_start,
                                  const void* cached_lens, void* out, long long total_tokens,
                                  long long batch, long long max_q_len, long long nq, long long nkv,
                                  long long head_dim, long long block_size, long long max_blocks,
                                  float scale, long long num_blocks, void* stream);

// ---- decode-step GEMMs with fused epilogues (gemm_decode.cu)
int gv_gemm_decode(const void* x, const void* w, const void* bias, void* out, long long M, long long N,
                   long long K, long long ldx, long long ldw, long long ldo, const void* ss_in,
                   long long ss_tiles, long long ss_ld, long long norm_h, float eps, long long swiglu,
                   long long force_splitk, void* stream);
// Weight of the GEMM that follows the next gv_gemm_decode* launch of this host thread (null clears).
int gv_gemm_decode_next(const void* w, long long N, long long K, long long ldw);
int gv_gemm_decode_residual(const void* x, const void* w, const void* bias, const void* residual,
                            void* x_out, void* ss_out, long long M, long long N, long long K,
                            long long ldx, long long ldw, long long ldo, long long ss_ld,
                            long long force_splitk, void* stream);
int gv_gemm_decode_rope(const void* x, const void* w, const void* bias, void* q_out, void* k_cache,
                        void* v_cache, const void* cos_sin, const void* positions, const void* slots,
                        const void* q_norm_w, const void* k_norm_w, long long M, long long K,
                        long long ldx, long long ldw, long long nq, long long nkv, float q_scale,
                        float qk_eps, long long max_pos, long long num_slots, const void* ss_in,
                        long long ss_tiles, long long ss_ld, long long norm_h, float eps,
                        long long force_splitk, void* stream);
int gv_gemm_allreduce_ss(const void* x, const void* w, const void* bias, const void* residual, void* out,
                         void* ss_out, long long ss_ld, long long M, long long N, long long K,
                         long long ldx, long long ldw, long long ldo, const void* peers,
                         long long recv_off, long long flags_off, void* state, long long rank,
                         long long R, long long m_cap, long long max_ctas, long long two_shot,
                         void* stream);

// ---- sampling
int gv_sample(const void* logits, long long is_f32, long long ld, long long batch, long long vocab,
              const void* temperature, const void* top_k, const void* top_p, long long seed,
              long long step, const void* step_ptr, long long index_offset, void* out_val,
              void* out_idx, void* stream);
int gv_sample_merge(const void* vals, const void* idx, long long ranks, long long batch,
                    void* tokens, void* stream);

// ---- MoE
int gv_router_topk(const void* logits, const void* bias, void* weights, void* ids, long long T,
                   long long E, long long K, long long mode, long long n_group,
                   long long topk_group, long long renorm, float route_scale, void* stream);
int gv_moe_permute(const void* x, const void* ids, void* counts, void* offsets, void* row_of,
                   void* xs, long long T, long long H, long long K, long long e_local,
                   long long e_start, long long rows_cap, void* stream);
// SwiGLU (+ fp8 quantisation) over the live rows of slot-addressed expert segments (see moe.cu).
int gv_moe_act_seg(const void* gu, void* act, void* q, void* scales, const void* seg_start,
                   const void* seg_end, long long G, long long d, long long ld_gu, long long lds,
                   float clamp, long long fp8, void* stream);
int gv_moe_unpermute(const void* ys, const void* weights, const void* row_of, void* out,
                     long long T, long long H, long long K, void* stream);
int gv_gemm_bf16_persistent(const void* x, const void* w, const void* bias, void* out, long long M,
                            long long N, long long K, long long ldx, long long ldw, long long ldo,
                            void* stream);
long long gv_set_sm_budget(long long sms);
long long gv_planned_sms();
int gv_gemm_persistent_tile(long long t, long long tilesM, long long tilesN, int* p0, int* q0);
int gv_grouped_gemm_bf16(const void* xs, const void* w, const void* offsets, void* out,
                         long long rows_cap, long long N, long long K, long long E, void* stream);

// ---- collectives over the symmetric heap (see collectives.cu, gemm_allreduce.cu)
int gv_collective(long long mode, long long is_f32, const void* x, void* out, long long n,
                  const void* peers, long long flags_off, long long stage_off,
                  long long stage_stride, void* state, long long rank, long long R, long long grid,
                  void* stream);
int gv_gemm_allreduce(const void* x, const void* w, const void* bias, const void* residual,
                      void* out, long long M, long long N, long long K, long long ldx,
                      long long ldw, long long ldo, const void* peers, long long recv_off,
                      long long flags_off, void* state, long long rank, long long R,
                      long long m_cap, long long max_ctas, long long two_shot, void* stream);

// ---- MLA (see mla.cu, bmm.cu)
int gv_mla_prepare(const void* a, const void* q_norm_w, const void* kv_norm_w, const void* cos_sin,
                   const void* positions, const void* slots, void* cache, void* qn, long long T,
                   long long ql, long long dc, long long dr, long long lda, long long ldq, float eps,
                   long long max_pos, long long num_slots, void* stream);
int gv_rope_interleaved(const void* q, const void* cos_sin, const void* positions, void* out,
                        long long T, long long heads, long long qstride, long long off, long long dr,
                        long long ostride, long long ooff, long long max_pos, void* stream);
int gv_mla_attention(const void* qf, const void* cache, const void* block_tables, const void* q_start,
                     const void* cached_lens, void* out, void* part_o, void* part_lse, long long T,
                     long long batch, long long heads, long long dc, long long dr,
                     long long block_size, long long max_blocks, long long nsplit, float scale,
                     long long num_blocks, const void* topk_idx, long long topk, void* stream);
// Decode-only absorbed MLA on tcgen05 (mla_tc.cu): heads % 128 == 0, dc 512, dr 64, block_size % 32 == 0.
int gv_mla_attention_tc(const void* qf, const void* cache, const void* block_tables, const void* seq_lens,
                        void* out, void* part_o, void* part_lse, long long batch, long long heads,
                        long long dc, long long dr, long long block_size, long long max_blocks,
                        long long nsplit, float scale, long long num_blocks, void* stream);
int gv_bmm_bf16(const void* x, const void* w, void* out, long long T, long long Hh, long long N,
                long long K, long long sx_t, long long sx_h, long long so_t, long long so_h,
                void* stream);

// ---- quantisation (quant.cu) and block-scaled fp8 GEMMs (gemm_fp8.cu)
int gv_quant_fp8_group128(const void* x, void* q, void* scales, long long T, long long K,
                          long long ldx, long long ldq, long long lds, const void* num, void* stream);
int gv_quant_i8_static(const void* x, const void* scale_recip, const void* offset, void* q,
                       long long rows, long long cols, void* stream);
int gv_quant_i8_dynamic(const void* x, void* q, void* scales, long long rows, long long cols,
                        const void* num, void* stream);
int gv_dequant_i32(const void* acc, const void* w_scale, const void* tok_scale, const void* bias,
                   void* out, long long rows, long long cols, void* stream);
// ---- W8A8 int8 GEMM with fused de-quantisation, int4 weight unpack (see gemm_i8.cu)
int gv_gemm_i8(const void* xq, const void* wq, const void* w_scale, const void* tok_scale,
               const void* bias, void* out, long long M, long long N, long long K, long long ldo,
               void* stream);
int gv_unpack_i4(const void* packed, void* out, long long nbytes, void* stream);
int gv_gemm_fp8(const void* xq, const void* x_scale, const void* wq, const void* w_scale, void* out,
                long long M, long long N, long long K, long long lds, long long ldo, void* stream);
int gv_grouped_gemm_fp8(const void* xq, const void* x_scale, const void* wq, const void* w_scale,
                        const void* offsets, void* out, long long rows_cap, long long N, long long K,
                        long long E, long long lds, void* stream);

// ---- segment forms of the grouped GEMMs and the expert-parallel dispatch / combine (moe_a2a.cu)
int gv_grouped_gemm_bf16_seg(const void* xs, const void* w, const void* seg_start, const void* seg_end,
                             void* out, long long rows_cap, long long N, long long K, long long E,
                             long long G, long long avg_rows, void* stream);
// SwiGLU in the epilogue: w rows interleaved in blocks of [16 gate | 16 up], out [rows_cap, N / 2]
int gv_grouped_gemm_bf16_swiglu(const void* xs, const void* w, const void* offsets, void* out,
                                long long rows_cap, long long N, long long K, long long E, float clamp,
                                void* stream);
int gv_grouped_gemm_bf16_swiglu_seg(const void* xs, const void* w, const void* seg_start,
                                    const void* seg_end, void* out, long long rows_cap, long long N,
                                    long long K, long long E, long long G, long long avg_rows, float clamp,
                                    void* stream);
int gv_grouped_gemm_fp8_seg(const void* xq, const void* x_scale, const void* wq, const void* w_scale,
                            const void* seg_start, const void* seg_end, void* out, long long rows_cap,
                            long long N, long long K, long long E, long long G, long long lds,
                            long long avg_rows, void* stream);
// offs: host long long[6] = byte offsets {rows, scales, meta, counters, ret, flags} in the slab;
// dims: host long long[6] = {rank, R, cap, H, e_local, fp8}
int gv_moe_a2a_dispatch(const void* x, const void* ids, void* row_of, long long T, long long K,
                        const void* peers, const void* offs, void* state, const void* dims,
                        void* stream);
int gv_moe_a2a_recv_prepare(void* seg_start, void* seg_end, const void* peers, const void* offs,
                            void* state, const void* dims, void* stream);
int gv_moe_a2a_combine_push(const void* ys, const void* seg_end, const void* peers, const void* offs,
                            void* state, const void* dims, void* stream);
int gv_moe_a2a_combine_wait(const void* peers, const void* offs, void* state, const void* dims,
                            void* stream);

// ---- sequence-parallel fused GEMMs (gemm_sp.cu)
int gv_gemm_rs(const void* x, const void* w, void* out, long long M, long long N, long long K,
               long long ldx, long long ldw, long long ldo, const void* peers, long long recv_off,
               long long recv_stride, long long cnt_off, void* state, long long rank, long long R,
               long long m_r_cap, void* stream);
int gv_ag_gemm_setup(void* maps_dev, const void* peers_host, long long stage_off, long long stage_stride,
                     long long m_r_cap, long long K, long long R, long long rank, void* stream);
int gv_ag_gemm(const void* x_local, const void* w, const void* bias, void* out, long long M, long long N,
               long long K, long long ldw, long long ldo, const void* maps_dev, const void* peers,
               long long stage_off, long long stage_stride, long long flags_off, void* state,
               long long rank, long long R, long long m_r_cap, void* stream);

// ---- gated delta-net linear attention (linear_attn.cu)
int gv_gdn_gate(const void* b, const void* a, const void* A_log, const void* dt_bias, void* beta, void* g,
                long long T, long long H, long long ldb, long long lda, void* stream);
int gv_gdn_conv1d_silu(const void* x, const void* w, const void* bias, void* conv_state,
                       const void* q_start, const void* slots, void* out, long long T, long long batch,
                       long long C, long long Kc, long long ldx, long long ldo, void* stream);
int gv_gdn_recurrent(const void* q, const void* k, const void* v, const void* g, const void* beta,
                     void* state, const void* q_start, const void* slots, void* out, long long batch,
                     long long Hk, long long Hv, long long dk, long long dv, long long ldq, long long ldk,
                     long long ldv, long long ldo, long long l2norm, float eps, void* stream);
int gv_gdn_norm_gate(const void* o, const void* z, const void* w, void* out, long long T, long long Hv,
                     long long dv, long long ldz, float eps, void* stream);

// ---- sparse attention support (dsa.cu)
int gv_indexer_scores(const void* q, const void* w, const void* k_cache, const void* block_tables,
                      const void* q_start, const void* cached_lens, void* scores, long long T,
                      long long batch, long long Hi, long long D, long long block_size,
                      long long max_blocks, long long lds, long long relu, long long num_blocks,
                      void* stream);
// tcgen05 form for D == 128, Hi % 16 == 0, Hi <= 128 (dsa_tc.cu); same arguments.
int gv_indexer_scores_tc(const void* q, const void* w, const void* k_cache, const void* block_tables,
                         const void* q_start, const void* cached_lens, void* scores, long long T,
                         long long batch, long long Hi, long long D, long long block_size,
                         long long max_blocks, long long lds, long long relu, long long num_blocks,
                         void* stream);
int gv_scatter_rows(const void* src, const void* slots, void* cache, long long T, long long row_bytes,
                    long long num_slots, void* stream);
int gv_topk_select(const void* scores, long long lds, const void* lens, long long rows, long long K,
                   void* out, void* stream);
int gv_gather_paged_rows(const void* cache, const void* block_tables, const void* idx, void* dense,
                         long long batch, long long K, long long row_bytes, long long block_size,
                         long long max_blocks, long long num_blocks, void* stream);

#ifdef __cplusplus
}
#endif
