// Python bindings of the sm_100a extension (module chatlearn_b200._C).
#include <torch/extension.h>

std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps);
std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dy,
                                    const at::Tensor& rstd);
at::Tensor swiglu_fwd(const at::Tensor& gu);
at::Tensor swiglu_bwd(const at::Tensor& gu, const at::Tensor& dy);
at::Tensor qk_norm_rope_fwd(const at::Tensor& x, int64_t n_heads, int64_t D, const c10::optional<at::Tensor>& w,
                            const at::Tensor& pos, const at::Tensor& inv_freq, double eps);
at::Tensor qk_norm_rope_bwd(const at::Tensor& dy, const at::Tensor& x, at::Tensor dx_out, int64_t n_heads,
                            int64_t D, const c10::optional<at::Tensor>& w, const at::Tensor& pos,
                            const at::Tensor& inv_freq, double eps);
std::vector<at::Tensor> grpo_loss_fwd(const at::Tensor& lp, const at::Tensor& old,
                                      const c10::optional<at::Tensor>& ref, const at::Tensor& adv,
                                      const at::Tensor& mask, const c10::optional<at::Tensor>& ent,
                                      double pos_clip, double neg_clip, double diff_clip, double final_clip,
                                      double kl_coef, double ent_coef, double inv_norm);
at::Tensor qkv_rope_append(const at::Tensor& qkv, int64_t nq, int64_t nkv, int64_t D, const c10::optional<at::Tensor>& qw,
                           const c10::optional<at::Tensor>& kw, const at::Tensor& pos, const at::Tensor& inv_freq,
                           const at::Tensor& slots, at::Tensor k_cache, at::Tensor v_cache, double eps,
                           const c10::optional<at::Tensor>& planes);
std::vector<at::Tensor> gemm_bf16_nt_planes(const at::Tensor& a, const at::Tensor& b);
at::Tensor planes_residual_rmsnorm(at::Tensor resid, const at::Tensor& planes, const c10::optional<at::Tensor>& w, double eps);
std::vector<at::Tensor> gspo_loss_fwd(const at::Tensor& lp, const at::Tensor& old, const c10::optional<at::Tensor>& ref,
                                      const at::Tensor& adv, const at::Tensor& mask, const c10::optional<at::Tensor>& ent,
                                      const at::Tensor& seq_ids, int64_t num_seqs, double pos_clip, double neg_clip,
                                      double diff_clip, double final_clip, double kl_coef, double ent_coef, double inv_norm);
void adamw_step(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                const c10::optional<at::Tensor>& out, int64_t step, double lr, double b1, double b2, double eps,
                double wd, const c10::optional<at::Tensor>& scale_t, double scale_v);
at::Tensor sumsq(const at::Tensor& x);
std::vector<at::Tensor> logits_stats(const at::Tensor& z, const at::Tensor& labels, double inv_temp);
at::Tensor logits_grad(const at::Tensor& z, const at::Tensor& labels, const at::Tensor& lse,
                       const at::Tensor& ent, const at::Tensor& g_lp, const c10::optional<at::Tensor>& g_ent,
                       double inv_temp, bool out_bf16);
std::vector<at::Tensor> sample(const at::Tensor& logits, const at::Tensor& u, double temperature, int64_t top_k,
                               double top_p, double min_p);
at::Tensor apply_penalties(const at::Tensor& logits, const at::Tensor& counts,
                           const c10::optional<at::Tensor>& prompt_mask, double presence, double frequency,
                           double repetition);
void kv_append(const at::Tensor& k, const at::Tensor& v, at::Tensor k_cache, at::Tensor v_cache,
               const at::Tensor& slots);
bool paged_decode_supported(int64_t dk, int64_t dv, int64_t bs, int64_t rep);
at::Tensor paged_decode(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                        const at::Tensor& block_tables, const c10::optional<at::Tensor>& q_seq,
                        const at::Tensor& ctx_len, double scale, int64_t num_splits);
bool paged_decode_tc_supported(int64_t dk, int64_t dv, int64_t bs, int64_t rep);
at::Tensor paged_decode_tc(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                           const at::Tensor& block_tables, const c10::optional<at::Tensor>& q_seq,
                           const at::Tensor& ctx_len, double scale, int64_t num_splits);
at::Tensor mla_paged_decode(const at::Tensor& q, const at::Tensor& cache, const at::Tensor& block_tables,
                            const at::Tensor& ctx_len, double scale, int64_t num_splits);
at::Tensor paged_decode_tc_grouped(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                                   const at::Tensor& block_tables, const at::Tensor& ctx_len, const at::Tensor& grp_q,
                                   const at::Tensor& grp_nblk, const at::Tensor& blk_start, double scale,
                                   int64_t prefix_splits, int64_t suffix_splits);
void weight_sync_run(const at::Tensor& desc_table, int64_t num_descs, int64_t total_tiles, int64_t src_dtype,
                     int64_t dst_dtype);
int64_t weight_sync_desc_size();
int64_t weight_sync_tile_elems();
void symm_allreduce(const std::vector<int64_t>& buf_ptrs, const std::vector<int64_t>& flag_ptrs, at::Tensor expect,
                    at::Tensor out, int64_t n, int64_t rank, int64_t num_slots);
at::Tensor symm_rs_pull_sumsq(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& flag_ptrs,
                              at::Tensor expect, at::Tensor shard, int64_t lo, int64_t rank, int64_t num_slots);
void symm_adamw_push(at::Tensor master, const at::Tensor& grad, at::Tensor m, at::Tensor v,
                     const std::vector<int64_t>& param_ptrs, const std::vector<int64_t>& flag_ptrs, at::Tensor expect,
                     int64_t lo, bool params_bf16, int64_t step, double lr, double b1, double b2, double eps, double wd,
                     const c10::optional<at::Tensor>& scale, int64_t rank, int64_t num_slots);
int64_t symm_last_status();
at::Tensor gdn_decode_step(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g,
                           const at::Tensor& beta, at::Tensor state, const at::Tensor& slots, const at::Tensor& fresh,
                           double scale);
void symm_push_chunks(const at::Tensor& src, const std::vector<int64_t>& dst_ptrs, int64_t chunk_bytes, bool all_to_all, int64_t rank);
void symm_group_barrier(const std::vector<int64_t>& flag_ptrs, at::Tensor expect, int64_t slot, int64_t num_slots, int64_t rank);
at::Tensor add_residual_rmsnorm(at::Tensor resid, const at::Tensor& delta, const c10::optional<at::Tensor>& w, double eps);
void grouped_gemm_bf16_nt_table(const at::Tensor& a, const at::Tensor& b, const at::Tensor& table, const at::Tensor& count,
                                at::Tensor out);
void symm_moe_barrier(const std::vector<int64_t>& flag_ptrs, at::Tensor expect, int64_t slot, int64_t num_slots, int64_t rank);
at::Tensor symm_moe_dispatch(const at::Tensor& x, const at::Tensor& idx, const std::vector<int64_t>& recv_x_ptrs,
                             const std::vector<int64_t>& cursor_ptrs, int64_t experts_per_rank, int64_t capacity);
std::vector<at::Tensor> symm_moe_region_table(const at::Tensor& cursor, int64_t capacity, int64_t rows_b);
at::Tensor symm_moe_combine(const std::vector<int64_t>& recv_y_ptrs, const at::Tensor& where, const at::Tensor& weights,
                            int64_t H, int64_t region_rows);
void symm_moe_swiglu(const at::Tensor& gu, at::Tensor y, const at::Tensor& table, const at::Tensor& count);
int64_t symm_moe_last_status();
bool attn_varlen_fwd_supported(int64_t head_dim);
std::vector<at::Tensor> attn_varlen_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                        const at::Tensor& cu_seqlens, double scale, bool causal);
void gemm_bf16_nt_scatter(const at::Tensor& a, const at::Tensor& b, const std::vector<int64_t>& dst, int64_t rows_per_rank);
at::Tensor symm_sum_slots(const at::Tensor& buf, int64_t world, int64_t rows, int64_t cols);
at::Tensor grouped_gemm_bf16_nt(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets);
at::Tensor grouped_gemm_bf16_nn(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets);
at::Tensor grouped_gemm_bf16_tn(const at::Tensor& a, const at::Tensor& b, const at::Tensor& offsets, at::Tensor out,
                                bool accumulate);
std::vector<at::Tensor> moe_router_topk(const at::Tensor& logits, int64_t k, bool sigmoid, bool norm,
                                        const c10::optional<at::Tensor>& bias, int64_t n_group, int64_t topk_group,
                                        double scale);
std::vector<at::Tensor> moe_permute(const at::Tensor& x, const at::Tensor& idx, const at::Tensor& offsets, int64_t total_rows);
at::Tensor moe_permute_at(const at::Tensor& x, const at::Tensor& pos, const c10::optional<at::Tensor>& scale,
                          int64_t total_rows);
at::Tensor moe_combine(const at::Tensor& y, const at::Tensor& pos, const c10::optional<at::Tensor>& weights);
at::Tensor moe_row_dot(const at::Tensor& dy, const at::Tensor& y, const at::Tensor& pos);
at::Tensor symm_ar_residual_rmsnorm(const std::vector<int64_t>& part_ptrs, const std::vector<int64_t>& flag_ptrs,
                                    at::Tensor expect, at::Tensor resid, const c10::optional<at::Tensor>& w, double eps,
                                    int64_t rank, int64_t num_slots);
at::Tensor gemm_bf16_nt(const at::Tensor& a, const at::Tensor& b, bool out_fp32);
void gemm_bf16_nt_out(const at::Tensor& a, const at::Tensor& b, at::Tensor out);
void gemm_set_tile_n(int64_t bn);
at::Tensor gemm_bf16_nn(const at::Tensor& a, const at::Tensor& b, bool out_fp32);
at::Tensor gemm_bf16_tn(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& out, bool accumulate,
                        bool out_fp32);
void gemm_bf16_nt_push(const at::Tensor& a, const at::Tensor& b, at::Tensor out, const std::vector<int64_t>& peer_out);
int64_t gemm_last_status();
void gemm_set_splitk(bool on);
const char* clb200_source_hash();
bool attn_fwd_sm100_supported(int64_t head_dim);
int64_t attn_bwd_sm100_last_status();
std::vector<at::Tensor> attn_bwd_sm100(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o,
                                       const at::Tensor& d_o, const at::Tensor& lse, const at::Tensor& cu_seqlens, double scale,
                                       bool causal);
int64_t attn_sm100_last_status();
std::vector<at::Tensor> attn_fwd_sm100(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                       const at::Tensor& cu_seqlens, double scale, bool causal);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd);
  m.def("grpo_loss_fwd", &grpo_loss_fwd);
  m.def("gspo_loss_fwd", &gspo_loss_fwd);
  m.def("qkv_rope_append", &qkv_rope_append, py::arg("qkv"), py::arg("nq"), py::arg("nkv"), py::arg("D"), py::arg("qw"),
        py::arg("kw"), py::arg("pos"), py::arg("inv_freq"), py::arg("slots"), py::arg("k_cache"), py::arg("v_cache"),
        py::arg("eps"), py::arg("planes") = c10::optional<at::Tensor>());
  m.def("gemm_bf16_nt_planes", &gemm_bf16_nt_planes);
  m.def("planes_residual_rmsnorm", &planes_residual_rmsnorm);
  m.def("adamw_step", &adamw_step);
  m.def("sumsq", &sumsq);
  m.def("logits_stats", &logits_stats);
  m.def("logits_grad", &logits_grad);
  m.def("sample", &sample);
  m.def("apply_penalties", &apply_penalties);
  m.def("kv_append", &kv_append);
  m.def("paged_decode_supported", &paged_decode_supported);
  m.def("paged_decode", &paged_decode);
  m.def("paged_decode_tc_supported", &paged_decode_tc_supported);
  m.def("paged_decode_tc", &paged_decode_tc);
  m.def("paged_decode_tc_grouped", &paged_decode_tc_grouped);
  m.def("mla_paged_decode", &mla_paged_decode);
  m.def("weight_sync_run", &weight_sync_run);
  m.def("weight_sync_desc_size", &weight_sync_desc_size);
  m.def("weight_sync_tile_elems", &weight_sync_tile_elems);
  m.def("symm_allreduce", &symm_allreduce);
  m.def("symm_rs_pull_sumsq", &symm_rs_pull_sumsq);
  m.def("symm_adamw_push", &symm_adamw_push);
  m.def("symm_last_status", &symm_last_status);
  m.def("add_residual_rmsnorm", &add_residual_rmsnorm);
  m.def("grouped_gemm_bf16_nt_table", &grouped_gemm_bf16_nt_table);
  m.def("symm_moe_barrier", &symm_moe_barrier);
  m.def("symm_moe_dispatch", &symm_moe_dispatch);
  m.def("symm_moe_region_table", &symm_moe_region_table);
  m.def("symm_moe_combine", &symm_moe_combine);
  m.def("symm_moe_swiglu", &symm_moe_swiglu);
  m.def("symm_moe_last_status", &symm_moe_last_status);
  m.def("attn_varlen_fwd_supported", &attn_varlen_fwd_supported);
  m.def("attn_varlen_fwd", &attn_varlen_fwd);
  m.def("gemm_bf16_nt_scatter", &gemm_bf16_nt_scatter);
  m.def("symm_sum_slots", &symm_sum_slots);
  m.def("grouped_gemm_bf16_nt", &grouped_gemm_bf16_nt);
  m.def("grouped_gemm_bf16_nn", &grouped_gemm_bf16_nn);
  m.def("grouped_gemm_bf16_tn", &grouped_gemm_bf16_tn, py::arg("a"), py::arg("b"), py::arg("offsets"), py::arg("out"),
        py::arg("accumulate") = false);
  m.def("moe_router_topk", &moe_router_topk);
  m.def("moe_permute", &moe_permute, py::arg("x"), py::arg("idx"), py::arg("offsets"), py::arg("total_rows") = -1);
  m.def("moe_permute_at", &moe_permute_at, py::arg("x"), py::arg("pos"), py::arg("scale"), py::arg("total_rows") = -1);
  m.def("moe_combine", &moe_combine);
  m.def("moe_row_dot", &moe_row_dot);
  m.def("symm_ar_residual_rmsnorm", &symm_ar_residual_rmsnorm);
  m.def("gdn_decode_step", &gdn_decode_step);
  m.def("symm_push_chunks", &symm_push_chunks);
  m.def("symm_group_barrier", &symm_group_barrier);
  m.def("gemm_bf16_nt", &gemm_bf16_nt);
  m.def("gemm_bf16_nt_out", &gemm_bf16_nt_out);
  m.def("gemm_set_tile_n", &gemm_set_tile_n);
  m.def("gemm_bf16_nn", &gemm_bf16_nn);
  m.def("gemm_bf16_tn", &gemm_bf16_tn);
  m.def("gemm_bf16_nt_push", &gemm_bf16_nt_push);
  m.def("gemm_last_status", &gemm_last_status);
  m.def("gemm_set_splitk", &gemm_set_splitk);
  m.def("attn_fwd_sm100_supported", &attn_fwd_sm100_supported);
  m.def("attn_sm100_last_status", &attn_sm100_last_status);
  m.def("attn_fwd_sm100", &attn_fwd_sm100);
  m.def("attn_bwd_sm100", &attn_bwd_sm100);
  m.def("attn_bwd_sm100_last_status", &attn_bwd_sm100_last_status);
  m.def("source_hash", []() { return std::string(clb200_source_hash()); });
}
