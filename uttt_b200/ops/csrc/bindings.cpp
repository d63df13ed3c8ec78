// Python bindings of the uttt_b200 sm_100a extension.
#include <torch/extension.h>

namespace uttt {
std::vector<at::Tensor> rms_norm_fwd(at::Tensor x, c10::optional<at::Tensor> w, double eps);
std::vector<at::Tensor> rms_norm_bwd(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> w, at::Tensor rstd);
std::vector<at::Tensor> rms_norm_gated_fwd(at::Tensor x, c10::optional<at::Tensor> w, at::Tensor gate, double eps);
std::vector<at::Tensor> rms_norm_gated_bwd(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> w, at::Tensor rstd,
                                           at::Tensor gate);
at::Tensor embedding_fwd(at::Tensor table, at::Tensor ids);
at::Tensor embedding_bwd(at::Tensor dy, at::Tensor ids, int64_t vocab);
std::vector<at::Tensor> add_rms_norm_fwd(at::Tensor x, at::Tensor delta, c10::optional<at::Tensor> w, double eps);
std::vector<at::Tensor> add_rms_norm_bwd(at::Tensor dy, c10::optional<at::Tensor> ds, at::Tensor s,
                                         c10::optional<at::Tensor> w, at::Tensor rstd);
at::Tensor rope_fwd(at::Tensor x, at::Tensor table, int64_t offset, bool inverse);
std::vector<at::Tensor> fw_qk_prep_fwd(at::Tensor x, c10::optional<at::Tensor> scale, c10::optional<at::Tensor> shift,
                                       at::Tensor table, int64_t heads, int64_t rope_dim, int64_t offset, int64_t l,
                                       bool silu, int64_t norm);
std::vector<at::Tensor> fw_qk_prep_bwd(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> scale,
                                       c10::optional<at::Tensor> shift, at::Tensor inv, at::Tensor table,
                                       int64_t heads, int64_t rope_dim, int64_t offset, int64_t l, bool silu,
                                       int64_t norm);
at::Tensor swiglu_fwd(at::Tensor y02);
at::Tensor swiglu_bwd(at::Tensor dh, at::Tensor y02);
std::vector<at::Tensor> swiglu_bwd_bwd(at::Tensor G, at::Tensor dh, at::Tensor y02);
std::vector<at::Tensor> fw_write_pw_fwd(at::Tensor y02, at::Tensor dh, at::Tensor lr);
std::vector<at::Tensor> fw_write_pw_bwd(at::Tensor C, at::Tensor Ch, at::Tensor y02, at::Tensor dh, at::Tensor lr);
at::Tensor permute_rows(at::Tensor x, at::Tensor dest, int64_t rows_padded, c10::optional<at::Tensor> w,
                        c10::optional<at::Tensor> offsets, c10::optional<at::Tensor> sizes);
at::Tensor unpermute_rows(at::Tensor y, at::Tensor dest, c10::optional<at::Tensor> w);
std::vector<at::Tensor> unpermute_rows_bwd(at::Tensor dout, at::Tensor y, at::Tensor dest, at::Tensor w,
                                           c10::optional<at::Tensor> offsets, c10::optional<at::Tensor> sizes);
void sumsq_accum(at::Tensor g, double scale, at::Tensor out);
void adamw_flat(at::Tensor p, at::Tensor g, at::Tensor m, at::Tensor v, c10::optional<at::Tensor> plow, double lr,
                double b1, double b2, double eps, double wd, int64_t step, at::Tensor gscale, at::Tensor apply,
                double gmul, int64_t decay_hi);
void ce_fwd_bwd_(at::Tensor logits, at::Tensor labels, at::Tensor loss, int64_t ignore_index);
int64_t launch_count();
std::vector<at::Tensor> build_group_plan(at::Tensor expert_idx, int64_t num_experts);
at::Tensor plucker_embed(at::Tensor image, at::Tensor fxfycxcy, at::Tensor c2w, at::Tensor is_target, int64_t patch);

at::Tensor gg_nt(at::Tensor x, at::Tensor w, at::Tensor tile_group, c10::optional<at::Tensor> out_buf,
                 c10::optional<at::Tensor> ready, int64_t ready_target, c10::optional<at::Tensor> done,
                 double wait_limit_ms);
int64_t gg_nt_done_per_tile(int64_t n);
at::Tensor gg_nn(at::Tensor x, at::Tensor w, at::Tensor tile_group);
at::Tensor gg_nt_swiglu(at::Tensor x, at::Tensor w02, at::Tensor tile_group, c10::optional<at::Tensor> ready,
                        int64_t ready_target, double wait_limit_ms);
std::vector<at::Tensor> gg_nt_swiglu_bwd(at::Tensor x, at::Tensor w02, at::Tensor dh, c10::optional<at::Tensor> lr,
                                         at::Tensor tile_group, bool want_h, bool want_y);
std::vector<at::Tensor> pair_plan(at::Tensor tile_group, at::Tensor offsets, int64_t tiles);
at::Tensor gg_nt_pair(at::Tensor x, at::Tensor w, at::Tensor tile_group, at::Tensor entries, at::Tensor count);
at::Tensor gg_nn_pair(at::Tensor x, at::Tensor w, at::Tensor tile_group, at::Tensor entries, at::Tensor count);
at::Tensor gg_nt_swiglu_pair(at::Tensor x, at::Tensor w02, at::Tensor tile_group, at::Tensor entries,
                             at::Tensor count);
std::vector<at::Tensor> gg_nt_swiglu_bwd_pair(at::Tensor x, at::Tensor w02, at::Tensor dh, c10::optional<at::Tensor> lr,
                                              at::Tensor tile_group, at::Tensor entries, at::Tensor count, bool want_h,
                                              bool want_y);
at::Tensor gg_tn_multi(std::vector<at::Tensor> as, std::vector<at::Tensor> bs, std::vector<at::Tensor> offsets,
                       int64_t num_groups, at::ScalarType out_dtype, c10::optional<at::Tensor> accumulate_into);
at::Tensor gg_tn_segments(at::Tensor a, at::Tensor b, at::Tensor offsets, int64_t num_groups, int64_t segments,
                          at::ScalarType out_dtype, c10::optional<at::Tensor> accumulate_into);
at::Tensor bmm_nt(at::Tensor a, at::Tensor b, double alpha, c10::optional<at::Tensor> d, double beta);
at::Tensor gemm_status(at::Tensor like);
at::Tensor bmm_general(at::Tensor a, at::Tensor b, int64_t mode, double alpha, c10::optional<at::Tensor> d, double beta);
void rs_sumsq(std::vector<int64_t> grad_ptrs, int64_t rank, int64_t shard_off, at::Tensor out, double scale,
              at::Tensor sumsq, bool grads_bf16, int64_t mc_ptr);
void adamw_scatter(at::Tensor p, at::Tensor g, at::Tensor m, at::Tensor v, std::vector<int64_t> compute_ptrs,
                   int64_t rank, int64_t shard_off, bool compute_bf16, double lr, double b1, double b2, double eps,
                   double wd, int64_t step, at::Tensor gscale, at::Tensor apply, int64_t decay_hi, int64_t mc_ptr);
std::vector<at::Tensor> swa_fwd(at::Tensor q, at::Tensor k, at::Tensor v, int64_t window, bool causal, double scale);
std::vector<at::Tensor> patch_decode_fwd(at::Tensor y, c10::optional<at::Tensor> target, int64_t views, int64_t height,
                                         int64_t width, int64_t patch);
at::Tensor patch_decode_bwd(at::Tensor rendering, c10::optional<at::Tensor> target, c10::optional<at::Tensor> g_render,
                            c10::optional<at::Tensor> g_sse, int64_t patch, at::ScalarType dtype);
at::Tensor ag_linear(at::Tensor x, std::vector<int64_t> shard_ptrs, int64_t rank, at::Tensor w_full, at::Tensor ready,
                     int64_t gather_ctas, double wait_limit_ms, int64_t withhold_from_block);
std::vector<at::Tensor> ep_plan(at::Tensor sizes_all, int64_t rank, int64_t B, int64_t E, int64_t tiles_cap);
void ep_push(at::Tensor src, c10::optional<at::Tensor> weights, at::Tensor idx, at::Tensor dest, at::Tensor offsets_local,
             at::Tensor sizes_local, at::Tensor remote_start, std::vector<int64_t> peer_ptrs, int64_t E,
             int64_t rows_per_batch, int64_t cap_rows, std::vector<int64_t> ready_ptrs);
at::Tensor ep_pull(std::vector<int64_t> peer_ptrs, c10::optional<at::Tensor> weights, at::Tensor idx, at::Tensor dest,
                   at::Tensor offsets_local, at::Tensor remote_start, int64_t E, int64_t rows_per_batch, int64_t D,
                   at::ScalarType dtype, int64_t cap_rows, std::vector<int64_t> done_ptrs, int64_t done_target,
                   double wait_limit_ms);
at::Tensor ep_pull_dot(at::Tensor local, std::vector<int64_t> peer_ptrs, at::Tensor idx, at::Tensor dest,
                       at::Tensor offsets_local, at::Tensor remote_start, int64_t E, int64_t rows_per_batch,
                       int64_t cap_rows);
std::vector<at::Tensor> frob_normalize_fwd(at::Tensor g, double eps);
at::Tensor frob_normalize_bwd(at::Tensor g, at::Tensor sumsq, at::Tensor dx, double eps);
bool pool_step_supported(int64_t D);
std::vector<at::Tensor> pool_step_fwd(at::Tensor m, at::Tensor d, double lr, int64_t mode);
std::vector<at::Tensor> pool_step_bwd(at::Tensor m, at::Tensor d, c10::optional<at::Tensor> gn,
                                      c10::optional<at::Tensor> gw, double lr, int64_t mode);
bool router_supported(int64_t D, int64_t E, int64_t topk);
std::vector<at::Tensor> router_fwd(at::Tensor rows, at::Tensor router, c10::optional<at::Tensor> bias, int64_t topk,
                                   int64_t rows_per_batch, double alpha, bool bias_in_logits, bool renorm,
                                   int64_t mode, double rscale, double norm_eps);
std::vector<at::Tensor> router_bwd(at::Tensor rows, at::Tensor router, at::Tensor probs, at::Tensor idx,
                                   c10::optional<at::Tensor> dweights, c10::optional<at::Tensor> dprobs_sum,
                                   int64_t rows_per_batch, double alpha, bool renorm, bool need_drows, int64_t mode,
                                   double rscale, double norm_eps, c10::optional<at::Tensor> logits);
std::vector<at::Tensor> swa_bwd(at::Tensor dout, at::Tensor q, at::Tensor k, at::Tensor v, at::Tensor o, at::Tensor lse,
                                int64_t window, bool causal, double scale);
}  // namespace uttt

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  using namespace uttt;
  m.def("rms_norm_fwd", &rms_norm_fwd);
  m.def("rms_norm_bwd", &rms_norm_bwd);
  m.def("rms_norm_gated_fwd", &rms_norm_gated_fwd);
  m.def("rms_norm_gated_bwd", &rms_norm_gated_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("add_rms_norm_fwd", &add_rms_norm_fwd);
  m.def("add_rms_norm_bwd", &add_rms_norm_bwd);
  m.def("rope_fwd", &rope_fwd);
  m.def("fw_qk_prep_fwd", &fw_qk_prep_fwd);
  m.def("fw_qk_prep_bwd", &fw_qk_prep_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("swiglu_bwd_bwd", &swiglu_bwd_bwd);
  m.def("fw_write_pw_fwd", &fw_write_pw_fwd);
  m.def("fw_write_pw_bwd", &fw_write_pw_bwd);
  m.def("permute_rows", &permute_rows, py::arg("x"), py::arg("dest"), py::arg("rows_padded"), py::arg("w"),
        py::arg("offsets") = py::none(), py::arg("sizes") = py::none());
  m.def("unpermute_rows", &unpermute_rows);
  m.def("unpermute_rows_bwd", &unpermute_rows_bwd, py::arg("dout"), py::arg("y"), py::arg("dest"), py::arg("w"),
        py::arg("offsets") = py::none(), py::arg("sizes") = py::none());
  m.def("sumsq_accum", &sumsq_accum);
  m.def("adamw_flat", &adamw_flat);
  m.def("ce_fwd_bwd_", &ce_fwd_bwd_);
  m.def("launch_count", &launch_count);
  m.def("build_group_plan", &build_group_plan);
  m.def("plucker_embed", &plucker_embed);
  m.def("gg_nt", &gg_nt, py::arg("x"), py::arg("w"), py::arg("tile_group"), py::arg("out") = py::none(),
        py::arg("ready") = py::none(), py::arg("ready_target") = 0, py::arg("done") = py::none(),
        py::arg("wait_limit_ms") = 0.0);
  m.def("gg_nt_done_per_tile", &gg_nt_done_per_tile);
  m.def("gg_nn", &gg_nn);
  m.def("gg_nt_swiglu", &gg_nt_swiglu, py::arg("x"), py::arg("w02"), py::arg("tile_group"),
        py::arg("ready") = py::none(), py::arg("ready_target") = 0, py::arg("wait_limit_ms") = 0.0);
  m.def("gg_nt_swiglu_bwd", &gg_nt_swiglu_bwd);
  m.def("pair_plan", &pair_plan);
  m.def("gg_nt_pair", &gg_nt_pair);
  m.def("gg_nn_pair", &gg_nn_pair);
  m.def("gg_nt_swiglu_pair", &gg_nt_swiglu_pair);
  m.def("gg_nt_swiglu_bwd_pair", &gg_nt_swiglu_bwd_pair);
  m.def("gg_tn_segments", &gg_tn_segments);
  m.def("gg_tn_multi", &gg_tn_multi);
  m.def("bmm_nt", &bmm_nt);
  m.def("gemm_status", &gemm_status);
  m.def("bmm_general", &bmm_general);
  m.def("swa_fwd", &swa_fwd);
  m.def("swa_bwd", &swa_bwd);
  m.def("patch_decode_fwd", &patch_decode_fwd);
  m.def("patch_decode_bwd", &patch_decode_bwd);
  m.def("ag_linear", &ag_linear, py::arg("x"), py::arg("shard_ptrs"), py::arg("rank"), py::arg("w_full"),
        py::arg("ready"), py::arg("gather_ctas"), py::arg("wait_limit_ms") = 0.0,
        py::arg("withhold_from_block") = -1);
  m.def("ep_plan", &ep_plan);
  m.def("ep_push", &ep_push, py::arg("src"), py::arg("weights"), py::arg("idx"), py::arg("dest"),
        py::arg("offsets_local"), py::arg("sizes_local"), py::arg("remote_start"), py::arg("peer_ptrs"), py::arg("E"),
        py::arg("rows_per_batch"), py::arg("cap_rows"), py::arg("ready_ptrs") = std::vector<int64_t>());
  m.def("ep_pull", &ep_pull, py::arg("peer_ptrs"), py::arg("weights"), py::arg("idx"), py::arg("dest"),
        py::arg("offsets_local"), py::arg("remote_start"), py::arg("E"), py::arg("rows_per_batch"), py::arg("D"),
        py::arg("dtype"), py::arg("cap_rows"), py::arg("done_ptrs") = std::vector<int64_t>(),
        py::arg("done_target") = 0, py::arg("wait_limit_ms") = 0.0);
  m.def("ep_pull_dot", &ep_pull_dot);
  m.def("frob_normalize_fwd", &frob_normalize_fwd);
  m.def("frob_normalize_bwd", &frob_normalize_bwd);
  m.def("pool_step_supported", &pool_step_supported);
  m.def("pool_step_fwd", &pool_step_fwd);
  m.def("pool_step_bwd", &pool_step_bwd);
  m.def("router_supported", &router_supported);
  m.def("router_fwd", &router_fwd);
  m.def("router_bwd", &router_bwd);
  m.def("rs_sumsq", &rs_sumsq);
  m.def("adamw_scatter", &adamw_scatter);
}
