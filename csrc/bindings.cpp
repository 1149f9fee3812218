// Python bindings of the sm_100a kernels (module `memarch_b200._C`).
#include <torch/extension.h>

namespace mb {
torch::Tensor gemm(torch::Tensor a, torch::Tensor b, c10::optional<torch::Tensor> out, c10::optional<torch::Tensor> out2,
                   c10::optional<torch::Tensor> aux, bool a_mn, bool b_mn, bool accumulate, int64_t epi, bool out_f32,
                   int64_t groups, c10::optional<torch::Tensor> counts, int64_t count_mode);
void gemm_set_debug(int64_t dbg, int64_t group_m);
int gemm_status(int device);
torch::Tensor gemm_peer(std::vector<int64_t> a_ptrs, int64_t seg_M, int64_t K, int64_t a_groups, int64_t a_pitch,
                        int64_t a_gs, int64_t a_g_off, torch::Tensor b, bool b_mn, c10::optional<torch::Tensor> out_local,
                        std::vector<int64_t> out_ptrs, int64_t out_ld, int64_t out_gs, int64_t out_g_off,
                        c10::optional<torch::Tensor> out2, c10::optional<torch::Tensor> aux, int64_t epi, int64_t groups);
void peer_barrier(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t channel, double timeout_ms);
int64_t peer_status_read();
void peer_reduce_to_local(std::vector<int64_t> in_ptrs, int64_t mc_in, torch::Tensor dst, int64_t offset, double scale);
void peer_broadcast_from_local(std::vector<int64_t> out_ptrs, int64_t mc_out, int64_t offset_bytes, int64_t nbytes, int64_t rank);
void peer_gather(std::vector<int64_t> src_ptrs, torch::Tensor dst, int64_t rank, int64_t C, int64_t g_off);
void peer_allreduce(std::vector<int64_t> in_ptrs, std::vector<int64_t> out_ptrs, int64_t mc_in, int64_t mc_out, int64_t offset,
                    int64_t numel, bool is_bf16, int64_t rank, double scale);
void gemm_set_pair(bool on);
std::vector<torch::Tensor> rmsnorm_fwd(torch::Tensor x, torch::Tensor w, double eps, bool out_bf16);
std::vector<torch::Tensor> rmsnorm_bwd(torch::Tensor dy, torch::Tensor x, torch::Tensor w, torch::Tensor rstd,
                                       c10::optional<torch::Tensor> add, bool want_lo);
std::vector<torch::Tensor> add_rmsnorm_fwd(torch::Tensor x, torch::Tensor y, torch::Tensor w, double eps);
torch::Tensor relu2_fwd(torch::Tensor a);
torch::Tensor relu2_bwd(torch::Tensor dh, torch::Tensor a);
torch::Tensor swiglu_fwd(torch::Tensor gu);
torch::Tensor swiglu_bwd(torch::Tensor dh, torch::Tensor gu);
torch::Tensor rope_qk(torch::Tensor qkv, torch::Tensor cos, torch::Tensor sin, double sign, bool half);
torch::Tensor resid_add(torch::Tensor x, torch::Tensor y);
torch::Tensor rope_merge_bwd(torch::Tensor dq, torch::Tensor dk, torch::Tensor dv, torch::Tensor cos, torch::Tensor sin, bool half);
void ce_rows(torch::Tensor logits, torch::Tensor y, torch::Tensor loss, c10::optional<torch::Tensor> gate,
             c10::optional<torch::Tensor> hit, c10::optional<torch::Tensor> dg);
torch::Tensor gather_rows(torch::Tensor src, torch::Tensor table, c10::optional<torch::Tensor> scale);
torch::Tensor gather_sum_rows(torch::Tensor src, torch::Tensor idx, c10::optional<torch::Tensor> w, int64_t N);
torch::Tensor row_dot(torch::Tensor go, torch::Tensor table, torch::Tensor ye);
int64_t instinct_step(torch::Tensor p, torch::Tensor grad, torch::Tensor m, c10::optional<torch::Tensor> w,
                      c10::optional<torch::Tensor> cs, torch::Tensor gvec, int64_t index, torch::Tensor stake,
                      torch::Tensor lr_t, c10::optional<torch::Tensor> rel, double beta, double wd, int64_t kind, bool sr,
                      torch::Tensor seed_t, c10::optional<torch::Tensor> frozen, c10::optional<torch::Tensor> scratch,
                      c10::optional<torch::Tensor> cs_ok, c10::optional<torch::Tensor> shadow, int64_t phase, int64_t col_rows);
std::vector<torch::Tensor> anchor_select(torch::Tensor s, torch::Tensor tau, int64_t A);
std::vector<torch::Tensor> moe_slots(torch::Tensor e_flat, int64_t E, int64_t C);
std::vector<torch::Tensor> lock_find(torch::Tensor x, int64_t vocab, int64_t n_keys, bool longest_only);
std::vector<torch::Tensor> moe_route_fwd(torch::Tensor logits, torch::Tensor real, torch::Tensor k_tok, int64_t k_max);
std::vector<torch::Tensor> mem_read_fwd(torch::Tensor q, torch::Tensor faces, torch::Tensor valid, torch::Tensor dim_pen,
                                        int64_t Fn, double scale);
std::vector<torch::Tensor> mem_read_bwd(torch::Tensor q, torch::Tensor faces, torch::Tensor valid, torch::Tensor w,
                                        torch::Tensor best, torch::Tensor dw, c10::optional<torch::Tensor> dsc, int64_t Fn,
                                        double scale);
std::vector<torch::Tensor> quant_rows_i8(torch::Tensor x);
torch::Tensor gemm_i8(torch::Tensor a, torch::Tensor b, torch::Tensor sa, torch::Tensor sb, bool out_f32);
std::vector<torch::Tensor> reread_fwd(torch::Tensor sc, torch::Tensor pos, torch::Tensor qpos, torch::Tensor rows,
                                      torch::Tensor ids, torch::Tensor table, torch::Tensor offset, torch::Tensor hv,
                                      torch::Tensor hb, torch::Tensor hh, torch::Tensor Wr, torch::Tensor cp, int64_t k);
std::vector<torch::Tensor> reread_bwd(torch::Tensor dgot, torch::Tensor dcostw, torch::Tensor top_j, torch::Tensor p,
                                      torch::Tensor sc, torch::Tensor pos, torch::Tensor qpos, torch::Tensor rows,
                                      torch::Tensor ids, torch::Tensor table, torch::Tensor offset, torch::Tensor hv,
                                      torch::Tensor hb, torch::Tensor hh, torch::Tensor Wr, torch::Tensor cp);
std::vector<torch::Tensor> rope_route_topk(torch::Tensor S, torch::Tensor lval, torch::Tensor lp, torch::Tensor avalid,
                                           torch::Tensor open_from, int64_t H, int64_t K, int64_t q0, double scale);
std::vector<torch::Tensor> attn_fwd_tc(torch::Tensor q, torch::Tensor k, torch::Tensor v, int64_t window, double scale);
int64_t attn_status_read();
std::vector<torch::Tensor> attn_bwd_tc(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor dout, torch::Tensor lse,
                                       torch::Tensor delta, int64_t window, double scale);
int64_t attn_bwd_status_read();
torch::Tensor embed_sum_fwd(torch::Tensor emb, torch::Tensor x, c10::optional<torch::Tensor> cand, c10::optional<torch::Tensor> sel,
                            c10::optional<torch::Tensor> phr, c10::optional<torch::Tensor> pidx);
std::vector<torch::Tensor> embed_sum_bwd(torch::Tensor dh, torch::Tensor emb, torch::Tensor x, c10::optional<torch::Tensor> cand,
                                         c10::optional<torch::Tensor> sel, int64_t P, c10::optional<torch::Tensor> pidx);
torch::Tensor table_pair_dot(torch::Tensor A, torch::Tensor Bt, torch::Tensor ia, torch::Tensor ib);
torch::Tensor moe_route_bwd(torch::Tensor probs, torch::Tensor top_e, torch::Tensor k_tok, torch::Tensor real, torch::Tensor dw,
                            c10::optional<torch::Tensor> dprobs, c10::optional<torch::Tensor> dpsum);
}  // namespace mb

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &mb::gemm, "tcgen05 GEMM C = A * B^T (bf16, fp32 accumulate in TMEM)");
  m.def("gemm_status", &mb::gemm_status, "read and clear the GEMM status word (0 = ok)");
  m.def("gemm_set_debug", &mb::gemm_set_debug, "pair kernel: test / measurement bits and row-tile group size of the tile order",
        pybind11::arg("dbg") = 0, pybind11::arg("group_m") = 0);
  m.def("gemm_set_pair", &mb::gemm_set_pair, "switch the CTA-pair (cta_group::2) GEMM kernel on or off");
  m.def("gemm_peer", &mb::gemm_peer, "segmented GEMM: A tiles from peer buffers, result rows to the owners' buffers");
  m.def("peer_barrier", &mb::peer_barrier, "bounded device-side barrier over symmetric flags");
  m.def("peer_status_read", &mb::peer_status_read);
  m.def("peer_reduce_to_local", &mb::peer_reduce_to_local, "this rank's slice of a staged buffer summed over all ranks into local memory");
  m.def("peer_broadcast_from_local", &mb::peer_broadcast_from_local, "this rank's slice of a symmetric buffer written to every peer");
  m.def("peer_gather", &mb::peer_gather, "rows of this rank's experts from every rank's dispatch buffer, one kernel");
  m.def("peer_allreduce", &mb::peer_allreduce, "one-shot all-reduce by peer loads/stores or NVLS multimem");
  m.def("rmsnorm_fwd", &mb::rmsnorm_fwd);
  m.def("rmsnorm_bwd", &mb::rmsnorm_bwd);
  m.def("add_rmsnorm_fwd", &mb::add_rmsnorm_fwd);
  m.def("relu2_fwd", &mb::relu2_fwd);
  m.def("relu2_bwd", &mb::relu2_bwd);
  m.def("swiglu_fwd", &mb::swiglu_fwd);
  m.def("swiglu_bwd", &mb::swiglu_bwd);
  m.def("rope_qk", &mb::rope_qk);
  m.def("resid_add", &mb::resid_add);
  m.def("rope_merge_bwd", &mb::rope_merge_bwd);
  m.def("ce_rows", &mb::ce_rows);
  m.def("gather_rows", &mb::gather_rows);
  m.def("gather_sum_rows", &mb::gather_sum_rows);
  m.def("row_dot", &mb::row_dot);
  m.def("instinct_step", &mb::instinct_step, pybind11::arg("p"), pybind11::arg("grad"), pybind11::arg("m"), pybind11::arg("w"),
        pybind11::arg("cs"), pybind11::arg("gvec"), pybind11::arg("index"), pybind11::arg("stake"), pybind11::arg("lr_t"),
        pybind11::arg("rel"), pybind11::arg("beta"), pybind11::arg("wd"), pybind11::arg("kind"), pybind11::arg("sr"),
        pybind11::arg("seed_t"), pybind11::arg("frozen"), pybind11::arg("scratch") = pybind11::none(),
        pybind11::arg("cs_ok") = pybind11::none(), pybind11::arg("shadow") = pybind11::none(), pybind11::arg("phase") = 0,
        pybind11::arg("col_rows") = 0);
  m.def("anchor_select", &mb::anchor_select);
  m.def("moe_slots", &mb::moe_slots);
  m.def("lock_find", &mb::lock_find);
  m.def("attn_fwd_tc", &mb::attn_fwd_tc, "causal / sliding-window attention forward on tcgen05 (head dim 64)");
  m.def("attn_status_read", &mb::attn_status_read);
  m.def("attn_bwd_tc", &mb::attn_bwd_tc, "causal / sliding-window attention backward on tcgen05 (head dim 64)");
  m.def("attn_bwd_status_read", &mb::attn_bwd_status_read);
  m.def("mem_read_fwd", &mb::mem_read_fwd);
  m.def("mem_read_bwd", &mb::mem_read_bwd);
  m.def("quant_rows_i8", &mb::quant_rows_i8);
  m.def("gemm_i8", &mb::gemm_i8);
  m.def("reread_fwd", &mb::reread_fwd);
  m.def("reread_bwd", &mb::reread_bwd);
  m.def("rope_route_topk", &mb::rope_route_topk);
  m.def("moe_route_fwd", &mb::moe_route_fwd);
  m.def("moe_route_bwd", &mb::moe_route_bwd);
  m.def("table_pair_dot", &mb::table_pair_dot, "out[n] = <A[ia[n]], B[ib[n]]>");
  m.def("embed_sum_fwd", &mb::embed_sum_fwd, "token + gated candidate + phrase rows in one gather-sum");
  m.def("embed_sum_bwd", &mb::embed_sum_bwd, "gradient rows scattered into the tables, d sel");
}
