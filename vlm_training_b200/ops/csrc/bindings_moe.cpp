// Bindings of the mixture-of-experts routing / permutation kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "moe_kernels.h"

using torch::Tensor;

static inline cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

// logits [T, E] bf16 / fp32 -> (weights [T, k] fp32, experts [T, k] int32)
static std::vector<Tensor> moe_route_fwd(const Tensor& logits, int64_t k, bool renorm) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  TORCH_CHECK(logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat, "router logits must be bf16 or fp32");
  c10::cuda::CUDAGuard guard(logits.device());
  const int T = logits.size(0), E = logits.size(1);
  Tensor w = torch::empty({T, k}, logits.options().dtype(torch::kFloat));
  Tensor e = torch::empty({T, k}, logits.options().dtype(torch::kInt));
  int r = vlmt_moe_route_fwd(logits.data_ptr(), logits.scalar_type() == at::kFloat, T, E, (int)k, renorm, w.data_ptr<float>(),
                             e.data_ptr<int>(), nullptr, cur());
  TORCH_CHECK(r == 0, "vlmt_moe_route_fwd failed with code ", r, " (at most 512 experts, k <= 32)");
  return {w, e};
}
static Tensor moe_route_bwd(const Tensor& logits, const Tensor& experts, const Tensor& weights, const Tensor& dweights, bool renorm) {
  TORCH_CHECK(logits.is_contiguous() && experts.is_contiguous() && weights.is_contiguous() && dweights.is_contiguous());
  TORCH_CHECK(experts.scalar_type() == at::kInt && weights.scalar_type() == at::kFloat && dweights.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor d = torch::empty_like(logits);
  int r = vlmt_moe_route_bwd(logits.data_ptr(), logits.scalar_type() == at::kFloat, experts.data_ptr<int>(), weights.data_ptr<float>(),
                             dweights.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), (int)experts.size(1), renorm,
                             d.data_ptr(), cur());
  TORCH_CHECK(r == 0, "vlmt_moe_route_bwd failed with code ", r);
  return d;
}
// experts [n_slots] int32 -> (counts [E], prefix [E + 1], dest [n_slots], slot_of_row [cap_rows]), all int32
static std::vector<Tensor> moe_plan(const Tensor& experts, int64_t E, int64_t cap_rows) {
  TORCH_CHECK(experts.is_cuda() && experts.scalar_type() == at::kInt && experts.is_contiguous());
  c10::cuda::CUDAGuard guard(experts.device());
  const long n = experts.numel();
  auto opt = experts.options();
  Tensor hist = torch::empty({std::max(1, vlmt_moe_plan_blocks(n)) * E}, opt);
  Tensor counts = torch::empty({E}, opt), prefix = torch::empty({E + 1}, opt), dest = torch::empty({n}, opt);
  Tensor slot_of_row = torch::empty({cap_rows}, opt);
  int r = vlmt_moe_plan(experts.data_ptr<int>(), n, (int)E, hist.data_ptr<int>(), counts.data_ptr<int>(), prefix.data_ptr<int>(),
                        dest.data_ptr<int>(), slot_of_row.data_ptr<int>(), cap_rows, cur());
  TORCH_CHECK(r == 0, "vlmt_moe_plan failed with code ", r);
  return {counts, prefix, dest, slot_of_row};
}
static Tensor moe_rows_from_tokens(const Tensor& src, const Tensor& slot_of_row, const Tensor& prefix, int64_t k,
                                   const c10::optional<Tensor>& scale) {
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == at::kBFloat16 && src.dim() == 2 && src.is_contiguous());
  TORCH_CHECK(slot_of_row.scalar_type() == at::kInt && prefix.scalar_type() == at::kInt);
  if (scale.has_value()) TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->is_contiguous());
  c10::cuda::CUDAGuard guard(src.device());
  const long cap = slot_of_row.numel();
  const int H = src.size(1);
  // the kernel writes every row of the tiles in use (padding rows as zeros); the rows of unused tiles are read by nobody
  // (the grouped GEMMs stop at the last used tile), so the capacity is not filled
  Tensor rows = torch::empty({cap, H}, src.options());
  int r = vlmt_moe_rows_from_tokens(src.data_ptr(), slot_of_row.data_ptr<int>(), prefix.data_ptr<int>(), (int)prefix.numel() - 1, (int)k, H,
                                    scale.has_value() ? scale->data_ptr<float>() : nullptr, rows.data_ptr(), cap, cur());
  TORCH_CHECK(r == 0, "vlmt_moe_rows_from_tokens failed with code ", r);
  return rows;
}
// -> (out [T, H] bf16 or undefined, dw [T, k] fp32 or undefined)
static std::vector<Tensor> moe_tokens_from_rows(const Tensor& rows, const Tensor& dest, const c10::optional<Tensor>& w, int64_t T, int64_t k,
                                                bool want_out, const c10::optional<Tensor>& g) {
  TORCH_CHECK(rows.is_cuda() && rows.scalar_type() == at::kBFloat16 && rows.dim() == 2 && rows.is_contiguous());
  TORCH_CHECK(dest.scalar_type() == at::kInt && dest.numel() == T * k);
  if (w.has_value()) TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == T * k);
  c10::cuda::CUDAGuard guard(rows.device());
  const int H = rows.size(1);
  Tensor out, dw;
  if (want_out) out = torch::empty({T, H}, rows.options());
  if (g.has_value()) {
    TORCH_CHECK(g->scalar_type() == at::kBFloat16 && g->is_contiguous() && g->size(0) == T && g->size(1) == H);
    dw = torch::empty({T, k}, rows.options().dtype(torch::kFloat));
  }
  int r = vlmt_moe_tokens_from_rows(rows.data_ptr(), dest.data_ptr<int>(), w.has_value() ? w->data_ptr<float>() : nullptr, (int)T, (int)k, H,
                                    want_out ? out.data_ptr() : nullptr, g.has_value() ? g->data_ptr() : nullptr,
                                    g.has_value() ? dw.data_ptr<float>() : nullptr, cur());
  TORCH_CHECK(r == 0, "vlmt_moe_tokens_from_rows failed with code ", r);
  return {out, dw};
}

// ------------------------------------------------------------------------------------------------ expert parallelism
Tensor vlmt_status_tensor();

static void fill_ptrs(const std::vector<int64_t>& v, void** out) {
  TORCH_CHECK(v.size() <= 16, "at most 16 expert-parallel ranks");
  for (size_t i = 0; i < v.size(); ++i) out[i] = reinterpret_cast<void*>(v[i]);
}
// experts [n_slots] int32 -> (hist scratch, counts [E], prefix [E + 1])
static std::vector<Tensor> moe_plan_count(const Tensor& experts, int64_t E) {
  TORCH_CHECK(experts.is_cuda() && experts.scalar_type() == at::kInt && experts.is_contiguous());
  c10::cuda::CUDAGuard guard(experts.device());
  const long n = experts.numel();
  auto opt = experts.options();
  Tensor hist = torch::empty({std::max(1, vlmt_moe_plan_blocks(n)) * E}, opt);
  Tensor counts = torch::empty({E}, opt), prefix = torch::empty({E + 1}, opt);
  int r = vlmt_moe_plan_count(experts.data_ptr<int>(), n, (int)E, hist.data_ptr<int>(), counts.data_ptr<int>(), prefix.data_ptr<int>(), cur());
  TORCH_CHECK(r == 0, "vlmt_moe_plan_count failed with code ", r);
  return {hist, counts, prefix};
}
// -> dest [n_slots] (row inside the owner's buffer, -1 when it does not fit)
static Tensor moe_plan_place_remote(const Tensor& experts, const Tensor& hist, const Tensor& prefix, const Tensor& row_base, int64_t cap_rows) {
  c10::cuda::CUDAGuard guard(experts.device());
  Tensor dest = torch::empty({experts.numel()}, experts.options());
  int r = vlmt_moe_plan_place(experts.data_ptr<int>(), experts.numel(), (int)row_base.numel(), hist.data_ptr<int>(), prefix.data_ptr<int>(),
                              row_base.data_ptr<int>(), dest.data_ptr<int>(), nullptr, cap_rows, cur());
  TORCH_CHECK(r == 0, "vlmt_moe_plan_place failed with code ", r);
  return dest;
}
static void ep_push_counts(const Tensor& counts, const std::vector<int64_t>& mats, int64_t me) {
  c10::cuda::CUDAGuard guard(counts.device());
  void* m[16];
  fill_ptrs(mats, m);
  int r = vlmt_ep_push_counts(counts.data_ptr<int>(), (int)counts.numel(), m, (int)mats.size(), (int)me, cur());
  TORCH_CHECK(r == 0, "vlmt_ep_push_counts failed with code ", r);
}
// counts_all [ep, E] int32 (local, symmetric) -> (row_base [E], prefix_local [El + 1], tot_local [El])
static std::vector<Tensor> ep_plan(const Tensor& counts_all, int64_t ep, int64_t me, int64_t cap_rows) {
  TORCH_CHECK(counts_all.scalar_type() == at::kInt && counts_all.is_contiguous());
  c10::cuda::CUDAGuard guard(counts_all.device());
  const int E = (int)(counts_all.numel() / ep), El = E / (int)ep;
  auto opt = counts_all.options();
  Tensor row_base = torch::empty({E}, opt), prefix_local = torch::empty({El + 1}, opt), tot_local = torch::empty({El}, opt);
  int r = vlmt_ep_plan(counts_all.data_ptr<int>(), (int)ep, E, (int)me, (int)cap_rows, row_base.data_ptr<int>(), prefix_local.data_ptr<int>(),
                       tot_local.data_ptr<int>(), vlmt_status_tensor().data_ptr<int>(), cur());
  TORCH_CHECK(r == 0, "vlmt_ep_plan failed with code ", r);
  return {row_base, prefix_local, tot_local};
}
static void ep_dispatch(const Tensor& src, const Tensor& experts, const Tensor& dest, const c10::optional<Tensor>& scale, int64_t k, int64_t El,
                        int64_t me, const std::vector<int64_t>& rows, const std::vector<int64_t>& srcs) {
  TORCH_CHECK(src.scalar_type() == at::kBFloat16 && src.is_contiguous() && src.dim() == 2);
  if (scale.has_value()) TORCH_CHECK(scale->scalar_type() == at::kFloat && scale->is_contiguous());
  c10::cuda::CUDAGuard guard(src.device());
  void* r_[16];
  void* s_[16];
  fill_ptrs(rows, r_);
  fill_ptrs(srcs, s_);
  int r = vlmt_ep_dispatch(src.data_ptr(), experts.data_ptr<int>(), dest.data_ptr<int>(), scale.has_value() ? scale->data_ptr<float>() : nullptr,
                           experts.numel(), (int)k, (int)src.size(1), (int)El, (int)me, r_, s_, (int)rows.size(), cur());
  TORCH_CHECK(r == 0, "vlmt_ep_dispatch failed with code ", r);
}
static void ep_zero_padding(Tensor& rows, Tensor& src_of_row, const Tensor& prefix_local, const Tensor& tot_local) {
  c10::cuda::CUDAGuard guard(rows.device());
  int r = vlmt_ep_zero_padding(rows.data_ptr(), src_of_row.data_ptr<int>(), prefix_local.data_ptr<int>(), tot_local.data_ptr<int>(),
                               (int)tot_local.numel(), (int)rows.size(1), rows.size(0), cur());
  TORCH_CHECK(r == 0, "vlmt_ep_zero_padding failed with code ", r);
}
static void ep_return(const Tensor& y, const Tensor& src_of_row, const Tensor& prefix_local, int64_t n_slots, const std::vector<int64_t>& backs) {
  TORCH_CHECK(y.scalar_type() == at::kBFloat16 && y.is_contiguous() && y.dim() == 2);
  c10::cuda::CUDAGuard guard(y.device());
  void* b[16];
  fill_ptrs(backs, b);
  int r = vlmt_ep_return(y.data_ptr(), src_of_row.data_ptr<int>(), prefix_local.data_ptr<int>(), (int)prefix_local.numel() - 1, n_slots,
                         (int)y.size(1), y.size(0), b, (int)backs.size(), cur());
  TORCH_CHECK(r == 0, "vlmt_ep_return failed with code ", r);
}

void bind_moe(pybind11::module_& m) {
  m.def("moe_plan_count", &moe_plan_count);
  m.def("moe_plan_place_remote", &moe_plan_place_remote);
  m.def("ep_push_counts", &ep_push_counts);
  m.def("ep_plan", &ep_plan);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_zero_padding", &ep_zero_padding);
  m.def("ep_return", &ep_return);
  m.def("moe_route_fwd", &moe_route_fwd);
  m.def("moe_route_bwd", &moe_route_bwd);
  m.def("moe_plan", &moe_plan);
  m.def("moe_rows_from_tokens", &moe_rows_from_tokens);
  m.def("moe_tokens_from_rows", &moe_tokens_from_rows);
}
