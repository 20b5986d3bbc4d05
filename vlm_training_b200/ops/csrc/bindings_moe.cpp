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
  Tensor rows = torch::zeros({cap, H}, src.options());   // rows of tiles that are not in use stay zero
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

void bind_moe(pybind11::module_& m) {
  m.def("moe_route_fwd", &moe_route_fwd);
  m.def("moe_route_bwd", &moe_route_bwd);
  m.def("moe_plan", &moe_plan);
  m.def("moe_rows_from_tokens", &moe_rows_from_tokens);
  m.def("moe_tokens_from_rows", &moe_tokens_from_rows);
}
