// Bindings of the fused collective kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm_kernels.h"

using torch::Tensor;

Tensor vlmt_status_tensor();

// state tensors are the local shard (master fp32; moments fp32 or bf16); `state_off` is the element offset of `lo` inside them
static void fused_rs_adamw_ag(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& param_ptrs, int64_t grad_mc,
                              int64_t param_mc, int64_t world, int64_t lo, int64_t hi, Tensor& master, Tensor& m, Tensor& v,
                              int64_t state_off, double lr, double b1, double b2, double eps, double wd, double bc1, double bc2,
                              double grad_scale, bool zero_own) {
  TORCH_CHECK((int64_t)grad_ptrs.size() == world && (int64_t)param_ptrs.size() == world);
  TORCH_CHECK(master.scalar_type() == at::kFloat, "master weights must be float32");
  TORCH_CHECK(m.scalar_type() == v.scalar_type() && (m.scalar_type() == at::kFloat || m.scalar_type() == at::kBFloat16),
              "Adam moments must both be float32 or both bfloat16");
  TORCH_CHECK(lo % 8 == 0 && hi % 8 == 0 && state_off % 8 == 0, "shard segment must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(master.device());
  void* g[16];
  void* p[16];
  TORCH_CHECK(world <= 16);
  for (int i = 0; i < world; ++i) { g[i] = reinterpret_cast<void*>(grad_ptrs[i]); p[i] = reinterpret_cast<void*>(param_ptrs[i]); }
  const bool sb = m.scalar_type() == at::kBFloat16;
  const int64_t esz = sb ? 2 : 4;
  int r = vlmt_fused_rs_adamw_ag(g, p, reinterpret_cast<void*>(grad_mc), reinterpret_cast<void*>(param_mc), (int)world, lo, hi,
                                 master.data_ptr<float>() + state_off, static_cast<char*>(m.data_ptr()) + state_off * esz,
                                 static_cast<char*>(v.data_ptr()) + state_off * esz, sb ? 1 : 0, (float)lr, (float)b1, (float)b2,
                                 (float)eps, (float)wd, (float)bc1, (float)bc2, (float)grad_scale, zero_own ? 1 : 0,
                                 vlmt_status_tensor().data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_fused_rs_adamw_ag failed with code ", r);
}

static void rs_reduce_sumsq(const std::vector<int64_t>& grad_ptrs, int64_t grad_mc, int64_t lo, int64_t hi, Tensor& red, int64_t red_off,
                            Tensor& sumsq) {
  const int world = (int)grad_ptrs.size();
  TORCH_CHECK(world <= 16 && red.scalar_type() == at::kFloat && sumsq.scalar_type() == at::kFloat && lo % 8 == 0 && hi % 8 == 0);
  c10::cuda::CUDAGuard guard(red.device());
  void* g[16];
  for (int i = 0; i < world; ++i) g[i] = reinterpret_cast<void*>(grad_ptrs[i]);
  int r = vlmt_rs_reduce_sumsq(g, reinterpret_cast<void*>(grad_mc), world, lo, hi, red.data_ptr<float>() + red_off, sumsq.data_ptr<float>(),
                               vlmt_status_tensor().data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_rs_reduce_sumsq failed with code ", r);
}
static void adamw_push(const Tensor& red, int64_t red_off, const Tensor& sumsq, double max_norm, const std::vector<int64_t>& param_ptrs,
                       int64_t param_mc, int64_t lo, int64_t hi, Tensor& master, Tensor& m, Tensor& v, int64_t state_off, double lr,
                       double b1, double b2, double eps, double wd, double bc1, double bc2, double grad_scale) {
  const int world = (int)param_ptrs.size();
  TORCH_CHECK(world <= 16 && master.scalar_type() == at::kFloat && m.scalar_type() == v.scalar_type());
  TORCH_CHECK(m.scalar_type() == at::kFloat || m.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(master.device());
  void* p[16];
  for (int i = 0; i < world; ++i) p[i] = reinterpret_cast<void*>(param_ptrs[i]);
  const bool sb = m.scalar_type() == at::kBFloat16;
  const int64_t esz = sb ? 2 : 4;
  int r = vlmt_adamw_push(red.data_ptr<float>() + red_off, sumsq.data_ptr<float>(), (float)max_norm, p, reinterpret_cast<void*>(param_mc),
                          world, lo, hi, master.data_ptr<float>() + state_off, static_cast<char*>(m.data_ptr()) + state_off * esz,
                          static_cast<char*>(v.data_ptr()) + state_off * esz, sb ? 1 : 0, (float)lr, (float)b1, (float)b2, (float)eps,
                          (float)wd, (float)bc1, (float)bc2, (float)grad_scale, vlmt_status_tensor().data_ptr<int>(),
                          at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_adamw_push failed with code ", r);
}

static void peer_sum_rows(const std::vector<int64_t>& partial_ptrs, int64_t row0, const c10::optional<Tensor>& residual, Tensor& out) {
  c10::cuda::CUDAGuard guard(out.device());
  void* p[16];
  const int world = (int)partial_ptrs.size();
  TORCH_CHECK(world <= 16 && out.is_contiguous() && out.scalar_type() == at::kBFloat16);
  for (int i = 0; i < world; ++i) p[i] = reinterpret_cast<void*>(partial_ptrs[i]);
  int r = vlmt_peer_sum_rows(p, world, row0, out.size(0), (int)out.size(1), residual.has_value() ? residual->data_ptr() : nullptr,
                             out.data_ptr(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_peer_sum_rows failed with code ", r);
}

static void fill_ptrs(const std::vector<int64_t>& v, void** out) {
  TORCH_CHECK(v.size() <= 16);
  for (size_t i = 0; i < v.size(); ++i) out[i] = reinterpret_cast<void*>(v[i]);
}
static void signal_peers(const std::vector<int64_t>& flag_ptrs, int64_t my_rank, int64_t epoch) {
  void* f[16];
  fill_ptrs(flag_ptrs, f);
  int r = vlmt_signal_peers(f, (int)flag_ptrs.size(), (int)my_rank, (int)epoch, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_signal_peers failed with code ", r);
}
// flag arrays are addressed as (base pointer, element offset) so one symmetric tensor can hold many flag rows
static void signal_peers_at(const std::vector<int64_t>& flag_ptrs, int64_t elem_offset, int64_t my_rank, int64_t epoch) {
  void* f[16];
  TORCH_CHECK(flag_ptrs.size() <= 16);
  for (size_t i = 0; i < flag_ptrs.size(); ++i) f[i] = reinterpret_cast<void*>(flag_ptrs[i] + elem_offset * 4);
  int r = vlmt_signal_peers(f, (int)flag_ptrs.size(), (int)my_rank, (int)epoch, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_signal_peers failed with code ", r);
}
static void wait_flags(int64_t my_flags, int64_t elem_offset, int64_t world, int64_t epoch, int64_t skip_rank) {
  Tensor st = vlmt_status_tensor();
  int r = vlmt_wait_flags(reinterpret_cast<const int*>(my_flags) + elem_offset, (int)world, (int)epoch, (int)skip_rank, st.data_ptr<int>(),
                          at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_wait_flags failed with code ", r);
}
static void pull_gather(const std::vector<int64_t>& slot_ptrs, Tensor& out, int64_t n_per_rank, int64_t my_flags, int64_t epoch) {
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(out.device());
  void* s[16];
  fill_ptrs(slot_ptrs, s);
  Tensor st = vlmt_status_tensor();
  int r = vlmt_pull_gather(s, out.data_ptr(), n_per_rank, (int)slot_ptrs.size(), reinterpret_cast<const int*>(my_flags), (int)epoch,
                           st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_pull_gather failed with code ", r);
}
static void pull_gather_range(const std::vector<int64_t>& slot_ptrs, Tensor& out, int64_t n_per_rank, int64_t lo, int64_t hi) {
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kBFloat16 && lo >= 0 && hi <= out.numel());
  c10::cuda::CUDAGuard guard(out.device());
  void* s[16];
  fill_ptrs(slot_ptrs, s);
  int r = vlmt_pull_gather_range(s, out.data_ptr(), n_per_rank, (int)slot_ptrs.size(), lo, hi, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_pull_gather_range failed with code ", r);
}
static void pull_reduce(const std::vector<int64_t>& slot_ptrs, Tensor& out, const c10::optional<Tensor>& residual, int64_t n_per_rank,
                        int64_t my_rank, int64_t my_flags, int64_t epoch) {
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(out.device());
  void* s[16];
  fill_ptrs(slot_ptrs, s);
  Tensor st = vlmt_status_tensor();
  int r = vlmt_pull_reduce(s, out.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr, n_per_rank, (int)slot_ptrs.size(),
                           (int)my_rank, reinterpret_cast<const int*>(my_flags), (int)epoch, st.data_ptr<int>(),
                           at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_pull_reduce failed with code ", r);
}

void bind_comm(pybind11::module_& m) {
  m.def("set_flag_wait_ms", [](int64_t ms) {
    int r = vlmt_set_flag_wait_ms((long)ms);
    TORCH_CHECK(r == 0, "vlmt_set_flag_wait_ms failed with code ", r);
  });
  m.def("signal_peers", &signal_peers);
  m.def("signal_peers_at", &signal_peers_at);
  m.def("wait_flags", &wait_flags);
  m.def("pull_gather", &pull_gather);
  m.def("pull_gather_range", &pull_gather_range);
  m.def("pull_reduce", &pull_reduce);
  m.def("fused_rs_adamw_ag", &fused_rs_adamw_ag);
  m.def("rs_reduce_sumsq", &rs_reduce_sumsq);
  m.def("adamw_push", &adamw_push);
  m.def("peer_sum_rows", &peer_sum_rows);
}
