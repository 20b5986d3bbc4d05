// Bindings of the attention kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention_sm100.h"

using torch::Tensor;
Tensor vlmt_status_tensor();

static std::vector<Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu, int64_t max_seqlen, bool causal,
                                    double scale, int64_t d_eff) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 3 && k.dim() == 3 && v.dim() == 3);
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous(), "q, k, v must be contiguous [T, H, D]");
  TORCH_CHECK(cu.scalar_type() == at::kInt && cu.is_cuda() && cu.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  const int T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  TORCH_CHECK(Hq % Hkv == 0 && k.size(2) == D && v.size(2) == D && k.size(0) == T && v.size(0) == T);
  // cu_seqlens must cover [0, T): every row then belongs to exactly one tile and is written by the kernel
  Tensor o = torch::empty_like(q);
  Tensor lse = torch::empty({Hq, T}, q.options().dtype(torch::kFloat));
  Tensor st = vlmt_status_tensor();
  int r = vlmt_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), cu.data_ptr<int>(),
                        (int)cu.numel() - 1, T, Hq, Hkv, D, (int)d_eff, (long)Hq * D, (long)Hkv * D, (long)Hkv * D, (float)scale, causal,
                        st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_attn_fwd failed with code ", r, " (head_dim ", D, ")");
  (void)max_seqlen;
  return {o, lse};
}

static std::vector<Tensor> attn_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& lse,
                                    const Tensor& cu, int64_t max_seqlen, bool causal, double scale, int64_t d_eff) {
  TORCH_CHECK(dout.is_contiguous() && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && o.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  const int T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  Tensor dq = torch::empty_like(q), dk = torch::empty_like(k), dv = torch::empty_like(v);
  Tensor delta = torch::empty({Hq, T}, q.options().dtype(torch::kFloat));
  Tensor st = vlmt_status_tensor();
  int r = vlmt_attn_bwd(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                        delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr<int>(), (int)cu.numel() - 1, T, Hq,
                        Hkv, D, (int)d_eff, (float)scale, causal, st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_attn_bwd failed with code ", r);
  (void)max_seqlen;
  return {dq, dk, dv};
}

void bind_attention(pybind11::module_& m) {
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
}
