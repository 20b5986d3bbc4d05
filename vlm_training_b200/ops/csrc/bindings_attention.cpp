// Bindings of the attention kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention_sm100.h"
#include "dsa_attention.h"

using torch::Tensor;
Tensor vlmt_status_tensor();

// [T, H, d] bf16 with unit channel stride; token and head strides multiples of 8 elements, 16-byte aligned base
static void check_heads(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3 && t.stride(2) == 1 && t.stride(1) % 8 == 0 &&
                  t.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              name, " must be bf16 [T, H, d] with unit channel stride and 16-byte aligned head / token strides");
}

static std::vector<Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu, int64_t max_seqlen, bool causal,
                                    double scale) {
  check_heads(q, "q"); check_heads(k, "k"); check_heads(v, "v");
  TORCH_CHECK(cu.scalar_type() == at::kInt && cu.is_cuda() && cu.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  const int T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  TORCH_CHECK(Hq % Hkv == 0 && k.size(2) == D && v.size(2) == D && k.size(0) == T && v.size(0) == T && v.size(1) == Hkv);
  // cu_seqlens must cover [0, T): every row then belongs to exactly one tile and is written by the kernel
  Tensor o = torch::empty({T, Hq, D}, q.options());
  Tensor lse = torch::empty({Hq, T}, q.options().dtype(torch::kFloat));
  Tensor st = vlmt_status_tensor();
  int r = vlmt_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), cu.data_ptr<int>(),
                        (int)cu.numel() - 1, T, Hq, Hkv, D, q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
                        (float)scale, causal, st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_attn_fwd failed with code ", r, " (head_dim ", D, ")");
  (void)max_seqlen;
  return {o, lse};
}

static std::vector<Tensor> attn_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& lse,
                                    const Tensor& cu, int64_t max_seqlen, bool causal, double scale) {
  check_heads(q, "q"); check_heads(k, "k"); check_heads(v, "v");
  TORCH_CHECK(dout.is_contiguous() && o.is_contiguous() && dout.scalar_type() == at::kBFloat16 && dout.sizes() == o.sizes());
  c10::cuda::CUDAGuard guard(q.device());
  const int T = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  Tensor dq = torch::empty({T, Hq, D}, q.options()), dk = torch::empty({T, Hkv, D}, q.options()), dv = torch::empty({T, Hkv, D}, q.options());
  Tensor delta = torch::empty({Hq, T}, q.options().dtype(torch::kFloat));
  Tensor st = vlmt_status_tensor();
  int r = vlmt_attn_bwd(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                        delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr<int>(), (int)cu.numel() - 1, T, Hq,
                        Hkv, D, q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), (float)scale, causal,
                        st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_attn_bwd failed with code ", r);
  (void)max_seqlen;
  return {dq, dk, dv};
}

// selected-key attention of one query block (dsa_attention.h): q [B, Hq, D], k / v [L, Hkv, D], sel [B, kk] int32
torch::Tensor vlmt_status_tensor();

// ``tensor_cores``: the tcgen05 kernel (head size 256, 8 query heads per kv head) instead of the CUDA-core one
static std::vector<Tensor> dsa_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& sel, double scale, bool tensor_cores) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous());
  TORCH_CHECK(sel.scalar_type() == at::kInt && sel.is_cuda() && sel.is_contiguous() && sel.dim() == 2 && sel.size(0) == q.size(0));
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  TORCH_CHECK(Hq % Hkv == 0 && k.size(2) == D && v.sizes() == k.sizes());
  Tensor o = torch::empty_like(q);
  Tensor lse = torch::empty({B, Hq}, q.options().dtype(torch::kFloat));
  if (tensor_cores && D == 256 && Hq / Hkv == 8) {
    Tensor st = vlmt_status_tensor();
    int r = vlmt_dsa_fwd_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), sel.data_ptr<int>(), o.data_ptr(), lse.data_ptr<float>(), B, Hkv,
                            (int)sel.size(1), (float)scale, st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(r == 0, "vlmt_dsa_fwd_tc failed with code ", r);
    return {o, lse};
  }
  int r = vlmt_dsa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), sel.data_ptr<int>(), o.data_ptr(), lse.data_ptr<float>(), B, Hkv, Hq / Hkv,
                       D, (int)sel.size(1), (float)scale, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_dsa_fwd failed with code ", r);
  return {o, lse};
}

// dk / dv are float32 [L, Hkv, D] accumulators owned by the caller (one per document, shared by its query blocks)
static Tensor dsa_bwd(const Tensor& d_o, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& sel, const Tensor& o,
                      const Tensor& lse, Tensor& dk, Tensor& dv, double scale, bool tensor_cores) {
  TORCH_CHECK(d_o.is_contiguous() && q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && o.is_contiguous() && sel.is_contiguous());
  TORCH_CHECK(d_o.scalar_type() == at::kBFloat16 && dk.scalar_type() == at::kFloat && dv.scalar_type() == at::kFloat);
  TORCH_CHECK(dk.is_contiguous() && dv.is_contiguous() && dk.numel() == k.numel() && dv.numel() == v.numel());
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), Hq = q.size(1), D = q.size(2), Hkv = k.size(1);
  Tensor dq = torch::empty({B, Hq, D}, q.options().dtype(torch::kFloat));
  if (tensor_cores && D == 256 && Hq / Hkv == 8) {
    Tensor st = vlmt_status_tensor();
    int r = vlmt_dsa_bwd_tc(q.data_ptr(), k.data_ptr(), v.data_ptr(), sel.data_ptr<int>(), o.data_ptr(), lse.data_ptr<float>(), d_o.data_ptr(),
                            dq.data_ptr<float>(), dk.data_ptr<float>(), dv.data_ptr<float>(), B, Hkv, (int)sel.size(1), (float)scale,
                            st.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(r == 0, "vlmt_dsa_bwd_tc failed with code ", r);
    return dq;
  }
  int r = vlmt_dsa_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), sel.data_ptr<int>(), o.data_ptr(), lse.data_ptr<float>(), d_o.data_ptr(),
                       dq.data_ptr<float>(), dk.data_ptr<float>(), dv.data_ptr<float>(), B, Hkv, Hq / Hkv, D, (int)sel.size(1), (float)scale,
                       at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(r == 0, "vlmt_dsa_bwd failed with code ", r);
  return dq;
}

// indexer scores + top-k of one query block: iq [T, 4, 64] / ik [T, 64] bf16, w [T, 4] fp32; queries are the tokens
// [q_tok0, q_tok0 + B) at document positions q_pos0.., keys the document's tokens from k_tok0.  -> sel int32 [B, kk]
static Tensor dsa_select(const Tensor& iq, const Tensor& ik, const Tensor& w, int64_t q_tok0, int64_t q_pos0, int64_t k_tok0, int64_t B,
                         int64_t kk) {
  TORCH_CHECK(iq.is_cuda() && iq.scalar_type() == at::kBFloat16 && iq.is_contiguous() && iq.dim() == 3 && iq.size(1) == 4 && iq.size(2) == 64,
              "indexer queries must be contiguous bf16 [T, 4, 64]");
  TORCH_CHECK(ik.scalar_type() == at::kBFloat16 && ik.is_contiguous() && ik.dim() == 2 && ik.size(1) == 64 && ik.size(0) == iq.size(0));
  TORCH_CHECK(w.scalar_type() == at::kFloat && w.is_contiguous() && w.dim() == 2 && w.size(1) == 4 && w.size(0) == iq.size(0));
  c10::cuda::CUDAGuard guard(iq.device());
  const int T = iq.size(0);
  const int n_keys = (int)(q_pos0 + B);
  TORCH_CHECK(q_tok0 >= 0 && q_tok0 + B <= T && k_tok0 >= 0 && k_tok0 + n_keys <= T && q_tok0 == k_tok0 + q_pos0, "block outside the row");
  const int ld = (n_keys + 3) & ~3;
  Tensor scores = torch::empty({B, ld}, iq.options().dtype(torch::kFloat));
  Tensor sel = torch::empty({B, kk}, iq.options().dtype(torch::kInt));
  Tensor st = vlmt_status_tensor();
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  int r = vlmt_dsa_index_scores(iq.data_ptr(), ik.data_ptr(), w.data_ptr<float>(), T, (int)q_tok0, (int)q_pos0, (int)k_tok0, (int)B, n_keys,
                                scores.data_ptr<float>(), ld, st.data_ptr<int>(), stream);
  TORCH_CHECK(r == 0, "vlmt_dsa_index_scores failed with code ", r);
  r = vlmt_dsa_topk(scores.data_ptr<float>(), (int)B, ld, (int)q_pos0, (int)kk, sel.data_ptr<int>(), stream);
  TORCH_CHECK(r == 0, "vlmt_dsa_topk failed with code ", r);
  return sel;
}

void bind_attention(pybind11::module_& m) {
  m.def("dsa_select", &dsa_select);
  m.def("dsa_fwd", &dsa_fwd);
  m.def("dsa_bwd", &dsa_bwd);
  m.def("dsa_supported", [](int64_t D, int64_t rep) { return vlmt_dsa_supported((int)D, (int)rep) != 0; });
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
}
