// Bindings of the intra-chunk kernels of the gated delta rule (gdn_chunk_sm100.h).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gdn_chunk_sm100.h"

using torch::Tensor;

torch::Tensor vlmt_status_tensor();

static inline cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

// [T, H, 128] bf16 whose heads are contiguous (stride 128, 1); the token stride is free (a slice of a wider projection)
static void check_tokens(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3 && t.size(2) == 128 && t.stride(2) == 1 && t.stride(1) == 128 &&
                  t.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0,
              name, " must be bf16 [T, H, 128] with contiguous heads and a 16-byte aligned token stride");
}
static void check_stack(const Tensor& t, int64_t H, int64_t N, int64_t rows, int64_t cols, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.dim() == 4 && t.size(0) == H && t.size(1) == N &&
                  t.size(2) == rows && t.size(3) == cols,
              name, " must be a contiguous bf16 [H, N, ", rows, ", ", cols, "] stack");
}
static void check_chunks(const Tensor& c) {
  TORCH_CHECK(c.is_cuda() && c.scalar_type() == at::kInt && c.is_contiguous() && c.dim() == 2 && c.size(1) == 2, "chunks must be int32 [N, 2]");
}

// -> w, u, kdec, qg [H,N,64,128]; P, Tm [H,N,64,64]; gc [H,N,64]; decay [H,N]
static std::vector<Tensor> gdn_prepare_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta,
                                           const Tensor& chunks, double scale, double eps) {
  check_tokens(q, "q"); check_tokens(k, "k"); check_tokens(v, "v"); check_chunks(chunks);
  const int64_t T = q.size(0), H = q.size(1), N = chunks.size(0);
  TORCH_CHECK(k.sizes() == q.sizes() && v.sizes() == q.sizes(), "q, k, v must have the same shape");
  TORCH_CHECK(g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && g.is_contiguous() && beta.is_contiguous() &&
                  g.dim() == 2 && g.size(0) == T && g.size(1) == H && beta.sizes() == g.sizes(), "g, beta must be contiguous fp32 [T, H]");
  c10::cuda::CUDAGuard guard(q.device());
  auto bo = q.options();
  auto fo = q.options().dtype(torch::kFloat);
  Tensor w = torch::empty({H, N, 64, 128}, bo), u = torch::empty({H, N, 64, 128}, bo), kdec = torch::empty({H, N, 64, 128}, bo),
         qg = torch::empty({H, N, 64, 128}, bo), P = torch::empty({H, N, 64, 64}, bo), Tm = torch::empty({H, N, 64, 64}, bo),
         gc = torch::empty({H, N, 64}, fo), decay = torch::empty({H, N}, fo);
  Tensor st = vlmt_status_tensor();
  int r = vlmt_gdn_prepare_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), g.data_ptr<float>(),
                               beta.data_ptr<float>(), chunks.data_ptr<int>(), (int)T, (int)H, (int)N, (float)scale, (float)eps, w.data_ptr(),
                               u.data_ptr(), kdec.data_ptr(), qg.data_ptr(), P.data_ptr(), Tm.data_ptr(), gc.data_ptr<float>(),
                               decay.data_ptr<float>(), st.data_ptr<int>(), cur());
  TORCH_CHECK(r == 0, "vlmt_gdn_prepare_fwd failed with code ", r);
  return {w, u, kdec, qg, P, Tm, gc, decay};
}

// o [T, H, 128]: rows of tokens that belong to no chunk are zero
// `covered`: the chunks cover all T tokens (no trailing tokens outside every document), so nothing needs a zero fill
static Tensor gdn_output_fwd(const Tensor& qg, const Tensor& P, const Tensor& states, const Tensor& vnew, const Tensor& chunks, int64_t T,
                             bool covered) {
  check_chunks(chunks);
  const int64_t H = qg.size(0), N = chunks.size(0);
  check_stack(qg, H, N, 64, 128, "qg"); check_stack(P, H, N, 64, 64, "P"); check_stack(states, H, N, 128, 128, "states");
  check_stack(vnew, H, N, 64, 128, "vnew");
  c10::cuda::CUDAGuard guard(qg.device());
  Tensor o = covered ? torch::empty({T, H, 128}, qg.options()) : torch::zeros({T, H, 128}, qg.options());
  Tensor st = vlmt_status_tensor();
  int r = vlmt_gdn_output_fwd(qg.data_ptr(), P.data_ptr(), states.data_ptr(), vnew.data_ptr(), chunks.data_ptr<int>(), (int)H, (int)N,
                              o.data_ptr(), st.data_ptr<int>(), cur());
  TORCH_CHECK(r == 0, "vlmt_gdn_output_fwd failed with code ", r);
  return o;
}

// -> dqg [H,N,64,128], dP [H,N,64,64], dvnew [H,N,64,128], dstates [H,N,128,128]
static std::vector<Tensor> gdn_output_bwd(const Tensor& dout, const Tensor& qg, const Tensor& P, const Tensor& states, const Tensor& vnew,
                                          const Tensor& chunks) {
  check_tokens(dout, "dout"); check_chunks(chunks);
  const int64_t T = dout.size(0), H = qg.size(0), N = chunks.size(0);
  TORCH_CHECK(dout.size(1) == H, "dout must be [T, H, 128]");
  check_stack(qg, H, N, 64, 128, "qg"); check_stack(P, H, N, 64, 64, "P"); check_stack(states, H, N, 128, 128, "states");
  check_stack(vnew, H, N, 64, 128, "vnew");
  c10::cuda::CUDAGuard guard(qg.device());
  auto bo = qg.options();
  Tensor dqg = torch::empty({H, N, 64, 128}, bo), dP = torch::empty({H, N, 64, 64}, bo), dvn = torch::empty({H, N, 64, 128}, bo),
         dS = torch::empty({H, N, 128, 128}, bo);
  Tensor st = vlmt_status_tensor();
  int r = vlmt_gdn_output_bwd(dout.data_ptr(), dout.stride(0), qg.data_ptr(), P.data_ptr(), states.data_ptr(), vnew.data_ptr(),
                              chunks.data_ptr<int>(), (int)T, (int)H, (int)N, dqg.data_ptr(), dP.data_ptr(), dvn.data_ptr(), dS.data_ptr(),
                              st.data_ptr<int>(), cur());
  TORCH_CHECK(r == 0, "vlmt_gdn_output_bwd failed with code ", r);
  return {dqg, dP, dvn, dS};
}

// -> dq, dk, dv [T, H, 128] bf16; dg, dbeta [T, H] fp32 (zero for tokens that belong to no chunk)
static std::vector<Tensor> gdn_prepare_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& beta, const Tensor& gc,
                                           const Tensor& chunks, double scale, double eps, const Tensor& states, const Tensor& adj,
                                           const Tensor& vnew, const Tensor& du, const Tensor& dqg, const Tensor& dP, const Tensor& P,
                                           const Tensor& Tm, bool covered) {
  check_tokens(q, "q"); check_tokens(k, "k"); check_tokens(v, "v"); check_chunks(chunks);
  const int64_t T = q.size(0), H = q.size(1), N = chunks.size(0);
  check_stack(states, H, N, 128, 128, "states"); check_stack(adj, H, N, 128, 128, "adj"); check_stack(vnew, H, N, 64, 128, "vnew");
  check_stack(du, H, N, 64, 128, "du"); check_stack(dqg, H, N, 64, 128, "dqg"); check_stack(dP, H, N, 64, 64, "dP");
  check_stack(P, H, N, 64, 64, "P"); check_stack(Tm, H, N, 64, 64, "Tm");
  TORCH_CHECK(beta.scalar_type() == at::kFloat && beta.is_contiguous() && gc.scalar_type() == at::kFloat && gc.is_contiguous() &&
                  gc.numel() == H * N * 64, "beta must be fp32 [T, H], gc fp32 [H, N, 64]");
  c10::cuda::CUDAGuard guard(q.device());
  auto bo = q.options();
  auto fo = q.options().dtype(torch::kFloat);
  auto alloc = [&](std::vector<int64_t> shape, const torch::TensorOptions& o) { return covered ? torch::empty(shape, o) : torch::zeros(shape, o); };
  Tensor dq = alloc({T, H, 128}, bo), dk = alloc({T, H, 128}, bo), dv = alloc({T, H, 128}, bo);
  Tensor dg = alloc({T, H}, fo), dbeta = alloc({T, H}, fo);
  Tensor st = vlmt_status_tensor();
  int r = vlmt_gdn_prepare_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), beta.data_ptr<float>(),
                               gc.data_ptr<float>(), chunks.data_ptr<int>(), (int)T, (int)H, (int)N, (float)scale, (float)eps,
                               states.data_ptr(), adj.data_ptr(), vnew.data_ptr(), du.data_ptr(), dqg.data_ptr(), dP.data_ptr(), P.data_ptr(),
                               Tm.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr<float>(), dbeta.data_ptr<float>(),
                               st.data_ptr<int>(), cur());
  TORCH_CHECK(r == 0, "vlmt_gdn_prepare_bwd failed with code ", r);
  return {dq, dk, dv, dg, dbeta};
}

void bind_gdn(pybind11::module_& m) {
  m.def("gdn_prepare_fwd", &gdn_prepare_fwd);
  m.def("gdn_output_fwd", &gdn_output_fwd);
  m.def("gdn_output_bwd", &gdn_output_bwd);
  m.def("gdn_prepare_bwd", &gdn_prepare_bwd);
}
