// pybind11 bindings: thin tensor -> raw-pointer shims over the C launchers.  All kernels run on
// the current CUDA stream of the tensors' device.  Shape/dtype validation lives here so the
// kernels can assume their contracts.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "elementwise.h"
#include "gdn_scan_sm100.h"
#include "gemm_sm100.h"
#include "loss_optim.h"

namespace {
using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
inline void check_contig(const Tensor& t, const char* name) { TORCH_CHECK(t.is_contiguous(), name, " must be contiguous"); }
inline const void* optptr(const c10::optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) g_num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return g_num_sms;
}

// One int32 status word per device; kernels with bounded waits write a code here when they give up.
Tensor g_status[16];
Tensor status_tensor() {
  int dev = at::cuda::current_device();
  if (!g_status[dev].defined()) g_status[dev] = torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev));
  return g_status[dev];
}

// ------------------------------------------------------------------ GEMM
// out[M,N] (+)= a * b^T (see gemm_sm100.h for the layout flags)
void gemm(const Tensor& a, const Tensor& b, Tensor& out, bool a_mn, bool b_mn, const c10::optional<Tensor>& bias, int64_t epilogue,
          bool accumulate) {
  check_bf16(a, "a"); check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2);
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "innermost strides must be 1");
  c10::cuda::CUDAGuard guard(a.device());
  const int M = a_mn ? a.size(1) : a.size(0);
  const int K = a_mn ? a.size(0) : a.size(1);
  const int N = b_mn ? b.size(1) : b.size(0);
  const int Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(out.size(0) == M && out.size(1) == N, "bad output shape");
  void* d_bf16 = nullptr; float* d_f32 = nullptr;
  if (out.scalar_type() == at::kFloat) d_f32 = out.data_ptr<float>();
  else { check_bf16(out, "out"); d_bf16 = out.data_ptr(); }
  if (bias.has_value()) { check_bf16(*bias, "bias"); TORCH_CHECK(bias->numel() == N); }
  Tensor st = status_tensor();
  int r = vlmt_gemm_bf16(a.data_ptr(), b.data_ptr(), d_bf16, d_f32, optptr(bias), M, N, K, (int)a.stride(0), (int)b.stride(0),
                         (int)out.stride(0), a_mn, b_mn, (int)epilogue, accumulate, st.data_ptr<int>(), num_sms(), cur_stream());
  TORCH_CHECK(r == 0, "vlmt_gemm_bf16 failed with code ", r);
}

// y-partials of a row-parallel linear pushed to their owners: rows [o*R, (o+1)*R) of a @ b^T go to dst_ptrs[o]
void gemm_rs_push(const Tensor& a, const Tensor& b, const std::vector<int64_t>& dst_ptrs, int64_t rows_per_rank, bool b_mn) {
  check_bf16(a, "a"); check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == (b_mn ? b.size(0) : b.size(1)));
  c10::cuda::CUDAGuard guard(a.device());
  void* dst[8];
  TORCH_CHECK(dst_ptrs.size() <= 8);
  for (size_t i = 0; i < dst_ptrs.size(); ++i) dst[i] = reinterpret_cast<void*>(dst_ptrs[i]);
  Tensor st = status_tensor();
  const int M = a.size(0), N = b_mn ? b.size(1) : b.size(0), K = a.size(1);
  int r = vlmt_gemm_bf16_rs_push(a.data_ptr(), b.data_ptr(), dst, (int)dst_ptrs.size(), (int)rows_per_rank, M, N, K, (int)a.stride(0),
                                 (int)b.stride(0), N, b_mn ? 1 : 0, st.data_ptr<int>(), num_sms(), cur_stream());
  TORCH_CHECK(r == 0, "vlmt_gemm_bf16_rs_push failed with code ", r);
}

// all-gather fused into the GEMM: out[world * R, N] = gather(x_local) @ op(b); x_full is this rank's [world * R, K] gathered
// buffer (symmetric memory; full_ptrs[r] is its address on rank r), flag_ptrs[r] rank r's flag array, flags_elem_offset the
// row of the flag arrays that this collective uses
void gemm_ag(const Tensor& x_local, Tensor& x_full, const Tensor& b, Tensor& out, const std::vector<int64_t>& full_ptrs,
             const std::vector<int64_t>& flag_ptrs, int64_t flags_elem_offset, Tensor& counter, int64_t epoch, int64_t rank, bool b_mn) {
  check_bf16(x_local, "x_local"); check_bf16(x_full, "x_full"); check_bf16(b, "b"); check_bf16(out, "out");
  check_contig(x_local, "x_local"); check_contig(x_full, "x_full");
  TORCH_CHECK(x_local.dim() == 2 && x_full.dim() == 2 && b.dim() == 2 && out.dim() == 2 && b.stride(1) == 1 && out.stride(1) == 1);
  const int world = (int)full_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && flag_ptrs.size() == full_ptrs.size() && rank >= 0 && rank < world);
  const int R = x_local.size(0), K = x_local.size(1);
  const int N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK(x_full.size(0) == (int64_t)R * world && x_full.size(1) == K && (b_mn ? b.size(0) : b.size(1)) == K, "gemm_ag: bad shapes");
  TORCH_CHECK(out.size(0) == x_full.size(0) && out.size(1) == N, "gemm_ag: bad output shape");
  TORCH_CHECK(full_ptrs[rank] == reinterpret_cast<int64_t>(x_full.data_ptr()), "gemm_ag: full_ptrs[rank] must be x_full");
  TORCH_CHECK(counter.scalar_type() == at::kInt && counter.is_cuda() && counter.numel() >= 1);
  c10::cuda::CUDAGuard guard(x_local.device());
  void* full[8];
  void* flg[8];
  for (int i = 0; i < world; ++i) {
    full[i] = reinterpret_cast<void*>(full_ptrs[i]);
    flg[i] = reinterpret_cast<void*>(flag_ptrs[i] + flags_elem_offset * 4);
  }
  Tensor st = status_tensor();
  int r = vlmt_gemm_bf16_ag(x_local.data_ptr(), x_full.data_ptr(), b.data_ptr(), out.data_ptr(), full, flg,
                            reinterpret_cast<const int*>(flag_ptrs[rank] + flags_elem_offset * 4),
                            reinterpret_cast<unsigned*>(counter.data_ptr<int>()), (int)epoch, world, (int)rank, R, N, K, (int)b.stride(0),
                            (int)out.stride(0), b_mn ? 1 : 0, st.data_ptr<int>(), num_sms(), cur_stream());
  TORCH_CHECK(r == 0, "vlmt_gemm_bf16_ag failed with code ", r);
}

// Y = X W^T (+ bias) with the weight's all-gather inside the kernel: `w` is the [N, K] view of the weight inside the local
// whole bucket `bucket` (flat bf16), `shard_ptrs` the shard base of every rank, `sync` an int32 tensor of 2 * world entries
// (flags, then counters; zero before the first use), `epoch` growing with every call that shares `sync`.
void gemm_wgather(const Tensor& x, const Tensor& w, Tensor& out, const c10::optional<Tensor>& bias, Tensor& bucket,
                  const std::vector<int64_t>& shard_ptrs, int64_t shard, int64_t rank, Tensor& sync, int64_t epoch) {
  check_bf16(x, "x"); check_bf16(w, "w"); check_bf16(out, "out"); check_bf16(bucket, "bucket");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && w.is_contiguous() && out.stride(1) == 1 &&
              bucket.is_contiguous());
  const int world = (int)shard_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world && sync.scalar_type() == at::kInt && sync.is_cuda() &&
              sync.numel() >= 2 * world);
  const int M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == M && out.size(1) == N, "gemm_wgather: bad shapes");
  const int64_t w_lo = (reinterpret_cast<char*>(w.data_ptr()) - reinterpret_cast<char*>(bucket.data_ptr())) / 2;
  TORCH_CHECK(w_lo >= 0 && w_lo + (int64_t)N * K <= bucket.numel() && shard * world >= bucket.numel(), "gemm_wgather: the weight is not inside the bucket");
  c10::cuda::CUDAGuard guard(x.device());
  const void* sp[8];
  for (int i = 0; i < world; ++i) sp[i] = reinterpret_cast<const void*>(shard_ptrs[i]);
  Tensor st = status_tensor();
  int r = vlmt_gemm_bf16_wgather(x.data_ptr(), out.data_ptr(), optptr(bias), M, N, K, (int)x.stride(0), (int)out.stride(0), bucket.data_ptr(),
                                 (long)w_lo, sp, (long)shard, world, (int)rank, sync.data_ptr<int>(),
                                 reinterpret_cast<unsigned*>(sync.data_ptr<int>() + world), (int)epoch, st.data_ptr<int>(), num_sms(),
                                 cur_stream());
  TORCH_CHECK(r == 0, "vlmt_gemm_bf16_wgather failed with code ", r);
}

// grouped GEMM over padded row groups (see gemm_sm100.h); prefix: int32 device tensor [groups + 1]
void gemm_grouped(const Tensor& a, const Tensor& b, Tensor& out, const Tensor& prefix, int64_t mode, bool b_mn) {
  check_bf16(a, "a"); check_bf16(b, "b"); check_bf16(out, "out");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(prefix.scalar_type() == at::kInt && prefix.is_cuda() && prefix.is_contiguous());
  c10::cuda::CUDAGuard guard(a.device());
  const int groups = (int)prefix.numel() - 1;
  int M, N, K;
  bool a_mn = false;
  if (mode == 1) {           // out[cap, N] = a[cap, K] x B_g
    M = a.size(0); K = a.size(1);
    N = b_mn ? b.size(1) : b.size(0) / groups;
    TORCH_CHECK((b_mn ? b.size(0) / groups : b.size(1)) == K, "contraction sizes differ");
    TORCH_CHECK(out.size(0) == M && out.size(1) == N, "bad output shape");
  } else {                   // out[g * M + m, n] = sum_rows a[row, m] b[row, n]
    a_mn = true; b_mn = true;
    K = a.size(0); M = a.size(1); N = b.size(1);
    TORCH_CHECK(b.size(0) == K && out.size(0) == (int64_t)M * groups && out.size(1) == N, "bad shapes");
  }
  Tensor st = status_tensor();
  int r = vlmt_gemm_bf16_grouped(a.data_ptr(), b.data_ptr(), out.data_ptr(), prefix.data_ptr<int>(), groups, (int)mode, M, N, K,
                                 (int)a.stride(0), (int)b.stride(0), (int)out.stride(0), a_mn, b_mn, st.data_ptr<int>(), num_sms(),
                                 cur_stream());
  TORCH_CHECK(r == 0, "vlmt_gemm_bf16_grouped failed with code ", r);
}

// chunk-to-chunk scan of the gated delta rule (gdn_scan_sm100.h); ranges: int32 device tensor [n_docs, 2]
std::vector<Tensor> gdn_scan(const Tensor& x1, const Tensor& x2, const Tensor& e, const Tensor& decay, const c10::optional<Tensor>& ext,
                             const Tensor& ranges, bool reverse, bool head_major) {
  check_bf16(x1, "x1"); check_bf16(x2, "x2"); check_bf16(e, "e");
  check_contig(x1, "x1"); check_contig(x2, "x2"); check_contig(e, "e"); check_contig(decay, "decay");
  TORCH_CHECK(x1.dim() == 4 && x1.size(2) == 64 && x1.size(3) == 128 && x2.sizes() == x1.sizes() && e.sizes() == x1.sizes(),
              "gdn_scan: operands must be [chunks, heads, 64, 128] (or [heads, chunks, 64, 128])");
  TORCH_CHECK(decay.scalar_type() == at::kFloat && decay.numel() == x1.size(0) * x1.size(1), "gdn_scan: decay must be fp32, one value per (chunk, head)");
  TORCH_CHECK(ranges.scalar_type() == at::kInt && ranges.is_cuda() && ranges.is_contiguous() && ranges.dim() == 2 && ranges.size(1) == 2);
  c10::cuda::CUDAGuard guard(x1.device());
  const int N = (int)x1.size(head_major ? 1 : 0), H = (int)x1.size(head_major ? 0 : 1);
  Tensor y = at::empty_like(e);
  Tensor states = at::empty({x1.size(0), x1.size(1), 128, 128}, x1.options());
  const void* extp = nullptr;
  if (ext.has_value()) {
    check_bf16(*ext, "ext"); check_contig(*ext, "ext");
    TORCH_CHECK(ext->sizes() == states.sizes(), "gdn_scan: ext must be [chunks, heads, 128, 128]");
    extp = ext->data_ptr();
  }
  Tensor st = status_tensor();
  int r = vlmt_gdn_scan(x1.data_ptr(), x2.data_ptr(), e.data_ptr(), decay.data_ptr<float>(), extp, y.data_ptr(), states.data_ptr(),
                        ranges.data_ptr<int>(), (int)ranges.size(0), N, H, head_major ? 1 : 0, reverse ? 1 : 0, st.data_ptr<int>(), cur_stream());
  TORCH_CHECK(r == 0, "vlmt_gdn_scan failed with code ", r);
  return {y, states};
}

// ------------------------------------------------------------------ norms
std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& res, const Tensor& w, double eps, bool offset) {
  check_bf16(x, "x"); check_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const int rows = x.numel() / D;
  TORCH_CHECK(D % 8 == 0, "last dim must be a multiple of 8");
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(torch::kFloat));
  Tensor r_out;
  if (res.has_value()) { check_bf16(*res, "residual"); check_contig(*res, "residual"); r_out = torch::empty_like(x); }
  const bool w32 = w.scalar_type() == at::kFloat;
  vlmt_rmsnorm_fwd(x.data_ptr(), optptr(res), w.data_ptr(), w32, y.data_ptr(), res.has_value() ? r_out.data_ptr() : nullptr,
                   rstd.data_ptr<float>(), rows, D, (float)eps, offset, cur_stream());
  if (res.has_value()) return {y, rstd, r_out};
  return {y, rstd};
}
// column sums of the per-block partial rows [blocks, D] (one small kernel; the order of the additions is fixed)
static Tensor sum_partials(const Tensor& partial) {
  Tensor out = torch::empty({partial.size(1)}, partial.options());
  vlmt_sum_rows_f32(partial.data_ptr<float>(), (int)partial.size(0), (int)partial.size(1), out.data_ptr<float>(), cur_stream());
  return out;
}
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, const c10::optional<Tensor>& dres,
                                bool offset) {
  check_bf16(dy, "dy"); check_contig(dy, "dy"); check_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const int rows = x.numel() / D;
  Tensor dx = torch::empty_like(x);
  const int blocks = vlmt_norm_blocks(rows);
  Tensor partial = torch::empty({blocks, D}, x.options().dtype(torch::kFloat));
  if (dres.has_value()) check_contig(*dres, "dres");
  vlmt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), w.scalar_type() == at::kFloat, rstd.data_ptr<float>(), optptr(dres),
                   dx.data_ptr(), partial.data_ptr<float>(), rows, D, offset, cur_stream());
  return {dx, sum_partials(partial)};
}
std::vector<Tensor> layernorm_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& b, double eps) {
  check_bf16(x, "x"); check_contig(x, "x"); check_bf16(w, "w");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const int rows = x.numel() / D;
  TORCH_CHECK(D % 8 == 0);
  Tensor y = torch::empty_like(x);
  Tensor mean = torch::empty({rows}, x.options().dtype(torch::kFloat)), rstd = torch::empty_like(mean);
  vlmt_layernorm_fwd(x.data_ptr(), w.data_ptr(), optptr(b), y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, D,
                     (float)eps, cur_stream());
  return {y, mean, rstd};
}
std::vector<Tensor> layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& mean, const Tensor& rstd) {
  check_contig(dy, "dy"); check_contig(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const int rows = x.numel() / D;
  Tensor dx = torch::empty_like(x);
  const int blocks = vlmt_norm_blocks(rows);
  Tensor pw = torch::empty({blocks, D}, x.options().dtype(torch::kFloat)), pb = torch::empty_like(pw);
  vlmt_layernorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr(),
                     pw.data_ptr<float>(), pb.data_ptr<float>(), rows, D, cur_stream());
  return {dx, sum_partials(pw), sum_partials(pb)};
}
std::vector<Tensor> rmsnorm_gated_fwd(const Tensor& x, const Tensor& z, const Tensor& w, double eps) {
  check_bf16(x, "x"); check_contig(x, "x"); check_contig(z, "z"); check_bf16(w, "w");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const int rows = x.numel() / D;
  Tensor y = torch::empty_like(x);
  Tensor rstd = torch::empty({rows}, x.options().dtype(torch::kFloat));
  vlmt_rmsnorm_gated_fwd(x.data_ptr(), z.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, D, (float)eps, cur_stream());
  return {y, rstd};
}
std::vector<Tensor> rmsnorm_gated_bwd(const Tensor& dy, const Tensor& x, const Tensor& z, const Tensor& w, const Tensor& rstd) {
  check_contig(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1);
  const int rows = x.numel() / D;
  Tensor dx = torch::empty_like(x), dz = torch::empty_like(x);
  const int blocks = vlmt_norm_blocks(rows);
  Tensor pw = torch::empty({blocks, D}, x.options().dtype(torch::kFloat));
  vlmt_rmsnorm_gated_bwd(dy.data_ptr(), x.data_ptr(), z.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dz.data_ptr(),
                         pw.data_ptr<float>(), rows, D, cur_stream());
  return {dx, dz, sum_partials(pw)};
}

// ------------------------------------------------------------------ activations
Tensor swiglu_fwd(const Tensor& gu) {
  check_bf16(gu, "gate_up"); check_contig(gu, "gate_up");
  c10::cuda::CUDAGuard guard(gu.device());
  const int I = gu.size(-1) / 2;
  TORCH_CHECK(I % 8 == 0);
  auto shape = gu.sizes().vec();
  shape.back() = I;
  Tensor out = torch::empty(shape, gu.options());
  vlmt_swiglu_fwd(gu.data_ptr(), out.data_ptr(), gu.numel() / (2 * I), I, cur_stream());
  return out;
}
Tensor swiglu_bwd(const Tensor& dout, const Tensor& gu) {
  check_contig(dout, "dout");
  c10::cuda::CUDAGuard guard(gu.device());
  const int I = gu.size(-1) / 2;
  Tensor dgu = torch::empty_like(gu);
  vlmt_swiglu_bwd(dout.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.numel() / (2 * I), I, cur_stream());
  return dgu;
}
Tensor sigmoid_mul_fwd(const Tensor& x, const Tensor& gate) {
  check_bf16(x, "x"); check_contig(x, "x"); check_contig(gate, "gate");
  TORCH_CHECK(x.numel() == gate.numel() && x.numel() % 8 == 0);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = torch::empty_like(x);
  vlmt_sigmoid_mul_fwd(x.data_ptr(), gate.data_ptr(), out.data_ptr(), x.numel(), cur_stream());
  return out;
}
std::vector<Tensor> sigmoid_mul_bwd(const Tensor& dout, const Tensor& x, const Tensor& gate) {
  check_contig(dout, "dout");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x), dg = torch::empty_like(gate);
  vlmt_sigmoid_mul_bwd(dout.data_ptr(), x.data_ptr(), gate.data_ptr(), dx.data_ptr(), dg.data_ptr(), x.numel(), cur_stream());
  return {dx, dg};
}
Tensor gelu_fwd(const Tensor& x, bool tanh_approx) {
  check_bf16(x, "x"); check_contig(x, "x");
  TORCH_CHECK(x.numel() % 8 == 0);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  vlmt_gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), tanh_approx, cur_stream());
  return y;
}
Tensor gelu_bwd(const Tensor& dy, const Tensor& x, bool tanh_approx) {
  check_contig(dy, "dy");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = torch::empty_like(x);
  vlmt_gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), tanh_approx, cur_stream());
  return dx;
}

// ------------------------------------------------------------------ qkv prep
std::vector<Tensor> qkv_norm_rope_fwd(const Tensor& qkv, int64_t n_q, int64_t n_kv, int64_t D, const c10::optional<Tensor>& qw,
                                      const c10::optional<Tensor>& kw, const Tensor& cosv, const Tensor& sinv, double eps, bool offset,
                                      bool gated) {
  check_bf16(qkv, "qkv"); check_contig(qkv, "qkv");
  TORCH_CHECK(cosv.scalar_type() == at::kFloat && cosv.is_contiguous() && sinv.is_contiguous());
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  const int R = cosv.size(-1);
  TORCH_CHECK(qkv.size(1) == (n_q * (gated ? 2 : 1) + 2 * n_kv) * D, "fused qkv width mismatch");
  auto o = qkv.options();
  Tensor q = torch::empty({T, n_q, D}, o), k = torch::empty({T, n_kv, D}, o), v = torch::empty({T, n_kv, D}, o);
  Tensor gate = gated ? torch::empty({T, n_q * D}, o) : Tensor();
  Tensor rstd = torch::empty({T, n_q + n_kv}, o.dtype(torch::kFloat));
  int r = vlmt_qkv_norm_rope_fwd(qkv.data_ptr(), optptr(qw), optptr(kw), cosv.data_ptr<float>(), sinv.data_ptr<float>(), q.data_ptr(),
                                 k.data_ptr(), v.data_ptr(), gated ? gate.data_ptr() : nullptr, rstd.data_ptr<float>(), T, n_q, n_kv, D, R,
                                 (float)eps, offset, gated, qw.has_value(), cur_stream());
  TORCH_CHECK(r == 0, "qkv_norm_rope: unsupported head_dim / rotary_dim combination (D=", D, ", R=", R, ")");
  if (gated) return {q, k, v, rstd, gate};
  return {q, k, v, rstd};
}
std::vector<Tensor> qkv_norm_rope_bwd(const Tensor& dq, const Tensor& dk, const Tensor& dv, const c10::optional<Tensor>& dgate,
                                      const Tensor& qkv, const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw,
                                      const Tensor& cosv, const Tensor& sinv, const Tensor& rstd, int64_t n_q, int64_t n_kv, int64_t D,
                                      bool offset, bool gated) {
  check_contig(dq, "dq"); check_contig(dk, "dk"); check_contig(dv, "dv");
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = qkv.size(0);
  const int R = cosv.size(-1);
  Tensor dqkv = torch::empty_like(qkv);
  const int blocks = vlmt_qkv_blocks((long)T * (n_q + 2 * n_kv));
  Tensor partial = torch::empty({blocks, 2, D}, qkv.options().dtype(torch::kFloat));
  int r = vlmt_qkv_norm_rope_bwd(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), optptr(dgate), qkv.data_ptr(), optptr(qw), optptr(kw),
                                 cosv.data_ptr<float>(), sinv.data_ptr<float>(), rstd.data_ptr<float>(), dqkv.data_ptr(),
                                 partial.data_ptr<float>(), T, n_q, n_kv, D, R, offset, gated, qw.has_value(), cur_stream());
  TORCH_CHECK(r >= 0, "qkv_norm_rope_bwd failed");
  Tensor dw = sum_partials(partial.view({blocks, 2 * D})).view({2, D});
  return {dqkv, dw[0], dw[1]};
}
// generic rotary on a strided [S, H, D] view -> contiguous [S, H, Dout>=D] (zero padded when Dout > D)
Tensor rope_generic(const Tensor& x, const Tensor& cosv, const Tensor& sinv, bool transpose, int64_t d_out) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 3 && x.stride(2) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  const int S = x.size(0), H = x.size(1), D = x.size(2);
  Tensor out = d_out > D ? torch::zeros({S, H, d_out}, x.options()) : torch::empty({S, H, D}, x.options());
  vlmt_rope_generic(x.data_ptr(), x.stride(0), x.stride(1), cosv.data_ptr<float>(), sinv.data_ptr<float>(), out.data_ptr(), out.stride(0),
                    out.stride(1), S, H, D, transpose, cur_stream());
  return out;
}

// ------------------------------------------------------------------ GDN glue
std::vector<Tensor> gdn_gates_fwd(const Tensor& a, const Tensor& b, const Tensor& A_log, const Tensor& dt_bias) {
  check_bf16(a, "a"); check_bf16(b, "b");
  TORCH_CHECK(a.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && a.stride(0) == b.stride(0));
  TORCH_CHECK(A_log.scalar_type() == at::kFloat && dt_bias.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(a.device());
  const long T = a.size(0);
  const int H = a.size(1);
  Tensor g = torch::empty({T, H}, a.options().dtype(torch::kFloat));
  Tensor beta = torch::empty({T, H}, a.options());
  vlmt_gdn_gates_fwd(a.data_ptr(), b.data_ptr(), a.stride(0), A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), g.data_ptr<float>(),
                     beta.data_ptr(), T, H, cur_stream());
  return {g, beta};
}
std::vector<Tensor> gdn_gates_bwd(const Tensor& dg, const Tensor& dbeta, const Tensor& a, const Tensor& b, const Tensor& A_log,
                                  const Tensor& dt_bias) {
  c10::cuda::CUDAGuard guard(a.device());
  const long T = a.size(0);
  const int H = a.size(1);
  Tensor dgc = dg.contiguous().to(torch::kFloat), dbc = dbeta.contiguous();
  Tensor da = torch::empty({T, H}, a.options()), db = torch::empty({T, H}, a.options());
  Tensor partial = torch::zeros({148 * 2, 2, H}, a.options().dtype(torch::kFloat));
  int grid = vlmt_gdn_gates_bwd(dgc.data_ptr<float>(), dbc.data_ptr(), a.data_ptr(), b.data_ptr(), a.stride(0), A_log.data_ptr<float>(),
                                dt_bias.data_ptr<float>(), da.data_ptr(), db.data_ptr(), H, partial.data_ptr<float>(), T, H, cur_stream());
  Tensor s = partial.narrow(0, 0, grid).sum(0);
  return {da, db, s[0], s[1]};
}
Tensor conv1d_silu_fwd(const Tensor& x, const Tensor& w, const Tensor& seq_idx) {
  check_bf16(x, "x"); check_bf16(w, "w");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && w.is_contiguous() && seq_idx.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), C = x.size(1), K = w.size(1);
  TORCH_CHECK(x.stride(0) % 8 == 0);
  Tensor y = torch::empty({T, C}, x.options());
  int r = vlmt_conv1d_silu_fwd(x.data_ptr(), x.stride(0), w.data_ptr(), seq_idx.data_ptr<int>(), y.data_ptr(), C, T, C, K, cur_stream());
  TORCH_CHECK(r == 0, "conv1d_silu: unsupported kernel size or channel count");
  return y;
}
std::vector<Tensor> conv1d_silu_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& seq_idx) {
  TORCH_CHECK(dy.stride(1) == 1 && x.stride(1) == 1);
  c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), C = x.size(1), K = w.size(1);
  Tensor dx = torch::empty({T, C}, x.options());
  const int slabs = vlmt_conv1d_bwd_slabs(T);
  Tensor partial = torch::zeros({slabs, C, K}, x.options().dtype(torch::kFloat));
  int r = vlmt_conv1d_silu_bwd(dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), seq_idx.data_ptr<int>(), dx.data_ptr(), C,
                               partial.data_ptr<float>(), T, C, K, cur_stream());
  TORCH_CHECK(r == 0);
  return {dx, partial.sum(0)};
}

// ------------------------------------------------------------------ rows
void rows_update(Tensor& out, const Tensor& index, const Tensor& src, bool add) {
  check_bf16(out, "out"); check_contig(out, "out"); check_contig(src, "src");
  TORCH_CHECK(index.scalar_type() == at::kLong && out.size(-1) % 8 == 0);
  c10::cuda::CUDAGuard guard(out.device());
  vlmt_rows_update(out.data_ptr(), index.data_ptr<long>(), src.data_ptr(), index.numel(), out.size(-1), add, cur_stream());
}
Tensor rows_gather(const Tensor& src, const Tensor& index) {
  check_bf16(src, "src"); check_contig(src, "src");
  c10::cuda::CUDAGuard guard(src.device());
  Tensor dst = torch::empty({index.numel(), src.size(-1)}, src.options());
  vlmt_rows_gather(dst.data_ptr(), index.data_ptr<long>(), src.data_ptr(), index.numel(), src.size(-1), cur_stream());
  return dst;
}

// ------------------------------------------------------------------ loss / optimizer
Tensor ce_fwd_bwd_(Tensor& logits, const Tensor& targets, double grad_scale, int64_t ignore_index) {
  check_bf16(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && targets.scalar_type() == at::kLong && targets.is_contiguous());
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor loss = torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat));
  vlmt_ce_fwd_bwd(logits.data_ptr(), logits.stride(0), targets.data_ptr<long>(), loss.data_ptr<float>(), (float)grad_scale,
                  (int)logits.size(0), (int)logits.size(1), ignore_index, cur_stream());
  return loss;
}
void adamw_(Tensor& grad, Tensor& master, Tensor& m, Tensor& v, c10::optional<Tensor> param, double lr, double b1, double b2,
            double eps, double wd, int64_t step, double grad_scale, bool zero_grad) {
  TORCH_CHECK(master.scalar_type() == at::kFloat && m.scalar_type() == v.scalar_type());
  TORCH_CHECK(m.scalar_type() == at::kFloat || m.scalar_type() == at::kBFloat16, "Adam moments must be fp32 or bf16");
  TORCH_CHECK(grad.is_contiguous() && master.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  c10::cuda::CUDAGuard guard(master.device());
  const double bc1 = 1.0 - std::pow(b1, (double)step), bc2 = 1.0 - std::pow(b2, (double)step);
  vlmt_adamw(grad.data_ptr(), grad.scalar_type() == at::kFloat, master.data_ptr<float>(), m.data_ptr(), v.data_ptr(),
             m.scalar_type() == at::kBFloat16, param.has_value() ? param->data_ptr() : nullptr, master.numel(), (float)lr, (float)b1, (float)b2, (float)eps, (float)wd,
             (float)bc1, (float)bc2, (float)grad_scale, zero_grad ? 1 : 0, cur_stream());
}
void sumsq_(const Tensor& x, Tensor& out) {
  c10::cuda::CUDAGuard guard(x.device());
  vlmt_sumsq(x.data_ptr(), x.scalar_type() == at::kFloat, x.numel(), out.data_ptr<float>(), cur_stream());
}

// column sums of a 2-D bf16 tensor in fp32 (bias gradients)
Tensor colsum(const Tensor& x) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.size(1) % 8 == 0 && x.stride(0) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, "colsum: bf16 [rows, cols], cols and row stride multiples of 8");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = x.size(0), cols = x.size(1);
  Tensor partial = torch::empty({vlmt_colsum_slabs(rows), cols}, x.options().dtype(torch::kFloat));
  Tensor out = torch::empty({cols}, x.options().dtype(torch::kFloat));
  vlmt_colsum(x.data_ptr(), x.stride(0), rows, cols, partial.data_ptr<float>(), out.data_ptr<float>(), cur_stream());
  return out;
}

Tensor status() { return status_tensor(); }

}  // namespace

// shared with the other binding translation units
torch::Tensor vlmt_status_tensor() { return status_tensor(); }

void bind_attention(pybind11::module_& m);
void bind_comm(pybind11::module_& m);
void bind_moe(pybind11::module_& m);
void bind_gdn(pybind11::module_& m);
void bind_fp8(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("memset_zero_", [](Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "memset_zero_: a contiguous CUDA tensor is required");
    c10::cuda::CUDAGuard guard(t.device());
    cudaError_t e = cudaMemsetAsync(t.data_ptr(), 0, (size_t)t.numel() * t.element_size(), cur_stream());
    TORCH_CHECK(e == cudaSuccess, "cudaMemsetAsync failed: ", cudaGetErrorString(e));
  });
  m.def("gemm_rs_push", &gemm_rs_push);
  m.def("gemm_ag", &gemm_ag);
  m.def("gemm_wgather", &gemm_wgather);
  m.def("gemm_set_flag_wait_ms", [](int64_t ms) {
    int r = vlmt_gemm_set_flag_wait_ms((long)ms);
    TORCH_CHECK(r == 0, "vlmt_gemm_set_flag_wait_ms failed with code ", r);
  });
  m.def("gemm_grouped", &gemm_grouped);
  m.def("gdn_scan", &gdn_scan);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("rmsnorm_gated_fwd", &rmsnorm_gated_fwd);
  m.def("rmsnorm_gated_bwd", &rmsnorm_gated_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("sigmoid_mul_fwd", &sigmoid_mul_fwd);
  m.def("sigmoid_mul_bwd", &sigmoid_mul_bwd);
  m.def("gelu_fwd", &gelu_fwd);
  m.def("gelu_bwd", &gelu_bwd);
  m.def("qkv_norm_rope_fwd", &qkv_norm_rope_fwd);
  m.def("qkv_norm_rope_bwd", &qkv_norm_rope_bwd);
  m.def("rope_generic", &rope_generic);
  m.def("gdn_gates_fwd", &gdn_gates_fwd);
  m.def("gdn_gates_bwd", &gdn_gates_bwd);
  m.def("conv1d_silu_fwd", &conv1d_silu_fwd);
  m.def("conv1d_silu_bwd", &conv1d_silu_bwd);
  m.def("rows_update", &rows_update);
  m.def("rows_gather", &rows_gather);
  m.def("ce_fwd_bwd_", &ce_fwd_bwd_);
  m.def("adamw_", &adamw_);
  m.def("sumsq_", &sumsq_);
  m.def("colsum", &colsum);
  m.def("status", &status);
  bind_attention(m);
  bind_comm(m);
  bind_moe(m);
  bind_gdn(m);
  bind_fp8(m);
}
