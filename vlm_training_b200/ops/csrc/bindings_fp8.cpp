// Bindings of the FP8 training path (fp8_sm100.h): tensor-wise dynamic quantisation and the FP8 GEMM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "fp8_sm100.h"

using torch::Tensor;

torch::Tensor vlmt_status_tensor();

static inline cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

static int sm_count() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }

// x: bf16 [rows, cols] (unit inner stride).  -> (q [rows, cols] uint8 or empty, q^T [cols, rows rounded up to 16] uint8 or
// empty, rec [2] float: max |x| and the factor that undoes the scaling)
static std::vector<Tensor> fp8_quantize(const Tensor& x, int64_t format, bool want_rm, bool want_t) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "fp8_quantize: x must be bf16 [rows, cols]");
  TORCH_CHECK(x.size(1) % 16 == 0 && x.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0,
              "fp8_quantize: cols must be a multiple of 16 and rows 16-byte aligned");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), cols = x.size(1), rows_pad = (rows + 15) / 16 * 16;
  auto bo = x.options().dtype(torch::kUInt8);
  Tensor rec = torch::empty({2}, x.options().dtype(torch::kFloat));
  Tensor rm = want_rm ? torch::empty({rows, cols}, bo) : torch::empty({0}, bo);
  Tensor tr = want_t ? torch::empty({cols, rows_pad}, bo) : torch::empty({0}, bo);
  int r = vlmt_fp8_amax(x.data_ptr(), x.stride(0), rows, cols, rec.data_ptr<float>(), cur());
  TORCH_CHECK(r == 0, "vlmt_fp8_amax failed with code ", r);
  r = vlmt_fp8_cast(x.data_ptr(), x.stride(0), rows, cols, rec.data_ptr<float>(), (int)format, want_rm ? rm.data_ptr() : nullptr, cols,
                    want_t ? tr.data_ptr() : nullptr, rows_pad, cur());
  TORCH_CHECK(r == 0, "vlmt_fp8_cast failed with code ", r);
  if (want_t && rows_pad != rows) tr = tr.narrow(1, 0, rows);
  return {rm, tr, rec};
}

// out [M, N] bf16 (+)= rec_a[1] * rec_b[1] * a [M, K] . b [N, K]^T with uint8 storage of the given formats
static void gemm_fp8(const Tensor& a, const Tensor& b, Tensor& out, const Tensor& rec_a, const Tensor& rec_b, int64_t a_format,
                     int64_t b_format, bool accumulate) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kByte && b.scalar_type() == at::kByte && a.dim() == 2 && b.dim() == 2 &&
                  a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == b.size(1), "gemm_fp8: a [M, K], b [N, K] uint8, K-major");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.stride(1) == 1 && out.size(0) == a.size(0) &&
                  out.size(1) == b.size(0), "gemm_fp8: out must be bf16 [M, N]");
  TORCH_CHECK(rec_a.scalar_type() == at::kFloat && rec_b.scalar_type() == at::kFloat && rec_a.numel() == 2 && rec_b.numel() == 2 &&
                  rec_a.is_cuda() && rec_b.is_cuda(), "gemm_fp8: scale records must be float [2] on the device");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor st = vlmt_status_tensor();
  int r = vlmt_gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1), a.stride(0), b.stride(0),
                        out.stride(0), (int)a_format, (int)b_format, rec_a.data_ptr<float>(), rec_b.data_ptr<float>(), accumulate ? 1 : 0,
                        st.data_ptr<int>(), sm_count(), cur());
  TORCH_CHECK(r == 0, "vlmt_gemm_fp8 failed with code ", r);
}

void bind_fp8(pybind11::module_& m) {
  m.def("fp8_quantize", &fp8_quantize);
  m.def("gemm_fp8", &gemm_fp8);
}
