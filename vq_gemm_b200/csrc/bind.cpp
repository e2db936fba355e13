// PyTorch-extension shim over the C ABI (include/vqg.h).  Keeps the reference's module surface
// (reference bind.cpp:3-8: `e2e_gemm(input, w, codebook)` and `gemm(input, w)`) and adds
// `vq_gemm` / `dequant` for the generalised weight format.  Unlike the reference's launchers it
// validates its arguments, allocates the output on the inputs' device, launches on torch's current
// stream, releases the GIL around the launch and prints nothing.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <utility>
#include <vector>
#include <unordered_map>

#include "../../include/vqg.h"

namespace {

void check(int st, const char* what) {
  TORCH_CHECK(st == VQG_OK, what, ": ", vqg_status_string(st), " (status ", st, ")");
}

// Scratch per (device, stream), zero-initialised once (the library keeps its counter region zero).  Calls on
// different streams may overlap on the GPU, so they must not share a buffer; a buffer that has to grow is
// replaced but kept alive, because a CUDA graph captured earlier may still hold its address.
at::Tensor workspace(const at::Device& dev, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, void*>, at::Tensor> cache;
  static std::vector<at::Tensor> retired;
  constexpr size_t kMin = size_t(64) << 20;
  void* stream = static_cast<void*>(at::cuda::getCurrentCUDAStream(dev.index()).stream());
  std::lock_guard<std::mutex> lk(mu);
  auto& t = cache[{static_cast<int>(dev.index()), stream}];
  if (!t.defined() || static_cast<size_t>(t.numel()) < bytes) {
    if (t.defined()) retired.push_back(t);
    t = torch::zeros({static_cast<int64_t>(std::max<size_t>(bytes, kMin))},
                     torch::TensorOptions().dtype(torch::kUInt8).device(dev));
  }
  return t;
}

int idx_bytes_of(const at::Tensor& t) {
  if (t.scalar_type() == at::kByte) return 1;
  if (t.scalar_type() == at::kShort || t.scalar_type() == at::kUInt16) return 2;
  TORCH_CHECK(false, "indices must be uint8 or (u)int16");
}

void check_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (there is no CPU path)");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

torch::Tensor vq_gemm(torch::Tensor x, torch::Tensor indices, torch::Tensor codebook, int64_t rows_per_codebook,
                      const std::string& layout_in) {
  check_cuda(x, "x"); check_cuda(indices, "indices"); check_cuda(codebook, "codebook");
  TORCH_CHECK(x.scalar_type() == at::kHalf && codebook.scalar_type() == at::kHalf, "x and codebook must be float16");
  TORCH_CHECK(x.dim() == 2 && indices.dim() == 2 && (codebook.dim() == 3 || codebook.dim() == 2), "bad ranks");
  TORCH_CHECK(indices.device() == x.device() && codebook.device() == x.device(), "tensors on different devices");
  const int64_t M = x.size(0), K = x.size(1);
  const int64_t v = codebook.size(-1);
  const int ib = idx_bytes_of(indices);
  std::string layout = layout_in;
  if (layout == "auto") {
    const bool is_bl = indices.size(1) * v == K;
    const bool is_ref = codebook.dim() == 3 && v == 2 && indices.size(0) == K && indices.size(1) % 4 == 0 &&
                        codebook.size(0) == indices.size(1) / 4 && codebook.size(1) == 256 && ib == 1;
    TORCH_CHECK(is_bl != is_ref, is_bl ? "shapes fit both weight formats; pass layout" : "shapes fit neither weight format");
    layout = is_ref ? "ref" : "bl";
  }
  int64_t N, C;
  int lay;
  if (layout == "ref") {
    TORCH_CHECK(indices.size(0) == K && codebook.dim() == 3 && codebook.size(0) * 4 == indices.size(1) &&
                    codebook.size(1) == 256 && v == 2 && ib == 1,
                "reference format needs w [K, Nq] uint8 and codebook [Nq/4, 256, 2]");
    N = 2 * indices.size(1); C = 256; lay = VQG_LAYOUT_REF; rows_per_codebook = 0;
  } else {
    TORCH_CHECK(layout == "bl", "unknown layout");
    TORCH_CHECK(indices.size(1) * v == K, "indices [N, K/v] do not match K and v");
    N = indices.size(0);
    const int64_t G = codebook.dim() == 3 ? codebook.size(0) : 1;
    C = codebook.size(-2);
    if (rows_per_codebook < 0) rows_per_codebook = (G == 1) ? 0 : N / G;
    lay = VQG_LAYOUT_BL;
  }
  c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty({M, N}, x.options());
  const size_t need = vqg_workspace_bytes(M, N, K, v, C, ib, rows_per_codebook, lay, VQG_PATH_AUTO);
  at::Tensor ws;
  if (need) ws = workspace(x.device(), need);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  int st;
  {
    pybind11::gil_scoped_release nogil;
    st = vqg_gemm(x.data_ptr(), indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), M, N, K, v, C, ib,
                  rows_per_codebook, lay, need ? ws.data_ptr() : nullptr, need ? ws.numel() : 0, stream);
  }
  check(st, "vq_gemm");
  return out;
}

torch::Tensor e2e_gemm(torch::Tensor input, torch::Tensor w, torch::Tensor codebook) {
  return vq_gemm(input, w, codebook, -1, "auto");
}

torch::Tensor gemm(torch::Tensor input, torch::Tensor w) {
  check_cuda(input, "input"); check_cuda(w, "w");
  TORCH_CHECK(input.scalar_type() == at::kHalf && w.scalar_type() == at::kHalf, "gemm expects float16");
  TORCH_CHECK(input.dim() == 2 && w.dim() == 2 && w.size(0) == input.size(1), "gemm expects input [M,K], w [K,N]");
  const int64_t M = input.size(0), K = input.size(1), N = w.size(1);
  c10::cuda::CUDAGuard guard(input.device());
  auto out = torch::empty({M, N}, input.options());
  const size_t need = vqg_dense_workspace_bytes(M, N, K, 1);
  at::Tensor ws = workspace(input.device(), need);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  int st;
  {
    pybind11::gil_scoped_release nogil;
    st = vqg_dense_gemm(input.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, 1, ws.data_ptr(), ws.numel(), stream);
  }
  check(st, "gemm");
  return out;
}

torch::Tensor dequant(torch::Tensor indices, torch::Tensor codebook, int64_t rows_per_codebook, const std::string& layout) {
  check_cuda(indices, "indices"); check_cuda(codebook, "codebook");
  TORCH_CHECK(codebook.scalar_type() == at::kHalf, "codebook must be float16");
  const int ib = idx_bytes_of(indices);
  c10::cuda::CUDAGuard guard(indices.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  torch::Tensor out;
  int st;
  if (layout == "ref") {
    const int64_t K = indices.size(0), Nq = indices.size(1);
    out = torch::empty({K, 2 * Nq}, codebook.options());
    st = vqg_dequant(indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), 2 * Nq, K, 2, 256, ib, 0, VQG_LAYOUT_REF, stream);
  } else {
    const int64_t v = codebook.size(-1), C = codebook.size(-2), N = indices.size(0), K = indices.size(1) * v;
    const int64_t G = codebook.dim() == 3 ? codebook.size(0) : 1;
    if (rows_per_codebook < 0) rows_per_codebook = (G == 1) ? 0 : N / G;
    out = torch::empty({N, K}, codebook.options());
    st = vqg_dequant(indices.data_ptr(), codebook.data_ptr(), out.data_ptr(), N, K, v, C, ib, rows_per_codebook,
                     VQG_LAYOUT_BL, stream);
  }
  check(st, "dequant");
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("e2e_gemm", &e2e_gemm, "VQ GEMM");
  m.def("gemm", &gemm, "Normal GEMM");
  m.def("vq_gemm", &vq_gemm, "VQ GEMM, generalised weight format", pybind11::arg("x"), pybind11::arg("indices"),
        pybind11::arg("codebook"), pybind11::arg("rows_per_codebook") = -1, pybind11::arg("layout") = "auto");
  m.def("dequant", &dequant, "bit-exact dequantised weights", pybind11::arg("indices"), pybind11::arg("codebook"),
        pybind11::arg("rows_per_codebook") = -1, pybind11::arg("layout") = "bl");
}
