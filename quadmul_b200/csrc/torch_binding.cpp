// Compiled PyTorch binding of the GEMM entry point: module `_quadmul_torch`, function `gemm`.
//
// Same call as the reference's extension function (extension.cpp:8-24, registered at extension.cpp:26-29):
// gemm(a, b, c, m, n, k) with packed A (m x k/2), packed B (n x k/2), int32 C (m x n), launched on the current
// stream of a's device, returning None.  Unlike the reference it checks its arguments, makes a's device current
// for the call, and raises when the library reports an error.  It only marshals: the work is qm_gemm_s4.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../../include/quadmul_b200.h"

namespace {

void check_operands(const torch::Tensor &a, const torch::Tensor &b, const torch::Tensor &c, int64_t m, int64_t n, int64_t k)
{
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "quadmul.gemm: a, b and c must be CUDA tensors");
    TORCH_CHECK(a.device() == b.device() && a.device() == c.device(), "quadmul.gemm: a, b and c must be on the same device");
    TORCH_CHECK(c.scalar_type() == torch::kInt32, "quadmul.gemm: c must be int32");
    TORCH_CHECK(a.element_size() == 1 && b.element_size() == 1, "quadmul.gemm: a and b must be 1-byte tensors (two nibbles per byte)");
    TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && c.is_contiguous(), "quadmul.gemm: tensors must be contiguous");
    TORCH_CHECK(m >= 0 && n >= 0 && k >= 0 && m <= INT32_MAX && n <= INT32_MAX && k <= INT32_MAX, "quadmul.gemm: bad m, n, k");
    TORCH_CHECK(a.numel() >= m * (k / 2) && b.numel() >= n * (k / 2) && c.numel() >= m * n,
                "quadmul.gemm: tensor smaller than m, n, k imply");
}

void gemm(torch::Tensor a, torch::Tensor b, torch::Tensor c, int64_t m, int64_t n, int64_t k)
{
    check_operands(a, b, c, m, n, k);
    c10::cuda::CUDAGuard guard(a.device());
    const int st = qm_gemm_s4(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)m, (int)n, (int)k,
                              at::cuda::getCurrentCUDAStream(a.get_device()).stream());
    TORCH_CHECK(st == QM_OK, "quadmul.gemm(m=", m, ", n=", n, ", k=", k, "): ", qm_status_string(st), " ", qm_last_cuda_error());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod)
{
    mod.def("gemm", &gemm, "packed int4 x int4 -> int32 matrix product on B200 (C = A * B^T)");
}
