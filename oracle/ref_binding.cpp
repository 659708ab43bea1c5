// Python binding for the five solver-path kernels of the reference and its per-expert inference GEMM, compiled FROM THE REFERENCE'S OWN .cu FILES
// where they lie (see oracle/ref_build.py).  Test infrastructure only: it lets the GPU parity tests call the
// reference's kernels on the same inputs as the engine, and it generates the golden vectors that pin the CPU oracle.
// The declarations repeat the signatures the reference's kernels.cpp declares (forge/backend/cuda/kernels.cpp:21-72);
// nothing else of the reference is reproduced here.
#include <torch/extension.h>
#include <tuple>

std::tuple<torch::Tensor, torch::Tensor> build_quantization_meta_cuda(torch::Tensor X, int64_t bit_width, bool symmetric);
std::tuple<torch::Tensor, torch::Tensor> mse_quantization_grid_cuda(torch::Tensor X, torch::Tensor scales, torch::Tensor qzeros,
                                                                   torch::Tensor candidates, float norm, int64_t bit_width,
                                                                   bool symmetric);
torch::Tensor gptq_solver_cuda(torch::Tensor W, torch::Tensor U, torch::Tensor scales, torch::Tensor qzeros, int64_t bits);
std::tuple<torch::Tensor, torch::Tensor> sparsegptq14_solver_cuda(torch::Tensor W, torch::Tensor U, torch::Tensor scales,
                                                                 torch::Tensor qzeros, int64_t bits);
torch::Tensor pack_sparsegptq14_to_u64x2_cuda(torch::Tensor qweight_rc, torch::Tensor M, torch::Tensor scales);
torch::Tensor moe_proj_unstructured_sparse14_int4symq_gemm(torch::Tensor qW2S1u64, torch::Tensor X);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("build_group_meta_packed", &build_quantization_meta_cuda);
    m.def("mse_scale_groups_packed", &mse_quantization_grid_cuda);
    m.def("gptq_solver", &gptq_solver_cuda);
    m.def("sparsegptq14_solver", &sparsegptq14_solver_cuda);
    m.def("pack_sparsegptq14_to_u64x2", &pack_sparsegptq14_to_u64x2_cuda);
    m.def("sparsegptq14_gemm", &moe_proj_unstructured_sparse14_int4symq_gemm);
}
