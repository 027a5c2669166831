#include "gemm_launch.cuh"
namespace rb {
int launch_gemm_bf16(const GemmArgs& a, int bn) { return launch_gemm_dtype<__nv_bfloat16>(a, bn); }
}  // namespace rb
