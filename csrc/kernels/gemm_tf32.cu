#include "gemm_launch.cuh"
namespace rb {
int launch_gemm_tf32(const GemmArgs& a, int bn) { return launch_gemm_dtype<float>(a, bn); }
}  // namespace rb
