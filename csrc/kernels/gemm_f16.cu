#include "gemm_launch.cuh"
namespace rb {
int launch_gemm_f16(const GemmArgs& a, int bn) { return launch_gemm_dtype<__half>(a, bn); }
}  // namespace rb
