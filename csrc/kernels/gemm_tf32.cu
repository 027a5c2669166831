#include "gemm_launch.cuh"
namespace rb {
// tf32 inputs: only K-major operands are instantiated (MN-major 32-bit operands need the
// 32-byte-base swizzle layout; the Python layer restages those operands instead).
int launch_gemm_tf32(const GemmArgs& a, int bn) {
  if (a.a_mn || a.b_mn) return 11;
  if (bn == 256) return launch_gemm_one<float, 256, false, false>(a);
  return launch_gemm_one<float, 128, false, false>(a);
}
}  // namespace rb
