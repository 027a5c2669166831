// CSR sparse x dense matmul for sm_100a: Y[i, :] = sum_{e in row i} val[e] * X[col[e], :].
// One warp per output row; lanes stride over the feature dimension with 128-bit accesses when
// the feature width allows it.  The backward pass is the same kernel on the pre-transposed CSR.
// Reference: rumus-graph/src/spmm.wgsl:32 (one thread per row, scalar feature loop).
#include "sm100_common.cuh"

namespace rb {

template <typename T>
__global__ void __launch_bounds__(256)
    spmm_csr_kernel(const int* __restrict__ rowptr, const int* __restrict__ col,
                    const float* __restrict__ val, const T* __restrict__ x, T* __restrict__ y,
                    int rows, int feat, int vec_ok) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const int e0 = rowptr[warp], e1 = rowptr[warp + 1];
  constexpr int VEC = 16 / sizeof(T);
  if (vec_ok) {
    for (int f = lane * VEC; f < feat; f += 32 * VEC) {
      float acc[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
      for (int e = e0; e < e1; ++e) {
        const float w = val ? val[e] : 1.f;
        const uint4 raw = *reinterpret_cast<const uint4*>(x + (long long)col[e] * feat + f);
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = fmaf(w, to_f32<T>(v[j]), acc[j]);
      }
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < VEC; ++j) oe[j] = from_f32<T>(acc[j]);
      *reinterpret_cast<uint4*>(y + (long long)warp * feat + f) = o;
    }
  } else {
    for (int f = lane; f < feat; f += 32) {
      float acc = 0.f;
      for (int e = e0; e < e1; ++e)
        acc = fmaf(val ? val[e] : 1.f, to_f32<T>(x[(long long)col[e] * feat + f]), acc);
      y[(long long)warp * feat + f] = from_f32<T>(acc);
    }
  }
}

}  // namespace rb

extern "C" int rb_spmm_csr(int dtype, const int* rowptr, const int* col, const float* val,
                           const void* x, void* y, int rows, int feat, void* stream) {
  using namespace rb;
  if (rows <= 0 || feat <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int esz = dtype == rbh::DT_F32 ? 4 : 2;
  const int vec = (feat % (16 / esz) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                  ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
  const unsigned blocks = (unsigned)(((long long)rows * 32 + 255) / 256);
  if (dtype == rbh::DT_BF16) spmm_csr_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(rowptr, col, val, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, feat, vec);
  else if (dtype == rbh::DT_F16) spmm_csr_kernel<__half><<<blocks, 256, 0, st>>>(rowptr, col, val, (const __half*)x, (__half*)y, rows, feat, vec);
  else spmm_csr_kernel<float><<<blocks, 256, 0, st>>>(rowptr, col, val, (const float*)x, (float*)y, rows, feat, vec);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
