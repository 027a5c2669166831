// Host launch helpers for the tcgen05 GEMM (one translation unit per input dtype
// instantiates these, so the three dtypes compile in parallel).
#pragma once
#include "gemm_tcgen05.cuh"

namespace rb {

struct GemmArgs {
  int dtype;  // rbh::DT_*
  int a_mn, b_mn;
  const void* A;
  long long lda;
  const void* B;
  long long ldb;
  GemmParams p;
  int max_ctas;  // 0 = all SMs
  cudaStream_t stream;
};

template <typename T, int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(320, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a,
                        const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  NoHooks hooks;
  gemm_cta_body<T, BN, A_MN, B_MN, NoHooks>(&tma_a, &tma_b, p, hooks, smem_raw, blockIdx.x,
                                            gridDim.x);
}

// Builds the two operand tensor maps.  Returns 0 on success.
template <typename T, int BN>
int make_gemm_tensor_maps(const GemmArgs& a, CUtensorMap* ta, CUtensorMap* tb) {
  using C = GemmCfg<T, BN>;
  const uint64_t esz = sizeof(T);
  int rc;
  {
    uint64_t dims[2], strides[2] = {esz, (uint64_t)a.lda * esz};
    uint32_t box[2];
    if (!a.a_mn) {
      dims[0] = (uint64_t)a.p.K; dims[1] = (uint64_t)a.p.M;
      box[0] = C::BK; box[1] = C::BM;
    } else {
      dims[0] = (uint64_t)a.p.M; dims[1] = (uint64_t)a.p.K;
      box[0] = C::CH; box[1] = C::BK;
    }
    rc = rbh::encode_tensor_map(ta, a.dtype, 2, const_cast<void*>(a.A), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    uint64_t dims[2], strides[2] = {esz, (uint64_t)a.ldb * esz};
    uint32_t box[2];
    if (!a.b_mn) {
      dims[0] = (uint64_t)a.p.K; dims[1] = (uint64_t)a.p.N;
      box[0] = C::BK; box[1] = BN;
    } else {
      dims[0] = (uint64_t)a.p.N; dims[1] = (uint64_t)a.p.K;
      box[0] = C::CH; box[1] = C::BK;
    }
    rc = rbh::encode_tensor_map(tb, a.dtype, 2, const_cast<void*>(a.B), dims, strides, box, 1);
  }
  return rc;
}

template <typename T, int BN, bool A_MN, bool B_MN>
int launch_gemm_one(const GemmArgs& a) {
  using C = GemmCfg<T, BN>;
  CUtensorMap ta, tb;
  int rc = make_gemm_tensor_maps<T, BN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  auto kern = gemm_tcgen05_kernel<T, BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return 2000 + (int)e;
    attr_set = true;
  }
  const int num_m = (a.p.M + C::BM - 1) / C::BM;
  const int num_n = (a.p.N + BN - 1) / BN;
  int ctas = rbh::sm_count();
  if (a.max_ctas > 0 && a.max_ctas < ctas) ctas = a.max_ctas;
  const int items = num_m * num_n * (a.p.split_k > 1 ? a.p.split_k : 1);
  const int grid = items < ctas ? items : ctas;
  kern<<<grid, C::NUM_THREADS, C::SMEM_BYTES, a.stream>>>(ta, tb, a.p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

template <typename T>
int launch_gemm_dtype(const GemmArgs& a, int bn) {
#define RB_DISPATCH_MAJOR(BN_)                                                   \
  if (!a.a_mn && !a.b_mn) return launch_gemm_one<T, BN_, false, false>(a);       \
  if (!a.a_mn && a.b_mn) return launch_gemm_one<T, BN_, false, true>(a);         \
  if (a.a_mn && !a.b_mn) return launch_gemm_one<T, BN_, true, false>(a);         \
  return launch_gemm_one<T, BN_, true, true>(a);
  if (bn == 256) {
    RB_DISPATCH_MAJOR(256)
  } else {
    RB_DISPATCH_MAJOR(128)
  }
#undef RB_DISPATCH_MAJOR
}

int launch_gemm_bf16(const GemmArgs& a, int bn);
int launch_gemm_f16(const GemmArgs& a, int bn);
int launch_gemm_tf32(const GemmArgs& a, int bn);

}  // namespace rb
