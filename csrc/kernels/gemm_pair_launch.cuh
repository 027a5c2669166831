// Host-side helpers shared by the launchers of the CTA-pair GEMM body (gemm_pair.cuh): tensor maps of
// the operands and of the output, and the number of clusters that can be resident.
#pragma once
#include "gemm_launch.cuh"
#include "gemm_pair.cuh"

namespace rb {

// Operand maps of the pair kernel: every CTA copies 128-row (A) / 128-column (B) boxes.
template <typename T, bool A_MN, bool B_MN>
int make_pair_operand_maps(const GemmArgs& a, CUtensorMap* ta, CUtensorMap* tb) {
  const uint64_t esz = sizeof(T);
  {
    uint64_t dims[2], strides[2] = {esz, (uint64_t)a.lda * esz};
    uint32_t box[2];
    if (!A_MN) { dims[0] = (uint64_t)a.p.K; dims[1] = (uint64_t)a.p.M; box[0] = G2_BK; box[1] = 128; }
    else       { dims[0] = (uint64_t)a.p.M; dims[1] = (uint64_t)a.p.K; box[0] = 64; box[1] = G2_BK; }
    const int rc = rbh::encode_tensor_map(ta, a.dtype, 2, const_cast<void*>(a.A), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    uint64_t dims[2], strides[2] = {esz, (uint64_t)a.ldb * esz};
    uint32_t box[2];
    if (!B_MN) { dims[0] = (uint64_t)a.p.K; dims[1] = (uint64_t)a.p.N; box[0] = G2_BK; box[1] = 128; }
    else       { dims[0] = (uint64_t)a.p.N; dims[1] = (uint64_t)a.p.K; box[0] = 64; box[1] = G2_BK; }
    const int rc = rbh::encode_tensor_map(tb, a.dtype, 2, const_cast<void*>(a.B), dims, strides, box, 1);
    if (rc) return rc;
  }
  return 0;
}

// Output map: boxes of 128 rows x 128 bytes, 128-byte swizzle (the layout of the staging tile).
inline int make_pair_output_map(const GemmParams& p, int in_dtype, CUtensorMap* tc) {
  const int odt = p.out_f32 ? rbh::DT_F32 : in_dtype;
  const uint64_t osz = p.out_f32 ? 4 : 2;
  uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)p.M}, strides[2] = {osz, (uint64_t)p.ldc * osz};
  uint32_t box[2] = {(uint32_t)(128 / osz), 128};
  return rbh::encode_tensor_map(tc, odt, 2, p.out, dims, strides, box, 1);
}

// Clusters of this kernel that can be resident at once (asked once per instantiation).
template <typename K>
int max_resident_clusters(K kern, int smem_bytes) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (rbh::sm_count() / 2));
  cfg.blockDim = dim3(G2_THREADS);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = rbh::sm_count() / 2;
  }
  return n;
}

}  // namespace rb
