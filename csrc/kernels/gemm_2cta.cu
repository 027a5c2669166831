// Two-CTA tcgen05 GEMM (cta_group::2): a cluster of two CTAs computes one 256 x 256 output tile.
//
// Why: with one CTA per tile (gemm_tcgen05.cuh, 128 x 256) every SM stages the whole 256-wide B
// tile, and the shared-memory read port (128 B/clk) — not the tensor pipe — bounds the main loop.
// In a CTA pair each SM stages only half of B (128 of the 256 columns) plus its own 128 rows of A;
// the pair's MMA (M = 256) reads both halves, so operand bytes per SM and per MMA drop by a third.
//
//   CTA r of the pair (r = 0 leader, 1 peer), per 64-element K block:
//     TMA: A rows [m0 + 128 r, +128)  -> own smem     (16 KB)
//          B cols [n0 + 128 r, +128)  -> own smem     (16 KB)
//          both CTAs' copies complete on the LEADER's `full` barrier (cta_group::2 form of the copy)
//     leader's MMA warp: tcgen05.mma.cta_group::2, M 256 x N 256 x K 16, four per K block;
//          accumulator rows [128 r, +128) live in CTA r's TMEM (256 fp32 columns, double buffered)
//     tcgen05.commit (cta_group::2) releases the stage in both CTAs (`empty`) and, after the last K
//          block, hands the accumulator to both CTAs' epilogue warps (`tmem_full`)
//     epilogue warps of CTA r store rows m0 + 128 r ...; they release the accumulator on the
//          leader's `tmem_empty` barrier (the peer's warps arrive remotely).
//
// Every wait is bounded (mbar_wait).  TMEM is allocated and freed by the MMA warp of both CTAs
// (the cta_group::2 forms of alloc / dealloc are collective over the pair), and no CTA leaves
// before both have finished their last tile (`done` barrier), so nothing is ever signalled into
// the shared memory of a CTA that has exited.  The copies carry no cluster-wide fan-out: each CTA
// loads its own half.
//
// Same epilogue as the one-CTA kernel (bias, activation, activation derivative, residual,
// pre-activation side output); static tile schedule over clusters; bf16 / fp16 operands in any of
// the four storage-major combinations.  Reference counterpart: the naive one-thread-per-output
// matmul of rumus/src/backend/gpu/shaders/matmul.wgsl:22.
#include <cstdlib>

#include "gemm_launch.cuh"

namespace rb {

constexpr int G2_BM = 256;          // rows of the pair's tile (128 per CTA)
constexpr int G2_BN = 256;          // columns of the tile (each CTA stages 128 of them)
constexpr int G2_BK = 64;           // 16-bit elements per K block (one 128-byte swizzle row)
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = 128 * 128;
constexpr int G2_B_BYTES = 128 * 128;
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_THREADS = 320;
constexpr int G2_EPI_WARPS = 8;
constexpr int G2_TMEM_COLS = 512;   // two accumulators of 256 fp32 columns
constexpr int G2_SMEM_BYTES = G2_STAGES * G2_STAGE_BYTES + 1024 + 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// copy of one box into this CTA's shared memory; the bytes are counted on `bar_cluster_addr`, which
// may be a barrier of the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// whole warp, uniform arguments; one elected lane issues
__device__ __forceinline__ void umma_f16_pair_w(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, e;\n\telect.sync _|e, 0xffffffff;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "@e tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// the barrier (anywhere in the cluster) receives one arrival once every MMA issued so far is complete
__device__ __forceinline__ void umma_commit_pair_w(uint32_t bar_cluster_addr) {
  asm volatile(
      "{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
      "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}\n" ::"r"(bar_cluster_addr)
      : "memory");
}

template <typename T, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
    gemm_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // both CTAs of a pair must use the same shared-memory offsets (the MMA addresses the peer's
  // operands by offset, remote arrivals address barriers by offset); the dynamic segment starts at
  // the same offset in every CTA of a kernel, so aligning the same way gives the same layout
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + G2_STAGES * G2_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + G2_STAGES * G2_B_BYTES);
  uint64_t* full_bar = bars;                        // leader's are used: both CTAs' copies complete here
  uint64_t* empty_bar = bars + G2_STAGES;           // per CTA: the leader's commit releases the stage
  uint64_t* tmem_full_bar = bars + 2 * G2_STAGES;   // [2] per CTA
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;     // [2] leader's are used (16 arrivals)
  uint64_t* done_bar = tmem_empty_bar + 2;          // per CTA: 16 arrivals (both CTAs' epilogue warps)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();      // 0 = leader, 1 = peer
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), 2 * G2_EPI_WARPS);
    }
    mbar_init(smem_u32(done_bar), 2 * G2_EPI_WARPS);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // barriers of both CTAs exist before anything is signalled across the pair
  cluster_sync_all();
  if (warp_idx == 1) {
    tmem_alloc_2cta(smem_u32(tmem_ptr_smem), G2_TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_m = (p.M + G2_BM - 1) / G2_BM;
  const int num_n = (p.N + G2_BN - 1) / G2_BN;
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  const int total_tiles = num_m * num_n;
  const int num_clusters = gridDim.x / 2;
  const int cluster_id = blockIdx.x / 2;
  const int group_m = p.group_m > 0 ? p.group_m : 8;
  auto tile_coords = [&](int tile, int& m_idx, int& n_idx) {
    const int group_size = group_m * num_n;
    const int g = tile / group_size;
    const int first_m = g * group_m;
    const int gm = min(num_m - first_m, group_m);
    const int r = tile - g * group_size;
    m_idx = first_m + r % gm;
    n_idx = r / gm;
  };
  constexpr int CH = 64;   // MN elements per 128-byte chunk of an MN-major operand

  if (warp_idx == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;     // K blocks loaded so far (the first G2_STAGES find their stage free)
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
        int m_idx, n_idx;
        tile_coords(tile, m_idx, n_idx);
        const int m0 = m_idx * G2_BM + (int)cta_rank * 128;    // this CTA's rows of A
        const int n0 = n_idx * G2_BN + (int)cta_rank * 128;    // this CTA's columns of B
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          // forwarding mode: the leader's commit only reached the leader's barrier; pass the release
          // of this stage on to the peer (not on the first round, when every stage starts out free)
          if (p.pair_release == 1 && leader && issued >= G2_STAGES)
            mbar_arrive_cluster(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * G2_STAGE_BYTES);
          const uint32_t a_dst = smem_u32(sA + stage * G2_A_BYTES);
          const uint32_t b_dst = smem_u32(sB + stage * G2_B_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d_pair(a_dst, &tma_a, leader_full, kb * G2_BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < 128 / CH; ++j)
              tma_load_2d_pair(a_dst + j * G2_BK * 128, &tma_a, leader_full, m0 + j * CH, kb * G2_BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, &tma_b, leader_full, kb * G2_BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < 128 / CH; ++j)
              tma_load_2d_pair(b_dst + j * G2_BK * 128, &tma_b, leader_full, n0 + j * CH, kb * G2_BK);
          }
          ++issued;
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land
    }
  } else if (warp_idx == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ---------------------------
    if (leader) {
      constexpr uint32_t idesc = make_idesc(UmmaFormat<T>::value, A_MN ? 1 : 0, B_MN ? 1 : 0, G2_BM, G2_BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * G2_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + stage * G2_A_BYTES);
          const uint32_t b_base = smem_u32(sB + stage * G2_B_BYTES);
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_base + k * 16 * 128, G2_BK * 128, 1024)
                                        : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k * 16 * 128, G2_BK * 128, 1024)
                                        : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_pair_w(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free again in both CTAs once these MMAs have read it
          umma_commit_pair_w(smem_u32(&empty_bar[stage]));
          if (p.pair_release == 0) umma_commit_pair_w(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair_w(smem_u32(&tmem_full_bar[acc]));
        if (p.pair_release == 0) umma_commit_pair_w(map_to_cta(smem_u32(&tmem_full_bar[acc]), 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) -----------------------------------
    const int quarter = warp_idx & 3;
    const int half = (warp_idx - 2) >> 2;               // 0: columns 0..127, 1: columns 128..255
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const uint32_t leader_empty0 = map_to_cta(smem_u32(&tmem_empty_bar[0]), 0);
    const uint32_t leader_empty1 = map_to_cta(smem_u32(&tmem_empty_bar[1]), 0);
    for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
      int m_idx, n_idx;
      tile_coords(tile, m_idx, n_idx);
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // forwarding mode: one warp of the leader hands the accumulator to the peer's epilogue
      if (p.pair_release == 1 && leader && warp_idx == 2 && lane == 0)
        mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_full_bar[acc]), 1));
      tc_fence_after();
      const long long row = static_cast<long long>(m_idx) * G2_BM + cta_rank * 128 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * G2_BN;
#pragma unroll 1
      for (int ci = 0; ci < 4; ++ci) {
        const int c = half * 4 + ci;
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n_idx * G2_BN + c * 32;
        const int ncols_valid = min(32, p.N - col);
        if (row < p.M && ncols_valid > 0) {
          if (p.out_f32)
            epilogue_chunk<T, float>(p, r, row, col, ncols_valid);
          else
            epilogue_chunk<T, T>(p, r, row, col, ncols_valid);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? leader_empty0 : leader_empty1);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    // this warp will not touch TMEM or signal any barrier again: tell both CTAs
    __syncwarp();
    if (lane == 0) {
      mbar_arrive_cluster(map_to_cta(smem_u32(done_bar), 0));
      mbar_arrive_cluster(map_to_cta(smem_u32(done_bar), 1));
    }
  }

  // ------------------------------ teardown ------------------------------------
  // Nobody leaves (and TMEM is not freed) before all 16 epilogue warps of the pair are through:
  // the leader's last commits into the peer's barriers precede the peer's last epilogue.
  if (warp_idx == 1) {
    bool ok = mbar_wait(smem_u32(done_bar), 0, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_EMPTY);
    (void)ok;
  }
  tc_fence_before();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, G2_TMEM_COLS);
  }
}

template <typename T, bool A_MN, bool B_MN>
int launch_gemm_2cta(const GemmArgs& a) {
  const uint64_t esz = sizeof(T);
  CUtensorMap ta, tb;
  {
    uint64_t dims[2], strides[2] = {esz, (uint64_t)a.lda * esz};
    uint32_t box[2];
    if (!A_MN) { dims[0] = (uint64_t)a.p.K; dims[1] = (uint64_t)a.p.M; box[0] = G2_BK; box[1] = 128; }
    else       { dims[0] = (uint64_t)a.p.M; dims[1] = (uint64_t)a.p.K; box[0] = 64; box[1] = G2_BK; }
    const int rc = rbh::encode_tensor_map(&ta, a.dtype, 2, const_cast<void*>(a.A), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  {
    uint64_t dims[2], strides[2] = {esz, (uint64_t)a.ldb * esz};
    uint32_t box[2];
    if (!B_MN) { dims[0] = (uint64_t)a.p.K; dims[1] = (uint64_t)a.p.N; box[0] = G2_BK; box[1] = 128; }
    else       { dims[0] = (uint64_t)a.p.N; dims[1] = (uint64_t)a.p.K; box[0] = 64; box[1] = G2_BK; }
    const int rc = rbh::encode_tensor_map(&tb, a.dtype, 2, const_cast<void*>(a.B), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  auto kern = gemm_2cta_kernel<T, A_MN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_BYTES);
  if (e != cudaSuccess) return 2000 + (int)e;
  const int tiles = ((a.p.M + G2_BM - 1) / G2_BM) * ((a.p.N + G2_BN - 1) / G2_BN);
  int clusters = rbh::sm_count() / 2;
  if (a.max_ctas > 0 && a.max_ctas / 2 < clusters) clusters = a.max_ctas / 2;
  if (clusters < 1) clusters = 1;
  if (tiles < clusters) clusters = tiles;
  kern<<<2 * clusters, G2_THREADS, G2_SMEM_BYTES, a.stream>>>(ta, tb, a.p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

template <typename T>
int launch_gemm_2cta_dtype(const GemmArgs& a) {
  if (!a.a_mn && !a.b_mn) return launch_gemm_2cta<T, false, false>(a);
  if (!a.a_mn && a.b_mn) return launch_gemm_2cta<T, false, true>(a);
  if (a.a_mn && !a.b_mn) return launch_gemm_2cta<T, true, false>(a);
  return launch_gemm_2cta<T, true, true>(a);
}

}  // namespace rb

extern "C" {

// Same contract as rb_gemm for 16-bit operands.  Returns 13 when the problem is outside what this
// kernel covers (fp32 operands, operands that are not TMA-legal).
int rb_gemm_2cta(int dtype, int a_mn, int b_mn, const void* A, long long lda, const void* B, long long ldb,
                 int M, int N, int K, void* out, long long ldc, int out_f32, const void* bias,
                 const void* residual, long long ldr, void* aux_out, long long ldaux_out, const void* aux_in,
                 long long ldaux_in, int act, int dact, float alpha, int max_ctas, void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 13;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (K <= 0 || !al(A) || !al(B) || (lda * 2) % 16 || (ldb * 2) % 16) return 13;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = a_mn; a.b_mn = b_mn; a.A = A; a.lda = lda; a.B = B; a.ldb = ldb;
  a.max_ctas = max_ctas;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p.M = M; p.N = N; p.K = K; p.out = out; p.bias = bias; p.residual = residual;
  p.aux_out = aux_out; p.aux_in = aux_in; p.ldc = ldc; p.ldr = ldr; p.ldaux_out = ldaux_out;
  p.ldaux_in = ldaux_in; p.act = act; p.dact = dact; p.out_f32 = out_f32; p.alpha = alpha;
  p.status = rbh::device_status_word();
  p.group_m = 4;      // 4 x 256 rows share a B column panel in L2, like 8 x 128 in the one-CTA kernel
  p.split_k = 1;
  p.sched = nullptr;
  {
    const char* e = getenv("RB_G2_RELEASE");     // "forward": see GemmParams::pair_release
    p.pair_release = (e && e[0] == 'f') ? 1 : 0;
  }
  const int osz = out_f32 ? 4 : 2;
  p.vec_ok = al(out) && (ldc * osz) % 16 == 0 && (!residual || (al(residual) && (ldr * osz) % 16 == 0)) &&
             (!aux_out || (al(aux_out) && (ldaux_out * osz) % 16 == 0)) &&
             (!aux_in || (al(aux_in) && (ldaux_in * osz) % 16 == 0));
  return dtype == rbh::DT_BF16 ? launch_gemm_2cta_dtype<__nv_bfloat16>(a) : launch_gemm_2cta_dtype<__half>(a);
}
}
