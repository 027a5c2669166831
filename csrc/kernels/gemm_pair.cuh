// Two-CTA tcgen05 GEMM body (cta_group::2): a cluster of two CTAs computes one 256 x 256 output
// tile; persistent, warp specialised, dynamically scheduled, with the same fused epilogue and the
// same producer / epilogue hooks as the one-CTA body (gemm_tcgen05.cuh), so the fused collective
// kernels can run on it.
//
// Why pairs: with one CTA per 128 x 256 tile every SM pulls 48 KB per 64-wide K block out of L2
// and through its shared memory; in a pair each SM stages its own 128 rows of A and only HALF of
// the B tile (128 of the 256 columns) — 32 KB per K block — and the pair's M = 256 MMA reads both
// halves.  A third less L2 -> SM traffic and shared-memory fill per FLOP.
//
//   CTA r of the pair (r = 0 leader, 1 peer), per K block:
//     TMA (own producer warp): A rows [m0 + 128 r, +128) and B columns [n0 + 128 r, +128) -> own smem;
//          both CTAs' copies are counted on the LEADER's `full` barrier (cta_group::2 form of the copy;
//          no fan-out to other CTAs: every CTA loads only what it keeps)
//     leader's MMA warp: tcgen05.mma.cta_group::2, M 256 x N 256 x K 16, four per K block;
//          accumulator rows [128 r, +128) live in CTA r's TMEM (256 fp32 columns, double buffered)
//     tcgen05.commit releases the stage in both CTAs and, after the last K block of a tile, hands
//          the accumulator to both CTAs' epilogue warps
//     epilogue warps of CTA r (8, warps 4..11: TMEM lane quarter x column half): TMEM -> registers -> fused
//          bias / activation / derivative / residual -> 128-byte-swizzled staging tile in shared
//          memory -> one TMA store per 128-row x 128-byte chunk (rows and columns beyond M, N are
//          clipped by the copy engine).  Outputs that are not TMA-legal take per-row stores.
//
// Tile ids come from the leader's producer thread (device-wide atomic counter, or a static stride)
// and travel to every consumer of both CTAs through a 4-deep ring in each CTA's shared memory
// (remote store + remote mbarrier arrive for the peer).
//
// Every wait is bounded.  TMEM is allocated / freed by the MMA warp of both CTAs (the cta_group::2
// forms are collective over the pair) and no CTA leaves before all 16 epilogue warps of the pair
// are through (`done` barrier), so nothing is signalled into the shared memory of a CTA that has
// exited.
#pragma once
#include "gemm_tcgen05.cuh"

namespace rb {

constexpr int G2_BN = 256;          // columns of the tile (each CTA stages 128 of them)
constexpr int G2_BK = 64;           // 16-bit elements per K block (one 128-byte swizzle row)
constexpr int G2_B_BYTES = 128 * 128;
constexpr int G2_THREADS = 384;     // warps 0..3: producer, MMA issuer, two idle; warps 4..11: epilogue
constexpr int G2_EPI_WARP0 = 4;
constexpr int G2_EPI_WARPS = 8;
constexpr int G2_TMEM_COLS = 512;   // two accumulators of 256 fp32 columns
constexpr int G2_STAGING_BYTES = 128 * 128;   // 128 rows x 128 bytes, one per column half
constexpr int G2_SCHED_CONSUMERS = 2 * G2_EPI_WARPS + 2;   // leader MMA warp, peer producer, 16 epilogue warps

// MT = 128-row blocks of A per CTA and tile.  MT = 1: 256 x 256 tiles, 6 stages of 32 KB, the two
// TMEM accumulators double-buffer consecutive tiles.  MT = 2: 512 x 256 tiles, 4 stages of 48 KB
// (a quarter less operand traffic per FLOP again), the two accumulators hold the tile's two row
// blocks; the epilogue hands each back as soon as it is drained, so the next tile's first MMAs only
// wait for the first of them.
template <int MT>
struct PairCfg {
  static constexpr int BM = 256 * MT;
  static constexpr int A_BYTES = MT * 128 * 128;
  static constexpr int STAGE_BYTES = A_BYTES + G2_B_BYTES;
  static constexpr int STAGES = MT == 1 ? 6 : 4;
  static constexpr int STAGING = 2 * G2_STAGING_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING + 1024 + 512;
  static constexpr int ACC_RELEASERS = 2 * G2_EPI_WARPS;   // epilogue warps of both CTAs drain every accumulator
};

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
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// try_wait that also orders against writes released by a thread of the OTHER CTA of the pair
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > RB_WAIT_BUDGET_NS) {
        record_error(status, code);
        *abort_flag = 1;
        return false;
      }
    }
  }
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
__device__ __forceinline__ void cta_sync_pair() {
  asm volatile("bar.sync 0, 384;" ::: "memory");
}
// Register re-allocation between warpgroups (four consecutive warps each): the producer / MMA
// warpgroup gives registers back, the two epilogue warpgroups take them.
__device__ __forceinline__ void regs_release_to_64() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 64;" ::: "memory");
}
__device__ __forceinline__ void regs_grow_to_216() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 216;" ::: "memory");
}
__device__ __forceinline__ void bar_sync_named(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// named barrier that also ANDs a predicate over its participants (same answer in every thread)
__device__ __forceinline__ bool bar_vote_and(int id, int threads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
      "bar.red.and.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(r)
      : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

// Everything of the fused epilogue except the final store: v = dact(aux_in) * act(alpha*acc + bias) + residual
// for 32 consecutive columns of one row; the pre-activation side output is stored here.
// EPI selects what is compiled in: EPI_FULL everything (decided at run time), EPI_LEAN none of the
// activation terms, EPI_GELU_AUX = store the pre-activation, then tanh-GELU (an MLP's first layer in
// forward), EPI_DGELU = multiply by the tanh-GELU derivative of a stored pre-activation (the data
// gradient of its second layer).  The specialised bodies are a few hundred instructions; the full one is
// large enough for its instruction fetch to show in the tile time.
enum { EPI_FULL = 0, EPI_LEAN = 1, EPI_GELU_AUX = 2, EPI_DGELU = 3 };

template <typename T, typename OT, int EPI = EPI_FULL>
__device__ __forceinline__ void epilogue_math32(const GemmParams& p, const uint32_t* acc_bits, long long row,
                                                int col, int ncols_valid, bool row_ok, float* v) {
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc_bits[i]) * p.alpha;
  if (p.bias) {
    const T* b = reinterpret_cast<const T*>(p.bias) + col;
    if (ncols_valid == 32 && (reinterpret_cast<uintptr_t>(b) & 15) == 0) {
      constexpr int PER = 16 / sizeof(T);
#pragma unroll
      for (int i = 0; i < 32 / PER; ++i) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(b) + i);
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int j = 0; j < PER; ++j) v[i * PER + j] += to_f32<T>(e[j]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols_valid) v[i] += to_f32<T>(b[i]);
    }
  }
  const bool vec = p.vec_ok != 0;
  if (!row_ok || ncols_valid <= 0) return;
  // the specialised flavours: the caller has checked which terms the call has
  if constexpr (EPI == EPI_GELU_AUX) {
    store_row32<OT>(reinterpret_cast<OT*>(p.aux_out), p.ldaux_out, row, col, ncols_valid, vec, v);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
  }
  if constexpr (EPI == EPI_DGELU) {
    float a[32];
    load_row32<OT>(reinterpret_cast<const OT*>(p.aux_in), p.ldaux_in, row, col, ncols_valid, vec, a);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= gelu_tanh_grad_fast(a[i]);
  }
  if constexpr (EPI == EPI_FULL) {
    if (p.aux_out) store_row32<OT>(reinterpret_cast<OT*>(p.aux_out), p.ldaux_out, row, col, ncols_valid, vec, v);
  }
  if constexpr (EPI == EPI_FULL) {
    // one loop per activation kind (a switch inside the unrolled loop would lay down every kind 32 times)
    if (p.act == ACT_RELU) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
    } else if (p.act == ACT_GELU) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
    } else if (p.act == ACT_SILU) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
    }
    if (p.aux_in) {
      float a[32];
      load_row32<OT>(reinterpret_cast<const OT*>(p.aux_in), p.ldaux_in, row, col, ncols_valid, vec, a);
      if (p.dact == ACT_RELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = a[i] > 0.0f ? v[i] : 0.0f;
      } else if (p.dact == ACT_GELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= gelu_tanh_grad_fast(a[i]);
      } else if (p.dact == ACT_SILU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= silu_grad(a[i]);
      }
    }
  }
  if (p.residual) {
    float r[32];
    load_row32<OT>(reinterpret_cast<const OT*>(p.residual), p.ldr, row, col, ncols_valid, vec, r);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += r[i];
  }
}

// 32 floats of row `r` (0..127) -> the 128-byte-swizzled staging tile (rows of 128 bytes);
// `piece` = which 32-column piece of the row's chunk (16-bit outputs: 2 pieces of 64 bytes; fp32: 1)
template <typename OT>
__device__ __forceinline__ void stage_row32(uint8_t* staging, int r, int piece, const float* v) {
  constexpr int NV = 32 * sizeof(OT) / 16;      // 16-byte vectors for 32 elements: 4 (16-bit) or 8 (fp32)
  uint8_t* rowp = staging + r * 128;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    uint4 q;
    if constexpr (sizeof(OT) == 4) {
      q = make_uint4(__float_as_uint(v[i * 4]), __float_as_uint(v[i * 4 + 1]), __float_as_uint(v[i * 4 + 2]),
                     __float_as_uint(v[i * 4 + 3]));
    } else {
      q = make_uint4(pack2<OT>(v[i * 8], v[i * 8 + 1]), pack2<OT>(v[i * 8 + 2], v[i * 8 + 3]),
                     pack2<OT>(v[i * 8 + 4], v[i * 8 + 5]), pack2<OT>(v[i * 8 + 6], v[i * 8 + 7]));
    }
    const int j = piece * NV + i;                // 16-byte chunk index inside the 128-byte row
    *reinterpret_cast<uint4*>(rowp + ((j ^ (r & 7)) << 4)) = q;
  }
}

// Lean epilogue of 32 consecutive columns of one row straight into 16 packed words:
// out = alpha * acc + bias + residual, eight columns at a time so that no 32-float temporary is live.
template <typename T>
__device__ __forceinline__ void lean_pack32(const GemmParams& p, const uint32_t* acc_bits, long long row, int col,
                                            int ncols_valid, bool row_ok, uint32_t* pk) {
  const T* b = p.bias ? reinterpret_cast<const T*>(p.bias) + col : nullptr;
  const T* rs = (p.residual && row_ok) ? reinterpret_cast<const T*>(p.residual) + row * p.ldr + col : nullptr;
  const bool full = ncols_valid == 32 && p.vec_ok && (!b || (reinterpret_cast<uintptr_t>(b) & 15) == 0);
  if (full) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(acc_bits[g * 8 + i]) * p.alpha;
      if (b) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(b) + g);
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += to_f32<T>(e[i]);
      }
      if (rs) {
        const uint4 q = *(reinterpret_cast<const uint4*>(rs) + g);
        const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += to_f32<T>(e[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) pk[g * 4 + i] = pack2<T>(f[2 * i], f[2 * i + 1]);
    }
  } else {
    // ragged edge or unaligned operands: element by element
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float f0 = __uint_as_float(acc_bits[2 * i]) * p.alpha, f1 = __uint_as_float(acc_bits[2 * i + 1]) * p.alpha;
      if (2 * i < ncols_valid) {
        if (b) f0 += to_f32<T>(b[2 * i]);
        if (rs) f0 += to_f32<T>(rs[2 * i]);
      }
      if (2 * i + 1 < ncols_valid) {
        if (b) f1 += to_f32<T>(b[2 * i + 1]);
        if (rs) f1 += to_f32<T>(rs[2 * i + 1]);
      }
      pk[i] = pack2<T>(f0, f1);
    }
  }
}

// 32 values of row `r`, already packed to 16-bit pairs, -> the staging tile (piece 0 or 1 of the row's chunk)
__device__ __forceinline__ void stage_packed32(uint8_t* staging, int r, int piece, const uint32_t* pk) {
  uint8_t* rowp = staging + r * 128;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int j = piece * 4 + i;
    *reinterpret_cast<uint4*>(rowp + ((j ^ (r & 7)) << 4)) =
        make_uint4(pk[i * 4], pk[i * 4 + 1], pk[i * 4 + 2], pk[i * 4 + 3]);
  }
}

template <typename T, int MT, int EPI, bool A_MN, bool B_MN, typename Hooks>
__device__ __forceinline__ void gemm_pair_body(const CUtensorMap* tma_a, const CUtensorMap* tma_b,
                                               const CUtensorMap* tma_c, const GemmParams& p, const Hooks& hooks,
                                               uint8_t* smem_raw, int cluster_id, int num_clusters) {
  using C = PairCfg<MT>;
  constexpr int STAGES = C::STAGES;
  // every flavour but the full one writes 16-bit output through the staged TMA store
  constexpr bool LEAN = EPI != EPI_FULL;
  static_assert(EPI == EPI_LEAN || MT == 1, "512-row tiles exist for the lean flavour only");
  // both CTAs of a pair must use the same shared-memory offsets (the MMA addresses the peer's
  // operands by offset, remote arrivals address barriers by offset); the dynamic segment starts at
  // the same offset in every CTA of a kernel, so aligning the same way gives the same layout
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * C::A_BYTES;
  uint8_t* sStage = sB + STAGES * G2_B_BYTES;                    // [2 halves][128 rows][128 bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + C::STAGING);
  uint64_t* full_bar = bars;                        // leader's are used: both CTAs' copies complete here
  uint64_t* empty_bar = bars + STAGES;              // per CTA: the leader's commits release the stage
  uint64_t* tmem_full_bar = bars + 2 * STAGES;      // [2] per CTA
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;     // [2] leader's are used (16 arrivals)
  uint64_t* sched_full = tmem_empty_bar + 2;        // [kSchedSlots] per CTA (one arrival: the leader's producer)
  uint64_t* sched_empty = sched_full + kSchedSlots; // [kSchedSlots] leader's are used
  uint64_t* done_bar = sched_empty + kSchedSlots;   // per CTA: 16 arrivals (both CTAs' epilogue warps)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(done_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* tile_ring = abort_flag + 1;         // [kSchedSlots] tile ids, -1 = no more work

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();      // 0 = leader, 1 = peer
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    prefetch_tensormap(tma_a);
    prefetch_tensormap(tma_b);
    if (p.tma_store) prefetch_tensormap(tma_c);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), C::ACC_RELEASERS);
    }
    for (int s = 0; s < kSchedSlots; ++s) {
      mbar_init(smem_u32(&sched_full[s]), 1);
      mbar_init(smem_u32(&sched_empty[s]), G2_SCHED_CONSUMERS);
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
  cta_sync_pair();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // 384 threads compile to 168 registers each; the epilogue of 512-row tiles holds two drained
  // accumulators (128 packed words) per thread, the other warpgroup needs almost nothing

  const int num_m = (p.M + C::BM - 1) / C::BM;
  const int num_n = (p.N + G2_BN - 1) / G2_BN;
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  const int total_tiles = num_m * num_n;
  const int group_m = p.group_m > 0 ? p.group_m : 4;
  auto tile_coords = [&](int tile, int& m_idx, int& n_idx) {
    if constexpr (Hooks::kCustomRaster) {
      hooks.raster(tile, num_m, num_n, m_idx, n_idx);
    } else {
      const int group_size = group_m * num_n;
      const int g = tile / group_size;
      const int first_m = g * group_m;
      const int gm = min(num_m - first_m, group_m);
      const int r = tile - g * group_size;
      m_idx = first_m + r % gm;
      n_idx = r / gm;
    }
  };
  // 128-row block of the matrix that CTA `cta_rank` holds as row block j of tile row m_idx: MMA j of
  // the tile covers rows [256 j, 256 j + 256) of it, the leader's rows first
  auto row_block = [&](int m_idx, int j) { return (m_idx * MT + j) * 2 + (int)cta_rank; };
  constexpr int CH = 64;   // MN elements per 128-byte chunk of an MN-major operand

  if (warp_idx < G2_EPI_WARP0) {
  regs_release_to_64();
  if (warp_idx == 0) {
    // ------------------------------ scheduler (leader) + TMA producer (both CTAs) ------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int static_tile = cluster_id, slot = 0;
      uint32_t slot_phase = 0;
      while (ok) {
        int tile;
        if (leader) {
          if (p.sched) {
            tile = atomicAdd(p.sched, 1);
          } else {
            tile = static_tile;
            static_tile += num_clusters;
          }
          if (tile >= total_tiles) tile = -1;
          ok = mbar_wait_cluster(smem_u32(&sched_empty[slot]), slot_phase ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          tile_ring[slot] = tile;
          st_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(&tile_ring[slot])), 1), static_cast<uint32_t>(tile));
          mbar_arrive(smem_u32(&sched_full[slot]));
          mbar_arrive_cluster(map_to_cta(smem_u32(&sched_full[slot]), 1));
        } else {
          ok = mbar_wait_cluster(smem_u32(&sched_full[slot]), slot_phase, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tile = tile_ring[slot];
          mbar_arrive_cluster(map_to_cta(smem_u32(&sched_empty[slot]), 0));
        }
        if (++slot == kSchedSlots) { slot = 0; slot_phase ^= 1; }
        if (tile < 0) break;
        int m_idx, n_idx;
        tile_coords(tile, m_idx, n_idx);
        const int n0 = n_idx * G2_BN + (int)cta_rank * 128;      // this CTA's columns of B
#pragma unroll
        for (int j = 0; j < MT; ++j)
          if (ok) ok = hooks.before_tile_load(row_block(m_idx, j), n_idx, abort_flag, p.status);
        for (int kbi = 0; kbi < num_kb && ok; ++kbi) {
          const int kb = hooks.map_kb(kbi, num_kb);
          ok = hooks.before_k_load(row_block(m_idx, 0), n_idx, kb, abort_flag, p.status);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          const uint32_t leader_full = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * C::STAGE_BYTES);
          const uint32_t b_dst = smem_u32(sB + stage * G2_B_BYTES);
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            const uint32_t a_dst = smem_u32(sA + stage * C::A_BYTES + j * 128 * 128);
            const int m0 = row_block(m_idx, j) * 128;
            if constexpr (!A_MN) {
              tma_load_2d_pair(a_dst, tma_a, leader_full, kb * G2_BK, m0);
            } else {
#pragma unroll
              for (int c = 0; c < 128 / CH; ++c)
                tma_load_2d_pair(a_dst + c * G2_BK * 128, tma_a, leader_full, m0 + c * CH, kb * G2_BK);
            }
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(b_dst, tma_b, leader_full, kb * G2_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < 128 / CH; ++c)
              tma_load_2d_pair(b_dst + c * G2_BK * 128, tma_b, leader_full, n0 + c * CH, kb * G2_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land
    }
  } else if (warp_idx == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ---------------------------
    if (leader) {
      constexpr uint32_t idesc = make_idesc(UmmaFormat<T>::value, A_MN ? 1 : 0, B_MN ? 1 : 0, 256, G2_BN);
      int stage = 0, slot = 0;
      uint32_t phase = 0, slot_phase = 0;
      uint32_t item = 0;          // accumulators handed out so far: buffer = item & 1, parity = (item >> 1) & 1
      bool ok = true;
      long long t_begin = 0, t_full = 0, t_tmem = 0, n_tiles = 0;
      if (p.dbg) t_begin = clock64();
      while (ok) {
        ok = mbar_wait(smem_u32(&sched_full[slot]), slot_phase, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
        if (!ok) break;
        const int tile = tile_ring[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sched_empty[slot]));
        if (++slot == kSchedSlots) { slot = 0; slot_phase ^= 1; }
        if (tile < 0) break;
        ++n_tiles;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          long long t0 = 0;
          if (p.dbg) t0 = clock64();
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
          if (!ok) break;
          if (p.dbg) t_full += clock64() - t0;
          tc_fence_after();
          const uint32_t b_base = smem_u32(sB + stage * G2_B_BYTES);
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            const uint32_t it = item + j;
            const int acc = it & 1;
            if (kb == 0) {
              if (p.dbg) t0 = clock64();
              ok = mbar_wait_cluster(smem_u32(&tmem_empty_bar[acc]), ((it >> 1) & 1) ^ 1, abort_flag, p.status,
                                     RB_ERR_TIMEOUT_TMEM_EMPTY);
              if (p.dbg) t_tmem += clock64() - t0;
              if (!ok) break;
              tc_fence_after();
            }
            const uint32_t tmem_d = tmem_base + acc * G2_BN;
            const uint32_t a_base = smem_u32(sA + stage * C::A_BYTES + j * 128 * 128);
#pragma unroll
            for (int k = 0; k < G2_BK / 16; ++k) {
              const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_base + k * 16 * 128, G2_BK * 128, 1024)
                                          : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
              const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_base + k * 16 * 128, G2_BK * 128, 1024)
                                          : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
              umma_f16_pair_w(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            if (kb == num_kb - 1) {
              // this accumulator is complete: hand it to both CTAs' epilogue warps
              umma_commit_pair_w(smem_u32(&tmem_full_bar[acc]));
              umma_commit_pair_w(map_to_cta(smem_u32(&tmem_full_bar[acc]), 1));
            }
          }
          if (!ok) break;
          // the stage is free again in both CTAs once these MMAs have read it
          umma_commit_pair_w(smem_u32(&empty_bar[stage]));
          umma_commit_pair_w(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        item += MT;
      }
      if (p.dbg && lane == 0) {
        long long* d = p.dbg + 8 * cluster_id;
        d[0] = clock64() - t_begin;
        d[1] = t_full;
        d[2] = t_tmem;
        d[3] = n_tiles;
      }
    }
  }
  } else {
    regs_grow_to_216();
    // ------------------------------ epilogue (both CTAs) -----------------------------------
    // The eight warps form two groups of four (one warp per TMEM lane quarter); group g handles
    // columns [128 g, 128 g + 128) of every accumulator and owns one staging tile.
    const int quarter = warp_idx & 3;
    const int group = (warp_idx - G2_EPI_WARP0) >> 2;
    const int group_bar = 3 + group;                    // named barrier of this group's 4 warps
    const bool issuer = (warp_idx & 3) == 0 && lane == 0;       // issues this group's TMA stores
    uint8_t* staging = sStage + group * G2_STAGING_BYTES;
    const int r_in_cta = quarter * 32 + lane;
    int slot = 0;
    uint32_t slot_phase = 0, item = 0;
    bool ok = true;
    const uint32_t leader_empty0 = map_to_cta(smem_u32(&tmem_empty_bar[0]), 0);
    const uint32_t leader_empty1 = map_to_cta(smem_u32(&tmem_empty_bar[1]), 0);
    const int osz = (!LEAN && p.out_f32) ? 4 : (int)sizeof(T);
    const int cw = 128 / osz;                           // columns per staged chunk (64 or 32)
    const int pieces = cw / 32;                         // 32-column pieces per chunk
    const bool use_tma = LEAN || p.tma_store;
    long long edbg[4] = {0, 0, 0, 0};   // cycles: full -> release (acc 0 / 1), full -> tile done; tiles
    while (ok) {
      ok = mbar_wait_cluster(smem_u32(&sched_full[slot]), slot_phase, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      ok = __all_sync(0xffffffffu, ok);
      const int tile = ok ? tile_ring[slot] : -1;
      __syncwarp();
      if (ok && lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&sched_empty[slot]), 0));
      if (++slot == kSchedSlots) { slot = 0; slot_phase ^= 1; }
      int m_idx = 0, n_idx = 0;
      if (tile >= 0) tile_coords(tile, m_idx, n_idx);
      const int col_g0 = n_idx * G2_BN + group * 128;
      if constexpr (LEAN && MT == 2) {
        // 512 x 256 tiles own all of TMEM, so the next tile's MMAs wait for this drain: both
        // accumulators are first emptied into registers (as packed 16-bit results) and handed back,
        // and only then written out
        uint32_t pk[2][4][16];
        long long t_a = 0;
        if (p.dbg) t_a = clock64();
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int acc = (item + j) & 1;
          const uint32_t acc_phase = ((item + j) >> 1) & 1;
          if (ok && tile >= 0) {
            ok = mbar_wait_cluster(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
          }
          ok = bar_vote_and(group_bar, 128, ok);        // the group goes on, or gives up, together
          const bool go = ok && tile >= 0;
          if (p.dbg && j == 0) t_a = clock64();
          tc_fence_after();
          const long long row = static_cast<long long>(row_block(m_idx, j)) * 128 + r_in_cta;
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * G2_BN + group * 128;
          // one 32-column piece at a time (load, epilogue arithmetic, pack); the accumulator goes back
          // to the MMA warp as soon as the last piece has landed in registers
          const bool rok = go && row < p.M;
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            uint32_t r[32];
            if (go) {
              tmem_ld_32x32b_x32(taddr + pc * 32, r);
              tmem_ld_wait();
            }
            if (pc == 3) {
              tc_fence_before();
              __syncwarp();
              if (go && lane == 0) mbar_arrive_cluster(acc == 0 ? leader_empty0 : leader_empty1);
              if (p.dbg && leader && warp_idx == G2_EPI_WARP0 && lane == 0) edbg[j] += clock64() - t_a;
            }
            const int c0 = col_g0 + pc * 32;
            lean_pack32<T>(p, r, row, c0, min(32, p.N - c0), rok, pk[j][pc]);
          }
        }
        if (!ok || tile < 0) break;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int m_blk = row_block(m_idx, j);
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            const int col0 = col_g0 + ch * 64;
            if (col0 < p.N && m_blk * 128 < p.M) {                // uniform over the group's 4 warps
              if (issuer) tma_store_wait_read<0>();
              bar_sync_named(group_bar, 128);
              stage_packed32(staging, r_in_cta, 0, pk[j][2 * ch]);
              stage_packed32(staging, r_in_cta, 1, pk[j][2 * ch + 1]);
              fence_proxy_async_smem();
              bar_sync_named(group_bar, 128);
              if (issuer) {
                tma_store_2d(tma_c, smem_u32(staging), col0, m_blk * 128);
                tma_store_commit();
              }
            }
          }
          if constexpr (Hooks::kNeedsStoreComplete) {
            if (issuer) tma_store_wait<0>();
            bar_sync_named(group_bar, 128);
          }
          if (lane == 0 && m_blk * 128 < p.M) hooks.after_tile_store(m_blk, n_idx, quarter);
        }
        if (p.dbg && leader && warp_idx == G2_EPI_WARP0 && lane == 0) { edbg[2] += clock64() - t_a; edbg[3] += 1; }
        item += MT;
        continue;
      }
      constexpr int gcols = 128;                        // columns of an accumulator this group handles
      const int gcol0 = group * 128;
      long long t_b = 0;
#pragma unroll 1
      for (int j = 0; j < MT; ++j) {
        const int acc = (item + j) & 1;
        const uint32_t acc_phase = ((item + j) >> 1) & 1;
        if (ok && tile >= 0) {
          ok = mbar_wait_cluster(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
          ok = __all_sync(0xffffffffu, ok);
        }
        // the four warps of a group meet at named barriers inside the tile: they go on, or give
        // up, together (a wait that ran out in one warp must not leave the others at a barrier)
        ok = bar_vote_and(group_bar, 128, ok);
        if (!ok || tile < 0) break;
        tc_fence_after();
        const int m_blk = row_block(m_idx, j);
        const long long row = static_cast<long long>(m_blk) * 128 + r_in_cta;
        const bool row_ok = row < p.M;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * G2_BN + gcol0;
        const uint32_t leader_empty = acc == 0 ? leader_empty0 : leader_empty1;
        if (p.dbg) t_b = clock64();
        if (use_tma) {
          const int nchunks = gcols / cw;
#pragma unroll 1
          for (int ch = 0; ch < nchunks; ++ch) {
            const int col0 = n_idx * G2_BN + gcol0 + ch * cw;
            const bool live = col0 < p.N && m_blk * 128 < p.M;    // uniform over the group's 4 warps
            float v[2][32];
            uint32_t r[2][32];
            if (live) {
#pragma unroll
              for (int pc = 0; pc < 2; ++pc)
                if (pc < pieces) tmem_ld_32x32b_x32(taddr + ch * cw + pc * 32, r[pc]);
              tmem_ld_wait();
            }
            if (ch == nchunks - 1) {
              // the accumulator has been read completely: hand it back before the arithmetic and the stores
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(leader_empty);
              if (p.dbg && leader && warp_idx == G2_EPI_WARP0 && lane == 0) edbg[0] += clock64() - t_b;
            }
            if (live) {
#pragma unroll
              for (int pc = 0; pc < 2; ++pc) {
                if (pc < pieces) {
                  const int col = col0 + pc * 32;
                  const int ncols_valid = min(32, p.N - col);
                  if constexpr (LEAN)
                    epilogue_math32<T, T, EPI>(p, r[pc], row, col, ncols_valid, row_ok, v[pc]);
                  else if (p.out_f32)
                    epilogue_math32<T, float>(p, r[pc], row, col, ncols_valid, row_ok, v[pc]);
                  else
                    epilogue_math32<T, T>(p, r[pc], row, col, ncols_valid, row_ok, v[pc]);
                }
              }
            }
            if (!live) continue;
            // the previous chunk's TMA store must have finished reading the staging tile
            if (issuer) tma_store_wait_read<0>();
            bar_sync_named(group_bar, 128);
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
              if (pc < pieces) {
                if constexpr (LEAN)
                  stage_row32<T>(staging, r_in_cta, pc, v[pc]);
                else if (p.out_f32)
                  stage_row32<float>(staging, r_in_cta, pc, v[pc]);
                else
                  stage_row32<T>(staging, r_in_cta, pc, v[pc]);
              }
            }
            fence_proxy_async_smem();
            bar_sync_named(group_bar, 128);
            if (issuer) {
              tma_store_2d(tma_c, smem_u32(staging), col0, m_blk * 128);
              tma_store_commit();
            }
          }
          if constexpr (Hooks::kNeedsStoreComplete) {
            if (issuer) tma_store_wait<0>();
            bar_sync_named(group_bar, 128);
          }
        } else if constexpr (!LEAN) {
#pragma unroll 1
          for (int ci = 0; ci < gcols / 32; ++ci) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + ci * 32, r);
            tmem_ld_wait();
            const int col = n_idx * G2_BN + gcol0 + ci * 32;
            const int ncols_valid = min(32, p.N - col);
            if (row_ok && ncols_valid > 0) {
              if (p.out_f32)
                epilogue_chunk<T, float>(p, r, row, col, ncols_valid);
              else
                epilogue_chunk<T, T>(p, r, row, col, ncols_valid);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_empty);
        }
        if (lane == 0 && m_blk * 128 < p.M) hooks.after_tile_store(m_blk, n_idx, quarter);
        if (p.dbg && leader && warp_idx == G2_EPI_WARP0 && lane == 0) { edbg[2] += clock64() - t_b; edbg[3] += 1; }
      }
      if (!ok || tile < 0) break;
      item += MT;
    }
    if (p.dbg && leader && warp_idx == G2_EPI_WARP0 && lane == 0) {
      long long* d = p.dbg + 8 * cluster_id + 4;
      d[0] = edbg[0]; d[1] = edbg[1]; d[2] = edbg[2]; d[3] = edbg[3];
    }
    // the staging tile must outlive the last store's read; then this warp will not touch TMEM or
    // signal any barrier again: tell both CTAs
    if (issuer) tma_store_wait_read<0>();
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
    bool ok = mbar_wait_cluster(smem_u32(done_bar), 0, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_EMPTY);
    (void)ok;
  }
  tc_fence_before();
  cta_sync_pair();
  if (warp_idx == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, G2_TMEM_COLS);
  }
  if (threadIdx.x == 0 && leader && p.sched) {
    // the last cluster to leave re-arms the scheduler words for the next launch that uses this slot
    const int prev = atomicAdd(p.sched + 1, 1);
    if (prev == num_clusters - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

}  // namespace rb
