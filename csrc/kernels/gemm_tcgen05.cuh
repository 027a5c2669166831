// Persistent warp-specialised GEMM for sm_100a: TMA -> shared-memory ring ->
// tcgen05.mma (cta_group::1, 128 x BN x 16B-K tiles) -> fp32 accumulators in
// TMEM (double buffered) -> epilogue warps (tcgen05.ld) -> global memory.
//
//   C[M,N] = dact(aux_in) * ( act(alpha * A[M,K] . B[K,N] + bias[N]) ) + residual[M,N]
//
// Operand storage ("major") is a template parameter so that the forward
// (x @ W with W stored [in,out]), dgrad (dY @ W^T) and wgrad (X^T @ dY) GEMMs of
// a Linear layer all run without any transposition pass:
//   A_MN = false : A stored [M,K] row-major (K contiguous)     true : stored [K,M] (M contiguous)
//   B_MN = false : B stored [N,K] row-major (K contiguous)     true : stored [K,N] (N contiguous)
//
// The reference framework's counterpart is a one-thread-per-output naive matmul
// (rumus/src/backend/gpu/shaders/matmul.wgsl:22) plus separate bias / activation
// dispatches (shaders/bias.wgsl:20, shaders/unary.wgsl:20); here those are one kernel.
//
// Roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..9 = epilogue (TMEM lane quarter = warp_idx % 4; warps 2..5 take the left half of the
// tile's columns, warps 6..9 the right half, so an activation-heavy epilogue on a short-K GEMM
// keeps up with the main loop).
//
// `Hooks` lets the fused collective kernels (all-gather -> GEMM, GEMM ->
// reduce-scatter) reuse this body: the producer asks the hook before loading a
// tile (e.g. wait for a peer's slab to land in local staging), the epilogue
// tells the hook when an output tile is complete.
#pragma once
#include "sm100_common.cuh"

namespace rb {

enum : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SILU = 3 };

struct GemmParams {
  int M, N, K;
  void* out;             // [M,N], leading dim ldc, dtype = out_f32 ? float : T
  const void* bias;      // [N] of T (float when T = float) or null
  const void* residual;  // [M,N] of out dtype, leading dim ldr, or null
  void* aux_out;         // [M,N] of out dtype: receives (alpha*acc + bias) before act, or null
  const void* aux_in;    // [M,N] of out dtype: result is multiplied by dact'(aux_in), or null
  long long ldc, ldr, ldaux_out, ldaux_in;
  int act;               // activation on (alpha*acc + bias)
  int dact;              // derivative kind used with aux_in
  int out_f32;
  int vec_ok;            // 16-byte vector access is legal for out/residual/aux
  float alpha;
  int* status;           // device status word
  int group_m;           // raster group (m-tiles walked before advancing n)
  int* sched;            // device int[2] {next tile, finished CTAs} for dynamic tile scheduling, or null
  int split_k;           // > 1: K is cut into this many slices, every (tile, slice) is a work item and
                         // the epilogue adds into a zero-initialised fp32 output (no bias/act/residual)
  int tma_store;         // two-CTA kernel only: the output goes through shared memory and TMA stores
                         // (needs a 16-byte aligned base and row pitch); 0 = per-row stores
  long long* dbg;        // two-CTA kernel only: when set, every pair's MMA warp leaves {cycles in the
                         // kernel, cycles waiting for operands, cycles waiting for an accumulator, tiles}
};

struct NoHooks {
  // Called by the producer thread before the first load of an output tile.
  // Returning false aborts the kernel (bounded wait ran out).
  __device__ __forceinline__ bool before_tile_load(int m_idx, int n_idx, volatile int* abort_flag,
                                                   int* status) const {
    return true;
  }
  // Called by the producer thread before each k-block load.
  __device__ __forceinline__ bool before_k_load(int m_idx, int n_idx, int kb,
                                                volatile int* abort_flag, int* status) const {
    return true;
  }
  // Order in which the K blocks of a tile are consumed (a permutation of 0..num_kb-1).
  __device__ __forceinline__ int map_kb(int kb, int num_kb) const { return kb; }
  // Called by one lane of each epilogue warp after its 32 rows of a tile are stored.
  __device__ __forceinline__ void after_tile_store(int m_idx, int n_idx, int quarter) const {}
  // Operand loads / output rows other than "tile (m_idx, kb) of a row-major matrix" (implicit-GEMM
  // convolution: operand tiles are patches of an NHWC tensor, output rows are pixels of a patch).
  // When set, the hook provides load_a / load_b (issue the copies of one K block, which must add up to
  // the stage's byte count) and out_row (tile row -> output row index, negative = no such row).
  static constexpr bool kCustomLoadA = false;
  static constexpr bool kCustomLoadB = false;
  static constexpr bool kCustomRows = false;
  // Whether after_tile_store needs the tile's global writes to be complete (it publishes them to
  // other GPUs); the two-CTA body then drains its TMA stores first.
  static constexpr bool kNeedsStoreComplete = false;
  // Maps a linear tile id of this CTA to (m_idx, n_idx); default = grouped raster.
  static constexpr bool kCustomRaster = false;
  __device__ __forceinline__ void raster(int tile, int num_m, int num_n, int& m_idx,
                                         int& n_idx) const {}
};

// A hook type that defines `static constexpr bool kPushOut = true`, `void* push_base(int m_idx)` and
// `uint8_t* push_stage(int epilogue_warp)` (4 KB of shared memory per epilogue warp) makes the epilogue
// store each tile, rounded to T, at push_base(m_idx)[row_in_tile * N + col] instead of into `out`; the
// destination may be another GPU's memory, so the rows are written as whole 128-byte segments.
template <typename H, typename = void>
struct hook_push_out {
  static constexpr bool value = false;
};
template <typename H>
struct hook_push_out<H, decltype((void)H::kPushOut)> {
  static constexpr bool value = H::kPushOut;
};

template <typename T, int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int ESZ = sizeof(T);
  static constexpr int BK = 128 / ESZ;      // one 128-byte swizzle row of K
  static constexpr int UMMA_K = 32 / ESZ;   // K per tcgen05.mma
  static constexpr int CH = 128 / ESZ;      // MN elements per 128-byte chunk (MN-major operands)
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int NUM_THREADS = 320;
  static constexpr int EPI_WARPS = 8;
  static constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + 1024 /*align*/ + 384 /*barriers, scheduler ring*/;
};

// Barrier over the 320 GEMM threads (warps 0..9).  The fused collective kernels launch wider
// CTAs whose extra warps have a different role or have exited, so the count is explicit.
constexpr int kSchedSlots = 4;
constexpr int kGemmThreads = 320;
constexpr int kGemmEpiWarps = 8;
__device__ __forceinline__ void cta_sync_gemm() {
  asm volatile("bar.sync 0, 320;" ::: "memory");
}

template <typename T>
__device__ __forceinline__ void issue_umma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                           uint32_t acc) {
  if constexpr (sizeof(T) == 4)
    umma_tf32(d, a, b, idesc, acc);
  else
    umma_f16(d, a, b, idesc, acc);
}
// whole-warp form: one elected lane issues (see umma_f16_w)
template <typename T>
__device__ __forceinline__ void issue_umma_w(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                             uint32_t acc) {
  if constexpr (sizeof(T) == 4)
    umma_tf32_w(d, a, b, idesc, acc);
  else
    umma_f16_w(d, a, b, idesc, acc);
}

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case ACT_RELU: return fmaxf(v, 0.0f);
    case ACT_GELU: return gelu_tanh(v);
    case ACT_SILU: return silu_f(v);
    default: return v;
  }
}
__device__ __forceinline__ float apply_dact(float x, int dact) {
  switch (dact) {
    case ACT_RELU: return x > 0.0f ? 1.0f : 0.0f;
    case ACT_GELU: return gelu_tanh_grad(x);
    case ACT_SILU: return silu_grad(x);
    default: return 1.0f;
  }
}

// Loads 32 consecutive elements of row-major `base[row*ld + col ...]` as floats.
template <typename OT>
__device__ __forceinline__ void load_row32(const OT* base, long long ld, long long row, int col,
                                           int ncols_valid, bool vec, float* dst) {
  const OT* p = base + row * ld + col;
  if (vec && ncols_valid == 32) {
    constexpr int PER = 16 / sizeof(OT);
#pragma unroll
    for (int i = 0; i < 32 / PER; ++i) {
      uint4 v = *reinterpret_cast<const uint4*>(p + i * PER);
      const OT* e = reinterpret_cast<const OT*>(&v);
#pragma unroll
      for (int j = 0; j < PER; ++j) dst[i * PER + j] = to_f32<OT>(e[j]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) dst[i] = (i < ncols_valid) ? to_f32<OT>(p[i]) : 0.0f;
  }
}
template <typename OT>
__device__ __forceinline__ void store_row32(OT* base, long long ld, long long row, int col,
                                            int ncols_valid, bool vec, const float* src) {
  OT* p = base + row * ld + col;
  if (vec && ncols_valid == 32) {
    constexpr int PER = 16 / sizeof(OT);
#pragma unroll
    for (int i = 0; i < 32 / PER; ++i) {
      uint4 v;
      OT* e = reinterpret_cast<OT*>(&v);
#pragma unroll
      for (int j = 0; j < PER; ++j) e[j] = from_f32<OT>(src[i * PER + j]);
      *reinterpret_cast<uint4*>(p + i * PER) = v;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols_valid) p[i] = from_f32<OT>(src[i]);
  }
}

template <typename T, typename OT>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t* acc_bits,
                                               long long row, int col, int ncols_valid) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc_bits[i]) * p.alpha;
  if (p.bias) {
    const T* b = reinterpret_cast<const T*>(p.bias) + col;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols_valid) v[i] += to_f32<T>(b[i]);
  }
  const bool vec = p.vec_ok != 0;
  if (p.aux_out) store_row32<OT>(reinterpret_cast<OT*>(p.aux_out), p.ldaux_out, row, col, ncols_valid, vec, v);
  // one loop per activation kind: a switch inside the unrolled loop would lay down every kind 32
  // times, and an epilogue that is mostly code the call never runs costs more to fetch than to execute
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
  if (p.residual) {
    float r[32];
    load_row32<OT>(reinterpret_cast<const OT*>(p.residual), p.ldr, row, col, ncols_valid, vec, r);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += r[i];
  }
  store_row32<OT>(reinterpret_cast<OT*>(p.out), p.ldc, row, col, ncols_valid, vec, v);
}

// split-K epilogue: out (fp32) += alpha * acc, 16-byte vector reductions where the row allows
__device__ __forceinline__ void epilogue_chunk_atomic(const GemmParams& p, const uint32_t* acc_bits,
                                                      long long row, int col, int ncols_valid) {
  float* o = reinterpret_cast<float*>(p.out) + row * p.ldc + col;
  if (p.vec_ok && ncols_valid == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + i * 4),
                   "f"(__uint_as_float(acc_bits[i * 4]) * p.alpha),
                   "f"(__uint_as_float(acc_bits[i * 4 + 1]) * p.alpha),
                   "f"(__uint_as_float(acc_bits[i * 4 + 2]) * p.alpha),
                   "f"(__uint_as_float(acc_bits[i * 4 + 3]) * p.alpha)
                   : "memory");
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < ncols_valid) atomicAdd(o + i, __uint_as_float(acc_bits[i]) * p.alpha);
  }
}

template <typename T, int BN, bool A_MN, bool B_MN, typename Hooks>
__device__ __forceinline__ void gemm_cta_body(const CUtensorMap* tma_a, const CUtensorMap* tma_b,
                                              const GemmParams& p, const Hooks& hooks,
                                              uint8_t* smem_raw, int cta_rank, int num_ctas) {
  using C = GemmCfg<T, BN>;
  constexpr int BM = C::BM, BK = C::BK, UMMA_K = C::UMMA_K, CH = C::CH;
  constexpr int STAGES = C::STAGES;

  // carve shared memory (tiles need 1024-byte alignment for the 128B swizzle)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * C::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * C::B_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full_bar = bars + 2 * STAGES;
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;
  uint64_t* sched_full = bars + 2 * STAGES + 4;    // [kSchedSlots] producer -> MMA / epilogue
  uint64_t* sched_empty = sched_full + kSchedSlots;  // [kSchedSlots]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(sched_empty + kSchedSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* tile_ring = abort_flag + 1;           // [kSchedSlots] tile ids, -1 = no more work

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tensormap(tma_a);
    prefetch_tensormap(tma_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), kGemmEpiWarps);
    }
    for (int s = 0; s < kSchedSlots; ++s) {
      mbar_init(smem_u32(&sched_full[s]), 1);
      mbar_init(smem_u32(&sched_empty[s]), 1 + kGemmEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  cta_sync_gemm();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BK - 1) / BK;
  const int split_k = p.split_k > 1 ? p.split_k : 1;
  const int kb_per = (num_kb + split_k - 1) / split_k;   // K blocks per slice (no slice is empty)
  const int total_tiles = num_m * num_n * split_k;      // work items: (tile, K slice)
  const int group_m = p.group_m > 0 ? p.group_m : 8;

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

  if (warp_idx == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int static_tile = cta_rank, slot = 0;
      uint32_t slot_phase = 0;
      while (ok) {
        // Tile source: a device-wide atomic counter when p.sched is set (CTAs that start late —
        // e.g. because a communication kernel holds some SMs — simply take fewer tiles), else
        // the static stride.  The id is handed to the MMA and epilogue warps through a small ring.
        int tile;
        if (p.sched) {
          tile = atomicAdd(p.sched, 1);
        } else {
          tile = static_tile;
          static_tile += num_ctas;
        }
        if (tile >= total_tiles) tile = -1;
        ok = mbar_wait(smem_u32(&sched_empty[slot]), slot_phase ^ 1, abort_flag, p.status,
                       RB_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        tile_ring[slot] = tile;
        mbar_arrive(smem_u32(&sched_full[slot]));
        if (++slot == kSchedSlots) {
          slot = 0;
          slot_phase ^= 1;
        }
        if (tile < 0) break;
        int m_idx, n_idx;
        const int ks = tile % split_k;
        tile_coords(tile / split_k, m_idx, n_idx);
        const int kb_end = min(num_kb, (ks + 1) * kb_per);
        ok = hooks.before_tile_load(m_idx, n_idx, abort_flag, p.status);
        for (int kbi = ks * kb_per; kbi < kb_end && ok; ++kbi) {
          const int kb = hooks.map_kb(kbi, num_kb);
          ok = hooks.before_k_load(m_idx, n_idx, kb, abort_flag, p.status);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status,
                         RB_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[stage]);
          mbar_arrive_expect_tx(bar, C::A_BYTES + C::B_BYTES);
          const uint32_t a_dst = smem_u32(sA + stage * C::A_BYTES);
          const uint32_t b_dst = smem_u32(sB + stage * C::B_BYTES);
          if constexpr (Hooks::kCustomLoadA) {
            hooks.load_a(a_dst, tma_a, bar, m_idx, kb);
          } else if constexpr (!A_MN) {
            tma_load_2d(a_dst, tma_a, bar, kb * BK, m_idx * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / CH; ++j)
              tma_load_2d(a_dst + j * BK * 128, tma_a, bar, m_idx * BM + j * CH, kb * BK);
          }
          if constexpr (Hooks::kCustomLoadB) {
            hooks.load_b(b_dst, tma_b, bar, n_idx, kb);
          } else if constexpr (!B_MN) {
            tma_load_2d(b_dst, tma_b, bar, kb * BK, n_idx * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / CH; ++j)
              tma_load_2d(b_dst + j * BK * 128, tma_b, bar, n_idx * BN + j * CH, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // give copies that are still in flight time to land before the CTA retires
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
      }
    }
  } else if (warp_idx == 1) {
    // ------------------------------ MMA issuer --------------------------------
    {   // whole warp, uniform control flow; one elected lane issues each MMA / commit
      constexpr uint32_t idesc = make_idesc(UmmaFormat<T>::value, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int slot = 0;
      uint32_t slot_phase = 0;
      while (ok) {
        ok = mbar_wait(smem_u32(&sched_full[slot]), slot_phase, abort_flag, p.status,
                       RB_ERR_TIMEOUT_FULL);
        if (!ok) break;
        const int tile = tile_ring[slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sched_empty[slot]));
        if (++slot == kSchedSlots) {
          slot = 0;
          slot_phase ^= 1;
        }
        if (tile < 0) break;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status,
                       RB_ERR_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const int ks = tile % split_k;
        const int kb_n = min(num_kb, (ks + 1) * kb_per) - ks * kb_per;
        for (int kb = 0; kb < kb_n; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status,
                         RB_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + stage * C::A_BYTES);
          const uint32_t b_base = smem_u32(sB + stage * C::B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc =
                A_MN ? make_smem_desc_sw128(a_base + k * UMMA_K * 128, BK * 128, 1024)
                     : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc =
                B_MN ? make_smem_desc_sw128(b_base + k * UMMA_K * 128, BK * 128, 1024)
                     : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            issue_umma_w<T>(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_w(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_w(smem_u32(&tmem_full_bar[acc]));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp_idx & 3;
    const int half = (warp_idx - 2) >> 2;           // 0: left half of the columns, 1: right half
    constexpr int CHUNKS_PER_HALF = BN / 64;        // 32-column chunks per epilogue warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int slot = 0;
    uint32_t slot_phase = 0;
    while (ok) {
      ok = mbar_wait(smem_u32(&sched_full[slot]), slot_phase, abort_flag, p.status,
                     RB_ERR_TIMEOUT_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int tile = tile_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sched_empty[slot]));
      if (++slot == kSchedSlots) {
        slot = 0;
        slot_phase ^= 1;
      }
      if (tile < 0) break;
      int m_idx, n_idx;
      tile_coords(tile / split_k, m_idx, n_idx);
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status,
                     RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      long long row = static_cast<long long>(m_idx) * BM + quarter * 32 + lane;
      bool row_ok = row < p.M;
      if constexpr (Hooks::kCustomRows) {
        row = hooks.out_row(m_idx, quarter * 32 + lane);
        row_ok = row >= 0;
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if constexpr (hook_push_out<Hooks>::value && sizeof(T) == 2) {
        // Push mode: the tile goes to push_base(m_idx), which may be another GPU's memory, where 16-byte
        // pieces scattered over 32 rows travel badly.  Two 32-column chunks at a time are rounded to T,
        // laid down in this warp's 32 x 128-byte staging block (16-byte pieces XOR-swizzled by row) and
        // written out as whole 128-byte row segments: 8 lanes per row, 4 rows per instruction.
        uint8_t* stg = hooks.push_stage((warp_idx - 2));
        T* base = reinterpret_cast<T*>(hooks.push_base(m_idx)) + static_cast<long long>(quarter * 32) * p.N;
        const int rows_ok = static_cast<int>(min(32ll, static_cast<long long>(p.M) - (static_cast<long long>(m_idx) * BM + quarter * 32)));
#pragma unroll 1
        for (int ci = 0; ci < CHUNKS_PER_HALF; ci += 2) {
          const int c = half * CHUNKS_PER_HALF + ci;
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(taddr + c * 32, r0);
          tmem_ld_32x32b_x32(taddr + c * 32 + 32, r1);
          tmem_ld_wait();
          const int col0 = n_idx * BN + c * 32;
          const int valid = min(64, p.N - col0);          // columns of this 64-wide piece that exist
          uint8_t* myrow = stg + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t* src = j < 4 ? r0 + j * 8 : r1 + (j - 4) * 8;
            uint4 q;
            q.x = pack2<T>(__uint_as_float(src[0]) * p.alpha, __uint_as_float(src[1]) * p.alpha);
            q.y = pack2<T>(__uint_as_float(src[2]) * p.alpha, __uint_as_float(src[3]) * p.alpha);
            q.z = pack2<T>(__uint_as_float(src[4]) * p.alpha, __uint_as_float(src[5]) * p.alpha);
            q.w = pack2<T>(__uint_as_float(src[6]) * p.alpha, __uint_as_float(src[7]) * p.alpha);
            *reinterpret_cast<uint4*>(myrow + ((j ^ (lane & 7)) << 4)) = q;
          }
          __syncwarp();
          const int jj = lane & 7;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3);
            const uint4 q = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((jj ^ (rr & 7)) << 4));
            if (rr < rows_ok && jj * 8 < valid)
              *reinterpret_cast<uint4*>(base + static_cast<long long>(rr) * p.N + col0 + jj * 8) = q;
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
      for (int ci = 0; ci < CHUNKS_PER_HALF; ++ci) {
        const int c = half * CHUNKS_PER_HALF + ci;
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n_idx * BN + c * 32;
        const int ncols_valid = min(32, p.N - col);
        if (row_ok && ncols_valid > 0) {
          if (split_k > 1)
            epilogue_chunk_atomic(p, r, row, col, ncols_valid);
          else if (p.out_f32)
            epilogue_chunk<T, float>(p, r, row, col, ncols_valid);
          else
            epilogue_chunk<T, T>(p, r, row, col, ncols_valid);
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        hooks.after_tile_store(m_idx, n_idx, quarter);
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  cta_sync_gemm();
  if (warp_idx == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && p.sched) {
    // the last CTA to leave re-arms the scheduler words for the next launch that uses this slot
    const int prev = atomicAdd(p.sched + 1, 1);
    if (prev == num_ctas - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

}  // namespace rb
