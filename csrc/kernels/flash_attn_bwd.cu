// FlashAttention backward for sm_100a (tcgen05 + TMEM + TMA), head_dim 128.
//
// One CTA (14 warps: 8 softmax, 4 dQ drain, 1 TMA, 1 MMA) owns a 128-row K/V tile of
// one (batch, kv-head) and sweeps the query tiles (64 rows each) that attend to it.  All five GEMMs of a tile pair run on
// tcgen05 with M = 128 by working on transposed score tiles:
//
//   S^T  [kv x q] = K . Q^T                 (recomputed)
//   dP^T [kv x q] = V . dO^T
//   P^T = exp2(S^T * c - LSE),  dS^T = P^T * (dP^T - D) * scale      (registers -> smem)
//   dV  [kv x d] += P^T  . dO                (accumulates in TMEM across q tiles)
//   dK  [kv x d] += dS^T . Q                 (accumulates in TMEM across q tiles)
//   dQ^T [d x q]  = K^T . dS^T               (read back, red.add into an fp32 dQ buffer)
//
// Every shared tile is a stack of [rows x 64] 128B-swizzled sub-tiles, which the
// tensor core can read either K-major (row = M/N index) or MN-major (row = K
// index), so Q, dO and K each serve two GEMMs from one copy.
//
// The reference has no fused attention backward: it re-runs the materialised
// softmax(QK^T)V composition when gradients are needed
// (rumus/src/tensor/ops.rs:2693-2709, rumus/src/nn/attention.rs:17-58).
#include "sm100_common.cuh"

namespace rb {

struct FaBwdParams {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale, scale_log2;
  const float* lse2;   // [B,H,sq_pad]  log-sum-exp in base-2 units (lse * log2 e)
  const float* delta;  // [B,H,sq_pad]  rowsum(dO * O)
  int sq_pad;          // row stride of both, a multiple of 64; padding holds finite values
  float* dq_accum;     // [B,Sq,H,128] fp32, zero-initialised
  void* dk;            // [B,Sk,Hkv,128] with element strides dkv_sb / dkv_ss / dkv_sh
  void* dv;            // same strides as dk
  long long dkv_sb, dkv_ss, dkv_sh;
  int* status;
};

struct FaBwdCfg {
  static constexpr int HD = 128, BKV = 128, BQ = 64, SUB = 2;
  static constexpr int KV_TILE = 128 * 128 * 2;   // [128 x 128] 16-bit = 32 KB (2 sub-tiles of 16 KB)
  static constexpr int KV_SUB = 128 * 128;        // 16 KB
  static constexpr int Q_TILE = 64 * 128 * 2;     // [64 x 128] = 16 KB (2 sub-tiles of 8 KB)
  static constexpr int Q_SUB = 64 * 128;          // 8 KB
  static constexpr int PT_BYTES = 128 * 128;      // [128 kv x 64 q] = 16 KB
  static constexpr int STAGES = 3;                // Q / dO ring
  static constexpr int SMEM_BYTES = 2 * KV_TILE + STAGES * 2 * Q_TILE + 2 * PT_BYTES +
                                    STAGES * 2 * 64 * 4 /*lse2, delta per stage*/ + 1024 + 256;
  // TMEM columns.  S^T is double buffered; dP^T and dQ^T of one iteration share a buffer (dP^T has
  // been consumed by the time dS^T exists), and that shared buffer is double buffered as well.
  // Once a softmax warp has read its 32 fp32 columns of S^T it writes P^T (16-bit, two values per
  // column) over the first 16 of them and dS^T over the last 16: the dV and dK GEMMs take their A
  // operand from there, which keeps 48 KB per tile off the shared-memory port (the port, not the
  // tensor pipe, is what limits this kernel).
  static constexpr int COL_ST = 0, COL_DPD = 128, COL_DV = 256, COL_DK = 384;
  // warp roles
  static constexpr int SOFTMAX_WARPS = 8, DRAIN_WARP0 = 8, TMA_WARP = 12, MMA_WARP = 13;
  static constexpr int THREADS = 14 * 32;
};
static_assert(FaBwdCfg::SMEM_BYTES <= 227 * 1024, "shared memory budget");

// Pipeline (b = it & 1, s = it % 3):
//   MMA warp      scores(it+1) -> S^T[b^1], dP^T[b^1]   |  wait P^T/dS^T(it)  |  dV, dK, dQ^T(it)
//   softmax x8    S^T[b] -> P^T[b] (smem), dP^T[b] -> dS^T[b] (smem)           (two warps per lane
//                 quarter, 32 query columns each)
//   drain x4      dQ^T[b] -> red.add into the fp32 dQ buffer
// so the exponentials of tile it+1, the accumulate GEMMs of tile it and the dQ atomics of tile
// it-1 run at the same time.
template <typename T>
__global__ void __launch_bounds__(FaBwdCfg::THREADS, 1)
    fa_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                  const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                  const FaBwdParams p) {
  using C = FaBwdCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::KV_TILE;
  uint8_t* sQ = sV + C::KV_TILE;               // [STAGES][Q_TILE]
  uint8_t* sdO = sQ + C::STAGES * C::Q_TILE;   // [STAGES][Q_TILE]
  uint8_t* sdST = sdO + C::STAGES * C::Q_TILE;  // [2][PT_BYTES]  (B operand of the dQ^T GEMM)
  float* sStat = reinterpret_cast<float*>(sdST + 2 * C::PT_BYTES);  // [STAGES][lse2 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + C::STAGES * 128);
  uint64_t* kv_full = bars;         // 1
  uint64_t* q_full = bars + 1;      // [3]
  uint64_t* q_empty = bars + 4;     // [3]
  uint64_t* st_full = bars + 7;     // [2]
  uint64_t* dpt_full = bars + 9;    // [2]
  uint64_t* pds_ready = bars + 11;  // [2]  P^T, dS^T of the tile are in place
  uint64_t* dq_full = bars + 13;    // [2]
  uint64_t* dq_free = bars + 15;    // [2]
  uint64_t* all_done = bars + 19;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x;
  const int hkv = blockIdx.y, b = blockIdx.z;
  const int group = p.H / p.Hkv;
  const int kv0 = kv_tile * C::BKV;
  const int off = p.Sk - p.Sq;
  const int n_q_tiles = (p.Sq + C::BQ - 1) / C::BQ;
  int q_tile_start = 0;
  if (p.causal) {
    const int first_q = kv0 - off;  // first query row that can see kv0
    q_tile_start = first_q > 0 ? first_q / C::BQ : 0;
  }
  const int tiles_per_head = n_q_tiles > q_tile_start ? n_q_tiles - q_tile_start : 0;
  const int n_iters = tiles_per_head * group;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tq);
    prefetch_tensormap(&tk);
    prefetch_tensormap(&tv);
    prefetch_tensormap(&tdo);
    mbar_init(smem_u32(kv_full), 1);
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&q_full[s]), 1);
      mbar_init(smem_u32(&q_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&st_full[s]), 1);
      mbar_init(smem_u32(&dpt_full[s]), 1);
      mbar_init(smem_u32(&pds_ready[s]), C::SOFTMAX_WARPS * 32);
      mbar_init(smem_u32(&dq_full[s]), 1);
      mbar_init(smem_u32(&dq_free[s]), 128);
    }
    mbar_init(smem_u32(all_done), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp_idx == C::MMA_WARP) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  auto iter_coords = [&](int it, int& qh, int& q0) {
    const int g = it / tiles_per_head;
    const int ti = it - g * tiles_per_head;
    qh = hkv * group + g;
    q0 = (q_tile_start + ti) * C::BQ;
  };

  if (warp_idx == C::TMA_WARP) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && n_iters > 0) {
      mbar_arrive_expect_tx(smem_u32(kv_full), 2 * C::KV_TILE);
#pragma unroll
      for (int s = 0; s < C::SUB; ++s) {
        tma_load_4d(smem_u32(sK + s * C::KV_SUB), &tk, smem_u32(kv_full), s * 64, kv0, hkv, b);
        tma_load_4d(smem_u32(sV + s * C::KV_SUB), &tv, smem_u32(kv_full), s * 64, kv0, hkv, b);
      }
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      for (int it = 0; it < n_iters && ok; ++it) {
        ok = mbar_wait(smem_u32(&q_empty[st]), ph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        int qh, q0;
        iter_coords(it, qh, q0);
        const uint32_t bar = smem_u32(&q_full[st]);
        mbar_arrive_expect_tx(bar, 2 * C::Q_TILE + 2 * 64 * 4);
        {
          // this tile's 64 row statistics ride on the same barrier
          const long long srow = (static_cast<long long>(b) * p.H + qh) * p.sq_pad + q0;
          bulk_load_1d(smem_u32(sStat + st * 128), p.lse2 + srow, 64 * 4, bar);
          bulk_load_1d(smem_u32(sStat + st * 128 + 64), p.delta + srow, 64 * 4, bar);
        }
#pragma unroll
        for (int s = 0; s < C::SUB; ++s) {
          tma_load_4d(smem_u32(sQ + st * C::Q_TILE + s * C::Q_SUB), &tq, bar, s * 64, q0, qh, b);
          tma_load_4d(smem_u32(sdO + st * C::Q_TILE + s * C::Q_SUB), &tdo, bar, s * 64, q0, qh, b);
        }
        if (++st == C::STAGES) {
          st = 0;
          ph ^= 1;
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
    }
  } else if (warp_idx == C::MMA_WARP) {
    // ------------------------------ MMA issuer --------------------------------
    if (n_iters > 0) {   // whole warp; one elected lane issues each instruction
      constexpr int F = UmmaFormat<T>::value;
      constexpr uint32_t idesc_st = make_idesc(F, 0, 0, 128, 64);    // K(A,Kmaj) x Q(B,Kmaj)
      constexpr uint32_t idesc_acc = make_idesc(F, 0, 1, 128, 128);  // P^T(A,Kmaj) x dO(B,N-maj)
      constexpr uint32_t idesc_dq = make_idesc(F, 1, 1, 128, 64);    // K^T(A,M-maj) x dS^T(B,N-maj)
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV);
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      // S^T and dP^T of tile `it` from Q/dO stage `st` into TMEM buffer it & 1
      auto issue_scores = [&](int it, int st) {
        const int buf = it & 1;
        const uint32_t q_base = smem_u32(sQ + st * C::Q_TILE);
        const uint32_t do_base = smem_u32(sdO + st * C::Q_TILE);
        // the two accumulators are interleaved: back-to-back MMAs into one accumulator would
        // each wait for the previous one's write-back
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // K dim = head_dim 128
          const uint32_t oa = (k >> 2) * C::KV_SUB + (k & 3) * 32;
          const uint32_t ob = (k >> 2) * C::Q_SUB + (k & 3) * 32;
          umma_f16_w(tmem_base + C::COL_ST + buf * 64, make_smem_desc_sw128(k_base + oa, 16, 1024),
                   make_smem_desc_sw128(q_base + ob, 16, 1024), idesc_st, k != 0);
          umma_f16_w(tmem_base + C::COL_DPD + buf * 64, make_smem_desc_sw128(v_base + oa, 16, 1024),
                   make_smem_desc_sw128(do_base + ob, 16, 1024), idesc_st, k != 0);
        }
        umma_commit_w(smem_u32(&st_full[buf]));
        umma_commit_w(smem_u32(&dpt_full[buf]));
      };
      if (ok) {
        ok = mbar_wait(smem_u32(&q_full[0]), 0, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after();
          issue_scores(0, 0);
        }
      }
      int st = 0;            // Q/dO stage of tile `it`
      uint32_t st_ph = 0;    // its ring phase
      for (int it = 0; it < n_iters && ok; ++it) {
        const int buf = it & 1;
        const uint32_t bph = (it >> 1) & 1;
        int st_n = st + 1;
        uint32_t ph_n = st_ph;
        if (st_n == C::STAGES) {
          st_n = 0;
          ph_n ^= 1;
        }
        if (it + 1 < n_iters) {
          ok = mbar_wait(smem_u32(&q_full[st_n]), ph_n, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
          if (!ok) break;
          if (it >= 1) {
            // the dP^T/dQ^T buffer of tile it+1 last held dQ^T of tile it-1: wait for its drain
            ok = mbar_wait(smem_u32(&dq_free[buf ^ 1]), ((it - 1) >> 1) & 1, abort_flag, p.status,
                           RB_ERR_TIMEOUT_TMEM_EMPTY);
            if (!ok) break;
          }
          tc_fence_after();
          issue_scores(it + 1, st_n);
        }
        ok = mbar_wait(smem_u32(&pds_ready[buf]), bph, abort_flag, p.status, RB_ERR_TIMEOUT_FLAG);
        if (!ok) break;
        tc_fence_after();
        const uint32_t q_base = smem_u32(sQ + st * C::Q_TILE);
        const uint32_t do_base = smem_u32(sdO + st * C::Q_TILE);
        const uint32_t dst_base = smem_u32(sdST + buf * C::PT_BYTES);
        const uint32_t pt_tmem = tmem_base + C::COL_ST + buf * 64;
        // dV += P^T . dO ; dK += dS^T . Q      (K dim = 64 query rows -> 4 steps; A from TMEM:
        // query columns [32h, 32h+32) live packed in columns 32h + {0..15} (P^T) / {16..31} (dS^T))
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          umma_f16_ts_w(tmem_base + C::COL_DV, pt_tmem + (k >> 1) * 32 + (k & 1) * 8,
                      make_smem_desc_sw128(do_base + k * 2048, C::Q_SUB, 1024), idesc_acc,
                      (it | k) != 0);
          umma_f16_ts_w(tmem_base + C::COL_DK, pt_tmem + 16 + (k >> 1) * 32 + (k & 1) * 8,
                      make_smem_desc_sw128(q_base + k * 2048, C::Q_SUB, 1024), idesc_acc,
                      (it | k) != 0);
          // dQ^T = K^T . dS^T  (K dim = 128 kv rows -> 8 steps) into the buffer dP^T(it) occupied
#pragma unroll
          for (int k2 = 2 * k; k2 < 2 * k + 2; ++k2)
            umma_f16_w(tmem_base + C::COL_DPD + buf * 64,
                     make_smem_desc_sw128(k_base + k2 * 2048, C::KV_SUB, 1024),
                     make_smem_desc_sw128(dst_base + k2 * 2048, C::PT_BYTES, 1024), idesc_dq,
                     k2 != 0);
        }
        umma_commit_w(smem_u32(&dq_full[buf]));
        umma_commit_w(smem_u32(&q_empty[st]));
        st = st_n;
        st_ph = ph_n;
      }
      if (ok) umma_commit_w(smem_u32(all_done));
    }
  } else if (warp_idx >= C::DRAIN_WARP0 && warp_idx < C::DRAIN_WARP0 + 4) {
    // ------------------------------ dQ drain warps ------------------------------
    if (n_iters > 0) {
      const int t = (warp_idx & 3) * 32 + lane;  // TMEM lane == d index of dQ^T
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp_idx & 3) * 32) << 16);
      bool ok = true;
      for (int it = 0; it < n_iters; ++it) {
        const int buf = it & 1;
        int qh, q0;
        iter_coords(it, qh, q0);
        ok = mbar_wait(smem_u32(&dq_full[buf]), (it >> 1) & 1, abort_flag, p.status,
                       RB_ERR_TIMEOUT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float* dq_base =
            p.dq_accum + ((static_cast<long long>(b) * p.Sq + q0) * p.H + qh) * C::HD + t;
        const long long qstride = static_cast<long long>(p.H) * C::HD;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(lane_addr + C::COL_DPD + buf * 64, r0);
        tmem_ld_32x32b_x32(lane_addr + C::COL_DPD + buf * 64 + 32, r1);
        tmem_ld_wait();
        // the values are in registers: hand the TMEM buffer back before the atomics
        tc_fence_before();
        mbar_arrive(smem_u32(&dq_free[buf]));
        if (q0 + C::BQ <= p.Sq) {
#pragma unroll
          for (int i = 0; i < 32; ++i) atomicAdd(dq_base + i * qstride, __uint_as_float(r0[i]));
#pragma unroll
          for (int i = 0; i < 32; ++i)
            atomicAdd(dq_base + (32 + i) * qstride, __uint_as_float(r1[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (q0 + i < p.Sq) atomicAdd(dq_base + i * qstride, __uint_as_float(r0[i]));
            if (q0 + 32 + i < p.Sq)
              atomicAdd(dq_base + (32 + i) * qstride, __uint_as_float(r1[i]));
          }
        }
      }
    }
  } else if (warp_idx < C::SOFTMAX_WARPS && n_iters > 0) {
    // ------------------------------ softmax warps ------------------------------
    const int t = (warp_idx & 3) * 32 + lane;   // kv row within tile == TMEM lane
    const int half = warp_idx >> 2;             // which 32 query columns
    const int kv = kv0 + t;
    const bool kv_ok = kv < p.Sk;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp_idx & 3) * 32) << 16);
    bool ok = true;
    int stage = 0;   // Q/dO/statistics ring slot of tile `it`
    for (int it = 0; it < n_iters; ++it) {
      const int buf = it & 1;
      const uint32_t bph = (it >> 1) & 1;
      int qh, q0;
      iter_coords(it, qh, q0);
      // S^T complete implies the tile's TMA stage (and with it the statistics) has landed
      ok = mbar_wait(smem_u32(&st_full[buf]), bph, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float4* lse_t = reinterpret_cast<const float4*>(sStat + stage * 128 + half * 32);
      const float4* delta_t = reinterpret_cast<const float4*>(sStat + stage * 128 + 64 + half * 32);
      if (++stage == C::STAGES) stage = 0;
      // no masking needed when the whole tile is in range and below the causal diagonal
      const bool full_tile = kv0 + C::BKV <= p.Sk && q0 + C::BQ <= p.Sq &&
                             (!p.causal || kv0 + C::BKV - 1 <= q0 + off);
      const uint32_t st_addr = lane_addr + C::COL_ST + buf * 64 + half * 32;
      float pr[32];
      {
        uint32_t r[32];
        tmem_ld_32x32b_x32(st_addr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 l4 = lse_t[i4];
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = i4 * 4 + j;
            pr[i] = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -ls[j]));
          }
        }
        if (!full_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int q = q0 + half * 32 + i;
            const bool valid = kv_ok && q < p.Sq && (!p.causal || kv <= q + off);
            pr[i] = valid ? pr[i] : 0.f;
          }
        }
      }
      // P^T (16-bit pairs) over this warp's first 16 S^T columns
      {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(pr[2 * i], pr[2 * i + 1]);
        tmem_st_32x32b_x16(st_addr, pk);
      }
      ok = mbar_wait(smem_u32(&dpt_full[buf]), bph, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + C::COL_DPD + buf * 64 + half * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 d4 = delta_t[i4];
          const float ds[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = i4 * 4 + j;
            pr[i] = pr[i] * (__uint_as_float(r[i]) - ds[j]) * p.scale;
          }
        }
      }
      if (it >= 2) {
        // the dS^T shared buffer of tile it-2 must have been consumed by its dQ^T GEMM
        ok = mbar_wait(smem_u32(&dq_full[buf]), ((it - 2) >> 1) & 1, abort_flag, p.status,
                       RB_ERR_TIMEOUT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(pr[2 * i], pr[2 * i + 1]);
        // dS^T: TMEM copy (A of the dK GEMM) and swizzled shared copy (B of the dQ^T GEMM)
        tmem_st_32x32b_x16(st_addr + 16, pk);
        uint8_t* rowp = sdST + buf * C::PT_BYTES + t * 128;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const int cc = half * 4 + c4;
          *reinterpret_cast<uint4*>(rowp + ((cc ^ (t & 7)) << 4)) =
              make_uint4(pk[c4 * 4], pk[c4 * 4 + 1], pk[c4 * 4 + 2], pk[c4 * 4 + 3]);
        }
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&pds_ready[buf]));
    }
    if (ok) {
      ok = mbar_wait(smem_u32(all_done), 0, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      // warps 0-3 store dV, warps 4-7 store dK
      tc_fence_after();
      const long long orow = static_cast<long long>(b) * p.dkv_sb + kv * p.dkv_ss + hkv * p.dkv_sh;
      T* outp = reinterpret_cast<T*>(half == 0 ? p.dv : p.dk) + orow;
      const uint32_t col0 = half == 0 ? C::COL_DV : C::COL_DK;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_addr + col0 + c * 32, r);
        tmem_ld_wait();
        if (kv_ok) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            T* e = reinterpret_cast<T*>(&v);
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(__uint_as_float(r[q * 8 + i]));
            *reinterpret_cast<uint4*>(outp + c * 32 + q * 8) = v;
          }
        }
      }
    }
  } else if (n_iters == 0) {
    // no query tile attends to this K/V tile: gradients are zero
    const int t = threadIdx.x;
    const int kv = kv0 + t;
    if (t < 128 && kv < p.Sk) {
      const long long orow = static_cast<long long>(b) * p.dkv_sb + kv * p.dkv_ss + hkv * p.dkv_sh;
      uint4 z = make_uint4(0, 0, 0, 0);
      for (int c = 0; c < C::HD / 8; ++c) {
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.dk) + orow + c * 8) = z;
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.dv) + orow + c * 8) = z;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp_idx == C::MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,q] = sum_d dO[b,q,h,d] * O[b,q,h,d] and lse2 = lse * log2(e), both written with the
// padded row stride the main kernel's bulk loads use.  HD = 128: half a warp per row, one 16-byte
// load of each tensor per lane.  Also converts nothing else: dq conversion is fa_dq_cast_kernel.
template <typename T>
__global__ void fa_bwd_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout,
                                    long long do_sb, long long do_ss, long long do_sh,
                                    const float* __restrict__ lse, float* __restrict__ delta,
                                    float* __restrict__ lse2, float* __restrict__ dq_zero, int B, int H, int Sq,
                                    int sq_pad) {
  const long long hw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const int l16 = threadIdx.x & 15;
  const long long total = static_cast<long long>(B) * Sq * H;
  const bool live = hw < total;
  const long long r = live ? hw : 0;
  const int h = r % H;
  const long long bq = r / H;
  const int q = bq % Sq;
  const int b = bq / Sq;
  float acc = 0.f;
  if (live) {
    // this row of the fp32 dQ accumulator starts at zero (the main kernel adds into it with reds)
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float4* dz = reinterpret_cast<float4*>(dq_zero + r * 128 + l16 * 8);
    dz[0] = z;
    dz[1] = z;
    const uint4 ov = *reinterpret_cast<const uint4*>(o + r * 128 + l16 * 8);
    const uint4 dv = *reinterpret_cast<const uint4*>(dout + b * do_sb + q * do_ss + h * do_sh + l16 * 8);
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* de = reinterpret_cast<const T*>(&dv);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += to_f32<T>(oe[j]) * to_f32<T>(de[j]);
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (live && l16 == 0) {
    const long long row = static_cast<long long>(b) * H + h;
    delta[row * sq_pad + q] = acc;
    lse2[row * sq_pad + q] = lse[row * Sq + q] * 1.4426950408889634f;
  }
}

// dq (fp32 accumulation buffer [B,Sq,H,128]) -> T with element strides {sb, ss, sh}
template <typename T>
__global__ void fa_dq_cast_kernel(const float* __restrict__ dq32, T* __restrict__ dq, long long sb,
                                  long long ss, long long sh, int B, int Sq, int H) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;  // 8 elements each
  const long long total = static_cast<long long>(B) * Sq * H * 16;
  if (i >= total) return;
  const int c = i & 15;
  const long long r = i >> 4;
  const int h = r % H;
  const long long bq = r / H;
  const int q = bq % Sq;
  const int b = bq / Sq;
  const float4 a0 = *reinterpret_cast<const float4*>(dq32 + i * 8);
  const float4 a1 = *reinterpret_cast<const float4*>(dq32 + i * 8 + 4);
  uint4 v;
  v.x = pack2<T>(a0.x, a0.y); v.y = pack2<T>(a0.z, a0.w);
  v.z = pack2<T>(a1.x, a1.y); v.w = pack2<T>(a1.z, a1.w);
  *reinterpret_cast<uint4*>(dq + b * sb + q * ss + h * sh + c * 8) = v;
}

template <typename T>
int launch_fa_bwd(int dtype, const void* q, const void* k, const void* v, const void* o,
                  const void* dout, const long long* qs, const long long* ks, const long long* vs,
                  const long long* dos, const float* lse, float* stats, const FaBwdParams& p,
                  cudaStream_t st) {
  using C = FaBwdCfg;
  {
    const long long rows = static_cast<long long>(p.B) * p.Sq * p.H;
    const int threads = 256;
    const long long blocks = (rows * 16 + threads - 1) / threads;
    fa_bwd_delta_kernel<T><<<(unsigned)blocks, threads, 0, st>>>(
        (const T*)o, (const T*)dout, dos[0], dos[1], dos[2], lse, stats,
        stats + static_cast<long long>(p.B) * p.H * p.sq_pad, p.dq_accum, p.B, p.H, p.Sq, p.sq_pad);
  }
  CUtensorMap tq, tk, tv, tdo;
  auto mk = [&](CUtensorMap* m, const void* base, const long long* s, int S, int heads, int rows) {
    uint64_t dims[4] = {(uint64_t)C::HD, (uint64_t)S, (uint64_t)heads, (uint64_t)p.B};
    uint64_t strides[4] = {2, (uint64_t)s[1] * 2, (uint64_t)s[2] * 2, (uint64_t)s[0] * 2};
    uint32_t box[4] = {64, (uint32_t)rows, 1, 1};
    return rbh::encode_tensor_map(m, dtype, 4, const_cast<void*>(base), dims, strides, box, 1);
  };
  int rc = mk(&tq, q, qs, p.Sq, p.H, C::BQ);
  if (!rc) rc = mk(&tk, k, ks, p.Sk, p.Hkv, C::BKV);
  if (!rc) rc = mk(&tv, v, vs, p.Sk, p.Hkv, C::BKV);
  if (!rc) rc = mk(&tdo, dout, dos, p.Sq, p.H, C::BQ);
  if (rc) return 1000 + rc;
  auto kern = fa_bwd_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return 2000 + (int)e;
  dim3 grid((p.Sk + C::BKV - 1) / C::BKV, p.Hkv, p.B);
  kern<<<grid, C::THREADS, C::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {
// head_dim must be 128.  Strides are {batch, seq, head} in elements.
// o is [B,Sq,H,128] contiguous; dq_accum is fp32 [B,Sq,H,128] scratch (zeroed by the first kernel);
// stats is fp32 scratch of 2*B*H*sq_pad elements, sq_pad = Sq rounded up to a multiple of 64,
// zero on entry (the kernel fills delta and the base-2 log-sum-exp; the padding must stay finite);
// dk/dv are [B,Sk,Hkv,128] views with element strides dkv_strides = {batch, seq, head}
// (rows of 128 contiguous, 16-byte aligned).
int rb_flash_attn_bwd(int dtype, int head_dim, const void* q, const void* k, const void* v,
                      const void* o, const void* dout, const float* lse, const long long* q_strides,
                      const long long* k_strides, const long long* v_strides,
                      const long long* do_strides, float* stats, float* dq_accum, void* dk,
                      void* dv, const long long* dkv_strides, int B, int H, int Hkv, int Sq, int Sk,
                      int causal, float scale, void* stream) {
  using namespace rb;
  if (head_dim != 128) return 20;
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0) return 0;
  FaBwdParams p;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk; p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.sq_pad = (Sq + 63) / 64 * 64;
  p.delta = stats;
  p.lse2 = stats + static_cast<long long>(B) * H * p.sq_pad;
  p.dq_accum = dq_accum; p.dk = dk; p.dv = dv;
  p.dkv_sb = dkv_strides[0]; p.dkv_ss = dkv_strides[1]; p.dkv_sh = dkv_strides[2];
  p.status = rbh::device_status_word();
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == rbh::DT_BF16)
    return launch_fa_bwd<__nv_bfloat16>(dtype, q, k, v, o, dout, q_strides, k_strides, v_strides, do_strides, lse, stats, p, st);
  if (dtype == rbh::DT_F16)
    return launch_fa_bwd<__half>(dtype, q, k, v, o, dout, q_strides, k_strides, v_strides, do_strides, lse, stats, p, st);
  return 20;
}

// dq32 [B,Sq,H,128] fp32 contiguous -> dq (dtype) with element strides {batch, seq, head}
int rb_fa_dq_cast(int dtype, const float* dq32, void* dq, const long long* strides, int B, int Sq,
                  int H, void* stream) {
  using namespace rb;
  const long long total = static_cast<long long>(B) * Sq * H * 16;
  if (total <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == rbh::DT_BF16)
    fa_dq_cast_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(dq32, (__nv_bfloat16*)dq, strides[0], strides[1], strides[2], B, Sq, H);
  else if (dtype == rbh::DT_F16)
    fa_dq_cast_kernel<__half><<<blocks, threads, 0, st>>>(dq32, (__half*)dq, strides[0], strides[1], strides[2], B, Sq, H);
  else
    return 20;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
