// FlashAttention forward for sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA owns a 128-row query tile of one (batch, head).  K/V tiles of 128 rows stream through a
// 2-stage TMA ring.  S = Q K^T and O += P V run on tcgen05 with S (double buffered) and O in TMEM.
//
// Two softmax warpgroups take the K/V tiles in turn (even tiles: warps 0-3, odd tiles: warps 4-7).
// Inside a warpgroup a thread owns one whole query row (TMEM lane == row, all 128 key columns), so
// the row maximum and sum never leave the thread: no exchange between threads, no barrier inside the
// softmax.  Each warpgroup keeps its own running maximum / sum and its own O accumulator in TMEM
// (even tiles -> columns [256, 256+D), odd tiles -> [384, 384+D)), rescaled in place only when the
// maximum moved by more than 2^8 (lazy rescale); the two partial results are merged once at the end,
// the way split-KV decoding merges its partitions.  P goes to a 128B-swizzled shared tile (one per
// warpgroup) that the second MMA consumes.  exp is exp2 with the softmax scale folded in.  LSE is
// saved for the backward pass.
//
// Layout: q/k/v/o are [B, S, H, D] views with arbitrary batch/seq/head strides
// (so the fused qkv projection output is consumed in place); D in {64, 128}.
//
// The reference kernel (rumus/src/backend/gpu/shaders/flash_attn.wgsl:35) is a
// forward-only scalar loop: one thread per query row, K/V tiles of <= 16 rows in
// 16 KB of workgroup memory (rumus/src/backend/gpu/compute.rs:2079-2138).
#include "sm100_common.cuh"

namespace rb {

struct FaFwdParams {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  void* o;           // [B, Sq, H, D] contiguous
  float* lse;        // [B, H, Sq]
  int* status;
};

template <int HD>
struct FaFwdCfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int SUB = HD / 64;             // 64-column sub-tiles per row
  static constexpr int TILE_BYTES = 128 * 128;    // one [128 x 64] 16-bit sub-tile
  static constexpr int Q_BYTES = SUB * TILE_BYTES;
  static constexpr int KV_BYTES = SUB * TILE_BYTES;  // per K or V tile
  static constexpr int P_BYTES = 2 * TILE_BYTES;     // [128 x 128]
  static constexpr int STAGES = 2;
  static constexpr int P_BUFS = 2;   // P double buffered: softmax(j+1) overlaps P(j).V(j)
  static constexpr int SMEM_BYTES = Q_BYTES + STAGES * 2 * KV_BYTES + P_BUFS * P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int S_COL0 = 0;       // S buffers at columns [0,128) and [128,256)
  static constexpr int O_COL = 256;      // O of the even tiles at [256, 256+HD), of the odd tiles at [384, 384+HD)
};

template <typename T, int HD>
__global__ void __launch_bounds__(320, 1)
    fa_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                  const __grid_constant__ CUtensorMap tv, const FaFwdParams p) {
  using C = FaFwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;                       // [STAGES][KV_BYTES]
  uint8_t* sV = sK + C::STAGES * C::KV_BYTES;          // [STAGES][KV_BYTES]
  uint8_t* sP = sV + C::STAGES * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::P_BUFS * C::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2] K tile landed
  uint64_t* kv_empty = bars + 3;   // [2] K slot free again (its S GEMM retired)
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* p_ready = bars + 7;    // [2]
  uint64_t* pv_done = bars + 9;    // [2]
  // bars 11..13 unused
  uint64_t* v_full = bars + 14;    // [2] V tile landed
  uint64_t* v_empty = bars + 16;   // [2] V slot free again (its P.V GEMM retired)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const int q_tile = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h_idx = blockIdx.y, b = blockIdx.z;
  const int hkv = h_idx / (p.H / p.Hkv);
  const int q0 = q_tile * C::BM;
  const int off = p.Sk - p.Sq;
  int n_tiles = (p.Sk + C::BN - 1) / C::BN;
  if (p.causal) {
    const int last_kv = min(p.Sk - 1, q0 + C::BM - 1 + off);
    n_tiles = last_kv < 0 ? 0 : last_kv / C::BN + 1;
  }

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tq);
    prefetch_tensormap(&tk);
    prefetch_tensormap(&tv);
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
      mbar_init(smem_u32(&s_full[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&p_ready[s]), 128);     // the 128 threads of the warpgroup that owns the tile
      mbar_init(smem_u32(&pv_done[s]), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp_idx == 9) {
    tmem_alloc(smem_u32(tmem_ptr_smem), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp_idx == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && n_tiles > 0) {
      mbar_arrive_expect_tx(smem_u32(q_full), C::Q_BYTES);
#pragma unroll
      for (int s = 0; s < C::SUB; ++s)
        tma_load_4d(smem_u32(sQ + s * C::TILE_BYTES), &tq, smem_u32(q_full), s * 64, q0, h_idx, b);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        // K and V travel on separate barriers: a K slot is free as soon as the S GEMM that read it
        // has retired, one P.V earlier than the V slot, which lets K(j) arrive before S(j) is due
        ok = mbar_wait(smem_u32(&kv_empty[st]), ph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        const uint32_t kbar = smem_u32(&kv_full[st]);
        mbar_arrive_expect_tx(kbar, C::KV_BYTES);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
          tma_load_4d(smem_u32(sK + st * C::KV_BYTES + s * C::TILE_BYTES), &tk, kbar, s * 64,
                      j * C::BN, hkv, b);
        ok = mbar_wait(smem_u32(&v_empty[st]), ph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        const uint32_t vbar = smem_u32(&v_full[st]);
        mbar_arrive_expect_tx(vbar, C::KV_BYTES);
#pragma unroll
        for (int s = 0; s < C::SUB; ++s)
          tma_load_4d(smem_u32(sV + st * C::KV_BYTES + s * C::TILE_BYTES), &tv, vbar, s * 64,
                      j * C::BN, hkv, b);
      }
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
    }
  } else if (warp_idx == 9) {
    // ------------------------------ MMA issuer --------------------------------
    if (n_tiles > 0) {   // whole warp; one elected lane issues each instruction
      constexpr uint32_t idesc_s = make_idesc(UmmaFormat<T>::value, 0, 0, 128, 128);
      constexpr uint32_t idesc_o = make_idesc(UmmaFormat<T>::value, 0, 1, 128, HD);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t q_base = smem_u32(sQ);
        const uint32_t k_base = smem_u32(sK + st * C::KV_BYTES);
        const uint32_t d = tmem_base + C::S_COL0 + (j & 1) * 128;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t o = (k >> 2) * C::TILE_BYTES + (k & 3) * 32;
          umma_f16_w(d, make_smem_desc_sw128(q_base + o, 16, 1024),
                   make_smem_desc_sw128(k_base + o, 16, 1024), idesc_s, k != 0);
        }
        umma_commit_w(smem_u32(&s_full[j & 1]));
        umma_commit_w(smem_u32(&kv_empty[st]));
      };
      if (ok) {
        ok = mbar_wait(smem_u32(&kv_full[0]), 0, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          ok = mbar_wait(smem_u32(&kv_full[(j + 1) & 1]), ((j + 1) >> 1) & 1, abort_flag, p.status,
                         RB_ERR_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = mbar_wait(smem_u32(&p_ready[j & 1]), (j >> 1) & 1, abort_flag, p.status,
                       RB_ERR_TIMEOUT_FLAG);
        if (!ok) break;
        const int st = j & 1;
        ok = mbar_wait(smem_u32(&v_full[st]), (j >> 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t p_base = smem_u32(sP + (j & 1) * C::P_BYTES);
        const uint32_t v_base = smem_u32(sV + st * C::KV_BYTES);
        const uint32_t d = tmem_base + C::O_COL + (j & 1) * 128;   // even / odd tiles accumulate apart
#pragma unroll
        for (int k = 0; k < C::BN / 16; ++k) {
          const uint32_t po = (k >> 2) * C::TILE_BYTES + (k & 3) * 32;
          umma_f16_w(d, make_smem_desc_sw128(p_base + po, 16, 1024),
                   make_smem_desc_sw128(v_base + k * 2048, C::TILE_BYTES, 1024), idesc_o,
                   (j >= 2 || k != 0) ? 1u : 0u);
        }
        umma_commit_w(smem_u32(&v_empty[st]));
        umma_commit_w(smem_u32(&pv_done[j & 1]));
      }
    }
  } else if (n_tiles > 0) {
    // ------------------------------ softmax warps -----------------------------
    const int wg = warp_idx >> 2;                 // 0: even K/V tiles, 1: odd K/V tiles
    const int t = (warp_idx & 3) * 32 + lane;     // row within the tile == TMEM lane
    const int row = q0 + t;                       // global query row
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp_idx & 3) * 32) << 16);
    const uint32_t o_mine = lane_addr + C::O_COL + wg * 128;     // this warpgroup's O accumulator
    float m_used = -INFINITY, l = 0.f;            // running maximum (log2 domain) and sum of this warpgroup's tiles
    bool ok = true;
    for (int j = wg; j < n_tiles; j += 2) {
      const uint32_t jph = (j >> 1) & 1;
      ok = mbar_wait(smem_u32(&s_full[wg]), jph, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + C::S_COL0 + wg * 128;
      const int kv0 = j * C::BN;
      const bool need_mask = (kv0 + C::BN > p.Sk) || (p.causal && kv0 + C::BN - 1 > q0 + off);
      const int kv_limit = p.causal ? min(p.Sk - 1, row + off) : p.Sk - 1;  // last valid kv index
      // pass 1: row maximum over the 128 columns, 64 at a time
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t sreg[2][32];
        tmem_ld_32x32b_x32(s_addr + hh * 64, sreg[0]);
        tmem_ld_32x32b_x32(s_addr + hh * 64 + 32, sreg[1]);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kv0 + hh * 64 + c * 32 + i <= kv_limit)
                mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sreg[c][i]));
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sreg[c][i]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      const bool need = m_new > m_used + 8.0f;  // also true on this warpgroup's first tile (m_used = -inf)
      if (j >= 2) {
        // the previous tile of this warpgroup (j - 2) used the same P buffer and the same O accumulator:
        // its P.V must have retired before P is overwritten or O is rescaled
        ok = mbar_wait(smem_u32(&pv_done[wg]), ((j - 2) >> 1) & 1, abort_flag, p.status,
                       RB_ERR_TIMEOUT_TMEM_EMPTY);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, need)) {       // the TMEM accesses below are warp-wide: uniform branch
        float alpha = 1.0f;
        if (need) {
          alpha = (m_used == -INFINITY) ? 0.0f : fast_exp2(m_used - m_new);
          m_used = m_new;
          l *= alpha;
        }
        if (j >= 2) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(o_mine + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(o_mine + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // pass 2: P = exp2(S*scale - m), row sum, store to this warpgroup's swizzled P tile
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* prow = sP + wg * C::P_BYTES + t * 128;
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t sreg[2][32];
        tmem_ld_32x32b_x32(s_addr + hh * 64, sreg[0]);
        tmem_ld_32x32b_x32(s_addr + hh * 64 + 32, sreg[1]);
        tmem_ld_wait();
        uint8_t* rowp = prow + hh * C::TILE_BYTES;       // sub-tile hh holds key columns [64 hh, 64 hh + 64)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(sreg[c][i]), p.scale_log2, neg_m));
            float p1 = fast_exp2(fmaf(__uint_as_float(sreg[c][i + 1]), p.scale_log2, neg_m));
            if (need_mask) {
              if (kv0 + hh * 64 + c * 32 + i > kv_limit) p0 = 0.f;
              if (kv0 + hh * 64 + c * 32 + i + 1 > kv_limit) p1 = 0.f;
            }
            l4[(i >> 1) & 3] += p0 + p1;
            packed[i >> 1] = pack2<T>(p0, p1);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int cc = c * 4 + q;
            *reinterpret_cast<uint4*>(rowp + ((cc ^ (t & 7)) << 4)) =
                make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
          }
        }
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_ready[wg]));
    }
    // ---- merge the two warpgroups' partial results and write the output ----
    // every P.V of both accumulators must have retired
    const int last0 = ((n_tiles - 1) & 1) == 0 ? n_tiles - 1 : n_tiles - 2;   // last even tile (always exists)
    const int last1 = ((n_tiles - 1) & 1) == 1 ? n_tiles - 1 : n_tiles - 2;   // last odd tile, or -1
    if (ok) {
      ok = mbar_wait(smem_u32(&pv_done[0]), (last0 >> 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_EMPTY);
      if (ok && last1 >= 0)
        ok = mbar_wait(smem_u32(&pv_done[1]), (last1 >> 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_EMPTY);
    }
    // (m, l) of the two warpgroups meet in shared memory (the Q tile is no longer needed: reuse it)
    float2* fin = reinterpret_cast<float2*>(sQ);            // [2][128]
    fin[wg * 128 + t] = make_float2(m_used, l);
    asm volatile("bar.sync 1, 256;" ::: "memory");          // the 8 softmax warps; reached on every path
    if (ok) {
      tc_fence_after();
      const float2 other = fin[(wg ^ 1) * 128 + t];
      const float m_all = fmaxf(m_used, other.x);
      const float f_me = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_all);
      const float f_ot = (other.x == -INFINITY) ? 0.f : fast_exp2(other.x - m_all);
      const float l_all = l * f_me + other.y * f_ot;
      const float inv_l = l_all > 0.f ? 1.0f / l_all : 0.f;
      const float w_even = (wg == 0 ? f_me : f_ot) * inv_l, w_odd = (wg == 0 ? f_ot : f_me) * inv_l;
      const bool has_odd = last1 >= 0;
      // warpgroup w writes output columns [w * HD/2, (w+1) * HD/2)
      T* orow = reinterpret_cast<T*>(p.o) + ((static_cast<long long>(b) * p.Sq + row) * p.H + h_idx) * HD +
                wg * (HD / 2);
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t re[32], ro[32];
        tmem_ld_32x32b_x32(lane_addr + C::O_COL + wg * (HD / 2) + c * 32, re);
        if (has_odd) tmem_ld_32x32b_x32(lane_addr + C::O_COL + 128 + wg * (HD / 2) + c * 32, ro);
        tmem_ld_wait();
        if (row < p.Sq) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            T* e = reinterpret_cast<T*>(&v);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float val = __uint_as_float(re[q * 8 + i]) * w_even;
              if (has_odd) val += __uint_as_float(ro[q * 8 + i]) * w_odd;
              e[i] = from_f32<T>(val);
            }
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = v;
          }
        }
      }
      if (wg == 0 && row < p.Sq)
        p.lse[(static_cast<long long>(b) * p.H + h_idx) * p.Sq + row] =
            (m_all + log2f(l_all)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp_idx == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <typename T, int HD>
int launch_fa_fwd(int dtype, const void* q, const void* k, const void* v, const long long* qs,
                  const long long* ks, const long long* vs, const FaFwdParams& p, cudaStream_t st) {
  using C = FaFwdCfg<HD>;
  CUtensorMap tq, tk, tv;
  auto mk = [&](CUtensorMap* m, const void* base, const long long* s, int S, int heads) {
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)S, (uint64_t)heads, (uint64_t)p.B};
    uint64_t strides[4] = {2, (uint64_t)s[1] * 2, (uint64_t)s[2] * 2, (uint64_t)s[0] * 2};
    uint32_t box[4] = {64, 128, 1, 1};
    return rbh::encode_tensor_map(m, dtype, 4, const_cast<void*>(base), dims, strides, box, 1);
  };
  int rc = mk(&tq, q, qs, p.Sq, p.H);
  if (!rc) rc = mk(&tk, k, ks, p.Sk, p.Hkv);
  if (!rc) rc = mk(&tv, v, vs, p.Sk, p.Hkv);
  if (rc) return 1000 + rc;
  auto kern = fa_fwd_kernel<T, HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return 2000 + (int)e;
  dim3 grid((p.Sq + C::BM - 1) / C::BM, p.H, p.B);
  kern<<<grid, 320, C::SMEM_BYTES, st>>>(tq, tk, tv, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {
// q/k/v strides are {batch, seq, head} in elements (innermost dim contiguous).
// o is [B,Sq,H,D] contiguous, lse is [B,H,Sq] fp32.
int rb_flash_attn_fwd(int dtype, int head_dim, const void* q, const void* k, const void* v,
                      const long long* q_strides, const long long* k_strides,
                      const long long* v_strides, void* o, float* lse, int B, int H, int Hkv,
                      int Sq, int Sk, int causal, float scale, void* stream) {
  using namespace rb;
  if (B <= 0 || H <= 0 || Sq <= 0) return 0;
  FaFwdParams p;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk; p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.o = o; p.lse = lse;
  p.status = rbh::device_status_word();
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == rbh::DT_BF16) {
    if (head_dim == 128) return launch_fa_fwd<__nv_bfloat16, 128>(dtype, q, k, v, q_strides, k_strides, v_strides, p, st);
    if (head_dim == 64) return launch_fa_fwd<__nv_bfloat16, 64>(dtype, q, k, v, q_strides, k_strides, v_strides, p, st);
  } else if (dtype == rbh::DT_F16) {
    if (head_dim == 128) return launch_fa_fwd<__half, 128>(dtype, q, k, v, q_strides, k_strides, v_strides, p, st);
    if (head_dim == 64) return launch_fa_fwd<__half, 64>(dtype, q, k, v, q_strides, k_strides, v_strides, p, st);
  }
  return 20;  // unsupported dtype / head_dim
}
}
