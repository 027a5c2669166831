// W4A16 GEMM for decode batches (1..128 tokens): Y[M,N] = X[M,K] . dequant(W4)[K,N] (+ bias)
//
// The weight stays packed all the way into shared memory; it is expanded to 16-bit there, inside
// the kernel that multiplies it, so HBM only ever sees 4 bits per weight:
//
//   packed words  --TMA (8 x 128 words, no swizzle)-->  raw ring (8 stages x 4 KB)
//   dequant warps: word -> 8 x 16-bit ((q - zp) * scale) -> one 16-byte store into the
//                  K-major, 128-byte-swizzled UMMA operand tile (128 weight columns x 64 k)
//   activations   --TMA (64 k x Mpad tokens, 128B swizzle)--> X ring
//   tcgen05.mma   D^T[128 weight columns, Mpad tokens] += Wt[128, 64] . Xt[64, Mpad]
//                 (operands swapped: the weight tile is the 128-row A operand, the token batch is
//                  the N dimension of the instruction, so a batch of 16 costs 16/128 of a full tile)
//   epilogue      TMEM lane = weight column, TMEM column = token; adds bias and stores, or adds
//                 into an fp32 workspace when K is split across CTAs.
//
// Packed layout (unchanged from the reference's quantizer, rumus-vision/src/quant.rs:42-126, and its
// kernel rumus-vision/src/shaders/qmatmul_int4.wgsl:41): word (k/8)*N + n holds k..k+7 of column n,
// nibble k%8; scales / zero points are [K/group, N].
//
// Roles (224 threads): warp 0 TMA of packed words, warp 1 MMA issuer + TMEM owner, warps 2..5
// dequantise (thread = weight column) and later run the epilogue, warp 6 TMA of activations.
// Every wait is bounded (mbar_wait): on expiry the status word is set and the CTA drains.
#include "sm100_common.cuh"

namespace rb {

constexpr int W4_BN = 128;         // weight columns per CTA = UMMA M
constexpr int W4_BK = 64;          // k per pipeline stage (one 128-byte swizzle row of 16-bit values)
constexpr int W4_RAW_STAGES = 8;   // 8 k-rows x 128 words x 4 B = 4 KB each
constexpr int W4_AB_STAGES = 3;
constexpr int W4_RAW_BYTES = 8 * W4_BN * 4;
constexpr int W4_A_BYTES = W4_BN * 128;
constexpr int W4_THREADS = 224;

struct W4Params {
  int M, N, K, Kp, group;
  int m_pad;                 // tokens rounded up to 16 (UMMA N)
  int kb_per_slice;          // k blocks of 64 per K slice
  const void* scales;
  const void* zps;
  const void* bias;          // [N] of T or null (applied only when the K range is not split)
  void* out;                 // [M,N] of T (unsplit)
  float* ws;                 // [M,N] fp32, zero-initialised (split K)
  int* tile_counters;        // split K: one int per column tile (zero before the launch), or null.
                             // With counters the CTA that adds the last K slice of a tile also converts
                             // it (ws + bias -> out) and puts ws and the counter back to zero, so neither
                             // a clearing pass before nor a conversion kernel after the launch is needed.
  int* status;
};

// The nibble is OR-ed onto an exponent on which integers are exact, and the subtraction that removes
// the exponent's value also centres the code: q - 8 in [-8, 7].  The value is then
// (q - 8) * scale + (8 - zp) * scale; centring halves the magnitude of the additive term, whose
// rounding to 16 bits is the largest error of this path (0.27 % of the product's norm in bf16
// against 0.70 % uncentred, measured on random weights; fp32 math rounded once gives 0.17 %).
template <typename T> struct W4Magic;
// bf16: 0x4300 | q  ==  128 + q exactly (8 significant bits cover 128..143)
template <> struct W4Magic<__nv_bfloat16> { static constexpr uint32_t bits = 0x43004300u; static constexpr float base = 136.f; };
// fp16: 0x6400 | q  ==  1024 + q exactly
template <> struct W4Magic<__half> { static constexpr uint32_t bits = 0x64006400u; static constexpr float base = 1032.f; };

template <typename T> struct Vec2;
template <> struct Vec2<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Vec2<__half> { using type = __half2; };

template <typename T>
__device__ __forceinline__ typename Vec2<T>::type splat2(float v);
template <> __device__ __forceinline__ __nv_bfloat162 splat2<__nv_bfloat16>(float v) { return __float2bfloat162_rn(v); }
template <> __device__ __forceinline__ __half2 splat2<__half>(float v) { return __float2half2_rn(v); }

template <typename TS> __device__ __forceinline__ float w4_sc(TS v);
template <> __device__ __forceinline__ float w4_sc<float>(float v) { return v; }
template <> __device__ __forceinline__ float w4_sc<__half>(__half v) { return __half2float(v); }

// One packed word (8 nibbles of consecutive k) -> 8 values of T in k order, as one 16-byte vector.
template <typename T>
__device__ __forceinline__ uint4 w4_expand(uint32_t w, typename Vec2<T>::type base2,
                                           typename Vec2<T>::type s2, typename Vec2<T>::type b2) {
  using V = typename Vec2<T>::type;
  uint32_t v[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    // nibbles p (low half) and p + 4 (high half), each placed on the magic exponent
    uint32_t u = ((w >> (4 * p)) & 0x000F000Fu) | W4Magic<T>::bits;
    V q = __hsub2(*reinterpret_cast<V*>(&u), base2);       // exact: q - 8 in -8..7
    V r = __hfma2(q, s2, b2);                              // (q - 8) * scale + (8 - zp) * scale
    v[p] = *reinterpret_cast<uint32_t*>(&r);
  }
  uint4 o;
  o.x = __byte_perm(v[0], v[1], 0x5410);   // k0 k1
  o.y = __byte_perm(v[2], v[3], 0x5410);   // k2 k3
  o.z = __byte_perm(v[0], v[1], 0x7632);   // k4 k5
  o.w = __byte_perm(v[2], v[3], 0x7632);   // k6 k7
  return o;
}

template <typename T, typename TS>
__global__ void __launch_bounds__(W4_THREADS, 1)
    w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                      const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int x_bytes = p.m_pad * 128;
  uint8_t* sA = smem;                                       // [AB_STAGES][128 x 128 B]
  uint8_t* sX = sA + W4_AB_STAGES * W4_A_BYTES;             // [AB_STAGES][m_pad x 128 B]
  uint8_t* sRaw = sX + W4_AB_STAGES * x_bytes;              // [RAW_STAGES][8 x 128 words]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + W4_RAW_STAGES * W4_RAW_BYTES);
  uint64_t* raw_full = bars;                                // TMA -> dequant
  uint64_t* raw_empty = raw_full + W4_RAW_STAGES;           // dequant (4 warps) -> TMA
  uint64_t* a_full = raw_empty + W4_RAW_STAGES;             // dequant (4 warps) -> MMA
  uint64_t* x_full = a_full + W4_AB_STAGES;                 // TMA -> MMA
  uint64_t* ab_empty = x_full + W4_AB_STAGES;               // MMA commit -> dequant, X producer
  uint64_t* acc_full = ab_empty + W4_AB_STAGES;             // MMA commit -> epilogue
  uint64_t* fin_bar = acc_full + 1;                         // epilogue warps: "my additions are out" (4 arrivals)
  uint64_t* fin2_bar = fin_bar + 1;                         // one thread: "last_flag is written"
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(fin2_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const int tmem_cols = p.m_pad <= 32 ? 32 : (p.m_pad <= 64 ? 64 : 128);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tma_w);
    prefetch_tensormap(&tma_x);
    for (int s = 0; s < W4_RAW_STAGES; ++s) {
      mbar_init(smem_u32(&raw_full[s]), 1);
      mbar_init(smem_u32(&raw_empty[s]), 4);
    }
    for (int s = 0; s < W4_AB_STAGES; ++s) {
      mbar_init(smem_u32(&a_full[s]), 4);
      mbar_init(smem_u32(&x_full[s]), 1);
      mbar_init(smem_u32(&ab_empty[s]), 1);
    }
    mbar_init(smem_u32(acc_full), 1);
    mbar_init(smem_u32(fin_bar), 4);
    mbar_init(smem_u32(fin2_bar), 1);
    *abort_flag = 0;
    *last_flag = 0;
    fence_barrier_init();
  }
  if (warp_idx == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const int n0 = blockIdx.x * W4_BN;
  const int num_kb = p.Kp / W4_BK;
  const int kb0 = blockIdx.y * p.kb_per_slice;
  const int kb1 = min(num_kb, kb0 + p.kb_per_slice);
  const int nkb = kb1 - kb0;     // > 0 by construction of the grid

  if (warp_idx == 0) {
    // ------------------------------ packed-weight TMA ------------------------------
    if (lane == 0) {
      bool ok = true;
      int r = 0;
      uint32_t ph = 0;
      for (int i = 0; i < nkb && ok; ++i) {
        ok = mbar_wait(smem_u32(&raw_empty[r]), ph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        const uint32_t bar = smem_u32(&raw_full[r]);
        mbar_arrive_expect_tx(bar, W4_RAW_BYTES);
        tma_load_2d(smem_u32(sRaw + r * W4_RAW_BYTES), &tma_w, bar, n0, (kb0 + i) * 8);
        if (++r == W4_RAW_STAGES) { r = 0; ph ^= 1; }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land
    }
  } else if (warp_idx == 6) {
    // ------------------------------ activation TMA ---------------------------------
    if (lane == 0) {
      bool ok = true;
      int s = 0;
      uint32_t ph = 0;
      for (int i = 0; i < nkb && ok; ++i) {
        ok = mbar_wait(smem_u32(&ab_empty[s]), ph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
        if (!ok) break;
        const uint32_t bar = smem_u32(&x_full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)x_bytes);
        tma_load_2d(smem_u32(sX + s * x_bytes), &tma_x, bar, (kb0 + i) * W4_BK, 0);
        if (++s == W4_AB_STAGES) { s = 0; ph ^= 1; }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);
    }
  } else if (warp_idx == 1) {
    // ------------------------------ MMA issuer -------------------------------------
    const uint32_t idesc = make_idesc(UmmaFormat<T>::value, 0, 0, W4_BN, p.m_pad);
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < nkb && ok; ++i) {
      ok = mbar_wait(smem_u32(&a_full[s]), ph, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(smem_u32(&x_full[s]), ph, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_base = smem_u32(sA + s * W4_A_BYTES);
      const uint32_t x_base = smem_u32(sX + s * x_bytes);
#pragma unroll
      for (int k = 0; k < W4_BK / 16; ++k) {
        const uint64_t adesc = make_smem_desc_sw128(a_base + k * 32, 16, 1024);
        const uint64_t bdesc = make_smem_desc_sw128(x_base + k * 32, 16, 1024);
        umma_f16_w(tmem_base, adesc, bdesc, idesc, (i | k) != 0 ? 1u : 0u);
      }
      umma_commit_w(smem_u32(&ab_empty[s]));
      if (++s == W4_AB_STAGES) { s = 0; ph ^= 1; }
    }
    if (ok) umma_commit_w(smem_u32(acc_full));
  } else {
    // ------------------------------ dequantise, then epilogue ----------------------
    using V = typename Vec2<T>::type;
    const int quarter = warp_idx & 3;               // TMEM lane quarter this warp may read
    const int nl = quarter * 32 + lane;             // weight column within the tile
    const int n = n0 + nl;
    const bool n_ok = n < p.N;
    const TS* scales = static_cast<const TS*>(p.scales);
    const TS* zps = static_cast<const TS*>(p.zps);
    const V base2 = splat2<T>(W4Magic<T>::base);
    const int kb_per_group = p.group / W4_BK;
    uint8_t* a_row = nullptr;
    bool ok = true;
    int r = 0, s = 0;
    uint32_t rph = 0, sph = 0;
    int g_cur = -1;
    V s2 = splat2<T>(0.f), b2 = splat2<T>(0.f);
    // scale / zero point of the next group are fetched one group ahead
    int g_next = (kb0 * W4_BK) / p.group;
    float sc_n = n_ok ? w4_sc<TS>(scales[(long long)g_next * p.N + n]) : 0.f;
    float zp_n = n_ok ? w4_sc<TS>(zps[(long long)g_next * p.N + n]) : 0.f;
    const int num_groups = p.Kp / p.group;
    for (int i = 0; i < nkb && ok; ++i) {
      const int kb = kb0 + i;
      const int g = kb / kb_per_group;
      if (g != g_cur) {
        g_cur = g;
        s2 = splat2<T>(sc_n);
        b2 = splat2<T>((8.f - zp_n) * sc_n);
        g_next = g + 1;
        if (g_next < num_groups && n_ok) {
          sc_n = w4_sc<TS>(scales[(long long)g_next * p.N + n]);
          zp_n = w4_sc<TS>(zps[(long long)g_next * p.N + n]);
        }
      }
      ok = mbar_wait(smem_u32(&raw_full[r]), rph, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t* raw = reinterpret_cast<const uint32_t*>(sRaw + r * W4_RAW_BYTES);
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = raw[j * W4_BN + nl];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&raw_empty[r]));
      if (++r == W4_RAW_STAGES) { r = 0; rph ^= 1; }

      ok = mbar_wait(smem_u32(&ab_empty[s]), sph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // row nl of the K-major tile: 8-row groups of 1024 B, 16-byte chunk c stored at c ^ (row % 8)
      a_row = sA + s * W4_A_BYTES + (nl >> 3) * 1024 + (nl & 7) * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 v = w4_expand<T>(w[j], base2, s2, b2);
        *reinterpret_cast<uint4*>(a_row + ((j ^ (nl & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();     // generic-proxy stores -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&a_full[s]));
      if (++s == W4_AB_STAGES) { s = 0; sph ^= 1; }
    }
    // ---- epilogue ----
    if (ok) {
      ok = mbar_wait(smem_u32(acc_full), 0, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool split = gridDim.y > 1;
      const float bias = (!split && p.bias && n_ok) ? to_f32<T>(static_cast<const T*>(p.bias)[n]) : 0.f;
      for (int c = 0; c < p.m_pad / 16; ++c) {
        uint32_t acc[16];
        tmem_ld_32x32b_x16(taddr + c * 16, acc);
        tmem_ld_wait();
        if (n_ok) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const int m = c * 16 + t;
            if (m < p.M) {
              const float v = __uint_as_float(acc[t]);
              if (split)
                atomicAdd(p.ws + (long long)m * p.N + n, v);
              else
                static_cast<T*>(p.out)[(long long)m * p.N + n] = from_f32<T>(v + bias);
            }
          }
        }
      }
      if (split && p.tile_counters) {
        // the K slice that arrives last at this column tile finishes it
        // (bounded mbarrier waits rather than a named barrier: a warp that gave up must not leave
        // the other three waiting for ever)
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(fin_bar));
        if (nl == 0) {
          if (mbar_wait(smem_u32(fin_bar), 0, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL))
            *last_flag = atomicAdd(p.tile_counters + blockIdx.x, 1) == (int)gridDim.y - 1 ? 1 : 0;
          mbar_arrive(smem_u32(fin2_bar));
        }
        bool fin_ok = mbar_wait(smem_u32(fin2_bar), 0, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
        fin_ok = __all_sync(0xffffffffu, fin_ok);
        if (fin_ok && *last_flag) {
          __threadfence();
          if (n_ok) {
            const float bs = p.bias ? to_f32<T>(static_cast<const T*>(p.bias)[n]) : 0.f;
            for (int m = 0; m < p.M; ++m) {
              float* w = p.ws + (long long)m * p.N + n;
              const float v = __ldcg(w);
              *w = 0.f;                                          // ready for the next launch
              static_cast<T*>(p.out)[(long long)m * p.N + n] = from_f32<T>(v + bs);
            }
          }
          if (nl == 0) p.tile_counters[blockIdx.x] = 0;
        }
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp_idx == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// y = T(ws + bias) after a split-K run
template <typename T>
__global__ void w4a16_finalize_kernel(const float* __restrict__ ws, const T* __restrict__ bias, T* __restrict__ y,
                                      long long total, int N) {
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    float v = ws[i];
    if (bias) v += to_f32<T>(bias[i % N]);
    y[i] = from_f32<T>(v);
  }
}

template <typename T, typename TS>
int launch_w4a16(int x_dtype, const void* x, long long ldx, const int* packed, W4Params p, int k_slices,
                 cudaStream_t st) {
  CUtensorMap tw, tx;
  {
    // packed words as a 2-D array of 32-bit elements [Kp/8 rows, N columns]
    uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)(p.Kp / 8)};
    uint64_t strides[2] = {4, (uint64_t)p.N * 4};
    uint32_t box[2] = {W4_BN, 8};
    const int rc = rbh::encode_tensor_map(&tw, rbh::DT_F32, 2, const_cast<int*>(packed), dims, strides, box, 0);
    if (rc) return 1000 + rc;
  }
  {
    // activations [M rows, K columns]; rows past M and columns past K read as zero
    uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.M};
    uint64_t strides[2] = {sizeof(T), (uint64_t)ldx * sizeof(T)};
    uint32_t box[2] = {W4_BK, (uint32_t)p.m_pad};
    const int rc = rbh::encode_tensor_map(&tx, x_dtype, 2, const_cast<void*>(x), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  const int smem = W4_AB_STAGES * (W4_A_BYTES + p.m_pad * 128) + W4_RAW_STAGES * W4_RAW_BYTES + 1024 + 256;
  auto kern = w4a16_gemm_kernel<T, TS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return 2000 + (int)e;
  dim3 grid((p.N + W4_BN - 1) / W4_BN, k_slices);
  kern<<<grid, W4_THREADS, smem, st>>>(tw, tx, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {

// Number of K slices the launcher would pick for this shape (the caller sizes the fp32 workspace
// [M, N] only when this is > 1).
int rb_w4a16_slices(int N, int Kp) {
  const int n_tiles = (N + rb::W4_BN - 1) / rb::W4_BN;
  const int num_kb = Kp / rb::W4_BK;
  int want = (2 * rbh::sm_count() + n_tiles - 1) / n_tiles;     // about two CTAs' worth of work per SM
  int max_slices = num_kb / 4;                                   // at least 256 k per slice
  if (max_slices < 1) max_slices = 1;
  if (want > max_slices) want = max_slices;
  if (want < 1) want = 1;
  // no empty slice: recompute from the per-slice length
  const int per = (num_kb + want - 1) / want;
  return (num_kb + per - 1) / per;
}

// Y[M,N] = X[M,K] . dequant(packed)[K,N] + bias.  Error 51 = shape / alignment outside what this
// kernel covers (the caller uses another path).  `ws` is only touched when the K range is split:
// with `tile_counters` (one zeroed int per 128 columns) it must be zero on entry and is zero again
// on return — one launch in total; without counters it is cleared here and converted by a second
// kernel.
int rb_w4a16_gemm(int x_dtype, int scale_dtype, const void* x, long long ldx, const int* packed,
                  const void* scales, const void* zps, const void* bias, void* y, float* ws,
                  int* tile_counters, int M, int N, int K, int Kp, int group, void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || (x_dtype != rbh::DT_BF16 && x_dtype != rbh::DT_F16)) return 51;
  if (Kp % W4_BK || group % W4_BK || Kp % group || N % 4 || K > Kp || K <= 0) return 51;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed)) & 15) return 51;
  if ((ldx * 2) % 16) return 51;
  cudaStream_t st = (cudaStream_t)stream;
  W4Params p;
  p.M = M; p.N = N; p.K = K; p.Kp = Kp; p.group = group;
  p.m_pad = (M + 15) / 16 * 16;
  const int k_slices = rb_w4a16_slices(N, Kp);
  p.kb_per_slice = (Kp / W4_BK + k_slices - 1) / k_slices;
  p.scales = scales; p.zps = zps; p.bias = bias; p.out = y; p.ws = ws;
  p.tile_counters = k_slices > 1 ? tile_counters : nullptr;
  p.status = rbh::device_status_word();
  if (k_slices > 1) {
    if (!ws) return 52;
    if (!tile_counters) cudaMemsetAsync(ws, 0, (size_t)M * N * sizeof(float), st);
  }
  int rc;
  if (x_dtype == rbh::DT_BF16)
    rc = scale_dtype == rbh::DT_F16 ? launch_w4a16<__nv_bfloat16, __half>(x_dtype, x, ldx, packed, p, k_slices, st)
                                    : launch_w4a16<__nv_bfloat16, float>(x_dtype, x, ldx, packed, p, k_slices, st);
  else
    rc = scale_dtype == rbh::DT_F16 ? launch_w4a16<__half, __half>(x_dtype, x, ldx, packed, p, k_slices, st)
                                    : launch_w4a16<__half, float>(x_dtype, x, ldx, packed, p, k_slices, st);
  if (rc) return rc;
  if (k_slices > 1 && !tile_counters) {
    const long long total = (long long)M * N;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)rbh::sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (x_dtype == rbh::DT_BF16)
      w4a16_finalize_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(ws, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, total, N);
    else
      w4a16_finalize_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(ws, (const __half*)bias, (__half*)y, total, N);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return 3000 + (int)e;
  }
  return 0;
}
}
