// W8A16 GEMM for batches of 1..128 rows: Y[M,N] = X[M,K] . dequant(Q8)[K,N] (+ bias)
//
// The INT8 block-quantised weight is expanded to 16-bit inside the kernel that multiplies it, in
// shared memory, so HBM only ever sees the quantised bytes (1.125 bytes per weight at block size 32):
//
//   dequant warps (thread = weight column): the column's K run is contiguous in the reference's
//                  layout, so a 64-wide K block of one column is a few words of block headers and
//                  int8 payload; they are fetched one K block ahead with plain 4-byte loads, turned
//                  into 16-bit values (q * scale) and stored as one 128-byte row of the K-major,
//                  128-byte-swizzled UMMA operand tile (128 weight columns x 64 k)
//   activations    --TMA (64 k x Mpad rows, 128B swizzle)--> X ring
//   tcgen05.mma    D^T[128 weight columns, Mpad rows] += Wt[128, 64] . Xt[64, Mpad]
//                  (operands swapped: the weight tile is the 128-row A operand, the batch is the N
//                   dimension of the instruction)
//   epilogue       TMEM lane = weight column, TMEM column = batch row; adds bias and stores, or adds
//                  into an fp32 workspace when K is split across CTAs (the CTA that adds a tile's
//                  last K slice converts it and puts workspace and counter back to zero).
//
// Quantised layout (unchanged from the reference: rumus/src/tensor/ops.rs:2290,
// rumus/src/backend/gpu/shaders/quantize.wgsl:30; its fused product is
// rumus/src/backend/gpu/shaders/matmul_q8.wgsl:38): the matrix is flattened column-major (element
// (k, n) at n*K + k) and cut into blocks of `bs` values; a block is a 4-byte header (f16 scale in the
// low 16 bits) followed by `bs` int8 values.
//
// Roles (192 threads): warp 0 TMA of activations, warp 1 MMA issuer + TMEM owner, warps 2..5
// dequantise and later run the epilogue.  Every wait is bounded (mbar_wait).
#include "sm100_common.cuh"

namespace rb {

constexpr int W8_BN = 128;         // weight columns per CTA = UMMA M
constexpr int W8_BK = 64;          // k per pipeline stage (one 128-byte swizzle row of 16-bit values)
constexpr int W8_STAGES = 4;
constexpr int W8_A_BYTES = W8_BN * 128;
constexpr int W8_THREADS = 192;

struct W8Params {
  int M, N, K, bs;
  int m_pad;                 // rows rounded up to 16 (UMMA N)
  int kb_per_slice;          // k blocks of 64 per K slice
  const unsigned char* q;    // quantised blocks
  const void* bias;          // [N] of T or null
  void* out;                 // [M,N] of T
  float* ws;                 // [M,N] fp32, zero on entry (split K)
  int* tile_counters;        // one int per column tile, zero on entry (split K)
  int* status;
};

// eight consecutive int8 (two words, k order) times `scale` -> eight values of T as one 16-byte vector
template <typename T>
__device__ __forceinline__ uint4 w8_expand(uint32_t lo, uint32_t hi, float scale) {
  // byte b of a word, biased by 128, placed on 2^23: exact integer in fp32; removing 2^23 + 128
  // recovers the signed value
  const uint32_t magic = 0x4B000000u;
  const float off = 8388608.f + 128.f;
  lo ^= 0x80808080u;
  hi ^= 0x80808080u;
  float f[8];
  f[0] = __uint_as_float(__byte_perm(lo, magic, 0x7440)) - off;
  f[1] = __uint_as_float(__byte_perm(lo, magic, 0x7441)) - off;
  f[2] = __uint_as_float(__byte_perm(lo, magic, 0x7442)) - off;
  f[3] = __uint_as_float(__byte_perm(lo, magic, 0x7443)) - off;
  f[4] = __uint_as_float(__byte_perm(hi, magic, 0x7440)) - off;
  f[5] = __uint_as_float(__byte_perm(hi, magic, 0x7441)) - off;
  f[6] = __uint_as_float(__byte_perm(hi, magic, 0x7442)) - off;
  f[7] = __uint_as_float(__byte_perm(hi, magic, 0x7443)) - off;
  return make_uint4(pack2<T>(f[0] * scale, f[1] * scale), pack2<T>(f[2] * scale, f[3] * scale),
                    pack2<T>(f[4] * scale, f[5] * scale), pack2<T>(f[6] * scale, f[7] * scale));
}

template <typename T>
__global__ void __launch_bounds__(W8_THREADS, 1)
    w8a16_gemm_kernel(const __grid_constant__ CUtensorMap tma_x, const W8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int x_bytes = p.m_pad * 128;
  uint8_t* sA = smem;                                       // [STAGES][128 x 128 B]
  uint8_t* sX = sA + W8_STAGES * W8_A_BYTES;                // [STAGES][m_pad x 128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sX + W8_STAGES * x_bytes);
  uint64_t* a_full = bars;                                  // dequant (4 warps) -> MMA
  uint64_t* x_full = a_full + W8_STAGES;                    // TMA -> MMA
  uint64_t* ab_empty = x_full + W8_STAGES;                  // MMA commit -> dequant, X producer
  uint64_t* acc_full = ab_empty + W8_STAGES;                // MMA commit -> epilogue
  uint64_t* fin_bar = acc_full + 1;                         // epilogue warps: "my additions are out" (4 arrivals)
  uint64_t* fin2_bar = fin_bar + 1;                         // one thread: "last_flag is written"
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(fin2_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp_idx = uniform_warp_idx();
  const int lane = threadIdx.x & 31;
  const int tmem_cols = p.m_pad <= 32 ? 32 : (p.m_pad <= 64 ? 64 : 128);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tma_x);
    for (int s = 0; s < W8_STAGES; ++s) {
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

  const int n0 = blockIdx.x * W8_BN;
  const int num_kb = (p.K + W8_BK - 1) / W8_BK;
  const int kb0 = blockIdx.y * p.kb_per_slice;
  const int kb1 = min(num_kb, kb0 + p.kb_per_slice);
  const int nkb = kb1 - kb0;     // > 0 by construction of the grid

  if (warp_idx == 0) {
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
        tma_load_2d(smem_u32(sX + s * x_bytes), &tma_x, bar, (kb0 + i) * W8_BK, 0);
        if (++s == W8_STAGES) { s = 0; ph ^= 1; }
      }
      if (!ok) for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land
    }
  } else if (warp_idx == 1) {
    // ------------------------------ MMA issuer -------------------------------------
    const uint32_t idesc = make_idesc(UmmaFormat<T>::value, 0, 0, W8_BN, p.m_pad);
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    for (int i = 0; i < nkb && ok; ++i) {
      ok = mbar_wait(smem_u32(&a_full[s]), ph, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(smem_u32(&x_full[s]), ph, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_base = smem_u32(sA + s * W8_A_BYTES);
      const uint32_t x_base = smem_u32(sX + s * x_bytes);
#pragma unroll
      for (int k = 0; k < W8_BK / 16; ++k) {
        const uint64_t adesc = make_smem_desc_sw128(a_base + k * 32, 16, 1024);
        const uint64_t bdesc = make_smem_desc_sw128(x_base + k * 32, 16, 1024);
        umma_f16_w(tmem_base, adesc, bdesc, idesc, (i | k) != 0 ? 1u : 0u);
      }
      umma_commit_w(smem_u32(&ab_empty[s]));
      if (++s == W8_STAGES) { s = 0; ph ^= 1; }
    }
    if (ok) umma_commit_w(smem_u32(acc_full));
  } else {
    // ------------------------------ dequantise, then epilogue ----------------------
    const int quarter = warp_idx & 3;               // TMEM lane quarter this warp may read
    const int nl = quarter * 32 + lane;             // weight column within the tile
    const int n = n0 + nl;
    const bool n_ok = n < p.N;
    const long long col_e0 = (long long)n * p.K;    // flat index of (0, n)
    const int bstride = p.bs + 4;
    bool ok = true;
    int s = 0;
    uint32_t sph = 0;
    // one K block of this column: eight pieces of 8 values (two payload words + the block header)
    uint32_t lo[8], hi[8], hd[8];
    auto fetch = [&](int kb) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int k = kb * W8_BK + j * 8;
        if (n_ok && k < p.K) {
          const long long e = col_e0 + k;
          const long long blk = e / p.bs;
          const int within = (int)(e - blk * p.bs);
          const unsigned char* b = p.q + blk * bstride;
          hd[j] = __ldg(reinterpret_cast<const uint32_t*>(b));
          const uint32_t* w = reinterpret_cast<const uint32_t*>(b + 4 + within);
          lo[j] = __ldg(w);
          hi[j] = __ldg(w + 1);
        } else {
          hd[j] = 0u; lo[j] = 0u; hi[j] = 0u;
        }
      }
    };
    fetch(kb0);
    for (int i = 0; i < nkb && ok; ++i) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __half sc = __ushort_as_half(static_cast<unsigned short>(hd[j] & 0xffffu));
        v[j] = w8_expand<T>(lo[j], hi[j], __half2float(sc));
      }
      if (i + 1 < nkb) fetch(kb0 + i + 1);          // in flight while this block is stored and multiplied
      ok = mbar_wait(smem_u32(&ab_empty[s]), sph ^ 1, abort_flag, p.status, RB_ERR_TIMEOUT_EMPTY);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      // row nl of the K-major tile: 8-row groups of 1024 B, 16-byte chunk c stored at c ^ (row % 8)
      uint8_t* a_row = sA + s * W8_A_BYTES + (nl >> 3) * 1024 + (nl & 7) * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(a_row + ((j ^ (nl & 7)) << 4)) = v[j];
      fence_proxy_async_smem();     // generic-proxy stores -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&a_full[s]));
      if (++s == W8_STAGES) { s = 0; sph ^= 1; }
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
              const float val = __uint_as_float(acc[t]);
              if (split)
                atomicAdd(p.ws + (long long)m * p.N + n, val);
              else
                static_cast<T*>(p.out)[(long long)m * p.N + n] = from_f32<T>(val + bias);
            }
          }
        }
      }
      if (split) {
        // the K slice that arrives last at this column tile finishes it (bounded mbarrier waits
        // rather than a named barrier: a warp that gave up must not leave the other three waiting)
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
              const float val = __ldcg(w);
              *w = 0.f;                                          // ready for the next launch
              static_cast<T*>(p.out)[(long long)m * p.N + n] = from_f32<T>(val + bs);
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

template <typename T>
int launch_w8a16(int x_dtype, const void* x, long long ldx, W8Params p, int k_slices, cudaStream_t st) {
  CUtensorMap tx;
  {
    // activations [M rows, K columns]; rows past M and columns past K read as zero
    uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.M};
    uint64_t strides[2] = {sizeof(T), (uint64_t)ldx * sizeof(T)};
    uint32_t box[2] = {W8_BK, (uint32_t)p.m_pad};
    const int rc = rbh::encode_tensor_map(&tx, x_dtype, 2, const_cast<void*>(x), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  const int smem = W8_STAGES * (W8_A_BYTES + p.m_pad * 128) + 1024 + 256;
  auto kern = w8a16_gemm_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return 2000 + (int)e;
  dim3 grid((p.N + W8_BN - 1) / W8_BN, k_slices);
  kern<<<grid, W8_THREADS, smem, st>>>(tx, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {

// K slices the launcher picks for this shape (the caller provides the fp32 workspace [M, N] and one
// counter per 128 columns only when this is > 1).
int rb_w8a16_slices(int N, int K) {
  const int n_tiles = (N + rb::W8_BN - 1) / rb::W8_BN;
  const int num_kb = (K + rb::W8_BK - 1) / rb::W8_BK;
  int want = (2 * rbh::sm_count() + n_tiles - 1) / n_tiles;     // about two CTAs' worth of work per SM
  int max_slices = num_kb / 4;                                   // at least 256 k per slice
  if (max_slices < 1) max_slices = 1;
  if (want > max_slices) want = max_slices;
  if (want < 1) want = 1;
  const int per = (num_kb + want - 1) / want;                    // no empty slice
  return (num_kb + per - 1) / per;
}

// Y[M,N] = X[M,K] . dequant(q)[K,N] + bias for M <= 128 rows of 16-bit activations.  Error 53 = shape
// or alignment outside what this kernel covers (the caller dequantises and uses the dense GEMM).
// `ws` / `tile_counters` must be zero on entry and are zero again on return.
int rb_w8a16_gemm(int x_dtype, const void* x, long long ldx, const unsigned char* q, int bs, const void* bias,
                  void* y, float* ws, int* tile_counters, int M, int N, int K, void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || (x_dtype != rbh::DT_BF16 && x_dtype != rbh::DT_F16)) return 53;
  if (K <= 0 || K % 8 || bs <= 0 || bs % 8) return 53;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 3) || (ldx * 2) % 16) return 53;
  W8Params p;
  p.M = M; p.N = N; p.K = K; p.bs = bs;
  p.m_pad = (M + 15) / 16 * 16;
  const int k_slices = rb_w8a16_slices(N, K);
  p.kb_per_slice = ((K + W8_BK - 1) / W8_BK + k_slices - 1) / k_slices;
  p.q = q; p.bias = bias; p.out = y; p.ws = ws; p.tile_counters = tile_counters;
  p.status = rbh::device_status_word();
  if (k_slices > 1 && (!ws || !tile_counters)) return 52;
  cudaStream_t st = (cudaStream_t)stream;
  return x_dtype == rbh::DT_BF16 ? launch_w8a16<__nv_bfloat16>(x_dtype, x, ldx, p, k_slices, st)
                                 : launch_w8a16<__half>(x_dtype, x, ldx, p, k_slices, st);
}
}
