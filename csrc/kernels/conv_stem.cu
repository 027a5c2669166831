// Direct convolution for an image stem: 3 input channels, 7x7 taps, stride 2, padding 3, 64 output
// channels, NHWC, 16-bit (the first layer of ResNet).  Forward and weight gradient; the stem needs no
// data gradient.  No patch matrix ever reaches HBM: the input is read once, the output written once.
//
// With 3 channels a pixel is 6 bytes, so the 64-channel TMA gather of the implicit-GEMM convolution
// does not apply.  Instead, per tile of 8 x 16 output pixels:
//
//   TMA          a 21-row x 136-element window of the image (rows of W*3 contiguous values; the x
//                coordinate is rounded down to a 16-byte boundary, rows and columns outside the image
//                arrive as zeros = the padding) lands in shared memory, un-swizzled;
//   128 threads  (thread = output pixel) each copy their 7 runs of 24 consecutive values - one per
//                tap row: the value before the receptive field, its 7 taps x 3 channels, two values
//                after; the three strangers are masked to zero - into one 336-byte row of a K-major,
//                128-byte-swizzled UMMA operand (K = 7 x 24 = 168, padded with a zero chunk to 176);
//   tcgen05.mma  forward:  D[128 pixels, 64] = patches[128, 176] . Wk[64, 176]^T (11 instructions);
//                gradient: D[k', 64] += patches^T . dY over the tile's 128 pixels (the patch rows are
//                read as an MN-major operand: the same bytes, another descriptor), accumulated in
//                TMEM over every tile of the CTA and added to the fp32 result with vector reds at
//                the end.
//
// Wk / dWk order K as kh*24 + 1 + kw*3 + ci (the host permutes the weight; the other slots are zero).
// Two CTAs per SM overlap one tile's copy-in with the other's MMA and stores.  Every wait is bounded.
//
// Replaces the reference's direct kernels for this layer: rumus-vision/src/shaders/conv2d_direct.wgsl:40,
// conv2d_backward_weight.wgsl:37.
#include "sm100_common.cuh"

namespace rb {

constexpr int ST_TW = 16, ST_TH = 8;              // output pixels per tile
constexpr int ST_PR = 2 * ST_TH + 5;              // window rows (21)
constexpr int ST_PW = 136;                        // window row pitch in elements (272 B)
constexpr int ST_PATCH_BYTES = ST_PR * ST_PW * 2; // 5712
constexpr int ST_KRUN = 24;                       // values per tap row in K
constexpr int ST_K = 176;                         // 7 * 24 = 168, + one zero chunk
constexpr int ST_KPAD = 192;                      // three 64-wide k blocks in Wk
constexpr int ST_N = 64;
constexpr int ST_CHUNK_BYTES = 128 * 128;         // one 64-wide k block of 128 pixel rows

struct StemParams {
  int B, H, W, Ho, Wo, tiles_w, tiles_h, tiles;
  const void* bias;      // [64] or null (forward)
  void* out;             // forward: [B, Ho, Wo, 64]
  float* dwk;            // gradient: [192, 64] fp32, zero on entry
  int* status;
};

__device__ __forceinline__ void stem_tile_coords(const StemParams& p, int t, int& n, int& oh0, int& ow0) {
  const int tx = t % p.tiles_w;
  const int ty = (t / p.tiles_w) % p.tiles_h;
  n = t / (p.tiles_w * p.tiles_h);
  oh0 = ty * ST_TH;
  ow0 = tx * ST_TW;
}

// window of tile (n, oh0, ow0): x = 6*ow0 - 16 (a multiple of 8 elements), y = 2*oh0 - 3
__device__ __forceinline__ void stem_load_window(uint32_t dst, const CUtensorMap* tx, uint32_t bar, int n,
                                                 int oh0, int ow0) {
  tma_load_3d(dst, tx, bar, 6 * ow0 - 16, 2 * oh0 - 3, n);
}

// thread = pixel (r, c) of the tile: 21 sixteen-byte chunks of operand row `pix`
__device__ __forceinline__ void stem_build_row(const uint8_t* patch, uint8_t* sA, int pix) {
  const int r = pix >> 4, c = pix & 15;
  uint8_t* row = sA + pix * 128;
  const int sw = pix & 7;
#pragma unroll
  for (int kh = 0; kh < 7; ++kh) {
    // values 6c+6 .. 6c+29 of window row 2r+kh: [stranger, 21 wanted, 2 strangers]
    const uint32_t* src = reinterpret_cast<const uint32_t*>(patch + (2 * r + kh) * (ST_PW * 2) + 12 * c + 12);
    uint32_t w[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) w[i] = src[i];
    w[0] &= 0xffff0000u;
    w[11] = 0u;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int q = kh * 3 + j;
      uint8_t* dst = row + (q >> 3) * ST_CHUNK_BYTES + (((q & 7) ^ sw) << 4);
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
  }
}

// ------------------------------------------------------------------------------------ forward
template <typename T>
__global__ void __launch_bounds__(128, 2)
    conv_stem_fwd_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                         const StemParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;                                  // 3 k blocks x [128 rows x 128 B]
  uint8_t* sW = sA + 3 * ST_CHUNK_BYTES;               // 3 k blocks x [64 rows x 128 B]
  uint8_t* sP = sW + 3 * 64 * 128;                     // 2 windows (each rounded up to 5760 B)
  constexpr int PSTRIDE = 5760;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * PSTRIDE);
  uint64_t* win_full = bars;                           // [2]
  uint64_t* w_full = bars + 2;
  uint64_t* mma_done = bars + 3;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp_idx = uniform_warp_idx();
  const int tid = threadIdx.x;
  if (tid == 0) {
    prefetch_tensormap(&tma_x);
    prefetch_tensormap(&tma_w);
    mbar_init(smem_u32(&win_full[0]), 1);
    mbar_init(smem_u32(&win_full[1]), 1);
    mbar_init(smem_u32(w_full), 1);
    mbar_init(smem_u32(mma_done), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp_idx == 0) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 64);
    tmem_relinquish();
  }
  // the zero chunk (K 168..175 = chunk 5 of k block 2) is written once: nothing else stores there
  *reinterpret_cast<uint4*>(sA + 2 * ST_CHUNK_BYTES + tid * 128 + ((5 ^ (tid & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_ptr_smem;

  int t = blockIdx.x;
  int issued = 0;            // windows requested so far (thread 0)
  if (tid == 0) {
    mbar_arrive_expect_tx(smem_u32(w_full), 3 * 64 * 128);
    for (int kb = 0; kb < 3; ++kb) tma_load_2d(smem_u32(sW + kb * 64 * 128), &tma_w, smem_u32(w_full), kb * 64, 0);
    if (t < p.tiles) {
      int n, oh0, ow0;
      stem_tile_coords(p, t, n, oh0, ow0);
      mbar_arrive_expect_tx(smem_u32(&win_full[0]), ST_PATCH_BYTES);
      stem_load_window(smem_u32(sP), &tma_x, smem_u32(&win_full[0]), n, oh0, ow0);
      issued = 1;
    }
  }
  bool ok = mbar_wait(smem_u32(w_full), 0, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
  ok = __syncthreads_and(ok);

  constexpr uint32_t idesc = make_idesc(UmmaFormat<T>::value, 0, 0, 128, ST_N);
  int it = 0;
  for (; ok && t < p.tiles; t += gridDim.x, ++it) {
    const int buf = it & 1;
    // the other window buffer was consumed by the previous iteration's build: request the next tile
    if (tid == 0 && t + (int)gridDim.x < p.tiles) {
      int n, oh0, ow0;
      stem_tile_coords(p, t + gridDim.x, n, oh0, ow0);
      mbar_arrive_expect_tx(smem_u32(&win_full[buf ^ 1]), ST_PATCH_BYTES);
      stem_load_window(smem_u32(sP + (buf ^ 1) * PSTRIDE), &tma_x, smem_u32(&win_full[buf ^ 1]), n, oh0, ow0);
      ++issued;
    }
    ok = mbar_wait(smem_u32(&win_full[buf]), (it >> 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
    if (ok) stem_build_row(sP + buf * PSTRIDE, sA, tid);
    fence_proxy_async_smem();      // generic-proxy stores -> visible to the tensor core's reads
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < ST_K / 16; ++k) {
        const uint64_t adesc = make_smem_desc_sw128(smem_u32(sA) + (k >> 2) * ST_CHUNK_BYTES + (k & 3) * 32, 16, 1024);
        const uint64_t bdesc = make_smem_desc_sw128(smem_u32(sW) + (k >> 2) * 64 * 128 + (k & 3) * 32, 16, 1024);
        umma_f16(tmem_d, adesc, bdesc, idesc, k != 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(mma_done));
    }
    ok = mbar_wait(smem_u32(mma_done), it & 1, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after();
    // epilogue: TMEM lane = pixel; 64 channels = 128 contiguous bytes of the NHWC output
    int n, oh0, ow0;
    stem_tile_coords(p, t, n, oh0, ow0);
    const int oh = oh0 + (tid >> 4), ow = ow0 + (tid & 15);
    uint32_t v[64];
    const uint32_t taddr = tmem_d + ((uint32_t)(warp_idx * 32) << 16);
    tmem_ld_32x32b_x32(taddr, v);
    tmem_ld_32x32b_x32(taddr + 32, v + 32);
    tmem_ld_wait();
    if (oh < p.Ho && ow < p.Wo) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + (((long long)n * p.Ho + oh) * p.Wo + ow) * ST_N);
      const T* bias = reinterpret_cast<const T*>(p.bias);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[j * 8 + e]) + (bias ? to_f32<T>(bias[j * 8 + e]) : 0.f);
        dst[j] = make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]), pack2<T>(f[6], f[7]));
      }
    }
    tc_fence_before();
    __syncthreads();               // every lane of the accumulator is read before the next tile's MMAs
  }
  // leave: copies still in flight (only after a failed wait) are given their time, then TMEM goes back
  if (tid == 0 && !ok) {
    for (int i = max(0, issued - 2); i < issued; ++i) mbar_drain(smem_u32(&win_full[i & 1]), (i >> 1) & 1, p.status);
  }
  tc_fence_before();
  __syncthreads();
  if (warp_idx == 0) tmem_dealloc(tmem_d, 64);
}

// ---------------------------------------------------------------------------- weight gradient
template <typename T>
__global__ void __launch_bounds__(128, 2)
    conv_stem_wgrad_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_dy,
                           const StemParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;                                  // 4 chunks of 64 k' x [128 pixel rows x 128 B]; chunk 3 stays zero
  uint8_t* sD = sA + 4 * ST_CHUNK_BYTES;               // 2 x dY tile [128 pixel rows x 128 B]
  uint8_t* sP = sD + 2 * ST_CHUNK_BYTES;               // 2 windows
  constexpr int PSTRIDE = 5760;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * PSTRIDE);
  uint64_t* full = bars;                               // [2]: window + dY tile
  uint64_t* mma_done = bars + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp_idx = uniform_warp_idx();
  const int tid = threadIdx.x;
  if (tid == 0) {
    prefetch_tensormap(&tma_x);
    prefetch_tensormap(&tma_dy);
    mbar_init(smem_u32(&full[0]), 1);
    mbar_init(smem_u32(&full[1]), 1);
    mbar_init(smem_u32(mma_done), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp_idx == 0) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 128);
    tmem_relinquish();
  }
  // zero what no build ever writes: chunks 5..7 of k block 2 (k' 168..191) and the whole of chunk 3
  {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    uint8_t* row2 = sA + 2 * ST_CHUNK_BYTES + tid * 128;
#pragma unroll
    for (int cj = 5; cj < 8; ++cj) *reinterpret_cast<uint4*>(row2 + ((cj ^ (tid & 7)) << 4)) = z;
    uint4* row3 = reinterpret_cast<uint4*>(sA + 3 * ST_CHUNK_BYTES + tid * 128);
#pragma unroll
    for (int cj = 0; cj < 8; ++cj) row3[cj] = z;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_ptr_smem;

  auto request = [&](int tile, int buf) {
    int n, oh0, ow0;
    stem_tile_coords(p, tile, n, oh0, ow0);
    const uint32_t bar = smem_u32(&full[buf]);
    mbar_arrive_expect_tx(bar, ST_PATCH_BYTES + ST_CHUNK_BYTES);
    stem_load_window(smem_u32(sP + buf * PSTRIDE), &tma_x, bar, n, oh0, ow0);
    tma_load_4d(smem_u32(sD + buf * ST_CHUNK_BYTES), &tma_dy, bar, 0, ow0, oh0, n);
  };
  int t = blockIdx.x;
  int issued = 0;
  if (tid == 0 && t < p.tiles) {
    request(t, 0);
    issued = 1;
  }
  // A = patches read MN-major (k' contiguous, 64 per 128-byte row chunk, chunks 16 KB apart),
  // B = dY read MN-major (64 output channels per row); K = the tile's 128 pixels
  constexpr uint32_t idesc = make_idesc(UmmaFormat<T>::value, 1, 1, 128, ST_N);
  bool ok = true;
  int it = 0;
  for (; t < p.tiles; t += gridDim.x, ++it) {
    const int buf = it & 1;
    // the previous tile's MMAs read sA and the other dY buffer: both are free once they retired
    if (it > 0) ok = mbar_wait(smem_u32(mma_done), (it - 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (tid == 0 && t + (int)gridDim.x < p.tiles) {
      request(t + gridDim.x, buf ^ 1);
      ++issued;
    }
    ok = mbar_wait(smem_u32(&full[buf]), (it >> 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_FULL);
    if (ok) stem_build_row(sP + buf * PSTRIDE, sA, tid);
    fence_proxy_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int mb = 0; mb < 2; ++mb) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t adesc = make_smem_desc_sw128(smem_u32(sA) + mb * 2 * ST_CHUNK_BYTES + k * 2048, ST_CHUNK_BYTES, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(sD + buf * ST_CHUNK_BYTES) + k * 2048, ST_CHUNK_BYTES, 1024);
          umma_f16(tmem_d + mb * ST_N, adesc, bdesc, idesc, (it | k) != 0 ? 1u : 0u);
        }
      }
      umma_commit(smem_u32(mma_done));
    }
  }
  if (ok && it > 0) {
    ok = mbar_wait(smem_u32(mma_done), (it - 1) & 1, abort_flag, p.status, RB_ERR_TIMEOUT_TMEM_FULL);
    ok = __syncthreads_and(ok);
    if (ok) {
      tc_fence_after();
      // accumulator row = k' (two blocks of 128), column = output channel
#pragma unroll 1
      for (int mb = 0; mb < 2; ++mb) {
        const int kq = mb * 128 + tid;
        uint32_t v[64];
        const uint32_t taddr = tmem_d + ((uint32_t)(warp_idx * 32) << 16) + mb * ST_N;
        tmem_ld_32x32b_x32(taddr, v);
        tmem_ld_32x32b_x32(taddr + 32, v + 32);
        tmem_ld_wait();
        if (kq < ST_KPAD) {
          float* o = p.dwk + kq * ST_N;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + i * 4),
                         "f"(__uint_as_float(v[4 * i])), "f"(__uint_as_float(v[4 * i + 1])),
                         "f"(__uint_as_float(v[4 * i + 2])), "f"(__uint_as_float(v[4 * i + 3]))
                         : "memory");
        }
      }
    }
  }
  if (tid == 0 && !ok) {
    for (int i = max(0, issued - 2); i < issued; ++i) mbar_drain(smem_u32(&full[i & 1]), (i >> 1) & 1, p.status);
  }
  tc_fence_before();
  __syncthreads();
  if (warp_idx == 0) tmem_dealloc(tmem_d, 128);
}

static int stem_geometry(StemParams& p, int B, int H, int W) {
  if (B <= 0 || H <= 0 || W <= 0 || (W % 8) != 0) return 60;
  p.B = B; p.H = H; p.W = W;
  p.Ho = (H + 6 - 7) / 2 + 1;
  p.Wo = (W + 6 - 7) / 2 + 1;
  p.tiles_w = (p.Wo + ST_TW - 1) / ST_TW;
  p.tiles_h = (p.Ho + ST_TH - 1) / ST_TH;
  const long long tiles = (long long)p.tiles_w * p.tiles_h * B;
  if (tiles > 0x7fffffff) return 60;
  p.tiles = (int)tiles;
  return 0;
}

// the image as [B][H][W*3] with a 136 x 21 x 1 window, no swizzle
static int stem_image_map(CUtensorMap* m, int dtype, const void* x, int B, int H, int W) {
  uint64_t dims[3] = {(uint64_t)W * 3, (uint64_t)H, (uint64_t)B};
  uint64_t strides[3] = {2, (uint64_t)W * 6, (uint64_t)W * 6 * H};
  uint32_t box[3] = {ST_PW, ST_PR, 1};
  return rbh::encode_tensor_map(m, dtype, 3, const_cast<void*>(x), dims, strides, box, 0);
}

}  // namespace rb

extern "C" {

// y[B, Ho, Wo, 64] = conv7x7/2 pad 3 of x[B, H, W, 3] with wk[64, 192] (K order kh*24 + 1 + kw*3 + ci, zeros
// elsewhere) + bias.  W % 8 == 0.  Returns 60 for anything else.
int rb_conv_stem_fwd(int dtype, const void* x, const void* wk, const void* bias, void* y, int B, int H, int W,
                     void* stream) {
  using namespace rb;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 60;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wk) | reinterpret_cast<uintptr_t>(y)) & 15) return 60;
  StemParams p{};
  int rc = stem_geometry(p, B, H, W);
  if (rc) return rc;
  p.bias = bias; p.out = y; p.status = rbh::device_status_word();
  CUtensorMap tx, tw;
  rc = stem_image_map(&tx, dtype, x, B, H, W);
  if (rc) return 1000 + rc;
  {
    uint64_t dims[2] = {ST_KPAD, ST_N}, strides[2] = {2, ST_KPAD * 2};
    uint32_t box[2] = {64, ST_N};
    rc = rbh::encode_tensor_map(&tw, dtype, 2, const_cast<void*>(wk), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  const int smem = 3 * ST_CHUNK_BYTES + 3 * 64 * 128 + 2 * 5760 + 64 + 1024;
  const int grid = p.tiles < 2 * rbh::sm_count() ? p.tiles : 2 * rbh::sm_count();
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == rbh::DT_BF16) {
    e = cudaFuncSetAttribute(conv_stem_fwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    conv_stem_fwd_kernel<__nv_bfloat16><<<grid, 128, smem, st>>>(tx, tw, p);
  } else {
    e = cudaFuncSetAttribute(conv_stem_fwd_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    conv_stem_fwd_kernel<__half><<<grid, 128, smem, st>>>(tx, tw, p);
  }
  return (int)cudaGetLastError();
}

// dwk[192, 64] (fp32, zero on entry) += patches(x)^T . dy, dy [B, Ho, Wo, 64]; row kh*24 + 1 + kw*3 + ci of
// dwk is the gradient of tap (kh, kw), input channel ci; the other rows are not meaningful.
int rb_conv_stem_wgrad(int dtype, const void* x, const void* dy, float* dwk, int B, int H, int W, void* stream) {
  using namespace rb;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 60;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dwk)) & 15) return 60;
  StemParams p{};
  int rc = stem_geometry(p, B, H, W);
  if (rc) return rc;
  p.dwk = dwk; p.status = rbh::device_status_word();
  CUtensorMap tx, td;
  rc = stem_image_map(&tx, dtype, x, B, H, W);
  if (rc) return 1000 + rc;
  {
    uint64_t dims[4] = {ST_N, (uint64_t)p.Wo, (uint64_t)p.Ho, (uint64_t)B};
    uint64_t strides[4] = {2, ST_N * 2, (uint64_t)p.Wo * ST_N * 2, (uint64_t)p.Ho * p.Wo * ST_N * 2};
    uint32_t box[4] = {ST_N, ST_TW, ST_TH, 1};
    rc = rbh::encode_tensor_map(&td, dtype, 4, const_cast<void*>(dy), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  const int smem = 6 * ST_CHUNK_BYTES + 2 * 5760 + 64 + 1024;
  const int grid = p.tiles < 2 * rbh::sm_count() ? p.tiles : 2 * rbh::sm_count();
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == rbh::DT_BF16) {
    e = cudaFuncSetAttribute(conv_stem_wgrad_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    conv_stem_wgrad_kernel<__nv_bfloat16><<<grid, 128, smem, st>>>(tx, td, p);
  } else {
    e = cudaFuncSetAttribute(conv_stem_wgrad_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    conv_stem_wgrad_kernel<__half><<<grid, 128, smem, st>>>(tx, td, p);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
