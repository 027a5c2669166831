// Implicit-GEMM convolution on the tcgen05 GEMM body: no im2col buffer is ever written.
//
// Activations are NHWC.  The producer warp of the GEMM fetches operand tiles straight out of the
// activation tensor with 4-D tiled TMA copies (dimensions C, W, H, B; traversal strides = the
// convolution stride; coordinates outside the image are filled with zeros by the copy engine, which
// is the padding):
//
//   forward      Y[pixels, Cout] = sum over taps (kh, kw) and 64-channel blocks of
//                X[patch of 128 output pixels shifted by the tap, 64 channels] . W[(kh,kw,c), Cout]
//                A tile = one box {64 channels, TW, TH, TN} (TW*TH*TN = 128 output pixels of TN images),
//                B tile = rows of the [Cout, KH*KW*Cin] weight matrix (plain 2-D copy)
//   data grad    the same kernel on dY with the taps mirrored and the weight matrix rearranged to
//                [Cin, (kh,kw,co)].  Stride s > 1: one launch per phase (ih + pad) mod s, (iw + pad) mod s
//                of the input pixels; a phase sees only the taps kh = phase + s*a, is a stride-1
//                gather over dY, and writes every s-th input pixel
//   weight grad  dW[Cout, (kh,kw,ci)] = sum over pixels dY[pixel, co] . X[pixel shifted by tap, ci]:
//                K runs over 8 x 8 patches of output pixels; A = boxes of dY (M-major operand),
//                B = boxes of X shifted by the tap (N-major operand); K is split across CTAs and the
//                partial products are added into an fp32 matrix.
//
// The reference computes convolutions directly as well, one thread per output element
// (rumus-vision/src/shaders/conv2d_direct.wgsl:40, conv2d_backward_data.wgsl:37,
// conv2d_backward_weight.wgsl:37; rationale rumus-vision/README.md:3-7).
#include "gemm_launch.cuh"

namespace rb {

struct ConvGeom {
  int B, Ho, Wo;          // output-pixel grid the GEMM rows (forward / data grad) or K (weight grad) run over
  int KH, KW, stride, dil;
  int off_h, off_w;       // input coordinate of tap (0,0) for output pixel 0: -pad (forward, weight grad), +pad (data grad)
  int tap_sign;           // +1: in = out*stride + off + k*dil (forward, weight grad); -1: in = out + off - k*dil (data grad)
  int TW, TH, TN;         // patch of output pixels per 128-row tile (forward / data grad)
  int tiles_w, tiles_h;
  int cblocks;            // 64-channel blocks of the gathered tensor
  int patches_w, patches_h;   // weight grad: 8 x 8 pixel patches per image
  int os, oe_h, oe_w;     // rows are written to pixel (h*os + oe_h, w*os + oe_w) of an OH x OW image
  int OH, OW;             //   (os = 1, oe = 0, OH x OW = Ho x Wo except for the phases of a strided data gradient)
};

struct ConvHooksBase {
  ConvGeom g;
  __device__ __forceinline__ bool before_tile_load(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ bool before_k_load(int, int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ int map_kb(int kb, int) const { return kb; }
  __device__ __forceinline__ void after_tile_store(int, int, int) const {}
  static constexpr bool kNeedsStoreComplete = false;
  static constexpr bool kCustomRaster = false;
  __device__ __forceinline__ void raster(int, int, int, int&, int&) const {}
};

// forward and stride-1 data gradient: rows of the GEMM are output pixels
struct ConvRowHooks : ConvHooksBase {
  static constexpr bool kCustomLoadA = true;
  static constexpr bool kCustomLoadB = false;
  static constexpr bool kCustomRows = true;
  __device__ __forceinline__ void load_a(uint32_t dst, const CUtensorMap* tma, uint32_t bar, int m_idx, int kb) const {
    const int tw = m_idx % g.tiles_w;
    const int t = m_idx / g.tiles_w;
    const int th = t % g.tiles_h, tn = t / g.tiles_h;
    const int tap = kb / g.cblocks, cblk = kb - tap * g.cblocks;
    const int kh = tap / g.KW, kw = tap - kh * g.KW;
    const int w = tw * g.TW * g.stride + g.off_w + g.tap_sign * kw * g.dil;
    const int h = th * g.TH * g.stride + g.off_h + g.tap_sign * kh * g.dil;
    tma_load_4d(dst, tma, bar, cblk * 64, w, h, tn * g.TN);
  }
  __device__ __forceinline__ void load_b(uint32_t, const CUtensorMap*, uint32_t, int, int) const {}
  __device__ __forceinline__ long long out_row(int m_idx, int r) const {
    const int tw = m_idx % g.tiles_w;
    const int t = m_idx / g.tiles_w;
    const int th = t % g.tiles_h, tn = t / g.tiles_h;
    const int w = tw * g.TW + r % g.TW;
    const int q = r / g.TW;
    const int h = th * g.TH + q % g.TH;
    const int n = tn * g.TN + q / g.TH;
    if (w >= g.Wo || h >= g.Ho || n >= g.B) return -1;
    return (static_cast<long long>(n) * g.OH + (h * g.os + g.oe_h)) * g.OW + (w * g.os + g.oe_w);
  }
};

// weight gradient: K runs over 8 x 8 patches of output pixels; BN = 128 -> two 64-wide chunks per operand
struct ConvWgradHooks : ConvHooksBase {
  static constexpr bool kCustomLoadA = true;
  static constexpr bool kCustomLoadB = true;
  static constexpr bool kCustomRows = false;
  __device__ __forceinline__ void patch(int kb, int& pw, int& ph, int& n) const {
    pw = kb % g.patches_w;
    const int t = kb / g.patches_w;
    ph = t % g.patches_h;
    n = t / g.patches_h;
  }
  // A = dY as an M-major operand: chunk j = 64 output channels x 64 pixels of the patch
  __device__ __forceinline__ void load_a(uint32_t dst, const CUtensorMap* tma, uint32_t bar, int m_idx, int kb) const {
    int pw, ph, n;
    patch(kb, pw, ph, n);
#pragma unroll
    for (int j = 0; j < 2; ++j) tma_load_4d(dst + j * 64 * 128, tma, bar, m_idx * 128 + j * 64, pw * 8, ph * 8, n);
  }
  // B = X shifted by the tap as an N-major operand: chunk j = 64 input channels of one tap
  __device__ __forceinline__ void load_b(uint32_t dst, const CUtensorMap* tma, uint32_t bar, int n_idx, int kb) const {
    int pw, ph, n;
    patch(kb, pw, ph, n);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int q = n_idx * 2 + j;
      const int tap = q / g.cblocks, cblk = q - tap * g.cblocks;
      const int kh = tap / g.KW, kw = tap - kh * g.KW;
      // chunks past the last tap still have to deliver their bytes: an image index past the batch reads zeros
      const int nn = tap < g.KH * g.KW ? n : g.B;
      tma_load_4d(dst + j * 64 * 128, tma, bar, cblk * 64, pw * 8 * g.stride + g.off_w + kw * g.dil,
                  ph * 8 * g.stride + g.off_h + kh * g.dil, nn);
    }
  }
  __device__ __forceinline__ long long out_row(int, int) const { return -1; }
};

template <typename T, int BN, bool A_MN, bool B_MN, typename Hooks>
__global__ void __launch_bounds__(320, 1)
    conv_igemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const GemmParams p, const Hooks hooks) {
  extern __shared__ uint8_t smem_raw[];
  gemm_cta_body<T, BN, A_MN, B_MN, Hooks>(&tma_a, &tma_b, p, hooks, smem_raw, blockIdx.x, gridDim.x);
}

// NHWC activation as a 4-D map {C, W, H, B}; `pw` x `ph` x `pn` pixels per box, every `stride`-th one
static int make_act_map(CUtensorMap* m, int dtype, const void* base, int B, int H, int W, int C, int pw, int ph,
                        int pn, int stride) {
  uint64_t dims[4] = {(uint64_t)C, (uint64_t)W, (uint64_t)H, (uint64_t)B};
  uint64_t strides[4] = {2, (uint64_t)C * 2, (uint64_t)W * C * 2, (uint64_t)H * W * C * 2};
  uint32_t box[4] = {64, (uint32_t)((pw - 1) * stride + 1), (uint32_t)((ph - 1) * stride + 1), (uint32_t)pn};
  uint32_t es[4] = {1, (uint32_t)stride, (uint32_t)stride, 1};
  return rbh::encode_tensor_map_strided(m, dtype, 4, const_cast<void*>(base), dims, strides, box, es, 1);
}

template <typename T, int BN, bool A_MN, bool B_MN, typename Hooks>
static int launch_conv(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, const Hooks& h,
                       int work_items, cudaStream_t st) {
  using C = GemmCfg<T, BN>;
  auto kern = conv_igemm_kernel<T, BN, A_MN, B_MN, Hooks>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return 2000 + (int)e;
  int ctas = rbh::sm_count();
  if (work_items < ctas) ctas = work_items;
  kern<<<ctas, C::NUM_THREADS, C::SMEM_BYTES, st>>>(ta, tb, p, h);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {

// Forward (mode 0) or stride-1 data gradient (mode 1) of a 2-D convolution, NHWC, 16-bit.
//   act   [B, H, W, C]      the tensor patches are gathered from (x for mode 0, dY for mode 1), C % 64 == 0
//   wmat  [N, KH*KW*C]      K-major weight matrix, K ordered (kh, kw, c); N = output channels of this GEMM
//   out   [B, Ho, Wo, N]    (Ho, Wo: output-pixel grid; for mode 1 the input image size)
//   tw/th/tn                patch of output pixels per tile, tw*th*tn == 128
// bias [N] and relu are optional epilogue terms.  Returns 60 for shapes outside what this path covers.
int rb_conv_igemm(int mode, int dtype, const void* act, const void* wmat, void* out, const void* bias, int relu,
                  int B, int H, int W, int C, int Ho, int Wo, int N, int KH, int KW, int stride, int pad, int dil,
                  int tw, int th, int tn, void* stream) {
  using namespace rb;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 60;
  if (C % 64 || N % 8 || tw * th * tn != 128 || (mode == 1 && stride != 1)) return 60;
  if ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(wmat) | reinterpret_cast<uintptr_t>(out)) & 15) return 60;
  ConvRowHooks h;
  ConvGeom& g = h.g;
  g.B = B; g.Ho = Ho; g.Wo = Wo; g.KH = KH; g.KW = KW; g.stride = stride; g.dil = dil;
  g.off_h = g.off_w = mode == 0 ? -pad : pad;
  g.tap_sign = mode == 0 ? 1 : -1;
  g.TW = tw; g.TH = th; g.TN = tn;
  g.tiles_w = (Wo + tw - 1) / tw; g.tiles_h = (Ho + th - 1) / th;
  g.cblocks = C / 64; g.patches_w = g.patches_h = 0;
  g.os = 1; g.oe_h = g.oe_w = 0; g.OH = Ho; g.OW = Wo;
  const int tiles_n = (B + tn - 1) / tn;
  const int num_m = g.tiles_w * g.tiles_h * tiles_n;
  const long long K = (long long)KH * KW * C;
  CUtensorMap ta, tb;
  int rc = make_act_map(&ta, dtype, act, B, H, W, C, tw, th, tn, stride);
  if (rc) return 1000 + rc;
  const int BN = N <= 128 ? 128 : 256;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N}, strides[2] = {2, (uint64_t)K * 2};
    uint32_t box[2] = {64, (uint32_t)BN};
    rc = rbh::encode_tensor_map(&tb, dtype, 2, const_cast<void*>(wmat), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  GemmParams p{};
  p.M = num_m * 128; p.N = N; p.K = (int)K;
  p.out = out; p.ldc = N; p.bias = bias; p.act = relu ? ACT_RELU : ACT_NONE; p.alpha = 1.f;
  p.vec_ok = 1; p.group_m = 8; p.split_k = 1;
  p.status = rbh::device_status_word();
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  const int items = num_m * ((N + BN - 1) / BN);
  cudaStream_t st = (cudaStream_t)stream;
#define RB_CONV_ROW(T_) \
  (BN == 128 ? launch_conv<T_, 128, false, false, ConvRowHooks>(ta, tb, p, h, items, st) \
             : launch_conv<T_, 256, false, false, ConvRowHooks>(ta, tb, p, h, items, st))
  return dtype == rbh::DT_BF16 ? RB_CONV_ROW(__nv_bfloat16) : RB_CONV_ROW(__half);
#undef RB_CONV_ROW
}

// One phase of the data gradient of a convolution with stride s > 1 (dilation 1): the input pixels
// (s*u + e_h, s*v + e_w) of dx [B, H, W, N] receive sum over the phase's taps (a, b) of
// dY[u + c_h - a, v + c_w - b, :] . wphase[n, (a, b, co)], dY [B, Hy, Wy, C], C % 64 == 0.
// wphase [N, KHp*KWp*C] holds the taps kh = rh + s*a, kw = rw + s*b of the phase (the caller derives
// e, c and the tap counts from rh, rw, s and the padding).  Other pixels of dx are not touched.
int rb_conv_igemm_dgrad_phase(int dtype, const void* dy, const void* wphase, void* dx, int B, int Hy, int Wy, int C,
                              int H, int W, int N, int KHp, int KWp, int s, int c_h, int c_w, int e_h, int e_w,
                              int tw, int th, int tn, void* stream) {
  using namespace rb;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 60;
  if (C % 64 || N % 8 || tw * th * tn != 128 || s < 1 || KHp < 1 || KWp < 1) return 60;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(wphase) | reinterpret_cast<uintptr_t>(dx)) & 15) return 60;
  if (e_h >= H || e_w >= W) return 0;
  ConvRowHooks h;
  ConvGeom& g = h.g;
  g.B = B; g.Ho = (H - e_h + s - 1) / s; g.Wo = (W - e_w + s - 1) / s;
  g.KH = KHp; g.KW = KWp; g.stride = 1; g.dil = 1;
  g.off_h = c_h; g.off_w = c_w; g.tap_sign = -1;
  g.TW = tw; g.TH = th; g.TN = tn;
  g.tiles_w = (g.Wo + tw - 1) / tw; g.tiles_h = (g.Ho + th - 1) / th;
  g.cblocks = C / 64; g.patches_w = g.patches_h = 0;
  g.os = s; g.oe_h = e_h; g.oe_w = e_w; g.OH = H; g.OW = W;
  const int tiles_n = (B + tn - 1) / tn;
  const int num_m = g.tiles_w * g.tiles_h * tiles_n;
  const long long K = (long long)KHp * KWp * C;
  CUtensorMap ta, tb;
  int rc = make_act_map(&ta, dtype, dy, B, Hy, Wy, C, tw, th, tn, 1);
  if (rc) return 1000 + rc;
  const int BN = N <= 128 ? 128 : 256;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N}, strides[2] = {2, (uint64_t)K * 2};
    uint32_t box[2] = {64, (uint32_t)BN};
    rc = rbh::encode_tensor_map(&tb, dtype, 2, const_cast<void*>(wphase), dims, strides, box, 1);
    if (rc) return 1000 + rc;
  }
  GemmParams p{};
  p.M = num_m * 128; p.N = N; p.K = (int)K;
  p.out = dx; p.ldc = N; p.act = ACT_NONE; p.alpha = 1.f;
  p.vec_ok = 1; p.group_m = 8; p.split_k = 1;
  p.status = rbh::device_status_word();
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  const int items = num_m * ((N + BN - 1) / BN);
  cudaStream_t st = (cudaStream_t)stream;
#define RB_CONV_ROW(T_) \
  (BN == 128 ? launch_conv<T_, 128, false, false, ConvRowHooks>(ta, tb, p, h, items, st) \
             : launch_conv<T_, 256, false, false, ConvRowHooks>(ta, tb, p, h, items, st))
  return dtype == rbh::DT_BF16 ? RB_CONV_ROW(__nv_bfloat16) : RB_CONV_ROW(__half);
#undef RB_CONV_ROW
}

// Weight gradient: dwmat[Cout, KH*KW*C] (fp32, zero on entry) += dY^T . patches(x).
//   dy [B, Ho, Wo, Cout], x [B, H, W, C]; C % 64 == 0, Cout % 8 == 0
int rb_conv_igemm_wgrad(int dtype, const void* dy, const void* x, float* dwmat, int B, int H, int W, int C, int Ho,
                        int Wo, int Cout, int KH, int KW, int stride, int pad, int dil, void* stream) {
  using namespace rb;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 60;
  if (C % 64 || Cout % 8) return 60;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dwmat)) & 15) return 60;
  ConvWgradHooks h;
  ConvGeom& g = h.g;
  g.B = B; g.Ho = Ho; g.Wo = Wo; g.KH = KH; g.KW = KW; g.stride = stride; g.dil = dil;
  g.off_h = g.off_w = -pad; g.tap_sign = 1;
  g.TW = g.TH = g.TN = 0; g.tiles_w = g.tiles_h = 0;
  g.cblocks = C / 64;
  g.patches_w = (Wo + 7) / 8; g.patches_h = (Ho + 7) / 8;
  const int num_kb = B * g.patches_w * g.patches_h;
  const int Ncols = KH * KW * C;
  CUtensorMap ta, tb;
  int rc = make_act_map(&ta, dtype, dy, B, Ho, Wo, Cout, 8, 8, 1, 1);
  if (rc) return 1000 + rc;
  rc = make_act_map(&tb, dtype, x, B, H, W, C, 8, 8, 1, stride);
  if (rc) return 1000 + rc;
  GemmParams p{};
  p.M = Cout; p.N = Ncols; p.K = num_kb * 64;
  p.out = dwmat; p.ldc = Ncols; p.out_f32 = 1; p.alpha = 1.f;
  p.vec_ok = (Ncols * 4) % 16 == 0; p.group_m = 8;
  p.status = rbh::device_status_word();
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  const int tiles = ((Cout + 127) / 128) * ((Ncols + 127) / 128);
  int split = (2 * rbh::sm_count() + tiles - 1) / tiles;            // about two work items per SM
  const int max_split = num_kb / 8 > 0 ? num_kb / 8 : 1;           // at least 8 K blocks per slice
  if (split > max_split) split = max_split;
  if (split < 2) split = 2;                                         // the epilogue adds: always the split-K form
  if (split > num_kb) split = num_kb;
  const int kb_per = (num_kb + split - 1) / split;
  p.split_k = (num_kb + kb_per - 1) / kb_per;
  if (p.split_k < 2) return 60;                                     // a single K block: not worth this path
  const int items = tiles * p.split_k;
  cudaStream_t st = (cudaStream_t)stream;
  return dtype == rbh::DT_BF16 ? launch_conv<__nv_bfloat16, 128, true, true, ConvWgradHooks>(ta, tb, p, h, items, st)
                               : launch_conv<__half, 128, true, true, ConvWgradHooks>(ta, tb, p, h, items, st);
}
}
