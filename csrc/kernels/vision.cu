// Vision kernels for sm_100a, NHWC (channels-last) activations:
//   im2col / col2im feeding the tcgen05 GEMM (implicit-GEMM convolution: forward, data gradient,
//   weight gradient), BatchNorm2d statistics / normalise (+residual, +ReLU) / backward,
//   max-pool (overlapping windows, local argmax index) and adaptive average pool.
//
// Reference counterparts: rumus/src/backend/gpu/shaders/conv.wgsl:30-142 (im2col/col2im, never
// dispatched), rumus-vision/src/shaders/conv2d_*.wgsl (one thread per output element direct
// conv), batch_norm.wgsl:34 / batch_norm_bw.wgsl:24 (one workgroup per channel; d_gamma/d_beta on
// the CPU), maxpool2d_*.wgsl (non-atomic scatter, wrong for overlapping windows),
// adaptive_pool.wgsl:25,62.
#include "sm100_common.cuh"

namespace rb {

// cols[m, (kh*KW + kw)*C + c] = x[b, ih, iw, c]   (zero outside), m = (b*Ho + oh)*Wo + ow
// Kpad >= KH*KW*C pads each row with zeros (TMA needs 16-byte row pitch).
template <typename T>
__global__ void im2col_nhwc_kernel(const T* __restrict__ x, T* __restrict__ cols, int B, int H,
                                   int W, int C, int KH, int KW, int Ho, int Wo, int stride,
                                   int pad, int dil, int Kpad) {
  const long long total = (long long)B * Ho * Wo * Kpad;
  const long long gs = (long long)gridDim.x * blockDim.x;
  const int Kdim = KH * KW * C;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int k = (int)(i % Kpad);
    const long long m = i / Kpad;
    T v = from_f32<T>(0.f);
    if (k < Kdim) {
      const int c = k % C;
      const int kk = k / C;
      const int kw = kk % KW, kh = kk / KW;
      const int ow = (int)(m % Wo);
      const long long t = m / Wo;
      const int oh = (int)(t % Ho);
      const int b = (int)(t / Ho);
      const int ih = oh * stride - pad + kh * dil;
      const int iw = ow * stride - pad + kw * dil;
      if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = x[(((long long)b * H + ih) * W + iw) * C + c];
    }
    cols[i] = v;
  }
}

// gather form of col2im: dx[b, ih, iw, c] = sum over (kh,kw) with a matching output position
template <typename T>
__global__ void col2im_nhwc_kernel(const T* __restrict__ dcols, T* __restrict__ dx, int B, int H,
                                   int W, int C, int KH, int KW, int Ho, int Wo, int stride,
                                   int pad, int dil, int Kpad) {
  const long long total = (long long)B * H * W * C;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int c = (int)(i % C);
    long long t = i / C;
    const int iw = (int)(t % W);
    t /= W;
    const int ih = (int)(t % H);
    const int b = (int)(t / H);
    float acc = 0.f;
    for (int kh = 0; kh < KH; ++kh) {
      const int nh = ih + pad - kh * dil;
      if (nh < 0 || nh % stride) continue;
      const int oh = nh / stride;
      if (oh >= Ho) continue;
      for (int kw = 0; kw < KW; ++kw) {
        const int nw = iw + pad - kw * dil;
        if (nw < 0 || nw % stride) continue;
        const int ow = nw / stride;
        if (ow >= Wo) continue;
        const long long m = ((long long)b * Ho + oh) * Wo + ow;
        acc += to_f32<T>(dcols[m * Kpad + (kh * KW + kw) * C + c]);
      }
    }
    dx[i] = from_f32<T>(acc);
  }
}

// ---------------------------------------------------------------------------------- batch norm
// stage 1: per-slab partial sums over rows of an [M, C] matrix: partials[slab][0][c] = sum x,
// partials[slab][1][c] = sum x^2  (or, in backward, sum dy' and sum dy'*xhat)
template <typename T, bool BWD>
__global__ void bn_partial_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                  const T* __restrict__ y, const float* __restrict__ mean,
                                  const float* __restrict__ rstd, float* __restrict__ partials,
                                  long long M, int C, int rows_per_slab, int relu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const long long r0 = (long long)blockIdx.y * rows_per_slab;
  const long long r1 = min(M, r0 + rows_per_slab);
  float a = 0.f, b = 0.f;
  float mu = 0.f, rs = 1.f;
  if (BWD) { mu = mean[c]; rs = rstd[c]; }
  for (long long r = r0; r < r1; ++r) {
    const float xv = to_f32<T>(x[r * C + c]);
    if (!BWD) {
      a += xv;
      b += xv * xv;
    } else {
      float d = to_f32<T>(dy[r * C + c]);
      if (relu && to_f32<T>(y[r * C + c]) <= 0.f) d = 0.f;
      a += d;
      b += d * (xv - mu) * rs;
    }
  }
  partials[((long long)blockIdx.y * 2) * C + c] = a;
  partials[((long long)blockIdx.y * 2 + 1) * C + c] = b;
}

// stage 2 (forward): mean / rstd, running-stat update (biased variance, as the reference)
__global__ void bn_finalize_fwd_kernel(const float* __restrict__ partials, int slabs, int C,
                                       long long M, float eps, float momentum,
                                       float* __restrict__ mean, float* __restrict__ rstd,
                                       float* __restrict__ running_mean,
                                       float* __restrict__ running_var) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, q = 0.f;
  for (int i = 0; i < slabs; ++i) {
    s += partials[((long long)i * 2) * C + c];
    q += partials[((long long)i * 2 + 1) * C + c];
  }
  const float mu = s / (float)M;
  const float var = fmaxf(q / (float)M - mu * mu, 0.f);
  mean[c] = mu;
  rstd[c] = rsqrtf(var + eps);
  if (running_mean) {
    running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mu;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * var;
  }
}
// stage 2 (backward): sums -> dgamma, dbeta, and the two per-channel coefficients of dx
template <typename T>
__global__ void bn_finalize_bwd_kernel(const float* __restrict__ partials, int slabs, int C,
                                       float* __restrict__ sums, T* __restrict__ dgamma,
                                       T* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, q = 0.f;
  for (int i = 0; i < slabs; ++i) {
    s += partials[((long long)i * 2) * C + c];
    q += partials[((long long)i * 2 + 1) * C + c];
  }
  sums[c] = s;
  sums[C + c] = q;
  dbeta[c] = from_f32<T>(s);
  dgamma[c] = from_f32<T>(q);
}
// y = relu( (x - mean) * rstd * gamma + beta + residual )
template <typename T>
__global__ void bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                const T* __restrict__ gamma, const T* __restrict__ beta,
                                const float* __restrict__ mean, const float* __restrict__ rstd,
                                T* __restrict__ y, long long n, int C, int relu) {
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gs) {
    const int c = (int)(i % C);
    float v = (to_f32<T>(x[i]) - mean[c]) * rstd[c] * to_f32<T>(gamma[c]) + to_f32<T>(beta[c]);
    if (res) v += to_f32<T>(res[i]);
    if (relu) v = fmaxf(v, 0.f);
    y[i] = from_f32<T>(v);
  }
}
// dx = gamma*rstd*(dy' - sum_dy/M - xhat*sum_dyxhat/M); dres = dy' (dy masked by the ReLU)
template <typename T>
__global__ void bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                    const T* __restrict__ y, const T* __restrict__ gamma,
                                    const float* __restrict__ mean, const float* __restrict__ rstd,
                                    const float* __restrict__ sums, T* __restrict__ dx,
                                    T* __restrict__ dres, long long n, int C, long long M,
                                    int relu, int training) {
  const long long gs = (long long)gridDim.x * blockDim.x;
  const float invM = 1.f / (float)M;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gs) {
    const int c = (int)(i % C);
    float d = to_f32<T>(dy[i]);
    if (relu && to_f32<T>(y[i]) <= 0.f) d = 0.f;
    if (dres) dres[i] = from_f32<T>(d);
    const float g = to_f32<T>(gamma[c]) * rstd[c];
    float o;
    if (training) {
      const float xh = (to_f32<T>(x[i]) - mean[c]) * rstd[c];
      o = g * (d - sums[c] * invM - xh * sums[C + c] * invM);
    } else {
      o = g * d;
    }
    dx[i] = from_f32<T>(o);
  }
}

// ---------------------------------------------------------------------------------- pooling
template <typename T>
__global__ void maxpool_nhwc_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                        signed char* __restrict__ idx, int B, int H, int W, int C,
                                        int K, int stride, int pad, int Ho, int Wo) {
  const long long total = (long long)B * Ho * Wo * C;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int c = (int)(i % C);
    long long t = i / C;
    const int ow = (int)(t % Wo);
    t /= Wo;
    const int oh = (int)(t % Ho);
    const int b = (int)(t / Ho);
    float best = -INFINITY;
    int bi = -1;
    for (int kh = 0; kh < K; ++kh) {
      const int ih = oh * stride - pad + kh;
      if (ih < 0 || ih >= H) continue;
      for (int kw = 0; kw < K; ++kw) {
        const int iw = ow * stride - pad + kw;
        if (iw < 0 || iw >= W) continue;
        const float v = to_f32<T>(x[(((long long)b * H + ih) * W + iw) * C + c]);
        if (v > best || bi < 0) { best = v; bi = kh * K + kw; }
      }
    }
    y[i] = from_f32<T>(bi < 0 ? 0.f : best);
    idx[i] = (signed char)bi;
  }
}
// gather form: every input pixel collects dy from the windows whose argmax it is (no atomics)
template <typename T>
__global__ void maxpool_nhwc_bwd_kernel(const T* __restrict__ dy, const signed char* __restrict__ idx,
                                        T* __restrict__ dx, int B, int H, int W, int C, int K,
                                        int stride, int pad, int Ho, int Wo) {
  const long long total = (long long)B * H * W * C;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int c = (int)(i % C);
    long long t = i / C;
    const int iw = (int)(t % W);
    t /= W;
    const int ih = (int)(t % H);
    const int b = (int)(t / H);
    float acc = 0.f;
    for (int kh = 0; kh < K; ++kh) {
      const int nh = ih + pad - kh;
      if (nh < 0 || nh % stride) continue;
      const int oh = nh / stride;
      if (oh >= Ho) continue;
      for (int kw = 0; kw < K; ++kw) {
        const int nw = iw + pad - kw;
        if (nw < 0 || nw % stride) continue;
        const int ow = nw / stride;
        if (ow >= Wo) continue;
        const long long o = (((long long)b * Ho + oh) * Wo + ow) * C + c;
        if (idx[o] == kh * K + kw) acc += to_f32<T>(dy[o]);
      }
    }
    dx[i] = from_f32<T>(acc);
  }
}
// adaptive average pool, bins [floor(o*H/Ho), ceil((o+1)*H/Ho))
template <typename T, bool BWD>
__global__ void adaptive_avgpool_nhwc_kernel(const T* __restrict__ src, T* __restrict__ dst, int B,
                                             int H, int W, int C, int Ho, int Wo) {
  // forward: src = x [B,H,W,C], dst = y [B,Ho,Wo,C];  backward: src = dy [B,Ho,Wo,C], dst = dx
  const long long total = BWD ? (long long)B * H * W * C : (long long)B * Ho * Wo * C;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int c = (int)(i % C);
    long long t = i / C;
    if (!BWD) {
      const int ow = (int)(t % Wo);
      t /= Wo;
      const int oh = (int)(t % Ho);
      const int b = (int)(t / Ho);
      const int h0 = (oh * H) / Ho, h1 = ((oh + 1) * H + Ho - 1) / Ho;
      const int w0 = (ow * W) / Wo, w1 = ((ow + 1) * W + Wo - 1) / Wo;
      float acc = 0.f;
      for (int h = h0; h < h1; ++h)
        for (int w = w0; w < w1; ++w) acc += to_f32<T>(src[(((long long)b * H + h) * W + w) * C + c]);
      dst[i] = from_f32<T>(acc / (float)((h1 - h0) * (w1 - w0)));
    } else {
      const int w = (int)(t % W);
      t /= W;
      const int h = (int)(t % H);
      const int b = (int)(t / H);
      float acc = 0.f;
      for (int oh = 0; oh < Ho; ++oh) {
        const int h0 = (oh * H) / Ho, h1 = ((oh + 1) * H + Ho - 1) / Ho;
        if (h < h0 || h >= h1) continue;
        for (int ow = 0; ow < Wo; ++ow) {
          const int w0 = (ow * W) / Wo, w1 = ((ow + 1) * W + Wo - 1) / Wo;
          if (w < w0 || w >= w1) continue;
          acc += to_f32<T>(src[(((long long)b * Ho + oh) * Wo + ow) * C + c]) /
                 (float)((h1 - h0) * (w1 - w0));
        }
      }
      dst[i] = from_f32<T>(acc);
    }
  }
}

inline unsigned vgrid(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = (long long)rbh::sm_count() * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

}  // namespace rb

#define RB_DISPATCH_T(dtype, CALL)                                       \
  if ((dtype) == rbh::DT_BF16) { using T = __nv_bfloat16; CALL; }        \
  else if ((dtype) == rbh::DT_F16) { using T = __half; CALL; }           \
  else { using T = float; CALL; }
#define RB_RET_LAST()                                 \
  do {                                                \
    cudaError_t e__ = cudaGetLastError();             \
    return e__ == cudaSuccess ? 0 : 3000 + (int)e__;  \
  } while (0)

extern "C" {

int rb_im2col_nhwc(int dtype, const void* x, void* cols, int B, int H, int W, int C, int KH, int KW,
                   int Ho, int Wo, int stride, int pad, int dil, int Kpad, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = (long long)B * Ho * Wo * Kpad;
  if (n <= 0) return 0;
  RB_DISPATCH_T(dtype, (im2col_nhwc_kernel<T><<<vgrid(n), 256, 0, st>>>((const T*)x, (T*)cols, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil, Kpad)));
  RB_RET_LAST();
}
int rb_col2im_nhwc(int dtype, const void* dcols, void* dx, int B, int H, int W, int C, int KH, int KW,
                   int Ho, int Wo, int stride, int pad, int dil, int Kpad, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = (long long)B * H * W * C;
  if (n <= 0) return 0;
  RB_DISPATCH_T(dtype, (col2im_nhwc_kernel<T><<<vgrid(n), 256, 0, st>>>((const T*)dcols, (T*)dx, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil, Kpad)));
  RB_RET_LAST();
}
int rb_bn_slabs(long long M) {
  long long s = (M + 255) / 256;
  if (s > 2048) s = 2048;
  if (s < 1) s = 1;
  return (int)s;
}
// scratch: slabs*2*C floats.  mean/rstd: [C] fp32 out.  running_* may be null (eval mode handled by caller).
int rb_bn_fwd(int dtype, const void* x, const void* res, const void* gamma, const void* beta, void* y,
              float* mean, float* rstd, float* running_mean, float* running_var, float* scratch,
              long long M, int C, float eps, float momentum, int relu, int training, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  if (M <= 0) return 0;
  if (training) {
    const int slabs = rb_bn_slabs(M);
    const int rps = (int)((M + slabs - 1) / slabs);
    dim3 grid((C + 63) / 64, slabs);
    RB_DISPATCH_T(dtype, (bn_partial_kernel<T, false><<<grid, 64, 0, st>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, scratch, M, C, rps, 0)));
    bn_finalize_fwd_kernel<<<(C + 127) / 128, 128, 0, st>>>(scratch, slabs, C, M, eps, momentum, mean, rstd, running_mean, running_var);
  }
  RB_DISPATCH_T(dtype, (bn_apply_kernel<T><<<vgrid(M * C), 256, 0, st>>>((const T*)x, (const T*)res, (const T*)gamma, (const T*)beta, mean, rstd, (T*)y, M * C, C, relu)));
  RB_RET_LAST();
}
// sums: [2*C] fp32 scratch; scratch: slabs*2*C floats
int rb_bn_bwd(int dtype, const void* x, const void* dy, const void* y, const void* gamma,
              const float* mean, const float* rstd, void* dx, void* dres, void* dgamma, void* dbeta,
              float* sums, float* scratch, long long M, int C, int relu, int training, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  if (M <= 0) return 0;
  const int slabs = rb_bn_slabs(M);
  const int rps = (int)((M + slabs - 1) / slabs);
  dim3 grid((C + 63) / 64, slabs);
  RB_DISPATCH_T(dtype, (bn_partial_kernel<T, true><<<grid, 64, 0, st>>>((const T*)x, (const T*)dy, (const T*)y, mean, rstd, scratch, M, C, rps, relu)));
  RB_DISPATCH_T(dtype, (bn_finalize_bwd_kernel<T><<<(C + 127) / 128, 128, 0, st>>>(scratch, slabs, C, sums, (T*)dgamma, (T*)dbeta)));
  RB_DISPATCH_T(dtype, (bn_bwd_apply_kernel<T><<<vgrid(M * C), 256, 0, st>>>((const T*)x, (const T*)dy, (const T*)y, (const T*)gamma, mean, rstd, sums, (T*)dx, (T*)dres, M * C, C, M, relu, training)));
  RB_RET_LAST();
}
int rb_maxpool_fwd(int dtype, const void* x, void* y, signed char* idx, int B, int H, int W, int C,
                   int K, int stride, int pad, int Ho, int Wo, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = (long long)B * Ho * Wo * C;
  if (n <= 0) return 0;
  RB_DISPATCH_T(dtype, (maxpool_nhwc_fwd_kernel<T><<<vgrid(n), 256, 0, st>>>((const T*)x, (T*)y, idx, B, H, W, C, K, stride, pad, Ho, Wo)));
  RB_RET_LAST();
}
int rb_maxpool_bwd(int dtype, const void* dy, const signed char* idx, void* dx, int B, int H, int W,
                   int C, int K, int stride, int pad, int Ho, int Wo, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = (long long)B * H * W * C;
  if (n <= 0) return 0;
  RB_DISPATCH_T(dtype, (maxpool_nhwc_bwd_kernel<T><<<vgrid(n), 256, 0, st>>>((const T*)dy, idx, (T*)dx, B, H, W, C, K, stride, pad, Ho, Wo)));
  RB_RET_LAST();
}
int rb_adaptive_avgpool(int dtype, int backward, const void* src, void* dst, int B, int H, int W,
                        int C, int Ho, int Wo, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = backward ? (long long)B * H * W * C : (long long)B * Ho * Wo * C;
  if (n <= 0) return 0;
  if (backward) {
    RB_DISPATCH_T(dtype, (adaptive_avgpool_nhwc_kernel<T, true><<<vgrid(n), 256, 0, st>>>((const T*)src, (T*)dst, B, H, W, C, Ho, Wo)));
  } else {
    RB_DISPATCH_T(dtype, (adaptive_avgpool_nhwc_kernel<T, false><<<vgrid(n), 256, 0, st>>>((const T*)src, (T*)dst, B, H, W, C, Ho, Wo)));
  }
  RB_RET_LAST();
}
}
