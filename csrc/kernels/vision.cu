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

// 16-byte forms for 16-bit types with C % 8 == 0 and Kpad == KH*KW*C: one thread moves 8 channels.
template <typename T>
__global__ void im2col_nhwc_vec8_kernel(const T* __restrict__ x, T* __restrict__ cols, int B, int H,
                                        int W, int C, int KH, int KW, int Ho, int Wo, int stride,
                                        int pad, int dil) {
  const int C8 = C >> 3;
  const int K8 = KH * KW * C8;                       // 16-byte chunks per cols row
  const long long total = (long long)B * Ho * Wo * K8;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int k8 = (int)(i % K8);
    const long long m = i / K8;
    const int c8 = k8 % C8;
    const int kk = k8 / C8;
    const int kw = kk % KW, kh = kk / KW;
    const int ow = (int)(m % Wo);
    const long long t = m / Wo;
    const int oh = (int)(t % Ho);
    const int b = (int)(t / Ho);
    const int ih = oh * stride - pad + kh * dil;
    const int iw = ow * stride - pad + kw * dil;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ih >= 0 && ih < H && iw >= 0 && iw < W)
      v = *reinterpret_cast<const uint4*>(x + (((long long)b * H + ih) * W + iw) * C + c8 * 8);
    reinterpret_cast<uint4*>(cols)[i] = v;
  }
}

template <typename T>
__global__ void col2im_nhwc_vec8_kernel(const T* __restrict__ dcols, T* __restrict__ dx, int B, int H,
                                        int W, int C, int KH, int KW, int Ho, int Wo, int stride,
                                        int pad, int dil) {
  const int C8 = C >> 3;
  const long long Kdim = (long long)KH * KW * C;
  const long long total = (long long)B * H * W * C8;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int c8 = (int)(i % C8);
    long long t = i / C8;
    const int iw = (int)(t % W);
    t /= W;
    const int ih = (int)(t % H);
    const int b = (int)(t / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
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
        const uint4 v = *reinterpret_cast<const uint4*>(dcols + m * Kdim + (kh * KW + kw) * C + c8 * 8);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += to_f32<T>(e[j]);
      }
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = from_f32<T>(acc[j]);
    reinterpret_cast<uint4*>(dx)[i] = o;
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

// ------------------------------------------------------------------ batch norm, 16-byte forms
// For 16-bit types with C % 8 == 0 and a power-of-two number of 8-channel groups (every ResNet
// layer): one thread owns 8 consecutive channels and moves them with one 16-byte access.
template <typename T>
__device__ __forceinline__ void unpack8f(const uint4& v, float* f) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = to_f32<T>(e[j]);
}
template <typename T>
__device__ __forceinline__ uint4 pack8f(const float* f) {
  uint4 v;
  T* e = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(f[j]);
  return v;
}

// 256 threads = cgb channel groups x (256 / cgb) row lanes; partial sums per slab as in
// bn_partial_kernel.  cgb = min(C / 8, 32).
template <typename T, bool BWD>
__global__ void __launch_bounds__(256)
    bn_partial_vec8_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                           const T* __restrict__ y, const float* __restrict__ mean,
                           const float* __restrict__ rstd, float* __restrict__ partials,
                           long long M, int C, int rows_per_slab, int relu, int cgb) {
  __shared__ float s_acc[256][17];
  const int tx = threadIdx.x % cgb, ty = threadIdx.x / cgb;
  const int lanes = 256 / cgb;
  const int c0 = (blockIdx.x * cgb + tx) * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_slab;
  const long long r1 = min(M, r0 + rows_per_slab);
  float a[8], b[8], mu[8], rs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    a[j] = b[j] = 0.f;
    mu[j] = BWD ? mean[c0 + j] : 0.f;
    rs[j] = BWD ? rstd[c0 + j] : 1.f;
  }
  // four rows in flight per thread: the loads of a batch are issued before any of them is used
  auto fold = [&](const uint4& xq, const uint4& dq, const uint4& yq) {
    float xv[8];
    unpack8f<T>(xq, xv);
    if (!BWD) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] += xv[j];
        b[j] += xv[j] * xv[j];
      }
    } else {
      float d[8];
      unpack8f<T>(dq, d);
      if (relu) {
        float yv[8];
        unpack8f<T>(yq, yv);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (yv[j] <= 0.f) d[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] += d[j];
        b[j] += d[j] * (xv[j] - mu[j]) * rs[j];
      }
    }
  };
  long long r = r0 + ty;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  for (; r + 3ll * lanes < r1; r += 4ll * lanes) {
    uint4 xq[4], dq[4], yq[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long o = (r + (long long)u * lanes) * C + c0;
      xq[u] = *reinterpret_cast<const uint4*>(x + o);
      dq[u] = BWD ? *reinterpret_cast<const uint4*>(dy + o) : zero4;
      yq[u] = (BWD && relu) ? *reinterpret_cast<const uint4*>(y + o) : zero4;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) fold(xq[u], dq[u], yq[u]);
  }
  for (; r < r1; r += lanes) {
    const long long o = r * C + c0;
    const uint4 xq = *reinterpret_cast<const uint4*>(x + o);
    const uint4 dq = BWD ? *reinterpret_cast<const uint4*>(dy + o) : zero4;
    const uint4 yq = (BWD && relu) ? *reinterpret_cast<const uint4*>(y + o) : zero4;
    fold(xq, dq, yq);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    s_acc[threadIdx.x][j] = a[j];
    s_acc[threadIdx.x][8 + j] = b[j];
  }
  __syncthreads();
  if (ty == 0) {
    for (int l = 1; l < lanes; ++l)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a[j] += s_acc[l * cgb + tx][j];
        b[j] += s_acc[l * cgb + tx][8 + j];
      }
    float* pa = partials + ((long long)blockIdx.y * 2) * C + c0;
    float* pb = partials + ((long long)blockIdx.y * 2 + 1) * C + c0;
    *reinterpret_cast<float4*>(pa) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(pa + 4) = make_float4(a[4], a[5], a[6], a[7]);
    *reinterpret_cast<float4*>(pb) = make_float4(b[0], b[1], b[2], b[3]);
    *reinterpret_cast<float4*>(pb + 4) = make_float4(b[4], b[5], b[6], b[7]);
  }
}

// Sums the slab partials of 32 channels with 8 slab slices per CTA; out2[0][c], out2[1][c] (smem)
__device__ __forceinline__ void bn_fold_partials(const float* __restrict__ partials, int slabs,
                                                 int C, int c, int slice, int cx, float& s,
                                                 float& q, float (*ss)[33], float (*sq)[33]) {
  s = 0.f;
  q = 0.f;
  if (c < C)
    for (int i = slice; i < slabs; i += 8) {
      s += partials[((long long)i * 2) * C + c];
      q += partials[((long long)i * 2 + 1) * C + c];
    }
  ss[slice][cx] = s;
  sq[slice][cx] = q;
  __syncthreads();
  if (slice == 0) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      s += ss[k][cx];
      q += sq[k][cx];
    }
  }
}

__global__ void __launch_bounds__(256)
    bn_finalize_fwd_par_kernel(const float* __restrict__ partials, int slabs, int C, long long M,
                               float eps, float momentum, float* __restrict__ mean,
                               float* __restrict__ rstd, float* __restrict__ running_mean,
                               float* __restrict__ running_var) {
  __shared__ float ss[8][33], sq[8][33];
  const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s, q;
  bn_fold_partials(partials, slabs, C, c, slice, cx, s, q, ss, sq);
  if (slice != 0 || c >= C) return;
  const float mu = s / (float)M;
  const float var = fmaxf(q / (float)M - mu * mu, 0.f);
  mean[c] = mu;
  rstd[c] = rsqrtf(var + eps);
  if (running_mean) {
    running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mu;
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * var;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
    bn_finalize_bwd_par_kernel(const float* __restrict__ partials, int slabs, int C,
                               float* __restrict__ sums, T* __restrict__ dgamma,
                               T* __restrict__ dbeta) {
  __shared__ float ss[8][33], sq[8][33];
  const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s, q;
  bn_fold_partials(partials, slabs, C, c, slice, cx, s, q, ss, sq);
  if (slice != 0 || c >= C) return;
  sums[c] = s;
  sums[C + c] = q;
  dbeta[c] = from_f32<T>(s);
  dgamma[c] = from_f32<T>(q);
}

// Per-channel coefficients live in registers: the grid stride is a multiple of the number of
// 8-channel groups (a power of two, at most 512; the launcher keeps gridDim.x even), so a thread
// meets the same 8 channels on every iteration and computes their coefficients once.  Reading
// mean / rstd / gamma / beta per element cost 16 scattered 4-byte loads per 8 channels and made
// these kernels L1-bound at ~1.8 TB/s; the 64-bit `i % groups` per element and a single 16-byte
// load in flight per thread held the second version near half of the copy bandwidth.
//   forward:  y = relu(x * a + b + res),  a = rstd * gamma,  b = beta - mean * a
__device__ __forceinline__ void load8f(const float* p, float* f) {
  const float4 v0 = *reinterpret_cast<const float4*>(p), v1 = *reinterpret_cast<const float4*>(p + 4);
  f[0] = v0.x; f[1] = v0.y; f[2] = v0.z; f[3] = v0.w;
  f[4] = v1.x; f[5] = v1.y; f[6] = v1.z; f[7] = v1.w;
}

template <typename T>
__global__ void __launch_bounds__(256, 4)
    bn_apply_vec8_kernel(const T* __restrict__ x, const T* __restrict__ res,
                         const T* __restrict__ gamma, const T* __restrict__ beta,
                         const float* __restrict__ mean, const float* __restrict__ rstd,
                         T* __restrict__ y, long long n8, int C, int relu) {
  const int CG = C >> 3;
  const long long gs = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int c0 = (int)(i0 & (CG - 1)) * 8;
  float av[8], bv[8];
  {
    float mu[8], g[8], be[8];
    load8f(rstd + c0, av);
    load8f(mean + c0, mu);
    unpack8f<T>(*reinterpret_cast<const uint4*>(gamma + c0), g);
    unpack8f<T>(*reinterpret_cast<const uint4*>(beta + c0), be);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      av[j] *= g[j];
      bv[j] = be[j] - mu[j] * av[j];
    }
  }
  const uint4* x4 = reinterpret_cast<const uint4*>(x);
  const uint4* r4 = reinterpret_cast<const uint4*>(res);
  uint4* y4 = reinterpret_cast<uint4*>(y);
  auto one = [&](const uint4& xq, const uint4& rq) {
    float xv[8], rv[8];
    unpack8f<T>(xq, xv);
    if (res) unpack8f<T>(rq, rv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = fmaf(xv[j], av[j], bv[j]);
      if (res) v += rv[j];
      if (relu) v = fmaxf(v, 0.f);
      xv[j] = v;
    }
    return pack8f<T>(xv);
  };
  long long i = i0;
  for (; i + 3 * gs < n8; i += 4 * gs) {
    uint4 xq[4], rq[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xq[u] = x4[i + u * gs];
      rq[u] = res ? r4[i + u * gs] : xq[u];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) y4[i + u * gs] = one(xq[u], rq[u]);
  }
  for (; i < n8; i += gs) {
    const uint4 xq = x4[i];
    const uint4 rq = res ? r4[i] : xq;
    y4[i] = one(xq, rq);
  }
}

//   backward: dx = A * d + Bc * x + Cc with d = dy masked by the ReLU, and (training)
//   A = gamma*rstd, Bc = -A*rstd*S2/M, Cc = -A*S1/M - Bc*mean;  (eval) Bc = Cc = 0
template <typename T>
__global__ void __launch_bounds__(256, 4)
    bn_bwd_apply_vec8_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                             const T* __restrict__ y, const T* __restrict__ gamma,
                             const float* __restrict__ mean, const float* __restrict__ rstd,
                             const float* __restrict__ sums, T* __restrict__ dx,
                             T* __restrict__ dres, long long n8, int C, long long M, int relu,
                             int training) {
  const int CG = C >> 3;
  const long long gs = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int c0 = (int)(i0 & (CG - 1)) * 8;
  float Av[8], Bv[8], Cv[8];
  {
    const float invM = 1.f / (float)M;
    float rs[8], mu[8], g[8], s1[8], s2[8];
    load8f(rstd + c0, rs);
    load8f(mean + c0, mu);
    unpack8f<T>(*reinterpret_cast<const uint4*>(gamma + c0), g);
    if (training) {
      load8f(sums + c0, s1);
      load8f(sums + C + c0, s2);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      Av[j] = g[j] * rs[j];
      Bv[j] = Cv[j] = 0.f;
      if (training) {
        Bv[j] = -Av[j] * rs[j] * s2[j] * invM;
        Cv[j] = -Av[j] * s1[j] * invM - Bv[j] * mu[j];
      }
    }
  }
  const uint4* x4 = reinterpret_cast<const uint4*>(x);
  const uint4* d4 = reinterpret_cast<const uint4*>(dy);
  const uint4* y4 = reinterpret_cast<const uint4*>(y);
  uint4* o4 = reinterpret_cast<uint4*>(dx);
  uint4* dr4 = reinterpret_cast<uint4*>(dres);
  auto one = [&](long long at, const uint4& dq, const uint4& yq, const uint4& xq) {
    float d[8], o[8];
    unpack8f<T>(dq, d);
    if (relu) {
      float yv[8];
      unpack8f<T>(yq, yv);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (yv[j] <= 0.f) d[j] = 0.f;
    }
    if (dres) dr4[at] = pack8f<T>(d);
    if (training) {
      float xv[8];
      unpack8f<T>(xq, xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = fmaf(Av[j], d[j], fmaf(Bv[j], xv[j], Cv[j]));
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = Av[j] * d[j];
    }
    o4[at] = pack8f<T>(o);
  };
  long long i = i0;
  for (; i + gs < n8; i += 2 * gs) {
    uint4 dq[2], yq[2], xq[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      dq[u] = d4[i + u * gs];
      yq[u] = relu ? y4[i + u * gs] : dq[u];
      xq[u] = training ? x4[i + u * gs] : dq[u];
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) one(i + u * gs, dq[u], yq[u], xq[u]);
  }
  for (; i < n8; i += gs) {
    const uint4 dq = d4[i];
    const uint4 yq = relu ? y4[i] : dq;
    const uint4 xq = training ? x4[i] : dq;
    one(i, dq, yq, xq);
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
// the same gather, eight channels (16 bytes of dy, 8 bytes of argmax codes) per thread
template <typename T>
__global__ void maxpool_nhwc_bwd_vec8_kernel(const T* __restrict__ dy, const signed char* __restrict__ idx,
                                             T* __restrict__ dx, int B, int H, int W, int C, int K,
                                             int stride, int pad, int Ho, int Wo) {
  const int C8 = C / 8;
  const long long total = (long long)B * H * W * C8;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int c8 = (int)(i % C8);
    long long t = i / C8;
    const int iw = (int)(t % W);
    t /= W;
    const int ih = (int)(t % H);
    const int b = (int)(t / H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
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
        const long long o = (((long long)b * Ho + oh) * Wo + ow) * C + c8 * 8;
        const uint2 codes = *reinterpret_cast<const uint2*>(idx + o);
        const uint4 g = *reinterpret_cast<const uint4*>(dy + o);
        const signed char* cd = reinterpret_cast<const signed char*>(&codes);
        const T* ge = reinterpret_cast<const T*>(&g);
        const int want = kh * K + kw;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (cd[j] == want) acc[j] += to_f32<T>(ge[j]);
      }
    }
    uint4 out;
    T* oe = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = from_f32<T>(acc[j]);
    *reinterpret_cast<uint4*>(dx + i * 8) = out;
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
#define RB_DISPATCH_16(dtype, CALL)                            \
  if ((dtype) == rbh::DT_BF16) { using T = __nv_bfloat16; CALL; } \
  else { using T = __half; CALL; }
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
  const bool a16 = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cols)) & 15) == 0;
  if (dtype != rbh::DT_F32 && C % 8 == 0 && Kpad == KH * KW * C && a16) {
    const long long n8 = n / 8;
    if (dtype == rbh::DT_BF16)
      im2col_nhwc_vec8_kernel<__nv_bfloat16><<<vgrid(n8), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)cols, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil);
    else
      im2col_nhwc_vec8_kernel<__half><<<vgrid(n8), 256, 0, st>>>((const __half*)x, (__half*)cols, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil);
    RB_RET_LAST();
  }
  RB_DISPATCH_T(dtype, (im2col_nhwc_kernel<T><<<vgrid(n), 256, 0, st>>>((const T*)x, (T*)cols, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil, Kpad)));
  RB_RET_LAST();
}
int rb_col2im_nhwc(int dtype, const void* dcols, void* dx, int B, int H, int W, int C, int KH, int KW,
                   int Ho, int Wo, int stride, int pad, int dil, int Kpad, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = (long long)B * H * W * C;
  if (n <= 0) return 0;
  const bool a16 = ((reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dcols)) & 15) == 0;
  if (dtype != rbh::DT_F32 && C % 8 == 0 && Kpad == KH * KW * C && a16) {
    const long long n8 = n / 8;
    if (dtype == rbh::DT_BF16)
      col2im_nhwc_vec8_kernel<__nv_bfloat16><<<vgrid(n8), 256, 0, st>>>((const __nv_bfloat16*)dcols, (__nv_bfloat16*)dx, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil);
    else
      col2im_nhwc_vec8_kernel<__half><<<vgrid(n8), 256, 0, st>>>((const __half*)dcols, (__half*)dx, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil);
    RB_RET_LAST();
  }
  RB_DISPATCH_T(dtype, (col2im_nhwc_kernel<T><<<vgrid(n), 256, 0, st>>>((const T*)dcols, (T*)dx, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil, Kpad)));
  RB_RET_LAST();
}
// Grid of the 16-byte batch-norm apply kernels: an even number of 256-thread CTAs (so the grid
// stride is a multiple of 512 channel groups), at most the four per SM that are resident.
static unsigned bn_grid(long long n8) {
  long long b = (n8 + 255) / 256;
  const long long cap = (long long)rbh::sm_count() * 4;
  if (b > cap) b = cap;
  b = (b + 1) & ~1ll;
  return (unsigned)b;
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
  const int cg = C / 8;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec8 = dtype != rbh::DT_F32 && C % 8 == 0 && C <= 4096 && (cg & (cg - 1)) == 0 && al16(x) &&
                    al16(res) && al16(gamma) && al16(beta) && al16(y) && al16(mean) && al16(rstd);
  const int cgb = cg < 32 ? cg : 32;
  if (training) {
    const int slabs = rb_bn_slabs(M);
    const int rps = (int)((M + slabs - 1) / slabs);
    if (vec8) {
      dim3 grid(cg / cgb, slabs);
      RB_DISPATCH_16(dtype, (bn_partial_vec8_kernel<T, false><<<grid, 256, 0, st>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, scratch, M, C, rps, 0, cgb)));
      bn_finalize_fwd_par_kernel<<<(C + 31) / 32, 256, 0, st>>>(scratch, slabs, C, M, eps, momentum, mean, rstd, running_mean, running_var);
    } else {
      dim3 grid((C + 63) / 64, slabs);
      RB_DISPATCH_T(dtype, (bn_partial_kernel<T, false><<<grid, 64, 0, st>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, scratch, M, C, rps, 0)));
      bn_finalize_fwd_kernel<<<(C + 127) / 128, 128, 0, st>>>(scratch, slabs, C, M, eps, momentum, mean, rstd, running_mean, running_var);
    }
  }
  if (vec8) {
    RB_DISPATCH_16(dtype, (bn_apply_vec8_kernel<T><<<bn_grid(M * cg), 256, 0, st>>>((const T*)x, (const T*)res, (const T*)gamma, (const T*)beta, mean, rstd, (T*)y, M * cg, C, relu)));
  } else {
    RB_DISPATCH_T(dtype, (bn_apply_kernel<T><<<vgrid(M * C), 256, 0, st>>>((const T*)x, (const T*)res, (const T*)gamma, (const T*)beta, mean, rstd, (T*)y, M * C, C, relu)));
  }
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
  const int cg = C / 8;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec8 = dtype != rbh::DT_F32 && C % 8 == 0 && C <= 4096 && (cg & (cg - 1)) == 0 && al16(x) &&
                    al16(dy) && al16(y) && al16(gamma) && al16(dx) && al16(dres) && al16(mean) && al16(rstd) &&
                    al16(sums);
  if (vec8) {
    const int cgb = cg < 32 ? cg : 32;
    dim3 grid(cg / cgb, slabs);
    RB_DISPATCH_16(dtype, (bn_partial_vec8_kernel<T, true><<<grid, 256, 0, st>>>((const T*)x, (const T*)dy, (const T*)y, mean, rstd, scratch, M, C, rps, relu, cgb)));
    RB_DISPATCH_16(dtype, (bn_finalize_bwd_par_kernel<T><<<(C + 31) / 32, 256, 0, st>>>(scratch, slabs, C, sums, (T*)dgamma, (T*)dbeta)));
    RB_DISPATCH_16(dtype, (bn_bwd_apply_vec8_kernel<T><<<bn_grid(M * cg), 256, 0, st>>>((const T*)x, (const T*)dy, (const T*)y, (const T*)gamma, mean, rstd, sums, (T*)dx, (T*)dres, M * cg, C, M, relu, training)));
    RB_RET_LAST();
  }
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
  const bool vec8 = dtype != rbh::DT_F32 && C % 8 == 0 &&
                    ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(idx) & 7) == 0;
  if (vec8) {
    if (dtype == rbh::DT_BF16)
      maxpool_nhwc_bwd_vec8_kernel<__nv_bfloat16><<<vgrid(n / 8), 256, 0, st>>>((const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, B, H, W, C, K, stride, pad, Ho, Wo);
    else
      maxpool_nhwc_bwd_vec8_kernel<__half><<<vgrid(n / 8), 256, 0, st>>>((const __half*)dy, idx, (__half*)dx, B, H, W, C, K, stride, pad, Ho, Wo);
    RB_RET_LAST();
  }
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
