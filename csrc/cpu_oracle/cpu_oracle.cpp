// Scalar fp32 CPU oracle: plain-loop restatement of the reference's CPU backend
// (rumus/src/backend/mod.rs:24-219 — the `Backend` trait — and the math of the shaders that have
// no CPU path there: flash attention, INT8/INT4 matmuls, direct convolution, SpMM).  Every GPU
// kernel in this tree is tested against PyTorch fp32; this library is the independent second
// opinion and the timed CPU baseline.  Contiguous row-major float buffers, C ABI.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

void orc_add(const float* a, const float* b, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = a[i] + b[i]; }
void orc_sub(const float* a, const float* b, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = a[i] - b[i]; }
void orc_mul(const float* a, const float* b, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = a[i] * b[i]; }
void orc_scale(const float* a, float s, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = a[i] * s; }
void orc_relu(const float* a, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = a[i] > 0.f ? a[i] : 0.f; }
void orc_relu_backward(const float* x, const float* g, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = x[i] > 0.f ? g[i] : 0.f; }
void orc_sigmoid(const float* a, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = 1.f / (1.f + std::exp(-a[i])); }
void orc_tanh(const float* a, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = std::tanh(a[i]); }
void orc_gelu(const float* a, float* o, long long n) {
  for (long long i = 0; i < n; ++i) {
    const float x = a[i];
    o[i] = 0.5f * x * (1.f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x)));
  }
}
void orc_leaky_relu(const float* a, float slope, float* o, long long n) { for (long long i = 0; i < n; ++i) o[i] = a[i] > 0.f ? a[i] : slope * a[i]; }

// C[m,n] = A[m,k] . B[k,n]   (i-k-j loop order)
void orc_matmul(const float* A, const float* B, float* C, int m, int k, int n) {
  std::fill(C, C + (long long)m * n, 0.f);
  for (int i = 0; i < m; ++i)
    for (int p = 0; p < k; ++p) {
      const float a = A[(long long)i * k + p];
      const float* b = B + (long long)p * n;
      float* c = C + (long long)i * n;
      for (int j = 0; j < n; ++j) c[j] += a * b[j];
    }
}
void orc_bmm(const float* A, const float* B, float* C, int batch, int m, int k, int n) {
  for (int b = 0; b < batch; ++b)
    orc_matmul(A + (long long)b * m * k, B + (long long)b * k * n, C + (long long)b * m * n, m, k, n);
}
void orc_add_bias(const float* x, const float* bias, float* o, int m, int n) {
  for (int i = 0; i < m; ++i) for (int j = 0; j < n; ++j) o[(long long)i * n + j] = x[(long long)i * n + j] + bias[j];
}
void orc_sum_rows(const float* x, float* o, int m, int n) {
  std::fill(o, o + n, 0.f);
  for (int i = 0; i < m; ++i) for (int j = 0; j < n; ++j) o[j] += x[(long long)i * n + j];
}
void orc_softmax(const float* x, float* o, int rows, int n) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (long long)r * n; float* orow = o + (long long)r * n;
    float mx = xr[0]; for (int j = 1; j < n; ++j) mx = std::max(mx, xr[j]);
    float s = 0.f; for (int j = 0; j < n; ++j) { orow[j] = std::exp(xr[j] - mx); s += orow[j]; }
    for (int j = 0; j < n; ++j) orow[j] /= s;
  }
}
void orc_softmax_backward(const float* y, const float* dy, float* dx, int rows, int n) {
  for (int r = 0; r < rows; ++r) {
    const float* yr = y + (long long)r * n; const float* dr = dy + (long long)r * n;
    float dot = 0.f; for (int j = 0; j < n; ++j) dot += yr[j] * dr[j];
    for (int j = 0; j < n; ++j) dx[(long long)r * n + j] = yr[j] * (dr[j] - dot);
  }
}
// save: [rows, 2] = (mean, invstd)
void orc_layer_norm(const float* x, const float* w, const float* b, float* o, float* save, int rows, int d, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (long long)r * d;
    float mean = 0.f; for (int j = 0; j < d; ++j) mean += xr[j]; mean /= d;
    float var = 0.f; for (int j = 0; j < d; ++j) { const float t = xr[j] - mean; var += t * t; } var /= d;
    const float inv = 1.f / std::sqrt(var + eps);
    if (save) { save[r * 2] = mean; save[r * 2 + 1] = inv; }
    for (int j = 0; j < d; ++j) o[(long long)r * d + j] = (xr[j] - mean) * inv * w[j] + b[j];
  }
}
void orc_layer_norm_backward(const float* x, const float* w, const float* dy, const float* save, float* dx,
                             float* dw, float* db, int rows, int d) {
  std::fill(dw, dw + d, 0.f); std::fill(db, db + d, 0.f);
  for (int r = 0; r < rows; ++r) {
    const float mean = save[r * 2], inv = save[r * 2 + 1];
    const float* xr = x + (long long)r * d; const float* dr = dy + (long long)r * d;
    float c1 = 0.f, c2 = 0.f;
    for (int j = 0; j < d; ++j) { const float xh = (xr[j] - mean) * inv; const float g = dr[j] * w[j]; c1 += g; c2 += g * xh; dw[j] += dr[j] * xh; db[j] += dr[j]; }
    c1 /= d; c2 /= d;
    for (int j = 0; j < d; ++j) { const float xh = (xr[j] - mean) * inv; dx[(long long)r * d + j] = inv * (dr[j] * w[j] - c1 - xh * c2); }
  }
}
void orc_embedding(const long long* idx, const float* w, float* o, long long tokens, int d) {
  for (long long t = 0; t < tokens; ++t) std::memcpy(o + t * d, w + idx[t] * d, sizeof(float) * d);
}
void orc_embedding_backward(const long long* idx, const float* dy, float* dw, long long tokens, int d, int vocab) {
  std::fill(dw, dw + (long long)vocab * d, 0.f);
  for (long long t = 0; t < tokens; ++t) for (int j = 0; j < d; ++j) dw[idx[t] * d + j] += dy[t * d + j];
}
// loss = mean_r (lse - x[r, t[r]]); grad = (softmax - onehot) / rows
float orc_cross_entropy(const float* x, const long long* tgt, float* grad, int rows, int n) {
  double total = 0.0;
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (long long)r * n;
    float mx = xr[0]; for (int j = 1; j < n; ++j) mx = std::max(mx, xr[j]);
    double s = 0.0; for (int j = 0; j < n; ++j) s += std::exp((double)xr[j] - mx);
    total += (mx + std::log(s)) - xr[tgt[r]];
    if (grad) for (int j = 0; j < n; ++j) grad[(long long)r * n + j] = (float)((std::exp((double)xr[j] - mx) / s - (j == tgt[r] ? 1.0 : 0.0)) / rows);
  }
  return (float)(total / rows);
}
// x [C,H,W] -> cols [C*k*k, Ho*Wo]
void orc_im2col(const float* x, float* cols, int C, int H, int W, int k, int stride, int pad) {
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  for (int c = 0; c < C; ++c) for (int kh = 0; kh < k; ++kh) for (int kw = 0; kw < k; ++kw) {
    const int row = (c * k + kh) * k + kw;
    for (int oh = 0; oh < Ho; ++oh) for (int ow = 0; ow < Wo; ++ow) {
      const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
      cols[(long long)row * Ho * Wo + oh * Wo + ow] = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? x[((long long)c * H + ih) * W + iw] : 0.f;
    }
  }
}
void orc_col2im(const float* cols, float* x, int C, int H, int W, int k, int stride, int pad) {
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  std::fill(x, x + (long long)C * H * W, 0.f);
  for (int c = 0; c < C; ++c) for (int kh = 0; kh < k; ++kh) for (int kw = 0; kw < k; ++kw) {
    const int row = (c * k + kh) * k + kw;
    for (int oh = 0; oh < Ho; ++oh) for (int ow = 0; ow < Wo; ++ow) {
      const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
      if (ih >= 0 && ih < H && iw >= 0 && iw < W) x[((long long)c * H + ih) * W + iw] += cols[(long long)row * Ho * Wo + oh * Wo + ow];
    }
  }
}
// direct convolution, NCHW, weight [Co,Ci,Kh,Kw] (rumus-vision conv2d_direct.wgsl math)
void orc_conv2d(const float* x, const float* w, const float* bias, float* y, int B, int Ci, int H, int W, int Co,
                int Kh, int Kw, int stride, int pad, int dil) {
  const int Ho = (H + 2 * pad - dil * (Kh - 1) - 1) / stride + 1, Wo = (W + 2 * pad - dil * (Kw - 1) - 1) / stride + 1;
  for (int b = 0; b < B; ++b) for (int co = 0; co < Co; ++co) for (int oh = 0; oh < Ho; ++oh) for (int ow = 0; ow < Wo; ++ow) {
    float acc = bias ? bias[co] : 0.f;
    for (int ci = 0; ci < Ci; ++ci) for (int kh = 0; kh < Kh; ++kh) for (int kw = 0; kw < Kw; ++kw) {
      const int ih = oh * stride - pad + kh * dil, iw = ow * stride - pad + kw * dil;
      if (ih >= 0 && ih < H && iw >= 0 && iw < W)
        acc += x[(((long long)b * Ci + ci) * H + ih) * W + iw] * w[(((long long)co * Ci + ci) * Kh + kh) * Kw + kw];
    }
    y[(((long long)b * Co + co) * Ho + oh) * Wo + ow] = acc;
  }
}
void orc_max_pool2d(const float* x, float* y, int* arg, int C, int H, int W, int k, int stride) {
  const int Ho = (H - k) / stride + 1, Wo = (W - k) / stride + 1;
  for (int c = 0; c < C; ++c) for (int oh = 0; oh < Ho; ++oh) for (int ow = 0; ow < Wo; ++ow) {
    float best = -INFINITY; int bi = 0;
    for (int kh = 0; kh < k; ++kh) for (int kw = 0; kw < k; ++kw) {
      const int idx = (c * H + oh * stride + kh) * W + ow * stride + kw;
      if (x[idx] > best) { best = x[idx]; bi = idx; }
    }
    y[(c * Ho + oh) * Wo + ow] = best; if (arg) arg[(c * Ho + oh) * Wo + ow] = bi;
  }
}
// batch norm over (B,H,W); save [C,2] = (mean, invstd); running stats use the biased variance
void orc_batch_norm(const float* x, const float* w, const float* b, float* rm, float* rv, float* y, float* save,
                    int B, int C, int H, int W, float eps, float momentum, int training) {
  const int sp = H * W; const long long n = (long long)B * sp;
  for (int c = 0; c < C; ++c) {
    float mean, var;
    if (training) {
      double s = 0; for (int bb = 0; bb < B; ++bb) for (int i = 0; i < sp; ++i) s += x[((long long)bb * C + c) * sp + i];
      mean = (float)(s / n);
      double q = 0; for (int bb = 0; bb < B; ++bb) for (int i = 0; i < sp; ++i) { const double d = x[((long long)bb * C + c) * sp + i] - mean; q += d * d; }
      var = (float)(q / n);
      if (save) { save[c * 2] = mean; save[c * 2 + 1] = 1.f / std::sqrt(var + eps); }
      rm[c] = (1.f - momentum) * rm[c] + momentum * mean; rv[c] = (1.f - momentum) * rv[c] + momentum * var;
    } else { mean = rm[c]; var = rv[c]; }
    const float inv = 1.f / std::sqrt(var + eps);
    for (int bb = 0; bb < B; ++bb) for (int i = 0; i < sp; ++i) { const long long f = ((long long)bb * C + c) * sp + i; y[f] = w[c] * (x[f] - mean) * inv + b[c]; }
  }
}
void orc_adaptive_avg_pool2d(const float* x, float* y, int C, int H, int W, int Ho, int Wo) {
  for (int c = 0; c < C; ++c) for (int oh = 0; oh < Ho; ++oh) for (int ow = 0; ow < Wo; ++ow) {
    const int h0 = oh * H / Ho, h1 = ((oh + 1) * H + Ho - 1) / Ho, w0 = ow * W / Wo, w1 = ((ow + 1) * W + Wo - 1) / Wo;
    float acc = 0.f; for (int h = h0; h < h1; ++h) for (int w = w0; w < w1; ++w) acc += x[(c * H + h) * W + w];
    y[(c * Ho + oh) * Wo + ow] = acc / ((h1 - h0) * (w1 - w0));
  }
}
// PCG-hash dropout (device variant: keep when hash >= p * 2^32)
static uint32_t pcg(uint32_t v) { uint32_t s = v * 747796405u + 2891336453u; uint32_t w = ((s >> ((s >> 28u) + 4u)) ^ s) * 277803737u; return (w >> 22u) ^ w; }
void orc_dropout(const float* x, float* y, long long n, uint32_t seed, float p) {
  const double thr = (double)p * 4294967296.0; const float sc = p < 1.f ? 1.f / (1.f - p) : 0.f;
  for (long long i = 0; i < n; ++i) y[i] = ((double)pcg(seed ^ (uint32_t)i) >= thr) ? x[i] * sc : 0.f;
}
// online-softmax attention on [BH, N, d] (flash_attn.wgsl math), causal optional
void orc_flash_attention(const float* q, const float* k, const float* v, float* o, int BH, int N, int d, int causal) {
  const float scale = 1.f / std::sqrt((float)d);
  std::vector<float> acc(d);
  for (int b = 0; b < BH; ++b) for (int i = 0; i < N; ++i) {
    float m = -INFINITY, l = 0.f; std::fill(acc.begin(), acc.end(), 0.f);
    const float* qi = q + ((long long)b * N + i) * d;
    const int jmax = causal ? i + 1 : N;
    for (int j = 0; j < jmax; ++j) {
      const float* kj = k + ((long long)b * N + j) * d; const float* vj = v + ((long long)b * N + j) * d;
      float s = 0.f; for (int t = 0; t < d; ++t) s += qi[t] * kj[t]; s *= scale;
      const float mn = std::max(m, s); const float corr = std::exp(m - mn); const float p = std::exp(s - mn);
      l = l * corr + p; for (int t = 0; t < d; ++t) acc[t] = acc[t] * corr + p * vj[t]; m = mn;
    }
    for (int t = 0; t < d; ++t) o[((long long)b * N + i) * d + t] = acc[t] / l;
  }
}
// y[m,n] = x[m,k] . ((q - zp) * scale), INT4 layout of rumus-vision/src/quant.rs
void orc_qmatmul_int4(const float* x, const int* packed, const float* scales, const float* zps, float* y, int m, int k, int n, int group) {
  for (int i = 0; i < m; ++i) for (int j = 0; j < n; ++j) {
    float acc = 0.f;
    for (int r = 0; r < k; ++r) {
      const uint32_t w = (uint32_t)packed[(long long)(r / 8) * n + j];
      const float qv = (float)((w >> (4 * (r % 8))) & 0xF);
      const int g = r / group;
      acc += x[(long long)i * k + r] * (qv - zps[(long long)g * n + j]) * scales[(long long)g * n + j];
    }
    y[(long long)i * n + j] = acc;
  }
}
// CSR SpMM
void orc_spmm(const int* rowptr, const int* col, const float* val, const float* x, float* y, int rows, int feat) {
  for (int r = 0; r < rows; ++r) for (int f = 0; f < feat; ++f) {
    float acc = 0.f; for (int e = rowptr[r]; e < rowptr[r + 1]; ++e) acc += (val ? val[e] : 1.f) * x[(long long)col[e] * feat + f];
    y[(long long)r * feat + f] = acc;
  }
}
void orc_adam_step(float* p, float* m, float* v, const float* g, long long n, float lr, float b1, float b2, float eps, float bc1, float bc2, float wd, int adamw) {
  for (long long i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + (1.f - b1) * g[i]; v[i] = b2 * v[i] + (1.f - b2) * g[i] * g[i];
    if (adamw) p[i] -= lr * wd * p[i];
    p[i] -= lr * (m[i] / bc1) / (std::sqrt(v[i] / bc2) + eps);
  }
}
void orc_sgd_step(float* p, float* vel, const float* g, long long n, float lr, float mu) {
  for (long long i = 0; i < n; ++i) { vel[i] = mu * vel[i] + g[i]; p[i] -= lr * vel[i]; }
}
}
