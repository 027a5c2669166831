// Row softmax (forward / backward) and fused cross-entropy (forward + gradient
// in one launch) for sm_100a.
//
// Reference counterparts: rumus/src/backend/gpu/shaders/softmax.wgsl:25,
// softmax_bw.wgsl:26 and cross_entropy.wgsl:32,124 (loss per row, gradient
// `(softmax - onehot) / B` precomputed in forward, then a single-workgroup sum).
// Here one CTA owns one row, streams it with 128-bit loads, keeps the
// max / sum-exp online, and the loss reduction is a deterministic second stage.
#include "sm100_common.cuh"

namespace rb {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float block_reduce_sum(float v, float* sbuf) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sbuf[w] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? sbuf[threadIdx.x] : 0.f;
  if (w == 0) r = warp_sum(r);
  if (threadIdx.x == 0) sbuf[0] = r;
  __syncthreads();
  return sbuf[0];
}
__device__ __forceinline__ float block_reduce_max(float v, float* sbuf) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sbuf[w] = v;
  __syncthreads();
  float r = (threadIdx.x < (blockDim.x >> 5)) ? sbuf[threadIdx.x] : -INFINITY;
  if (w == 0) r = warp_max(r);
  if (threadIdx.x == 0) sbuf[0] = r;
  __syncthreads();
  return sbuf[0];
}

// online (max, sum) merge
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  float mm = fmaxf(m, m2);
  if (mm == -INFINITY) { m = mm; s = 0.f; return; }
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

template <typename T>
__device__ __forceinline__ void row_max_sum(const T* row, int n, bool vec, float& m_out,
                                            float& s_out, float* sbuf) {
  constexpr int VEC = 16 / sizeof(T);
  float m = -INFINITY, s = 0.f;
  if (vec) {
    for (int c = threadIdx.x * VEC; c < n; c += blockDim.x * VEC) {
      uint4 raw = *reinterpret_cast<const uint4*>(row + c);
      const T* e = reinterpret_cast<const T*>(&raw);
      float lm = -INFINITY;
#pragma unroll
      for (int j = 0; j < VEC; ++j) lm = fmaxf(lm, to_f32<T>(e[j]));
      float ls = 0.f;
#pragma unroll
      for (int j = 0; j < VEC; ++j) ls += __expf(to_f32<T>(e[j]) - lm);
      online_merge(m, s, lm, ls);
    }
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float v = to_f32<T>(row[c]);
      online_merge(m, s, v, 1.f);
    }
  }
  const float gm = block_reduce_max(m, sbuf);
  const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_reduce_sum(contrib, sbuf);
  m_out = gm;
  s_out = gs;
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
    softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int n, int vec) {
  __shared__ float sbuf[32];
  constexpr int VEC = 16 / sizeof(T);
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = x + r * n;
    T* yr = y + r * n;
    float m, s;
    row_max_sum<T>(xr, n, vec, m, s, sbuf);
    const float inv = 1.f / s;
    if (vec) {
      for (int c = threadIdx.x * VEC; c < n; c += blockDim.x * VEC) {
        uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
        const T* e = reinterpret_cast<const T*>(&raw);
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < VEC; ++j) oe[j] = from_f32<T>(__expf(to_f32<T>(e[j]) - m) * inv);
        *reinterpret_cast<uint4*>(yr + c) = o;
      }
    } else {
      for (int c = threadIdx.x; c < n; c += blockDim.x)
        yr[c] = from_f32<T>(__expf(to_f32<T>(xr[c]) - m) * inv);
    }
  }
}

// dx = y * (dy - sum(dy*y))
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
    softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                       long long rows, int n) {
  __shared__ float sbuf[32];
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* yr = y + r * n;
    const T* dr = dy + r * n;
    float dot = 0.f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) dot += to_f32<T>(yr[c]) * to_f32<T>(dr[c]);
    dot = block_reduce_sum(dot, sbuf);
    for (int c = threadIdx.x; c < n; c += blockDim.x)
      dx[r * n + c] = from_f32<T>(to_f32<T>(yr[c]) * (to_f32<T>(dr[c]) - dot));
  }
}

// Fused cross entropy.  loss_rows[r] = lse(logits[r]) - logits[r, target[r]].
// dlogits[r, c] = (softmax(logits[r])[c] - [c == target]) * grad_scale   (optional)
// Rows whose target is < 0 are ignored (loss 0, zero gradient).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
    cross_entropy_kernel(const T* __restrict__ logits, const long long* __restrict__ targets,
                         float* __restrict__ loss_rows, T* __restrict__ dlogits, long long rows,
                         int n, long long ld, float grad_scale, int vec) {
  __shared__ float sbuf[32];
  constexpr int VEC = 16 / sizeof(T);
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* xr = logits + r * ld;
    const long long tgt = targets[r];
    if (tgt < 0 || tgt >= n) {
      if (threadIdx.x == 0) loss_rows[r] = 0.f;
      if (dlogits)
        for (int c = threadIdx.x; c < n; c += blockDim.x) dlogits[r * ld + c] = from_f32<T>(0.f);
      continue;
    }
    // read the target logit before any thread may overwrite the row (dlogits may alias logits)
    float tl = 0.f;
    if (threadIdx.x == 0) tl = to_f32<T>(xr[tgt]);
    float m, s;
    row_max_sum<T>(xr, n, vec, m, s, sbuf);
    if (threadIdx.x == 0) loss_rows[r] = (m + __logf(s)) - tl;
    if (dlogits) {
      const float inv = grad_scale / s;
      T* dr = dlogits + r * ld;
      if (vec) {
        for (int c = threadIdx.x * VEC; c < n; c += blockDim.x * VEC) {
          uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
          const T* e = reinterpret_cast<const T*>(&raw);
          uint4 o;
          T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            float g = __expf(to_f32<T>(e[j]) - m) * inv;
            if (c + j == tgt) g -= grad_scale;
            oe[j] = from_f32<T>(g);
          }
          *reinterpret_cast<uint4*>(dr + c) = o;
        }
      } else {
        for (int c = threadIdx.x; c < n; c += blockDim.x) {
          float g = __expf(to_f32<T>(xr[c]) - m) * inv;
          if (c == tgt) g -= grad_scale;
          dr[c] = from_f32<T>(g);
        }
      }
    }
  }
}

// deterministic sum of `n` floats times `scale` -> out[0]   (single CTA)
__global__ void __launch_bounds__(1024) reduce_sum_kernel(const float* __restrict__ v, long long n,
                                                           float scale, float* __restrict__ out) {
  __shared__ float sbuf[32];
  float acc = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) acc += v[i];
  acc = block_reduce_sum(acc, sbuf);
  if (threadIdx.x == 0) out[0] = acc * scale;
}

template <typename T>
static bool vec_ok(const void* a, const void* b, long long ld) {
  constexpr int VEC = 16 / sizeof(T);
  return ld % VEC == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
         (b == nullptr || (reinterpret_cast<uintptr_t>(b) & 15) == 0);
}

}  // namespace rb

extern "C" {

int rb_softmax_fwd(int dtype, const void* x, void* y, long long rows, int n, void* stream) {
  using namespace rb;
  if (rows <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)(rows < 65535 * 4 ? rows : 65535 * 4);
  if (dtype == rbh::DT_BF16)
    softmax_fwd_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, st>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, n, vec_ok<__nv_bfloat16>(x, y, n) && n % 8 == 0);
  else if (dtype == rbh::DT_F16)
    softmax_fwd_kernel<__half><<<grid, kRowThreads, 0, st>>>((const __half*)x, (__half*)y, rows, n,
                                                            vec_ok<__half>(x, y, n) && n % 8 == 0);
  else
    softmax_fwd_kernel<float><<<grid, kRowThreads, 0, st>>>((const float*)x, (float*)y, rows, n,
                                                           vec_ok<float>(x, y, n) && n % 4 == 0);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_softmax_bwd(int dtype, const void* y, const void* dy, void* dx, long long rows, int n,
                   void* stream) {
  using namespace rb;
  if (rows <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)(rows < 65535 * 4 ? rows : 65535 * 4);
  if (dtype == rbh::DT_BF16)
    softmax_bwd_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, st>>>(
        (const __nv_bfloat16*)y, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, rows, n);
  else if (dtype == rbh::DT_F16)
    softmax_bwd_kernel<__half><<<grid, kRowThreads, 0, st>>>((const __half*)y, (const __half*)dy,
                                                            (__half*)dx, rows, n);
  else
    softmax_bwd_kernel<float><<<grid, kRowThreads, 0, st>>>((const float*)y, (const float*)dy,
                                                           (float*)dx, rows, n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

// loss_out[0] = loss_scale * sum_r loss_rows[r]; dlogits may be null (forward only) and may
// alias logits (in-place gradient).
int rb_cross_entropy(int dtype, const void* logits, const long long* targets, float* loss_rows,
                     float* loss_out, void* dlogits, long long rows, int n, long long ld,
                     float grad_scale, float loss_scale, void* stream) {
  using namespace rb;
  if (rows <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)(rows < 65535 * 4 ? rows : 65535 * 4);
  if (dtype == rbh::DT_BF16)
    cross_entropy_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, st>>>(
        (const __nv_bfloat16*)logits, targets, loss_rows, (__nv_bfloat16*)dlogits, rows, n, ld,
        grad_scale, vec_ok<__nv_bfloat16>(logits, dlogits, ld) && n % 8 == 0);
  else if (dtype == rbh::DT_F16)
    cross_entropy_kernel<__half><<<grid, kRowThreads, 0, st>>>(
        (const __half*)logits, targets, loss_rows, (__half*)dlogits, rows, n, ld, grad_scale,
        vec_ok<__half>(logits, dlogits, ld) && n % 8 == 0);
  else
    cross_entropy_kernel<float><<<grid, kRowThreads, 0, st>>>(
        (const float*)logits, targets, loss_rows, (float*)dlogits, rows, n, ld, grad_scale,
        vec_ok<float>(logits, dlogits, ld) && n % 4 == 0);
  if (loss_out) reduce_sum_kernel<<<1, 1024, 0, st>>>(loss_rows, rows, loss_scale, loss_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_reduce_sum_f32(const float* v, long long n, float scale, float* out, void* stream) {
  rb::reduce_sum_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(v, n, scale, out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
