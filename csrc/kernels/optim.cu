// Fused optimizer kernels for sm_100a.
//
// The reference launches one tiny kernel per parameter
// (rumus/src/backend/gpu/shaders/optim.wgsl:23,53, adamw.wgsl:26, dispatched from
// rumus/src/optim/{sgd,adam,adamw}.rs) and computes the clip norm with a
// single-workgroup reduction per parameter (shaders/reduce_sum_sq.wgsl:21).
// Here a whole parameter list is updated by ONE launch (a table of up to 32
// tensors x 4 pointers is passed by value), fp32 master weights / moments are
// updated with 128-bit accesses, the low-precision model copy is written back in
// the same pass, and gradient unscale + clip + the non-finite "skip" decision
// are read from device memory so a step can be captured in a CUDA graph.
#include "sm100_common.cuh"

namespace rb {

constexpr int kMaxTensors = 32;
constexpr int kMaxBlocks = 320;
constexpr int kChunk = 2048 * 16;  // elements per CTA chunk

struct TensorTable {
  void* grad[kMaxTensors];
  float* master[kMaxTensors];
  float* m[kMaxTensors];
  float* v[kMaxTensors];
  void* model[kMaxTensors];  // low-precision copy to refresh (or null)
  long long numel[kMaxTensors];
  unsigned char block_tensor[kMaxBlocks];
  int block_chunk[kMaxBlocks];
};

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay;
  float bc1, bc2;           // 1 - beta^t (host computed) — ignored when step_ptr != null
  int adamw;                // 1: decoupled decay (p -= lr*wd*p before the Adam step), 0: none
  const float* grad_scale;  // optional device scalar multiplied into every gradient
  const int* skip;          // optional device flag: non-zero -> leave everything untouched
  const int* step_ptr;      // optional device step counter (t >= 1)
};

template <typename TG>
__device__ __forceinline__ void adam_range(const TG* __restrict__ g, float* __restrict__ p,
                                           float* __restrict__ m, float* __restrict__ v,
                                           TG* __restrict__ model, long long begin, long long end,
                                           const AdamHyper& h, float bc1, float bc2, float gs) {
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float grad = to_f32<TG>(g[i]) * gs;
    float mi = h.beta1 * m[i] + (1.f - h.beta1) * grad;
    float vi = h.beta2 * v[i] + (1.f - h.beta2) * grad * grad;
    m[i] = mi;
    v[i] = vi;
    float pi = p[i];
    if (h.adamw) pi -= h.lr * h.weight_decay * pi;
    pi -= h.lr * (mi / bc1) / (sqrtf(vi / bc2) + h.eps);
    p[i] = pi;
    if (model) model[i] = from_f32<TG>(pi);
  }
}

template <typename TG>
__global__ void __launch_bounds__(512) multi_tensor_adam_kernel(const TensorTable tab, AdamHyper h) {
  if (h.skip && *h.skip) return;
  float bc1 = h.bc1, bc2 = h.bc2;
  if (h.step_ptr) {
    const float t = (float)(*h.step_ptr);
    bc1 = 1.f - __powf(h.beta1, t);
    bc2 = 1.f - __powf(h.beta2, t);
  }
  const float gs = h.grad_scale ? *h.grad_scale : 1.f;
  const int t = tab.block_tensor[blockIdx.x];
  const long long begin = (long long)tab.block_chunk[blockIdx.x] * kChunk;
  const long long end = min(tab.numel[t], begin + kChunk);
  adam_range<TG>((const TG*)tab.grad[t], tab.master[t], tab.m[t], tab.v[t], (TG*)tab.model[t], begin,
                 end, h, bc1, bc2, gs);
}

// Flat-arena Adam: one contiguous range, vectorised.
template <typename TG>
__global__ void __launch_bounds__(256)
    adam_flat_kernel(const TG* __restrict__ g, float* __restrict__ p, float* __restrict__ m,
                     float* __restrict__ v, TG* __restrict__ model, long long n, AdamHyper h) {
  if (h.skip && *h.skip) return;
  float bc1 = h.bc1, bc2 = h.bc2;
  if (h.step_ptr) {
    const float t = (float)(*h.step_ptr);
    bc1 = 1.f - __powf(h.beta1, t);
    bc2 = 1.f - __powf(h.beta2, t);
  }
  const float gs = h.grad_scale ? *h.grad_scale : 1.f;
  const float rbc1 = 1.f / bc1, rbc2 = 1.f / bc2;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float gr[4];
      if constexpr (sizeof(TG) == 4) {
        float4 gv = *reinterpret_cast<const float4*>(g + i);
        gr[0] = gv.x; gr[1] = gv.y; gr[2] = gv.z; gr[3] = gv.w;
      } else {
        uint2 raw = *reinterpret_cast<const uint2*>(g + i);
        const TG* e = reinterpret_cast<const TG*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) gr[j] = to_f32<TG>(e[j]);
      }
      float4 pv = *reinterpret_cast<float4*>(p + i);
      float4 mv = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float* pp = &pv.x; float* mp = &mv.x; float* vp = &vv.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float grad = gr[j] * gs;
        mp[j] = h.beta1 * mp[j] + (1.f - h.beta1) * grad;
        vp[j] = h.beta2 * vp[j] + (1.f - h.beta2) * grad * grad;
        if (h.adamw) pp[j] -= h.lr * h.weight_decay * pp[j];
        pp[j] -= h.lr * (mp[j] * rbc1) / (sqrtf(vp[j] * rbc2) + h.eps);
      }
      *reinterpret_cast<float4*>(p + i) = pv;
      *reinterpret_cast<float4*>(m + i) = mv;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (model) {
        if constexpr (sizeof(TG) == 4) {
          *reinterpret_cast<float4*>(model + i) = pv;
        } else {
          uint2 o;
          TG* oe = reinterpret_cast<TG*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) oe[j] = from_f32<TG>(pp[j]);
          *reinterpret_cast<uint2*>(model + i) = o;
        }
      }
    } else {
      for (long long k = i; k < n; ++k) {
        const float grad = to_f32<TG>(g[k]) * gs;
        float mi = h.beta1 * m[k] + (1.f - h.beta1) * grad;
        float vi = h.beta2 * v[k] + (1.f - h.beta2) * grad * grad;
        m[k] = mi; v[k] = vi;
        float pi = p[k];
        if (h.adamw) pi -= h.lr * h.weight_decay * pi;
        pi -= h.lr * (mi * rbc1) / (sqrtf(vi * rbc2) + h.eps);
        p[k] = pi;
        if (model) model[k] = from_f32<TG>(pi);
      }
    }
  }
}

struct SgdHyper {
  float lr, momentum, weight_decay;
  const float* grad_scale;
  const int* skip;
};

// v = mu*v + g ; p -= lr*v    (momentum buffer lives in tab.m; tab.v unused)
template <typename TG>
__global__ void __launch_bounds__(512) multi_tensor_sgd_kernel(const TensorTable tab, SgdHyper h) {
  if (h.skip && *h.skip) return;
  const float gs = h.grad_scale ? *h.grad_scale : 1.f;
  const int t = tab.block_tensor[blockIdx.x];
  const long long begin = (long long)tab.block_chunk[blockIdx.x] * kChunk;
  const long long end = min(tab.numel[t], begin + kChunk);
  const TG* g = (const TG*)tab.grad[t];
  float* p = tab.master[t];
  float* mom = tab.m[t];
  TG* model = (TG*)tab.model[t];
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    float grad = to_f32<TG>(g[i]) * gs;
    float pi = p[i];
    if (h.weight_decay != 0.f) grad += h.weight_decay * pi;
    float vel = grad;
    if (mom) {
      vel = h.momentum * mom[i] + grad;
      mom[i] = vel;
    }
    pi -= h.lr * vel;
    p[i] = pi;
    if (model) model[i] = from_f32<TG>(pi);
  }
}

// sum of squares, stage 1: one partial per CTA (optionally also flags non-finite values)
template <typename T>
__global__ void __launch_bounds__(512)
    sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partials,
                         int* __restrict__ found_inf) {
  __shared__ float sbuf[16];
  float acc = 0.f;
  bool bad = false;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = to_f32<T>(x[i]);
    acc += v * v;
    bad |= !isfinite(v);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sbuf[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < (blockDim.x >> 5) ? sbuf[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) partials[blockIdx.x] = r;
  }
  if (bad && found_inf) *found_inf = 1;
}
// stage 2: norm = sqrt(sum partials); clip_coef = min(1, max_norm / (norm + 1e-6))
__global__ void __launch_bounds__(1024)
    norm_finalize_kernel(const float* __restrict__ partials, int n, float max_norm,
                         float extra_scale, float* __restrict__ norm_out,
                         float* __restrict__ coef_out) {
  __shared__ float sbuf[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partials[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sbuf[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = sbuf[threadIdx.x];
    r = warp_sum(r);
    if (threadIdx.x == 0) {
      const float norm = sqrtf(r) * extra_scale;
      if (norm_out) norm_out[0] = norm;
      if (coef_out) {
        float c = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
        coef_out[0] = c * extra_scale;
      }
    }
  }
}

// x *= *scale_ptr (or `scale`), sets *found_inf when a non-finite value is seen
template <typename T>
__global__ void scale_check_kernel(T* __restrict__ x, long long n, const float* scale_ptr,
                                   float scale, int* __restrict__ found_inf) {
  const float s = scale_ptr ? *scale_ptr : scale;
  bool bad = false;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = to_f32<T>(x[i]);
    bad |= !isfinite(v);
    x[i] = from_f32<T>(v * s);
  }
  if (bad && found_inf) *found_inf = 1;
}

// Loss-scale bookkeeping on the device (no host read of the overflow flag, so the host can keep
// launching the next step): after an overflow the scale is multiplied by `backoff` and the run of clean
// steps starts again; every `interval` clean steps it is multiplied by `growth`.
__global__ void scaler_update_kernel(float* scale, float* inv_scale, int* good_steps, const int* found_inf,
                                     float growth, float backoff, int interval) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  float s = *scale;
  int g = *good_steps;
  if (*found_inf != 0) {
    s *= backoff;
    g = 0;
  } else {
    g += 1;
    if (interval > 0 && g % interval == 0) s *= growth;
  }
  *scale = s;
  *inv_scale = 1.f / s;
  *good_steps = g;
}

}  // namespace rb

extern "C" {

int rb_scaler_update(float* scale, float* inv_scale, int* good_steps, const int* found_inf, float growth,
                     float backoff, int interval, void* stream) {
  rb::scaler_update_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(scale, inv_scale, good_steps, found_inf, growth, backoff,
                                                              interval);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}


struct RbTensorList {
  int count;
  void** grad;
  float** master;
  float** m;
  float** v;
  void** model;
  long long* numel;
};

static int fill_and_launch(const RbTensorList* l, int gdtype, bool adam, const rb::AdamHyper* ah,
                           const rb::SgdHyper* sh, cudaStream_t st) {
  using namespace rb;
  TensorTable tab;
  int nt = 0, nb = 0;
  auto flush = [&]() -> int {
    if (nb == 0) return 0;
    if (adam) {
      if (gdtype == rbh::DT_BF16) multi_tensor_adam_kernel<__nv_bfloat16><<<nb, 512, 0, st>>>(tab, *ah);
      else if (gdtype == rbh::DT_F16) multi_tensor_adam_kernel<__half><<<nb, 512, 0, st>>>(tab, *ah);
      else multi_tensor_adam_kernel<float><<<nb, 512, 0, st>>>(tab, *ah);
    } else {
      if (gdtype == rbh::DT_BF16) multi_tensor_sgd_kernel<__nv_bfloat16><<<nb, 512, 0, st>>>(tab, *sh);
      else if (gdtype == rbh::DT_F16) multi_tensor_sgd_kernel<__half><<<nb, 512, 0, st>>>(tab, *sh);
      else multi_tensor_sgd_kernel<float><<<nb, 512, 0, st>>>(tab, *sh);
    }
    nt = 0;
    nb = 0;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 3000 + (int)e;
  };
  int launches = 0;
  for (int i = 0; i < l->count; ++i) {
    const long long n = l->numel[i];
    if (n <= 0) continue;
    const int chunks = (int)((n + kChunk - 1) / kChunk);
    int c = 0;
    while (c < chunks) {
      if (nt == kMaxTensors || nb == kMaxBlocks) {
        int rc = flush();
        if (rc) return -rc;
        ++launches;
      }
      // (re)register tensor i in the table
      const int slot = nt++;
      tab.grad[slot] = l->grad[i];
      tab.master[slot] = l->master[i];
      tab.m[slot] = l->m ? l->m[i] : nullptr;
      tab.v[slot] = l->v ? l->v[i] : nullptr;
      tab.model[slot] = l->model ? l->model[i] : nullptr;
      tab.numel[slot] = n;
      while (c < chunks && nb < kMaxBlocks) {
        tab.block_tensor[nb] = (unsigned char)slot;
        tab.block_chunk[nb] = c;
        ++nb;
        ++c;
      }
    }
  }
  if (nb) {
    int rc = flush();
    if (rc) return -rc;
    ++launches;
  }
  return launches;
}

// Returns the number of kernel launches (>= 0) or a negative error.
int rb_multi_tensor_adam(const RbTensorList* l, int grad_dtype, float lr, float beta1, float beta2,
                         float eps, float weight_decay, float bc1, float bc2, int adamw,
                         const float* grad_scale, const int* skip, const int* step_ptr,
                         void* stream) {
  rb::AdamHyper h{lr, beta1, beta2, eps, weight_decay, bc1, bc2, adamw, grad_scale, skip, step_ptr};
  return fill_and_launch(l, grad_dtype, true, &h, nullptr, (cudaStream_t)stream);
}
int rb_multi_tensor_sgd(const RbTensorList* l, int grad_dtype, float lr, float momentum,
                        float weight_decay, const float* grad_scale, const int* skip,
                        void* stream) {
  rb::SgdHyper h{lr, momentum, weight_decay, grad_scale, skip};
  return fill_and_launch(l, grad_dtype, false, nullptr, &h, (cudaStream_t)stream);
}
int rb_adam_flat(int grad_dtype, const void* g, float* p, float* m, float* v, void* model,
                 long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                 float bc1, float bc2, int adamw, const float* grad_scale, const int* skip,
                 const int* step_ptr, void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  AdamHyper h{lr, beta1, beta2, eps, weight_decay, bc1, bc2, adamw, grad_scale, skip, step_ptr};
  cudaStream_t st = (cudaStream_t)stream;
  long long blocks = (n / 4 + 255) / 256;
  const long long cap = (long long)rbh::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (grad_dtype == rbh::DT_BF16)
    adam_flat_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)g, p, m, v, (__nv_bfloat16*)model, n, h);
  else if (grad_dtype == rbh::DT_F16)
    adam_flat_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((const __half*)g, p, m, v, (__half*)model, n, h);
  else
    adam_flat_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)g, p, m, v, (float*)model, n, h);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

// Stage 1 of a global L2 norm over one tensor: writes `blocks` partials starting at partials[offset].
// Returns the number of partials written (>= 0) or a negative error.
int rb_sumsq_partials(int dtype, const void* x, long long n, float* partials, int max_blocks,
                      int* found_inf, void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  long long blocks = (n + 512 * 8 - 1) / (512 * 8);
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  if (dtype == rbh::DT_BF16) sumsq_partial_kernel<__nv_bfloat16><<<(unsigned)blocks, 512, 0, st>>>((const __nv_bfloat16*)x, n, partials, found_inf);
  else if (dtype == rbh::DT_F16) sumsq_partial_kernel<__half><<<(unsigned)blocks, 512, 0, st>>>((const __half*)x, n, partials, found_inf);
  else sumsq_partial_kernel<float><<<(unsigned)blocks, 512, 0, st>>>((const float*)x, n, partials, found_inf);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? (int)blocks : -(3000 + (int)e);
}
int rb_norm_finalize(const float* partials, int n, float max_norm, float extra_scale,
                     float* norm_out, float* coef_out, void* stream) {
  rb::norm_finalize_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(partials, n, max_norm, extra_scale, norm_out, coef_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
int rb_scale_check(int dtype, void* x, long long n, const float* scale_ptr, float scale,
                   int* found_inf, void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)rbh::sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (dtype == rbh::DT_BF16) scale_check_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((__nv_bfloat16*)x, n, scale_ptr, scale, found_inf);
  else if (dtype == rbh::DT_F16) scale_check_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>((__half*)x, n, scale_ptr, scale, found_inf);
  else scale_check_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((float*)x, n, scale_ptr, scale, found_inf);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
