// LayerNorm / RMSNorm forward and backward for sm_100a.
//
// One warp per row, 128-bit loads, fp32 statistics.  A row is kept packed in
// registers between the statistics pass and the normalise pass when it fits
// (up to 32 vectors per lane); longer rows are re-read (they come from L1/L2).
// Optional fusions: forward adds a residual stream first and writes the sum out
// (`h = x + res`), backward adds an incoming residual-stream gradient to dx.
//
// Backward produces dx per row and accumulates d_gamma / d_beta per CTA in
// shared memory; every CTA writes one partial row to a scratch buffer
// [num_ctas, 2, D] that a second kernel reduces.  The reference does this with
// three kernels plus two generic reductions
// (rumus/src/backend/gpu/shaders/layer_norm.wgsl:29, layer_norm_bw.wgsl:30,
// layer_norm_grad_weight.wgsl:30, rumus/src/autograd/backward.rs:539).
#include "sm100_common.cuh"

namespace rb {

template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    return to_f32<T>(reinterpret_cast<const T*>(&raw)[i]);
  }
  __device__ __forceinline__ void set(int i, float v) {
    reinterpret_cast<T*>(&raw)[i] = from_f32<T>(v);
  }
};

// Generic per-row accessor: vector path when `vec` (D % VEC == 0 and 16-byte aligned rows)
template <typename T>
__device__ __forceinline__ float ld(const T* p, long long i) {
  return to_f32<T>(p[i]);
}

constexpr int kNormWarps = 8;

__host__ __device__ __forceinline__ int skew(int i) { return i + (i >> 5); }

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T, bool RMS, int ITERS>
__global__ void __launch_bounds__(kNormWarps * 32)
    norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ gamma,
                    const T* __restrict__ beta, T* __restrict__ y, T* __restrict__ h_out,
                    float* __restrict__ stats /* [rows,2]: mean, rstd */, long long rows, int D,
                    float eps) {
  constexpr int VEC = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kNormWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kNormWarps;
  for (long long row = warp; row < rows; row += nwarps) {
    const T* xr = x + row * D;
    const T* rr = res ? res + row * D : nullptr;
    float sum = 0.f, sumsq = 0.f;
    if constexpr (ITERS > 0) {
      Vec16<T> cache[ITERS];
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int c = (it * 32 + lane) * VEC;
        if (c < D) {
          cache[it].raw = *reinterpret_cast<const uint4*>(xr + c);
          if (rr) {
            Vec16<T> rv;
            rv.raw = *reinterpret_cast<const uint4*>(rr + c);
#pragma unroll
            for (int j = 0; j < VEC; ++j) cache[it].set(j, cache[it].get(j) + rv.get(j));
            if (h_out) *reinterpret_cast<uint4*>(h_out + row * D + c) = cache[it].raw;
          }
#pragma unroll
          for (int j = 0; j < VEC; ++j) sum += cache[it].get(j);
        }
      }
      sum = warp_sum(sum);
      const float mean = RMS ? 0.f : sum / D;
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int c = (it * 32 + lane) * VEC;
        if (c < D) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            float d = cache[it].get(j) - mean;
            sumsq += d * d;
          }
        }
      }
      sumsq = warp_sum(sumsq);
      const float rstd = rsqrtf(sumsq / D + eps);
      if (lane == 0 && stats) {
        stats[row * 2] = mean;
        stats[row * 2 + 1] = rstd;
      }
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int c = (it * 32 + lane) * VEC;
        if (c < D) {
          Vec16<T> g, b, o;
          g.raw = *reinterpret_cast<const uint4*>(gamma + c);
          if (!RMS && beta) b.raw = *reinterpret_cast<const uint4*>(beta + c);
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            float v = (cache[it].get(j) - mean) * rstd * g.get(j);
            if (!RMS && beta) v += b.get(j);
            o.set(j, v);
          }
          *reinterpret_cast<uint4*>(y + row * D + c) = o.raw;
        }
      }
    } else {
      // generic path: scalar, any D / alignment, three passes
      for (int c = lane; c < D; c += 32) {
        float v = ld(xr, c) + (rr ? ld(rr, c) : 0.f);
        if (rr && h_out) h_out[row * D + c] = from_f32<T>(v);
        sum += v;
      }
      sum = warp_sum(sum);
      const float mean = RMS ? 0.f : sum / D;
      for (int c = lane; c < D; c += 32) {
        float v = (rr && h_out) ? ld(h_out + row * D, c) : ld(xr, c) + (rr ? ld(rr, c) : 0.f);
        float d = v - mean;
        sumsq += d * d;
      }
      sumsq = warp_sum(sumsq);
      const float rstd = rsqrtf(sumsq / D + eps);
      if (lane == 0 && stats) {
        stats[row * 2] = mean;
        stats[row * 2 + 1] = rstd;
      }
      for (int c = lane; c < D; c += 32) {
        float v = (rr && h_out) ? ld(h_out + row * D, c) : ld(xr, c) + (rr ? ld(rr, c) : 0.f);
        float o = (v - mean) * rstd * ld(gamma, c);
        if (!RMS && beta) o += ld(beta, c);
        y[row * D + c] = from_f32<T>(o);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------
// x here is the *normalised input* (h when a residual was fused in forward).
template <typename T, bool RMS>
__global__ void __launch_bounds__(kNormWarps * 32)
    norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                    const float* __restrict__ stats, const T* __restrict__ dres,
                    T* __restrict__ dx, float* __restrict__ partials /* [grid,2,D] */,
                    long long rows, int D, int vec_ok) {
  // [2][D] accumulators, stored skewed (one pad float per 32) so that the 32 lanes of one
  // shared-memory atomic — addresses lane*VEC + j — fall into 32 different banks
  extern __shared__ float s_acc[];
  const int DS = skew(D) + 1;
  float* s_dg = s_acc;
  float* s_db = s_acc + DS;
  for (int i = threadIdx.x; i < 2 * DS; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  constexpr int VEC = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kNormWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kNormWarps;
  for (long long row = warp; row < rows; row += nwarps) {
    const T* xr = x + row * D;
    const T* dyr = dy + row * D;
    const float mean = RMS ? 0.f : stats[row * 2];
    const float rstd = stats[row * 2 + 1];
    float c1 = 0.f, c2 = 0.f;  // sum(dy*g), sum(dy*g*xhat)
    if (vec_ok) {
      for (int c = lane * VEC; c < D; c += 32 * VEC) {
        Vec16<T> xv, dv, gv;
        xv.raw = *reinterpret_cast<const uint4*>(xr + c);
        dv.raw = *reinterpret_cast<const uint4*>(dyr + c);
        gv.raw = *reinterpret_cast<const uint4*>(gamma + c);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          float xh = (xv.get(j) - mean) * rstd;
          float dg = dv.get(j) * gv.get(j);
          c1 += dg;
          c2 += dg * xh;
        }
      }
    } else {
      for (int c = lane; c < D; c += 32) {
        float xh = (ld(xr, c) - mean) * rstd;
        float dg = ld(dyr, c) * ld(gamma, c);
        c1 += dg;
        c2 += dg * xh;
      }
    }
    c1 = warp_sum(c1) / D;
    c2 = warp_sum(c2) / D;
    if (RMS) c1 = 0.f;
    if (vec_ok) {
      for (int c = lane * VEC; c < D; c += 32 * VEC) {
        Vec16<T> xv, dv, gv, rv, ov;
        xv.raw = *reinterpret_cast<const uint4*>(xr + c);
        dv.raw = *reinterpret_cast<const uint4*>(dyr + c);
        gv.raw = *reinterpret_cast<const uint4*>(gamma + c);
        if (dres) rv.raw = *reinterpret_cast<const uint4*>(dres + row * D + c);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          float xh = (xv.get(j) - mean) * rstd;
          float d = dv.get(j);
          float o = rstd * (d * gv.get(j) - c1 - xh * c2);
          if (dres) o += rv.get(j);
          ov.set(j, o);
          atomicAdd(&s_dg[skew(c + j)], d * xh);
          if (!RMS) atomicAdd(&s_db[skew(c + j)], d);
        }
        *reinterpret_cast<uint4*>(dx + row * D + c) = ov.raw;
      }
    } else {
      for (int c = lane; c < D; c += 32) {
        float xh = (ld(xr, c) - mean) * rstd;
        float d = ld(dyr, c);
        float o = rstd * (d * ld(gamma, c) - c1 - xh * c2);
        if (dres) o += ld(dres + row * D, c);
        dx[row * D + c] = from_f32<T>(o);
        atomicAdd(&s_dg[skew(c)], d * xh);
        if (!RMS) atomicAdd(&s_db[skew(c)], d);
      }
    }
  }
  __syncthreads();
  float* out = partials + (long long)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    out[i] = s_dg[skew(i)];
    out[D + i] = s_db[skew(i)];
  }
}

// partials [n,2,D] -> dgamma[D], dbeta[D] (dbeta may be null)
template <typename T>
__global__ void norm_bwd_reduce_kernel(const float* __restrict__ partials, int n, int D,
                                       T* __restrict__ dgamma, T* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float g = 0.f, b = 0.f;
  for (int i = 0; i < n; ++i) {
    g += partials[(long long)i * 2 * D + c];
    b += partials[(long long)i * 2 * D + D + c];
  }
  dgamma[c] = from_f32<T>(g);
  if (dbeta) dbeta[c] = from_f32<T>(b);
}

template <typename T, bool RMS>
int launch_norm_fwd(const void* x, const void* res, const void* gamma, const void* beta, void* y,
                    void* h_out, float* stats, long long rows, int D, float eps, cudaStream_t st) {
  constexpr int VEC = Vec16<T>::N;
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = (D % VEC == 0) && al(x) && al(res) && al(gamma) && al(beta) && al(y) && al(h_out);
  const int iters = vec ? (D + 32 * VEC - 1) / (32 * VEC) : 0;
  long long blocks = (rows + kNormWarps - 1) / kNormWarps;
  const long long maxb = (long long)rbh::sm_count() * 8;
  if (blocks > maxb) blocks = maxb;
  if (blocks < 1) blocks = 1;
#define RB_NORM_LAUNCH(IT)                                                                        \
  norm_fwd_kernel<T, RMS, IT><<<(unsigned)blocks, kNormWarps * 32, 0, st>>>(                       \
      (const T*)x, (const T*)res, (const T*)gamma, (const T*)beta, (T*)y, (T*)h_out, stats, rows, \
      D, eps)
  if (!vec || iters > 32) RB_NORM_LAUNCH(0);
  else if (iters <= 1) RB_NORM_LAUNCH(1);
  else if (iters <= 2) RB_NORM_LAUNCH(2);
  else if (iters <= 4) RB_NORM_LAUNCH(4);
  else if (iters <= 8) RB_NORM_LAUNCH(8);
  else if (iters <= 16) RB_NORM_LAUNCH(16);
  else RB_NORM_LAUNCH(32);
#undef RB_NORM_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

inline int norm_bwd_grid(long long rows) {
  long long blocks = (rows + kNormWarps - 1) / kNormWarps;
  const long long maxb = (long long)rbh::sm_count() * 2;
  if (blocks > maxb) blocks = maxb;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <typename T, bool RMS>
int launch_norm_bwd(const void* x, const void* dy, const void* gamma, const float* stats,
                    const void* dres, void* dx, void* dgamma, void* dbeta, float* partials,
                    int grid, long long rows, int D, cudaStream_t st) {
  constexpr int VEC = Vec16<T>::N;
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int vec = (D % VEC == 0) && al(x) && al(dy) && al(gamma) && al(dres) && al(dx);
  const size_t smem = (size_t)2 * (skew(D) + 1) * sizeof(float);
  auto kern = norm_bwd_kernel<T, RMS>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return 2000 + (int)e;
  }
  kern<<<grid, kNormWarps * 32, smem, st>>>((const T*)x, (const T*)dy, (const T*)gamma, stats,
                                            (const T*)dres, (T*)dx, partials, rows, D, vec);
  norm_bwd_reduce_kernel<T><<<(D + 255) / 256, 256, 0, st>>>(partials, grid, D, (T*)dgamma,
                                                           RMS ? nullptr : (T*)dbeta);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {

// y = norm(x (+res)) ; h_out receives x+res when res != null.  stats [rows,2] fp32 (mean, rstd).
int rb_norm_fwd(int dtype, int rms, const void* x, const void* res, const void* gamma,
                const void* beta, void* y, void* h_out, float* stats, long long rows, int D,
                float eps, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows <= 0) return 0;
#define RB_CALL(T)                                                                               \
  (rms ? launch_norm_fwd<T, true>(x, res, gamma, beta, y, h_out, stats, rows, D, eps, st)       \
       : launch_norm_fwd<T, false>(x, res, gamma, beta, y, h_out, stats, rows, D, eps, st))
  if (dtype == rbh::DT_BF16) return RB_CALL(__nv_bfloat16);
  if (dtype == rbh::DT_F16) return RB_CALL(__half);
  return RB_CALL(float);
#undef RB_CALL
}

// Number of partial rows the backward kernel writes for `rows` rows:
// the caller provides scratch of rb_norm_bwd_partials(rows) * 2 * D floats.
int rb_norm_bwd_partials(long long rows) { return rb::norm_bwd_grid(rows); }

int rb_norm_bwd(int dtype, int rms, const void* x, const void* dy, const void* gamma,
                const float* stats, const void* dres, void* dx, void* dgamma, void* dbeta,
                float* partials, long long rows, int D, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows <= 0) return 0;
  const int grid = norm_bwd_grid(rows);
#define RB_CALL(T)                                                                                 \
  (rms ? launch_norm_bwd<T, true>(x, dy, gamma, stats, dres, dx, dgamma, dbeta, partials, grid,   \
                                  rows, D, st)                                                     \
       : launch_norm_bwd<T, false>(x, dy, gamma, stats, dres, dx, dgamma, dbeta, partials, grid,  \
                                   rows, D, st))
  if (dtype == rbh::DT_BF16) return RB_CALL(__nv_bfloat16);
  if (dtype == rbh::DT_F16) return RB_CALL(__half);
  return RB_CALL(float);
#undef RB_CALL
}
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the norm backward (declared in rumus_b200_noalloc.h)
// ---------------------------------------------------------------------------
#include <mutex>
#include <stdio.h>

#include "rumus_b200_noalloc.h"

namespace {

constexpr int kNoAllocMaxParts = RB_NORM_BWD_NOALLOC_MAX_PARTIALS;
constexpr int kNoAllocMaxDim = RB_NORM_BWD_NOALLOC_MAX_DIM;

// Scratch for the per-CTA (d_gamma, d_beta) partial rows: [parts, 2, D] floats, 2 MiB.
// It lives in the library image, so every GPU that loads the library holds it until exit.
static __device__ __align__(256) float g_norm_bwd_scratch[kNoAllocMaxParts * 2 * kNoAllocMaxDim];

// In host code `g_norm_bwd_scratch` is only a host-side stand-in for the symbol; the device
// address has to be looked up per device (with that device current) and cached.
float* g_noalloc_scratch_addr[16] = {nullptr};
std::mutex g_noalloc_mu;

}  // namespace

extern "C" int rb_norm_bwd_noalloc_max_dim() { return kNoAllocMaxDim; }

extern "C" int rb_norm_bwd_noalloc(int dtype, int rms, const void* x, const void* dy,
                                   const void* gamma, const float* stats, const void* dres,
                                   void* dx, void* dgamma, void* dbeta, long long rows, int D,
                                   void* stream) {
  using namespace rb;
  if (rows <= 0) return 0;
  if (D <= 0 || D > kNoAllocMaxDim) {
    fprintf(stderr,
            "rb_norm_bwd_noalloc: row length %d is outside the built-in scratch (1..%d); use "
            "rb_norm_bwd with caller-provided scratch instead\n",
            D, kNoAllocMaxDim);
    return RB_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return RB_NOALLOC_ERR_DEVICE;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_scratch_addr[dev]) {
      float* p = nullptr;
      cudaError_t e = cudaGetSymbolAddress((void**)&p, g_norm_bwd_scratch);
      if (e != cudaSuccess || p == nullptr) {
        fprintf(stderr, "rb_norm_bwd_noalloc: cudaGetSymbolAddress failed: %s\n",
                cudaGetErrorString(e));
        return RB_NOALLOC_ERR_SYMBOL;
      }
      g_noalloc_scratch_addr[dev] = p;
    }
    scratch = g_noalloc_scratch_addr[dev];
  }
  cudaStream_t st = (cudaStream_t)stream;
  int grid = norm_bwd_grid(rows);
  if (grid > kNoAllocMaxParts) grid = kNoAllocMaxParts;
#define RB_CALL(T)                                                                               \
  (rms ? launch_norm_bwd<T, true>(x, dy, gamma, stats, dres, dx, dgamma, dbeta, scratch, grid,  \
                                  rows, D, st)                                                   \
       : launch_norm_bwd<T, false>(x, dy, gamma, stats, dres, dx, dgamma, dbeta, scratch, grid, \
                                   rows, D, st))
  if (dtype == rbh::DT_BF16) return RB_CALL(__nv_bfloat16);
  if (dtype == rbh::DT_F16) return RB_CALL(__half);
  return RB_CALL(float);
#undef RB_CALL
}
