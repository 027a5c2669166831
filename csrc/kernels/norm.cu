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

// Column-owner variant used when rows are 16-byte vectors and D <= 128 * VEC * NCHUNK: a group of
// 128 threads works on one row, thread t owning the 16-byte chunks t, t+128, ... of every row
// the group visits.  x and dy stay in registers between the two row reductions and the dx pass,
// and d_gamma / d_beta accumulate in registers (no shared-memory atomics); the four groups of a
// CTA fold their accumulators through shared memory once at the end.
constexpr int kColGroupThreads = 128;

// kColGroups row groups per CTA: 4 while the accumulators fit 128 registers, 2 for wider rows
template <typename T, bool RMS, int NCHUNK, int kColGroups>
__global__ void __launch_bounds__(kColGroups* kColGroupThreads)
    norm_bwd_cols_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                         const T* __restrict__ gamma, const float* __restrict__ stats,
                         const T* __restrict__ dres, T* __restrict__ dx,
                         float* __restrict__ partials /* [grid,2,D] */, long long rows, int D) {
  constexpr int VEC = Vec16<T>::N;
  extern __shared__ float s_fold[];                       // [2][D]
  __shared__ float s_red[2][kColGroups][4][2];            // [buffer][group][warp][c1,c2]
  const int grp = threadIdx.x / kColGroupThreads;
  const int tg = threadIdx.x % kColGroupThreads;
  const int wg = tg >> 5, lane = tg & 31;
  float acc_g[NCHUNK][VEC], acc_b[NCHUNK][VEC];
  Vec16<T> gv[NCHUNK];
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int c = (i * kColGroupThreads + tg) * VEC;
    gv[i].raw = c < D ? *reinterpret_cast<const uint4*>(gamma + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc_g[i][j] = acc_b[i][j] = 0.f;
  }
  const float inv_d = 1.f / (float)D;
  int buf = 0;
  const long long row_step = (long long)gridDim.x * kColGroups;
  // every group runs the same number of trips so that the named barrier below stays matched
  const long long trips = (rows + row_step - 1) / row_step;
  // software pipeline: the next row's x / dy are requested before the current row is reduced
  Vec16<T> xn[NCHUNK], dn[NCHUNK];
  auto fetch = [&](long long row) {
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int c = (i * kColGroupThreads + tg) * VEC;
      if (row < rows && c < D) {
        xn[i].raw = *reinterpret_cast<const uint4*>(x + row * D + c);
        dn[i].raw = *reinterpret_cast<const uint4*>(dy + row * D + c);
      } else {
        xn[i].raw = make_uint4(0, 0, 0, 0);
        dn[i].raw = make_uint4(0, 0, 0, 0);
      }
    }
  };
  fetch((long long)blockIdx.x * kColGroups + grp);
  for (long long trip = 0; trip < trips; ++trip) {
    const long long row = trip * row_step + (long long)blockIdx.x * kColGroups + grp;
    const bool live = row < rows;
    Vec16<T> xv[NCHUNK], dv[NCHUNK];
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      xv[i] = xn[i];
      dv[i] = dn[i];
    }
    if (trip + 1 < trips) fetch(row + row_step);
    float mean = 0.f, rstd = 0.f;
    if (live) {
      mean = RMS ? 0.f : stats[row * 2];
      rstd = stats[row * 2 + 1];
    }
    float c1 = 0.f, c2 = 0.f;  // sum(dy*g), sum(dy*g*xhat)
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i)
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float xh = (xv[i].get(j) - mean) * rstd;
        const float dg = dv[i].get(j) * gv[i].get(j);
        c1 += dg;
        c2 += dg * xh;
      }
    c1 = warp_sum(c1);
    c2 = warp_sum(c2);
    if (lane == 0) {
      s_red[buf][grp][wg][0] = c1;
      s_red[buf][grp][wg][1] = c2;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(kColGroupThreads) : "memory");
    c1 = (s_red[buf][grp][0][0] + s_red[buf][grp][1][0] + s_red[buf][grp][2][0] +
          s_red[buf][grp][3][0]) * inv_d;
    c2 = (s_red[buf][grp][0][1] + s_red[buf][grp][1][1] + s_red[buf][grp][2][1] +
          s_red[buf][grp][3][1]) * inv_d;
    buf ^= 1;
    if (RMS) c1 = 0.f;
    if (live) {
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int c = (i * kColGroupThreads + tg) * VEC;
        if (c < D) {
          Vec16<T> rv, ov;
          if (dres) rv.raw = *reinterpret_cast<const uint4*>(dres + row * D + c);
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            const float xh = (xv[i].get(j) - mean) * rstd;
            const float d = dv[i].get(j);
            float o = rstd * (d * gv[i].get(j) - c1 - xh * c2);
            if (dres) o += rv.get(j);
            ov.set(j, o);
            acc_g[i][j] += d * xh;
            acc_b[i][j] += d;
          }
          *reinterpret_cast<uint4*>(dx + row * D + c) = ov.raw;
        }
      }
    }
  }
  // fold the four groups: group 0 stores, the others add in turn
  for (int gsel = 0; gsel < kColGroups; ++gsel) {
    if (grp == gsel) {
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int c = (i * kColGroupThreads + tg) * VEC;
        if (c < D) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            if (gsel == 0) {
              s_fold[c + j] = acc_g[i][j];
              s_fold[D + c + j] = acc_b[i][j];
            } else {
              s_fold[c + j] += acc_g[i][j];
              s_fold[D + c + j] += acc_b[i][j];
            }
          }
        }
      }
    }
    __syncthreads();
  }
  float* out = partials + (long long)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) out[i] = s_fold[i];
}

// Ring variant of the column-owner kernel: the rows a group will visit next are already on their way
// into shared memory (untiled bulk copies completing on an mbarrier: x, dy and the residual-stream
// gradient of `stages` rows per group), so the bytes in flight are bounded by shared memory (~190 KB per
// SM), not by the registers a thread can spare for prefetched rows (the register-prefetch form above
// keeps 8 KB per group in flight and loads the residual gradient late, which held it at 2.6-2.8 TB/s).
// One persistent CTA per SM; thread / chunk ownership, the two row reductions and the register-resident
// d_gamma / d_beta accumulators are the same as in norm_bwd_cols_kernel.
template <typename T, bool RMS, int NCHUNK, int kColGroups>
__global__ void __launch_bounds__(kColGroups* kColGroupThreads)
    norm_bwd_ring_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                         const T* __restrict__ gamma, const float* __restrict__ stats,
                         const T* __restrict__ dres, T* __restrict__ dx,
                         float* __restrict__ partials /* [grid,2,D] */, long long rows, int D,
                         int stages, int* status) {
  constexpr int VEC = Vec16<T>::N;
  extern __shared__ uint8_t ring_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ring_raw) + 127) & ~static_cast<uintptr_t>(127));
  const int row_bytes = D * (int)sizeof(T);
  const int stage_bytes = 3 * row_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)kColGroups * stages * stage_bytes);   // [group][stage]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kColGroups * stages);
  __shared__ float s_red[2][kColGroups][4][2];            // [buffer][group][warp][c1,c2]
  __shared__ int s_stop[2][kColGroups];                   // the abort flag as one thread of the group saw it
  const int grp = threadIdx.x / kColGroupThreads;
  const int tg = threadIdx.x % kColGroupThreads;
  const int wg = tg >> 5, lane = tg & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kColGroups * stages; ++i) mbar_init(smem_u32(&bars[i]), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  uint8_t* my_ring = ring + (size_t)grp * stages * stage_bytes;
  uint64_t* my_bars = bars + grp * stages;
  const long long row_step = (long long)gridDim.x * kColGroups;
  const long long first = (long long)blockIdx.x * kColGroups + grp;
  // every group runs the same number of trips so that the named barrier below stays matched
  const long long trips = (rows + row_step - 1) / row_step;
  auto request = [&](long long row, int stage) {       // one thread per group
    const uint32_t bar = smem_u32(&my_bars[stage]);
    uint8_t* dst = my_ring + (size_t)stage * stage_bytes;
    mbar_arrive_expect_tx(bar, (dres ? 3 : 2) * row_bytes);
    bulk_load_1d(smem_u32(dst), x + row * D, row_bytes, bar);
    bulk_load_1d(smem_u32(dst + row_bytes), dy + row * D, row_bytes, bar);
    if (dres) bulk_load_1d(smem_u32(dst + 2 * row_bytes), dres + row * D, row_bytes, bar);
  };
  long long requested = 0;                              // trips whose copies were issued (thread tg == 0)
  if (tg == 0) {
    for (int s0 = 0; s0 < stages; ++s0) {
      const long long row = first + s0 * row_step;
      if (row < rows) {
        request(row, s0);
        requested = s0 + 1;
      }
    }
  }
  float acc_g[NCHUNK][VEC], acc_b[NCHUNK][VEC];
  Vec16<T> gv[NCHUNK];
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int c = (i * kColGroupThreads + tg) * VEC;
    gv[i].raw = c < D ? *reinterpret_cast<const uint4*>(gamma + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc_g[i][j] = acc_b[i][j] = 0.f;
  }
  const float inv_d = 1.f / (float)D;
  int buf = 0, stage = 0;
  uint32_t phase = 0;
  long long trip = 0;
  for (; trip < trips; ++trip) {
    const long long row = trip * row_step + first;
    const bool live = row < rows;
    Vec16<T> xv[NCHUNK], dv[NCHUNK], rv[NCHUNK];
    float mean = 0.f, rstd = 0.f;
    if (live) {
      mean = RMS ? 0.f : stats[row * 2];
      rstd = stats[row * 2 + 1];
      mbar_wait(smem_u32(&my_bars[stage]), phase, abort_flag, status, RB_ERR_TIMEOUT_FULL);
      const uint8_t* src = my_ring + (size_t)stage * stage_bytes;
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int c = (i * kColGroupThreads + tg) * VEC;
        if (c < D) {
          xv[i].raw = *reinterpret_cast<const uint4*>(src + (size_t)c * sizeof(T));
          dv[i].raw = *reinterpret_cast<const uint4*>(src + row_bytes + (size_t)c * sizeof(T));
          rv[i].raw = dres ? *reinterpret_cast<const uint4*>(src + 2 * row_bytes + (size_t)c * sizeof(T))
                           : make_uint4(0, 0, 0, 0);
        } else {
          xv[i].raw = dv[i].raw = rv[i].raw = make_uint4(0, 0, 0, 0);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) xv[i].raw = dv[i].raw = rv[i].raw = make_uint4(0, 0, 0, 0);
    }
    float c1 = 0.f, c2 = 0.f;  // sum(dy*g), sum(dy*g*xhat)
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i)
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float xh = (xv[i].get(j) - mean) * rstd;
        const float dg = dv[i].get(j) * gv[i].get(j);
        c1 += dg;
        c2 += dg * xh;
      }
    c1 = warp_sum(c1);
    c2 = warp_sum(c2);
    if (lane == 0) {
      s_red[buf][grp][wg][0] = c1;
      s_red[buf][grp][wg][1] = c2;
    }
    if (tg == 0) s_stop[buf][grp] = *abort_flag;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(kColGroupThreads) : "memory");
    // after a wait that ran out the group leaves together: every thread acts on the one reading of the
    // flag taken before the barrier (a thread that reads the flag for itself could leave alone and
    // strand the others at the next barrier); a flag raised later is seen one row later
    if (s_stop[buf][grp]) break;
    // every thread of the group has taken its part of this stage: it can receive a later row
    if (tg == 0 && live) {
      const long long next = row + (long long)stages * row_step;
      if (next < rows) {
        request(next, stage);
        requested = trip + stages + 1;
      }
    }
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
    }
    c1 = (s_red[buf][grp][0][0] + s_red[buf][grp][1][0] + s_red[buf][grp][2][0] +
          s_red[buf][grp][3][0]) * inv_d;
    c2 = (s_red[buf][grp][0][1] + s_red[buf][grp][1][1] + s_red[buf][grp][2][1] +
          s_red[buf][grp][3][1]) * inv_d;
    buf ^= 1;
    if (RMS) c1 = 0.f;
    if (live) {
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int c = (i * kColGroupThreads + tg) * VEC;
        if (c < D) {
          Vec16<T> ov;
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            const float xh = (xv[i].get(j) - mean) * rstd;
            const float d = dv[i].get(j);
            float o = rstd * (d * gv[i].get(j) - c1 - xh * c2);
            if (dres) o += rv[i].get(j);
            ov.set(j, o);
            acc_g[i][j] += d * xh;
            acc_b[i][j] += d;
          }
          *reinterpret_cast<uint4*>(dx + row * D + c) = ov.raw;
        }
      }
    }
  }
  // after a failed wait: give the copies still in flight their time before the ring is reused below
  if (tg == 0 && trip < trips) {
    for (long long t2 = trip; t2 < requested; ++t2)
      mbar_drain(smem_u32(&my_bars[t2 % stages]), (uint32_t)((t2 / stages) & 1), status);
  }
  __syncthreads();
  // fold the groups through the (now idle) ring: group 0 stores, the others add in turn
  float* s_fold = reinterpret_cast<float*>(ring);
  for (int gsel = 0; gsel < kColGroups; ++gsel) {
    if (grp == gsel) {
#pragma unroll
      for (int i = 0; i < NCHUNK; ++i) {
        const int c = (i * kColGroupThreads + tg) * VEC;
        if (c < D) {
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            if (gsel == 0) {
              s_fold[c + j] = acc_g[i][j];
              s_fold[D + c + j] = acc_b[i][j];
            } else {
              s_fold[c + j] += acc_g[i][j];
              s_fold[D + c + j] += acc_b[i][j];
            }
          }
        }
      }
    }
    __syncthreads();
  }
  float* out = partials + (long long)blockIdx.x * 2 * D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) out[i] = s_fold[i];
}

// partials [n,2,D] -> dgamma[D], dbeta[D] (dbeta may be null)
template <typename T>
__global__ void __launch_bounds__(256)
    norm_bwd_reduce_kernel(const float* __restrict__ partials, int n, int D,
                           T* __restrict__ dgamma, T* __restrict__ dbeta) {
  // 32 columns x 8 row slices per CTA: each slice strides over the partial rows, then the
  // slices fold through shared memory
  __shared__ float sg[8][33], sb[8][33];
  const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float g = 0.f, b = 0.f;
  if (c < D) {
    for (int i = slice; i < n; i += 8) {
      g += partials[(long long)i * 2 * D + c];
      b += partials[(long long)i * 2 * D + D + c];
    }
  }
  sg[slice][cx] = g;
  sb[slice][cx] = b;
  __syncthreads();
  if (slice == 0 && c < D) {
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      g += sg[k][cx];
      b += sb[k][cx];
    }
    dgamma[c] = from_f32<T>(g);
    if (dbeta) dbeta[c] = from_f32<T>(b);
  }
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
  const int chunks = (D + kColGroupThreads * VEC - 1) / (kColGroupThreads * VEC);
  if (vec && chunks <= 4) {
    // ring kernel: one persistent CTA per SM, `stages` rows per group in flight in shared memory
    const int groups = chunks <= 2 ? 4 : 2;
    const int row_bytes = D * (int)sizeof(T);
    int stages = (200 * 1024) / (groups * 3 * row_bytes);
    if (stages > 8) stages = 8;
    static const bool ring_on = [] {
      const char* e = getenv("RB_NORM_RING");
      return !(e && e[0] == '0');
    }();
    if (ring_on && stages >= 2) {
      if (grid > rbh::sm_count()) grid = rbh::sm_count();
      const size_t smem = (size_t)groups * stages * 3 * row_bytes + (size_t)groups * stages * 8 + 16 + 128;
      cudaError_t e1 = cudaSuccess;
#define RB_RING(N, G)                                                                                      \
  do {                                                                                                     \
    auto k = norm_bwd_ring_kernel<T, RMS, N, G>;                                                           \
    e1 = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
    if (e1 == cudaSuccess)                                                                                 \
      k<<<grid, G * kColGroupThreads, smem, st>>>((const T*)x, (const T*)dy, (const T*)gamma, stats,       \
                                                  (const T*)dres, (T*)dx, partials, rows, D, stages,       \
                                                  rbh::device_status_word());                              \
  } while (0)
      if (chunks == 1) RB_RING(1, 4);
      else if (chunks == 2) RB_RING(2, 4);
      else if (chunks == 3) RB_RING(3, 2);
      else RB_RING(4, 2);
#undef RB_RING
      if (e1 != cudaSuccess) return 2000 + (int)e1;
      norm_bwd_reduce_kernel<T><<<(D + 31) / 32, 256, 0, st>>>(partials, grid, D, (T*)dgamma,
                                                               RMS ? nullptr : (T*)dbeta);
      cudaError_t e2 = cudaGetLastError();
      return e2 == cudaSuccess ? 0 : 3000 + (int)e2;
    }
    const size_t fold = (size_t)2 * D * sizeof(float);
#define RB_COLS(N, G)                                                                            \
  norm_bwd_cols_kernel<T, RMS, N, G><<<grid, G * kColGroupThreads, fold, st>>>(                  \
      (const T*)x, (const T*)dy, (const T*)gamma, stats, (const T*)dres, (T*)dx, partials, rows, D)
    if (chunks == 1) RB_COLS(1, 4);
    else if (chunks == 2) RB_COLS(2, 4);
    else if (chunks == 3) RB_COLS(3, 2);
    else RB_COLS(4, 2);
#undef RB_COLS
    norm_bwd_reduce_kernel<T><<<(D + 31) / 32, 256, 0, st>>>(partials, grid, D, (T*)dgamma,
                                                             RMS ? nullptr : (T*)dbeta);
    cudaError_t e2 = cudaGetLastError();
    return e2 == cudaSuccess ? 0 : 3000 + (int)e2;
  }
  const size_t smem = (size_t)2 * (skew(D) + 1) * sizeof(float);
  auto kern = norm_bwd_kernel<T, RMS>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return 2000 + (int)e;
  }
  kern<<<grid, kNormWarps * 32, smem, st>>>((const T*)x, (const T*)dy, (const T*)gamma, stats,
                                            (const T*)dres, (T*)dx, partials, rows, D, vec);
  norm_bwd_reduce_kernel<T><<<(D + 31) / 32, 256, 0, st>>>(partials, grid, D, (T*)dgamma,
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
