// Weight-only quantisation kernels for sm_100a.
//
// INT4 (group-wise asymmetric, AWQ/GPTQ-style storage; format of rumus-vision/src/quant.rs:42-126):
//   packed int32 [Kp/8, N], word (k/8)*N + n, nibble k%8; scales / zero-points [Kp/group, N]
//   (fp16 or fp32); w[k,n] = (q - zp) * scale.
//   * int4_gemv: y[M,N] = x[M,K] . dequant(W) for small M (decode): streams the 4-bit weights
//     once at HBM speed, 16-byte loads (4 columns per thread), split-K across CTAs with fp32
//     partials in scratch and a deterministic reduce;
//   * int4_dequant: expands W to a dense 16-bit [K,N] matrix for the tcgen05 GEMM (prefill and
//     the transposed product used in backward).
//   Reference kernels: rumus-vision/src/shaders/qmatmul_int4.wgsl:41 (one thread per output,
//   serial K loop), qmatmul_int4_transpose.wgsl:38.
//
// INT8 block format of rumus/src/backend/gpu/shaders/quantize.wgsl:30 / dequantize.wgsl:33 /
// matmul_q8.wgsl:38: the matrix is laid out column-major, cut into blocks of `bs` values, each
// block = 4-byte header (f16 scale in the low half) + bs int8 values.
#include "sm100_common.cuh"

namespace rb {

template <typename TS>
__device__ __forceinline__ float sc_f32(TS v);
template <>
__device__ __forceinline__ float sc_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float sc_f32<__half>(__half v) { return __half2float(v); }

constexpr int kGemvThreads = 128;
constexpr int kGemvMaxM = 32;

// grid: (ceil(N / (4*128)), splits).  Each thread owns 4 consecutive columns and MT rows of x
// (MT = the launch's row bucket 1/2/4/8/16/32, so the accumulators stay in registers and no work
// is predicated away for small batches).  Per 8 packed k values a thread dequantises its 32
// weights once and then, per row, reads the 8 activations with two 16-byte shared loads and does
// 32 FMAs.
template <typename TX, typename TS, int MT>
__global__ void __launch_bounds__(kGemvThreads)
    int4_gemv_kernel(const TX* __restrict__ x, const int* __restrict__ packed,
                     const TS* __restrict__ scales, const TS* __restrict__ zps,
                     float* __restrict__ partials /* [splits, M, N] */, int M, int N, int K, int Kp,
                     int group, int k8_per_split) {
  extern __shared__ __align__(16) float sx[];  // [M][k8_per_split*8] activations of this split
  const int n0 = (blockIdx.x * kGemvThreads + threadIdx.x) * 4;
  const int k8_begin = blockIdx.y * k8_per_split;
  const int k8_end = min(Kp / 8, k8_begin + k8_per_split);
  const int kspan = k8_per_split * 8;          // row pitch in shared memory (a multiple of 8)
  const int klive = (k8_end - k8_begin) * 8;
  for (int i = threadIdx.x; i < M * klive; i += blockDim.x) {
    const int m = i / klive, kk = i - m * klive;
    const int k = k8_begin * 8 + kk;
    sx[m * kspan + kk] = k < K ? to_f32<TX>(x[(long long)m * K + k]) : 0.f;
  }
  __syncthreads();
  if (n0 >= N) return;
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = 0.f;
  const bool full4 = (n0 + 3 < N) && (N % 4 == 0);
  const int g8 = group / 8;   // packed words per quantisation group (the split is a multiple of it)
  for (int kg = k8_begin; kg < k8_end; kg += g8) {
    const int g = (kg * 8) / group;
    float sc[4], zp[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = min(n0 + j, N - 1);
      sc[j] = sc_f32<TS>(scales[(long long)g * N + n]);
      zp[j] = sc_f32<TS>(zps[(long long)g * N + n]);
    }
    const int kg_end = min(k8_end, kg + g8);
    // four packed rows per trip, loaded before any of them is used: with one load in flight per
    // thread the kernel reached a sixth of the HBM rate at batch 1
    for (int k8 = kg; k8 < kg_end; k8 += 4) {
      int w[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kk = k8 + u;
        if (kk < kg_end && full4) {
          const int4 v = *reinterpret_cast<const int4*>(packed + (long long)kk * N + n0);
          w[u][0] = v.x; w[u][1] = v.y; w[u][2] = v.z; w[u][3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            w[u][j] = (kk < kg_end && n0 + j < N) ? packed[(long long)kk * N + n0 + j] : 0;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (k8 + u >= kg_end) break;
        float wv[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            wv[i][j] = ((float)((static_cast<unsigned>(w[u][j]) >> (4 * i)) & 0xF) - zp[j]) * sc[j];
        const float* xs = sx + (k8 + u - k8_begin) * 8;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m < M) {
            const float4 x0 = *reinterpret_cast<const float4*>(xs + m * kspan);
            const float4 x1 = *reinterpret_cast<const float4*>(xs + m * kspan + 4);
            const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
              for (int j = 0; j < 4; ++j) acc[m][j] = fmaf(xv[i], wv[i][j], acc[m][j]);
          }
        }
      }
    }
  }
  float* out = partials + (long long)blockIdx.y * M * N;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    if (m < M) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + j < N) out[(long long)m * N + n0 + j] = acc[m][j];
    }
  }
}

template <typename TX>
__global__ void gemv_reduce_kernel(const float* __restrict__ partials, int splits, long long MN,
                                   int N, const TX* __restrict__ bias, TX* __restrict__ y) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= MN) return;
  float a = 0.f;
  for (int s = 0; s < splits; ++s) a += partials[(long long)s * MN + i];
  if (bias) a += to_f32<TX>(bias[i % N]);
  y[i] = from_f32<TX>(a);
}

// dense[k, n] = (q - zp) * scale  for k < K
template <typename TO, typename TS>
__global__ void int4_dequant_kernel(const int* __restrict__ packed, const TS* __restrict__ scales,
                                    const TS* __restrict__ zps, TO* __restrict__ dense, int N, int K,
                                    int group) {
  const long long total = (long long)((K + 7) / 8) * N;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int n = (int)(i % N);
    const int k8 = (int)(i / N);
    const unsigned w = static_cast<unsigned>(packed[i]);
    const int g = (k8 * 8) / group;
    const float sc = sc_f32<TS>(scales[(long long)g * N + n]);
    const float zp = sc_f32<TS>(zps[(long long)g * N + n]);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = k8 * 8 + j;
      if (k < K) dense[(long long)k * N + n] = from_f32<TO>(((float)((w >> (4 * j)) & 0xF) - zp) * sc);
    }
  }
}

// 16-bit outputs with N % 8 == 0: one thread dequantises 8 columns x 8 k rows (two 16-byte loads of
// packed words, eight 16-byte stores) instead of one column with 2-byte stores.
template <typename TO, typename TS>
__global__ void int4_dequant_vec8_kernel(const int* __restrict__ packed, const TS* __restrict__ scales,
                                         const TS* __restrict__ zps, TO* __restrict__ dense, int N,
                                         int K, int group) {
  const int N8 = N >> 3;
  const long long total = (long long)((K + 7) / 8) * N8;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int n0 = (int)(i % N8) * 8;
    const int k8 = (int)(i / N8);
    const int4 w0 = *reinterpret_cast<const int4*>(packed + (long long)k8 * N + n0);
    const int4 w1 = *reinterpret_cast<const int4*>(packed + (long long)k8 * N + n0 + 4);
    const unsigned w[8] = {(unsigned)w0.x, (unsigned)w0.y, (unsigned)w0.z, (unsigned)w0.w,
                           (unsigned)w1.x, (unsigned)w1.y, (unsigned)w1.z, (unsigned)w1.w};
    const int g = (k8 * 8) / group;
    float sc[8], zp[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      sc[c] = sc_f32<TS>(scales[(long long)g * N + n0 + c]);
      zp[c] = sc_f32<TS>(zps[(long long)g * N + n0 + c]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int k = k8 * 8 + j;
      if (k < K) {
        uint4 o;
        TO* e = reinterpret_cast<TO*>(&o);
#pragma unroll
        for (int c = 0; c < 8; ++c)
          e[c] = from_f32<TO>(((float)((w[c] >> (4 * j)) & 0xF) - zp[c]) * sc[c]);
        *reinterpret_cast<uint4*>(dense + (long long)k * N + n0) = o;
      }
    }
  }
}

// ---- INT8 blocks -------------------------------------------------------------------------
// src is the [K, N] matrix; block b covers flat column-major elements [b*bs, (b+1)*bs)
template <typename T>
__global__ void q8_quantize_kernel(const T* __restrict__ src, unsigned char* __restrict__ dst, int K,
                                   int N, int bs, long long numel) {
  const long long b = blockIdx.x;
  const long long e0 = b * bs;
  __shared__ float smax[32];
  float mx = 0.f;
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const long long e = e0 + i;
    if (e < numel) {
      const long long n = e / K, k = e % K;
      mx = fmaxf(mx, fabsf(to_f32<T>(src[k * N + n])));
    }
  }
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) smax[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < (blockDim.x >> 5) ? smax[threadIdx.x] : 0.f;
    r = warp_max(r);
    if (threadIdx.x == 0) smax[0] = r;
  }
  __syncthreads();
  const float absmax = smax[0];
  const float scale = absmax == 0.f ? 1.f : absmax / 127.f;
  const float inv = absmax == 0.f ? 0.f : 127.f / absmax;
  unsigned char* out = dst + b * (4 + bs);
  if (threadIdx.x == 0) {
    // 4-byte header: f16 scale in the low half, zero in the high half (blocks are 4-byte aligned)
    *reinterpret_cast<uint32_t*>(out) = (uint32_t)__half_as_ushort(__float2half_rn(scale));
  }
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const long long e = e0 + i;
    int q = 0;
    if (e < numel) {
      const long long n = e / K, k = e % K;
      q = max(-128, min(127, __float2int_rn(to_f32<T>(src[k * N + n]) * inv)));
    }
    out[4 + i] = (unsigned char)(signed char)q;
  }
}
template <typename T>
__global__ void q8_dequantize_kernel(const unsigned char* __restrict__ src, T* __restrict__ dst,
                                     int K, int N, int bs, long long numel) {
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < numel; e += gs) {
    const long long b = e / bs;
    const int i = (int)(e - b * bs);
    const unsigned char* blk = src + b * (4 + bs);
    const unsigned short bits = (unsigned short)blk[0] | ((unsigned short)blk[1] << 8);
    const float scale = __half2float(*reinterpret_cast<const __half*>(&bits));
    const float v = (float)(signed char)blk[4 + i] * scale;
    const long long n = e / K, k = e % K;
    dst[k * N + n] = from_f32<T>(v);
  }
}

}  // namespace rb

extern "C" {

// scratch needed: rb_int4_gemv_splits(K) * M * N floats.
int rb_int4_gemv_splits(int Kp, int N) {
  // enough CTAs to fill the machine: columns give N/512 CTAs, the rest comes from K splits
  const int col_ctas = (N + 511) / 512;
  int want = (2 * rbh::sm_count() + col_ctas - 1) / col_ctas;
  const int k8 = Kp / 8;
  int max_splits = k8 / 16;  // at least 128 rows of K per split
  if (max_splits < 1) max_splits = 1;
  if (want > max_splits) want = max_splits;
  if (want < 1) want = 1;
  return want;
}

int rb_int4_gemv(int x_dtype, int scale_dtype, const void* x, const int* packed, const void* scales,
                 const void* zps, const void* bias, void* y, float* scratch, int M, int N, int K,
                 int Kp, int group, void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if (M > kGemvMaxM) return 50;
  cudaStream_t st = (cudaStream_t)stream;
  const int splits = rb_int4_gemv_splits(Kp, N);
  int k8_per_split = (Kp / 8 + splits - 1) / splits;
  // keep splits aligned to groups so a thread's (scale, zp) cache changes at most once per group
  const int g8 = group / 8;
  k8_per_split = (k8_per_split + g8 - 1) / g8 * g8;
  const int real_splits = (Kp / 8 + k8_per_split - 1) / k8_per_split;
  dim3 grid((N + 4 * kGemvThreads - 1) / (4 * kGemvThreads), real_splits);
  const size_t smem = (size_t)M * k8_per_split * 8 * sizeof(float);
#define RB_GEMV_MT(TX, TS, MT_)                                                                   \
  do {                                                                                           \
    auto kern = int4_gemv_kernel<TX, TS, MT_>;                                                   \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    kern<<<grid, kGemvThreads, smem, st>>>((const TX*)x, packed, (const TS*)scales, (const TS*)zps, \
                                           scratch, M, N, K, Kp, group, k8_per_split);           \
  } while (0)
#define RB_GEMV(TX, TS)                                                                          \
  do {                                                                                           \
    if (M <= 1) RB_GEMV_MT(TX, TS, 1);                                                           \
    else if (M <= 2) RB_GEMV_MT(TX, TS, 2);                                                      \
    else if (M <= 4) RB_GEMV_MT(TX, TS, 4);                                                      \
    else if (M <= 8) RB_GEMV_MT(TX, TS, 8);                                                      \
    else if (M <= 16) RB_GEMV_MT(TX, TS, 16);                                                    \
    else RB_GEMV_MT(TX, TS, 32);                                                                 \
    gemv_reduce_kernel<TX><<<(unsigned)(((long long)M * N + 255) / 256), 256, 0, st>>>(          \
        scratch, real_splits, (long long)M * N, N, (const TX*)bias, (TX*)y);                     \
  } while (0)
  if (x_dtype == rbh::DT_BF16) {
    if (scale_dtype == rbh::DT_F16) RB_GEMV(__nv_bfloat16, __half); else RB_GEMV(__nv_bfloat16, float);
  } else if (x_dtype == rbh::DT_F16) {
    if (scale_dtype == rbh::DT_F16) RB_GEMV(__half, __half); else RB_GEMV(__half, float);
  } else {
    if (scale_dtype == rbh::DT_F16) RB_GEMV(float, __half); else RB_GEMV(float, float);
  }
#undef RB_GEMV_MT
#undef RB_GEMV
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_int4_dequant(int out_dtype, int scale_dtype, const int* packed, const void* scales,
                    const void* zps, void* dense, int N, int K, int group, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long total = (long long)((K + 7) / 8) * N;
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)rbh::sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (out_dtype != rbh::DT_F32 && N % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(dense)) & 15) == 0) {
    long long b8 = (total / 8 + 255) / 256;
    if (b8 > cap) b8 = cap;
    if (b8 < 1) b8 = 1;
#define RB_DQ8(TO, TS) int4_dequant_vec8_kernel<TO, TS><<<(unsigned)b8, 256, 0, st>>>(packed, (const TS*)scales, (const TS*)zps, (TO*)dense, N, K, group)
    if (out_dtype == rbh::DT_BF16) { if (scale_dtype == rbh::DT_F16) RB_DQ8(__nv_bfloat16, __half); else RB_DQ8(__nv_bfloat16, float); }
    else { if (scale_dtype == rbh::DT_F16) RB_DQ8(__half, __half); else RB_DQ8(__half, float); }
#undef RB_DQ8
    cudaError_t e8 = cudaGetLastError();
    return e8 == cudaSuccess ? 0 : 3000 + (int)e8;
  }
#define RB_DQ(TO, TS) int4_dequant_kernel<TO, TS><<<(unsigned)blocks, 256, 0, st>>>(packed, (const TS*)scales, (const TS*)zps, (TO*)dense, N, K, group)
  if (out_dtype == rbh::DT_BF16) { if (scale_dtype == rbh::DT_F16) RB_DQ(__nv_bfloat16, __half); else RB_DQ(__nv_bfloat16, float); }
  else if (out_dtype == rbh::DT_F16) { if (scale_dtype == rbh::DT_F16) RB_DQ(__half, __half); else RB_DQ(__half, float); }
  else { if (scale_dtype == rbh::DT_F16) RB_DQ(float, __half); else RB_DQ(float, float); }
#undef RB_DQ
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_q8_quantize(int dtype, const void* src, unsigned char* dst, int K, int N, int bs, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long numel = (long long)K * N;
  const long long nb = (numel + bs - 1) / bs;
  if (nb <= 0) return 0;
  if (dtype == rbh::DT_BF16) q8_quantize_kernel<__nv_bfloat16><<<(unsigned)nb, 64, 0, st>>>((const __nv_bfloat16*)src, dst, K, N, bs, numel);
  else if (dtype == rbh::DT_F16) q8_quantize_kernel<__half><<<(unsigned)nb, 64, 0, st>>>((const __half*)src, dst, K, N, bs, numel);
  else q8_quantize_kernel<float><<<(unsigned)nb, 64, 0, st>>>((const float*)src, dst, K, N, bs, numel);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
int rb_q8_dequantize(int dtype, const unsigned char* src, void* dst, int K, int N, int bs, void* stream) {
  using namespace rb;
  cudaStream_t st = (cudaStream_t)stream;
  const long long numel = (long long)K * N;
  if (numel <= 0) return 0;
  long long blocks = (numel + 255) / 256;
  const long long cap = (long long)rbh::sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (dtype == rbh::DT_BF16) q8_dequantize_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(src, (__nv_bfloat16*)dst, K, N, bs, numel);
  else if (dtype == rbh::DT_F16) q8_dequantize_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(src, (__half*)dst, K, N, bs, numel);
  else q8_dequantize_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(src, (float*)dst, K, N, bs, numel);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
