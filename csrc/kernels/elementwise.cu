// Pointwise and gather/scatter kernels for sm_100a: activations (+ backward),
// SwiGLU, binary ops, scale, dtype casts, dropout, embedding gather /
// scatter-add, rotary position embedding, bias-gradient column sums.
//
// Reference counterparts: rumus/src/backend/gpu/shaders/{elementwise,unary,
// activations,cast,fused_dropout,embedding,bias,fused_scale}.wgsl — most of
// which the reference never dispatches (it runs the CPU loops in
// rumus/src/backend/cpu.rs instead); here they all run on the device with
// 128-bit accesses and grid-stride loops.
#include "sm100_common.cuh"

namespace rb {

enum : int {
  UN_RELU = 1, UN_GELU = 2, UN_SILU = 3, UN_SIGMOID = 4, UN_TANH = 5, UN_LEAKY = 6, UN_SCALE = 7,
  UN_COPY = 8,
};
enum : int { BIN_ADD = 1, BIN_SUB = 2, BIN_MUL = 3 };

__device__ __forceinline__ float unary_f(float x, int op, float a) {
  switch (op) {
    case UN_RELU: return fmaxf(x, 0.f);
    case UN_GELU: return gelu_tanh(x);
    case UN_SILU: return silu_f(x);
    case UN_SIGMOID: return 1.f / (1.f + __expf(-x));
    case UN_TANH: return tanhf(x);
    case UN_LEAKY: return x > 0.f ? x : a * x;
    case UN_SCALE: return a * x;
    default: return x;
  }
}
// derivative w.r.t. the *input* x
__device__ __forceinline__ float unary_grad(float x, int op, float a) {
  switch (op) {
    case UN_RELU: return x > 0.f ? 1.f : 0.f;
    case UN_GELU: return gelu_tanh_grad(x);
    case UN_SILU: return silu_grad(x);
    case UN_SIGMOID: { float s = 1.f / (1.f + __expf(-x)); return s * (1.f - s); }
    case UN_TANH: { float t = tanhf(x); return 1.f - t * t; }
    case UN_LEAKY: return x > 0.f ? 1.f : a;
    case UN_SCALE: return a;
    default: return 1.f;
  }
}

template <typename TI, typename TO>
__global__ void unary_kernel(const TI* __restrict__ x, TO* __restrict__ y, long long n, int op,
                             float a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = from_f32<TO>(unary_f(to_f32<TI>(x[i]), op, a));
}
// dx = dy * f'(x)
template <typename T>
__global__ void unary_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                 T* __restrict__ dx, long long n, int op, float a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = from_f32<T>(to_f32<T>(dy[i]) * unary_grad(to_f32<T>(x[i]), op, a));
}
template <typename T>
__global__ void binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y,
                              long long n, int op, float alpha) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float u = to_f32<T>(a[i]), v = to_f32<T>(b[i]) * alpha;
    y[i] = from_f32<T>(op == BIN_ADD ? u + v : op == BIN_SUB ? u - v : u * v);
  }
}

// SwiGLU on a fused [rows, 2*F] gate|up buffer:  y = silu(gate) * up
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ y, long long rows, int F,
                                  long long ld) {
  const long long n = rows * F;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = i / F;
    const int c = (int)(i - r * F);
    float g = to_f32<T>(gu[r * ld + c]), u = to_f32<T>(gu[r * ld + F + c]);
    y[i] = from_f32<T>(silu_f(g) * u);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dy,
                                  T* __restrict__ dgu, long long rows, int F, long long ld) {
  const long long n = rows * F;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = i / F;
    const int c = (int)(i - r * F);
    float g = to_f32<T>(gu[r * ld + c]), u = to_f32<T>(gu[r * ld + F + c]);
    float d = to_f32<T>(dy[i]);
    dgu[r * ld + c] = from_f32<T>(d * u * silu_grad(g));
    dgu[r * ld + F + c] = from_f32<T>(d * silu_f(g));
  }
}

// PCG hash dropout (same generator as rumus/src/backend/gpu/shaders/fused_dropout.wgsl:22-27):
// keep when hash(seed ^ i) >= p * 2^32; kept values are scaled by 1/(1-p).  The mask is
// recomputed in backward from (seed, i) instead of being stored.
__device__ __forceinline__ uint32_t pcg_hash(uint32_t v) {
  uint32_t state = v * 747796405u + 2891336453u;
  uint32_t word = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
  return (word >> 22u) ^ word;
}
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n,
                               uint32_t seed, uint32_t threshold, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const bool keep = pcg_hash(seed ^ (uint32_t)i) >= threshold;
    y[i] = from_f32<T>(keep ? to_f32<T>(x[i]) * scale : 0.f);
  }
}

// embedding gather: out[t, :] = W[idx[t], :] (+ pos[t % S, :])
template <typename T>
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx, const T* __restrict__ W,
                                     const T* __restrict__ pos, T* __restrict__ out,
                                     long long tokens, int D, int S, int vocab) {
  constexpr int VEC = 16 / sizeof(T);
  const int vecs = D / VEC;
  const long long n = tokens * vecs;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long t = i / vecs;
    const int c = (int)(i - t * vecs) * VEC;
    long long row = idx[t];
    row = row < 0 ? 0 : (row >= vocab ? vocab - 1 : row);
    uint4 w = *reinterpret_cast<const uint4*>(W + row * D + c);
    if (pos) {
      uint4 pv = *reinterpret_cast<const uint4*>(pos + (t % S) * D + c);
      T* we = reinterpret_cast<T*>(&w);
      const T* pe = reinterpret_cast<const T*>(&pv);
#pragma unroll
      for (int j = 0; j < VEC; ++j) we[j] = from_f32<T>(to_f32<T>(we[j]) + to_f32<T>(pe[j]));
    }
    *reinterpret_cast<uint4*>(out + t * D + c) = w;
  }
}
template <typename T>
__global__ void embedding_fwd_scalar_kernel(const long long* __restrict__ idx,
                                            const T* __restrict__ W, const T* __restrict__ pos,
                                            T* __restrict__ out, long long tokens, int D, int S,
                                            int vocab) {
  const long long n = tokens * D;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long t = i / D;
    const int c = (int)(i - t * D);
    long long row = idx[t];
    row = row < 0 ? 0 : (row >= vocab ? vocab - 1 : row);
    float v = to_f32<T>(W[row * D + c]);
    if (pos) v += to_f32<T>(pos[(t % S) * D + c]);
    out[i] = from_f32<T>(v);
  }
}
// scatter-add into an fp32 gradient table (dW32 must be zeroed by the caller);
// dpos32 (optional) accumulates the positional-embedding gradient.
template <typename T>
__global__ void embedding_bwd_kernel(const long long* __restrict__ idx, const T* __restrict__ dout,
                                     float* __restrict__ dW32, float* __restrict__ dpos32,
                                     long long tokens, int D, int S, int vocab) {
  const long long n = tokens * D;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long t = i / D;
    const int c = (int)(i - t * D);
    long long row = idx[t];
    if (row < 0 || row >= vocab) continue;
    const float g = to_f32<T>(dout[i]);
    atomicAdd(&dW32[row * D + c], g);
    if (dpos32) atomicAdd(&dpos32[(t % S) * D + c], g);
  }
}

// Rotary embedding applied in place to q and k living inside a fused buffer.
// x: [tokens, ld] ; heads at column offset `col0 + h*hd`; pairs (i, i + hd/2)  (NeoX / Llama layout)
// position of token t = pos_ids ? pos_ids[t] : t % S.  sign = +1 forward, -1 backward (inverse rotation).
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const long long* __restrict__ pos_ids,
                            long long tokens, int S, int heads, int hd, long long ld, int col0,
                            float theta, float sign) {
  const int half = hd / 2;
  const long long n = tokens * heads * half;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int p = (int)(i % half);
    const long long th = i / half;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    const float posf = (float)(pos_ids ? pos_ids[t] : (t % S));
    const float inv_freq = __powf(theta, -2.0f * (float)p / (float)hd);
    float sn, cs;
    sincosf(posf * inv_freq, &sn, &cs);
    sn *= sign;
    T* base = x + t * ld + col0 + h * hd;
    const float a = to_f32<T>(base[p]), b = to_f32<T>(base[p + half]);
    base[p] = from_f32<T>(a * cs - b * sn);
    base[p + half] = from_f32<T>(b * cs + a * sn);
  }
}

// column sums of a [rows, N] matrix (bias gradient): out[c] = sum_r x[r, c]
// two-stage: grid.y slabs of rows write partials [slabs, N], then reduce.
template <typename T>
__global__ void colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ partials,
                                      long long rows, int N, long long ld, int rows_per_slab) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  const long long r0 = (long long)blockIdx.y * rows_per_slab;
  const long long r1 = min(rows, r0 + rows_per_slab);
  float acc = 0.f;
  for (long long r = r0; r < r1; ++r) acc += to_f32<T>(x[r * ld + c]);
  partials[(long long)blockIdx.y * N + c] = acc;
}
// vector variant: each thread owns VEC consecutive columns (16-byte loads), 4 rows in flight
template <typename T>
__global__ void __launch_bounds__(128)
    colsum_partial_vec_kernel(const T* __restrict__ x, float* __restrict__ partials, long long rows,
                              int N, long long ld, int rows_per_slab) {
  constexpr int VEC = 16 / sizeof(T);
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= N) return;
  const long long r0 = (long long)blockIdx.y * rows_per_slab;
  const long long r1 = min(rows, r0 + rows_per_slab);
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  long long r = r0;
  for (; r + 4 <= r1; r += 4) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(x + (r + u) * ld + c);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += to_f32<T>(e[j]);
    }
  }
  for (; r < r1; ++r) {
    uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + c);
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] += to_f32<T>(e[j]);
  }
  float* out = partials + (long long)blockIdx.y * N + c;
#pragma unroll
  for (int j = 0; j < VEC; ++j) out[j] = acc[j];
}
template <typename T>
__global__ void __launch_bounds__(256)
    colsum_final_kernel(const float* __restrict__ partials, int slabs, int N, T* __restrict__ out) {
  // 32 columns x 8 slab slices per CTA, folded through shared memory
  __shared__ float sa[8][33];
  const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (c < N)
    for (int s = slice; s < slabs; s += 8) acc += partials[(long long)s * N + c];
  sa[slice][cx] = acc;
  __syncthreads();
  if (slice == 0 && c < N) {
#pragma unroll
    for (int k = 1; k < 8; ++k) acc += sa[k][cx];
    out[c] = from_f32<T>(acc);
  }
}

inline unsigned ew_grid(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)rbh::sm_count() * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

}  // namespace rb

#define RB_DISPATCH_T(dtype, CALL)                 \
  if ((dtype) == rbh::DT_BF16) { using T = __nv_bfloat16; CALL; }      \
  else if ((dtype) == rbh::DT_F16) { using T = __half; CALL; }         \
  else { using T = float; CALL; }

#define RB_RET_LAST()                                   \
  do {                                                  \
    cudaError_t e__ = cudaGetLastError();               \
    return e__ == cudaSuccess ? 0 : 3000 + (int)e__;    \
  } while (0)

extern "C" {

int rb_unary(int dtype, const void* x, void* y, long long n, int op, float a, void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  RB_DISPATCH_T(dtype, (unary_kernel<T, T><<<ew_grid(n, 256), 256, 0, st>>>((const T*)x, (T*)y, n, op, a)));
  RB_RET_LAST();
}
int rb_unary_bwd(int dtype, const void* x, const void* dy, void* dx, long long n, int op, float a,
                 void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  RB_DISPATCH_T(dtype, (unary_bwd_kernel<T><<<ew_grid(n, 256), 256, 0, st>>>((const T*)x, (const T*)dy, (T*)dx, n, op, a)));
  RB_RET_LAST();
}
int rb_binary(int dtype, const void* a, const void* b, void* y, long long n, int op, float alpha,
              void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  RB_DISPATCH_T(dtype, (binary_kernel<T><<<ew_grid(n, 256), 256, 0, st>>>((const T*)a, (const T*)b, (T*)y, n, op, alpha)));
  RB_RET_LAST();
}
// dtype cast with optional scale: y = scale * x
int rb_cast(int src_dtype, int dst_dtype, const void* x, void* y, long long n, float scale,
            void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned g = ew_grid(n, 256);
#define RB_CAST(TI, TO) unary_kernel<TI, TO><<<g, 256, 0, st>>>((const TI*)x, (TO*)y, n, UN_SCALE, scale)
  if (src_dtype == rbh::DT_F32 && dst_dtype == rbh::DT_BF16) RB_CAST(float, __nv_bfloat16);
  else if (src_dtype == rbh::DT_F32 && dst_dtype == rbh::DT_F16) RB_CAST(float, __half);
  else if (src_dtype == rbh::DT_BF16 && dst_dtype == rbh::DT_F32) RB_CAST(__nv_bfloat16, float);
  else if (src_dtype == rbh::DT_F16 && dst_dtype == rbh::DT_F32) RB_CAST(__half, float);
  else if (src_dtype == rbh::DT_F16 && dst_dtype == rbh::DT_BF16) RB_CAST(__half, __nv_bfloat16);
  else if (src_dtype == rbh::DT_BF16 && dst_dtype == rbh::DT_F16) RB_CAST(__nv_bfloat16, __half);
  else if (src_dtype == rbh::DT_F32) RB_CAST(float, float);
  else if (src_dtype == rbh::DT_BF16) RB_CAST(__nv_bfloat16, __nv_bfloat16);
  else RB_CAST(__half, __half);
#undef RB_CAST
  RB_RET_LAST();
}
int rb_swiglu_fwd(int dtype, const void* gu, void* y, long long rows, int F, long long ld,
                  void* stream) {
  using namespace rb;
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  RB_DISPATCH_T(dtype, (swiglu_fwd_kernel<T><<<ew_grid(rows * F, 256), 256, 0, st>>>((const T*)gu, (T*)y, rows, F, ld)));
  RB_RET_LAST();
}
int rb_swiglu_bwd(int dtype, const void* gu, const void* dy, void* dgu, long long rows, int F,
                  long long ld, void* stream) {
  using namespace rb;
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  RB_DISPATCH_T(dtype, (swiglu_bwd_kernel<T><<<ew_grid(rows * F, 256), 256, 0, st>>>((const T*)gu, (const T*)dy, (T*)dgu, rows, F, ld)));
  RB_RET_LAST();
}
int rb_dropout(int dtype, const void* x, void* y, long long n, unsigned seed, float p, void* stream) {
  using namespace rb;
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  double thr = (double)p * 4294967296.0;
  const uint32_t threshold = thr >= 4294967295.0 ? 0xffffffffu : (uint32_t)thr;
  const float scale = p < 1.f ? 1.f / (1.f - p) : 0.f;
  RB_DISPATCH_T(dtype, (dropout_kernel<T><<<ew_grid(n, 256), 256, 0, st>>>((const T*)x, (T*)y, n, seed, threshold, scale)));
  RB_RET_LAST();
}
int rb_embedding_fwd(int dtype, const long long* idx, const void* W, const void* pos, void* out,
                     long long tokens, int D, int S, int vocab, void* stream) {
  using namespace rb;
  if (tokens <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int esz = dtype == rbh::DT_F32 ? 4 : 2;
  const bool vec = (D % (16 / esz) == 0) && al(W) && al(pos) && al(out);
  if (vec) {
    RB_DISPATCH_T(dtype, (embedding_fwd_kernel<T><<<ew_grid(tokens * (D / (16 / (int)sizeof(T))), 256), 256, 0, st>>>(idx, (const T*)W, (const T*)pos, (T*)out, tokens, D, S, vocab)));
  } else {
    RB_DISPATCH_T(dtype, (embedding_fwd_scalar_kernel<T><<<ew_grid(tokens * D, 256), 256, 0, st>>>(idx, (const T*)W, (const T*)pos, (T*)out, tokens, D, S, vocab)));
  }
  RB_RET_LAST();
}
int rb_embedding_bwd(int dtype, const long long* idx, const void* dout, float* dW32, float* dpos32,
                     long long tokens, int D, int S, int vocab, void* stream) {
  using namespace rb;
  if (tokens <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  RB_DISPATCH_T(dtype, (embedding_bwd_kernel<T><<<ew_grid(tokens * D, 256), 256, 0, st>>>(idx, (const T*)dout, dW32, dpos32, tokens, D, S, vocab)));
  RB_RET_LAST();
}
int rb_rope(int dtype, void* x, const long long* pos_ids, long long tokens, int S, int heads, int hd,
            long long ld, int col0, float theta, int backward, void* stream) {
  using namespace rb;
  if (tokens <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const long long n = tokens * heads * (hd / 2);
  RB_DISPATCH_T(dtype, (rope_kernel<T><<<ew_grid(n, 256), 256, 0, st>>>((T*)x, pos_ids, tokens, S, heads, hd, ld, col0, theta, backward ? -1.f : 1.f)));
  RB_RET_LAST();
}
// number of row slabs rb_colsum uses; scratch needed = slabs * N floats
int rb_colsum_slabs(long long rows) {
  long long s = (rows + 63) / 64;
  if (s > 512) s = 512;
  if (s < 1) s = 1;
  return (int)s;
}
int rb_colsum(int dtype, const void* x, void* out, float* scratch, long long rows, int N,
              long long ld, void* stream) {
  using namespace rb;
  if (N <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int slabs = rb_colsum_slabs(rows);
  const int rps = (int)((rows + slabs - 1) / slabs);
  const int esz = dtype == rbh::DT_F32 ? 4 : 2;
  const int vec = 16 / esz;
  const bool vec_ok = (N % vec == 0) && ((ld * esz) % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (vec_ok) {
    dim3 grid((N / vec + 127) / 128, slabs);
    RB_DISPATCH_T(dtype, (colsum_partial_vec_kernel<T><<<grid, 128, 0, st>>>((const T*)x, scratch, rows, N, ld, rps)));
  } else {
    dim3 grid((N + 127) / 128, slabs);
    RB_DISPATCH_T(dtype, (colsum_partial_kernel<T><<<grid, 128, 0, st>>>((const T*)x, scratch, rows, N, ld, rps)));
  }
  RB_DISPATCH_T(dtype, (colsum_final_kernel<T><<<(N + 31) / 32, 256, 0, st>>>(scratch, slabs, N, (T*)out)));
  RB_RET_LAST();
}
}
