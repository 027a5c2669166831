// GEMM entry point: picks the tcgen05 path when the operands satisfy the TMA
// alignment rules (16-byte aligned bases, leading dimensions that are multiples
// of 16 bytes) and otherwise a tiled SIMT kernel that accepts any strides.  The
// SIMT kernel also serves batched matmul on small or oddly shaped problems
// (reference: rumus/src/backend/gpu/shaders/matmul.wgsl:22, shaders/bmm.wgsl:22).
#include "gemm_launch.cuh"

namespace rb {

template <typename T, typename OT>
__global__ void __launch_bounds__(256)
    gemm_simt_kernel(const T* __restrict__ A, long long sam, long long sak, long long sab,
                     const T* __restrict__ B, long long sbk, long long sbn, long long sbb,
                     GemmParams p, long long out_batch_stride) {
  // 64x64 output tile, 16x16 threads, 4x4 outputs per thread, K step 16
  __shared__ float sA[16][65];
  __shared__ float sB[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const long long batch = blockIdx.z;
  A += batch * sab;
  B += batch * sbb;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int mm = i & 63, kk = i >> 6;
      int m = m0 + mm, k = k0 + kk;
      sA[kk][mm] = (m < p.M && k < p.K) ? to_f32<T>(A[m * sam + k * sak]) : 0.0f;
      int nn = i & 63;
      int n = n0 + nn;
      sB[kk][nn] = (n < p.N && k < p.K) ? to_f32<T>(B[k * sbk + n * sbn]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sB[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  OT* out = reinterpret_cast<OT*>(p.out) + batch * out_batch_stride;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j] * p.alpha;
      if (p.bias) v += to_f32<T>(reinterpret_cast<const T*>(p.bias)[n]);
      if (p.aux_out) reinterpret_cast<OT*>(p.aux_out)[m * p.ldaux_out + n] = from_f32<OT>(v);
      v = apply_act(v, p.act);
      if (p.aux_in)
        v *= apply_dact(to_f32<OT>(reinterpret_cast<const OT*>(p.aux_in)[m * p.ldaux_in + n]), p.dact);
      if (p.residual) v += to_f32<OT>(reinterpret_cast<const OT*>(p.residual)[m * p.ldr + n]);
      out[m * p.ldc + n] = from_f32<OT>(v);
    }
  }
}

template <typename T>
int launch_simt(const GemmArgs& a, int batch, long long sab, long long sbb, long long scb) {
  long long sam = a.a_mn ? 1 : a.lda, sak = a.a_mn ? a.lda : 1;
  long long sbk = a.b_mn ? a.ldb : 1, sbn = a.b_mn ? 1 : a.ldb;
  dim3 grid((a.p.N + 63) / 64, (a.p.M + 63) / 64, batch);
  if (a.p.out_f32)
    gemm_simt_kernel<T, float><<<grid, 256, 0, a.stream>>>(
        (const T*)a.A, sam, sak, sab, (const T*)a.B, sbk, sbn, sbb, a.p, scb);
  else
    gemm_simt_kernel<T, T><<<grid, 256, 0, a.stream>>>((const T*)a.A, sam, sak, sab, (const T*)a.B,
                                                       sbk, sbn, sbb, a.p, scb);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace rb

extern "C" {

// path: 0 = auto, 1 = force tcgen05 (fails with status 10 if the operands are not TMA-legal),
//       2 = force SIMT.  bn: 0 = auto, 128 or 256.
// Returns 0 on success; *path_used (optional) reports 1 (tcgen05) or 2 (SIMT).
int rb_gemm(int dtype, int a_mn, int b_mn, const void* A, long long lda, const void* B,
            long long ldb, int M, int N, int K, void* out, long long ldc, int out_f32,
            const void* bias, const void* residual, long long ldr, void* aux_out,
            long long ldaux_out, const void* aux_in, long long ldaux_in, int act, int dact,
            float alpha, int path, int bn, int max_ctas, int split_k, int* path_used,
            void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = a_mn; a.b_mn = b_mn; a.A = A; a.lda = lda; a.B = B; a.ldb = ldb;
  a.max_ctas = max_ctas;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p.M = M; p.N = N; p.K = K; p.out = out; p.bias = bias; p.residual = residual;
  p.aux_out = aux_out; p.aux_in = aux_in; p.ldc = ldc; p.ldr = ldr; p.ldaux_out = ldaux_out;
  p.ldaux_in = ldaux_in; p.act = act; p.dact = dact; p.out_f32 = out_f32; p.alpha = alpha;
  p.status = rbh::device_status_word();
  p.group_m = 8;
  p.split_k = 1;
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  const int esz = dtype == rbh::DT_F32 ? 4 : 2;
  const int osz = out_f32 ? 4 : esz;
  p.vec_ok = aligned16(out) && (ldc * osz) % 16 == 0 &&
             (!residual || (aligned16(residual) && (ldr * osz) % 16 == 0)) &&
             (!aux_out || (aligned16(aux_out) && (ldaux_out * osz) % 16 == 0)) &&
             (!aux_in || (aligned16(aux_in) && (ldaux_in * osz) % 16 == 0));
  const bool tma_ok = K > 0 && aligned16(A) && aligned16(B) && (lda * esz) % 16 == 0 &&
                      (ldb * esz) % 16 == 0;
  bool use_tc = tma_ok && (long long)M * N * K >= (1ll << 18);
  if (path == 1) {
    if (!tma_ok) return 10;
    use_tc = true;
  } else if (path == 2) {
    use_tc = false;
  }
  if (path_used) *path_used = use_tc ? 1 : 2;
  if (!use_tc) {
    if (dtype == rbh::DT_BF16) return launch_simt<__nv_bfloat16>(a, 1, 0, 0, 0);
    if (dtype == rbh::DT_F16) return launch_simt<__half>(a, 1, 0, 0, 0);
    return launch_simt<float>(a, 1, 0, 0, 0);
  }
  if (bn == 0) {
    const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
    bn = (N <= 128 || tiles256 < rbh::sm_count()) ? 128 : 256;
  }
  if (split_k > 1) {
    // split-K adds into a zero-initialised fp32 output and has no fused epilogue
    if (!out_f32 || bias || residual || aux_out || aux_in || act || dact) return 12;
    const int bk = dtype == rbh::DT_F32 ? 32 : 64;
    const int num_kb = (K + bk - 1) / bk;
    if (split_k > num_kb) split_k = num_kb;
    const int kb_per = (num_kb + split_k - 1) / split_k;
    split_k = (num_kb + kb_per - 1) / kb_per;   // no empty slice
    p.split_k = split_k;
  }
  if (dtype == rbh::DT_BF16) return launch_gemm_bf16(a, bn);
  if (dtype == rbh::DT_F16) return launch_gemm_f16(a, bn);
  return launch_gemm_tf32(a, bn);
}

// Batched matmul C[b] = A[b] . B[b] on the SIMT kernel (any strides).
int rb_bmm_simt(int dtype, int a_mn, int b_mn, const void* A, long long lda, long long sab,
                const void* B, long long ldb, long long sbb, int batch, int M, int N, int K,
                void* out, long long ldc, long long scb, int out_f32, float alpha, void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = a_mn; a.b_mn = b_mn; a.A = A; a.lda = lda; a.B = B; a.ldb = ldb;
  a.max_ctas = 0;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p = GemmParams{};
  p.M = M; p.N = N; p.K = K; p.out = out; p.ldc = ldc; p.out_f32 = out_f32; p.alpha = alpha;
  if (dtype == rbh::DT_BF16) return launch_simt<__nv_bfloat16>(a, batch, sab, sbb, scb);
  if (dtype == rbh::DT_F16) return launch_simt<__half>(a, batch, sab, sbb, scb);
  return launch_simt<float>(a, batch, sab, sbb, scb);
}
}
