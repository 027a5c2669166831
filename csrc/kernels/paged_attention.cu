// Serving kernels for sm_100a: paged-KV decode attention (split-KV, block-table gather),
// KV-cache append, greedy sampling (row argmax).
//
// The reference server keeps a dense zero-filled cache and a mock model
// (rumus-serve/src/model.rs:14-142) and scans the vocabulary on the CPU for the argmax
// (rumus-serve/src/scheduler.rs:101-135); none of these kernels has a counterpart there.
//
// Cache layout: k_cache / v_cache [num_blocks, block_size, Hkv, D] (token-major) or, in the `_hm`
// entry points, [num_blocks, Hkv, block_size, D] (head-major); a sequence's logical token t lives in
// physical block block_table[b][t / block_size] at offset t % block_size.
#include "sm100_common.cuh"

namespace rb {

constexpr int kPaWarps = 4;

// grid (H, B, splits), 128 threads.  D = 128: eight lanes share one token (16 dims = two 16-byte
// loads of K and of V per lane), so a warp works on four tokens at once and every 8-lane group
// carries its own online-softmax state; two tokens per group are in flight per trip.  (One token
// per warp with 8-byte loads left the kernel latency bound at about half the HBM rate.)
// partial_o [B,H,splits,D] fp32, partial_ml [B,H,splits,2] (running max in log2 domain, sum).
template <typename T>
__device__ __forceinline__ void pa_load16(const T* p, float* f) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
  const T* ea = reinterpret_cast<const T*>(&a);
  const T* eb = reinterpret_cast<const T*>(&b);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    f[j] = to_f32<T>(ea[j]);
    f[8 + j] = to_f32<T>(eb[j]);
  }
}

// HM = head-major cache [num_blocks, Hkv, block_size, D]: one head's tokens of a block are
// contiguous (block_size * 256 B), so the four tokens a warp reads per trip are one 1 KiB run
// instead of four 256-byte pieces a whole token row (Hkv * 256 B) apart.
template <typename T, bool HM = false>
__global__ void __launch_bounds__(kPaWarps * 32)
    paged_decode_attn_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                             const T* __restrict__ v_cache, const int* __restrict__ block_tables,
                             const int* __restrict__ ctx_lens, float* __restrict__ partial_o,
                             float* __restrict__ partial_ml, int H, int Hkv, int block_size,
                             int max_blocks, int splits, float scale_log2) {
  constexpr int D = 128;
  constexpr int G = kPaWarps * 4;   // token groups per CTA
  const int h = blockIdx.x, b = blockIdx.y, sp = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, sub = lane & 7;
  const int gid = warp * 4 + grp;
  const int hkv = h / (H / Hkv);
  const int ctx = ctx_lens[b];
  const int per = (ctx + splits - 1) / splits;
  const int t0 = sp * per, t1 = min(ctx, t0 + per);
  float qv[16];
  pa_load16<T>(q + ((long long)b * H + h) * D + sub * 16, qv);
#pragma unroll
  for (int j = 0; j < 16; ++j) qv[j] *= scale_log2;
  float m = -INFINITY, l = 0.f, acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  const int* table = block_tables + (long long)b * max_blocks;
  auto row_base = [&](int t) -> long long {
    const int blk = table[t / block_size];
    if constexpr (HM)
      return (((long long)blk * Hkv + hkv) * block_size + (t % block_size)) * D + sub * 16;
    else
      return (((long long)blk * block_size + (t % block_size)) * Hkv + hkv) * D + sub * 16;
  };
  // every lane runs every trip (the shuffles are warp wide); out-of-range tokens are skipped
  for (int tb = t0; tb < t1; tb += 2 * G) {
    const int ta = tb + gid, tc = tb + G + gid;
    const bool va = ta < t1, vc = tc < t1;
    float ka[16], vaa[16], kc[16], vcc[16];
    if (va) {
      const long long base = row_base(ta);
      pa_load16<T>(k_cache + base, ka);
      pa_load16<T>(v_cache + base, vaa);
    }
    if (vc) {
      const long long base = row_base(tc);
      pa_load16<T>(k_cache + base, kc);
      pa_load16<T>(v_cache + base, vcc);
    }
    float sa = 0.f, sc = 0.f;
    if (va) {
#pragma unroll
      for (int j = 0; j < 16; ++j) sa = fmaf(qv[j], ka[j], sa);
    }
    if (vc) {
#pragma unroll
      for (int j = 0; j < 16; ++j) sc = fmaf(qv[j], kc[j], sc);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      sa += __shfl_xor_sync(0xffffffffu, sa, o);
      sc += __shfl_xor_sync(0xffffffffu, sc, o);
    }
    if (va) {
      const float mn = fmaxf(m, vc ? fmaxf(sa, sc) : sa);
      const float corr = fast_exp2(m - mn);   // m = -inf on the first token: exp2(-inf) = 0
      const float pa = fast_exp2(sa - mn);
      const float pc = vc ? fast_exp2(sc - mn) : 0.f;
      l = l * corr + pa + pc;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float v = acc[j] * corr + pa * vaa[j];
        if (vc) v = fmaf(pc, vcc[j], v);
        acc[j] = v;
      }
      m = mn;
    }
  }
  // merge the 16 token groups of this CTA
  __shared__ float s_m[G], s_l[G], s_acc[G][D];
  if (sub == 0) { s_m[gid] = m; s_l[gid] = l; }
#pragma unroll
  for (int j = 0; j < 16; ++j) s_acc[gid][sub * 16 + j] = acc[j];
  __syncthreads();
  {
    const int d = threadIdx.x;   // 128 threads, one output dim each
    float gm = -INFINITY;
#pragma unroll
    for (int g = 0; g < G; ++g) gm = fmaxf(gm, s_m[g]);
    float gl = 0.f, o = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float f = s_m[g] == -INFINITY ? 0.f : fast_exp2(s_m[g] - gm);
      gl += s_l[g] * f;
      o += s_acc[g][d] * f;
    }
    const long long pi = ((long long)b * H + h) * splits + sp;
    partial_o[pi * D + d] = o;
    if (d == 0) { partial_ml[pi * 2] = gm; partial_ml[pi * 2 + 1] = gl; }
  }
}

template <typename T>
__global__ void paged_decode_reduce_kernel(const float* __restrict__ partial_o,
                                           const float* __restrict__ partial_ml, T* __restrict__ out,
                                           int splits) {
  constexpr int D = 128;
  const long long bh = blockIdx.x;
  const int d = threadIdx.x;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, partial_ml[(bh * splits + s) * 2]);
  float gl = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = partial_ml[(bh * splits + s) * 2];
    const float f = ms == -INFINITY ? 0.f : fast_exp2(ms - gm);
    gl += partial_ml[(bh * splits + s) * 2 + 1] * f;
    o += partial_o[(bh * splits + s) * D + d] * f;
  }
  out[bh * D + d] = from_f32<T>(gl > 0.f ? o / gl : 0.f);
}

// cache[slot[t], hkv, :] = src[t, hkv, :]   (src rows may be strided: fused qkv buffer)
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src,
                                 long long src_stride, const long long* __restrict__ slots,
                                 T* __restrict__ k_cache, T* __restrict__ v_cache, int tokens,
                                 int row_elems) {
  const int vecs = row_elems / 8;
  const long long total = (long long)tokens * vecs;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int t = (int)(i / vecs);
    const int c = (int)(i - (long long)t * vecs) * 8;
    const long long slot = slots[t];
    if (slot < 0) continue;
    *reinterpret_cast<uint4*>(k_cache + slot * row_elems + c) =
        *reinterpret_cast<const uint4*>(k_src + t * src_stride + c);
    *reinterpret_cast<uint4*>(v_cache + slot * row_elems + c) =
        *reinterpret_cast<const uint4*>(v_src + t * src_stride + c);
  }
}

// Head-major cache: cache[slot / bs, hkv, slot % bs, :] = src[t, hkv, :]
template <typename T>
__global__ void kv_append_hm_kernel(const T* __restrict__ k_src, const T* __restrict__ v_src,
                                    long long src_stride, const long long* __restrict__ slots,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache, int tokens, int Hkv,
                                    int D, int block_size) {
  const int vecs_per_head = D / 8;
  const int vecs = Hkv * vecs_per_head;
  const long long total = (long long)tokens * vecs;
  const long long gs = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gs) {
    const int t = (int)(i / vecs);
    const int r = (int)(i - (long long)t * vecs);
    const int hkv = r / vecs_per_head;
    const int c = (r - hkv * vecs_per_head) * 8;
    const long long slot = slots[t];
    if (slot < 0) continue;
    const long long blk = slot / block_size, off = slot % block_size;
    const long long dst = ((blk * Hkv + hkv) * block_size + off) * D + c;
    const long long src = t * src_stride + (long long)hkv * D + c;
    *reinterpret_cast<uint4*>(k_cache + dst) = *reinterpret_cast<const uint4*>(k_src + src);
    *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v_src + src);
  }
}

// out_idx[r] = argmax_c x[r, c] (first maximum), out_val[r] = the maximum
template <typename T>
__global__ void __launch_bounds__(256)
    argmax_kernel(const T* __restrict__ x, long long ld, int n, long long* __restrict__ out_idx,
                  float* __restrict__ out_val) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const T* row = x + (long long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = to_f32<T>(row[c]);
    if (v > best || (v == best && c < bi)) { best = v; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    out_idx[blockIdx.x] = bi;
    if (out_val) out_val[blockIdx.x] = best;
  }
}

}  // namespace rb

extern "C" {

int rb_paged_decode_splits(int max_ctx) {
  int s = (max_ctx + 511) / 512;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  return s;
}

// q [B,H,128]; out [B,H,128]; scratch_o: B*H*splits*128 floats; scratch_ml: B*H*splits*2 floats
int rb_paged_decode_attn(int dtype, const void* q, const void* k_cache, const void* v_cache,
                         const int* block_tables, const int* ctx_lens, void* out, float* scratch_o,
                         float* scratch_ml, int B, int H, int Hkv, int head_dim, int block_size,
                         int max_blocks, int splits, float scale, void* stream) {
  using namespace rb;
  if (head_dim != 128) return 20;
  if (B <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(H, B, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (dtype == rbh::DT_BF16) {
    paged_decode_attn_kernel<__nv_bfloat16><<<grid, kPaWarps * 32, 0, st>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        block_tables, ctx_lens, scratch_o, scratch_ml, H, Hkv, block_size, max_blocks, splits, sl2);
    paged_decode_reduce_kernel<__nv_bfloat16><<<B * H, 128, 0, st>>>(scratch_o, scratch_ml, (__nv_bfloat16*)out, splits);
  } else if (dtype == rbh::DT_F16) {
    paged_decode_attn_kernel<__half><<<grid, kPaWarps * 32, 0, st>>>(
        (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, block_tables, ctx_lens,
        scratch_o, scratch_ml, H, Hkv, block_size, max_blocks, splits, sl2);
    paged_decode_reduce_kernel<__half><<<B * H, 128, 0, st>>>(scratch_o, scratch_ml, (__half*)out, splits);
  } else {
    return 20;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_kv_append(int dtype, const void* k_src, const void* v_src, long long src_stride,
                 const long long* slots, void* k_cache, void* v_cache, int tokens, int row_elems,
                 void* stream) {
  using namespace rb;
  if (tokens <= 0) return 0;
  if (row_elems % 8 != 0 || src_stride % 8 != 0) return 21;
  cudaStream_t st = (cudaStream_t)stream;
  const long long total = (long long)tokens * (row_elems / 8);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == rbh::DT_BF16)
    kv_append_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src, src_stride, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tokens, row_elems);
  else if (dtype == rbh::DT_F16)
    kv_append_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)k_src, (const __half*)v_src, src_stride, slots, (__half*)k_cache, (__half*)v_cache, tokens, row_elems);
  else
    return 20;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

// Head-major variants (cache [num_blocks, Hkv, block_size, 128]); same arguments otherwise.
int rb_paged_decode_attn_hm(int dtype, const void* q, const void* k_cache, const void* v_cache,
                            const int* block_tables, const int* ctx_lens, void* out, float* scratch_o,
                            float* scratch_ml, int B, int H, int Hkv, int head_dim, int block_size,
                            int max_blocks, int splits, float scale, void* stream) {
  using namespace rb;
  if (head_dim != 128) return 20;
  if (B <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(H, B, splits);
  const float sl2 = scale * 1.4426950408889634f;
  if (dtype == rbh::DT_BF16) {
    paged_decode_attn_kernel<__nv_bfloat16, true><<<grid, kPaWarps * 32, 0, st>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        block_tables, ctx_lens, scratch_o, scratch_ml, H, Hkv, block_size, max_blocks, splits, sl2);
    paged_decode_reduce_kernel<__nv_bfloat16><<<B * H, 128, 0, st>>>(scratch_o, scratch_ml, (__nv_bfloat16*)out, splits);
  } else if (dtype == rbh::DT_F16) {
    paged_decode_attn_kernel<__half, true><<<grid, kPaWarps * 32, 0, st>>>(
        (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, block_tables, ctx_lens,
        scratch_o, scratch_ml, H, Hkv, block_size, max_blocks, splits, sl2);
    paged_decode_reduce_kernel<__half><<<B * H, 128, 0, st>>>(scratch_o, scratch_ml, (__half*)out, splits);
  } else {
    return 20;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_kv_append_hm(int dtype, const void* k_src, const void* v_src, long long src_stride,
                    const long long* slots, void* k_cache, void* v_cache, int tokens, int Hkv, int D,
                    int block_size, void* stream) {
  using namespace rb;
  if (tokens <= 0) return 0;
  if (D % 8 != 0 || src_stride % 8 != 0) return 21;
  cudaStream_t st = (cudaStream_t)stream;
  const long long total = (long long)tokens * Hkv * (D / 8);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == rbh::DT_BF16)
    kv_append_hm_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src, src_stride, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tokens, Hkv, D, block_size);
  else if (dtype == rbh::DT_F16)
    kv_append_hm_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)k_src, (const __half*)v_src, src_stride, slots, (__half*)k_cache, (__half*)v_cache, tokens, Hkv, D, block_size);
  else
    return 20;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_argmax(int dtype, const void* x, long long ld, int rows, int n, long long* out_idx,
              float* out_val, void* stream) {
  using namespace rb;
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == rbh::DT_BF16) argmax_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((const __nv_bfloat16*)x, ld, n, out_idx, out_val);
  else if (dtype == rbh::DT_F16) argmax_kernel<__half><<<rows, 256, 0, st>>>((const __half*)x, ld, n, out_idx, out_val);
  else argmax_kernel<float><<<rows, 256, 0, st>>>((const float*)x, ld, n, out_idx, out_val);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
