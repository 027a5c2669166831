// Two-CTA tcgen05 GEMM (cta_group::2), stand-alone launcher of the pair body in gemm_pair.cuh:
// clusters of two CTAs compute 256 x 256 or 512 x 256 output tiles, persistent, dynamically
// scheduled, TMA-store epilogue.  bf16 / fp16 operands in any of the four storage-major
// combinations, same fused epilogue as the one-CTA kernel.  Reference counterpart: the naive
// one-thread-per-output matmul of rumus/src/backend/gpu/shaders/matmul.wgsl:22.
#include <cstdlib>

#include "gemm_pair_launch.cuh"

namespace rb {

template <typename T, int MT, int EPI, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
    gemm_2cta_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const __grid_constant__ CUtensorMap tma_c, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  NoHooks hooks;
  gemm_pair_body<T, MT, EPI, A_MN, B_MN, NoHooks>(&tma_a, &tma_b, &tma_c, p, hooks, smem_raw, blockIdx.x / 2,
                                             gridDim.x / 2);
}

static long long* g_pair_dbg = nullptr;

template <typename T, int MT, int EPI, bool A_MN, bool B_MN>
int launch_gemm_2cta(GemmArgs& a) {
  using C = PairCfg<MT>;
  CUtensorMap ta, tb, tc;
  int rc = make_pair_operand_maps<T, A_MN, B_MN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  if (a.p.tma_store) {
    rc = make_pair_output_map(a.p, a.dtype, &tc);
    if (rc) return 1000 + rc;
  } else {
    tc = ta;
  }
  auto kern = gemm_2cta_kernel<T, MT, EPI, A_MN, B_MN>;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return 2000 + (int)e;
    resident = max_resident_clusters(kern, C::SMEM_BYTES);
  }
  const int tiles = ((a.p.M + C::BM - 1) / C::BM) * ((a.p.N + G2_BN - 1) / G2_BN);
  int clusters = resident;
  if (a.max_ctas > 0 && a.max_ctas / 2 < clusters) clusters = a.max_ctas / 2;
  if (clusters < 1) clusters = 1;
  if (tiles < clusters) clusters = tiles;
  kern<<<2 * clusters, G2_THREADS, C::SMEM_BYTES, a.stream>>>(ta, tb, tc, a.p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

template <typename T, int MT, int EPI>
int launch_gemm_2cta_major(GemmArgs& a) {
  if (!a.a_mn && !a.b_mn) return launch_gemm_2cta<T, MT, EPI, false, false>(a);
  if (!a.a_mn && a.b_mn) return launch_gemm_2cta<T, MT, EPI, false, true>(a);
  if constexpr (EPI == EPI_FULL || EPI == EPI_LEAN) {
    if (a.a_mn && !a.b_mn) return launch_gemm_2cta<T, MT, EPI, true, false>(a);
    return launch_gemm_2cta<T, MT, EPI, true, true>(a);
  }
  return -1;       // the activation flavours are built for a K-major A (activations, output gradients) only
}

// Flavours of the kernel.  LEAN: 16-bit output through the TMA-store epilogue with only the
// common epilogue terms (alpha, bias, residual) compiled in; its epilogue code is a few KB, which is
// what keeps the drain of 512-row tiles short (the epilogue of the full flavour — every activation,
// derivative, side output, fp32 output, per-row stores — is so much code that fetching it costs more
// than executing it).  GELU_AUX / DGELU: the two activation epilogues of a transformer MLP (first
// layer forward: bias, pre-activation side output, tanh-GELU; second layer's data gradient: times
// the GELU derivative of the stored pre-activation), specialised for the same reason.  FULL:
// everything, decided at run time.  All but LEAN use 256-row tiles, where the epilogue of one tile
// runs under the main loop of the next.
template <typename T>
int launch_gemm_2cta_flavour(GemmArgs& a, int mt) {
  const GemmParams& p = a.p;
  const bool staged16 = p.tma_store && !p.out_f32;
  const bool lean = staged16 && !p.aux_out && !p.aux_in && p.act == ACT_NONE;
  if (lean) return mt == 2 ? launch_gemm_2cta_major<T, 2, EPI_LEAN>(a) : launch_gemm_2cta_major<T, 1, EPI_LEAN>(a);
  const char* sp = getenv("RB_G2_SPECIAL");        // "0": always take the full flavour for activation epilogues
  if (staged16 && !a.a_mn && !(sp && sp[0] == '0')) {
    if (p.aux_out && !p.aux_in && p.act == ACT_GELU) return launch_gemm_2cta_major<T, 1, EPI_GELU_AUX>(a);
    if (p.aux_in && !p.aux_out && p.act == ACT_NONE && p.dact == ACT_GELU) return launch_gemm_2cta_major<T, 1, EPI_DGELU>(a);
  }
  return launch_gemm_2cta_major<T, 1, EPI_FULL>(a);
}

// Rows of A per CTA and tile.  512 x 256 tiles move a quarter less operand data per FLOP than
// 256 x 256 ones but hold all of TMEM, so their epilogue is exposed once per tile.  Measured back to
// back under the power cap (bf16, M 16384): wide outputs (N 8192: 1241 vs 1220 TFLOP/s, N 50304: 1218
// vs 1181) gain from the larger tile, narrow ones (N 2048: 1273 vs 1300 at K 8192, 1078 vs 1143 at
// K 2048) do not; neither does a problem whose 512-row tiles leave the last wave of clusters emptier.
int pick_pair_mt(int M, int N, int clusters) {
  if (M <= 256 || N < 4096) return 1;
  auto waves = [&](int bm) {
    const long long t = (long long)((M + bm - 1) / bm) * ((N + G2_BN - 1) / G2_BN);
    const long long w = (t + clusters - 1) / clusters;
    return (double)t / (double)(w * clusters);
  };
  return waves(512) * 1.05 >= waves(256) ? 2 : 1;
}

}  // namespace rb

extern "C" {

// Debug hook: when set (device pointer to 8 * clusters long longs), every launch makes each pair's
// MMA warp record {cycles in the kernel, cycles waiting for operands, cycles waiting for an
// accumulator, tiles done}.  Null switches it off.
void rb_gemm_2cta_set_debug(long long* buf) { rb::g_pair_dbg = buf; }

// Same contract as rb_gemm for 16-bit operands.  mt: 0 = choose, 1 = 256 x 256 tiles, 2 = 512 x 256.
// Returns 13 when the problem is outside what this kernel covers (fp32 operands, operands that are
// not TMA-legal).
int rb_gemm_2cta(int dtype, int a_mn, int b_mn, const void* A, long long lda, const void* B, long long ldb,
                 int M, int N, int K, void* out, long long ldc, int out_f32, const void* bias,
                 const void* residual, long long ldr, void* aux_out, long long ldaux_out, const void* aux_in,
                 long long ldaux_in, int act, int dact, float alpha, int max_ctas, int mt, void* stream) {
  using namespace rb;
  if (M <= 0 || N <= 0) return 0;
  if (dtype != rbh::DT_BF16 && dtype != rbh::DT_F16) return 13;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (K <= 0 || !al(A) || !al(B) || (lda * 2) % 16 || (ldb * 2) % 16) return 13;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = a_mn; a.b_mn = b_mn; a.A = A; a.lda = lda; a.B = B; a.ldb = ldb;
  a.max_ctas = max_ctas;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p.M = M; p.N = N; p.K = K; p.out = out; p.bias = bias; p.residual = residual;
  p.aux_out = aux_out; p.aux_in = aux_in; p.ldc = ldc; p.ldr = ldr; p.ldaux_out = ldaux_out;
  p.ldaux_in = ldaux_in; p.act = act; p.dact = dact; p.out_f32 = out_f32; p.alpha = alpha;
  p.status = rbh::device_status_word();
  p.split_k = 1;
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  p.dbg = g_pair_dbg;
  const int osz = out_f32 ? 4 : 2;
  p.vec_ok = al(out) && (ldc * osz) % 16 == 0 && (!residual || (al(residual) && (ldr * osz) % 16 == 0)) &&
             (!aux_out || (al(aux_out) && (ldaux_out * osz) % 16 == 0)) &&
             (!aux_in || (al(aux_in) && (ldaux_in * osz) % 16 == 0));
  p.tma_store = al(out) && (ldc * osz) % 16 == 0;
  {
    const char* e = getenv("RB_G2_TMA_STORE");
    if (e && e[0] == '0') p.tma_store = 0;
  }
  if (mt != 1 && mt != 2) {
    const char* e = getenv("RB_G2_MT");
    mt = e ? atoi(e) : 0;
    if (mt != 1 && mt != 2) mt = pick_pair_mt(M, N, rbh::sm_count() / 2);
  }
  // tiles sharing a B column panel are walked together: about 1024 rows of A per group
  p.group_m = mt == 2 ? 2 : 4;
  {
    const char* e = getenv("RB_G2_GROUP_M");
    if (e && atoi(e) > 0) p.group_m = atoi(e);
  }
  return dtype == rbh::DT_BF16 ? launch_gemm_2cta_flavour<__nv_bfloat16>(a, mt) : launch_gemm_2cta_flavour<__half>(a, mt);
}
}
