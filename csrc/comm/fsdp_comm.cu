// FSDP communication kernels over the symmetric arena (NVLink P2P / NVLS):
//
//  * rs_adam  — gradient reduce-scatter FUSED with the sharded Adam(W) update.  Each rank reads
//    its slice of every peer's flat gradient buffer (plain P2P loads, or ONE multimem.ld_reduce
//    per 16 bytes when the arena is bound to an NVLS multicast object), averages in fp32,
//    updates its fp32 master shard and moments, and writes the low-precision parameter shard in
//    place inside its own flat parameter buffer.  The reduced gradient never exists in memory.
//  * all_gather — every rank pulls the peers' freshly updated parameter shards into its own flat
//    parameter buffer with plain P2P loads; per-chunk ready flags let a consumer (the fused
//    all-gather -> GEMM kernel) start on chunks that have landed.
//  * allreduce_unscale — data-parallel gradient all-reduce fused with the loss-scale unscale
//    (x 1/(scale*world)) and the non-finite check; two-shot over the arena.
//
// Synchronisation is by monotonically increasing epoch flags pushed into the peers' flag arrays
// (st.release.sys) and polled locally (ld.acquire.sys) with a time budget; nothing blocks
// forever and nothing is reset between steps.
//
// Reference: FSDP gathers shards and exchanges FULL gradients through host memory under a mutex
// (rumus/src/nn/fsdp.rs:139-167, rumus/src/autograd/backward.rs:1157-1241); data-parallel
// averaging maps every gradient to the host (rumus/src/nn/parallel.rs:151-250).
#include "comm_common.cuh"
#include <cstdlib>

namespace rb {

// Threads per communication CTA (env RB_COMM_THREADS, default 512).  Measured on 2 GPUs with a
// 105M-parameter unit: 148 CTAs x 512 threads run reduce-scatter+Adam in 346 us (NCCL
// reduce-scatter + the flat Adam kernel: 556 us); 256 threads need 296 CTAs for the same time.
static int comm_threads() {
  static const int n = [] {
    const char* e = std::getenv("RB_COMM_THREADS");
    int v = e ? std::atoi(e) : 512;
    if (v < 64) v = 64;
    if (v > 512) v = 512;
    return v / 32 * 32;
  }();
  return n;
}


struct RsAdamParams {
  PeerTable peers;
  long long grad_off;         // bytes: the unit's flat gradient buffer in the arena
  long long param_off;        // bytes: the unit's flat parameter buffer in the arena
  long long shard_lo;         // elements: start of this rank's shard inside the unit
  long long shard_n;          // elements in the shard (multiple of 8)
  float* master;
  float* m;
  float* v;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int adamw;
  const float* grad_scale;    // optional device scalar
  const int* skip;            // optional device flag
  long long grad_flags_off;   // bytes: int[world] "gradients of rank r are complete" (epoch)
  long long param_flags_off;  // bytes: int[world] "parameter shard of rank r is updated" (epoch)
  int epoch;
  int* done_counter;          // local scratch int (zero between launches)
  int use_multimem;
  int* status;
};

template <typename TG>
__device__ __forceinline__ void unpack8(uint4 raw, float* f) {
  const TG* e = reinterpret_cast<const TG*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = to_f32<TG>(e[j]);
}

template <typename TG>
__global__ void __launch_bounds__(512) rs_adam_kernel(const RsAdamParams p) {
  __shared__ int s_ok;
  const PeerTable& pt = p.peers;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      // everything this rank wrote into its gradient buffer (earlier kernels on this stream)
      // becomes visible to the peers that observe the flag
      __threadfence_system();
      for (int r = 0; r < pt.world; ++r)
        st_release_sys(peer_ptr<int>(pt, r, p.grad_flags_off) + pt.rank, p.epoch);
    }
    bool ok = true;
    for (int r = 0; r < pt.world && ok; ++r)
      ok = wait_flag_sys(peer_ptr<int>(pt, pt.rank, p.grad_flags_off) + r, p.epoch, p.status,
                         RB_ERR_TIMEOUT_FLAG);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;

  const bool skip = p.skip && *p.skip;
  const float gs = (p.grad_scale ? *p.grad_scale : 1.f) / (float)pt.world;
  const float rbc1 = 1.f / p.bc1, rbc2 = 1.f / p.bc2;
  const long long nvec = p.shard_n / 8;
  TG* my_param = peer_ptr<TG>(pt, pt.rank, p.param_off) + p.shard_lo;
  // Each thread handles kUnroll vectors of 8 elements per trip and issues the kUnroll peer loads of
  // one source back to back: a peer load takes microseconds, so the bytes in flight per thread
  // decide the NVLink bandwidth this kernel reaches.
  constexpr int kUnroll = 4;
  const long long trip = (long long)gridDim.x * blockDim.x * kUnroll;
  for (long long base = (long long)blockIdx.x * blockDim.x * kUnroll + threadIdx.x; base < nvec;
       base += trip) {
    float g[kUnroll][8];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) g[u][j] = 0.f;
    if (p.use_multimem) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const long long i = base + (long long)u * blockDim.x;
        if (i < nvec) {
          const char* mc = reinterpret_cast<const char*>(pt.mc_base) + p.grad_off +
                           (p.shard_lo + i * 8) * (long long)sizeof(TG);
          unpack8<TG>(multimem_ld_reduce_16<TG>(mc), g[u]);
        }
      }
    } else {
      for (int k = 0; k < pt.world; ++k) {
        const int r = (pt.rank + k) % pt.world;
        const TG* src = peer_ptr<TG>(pt, r, p.grad_off) + p.shard_lo;
        uint4 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const long long i = base + (long long)u * blockDim.x;
          raw[u] = i < nvec ? ld_nc_v4(src + i * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          float f[8];
          unpack8<TG>(raw[u], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) g[u][j] += f[j];
        }
      }
    }
    if (skip) continue;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = base + (long long)u * blockDim.x;
      if (i >= nvec) break;
      float4 pv[2], mv[2], vv[2];
      pv[0] = *reinterpret_cast<float4*>(p.master + i * 8);
      pv[1] = *reinterpret_cast<float4*>(p.master + i * 8 + 4);
      mv[0] = *reinterpret_cast<float4*>(p.m + i * 8);
      mv[1] = *reinterpret_cast<float4*>(p.m + i * 8 + 4);
      vv[0] = *reinterpret_cast<float4*>(p.v + i * 8);
      vv[1] = *reinterpret_cast<float4*>(p.v + i * 8 + 4);
      float* pp = &pv[0].x;
      float* mp = &mv[0].x;
      float* vp = &vv[0].x;
      uint4 outv;
      TG* oe = reinterpret_cast<TG*>(&outv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float grad = g[u][j] * gs;
        mp[j] = p.beta1 * mp[j] + (1.f - p.beta1) * grad;
        vp[j] = p.beta2 * vp[j] + (1.f - p.beta2) * grad * grad;
        if (p.adamw) pp[j] -= p.lr * p.weight_decay * pp[j];
        pp[j] -= p.lr * (mp[j] * rbc1) / (sqrtf(vp[j] * rbc2) + p.eps);
        oe[j] = from_f32<TG>(pp[j]);
      }
      *reinterpret_cast<float4*>(p.master + i * 8) = pv[0];
      *reinterpret_cast<float4*>(p.master + i * 8 + 4) = pv[1];
      *reinterpret_cast<float4*>(p.m + i * 8) = mv[0];
      *reinterpret_cast<float4*>(p.m + i * 8 + 4) = mv[1];
      *reinterpret_cast<float4*>(p.v + i * 8) = vv[0];
      *reinterpret_cast<float4*>(p.v + i * 8 + 4) = vv[1];
      *reinterpret_cast<uint4*>(my_param + i * 8) = outv;
    }
  }
  // last CTA to finish publishes "my parameter shard is updated"
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < pt.world; ++r)
        st_release_sys(peer_ptr<int>(pt, r, p.param_flags_off) + pt.rank, p.epoch);
    }
  }
}

// ---------------------------------------------------------------------------------------------
struct AgParams {
  PeerTable peers;
  long long buf_off;          // bytes: gathered buffer (same offset on every rank)
  long long shard_bytes;      // bytes per rank (multiple of 16)
  long long src_flags_off;    // bytes: int[world] "shard of rank r is ready" (epoch), or -1
  int* chunk_flags;           // local int[world * chunks_per_shard] or null
  long long chunk_bytes;
  int chunks_per_shard;
  int epoch;
  int* status;
};

// Copy role: CTA `cta` of `n_ctas` pulls its share of every peer shard.
__device__ __forceinline__ void ag_copy_role(const AgParams& p, int cta, int n_ctas) {
  __shared__ int s_ok;
  const PeerTable& pt = p.peers;
  char* local = peer_ptr<char>(pt, pt.rank, p.buf_off);
  for (int k = 1; k < pt.world; ++k) {
    const int src = (pt.rank + k) % pt.world;
    if (threadIdx.x == 0) {
      bool ok = true;
      if (p.src_flags_off >= 0)
        ok = wait_flag_sys(peer_ptr<int>(pt, pt.rank, p.src_flags_off) + src, p.epoch, p.status,
                           RB_ERR_TIMEOUT_FLAG);
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) return;
    const char* remote = peer_ptr<char>(pt, src, p.buf_off) + (long long)src * p.shard_bytes;
    char* dst = local + (long long)src * p.shard_bytes;
    for (int c = cta; c < p.chunks_per_shard; c += n_ctas) {
      const long long lo = (long long)c * p.chunk_bytes;
      const long long hi = min(p.shard_bytes, lo + p.chunk_bytes);
      copy_range_16(dst, remote, lo, hi);
      if (p.chunk_flags) {
        __threadfence();
        fence_proxy_async();  // the consumer reads these bytes through TMA (async proxy)
        __syncthreads();
        if (threadIdx.x == 0) st_release_gpu(p.chunk_flags + src * p.chunks_per_shard + c, p.epoch);
      }
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(512) all_gather_kernel(const AgParams p) {
  ag_copy_role(p, blockIdx.x, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
struct ArParams {
  PeerTable peers;
  long long buf_off;        // bytes: flat gradient bucket in the arena
  long long numel;          // elements (multiple of 8 * world)
  long long enter_flags_off, exit_flags_off;  // int[world] each
  long long inf_flags_off;  // int[world]: (epoch << 1) | saw_nonfinite
  int epoch;
  const float* inv_scale;   // optional device scalar (1 / loss_scale)
  float extra_scale;        // host scalar, e.g. 1 / world for a mean
  int* found_inf;           // local device int: set to 1 if ANY rank saw a non-finite value
  int* done_counter;
  int use_multimem;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(512) allreduce_unscale_kernel(const ArParams p) {
  __shared__ int s_ok;
  __shared__ int s_bad;
  const PeerTable& pt = p.peers;
  if (threadIdx.x == 0) {
    s_bad = 0;
    bool ok = true;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < pt.world; ++r)
        st_release_sys(peer_ptr<int>(pt, r, p.enter_flags_off) + pt.rank, p.epoch);
    }
    for (int r = 0; r < pt.world && ok; ++r)
      ok = wait_flag_sys(peer_ptr<int>(pt, pt.rank, p.enter_flags_off) + r, p.epoch, p.status,
                         RB_ERR_TIMEOUT_BARRIER);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  constexpr int VEC = 16 / sizeof(T);
  const float scale = (p.inv_scale ? *p.inv_scale : 1.f) * p.extra_scale;
  const long long slice = p.numel / pt.world;
  const long long lo = slice * pt.rank;
  const long long nvec = slice / VEC;
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool bad = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const long long e = lo + i * VEC;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    if (p.use_multimem) {
      uint4 raw = multimem_ld_reduce_16<T>(reinterpret_cast<const char*>(pt.mc_base) + p.buf_off +
                                           e * (long long)sizeof(T));
      const T* el = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = to_f32<T>(el[j]);
    } else {
      for (int k = 0; k < pt.world; ++k) {
        const int r = (pt.rank + k) % pt.world;
        uint4 raw = ld_nc_v4(peer_ptr<T>(pt, r, p.buf_off) + e);
        const T* el = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] += to_f32<T>(el[j]);
      }
    }
    uint4 outv;
    T* oe = reinterpret_cast<T*>(&outv);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float v = acc[j] * scale;
      bad |= !isfinite(v);
      oe[j] = from_f32<T>(v);
    }
    if (p.use_multimem) {
      multimem_st_v4(reinterpret_cast<char*>(pt.mc_base) + p.buf_off + e * (long long)sizeof(T), outv);
    } else {
      for (int k = 0; k < pt.world; ++k) {
        const int r = (pt.rank + k) % pt.world;
        st_v4(peer_ptr<T>(pt, r, p.buf_off) + e, outv);
      }
    }
  }
  if (bad) s_bad = 1;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_bad) atomicExch(p.found_inf, 1);
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      // this rank's slice is written everywhere: tell the peers, carrying the non-finite bit
      *p.done_counter = 0;
      __threadfence_system();
      const int local_bad = atomicAdd(p.found_inf, 0) ? 1 : 0;
      for (int r = 0; r < pt.world; ++r) {
        st_release_sys(peer_ptr<int>(pt, r, p.inf_flags_off) + pt.rank, (p.epoch << 1) | local_bad);
        st_release_sys(peer_ptr<int>(pt, r, p.exit_flags_off) + pt.rank, p.epoch);
      }
      // wait for every peer's slice, then merge the non-finite bits so all ranks agree
      bool ok = true;
      int any_bad = local_bad;
      for (int r = 0; r < pt.world && ok; ++r) {
        ok = wait_flag_sys(peer_ptr<int>(pt, pt.rank, p.exit_flags_off) + r, p.epoch, p.status,
                           RB_ERR_TIMEOUT_BARRIER);
        if (ok) {
          const int* f = peer_ptr<int>(pt, pt.rank, p.inf_flags_off) + r;
          ok = wait_flag_sys(f, p.epoch << 1, p.status, RB_ERR_TIMEOUT_BARRIER);
          any_bad |= (ld_acquire_sys(f) & 1);
        }
      }
      if (any_bad) *p.found_inf = 1;
    }
  }
}

// Publish `epoch` into slot [rank] of every peer's flag array (one thread).
__global__ void signal_peers_kernel(PeerTable pt, long long flags_off, int epoch) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < pt.world; ++r)
      st_release_sys(peer_ptr<int>(pt, r, flags_off) + pt.rank, epoch);
  }
}

// Waits (bounded by `budget_ns`) for *flag >= epoch.  Used by the failure-detection tests: with a
// flag that nothing sets the wait runs out, the status word gets RB_ERR_TIMEOUT_FLAG and the
// kernel returns normally.
__global__ void wait_flag_probe_kernel(const int* flag, int epoch, unsigned long long budget_ns,
                                       int* status, int* result) {
  if (threadIdx.x == 0 && blockIdx.x == 0)
    *result = wait_flag_sys(flag, epoch, status, RB_ERR_TIMEOUT_FLAG, nullptr, budget_ns) ? 1 : 0;
}

// One-warp gate launched in front of a many-CTA worker kernel on the same stream: optionally
// publishes this rank's flag, then waits (bounded) for every peer's flag.  The worker repeats the
// same checks and finds them satisfied, so no worker CTA ever sits on an SM waiting for a peer
// that is still computing: while this rank is ahead of its peers only this warp is resident.
__global__ void flag_gate_kernel(PeerTable pt, long long flags_off, int epoch, int do_signal,
                                 int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (do_signal) {
    __threadfence_system();
    for (int r = 0; r < pt.world; ++r)
      st_release_sys(peer_ptr<int>(pt, r, flags_off) + pt.rank, epoch);
  }
  for (int r = 0; r < pt.world; ++r)
    if (!wait_flag_sys(peer_ptr<int>(pt, pt.rank, flags_off) + r, epoch, status, RB_ERR_TIMEOUT_FLAG))
      return;
}

// ---------------------------------------------------------------------------------------------
// Gather of persistent shards into a LOCAL full-size buffer (parameters resharded between uses):
// every rank keeps its shard of a unit in a small arena buffer at the same offset; the full vector
// is assembled in memory that no peer ever reads (a slot shared by several units), so reusing the
// slot needs no cross-rank handshake.  Shard `r` lands at dst + r * shard_bytes; the local shard is
// copied too.
struct SgParams {
  PeerTable peers;
  long long src_off;          // bytes: the shard buffer (same offset on every rank)
  char* dst;                  // local, world * shard_bytes
  long long shard_bytes;      // multiple of 16
  long long src_flags_off;    // int[world] "shard of rank r has been updated" (epoch), or -1
  long long chunk_bytes;
  int chunks_per_shard;
  int epoch;
  int* status;
};

__global__ void __launch_bounds__(512) shard_gather_kernel(const SgParams p) {
  __shared__ int s_ok;
  const PeerTable& pt = p.peers;
  for (int k = 0; k < pt.world; ++k) {
    const int src = (pt.rank + k) % pt.world;
    if (threadIdx.x == 0) {
      bool ok = true;
      if (k > 0 && p.src_flags_off >= 0)
        ok = wait_flag_sys(peer_ptr<int>(pt, pt.rank, p.src_flags_off) + src, p.epoch, p.status,
                           RB_ERR_TIMEOUT_FLAG);
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) return;
    const char* remote = peer_ptr<char>(pt, src, p.src_off);
    char* dst = p.dst + (long long)src * p.shard_bytes;
    for (int c = blockIdx.x; c < p.chunks_per_shard; c += gridDim.x) {
      const long long lo = (long long)c * p.chunk_bytes;
      const long long hi = min(p.shard_bytes, lo + p.chunk_bytes);
      copy_range_16(dst, remote, lo, hi);
    }
    __syncthreads();
  }
}

static PeerTable make_table(void* const* bases, void* mc_base, int world, int rank) {
  PeerTable t;
  for (int i = 0; i < kMaxRanks; ++i) t.base[i] = i < world ? bases[i] : nullptr;
  t.mc_base = mc_base;
  t.world = world;
  t.rank = rank;
  return t;
}

}  // namespace rb

extern "C" {

int rb_rs_adam(int dtype, void* const* bases, void* mc_base, int world, int rank,
               long long grad_off, long long param_off, long long shard_lo, long long shard_n,
               float* master, float* m, float* v, float lr, float beta1, float beta2, float eps,
               float weight_decay, float bc1, float bc2, int adamw, const float* grad_scale,
               const int* skip, long long grad_flags_off, long long param_flags_off, int epoch,
               int* done_counter, int use_multimem, int ctas, void* stream) {
  using namespace rb;
  if (world > kMaxRanks || shard_n % 8 != 0) return 30;
  RsAdamParams p;
  p.peers = make_table(bases, mc_base, world, rank);
  p.grad_off = grad_off; p.param_off = param_off; p.shard_lo = shard_lo; p.shard_n = shard_n;
  p.master = master; p.m = m; p.v = v;
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
  p.bc1 = bc1; p.bc2 = bc2; p.adamw = adamw; p.grad_scale = grad_scale; p.skip = skip;
  p.grad_flags_off = grad_flags_off; p.param_flags_off = param_flags_off; p.epoch = epoch;
  p.done_counter = done_counter; p.use_multimem = use_multimem && mc_base != nullptr;
  p.status = rbh::device_status_word();
  if (ctas <= 0) ctas = 32;
  cudaStream_t st = (cudaStream_t)stream;
  flag_gate_kernel<<<1, 32, 0, st>>>(p.peers, grad_flags_off, epoch, 1, p.status);
  if (dtype == rbh::DT_BF16) rs_adam_kernel<__nv_bfloat16><<<ctas, comm_threads(), 0, st>>>(p);
  else if (dtype == rbh::DT_F16) rs_adam_kernel<__half><<<ctas, comm_threads(), 0, st>>>(p);
  else return 31;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_wait_flag_probe(const int* flag, int epoch, long long budget_ms, int* result, void* stream) {
  using namespace rb;
  wait_flag_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(
      flag, epoch, (unsigned long long)budget_ms * 1000000ull, rbh::device_status_word(), result);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_signal_peers(void* const* bases, int world, int rank, long long flags_off, int epoch,
                    void* stream) {
  using namespace rb;
  if (world > kMaxRanks) return 30;
  signal_peers_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_table(bases, nullptr, world, rank),
                                                          flags_off, epoch);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

// Group barrier on the stream: publish `epoch` in slot [rank] of every rank's flag array at
// `flags_off`, then wait (bounded) until every rank's slot in the local array has reached it.  One warp.
int rb_group_barrier(void* const* bases, int world, int rank, long long flags_off, int epoch,
                     void* stream) {
  using namespace rb;
  if (world > kMaxRanks) return 30;
  flag_gate_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(make_table(bases, nullptr, world, rank), flags_off,
                                                      epoch, 1, rbh::device_status_word());
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_all_gather(void* const* bases, int world, int rank, long long buf_off, long long shard_bytes,
                  long long src_flags_off, int* chunk_flags, long long chunk_bytes, int epoch,
                  int ctas, void* stream) {
  using namespace rb;
  if (world > kMaxRanks || shard_bytes % 16 != 0) return 30;
  AgParams p;
  p.peers = make_table(bases, nullptr, world, rank);
  p.buf_off = buf_off; p.shard_bytes = shard_bytes; p.src_flags_off = src_flags_off;
  p.chunk_flags = chunk_flags;
  if (ctas <= 0) ctas = 16;
  if (chunk_bytes <= 0) {
    // no consumer is waiting on chunk flags: cut each shard into about four pieces per CTA so
    // that every CTA copies (a single piece would leave the whole copy to CTA 0)
    chunk_bytes = (shard_bytes / ((long long)ctas * 4) + 4095) / 4096 * 4096;
    if (chunk_bytes < 65536) chunk_bytes = 65536;
  }
  p.chunk_bytes = chunk_bytes;
  p.chunks_per_shard = (int)((shard_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
  p.epoch = epoch;
  p.status = rbh::device_status_word();
  if (ctas <= 0) ctas = 16;
  if (src_flags_off >= 0)
    flag_gate_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p.peers, src_flags_off, epoch, 0, p.status);
  all_gather_kernel<<<ctas, comm_threads(), 0, (cudaStream_t)stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

// Assemble a unit's full parameter vector in local memory `dst` from every rank's shard buffer at
// arena offset `src_off` (see shard_gather_kernel).  With `src_flags_off >= 0` a peer's shard is
// read only once its flag has reached `epoch`.
int rb_shard_gather(void* const* bases, int world, int rank, long long src_off, void* dst,
                    long long shard_bytes, long long src_flags_off, int epoch, int ctas, void* stream) {
  using namespace rb;
  if (world > kMaxRanks || shard_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(dst) & 15)) return 30;
  SgParams p;
  p.peers = make_table(bases, nullptr, world, rank);
  p.src_off = src_off; p.dst = static_cast<char*>(dst); p.shard_bytes = shard_bytes;
  p.src_flags_off = src_flags_off; p.epoch = epoch;
  if (ctas <= 0) ctas = 16;
  p.chunk_bytes = (shard_bytes / ((long long)ctas * 4) + 4095) / 4096 * 4096;
  if (p.chunk_bytes < 65536) p.chunk_bytes = 65536;
  p.chunks_per_shard = (int)((shard_bytes + p.chunk_bytes - 1) / p.chunk_bytes);
  p.status = rbh::device_status_word();
  if (src_flags_off >= 0)
    flag_gate_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p.peers, src_flags_off, epoch, 0, p.status);
  shard_gather_kernel<<<ctas, comm_threads(), 0, (cudaStream_t)stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

int rb_allreduce_unscale(int dtype, void* const* bases, void* mc_base, int world, int rank,
                         long long buf_off, long long numel, long long enter_flags_off,
                         long long exit_flags_off, long long inf_flags_off, int epoch,
                         const float* inv_scale, float extra_scale, int* found_inf,
                         int* done_counter, int use_multimem, int ctas, void* stream) {
  using namespace rb;
  const int vec = dtype == rbh::DT_F32 ? 4 : 8;
  if (world > kMaxRanks || numel % ((long long)vec * world) != 0) return 30;
  ArParams p;
  p.peers = make_table(bases, mc_base, world, rank);
  p.buf_off = buf_off; p.numel = numel; p.enter_flags_off = enter_flags_off;
  p.exit_flags_off = exit_flags_off; p.inf_flags_off = inf_flags_off; p.epoch = epoch;
  p.inv_scale = inv_scale; p.extra_scale = extra_scale; p.found_inf = found_inf;
  p.done_counter = done_counter; p.use_multimem = use_multimem && mc_base != nullptr;
  p.status = rbh::device_status_word();
  if (ctas <= 0) ctas = 32;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == rbh::DT_BF16) allreduce_unscale_kernel<__nv_bfloat16><<<ctas, comm_threads(), 0, st>>>(p);
  else if (dtype == rbh::DT_F16) allreduce_unscale_kernel<__half><<<ctas, comm_threads(), 0, st>>>(p);
  else allreduce_unscale_kernel<float><<<ctas, comm_threads(), 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
