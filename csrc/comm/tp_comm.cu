// Fused collective + GEMM kernels over the symmetric arena (NVLink P2P), built on the tcgen05
// GEMM body (csrc/kernels/gemm_tcgen05.cuh):
//
//  * ag_gemm  — ALL-GATHER -> GEMM in one launch.  A few "copy" CTAs pull the peers' shards of
//    the gathered operand into this GPU's own staging buffer with plain P2P loads and publish
//    per-chunk ready flags; the GEMM CTAs (same kernel) start on tiles / K blocks whose operand
//    bytes are local already and wait (bounded) on the flags of the rest.  All TMA loads read
//    LOCAL memory, without multicast.  Two uses:
//      - tensor-parallel column-parallel linear: the sequence-sharded activation A [M/T, K] of
//        every rank is gathered along M (flags are checked per output row tile, tiles of this
//        rank's own rows are scheduled first);
//      - FSDP: the weight B [K, N] is a slab of the unit's flat parameter vector, gathered along
//        K (flags are checked per K block, K blocks inside this rank's shard go first).
//  * gemm_rs  — GEMM -> REDUCE-SCATTER in one launch (row-parallel linear).  GEMM CTAs write
//    partial output tiles into the local staging buffer and signal the tile's owner rank; a few
//    "reduce" CTAs on the owner wait for all ranks' signals, read the partial tiles from every
//    peer over NVLink, add them in fp32 (plus optional bias / residual) and write the rank's
//    [M/T, N] slab of the result.  Tiles owned by other ranks are computed first.
//
// Reference: RowParallelLinear copies the partial output to the host, averages (sic) under a
// mutex and copies back (rumus-distributed/src/tensor_parallel.rs:69-84); ColumnParallelLinear
// replicates the input (tensor_parallel.rs:30-36).
#include "../kernels/gemm_launch.cuh"
#include "comm_common.cuh"
#include "../kernels/gemm_pair_launch.cuh"

namespace rb {

struct AgParamsTp {  // same fields as AgParams in fsdp_comm.cu (kept local to this TU)
  PeerTable peers;
  long long buf_off, shard_bytes, src_flags_off;
  int* chunk_flags;
  long long chunk_bytes;
  int chunks_per_shard;
  int epoch;
  int* status;
};

__device__ __forceinline__ void ag_copy_role_tp(const AgParamsTp& p, int cta, int n_ctas) {
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
      __threadfence();
      fence_proxy_async();
      __syncthreads();
      if (threadIdx.x == 0) st_release_gpu(p.chunk_flags + src * p.chunks_per_shard + c, p.epoch);
    }
    __syncthreads();
  }
}

struct GatherHooks {
  const int* chunk_flags;
  long long shard_bytes, chunk_bytes;
  int chunks_per_shard, epoch, rank, world;
  int gather_a;         // 1: rows of A are gathered (checked per M tile); 0: rows of B (per K block)
  long long row_bytes;  // bytes per gathered row (K*esz for A, N*esz for an N-major B)
  long long base_off;   // bytes: first row of the operand inside the gathered buffer
  int rows_per_step;    // 128 (A tile rows) or BK (B rows per K block)
  int total_rows;       // M or K
  int first_local_step; // K block where this rank's own shard starts (rotation origin of a gathered B)
  int raster_first;     // row tile (in the kernel's tile height) where this rank's own rows start (gathered A)
  int raster_group;     // row tiles walked together per column panel
  mutable unsigned long long ready[4];  // chunks already seen ready (<= 256 chunks)
  mutable int remaining;                // remote chunks not yet seen ready by this thread

  // Byte offsets inside the gathered buffer fit 32 bits (the launcher checks world * shard_bytes < 4 GB):
  // the producer lane runs this before every K block of a gathered weight, so it has to cost tens of
  // cycles, not the hundreds that 64-bit divisions take, and nothing once every chunk has been seen.
  __device__ __forceinline__ bool range_ready(long long lo, long long hi, volatile int* abort_flag,
                                              int* status) const {
    if (remaining <= 0) return true;
    const uint32_t shard = (uint32_t)shard_bytes, chunk = (uint32_t)chunk_bytes;
    bool waited = false;
    for (uint32_t b = (uint32_t)lo; b < (uint32_t)hi;) {
      const uint32_t src = b / shard;
      const uint32_t in_shard = b - src * shard;
      const uint32_t c = in_shard / chunk;
      const uint32_t chunk_end = src * shard + min(shard, (c + 1) * chunk);
      if ((int)src != rank && (int)src < world) {
        const int idx = (int)src * chunks_per_shard + (int)c;
        const unsigned long long bit = 1ull << (idx & 63);
        if (!(ready[(idx >> 6) & 3] & bit)) {
          if (!wait_flag_gpu(chunk_flags + idx, epoch, status, RB_ERR_TIMEOUT_FLAG, abort_flag))
            return false;
          ready[(idx >> 6) & 3] |= bit;
          --remaining;
          waited = true;
        }
      }
      b = chunk_end;
    }
    if (waited) fence_proxy_async();
    return true;
  }

  __device__ __forceinline__ bool before_tile_load(int m_idx, int n_idx, volatile int* abort_flag,
                                                   int* status) const {
    if (!gather_a) return true;
    const long long r0 = (long long)m_idx * rows_per_step;
    const long long r1 = min((long long)total_rows, r0 + rows_per_step);
    return range_ready(base_off + r0 * row_bytes, base_off + r1 * row_bytes, abort_flag, status);
  }
  __device__ __forceinline__ bool before_k_load(int m_idx, int n_idx, int kb,
                                                volatile int* abort_flag, int* status) const {
    if (gather_a) return true;
    const long long r0 = (long long)kb * rows_per_step;
    const long long r1 = min((long long)total_rows, r0 + rows_per_step);
    return range_ready(base_off + r0 * row_bytes, base_off + r1 * row_bytes, abort_flag, status);
  }
  __device__ __forceinline__ int map_kb(int kb, int num_kb) const {
    if (gather_a) return kb;
    int k = kb + first_local_step;
    return k >= num_kb ? k - num_kb : k;
  }
  __device__ __forceinline__ void after_tile_store(int, int, int) const {}
  static constexpr bool kCustomLoadA = false, kCustomLoadB = false, kCustomRows = false;
  static constexpr bool kNeedsStoreComplete = false;
  static constexpr bool kCustomRaster = true;
  __device__ __forceinline__ void raster(int tile, int num_m, int num_n, int& m_idx,
                                         int& n_idx) const {
    // grouped raster (8 row tiles per group), rotated so this rank's own rows come first
    const int group_m = raster_group;
    const int group_size = group_m * num_n;
    const int g = tile / group_size;
    const int first_m = g * group_m;
    const int gm = min(num_m - first_m, group_m);
    const int r = tile - g * group_size;
    int m = first_m + r % gm;
    n_idx = r / gm;
    if (gather_a) {
      m += raster_first;
      if (m >= num_m) m -= num_m;
    }
    m_idx = m;
  }
};

template <typename T, int BN, bool B_MN>
__global__ void __launch_bounds__(512, 1)
    ag_gemm_kernel(const __grid_constant__ CUtensorMap tma_a,
                   const __grid_constant__ CUtensorMap tma_b, const GemmParams gp,
                   const AgParamsTp ap, GatherHooks hooks, int n_copy_ctas) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_copy_ctas) {
    ag_copy_role_tp(ap, blockIdx.x, n_copy_ctas);
    // with the dynamic tile scheduler a copy CTA joins the GEMM once its share is gathered
    // (its SM would otherwise idle for the rest of the kernel)
    if (gp.sched == nullptr) return;
    asm volatile("bar.sync 2, 512;" ::: "memory");
  }
  if (threadIdx.x >= kGemmThreads) return;  // GEMM CTAs use 10 warps; the block is sized for the copy role
  hooks.ready[0] = hooks.ready[1] = hooks.ready[2] = hooks.ready[3] = 0ull;
  hooks.remaining = (hooks.world - 1) * hooks.chunks_per_shard;
  if (gp.sched != nullptr)
    gemm_cta_body<T, BN, false, B_MN, GatherHooks>(&tma_a, &tma_b, gp, hooks, smem_raw, blockIdx.x,
                                                   gridDim.x);
  else
    gemm_cta_body<T, BN, false, B_MN, GatherHooks>(&tma_a, &tma_b, gp, hooks, smem_raw,
                                                   blockIdx.x - n_copy_ctas, gridDim.x - n_copy_ctas);
}

// The same on the CTA-pair GEMM body (clusters of two CTAs, 256-row tiles, TMA-store epilogue): copy
// CTAs come in whole clusters, and with the dynamic tile scheduler a copy cluster joins the GEMM once
// its share is gathered.  Every load of the gathered operand is a plain TMA copy of this GPU's own
// staging buffer.
template <typename T, int EPI, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
    ag_gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const __grid_constant__ CUtensorMap tma_c, const GemmParams gp, const AgParamsTp ap,
                        GatherHooks hooks, int n_copy_ctas) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_copy_ctas) {
    ag_copy_role_tp(ap, blockIdx.x, n_copy_ctas);
    if (gp.sched == nullptr) return;
    __syncthreads();
  }
  hooks.ready[0] = hooks.ready[1] = hooks.ready[2] = hooks.ready[3] = 0ull;
  hooks.remaining = (hooks.world - 1) * hooks.chunks_per_shard;
  if (gp.sched != nullptr)
    gemm_pair_body<T, 1, EPI, false, B_MN, GatherHooks>(&tma_a, &tma_b, &tma_c, gp, hooks, smem_raw, blockIdx.x / 2,
                                                         gridDim.x / 2);
  else
    gemm_pair_body<T, 1, EPI, false, B_MN, GatherHooks>(&tma_a, &tma_b, &tma_c, gp, hooks, smem_raw,
                                                         (blockIdx.x - n_copy_ctas) / 2, (gridDim.x - n_copy_ctas) / 2);
}

// ---------------------------------------------------------------------------------------------
struct RsHooks {
  PeerTable peers;
  long long tile_flags_off;  // bytes: int[tiles_per_owner][world] on every rank
  int* tile_counters;        // local int[num_m * num_n], monotonically increasing
  int epoch, num_n, m_tiles_per_rank;   // m_tiles_per_rank: 128-row blocks of the output per owner
  int raster_m_per_rank;                // row tiles of the kernel's tile height per owner

  __device__ __forceinline__ bool before_tile_load(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ bool before_k_load(int, int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ int map_kb(int kb, int) const { return kb; }
  // m_idx: 128-row block of the output (both kernels store and count per 128 x 256 block)
  __device__ __forceinline__ void after_tile_store(int m_idx, int n_idx, int quarter) const {
    __threadfence_system();
    const int prev = atomicAdd(tile_counters + m_idx * num_n + n_idx, 1);
    if ((prev % kGemmEpiWarps) == kGemmEpiWarps - 1) {
      const int owner = m_idx / m_tiles_per_rank;
      const int local_tile = (m_idx - owner * m_tiles_per_rank) * num_n + n_idx;
      __threadfence_system();
      st_release_sys(peer_ptr<int>(peers, owner, tile_flags_off) + local_tile * peers.world + peers.rank,
                     epoch);
    }
  }
  static constexpr bool kCustomLoadA = false, kCustomLoadB = false, kCustomRows = false;
  static constexpr bool kNeedsStoreComplete = true;
  static constexpr bool kCustomRaster = true;
  __device__ __forceinline__ void raster(int tile, int num_m, int num_n_, int& m_idx,
                                         int& n_idx) const {
    const int per_owner = raster_m_per_rank * num_n_;
    const int k = tile / per_owner;
    const int owner = (peers.rank + 1 + k) % peers.world;  // own tiles last
    const int local = tile - k * per_owner;
    n_idx = local % num_n_;
    m_idx = owner * raster_m_per_rank + local / num_n_;
  }
};

struct RsReduceParams {
  PeerTable peers;
  long long partial_off;   // bytes: [M, N] partial buffer of T in the arena
  long long tile_flags_off;
  void* out;               // [M/T, N] of T (local)
  const void* bias;        // [N] or null
  const void* residual;    // [M/T, N] or null
  int M, N, BN, epoch, num_n, m_tiles_per_rank;
  int* status;
};

// Run by `nthr` threads of the CTA (tid = 0 .. nthr-1) that meet at named barrier `bar_id`; kU 16-byte
// vectors per thread and source are in flight at a time.
template <typename T, int kU = 4>
__device__ __forceinline__ void rs_reduce_role(const RsReduceParams& p, int cta, int n_ctas, int tid, int nthr,
                                               int bar_id) {
  __shared__ int s_ok;
  const PeerTable& pt = p.peers;
  const int tiles = p.m_tiles_per_rank * p.num_n;
  const int rows_per_rank = p.M / pt.world;
  auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthr) : "memory"); };
  for (int t = cta; t < tiles; t += n_ctas) {
    if (tid == 0) {
      bool ok = true;
      const int* f = peer_ptr<int>(pt, pt.rank, p.tile_flags_off) + t * pt.world;
      for (int r = 0; r < pt.world && ok; ++r)
        ok = wait_flag_sys(f + r, p.epoch, p.status, RB_ERR_TIMEOUT_FLAG);
      s_ok = ok ? 1 : 0;
    }
    group_sync();
    if (!s_ok) return;
    const int m_local = (t / p.num_n) * 128;
    const int n0 = (t % p.num_n) * p.BN;
    const int ncols = min(p.BN, p.N - n0);
    const int vec_per_row = ncols / 8;
    const int nrows = min(128, rows_per_rank - m_local);
    // kU vectors per thread and trip, the kU loads of one source issued back to back: a peer
    // load takes microseconds, so the bytes in flight per thread set the reducer's bandwidth
    const int nvec = nrows * vec_per_row;
    for (int i0 = tid; i0 < nvec; i0 += nthr * kU) {
      float acc[kU][8];
      long long goff[kU];
      int cc[kU], rr[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int i = i0 + u * nthr;
        const int r = i < nvec ? i / vec_per_row : 0;
        rr[u] = r;
        cc[u] = n0 + ((i < nvec ? i : 0) - r * vec_per_row) * 8;
        goff[u] = ((long long)pt.rank * rows_per_rank + m_local + r) * p.N + cc[u];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
      }
      for (int k = 0; k < pt.world; ++k) {
        const int src = (pt.rank + k) % pt.world;
        const T* base = peer_ptr<T>(pt, src, p.partial_off);
        uint4 raw[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u)
          raw[u] = (i0 + u * nthr) < nvec ? ld_nc_v4(base + goff[u]) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] += to_f32<T>(e[j]);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (i0 + u * nthr >= nvec) break;
        const int c = cc[u];
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] += to_f32<T>(reinterpret_cast<const T*>(p.bias)[c + j]);
        }
        const long long orow = (long long)(m_local + rr[u]);
        if (p.residual) {
          uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.residual) + orow * p.N + c);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] += to_f32<T>(e[j]);
        }
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) oe[j] = from_f32<T>(acc[u][j]);
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + orow * p.N + c) = o;
      }
    }
    group_sync();
  }
}

template <typename T, int BN, bool B_MN>
__global__ void __launch_bounds__(512, 1)
    gemm_rs_kernel(const __grid_constant__ CUtensorMap tma_a,
                   const __grid_constant__ CUtensorMap tma_b, const GemmParams gp,
                   const RsHooks hooks, const RsReduceParams rp, int n_reduce_ctas) {
  extern __shared__ uint8_t smem_raw[];
  if (n_reduce_ctas == 0) {
    // unified mode: every CTA computes tiles until the scheduler runs dry (tiles owned by the
    // other ranks first), then every CTA reduces a share of this rank's own tiles.  No SM is
    // parked on a flag while there is still GEMM work, and the reduction runs at full width.
    if (threadIdx.x < kGemmThreads)
      gemm_cta_body<T, BN, false, B_MN, RsHooks>(&tma_a, &tma_b, gp, hooks, smem_raw, blockIdx.x,
                                                 gridDim.x);
    asm volatile("bar.sync 2, 512;" ::: "memory");
    rs_reduce_role<T>(rp, blockIdx.x, gridDim.x, threadIdx.x, 512, 0);
    return;
  }
  if ((int)blockIdx.x < n_reduce_ctas) {
    rs_reduce_role<T>(rp, blockIdx.x, n_reduce_ctas, threadIdx.x, 512, 0);
    return;
  }
  if (threadIdx.x >= kGemmThreads) return;
  gemm_cta_body<T, BN, false, B_MN, RsHooks>(&tma_a, &tma_b, gp, hooks, smem_raw,
                                             blockIdx.x - n_reduce_ctas, gridDim.x - n_reduce_ctas);
}

// GEMM -> reduce-scatter on the CTA-pair body (unified mode only): every cluster computes 256-row tiles
// until the scheduler runs dry, tiles owned by the other ranks first; then the two epilogue warpgroups
// of every CTA (they hold the registers at that point) reduce a share of this rank's own blocks.
template <typename T, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
    gemm_rs_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const __grid_constant__ CUtensorMap tma_c, const GemmParams gp, const RsHooks hooks,
                        const RsReduceParams rp) {
  extern __shared__ uint8_t smem_raw[];
  gemm_pair_body<T, 1, EPI_LEAN, false, B_MN, RsHooks>(&tma_a, &tma_b, &tma_c, gp, hooks, smem_raw, blockIdx.x / 2,
                                                        gridDim.x / 2);
  const int tid = (int)threadIdx.x - G2_EPI_WARP0 * 32;
  if (tid < 0) return;
  rs_reduce_role<T, 8>(rp, blockIdx.x, gridDim.x, tid, G2_EPI_WARPS * 32, 5);   // 256 threads: twice the vectors each
}

// ---------------------------------------------------------------------------------------------
// GEMM -> reduce-scatter, push form.  The epilogue of a tile stores it, rounded to T, straight into the
// OWNER's memory: every rank has one slot [M/W, N] per source rank, so the stores of different ranks never
// meet and need no atomics (adding into one shared sum with reds — fp32 or packed 16-bit — made the kernel
// atomic-bound: 585-618 us against 342 us for the pull form at 2 ranks, remote reds ran at ~100 GB/s).
// The transfers ride under the main loop as posted writes; what is left at the end is a LOCAL pass
//   out[M/W, N] = T(sum over sources of slot[src] + bias + residual).
// Two slot sets alternate from call to call: a rank can reach its next-but-one call only after every
// peer signalled the call in between, which a peer does after the pass that read this call's slots.
struct RsPushHooks {
  PeerTable peers;
  long long slots_off;       // bytes: this call's slot set [W][M/W, N] of T (same offset on every rank)
  long long done_flags_off;  // bytes: int[world] on every rank: flag[r] = epoch once rank r stored all it has
  int* owner_counters;       // local int[world], zero between calls
  int epoch, num_n, m_tiles_per_rank, N;
  uint8_t* stage;            // shared memory: 4 KB per epilogue warp (set by the kernel)

  __device__ __forceinline__ bool before_tile_load(int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ bool before_k_load(int, int, int, volatile int*, int*) const { return true; }
  __device__ __forceinline__ int map_kb(int kb, int) const { return kb; }
  __device__ __forceinline__ uint8_t* push_stage(int epi_warp) const { return stage + epi_warp * 4096; }
  __device__ __forceinline__ void* push_base(int m_idx) const {
    const int owner = m_idx / m_tiles_per_rank;
    const int blk = m_idx - owner * m_tiles_per_rank;
    const long long row0 = static_cast<long long>(peers.rank) * m_tiles_per_rank * 128 + static_cast<long long>(blk) * 128;
    return peer_ptr<char>(peers, owner, slots_off) + row0 * N * 2;
  }
  // one lane per epilogue warp, after the warp's stores of this tile: the last arrival of all tiles this
  // rank computes for `owner` tells the owner that this rank's slot is complete
  __device__ __forceinline__ void after_tile_store(int m_idx, int, int) const {
    __threadfence_system();
    const int owner = m_idx / m_tiles_per_rank;
    const int total = m_tiles_per_rank * num_n * kGemmEpiWarps;
    const int prev = atomicAdd(owner_counters + owner, 1);
    if (prev == total - 1) {
      owner_counters[owner] = 0;     // last arrival of this call: the next call (any shape) starts from zero
      __threadfence_system();
      st_release_sys(peer_ptr<int>(peers, owner, done_flags_off) + peers.rank, epoch);
    }
  }
  static constexpr bool kCustomLoadA = false, kCustomLoadB = false, kCustomRows = false;
  static constexpr bool kNeedsStoreComplete = false;
  static constexpr bool kCustomRaster = true;
  static constexpr bool kPushOut = true;
  __device__ __forceinline__ void raster(int tile, int num_m, int num_n_, int& m_idx, int& n_idx) const {
    const int per_owner = m_tiles_per_rank * num_n_;
    const int k = tile / per_owner;
    const int owner = (peers.rank + 1 + k) % peers.world;  // other ranks' tiles first: their stores travel
    const int local = tile - k * per_owner;                // while this rank still computes its own
    n_idx = local % num_n_;
    m_idx = owner * m_tiles_per_rank + local / num_n_;
  }
};

struct RsPushFinalParams {
  PeerTable peers;
  long long slots_off, done_flags_off;
  void* out;              // [M/W, N] of T
  const void* bias;       // [N] or null
  const void* residual;   // [M/W, N] or null
  long long numel;        // M/W * N
  int N, epoch;
  int* status;
};

template <typename T>
__device__ __forceinline__ void rs_push_final_role(const RsPushFinalParams& p, int cta, int n_ctas) {
  __shared__ int s_ok;
  const PeerTable& pt = p.peers;
  if (threadIdx.x == 0) {
    bool ok = true;
    const int* f = peer_ptr<int>(pt, pt.rank, p.done_flags_off);
    for (int r = 0; r < pt.world && ok; ++r) ok = wait_flag_sys(f + r, p.epoch, p.status, RB_ERR_TIMEOUT_FLAG);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const uint4* slots = peer_ptr<uint4>(pt, pt.rank, p.slots_off);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  const uint4* res = reinterpret_cast<const uint4*>(p.residual);
  uint4* out = reinterpret_cast<uint4*>(p.out);
  const long long nvec = p.numel / 8;
  const long long stride = static_cast<long long>(n_ctas) * blockDim.x;
  auto add8 = [](float* v, const uint4& q) {
    const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += to_f32<T>(e[j]);
  };
  for (long long i = static_cast<long long>(cta) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    // the peers' stores arrived in this GPU's L2 over NVLink: read the slots there
    uint4 q[kMaxRanks];
#pragma unroll
    for (int k = 0; k < kMaxRanks; ++k)
      if (k < pt.world) q[k] = __ldcg(slots + static_cast<long long>(k) * nvec + i);
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < kMaxRanks; ++k)
      if (k < pt.world) add8(v, q[k]);
    if (bias) add8(v, *reinterpret_cast<const uint4*>(bias + static_cast<int>((i * 8) % p.N)));
    if (res) add8(v, res[i]);
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = from_f32<T>(v[j]);
    out[i] = o;
  }
}

template <typename T, int BN, bool B_MN>
__global__ void __launch_bounds__(512, 1)
    gemm_rs_push_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const GemmParams gp, const RsPushHooks hooks_in, const RsPushFinalParams fp) {
  extern __shared__ uint8_t smem_raw[];
  RsPushHooks hooks = hooks_in;
  hooks.stage = smem_raw + GemmCfg<T, BN>::SMEM_BYTES;       // behind the GEMM body's own shared memory
  if (threadIdx.x < kGemmThreads)
    gemm_cta_body<T, BN, false, B_MN, RsPushHooks>(&tma_a, &tma_b, gp, hooks, smem_raw, blockIdx.x, gridDim.x);
  asm volatile("bar.sync 2, 512;" ::: "memory");
  rs_push_final_role<T>(fp, blockIdx.x, gridDim.x);
}

static PeerTable make_table_tp(void* const* bases, int world, int rank) {
  PeerTable t;
  for (int i = 0; i < kMaxRanks; ++i) t.base[i] = i < world ? bases[i] : nullptr;
  t.mc_base = nullptr;
  t.world = world;
  t.rank = rank;
  return t;
}

template <typename T, bool B_MN>
int launch_ag_gemm(const GemmArgs& a, const AgParamsTp& ap, const GatherHooks& h, int n_copy,
                   int gemm_ctas) {
  constexpr int BN = 256;
  using C = GemmCfg<T, BN>;
  CUtensorMap ta, tb;
  int rc = make_gemm_tensor_maps<T, BN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  auto kern = ag_gemm_kernel<T, BN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return 2000 + (int)e;
  const int tiles = ((a.p.M + 127) / 128) * ((a.p.N + BN - 1) / BN);
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  kern<<<n_copy + gemm_ctas, 512, C::SMEM_BYTES, a.stream>>>(ta, tb, a.p, ap, h, n_copy);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

template <typename T, bool B_MN>
int launch_gemm_rs(const GemmArgs& a, const RsHooks& h, const RsReduceParams& rp, int n_red,
                   int gemm_ctas) {
  constexpr int BN = 256;
  using C = GemmCfg<T, BN>;
  CUtensorMap ta, tb;
  int rc = make_gemm_tensor_maps<T, BN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  auto kern = gemm_rs_kernel<T, BN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return 2000 + (int)e;
  const int tiles = ((a.p.M + 127) / 128) * ((a.p.N + BN - 1) / BN);
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  kern<<<n_red + gemm_ctas, 512, C::SMEM_BYTES, a.stream>>>(ta, tb, a.p, h, rp, n_red);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

template <typename T, bool B_MN>
int launch_gemm_rs_push(const GemmArgs& a, const RsPushHooks& h, const RsPushFinalParams& fp) {
  constexpr int BN = 256;
  using C = GemmCfg<T, BN>;
  CUtensorMap ta, tb;
  int rc = make_gemm_tensor_maps<T, BN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  auto kern = gemm_rs_push_kernel<T, BN, B_MN>;
  constexpr int smem = C::SMEM_BYTES + kGemmEpiWarps * 4096;   // + the epilogue warps' staging blocks
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return 2000 + (int)e;
  // every SM takes part in the final pass, whatever the number of tiles
  kern<<<rbh::sm_count(), 512, smem, a.stream>>>(ta, tb, a.p, h, fp);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

// Launch of the pair kernels: clusters of two CTAs, one cluster per SM pair.
static bool tp_pair_enabled() {
  static const bool on = [] {
    const char* e = getenv("RB_TP_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename T, int EPI, bool B_MN>
int launch_ag_gemm_pair(GemmArgs& a, const AgParamsTp& ap, const GatherHooks& h, int n_copy) {
  using C = PairCfg<1>;
  CUtensorMap ta, tb, tc;
  int rc = make_pair_operand_maps<T, false, B_MN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  if (a.p.tma_store) {
    rc = make_pair_output_map(a.p, a.dtype, &tc);
    if (rc) return 1000 + rc;
  } else {
    tc = ta;
  }
  auto kern = ag_gemm_pair_kernel<T, EPI, B_MN>;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return 2000 + (int)e;
    resident = max_resident_clusters(kern, C::SMEM_BYTES);
  }
  n_copy = (n_copy + 1) & ~1;                      // whole clusters
  int clusters = resident;
  if (a.p.sched == nullptr) {
    // static schedule: copy clusters never join, the rest split the tiles
    const int tiles = ((a.p.M + C::BM - 1) / C::BM) * ((a.p.N + G2_BN - 1) / G2_BN);
    int gemm_clusters = clusters - n_copy / 2;
    if (gemm_clusters < 1) gemm_clusters = 1;
    if (gemm_clusters > tiles) gemm_clusters = tiles;
    clusters = gemm_clusters + n_copy / 2;
  }
  if (clusters * 2 <= n_copy) clusters = n_copy / 2 + 1;
  kern<<<2 * clusters, G2_THREADS, C::SMEM_BYTES, a.stream>>>(ta, tb, tc, a.p, ap, h, n_copy);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

template <typename T, bool B_MN>
int launch_gemm_rs_pair(GemmArgs& a, const RsHooks& h, const RsReduceParams& rp) {
  using C = PairCfg<1>;
  CUtensorMap ta, tb, tc;
  int rc = make_pair_operand_maps<T, false, B_MN>(a, &ta, &tb);
  if (rc) return 1000 + rc;
  rc = make_pair_output_map(a.p, a.dtype, &tc);
  if (rc) return 1000 + rc;
  auto kern = gemm_rs_pair_kernel<T, B_MN>;
  static int resident = 0;
  if (resident == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return 2000 + (int)e;
    resident = max_resident_clusters(kern, C::SMEM_BYTES);
  }
  // every resident cluster is launched even when there are fewer tiles: all CTAs take part in the reduction
  kern<<<2 * resident, G2_THREADS, C::SMEM_BYTES, a.stream>>>(ta, tb, tc, a.p, h, rp);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}

}  // namespace rb

extern "C" {

// out[M,N] = A[M,K] . B[K,N] (+bias, activation, residual) where ONE operand lives in a gathered
// staging buffer inside the arena (W shards of `shard_bytes`, this rank's shard already in place):
//   gather_a = 1: A = staging + a_off (rows gathered along M);  B is a local pointer
//   gather_a = 0: B = staging + b_off (N-major [K,N], rows gathered along K); A is a local pointer
// b_mn: 1 = B stored [K,N], 0 = B stored [N,K].   src_flags_off < 0: peers' shards are known ready.
int rb_ag_gemm(int dtype, void* const* bases, int world, int rank, long long buf_off,
               long long shard_bytes, long long src_flags_off, int* chunk_flags,
               long long chunk_bytes, int epoch, int gather_a, long long operand_off,
               const void* other, long long ld_other, int b_mn, int M, int N, int K, void* out,
               long long ldc, const void* bias, const void* residual, long long ldr, int act,
               void* aux_out, int n_copy_ctas, void* stream) {
  using namespace rb;
  if (world > kMaxRanks || shard_bytes % 16 != 0) return 30;
  if ((long long)world * shard_bytes >= (1ll << 32)) return 31;   // the readiness check works on 32-bit offsets
  const int esz = 2;
  AgParamsTp ap;
  ap.peers = make_table_tp(bases, world, rank);
  ap.buf_off = buf_off; ap.shard_bytes = shard_bytes; ap.src_flags_off = src_flags_off;
  ap.chunk_flags = chunk_flags;
  {
    // the ready bitmap of a GEMM warp has 256 bits: a shard too large for the requested chunk size is
    // cut into larger chunks instead of being refused
    const long long max_cps = 256 / world;
    if (chunk_bytes < 16 || (shard_bytes + chunk_bytes - 1) / chunk_bytes > max_cps) {
      chunk_bytes = (shard_bytes + max_cps - 1) / max_cps;
      chunk_bytes = (chunk_bytes + 1023) / 1024 * 1024;
    }
  }
  ap.chunk_bytes = chunk_bytes;
  ap.chunks_per_shard = (int)((shard_bytes + chunk_bytes - 1) / chunk_bytes);
  if (ap.chunks_per_shard * world > 256) return 32;
  ap.epoch = epoch;
  ap.status = rbh::device_status_word();
  char* staging = reinterpret_cast<char*>(bases[rank]) + buf_off;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = 0; a.b_mn = b_mn;
  if (gather_a) {
    a.A = staging + operand_off; a.lda = K;
    a.B = other; a.ldb = ld_other;
  } else {
    if (!b_mn) return 33;  // a K-gathered weight must be stored [K,N]
    a.A = other; a.lda = ld_other;
    a.B = staging + operand_off; a.ldb = N;
  }
  a.max_ctas = 0;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p = GemmParams{};
  p.M = M; p.N = N; p.K = K; p.out = out; p.ldc = ldc; p.bias = bias; p.residual = residual;
  p.ldr = ldr; p.act = act; p.aux_out = aux_out; p.ldaux_out = N; p.alpha = 1.f;
  p.status = ap.status; p.group_m = 8;
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  p.vec_ok = al(out) && (ldc * esz) % 16 == 0 && (!residual || (al(residual) && (ldr * esz) % 16 == 0)) &&
             (!aux_out || al(aux_out)) && (N * esz) % 16 == 0;
  if (!al(a.A) || !al(a.B) || (a.lda * esz) % 16 || (a.ldb * esz) % 16) return 10;
  GatherHooks h;
  h.chunk_flags = chunk_flags; h.shard_bytes = shard_bytes; h.chunk_bytes = chunk_bytes;
  h.chunks_per_shard = ap.chunks_per_shard; h.epoch = epoch; h.rank = rank; h.world = world;
  h.gather_a = gather_a;
  h.base_off = operand_off;
  if (gather_a) {
    h.row_bytes = (long long)K * esz; h.rows_per_step = 128; h.total_rows = M;
  } else {
    h.row_bytes = (long long)N * esz; h.rows_per_step = 64; h.total_rows = K;
  }
  {
    // first tile / K block that lies completely inside this rank's shard
    const long long step_bytes = h.row_bytes * h.rows_per_step;
    long long lo = (long long)rank * shard_bytes - operand_off;
    long long s = lo <= 0 ? 0 : (lo + step_bytes - 1) / step_bytes;
    const int nsteps = (h.total_rows + h.rows_per_step - 1) / h.rows_per_step;
    h.first_local_step = (int)(s >= nsteps ? 0 : s);
  }
  h.ready[0] = h.ready[1] = h.ready[2] = h.ready[3] = 0;
  h.remaining = 0;
  h.raster_first = gather_a ? h.first_local_step : 0;
  h.raster_group = 8;
  int ncopy = n_copy_ctas > 0 ? n_copy_ctas : 16;
  if (world == 1) ncopy = 0;
  // CTA-pair body: 16-bit operands, at least one 256 x 256 tile, output rows the TMA store can address
  p.tma_store = al(out) && (ldc * esz) % 16 == 0;
  // Measured on the Llama-7B shapes: at 2 ranks the pair body wins (323 vs 346 us); at 4 ranks its copy
  // CTAs (384 threads instead of 512) gather more slowly and the GEMM waits for them (261 vs 227 us with 32
  // copy CTAs), so larger groups stay on the one-CTA body.  RB_TP_PAIR_MAX_WORLD overrides.
  static const int pair_max_world = [] {
    const char* e = getenv("RB_TP_PAIR_MAX_WORLD");
    return e ? atoi(e) : 2;
  }();
  if (tp_pair_enabled() && world <= pair_max_world && M >= 256 && N >= 256 &&
      (p.tma_store || act != ACT_NONE || aux_out)) {
    p.group_m = 4;
    h.raster_group = 4;
    // rotation origin in 256-row tiles: the first tile that lies completely inside this rank's shard
    h.raster_first = gather_a ? (h.first_local_step + 1) / 2 : 0;
    if (h.raster_first >= (M + 255) / 256) h.raster_first = 0;
    const bool lean = p.tma_store && act == ACT_NONE && !aux_out;
#define RB_AG_PAIR(T_)                                                                                     \
  (lean ? (b_mn ? launch_ag_gemm_pair<T_, EPI_LEAN, true>(a, ap, h, ncopy)                                 \
                : launch_ag_gemm_pair<T_, EPI_LEAN, false>(a, ap, h, ncopy))                               \
        : (b_mn ? launch_ag_gemm_pair<T_, EPI_FULL, true>(a, ap, h, ncopy)                                 \
                : launch_ag_gemm_pair<T_, EPI_FULL, false>(a, ap, h, ncopy)))
    if (dtype == rbh::DT_BF16) return RB_AG_PAIR(__nv_bfloat16);
    if (dtype == rbh::DT_F16) return RB_AG_PAIR(__half);
#undef RB_AG_PAIR
    return 31;
  }
  const int gemm_ctas = rbh::sm_count() - ncopy;
  if (dtype == rbh::DT_BF16)
    return b_mn ? launch_ag_gemm<__nv_bfloat16, true>(a, ap, h, ncopy, gemm_ctas)
                : launch_ag_gemm<__nv_bfloat16, false>(a, ap, h, ncopy, gemm_ctas);
  if (dtype == rbh::DT_F16)
    return b_mn ? launch_ag_gemm<__half, true>(a, ap, h, ncopy, gemm_ctas)
                : launch_ag_gemm<__half, false>(a, ap, h, ncopy, gemm_ctas);
  return 31;
}

// Row-parallel linear: out[M/W, N] (this rank's rows) = sum_r A_r[M, K_r] . B_r[K_r, N] (+bias, +residual).
// partial_off: [M, N] staging buffer of the compute dtype in the arena (same offset on every rank);
// tile_flags_off: int[(M/W/128) * ceil(N/256) * W] in the arena; tile_counters: local int[M/128 * ceil(N/256)].
int rb_gemm_rs(int dtype, void* const* bases, int world, int rank, const void* A, long long lda,
               const void* B, long long ldb, int b_mn, int M, int N, int K, long long partial_off,
               long long tile_flags_off, int* tile_counters, int epoch, void* out,
               const void* bias, const void* residual, int n_reduce_ctas, void* stream) {
  using namespace rb;
  if (world > kMaxRanks) return 30;
  if (M % (128 * world) != 0 || N % 8 != 0) return 34;
  const int esz = 2;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = 0; a.b_mn = b_mn; a.A = A; a.lda = lda; a.B = B; a.ldb = ldb;
  a.max_ctas = 0;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p = GemmParams{};
  p.M = M; p.N = N; p.K = K;
  p.out = reinterpret_cast<char*>(bases[rank]) + partial_off;
  p.ldc = N; p.alpha = 1.f; p.vec_ok = 1; p.group_m = 8;
  p.status = rbh::device_status_word();
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al(A) || !al(B) || (lda * esz) % 16 || (ldb * esz) % 16 || partial_off % 16) return 10;
  RsHooks h;
  h.peers = make_table_tp(bases, world, rank);
  h.tile_flags_off = tile_flags_off; h.tile_counters = tile_counters; h.epoch = epoch;
  h.num_n = (N + 255) / 256;
  h.m_tiles_per_rank = M / world / 128;
  h.raster_m_per_rank = h.m_tiles_per_rank;
  RsReduceParams rp;
  rp.peers = h.peers; rp.partial_off = partial_off; rp.tile_flags_off = tile_flags_off;
  rp.out = out; rp.bias = bias; rp.residual = residual; rp.M = M; rp.N = N; rp.BN = 256;
  rp.epoch = epoch; rp.num_n = h.num_n; rp.m_tiles_per_rank = h.m_tiles_per_rank;
  rp.status = p.status;
  int nred = n_reduce_ctas > 0 ? n_reduce_ctas : 0;   // 0: unified mode (see gemm_rs_kernel)
  // Measured at 2 ranks on 8192 x 4096 x 5504: 400 us on the pair body against 342 us on the one-CTA body
  // (long K: the one-CTA main loop is already at rate, and the pair kernel reduces with 256 threads per
  // CTA instead of 512), so the pair form is opt-in (RB_TP_PAIR_RS=1) until it wins.
  static const bool rs_pair = [] {
    const char* e = getenv("RB_TP_PAIR_RS");
    return e && e[0] == '1';
  }();
  if (rs_pair && tp_pair_enabled() && nred == 0 && M % (256 * world) == 0 && N >= 256 && (N * esz) % 16 == 0) {
    p.tma_store = 1;
    p.group_m = 4;
    h.raster_m_per_rank = M / world / 256;
    if (dtype == rbh::DT_BF16)
      return b_mn ? launch_gemm_rs_pair<__nv_bfloat16, true>(a, h, rp) : launch_gemm_rs_pair<__nv_bfloat16, false>(a, h, rp);
    if (dtype == rbh::DT_F16)
      return b_mn ? launch_gemm_rs_pair<__half, true>(a, h, rp) : launch_gemm_rs_pair<__half, false>(a, h, rp);
    return 31;
  }
  const int gemm_ctas = rbh::sm_count() - nred;
  if (dtype == rbh::DT_BF16)
    return b_mn ? launch_gemm_rs<__nv_bfloat16, true>(a, h, rp, nred, gemm_ctas)
                : launch_gemm_rs<__nv_bfloat16, false>(a, h, rp, nred, gemm_ctas);
  if (dtype == rbh::DT_F16)
    return b_mn ? launch_gemm_rs<__half, true>(a, h, rp, nred, gemm_ctas)
                : launch_gemm_rs<__half, false>(a, h, rp, nred, gemm_ctas);
  return 31;
}

// Row-parallel linear, push form: out[M/W, N] = T(sum_r A_r[M, K_r] . B_r[K_r, N] + bias + residual).
// slots_off: [W][M/W, N] slot set of the compute dtype in the arena (the caller alternates between two
// sets); done_flags_off: int[W] in the arena; owner_counters: local int[W], zero between calls.
int rb_gemm_rs_push(int dtype, void* const* bases, int world, int rank, const void* A, long long lda,
                    const void* B, long long ldb, int b_mn, int M, int N, int K, long long slots_off,
                    long long done_flags_off, int* owner_counters, int epoch, void* out, const void* bias,
                    const void* residual, void* stream) {
  using namespace rb;
  if (world > kMaxRanks) return 30;
  if (M % (128 * world) != 0 || N % 8 != 0 || slots_off % 16 != 0) return 34;
  const int esz = 2;
  GemmArgs a{};
  a.dtype = dtype; a.a_mn = 0; a.b_mn = b_mn; a.A = A; a.lda = lda; a.B = B; a.ldb = ldb;
  a.max_ctas = 0;
  a.stream = (cudaStream_t)stream;
  GemmParams& p = a.p;
  p = GemmParams{};
  p.M = M; p.N = N; p.K = K; p.out = nullptr; p.ldc = N; p.alpha = 1.f; p.vec_ok = 1; p.group_m = 8;
  p.status = rbh::device_status_word();
  p.sched = rbh::dynamic_tiles() ? rbh::next_sched_slot() : nullptr;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al(A) || !al(B) || !al(out) || !al(bias) || !al(residual) || (lda * esz) % 16 || (ldb * esz) % 16) return 10;
  RsPushHooks h;
  h.peers = make_table_tp(bases, world, rank);
  h.slots_off = slots_off; h.done_flags_off = done_flags_off; h.owner_counters = owner_counters; h.epoch = epoch;
  h.num_n = (N + 255) / 256; h.m_tiles_per_rank = M / world / 128; h.N = N; h.stage = nullptr;
  RsPushFinalParams fp;
  fp.peers = h.peers; fp.slots_off = slots_off; fp.done_flags_off = done_flags_off; fp.out = out; fp.bias = bias;
  fp.residual = residual; fp.numel = (long long)(M / world) * N; fp.N = N; fp.epoch = epoch; fp.status = p.status;
  if (dtype == rbh::DT_BF16)
    return b_mn ? launch_gemm_rs_push<__nv_bfloat16, true>(a, h, fp) : launch_gemm_rs_push<__nv_bfloat16, false>(a, h, fp);
  if (dtype == rbh::DT_F16)
    return b_mn ? launch_gemm_rs_push<__half, true>(a, h, fp) : launch_gemm_rs_push<__half, false>(a, h, fp);
  return 31;
}
}
