// Latency-bound all-reduce for decode-sized messages (a few KB to about a MB) over the symmetric arena.
//
// Each rank's partial result already sits in its own arena buffer (the row-parallel GEMM wrote it
// there).  One kernel per rank then
//   1. tells every peer "my partial of epoch e is in place" (one system-scope flag store per peer),
//   2. waits (bounded) until all peers said the same,
//   3. reads every rank's partial with plain peer loads — or, with an NVLS mapping, ONE
//      multimem.ld_reduce per 16 bytes that the switch sums — adds them in fp32, optionally adds a
//      local residual, and writes the result to a local tensor.
// One flag round, no copy-in, no copy-out, no exit barrier: the caller alternates between two arena
// buffers, which is enough because a rank can only reach its next-but-one write of a buffer after all
// peers signalled the epoch in between, and they signal it only after they finished reading this one.
//
// The reference's tensor-parallel reduction copies the partial output to the host, averages under a
// mutex and copies it back (rumus-distributed/src/tensor_parallel.rs:69-84,
// rumus-distributed/src/collective.rs:42-78).
#include "comm_common.cuh"

namespace rb {

struct OneShotParams {
  PeerTable peers;
  long long buf_off;     // bytes: this epoch's partial buffer (same offset on every rank)
  long long flags_off;   // bytes: int[world] epoch flags in the arena
  int epoch;
  const int* epoch_base; // device int added to `epoch` (null: 0).  A captured launch is replayed with the
                         // arguments it was captured with; the caller advances this word between replays
  long long numel;       // multiple of 16 bytes worth of elements
  const void* residual;  // local [numel] or null
  void* out;             // local [numel]
  int use_multimem;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(256) oneshot_allreduce_kernel(const OneShotParams p) {
  __shared__ int s_ok;
  const PeerTable& pt = p.peers;
  if (threadIdx.x == 0) {
    const int epoch = p.epoch + (p.epoch_base ? *p.epoch_base : 0);
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < pt.world; ++r)
        st_release_sys(peer_ptr<int>(pt, r, p.flags_off) + pt.rank, epoch);
    }
    bool ok = true;
    for (int r = 0; r < pt.world && ok; ++r)
      ok = wait_flag_sys(peer_ptr<int>(pt, pt.rank, p.flags_off) + r, epoch, p.status, RB_ERR_TIMEOUT_FLAG);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  constexpr int VEC = 16 / sizeof(T);
  const long long nvec = p.numel / VEC;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float acc[VEC];
    if (p.use_multimem) {
      const uint4 raw = multimem_ld_reduce_16<T>(reinterpret_cast<const char*>(pt.mc_base) + p.buf_off + i * 16);
      const T* el = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = to_f32<T>(el[j]);
    } else {
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < pt.world) raw[k] = ld_nc_v4(peer_ptr<char>(pt, (pt.rank + k) % pt.world, p.buf_off) + i * 16);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k) {
        if (k < pt.world) {
          const T* el = reinterpret_cast<const T*>(&raw[k]);
#pragma unroll
          for (int j = 0; j < VEC; ++j) acc[j] += to_f32<T>(el[j]);
        }
      }
    }
    if (p.residual) {
      const uint4 rr = *(reinterpret_cast<const uint4*>(p.residual) + i);
      const T* el = reinterpret_cast<const T*>(&rr);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += to_f32<T>(el[j]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < VEC; ++j) oe[j] = from_f32<T>(acc[j]);
    *(reinterpret_cast<uint4*>(p.out) + i) = o;
  }
}

}  // namespace rb

extern "C" {

// out[numel] = residual[numel] + sum over ranks of (arena buffer at buf_off)[numel]; see the file
// comment for the protocol.  numel * element size must be a multiple of 16 bytes.  The epoch the ranks
// agree on is `epoch` + *epoch_base (epoch_base: a device int, or null for 0).
int rb_oneshot_allreduce(int dtype, void* const* bases, void* mc_base, int world, int rank, long long buf_off,
                         long long flags_off, int epoch, long long numel, const void* residual, void* out,
                         int use_multimem, int ctas, const int* epoch_base, void* stream) {
  using namespace rb;
  if (world > kMaxRanks) return 30;
  const int esz = dtype == rbh::DT_F32 ? 4 : 2;
  if ((numel * esz) % 16 || buf_off % 16) return 35;
  OneShotParams p;
  for (int i = 0; i < kMaxRanks; ++i) p.peers.base[i] = i < world ? bases[i] : nullptr;
  p.peers.mc_base = mc_base; p.peers.world = world; p.peers.rank = rank;
  p.buf_off = buf_off; p.flags_off = flags_off; p.epoch = epoch; p.epoch_base = epoch_base; p.numel = numel;
  p.residual = residual; p.out = out;
  p.use_multimem = use_multimem && mc_base != nullptr;
  p.status = rbh::device_status_word();
  const long long nvec = numel * esz / 16;
  long long want = (nvec + 255) / 256;
  if (ctas <= 0) ctas = 32;
  if (want < ctas) ctas = (int)(want < 1 ? 1 : want);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == rbh::DT_BF16) oneshot_allreduce_kernel<__nv_bfloat16><<<ctas, 256, 0, st>>>(p);
  else if (dtype == rbh::DT_F16) oneshot_allreduce_kernel<__half><<<ctas, 256, 0, st>>>(p);
  else oneshot_allreduce_kernel<float><<<ctas, 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 3000 + (int)e;
}
}
