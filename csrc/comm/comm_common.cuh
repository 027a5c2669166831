// Device-side building blocks for kernels that talk to peer GPUs over NVLink:
// system-scope release/acquire flag operations, bounded waits, peer pointer
// tables and NVLS multimem loads/stores.
//
// Every rank maps the same "symmetric arena" (one allocation per rank, exchanged
// once on the host); a buffer is named by its byte offset in the arena, so a
// peer's copy is `peer_base[r] + offset`.  Flags are 32-bit epoch counters that
// only grow: a waiter spins until `flag >= epoch`, nothing is ever reset, so a
// kernel can be launched again without a clearing pass.
//
// The reference stages every collective through host memory and a
// Mutex/Condvar rendezvous (rumus-distributed/src/collective.rs:16-79); a peer
// that never arrives blocks its partners forever.  Here every wait has a time
// budget and reports a status instead.
#pragma once
#include "../kernels/sm100_common.cuh"

namespace rb {

constexpr int kMaxRanks = 8;

struct PeerTable {
  void* base[kMaxRanks];  // arena base of every rank, as mapped in this process
  void* mc_base;          // multicast (NVLS) mapping of the arena, or null
  int world;
  int rank;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

#ifndef RB_COMM_WAIT_BUDGET_NS
#define RB_COMM_WAIT_BUDGET_NS 10000000000ull  // 10 s: a peer may still be finishing its step
#endif

// Spin until *flag >= epoch (system scope).  Returns false when the budget ran out
// (status word gets `code`) or when `abort_flag` (optional, CTA shared) was raised.
__device__ __forceinline__ bool wait_flag_sys(const int* flag, int epoch, int* status, int code,
                                              volatile int* abort_flag = nullptr,
                                              unsigned long long budget_ns = RB_COMM_WAIT_BUDGET_NS) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_sys(flag) >= epoch) return true;
    if ((++spins & 0x3f) == 0) {
      if (abort_flag && *abort_flag) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        record_error(status, code);
        if (abort_flag) *abort_flag = 1;
        return false;
      }
      __nanosleep(100);
    }
  }
}
__device__ __forceinline__ bool wait_flag_gpu(const int* flag, int epoch, int* status, int code,
                                              volatile int* abort_flag = nullptr,
                                              unsigned long long budget_ns = RB_COMM_WAIT_BUDGET_NS) {
  if (ld_acquire_gpu(flag) >= epoch) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_gpu(flag) >= epoch) return true;
    if ((++spins & 0x3f) == 0) {
      if (abort_flag && *abort_flag) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        record_error(status, code);
        if (abort_flag) *abort_flag = 1;
        return false;
      }
      __nanosleep(100);
    }
  }
}

template <typename T>
__device__ __forceinline__ T* peer_ptr(const PeerTable& t, int r, long long byte_off) {
  return reinterpret_cast<T*>(reinterpret_cast<char*>(t.base[r]) + byte_off);
}

// 16-byte load that bypasses L1 (peer memory is not coherent in L1)
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}


// Copy [lo, hi) bytes (multiples of 16) from peer memory to local memory with the whole CTA,
// keeping eight 16-byte loads in flight per thread to cover the NVLink round trip.
__device__ __forceinline__ void copy_range_16(char* dst, const char* src, long long lo, long long hi) {
  const long long step = (long long)blockDim.x * 16;
  long long o = lo + (long long)threadIdx.x * 16;
  for (; o + 7 * step < hi; o += 8 * step) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = ld_nc_v4(src + o + j * step);
#pragma unroll
    for (int j = 0; j < 8; ++j) st_v4(dst + o + j * step, v[j]);
  }
  for (; o < hi; o += step) st_v4(dst + o, ld_nc_v4(src + o));
}

// NVLS: one load returns the sum over all ranks' copies (reduced inside the switch)
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_ptr)
      : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_ptr)
      : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
// NVLS: one store lands in every rank's copy
__device__ __forceinline__ void multimem_st_v4(void* mc_ptr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce_16(const void* mc_ptr);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_16<__nv_bfloat16>(const void* p) {
  return multimem_ld_reduce_bf16x8(p);
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_16<__half>(const void* p) {
  return multimem_ld_reduce_f16x8(p);
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_16<float>(const void* p) {
  float4 f = multimem_ld_reduce_f32x4(p);
  return make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z),
                    __float_as_uint(f.w));
}

// A cross-rank barrier on flag slots: every rank bumps slot [my_rank] on every peer to `epoch`,
// then waits until all slots of its own array reached `epoch`.  `flags_off` is the byte offset of
// an int[world] array in the arena.  Call from ONE thread.
__device__ __forceinline__ bool barrier_all_ranks(const PeerTable& t, long long flags_off, int epoch,
                                                  int* status) {
  __threadfence_system();
  for (int r = 0; r < t.world; ++r) st_release_sys(peer_ptr<int>(t, r, flags_off) + t.rank, epoch);
  bool ok = true;
  for (int r = 0; r < t.world && ok; ++r)
    ok = wait_flag_sys(peer_ptr<int>(t, t.rank, flags_off) + r, epoch, status, RB_ERR_TIMEOUT_BARRIER);
  return ok;
}

}  // namespace rb
