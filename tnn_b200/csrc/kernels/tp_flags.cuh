// Cross-GPU flag primitives and the parameter blocks of the tensor-parallel (TP) push protocol.
//
// Protocol. Every hand-off between TP ranks is a PUSH followed by a counter update:
//   * the kernel that PRODUCES rows (layer-norm forward / backward, or a GEMM epilogue) stores them with
//     plain peer stores into the consumer rank's memory, then - after a system-scope fence - adds the
//     amount it delivered to a 32-bit counter in the consumer's memory (one counter per 128-row block);
//   * the kernel that CONSUMES them (a GEMM's TMA producer warp, or a layer-norm kernel) polls the local
//     counter until it has reached  units_per_pass x pass_number  and then reads local memory only.
// Counters only ever grow; the pass number lives in device memory (one word per chain, slot and
// direction, bumped once at the start of a pass) so that a captured CUDA graph advances on replay.
// No kernel waits for a peer to *reach* it: a producer never waits at all, so the only cross-rank
// dependency is "data produced earlier in the peer's stream", and ranks cannot deadlock.
// Every poll is bounded (about 2 s); on expiry the caller records ST_TIMEOUT_PEER and carries on.
//
// The reference has no tensor parallelism; these replace ncclAllGather / ncclReduceScatter around GEMMs.
#pragma once
#include "ptx.cuh"

namespace tnnb {

static constexpr int TP_MAX = 8;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Relaxed system-scope add; the caller has issued __threadfence_system() after the stores it publishes.
__device__ __forceinline__ void red_add_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Spin until *p (system or gpu scope) has reached `want` (wrap-safe), for at most ~2 s.
template <bool SYS>
__device__ __forceinline__ bool spin_until(const uint32_t* p, uint32_t want) {
  uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
  if (static_cast<int32_t>(v - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0;; ++i) {
    v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (static_cast<int32_t>(v - want) >= 0) return true;
    if ((i & 63u) == 63u && globaltimer_ns() - t0 > 2000000000ull) return false;
    __nanosleep(40);
  }
}

// Rows this rank produces that the other ranks of the group need (the all-gather direction).
// dst[i] / ready[i] address peer i's copy of the gather buffer / its row-block counters, both already
// offset so that row 0 of the producing kernel is row `row0` of the gather buffer.
struct TpPush {
  int n;                    // number of peers (0: nothing to push)
  int row0;                 // global row of the kernel's row 0 (multiple of 8)
  long long rows;           // only rows [0, rows) of the kernel are pushed (a multiple of 8; the consuming GEMM sends the rest)
  __nv_bfloat16* dst[TP_MAX - 1];
  uint32_t* ready[TP_MAX - 1];   // base of the peer's counter array ([M/128])
  int bulk;                 // 1: rows go out through shared memory with the bulk-copy unit instead of SM stores
};

// Partial sums the other ranks pushed for rows this rank owns (the reduce-scatter direction): the
// consuming kernel adds src[i][row, :] for every i after counter[row / 128] has reached `units` x pass.
struct TpPull {
  int n;                    // number of peers (0: nothing to add)
  const __nv_bfloat16* src[TP_MAX - 1];
  const uint32_t* arrived;  // [rows/128] counters in local memory
  const uint32_t* pass;     // device word: number of passes including the current one
  uint32_t units;           // what one pass adds to each counter
  int* status;
};

// Add the peers' partial results for 8 consecutive elements of row r (the caller has waited for them).
__device__ __forceinline__ void tp_pull_add8(const TpPull& pull, long long off, float (&v)[8]) {
  for (int s = 0; s < pull.n; ++s) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(pull.src[s] + off));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] += __uint_as_float(w[k] << 16);
      v[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
    }
  }
}
// One warp: wait until the partial results for row r have arrived (bounded; records ST_TIMEOUT_PEER).
__device__ __forceinline__ void tp_pull_wait(const TpPull& pull, long long r, uint32_t want, int lane) {
  bool ok = true;
  if (lane == 0) ok = spin_until<true>(pull.arrived + (r >> 7), want);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  __syncwarp();  // orders the other lanes' reads of the inbox after lane 0's acquire
  if (!ok && lane == 0 && pull.status) atomicCAS(pull.status, 0, ST_TIMEOUT_PEER);
}
// End of a pushing kernel: publish the rows this block stored into the peers' buffers. Blocks own groups of
// `wpb` consecutive rows (a multiple of 8 that divides 128), so a group never straddles a 128-row block.
__device__ __forceinline__ void tp_push_signal(const TpPush& push, long long rows, int wpb) {
  __syncthreads();
  rows = min(rows, push.rows);
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (long long base = (long long)blockIdx.x * wpb; base < rows; base += (long long)gridDim.x * wpb) {
      const uint32_t n = (uint32_t)min((long long)wpb, rows - base);
      for (int i = 0; i < push.n; ++i) red_add_sys(push.ready[i] + ((push.row0 + base) >> 7), n);
    }
  }
}

}  // namespace tnnb
