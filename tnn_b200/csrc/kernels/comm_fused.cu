// Fused compute + collective kernels over NVLink peer memory (plain P2P loads and
// stores issued from SM code; no NCCL call, no multicast TMA), plus the symmetric
// heap they operate on.
//
//   tnnb_tp_push / tnnb_tp_resolve   stand-alone forms of the tensor-parallel hand-offs (rows pushed into the
//       peers' gather buffers; partial sums pulled from the inbox) for chains that do not begin or end with a
//       layer norm. The fused all-gather -> GEMM and GEMM -> reduce-scatter kernels themselves are the
//       tensor-parallel variants of the CTA-pair GEMM (gemm_tcgen05.cu, tnnb_gemm_tp).
//   tnnb_dp_step   data-parallel gradient reduce-scatter + optimizer + parameter
//       all-gather in ONE kernel: each rank pulls its slice of every peer's fp32
//       gradient buffer, sums, applies AdamW / SGD-momentum to its fp32 master
//       slice and stores the new bf16 parameters into every peer's parameter
//       buffer. Bracketed by two cross-rank flag barriers.
//
// The reference has no collective at all (its data-parallel mode is a stub,
// include/distributed/coordinator.hpp:38,618-620); the baseline these replace is
// ncclAllGather/ncclReduceScatter around the plain GEMM and the optimizer.
//
// Every cross-rank wait is a bounded spin (about 2 s) that records
// ST_TIMEOUT_PEER in the status word and lets the kernel finish.
#include "gemm_tcgen05.h"
#include <cstdlib>

#include "ptx.cuh"
#include "tp_flags.cuh"

namespace tnnb {

typedef __nv_bfloat16 bf16;
static constexpr int MAX_PEERS = TP_MAX;

struct PeerFlags {
  int rank, world;
  uint32_t* flags[MAX_PEERS];  // flags[r] = base of rank r's barrier slots (symmetric); slot [src]
};

// One warp: publish `epoch` in every peer's slot for this rank, then wait for every peer's epoch.
__device__ __forceinline__ bool peer_barrier_warp(const PeerFlags& f, uint32_t epoch, int lane) {
  __threadfence_system();
  bool ok = true;
  if (lane < f.world && lane != f.rank) st_release_sys(f.flags[lane] + f.rank, epoch);
  if (lane < f.world && lane != f.rank) ok = spin_until<true>(f.flags[f.rank] + lane, epoch);
  return __all_sync(0xffffffffu, ok);
}

// ===================================================== stand-alone push / resolve
// The tensor-parallel hand-offs normally ride inside the layer-norm kernels and the GEMM epilogues
// (layernorm.cu, gemm_tcgen05.cu). These two kernels do the same for a chain that does not start or end with a
// layer norm: one warp per row, eight rows per block.
__global__ void __launch_bounds__(256)
tp_push_kernel(const bf16* __restrict__ src, bf16* __restrict__ local_dst, long long rows, int C,
               const __grid_constant__ TpPush push) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int chunks = C >> 3;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + r * C + c * 8);
      if (local_dst) *reinterpret_cast<uint4*>(local_dst + r * C + c * 8) = v;
      for (int t = 0; t < push.n; ++t) *reinterpret_cast<uint4*>(push.dst[t] + r * C + c * 8) = v;
    }
  }
  if (push.n) tp_push_signal(push, rows, wpb);
}

// The same push done by the bulk-copy unit instead of SM stores: one thread per block streams 8-row pieces
// local memory -> shared memory -> every peer's buffer (cp.async.bulk both ways, no multicast), PB_STAGES pieces
// in flight per block, and publishes its pieces after its last store has completed. rows % 8 == 0.
static constexpr int PB_STAGES = 4;
__global__ void __launch_bounds__(32)
tp_push_bulk_kernel(const bf16* __restrict__ src, bf16* __restrict__ local_dst, long long rows, int C,
                    const __grid_constant__ TpPush push, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t pb_smem[];
  __shared__ __align__(8) uint64_t full[PB_STAGES];
  if (threadIdx.x != 0) return;
  const uint32_t piece = (uint32_t)C * 16u;  // 8 rows of bf16
  const long long pieces = rows >> 3;
  const long long mine = pieces > blockIdx.x ? (pieces - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  for (int s = 0; s < PB_STAGES; ++s) mbar_init(&full[s], 1);
  mbar_fence_init();
  auto load = [&](long long k) {
    const int s = (int)(k % PB_STAGES);
    const long long pc = blockIdx.x + k * gridDim.x;
    mbar_expect_tx(&full[s], piece);
    bulk_load_g2s(pb_smem + (size_t)s * piece, src + pc * 8 * C, piece, &full[s]);
  };
  long long issued = 0, done = 0;
  for (; issued < mine && issued < PB_STAGES; ++issued) load(issued);
  for (long long k = 0; k < mine; ++k) {
    const int s = (int)(k % PB_STAGES);
    if (!mbar_wait(&full[s], (uint32_t)((k / PB_STAGES) & 1))) {
      if (status) atomicOr(status, ST_TIMEOUT_PEER);
      break;
    }
    const long long pc = blockIdx.x + k * gridDim.x;
    for (int t = 0; t < push.n; ++t) bulk_store_s2g(push.dst[t] + pc * 8 * C, pb_smem + (size_t)s * piece, piece);
    if (local_dst) bulk_store_s2g(local_dst + pc * 8 * C, pb_smem + (size_t)s * piece, piece);
    bulk_commit_group();
    done = k + 1;
    if (k >= 1 && k - 1 + PB_STAGES < mine) {  // the stage of the piece before this one is free once it was read
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      load(issued++);
    }
  }
  bulk_wait_group0();
  // loads that were issued but never consumed (only after a timeout): let them land before the block exits
  for (long long k = done; k < issued; ++k) mbar_wait(&full[k % PB_STAGES], (uint32_t)((k / PB_STAGES) & 1));
  if (push.n && done) {
    __threadfence_system();
    for (long long k = 0; k < done; ++k) {
      const long long r = (blockIdx.x + k * gridDim.x) * 8;
      for (int i = 0; i < push.n; ++i) red_add_sys(push.ready[i] + ((push.row0 + r) >> 7), 8u);
    }
  }
}

__global__ void __launch_bounds__(256)
tp_resolve_kernel(const bf16* __restrict__ a, bf16* __restrict__ out, long long rows, int C,
                  const __grid_constant__ TpPull pull) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int chunks = C >> 3;
  const uint32_t want = pull.n ? pull.units * *pull.pass : 0u;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    if (pull.n) tp_pull_wait(pull, r, want, lane);
    for (int c = lane; c < chunks; c += 32) {
      const uint4 raw = *reinterpret_cast<const uint4*>(a + r * C + c * 8);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      float v[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[2 * k] = __uint_as_float(w[k] << 16);
        v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
      }
      tp_pull_add8(pull, r * C + c * 8, v);
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
        o[k] = *reinterpret_cast<uint32_t*>(&h2);
      }
      *reinterpret_cast<uint4*>(out + r * C + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ===================================================== DP: reduce + optimizer + broadcast
struct DpParams {
  PeerFlags peers;
  int dp, dp_rank;
  const float* grads[MAX_PEERS];  // every DP peer's flat fp32 gradient buffer
  bf16* params_lp[MAX_PEERS];     // every DP peer's flat bf16 parameter buffer (null: fp32 params)
  float* params_f32[MAX_PEERS];   // used instead when parameters are fp32
  float* master;                  // local fp32 master (full length; only [lo,hi) is touched)
  float* m;                       // Adam first moment / SGD velocity, local, indexed from lo
  float* v;                       // Adam second moment, local, indexed from lo
  long long lo, hi;               // slice owned by this rank
  int opt;                        // 0 AdamW, 1 SGD(momentum)
  float lr, b1, b2, eps, wd, bc1, bc2, gscale, momentum;
  const float* hyper;             // optional device {lr, bc1, bc2, gscale}
  uint32_t epoch;             // call counter: host value ...
  const uint32_t* epoch_ptr;  // ... plus an optional device-resident counter (CUDA-graph replays)
  uint32_t* go_flag;              // local
  uint32_t* done_count;           // local
  int* status;
};

__global__ void __launch_bounds__(512)
dp_step_kernel(const DpParams p) {
  __shared__ int s_ok;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t EPOCH = p.epoch + (p.epoch_ptr ? *p.epoch_ptr : 0u);
  // ---- barrier 1: every peer has finished writing its gradients ----
  if (blockIdx.x == 0 && warp == 0) {
    const bool ok = peer_barrier_warp(p.peers, 2 * EPOCH - 1, lane);
    if (lane == 0) {
      if (!ok && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER);
      st_release_gpu(p.go_flag, EPOCH);
    }
  }
  if (threadIdx.x == 0) s_ok = spin_until<false>(p.go_flag, EPOCH) ? 1 : 0;
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER);
    return;
  }
  float lr = p.lr, bc1 = p.bc1, bc2 = p.bc2, gscale = p.gscale;
  if (p.hyper) {
    lr = p.hyper[0];
    bc1 = p.hyper[1];
    bc2 = p.hyper[2];
    gscale = p.hyper[3];
  }
  // ---- reduce my slice over all peers, update, broadcast ----
  const long long n4 = (p.hi - p.lo) / 4;  // slice is a multiple of 8 elements
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long e = p.lo + i * 4;
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < p.dp; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(p.grads[r] + e);
      g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
    }
    float gv[4] = {g.x * gscale, g.y * gscale, g.z * gscale, g.w * gscale};
    float4 w4 = *reinterpret_cast<float4*>(p.master + e);
    float w[4] = {w4.x, w4.y, w4.z, w4.w};
    float4 m4 = *reinterpret_cast<float4*>(p.m + i * 4);
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    if (p.opt == 0) {
      float4 v4 = *reinterpret_cast<float4*>(p.v + i * 4);
      float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        mm[k] = p.b1 * mm[k] + (1.f - p.b1) * gv[k];
        vv[k] = p.b2 * vv[k] + (1.f - p.b2) * gv[k] * gv[k];
        const float upd = lr * (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + p.eps);
        w[k] = w[k] - upd - p.wd * lr * w[k];
      }
      *reinterpret_cast<float4*>(p.v + i * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        mm[k] = p.momentum * mm[k] - lr * gv[k];
        w[k] += mm[k];
      }
    }
    *reinterpret_cast<float4*>(p.m + i * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(p.master + e) = make_float4(w[0], w[1], w[2], w[3]);
    if (p.params_lp[0]) {
      __align__(8) bf16 o[4] = {__float2bfloat16(w[0]), __float2bfloat16(w[1]), __float2bfloat16(w[2]), __float2bfloat16(w[3])};
      for (int r = 0; r < p.dp; ++r) *reinterpret_cast<uint2*>(p.params_lp[r] + e) = *reinterpret_cast<uint2*>(o);
    } else {
      for (int r = 0; r < p.dp; ++r)
        if (p.params_f32[r] != p.master) *reinterpret_cast<float4*>(p.params_f32[r] + e) = make_float4(w[0], w[1], w[2], w[3]);
    }
  }
  // ---- barrier 2: all my stores are out; wait until every peer's stores are in ----
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(p.done_count, 1u);
    s_ok = (prev + 1 == gridDim.x * EPOCH) ? 1 : 0;  // counter is cumulative over calls
  }
  __syncthreads();
  if (s_ok && warp == 0) {
    const bool ok = peer_barrier_warp(p.peers, 2 * EPOCH, lane);
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER);
  }
}

// ===================================================== stream-ordered flag wait / set
// A one-thread kernel that makes the stream wait until a 32-bit flag (local or peer memory) has reached
// `want`, for at most `timeout_ns`; on expiry it records ST_TIMEOUT_PEER in the status word and returns,
// so the stream and the context stay usable. With tnnb_flag_set it gives ranks a way to order their
// streams against each other without a collective call.
__global__ void flag_wait_kernel(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0;; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - want) >= 0) return;
    if ((i & 15u) == 15u && globaltimer_ns() - t0 > timeout_ns) {
      if (status) atomicCAS(status, 0, ST_TIMEOUT_PEER);
      return;
    }
    __nanosleep(100);
  }
}
__global__ void flag_set_kernel(uint32_t* flag, uint32_t value) {
  __threadfence_system();
  st_release_sys(flag, value);
}

}  // namespace tnnb

using namespace tnnb;

extern "C" {

// ---------------------------------------------------------------- symmetric heap
// Plain device allocations that are exported to the other ranks of the node with CUDA IPC.
int tnnb_symm_malloc(void** out, unsigned long long bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return -(int)e - 1000;
  e = cudaMemset(*out, 0, bytes);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}
int tnnb_symm_free(void* p) {
  cudaError_t e = cudaFree(p);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}
int tnnb_ipc_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return -(int)e - 1000;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
int tnnb_ipc_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}
int tnnb_ipc_close(void* p) {
  cudaError_t e = cudaIpcCloseMemHandle(p);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// Copy rows [0, rows) of src ([rows, C] bf16, C % 8 == 0) into local_dst (may be null) and into n_push peers'
// buffers, then publish them: dst[i] / ready[i] as in tnnb_layernorm_fwd_tp.
int tnnb_tp_push(const void* src, void* local_dst, long long rows, int C, int n_push, void** push_dst, void** push_ready,
                 long long push_row0, void* stream) {
  if (C % 8 || rows <= 0 || n_push < 0 || n_push > TP_MAX - 1 || (push_row0 % 8) || push_row0 < 0) return -3;
  TpPush push{};
  push.n = n_push;
  push.row0 = (int)push_row0;
  push.rows = rows;
  for (int i = 0; i < n_push; ++i) {
    if (!push_dst[i] || !push_ready[i] || ((uintptr_t)push_dst[i] & 15)) return -4;
    push.dst[i] = (bf16*)push_dst[i];
    push.ready[i] = (uint32_t*)push_ready[i];
  }
  const long long g = (rows + 7) / 8;
  const int grid = (int)(g > 148 * 8 ? 148 * 8 : g);
  tp_push_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)src, (bf16*)local_dst, rows, C, push);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// The push through the bulk-copy unit (tp_push_bulk_kernel): rows % 8 == 0, C * 16 bytes per piece <= 48 KB.
int tnnb_tp_push_bulk(const void* src, void* local_dst, long long rows, int C, int n_push, void** push_dst,
                      void** push_ready, long long push_row0, int ctas, int* status, void* stream) {
  if (C % 8 || rows <= 0 || (rows % 8) || n_push < 0 || n_push > TP_MAX - 1 || (push_row0 % 8) || push_row0 < 0) return -3;
  if (((uintptr_t)src & 15) || ((uintptr_t)local_dst & 15) || (size_t)C * 16 > 48 * 1024) return -4;
  TpPush push{};
  push.n = n_push;
  push.row0 = (int)push_row0;
  push.rows = rows;
  for (int i = 0; i < n_push; ++i) {
    if (!push_dst[i] || !push_ready[i] || ((uintptr_t)push_dst[i] & 15)) return -4;
    push.dst[i] = (bf16*)push_dst[i];
    push.ready[i] = (uint32_t*)push_ready[i];
  }
  const size_t smem = (size_t)PB_STAGES * C * 16;
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(tp_push_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 48 * 1024);
    attr_done = true;
  }
  const long long pieces = rows / 8;
  if (ctas <= 0) ctas = 148 * 2;
  const int grid = (int)(pieces < ctas ? pieces : ctas);
  tp_push_bulk_kernel<<<grid, 32, smem, (cudaStream_t)stream>>>((const bf16*)src, (bf16*)local_dst, rows, C, push, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// out[rows, C] = a + sum of pull_src[0..n_pull) once arrived[row / 128] has reached units x *pass.
int tnnb_tp_resolve(const void* a, void* out, long long rows, int C, int n_pull, void** pull_src, const void* arrived,
                    const void* pass, unsigned int units, int* status, void* stream) {
  if (C % 8 || rows <= 0 || n_pull < 0 || n_pull > TP_MAX - 1) return -3;
  TpPull pull{};
  pull.n = n_pull;
  for (int i = 0; i < n_pull; ++i) {
    if (!pull_src[i] || ((uintptr_t)pull_src[i] & 15)) return -4;
    pull.src[i] = (const bf16*)pull_src[i];
  }
  if (n_pull && (!arrived || !pass)) return -5;
  pull.arrived = (const uint32_t*)arrived;
  pull.pass = (const uint32_t*)pass;
  pull.units = units;
  pull.status = status;
  const long long g = (rows + 7) / 8;
  const int grid = (int)(g > 148 * 8 ? 148 * 8 : g);
  tp_resolve_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)a, (bf16*)out, rows, C, pull);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// Stream-ordered bounded wait on / release store to a flag; see flag_wait_kernel. timeout_ns is capped at 10 s.
int tnnb_flag_wait(const void* flag, unsigned int want, unsigned long long timeout_ns, int* status, void* stream) {
  if (!flag || ((uintptr_t)flag & 3)) return -3;
  if (timeout_ns > 10000000000ull) timeout_ns = 10000000000ull;
  flag_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((const uint32_t*)flag, want, timeout_ns, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}
int tnnb_flag_set(void* flag, unsigned int value, void* stream) {
  if (!flag || ((uintptr_t)flag & 3)) return -3;
  flag_set_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((uint32_t*)flag, value);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

int tnnb_dp_step(int dp, int dp_rank, void** barrier_flags, void** grads, void** params_lp, void** params_f32,
                 void* master, void* m, void* v, long long lo, long long hi, int opt, float lr, float b1, float b2,
                 float eps, float wd, float bc1, float bc2, float gscale, float momentum, const void* hyper,
                 unsigned int epoch, const void* epoch_ptr, void* go_flag, void* done_count, int* status, void* stream) {
  if (dp < 1 || dp > MAX_PEERS || dp_rank < 0 || dp_rank >= dp) return -2;
  if ((lo % 8) || (hi % 8) || hi < lo) return -3;
  DpParams p{};
  p.peers.rank = dp_rank; p.peers.world = dp;
  p.dp = dp; p.dp_rank = dp_rank;
  for (int r = 0; r < dp; ++r) {
    p.peers.flags[r] = (uint32_t*)barrier_flags[r];
    p.grads[r] = (const float*)grads[r];
    p.params_lp[r] = params_lp ? (bf16*)params_lp[r] : nullptr;
    p.params_f32[r] = params_f32 ? (float*)params_f32[r] : nullptr;
  }
  p.master = (float*)master; p.m = (float*)m; p.v = (float*)v;
  p.lo = lo; p.hi = hi; p.opt = opt;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd; p.bc1 = bc1; p.bc2 = bc2; p.gscale = gscale; p.momentum = momentum;
  p.hyper = (const float*)hyper; p.epoch = epoch; p.epoch_ptr = (const uint32_t*)epoch_ptr;
  p.go_flag = (uint32_t*)go_flag; p.done_count = (uint32_t*)done_count; p.status = status;
  // Small blocks: 192 threads x 50 registers leave room beside a resident GEMM CTA (320 threads x 168 registers), so a
  // bucket launched on the second stream really runs under the backward pass instead of waiting for a free SM between
  // two GEMM kernels; with 512-thread blocks it could not. Four blocks per SM keep the standalone rate. Block 0 is
  // dispatched first, and it is the one that releases the others, so blocks beyond the resident set cannot starve it.
  // TNNB_DP_THREADS selects another block size for measurements.
  static int threads = 0;
  if (threads == 0) {
    const char* e = getenv("TNNB_DP_THREADS");
    const int t = e ? atoi(e) : 192;
    threads = (t >= 64 && t <= 512 && t % 32 == 0) ? t : 192;
  }
  const int grid = sm_count() * (threads <= 256 ? 4 : 1);
  dp_step_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // extern "C"
