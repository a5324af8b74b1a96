// bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma
// with the fp32 accumulator in TMEM -> tcgen05.ld epilogue.
//
//   D[M,N] (+)= op(A)[M,K] * op(B)[N,K]^T   (+ bias, GELU, dGELU, ReLU, residual)
//
// Either operand may be "K-major" (stored [rows, K], K contiguous) or
// "MN-major" (stored [K, rows], rows contiguous), which is what lets one
// kernel serve the three products of a dense layer without a transpose pass:
//   forward  Y  = X  * W^T      A K-major,  B K-major
//   dgrad    dX = dY * W        A K-major,  B MN-major
//   wgrad    dW += dY^T * X     A MN-major, B MN-major, fp32 atomic split-K
// The reference obtains these from cublasGemmEx / cuDNN matmul graphs
// (src/math/cuda/gemm.cu:72-112, src/nn/engines/cudnn_engine.cu:113-326).
//
// Structure: persistent CTAs (one per SM), 10 warps.
//   warp 0      TMA producer (one lane), STAGES-deep ring of (A,B) k-blocks
//   warp 1      TMEM owner + MMA issuer (one lane), two accumulators so the
//               epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-9   epilogue: TMEM -> registers -> fused math -> per-warp staging tile in shared
//               memory -> global memory in whole 128-byte lines
//               (two warps per 32-lane TMEM quarter, each owning half of the columns)
// Two kernels share this structure: a single-CTA one (128 x 256 or 128 x 128 tiles) and a CTA-pair
// one (`cta_group::2`, 256 x 256 tiles over two SMs), which is the default for large problems.
// Every barrier wait is bounded; on expiry the kernel records a status code,
// raises a CTA-wide abort flag and unwinds (TMEM is always released).
#include "gemm_tcgen05.h"

#include <cstdlib>
#include <mutex>

#include "ptx.cuh"
#include "tp_flags.cuh"

namespace tnnb {

// Tensor-parallel extension of the CTA-pair kernel (tnnb_gemm_tp; protocol in tp_flags.cuh).
//   mode 1  all-gather -> GEMM: rows of A that another rank owns are pushed into the local A buffer by
//           that rank; the TMA producer polls the row block's counter before it loads a tile of such rows.
//           Tiles of the locally owned rows run first. The push itself is done by two extra warps of this very
//           kernel (push_n > 0): while the tensor cores work on the local tiles they copy this rank's rows
//           into every peer's buffer with plain 16-byte stores, piece by piece in row order, and bump the
//           peer's row-block counter after each piece - the transfer hides behind the local half of the GEMM
//           on both sides and blocks nobody but the two warps that issue it.
//   mode 2  GEMM -> reduce-scatter: the epilogue stores the bf16 partial sums of rows another rank owns
//           straight into that rank's inbox (peer stores) and the rows this rank owns into the local
//           output (with the bias); remote tiles run first and their counters are bumped as soon as the
//           CTA has finished its last remote tile. The kernel itself never waits for a peer.
struct TpExt {
  int mode, tp, rank;
  int rows_per_rank;   // rows of M owned by each rank (multiple of 128)
  int pair_blocks_per_rank;  // rows_per_rank / 256, or 0 when that is not whole (tile order then stays plain)
  const uint32_t* pass;      // device word: number of passes including the current one
  int* status;
  // mode 1
  const uint32_t* a_ready;   // [M/128] cumulative rows landed per 128-row block of A (local memory)
  int push_n;                // number of peers this rank's rows of A are sent to by this kernel (0: none)
  int push_first_block;      // first 128-row block (inside this rank's rows) the kernel sends; earlier ones were sent by the producer
  const __nv_bfloat16* push_src;        // this rank's A buffer (all M rows; only its own rows are read)
  long long push_ld;                    // row pitch of A in elements (the same on every rank)
  __nv_bfloat16* push_dst[TP_MAX - 1];  // peer i's A buffer
  uint32_t* push_ready[TP_MAX - 1];     // peer i's counters [M/128]
  // mode 2
  void* out[TP_MAX];         // out[o]: [rows_per_rank, ldo] block that receives the rows owned by rank o
  long long ldo;
  uint32_t* arrived[TP_MAX]; // arrived[o]: rank o's counters, one per 128-row block of its rows
};

struct GemmParams {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int split_k, kb_per_split;
  void* D;
  long long ldd;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux_in;
  __nv_bfloat16* aux_out;
  long long ld_aux;
  const __nv_bfloat16* resid;
  long long ld_res;
  int flags;
  int* status;
  int batch;                    // batched form (single-CTA kernel): number of independent products ...
  long long batch_stride_d;     // ... and the distance between their outputs, in elements of D
};

template <int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int BK = 64;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + 8 * 4096;  // + per-warp epilogue staging
};

// Where a tile's result goes: the call's output, or (tensor-parallel reduce-scatter) the block of the rank
// that owns the tile's rows, with the bias applied only by the owner.
struct EpiOut {
  void* D;
  long long ldd;
  int flags;
};

// Fused element-wise part of the epilogue for 32 accumulator columns of one row (row < M, col0 < N).
__device__ __forceinline__ void epilogue_math(const GemmParams& p, const EpiOut& eo, float (&v)[32], int row, int col0) {
  const int flags = eo.flags;
  const bool full = (col0 + 32 <= p.N);

  if (flags & EPI_BIAS) {
    if (full && ((reinterpret_cast<uintptr_t>(p.bias + col0) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {  // the same address in every lane: a broadcast
        const uint4 raw = *reinterpret_cast<const uint4*>(p.bias + col0 + j);
        const __nv_bfloat16* t = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j + k] += __bfloat162float(t[k]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full || col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
    }
  }
  if (flags & EPI_GELU) {
    if (p.aux_out) {
      __nv_bfloat16* z = p.aux_out + (long long)row * p.ld_aux + col0;
      if (full && (p.ld_aux % 8 == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          __align__(16) __nv_bfloat16 t[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) t[k] = __float2bfloat16(v[j + k]);
          *reinterpret_cast<uint4*>(z + j) = *reinterpret_cast<uint4*>(t);
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) z[j] = __float2bfloat16(v[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
  }
  if (flags & EPI_DGELU) {
    const __nv_bfloat16* z = p.aux_in + (long long)row * p.ld_aux + col0;
    if (full && (p.ld_aux % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(z + j);
        const __nv_bfloat16* t = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j + k] *= gelu_tanh_grad(__bfloat162float(t[k]));
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] *= gelu_tanh_grad(__bfloat162float(z[j]));
    }
  }
  if (flags & EPI_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
  }
  if (flags & EPI_RESID) {
    const __nv_bfloat16* rs = p.resid + (long long)row * p.ld_res + col0;
    if (full && (p.ld_res % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(rs + j);
        const __nv_bfloat16* t = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j + k] += __bfloat162float(t[k]);
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += __bfloat162float(rs[j]);
    }
  }

}

// Row-per-lane store of 32 columns (each lane writes its own row): used for ragged edges and for the
// output forms the coalescing path below does not cover.
__device__ __forceinline__ void epilogue_store_rowwise(const GemmParams& p, const EpiOut& eo, const float (&v)[32], int row, int col0) {
  const int flags = eo.flags;
  const bool full = (col0 + 32 <= p.N);
  if (flags & EPI_ATOMIC) {
    float* d = reinterpret_cast<float*>(eo.D) + (long long)row * eo.ldd + col0;
    if (full && (eo.ldd % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + j), "f"(v[j]),
                     "f"(v[j + 1]), "f"(v[j + 2]), "f"(v[j + 3])
                     : "memory");
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) atomicAdd(d + j, v[j]);
    }
  } else if (flags & EPI_OUT_F32) {
    float* d = reinterpret_cast<float*>(eo.D) + (long long)row * eo.ldd + col0;
    if (full && (eo.ldd % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (flags & EPI_ACCUM) {
          float4 old = *reinterpret_cast<float4*>(d + j);
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        *reinterpret_cast<float4*>(d + j) = o;
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) d[j] = (flags & EPI_ACCUM) ? d[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(eo.D) + (long long)row * eo.ldd + col0;
    if (full && (eo.ldd % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        __align__(16) __nv_bfloat16 t[8];
        if (flags & EPI_ACCUM) {
          uint4 raw = *reinterpret_cast<const uint4*>(d + j);
          const __nv_bfloat16* o = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
          for (int k = 0; k < 8; ++k) t[k] = __float2bfloat16(v[j + k] + __bfloat162float(o[k]));
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) t[k] = __float2bfloat16(v[j + k]);
        }
        *reinterpret_cast<uint4*>(d + j) = *reinterpret_cast<uint4*>(t);
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N)
          d[j] = __float2bfloat16((flags & EPI_ACCUM) ? v[j] + __bfloat162float(d[j]) : v[j]);
    }
  }
}


// ---- coalescing epilogue ------------------------------------------------------------------------
// tcgen05.ld hands every lane one ROW of the accumulator, so a direct store touches 32 different
// 128-byte lines per instruction. Each epilogue warp therefore owns a 4 KB staging tile in shared
// memory ([32 rows][128 B], 16-byte chunks XOR-swizzled by row): lanes write their row into it, and the
// warp reads it back with 8 lanes per row so that every global store / reduction instruction covers
// four complete 128-byte lines.
__device__ __forceinline__ uint32_t stage_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// bf16 output, 64 columns [col0, col0+64) of rows [row_base, row_base+32): lane = row has written its
// 64 values (as packed bf16) to the staging tile. Requires ldd % 8 == 0 and col0 + 64 <= N.
__device__ __forceinline__ void stage_flush_bf16(const GemmParams& p, const EpiOut& eo, const uint8_t* stage, int lane, int row_base, int col0) {
  __syncwarp();
  __nv_bfloat16* D = reinterpret_cast<__nv_bfloat16*>(eo.D);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3), c = lane & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + stage_off(r, c));
    if (row_base + r < p.M) *reinterpret_cast<uint4*>(D + (long long)(row_base + r) * eo.ldd + col0 + c * 8) = v;
  }
  __syncwarp();
}
// fp32 output (store, accumulate or atomic add), 32 columns. Requires ldd % 4 == 0 and col0 + 32 <= N.
__device__ __forceinline__ void stage_flush_f32(const GemmParams& p, const EpiOut& eo, const uint8_t* stage, int lane, int row_base, int col0) {
  __syncwarp();
  float* D = reinterpret_cast<float*>(eo.D);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3), c = lane & 7;
    float4 v = *reinterpret_cast<const float4*>(stage + stage_off(r, c));
    if (row_base + r < p.M) {
      float* d = D + (long long)(row_base + r) * eo.ldd + col0 + c * 4;
      if (eo.flags & EPI_ATOMIC) {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
      } else {
        if (eo.flags & EPI_ACCUM) {
          const float4 o = *reinterpret_cast<const float4*>(d);
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *reinterpret_cast<float4*>(d) = v;
      }
    }
  }
  __syncwarp();
}

// One warp's share of a tile: `nchunks` groups of 32 accumulator columns starting at TMEM address t_addr /
// global column col_base, rows row_base + lane. Chooses the coalescing path where its conditions hold.
__device__ __forceinline__ void epilogue_warp(const GemmParams& p, const EpiOut& eo, uint32_t t_addr, int nchunks, int row_base,
                                              int col_base, int lane, uint8_t* stage) {
  const int row = row_base + lane;
  const bool f32 = (eo.flags & (EPI_ATOMIC | EPI_OUT_F32)) != 0;
  const bool staged_ok = f32 ? (eo.ldd % 4 == 0) : (eo.ldd % 8 == 0 && !(eo.flags & EPI_ACCUM));
#pragma unroll 1
  for (int c = 0; c < nchunks; c += 2) {
    const int col0 = col_base + c * 32;
    if (col0 >= p.N) {  // whole pair of chunks is outside the matrix (tcgen05.ld is not needed)
      continue;
    }
    const bool pair_staged = staged_ok && (col0 + 64 <= p.N) && (c + 1 < nchunks);
    // both chunks of the pair are requested from tensor memory before the single wait: the epilogue is bound by the
    // latency of its dependent chain (two warps per scheduler), not by issue slots
    uint32_t rr[2][32];
    tmem_ld_32x32(t_addr + c * 32, rr[0]);  // warp-collective: never under a per-lane condition
    if (c + 1 < nchunks) tmem_ld_32x32(t_addr + (c + 1) * 32, rr[1]);
    tmem_ld_wait();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (c + h >= nchunks) break;
      const int cc = col0 + h * 32;
      if (cc >= p.N) continue;
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[h][j]);
      if (row < p.M) epilogue_math(p, eo, v, row, cc);
      if (!pair_staged) {
        if (row < p.M) epilogue_store_rowwise(p, eo, v, row, cc);
      } else if (f32) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          *reinterpret_cast<float4*>(stage + stage_off(lane, k)) = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
        stage_flush_f32(p, eo, stage, lane, row_base, cc);
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * k + 2 * j], v[8 * k + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h2);
          }
          *reinterpret_cast<uint4*>(stage + stage_off(lane, h * 4 + k)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (h == 1) stage_flush_bf16(p, eo, stage, lane, row_base, col0);
      }
    }
  }
}

// BATCHED: the tensor maps have a third (batch) dimension and the work list runs over batch x tiles; used for the
// per-head products of attention with head sizes the flash kernels do not cover.
template <int BN, int A_MN, int B_MN, bool BATCHED = false>
__global__ void __launch_bounds__(320, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int per_batch = tiles * p.split_k;
  const int total_work = per_batch * (BATCHED ? p.batch : 1);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int last_stage = -1;
      uint32_t last_phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; ok && work < total_work; work += gridDim.x) {
        const int bi = BATCHED ? work / per_batch : 0;
        const int w = work - bi * per_batch;
        const int ks = w / tiles;
        const int t = w - ks * tiles;
        const int nb = t / p.num_m_blocks;
        const int mb = t - nb * p.num_m_blocks;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_k_blocks);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* a_dst = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          if (A_MN == 0) {
            if (BATCHED) tma_load_3d(a_dst, &tmA, &full[stage], kb * 64, mb * 128, bi);
            else tma_load_2d(a_dst, &tmA, &full[stage], kb * 64, mb * 128);
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (BATCHED) tma_load_3d(a_dst + i * 8192, &tmA, &full[stage], mb * 128 + i * 64, kb * 64, bi);
              else tma_load_2d(a_dst + i * 8192, &tmA, &full[stage], mb * 128 + i * 64, kb * 64);
            }
          }
          if (B_MN == 0) {
            if (BATCHED) tma_load_3d(b_dst, &tmB, &full[stage], kb * 64, nb * BN, bi);
            else tma_load_2d(b_dst, &tmB, &full[stage], kb * 64, nb * BN);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) {
              if (BATCHED) tma_load_3d(b_dst + i * 8192, &tmB, &full[stage], nb * BN + i * 64, kb * 64, bi);
              else tma_load_2d(b_dst + i * 8192, &tmB, &full[stage], nb * BN + i * 64, kb * 64);
            }
          }
          last_stage = stage;
          last_phase = phase;
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      // On an abort, let the newest copy land before the CTA retires.
      if (!ok && last_stage >= 0) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(&full[last_stage], last_phase)) {
          if (globaltimer_ns() - t0 > 200000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; ok && work < total_work; work += gridDim.x) {
        const int ks = (BATCHED ? work % per_batch : work) / tiles;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_k_blocks);
        if (!wait_or_abort(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&full[stage], phase, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          // one descriptor per operand and k-block; its address field counts 16-byte units, so a k-step is an add
          const uint64_t ad0 = A_MN ? make_smem_desc(a_addr, 8192, 1024) : make_smem_desc(a_addr, 16, 1024);
          const uint64_t bd0 = B_MN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_ss(d_tmem, ad0 + k * (A_MN ? 128 : 2), bd0 + k * (B_MN ? 128 : 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          tc_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;  // eight epilogue warps: two per quarter, each takes half of the columns
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int work = blockIdx.x; work < total_work; work += gridDim.x) {
      const int bi = BATCHED ? work / per_batch : 0;
      const int w = work - bi * per_batch;
      const int ks = w / tiles;
      const int t = w - ks * tiles;
      const int nb = t / p.num_m_blocks;
      const int mb = t - nb * p.num_m_blocks;
      if (!wait_or_abort(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16) + half * (BN / 2);
      const long long d_off = BATCHED ? (long long)bi * p.batch_stride_d * ((p.flags & (EPI_ATOMIC | EPI_OUT_F32)) ? 4 : 2) : 0;
      const EpiOut eo = {static_cast<uint8_t*>(p.D) + d_off, p.ldd, p.flags};
      epilogue_warp(p, eo, t_addr, BN / 64, mb * 128 + q * 32, nb * BN + half * (BN / 2), lane,
                    smem + STAGES * Cfg::STAGE_BYTES + 256 + (warp - 2) * 4096);
      tc_fence_before();
      mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------- CTA-pair kernel
// The same product on 256 x 256 tiles computed by a CTA PAIR (cluster of two, `cta_group::2`): each CTA
// stages its own 128 rows of A and HALF of the B tile (128 of the 256 N rows) per k-block, the even CTA's
// MMA thread issues one 256 x 256 x 16 instruction that reads both CTAs' shared memory and writes 128
// accumulator rows into each CTA's TMEM. Per SM this halves the B traffic through shared memory, which is
// what limits the single-CTA kernel (12 KB per instruction read by the tensor core plus the same written
// by TMA), and leaves room for six stages.
//   full[s]   lives in the even CTA; both CTAs' TMA loads count their bytes on it (no multicast of data)
//   empty[s]  one per CTA, signalled by a multicast tcgen05.commit
//   tfull[a]  one per CTA (multicast commit); tempty[a] in the even CTA, 8 local + 8 remote warp arrivals
template <int BN, int COMM = 0>
struct Gemm2Cfg {
  static constexpr int A_BYTES = 128 * 64 * 2;
  static constexpr int B_BYTES = (BN / 2) * 64 * 2;  // this CTA's half of the BN-row B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // mode 1 (COMM == 1) gives one operand stage to the two 16 KB stages of its copy thread (the 384-wide tile has
  // the room to spare)
  static constexpr int COPY_BYTES = (COMM == 1) ? 2 * 16384 : 0;
  static constexpr int STAGES = (BN == 384) ? 4 : (BN == 256) ? 6 - (COMM == 1 ? 1 : 0) : 8 - (COMM == 1 ? 2 : 0);
  static constexpr int ACCS = (BN == 384) ? 1 : 2;  // 384 columns leave no room for a second accumulator
  static constexpr int COPY_OFF = STAGES * STAGE_BYTES + 256 + 8 * 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + 8 * 4096 + COPY_BYTES;  // + per-warp epilogue staging
};
static_assert(Gemm2Cfg<256, 1>::SMEM_BYTES <= 227 * 1024 && Gemm2Cfg<384, 1>::SMEM_BYTES <= 227 * 1024 &&
              Gemm2Cfg<128, 1>::SMEM_BYTES <= 227 * 1024, "mode-1 shared memory");

// Tile order of the tensor-parallel variants: the 256-row blocks are grouped by the rank that owns their rows;
// mode 1 runs the group of this rank first (its operand rows are already here), mode 2 runs it last (the partial
// sums for the peers have the longest way to go). Inside a group the row block index runs fastest, as in the
// plain order, so that neighbouring CTA pairs share a B tile.
template <int COMM>
__device__ __forceinline__ void pair_decode_tile(const GemmParams& p, const TpExt& x, int t, int& mb, int& nb) {
  if (COMM == 0 || x.pair_blocks_per_rank == 0) {
    nb = t / p.num_m_blocks;
    mb = t - nb * p.num_m_blocks;
    return;
  }
  const int bpr = x.pair_blocks_per_rank;
  const int per_group = bpr * p.num_n_blocks;
  const int g = t / per_group;
  const int u = t - g * per_group;
  const int owner = (x.rank + g + (COMM == 2 ? 1 : 0)) % x.tp;
  if (COMM == 1 && g > 0) {  // a peer's rows: row block by row block, the order they arrive in
    const int j = u / p.num_n_blocks;
    nb = u - j * p.num_n_blocks;
    mb = owner * bpr + j;
  } else {
    nb = u / bpr;
    mb = owner * bpr + (u - nb * bpr);
  }
}

// Reduce-scatter side: publish the partial sums this warp stored for its remote tiles. `upto` = first work item
// that is NOT covered (the warp has finished every tile before it). One system-scope fence, then one counter add
// per remote tile: the amount is the number of 32-column chunks the warp wrote, so the consumer's target,
// 4 x ceil(N / 32) per 128-row block and pass, does not depend on the tile width.
template <int BN>
__device__ __forceinline__ void tp_signal_remote_tiles(const GemmParams& p, const TpExt& x, int pair, int num_pairs, int upto,
                                                       uint32_t cta_rank, int half, int lane) {
  __syncwarp();
  if (lane == 0) {
    __threadfence_system();
    for (int work = pair; work < upto; work += num_pairs) {
      int mb, nb;
      pair_decode_tile<2>(p, x, work, mb, nb);
      const int row0 = mb * 256 + (int)cta_rank * 128;
      if (row0 >= p.M) continue;
      const int owner = row0 / x.rows_per_rank;
      if (owner == x.rank) continue;
      const int ncols = (BN == 384) ? 192 : BN / 2;
      const int c0 = nb * BN + half * ncols;
      const int c1 = min(c0 + ncols, p.N);
      if (c1 <= c0) continue;
      red_add_sys(x.arrived[owner] + (row0 - owner * x.rows_per_rank) / 128, (uint32_t)((c1 - c0 + 31) / 32));
    }
  }
  __syncwarp();
}

// Copy warp of mode 1 (one extra warp per CTA, one working thread): send this rank's rows of A to the peers with the
// bulk-copy unit while the tensor core works on the tiles of the rows that are already here. A piece is up to eight
// whole rows inside one 128-row block (at most TP_COPY_STAGE bytes); it is loaded from this rank's buffer into a
// shared-memory stage and stored from there into every peer's buffer (cp.async.bulk both ways, no multicast).
// Pieces are dealt to the CTAs of the grid in row order and each is published as soon as its stores have
// completed, so the row blocks fill up in the order in which the peers' GEMMs ask for them.
#define TP_COPY_WARPS 1
static constexpr int TP_COPY_STAGES = 2;
static constexpr int TP_COPY_STAGE = 16384;
__device__ __forceinline__ void tp_push_rows_bulk(const GemmParams& p, const TpExt& x, uint8_t* stage, uint64_t* bars,
                                                  int cta, int nctas) {
  const uint32_t row_bytes = (uint32_t)p.K * 2u;  // K % 8 == 0 and K * 2 <= TP_COPY_STAGE are checked on the host
  int piece_rows = 8;
  while (piece_rows > 1 && piece_rows * row_bytes > (uint32_t)TP_COPY_STAGE) piece_rows >>= 1;
  if (x.push_ld != p.K) piece_rows = 1;  // padded rows: only one row is contiguous
  const uint32_t bytes = piece_rows * row_bytes;
  const int total = (x.rows_per_rank / 128 - x.push_first_block) * (128 / piece_rows);
  const long long my0 = (long long)x.rank * x.rows_per_rank + (long long)x.push_first_block * 128;
  const int mine = total > cta ? (total - cta + nctas - 1) / nctas : 0;
  auto row_of = [&](int k) { return my0 + (long long)(cta + k * nctas) * piece_rows; };
  auto load = [&](int k) {
    const int s = k % TP_COPY_STAGES;
    mbar_expect_tx(&bars[s], bytes);
    bulk_load_g2s(stage + s * TP_COPY_STAGE, x.push_src + row_of(k) * x.push_ld, bytes, &bars[s]);
  };
  auto publish = [&](int k) {  // the stores of piece k have completed
    __threadfence_system();
    const long long r0 = row_of(k);
    for (int i = 0; i < x.push_n; ++i) red_add_sys(x.push_ready[i] + (r0 >> 7), (uint32_t)piece_rows);
  };
  int issued = 0, done = 0;
  for (; issued < mine && issued < TP_COPY_STAGES; ++issued) load(issued);
  for (int k = 0; k < mine; ++k) {
    const int s = k % TP_COPY_STAGES;
    if (!mbar_wait(&bars[s], (uint32_t)((k / TP_COPY_STAGES) & 1))) {
      if (p.status) atomicOr(p.status, ST_TIMEOUT_PRODUCER);
      break;
    }
    const long long r0 = row_of(k);
    for (int i = 0; i < x.push_n; ++i) bulk_store_s2g(x.push_dst[i] + r0 * x.push_ld, stage + s * TP_COPY_STAGE, bytes);
    bulk_commit_group();
    done = k + 1;
    if (k >= 1) {
      asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");  // piece k - 1 has arrived: its stage is free as well
      publish(k - 1);
      if (issued < mine) load(issued++);
    }
  }
  bulk_wait_group0();
  if (done) publish(done - 1);
  // loads issued but not consumed (only after a time-out): let them land before the block's shared memory goes away
  for (int k = done; k < issued; ++k) mbar_wait(&bars[k % TP_COPY_STAGES], (uint32_t)((k / TP_COPY_STAGES) & 1));
}

template <int BN, int A_MN, int B_MN, int COMM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(COMM == 1 ? 320 + 32 * TP_COPY_WARPS : 320, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                              const GemmParams p, const __grid_constant__ TpExt tpx) {
  using Cfg = Gemm2Cfg<BN, COMM>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int HALF = BN / 2;  // B rows (output columns) staged by each CTA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs, 1: partner
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 16);
    }
    if (COMM == 1)
      for (int s = 0; s < TP_COPY_STAGES; ++s) mbar_init(&full[24 + s], 1);  // copy thread's stages (byte 192 of the barrier block)
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers and tensor memory exist before anything refers to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.num_m_blocks * p.num_n_blocks;  // in units of 256 x BN
  const int total_work = tiles * p.split_k;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t a_want = (COMM == 1) ? 128u * *tpx.pass : 0u;
      for (int work = pair; ok && work < total_work; work += num_pairs) {
        const int ks = work / tiles;
        const int t = work - ks * tiles;
        int mb, nb;
        pair_decode_tile<COMM>(p, tpx, t, mb, nb);
        const int row0 = mb * 256 + (int)rank * 128;   // this CTA's rows of A
        const int col0 = nb * BN + (int)rank * HALF;   // this CTA's rows of B (output columns)
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_k_blocks);
        if (COMM == 1 && row0 < p.M && row0 / tpx.rows_per_rank != tpx.rank) {
          // rows pushed by their owner: wait until the whole 128-row block has landed, then make the peer's
          // (generic-proxy) stores visible to the TMA reads that follow
          if (!spin_until<true>(tpx.a_ready + (row0 >> 7), a_want)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_PEER);
            ok = false;
            break;
          }
          fence_proxy_async_all();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
          uint8_t* a_dst = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          if (A_MN == 0) {
            tma_load_2d_pair(a_dst, &tmA, bar, kb * 64, row0);
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) tma_load_2d_pair(a_dst + i * 8192, &tmA, bar, row0 + i * 64, kb * 64);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(b_dst, &tmB, bar, kb * 64, col0);
          } else {
#pragma unroll
            for (int i = 0; i < HALF / 64; ++i) tma_load_2d_pair(b_dst + i * 8192, &tmB, bar, col0 + i * 64, kb * 64);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, BN == 384 ? 256 : BN, A_MN, B_MN);
      constexpr uint32_t idesc_tail = make_idesc_bf16(256, 128, A_MN, B_MN);  // BN == 384 only
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int work = pair; ok && work < total_work; work += num_pairs) {
        const int ks = work / tiles;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.num_k_blocks);
        if (!wait_or_abort(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (BN == 384 ? 0 : BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!wait_or_abort(&full[stage], phase, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          const uint64_t ad0 = A_MN ? make_smem_desc(a_addr, 8192, 1024) : make_smem_desc(a_addr, 16, 1024);
          const uint64_t bd0 = B_MN ? make_smem_desc(b_addr, 8192, 1024) : make_smem_desc(b_addr, 16, 1024);
          // this CTA's B rows 128..191 (BN == 384 only): two 64-row boxes further when MN-major
          const uint64_t bt0 = B_MN ? make_smem_desc(b_addr + 2 * 8192, 8192, 1024) : make_smem_desc(b_addr + 128 * 128, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t ad = ad0 + k * (A_MN ? 128 : 2);
            tc_mma_ss_pair(d_tmem, ad, bd0 + k * (B_MN ? 128 : 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            if (BN == 384) tc_mma_ss_pair(d_tmem + 256, ad, bt0 + k * (B_MN ? 128 : 2), idesc_tail, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty[stage], 3);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit_pair(&tfull[acc], 3);
        if (Cfg::ACCS == 2) acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (COMM == 1 && warp >= 10) {
    if (tpx.push_n > 0)
      if (lane == 0) tp_push_rows_bulk(p, tpx, smem + Cfg::COPY_OFF, &full[24], (int)blockIdx.x, (int)gridDim.x);
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t tempty_remote[2] = {mapa_shared(smem_u32(&tempty[0]), 0), mapa_shared(smem_u32(&tempty[1]), 0)};
    bool unsignalled = false;  // COMM == 2: remote tiles stored but not yet published
    int work = pair;
    for (; work < total_work; work += num_pairs) {
      const int ks = work / tiles;
      const int t = work - ks * tiles;
      int mb, nb;
      pair_decode_tile<COMM>(p, tpx, t, mb, nb);
      const int row_cta = mb * 256 + (int)rank * 128;
      EpiOut eo = {p.D, p.ldd, p.flags};
      if (COMM == 2) {
        const int owner = min(row_cta / tpx.rows_per_rank, tpx.tp - 1);
        const bool remote = owner != tpx.rank;
        if (!remote && unsignalled) {  // the last remote tile of this CTA is behind us
          tp_signal_remote_tiles<BN>(p, tpx, pair, num_pairs, work, rank, half, lane);
          unsignalled = false;
        }
        // block of the owning rank, addressed with the global row index
        eo.D = reinterpret_cast<__nv_bfloat16*>(tpx.out[owner]) - (long long)owner * tpx.rows_per_rank * tpx.ldo;
        eo.ldd = tpx.ldo;
        if (remote) eo.flags = p.flags & ~EPI_BIAS;
        unsignalled = unsignalled || (remote && row_cta < p.M);
      }
      if (!wait_or_abort(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      uint8_t* stage_tile = smem + STAGES * Cfg::STAGE_BYTES + 256 + (warp - 2) * 4096;
      const int row_base = row_cta + q * 32;
      if (BN == 384) {
        // warp half h owns output columns [h*192, h*192+192): 128 from the first product, 64 from the second
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        epilogue_warp(p, eo, t_lane + half * 128, 4, row_base, nb * BN + half * 192, lane, stage_tile);
        epilogue_warp(p, eo, t_lane + 256 + half * 64, 2, row_base, nb * BN + half * 192 + 128, lane, stage_tile);
      } else {
        const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16) + half * HALF;
        epilogue_warp(p, eo, t_addr, HALF / 32, row_base, nb * BN + half * HALF, lane, stage_tile);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_remote[acc]);
      if (Cfg::ACCS == 2) acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    // also after an aborted loop: whatever was stored is published, the peers' counters stay consistent
    if (COMM == 2 && unsignalled) tp_signal_remote_tiles<BN>(p, tpx, pair, num_pairs, work, rank, half, lane);
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // no CTA frees tensor memory or exits while its partner may still touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

int encode_tmap_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box,
                     const uint32_t* elem_strides) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = elem_strides ? elem_strides[i] : 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdim, gstr,
                  bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 100;
}

// Same as encode_tmap_bf16 for fp32 elements (128-byte swizzle: the inner box extent is at most 32 elements).
int encode_tmap_f32(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 100;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, int A_MN, int B_MN, bool BATCHED = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN, BATCHED>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmCfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
    attr_set = true;
  }
  kern<<<grid, 320, GemmCfg<BN>::SMEM_BYTES, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

template <int BN, int A_MN, int B_MN, int COMM = 0>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream,
                            const TpExt& tpx = TpExt{}) {
  auto kern = gemm_bf16_tcgen05_pair_kernel<BN, A_MN, B_MN, COMM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Cfg<BN, COMM>::SMEM_BYTES);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
    attr_set = true;
  }
  kern<<<grid, COMM == 1 ? 320 + 32 * TP_COPY_WARPS : 320, Gemm2Cfg<BN, COMM>::SMEM_BYTES, stream>>>(ta, tb, p, tpx);  // cluster of two through __cluster_dims__
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

}  // namespace tnnb

using namespace tnnb;

static int gemm_dispatch(const void* A, const void* B, void* D, int M, int N, int K, int a_mn,
                         int b_mn, long long lda, long long ldb, long long ldd,
                         const void* bias, const void* aux_in, void* aux_out,
                         long long ld_aux, const void* resid, long long ld_res, int flags,
                         int split_k, int force_bn, int* status, void* stream_, const TpExt* tpx) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((lda % 8) || (ldb % 8)) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -4;
  if ((flags & EPI_BIAS) && !bias) return -5;
  if ((flags & EPI_DGELU) && !aux_in) return -5;
  if ((flags & EPI_RESID) && !resid) return -5;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  // 256 x 256 tiles on CTA pairs whenever the problem has at least one such tile's worth of rows and
  // columns (force_bn: 512 forces the pair kernel, 128 / 256 force the single-CTA tile widths)
  int pair_bn = 0;  // force_bn = 1024 + 256 / 384: the pair kernel with that tile width
  if (force_bn >= 1024) {
    pair_bn = force_bn - 1024;
    force_bn = 512;
  }
  const bool pair = (force_bn == 512) || (force_bn == 0 && M > 128 && N > 128);
  p.num_m_blocks = pair ? (M + 255) / 256 : (M + 127) / 128;
  p.num_k_blocks = (K + 63) / 64;
  int bn = force_bn;
  if (pair) {
    // 256-wide tiles (narrower pair tiles are limited by shared-memory bandwidth: A is re-read per 128
    // columns), or 384-wide ones with a single accumulator when they need clearly fewer waves of CTA pairs
    // (N = 768 with 8192 rows: 64 tiles on 74 pairs instead of 96).
    const int units = sm_count() / 2;
    const long long sk = split_k > 0 ? split_k : 1;
    const long long w256 = ((long long)p.num_m_blocks * ((N + 255) / 256) * sk + units - 1) / units * 256;
    const long long w384 = ((long long)p.num_m_blocks * ((N + 383) / 384) * sk + units - 1) / units * 384;
    bn = ((force_bn == 0 || tpx) && !(flags & EPI_ATOMIC) && w384 * 10 <= w256 * 8) ? 384 : 256;
    if (pair_bn == 256 || pair_bn == 384) bn = pair_bn;
  } else if (bn != 128 && bn != 256) {
    const int t256 = p.num_m_blocks * ((N + 255) / 256);
    bn = (N > 128 && t256 * (split_k > 0 ? split_k : 1) >= sm_count()) ? 256 : 128;
    if (N > 128 && (flags & EPI_ATOMIC)) bn = 256;
  }
  p.num_n_blocks = (N + bn - 1) / bn;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  if (split_k <= 0) {
    split_k = 1;
    if (flags & EPI_ATOMIC) {
      // Enough (tile, k-range) work items to fill the machine about twice.
      const int units = pair ? sm_count() / 2 : sm_count();
      const int want = (2 * units + tiles - 1) / tiles;
      split_k = max(1, min(want, p.num_k_blocks / 4 > 0 ? p.num_k_blocks / 4 : 1));
    }
  }
  if (split_k > 1 && !(flags & EPI_ATOMIC)) return -6;
  split_k = min(split_k, p.num_k_blocks);
  p.kb_per_split = (p.num_k_blocks + split_k - 1) / split_k;
  p.split_k = (p.num_k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  p.D = D; p.ldd = ldd;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  p.ld_aux = ld_aux;
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.ld_res = ld_res;
  p.flags = flags;
  p.status = status;
  p.batch = 1;
  p.batch_stride_d = 0;

  CUtensorMap ta, tb;
  int rc;
  if (!a_mn) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, 128};
    rc = encode_tmap_bf16(&ta, A, 2, dims, str, box, nullptr);
  } else {
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, 64};
    rc = encode_tmap_bf16(&ta, A, 2, dims, str, box, nullptr);
  }
  if (rc) return rc;
  if (!b_mn) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, pair ? (uint32_t)bn / 2 : (uint32_t)bn};
    rc = encode_tmap_bf16(&tb, B, 2, dims, str, box, nullptr);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, 64};
    rc = encode_tmap_bf16(&tb, B, 2, dims, str, box, nullptr);
  }
  if (rc) return rc;

  if (pair && tpx) {
    // tensor-parallel variants: A is always K-major, no split-K
    if (a_mn || p.split_k != 1) return -6;
    const int grid2 = 2 * min(tiles, sm_count() / 2);
#define TNNB_TP(BN_, BM_, CM) return launch_gemm_pair<BN_, 0, BM_, CM>(ta, tb, p, grid2, stream, *tpx)
    if (tpx->mode == 1) {
      if (bn == 256) { if (b_mn) TNNB_TP(256, 1, 1); TNNB_TP(256, 0, 1); }
      if (b_mn) TNNB_TP(384, 1, 1); TNNB_TP(384, 0, 1);
    } else {
      if (bn == 256) { if (b_mn) TNNB_TP(256, 1, 2); TNNB_TP(256, 0, 2); }
      if (b_mn) TNNB_TP(384, 1, 2); TNNB_TP(384, 0, 2);
    }
#undef TNNB_TP
  }
  if (pair) {
    const int grid2 = 2 * min(tiles * p.split_k, sm_count() / 2);
#define TNNB_PAIR(BN_, AM, BM_) return launch_gemm_pair<BN_, AM, BM_>(ta, tb, p, grid2, stream)
    if (bn == 256) {
      if (!a_mn && !b_mn) TNNB_PAIR(256, 0, 0);
      if (!a_mn && b_mn) TNNB_PAIR(256, 0, 1);
      if (a_mn && !b_mn) TNNB_PAIR(256, 1, 0);
      TNNB_PAIR(256, 1, 1);
    }
    if (!a_mn && !b_mn) TNNB_PAIR(384, 0, 0);
    if (!a_mn && b_mn) TNNB_PAIR(384, 0, 1);
    if (a_mn && !b_mn) TNNB_PAIR(384, 1, 0);
    TNNB_PAIR(384, 1, 1);
#undef TNNB_PAIR
  }
  const int grid = min(tiles * p.split_k, sm_count());
#define TNNB_LAUNCH(BN_, AM, BM_) return launch_gemm<BN_, AM, BM_>(ta, tb, p, grid, stream)
  if (bn == 256) {
    if (!a_mn && !b_mn) TNNB_LAUNCH(256, 0, 0);
    if (!a_mn && b_mn) TNNB_LAUNCH(256, 0, 1);
    if (a_mn && !b_mn) TNNB_LAUNCH(256, 1, 0);
    TNNB_LAUNCH(256, 1, 1);
  } else {
    if (!a_mn && !b_mn) TNNB_LAUNCH(128, 0, 0);
    if (!a_mn && b_mn) TNNB_LAUNCH(128, 0, 1);
    if (a_mn && !b_mn) TNNB_LAUNCH(128, 1, 0);
    TNNB_LAUNCH(128, 1, 1);
  }
#undef TNNB_LAUNCH
}

extern "C" int tnnb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int a_mn,
                              int b_mn, long long lda, long long ldb, long long ldd,
                              const void* bias, const void* aux_in, void* aux_out,
                              long long ld_aux, const void* resid, long long ld_res, int flags,
                              int split_k, int force_bn, int* status, void* stream_) {
  return gemm_dispatch(A, B, D, M, N, K, a_mn, b_mn, lda, ldb, ldd, bias, aux_in, aux_out, ld_aux, resid, ld_res, flags,
                       split_k, force_bn, status, stream_, nullptr);
}

// `batch` independent products D[b] = op(A[b]) * op(B[b])^T on the single-CTA kernel: operand b starts stride_a /
// stride_b elements after operand b - 1 (multiples of 8), output b stride_d elements of D's type after the previous
// one. flags: 0 (bf16 output) or EPI_OUT_F32. Used for attention with head sizes other than 64: scores and
// probabilities of all heads in one launch each.
extern "C" int tnnb_gemm_bf16_batched(const void* A, const void* B, void* D, int M, int N, int K, int a_mn, int b_mn,
                                      long long lda, long long ldb, long long ldd, int batch, long long stride_a,
                                      long long stride_b, long long stride_d, int flags, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -2;
  if ((lda % 8) || (ldb % 8) || (stride_a % 8) || (stride_b % 8)) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -4;
  if (flags & ~EPI_OUT_F32) return -6;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.num_m_blocks = (M + 127) / 128;
  p.num_k_blocks = (K + 63) / 64;
  const int bn = (N > 128) ? 256 : 128;
  p.num_n_blocks = (N + bn - 1) / bn;
  p.split_k = 1;
  p.kb_per_split = p.num_k_blocks;
  p.D = D; p.ldd = ldd;
  p.flags = flags;
  p.status = status;
  p.batch = batch;
  p.batch_stride_d = stride_d;
  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[3] = {(uint64_t)(a_mn ? M : K), (uint64_t)(a_mn ? K : M), (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)lda * 2, (uint64_t)stride_a * 2};
    uint32_t box[3] = {64, (uint32_t)(a_mn ? 64 : 128), 1};
    if ((rc = encode_tmap_bf16(&ta, A, 3, dims, str, box, nullptr))) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)(b_mn ? N : K), (uint64_t)(b_mn ? K : N), (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)ldb * 2, (uint64_t)stride_b * 2};
    uint32_t box[3] = {64, (uint32_t)(b_mn ? 64 : bn), 1};
    if ((rc = encode_tmap_bf16(&tb, B, 3, dims, str, box, nullptr))) return rc;
  }
  const int grid = min(p.num_m_blocks * p.num_n_blocks * batch, sm_count());
#define TNNB_B(BN_, AM, BM_) return launch_gemm<BN_, AM, BM_, true>(ta, tb, p, grid, stream)
  if (bn == 256) {
    if (!a_mn && !b_mn) TNNB_B(256, 0, 0);
    if (!a_mn && b_mn) TNNB_B(256, 0, 1);
    if (a_mn && !b_mn) TNNB_B(256, 1, 0);
    TNNB_B(256, 1, 1);
  }
  if (!a_mn && !b_mn) TNNB_B(128, 0, 0);
  if (!a_mn && b_mn) TNNB_B(128, 0, 1);
  if (a_mn && !b_mn) TNNB_B(128, 1, 0);
  TNNB_B(128, 1, 1);
#undef TNNB_B
}

// Tensor-parallel GEMMs on the CTA-pair kernel (protocol: tp_flags.cuh). A is [M, K] K-major.
//   mode 1  Y[M, N] = A * op(B)^T where the rows of A owned by other ranks (row r belongs to rank
//           r / rows_per_rank) are pushed into A by their owners; a_ready = this rank's counters [M / 128].
//   mode 2  partial sums of the rows owned by rank o go to out[o] ([rows_per_rank, ldo], bf16): out[rank] is the
//           local output (bias applied), out[o != rank] this rank's slot in o's inbox; arrived[o] = rank o's
//           counters [rows_per_rank / 128]. D / ldd are ignored.
//           n_push > 0: the kernel also sends this rank's rows of A to n_push peers (push_dst[i] = base of peer i's
//           A buffer, push_ready[i] = peer i's counters), starting at its 128-row block push_first_block - the
//           blocks before it were delivered by the kernel that produced the rows; 0 when that kernel delivered all.
// pass = device word holding the number of passes including this one. out / arrived are arrays of tp pointers.
extern "C" int tnnb_gemm_tp(int mode, const void* A, const void* B, void* D, int M, int N, int K, int b_mn, long long lda,
                            long long ldb, long long ldd, const void* bias, const void* aux_in, void* aux_out, long long ld_aux,
                            int flags, int tp, int rank, int rows_per_rank, const void* pass, const void* a_ready, void** out,
                            long long ldo, void** arrived, int n_push, void** push_dst, void** push_ready, int push_first_block,
                            int force_bn, int* status, void* stream_) {
  if (mode != 1 && mode != 2) return -2;
  if (tp < 1 || tp > TP_MAX || rank < 0 || rank >= tp || !pass) return -2;
  if (rows_per_rank <= 0 || rows_per_rank % 128 || (long long)rows_per_rank * tp != M) return -8;
  if (flags & (EPI_ATOMIC | EPI_OUT_F32 | EPI_ACCUM | EPI_RESID)) return -6;
  TpExt x{};
  x.mode = mode; x.tp = tp; x.rank = rank; x.rows_per_rank = rows_per_rank;
  x.pair_blocks_per_rank = (rows_per_rank % 256 == 0) ? rows_per_rank / 256 : 0;
  x.pass = static_cast<const uint32_t*>(pass);
  x.status = status;
  if (mode == 1) {
    if (!a_ready || !D) return -5;
    x.a_ready = static_cast<const uint32_t*>(a_ready);
    if (n_push < 0 || n_push > TP_MAX - 1) return -2;
    if (n_push > 0) {
      if (!push_dst || !push_ready || (K % 8)) return -5;
      if ((long long)K * 2 > TP_COPY_STAGE) return -3;  // a row must fit one stage of the copy thread
      if (push_first_block < 0 || push_first_block > rows_per_rank / 128) return -3;
      x.push_n = n_push;
      x.push_first_block = push_first_block;
      x.push_src = static_cast<const __nv_bfloat16*>(A);
      x.push_ld = lda;
      for (int i = 0; i < n_push; ++i) {
        if (!push_dst[i] || !push_ready[i] || (reinterpret_cast<uintptr_t>(push_dst[i]) & 15)) return -4;
        x.push_dst[i] = static_cast<__nv_bfloat16*>(push_dst[i]);
        x.push_ready[i] = static_cast<uint32_t*>(push_ready[i]);
      }
    }
  } else {
    if (!out || !arrived || (ldo % 8)) return -5;
    for (int o = 0; o < tp; ++o) {
      if (!out[o] || (o != rank && !arrived[o])) return -5;
      x.out[o] = out[o];
      x.arrived[o] = static_cast<uint32_t*>(arrived[o]);
    }
    x.ldo = ldo;
    D = out[rank];
    ldd = ldo;
  }
  const int fb = (force_bn == 256 || force_bn == 384) ? force_bn + 1024 : 512;  // always the pair kernel
  return gemm_dispatch(A, B, D, M, N, K, 0, b_mn, lda, ldb, ldd, bias, aux_in, aux_out, ld_aux, nullptr, 0, flags, 1, fb,
                       status, stream_, &x);
}
