// Flash attention for sm_100a (head dim 64, bf16, causal or full), forward and
// backward, on tcgen05 tensor cores with TMEM accumulators and TMA-fed tiles.
//
// Q, K, V are read straight out of the packed projection output
// qkv[B, S, 3, H, 64] and O / dO use [B, S, H, 64], so none of the
// [B,S,H,D] <-> [B,H,S,D] transposes of the reference block exist here
// (src/nn/blocks_impl/flash_attention_block.cpp:109-132,193-250 launches 4 in
// forward and 8 in backward around cuDNN's sdpa / sdpa_backward graphs,
// src/nn/engines/cudnn_engine.cu:1479-1621).
//
// Forward, one CTA per (128-row Q tile, head, batch), two CTAs per SM:
//   warp 0   TMA: Q once, then (K_j, V_j) into a two-stage ring
//   warp 1   MMA: S = Q K_j^T -> TMEM; after the softmax warps have published
//            P_j (bf16, 128B-swizzled shared memory) O_j = P_j V_j -> TMEM
//   warps 2-5  one thread per Q row (TMEM lane == row): online softmax with no
//            shuffles, running O kept in registers, O_j folded in from TMEM
// Memory is O(S): only the log-sum-exp per row is kept for the backward.
//
// Backward = a row-wise preprocess (delta = sum O*dO) and two tile kernels that
// recompute P from Q, K and the saved log-sum-exp:
//   dK/dV  one CTA per K/V tile, loops over Q tiles, transposed products so
//          that every shared-memory operand it writes is K-major:
//          S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q
//   dQ     one CTA per Q tile, loops over K/V tiles: dQ += dS K
// K, V, Q, dO tiles double as MN-major operands (their rows become the
// reduction index), so no transposed copy is ever made.
// All barrier waits are bounded (status word + CTA abort flag).
#include "gemm_tcgen05.h"
#include "ptx.cuh"

namespace tnnb {

typedef __nv_bfloat16 bf16;

struct AttnParams {
  int B, S, H;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  bf16* O;           // [B,S,H,64]
  float* LSE;        // [B,H,S] in scaled log2 units
  const float* delta;  // [B,H,S]
  float* dq_acc;       // [B,S,H,64] fp32, zeroed before the backward kernel
  bf16* dQ;          // dqkv + 0        row pitch 3*H*64
  bf16* dK;          // dqkv + H*64
  bf16* dV;          // dqkv + 2*H*64
  int* status;
};

static constexpr int TILE_BYTES = 128 * 64 * 2;  // one [128 x 64] bf16 tile

#ifdef TNNB_TRACE
// Debug builds only: per-phase clock64 stamps of CTA (0,0,0), compute warp 2 lane 0 and the MMA thread.
__device__ long long g_trace[2][512];
#define TRACE(who, idx) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (idx) < 512) g_trace[who][idx] = clock64(); } while (0)
#else
#define TRACE(who, idx) do { } while (0)
#endif

__device__ __forceinline__ void tmem_ld_32x32f(uint32_t taddr, float (&f)[32]) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
}

// Write 32 fp32 values of row `row` as bf16 into columns [c0, c0+32) of a
// K-major 128B-swizzled [128 x 128] tile made of two [128 x 64] blocks.
__device__ __forceinline__ void store_row_chunk_sw128(uint8_t* tile, int row, int c0, const float (&f)[32]) {
  uint8_t* blk = tile + (c0 >> 6) * TILE_BYTES;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    __align__(16) bf16 t[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) t[k] = __float2bfloat16(f[c * 8 + k]);
    *reinterpret_cast<uint4*>(blk + sw128_offset(row, chunk0 + c)) = *reinterpret_cast<uint4*>(t);
  }
}

// ------------------------------------------------------------------ forward
// One CTA per PAIR of 128-row Q tiles (A = rows [q0, q0+128), B = the next 128), one CTA per SM:
//   warp 0      TMA: both Q tiles once, then (K_j, V_j) into a two-stage ring shared by A and B
//   warp 1      MMA: S_X = Q_X K_j^T -> TMEM (128 columns each), O_X += P_X V_j accumulated IN TMEM
//   warps 2-5   softmax of tile A, warps 6-9 softmax of tile B: one thread per Q row (TMEM lane)
// While one tile's threads are busy with exponentials the tensor core runs the other tile's products
// and the next S of the same tile (S is consumed into registers in one tcgen05.ld, which frees its
// TMEM columns at once). The running maximum is only raised when a row's new maximum exceeds it by
// more than 2^8 ("lazy rescale"): then, and only then, O is corrected in TMEM (ld, scale, st).
struct FwdSmem {
  static constexpr int Q = 0;                          // two [128 x 64] tiles
  static constexpr int K0 = Q + 2 * TILE_BYTES;        // stage s: K at K0 + s*2*TILE, V right after
  static constexpr int P = K0 + 4 * TILE_BYTES;        // P_A then P_B, [128 x 128] bf16 each
  static constexpr int BARS = P + 4 * TILE_BYTES;
  static constexpr int TOTAL = BARS + 256;
};

__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_ARG);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FwdSmem::BARS);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;    // [2]  per Q tile
  uint64_t* s_free = bars + 7;    // [2]
  uint64_t* p_ready = bars + 9;   // [2]
  uint64_t* o_full = bars + 11;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the tile index is the slowest grid dimension and runs backwards: every head's heaviest (latest) causal
  // tiles are handed out first and the lightest fill the tail of the last wave
  const int pair = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int q0 = pair * 256;
  const int n_kv_all = (p.S + 127) / 128;
  // number of K/V tiles each Q tile needs (causal: up to and including its diagonal tile)
  const int n_a = p.causal ? min(2 * pair + 1, n_kv_all) : n_kv_all;
  const int n_b = p.causal ? min(2 * pair + 2, n_kv_all) : n_kv_all;
  const int n_kv = n_b;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 4);
      mbar_init(&p_ready[s], 128);
      mbar_init(&o_full[s], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S_A 0..127, S_B 128..255, O_A 256..319, O_B 320..383

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      tma_load_4d(smem + FwdSmem::Q, &tmQ, q_full, 0, h, q0, b);
      tma_load_4d(smem + FwdSmem::Q + TILE_BYTES, &tmQ, q_full, 0, h, q0 + 128, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (!wait_or_abort(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
          break;
        }
        mbar_expect_tx(&kv_full[s], 2 * TILE_BYTES);
        uint8_t* kdst = smem + FwdSmem::K0 + s * 2 * TILE_BYTES;
        tma_load_4d(kdst, &tmK, &kv_full[s], 0, h, j * 128, b);
        tma_load_4d(kdst + TILE_BYTES, &tmV, &kv_full[s], 0, h, j * 128, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
      const uint32_t q_addr = smem_u32(smem + FwdSmem::Q);
      const uint32_t p_addr = smem_u32(smem + FwdSmem::P);
      // This one thread issues 24 MMAs per K/V step. Everything about their descriptors that does not change is
      // built once: the address field of a descriptor counts 16-byte units, so a k-step or a stage is an add.
      constexpr uint32_t T16 = TILE_BYTES / 16;
      const uint64_t q_desc = make_smem_desc(q_addr, 16, 1024);                                       // + x * T16
      const uint64_t p_desc = make_smem_desc(p_addr, 16, 1024);                                       // + x * 2 * T16
      const uint64_t k_desc = make_smem_desc(smem_u32(smem + FwdSmem::K0), 16, 1024);                 // + stage * 2 * T16
      const uint64_t v_desc = make_smem_desc(smem_u32(smem + FwdSmem::K0 + TILE_BYTES), 8192, 1024);  // + stage * 2 * T16
      auto issue_qk = [&](int x, int j) {
        const uint64_t qd = q_desc + x * T16, kd = k_desc + (j & 1) * 2 * T16;
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_ss(tmem_base + x * 128, qd + k * 2, kd + k * 2, idesc_s, k > 0);
        tc_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j) {
        const uint64_t pd = p_desc + x * 2 * T16, vd = v_desc + (j & 1) * 2 * T16;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_ss(tmem_base + 256 + x * 64, pd + (k >> 2) * T16 + (k & 3) * 2, vd + k * 128, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(&o_full[x]);
      };
      bool ok = wait_or_abort(q_full, 0, abort_flag) && wait_or_abort(&kv_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        issue_qk(1, 0);
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        if (j + 1 < n_kv) {  // next scores first: they overlap with this step's softmax
          ok = wait_or_abort(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag);
          if (ok && j + 1 < n_a) {
            ok = wait_or_abort(&s_free[0], j & 1, abort_flag);
            if (ok) {
              tc_fence_after();
              issue_qk(0, j + 1);
            }
          }
          if (ok) ok = wait_or_abort(&s_free[1], j & 1, abort_flag);
          if (ok) {
            tc_fence_after();
            issue_qk(1, j + 1);
          }
        }
        if (ok && j < n_a) {
          ok = wait_or_abort(&p_ready[0], j & 1, abort_flag);
          if (ok) {
            tc_fence_after();
            issue_pv(0, j);
          }
        }
        if (ok) ok = wait_or_abort(&p_ready[1], j & 1, abort_flag);
        if (ok) {
          tc_fence_after();
          issue_pv(1, j);
          tc_commit(&kv_empty[j & 1]);
        }
      }
      if (!ok) raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
    }
  } else {
    const int x = (warp - 2) >> 2;  // 0: tile A, 1: tile B
    const int quarter = warp & 3;   // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;
    const int q_idx = q0 + x * 128 + row;
    const int n_x = x ? n_b : n_a;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tm_S = tmem_base + x * 128 + lane_off;
    const uint32_t tm_O = tmem_base + 256 + x * 64 + lane_off;
    uint8_t* p_tile = smem + FwdSmem::P + x * 2 * TILE_BYTES;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_x; ++j) {
      if (!wait_or_abort(&s_full[x], j & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sr[128];
      tmem_ld_32x128_wait(tm_S, sr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[x]);  // S_X may be overwritten by the next product
      const int kv0 = j * 128;
      const bool need_mask = (p.causal && kv0 + 127 > q0 + x * 128) || (kv0 + 128 > p.S);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const int kv = kv0 + i;
          if ((p.causal && kv > q_idx) || kv >= p.S) sr[i] = 0xff800000u;  // -inf
        }
      }
      float mx0 = __uint_as_float(sr[0]), mx1 = __uint_as_float(sr[1]), mx2 = __uint_as_float(sr[2]),
            mx3 = __uint_as_float(sr[3]);
#pragma unroll
      for (int i = 4; i < 128; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
        mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
      }
      const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
      bool waited_o = false;
      if (j == 0) {
        m_run = (m_tile == -INFINITY) ? 0.f : m_tile;
      } else {
        const bool raise = m_tile > m_run + 8.f;
        if (__any_sync(0xffffffffu, raise)) {  // warp-uniform: tcgen05.ld/st are warp-collective
          float alpha = 1.f;
          if (raise) {
            alpha = exp2f(m_run - m_tile);
            m_run = m_tile;
            l_run *= alpha;
          }
          if (!wait_or_abort(&o_full[x], (j - 1) & 1, abort_flag)) {
            ok = false;
            break;
          }
          waited_o = true;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tm_O + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tm_O + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // P_X(j-1) must have been consumed before its shared-memory tile is overwritten
      if (j > 0 && !waited_o && !wait_or_abort(&o_full[x], (j - 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint32_t pk[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float e0 = exp2f(fmaf(__uint_as_float(sr[c * 8 + 2 * k]), p.scale_log2, -m_run));
          const float e1 = exp2f(fmaf(__uint_as_float(sr[c * 8 + 2 * k + 1]), p.scale_log2, -m_run));
          l0 += e0;
          l1 += e1;
          __nv_bfloat162 h2 = __floats2bfloat162_rn(e0, e1);
          pk[k] = *reinterpret_cast<uint32_t*>(&h2);
        }
        *reinterpret_cast<uint4*>(p_tile + (c >> 3) * TILE_BYTES + sw128_offset(row, c & 7)) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run += l0 + l1;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready[x]);
    }
    if (!ok && lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
    if (ok && n_x > 0) {
      if (wait_or_abort(&o_full[x], (n_x - 1) & 1, abort_flag)) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        bf16* orow = p.O + (((long long)b * p.S + q_idx) * p.H + h) * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tm_O + c * 32, r);
          tmem_ld_wait();
          if (q_idx < p.S) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t pk[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * k]) * inv,
                                                           __uint_as_float(r[g * 8 + 2 * k + 1]) * inv);
                pk[k] = *reinterpret_cast<uint32_t*>(&h2);
              }
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
        if (q_idx < p.S && p.LSE)
          p.LSE[((long long)b * p.H + h) * p.S + q_idx] = (l_run > 0.f) ? m_run + log2f(l_run) : INFINITY;
      } else if (lane == 0) {
        raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// --------------------------------------------------------------- preprocess
// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d]. Eight lanes per (b,s,h) row of 64 values, 16 bytes per lane and
// tensor, so a warp covers four rows per trip with two 512-byte requests (both tensors are 16-byte aligned: the
// entry point checks it).
__global__ void attn_delta_kernel(const bf16* __restrict__ O, const bf16* __restrict__ dO,
                                  float* __restrict__ delta, int B, int S, int H) {
  const long long total = (long long)B * S * H;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  {
    const int sub = lane >> 3, l8 = lane & 7;
    for (long long g = warp0; g * 4 < total; g += nwarps) {
      const long long r = g * 4 + sub;
      float v = 0.f;
      if (r < total) {
        const uint4 a = reinterpret_cast<const uint4*>(O + r * 64)[l8];
        const uint4 d = reinterpret_cast<const uint4*>(dO + r * 64)[l8];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
          v += __uint_as_float(aw[i] << 16) * __uint_as_float(dw[i] << 16) +
               __uint_as_float(aw[i] & 0xffff0000u) * __uint_as_float(dw[i] & 0xffff0000u);
      }
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      if (l8 == 0 && r < total) {
        const long long hh = r % H;
        const long long bs = r / H;
        const long long s = bs % S, bb = bs / S;
        delta[(bb * H + hh) * S + s] = v;
      }
    }
  }
}

// ----------------------------------------------------------------- backward
// One kernel for dK, dV and dQ. One CTA per 128-row K/V tile (resident in shared memory), looping
// over the Q tiles that attend to it. Per step, with everything transposed so that each operand the
// CTA writes to shared memory is usable as stored:
//     S^T  = K Q_i^T            dP^T = V dO_i^T                          (TMEM, 128 columns each)
//     P^T  = exp2(S^T * c - LSE_q)      dS^T = P^T o (dP^T - delta_q)     (8 compute warps)
//     dV  += P^T dO_i           dK  += dS^T Q_i                          (TMEM accumulators)
//     dQ_i = (dS^T)^T K         (the dS^T tile read as an MN-major A operand; fresh accumulator)
// dQ_i partial sums of the different K/V tiles are added into an fp32 buffer with vector reductions
// and converted to bf16 afterwards. The scores of step i+1 are issued as soon as the compute warps
// have pulled step i's S^T / dP^T into registers, so the tensor core works during the exponentials.
// Compute warp w handles TMEM lane quarter (w & 3) and the column half ((w - 2) >> 2).
struct BwdSmem {
  static constexpr int K = 0;
  static constexpr int V = K + TILE_BYTES;
  static constexpr int QSTAGES = 3;
  static constexpr int Q0 = V + TILE_BYTES;                  // stage s: Q at Q0 + s*2*TILE, dO right after
  static constexpr int PT = Q0 + QSTAGES * 2 * TILE_BYTES;   // P^T  [128 kv x 128 q]
  static constexpr int DST = PT + 2 * TILE_BYTES;            // dS^T [128 kv x 128 q]
  static constexpr int DQS = DST + 2 * TILE_BYTES;           // per compute warp: [32 rows x 32 fp32] dQ staging tile
  static constexpr int STATS = DQS + 8 * 4096;               // [2 slots][2][128] fp32: LSE, delta (slot = step parity)
  static constexpr int BARS = STATS + 2 * 2 * 128 * 4;
  static constexpr int TOTAL = BARS + 256;
  static_assert(TOTAL <= 232448, "exceeds the 227 KB of dynamic shared memory a CTA may use");
};

__global__ void __launch_bounds__(320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmDQ, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_ARG);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BwdSmem::BARS);
  uint64_t* kv_full = bars;
  constexpr int QS = BwdSmem::QSTAGES;
  uint64_t* q_full = bars + 1;    // [QS]  TMA bytes of Q_i and dO_i
  uint64_t* q_empty = bars + 4;   // [QS]
  uint64_t* s_full = bars + 7;    // S^T and dP^T ready
  uint64_t* s_free = bars + 8;    // ... and pulled into registers (8 warps)
  uint64_t* p_ready = bars + 9;   // P^T and dS^T published
  uint64_t* acc_done = bars + 10; // dV / dK / dQ products of the step finished
  uint64_t* dq_free = bars + 11;  // dQ accumulator drained (8 warps)
  uint64_t* st_full = bars + 12;  // [2]  LSE / delta of the step staged by the 256 compute threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* stats = reinterpret_cast<float*>(smem + BwdSmem::STATS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // slowest grid dimension = K/V tile: tile 0 (attended by every Q tile under a causal mask) goes out first
  const int kt = blockIdx.z, h = blockIdx.x, b = blockIdx.y;
  const int kv0 = kt * 128;
  const int n_q_all = (p.S + 127) / 128;
  const int qt_begin = p.causal ? kt : 0;
  const int n_steps = n_q_all - qt_begin;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < QS; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 8);
    mbar_init(p_ready, 256);
    mbar_init(acc_done, 1);
    mbar_init(dq_free, 8);
    mbar_init(&st_full[0], 256);
    mbar_init(&st_full[1], 256);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_ST = tmem_base, tm_DPT = tmem_base + 128, tm_dV = tmem_base + 256, tm_dK = tmem_base + 320,
                 tm_dQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_4d(smem + BwdSmem::K, &tmK, kv_full, 0, h, kv0, b);
      tma_load_4d(smem + BwdSmem::V, &tmV, kv_full, 0, h, kv0, b);
      for (int it = 0; it < n_steps; ++it) {
        const int s = it % QS;
        if (!wait_or_abort(&q_empty[s], ((it / QS) & 1) ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
          break;
        }
        mbar_expect_tx(&q_full[s], 2 * TILE_BYTES);
        uint8_t* qdst = smem + BwdSmem::Q0 + s * 2 * TILE_BYTES;
        const int qrow0 = (qt_begin + it) * 128;
        tma_load_4d(qdst, &tmQ, &q_full[s], 0, h, qrow0, b);
        tma_load_4d(qdst + TILE_BYTES, &tmdO, &q_full[s], 0, h, qrow0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_g = make_idesc_bf16(128, 64, 0, 1);
      constexpr uint32_t idesc_q = make_idesc_bf16(128, 64, 1, 1);
      const uint32_t k_addr = smem_u32(smem + BwdSmem::K), v_addr = smem_u32(smem + BwdSmem::V);
      const uint32_t pt_addr = smem_u32(smem + BwdSmem::PT), dst_addr = smem_u32(smem + BwdSmem::DST);
      // 32 MMAs per step from this one thread: descriptors are built once and moved by adds (address field in
      // 16-byte units)
      constexpr uint32_t T16 = TILE_BYTES / 16;
      const uint64_t k_km = make_smem_desc(k_addr, 16, 1024), k_mn = make_smem_desc(k_addr, 8192, 1024);
      const uint64_t v_km = make_smem_desc(v_addr, 16, 1024);
      const uint64_t pt_km = make_smem_desc(pt_addr, 16, 1024), dst_km = make_smem_desc(dst_addr, 16, 1024);
      const uint64_t dst_mn = make_smem_desc(dst_addr, TILE_BYTES, 1024);
      const uint64_t q0_km = make_smem_desc(smem_u32(smem + BwdSmem::Q0), 16, 1024);    // stage s: + s * 2 * T16; dO: + T16
      const uint64_t q0_mn = make_smem_desc(smem_u32(smem + BwdSmem::Q0), 8192, 1024);
      auto issue_scores = [&](int it) {
        const uint64_t qd = q0_km + (it % QS) * 2 * T16, dod = qd + T16;
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_ss(tm_ST, k_km + k * 2, qd + k * 2, idesc_s, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_ss(tm_DPT, v_km + k * 2, dod + k * 2, idesc_s, k > 0);
        tc_commit(s_full);
      };
      bool ok = n_steps > 0 && wait_or_abort(kv_full, 0, abort_flag) && wait_or_abort(&q_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int it = 0; ok && it < n_steps; ++it) {
        const int s = it % QS;
        if (it + 1 < n_steps) {
          ok = wait_or_abort(&q_full[(it + 1) % QS], ((it + 1) / QS) & 1, abort_flag) &&
               wait_or_abort(s_free, it & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          TRACE(1, it * 8 + 0);
          issue_scores(it + 1);
        }
        TRACE(1, it * 8 + 1);
        ok = wait_or_abort(p_ready, it & 1, abort_flag) && (it == 0 || wait_or_abort(dq_free, (it - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        TRACE(1, it * 8 + 2);
        const uint64_t q_mn = q0_mn + s * 2 * T16, do_mn = q_mn + T16;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_ss(tm_dV, pt_km + (k >> 2) * T16 + (k & 3) * 2, do_mn + k * 128, idesc_g, (it > 0 || k > 0));
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_ss(tm_dK, dst_km + (k >> 2) * T16 + (k & 3) * 2, q_mn + k * 128, idesc_g, (it > 0 || k > 0));
        tc_commit(&q_empty[s]);
        // dQ_i[q, d] = sum_kv dS^T[kv, q] K[kv, d]: both operands MN-major, 16 kv rows per instruction
#pragma unroll
        for (int k = 0; k < 8; ++k) tc_mma_ss(tm_dQ, dst_mn + k * 128, k_mn + k * 128, idesc_q, k > 0);
        tc_commit(acc_done);
        TRACE(1, it * 8 + 3);
      }
      if (!ok && n_steps > 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;  // TMEM lane: kv row for S^T/dP^T/dV/dK, q row for dQ
    const int kv_idx = kv0 + row;
    const int tid = threadIdx.x - 64;     // 0..255
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const long long bh = (long long)b * p.H + h;
    bool ok = true;

    // Add this warp's [32 q rows x 32 columns] of the finished dQ accumulator of Q tile `qt` into the fp32
    // buffer: registers -> swizzled staging tile of the warp -> one TMA reduce (rows past S are clipped).
    uint8_t* dq_stage = smem + BwdSmem::DQS + (warp - 2) * 4096;
    auto drain_stage = [&]() {  // TMEM -> registers -> staging tile (no fence yet)
      if (lane == 0) bulk_wait_group_read0();  // the warp's previous reduce has consumed the staging tile
      __syncwarp();
      uint32_t r[32];
      tmem_ld_32x32(tm_dQ + lane_off + half * 32, r);
      tmem_ld_wait();
      tc_fence_before();
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<float4*>(dq_stage + sw128_offset(lane, c)) =
            make_float4(__uint_as_float(r[c * 4]) * p.scale, __uint_as_float(r[c * 4 + 1]) * p.scale,
                        __uint_as_float(r[c * 4 + 2]) * p.scale, __uint_as_float(r[c * 4 + 3]) * p.scale);
    };
    auto drain_issue = [&](int qt) {  // after every lane's fence.proxy.async
      __syncwarp();
      if (lane == 0) {
        tma_reduce_add_4d(&tmDQ, dq_stage, half * 32, h, qt * 128 + quarter * 32, b);
        bulk_commit_group();
      }
    };

    // LSE (threads 0-127) / delta (128-255) of a Q tile, fetched one step ahead
    auto load_stat = [&](int it) -> float {
      const int qi = (qt_begin + it) * 128 + (tid & 127);
      if (tid < 128) return qi < p.S ? p.LSE[bh * p.S + qi] : INFINITY;
      return qi < p.S ? p.delta[bh * p.S + qi] : 0.f;
    };
    float stat_next = n_steps > 0 ? load_stat(0) : 0.f;

    for (int it = 0; it < n_steps; ++it) {
      const int qrow0 = (qt_begin + it) * 128;
      if (warp == 2 && lane == 0) TRACE(0, it * 8 + 0);
      stats[(it & 1) * 256 + tid] = stat_next;
      mbar_arrive(&st_full[it & 1]);
      if (it + 1 < n_steps) stat_next = load_stat(it + 1);
      if (!wait_or_abort(&st_full[it & 1], (it >> 1) & 1, abort_flag) || !wait_or_abort(s_full, it & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (warp == 2 && lane == 0) TRACE(0, it * 8 + 1);
      uint32_t sr[64], dr[64];
      tmem_ld2_32x64_wait(tm_ST + lane_off + half * 64, tm_DPT + lane_off + half * 64, sr, dr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      if (warp == 2 && lane == 0) TRACE(0, it * 8 + 2);
      const float4* lse4 = reinterpret_cast<const float4*>(stats + (it & 1) * 256 + half * 64);
      const float4* dlt4 = reinterpret_cast<const float4*>(stats + (it & 1) * 256 + 128 + half * 64);
      const bool need_mask = (p.causal && qt_begin + it == kt) || (kv0 + 128 > p.S);
      // phase 1: exponent arguments (in place), phase 2: 64 independent exponentials, phase 3: dS and packing.
      // Keeping the phases apart gives the scheduler long runs of independent instructions per pipe.
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const float4 l4 = lse4[g];
        sr[g * 4 + 0] = __float_as_uint(fmaf(__uint_as_float(sr[g * 4 + 0]), p.scale_log2, -l4.x));
        sr[g * 4 + 1] = __float_as_uint(fmaf(__uint_as_float(sr[g * 4 + 1]), p.scale_log2, -l4.y));
        sr[g * 4 + 2] = __float_as_uint(fmaf(__uint_as_float(sr[g * 4 + 2]), p.scale_log2, -l4.z));
        sr[g * 4 + 3] = __float_as_uint(fmaf(__uint_as_float(sr[g * 4 + 3]), p.scale_log2, -l4.w));
      }
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int qi = qrow0 + half * 64 + c;
          if ((p.causal && qi < kv_idx) || kv_idx >= p.S) sr[c] = 0xff800000u;  // exp2(-inf) = 0
        }
      }
#pragma unroll
      for (int c = 0; c < 64; ++c) sr[c] = __float_as_uint(exp2f(__uint_as_float(sr[c])));
      uint32_t pp[32], dd[32];
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        const float4 d4 = dlt4[g];
        const float e0 = __uint_as_float(sr[g * 4]), e1 = __uint_as_float(sr[g * 4 + 1]), e2 = __uint_as_float(sr[g * 4 + 2]),
                    e3 = __uint_as_float(sr[g * 4 + 3]);
        __nv_bfloat162 a0 = __floats2bfloat162_rn(e0, e1), a1 = __floats2bfloat162_rn(e2, e3);
        __nv_bfloat162 b0 = __floats2bfloat162_rn(e0 * (__uint_as_float(dr[g * 4]) - d4.x), e1 * (__uint_as_float(dr[g * 4 + 1]) - d4.y));
        __nv_bfloat162 b1 = __floats2bfloat162_rn(e2 * (__uint_as_float(dr[g * 4 + 2]) - d4.z), e3 * (__uint_as_float(dr[g * 4 + 3]) - d4.w));
        pp[g * 2] = *reinterpret_cast<uint32_t*>(&a0);
        pp[g * 2 + 1] = *reinterpret_cast<uint32_t*>(&a1);
        dd[g * 2] = *reinterpret_cast<uint32_t*>(&b0);
        dd[g * 2 + 1] = *reinterpret_cast<uint32_t*>(&b1);
      }
      if (warp == 2 && lane == 0) TRACE(0, it * 8 + 3);
      if (it > 0) {
        // the previous step's products are done: its dQ can be drained and P^T / dS^T overwritten
        if (!wait_or_abort(acc_done, (it - 1) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (warp == 2 && lane == 0) TRACE(0, it * 8 + 4);
        drain_stage();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_free);
      }
      if (warp == 2 && lane == 0) TRACE(0, it * 8 + 5);
      uint8_t* pt = smem + BwdSmem::PT + half * TILE_BYTES;
      uint8_t* dt = smem + BwdSmem::DST + half * TILE_BYTES;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t off = sw128_offset(row, c);
        *reinterpret_cast<uint4*>(pt + off) = make_uint4(pp[c * 4], pp[c * 4 + 1], pp[c * 4 + 2], pp[c * 4 + 3]);
        *reinterpret_cast<uint4*>(dt + off) = make_uint4(dd[c * 4], dd[c * 4 + 1], dd[c * 4 + 2], dd[c * 4 + 3]);
      }
      fence_proxy_async_smem();  // covers the dQ staging tile as well as P^T / dS^T
      tc_fence_before();
      mbar_arrive(p_ready);
      if (it > 0) drain_issue(qt_begin + it - 1);
      if (warp == 2 && lane == 0) TRACE(0, it * 8 + 6);
    }
    if (!ok && lane == 0) {
      raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
      bulk_wait_group0();
    }
    if (ok && n_steps > 0) {
      if (wait_or_abort(acc_done, (n_steps - 1) & 1, abort_flag)) {
        tc_fence_after();
        drain_stage();
        fence_proxy_async_smem();
        drain_issue(qt_begin + n_steps - 1);
        // tcgen05.ld is warp-collective: every lane loads, only in-range rows store.
        const bool live = kv_idx < p.S;
        const long long roff = (((long long)b * p.S + (live ? kv_idx : 0)) * 3 * p.H + h) * 64 + half * 32;
        uint32_t r[32];
        tmem_ld_32x32(tm_dV + lane_off + half * 32, r);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t pk[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * k]), __uint_as_float(r[g * 8 + 2 * k + 1]));
              pk[k] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(p.dV + roff + g * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
        tmem_ld_32x32(tm_dK + lane_off + half * 32, r);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t pk[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * k]) * p.scale,
                                                         __uint_as_float(r[g * 8 + 2 * k + 1]) * p.scale);
              pk[k] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(p.dK + roff + g * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      } else if (lane == 0) {
        raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
      }
      if (lane == 0) bulk_wait_group0();  // the staging tile must outlive the last reduce
    } else if (ok && kv_idx < p.S) {
      // no Q tile attends to this K/V tile: gradients are zero
      const long long roff = (((long long)b * p.S + kv_idx) * 3 * p.H + h) * 64 + half * 32;
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4*>(p.dV + roff + c * 8) = z;
        *reinterpret_cast<uint4*>(p.dK + roff + c * 8) = z;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// dQ: fp32 accumulator [B*S, E] -> bf16 rows of pitch 3E inside dqkv. Eight elements per thread.
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, bf16* __restrict__ dq, long long rows, int E) {
  const long long per_row = E / 8;
  const long long total = rows * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row, c = (i - r * per_row) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + r * E + c);
    const float4 b2 = *reinterpret_cast<const float4*>(acc + r * E + c + 4);
    __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(b2.x, b2.y), h3 = __floats2bfloat162_rn(b2.z, b2.w);
    *reinterpret_cast<uint4*>(dq + r * 3 * E + c) =
        make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1), *reinterpret_cast<uint32_t*>(&h2),
                   *reinterpret_cast<uint32_t*>(&h3));
  }
}

// --------------------------------------------------------------------- host
// 4-D map over x[B, S, pitch...] selecting head h: dims {64, H, S, B}.
static int make_head_map(CUtensorMap* m, const void* base, int B, int S, int H, long long row_pitch_elems) {
  uint64_t dims[4] = {64, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t str[3] = {64 * 2, (uint64_t)row_pitch_elems * 2, (uint64_t)row_pitch_elems * 2 * (uint64_t)S};
  uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap_bf16(m, base, 4, dims, str, box, nullptr);
}

template <typename K>
static int set_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // namespace tnnb

using namespace tnnb;

extern "C" {

// qkv: [B,S,3,H,64] bf16; out: [B,S,H,64] bf16; lse: [B,H,S] fp32 (scaled log2 units).
int tnnb_attn_fwd(const void* qkv, void* out, void* lse, int B, int S, int H, int D, int causal, float scale,
                  int* status, void* stream) {
  if (D != 64) return -7;
  if ((uintptr_t)qkv & 15 || (uintptr_t)out & 15) return -4;
  const long long E = (long long)H * 64;
  const bf16* base = (const bf16*)qkv;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_head_map(&tq, base, B, S, H, 3 * E))) return rc;
  if ((rc = make_head_map(&tk, base + E, B, S, H, 3 * E))) return rc;
  if ((rc = make_head_map(&tv, base + 2 * E, B, S, H, 3 * E))) return rc;
  AttnParams p{};
  p.B = B; p.S = S; p.H = H; p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = (bf16*)out;
  p.LSE = (float*)lse;
  p.status = status;
  static bool once = false;
  if (!once) {
    if ((rc = set_smem(attn_fwd_kernel, FwdSmem::TOTAL))) return rc;
    once = true;
  }
  if (B > 65535 || (S + 255) / 256 > 65535) return -3;  // grid y / z limits
  dim3 grid(H, B, (S + 255) / 256);
  attn_fwd_kernel<<<grid, 320, FwdSmem::TOTAL, (cudaStream_t)stream>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// dqkv: [B,S,3,H,64] bf16 (fully overwritten); delta: [B,H,S] fp32 and dq_acc: [B,S,H,64] fp32 are
// scratch owned by the caller (dq_acc is zeroed here).
int tnnb_attn_bwd(const void* qkv, const void* out, const void* dout, const void* lse, void* delta, void* dq_acc,
                  void* dqkv, int B, int S, int H, int D, int causal, float scale, int* status, void* stream) {
  if (D != 64) return -7;
  if (((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)dout | (uintptr_t)dqkv | (uintptr_t)dq_acc) & 15) return -4;
  cudaStream_t st = (cudaStream_t)stream;
  const long long E = (long long)H * 64;
  const bf16* base = (const bf16*)qkv;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_head_map(&tq, base, B, S, H, 3 * E))) return rc;
  if ((rc = make_head_map(&tk, base + E, B, S, H, 3 * E))) return rc;
  if ((rc = make_head_map(&tv, base + 2 * E, B, S, H, 3 * E))) return rc;
  if ((rc = make_head_map(&tdo, dout, B, S, H, E))) return rc;
  CUtensorMap tdq;
  {
    uint64_t dims[4] = {64, (uint64_t)H, (uint64_t)S, (uint64_t)B};
    uint64_t str[3] = {64 * 4, (uint64_t)E * 4, (uint64_t)E * 4 * (uint64_t)S};
    uint32_t box[4] = {32, 1, 32, 1};
    if ((rc = encode_tmap_f32(&tdq, dq_acc, 4, dims, str, box))) return rc;
  }
  AttnParams p{};
  p.B = B; p.S = S; p.H = H; p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.LSE = (float*)lse;
  p.delta = (const float*)delta;
  p.dq_acc = (float*)dq_acc;
  p.dQ = (bf16*)dqkv;
  p.dK = (bf16*)dqkv + E;
  p.dV = (bf16*)dqkv + 2 * E;
  p.status = status;
  static bool once = false;
  if (!once) {
    if ((rc = set_smem(attn_bwd_kernel, BwdSmem::TOTAL))) return rc;
    once = true;
  }
  const long long rows = (long long)B * S * H;
  cudaMemsetAsync(dq_acc, 0, sizeof(float) * (size_t)B * S * E, st);
  const long long dw = (rows + 3) / 4;  // warps of work for the delta kernel, eight per block
  int g = (int)((dw + 7) / 8 > 148 * 8 ? 148 * 8 : (dw + 7) / 8);
  attn_delta_kernel<<<g, 256, 0, st>>>((const bf16*)out, (const bf16*)dout, (float*)delta, B, S, H);
  if (B > 65535 || (S + 127) / 128 > 65535) return -3;  // grid y / z limits
  dim3 grid(H, B, (S + 127) / 128);
  attn_bwd_kernel<<<grid, 320, BwdSmem::TOTAL, st>>>(tq, tk, tv, tdo, tdq, p);
  attn_dq_convert_kernel<<<148 * 4, 256, 0, st>>>((const float*)dq_acc, (bf16*)dqkv, (long long)B * S, (int)E);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

#ifdef TNNB_TRACE
int tnnb_attn_trace_dump(void* host_out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(host_out, g_trace, sizeof(g_trace));
}
#endif

}  // extern "C"
