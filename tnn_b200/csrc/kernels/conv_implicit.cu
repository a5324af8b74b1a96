// NHWC convolution as an implicit GEMM on tcgen05: no patch matrix is ever written.
//
// The 128 rows of an output tile are a small spatial box of output pixels, TN images x TH rows x TW columns
// (TN*TH*TW = 128). For every filter tap (kh, kw) and block of 64 input channels, TMA fetches the matching box
// of the input - the same box shifted by (kh - pad, kw - pad), with the convolution stride as the tensor
// map's element stride - straight into 128-byte-swizzled shared memory, where it is a K-major A operand like
// any GEMM tile; pixels outside the image arrive as zeros, which is exactly the zero padding. The weights
// [O, KH*KW*C] are the K-major B operand. Requires C % 64 == 0 (every ResNet / WRN layer but the 3-channel
// stem, which keeps the gather kernel).
//
//   forward   y[n,oh,ow,o] = bias[o] + sum_{kh,kw,c} x[n, oh*s+kh-p, ow*s+kw-p, c] * w[o,kh,kw,c]
//   dgrad     (stride 1) the same kernel on dy with the filter rotated by 180 degrees and its
//             channel axes swapped (a small host-side weight transform), pad' = k - 1 - pad
//   wgrad     dw[o,kh,kw,c] += sum_pixels dy[pix, o] * x[pix shifted by the tap, c]: per tap a GEMM whose
//             reduction index is the pixel; both operands are MN-major boxes of 64 pixels; split over
//             pixel ranges with fp32 vector reductions into dw
//
// Reference semantics: src/nn/engines/cpu_engine.cpp:617-734 (the reference itself calls cuDNN conv graphs,
// src/nn/engines/cudnn_engine.cu:328-528). Kernel structure as in gemm_tcgen05.cu: TMA producer warp, MMA
// warp with two TMEM accumulators, eight epilogue warps, every wait bounded.
#include "gemm_tcgen05.h"
#include "ptx.cuh"

namespace tnnb {

typedef __nv_bfloat16 bf16;

struct ConvParams {
  int N, OH, OW, O;             // output geometry (rows of the implicit GEMM are output pixels)
  int KH, KW, SH, SW, PH, PW;   // filter taps, stride, padding
  int cblocks;                  // C / 64
  int TN, TH, TW, lgTH, lgTW;   // pixel box of a tile (TH, TW powers of two)
  int tiles_n, tiles_h, tiles_w;
  int num_m_tiles, num_n_blocks, num_k_blocks;
  bf16* Y;                      // [N, YH, YW, O]: output position (oh, ow) is pixel (oh * ys + yo, ow * xs + xo)
  int YH, YW, ys, xs, yo, xo;   // plain convolution: YH = OH, YW = OW, ys = xs = 1, yo = xo = 0
  const bf16* bias;
  int relu;
  int* status;
};

template <int BN>
struct ConvCfg {
  static constexpr int A_BYTES = 128 * 64 * 2;
  static constexpr int B_BYTES = BN * 64 * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BARS = STAGES * STAGE_BYTES;
  static constexpr int STAGING = BARS + 256;
  static constexpr int SMEM_BYTES = STAGING + 8 * 4096 + 1024;
};

__device__ __forceinline__ uint32_t vstage_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// row r (0..127) of tile (ni, hi, wi) -> linear output pixel, or -1 outside the tensor
__device__ __forceinline__ long long conv_out_row(const ConvParams& p, int ni, int hi, int wi, int r) {
  const int tw = r & (p.TW - 1);
  const int th = (r >> p.lgTW) & (p.TH - 1);
  const int tn = r >> (p.lgTW + p.lgTH);
  const int n = ni * p.TN + tn, oh = hi * p.TH + th, ow = wi * p.TW + tw;
  if (n >= p.N || oh >= p.OH || ow >= p.OW) return -1;
  return ((long long)n * p.YH + (oh * p.ys + p.yo)) * p.YW + (ow * p.xs + p.xo);
}

template <int BN>
__global__ void __launch_bounds__(320, 1)
conv_fwd_implicit_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const ConvParams p) {
  using Cfg = ConvCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BARS);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.num_m_tiles * p.num_n_blocks;
  const int per_img = p.tiles_h * p.tiles_w;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        const int nb = t / p.num_m_tiles, mt = t - nb * p.num_m_tiles;
        const int ni = mt / per_img, rem = mt - ni * per_img;
        const int hi = rem / p.tiles_w, wi = rem - hi * p.tiles_w;
        const int n0 = ni * p.TN, ih0 = hi * p.TH * p.SH - p.PH, iw0 = wi * p.TW * p.SW - p.PW;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          const int tap = kb / p.cblocks, c0 = (kb - tap * p.cblocks) * 64;
          const int kh = tap / p.KW, kw = tap - kh * p.KW;
          if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* a_dst = smem + stage * Cfg::STAGE_BYTES;
          tma_load_4d(a_dst, &tmX, &full[stage], c0, iw0 + kw, ih0 + kh, n0);  // the channel coordinate is 64-aligned
          tma_load_2d(a_dst + Cfg::A_BYTES, &tmW, &full[stage], kb * 64, nb * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN, 0, 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        if (!wait_or_abort(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!wait_or_abort(&full[stage], phase, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          // the address field of a descriptor counts 16-byte units: a k-step is an add
          const uint64_t a_desc0 = make_smem_desc(a_addr, 16, 1024), b_desc0 = make_smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_ss(d_tmem, a_desc0 + k * 2, b_desc0 + k * 2, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
    const int q = warp & 3, half = (warp - 2) >> 2;
    uint8_t* stage_tile = smem + Cfg::STAGING + (warp - 2) * 4096;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      const int nb = t / p.num_m_tiles, mt = t - nb * p.num_m_tiles;
      const int ni = mt / per_img, rem = mt - ni * per_img;
      const int hi = rem / p.tiles_w, wi = rem - hi * p.tiles_w;
      if (!wait_or_abort(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16) + half * (BN / 2);
      const int col_base = nb * BN + half * (BN / 2);
      // output pixels of the eight rows this lane stores in the coalesced phase (rows i*4 + lane/8 of the warp)
      long long orow[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) orow[i] = conv_out_row(p, ni, hi, wi, q * 32 + i * 4 + (lane >> 3));
#pragma unroll 1
      for (int c = 0; c < BN / 64; c += 2) {
        const int col0 = col_base + c * 32;
        if (col0 >= p.O) continue;   // O % 64 == 0: a pair of chunks is entirely inside or outside
        uint32_t rr[2][32];  // both chunks requested before the one wait
        tmem_ld_32x32(t_addr + c * 32, rr[0]);
        tmem_ld_32x32(t_addr + (c + 1) * 32, rr[1]);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int cc = col0 + h * 32;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[h][j]);
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(p.bias[cc + j]);  // same address in every lane: a broadcast
          }
          if (p.relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * k + 2 * j], v[8 * k + 2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(stage_tile + vstage_off(lane, h * 4 + k)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3), c16 = lane & 7;
          if (orow[i] >= 0)
            *reinterpret_cast<uint4*>(p.Y + orow[i] * p.O + col0 + c16 * 8) = *reinterpret_cast<const uint4*>(stage_tile + vstage_off(rr, c16));
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
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

// ----------------------------------------------------- forward, 64 channels: input tile with halo loaded once
// For C = 64 the k-blocks of the kernel above are the filter taps, and each of them fetches the same 128 pixels
// again, shifted by one: nine 16 KB loads per tile, which makes 64-channel 3 x 3 layers L2-bandwidth bound. Here a
// tile is 16 x 8 output pixels of one image and ONE TMA box brings its input window with the halo,
// (16 + KH - 1) rows of 16 pixels (the row pitch is 16 so that every 8-pixel row of the tile starts a whole
// number of 1024-byte swizzle repeats after the one above it). The A operand of tap (kh, kw) is that same
// shared-memory tile read through a descriptor whose start is moved by kh rows and kw pixels and whose 8-row groups
// are one pitch (2048 bytes) apart. The 64-row filter matrix of all taps stays in shared memory for the CTA's
// lifetime. Stride 1, KH <= 3, KW <= 3, C == 64, O == 64.
struct HaloCfg {
  static constexpr int PITCH = 16, TH = 16, TW = 8, MAXROWS = TH + 2;
  static constexpr int HALO_BYTES = MAXROWS * PITCH * 128;  // 36 KB
  static constexpr int STAGES = 3;
  static constexpr int MAXTAPS = 9;
  static constexpr int W_BYTES = MAXTAPS * 64 * 128;         // 72 KB
  static constexpr int HALO0 = W_BYTES;
  static constexpr int BARS = HALO0 + STAGES * HALO_BYTES;
  static constexpr int STAGING = BARS + 256;
  static constexpr int SMEM_BYTES = STAGING + 4 * 4096 + 1024;
};
static_assert(HaloCfg::SMEM_BYTES <= 227 * 1024, "halo kernel shared memory");

__global__ void __launch_bounds__(192, 1)
conv_fwd_halo_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const ConvParams p) {
  // tmX: box {64, 16, TH + KH - 1, 1}
  using Cfg = HaloCfg;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BARS);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* wfull = tempty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(wfull + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.KH * p.KW;
  const uint32_t halo_bytes = (uint32_t)(Cfg::TH + p.KH - 1) * Cfg::PITCH * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    mbar_init(wfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.num_m_tiles;
  const int per_img = p.tiles_h * p.tiles_w;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(wfull, (uint32_t)taps * 64u * 128u);
      for (int t = 0; t < taps; ++t) tma_load_2d(smem + t * 8192, &tmW, wfull, t * 64, 0);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int ni = t / per_img, rem = t - ni * per_img;
        const int hi = rem / p.tiles_w, wi = rem - hi * p.tiles_w;
        if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
          break;
        }
        mbar_expect_tx(&full[stage], halo_bytes);
        tma_load_4d(smem + Cfg::HALO0 + stage * Cfg::HALO_BYTES, &tmX, &full[stage], 0, wi * Cfg::TW - p.PW, hi * Cfg::TH - p.PH, ni);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 64, 0, 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = wait_or_abort(wfull, 0, abort_flag);
      if (!ok) raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
      // One thread issues 36 short MMAs (128 x 64 x 16) per tile: what it spends per instruction on building
      // descriptors bounds the kernel, so everything that does not depend on the tile is worked out here. A
      // descriptor's low bits are the shared-memory address in 16-byte units, so windows and k-steps are plain adds.
      const uint64_t b_desc0 = make_smem_desc(smem_u32(smem), 16, 1024);
      uint32_t tap_off[Cfg::MAXTAPS];  // start of tap (kh, kw) inside the halo tile, in 16-byte units
#pragma unroll
      for (int tap = 0; tap < Cfg::MAXTAPS; ++tap) tap_off[tap] = (uint32_t)((tap / p.KW) * Cfg::PITCH + (tap % p.KW)) * 8u;
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        if (!wait_or_abort(&tempty[acc], acc_phase ^ 1, abort_flag) || !wait_or_abort(&full[stage], phase, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 64;
        // The window of tap (kh, kw) starts kh rows and kw pixels into the tile. Its start is no longer a multiple
        // of 1024 bytes, which is fine: the tensor core applies the 128-byte swizzle to the absolute shared-memory
        // address of every row, exactly as TMA did when it wrote the tile (the descriptor's base offset field stays
        // 0 - setting it to the start row gave wrong sums on B200).
        const uint64_t a_desc0 = make_smem_desc(smem_u32(smem + Cfg::HALO0 + stage * Cfg::HALO_BYTES), 16, Cfg::PITCH * 128);
#pragma unroll
        for (int tap = 0; tap < Cfg::MAXTAPS; ++tap) {
          if (tap < taps) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_ss(d_tmem, a_desc0 + tap_off[tap] + k * 2, b_desc0 + tap * 512 + k * 2, idesc, (tap > 0 || k > 0) ? 1u : 0u);
          }
        }
        tc_commit(&empty[stage]);
        tc_commit(&tfull[acc]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;  // warps 2..5: TMEM lane quarter
    uint8_t* stage_tile = smem + Cfg::STAGING + (warp - 2) * 4096;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      const int ni = t / per_img, rem = t - ni * per_img;
      const int hi = rem / p.tiles_w, wi = rem - hi * p.tiles_w;
      if (!wait_or_abort(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * 64 + (static_cast<uint32_t>(q * 32) << 16);
      long long orow[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) orow[i] = conv_out_row(p, ni, hi, wi, q * 32 + i * 4 + (lane >> 3));
      uint32_t rr[2][32];  // both chunks requested before the one wait
      tmem_ld_32x32(t_addr, rr[0]);
      tmem_ld_32x32(t_addr + 32, rr[1]);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[h][j]);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += __bfloat162float(p.bias[h * 32 + j]);
        }
        if (p.relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * k + 2 * j], v[8 * k + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h2);
          }
          *reinterpret_cast<uint4*>(stage_tile + vstage_off(lane, h * 4 + k)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);  // the accumulator is in registers / shared memory now
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + (lane >> 3), c16 = lane & 7;
        if (orow[i] >= 0)
          *reinterpret_cast<uint4*>(p.Y + orow[i] * p.O + c16 * 8) = *reinterpret_cast<const uint4*>(stage_tile + vstage_off(rr, c16));
      }
      __syncwarp();
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

// ------------------------------------------------------------------------------------------ weight gradient
struct WgradParams {
  int N, OH, OW, O, C;
  int KH, KW, SH, SW, PH, PW;
  int TN, TH, TW;               // pixel box of one reduction block (TN*TH*TW = 64)
  int tiles_n, tiles_h, tiles_w;
  int num_o_blocks, num_c_blocks;   // 128-row blocks of O, BN-column blocks of C
  int pix_blocks, split, blocks_per_split;
  float* dW;                    // [O, KH*KW*C] fp32, accumulated into
  int* status;
};

template <int BN>
struct WgradCfg {
  static constexpr int A_BYTES = 2 * 64 * 64 * 2;         // two [64 pixels x 64 o] boxes
  static constexpr int B_BYTES = (BN / 64) * 64 * 64 * 2; // BN/64 boxes of [64 pixels x 64 c]
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BARS = STAGES * STAGE_BYTES;
  static constexpr int STAGING = BARS + 256;
  static constexpr int SMEM_BYTES = STAGING + 8 * 4096 + 1024;
};

template <int BN>
__global__ void __launch_bounds__(320, 1)
conv_wgrad_implicit_kernel(const __grid_constant__ CUtensorMap tmDY, const __grid_constant__ CUtensorMap tmX, const WgradParams p) {
  using Cfg = WgradCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BARS);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // work item = (split, tap, c block, o block)
  const int taps = p.KH * p.KW;
  const int total = p.split * taps * p.num_c_blocks * p.num_o_blocks;
  const int per_img = p.tiles_h * p.tiles_w;
  auto decode = [&](int w, int& ob, int& cb, int& tap, int& sp) {
    ob = w % p.num_o_blocks; w /= p.num_o_blocks;
    cb = w % p.num_c_blocks; w /= p.num_c_blocks;
    tap = w % taps;
    sp = w / taps;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total; w += gridDim.x) {
        int ob, cb, tap, sp;
        decode(w, ob, cb, tap, sp);
        const int kh = tap / p.KW, kw = tap - kh * p.KW;
        const int pb0 = sp * p.blocks_per_split, pb1 = min(pb0 + p.blocks_per_split, p.pix_blocks);
        for (int pb = pb0; pb < pb1; ++pb) {
          const int ni = pb / per_img, rem = pb - ni * per_img;
          const int hi = rem / p.tiles_w, wi = rem - hi * p.tiles_w;
          if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* a_dst = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
#pragma unroll
          for (int i = 0; i < 2; ++i)
            tma_load_4d(a_dst + i * 8192, &tmDY, &full[stage], ob * 128 + i * 64, wi * p.TW, hi * p.TH, ni * p.TN);
#pragma unroll
          for (int i = 0; i < BN / 64; ++i)
            tma_load_4d(b_dst + i * 8192, &tmX, &full[stage], cb * BN + i * 64, wi * p.TW * p.SW + kw - p.PW,
                        hi * p.TH * p.SH + kh - p.PH, ni * p.TN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN, 1, 1);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total; w += gridDim.x) {
        int ob, cb, tap, sp;
        decode(w, ob, cb, tap, sp);
        const int pb0 = sp * p.blocks_per_split, pb1 = min(pb0 + p.blocks_per_split, p.pix_blocks);
        if (!wait_or_abort(&tempty[acc], acc_phase ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int pb = pb0; pb < pb1; ++pb) {
          if (!wait_or_abort(&full[stage], phase, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
          const uint64_t a_desc0 = make_smem_desc(a_addr, 8192, 1024), b_desc0 = make_smem_desc(b_addr, 8192, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 16 pixels per instruction; both operands MN-major
            tc_mma_ss(d_tmem, a_desc0 + k * 128, b_desc0 + k * 128, idesc, (pb > pb0 || k > 0) ? 1u : 0u);
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
    const int q = warp & 3, half = (warp - 2) >> 2;
    uint8_t* stage_tile = smem + Cfg::STAGING + (warp - 2) * 4096;
    const long long ldw = (long long)taps * p.C;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x) {
      int ob, cb, tap, sp;
      decode(w, ob, cb, tap, sp);
      if (!wait_or_abort(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16) + half * (BN / 2);
      const int row_base = ob * 128 + q * 32;                 // output channel o
      const int col_base = cb * BN + half * (BN / 2);         // input channel c
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        const int col0 = col_base + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (col0 >= p.C) continue;  // C % 64 == 0: whole chunk outside
#pragma unroll
        for (int k = 0; k < 8; ++k)
          *reinterpret_cast<float4*>(stage_tile + vstage_off(lane, k)) =
              make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]), __uint_as_float(r[4 * k + 2]), __uint_as_float(r[4 * k + 3]));
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3), c4 = lane & 7;
          const float4 v = *reinterpret_cast<const float4*>(stage_tile + vstage_off(rr, c4));
          if (row_base + rr < p.O) {
            float* d = p.dW + (long long)(row_base + rr) * ldw + (long long)tap * p.C + col0 + c4 * 4;
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
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

// ------------------------------------------- weight gradient, 64 channels: one input window for all filter taps
// dW[o, kh, kw, c] = sum over pixels of dy[pixel, o] * x[pixel + (kh, kw) - pad, c]. The general kernel below
// fetches x once per tap and fills half of every 128 x 128 tile with zeros when C = O = 64. Here a CTA walks over
// 16 x 8 pixel tiles; per tile ONE box brings the x window with its halo (as in conv_fwd_halo_kernel: row pitch 16,
// taps addressed by moving the descriptor start) and one box the dy tile, and all taps are accumulated at once:
// the A operand (MN-major, rows = pixels, 64 channels per row) of one MMA covers TWO taps - its second 64-channel
// block is the same window one pixel (or one row) further on, which the leading-dimension offset of the
// descriptor expresses - so nine taps take five 128 x 64 accumulators [(tap, c), o]. They stay in tensor memory
// for all tiles of the CTA and are added to dW once at the end. Stride 1, KH <= 3, KW <= 3, C == O == 64.
struct WgradHaloCfg {
  static constexpr int PITCH = 16, TH = 16, TW = 8;
  static constexpr int X_BYTES = (TH + 2) * PITCH * 128;  // 36 KB
  static constexpr int DY_BYTES = TH * TW * 128;          // 16 KB
  static constexpr int STAGE_BYTES = X_BYTES + DY_BYTES;
  static constexpr int STAGES = 4;
  static constexpr int BARS = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = BARS + 256 + 1024;
};
static_assert(WgradHaloCfg::SMEM_BYTES <= 227 * 1024, "wgrad halo kernel shared memory");

__global__ void __launch_bounds__(192, 1)
conv_wgrad_halo_kernel(const __grid_constant__ CUtensorMap tmDY, const __grid_constant__ CUtensorMap tmX, const WgradParams p) {
  using Cfg = WgradHaloCfg;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BARS);
  uint64_t* empty = full + STAGES;
  uint64_t* done = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.KH * p.KW;
  const int groups = (taps + 1) / 2;
  const uint32_t x_bytes = (uint32_t)(Cfg::TH + p.KH - 1) * Cfg::PITCH * 128u;
  // tap t -> byte shift of its window inside the halo tile; pairs are taken in this order
  auto shift = [&](int t) { return (uint32_t)((t / p.KW) * Cfg::PITCH + (t % p.KW)) * 128u; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmDY);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles = p.pix_blocks;
  const int per_img = p.tiles_h * p.tiles_w;
  const bool any = (int)blockIdx.x < tiles;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int ni = t / per_img, rem = t - ni * per_img;
        const int hi = rem / p.tiles_w, wi = rem - hi * p.tiles_w;
        if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
          break;
        }
        mbar_expect_tx(&full[stage], x_bytes + Cfg::DY_BYTES);
        uint8_t* dst = smem + stage * Cfg::STAGE_BYTES;
        tma_load_4d(dst, &tmX, &full[stage], 0, wi * Cfg::TW - p.PW, hi * Cfg::TH - p.PH, ni);
        tma_load_4d(dst + Cfg::X_BYTES, &tmDY, &full[stage], 0, wi * Cfg::TW, hi * Cfg::TH, ni);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && any) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 64, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true, first = true;
      // per group of two taps: the A descriptor without the tile's base address (window start of the first tap,
      // distance to the second tap's window as leading-dimension offset) - 40 MMAs per tile then cost two adds each
      constexpr int MAXG = 5;
      uint64_t g_desc[MAXG];
#pragma unroll
      for (int g = 0; g < MAXG; ++g) {
        const int t0 = min(2 * g, taps - 1), t1 = min(2 * g + 1, taps - 1);
        const uint32_t lbo = (t1 > t0) ? shift(t1) - shift(t0) : 128u;  // odd tap count: the second half is never read back
        g_desc[g] = make_smem_desc(shift(t0), lbo, Cfg::PITCH * 128);
      }
      for (int t = blockIdx.x; ok && t < tiles; t += gridDim.x) {
        if (!wait_or_abort(&full[stage], phase, abort_flag)) {
          raise_abort(p.status, abort_flag, ST_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t x_addr = smem_u32(smem + stage * Cfg::STAGE_BYTES);
        const uint64_t dy_desc0 = make_smem_desc(x_addr + Cfg::X_BYTES, 8192, 1024);
        const uint32_t x16 = x_addr >> 4;
#pragma unroll
        for (int g = 0; g < MAXG; ++g) {
          if (g < groups) {
#pragma unroll
            for (int k = 0; k < 8; ++k)  // 16 pixels (two tile rows) per instruction
              tc_mma_ss(tmem_base + g * 64, g_desc[g] + x16 + k * (2 * Cfg::PITCH * 128 / 16), dy_desc0 + k * 128, idesc,
                        (first && k == 0) ? 0u : 1u);
          }
        }
        first = false;
        tc_commit(&empty[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) tc_commit(done);
    }
  } else if (any) {
    // warps 2..5: add the accumulators to dW. Lane = row (tap, c) of the group, register j = output channel o;
    // for a fixed o the 32 lanes of a warp hit 32 consecutive floats.
    const int q = warp & 3;
    if (wait_or_abort(done, 0, abort_flag)) {
      tc_fence_after();
      const long long ldw = (long long)taps * 64;
      for (int g = 0; g < groups; ++g) {
        const int row = q * 32 + lane;
        const int tap = 2 * g + (row >> 6), c = row & 63;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + g * 64 + h * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
          tmem_ld_wait();
          if (tap < taps) {
            float* d = p.dW + (long long)tap * 64 + c;
#pragma unroll
            for (int j = 0; j < 32; ++j) atomicAdd(d + (long long)(h * 32 + j) * ldw, __uint_as_float(r[j]));
          }
        }
      }
    } else if (lane == 0) {
      raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------ host
static int ilog2(int v) {
  int l = 0;
  while ((1 << l) < v) ++l;
  return l;
}

// Pixel box (TN, TH, TW) with TN*TH*TW == rows that wastes the fewest rows on this output geometry.
static void pick_box(int rows, int N, int OH, int OW, int& TN, int& TH, int& TW) {
  long long best = -1;
  for (int th = 1; th <= 16; th *= 2)
    for (int tw = 1; tw <= 16; tw *= 2) {
      if (rows % (th * tw)) continue;
      const int tn = rows / (th * tw);
      if (tn > 256) continue;
      const long long padded = (long long)((N + tn - 1) / tn) * tn * ((OH + th - 1) / th) * th * ((OW + tw - 1) / tw) * tw;
      // prefer wide boxes on ties: longer contiguous runs per TMA row
      if (best < 0 || padded < best || (padded == best && tw > TW)) {
        best = padded;
        TN = tn; TH = th; TW = tw;
      }
    }
}

static int map_nhwc(CUtensorMap* m, const void* base, int N, int H, int W, int C, int bc, int bw, int bh, int bn, int sw, int sh) {
  uint64_t dims[4] = {(uint64_t)C, (uint64_t)W, (uint64_t)H, (uint64_t)N};
  uint64_t str[3] = {(uint64_t)C * 2, (uint64_t)W * C * 2, (uint64_t)H * W * C * 2};
  // with an element stride s the box extent is given in input elements: bw * s of them yield bw loaded elements
  uint32_t box[4] = {(uint32_t)bc, (uint32_t)((bw - 1) * sw + 1), (uint32_t)((bh - 1) * sh + 1), (uint32_t)bn};
  uint32_t es[4] = {1, (uint32_t)sw, (uint32_t)sh, 1};
  return encode_tmap_bf16(m, base, 4, dims, str, box, es);
}

template <typename K>
static int set_smem_attr(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // namespace tnnb

using namespace tnnb;

// x [N,H,W,C] bf16, w [O,KH,KW,C] bf16, C % 64 == 0, O % 64 == 0, bias may be null. OH x OW output positions per
// image are computed (position (oh, ow) reads input rows oh * SH - PH + kh, columns ow * SW - PW + kw; outside the
// image reads zero; PH / PW may be negative) and written to pixel (oh * ys + yo, ow * xs + xo) of y [N,YH,YW,O]:
// with ys / xs > 1 one call fills one parity class of a larger image (data gradient of a strided convolution).
static int conv_fwd_implicit_impl(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int C, int O,
                                  int KH, int KW, int SH, int SW, int PH, int PW, int OH, int OW, int YH, int YW, int ys,
                                  int xs, int yo, int xo, int relu, int* status, void* stream) {
  if (C % 64 || O % 64 || C <= 0 || O <= 0) return -3;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return -4;
  if (ys < 1 || xs < 1 || yo < 0 || xo < 0 || OH <= 0 || OW <= 0) return -2;
  if ((long long)(OH - 1) * ys + yo >= YH || (long long)(OW - 1) * xs + xo >= YW) return -2;  // every write inside y
  ConvParams p{};
  p.N = N; p.O = O;
  p.OH = OH;
  p.OW = OW;
  p.YH = YH; p.YW = YW; p.ys = ys; p.xs = xs; p.yo = yo; p.xo = xo;
  p.KH = KH; p.KW = KW; p.SH = SH; p.SW = SW; p.PH = PH; p.PW = PW;
  p.cblocks = C / 64;
  pick_box(128, N, p.OH, p.OW, p.TN, p.TH, p.TW);
  p.lgTH = ilog2(p.TH); p.lgTW = ilog2(p.TW);
  p.tiles_n = (N + p.TN - 1) / p.TN; p.tiles_h = (p.OH + p.TH - 1) / p.TH; p.tiles_w = (p.OW + p.TW - 1) / p.TW;
  p.num_m_tiles = p.tiles_n * p.tiles_h * p.tiles_w;
  const int bn = (O > 128) ? 256 : 128;
  p.num_n_blocks = (O + bn - 1) / bn;
  p.num_k_blocks = KH * KW * p.cblocks;
  p.Y = (bf16*)y; p.bias = (const bf16*)bias; p.relu = relu; p.status = status;
  CUtensorMap tx, tw;
  int rc;
  if ((rc = map_nhwc(&tx, x, N, H, W, C, 64, p.TW, p.TH, p.TN, SW, SH))) return rc;
  {
    uint64_t dims[2] = {(uint64_t)KH * KW * C, (uint64_t)O};
    uint64_t str[1] = {(uint64_t)KH * KW * C * 2};
    uint32_t box[2] = {64, (uint32_t)bn};
    if ((rc = encode_tmap_bf16(&tw, w, 2, dims, str, box, nullptr))) return rc;
  }
  const int grid = min(p.num_m_tiles * p.num_n_blocks, sm_count());
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) {
    static bool once = false;
    if (!once) { if ((rc = set_smem_attr(conv_fwd_implicit_kernel<256>, ConvCfg<256>::SMEM_BYTES))) return rc; once = true; }
    conv_fwd_implicit_kernel<256><<<grid, 320, ConvCfg<256>::SMEM_BYTES, st>>>(tx, tw, p);
  } else {
    static bool once = false;
    if (!once) { if ((rc = set_smem_attr(conv_fwd_implicit_kernel<128>, ConvCfg<128>::SMEM_BYTES))) return rc; once = true; }
    conv_fwd_implicit_kernel<128><<<grid, 320, ConvCfg<128>::SMEM_BYTES, st>>>(tx, tw, p);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

extern "C" {

// The plain convolution: y [N,OH,OW,O] with OH = (H + 2 PH - KH) / SH + 1.
int tnnb_conv2d_fwd_implicit(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int C, int O, int KH,
                             int KW, int SH, int SW, int PH, int PW, int relu, int* status, void* stream) {
  const int OH = (H + 2 * PH - KH) / SH + 1, OW = (W + 2 * PW - KW) / SW + 1;
  return conv_fwd_implicit_impl(x, w, bias, y, N, H, W, C, O, KH, KW, SH, SW, PH, PW, OH, OW, OH, OW, 1, 1, 0, 0, relu, status,
                                stream);
}

// 64 -> 64 channels, stride 1, KH <= 3, KW <= 3 (conv_fwd_halo_kernel): y [N,OH,OW,64] with OH = H + 2 PH - KH + 1.
int tnnb_conv2d_fwd_halo(const void* x, const void* w, const void* bias, void* y, int N, int H, int W, int C, int O, int KH, int KW,
                         int PH, int PW, int relu, int* status, void* stream) {
  if (C != 64 || O != 64 || KH < 1 || KH > 3 || KW < 1 || KW > 3 || PH < 0 || PW < 0) return -3;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return -4;
  ConvParams p{};
  p.N = N; p.O = O;
  p.OH = H + 2 * PH - KH + 1;
  p.OW = W + 2 * PW - KW + 1;
  if (p.OH <= 0 || p.OW <= 0) return -2;
  p.YH = p.OH; p.YW = p.OW; p.ys = p.xs = 1; p.yo = p.xo = 0;
  p.KH = KH; p.KW = KW; p.SH = p.SW = 1; p.PH = PH; p.PW = PW;
  p.cblocks = 1;
  p.TN = 1; p.TH = HaloCfg::TH; p.TW = HaloCfg::TW;
  p.lgTH = ilog2(p.TH); p.lgTW = ilog2(p.TW);
  p.tiles_n = N; p.tiles_h = (p.OH + p.TH - 1) / p.TH; p.tiles_w = (p.OW + p.TW - 1) / p.TW;
  p.num_m_tiles = p.tiles_n * p.tiles_h * p.tiles_w;
  p.num_n_blocks = 1;
  p.num_k_blocks = KH * KW;
  p.Y = (bf16*)y; p.bias = (const bf16*)bias; p.relu = relu; p.status = status;
  CUtensorMap tx, tw;
  int rc;
  if ((rc = map_nhwc(&tx, x, N, H, W, C, 64, HaloCfg::PITCH, HaloCfg::TH + KH - 1, 1, 1, 1))) return rc;
  {
    uint64_t dims[2] = {(uint64_t)KH * KW * C, (uint64_t)O};
    uint64_t str[1] = {(uint64_t)KH * KW * C * 2};
    uint32_t box[2] = {64, 64};
    if ((rc = encode_tmap_bf16(&tw, w, 2, dims, str, box, nullptr))) return rc;
  }
  static bool once = false;
  if (!once) { if ((rc = set_smem_attr(conv_fwd_halo_kernel, HaloCfg::SMEM_BYTES))) return rc; once = true; }
  const int grid = min(p.num_m_tiles, sm_count());
  conv_fwd_halo_kernel<<<grid, 192, HaloCfg::SMEM_BYTES, (cudaStream_t)stream>>>(tx, tw, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// One parity class of a larger output (see conv_fwd_implicit_impl).
int tnnb_conv2d_fwd_implicit_strided(const void* x, const void* w, void* y, int N, int H, int W, int C, int O, int KH, int KW,
                                     int PH, int PW, int OH, int OW, int YH, int YW, int ys, int xs, int yo, int xo, int* status,
                                     void* stream) {
  return conv_fwd_implicit_impl(x, w, nullptr, y, N, H, W, C, O, KH, KW, 1, 1, PH, PW, OH, OW, YH, YW, ys, xs, yo, xo, 0, status,
                                stream);
}

// C == O == 64, stride 1, KH <= 3, KW <= 3 (conv_wgrad_halo_kernel): dw [64,KH,KW,64] fp32 += the weight gradient.
int tnnb_conv2d_wgrad_halo(const void* x, const void* dy, void* dw, int N, int H, int W, int C, int O, int KH, int KW, int PH,
                           int PW, int* status, void* stream) {
  if (C != 64 || O != 64 || KH < 1 || KH > 3 || KW < 1 || KW > 3 || PH < 0 || PW < 0) return -3;
  if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dw) & 15) return -4;
  WgradParams p{};
  p.N = N; p.O = O; p.C = C;
  p.OH = H + 2 * PH - KH + 1;
  p.OW = W + 2 * PW - KW + 1;
  if (p.OH <= 0 || p.OW <= 0) return -2;
  p.KH = KH; p.KW = KW; p.SH = p.SW = 1; p.PH = PH; p.PW = PW;
  p.TN = 1; p.TH = WgradHaloCfg::TH; p.TW = WgradHaloCfg::TW;
  p.tiles_n = N; p.tiles_h = (p.OH + p.TH - 1) / p.TH; p.tiles_w = (p.OW + p.TW - 1) / p.TW;
  p.pix_blocks = p.tiles_n * p.tiles_h * p.tiles_w;
  p.dW = (float*)dw; p.status = status;
  CUtensorMap tdy, tx;
  int rc;
  if ((rc = map_nhwc(&tx, x, N, H, W, C, 64, WgradHaloCfg::PITCH, WgradHaloCfg::TH + KH - 1, 1, 1, 1))) return rc;
  if ((rc = map_nhwc(&tdy, dy, N, p.OH, p.OW, O, 64, WgradHaloCfg::TW, WgradHaloCfg::TH, 1, 1, 1))) return rc;
  static bool once = false;
  if (!once) { if ((rc = set_smem_attr(conv_wgrad_halo_kernel, WgradHaloCfg::SMEM_BYTES))) return rc; once = true; }
  const int grid = min(p.pix_blocks, sm_count());
  conv_wgrad_halo_kernel<<<grid, 192, WgradHaloCfg::SMEM_BYTES, (cudaStream_t)stream>>>(tdy, tx, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// dw [O,KH,KW,C] fp32 += correlation of x [N,H,W,C] with dy [N,OH,OW,O]. C % 64 == 0, O % 64 == 0.
int tnnb_conv2d_wgrad_implicit(const void* x, const void* dy, void* dw, int N, int H, int W, int C, int O, int KH, int KW, int SH,
                               int SW, int PH, int PW, int* status, void* stream) {
  if (C % 64 || O % 64 || C <= 0 || O <= 0) return -3;
  if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dw) & 15) return -4;
  WgradParams p{};
  p.N = N; p.O = O; p.C = C;
  p.OH = (H + 2 * PH - KH) / SH + 1;
  p.OW = (W + 2 * PW - KW) / SW + 1;
  if (p.OH <= 0 || p.OW <= 0) return -2;
  p.KH = KH; p.KW = KW; p.SH = SH; p.SW = SW; p.PH = PH; p.PW = PW;
  pick_box(64, N, p.OH, p.OW, p.TN, p.TH, p.TW);
  p.tiles_n = (N + p.TN - 1) / p.TN; p.tiles_h = (p.OH + p.TH - 1) / p.TH; p.tiles_w = (p.OW + p.TW - 1) / p.TW;
  p.pix_blocks = p.tiles_n * p.tiles_h * p.tiles_w;
  const int bn = (C > 128) ? 256 : 128;
  p.num_o_blocks = (O + 127) / 128;
  p.num_c_blocks = (C + bn - 1) / bn;
  const int base_items = KH * KW * p.num_o_blocks * p.num_c_blocks;
  int split = (2 * sm_count() + base_items - 1) / base_items;
  if (split > p.pix_blocks / 8) split = p.pix_blocks / 8;
  if (split < 1) split = 1;
  p.blocks_per_split = (p.pix_blocks + split - 1) / split;
  p.split = (p.pix_blocks + p.blocks_per_split - 1) / p.blocks_per_split;
  p.dW = (float*)dw; p.status = status;
  CUtensorMap tdy, tx;
  int rc;
  if ((rc = map_nhwc(&tdy, dy, N, p.OH, p.OW, O, 64, p.TW, p.TH, p.TN, 1, 1))) return rc;
  if ((rc = map_nhwc(&tx, x, N, H, W, C, 64, p.TW, p.TH, p.TN, SW, SH))) return rc;
  const int grid = min(p.split * base_items, sm_count());
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) {
    static bool once = false;
    if (!once) { if ((rc = set_smem_attr(conv_wgrad_implicit_kernel<256>, WgradCfg<256>::SMEM_BYTES))) return rc; once = true; }
    conv_wgrad_implicit_kernel<256><<<grid, 320, WgradCfg<256>::SMEM_BYTES, st>>>(tdy, tx, p);
  } else {
    static bool once = false;
    if (!once) { if ((rc = set_smem_attr(conv_wgrad_implicit_kernel<128>, WgradCfg<128>::SMEM_BYTES))) return rc; once = true; }
    conv_wgrad_implicit_kernel<128><<<grid, 320, WgradCfg<128>::SMEM_BYTES, st>>>(tdy, tx, p);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // extern "C"
