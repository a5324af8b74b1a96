// Fused compute + collective kernels over NVLink peer memory (plain P2P loads and
// stores issued from SM code; no NCCL call, no multicast TMA), plus the symmetric
// heap they operate on.
//
//   tnnb_gemm_ag   all-gather -> GEMM   Y[M, N] = AllGather_rows(X)[M, K] * op(W)^T
//       Every rank owns rows [r*M/tp, (r+1)*M/tp) of a symmetric [M, K] buffer.
//       Four copy warps per CTA of the persistent GEMM pull pieces (about 32 KB) of
//       the peers' row blocks into the local buffer with plain 16-byte loads,
//       sixteen in flight per thread (each byte crosses NVLink exactly once), and
//       set the piece's flag; the TMA producer runs every tile of the locally
//       owned rows first and checks the flags only when it reaches a peer's block,
//       so the transfer hides behind the local tiles. Operands reach the tensor
//       core by TMA from LOCAL memory only.
//   tnnb_gemm_rs   GEMM -> reduce-scatter   Y_r[M/tp, N] = sum_s (A_s * op(W_s)^T)[rows of r]
//       Tiles whose rows belong to a peer are computed first and their bf16
//       partial sums are stored from the epilogue (through a per-warp staging tile,
//       in whole 128-byte lines) into that peer's inbox, followed by a release
//       store of the call number into the flag of (tile, row quarter, column
//       half); tiles of the rank's own rows come last and add the peers' partials
//       (acquire on the flags) and the bias before the final store.
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

namespace tnnb {

typedef __nv_bfloat16 bf16;
static constexpr int MAX_PEERS = 8;

// ------------------------------------------------------------ flag primitives
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
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Spin until *p (system or gpu scope) has reached `want` (wrap-safe), for at most ~2 s.
template <bool SYS>
__device__ __forceinline__ bool spin_until(const uint32_t* p, uint32_t want) {
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0;; ++i) {
    const uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (static_cast<int32_t>(v - want) >= 0) return true;
    if ((i & 63u) == 63u && globaltimer_ns() - t0 > 2000000000ull) return false;
    __nanosleep(40);
  }
}

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

// ================================================================ fused GEMMs
enum CommMode { MODE_AG = 1, MODE_RS = 2 };

struct CommGemmParams {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int tp, rank, rows_per_rank, blocks_per_rank;
  uint32_t epoch;             // call counter: host value ...
  const uint32_t* epoch_ptr;  // ... plus an optional device-resident counter (CUDA-graph replays)
  int* status;
  const bf16* bias;
  PeerFlags peers;
  // --- all-gather side ---
  const bf16* ag_src[MAX_PEERS];  // peer r's [M, lda] buffer
  bf16* ag_dst;                   // this rank's [M, lda] buffer
  long long lda;
  uint32_t* chunk_flags[MAX_PEERS];  // rank r's piece flags (128 per row block); [rank] is local
  uint32_t* go_flag;              // local
  bf16* D;                        // MODE_AG: [M, N] output ; MODE_RS: [rows_per_rank, N] output
  long long ldd;
  // --- reduce-scatter side ---
  bf16* inbox_remote[MAX_PEERS];       // on owner o: slot that belongs to this rank, [rows_per_rank, ldi]
  const bf16* inbox_local[MAX_PEERS];  // local slot written by source s
  uint32_t* tile_flag_remote[MAX_PEERS];
  const uint32_t* tile_flag_local[MAX_PEERS];
  long long ldi;
  // --- extra epilogue of the all-gather GEMM: 1 = GELU (pre-activation saved to aux), 2 = times GELU'(aux) ---
  int epi;
  bf16* aux;  // [M, N], row pitch ldd
};

template <int BN, int MODE>
struct CommCfg {
  static constexpr int A_BYTES = 128 * 64 * 2;
  static constexpr int B_BYTES = BN * 64 * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  // all-gather: 4 epilogue warps + 4 copy warps; reduce-scatter: 8 epilogue warps
  static constexpr int EPI_WARPS = (MODE == MODE_AG) ? 4 : 8;
  static constexpr int THREADS = 320;
  static constexpr int COPY_THREADS = 128;  // all-gather: warps 6-9
  static constexpr int COPY_BYTES = 0;
  static constexpr int BARS = STAGES * STAGE_BYTES;          // 256 bytes of barriers
  static constexpr int STAGING = BARS + 256;                 // per epilogue warp 4 KB
  static constexpr int COPY = STAGING + EPI_WARPS * 4096;
  static constexpr int SMEM_BYTES = COPY + COPY_BYTES + 1024;
};

// Tile order. MODE_AG: every tile of the locally owned row blocks first (their operands are already
// here), then the peers' row blocks in the order the copy warps bring them in. MODE_RS: tiles whose rows
// belong to a peer first (their partial sums have the longest way to go), own rows last. Within the
// peers' part the order is row block by row block (all column tiles of a block before the next block),
// which is the order the data arrives in: the first remote tile needs one block, not all of them.
template <int MODE>
__device__ __forceinline__ void decode_tile(const CommGemmParams& p, int t, int& mb, int& nb) {
  const int bpr = p.blocks_per_rank;
  const int first_local = p.rank * bpr;
  const int remote_blocks = p.num_m_blocks - bpr;
  const int first_tiles = (MODE == MODE_AG ? bpr : remote_blocks) * p.num_n_blocks;
  const bool local = (MODE == MODE_AG) ? (t < first_tiles) : (t >= first_tiles);
  const int u = (t < first_tiles) ? t : t - first_tiles;
  const int j = u / p.num_n_blocks;  // row block inside its group
  nb = u - j * p.num_n_blocks;
  mb = local ? first_local + j : (first_local + bpr + j) % p.num_m_blocks;
}

__device__ __forceinline__ uint32_t cstage_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

template <int BN, int B_MN, int MODE>
__global__ void __launch_bounds__(CommCfg<BN, MODE>::THREADS, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const CommGemmParams p) {
  using Cfg = CommCfg<BN, MODE>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int EW = Cfg::EPI_WARPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::BARS);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* cbar = tempty + 2;  // [2] bounce buffers of the copy warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(cbar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t EPOCH = p.epoch + (p.epoch_ptr ? *p.epoch_ptr : 0u);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], EW);
      mbar_init(&cbar[a], 1);
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
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  // all-gather: a peer's 128-row block arrives as `cpb` pieces of `piece_rows` rows (about 32 KB each)
  const int piece_rows = max(1, min(128, 32768 / (p.K * 2)));
  const int cpb = (128 + piece_rows - 1) / piece_rows;

  if (warp == 0) {
    // lane 0 issues the TMA loads; the whole warp checks the piece flags of a peer's row block
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      int mb, nb;
      decode_tile<MODE>(p, t, mb, nb);
      if (MODE == MODE_AG && mb / p.blocks_per_rank != p.rank) {
        bool landed = true;
        for (int i = lane; i < cpb; i += 32) landed = spin_until<false>(p.chunk_flags[p.rank] + mb * 128 + i, EPOCH) && landed;
        landed = __all_sync(0xffffffffu, landed);
        if (!landed) {
          if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_PEER);
          break;
        }
        fence_proxy_async_all();
      }
      if (lane == 0) {
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!wait_or_abort(&empty[stage], phase ^ 1, abort_flag)) {
            raise_abort(p.status, abort_flag, ST_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* a_dst = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_dst = a_dst + Cfg::A_BYTES;
          tma_load_2d(a_dst, &tmA, &full[stage], kb * 64, mb * 128);
          if (B_MN == 0) {
            tma_load_2d(b_dst, &tmB, &full[stage], kb * 64, nb * BN);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(b_dst + i * 8192, &tmB, &full[stage], nb * BN + i * 64, kb * 64);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN, 0, B_MN);
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
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t ad = make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(b_addr + k * 2048, 8192, 1024) : make_smem_desc(b_addr + k * 32, 16, 1024);
            tc_mma_ss(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
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
  } else if (warp < 2 + EW) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                               // TMEM lane quarter
    const int half = (EW == 8) ? ((warp - 2) >> 2) : 0;   // column half when eight warps share a tile
    constexpr int COLS = BN / (EW / 4);                   // accumulator columns of this warp
    uint8_t* stage_tile = smem + Cfg::STAGING + (warp - 2) * 4096;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      int mb, nb;
      decode_tile<MODE>(p, t, mb, nb);
      if (!wait_or_abort(&tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after();
      const int row_base = mb * 128 + q * 32;             // global row of lane 0
      const int row = row_base + lane;
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16) + half * COLS;
      const int col_base = nb * BN + half * COLS;
      const int owner = (MODE == MODE_RS) ? mb / p.blocks_per_rank : p.rank;
      const int lrow_base = row_base - owner * p.rows_per_rank;   // row inside the owner's block (MODE_RS)
      const int fidx = ((mb - owner * p.blocks_per_rank) * p.num_n_blocks + nb) * 8 + q * 2 + half;
      const bool remote = (MODE == MODE_RS) && owner != p.rank;
      if (MODE == MODE_RS && !remote) {
        // every source must have delivered this warp's part of the tile for this call
        bool peers_ok = true;
        for (int s = 0; s < p.tp; ++s)
          if (s != p.rank) peers_ok = spin_until<true>(p.tile_flag_local[s] + fidx, EPOCH) && peers_ok;
        peers_ok = __all_sync(0xffffffffu, peers_ok);
        if (!peers_ok && lane == 0) raise_abort(p.status, abort_flag, ST_TIMEOUT_PEER);
      }
      // destination of bf16 rows for the coalesced flush: the output, or the owner's inbox
      bf16* dst = remote ? p.inbox_remote[owner] : p.D;
      const long long dld = remote ? p.ldi : p.ldd;
      const int drow_base = (MODE == MODE_RS) ? lrow_base : row_base;
      const int drows = (MODE == MODE_RS) ? p.rows_per_rank : p.M;
#pragma unroll 1
      for (int c = 0; c < COLS / 32; c += 2) {
        const int col0 = col_base + c * 32;
        if (col0 >= p.N) continue;
        const bool vec_ok = (col0 + 64 <= p.N) && (dld % 8 == 0) && (p.ldi % 8 == 0);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + (c + h) * 32, r);
          tmem_ld_wait();
          const int cc = col0 + h * 32;
          if (cc >= p.N) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (MODE == MODE_RS && !remote && vec_ok) {
            // own rows: fp32 partial through the staging tile, the peers' partials and the bias are added
            // in the coalesced phase (8 lanes per row, 4 columns each)
#pragma unroll
            for (int k = 0; k < 8; ++k)
              *reinterpret_cast<float4*>(stage_tile + cstage_off(lane, k)) = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
            __syncwarp();
            float4 a[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = *reinterpret_cast<const float4*>(stage_tile + cstage_off(i * 4 + (lane >> 3), lane & 7));
            const int c4 = lane & 7;
            for (int s = 0; s < p.tp; ++s) {
              if (s == p.rank) continue;
              uint2 raw[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {  // eight independent loads in flight before any is used
                const int lr = lrow_base + i * 4 + (lane >> 3);
                raw[i] = make_uint2(0, 0);
                if (lr < drows)
                  asm volatile("ld.relaxed.gpu.global.v2.u32 {%0,%1}, [%2];" : "=r"(raw[i].x), "=r"(raw[i].y)
                               : "l"(p.inbox_local[s] + (long long)lr * p.ldi + cc + c4 * 4));
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                a[i].x += __uint_as_float(raw[i].x << 16); a[i].y += __uint_as_float(raw[i].x & 0xffff0000u);
                a[i].z += __uint_as_float(raw[i].y << 16); a[i].w += __uint_as_float(raw[i].y & 0xffff0000u);
              }
            }
            float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.bias) {
              const uint2 braw = *reinterpret_cast<const uint2*>(p.bias + cc + c4 * 4);
              bb = make_float4(__uint_as_float(braw.x << 16), __uint_as_float(braw.x & 0xffff0000u), __uint_as_float(braw.y << 16),
                               __uint_as_float(braw.y & 0xffff0000u));
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int lr = lrow_base + i * 4 + (lane >> 3);
              if (lr < drows) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a[i].x + bb.x, a[i].y + bb.y), hi = __floats2bfloat162_rn(a[i].z + bb.z, a[i].w + bb.w);
                *reinterpret_cast<uint2*>(p.D + (long long)lr * p.ldd + cc + c4 * 4) =
                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
              }
            }
            __syncwarp();
            continue;
          }
          if (MODE == MODE_RS && !remote) {  // ragged edge of an own tile: row-per-lane
            const int lr = lrow_base + lane;
            if (lr < drows) {
              for (int j = 0; j < 32 && cc + j < p.N; ++j) {
                float a = v[j];
                for (int s = 0; s < p.tp; ++s)
                  if (s != p.rank) a += __bfloat162float(p.inbox_local[s][(long long)lr * p.ldi + cc + j]);
                if (p.bias) a += __bfloat162float(p.bias[cc + j]);
                p.D[(long long)lr * p.ldd + cc + j] = __float2bfloat16(a);
              }
            }
            continue;
          }
          // all-gather GEMM: bias and the optional GELU pair, row-per-lane
          bool store_aux = false;
          if (MODE == MODE_AG) {
            const bool fullc = cc + 32 <= p.N;
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (fullc || cc + j < p.N) v[j] += __bfloat162float(p.bias[cc + j]);
            }
            if (p.epi == 2 && row < p.M) {
              const bf16* ax = p.aux + (long long)row * p.ldd + cc;
              if (fullc && (p.ldd % 8 == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(ax + j);
                  const bf16* tt = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
                  for (int k = 0; k < 8; ++k) v[j + k] *= gelu_tanh_grad(__bfloat162float(tt[k]));
                }
              } else {
                for (int j = 0; j < 32 && cc + j < p.N; ++j) v[j] *= gelu_tanh_grad(__bfloat162float(ax[j]));
              }
            }
            store_aux = (p.epi == 1);
          }
          if (!vec_ok) {  // ragged edge: row-per-lane stores
            const int dr = drow_base + lane;
            if (dr < drows) {
              for (int j = 0; j < 32 && cc + j < p.N; ++j) {
                float a = v[j];
                if (store_aux) {
                  const bf16 z = __float2bfloat16(a);
                  p.aux[(long long)row * p.ldd + cc + j] = z;
                  a = gelu_tanh(__bfloat162float(z));
                }
                dst[(long long)dr * dld + cc + j] = __float2bfloat16(a);
              }
            }
            continue;
          }
          // coalesced path: 64 columns of bf16 per flush (this chunk fills half of the staging rows)
          if (store_aux) {
            // pre-activation first (it is what the backward pass needs), through its own flush
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * k + 2 * j], v[8 * k + 2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&h2);
                v[8 * k + 2 * j] = gelu_tanh(__low2float(h2));
                v[8 * k + 2 * j + 1] = gelu_tanh(__high2float(h2));
              }
              *reinterpret_cast<uint4*>(stage_tile + cstage_off(lane, k)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // 32 columns = 64 bytes per row: 4 lanes per row
              const int rr = i * 8 + (lane >> 2), c16 = lane & 3;
              if (i < 4 && row_base + rr < p.M)
                *reinterpret_cast<uint4*>(p.aux + (long long)(row_base + rr) * p.ldd + cc + c16 * 8) =
                    *reinterpret_cast<const uint4*>(stage_tile + cstage_off(rr, c16));
            }
            __syncwarp();
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * k + 2 * j], v[8 * k + 2 * j + 1]);
              w[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(stage_tile + cstage_off(lane, h * 4 + k)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (h == 1) {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3), c16 = lane & 7;
              if (drow_base + rr < drows)
                *reinterpret_cast<uint4*>(dst + (long long)(drow_base + rr) * dld + col0 + c16 * 8) =
                    *reinterpret_cast<const uint4*>(stage_tile + cstage_off(rr, c16));
            }
            __syncwarp();
          }
        }
      }
      if (remote) {
        // make this warp's rows of partial sums visible at the owner, then publish the call number in the
        // flag of (tile, row quarter, column half): the owner's warp with the same (q, half) needs exactly these
        __threadfence_system();
        __syncwarp();
        if (lane == 0) st_release_sys(p.tile_flag_remote[owner] + fidx, EPOCH);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  } else if (MODE == MODE_AG) {
    // ---------------------------------------------------------------- all-gather copy (warps 6 to 9)
    // PULL with plain 16-byte loads: the 128 copy threads of every CTA bring pieces (about 32 KB, whole rows) of
    // the peers' row blocks into the local buffer, sixteen loads in flight per thread, in the order the tiles
    // need them, and set the piece's flag. (Bulk async copies were measured slower here in both directions:
    // a remote bulk load has a long latency and few can be in flight per SM, a remote bulk store completes late.)
    constexpr int CT = Cfg::COPY_THREADS;
    const int cw = threadIdx.x - 192;  // 0..CT-1
    if (blockIdx.x == 0 && warp == 6) {
      // a peer's rows may be read once every rank has reached this kernel
      const bool ok = peer_barrier_warp(p.peers, EPOCH, lane);
      if (lane == 0) {
        if (!ok && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER);
        st_release_gpu(p.go_flag, EPOCH);  // released even on a timeout so that nothing waits twice
      }
    }
    if (cw == 0 && !spin_until<false>(p.go_flag, EPOCH) && p.status) atomicCAS(p.status, 0, ST_TIMEOUT_PEER);
    asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory");  // the copy warps only
    const int remote_blocks = p.num_m_blocks - p.blocks_per_rank;
    const int total = remote_blocks * cpb;
    const int chunks_per_row = p.K / 8;
    for (int c = blockIdx.x; c < total; c += gridDim.x) {
      const int j = c / cpb, part = c - j * cpb;
      const int mb = (p.rank * p.blocks_per_rank + p.blocks_per_rank + j) % p.num_m_blocks;
      const int r0 = part * piece_rows;
      const int nrows = min(piece_rows, 128 - r0);
      const bf16* src = p.ag_src[mb / p.blocks_per_rank] + ((long long)mb * 128 + r0) * p.lda;
      bf16* dst = p.ag_dst + ((long long)mb * 128 + r0) * p.lda;
      const int n16 = nrows * chunks_per_row;
      for (int e0 = 0; e0 < n16; e0 += CT * 16) {
        uint4 v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int e = e0 + u * CT + cw;
          if (e < n16) {
            const int rr = e / chunks_per_row, cc = e - rr * chunks_per_row;
            v[u] = *reinterpret_cast<const uint4*>(src + (long long)rr * p.lda + cc * 8);
          }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int e = e0 + u * CT + cw;
          if (e < n16) {
            const int rr = e / chunks_per_row, cc = e - rr * chunks_per_row;
            *reinterpret_cast<uint4*>(dst + (long long)rr * p.lda + cc * 8) = v[u];
          }
        }
      }
      __threadfence();
      fence_proxy_async_all();
      asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory");
      if (cw == 0) st_release_gpu(p.chunk_flags[p.rank] + mb * 128 + part, EPOCH);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
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

template <typename K>
static int set_dyn_smem(K kern, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

template <int BN, int B_MN, int MODE>
static int launch_comm(const CUtensorMap& ta, const CUtensorMap& tb, const CommGemmParams& p, int grid, cudaStream_t st) {
  auto kern = gemm_comm_kernel<BN, B_MN, MODE>;
  static bool once = false;
  if (!once) {
    int rc = set_dyn_smem(kern, CommCfg<BN, MODE>::SMEM_BYTES);
    if (rc) return rc;
    once = true;
  }
  kern<<<grid, CommCfg<BN, MODE>::THREADS, CommCfg<BN, MODE>::SMEM_BYTES, st>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
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

// Arrays of `tp` pointers are indexed by tensor-parallel rank; entries for this rank may be null
// where they are not needed. mode: 1 = all-gather->GEMM, 2 = GEMM->reduce-scatter.
int tnnb_gemm_comm(int mode, int M, int N, int K, int b_mn, const void* A, long long lda, const void* B,
                   long long ldb, void* D, long long ldd, const void* bias, int tp, int rank, int rows_per_rank,
                   unsigned int epoch, const void* epoch_ptr, void** barrier_flags, void** ag_src, void** chunk_flags,
                   void* go_flag,
                   void** inbox_remote, void** inbox_local, void** tile_flag_remote, void** tile_flag_local,
                   long long ldi, int epi, void* aux, int* status, void* stream) {
  if (tp < 1 || tp > MAX_PEERS || rank < 0 || rank >= tp) return -2;
  if (rows_per_rank % 128 || rows_per_rank * tp != M) return -8;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -3;
  CommGemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.num_m_blocks = M / 128;
  p.num_k_blocks = (K + 63) / 64;
  const int bn = (N > 128) ? 256 : 128;
  p.num_n_blocks = (N + bn - 1) / bn;
  p.tp = tp; p.rank = rank; p.rows_per_rank = rows_per_rank; p.blocks_per_rank = rows_per_rank / 128;
  p.epoch = epoch; p.epoch_ptr = (const uint32_t*)epoch_ptr; p.status = status; p.bias = (const bf16*)bias;
  p.peers.rank = rank; p.peers.world = tp;
  for (int r = 0; r < tp; ++r) {
    p.peers.flags[r] = barrier_flags ? (uint32_t*)barrier_flags[r] : nullptr;
    p.ag_src[r] = ag_src ? (const bf16*)ag_src[r] : nullptr;
    p.inbox_remote[r] = inbox_remote ? (bf16*)inbox_remote[r] : nullptr;
    p.inbox_local[r] = inbox_local ? (const bf16*)inbox_local[r] : nullptr;
    p.tile_flag_remote[r] = tile_flag_remote ? (uint32_t*)tile_flag_remote[r] : nullptr;
    p.tile_flag_local[r] = tile_flag_local ? (const uint32_t*)tile_flag_local[r] : nullptr;
  }
  p.ag_dst = (bf16*)A; p.lda = lda;
  for (int r = 0; r < tp; ++r) p.chunk_flags[r] = chunk_flags ? (uint32_t*)((void**)chunk_flags)[r] : nullptr;
  p.go_flag = (uint32_t*)go_flag;
  p.D = (bf16*)D; p.ldd = ldd; p.ldi = ldi;
  p.epi = epi; p.aux = (bf16*)aux;
  if (epi && !aux) return -5;
  if (mode == MODE_AG && (K % 8)) return -3;

  CUtensorMap ta, tb;
  int rc;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, 128};
    if ((rc = encode_tmap_bf16(&ta, A, 2, dims, str, box, nullptr))) return rc;
  }
  if (!b_mn) {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, (uint32_t)bn};
    rc = encode_tmap_bf16(&tb, B, 2, dims, str, box, nullptr);
  } else {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, 64};
    rc = encode_tmap_bf16(&tb, B, 2, dims, str, box, nullptr);
  }
  if (rc) return rc;
  const int grid = min(p.num_m_blocks * p.num_n_blocks, sm_count());
  cudaStream_t st = (cudaStream_t)stream;
#define CL(BN_, BM_, MD_) return launch_comm<BN_, BM_, MD_>(ta, tb, p, grid, st)
  if (mode == MODE_AG) {
    if (bn == 256) { if (b_mn) CL(256, 1, MODE_AG); CL(256, 0, MODE_AG); }
    if (b_mn) CL(128, 1, MODE_AG); CL(128, 0, MODE_AG);
  } else if (mode == MODE_RS) {
    if (bn == 256) { if (b_mn) CL(256, 1, MODE_RS); CL(256, 0, MODE_RS); }
    if (b_mn) CL(128, 1, MODE_RS); CL(128, 0, MODE_RS);
  }
#undef CL
  return -2;
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
