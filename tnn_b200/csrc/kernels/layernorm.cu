// Layer normalisation over the last dimension, fused with the residual add and
// dropout that surround it in a pre-LN transformer block:
//
//   forward   x_out = x_in + dropout(delta)          (delta optional)
//             h     = (x_out - mean) * rstd * gamma + beta
//   backward  dx    = dres + LN'(dh)                  (dres optional)
//             ddelta = dropout'(dx)                   (optional)
//             dgamma += sum dh * xhat, dbeta += sum dh  (fp32 atomics)
//
// One warp per row, the row held in registers (one read, one write). The
// reference runs layernorm through cuDNN graphs (cudnn_engine.cu:867-1075) or
// a one-thread-per-row fallback (cuda_engine.cu:962-1047) and launches the
// residual add and dropout separately; semantics (biased variance, eps inside
// the square root) follow src/nn/engines/cpu_engine.cpp:513-614.
//
// Tensor-parallel variants (template flag TP; protocol in tp_flags.cuh). With sequence parallelism every rank
// normalises its own rows, and the kernels on both sides of a layer norm are the fused GEMMs of the tensor-parallel
// transformer block, so the layer-norm kernels are where rows change hands:
//   pull  the `delta` (forward) / `dh` (backward) operand is the sum of the local partial result and the partial
//         results the peers' GEMM epilogues pushed into this rank's inbox; a warp polls the arrival counter of
//         its row's 128-row block before it reads the inbox.
//   push  `h` (forward) / `ddelta` (backward) is also stored into every peer's copy of the gather buffer, and the
//         block adds the rows it delivered to the peers' row-block counters once it has finished.
#include <cstdlib>

#include "ptx.cuh"
#include "tp_flags.cuh"

namespace tnnb {

typedef __nv_bfloat16 bf16;
struct alignas(16) LBf8 {
  bf16 v[8];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int MAXCH, bool TP>
__global__ void __launch_bounds__(256)
ln_fwd_kernel(const bf16* __restrict__ x_in, const bf16* __restrict__ delta, bf16* __restrict__ x_out,
              bf16* __restrict__ h, const bf16* __restrict__ gamma, const bf16* __restrict__ beta,
              float* __restrict__ mean_o, float* __restrict__ rstd_o, long long rows, int C, float eps,
              float p, unsigned long long seed, const unsigned long long* __restrict__ seed_off,
              const __grid_constant__ TpPull pull, const __grid_constant__ TpPush push) {
  seed = mix_seed(seed, seed_off);
  const uint32_t pull_want = (TP && pull.n) ? pull.units * *pull.pass : 0u;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int chunks = C >> 3;
  const float inv_keep = 1.f / (1.f - p);
  const uint32_t thr = dropout_threshold(p);
  // bulk push: every warp owns two row-sized staging buffers; lane 0 sends a finished row to each peer with one
  // bulk copy and reuses a buffer once the copy that last read it is done with shared memory
  extern __shared__ __align__(128) uint8_t ln_stage[];
  const bool bulk = TP && push.n && push.bulk;
  bf16* my_stage = reinterpret_cast<bf16*>(ln_stage) + (size_t)(threadIdx.x >> 5) * 2 * C;
  int sent = 0;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    float v[MAXCH][8];
    float s = 0.f;
    if (TP && pull.n) tp_pull_wait(pull, r, pull_want, lane);
    const bool send = bulk && r < push.rows;
    bf16* stage = my_stage + (sent & 1) * C;
    if (send && sent >= 2) {
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        LBf8 a = *reinterpret_cast<const LBf8*>(x_in + r * C + c * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] = __bfloat162float(a.v[k]);
        if (delta) {
          LBf8 d = *reinterpret_cast<const LBf8*>(delta + r * C + c * 8);
          float dsum[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) dsum[k] = __bfloat162float(d.v[k]);
          if (TP && pull.n) tp_pull_add8(pull, r * C + c * 8, dsum);
          const uint32_t keep = p > 0.f ? dropout_keep8(seed, (uint64_t)(r * chunks + c), thr) : 0xffu;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float dv = dsum[k];
            if (p > 0.f) dv = (keep >> k) & 1u ? dv * inv_keep : 0.f;
            // Round the residual stream to bf16 first so that the saved x_out and
            // the statistics below describe exactly the same numbers.
            v[i][k] = __bfloat162float(__float2bfloat16(v[i][k] + dv));
          }
          LBf8 o;
#pragma unroll
          for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16(v[i][k]);
          *reinterpret_cast<LBf8*>(x_out + r * C + c * 8) = o;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s += v[i][k];
      }
    }
    const float mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      if (lane + i * 32 < chunks) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float d = v[i][k] - mean;
          q += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    if (lane == 0) {
      mean_o[r] = mean;
      rstd_o[r] = rstd;
    }
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        LBf8 o;
        if (gamma) {
          LBf8 g = *reinterpret_cast<const LBf8*>(gamma + c * 8);
          LBf8 b = *reinterpret_cast<const LBf8*>(beta + c * 8);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            o.v[k] = __float2bfloat16((v[i][k] - mean) * rstd * __bfloat162float(g.v[k]) + __bfloat162float(b.v[k]));
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16((v[i][k] - mean) * rstd);
        }
        *reinterpret_cast<LBf8*>(h + r * C + c * 8) = o;
        if (send) {
          *reinterpret_cast<LBf8*>(stage + c * 8) = o;
        } else if (TP && r < push.rows) {
          for (int t = 0; t < push.n; ++t) *reinterpret_cast<LBf8*>(push.dst[t] + r * C + c * 8) = o;
        }
      }
    }
    if (send) {
      fence_proxy_async_smem();  // the lanes' stores to the staging row, before the bulk copy reads it
      __syncwarp();
      if (lane == 0) {
        for (int t = 0; t < push.n; ++t) bulk_store_s2g(push.dst[t] + r * C, stage, (uint32_t)C * 2u);
        bulk_commit_group();
      }
      ++sent;
    }
  }
  if (bulk && lane == 0) bulk_wait_group0();  // the rows have left before they are published
  if (TP && push.n) tp_push_signal(push, rows, wpb);
}

// Backward. One warp per row with the row held in registers as packed bf16; the dgamma / dbeta partial
// sums of a warp live in its private slice of shared memory (plain read-modify-write, no atomics), which
// keeps the register count low enough for several 256-thread blocks per SM - the kernel is bandwidth bound
// and needs that many loads in flight (three blocks at C <= 768).
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int MAXCH, bool TP>
__global__ void __launch_bounds__(256, (MAXCH <= 3) ? 3 : 2)
ln_bwd_kernel(const bf16* __restrict__ dh, const bf16* __restrict__ x, const float* __restrict__ mean_i,
              const float* __restrict__ rstd_i, const bf16* __restrict__ gamma, const bf16* __restrict__ dres,
              bf16* __restrict__ dx, bf16* __restrict__ ddelta, float* __restrict__ dgamma,
              float* __restrict__ dbeta, long long rows, int C, float p, unsigned long long seed,
              const unsigned long long* __restrict__ seed_off, const __grid_constant__ TpPull pull, const __grid_constant__ TpPush push,
              float* __restrict__ dbias) {
  // dbias (fp32 [C], optional): += column sums of ddelta - the bias gradient of the dense layer whose output was
  // added to the residual stream in front of this layer norm (a third accumulator beside dgamma / dbeta instead of a
  // separate pass over ddelta).
  seed = mix_seed(seed, seed_off);
  const uint32_t pull_want = (TP && pull.n) ? pull.units * *pull.pass : 0u;
  extern __shared__ float sm[];  // [warps][2][C]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  const int chunks = C >> 3;
  const float inv_keep = 1.f / (1.f - p);
  const uint32_t thr = dropout_threshold(p);
  const int nacc = dbias ? 3 : 2;
  float* acc_g = sm + (size_t)warp * nacc * C;
  float* acc_b = acc_g + C;
  float* acc_d = acc_b + C;  // only when dbias
  for (int i = lane; i < nacc * C; i += 32) acc_g[i] = 0.f;
  __syncwarp();
  const uint4 ones = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);  // bf16 1.0 x 8
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  for (long long r = (long long)blockIdx.x * wpb + warp; r < rows; r += (long long)gridDim.x * wpb) {
    uint4 xa[MAXCH], da[MAXCH], ra[MAXCH];
    if (TP && pull.n) tp_pull_wait(pull, r, pull_want, lane);
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      const bool in = c < chunks;
      xa[i] = in ? *reinterpret_cast<const uint4*>(x + r * C + c * 8) : zero4;
      da[i] = in ? *reinterpret_cast<const uint4*>(dh + r * C + c * 8) : zero4;
      ra[i] = (in && dres) ? *reinterpret_cast<const uint4*>(dres + r * C + c * 8) : zero4;
      if (TP && pull.n && in) {  // dh = local partial + the peers' partials, rounded to bf16 like a reduce-scatter result
        float t[8];
        unpack8(da[i], t);
        tp_pull_add8(pull, r * C + c * 8, t);
        da[i] = make_uint4(pack2(t[0], t[1]), pack2(t[2], t[3]), pack2(t[4], t[5]), pack2(t[6], t[7]));
      }
    }
    const float mean = mean_i[r], rstd = rstd_i[r];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        float xv[8], gv[8], gm[8];
        unpack8(xa[i], xv);
        unpack8(da[i], gv);
        unpack8(gamma ? *reinterpret_cast<const uint4*>(gamma + c * 8) : ones, gm);
        const float4 t0 = *reinterpret_cast<float4*>(acc_g + c * 8), t1 = *reinterpret_cast<float4*>(acc_g + c * 8 + 4);
        const float4 u0 = *reinterpret_cast<float4*>(acc_b + c * 8), u1 = *reinterpret_cast<float4*>(acc_b + c * 8 + 4);
        float ag[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
        float ab[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (xv[k] - mean) * rstd;
          ag[k] += gv[k] * xh;
          ab[k] += gv[k];
          const float dy = gv[k] * gm[k];
          s1 += dy;
          s2 += dy * xh;
        }
        *reinterpret_cast<float4*>(acc_g + c * 8) = make_float4(ag[0], ag[1], ag[2], ag[3]);
        *reinterpret_cast<float4*>(acc_g + c * 8 + 4) = make_float4(ag[4], ag[5], ag[6], ag[7]);
        *reinterpret_cast<float4*>(acc_b + c * 8) = make_float4(ab[0], ab[1], ab[2], ab[3]);
        *reinterpret_cast<float4*>(acc_b + c * 8 + 4) = make_float4(ab[4], ab[5], ab[6], ab[7]);
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        float xv[8], gv[8], gm[8], rv[8], o[8];
        unpack8(xa[i], xv);
        unpack8(da[i], gv);
        unpack8(ra[i], rv);
        unpack8(gamma ? *reinterpret_cast<const uint4*>(gamma + c * 8) : ones, gm);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (xv[k] - mean) * rstd;
          o[k] = rstd * (gv[k] * gm[k] - s1 - xh * s2) + rv[k];
        }
        const uint4 w = make_uint4(pack2(o[0], o[1]), pack2(o[2], o[3]), pack2(o[4], o[5]), pack2(o[6], o[7]));
        *reinterpret_cast<uint4*>(dx + r * C + c * 8) = w;
        if (ddelta) {
          float t[8];
          unpack8(w, t);  // dropout acts on the rounded dx, like a separate pass would
          if (p > 0.f) {
            const uint32_t keep = dropout_keep8(seed, (uint64_t)(r * chunks + c), thr);
#pragma unroll
            for (int k = 0; k < 8; ++k) t[k] = (keep >> k) & 1u ? t[k] * inv_keep : 0.f;
          }
          const uint4 dd = make_uint4(pack2(t[0], t[1]), pack2(t[2], t[3]), pack2(t[4], t[5]), pack2(t[6], t[7]));
          *reinterpret_cast<uint4*>(ddelta + r * C + c * 8) = dd;
          if (dbias) {
            float4 d0 = *reinterpret_cast<float4*>(acc_d + c * 8), d1 = *reinterpret_cast<float4*>(acc_d + c * 8 + 4);
            float td[8];
            unpack8(dd, td);  // the values as stored
            d0.x += td[0]; d0.y += td[1]; d0.z += td[2]; d0.w += td[3];
            d1.x += td[4]; d1.y += td[5]; d1.z += td[6]; d1.w += td[7];
            *reinterpret_cast<float4*>(acc_d + c * 8) = d0;
            *reinterpret_cast<float4*>(acc_d + c * 8 + 4) = d1;
          }
          if (TP && r < push.rows) {
            for (int u = 0; u < push.n; ++u) *reinterpret_cast<uint4*>(push.dst[u] + r * C + c * 8) = dd;
          }
        }
      }
    }
  }
  if (TP && push.n) tp_push_signal(push, rows, wpb);
  if (dgamma || dbias) {
    __syncthreads();
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
      float g = 0.f, bb = 0.f, dd = 0.f;
      for (int w = 0; w < wpb; ++w) {
        g += sm[(size_t)w * nacc * C + i];
        bb += sm[(size_t)w * nacc * C + C + i];
        if (dbias) dd += sm[(size_t)w * nacc * C + 2 * C + i];
      }
      if (dgamma) {
        atomicAdd(dgamma + i, g);
        atomicAdd(dbeta + i, bb);
      }
      if (dbias) atomicAdd(dbias + i, dd);
    }
  }
}

}  // namespace tnnb

using namespace tnnb;

static inline int pick_maxch(int C) {
  const int chunks = C / 8;
  const int per_lane = (chunks + 31) / 32;
  return per_lane <= 3 ? 3 : per_lane <= 5 ? 5 : per_lane <= 8 ? 8 : 0;
}

// Fill the parameter blocks of the tensor-parallel variants from flat C arguments (see tnnb_layernorm_fwd_tp).
static int make_tp_blocks(TpPull& pull, TpPush& push, int n_pull, void** pull_src, const void* arrived, const void* pass,
                          unsigned int units, int n_push, void** push_dst, void** push_ready, long long push_row0,
                          long long push_rows, int* status) {
  if (n_pull < 0 || n_pull > TP_MAX - 1 || n_push < 0 || n_push > TP_MAX - 1) return -2;
  pull = TpPull{};
  push = TpPush{};
  pull.n = n_pull;
  if (n_pull) {
    if (!pull_src || !arrived || !pass) return -5;
    for (int i = 0; i < n_pull; ++i) {
      if (!pull_src[i] || ((uintptr_t)pull_src[i] & 15)) return -4;
      pull.src[i] = (const bf16*)pull_src[i];
    }
    pull.arrived = (const uint32_t*)arrived;
    pull.pass = (const uint32_t*)pass;
    pull.units = units;
    pull.status = status;
  }
  push.n = n_push;
  const char* ln_bulk = getenv("TNNB_TP_LN_BULK");  // read per call: a test or benchmark may switch it
  push.bulk = ln_bulk ? atoi(ln_bulk) : 0;
  if (n_push) {
    if (!push_dst || !push_ready || push_row0 < 0 || (push_row0 % 8) || push_rows < 0 || (push_rows % 8)) return -5;
    push.row0 = (int)push_row0;
    push.rows = push_rows;
    for (int i = 0; i < n_push; ++i) {
      if (!push_dst[i] || !push_ready[i] || ((uintptr_t)push_dst[i] & 15)) return -4;
      push.dst[i] = (bf16*)push_dst[i];
      push.ready[i] = (uint32_t*)push_ready[i];
    }
  }
  return 0;
}

static int layernorm_fwd_impl(const void* x_in, const void* delta, void* x_out, void* h, const void* gamma,
                              const void* beta, void* mean, void* rstd, long long rows, int C, float eps, float p,
                              unsigned long long seed, const void* seed_off, void* stream, const TpPull* pull,
                              const TpPush* push) {
  if (C % 8 || rows <= 0) return -3;
  if ((delta == nullptr) != (x_out == nullptr)) return -5;
  const int mc = pick_maxch(C);
  if (!mc) return -7;
  const int block = 256, wpb = 8;
  long long g = (rows + wpb - 1) / wpb;
  int grid = (int)(g > 148 * 8 ? 148 * 8 : g);
  cudaStream_t st = (cudaStream_t)stream;
  TpPush push_local;
  if (push) {  // the staging rows of the bulk push must fit the default dynamic shared memory
    push_local = *push;
    if ((size_t)wpb * 2 * C * sizeof(bf16) > 48 * 1024) push_local.bulk = 0;
    push = &push_local;
  }
  const size_t stage_bytes = (push && push->n && push->bulk) ? (size_t)wpb * 2 * C * sizeof(bf16) : 0;
#define LN_F(MC, TP_, PL, PS)                                                                                       \
  ln_fwd_kernel<MC, TP_><<<grid, block, stage_bytes, st>>>((const bf16*)x_in, (const bf16*)delta, (bf16*)x_out, (bf16*)h,      \
                                                 (const bf16*)gamma, (const bf16*)beta, (float*)mean, (float*)rstd, \
                                                 rows, C, eps, p, seed, (const unsigned long long*)seed_off, PL, PS)
  if (pull) {
    if (mc == 3) LN_F(3, true, *pull, *push); else if (mc == 5) LN_F(5, true, *pull, *push); else LN_F(8, true, *pull, *push);
  } else {
    if (mc == 3) LN_F(3, false, TpPull{}, TpPush{}); else if (mc == 5) LN_F(5, false, TpPull{}, TpPush{}); else LN_F(8, false, TpPull{}, TpPush{});
  }
#undef LN_F
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

extern "C" {

// rows x C, C % 8 == 0 and C <= 2048. delta/x_out may be null together
// (plain layernorm of x_in); gamma/beta may be null together (no affine).
int tnnb_layernorm_fwd(const void* x_in, const void* delta, void* x_out, void* h, const void* gamma,
                       const void* beta, void* mean, void* rstd, long long rows, int C, float eps, float p,
                       unsigned long long seed, const void* seed_off, void* stream) {
  return layernorm_fwd_impl(x_in, delta, x_out, h, gamma, beta, mean, rstd, rows, C, eps, p, seed, seed_off, stream,
                            nullptr, nullptr);
}

// Tensor-parallel form. pull: delta is the sum of `delta` and pull_src[0..n_pull) (each [rows, C], local memory)
// once arrived[row / 128] has reached units x *pass. push: rows [0, push_rows) of h are also stored to push_dst[i]
// (peer i's gather buffer, already offset to this rank's first row) and the rows delivered are added to
// push_ready[i][(push_row0 + row) / 128]; the rest of the rows is sent by the GEMM that consumes the buffer.
int tnnb_layernorm_fwd_tp(const void* x_in, const void* delta, void* x_out, void* h, const void* gamma,
                          const void* beta, void* mean, void* rstd, long long rows, int C, float eps, float p,
                          unsigned long long seed, const void* seed_off, int n_pull, void** pull_src,
                          const void* arrived, const void* pass, unsigned int units, int n_push, void** push_dst,
                          void** push_ready, long long push_row0, long long push_rows, int* status, void* stream) {
  TpPull pull;
  TpPush push;
  const int rc = make_tp_blocks(pull, push, n_pull, pull_src, arrived, pass, units, n_push, push_dst, push_ready, push_row0,
                                push_rows, status);
  if (rc) return rc;
  if (n_pull && !delta) return -5;
  return layernorm_fwd_impl(x_in, delta, x_out, h, gamma, beta, mean, rstd, rows, C, eps, p, seed, seed_off, stream, &pull,
                            &push);
}

}  // extern "C"

static int layernorm_bwd_impl(const void* dh, const void* x, const void* mean, const void* rstd, const void* gamma,
                              const void* dres, void* dx, void* ddelta, void* dgamma, void* dbeta, long long rows,
                              int C, float p, unsigned long long seed, const void* seed_off, void* stream,
                              const TpPull* pull, const TpPush* push, void* dbias = nullptr) {
  if (C % 8 || rows <= 0) return -3;
  if (dbias && !ddelta) return -5;
  const int mc = pick_maxch(C);
  if (!mc) return -7;
  const int block = 256, wpb = 8;
  long long g = (rows + wpb - 1) / wpb;
  const int per_sm = (mc == 3) ? 3 : (mc == 5) ? 2 : 1;
  int grid = (int)(g > 148 * per_sm ? 148 * per_sm : g);
  size_t smem = (size_t)wpb * (dbias ? 3 : 2) * C * sizeof(float);  // <= 192 KB at C = 2048
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(ln_bwd_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 768 * 4);
    cudaFuncSetAttribute(ln_bwd_kernel<5, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 1280 * 4);
    cudaFuncSetAttribute(ln_bwd_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 2048 * 4);
    cudaFuncSetAttribute(ln_bwd_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 768 * 4);
    cudaFuncSetAttribute(ln_bwd_kernel<5, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 1280 * 4);
    cudaFuncSetAttribute(ln_bwd_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 2048 * 4);
    attr_done = true;
  }
  cudaStream_t st = (cudaStream_t)stream;
#define LN_B(MC, TP_, PL, PS)                                                                                          \
  ln_bwd_kernel<MC, TP_><<<grid, block, smem, st>>>((const bf16*)dh, (const bf16*)x, (const float*)mean,               \
                                                    (const float*)rstd, (const bf16*)gamma, (const bf16*)dres,         \
                                                    (bf16*)dx, (bf16*)ddelta, (float*)dgamma, (float*)dbeta, rows, C, \
                                                    p, seed, (const unsigned long long*)seed_off, PL, PS, (float*)dbias)
  if (pull) {
    if (mc == 3) LN_B(3, true, *pull, *push); else if (mc == 5) LN_B(5, true, *pull, *push); else LN_B(8, true, *pull, *push);
  } else {
    if (mc == 3) LN_B(3, false, TpPull{}, TpPush{}); else if (mc == 5) LN_B(5, false, TpPull{}, TpPush{}); else LN_B(8, false, TpPull{}, TpPush{});
  }
#undef LN_B
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

extern "C" {

// dgamma/dbeta (fp32 [C]) are accumulated into; pass null to skip them.
int tnnb_layernorm_bwd(const void* dh, const void* x, const void* mean, const void* rstd, const void* gamma,
                       const void* dres, void* dx, void* ddelta, void* dgamma, void* dbeta, long long rows,
                       int C, float p, unsigned long long seed, const void* seed_off, void* stream) {
  return layernorm_bwd_impl(dh, x, mean, rstd, gamma, dres, dx, ddelta, dgamma, dbeta, rows, C, p, seed, seed_off, stream,
                            nullptr, nullptr);
}

// The same with dbias (fp32 [C]) += column sums of ddelta: the bias gradient of the dense layer in front of the norm.
int tnnb_layernorm_bwd_db(const void* dh, const void* x, const void* mean, const void* rstd, const void* gamma,
                          const void* dres, void* dx, void* ddelta, void* dgamma, void* dbeta, void* dbias, long long rows,
                          int C, float p, unsigned long long seed, const void* seed_off, void* stream) {
  return layernorm_bwd_impl(dh, x, mean, rstd, gamma, dres, dx, ddelta, dgamma, dbeta, rows, C, p, seed, seed_off, stream,
                            nullptr, nullptr, dbias);
}

// Tensor-parallel form: dh is the sum of `dh` and the pulled partials; ddelta is also pushed (arguments as in
// tnnb_layernorm_fwd_tp).
int tnnb_layernorm_bwd_tp(const void* dh, const void* x, const void* mean, const void* rstd, const void* gamma,
                          const void* dres, void* dx, void* ddelta, void* dgamma, void* dbeta, long long rows,
                          int C, float p, unsigned long long seed, const void* seed_off, int n_pull, void** pull_src,
                          const void* arrived, const void* pass, unsigned int units, int n_push, void** push_dst,
                          void** push_ready, long long push_row0, long long push_rows, int* status, void* stream) {
  TpPull pull;
  TpPush push;
  const int rc = make_tp_blocks(pull, push, n_pull, pull_src, arrived, pass, units, n_push, push_dst, push_ready, push_row0,
                                push_rows, status);
  if (rc) return rc;
  if (n_push && !ddelta) return -5;
  return layernorm_bwd_impl(dh, x, mean, rstd, gamma, dres, dx, ddelta, dgamma, dbeta, rows, C, p, seed, seed_off, stream,
                            &pull, &push);
}

// Tensor-parallel form with the bias gradient of tnnb_layernorm_bwd_db.
int tnnb_layernorm_bwd_tp_db(const void* dh, const void* x, const void* mean, const void* rstd, const void* gamma,
                             const void* dres, void* dx, void* ddelta, void* dgamma, void* dbeta, void* dbias, long long rows,
                             int C, float p, unsigned long long seed, const void* seed_off, int n_pull, void** pull_src,
                             const void* arrived, const void* pass, unsigned int units, int n_push, void** push_dst,
                             void** push_ready, long long push_row0, long long push_rows, int* status, void* stream) {
  TpPull pull;
  TpPush push;
  const int rc = make_tp_blocks(pull, push, n_pull, pull_src, arrived, pass, units, n_push, push_dst, push_ready, push_row0,
                                push_rows, status);
  if (rc) return rc;
  if (n_push && !ddelta) return -5;
  return layernorm_bwd_impl(dh, x, mean, rstd, gamma, dres, dx, ddelta, dgamma, dbeta, rows, C, p, seed, seed_off, stream,
                            &pull, &push, dbias);
}

}  // extern "C"
