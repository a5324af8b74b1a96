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
#include "ptx.cuh"

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

template <int MAXCH>
__global__ void __launch_bounds__(256)
ln_fwd_kernel(const bf16* __restrict__ x_in, const bf16* __restrict__ delta, bf16* __restrict__ x_out,
              bf16* __restrict__ h, const bf16* __restrict__ gamma, const bf16* __restrict__ beta,
              float* __restrict__ mean_o, float* __restrict__ rstd_o, long long rows, int C, float eps,
              float p, unsigned long long seed, const unsigned long long* __restrict__ seed_off) {
  seed = mix_seed(seed, seed_off);
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int chunks = C >> 3;
  const float inv_keep = 1.f / (1.f - p);
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    float v[MAXCH][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        LBf8 a = *reinterpret_cast<const LBf8*>(x_in + r * C + c * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[i][k] = __bfloat162float(a.v[k]);
        if (delta) {
          LBf8 d = *reinterpret_cast<const LBf8*>(delta + r * C + c * 8);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float dv = __bfloat162float(d.v[k]);
            if (p > 0.f) dv = hash_uniform(seed, r * C + c * 8 + k) >= p ? dv * inv_keep : 0.f;
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
      }
    }
  }
}

template <int MAXCH>
__global__ void __launch_bounds__(256)
ln_bwd_kernel(const bf16* __restrict__ dh, const bf16* __restrict__ x, const float* __restrict__ mean_i,
              const float* __restrict__ rstd_i, const bf16* __restrict__ gamma, const bf16* __restrict__ dres,
              bf16* __restrict__ dx, bf16* __restrict__ ddelta, float* __restrict__ dgamma,
              float* __restrict__ dbeta, long long rows, int C, float p, unsigned long long seed,
              const unsigned long long* __restrict__ seed_off) {
  seed = mix_seed(seed, seed_off);
  extern __shared__ float sm[];  // [2][C]
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int chunks = C >> 3;
  const float inv_keep = 1.f / (1.f - p);
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) sm[i] = 0.f;
  __syncthreads();

  float gw[MAXCH][8];
  float ag[MAXCH][8], ab[MAXCH][8];
#pragma unroll
  for (int i = 0; i < MAXCH; ++i) {
    const int c = lane + i * 32;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      ag[i][k] = 0.f;
      ab[i][k] = 0.f;
      gw[i][k] = 1.f;
    }
    if (gamma && c < chunks) {
      LBf8 g = *reinterpret_cast<const LBf8*>(gamma + c * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) gw[i][k] = __bfloat162float(g.v[k]);
    }
  }

  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    const float mean = mean_i[r], rstd = rstd_i[r];
    float xh[MAXCH][8], dy[MAXCH][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        LBf8 a = *reinterpret_cast<const LBf8*>(x + r * C + c * 8);
        LBf8 d = *reinterpret_cast<const LBf8*>(dh + r * C + c * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[i][k] = (__bfloat162float(a.v[k]) - mean) * rstd;
          const float g = __bfloat162float(d.v[k]);
          ag[i][k] += g * xh[i][k];
          ab[i][k] += g;
          dy[i][k] = g * gw[i][k];
          s1 += dy[i][k];
          s2 += dy[i][k] * xh[i][k];
        }
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rstd * (dy[i][k] - s1 - xh[i][k] * s2);
        if (dres) {
          LBf8 rr = *reinterpret_cast<const LBf8*>(dres + r * C + c * 8);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += __bfloat162float(rr.v[k]);
        }
        LBf8 w;
#pragma unroll
        for (int k = 0; k < 8; ++k) w.v[k] = __float2bfloat16(o[k]);
        *reinterpret_cast<LBf8*>(dx + r * C + c * 8) = w;
        if (ddelta) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float t = __bfloat162float(w.v[k]);
            if (p > 0.f) t = hash_uniform(seed, r * C + c * 8 + k) >= p ? t * inv_keep : 0.f;
            w.v[k] = __float2bfloat16(t);
          }
          *reinterpret_cast<LBf8*>(ddelta + r * C + c * 8) = w;
        }
      }
    }
  }
  if (dgamma) {
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          atomicAdd(&sm[c * 8 + k], ag[i][k]);
          atomicAdd(&sm[C + c * 8 + k], ab[i][k]);
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
      atomicAdd(dgamma + i, sm[i]);
      atomicAdd(dbeta + i, sm[C + i]);
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

extern "C" {

// rows x C, C % 8 == 0 and C <= 2048. delta/x_out may be null together
// (plain layernorm of x_in); gamma/beta may be null together (no affine).
int tnnb_layernorm_fwd(const void* x_in, const void* delta, void* x_out, void* h, const void* gamma,
                       const void* beta, void* mean, void* rstd, long long rows, int C, float eps, float p,
                       unsigned long long seed, const void* seed_off, void* stream) {
  if (C % 8 || rows <= 0) return -3;
  if ((delta == nullptr) != (x_out == nullptr)) return -5;
  const int mc = pick_maxch(C);
  if (!mc) return -7;
  const int block = 256, wpb = 8;
  long long g = (rows + wpb - 1) / wpb;
  int grid = (int)(g > 148 * 8 ? 148 * 8 : g);
  cudaStream_t st = (cudaStream_t)stream;
#define LN_F(MC)                                                                                          \
  ln_fwd_kernel<MC><<<grid, block, 0, st>>>((const bf16*)x_in, (const bf16*)delta, (bf16*)x_out, (bf16*)h, \
                                            (const bf16*)gamma, (const bf16*)beta, (float*)mean,          \
                                            (float*)rstd, rows, C, eps, p, seed, (const unsigned long long*)seed_off)
  if (mc == 3) LN_F(3); else if (mc == 5) LN_F(5); else LN_F(8);
#undef LN_F
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

// dgamma/dbeta (fp32 [C]) are accumulated into; pass null to skip them.
int tnnb_layernorm_bwd(const void* dh, const void* x, const void* mean, const void* rstd, const void* gamma,
                       const void* dres, void* dx, void* ddelta, void* dgamma, void* dbeta, long long rows,
                       int C, float p, unsigned long long seed, const void* seed_off, void* stream) {
  if (C % 8 || rows <= 0) return -3;
  const int mc = pick_maxch(C);
  if (!mc) return -7;
  const int block = 256, wpb = 8;
  long long g = (rows + wpb - 1) / wpb;
  int grid = (int)(g > 148 * 2 ? 148 * 2 : g);
  size_t smem = 2 * (size_t)C * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
#define LN_B(MC)                                                                                              \
  ln_bwd_kernel<MC><<<grid, block, smem, st>>>((const bf16*)dh, (const bf16*)x, (const float*)mean,           \
                                               (const float*)rstd, (const bf16*)gamma, (const bf16*)dres,     \
                                               (bf16*)dx, (bf16*)ddelta, (float*)dgamma, (float*)dbeta, rows, \
                                               C, p, seed, (const unsigned long long*)seed_off)
  if (mc == 3) LN_B(3); else if (mc == 5) LN_B(5); else LN_B(8);
#undef LN_B
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // extern "C"
