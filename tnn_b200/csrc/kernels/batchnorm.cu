// Batch normalisation over [M, C] (M = N*H*W, channels last), bf16 I/O, fp32 statistics.
//
//   training forward   two passes: per-channel sum / sum of squares (block partials in fp32,
//                      combined with double atomics) then normalise + affine (+ReLU); the
//                      second kernel also updates the running statistics (unbiased variance)
//                      and stores mean / inv_std for the backward
//   backward           two passes: sum(dy), sum(dy * xhat) with the ReLU mask taken from the
//                      saved output, then dx = gamma*inv_std/M * (M*dy - sum(dy) - xhat*sum(dy*xhat))
//   inference          one pass with the running statistics
//
// Semantics follow src/nn/engines/cpu_engine.cpp:378-511 (biased variance for normalisation,
// unbiased for the running estimate, ReLU mask applied to dy first). The reference runs cuDNN
// batchnorm graphs (cudnn_engine.cu:580-865) or block-per-channel NCHW kernels
// (cuda_engine.cu:295-672). Each pass moves 16-byte vectors and reads x exactly once.
#include "ptx.cuh"

TNNB_BOUNDS_TU(batchnorm)

namespace tnnb {

typedef __nv_bfloat16 bf16;

// Thread layout of all kernels here: a block of 256 threads is `cl` channel groups of 8 channels x `256 / cl` row
// lanes, with cl = the largest power of two <= min(32, C / 8), so that narrow tensors (C = 64: 8 groups x 32 row
// lanes) keep every thread busy. grid = (ceil(C / 8 / cl), row splits).
struct BnLane {
  int cl, cx, ry, nry, c0;
};
__device__ __forceinline__ BnLane bn_lane(int C) {
  BnLane l;
  const int groups = C >> 3;
  l.cl = 32;
  while (l.cl > groups) l.cl >>= 1;
  l.cx = threadIdx.x & (l.cl - 1);
  l.ry = threadIdx.x / l.cl;
  l.nry = 256 / l.cl;
  l.c0 = (blockIdx.x * l.cl + l.cx) * 8;
  return l;
}
static constexpr int BN_U = 4;  // rows in flight per thread and trip of the row loops
static int bn_cl(int C) {
  int cl = 32;
  while (cl > (C >> 3)) cl >>= 1;
  return cl < 1 ? 1 : cl;
}

// ws: double[2*C] (sum, sum of squares) - or (sum dy, sum dy*xhat) for the backward.
// MASK (backward with a fused ReLU): 0 = none, 1 = y > 0 read from the saved output, 2 = recomputed from x.
template <bool BWD, int MASK>
__global__ void __launch_bounds__(256, 2)
bn_reduce_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                 const bf16* __restrict__ gamma, const bf16* __restrict__ beta,
                 const float* __restrict__ mean, const float* __restrict__ rstd, double* __restrict__ ws, long long M,
                 int C, long long rows_per_block) {
  __shared__ float red[2][256][9];
  const BnLane ln = bn_lane(C);
  const int cx = ln.cx, ry = ln.ry, c0 = ln.c0, nry = ln.nry;
  const long long r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  float a[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a[k] = 0.f, b[k] = 0.f;
  if (c0 < C) {
    float mu[8], rs[8], sc[8], sh[8];
    // Fused ReLU without the saved output: the mask y > 0 is recomputed from x with the forward's own expression
    // (same fp32 scale and shift), which saves one of the three tensor reads of this pass.
    constexpr bool remask = BWD && MASK == 2;
    constexpr bool relu = BWD && MASK != 0;
    if (BWD) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        mu[k] = mean[c0 + k], rs[k] = rstd[c0 + k];
        sc[k] = (gamma ? __bfloat162float(gamma[c0 + k]) : 1.f) * rs[k];
        sh[k] = (beta ? __bfloat162float(beta[c0 + k]) : 0.f) - mu[k] * sc[k];
      }
    }
    // BN_U rows per trip: all loads of a trip are issued before the first use, which keeps enough bytes in flight
    // per SM to cover the DRAM latency. Rows past the end load nothing and contribute zeros.
    constexpr int U = BWD ? BN_U : 2 * BN_U;  // the forward statistics pass reads one tensor: twice the rows
    for (long long r = r0 + ry; r < r1; r += U * nry) {
      uint4 xr[U], gr[BWD ? U : 1], yr[MASK == 1 ? U : 1];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long rr = r + (long long)u * nry;
        const bool ok = rr < r1 && TNNB_CHECK(rr * C + c0 + 7, M * (long long)C);  // lane layout vs. tensor extent
        xr[u] = make_uint4(0, 0, 0, 0);
        if (BWD) gr[BWD ? u : 0] = make_uint4(0, 0, 0, 0);
        if (MASK == 1) yr[MASK == 1 ? u : 0] = make_uint4(0, 0, 0, 0);
        if (ok) {
          xr[u] = *reinterpret_cast<const uint4*>(x + rr * C + c0);
          if (BWD) gr[BWD ? u : 0] = *reinterpret_cast<const uint4*>(dy + rr * C + c0);
          if (MASK == 1) yr[MASK == 1 ? u : 0] = *reinterpret_cast<const uint4*>(y + rr * C + c0);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const bf16* xv = reinterpret_cast<const bf16*>(&xr[u]);
        if (!BWD) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float v = __bfloat162float(xv[k]);
            a[k] += v;
            b[k] += v * v;
          }
        } else {
          const bf16* gv = reinterpret_cast<const bf16*>(&gr[BWD ? u : 0]);
          const bf16* yv = reinterpret_cast<const bf16*>(&yr[MASK == 1 ? u : 0]);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float g = __bfloat162float(gv[k]);
            const float xf = __bfloat162float(xv[k]);
            if (remask) {
              if (!(__bfloat162float(__float2bfloat16(xf * sc[k] + sh[k])) > 0.f)) g = 0.f;
            } else if (relu && !(__bfloat162float(yv[k]) > 0.f)) {
              g = 0.f;
            }
            a[k] += g;
            b[k] += g * (xf - mu[k]) * rs[k];
          }
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[0][threadIdx.x][k] = a[k], red[1][threadIdx.x][k] = b[k];
  __syncthreads();
  if (ry < 2 && c0 < C) {  // row lane 0 sums the `sum` partials, row lane 1 the second moment's
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float s = 0.f;
      for (int j = 0; j < nry; ++j) s += red[ry][j * ln.cl + cx][k];
      atomicAdd(ws + (long long)ry * C + c0 + k, (double)s);
    }
  }
}

// RES: y = relu?(bn(x) + resid) - the closing add (+ ReLU) of a residual block folded into the block's last batch norm.
// `relu` bit 0 = ReLU; bit 1 (RES only) = the residual joins AFTER the activation: y = relu?(bn(x)) + resid, the
// form of blocks whose last batch norm carries the ReLU and whose add is the block's output.
template <bool RES>
__global__ void __launch_bounds__(256)
bn_fwd_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ resid, bf16* __restrict__ yout, const bf16* __restrict__ gamma,
                    const bf16* __restrict__ beta, const double* __restrict__ ws, float* __restrict__ mean_o,
                    float* __restrict__ rstd_o, float* __restrict__ run_mean, float* __restrict__ run_var, long long M, int C,
                    long long rows_per_block, float eps, float momentum, int relu, int training) {
  const BnLane ln = bn_lane(C);
  const int ry = ln.ry, c0 = ln.c0, nry = ln.nry;
  if (c0 >= C) return;
  float sc[8], sh[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float mu, var;
    if (training) {
      const double m = ws[c0 + k] / (double)M;
      double v = ws[C + c0 + k] / (double)M - m * m;
      if (v < 0) v = 0;
      mu = (float)m;
      var = (float)v;
    } else {
      mu = run_mean[c0 + k];
      var = run_var[c0 + k];
    }
    const float rs = rsqrtf(var + eps);
    if (training && blockIdx.y == 0 && ry == 0) {
      mean_o[c0 + k] = mu;
      rstd_o[c0 + k] = rs;
      const float unb = M > 1 ? var * (float)((double)M / (double)(M - 1)) : var;
      run_mean[c0 + k] = (1.f - momentum) * run_mean[c0 + k] + momentum * mu;
      run_var[c0 + k] = (1.f - momentum) * run_var[c0 + k] + momentum * unb;
    }
    const float g = gamma ? __bfloat162float(gamma[c0 + k]) : 1.f;
    const float b = beta ? __bfloat162float(beta[c0 + k]) : 0.f;
    sc[k] = g * rs;
    sh[k] = b - mu * sc[k];
  }
  const long long r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  for (long long r = r0 + ry; r < r1; r += BN_U * nry) {
    uint4 xr[BN_U], rr4[RES ? BN_U : 1];
    bool ok[BN_U];
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const long long rr = r + (long long)u * nry;
      ok[u] = rr < r1 && TNNB_CHECK(rr * C + c0 + 7, M * (long long)C);  // lane layout vs. tensor extent
      xr[u] = make_uint4(0, 0, 0, 0);
      if (RES) rr4[RES ? u : 0] = make_uint4(0, 0, 0, 0);
      if (ok[u]) {
        xr[u] = *reinterpret_cast<const uint4*>(x + rr * C + c0);
        if (RES) rr4[RES ? u : 0] = *reinterpret_cast<const uint4*>(resid + rr * C + c0);
      }
    }
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const bf16* xv = reinterpret_cast<const bf16*>(&xr[u]);
      const bf16* rv = reinterpret_cast<const bf16*>(&rr4[RES ? u : 0]);
      __align__(16) bf16 o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float v = __bfloat162float(xv[k]) * sc[k] + sh[k];
        if (RES && !(relu & 2)) v = __bfloat162float(__float2bfloat16(v)) + __bfloat162float(rv[k]);  // the sum of two bf16 tensors, as a separate add would see it
        if (relu & 1) v = fmaxf(v, 0.f);
        if (RES && (relu & 2)) v = __bfloat162float(__float2bfloat16(v)) + __bfloat162float(rv[k]);
        o[k] = __float2bfloat16(v);
      }
      if (ok[u]) *reinterpret_cast<uint4*>(yout + (r + (long long)u * nry) * C + c0) = *reinterpret_cast<uint4*>(o);
    }
  }
}

template <int MASK>
__global__ void __launch_bounds__(256, 2)
bn_bwd_apply_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, const bf16* __restrict__ y,
                    const bf16* __restrict__ gamma, const bf16* __restrict__ beta, const float* __restrict__ mean,
                    const float* __restrict__ rstd,
                    const double* __restrict__ ws, bf16* __restrict__ dx, float* __restrict__ dgamma,
                    float* __restrict__ dbeta, long long M, int C, long long rows_per_block) {
  const BnLane ln = bn_lane(C);
  const int ry = ln.ry, c0 = ln.c0, nry = ln.nry;
  if (c0 >= C) return;
  float mu[8], rs[8], k1[8], sg[8], sgx[8], sc[8], sh[8];
  constexpr bool remask = MASK == 2, relu = MASK != 0;  // see bn_reduce_kernel
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    mu[k] = mean[c0 + k];
    rs[k] = rstd[c0 + k];
    sc[k] = (gamma ? __bfloat162float(gamma[c0 + k]) : 1.f) * rs[k];
    sh[k] = (beta ? __bfloat162float(beta[c0 + k]) : 0.f) - mu[k] * sc[k];
    sg[k] = (float)ws[c0 + k];
    sgx[k] = (float)ws[C + c0 + k];
    k1[k] = (gamma ? __bfloat162float(gamma[c0 + k]) : 1.f) * rs[k] / (float)M;
    if (blockIdx.y == 0 && ry == 0 && dgamma) {
      dgamma[c0 + k] += sgx[k];
      dbeta[c0 + k] += sg[k];
    }
  }
  const long long r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  for (long long r = r0 + ry; r < r1; r += BN_U * nry) {
    uint4 xr[BN_U], gr[BN_U], yr[MASK == 1 ? BN_U : 1];
    bool ok[BN_U];
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const long long rr = r + (long long)u * nry;
      ok[u] = rr < r1 && TNNB_CHECK(rr * C + c0 + 7, M * (long long)C);  // lane layout vs. tensor extent
      xr[u] = gr[u] = make_uint4(0, 0, 0, 0);
      if (MASK == 1) yr[MASK == 1 ? u : 0] = make_uint4(0, 0, 0, 0);
      if (ok[u]) {
        xr[u] = *reinterpret_cast<const uint4*>(x + rr * C + c0);
        gr[u] = *reinterpret_cast<const uint4*>(dy + rr * C + c0);
        if (MASK == 1) yr[MASK == 1 ? u : 0] = *reinterpret_cast<const uint4*>(y + rr * C + c0);
      }
    }
#pragma unroll
    for (int u = 0; u < BN_U; ++u) {
      const bf16* xv = reinterpret_cast<const bf16*>(&xr[u]);
      const bf16* gv = reinterpret_cast<const bf16*>(&gr[u]);
      const bf16* yv = reinterpret_cast<const bf16*>(&yr[MASK == 1 ? u : 0]);
      __align__(16) bf16 o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float g = __bfloat162float(gv[k]);
        const float xf = __bfloat162float(xv[k]);
        if (remask) {
          if (!(__bfloat162float(__float2bfloat16(xf * sc[k] + sh[k])) > 0.f)) g = 0.f;
        } else if (relu && !(__bfloat162float(yv[k]) > 0.f)) {
          g = 0.f;
        }
        const float xh = (xf - mu[k]) * rs[k];
        o[k] = __float2bfloat16(k1[k] * ((float)M * g - sg[k] - xh * sgx[k]));
      }
      if (ok[u]) *reinterpret_cast<uint4*>(dx + (r + (long long)u * nry) * C + c0) = *reinterpret_cast<uint4*>(o);
    }
  }
}

// per_sm: blocks per SM the grid is sized for. Every kernel here runs as a single wave of its resident block count
// (set by its registers): measured faster than several short waves, each of which ramps up and drains.
static void bn_grid(long long M, int C, dim3& grid, long long& rpb, int per_sm = 6) {
  const int cl = bn_cl(C);
  const int gx = ((C >> 3) + cl - 1) / cl;
  int gy = (per_sm * 148 + gx - 1) / gx;
  rpb = (M + gy - 1) / gy;
  const int nry = 256 / cl;
  if (rpb < 4 * nry) rpb = 4 * nry;
  gy = (int)((M + rpb - 1) / rpb);
  grid = dim3(gx, gy);
}

}  // namespace tnnb

using namespace tnnb;

extern "C" {

// ws: double[2*C] scratch owned by the caller (zeroed here). gamma/beta may be null.
static int bn_fwd_impl(const void* x, const void* resid, void* y, const void* gamma, const void* beta, void* ws, void* mean, void* rstd,
                       void* run_mean, void* run_var, long long M, int C, float eps, float momentum, int relu, int training,
                       void* stream) {
  if (C % 8 || ((uintptr_t)x & 15) || ((uintptr_t)y & 15) || ((uintptr_t)resid & 15)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid;
  long long rpb;
  bn_grid(M, C, grid, rpb, resid ? 3 : 4);  // one wave of the apply kernel's resident blocks (64 / 80 registers)
  if (training) {
    cudaMemsetAsync(ws, 0, sizeof(double) * 2 * C, st);
    dim3 rgrid;
    long long rrpb;
    bn_grid(M, C, rgrid, rrpb, 3);
    bn_reduce_kernel<false, 0><<<rgrid, 256, 0, st>>>((const bf16*)x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, (double*)ws, M, C, rrpb);
  }
  if (resid)
    bn_fwd_apply_kernel<true><<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)resid, (bf16*)y, (const bf16*)gamma, (const bf16*)beta,
                                                    (const double*)ws, (float*)mean, (float*)rstd, (float*)run_mean,
                                                    (float*)run_var, M, C, rpb, eps, momentum, relu, training);
  else
    bn_fwd_apply_kernel<false><<<grid, 256, 0, st>>>((const bf16*)x, nullptr, (bf16*)y, (const bf16*)gamma, (const bf16*)beta,
                                                     (const double*)ws, (float*)mean, (float*)rstd, (float*)run_mean,
                                                     (float*)run_var, M, C, rpb, eps, momentum, relu, training);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

int tnnb_batchnorm_fwd(const void* x, void* y, const void* gamma, const void* beta, void* ws, void* mean, void* rstd,
                       void* run_mean, void* run_var, long long M, int C, float eps, float momentum, int relu, int training,
                       void* stream) {
  return bn_fwd_impl(x, nullptr, y, gamma, beta, ws, mean, rstd, run_mean, run_var, M, C, eps, momentum, relu, training, stream);
}

// y = relu?(bn(x) + resid), or with relu bit 1 set y = relu?(bn(x)) + resid: resid has the shape of x (bf16,
// 16-byte aligned).
int tnnb_batchnorm_fwd_res(const void* x, const void* resid, void* y, const void* gamma, const void* beta, void* ws, void* mean,
                           void* rstd, void* run_mean, void* run_var, long long M, int C, float eps, float momentum, int relu,
                           int training, void* stream) {
  if (!resid) return -5;
  return bn_fwd_impl(x, resid, y, gamma, beta, ws, mean, rstd, run_mean, run_var, M, C, eps, momentum, relu, training, stream);
}

// Fused ReLU (relu != 0): with y == null the mask is recomputed from x, gamma, beta, mean and rstd (beta is read only
// then); with the saved forward output y it is y > 0. dgamma/dbeta (fp32) accumulate; may be null.
int tnnb_batchnorm_bwd(const void* x, const void* dy, const void* y, const void* gamma, const void* beta, const void* mean,
                       const void* rstd, void* ws, void* dx, void* dgamma, void* dbeta, long long M, int C, int relu,
                       void* stream) {
  if (C % 8 || ((uintptr_t)x & 15) || ((uintptr_t)dy & 15) || ((uintptr_t)dx & 15)) return -3;
  if (relu && !y && gamma && !beta) return -5;  // an affine layer's mask needs its shift
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid;
  long long rpb;
  bn_grid(M, C, grid, rpb, 2);
  cudaMemsetAsync(ws, 0, sizeof(double) * 2 * C, st);
  dim3 rgrid;
  long long rrpb;
  bn_grid(M, C, rgrid, rrpb, 2);
#define TNNB_BN_BWD(MASK)                                                                                              \
  do {                                                                                                                 \
    bn_reduce_kernel<true, MASK><<<rgrid, 256, 0, st>>>((const bf16*)x, (const bf16*)dy, (const bf16*)y, (const bf16*)gamma, \
                                                       (const bf16*)beta, (const float*)mean, (const float*)rstd,       \
                                                       (double*)ws, M, C, rrpb);                                        \
    bn_bwd_apply_kernel<MASK><<<grid, 256, 0, st>>>((const bf16*)x, (const bf16*)dy, (const bf16*)y, (const bf16*)gamma,  \
                                                    (const bf16*)beta, (const float*)mean, (const float*)rstd,          \
                                                    (const double*)ws, (bf16*)dx, (float*)dgamma, (float*)dbeta, M, C,  \
                                                    rpb);                                                               \
  } while (0)
  if (!relu) TNNB_BN_BWD(0);
  else if (y) TNNB_BN_BWD(1);
  else TNNB_BN_BWD(2);
#undef TNNB_BN_BWD
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free training-mode forward (declared in batchnorm_noalloc.h; no counterpart in the
// reference). Same kernels and launch shapes as tnnb_batchnorm_fwd; the only difference is where
// the per-channel partial sums live: in the fixed array below instead of a caller-supplied buffer.
// ---------------------------------------------------------------------------------------------
#include "batchnorm_noalloc.h"

static __device__ __align__(256) double g_bn_noalloc_scratch[2 * TNNB_BN_NOALLOC_MAX_CHANNELS];  // 64 KiB per device

namespace {
constexpr int kMaxDevices = 64;
double* g_bn_noalloc_ptr[kMaxDevices] = {};  // device address of the array above, per device ordinal
}

extern "C" {

int tnnb_batchnorm_fwd_noalloc(const void* x, void* y, const void* gamma, const void* beta, void* mean, void* rstd,
                               void* run_mean, void* run_var, long long M, int C, float eps, float momentum, int relu,
                               void* stream) {
  if (M <= 0 || C <= 0 || !x || !y || !mean || !rstd || !run_mean || !run_var) return TNNB_NOALLOC_BAD_ARG;
  if (C > TNNB_BN_NOALLOC_MAX_CHANNELS) return TNNB_NOALLOC_TOO_LARGE;
  if (C % 8 || ((uintptr_t)x & 15) || ((uintptr_t)y & 15)) return TNNB_NOALLOC_MISALIGNED;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TNNB_NOALLOC_SETUP_FAILED;
  if (!g_bn_noalloc_ptr[dev]) {  // first call on this device: look the array up once
    double* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_bn_noalloc_scratch) != cudaSuccess || !p) {
      (void)cudaGetLastError();
      return TNNB_NOALLOC_SETUP_FAILED;
    }
    g_bn_noalloc_ptr[dev] = p;
  }
  double* ws = g_bn_noalloc_ptr[dev];
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid;
  long long rpb;
  bn_grid(M, C, grid, rpb);
  // The reduce kernel accumulates with atomics, so the 2*C sums it uses must start at zero.
  if (cudaMemsetAsync(ws, 0, sizeof(double) * 2 * C, st) != cudaSuccess) return TNNB_NOALLOC_LAUNCH_FAILED;
  bn_reduce_kernel<false, 0><<<grid, 256, 0, st>>>((const bf16*)x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, ws, M, C, rpb);
  bn_fwd_apply_kernel<false><<<grid, 256, 0, st>>>((const bf16*)x, nullptr, (bf16*)y, (const bf16*)gamma, (const bf16*)beta, ws, (float*)mean,
                                            (float*)rstd, (float*)run_mean, (float*)run_var, M, C, rpb, eps, momentum, relu, 1);
  return cudaGetLastError() == cudaSuccess ? TNNB_NOALLOC_OK : TNNB_NOALLOC_LAUNCH_FAILED;
}

int tnnb_batchnorm_noalloc_max_channels(void) { return TNNB_BN_NOALLOC_MAX_CHANNELS; }

const char* tnnb_noalloc_strerror(int rc) {
  switch (rc) {
    case TNNB_NOALLOC_OK: return "ok";
    case TNNB_NOALLOC_BAD_ARG: return "null pointer or non-positive size";
    case TNNB_NOALLOC_TOO_LARGE: return "channel count exceeds TNNB_BN_NOALLOC_MAX_CHANNELS (4096): use tnnb_batchnorm_fwd with a caller-owned workspace";
    case TNNB_NOALLOC_MISALIGNED: return "channels must be a multiple of 8 and x/y 16-byte aligned";
    case TNNB_NOALLOC_SETUP_FAILED: return "could not obtain the address of the built-in scratch array on the current device";
    case TNNB_NOALLOC_LAUNCH_FAILED: return "memset or kernel launch failed";
    default: return "unknown code";
  }
}

}  // extern "C"
