// NHWC convolution support kernels and pooling.
//
// Convolutions run on the tcgen05 GEMM (gemm_tcgen05.cu): 1x1 / stride-1 layers are
// a GEMM over the activation tensor as it is; every other geometry goes through
// the patch matrices built here:
//   im2col   cols[(n,oh,ow), (kh,kw,c)] = x[n, oh*s+kh-p, ow*s+kw-p, c]  (0 outside)
//   col2im   dx[n,h,w,c] = sum over the taps (kh,kw) that read pixel (h,w) of
//            dcols[(n,oh,ow),(kh,kw,c)]   - a gather, so no atomics
// Weights [O,KH,KW,C] are already the [O, K] operand of that GEMM.
// Semantics follow the reference CPU engine (src/nn/engines/cpu_engine.cpp:617-734,
// pools :66-210; average pooling divides by the in-image count as in
// src/nn/engines/cuda_engine.cu:141-194). The reference calls cuDNN conv graphs
// (cudnn_engine.cu:328-578) and scatter kernels with atomics for the pool backward.
#include "ptx.cuh"

TNNB_BOUNDS_TU(conv_pool)

namespace tnnb {

typedef __nv_bfloat16 bf16;

struct ConvGeo {
  int N, H, W, C, KH, KW, SH, SW, PH, PW, OH, OW;
  int Kld;  // row pitch of the patch matrix in elements (>= KH*KW*C, multiple of 8)
};

// VEC = 8: C % 8 == 0, one 16-byte move per thread. VEC = 1 (any C, e.g. the 3-channel stem): each thread still
// writes one 16-byte group of eight consecutive columns of the row (Kld % 8 == 0), gathering its eight elements
// with scalar loads - the write side, which is the larger one, stays coalesced.
template <int VEC>
__global__ void im2col_kernel(const bf16* __restrict__ x, bf16* __restrict__ cols, ConvGeo g) {
  if (VEC == 8) {
    const int cv = g.C / 8;
    const long long per_row = (long long)g.KH * g.KW * cv;
    const long long total = (long long)g.N * g.OH * g.OW * per_row;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const int c = (int)(i % cv);
      long long r = i / cv;
      const int kw = (int)(r % g.KW); r /= g.KW;
      const int kh = (int)(r % g.KH); r /= g.KH;
      const long long pix = r;  // (n, oh, ow)
      const int ow = (int)(pix % g.OW);
      const int oh = (int)((pix / g.OW) % g.OH);
      const int n = (int)(pix / ((long long)g.OW * g.OH));
      const int ih = oh * g.SH + kh - g.PH, iw = ow * g.SW + kw - g.PW;
      const long long doff = pix * g.Kld + ((long long)(kh * g.KW + kw) * g.C) + c * 8;
      if (!TNNB_CHECK(doff + 7, (long long)g.N * g.OH * g.OW * g.Kld)) continue;
      bf16* dst = cols + doff;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) {
        const long long soff = (((long long)n * g.H + ih) * g.W + iw) * g.C + c * 8;
        if (TNNB_CHECK(soff + 7, (long long)g.N * g.H * g.W * g.C)) v = *reinterpret_cast<const uint4*>(x + soff);
      }
      *reinterpret_cast<uint4*>(dst) = v;
    }
  } else {
    const int K = g.KH * g.KW * g.C;
    const int groups = g.Kld / 8;  // 16-byte groups per row, padding columns included (written as zeros)
    const long long total = (long long)g.N * g.OH * g.OW * groups;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const int gi = (int)(i % groups);
      const long long pix = i / groups;
      const int ow = (int)(pix % g.OW);
      const int oh = (int)((pix / g.OW) % g.OH);
      const int n = (int)(pix / ((long long)g.OW * g.OH));
      const bf16* img = x + (long long)n * g.H * g.W * g.C;
      __align__(16) bf16 v[8];
      // In NHWC the (kw, c) run of one filter row is contiguous in the image, so a column index k = kh * KW*C + kp
      // maps to img[(ih * W + iw0) * C + kp]; the horizontal bounds become a range of kp. One division per thread
      // instead of six per element - with three channels this kernel is bound by integer arithmetic, not by memory.
      const int kwc = g.KW * g.C;
      const int ih0 = oh * g.SH - g.PH, iw0 = ow * g.SW - g.PW;
      const int lo = (iw0 < 0 ? -iw0 : 0) * g.C;
      const int hi = (g.W - iw0 < g.KW ? g.W - iw0 : g.KW) * g.C;
      int kh = (gi * 8) / kwc;
      int kp = gi * 8 - kh * kwc;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        bf16 e = __float2bfloat16(0.f);
        const int ih = ih0 + kh;
        if (gi * 8 + j < K && ih >= 0 && ih < g.H && kp >= lo && kp < hi) {
          const long long off = ((long long)ih * g.W + iw0) * g.C + kp;
          if (TNNB_CHECK(off, (long long)g.H * g.W * g.C)) e = img[off];
        }
        v[j] = e;
        if (++kp == kwc) {
          kp = 0;
          ++kh;
        }
      }
      *reinterpret_cast<uint4*>(cols + pix * g.Kld + gi * 8) = *reinterpret_cast<const uint4*>(v);
    }
  }
}

template <int VEC>
__global__ void col2im_kernel(const bf16* __restrict__ dcols, bf16* __restrict__ dx, ConvGeo g) {
  const int cv = g.C / VEC;
  const long long total = (long long)g.N * g.H * g.W * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv);
    long long r = i / cv;
    const int w = (int)(r % g.W); r /= g.W;
    const int h = (int)(r % g.H);
    const int n = (int)(r / g.H);
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
    // the output pixels whose window covers (h, w), as index ranges (two divisions per axis, see pool_bwd_kernel)
    const int th = h + g.PH, tw = w + g.PW;
    const int oh_hi = min(th / g.SH, g.OH - 1), ow_hi = min(tw / g.SW, g.OW - 1);
    const int oh_lo = th - g.KH + 1 > 0 ? (th - g.KH + g.SH) / g.SH : 0;
    const int ow_lo = tw - g.KW + 1 > 0 ? (tw - g.KW + g.SW) / g.SW : 0;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      const int kh = th - oh * g.SH;
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const int kw = tw - ow * g.SW;
        const long long soff = (((long long)n * g.OH + oh) * g.OW + ow) * g.Kld + (long long)(kh * g.KW + kw) * g.C + c * VEC;
        if (!TNNB_CHECK(soff + VEC - 1, (long long)g.N * g.OH * g.OW * g.Kld)) continue;
        const bf16* src = dcols + soff;
        if (VEC == 8) {
          uint4 raw = *reinterpret_cast<const uint4*>(src);
          const bf16* t8 = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += __bfloat162float(t8[k]);
        } else {
          acc[0] += __bfloat162float(*src);
        }
      }
    }
    bf16* dst = dx + i * VEC;
    if (VEC == 8) {
      __align__(16) bf16 o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = __float2bfloat16(acc[k]);
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(o);
    } else {
      *dst = __float2bfloat16(acc[0]);
    }
  }
}

// mode 0: max (window clipped to the image, uint8 window-relative argmax saved), 1: average over
// the in-image elements. One thread per (n, oh, ow, 8 channels).
__global__ void pool_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, unsigned char* __restrict__ idx,
                                ConvGeo g, int mode) {
  const int cv = g.C / 8;
  const long long total = (long long)g.N * g.OH * g.OW * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv);
    long long r = i / cv;
    const int ow = (int)(r % g.OW); r /= g.OW;
    const int oh = (int)(r % g.OH);
    const int n = (int)(r / g.OH);
    float best[8], sum[8];
    unsigned char bi[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) best[k] = -INFINITY, sum[k] = 0.f, bi[k] = 255;
    int cnt = 0;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int ih = oh * g.SH + kh - g.PH;
      if (ih < 0 || ih >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int iw = ow * g.SW + kw - g.PW;
        if (iw < 0 || iw >= g.W) continue;
        uint4 raw = *reinterpret_cast<const uint4*>(x + (((long long)n * g.H + ih) * g.W + iw) * g.C + c * 8);
        const bf16* t8 = reinterpret_cast<const bf16*>(&raw);
        ++cnt;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float v = __bfloat162float(t8[k]);
          sum[k] += v;
          if (v > best[k]) best[k] = v, bi[k] = (unsigned char)(kh * g.KW + kw);
        }
      }
    }
    __align__(16) bf16 o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      o[k] = __float2bfloat16(mode == 0 ? (bi[k] != 255 ? best[k] : 0.f) : (cnt ? sum[k] / cnt : 0.f));
    *reinterpret_cast<uint4*>(y + i * 8) = *reinterpret_cast<uint4*>(o);
    if (mode == 0 && idx) *reinterpret_cast<uint2*>(idx + i * 8) = *reinterpret_cast<uint2*>(bi);
  }
}

// Gather form of the pool backward: every input pixel sums the outputs whose window covers it
// (max: only where the saved argmax points back at it; average: dy / in-image count).
__global__ void pool_bwd_kernel(const bf16* __restrict__ dy, const unsigned char* __restrict__ idx, bf16* __restrict__ dx,
                                ConvGeo g, int mode) {
  const int cv = g.C / 8;
  const long long total = (long long)g.N * g.H * g.W * cv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % cv);
    long long r = i / cv;
    const int w = (int)(r % g.W); r /= g.W;
    const int h = (int)(r % g.H);
    const int n = (int)(r / g.H);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // Output rows whose window covers input row h: oh * SH - PH <= h < oh * SH - PH + KH. The range is computed with
    // two divisions per axis instead of a divisibility test per filter tap (the kernel was bound by integer
    // arithmetic, not by memory).
    const int th = h + g.PH, tw = w + g.PW;
    const int oh_hi = min(th / g.SH, g.OH - 1), ow_hi = min(tw / g.SW, g.OW - 1);
    const int oh_lo = th - g.KH + 1 > 0 ? (th - g.KH + g.SH) / g.SH : 0;
    const int ow_lo = tw - g.KW + 1 > 0 ? (tw - g.KW + g.SW) / g.SW : 0;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      const int kh = th - oh * g.SH;
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const int kw = tw - ow * g.SW;
        const long long o = ((((long long)n * g.OH + oh) * g.OW + ow) * cv + c) * 8;
        if (!TNNB_CHECK(o + 7, (long long)g.N * g.OH * g.OW * g.C)) continue;
        uint4 raw = *reinterpret_cast<const uint4*>(dy + o);
        const bf16* t8 = reinterpret_cast<const bf16*>(&raw);
        if (mode == 0) {
          uint2 ir = *reinterpret_cast<const uint2*>(idx + o);
          const unsigned char* b8 = reinterpret_cast<const unsigned char*>(&ir);
          const unsigned char me = (unsigned char)(kh * g.KW + kw);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (b8[k] != 255) (void)TNNB_CHECK(b8[k], g.KH * g.KW);  // a saved position outside the window (255 = empty window)
            if (b8[k] == me) acc[k] += __bfloat162float(t8[k]);
          }
        } else {
          const int h0 = max(oh * g.SH - g.PH, 0), h1 = min(oh * g.SH - g.PH + g.KH, g.H);
          const int w0 = max(ow * g.SW - g.PW, 0), w1 = min(ow * g.SW - g.PW + g.KW, g.W);
          const float inv = 1.f / (float)max((h1 - h0) * (w1 - w0), 1);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += __bfloat162float(t8[k]) * inv;
        }
      }
    }
    __align__(16) bf16 o8[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) o8[k] = __float2bfloat16(acc[k]);
    *reinterpret_cast<uint4*>(dx + i * 8) = *reinterpret_cast<uint4*>(o8);
  }
}

static inline int grid1d(long long n, int block) {
  long long g = (n + block - 1) / block;
  const long long cap = 148ll * 32;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace tnnb

using namespace tnnb;

static ConvGeo make_geo(int N, int H, int W, int C, int KH, int KW, int SH, int SW, int PH, int PW, int Kld) {
  ConvGeo g{N, H, W, C, KH, KW, SH, SW, PH, PW, (H + 2 * PH - KH) / SH + 1, (W + 2 * PW - KW) / SW + 1, Kld};
  return g;
}

#define RC_LAST()                                       \
  do {                                                  \
    cudaError_t e__ = cudaGetLastError();               \
    return e__ == cudaSuccess ? 0 : -(int)e__ - 1000;   \
  } while (0)

extern "C" {

// cols: [N*OH*OW, Kld] bf16; columns >= KH*KW*C (padding of the pitch) are left untouched.
int tnnb_im2col(const void* x, void* cols, int N, int H, int W, int C, int KH, int KW, int SH, int SW, int PH, int PW,
                int Kld, void* stream) {
  ConvGeo g = make_geo(N, H, W, C, KH, KW, SH, SW, PH, PW, Kld);
  if (g.OH <= 0 || g.OW <= 0 || Kld < KH * KW * C) return -2;
  if (Kld % 8 || ((uintptr_t)cols & 15)) return -3;
  const bool vec = (C % 8 == 0) && !((uintptr_t)x & 15);
  const long long total = (long long)N * g.OH * g.OW * (vec ? (long long)KH * KW * (C / 8) : Kld / 8);
  if (vec) im2col_kernel<8><<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)cols, g);
  else im2col_kernel<1><<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)cols, g);
  RC_LAST();
}

int tnnb_col2im(const void* dcols, void* dx, int N, int H, int W, int C, int KH, int KW, int SH, int SW, int PH, int PW,
                int Kld, void* stream) {
  ConvGeo g = make_geo(N, H, W, C, KH, KW, SH, SW, PH, PW, Kld);
  if (g.OH <= 0 || g.OW <= 0) return -2;
  const bool vec = (C % 8 == 0) && (Kld % 8 == 0) && !(((uintptr_t)dx | (uintptr_t)dcols) & 15);
  const long long total = (long long)N * H * W * (vec ? C / 8 : C);
  if (vec) col2im_kernel<8><<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)dcols, (bf16*)dx, g);
  else col2im_kernel<1><<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)dcols, (bf16*)dx, g);
  RC_LAST();
}

// C % 8 == 0 and pool windows of at most 255 elements. idx (uint8, same shape as y) may be null.
int tnnb_pool_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, int KH, int KW, int SH, int SW, int PH,
                  int PW, int mode, void* stream) {
  if (C % 8 || KH * KW > 254) return -3;
  ConvGeo g = make_geo(N, H, W, C, KH, KW, SH, SW, PH, PW, 0);
  const long long total = (long long)N * g.OH * g.OW * (C / 8);
  pool_fwd_kernel<<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, (unsigned char*)idx, g, mode);
  RC_LAST();
}

int tnnb_pool_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int KH, int KW, int SH, int SW,
                  int PH, int PW, int mode, void* stream) {
  if (C % 8) return -3;
  ConvGeo g = make_geo(N, H, W, C, KH, KW, SH, SW, PH, PW, 0);
  const long long total = (long long)N * H * W * (C / 8);
  pool_bwd_kernel<<<grid1d(total, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const unsigned char*)idx, (bf16*)dx, g, mode);
  RC_LAST();
}

}  // extern "C"
