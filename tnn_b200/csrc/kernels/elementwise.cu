// Bandwidth-bound element-wise kernels (bf16 I/O, fp32 math, 16-byte vectors):
// activations, binary ops, dropout with a regenerable counter-based mask,
// token+position embedding and its scatter-add gradient, bias-gradient column
// sums. They replace the reference's one-element-per-thread kernels
// (src/nn/activations_impl/cuda/*.cu, src/nn/engines/cudnn_engine.cu:31-50,
// 1077-1233, src/ops/cuda/kernels.cu:30-591).
#include "ptx.cuh"

TNNB_BOUNDS_TU(elementwise)

namespace tnnb {

typedef __nv_bfloat16 bf16;

struct alignas(16) Bf8 {
  bf16 v[8];
};

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  Bf8 r = *reinterpret_cast<const Bf8*>(p);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(r.v[i]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  Bf8 r;
#pragma unroll
  for (int i = 0; i < 8; ++i) r.v[i] = __float2bfloat16(f[i]);
  *reinterpret_cast<Bf8*>(p) = r;
}

enum ActKind { ACT_RELU = 0, ACT_GELU = 1, ACT_ELU = 2, ACT_LEAKY = 3, ACT_SIGMOID = 4, ACT_TANH = 5, ACT_LINEAR = 6 };

__device__ __forceinline__ float act_fwd(int kind, float x, float alpha) {
  switch (kind) {
    case ACT_RELU: return fmaxf(x, 0.f);
    case ACT_GELU: return gelu_tanh(x);
    case ACT_ELU: return x > 0.f ? x : alpha * (__expf(x) - 1.f);
    case ACT_LEAKY: return x > 0.f ? x : alpha * x;
    case ACT_SIGMOID: return 1.f / (1.f + __expf(-x));
    case ACT_TANH: return tanhf(x);
    default: return x;
  }
}
// Derivative with respect to the input x (the saved tensor is the input).
__device__ __forceinline__ float act_bwd(int kind, float x, float alpha) {
  switch (kind) {
    case ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case ACT_GELU: return gelu_tanh_grad(x);
    case ACT_ELU: return x > 0.f ? 1.f : alpha * __expf(x);
    case ACT_LEAKY: return x > 0.f ? 1.f : alpha;
    case ACT_SIGMOID: {
      float s = 1.f / (1.f + __expf(-x));
      return s * (1.f - s);
    }
    case ACT_TANH: {
      float t = tanhf(x);
      return 1.f - t * t;
    }
    default: return 1.f;
  }
}

__global__ void act_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n, int kind,
                               float alpha) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    float f[8];
    load8(x + i, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = act_fwd(kind, f[k], alpha);
    store8(y + i, f);
  }
  if (i < n && i + 8 > n)
    for (long long j = i; j < n; ++j) y[j] = __float2bfloat16(act_fwd(kind, __bfloat162float(x[j]), alpha));
}

__global__ void act_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                               bf16* __restrict__ dx, long long n, int kind, float alpha) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    float f[8], g[8];
    load8(x + i, f);
    load8(dy + i, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] *= act_bwd(kind, f[k], alpha);
    store8(dx + i, g);
  }
  if (i < n && i + 8 > n)
    for (long long j = i; j < n; ++j)
      dx[j] = __float2bfloat16(__bfloat162float(dy[j]) * act_bwd(kind, __bfloat162float(x[j]), alpha));
}

// out = a (op) b, op: 0 add, 1 sub, 2 mul, 3 div.  relu!=0 applies max(.,0).
__global__ void binary_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                              bf16* __restrict__ o, long long n, int op, int relu) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    float f[8], g[8];
    load8(a + i, f);
    load8(b + i, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float r = op == 0 ? f[k] + g[k] : op == 1 ? f[k] - g[k] : op == 2 ? f[k] * g[k] : f[k] / g[k];
      f[k] = relu ? fmaxf(r, 0.f) : r;
    }
    store8(o + i, f);
  }
  if (i < n && i + 8 > n)
    for (long long j = i; j < n; ++j) {
      float x = __bfloat162float(a[j]), y = __bfloat162float(b[j]);
      float r = op == 0 ? x + y : op == 1 ? x - y : op == 2 ? x * y : x / y;
      o[j] = __float2bfloat16(relu ? fmaxf(r, 0.f) : r);
    }
}

// y = keep ? x / (1-p) : 0, keep regenerated from (seed, element index).
__global__ void dropout_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n, float p,
                               unsigned long long seed, const unsigned long long* __restrict__ seed_off) {
  seed = mix_seed(seed, seed_off);
  const float inv = 1.f / (1.f - p);
  const uint32_t thr = dropout_threshold(p);
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 8;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (; i + 8 <= n; i += stride) {
    float f[8];
    load8(x + i, f);
    const uint32_t keep = dropout_keep8(seed, (uint64_t)(i >> 3), thr);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = (keep >> k) & 1u ? f[k] * inv : 0.f;
    store8(y + i, f);
  }
  if (i < n && i + 8 > n) {
    const uint32_t keep = dropout_keep8(seed, (uint64_t)(i >> 3), thr);
    for (long long j = i; j < n; ++j)
      y[j] = __float2bfloat16((keep >> (int)(j - i)) & 1u ? __bfloat162float(x[j]) * inv : 0.f);
  }
}

// out[r, :] = wte[clamp(id[r])] (+ wpe[r % S]) then optional dropout.
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ wte,
                                     const bf16* __restrict__ wpe, bf16* __restrict__ out,
                                     long long rows, int E, int S, long long vocab,
                                     long long padding_idx, float p, unsigned long long seed,
                                     const unsigned long long* __restrict__ seed_off) {
  seed = mix_seed(seed, seed_off);
  const int chunks = E / 8;
  const float inv = 1.f / (1.f - p);
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    long long id = ids[r];
    const bool pad = (id == padding_idx);
    if (!pad) (void)TNNB_CHECK(id, vocab);  // checked build: report the id; both builds read row 0 instead
    if (id < 0 || id >= vocab) id = 0;
    const bf16* trow = wte + id * E;
    const bf16* prow = wpe ? wpe + (long long)(r % S) * E : nullptr;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
      float f[8], g[8];
      load8(trow + c * 8, f);
      if (pad)
        for (int k = 0; k < 8; ++k) f[k] = 0.f;
      if (prow) {
        load8(prow + c * 8, g);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] += g[k];
      }
      if (p > 0.f) {
        const uint32_t keep = dropout_keep8(seed, (uint64_t)(r * chunks + c), dropout_threshold(p));
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = (keep >> k) & 1u ? f[k] * inv : 0.f;
      }
      store8(out + r * E + c * 8, f);
    }
  }
}

// dwte[id[r]] += dropout'(dy[r]);  dwpe[r % S] += dropout'(dy[r])  (fp32 atomics)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ dy,
                                     float* __restrict__ dwte, float* __restrict__ dwpe,
                                     long long rows, int E, int S, long long vocab,
                                     long long padding_idx, float p, unsigned long long seed,
                                     const unsigned long long* __restrict__ seed_off) {
  seed = mix_seed(seed, seed_off);
  const int chunks = E / 8;
  const float inv = 1.f / (1.f - p);
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    long long id = ids[r];
    const bool pad = (id == padding_idx);
    if (!pad) (void)TNNB_CHECK(id, vocab);
    if (id < 0 || id >= vocab) id = 0;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
      float g[8];
      load8(dy + r * E + c * 8, g);
      if (p > 0.f) {
        const uint32_t keep = dropout_keep8(seed, (uint64_t)(r * chunks + c), dropout_threshold(p));
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = (keep >> k) & 1u ? g[k] * inv : 0.f;
      }
      if (!pad && dwte) {
        float* d = dwte + id * E + c * 8;
        asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(d), "f"(g[0]), "f"(g[1]), "f"(g[2]), "f"(g[3]) : "memory");
        asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(d + 4), "f"(g[4]), "f"(g[5]), "f"(g[6]), "f"(g[7]) : "memory");
      }
      if (dwpe) {
        float* d = dwpe + (long long)(r % S) * E + c * 8;
        asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(d), "f"(g[0]), "f"(g[1]), "f"(g[2]), "f"(g[3]) : "memory");
        asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(d + 4), "f"(g[4]), "f"(g[5]), "f"(g[6]), "f"(g[7]) : "memory");
      }
    }
  }
}

// db[n] += sum_m dy[m, n].  Block = 8 column-chunks (64 columns, one 128-byte line per row) x 32 row
// lanes, four independent 16-byte loads in flight per thread; narrow column tiles give enough blocks
// to fill the GPU while keeping the number of atomic adds per output element small.
__global__ void __launch_bounds__(256)
colsum_kernel(const bf16* __restrict__ dy, long long ld, float* __restrict__ db, long long M, int N, int rows_per_block) {
  __shared__ float red[32][8][9];
  const int cx = threadIdx.x, ry = threadIdx.y;
  const int col = (blockIdx.x * 8 + cx) * 8;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = min(M, r0 + rows_per_block);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col + 8 <= N && (ld % 8 == 0) && (reinterpret_cast<uintptr_t>(dy) & 15) == 0) {  // 16-byte row loads need both
    long long r = r0 + ry;
    for (; r + 96 < r1; r += 128) {
      float f0[8], f1[8], f2[8], f3[8];
      load8(dy + r * ld + col, f0);
      load8(dy + (r + 32) * ld + col, f1);
      load8(dy + (r + 64) * ld + col, f2);
      load8(dy + (r + 96) * ld + col, f3);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += (f0[k] + f1[k]) + (f2[k] + f3[k]);
    }
    for (; r < r1; r += 32) {
      float f[8];
      load8(dy + r * ld + col, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
  } else if (col < N) {
    for (long long r = r0 + ry; r < r1; r += 32)
      for (int k = 0; k < 8 && col + k < N; ++k) acc[k] += __bfloat162float(dy[r * ld + col + k]);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[ry][cx][k] = acc[k];
  __syncthreads();
  const int t = ry * 8 + cx;
  if (t < 64) {  // one thread per column of the tile
    const int c = t >> 3, k = t & 7;
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) s += red[j][c][k];
    const int oc = (blockIdx.x * 8 + c) * 8 + k;
    if (oc < N) atomicAdd(db + oc, s);
  }
}

// dst(bf16) = src(fp32) and back; used for parameter casts of flat buffers.
__global__ void cast_f32_bf16_kernel(const float* __restrict__ s, bf16* __restrict__ d, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) d[i] = __float2bfloat16(s[i]);
}

static inline int grid_for(long long n, int per_thread, int block) {
  long long g = (n + (long long)per_thread * block - 1) / ((long long)per_thread * block);
  long long cap = 148ll * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

// ------------------------------------------------------------------ row softmax of attention scores
// For head sizes the flash kernels do not cover, attention runs as batched GEMMs with the scores materialised
// (ops/raw.py): these two kernels are the softmax between the products. One warp per score row.
//   forward   x = s * scale (masked above the diagonal when causal);  P = softmax(x) as bf16;
//             lse2 = log2 of the row's sum of exp(x)  (the unit the flash kernels use)
//   backward  p = exp2(x * log2e - lse2);  P = p as bf16;  dS = p * (dP - delta) * scale as bf16
__global__ void __launch_bounds__(256)
attn_softmax_fwd_kernel(const float* __restrict__ S, bf16* __restrict__ P, float* __restrict__ lse2, long long rows, int Sq,
                        int Sk, long long ld, float scale, int causal) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    const int qi = (int)(r % Sq);
    const int lim = causal ? min(Sk, qi + 1) : Sk;  // keys [0, lim) take part
    const float* s = S + r * ld;
    float m = -INFINITY;
    for (int k = lane; k < lim; k += 32) m = fmaxf(m, s[k] * scale);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
    for (int k = lane; k < lim; k += 32) sum += __expf(s[k] * scale - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    bf16* p = P + r * ld;
    for (int k = lane; k < Sk; k += 32) p[k] = __float2bfloat16(k < lim ? __expf(s[k] * scale - m) * inv : 0.f);
    if (lane == 0) lse2[r] = (m + __logf(sum)) * 1.4426950408889634f;
  }
}

__global__ void __launch_bounds__(256)
attn_softmax_bwd_kernel(const float* __restrict__ S, const float* __restrict__ dP, const float* __restrict__ lse2,
                        const float* __restrict__ delta, bf16* __restrict__ P, bf16* __restrict__ dS, long long rows, int Sq,
                        int Sk, long long ld, float scale, int causal) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    const int qi = (int)(r % Sq);
    const int lim = causal ? min(Sk, qi + 1) : Sk;
    const float l2 = lse2[r], dl = delta[r];
    const float c = scale * 1.4426950408889634f;
    for (int k = lane; k < Sk; k += 32) {
      const float pv = k < lim ? exp2f(S[r * ld + k] * c - l2) : 0.f;
      P[r * ld + k] = __float2bfloat16(pv);
      dS[r * ld + k] = __float2bfloat16(pv * (dP[r * ld + k] - dl) * scale);
    }
  }
}

}  // namespace tnnb

using namespace tnnb;

#define LAUNCH_RC()                                         \
  do {                                                      \
    cudaError_t e__ = cudaGetLastError();                   \
    return e__ == cudaSuccess ? 0 : -(int)e__ - 1000;       \
  } while (0)

extern "C" {

int tnnb_act_fwd(const void* x, void* y, long long n, int kind, float alpha, void* stream) {
  if (((uintptr_t)x | (uintptr_t)y) & 15) return -4;
  act_fwd_kernel<<<grid_for(n, 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n, kind, alpha);
  LAUNCH_RC();
}
int tnnb_act_bwd(const void* x, const void* dy, void* dx, long long n, int kind, float alpha, void* stream) {
  if (((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) & 15) return -4;
  act_bwd_kernel<<<grid_for(n, 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)dy, (bf16*)dx, n, kind, alpha);
  LAUNCH_RC();
}
int tnnb_binary(const void* a, const void* b, void* o, long long n, int op, int relu, void* stream) {
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)o) & 15) return -4;
  binary_kernel<<<grid_for(n, 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)a, (const bf16*)b, (bf16*)o, n, op, relu);
  LAUNCH_RC();
}
int tnnb_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, const void* seed_off,
                 void* stream) {
  if (((uintptr_t)x | (uintptr_t)y) & 15) return -4;
  if (p < 0.f || p >= 1.f) return -2;
  dropout_kernel<<<grid_for(n, 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n, p, seed,
                                                                        (const unsigned long long*)seed_off);
  LAUNCH_RC();
}
int tnnb_embedding_fwd(const void* ids, const void* wte, const void* wpe, void* out, long long rows, int E,
                       int S, long long vocab, long long padding_idx, float p, unsigned long long seed,
                       const void* seed_off, void* stream) {
  if (E % 8) return -3;
  int grid = (int)(rows < 148 * 8 ? rows : 148 * 8);
  embedding_fwd_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const long long*)ids, (const bf16*)wte, (const bf16*)wpe,
                                                              (bf16*)out, rows, E, S, vocab, padding_idx, p, seed,
                                                              (const unsigned long long*)seed_off);
  LAUNCH_RC();
}
int tnnb_embedding_bwd(const void* ids, const void* dy, void* dwte, void* dwpe, long long rows, int E, int S,
                       long long vocab, long long padding_idx, float p, unsigned long long seed, const void* seed_off,
                       void* stream) {
  if (E % 8) return -3;
  int grid = (int)(rows < 148 * 8 ? rows : 148 * 8);
  embedding_bwd_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((const long long*)ids, (const bf16*)dy, (float*)dwte,
                                                              (float*)dwpe, rows, E, S, vocab, padding_idx, p, seed,
                                                              (const unsigned long long*)seed_off);
  LAUNCH_RC();
}
int tnnb_colsum_accum(const void* dy, long long ld, void* db, long long M, int N, void* stream) {
  const int gx = (N + 63) / 64;
  int want_y = (4 * 148 + gx - 1) / gx;
  if (want_y > 64) want_y = 64;  // at most 64 atomic adds per output element
  long long rpb = (M + want_y - 1) / want_y;
  rpb = (rpb + 127) / 128 * 128;
  const int gy = (int)((M + rpb - 1) / rpb);
  colsum_kernel<<<dim3(gx, gy), dim3(8, 32), 0, (cudaStream_t)stream>>>((const bf16*)dy, ld, (float*)db, M, N, (int)rpb);
  LAUNCH_RC();
}
// Scores S and outputs P (and dS) are [rows, ld] with rows = batch * Sq consecutive query rows, Sk valid columns.
int tnnb_attn_softmax_fwd(const void* S, void* P, void* lse2, long long rows, int Sq, int Sk, long long ld, float scale,
                          int causal, void* stream) {
  if (rows <= 0 || Sq <= 0 || Sk <= 0 || ld < Sk) return -3;
  const long long g = (rows + 7) / 8;
  attn_softmax_fwd_kernel<<<(int)(g > 148 * 16 ? 148 * 16 : g), 256, 0, (cudaStream_t)stream>>>(
      (const float*)S, (bf16*)P, (float*)lse2, rows, Sq, Sk, ld, scale, causal);
  LAUNCH_RC();
}
int tnnb_attn_softmax_bwd(const void* S, const void* dP, const void* lse2, const void* delta, void* P, void* dS, long long rows,
                          int Sq, int Sk, long long ld, float scale, int causal, void* stream) {
  if (rows <= 0 || Sq <= 0 || Sk <= 0 || ld < Sk) return -3;
  const long long g = (rows + 7) / 8;
  attn_softmax_bwd_kernel<<<(int)(g > 148 * 16 ? 148 * 16 : g), 256, 0, (cudaStream_t)stream>>>(
      (const float*)S, (const float*)dP, (const float*)lse2, (const float*)delta, (bf16*)P, (bf16*)dS, rows, Sq, Sk, ld, scale,
      causal);
  LAUNCH_RC();
}
int tnnb_cast_f32_bf16(const void* s, void* d, long long n, void* stream) {
  cast_f32_bf16_kernel<<<grid_for(n, 4, 256), 256, 0, (cudaStream_t)stream>>>((const float*)s, (bf16*)d, n);
  LAUNCH_RC();
}

}  // extern "C"
