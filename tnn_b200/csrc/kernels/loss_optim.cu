// Softmax cross-entropy (forward + gradient + argmax-correct count in one pass
// over the logits, no host synchronisation) and flat-buffer optimizer updates.
//
// Loss semantics follow the reference (src/nn/loss_impl/cuda/loss_ops.cu:75-192):
// per row loss = log sum exp(z - max) + max - z[label], averaged over rows;
// gradient (softmax - onehot) * scale. The reference runs two kernels plus a
// two-stage reduction and a blocking device-to-host copy of the scalar.
//
// Optimizer semantics follow src/nn/optimizers_impl/cuda/{adam,sgd}_kernels.cu:
// SGD momentum v = mu*v - lr*g, p += v; Adam with bias correction and
// p -= lr*m^/(sqrt(v^)+eps) + wd*lr*p. The reference launches one kernel per
// tensor; here one launch covers the whole flat parameter buffer, keeps fp32
// master weights and writes the bf16 compute copy in the same pass.
#include "ptx.cuh"

namespace tnnb {

typedef __nv_bfloat16 bf16;
struct alignas(16) CBf8 {
  bf16 v[8];
};

__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  v = l < nw ? sh[l] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  v = l < nw ? sh[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One CTA per row; the row lives in registers (MAXCH chunks of 8 per thread).
// grad may alias logits (in-place). ld is the row pitch in elements (% 8 == 0).
template <int MAXCH, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_ce_kernel(const bf16* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                  bf16* grad, long long ldg, float* __restrict__ row_loss, float* __restrict__ loss_sum,
                  int* __restrict__ corrects, long long rows, int V, float grad_scale, float loss_scale) {
  __shared__ float sh[32];
  __shared__ int sh_arg[32];
  const int chunks = (V + 7) >> 3;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const bf16* z = logits + r * ld;
    float v[MAXCH][8];
    float mx = -INFINITY;
    int arg = 0;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < chunks) {
        CBf8 a = *reinterpret_cast<const CBf8*>(z + c * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int col = c * 8 + k;
          v[i][k] = col < V ? __bfloat162float(a.v[k]) : -INFINITY;
          if (v[i][k] > mx) {
            mx = v[i][k];
            arg = col;
          }
        }
      }
    }
    // arg-max across the block (lowest index wins ties, like a serial scan)
    float m2 = mx;
    int a2 = arg;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m2, o);
      int oa = __shfl_xor_sync(0xffffffffu, a2, o);
      if (om > m2 || (om == m2 && oa < a2)) {
        m2 = om;
        a2 = oa;
      }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) {
      sh[w] = m2;
      sh_arg[w] = a2;
    }
    __syncthreads();
    m2 = l < THREADS / 32 ? sh[l] : -INFINITY;
    a2 = l < THREADS / 32 ? sh_arg[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m2, o);
      int oa = __shfl_xor_sync(0xffffffffu, a2, o);
      if (om > m2 || (om == m2 && oa < a2)) {
        m2 = om;
        a2 = oa;
      }
    }
    const float rmax = m2;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXCH; ++i) {
      if (threadIdx.x + i * THREADS < chunks) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[i][k] = __expf(v[i][k] - rmax);
          s += v[i][k];
        }
      }
    }
    s = block_reduce_sum(s, sh);
    const long long lab = labels[r];
    const float inv = 1.f / s;
    if (threadIdx.x == 0) {
      float zl = (lab >= 0 && lab < V) ? __bfloat162float(z[lab]) : rmax;
      float loss = __logf(s) + rmax - zl;
      if (row_loss) row_loss[r] = loss;
      if (loss_sum) atomicAdd(loss_sum, loss * loss_scale);
      if (corrects && a2 == (int)lab) atomicAdd(corrects, 1);
    }
    if (grad) {
      bf16* g = grad + r * ldg;
#pragma unroll
      for (int i = 0; i < MAXCH; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c < chunks) {
          CBf8 o;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int col = c * 8 + k;
            float gv = v[i][k] * inv - (col == lab ? 1.f : 0.f);
            o.v[k] = __float2bfloat16(col < V ? gv * grad_scale : 0.f);
          }
          *reinterpret_cast<CBf8*>(g + c * 8) = o;
        }
      }
    }
    __syncthreads();
  }
}

// p_master (fp32) is always updated; p_lp (bf16 compute copy) is written when given.
__global__ void adam_kernel(float* __restrict__ master, bf16* __restrict__ p_lp, const float* __restrict__ grad,
                            float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1,
                            float b2, float eps, float wd, float bc1, float bc2, float gscale,
                            const float* __restrict__ hyper) {
  // hyper = {lr, bc1, bc2, gscale} in device memory: lets a captured CUDA graph
  // see a new learning rate / step count on every replay.
  if (hyper) {
    lr = hyper[0];
    bc1 = hyper[1];
    bc2 = hyper[2];
    gscale = hyper[3];
  }
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const float g = grad[i] * gscale;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float pw = master[i];
    const float upd = lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    pw = pw - upd - wd * lr * pw;
    master[i] = pw;
    if (p_lp) p_lp[i] = __float2bfloat16(pw);
  }
}

__global__ void sgd_kernel(float* __restrict__ master, bf16* __restrict__ p_lp, const float* __restrict__ grad,
                           float* __restrict__ vel, long long n, float lr, float mu, float gscale,
                           const float* __restrict__ hyper) {
  if (hyper) {
    lr = hyper[0];
    gscale = hyper[3];
  }
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const float g = grad[i] * gscale;
    float pw = master[i];
    if (vel) {
      const float vv = mu * vel[i] - lr * g;
      vel[i] = vv;
      pw += vv;
    } else {
      pw -= lr * g;
    }
    master[i] = pw;
    if (p_lp) p_lp[i] = __float2bfloat16(pw);
  }
}

}  // namespace tnnb

using namespace tnnb;

extern "C" {

// logits [rows, V] bf16 with row pitch ld (multiple of 8 elements, 16-byte
// aligned base). grad may be null, or alias logits. loss_sum accumulates
// loss*loss_scale (zero it first); corrects accumulates argmax==label counts.
int tnnb_softmax_ce(const void* logits, long long ld, const void* labels, void* grad, long long ldg,
                    void* row_loss, void* loss_sum, void* corrects, long long rows, int V, float grad_scale,
                    float loss_scale, void* stream) {
  if (ld % 8 || (grad && ldg % 8) || ((uintptr_t)logits & 15) || ((uintptr_t)grad & 15)) return -3;
  if (ld < ((V + 7) / 8) * 8 || (grad && ldg < ((V + 7) / 8) * 8)) return -3;
  cudaStream_t st = (cudaStream_t)stream;
  const int chunks = (V + 7) / 8;
  int grid = (int)(rows < 148 * 4 ? rows : 148 * 4);
#define CE(MC, TH)                                                                                         \
  softmax_ce_kernel<MC, TH><<<grid, TH, 0, st>>>((const bf16*)logits, ld, (const long long*)labels,       \
                                                 (bf16*)grad, ldg, (float*)row_loss, (float*)loss_sum,    \
                                                 (int*)corrects, rows, V, grad_scale, loss_scale)
  if (chunks <= 128) CE(1, 128);
  else if (chunks <= 256 * 2) CE(2, 256);
  else if (chunks <= 1024 * 4) CE(4, 1024);
  else if (chunks <= 1024 * 8) CE(8, 1024);
  else return -7;
#undef CE
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

int tnnb_adam_step(void* master, void* p_lp, const void* grad, void* m, void* v, long long n, float lr,
                   float b1, float b2, float eps, float wd, float bc1, float bc2, float gscale, const void* hyper,
                   void* stream) {
  long long g = (n + 1023) / 1024;
  int grid = (int)(g > 148 * 8 ? 148 * 8 : (g < 1 ? 1 : g));
  adam_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((float*)master, (bf16*)p_lp, (const float*)grad, (float*)m,
                                                     (float*)v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale,
                                                     (const float*)hyper);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

int tnnb_sgd_step(void* master, void* p_lp, const void* grad, void* vel, long long n, float lr, float mu,
                  float gscale, const void* hyper, void* stream) {
  long long g = (n + 1023) / 1024;
  int grid = (int)(g > 148 * 8 ? 148 * 8 : (g < 1 ? 1 : g));
  sgd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((float*)master, (bf16*)p_lp, (const float*)grad, (float*)vel,
                                                    n, lr, mu, gscale, (const float*)hyper);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -(int)e - 1000;
}

}  // extern "C"
