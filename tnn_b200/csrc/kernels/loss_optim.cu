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

TNNB_BOUNDS_TU(loss_optim)

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

// Large vocabularies: the row is streamed through shared memory. Two persistent CTAs per SM, each with
// one row buffer: a bulk copy brings the row in, the 512 threads make three passes over it (max +
// arg-max, exp + sum written back as bf16, gradient in place) and a bulk copy takes the gradient out,
// so global memory sees exactly one read and one write of the logits; while one CTA of the SM
// computes, the other one's copies are in flight.
static constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS, 2)
softmax_ce_stream_kernel(const bf16* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                         bf16* grad, long long ldg, float* __restrict__ row_loss, float* __restrict__ loss_sum,
                         int* __restrict__ corrects, long long rows, int V, float grad_scale, float loss_scale,
                         int* status) {
  extern __shared__ __align__(128) uint8_t ce_smem[];
  __shared__ float sh[32];
  __shared__ int sh_arg[32];
  __shared__ float sh_zl;
  __shared__ __align__(8) uint64_t full;
  __shared__ uint32_t abort_word;
  const int chunks = (V + 7) >> 3;
  const uint32_t row_bytes = (uint32_t)chunks * 16u;
  volatile uint32_t* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&full, 1);
    abort_word = 0;
    mbar_fence_init();
  }
  __syncthreads();
  int k = 0;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x, ++k) {
    if (threadIdx.x == 0) {
      bulk_wait_group_read0();  // the previous row's gradient has left the buffer
      mbar_expect_tx(&full, row_bytes);
      bulk_load_g2s(ce_smem, logits + r * ld, row_bytes, &full);
    }
    if (!wait_or_abort(&full, k & 1, abort_flag)) {
      if (threadIdx.x == 0) raise_abort(status, abort_flag, ST_TIMEOUT_EPILOGUE);
      break;
    }
    uint4* row = reinterpret_cast<uint4*>(ce_smem);
    bf16* row_e = reinterpret_cast<bf16*>(ce_smem);
    const long long lab = labels[r];
    if (threadIdx.x == 0) (void)TNNB_CHECK(lab, V);  // checked build: report the label; both builds leave it out of the loss
    // Columns V .. 8*chunks-1 of the last chunk hold whatever the row pitch contains: make them -inf once
    // (exp gives 0, the gradient 0) so that the passes below need no per-element bounds checks.
    if (threadIdx.x < 8 && (chunks - 1) * 8 + (int)threadIdx.x >= V)
      reinterpret_cast<uint16_t*>(ce_smem)[(chunks - 1) * 8 + threadIdx.x] = 0xff80u;
    if (threadIdx.x == 0) sh_zl = (lab >= 0 && lab < V) ? __bfloat162float(row_e[lab]) : NAN;
    __syncthreads();
    // pass 1: row maximum with packed bf16 max (exact), remembering the first chunk that attains it
    float mx = -INFINITY;
    int arg_chunk = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += CE_THREADS) {
      const uint4 u = row[c];
      __nv_bfloat162 m = __hmax2(__hmax2(*reinterpret_cast<const __nv_bfloat162*>(&u.x), *reinterpret_cast<const __nv_bfloat162*>(&u.y)),
                                 __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&u.z), *reinterpret_cast<const __nv_bfloat162*>(&u.w)));
      const float cm = fmaxf(__low2float(m), __high2float(m));
      if (cm > mx) {
        mx = cm;
        arg_chunk = c;
      }
    }
    float m2 = mx;
    int a2 = arg_chunk;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m2, o);
      const int oa = __shfl_xor_sync(0xffffffffu, a2, o);
      if (om > m2 || (om == m2 && oa < a2)) { m2 = om; a2 = oa; }
    }
    const int wi = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sh[wi] = m2; sh_arg[wi] = a2; }
    __syncthreads();
    m2 = l < CE_THREADS / 32 ? sh[l] : -INFINITY;
    a2 = l < CE_THREADS / 32 ? sh_arg[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m2, o);
      const int oa = __shfl_xor_sync(0xffffffffu, a2, o);
      if (om > m2 || (om == m2 && oa < a2)) { m2 = om; a2 = oa; }
    }
    const float rmax = m2;
    int amax = 0;
    if (threadIdx.x == 0 && corrects) {  // first element of the winning chunk that equals the maximum
      amax = a2 * 8;
      for (int j = 0; j < 8; ++j)
        if (__bfloat162float(row_e[a2 * 8 + j]) == rmax) {
          amax = a2 * 8 + j;
          break;
        }
    }
    __syncthreads();  // every thread has read sh / the winning chunk before pass 2 rewrites the row
    // pass 2: e = exp(z - max) = exp2(z*log2(e) - max*log2(e)), summed in fp32 and written back as bf16
    const float kL = 1.4426950408889634f, nb = -rmax * kL;
    float s0 = 0.f, s1 = 0.f;
    for (int c = threadIdx.x; c < chunks; c += CE_THREADS) {
      const uint4 u = row[c];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e0 = exp2f(fmaf(__uint_as_float(w[i] << 16), kL, nb));
        const float e1 = exp2f(fmaf(__uint_as_float(w[i] & 0xffff0000u), kL, nb));
        s0 += e0;
        s1 += e1;
        __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
        o[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      row[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    const float s = block_reduce_sum(s0 + s1, sh);
    const float inv = 1.f / s;
    if (threadIdx.x == 0) {
      const float zl = (lab >= 0 && lab < V) ? sh_zl : rmax;
      const float loss = __logf(s) + rmax - zl;
      if (row_loss) row_loss[r] = loss;
      if (loss_sum) atomicAdd(loss_sum, loss * loss_scale);
      if (corrects && amax == (int)lab) atomicAdd(corrects, 1);
    }
    if (grad) {
      // pass 3: gradient in place (the label's element is patched afterwards), then one bulk copy out
      const float gs = inv * grad_scale;
      for (int c = threadIdx.x; c < chunks; c += CE_THREADS) {
        const uint4 u = row[c];
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(w[i] << 16) * gs, __uint_as_float(w[i] & 0xffff0000u) * gs);
          o[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        row[c] = make_uint4(o[0], o[1], o[2], o[3]);
      }
      __syncthreads();
      if (threadIdx.x == 0 && lab >= 0 && lab < V)
        row_e[lab] = __float2bfloat16(__bfloat162float(row_e[lab]) - grad_scale);
      fence_proxy_async_smem();
      __syncthreads();
      if (threadIdx.x == 0) {
        bulk_store_s2g(grad + r * ldg, ce_smem, row_bytes);
        bulk_commit_group();
      }
    } else {
      __syncthreads();
    }
  }
  if (threadIdx.x == 0) bulk_wait_group0();
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
      (void)TNNB_CHECK(lab, V);
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
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float ib1 = 1.f / bc1, ib2 = 1.f / bc2;
  auto update = [&](float g, float& mi, float& vi, float& pw) {
    g *= gscale;
    mi = b1 * mi + (1.f - b1) * g;
    vi = b2 * vi + (1.f - b2) * g * g;
    const float upd = lr * (mi * ib1) / (sqrtf(vi * ib2) + eps);
    pw = pw - upd - wd * lr * pw;
  };
  // 16-byte accesses when every buffer allows it (four independent streams per thread)
  const bool vec = ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15) == 0 && (reinterpret_cast<uintptr_t>(p_lp) & 7) == 0;
  const long long n4 = vec ? n / 4 : 0;
  for (long long j = tid; j < n4; j += stride) {
    const float4 g4 = reinterpret_cast<const float4*>(grad)[j];
    float4 m4 = reinterpret_cast<float4*>(m)[j], v4 = reinterpret_cast<float4*>(v)[j], p4 = reinterpret_cast<float4*>(master)[j];
    update(g4.x, m4.x, v4.x, p4.x);
    update(g4.y, m4.y, v4.y, p4.y);
    update(g4.z, m4.z, v4.z, p4.z);
    update(g4.w, m4.w, v4.w, p4.w);
    reinterpret_cast<float4*>(m)[j] = m4;
    reinterpret_cast<float4*>(v)[j] = v4;
    reinterpret_cast<float4*>(master)[j] = p4;
    if (p_lp) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p4.x, p4.y), hi = __floats2bfloat162_rn(p4.z, p4.w);
      reinterpret_cast<uint2*>(p_lp)[j] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
  for (long long i = n4 * 4 + tid; i < n; i += stride) {
    float mi = m[i], vi = v[i], pw = master[i];
    update(grad[i], mi, vi, pw);
    m[i] = mi;
    v[i] = vi;
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
  const size_t stream_smem = ((size_t)chunks * 16 + 127) & ~(size_t)127;
  if (chunks > 1024 && stream_smem <= 112 * 1024) {
    static bool attr_done = false;
    if (!attr_done) {
      cudaFuncSetAttribute(softmax_ce_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
      attr_done = true;
    }
    const int g2 = (int)(rows < 296 ? rows : 296);
    softmax_ce_stream_kernel<<<g2, CE_THREADS, stream_smem, st>>>((const bf16*)logits, ld, (const long long*)labels,
                                                                 (bf16*)grad, ldg, (float*)row_loss, (float*)loss_sum,
                                                                 (int*)corrects, rows, V, grad_scale, loss_scale, nullptr);
    cudaError_t e2 = cudaGetLastError();
    return e2 == cudaSuccess ? 0 : -(int)e2 - 1000;
  }
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
