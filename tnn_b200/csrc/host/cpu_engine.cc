// fp32 CPU engine: NHWC reference implementations of every operator, written
// for clarity first and OpenMP-parallel over the outer dimension. It is (a) the
// numerical oracle the GPU kernels are tested against and (b) the engine behind
// device_type "CPU" for the small-CNN configuration. Semantics follow the
// reference CPU engine (src/nn/engines/cpu_engine.cpp: dense :25-44, pools
// :66-210, batchnorm :378-511, layernorm :513-614, conv :617-734) and its loss /
// optimizer kernels (src/nn/loss_impl/cpu/loss_ops.cpp, optimizers_impl/cpu).
#include <pybind11/numpy.h>
#include <pybind11/stl.h>
#include <pybind11/pybind11.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <vector>

namespace py = pybind11;
using farr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using iarr = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;

namespace tnnb {

// C[M,N] (+)= A * B with optional transposes; row-major, register-blocked 4x16 inner kernel.
static void sgemm(bool ta, bool tb, int M, int N, int K, const float* A, int lda, const float* B, int ldb, float* C,
                  int ldc, bool accumulate) {
  auto a = [&](int m, int k) { return ta ? A[(size_t)k * lda + m] : A[(size_t)m * lda + k]; };
#pragma omp parallel for schedule(static)
  for (int m0 = 0; m0 < M; m0 += 4) {
    const int mb = std::min(4, M - m0);
    std::vector<float> acc(4 * 16);
    for (int n0 = 0; n0 < N; n0 += 16) {
      const int nb = std::min(16, N - n0);
      std::fill(acc.begin(), acc.end(), 0.f);
      for (int k = 0; k < K; ++k) {
        float bv[16];
        if (tb)
          for (int j = 0; j < nb; ++j) bv[j] = B[(size_t)(n0 + j) * ldb + k];
        else
          for (int j = 0; j < nb; ++j) bv[j] = B[(size_t)k * ldb + n0 + j];
        for (int i = 0; i < mb; ++i) {
          const float av = a(m0 + i, k);
          for (int j = 0; j < nb; ++j) acc[i * 16 + j] += av * bv[j];
        }
      }
      for (int i = 0; i < mb; ++i)
        for (int j = 0; j < nb; ++j) {
          float& c = C[(size_t)(m0 + i) * ldc + n0 + j];
          c = accumulate ? c + acc[i * 16 + j] : acc[i * 16 + j];
        }
    }
  }
}

static farr dense_fwd(farr x, farr w, py::object bias) {
  const int M = (int)x.shape(0), K = (int)x.shape(1), N = (int)w.shape(0);
  if (w.shape(1) != K) throw std::runtime_error("dense_fwd: weight shape mismatch");
  farr y({M, N});
  sgemm(false, true, M, N, K, x.data(), K, w.data(), K, y.mutable_data(), N, false);
  if (!bias.is_none()) {
    farr b = bias.cast<farr>();
    float* yp = y.mutable_data();
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) yp[(size_t)m * N + n] += b.data()[n];
  }
  return y;
}
// returns dx; dw (and db) accumulate in place
static farr dense_bwd(farr dy, farr x, farr w, farr dw, py::object db) {
  const int M = (int)x.shape(0), K = (int)x.shape(1), N = (int)w.shape(0);
  sgemm(true, false, N, K, M, dy.data(), N, x.data(), K, dw.mutable_data(), K, true);
  if (!db.is_none()) {
    farr b = db.cast<farr>();
    float* bp = b.mutable_data();
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) bp[n] += dy.data()[(size_t)m * N + n];
  }
  farr dx({M, K});
  sgemm(false, false, M, K, N, dy.data(), N, w.data(), K, dx.mutable_data(), K, false);
  return dx;
}

struct ConvGeom {
  int N, H, W, C, O, KH, KW, SH, SW, PH, PW, OH, OW;
};
static ConvGeom conv_geom(const farr& x, const farr& w, int sh, int sw, int ph, int pw) {
  ConvGeom g{(int)x.shape(0), (int)x.shape(1), (int)x.shape(2), (int)x.shape(3), (int)w.shape(0), (int)w.shape(1),
             (int)w.shape(2), sh, sw, ph, pw, 0, 0};
  if (w.shape(3) != g.C) throw std::runtime_error("conv2d: channel mismatch");
  g.OH = (g.H + 2 * ph - g.KH) / sh + 1;
  g.OW = (g.W + 2 * pw - g.KW) / sw + 1;
  return g;
}

static farr conv2d_fwd(farr x, farr w, py::object bias, int sh, int sw, int ph, int pw) {
  const ConvGeom g = conv_geom(x, w, sh, sw, ph, pw);
  farr y({g.N, g.OH, g.OW, g.O});
  const float* xp = x.data();
  const float* wp = w.data();
  const float* bp = bias.is_none() ? nullptr : bias.cast<farr>().data();
  std::vector<float> bcopy;
  if (bp) bcopy.assign(bp, bp + g.O), bp = bcopy.data();
  float* yp = y.mutable_data();
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < g.N; ++n)
    for (int oh = 0; oh < g.OH; ++oh)
      for (int ow = 0; ow < g.OW; ++ow) {
        float* out = yp + (((size_t)n * g.OH + oh) * g.OW + ow) * g.O;
        for (int o = 0; o < g.O; ++o) out[o] = bp ? bp[o] : 0.f;
        for (int kh = 0; kh < g.KH; ++kh) {
          const int ih = oh * g.SH + kh - g.PH;
          if (ih < 0 || ih >= g.H) continue;
          for (int kw = 0; kw < g.KW; ++kw) {
            const int iw = ow * g.SW + kw - g.PW;
            if (iw < 0 || iw >= g.W) continue;
            const float* in = xp + (((size_t)n * g.H + ih) * g.W + iw) * g.C;
            for (int o = 0; o < g.O; ++o) {
              const float* wk = wp + (((size_t)o * g.KH + kh) * g.KW + kw) * g.C;
              float s = 0.f;
              for (int c = 0; c < g.C; ++c) s += in[c] * wk[c];
              out[o] += s;
            }
          }
        }
      }
  return y;
}

static farr conv2d_dgrad(farr dy, farr w, std::vector<int> xshape, int sh, int sw, int ph, int pw) {
  farr dx({xshape[0], xshape[1], xshape[2], xshape[3]});
  const ConvGeom g = conv_geom(dx, w, sh, sw, ph, pw);
  std::memset(dx.mutable_data(), 0, sizeof(float) * dx.size());
  const float* gp = dy.data();
  const float* wp = w.data();
  float* dp = dx.mutable_data();
#pragma omp parallel for schedule(static)
  for (int n = 0; n < g.N; ++n)
    for (int oh = 0; oh < g.OH; ++oh)
      for (int ow = 0; ow < g.OW; ++ow) {
        const float* go = gp + (((size_t)n * g.OH + oh) * g.OW + ow) * g.O;
        for (int kh = 0; kh < g.KH; ++kh) {
          const int ih = oh * g.SH + kh - g.PH;
          if (ih < 0 || ih >= g.H) continue;
          for (int kw = 0; kw < g.KW; ++kw) {
            const int iw = ow * g.SW + kw - g.PW;
            if (iw < 0 || iw >= g.W) continue;
            float* di = dp + (((size_t)n * g.H + ih) * g.W + iw) * g.C;
            for (int o = 0; o < g.O; ++o) {
              const float gv = go[o];
              const float* wk = wp + (((size_t)o * g.KH + kh) * g.KW + kw) * g.C;
              for (int c = 0; c < g.C; ++c) di[c] += gv * wk[c];
            }
          }
        }
      }
  return dx;
}

// dw and db accumulate
static void conv2d_wgrad(farr x, farr dy, farr dw, py::object db, int sh, int sw, int ph, int pw) {
  const ConvGeom g = conv_geom(x, dw, sh, sw, ph, pw);
  const float* xp = x.data();
  const float* gp = dy.data();
  float* wp = dw.mutable_data();
#pragma omp parallel for schedule(static)
  for (int o = 0; o < g.O; ++o)
    for (int n = 0; n < g.N; ++n)
      for (int oh = 0; oh < g.OH; ++oh)
        for (int ow = 0; ow < g.OW; ++ow) {
          const float gv = gp[(((size_t)n * g.OH + oh) * g.OW + ow) * g.O + o];
          if (gv == 0.f) continue;
          for (int kh = 0; kh < g.KH; ++kh) {
            const int ih = oh * g.SH + kh - g.PH;
            if (ih < 0 || ih >= g.H) continue;
            for (int kw = 0; kw < g.KW; ++kw) {
              const int iw = ow * g.SW + kw - g.PW;
              if (iw < 0 || iw >= g.W) continue;
              const float* in = xp + (((size_t)n * g.H + ih) * g.W + iw) * g.C;
              float* wk = wp + (((size_t)o * g.KH + kh) * g.KW + kw) * g.C;
              for (int c = 0; c < g.C; ++c) wk[c] += gv * in[c];
            }
          }
        }
  if (!db.is_none()) {
    farr b = db.cast<farr>();
    float* bp = b.mutable_data();
    const size_t rows = (size_t)g.N * g.OH * g.OW;
    for (size_t r = 0; r < rows; ++r)
      for (int o = 0; o < g.O; ++o) bp[o] += gp[r * g.O + o];
  }
}

// returns (y, mean, inv_std); running stats updated in place. x is [M, C].
static py::tuple batchnorm_fwd(farr x, py::object gamma, py::object beta, farr run_mean, farr run_var, float eps,
                               float momentum, bool relu, bool training) {
  const size_t M = (size_t)x.shape(0);
  const int C = (int)x.shape(1);
  farr y({(py::ssize_t)M, (py::ssize_t)C}), mean(C), inv(C);
  const float* g = gamma.is_none() ? nullptr : gamma.cast<farr>().data();
  const float* b = beta.is_none() ? nullptr : beta.cast<farr>().data();
  std::vector<float> gc, bc;
  if (g) gc.assign(g, g + C), g = gc.data();
  if (b) bc.assign(b, b + C), b = bc.data();
  const float* xp = x.data();
  float* yp = y.mutable_data();
  float* rm = run_mean.mutable_data();
  float* rv = run_var.mutable_data();
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c) {
    float mu, is;
    if (training) {
      double s = 0, q = 0;
      for (size_t m = 0; m < M; ++m) s += xp[m * C + c];
      mu = (float)(s / M);
      for (size_t m = 0; m < M; ++m) {
        const double d = xp[m * C + c] - mu;
        q += d * d;
      }
      const float var = (float)(q / M);
      is = 1.f / std::sqrt(var + eps);
      const float unbiased = M > 1 ? var * (float)M / (float)(M - 1) : var;
      rm[c] = (1.f - momentum) * rm[c] + momentum * mu;
      rv[c] = (1.f - momentum) * rv[c] + momentum * unbiased;
    } else {
      mu = rm[c];
      is = 1.f / std::sqrt(rv[c] + eps);
    }
    mean.mutable_data()[c] = mu;
    inv.mutable_data()[c] = is;
    const float sc = g ? g[c] * is : is, sft = (b ? b[c] : 0.f) - mu * sc;
    for (size_t m = 0; m < M; ++m) {
      float v = xp[m * C + c] * sc + sft;
      yp[m * C + c] = relu ? std::max(v, 0.f) : v;
    }
  }
  return py::make_tuple(y, mean, inv);
}

static farr batchnorm_bwd(farr dy, farr x, farr y, farr mean, farr inv, py::object gamma, py::object dgamma,
                          py::object dbeta, bool relu) {
  const size_t M = (size_t)x.shape(0);
  const int C = (int)x.shape(1);
  farr dx({(py::ssize_t)M, (py::ssize_t)C});
  const float* g = gamma.is_none() ? nullptr : gamma.cast<farr>().data();
  std::vector<float> gc;
  if (g) gc.assign(g, g + C), g = gc.data();
  float* dg = dgamma.is_none() ? nullptr : dgamma.cast<farr>().mutable_data();
  float* db = dbeta.is_none() ? nullptr : dbeta.cast<farr>().mutable_data();
  const float *gp = dy.data(), *xp = x.data(), *yp = y.data();
  float* dp = dx.mutable_data();
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c) {
    const float mu = mean.data()[c], is = inv.data()[c];
    double sg = 0, sgx = 0;
    for (size_t m = 0; m < M; ++m) {
      float gv = gp[m * C + c];
      if (relu && yp[m * C + c] <= 0.f) gv = 0.f;
      sg += gv;
      sgx += gv * (xp[m * C + c] - mu) * is;
    }
    if (dg) dg[c] += (float)sgx;
    if (db) db[c] += (float)sg;
    const float k = (g ? g[c] : 1.f) * is / (float)M;
    for (size_t m = 0; m < M; ++m) {
      float gv = gp[m * C + c];
      if (relu && yp[m * C + c] <= 0.f) gv = 0.f;
      const float xh = (xp[m * C + c] - mu) * is;
      dp[m * C + c] = k * ((float)M * gv - (float)sg - xh * (float)sgx);
    }
  }
  return dx;
}

static py::tuple layernorm_fwd(farr x, py::object gamma, py::object beta, float eps) {
  const size_t R = (size_t)x.shape(0);
  const int C = (int)x.shape(1);
  farr y({(py::ssize_t)R, (py::ssize_t)C}), mean((py::ssize_t)R), rstd((py::ssize_t)R);
  const float* g = gamma.is_none() ? nullptr : gamma.cast<farr>().data();
  const float* b = beta.is_none() ? nullptr : beta.cast<farr>().data();
  std::vector<float> gc, bc;
  if (g) gc.assign(g, g + C), g = gc.data();
  if (b) bc.assign(b, b + C), b = bc.data();
#pragma omp parallel for schedule(static)
  for (size_t r = 0; r < R; ++r) {
    const float* xr = x.data() + r * C;
    double s = 0, q = 0;
    for (int c = 0; c < C; ++c) s += xr[c];
    const float mu = (float)(s / C);
    for (int c = 0; c < C; ++c) q += (xr[c] - mu) * (xr[c] - mu);
    const float is = 1.f / std::sqrt((float)(q / C) + eps);
    mean.mutable_data()[r] = mu;
    rstd.mutable_data()[r] = is;
    float* yr = y.mutable_data() + r * C;
    for (int c = 0; c < C; ++c) yr[c] = (xr[c] - mu) * is * (g ? g[c] : 1.f) + (b ? b[c] : 0.f);
  }
  return py::make_tuple(y, mean, rstd);
}

static farr layernorm_bwd(farr dy, farr x, farr mean, farr rstd, py::object gamma, py::object dgamma, py::object dbeta) {
  const size_t R = (size_t)x.shape(0);
  const int C = (int)x.shape(1);
  farr dx({(py::ssize_t)R, (py::ssize_t)C});
  const float* g = gamma.is_none() ? nullptr : gamma.cast<farr>().data();
  std::vector<float> gc;
  if (g) gc.assign(g, g + C), g = gc.data();
  float* dg = dgamma.is_none() ? nullptr : dgamma.cast<farr>().mutable_data();
  float* db = dbeta.is_none() ? nullptr : dbeta.cast<farr>().mutable_data();
  for (size_t r = 0; r < R; ++r) {
    const float* xr = x.data() + r * C;
    const float* gr = dy.data() + r * C;
    const float mu = mean.data()[r], is = rstd.data()[r];
    double s1 = 0, s2 = 0;
    for (int c = 0; c < C; ++c) {
      const float xh = (xr[c] - mu) * is, d = gr[c] * (g ? g[c] : 1.f);
      s1 += d;
      s2 += d * xh;
      if (dg) dg[c] += gr[c] * xh;
      if (db) db[c] += gr[c];
    }
    float* dr = dx.mutable_data() + r * C;
    for (int c = 0; c < C; ++c) {
      const float xh = (xr[c] - mu) * is, d = gr[c] * (g ? g[c] : 1.f);
      dr[c] = is * (d - (float)(s1 / C) - xh * (float)(s2 / C));
    }
  }
  return dx;
}

// max pooling: (y, window-relative argmax index or -1); avg pooling divides by the in-image count
static py::tuple pool2d_fwd(farr x, bool is_max, int kh_, int kw_, int sh, int sw, int ph, int pw) {
  const int N = (int)x.shape(0), H = (int)x.shape(1), W = (int)x.shape(2), C = (int)x.shape(3);
  const int OH = (H + 2 * ph - kh_) / sh + 1, OW = (W + 2 * pw - kw_) / sw + 1;
  farr y({N, OH, OW, C});
  iarr idx({N, OH, OW, C});
#pragma omp parallel for collapse(2) schedule(static)
  for (int n = 0; n < N; ++n)
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow)
        for (int c = 0; c < C; ++c) {
          float best = -INFINITY, sum = 0.f;
          int bi = -1, cnt = 0;
          for (int kh = 0; kh < kh_; ++kh) {
            const int ih = oh * sh + kh - ph;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < kw_; ++kw) {
              const int iw = ow * sw + kw - pw;
              if (iw < 0 || iw >= W) continue;
              const float v = x.data()[(((size_t)n * H + ih) * W + iw) * C + c];
              sum += v;
              ++cnt;
              if (v > best) best = v, bi = kh * kw_ + kw;
            }
          }
          const size_t o = (((size_t)n * OH + oh) * OW + ow) * C + c;
          y.mutable_data()[o] = is_max ? (bi >= 0 ? best : 0.f) : (cnt ? sum / cnt : 0.f);
          idx.mutable_data()[o] = bi;
        }
  return py::make_tuple(y, idx);
}

static farr pool2d_bwd(farr dy, iarr idx, std::vector<int> xs, bool is_max, int kh_, int kw_, int sh, int sw, int ph, int pw) {
  const int N = xs[0], H = xs[1], W = xs[2], C = xs[3];
  const int OH = (int)dy.shape(1), OW = (int)dy.shape(2);
  farr dx({N, H, W, C});
  std::memset(dx.mutable_data(), 0, sizeof(float) * dx.size());
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int oh = 0; oh < OH; ++oh)
      for (int ow = 0; ow < OW; ++ow)
        for (int c = 0; c < C; ++c) {
          const size_t o = (((size_t)n * OH + oh) * OW + ow) * C + c;
          const float g = dy.data()[o];
          if (is_max) {
            const int bi = idx.data()[o];
            if (bi < 0) continue;
            const int ih = oh * sh + bi / kw_ - ph, iw = ow * sw + bi % kw_ - pw;
            dx.mutable_data()[(((size_t)n * H + ih) * W + iw) * C + c] += g;
          } else {
            int cnt = 0;
            for (int kh = 0; kh < kh_; ++kh)
              for (int kw = 0; kw < kw_; ++kw) {
                const int ih = oh * sh + kh - ph, iw = ow * sw + kw - pw;
                cnt += (ih >= 0 && ih < H && iw >= 0 && iw < W);
              }
            if (!cnt) continue;
            for (int kh = 0; kh < kh_; ++kh)
              for (int kw = 0; kw < kw_; ++kw) {
                const int ih = oh * sh + kh - ph, iw = ow * sw + kw - pw;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) dx.mutable_data()[(((size_t)n * H + ih) * W + iw) * C + c] += g / cnt;
              }
          }
        }
  return dx;
}

static farr relu_fwd(farr x) {
  farr y(x.size());
  for (py::ssize_t i = 0; i < x.size(); ++i) y.mutable_data()[i] = std::max(x.data()[i], 0.f);
  y.resize(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
  return y;
}
static farr relu_bwd(farr x, farr dy) {
  farr d(x.size());
  for (py::ssize_t i = 0; i < x.size(); ++i) d.mutable_data()[i] = x.data()[i] > 0.f ? dy.data()[i] : 0.f;
  d.resize(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
  return d;
}
static float gelu_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + std::tanh(u));
}
static farr gelu_fwd(farr x) {
  farr y(x.size());
  for (py::ssize_t i = 0; i < x.size(); ++i) y.mutable_data()[i] = gelu_f(x.data()[i]);
  y.resize(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
  return y;
}

// returns (mean loss, grad (softmax - onehot)/rows, corrects)
static py::tuple softmax_ce(farr logits, iarr labels) {
  const size_t R = (size_t)logits.shape(0);
  const int V = (int)logits.shape(1);
  farr grad({(py::ssize_t)R, (py::ssize_t)V});
  double total = 0;
  long corrects = 0;
#pragma omp parallel for reduction(+ : total, corrects) schedule(static)
  for (size_t r = 0; r < R; ++r) {
    const float* z = logits.data() + r * V;
    float mx = z[0];
    int arg = 0;
    for (int v = 1; v < V; ++v)
      if (z[v] > mx) mx = z[v], arg = v;
    double s = 0;
    for (int v = 0; v < V; ++v) s += std::exp((double)z[v] - mx);
    const int lab = labels.data()[r];
    total += std::log(s) + mx - z[lab];
    corrects += (arg == lab);
    float* g = grad.mutable_data() + r * V;
    for (int v = 0; v < V; ++v) g[v] = (float)(std::exp((double)z[v] - mx) / s) / (float)R;
    g[lab] -= 1.f / (float)R;
  }
  return py::make_tuple((float)(total / R), grad, corrects);
}

static void sgd_step(farr p, farr g, py::object vel, float lr, float mu) {
  float* pp = p.mutable_data();
  const float* gp = g.data();
  if (vel.is_none()) {
    for (py::ssize_t i = 0; i < p.size(); ++i) pp[i] -= lr * gp[i];
  } else {
    float* vp = vel.cast<farr>().mutable_data();
    for (py::ssize_t i = 0; i < p.size(); ++i) {
      vp[i] = mu * vp[i] - lr * gp[i];
      pp[i] += vp[i];
    }
  }
}
static void adam_step(farr p, farr g, farr m, farr v, float lr, float b1, float b2, float eps, float wd, int step) {
  const float bc1 = 1.f - std::pow(b1, (float)step), bc2 = 1.f - std::pow(b2, (float)step);
  float *pp = p.mutable_data(), *mp = m.mutable_data(), *vp = v.mutable_data();
  const float* gp = g.data();
  for (py::ssize_t i = 0; i < p.size(); ++i) {
    mp[i] = b1 * mp[i] + (1.f - b1) * gp[i];
    vp[i] = b2 * vp[i] + (1.f - b2) * gp[i] * gp[i];
    const float upd = lr * (mp[i] / bc1) / (std::sqrt(vp[i] / bc2) + eps);
    pp[i] = pp[i] - upd - wd * lr * pp[i];
  }
}

void bind_cpu_engine(py::module_& m) {
  py::module_ c = m.def_submodule("cpu", "fp32 NHWC reference engine (oracle and CPU baseline)");
  c.def("dense_fwd", &dense_fwd, py::arg("x"), py::arg("w"), py::arg("bias") = py::none());
  c.def("dense_bwd", &dense_bwd);
  c.def("conv2d_fwd", &conv2d_fwd);
  c.def("conv2d_dgrad", &conv2d_dgrad);
  c.def("conv2d_wgrad", &conv2d_wgrad);
  c.def("batchnorm_fwd", &batchnorm_fwd);
  c.def("batchnorm_bwd", &batchnorm_bwd);
  c.def("layernorm_fwd", &layernorm_fwd);
  c.def("layernorm_bwd", &layernorm_bwd);
  c.def("pool2d_fwd", &pool2d_fwd);
  c.def("pool2d_bwd", &pool2d_bwd);
  c.def("relu_fwd", &relu_fwd);
  c.def("relu_bwd", &relu_bwd);
  c.def("gelu_fwd", &gelu_fwd);
  c.def("softmax_ce", &softmax_ce);
  c.def("sgd_step", &sgd_step);
  c.def("adam_step", &adam_step);
}

}  // namespace tnnb
