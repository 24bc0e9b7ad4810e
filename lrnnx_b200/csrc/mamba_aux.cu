// Elementwise companions of the selective scan inside a Mamba block: the depthwise causal
// convolution (+ SiLU) before the scan, its one-token update for decoding, and the fused
// residual-add + RMSNorm before the block.  All three are HBM-bound: every element is read once
// and written once with 16-byte accesses.
//   causal conv:  lrnnx/models/ltv/mamba.py:270-279 (nn.Conv1d(groups=d_inner, padding=d_conv-1)
//                 truncated to L, then SiLU) and :394-409 (roll + dot + SiLU in step());
//   add + norm:   lrnnx/ops/triton/layer_norm.py:994-1094 (rms_norm_fn with residual, prenorm).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int CVT = 256;          // threads per CTA of the convolution kernels
constexpr int CVE = 8;            // timesteps per thread
constexpr int MAXW = 4;           // widest convolution

template <typename T> __device__ __forceinline__ float tof(T v);
template <> __device__ __forceinline__ float tof<float>(float v) { return v; }
template <> __device__ __forceinline__ float tof<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float tof<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T fromf(float v);
template <> __device__ __forceinline__ float fromf<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 fromf<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half fromf<__half>(float v) { return __float2half_rn(v); }

// 8 consecutive elements of a row starting at t (t a multiple of 8); positions outside [0, L)
// read as zero.  16-byte accesses where the address allows, element accesses otherwise.
__device__ __forceinline__ bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
template <typename T> __device__ __forceinline__ void load8(const T *row, int t, int L, float (&v)[CVE]) {
  if (t >= 0 && t + CVE <= L && al16(row + t)) {
    if constexpr (sizeof(T) == 2) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(row + t);
      const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
      for (int i = 0; i < CVE; ++i) v[i] = tof(e[i]);
    } else {
      const float4 a = *reinterpret_cast<const float4 *>(row + t), b = *reinterpret_cast<const float4 *>(row + t + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < CVE; ++i) v[i] = (t + i >= 0 && t + i < L) ? tof(row[t + i]) : 0.f;
  }
}
template <typename T> __device__ __forceinline__ void store8(T *row, int t, int L, const float (&v)[CVE]) {
  if (t + CVE <= L && al16(row + t)) {
    if constexpr (sizeof(T) == 2) {
      uint4 raw;
      T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
      for (int i = 0; i < CVE; ++i) e[i] = fromf<T>(v[i]);
      *reinterpret_cast<uint4 *>(row + t) = raw;
    } else {
      *reinterpret_cast<float4 *>(row + t) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(row + t + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < CVE; ++i)
      if (t + i < L) row[t + i] = fromf<T>(v[i]);
  }
}

__device__ __forceinline__ float silu_f(float x) { return x * sigmoidf_(x); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = sigmoidf_(x);
  return s * (1.f + x * (1.f - s));
}

// out[b, d, t] = act(bias[d] + sum_k w[d, k] x[b, d, t - (W-1) + k])
// Threads per row of an item: 256 for rows of 2048 steps or more, the next power of two above L / 8
// for shorter rows, so that a CTA of 256 threads covers 256 / tpr batch rows at once and no thread
// idles past the end of a short row.
__host__ __device__ __forceinline__ int conv_tpr(int L) {
  int t = 1;
  while (t < CVT && t * CVE < L) t <<= 1;
  return t;
}

// A CTA owns one channel (its taps are read once) and walks that channel's work items, an item
// being up to CVT * CVE consecutive steps of one batch row (or of several short rows): few, long-lived CTAs instead of one per item
// (the kernel moves 4 bytes per thread-instruction; the rate at which thread blocks can be
// started would bound it otherwise).
template <typename T>
__global__ void __launch_bounds__(CVT) conv1d_fwd_kernel(const b200_conv1d_args p) {
  const int d = blockIdx.x;
  const int W = p.width, L = p.seqlen;
  const int tpr = conv_tpr(L), rpi = CVT / tpr;          // threads per row, batch rows per item
  const int nblk = (L + tpr * CVE - 1) / (tpr * CVE), items = ((p.batch + rpi - 1) / rpi) * nblk;
  const int sub = threadIdx.x / tpr, tt = threadIdx.x - sub * tpr;
  // the taps right-aligned in a window of MAXW (zeros in front): every register index below is a
  // compile-time constant whatever the width
  float w[MAXW];
#pragma unroll
  for (int k = 0; k < MAXW; ++k)
    w[k] = k >= MAXW - W ? tof(reinterpret_cast<const T *>(p.weight)[(int64_t)d * W + k - (MAXW - W)]) : 0.f;
  const float bias = p.bias ? tof(reinterpret_cast<const T *>(p.bias)[d]) : 0.f;
  for (int item = blockIdx.y; item < items; item += gridDim.y) {
    const int bg = item / nblk;
    const int b = bg * rpi + sub;
    const int t = ((item - bg * nblk) * tpr + tt) * CVE;
    if (t >= L || b >= p.batch) continue;
    const T *x = reinterpret_cast<const T *>(p.x) + (int64_t)b * p.x_bs + (int64_t)d * p.x_ds;
    T *out = reinterpret_cast<T *>(p.out) + (int64_t)b * p.out_bs + (int64_t)d * p.out_ds;
    float prev[CVE], cur[CVE], y[CVE];
    load8<T>(x, t - CVE, L, prev);
    load8<T>(x, t, L, cur);
#pragma unroll
    for (int i = 0; i < CVE; ++i) {
      float acc = bias;
#pragma unroll
      for (int k = 0; k < MAXW; ++k) {
        const int j = i - (MAXW - 1) + k;              // offset inside [prev | cur]
        acc = fmaf(w[k], j >= 0 ? cur[j] : prev[CVE + j], acc);
      }
      y[i] = p.silu ? silu_f(acc) : acc;
    }
    store8<T>(out, t, L, y);
  }
}

// dx, and per-thread partial sums of dweight / dbias folded per CTA into float32 accumulators
template <typename T>
__global__ void __launch_bounds__(CVT) conv1d_bwd_kernel(const b200_conv1d_args p) {
  const int d = blockIdx.x;                         // a CTA owns one channel, as in the forward kernel
  const int W = p.width, L = p.seqlen;
  const int tpr = conv_tpr(L), rpi = CVT / tpr;          // threads per row, batch rows per item
  const int nblk = (L + tpr * CVE - 1) / (tpr * CVE), items = ((p.batch + rpi - 1) / rpi) * nblk;
  const int sub = threadIdx.x / tpr, tt = threadIdx.x - sub * tpr;
  // the taps right-aligned in a window of MAXW (zeros in front): every register index below is a
  // compile-time constant whatever the width
  float w[MAXW];
#pragma unroll
  for (int k = 0; k < MAXW; ++k)
    w[k] = k >= MAXW - W ? tof(reinterpret_cast<const T *>(p.weight)[(int64_t)d * W + k - (MAXW - W)]) : 0.f;
  const float bias = p.bias ? tof(reinterpret_cast<const T *>(p.bias)[d]) : 0.f;
  float dw[MAXW] = {0.f, 0.f, 0.f, 0.f}, db = 0.f;
  for (int item = blockIdx.y; item < items; item += gridDim.y) {
    const int bg = item / nblk;
    const int b = bg * rpi + sub;
    const int t = ((item - bg * nblk) * tpr + tt) * CVE;
    if (t >= L || b >= p.batch) continue;
    const T *x = reinterpret_cast<const T *>(p.x) + (int64_t)b * p.x_bs + (int64_t)d * p.x_ds;
    const T *dout = reinterpret_cast<const T *>(p.dout) + (int64_t)b * p.dout_bs + (int64_t)d * p.dout_ds;
    T *dx = reinterpret_cast<T *>(p.dx) + (int64_t)b * p.dx_bs + (int64_t)d * p.dx_ds;
    // x over [t - 8, t + 16), dout over [t, t + 16): the gradient of the pre-activation is needed
    // for this thread's 8 steps and the W - 1 steps after them
    float xs[3 * CVE], g[2 * CVE];
    {
      float a[CVE];
      load8<T>(x, t - CVE, L, a);
#pragma unroll
      for (int i = 0; i < CVE; ++i) xs[i] = a[i];
      load8<T>(x, t, L, a);
#pragma unroll
      for (int i = 0; i < CVE; ++i) xs[CVE + i] = a[i];
      load8<T>(x, t + CVE, L, a);
#pragma unroll
      for (int i = 0; i < CVE; ++i) xs[2 * CVE + i] = a[i];
      load8<T>(dout, t, L, a);
#pragma unroll
      for (int i = 0; i < CVE; ++i) g[i] = a[i];
      load8<T>(dout, t + CVE, L, a);
#pragma unroll
      for (int i = 0; i < CVE; ++i) g[CVE + i] = a[i];
    }
    float dpre[CVE + MAXW - 1];
#pragma unroll
    for (int i = 0; i < CVE + MAXW - 1; ++i) {
      float gi = g[i];                                // zero past L
      if (p.silu) {
        float acc = bias;
#pragma unroll
        for (int k = 0; k < MAXW; ++k) acc = fmaf(w[k], xs[CVE + i - (MAXW - 1) + k], acc);
        gi *= dsilu_f(acc);
      }
      dpre[i] = gi;
    }
    float dxv[CVE];
#pragma unroll
    for (int i = 0; i < CVE; ++i) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < MAXW; ++k) acc = fmaf(w[k], dpre[i + (MAXW - 1) - k], acc);   // x[t+i] feeds out[t+i+(MAXW-1)-k] through tap k
      dxv[i] = acc;
      db += dpre[i];
#pragma unroll
      for (int k = 0; k < MAXW; ++k) dw[k] = fmaf(dpre[i], xs[CVE + i - (MAXW - 1) + k], dw[k]);
    }
    store8<T>(dx, t, L, dxv);
  }
  // CTA reduction of the parameter gradients (summed over the CTA's items), then one atomic per CTA and parameter
  __shared__ float red[CVT / 32][MAXW + 1];
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < MAXW; ++k) dw[k] = warp_sum(dw[k]);
  db = warp_sum(db);
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < MAXW; ++k) red[wp][k] = dw[k];
    red[wp][MAXW] = db;
  }
  __syncthreads();
  if (threadIdx.x <= MAXW) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < CVT / 32; ++i) s += red[i][threadIdx.x];
    if ((int)threadIdx.x >= MAXW - W && threadIdx.x < MAXW)
      atomicAdd(reinterpret_cast<float *>(p.dweight) + (int64_t)d * W + threadIdx.x - (MAXW - W), s);
    if (threadIdx.x == MAXW && p.dbias) atomicAdd(reinterpret_cast<float *>(p.dbias) + d, s);
  }
}

// one token: state <- [state[1:], x]; out = act(bias + sum_k w[k] state[k])
template <typename T>
__global__ void __launch_bounds__(256) conv1d_update_kernel(const b200_conv1d_args p) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= (int64_t)p.batch * p.dim) return;
  const int b = (int)(i / p.dim), d = (int)(i % p.dim);
  const int W = p.width;
  T *st = reinterpret_cast<T *>(p.state) + (int64_t)b * p.state_bs + (int64_t)d * p.state_ds;
  const float xv = tof(reinterpret_cast<const T *>(p.x)[(int64_t)b * p.x_bs + (int64_t)d * p.x_ds]);
  float acc = p.bias ? tof(reinterpret_cast<const T *>(p.bias)[d]) : 0.f;
  float s[MAXW];
#pragma unroll
  for (int k = 0; k < MAXW; ++k) s[k] = (k + 1 < W) ? tof(st[k + 1]) : 0.f;
#pragma unroll
  for (int k = 0; k < MAXW; ++k) {
    if (k < W) {
      const float v = (k == W - 1) ? xv : s[k];
      st[k] = fromf<T>(v);
      acc = fmaf(tof(reinterpret_cast<const T *>(p.weight)[(int64_t)d * W + k]), v, acc);
    }
  }
  reinterpret_cast<T *>(p.out)[(int64_t)b * p.out_bs + (int64_t)d * p.out_ds] = fromf<T>(p.silu ? silu_f(acc) : acc);
}

// ------------------------------------------------------------------ residual add + RMSNorm
// A CTA of NT threads walks rows; a thread owns NV 16-byte vectors (8 columns each) of a row.
// (NT, NV) is picked per call so that most threads have work: (128, 1) up to 1024 columns,
// (256, 1) up to 2048, (256, 2) up to 4096.
constexpr int MAXCOLS = 4096;

template <typename T> __device__ __forceinline__ void ldv(const T *p, float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = tof(e[i]);
  } else {
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}
template <typename T> __device__ __forceinline__ void stv(T *p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw;
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = fromf<T>(v[i]);
    *reinterpret_cast<uint4 *>(p) = raw;
  } else {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

template <int NT> __device__ __forceinline__ float block_sum(float v, float *red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  __syncthreads();                 // red may still be read from the previous use
  if (lane == 0) red[wp] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) s += red[i];
  return s;
}

// z = x + residual (stored as residual_out when asked for); y = z * rstd * w, rstd = rsqrt(mean z^2 + eps)
template <typename T, typename R, int NT, int NV>
__global__ void __launch_bounds__(NT) rmsnorm_fwd_kernel(const b200_rmsnorm_args p) {
  __shared__ float red[NT / 32];
  const int H = p.cols;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T *x = reinterpret_cast<const T *>(p.x) + row * p.x_rs;
    const R *res = p.residual ? reinterpret_cast<const R *>(p.residual) + row * p.residual_rs : nullptr;
    float z[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * NT + threadIdx.x) * 8;
      if (c < H) {
        ldv<T>(x + c, z[j]);
        if (res) {
          float r[8];
          ldv<R>(res + c, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) z[j][i] += r[i];
        }
        if (p.residual_out) {
          // the sum is rounded to the residual dtype first, as the reference stores it before normalising
          R *ro = reinterpret_cast<R *>(p.residual_out) + row * p.residual_out_rs + c;
          stv<R>(ro, z[j]);
          if constexpr (sizeof(R) == 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) z[j][i] = tof(fromf<R>(z[j][i]));
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(z[j][i], z[j][i], ss);
      }
    }
    ss = block_sum<NT>(ss, red);
    const float rstd = rsqrtf(ss / (float)H + p.eps);
    if (threadIdx.x == 0 && p.rstd) reinterpret_cast<float *>(p.rstd)[row] = rstd;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * NT + threadIdx.x) * 8;
      if (c < H) {
        float w[8], y[8];
        ldv<T>(reinterpret_cast<const T *>(p.weight) + c, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = z[j][i] * rstd * w[i];
        stv<T>(reinterpret_cast<T *>(p.y) + row * p.y_rs + c, y);
      }
    }
  }
}

// dz = (w dy - zhat mean(zhat w dy)) rstd + dresidual;  dw += dy zhat  (per-thread partial, one atomic per CTA column)
template <typename T, typename R, int NT, int NV>
__global__ void __launch_bounds__(NT) rmsnorm_bwd_kernel(const b200_rmsnorm_args p) {
  __shared__ float red[NT / 32];
  const int H = p.cols;
  float dwacc[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const R *z = reinterpret_cast<const R *>(p.residual_out) + row * p.residual_out_rs;   // the normalised input
    const T *dy = reinterpret_cast<const T *>(p.dy) + row * p.dy_rs;
    const float rstd = reinterpret_cast<const float *>(p.rstd)[row];
    float zh[NV][8], wdy[NV][8];
    float c1 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * NT + threadIdx.x) * 8;
      if (c < H) {
        float w[8], g[8];
        ldv<R>(z + c, zh[j]);
        ldv<T>(dy + c, g);
        ldv<T>(reinterpret_cast<const T *>(p.weight) + c, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          zh[j][i] *= rstd;
          wdy[j][i] = g[i] * w[i];
          c1 = fmaf(zh[j][i], wdy[j][i], c1);
          dwacc[j][i] = fmaf(g[i], zh[j][i], dwacc[j][i]);
        }
      }
    }
    c1 = block_sum<NT>(c1, red) / (float)H;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * NT + threadIdx.x) * 8;
      if (c < H) {
        float dz[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) dz[i] = (wdy[j][i] - zh[j][i] * c1) * rstd;
        if (p.dresidual) {
          float r[8];
          ldv<R>(reinterpret_cast<const R *>(p.dresidual) + row * p.dresidual_rs + c, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) dz[i] += r[i];
        }
        // one gradient for both inputs of the add: dx (dtype of x) and, when asked for, dresidual_in
        stv<T>(reinterpret_cast<T *>(p.dx) + row * p.dx_rs + c, dz);
        if (p.dresidual_in) stv<R>(reinterpret_cast<R *>(p.dresidual_in) + row * p.dresidual_in_rs + c, dz);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = (j * NT + threadIdx.x) * 8;
    if (c < H) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(reinterpret_cast<float *>(p.dweight) + c + i, dwacc[j][i]);
    }
  }
}

// The same backward for rows of up to 1024 columns: a warp owns a row (lane l holds the 8-column
// vectors l, l + 32, ...), so a row costs one warp reduction and no block barrier, and the warps of
// an SM have independent rows in flight.  The weight-gradient partials stay in registers over the
// warp's rows, are summed per CTA in shared memory and leave as one atomic per CTA and column.
constexpr int NWT = 256;          // threads per CTA of the warp-per-row kernel
template <typename T, typename R, int NV>
__global__ void __launch_bounds__(NWT) rmsnorm_bwd_warp_kernel(const b200_rmsnorm_args p) {
  __shared__ float sdw[NV * 256];
  const int H = p.cols;
  const int lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < NV * 256; c += NWT) sdw[c] = 0.f;
  __syncthreads();
  float dwacc[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
  const int64_t nwarps = (int64_t)gridDim.x * (NWT / 32);
  for (int64_t row = (int64_t)blockIdx.x * (NWT / 32) + (threadIdx.x >> 5); row < p.rows; row += nwarps) {
    const R *z = reinterpret_cast<const R *>(p.residual_out) + row * p.residual_out_rs;
    const T *dy = reinterpret_cast<const T *>(p.dy) + row * p.dy_rs;
    const float rstd = reinterpret_cast<const float *>(p.rstd)[row];
    float zh[NV][8], wdy[NV][8];
    float c1 = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < H) {
        float w[8], g[8];
        ldv<R>(z + c, zh[j]);
        ldv<T>(dy + c, g);
        ldv<T>(reinterpret_cast<const T *>(p.weight) + c, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          zh[j][i] *= rstd;
          wdy[j][i] = g[i] * w[i];
          c1 = fmaf(zh[j][i], wdy[j][i], c1);
          dwacc[j][i] = fmaf(g[i], zh[j][i], dwacc[j][i]);
        }
      }
    }
    c1 = warp_sum(c1) / (float)H;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = (j * 32 + lane) * 8;
      if (c < H) {
        float dz[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) dz[i] = (wdy[j][i] - zh[j][i] * c1) * rstd;
        if (p.dresidual) {
          float r[8];
          ldv<R>(reinterpret_cast<const R *>(p.dresidual) + row * p.dresidual_rs + c, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) dz[i] += r[i];
        }
        stv<T>(reinterpret_cast<T *>(p.dx) + row * p.dx_rs + c, dz);
        if (p.dresidual_in) stv<R>(reinterpret_cast<R *>(p.dresidual_in) + row * p.dresidual_in_rs + c, dz);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = (j * 32 + lane) * 8;
    if (c < H) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&sdw[c + i], dwacc[j][i]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += NWT) atomicAdd(reinterpret_cast<float *>(p.dweight) + c, sdw[c]);
}

// ------------------------------------------------------------------ cross-entropy over a wide row
// A CTA owns a row.  Forward: one pass, each thread keeps a running (max, sum of exp) over its
// 8-element vectors, merged across the CTA.  Backward: one pass, exp(x - lse) written back in
// the logits' dtype.  Rows that are not 16-byte aligned take element accesses.
constexpr int XT = 512;           // threads per CTA of the cross-entropy kernels
constexpr float kLog2eF = 1.4426950408889634f, kLn2F = 0.6931471805599453f;

template <typename T>
__global__ void __launch_bounds__(XT) xent_fwd_kernel(const b200_xent_args p) {
  __shared__ float red_m[XT / 32], red_s[XT / 32];
  const int64_t row = blockIdx.x;
  const T *x = reinterpret_cast<const T *>(p.logits) + row * p.logits_rs;
  const int V = p.cols;
  const bool vec = al16(x) && (V % 8 == 0);
  float m = -INFINITY, sum = 0.f;      // in units of log2: m = max x log2e, sum = sum 2^(x log2e - m)
  auto take = [&](float v) {
    const float y = v * kLog2eF;
    if (y > m) {
      sum = sum * exp2f(m - y) + 1.f;
      m = y;
    } else {
      sum += exp2f(y - m);
    }
  };
  if (vec) {
    for (int c = threadIdx.x * 8; c < V; c += XT * 8) {
      float v[8];
      ldv<T>(x + c, v);
      float vm = v[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) vm = fmaxf(vm, v[i]);
      const float y = vm * kLog2eF;
      if (y > m) {
        sum *= exp2f(m - y);
        m = y;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += exp2f(fmaf(v[i], kLog2eF, -m));
    }
  } else {
    for (int c = threadIdx.x; c < V; c += XT) take(tof(x[c]));
  }
  // merge (m, sum) over the warp, then over the CTA
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
    const float nm = fmaxf(m, om);
    sum = (m == -INFINITY ? 0.f : sum * exp2f(m - nm)) + (om == -INFINITY ? 0.f : os * exp2f(om - nm));
    m = nm;
  }
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  if (lane == 0) { red_m[wp] = m; red_s[wp] = sum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = -INFINITY;
    for (int i = 0; i < XT / 32; ++i) M = fmaxf(M, red_m[i]);
    float S = 0.f;
    for (int i = 0; i < XT / 32; ++i)
      if (red_m[i] != -INFINITY) S += red_s[i] * exp2f(red_m[i] - M);
    const float lse = (M + log2f(S)) * kLn2F;
    const int64_t label = reinterpret_cast<const int64_t *>(p.labels)[row];
    reinterpret_cast<float *>(p.lse)[row] = lse;
    float loss = 0.f;
    if (label != p.ignore_index && label >= 0 && label < V) loss = lse - tof(x[label]);
    reinterpret_cast<float *>(p.loss)[row] = loss;
  }
}

template <typename T>
__global__ void __launch_bounds__(XT) xent_bwd_kernel(const b200_xent_args p) {
  const int64_t row = blockIdx.x;
  const T *x = reinterpret_cast<const T *>(p.logits) + row * p.logits_rs;
  T *dx = reinterpret_cast<T *>(p.dlogits) + row * p.dlogits_rs;
  const int V = p.cols;
  const int64_t label = reinterpret_cast<const int64_t *>(p.labels)[row];
  const bool counted = label != p.ignore_index && label >= 0 && label < V;
  const float scale = counted ? reinterpret_cast<const float *>(p.scale)[0] : 0.f;
  const float off = reinterpret_cast<const float *>(p.lse)[row] * kLog2eF;
  const bool vec = al16(x) && al16(dx) && (V % 8 == 0);
  if (vec) {
    for (int c = threadIdx.x * 8; c < V; c += XT * 8) {
      float v[8];
      if (counted) {
        ldv<T>(x + c, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (exp2f(fmaf(v[i], kLog2eF, -off)) - ((int64_t)(c + i) == label ? 1.f : 0.f)) * scale;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      stv<T>(dx + c, v);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += XT) {
      float v = 0.f;
      if (counted) v = (exp2f(fmaf(tof(x[c]), kLog2eF, -off)) - ((int64_t)c == label ? 1.f : 0.f)) * scale;
      dx[c] = fromf<T>(v);
    }
  }
}

int check_xent(const b200_xent_args &a, bool bwd) {
  B200_REQUIRE(a.logits && a.labels && a.lse, B200_ERR_NULL, "xent: logits, labels and lse must be non-null");
  B200_REQUIRE(a.rows > 0 && a.cols > 0 && a.rows < (int64_t(1) << 31), B200_ERR_SHAPE, "xent: sizes must be positive");
  B200_REQUIRE(a.dtype == B200_F32 || a.dtype == B200_F16 || a.dtype == B200_BF16, B200_ERR_DTYPE, "xent: unknown dtype");
  if (!bwd) B200_REQUIRE(a.loss, B200_ERR_NULL, "xent_fwd: loss must be non-null");
  else B200_REQUIRE(a.dlogits && a.scale, B200_ERR_NULL, "xent_bwd: dlogits and scale must be non-null");
  return 0;
}

int check_conv(const b200_conv1d_args &a, bool bwd, bool update) {
  B200_REQUIRE(a.x && a.weight && (bwd || a.out), B200_ERR_NULL, "conv1d: x, weight, out must be non-null");
  B200_REQUIRE(a.batch > 0 && a.dim > 0 && (update || a.seqlen > 0), B200_ERR_SHAPE, "conv1d: sizes must be positive");
  B200_REQUIRE(a.width >= 2 && a.width <= MAXW, B200_ERR_SHAPE, "conv1d: width must be 2, 3 or 4 (got %d)", a.width);
  B200_REQUIRE(a.dtype == B200_F32 || a.dtype == B200_F16 || a.dtype == B200_BF16, B200_ERR_DTYPE, "conv1d: unknown dtype");
  if (update) {
    B200_REQUIRE(a.state, B200_ERR_NULL, "conv1d_update: state must be non-null");
    return 0;
  }
  if (bwd) {
    B200_REQUIRE(a.dout && a.dx && a.dweight, B200_ERR_NULL, "conv1d_bwd: dout, dx, dweight must be non-null");
    B200_REQUIRE(!a.bias || a.dbias, B200_ERR_NULL, "conv1d_bwd: dbias is required when bias is given");
  }
  B200_REQUIRE((int64_t)a.batch * ((a.seqlen + CVT * CVE - 1) / (CVT * CVE)) < (int64_t(1) << 31), B200_ERR_SHAPE,
               "conv1d: too many (batch, block) items per channel");
  return 0;
}

// grid of the convolution kernels: a column of CTAs per channel, as many per channel as it takes
// to put about two CTAs on every resident slot (8 per SM), and never more than the channel has items
dim3 conv_grid(const b200_conv1d_args &a) {
  const int tpr = conv_tpr(a.seqlen), rpi = CVT / tpr;
  const int64_t nblk = (a.seqlen + tpr * CVE - 1) / (tpr * CVE), items = (int64_t)((a.batch + rpi - 1) / rpi) * nblk;
  const int64_t slots = (int64_t)sm_count_current() * 8;
  int64_t gy = (2 * slots + a.dim - 1) / a.dim;
  gy = gy < 1 ? 1 : (gy > items ? items : gy);
  if (gy > 65535) gy = 65535;
  return dim3((unsigned)a.dim, (unsigned)gy);
}

int check_norm(const b200_rmsnorm_args &a, bool bwd) {
  B200_REQUIRE(a.weight && a.rows > 0 && a.cols > 0, B200_ERR_NULL, "rmsnorm: weight must be non-null, sizes positive");
  B200_REQUIRE(a.cols % 8 == 0 && a.cols <= MAXCOLS, B200_ERR_SHAPE,
               "rmsnorm: the row length must be a multiple of 8 and at most %d (got %d)", MAXCOLS, a.cols);
  B200_REQUIRE(a.dtype == B200_F32 || a.dtype == B200_F16 || a.dtype == B200_BF16, B200_ERR_DTYPE, "rmsnorm: unknown dtype");
  B200_REQUIRE(a.residual_dtype == a.dtype || a.residual_dtype == B200_F32, B200_ERR_DTYPE,
               "rmsnorm: the residual is kept in the activation dtype or in float32");
  if (!bwd) {
    B200_REQUIRE(a.x && a.y, B200_ERR_NULL, "rmsnorm_fwd: x and y must be non-null");
  } else {
    B200_REQUIRE(a.dy && a.dx && a.dweight && a.rstd && a.residual_out, B200_ERR_NULL,
                 "rmsnorm_bwd: dy, dx, dweight, rstd and residual_out (the normalised input) must be non-null");
  }
  return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

#define DISPATCH_T(dt, CALL)                         \
  if ((dt) == B200_F32) { using T = float; CALL; }   \
  else if ((dt) == B200_BF16) { using T = __nv_bfloat16; CALL; } \
  else { using T = __half; CALL; }

extern "C" {

int b200_conv1d_fwd(const b200_conv1d_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "conv1d_fwd: null argument block");
  if (int e = check_conv(*args, false, false)) return e;
  const dim3 grid = conv_grid(*args);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH_T(args->dtype, (conv1d_fwd_kernel<T><<<grid, CVT, 0, st>>>(*args)));
  return launch_status();
}

int b200_conv1d_bwd(const b200_conv1d_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "conv1d_bwd: null argument block");
  if (int e = check_conv(*args, true, false)) return e;
  const dim3 grid = conv_grid(*args);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH_T(args->dtype, (conv1d_bwd_kernel<T><<<grid, CVT, 0, st>>>(*args)));
  return launch_status();
}

int b200_conv1d_update(const b200_conv1d_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "conv1d_update: null argument block");
  if (int e = check_conv(*args, false, true)) return e;
  const int64_t n = (int64_t)args->batch * args->dim;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH_T(args->dtype, (conv1d_update_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(*args)));
  return launch_status();
}

// The backward adds a per-CTA partial of dweight with one atomic per column: fewer, longer-lived
// CTAs keep those atomics (all CTAs hit the same `cols` addresses) off the critical path.
#define NORM_LAUNCH(KERNEL, R_, NT_, NV_)                                                                    \
  do {                                                                                                       \
    const int64_t want = (int64_t)sm_count_current() * (is_bwd ? 4 : 2048 / NT_);                            \
    const unsigned grid = (unsigned)(args->rows < want ? args->rows : want);                                 \
    DISPATCH_T(args->dtype, (KERNEL<T, R_, NT_, NV_><<<grid, NT_, 0, st>>>(*args)));                          \
  } while (0)
#define NORM_SHAPES(KERNEL, R_)                                                \
  do {                                                                         \
    if (args->cols <= 1024) NORM_LAUNCH(KERNEL, R_, 128, 1);                   \
    else if (args->cols <= 2048) NORM_LAUNCH(KERNEL, R_, 256, 1);              \
    else NORM_LAUNCH(KERNEL, R_, 256, 2);                                      \
  } while (0)

int b200_rmsnorm_fwd(const b200_rmsnorm_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "rmsnorm_fwd: null argument block");
  if (int e = check_norm(*args, false)) return e;
  constexpr bool is_bwd = false;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (args->residual_dtype == B200_F32 && args->dtype != B200_F32) NORM_SHAPES(rmsnorm_fwd_kernel, float);
  else NORM_SHAPES(rmsnorm_fwd_kernel, T);
  return launch_status();
}

#define NORM_WARP_LAUNCH(R_, NV_)                                                                        \
  do {                                                                                                  \
    DISPATCH_T(args->dtype, (rmsnorm_bwd_warp_kernel<T, R_, NV_><<<grid, NWT, 0, st>>>(*args)));         \
  } while (0)
#define NORM_WARP_SHAPES(R_)                              \
  do {                                                    \
    if (args->cols <= 256) NORM_WARP_LAUNCH(R_, 1);       \
    else if (args->cols <= 512) NORM_WARP_LAUNCH(R_, 2);  \
    else if (args->cols <= 768) NORM_WARP_LAUNCH(R_, 3);  \
    else NORM_WARP_LAUNCH(R_, 4);                         \
  } while (0)

int b200_rmsnorm_bwd(const b200_rmsnorm_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "rmsnorm_bwd: null argument block");
  if (int e = check_norm(*args, true)) return e;
  constexpr bool is_bwd = true;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (args->cols <= 1024) {
    // warp per row: two CTAs of 8 warps per SM, fewer when there are fewer rows than warps
    const int64_t want = (int64_t)sm_count_current() * 2, need = (args->rows + NWT / 32 - 1) / (NWT / 32);
    const unsigned grid = (unsigned)(need < want ? need : want);
    if (args->residual_dtype == B200_F32 && args->dtype != B200_F32) NORM_WARP_SHAPES(float);
    else NORM_WARP_SHAPES(T);
    return launch_status();
  }
  if (args->residual_dtype == B200_F32 && args->dtype != B200_F32) NORM_SHAPES(rmsnorm_bwd_kernel, float);
  else NORM_SHAPES(rmsnorm_bwd_kernel, T);
  return launch_status();
}

int b200_xent_fwd(const b200_xent_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "xent_fwd: null argument block");
  if (int e = check_xent(*args, false)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH_T(args->dtype, (xent_fwd_kernel<T><<<(unsigned)args->rows, XT, 0, st>>>(*args)));
  return launch_status();
}

int b200_xent_bwd(const b200_xent_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "xent_bwd: null argument block");
  if (int e = check_xent(*args, true)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  DISPATCH_T(args->dtype, (xent_bwd_kernel<T><<<(unsigned)args->rows, XT, 0, st>>>(*args)));
  return launch_status();
}

}  // extern "C"
