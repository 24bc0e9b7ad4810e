// S4 structured kernels for sm_100a: symmetric Cauchy multiply and log-Vandermonde
// multiply, forward and backward.
//
// Math (csrc/s4/cauchy_cuda.cu:68-79,144-170,211-331 of lrnnx), n = half spectrum:
//   cauchy  out[b,l] = sum_n v/(z_l - w) + conj(v)/(z_l - conj(w))
//           dv[b,n]  = sum_l dout/(conj(z) - conj(w)) + conj(dout)/(z - conj(w))
//           dw[b,n]  = conj(v) sum_l dout/(conj(z) - conj(w))^2 + conj(dout)/(z - conj(w))^2
//   vand    out[b,l] = 2 Re sum_n v exp(x l)
//           dv[b,n]  = 2 sum_l dout conj(exp(x l));  dx[b,n] = 2 conj(v) sum_l dout l conj(exp(x l))
//
// These kernels are bound by the fp32 pipe (two complex reciprocals, or one complex
// exponential, per (b, l, n)), not by memory.  Forward: one thread owns FL output
// positions and loops over n with (v, w) broadcast from shared memory, so there is no
// cross-thread reduction.  Backward: a CTA owns (batch row, tile of TN poles, chunk of
// the sequence); threads stride over the chunk with TN complex accumulators each; CTA
// partials go to a scratch buffer and a second kernel folds the chunks in order.
#include "common.cuh"
#include <atomic>
#include "dispatch.h"

namespace b200 {
namespace {

constexpr int FT = 256;       // forward threads
constexpr int FL = 2;         // output positions per thread (Cauchy)
constexpr int VFL = 8;        // output positions per thread (Vandermonde), FT apart
constexpr int NMAX_SMEM = 1024;
constexpr int BTT = 256;      // backward threads
constexpr int TN = 4;         // poles per backward CTA
constexpr int BWARPS_ = BTT / 32;

// 1 / d with the SFU reciprocal (max. error 1 ulp) instead of an IEEE division: the two
// reciprocals per (row, frequency, pole) are the kernels' dominant cost.
__device__ __forceinline__ cf crecip(cf d) {
  float inv;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(d.re * d.re + d.im * d.im));
  return cf(d.re * inv, -d.im * inv);
}

__global__ void __launch_bounds__(FT) cauchy_fwd_kernel(const cf *__restrict__ v, const cf *__restrict__ z,
                                                        const cf *__restrict__ w, cf *__restrict__ out, int n, int L) {
  __shared__ float4 vw[NMAX_SMEM];
  const int b = blockIdx.y;
  const int l0 = blockIdx.x * FT * FL + threadIdx.x;
  cf zz[FL], acc[FL];
#pragma unroll
  for (int j = 0; j < FL; ++j) {
    const int l = l0 + j * FT;
    zz[j] = l < L ? z[l] : cf(2.f, 0.f);
    acc[j] = cf(0.f, 0.f);
  }
  for (int nb = 0; nb < n; nb += NMAX_SMEM) {
    const int cnt = min(NMAX_SMEM, n - nb);
    __syncthreads();
    for (int i = threadIdx.x; i < cnt; i += FT) {
      const cf vv = v[(int64_t)b * n + nb + i], ww = w[(int64_t)b * n + nb + i];
      vw[i] = make_float4(vv.re, vv.im, ww.re, ww.im);
    }
    __syncthreads();
#pragma unroll 4
    for (int i = 0; i < cnt; ++i) {
      const float4 t = vw[i];
      const cf vv(t.x, t.y), ww(t.z, t.w);
#pragma unroll
      for (int j = 0; j < FL; ++j) {
        acc[j] = acc[j] + vv * crecip(zz[j] - ww) + conj(vv) * crecip(zz[j] - conj(ww));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < FL; ++j) {
    const int l = l0 + j * FT;
    if (l < L) out[(int64_t)b * L + l] = acc[j];
  }
}

__global__ void __launch_bounds__(FT) vand_fwd_kernel(const cf *__restrict__ v, const cf *__restrict__ x,
                                                      float *__restrict__ out, int n, int L) {
  // A thread owns VFL positions l0, l0 + FT, ...: exp(x l) is evaluated exactly at l0 and advanced
  // by the per-pole constant exp(x FT) (a complex multiply instead of an exp and a sin/cos per term).
  __shared__ float4 vx[NMAX_SMEM];
  __shared__ float2 wstep[NMAX_SMEM];
  const int b = blockIdx.y;
  const int l0 = blockIdx.x * FT * VFL + threadIdx.x;
  const float lf = (float)l0;
  float acc[VFL];
#pragma unroll
  for (int j = 0; j < VFL; ++j) acc[j] = 0.f;
  for (int nb = 0; nb < n; nb += NMAX_SMEM) {
    const int cnt = min(NMAX_SMEM, n - nb);
    __syncthreads();
    for (int i = threadIdx.x; i < cnt; i += FT) {
      const cf vv = v[(int64_t)b * n + nb + i], xx = x[(int64_t)b * n + nb + i];
      vx[i] = make_float4(vv.re, vv.im, xx.re, xx.im);
      const cf w = cexp(xx * (float)FT);
      wstep[i] = make_float2(w.re, w.im);
    }
    __syncthreads();
#pragma unroll 2
    for (int i = 0; i < cnt; ++i) {
      const float4 t = vx[i];
      const float2 ws = wstep[i];
      const cf xx(t.z, t.w), W(ws.x, ws.y);
      cf E = cexp(xx * lf) * cf(t.x, t.y);      // v exp(x l0)
#pragma unroll
      for (int j = 0; j < VFL; ++j) {
        acc[j] += E.re;
        E = E * W;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VFL; ++j) {
    const int l = l0 + j * FT;
    if (l < L) out[(int64_t)b * L + l] = 2.f * acc[j];
  }
}

// Partial sums of one (batch row, pole tile, sequence chunk).  scratch layout:
// [batch][n][n_chunks][2] complex (first: dv partial, second: dw / dx partial).
template <bool VAND>
__global__ void __launch_bounds__(BTT) s4_bwd_partial_kernel(const cf *__restrict__ z, const cf *__restrict__ w,
                                                             const void *__restrict__ dout_, cf *__restrict__ scratch,
                                                             int n, int L, int l_chunk, int n_chunks) {
  __shared__ cf red[2 * TN][BWARPS_];
  const int b = blockIdx.z, chunk = blockIdx.y, n0 = blockIdx.x * TN;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  cf wn[TN];
#pragma unroll
  for (int k = 0; k < TN; ++k) wn[k] = (n0 + k < n) ? w[(int64_t)b * n + n0 + k] : cf(3.f, 3.f);
  cf a1[TN], a2[TN];
#pragma unroll
  for (int k = 0; k < TN; ++k) { a1[k] = cf(0.f, 0.f); a2[k] = cf(0.f, 0.f); }
  const int lbeg = chunk * l_chunk, lend = min(L, lbeg + l_chunk);
  // Vandermonde: exp(w l) advanced by the per-pole constant exp(w BTT) between the positions of
  // a thread (BTT apart), re-evaluated exactly every 16 positions
  cf Ek[TN], Wk[TN];
  if constexpr (VAND) {
#pragma unroll
    for (int k = 0; k < TN; ++k) Wk[k] = cexp(wn[k] * (float)BTT);
  }
  int iter = 0;
  for (int l = lbeg + threadIdx.x; l < lend; l += BTT, ++iter) {
    if constexpr (!VAND) {
      const cf d = reinterpret_cast<const cf *>(dout_)[(int64_t)b * L + l];
      const cf zl = z[l];
#pragma unroll
      for (int k = 0; k < TN; ++k) {
        const cf wc = conj(wn[k]);
        const cf r1 = crecip(conj(zl) - wc), r2 = crecip(zl - wc);
        a1[k] = a1[k] + d * r1 + conj(d) * r2;
        a2[k] = a2[k] + d * (r1 * r1) + conj(d) * (r2 * r2);
      }
    } else {
      const float d = reinterpret_cast<const float *>(dout_)[(int64_t)b * L + l];
      const float lf = (float)l;
      const bool exact = (iter & 15) == 0;
#pragma unroll
      for (int k = 0; k < TN; ++k) {
        Ek[k] = exact ? cexp(wn[k] * lf) : Ek[k] * Wk[k];
        const cf e = conj(Ek[k]) * d;
        a1[k] = a1[k] + e;
        a2[k] = a2[k] + e * lf;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < TN; ++k) {
    a1[k] = warp_sum(a1[k]);
    a2[k] = warp_sum(a2[k]);
    if (lane == 0) { red[2 * k][warp] = a1[k]; red[2 * k + 1][warp] = a2[k]; }
  }
  __syncthreads();
  if (threadIdx.x < 2 * TN) {
    cf s = cf(0.f, 0.f);
#pragma unroll
    for (int wv = 0; wv < BWARPS_; ++wv) s = s + red[threadIdx.x][wv];
    const int k = threadIdx.x >> 1, which = threadIdx.x & 1;
    if (n0 + k < n) scratch[(((int64_t)b * n + n0 + k) * n_chunks + chunk) * 2 + which] = s;
  }
}

template <bool VAND>
__global__ void s4_bwd_fold_kernel(const cf *__restrict__ v, const cf *__restrict__ scratch, cf *__restrict__ dv,
                                   cf *__restrict__ dw, int64_t total, int n_chunks) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  cf s1 = cf(0.f, 0.f), s2 = cf(0.f, 0.f);
  for (int c = 0; c < n_chunks; ++c) {
    s1 = s1 + scratch[(i * n_chunks + c) * 2];
    s2 = s2 + scratch[(i * n_chunks + c) * 2 + 1];
  }
  if (VAND) { s1 = s1 * 2.f; s2 = s2 * 2.f; }
  dv[i] = s1;
  dw[i] = conj(v[i]) * s2;
}

int chunking(int batch, int n, int L, int &l_chunk) {
  const int64_t tiles = (int64_t)batch * ((n + TN - 1) / TN);
  int want = (int)((sm_count_current() * 4 + tiles - 1) / tiles);          // enough CTAs to fill the GPU
  const int max_chunks = (L + 1023) / 1024;                 // at least 1024 positions per CTA
  if (want > max_chunks) want = max_chunks;
  if (want < 1) want = 1;
  l_chunk = (L + want - 1) / want;
  l_chunk = ((l_chunk + BTT - 1) / BTT) * BTT;
  return (L + l_chunk - 1) / l_chunk;
}

int check(const b200_s4_args &a, bool bwd, bool vand) {
  B200_REQUIRE(a.v && a.w && (vand || a.z), B200_ERR_NULL, "s4: v, z, w must be non-null");
  B200_REQUIRE(a.batch > 0 && a.n > 0 && a.seqlen > 0, B200_ERR_SHAPE, "s4: batch, n, seqlen must be positive");
  B200_REQUIRE(a.batch <= 65535, B200_ERR_SHAPE, "s4: batch must be <= 65535");
  if (!bwd) {
    B200_REQUIRE(a.out, B200_ERR_NULL, "s4: out must be non-null");
  } else {
    B200_REQUIRE(a.dout && a.dv && a.dw && a.scratch, B200_ERR_NULL, "s4: dout, dv, dw, scratch must be non-null");
    B200_REQUIRE(a.scratch_bytes >= b200_s4_bwd_scratch_bytes(a.batch, a.n, a.seqlen), B200_ERR_SHAPE,
                 "s4: scratch too small (%lld bytes, need %lld)", (long long)a.scratch_bytes,
                 (long long)b200_s4_bwd_scratch_bytes(a.batch, a.n, a.seqlen));
  }
  return 0;
}

template <bool VAND> int run_bwd(const b200_s4_args &a, cudaStream_t st) {
  int l_chunk;
  const int n_chunks = chunking(a.batch, a.n, a.seqlen, l_chunk);
  dim3 grid((a.n + TN - 1) / TN, n_chunks, a.batch);
  s4_bwd_partial_kernel<VAND><<<grid, BTT, 0, st>>>(
      reinterpret_cast<const cf *>(a.z), reinterpret_cast<const cf *>(a.w), a.dout,
      reinterpret_cast<cf *>(a.scratch), a.n, a.seqlen, l_chunk, n_chunks);
  if (int e = launch_status()) return e;
  const int64_t total = (int64_t)a.batch * a.n;
  s4_bwd_fold_kernel<VAND><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const cf *>(a.v), reinterpret_cast<const cf *>(a.scratch), reinterpret_cast<cf *>(a.dv),
      reinterpret_cast<cf *>(a.dw), total, n_chunks);
  return launch_status();
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int64_t b200_s4_bwd_scratch_bytes(int32_t batch, int32_t n, int32_t seqlen) {
  if (batch <= 0 || n <= 0 || seqlen <= 0) return 0;
  int l_chunk;
  const int n_chunks = chunking(batch, n, seqlen, l_chunk);
  return (int64_t)batch * n * n_chunks * 2 * (int64_t)sizeof(cf);
}

int b200_cauchy_fwd(const b200_s4_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "cauchy_fwd: null argument block");
  if (int e = check(*args, false, false)) return e;
  dim3 grid((args->seqlen + FT * FL - 1) / (FT * FL), args->batch);
  cauchy_fwd_kernel<<<grid, FT, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const cf *>(args->v), reinterpret_cast<const cf *>(args->z),
      reinterpret_cast<const cf *>(args->w), reinterpret_cast<cf *>(args->out), args->n, args->seqlen);
  return launch_status();
}

int b200_cauchy_bwd(const b200_s4_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "cauchy_bwd: null argument block");
  if (int e = check(*args, true, false)) return e;
  return run_bwd<false>(*args, reinterpret_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Cauchy backward without any allocation by anybody.
//
// Some users of this library cannot hand it device memory beyond the tensors of
// the call: a plain C or C++ host that links the ABI without a framework
// allocator, or a serving loop that runs under a frozen memory budget where a
// cudaMalloc (which may synchronise the device or fail late) is not acceptable.
// For them the per-chunk partial sums live in a fixed array inside the library
// image.  Every GPU that loads the library holds the array until the process
// exits; its size bounds the problem size.
static __device__ __align__(256) unsigned char g_cauchy_static_scratch[B200_CAUCHY_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle; the device address has to be
// asked for, per device, with that device current.
static std::atomic<void *> g_static_scratch_ptr[64];

static int static_scratch_for_current_device(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_error("cudaGetDevice: %s", cudaGetErrorString(e)); return (int)e; }
  B200_REQUIRE(dev >= 0 && dev < 64, B200_ERR_UNSUPPORTED, "cauchy_bwd_static: device ordinal %d not supported", dev);
  void *ptr = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    e = cudaGetSymbolAddress(&ptr, g_cauchy_static_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : B200_ERR_UNSUPPORTED;
    }
    g_static_scratch_ptr[dev].store(ptr, std::memory_order_release);   // same value from every thread
  }
  *out = ptr;
  return 0;
}

int b200_cauchy_bwd_static(const b200_s4_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "cauchy_bwd_static: null argument block");
  const int64_t need = b200_s4_bwd_scratch_bytes(args->batch, args->n, args->seqlen);
  B200_REQUIRE(need <= (int64_t)B200_CAUCHY_STATIC_SCRATCH_BYTES, B200_ERR_TOO_LARGE,
               "cauchy_bwd_static: this problem needs %lld bytes of scratch, the built-in area holds %lld; "
               "use b200_cauchy_bwd with caller-provided scratch",
               (long long)need, (long long)B200_CAUCHY_STATIC_SCRATCH_BYTES);
  b200_s4_args a = *args;
  void *ptr = nullptr;
  if (int e = static_scratch_for_current_device(&ptr)) return e;
  a.scratch = ptr;
  a.scratch_bytes = B200_CAUCHY_STATIC_SCRATCH_BYTES;
  if (int e = check(a, true, false)) return e;
  // Nothing in the area has to start at zero: the first kernel writes every partial-sum slot
  // that the second kernel reads.
  return run_bwd<false>(a, reinterpret_cast<cudaStream_t>(stream));
}

int b200_vand_fwd(const b200_s4_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "vand_fwd: null argument block");
  if (int e = check(*args, false, true)) return e;
  dim3 grid((args->seqlen + FT * VFL - 1) / (FT * VFL), args->batch);
  vand_fwd_kernel<<<grid, FT, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const cf *>(args->v), reinterpret_cast<const cf *>(args->w),
      reinterpret_cast<float *>(args->out), args->n, args->seqlen);
  return launch_status();
}

int b200_vand_bwd(const b200_s4_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "vand_bwd: null argument block");
  if (int e = check(*args, true, true)) return e;
  return run_bwd<true>(*args, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
