// Sequence-parallel fix-up pass of the selective scan (no counterpart in lrnnx, which is
// single-GPU).  A rank that scanned its slice of the sequence from a zero state receives the
// state h_in that actually enters the slice (folded from the summaries of the earlier ranks)
// and adds what that state contributes:
//     out[t]   += sum_n C[t, n] * exp(A_n * cum_t) * h_in[n],   cum_t = sum_{k <= t} delta'_k
//     x[c].h   += x[c].P * h_in,      x[c].P *= p_in            (checkpoints of the slice)
// and recomputes out_z = out * silu(z) where out changed.  delta' is delta after bias and
// softplus.  Valid for real A with a = exp(delta' A) ("mamba", and "zoh"/"dirac" without
// deltaA, whose transition is the same) and variable C.
//
// One warp per (batch, channel) row, one timestep per lane, 32 steps per iteration: delta is
// read coalesced, its running sum is a warp scan plus a carried total, and C[n, t] is a
// coalesced read per state.  The contribution decays like exp(A cum_t); a row stops as soon
// as its slowest-decaying state is below 2^-32 (fp32 output) or 2^-14 (16-bit output) of its
// entry value — far under the output's own rounding —, so the pass usually
// touches only the first few hundred steps of a slice instead of all of it.
#include "common.cuh"
#include "dispatch.h"

namespace b200 {
namespace {

constexpr int SPW = 4;   // rows (warps) per CTA

__global__ void __launch_bounds__(SPW * 32) selscan_fixup_kernel(const b200_selscan_fixup_args q) {
  const b200_selscan_fwd_args &p = q.f;
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * SPW + warp;
  if (row >= (int64_t)p.batch * p.dim) return;
  // blockIdx.y = segment of the slice; segment s covers [s*seg_len, (s+1)*seg_len)
  const int nseg = q.n_segments > 1 ? q.n_segments : 1;
  const int seg = (int)blockIdx.y;
  const int t_begin = nseg > 1 ? seg * q.seg_len : 0;
  const int t_end = nseg > 1 ? min(p.seqlen, t_begin + q.seg_len) : p.seqlen;
  if (t_begin >= t_end) return;
  const int b = (int)(row / p.dim), d = (int)(row % p.dim);
  const int g = d / (p.dim / p.n_groups);
  const int N = p.dstate, dt = p.dtype;
  const int n_chunks = (p.seqlen + kChunk - 1) / kChunk;
  float *A2 = sm + warp * 2 * N;     // A * log2(e)
  float *hin = A2 + N;
  const float *A = reinterpret_cast<const float *>(p.A) + (int64_t)d * p.A_ds;
  const float *hsrc = reinterpret_cast<const float *>(q.h_in) + ((int64_t)seg * p.batch * p.dim + row) * N;
  const float *psrc = reinterpret_cast<const float *>(q.p_in) + ((int64_t)seg * p.batch * p.dim + row) * N;
  float amax = -INFINITY;            // slowest decay of the row
  float hmax = 0.f;
  bool bad = false;                  // a non-finite incoming state: fmaxf drops NaN, so it is tracked apart
  for (int n = lane; n < N; n += 32) {
    const float a = A[(int64_t)n * p.A_ns];
    A2[n] = a * kLog2e;
    hin[n] = hsrc[n];
    amax = fmaxf(amax, a * kLog2e);
    hmax = fmaxf(hmax, fabsf(hsrc[n]));
    bad |= !(fabsf(hsrc[n]) <= 3.4e38f);
  }
  bad = __any_sync(0xffffffffu, bad);
  hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, 16));
  hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, 8));
  hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, 4));
  hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, 2));
  hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, 1));
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  __syncwarp();
  // checkpoints: state and product entries of every chunk of the slice
  float *xrow = reinterpret_cast<float *>(p.x) + row * n_chunks * 2 * N;
  const int c_begin = t_begin / kChunk, c_end = (t_end + kChunk - 1) / kChunk;
  for (int i = lane + c_begin * N; i < c_end * N; i += 32) {
    const int c = i / N, n = i % N;
    const float P = xrow[(int64_t)c * 2 * N + 2 * n];
    xrow[(int64_t)c * 2 * N + 2 * n + 1] += P * hin[n];
    xrow[(int64_t)c * 2 * N + 2 * n] = P * psrc[n];
  }
  const int64_t dl_off = (int64_t)b * p.delta_bs + (int64_t)d * p.delta_ds;
  const int64_t o_off = (int64_t)b * p.out_bs + (int64_t)d * p.out_ds;
  const int64_t z_off = (int64_t)b * p.z_bs + (int64_t)d * p.z_ds;
  const int64_t oz_off = (int64_t)b * p.out_z_bs + (int64_t)d * p.out_z_ds;
  const int64_t c_off = (int64_t)b * p.C_bs + (int64_t)g * p.C_gs;
  const float bias = p.delta_bias ? reinterpret_cast<const float *>(p.delta_bias)[d] : 0.f;
  float carry = 0.f;                 // sum of delta' over the steps already processed
  // a NaN or infinite state reaches every later step of the unsplit scan: no early exit then
  const float cutoff = bad ? -INFINITY : (dt == B200_F32 ? -32.f : -14.f);
  if (hmax == 0.f && !bad) return;   // nothing enters this segment (first segment of the first rank)
  const int L = t_end;
  constexpr int K = 4;               // 32-step sub-blocks per iteration (independent loads and scans in flight)
  for (int t0 = t_begin; t0 < L; t0 += 32 * K) {
    if (amax * carry < cutoff) break;   // every state has decayed away (carry is warp-uniform)
    float cum[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int t = t0 + k * 32 + lane;
      float dv = 0.f;
      if (t < L) {
        dv = ld_act(p.delta, dt, dl_off + t) + bias;
        if (p.delta_softplus) dv = softplus20(dv);
      }
      cum[k] = dv;
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const float v = __shfl_up_sync(0xffffffffu, cum[k], off);
        if (lane >= off) cum[k] += v;
      }
    }
    const float carry_before = carry;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      cum[k] += carry;
      carry = __shfl_sync(0xffffffffu, cum[k], 31);
    }
    float acc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) acc[k] = 0.f;
#pragma unroll 4
    for (int n = 0; n < N; ++n) {
      if (A2[n] * carry_before < cutoff) continue;   // this state has already decayed away (warp-uniform)
      const float a2 = A2[n], hn = hin[n];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const int t = t0 + k * 32 + lane;
        const float cv = t < L ? ld_act(p.C, dt, c_off + (int64_t)n * p.C_ns + t) : 0.f;
        acc[k] = fmaf(cv * exp2f(a2 * cum[k]), hn, acc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int t = t0 + k * 32 + lane;
      if (t < L) {
        // out holds the rounded zero-state result; the correction is added in fp32
        const float o = ld_act(p.out, dt, o_off + t) + acc[k];
        st_act(p.out, dt, o_off + t, o);
        if (p.z) {
          const float zv = ld_act(p.z, dt, z_off + t);
          st_act(p.out_z, dt, oz_off + t, o * zv * sigmoidf_(zv));
        }
      }
    }
  }
}

// ---- vectorized variant: 8 consecutive timesteps per lane (256 per iteration), 16-byte typed
// loads and stores.  Needs 16-byte aligned rows, a sequence length and segment starts that are
// multiples of 8 — what the throughput forward kernel, the only producer of in-GPU segments,
// requires as well.
template <typename T> struct V8;
template <> struct V8<float> {
  __device__ static void load(const float *p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ static void store(float *p, const float (&v)[8]) {
    reinterpret_cast<float4 *>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct V8<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__nv_bfloat16 *p, const float (&v)[8]) {
    uint4 t;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = t;
  }
};
template <> struct V8<__half> {
  __device__ static void load(const __half *p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store(__half *p, const float (&v)[8]) {
    uint4 t;
    __half2 *h = reinterpret_cast<__half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = t;
  }
};

template <typename T>
__global__ void __launch_bounds__(SPW * 32) selscan_fixup_vec_kernel(const b200_selscan_fixup_args q) {
  const b200_selscan_fwd_args &p = q.f;
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * SPW + warp;
  if (row >= (int64_t)p.batch * p.dim) return;
  const int nseg = q.n_segments > 1 ? q.n_segments : 1;
  const int seg = (int)blockIdx.y;
  const int t_begin = nseg > 1 ? seg * q.seg_len : 0;
  const int L = nseg > 1 ? min(p.seqlen, t_begin + q.seg_len) : p.seqlen;
  if (t_begin >= L) return;
  const int b = (int)(row / p.dim), d = (int)(row % p.dim);
  const int g = d / (p.dim / p.n_groups);
  const int N = p.dstate;
  const int n_chunks = (p.seqlen + kChunk - 1) / kChunk;
  float *A2 = sm + warp * 2 * N;     // A * log2(e)
  float *hin = A2 + N;
  const float *A = reinterpret_cast<const float *>(p.A) + (int64_t)d * p.A_ds;
  const float *hsrc = reinterpret_cast<const float *>(q.h_in) + ((int64_t)seg * p.batch * p.dim + row) * N;
  const float *psrc = reinterpret_cast<const float *>(q.p_in) + ((int64_t)seg * p.batch * p.dim + row) * N;
  float amax = -INFINITY, hmax = 0.f;
  bool bad = false;                  // a non-finite incoming state: fmaxf drops NaN, so it is tracked apart
  for (int n = lane; n < N; n += 32) {
    const float a = A[(int64_t)n * p.A_ns];
    A2[n] = a * kLog2e;
    hin[n] = hsrc[n];
    amax = fmaxf(amax, a * kLog2e);
    hmax = fmaxf(hmax, fabsf(hsrc[n]));
    bad |= !(fabsf(hsrc[n]) <= 3.4e38f);
  }
  bad = __any_sync(0xffffffffu, bad);
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    hmax = fmaxf(hmax, __shfl_xor_sync(0xffffffffu, hmax, m));
  }
  __syncwarp();
  float *xrow = reinterpret_cast<float *>(p.x) + row * n_chunks * 2 * N;
  const int c_begin = t_begin / kChunk, c_end = (L + kChunk - 1) / kChunk;
  for (int i = lane + c_begin * N; i < c_end * N; i += 32) {
    const int c = i / N, n = i % N;
    const float P = xrow[(int64_t)c * 2 * N + 2 * n];
    xrow[(int64_t)c * 2 * N + 2 * n + 1] += P * hin[n];
    xrow[(int64_t)c * 2 * N + 2 * n] = P * psrc[n];
  }
  if (hmax == 0.f && !bad) return;   // nothing enters this segment
  const T *dl = reinterpret_cast<const T *>(p.delta) + (int64_t)b * p.delta_bs + (int64_t)d * p.delta_ds;
  const T *Cg = reinterpret_cast<const T *>(p.C) + (int64_t)b * p.C_bs + (int64_t)g * p.C_gs;
  T *out = reinterpret_cast<T *>(p.out) + (int64_t)b * p.out_bs + (int64_t)d * p.out_ds;
  const T *zr = p.z ? reinterpret_cast<const T *>(p.z) + (int64_t)b * p.z_bs + (int64_t)d * p.z_ds : nullptr;
  T *oz = p.z ? reinterpret_cast<T *>(p.out_z) + (int64_t)b * p.out_z_bs + (int64_t)d * p.out_z_ds : nullptr;
  const float bias = p.delta_bias ? reinterpret_cast<const float *>(p.delta_bias)[d] : 0.f;
  // a NaN or infinite state reaches every later step of the unsplit scan: no early exit then
  const float cutoff = bad ? -INFINITY : (sizeof(T) == 4 ? -32.f : -14.f);
  float carry = 0.f;                 // sum of delta' over the steps already processed (warp-uniform)
  for (int t0 = t_begin; t0 < L; t0 += 256) {
    if (amax * carry < cutoff) break;   // every state has decayed away
    const int t = t0 + lane * 8;
    const bool live = t < L;            // L and t are multiples of 8: a lane's 8 steps are all valid or all past the end
    float cum[8];
    if (live) {
      V8<T>::load(dl + t, cum);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float dv = cum[i] + bias;
        if (p.delta_softplus) dv = softplus20(dv);
        cum[i] = dv;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) cum[i] = 0.f;
    }
#pragma unroll
    for (int i = 1; i < 8; ++i) cum[i] += cum[i - 1];
    float incl = cum[7];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    const float before = carry + incl - cum[7];      // delta' summed over everything before this lane
    const float carry_before = carry;
    carry += __shfl_sync(0xffffffffu, incl, 31);
#pragma unroll
    for (int i = 0; i < 8; ++i) cum[i] += before;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int n = 0; n < N; ++n) {
      const float a2 = A2[n];
      if (a2 * carry_before < cutoff) continue;      // this state has already decayed away (warp-uniform)
      if (live) {
        const float hn = hin[n];
        float cv[8];
        V8<T>::load(Cg + (int64_t)n * p.C_ns + t, cv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a2 * cum[i]));
          acc[i] = fmaf(cv[i] * e, hn, acc[i]);
        }
      }
    }
    if (live) {
      // out holds the rounded zero-state result; the correction is added in fp32
      float o[8];
      V8<T>::load(out + t, o);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += acc[i];
      V8<T>::store(out + t, o);
      if (zr) {
        float zv[8];
        V8<T>::load(zr + t, zv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] *= zv[i] * sigmoidf_(zv[i]);
        V8<T>::store(oz + t, o);
      }
    }
  }
}

// One thread per (batch, channel, state): sequential fold of the segments' (product, state)
// summaries, read from the last checkpoint entry of every segment.
__global__ void selscan_fold_kernel(const float *__restrict__ x, float *__restrict__ h_in, float *__restrict__ p_in,
                                    int64_t rows, int N, int n_chunks, int chunks_per_seg, int n_seg) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * N) return;
  const int64_t row = i / N;
  const int n = (int)(i % N);
  float h = 0.f, pr = 1.f;
  for (int s = 0; s < n_seg; ++s) {
    h_in[((int64_t)s * rows + row) * N + n] = h;
    p_in[((int64_t)s * rows + row) * N + n] = pr;
    const int last = min((s + 1) * chunks_per_seg, n_chunks) - 1;
    const float P = x[(row * n_chunks + last) * 2 * N + 2 * n];
    const float hs = x[(row * n_chunks + last) * 2 * N + 2 * n + 1];
    h = fmaf(P, h, hs);
    pr *= P;
  }
}

bool fixup_vec_ok(const b200_selscan_fixup_args &q) {
  const b200_selscan_fwd_args &a = q.f;
  const int es = a.dtype == B200_F32 ? 4 : 2;
  const int64_t m = 16 / es;
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (a.seqlen % 8 != 0 || (q.n_segments > 1 && q.seg_len % 8 != 0)) return false;
  if (!al(a.delta) || !al(a.C) || !al(a.out) || a.delta_bs % m || a.delta_ds % m || a.out_bs % m || a.out_ds % m ||
      a.C_bs % m || a.C_gs % m || a.C_ns % m)
    return false;
  if (a.z && (!al(a.z) || !al(a.out_z) || a.z_bs % m || a.z_ds % m || a.out_z_bs % m || a.out_z_ds % m)) return false;
  return true;
}

// Adjoint summary of a slice (the transposed map of the fix-up): G[n] = sum_t exp(A_n cum_t) C[t, n] dy_t
// with dy = dout * silu(z).  One warp per (batch, channel) row, one timestep per lane; per 32-step
// block the running sum of delta is a warp scan plus the carried total, every state's terms are
// summed over the lanes, and the row stops once its slowest-decaying state has fallen below 2^-40
// of its entry value (delta' >= 0 and A < 0 make the weights non-increasing; rows where that does
// not hold run to the end).
__global__ void __launch_bounds__(SPW * 32) selscan_adjsum_kernel(const b200_selscan_adjsum_args q) {
  const b200_selscan_fwd_args &p = q.f;
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * SPW + warp;
  if (row >= (int64_t)p.batch * p.dim) return;
  const int b = (int)(row / p.dim), d = (int)(row % p.dim);
  const int g = d / (p.dim / p.n_groups);
  const int N = p.dstate, dt = p.dtype, L = p.seqlen;
  float *A2 = sm + warp * 2 * N;
  float *acc = A2 + N;
  const float *A = reinterpret_cast<const float *>(p.A) + (int64_t)d * p.A_ds;
  float amax = -INFINITY;
  for (int n = lane; n < N; n += 32) {
    const float a = A[(int64_t)n * p.A_ns] * kLog2e;
    A2[n] = a;
    acc[n] = 0.f;
    amax = fmaxf(amax, a);
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  __syncwarp();
  const bool may_stop = p.delta_softplus && amax < 0.f;      // weights cannot grow again
  const int64_t dl_off = (int64_t)b * p.delta_bs + (int64_t)d * p.delta_ds;
  const int64_t z_off = (int64_t)b * p.z_bs + (int64_t)d * p.z_ds;
  const int64_t do_off = (int64_t)b * q.dout_bs + (int64_t)d * q.dout_ds;
  const int64_t c_off = (int64_t)b * p.C_bs + (int64_t)g * p.C_gs;
  const float bias = p.delta_bias ? reinterpret_cast<const float *>(p.delta_bias)[d] : 0.f;
  float carry = 0.f;
  for (int t0 = 0; t0 < L; t0 += 32) {
    if (may_stop && amax * carry < -40.f) break;
    const int t = t0 + lane;
    float dv = 0.f, dy = 0.f;
    if (t < L) {
      dv = ld_act(p.delta, dt, dl_off + t) + bias;
      if (p.delta_softplus) dv = softplus20(dv);
      dy = ld_act(q.dout, dt, do_off + t);
      if (p.z) {
        const float zv = ld_act(p.z, dt, z_off + t);
        dy *= zv * sigmoidf_(zv);
      }
    }
    float cum = dv;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, cum, off);
      if (lane >= off) cum += v;
    }
    cum += carry;
    carry = __shfl_sync(0xffffffffu, cum, 31);
    for (int n = 0; n < N; ++n) {
      const float cv = t < L ? ld_act(p.C, dt, c_off + (int64_t)n * p.C_ns + t) : 0.f;
      float term = cv * exp2f(A2[n] * cum) * dy;
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) term += __shfl_xor_sync(0xffffffffu, term, m);
      if (lane == 0) acc[n] += term;
    }
  }
  __syncwarp();
  float *G = reinterpret_cast<float *>(q.G) + row * N;
  for (int n = lane; n < N; n += 32) G[n] = acc[n];
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_selscan_fixup(const b200_selscan_fixup_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "selscan_fixup: null argument block");
  const b200_selscan_fwd_args &a = args->f;
  B200_REQUIRE(a.delta && a.A && a.C && a.out && a.x && args->h_in && args->p_in, B200_ERR_NULL,
               "selscan_fixup: delta, A, C, out, x, h_in, p_in must be non-null");
  B200_REQUIRE(!a.z || a.out_z, B200_ERR_NULL, "selscan_fixup: out_z is required when z is given");
  B200_REQUIRE(a.batch > 0 && a.dim > 0 && a.seqlen > 0 && a.dstate > 0 && a.dstate <= kMaxDState && a.n_groups >= 1 &&
                   a.dim % a.n_groups == 0,
               B200_ERR_SHAPE, "selscan_fixup: bad sizes");
  B200_REQUIRE(!a.is_complex && a.var_B && a.var_C && !a.deltaA &&
                   (a.method == B200_DISC_MAMBA || a.method == B200_DISC_ZOH || a.method == B200_DISC_DIRAC),
               B200_ERR_UNSUPPORTED,
               "selscan_fixup supports real A, variable B and C, no deltaA and the mamba / zoh / dirac transitions");
  const int64_t rows = (int64_t)a.batch * a.dim;
  const size_t smem = (size_t)SPW * 2 * a.dstate * sizeof(float);
  B200_REQUIRE(args->n_segments <= 1 || (args->seg_len > 0 && args->seg_len % kChunk == 0), B200_ERR_SHAPE,
               "selscan_fixup: seg_len must be a positive multiple of 2048 when n_segments > 1");
  const dim3 grid((unsigned)((rows + SPW - 1) / SPW), (unsigned)(args->n_segments > 1 ? args->n_segments : 1));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (fixup_vec_ok(*args)) {
    if (a.dtype == B200_F32) selscan_fixup_vec_kernel<float><<<grid, SPW * 32, smem, st>>>(*args);
    else if (a.dtype == B200_BF16) selscan_fixup_vec_kernel<__nv_bfloat16><<<grid, SPW * 32, smem, st>>>(*args);
    else selscan_fixup_vec_kernel<__half><<<grid, SPW * 32, smem, st>>>(*args);
  } else {
    selscan_fixup_kernel<<<grid, SPW * 32, smem, st>>>(*args);
  }
  return launch_status();
}

extern "C" int b200_selscan_fold(const b200_selscan_fixup_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "selscan_fold: null argument block");
  const b200_selscan_fwd_args &a = args->f;
  B200_REQUIRE(a.x && args->h_in && args->p_in, B200_ERR_NULL, "selscan_fold: x, h_in, p_in must be non-null");
  B200_REQUIRE(!a.is_complex, B200_ERR_UNSUPPORTED, "selscan_fold supports real A");
  B200_REQUIRE(a.batch > 0 && a.dim > 0 && a.seqlen > 0 && a.dstate > 0, B200_ERR_SHAPE, "selscan_fold: bad sizes");
  B200_REQUIRE(args->n_segments > 1 && args->seg_len > 0 && args->seg_len % kChunk == 0, B200_ERR_SHAPE,
               "selscan_fold: n_segments > 1 and a seg_len that is a positive multiple of 2048 are required");
  const int64_t rows = (int64_t)a.batch * a.dim;
  const int n_chunks = (a.seqlen + kChunk - 1) / kChunk;
  const int64_t total = rows * a.dstate;
  selscan_fold_kernel<<<(unsigned)((total + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float *>(a.x), reinterpret_cast<float *>(const_cast<void *>(args->h_in)),
      reinterpret_cast<float *>(const_cast<void *>(args->p_in)), rows, a.dstate, n_chunks, args->seg_len / kChunk,
      args->n_segments);
  return launch_status();
}

extern "C" int b200_selscan_adjoint_summary(const b200_selscan_adjsum_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "selscan_adjoint_summary: null argument block");
  const b200_selscan_fwd_args &a = args->f;
  B200_REQUIRE(a.delta && a.A && a.C && args->dout && args->G, B200_ERR_NULL,
               "selscan_adjoint_summary: delta, A, C, dout, G must be non-null");
  B200_REQUIRE(a.batch > 0 && a.dim > 0 && a.seqlen > 0 && a.dstate > 0 && a.dstate <= kMaxDState && a.n_groups >= 1 &&
                   a.dim % a.n_groups == 0,
               B200_ERR_SHAPE, "selscan_adjoint_summary: bad sizes");
  B200_REQUIRE(!a.is_complex && a.var_C && !a.deltaA &&
                   (a.method == B200_DISC_MAMBA || a.method == B200_DISC_ZOH || a.method == B200_DISC_DIRAC),
               B200_ERR_UNSUPPORTED,
               "selscan_adjoint_summary supports real A, variable C, no deltaA and the mamba / zoh / dirac transitions");
  const int64_t rows = (int64_t)a.batch * a.dim;
  const size_t smem = (size_t)SPW * 2 * a.dstate * sizeof(float);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  selscan_adjsum_kernel<<<(unsigned)((rows + SPW - 1) / SPW), SPW * 32, smem, st>>>(*args);
  return launch_status();
}
