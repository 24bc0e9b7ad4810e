// One-token selective state update (decode step) for sm_100a.
//
// Replaces the Triton kernel of lrnnx/ops/triton/selective_state_update.py:17-297:
//   dt' = softplus(dt + dt_bias)              (softplus only when requested, pass-through above 20)
//   a   = exp(A * dA)        for zoh / bilinear / dirac / mamba   (dA = deltaA if given else dt')
//         A ** dA            for rglru
//         1 - 1/(dt'^2 + 1/2) for s7
//   bb  = B (exp(A dt') - 1)/A | B dt'/(1 - A dt'/2) | B | B | B sqrt(1 - a^2) | B dt'
//         (zoh | bilinear | dirac | s7 | rglru | mamba)
//   state <- state * a + bb * x   (stored in the state's dtype, in place)
//   out = sum_n state * C (+ D x) (* z sigmoid(z))
//
// The step is bound by the state traffic (read + write of batch*dim*dstate
// elements).  A group of LPR lanes owns one (batch, head, channel) row; each lane
// moves VEC consecutive states with one 16-byte access when the state and A rows
// are dense, so a warp reads and writes whole 128-byte lines; the row sum is a
// shuffle reduction over the LPR lanes.  Strides (including 0 for broadcast
// dimensions) and per-tensor dtypes are honoured on every operand.
#include "common.cuh"
#include "dispatch.h"

namespace b200 {
namespace {

template <typename T> struct Vec16;   // 16-byte vector of state elements
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float v[4];
  __device__ void load(const float *p) { float4 t = *reinterpret_cast<const float4 *>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
  __device__ void store(float *p) const { *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  float v[8];
  __device__ void load(const __nv_bfloat16 *p) {
    uint4 t = *reinterpret_cast<const uint4 *>(p);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ void store(__nv_bfloat16 *p) const {
    uint4 t;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = t;
  }
};
template <> struct Vec16<__half> {
  static constexpr int N = 8;
  float v[8];
  __device__ void load(const __half *p) {
    uint4 t = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ void store(__half *p) const {
    uint4 t;
    __half2 *h = reinterpret_cast<__half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = t;
  }
};

struct RowScalars { float x, dt, dA, Dv, z; bool has_z; };   // generic kernel only

__device__ __forceinline__ void step_coef(int method, float A, float dt, float dA, float &a, float &kb) {
  // a: transition; kb: factor multiplying B (per state)
  if (method == B200_DISC_RGLRU) {
    a = expf(dA * logf(A));
    kb = sqrtf(1.f - a * a);
  } else if (method == B200_DISC_S7) {
    a = 1.f - 1.f / (dt * dt + 0.5f);
    kb = 1.f;
  } else {
    a = expf(A * dA);
    if (method == B200_DISC_ZOH) kb = (expf(A * dt) - 1.f) / A;
    else if (method == B200_DISC_BILINEAR) kb = dt / (1.f - 0.5f * dt * A);
    else if (method == B200_DISC_DIRAC) kb = 1.f;
    else kb = dt;
  }
}

__device__ __forceinline__ RowScalars load_row(const b200_ssu_args &p, int b, int h, int m) {
  RowScalars r;
  r.x = ld_act(p.x, p.x_dtype, (int64_t)b * p.x_bs + (int64_t)h * p.x_hs + (int64_t)m * p.x_ds);
  float dt = ld_act(p.dt, p.dt_dtype, (int64_t)b * p.dt_bs + (int64_t)h * p.dt_hs + (int64_t)m * p.dt_ds);
  if (p.dt_bias) dt += ld_act(p.dt_bias, p.dt_bias_dtype, (int64_t)h * p.dt_bias_hs + (int64_t)m * p.dt_bias_ds);
  if (p.dt_softplus) dt = softplus20(dt);
  r.dt = dt;
  r.dA = p.deltaA ? ld_act(p.deltaA, p.deltaA_dtype,
                           (int64_t)b * p.deltaA_bs + (int64_t)h * p.deltaA_hs + (int64_t)m * p.deltaA_ds)
                  : dt;
  r.Dv = p.D ? ld_act(p.D, p.D_dtype, (int64_t)h * p.D_hs + (int64_t)m * p.D_ds) : 0.f;
  r.has_z = p.z != nullptr;
  r.z = r.has_z ? ld_act(p.z, p.z_dtype, (int64_t)b * p.z_bs + (int64_t)h * p.z_hs + (int64_t)m * p.z_ds) : 0.f;
  return r;
}

template <typename T> __device__ __forceinline__ float ldt(const void *p, int64_t i);
template <> __device__ __forceinline__ float ldt<float>(const void *p, int64_t i) { return reinterpret_cast<const float *>(p)[i]; }
template <> __device__ __forceinline__ float ldt<__nv_bfloat16>(const void *p, int64_t i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}
template <> __device__ __forceinline__ float ldt<__half>(const void *p, int64_t i) {
  return __half2float(reinterpret_cast<const __half *>(p)[i]);
}
template <typename T> __device__ __forceinline__ void stt(void *p, int64_t i, float v);
template <> __device__ __forceinline__ void stt<float>(void *p, int64_t i, float v) { reinterpret_cast<float *>(p)[i] = v; }
template <> __device__ __forceinline__ void stt<__nv_bfloat16>(void *p, int64_t i, float v) {
  reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ void stt<__half>(void *p, int64_t i, float v) {
  reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
}

// Dense rows: state and A contiguous along dstate, 16-byte aligned; A, D, dt_bias float32;
// x, dt, z, deltaA, B, C, out all of type XT.  Every load of a thread is issued up front and
// unconditionally typed, so the ~14 independent loads overlap instead of forming a chain.
// RPT rows per lane group (rows r, r + ROWS, ...; all in the same (batch, head) when RPT > 1, so
// they share B and C): the state, A and scalar loads of all RPT rows are in flight together,
// which is what keeps enough bytes in flight to approach the HBM rate on a one-pass kernel.
template <typename ST, typename XT, int LPR, int RPT>
__global__ void __launch_bounds__(128, RPT > 1 ? 6 : 8) ssu_vec_kernel(const b200_ssu_args p) {
  constexpr int VEC = Vec16<ST>::N;
  constexpr int ROWS = 128 / LPR;
  const int sub = threadIdx.x % LPR;
  const int64_t nrows = (int64_t)p.batch * p.nheads * p.dim;
  const int64_t row0 = (int64_t)blockIdx.x * ROWS * RPT + threadIdx.x / LPR;
  // with RPT > 1 the launcher guarantees dim % (ROWS * RPT) == 0: no partial CTAs, one (b, h) per CTA
  const bool active = row0 < nrows;   // inactive lanes recompute row 0 and store nothing (they stay for the shuffles)
  // 32-bit row decomposition (the launcher sends row counts >= 2^31 to the generic kernel):
  // 64-bit div/mod would cost more instructions than the whole update of the row
  const uint32_t rr = active ? (uint32_t)row0 : 0u;
  const uint32_t rq = rr / (uint32_t)p.dim;
  const int m0 = (int)(rr - rq * (uint32_t)p.dim);
  const int b = (int)(rq / (uint32_t)p.nheads);
  const int h = (int)(rq - (uint32_t)b * (uint32_t)p.nheads);
  const int sb = p.state_batch_indices ? p.state_batch_indices[b] : b;
  const int g = h / (p.nheads / p.ngroups);
  const int64_t boff = (int64_t)b * p.B_bs + (int64_t)g * p.B_gs;
  const int64_t coff = (int64_t)b * p.C_bs + (int64_t)g * p.C_gs;
  float xv[RPT], dt[RPT], dA[RPT], Dv[RPT], zv[RPT];
#pragma unroll
  for (int k = 0; k < RPT; ++k) {
    const int m = m0 + k * ROWS;
    xv[k] = ldt<XT>(p.x, (int64_t)b * p.x_bs + (int64_t)h * p.x_hs + (int64_t)m * p.x_ds);
    dt[k] = ldt<XT>(p.dt, (int64_t)b * p.dt_bs + (int64_t)h * p.dt_hs + (int64_t)m * p.dt_ds);
    if (p.dt_bias) dt[k] += reinterpret_cast<const float *>(p.dt_bias)[(int64_t)h * p.dt_bias_hs + (int64_t)m * p.dt_bias_ds];
    Dv[k] = p.D ? reinterpret_cast<const float *>(p.D)[(int64_t)h * p.D_hs + (int64_t)m * p.D_ds] : 0.f;
    zv[k] = p.z ? ldt<XT>(p.z, (int64_t)b * p.z_bs + (int64_t)h * p.z_hs + (int64_t)m * p.z_ds) : 0.f;
    dA[k] = p.deltaA ? ldt<XT>(p.deltaA, (int64_t)b * p.deltaA_bs + (int64_t)h * p.deltaA_hs + (int64_t)m * p.deltaA_ds) : 0.f;
  }
  float acc[RPT];
#pragma unroll
  for (int k = 0; k < RPT; ++k) acc[k] = 0.f;
  for (int n0 = sub * VEC; n0 < p.dstate; n0 += LPR * VEC) {
    Vec16<ST> sv[RPT];
    float Av[RPT][VEC], Bn[VEC], Cn[VEC];
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
      const int m = m0 + k * ROWS;
      ST *srow = reinterpret_cast<ST *>(p.state) + (int64_t)sb * p.state_bs + (int64_t)h * p.state_hs + (int64_t)m * p.state_ds;
      const float *arow = reinterpret_cast<const float *>(p.A) + (int64_t)h * p.A_hs + (int64_t)m * p.A_ds;
      sv[k].load(srow + n0);
#pragma unroll
      for (int i = 0; i < VEC; ++i) Av[k][i] = arow[(int64_t)(n0 + i) * p.A_ns];
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      Bn[i] = ldt<XT>(p.B, boff + (int64_t)(n0 + i) * p.B_ns);
      Cn[i] = ldt<XT>(p.C, coff + (int64_t)(n0 + i) * p.C_ns);
    }
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
      float d = dt[k];
      if (p.dt_softplus) d = softplus20(d);
      const float da = p.deltaA ? dA[k] : d;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float a, kb;
        step_coef(p.method, Av[k][i], d, da, a, kb);
        const float s = sv[k].v[i] * a + kb * Bn[i] * xv[k];
        sv[k].v[i] = s;
        acc[k] += s * Cn[i];
      }
      if (active) {
        const int m = m0 + k * ROWS;
        ST *srow = reinterpret_cast<ST *>(p.state) + (int64_t)sb * p.state_bs + (int64_t)h * p.state_hs + (int64_t)m * p.state_ds;
        sv[k].store(srow + n0);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < RPT; ++k) {
    float a = acc[k];
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (active && sub == 0) {
      float out = a + Dv[k] * xv[k];
      if (p.z) out *= zv[k] * sigmoidf_(zv[k]);
      stt<XT>(p.out, (int64_t)b * p.out_bs + (int64_t)h * p.out_hs + (int64_t)(m0 + k * ROWS) * p.out_ds, out);
    }
  }
}

// Any strides / dtypes: one lane per state element, LPR lanes per row.
template <int LPR>
__global__ void __launch_bounds__(128) ssu_generic_kernel(const b200_ssu_args p) {
  constexpr int ROWS = 128 / LPR;
  const int sub = threadIdx.x % LPR;
  const int64_t row = (int64_t)blockIdx.x * ROWS + threadIdx.x / LPR;
  const int64_t nrows = (int64_t)p.batch * p.nheads * p.dim;
  const bool active = row < nrows;
  const int64_t rr = active ? row : 0;
  const int m = (int)(rr % p.dim);
  const int h = (int)((rr / p.dim) % p.nheads);
  const int b = (int)(rr / ((int64_t)p.dim * p.nheads));
  const int sb = p.state_batch_indices ? p.state_batch_indices[b] : b;
  const int g = h / (p.nheads / p.ngroups);
  const RowScalars r = load_row(p, b, h, m);
  const int64_t soff = (int64_t)sb * p.state_bs + (int64_t)h * p.state_hs + (int64_t)m * p.state_ds;
  const int64_t aoff = (int64_t)h * p.A_hs + (int64_t)m * p.A_ds;
  const int64_t boff = (int64_t)b * p.B_bs + (int64_t)g * p.B_gs;
  const int64_t coff = (int64_t)b * p.C_bs + (int64_t)g * p.C_gs;
  float acc = 0.f;
  for (int n = sub; n < p.dstate; n += LPR) {
    const float An = ld_act(p.A, p.A_dtype, aoff + (int64_t)n * p.A_ns);
    const float Bn = ld_act(p.B, p.bc_dtype, boff + (int64_t)n * p.B_ns);
    const float Cn = ld_act(p.C, p.bc_dtype, coff + (int64_t)n * p.C_ns);
    float a, kb;
    step_coef(p.method, An, r.dt, r.dA, a, kb);
    if (active) {
      const float s = ld_act(p.state, p.state_dtype, soff + (int64_t)n * p.state_ns) * a + kb * Bn * r.x;
      st_act(p.state, p.state_dtype, soff + (int64_t)n * p.state_ns, s);
      acc += s * Cn;
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (active && sub == 0) {
    float out = acc + r.Dv * r.x;
    if (r.has_z) out *= r.z * sigmoidf_(r.z);
    st_act(p.out, p.x_dtype, (int64_t)b * p.out_bs + (int64_t)h * p.out_hs + (int64_t)m * p.out_ds, out);
  }
}

template <typename ST, typename XT, int LPR> int launch_vec_l(const b200_ssu_args &a, cudaStream_t st) {
  constexpr int ROWS = 128 / LPR;
  const int64_t nrows = (int64_t)a.batch * a.nheads * a.dim;
  if (a.dim % (ROWS * 2) == 0) {
    ssu_vec_kernel<ST, XT, LPR, 2><<<(unsigned)(nrows / (ROWS * 2)), 128, 0, st>>>(a);
  } else {
    ssu_vec_kernel<ST, XT, LPR, 1><<<(unsigned)((nrows + ROWS - 1) / ROWS), 128, 0, st>>>(a);
  }
  return launch_status();
}
template <typename ST, typename XT> int launch_vec(const b200_ssu_args &a, cudaStream_t st) {
  constexpr int VEC = Vec16<ST>::N;
  int lpr = 1;
  while (lpr < 32 && lpr * VEC < a.dstate) lpr <<= 1;
  switch (lpr) {
    case 1: return launch_vec_l<ST, XT, 1>(a, st);
    case 2: return launch_vec_l<ST, XT, 2>(a, st);
    case 4: return launch_vec_l<ST, XT, 4>(a, st);
    case 8: return launch_vec_l<ST, XT, 8>(a, st);
    case 16: return launch_vec_l<ST, XT, 16>(a, st);
    default: return launch_vec_l<ST, XT, 32>(a, st);
  }
}
template <typename ST> int launch_vec_x(const b200_ssu_args &a, cudaStream_t st) {
  if (a.x_dtype == B200_F32) return launch_vec<ST, float>(a, st);
  if (a.x_dtype == B200_BF16) return launch_vec<ST, __nv_bfloat16>(a, st);
  return launch_vec<ST, __half>(a, st);
}

int launch_generic(const b200_ssu_args &a, cudaStream_t st) {
  const int64_t nrows = (int64_t)a.batch * a.nheads * a.dim;
  int lpr = 1;
  while (lpr < 32 && lpr < a.dstate) lpr <<= 1;
  const unsigned grid = (unsigned)((nrows + (128 / lpr) - 1) / (128 / lpr));
  switch (lpr) {
    case 1: ssu_generic_kernel<1><<<grid, 128, 0, st>>>(a); break;
    case 2: ssu_generic_kernel<2><<<grid, 128, 0, st>>>(a); break;
    case 4: ssu_generic_kernel<4><<<grid, 128, 0, st>>>(a); break;
    case 8: ssu_generic_kernel<8><<<grid, 128, 0, st>>>(a); break;
    case 16: ssu_generic_kernel<16><<<grid, 128, 0, st>>>(a); break;
    default: ssu_generic_kernel<32><<<grid, 128, 0, st>>>(a); break;
  }
  return launch_status();
}

bool dtype_ok(int d) { return d == B200_F32 || d == B200_F16 || d == B200_BF16; }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_ssu_step(const b200_ssu_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "ssu_step: null argument block");
  const b200_ssu_args &a = *args;
  B200_REQUIRE(a.state && a.x && a.dt && a.A && a.B && a.C && a.out, B200_ERR_NULL,
               "ssu_step: state, x, dt, A, B, C, out must be non-null");
  B200_REQUIRE(a.batch > 0 && a.nheads > 0 && a.dim > 0 && a.dstate > 0 && a.ngroups > 0, B200_ERR_SHAPE,
               "ssu_step: sizes must be positive");
  B200_REQUIRE(a.nheads % a.ngroups == 0, B200_ERR_SHAPE, "nheads must be divisible by ngroups");
  B200_REQUIRE(a.method >= B200_DISC_ZOH && a.method <= B200_DISC_S7, B200_ERR_DTYPE, "ssu_step: unknown discretization");
  B200_REQUIRE(dtype_ok(a.state_dtype) && dtype_ok(a.x_dtype) && dtype_ok(a.dt_dtype) && dtype_ok(a.A_dtype) &&
                   dtype_ok(a.bc_dtype),
               B200_ERR_DTYPE, "ssu_step: unknown dtype");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int es = act_size(a.state_dtype);
  const int vec = 16 / es;
  const bool dense = a.state_ns == 1 && a.dstate % vec == 0 && a.A_dtype == B200_F32 &&
                     (reinterpret_cast<uintptr_t>(a.state) % 16 == 0) &&
                     (a.state_bs * es) % 16 == 0 && (a.state_hs * es) % 16 == 0 && (a.state_ds * es) % 16 == 0 &&
                     (a.A_ns != 1 || ((reinterpret_cast<uintptr_t>(a.A) % 16 == 0) && a.A_hs % 4 == 0 && a.A_ds % 4 == 0));
  // the typed kernel wants one activation dtype (x, dt, z, deltaA, B, C) and float32 D / dt_bias
  const bool uniform = a.dt_dtype == a.x_dtype && a.bc_dtype == a.x_dtype && (!a.z || a.z_dtype == a.x_dtype) &&
                       (!a.deltaA || a.deltaA_dtype == a.x_dtype) && (!a.D || a.D_dtype == B200_F32) &&
                       (!a.dt_bias || a.dt_bias_dtype == B200_F32);
  if (dense && uniform && (int64_t)a.batch * a.nheads * a.dim < (int64_t(1) << 31)) {
    if (a.state_dtype == B200_F32) return launch_vec_x<float>(a, st);
    if (a.state_dtype == B200_BF16) return launch_vec_x<__nv_bfloat16>(a, st);
    return launch_vec_x<__half>(a, st);
  }
  return launch_generic(a, st);
}
