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

struct RowScalars { float x, dt, dA, Dv, z; bool has_z; };

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

// Dense rows: state and A contiguous along dstate, 16-byte aligned; A float32.
template <typename ST, int LPR>
__global__ void __launch_bounds__(128) ssu_vec_kernel(const b200_ssu_args p) {
  constexpr int VEC = Vec16<ST>::N;
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
  ST *srow = reinterpret_cast<ST *>(p.state) + (int64_t)sb * p.state_bs + (int64_t)h * p.state_hs + (int64_t)m * p.state_ds;
  const float *arow = reinterpret_cast<const float *>(p.A) + (int64_t)h * p.A_hs + (int64_t)m * p.A_ds;
  const int64_t boff = (int64_t)b * p.B_bs + (int64_t)g * p.B_gs;
  const int64_t coff = (int64_t)b * p.C_bs + (int64_t)g * p.C_gs;
  float acc = 0.f;
  for (int n0 = sub * VEC; n0 < p.dstate; n0 += LPR * VEC) {
    Vec16<ST> sv;
    if (active) sv.load(srow + n0);
    float Av[VEC];
    if (p.A_ns == 1) {
#pragma unroll
      for (int q = 0; q < VEC / 4; ++q) {
        const float4 t = *reinterpret_cast<const float4 *>(arow + n0 + 4 * q);
        Av[4 * q] = t.x; Av[4 * q + 1] = t.y; Av[4 * q + 2] = t.z; Av[4 * q + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) Av[i] = arow[(int64_t)(n0 + i) * p.A_ns];
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float Bn = ld_act(p.B, p.bc_dtype, boff + (int64_t)(n0 + i) * p.B_ns);
      const float Cn = ld_act(p.C, p.bc_dtype, coff + (int64_t)(n0 + i) * p.C_ns);
      float a, kb;
      step_coef(p.method, Av[i], r.dt, r.dA, a, kb);
      const float s = sv.v[i] * a + kb * Bn * r.x;
      sv.v[i] = s;
      acc += s * Cn;
    }
    if (active) sv.store(srow + n0);
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (active && sub == 0) {
    float out = acc + r.Dv * r.x;
    if (r.has_z) out *= r.z * sigmoidf_(r.z);
    st_act(p.out, p.x_dtype, (int64_t)b * p.out_bs + (int64_t)h * p.out_hs + (int64_t)m * p.out_ds, out);
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

template <typename ST> int launch_vec(const b200_ssu_args &a, cudaStream_t st) {
  constexpr int VEC = Vec16<ST>::N;
  const int64_t nrows = (int64_t)a.batch * a.nheads * a.dim;
  int lpr = 1;
  while (lpr < 32 && lpr * VEC < a.dstate) lpr <<= 1;
  const unsigned grid = (unsigned)((nrows + (128 / lpr) - 1) / (128 / lpr));
  switch (lpr) {
    case 1: ssu_vec_kernel<ST, 1><<<grid, 128, 0, st>>>(a); break;
    case 2: ssu_vec_kernel<ST, 2><<<grid, 128, 0, st>>>(a); break;
    case 4: ssu_vec_kernel<ST, 4><<<grid, 128, 0, st>>>(a); break;
    case 8: ssu_vec_kernel<ST, 8><<<grid, 128, 0, st>>>(a); break;
    case 16: ssu_vec_kernel<ST, 16><<<grid, 128, 0, st>>>(a); break;
    default: ssu_vec_kernel<ST, 32><<<grid, 128, 0, st>>>(a); break;
  }
  return launch_status();
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
  if (dense) {
    if (a.state_dtype == B200_F32) return launch_vec<float>(a, st);
    if (a.state_dtype == B200_BF16) return launch_vec<__nv_bfloat16>(a, st);
    return launch_vec<__half>(a, st);
  }
  return launch_generic(a, st);
}
