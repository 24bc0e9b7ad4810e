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

__device__ int g_ssu_status = 0;   // set to non-zero when a bounded barrier wait expires

// host read of the status word (used by b200_device_status)
int ssu_status_read() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ssu_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

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

// ---------------------------------------------------------------------------------------------
// Bulk-copy pipeline for dense operands.  A one-pass kernel with one 16-byte load per thread keeps
// too few bytes in flight to reach the HBM rate, so here persistent CTAs stream tiles of 128 rows
// through a 3-slot shared-memory ring: one thread issues 1-D bulk asynchronous copies (the TMA
// engine) of the tile's state rows and per-row scalars onto the slot's mbarrier, the CTA updates
// the state in place in shared memory, and the new state and the outputs leave through bulk
// shared->global copies.  Two tiles per CTA are in flight while a third is computed.  Per tile:
//   phase A  one thread per row: dt' = softplus(dt + bias), x and deltaA as float32
//   phase B  LPR lanes per row: the state update and the row's partial sum of state * C
//            (A comes straight from global memory: it is shared by all batch rows and L2-resident)
//   phase C  one thread per row: + D x, * silu(z), conversion to the output dtype
// so the per-row scalar work is done once per row and not once per lane of the row.
constexpr int TR = 128;   // rows per tile
constexpr int TNS = 4;    // ring slots
constexpr int TT = 256;   // threads per CTA

template <typename ST, typename XT, int LPR> struct TmaSlot {
  static constexpr int VEC = 16 / (int)sizeof(ST);
  static constexpr int N = LPR * VEC;                    // dstate handled by this instantiation
  static constexpr int ST_B = TR * N * (int)sizeof(ST);
  static constexpr int X_B = TR * (int)sizeof(XT);       // x, dt, z, deltaA, out
  static constexpr int F_B = TR * 4;                     // D, dt_bias
  static constexpr int BC_B = N * (int)sizeof(XT);       // a multiple of 16 for every supported N
  static constexpr int OFF_S = 0;
  static constexpr int OFF_X = OFF_S + ST_B;
  static constexpr int OFF_DT = OFF_X + X_B;
  static constexpr int OFF_Z = OFF_DT + X_B;
  static constexpr int OFF_DA = OFF_Z + X_B;
  static constexpr int OFF_OUT = OFF_DA + X_B;
  static constexpr int OFF_D = OFF_OUT + X_B;
  static constexpr int OFF_BIAS = OFF_D + F_B;
  static constexpr int OFF_B = OFF_BIAS + F_B;
  static constexpr int OFF_C = OFF_B + BC_B;
  static constexpr int SIZE = (OFF_C + BC_B + 127) / 128 * 128;
  static constexpr int OFF_ROW = TNS * SIZE;             // float [4][TR]: dt', x, deltaA, row sums
  static constexpr int OFF_BAR = OFF_ROW + 4 * TR * 4;
  static constexpr int TOTAL = OFF_BAR + TNS * 8;
};

template <typename XT> __device__ __forceinline__ float lds_act(const unsigned char *base, int i) {
  return ldt<XT>(base, i);
}

template <typename ST, typename XT, int LPR>
__global__ void __launch_bounds__(TT, 4) ssu_tma_kernel(const b200_ssu_args p, int tiles_per_bh) {
  using SL = TmaSlot<ST, XT, LPR>;
  // a warp owns 16 consecutive rows of the tile through all three phases, so the phases are
  // separated by warp barriers only; the one block barrier per tile precedes the bulk stores
  constexpr int VEC = SL::VEC, N = SL::N, WROWS = TR / (TT / 32), RPP = 32 / LPR, PASSES = WROWS / RPP;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + SL::OFF_BAR);
  float *row_d = reinterpret_cast<float *>(smem + SL::OFF_ROW), *row_x = row_d + TR, *row_da = row_d + 2 * TR,
        *row_acc = row_d + 3 * TR;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, part = lane % LPR;
  const int r0 = warp * WROWS + lane / LPR;         // first row of this lane group in phase B
  const int rowA = warp * WROWS + lane;             // row of this lane in phases A and C (lanes < WROWS)
  const uint32_t ntiles = (uint32_t)p.batch * (uint32_t)p.nheads * (uint32_t)tiles_per_bh;   // < 2^31 (host check)
  const int my = (int)((ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const int es = (int)sizeof(ST);

  // A CTA's tiles are blockIdx.x + it * gridDim.x; a position in that sequence is kept as
  // (batch*heads index, tile inside it) and advanced by the decomposed grid stride, so that the
  // per-tile index arithmetic needs no division (it was a quarter of the kernel's instructions).
  struct Pos { uint32_t bh, mt; };
  const uint32_t step_bh = gridDim.x / (uint32_t)tiles_per_bh, step_mt = gridDim.x % (uint32_t)tiles_per_bh;
  auto first_pos = [&]() { Pos q; q.bh = blockIdx.x / (uint32_t)tiles_per_bh; q.mt = blockIdx.x % (uint32_t)tiles_per_bh; return q; };
  auto advance = [&](Pos &q) {
    q.bh += step_bh;
    q.mt += step_mt;
    if (q.mt >= (uint32_t)tiles_per_bh) { q.mt -= (uint32_t)tiles_per_bh; q.bh += 1; }
  };
  struct Tile { int b, h, m0, sb, g; };
  auto tile_of = [&](const Pos &q, bool need_sb) {
    Tile t;
    t.m0 = (int)q.mt * TR;
    if (p.nheads == 1) { t.b = (int)q.bh; t.h = 0; t.g = 0; }
    else {
      t.b = (int)(q.bh / (uint32_t)p.nheads);
      t.h = (int)(q.bh - (uint32_t)t.b * (uint32_t)p.nheads);
      t.g = t.h / (p.nheads / p.ngroups);
    }
    t.sb = (need_sb && p.state_batch_indices) ? p.state_batch_indices[t.b] : t.b;
    return t;
  };
  Pos pf = first_pos();        // position of the next tile to load (used by the issuing thread)
  int pf_it = 0;
  auto issue = [&]() {   // one thread: loads tile pf_it and advances
    const int it = pf_it;
    if (it >= my) return;
    const Tile t = tile_of(pf, true);
    ++pf_it;
    advance(pf);
    unsigned char *s = smem + (size_t)(it % TNS) * SL::SIZE;
    uint64_t *bar = &full[it % TNS];
    uint32_t bytes = SL::ST_B + 2 * SL::X_B + 2 * SL::BC_B;
    if (p.z) bytes += SL::X_B;
    if (p.deltaA) bytes += SL::X_B;
    if (p.D) bytes += SL::F_B;
    if (p.dt_bias) bytes += SL::F_B;
    mbar_expect_tx(bar, bytes);
    const XT *xp = reinterpret_cast<const XT *>(p.x), *dtp = reinterpret_cast<const XT *>(p.dt);
    bulk_g2s(s + SL::OFF_S, reinterpret_cast<const unsigned char *>(p.state) +
                                ((int64_t)t.sb * p.state_bs + (int64_t)t.h * p.state_hs + (int64_t)t.m0 * p.state_ds) * es,
             SL::ST_B, bar);
    bulk_g2s(s + SL::OFF_X, xp + (int64_t)t.b * p.x_bs + (int64_t)t.h * p.x_hs + t.m0, SL::X_B, bar);
    bulk_g2s(s + SL::OFF_DT, dtp + (int64_t)t.b * p.dt_bs + (int64_t)t.h * p.dt_hs + t.m0, SL::X_B, bar);
    if (p.z)
      bulk_g2s(s + SL::OFF_Z, reinterpret_cast<const XT *>(p.z) + (int64_t)t.b * p.z_bs + (int64_t)t.h * p.z_hs + t.m0, SL::X_B, bar);
    if (p.deltaA)
      bulk_g2s(s + SL::OFF_DA,
               reinterpret_cast<const XT *>(p.deltaA) + (int64_t)t.b * p.deltaA_bs + (int64_t)t.h * p.deltaA_hs + t.m0, SL::X_B, bar);
    if (p.D) bulk_g2s(s + SL::OFF_D, reinterpret_cast<const float *>(p.D) + (int64_t)t.h * p.D_hs + t.m0, SL::F_B, bar);
    if (p.dt_bias)
      bulk_g2s(s + SL::OFF_BIAS, reinterpret_cast<const float *>(p.dt_bias) + (int64_t)t.h * p.dt_bias_hs + t.m0, SL::F_B, bar);
    bulk_g2s(s + SL::OFF_B, reinterpret_cast<const XT *>(p.B) + (int64_t)t.b * p.B_bs + (int64_t)t.g * p.B_gs, SL::BC_B, bar);
    bulk_g2s(s + SL::OFF_C, reinterpret_cast<const XT *>(p.C) + (int64_t)t.b * p.C_bs + (int64_t)t.g * p.C_gs, SL::BC_B, bar);
  };

  if (tid == 0) {
    for (int i = 0; i < TNS; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (tid == 0) {
    for (int i = 0; i < TNS - 1; ++i) issue();
  }
  Pos cur = first_pos();
  const bool plain_exp = p.method == B200_DISC_MAMBA || p.method == B200_DISC_DIRAC;
  bool failed = false;
  int fail_it = 0;
  for (int it = 0; it < my; ++it) {
    unsigned char *s = smem + (size_t)(it % TNS) * SL::SIZE;
    const Tile t = tile_of(cur, false);
    // A rows of this thread's passes: plain 16-byte loads, issued before the wait for the tile
    float Av[PASSES][VEC];
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
      const float *arow = reinterpret_cast<const float *>(p.A) + (int64_t)t.h * p.A_hs +
                          (int64_t)(t.m0 + r0 + j * RPP) * N + part * VEC;
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        const float4 a4 = *reinterpret_cast<const float4 *>(arow + i);
        Av[j][i] = a4.x; Av[j][i + 1] = a4.y; Av[j][i + 2] = a4.z; Av[j][i + 3] = a4.w;
      }
    }
    if (!failed && !mbar_wait(&full[it % TNS], (uint32_t)(it / TNS) & 1u)) failed = true;
    // ---- phase A: per-row scalars
    if (lane < WROWS) {
      float d = lds_act<XT>(s + SL::OFF_DT, rowA);
      if (p.dt_bias) d += reinterpret_cast<const float *>(s + SL::OFF_BIAS)[rowA];
      if (p.dt_softplus) d = softplus20(d);
      row_d[rowA] = d;
      row_x[rowA] = lds_act<XT>(s + SL::OFF_X, rowA);
      row_da[rowA] = p.deltaA ? lds_act<XT>(s + SL::OFF_DA, rowA) : d;
    }
    float Bn[VEC], Cn[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      Bn[i] = lds_act<XT>(s + SL::OFF_B, part * VEC + i);
      Cn[i] = lds_act<XT>(s + SL::OFF_C, part * VEC + i);
    }
    __syncwarp();
    // ---- phase B: state update
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
      const int row = r0 + j * RPP;
      const float xv = row_x[row], d = row_d[row], da = row_da[row];
      ST *srow = reinterpret_cast<ST *>(s + SL::OFF_S) + row * N + part * VEC;
      Vec16<ST> sv;
      sv.load(srow);
      float acc = 0.f;
      if (plain_exp) {     // a = exp(A dA) by the SFU's ex2 (relative error 2^-22); input gain dt (mamba) or 1 (dirac)
        const float da2 = da * kLog2e, kx = (p.method == B200_DISC_MAMBA ? d : 1.f) * xv;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float a;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(a) : "f"(Av[j][i] * da2));
          const float v = fmaf(sv.v[i], a, kx * Bn[i]);
          sv.v[i] = v;
          acc = fmaf(v, Cn[i], acc);
        }
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          float a, kb;
          step_coef(p.method, Av[j][i], d, da, a, kb);
          const float v = sv.v[i] * a + kb * Bn[i] * xv;
          sv.v[i] = v;
          acc += v * Cn[i];
        }
      }
      sv.store(srow);
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (part == 0) row_acc[row] = acc;
    }
    __syncwarp();
    // ---- phase C: outputs
    if (lane < WROWS) {
      float out = row_acc[rowA];
      if (p.D) out += reinterpret_cast<const float *>(s + SL::OFF_D)[rowA] * row_x[rowA];
      if (p.z) {
        const float zv = lds_act<XT>(s + SL::OFF_Z, rowA);
        out *= zv * sigmoidf_(zv);
      }
      stt<XT>(s + SL::OFF_OUT, rowA, out);
    }
    fence_proxy_async();
    // A tile whose loads did not arrive holds garbage: nothing of it may reach the caller's state
    // (updated in place) or out.  Every thread leaves the loop together; no store, no new load.
    if (__syncthreads_or(failed ? 1 : 0)) {
      failed = true;
      fail_it = it;
      break;
    }
    if (tid == 0) {
      const Tile ts = tile_of(cur, true);
      bulk_s2g(reinterpret_cast<unsigned char *>(p.state) +
                   ((int64_t)ts.sb * p.state_bs + (int64_t)ts.h * p.state_hs + (int64_t)ts.m0 * p.state_ds) * es,
               s + SL::OFF_S, SL::ST_B);
      bulk_s2g(reinterpret_cast<XT *>(p.out) + (int64_t)ts.b * p.out_bs + (int64_t)ts.h * p.out_hs + ts.m0, s + SL::OFF_OUT,
               SL::X_B);
      bulk_commit();
      // the slot refilled next held tile it-1: its stores (the group before this one) must have been read out
      bulk_wait_read<1>();
      issue();
    }
    advance(cur);
  }
  if (tid == 0) {
    bulk_wait<0>();      // stores of the tiles completed before a failure, or of the last tiles
    if (failed) {
      // loads still in flight into this CTA's slots: give each a last bounded wait before the CTA
      // (and its shared memory) goes away
      for (int k = fail_it + 1; k < my && k < fail_it + TNS - 1; ++k)
        mbar_wait(&full[k % TNS], (uint32_t)(k / TNS) & 1u, 1u << 20);
      atomicExch(&g_ssu_status, 3);
    }
  }
}

int ssu_sm_count() { return sm_count_current(); }

template <typename ST, typename XT, int LPR> int launch_tma_l(const b200_ssu_args &a, cudaStream_t st) {
  using SL = TmaSlot<ST, XT, LPR>;
  auto k = ssu_tma_kernel<ST, XT, LPR>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SL::TOTAL);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return (int)e; }
  const int tiles_per_bh = a.dim / TR;
  const int64_t ntiles = (int64_t)a.batch * a.nheads * tiles_per_bh;
  int per_sm = (227 * 1024) / (SL::TOTAL + 1024);
  per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);   // the launch bounds allow 4 CTAs per SM
  int64_t grid = (int64_t)ssu_sm_count() * per_sm;
  if (grid > ntiles) grid = ntiles;
  k<<<(unsigned)grid, TT, SL::TOTAL, st>>>(a, tiles_per_bh);
  return launch_status();
}
template <typename ST, typename XT> int launch_tma(const b200_ssu_args &a, cudaStream_t st) {
  constexpr int VEC = 16 / (int)sizeof(ST);
  return a.dstate == 2 * VEC ? launch_tma_l<ST, XT, 2>(a, st) : launch_tma_l<ST, XT, 4>(a, st);
}
template <typename ST> int launch_tma_x(const b200_ssu_args &a, cudaStream_t st) {
  if (a.x_dtype == B200_F32) return launch_tma<ST, float>(a, st);
  if (a.x_dtype == B200_BF16) return launch_tma<ST, __nv_bfloat16>(a, st);
  return launch_tma<ST, __half>(a, st);
}

// Operands the bulk-copy pipeline can address: dense state / A tiles, unit-stride rows for the
// per-row tensors, every tile start on a 16-byte boundary.
bool tma_ok(const b200_ssu_args &a) {
  const int es = act_size(a.state_dtype), xs = act_size(a.x_dtype);
  const int vec = 16 / es;
  if (a.dstate != 2 * vec && a.dstate != 4 * vec) return false;
  if (a.dim % TR != 0) return false;
  auto al = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const int64_t xm = 16 / xs;   // elements of the activation dtype per 16 bytes
  if (a.state_ns != 1 || a.state_ds != a.dstate || !al(a.state) || (a.state_bs * es) % 16 || (a.state_hs * es) % 16) return false;
  if (a.A_ns != 1 || a.A_ds != a.dstate || !al(a.A) || a.A_hs % 4) return false;
  if (a.x_ds != 1 || !al(a.x) || a.x_bs % xm || a.x_hs % xm) return false;
  if (a.dt_ds != 1 || !al(a.dt) || a.dt_bs % xm || a.dt_hs % xm) return false;
  if (a.out_ds != 1 || !al(a.out) || a.out_bs % xm || a.out_hs % xm) return false;
  if (a.z && (a.z_ds != 1 || !al(a.z) || a.z_bs % xm || a.z_hs % xm)) return false;
  if (a.deltaA && (a.deltaA_ds != 1 || !al(a.deltaA) || a.deltaA_bs % xm || a.deltaA_hs % xm)) return false;
  if (a.D && (a.D_ds != 1 || !al(a.D) || a.D_hs % 4)) return false;
  if (a.dt_bias && (a.dt_bias_ds != 1 || !al(a.dt_bias) || a.dt_bias_hs % 4)) return false;
  if (a.B_ns != 1 || !al(a.B) || a.B_bs % xm || a.B_gs % xm) return false;
  if (a.C_ns != 1 || !al(a.C) || a.C_bs % xm || a.C_gs % xm) return false;
  return true;
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
  // lrnnx's Triton kernel (selective_state_update.py:168-176) and its selective_state_update_ref
  // (:551-553) give different transitions for "s7" with deltaA (exp(A deltaA) against the S7
  // formula of dt), and no lrnnx layer passes both: the combination is refused.
  B200_REQUIRE(!(a.method == B200_DISC_S7 && a.deltaA), B200_ERR_UNSUPPORTED,
               "ssu_step: deltaA is not defined for the s7 discretization");
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
    if (tma_ok(a)) {
      if (a.state_dtype == B200_F32) return launch_tma_x<float>(a, st);
      if (a.state_dtype == B200_BF16) return launch_tma_x<__nv_bfloat16>(a, st);
      return launch_tma_x<__half>(a, st);
    }
    if (a.state_dtype == B200_F32) return launch_vec_x<float>(a, st);
    if (a.state_dtype == B200_BF16) return launch_vec_x<__nv_bfloat16>(a, st);
    return launch_vec_x<__half>(a, st);
  }
  return launch_generic(a, st);
}
