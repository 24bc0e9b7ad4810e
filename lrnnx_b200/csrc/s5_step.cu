// One-token update of the S5 (simplified) recurrence with fused projections.
//
// Math (lrnnx/ops/triton/simplified_state_update.py:404-469): Bu = B x; state <- a state + k Bu
// with a, k from the discretization of A with dt / deltaA; out = (2 or 1) * Re(C state) + D x.
// One CTA per batch row.  Phase 1: a warp per state p, lanes stride over the H inputs with
// coalesced 8-byte loads of B[p, :], warp sum, then the state update (written to global memory
// and kept in shared memory).  Phase 2: a warp per output h, lanes stride over the P states
// (C[h, :] coalesced) and over the H inputs for the D term.  B, C and D are shared by all batch
// rows and stay L2-resident; the step is bound by their L2 reads, not by HBM.
#include "common.cuh"
#include "dispatch.h"

namespace b200 {
namespace {

constexpr int S5T = 256;

__global__ void __launch_bounds__(S5T) s5_step_kernel(const b200_s5_step_args p) {
  extern __shared__ float sm[];
  float *xs = sm;                                   // [H]
  cf *st = reinterpret_cast<cf *>(sm + ((p.H + 1) & ~1));   // [P]
  const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float *x = reinterpret_cast<const float *>(p.x) + (int64_t)b * p.x_bs;
  for (int i = tid; i < p.H; i += S5T) xs[i] = x[i];
  __syncthreads();
  cf *state = reinterpret_cast<cf *>(p.state) + (int64_t)b * p.state_bs;
  const float *dt = reinterpret_cast<const float *>(p.dt) + (int64_t)b * p.dt_bs;
  const float *dA = p.deltaA ? reinterpret_cast<const float *>(p.deltaA) + (int64_t)b * p.deltaA_bs : dt;
  const cf *A = reinterpret_cast<const cf *>(p.A);
  const cf *B = reinterpret_cast<const cf *>(p.B);
  const cf *C = reinterpret_cast<const cf *>(p.C);
  for (int s = warp; s < p.P; s += S5T / 32) {
    const cf *Brow = B + (int64_t)s * p.H;
    cf acc = cf(0.f, 0.f);
    for (int h = lane; h < p.H; h += 32) acc = acc + Brow[h] * xs[h];
    acc = warp_sum(acc);
    if (lane == 0) {
      const cf An = A[s];
      const float d = dt[s], da = dA[s];
      cf a, k;
      if (p.method == B200_DISC_BILINEAR) {
        const cf v = An * (0.5f * da);
        a = (cf(1.f, 0.f) + v) / (cf(1.f, 0.f) - v);
        k = (cf(1.f, 0.f) / (cf(1.f, 0.f) - An * (0.5f * d))) * d;
      } else if (p.method == B200_DISC_ZOH) {
        a = cexp(An * da);
        k = (cexp(An * d) - cf(1.f, 0.f)) / An;
      } else {
        a = cexp(An * da);
        k = cf(1.f, 0.f);
      }
      const cf ns = a * state[s] + k * acc;
      state[s] = ns;
      st[s] = ns;
    }
  }
  __syncthreads();
  const float scale = p.conj_sym ? 2.f : 1.f;
  const float *D = reinterpret_cast<const float *>(p.D);
  float *out = reinterpret_cast<float *>(p.out) + (int64_t)b * p.out_bs;
  for (int h = warp; h < p.H; h += S5T / 32) {
    const cf *Crow = C + (int64_t)h * p.P;
    float acc = 0.f;
    for (int s = lane; s < p.P; s += 32) {
      const cf c = Crow[s], v = st[s];
      acc += c.re * v.re - c.im * v.im;
    }
    acc *= scale;
    if (D) {
      const float *Drow = D + (int64_t)h * p.H;
      for (int k = lane; k < p.H; k += 32) acc += Drow[k] * xs[k];
    }
    acc = warp_sum(acc);
    if (lane == 0) out[h] = acc;
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_s5_step(const b200_s5_step_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "s5_step: null argument block");
  const b200_s5_step_args &a = *args;
  B200_REQUIRE(a.state && a.x && a.dt && a.A && a.B && a.C && a.out, B200_ERR_NULL,
               "s5_step: state, x, dt, A, B, C, out must be non-null");
  B200_REQUIRE(a.batch > 0 && a.P > 0 && a.H > 0, B200_ERR_SHAPE, "s5_step: batch, P, H must be positive");
  B200_REQUIRE(a.method == B200_DISC_ZOH || a.method == B200_DISC_BILINEAR || a.method == B200_DISC_DIRAC,
               B200_ERR_DTYPE, "s5_step supports the zoh, bilinear and dirac discretizations");
  const size_t smem = (size_t)(((a.H + 1) & ~1) + 2 * a.P) * sizeof(float);
  B200_REQUIRE(smem <= 200 * 1024, B200_ERR_TOO_LARGE, "s5_step: H + 2P floats must fit in shared memory");
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(s5_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return (int)e; }
  }
  s5_step_kernel<<<(unsigned)a.batch, S5T, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return launch_status();
}
