// Shared device/host helpers for the sm_100a scan kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <cstdio>
#include <cstdarg>
#include "../../include/lrnnx_b200.h"

namespace b200 {

// ---------------------------------------------------------------- host side
void set_error(const char *fmt, ...);

#define B200_REQUIRE(cond, code, ...)            \
  do {                                           \
    if (!(cond)) {                               \
      ::b200::set_error(__VA_ARGS__);            \
      return (code);                             \
    }                                            \
  } while (0)

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("CUDA launch failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// Number of SMs of the current device (cached per device ordinal; 148 if the query fails).
inline int sm_count_current() {
  static int cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cache[dev];
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;     // benign race: every writer stores the same value
  }
  return n;
}

constexpr int kChunk = 2048;   // checkpoint spacing of the x tensor (timesteps)
constexpr int kMaxDState = 256;
constexpr float kLog2e = 1.4426950408889634f;

// -------------------------------------------------------------- device side
struct cf {            // complex float, layout-compatible with complex64
  float re, im;
  cf() = default;
  __host__ __device__ constexpr cf(float r, float i = 0.f) : re(r), im(i) {}
};
__device__ __forceinline__ cf operator+(cf a, cf b) { return cf(a.re + b.re, a.im + b.im); }
__device__ __forceinline__ cf operator-(cf a, cf b) { return cf(a.re - b.re, a.im - b.im); }
__device__ __forceinline__ cf operator*(cf a, cf b) {
  return cf(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
}
__device__ __forceinline__ cf operator*(float s, cf a) { return cf(s * a.re, s * a.im); }
__device__ __forceinline__ cf operator*(cf a, float s) { return cf(s * a.re, s * a.im); }
__device__ __forceinline__ cf conj(cf a) { return cf(a.re, -a.im); }
__device__ __forceinline__ float conj(float a) { return a; }
__device__ __forceinline__ cf operator/(cf a, cf b) {
  float inv = 1.f / (b.re * b.re + b.im * b.im);
  return cf((a.re * b.re + a.im * b.im) * inv, (a.im * b.re - a.re * b.im) * inv);
}
// sin and cos to about 1 ulp for |x| up to ~1e5: three-constant Cody-Waite reduction by
// pi/2 and the classic single-precision minimax polynomials on [-pi/4, pi/4].  The
// recurrences multiply thousands of these factors, so the SFU approximations
// (abs. error 2^-21) are not accurate enough for the phase.
__device__ __forceinline__ void sincos_cw(float x, float &sn, float &cs) {
  const float q = rintf(x * 0.6366197723675814f);
  const int qi = (int)q;
  float r = fmaf(-q, 1.5707962513e+0f, x);
  r = fmaf(-q, 7.5497894159e-8f, r);
  r = fmaf(-q, 5.3903029534e-15f, r);
  const float r2 = r * r;
  const float ps = fmaf(fmaf(fmaf(-1.9515295891e-4f, r2, 8.3321608736e-3f), r2, -1.6666654611e-1f), r2 * r, r);
  const float pc = fmaf(fmaf(fmaf(2.443315711809948e-5f, r2, -1.388731625493765e-3f), r2, 4.166664568298827e-2f),
                        r2 * r2, fmaf(-0.5f, r2, 1.f));
  const float s0 = (qi & 1) ? pc : ps;
  const float c0 = (qi & 1) ? ps : pc;
  sn = (qi & 2) ? -s0 : s0;
  cs = ((qi + 1) & 2) ? -c0 : c0;
}
__device__ __forceinline__ cf cexp(cf z) {
  // magnitude by the SFU's ex2 (relative error 2^-22, the same class as expf's 1 ulp)
  float e, s, c;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z.re * kLog2e));
  sincos_cw(z.im, s, c);
  return cf(e * c, e * s);
}
__device__ __forceinline__ float realpart(float a) { return a; }
__device__ __forceinline__ float realpart(cf a) { return a.re; }

template <typename V> __device__ __forceinline__ V v_one();
template <> __device__ __forceinline__ float v_one<float>() { return 1.f; }
template <> __device__ __forceinline__ cf v_one<cf>() { return cf(1.f, 0.f); }
template <typename V> __device__ __forceinline__ V v_zero();
template <> __device__ __forceinline__ float v_zero<float>() { return 0.f; }
template <> __device__ __forceinline__ cf v_zero<cf>() { return cf(0.f, 0.f); }

__device__ __forceinline__ float shfl_up(float v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ __forceinline__ cf shfl_up(cf v, int d) {
  return cf(__shfl_up_sync(0xffffffffu, v.re, d), __shfl_up_sync(0xffffffffu, v.im, d));
}
__device__ __forceinline__ float shfl_down(float v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
__device__ __forceinline__ cf shfl_down(cf v, int d) {
  return cf(__shfl_down_sync(0xffffffffu, v.re, d), __shfl_down_sync(0xffffffffu, v.im, d));
}
__device__ __forceinline__ float shfl_idx(float v, int l) { return __shfl_sync(0xffffffffu, v, l); }
__device__ __forceinline__ cf shfl_idx(cf v, int l) {
  return cf(__shfl_sync(0xffffffffu, v.re, l), __shfl_sync(0xffffffffu, v.im, l));
}
__device__ __forceinline__ float shfl_xor(float v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ __forceinline__ cf shfl_xor(cf v, int m) {
  return cf(__shfl_xor_sync(0xffffffffu, v.re, m), __shfl_xor_sync(0xffffffffu, v.im, m));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ cf warp_sum(cf v) { return cf(warp_sum(v.re), warp_sum(v.im)); }

// activation element load/store with a run-time dtype (generic kernels only)
__device__ __forceinline__ float ld_act(const void *p, int dtype, int64_t i) {
  if (dtype == B200_F32) return reinterpret_cast<const float *>(p)[i];
  if (dtype == B200_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
  return __half2float(reinterpret_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void st_act(void *p, int dtype, int64_t i, float v) {
  if (dtype == B200_F32) reinterpret_cast<float *>(p)[i] = v;
  else if (dtype == B200_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
}
__host__ __device__ inline int act_size(int dtype) { return dtype == B200_F32 ? 4 : 2; }

// softplus with the pass-through above 20 used by the reference
// (csrc/selective_scan/selective_scan.cuh:172-174); log1p(e) evaluated as
// log(1+e) * e / ((1+e) - 1) so that tiny e keeps full relative accuracy.
__device__ __forceinline__ float softplus20(float x) {
  if (x > 20.f) return x;
  float e = __expf(x);
  float u = 1.f + e;
  float d = u - 1.f;
  return d == 0.f ? e : __logf(u) * __fdividef(e, d);
}
__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// ------------------------------------------------- mbarrier / bulk-copy PTX
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: returns false if the phase did not complete within `limit`
// polls (the caller records the failure and bails out instead of hanging).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 26)) {
  uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// 1-D bulk asynchronous copy global -> shared, completion counted on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// 1-D bulk asynchronous copy shared -> global (bulk-group completion).
__device__ __forceinline__ void bulk_s2g(void *dst, const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

}  // namespace b200
