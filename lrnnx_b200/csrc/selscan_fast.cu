// Throughput kernels for the hot S6 (Mamba) shape class of the selective scan:
// real A, "mamba" discretization, variable B and C, dstate 16, 16-byte aligned rows.
//
// The scan is bound by the SFU (one ex2 per (t, n)) and the fp32 pipe, not by HBM, so the
// design minimises issue slots per (t, n):
//  * a thread owns 2 channels x 8 consecutive timesteps and keeps the two channels in the
//    halves of float2 registers, so the recurrence runs on Blackwell's packed fp32
//    instructions (__ffma2_rn / __fmul2_rn: two FMAs per issue slot);
//  * a CTA of 8 warps owns 16 channels of one (batch, group); the B and C tiles of a
//    256-step stage are staged once per CTA in shared memory and reused by all 16
//    channels, and each B/C value a thread reads serves both of its channels;
//  * all operands of a stage arrive through asynchronous 16-byte global->shared copies
//    (double-buffered, one stage ahead); fp32 rows are stored in a permuted order
//    (16-byte piece q of a row goes to slot (q&1)*32 + q/2) so that the lane-blocked
//    128-bit shared loads are bank-conflict free; 16-bit rows are conflict-free as they are;
//  * within a stage: thread-serial scan of 8 steps, 5-step warp-shuffle scan of the lane
//    aggregates, carry between stages in shared memory.
// Results match csrc/selective_scan/selective_scan.cuh:73-382 of lrnnx for this shape class.
#include "common.cuh"
#include "dispatch.h"

namespace b200 {
namespace {

constexpr int XI = 8;                // timesteps per lane
constexpr int XSTAGE = 32 * XI;      // 256 timesteps per stage
constexpr int XWARPS = 8;            // warps per CTA
constexpr int XCH = 2 * XWARPS;      // channels per CTA

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, int src_bytes) {
  // copies src_bytes (0..16) and zero-fills the rest of the 16-byte destination
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T> struct Row;   // a 256-step row of T in shared memory
template <> struct Row<float> {
  static constexpr int PIECES = 64;                 // 16-byte pieces per row
  static constexpr int EPP = 4;                     // elements per piece
  __device__ static int slot(int q) { return (q & 1) * 32 + (q >> 1); }
  // lane-blocked read of 8 consecutive elements starting at 8*lane
  __device__ static void read8(const void *row, int lane, float (&v)[8]) {
    const float4 *r = reinterpret_cast<const float4 *>(row);
    const float4 a = r[lane], b = r[32 + lane];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ static void store8(float *g, const float (&v)[8]) {
    reinterpret_cast<float4 *>(g)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(g)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Row<__nv_bfloat16> {
  static constexpr int PIECES = 32;
  static constexpr int EPP = 8;
  __device__ static int slot(int q) { return q; }
  __device__ static void read8(const void *row, int lane, float (&v)[8]) {
    const uint4 t = reinterpret_cast<const uint4 *>(row)[lane];
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store8(__nv_bfloat16 *g, const float (&v)[8]) {
    uint4 t;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(g) = t;
  }
};
template <> struct Row<__half> {
  static constexpr int PIECES = 32;
  static constexpr int EPP = 8;
  __device__ static int slot(int q) { return q; }
  __device__ static void read8(const void *row, int lane, float (&v)[8]) {
    const uint4 t = reinterpret_cast<const uint4 *>(row)[lane];
    const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  __device__ static void store8(__half *g, const float (&v)[8]) {
    uint4 t;
    __half2 *h = reinterpret_cast<__half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4 *>(g) = t;
  }
};

// Asynchronous copy of `nrows` 256-step rows (global row r at src + r*row_stride + t0) into
// shared rows of ROWB bytes each, zero-filled past the end of the sequence.
template <typename T>
__device__ __forceinline__ void stage_rows(unsigned char *dst, const T *src, int64_t row_stride, int nrows, int t0,
                                           int L, int tid, int nthreads) {
  constexpr int PIECES = Row<T>::PIECES, EPP = Row<T>::EPP;
  constexpr int ROWB = XSTAGE * (int)sizeof(T);
  for (int i = tid; i < nrows * PIECES; i += nthreads) {
    const int r = i / PIECES, q = i % PIECES;
    const int t = t0 + q * EPP;
    int valid = (L - t) * (int)sizeof(T);
    valid = valid < 0 ? 0 : (valid > 16 ? 16 : valid);
    const T *g = src + (int64_t)r * row_stride + (valid > 0 ? t : 0);
    cp_async16(dst + (size_t)r * ROWB + Row<T>::slot(q) * 16, g, valid);
  }
}

}  // namespace
}  // namespace b200

#include "selscan_fast_fwd.inc"
#include "selscan_fast_bwd.inc"
