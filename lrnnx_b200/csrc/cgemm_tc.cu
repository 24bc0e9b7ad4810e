// Complex projections around the S5 scan on the 5th-generation tensor cores (tcgen05 + TMEM):
//     out[b] (M x N) = W (M x K) * X[b] (K x N),      complex64, N contiguous,
// the shape of  Bu = B~ u,  y = C~ x  and of the two data gradients  du = B~^H dBu,  dx = C~^H dy
// of lrnnx's simplified_scan_fn / s5_inner_fn (lrnnx/ops/simplified_scan.py:67,87,136,165,401,419,
// 483-524), which lrnnx evaluates with torch.einsum (cuBLAS SIMT cgemm).
//
// Arithmetic.  With X' the (K x 2N) float view of X (re/im interleaved along N),
//     D1 = Re(W) X',   D2 = Im(W) X'     (two real GEMMs sharing the activation tile)
//     out_re[n] = D1[2n] - D2[2n+1],   out_im[n] = D1[2n+1] + D2[2n]
// so the activation is consumed exactly as it lies in memory and only the small weight is split
// into planes.  fp32-class accuracy on TF32 tensor cores comes from the 3xTF32 split
//     a b ~= a_hi b_hi + a_lo b_hi + a_hi b_lo,   x_hi = tf32(x), x_lo = tf32(x - x_hi),
// i.e. six tcgen05.mma per K step.  The weight planes (Re hi, Re lo, Im hi, Im lo) are prepared
// once per call on the host side; the low part of the activation tile is produced inside the
// kernel, in shared memory, by the warps that later run the epilogue: it is elementwise, so it is
// written at the same (swizzled) offsets the TMA used for the tile and no layout knowledge is needed.
//
// One CTA per 128 x 64-complex output tile: warp 0 issues the TMA loads (128-byte swizzled
// tiles, 2-stage ring on mbarriers), warp 1 allocates 256 TMEM columns and issues the MMAs
// (M = 128, N = 128 floats, K = 8 per instruction; A = weight plane, K-major, 128-byte swizzle;
// B = activation, MN-major, 128-byte swizzle of 32-byte chunks), warps 2-5 split the activation tile during the main loop and afterwards read the
// two accumulators with tcgen05.ld, combine them and store complex rows.  Every mbarrier wait is
// bounded; an expired wait sets the status word, skips the stores and still frees the TMEM.
#include "common.cuh"
#include "dispatch.h"
#include "tc_common.cuh"
#include <cstring>

namespace b200 {
namespace {

using namespace tc;

__device__ int g_cgemm_status = 0;

constexpr int GM = 128;               // weight rows per CTA
constexpr int GN = 128;               // activation floats per CTA (64 complex columns)
constexpr int GK = 32;                // floats of K per stage: one 128-byte swizzle row
constexpr int NSTAGE = 2;
constexpr int TILE = GM * GK * 4;     // 16 KB: a weight-plane tile; an activation tile has the same size
constexpr int STAGE_BYTES = 6 * TILE; // Re hi, Re lo, Im hi, Im lo, X hi, X lo
constexpr int TX_BYTES = 5 * TILE;    // what the TMA delivers per stage (X lo is produced in place)
constexpr int NTHREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr uint32_t WAIT_LIMIT = 1u << 24;

struct GemmMaps {
  CUtensorMap w;      // (K, 4 M) float32, box (32, 128)
  CUtensorMap x;      // (2 N, batch K) float32, box (32, 32)
};

// weight-plane tile, K-major: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t a_desc(uint32_t addr) { return smem_desc(addr, 16, 1024, 2); }
// activation tile, MN-major: 32-float column groups 4096 bytes apart, 4-row K groups 512 bytes apart
__device__ __forceinline__ uint64_t b_desc(uint32_t addr) { return smem_desc(addr, 4096, 512, 1); }
// instruction descriptor: D f32, A and B tf32, A K-major, B MN-major, M = 128, N = 128
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((GN >> 3) << 17) | ((GM >> 4) << 24);

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate,
                                         uint32_t idesc = kIdesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// The tensor core truncates a 32-bit operand to TF32, so the high part of x is what it reads from
// the tile as it is; the low part x - trunc(x) is exact in float32 and is rounded to the nearest
// TF32 here (the hardware would truncate it, a one-sided error that adds up over K).
__device__ __forceinline__ float tf32_low(float v) {
  const float r = v - __uint_as_float(__float_as_uint(v) & 0xffffe000u);
  return __uint_as_float((__float_as_uint(r) + 0x1000u) & 0xffffe000u);
}
__global__ void __launch_bounds__(NTHREADS, 1)
cgemm_wx_kernel(const __grid_constant__ GemmMaps maps, const b200_cgemm_args p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment of the tiles (the swizzle atom) is established by hand: the dynamic
  // shared-memory base is only guaranteed to be 16-byte aligned
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[NSTAGE], empty[NSTAGE], lo_ready[NSTAGE], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * GN;              // float column of the activation view
  const int m0 = blockIdx.y * GM;
  const int b = blockIdx.z;
  const int nk = p.K / GK;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&lo_ready[s], 4);            // one arrival per transforming warp
    }
    mbar_init(&acc_done, 1);
    fail_s = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int ks = 0; ks < nk; ++ks) {
        const int s = ks % NSTAGE;
        if (ks >= NSTAGE && !mbar_wait(&empty[s], ((ks / NSTAGE) - 1) & 1, WAIT_LIMIT)) { atomicExch(&fail_s, 1); break; }
        unsigned char *st = smem + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full[s], TX_BYTES);
        const int k0 = ks * GK;
#pragma unroll
        for (int pl = 0; pl < 4; ++pl) tma_2d(st + pl * TILE, &maps.w, k0, pl * p.M + m0, &full[s]);
#pragma unroll
        for (int j = 0; j < GN / 32; ++j) tma_2d(st + 4 * TILE + j * 4096, &maps.x, n0 + 32 * j, b * p.K + k0, &full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t d1 = tmem_base, d2 = tmem_base + GN;
      bool ok = true;
      for (int ks = 0; ks < nk && ok; ++ks) {
        const int s = ks % NSTAGE;
        const uint32_t ph = (ks / NSTAGE) & 1;
        if (!mbar_wait(&full[s], ph, WAIT_LIMIT)) { ok = false; break; }
        tc_fence_after();
        const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
        // products with the high part of the activation
#pragma unroll
        for (int kk = 0; kk < GK / 8; ++kk) {
          const uint64_t bh = b_desc(st + 4 * TILE + kk * 1024);
          const uint32_t acc = (ks > 0 || kk > 0) ? 1u : 0u;
          mma_tf32(d1, a_desc(st + 0 * TILE + kk * 32), bh, acc);
          mma_tf32(d1, a_desc(st + 1 * TILE + kk * 32), bh, 1u);
          mma_tf32(d2, a_desc(st + 2 * TILE + kk * 32), bh, acc);
          mma_tf32(d2, a_desc(st + 3 * TILE + kk * 32), bh, 1u);
        }
        // products with its low part, once the other warps have written it
        if (!mbar_wait(&lo_ready[s], ph, WAIT_LIMIT)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < GK / 8; ++kk) {
          const uint64_t bl = b_desc(st + 5 * TILE + kk * 1024);
          mma_tf32(d1, a_desc(st + 0 * TILE + kk * 32), bl, 1u);
          mma_tf32(d2, a_desc(st + 2 * TILE + kk * 32), bl, 1u);
        }
        mma_commit(&empty[s]);        // the stage may be refilled once these MMAs have read it
      }
      if (!ok) atomicExch(&fail_s, 1);
      mma_commit(&acc_done);
    }
  } else {
    // ------------------------------------------------------------------ activation split, then epilogue
    const int et = tid - 64;                    // 0..127
    bool ok = true;
    for (int ks = 0; ks < nk && ok; ++ks) {
      const int s = ks % NSTAGE;
      if (!mbar_wait(&full[s], (ks / NSTAGE) & 1, WAIT_LIMIT)) { ok = false; break; }
      const float4 *hi = reinterpret_cast<const float4 *>(smem + (size_t)s * STAGE_BYTES + 4 * TILE);
      float4 *lo = reinterpret_cast<float4 *>(smem + (size_t)s * STAGE_BYTES + 5 * TILE);
#pragma unroll
      for (int i = 0; i < TILE / 16 / 128; ++i) {
        const float4 v = hi[i * 128 + et];
        float4 r;
        r.x = tf32_low(v.x);
        r.y = tf32_low(v.y);
        r.z = tf32_low(v.z);
        r.w = tf32_low(v.w);
        lo[i * 128 + et] = r;
      }
      fence_proxy_async();                      // generic-proxy writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&lo_ready[s]);
    }
    if (!ok) atomicExch(&fail_s, 1);
    // epilogue: TMEM lane = output row; this warp reads the lane quarter it is allowed to
    if (ok && mbar_wait(&acc_done, 0, WAIT_LIMIT) && fail_s == 0) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = q * 32 + lane;
      float2 *orow = reinterpret_cast<float2 *>(p.out) + (int64_t)b * p.out_bs + (int64_t)(m0 + row) * p.out_ms + n0 / 2;
#pragma unroll 1
      for (int c = 0; c < GN / 32; ++c) {
        float v1[32], v2[32];
        const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + c * 32;
        tmem_ld32(ta, v1);
        tmem_ld32(ta + GN, v2);
        float4 *dst = reinterpret_cast<float4 *>(orow + c * 16);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          dst[j] = make_float4(v1[4 * j] - v2[4 * j + 1], v1[4 * j + 1] + v2[4 * j], v1[4 * j + 2] - v2[4 * j + 3],
                               v1[4 * j + 3] + v2[4 * j + 2]);
      }
    } else {
      atomicExch(&fail_s, 1);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (tid == 0 && fail_s) atomicExch(&g_cgemm_status, 5);
}

// ---------------------------------------------------------------------------------------------
// Weight gradients of the projections:  dW (M x N) = sum over batch and time of G[b] U[b]^H,
// G (batch, M, L), U (batch, N, L) complex64 with L contiguous: dB~ = sum dBu u^H, dC~ = sum dy x^H
// (lrnnx/ops/simplified_scan.py:139,168,495,520).  Both operands are K-major here (the contraction
// runs along their contiguous dimension), and with g', u' the float views interleaved along L
//     Re dW = g' . u',     Im dW = g' . w',   w'[2l] = -u'[2l+1],  w'[2l+1] = u'[2l]
// so the imaginary part needs a pair-swapped, sign-flipped copy of the U tile.  The swap stays
// inside 16-byte chunks, so like the TF32 low parts it is produced in shared memory at the tile's
// own (swizzled) offsets.  Six tiles per stage: G, U from the TMA; G_lo, U_lo, W, W_lo from the
// transforming warps.  The long contraction (batch x 2L floats) is cut over grid.z into pieces of 16
// stages; every CTA adds its 128 x 128 partial result to the zero-filled output with float32
// vector reductions.
constexpr uint32_t kIdescKK = kIdesc & ~(1u << 16);      // both operands K-major

struct GradMaps {
  CUtensorMap g;      // (2 L, batch M) float32, box (32, 128)
  CUtensorMap u;      // (2 L, batch N) float32, box (32, 128)
};

__global__ void __launch_bounds__(NTHREADS, 1)
cgemm_ggh_kernel(const __grid_constant__ GradMaps maps, const b200_cgemm_grad_args p, int stages_per_cta) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[NSTAGE], empty[NSTAGE], lo_ready[NSTAGE], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * GN, m0 = blockIdx.y * GM;
  const int per_batch = 2 * p.L / GK;                      // stages per batch entry
  const int total = p.batch * per_batch;
  const int s_begin = blockIdx.z * stages_per_cta;
  const int nk = min(stages_per_cta, total - s_begin);
  // tile slots of a stage: 0 G, 1 G_lo, 2 U, 3 U_lo, 4 W, 5 W_lo

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&lo_ready[s], 4);
    }
    mbar_init(&acc_done, 1);
    fail_s = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (nk > 0) {
    if (warp == 0) {
      if (lane == 0) {
        for (int ks = 0; ks < nk; ++ks) {
          const int s = ks % NSTAGE;
          if (ks >= NSTAGE && !mbar_wait(&empty[s], ((ks / NSTAGE) - 1) & 1, WAIT_LIMIT)) { atomicExch(&fail_s, 1); break; }
          unsigned char *st = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], 2 * TILE);
          const int sg = s_begin + ks;
          const int b = sg / per_batch, l0 = (sg % per_batch) * GK;
          tma_2d(st + 0 * TILE, &maps.g, l0, b * p.M + m0, &full[s]);
          tma_2d(st + 2 * TILE, &maps.u, l0, b * p.N + n0, &full[s]);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        const uint32_t dre = tmem_base, dim_ = tmem_base + GN;
        bool ok = true;
        for (int ks = 0; ks < nk && ok; ++ks) {
          const int s = ks % NSTAGE;
          const uint32_t ph = (ks / NSTAGE) & 1;
          if (!mbar_wait(&full[s], ph, WAIT_LIMIT)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
#pragma unroll
          for (int kk = 0; kk < GK / 8; ++kk)
            mma_tf32(dre, a_desc(st + 0 * TILE + kk * 32), a_desc(st + 2 * TILE + kk * 32), (ks > 0 || kk > 0) ? 1u : 0u, kIdescKK);
          if (!mbar_wait(&lo_ready[s], ph, WAIT_LIMIT)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < GK / 8; ++kk) {
            const uint64_t g = a_desc(st + 0 * TILE + kk * 32), gl = a_desc(st + 1 * TILE + kk * 32);
            const uint64_t u = a_desc(st + 2 * TILE + kk * 32), ul = a_desc(st + 3 * TILE + kk * 32);
            const uint64_t w = a_desc(st + 4 * TILE + kk * 32), wl = a_desc(st + 5 * TILE + kk * 32);
            mma_tf32(dre, gl, u, 1u, kIdescKK);
            mma_tf32(dre, g, ul, 1u, kIdescKK);
            mma_tf32(dim_, g, w, (ks > 0 || kk > 0) ? 1u : 0u, kIdescKK);
            mma_tf32(dim_, gl, w, 1u, kIdescKK);
            mma_tf32(dim_, g, wl, 1u, kIdescKK);
          }
          mma_commit(&empty[s]);
        }
        if (!ok) atomicExch(&fail_s, 1);
        mma_commit(&acc_done);
      }
    } else {
      const int et = tid - 64;
      bool ok = true;
      for (int ks = 0; ks < nk && ok; ++ks) {
        const int s = ks % NSTAGE;
        if (!mbar_wait(&full[s], (ks / NSTAGE) & 1, WAIT_LIMIT)) { ok = false; break; }
        float4 *t = reinterpret_cast<float4 *>(smem + (size_t)s * STAGE_BYTES);
        constexpr int T4 = TILE / 16;           // float4 per tile
#pragma unroll
        for (int i = 0; i < T4 / 128; ++i) {
          const int o = i * 128 + et;
          const float4 g = t[o], u = t[2 * T4 + o];
          t[T4 + o] = make_float4(tf32_low(g.x), tf32_low(g.y), tf32_low(g.z), tf32_low(g.w));
          const float4 ul = make_float4(tf32_low(u.x), tf32_low(u.y), tf32_low(u.z), tf32_low(u.w));
          t[3 * T4 + o] = ul;
          t[4 * T4 + o] = make_float4(-u.y, u.x, -u.w, u.z);
          t[5 * T4 + o] = make_float4(-ul.y, ul.x, -ul.w, ul.z);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&lo_ready[s]);
      }
      if (!ok) atomicExch(&fail_s, 1);
      if (ok && mbar_wait(&acc_done, 0, WAIT_LIMIT) && fail_s == 0) {
        tc_fence_after();
        const int q = warp & 3;
        const int row = q * 32 + lane;
        // A thread holds one output row (its TMEM lane), 32 columns at a time.  The chunk is turned
        // through shared memory (the stage buffers are free now) so that a warp adds 32 consecutive
        // complex elements of one row per instruction: coalesced {re, im} vector reductions.
        float2 *turn = reinterpret_cast<float2 *>(smem) + (size_t)q * 32 * 33;
        (void)row;
#pragma unroll 1
        for (int c = 0; c < GN / 32; ++c) {
          float vr[32], vi[32];
          const uint32_t ta = tmem_base + ((uint32_t)(q * 32) << 16) + c * 32;
          tmem_ld32(ta, vr);
          tmem_ld32(ta + GN, vi);
#pragma unroll
          for (int j = 0; j < 32; ++j) turn[lane * 33 + j] = make_float2(vr[j], vi[j]);
          __syncwarp();
          float *obase = reinterpret_cast<float *>(p.out) + ((int64_t)(m0 + q * 32) * p.N + n0 + c * 32 + lane) * 2;
#pragma unroll 8
          for (int r = 0; r < 32; ++r) {
            const float2 v = turn[r * 33 + lane];
            asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(obase + (int64_t)r * p.N * 2), "f"(v.x), "f"(v.y) : "memory");
          }
          __syncwarp();
        }
      } else {
        atomicExch(&fail_s, 1);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (tid == 0 && fail_s) atomicExch(&g_cgemm_status, 6);
}

// Weight planes for cgemm_wx_kernel: (4, M, K) float32 = tf32(Re W), tf32(Re W - that), and the same
// for Im W, from a complex64 matrix addressed by element strides (a transposed view costs nothing)
// and optionally conjugated.
__global__ void cgemm_planes_kernel(const float2 *w, int M, int K, int64_t rs, int64_t cs, int conj, float *planes) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)M * K) return;
  const int m = (int)(i / K), k = (int)(i % K);
  float2 v = w[(int64_t)m * rs + (int64_t)k * cs];
  if (conj) v.y = -v.y;
  const float rh = __uint_as_float((__float_as_uint(v.x) + 0x1000u) & 0xffffe000u);
  const float ih = __uint_as_float((__float_as_uint(v.y) + 0x1000u) & 0xffffe000u);
  const float rl = v.x - rh, il = v.y - ih;
  const int64_t MK = (int64_t)M * K;
  planes[i] = rh;
  planes[MK + i] = __uint_as_float((__float_as_uint(rl) + 0x1000u) & 0xffffe000u);
  planes[2 * MK + i] = ih;
  planes[3 * MK + i] = __uint_as_float((__float_as_uint(il) + 0x1000u) & 0xffffe000u);
}

bool make_map(CUtensorMap *m, const void *base, uint64_t inner, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
              CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {32, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int cgemm_status_read() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_cgemm_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace b200

using namespace b200;


extern "C" int b200_cgemm_grad(const b200_cgemm_grad_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "cgemm_grad: null argument block");
  const b200_cgemm_grad_args &a = *args;
  B200_REQUIRE(a.g && a.u && a.out, B200_ERR_NULL, "cgemm_grad: g, u, out must be non-null");
  B200_REQUIRE(a.batch > 0 && a.M > 0 && a.N > 0 && a.L > 0, B200_ERR_SHAPE, "cgemm_grad: sizes must be positive");
  B200_REQUIRE(a.M % GM == 0 && a.N % GN == 0 && (2 * (int64_t)a.L) % GK == 0, B200_ERR_SHAPE,
               "cgemm_grad: M and N must be multiples of %d, L of %d (got M=%d N=%d L=%d)", GM, GK / 2, a.M, a.N, a.L);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a.g) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.u) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a.out) & 7) == 0,
               B200_ERR_ALIGN, "cgemm_grad: operands must be 16-byte aligned");
  B200_REQUIRE((int64_t)a.batch * a.M < (int64_t(1) << 31) && (int64_t)a.batch * a.N < (int64_t(1) << 31), B200_ERR_SHAPE,
               "cgemm_grad: batch * rows too large");
  GradMaps maps;
  memset(&maps, 0, sizeof(maps));
  B200_REQUIRE(make_map(&maps.g, a.g, 2ull * a.L, (uint64_t)a.batch * a.M, 8ull * a.L, GM, CU_TENSOR_MAP_SWIZZLE_128B) &&
                   make_map(&maps.u, a.u, 2ull * a.L, (uint64_t)a.batch * a.N, 8ull * a.L, GN, CU_TENSOR_MAP_SWIZZLE_128B),
               B200_ERR_UNSUPPORTED, "cgemm_grad: tensor-map encoding failed");
  const int smem = NSTAGE * STAGE_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(cgemm_ggh_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return (int)e; }
  // Cut the contraction into pieces of at most 16 stages (512 floats of K).  More pieces than SMs
  // is deliberate: the tensor core adds into its float32 accumulator with truncation, a one-sided
  // error that grows linearly with the length of one accumulation chain, whereas the pieces are
  // combined by round-to-nearest float32 reductions.
  const int64_t total = (int64_t)a.batch * (2 * (int64_t)a.L / GK);
  const int per = total < 16 ? (int)total : 16;
  const int64_t splits = (total + per - 1) / per;
  B200_REQUIRE(splits <= 65535, B200_ERR_SHAPE, "cgemm_grad: batch * L too large (%lld pieces)", (long long)splits);
  const dim3 grid((unsigned)(a.N / GN), (unsigned)(a.M / GM), (unsigned)splits);
  cgemm_ggh_kernel<<<grid, NTHREADS, smem, reinterpret_cast<cudaStream_t>(stream)>>>(maps, a, per);
  return launch_status();
}

extern "C" int b200_cgemm_planes(const b200_cgemm_planes_args *args, void *stream) {
  B200_REQUIRE(args && args->w && args->planes, B200_ERR_NULL, "cgemm_planes: w and planes must be non-null");
  B200_REQUIRE(args->M > 0 && args->K > 0, B200_ERR_SHAPE, "cgemm_planes: sizes must be positive");
  const int64_t n = (int64_t)args->M * args->K;
  cgemm_planes_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float2 *>(args->w), args->M, args->K, args->w_rs, args->w_cs, args->conj,
      reinterpret_cast<float *>(args->planes));
  return launch_status();
}

extern "C" int b200_cgemm_wx(const b200_cgemm_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "cgemm_wx: null argument block");
  const b200_cgemm_args &a = *args;
  B200_REQUIRE(a.w_planes && a.x && a.out, B200_ERR_NULL, "cgemm_wx: w_planes, x, out must be non-null");
  B200_REQUIRE(a.batch > 0 && a.M > 0 && a.K > 0 && a.N > 0, B200_ERR_SHAPE, "cgemm_wx: sizes must be positive");
  B200_REQUIRE(a.M % GM == 0 && a.K % GK == 0 && (2 * (int64_t)a.N) % GN == 0, B200_ERR_SHAPE,
               "cgemm_wx: M must be a multiple of %d, K of %d, N of %d (got M=%d K=%d N=%d)", GM, GK, GN / 2, a.M, a.K, a.N);
  B200_REQUIRE(a.x_ks == a.N && a.x_bs == (int64_t)a.K * a.N, B200_ERR_UNSUPPORTED, "cgemm_wx: x must be a dense (batch, K, N) tensor");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a.w_planes) & 15) == 0 && a.out_ms % 2 == 0 && a.out_bs % 2 == 0,
               B200_ERR_ALIGN, "cgemm_wx: operands must be 16-byte aligned");
  B200_REQUIRE((int64_t)a.batch * a.K < (int64_t(1) << 31), B200_ERR_SHAPE, "cgemm_wx: batch * K too large");
  GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  B200_REQUIRE(make_map(&maps.w, a.w_planes, (uint64_t)a.K, 4ull * a.M, (uint64_t)a.K * 4, GM, CU_TENSOR_MAP_SWIZZLE_128B) &&
                   make_map(&maps.x, a.x, 2ull * a.N, (uint64_t)a.batch * a.K, 8ull * a.N, GK,
                            CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B),
               B200_ERR_UNSUPPORTED, "cgemm_wx: tensor-map encoding failed");
  const int smem = NSTAGE * STAGE_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(cgemm_wx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return (int)e; }
  const dim3 grid((unsigned)(2 * (int64_t)a.N / GN), (unsigned)(a.M / GM), (unsigned)a.batch);
  cgemm_wx_kernel<<<grid, NTHREADS, smem, reinterpret_cast<cudaStream_t>(stream)>>>(maps, a);
  return launch_status();
}
