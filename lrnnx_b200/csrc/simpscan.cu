// Simplified (diagonal, complex-input) scan for sm_100a — forward and backward.
//
// Math (csrc/simplified_scan/simplified_scan.cuh:85-262 and
// simplified_scan_backward.cuh:91-420 of lrnnx): per row (batch b, state p) and
// state slot s,  h_t = a_t h_{t-1} + k_t u_t  with complex u and
//   ZOH      a = exp(A dA_t),            k = (exp(A d_t) - 1) / A
//   BILINEAR a = (1+A dA_t/2)/(1-A dA_t/2), k = d_t / (1 - A d_t/2)
//   DIRAC    a = exp(A dA_t),            k = 1
// (dA_t = deltaA_t when given, else d_t = delta_t), out_t = sum_s h_t B_s C_s.
//
// Forward: one warp per row, 10 consecutive timesteps per lane (320 per
// stage).  Each warp runs its own 3-slot pipeline: lane 0 issues 1-D bulk
// asynchronous copies (cp.async.bulk, the TMA engine) of the stage's u / delta
// (/ deltaA) row segments into the warp's shared-memory slots and the warp
// waits on the slot's mbarrier; the 80-byte per-lane stride makes the
// lane-blocked 128-bit shared loads bank-conflict free.  The result is written
// over the u slot and leaves through a bulk shared->global copy.  Rows whose
// addresses are not 16-byte aligned, and the ragged last stage, use plain
// loads/stores on the same layout.
//
// Backward: persistent 256-thread CTAs walk the 2048-step checkpoint chunks of
// their rows in reverse with 8 timesteps per thread, so a whole chunk is
// resident in registers: states are recomputed from the chunk's checkpoint
// with a block scan, the adjoint g_t = conj(a_{t+1}) g_{t+1} + dout_t conj(C)
// runs as a reverse block scan in the same pass, and du / ddelta / ddeltaA /
// dA / dB / dC follow.  Each warp moves its own 256-step slice of a chunk:
// double-buffered bulk loads on per-warp mbarriers (a slice is refilled as
// soon as the warp holds it in registers) and bulk stores from a per-warp
// staging slice, so the one block barrier per chunk is the scan exchange.
#include <cuda.h>   // CUtensorMap and its enums (types only: the encoder is looked up at run time)

#include "common.cuh"
#include "dispatch.h"

namespace b200 {

__device__ int g_simpscan_status = 0;   // set to non-zero when a bounded barrier wait expires

namespace {

// Coefficients of one step: a (state transition) and k (input gain).  SAME: the transition uses
// the input's step size (no separate deltaA), so zero-order hold needs one complex exponential
// per step, not two.  invA = 1 / A is formed once per (row, state).
template <int DM, bool SAME>
__device__ __forceinline__ void s5_coef(cf A, cf invA, float d, float dA, cf &a, cf &k) {
  if constexpr (DM == B200_DISC_ZOH) {
    a = cexp(A * dA);
    const cf E = SAME ? a : cexp(A * d);
    k = (E - cf(1.f, 0.f)) * invA;
  } else if constexpr (DM == B200_DISC_BILINEAR) {
    const cf vA = A * (0.5f * dA);
    a = (cf(1.f, 0.f) + vA) / (cf(1.f, 0.f) - vA);
    k = (cf(1.f, 0.f) / (cf(1.f, 0.f) - A * (0.5f * d))) * d;
  } else {
    a = cexp(A * dA);
    k = cf(1.f, 0.f);
  }
}

// ------------------------------------------------------------------ forward
constexpr int FI = 10;               // timesteps per lane
constexpr int FSTAGE = 32 * FI;      // 320
constexpr int FWARPS = 2;            // rows per CTA
constexpr int FNS = 3;               // pipeline slots per warp
constexpr int F_U_BYTES = FSTAGE * 8;
constexpr int F_D_BYTES = FSTAGE * 4;

// Operands past the end of the row are zero-filled, which makes them neutral without any
// masking: delta = 0 gives a = 1 for all three methods and u = 0 gives a zero input term.
template <int DM, bool HAS_DA, bool S1>
__global__ void __launch_bounds__(FWARPS * 32, 7) simpscan_fwd_kernel(const b200_simpscan_args p) {
  constexpr int SLOT_BYTES = F_U_BYTES + F_D_BYTES * (HAS_DA ? 2 : 1);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = p.seqlen, S = S1 ? 1 : p.dstate;
  const int n_chunks = (L + kChunk - 1) / kChunk;
  const int nst = (L + FSTAGE - 1) / FSTAGE;
  // persistent warps: warp gw owns rows gw, gw + W, gw + 2W, ...; the stages of all its rows form
  // one stream that the 3-slot pipeline runs through without draining between rows
  const int64_t nrows = (int64_t)p.batch * p.dim;
  const int64_t W = (int64_t)gridDim.x * FWARPS;
  const int64_t gw = (int64_t)blockIdx.x * FWARPS + warp;
  if (gw >= nrows) return;
  const int my_rows = (int)((nrows - gw + W - 1) / W);
  const int total = my_rows * nst;
  // shared memory: [FWARPS][FNS] slots | [FWARPS][FNS] mbarriers | [FWARPS][2*S] carry
  unsigned char *wbase = smem_raw + (size_t)warp * FNS * SLOT_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (size_t)FWARPS * FNS * SLOT_BYTES) + warp * FNS;
  cf *carry = reinterpret_cast<cf *>(smem_raw + (size_t)FWARPS * FNS * SLOT_BYTES + FWARPS * FNS * 8) +
              (size_t)warp * 2 * S;

  struct RowPtrs { const cf *u; const float *d; const float *dA; cf *o; bool tma; };
  auto row_ptrs = [&](int64_t row) {
    const int b = (int)(row / p.dim), d = (int)(row % p.dim);
    RowPtrs r;
    r.u = reinterpret_cast<const cf *>(p.u) + (int64_t)b * p.u_bs + (int64_t)d * p.u_ds;
    r.d = reinterpret_cast<const float *>(p.delta) + (int64_t)b * p.delta_bs + (int64_t)d * p.delta_ds;
    r.dA = HAS_DA ? reinterpret_cast<const float *>(p.deltaA) + (int64_t)b * p.deltaA_bs + (int64_t)d * p.deltaA_ds
                  : nullptr;
    r.o = reinterpret_cast<cf *>(p.out) + (int64_t)b * p.out_bs + (int64_t)d * p.out_ds;
    r.tma = ((reinterpret_cast<uintptr_t>(r.u) | reinterpret_cast<uintptr_t>(r.d) | reinterpret_cast<uintptr_t>(r.o)) & 15) == 0;
    if (HAS_DA) r.tma = r.tma && ((reinterpret_cast<uintptr_t>(r.dA) & 15) == 0);
    return r;
  };

  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < FNS; ++k) mbar_init(&bars[k], 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncwarp();

  auto slot_u = [&](int k) { return reinterpret_cast<cf *>(wbase + (size_t)k * SLOT_BYTES); };
  auto slot_d = [&](int k) { return reinterpret_cast<float *>(wbase + (size_t)k * SLOT_BYTES + F_U_BYTES); };
  auto slot_dA = [&](int k) {
    return reinterpret_cast<float *>(wbase + (size_t)k * SLOT_BYTES + F_U_BYTES + F_D_BYTES);
  };
  // stage f of the stream: bulk (TMA) copies when the row is 16-byte aligned and the stage is
  // full, or is the last one of a row whose length is a multiple of 4 (the copies then cover the
  // valid part only and the lanes past it substitute the neutral operands in registers)
  const bool partial_ok = (L % 4) == 0;
  // The prefetch position (item pf_f = stage pf_s of row pf_row, slot pf_k) advances without
  // divisions and the row's pointers are computed once per row: index arithmetic (64-bit
  // divisions per stage) was a fifth of this kernel's instructions.
  int pf_f = 0, pf_s = 0, pf_k = 0;
  int64_t pf_row = gw;
  RowPtrs pr = row_ptrs(gw);
  auto issue = [&]() {   // lane 0 only: issues item pf_f and advances
    const int f = pf_f, s = pf_s, k = pf_k;
    if (f >= total) return;
    const RowPtrs r = pr;
    ++pf_f;
    if (++pf_k == FNS) pf_k = 0;
    if (++pf_s == nst) {
      pf_s = 0;
      pf_row += W;
      if (pf_f < total) pr = row_ptrs(pf_row);
    }
    const int valid = min(FSTAGE, L - s * FSTAGE);
    if (valid < FSTAGE && !partial_ok) return;
    if (!r.tma) return;
    const int64_t t0 = (int64_t)s * FSTAGE;
    mbar_expect_tx(&bars[k], valid * (8 + (HAS_DA ? 8 : 4)));
    bulk_g2s(slot_u(k), r.u + t0, valid * 8, &bars[k]);
    bulk_g2s(slot_d(k), r.d + t0, valid * 4, &bars[k]);
    if (HAS_DA) bulk_g2s(slot_dA(k), r.dA + t0, valid * 4, &bars[k]);
  };
  if (lane == 0) { issue(); issue(); }

  uint32_t phase_bits = 0;   // bit k: parity the next wait on slot k expects
  bool failed = false;
  RowPtrs rp = row_ptrs(gw);
  int64_t row = gw;
  cf A0, BC0, Pc0, hc0;
  bool bc_one = false;
  const cf *Ap = nullptr, *Bp = nullptr, *Cp = nullptr;
  cf *xrow = nullptr;
  int s = -1, k = -1;
  for (int f = 0; f < total; ++f) {
    if (++s == nst) s = 0;
    if (++k == FNS) k = 0;
    if (s == 0) {   // new row
      if (f > 0) row += W;
      rp = row_ptrs(row);
      const int d = (int)(row % p.dim);
      Ap = reinterpret_cast<const cf *>(p.A) + (int64_t)d * p.A_ds;
      Bp = reinterpret_cast<const cf *>(p.B) + (int64_t)d * p.B_ds;
      Cp = reinterpret_cast<const cf *>(p.C) + (int64_t)d * p.C_ds;
      xrow = reinterpret_cast<cf *>(p.x) + row * n_chunks * 2 * S;
      A0 = Ap[0];
      BC0 = Bp[0] * Cp[0];
      bc_one = S1 && BC0.re == 1.f && BC0.im == 0.f;
      Pc0 = cf(1.f, 0.f);
      hc0 = cf(0.f, 0.f);
    }
    const int t0 = s * FSTAGE;
    const int valid = min(FSTAGE, L - t0);
    const bool async_stage = rp.tma && (valid == FSTAGE || partial_ok);
    cf *su = slot_u(k);
    float *sd = slot_d(k), *sdA = slot_dA(k);
    if (async_stage) {
      if (!mbar_wait(&bars[k], (phase_bits >> k) & 1u)) { failed = true; break; }
      phase_bits ^= (1u << k);
    } else {
      // ragged or unaligned stage: coalesced plain loads into the same layout (after any bulk
      // store that still reads this slot), zero-filled past the end of the row
      if (lane == 0) bulk_wait_read<0>();
      __syncwarp();
      for (int i = lane; i < FSTAGE; i += 32) {
        const int t = t0 + i;
        su[i] = t < L ? rp.u[t] : cf(0.f, 0.f);
        sd[i] = t < L ? rp.d[t] : 0.f;
        if (HAS_DA) sdA[i] = t < L ? rp.dA[t] : 0.f;
      }
      __syncwarp();
    }
    cf u[FI];
    float dl[FI], dAv[FI];
    {
      const float4 *s4 = reinterpret_cast<const float4 *>(su + lane * FI);
#pragma unroll
      for (int j = 0; j < FI / 2; ++j) {
        const float4 v = s4[j];
        u[2 * j] = cf(v.x, v.y);
        u[2 * j + 1] = cf(v.z, v.w);
      }
      const float2 *d2 = reinterpret_cast<const float2 *>(sd + lane * FI);
      const float2 *dA2 = reinterpret_cast<const float2 *>(sdA + lane * FI);
#pragma unroll
      for (int j = 0; j < FI / 2; ++j) {
        const float2 v = d2[j];
        dl[2 * j] = v.x;
        dl[2 * j + 1] = v.y;
        if (HAS_DA) {
          const float2 w = dA2[j];
          dAv[2 * j] = w.x;
          dAv[2 * j + 1] = w.y;
        } else {
          dAv[2 * j] = v.x;
          dAv[2 * j + 1] = v.y;
        }
      }
    }
    if (valid < FSTAGE && async_stage) {   // partial bulk copy: the slot's tail holds stale data
#pragma unroll
      for (int i = 0; i < FI; ++i) {
        if (lane * FI + i >= valid) { u[i] = cf(0.f, 0.f); dl[i] = 0.f; dAv[i] = 0.f; }
      }
    }
    cf out[FI];
    if (!S1) {
#pragma unroll
      for (int i = 0; i < FI; ++i) out[i] = cf(0.f, 0.f);
    }
    // positions of this stage whose state is a checkpoint: the end of a 2048-step chunk and/or
    // the end of the row (a 320-step stage holds at most one of each)
    const int tend = min(L, t0 + FSTAGE);
    const int boundary = (tend / kChunk) * kChunk;
    const int ck_a = (boundary > t0) ? boundary - 1 - t0 : -1;
    const int ck_b = (tend == L && (L % kChunk) != 0) ? L - 1 - t0 : -1;
    // A step size that does not change over the warp's timesteps (a time-invariant system) needs
    // one coefficient evaluation instead of one per timestep.
    bool same_step = true;
#pragma unroll
    for (int i = 1; i < FI; ++i) same_step = same_step && dl[i] == dl[0] && dAv[i] == dAv[0];
    same_step = __all_sync(0xffffffffu, same_step);
    for (int si = 0; si < S; ++si) {
      const cf An = S1 ? A0 : Ap[(int64_t)si * p.A_ns];
      const cf invAn = cf(1.f, 0.f) / An;
      const cf BC = S1 ? BC0 : Bp[(int64_t)si * p.B_ns] * Cp[(int64_t)si * p.C_ns];
      cf a[FI], h[FI];
      if (same_step) {
        cf a0, k0;
        s5_coef<DM, !HAS_DA>(An, invAn, dl[0], dAv[0], a0, k0);
#pragma unroll
        for (int i = 0; i < FI; ++i) {
          a[i] = a0;
          h[i] = (DM == B200_DISC_DIRAC) ? u[i] : k0 * u[i];
        }
      } else {
#pragma unroll
        for (int i = 0; i < FI; ++i) {
          if constexpr (DM == B200_DISC_DIRAC) {
            a[i] = cexp(An * dAv[i]);
            h[i] = u[i];
          } else {
            cf kk;
            s5_coef<DM, !HAS_DA>(An, invAn, dl[i], dAv[i], a[i], kk);
            h[i] = kk * u[i];
          }
        }
      }
      cf P = a[0], hh = h[0];
#pragma unroll
      for (int i = 1; i < FI; ++i) {
        hh = a[i] * hh + h[i];
        P = P * a[i];
        h[i] = hh;
        a[i] = P;
      }
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        cf Pp = shfl_up(P, off), hp = shfl_up(hh, off);
        if (lane >= off) { hh = P * hp + hh; P = P * Pp; }
      }
      cf Pex = shfl_up(P, 1), hex = shfl_up(hh, 1);
      if (lane == 0) { Pex = cf(1.f, 0.f); hex = cf(0.f, 0.f); }
      cf Pc = Pc0, hc = hc0;
      if (!S1) {
        if (s > 0) { Pc = carry[2 * si]; hc = carry[2 * si + 1]; }
        else { Pc = cf(1.f, 0.f); hc = cf(0.f, 0.f); }
      }
      const cf hin = Pex * hc + hex;
#pragma unroll
      for (int i = 0; i < FI; ++i) {
        h[i] = a[i] * hin + h[i];
        if (S1) out[i] = bc_one ? h[i] : h[i] * BC;
        else out[i] = out[i] + h[i] * BC;
      }
      if (ck_a >= 0 || ck_b >= 0) {
        const cf Pin = Pex * Pc;
#pragma unroll
        for (int i = 0; i < FI; ++i) {
          const int pos = lane * FI + i;
          if (pos == ck_a || pos == ck_b) {
            cf *xr = xrow + (int64_t)((t0 + pos) / kChunk) * 2 * S;
            xr[2 * si] = a[i] * Pin;
            xr[2 * si + 1] = h[i];
          }
        }
      }
      const cf Ptot = shfl_idx(P, 31), htot = shfl_idx(hh, 31);
      if (S1) {
        hc0 = Ptot * hc + htot;
        Pc0 = Pc * Ptot;
      } else {
        __syncwarp();
        if (lane == 0) {
          carry[2 * si] = Pc * Ptot;
          carry[2 * si + 1] = Ptot * hc + htot;
        }
        __syncwarp();
      }
    }
    // prefetch stage f+2 into the slot used by stage f-1 (its bulk store must have finished reading)
    if (lane == 0 && f + 2 < total) {
      bulk_wait_read<0>();
      issue();
    }
    if (async_stage) {
      float4 *s4 = reinterpret_cast<float4 *>(su + lane * FI);
#pragma unroll
      for (int j = 0; j < FI / 2; ++j) s4[j] = make_float4(out[2 * j].re, out[2 * j].im, out[2 * j + 1].re, out[2 * j + 1].im);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        bulk_s2g(rp.o + t0, su, valid * 8);
        bulk_commit();
      }
    } else {
#pragma unroll
      for (int i = 0; i < FI; ++i) {
        const int t = t0 + lane * FI + i;
        if (t < L) rp.o[t] = out[i];
      }
      __syncwarp();   // the slot may be refilled by plain loads of the next stage
    }
  }
  if (lane == 0) bulk_wait<0>();
  if (failed && lane == 0) atomicExch(&g_simpscan_status, 1);
}

// ----------------------------------------------------------------- backward
// Tensor maps of the activation tensors viewed as rows of 128 bytes, with the 128-byte swizzle:
// the TMA engine XORs the 16-byte chunk index of every row with the row index (mod 8) on the way
// into shared memory, which spreads a lane's 64-byte (32-byte) run over all bank groups, so the
// lane-blocked 128-bit shared loads and stores of a warp are conflict-free.  (With linear bulk
// copies the 64-byte lane stride gives 4-way conflicts, and the shared-memory pipe, not the
// issue slots, bounded this kernel.)
struct TmaMaps {
  CUtensorMap u, dout, h, d, dA, du, dd, ddA;
};
__device__ __forceinline__ int swz128(int byte_off) { return byte_off ^ (((byte_off >> 7) & 7) << 4); }
__device__ __forceinline__ void tensor_g2s(void *dst, const CUtensorMap *map, int row, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(row), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tensor_s2g(const CUtensorMap *map, int row, const void *src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(0), "r"(row), "r"(smem_u32(src))
               : "memory");
}

constexpr int BT = 256;               // threads per CTA
constexpr int BI = 8;                 // timesteps per thread (BT*BI = 2048 = one checkpoint chunk)
constexpr int BWARPS = BT / 32;
constexpr int B_U_BYTES = kChunk * 8;
constexpr int B_D_BYTES = kChunk * 4;

struct __align__(16) BwdShared {
  cf wtot_a[2][BWARPS];     // per-warp aggregates of the forward scan (double-buffered by iteration parity)
  cf wtot_h[2][BWARPS];
  cf rtot_q[2][BWARPS];     // per-warp aggregates of the reverse scan
  cf rtot_g[2][BWARPS];
  cf red[3][BWARPS];        // block reduction scratch for dA, dB, dC
  uint64_t full[2][BWARPS]; // warp w's 256-step slice of chunk buffer k has been filled by its bulk copies
};

// NEED_BC = false skips dB / dC (the host passes null pointers: the caller scans B u with
// identity B and C and has no use for them).
template <int DM, bool HAS_DA, bool S1, bool NEED_BC, bool SWZ>
__global__ void __launch_bounds__(BT, 2)
simpscan_bwd_kernel(const b200_simpscan_args p, const __grid_constant__ TmaMaps maps) {
  constexpr int BUF_BYTES = 2 * B_U_BYTES + B_D_BYTES * (HAS_DA ? 2 : 1);   // u, dout, delta (, deltaA)
  constexpr int OUT_BYTES = B_U_BYTES + B_D_BYTES * (HAS_DA ? 2 : 1);       // du, ddelta (, ddeltaA)
  constexpr int SL = 32 * BI;                       // timesteps per warp slice
  extern __shared__ __align__(128) unsigned char smem_dyn[];
  // the swizzle pattern of the tensor copies repeats every 1024 bytes: slices start on such boundaries
  unsigned char *smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  // layout: buf[2] | out staging | BwdShared | per-state: gcar[2], accA, accB, accC (cf each)
  unsigned char *out_stage = smem_raw + 2 * (size_t)BUF_BYTES;
  BwdShared &sh = *reinterpret_cast<BwdShared *>(out_stage + OUT_BYTES);
  cf *st_arr = reinterpret_cast<cf *>(out_stage + OUT_BYTES + sizeof(BwdShared));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int L = p.seqlen, S = S1 ? 1 : p.dstate;
  const int n_chunks = (L + kChunk - 1) / kChunk;
  cf *gcar = st_arr, *accA = st_arr + 2 * S, *accB = st_arr + 3 * S, *accC = st_arr + 4 * S;
  // persistent CTAs: CTA g owns rows g, g + G, ...; the chunks of all its rows (each row walked
  // from its last chunk to its first) form one stream for the two-buffer pipeline
  const int64_t nrows = (int64_t)p.batch * p.dim;
  const int my_rows = (int)((nrows - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const int total = my_rows * n_chunks;

  struct RowPtrs { const cf *u, *dout; const float *d, *dA; cf *du; float *dd, *ddA; bool tma; };
  auto row_ptrs = [&](int64_t row) {
    const int b = (int)(row / p.dim), d = (int)(row % p.dim);
    RowPtrs r;
    r.u = reinterpret_cast<const cf *>(p.u) + (int64_t)b * p.u_bs + (int64_t)d * p.u_ds;
    r.dout = reinterpret_cast<const cf *>(p.dout) + (int64_t)b * p.dout_bs + (int64_t)d * p.dout_ds;
    r.d = reinterpret_cast<const float *>(p.delta) + (int64_t)b * p.delta_bs + (int64_t)d * p.delta_ds;
    r.dA = HAS_DA ? reinterpret_cast<const float *>(p.deltaA) + (int64_t)b * p.deltaA_bs + (int64_t)d * p.deltaA_ds
                  : nullptr;
    r.du = reinterpret_cast<cf *>(p.du) + (int64_t)b * p.du_bs + (int64_t)d * p.du_ds;
    r.dd = reinterpret_cast<float *>(p.ddelta) + (int64_t)b * p.ddelta_bs + (int64_t)d * p.ddelta_ds;
    r.ddA = HAS_DA ? reinterpret_cast<float *>(p.ddeltaA) + (int64_t)b * p.ddeltaA_bs + (int64_t)d * p.ddeltaA_ds
                   : nullptr;
    r.tma = ((reinterpret_cast<uintptr_t>(r.u) | reinterpret_cast<uintptr_t>(r.dout) | reinterpret_cast<uintptr_t>(r.d) |
              reinterpret_cast<uintptr_t>(r.du) | reinterpret_cast<uintptr_t>(r.dd)) & 15) == 0;
    if (HAS_DA) r.tma = r.tma && (((reinterpret_cast<uintptr_t>(r.dA) | reinterpret_cast<uintptr_t>(r.ddA)) & 15) == 0);
    return r;
  };
  auto buf_u = [&](int k) { return reinterpret_cast<cf *>(smem_raw + (size_t)k * BUF_BYTES); };
  auto buf_do = [&](int k) { return reinterpret_cast<cf *>(smem_raw + (size_t)k * BUF_BYTES + B_U_BYTES); };
  auto buf_d = [&](int k) { return reinterpret_cast<float *>(smem_raw + (size_t)k * BUF_BYTES + 2 * B_U_BYTES); };
  auto buf_dA = [&](int k) {
    return reinterpret_cast<float *>(smem_raw + (size_t)k * BUF_BYTES + 2 * B_U_BYTES + B_D_BYTES);
  };
  // stream item f: row blockIdx.x + (f / n_chunks) * gridDim.x, chunk n_chunks - 1 - f % n_chunks.
  // Every warp runs its own pipeline on its 256-step slice of the chunk: lane 0 issues the
  // slice's bulk loads and stores, the warp alone reads and writes the slice, so loads and
  // stores need no block-wide synchronisation.
  // the prefetch position (item pf_f = row pf_row, chunk pf_c) advances without divisions and the
  // tensor-copy path needs no row pointers
  int pf_f = 0, pf_c = n_chunks - 1;
  int64_t pf_row = blockIdx.x;
  auto issue = [&]() {   // lane 0 of a warp: issues item pf_f and advances
    const int f = pf_f, c = pf_c;
    const int64_t frow = pf_row;
    if (f >= total) return;
    ++pf_f;
    if (--pf_c < 0) { pf_c = n_chunks - 1; pf_row += gridDim.x; }
    if ((c + 1) * kChunk > L) return;
    RowPtrs r = RowPtrs();
    if (!SWZ) {
      r = row_ptrs(frow);
      if (!r.tma) return;
    }
    const int k = f & 1;
    const int64_t t0 = (int64_t)c * kChunk + warp * SL;
    uint64_t *bar = &sh.full[k][warp];
    mbar_expect_tx(bar, BUF_BYTES / BWARPS);
    if (SWZ) {   // rows of 128 bytes of the contiguous (batch, dim, seqlen) tensors
      const int64_t e0 = frow * L + t0;
      const int rc = (int)(e0 >> 4), rf = (int)(e0 >> 5);
      tensor_g2s(buf_u(k) + warp * SL, &maps.u, rc, bar);
      tensor_g2s(buf_do(k) + warp * SL, &maps.dout, rc, bar);
      tensor_g2s(buf_d(k) + warp * SL, &maps.d, rf, bar);
      if (HAS_DA) tensor_g2s(buf_dA(k) + warp * SL, &maps.dA, rf, bar);
    } else {
      bulk_g2s(buf_u(k) + warp * SL, r.u + t0, B_U_BYTES / BWARPS, bar);
      bulk_g2s(buf_do(k) + warp * SL, r.dout + t0, B_U_BYTES / BWARPS, bar);
      bulk_g2s(buf_d(k) + warp * SL, r.d + t0, B_D_BYTES / BWARPS, bar);
      if (HAS_DA) bulk_g2s(buf_dA(k) + warp * SL, r.dA + t0, B_D_BYTES / BWARPS, bar);
    }
  };

  if (tid == 0) {
    for (int i = 0; i < 2 * BWARPS; ++i) mbar_init(&sh.full[0][0] + i, 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (lane == 0) { issue(); issue(); }

  // A bounded wait that expires marks the thread as failed; a failed thread skips every later
  // wait and its warp stores no further du / ddelta (the status word says that the outputs are
  // incomplete) but keeps taking part in the block barriers, so the CTA always terminates.
  bool failed = false;
  auto wait = [&](uint64_t *bar, uint32_t parity) {
    if (!failed && !mbar_wait(bar, parity, 1u << 21)) failed = true;
  };
  uint32_t full_phase = 0;
  uint32_t iter = 0;          // (chunk, state) iterations so far: parity of the exchange arrays
  bool stores_pending = false;
  RowPtrs rp = row_ptrs(blockIdx.x);
  int64_t row = blockIdx.x;
  const cf *Ap = nullptr, *Cp = nullptr, *xrow = nullptr;
  cf A0, C0;
  bool c_one = false;
  cf dA_acc, dB_acc, dC_acc;   // per-thread partial sums over the row (single-state rows)
  int j = -1;
  for (int f = 0; f < total; ++f) {
    if (++j == n_chunks) j = 0;
    const int c = n_chunks - 1 - j;
    if (j == 0) {   // new row
      if (f > 0) row += gridDim.x;
      rp = row_ptrs(row);
      const int d = (int)(row % p.dim);
      Ap = reinterpret_cast<const cf *>(p.A) + (int64_t)d * p.A_ds;
      Cp = reinterpret_cast<const cf *>(p.C) + (int64_t)d * p.C_ds;
      xrow = p.x ? reinterpret_cast<const cf *>(p.x) + row * n_chunks * 2 * S : nullptr;
      A0 = Ap[0];
      C0 = Cp[0];
      c_one = S1 && C0.re == 1.f && C0.im == 0.f;
      dA_acc = dB_acc = dC_acc = cf(0.f, 0.f);
      if (!S1) {
        __syncthreads();   // the previous row's tail has consumed acc*
        for (int i = tid; i < S; i += BT) accA[i] = accB[i] = accC[i] = cf(0.f, 0.f);
      }
    }
    const int k = f & 1;
    const int t0 = c * kChunk;
    const bool async_chunk = rp.tma && (c + 1) * kChunk <= L;
    cf *su = buf_u(k), *sdo = buf_do(k);
    float *sd = buf_d(k), *sdA = buf_dA(k);
    if (async_chunk) {
      wait(&sh.full[k][warp], (full_phase >> k) & 1u);
      full_phase ^= (1u << k);
    } else {
      for (int i = warp * SL + lane; i < (warp + 1) * SL; i += 32) {
        const int t = t0 + i;
        su[i] = t < L ? rp.u[t] : cf(0.f, 0.f);
        sdo[i] = t < L ? rp.dout[t] : cf(0.f, 0.f);
        sd[i] = t < L ? rp.d[t] : 0.f;
        if (HAS_DA) sdA[i] = t < L ? rp.dA[t] : 0.f;
      }
      __syncwarp();
    }

    cf u[BI], dy[BI];
    float dl[BI], dAv[BI];
    // slice layout: swizzled by the tensor copies, linear after plain loads
    const bool sw = SWZ && async_chunk;
    auto off_c = [&](int q) { const int o = lane * 64 + q * 16; return sw ? swz128(o) : o; };   // complex slices
    auto off_f = [&](int q) { const int o = lane * 32 + q * 16; return sw ? swz128(o) : o; };   // float slices
    {
      const unsigned char *s4 = reinterpret_cast<const unsigned char *>(su + warp * SL);
      const unsigned char *o4 = reinterpret_cast<const unsigned char *>(sdo + warp * SL);
#pragma unroll
      for (int q = 0; q < BI / 2; ++q) {
        const int o = off_c(q);
        const float4 v = *reinterpret_cast<const float4 *>(s4 + o), w = *reinterpret_cast<const float4 *>(o4 + o);
        u[2 * q] = cf(v.x, v.y);
        u[2 * q + 1] = cf(v.z, v.w);
        dy[2 * q] = cf(w.x, w.y);
        dy[2 * q + 1] = cf(w.z, w.w);
      }
      const unsigned char *d4 = reinterpret_cast<const unsigned char *>(sd + warp * SL);
      const unsigned char *dA4 = reinterpret_cast<const unsigned char *>(sdA + warp * SL);
#pragma unroll
      for (int q = 0; q < BI / 4; ++q) {
        const int o = off_f(q);
        const float4 v = *reinterpret_cast<const float4 *>(d4 + o);
        dl[4 * q] = v.x; dl[4 * q + 1] = v.y; dl[4 * q + 2] = v.z; dl[4 * q + 3] = v.w;
        if (HAS_DA) {
          const float4 w = *reinterpret_cast<const float4 *>(dA4 + o);
          dAv[4 * q] = w.x; dAv[4 * q + 1] = w.y; dAv[4 * q + 2] = w.z; dAv[4 * q + 3] = w.w;
        }
      }
      if (!HAS_DA) {
#pragma unroll
        for (int i = 0; i < BI; ++i) dAv[i] = dl[i];
      }
    }
    // the warp's slice now lives in registers: refill it with the stream item two steps ahead
    __syncwarp();
    if (lane == 0) issue();
    bool same_step = true;
#pragma unroll
    for (int i = 1; i < BI; ++i) same_step = same_step && dl[i] == dl[0] && dAv[i] == dAv[0];
    same_step = __all_sync(0xffffffffu, same_step);
    cf du[BI];
    float ddl[BI], ddA[BI];
    if (!S1) {
#pragma unroll
      for (int i = 0; i < BI; ++i) { du[i] = cf(0.f, 0.f); ddl[i] = 0.f; ddA[i] = 0.f; }
    }

    for (int si = 0; si < S; ++si) {
      const int par = iter & 1;
      ++iter;
      const cf An = S1 ? A0 : Ap[(int64_t)si * p.A_ns];
      const cf invAn = cf(1.f, 0.f) / An;
      const cf Cc = conj(S1 ? C0 : Cp[(int64_t)si * p.C_ns]);
      // checkpoint of the previous chunk: issued early so the load overlaps the local scans
      cf hpre = cf(0.f, 0.f);
      if (c > 0) hpre = xrow[(int64_t)(c - 1) * 2 * S + 2 * si + 1];
      constexpr bool kUnitK = (DM == B200_DISC_DIRAC);   // k_t = 1: the input term is u_t itself
      cf a[BI], kk[kUnitK ? 1 : BI], h[BI];
      if (same_step) {   // time-invariant step size: one coefficient evaluation for the thread
        cf a0, k0;
        s5_coef<DM, !HAS_DA>(An, invAn, dl[0], dAv[0], a0, k0);
#pragma unroll
        for (int i = 0; i < BI; ++i) {
          a[i] = a0;
          if constexpr (!kUnitK) kk[i] = k0;
        }
      } else {
#pragma unroll
        for (int i = 0; i < BI; ++i) {
          if constexpr (kUnitK) a[i] = cexp(An * dAv[i]);
          else s5_coef<DM, !HAS_DA>(An, invAn, dl[i], dAv[i], a[i], kk[i]);
        }
      }
      auto beta = [&](int i) { return kUnitK ? u[i] : kk[kUnitK ? 0 : i] * u[i]; };
      auto seed = [&](int i) { return c_one ? dy[i] : dy[i] * Cc; };   // dout_t conj(C)
      // forward, pass 1: per-thread aggregate of h_t = a_t h_{t-1} + beta_t
      cf P = cf(1.f, 0.f), hh = cf(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < BI; ++i) {
        hh = a[i] * hh + beta(i);
        P = P * a[i];
      }
      // reverse, pass 1.  Inside a thread the adjoint g_t = seed_t + conj(a_{t+1}) g_{t+1} runs
      // on g itself; across threads, warps and chunks it is carried as q_t = conj(a_t) g_t, so
      // every transition used is the thread's own (no coefficient crosses a boundary) and the
      // thread's transition product is the conjugate of the forward one.
      cf gg = seed(BI - 1), Q = conj(P);
#pragma unroll
      for (int i = BI - 2; i >= 0; --i) gg = conj(a[i + 1]) * gg + seed(i);
      gg = conj(a[0]) * gg;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const cf Pp = shfl_up(P, off), hp = shfl_up(hh, off);
        const cf Qr = shfl_down(Q, off), gr = shfl_down(gg, off);
        if (lane >= off) { hh = P * hp + hh; P = P * Pp; }
        if (lane + off < 32) { gg = gg + Q * gr; Q = Q * Qr; }
      }
      if (lane == 31) { sh.wtot_a[par][warp] = P; sh.wtot_h[par][warp] = hh; }
      if (lane == 0) { sh.rtot_q[par][warp] = Q; sh.rtot_g[par][warp] = gg; }
      __syncthreads();   // the only block barrier of the iteration
      for (int w = 0; w < warp; ++w) hpre = sh.wtot_a[par][w] * hpre + sh.wtot_h[par][w];
      cf qpost = (j == 0) ? cf(0.f, 0.f) : gcar[(f & 1) * S + si];   // q entering the chunk from the later one
      for (int w = BWARPS - 1; w > warp; --w) qpost = sh.rtot_g[par][w] + sh.rtot_q[par][w] * qpost;
      cf Pex = shfl_up(P, 1), hex = shfl_up(hh, 1);
      if (lane == 0) { Pex = cf(1.f, 0.f); hex = cf(0.f, 0.f); }
      const cf hin = Pex * hpre + hex;       // state entering this thread's first item
      const cf g_right = shfl_down(gg, 1), Q_right = shfl_down(Q, 1);
      cf qin = g_right + Q_right * qpost;    // q of the first item of the next thread
      if (lane == 31) qin = qpost;
      if (tid == 0) gcar[((f + 1) & 1) * S + si] = gg + Q * qpost;   // q of the first step of this chunk
      // forward, pass 2: the states
      {
        cf hc = hin;
#pragma unroll
        for (int i = 0; i < BI; ++i) {
          hc = a[i] * hc + beta(i);
          h[i] = hc;
        }
      }
      // reverse, pass 2: adjoints and gradients
      cf dA_l = cf(0.f, 0.f), dB_l = cf(0.f, 0.f), dC_l = cf(0.f, 0.f);
      cf q = qin;
#pragma unroll
      for (int i = BI - 1; i >= 0; --i) {
        const cf hprev = (i == 0) ? hin : h[i - 1];
        const cf G = (i == BI - 1) ? seed(i) + q : conj(a[i == BI - 1 ? i : i + 1]) * q + seed(i);   // g_t
        q = G;
        const cf t = G * conj(h[i] - beta(i));   // g_t conj(a_t h_{t-1}), with a_t h_{t-1} = h_t - beta_t
        const float dv = dl[i], dav = dAv[i];
        if constexpr (kUnitK) {
          du[i] = S1 ? G : du[i] + G;
          if (NEED_BC) dB_l = dB_l + G * conj(u[i]);
        } else {
          du[i] = S1 ? G * conj(kk[kUnitK ? 0 : i]) : du[i] + G * conj(kk[kUnitK ? 0 : i]);
          if (NEED_BC) dB_l = dB_l + G * conj(beta(i));
        }
        if (NEED_BC) dC_l = dC_l + dy[i] * conj(h[i]);
        float d_dl = 0.f, d_dA = 0.f;
        if constexpr (DM == B200_DISC_ZOH) {
          const cf E = HAS_DA ? kk[kUnitK ? 0 : i] * An + cf(1.f, 0.f) : a[i];   // exp(A dv) = 1 + k A
          d_dA = (t * conj(An)).re;
          d_dl = (G * conj(E * u[i])).re;
          dA_l = dA_l + t * dav + G * conj(u[i] * ((E * dv - kk[kUnitK ? 0 : i]) * invAn));
        } else if constexpr (DM == B200_DISC_BILINEAR) {
          const cf r = cf(1.f, 0.f) / (cf(1.f, 0.f) - An * (0.5f * dv));
          const cf rA = cf(1.f, 0.f) / (cf(1.f, 0.f) - An * (0.5f * dav));
          const cf r2 = r * r, rA2 = rA * rA;
          d_dA = (G * conj(hprev * An * rA2)).re;
          d_dl = (G * conj(r2 * u[i])).re;
          dA_l = dA_l + G * conj(hprev * rA2 * dav + r2 * u[i] * (0.5f * dv * dv));
        } else {
          d_dA = (t * conj(An)).re;
          dA_l = dA_l + t * dav;
        }
        if (S1) {
          if (HAS_DA) { ddl[i] = d_dl; ddA[i] = d_dA; }
          else ddl[i] = d_dl + d_dA;
        } else {
          if (HAS_DA) { ddl[i] += d_dl; ddA[i] += d_dA; }
          else ddl[i] += d_dl + d_dA;
        }
      }
      if (S1) {
        dA_acc = dA_acc + dA_l;
        dB_acc = dB_acc + dB_l;
        dC_acc = dC_acc + dC_l;
      } else {
        dA_l = warp_sum(dA_l);
        dB_l = warp_sum(dB_l);
        dC_l = warp_sum(dC_l);
        // sh.red is free: its readers of the previous iteration arrived at this iteration's barrier
        if (lane == 0) { sh.red[0][warp] = dA_l; sh.red[1][warp] = dB_l; sh.red[2][warp] = dC_l; }
        __syncthreads();
        if (tid < 3) {
          cf acc = cf(0.f, 0.f);
#pragma unroll
          for (int w = 0; w < BWARPS; ++w) acc = acc + sh.red[tid][w];
          cf *dst = tid == 0 ? accA : (tid == 1 ? accB : accC);
          dst[si] = dst[si] + acc;
        }
      }
    }
    // ---- write du / ddelta (/ ddeltaA) through the staging area
    if (async_chunk) {
      if (lane == 0 && stores_pending) bulk_wait_read<0>();   // the warp's previous stores have left its staging slice
      __syncwarp();
      cf *so = reinterpret_cast<cf *>(out_stage);
      float *sod = reinterpret_cast<float *>(out_stage + B_U_BYTES);
      float *sodA = reinterpret_cast<float *>(out_stage + B_U_BYTES + B_D_BYTES);
      unsigned char *s4 = reinterpret_cast<unsigned char *>(so + warp * SL);
#pragma unroll
      for (int q = 0; q < BI / 2; ++q)
        *reinterpret_cast<float4 *>(s4 + off_c(q)) = make_float4(du[2 * q].re, du[2 * q].im, du[2 * q + 1].re, du[2 * q + 1].im);
      unsigned char *d4 = reinterpret_cast<unsigned char *>(sod + warp * SL);
#pragma unroll
      for (int q = 0; q < BI / 4; ++q)
        *reinterpret_cast<float4 *>(d4 + off_f(q)) = make_float4(ddl[4 * q], ddl[4 * q + 1], ddl[4 * q + 2], ddl[4 * q + 3]);
      if (HAS_DA) {
        unsigned char *dA4 = reinterpret_cast<unsigned char *>(sodA + warp * SL);
#pragma unroll
        for (int q = 0; q < BI / 4; ++q)
          *reinterpret_cast<float4 *>(dA4 + off_f(q)) = make_float4(ddA[4 * q], ddA[4 * q + 1], ddA[4 * q + 2], ddA[4 * q + 3]);
      }
      fence_proxy_async();
      __syncwarp();
      const bool warp_failed = __any_sync(0xffffffffu, failed);   // a warp that gave up on a wait stores nothing more
      if (lane == 0 && !warp_failed) {
        const int w0 = warp * SL;
        if (SWZ) {
          const int64_t e0 = row * L + t0 + w0;
          tensor_s2g(&maps.du, (int)(e0 >> 4), so + w0);
          tensor_s2g(&maps.dd, (int)(e0 >> 5), sod + w0);
          if (HAS_DA) tensor_s2g(&maps.ddA, (int)(e0 >> 5), sodA + w0);
        } else {
          bulk_s2g(rp.du + t0 + w0, so + w0, B_U_BYTES / BWARPS);
          bulk_s2g(rp.dd + t0 + w0, sod + w0, B_D_BYTES / BWARPS);
          if (HAS_DA) bulk_s2g(rp.ddA + t0 + w0, sodA + w0, B_D_BYTES / BWARPS);
        }
        bulk_commit();
      }
      stores_pending = true;
    } else {
#pragma unroll
      for (int i = 0; i < BI; ++i) {
        const int t = t0 + tid * BI + i;
        if (t < L && !failed) {
          rp.du[t] = du[i];
          rp.dd[t] = ddl[i];
          if (HAS_DA) rp.ddA[t] = ddA[i];
        }
      }
    }
    // ---- end of a row: fold the parameter gradients into dA / dB / dC
    if (c == 0) {
      const int d = (int)(row % p.dim);
      cf *dAp = reinterpret_cast<cf *>(p.dA) + (int64_t)d * p.A_ds;
      cf *dBp = NEED_BC ? reinterpret_cast<cf *>(p.dB) + (int64_t)d * p.B_ds : nullptr;
      cf *dCp = NEED_BC ? reinterpret_cast<cf *>(p.dC) + (int64_t)d * p.C_ds : nullptr;
      if (S1) {
        const cf ra = warp_sum(dA_acc);
        cf rb, rc;
        if (NEED_BC) { rb = warp_sum(dB_acc); rc = warp_sum(dC_acc); }
        __syncthreads();   // sh.red is free (its readers of the previous row are done)
        if (lane == 0) { sh.red[0][warp] = ra; sh.red[1][warp] = rb; sh.red[2][warp] = rc; }
        __syncthreads();
        if (tid < (NEED_BC ? 3 : 1)) {
          cf acc = cf(0.f, 0.f);
#pragma unroll
          for (int w = 0; w < BWARPS; ++w) acc = acc + sh.red[tid][w];
          cf *dst = tid == 0 ? dAp : (tid == 1 ? dBp : dCp);
          atomicAdd(&dst->re, acc.re);
          atomicAdd(&dst->im, acc.im);
        }
      } else {
        __syncthreads();
        for (int i = tid; i < S; i += BT) {
          atomicAdd(&dAp[(int64_t)i * p.A_ns].re, accA[i].re);
          atomicAdd(&dAp[(int64_t)i * p.A_ns].im, accA[i].im);
          if (NEED_BC) {
            atomicAdd(&dBp[(int64_t)i * p.B_ns].re, accB[i].re);
            atomicAdd(&dBp[(int64_t)i * p.B_ns].im, accB[i].im);
            atomicAdd(&dCp[(int64_t)i * p.C_ns].re, accC[i].re);
            atomicAdd(&dCp[(int64_t)i * p.C_ns].im, accC[i].im);
          }
        }
      }
    }
  }
  if (lane == 0) bulk_wait<0>();
  __syncthreads();
  if (failed) atomicExch(&g_simpscan_status, 2);
}

// --------------------------------------------- backward from the forward output (single state)
// For single-state rows the forward output is the state sequence itself, out_t = h_t B C.  When
// the caller hands it back (the autograd wrapper keeps it anyway), the backward needs no forward
// recomputation at all: a_t h_{t-1} = h_t - beta_t, so only the reverse (adjoint) scan is left.
// Without the checkpoints the tile size is free: 128-thread CTAs walk 1024-step tiles (four
// CTAs per SM), each warp with its own 256-step slice pipeline; du and ddelta are written over
// the u / delta slices in shared memory and leave through bulk stores.  8 bytes per element more
// traffic than the recomputing kernel, a third fewer instructions.
constexpr int HSL = 32 * BI;          // 256 timesteps per warp slice

template <int HWARPS> struct __align__(16) BwdHShared {
  cf rtot_q[2][HWARPS];     // per-warp aggregates of the reverse scan (double-buffered by tile parity)
  cf rtot_g[2][HWARPS];
  cf red[3][HWARPS];
  cf gcar[2];               // q entering the tile from the later one (double-buffered)
  uint64_t full_rw[2][HWARPS];   // u / delta slices (double-buffered: outputs are written over them)
  uint64_t full_ro[HWARPS];      // dout / h slices (single: refilled as soon as they sit in registers)
};

template <int DM, bool HAS_DA, bool NEED_BC, int HT, bool SWZ>
__global__ void __launch_bounds__(HT, 512 / HT)
simpscan_bwd_h_kernel(const b200_simpscan_args p, const __grid_constant__ TmaMaps maps) {
  constexpr int HWARPS = HT / 32, HTILE = HT * BI;   // warps per CTA, timesteps per tile
  constexpr int WU = HSL * 8, WD = HSL * 4;
  constexpr int ROB = 2 * WU;                             // dout | h of one warp slice (read-only)
  constexpr int RWB = WU + WD * (HAS_DA ? 2 : 1);         // u | delta (| deltaA): overwritten by du | ddelta (| ddeltaA)
  extern __shared__ __align__(128) unsigned char smem_dyn[];
  // the swizzle pattern repeats every 1024 bytes: slices start on 1024-byte boundaries
  unsigned char *smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  BwdHShared<HWARPS> &sh = *reinterpret_cast<BwdHShared<HWARPS> *>(smem_raw + HWARPS * (ROB + 2 * RWB));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int L = p.seqlen;
  const int n_tiles = (L + HTILE - 1) / HTILE;
  const int64_t nrows = (int64_t)p.batch * p.dim;
  const int my_rows = (int)((nrows - blockIdx.x + gridDim.x - 1) / gridDim.x);
  const int total = my_rows * n_tiles;

  struct RowPtrs { const cf *u, *dout, *h; const float *d, *dA; cf *du; float *dd, *ddA; bool tma; };
  auto row_ptrs = [&](int64_t row) {
    const int b = (int)(row / p.dim), d = (int)(row % p.dim);
    RowPtrs r;
    r.u = reinterpret_cast<const cf *>(p.u) + (int64_t)b * p.u_bs + (int64_t)d * p.u_ds;
    r.dout = reinterpret_cast<const cf *>(p.dout) + (int64_t)b * p.dout_bs + (int64_t)d * p.dout_ds;
    r.h = reinterpret_cast<const cf *>(p.out) + (int64_t)b * p.out_bs + (int64_t)d * p.out_ds;
    r.d = reinterpret_cast<const float *>(p.delta) + (int64_t)b * p.delta_bs + (int64_t)d * p.delta_ds;
    r.dA = HAS_DA ? reinterpret_cast<const float *>(p.deltaA) + (int64_t)b * p.deltaA_bs + (int64_t)d * p.deltaA_ds
                  : nullptr;
    r.du = reinterpret_cast<cf *>(p.du) + (int64_t)b * p.du_bs + (int64_t)d * p.du_ds;
    r.dd = reinterpret_cast<float *>(p.ddelta) + (int64_t)b * p.ddelta_bs + (int64_t)d * p.ddelta_ds;
    r.ddA = HAS_DA ? reinterpret_cast<float *>(p.ddeltaA) + (int64_t)b * p.ddeltaA_bs + (int64_t)d * p.ddeltaA_ds
                   : nullptr;
    r.tma = ((reinterpret_cast<uintptr_t>(r.u) | reinterpret_cast<uintptr_t>(r.dout) | reinterpret_cast<uintptr_t>(r.h) |
              reinterpret_cast<uintptr_t>(r.d) | reinterpret_cast<uintptr_t>(r.du) | reinterpret_cast<uintptr_t>(r.dd)) & 15) == 0;
    if (HAS_DA) r.tma = r.tma && (((reinterpret_cast<uintptr_t>(r.dA) | reinterpret_cast<uintptr_t>(r.ddA)) & 15) == 0);
    return r;
  };
  unsigned char *ro = smem_raw + (size_t)warp * ROB;
  auto rwbuf = [&](int k) { return smem_raw + (size_t)HWARPS * ROB + (size_t)(k * HWARPS + warp) * RWB; };
  // stream item f: row blockIdx.x + (f / n_tiles) * gridDim.x, tile n_tiles - 1 - f % n_tiles.
  // The prefetch position (item pf_f = row pf_row, tile pf_c) advances without divisions, and the
  // tensor-copy path needs no row pointers at all: index arithmetic was a fifth of this kernel.
  int pf_f = 0, pf_c = n_tiles - 1;
  int64_t pf_row = blockIdx.x;
  auto advance = [&]() {
    ++pf_f;
    if (--pf_c < 0) { pf_c = n_tiles - 1; pf_row += gridDim.x; }
  };
  // `which` selects the read-only slices (1), the overwritten ones (2) or both (3) of item pf_f
  auto issue = [&](int which) {   // lane 0 of a warp
    const int f = pf_f, c = pf_c;
    if (f >= total) return;
    if ((c + 1) * HTILE > L) return;
    RowPtrs r = RowPtrs();
    if (!SWZ) {
      r = row_ptrs(pf_row);
      if (!r.tma) return;
    }
    const int64_t t0 = (int64_t)c * HTILE + warp * HSL;
    // row of 128 bytes at which the slice starts in a contiguous (batch, dim, seqlen) tensor
    const int64_t e0 = pf_row * L + t0;
    const int rc = (int)(e0 >> 4), rf = (int)(e0 >> 5);   // complex64 / float32 tensors
    if (which & 1) {
      uint64_t *bar = &sh.full_ro[warp];
      mbar_expect_tx(bar, ROB);
      if (SWZ) {
        tensor_g2s(ro, &maps.dout, rc, bar);
        tensor_g2s(ro + WU, &maps.h, rc, bar);
      } else {
        bulk_g2s(ro, r.dout + t0, WU, bar);
        bulk_g2s(ro + WU, r.h + t0, WU, bar);
      }
    }
    if (which & 2) {
      unsigned char *s = rwbuf(f & 1);
      uint64_t *bar = &sh.full_rw[f & 1][warp];
      mbar_expect_tx(bar, RWB);
      if (SWZ) {
        tensor_g2s(s, &maps.u, rc, bar);
        tensor_g2s(s + WU, &maps.d, rf, bar);
        if (HAS_DA) tensor_g2s(s + WU + WD, &maps.dA, rf, bar);
      } else {
        bulk_g2s(s, r.u + t0, WU, bar);
        bulk_g2s(s + WU, r.d + t0, WD, bar);
        if (HAS_DA) bulk_g2s(s + WU + WD, r.dA + t0, WD, bar);
      }
    }
  };

  if (tid == 0) {
    for (int i = 0; i < 2 * HWARPS; ++i) mbar_init(&sh.full_rw[0][0] + i, 1);
    for (int i = 0; i < HWARPS; ++i) mbar_init(&sh.full_ro[i], 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (lane == 0) issue(3);
  advance();

  bool failed = false;
  auto wait = [&](uint64_t *bar, uint32_t parity) {
    if (!failed && !mbar_wait(bar, parity, 1u << 21)) failed = true;
  };
  uint32_t full_phase = 0;   // bits 0, 1: the two overwritten buffers; bit 2: the read-only slices
  bool stores_pending = false;
  RowPtrs rp = row_ptrs(blockIdx.x);
  int64_t row = blockIdx.x;
  cf A0, invA0, Cc, inv_bc;
  bool c_one = false, bc_one = false;
  cf dA_acc, dB_acc, dC_acc;
  int j = -1;
  for (int f = 0; f < total; ++f) {
    if (++j == n_tiles) j = 0;
    const int c = n_tiles - 1 - j;
    if (j == 0) {   // new row
      if (f > 0) row += gridDim.x;
      rp = row_ptrs(row);
      const int d = (int)(row % p.dim);
      A0 = reinterpret_cast<const cf *>(p.A)[(int64_t)d * p.A_ds];
      invA0 = cf(1.f, 0.f) / A0;
      const cf B0 = reinterpret_cast<const cf *>(p.B)[(int64_t)d * p.B_ds];
      const cf C0 = reinterpret_cast<const cf *>(p.C)[(int64_t)d * p.C_ds];
      const cf bc = B0 * C0;
      Cc = conj(C0);
      c_one = C0.re == 1.f && C0.im == 0.f;
      bc_one = bc.re == 1.f && bc.im == 0.f;
      inv_bc = cf(1.f, 0.f) / bc;
      dA_acc = dB_acc = dC_acc = cf(0.f, 0.f);
    }
    const int k = f & 1;
    const int t0 = c * HTILE;                 // first step of the tile
    const int tw = t0 + warp * HSL;           // first step of this warp's slice
    const bool async_tile = rp.tma && (c + 1) * HTILE <= L;
    unsigned char *s = rwbuf(k);
    cf *su = reinterpret_cast<cf *>(s), *sdo = reinterpret_cast<cf *>(ro), *shh = reinterpret_cast<cf *>(ro + WU);
    float *sd = reinterpret_cast<float *>(s + WU), *sdA = reinterpret_cast<float *>(s + WU + WD);
    if (async_tile) {
      wait(&sh.full_rw[k][warp], (full_phase >> k) & 1u);
      wait(&sh.full_ro[warp], (full_phase >> 2) & 1u);
      full_phase ^= (1u << k) | 4u;
    } else {
      for (int i = lane; i < HSL; i += 32) {
        const int t = tw + i;
        su[i] = t < L ? rp.u[t] : cf(0.f, 0.f);
        sdo[i] = t < L ? rp.dout[t] : cf(0.f, 0.f);
        shh[i] = t < L ? rp.h[t] : cf(0.f, 0.f);
        sd[i] = t < L ? rp.d[t] : 0.f;
        if (HAS_DA) sdA[i] = t < L ? rp.dA[t] : 0.f;
      }
      __syncwarp();
    }
    cf u[BI], dy[BI], h[BI];
    float dl[BI], dAv[BI];
    const bool sw = SWZ && async_tile;      // swizzled (tensor copy) or linear (plain loads) slice layout
    auto off_c = [&](int q) { const int o = lane * 64 + q * 16; return sw ? swz128(o) : o; };   // complex slices
    auto off_f = [&](int q) { const int o = lane * 32 + q * 16; return sw ? swz128(o) : o; };   // float slices
    {
      const unsigned char *s4 = reinterpret_cast<const unsigned char *>(su);
      const unsigned char *o4 = reinterpret_cast<const unsigned char *>(sdo);
      const unsigned char *h4 = reinterpret_cast<const unsigned char *>(shh);
#pragma unroll
      for (int q = 0; q < BI / 2; ++q) {
        const int o = off_c(q);
        const float4 v = *reinterpret_cast<const float4 *>(s4 + o), w = *reinterpret_cast<const float4 *>(o4 + o),
                     x = *reinterpret_cast<const float4 *>(h4 + o);
        u[2 * q] = cf(v.x, v.y);
        u[2 * q + 1] = cf(v.z, v.w);
        dy[2 * q] = cf(w.x, w.y);
        dy[2 * q + 1] = cf(w.z, w.w);
        h[2 * q] = cf(x.x, x.y);
        h[2 * q + 1] = cf(x.z, x.w);
      }
      const unsigned char *d4 = reinterpret_cast<const unsigned char *>(sd);
      const unsigned char *dA4 = reinterpret_cast<const unsigned char *>(sdA);
#pragma unroll
      for (int q = 0; q < BI / 4; ++q) {
        const int o = off_f(q);
        const float4 v = *reinterpret_cast<const float4 *>(d4 + o);
        dl[4 * q] = v.x; dl[4 * q + 1] = v.y; dl[4 * q + 2] = v.z; dl[4 * q + 3] = v.w;
        if (HAS_DA) {
          const float4 w = *reinterpret_cast<const float4 *>(dA4 + o);
          dAv[4 * q] = w.x; dAv[4 * q + 1] = w.y; dAv[4 * q + 2] = w.z; dAv[4 * q + 3] = w.w;
        }
      }
      if (!HAS_DA) {
#pragma unroll
        for (int i = 0; i < BI; ++i) dAv[i] = dl[i];
      }
    }
    if (!bc_one) {
#pragma unroll
      for (int i = 0; i < BI; ++i) h[i] = h[i] * inv_bc;
    }
    // the state before this lane's first step (only the bilinear gradient needs h_{t-1} itself)
    cf hprev0 = cf(0.f, 0.f);
    if constexpr (DM == B200_DISC_BILINEAR) {
      hprev0 = shfl_up(h[BI - 1], 1);
      if (lane == 0) {
        hprev0 = tw > 0 ? rp.h[tw - 1] : cf(0.f, 0.f);
        if (!bc_one) hprev0 = hprev0 * inv_bc;
      }
    }
    // the read-only slices sit in registers: refill them at once; the other overwritten buffer
    // first has to be read out by the stores of the previous item
    __syncwarp();
    if (lane == 0) {
      issue(1);
      if (stores_pending) bulk_wait_read<0>();
      issue(2);
    }
    advance();
    bool same_step = true;
#pragma unroll
    for (int i = 1; i < BI; ++i) same_step = same_step && dl[i] == dl[0] && dAv[i] == dAv[0];
    same_step = __all_sync(0xffffffffu, same_step);
    constexpr bool kUnitK = (DM == B200_DISC_DIRAC);
    cf a[BI], kk[kUnitK ? 1 : BI];
    if (same_step) {
      cf a0, k0;
      s5_coef<DM, !HAS_DA>(A0, invA0, dl[0], dAv[0], a0, k0);
#pragma unroll
      for (int i = 0; i < BI; ++i) {
        a[i] = a0;
        if constexpr (!kUnitK) kk[i] = k0;
      }
    } else {
#pragma unroll
      for (int i = 0; i < BI; ++i) {
        if constexpr (kUnitK) a[i] = cexp(A0 * dAv[i]);
        else s5_coef<DM, !HAS_DA>(A0, invA0, dl[i], dAv[i], a[i], kk[i]);
      }
    }
    auto beta = [&](int i) { return kUnitK ? u[i] : kk[kUnitK ? 0 : i] * u[i]; };
    auto seed = [&](int i) { return c_one ? dy[i] : dy[i] * Cc; };
    // reverse scan of g_t = seed_t + conj(a_{t+1}) g_{t+1}, carried across threads as q_t = conj(a_t) g_t
    cf gg = seed(BI - 1), Q = conj(a[BI - 1]);
#pragma unroll
    for (int i = BI - 2; i >= 0; --i) {
      gg = conj(a[i + 1]) * gg + seed(i);
      Q = Q * conj(a[i]);
    }
    gg = conj(a[0]) * gg;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const cf Qr = shfl_down(Q, off), gr = shfl_down(gg, off);
      if (lane + off < 32) { gg = gg + Q * gr; Q = Q * Qr; }
    }
    const int par = f & 1;
    if (lane == 0) { sh.rtot_q[par][warp] = Q; sh.rtot_g[par][warp] = gg; }
    __syncthreads();   // the only block barrier of the tile
    cf qpost = (j == 0) ? cf(0.f, 0.f) : sh.gcar[par];
    for (int w = HWARPS - 1; w > warp; --w) qpost = sh.rtot_g[par][w] + sh.rtot_q[par][w] * qpost;
    const cf g_right = shfl_down(gg, 1), Q_right = shfl_down(Q, 1);
    cf qin = g_right + Q_right * qpost;
    if (lane == 31) qin = qpost;
    if (tid == 0) sh.gcar[par ^ 1] = gg + Q * qpost;
    // adjoints and gradients
    cf dA_l = cf(0.f, 0.f), dB_l = cf(0.f, 0.f), dC_l = cf(0.f, 0.f);
    cf du[BI];
    float ddl[BI], ddA[BI];
    cf q = qin;
#pragma unroll
    for (int i = BI - 1; i >= 0; --i) {
      const cf G = (i == BI - 1) ? seed(i) + q : conj(a[i == BI - 1 ? i : i + 1]) * q + seed(i);   // g_t
      q = G;
      const cf t = G * conj(h[i] - beta(i));   // g_t conj(a_t h_{t-1})
      const float dv = dl[i], dav = dAv[i];
      if constexpr (kUnitK) {
        du[i] = G;
        if (NEED_BC) dB_l = dB_l + G * conj(u[i]);
      } else {
        du[i] = G * conj(kk[kUnitK ? 0 : i]);
        if (NEED_BC) dB_l = dB_l + G * conj(beta(i));
      }
      if (NEED_BC) dC_l = dC_l + dy[i] * conj(h[i]);
      float d_dl = 0.f, d_dA = 0.f;
      if constexpr (DM == B200_DISC_ZOH) {
        const cf E = HAS_DA ? kk[kUnitK ? 0 : i] * A0 + cf(1.f, 0.f) : a[i];   // exp(A dv) = 1 + k A
        d_dA = (t * conj(A0)).re;
        d_dl = (G * conj(E * u[i])).re;
        dA_l = dA_l + t * dav + G * conj(u[i] * ((E * dv - kk[kUnitK ? 0 : i]) * invA0));
      } else if constexpr (DM == B200_DISC_BILINEAR) {
        const cf hprev = (i == 0) ? hprev0 : h[i == 0 ? 0 : i - 1];
        const cf r = cf(1.f, 0.f) / (cf(1.f, 0.f) - A0 * (0.5f * dv));
        const cf rA = cf(1.f, 0.f) / (cf(1.f, 0.f) - A0 * (0.5f * dav));
        const cf r2 = r * r, rA2 = rA * rA;
        d_dA = (G * conj(hprev * A0 * rA2)).re;
        d_dl = (G * conj(r2 * u[i])).re;
        dA_l = dA_l + G * conj(hprev * rA2 * dav + r2 * u[i] * (0.5f * dv * dv));
      } else {
        d_dA = (t * conj(A0)).re;
        dA_l = dA_l + t * dav;
      }
      if (HAS_DA) { ddl[i] = d_dl; ddA[i] = d_dA; }
      else ddl[i] = d_dl + d_dA;
    }
    dA_acc = dA_acc + dA_l;
    dB_acc = dB_acc + dB_l;
    dC_acc = dC_acc + dC_l;
    // ---- du / ddelta (/ ddeltaA): over the u / delta (/ deltaA) slices, then bulk stores
    if (async_tile) {
      unsigned char *s4 = reinterpret_cast<unsigned char *>(su);
#pragma unroll
      for (int qq = 0; qq < BI / 2; ++qq)
        *reinterpret_cast<float4 *>(s4 + off_c(qq)) =
            make_float4(du[2 * qq].re, du[2 * qq].im, du[2 * qq + 1].re, du[2 * qq + 1].im);
      unsigned char *d4 = reinterpret_cast<unsigned char *>(sd);
#pragma unroll
      for (int qq = 0; qq < BI / 4; ++qq)
        *reinterpret_cast<float4 *>(d4 + off_f(qq)) = make_float4(ddl[4 * qq], ddl[4 * qq + 1], ddl[4 * qq + 2], ddl[4 * qq + 3]);
      if (HAS_DA) {
        unsigned char *dA4 = reinterpret_cast<unsigned char *>(sdA);
#pragma unroll
        for (int qq = 0; qq < BI / 4; ++qq)
          *reinterpret_cast<float4 *>(dA4 + off_f(qq)) = make_float4(ddA[4 * qq], ddA[4 * qq + 1], ddA[4 * qq + 2], ddA[4 * qq + 3]);
      }
      fence_proxy_async();
      __syncwarp();
      const bool warp_failed = __any_sync(0xffffffffu, failed);   // a warp that gave up on a wait stores nothing more
      if (lane == 0 && !warp_failed) {
        if (SWZ) {
          const int64_t e0 = row * L + tw;
          tensor_s2g(&maps.du, (int)(e0 >> 4), su);
          tensor_s2g(&maps.dd, (int)(e0 >> 5), sd);
          if (HAS_DA) tensor_s2g(&maps.ddA, (int)(e0 >> 5), sdA);
        } else {
          bulk_s2g(rp.du + tw, su, WU);
          bulk_s2g(rp.dd + tw, sd, WD);
          if (HAS_DA) bulk_s2g(rp.ddA + tw, sdA, WD);
        }
        bulk_commit();
      }
      stores_pending = true;
    } else {
#pragma unroll
      for (int i = 0; i < BI; ++i) {
        const int t = tw + lane * BI + i;
        if (t < L && !failed) {
          rp.du[t] = du[i];
          rp.dd[t] = ddl[i];
          if (HAS_DA) rp.ddA[t] = ddA[i];
        }
      }
      __syncwarp();   // the slice may be refilled by plain loads two items later
    }
    // ---- end of a row: fold the parameter gradients into dA / dB / dC
    if (c == 0) {
      const int d = (int)(row % p.dim);
      cf *dAp = reinterpret_cast<cf *>(p.dA) + (int64_t)d * p.A_ds;
      cf *dBp = NEED_BC ? reinterpret_cast<cf *>(p.dB) + (int64_t)d * p.B_ds : nullptr;
      cf *dCp = NEED_BC ? reinterpret_cast<cf *>(p.dC) + (int64_t)d * p.C_ds : nullptr;
      const cf ra = warp_sum(dA_acc);
      cf rb, rc;
      if (NEED_BC) { rb = warp_sum(dB_acc); rc = warp_sum(dC_acc); }
      __syncthreads();   // sh.red is free (its readers of the previous row are done)
      if (lane == 0) { sh.red[0][warp] = ra; sh.red[1][warp] = rb; sh.red[2][warp] = rc; }
      __syncthreads();
      if (tid < (NEED_BC ? 3 : 1)) {
        cf acc = cf(0.f, 0.f);
#pragma unroll
        for (int w = 0; w < HWARPS; ++w) acc = acc + sh.red[tid][w];
        cf *dst = tid == 0 ? dAp : (tid == 1 ? dBp : dCp);
        atomicAdd(&dst->re, acc.re);
        atomicAdd(&dst->im, acc.im);
      }
    }
  }
  if (lane == 0) bulk_wait<0>();
  __syncthreads();
  if (failed) atomicExch(&g_simpscan_status, 4);
}

int sm_count() { return sm_count_current(); }

template <typename K> int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return (int)e; }
  }
  return 0;
}

template <int DM, bool HAS_DA, bool S1> int launch_fwd_s(const b200_simpscan_args &a, cudaStream_t st) {
  constexpr int SLOT_BYTES = F_U_BYTES + F_D_BYTES * (HAS_DA ? 2 : 1);
  const int64_t rows = (int64_t)a.batch * a.dim;
  const size_t smem = (size_t)FWARPS * FNS * SLOT_BYTES + FWARPS * FNS * 8 + (size_t)FWARPS * 2 * a.dstate * sizeof(cf);
  auto k = simpscan_fwd_kernel<DM, HAS_DA, S1>;
  if (int e = set_smem(k, smem)) return e;
  int64_t grid = (rows + FWARPS - 1) / FWARPS;
  const int64_t resident = (int64_t)sm_count() * 7;   // CTAs that fit at once (7 per SM)
  if (grid > resident) grid = resident;
  k<<<(unsigned)grid, FWARPS * 32, smem, st>>>(a);
  return launch_status();
}
template <int DM, bool HAS_DA> int launch_fwd(const b200_simpscan_args &a, cudaStream_t st) {
  return a.dstate == 1 ? launch_fwd_s<DM, HAS_DA, true>(a, st) : launch_fwd_s<DM, HAS_DA, false>(a, st);
}
// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link libcuda
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    tried = true;
  }
  return fn;
}
// A contiguous tensor of `bytes` bytes as rows of 128 bytes (32 floats), boxes of `box_rows` rows, 128-byte swizzle.
bool make_row_map(CUtensorMap *m, const void *base, uint64_t bytes, uint32_t box_rows) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc || !base) return false;
  const cuuint64_t dims[2] = {32, bytes / 128};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {32, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor maps for the backward kernels: possible when every activation tensor is a contiguous
// (batch, dim, seqlen) array made of whole 128-byte rows.
bool build_bwd_maps(const b200_simpscan_args &a, bool has_dA, bool with_h, TmaMaps &maps) {
  memset(&maps, 0, sizeof(maps));
  const int64_t rows = (int64_t)a.batch * a.dim, L = a.seqlen, DL = (int64_t)a.dim * L;
  auto dense = [&](int64_t bs, int64_t ds) { return ds == L && bs == DL; };
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  bool ok = L % 32 == 0 && rows * L / 16 < (int64_t(1) << 31) && dense(a.u_bs, a.u_ds) && dense(a.dout_bs, a.dout_ds) &&
            dense(a.delta_bs, a.delta_ds) && dense(a.du_bs, a.du_ds) && dense(a.ddelta_bs, a.ddelta_ds) && al16(a.u) &&
            al16(a.dout) && al16(a.delta) && al16(a.du) && al16(a.ddelta);
  if (with_h) ok = ok && dense(a.out_bs, a.out_ds) && al16(a.out);
  if (has_dA) ok = ok && dense(a.deltaA_bs, a.deltaA_ds) && dense(a.ddeltaA_bs, a.ddeltaA_ds) && al16(a.deltaA) && al16(a.ddeltaA);
  if (!ok) return false;
  const uint64_t cb = (uint64_t)rows * L * 8, fb = (uint64_t)rows * L * 4;
  ok = make_row_map(&maps.u, a.u, cb, 16) && make_row_map(&maps.dout, a.dout, cb, 16) && make_row_map(&maps.d, a.delta, fb, 8) &&
       make_row_map(&maps.du, a.du, cb, 16) && make_row_map(&maps.dd, a.ddelta, fb, 8);
  if (with_h) ok = ok && make_row_map(&maps.h, a.out, cb, 16);
  if (has_dA) ok = ok && make_row_map(&maps.dA, a.deltaA, fb, 8) && make_row_map(&maps.ddA, a.ddeltaA, fb, 8);
  return ok;
}

template <int DM, bool HAS_DA, bool S1, bool NEED_BC> int launch_bwd_s(const b200_simpscan_args &a, cudaStream_t st) {
  constexpr int BUF_BYTES = 2 * B_U_BYTES + B_D_BYTES * (HAS_DA ? 2 : 1);
  constexpr int OUT_BYTES = B_U_BYTES + B_D_BYTES * (HAS_DA ? 2 : 1);
  const int64_t rows = (int64_t)a.batch * a.dim;
  const size_t smem = 2 * (size_t)BUF_BYTES + OUT_BYTES + sizeof(BwdShared) + (size_t)5 * a.dstate * sizeof(cf) + 1024;
  TmaMaps maps;
  const bool swz = build_bwd_maps(a, HAS_DA, false, maps);
  auto k = swz ? simpscan_bwd_kernel<DM, HAS_DA, S1, NEED_BC, true> : simpscan_bwd_kernel<DM, HAS_DA, S1, NEED_BC, false>;
  if (int e = set_smem(k, smem)) return e;
  int64_t grid = rows;
  const int64_t resident = (int64_t)sm_count() * (HAS_DA ? 1 : 2);   // CTAs that fit at once
  if (grid > resident) grid = resident;
  k<<<(unsigned)grid, BT, smem, st>>>(a, maps);
  return launch_status();
}

template <int DM, bool HAS_DA, bool NEED_BC, int HT> int launch_bwd_h_t(const b200_simpscan_args &a, cudaStream_t st) {
  constexpr int HWARPS = HT / 32;
  constexpr int ROB = 2 * HSL * 8, RWB = HSL * 8 + HSL * 4 * (HAS_DA ? 2 : 1);
  const int64_t rows = (int64_t)a.batch * a.dim;
  const size_t smem = (size_t)HWARPS * (ROB + 2 * RWB) + sizeof(BwdHShared<HWARPS>) + 1024;
  TmaMaps maps;
  const bool swz = build_bwd_maps(a, HAS_DA, true, maps);
  auto k = swz ? simpscan_bwd_h_kernel<DM, HAS_DA, NEED_BC, HT, true> : simpscan_bwd_h_kernel<DM, HAS_DA, NEED_BC, HT, false>;
  if (int e = set_smem(k, smem)) return e;
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  per_sm = per_sm > 512 / HT ? 512 / HT : (per_sm < 1 ? 1 : per_sm);
  int64_t grid = rows;
  const int64_t resident = (int64_t)sm_count() * per_sm;
  if (grid > resident) grid = resident;
  k<<<(unsigned)grid, HT, smem, st>>>(a, maps);
  return launch_status();
}
template <int DM, bool HAS_DA, bool NEED_BC> int launch_bwd_h(const b200_simpscan_args &a, cudaStream_t st) {
  return launch_bwd_h_t<DM, HAS_DA, NEED_BC, 128>(a, st);
}
template <int DM, bool HAS_DA> int launch_bwd(const b200_simpscan_args &a, cudaStream_t st) {
  if (a.dstate == 1 && a.out)   // the forward output is the state sequence: no recomputation
    return a.dB ? launch_bwd_h<DM, HAS_DA, true>(a, st) : launch_bwd_h<DM, HAS_DA, false>(a, st);
  if (a.dstate != 1) return launch_bwd_s<DM, HAS_DA, false, true>(a, st);
  return a.dB ? launch_bwd_s<DM, HAS_DA, true, true>(a, st) : launch_bwd_s<DM, HAS_DA, true, false>(a, st);
}

int check(const b200_simpscan_args &a, bool bwd) {
  B200_REQUIRE(a.u && a.delta && a.A && a.B && a.C, B200_ERR_NULL, "simpscan: u, delta, A, B, C must be non-null");
  B200_REQUIRE(a.batch > 0 && a.dim > 0 && a.seqlen > 0 && a.dstate > 0, B200_ERR_SHAPE,
               "simpscan: batch, dim, seqlen, dstate must be positive");
  B200_REQUIRE(a.dstate <= kMaxDState, B200_ERR_SHAPE, "simplified_scan only supports state dimension <= 256");
  B200_REQUIRE(a.method == B200_DISC_ZOH || a.method == B200_DISC_BILINEAR || a.method == B200_DISC_DIRAC,
               B200_ERR_DTYPE, "simplified_scan supports the zoh, bilinear and dirac discretizations");
  if (!bwd) {
    B200_REQUIRE(a.out && a.x, B200_ERR_NULL, "simpscan_fwd: out and x must be non-null");
  } else {
    B200_REQUIRE(a.dout && a.du && a.ddelta && a.dA, B200_ERR_NULL,
                 "simpscan_bwd: dout, du, ddelta, dA must be non-null");
    B200_REQUIRE((a.dB != nullptr) == (a.dC != nullptr), B200_ERR_NULL,
                 "simpscan_bwd: dB and dC must be both given or both null");
    B200_REQUIRE((a.dB && a.dC) || a.dstate == 1, B200_ERR_NULL,
                 "simpscan_bwd: dB and dC may be null only when dstate == 1");
    B200_REQUIRE(a.x || a.seqlen <= kChunk, B200_ERR_NULL, "simpscan_bwd: x is required when seqlen > 2048");
    B200_REQUIRE(!a.deltaA || a.ddeltaA, B200_ERR_NULL, "simpscan_bwd: ddeltaA is required when deltaA is given");
  }
  return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_simpscan_fwd(const b200_simpscan_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "simpscan_fwd: null argument block");
  if (int e = check(*args, false)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool dA = args->deltaA != nullptr;
  switch (args->method) {
    case B200_DISC_ZOH: return dA ? launch_fwd<B200_DISC_ZOH, true>(*args, st) : launch_fwd<B200_DISC_ZOH, false>(*args, st);
    case B200_DISC_BILINEAR: return dA ? launch_fwd<B200_DISC_BILINEAR, true>(*args, st) : launch_fwd<B200_DISC_BILINEAR, false>(*args, st);
    default: return dA ? launch_fwd<B200_DISC_DIRAC, true>(*args, st) : launch_fwd<B200_DISC_DIRAC, false>(*args, st);
  }
}

int b200_simpscan_bwd(const b200_simpscan_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "simpscan_bwd: null argument block");
  if (int e = check(*args, true)) return e;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool dA = args->deltaA != nullptr;
  switch (args->method) {
    case B200_DISC_ZOH: return dA ? launch_bwd<B200_DISC_ZOH, true>(*args, st) : launch_bwd<B200_DISC_ZOH, false>(*args, st);
    case B200_DISC_BILINEAR: return dA ? launch_bwd<B200_DISC_BILINEAR, true>(*args, st) : launch_bwd<B200_DISC_BILINEAR, false>(*args, st);
    default: return dA ? launch_bwd<B200_DISC_DIRAC, true>(*args, st) : launch_bwd<B200_DISC_DIRAC, false>(*args, st);
  }
}

// Non-zero after a kernel gave up on a bounded barrier wait (diagnostic; synchronises the device).
int b200_device_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_simpscan_status, sizeof(int)) != cudaSuccess) return -1;
  const int w = ssu_status_read();
  if (w < 0) return -1;
  const int g = cgemm_status_read();
  if (g < 0) return -1;
  return v ? v : (w ? w : g);
}

}  // extern "C"
