// Linear layer for a handful of tokens (one decoding step): out (M x N) = x (M x K) W^T with
// W (N x K) row-major 16-bit (an nn.Linear weight), M <= 64, float32 accumulation.
//
// The four projections of a Mamba block's step() (lrnnx/models/ltv/mamba.py:355-487: in_proj,
// x_proj, dt_proj, out_proj) and the LM head move each weight once per generated token and do
// almost no arithmetic on it: the kernel is a weight stream, HBM-bound, and is organised for
// bytes in flight, not for tensor throughput.
//   * A CTA owns BN output features and all M tokens, and a slice of K.  The K slices of a feature
//     tile belong to the CTAs of one thread-block cluster (1, 2, 4 or 8), picked so that the grid
//     has one to two CTAs per SM whatever N is.
//   * Weight and activation tiles (BN x 64 and 64 x 64 elements) arrive by 16-byte cp.async into a
//     4-stage ring of 128-byte-row, XOR-swizzled shared-memory tiles; eight warps (16 tokens x half
//     of the features each) consume them with ldmatrix + mma.sync.m16n8k16.  Measured at 64 tokens:
//     faster than the library GEMM for narrow outputs (160 features over K = 4096: 4.7 against 7.0 us),
//     slower for wide ones (8192 features: 13 to 17 against 8.2 us; a tcgen05 variant with the weight as
//     the 128-row operand, TMA tiles and a TMEM accumulator was correct but no faster, 12.3 us: at one
//     CTA per SM both are held near 45 GB/s per SM by the activation tile every CTA re-reads from
//     L2 next to its weight stream); the Python wrapper uses the kernel for narrow outputs only.
//   * The partial sums of the cluster's CTAs meet in distributed shared memory: CTA r owns token rows
//     [r 64/S, (r+1) 64/S); every CTA posts its partial values for those rows into r's receive buffer
//     (plain remote stores), and after one cluster barrier r adds up the S contributions in rank
//     order.  No atomics: the result does not depend on arrival order, so decoding is reproducible.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int SK_M = 64;          // token rows of a tile (M is padded up to it)
constexpr int SK_BK = 64;         // K elements per pipeline stage (one 128-byte row)
constexpr int SK_STAGES = 4;
constexpr int SK_THREADS = 256;    // 8 warps: 4 token groups of 16 x 2 halves of the feature tile

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool pred) {
  const int sz = pred ? 16 : 0;     // size 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T> struct MmaOp;
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct MmaOp<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
__device__ __forceinline__ __nv_bfloat16 cvt16(float v, __nv_bfloat16) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ __half cvt16(float v, __half) { return __float2half_rn(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

// byte offset of the 16-byte chunk `chunk` (0..7) of row `row` in a tile of 128-byte rows
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <int BN> struct SkSmem {
  static constexpr int W_BYTES = BN * 128;
  static constexpr int X_BYTES = SK_M * 128;
  static constexpr int STAGE = W_BYTES + X_BYTES;
  static constexpr int PIPE = SK_STAGES * STAGE;
  static constexpr int PROW = BN + 8;                        // floats per row of the partial tile (8 rows of a
                                                             // fragment store land in distinct 32-byte segments)
  static constexpr int PART = SK_M * PROW * 4;               // receive buffer: S slots of 64 / S token rows, float32
  static constexpr int TOTAL = PIPE + PART;
};

template <typename T, int BN>
__global__ void __launch_bounds__(SK_THREADS) skinny_linear_kernel(const b200_skinny_linear_args p) {
  using SM = SkSmem<BN>;
  extern __shared__ __align__(128) unsigned char smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();           // K slices (cluster spans blockIdx.x)
  const int ks = (int)cluster.block_rank();
  const int tile = blockIdx.x / S;
  const int n0 = tile * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k_per = p.K / S;                          // multiple of SK_BK (checked by the host)
  const int k_begin = ks * k_per;
  const int n_chunks = k_per / SK_BK;
  const T *W = reinterpret_cast<const T *>(p.weight);
  const T *X = reinterpret_cast<const T *>(p.x);
  const uint32_t sbase = smem_u32(smem);

  auto load_stage = [&](int stage, int chunk) {
    const int k0 = k_begin + chunk * SK_BK;
    const uint32_t ws = sbase + stage * SM::STAGE, xs = ws + SM::W_BYTES;
    // weight tile: BN rows x 8 chunks of 16 bytes
#pragma unroll
    for (int i = tid; i < BN * 8; i += SK_THREADS) {
      const int r = i >> 3, c = i & 7;
      const bool ok = n0 + r < p.N;
      cp_async16(ws + swz(r, c), W + (int64_t)(ok ? n0 + r : 0) * p.w_rs + k0 + c * 8, ok);
    }
#pragma unroll
    for (int i = tid; i < SK_M * 8; i += SK_THREADS) {
      const int r = i >> 3, c = i & 7;
      const bool ok = r < p.M;
      cp_async16(xs + swz(r, c), X + (int64_t)(ok ? r : 0) * p.x_rs + k0 + c * 8, ok);
    }
  };

  constexpr int HN = BN / 2;                          // features per warp
  const int wm = warp & 3, wn = warp >> 2;
  float acc[HN / 8][4];
#pragma unroll
  for (int j = 0; j < HN / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;

#pragma unroll
  for (int s = 0; s < SK_STAGES - 1; ++s) {
    if (s < n_chunks) load_stage(s, s);
    cp_async_commit();
  }
  for (int c = 0; c < n_chunks; ++c) {
    cp_async_wait<SK_STAGES - 2>();
    __syncthreads();                                  // stage c landed for every thread; stage c-1 is free again
    {
      const int nxt = c + SK_STAGES - 1;
      if (nxt < n_chunks) load_stage(nxt % SK_STAGES, nxt);
      cp_async_commit();
    }
    const uint32_t ws = sbase + (c % SK_STAGES) * SM::STAGE, xs = ws + SM::W_BYTES;
#pragma unroll
    for (int kk = 0; kk < SK_BK / 16; ++kk) {
      uint32_t a[4];
      ldsm4(xs + swz(wm * 16 + (lane & 15), kk * 2 + (lane >> 4)), a);
#pragma unroll
      for (int j = 0; j < HN / 16; ++j) {
        uint32_t b[4];     // {n-tile 2j: k 0-7, k 8-15; n-tile 2j+1: k 0-7, k 8-15}
        ldsm4(ws + swz(wn * HN + j * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)), b);
        MmaOp<T>::run(acc[2 * j], a, b[0], b[1]);
        MmaOp<T>::run(acc[2 * j + 1], a, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  // Token rows are dealt out to the cluster's CTAs: rank r owns rows [r 64 / S, (r + 1) 64 / S).  Every
  // warp posts its fragment values straight into the owner's receive buffer, slot [sender rank][row],
  // with plain stores into distributed shared memory (nothing waits on a remote round trip); after one
  // cluster barrier every CTA adds up its S slots from its own shared memory, in rank order.
  float *recv = reinterpret_cast<float *>(smem + SM::PIPE);
  const int log2s = 31 - __clz(S);
  const int rows_per = SK_M >> log2s;
  {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = wm * 16 + g + half * 8;
      const int owner = row >> (6 - log2s);
      float *dst = (S > 1 ? cluster.map_shared_rank(recv, owner) : recv) + (ks * rows_per + (row & (rows_per - 1))) * SM::PROW;
#pragma unroll
      for (int j = 0; j < HN / 8; ++j) {
        const int col = wn * HN + j * 8 + t4 * 2;
        *reinterpret_cast<float2 *>(dst + col) = make_float2(acc[j][2 * half], acc[j][2 * half + 1]);
      }
    }
  }
  if (S > 1) cluster.sync();
  else __syncthreads();

  T *out = reinterpret_cast<T *>(p.out);
  const T *bias = reinterpret_cast<const T *>(p.bias);
  for (int i = tid; i < rows_per * (BN / 4); i += SK_THREADS) {
    const int rl = i / (BN / 4), c4 = (i % (BN / 4)) * 4;
    const int r = ks * rows_per + rl;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < S; ++q) {
      const float4 v = *reinterpret_cast<const float4 *>(recv + (q * rows_per + rl) * SM::PROW + c4);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    if (r < p.M) {
      const float vals[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = n0 + c4 + e;
        if (n < p.N) {
          float v = vals[e];
          if (bias) v += to_float(bias[n]);
          out[(int64_t)r * p.out_rs + n] = cvt16(v, T());
        }
      }
    }
  }
}

template <typename T, int BN>
int launch_skinny(const b200_skinny_linear_args &a, int S, cudaStream_t st) {
  using SM = SkSmem<BN>;
  auto kernel = skinny_linear_kernel<T, BN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) != cudaSuccess)
      return launch_status();
    attr_set[dev] = true;
  }
  const int tiles = (a.N + BN - 1) / BN;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * S));
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = SM::TOTAL;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, a) != cudaSuccess) return launch_status();
  return launch_status();
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_skinny_linear(const b200_skinny_linear_args *args, void *stream) {
  B200_REQUIRE(args, B200_ERR_NULL, "skinny_linear: null argument block");
  const b200_skinny_linear_args &a = *args;
  B200_REQUIRE(a.x && a.weight && a.out, B200_ERR_NULL, "skinny_linear: x, weight, out must be non-null");
  B200_REQUIRE(a.dtype == B200_BF16 || a.dtype == B200_F16, B200_ERR_DTYPE, "skinny_linear: bfloat16 or float16 only");
  B200_REQUIRE(a.M >= 1 && a.M <= SK_M && a.N >= 1 && a.K >= SK_BK && a.K % SK_BK == 0, B200_ERR_SHAPE,
               "skinny_linear: 1 <= M <= 64, N >= 1, K a positive multiple of 64 (got M=%d N=%d K=%d)", a.M, a.N, a.K);
  B200_REQUIRE(a.x_rs % 8 == 0 && a.w_rs % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(a.weight) & 15) == 0,
               B200_ERR_ALIGN, "skinny_linear: rows of x and weight must start on 16-byte boundaries");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // K slices per feature tile: at most 8 (the portable cluster size), each at least two pipeline stages long;
  // feature tile: the widest of 128 / 64 / 32 that still gives every SM a CTA
  const int sms = sm_count_current();
  int s_max = 1;
  while (s_max < 8 && a.K % (SK_BK * s_max * 2) == 0 && a.K / (s_max * 2) >= 2 * SK_BK) s_max *= 2;
  int BN = 128;
  if ((a.N + 127) / 128 * s_max < sms) BN = 64;
  if (BN == 64 && (a.N + 63) / 64 * s_max < sms) BN = 32;
  const int tiles = (a.N + BN - 1) / BN;
  int S = 1;
  while (S < s_max && tiles * S * 2 <= 2 * sms) S *= 2;
#define SK_LAUNCH(T_)                                                     \
  (BN == 128 ? launch_skinny<T_, 128>(a, S, st) : BN == 64 ? launch_skinny<T_, 64>(a, S, st) : launch_skinny<T_, 32>(a, S, st))
  return a.dtype == B200_BF16 ? SK_LAUNCH(__nv_bfloat16) : SK_LAUNCH(__half);
#undef SK_LAUNCH
}
