// Linear layer of a decoding step for wide outputs, on the 5th-generation tensor cores:
//     out (M x N) = x (M x K) W^T,   W (N x K) row-major 16-bit,  M <= 64 tokens.
// The weight is the MMA's 128-row operand and the tokens are its N dimension (D = W_tile x^T, one
// 128-feature x 64-token float32 accumulator in 64 TMEM columns), so the tensor core works on
// full-height tiles although only 64 tokens exist, and a CTA is nothing but a weight stream:
//   warp 0      TMA producer: per 64-element K step a (128 x 64) weight tile and the (64 x 64)
//               activation tile, 128-byte swizzled, into a 6-stage ring on mbarriers (144 KB in
//               flight per SM);
//   warp 1      allocates TMEM and issues four tcgen05.mma.kind::f16 (K = 16) per stage, both
//               operands K-major, committing every stage back to the producer;
//   warps 2-5   epilogue: tcgen05.ld of the accumulator, partial tile parked in shared memory.
// K is cut over the CTAs of a thread-block cluster (1, 2, 4 or 8 slices of a feature tile) so that
// about one CTA runs per SM whatever N is; the slices' partial tiles are added up through
// distributed shared memory in rank order (no atomics: the result is reproducible) and stored as
// 16-bit rows of out.  Every mbarrier wait is bounded; an expired wait sets a status word, the
// stores are skipped, the cluster barriers are still reached and the TMEM is freed.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"
#include "dispatch.h"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

using namespace tc;

__device__ int g_linear_status = 0;

constexpr int LM_F = 128;                 // features (weight rows) per tile
constexpr int LM_T = 64;                  // tokens per tile
constexpr int LM_K = 64;                  // K elements per stage: one 128-byte swizzle row
constexpr int LM_STAGES = 6;
constexpr int LM_WTILE = LM_F * 128;      // 16 KB
constexpr int LM_XTILE = LM_T * 128;      // 8 KB
constexpr int LM_STAGE = LM_WTILE + LM_XTILE;
constexpr int LM_PROW = LM_F + 4;         // floats per token row of the partial tile
constexpr int LM_PART = LM_T * LM_PROW * 4;
constexpr int LM_SMEM = LM_STAGES * LM_STAGE + 1024;     // + room to align the ring to 1024 bytes
constexpr int LM_THREADS = 192;
constexpr int LM_TMEM_COLS = 64;
constexpr uint32_t LM_WAIT = 1u << 24;
static_assert(LM_PART <= LM_STAGES * LM_STAGE, "the partial tile reuses the ring");

struct LinearMaps {
  CUtensorMap w;      // (K, N) 16-bit, box (64, 128)
  CUtensorMap x;      // (K, M) 16-bit, box (64, 64)
};

// K-major tile of 128-byte rows, 8-row groups 1024 bytes apart, 128-byte swizzle
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t addr) { return smem_desc(addr, 16, 1024, 2); }

// instruction descriptor: D f32; A, B bf16 (1) or f16 (0), both K-major; M = 128, N = 64
__host__ __device__ constexpr uint32_t linear_idesc(bool bf16) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((uint32_t)(LM_T >> 3) << 17) |
         ((uint32_t)(LM_F >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <typename T> __device__ __forceinline__ float as_f32(T v);
template <> __device__ __forceinline__ float as_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float as_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__global__ void __launch_bounds__(LM_THREADS, 1)
linear_tc_kernel(const __grid_constant__ LinearMaps maps, const b200_skinny_linear_args p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full[LM_STAGES], empty[LM_STAGES], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();
  const int ks_rank = (int)cluster.block_rank();
  const int tile = blockIdx.x / S;
  const int n0 = tile * LM_F;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k_per = p.K / S;
  const int k_begin = ks_rank * k_per;
  const int nk = k_per / LM_K;
  constexpr uint32_t idesc = linear_idesc(std::is_same<T, __nv_bfloat16>::value);

  if (tid == 0) {
    for (int s = 0; s < LM_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_done, 1);
    fail_s = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(LM_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {
      for (int ks = 0; ks < nk; ++ks) {
        const int s = ks % LM_STAGES;
        if (ks >= LM_STAGES && !mbar_wait(&empty[s], ((ks / LM_STAGES) - 1) & 1, LM_WAIT)) { atomicExch(&fail_s, 1); break; }
        unsigned char *st = smem + (size_t)s * LM_STAGE;
        mbar_expect_tx(&full[s], LM_STAGE);
        const int k0 = k_begin + ks * LM_K;
        tma_2d(st, &maps.w, k0, n0, &full[s]);
        tma_2d(st + LM_WTILE, &maps.x, k0, 0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int ks = 0; ks < nk && ok; ++ks) {
        const int s = ks % LM_STAGES;
        if (!mbar_wait(&full[s], (ks / LM_STAGES) & 1, LM_WAIT)) { ok = false; break; }
        tc_fence_after();
        const uint32_t st = smem_u32(smem + (size_t)s * LM_STAGE);
#pragma unroll
        for (int kk = 0; kk < LM_K / 16; ++kk)
          mma_f16(tmem_base, kmajor_desc(st + kk * 32), kmajor_desc(st + LM_WTILE + kk * 32), (ks > 0 || kk > 0) ? 1u : 0u, idesc);
        mma_commit(&empty[s]);
      }
      if (!ok) atomicExch(&fail_s, 1);
      mma_commit(&acc_done);
    }
  }
  // every thread meets here; the epilogue warps then wait for the accumulator
  float *part = reinterpret_cast<float *>(smem);
  if (warp >= 2) {
    const bool ok = mbar_wait(&acc_done, 0, LM_WAIT);
    if (!ok) atomicExch(&fail_s, 1);
    tc_fence_after();
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int f = q * 32 + lane;                 // feature row inside the tile
#pragma unroll
    for (int c = 0; c < LM_T / 32; ++c) {
      float v[32];
      tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c * 32, v);
      // the ring is free once acc_done has fired (every MMA that read it has completed)
#pragma unroll
      for (int j = 0; j < 32; ++j) part[(c * 32 + j) * LM_PROW + f] = v[j];
    }
  }
  tc_fence_before();
  if (S > 1) cluster.sync();
  else __syncthreads();
  const bool good = (fail_s == 0);

  // rank r adds up token rows [r 64 / S, (r + 1) 64 / S) over the cluster's partial tiles, in rank order
  const int rows_per = LM_T / S;
  const int r_begin = ks_rank * rows_per;
  T *out = reinterpret_cast<T *>(p.out);
  const T *bias = reinterpret_cast<const T *>(p.bias);
  if (good) {
    for (int i = tid; i < rows_per * (LM_F / 4); i += LM_THREADS) {
      const int r = r_begin + i / (LM_F / 4), c4 = (i % (LM_F / 4)) * 4;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int qk = 0; qk < S; ++qk) {
        const float *src = S > 1 ? cluster.map_shared_rank(part, qk) : part;
        const float4 v = *reinterpret_cast<const float4 *>(src + r * LM_PROW + c4);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      if (r < p.M) {
        const float vals[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = n0 + c4 + e;
          if (n < p.N) {
            float v = vals[e];
            if (bias) v += as_f32<T>(bias[n]);
            out[(int64_t)r * p.out_rs + n] = from_f32<T>(v);
          }
        }
      }
    }
  }
  if (S > 1) cluster.sync();                      // nobody leaves while its partial tile is still being read
  else __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(LM_TMEM_COLS) : "memory");
  }
  if (tid == 0 && !good) atomicExch(&g_linear_status, 7);
}

bool make_map16(CUtensorMap *m, const void *base, bool bf16, uint64_t inner, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {inner, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)LM_K, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims,
             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T> int launch_linear_tc(const b200_skinny_linear_args &a, const LinearMaps &maps, int S, cudaStream_t st) {
  auto kernel = linear_tc_kernel<T>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LM_SMEM) != cudaSuccess) return launch_status();
    attr_set[dev] = true;
  }
  const int tiles = (a.N + LM_F - 1) / LM_F;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * S));
  cfg.blockDim = dim3(LM_THREADS);
  cfg.dynamicSmemBytes = LM_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, maps, a) != cudaSuccess) return launch_status();
  return launch_status();
}

}  // namespace

int linear_status_read() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_linear_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// wide outputs with 16-byte aligned, 16-byte-stride rows: at least one 128-feature tile per eight SMs
bool linear_tc_supported(const b200_skinny_linear_args &a) {
  if (a.N < 1024 || a.K < 512 || a.K % LM_K != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.x) & 15) || (reinterpret_cast<uintptr_t>(a.weight) & 15)) return false;
  if (a.x_rs % 8 || a.w_rs % 8) return false;
  return encoder() != nullptr;
}

int linear_tc(const b200_skinny_linear_args &a, cudaStream_t st) {
  const bool bf16 = a.dtype == B200_BF16;
  LinearMaps maps;
  B200_REQUIRE(make_map16(&maps.w, a.weight, bf16, (uint64_t)a.K, (uint64_t)a.N, (uint64_t)a.w_rs * 2, LM_F) &&
                   make_map16(&maps.x, a.x, bf16, (uint64_t)a.K, (uint64_t)a.M, (uint64_t)a.x_rs * 2, LM_T),
               B200_ERR_UNSUPPORTED, "skinny_linear: the tensor maps of weight / x could not be encoded");
  const int sms = sm_count_current();
  const int tiles = (a.N + LM_F - 1) / LM_F;
  int S = 1;      // K slices: as many as keep the grid within one CTA per SM, each at least four stages long
  while (S < 8 && tiles * S * 2 <= sms && a.K % (LM_K * S * 2) == 0 && a.K / (S * 2) >= 4 * LM_K) S *= 2;
  return bf16 ? launch_linear_tc<__nv_bfloat16>(a, maps, S, st) : launch_linear_tc<__half>(a, maps, S, st);
}

}  // namespace b200
