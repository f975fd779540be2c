// C = A @ B on the 5th-generation tensor cores (K3 / K4): fp16 / bf16 inputs, and fp32 inputs
// as tf32 (what `nl.dot` does for fp32 blocks, newt/compiler/codegen.py:2195-2197).
//
// This is what `nl.dot` inside a K loop lowers to.  The reference stages
// operands with cp.async into an XOR-swizzled ring and multiplies with
// ldmatrix + mma.sync (newt/compiler/codegen.py:2296-2369, 2498-2558); here:
//
//   * operands arrive by TMA (cp.async.bulk.tensor.2d) into a ring of STAGES
//     shared-memory slots with the hardware 128-byte swizzle; out-of-range
//     rows/columns are zero-filled by the tensor map, which is exactly the
//     `mask=..., other=0.0` of the kernel source;
//   * one thread issues tcgen05.mma (M = 128, N = BLOCK_N, K = 16 per
//     instruction) reading both operands through shared-memory descriptors;
//     A is [M,K] row-major  -> K-major operand,
//     B is [K,N] row-major  -> MN-major operand (no transpose pass needed), or is handed
//     over transposed, [N,K] -> K-major operand.  An fp32 (tf32) B as [K,N] is MN-major too,
//     under the 32-byte-atom form of the swizzle; one whose base or pitch bulk copies cannot
//     fetch goes through a transposing pass into a caller-provided workspace first
//     (nb200_gemm_tf32);
//   * the fp32 accumulator lives in tensor memory, double-buffered, so the
//     epilogue of tile i (tcgen05.ld -> round -> store) overlaps the MMAs of
//     tile i+1;
//   * mbarriers carry every hand-off: TMA -> MMA (full), MMA -> TMA (empty, via
//     tcgen05.commit), MMA -> epilogue (acc_full), epilogue -> MMA (acc_empty).
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM
// owner, warps 2..5 epilogue (each owns the 32 TMEM lanes its warp id maps to).
// The grid is persistent: one CTA per SM walks output tiles in an order that
// keeps a band of GROUP_M row-blocks hot in L2.
//
// Tensor-bound: 2*M*N*K flop per launch.

#include <string.h>

#include <mutex>

#include "gemm_device.cuh"

namespace nb200 {
namespace {

using namespace sm100;

// ---- the kernels built ahead of time: the plain product, every tile and ring depth ------

using gemm::GemmParams;
using gemm::kBlockM;
using gemm::kThreads;

template <int BN, int STAGES, int KSUB, int DT, int CT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ GemmParams p) {
  gemm::gemm_body<BN, STAGES, KSUB, DT, CT, gemm::NoEpilogue>(tmap_a, tmap_b, p,
                                                              gemm::NoEpilogueArgs{0});
}

template <int STAGES, int KSUB, int DT, int CT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ GemmParams p) {
  gemm::gemm_pair_body<STAGES, KSUB, DT, CT, gemm::NoEpilogue>(tmap_a, tmap_b, p,
                                                               gemm::NoEpilogueArgs{0});
}

template <int STAGES, int KSUB, int DT, int CT>
__global__ void __launch_bounds__(gemm::kThreads, 1)
    gemm_pair_wide_kernel(const __grid_constant__ CUtensorMap tmap_a,
                          const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ GemmParams p) {
  gemm::gemm_pair_body<STAGES, KSUB, DT, CT, gemm::NoEpilogue, 2>(tmap_a, tmap_b, p,
                                                                  gemm::NoEpilogueArgs{0});
}

// ---- host ----------------------------------------------------------------------

struct Resolved {
  int block_n;
  int block_k;
  int stages;
  bool pair;
};

// a ring slot holds `ksub` slabs of K: 128 bytes for every row of A and column of B each
int smem_bytes_for(int block_n, int stages, int ksub) {
  return stages * ksub * (kBlockM * 128 + 128 * block_n) + 1024 + (int)gemm::kEpilogueStageBytes;
}

// `row_k`: K elements per 128-byte row (64 for 16-bit operands, 32 for tf32); block_k is
// resolved in elements of the operand type.
int resolve_config(const nb200_gemm_config* cfg, int64_t m, int64_t n, int row_k, Resolved* out) {
  const int kBlockK = row_k;
  int bm = cfg ? cfg->block_m : 0, bn = cfg ? cfg->block_n : 0, bk = cfg ? cfg->block_k : 0;
  int stages = cfg ? cfg->stages : 0;
  bool pair = cfg && (cfg->cta_pair || bm == 2 * kBlockM);
  if (!cfg || (bm == 0 && bn == 0 && bk == 0 && !cfg->cta_pair)) {
    // library default: CTA pairs once they fill the machine (74 pairs), else single CTAs
    pair = cdiv64(m, 2 * kBlockM) * cdiv64(n, 256) >= device_info().sm_count / 2;
    // ... 256 x 512 tiles (a third less traffic from L2 per flop: 4.5 % faster per flop at
    // 8192^3) when the rounds they need over the resident pairs cost less than the rounds of
    // 256 x 256 tiles do -- a last round that is mostly empty weighs more than the tile shape
    if (pair) {
      const int64_t pairs = device_info().sm_count / 2;
      const int64_t rounds256 = cdiv64(cdiv64(m, 2 * kBlockM) * cdiv64(n, 256), pairs);
      const int64_t rounds512 = cdiv64(cdiv64(m, 2 * kBlockM) * cdiv64(n, 512), pairs);
      if (rounds512 * 2 * 100 < rounds256 * 104) bn = 512;
    }
  }
  out->pair = pair;
  if (pair) {
    if (bm != 0 && bm != 2 * kBlockM)
      return fail(NB200_E_INVALID, "block_m=%d: a CTA pair computes 256-row tiles", bm);
    if (bn != 0 && bn != 256 && bn != 512)
      return fail(NB200_E_INVALID, "block_n=%d: CTA-pair tiles are 256 or 512 columns wide", bn);
    if (bn == 512) {
      // two 256-column MMAs per K step on one accumulator of all 512 tensor-memory columns: a
      // third less traffic from L2 per flop, no second accumulator for the epilogue to hide behind
      if (bk != 0 && bk != kBlockK && bk != 2 * kBlockK)
        return fail(NB200_E_INVALID, "block_k=%d: a 512-column ring slot holds %d or %d elements of K",
                    bk, kBlockK, 2 * kBlockK);
      out->block_n = 512;
      out->block_k = bk == 2 * kBlockK ? bk : kBlockK;
      out->stages = bk == 2 * kBlockK ? 2 : 4;
      return 0;
    }
    if (bk != 0 && bk != kBlockK && bk != 2 * kBlockK && bk != 3 * kBlockK)
      return fail(NB200_E_INVALID,
                  "block_k=%d: a CTA-pair ring slot holds %d, %d or %d elements of K", bk, kBlockK,
                  2 * kBlockK, 3 * kBlockK);
    out->block_k = bk == 0 ? 2 * kBlockK : bk;
    if (stages != 0 && (stages < 1 || stages > 8))
      return fail(NB200_E_INVALID, "stages=%d: supported 1..8", stages);
    out->block_n = 256;
    // ring depth: 3 slots of 128 K-elements, 2 of 192, 4..6 of 64 (the epilogue's 32 KB of
    // staging leaves no room for a seventh)
    out->stages = out->block_k == 2 * kBlockK ? 3 : (out->block_k == 3 * kBlockK ? 2 :
                  (stages == 0 ? 6 : (stages >= 6 ? 6 : (stages >= 5 ? 5 : 4))));
    return 0;
  }
  if (bm != 0 && bm != kBlockM)
    return fail(NB200_E_INVALID, "block_m=%d: MMA tiles are 128 rows (256 for a CTA pair)", bm);
  if (bn == 0) bn = n <= 64 ? 64 : (n <= 128 ? 128 : 256);
  if (bn != 64 && bn != 128 && bn != 256)
    return fail(NB200_E_INVALID, "block_n=%d: supported 64, 128, 256", bn);
  if (bk == 2 * kBlockK && bn != 256) {   // two K slabs per ring slot: half as many copies to issue
    out->block_n = bn;
    out->block_k = bk;
    out->stages = bn == 64 ? 4 : 3;
    return 0;
  }
  if (bk != 0 && bk != kBlockK)
    return fail(NB200_E_INVALID,
                "block_k=%d: a ring slot holds %d elements of K (%d too for 64 and 128 columns)", bk,
                kBlockK, 2 * kBlockK);
  // ring depths with a compiled instance, deepest first (bounded by 227 KB of shared memory)
  static const int depth256[] = {4, 3, 2, 0}, depth128[] = {6, 4, 3, 2, 0}, depth64[] = {8, 6, 4, 2, 0};
  const int* depths = bn == 256 ? depth256 : (bn == 128 ? depth128 : depth64);
  if (stages == 0) stages = depths[0];
  if (stages < 1 || stages > 8) return fail(NB200_E_INVALID, "stages=%d: supported 1..8", stages);
  int pick = 2;  // a ring needs two slots; num_stages=1 of the operator API maps here
  for (const int* d = depths; *d; ++d)
    if (*d <= stages) {
      pick = *d;
      break;
    }
  stages = pick;
  out->block_n = bn;
  out->block_k = kBlockK;
  out->stages = stages;
  return 0;
}

int check_problem(const void* a, const void* b, const void* c, int64_t m, int64_t n, int64_t k,
                  int64_t lda, int64_t ldb, int64_t ldc, int dtype, bool b_kmajor) {
  if (dtype != NB200_F16 && dtype != NB200_BF16 && dtype != NB200_F32)
    return fail(NB200_E_UNSUPPORTED, "gemm: dtype code %d (fp16, bf16, and fp32 as tf32)", dtype);
  const int eb = dtype == NB200_F32 ? 4 : 2;
  if (m < 0 || n < 0 || k < 0) return fail(NB200_E_INVALID, "gemm: negative extent");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return fail(NB200_E_INVALID, "gemm: extent beyond int32");
  if (m == 0 || n == 0) return 0;
  if (!c || (k > 0 && (!a || !b))) return fail(NB200_E_INVALID, "gemm: null tensor pointer");
  if (k == 0) return 0;  // C is cleared; A and B are never read
  if (lda < k || ldb < (b_kmajor ? k : n) || ldc < n)
    return fail(NB200_E_INVALID, "gemm: row stride smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                (long long)lda, (long long)ldb, (long long)ldc);
  // TMA: 16-byte aligned base and row pitch
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
    return fail(NB200_E_UNSUPPORTED, "gemm: A and B must be 16-byte aligned for TMA");
  if ((lda * eb) % 16 || (ldb * eb) % 16)
    return fail(NB200_E_UNSUPPORTED,
                "gemm: row pitch of A (%lld) and B (%lld) elements must be a multiple of %d for TMA",
                (long long)lda, (long long)ldb, 16 / eb);
  return 0;
}

// the instance for (operand type, type of C): C is the operand type, or fp32 for 16-bit
// operands whose accumulator is wanted unrounded
#define NB200_PICK(KERNEL, ...)                                                              \
  (dtype == NB200_F32    ? (const void*)KERNEL<__VA_ARGS__, NB200_F32, NB200_F32>            \
   : dtype == NB200_BF16 ? (c_f32 ? (const void*)KERNEL<__VA_ARGS__, NB200_BF16, NB200_F32>  \
                                  : (const void*)KERNEL<__VA_ARGS__, NB200_BF16, NB200_BF16>) \
                         : (c_f32 ? (const void*)KERNEL<__VA_ARGS__, NB200_F16, NB200_F32>   \
                                  : (const void*)KERNEL<__VA_ARGS__, NB200_F16, NB200_F16>))

template <int BN, int STAGES, int KSUB = 1>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int dtype, bool c_f32,
           int grid, cudaStream_t stream) {
  const int smem = smem_bytes_for(BN, STAGES, KSUB);
  const void* kern = NB200_PICK(gemm_kernel, BN, STAGES, KSUB);
  if (int rc = prepare_kernel(kern, smem)) return rc;
  void* args[3] = {(void*)&ta, (void*)&tb, (void*)&p};
  return cuda_check(cudaLaunchKernel(kern, dim3(grid), dim3(kThreads), args, smem, stream), "gemm launch");
}

// How many clusters of a pair kernel the device holds at once (asked once per device and instance).
int pair_capacity(const void* kern, int smem, int* clusters) {
  cudaLaunchConfig_t lc = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.blockDim = dim3(kThreads);
  lc.dynamicSmemBytes = smem;
  lc.attrs = attr;
  lc.numAttrs = 1;
  lc.gridDim = dim3(2);
  if (int rc = cluster_capacity(kern, &lc, clusters)) return rc;
  if (*clusters < 1) return fail(NB200_E_CUDA, "gemm: the device cannot host a CTA pair");
  return 0;
}

// The same, but never more than there are tiles: the grid of a launch whose tiles stay whole.
int pair_clusters(const void* kern, int smem, const GemmParams& p, int* clusters) {
  if (int rc = pair_capacity(kern, smem, clusters)) return rc;
  const long long tiles = (long long)cdiv64(p.m, 2 * kBlockM) * p.n_blocks;
  if (tiles < *clusters) *clusters = (int)tiles;
  return 0;
}

int pair_smem_bytes(int stages, int ksub, int nsub = 1) {
  return stages * ksub * (kBlockM * 128 + nsub * 128 * 128) + 1024 + (int)gemm::kEpilogueStageBytes;
}

// The compiled instance of the pair kernels a resolved configuration runs on.
struct PairInstance {
  const void* kern;
  int smem, ksub, nsub;
};

PairInstance pair_instance(const Resolved& cfg, int row_k, int dtype, bool c_f32) {
  PairInstance r;
  if (cfg.block_n == 512) {
    r.nsub = 2;
    r.ksub = cfg.block_k == 2 * row_k ? 2 : 1;
    r.kern = r.ksub == 2 ? NB200_PICK(gemm_pair_wide_kernel, 2, 2) : NB200_PICK(gemm_pair_wide_kernel, 4, 1);
    r.smem = pair_smem_bytes(r.ksub == 2 ? 2 : 4, r.ksub, 2);
    return r;
  }
  r.nsub = 1;
  int stages;
  if (cfg.block_k == 2 * row_k) {
    stages = 3, r.ksub = 2, r.kern = NB200_PICK(gemm_pair_kernel, 3, 2);
  } else if (cfg.block_k == 3 * row_k) {
    stages = 2, r.ksub = 3, r.kern = NB200_PICK(gemm_pair_kernel, 2, 3);
  } else {
    r.ksub = 1;
    stages = cfg.stages == 4 || cfg.stages == 5 ? cfg.stages : 6;
    r.kern = stages == 4 ? NB200_PICK(gemm_pair_kernel, 4, 1)
           : stages == 5 ? NB200_PICK(gemm_pair_kernel, 5, 1)
                         : NB200_PICK(gemm_pair_kernel, 6, 1);
  }
  r.smem = pair_smem_bytes(stages, r.ksub);
  return r;
}

int launch_pair(const PairInstance& inst, const CUtensorMap& ta, const CUtensorMap& tb,
                const GemmParams& p, int clusters, cudaStream_t stream) {
  cudaLaunchConfig_t lc = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.blockDim = dim3(kThreads);
  lc.dynamicSmemBytes = inst.smem;
  lc.stream = stream;
  lc.attrs = attr;
  lc.numAttrs = 1;
  lc.gridDim = dim3(2 * clusters);
  void* args[3] = {(void*)&ta, (void*)&tb, (void*)&p};
  return cuda_check(cudaLaunchKernelExC(&lc, inst.kern, args), "gemm pair launch");
}

// The split tail of a pair launch (GemmParams::sk_tiles ...): with `capacity` clusters resident
// and `tiles` tiles of `k_rounds` ring slots each, the tiles of the last, partly filled round are
// cut along K into as many equal parts as there are clusters per tile, one part per cluster.
// Splitting saves the k rounds the idle part of the chip would have sat through (~0.33 us each
// for a 256 x 256 tile on a B200, twice that for 512 columns) and costs the partial sums' way
// through L2 and a second launch: 17-23 k rounds' worth, measured (4096^3 in 256 x 256 tiles saves
// 32 and goes from 96.2 to 93.2 us; 2048^3 in 256 x 512 tiles saves 16 and loses 1 us).  The rule
// asks for more than 28 saved k rounds.  Knob gemm_split_tail: 1 = split whenever a part still
// has four k rounds, negative = never.
struct SplitPlan {
  int tiles, parts, len;   // tiles == 0: nothing is split
};
SplitPlan split_tail_plan(long long tiles, int k_rounds, int capacity) {
  SplitPlan none = {0, 0, 0};
  const int knob = tuning("gemm_split_tail", 0);
  if (knob < 0) return none;
  const int rest = (int)(tiles % capacity);
  if (rest == 0 || capacity / rest < 2) return none;
  int parts = capacity / rest;
  if (parts > k_rounds / 4) parts = k_rounds / 4;
  if (parts < 2) return none;
  const int len = (k_rounds + parts - 1) / parts;
  parts = (k_rounds + len - 1) / len;            // none of them empty
  if (knob == 0 && k_rounds - len <= 28) return none;
  return SplitPlan{rest, parts, len};
}

// Bytes of the workspace a split tail needs: a slot per cluster, a slot = one fp32 tile.
size_t split_workspace_bytes(int capacity, int nsub) {
  return (size_t)capacity * 256 * (256 * nsub) * 4;
}

// Adds up the parts of the split tiles and stores C: what the pair kernel's epilogue does for a
// whole tile.  Part s of split tile t lies in slot s * sk_tiles + t.  A thread has one row and 16
// columns (whole 32-byte sectors of a 16-bit C); its warp the 32 rows one epilogue warp of one
// CTA wrote.
// MANY = false, grid (BN / 16, split tiles): a block of 8 warps takes the 256 rows of a tile and
// every thread adds the parts one after the other -- tiles in two to seven parts.
// MANY = true, grid (BN / 16, 8 per split tile): a block takes 32 rows, its warp g adds parts g,
// g + 8, ... and warp 0 adds the eight sums in order -- a very small C, many parts per tile.
// Either way the order of the additions is fixed, so the result does not depend on which part
// was written last.  L2-bound: 4 bytes per element and part.
template <int CT, int BN, bool MANY>
__global__ void __launch_bounds__(256) split_reduce_kernel(const GemmParams p) {
  using OutT = typename gemm::ElemType<CT>::T;
  __shared__ float sums[MANY ? 8 : 1][16][32];
  const int t = MANY ? blockIdx.y >> 3 : blockIdx.y;
  const int rows32 = MANY ? (blockIdx.y & 7) : (threadIdx.x >> 5);
  const int m_blocks2 = (p.m + 2 * kBlockM - 1) / (2 * kBlockM);
  int mb, nb;
  gemm::tile_coords(m_blocks2 * p.n_blocks - p.sk_tiles + t, m_blocks2, p.n_blocks, p.group_m, &mb, &nb);
  const int g = MANY ? (threadIdx.x >> 5) : 0, lane = threadIdx.x & 31;
  const int row = mb * 2 * kBlockM + rows32 * 32 + lane;
  const int col = nb * BN + blockIdx.x * 16;
  if (col >= p.n) return;
  const long long piece = ((long long)rows32 * (BN / 4) + blockIdx.x * 4) * 32 + lane;   // 16-byte pieces
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  for (int s = g; s < p.sk_parts; s += MANY ? 8 : 1) {
    const float4* src =
        reinterpret_cast<const float4*>(p.sk_ws + (long long)(s * p.sk_tiles + t) * (256LL * BN)) + piece;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 v = __ldcg(src + j * 32);
      acc[4 * j] += v.x;
      acc[4 * j + 1] += v.y;
      acc[4 * j + 2] += v.z;
      acc[4 * j + 3] += v.w;
    }
  }
  if constexpr (MANY) {
#pragma unroll
    for (int j = 0; j < 16; ++j) sums[g][j][lane] = acc[j];
    __syncthreads();
    if (g != 0) return;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float v = sums[0][j][lane];
#pragma unroll
      for (int w = 1; w < 8; ++w) v += sums[w][j][lane];
      acc[j] = v;
    }
  }
  if (row >= p.m) return;
  OutT* crow = static_cast<OutT*>(p.c) + (long long)row * p.ldc + col;
  if (p.c_vec_ok && col + 16 <= p.n) {
    if constexpr (CT == NB200_F32) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        reinterpret_cast<float4*>(crow)[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    } else {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if constexpr (CT == NB200_BF16) {
          __nv_bfloat162 v2 = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&v2);
        } else {
          __half2 v2 = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&v2);
        }
      }
      reinterpret_cast<uint4*>(crow)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(crow)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (col + j < p.n) {
        if constexpr (CT == NB200_F32) crow[j] = acc[j];
        else if constexpr (CT == NB200_BF16) crow[j] = __float2bfloat16_rn(acc[j]);
        else crow[j] = __float2half_rn(acc[j]);
      }
  }
}

template <int BN>
int launch_split_reduce(const GemmParams& p, int dtype, cudaStream_t stream) {
  const bool many = p.sk_parts >= 8;
  const dim3 grid(BN / 16, p.sk_tiles * (many ? 8 : 1));
#define NB200_SPLIT_SUM(CT_)                                                  \
  if (many) split_reduce_kernel<CT_, BN, true><<<grid, 256, 0, stream>>>(p);  \
  else split_reduce_kernel<CT_, BN, false><<<grid, 256, 0, stream>>>(p);
  if (dtype == NB200_F32) { NB200_SPLIT_SUM(NB200_F32) }
  else if (dtype == NB200_BF16) { NB200_SPLIT_SUM(NB200_BF16) }
  else { NB200_SPLIT_SUM(NB200_F16) }
#undef NB200_SPLIT_SUM
  return cuda_check(cudaGetLastError(), "gemm split-tail sum launch");
}

}  // namespace

// ---- tensor-map encoding ---------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                            const uint64_t* strides_bytes, const uint32_t* box) {
  return encode_tensor_map(out, base, 2, rank, dims, strides_bytes, box);
}

int encode_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      bool atom32) {
  static EncodeTiledFn encode = nullptr;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
        return fail(NB200_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
      encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  // the payload is moved as raw bits; the element type only sets the size
  CUresult r = encode(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16,
                      (cuuint32_t)rank,
                      const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(NB200_E_INVALID, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace nb200

using namespace nb200;

namespace nb200 {
namespace {

// dst[r][c] = src[r * row_stride + c * col_stride]: a matrix given with any two strides is
// copied into a row-major one whose pitch bulk tensor copies accept.  64 x 64 tiles through
// shared memory, walked along whichever source direction is the closer to unit stride, so
// that both the reads and the writes coalesce.  HBM-bound: 2 * sizeof(T) bytes per element.
template <typename T>
__global__ void __launch_bounds__(256) repitch_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                      int rows, int cols, long long row_stride,
                                                      long long col_stride, long long dst_pitch) {
  __shared__ T tile[64][64 + 4 / sizeof(T)];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const bool along_rows = col_stride > row_stride;     // a transposed source
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = along_rows ? (i & 63) : (i >> 6), c = along_rows ? (i >> 6) : (i & 63);
    if (r0 + r < rows && c0 + c < cols)
      tile[r][c] = src[(long long)(r0 + r) * row_stride + (long long)(c0 + c) * col_stride];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    if (r0 + r < rows && c0 + c < cols) dst[(long long)(r0 + r) * dst_pitch + c0 + c] = tile[r][c];
  }
}

}  // namespace
}  // namespace nb200

extern "C" int nb200_repitch(const void* src, void* dst, int64_t rows, int64_t cols,
                             int64_t row_stride, int64_t col_stride, int64_t dst_pitch,
                             int elem_bytes, void* stream) {
  if (elem_bytes != 2 && elem_bytes != 4)
    return fail(NB200_E_UNSUPPORTED, "repitch: elements of %d bytes (2 or 4)", elem_bytes);
  if (rows < 0 || cols < 0 || rows > INT32_MAX || cols > INT32_MAX)
    return fail(NB200_E_INVALID, "repitch: extent out of range");
  if (rows == 0 || cols == 0) return 0;
  if (!src || !dst) return fail(NB200_E_INVALID, "repitch: null pointer");
  if (dst_pitch < cols) return fail(NB200_E_INVALID, "repitch: destination pitch smaller than a row");
  if (row_stride < 0 || col_stride < 0) return fail(NB200_E_UNSUPPORTED, "repitch: negative stride");
  const long long gx = cdiv64(cols, 64), gy = cdiv64(rows, 64);
  if (gy > 65535) return fail(NB200_E_UNSUPPORTED, "repitch: more than 65535 * 64 rows");
  const dim3 grid((unsigned)gx, (unsigned)gy);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (elem_bytes == 2)
    repitch_kernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(src),
                                                  static_cast<uint16_t*>(dst), (int)rows, (int)cols,
                                                  row_stride, col_stride, dst_pitch);
  else
    repitch_kernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(src),
                                                  static_cast<uint32_t*>(dst), (int)rows, (int)cols,
                                                  row_stride, col_stride, dst_pitch);
  return cuda_check(cudaGetLastError(), "repitch launch");
}

extern "C" int nb200_gemm_check(const void* a, const void* b, const void* c, int64_t m, int64_t n,
                                int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                                const nb200_gemm_config* config) {
  if (dtype == NB200_F32) {
    // as nb200_gemm_tf32 will see it: B replaced by its transposed copy in the workspace
    if (k > 0 && m > 0 && n > 0 && (!b || ldb < n))
      return fail(NB200_E_INVALID, "gemm: B is null or its row stride is smaller than the row");
    if (int rc = check_problem(a, a, c, m, n, k, lda, (k + 3) / 4 * 4, ldc, dtype, true)) return rc;
  } else if (int rc = check_problem(a, b, c, m, n, k, lda, ldb, ldc, dtype, false)) {
    return rc;
  }
  Resolved r;
  return resolve_config(config, m, n, dtype == NB200_F32 ? 32 : 64, &r);
}

namespace nb200 {

// Everything a launch needs, worked out on the host: the resolved tile configuration, the two
// tensor maps and the kernel's parameter block.  `c_bytes`: size of an element of C.
struct PlannedGemm {
  Resolved cfg;
  CUtensorMap ta, tb;
  GemmParams p;
  int row_k;
  bool nothing_to_do;   // an empty C
  bool only_clear;      // K == 0: C is its zero initial value
};

int plan_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
              int64_t ldb, int64_t ldc, int dtype, int c_bytes, const nb200_gemm_config* config,
              bool b_kmajor, PlannedGemm* out) {
  if (int rc = check_problem(a, b, c, m, n, k, lda, ldb, ldc, dtype, b_kmajor)) return rc;
  const int eb = dtype == NB200_F32 ? 4 : 2;   // bytes per element
  const int row_k = 128 / eb;                  // K elements per 128-byte row = columns per slab of B
  out->row_k = row_k;
  Resolved& cfg = out->cfg;
  if (int rc = resolve_config(config, m, n, row_k, &cfg)) return rc;
  out->nothing_to_do = m == 0 || n == 0;
  out->only_clear = !out->nothing_to_do && k == 0;
  if (out->nothing_to_do || out->only_clear) return 0;

  // K slabs per ring slot of the pair kernel; the one-CTA kernel's slots hold one
  const int ksub = cfg.block_k == 2 * row_k ? 2 : cfg.block_k == 3 * row_k ? 3 : 1;
  const bool whole_k_rows = k % row_k == 0;
  // A slot wants one copy per operand (see GemmParams::wide_a).  The 3-D views reach past a
  // ragged edge into the next row, so they are used only where there is no such edge.
  const bool wide_a = ksub > 1 && whole_k_rows;
  bool wide_b;
  if (wide_a) {   // [K / row, M, row]
    const uint64_t dims[3] = {(uint64_t)row_k, (uint64_t)m, (uint64_t)(k / row_k)};
    const uint64_t strides[2] = {(uint64_t)lda * eb, 128};
    const uint32_t box[3] = {(uint32_t)row_k, (uint32_t)kBlockM, (uint32_t)ksub};
    if (int rc = encode_tensor_map(&out->ta, a, eb, 3, dims, strides, box)) return rc;
  } else {
    const uint64_t dims[2] = {(uint64_t)k, (uint64_t)m};
    const uint64_t strides[1] = {(uint64_t)lda * eb};
    const uint32_t box[2] = {(uint32_t)row_k, (uint32_t)kBlockM};
    if (int rc = encode_tensor_map(&out->ta, a, eb, 2, dims, strides, box)) return rc;
  }
  if (b_kmajor) {   // rows of B^T: one box per CTA and K slab
    const uint32_t rows = (uint32_t)(cfg.pair ? 128 : cfg.block_n);
    wide_b = wide_a;
    if (wide_b) {
      const uint64_t dims[3] = {(uint64_t)row_k, (uint64_t)n, (uint64_t)(k / row_k)};
      const uint64_t strides[2] = {(uint64_t)ldb * eb, 128};
      const uint32_t box[3] = {(uint32_t)row_k, rows, (uint32_t)ksub};
      if (int rc = encode_tensor_map(&out->tb, b, eb, 3, dims, strides, box)) return rc;
    } else {
      const uint64_t dims[2] = {(uint64_t)k, (uint64_t)n};
      const uint64_t strides[1] = {(uint64_t)ldb * eb};
      const uint32_t box[2] = {(uint32_t)row_k, rows};
      if (int rc = encode_tensor_map(&out->tb, b, eb, 2, dims, strides, box)) return rc;
    }
  } else {
    const int slabs = (cfg.pair ? 128 : cfg.block_n) / row_k;   // column slabs per CTA
    const bool atom32 = eb == 4;   // an MN-major tf32 operand: the swizzle works on 32-byte atoms
    wide_b = n % row_k == 0 && slabs * ksub > 1;
    if (wide_b) {   // [N / slab, K, slab]
      const uint64_t dims[3] = {(uint64_t)row_k, (uint64_t)k, (uint64_t)(n / row_k)};
      const uint64_t strides[2] = {(uint64_t)ldb * eb, 128};
      const uint32_t box[3] = {(uint32_t)row_k, (uint32_t)(row_k * ksub), (uint32_t)slabs};
      if (int rc = encode_tensor_map(&out->tb, b, eb, 3, dims, strides, box, atom32)) return rc;
    } else {
      const uint64_t dims[2] = {(uint64_t)n, (uint64_t)k};
      const uint64_t strides[1] = {(uint64_t)ldb * eb};
      const uint32_t box[2] = {(uint32_t)row_k, (uint32_t)row_k};
      if (int rc = encode_tensor_map(&out->tb, b, eb, 2, dims, strides, box, atom32)) return rc;
    }
  }

  GemmParams& p = out->p;
  memset(&p, 0, sizeof(p));
  p.c = c;
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.m_blocks = (int)cdiv64(m, kBlockM);
  p.n_blocks = (int)cdiv64(n, cfg.block_n);
  p.k_blocks = (int)cdiv64(k, row_k);
  const int mma_m = cfg.pair ? 2 * kBlockM : kBlockM;
  const int mma_n = cfg.pair ? 256 : cfg.block_n;   // a 512-column pair tile is two MMAs wide
  p.idesc = dtype == NB200_F32
                ? sm100::instr_desc_tf32(mma_m, mma_n, false, !b_kmajor)
                : sm100::instr_desc_f16(mma_m, mma_n, dtype == NB200_BF16, false, !b_kmajor);
  p.b_kmajor = b_kmajor ? 1 : 0;
  p.wide_a = wide_a ? 1 : 0;
  p.group_m = tuning("gemm_group_m", 0) > 0 ? tuning("gemm_group_m", 0) : gemm::kGroupM;
  // 512-column tiles: the last ring of k rounds ends columns 0..255 first, and with a long K the
  // first ring starts with them as well (1622 -> 1633 -> 1643 TFLOP/s at 8192^3 bf16; the start
  // gives nothing below ~32 k rounds).  Knob gemm_half_tail: 1 = end only, 2 = both, negative = off.
  {
    const int knob = tuning("gemm_half_tail", 0);
    p.half_tail = knob < 0 ? 0 : knob > 0 ? knob : ksub > 1 ? 0 : (p.k_blocks >= 32 ? 2 : 1);   // nothing for the two-slot ring
  }
  p.wide_b = wide_b ? 1 : 0;
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(c) & 15) == 0 && (ldc * c_bytes) % 16 == 0) ? 1 : 0;
  p.c_tma = 0;
  if (p.c_vec_ok && tuning("gemm_c_tma", 0) >= 0) {
    // C for the epilogue's copies: boxes of 32 rows x 128 bytes (one pass of one epilogue warp)
    const uint64_t cdims[2] = {(uint64_t)n, (uint64_t)m};
    const uint64_t cstrides[1] = {(uint64_t)ldc * (uint64_t)c_bytes};
    const uint32_t cbox[2] = {(uint32_t)(128 / c_bytes), 32u};
    if (encode_tensor_map(&p.tmap_c, c, c_bytes, 2, cdims, cstrides, cbox) == 0) p.c_tma = 1;
  }
  p.wait_limit_ns = wait_limit_ns();
  p.status = device_status_ptr();
  if (!p.status) return fail(NB200_E_CUDA, "gemm: device status word is not addressable");
  return 0;
}

// C = A @ B with B given either as [K, N] (b_kmajor = false) or transposed as [N, K].
int gemm_impl(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
              int64_t ldb, int64_t ldc, int dtype, const nb200_gemm_config* config, bool b_kmajor,
              cudaStream_t stream, bool c_f32 = false, void* split_ws = nullptr,
              size_t split_ws_bytes = 0) {
  const int cb = (c_f32 || dtype == NB200_F32) ? 4 : 2;   // bytes per element of C
  PlannedGemm g;
  if (int rc = plan_gemm(a, b, c, m, n, k, lda, ldb, ldc, dtype, cb, config, b_kmajor, &g)) return rc;
  if (g.nothing_to_do) return 0;
  if (g.only_clear)  // empty reduction: the accumulator is its zero initial value
    return cuda_check(cudaMemset2DAsync(c, (size_t)ldc * cb, 0, (size_t)n * cb, (size_t)m, stream),
                      "gemm k=0 clear");
  const Resolved& cfg = g.cfg;
  const GemmParams& p = g.p;

  if (cfg.pair) {
    const PairInstance inst = pair_instance(cfg, g.row_k, dtype, c_f32);
    if (int rc = prepare_kernel(inst.kern, inst.smem)) return rc;
    int capacity = 0;
    if (int rc = pair_capacity(inst.kern, inst.smem, &capacity)) return rc;
    const long long tiles = (long long)cdiv64(p.m, 2 * kBlockM) * p.n_blocks;
    if (split_ws) {
      const int k_rounds = (p.k_blocks + inst.ksub - 1) / inst.ksub;
      const SplitPlan sp = split_tail_plan(tiles, k_rounds, capacity);
      if (sp.tiles > 0 && split_ws_bytes >= split_workspace_bytes(capacity, inst.nsub) &&
          (reinterpret_cast<uintptr_t>(split_ws) & 15) == 0) {
        GemmParams q = p;
        q.sk_tiles = sp.tiles;
        q.sk_parts = sp.parts;
        q.sk_len = sp.len;
        q.sk_ws = static_cast<float*>(split_ws);
        if (int rc = launch_pair(inst, g.ta, g.tb, q, capacity, stream)) return rc;
        return inst.nsub == 2 ? launch_split_reduce<512>(q, dtype, stream)
                              : launch_split_reduce<256>(q, dtype, stream);
      }
    }
    return launch_pair(inst, g.ta, g.tb, p, (int)(tiles < capacity ? tiles : capacity), stream);
  }
  const int64_t tiles = (int64_t)p.m_blocks * p.n_blocks;
  const int sms = device_info().sm_count;
  const int grid = (int)(tiles < sms ? tiles : sms);

  if (cfg.block_k == 2 * g.row_k)
    return cfg.block_n == 64 ? launch<64, 4, 2>(g.ta, g.tb, p, dtype, c_f32, grid, stream)
                             : launch<128, 3, 2>(g.ta, g.tb, p, dtype, c_f32, grid, stream);
#define NB200_GEMM_CASE(BN_, ST_)                  \
  if (cfg.block_n == BN_ && cfg.stages == ST_)     \
    return launch<BN_, ST_>(g.ta, g.tb, p, dtype, c_f32, grid, stream);
  NB200_GEMM_CASE(256, 4)
  NB200_GEMM_CASE(256, 3)
  NB200_GEMM_CASE(256, 2)
  NB200_GEMM_CASE(128, 6)
  NB200_GEMM_CASE(128, 4)
  NB200_GEMM_CASE(128, 3)
  NB200_GEMM_CASE(128, 2)
  NB200_GEMM_CASE(64, 8)
  NB200_GEMM_CASE(64, 6)
  NB200_GEMM_CASE(64, 4)
  NB200_GEMM_CASE(64, 2)
#undef NB200_GEMM_CASE
  return fail(NB200_E_UNSUPPORTED, "gemm: no kernel instance for block_n=%d stages=%d",
              cfg.block_n, cfg.stages);
}

namespace {

// dst[n][k] = src[k][n] for fp32: 64 x 64 tiles through shared memory, 16-byte accesses on
// both sides where the tile is whole and the pitches allow it, element by element at the
// ragged edges.  HBM-bound: 8 bytes per element.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                            int rows, int cols, long long ld_src, long long ld_dst,
                                                            int vec_ok) {
  __shared__ float tile[64][65];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads
  const bool whole = vec_ok && r0 + 64 <= rows && c0 + 64 <= cols;
  if (whole) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 16 * i;
      const float4 v = *reinterpret_cast<const float4*>(src + (long long)(r0 + r) * ld_src + c0 + 4 * tx);
      tile[r][4 * tx] = v.x;
      tile[r][4 * tx + 1] = v.y;
      tile[r][4 * tx + 2] = v.z;
      tile[r][4 * tx + 3] = v.w;
    }
  } else {
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
      const int r = i >> 6, c = i & 63;
      if (r0 + r < rows && c0 + c < cols) tile[r][c] = src[(long long)(r0 + r) * ld_src + c0 + c];
    }
  }
  __syncthreads();
  if (whole) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = ty + 16 * i;   // a source column = a destination row
      const float4 v = make_float4(tile[4 * tx][c], tile[4 * tx + 1][c], tile[4 * tx + 2][c],
                                   tile[4 * tx + 3][c]);
      *reinterpret_cast<float4*>(dst + (long long)(c0 + c) * ld_dst + r0 + 4 * tx) = v;
    }
  } else {
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
      const int c = i >> 6, r = i & 63;
      if (r0 + r < rows && c0 + c < cols) dst[(long long)(c0 + c) * ld_dst + r0 + r] = tile[r][c];
    }
  }
}

}  // namespace

// Row pitch (elements) of the transposed copy of a [K, N] fp32 matrix: K rounded up to the
// 16 bytes TMA wants -- and 128 bytes more when that makes rows a multiple of 32 KB apart, where
// the transposing pass would write all of a tile's 64 rows into the same few DRAM channels
// (measured at K = 8192: 2.1 TB/s instead of 5 TB/s).
int64_t tf32_workspace_pitch(int64_t k) {
  const int64_t pitch = (k + 3) / 4 * 4;
  return pitch % 8192 == 0 && pitch > 0 ? pitch + 32 : pitch;
}

// fp32 C = A @ B with B as [K, N].  A B that bulk tensor copies can fetch as it lies (16-byte
// aligned base and pitch) is read in place as an MN-major tf32 operand; any other B is first
// transposed into the workspace, [N, pitch], and read K-major.
int gemm_tf32_via(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
                  int64_t ldb, int64_t ldc, const nb200_gemm_config* config, void* workspace,
                  cudaStream_t stream) {
  if (m < 0 || n < 0 || k < 0) return fail(NB200_E_INVALID, "gemm: negative extent");
  if (n > INT32_MAX || k > INT32_MAX) return fail(NB200_E_INVALID, "gemm: extent beyond int32");
  if ((reinterpret_cast<uintptr_t>(b) & 15) == 0 && ldb % 4 == 0 && tuning("tf32_in_place", 1))
    return gemm_impl(a, b, c, m, n, k, lda, ldb, ldc, NB200_F32, config, false, stream);
  const int64_t pitch = tf32_workspace_pitch(k);
  if (m > 0 && n > 0 && k > 0) {
    if (!b) return fail(NB200_E_INVALID, "gemm: null tensor pointer");
    if (ldb < n) return fail(NB200_E_INVALID, "gemm: row stride of B smaller than the row");
    const dim3 grid((unsigned)cdiv64(n, 64), (unsigned)cdiv64(k, 64));
    if (grid.y > 65535u) return fail(NB200_E_INVALID, "gemm: K too large for the transposing pass");
    const int vec_ok = (reinterpret_cast<uintptr_t>(b) & 15) == 0 && ldb % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(workspace) & 15) == 0;   // pitch % 4 == 0 always
    transpose_f32_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(b),
                                                   static_cast<float*>(workspace), (int)k, (int)n, ldb,
                                                   pitch, vec_ok);
    if (int rc = cuda_check(cudaGetLastError(), "transpose launch")) return rc;
  }
  return gemm_impl(a, workspace, c, m, n, k, lda, pitch, ldc, NB200_F32, config, true, stream);
}

}  // namespace nb200

extern "C" int nb200_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                          int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                          const nb200_gemm_config* config, void* stream) {
  return gemm_impl(a, b, c, m, n, k, lda, ldb, ldc, dtype, config, false,
                   static_cast<cudaStream_t>(stream));
}

extern "C" int nb200_gemm_bt(const void* a, const void* bt, void* c, int64_t m, int64_t n, int64_t k,
                             int64_t lda, int64_t ldbt, int64_t ldc, int dtype,
                             const nb200_gemm_config* config, void* stream) {
  return gemm_impl(a, bt, c, m, n, k, lda, ldbt, ldc, dtype, config, true,
                   static_cast<cudaStream_t>(stream));
}

namespace nb200 {
namespace {
// The tile a split launch runs on when the caller leaves the choice to the library: the default
// of nb200_gemm looks at M and N only and gives a small C single-CTA tiles, which cannot be split;
// with a K long enough for the split to pay, 256 x 256 pair tiles are the better answer.
const nb200_gemm_config* config_for_split(const nb200_gemm_config* config, int64_t m, int64_t n,
                                          int64_t k, int dtype, nb200_gemm_config* storage) {
  if (config && (config->block_m || config->block_n || config->block_k || config->stages || config->cta_pair))
    return config;
  if (m <= 0 || n <= 0 || k <= 0) return config;
  const int row_k = dtype == NB200_F32 ? 32 : 64;
  const nb200_gemm_config pair256 = {256, 256, row_k, 6, 1};
  Resolved cfg;
  if (resolve_config(&pair256, m, n, row_k, &cfg) != 0) return config;
  const PairInstance inst = pair_instance(cfg, row_k, dtype, false);
  int capacity = 0;
  if (prepare_kernel(inst.kern, inst.smem) != 0 || pair_capacity(inst.kern, inst.smem, &capacity) != 0)
    return config;
  const long long tiles = (long long)cdiv64(m, 2 * kBlockM) * cdiv64(n, 256);
  if (split_tail_plan(tiles, (int)cdiv64(k, row_k), capacity).tiles == 0) return config;
  *storage = pair256;
  return storage;
}
}  // namespace
}  // namespace nb200

extern "C" int64_t nb200_gemm_split_workspace_bytes(int64_t m, int64_t n, int64_t k, int dtype,
                                                    const nb200_gemm_config* config) {
  if (dtype != NB200_F16 && dtype != NB200_BF16 && dtype != NB200_F32) return 0;
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  const int row_k = dtype == NB200_F32 ? 32 : 64;
  nb200_gemm_config chosen;
  config = config_for_split(config, m, n, k, dtype, &chosen);
  Resolved cfg;
  if (resolve_config(config, m, n, row_k, &cfg) != 0 || !cfg.pair) return 0;
  const PairInstance inst = pair_instance(cfg, row_k, dtype, false);
  int capacity = 0;
  if (prepare_kernel(inst.kern, inst.smem) != 0 || pair_capacity(inst.kern, inst.smem, &capacity) != 0)
    return 0;
  const long long tiles = (long long)cdiv64(m, 2 * kBlockM) * cdiv64(n, cfg.block_n);
  const int k_rounds = (int)cdiv64(cdiv64(k, row_k), inst.ksub);
  return split_tail_plan(tiles, k_rounds, capacity).tiles > 0
             ? (int64_t)split_workspace_bytes(capacity, inst.nsub) : 0;
}

extern "C" int nb200_gemm_split(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                                int64_t lda, int64_t ldb, int64_t ldc, int dtype, int b_transposed,
                                const nb200_gemm_config* config, void* workspace,
                                int64_t workspace_bytes, void* stream) {
  nb200_gemm_config chosen;
  if (workspace && workspace_bytes > 0) config = config_for_split(config, m, n, k, dtype, &chosen);
  return gemm_impl(a, b, c, m, n, k, lda, ldb, ldc, dtype, config, b_transposed != 0,
                   static_cast<cudaStream_t>(stream), false, workspace,
                   workspace_bytes > 0 ? (size_t)workspace_bytes : 0);
}

extern "C" int nb200_gemm_acc32(const void* a, const void* b, float* c, int64_t m, int64_t n,
                                int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                                int b_transposed, const nb200_gemm_config* config, void* stream) {
  if (dtype != NB200_F16 && dtype != NB200_BF16)
    return fail(NB200_E_UNSUPPORTED, "gemm_acc32: fp16 or bf16 operands (fp32 ones already give an "
                                     "fp32 result through nb200_gemm_tf32 / nb200_gemm_bt)");
  return gemm_impl(a, b, c, m, n, k, lda, ldb, ldc, dtype, config, b_transposed != 0,
                   static_cast<cudaStream_t>(stream), true);
}

extern "C" int64_t nb200_gemm_params_bytes(void) { return (int64_t)sizeof(gemm::GemmParams); }

extern "C" int nb200_gemm_plan(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                               int64_t lda, int64_t ldb, int64_t ldc, int dtype, int c_dtype,
                               int b_transposed, const nb200_gemm_config* config, void* tensor_map_a,
                               void* tensor_map_b, void* params, nb200_gemm_launch* launch) {
  if (dtype != NB200_F16 && dtype != NB200_BF16)
    return fail(NB200_E_UNSUPPORTED, "gemm_plan: fp16 or bf16 operands");
  if (c_dtype != NB200_F16 && c_dtype != NB200_BF16 && c_dtype != NB200_F32)
    return fail(NB200_E_INVALID, "gemm_plan: unknown dtype code %d for C", c_dtype);
  if (!tensor_map_a || !tensor_map_b || !params || !launch)
    return fail(NB200_E_INVALID, "gemm_plan: null output buffer");
  if ((reinterpret_cast<uintptr_t>(tensor_map_a) | reinterpret_cast<uintptr_t>(tensor_map_b)) & 63)
    return fail(NB200_E_INVALID, "gemm_plan: tensor maps must be 64-byte aligned");
  PlannedGemm g;
  if (int rc = plan_gemm(a, b, c, m, n, k, lda, ldb, ldc, dtype, c_dtype == NB200_F32 ? 4 : 2, config,
                         b_transposed != 0, &g))
    return rc;
  memset(launch, 0, sizeof(*launch));
  launch->nothing = g.nothing_to_do ? 1 : 0;
  launch->only_clear = g.only_clear ? 1 : 0;
  if (g.nothing_to_do || g.only_clear) return 0;
  memcpy(tensor_map_a, &g.ta, sizeof(CUtensorMap));
  memcpy(tensor_map_b, &g.tb, sizeof(CUtensorMap));
  memcpy(params, &g.p, sizeof(g.p));
  launch->block = kThreads;
  launch->block_n = g.cfg.block_n;
  if (g.cfg.pair) {
    // the instances the library has itself: 3 slots of two K slabs, 2 of three, 4..6 of one
    int stages = g.cfg.stages, ksub = 1;
    const bool wide = g.cfg.block_n == 512;
    if (wide) ksub = g.cfg.block_k == 2 * g.row_k ? 2 : 1;
    else if (g.cfg.block_k == 2 * g.row_k) stages = 3, ksub = 2;
    else if (g.cfg.block_k == 3 * g.row_k) stages = 2, ksub = 3;
    else stages = stages < 4 ? 4 : (stages > 6 ? 6 : stages);
    launch->pair = 1;
    launch->stages = stages;
    launch->ksub = ksub;
    launch->cluster = 2;
    launch->smem_bytes = pair_smem_bytes(stages, ksub, wide ? 2 : 1);
    // as many pairs as the device holds of the library's own instance of this shape
    const void* twin = wide ? (ksub == 2 ? (const void*)gemm_pair_wide_kernel<2, 2, NB200_BF16, NB200_BF16>
                                         : (const void*)gemm_pair_wide_kernel<4, 1, NB200_BF16, NB200_BF16>)
                     : stages == 3 && ksub == 2 ? (const void*)gemm_pair_kernel<3, 2, NB200_BF16, NB200_BF16>
                     : stages == 2 && ksub == 3 ? (const void*)gemm_pair_kernel<2, 3, NB200_BF16, NB200_BF16>
                     : stages == 4 ? (const void*)gemm_pair_kernel<4, 1, NB200_BF16, NB200_BF16>
                     : stages == 5 ? (const void*)gemm_pair_kernel<5, 1, NB200_BF16, NB200_BF16>
                                   : (const void*)gemm_pair_kernel<6, 1, NB200_BF16, NB200_BF16>;
    if (int rc = prepare_kernel(twin, launch->smem_bytes)) return rc;
    int clusters = 0;
    if (int rc = pair_clusters(twin, launch->smem_bytes, g.p, &clusters)) return rc;
    launch->grid = 2 * clusters;
    return 0;
  }
  launch->stages = g.cfg.stages;
  launch->ksub = g.cfg.block_k == 2 * g.row_k ? 2 : 1;
  launch->cluster = 1;
  launch->smem_bytes = smem_bytes_for(g.cfg.block_n, g.cfg.stages, launch->ksub);
  const int64_t tiles = (int64_t)g.p.m_blocks * g.p.n_blocks;
  const int sms = device_info().sm_count;
  launch->grid = (int)(tiles < sms ? tiles : sms);
  return 0;
}

extern "C" int64_t nb200_gemm_tf32_workspace_bytes(int64_t n, int64_t k) {
  return n < 0 || k < 0 ? 0 : n * tf32_workspace_pitch(k) * 4;
}

extern "C" int nb200_gemm_tf32(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                               int64_t lda, int64_t ldb, int64_t ldc, const nb200_gemm_config* config,
                               void* workspace, int64_t workspace_bytes, void* stream) {
  if (m > 0 && n > 0 && k > 0) {
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15))
      return fail(NB200_E_INVALID, "gemm_tf32: the workspace must be a 16-byte aligned device buffer");
    if (workspace_bytes < nb200_gemm_tf32_workspace_bytes(n, k))
      return fail(NB200_E_INVALID, "gemm_tf32: workspace of %lld bytes, %lld needed",
                  (long long)workspace_bytes, (long long)nb200_gemm_tf32_workspace_bytes(n, k));
  }
  return gemm_tf32_via(a, b, c, m, n, k, lda, ldb, ldc, config, workspace,
                       static_cast<cudaStream_t>(stream));
}

// ---- the same product for callers that have no workspace to give ---------------------
//
// Scratch for the transposed copy of B, inside the library image: 4 MiB on every GPU that
// loads the library, for as long as the process lives.
#define NB200_TF32_STATIC_FLOATS (1 << 20)
static __device__ __align__(256) float g_tf32_static_scratch[NB200_TF32_STATIC_FLOATS];

namespace nb200 {
namespace {

// Device address of the scratch array on the current device.  The array's name means
// something only to device code; host code has to ask the runtime where it lives, once per
// device and with that device current.
float* tf32_static_scratch(int* rc) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static float* address[kMaxDevices] = {};
  *rc = 0;
  int dev = -1;
  if ((*rc = cuda_check(cudaGetDevice(&dev), "current device")) != 0) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) {
    *rc = fail(NB200_E_UNSUPPORTED, "gemm_tf32_static: device index %d beyond %d", dev, kMaxDevices - 1);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!address[dev]) {
    void* ptr = nullptr;
    if ((*rc = cuda_check(cudaGetSymbolAddress(&ptr, g_tf32_static_scratch),
                          "address of the static tf32 scratch")) != 0)
      return nullptr;
    address[dev] = static_cast<float*>(ptr);
  }
  return address[dev];
}

}  // namespace
}  // namespace nb200

extern "C" int nb200_gemm_tf32_static(const void* a, const void* b, void* c, int64_t m, int64_t n,
                                      int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                                      const nb200_gemm_config* config, void* stream) {
  if (m < 0 || n < 0 || k < 0) return fail(NB200_E_INVALID, "gemm: negative extent");
  const int64_t need = n * tf32_workspace_pitch(k);   // floats of the transposed copy
  if (m > 0 && n > 0 && k > 0 && need > NB200_TF32_STATIC_FLOATS)
    return fail(NB200_E_UNSUPPORTED,
                "gemm_tf32_static: B transposed needs %lld floats, the built-in scratch holds %d "
                "(n * round_up(k, 4) <= 1048576, a k that is a multiple of 8192 counting 32 more); "
                "use nb200_gemm_tf32 with a workspace",
                (long long)need, NB200_TF32_STATIC_FLOATS);
  int rc = 0;
  float* scratch = tf32_static_scratch(&rc);
  if (rc) return rc;
  return gemm_tf32_via(a, b, c, m, n, k, lda, ldb, ldc, config, scratch,
                       static_cast<cudaStream_t>(stream));
}

#ifdef NB200_GEMM_TRACE
extern "C" int nb200_debug_gemm_trace(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, nb200::gemm::g_gemm_trace, sizeof(nb200::gemm::g_gemm_trace));
}
#endif
