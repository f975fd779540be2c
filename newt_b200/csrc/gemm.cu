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
//     over transposed, [N,K] -> K-major operand.  tf32 operands are read K-major only (an
//     MN-major B gives zeros), so an fp32 B as [K,N] goes through a transposing pass into a
//     caller-provided workspace first (nb200_gemm_tf32);
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
#include <type_traits>

#include "sm100.cuh"

namespace nb200 {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;
// fp32 operands run as tf32 (kind::tf32 reads the upper 19 bits of each word): everything
// below is laid out in 128-byte rows, so a row holds 32 K-elements instead of 64, a slab of B
// 32 columns instead of 64, and one MMA consumes 8 K-elements instead of 16 -- the same 32
// bytes.  Stage sizes, descriptor strides along K of A and the MMA count do not change.
template <int DT>
struct Elem {
  static constexpr int kBytes = DT == NB200_F32 ? 4 : 2;
  static constexpr int kPerRow = 128 / kBytes;   // K elements per stage = columns per slab of B
  using Out = typename std::conditional<DT == NB200_F32, float,
              typename std::conditional<DT == NB200_BF16, __nv_bfloat16, __half>::type>::type;
};
template <int DT>
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                       uint32_t acc) {
  if constexpr (DT == NB200_F32) mma_tf32_ss(d, a, b, idesc, acc);
  else mma_f16_ss(d, a, b, idesc, acc);
}
template <int DT>
__device__ __forceinline__ void mma_ss_pair(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                            uint32_t acc) {
  if constexpr (DT == NB200_F32) mma_tf32_ss_pair(d, a, b, idesc, acc);
  else mma_f16_ss_pair(d, a, b, idesc, acc);
}
// 32 accumulator columns of one row -> global memory, one rounding (none for fp32)
template <int DT>
__device__ __forceinline__ void store_chunk(typename Elem<DT>::Out* crow, int col0, int n,
                                            bool vec_ok, const uint32_t (&r)[32]) {
  using OutT = typename Elem<DT>::Out;
  if constexpr (DT == NB200_F32) {
#pragma unroll
    for (int g = 0; g < 8; ++g) {   // 4 columns = 16 bytes per group
      const int col = col0 + g * 4;
      if (vec_ok && col + 4 <= n) {
        *reinterpret_cast<uint4*>(crow + col) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (col + j < n) crow[col + j] = __uint_as_float(r[g * 4 + j]);
      }
    }
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g) {   // 8 columns = 16 bytes per group
      const int col = col0 + g * 8;
      uint32_t packed[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float lo = __uint_as_float(r[g * 8 + 2 * h]);
        const float hi = __uint_as_float(r[g * 8 + 2 * h + 1]);
        if constexpr (DT == NB200_BF16) {
          __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
          packed[h] = *reinterpret_cast<uint32_t*>(&v);
        } else {
          __half2 v = __floats2half2_rn(lo, hi);
          packed[h] = *reinterpret_cast<uint32_t*>(&v);
        }
      }
      if (vec_ok && col + 8 <= n) {
        *reinterpret_cast<uint4*>(crow + col) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      } else {
        const OutT* e = reinterpret_cast<const OutT*>(packed);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col + j < n) crow[col + j] = e[j];
      }
    }
  }
}
constexpr int kThreads = 192;
constexpr int kGroupM = 8;      // row-blocks per L2 band of the tile order

struct GemmParams {
  void* c;
  long long ldc;
  int m, n, k;
  int m_blocks, n_blocks, k_blocks;
  uint32_t idesc;
  int c_vec_ok;  // C base and row pitch are 16-byte aligned
  int b_kmajor;  // B is given transposed ([N, K], K contiguous); always so for tf32
  int c_f32;     // 16-bit operands, but C takes the fp32 accumulator unrounded
  unsigned long long wait_limit_ns;
  unsigned int* status;
};

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int* mb,
                                            int* nb) {
  // bands of kGroupM row-blocks; inside a band, column-blocks advance slowest
  const int band_tiles = kGroupM * n_blocks;
  const int band = tile / band_tiles;
  const int first_m = band * kGroupM;
  const int rows = min(kGroupM, m_blocks - first_m);
  const int in_band = tile - band * band_tiles;
  *mb = first_m + in_band % rows;
  *nb = in_band / rows;
}

template <int BN, int STAGES, int DT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  constexpr int kBK = Elem<DT>::kPerRow;                // K elements per stage
  constexpr int kSlab = Elem<DT>::kPerRow;              // columns of B per slab
  constexpr uint32_t kABytes = kBlockM * 128;           // 16 KB
  constexpr uint32_t kBSlab = kBK * 128;                // one slab of B: 8 KB (4 KB for tf32)
  constexpr uint32_t kBBytes = kBSlab * (BN / kSlab);
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators, BN fp32 columns each

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1 KB
  const WaitCtx ctx{&abort_flag, p.status, p.wait_limit_ns};

  if (threadIdx.x == 0) {
    abort_flag = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full_bar[b]), 1);
      mbar_init(smem_u32(&acc_empty_bar[b]), 4);  // one arrival per epilogue warp
    }
    mbar_init_fence();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  const int num_tiles = p.m_blocks * p.n_blocks;
  // The tensor core takes tf32 operands K-major only (an MN-major B gives zeros), so fp32
  // always comes with B transposed; for 16-bit types it is the caller's choice.
  const bool b_kmajor = DT == NB200_F32 || p.b_kmajor != 0;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p.m_blocks, p.n_blocks, &mb, &nb);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, ctx, ST_WAIT_SMEM_EMPTY, tile);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          mbar_arrive_expect_tx(bar, kStageBytes);
          tma_load_2d(a_dst, &tmap_a, kb * kBK, mb * kBlockM, bar);
          if (b_kmajor) {   // BN rows of B^T, one 128-byte row of K each
            tma_load_2d(a_dst + kABytes, &tmap_b, kb * kBK, nb * BN, bar);
          } else {
#pragma unroll
            for (int j = 0; j < BN / kSlab; ++j)
              tma_load_2d(a_dst + kABytes + j * kBSlab, &tmap_b, nb * BN + j * kSlab, kb * kBK, bar);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop and waits; one elected lane issues, so the warp's
    // control flow stays uniform and descriptors live in uniform registers.
    {
      const bool elected = elect_one();
      auto wait_all = [&](uint64_t* bar, uint32_t parity, unsigned int code, int tile) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, ctx, code, tile));
      };
      // A: K-major, 8-row groups 1024 B apart.  B: MN-major, 8-row K groups
      // 1024 B apart, 64-column slabs kBSlab apart.
      constexpr uint64_t kADesc = smem_desc_sw128(16, 1024);
      constexpr uint64_t kBDesc = smem_desc_sw128(kBSlab, 1024);
      const uint32_t b_step = b_kmajor ? 2u : uint32_t(2 * kBK);   // descriptor units of 16 B per MMA
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = wait_all(&acc_empty_bar[buf], acc_phase ^ 1, ST_WAIT_ACC_EMPTY, tile);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          ok = wait_all(&full_bar[stage], phase, ST_WAIT_TMA_FULL, tile);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint64_t a_desc = with_address(kADesc, a_addr);
          const uint64_t b_desc = with_address(b_kmajor ? kADesc : kBDesc, a_addr + kABytes);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            // +32 B along K inside a K-major swizzle row; + a quarter of the stage's K-rows
            // (128 B each) inside an MN-major slab of B
            if (elected)
              mma_ss<DT>(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * b_step),
                         p.idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          if (elected) mma_commit(smem_u32(&empty_bar[stage]));  // slot reusable once these retire
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && elected) mma_commit(smem_u32(&acc_full_bar[buf]));
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    using OutT = typename Elem<DT>::Out;
    OutT* c = static_cast<OutT*>(p.c);
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(tile, p.m_blocks, p.n_blocks, &mb, &nb);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(smem_u32(&acc_full_bar[buf]), acc_phase, ctx, ST_WAIT_ACC_FULL, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = mb * kBlockM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN;
      OutT* crow = c + (long long)row * p.ldc;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = nb * BN + c0;
        if (col0 >= p.n) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        if (row < p.m) {
          if (DT != NB200_F32 && p.c_f32)
            store_chunk<NB200_F32>(static_cast<float*>(p.c) + (long long)row * p.ldc, col0, p.n,
                                   p.c_vec_ok != 0, r);
          else
            store_chunk<DT>(crow, col0, p.n, p.c_vec_ok != 0, r);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[buf]));
    }
  }

  __syncthreads();
  if (abort_flag) {
    // give bulk copies that may still be in flight time to land before the
    // shared memory they target is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- CTA-pair variant: 256 x 256 output tile per cluster of two CTAs ---------------
//
// Each CTA of the pair loads its own 128 rows of A and its own 128 columns of B (no
// multicast), so a stage costs 32 KB per CTA instead of 48 KB and the ring can be 6-7
// deep; the leader CTA issues one tcgen05.mma.cta_group::2 (M = 256) that reads both
// CTAs' shared memory and accumulates 128 rows in each CTA's tensor memory.
// Barriers: `full` lives in the leader; the leader's producer announces the bytes of both
// CTAs' copies and every copy (cta_group::2 form) reports its bytes there, so nothing but
// the copies themselves crosses to the other SM per stage (a remote release-arrive per
// stage capped the ring at one slot per ~0.8 us).  `empty` and `acc_full` exist in both
// CTAs and the leader commits to each; `acc_empty` lives in the leader and collects the
// epilogue warps of both CTAs, once per tile.
// KSUB 64-element K slabs share one ring slot (one barrier round trip and one pair of
// commits per slot).
template <int STAGES, int KSUB, int DT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  constexpr int BN = 256;                                // cluster tile width
  constexpr int kBK = Elem<DT>::kPerRow;                 // K elements per 128-byte row
  constexpr int kSlab = Elem<DT>::kPerRow;               // columns of B per slab
  constexpr uint32_t kABytes = kBlockM * 128;            // this CTA's 128 rows of A: 16 KB
  constexpr uint32_t kBSlab = kBK * 128;                 // one slab of B: 8 KB (4 KB for tf32)
  constexpr uint32_t kBBytes = kBSlab * (128 / kSlab);   // this CTA's 128 columns of B
  constexpr uint32_t kSlabBytes = kABytes + kBBytes;     // 32 KB per 64 elements of K
  constexpr uint32_t kStageBytes = KSUB * kSlabBytes;
  constexpr uint32_t kTmemCols = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const WaitCtx ctx{&abort_flag, p.status, p.wait_limit_ns};

  if (threadIdx.x == 0) {
    abort_flag = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);    // the leader's copy is the one in use
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full_bar[b]), 1);
      mbar_init(smem_u32(&acc_empty_bar[b]), 8);  // four epilogue warps in each CTA
    }
    mbar_init_fence();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc_pair(smem_u32(&tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  const bool b_kmajor = DT == NB200_F32 || p.b_kmajor != 0;   // see gemm_kernel
  const int m_blocks2 = (p.m + 2 * kBlockM - 1) / (2 * kBlockM);
  const int num_tiles = m_blocks2 * p.n_blocks;
  const int first = cluster_id_x(), step = cluster_count_x();
  const int k_rounds = (p.k_blocks + KSUB - 1) / KSUB;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first; tile < num_tiles && ok; tile += step) {
        int mb, nb;
        tile_coords(tile, m_blocks2, p.n_blocks, &mb, &nb);
        const int row0 = mb * 2 * kBlockM + rank * kBlockM;
        const int col0 = nb * BN + rank * (BN / 2);
        for (int kb = 0; kb < k_rounds; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, ctx, ST_WAIT_SMEM_EMPTY, tile);
          if (!ok) break;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * kStageBytes);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {   // slabs past K are zero-filled by the tensor map
            const uint32_t a_dst = smem_base + stage * kStageBytes + sub * kSlabBytes;
            const int k0 = (kb * KSUB + sub) * kBK;
            tma_load_2d_pair(a_dst, &tmap_a, k0, row0, bar);
            if (b_kmajor) {   // this CTA's 128 rows of B^T
              tma_load_2d_pair(a_dst + kABytes, &tmap_b, k0, col0, bar);
            } else {
#pragma unroll
              for (int j = 0; j < 128 / kSlab; ++j)
                tma_load_2d_pair(a_dst + kABytes + j * kBSlab, &tmap_b, col0 + j * kSlab, k0, bar);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only; whole warp, elected lane issues) --------
    if (leader) {
      const bool elected = elect_one();
      auto wait_all = [&](uint64_t* bar, uint32_t parity, unsigned int code, int tile) -> bool {
        return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, ctx, code, tile));
      };
      // the barriers the commits signal, in each CTA's window of the cluster address space
      // (barrier i of an array is 8 bytes after barrier i-1 there as well)
      const uint32_t empty0 = map_to_cta(smem_u32(&empty_bar[0]), 0);
      const uint32_t empty1 = map_to_cta(smem_u32(&empty_bar[0]), 1);
      const uint32_t acc_full0 = map_to_cta(smem_u32(&acc_full_bar[0]), 0);
      const uint32_t acc_full1 = map_to_cta(smem_u32(&acc_full_bar[0]), 1);
      constexpr uint64_t kADesc = smem_desc_sw128(16, 1024);
      constexpr uint64_t kBDesc = smem_desc_sw128(kBSlab, 1024);
      const uint32_t b_step = b_kmajor ? 2u : uint32_t(2 * kBK);   // descriptor units of 16 B per MMA
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = first; tile < num_tiles && ok; tile += step, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = wait_all(&acc_empty_bar[buf], acc_phase ^ 1, ST_WAIT_ACC_EMPTY, tile);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < k_rounds; ++kb) {
          ok = wait_all(&full_bar[stage], phase, ST_WAIT_TMA_FULL, tile);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const uint32_t a_addr = smem_base + stage * kStageBytes + sub * kSlabBytes;
            const uint64_t a_desc = with_address(kADesc, a_addr);
            const uint64_t b_desc = with_address(b_kmajor ? kADesc : kBDesc, a_addr + kABytes);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              if (elected)
                mma_ss_pair<DT>(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * b_step),
                                p.idesc, (kb | sub | kk) != 0 ? 1u : 0u);
          }
          // the slot is free in both CTAs once these MMAs retire
          if (elected) {
            mma_commit_pair(empty0 + stage * 8);
            mma_commit_pair(empty1 + stage * 8);
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && elected) {
          mma_commit_pair(acc_full0 + buf * 8);
          mma_commit_pair(acc_full1 + buf * 8);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 128 rows of the 256-row tile ----------------
    const int quarter = warp & 3;
    using OutT = typename Elem<DT>::Out;
    OutT* c = static_cast<OutT*>(p.c);
    int it = 0;
    bool ok = true;
    for (int tile = first; tile < num_tiles && ok; tile += step, ++it) {
      int mb, nb;
      tile_coords(tile, m_blocks2, p.n_blocks, &mb, &nb);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(smem_u32(&acc_full_bar[buf]), acc_phase, ctx, ST_WAIT_ACC_FULL, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = mb * 2 * kBlockM + rank * kBlockM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN;
      OutT* crow = c + (long long)row * p.ldc;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = nb * BN + c0;
        if (col0 >= p.n) break;
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        if (row < p.m) {
          if (DT != NB200_F32 && p.c_f32)
            store_chunk<NB200_F32>(static_cast<float*>(p.c) + (long long)row * p.ldc, col0, p.n,
                                   p.c_vec_ok != 0, r);
          else
            store_chunk<DT>(crow, col0, p.n, p.c_vec_ok != 0, r);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[buf]), 0));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  cluster_sync_all();   // nobody leaves while the other CTA may still touch its barriers or tiles
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ---- host ----------------------------------------------------------------------

struct Resolved {
  int block_n;
  int block_k;
  int stages;
  bool pair;
};

int smem_bytes_for(int block_n, int stages) {   // a stage is 128 bytes of K for every row and column
  return stages * (kBlockM * 128 + 128 * block_n) + 1024;
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
  }
  out->pair = pair;
  if (pair) {
    if (bm != 0 && bm != 2 * kBlockM)
      return fail(NB200_E_INVALID, "block_m=%d: a CTA pair computes 256-row tiles", bm);
    if (bn != 0 && bn != 256)
      return fail(NB200_E_INVALID, "block_n=%d: CTA-pair tiles are 256 columns wide", bn);
    if (bk != 0 && bk != kBlockK && bk != 2 * kBlockK && bk != 3 * kBlockK)
      return fail(NB200_E_INVALID,
                  "block_k=%d: a CTA-pair ring slot holds %d, %d or %d elements of K", bk, kBlockK,
                  2 * kBlockK, 3 * kBlockK);
    out->block_k = bk == 0 ? 2 * kBlockK : bk;
    if (stages != 0 && (stages < 1 || stages > 8))
      return fail(NB200_E_INVALID, "stages=%d: supported 1..8", stages);
    out->block_n = 256;
    // ring depth: 3 slots of 128 K-elements, 2 of 192, 4..7 of 64
    out->stages = out->block_k == 2 * kBlockK ? 3 : (out->block_k == 3 * kBlockK ? 2 :
                  (stages == 0 ? 6 : (stages >= 7 ? 7 : (stages >= 6 ? 6 : (stages >= 5 ? 5 : 4)))));
    return 0;
  }
  if (bm != 0 && bm != kBlockM)
    return fail(NB200_E_INVALID, "block_m=%d: MMA tiles are 128 rows (256 for a CTA pair)", bm);
  if (bk != 0 && bk != kBlockK)
    return fail(NB200_E_INVALID, "block_k=%d: the TMA ring moves %d-element K slabs", bk, kBlockK);
  if (bn == 0) bn = n <= 64 ? 64 : (n <= 128 ? 128 : 256);
  if (bn != 64 && bn != 128 && bn != 256)
    return fail(NB200_E_INVALID, "block_n=%d: supported 64, 128, 256", bn);
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
  if (dtype == NB200_F32 && !b_kmajor)
    return fail(NB200_E_UNSUPPORTED,
                "gemm: fp32 operands run as tf32, which the tensor core reads K-major only: pass B "
                "transposed (nb200_gemm_bt) or let nb200_gemm_tf32 transpose it into a workspace");
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

template <int BN, int STAGES>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int dtype, int grid,
           cudaStream_t stream) {
  const int smem = smem_bytes_for(BN, STAGES);
  auto go = [&](auto kern) {
    if (int rc = prepare_kernel((const void*)kern, smem)) return rc;
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
    return cuda_check(cudaGetLastError(), "gemm launch");
  };
  if (dtype == NB200_BF16) return go(gemm_kernel<BN, STAGES, NB200_BF16>);
  if (dtype == NB200_F32) return go(gemm_kernel<BN, STAGES, NB200_F32>);
  return go(gemm_kernel<BN, STAGES, NB200_F16>);
}

template <int STAGES, int KSUB>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int dtype,
                cudaStream_t stream) {
  const int smem = STAGES * KSUB * (kBlockM * 128 + 128 * 128) + 1024;
  const void* kern = dtype == NB200_BF16 ? (const void*)gemm_pair_kernel<STAGES, KSUB, NB200_BF16>
                     : dtype == NB200_F32 ? (const void*)gemm_pair_kernel<STAGES, KSUB, NB200_F32>
                                          : (const void*)gemm_pair_kernel<STAGES, KSUB, NB200_F16>;
  if (int rc = prepare_kernel(kern, smem)) return rc;
  cudaLaunchConfig_t lc = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.blockDim = dim3(kThreads);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  lc.attrs = attr;
  lc.numAttrs = 1;
  // as many pairs as the device can hold at once, never more than there are tiles
  lc.gridDim = dim3(2);
  int clusters = 0;
  if (int rc = cluster_capacity(kern, &lc, &clusters)) return rc;
  if (clusters < 1) return fail(NB200_E_CUDA, "gemm: the device cannot host a CTA pair");
  const long long tiles = (long long)cdiv64(p.m, 2 * kBlockM) * p.n_blocks;
  if (tiles < clusters) clusters = (int)tiles;
  lc.gridDim = dim3(2 * clusters);
  void* args[3] = {(void*)&ta, (void*)&tb, (void*)&p};
  return cuda_check(cudaLaunchKernelExC(&lc, kern, args), "gemm pair launch");
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
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box) {
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
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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
// C = A @ B with B given either as [K, N] (b_kmajor = false) or transposed as [N, K].
int gemm_impl(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
              int64_t ldb, int64_t ldc, int dtype, const nb200_gemm_config* config, bool b_kmajor,
              cudaStream_t stream, bool c_f32 = false) {
  if (int rc = check_problem(a, b, c, m, n, k, lda, ldb, ldc, dtype, b_kmajor)) return rc;
  const int eb = dtype == NB200_F32 ? 4 : 2;   // bytes per element
  const int row_k = 128 / eb;                  // K elements per 128-byte row = columns per slab of B
  Resolved cfg;
  if (int rc = resolve_config(config, m, n, row_k, &cfg)) return rc;
  if (m == 0 || n == 0) return 0;
  const int cb = c_f32 ? 4 : eb;                // bytes per element of C
  if (k == 0)  // empty reduction: the accumulator is its zero initial value
    return cuda_check(cudaMemset2DAsync(c, (size_t)ldc * cb, 0, (size_t)n * cb, (size_t)m, stream),
                      "gemm k=0 clear");

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {(uint64_t)k, (uint64_t)m};
    const uint64_t strides[1] = {(uint64_t)lda * eb};
    const uint32_t box[2] = {(uint32_t)row_k, (uint32_t)kBlockM};
    if (int rc = encode_tensor_map(&ta, a, eb, 2, dims, strides, box)) return rc;
  }
  if (b_kmajor) {   // rows of B^T: one box per CTA and stage
    const uint64_t dims[2] = {(uint64_t)k, (uint64_t)n};
    const uint64_t strides[1] = {(uint64_t)ldb * eb};
    const uint32_t box[2] = {(uint32_t)row_k, (uint32_t)(cfg.pair ? 128 : cfg.block_n)};
    if (int rc = encode_tensor_map(&tb, b, eb, 2, dims, strides, box)) return rc;
  } else {
    const uint64_t dims[2] = {(uint64_t)n, (uint64_t)k};
    const uint64_t strides[1] = {(uint64_t)ldb * eb};
    const uint32_t box[2] = {(uint32_t)row_k, (uint32_t)row_k};
    if (int rc = encode_tensor_map(&tb, b, eb, 2, dims, strides, box)) return rc;
  }

  GemmParams p;
  p.c = c;
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.m_blocks = (int)cdiv64(m, kBlockM);
  p.n_blocks = (int)cdiv64(n, cfg.block_n);
  p.k_blocks = (int)cdiv64(k, row_k);
  const int mma_m = cfg.pair ? 2 * kBlockM : kBlockM;
  p.idesc = dtype == NB200_F32
                ? sm100::instr_desc_tf32(mma_m, cfg.block_n, false, false)
                : sm100::instr_desc_f16(mma_m, cfg.block_n, dtype == NB200_BF16, false, !b_kmajor);
  p.b_kmajor = b_kmajor ? 1 : 0;
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(c) & 15) == 0 && (ldc * cb) % 16 == 0) ? 1 : 0;
  p.c_f32 = c_f32 ? 1 : 0;
  p.wait_limit_ns = wait_limit_ns();
  p.status = device_status_ptr();
  if (!p.status) return fail(NB200_E_CUDA, "gemm: device status word is not addressable");

  if (cfg.pair) {
    if (cfg.block_k == 2 * row_k) return launch_pair<3, 2>(ta, tb, p, dtype, stream);
    if (cfg.block_k == 3 * row_k) return launch_pair<2, 3>(ta, tb, p, dtype, stream);
    switch (cfg.stages) {
      case 4: return launch_pair<4, 1>(ta, tb, p, dtype, stream);
      case 5: return launch_pair<5, 1>(ta, tb, p, dtype, stream);
      case 6: return launch_pair<6, 1>(ta, tb, p, dtype, stream);
      default: return launch_pair<7, 1>(ta, tb, p, dtype, stream);
    }
  }
  const int64_t tiles = (int64_t)p.m_blocks * p.n_blocks;
  const int sms = device_info().sm_count;
  const int grid = (int)(tiles < sms ? tiles : sms);

#define NB200_GEMM_CASE(BN_, ST_) \
  if (cfg.block_n == BN_ && cfg.stages == ST_) return launch<BN_, ST_>(ta, tb, p, dtype, grid, stream);
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

// B [K, N] -> workspace [N, pitch]; then the K-major GEMM.
int gemm_tf32_via(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int64_t lda,
                  int64_t ldb, int64_t ldc, const nb200_gemm_config* config, void* workspace,
                  cudaStream_t stream) {
  if (m < 0 || n < 0 || k < 0) return fail(NB200_E_INVALID, "gemm: negative extent");
  if (n > INT32_MAX || k > INT32_MAX) return fail(NB200_E_INVALID, "gemm: extent beyond int32");
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

extern "C" int nb200_gemm_acc32(const void* a, const void* b, float* c, int64_t m, int64_t n,
                                int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                                int b_transposed, const nb200_gemm_config* config, void* stream) {
  if (dtype != NB200_F16 && dtype != NB200_BF16)
    return fail(NB200_E_UNSUPPORTED, "gemm_acc32: fp16 or bf16 operands (fp32 ones already give an "
                                     "fp32 result through nb200_gemm_tf32 / nb200_gemm_bt)");
  return gemm_impl(a, b, c, m, n, k, lda, ldb, ldc, dtype, config, b_transposed != 0,
                   static_cast<cudaStream_t>(stream), true);
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
