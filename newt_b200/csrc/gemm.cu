// C = A @ B for 16-bit inputs on the 5th-generation tensor cores (K3 / K4).
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
//     B is [K,N] row-major  -> MN-major operand (no transpose pass needed);
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
constexpr int kBlockK = 64;     // 64 16-bit elements = one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr int kGroupM = 8;      // row-blocks per L2 band of the tile order

struct GemmParams {
  void* c;
  long long ldc;
  int m, n, k;
  int m_blocks, n_blocks, k_blocks;
  uint32_t idesc;
  int c_vec_ok;  // C base and row pitch are 16-byte aligned
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

template <int BN, int STAGES, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  constexpr uint32_t kABytes = kBlockM * kBlockK * 2;   // 16 KB
  constexpr uint32_t kBSlab = kBlockK * 64 * 2;         // one 64-column slab of B: 8 KB
  constexpr uint32_t kBBytes = kBSlab * (BN / 64);
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators, BN fp32 columns each

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1 KB
  const WaitCtx ctx{&abort_flag, p.status};

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
          tma_load_2d(a_dst, &tmap_a, kb * kBlockK, mb * kBlockM, bar);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(a_dst + kABytes + j * kBSlab, &tmap_b, nb * BN + j * 64, kb * kBlockK,
                        bar);
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
          const uint64_t b_desc = with_address(kBDesc, a_addr + kABytes);
#pragma unroll
          for (int kk = 0; kk < kBlockK / 16; ++kk) {
            // +32 B along K inside A's swizzle row; +16 K-rows (2048 B) inside B's slab
            if (elected)
              mma_f16_ss(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 128),
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
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
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
#pragma unroll
          for (int g = 0; g < 4; ++g) {  // 8 columns = 16 bytes per group
            const int col = col0 + g * 8;
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float lo = __uint_as_float(r[g * 8 + 2 * h]);
              const float hi = __uint_as_float(r[g * 8 + 2 * h + 1]);
              if constexpr (BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            if (p.c_vec_ok && col + 8 <= p.n) {
              *reinterpret_cast<uint4*>(crow + col) =
                  make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              const OutT* e = reinterpret_cast<const OutT*>(packed);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (col + j < p.n) crow[col + j] = e[j];
            }
          }
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
template <int STAGES, int KSUB, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  constexpr int BN = 256;                                // cluster tile width
  constexpr uint32_t kABytes = kBlockM * kBlockK * 2;    // this CTA's 128 rows of A: 16 KB
  constexpr uint32_t kBSlab = kBlockK * 64 * 2;          // 64 columns of B: 8 KB
  constexpr uint32_t kBBytes = kBSlab * 2;               // this CTA's 128 columns of B
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
  const WaitCtx ctx{&abort_flag, p.status};

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
            const int k0 = (kb * KSUB + sub) * kBlockK;
            tma_load_2d_pair(a_dst, &tmap_a, k0, row0, bar);
            tma_load_2d_pair(a_dst + kABytes, &tmap_b, col0, k0, bar);
            tma_load_2d_pair(a_dst + kABytes + kBSlab, &tmap_b, col0 + 64, k0, bar);
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
            const uint64_t b_desc = with_address(kBDesc, a_addr + kABytes);
#pragma unroll
            for (int kk = 0; kk < kBlockK / 16; ++kk)
              if (elected)
                mma_f16_ss_pair(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 128),
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
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
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
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float lo = __uint_as_float(r[g * 8 + 2 * h]);
              const float hi = __uint_as_float(r[g * 8 + 2 * h + 1]);
              if constexpr (BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            if (p.c_vec_ok && col + 8 <= p.n) {
              *reinterpret_cast<uint4*>(crow + col) =
                  make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              const OutT* e = reinterpret_cast<const OutT*>(packed);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (col + j < p.n) crow[col + j] = e[j];
            }
          }
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

int smem_bytes_for(int block_n, int stages) {
  return stages * (kBlockM * kBlockK * 2 + kBlockK * block_n * 2) + 1024;
}

int resolve_config(const nb200_gemm_config* cfg, int64_t m, int64_t n, Resolved* out) {
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
                  "block_k=%d: a CTA-pair ring slot holds 64, 128 or 192 elements of K", bk);
    out->block_k = bk == 0 ? 2 * kBlockK : bk;
    if (stages != 0 && (stages < 1 || stages > 8))
      return fail(NB200_E_INVALID, "stages=%d: supported 1..8", stages);
    out->block_n = 256;
    // ring depth: 3 slots of 128 K-elements, 2 of 192, 4..7 of 64
    out->stages = out->block_k == 128 ? 3 : (out->block_k == 192 ? 2 :
                  (stages == 0 ? 6 : (stages >= 7 ? 7 : (stages >= 6 ? 6 : (stages >= 5 ? 5 : 4)))));
    return 0;
  }
  if (bm != 0 && bm != kBlockM)
    return fail(NB200_E_INVALID, "block_m=%d: MMA tiles are 128 rows (256 for a CTA pair)", bm);
  if (bk != 0 && bk != kBlockK)
    return fail(NB200_E_INVALID, "block_k=%d: the TMA ring moves 64-element K slabs", bk);
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
                  int64_t lda, int64_t ldb, int64_t ldc, int dtype) {
  if (dtype != NB200_F16 && dtype != NB200_BF16)
    return fail(NB200_E_UNSUPPORTED, "gemm: dtype code %d (fp16 and bf16 only)", dtype);
  if (m < 0 || n < 0 || k < 0) return fail(NB200_E_INVALID, "gemm: negative extent");
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX)
    return fail(NB200_E_INVALID, "gemm: extent beyond int32");
  if (m == 0 || n == 0) return 0;
  if (!c || (k > 0 && (!a || !b))) return fail(NB200_E_INVALID, "gemm: null tensor pointer");
  if (k == 0) return 0;  // C is cleared; A and B are never read
  if (lda < k || ldb < n || ldc < n)
    return fail(NB200_E_INVALID, "gemm: row stride smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                (long long)lda, (long long)ldb, (long long)ldc);
  // TMA: 16-byte aligned base and row pitch
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15))
    return fail(NB200_E_UNSUPPORTED, "gemm: A and B must be 16-byte aligned for TMA");
  if ((lda * 2) % 16 || (ldb * 2) % 16)
    return fail(NB200_E_UNSUPPORTED,
                "gemm: row pitch of A (%lld) and B (%lld) elements must be a multiple of 8 for TMA",
                (long long)lda, (long long)ldb);
  return 0;
}

template <int BN, int STAGES>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, bool bf16, int grid,
           cudaStream_t stream) {
  const int smem = smem_bytes_for(BN, STAGES);
  auto set = [&](auto kern) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  };
  if (bf16) {
    auto kern = gemm_kernel<BN, STAGES, true>;
    if (cudaError_t e = set(kern)) return cuda_check(e, "gemm smem attribute");
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  } else {
    auto kern = gemm_kernel<BN, STAGES, false>;
    if (cudaError_t e = set(kern)) return cuda_check(e, "gemm smem attribute");
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, p);
  }
  return cuda_check(cudaGetLastError(), "gemm launch");
}

template <int STAGES, int KSUB>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, bool bf16,
                cudaStream_t stream) {
  const int smem = STAGES * KSUB * (kBlockM * kBlockK * 2 + kBlockK * 128 * 2) + 1024;
  const void* kern = bf16 ? (const void*)gemm_pair_kernel<STAGES, KSUB, true>
                          : (const void*)gemm_pair_kernel<STAGES, KSUB, false>;
  if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))
    return cuda_check(e, "gemm pair smem attribute");
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
  if (cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, kern, &lc))
    return cuda_check(e, "cluster occupancy query");
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
  // the 16-bit payload is moved as raw bits; the element type only sets the size
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, (cuuint32_t)rank,
                      const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(NB200_E_INVALID, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_gemm_check(const void* a, const void* b, const void* c, int64_t m, int64_t n,
                                int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                                const nb200_gemm_config* config) {
  if (int rc = check_problem(a, b, c, m, n, k, lda, ldb, ldc, dtype)) return rc;
  Resolved r;
  return resolve_config(config, m, n, &r);
}

extern "C" int nb200_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                          int64_t lda, int64_t ldb, int64_t ldc, int dtype,
                          const nb200_gemm_config* config, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (int rc = check_problem(a, b, c, m, n, k, lda, ldb, ldc, dtype)) return rc;
  Resolved cfg;
  if (int rc = resolve_config(config, m, n, &cfg)) return rc;
  if (m == 0 || n == 0) return 0;
  if (k == 0)  // empty reduction: the accumulator is its zero initial value
    return cuda_check(cudaMemset2DAsync(c, (size_t)ldc * 2, 0, (size_t)n * 2, (size_t)m, stream),
                      "gemm k=0 clear");

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {(uint64_t)k, (uint64_t)m};
    const uint64_t strides[1] = {(uint64_t)lda * 2};
    const uint32_t box[2] = {(uint32_t)kBlockK, (uint32_t)kBlockM};
    if (int rc = encode_tensor_map_16bit(&ta, a, 2, dims, strides, box)) return rc;
  }
  {
    const uint64_t dims[2] = {(uint64_t)n, (uint64_t)k};
    const uint64_t strides[1] = {(uint64_t)ldb * 2};
    const uint32_t box[2] = {64u, (uint32_t)kBlockK};
    if (int rc = encode_tensor_map_16bit(&tb, b, 2, dims, strides, box)) return rc;
  }

  GemmParams p;
  p.c = c;
  p.ldc = ldc;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.m_blocks = (int)cdiv64(m, kBlockM);
  p.n_blocks = (int)cdiv64(n, cfg.block_n);
  p.k_blocks = (int)cdiv64(k, kBlockK);
  const bool bf16 = dtype == NB200_BF16;
  p.idesc = sm100::instr_desc_f16(cfg.pair ? 2 * kBlockM : kBlockM, cfg.block_n, bf16, false, true);
  p.c_vec_ok = ((reinterpret_cast<uintptr_t>(c) & 15) == 0 && (ldc * 2) % 16 == 0) ? 1 : 0;
  p.status = device_status_ptr();
  if (!p.status) return fail(NB200_E_CUDA, "gemm: device status word is not addressable");

  if (cfg.pair) {
    if (cfg.block_k == 128) return launch_pair<3, 2>(ta, tb, p, bf16, stream);
    if (cfg.block_k == 192) return launch_pair<2, 3>(ta, tb, p, bf16, stream);
    switch (cfg.stages) {
      case 4: return launch_pair<4, 1>(ta, tb, p, bf16, stream);
      case 5: return launch_pair<5, 1>(ta, tb, p, bf16, stream);
      case 6: return launch_pair<6, 1>(ta, tb, p, bf16, stream);
      default: return launch_pair<7, 1>(ta, tb, p, bf16, stream);
    }
  }
  const int64_t tiles = (int64_t)p.m_blocks * p.n_blocks;
  const int sms = device_info().sm_count;
  const int grid = (int)(tiles < sms ? tiles : sms);

#define NB200_GEMM_CASE(BN_, ST_) \
  if (cfg.block_n == BN_ && cfg.stages == ST_) return launch<BN_, ST_>(ta, tb, p, bf16, grid, stream);
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
