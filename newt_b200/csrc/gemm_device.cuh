// Device side of C = A @ B on the 5th-generation tensor cores: the two kernels of gemm.cu as
// function templates, so that the same text is compiled ahead of time (nvcc, the plain product)
// and at run time (NVRTC, a kernel that brings code of its own to run on the accumulator before
// the store).  Nothing here needs a host header.
//
//   gemm_body<BN, STAGES, DT, CT, EPI>        one CTA per 128 x BN tile
//   gemm_pair_body<STAGES, KSUB, DT, CT, EPI>  a cluster of two CTAs per 256 x 256 tile
//
// DT: operand type code (NB200_F16 / BF16, or F32 run as tf32), CT: type code of C, EPI: the
// epilogue functor (NoEpilogue for the plain product).  Callers wrap a body in a __global__
// function with `__launch_bounds__(192, 1)` whose tensor maps are `__grid_constant__`.
#pragma once

#include "sm100.cuh"

namespace nb200 {
namespace gemm {

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
};
template <int DT> struct ElemType { using T = __half; };
template <> struct ElemType<NB200_F32> { using T = float; };
template <> struct ElemType<NB200_BF16> { using T = __nv_bfloat16; };
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
__device__ __forceinline__ void store_chunk(typename ElemType<DT>::T* crow, int col0, int n,
                                            bool vec_ok, const uint32_t (&r)[32]) {
  using OutT = typename ElemType<DT>::T;
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
template <class A, class B> struct std_is_same { static constexpr bool value = false; };
template <class A> struct std_is_same<A, A> { static constexpr bool value = true; };
constexpr int kThreads = 192;
constexpr int kGroupM = 16;     // row-blocks per L2 band of the tile order

// Time stamps of one CTA's roles, for development builds only (-DNB200_GEMM_TRACE; the shipped
// library and the kernels compiled at run time have none of this).
#ifdef NB200_GEMM_TRACE
__device__ long long g_gemm_trace[4][128][2];
#define GTRACE_DECL int gtrace_n = 0;
#define GTRACE(role, id, cond)                                               \
  if (blockIdx.x == NB200_GEMM_TRACE && (cond) && gtrace_n < 128) {          \
    g_gemm_trace[role][gtrace_n][0] = (id);                                  \
    g_gemm_trace[role][gtrace_n][1] = clock64();                             \
    ++gtrace_n;                                                              \
  }
#else
#define GTRACE_DECL
#define GTRACE(role, id, cond)
#endif

struct GemmParams {
  void* c;
  long long ldc;
  int m, n, k;
  int m_blocks, n_blocks, k_blocks;
  uint32_t idesc;
  int c_vec_ok;  // C base and row pitch are 16-byte aligned
  int b_kmajor;  // B is given transposed ([N, K], K contiguous)
  // One bulk copy costs its issuing thread over a hundred cycles whatever its size, so a ring
  // slot is filled with as few copies as the shapes allow.  wide_a / wide_b: the tensor map is
  // the 3-D view [K / row, rows, row] (K-major operands; needs K to be whole 128-byte rows) or
  // [N / slab, K, slab] (B as [K, N]; needs N to be whole slabs), and one copy brings every K
  // slab of the slot, or every column slab of B, at once.  Otherwise the maps are 2-D and the
  // slot is filled slab by slab, zero-filled at the ragged edges.
  int wide_a, wide_b;
  int group_m;   // row-blocks per L2 band of the tile order
  int half_tail; // 512-column tile: the last ring's worth of k rounds finishes columns 0..255 first
  unsigned long long wait_limit_ns;
  unsigned int* status;
  // Split tail (pair kernels): the last sk_tiles tiles are not handed out whole but cut along
  // K into sk_parts parts of sk_len k rounds, one part per cluster, so the last round of a
  // launch keeps the chip busy; a part leaves its fp32 partial sums in sk_ws and a second kernel
  // adds the parts up (see SplitTail).  0 = every tile whole.
  int sk_tiles, sk_parts, sk_len;
  float* sk_ws;             // a slot per cluster, a slot = one fp32 accumulator tile
  // C as a tensor map with boxes of 32 rows x 128 bytes under the 128-byte swizzle -- one pass of
  // one epilogue warp, laid out as `drain_rows` stages it -- when C can be written by the copy
  // engine (c_tma: 16-byte aligned base and pitch).  The kernel takes this struct as a
  // __grid_constant__ parameter, so the map is read where the launch put it.
  int c_tma;
  alignas(64) CUtensorMap tmap_c;
};

// What runs between the accumulator and the store, in two steps.  `fetch` gets the row and
// the first of 32 consecutive columns and reads whatever else the code needs there (a bias, a
// residual) into a `Staged`; it runs while the accumulator's read from tensor memory is in
// flight.  `apply` then gets those 32 columns of one row of the fp32 accumulator (row `row`,
// columns `col0`..`col0 + 31` of C; entries past the matrix edge are never stored) and may
// change them in place: a bias, an activation, a scaling -- the code a kernel has after its k
// loop (newt/compiler/codegen.py:1854-1871 keeps it in the same kernel too).  The plain product
// uses NoEpilogue; kernels compiled at run time bring their own functor and its argument struct.
struct NoEpilogueArgs {
  int unused;
};
struct NoEpilogue {
  using Args = NoEpilogueArgs;
  struct Staged {};
  static __device__ __forceinline__ void fetch(Staged&, int, int, const Args&) {}
  static __device__ __forceinline__ void apply(float (&)[32], const Staged&, int, int, const Args&) {}
};

// The order in which a cluster works through a launch: its whole tiles (tile = cluster,
// cluster + clusters, ... below the split ones), then at most one part of a split tile, as
// segments (tile, first k round, end k round).  The three roles of a CTA run the same sequence.
// Split tile t (of sk_tiles) is cut into sk_parts stretches of sk_len k rounds, the same
// stretches for every tile; part s of tile t goes to cluster s * sk_tiles + t, so the clusters
// that read the same rows of A or columns of B over the same stretch of K run side by side and
// share them in L2, as whole tiles of one round do.
struct SplitTail {
  int dp_tiles, clusters, k_rounds, sk_tiles, parts, len;
  int next_tile, cluster;
  bool part_taken;

  __device__ __forceinline__ SplitTail(const GemmParams& p, int num_tiles, int k_rounds_, int cluster_,
                                       int clusters_)
      : dp_tiles(num_tiles - p.sk_tiles), clusters(clusters_), k_rounds(k_rounds_), sk_tiles(p.sk_tiles),
        parts(p.sk_parts), len(p.sk_len), next_tile(cluster_), cluster(cluster_), part_taken(false) {}
  // Next segment; split = index of the tile among the split ones when the segment is a part of
  // one (its partial sums go to slot `cluster` of the workspace), else -1.
  __device__ __forceinline__ bool next(int* tile, int* kb0, int* kb1, int* split) {
    if (next_tile < dp_tiles) {
      *tile = next_tile;
      *kb0 = 0;
      *kb1 = k_rounds;
      *split = -1;
      next_tile += clusters;
      return true;
    }
    if (part_taken || cluster >= sk_tiles * parts) return false;
    part_taken = true;
    const int s = cluster / sk_tiles, t = cluster - s * sk_tiles;
    *tile = dp_tiles + t;
    *kb0 = s * len;
    *kb1 = min(k_rounds, (s + 1) * len);
    *split = t;
    return true;
  }
};

// A slot of the workspace is laid out [CTA of the pair][epilogue warp][column / 4][row] in
// 16-byte pieces, so a warp's accesses are whole 512-byte runs.
template <int COLS>
__device__ __forceinline__ void dump_rows(uint32_t t_row, float* dst, int lane) {
#pragma unroll 1
  for (int c0 = 0; c0 < COLS; c0 += 32) {
    uint32_t r[32];
    tmem_ld_cols<32>(t_row + c0, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      __stcg(reinterpret_cast<float4*>(dst + ((c0 / 4 + j) * 32 + lane) * 4),
             make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
  }
}

// The epilogue of one warp: its 32 rows (tensor-memory lanes) of a BN-column accumulator go
// to C.  A thread holds one row, so storing from registers would write 16 bytes to each of 32
// rows per instruction -- half-filled 32-byte sectors, which made the epilogue of a 128 x 256
// tile take ~4900 cycles.  Instead a pass of 128 bytes of C per row (64 columns of a 16-bit C,
// 32 of an fp32 C) is rounded and parked in one of this warp's two 4 KB areas of shared memory
// (16-byte pieces XOR-swizzled by the row: conflict-free, and the 128-byte swizzle of a tensor
// map).  From there the copy engine writes it to C (`tmap_c`; clipped at the edges of the
// matrix) while the warp works on the next pass in the other area; without a tensor map of C
// the warp writes four whole 128-byte rows per instruction itself.  Ragged edges of an
// unaligned C take the register path.
constexpr uint32_t kEpilogueStageBytes = 4 * 2 * 32 * 128;   // four epilogue warps, two staging areas each

template <int BN, int CT, class EPI>
__device__ __forceinline__ void drain_rows(uint32_t t_row, void* c, long long ldc, int row0,
                                           int col_base, int m, int n, bool vec_ok, uint32_t stage,
                                           int lane, const typename EPI::Args& ea,
                                           const CUtensorMap* tmap_c = nullptr, int* flip = nullptr) {
  using OutT = typename ElemType<CT>::T;
  constexpr int kPass = 128 / (int)sizeof(OutT);     // columns per pass
  constexpr int kPer16 = 16 / (int)sizeof(OutT);     // columns per 16-byte piece
  const int row = row0 + lane;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += kPass) {
    const int col0 = col_base + c0;
    if (col0 >= n) break;   // uniform across the warp
    uint32_t r[kPass];
    tmem_ld_cols<kPass>(t_row + c0, r);
    typename EPI::Staged staged[kPass / 32];
    if constexpr (!std_is_same<EPI, NoEpilogue>::value) {
#pragma unroll
      for (int q = 0; q < kPass / 32; ++q) EPI::fetch(staged[q], row, col0 + q * 32, ea);
    }
    tmem_ld_wait();
    if constexpr (!std_is_same<EPI, NoEpilogue>::value) {
#pragma unroll
      for (int q = 0; q < kPass / 32; ++q) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[q * 32 + j]);
        EPI::apply(v, staged[q], row, col0 + q * 32, ea);
#pragma unroll
        for (int j = 0; j < 32; ++j) r[q * 32 + j] = __float_as_uint(v[j]);
      }
    }
    if (tmap_c != nullptr || (vec_ok && col0 + kPass <= n)) {
      // With the copy engine doing the stores the warp's two staging areas take turns: the
      // engine drains one (an SM writes ~32 bytes per clock towards L2: ~650 cycles for the 16 KB
      // of a pass of the four warps) while the next pass is read, rounded and staged in the other.
      // (`flip` runs on over calls, so the areas alternate whatever the number of passes)
      const uint32_t area = tmap_c != nullptr ? stage + ((*flip)++ & 1) * 4096 : stage;
      if (tmap_c != nullptr) {   // ... once the copy before last has been read out of it
        if (lane == 0) bulk_wait_group_read<1>();
        __syncwarp();
      }
      const uint32_t mine = area + lane * 128;
#pragma unroll
      for (int pc = 0; pc < 8; ++pc) {
        uint32_t w[4];
        if constexpr (CT == NB200_F32) {
#pragma unroll
          for (int h = 0; h < 4; ++h) w[h] = r[pc * 4 + h];
        } else {
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const float lo = __uint_as_float(r[pc * 8 + 2 * h]);
            const float hi = __uint_as_float(r[pc * 8 + 2 * h + 1]);
            if constexpr (CT == NB200_BF16) {
              __nv_bfloat162 v2 = __floats2bfloat162_rn(lo, hi);
              w[h] = *reinterpret_cast<uint32_t*>(&v2);
            } else {
              __half2 v2 = __floats2half2_rn(lo, hi);
              w[h] = *reinterpret_cast<uint32_t*>(&v2);
            }
          }
        }
        st_shared_v4(mine + ((pc ^ (lane & 7)) << 4), w[0], w[1], w[2], w[3]);
      }
      if (tmap_c != nullptr) {
        // one copy of 32 rows x 128 bytes (clipped at the edges of C)
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < m) {
          tma_store_2d(tmap_c, area, col0, row0);
          bulk_commit_group();
        }
        continue;
      }
      __syncwarp();
      const int pc = lane & 7;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = i * 4 + (lane >> 3);
        uint32_t w0, w1, w2, w3;
        ld_shared_v4(area + rr * 128 + ((pc ^ (rr & 7)) << 4), w0, w1, w2, w3);
        if (row0 + rr < m)
          *reinterpret_cast<uint4*>(static_cast<OutT*>(c) + (long long)(row0 + rr) * ldc + col0 +
                                    pc * kPer16) = make_uint4(w0, w1, w2, w3);
      }
      __syncwarp();
    } else if (row < m) {
      OutT* crow = static_cast<OutT*>(c) + (long long)row * ldc;
#pragma unroll
      for (int q = 0; q < kPass / 32; ++q)
        store_chunk<CT>(crow, col0 + q * 32, n, vec_ok,
                        *reinterpret_cast<const uint32_t (*)[32]>(&r[q * 32]));
    }
  }
}

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int group_m,
                                            int* mb, int* nb) {
  // bands of group_m row-blocks; inside a band, column-blocks advance slowest
  const int band_tiles = group_m * n_blocks;
  const int band = tile / band_tiles;
  const int first_m = band * group_m;
  const int rows = min(group_m, m_blocks - first_m);
  const int in_band = tile - band * band_tiles;
  *mb = first_m + in_band % rows;
  *nb = in_band / rows;
}

// A ring slot holds KSUB slabs of K (a slab = one 128-byte row of K per row of A and per
// column of B): first A's KSUB slabs, 16 KB each; then B -- given as [N, K], its KSUB slabs
// like A's; given as [K, N], column slab after column slab, each with the K rows of all KSUB
// slabs one after the other.
template <int BN, int STAGES, int KSUB, int DT, int CT, class EPI>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                          const GemmParams& p, const typename EPI::Args& ea) {
  constexpr int kBK = Elem<DT>::kPerRow;                // K elements per slab
  constexpr int kSlab = Elem<DT>::kPerRow;              // columns of B per slab
  constexpr uint32_t kABytes = kBlockM * 128;           // 16 KB
  constexpr uint32_t kBSlab = kBK * 128;                // one slab of B: 8 KB (4 KB for tf32)
  constexpr uint32_t kBBytes = kBSlab * (BN / kSlab);
  constexpr uint32_t kStageBytes = KSUB * (kABytes + kBBytes);
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators, BN fp32 columns each

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1 KB
  const uint32_t epi_stage = smem_base + STAGES * kStageBytes;       // behind the ring
  const WaitCtx ctx{&abort_flag, p.status, p.wait_limit_ns};
  GTRACE_DECL
  GTRACE(0, 0, threadIdx.x == 0)      // kernel entered

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
    if (p.c_tma) prefetch_tensormap(&p.tmap_c);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  GTRACE(0, 1, threadIdx.x == 0)      // set up

  const int num_tiles = p.m_blocks * p.n_blocks;
  const int k_rounds = (p.k_blocks + KSUB - 1) / KSUB;
  // B as [K, N] is an MN-major operand: for 16-bit types under the plain 128-byte swizzle, for
  // tf32 under its 32-byte-atom form (see smem_desc_sw128_atom32).
  const bool b_kmajor = p.b_kmajor != 0;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, &mb, &nb);
        for (int kb = 0; kb < k_rounds; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, ctx, ST_WAIT_SMEM_EMPTY, tile);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + KSUB * kABytes;
          const int slab0 = kb * KSUB;
          mbar_arrive_expect_tx(bar, kStageBytes);
          if (KSUB > 1 && p.wide_a) {
            tma_load_3d(a_dst, &tmap_a, 0, mb * kBlockM, slab0, bar);
          } else {
#pragma unroll
            for (int sub = 0; sub < KSUB; ++sub)
              tma_load_2d(a_dst + sub * kABytes, &tmap_a, (slab0 + sub) * kBK, mb * kBlockM, bar);
          }
          if (b_kmajor) {   // BN rows of B^T, laid out like A
            if (KSUB > 1 && p.wide_b) {
              tma_load_3d(b_dst, &tmap_b, 0, nb * BN, slab0, bar);
            } else {
#pragma unroll
              for (int sub = 0; sub < KSUB; ++sub)
                tma_load_2d(b_dst + sub * kBBytes, &tmap_b, (slab0 + sub) * kBK, nb * BN, bar);
            }
          } else if (p.wide_b) {   // all column slabs of the tile, KSUB * 64 rows of K each
            tma_load_3d(b_dst, &tmap_b, 0, slab0 * kBK, nb * (BN / kSlab), bar);
          } else {
#pragma unroll
            for (int j = 0; j < BN / kSlab; ++j)
#pragma unroll
              for (int sub = 0; sub < KSUB; ++sub)
                tma_load_2d(b_dst + (j * KSUB + sub) * kBSlab, &tmap_b, nb * BN + j * kSlab,
                            (slab0 + sub) * kBK, bar);
          }
          GTRACE(0, 100 + kb, (kb & 7) == 0)     // copies of k block kb issued
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
      constexpr uint64_t kBDesc = DT == NB200_F32 ? smem_desc_sw128_atom32(KSUB * kBSlab, 512)
                                                  : smem_desc_sw128(KSUB * kBSlab, 1024);
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
        for (int kb = 0; kb < k_rounds; ++kb) {
          ok = wait_all(&full_bar[stage], phase, ST_WAIT_TMA_FULL, tile);
          if (!ok) break;
          tc_fence_after_sync();
          GTRACE(1, 100 + kb, elected && (kb & 7) == 0)  // k block kb landed
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint32_t b_addr = a_addr + KSUB * kABytes;
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const uint64_t a_desc = with_address(kADesc, a_addr + sub * kABytes);
            const uint64_t b_desc = b_kmajor ? with_address(kADesc, b_addr + sub * kBBytes)
                                             : with_address(kBDesc, b_addr + sub * kBSlab);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              // +32 B along K inside a K-major swizzle row; + a quarter of a slab's K rows
              // (128 B each) inside an MN-major slab of B
              if (elected)
                mma_ss<DT>(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * b_step),
                           p.idesc, (kb | sub | kk) != 0 ? 1u : 0u);
            }
          }
          if (elected) mma_commit(smem_u32(&empty_bar[stage]));  // slot reusable once these retire
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && elected) mma_commit(smem_u32(&acc_full_bar[buf]));
        GTRACE(1, 2, elected)           // last product issued
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const CUtensorMap* tmap_c = p.c_tma ? &p.tmap_c : nullptr;
    int flip = 0;   // which of the warp's two staging areas the next pass takes
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(tile, p.m_blocks, p.n_blocks, p.group_m, &mb, &nb);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(smem_u32(&acc_full_bar[buf]), acc_phase, ctx, ST_WAIT_ACC_FULL, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      GTRACE(2, 3, threadIdx.x == 64)   // accumulator complete
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN;
      drain_rows<BN, CT, EPI>(t_row, p.c, p.ldc, mb * kBlockM + quarter * 32, nb * BN, p.m, p.n,
                              p.c_vec_ok != 0, epi_stage + quarter * (2 * 32 * 128), lane, ea, tmap_c, &flip);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[buf]));
      GTRACE(2, 4, threadIdx.x == 64)   // tile stored
    }
    if (tmap_c != nullptr && lane == 0) bulk_wait_group_all();   // this thread's copies to C are done
  }

  __syncthreads();
  GTRACE(0, 5, threadIdx.x == 0)        // all roles done
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
template <int STAGES, int KSUB, int DT, int CT, class EPI, int NSUB = 1>
__device__ __forceinline__ void gemm_pair_body(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                               const GemmParams& p, const typename EPI::Args& ea) {
  constexpr int BN = 256 * NSUB;                         // cluster tile width: NSUB MMAs of 256 columns
  constexpr int kAccBufs = NSUB == 1 ? 2 : 1;            // a 512-column tile takes all of tensor memory
  constexpr int kBK = Elem<DT>::kPerRow;                 // K elements per 128-byte row
  constexpr int kSlab = Elem<DT>::kPerRow;               // columns of B per slab
  constexpr uint32_t kABytes = kBlockM * 128;            // this CTA's 128 rows of A: 16 KB
  constexpr uint32_t kBSlab = kBK * 128;                 // one slab of B: 8 KB (4 KB for tf32)
  constexpr uint32_t kBBytes = kBSlab * (128 / kSlab);   // this CTA's 128 columns of one MMA's B
  constexpr uint32_t kSlabBytes = kABytes + NSUB * kBBytes;   // 32 (48) KB per 64 elements of K
  constexpr uint32_t kStageBytes = KSUB * kSlabBytes;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full_bar[2], acc_empty_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_stage = smem_base + STAGES * kStageBytes;       // behind the ring
  const WaitCtx ctx{&abort_flag, p.status, p.wait_limit_ns};
  GTRACE_DECL
  GTRACE(0, 0, threadIdx.x == 0)      // kernel entered

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
    if (p.c_tma) prefetch_tensormap(&p.tmap_c);
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
  GTRACE(0, 1, threadIdx.x == 0)      // set up

  const bool b_kmajor = p.b_kmajor != 0;
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
      SplitTail seq(p, num_tiles, k_rounds, first, step);
      int tile, kb0, kb1, split;
      while (ok && seq.next(&tile, &kb0, &kb1, &split)) {
        int mb, nb;
        tile_coords(tile, m_blocks2, p.n_blocks, p.group_m, &mb, &nb);
        const int row0 = mb * 2 * kBlockM + rank * kBlockM;
        const int col0 = nb * BN + rank * 128;   // of the first MMA; the second is 256 further
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, ctx, ST_WAIT_SMEM_EMPTY, tile);
          if (!ok) break;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * kStageBytes);
          // A slot: this CTA's A rows for KSUB slabs of K, then its share of B.  Slabs past K
          // and rows or columns past the matrix are zero-filled by the tensor maps.
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + KSUB * kABytes;
          const int slab0 = kb * KSUB;
          if (p.wide_a) {
            tma_load_3d_pair(a_dst, &tmap_a, 0, row0, slab0, bar);
          } else {
#pragma unroll
            for (int sub = 0; sub < KSUB; ++sub)
              tma_load_2d_pair(a_dst + sub * kABytes, &tmap_a, (slab0 + sub) * kBK, row0, bar);
          }
#pragma unroll
          for (int h = 0; h < NSUB; ++h) {   // this CTA's 128 columns of each 256-column MMA
            const uint32_t bh_dst = b_dst + h * KSUB * kBBytes;
            const int colh = col0 + h * 256;
            if (b_kmajor) {   // 128 rows of B^T, laid out like A
              if (p.wide_b) {
                tma_load_3d_pair(bh_dst, &tmap_b, 0, colh, slab0, bar);
              } else {
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                  tma_load_2d_pair(bh_dst + sub * kBBytes, &tmap_b, (slab0 + sub) * kBK, colh, bar);
              }
            } else if (p.wide_b) {   // both column slabs, KSUB * 64 rows of K each
              tma_load_3d_pair(bh_dst, &tmap_b, 0, slab0 * kBK, colh / kSlab, bar);
            } else {
#pragma unroll
              for (int j = 0; j < 128 / kSlab; ++j)
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                  tma_load_2d_pair(bh_dst + (j * KSUB + sub) * kBSlab, &tmap_b, colh + j * kSlab,
                                   (slab0 + sub) * kBK, bar);
            }
          }
          GTRACE(0, 100 + kb, (kb & 7) == 0)     // copies of k round kb issued
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
      constexpr uint64_t kBDesc = DT == NB200_F32 ? smem_desc_sw128_atom32(KSUB * kBSlab, 512)
                                                  : smem_desc_sw128(KSUB * kBSlab, 1024);   // column slabs of B
      const uint32_t b_step = b_kmajor ? 2u : uint32_t(2 * kBK);   // descriptor units of 16 B per MMA
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      SplitTail seq(p, num_tiles, k_rounds, first, step);
      int tile, kb0, kb1, split;
      for (; ok && seq.next(&tile, &kb0, &kb1, &split); ++it) {
        // Two accumulators of 256 columns take turns (NSUB = 1); the one 512-column accumulator
        // of the wide tile is handed back in halves, acc_empty[h] for columns 256 h ..., so the
        // first MMAs of the next tile start while the epilogue still drains the other half.
        const int buf = kAccBufs == 2 ? (it & 1) : 0;
        const uint32_t acc_phase = kAccBufs == 2 ? ((it >> 1) & 1) : (it & 1);
        ok = wait_all(&acc_empty_bar[buf], acc_phase ^ 1, ST_WAIT_ACC_EMPTY, tile);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * 256;
        bool half1_free = NSUB == 1;
        // the MMAs of one 256-column half over the K slabs of one ring slot
        auto issue = [&](int h, int slot, bool first_round) {
          const uint32_t a_addr = smem_base + slot * kStageBytes;
          const uint32_t bh_addr = a_addr + KSUB * kABytes + h * KSUB * kBBytes;
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            // K-major operands: slab `sub` is a block of its own.  B as [K, N]: a column slab
            // holds the K rows of all KSUB slabs one after the other.
            const uint64_t a_desc = with_address(kADesc, a_addr + sub * kABytes);
            const uint64_t b_desc = b_kmajor ? with_address(kADesc, bh_addr + sub * kBBytes)
                                             : with_address(kBDesc, bh_addr + sub * kBSlab);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              if (elected)
                mma_ss_pair<DT>(d_tmem + h * 256, a_desc + (uint64_t)(kk * 2),
                                b_desc + (uint64_t)(kk * b_step), p.idesc,
                                (!first_round || (sub | kk) != 0) ? 1u : 0u);
          }
        };
        auto free_half1 = [&]() -> bool {
          if (!half1_free) {
            if (!wait_all(&acc_empty_bar[1], acc_phase ^ 1, ST_WAIT_ACC_EMPTY, tile)) return false;
            tc_fence_after_sync();
            half1_free = true;
          }
          return true;
        };
        // The wide tile has one accumulator, so the tensor core waits while the epilogue drains
        // columns 0..255 of the tile before (every pair stores at the same moment; ~4300 cycles).
        // The last ring's worth of k rounds is therefore issued half by half: columns 0..255 are
        // complete, and on their way out, while the MMAs of columns 256..511 still run.
        const int tail0 = (NSUB == 2 && p.half_tail) ? max(kb0, kb1 - STAGES) : kb1;
        // The same at the start of a tile, the other way round: columns 256..511 of the tile
        // before are the last to leave, so the first ring's worth of k rounds runs its columns
        // 0..255 first.
        const int head1 = (NSUB == 2 && p.half_tail > 1) ? min(kb0 + STAGES, tail0) : kb0;
        if constexpr (NSUB == 2) {
          if (head1 > kb0) {
            int st = stage;
            uint32_t ph = phase;
            for (int kb = kb0; kb < head1 && ok; ++kb) {
              ok = wait_all(&full_bar[st], ph, ST_WAIT_TMA_FULL, tile);
              if (!ok) break;
              tc_fence_after_sync();
              issue(0, st, kb == kb0);
              if (++st == STAGES) st = 0, ph ^= 1;
            }
            if (ok) ok = free_half1();
            for (int kb = kb0; kb < head1 && ok; ++kb) {
              issue(1, stage, kb == kb0);
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
            if (!ok) break;
          }
        }
        for (int kb = head1; kb < tail0; ++kb) {
          ok = wait_all(&full_bar[stage], phase, ST_WAIT_TMA_FULL, tile);
          if (!ok) break;
          tc_fence_after_sync();
          GTRACE(1, 100 + kb, elected && (kb & 7) == 0)  // k round kb landed
          issue(0, stage, kb == kb0);
          if constexpr (NSUB == 2) {
            ok = free_half1();
            if (!ok) break;
            issue(1, stage, kb == kb0);
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
        if constexpr (NSUB == 2) {
          if (ok && tail0 < kb1) {
            int st = stage;
            uint32_t ph = phase;
            for (int kb = tail0; kb < kb1 && ok; ++kb) {
              ok = wait_all(&full_bar[st], ph, ST_WAIT_TMA_FULL, tile);
              if (!ok) break;
              tc_fence_after_sync();
              issue(0, st, kb == kb0);
              if (++st == STAGES) st = 0, ph ^= 1;
            }
            if (ok && elected) {
              mma_commit_pair(acc_full0);
              mma_commit_pair(acc_full1);
            }
            __syncwarp();
            if (ok) ok = free_half1();
            for (int kb = tail0; kb < kb1 && ok; ++kb) {
              issue(1, stage, kb == kb0);
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
              mma_commit_pair(acc_full0 + 8);
              mma_commit_pair(acc_full1 + 8);
            }
          } else if (ok && elected) {   // both halves end together
            mma_commit_pair(acc_full0);
            mma_commit_pair(acc_full1);
            mma_commit_pair(acc_full0 + 8);
            mma_commit_pair(acc_full1 + 8);
          }
        } else if (ok && elected) {
          mma_commit_pair(acc_full0 + buf * 8);
          mma_commit_pair(acc_full1 + buf * 8);
        }
        GTRACE(1, 2, elected)           // last product issued
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 128 rows of the 256-row tile ----------------
    const int quarter = warp & 3;
    const CUtensorMap* tmap_c = p.c_tma ? &p.tmap_c : nullptr;
    int flip = 0;   // which of the warp's two staging areas the next pass takes
    int it = 0;
    bool ok = true;
    SplitTail seq(p, num_tiles, k_rounds, first, step);
    int tile, kb0, kb1, split;
    for (; ok && seq.next(&tile, &kb0, &kb1, &split); ++it) {
      int mb, nb;
      tile_coords(tile, m_blocks2, p.n_blocks, p.group_m, &mb, &nb);
      const int buf = kAccBufs == 2 ? (it & 1) : 0;
      const uint32_t acc_phase = kAccBufs == 2 ? ((it >> 1) & 1) : (it & 1);
      ok = mbar_wait(smem_u32(&acc_full_bar[buf]), acc_phase, ctx, ST_WAIT_ACC_FULL, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      GTRACE(2, 3, threadIdx.x == 64)   // accumulator complete (its columns 0..255 for a wide tile)
      // the second half of a wide tile's accumulator has a barrier of its own
      auto second_half = [&]() -> bool {
        bool there = mbar_wait(smem_u32(&acc_full_bar[1]), acc_phase, ctx, ST_WAIT_ACC_FULL, tile);
        there = __all_sync(0xffffffffu, there);
        if (there) tc_fence_after_sync();
        return there;
      };
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * 256;
      if (split >= 0) {
        // A part of a split tile: its fp32 partial sums go to this segment's slot and the
        // accumulator is handed back; split_reduce_kernel adds the parts up after this kernel.
        if constexpr (NSUB == 2) {
          ok = second_half();
          if (!ok) break;
        }
        dump_rows<BN>(t_row, p.sk_ws + first * (256LL * BN) + (long long)(rank * 4 + quarter) * (BN * 32),
                      lane);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (NSUB == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[0]), 0));
          mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[NSUB == 2 ? 1 : buf]), 0));
        }
        continue;
      }
      if constexpr (NSUB == 2) {
        drain_rows<256, CT, EPI>(t_row, p.c, p.ldc, mb * 2 * kBlockM + rank * kBlockM + quarter * 32,
                                 nb * BN, p.m, p.n, p.c_vec_ok != 0, epi_stage + quarter * (2 * 32 * 128),
                                 lane, ea, tmap_c, &flip);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[0]), 0));
        ok = second_half();
        if (!ok) break;
        drain_rows<256, CT, EPI>(t_row + 256, p.c, p.ldc,
                                 mb * 2 * kBlockM + rank * kBlockM + quarter * 32, nb * BN + 256, p.m,
                                 p.n, p.c_vec_ok != 0, epi_stage + quarter * (2 * 32 * 128), lane, ea, tmap_c, &flip);
      } else {
        drain_rows<BN, CT, EPI>(t_row, p.c, p.ldc, mb * 2 * kBlockM + rank * kBlockM + quarter * 32,
                                nb * BN, p.m, p.n, p.c_vec_ok != 0, epi_stage + quarter * (2 * 32 * 128),
                                lane, ea, tmap_c, &flip);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[NSUB == 2 ? 1 : buf]), 0));
      GTRACE(2, 4, threadIdx.x == 64)   // tile stored
    }
    if (tmap_c != nullptr && lane == 0) bulk_wait_group_all();   // this thread's copies to C are done
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  cluster_sync_all();   // nobody leaves while the other CTA may still touch its barriers or tiles
  GTRACE(0, 5, threadIdx.x == 0)        // all roles done
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}


}  // namespace gemm
}  // namespace nb200
