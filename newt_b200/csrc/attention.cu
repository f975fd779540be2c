// Fused attention forward on tcgen05 (K5):  O = softmax(scale * Q K^T [+ causal]) V.
//
// The program being replaced is the flash-style loop of
// examples/05_fused_attention.py:14-48 -- per Q tile, walk the KV blocks keeping a
// running row maximum m_i, a running row sum l_i and an fp32 output accumulator;
// P is rounded to the input type before the PV product (:43).  In the reference
// both dots are staged synchronously and the accumulator round-trips through
// shared memory every iteration (newt/compiler/codegen.py:1824-1852, 719-776).
//
// Here one CTA owns a 128-row Q tile of one (batch, head):
//   warp 0      TMA producer: Q once, then K and V blocks of 128 rows into two rings
//   warp 1      MMA issuer:   S_j = Q K_j^T (Q read from tensor memory, where the softmax
//               warps copy it once; K from shared memory; S in tensor memory) and
//               O += P_j V_j (P read from tensor memory, V from shared memory as an
//               MN-major operand, so no transpose of V is ever made)
//   warps 2..5  softmax: thread t owns row t of the tile -- a TMEM lane -- so row
//               max and row sum are plain register loops, no shuffles.  P_j is
//               written back over S_j as packed 16-bit pairs.
// S is double-buffered: Q K_{j+1}^T runs on the tensor core while the softmax
// warps work on S_j.  The output accumulator is only rescaled when the running
// maximum moves by more than 2^8 (the rescale is exact in effect: the final
// division by l_i undoes whatever reference point the exponentials used).
// Scores are kept in the log2 domain: p = 2^(s * scale * log2(e) - m).
//
// Causal tiles skip the KV blocks above the diagonal and mask only the diagonal
// block.  Tensor-bound; flop per launch = 4 * BH * Sq * Skv * D (halved if causal).

#include <type_traits>

#include "sm100.cuh"

namespace nb200 {
namespace {

using namespace sm100;

constexpr int kTileM = 128;   // Q rows per CTA = TMEM lanes
constexpr int kTileN = 128;   // KV rows per block
constexpr int kThreads = 192;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnParams {
  void* o;
  long long o_head_stride, o_row_stride;
  int bh, seq_q, seq_kv, n_q_tiles;
  float scale_log2;  // scale * log2(e)
  int causal;
  uint32_t idesc_qk, idesc_pv;
  unsigned int* status;
};

enum : unsigned int {
  ST_ATTN_Q = 16, ST_ATTN_K_FULL, ST_ATTN_K_EMPTY, ST_ATTN_V_FULL, ST_ATTN_V_EMPTY,
  ST_ATTN_S_FULL, ST_ATTN_P_FULL, ST_ATTN_PV_DONE
};

template <int D, int STAGES, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  constexpr int kChunks = D / 64;                       // 64-element (128-byte) column chunks
  constexpr uint32_t kChunkBytes = 128 * 128;           // 128 rows x 128 B
  constexpr uint32_t kTileBytes = kChunks * kChunkBytes;  // one Q, K or V tile
  constexpr uint32_t kSCol0 = 0, kSCol1 = kTileN, kOCol = 2 * kTileN;
  constexpr uint32_t kQCol = kOCol + kTileN;   // Q as packed 16-bit pairs: D / 2 columns
  constexpr uint32_t kTmemCols = 512;
  // block j uses S buffer j % 2 for the (j / 2)-th time
  auto buf_of = [](int j) { return j & 1; };
  auto par_of = [](int j) { return uint32_t((j >> 1) & 1); };

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  __shared__ uint64_t s_full[2], p_full[2], pv_done[2], q_tmem_full;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + kTileBytes;
  const uint32_t v_smem = k_smem + STAGES * kTileBytes;
  const WaitCtx ctx{&abort_flag, p.status};

  // heaviest causal tiles of a head first; tiles of one head are adjacent so its K/V stay in L2
  const int head = blockIdx.x / p.n_q_tiles;
  const int q_tile = p.n_q_tiles - 1 - (blockIdx.x % p.n_q_tiles);
  const int q0 = q_tile * kTileM;
  int kv_end = p.seq_kv;
  if (p.causal) kv_end = min(kv_end, q0 + kTileM);
  const int n_blocks = (kv_end + kTileN - 1) / kTileN;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    mbar_init(smem_u32(&q_tmem_full), 4);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_full[b]), 1);
      mbar_init(smem_u32(&p_full[b]), 4);   // one arrival per softmax warp
      mbar_init(smem_u32(&pv_done[b]), 1);
    }
    mbar_init_fence();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(&q_full), kTileBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c)
        tma_load_3d(q_smem + c * kChunkBytes, &tmap_q, c * 64, q0, head, smem_u32(&q_full));
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int slot = j % STAGES;
        const uint32_t par = (j / STAGES) & 1;
        ok = mbar_wait(smem_u32(&k_empty[slot]), par ^ 1, ctx, ST_ATTN_K_EMPTY, j);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&k_full[slot]), kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(k_smem + slot * kTileBytes + c * kChunkBytes, &tmap_k, c * 64, j * kTileN,
                      head, smem_u32(&k_full[slot]));
        ok = mbar_wait(smem_u32(&v_empty[slot]), par ^ 1, ctx, ST_ATTN_V_EMPTY, j);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&v_full[slot]), kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(v_smem + slot * kTileBytes + c * kChunkBytes, &tmap_v, c * 64, j * kTileN,
                      head, smem_u32(&v_full[slot]));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // Q and K tiles: K-major, rows of 128 B, 8-row groups 1024 B apart, one 16 KB chunk per
      // 64 columns of D.  V tile: MN-major, 64-column slabs kChunkBytes apart.
      constexpr uint64_t kKMajor = smem_desc_sw128(16, 1024);
      constexpr uint64_t kVDesc = smem_desc_sw128(kChunkBytes, 1024);
      // Q is read from tensor memory (copied there by the softmax warps): S = Q K^T then
      // costs shared-memory bandwidth for K only.  This kernel is bound by that bandwidth.
      bool ok = mbar_wait(smem_u32(&q_tmem_full), 0, ctx, ST_ATTN_Q, 0);
      if (ok) tc_fence_after_sync();

      auto issue_s = [&](int j) -> bool {
        const int slot = j % STAGES, buf = buf_of(j);
        if (!mbar_wait(smem_u32(&k_full[slot]), (j / STAGES) & 1, ctx, ST_ATTN_K_FULL, j))
          return false;
        // S buffer `buf` was last read (as P) by the PV product of block j-2.  That product was issued by this thread before this point and MMAs execute
        // in issue order, so no wait is needed -- and waiting for its completion here kept the
        // softmax warps idle for ~500 cycles per block.
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (buf ? kSCol1 : kSCol0);
        const uint32_t kb = k_smem + slot * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kChunkBytes + (kk % 4) * 32;
          mma_f16_ts(d_tmem, tmem_base + kQCol + kk * 8, with_address(kKMajor, kb + off),
                     p.idesc_qk, kk != 0 ? 1u : 0u);
        }
        mma_commit(smem_u32(&k_empty[slot]));
        mma_commit(smem_u32(&s_full[buf]));
        return true;
      };

      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) {
          ok = issue_s(j + 1);   // overlaps the softmax of block j
          if (!ok) break;
        }
        const int slot = j % STAGES, buf = buf_of(j);
        ok = mbar_wait(smem_u32(&p_full[buf]), par_of(j), ctx, ST_ATTN_P_FULL, j) &&
             mbar_wait(smem_u32(&v_full[slot]), (j / STAGES) & 1, ctx, ST_ATTN_V_FULL, j);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t p_tmem = tmem_base + (buf ? kSCol1 : kSCol0);
        const uint32_t vb = v_smem + slot * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kTileN / 16; ++kk) {
          // 16 K-elements of P = 8 packed columns; 16 KV rows of V = 2048 B
          mma_f16_ts(tmem_base + kOCol, p_tmem + kk * 8, with_address(kVDesc, vb + kk * 2048),
                     p.idesc_pv, (j | kk) != 0 ? 1u : 0u);
        }
        mma_commit(smem_u32(&v_empty[slot]));
        mma_commit(smem_u32(&pv_done[buf]));
      }
    }
  } else {
    // ---------------- softmax + epilogue: one thread per row ----------------
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int quarter = warp & 3;
    const int row = q0 + quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const float c = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;

    // Q tile: shared memory (TMA layout: rows of 128 B, 16-byte units XOR-swizzled with the
    // row index) -> this thread's row of tensor memory, as the A operand of S = Q K^T
    ok = mbar_wait(smem_u32(&q_full), 0, ctx, ST_ATTN_Q, 1);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const int r = quarter * 32 + lane;
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        uint32_t qreg[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint32_t addr = q_smem + ch * kChunkBytes + r * 128 + ((u ^ (r & 7)) << 4);
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(qreg[4 * u]), "=r"(qreg[4 * u + 1]), "=r"(qreg[4 * u + 2]),
                         "=r"(qreg[4 * u + 3])
                       : "r"(addr));
        }
        tmem_st_32x32(tmem_base + lane_base + kQCol + ch * 32, qreg);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&q_tmem_full));
    }

    for (int j = 0; j < n_blocks && ok; ++j) {
      const int buf = buf_of(j);
      ok = mbar_wait(smem_u32(&s_full[buf]), par_of(j), ctx, ST_ATTN_S_FULL, j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + lane_base + (buf ? kSCol1 : kSCol0);
      uint32_t s[4][32];
#pragma unroll
      for (int q = 0; q < 4; ++q) tmem_ld_32x32(s_tmem + q * 32, s[q]);
      tmem_ld_wait();

      const int kv0 = j * kTileN;
      const bool edge = (p.causal && kv0 + kTileN - 1 > q0) || (kv0 + kTileN > p.seq_kv);
      if (edge) {
        const int limit = p.causal ? min(row, p.seq_kv - 1) : p.seq_kv - 1;  // last visible column
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv0 + q * 32 + i > limit) s[q][i] = __float_as_uint(-INFINITY);
      }
      // four independent chains of three-input maxima: the row maximum in 16 dependent steps
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(s[q][i]),
                                   __uint_as_float(s[q][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_run, mx * c);
      // rows past seq_q (and nothing else) can be fully masked; keep them finite
      const bool need = (m_new - m_run > kRescaleThreshold) && (m_new > -INFINITY);
      if (j == 0) {
        if (need) m_run = m_new;
      } else if (__any_sync(0xffffffffu, need)) {
        float alpha = 1.0f;
        if (need) {
          alpha = exp2_approx(m_run - m_new);
          m_run = m_new;
          l_run *= alpha;
        }
        // O holds the products up to block j-1: wait for that PV to retire, then rescale
        const int pb = buf_of(j - 1);
        ok = mbar_wait(smem_u32(&pv_done[pb]), par_of(j - 1), ctx, ST_ATTN_PV_DONE, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int q = 0; q < D / 32; ++q) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + lane_base + kOCol + q * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem_base + lane_base + kOCol + q * 32, o);
        }
      }
      const float m_use = m_run > -INFINITY ? m_run : 0.0f;
      // two scores per fma / add (packed fp32), four partial sums
      const unsigned long long c2 = pack2(c, c), negm2 = pack2(-m_use, -m_use);
      unsigned long long sum2[2] = {0ull, 0ull};
#pragma unroll
      for (int h = 0; h < 2; ++h) {   // 64 scores -> 32 packed columns per store
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float a = __uint_as_float(s[2 * h + i / 16][(2 * i) % 32]);
          const float b = __uint_as_float(s[2 * h + i / 16][(2 * i) % 32 + 1]);
          float ta, tb;
          unpack2(fma2(pack2(a, b), c2, negm2), ta, tb);
          const float pa = exp2_approx(ta);
          const float pb2 = exp2_approx(tb);
          sum2[i & 1] = add2(sum2[i & 1], pack2(pa, pb2));
          if constexpr (BF16) {
            __nv_bfloat162 v = __floats2bfloat162_rn(pa, pb2);
            pk[i] = *reinterpret_cast<uint32_t*>(&v);
          } else {
            __half2 v = __floats2half2_rn(pa, pb2);
            pk[i] = *reinterpret_cast<uint32_t*>(&v);
          }
        }
        tmem_st_32x32(s_tmem + h * 32, pk);
      }
      float s0, s1, s2, s3;
      unpack2(sum2[0], s0, s1);
      unpack2(sum2[1], s2, s3);
      l_run += (s0 + s1) + (s2 + s3);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[buf]));
    }

    if (ok && n_blocks > 0) {
      const int lb = buf_of(n_blocks - 1);
      ok = mbar_wait(smem_u32(&pv_done[lb]), par_of(n_blocks - 1), ctx, ST_ATTN_PV_DONE,
                     n_blocks);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && n_blocks > 0) {
      tc_fence_after_sync();
      const float inv = 1.0f / l_run;
      OutT* orow = static_cast<OutT*>(p.o) + (long long)head * p.o_head_stride +
                   (long long)row * p.o_row_stride;
      const bool vec = ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_base + kOCol + q * 32, o);
        tmem_ld_wait();
        if (row < p.seq_q) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float lo = __uint_as_float(o[g * 8 + 2 * h]) * inv;
              const float hi = __uint_as_float(o[g * 8 + 2 * h + 1]) * inv;
              if constexpr (BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            OutT* dst = orow + q * 32 + g * 8;
            if (vec) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              const OutT* e = reinterpret_cast<const OutT*>(packed);
#pragma unroll
              for (int t = 0; t < 8; ++t) dst[t] = e[t];
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let in-flight bulk copies land
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- two Q tiles per CTA ---------------------------------------------------------
//
// Same algorithm, scheduled for overlap: a CTA owns 256 query rows as two 128-row tiles
// X = 0, 1, each with its own S/P and O regions of tensor memory (4 x 128 columns) and its
// own group of four softmax warps.  The MMA warp interleaves the two tiles,
//     S_0(0) S_1(0) | PV_0(j) S_0(j+1) PV_1(j) S_1(j+1) | ...
// so while group 0 works on S_0(j+1) the tensor core runs PV_1(j) and S_1(j+1), and the two
// softmax groups (two warps per SM sub-partition) hide each other's latencies.  S_X(j+1) is
// issued right after PV_X(j): MMAs of one thread execute in order, so it cannot overtake the
// read of P_X(j) that shares its columns.  K and V blocks are loaded once for both tiles.
constexpr int kThreads2 = 320;   // TMA warp, MMA warp, 2 x 4 softmax warps

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads2, 1)
    attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q,
                     const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  constexpr int STAGES = 2;
  constexpr int kChunks = D / 64;
  constexpr uint32_t kChunkBytes = 128 * 128;
  constexpr uint32_t kTileBytes = kChunks * kChunkBytes;
  constexpr uint32_t kTmemCols = 512;
  // tensor memory: S/P of tile X at X*128, O of tile X at 256 + X*128

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  __shared__ uint64_t s_full[2], p_full[2], pv_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;                       // two Q tiles
  const uint32_t k_smem = q_smem + 2 * kTileBytes;
  const uint32_t v_smem = k_smem + STAGES * kTileBytes;
  const WaitCtx ctx{&abort_flag, p.status};

  const int n_q_pairs = (p.n_q_tiles + 1) / 2;
  const int head = blockIdx.x / n_q_pairs;
  const int q_pair = n_q_pairs - 1 - (blockIdx.x % n_q_pairs);   // heaviest causal work first
  const int q0 = q_pair * 2 * kTileM;
  // KV blocks each tile needs
  int nblk[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int qx = q0 + x * kTileM;
    int kv_end = p.seq_kv;
    if (p.causal) kv_end = min(kv_end, qx + kTileM);
    nblk[x] = qx < p.seq_q ? (kv_end + kTileN - 1) / kTileN : 0;
  }
  const int n_max = max(nblk[0], nblk[1]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
    }
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&s_full[x]), 1);
      mbar_init(smem_u32(&p_full[x]), 4);
      mbar_init(smem_u32(&pv_done[x]), 1);
    }
    mbar_init_fence();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == 1) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(&q_full), 2 * kTileBytes);   // rows past seq_q are zero-filled
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(q_smem + x * kTileBytes + c * kChunkBytes, &tmap_q, c * 64,
                      q0 + x * kTileM, head, smem_u32(&q_full));
      bool ok = true;
      for (int j = 0; j < n_max && ok; ++j) {
        const int slot = j % STAGES;
        const uint32_t par = (j / STAGES) & 1;
        ok = mbar_wait(smem_u32(&k_empty[slot]), par ^ 1, ctx, ST_ATTN_K_EMPTY, j);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&k_full[slot]), kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(k_smem + slot * kTileBytes + c * kChunkBytes, &tmap_k, c * 64, j * kTileN,
                      head, smem_u32(&k_full[slot]));
        ok = mbar_wait(smem_u32(&v_empty[slot]), par ^ 1, ctx, ST_ATTN_V_EMPTY, j);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&v_full[slot]), kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(v_smem + slot * kTileBytes + c * kChunkBytes, &tmap_v, c * 64, j * kTileN,
                      head, smem_u32(&v_full[slot]));
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint64_t kKMajor = smem_desc_sw128(16, 1024);
      constexpr uint64_t kVDesc = smem_desc_sw128(kChunkBytes, 1024);
      bool ok = mbar_wait(smem_u32(&q_full), 0, ctx, ST_ATTN_Q, 0);

      // S_x(j) = Q_x K_j^T into tile x's S columns; the caller has waited for K_j
      auto issue_s = [&](int x, int j) {
        const uint32_t kb = k_smem + (j % STAGES) * kTileBytes;
        const uint32_t qb = q_smem + x * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kChunkBytes + (kk % 4) * 32;
          mma_f16_ss(tmem_base + x * kTileN, with_address(kKMajor, qb + off),
                     with_address(kKMajor, kb + off), p.idesc_qk, kk != 0 ? 1u : 0u);
        }
        mma_commit(smem_u32(&s_full[x]));
      };

      if (ok && n_max > 0) {
        ok = mbar_wait(smem_u32(&k_full[0]), 0, ctx, ST_ATTN_K_FULL, 0);
        if (ok) {
          tc_fence_after_sync();
          if (nblk[0] > 0) issue_s(0, 0);
          if (nblk[1] > 0) issue_s(1, 0);
          mma_commit(smem_u32(&k_empty[0]));
        }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int slot = j % STAGES;
        const bool more = j + 1 < n_max;
        bool have_v = false, have_k = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (j >= nblk[x]) continue;
          ok = mbar_wait(smem_u32(&p_full[x]), j & 1, ctx, ST_ATTN_P_FULL, j);
          if (ok && !have_v) {
            ok = mbar_wait(smem_u32(&v_full[slot]), (j / STAGES) & 1, ctx, ST_ATTN_V_FULL, j);
            have_v = true;
          }
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t vb = v_smem + slot * kTileBytes;
#pragma unroll
          for (int kk = 0; kk < kTileN / 16; ++kk)
            mma_f16_ts(tmem_base + 2 * kTileN + x * kTileN, tmem_base + x * kTileN + kk * 8,
                       with_address(kVDesc, vb + kk * 2048), p.idesc_pv, (j | kk) != 0 ? 1u : 0u);
          mma_commit(smem_u32(&pv_done[x]));
          if (j + 1 < nblk[x]) {
            if (!have_k) {
              ok = mbar_wait(smem_u32(&k_full[(j + 1) % STAGES]), ((j + 1) / STAGES) & 1, ctx,
                             ST_ATTN_K_FULL, j + 1);
              have_k = true;
              if (!ok) break;
              tc_fence_after_sync();
            }
            issue_s(x, j + 1);   // ordered after PV_x(j), which reads the columns it overwrites
          }
        }
        if (!ok) break;
        mma_commit(smem_u32(&v_empty[slot]));
        if (more) mma_commit(smem_u32(&k_empty[(j + 1) % STAGES]));
      }
    }
  } else {
    // ---------------- softmax + epilogue: group x owns tile x, one thread per row ----------------
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int x = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int qx = q0 + x * kTileM;
    const int row = qx + quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + x * kTileN;
    const uint32_t o_tmem = tmem_base + lane_base + 2 * kTileN + x * kTileN;
    const int n_blocks = nblk[x];
    const float c = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;

    for (int j = 0; j < n_blocks; ++j) {
      ok = mbar_wait(smem_u32(&s_full[x]), j & 1, ctx, ST_ATTN_S_FULL, j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int kv0 = j * kTileN;
      const bool edge = (p.causal && kv0 + kTileN - 1 > qx) || (kv0 + kTileN > p.seq_kv);
      const int limit = p.causal ? min(row, p.seq_kv - 1) : p.seq_kv - 1;  // last visible column

      // pass 1: row maximum, 64 columns at a time
      float mx = -INFINITY;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t s[2][32];
        tmem_ld_32x32(s_tmem + h * 64, s[0]);
        tmem_ld_32x32(s_tmem + h * 64 + 32, s[1]);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(s[q][i]);
            if (edge && kv0 + h * 64 + q * 32 + i > limit) v = -INFINITY;
            mx = fmaxf(mx, v);
          }
      }
      const float m_new = fmaxf(m_run, mx * c);
      const bool need = (m_new - m_run > kRescaleThreshold) && (m_new > -INFINITY);
      if (j == 0) {
        if (need) m_run = m_new;
      } else if (__any_sync(0xffffffffu, need)) {
        float alpha = 1.0f;
        if (need) {
          alpha = exp2_approx(m_run - m_new);
          m_run = m_new;
          l_run *= alpha;
        }
        ok = mbar_wait(smem_u32(&pv_done[x]), (j - 1) & 1, ctx, ST_ATTN_PV_DONE, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int q = 0; q < D / 32; ++q) {
          uint32_t o[32];
          tmem_ld_32x32(o_tmem + q * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(o_tmem + q * 32, o);
        }
      }
      const float m_use = m_run > -INFINITY ? m_run : 0.0f;

      // pass 2: exponentials, row sum, P written over the S columns already consumed
      float sum = 0.0f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t s[2][32];
        tmem_ld_32x32(s_tmem + h * 64, s[0]);
        tmem_ld_32x32(s_tmem + h * 64 + 32, s[1]);
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float a = __uint_as_float(s[i / 16][(2 * i) % 32]);
          float b = __uint_as_float(s[i / 16][(2 * i) % 32 + 1]);
          if (edge) {
            if (kv0 + h * 64 + 2 * i > limit) a = -INFINITY;
            if (kv0 + h * 64 + 2 * i + 1 > limit) b = -INFINITY;
          }
          const float pa = exp2_approx(fmaf(a, c, -m_use));
          const float pb = exp2_approx(fmaf(b, c, -m_use));
          sum += pa + pb;
          if constexpr (BF16) {
            __nv_bfloat162 v = __floats2bfloat162_rn(pa, pb);
            pk[i] = *reinterpret_cast<uint32_t*>(&v);
          } else {
            __half2 v = __floats2half2_rn(pa, pb);
            pk[i] = *reinterpret_cast<uint32_t*>(&v);
          }
        }
        tmem_st_32x32(s_tmem + h * 32, pk);
      }
      l_run += sum;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[x]));
    }

    if (ok && n_blocks > 0) {
      ok = mbar_wait(smem_u32(&pv_done[x]), (n_blocks - 1) & 1, ctx, ST_ATTN_PV_DONE, n_blocks);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && n_blocks > 0) {
      tc_fence_after_sync();
      const float inv = 1.0f / l_run;
      OutT* orow = static_cast<OutT*>(p.o) + (long long)head * p.o_head_stride +
                   (long long)row * p.o_row_stride;
      const bool vec = ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t o[32];
        tmem_ld_32x32(o_tmem + q * 32, o);
        tmem_ld_wait();
        if (row < p.seq_q) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float lo = __uint_as_float(o[g * 8 + 2 * h]) * inv;
              const float hi = __uint_as_float(o[g * 8 + 2 * h + 1]) * inv;
              if constexpr (BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            OutT* dst = orow + q * 32 + g * 8;
            if (vec) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              const OutT* e = reinterpret_cast<const OutT*>(packed);
#pragma unroll
              for (int t = 0; t < 8; ++t) dst[t] = e[t];
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ----------------------------------------------------------------------

template <int D, int STAGES>
int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                const AttnParams& p, bool bf16, cudaStream_t stream) {
  const int smem = (1 + 2 * STAGES) * (D / 64) * 128 * 128 + 1024;
  const int grid = p.bh * p.n_q_tiles;
  auto go = [&](auto kern) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_check(e, "attention smem attribute");
    kern<<<grid, kThreads, smem, stream>>>(tq, tk, tv, p);
    return cuda_check(cudaGetLastError(), "attention launch");
  };
  return bf16 ? go(attn_fwd_kernel<D, STAGES, true>) : go(attn_fwd_kernel<D, STAGES, false>);
}

template <int D>
int launch_attn2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                 const AttnParams& p, bool bf16, cudaStream_t stream) {
  const int smem = (2 + 2 * 2) * (D / 64) * 128 * 128 + 1024;   // two Q tiles, 2-deep K and V rings
  const int grid = p.bh * ((p.n_q_tiles + 1) / 2);
  auto go = [&](auto kern) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_check(e, "attention smem attribute");
    kern<<<grid, kThreads2, smem, stream>>>(tq, tk, tv, p);
    return cuda_check(cudaGetLastError(), "attention launch");
  };
  return bf16 ? go(attn_fwd2_kernel<D, true>) : go(attn_fwd2_kernel<D, false>);
}

int encode_qkv_map(CUtensorMap* map, const void* base, int64_t bh, int64_t seq, int64_t d,
                   int64_t head_stride, int64_t row_stride) {
  const uint64_t dims[3] = {(uint64_t)d, (uint64_t)seq, (uint64_t)bh};
  const uint64_t strides[2] = {(uint64_t)row_stride * 2, (uint64_t)head_stride * 2};
  const uint32_t box[3] = {64u, 128u, 1u};
  return encode_tensor_map_16bit(map, base, 3, dims, strides, box);
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" int nb200_attention_fwd(const void* q, const void* k, const void* v, void* o,
                                   int64_t batch_heads, int64_t seq_q, int64_t seq_kv, int64_t d,
                                   int64_t q_hs, int64_t q_rs, int64_t k_hs, int64_t k_rs,
                                   int64_t v_hs, int64_t v_rs, int64_t o_hs, int64_t o_rs,
                                   float scale, int causal, int dtype, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype != NB200_F16 && dtype != NB200_BF16)
    return fail(NB200_E_UNSUPPORTED, "attention: dtype code %d (fp16 and bf16 only)", dtype);
  if (batch_heads < 0 || seq_q < 0 || seq_kv < 0)
    return fail(NB200_E_INVALID, "attention: negative extent");
  if (d != 64 && d != 128)
    return fail(NB200_E_UNSUPPORTED, "attention: head_dim %lld (64 and 128 only)", (long long)d);
  if (batch_heads == 0 || seq_q == 0) return 0;
  if (seq_kv == 0)
    return fail(NB200_E_INVALID, "attention: empty key/value sequence (softmax of nothing)");
  if (!q || !k || !v || !o) return fail(NB200_E_INVALID, "attention: null tensor pointer");
  if (batch_heads > 65535LL * 1024 || seq_q > INT32_MAX || seq_kv > INT32_MAX)
    return fail(NB200_E_INVALID, "attention: extent too large");
  if (!(scale > 0.0f)) return fail(NB200_E_INVALID, "attention: scale must be positive");
  const void* ptrs[3] = {q, k, v};
  const int64_t strides[6] = {q_hs, q_rs, k_hs, k_rs, v_hs, v_rs};
  for (int i = 0; i < 3; ++i) {
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)
      return fail(NB200_E_UNSUPPORTED, "attention: Q, K and V must be 16-byte aligned for TMA");
    if (strides[2 * i] % 8 || strides[2 * i + 1] % 8 || strides[2 * i + 1] < d)
      return fail(NB200_E_UNSUPPORTED,
                  "attention: head and row strides of Q/K/V must be multiples of 8 elements");
  }

  CUtensorMap tq, tk, tv;
  if (int rc = encode_qkv_map(&tq, q, batch_heads, seq_q, d, q_hs, q_rs)) return rc;
  if (int rc = encode_qkv_map(&tk, k, batch_heads, seq_kv, d, k_hs, k_rs)) return rc;
  if (int rc = encode_qkv_map(&tv, v, batch_heads, seq_kv, d, v_hs, v_rs)) return rc;

  AttnParams p;
  p.o = o;
  p.o_head_stride = o_hs;
  p.o_row_stride = o_rs;
  p.bh = (int)batch_heads;
  p.seq_q = (int)seq_q;
  p.seq_kv = (int)seq_kv;
  p.n_q_tiles = (int)cdiv64(seq_q, kTileM);
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  const bool bf16 = dtype == NB200_BF16;
  p.idesc_qk = sm100::instr_desc_f16(kTileM, kTileN, bf16, false, false);
  p.idesc_pv = sm100::instr_desc_f16(kTileM, (int)d, bf16, false, true);
  p.status = device_status_ptr();
  if (!p.status) return fail(NB200_E_CUDA, "attention: device status word is not addressable");
  if ((int64_t)p.bh * p.n_q_tiles > INT32_MAX)
    return fail(NB200_E_INVALID, "attention: too many tiles for one launch");

  // "attn_variant" = 2 selects the two-tile kernel; the one-tile kernel is the default (it is
  // the faster of the two as measured so far)
  const int variant = tuning("attn_variant", 0);
  if (variant == 2) {
    if (d == 128) return launch_attn2<128>(tq, tk, tv, p, bf16, stream);
    return launch_attn2<64>(tq, tk, tv, p, bf16, stream);
  }
  const int stages = tuning("attn_stages", 0);
  if (d == 128) {
    if (stages == 3) return launch_attn<128, 3>(tq, tk, tv, p, bf16, stream);
    return launch_attn<128, 2>(tq, tk, tv, p, bf16, stream);
  }
  if (stages == 2) return launch_attn<64, 2>(tq, tk, tv, p, bf16, stream);
  return launch_attn<64, 3>(tq, tk, tv, p, bf16, stream);
}
