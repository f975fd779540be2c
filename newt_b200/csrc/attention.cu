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
//   warp 0      TMA producer: Q once, then K and V blocks of 128 rows into two rings of three
//   warp 1      issues S_j = Q K_j^T (operands in shared memory, S in tensor memory)
//   warp 2      issues O += P_j V_j (P read from tensor memory, V from shared memory as an
//               MN-major operand, so no transpose of V is ever made)
//   warps 3..6  softmax: thread t owns row t of the tile -- a TMEM lane -- so row max and
//               row sum are plain register loops, no shuffles.  P_j is written back over
//               S_j as packed 16-bit pairs.
// S is triple-buffered: S_{j+1} and S_{j+2} are computed while the softmax warps work on
// S_j, and each MMA warp's instruction stream (waits, eight MMAs, one commit per block)
// is shorter than the tensor core's time for the block.  Every commit serves two waiters:
// "S_j complete" also frees K slot j, "PV_j retired" also frees V slot j and S/P buffer j.
// The exponentials of a block use the reference maximum known before the block; the block's
// own maximum is taken in the same loop and moves the reference afterwards, and only when it
// is more than 2^8 above it (exact in effect: the final division by l_i undoes whatever
// reference point the exponentials used).
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
constexpr int kRing = 3;      // depth of the K ring, the V ring and the S/P buffers
constexpr int kWarpTma = 0, kWarpQK = 1, kWarpPV = 2;   // warps 3..6: softmax, one row per thread
constexpr int kThreads = 224;
constexpr float kRescaleThreshold = 8.0f;    // log2 units: move the reference before the next block
constexpr float kOverflowThreshold = 14.0f;  // log2 units: redo the block (2^14 still fits 16 bits)

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
  ST_ATTN_S_FULL, ST_ATTN_P_FULL, ST_ATTN_PV_DONE, ST_ATTN_LAYOUT
};

// What a CTA keeps in shared memory besides the tiles.
//   s_full[x]:  S of the block in slot x is complete (softmax may read it, K slot x is free)
//   p_full[x]:  P of that block is in tensor memory (one arrival per softmax warp)
//   pv_done[x]: its PV product has retired (V slot x and S/P buffer x are free, O is current)
struct AttnShared {
  uint64_t q_full, k_full[kRing], v_full[kRing];
  uint64_t s_full[kRing], p_full[kRing], pv_done[kRing];
  uint32_t tmem_slot;
  uint32_t abort_flag;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  constexpr int kChunks = D / 64;                       // 64-element (128-byte) column chunks
  constexpr uint32_t kChunkBytes = 128 * 128;           // 128 rows x 128 B
  constexpr uint32_t kTileBytes = kChunks * kChunkBytes;  // one Q, K or V tile
  // tensor memory: three S/P buffers of 128 columns and the output accumulator = 512 columns
  constexpr uint32_t kOCol = kRing * kTileN;
  constexpr uint32_t kTmemCols = 512;
  // block j uses slot j % 3 (of the K ring, the V ring and the S/P buffers) for the (j / 3)-th time
  auto slot_of = [](int j) { return j % kRing; };
  auto par_of = [](int j) { return uint32_t((j / kRing) & 1); };

  // Everything in shared memory is carved from the dynamic allocation (no static part, so
  // the 128-byte-swizzled tiles start on the 1024-byte boundary the allocation starts on):
  // Q tile, K ring, V ring, then the barriers and the exchange buffer.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  AttnShared& sh = *reinterpret_cast<AttnShared*>(smem_raw + (1 + 2 * kRing) * kTileBytes);
  uint64_t& q_full = sh.q_full;
  uint64_t* k_full = sh.k_full;
  uint64_t* v_full = sh.v_full;
  uint64_t* s_full = sh.s_full;
  uint64_t* p_full = sh.p_full;
  uint64_t* pv_done = sh.pv_done;
  volatile uint32_t& abort_flag = sh.abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_smem = smem_u32(smem_raw);
  const uint32_t k_smem = q_smem + kTileBytes;
  const uint32_t v_smem = k_smem + kRing * kTileBytes;
  const WaitCtx ctx{&sh.abort_flag, p.status};
  if (q_smem & 1023u) {   // the tiles would be misread; uniform over the CTA
    if (threadIdx.x == 0 && atomicCAS(&p.status[0], 0u, (unsigned)ST_ATTN_LAYOUT) == 0u)
      p.status[1] = q_smem;
    return;
  }

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
#pragma unroll
    for (int x = 0; x < kRing; ++x) {
      mbar_init(smem_u32(&k_full[x]), 1);
      mbar_init(smem_u32(&v_full[x]), 1);
      mbar_init(smem_u32(&s_full[x]), 1);
      mbar_init(smem_u32(&p_full[x]), 4);   // one arrival per softmax warp
      mbar_init(smem_u32(&pv_done[x]), 1);
    }
    mbar_init_fence();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == kWarpQK) {
    __syncwarp();
    tmem_alloc(smem_u32(&sh.tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh.tmem_slot;

  // a whole warp waits (so that its control flow stays uniform); false = give up
  auto wait_all = [&](uint64_t* bar, uint32_t parity, unsigned int code, int j) -> bool {
    return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, ctx, code, j));
  };
  // Q and K tiles: K-major, rows of 128 B, 8-row groups 1024 B apart, one 16 KB chunk per
  // 64 columns of D.  V tile: MN-major, 64-column slabs kChunkBytes apart.
  constexpr uint64_t kKMajor = smem_desc_sw128(16, 1024);
  constexpr uint64_t kVDesc = smem_desc_sw128(kChunkBytes, 1024);

  if (warp == kWarpTma) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(smem_u32(&q_full), kTileBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c)
        tma_load_3d(q_smem + c * kChunkBytes, &tmap_q, c * 64, q0, head, smem_u32(&q_full));
      // K slot x is free once the S product that read it is complete, V slot x once the PV
      // product is: the barriers the MMA warps commit to anyway.  K runs a whole ring ahead
      // of V because S = Q K^T is issued blocks before the PV product of the same block.
      auto load = [&](const CUtensorMap* map, uint32_t ring, uint64_t* free_bar, uint64_t* full_bar,
                      unsigned int code, int j) -> bool {
        const int x = slot_of(j);
        if (!mbar_wait(smem_u32(&free_bar[x]), par_of(j) ^ 1, ctx, code, j)) return false;
        mbar_arrive_expect_tx(smem_u32(&full_bar[x]), kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(ring + x * kTileBytes + c * kChunkBytes, map, c * 64, j * kTileN, head,
                      smem_u32(&full_bar[x]));
        return true;
      };
      bool ok = true;
      for (int j = 0; j < kRing && j < n_blocks && ok; ++j)
        ok = load(&tmap_k, k_smem, s_full, k_full, ST_ATTN_K_EMPTY, j);
      for (int j = 0; j < n_blocks && ok; ++j) {
        ok = load(&tmap_v, v_smem, pv_done, v_full, ST_ATTN_V_EMPTY, j);
        if (ok && j + kRing < n_blocks)
          ok = load(&tmap_k, k_smem, s_full, k_full, ST_ATTN_K_EMPTY, j + kRing);
      }
    }
  } else if (warp == kWarpQK) {
    // ---------------- issuer of S_j = Q K_j^T ----------------
    // The whole warp walks the loop and waits; one elected lane issues, so addresses and
    // descriptors stay in uniform registers.  Two issuing warps (this one and the PV warp)
    // because one thread's instruction stream -- waits, sixteen MMAs and the commits of a
    // block -- took longer than the tensor core needs for the block.
    const bool elected = elect_one();
    bool ok = wait_all(&q_full, 0, ST_ATTN_Q, 0);
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int x = slot_of(j);
      // S/P buffer x was read (as P) by the PV product of block j-3
      ok = wait_all(&pv_done[x], par_of(j) ^ 1, ST_ATTN_PV_DONE, j) &&
           wait_all(&k_full[x], par_of(j), ST_ATTN_K_FULL, j);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + x * kTileN;
      const uint32_t kb = k_smem + x * kTileBytes;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk / 4) * kChunkBytes + (kk % 4) * 32;
        const uint64_t qd = with_address(kKMajor, q_smem + off);
        const uint64_t kd = with_address(kKMajor, kb + off);
        if (elected) mma_f16_ss(d_tmem, qd, kd, p.idesc_qk, kk != 0 ? 1u : 0u);
      }
      if (elected) mma_commit(smem_u32(&s_full[x]));
      __syncwarp();
    }
  } else if (warp == kWarpPV) {
    // ---------------- issuer of O += P_j V_j ----------------
    const bool elected = elect_one();
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int x = slot_of(j);
      ok = wait_all(&v_full[x], par_of(j), ST_ATTN_V_FULL, j) &&
           wait_all(&p_full[x], par_of(j), ST_ATTN_P_FULL, j);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t p_tmem = tmem_base + x * kTileN;
      const uint32_t vb = v_smem + x * kTileBytes;
#pragma unroll
      for (int kk = 0; kk < kTileN / 16; ++kk) {
        // 16 K-elements of P = 8 packed columns; 16 KV rows of V = 2048 B
        const uint64_t vd = with_address(kVDesc, vb + kk * 2048);
        if (elected)
          mma_f16_ts(tmem_base + kOCol, p_tmem + kk * 8, vd, p.idesc_pv, (j | kk) != 0 ? 1u : 0u);
      }
      if (elected) mma_commit(smem_u32(&pv_done[x]));
      __syncwarp();
    }
  } else {
    // ---------------- softmax + epilogue: one thread per row ----------------
    // Thread t of the four warps owns row t of the tile -- a TMEM lane -- so row maximum and
    // row sum are register loops.  The exponentials of a block use the reference maximum
    // m_run known before the block; the block's own maximum is taken in the same loop (ALU
    // work in the shadow of the special-function unit, which is the unit that bounds this
    // loop) and acts afterwards:
    //   - if it exceeds m_run by more than 2^14 (always in the first block, where m_run is
    //     -inf; otherwise rare) the probabilities could overflow 16 bits: the reference moves
    //     and the block is exponentiated again;
    //   - if it exceeds m_run by more than 2^8 the reference moves before the next block.
    // Moving the reference rescales O and l_i by 2^(old - new); the final division by l_i
    // undoes whatever reference the exponentials used, so laziness costs no accuracy.
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int quarter = warp & 3;   // the TMEM lanes a warp may touch: 32 * (warp % 4)
    const int row = q0 + quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const float c = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.0f;
    float m_seen = -INFINITY;       // largest scaled score met so far (>= m_run)
    bool ok = true;

    // Moves the reference of the lanes with `move` set to m_seen.  O holds the products up
    // to block j-1 (nothing for j = 0): wait for that PV to retire, then rescale the row.
    auto move_reference = [&](bool move, int j) -> bool {
      float alpha = 1.0f;
      if (move) {
        alpha = exp2_approx(m_run - m_seen);   // 0 when m_run is -inf
        m_run = m_seen;
        l_run *= alpha;
      }
      if (j == 0) return true;
      const int pb = slot_of(j - 1);
      bool good = mbar_wait(smem_u32(&pv_done[pb]), par_of(j - 1), ctx, ST_ATTN_PV_DONE, j);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
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
      return true;
    };

    bool s_ready = false;   // answer to an early, non-blocking look at the next block's barrier
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int buf = slot_of(j);
      if (!__all_sync(0xffffffffu, s_ready)) {
        ok = mbar_wait(smem_u32(&s_full[buf]), par_of(j), ctx, ST_ATTN_S_FULL, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + lane_base + buf * kTileN;
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
      // the reference the previous block asked for (comparisons with -inf - -inf are false)
      if (__any_sync(0xffffffffu, m_seen - m_run > kRescaleThreshold)) {
        ok = move_reference(m_seen - m_run > kRescaleThreshold, j);
        if (!ok) break;
      }

      // S runs ahead of the softmax, so the next block is usually complete by now: ask while
      // the exponentials hide the round trip to the barrier
      s_ready = j + 1 < n_blocks &&
                mbar_test_wait(smem_u32(&s_full[slot_of(j + 1)]), par_of(j + 1));
      float block_sum = 0.0f;
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        const float m_use = m_run > -INFINITY ? m_run : 0.0f;
        // two scores per fma / add (packed fp32), four partial sums, four chains of maxima
        const unsigned long long c2 = pack2(c, c), negm2 = pack2(-m_use, -m_use);
        unsigned long long sum2[2] = {0ull, 0ull};
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
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
            mx4[i & 3] = max3(mx4[i & 3], a, b);
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
        block_sum = (s0 + s1) + (s2 + s3);
        m_seen = fmaxf(m_seen, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * c);
        // rows past seq_q (and nothing else) can be fully masked: -inf - -inf compares false
        const bool again = m_seen - m_run > kOverflowThreshold;
        if (pass == 1 || !__any_sync(0xffffffffu, again)) break;
        tmem_st_wait();   // the stores of this pass are replaced by the next one's
        ok = move_reference(again, j);
        if (!ok) break;
      }
      if (!ok) break;
      l_run += block_sum;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&p_full[buf]));
    }

    if (ok && n_blocks > 0) {
      const int lb = slot_of(n_blocks - 1);
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
  if (warp == kWarpQK) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ------------------------------------------------------------------------

template <int D>
int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                const AttnParams& p, bool bf16, cudaStream_t stream) {
  const int smem = (1 + 2 * kRing) * (D / 64) * 128 * 128 + (int)sizeof(AttnShared);
  const int grid = p.bh * p.n_q_tiles;
  auto go = [&](auto kern) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_check(e, "attention smem attribute");
    kern<<<grid, kThreads, smem, stream>>>(tq, tk, tv, p);
    return cuda_check(cudaGetLastError(), "attention launch");
  };
  return bf16 ? go(attn_fwd_kernel<D, true>) : go(attn_fwd_kernel<D, false>);
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

  if (d == 128) return launch_attn<128>(tq, tk, tv, p, bf16, stream);
  return launch_attn<64>(tq, tk, tv, p, bf16, stream);
}
