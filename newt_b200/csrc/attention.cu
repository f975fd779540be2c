// Fused attention forward on tcgen05 (K5):  O = softmax(scale * Q K^T [+ causal]) V.
//
// The program being replaced is the flash-style loop of
// examples/05_fused_attention.py:14-48 -- per Q tile, walk the KV blocks keeping a
// running row maximum m_i, a running row sum l_i and an fp32 output accumulator;
// P is rounded to the input type before the PV product (:43).  In the reference
// both dots are staged synchronously and the accumulator round-trips through
// shared memory every iteration (newt/compiler/codegen.py:1824-1852, 719-776).
//
// Here a persistent CTA per SM walks 128-row Q tiles of (batch, head) pairs:
//   warp 0       TMA producer: Q per tile, K and V blocks of 128 rows into two rings of three
//   warp 1       issues S = Q K^T (operands in shared memory, S in tensor memory)
//   warp 2       issues O += P V (P read from tensor memory, V from shared memory as an
//                MN-major operand, so no transpose of V is ever made)
//   warps 3..10  softmax: two groups of four warps take alternate KV blocks; in both, thread
//                t owns row t of the tile -- a TMEM lane -- so row max and row sum are plain
//                register loops, no shuffles.  P is written back over S as packed 16-bit
//                pairs.  The group of a tile's last block stores O; the other one is by
//                then on the next tile.
// S is triple-buffered and runs two blocks ahead of the softmax, and each MMA warp's
// instruction stream (waits, eight MMAs, one commit per block) is shorter than the tensor
// core's time for the block.  Every commit serves two waiters: "S complete" also frees the
// K slot, "PV retired" also frees the V slot and the S/P buffer.
// The reference maximum that P is scaled against only moves when a block maximum is more than
// 2^8 above it (exact in effect: the final division by l_i undoes whatever reference point
// the exponentials used); the softmax section states the rule both groups follow.
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
constexpr int kWarpTma = 0, kWarpQK = 1, kWarpPV = 2, kWarpSoftmax = 3;   // 3..10: two softmax groups
constexpr int kThreads = 32 * (kWarpSoftmax + 8);
constexpr int kMaxSlots = 3;  // block maxima in flight between the two softmax groups
constexpr float kRescaleThreshold = 8.0f;    // log2 units: how far a row maximum may run ahead of the reference

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
  ST_ATTN_S_FULL, ST_ATTN_P_FULL, ST_ATTN_PV_DONE, ST_ATTN_LAYOUT, ST_ATTN_MAX_DONE, ST_ATTN_O_FREE,
  ST_ATTN_SUM
};

// What a CTA keeps in shared memory besides the tiles.  Blocks are counted over the whole
// life of the CTA (g = 0, 1, ... across its tiles); block g uses slot g % 3 of the K ring, the
// V ring and the S/P buffers, and slot g % 3 of the block maxima.
//   s_full[x]:  S of the block in slot x is complete (softmax may read it, K slot x is free)
//   p_full[x]:  P of that block is in tensor memory (one arrival per warp of its softmax group)
//   pv_done[x]: its PV product has retired (V slot x and S/P buffer x are free, O is current)
//   q_free:     every S product of the tile has retired (the Q tile may be overwritten)
//   o_free:     the epilogue has read O (the next tile's first PV product may overwrite it)
struct AttnShared {
  uint64_t q_full, q_free, o_free, sum_done, sum_read;
  uint64_t k_full[kRing], v_full[kRing];
  uint64_t s_full[kRing], p_full[kRing], pv_done[kRing];
  uint64_t max_done[kMaxSlots];          // block_max[x] is published (one arrival per warp of a group)
  uint32_t tmem_slot;
  uint32_t abort_flag;
  float block_max[kMaxSlots][kTileM];    // scaled row maxima of the blocks in flight
  float2 row_part[kTileM];               // (partial row sum, its reference) of the group that
                                         // does not close the tile
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
  auto slot_of = [](int g) { return g % kRing; };
  auto par_of = [](int g) { return uint32_t((g / kRing) & 1); };

  // Everything in shared memory is carved from the dynamic allocation (no static part, so
  // the 128-byte-swizzled tiles start on the 1024-byte boundary the allocation starts on):
  // Q tile, K ring, V ring, then the barriers and the exchange buffers.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  AttnShared& sh = *reinterpret_cast<AttnShared*>(smem_raw + (1 + 2 * kRing) * kTileBytes);
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

  // The grid is persistent.  The tile list runs head by head (so the K/V of the few heads in
  // flight stay in L2) and, inside a head, alternates between the ends: last Q tile, first,
  // last but one, second, ...  CTA b takes the pairs of neighbours b, b + gridDim.x, ... of
  // that list, so with a causal mask every pair costs the same number of KV blocks and the
  // CTAs finish together.  Going from one tile to the next costs no start-up: the next Q and
  // K blocks are loaded and the next S products issued while the softmax groups finish the
  // current tile.
  const int num_tiles = p.bh * p.n_q_tiles;
  auto nth_tile = [&](int it) {   // index in the list of the it-th tile of this CTA
    return 2 * (int(blockIdx.x) + (it >> 1) * int(gridDim.x)) + (it & 1);
  };
  struct Tile {
    int head, q0, n_blocks;
  };
  auto tile_at = [&](int t) {
    Tile tile;
    tile.head = t / p.n_q_tiles;
    const int k = t % p.n_q_tiles;
    tile.q0 = ((k & 1) ? (k >> 1) : p.n_q_tiles - 1 - (k >> 1)) * kTileM;
    int kv_end = p.seq_kv;
    if (p.causal) kv_end = min(kv_end, tile.q0 + kTileM);
    tile.n_blocks = (kv_end + kTileN - 1) / kTileN;
    return tile;
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&sh.q_full), 1);
    mbar_init(smem_u32(&sh.q_free), 1);
    mbar_init(smem_u32(&sh.o_free), 4);     // one arrival per warp of the group that closes a tile
    mbar_init(smem_u32(&sh.sum_done), 4);   // ... of the other group
    mbar_init(smem_u32(&sh.sum_read), 4);
#pragma unroll
    for (int x = 0; x < kRing; ++x) {
      mbar_init(smem_u32(&k_full[x]), 1);
      mbar_init(smem_u32(&v_full[x]), 1);
      mbar_init(smem_u32(&s_full[x]), 1);
      mbar_init(smem_u32(&p_full[x]), 4);   // one arrival per warp of the block's softmax group
      mbar_init(smem_u32(&pv_done[x]), 1);
    }
#pragma unroll
    for (int x = 0; x < kMaxSlots; ++x) mbar_init(smem_u32(&sh.max_done[x]), 4);
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
  auto wait_all = [&](uint64_t* bar, uint32_t parity, unsigned int code, int g) -> bool {
    return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, ctx, code, g));
  };
  // Q and K tiles: K-major, rows of 128 B, 8-row groups 1024 B apart, one 16 KB chunk per
  // 64 columns of D.  V tile: MN-major, 64-column slabs kChunkBytes apart.
  constexpr uint64_t kKMajor = smem_desc_sw128(16, 1024);
  constexpr uint64_t kVDesc = smem_desc_sw128(kChunkBytes, 1024);

  if (warp == kWarpTma) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      bool ok = true;
      int g0 = 0;   // blocks of the tiles before this one
      for (int it = 0, t = nth_tile(0); t < num_tiles && ok; ++it, t = nth_tile(it)) {
        const Tile tile = tile_at(t);
        // K slot x is free once the S product that read it is complete, V slot x once the PV
        // product is: the barriers the MMA warps commit to anyway.
        auto load = [&](const CUtensorMap* map, uint32_t ring, uint64_t* free_bar,
                        uint64_t* full_bar, unsigned int code, int j) -> bool {
          const int g = g0 + j, x = slot_of(g);
          if (!mbar_wait(smem_u32(&free_bar[x]), par_of(g) ^ 1, ctx, code, g)) return false;
          mbar_arrive_expect_tx(smem_u32(&full_bar[x]), kTileBytes);
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            tma_load_3d(ring + x * kTileBytes + c * kChunkBytes, map, c * 64, j * kTileN, tile.head,
                        smem_u32(&full_bar[x]));
          return true;
        };
        // the Q tile is free once the previous tile's S products have all retired
        ok = mbar_wait(smem_u32(&sh.q_free), (it & 1) ^ 1, ctx, ST_ATTN_Q, it);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&sh.q_full), kTileBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(q_smem + c * kChunkBytes, &tmap_q, c * 64, tile.q0, tile.head,
                      smem_u32(&sh.q_full));
        // K runs a whole ring ahead of V because S = Q K^T is issued blocks before the PV
        // product of the same block
        for (int j = 0; j < kRing && j < tile.n_blocks && ok; ++j)
          ok = load(&tmap_k, k_smem, s_full, k_full, ST_ATTN_K_EMPTY, j);
        for (int j = 0; j < tile.n_blocks && ok; ++j) {
          ok = load(&tmap_v, v_smem, pv_done, v_full, ST_ATTN_V_EMPTY, j);
          if (ok && j + kRing < tile.n_blocks)
            ok = load(&tmap_k, k_smem, s_full, k_full, ST_ATTN_K_EMPTY, j + kRing);
        }
        g0 += tile.n_blocks;
      }
    }
  } else if (warp == kWarpQK) {
    // ---------------- issuer of S = Q K^T ----------------
    // The whole warp walks the loop and waits; one elected lane issues, so addresses and
    // descriptors stay in uniform registers.  Two issuing warps (this one and the PV warp)
    // because one thread's instruction stream -- waits, sixteen MMAs and the commits of a
    // block -- took longer than the tensor core needs for the block.
    const bool elected = elect_one();
    bool ok = true;
    int g0 = 0;
    for (int it = 0, t = nth_tile(0); t < num_tiles && ok; ++it, t = nth_tile(it)) {
      const Tile tile = tile_at(t);
      ok = wait_all(&sh.q_full, it & 1, ST_ATTN_Q, it);
      for (int j = 0; j < tile.n_blocks && ok; ++j) {
        const int g = g0 + j, x = slot_of(g);
        // S/P buffer x was read (as P) by the PV product of block g-3
        ok = wait_all(&pv_done[x], par_of(g) ^ 1, ST_ATTN_PV_DONE, g) &&
             wait_all(&k_full[x], par_of(g), ST_ATTN_K_FULL, g);
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
        if (elected) {
          mma_commit(smem_u32(&s_full[x]));
          if (j == tile.n_blocks - 1) mma_commit(smem_u32(&sh.q_free));
        }
        __syncwarp();
      }
      g0 += tile.n_blocks;
    }
  } else if (warp == kWarpPV) {
    // ---------------- issuer of O += P V ----------------
    const bool elected = elect_one();
    bool ok = true;
    int g0 = 0;
    for (int it = 0, t = nth_tile(0); t < num_tiles && ok; ++it, t = nth_tile(it)) {
      const Tile tile = tile_at(t);
      // the first product of a tile overwrites O: the previous tile's epilogue must have read it
      ok = wait_all(&sh.o_free, (it & 1) ^ 1, ST_ATTN_O_FREE, it);
      for (int j = 0; j < tile.n_blocks && ok; ++j) {
        const int g = g0 + j, x = slot_of(g);
        ok = wait_all(&v_full[x], par_of(g), ST_ATTN_V_FULL, g) &&
             wait_all(&p_full[x], par_of(g), ST_ATTN_P_FULL, g);
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
      g0 += tile.n_blocks;
    }
  } else {
    // ---------------- softmax + epilogue: two groups of four warps, alternating blocks ------
    // Group g (warps 3+4g .. 6+4g) handles the KV blocks n of a tile with n % 2 == g; in both
    // groups thread t owns row t of the tile -- a TMEM lane -- so row maximum and row sum are
    // register loops.  With one group, a scheduler's only softmax warp could not overlap its
    // own phases (TMEM load + row maximum on the ALU, then 128 exponentials per row on the
    // special-function unit, which is the unit that bounds this loop); with two, one group's
    // maxima run under the other's exponentials.
    //
    // Both groups must scale P against the same reference maximum R_n, because O is one
    // accumulator.  R_n follows a rule that every thread of a row can replay from the block
    // maxima alone:  M_n = max(M_{n-1}, max of block n),  R_n = M_n if M_n - R_{n-1} > 2^8
    // (or nothing seen yet), else R_{n-1}.  A thread publishes its block maximum in shared
    // memory; the thread of the other group reads it one block later (the barrier it waits
    // on is normally complete).  The group whose block changes the reference rescales O after
    // the previous PV product has retired.  Each group keeps its own partial row sum, in
    // terms of the last reference it used; the two are combined at the end of the tile.
    // P never exceeds 2^8, and the final division by l_i undoes whatever reference was used.
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int quarter = warp & 3;   // the TMEM lanes a warp may touch: 32 * (warp % 4)
    const int group = (warp - kWarpSoftmax) >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const float c = p.scale_log2;
    bool ok = true;
    int g0 = 0;
    int first = 0;   // the group that takes the even blocks of this tile
    for (int it = 0, t = nth_tile(0); t < num_tiles && ok; ++it, t = nth_tile(it)) {
      const Tile tile = tile_at(t);
      const int row = tile.q0 + r;
      // The group of the last block closes the tile (combines the row sums, stores O); the
      // other one goes straight on to block 0 of the next tile.
      const int closer = (tile.n_blocks - 1 + first) & 1;
      float m_all = -INFINITY;    // M: largest scaled score of the blocks replayed so far
      float ref = -INFINITY;      // R of the last block replayed
      float l_part = 0.0f;        // this group's part of the row sum ...
      float l_ref = -INFINITY;    // ... in terms of this reference
      auto advance = [&](float block_max) {   // the rule above
        m_all = fmaxf(m_all, block_max);
        if (m_all - ref > kRescaleThreshold) ref = m_all;   // false while m_all is -inf
      };

      bool s_ready = false;   // answer to an early, non-blocking look at the next block's barrier
      for (int n = group ^ first; n < tile.n_blocks && ok; n += 2) {
        const int g = g0 + n, buf = slot_of(g);
        if (!__all_sync(0xffffffffu, s_ready)) {
          ok = mbar_wait(smem_u32(&s_full[buf]), par_of(g), ctx, ST_ATTN_S_FULL, g);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        tc_fence_after_sync();
        // the other group's maximum of block n-1 is usually published by now: ask while the
        // first pass hides the round trip to the barrier
        const bool max_ready =
            n > 0 && mbar_test_wait(smem_u32(&sh.max_done[(g - 1) % kMaxSlots]), ((g - 1) / kMaxSlots) & 1);
        const uint32_t s_tmem = tmem_base + lane_base + buf * kTileN;
        const int kv0 = n * kTileN;
        const bool edge = (p.causal && kv0 + kTileN - 1 > tile.q0) || (kv0 + kTileN > p.seq_kv);
        const int limit = p.causal ? min(row, p.seq_kv - 1) : p.seq_kv - 1;   // last visible column
        // 64 scores of the row at a time (S stays in tensor memory between the two passes)
        auto fetch = [&](int h, uint32_t (&s)[2][32]) {
          tmem_ld_32x32(s_tmem + h * 64, s[0]);
          tmem_ld_32x32(s_tmem + h * 64 + 32, s[1]);
          tmem_ld_wait();
          if (edge) {
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (kv0 + h * 64 + q * 32 + i > limit) s[q][i] = __float_as_uint(-INFINITY);
          }
        };

        // ---- pass 1: the block's row maximum, published for the other group ----
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        {
          uint32_t s[4][32];   // the whole row at once: nothing else is live in this pass
#pragma unroll
          for (int q = 0; q < 4; ++q) tmem_ld_32x32(s_tmem + q * 32, s[q]);
          tmem_ld_wait();
          if (edge) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (kv0 + q * 32 + i > limit) s[q][i] = __float_as_uint(-INFINITY);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(s[q][i]),
                                       __uint_as_float(s[q][i + 1]));
        }
        const float block_max = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * c;
        sh.block_max[g % kMaxSlots][r] = block_max;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.max_done[g % kMaxSlots]));

        // ---- replay the rule over block n-1 (the other group's) and block n ----
        if (n > 0) {
          if (!__all_sync(0xffffffffu, max_ready)) {
            ok = mbar_wait(smem_u32(&sh.max_done[(g - 1) % kMaxSlots]), ((g - 1) / kMaxSlots) & 1, ctx,
                           ST_ATTN_MAX_DONE, g);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          advance(sh.block_max[(g - 1) % kMaxSlots][r]);
        }
        const float ref_before = ref;   // R_{n-1}
        advance(block_max);
        if (n > 0 && __any_sync(0xffffffffu, ref != ref_before)) {
          // O holds the products up to block n-1 in terms of R_{n-1}
          ok = mbar_wait(smem_u32(&pv_done[slot_of(g - 1)]), par_of(g - 1), ctx, ST_ATTN_PV_DONE, g);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const float alpha = ref != ref_before ? exp2_approx(ref_before - ref) : 1.0f;
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
        if (l_ref != ref) {   // two blocks of references may have passed
          l_part *= l_ref > -INFINITY ? exp2_approx(l_ref - ref) : 0.0f;
          l_ref = ref;
        }

        // S runs ahead of the softmax, so this group's next block is usually complete by now
        s_ready = n + 2 < tile.n_blocks &&
                  mbar_test_wait(smem_u32(&s_full[slot_of(g + 2)]), par_of(g + 2));
        // ---- pass 2: P = 2^(S * scale - R_n), packed over the scores already consumed ----
        const float m_use = ref > -INFINITY ? ref : 0.0f;   // rows past seq_q see nothing at all
        const unsigned long long c2 = pack2(c, c), negm2 = pack2(-m_use, -m_use);
        unsigned long long sum2[2] = {0ull, 0ull};
#pragma unroll
        for (int h = 0; h < 2; ++h) {   // 64 scores -> 32 packed columns per store
          uint32_t s[2][32];
          fetch(h, s);
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float a = __uint_as_float(s[i / 16][(2 * i) % 32]);
            const float b = __uint_as_float(s[i / 16][(2 * i) % 32 + 1]);
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
          // columns [32h, 32h+32) of the buffer: scores 0..63 / 64..127 were read above
          tmem_st_32x32(s_tmem + h * 32, pk);
        }
        float s0, s1, s2, s3;
        unpack2(sum2[0], s0, s1);
        unpack2(sum2[1], s2, s3);
        l_part += (s0 + s1) + (s2 + s3);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&p_full[buf]));
      }
      if (!ok) break;

      g0 += tile.n_blocks;
      first = closer ^ 1;
      if (group != closer) {
        // hand the partial sum over (the previous hand-over must have been read)
        ok = mbar_wait(smem_u32(&sh.sum_read), (it & 1) ^ 1, ctx, ST_ATTN_SUM, it);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        sh.row_part[r] = make_float2(l_part, l_ref);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.sum_done));
        continue;
      }
      // ---- close the tile: O is complete once the last PV product has retired ----
      const int g_last = g0 - 1;
      ok = mbar_wait(smem_u32(&pv_done[slot_of(g_last)]), par_of(g_last), ctx, ST_ATTN_PV_DONE, g_last) &&
           mbar_wait(smem_u32(&sh.sum_done), it & 1, ctx, ST_ATTN_SUM, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      // this group's sum is in terms of the last reference, which is the one O is in;
      // references only ever rise, so the other group's is not above it
      const float2 other = sh.row_part[r];
      const float inv =
          1.0f / (l_part + (other.y > -INFINITY ? other.x * exp2_approx(other.y - ref) : 0.0f));
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh.sum_read));

      OutT* orow = static_cast<OutT*>(p.o) + (long long)tile.head * p.o_head_stride +
                   (long long)row * p.o_row_stride;
      const bool vec = ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_base + kOCol + q * 32, o);
        tmem_ld_wait();
        if (q == D / 32 - 1) {
          // O is in registers: the next tile's first PV product may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh.o_free));
        }
        if (row < p.seq_q) {
#pragma unroll
          for (int gq = 0; gq < 4; ++gq) {
            uint32_t packed[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float lo = __uint_as_float(o[gq * 8 + 2 * h]) * inv;
              const float hi = __uint_as_float(o[gq * 8 + 2 * h + 1]) * inv;
              if constexpr (BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                packed[h] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            OutT* dst = orow + q * 32 + gq * 8;
            if (vec) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
              const OutT* e = reinterpret_cast<const OutT*>(packed);
#pragma unroll
              for (int tt = 0; tt < 8; ++tt) dst[tt] = e[tt];
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
  // persistent: one CTA per SM, never more than there are pairs of tiles
  int grid = device_info().sm_count;
  const long long pairs = ((long long)p.bh * p.n_q_tiles + 1) / 2;
  if (pairs < grid) grid = (int)pairs;
  auto go = [&](auto kern) {
    if (int rc = prepare_kernel((const void*)kern, smem)) return rc;
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
