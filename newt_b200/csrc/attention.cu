// Fused attention forward on tcgen05 (K5):  O = softmax(scale * Q K^T [+ causal]) V.
//
// The program being replaced is the flash-style loop of
// examples/05_fused_attention.py:14-48 -- per Q tile, walk the KV blocks keeping a
// running row maximum m_i, a running row sum l_i and an fp32 output accumulator;
// P is rounded to the input type before the PV product (:43).  In the reference
// both dots are staged synchronously and the accumulator round-trips through
// shared memory every iteration (newt/compiler/codegen.py:1824-1852, 719-776).
//
// Here a persistent CTA per SM (512 threads, four warpgroups) walks *pairs* of neighbouring
// 128-row Q tiles of one (batch, head); the two tiles share every K/V block (loaded once,
// used twice) and take turns on the tensor core, so one tile's two products run while the
// other tile's softmax does:
//   warp 0         TMA producer: the two Q tiles per pair, K and V blocks of 128 rows in one
//                  ring of five slots (K0 V0 K1 V1 ...)
//   warp 1         issues, for both tiles in turn, S_t = Q_t K^T and O_t += P_t V (P read from
//                  tensor memory, V from shared memory as an MN-major operand: no transpose)
//   warps 4..7     softmax of tile 0: thread r owns row r -- a TMEM lane -- so row max and
//   warps 8..11    row sum are register loops, no shuffles (the same for tile 1).  The 128
//                  scores of a row are read from tensor memory once and stay in registers; P
//                  is written over S as packed 16-bit pairs and handed over in two halves, so
//                  the first half of the PV product runs under the second half's exponentials.
//   warps 12..15   epilogue: O_t / l_t -> global, while the softmax warps are already on the
//                  next pair
// The warpgroups re-divide the register file (setmaxnreg): 208 registers per softmax thread,
// 40 and 56 for the others.
// Tensor memory: S0 | S1 (128 columns each, P_t over the first 64 of S_t) | O0 | O1 = 512.
// The order in which one thread issues  ... PV_t(j), QK_t(j+1) ...  is the order the tensor core
// executes them in, so S_t(j+1) lands only after P_t(j) has been read; a softmax group is told
// "S_t(j) complete" by a commit that also covers PV_t(j-1), so it may rescale O_t right away.
// One issuer, strictly alternating between the tiles, is what keeps them half a period apart
// (two issuing warps, one per tile, interleave their products, finish together, and both
// softmax groups then run -- and wait -- together: measured 25 % slower).
// The reference maximum that P is scaled against only moves when a block maximum is more than
// 2^8 above it (exact in effect: the final division by l_i undoes whatever reference point
// the exponentials used); the row sum is kept in terms of the same reference.
// Scores are kept in the log2 domain: p = 2^(s * scale * log2(e) - m).
//
// Causal tiles skip the KV blocks above the diagonal and mask only the diagonal
// block.  Tensor-bound; flop per launch = 4 * BH * Sq * Skv * D (halved if causal).

#include <type_traits>

#include "sm100.cuh"

namespace nb200 {
namespace {

using namespace sm100;

constexpr int kTileM = 128;   // Q rows per tile = TMEM lanes
constexpr int kTileN = 128;   // KV rows per block
constexpr int kKvSlots = 5;   // ring of K and V blocks (alternating)
constexpr int kWarpTma = 0, kWarpMma = 1, kWarpSoftmax = 4, kWarpEpilogue = 12;
constexpr int kThreads = 512;
constexpr float kRescaleThreshold = 8.0f;    // log2 units: how far a row maximum may run ahead of the reference
// registers per thread after the warpgroups re-divide the register file (multiples of 8;
// 128 * (40 + 2 * 208 + 56) = 65536)
constexpr int kRegsIssue = 40, kRegsSoftmax = 208, kRegsEpilogue = 56;

struct AttnParams {
  void* o;
  long long o_head_stride, o_row_stride;
  int bh, seq_q, seq_kv, n_q_tiles;
  float scale_log2;  // scale * log2(e)
  int causal;
  uint32_t idesc_qk, idesc_pv;
  unsigned long long wait_limit_ns;
  unsigned int* status;
};

enum : unsigned int {
  ST_ATTN_Q_FULL = 16, ST_ATTN_Q_EMPTY, ST_ATTN_KV_FULL, ST_ATTN_KV_EMPTY, ST_ATTN_S_FULL,
  ST_ATTN_P_FULL, ST_ATTN_O_FULL, ST_ATTN_O_EMPTY, ST_ATTN_L_FULL, ST_ATTN_L_EMPTY, ST_ATTN_LAYOUT
};

// What a CTA keeps in shared memory besides the tiles.  Index t is the tile of the pair.
//   q_full[t] / q_empty[t]    Q_t has landed / every S product of the pair that reads it retired
//   kv_full[x] / kv_empty[x]  ring slot x holds its K or V block / the products that read it retired
//   s_full[t]                 S_t of the tile's current block is complete (and every product issued
//                             before it, the previous block's PV_t among them)
//   p_full[t][h]              half h (64 KV rows) of P_t of that block is in tensor memory (one
//                             arrival per softmax warp)
//   o_full[t] / o_empty[t]    the pair's last PV_t retired / the epilogue has O_t in registers
//   l_full[t] / l_empty[t]    the row sums of tile t are in row_sum[t] / have been read
struct AttnShared {
  uint64_t q_full[2], q_empty[2];
  uint64_t kv_full[kKvSlots], kv_empty[kKvSlots];
  uint64_t s_full[2], p_full[2][2];
  uint64_t o_full[2], o_empty[2];
  uint64_t l_full[2], l_empty[2];
  uint32_t tmem_slot;
  uint32_t abort_flag;
  float row_sum[2][kTileM];
};

// Cycle counters of one softmax thread and one issuing thread of CTA 0, compiled in only with
// -DNB200_ATTN_PROFILE (a development build; the shipped library has none of this).
#ifdef NB200_ATTN_PROFILE
__device__ long long g_attn_prof[32];
#define PROF_DECL(n) long long prof_acc[n] = {}; long long prof_t = clock64();
#define PROF_LAP(i) { const long long now = clock64(); prof_acc[i] += now - prof_t; prof_t = now; }
#define PROF_DUMP(base, n, cond) if (cond) { for (int i_ = 0; i_ < n; ++i_) g_attn_prof[base + i_] = prof_acc[i_]; }
// event trace of CTA 0: role (0 softmax 0, 1 softmax 1, 2 issuing warp), up to 512 events each
__device__ long long g_attn_trace[3][512][2];
#define TRACE_DECL int trace_n = 0;
#define TRACE(role, id, cond) if (blockIdx.x == 0 && (cond) && trace_n < 512) { g_attn_trace[role][trace_n][0] = (id); g_attn_trace[role][trace_n][1] = clock64(); ++trace_n; }
#else
#define TRACE_DECL
#define TRACE(role, id, cond)
#define PROF_DECL(n)
#define PROF_LAP(i)
#define PROF_DUMP(base, n, cond)
#endif

template <int N>
__device__ __forceinline__ void set_max_registers_up() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void set_max_registers_down() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                    const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  constexpr int kChunks = D / 64;                       // 64-element (128-byte) column chunks
  constexpr uint32_t kChunkBytes = 128 * 128;           // 128 rows x 128 B
  constexpr uint32_t kTileBytes = kChunks * kChunkBytes;  // one Q, K or V tile
  constexpr uint32_t kOCol = 2 * kTileN;                // O_0 at 256, O_1 at 384
  constexpr uint32_t kTmemCols = 512;

  // Everything in shared memory is carved from the dynamic allocation (no static part, so
  // the 128-byte-swizzled tiles start on the 1024-byte boundary the allocation starts on):
  // Q_0, Q_1, the K/V ring, then the barriers and the row sums.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  AttnShared& sh = *reinterpret_cast<AttnShared*>(smem_raw + (2 + kKvSlots) * kTileBytes);
  volatile uint32_t& abort_flag = sh.abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_smem = smem_u32(smem_raw);
  const uint32_t kv_smem = q_smem + 2 * kTileBytes;
  const WaitCtx ctx{&sh.abort_flag, p.status, p.wait_limit_ns};
  if (q_smem & 1023u) {   // the tiles would be misread; uniform over the CTA
    if (threadIdx.x == 0 && atomicCAS(&p.status[0], 0u, (unsigned)ST_ATTN_LAYOUT) == 0u)
      p.status[1] = q_smem;
    return;
  }

  // The grid is persistent.  A work item is a pair of neighbouring Q tiles (2i, 2i+1) of one
  // head.  The list of items runs head by head (so the K/V of the few heads in flight stay in
  // L2) and, inside a head, alternates between the ends: last pair, first, last but one,
  // second, ...  CTA b takes the neighbours 2(b + k * gridDim.x), +1 of that list, so with a
  // causal mask every CTA gets the same number of KV blocks per round.
  const int n_pairs = (p.n_q_tiles + 1) >> 1;
  const int num_items = p.bh * n_pairs;
  auto nth_item = [&](int it) {   // index in the list of the it-th item of this CTA
    return 2 * (int(blockIdx.x) + (it >> 1) * int(gridDim.x)) + (it & 1);
  };
  struct Item {
    int head, q0[2], nb[2], nb_max;
  };
  auto item_at = [&](int t) {
    Item item;
    item.head = t / n_pairs;
    const int k = t % n_pairs;
    const int pair = (k & 1) ? (k >> 1) : n_pairs - 1 - (k >> 1);
#pragma unroll
    for (int tt = 0; tt < 2; ++tt) {
      item.q0[tt] = (2 * pair + tt) * kTileM;
      int kv_end = p.seq_kv;
      if (p.causal) kv_end = min(kv_end, item.q0[tt] + kTileM);
      item.nb[tt] = item.q0[tt] < p.seq_q ? (kv_end + kTileN - 1) / kTileN : 0;   // 0: no such tile
    }
    item.nb_max = max(item.nb[0], item.nb[1]);
    return item;
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&sh.q_full[t]), 1);
      mbar_init(smem_u32(&sh.q_empty[t]), 1);
      mbar_init(smem_u32(&sh.s_full[t]), 1);
      mbar_init(smem_u32(&sh.p_full[t][0]), 4);  // one arrival per warp of the tile's softmax group
      mbar_init(smem_u32(&sh.p_full[t][1]), 4);
      mbar_init(smem_u32(&sh.o_full[t]), 1);
      mbar_init(smem_u32(&sh.o_empty[t]), 4);    // ... per epilogue warp
      mbar_init(smem_u32(&sh.l_full[t]), 4);
      mbar_init(smem_u32(&sh.l_empty[t]), 4);
    }
#pragma unroll
    for (int x = 0; x < kKvSlots; ++x) {
      mbar_init(smem_u32(&sh.kv_full[x]), 1);
      mbar_init(smem_u32(&sh.kv_empty[x]), 1);   // the issuing warp's commit
    }
    mbar_init_fence();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == kWarpMma) {
    __syncwarp();
    tmem_alloc(smem_u32(&sh.tmem_slot), kTmemCols);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh.tmem_slot;

  // a whole warp waits (so that its control flow stays uniform); false = give up
  auto wait_all = [&](uint64_t* bar, uint32_t parity, unsigned int code, int detail) -> bool {
    return __all_sync(0xffffffffu, mbar_wait_nocall(smem_u32(bar), parity, ctx, code, detail));
  };
  // Q and K tiles: K-major, rows of 128 B, 8-row groups 1024 B apart, one 16 KB chunk per
  // 64 columns of D.  V tile: MN-major, 64-column slabs kChunkBytes apart.
  constexpr uint64_t kKMajor = smem_desc_sw128(16, 1024);
  constexpr uint64_t kVDesc = smem_desc_sw128(kChunkBytes, 1024);

  if (warp < kWarpSoftmax) {
    set_max_registers_down<kRegsIssue>();
    if (warp == kWarpTma) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        bool ok = true;
        int g = 0;                 // K/V blocks loaded so far: block g lives in slot g % kKvSlots
        int cnt[2] = {0, 0};       // pairs so far in which tile t took part
        for (int it = 0, t = nth_item(0); t < num_items && ok; ++it, t = nth_item(it)) {
          const Item item = item_at(t);
          auto load_kv = [&](const CUtensorMap* map, int j) -> bool {
            const int x = g % kKvSlots;
            if (!mbar_wait_nocall(smem_u32(&sh.kv_empty[x]), ((g / kKvSlots) & 1) ^ 1, ctx, ST_ATTN_KV_EMPTY, g))
              return false;
            const uint32_t bar = smem_u32(&sh.kv_full[x]);
            mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
            for (int c = 0; c < kChunks; ++c)
              tma_load_3d(kv_smem + x * kTileBytes + c * kChunkBytes, map, c * 64, j * kTileN,
                          item.head, bar);
            ++g;
            return true;
          };
          // a Q tile is free once the previous pair's S products that read it have retired
#pragma unroll
          for (int tt = 0; tt < 2; ++tt) {
            if (item.nb[tt] == 0 || !ok) continue;
            ok = mbar_wait_nocall(smem_u32(&sh.q_empty[tt]), (cnt[tt] & 1) ^ 1, ctx, ST_ATTN_Q_EMPTY, it);
            if (!ok) break;
            const uint32_t bar = smem_u32(&sh.q_full[tt]);
            mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
            for (int c = 0; c < kChunks; ++c)
              tma_load_3d(q_smem + tt * kTileBytes + c * kChunkBytes, &tmap_q, c * 64, item.q0[tt],
                          item.head, bar);
            ++cnt[tt];
          }
          for (int j = 0; j < item.nb_max && ok; ++j)
            ok = load_kv(&tmap_k, j) && load_kv(&tmap_v, j);
        }
      }
    } else if (warp == kWarpMma) {
      // ---------------- issuer of S_t = Q_t K^T and O_t += P_t V, both tiles ----------------
      // The whole warp walks the loop and waits; one elected lane issues, so addresses and
      // descriptors stay in uniform registers.  Per KV block j the order is
      //   wait P_0(j): PV_0(j), QK_0(j+1);   wait P_1(j): PV_1(j), QK_1(j+1)
      // One issuer, strictly alternating, is what keeps the two tiles half a period apart: the
      // tensor core works on one tile while the other tile's softmax has the special-function
      // unit to itself.  (Two issuing warps, one per tile, interleave their products on the
      // tensor core, finish together, and both softmax groups then run -- and wait -- together.)
      const bool elected = elect_one();
      bool ok = true;
      int g = 0;                  // K/V blocks consumed so far (ring position)
      int cnt[2] = {0, 0};        // pairs so far in which tile t took part
      int blk[2] = {0, 0};        // blocks of tile t so far
      PROF_DECL(8)
      TRACE_DECL
      auto kv_wait = [&](int gi) -> bool {
        return wait_all(&sh.kv_full[gi % kKvSlots], (gi / kKvSlots) & 1, ST_ATTN_KV_FULL, gi);
      };
      auto kv_release = [&](int gi) {   // free once every product issued so far has retired
        if (elected) mma_commit(smem_u32(&sh.kv_empty[gi % kKvSlots]));
      };
      auto qk = [&](int tt, int gi) {     // S_t = Q_t K^T for the K block in ring position gi
        const uint32_t qb = q_smem + tt * kTileBytes;
        const uint32_t kb = kv_smem + (gi % kKvSlots) * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kChunkBytes + (kk % 4) * 32;
          const uint64_t qd = with_address(kKMajor, qb + off);
          const uint64_t kd = with_address(kKMajor, kb + off);
          if (elected) mma_f16_ss(tmem_base + tt * kTileN, qd, kd, p.idesc_qk, kk != 0 ? 1u : 0u);
        }
        if (elected) mma_commit(smem_u32(&sh.s_full[tt]));
      };
      auto pv = [&](int tt, int gi, int h, bool first) {   // O_t (+)= P_t V, KV rows 64h.. of the block
        const uint32_t vb = kv_smem + (gi % kKvSlots) * kTileBytes;
        const uint32_t p_tmem = tmem_base + tt * kTileN;
#pragma unroll
        for (int kk = 4 * h; kk < 4 * h + 4; ++kk) {
          // 16 K-elements of P = 8 packed columns; 16 KV rows of V = 2048 B
          const uint64_t vd = with_address(kVDesc, vb + kk * 2048);
          if (elected)
            mma_f16_ts(tmem_base + kOCol + tt * kTileN, p_tmem + kk * 8, vd, p.idesc_pv,
                       (first && kk == 0) ? 0u : 1u);
        }
      };
      for (int it = 0, t = nth_item(0); t < num_items && ok; ++it, t = nth_item(it)) {
        const Item item = item_at(t);
#pragma unroll
        for (int tt = 0; tt < 2; ++tt)
          if (ok && item.nb[tt] > 0) ok = wait_all(&sh.q_full[tt], cnt[tt] & 1, ST_ATTN_Q_FULL, it);
        ok = ok && kv_wait(g);            // K block 0
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
          if (item.nb[tt] > 0) {
            qk(tt, g);
            if (item.nb[tt] == 1 && elected) mma_commit(smem_u32(&sh.q_empty[tt]));
          }
        }
        kv_release(g);
        __syncwarp();
        ++g;
        for (int j = 0; j < item.nb_max && ok; ++j) {
          // ring positions: V block j at g, K block j + 1 at g + 1
          const bool more = j + 1 < item.nb_max;
          PROF_LAP(0)
          ok = kv_wait(g);
          PROF_LAP(1)
          bool k_ready = false;
#pragma unroll
          for (int tt = 0; tt < 2; ++tt) {
            if (!ok) break;
            if (j < item.nb[tt]) {
              ok = wait_all(&sh.p_full[tt][0], blk[tt] & 1, ST_ATTN_P_FULL, blk[tt]);
              // the first product of a pair overwrites O_t: the epilogue must have read it
              if (ok && j == 0) ok = wait_all(&sh.o_empty[tt], (cnt[tt] & 1) ^ 1, ST_ATTN_O_EMPTY, it);
              if (!ok) break;
              PROF_LAP(2 + 3 * tt)
              TRACE(2, 10 * tt + 0, elected)     // P half 0 seen
              tc_fence_after_sync();
              pv(tt, g, 0, j == 0);
              TRACE(2, 10 * tt + 1, elected)     // PV half 0 issued
              ok = wait_all(&sh.p_full[tt][1], blk[tt] & 1, ST_ATTN_P_FULL, blk[tt]);
              ++blk[tt];
              if (!ok) break;
              TRACE(2, 10 * tt + 2, elected)     // P half 1 seen
              tc_fence_after_sync();
              pv(tt, g, 1, false);
              TRACE(2, 10 * tt + 3, elected)     // PV half 1 issued
              if (j == item.nb[tt] - 1 && elected) mma_commit(smem_u32(&sh.o_full[tt]));
              PROF_LAP(3 + 3 * tt)
            }
            if (tt == 1) kv_release(g);   // both tiles' products with V block j are issued
            if (j + 1 < item.nb[tt]) {
              if (!k_ready) {
                ok = kv_wait(g + 1);
                if (!ok) break;
                tc_fence_after_sync();
                k_ready = true;
              }
              TRACE(2, 10 * tt + 4, elected)     // K ready
              qk(tt, g + 1);
              if (j + 2 == item.nb[tt] && elected) mma_commit(smem_u32(&sh.q_empty[tt]));
              PROF_LAP(4 + 3 * tt)
              TRACE(2, 10 * tt + 5, elected)     // QK issued
            }
            __syncwarp();
          }
          if (!ok) break;
          if (more) {
            if (!k_ready) ok = kv_wait(g + 1);   // nobody used it: hand it back all the same
            kv_release(g + 1);
            __syncwarp();
          }
          g += more ? 2 : 1;
        }
#pragma unroll
        for (int tt = 0; tt < 2; ++tt)
          if (item.nb[tt] > 0) ++cnt[tt];
      }
      PROF_DUMP(16, 8, blockIdx.x == 0 && lane == 0)
    }
  } else if (warp < kWarpEpilogue) {
    // ---------------- softmax of tile tt: thread r owns row r ----------------
    set_max_registers_up<kRegsSoftmax>();
    const int tt = (warp - kWarpSoftmax) >> 2;
    const int quarter = warp & 3;   // the TMEM lanes a warp may touch: 32 * (warp % 4)
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + tt * kTileN;
    const uint32_t o_tmem = tmem_base + lane_base + kOCol + tt * kTileN;
    const float c = p.scale_log2;
    bool ok = true;
    int cnt = 0, blk = 0;
    PROF_DECL(8)
    TRACE_DECL
    for (int it = 0, t = nth_item(0); t < num_items && ok; ++it, t = nth_item(it)) {
      const Item item = item_at(t);
      const int nbt = item.nb[tt];
      if (nbt == 0) continue;
      const int q0 = item.q0[tt];
      const int row = q0 + r;
      const int limit = p.causal ? min(row, p.seq_kv - 1) : p.seq_kv - 1;   // last visible column
      float m_all = -INFINITY;    // largest scaled score seen so far
      float ref = -INFINITY;      // the reference P and O are in terms of
      float l_sum = 0.0f;         // row sum in terms of ref

      for (int n = 0; n < nbt && ok; ++n, ++blk) {
        PROF_LAP(0)
        ok = mbar_wait_nocall(smem_u32(&sh.s_full[tt]), blk & 1, ctx, ST_ATTN_S_FULL, blk);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        PROF_LAP(1)
        TRACE(tt, 0, r == 0)      // S seen
        const int kv0 = n * kTileN;
        const bool edge = (p.causal && kv0 + kTileN - 1 > q0) || (kv0 + kTileN > p.seq_kv);

        // the 128 scores of the row: read once, kept in registers for both steps
        uint32_t s[4][32];
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
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(s[q][i]),
                                     __uint_as_float(s[q][i + 1]));
        m_all = fmaxf(m_all, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * c);
        PROF_LAP(2)
        const float ref_before = ref;
        if (m_all - ref > kRescaleThreshold) ref = m_all;   // false while m_all is -inf
        if (n > 0 && __any_sync(0xffffffffu, ref != ref_before)) {
          // O_t holds the products up to block n-1 in terms of the old reference; they have
          // retired (the commit behind s_full covers them) and PV_t(n) waits for this block's P
          const float alpha = (ref != ref_before && ref_before > -INFINITY) ? exp2_approx(ref_before - ref) : 1.0f;
#pragma unroll
          for (int q = 0; q < D / 32; ++q) {
            uint32_t o[32];
            tmem_ld_32x32(o_tmem + q * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_tmem + q * 32, o);
          }
          tmem_st_wait();
          l_sum *= alpha;
        }
        PROF_LAP(3)
        TRACE(tt, 1, r == 0)      // max known

        // P = 2^(S * scale - ref), packed in pairs over the first 64 columns of the buffer; each
        // half (64 KV rows) is handed to the PV product as soon as it is written
        const float m_use = ref > -INFINITY ? ref : 0.0f;   // a row that sees nothing at all
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
          // columns [32h, 32h+32) of the buffer; every score is in registers by now
          tmem_st_32x32(s_tmem + h * 32, pk);
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh.p_full[tt][h]));
          PROF_LAP(4 + h)
          TRACE(tt, 2 + h, r == 0)  // P half h signalled
        }
        float s0, s1, s2, s3;
        unpack2(sum2[0], s0, s1);
        unpack2(sum2[1], s2, s3);
        l_sum += (s0 + s1) + (s2 + s3);
#ifdef NB200_ATTN_PROFILE
        prof_acc[7] += 1;
#endif
      }
      if (!ok) break;

      // hand the row sums to the epilogue (its previous read must be over) and go on
      ok = mbar_wait_nocall(smem_u32(&sh.l_empty[tt]), (cnt & 1) ^ 1, ctx, ST_ATTN_L_EMPTY, it);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      sh.row_sum[tt][r] = l_sum;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh.l_full[tt]));
      ++cnt;
      PROF_LAP(6)
    }
    PROF_DUMP(8 * tt, 8, blockIdx.x == 0 && r == 0)
  } else {
    // ---------------- epilogue: O_t / l_t -> global, one rounding ----------------
    set_max_registers_down<kRegsEpilogue>();
    using OutT = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    bool ok = true;
    int cnt[2] = {0, 0};
    for (int it = 0, t = nth_item(0); t < num_items && ok; ++it, t = nth_item(it)) {
      const Item item = item_at(t);
#pragma unroll
      for (int tt = 0; tt < 2; ++tt) {
        if (item.nb[tt] == 0 || !ok) continue;
        ok = mbar_wait_nocall(smem_u32(&sh.l_full[tt]), cnt[tt] & 1, ctx, ST_ATTN_L_FULL, it) &&
             mbar_wait_nocall(smem_u32(&sh.o_full[tt]), cnt[tt] & 1, ctx, ST_ATTN_O_FULL, it);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++cnt[tt];
        tc_fence_after_sync();
        const float inv = 1.0f / sh.row_sum[tt][r];
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.l_empty[tt]));

        const int row = item.q0[tt] + r;
        const uint32_t o_tmem = tmem_base + lane_base + kOCol + tt * kTileN;
        OutT* orow = static_cast<OutT*>(p.o) + (long long)item.head * p.o_head_stride +
                     (long long)row * p.o_row_stride;
        const bool vec = ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
#pragma unroll
        for (int q = 0; q < D / 32; ++q) {
          uint32_t o[32];
          tmem_ld_32x32(o_tmem + q * 32, o);
          tmem_ld_wait();
          if (q == D / 32 - 1) {
            // O_t is in registers: the next pair's first PV_t may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.o_empty[tt]));
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
                for (int e8 = 0; e8 < 8; ++e8) dst[e8] = e[e8];
              }
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
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ------------------------------------------------------------------------

template <int D>
int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                const AttnParams& p, bool bf16, cudaStream_t stream) {
  const int smem = (2 + kKvSlots) * (D / 64) * 128 * 128 + (int)sizeof(AttnShared);
  // persistent: one CTA per SM, never more than there are couples of work items
  int grid = device_info().sm_count;
  const long long items = (long long)p.bh * ((p.n_q_tiles + 1) / 2);
  const long long couples = (items + 1) / 2;
  if (couples < grid) grid = (int)couples;
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

#ifdef NB200_ATTN_PROFILE
extern "C" int nb200_debug_read(long long* out) {
  return cuda_check(cudaMemcpyFromSymbol(out, g_attn_prof, sizeof(long long) * 32), "profile read");
}
extern "C" int nb200_debug_trace(long long* out) {
  return cuda_check(cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(long long) * 3 * 512 * 2), "trace read");
}
#endif

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
  p.wait_limit_ns = wait_limit_ns();
  p.status = device_status_ptr();
  if (!p.status) return fail(NB200_E_CUDA, "attention: device status word is not addressable");
  if ((int64_t)p.bh * p.n_q_tiles > INT32_MAX)
    return fail(NB200_E_INVALID, "attention: too many tiles for one launch");

  if (d == 128) return launch_attn<128>(tq, tk, tv, p, bf16, stream);
  return launch_attn<64>(tq, tk, tv, p, bf16, stream);
}
