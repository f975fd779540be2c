// Row programs of the newt operator API as hand-written sm_100a kernels:
//   K0  out = x + y                      (examples/01_vector_add.py:14-21)
//   K1  fused row softmax, fp32          (examples/02_fused_softmax.py:15-24)
//   K2  layernorm forward                (examples/03_layernorm.py:13-27)
//
// One template serves K1 and K2.  A row is held entirely in registers: every
// thread owns ITEMS 16-byte vectors, interleaved so that a warp reads 512
// contiguous bytes per load instruction (the reference reaches the same access
// shape through a runtime-checked fast path, newt/compiler/codegen.py:1631-1680).
// TPR threads cooperate on one row (32 = one row per warp, no shared memory;
// more = one row per CTA with a two-level shuffle + shared-memory reduction),
// RPB rows are packed per CTA.  The grid is persistent: it is sized to the
// number of CTAs the device can hold and each CTA walks rows with a stride,
// loading the next row's vectors before it reduces the current one, so the
// reductions of one row overlap the HBM latency of the next.
//
// All of this is HBM-bound streaming work; nothing here uses tensor cores.

#include "common.cuh"

namespace nb200 {
namespace {

constexpr int kWarp = 32;

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerVec = 4;
  __device__ static float to_f32(float v) { return v; }
  __device__ static float from_f32(float v) { return v; }
};
template <>
struct Elem<__half> {
  static constexpr int kPerVec = 8;
  __device__ static float to_f32(__half v) { return __half2float(v); }
  __device__ static __half from_f32(float v) { return __float2half_rn(v); }
  __device__ static uint32_t pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerVec = 8;
  __device__ static float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
  __device__ static uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};

// One 16-byte vector of T, addressable both ways.
template <typename T>
union alignas(16) Vec {
  uint4 raw;
  T e[Elem<T>::kPerVec];
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Loads the vector that covers columns [col, col + kPerVec) of a row.  Lanes
// past `n` get `fill`.  `vec_ok` says the row base is 16-byte aligned.
// FAST is the launch-time promise that every row base is 16-byte aligned and
// that n is a multiple of the vector width, so a vector is either entirely
// inside the row or entirely padding and no element-wise fallback is compiled.
template <typename T, bool FAST = false>
__device__ __forceinline__ Vec<T> load_vec(const T* row, int col, int n, bool vec_ok, T fill) {
  constexpr int E = Elem<T>::kPerVec;
  Vec<T> v;
  if ((FAST || vec_ok) && col + E <= n) {
    v.raw = ld_stream(row + col);
  } else {
#pragma unroll
    for (int j = 0; j < E; ++j) v.e[j] = (!FAST && col + j < n) ? row[col + j] : fill;
  }
  return v;
}

template <typename T, bool FAST = false>
__device__ __forceinline__ void store_vec(T* row, int col, int n, bool vec_ok, const Vec<T>& v) {
  constexpr int E = Elem<T>::kPerVec;
  if ((FAST || vec_ok) && col + E <= n) {
    st_stream(row + col, v.raw);
  } else if constexpr (!FAST) {
#pragma unroll
    for (int j = 0; j < E; ++j)
      if (col + j < n) row[col + j] = v.e[j];
  }
}

struct SumOp {
  __device__ static float apply(float a, float b) { return a + b; }
};
struct MaxOp {
  __device__ static float apply(float a, float b) { return fmaxf(a, b); }
};

// Reduction over the TPR threads of one row.  For TPR > 32 the per-warp
// results meet in `slot` (one float per warp of the row) behind a named barrier
// that only the row's own TPR threads join, so several rows can share a CTA.
// Callers alternate between two slots, which makes one barrier per reduction
// enough.
template <class Op, int TPR>
__device__ __forceinline__ float row_reduce(float v, float* slot, int barrier_id) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (TPR > kWarp) {
    constexpr int W = TPR / kWarp;
    const int warp_in_row = (threadIdx.x % TPR) / kWarp;
    if ((threadIdx.x & 31) == 0) slot[warp_in_row] = v;
    asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "n"(TPR) : "memory");
    v = slot[0];
#pragma unroll
    for (int w = 1; w < W; ++w) v = Op::apply(v, slot[w]);
  }
  return v;
}

// exp(t) for t <= 0 as 2^(t * log2 e) on the special-function unit.  The
// product is formed with the constant split in two so that the rounding of
// log2(e) does not grow with |t|; what remains is the rounding of the product
// itself (half an ulp of |t| * 1.44) and ex2.approx's 2^-22 relative error:
// below 3e-6 relative for every finite input, against the 1e-5 bar.
__device__ __forceinline__ float exp_neg(float t) {
  constexpr float kLog2eHi = 1.44269502162933349609375f;
  constexpr float kLog2eLo = 1.92596299112661746e-8f;
  float y = fmaf(t, kLog2eLo, t * kLog2eHi);
  float r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(r) : "f"(y));
  return r;
}

enum class RowKind { Softmax, LayerNorm };

struct RowParams {
  const void* x;
  const void* w;
  const void* b;
  void* out;
  int rows;
  int n;
  int64_t stride_x;
  int64_t stride_out;
  float eps;
  int wb_in_smem;  // layernorm: weight/bias staged once per CTA in shared memory as fp32
};

// Register budget: a thread holds one row slice as fp32 values plus the raw
// vectors of the next row.  With up to 16 values per thread that fits in 64
// registers (1024 resident threads per SM); 32 values need about 80 (768
// threads); more get 128 (512 threads).  Every resident thread keeps up to
// 64 bytes of loads in flight, i.e. 48-64 KB per SM, above the ~35 KB that HBM
// latency x bandwidth needs.
template <int VALUES, int THREADS>
struct RowOccupancy {
  static constexpr int kThreadsPerSm = VALUES <= 16 ? 1024 : (VALUES <= 32 ? 768 : 512);
  static constexpr int kMinBlocks = kThreadsPerSm / THREADS > 0 ? kThreadsPerSm / THREADS : 1;
};

template <RowKind KIND, typename T, int ITEMS, int TPR, int RPB, bool FAST>
__global__ void __launch_bounds__(TPR* RPB, RowOccupancy<ITEMS * Elem<T>::kPerVec, TPR * RPB>::kMinBlocks)
    row_kernel(RowParams p) {
  constexpr int E = Elem<T>::kPerVec;
  constexpr int W = TPR > kWarp ? TPR / kWarp : 1;
  __shared__ float red[RPB][2][W];
  extern __shared__ float4 wb_smem[];  // fp32 weight then bias, as float4 [ITEMS][E/4][TPR] each

  const int lane_in_row = threadIdx.x % TPR;
  const int row_in_cta = threadIdx.x / TPR;
  const int n = p.n;
  const bool full = n == ITEMS * TPR * E;  // no padded lanes: predicates drop out
  const T* x = static_cast<const T*>(p.x);
  T* out = static_cast<T*>(p.out);
  const T fill = Elem<T>::from_f32(KIND == RowKind::Softmax ? -INFINITY : 0.0f);
  const T* w = static_cast<const T*>(p.w);
  const T* b = static_cast<const T*>(p.b);
  bool w_ok = false, b_ok = false;

  if constexpr (KIND == RowKind::LayerNorm) {
    w_ok = (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    b_ok = (reinterpret_cast<uintptr_t>(b) & 15) == 0;
    if (p.wb_in_smem) {
      // consecutive threads own consecutive float4 slots: no bank conflicts
      float4* ws4 = wb_smem;
      float4* bs4 = wb_smem + ITEMS * (E / 4) * TPR;
      if (row_in_cta == 0) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const int col = (i * TPR + lane_in_row) * E;
          const Vec<T> wv = load_vec<T, FAST>(w, col, n, w_ok, Elem<T>::from_f32(0.0f));
          const Vec<T> bv = load_vec<T, FAST>(b, col, n, b_ok, Elem<T>::from_f32(0.0f));
#pragma unroll
          for (int h = 0; h < E / 4; ++h) {
            const int slot = (i * (E / 4) + h) * TPR + lane_in_row;
            ws4[slot] = make_float4(Elem<T>::to_f32(wv.e[4 * h]), Elem<T>::to_f32(wv.e[4 * h + 1]),
                                    Elem<T>::to_f32(wv.e[4 * h + 2]), Elem<T>::to_f32(wv.e[4 * h + 3]));
            bs4[slot] = make_float4(Elem<T>::to_f32(bv.e[4 * h]), Elem<T>::to_f32(bv.e[4 * h + 1]),
                                    Elem<T>::to_f32(bv.e[4 * h + 2]), Elem<T>::to_f32(bv.e[4 * h + 3]));
          }
        }
      }
      __syncthreads();
    }
  }

  const int step = gridDim.x * RPB;
  int row = blockIdx.x * RPB + row_in_cta;
  Vec<T> nxt[ITEMS];
  if (row < p.rows) {
    const T* xr = x + (int64_t)row * p.stride_x;
    const bool ok = (reinterpret_cast<uintptr_t>(xr) & 15) == 0;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
      nxt[i] = load_vec<T, FAST>(xr, (i * TPR + lane_in_row) * E, n, ok, fill);
  }
  float* red0 = red[row_in_cta][0];
  float* red1 = red[row_in_cta][1];
  const int bar_id = 1 + row_in_cta;

  // The TPR threads of a row always agree on `row`, so the loop condition is
  // uniform across everyone who joins the row's named barrier.
  for (; row < p.rows; row += step) {
    float v[ITEMS * E];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
#pragma unroll
      for (int j = 0; j < E; ++j) v[i * E + j] = Elem<T>::to_f32(nxt[i].e[j]);

    // put the next row's loads in flight before reducing this one
    const int next = row + step;
    if (next < p.rows) {
      const T* xr = x + (int64_t)next * p.stride_x;
      const bool ok = (reinterpret_cast<uintptr_t>(xr) & 15) == 0;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i)
        nxt[i] = load_vec<T, FAST>(xr, (i * TPR + lane_in_row) * E, n, ok, fill);
    }

    T* orow = out + (int64_t)row * p.stride_out;
    const bool out_ok = (reinterpret_cast<uintptr_t>(orow) & 15) == 0;

    if constexpr (KIND == RowKind::Softmax) {
      float m = v[0];
#pragma unroll
      for (int k = 1; k < ITEMS * E; ++k) m = fmaxf(m, v[k]);
      m = row_reduce<MaxOp, TPR>(m, red0, bar_id);
      float s = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS * E; ++k) {
        v[k] = exp_neg(v[k] - m);  // masked lanes hold -inf and give 0
        s += v[k];
      }
      s = row_reduce<SumOp, TPR>(s, red1, bar_id);
      // one reciprocal per row, then a multiply per element: within 1.5 ulp of
      // the reference's per-element division
      const float inv = 1.0f / s;
#pragma unroll
      for (int k = 0; k < ITEMS * E; ++k) v[k] *= inv;
    } else {
      const float fn = (float)n;
      float s = 0.0f;
#pragma unroll
      for (int k = 0; k < ITEMS * E; ++k) s += v[k];  // masked lanes hold 0
      const float mean = row_reduce<SumOp, TPR>(s, red0, bar_id) / fn;
      float q = 0.0f;
      if (full) {
#pragma unroll
        for (int k = 0; k < ITEMS * E; ++k) {
          v[k] -= mean;
          q = fmaf(v[k], v[k], q);
        }
      } else {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
#pragma unroll
          for (int j = 0; j < E; ++j) {
            // FAST: a vector is all row or all padding, one test per vector
            const int col = (i * TPR + lane_in_row) * E + (FAST ? 0 : j);
            const float d = col < n ? v[i * E + j] - mean : 0.0f;
            v[i * E + j] = d;
            q = fmaf(d, d, q);
          }
      }
      const float var = row_reduce<SumOp, TPR>(q, red1, bar_id) / fn;
      const float rstd = rsqrtf(var + p.eps);
      if (p.wb_in_smem) {
        const float4* ws4 = wb_smem;
        const float4* bs4 = wb_smem + ITEMS * (E / 4) * TPR;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
#pragma unroll
          for (int j = 0; j < E; j += 4) {
            const int q4 = (i * (E / 4) + j / 4) * TPR + lane_in_row;
            const float4 wv = ws4[q4], bv = bs4[q4];
            v[i * E + j + 0] = fmaf(v[i * E + j + 0] * rstd, wv.x, bv.x);
            v[i * E + j + 1] = fmaf(v[i * E + j + 1] * rstd, wv.y, bv.y);
            v[i * E + j + 2] = fmaf(v[i * E + j + 2] * rstd, wv.z, bv.z);
            v[i * E + j + 3] = fmaf(v[i * E + j + 3] * rstd, wv.w, bv.w);
          }
      } else {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const int col = (i * TPR + lane_in_row) * E;
          const Vec<T> wv = load_vec<T, FAST>(w, col, n, w_ok, Elem<T>::from_f32(0.0f));
          const Vec<T> bv = load_vec<T, FAST>(b, col, n, b_ok, Elem<T>::from_f32(0.0f));
#pragma unroll
          for (int j = 0; j < E; ++j)
            v[i * E + j] = fmaf(v[i * E + j] * rstd, Elem<T>::to_f32(wv.e[j]),
                                Elem<T>::to_f32(bv.e[j]));
        }
      }
    }

#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      Vec<T> o;
      if constexpr (sizeof(T) == 2) {
        // two lanes per conversion instruction: the scalar cvt.rn.bf16.f32 issues at a fraction
        // of the packed form's rate on sm_100a
        uint32_t* words = reinterpret_cast<uint32_t*>(&o.raw);
#pragma unroll
        for (int j = 0; j < E; j += 2) words[j / 2] = Elem<T>::pack2(v[i * E + j], v[i * E + j + 1]);
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) o.e[j] = Elem<T>::from_f32(v[i * E + j]);
      }
      store_vec<T, FAST>(orow, (i * TPR + lane_in_row) * E, n, out_ok, o);
    }
  }
}

// ---- K0 --------------------------------------------------------------------

__device__ __forceinline__ uint4 add4(uint4 a, uint4 b) {
  uint4 r;
  r.x = __float_as_uint(__uint_as_float(a.x) + __uint_as_float(b.x));
  r.y = __float_as_uint(__uint_as_float(a.y) + __uint_as_float(b.y));
  r.z = __float_as_uint(__uint_as_float(a.z) + __uint_as_float(b.z));
  r.w = __float_as_uint(__uint_as_float(a.w) + __uint_as_float(b.w));
  return r;
}

// U vectors per operand per thread and trip.  PERSISTENT: a grid of as many CTAs as the device
// holds walks the array with a stride; otherwise every CTA takes one chunk of 256 * U vectors
// and the hardware scheduler hands out chunks in address order (what keeps DRAM pages open
// across the three streams).
template <int U, bool PERSISTENT>
__global__ void __launch_bounds__(256) add_f32_kernel(const float* __restrict__ x,
                                                      const float* __restrict__ y,
                                                      float* __restrict__ out, int64_t n,
                                                      int vec_ok) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (vec_ok) {
    const int64_t nvec = n / 4;
    const int64_t stride = PERSISTENT ? nthreads * U : nvec;   // one trip when not persistent
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x * U; base < nvec; base += stride) {
      uint4 a[U], b[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = base + u * blockDim.x + threadIdx.x;
        if (i < nvec) {
          a[u] = ld_stream(x + 4 * i);
          b[u] = ld_stream(y + 4 * i);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = base + u * blockDim.x + threadIdx.x;
        if (i < nvec) st_stream(out + 4 * i, add4(a[u], b[u]));
      }
    }
    for (int64_t i = nvec * 4 + tid; i < n; i += nthreads) out[i] = x[i] + y[i];
  } else {
    for (int64_t i = tid; i < n; i += nthreads) out[i] = x[i] + y[i];
  }
}

// ---- dispatch ----------------------------------------------------------------

struct RowConfig {
  int tpr;
  int items;
};

// Smallest register tile that holds a row of n elements, 16 bytes per vector.
bool pick_row_config(int64_t n, int elems_per_vec, RowConfig* cfg) {
  static const RowConfig table[] = {{32, 1},  {32, 2},  {32, 4},  {32, 8},  {128, 4},
                                    {256, 4}, {256, 8}, {512, 8}, {1024, 8}};
  const int force_tpr = tuning("row_tpr", 0), force_items = tuning("row_items", 0);
  if (force_tpr && force_items) {
    if ((int64_t)force_tpr * force_items * elems_per_vec < n) return false;
    *cfg = {force_tpr, force_items};
    return true;
  }
  for (const RowConfig& c : table)
    if ((int64_t)c.tpr * c.items * elems_per_vec >= n) {
      *cfg = c;
      return true;
    }
  return false;
}

template <RowKind KIND, typename T, int ITEMS, int TPR, int RPB, bool FAST>
int launch_row_variant(const RowParams& p, cudaStream_t stream) {
  auto kern = row_kernel<KIND, T, ITEMS, TPR, RPB, FAST>;
  const DeviceInfo& dev = device_info();
  RowParams q = p;
  size_t smem = 0;
  if (KIND == RowKind::LayerNorm) {
    // weight and bias as fp32, staged once per persistent CTA
    const size_t want_smem = (size_t)2 * ITEMS * TPR * Elem<T>::kPerVec * sizeof(float);
    if (want_smem * RowOccupancy<ITEMS * Elem<T>::kPerVec, TPR * RPB>::kMinBlocks <= 200 * 1024) {
      smem = want_smem;
      q.wb_in_smem = 1;
      if (smem > 48 * 1024) {
        if (int rc = prepare_kernel((const void*)kern, (int)smem)) return rc;
      }
    }
  }
  int per_sm = tuning("row_ctas_per_sm", 0);
  if (per_sm <= 0) {
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, TPR * RPB, smem);
    if (e != cudaSuccess) return cuda_check(e, "occupancy query");
    if (per_sm < 1) per_sm = 1;
  }
  int64_t want = cdiv64(p.rows, RPB);
  int64_t cap = (int64_t)dev.sm_count * per_sm;
  const int grid = (int)(want < cap ? want : cap);
  kern<<<grid, TPR * RPB, smem, stream>>>(q);
  return cuda_check(cudaGetLastError(), "row kernel launch");
}

// FAST needs 16-byte aligned row bases for every tensor and whole vectors only.
template <typename T>
bool rows_are_vector_friendly(const RowParams& p) {
  constexpr int E = Elem<T>::kPerVec;
  auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (p.n % E || p.stride_x % E || p.stride_out % E) return false;
  if (!aligned(p.x) || !aligned(p.out)) return false;
  if (p.w && (!aligned(p.w) || !aligned(p.b))) return false;
  return true;
}

template <RowKind KIND, typename T, int ITEMS, int TPR, int RPB>
int launch_row(const RowParams& p, cudaStream_t stream) {
  if (rows_are_vector_friendly<T>(p) && !tuning("row_force_slow", 0))
    return launch_row_variant<KIND, T, ITEMS, TPR, RPB, true>(p, stream);
  return launch_row_variant<KIND, T, ITEMS, TPR, RPB, false>(p, stream);
}

template <RowKind KIND, typename T>
int dispatch_row(const RowParams& p, cudaStream_t stream) {
  RowConfig c;
  if (!pick_row_config(p.n, Elem<T>::kPerVec, &c))
    return fail(NB200_E_UNSUPPORTED,
                "row of %d elements does not fit the register tile (max %d)", p.n,
                1024 * 8 * Elem<T>::kPerVec);
  // rows per CTA: 4 when a warp owns a row; 2 for 128-thread rows so that a
  // 256-thread CTA shares one staged copy of weight and bias
  const int rpb = tuning("row_rpb", 0);
#define NB200_ROW_CASE(TPR_, ITEMS_, RPB_)                          \
  if (c.tpr == TPR_ && c.items == ITEMS_ && (rpb == 0 || rpb == RPB_)) \
    return launch_row<KIND, T, ITEMS_, TPR_, RPB_>(p, stream);
  NB200_ROW_CASE(32, 1, 4)
  NB200_ROW_CASE(32, 2, 4)
  NB200_ROW_CASE(32, 4, 4)
  NB200_ROW_CASE(32, 8, 4)
  NB200_ROW_CASE(128, 4, 2)
  NB200_ROW_CASE(128, 4, 1)
  NB200_ROW_CASE(128, 8, 1)
  NB200_ROW_CASE(256, 2, 1)
  NB200_ROW_CASE(256, 4, 1)
  NB200_ROW_CASE(256, 8, 1)
  NB200_ROW_CASE(512, 2, 1)
  NB200_ROW_CASE(512, 4, 1)
  NB200_ROW_CASE(512, 8, 1)
  NB200_ROW_CASE(1024, 8, 1)
#undef NB200_ROW_CASE
  return fail(NB200_E_INVALID,
              "no row kernel for threads-per-row=%d vectors-per-thread=%d rows-per-cta=%d", c.tpr,
              c.items, rpb);
}

int check_rows(const void* x, const void* out, int64_t rows, int64_t n) {
  if (rows < 0 || n < 0) return fail(NB200_E_INVALID, "negative size (rows=%lld n=%lld)",
                                     (long long)rows, (long long)n);
  if (rows > INT32_MAX || n > INT32_MAX)
    return fail(NB200_E_INVALID, "rows / n beyond int32 (rows=%lld n=%lld)", (long long)rows,
                (long long)n);
  if (rows > 0 && n > 0 && (!x || !out)) return fail(NB200_E_INVALID, "null tensor pointer");
  return 0;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" int nb200_add_f32(const float* x, const float* y, float* out, int64_t n,
                             void* stream) {
  if (n < 0) return fail(NB200_E_INVALID, "negative length %lld", (long long)n);
  if (n == 0) return 0;
  if (!x || !y || !out) return fail(NB200_E_INVALID, "null tensor pointer");
  const int vec_ok = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                       reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const DeviceInfo& dev = device_info();
  const int threads = 256;
  cudaStream_t st = (cudaStream_t)stream;
  // "add_variant": 0 = default, 1 = persistent x4, 2 = chunked x4, 3 = chunked x8, 4 = persistent x8
  const int variant = tuning("add_variant", 0);
  const int64_t cap = (int64_t)dev.sm_count * 8;
  auto persistent_grid = [&](int u) {
    const int64_t want = cdiv64(vec_ok ? cdiv64(n, 4) : n, threads * u);
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
  };
  auto chunked_grid = [&](int u) -> int64_t { return cdiv64(cdiv64(n, 4), threads * u); };
  if (!vec_ok || variant == 1) {
    add_f32_kernel<4, true><<<persistent_grid(4), threads, 0, st>>>(x, y, out, n, vec_ok);
  } else if (variant == 4) {
    add_f32_kernel<8, true><<<persistent_grid(8), threads, 0, st>>>(x, y, out, n, vec_ok);
  } else if (variant == 3 && chunked_grid(8) <= INT32_MAX) {
    add_f32_kernel<8, false><<<(int)chunked_grid(8), threads, 0, st>>>(x, y, out, n, vec_ok);
  } else if (chunked_grid(4) <= INT32_MAX) {
    add_f32_kernel<4, false><<<(int)chunked_grid(4), threads, 0, st>>>(x, y, out, n, vec_ok);
  } else {
    add_f32_kernel<4, true><<<persistent_grid(4), threads, 0, st>>>(x, y, out, n, vec_ok);
  }
  return cuda_check(cudaGetLastError(), "add_f32 launch");
}

extern "C" int nb200_softmax_f32(const float* x, float* out, int64_t rows, int64_t n,
                                 int64_t stride_x, int64_t stride_out, void* stream) {
  if (int rc = check_rows(x, out, rows, n)) return rc;
  if (rows == 0 || n == 0) return 0;
  RowParams p{x, nullptr, nullptr, out, (int)rows, (int)n, stride_x, stride_out, 0.0f, 0};
  return dispatch_row<RowKind::Softmax, float>(p, (cudaStream_t)stream);
}

extern "C" int nb200_layernorm(const void* x, const void* w, const void* b, void* out,
                               int64_t rows, int64_t n, int64_t stride_x, int64_t stride_out,
                               float eps, int dtype, void* stream) {
  if (int rc = check_rows(x, out, rows, n)) return rc;
  if (rows == 0 || n == 0) return 0;
  if (!w || !b) return fail(NB200_E_INVALID, "null weight / bias pointer");
  RowParams p{x, w, b, out, (int)rows, (int)n, stride_x, stride_out, eps, 0};
  switch (dtype) {
    case NB200_F32:
      return dispatch_row<RowKind::LayerNorm, float>(p, (cudaStream_t)stream);
    case NB200_F16:
      return dispatch_row<RowKind::LayerNorm, __half>(p, (cudaStream_t)stream);
    case NB200_BF16:
      return dispatch_row<RowKind::LayerNorm, __nv_bfloat16>(p, (cudaStream_t)stream);
    default:
      return fail(NB200_E_INVALID, "unknown dtype code %d", dtype);
  }
}
