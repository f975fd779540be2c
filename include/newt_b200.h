/*
 * newt_b200 -- C ABI of the sm_100a kernel library behind the newt / deuteron
 * operator API.
 *
 * The reference project (arpitsinghgautam/newt) has no C ABI of its own: its
 * boundary is `cuLaunchKernel` on a kernel that its compiler generated as text
 * (newt/runtime/cuda.py:216-234, newt/runtime/jit.py:190-223).  Every entry
 * point below therefore names the *user-level kernel* of the reference whose
 * generated code it replaces, and the launcher call it stands in for.
 *
 * Conventions
 *   - all pointers are DEVICE pointers owned by the caller, unless the name
 *     ends in `_host`;
 *   - sizes and strides are in ELEMENTS, int64;
 *   - `stream` is a CUstream / cudaStream_t passed as void* (NULL = default);
 *   - the return value is 0 on success, else one of NB200_E_*; a message for
 *     the last failure on the calling thread is available from
 *     nb200_last_error();
 *   - nothing here allocates device memory unless its comment says so.
 */
#ifndef NEWT_B200_H
#define NEWT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB200_ABI_VERSION 1

enum nb200_error {
  NB200_OK = 0,
  NB200_E_INVALID = 1,     /* bad argument (size, alignment, dtype, config)   */
  NB200_E_UNSUPPORTED = 2, /* legal request that no kernel here covers yet    */
  NB200_E_CUDA = 3,        /* CUDA runtime / driver call failed               */
  NB200_E_DEVICE = 4       /* a kernel reported a bounded-wait expiry         */
};

enum nb200_dtype {
  NB200_F32 = 0,
  NB200_F16 = 1,
  NB200_BF16 = 2
};

/* Library / ABI identification.  No reference counterpart. */
int nb200_abi_version(void);
const char* nb200_last_error(void);

/* Reads and clears the per-device status word that kernels with bounded waits
 * (mbarrier / TMEM allocation spins) set when a wait expires.  Synchronises
 * the device.  Returns 0 and *status = 0 when every kernel finished normally.
 * Stands where the reference has nothing: a hung kernel there is a hung GPU. */
int nb200_read_status(uint32_t* status, uint32_t* detail);

/* Sets an integer tuning knob by name (0 = back to the built-in heuristic).
 * Plays the role of the launch keywords `num_warps` / `num_stages` of the
 * operator API (newt/runtime/jit.py:169-174) for choices the library would
 * otherwise make itself:
 *   "row_tpr"          threads that cooperate on one row (32,128,256,512,1024)
 *   "row_items"        16-byte vectors each of those threads holds (1,2,4,8)
 *   "row_ctas_per_sm"  resident CTAs per SM of the persistent row grid
 *   "row_rpb"          rows that share one CTA (1, 2 or 4)
 *   "row_force_slow"   1: the row kernels' element-wise path even where rows are vector-friendly
 *   "add_variant"      K0's walk: 1 persistent grid x4 loads, 2 chunks in address order x4
 *                      (the default), 3 chunks x8, 4 persistent x8
 *   "tf32_in_place"    0: nb200_gemm_tf32 always transposes B into its workspace
 *   "gemm_group_m"     row-blocks per band of the GEMM tile order (L2 reuse of B columns; 16)
 *   "gemm_split_tail"  see nb200_gemm_split
 *   "gemm_c_tma"       negative: the GEMM epilogue stores C with the SMs' own 16-byte stores even where
 *                      C could be a tensor map for the copy engine (16-byte aligned base and pitch)
 *   "gemm_half_tail"   256 x 512 tiles: 1 = the last ring of k steps finishes columns 0..255 first (their
 *                      way out to C then overlaps the MMAs of columns 256..511), 2 = the first ring
 *                      starts with them as well (the default from 32 k steps up), negative = neither
 *   "wait_limit_us"    how long one device-side wait (an mbarrier spin of the tensor-core
 *                      kernels) may last before the kernel gives up, records a code in the
 *                      status word and returns; 2 000 000 (2 s) when unset */
int nb200_set_tuning(const char* key, int value);

/* Diagnostic: launches one warp that waits, with the current "wait_limit_us", on a barrier
 * nothing will ever signal.  The wait runs out, the kernel records status code 6 with
 * `detail` as given and returns by itself -- nothing traps, nothing spins for ever.  Lets a
 * caller (and the tests) see the failure path end to end: nb200_read_status() afterwards
 * reports NB200_E_DEVICE once, then is clean again, and the device stays usable.  No
 * reference counterpart. */
int nb200_selftest_wait_timeout(uint32_t detail, void* stream);

/* ---- K0: out = x + y -------------------------------------------------------
 * Replaces the code generated for `add_kernel`
 * (examples/01_vector_add.py:14-21; launcher :27-28). fp32, bit-exact. */
int nb200_add_f32(const float* x, const float* y, float* out, int64_t n,
                  void* stream);

/* ---- K1: row softmax -------------------------------------------------------
 * Replaces the code generated for `softmax_kernel`
 * (examples/02_fused_softmax.py:15-24; launcher :27-33): per row
 * max-subtract, expf, sum, true division; fp32 in/out.
 * `rows` programs, `n` valid columns, row strides in elements. */
int nb200_softmax_f32(const float* x, float* out, int64_t rows, int64_t n,
                      int64_t stride_x, int64_t stride_out, void* stream);

/* ---- K2: layernorm forward -------------------------------------------------
 * Replaces the code generated for `layernorm_kernel`
 * (examples/03_layernorm.py:13-27; launcher :30-36): two-pass statistics in
 * fp32 (mean, then variance of the centred row), rsqrtf(var + eps),
 * y = (x - mean) * rstd * w + b, one rounding at the store.
 * `dtype` is the element type of x, w, b and out (NB200_F32/F16/BF16). */
int nb200_layernorm(const void* x, const void* w, const void* b, void* out,
                    int64_t rows, int64_t n, int64_t stride_x,
                    int64_t stride_out, float eps, int dtype, void* stream);

/* ---- K3 / K4: C = A @ B ----------------------------------------------------
 * Replaces the code generated for `matmul_kernel`
 * (examples/04_matmul.py:14-45, benchmarks/bench.py:90-108) and for the
 * deuteron tile loop (examples/deuteron/01_matmul.py:12-18), i.e. what
 * `nl.dot` lowers to (newt/compiler/codegen.py:2174-2418).
 * A is [M,K] with row stride lda, B is [K,N] with row stride ldb, C is [M,N]
 * with row stride ldc; innermost strides are 1.  fp16 or bf16 inputs, fp32
 * accumulation in tensor memory, one rounding to `dtype` at the store.
 * fp32 inputs run as tf32 with an fp32 result, as `nl.dot` does for fp32 blocks
 * (newt/language.py:165-167, newt/compiler/codegen.py:2195-2197): like the 16-bit
 * types, nb200_gemm reads an fp32 B in place (an MN-major operand; its base and row
 * pitch must be 16-byte aligned, as for every operand).  nb200_gemm_tf32 below also
 * takes a B that is not.
 *
 * The config mirrors the launch knobs of the operator API: the tile comes
 * from the kernel's BLOCK_M/BLOCK_N/BLOCK_K constexprs, `stages` from
 * `num_stages` (depth of the TMA/mbarrier ring), `cta_pair` selects 2-CTA
 * tcgen05 (cluster of two CTAs sharing one 256-row MMA).  Zero fields mean
 * "library default": CTA pairs when the problem has at least one 256x256 tile
 * per pair of SMs -- 256x512 tiles (two MMAs per K step, 64-element K slots) when
 * the rounds those need over the resident pairs cost less than the rounds of
 * 256x256 tiles (128-element K slots) do -- and single-CTA 128xN tiles otherwise. */
typedef struct nb200_gemm_config {
  int32_t block_m; /* 128 (one CTA) or 256 (CTA pair)                        */
  int32_t block_n; /* 64, 128 or 256; a CTA pair takes 256 or 512            */
  int32_t block_k; /* 64; a CTA pair also takes 128 (default) and 192 (fp32: 32 / 64 / 96) */
  int32_t stages;  /* 1..8; snapped to a depth that fits 227 KB of shared mem */
  int32_t cta_pair;/* 0 or 1                                                 */
  int32_t reserved[3];
} nb200_gemm_config;

int nb200_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n,
               int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int dtype,
               const nb200_gemm_config* config, void* stream);

/* The same product with B given transposed: `bt` is [N,K] with row stride ldbt, i.e. what
 * `nl.dot(a, nl.trans(bt_tile))` computes (nl.trans: newt/compiler/codegen.py:1824-1852) or a
 * matmul_kernel called with stride_bk = 1.  All three dtypes. */
int nb200_gemm_bt(const void* a, const void* bt, void* c, int64_t m, int64_t n,
                  int64_t k, int64_t lda, int64_t ldbt, int64_t ldc, int dtype,
                  const nb200_gemm_config* config, void* stream);

/* fp32 C = A @ B with B as [K,N] (the layout of tests/test_matmul.py:67-70 and of
 * bench_matmul_tf32, benchmarks/bench.py:291-294) whatever B's base and pitch: a B that bulk
 * tensor copies can fetch (16-byte aligned base and row pitch) is read in place, exactly as
 * nb200_gemm does; any other is first transposed into `workspace`, a caller-owned device
 * buffer of at least nb200_gemm_tf32_workspace_bytes(n, k) bytes, 16-byte aligned, which the
 * call may overwrite completely, and the product then runs as nb200_gemm_bt (the transposing
 * pass moves 8 bytes per element of B).  Knob `tf32_in_place` = 0 forces the transposing
 * pass. */
int64_t nb200_gemm_tf32_workspace_bytes(int64_t n, int64_t k);
int nb200_gemm_tf32(const void* a, const void* b, void* c, int64_t m, int64_t n,
                    int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                    const nb200_gemm_config* config, void* workspace,
                    int64_t workspace_bytes, void* stream);

/* nb200_gemm_tf32 -- the product `nl.dot` of fp32 blocks stands for (newt/language.py:165-167:
 * tf32 operands, fp32 accumulation; generated at newt/compiler/codegen.py:2474-2487) -- for
 * callers that cannot bring a workspace.  (The entry point itself has no counterpart in the
 * reference, whose generated kernels never need scratch memory.)  A drop-in behind the
 * reference's launcher is such a caller: `JITFunction._run` hands a kernel nothing but the
 * user's own tensors and scalars (newt/runtime/jit.py:166-223) and the package allocates no
 * device memory of its own, so there is no allocator to ask; the same goes for a host that has
 * given all device memory to its own pool, where a cudaMalloc from a plug-in fails or stalls
 * the device.  The transposed copy of B goes into a 4 MiB array inside the library image
 * (held by every GPU that loads the library until the process exits), so the product is
 * limited to n * round_up(k, 4) <= 1048576 (e.g. 1024 x 1024; a k that is a multiple of 8192
 * counts 32 more, see nb200_gemm_tf32_workspace_bytes); larger ones are refused with
 * NB200_E_UNSUPPORTED and the limit in the message.  The call allocates nothing.  Its first
 * call on a device looks up the array's device address (once per device; make that first
 * call outside any stream capture).  The address is remembered per device ordinal, for the
 * device's primary context (the one the CUDA runtime and torch use): it is not valid after a
 * cudaDeviceReset, nor for a second context created on the same device through the driver
 * API.  All calls on a device share the array and each
 * overwrites what the last one left there -- nothing in it needs clearing, the product reads
 * only what its own transposing pass wrote -- so two calls that overlap on the GPU (different
 * streams, no dependency between them) race; calls on one stream are ordered and safe. */
int nb200_gemm_tf32_static(const void* a, const void* b, void* c, int64_t m, int64_t n,
                           int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                           const nb200_gemm_config* config, void* stream);

/* nb200_gemm / nb200_gemm_bt (b_transposed != 0) with a split tail.  The CTA-pair kernels hand
 * tiles out whole, one per pair and round; when the last round would fill at most half of the
 * chip -- above all a small C with a long K: 1024 x 1024 x 16384 is 16 tiles for 74 pairs -- the
 * tiles of that round are instead cut along K into as many equal parts as there are pairs per
 * tile (the same stretches of K for every tile, so pairs that read the same rows of A or columns
 * of B run side by side and share them in L2), a part leaves its fp32 partial sums in
 * `workspace`, and a second kernel on the same stream adds the parts of each tile and stores C.
 * The parts are always added in the same order, so results do not vary from run to run (they
 * differ from the unsplit product by fp32 reassociation only).  Measured on a B200, bf16, whole
 * tiles -> split / torch.matmul, us: 1024 x 1024 x 16384  84 -> 44 / 43;  512 x 512 x 65536
 * 297 -> 48 / 56;  256 x 256 x 65536  297 -> 32 / 38;  4096^3 in 256 x 256 tiles  96 -> 93 / 94.
 * The reference has no counterpart: its matmul_kernel (examples/04_matmul.py:16-45) owns one
 * tile per program.
 * `workspace`: 16-byte aligned device memory of at least
 * nb200_gemm_split_workspace_bytes(m, n, k, dtype, config) bytes, the caller's; nothing in it
 * needs clearing, and it must not be shared by launches that can overlap on the GPU.  The query
 * returns 0 when the tiles of this problem stay whole: single-CTA tiles, a last round more than
 * half full, or a split that would cost more in partial sums than it saves in idle k steps
 * (fewer than ~28 per pair); with a null or smaller workspace the call is nb200_gemm /
 * nb200_gemm_bt.  With `config` null or all zeros the library takes 256 x 256 pair tiles where
 * that makes a split pay (the default of nb200_gemm gives a small C single-CTA tiles).  Knob "gemm_split_tail": 1 = split whenever a part still has four k steps,
 * negative = never, 0 = by the measured costs. */
int64_t nb200_gemm_split_workspace_bytes(int64_t m, int64_t n, int64_t k, int dtype,
                                         const nb200_gemm_config* config);
int nb200_gemm_split(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                     int64_t lda, int64_t ldb, int64_t ldc, int dtype, int b_transposed,
                     const nb200_gemm_config* config, void* workspace, int64_t workspace_bytes,
                     void* stream);

/* nb200_gemm / nb200_gemm_bt (b_transposed != 0) for fp16 or bf16 operands with C taking the
 * fp32 accumulator unrounded: C is float [M, N] with row stride ldc.  What a matmul with an
 * epilogue fused after its k loop needs (bias, activation, scaling applied to the fp32
 * accumulator before the one rounding at the store, newt/compiler/codegen.py:1718-1723): the
 * product runs here, the epilogue reads C. */
int nb200_gemm_acc32(const void* a, const void* b, float* c, int64_t m, int64_t n, int64_t k,
                     int64_t lda, int64_t ldb, int64_t ldc, int dtype, int b_transposed,
                     const nb200_gemm_config* config, void* stream);

/* The host half of nb200_gemm / nb200_gemm_bt without the launch, for a kernel compiled at run
 * time from the library's own device templates (csrc/gemm_device.cuh) with code of the
 * caller's spliced into the epilogue -- what the reference does for everything after a k loop
 * (newt/compiler/codegen.py:1854-1871, tests/test_ops.py:458-474).  Validates the problem as
 * nb200_gemm does, resolves `config`, encodes the two tensor maps into `tensor_map_a` /
 * `tensor_map_b` (128 bytes each, 64-byte aligned), fills `params` (the kernels' GemmParams; at
 * least nb200_gemm_params_bytes() bytes) and says in `launch` which template instance to
 * compile and how to launch it.  `c_dtype` is the element type of C (any of the three codes);
 * fp16 / bf16 operands only.  The kernel wrapper takes the two tensor maps and the parameter
 * block as `const __grid_constant__` parameters: the block holds the tensor map of C that the
 * epilogue's copies read, and a tensor map has to be read from where the launch put it, not
 * from a thread's copy. */
typedef struct nb200_gemm_launch {
  int32_t pair;        /* 1: gemm_pair_body<stages, ksub, ..> in clusters of two; 0: gemm_body<block_n, stages, ..> */
  int32_t block_n, stages, ksub;
  int32_t grid, block, cluster; /* CTAs, threads per CTA, CTAs per cluster (1: no cluster) */
  int32_t smem_bytes;  /* dynamic shared memory per CTA */
  int32_t nothing;     /* 1: C is empty, nothing to launch */
  int32_t only_clear;  /* 1: K == 0, C is all zeros and nothing is to be launched */
  int32_t reserved[6];
} nb200_gemm_launch;
int64_t nb200_gemm_params_bytes(void);
int nb200_gemm_plan(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                    int64_t lda, int64_t ldb, int64_t ldc, int dtype, int c_dtype, int b_transposed,
                    const nb200_gemm_config* config, void* tensor_map_a, void* tensor_map_b,
                    void* params, nb200_gemm_launch* launch);

/* dst[r][c] = src[r * row_stride + c * col_stride] for 2- or 4-byte elements (strides and
 * dst_pitch in elements): copies a matrix given with any two strides -- a row pitch that is
 * not a multiple of 16 bytes, a misaligned base, a transposed A -- into a row-major buffer
 * the caller owns, so that nb200_gemm can fetch it.  (No counterpart in the reference, whose
 * cp.async staging takes any stride, newt/compiler/codegen.py:2560-2654; bulk tensor copies do
 * not.)  Moves 2 * elem_bytes per element. */
int nb200_repitch(const void* src, void* dst, int64_t rows, int64_t cols, int64_t row_stride,
                  int64_t col_stride, int64_t dst_pitch, int elem_bytes, void* stream);

/* Returns 0 when (dtype, shape, strides, pointers, config) can run on the
 * TMA/tcgen05 path, else NB200_E_* with the reason in nb200_last_error().
 * Launches nothing; lets an autotuner discard configurations analytically
 * (the reference discards them by catching launch failures,
 * newt/runtime/autotuner.py:76-81).  For NB200_F32 it answers for nb200_gemm_tf32 (B as
 * [K,N], any pitch). */
int nb200_gemm_check(const void* a, const void* b, const void* c, int64_t m,
                     int64_t n, int64_t k, int64_t lda, int64_t ldb,
                     int64_t ldc, int dtype, const nb200_gemm_config* config);

/* ---- K5: fused attention forward -------------------------------------------
 * Replaces the code generated for `attention_kernel`
 * (examples/05_fused_attention.py:14-48), extended to batch x heads and an
 * optional causal mask: O = softmax(scale * Q K^T [+ causal]) V with an fp32
 * online softmax; P is rounded to the input dtype before the PV product, as
 * the reference does at :43.
 * Q,O are [batch*heads, seq_q, d]; K,V are [batch*heads, seq_kv, d]; the
 * three strides of each tensor are (head stride, row stride, 1). d = 64/128. */
int nb200_attention_fwd(const void* q, const void* k, const void* v, void* o,
                        int64_t batch_heads, int64_t seq_q, int64_t seq_kv,
                        int64_t d, int64_t q_head_stride, int64_t q_row_stride,
                        int64_t k_head_stride, int64_t k_row_stride,
                        int64_t v_head_stride, int64_t v_row_stride,
                        int64_t o_head_stride, int64_t o_row_stride,
                        float scale, int causal, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NEWT_B200_H */
