/*
 * b200ops -- C ABI of the B200 (sm_100a) operator launcher.
 *
 * This library stands where the reference's native call path stands
 * (helion_mlir_backend/_compiler/native/call.cpp): the reference packs memref
 * descriptors and calls a JIT-compiled `void entry(void**)` on the CPU
 * (call.cpp:160-198); here every operator of helion_mlir_utils is one
 * `extern "C"` entry point that validates its operands, enqueues hand-written
 * CUDA kernels on the caller's stream and returns. No entry point synchronises
 * the host, allocates device memory (except the b200_pool_* family) or owns
 * its operands. A bound Python/C caller only needs plain pointers and sizes.
 *
 * Return value of every entry point that returns int:
 *    0                 success (work enqueued)
 *   >0                 refusal: the operands cannot be handled (B200_E_*); like
 *                      the reference's refusals (call.cpp:360-368) nothing ran
 *   <0                 -(cudaError_t) of a failed CUDA runtime call
 * b200_strerror() turns either into text.
 */
#ifndef B200OPS_H_
#define B200OPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200OPS_ABI_VERSION 1

/* Element types of operands. */
enum { B200_F32 = 0, B200_BF16 = 1 };

/* Refusal codes (positive returns). */
enum {
  B200_OK = 0,
  B200_E_DTYPE = 1,     /* unsupported or mismatched element type */
  B200_E_SHAPE = 2,     /* sizes do not fit the operator */
  B200_E_STRIDE = 3,    /* a leading dimension smaller than the row, or not contiguous where required */
  B200_E_ALIGN = 4,     /* pointer alignment the kernel needs is missing */
  B200_E_ALIAS = 5,     /* an output overlaps an input that is not its in-place partner */
  B200_E_NULL = 6,      /* a required pointer is NULL */
  B200_E_ARG = 7,       /* an enum or option value out of range */
  B200_E_WORKSPACE = 8, /* scratch memory missing or too small */
  B200_E_DEVICE = 9,    /* no sm_100 device is current, or the driver entry points are missing */
  B200_E_DISABLED = 10, /* b200_set_enabled(0) was called */
  B200_E_TOO_LARGE = 11 /* a size beyond what a fixed-size resource of the entry point holds */
};

/* Activations fused after the affine part of an epilogue. `alpha` is the
 * negative slope of B200_ACT_LEAKY_RELU and ignored otherwise. */
enum {
  B200_ACT_IDENTITY = 0,
  B200_ACT_RELU = 1,
  B200_ACT_GELU_ERF = 2,
  B200_ACT_GELU_TANH = 3,
  B200_ACT_SIGMOID = 4,
  B200_ACT_TANH = 5,
  B200_ACT_SILU = 6,
  B200_ACT_LEAKY_RELU = 7,
  B200_ACT_COUNT_ = 8
};

/* Operand layouts of b200_gemm. "A" is the M x K operand, "B" the K x N one. */
enum {
  B200_LAYOUT_ROW = 0,           /* A: [M,K] row-major (ld = elements per row); B: [K,N] row-major */
  B200_LAYOUT_COL = 1,           /* A: stored [K,M] (trans_a); B: stored [N,K] (trans_b, nn.Linear weights) */
  B200_LAYOUT_BLOCKED = 2,       /* A: [M/32,K/32,32,32]; B: [N/32,K/32,32(k),32(n)]
                                    (helion_mlir_utils/matmul.py:92-132 pack_a_blocked / pack_b_blocked) */
  B200_LAYOUT_BLOCKED_VNNI = 3,  /* B only: [N/32,K/32,16,32,2], out[j,i,r,n,p]=B[32i+2r+p,32j+n]
                                    (matmul.py:947-958 pack_b_blocked_vnni) */
  B200_LAYOUT_VNNI_PANELS = 4    /* B only: [N/P,K/2,P,2], out[q,c,n,v]=W[qP+n,2c+v]
                                    (matmul.py:1138-1157 pack_b_vnni_t); `b_panel` = P */
};

/*
 * One GEMM / batched GEMM:  C = act(((A @ B) + bias) * scale + shift)
 *
 * Replaces the compiled bodies of helion_mlir_utils/matmul.py:
 *   _matmul_fused_pack (259-328), _matmul_f32_fused_pack (1302-1370),
 *   _matmul_blocked_kernel/_bias/_affine (156-228, 862-904),
 *   _matmul_prepacked_vnni (534-590), _matmul_prepacked_rows (593-627),
 *   _split_k_partials + _sum_partials (1195-1221), _bmm_direct (1842-1855),
 *   _bmm_batched (1864-1882).
 * Accumulation is always f32; bias/scale/shift are applied in f32 in that
 * order, then the activation, then one rounding to `out_dtype`.
 */
typedef struct b200_gemm_desc {
  int32_t dtype;      /* B200_F32 or B200_BF16: element type of A and B */
  int32_t out_dtype;  /* element type of C (f32 accumulators rounded once) */
  int32_t a_layout;   /* B200_LAYOUT_ROW / _COL / _BLOCKED */
  int32_t b_layout;   /* any B200_LAYOUT_* */
  int32_t b_panel;    /* columns per panel for B200_LAYOUT_VNNI_PANELS, else 0 */
  int32_t epilogue;   /* B200_ACT_* */
  float alpha;        /* leaky-relu slope */
  int32_t vec_dtype;  /* element type of bias/scale/shift */
  int64_t m, n, k;    /* logical sizes; blocked/panel layouts are padded with zeros beyond them */
  int64_t batch;      /* >= 1; the batch is a grid dimension */
  int64_t lda, ldb, ldc;                 /* leading dimensions in elements (ROW/COL layouts, and C) */
  int64_t stride_a, stride_b, stride_c;  /* elements between consecutive batches */
  const void* a;
  const void* b;
  void* c;            /* [batch, M, ldc] row-major */
  const void* bias;   /* NULL or [bias_n] */
  const void* scale;  /* NULL or [scale_n] */
  const void* shift;  /* NULL or [shift_n] */
  int64_t bias_n, scale_n, shift_n;      /* n, or 1 for a broadcast scalar */
  /* K splits. 0/1: none. >1 with workspace==NULL: the splits of one output tile
   * run back to back on one CTA and are added in the order s=0..S-1.
   * >1 with a workspace of S*batch*M*N floats: partial products are written
   * there by parallel CTAs and summed in the order s=0..S-1 by a second kernel. */
  int32_t split_k;
  int32_t tile_m, tile_n, tile_k;        /* block_sizes hint (0: choose). tile_n >= 128 is snapped to a multiple of
                                          * 64 <= 256 and used; smaller positive hints leave the choice to the
                                          * launcher; tile_n < 0 fixes the width to -tile_n (tuning). tile_m and
                                          * tile_k are accepted and ignored: rows are 128 per CTA, K stages 64. */
  void* workspace;
  size_t workspace_bytes;
  int32_t force_kernel;  /* 0 auto, 1 tensor-core (tcgen05) path or refuse, 2 SIMT FFMA path,
                            3 tensor-core path with one CTA per tile, 4 with a CTA pair per tile (where the tile allows) */
  int32_t reserved_;
} b200_gemm_desc;

int b200_gemm(const b200_gemm_desc* desc, void* stream);

/* What b200_gemm would launch for `desc`: writes a short description such as
 * "umma_bf16 tile=128x256x64 stages=4 grid=148" into buf. Returns like b200_gemm
 * (a refusal code says why nothing would run). */
int b200_gemm_explain(const b200_gemm_desc* desc, char* buf, size_t buf_len);

/* Bytes of workspace b200_gemm needs for the parallel split-K form of `desc`. */
size_t b200_gemm_workspace_bytes(const b200_gemm_desc* desc);

/* b200_gemm for activations and results that live in host memory (the reference's
 * operators take host tensors: matmul.py:1384-1432 `matmul`, linear.py `linear`;
 * here the weights B and the epilogue vectors stay on the device). `desc` as for
 * b200_gemm except that desc->a and desc->c are ignored: A is read from `a_host`
 * (row-major, lda elements per row, batch 1) and C written to `c_host` (ldc
 * elements per row). The rows move in chunks of `chunk_rows` (<= 0: about 16 MiB of
 * A) through a library-owned ring of device staging buffers on two copy streams
 * while the GEMM of each chunk runs on `stream`; copy-in, GEMM and copy-out of
 * neighbouring chunks overlap, and so do back-to-back calls. Host memory should
 * be pinned (cudaHostAlloc / cudaHostRegister): pageable memory works but copies
 * synchronously. On return everything is enqueued; `stream` waits for the last
 * copy-out, so synchronising `stream` makes `c_host` readable. `a_host` must hold
 * its data when the call is made and stay unchanged until then, with one
 * exception: rows that an earlier b200_gemm_host_rows call on this device writes as
 * its `c_host` (a chained call) need no synchronisation in between, the copy-in
 * waits for that copy-out. The copy-in stream is NOT ordered after other work on
 * `stream`: host rows produced by such work asynchronously must be complete (or
 * `stream` synchronised) before the call. The first call on
 * a device creates the streams and allocates the ring (cudaMalloc); a later call
 * that needs a larger ring synchronises and reallocates. */
int b200_gemm_host_rows(const b200_gemm_desc* desc, const void* a_host, void* c_host, int64_t chunk_rows,
                        void* stream);
/* Waits for the copy streams of the current device and frees its staging ring. */
int b200_host_rows_release(void);

/* Softmax attention per head: out[h] = softmax(scale * q[h] k[h]^T) v[h], the
 * online-softmax kernel the reference's tests carry as a Helion body
 * (tests/harness.py:263-300 `_attention`, tests/test_numerics.py:141-158
 * `attention`). q, out: [heads, seq_q, dim]; k, v: [heads, seq_k, dim]; all
 * contiguous bf16 (B200_BF16 is the only dtype; others are refused with
 * B200_E_DTYPE and the host side composes the operators instead), dim 64 or 128,
 * 16-byte aligned. Scores and the output accumulate in f32; the probabilities
 * are rounded to bf16 for the second product, as the body's `p.to(q.dtype)` does.
 * seq_k == 0 writes zeros. `scale` must be finite and non-zero (B200_E_ARG). */
int b200_attention(int32_t dtype, const void* q, const void* k, const void* v, void* out, int64_t heads,
                   int64_t seq_q, int64_t seq_k, int64_t dim, float scale, void* stream);

/* Layout conversions (bit-exact copies with zero fill). `kind`: */
enum {
  B200_PACK_PAD_2D = 0,         /* [r,c] -> [rows_pad, cols_pad]                       matmul.py:78-89 */
  B200_PACK_A_BLOCKED = 1,      /* [M,K] -> [Mp/32,Kp/32,32,32]                        matmul.py:92-99 */
  B200_PACK_A_BLOCKED_T = 2,    /* [K,M] -> same                                       matmul.py:102-109 */
  B200_PACK_B_BLOCKED = 3,      /* [K,N] -> [Np/32,Kp/32,32,32]                        matmul.py:112-119 */
  B200_PACK_B_BLOCKED_T = 4,    /* [N,K] -> same                                       matmul.py:122-129 */
  B200_PACK_B_VNNI = 5,         /* [K,N] -> [Np/32,Kp/32,16,32,2]                      matmul.py:132-141 */
  B200_PACK_B_VNNI_T = 6,       /* [N,K] -> same                                       matmul.py:144-153 */
  B200_PACK_B_VNNI_PANELS_T = 7,/* [N,K] -> [Np/P,Kp/2,P,2]                            matmul.py:972-983 */
  /* inverse conversions used by the tensor-core GEMM for VNNI operands */
  B200_UNPACK_B_VNNI_TO_NK = 8,        /* [Np/32,Kp/32,16,32,2] -> [Np,Kp] row-major (K contiguous) */
  B200_UNPACK_B_VNNI_PANELS_TO_NK = 9, /* [Np/P,Kp/2,P,2] -> [Np,Kp] */
  B200_UNPACK_A_BLOCKED_TO_MK = 10,    /* [Mp/32,Kp/32,32,32] -> [Mp,Kp] row-major */
  B200_UNPACK_B_BLOCKED_TO_NK = 11,    /* [Np/32,Kp/32,32(k),32(n)] -> [Np,Kp] row-major (K contiguous) */
  B200_PACK_COUNT_ = 12
};

/* src: `rows` x `cols` row-major with leading dimension `ld` (elements);
 * dst: contiguous, sized for rows_pad x cols_pad logical elements of the
 * source orientation described by `kind`. `panel` only for *_PANELS_*. */
int b200_pack(int32_t kind, int32_t dtype, const void* src, int64_t rows, int64_t cols, int64_t ld,
              void* dst, int64_t rows_pad, int64_t cols_pad, int32_t panel, void* stream);

/* Row-wise softmax of x [M,N] (contiguous rows, leading dimension ld) into y.
 * y may equal x (in place). f32 arithmetic, one rounding to `dtype`.
 * Replaces _softmax_kernel / _softmax_one_kernel (normalization.py:28-87). */
int b200_softmax(int32_t dtype, const void* x, void* y, int64_t m, int64_t n, int64_t ld, void* stream);

/* Binary epilogue of group_norm: y (op) extra[channel]. */
enum { B200_NORM_EXTRA_NONE = 0, B200_NORM_EXTRA_ADD = 1, B200_NORM_EXTRA_MUL = 2 };

/* GroupNorm over x [M, groups*group_size] (contiguous): per (row, group) mean and
 * biased variance in f32 (two passes over registers), y = (x-mean)*rsqrt(var+eps)*w+b,
 * then `extra_op` with extra[channel], then activation `act`. weight/bias/extra are
 * [groups*group_size] of `param_dtype`; weight or bias may be NULL (1 and 0).
 * layer_norm is groups == 1. y may equal x.
 * Replaces _group_norm_kernel (normalization.py:94-123). */
int b200_group_norm(int32_t dtype, int32_t param_dtype, const void* x, void* y, int64_t m, int64_t groups,
                    int64_t group_size, const void* weight, const void* bias, const void* extra,
                    int32_t extra_op, int32_t act, float alpha, float eps, void* stream);

/* y = x * rsqrt(mean(x^2) + eps) * weight, rows of x [M,N]; weight may be NULL.
 * No counterpart kernel in the reference; nearest body is _group_norm_kernel. */
int b200_rms_norm(int32_t dtype, int32_t param_dtype, const void* x, void* y, int64_t m, int64_t n,
                  const void* weight, float eps, void* stream);

/* What b200_softmax (op 0), b200_group_norm (1) or b200_rms_norm (2) would launch for rows of
 * `n` elements `ld` apart with these operands: the kernel family, threads and values per
 * thread per row, rows per CTA, whether the row has a tail, is kept in 16 bits, or is taken
 * two rows at a time. Host arithmetic only (needs no GPU; the pointers are only tested for
 * alignment and presence). The counterpart of explain() for the row-wise operators
 * (_compiler/call_trace.py:84-217 reports the path a call takes). Returns 0 or a refusal code. */
int b200_rowwise_explain(int32_t op, int32_t dtype, int32_t param_dtype, const void* x, const void* y, int64_t n,
                         int64_t ld, int64_t groups, const void* weight, const void* bias, const void* extra,
                         int32_t extra_op, int32_t act, char* out, size_t out_len);

/* Row reductions of x [M,N] (ld = row stride) into out [M] of `dtype`:
 *   B200_REDUCE_ROW_SUM:  act(sum_n x[m,n])                 reduction.py:79-121
 *   B200_REDUCE_ROW_DOT:  act(sum_n x[m,n] * v[n]), v f32   reduction.py:166-212
 *   B200_REDUCE_MATVEC:   sum_k a[m,k] * v[k], v of dtype   reduction.py:24-67  */
enum { B200_REDUCE_ROW_SUM = 0, B200_REDUCE_ROW_DOT = 1, B200_REDUCE_MATVEC = 2 };
int b200_row_reduce(int32_t kind, int32_t dtype, const void* x, const void* v, void* out, int64_t m,
                    int64_t n, int64_t ld, int32_t act, float alpha, void* stream);

/* What b200_row_reduce (kind B200_REDUCE_*) or b200_column_sum (kind 3) would launch for an
 * [m, n] operand with rows `ld` apart: threads per row and rows per CTA, or the strips, chunks
 * and scratch of the column sum. Host arithmetic only (needs no GPU; the pointers are only
 * tested for alignment). Counterpart of explain() (_compiler/call_trace.py:84-217) for the
 * reductions. Returns 0 or a refusal code. */
int b200_reduce_explain(int32_t kind, int32_t dtype, const void* x, const void* v, int64_t m, int64_t n, int64_t ld,
                        char* out, size_t out_len);

/* Column sums of x [M,N] into out [N] f32, fixed summation order (no atomics).
 * `workspace` holds b200_column_sum_workspace_bytes(m, n) bytes of partial sums
 * (may be NULL when that is 0). Replaces _column_sum_kernel (reduction.py:124-163). */
size_t b200_column_sum_workspace_bytes(int64_t m, int64_t n);
int b200_column_sum(int32_t dtype, const void* x, float* out, int64_t m, int64_t n, int64_t ld,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * b200_column_sum without any allocation and without caller scratch. It has no
 * counterpart in the reference; it exists for hosts that cannot hand the library
 * memory at call time: a serving process whose device memory is fully budgeted at
 * start-up (weights, caches and activations planned to the last megabyte, so a
 * later cudaMalloc may fail or is forbidden by policy), or a latency-critical loop
 * that cannot afford the device-wide synchronisation an allocation or a free can
 * imply. The partial sums live in a fixed array of B200_COLUMN_SUM_STATIC_MAX_BYTES
 * inside the library's device image (so every GPU that loads the library holds
 * that much memory until the process ends).
 *
 * - Shapes whose partial sums (b200_column_sum_workspace_bytes(m, n)) exceed the
 *   array are refused with B200_E_TOO_LARGE; nothing runs. With the present
 *   two-stage plan (row chunks x columns of at most 1024 x 512 partial sums) no shape needs
 *   more than 2,097,152 bytes, which the 2 MiB array just holds; the check is
 *   what keeps that true if the plan's constants change.
 * - The first call on each device looks up the array's device address
 *   (cudaGetSymbolAddress, with that device current). Make that first call outside
 *   any stream capture; later calls do no set-up.
 * - No cudaMalloc, cudaFree or other allocating routine is called, on any call.
 * - All calls on a device share the one array and it keeps the last call's
 *   contents (the kernels overwrite what they read, so no clearing is needed).
 *   Two calls that may overlap on the GPU (different streams, or the same call
 *   from two threads without ordering) race on it: order them.
 */
#define B200_COLUMN_SUM_STATIC_MAX_BYTES (2u << 20)
int b200_column_sum_static(int32_t dtype, const void* x, float* out, int64_t m, int64_t n, int64_t ld,
                           void* stream);
/* The size check b200_column_sum_static applies, against any capacity: 0 when the
 * partial sums of an m x n column sum fit `capacity` bytes, B200_E_TOO_LARGE when
 * they do not (the entry point passes B200_COLUMN_SUM_STATIC_MAX_BYTES). Host
 * arithmetic only: callable without a device. No counterpart in the reference. */
int b200_column_sum_static_fits(int64_t m, int64_t n, size_t capacity);

/* Elementwise y = f(x) over `count` contiguous elements; y may equal x.
 * Replaces _relu_kernel, _leaky_relu_kernel, _scalar_mul_kernel (elementwise.py:14-41). */
enum { B200_ELT_RELU = 0, B200_ELT_LEAKY_RELU = 1, B200_ELT_SCALAR_MUL = 2 };
int b200_eltwise(int32_t kind, int32_t dtype, const void* x, void* y, int64_t count, float param, void* stream);

/*
 * Device-side reuse pool: the output_pool of the reference
 * (helion_mlir_backend/_compiler/output_pool.py) keeps page-faulted host
 * mappings for reuse; here blocks of device memory are kept instead, per
 * device, reused for the same rounded size, at most `max_bytes` and 64 free
 * blocks, oldest out first. A freed block may be handed out again at once to a
 * request on the stream that last used it; to another stream only after the
 * work recorded at free time has finished.
 */
int b200_pool_alloc(size_t bytes, void* stream, void** out_ptr, int32_t* out_hit);
int b200_pool_free(void* ptr, void* stream);
int b200_pool_set_limit(size_t max_bytes);
int b200_pool_release(void);
typedef struct b200_pool_stats_t {
  uint64_t hits, misses, free_blocks, free_bytes, max_bytes, live_blocks, live_bytes;
} b200_pool_stats_t;
int b200_pool_stats(b200_pool_stats_t* out);
/* Test hook: the pool's next `count` device allocations fail (as if out of memory)
 * without reaching the driver, so that the release-and-retry of b200_pool_alloc
 * can be exercised on the host. The reference provokes the same path by capping
 * the address space (tests/test_output_pool.py:683-709); a device is not driven
 * out of memory for a test. 0 clears it. */
int b200_pool_inject_alloc_failures(int32_t count);

/* Per-operator counters since load: launches and refusals (cf. KernelRun's
 * native_calls / refusals, call.cpp:841-850). */
typedef struct b200_counters_t {
  uint64_t launches;      /* kernels enqueued */
  uint64_t calls;         /* successful entry-point calls */
  uint64_t refusals;      /* positive returns */
  uint64_t cuda_errors;   /* negative returns */
  int32_t last_refusal;   /* code of the latest refusal */
  int32_t reserved_;
} b200_counters_t;
int b200_get_counters(b200_counters_t* out);
int b200_reset_counters(void);

/* ---- column-sharded linear with the all-gather fused into the GEMM ----
 *
 * No counterpart in the reference (one process, one CPU). A linear layer whose
 * weight is split along N over the G GPUs of a box computes its columns of y on
 * each GPU; every GPU needs all of y. Instead of a GEMM followed by an NCCL
 * all-gather, b200_gemm_to_peers stores each finished piece of its columns into all
 * G copies of y (plain stores through peer pointers over NVLink while the tensor
 * cores work on the next tile), and when its last CTA has stored it raises one flag
 * word on every GPU. b200_peer_wait, enqueued after it, returns when all G flags
 * of this GPU have been raised: y is then complete here.
 *
 * Memory: the copies of y and the flag words must be mapped in every rank's
 * process: b200_symm_alloc (cudaMalloc + zero fill + an IPC handle to send to the
 * other ranks, e.g. through torch.distributed), b200_symm_open (maps a peer's
 * handle, enabling peer access), b200_symm_close / b200_symm_free. Operands (A, B,
 * bias) are always read from the calling GPU's own memory.
 *
 * Waits are bounded: after `budget_ns` b200_peer_wait gives up, ORs 32 into the
 * kernel status word and returns; nothing hangs if a peer never arrives. A rank must
 * not start a GEMM into a copy of y that a peer may still be reading: alternate two
 * buffers and keep each rank's calls in stream order (helion_mlir_utils.sharding). */
#define B200_MAX_PEERS 8
#define B200_IPC_HANDLE_BYTES 64
typedef struct b200_peer_out {
  int32_t count;                   /* G: copies of C, this GPU's included */
  int32_t rank;                    /* index of this GPU's own copy: c[rank] == desc->c */
  int32_t epoch;                   /* value the flags are set to (increase it per call) */
  int32_t reserved_;
  void* c[B200_MAX_PEERS];         /* where C starts in copy j (device pointers valid on this GPU) */
  int32_t* flags[B200_MAX_PEERS];  /* the word on GPU j that this GPU raises */
  uint32_t* done_counter;          /* a zeroed word on this GPU, private to these calls */
  const void* store_maps;          /* NULL, or what b200_peer_store_maps wrote for these c[]: the results then
                                      leave as one bulk tensor store per copy and 32 x 64 piece */
} b200_peer_out;
int b200_gemm_to_peers(const b200_gemm_desc* desc, const b200_peer_out* out, void* stream);
/* Set-up for bulk tensor stores: encodes one store descriptor per copy (c[j] = where this
 * rank's columns start in copy j, `rows` x `cols` bf16 values, rows `ld` elements apart) and
 * writes them to `device_maps` (count x 128 bytes of this GPU's memory, 64-byte aligned).
 * Synchronous; call once per set of copies, then pass `device_maps` as store_maps. */
int b200_peer_store_maps(void* device_maps, void* const* c, int32_t count, int64_t rows, int64_t cols, int64_t ld);
/* Waits (on the device, `stream` order) until flags[0..count) have all reached `epoch`. */
int b200_peer_wait(const int32_t* flags, int32_t count, int32_t epoch, uint64_t budget_ns, void* stream);
int b200_symm_alloc(size_t bytes, void** out_ptr, void* out_handle /* B200_IPC_HANDLE_BYTES */);
int b200_symm_open(const void* handle /* B200_IPC_HANDLE_BYTES */, void** out_ptr);
int b200_symm_close(void* ptr);
int b200_symm_free(void* ptr);

/* Device error word written by kernels whose bounded waits ran out
 * (0 = none). Reading it synchronises the given stream. */
int b200_read_kernel_status(void* stream, int32_t* out_status);

/* Self-test of the failure path of the kernels' bounded waits (no counterpart in
 * the reference, whose failure handling is host-side: compile time-outs,
 * _compiler/execution.py:611-647). Launches one warp that waits, for at most
 * `budget_ns` (1..1e9), on a barrier nothing arrives on. The wait must give up,
 * OR the bit 16 into the kernel status word and return normally: afterwards
 * b200_read_kernel_status reports 16 and the context keeps working. Nothing
 * faults, traps or hangs. */
int b200_selftest_wait_timeout(uint64_t budget_ns, void* stream);

const char* b200_strerror(int code);
int b200_abi_version(void);
/* 0 makes every compute entry point refuse with B200_E_DISABLED (set_native_call(False)). */
int b200_set_enabled(int enabled);
/* Number of SMs of the current device (0 if none). */
int b200_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H_ */
