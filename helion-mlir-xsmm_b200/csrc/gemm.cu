// b200_gemm: validation and kernel choice.
//
// Paths, in order of preference:
//   tensor cores  bf16 operands whose rows TMA can describe (16-byte aligned bases
//                 and pitches), plain ROW/COL layouts and 32x32-blocked A directly (the
//                 blocks are what a 5-D tensor map walks); the blocked / VNNI layouts of B
//                 through one unpack to K-contiguous rows in the caller's workspace
//                 f32 operands (plain or 32x32-blocked, batched or not) as a six-term
//                 bf16 split over a 6x longer K
//   FFMA          everything else (small or oddly pitched f32, explicit f32 split-K), exact f32
// The choice mirrors the dispatcher of helion_mlir_utils/matmul.py:1446-1570
// (bf16 -> fused kernel, f32 -> split-K / fused / blocked) with the CPU tile
// heuristics replaced by the SM count; block_sizes arrive as tile_m/n/k hints.
#include <cstdio>
#include <cstring>

#include "gemm_common.cuh"

namespace b200 {

int explain_gemm_umma(const b200_gemm_desc& d, char* buf, size_t len);
int run_wait_timeout_selftest(unsigned long long budget_ns, cudaStream_t stream);
int run_gemm_simt(const b200_gemm_desc& d, const GemmOperand& a, const GemmOperand& b, const GemmEpilogue& epi,
                  int splits, float* workspace, cudaStream_t stream);

namespace {

// f32 operands on the tensor cores: each f32 value is split into three bf16 parts
// and the six largest cross products are summed by one bf16 GEMM over a six times
// longer K (the bf16 analogue of 3xTF32; products of bf16 parts are exact in f32).
// The tensor core's f32 accumulation truncates, a bias that grows with the length
// and magnitude of a running sum. So the widened K is cut into chunks of at most
// kSplitChunkK elements that are added in f32 in ascending order (serial split-K, or
// parallel partial sums when there are few tiles): the error then no longer grows with K
// (measured relative Frobenius error 1.0e-6 at 1024^3, 4.4e-6 at 4096^3, bar 1e-5).
// Operands that are not finite, or beyond bf16's range (|x| > 3.39e38), have no such
// split: their products come out NaN where exact f32 arithmetic gives an infinity.
constexpr int kSplitTerms = 6;
constexpr int64_t kSplitChunkK = 2048;
constexpr int64_t kSplitMaxK = int64_t(1) << 17;
constexpr int64_t kSplitMinWork = int64_t(1) << 24;  // batch*m*n*k below this stays on the FFMA kernel

// K of one copy in the widened operands: whole 16-byte pieces of bf16.
inline int64_t split_k_wide(const b200_gemm_desc& d) { return round_up(d.k, 8); }

struct Resolved {
  GemmOperand a, b;
  GemmEpilogue epi;
  int64_t k_pad;        // K as the packed layouts pad it
  int64_t n_pad;        // N as the packed B layout pads it
  bool b_is_vnni;
  int64_t m_pad;          // M as the blocked A layout pads it
  size_t unpack_bytes;    // workspace for a packed B unpacked to [n_pad, k_pad] bf16
  size_t partial_bytes; // workspace for parallel split-K partials
  size_t split_a_bytes, split_b_bytes;  // workspace for the six-fold bf16 split of f32 operands (0: not applicable)
  size_t split_partial_bytes;  // ... and for its K chunks as parallel partial sums (0: chunks run back to back)
};

// K chunks of the widened product. At least one per kSplitChunkK elements; when the
// chunks run as parallel work items (few output tiles), as many more as there are idle
// CTA pairs for, so that each chunk is shorter (1024^3: 16 tiles x 4 chunks of 1536 on
// 74 pairs instead of 3 of 2048). Shorter chunks only make the f32 sum more exact.
int64_t split_chunk_count(const b200_gemm_desc& d, bool* parallel) {
  const int64_t wide_k = split_k_wide(d) * kSplitTerms;
  int64_t chunks = ceil_div(wide_k, kSplitChunkK);
  const int64_t pair_tiles = ceil_div(d.m, 256) * ceil_div(d.n, 256) * d.batch;
  const int64_t pairs = device_info().sm_count / 2;
  *parallel = chunks > 1 && pair_tiles * chunks <= pairs;
  if (*parallel) {
    const int64_t room = pairs / pair_tiles;
    for (int64_t c = room; c > chunks; --c) {
      if (wide_k % (c * 64) == 0 && wide_k / c >= 512) {
        chunks = c;
        break;
      }
    }
  }
  return chunks;
}

// Whether the f32 GEMM `d` can run as a widened bf16 GEMM: plain or 32x32-blocked
// operands (the widening pass reads either), any batch, no explicit split-K (that
// keeps the exact kernel and its partial sums).
bool f32_split_applies(const b200_gemm_desc& d) {
  if (d.dtype != B200_F32 || d.a_layout > B200_LAYOUT_BLOCKED || d.b_layout > B200_LAYOUT_BLOCKED) return false;
  if (d.split_k > 1 || d.k < 1 || d.k > kSplitMaxK || d.force_kernel == 2) return false;
  if (static_cast<double>(d.batch) * d.m * d.n * d.k < static_cast<double>(kSplitMinWork)) return false;
  // [K, M] / [K, N] operands are widened along their rows: the row pitch stays m / n elements
  if (d.a_layout == B200_LAYOUT_COL && d.m % 8) return false;
  if (d.b_layout == B200_LAYOUT_ROW && d.n % 8) return false;
  return true;
}

int validate(const b200_gemm_desc* d, Resolved* r) {
  if (!d) return B200_E_NULL;
  if (!valid_dtype(d->dtype) || !valid_dtype(d->out_dtype) || !valid_dtype(d->vec_dtype)) return B200_E_DTYPE;
  if (d->a_layout < 0 || d->a_layout > B200_LAYOUT_BLOCKED) return B200_E_ARG;
  if (d->b_layout < 0 || d->b_layout > B200_LAYOUT_VNNI_PANELS) return B200_E_ARG;
  if (d->epilogue < 0 || d->epilogue >= B200_ACT_COUNT_) return B200_E_ARG;
  if (d->force_kernel < 0 || d->force_kernel > 4) return B200_E_ARG;
  if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 1) return B200_E_SHAPE;
  if (d->split_k < 0 || d->split_k > 1024) return B200_E_ARG;
  if ((d->b_layout == B200_LAYOUT_BLOCKED_VNNI || d->b_layout == B200_LAYOUT_VNNI_PANELS) && d->dtype != B200_BF16)
    return B200_E_DTYPE;
  if (d->b_layout == B200_LAYOUT_VNNI_PANELS && (d->b_panel <= 0 || d->b_panel % 32)) return B200_E_ARG;
  if (d->m == 0 || d->n == 0) return 0;
  if (!d->c || (d->k > 0 && (!d->a || !d->b))) return B200_E_NULL;
  const size_t es = dtype_size(d->dtype);
  if (!aligned(d->a, es) || !aligned(d->b, es) || !aligned(d->c, dtype_size(d->out_dtype))) return B200_E_ALIGN;
  if (d->ldc < d->n) return B200_E_STRIDE;
  if (d->a_layout == B200_LAYOUT_ROW && d->lda < d->k) return B200_E_STRIDE;
  if (d->a_layout == B200_LAYOUT_COL && d->lda < d->m) return B200_E_STRIDE;
  if (d->b_layout == B200_LAYOUT_ROW && d->ldb < d->n) return B200_E_STRIDE;
  if (d->b_layout == B200_LAYOUT_COL && d->ldb < d->k) return B200_E_STRIDE;
  const int64_t vec_n[3] = {d->bias_n, d->scale_n, d->shift_n};
  const void* vec_p[3] = {d->bias, d->scale, d->shift};
  for (int i = 0; i < 3; ++i)
    if (vec_p[i] && vec_n[i] != 1 && vec_n[i] != d->n) return B200_E_SHAPE;

  // C must not overlap A or B: CTAs read operands while others store results.
  const uintptr_t c0 = reinterpret_cast<uintptr_t>(d->c);
  const uintptr_t c1 = c0 + static_cast<uintptr_t>(((d->batch - 1) * d->stride_c + (d->m - 1) * d->ldc + d->n) *
                                                   static_cast<int64_t>(dtype_size(d->out_dtype)));
  const int64_t k32 = round_up(d->k, 32);
  auto span = [&](const void* p, int64_t elems, int64_t stride) {
    const uintptr_t p0 = reinterpret_cast<uintptr_t>(p);
    const uintptr_t p1 = p0 + static_cast<uintptr_t>(((d->batch - 1) * stride + elems) * static_cast<int64_t>(es));
    return p0 < c1 && c0 < p1;
  };
  int64_t a_elems, b_elems;
  switch (d->a_layout) {
    case B200_LAYOUT_ROW: a_elems = (d->m - 1) * d->lda + d->k; break;
    case B200_LAYOUT_COL: a_elems = (d->k - 1) * d->lda + d->m; break;
    default: a_elems = round_up(d->m, 32) * k32;
  }
  r->k_pad = k32;
  r->n_pad = d->n;
  switch (d->b_layout) {
    case B200_LAYOUT_ROW: b_elems = (d->k - 1) * d->ldb + d->n; break;
    case B200_LAYOUT_COL: b_elems = (d->n - 1) * d->ldb + d->k; break;
    case B200_LAYOUT_VNNI_PANELS:
      r->n_pad = round_up(d->n, d->b_panel);
      b_elems = r->n_pad * k32;
      break;
    default:
      r->n_pad = round_up(d->n, 32);
      b_elems = r->n_pad * k32;
  }
  if (d->k > 0 && (span(d->a, a_elems, d->stride_a) || span(d->b, b_elems, d->stride_b))) return B200_E_ALIAS;

  r->a = GemmOperand{d->a, d->a_layout, 0, d->lda, k32 / 32};
  r->b = GemmOperand{d->b, d->b_layout, d->b_panel, d->ldb,
                     d->b_layout == B200_LAYOUT_VNNI_PANELS ? k32 / 2 : k32 / 32};
  r->epi = GemmEpilogue{d->bias,           d->scale,          d->shift,
                        d->bias_n == 1,    d->scale_n == 1,   d->shift_n == 1,
                        d->vec_dtype == B200_BF16, d->epilogue, d->alpha};
  r->b_is_vnni = d->b_layout == B200_LAYOUT_BLOCKED_VNNI || d->b_layout == B200_LAYOUT_VNNI_PANELS;
  r->m_pad = round_up(d->m, 32);
  const bool bf16 = d->dtype == B200_BF16;
  r->unpack_bytes = (bf16 && d->b_layout >= B200_LAYOUT_BLOCKED)
                        ? static_cast<size_t>(round_up(r->n_pad * k32 * 2, 256))
                        : 0;
  r->partial_bytes =
      d->split_k > 1 ? static_cast<size_t>(d->split_k) * d->batch * d->m * d->n * sizeof(float) : 0;
  r->split_a_bytes = r->split_b_bytes = r->split_partial_bytes = 0;
  if (f32_split_applies(*d)) {
    const int64_t kw = split_k_wide(*d);
    r->split_a_bytes = static_cast<size_t>(round_up(d->batch * d->m * kw * kSplitTerms * 2, 256));
    r->split_b_bytes = static_cast<size_t>(round_up(d->batch * d->n * kw * kSplitTerms * 2, 256));
    // Few output tiles: the K chunks of the widened product (added in f32 either way, in
    // the same order) run as parallel work items into partial sums, so that the chunks of
    // one tile occupy several SMs instead of running back to back on one.
    bool parallel = false;
    const int64_t chunks = split_chunk_count(*d, &parallel);
    if (parallel) r->split_partial_bytes = static_cast<size_t>(round_up(chunks * d->batch * d->m * d->n * 4, 256));
  }
  return 0;
}

// The descriptor the tensor-core kernel sees once packed operands have been
// unpacked: A as row-major [m_pad, k_pad], B as K-contiguous [n_pad, k_pad].
b200_gemm_desc unpacked_desc(const b200_gemm_desc& d, const Resolved& r, void* b_unpacked) {
  b200_gemm_desc u = d;
  if (r.unpack_bytes) {
    u.b = b_unpacked;
    u.b_layout = B200_LAYOUT_COL;
    u.ldb = r.k_pad;
    u.stride_b = r.n_pad * r.k_pad;
  }
  return u;
}

enum Path { kPathUmma, kPathUmmaUnpack, kPathUmmaSplitF32, kPathSimt };

// The bf16 GEMM over the widened K that stands for the f32 GEMM `d`: A as [M, 6K]
// (or [6K, M] for a [K, M] source), B as [N, 6K] (or [6K, N] for a [K, N] source).
b200_gemm_desc split_desc(const b200_gemm_desc& d, void* a_wide, void* b_wide) {
  b200_gemm_desc u = d;
  const int64_t kw = split_k_wide(d);
  u.dtype = B200_BF16;
  u.a = a_wide;
  u.b = b_wide;
  u.k = kw * kSplitTerms;
  u.a_layout = d.a_layout == B200_LAYOUT_COL ? B200_LAYOUT_COL : B200_LAYOUT_ROW;
  u.b_layout = d.b_layout == B200_LAYOUT_ROW ? B200_LAYOUT_ROW : B200_LAYOUT_COL;
  u.lda = u.a_layout == B200_LAYOUT_ROW ? u.k : d.m;
  u.ldb = u.b_layout == B200_LAYOUT_COL ? u.k : d.n;
  u.stride_a = d.m * u.k;
  u.stride_b = d.n * u.k;
  // chunks of the widened K are added in f32 by the epilogue (needs an f32 result)
  bool parallel = false;
  u.split_k = static_cast<int32_t>(split_chunk_count(d, &parallel));
  if (u.split_k < 2) u.split_k = 0;
  u.workspace = nullptr;
  u.workspace_bytes = 0;
  return u;
}

// The two operands of `d` as the widening pass reads them.
void split_operands(const b200_gemm_desc& d, void* a_wide, void* b_wide, SplitOperand* a, SplitOperand* b) {
  const int64_t kw = split_k_wide(d), kblocks = round_up(d.k, 32) / 32;
  *a = SplitOperand{static_cast<const float*>(d.a), static_cast<__nv_bfloat16*>(a_wide), d.batch, 0, 0, 0, d.stride_a, kw,
                    0, 0, 1};
  if (d.a_layout == B200_LAYOUT_COL) {  // [K, M]: widened along the rows
    a->rows = d.k, a->cols = d.m, a->ld = d.lda, a->along_cols = 0;
  } else {
    a->rows = d.m, a->cols = d.k;
    a->ld = d.a_layout == B200_LAYOUT_ROW ? d.lda : kblocks;
    a->layout = d.a_layout == B200_LAYOUT_ROW ? 0 : 1;
  }
  *b = SplitOperand{static_cast<const float*>(d.b), static_cast<__nv_bfloat16*>(b_wide), d.batch, 0, 0, 0, d.stride_b, kw,
                    0, 1, 1};
  if (d.b_layout == B200_LAYOUT_ROW) {  // [K, N]: widened along the rows
    b->rows = d.k, b->cols = d.n, b->ld = d.ldb, b->along_cols = 0;
  } else {
    b->rows = d.n, b->cols = d.k;
    b->ld = d.b_layout == B200_LAYOUT_COL ? d.ldb : kblocks;
    b->layout = d.b_layout == B200_LAYOUT_COL ? 0 : 2;
  }
}

// Chooses the path; `*why` gets the refusal of the tensor-core path when it is not taken.
Path choose(const b200_gemm_desc& d, const Resolved& r, int* why) {
  *why = 0;
  if (d.force_kernel == 2) return kPathSimt;
  if (d.k == 0) return kPathSimt;
  if (r.unpack_bytes) {
    if (d.batch != 1) {
      *why = B200_E_SHAPE;
      return kPathSimt;
    }
    if (!d.workspace || d.workspace_bytes < r.unpack_bytes || !aligned(d.workspace, 256)) {
      *why = B200_E_WORKSPACE;
      return kPathSimt;
    }
    uint8_t* ws = static_cast<uint8_t*>(d.workspace);
    b200_gemm_desc u = unpacked_desc(d, r, ws);
    *why = umma_supports(u);
    return *why == 0 ? kPathUmmaUnpack : kPathSimt;
  }
  if (r.split_a_bytes) {
    if (!d.workspace || d.workspace_bytes < r.split_a_bytes + r.split_b_bytes || !aligned(d.workspace, 256)) {
      *why = B200_E_WORKSPACE;
      return kPathSimt;
    }
    uint8_t* ws = static_cast<uint8_t*>(d.workspace);
    *why = umma_supports(split_desc(d, ws, ws + r.split_a_bytes));
    return *why == 0 ? kPathUmmaSplitF32 : kPathSimt;
  }
  *why = umma_supports(d);
  return *why == 0 ? kPathUmma : kPathSimt;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" size_t b200_gemm_workspace_bytes(const b200_gemm_desc* desc) {
  Resolved r{};
  if (validate(desc, &r) != 0 || desc->m == 0 || desc->n == 0) return 0;
  return r.unpack_bytes + r.partial_bytes + r.split_a_bytes + r.split_b_bytes + r.split_partial_bytes;
}

extern "C" int b200_gemm(const b200_gemm_desc* desc, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  Resolved r{};
  const int bad = validate(desc, &r);
  if (bad) return refuse(bad);
  const b200_gemm_desc& d = *desc;
  if (d.m == 0 || d.n == 0) return finish(0);
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int why = 0;
  const Path path = choose(d, r, &why);
  if (path == kPathSimt && d.force_kernel != 0 && d.force_kernel != 2) return refuse(why ? why : B200_E_ARG);

  // Workspace carve-up: [unpacked A][unpacked B][split-K partials].
  uint8_t* ws = static_cast<uint8_t*>(d.workspace);
  size_t ws_left = d.workspace ? d.workspace_bytes : 0;
  void* b_unpacked = nullptr;
  if (path == kPathUmmaUnpack) {
    b_unpacked = ws;
    ws += r.unpack_bytes;
    ws_left -= r.unpack_bytes;
  }
  float* partials = nullptr;
  if (d.split_k > 1 && ws_left >= r.partial_bytes && ws_left > 0 && aligned(ws, 16)) partials = reinterpret_cast<float*>(ws);

  if (path == kPathSimt) return run_gemm_simt(d, r.a, r.b, r.epi, d.split_k, partials, s);

  if (path == kPathUmmaSplitF32) {
    uint8_t* wide = static_cast<uint8_t*>(d.workspace);
    SplitOperand wide_a, wide_b;
    split_operands(d, wide, wide + r.split_a_bytes, &wide_a, &wide_b);
    const int rc = launch_split_f32(wide_a, wide_b, s);
    if (rc != 0) return finish(rc);
    float* chunk_partials = nullptr;
    if (r.split_partial_bytes && d.workspace_bytes >= r.split_a_bytes + r.split_b_bytes + r.split_partial_bytes)
      chunk_partials = reinterpret_cast<float*>(wide + r.split_a_bytes + r.split_b_bytes);
    return run_gemm_umma(split_desc(d, wide, wide + r.split_a_bytes), r.epi, chunk_partials, s);
  }

  if (path == kPathUmmaUnpack) {
    if (r.unpack_bytes) {
      const int kind = d.b_layout == B200_LAYOUT_VNNI_PANELS  ? B200_UNPACK_B_VNNI_PANELS_TO_NK
                       : d.b_layout == B200_LAYOUT_BLOCKED_VNNI ? B200_UNPACK_B_VNNI_TO_NK
                                                                : B200_UNPACK_B_BLOCKED_TO_NK;
      const int rc = b200_pack(kind, B200_BF16, d.b, 0, 0, 0, b_unpacked, r.n_pad, r.k_pad, d.b_panel, stream);
      if (rc != 0) return rc;
    }
    const b200_gemm_desc u = unpacked_desc(d, r, b_unpacked);
    return run_gemm_umma(u, r.epi, partials, s);
  }
  return run_gemm_umma(d, r.epi, partials, s);
}

// The GEMM of b200_gemm with its result stored into `out->count` copies of C: this GPU's
// (desc->c, which must be out->c[out->rank]) and its peers' (device pointers into their
// memory, mapped here). Tensor-core path only (bf16 operands in plain layouts, one
// problem, no split-K): refused otherwise, never run another way.
extern "C" int b200_gemm_to_peers(const b200_gemm_desc* desc, const b200_peer_out* out, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!out) return refuse(B200_E_NULL);
  Resolved r{};
  const int bad = validate(desc, &r);
  if (bad) return refuse(bad);
  const b200_gemm_desc& d = *desc;
  if (out->count < 1 || out->count > B200_MAX_PEERS || out->rank < 0 || out->rank >= out->count) return refuse(B200_E_ARG);
  if (!out->done_counter || !aligned(out->done_counter, 4)) return refuse(B200_E_NULL);
  for (int j = 0; j < out->count; ++j)
    if (!out->c[j] || !out->flags[j] || !aligned(out->flags[j], 4)) return refuse(B200_E_NULL);
  if (out->c[out->rank] != d.c) return refuse(B200_E_ARG);
  if (d.m == 0 || d.n == 0 || d.k == 0) return refuse(B200_E_SHAPE);  // the flags are only raised by a launch
  if (d.batch != 1 || d.split_k > 1) return refuse(B200_E_ARG);
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  int why = 0;
  if (choose(d, r, &why) != kPathUmma) return refuse(why ? why : B200_E_ARG);
  PeerOut peers{};
  peers.count = out->count;
  peers.epoch = out->epoch;
  for (int j = 0; j < out->count; ++j) {
    peers.delta[j] = static_cast<int64_t>(reinterpret_cast<intptr_t>(out->c[j]) - reinterpret_cast<intptr_t>(d.c));
    peers.flags[j] = out->flags[j];
  }
  peers.done_counter = out->done_counter;
  peers.store_maps = out->store_maps;
  if (out->store_maps && !aligned(out->store_maps, 64)) return refuse(B200_E_ALIGN);
  return run_gemm_umma(d, r.epi, nullptr, static_cast<cudaStream_t>(stream), &peers);
}

extern "C" int b200_peer_store_maps(void* device_maps, void* const* c, int32_t count, int64_t rows, int64_t cols,
                                    int64_t ld) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  return store_peer_maps(device_maps, c, count, rows, cols, ld);
}

extern "C" int b200_peer_wait(const int32_t* flags, int32_t count, int32_t epoch, uint64_t budget_ns, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!flags) return refuse(B200_E_NULL);
  if (count < 1 || count > B200_MAX_PEERS || budget_ns == 0 || budget_ns > 10000000000ull) return refuse(B200_E_ARG);
  return run_peer_wait(flags, count, epoch, budget_ns, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_gemm_explain(const b200_gemm_desc* desc, char* buf, size_t buf_len) {
  if (!buf || buf_len == 0) return B200_E_NULL;
  buf[0] = 0;
  Resolved r{};
  const int bad = validate(desc, &r);
  if (bad) {
    snprintf(buf, buf_len, "refused: %s", b200_strerror(bad));
    return bad;
  }
  int why = 0;
  const Path path = choose(*desc, r, &why);
  if (path == kPathSimt) {
    snprintf(buf, buf_len, "simt_ffma tile=128x128x16 (tensor-core path not taken: %s)",
             desc->force_kernel == 2 ? "forced" : b200_strerror(why));
    return (desc->force_kernel != 0 && desc->force_kernel != 2) ? (why ? why : B200_E_ARG) : 0;
  }
  uint8_t* ws = static_cast<uint8_t*>(desc->workspace);
  b200_gemm_desc u = *desc;
  if (path == kPathUmmaUnpack) u = unpacked_desc(*desc, r, ws);
  if (path == kPathUmmaSplitF32) u = split_desc(*desc, ws, ws + r.split_a_bytes);
  char inner[200];
  explain_gemm_umma(u, inner, sizeof inner);
  snprintf(buf, buf_len, "%s%s",
           path == kPathUmmaUnpack     ? "unpack B to K-contiguous rows + "
           : path == kPathUmmaSplitF32 ? "f32 as 6 bf16 cross products (K x6) + "
                                       : "",
           inner);
  return 0;
}

extern "C" int b200_selftest_wait_timeout(uint64_t budget_ns, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (budget_ns == 0 || budget_ns > 1000000000ull) return refuse(B200_E_ARG);  // at most one second
  return run_wait_timeout_selftest(budget_ns, static_cast<cudaStream_t>(stream));
}
