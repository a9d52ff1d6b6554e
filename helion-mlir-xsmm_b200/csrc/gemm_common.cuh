// Pieces shared by the GEMM paths: operand addressing for every accepted layout,
// the fused epilogue, and the ordered split-K reduction.
#pragma once

#include "common.cuh"

namespace b200 {

struct GemmOperand {
  const void* p;
  int32_t layout;
  int32_t panel;
  int64_t ld;       // ROW/COL layouts
  int64_t kblocks;  // padded K / 32 (blocked layouts); padded K / 2 for panels
};

struct GemmEpilogue {
  const void* bias;
  const void* scale;
  const void* shift;
  int32_t bias_scalar, scale_scalar, shift_scalar;  // broadcast a single value
  int32_t vec_bf16;
  int32_t act;
  float alpha;
};

__device__ __forceinline__ float load_vec(const void* p, int64_t i, int bf16) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : static_cast<const float*>(p)[i];
}

// act(((acc + bias) * scale) + shift), all in f32
// (helion_mlir_utils/matmul.py:321-327 applies them in this order).
__device__ __forceinline__ float run_epilogue(const GemmEpilogue& e, float acc, int64_t col) {
  if (e.bias) acc += load_vec(e.bias, e.bias_scalar ? 0 : col, e.vec_bf16);
  if (e.scale) acc *= load_vec(e.scale, e.scale_scalar ? 0 : col, e.vec_bf16);
  if (e.shift) acc += load_vec(e.shift, e.shift_scalar ? 0 : col, e.vec_bf16);
  return apply_act(e.act, acc, e.alpha);
}

// Element offset of A(m, k) / B(k, n) in each layout.
__device__ __forceinline__ int64_t offset_a(const GemmOperand& a, int64_t m, int64_t k) {
  switch (a.layout) {
    case B200_LAYOUT_ROW:
      return m * a.ld + k;
    case B200_LAYOUT_COL:
      return k * a.ld + m;
    default:  // [M/32][K/32][32 m][32 k]
      return (((m >> 5) * a.kblocks + (k >> 5)) << 10) + ((m & 31) << 5) + (k & 31);
  }
}
__device__ __forceinline__ int64_t offset_b(const GemmOperand& b, int64_t k, int64_t n) {
  switch (b.layout) {
    case B200_LAYOUT_ROW:
      return k * b.ld + n;
    case B200_LAYOUT_COL:
      return n * b.ld + k;
    case B200_LAYOUT_BLOCKED:  // [N/32][K/32][32 k][32 n]
      return (((n >> 5) * b.kblocks + (k >> 5)) << 10) + ((k & 31) << 5) + (n & 31);
    case B200_LAYOUT_BLOCKED_VNNI:  // [N/32][K/32][16][32 n][2]
      return (((n >> 5) * b.kblocks + (k >> 5)) << 10) + (((k & 31) >> 1) << 6) + ((n & 31) << 1) + (k & 1);
    default: {  // panels [N/P][K/2][P][2]; kblocks = padded K / 2
      const int64_t q = n / b.panel, nn = n - q * b.panel;
      return ((q * b.kblocks + (k >> 1)) * b.panel + nn) * 2 + (k & 1);
    }
  }
}

// Destinations of a GEMM whose result goes to every GPU of a group (the fused form of a
// column-sharded linear followed by an all-gather): the epilogue stores each finished
// piece of C into every copy through peer pointers (plain stores over NVLink; operands
// are only ever loaded from this GPU's own memory), and when the last CTA has stored, one
// flag per destination says so.
struct PeerOut {
  int32_t count;           // copies of C, this GPU's own included
  int32_t epoch;           // value written to the flags
  int64_t delta[8];        // byte offset from this GPU's C to copy j
  int32_t* flags[8];       // word on GPU j that this GPU's kernel sets to `epoch` when its stores are done
  uint32_t* done_counter;  // on this GPU: CTAs that have finished (reset by the last one)
  const void* store_maps;  // on this GPU: `count` tensor maps, one per copy (NULL: plain stores)
};

int run_gemm_umma(const b200_gemm_desc& d, const GemmEpilogue& epi, float* partials, cudaStream_t stream,
                  const PeerOut* peers = nullptr);
int umma_supports(const b200_gemm_desc& d);
int store_peer_maps(void* device_maps, void* const* c, int count, int64_t rows, int64_t cols, int64_t ld);
int run_peer_wait(const int32_t* flags, int count, int32_t epoch, unsigned long long budget_ns, cudaStream_t stream);

// One f32 operand to be widened into its six-fold bf16 split (split_f32_kernel, pack.cu).
struct SplitOperand {
  const float* src;
  __nv_bfloat16* dst;
  int64_t batch, rows, cols;  // extent of the logical matrix read from the source
  int64_t ld, batch_stride;   // source, in elements; blocked sources: ld = 32-blocks per block row
  int64_t k_wide;             // contraction length of one copy in the widened operand (zero beyond the source's)
  int32_t layout;             // 0 rows of `ld`; 1 blocks [rows/32][cols/32][32 r][32 c]; 2 blocks [rows/32][cols/32][32 c][32 r]
  int32_t is_b, along_cols;
};
int launch_split_f32(const SplitOperand& a, const SplitOperand& b, cudaStream_t stream);

// out = act((sum_s partial[s] + bias) * scale + shift), s ascending.
// partial is [splits][batch*m*n] f32 (rows contiguous, n wide); out rows are ldc wide.
int launch_splitk_reduce(const float* partial, int splits, int64_t batch, int64_t m, int64_t n, void* out,
                         int out_bf16, int64_t ldc, int64_t stride_c, const GemmEpilogue& epi, cudaStream_t stream);

}  // namespace b200
