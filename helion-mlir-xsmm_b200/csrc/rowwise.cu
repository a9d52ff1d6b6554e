// Row-wise softmax / GroupNorm (LayerNorm) / RMSNorm for sm_100a.
//
// Bandwidth-bound kernels: every element of x is read from HBM once (one
// 128-bit load where rows are 16-byte aligned), kept in registers while the row
// statistics are reduced (warp shuffles, then shared memory across the warps of
// a row), and written once. A row is owned by `tpr` threads (a power of two from 4
// up, or any number of whole warps that covers the row exactly, up to 512; 1024 in the
// two-pass kernel); a CTA holds 256/tpr rows (at least one) and walks the rows with a
// grid stride, so the grid is sized to the SM count times the resident CTAs.
//
// Arithmetic follows the bodies these kernels replace
// (helion_mlir_utils/normalization.py): softmax = exp(x - rowmax) * (1 / sum)
// (lines 52-72: multiply by the reciprocal), GroupNorm = two-pass mean then
// biased variance of the centred values (lines 114-122), everything in f32 with
// one rounding to the output type.
#include <cstdio>

#include "common.cuh"

namespace b200 {
namespace {

enum RowOp { kSoftmax = 0, kGroupNorm = 1, kRmsNorm = 2 };

struct RowParams {
  const void* x;
  void* y;
  int64_t rows;    // logical rows (M, or M*groups for GroupNorm)
  int64_t n;       // row length
  int64_t ld;      // elements between rows
  int64_t groups;  // GroupNorm: rows per parameter period
  const void* weight;
  const void* bias;
  const void* extra;
  int32_t param_bf16;  // element type of weight/bias/extra
  int32_t extra_op;
  int32_t act;
  float alpha;
  float eps;
  int32_t tpr;        // threads per row
  int32_t param_vec;  // weight/bias/extra are 16-byte aligned: vector loads
  int32_t part;       // lean kernel: consecutive row groups per CTA (0: the grid strides over the rows)
};

__device__ __forceinline__ float load_param(const void* p, int64_t i, int bf16) {
  return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
              : reinterpret_cast<const float*>(p)[i];
}

constexpr int kMaxWarpsPerRow = 32;
constexpr int64_t kRowBytesInFlight = 48 * 1024;  // per SM, for the kernels that load a row ahead

// Reduces `v` over the `tpr` threads of a row. `scratch` has room for
// rows_per_cta * warps_per_row floats. Every thread of the CTA must call this.
template <bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float* scratch, int warps_per_row, int row_in_cta,
                                            int warp_in_row, int lane, int width = 32) {
  // `width` = min(tpr, 32) lanes hold the row: rows narrower than a warp share it.
  for (int o = width >> 1; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, other) : v + other;
  }
  if (warps_per_row <= 1) return v;
  if (lane == 0) scratch[row_in_cta * warps_per_row + warp_in_row] = v;
  __syncthreads();
  // Fixed order over the warps of the row: every thread gets the same bits.
  float r = scratch[row_in_cta * warps_per_row];
  for (int w = 1; w < warps_per_row; ++w) {
    const float o = scratch[row_in_cta * warps_per_row + w];
    r = IS_MAX ? fmaxf(r, o) : r + o;
  }
  return r;
}

// EPV parameters (weight / bias / extra) starting at element `i` as floats.
// `vec`: the pointer is 16-byte aligned and `i` a multiple of EPV, so one or two
// vector loads (cached: every row reads the same parameters) replace EPV scalar ones.
template <int EPV>
__device__ __forceinline__ void load_params(const void* p, int64_t i, int bf16, bool vec, float (&out)[EPV]) {
  if (EPV > 1 && vec) {
    if (bf16) {
      if (EPV == 8) {
        unpack16(ld_plain16(static_cast<const __nv_bfloat16*>(p) + i), reinterpret_cast<float(&)[8]>(out));
      } else {  // 4 bf16 = 8 bytes
        const uint2 q = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + i);
        out[0] = __uint_as_float(q.x << 16);
        out[1] = __uint_as_float(q.x & 0xffff0000u);
        out[2 % EPV] = __uint_as_float(q.y << 16);
        out[3 % EPV] = __uint_as_float(q.y & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int j = 0; j < EPV; j += 4) {
        const float4 q = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i + j);
        out[j] = q.x;
        out[(j + 1) % EPV] = q.y;
        out[(j + 2) % EPV] = q.z;
        out[(j + 3) % EPV] = q.w;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < EPV; ++j) out[j] = load_param(p, i + j, bf16);
  }
}

// VPT values per thread held in registers. VEC: 16-byte accesses (rows 16-byte
// aligned and n a multiple of the vector width), else element accesses. FULL:
// n == tpr * VPT, so no lane is masked. MAXT: the largest CTA the instantiation
// is launched with (register budget).
template <typename T, bool VEC, int VPT, int OP, int MAXT, bool FULL>
__global__ void __launch_bounds__(MAXT) rowwise_kernel(const RowParams p) {
  constexpr int EPV = VEC ? Elem<T>::kVec : 1;
  constexpr int NV = VPT / EPV;
  constexpr float kLog2e = 1.4426950408889634f;
  static_assert(NV >= 1, "values per thread below one vector");
  __shared__ float red_a[kMaxWarpsPerRow];
  __shared__ float red_b[kMaxWarpsPerRow];

  const int tpr = p.tpr;
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int t = threadIdx.x - row_in_cta * tpr;
  const int lane = threadIdx.x & 31;
  const int warps_per_row = tpr >> 5;
  const int width = tpr < 32 ? tpr : 32;
  const int warp_in_row = t >> 5;
  const T* __restrict__ x = reinterpret_cast<const T*>(p.x);
  T* __restrict__ y = reinterpret_cast<T*>(p.y);
  const int n = static_cast<int>(p.n);
  const float inv_n = 1.f / static_cast<float>(n);
  const int col0 = t * EPV;          // first column of this thread
  const int col_step = tpr * EPV;    // columns between its vectors
  const bool pvec = p.param_vec != 0;

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_cta; base < p.rows;
       base += static_cast<int64_t>(gridDim.x) * rows_per_cta) {
    const int64_t row = base + row_in_cta;
    const bool live = row < p.rows;
    const T* xr = x + row * p.ld + col0;
    T* yr = y + row * p.ld + col0;

    float v[NV][EPV];
    bool have[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      have[i] = live && (FULL || col0 + i * col_step < n);
      if constexpr (VEC) {
        if (have[i]) {
          float tmp[EPV];
          unpack16(ld_stream16(xr + i * col_step), tmp);
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[i][j] = tmp[j];
        }
      } else {
        if (have[i]) v[i][0] = Elem<T>::load(xr + i * col_step);
      }
    }

    if (OP == kSoftmax) {
      // NaN needs no special care in the maximum: a NaN element makes its own
      // exponential NaN, hence the row sum and every output of the row, as torch gives.
      float top = -INFINITY;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) top = fmaxf(top, v[i][j]);
        }
      top = row_reduce<true>(top, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
      // exp(x - top) = 2^((x - top) * log2e): the difference first, so that it is
      // exact near the maximum whatever the magnitude of the row.
      float total = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) {
            v[i][j] = fast_exp2((v[i][j] - top) * kLog2e);
            total += v[i][j];
          }
        }
      total = row_reduce<false>(total, red_b, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float inv = 1.f / total;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV; ++j) v[i][j] *= inv;
    } else if (OP == kGroupNorm) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) s += v[i][j];
        }
      s = row_reduce<false>(s, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float mean = s * inv_n;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) {
            v[i][j] -= mean;
            q = fmaf(v[i][j], v[i][j], q);
          }
        }
      q = row_reduce<false>(q, red_b, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float rstd = rsqrtf(q * inv_n + p.eps);
      const int64_t chan0 = (p.groups > 1 ? (row % p.groups) : 0) * n + col0;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
          const int64_t c = chan0 + i * col_step;
          float w[EPV], b[EPV], e[EPV];
          if (p.weight) load_params<EPV>(p.weight, c, p.param_bf16, pvec, w);
          if (p.bias) load_params<EPV>(p.bias, c, p.param_bf16, pvec, b);
          if (p.extra_op != B200_NORM_EXTRA_NONE) load_params<EPV>(p.extra, c, p.param_bf16, pvec, e);
#pragma unroll
          for (int j = 0; j < EPV; ++j) {
            float r = v[i][j] * rstd;
            if (p.weight) r *= w[j];
            if (p.bias) r += b[j];
            if (p.extra_op == B200_NORM_EXTRA_ADD) r += e[j];
            if (p.extra_op == B200_NORM_EXTRA_MUL) r *= e[j];
            v[i][j] = r;
          }
          if (p.act != B200_ACT_IDENTITY) {
#pragma unroll
            for (int j = 0; j < EPV; ++j) v[i][j] = apply_act(p.act, v[i][j], p.alpha);
          }
        }
    } else {  // kRmsNorm
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) q = fmaf(v[i][j], v[i][j], q);
        }
      q = row_reduce<false>(q, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float rstd = rsqrtf(q * inv_n + p.eps);
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (have[i]) {
          float w[EPV];
          if (p.weight) load_params<EPV>(p.weight, col0 + i * col_step, p.param_bf16, pvec, w);
#pragma unroll
          for (int j = 0; j < EPV; ++j) {
            float r = v[i][j] * rstd;
            if (p.weight) r *= w[j];
            v[i][j] = r;
          }
        }
      // red_b is untouched by this op: keep the two-barrier cadence the other
      // ops have so the next row's first reduction cannot overtake readers.
      if (warps_per_row > 1) __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (!have[i]) continue;
      if constexpr (VEC) {
        float tmp[EPV];
#pragma unroll
        for (int j = 0; j < EPV; ++j) tmp[j] = v[i][j];
        st_stream16(yr + i * col_step, pack16(tmp));
      } else {
        Elem<T>::store(yr + i * col_step, v[i][0]);
      }
    }
  }
}

// The common case without any masking or run-time feature tests: whole vectors
// (n == tpr * VPT), 16-byte aligned rows and parameters, weight (and bias) present,
// no extra operand, no activation. PT is the parameters' element type.
template <int EPV, typename PT>
__device__ __forceinline__ void load_param_vec(const PT* p, float (&out)[EPV]) {
  constexpr int PER = 16 / sizeof(PT);  // parameters per 16-byte load
  if constexpr (EPV == PER) {
    unpack16(ld_plain16(p), out);
  } else if constexpr (EPV == 2 * PER) {  // 8 bf16 values with f32 parameters: two loads
    const uint4 lo = ld_plain16(p), hi = ld_plain16(p + PER);
    out[0] = __uint_as_float(lo.x);
    out[1] = __uint_as_float(lo.y);
    out[2] = __uint_as_float(lo.z);
    out[3] = __uint_as_float(lo.w);
    out[4] = __uint_as_float(hi.x);
    out[5] = __uint_as_float(hi.y);
    out[6] = __uint_as_float(hi.z);
    out[7] = __uint_as_float(hi.w);
  } else {  // 4 f32 values with bf16 parameters: 8 bytes
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    out[0] = __uint_as_float(q.x << 16);
    out[1] = __uint_as_float(q.x & 0xffff0000u);
    out[2] = __uint_as_float(q.y << 16);
    out[3] = __uint_as_float(q.y & 0xffff0000u);
  }
}

// TAIL: n < tpr * VPT, so the last vectors of some threads lie beyond the row. They are
// not loaded but filled with the neutral value of the reduction (-inf for the maximum,
// whose exponential is 0; 0 for the sums), left out of the centred sum of squares, and
// neither read their parameters nor are stored.
template <typename T, typename PT, int VPT, int OP, int MAXT, bool TAIL>
__global__ void __launch_bounds__(MAXT) rowwise_lean_kernel(const RowParams p) {
  constexpr int EPV = Elem<T>::kVec;
  constexpr int NV = VPT / EPV;
  constexpr uint32_t kFillWord = OP != kSoftmax ? 0u : (sizeof(T) == 2 ? 0xff80ff80u : 0xff800000u);
  constexpr float kLog2e = 1.4426950408889634f;
  // bf16 norms keep the row in its 16-bit form and widen it again in each pass where that
  // buys resident CTAs or avoids spills: 56 or 64 values per thread with a tail (as f32 beside
  // the next row's loads they spilt 216 to 432 bytes per thread; layer_norm of [8388, 32000]
  // ran at 2.3 TB/s), and 32 values per thread in CTAs of 256 (80 instead of 92 registers,
  // three CTAs per SM instead of two: layer_norm [65536, 4096] 5778 -> 6041 GB/s, [32768, 8192]
  // 5620 -> 5881; rms_norm 6276 -> 6403).
  constexpr bool LAZY = sizeof(T) == 2 && OP != kSoftmax && ((TAIL && VPT >= 56) || (VPT == 32 && MAXT == 256));
  __shared__ float red_a[kMaxWarpsPerRow];
  __shared__ float red_b[kMaxWarpsPerRow];
  const int tpr = p.tpr;
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int t = threadIdx.x - row_in_cta * tpr;
  const int lane = threadIdx.x & 31;
  const int warps_per_row = tpr >> 5;
  const int width = tpr < 32 ? tpr : 32;
  const int warp_in_row = t >> 5;
  const int col0 = t * EPV, col_step = tpr * EPV;
  const T* __restrict__ x = reinterpret_cast<const T*>(p.x) + col0;
  T* __restrict__ y = reinterpret_cast<T*>(p.y) + col0;
  const PT* __restrict__ weight = reinterpret_cast<const PT*>(p.weight) + col0;
  const PT* __restrict__ bias = reinterpret_cast<const PT*>(p.bias) + col0;
  const float inv_n = 1.f / static_cast<float>(p.n);
  const int n = static_cast<int>(p.n);
  auto within = [&](int i) { return !TAIL || col0 + i * col_step < n; };
  const uint4 fill = make_uint4(kFillWord, kFillWord, kFillWord, kFillWord);

  // The next row's loads are issued before this row's reductions, so that a CTA
  // always has a row in flight (twice the bytes in flight for NV more registers).
  // p.part > 0: a CTA takes p.part consecutive groups of rows_per_cta rows and ends; else the
  // grid strides over the rows.
  const int64_t row_stride = p.part > 0 ? rows_per_cta : static_cast<int64_t>(gridDim.x) * rows_per_cta;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * rows_per_cta * (p.part > 0 ? p.part : 1);
  const int64_t row_end = p.part > 0 && first + static_cast<int64_t>(p.part) * rows_per_cta < p.rows
                              ? first + static_cast<int64_t>(p.part) * rows_per_cta : p.rows;
  uint4 raw[NV];
  {
    const int64_t r0 = first + row_in_cta;
    const T* xr = x + (r0 < p.rows ? r0 : p.rows - 1) * p.ld;  // dead rows re-read a valid row, store nothing
#pragma unroll
    for (int i = 0; i < NV; ++i) raw[i] = within(i) ? ld_stream16(xr + i * col_step) : fill;
  }
  for (int64_t base = first; base < row_end; base += row_stride) {
    const int64_t row = base + row_in_cta;
    const bool live = row < p.rows;
    const int64_t row_c = live ? row : p.rows - 1;
    float v[NV][EPV];
    uint4 held[LAZY ? NV : 1];
    if constexpr (LAZY) {
#pragma unroll
      for (int i = 0; i < NV; ++i) held[i] = raw[i];
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) unpack16(raw[i], v[i]);
    }
    if (base + row_stride < row_end) {
      const int64_t rn = row + row_stride;
      const T* xn = x + (rn < p.rows ? rn : p.rows - 1) * p.ld;
#pragma unroll
      for (int i = 0; i < NV; ++i) raw[i] = within(i) ? ld_stream16(xn + i * col_step) : fill;
    }

    if (OP == kSoftmax) {
      float top = -INFINITY;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV; ++j) top = fmaxf(top, v[i][j]);
      top = row_reduce<true>(top, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
      // (x - top) * log2e, the sums and the final scaling on pairs (packed f32x2).
      const uint64_t neg_top2 = pack_f32x2(-top, -top), log2e2 = pack_f32x2(kLog2e, kLog2e);
      uint64_t pair[NV][EPV / 2];
      uint64_t total2 = 0;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          float a, b;
          unpack_f32x2(mul_f32x2(add_f32x2(pack_f32x2(v[i][2 * j], v[i][2 * j + 1]), neg_top2), log2e2), a, b);
          pair[i][j] = pack_f32x2(fast_exp2(a), fast_exp2(b));
          total2 = add_f32x2(total2, pair[i][j]);
        }
      float t_lo, t_hi;
      unpack_f32x2(total2, t_lo, t_hi);
      const float total = row_reduce<false>(t_lo + t_hi, red_b, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float inv = 1.f / total;
      const uint64_t inv2 = pack_f32x2(inv, inv);
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) unpack_f32x2(mul_f32x2(pair[i][j], inv2), v[i][2 * j], v[i][2 * j + 1]);
    } else if (LAZY) {
      // The row stays in its 16-bit form (half the registers) and is widened again in each of
      // the passes; the operations per value and their order are those of the branches below.
      auto widen = [&](int i, uint64_t (&out)[EPV / 2]) {
        float f[EPV];
        unpack16(held[i], f);
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) out[j] = pack_f32x2(f[2 * j], f[2 * j + 1]);
      };
      uint64_t centre2 = 0;  // (-mean, -mean) for group_norm, (0, 0) for rms_norm
      if (OP == kGroupNorm) {
        uint64_t s2 = 0;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          uint64_t w2[EPV / 2];
          widen(i, w2);
#pragma unroll
          for (int j = 0; j < EPV / 2; ++j) s2 = add_f32x2(s2, w2[j]);
        }
        float s_lo, s_hi;
        unpack_f32x2(s2, s_lo, s_hi);
        const float s = row_reduce<false>(s_lo + s_hi, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
        const float mean = s * inv_n;
        centre2 = pack_f32x2(-mean, -mean);
      }
      uint64_t q2 = 0;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (!within(i)) continue;
        uint64_t w2[EPV / 2];
        widen(i, w2);
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          const uint64_t d = OP == kGroupNorm ? add_f32x2(w2[j], centre2) : w2[j];
          q2 = fma_f32x2(d, d, q2);
        }
      }
      float q_lo, q_hi;
      unpack_f32x2(q2, q_lo, q_hi);
      const float q = row_reduce<false>(q_lo + q_hi, OP == kGroupNorm ? red_b : red_a, warps_per_row, row_in_cta,
                                        warp_in_row, lane, width);
      const float rstd = rsqrtf(q * inv_n + p.eps);
      const uint64_t rstd2 = pack_f32x2(rstd, rstd);
      const int chan0 = OP == kGroupNorm && p.groups > 1 ? static_cast<int>(row_c % p.groups) * static_cast<int>(p.n) : 0;
      T* yr = y + row * p.ld;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (!within(i)) continue;
        uint64_t w2[EPV / 2];
        widen(i, w2);
        float w[EPV], b[EPV], out[EPV];
        load_param_vec<EPV, PT>(weight + chan0 + i * col_step, w);
        if (OP == kGroupNorm) load_param_vec<EPV, PT>(bias + chan0 + i * col_step, b);
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          const uint64_t d = OP == kGroupNorm ? add_f32x2(w2[j], centre2) : w2[j];
          const uint64_t scaled = mul_f32x2(d, rstd2), gain = pack_f32x2(w[2 * j], w[2 * j + 1]);
          w2[j] = OP == kGroupNorm ? fma_f32x2(scaled, gain, pack_f32x2(b[2 * j], b[2 * j + 1])) : mul_f32x2(scaled, gain);
        }
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) unpack_f32x2(w2[j], out[2 * j], out[2 * j + 1]);
        if (live) st_stream16(yr + i * col_step, pack16(out));
      }
      if (OP == kRmsNorm && warps_per_row > 1) __syncthreads();  // same two-barrier cadence as the other ops
    } else if (OP == kGroupNorm) {
      // The arithmetic runs on pairs (packed f32x2 instructions: one issue slot for two
      // values; the bf16 kernels are bound by instruction issue, not by HBM). Per value
      // the operations and their order are those of the scalar form: sum, centre,
      // sum of squares, scale, multiply-add with weight and bias.
      uint64_t pair[NV][EPV / 2];
      uint64_t s2 = 0;  // (+0, +0)
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          pair[i][j] = pack_f32x2(v[i][2 * j], v[i][2 * j + 1]);
          s2 = add_f32x2(s2, pair[i][j]);
        }
      float s_lo, s_hi;
      unpack_f32x2(s2, s_lo, s_hi);
      const float s = row_reduce<false>(s_lo + s_hi, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float mean = s * inv_n;
      const uint64_t neg_mean2 = pack_f32x2(-mean, -mean);
      uint64_t q2 = 0;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          pair[i][j] = add_f32x2(pair[i][j], neg_mean2);
          if (within(i)) q2 = fma_f32x2(pair[i][j], pair[i][j], q2);
        }
      float q_lo, q_hi;
      unpack_f32x2(q2, q_lo, q_hi);
      const float q = row_reduce<false>(q_lo + q_hi, red_b, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float rstd = rsqrtf(q * inv_n + p.eps);
      const uint64_t rstd2 = pack_f32x2(rstd, rstd);
      const int chan0 = p.groups > 1 ? static_cast<int>(row_c % p.groups) * static_cast<int>(p.n) : 0;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (!within(i)) continue;
        float w[EPV], b[EPV];
        load_param_vec<EPV, PT>(weight + chan0 + i * col_step, w);
        load_param_vec<EPV, PT>(bias + chan0 + i * col_step, b);
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j)
          unpack_f32x2(fma_f32x2(mul_f32x2(pair[i][j], rstd2), pack_f32x2(w[2 * j], w[2 * j + 1]),
                                 pack_f32x2(b[2 * j], b[2 * j + 1])),
                       v[i][2 * j], v[i][2 * j + 1]);
      }
    } else {
      uint64_t pair[NV][EPV / 2];
      uint64_t q2 = 0;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          pair[i][j] = pack_f32x2(v[i][2 * j], v[i][2 * j + 1]);
          q2 = fma_f32x2(pair[i][j], pair[i][j], q2);
        }
      float q_lo, q_hi;
      unpack_f32x2(q2, q_lo, q_hi);
      const float q = row_reduce<false>(q_lo + q_hi, red_a, warps_per_row, row_in_cta, warp_in_row, lane, width);
      const float rstd = rsqrtf(q * inv_n + p.eps);
      const uint64_t rstd2 = pack_f32x2(rstd, rstd);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if (!within(i)) continue;
        float w[EPV];
        load_param_vec<EPV, PT>(weight + i * col_step, w);
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j)
          unpack_f32x2(mul_f32x2(mul_f32x2(pair[i][j], rstd2), pack_f32x2(w[2 * j], w[2 * j + 1])), v[i][2 * j],
                       v[i][2 * j + 1]);
      }
      if (warps_per_row > 1) __syncthreads();  // same two-barrier cadence as the other ops
    }
    if (live && !LAZY) {
      T* yr = y + row * p.ld;
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (within(i)) st_stream16(yr + i * col_step, pack16(v[i]));
    }
  }
}

// Sums `v[0..R)` over the threads of a row group, as row_reduce does for one value: every
// thread of the group gets the same bits. `scratch` holds R floats per warp of the CTA.
template <int R>
__device__ __forceinline__ void row_reduce_sums(float (&v)[R], float* scratch, int warps_per_row, int group,
                                                int warp_in_row, int lane, int width) {
  for (int o = width >> 1; o > 0; o >>= 1) {
#pragma unroll
    for (int k = 0; k < R; ++k) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
  }
  if (warps_per_row <= 1) return;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < R; ++k) scratch[(group * warps_per_row + warp_in_row) * R + k] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < R; ++k) {
    float r = scratch[group * warps_per_row * R + k];
    for (int w = 1; w < warps_per_row; ++w) r += scratch[(group * warps_per_row + w) * R + k];
    v[k] = r;
  }
}

// LayerNorm / RMSNorm of bf16 rows, two consecutive rows per group of `tpr` threads: a thread
// holds the same columns of both rows, so the parameters of those columns are loaded and
// widened once for the two (with f32 parameters the one-row form is bound by L1 bandwidth:
// four bytes of weight and bias per byte of x). Per value the
// operations and their order are those of rowwise_lean_kernel. Whole vectors, vector
// parameters, weight (and bias) present, one parameter set for all rows (groups == 1).
template <typename T, typename PT, int VPT, int OP, bool TAIL>
__global__ void __launch_bounds__(256) rowwise_pair_kernel(const RowParams p) {
  static_assert(OP != kSoftmax, "the norms only");
  constexpr int EPV = Elem<T>::kVec;
  constexpr int NV = VPT / EPV;
  constexpr int R = 2;
  __shared__ float red_a[8 * R];
  __shared__ float red_b[8 * R];
  const int tpr = p.tpr;
  const int groups_per_cta = blockDim.x / tpr;
  const int group = threadIdx.x / tpr;
  const int t = threadIdx.x - group * tpr;
  const int lane = threadIdx.x & 31;
  const int warps_per_row = tpr >> 5;
  const int width = tpr < 32 ? tpr : 32;
  const int warp_in_row = t >> 5;
  const int col0 = t * EPV, col_step = tpr * EPV;
  const T* __restrict__ x = reinterpret_cast<const T*>(p.x) + col0;
  T* __restrict__ y = reinterpret_cast<T*>(p.y) + col0;
  const PT* __restrict__ weight = reinterpret_cast<const PT*>(p.weight) + col0;
  const PT* __restrict__ bias = reinterpret_cast<const PT*>(p.bias) + col0;
  const float inv_n = 1.f / static_cast<float>(p.n);
  const int n = static_cast<int>(p.n);
  auto within = [&](int i) { return !TAIL || col0 + i * col_step < n; };
  const uint4 zeros = make_uint4(0u, 0u, 0u, 0u);
  const int64_t rows_per_cta = static_cast<int64_t>(groups_per_cta) * R;
  const int64_t row_stride = static_cast<int64_t>(gridDim.x) * rows_per_cta;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * rows_per_cta;
  uint4 raw[R][NV];
  auto fetch = [&](int64_t base) {  // rows past the end re-read the last row, store nothing
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const int64_t r = base + group * R + k;
      const T* xr = x + (r < p.rows ? r : p.rows - 1) * p.ld;
#pragma unroll
      for (int i = 0; i < NV; ++i) raw[k][i] = within(i) ? ld_stream16(xr + i * col_step) : zeros;
    }
  };
  fetch(first);
  for (int64_t base = first; base < p.rows; base += row_stride) {
    const int64_t row0 = base + group * R;
    uint64_t pair[R][NV][EPV / 2];
#pragma unroll
    for (int k = 0; k < R; ++k)
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        float f[EPV];
        unpack16(raw[k][i], f);
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) pair[k][i][j] = pack_f32x2(f[2 * j], f[2 * j + 1]);
      }
    if (base + row_stride < p.rows) fetch(base + row_stride);

    if (OP == kGroupNorm) {
      float s[R];
#pragma unroll
      for (int k = 0; k < R; ++k) {
        uint64_t s2 = 0;
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
          for (int j = 0; j < EPV / 2; ++j) s2 = add_f32x2(s2, pair[k][i][j]);
        float lo, hi;
        unpack_f32x2(s2, lo, hi);
        s[k] = lo + hi;
      }
      row_reduce_sums<R>(s, red_a, warps_per_row, group, warp_in_row, lane, width);
#pragma unroll
      for (int k = 0; k < R; ++k) {
        const float mean = s[k] * inv_n;
        const uint64_t neg_mean2 = pack_f32x2(-mean, -mean);
#pragma unroll
        for (int i = 0; i < NV; ++i)
#pragma unroll
          for (int j = 0; j < EPV / 2; ++j) pair[k][i][j] = add_f32x2(pair[k][i][j], neg_mean2);
      }
    }
    float q[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      uint64_t q2 = 0;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j)
          if (within(i)) q2 = fma_f32x2(pair[k][i][j], pair[k][i][j], q2);
      float lo, hi;
      unpack_f32x2(q2, lo, hi);
      q[k] = lo + hi;
    }
    row_reduce_sums<R>(q, OP == kGroupNorm ? red_b : red_a, warps_per_row, group, warp_in_row, lane, width);
    uint64_t rstd2[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const float rstd = rsqrtf(q[k] * inv_n + p.eps);
      rstd2[k] = pack_f32x2(rstd, rstd);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (!within(i)) continue;
      float w[EPV], b[EPV];
      load_param_vec<EPV, PT>(weight + i * col_step, w);
      if (OP == kGroupNorm) load_param_vec<EPV, PT>(bias + i * col_step, b);
#pragma unroll
      for (int k = 0; k < R; ++k) {
        float out[EPV];
#pragma unroll
        for (int j = 0; j < EPV / 2; ++j) {
          const uint64_t scaled = mul_f32x2(pair[k][i][j], rstd2[k]), gain = pack_f32x2(w[2 * j], w[2 * j + 1]);
          unpack_f32x2(OP == kGroupNorm ? fma_f32x2(scaled, gain, pack_f32x2(b[2 * j], b[2 * j + 1])) : mul_f32x2(scaled, gain),
                       out[2 * j], out[2 * j + 1]);
        }
        if (row0 + k < p.rows) st_stream16(y + (row0 + k) * p.ld + i * col_step, pack16(out));
      }
    }
    if (OP == kRmsNorm && warps_per_row > 1) __syncthreads();  // two barriers per row pair, as the other op
  }
}

// Rows too long for registers: one CTA of 1024 threads per row, two passes over the
// row for softmax and RMSNorm, three for GroupNorm (mean, centred variance, output);
// the later passes hit L2 for rows up to tens of MB. VEC: 16-byte accesses.
template <typename T, int OP, bool VEC>
__global__ void __launch_bounds__(1024) rowwise_long_kernel(const RowParams p) {
  constexpr int EPV = VEC ? Elem<T>::kVec : 1;
  constexpr float kLog2e = 1.4426950408889634f;
  __shared__ float red_a[kMaxWarpsPerRow];
  __shared__ float red_b[kMaxWarpsPerRow];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* x = reinterpret_cast<const T*>(p.x);
  T* y = reinterpret_cast<T*>(p.y);
  const int64_t n = p.n;
  const int64_t first = static_cast<int64_t>(threadIdx.x) * EPV, step = static_cast<int64_t>(blockDim.x) * EPV;
  const float inv_n = 1.f / static_cast<float>(n);
  auto load = [](const T* at, float (&v)[EPV]) {
    if constexpr (VEC) {
      unpack16(ld_plain16(at), v);
    } else {
      v[0] = Elem<T>::load(at);
    }
  };
  auto store = [](T* at, const float (&v)[EPV]) {
    if constexpr (VEC) {
      st_stream16(at, pack16(v));
    } else {
      Elem<T>::store(at, v[0]);
    }
  };
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* xr = x + row * p.ld;
    T* yr = y + row * p.ld;
    if (OP == kSoftmax) {
      // One pass for maximum and sum: each thread keeps the sum relative to its own
      // running maximum and rescales it when the maximum grows.
      float top = -INFINITY, sum = 0.f;
#pragma unroll 2
      for (int64_t c = first; c < n; c += step) {
        float v[EPV];
        load(xr + c, v);
        float vmax = v[0];
#pragma unroll
        for (int j = 1; j < EPV; ++j) vmax = fmaxf(vmax, v[j]);
        if (vmax > top) {
          sum *= fast_exp2((top - vmax) * kLog2e);  // top = -inf: sum was 0 and stays 0
          top = vmax;
        }
#pragma unroll
        for (int j = 0; j < EPV; ++j) sum += (v[j] == -INFINITY) ? 0.f : fast_exp2((v[j] - top) * kLog2e);
      }
      const float row_top = row_reduce<true>(top, red_a, warps, 0, warp, lane);
      const float scaled = (top == -INFINITY) ? sum : sum * fast_exp2((top - row_top) * kLog2e);
      const float total = row_reduce<false>(scaled, red_b, warps, 0, warp, lane);
      const float inv = 1.f / total;
#pragma unroll 2
      for (int64_t c = first; c < n; c += step) {
        float v[EPV];
        load(xr + c, v);
#pragma unroll
        for (int j = 0; j < EPV; ++j) v[j] = fast_exp2((v[j] - row_top) * kLog2e) * inv;
        store(yr + c, v);
      }
    } else if (OP == kGroupNorm) {
      float s = 0.f;
#pragma unroll 2
      for (int64_t c = first; c < n; c += step) {
        float v[EPV];
        load(xr + c, v);
#pragma unroll
        for (int j = 0; j < EPV; ++j) s += v[j];
      }
      s = row_reduce<false>(s, red_a, warps, 0, warp, lane);
      const float mean = s * inv_n;
      float q = 0.f;
#pragma unroll 2
      for (int64_t c = first; c < n; c += step) {
        float v[EPV];
        load(xr + c, v);
#pragma unroll
        for (int j = 0; j < EPV; ++j) {
          const float d = v[j] - mean;
          q += d * d;
        }
      }
      q = row_reduce<false>(q, red_b, warps, 0, warp, lane);
      const float rstd = rsqrtf(q * inv_n + p.eps);
      const int64_t chan0 = (p.groups > 1 ? (row % p.groups) : 0) * n;
      for (int64_t c = first; c < n; c += step) {
        float v[EPV], w[EPV];
        load(xr + c, v);
#pragma unroll
        for (int j = 0; j < EPV; ++j) v[j] = (v[j] - mean) * rstd;
        if (p.weight) {
          load_params<EPV>(p.weight, chan0 + c, p.param_bf16, p.param_vec, w);
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] *= w[j];
        }
        if (p.bias) {
          load_params<EPV>(p.bias, chan0 + c, p.param_bf16, p.param_vec, w);
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] += w[j];
        }
        if (p.extra_op != B200_NORM_EXTRA_NONE) {
          load_params<EPV>(p.extra, chan0 + c, p.param_bf16, p.param_vec, w);
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] = p.extra_op == B200_NORM_EXTRA_ADD ? v[j] + w[j] : v[j] * w[j];
        }
#pragma unroll
        for (int j = 0; j < EPV; ++j) v[j] = apply_act(p.act, v[j], p.alpha);
        store(yr + c, v);
      }
    } else {
      float q = 0.f;
#pragma unroll 2
      for (int64_t c = first; c < n; c += step) {
        float v[EPV];
        load(xr + c, v);
#pragma unroll
        for (int j = 0; j < EPV; ++j) q += v[j] * v[j];
      }
      q = row_reduce<false>(q, red_a, warps, 0, warp, lane);
      const float rstd = rsqrtf(q * inv_n + p.eps);
      for (int64_t c = first; c < n; c += step) {
        float v[EPV], w[EPV];
        load(xr + c, v);
#pragma unroll
        for (int j = 0; j < EPV; ++j) v[j] *= rstd;
        if (p.weight) {
          load_params<EPV>(p.weight, c, p.param_bf16, p.param_vec, w);
#pragma unroll
          for (int j = 0; j < EPV; ++j) v[j] *= w[j];
        }
        store(yr + c, v);
      }
      __syncthreads();
    }
    // In-place rows: all reads of this row by this CTA are done (each thread
    // re-reads only the columns it writes), so no extra barrier is needed.
  }
}

template <typename T, bool VEC, int VPT, int OP, int MAXT, bool FULL>
int launch_rowwise_full(const RowParams& p, int cta_threads, cudaStream_t stream) {
  const int rows_per_cta = cta_threads / p.tpr;
  int per_sm = 0;
  auto kernel = rowwise_kernel<T, VEC, VPT, OP, MAXT, FULL>;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, cta_threads, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int64_t wanted = ceil_div(p.rows, rows_per_cta);
  const int64_t resident = static_cast<int64_t>(device_info().sm_count) * per_sm;
  const unsigned grid = static_cast<unsigned>(wanted < resident ? wanted : resident);
  kernel<<<grid, cta_threads, 0, stream>>>(p);
  return launched();
}

template <typename T, typename PT, int VPT, int OP, int MAXT, bool TAIL>
int launch_rowwise_lean(const RowParams& p, int cta_threads, cudaStream_t stream) {
  const int rows_per_cta = cta_threads / p.tpr;
  int per_sm = 0;
  auto kernel = rowwise_lean_kernel<T, PT, VPT, OP, MAXT, TAIL>;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, cta_threads, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int64_t wanted = ceil_div(p.rows, rows_per_cta);
  // No more resident CTAs per SM than put kRowBytesInFlight of loads in flight (each thread
  // keeps the next row's VPT values in flight while it reduces this row's). For the six
  // kernels of [32768, 4096] that is three CTAs of 256 threads x 64 bytes; a fourth (the f32
  // softmax and rms_norm fit four) made them 1.5 % slower together (6038 against 6131 GB/s;
  // two CTAs: 5815, one: 4260).
  const int64_t cta_bytes = static_cast<int64_t>(cta_threads) * VPT * sizeof(T);
  const int enough = static_cast<int>(ceil_div(kRowBytesInFlight, cta_bytes));
  if (per_sm > enough) per_sm = enough;
  const int64_t resident = static_cast<int64_t>(device_info().sm_count) * per_sm;
  // f32 rows, and bf16 rows that share a warp, run faster when a CTA takes a few consecutive
  // row groups and ends than when a grid of resident CTAs strides over all rows in step
  // (GB/s, softmax / layer_norm / rms_norm: f32 [32768, 4096] 6317 / 6342 / 6091 -> 6657 / 6276 /
  // 6650 with two groups per CTA; f32 [16384, 8192] 5872 / 5682 / 5806 -> 6461 / 6264 / 6470
  // with four; bf16 [262144, 1024] 6041 / 5875 / 6081 -> 6538 / 6147 / 6697; wider bf16 rows
  // lose: [65536, 4096] 6193 / 5779 / 6322 -> 6001 / 5482 / 6355). One group per CTA fetches
  // nothing ahead and 16 or 32 groups approach the strided form again.
  // (bf16 rows of 768 values, 24 per thread, lose too: layer_norm 6188 -> 5536.) Two groups
  // where three CTAs are resident, four where two are and for group_norm (f32 layer_norm of
  // 4096 columns: 6020 with two, 6320 with four); a single resident CTA strides.
  const bool chunked = (sizeof(T) == 4 || (p.tpr <= 32 && VPT == 32)) && per_sm >= 2;
  const int chunk = chunked ? (per_sm >= 3 && OP != kGroupNorm ? 2 : 4) : 0;
  if (chunk > 0 && wanted > resident * chunk) {
    RowParams q = p;
    q.part = chunk;
    kernel<<<static_cast<unsigned>(ceil_div(wanted, chunk)), cta_threads, 0, stream>>>(q);
    return launched();
  }
  kernel<<<static_cast<unsigned>(wanted < resident ? wanted : resident), cta_threads, 0, stream>>>(p);
  return launched();
}

template <typename T, typename PT, int VPT, int OP, bool TAIL>
int launch_rowwise_pair(const RowParams& p, int cta_threads, cudaStream_t stream) {
  const int64_t rows_per_cta = static_cast<int64_t>(cta_threads / p.tpr) * 2;
  int per_sm = 0;
  auto kernel = rowwise_pair_kernel<T, PT, VPT, OP, TAIL>;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, cta_threads, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int64_t cta_bytes = static_cast<int64_t>(cta_threads) * VPT * 2 * sizeof(T);
  const int enough = static_cast<int>(ceil_div(kRowBytesInFlight, cta_bytes));
  if (per_sm > enough) per_sm = enough;
  const int64_t wanted = ceil_div(p.rows, rows_per_cta);
  const int64_t resident = static_cast<int64_t>(device_info().sm_count) * per_sm;
  kernel<<<static_cast<unsigned>(wanted < resident ? wanted : resident), cta_threads, 0, stream>>>(p);
  return launched();
}

// Threads per row (whole warps) and values per thread for a row of `n` elements that no
// power-of-two number of threads covers exactly (768, 5120, 11008, 12288 ...). An exact
// cover (n == tpr * vpt) is looked for first, then one whose last vectors partly lie beyond
// the row. Either way the lean kernel applies, where the masked kernel, which keeps no row in
// flight ahead, ran at 1.3 to 3.4 TB/s (bf16, 10240 to 12288 columns). Values per thread are
// tried in the order 64, 96 or 128, then 48 or 32, then 16 bytes of loads per thread; the
// first whose resident CTAs (by an estimate of the registers) put 40 KB in flight is taken,
// else the one with the most. {0, 0}: none (rows shorter than a warp's vectors). Measured
// (TB/s, softmax / layer_norm / rms_norm, about 1 GB of rows), masked kernel -> this:
// bf16 768: 4.8 / 2.5 / 3.7 -> 5.8 / 6.2 / 5.9; bf16 12288: 3.5 / 1.4 / 2.8 -> 6.2 / 5.9 / 6.4;
// f32 5120: 6.2 / 3.1 / 4.2 -> 5.8 / 5.6 / 5.8; f32 11008 (a tail): 4.8 / 3.5 / 3.0 -> 5.3 / 5.0 / 6.1.
// Values per thread of f32 rows are tried from 16: [32768, 4096] as 128 threads x 32 values
// ran at 5.8 / 5.6 / 5.8 against 6.2 / 6.3 / 6.0 as 256 x 16.
struct RowCover {
  int tpr, vpt;
};
inline RowCover row_cover(int64_t n, int elem_bytes) {
  const int epv = 16 / elem_bytes;
  const int order_f32[4] = {16, 24, 32, 8}, order_bf16[5] = {32, 64, 24, 16, 8};
  const int* order = elem_bytes == 2 ? order_bf16 : order_f32;
  const int count = elem_bytes == 2 ? 5 : 4;
  for (int tail = 0; tail < 2; ++tail) {
    RowCover best{0, 0};
    int64_t best_bytes = 0;
    for (int k = 0; k < count; ++k) {
      const int vpt = order[k];
      int64_t tpr;
      if (!tail) {
        if (n % vpt) continue;
        tpr = n / vpt;
        if (tpr % 32) continue;
      } else {
        // (64 bf16 values with a tail: the norms keep the row in 16 bits there, see LAZY; held
        // as f32 they spilt and layer_norm of [24385, 11008] ran at 2.2 TB/s, now 4.9)
        tpr = ceil_div(ceil_div(n, static_cast<int64_t>(vpt)), int64_t(32)) * 32;
        if (tpr * (vpt - epv) >= n) continue;  // no thread's last vector starts within the row: fewer values do
      }
      if (tpr > (vpt >= 32 ? 512 : 256)) continue;
      const int64_t cta = tpr >= 256 ? tpr : tpr * (256 / tpr);
      const int64_t regs = vpt == 8 ? 48 : vpt == 16 ? 66 : vpt == 24 ? (elem_bytes == 4 ? 100 : 64)
                                                     : vpt == 32 ? (elem_bytes == 4 ? 128 : 104) : 128;
      int64_t ctas = 65536 / (regs * cta);
      if (ctas > 2048 / cta) ctas = 2048 / cta;
      if (ctas < 1) ctas = 1;
      const int64_t bytes = ctas * (cta / tpr) * n * elem_bytes;  // the rows that the resident CTAs hold
      if (bytes >= 40 * 1024) return RowCover{static_cast<int>(tpr), vpt};
      if (bytes > best_bytes) {
        best_bytes = bytes;
        best = RowCover{static_cast<int>(tpr), vpt};
      }
    }
    if (best.tpr) return best;
  }
  return RowCover{0, 0};
}

// Threads per row, values per thread and CTA size for rows of `n` elements of `elem_bytes`
// (host arithmetic only; `vec`: 16-byte accesses are possible). two_pass: the row does not fit
// the registers of 512 threads and takes the one-CTA-per-row kernel.
struct RowPlan {
  int tpr, vpt, cta_threads;
  bool two_pass;
};

// Whether the two-rows-per-group form takes a layer_norm (see launch_rowwise).
inline bool pair_case(int elem_bytes, int op, const RowPlan& plan, bool param_bf16, int64_t groups) {
  return elem_bytes == 2 && op == kGroupNorm && plan.vpt == 32 && plan.cta_threads <= 256 && !param_bf16 && groups <= 1 &&
         (plan.cta_threads / plan.tpr) % 2 == 0;
}

// Whether the lean kernel applies: whole vectors, vector parameters, plain affine form.
inline bool lean_case(const RowParams& p, int op, int vpt, int epv) {
  if (p.n > static_cast<int64_t>(p.tpr) * vpt || vpt % epv) return false;
  if (op == kSoftmax) return true;
  if (!p.param_vec || p.extra_op != B200_NORM_EXTRA_NONE || p.act != B200_ACT_IDENTITY || !p.weight) return false;
  if (op == kGroupNorm) return p.bias != nullptr && p.groups * p.n < (int64_t(1) << 30);
  return true;
}

template <typename T, bool VEC, int VPT, int OP, int MAXT>
int launch_rowwise(const RowParams& p, int cta_threads, cudaStream_t stream) {
  if constexpr (VEC) {
    if constexpr (sizeof(T) == 2 && VPT == 32 && OP == kGroupNorm && MAXT == 256) {
      // bf16 rows of up to 4096 values with f32 weight and bias: the same threads as two rows of
      // 16 values each, so that the parameters (four bytes from L1 per byte of x) are loaded
      // once for two rows. layer_norm, GB/s: [65536, 4096] 3890 -> 5142, [262144, 1024] 4874 ->
      // 5464, [2097152, 128] 5101 -> 5879. With bf16 parameters the one-row form is faster (5806
      // against 5159 at 4096 columns), and rms_norm gains nothing either way.
      if (lean_case(p, OP, VPT, Elem<T>::kVec) &&
          pair_case(sizeof(T), OP, RowPlan{p.tpr, VPT, cta_threads, false}, p.param_bf16 != 0, p.groups)) {
        RowParams q = p;
        q.tpr = 2 * p.tpr;
        return p.n != static_cast<int64_t>(p.tpr) * VPT ? launch_rowwise_pair<T, float, 16, OP, true>(q, cta_threads, stream)
                                                        : launch_rowwise_pair<T, float, 16, OP, false>(q, cta_threads, stream);
      }
    }
    if (lean_case(p, OP, VPT, Elem<T>::kVec)) {
      if (p.n == static_cast<int64_t>(p.tpr) * VPT) {
        if (p.param_bf16) return launch_rowwise_lean<T, __nv_bfloat16, VPT, OP, MAXT, false>(p, cta_threads, stream);
        return launch_rowwise_lean<T, float, VPT, OP, MAXT, false>(p, cta_threads, stream);
      }
      if (p.param_bf16) return launch_rowwise_lean<T, __nv_bfloat16, VPT, OP, MAXT, true>(p, cta_threads, stream);
      return launch_rowwise_lean<T, float, VPT, OP, MAXT, true>(p, cta_threads, stream);
    }
  }
  return launch_rowwise_full<T, VEC, VPT, OP, MAXT, false>(p, cta_threads, stream);
}

template <typename T, bool VEC, int OP>
int dispatch_vpt(const RowParams& p, int vpt, int cta_threads, cudaStream_t stream) {
  switch (vpt) {
    case 8:
      return launch_rowwise<T, VEC, 8, OP, 256>(p, cta_threads, stream);
    case 16:
      return launch_rowwise<T, VEC, 16, OP, 256>(p, cta_threads, stream);
    case 24:  // three (bf16) or six (f32) vectors: rows of 768, 1536, 3072 ... elements
      return launch_rowwise<T, VEC, 24, OP, 256>(p, cta_threads, stream);
    case 40:  // bf16 rows of 512 threads whose length is no multiple of 512 x 64: the fewest
    case 48:  // vectors per thread that cover the row (64 values with a tail spill in the norms:
    case 56:  // layer_norm of [13421, 20000] ran at 1.6 TB/s)
      if constexpr (sizeof(T) == 2 && VEC) {
        if (vpt == 40) return launch_rowwise<T, VEC, 40, OP, 512>(p, cta_threads, stream);
        if (vpt == 48) return launch_rowwise<T, VEC, 48, OP, 512>(p, cta_threads, stream);
        return launch_rowwise<T, VEC, 56, OP, 512>(p, cta_threads, stream);
      }
      [[fallthrough]];
    case 64:  // bf16 rows only: 64 f32 values beside their 16-byte loads do not fit 128 registers
      if constexpr (sizeof(T) == 2) return launch_rowwise<T, VEC, 64, OP, 512>(p, cta_threads, stream);
      return refuse(B200_E_SHAPE);
    default:
      if (cta_threads > 256) return launch_rowwise<T, VEC, 32, OP, 512>(p, cta_threads, stream);  // tpr = 512: 128 registers per thread, no spills
      return launch_rowwise<T, VEC, 32, OP, 256>(p, cta_threads, stream);
  }
}

inline RowPlan plan_rows(int64_t n, int elem_bytes, bool vec) {
  const int kvec = 16 / elem_bytes;
  const int64_t units = vec ? n / kvec : n;  // accesses per row
  const int per_unit = vec ? kvec : 1;
  // Threads per row: up to 256 at 16 values per thread, then 32 values per
  // thread, then wider CTAs (which are held to 64 registers per thread).
  // (bf16 rows aim at 32 values per thread from the start: 64 bytes of loads in flight per
  // thread, as for f32, and half as many warps to reduce across)
  const int first = elem_bytes == 2 && vec ? 32 : 16;
  const int units16 = first / per_unit > 0 ? first / per_unit : 1, units32 = 32 / per_unit;
  // Rows of less than a warp's worth of values share a warp (down to 4 threads per row).
  int tpr = 4;
  while (tpr < 256 && static_cast<int64_t>(tpr) * units16 < units) tpr <<= 1;
  while (tpr < 512 && static_cast<int64_t>(tpr) * units32 < units) tpr <<= 1;
  const int64_t per_thread_units = ceil_div(units, tpr);
  const int64_t vpt_needed = per_thread_units * per_unit;
  // 512 threads (128 registers per thread, one CTA per SM) hold up to 32 f32 or 64 bf16
  // values each; longer rows go through the two-pass kernel. Measured at 32768 columns:
  // bf16 5.5 TB/s in registers against 3.9 for the two passes; f32 4.0 (64 values spill)
  // against 5.0; a 1024-thread CTA, held to 64 registers, 3.7.
  if (vpt_needed > (elem_bytes == 2 ? 64 : 32)) return RowPlan{1024, 0, 1024, true};
  int vpt = vpt_needed <= 8 ? 8 : (vpt_needed <= 16 ? 16 : (vpt_needed <= 32 ? 32 : 64));
  if (elem_bytes == 2 && vec && vpt == 64) vpt = static_cast<int>(round_up(vpt_needed, 8));  // 40, 48, 56 or 64
  int cta_threads = tpr > 256 ? tpr : 256;
  // The power-of-two cover above is kept where it is exact, but for bf16 rows of 512 threads
  // x 32 values: one such CTA fits an SM and keeps 32 KB in flight (layer_norm of
  // [8192, 16384]: 4.45 TB/s), two CTAs of 256 x 64 keep 64 KB (5.84 TB/s).
  const bool exact = n == static_cast<int64_t>(tpr) * vpt;
  if (vec && tpr >= 32 && (!exact || (elem_bytes == 2 && tpr == 512 && vpt == 32))) {
    const RowCover cover = row_cover(n, elem_bytes);
    if (cover.tpr) {
      tpr = cover.tpr;
      vpt = cover.vpt;
      cta_threads = tpr >= 256 ? tpr : tpr * (256 / tpr);
    }
  }
  return RowPlan{tpr, vpt, cta_threads, false};
}

template <typename T, int OP>
int run_rowwise(RowParams p, cudaStream_t stream) {
  if (p.rows == 0 || p.n == 0) return finish(0);
  const DeviceInfo& dev = device_info();
  if (dev.sm_count == 0) return refuse(B200_E_DEVICE);
  const int kvec = Elem<T>::kVec;
  const bool vec = (p.n % kvec == 0) && (p.ld % kvec == 0) && aligned(p.x, 16) && aligned(p.y, 16);
  const RowPlan plan = plan_rows(p.n, sizeof(T), vec);
  p.param_vec = vec && aligned(p.weight, 16) && aligned(p.bias, 16) && aligned(p.extra, 16);
  p.tpr = plan.tpr;
  if (plan.two_pass) {
    const int64_t resident = static_cast<int64_t>(dev.sm_count) * 2;
    const unsigned grid = static_cast<unsigned>(p.rows < resident ? p.rows : resident);
    if (vec)
      rowwise_long_kernel<T, OP, true><<<grid, 1024, 0, stream>>>(p);
    else
      rowwise_long_kernel<T, OP, false><<<grid, 1024, 0, stream>>>(p);
    return launched();
  }
  if (vec) return dispatch_vpt<T, true, OP>(p, plan.vpt, plan.cta_threads, stream);
  return dispatch_vpt<T, false, OP>(p, plan.vpt, plan.cta_threads, stream);
}

template <int OP>
int run_rowwise_dtype(int32_t dtype, const RowParams& p, cudaStream_t stream) {
  if (dtype == B200_F32) return run_rowwise<float, OP>(p, stream);
  return run_rowwise<__nv_bfloat16, OP>(p, stream);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_softmax(int32_t dtype, const void* x, void* y, int64_t m, int64_t n, int64_t ld, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype)) return refuse(B200_E_DTYPE);
  if (m < 0 || n < 0) return refuse(B200_E_SHAPE);
  if (m == 0 || n == 0) return finish(0);
  if (!x || !y) return refuse(B200_E_NULL);
  if (ld < n) return refuse(B200_E_STRIDE);
  if (!aligned(x, dtype_size(dtype)) || !aligned(y, dtype_size(dtype))) return refuse(B200_E_ALIGN);
  RowParams p{};
  p.x = x;
  p.y = y;
  p.rows = m;
  p.n = n;
  p.ld = ld;
  p.groups = 1;
  return run_rowwise_dtype<kSoftmax>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_group_norm(int32_t dtype, int32_t param_dtype, const void* x, void* y, int64_t m, int64_t groups,
                               int64_t group_size, const void* weight, const void* bias, const void* extra,
                               int32_t extra_op, int32_t act, float alpha, float eps, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype) || !valid_dtype(param_dtype)) return refuse(B200_E_DTYPE);
  if (m < 0 || groups < 1 || group_size < 0) return refuse(B200_E_SHAPE);
  if (extra_op < 0 || extra_op > B200_NORM_EXTRA_MUL || act < 0 || act >= B200_ACT_COUNT_) return refuse(B200_E_ARG);
  if (m == 0 || group_size == 0) return finish(0);
  if (!x || !y || (extra_op != B200_NORM_EXTRA_NONE && !extra)) return refuse(B200_E_NULL);
  RowParams p{};
  p.x = x;
  p.y = y;
  p.rows = m * groups;
  p.n = group_size;
  p.ld = group_size;
  p.groups = groups;
  p.weight = weight;
  p.bias = bias;
  p.extra = extra;
  p.param_bf16 = param_dtype == B200_BF16;
  p.extra_op = extra_op;
  p.act = act;
  p.alpha = alpha;
  p.eps = eps;
  return run_rowwise_dtype<kGroupNorm>(dtype, p, static_cast<cudaStream_t>(stream));
}

extern "C" int b200_rowwise_explain(int32_t op, int32_t dtype, int32_t param_dtype, const void* x, const void* y,
                                    int64_t n, int64_t ld, int64_t groups, const void* weight, const void* bias,
                                    const void* extra, int32_t extra_op, int32_t act, char* out, size_t out_len) {
  if (!out || out_len == 0) return B200_E_NULL;
  out[0] = 0;
  if (op < kSoftmax || op > kRmsNorm) return B200_E_ARG;
  if (!valid_dtype(dtype) || !valid_dtype(param_dtype)) return B200_E_DTYPE;
  if (n < 1 || ld < n) return B200_E_SHAPE;
  const int size = static_cast<int>(dtype_size(dtype)), kvec = 16 / size;
  const bool vec = (n % kvec == 0) && (ld % kvec == 0) && aligned(x, 16) && aligned(y, 16);
  const RowPlan plan = plan_rows(n, size, vec);
  if (plan.two_pass) {
    snprintf(out, out_len, "rowwise_long_kernel: one CTA of 1024 threads per row, %d sweeps, %s accesses",
             op == kGroupNorm ? 3 : 2, vec ? "16-byte" : "element");
    return 0;
  }
  RowParams p{};
  p.n = n;
  p.tpr = plan.tpr;
  p.groups = groups < 1 ? 1 : groups;
  p.weight = weight;
  p.bias = bias;
  p.extra_op = extra_op;
  p.act = act;
  p.param_bf16 = param_dtype == B200_BF16;
  p.param_vec = vec && aligned(weight, 16) && aligned(bias, 16) && aligned(extra, 16);
  const bool lean = vec && lean_case(p, op, plan.vpt, kvec);
  const bool tail = n != static_cast<int64_t>(plan.tpr) * plan.vpt;
  if (lean && pair_case(size, op, plan, p.param_bf16 != 0, p.groups)) {
    snprintf(out, out_len, "rowwise_pair_kernel: two rows per group of %d threads x 16 values, %d groups per CTA of %d threads%s",
             2 * plan.tpr, plan.cta_threads / (2 * plan.tpr), plan.cta_threads, tail ? ", tail" : "");
    return 0;
  }
  const bool lazy = lean && size == 2 && op != kSoftmax &&
                    ((tail && plan.vpt >= 56) || (plan.vpt == 32 && plan.cta_threads <= 256));
  snprintf(out, out_len, "%s: %d threads x %d values per row, %d rows per CTA of %d threads%s%s",
           lean ? "rowwise_lean_kernel" : (vec ? "rowwise_kernel (masked)" : "rowwise_kernel (masked, element accesses)"), plan.tpr,
           plan.vpt, plan.cta_threads / plan.tpr, plan.cta_threads, lean && tail ? ", tail" : "", lazy ? ", row kept in 16 bits" : "");
  return 0;
}

extern "C" int b200_rms_norm(int32_t dtype, int32_t param_dtype, const void* x, void* y, int64_t m, int64_t n,
                             const void* weight, float eps, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype) || !valid_dtype(param_dtype)) return refuse(B200_E_DTYPE);
  if (m < 0 || n < 0) return refuse(B200_E_SHAPE);
  if (m == 0 || n == 0) return finish(0);
  if (!x || !y) return refuse(B200_E_NULL);
  RowParams p{};
  p.x = x;
  p.y = y;
  p.rows = m;
  p.n = n;
  p.ld = n;
  p.groups = 1;
  p.weight = weight;
  p.param_bf16 = param_dtype == B200_BF16;
  p.eps = eps;
  return run_rowwise_dtype<kRmsNorm>(dtype, p, static_cast<cudaStream_t>(stream));
}
