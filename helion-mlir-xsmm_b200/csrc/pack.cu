// Layout conversions for sm_100a: the packs of helion_mlir_utils/matmul.py
// (pad_2d, pack_a_blocked[_t], pack_b_blocked[_t], pack_b_blocked_vnni[_t],
// pack_b_vnni_t) and the inverse of the two VNNI layouts, used to hand VNNI
// weights to the tensor-core GEMM as plain K-contiguous [N, K].
//
// All are bit-exact copies with zero fill past the source, so they are
// HBM-bound: 2 bytes moved per byte packed. The forward packs map one thread to
// `W` consecutive destination elements (16 bytes where the layout keeps that many
// source elements adjacent); the VNNI unpacks are tiled transposes of 32-bit K
// pairs through shared memory, 128-byte segments on both sides.
#include "gemm_common.cuh"

namespace b200 {
namespace {

struct PackParams {
  const void* src;
  void* dst;
  int64_t rows, cols, ld;      // source as stored
  int64_t rows_pad, cols_pad;  // padded sizes in the source's orientation
  int64_t total;               // destination elements
  int32_t panel;
};

// Source coordinates (stored row, stored column) of destination element `o`.
template <int KIND>
__device__ __forceinline__ void source_of(const PackParams& p, int64_t o, int64_t& r, int64_t& c) {
  if (KIND == B200_PACK_PAD_2D) {
    r = o / p.cols_pad;
    c = o - r * p.cols_pad;
    return;
  }
  if (KIND == B200_PACK_B_VNNI_PANELS_T) {
    // dst [Np/P][Kp/2][P][2]; src [N,K]: rows_pad = Np, cols_pad = Kp
    const int64_t v = o & 1, nn = (o >> 1) % p.panel;
    const int64_t rest = (o >> 1) / p.panel;
    const int64_t pairs = p.cols_pad >> 1;
    const int64_t cc = rest % pairs, q = rest / pairs;
    r = q * p.panel + nn;
    c = 2 * cc + v;
    return;
  }
  const int64_t in_block = o & 1023, block = o >> 10;
  int64_t major, kb, mn, k;  // block index along M or N, along K; offsets inside
  if (KIND == B200_PACK_B_VNNI || KIND == B200_PACK_B_VNNI_T) {
    const int64_t pbit = in_block & 1, nn = (in_block >> 1) & 31, rr = in_block >> 6;
    k = 2 * rr + pbit;
    mn = nn;
  } else if (KIND == B200_PACK_A_BLOCKED || KIND == B200_PACK_A_BLOCKED_T) {
    mn = in_block >> 5;  // [32 m][32 k]
    k = in_block & 31;
  } else {
    k = in_block >> 5;  // [32 k][32 n]
    mn = in_block & 31;
  }
  // K extent in the source's orientation.
  const bool k_is_cols = (KIND == B200_PACK_A_BLOCKED || KIND == B200_PACK_B_BLOCKED_T || KIND == B200_PACK_B_VNNI_T);
  const int64_t kblocks = (k_is_cols ? p.cols_pad : p.rows_pad) >> 5;
  kb = block % kblocks;
  major = block / kblocks;
  const int64_t gm = major * 32 + mn, gk = kb * 32 + k;
  if (k_is_cols) {
    r = gm;
    c = gk;
  } else {
    r = gk;
    c = gm;
  }
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256) pack_gather_kernel(const PackParams p) {
  const T* __restrict__ src = static_cast<const T*>(p.src);
  T* __restrict__ dst = static_cast<T*>(p.dst);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < p.total; o += stride) {
    int64_t r, c;
    source_of<KIND>(p, o, r, c);
    T value;
    if (r < p.rows && c < p.cols) {
      value = src[r * p.ld + c];
    } else {
      memset(&value, 0, sizeof(T));
    }
    dst[o] = value;
  }
}

// Forward packs whose destination keeps W source elements adjacent: each thread
// moves one 16-byte group when the whole group lies inside the source and both
// sides are aligned, else element by element.
template <typename T, int KIND>
__global__ void __launch_bounds__(256) pack_rows_kernel(const PackParams p) {
  constexpr int W = 16 / sizeof(T);
  const T* __restrict__ src = static_cast<const T*>(p.src);
  T* __restrict__ dst = static_cast<T*>(p.dst);
  const int64_t groups = p.total / W;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g < groups; g += stride) {
    int64_t r, c;
    source_of<KIND>(p, g * W, r, c);
    const T* s = src + r * p.ld + c;
    if (r < p.rows && c + W <= p.cols && ((reinterpret_cast<uintptr_t>(s) & 15) == 0)) {
      st_stream16(dst + g * W, ld_stream16(s));
    } else {
#pragma unroll
      for (int j = 0; j < W; ++j) {
        T value;
        if (r < p.rows && c + j < p.cols) {
          value = s[j];
        } else {
          memset(&value, 0, sizeof(T));
        }
        dst[g * W + j] = value;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Transposing packs through shared memory. A CTA moves a tile of 32 source rows by
// 512 bytes: the read phase takes 16-byte vectors along the source rows (a warp
// reads one row's 512 bytes), the write phase 16-byte vectors along the source
// columns, which is the direction the destination is contiguous in. UNIT is the
// size of what is transposed: one element, or a bf16 K pair (4 bytes) for VNNI.
// Shared rows are padded by one word, so the column gathers of the write phase are
// conflict-free; the row stores of the read phase take four wavefronts each, which
// shared memory has to spare next to an HBM stream.
//   PACK_A_BLOCKED_T  src [K, M]: dst[m/32][k/32][m%32][k%32]           (elements)
//   PACK_B_BLOCKED_T  src [N, K]: dst[n/32][k/32][k%32][n%32]           (elements)
//   PACK_B_VNNI_T     src [N, K]: dst[n/32][c][n%32] pairs, c = k/2     (panel = 32)
//   PACK_B_VNNI_PANELS_T          dst[n/P][c][n%P]  pairs
//   UNPACK_B_VNNI_PANELS_TO_NK    src[n/P][c][n%P] pairs -> dst[n][c]   (P >= 64)
// ---------------------------------------------------------------------------
template <typename T, int UNIT, int KIND>
__global__ void __launch_bounds__(256) pack_transpose_kernel(const PackParams p) {
  constexpr int kUnitsPerRow = 512 / UNIT;      // tile columns, in units
  constexpr int kVecUnits = 16 / UNIT;          // units per 16-byte vector
  constexpr int kElemsPerUnit = UNIT / static_cast<int>(sizeof(T));
  constexpr int kPitchWords = 128 + 1;
  constexpr int kRunVectors = 32 * UNIT / 16;   // vectors in a destination run of 32 units
  __shared__ uint32_t tile[32 * kPitchWords];
  const T* __restrict__ src = static_cast<const T*>(p.src);
  uint8_t* __restrict__ dst = static_cast<uint8_t*>(p.dst);
  const int64_t row0 = static_cast<int64_t>(blockIdx.y) * 32;            // first source row of the tile
  const int64_t unit0 = static_cast<int64_t>(blockIdx.x) * kUnitsPerRow;  // first source column, in units

  // ---- read: 32 rows x 32 vectors
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int v = threadIdx.x + 256 * i;
    const int r = v >> 5, cv = (v & 31) * kVecUnits;
    const int64_t row = row0 + r;
    const int64_t col = (unit0 + cv) * kElemsPerUnit;  // first element of the vector
    constexpr int kVecElems = 16 / static_cast<int>(sizeof(T));
    uint4 q = make_uint4(0, 0, 0, 0);
    if (KIND == B200_UNPACK_B_VNNI_PANELS_TO_NK) {
      // source [panel z][pair row][p.panel columns] of K pairs, all of it valid and 16-byte aligned
      if (row < (p.cols_pad >> 1) && unit0 + cv < p.panel)
        q = ld_stream16(reinterpret_cast<const uint32_t*>(p.src) +
                        (static_cast<int64_t>(blockIdx.z) * (p.cols_pad >> 1) + row) * p.panel + unit0 + cv);
    } else if (row < p.rows && col < p.cols) {
      const T* at = src + row * p.ld + col;
      if (col + kVecElems <= p.cols && (reinterpret_cast<uintptr_t>(at) & 15) == 0) {
        q = ld_stream16(at);
      } else {
        T e[kVecElems];
#pragma unroll
        for (int j = 0; j < kVecElems; ++j) {
          if (col + j < p.cols) {
            e[j] = at[j];
          } else {
            memset(&e[j], 0, sizeof(T));
          }
        }
        memcpy(&q, e, 16);
      }
    }
    uint32_t* w = &tile[r * kPitchWords + (cv * UNIT) / 4];
    w[0] = q.x;
    w[1] = q.y;
    w[2] = q.z;
    w[3] = q.w;
  }
  __syncthreads();

  // ---- write: for every source column a run of 32 units, 16 bytes per thread
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int w = threadIdx.x + 256 * i;
    const int g = w % kRunVectors, c = w / kRunVectors;
    const int64_t unit = unit0 + c;  // source column of this run, in units
    uint32_t out[4];
    if (UNIT == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) out[k] = tile[(g * 4 + k) * kPitchWords + c];
    } else {
      const uint16_t* halves = reinterpret_cast<const uint16_t*>(tile);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t lo = halves[(g * 8 + 2 * k) * kPitchWords * 2 + c];
        const uint32_t hi = halves[(g * 8 + 2 * k + 1) * kPitchWords * 2 + c];
        out[k] = lo | (hi << 16);
      }
    }
    int64_t offset;  // destination offset of the run's first unit, in units
    bool inside;
    if (KIND == B200_PACK_A_BLOCKED_T) {
      // source rows are k, columns m: row0 / 32 is the K block
      const int64_t kblocks = p.rows_pad >> 5;
      inside = unit < p.cols_pad;
      offset = (((unit >> 5) * kblocks + (row0 >> 5)) << 10) + ((unit & 31) << 5);
    } else if (KIND == B200_PACK_B_BLOCKED_T) {
      // source rows are n, columns k
      const int64_t kblocks = p.cols_pad >> 5;
      inside = unit < p.cols_pad;
      offset = (((row0 >> 5) * kblocks + (unit >> 5)) << 10) + ((unit & 31) << 5);
    } else if (KIND == B200_UNPACK_B_VNNI_PANELS_TO_NK) {
      // source rows are pairs, columns the panel's n: dst32[z * panel + n][pair]
      inside = unit < p.panel && row0 + g * kVecUnits < (p.cols_pad >> 1);  // the last tile of pairs may be short
      offset = (static_cast<int64_t>(blockIdx.z) * p.panel + unit) * (p.cols_pad >> 1) + row0;
    } else {
      // K pairs: source rows are n, columns pairs; panels of p.panel rows (32 for the blocked VNNI layout)
      const int64_t pairs = p.cols_pad >> 1;
      const int64_t panel = KIND == B200_PACK_B_VNNI_T ? 32 : p.panel;
      inside = unit < pairs;
      offset = ((row0 / panel) * pairs + unit) * panel + (row0 % panel);
    }
    if (inside)
      st_stream16(dst + (offset + g * kVecUnits) * UNIT, make_uint4(out[0], out[1], out[2], out[3]));
  }
}

// [K, N] -> VNNI blocks dst[n/32][c][n%32][2], c = k/2: rows 2c and 2c+1 interleaved
// element by element. A thread takes 8 columns of both rows (16 bytes each) and
// writes 32 contiguous bytes; four lanes fill one 128-byte run of a block.
__global__ void __launch_bounds__(256) pack_vnni_rows_kernel(const PackParams p) {
  const __nv_bfloat16* __restrict__ src = static_cast<const __nv_bfloat16*>(p.src);
  uint8_t* __restrict__ dst = static_cast<uint8_t*>(p.dst);
  const int64_t pairs = p.rows_pad >> 1, groups = p.cols_pad >> 3;  // source rows are k, columns n
  const int64_t total = pairs * groups;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < total; u += stride) {
    const int64_t c = u / groups, n0 = (u - c * groups) << 3;
    uint4 rows[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t k = 2 * c + h;
      rows[h] = make_uint4(0, 0, 0, 0);
      if (k < p.rows && n0 < p.cols) {
        const __nv_bfloat16* at = src + k * p.ld + n0;
        if (n0 + 8 <= p.cols && (reinterpret_cast<uintptr_t>(at) & 15) == 0) {
          rows[h] = ld_stream16(at);
        } else {
          __nv_bfloat16 e[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) e[j] = (n0 + j < p.cols) ? at[j] : __float2bfloat16_rn(0.f);
          memcpy(&rows[h], e, 16);
        }
      }
    }
    const uint32_t a[4] = {rows[0].x, rows[0].y, rows[0].z, rows[0].w};
    const uint32_t b[4] = {rows[1].x, rows[1].y, rows[1].z, rows[1].w};
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[2 * j] = __byte_perm(a[j], b[j], 0x5410);      // (row 2c, row 2c+1) of column 2j
      out[2 * j + 1] = __byte_perm(a[j], b[j], 0x7632);  // of column 2j + 1
    }
    uint8_t* at = dst + (((n0 >> 5) * pairs + c) * 64 + (n0 & 31) * 2) * 2;
    st_stream16(at, make_uint4(out[0], out[1], out[2], out[3]));
    st_stream16(at + 16, make_uint4(out[4], out[5], out[6], out[7]));
  }
}

// VNNI -> [Np, Kp] (K contiguous), as a transpose of 32-bit K pairs:
//   blocks: src32[j][kb][r][nn]  -> dst32[32j+nn][16kb+r]
//   panels: src32[q][c][nn]      -> dst32[qP+nn][c]
// One CTA moves a 32(n) x 32(pairs) tile; grid.x walks pair tiles, grid.y n tiles.
template <bool PANELS>
__global__ void __launch_bounds__(256) unpack_vnni_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                                          int64_t n_pad, int64_t pairs, int32_t panel) {
  __shared__ uint32_t tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t n0 = static_cast<int64_t>(blockIdx.y) * 32, c0 = static_cast<int64_t>(blockIdx.x) * 32;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t c = c0 + ty + 8 * i;  // pair index
    const int64_t n = n0 + tx;
    uint32_t value = 0;
    if (c < pairs && n < n_pad) {
      int64_t off;
      if (PANELS) {
        off = ((n / panel) * pairs + c) * panel + (n % panel);
      } else {
        off = (((n >> 5) * (pairs >> 4) + (c >> 4)) * 16 + (c & 15)) * 32 + (n & 31);
      }
      value = src[off];
    }
    tile[ty + 8 * i][tx] = value;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t n = n0 + ty + 8 * i;
    const int64_t c = c0 + tx;
    if (c < pairs && n < n_pad) dst[n * pairs + c] = tile[tx][ty + 8 * i];
  }
}

// Blocked A [Mp/32][Kp/32][32][32] -> row-major [Mp][Kp]: 32-element row segments
// are contiguous on both sides; one thread moves 16 bytes.
template <typename T>
__global__ void __launch_bounds__(256) unpack_a_blocked_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                               int64_t m_pad, int64_t k_pad) {
  constexpr int W = 16 / sizeof(T);
  const int64_t units = m_pad * k_pad / W;
  const int64_t kblocks = k_pad >> 5;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += stride) {
    const int64_t e = u * W, m = e / k_pad, k = e - m * k_pad;
    const int64_t off = (((m >> 5) * kblocks + (k >> 5)) << 10) + ((m & 31) << 5) + (k & 31);
    st_stream16(dst + e, ld_stream16(src + off));
  }
}

// Blocked B [Np/32][Kp/32][32 k][32 n] -> [Np][Kp]: one 32x32 block per CTA,
// transposed through shared memory.
template <typename T>
__global__ void __launch_bounds__(256) unpack_b_blocked_kernel(const T* __restrict__ src, T* __restrict__ dst,
                                                               int64_t n_pad, int64_t k_pad) {
  __shared__ T tile[32][33];
  const int64_t kblocks = k_pad >> 5;
  const int64_t block = blockIdx.x;
  const int64_t nb = block / kblocks, kb = block - nb * kblocks;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const T* s = src + (block << 10);
#pragma unroll
  for (int i = 0; i < 4; ++i) tile[ty + 8 * i][tx] = s[(ty + 8 * i) * 32 + tx];  // [k][n]
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = ty + 8 * i;
    dst[(nb * 32 + n) * k_pad + kb * 32 + tx] = tile[tx][n];
  }
}

// f32 -> three bf16 parts x = x1 + x2 + x3 (each the bf16 rounding of what is left),
// written six times side by side along the contraction dimension so that one bf16
// GEMM over the widened K sums the six largest cross products of an f32 product:
//   A operand parts (3,2,1,2,1,1), B operand parts (1,2,3,1,2,1)
//   -> a3 b1 + a2 b2 + a1 b3 + a2 b1 + a1 b2 + a1 b1, smallest terms first so that
//      they are not absorbed by a large running sum.
// A value that is not finite, or that rounds to infinity in bf16, has no such split
// (x - bf16(x) is NaN): its products come out NaN where exact f32 gives an infinity.
//
// One launch widens both operands of a GEMM. along_cols: the contraction dimension is
// the column dimension of the logical matrix (copies side by side in a row, out
// [batch][rows][6 * k_wide]); else the row dimension (out [batch][6 * k_wide][cols]).
// k_wide >= the source's K: the rest of every copy is zero.
// A work item is eight consecutive elements of the widened operand's contiguous dimension
// (whole 16-byte pieces of bf16 on the way out, two 16-byte loads on the way in when the
// source allows).
__device__ __forceinline__ void split_eight(const SplitOperand& o, int64_t item) {
  const int64_t lead = o.along_cols ? o.rows : o.k_wide, inner = o.along_cols ? o.k_wide : o.cols;
  const int64_t inner8 = inner >> 3;
  const int64_t per_batch = lead * inner8;
  const int64_t bi = item / per_batch, rem = item - bi * per_batch;
  const int64_t r = rem / inner8, c = (rem - r * inner8) << 3;
  float x[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = 0.f;
  if (r < o.rows && c < o.cols) {
    const float* src = o.src + bi * o.batch_stride;
    if (o.layout == 2) {  // [rows/32][cols/32][32 c][32 r]: consecutive c are 32 elements apart
      const float* at = src + (((r >> 5) * o.ld + (c >> 5)) << 10) + ((c & 31) << 5) + (r & 31);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c + j < o.cols) x[j] = at[j << 5];
    } else {
      const float* at = o.layout == 0 ? src + r * o.ld + c : src + (((r >> 5) * o.ld + (c >> 5)) << 10) + ((r & 31) << 5) + (c & 31);
      if (c + 8 <= o.cols && (reinterpret_cast<uintptr_t>(at) & 15) == 0) {
        const float4 lo = *reinterpret_cast<const float4*>(at), hi = *reinterpret_cast<const float4*>(at + 4);
        x[0] = lo.x, x[1] = lo.y, x[2] = lo.z, x[3] = lo.w, x[4] = hi.x, x[5] = hi.y, x[6] = hi.z, x[7] = hi.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (c + j < o.cols) x[j] = at[j];
      }
    }
  }
  // parts[t][j]: part t (0 largest) of element j, as bf16 bits
  uint32_t packed[3][4];
#pragma unroll
  for (int j = 0; j < 8; j += 2) {
    uint32_t bits[3][2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const __nv_bfloat16 p0 = __float2bfloat16_rn(x[j + e]);
      const float r1 = x[j + e] - __bfloat162float(p0);
      const __nv_bfloat16 p1 = __float2bfloat16_rn(r1);
      const __nv_bfloat16 p2 = __float2bfloat16_rn(r1 - __bfloat162float(p1));
      bits[0][e] = __bfloat16_as_ushort(p0), bits[1][e] = __bfloat16_as_ushort(p1), bits[2][e] = __bfloat16_as_ushort(p2);
    }
#pragma unroll
    for (int t = 0; t < 3; ++t) packed[t][j >> 1] = bits[t][0] | (bits[t][1] << 16);
  }
  const int pattern_a[6] = {2, 1, 0, 1, 0, 0}, pattern_b[6] = {0, 1, 2, 0, 1, 0};
  __nv_bfloat16* dst = o.dst + bi * 6 * lead * inner;
#pragma unroll
  for (int t = 0; t < 6; ++t) {
    const int part = o.is_b ? pattern_b[t] : pattern_a[t];
    const uint4 q = make_uint4(packed[part][0], packed[part][1], packed[part][2], packed[part][3]);
    __nv_bfloat16* to = o.along_cols ? dst + r * (6 * inner) + t * inner + c : dst + (t * lead + r) * inner + c;
    *reinterpret_cast<uint4*>(to) = q;
  }
}

__global__ void __launch_bounds__(256) split_f32_kernel(const SplitOperand a, const SplitOperand b, int64_t items_a,
                                                        int64_t items) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < items; i += stride) {
    if (i < items_a)
      split_eight(a, i);
    else
      split_eight(b, i - items_a);
  }
}

template <typename T, int KIND, bool ROWS>
int launch_pack(const PackParams& p, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  const int64_t items = ROWS ? p.total / (16 / sizeof(T)) : p.total;
  const int64_t wanted = ceil_div(items, 256);
  const int64_t resident = static_cast<int64_t>(dev.sm_count) * 16;
  const unsigned grid = static_cast<unsigned>(wanted < resident ? wanted : resident);
  if (ROWS)
    pack_rows_kernel<T, KIND><<<grid, 256, 0, stream>>>(p);
  else
    pack_gather_kernel<T, KIND><<<grid, 256, 0, stream>>>(p);
  return launched();
}

// Grid of the transposing packs: source rows in blocks of 32, source columns (in
// units) in tiles of 512 bytes. Falls back to the gather kernel beyond the grid limits.
template <typename T, int UNIT, int KIND>
int launch_transpose(const PackParams& p, int64_t rows_pad, int64_t units_pad, cudaStream_t stream) {
  const int64_t tiles_r = ceil_div(rows_pad, 32), tiles_c = ceil_div(units_pad, 512 / UNIT);
  if (tiles_r > 65535 || tiles_c > 0x7fffffff) return launch_pack<T, KIND, false>(p, stream);
  const dim3 grid(static_cast<unsigned>(tiles_c), static_cast<unsigned>(tiles_r));
  pack_transpose_kernel<T, UNIT, KIND><<<grid, 256, 0, stream>>>(p);
  return launched();
}

template <typename T>
int run_pack(int kind, const PackParams& p, cudaStream_t stream) {
  constexpr int W = 16 / sizeof(T);
  const bool dst16 = aligned(p.dst, 16);
  switch (kind) {
    case B200_PACK_PAD_2D:
      if (dst16 && p.cols_pad % W == 0) return launch_pack<T, B200_PACK_PAD_2D, true>(p, stream);
      return launch_pack<T, B200_PACK_PAD_2D, false>(p, stream);
    case B200_PACK_A_BLOCKED:  // 32 k adjacent in source rows
      if (dst16) return launch_pack<T, B200_PACK_A_BLOCKED, true>(p, stream);
      return launch_pack<T, B200_PACK_A_BLOCKED, false>(p, stream);
    case B200_PACK_A_BLOCKED_T:
      if (dst16) return launch_transpose<T, sizeof(T), B200_PACK_A_BLOCKED_T>(p, p.rows_pad, p.cols_pad, stream);
      return launch_pack<T, B200_PACK_A_BLOCKED_T, false>(p, stream);
    case B200_PACK_B_BLOCKED:  // 32 n adjacent in source rows
      if (dst16) return launch_pack<T, B200_PACK_B_BLOCKED, true>(p, stream);
      return launch_pack<T, B200_PACK_B_BLOCKED, false>(p, stream);
    case B200_PACK_B_BLOCKED_T:
      if (dst16) return launch_transpose<T, sizeof(T), B200_PACK_B_BLOCKED_T>(p, p.rows_pad, p.cols_pad, stream);
      return launch_pack<T, B200_PACK_B_BLOCKED_T, false>(p, stream);
    case B200_PACK_B_VNNI:
      if (dst16 && sizeof(T) == 2) {
        const int64_t units = (p.rows_pad >> 1) * (p.cols_pad >> 3);
        const int64_t wanted = ceil_div(units, 256), resident = static_cast<int64_t>(device_info().sm_count) * 8;
        pack_vnni_rows_kernel<<<static_cast<unsigned>(wanted < resident ? wanted : resident), 256, 0, stream>>>(p);
        return launched();
      }
      return launch_pack<T, B200_PACK_B_VNNI, false>(p, stream);
    case B200_PACK_B_VNNI_T:
      // K pairs as 4-byte units need an even row pitch and a 4-byte aligned source
      if (dst16 && sizeof(T) == 2 && p.ld % 2 == 0 && aligned(p.src, 4))
        return launch_transpose<T, 4, B200_PACK_B_VNNI_T>(p, p.rows_pad, p.cols_pad >> 1, stream);
      return launch_pack<T, B200_PACK_B_VNNI_T, false>(p, stream);
    default:
      if (dst16 && sizeof(T) == 2 && p.ld % 2 == 0 && aligned(p.src, 4))
        return launch_transpose<T, 4, B200_PACK_B_VNNI_PANELS_T>(p, p.rows_pad, p.cols_pad >> 1, stream);
      return launch_pack<T, B200_PACK_B_VNNI_PANELS_T, false>(p, stream);
  }
}

}  // namespace

// Widens both f32 operands of a GEMM into their six-fold bf16 splits (see split_f32_kernel).
int launch_split_f32(const SplitOperand& a, const SplitOperand& b, cudaStream_t stream) {
  // eight elements of the contiguous dimension per work item: that dimension (the widened K,
  // or M / N of a [K, M] / [K, N] operand) is a multiple of 8 and the destinations 16-byte aligned
  auto count = [](const SplitOperand& o) {
    return o.batch * (o.along_cols ? o.rows * (o.k_wide >> 3) : o.k_wide * (o.cols >> 3));
  };
  const int64_t items_a = count(a), items = items_a + count(b);
  const int64_t wanted = ceil_div(items, 256), resident = static_cast<int64_t>(device_info().sm_count) * 16;
  const unsigned grid = static_cast<unsigned>(wanted < resident ? (wanted > 0 ? wanted : 1) : resident);
  split_f32_kernel<<<grid, 256, 0, stream>>>(a, b, items_a, items);
  return check_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_pack(int32_t kind, int32_t dtype, const void* src, int64_t rows, int64_t cols, int64_t ld,
                         void* dst, int64_t rows_pad, int64_t cols_pad, int32_t panel, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype)) return refuse(B200_E_DTYPE);
  if (kind < 0 || kind >= B200_PACK_COUNT_) return refuse(B200_E_ARG);
  if (rows < 0 || cols < 0 || rows_pad < 0 || cols_pad < 0) return refuse(B200_E_SHAPE);
  if (rows_pad == 0 || cols_pad == 0) return finish(0);
  if (!dst || (rows > 0 && cols > 0 && !src)) return refuse(B200_E_NULL);
  if (ld < cols) return refuse(B200_E_STRIDE);
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (kind == B200_UNPACK_B_VNNI_TO_NK || kind == B200_UNPACK_B_VNNI_PANELS_TO_NK) {
    // rows_pad = Np, cols_pad = Kp of the [N, K] destination; the source is the packed tensor.
    if (dtype != B200_BF16) return refuse(B200_E_DTYPE);
    const bool panels = kind == B200_UNPACK_B_VNNI_PANELS_TO_NK;
    if (cols_pad % 2) return refuse(B200_E_SHAPE);
    if (panels ? (panel <= 0 || rows_pad % panel) : (rows_pad % 32 || cols_pad % 32)) return refuse(B200_E_SHAPE);
    if (!aligned(src, 4) || !aligned(dst, 4)) return refuse(B200_E_ALIGN);
    const int64_t pairs = cols_pad / 2;
    const dim3 grid(static_cast<unsigned>(ceil_div(pairs, 32)), static_cast<unsigned>(ceil_div(rows_pad, 32)));
    if (grid.y > 65535) return refuse(B200_E_SHAPE);
    if (panels && panel >= 64 && panel % 4 == 0 && pairs % 4 == 0 && aligned(src, 16) && aligned(dst, 16) &&
        rows_pad / panel <= 65535 && ceil_div(pairs, 32) <= 65535) {
      // wide panels: the tiled transpose (16-byte accesses on both sides)
      PackParams p{};
      p.src = src;
      p.dst = dst;
      p.rows_pad = rows_pad;
      p.cols_pad = cols_pad;
      p.panel = panel;
      const dim3 tiles(static_cast<unsigned>(ceil_div(panel, 128)), static_cast<unsigned>(ceil_div(pairs, 32)),
                       static_cast<unsigned>(rows_pad / panel));
      pack_transpose_kernel<__nv_bfloat16, 4, B200_UNPACK_B_VNNI_PANELS_TO_NK><<<tiles, 256, 0, s>>>(p);
      return launched();
    }
    if (panels)
      unpack_vnni_kernel<true><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst),
                                                    rows_pad, pairs, panel);
    else
      unpack_vnni_kernel<false><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst),
                                                     rows_pad, pairs, panel);
    return launched();
  }

  if (kind == B200_UNPACK_A_BLOCKED_TO_MK || kind == B200_UNPACK_B_BLOCKED_TO_NK) {
    // rows_pad x cols_pad are Mp x Kp (A) or Np x Kp (B) of the row-major destination.
    if (rows_pad % 32 || cols_pad % 32) return refuse(B200_E_SHAPE);
    if (!aligned(src, 16) || !aligned(dst, 16)) return refuse(B200_E_ALIGN);
    const int64_t blocks = (rows_pad >> 5) * (cols_pad >> 5);
    if (kind == B200_UNPACK_A_BLOCKED_TO_MK) {
      const int64_t units = rows_pad * cols_pad / (16 / static_cast<int64_t>(dtype_size(dtype)));
      const int64_t wanted = ceil_div(units, 256), resident = static_cast<int64_t>(device_info().sm_count) * 16;
      const unsigned grid = static_cast<unsigned>(wanted < resident ? wanted : resident);
      if (dtype == B200_F32)
        unpack_a_blocked_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(src), static_cast<float*>(dst),
                                                            rows_pad, cols_pad);
      else
        unpack_a_blocked_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
            static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows_pad, cols_pad);
    } else {
      if (blocks > 0x7fffffff) return refuse(B200_E_SHAPE);
      if (dtype == B200_F32)
        unpack_b_blocked_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
            static_cast<const float*>(src), static_cast<float*>(dst), rows_pad, cols_pad);
      else
        unpack_b_blocked_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
            static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows_pad, cols_pad);
    }
    return launched();
  }

  if (rows_pad < rows || cols_pad < cols) return refuse(B200_E_SHAPE);
  if (kind == B200_PACK_B_VNNI_PANELS_T) {
    if (panel <= 0 || panel % 32 || rows_pad % panel || cols_pad % 2) return refuse(B200_E_SHAPE);
  } else if (kind != B200_PACK_PAD_2D) {
    if (rows_pad % 32 || cols_pad % 32) return refuse(B200_E_SHAPE);
  }
  PackParams p{};
  p.src = src;
  p.dst = dst;
  p.rows = rows;
  p.cols = cols;
  p.ld = ld;
  p.rows_pad = rows_pad;
  p.cols_pad = cols_pad;
  p.total = rows_pad * cols_pad;
  p.panel = panel;
  return dtype == B200_F32 ? run_pack<float>(kind, p, s) : run_pack<__nv_bfloat16>(kind, p, s);
}
