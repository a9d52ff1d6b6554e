// Row reductions (row_sum, row_dot, matvec) and column sums for sm_100a.
//
// All are one pass over x from HBM with f32 accumulation and a fixed summation
// order (thread-strided partial sums, xor-shuffle tree, then the warps of a row
// in index order), so two runs give the same bits. They replace
// _row_sum_kernel, _row_dot_kernel, _matvec_kernel and _column_sum_kernel of
// helion_mlir_utils/reduction.py.
#include <mutex>

#include <cstdio>

#include "common.cuh"

namespace b200 {
namespace {

struct ReduceParams {
  const void* x;
  const void* v;
  void* out;
  int64_t m, n, ld;
  int32_t act;
  float alpha;
  int32_t tpr;
};

// KIND: 0 row_sum, 1 row_dot (v f32), 2 matvec (v of T)
// `tpr` threads share a row (a power of two from 4 to 256): narrow rows put several
// rows in one warp so that no lane idles, wide rows spread over up to 8 warps.
template <typename T, bool VEC, int KIND>
__global__ void __launch_bounds__(256) row_reduce_kernel(const ReduceParams p) {
  constexpr int EPV = VEC ? Elem<T>::kVec : 1;
  __shared__ float red[8];
  const int tpr = p.tpr;
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int t = threadIdx.x - row_in_cta * tpr;
  const int lane = threadIdx.x & 31;
  const int warps_per_row = tpr >> 5;
  const int warp_in_row = t >> 5;
  const T* x = reinterpret_cast<const T*>(p.x);
  T* out = reinterpret_cast<T*>(p.out);
  const float* vf = reinterpret_cast<const float*>(p.v);
  const T* vt = reinterpret_cast<const T*>(p.v);
  const int64_t step = static_cast<int64_t>(tpr) * EPV;

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_cta; base < p.m;
       base += static_cast<int64_t>(gridDim.x) * rows_per_cta) {
    const int64_t row = base + row_in_cta;
    const bool live = row < p.m;
    const T* xr = x + row * p.ld;
    float acc = 0.f;
    if (live) {
#pragma unroll 4
      for (int64_t col = static_cast<int64_t>(t) * EPV; col < p.n; col += step) {
        float xv[EPV];
        if constexpr (VEC) {
          unpack16(ld_stream16(xr + col), xv);
        } else {
          xv[0] = Elem<T>::load(xr + col);
        }
        if (KIND == 0) {
#pragma unroll
          for (int j = 0; j < EPV; ++j) acc += xv[j];
        } else if (KIND == 1) {
          if constexpr (VEC) {
            // the vector in 16-byte loads too (it is re-read by every row, from L1/L2)
#pragma unroll
            for (int q = 0; q < EPV / 4; ++q) {
              const float4 w = __ldg(reinterpret_cast<const float4*>(vf + col) + q);
              acc += xv[4 * q] * w.x;
              acc += xv[4 * q + 1] * w.y;
              acc += xv[4 * q + 2] * w.z;
              acc += xv[4 * q + 3] * w.w;
            }
          } else {
            acc += xv[0] * __ldg(vf + col);
          }
        } else {
          if constexpr (VEC) {
            float wv[EPV];
            unpack16(__ldg(reinterpret_cast<const uint4*>(vt + col)), wv);
#pragma unroll
            for (int j = 0; j < EPV; ++j) acc += xv[j] * wv[j];
          } else {
            acc += xv[0] * Elem<T>::load(vt + col);
          }
        }
      }
    }
    // Sum over the row's threads: an xor tree inside the (sub-)warp, then the warps in order.
    for (int offset = (tpr < 32 ? tpr : 32) >> 1; offset > 0; offset >>= 1)
      acc += __shfl_xor_sync(0xffffffffu, acc, offset);
    if (warps_per_row > 1) {
      if (lane == 0) red[row_in_cta * warps_per_row + warp_in_row] = acc;
      __syncthreads();
      acc = red[row_in_cta * warps_per_row];
      for (int w = 1; w < warps_per_row; ++w) acc += red[row_in_cta * warps_per_row + w];
      __syncthreads();
    }
    if (live && t == 0) Elem<T>::store(out + row, apply_act(p.act, acc, p.alpha));
  }
}

// row_dot / matvec with R consecutive rows per group of `tpr` threads: a thread reads its
// columns of the vector once for the R rows (the vector's loads, from L1, were two to one
// against the row's own bytes for bf16 rows with an f32 vector, and the kernel was bound by
// them). Each row's sum is accumulated in the same order as in row_reduce_kernel.
template <typename T, bool VEC, int KIND, int R>
__global__ void __launch_bounds__(256) row_dot_rows_kernel(const ReduceParams p) {
  static_assert(KIND != 0, "row_dot and matvec only");
  constexpr int EPV = VEC ? Elem<T>::kVec : 1;
  __shared__ float red[8 * R];
  const int tpr = p.tpr;
  const int groups_per_cta = blockDim.x / tpr;
  const int group = threadIdx.x / tpr;
  const int t = threadIdx.x - group * tpr;
  const int lane = threadIdx.x & 31;
  const int warps_per_row = tpr >> 5;
  const int warp_in_row = t >> 5;
  const T* x = reinterpret_cast<const T*>(p.x);
  T* out = reinterpret_cast<T*>(p.out);
  const float* vf = reinterpret_cast<const float*>(p.v);
  const T* vt = reinterpret_cast<const T*>(p.v);
  const int64_t step = static_cast<int64_t>(tpr) * EPV;
  const int64_t rows_per_cta = static_cast<int64_t>(groups_per_cta) * R;

  for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_cta; base < p.m;
       base += static_cast<int64_t>(gridDim.x) * rows_per_cta) {
    const int64_t row0 = base + static_cast<int64_t>(group) * R;
    const T* xr[R];
#pragma unroll
    for (int k = 0; k < R; ++k) xr[k] = x + (row0 + k < p.m ? row0 + k : p.m - 1) * p.ld;  // rows past the end re-read the last
    float acc[R];
#pragma unroll
    for (int k = 0; k < R; ++k) acc[k] = 0.f;
#pragma unroll 2
    for (int64_t col = static_cast<int64_t>(t) * EPV; col < p.n; col += step) {
      float xv[R][EPV];
#pragma unroll
      for (int k = 0; k < R; ++k) {
        if constexpr (VEC) {
          unpack16(ld_stream16(xr[k] + col), xv[k]);
        } else {
          xv[k][0] = Elem<T>::load(xr[k] + col);
        }
      }
      float wv[EPV];
      if constexpr (VEC) {
        if (KIND == 1) {
#pragma unroll
          for (int q = 0; q < EPV / 4; ++q) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(vf + col) + q);
            wv[4 * q] = w.x;
            wv[4 * q + 1] = w.y;
            wv[4 * q + 2] = w.z;
            wv[4 * q + 3] = w.w;
          }
        } else {
          unpack16(__ldg(reinterpret_cast<const uint4*>(vt + col)), wv);
        }
      } else {
        wv[0] = KIND == 1 ? __ldg(vf + col) : Elem<T>::load(vt + col);
      }
#pragma unroll
      for (int k = 0; k < R; ++k)
#pragma unroll
        for (int j = 0; j < EPV; ++j) acc[k] += xv[k][j] * wv[j];
    }
    for (int offset = (tpr < 32 ? tpr : 32) >> 1; offset > 0; offset >>= 1) {
#pragma unroll
      for (int k = 0; k < R; ++k) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], offset);
    }
    if (warps_per_row > 1) {
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < R; ++k) red[(group * warps_per_row + warp_in_row) * R + k] = acc[k];
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < R; ++k) {
        float r = red[group * warps_per_row * R + k];
        for (int w = 1; w < warps_per_row; ++w) r += red[(group * warps_per_row + w) * R + k];
        acc[k] = r;
      }
      __syncthreads();
    }
    if (t == 0) {
#pragma unroll
      for (int k = 0; k < R; ++k)
        if (row0 + k < p.m) Elem<T>::store(out + row0 + k, apply_act(p.act, acc[k], p.alpha));
    }
  }
}

constexpr int kDotRows = 4;
template <typename T, bool VEC, int KIND>
int launch_row_dot_rows(const ReduceParams& p, int sm_count, cudaStream_t stream) {
  static const int per_sm = [] {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, row_dot_rows_kernel<T, VEC, KIND, kDotRows>, 256, 0) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 4;
    }
    return n;
  }();
  const int64_t wanted = ceil_div(p.m, static_cast<int64_t>(256 / p.tpr) * kDotRows);
  const int64_t resident = static_cast<int64_t>(sm_count) * per_sm;
  row_dot_rows_kernel<T, VEC, KIND, kDotRows><<<static_cast<unsigned>(wanted < resident ? wanted : resident), 256, 0, stream>>>(p);
  return launched();
}

// CTAs of 256 threads that fit one SM, asked of the runtime once per instantiation: the
// grid is persistent (rows strided by the grid), so CTAs beyond what is resident would run
// as a second, mostly empty round (row_dot on bf16 rows needs 40 registers: six CTAs per
// SM, and with a grid of eight per SM it ran at half the bandwidth of row_sum).
template <typename T, bool VEC, int KIND>
int resident_ctas_per_sm() {
  static const int per_sm = [] {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, row_reduce_kernel<T, VEC, KIND>, 256, 0) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 4;
    }
    return n;
  }();
  return per_sm;
}

template <typename T, bool VEC, int KIND>
int launch_row_reduce_kind(const ReduceParams& p, int64_t wanted, int sm_count, cudaStream_t stream) {
  const int64_t resident = static_cast<int64_t>(sm_count) * resident_ctas_per_sm<T, VEC, KIND>();
  const unsigned grid = static_cast<unsigned>(wanted < resident ? wanted : resident);
  row_reduce_kernel<T, VEC, KIND><<<grid, 256, 0, stream>>>(p);
  return launched();
}

template <typename T, bool VEC>
int launch_row_reduce(int kind, const ReduceParams& p, int64_t wanted, int sm_count, cudaStream_t stream) {
  switch (kind) {
    case B200_REDUCE_ROW_SUM:
      return launch_row_reduce_kind<T, VEC, 0>(p, wanted, sm_count, stream);
    case B200_REDUCE_ROW_DOT:
      // bf16 rows with the f32 vector: four rows per group of threads (GB/s, [65536, 4096]
      // 5031 -> 5711, [174762, 1536] 5056 -> 5975). f32 rows lose 4-8 % that way, matvec
      // (a vector of the rows' own type) gains and loses by shape: both stay one row per group.
      if constexpr (sizeof(T) == 2 && VEC) return launch_row_dot_rows<T, VEC, 1>(p, sm_count, stream);
      return launch_row_reduce_kind<T, VEC, 1>(p, wanted, sm_count, stream);
    default:
      return launch_row_reduce_kind<T, VEC, 2>(p, wanted, sm_count, stream);
  }
}

// Threads per row of the row reductions for rows of `units` accesses (see run_row_reduce).
inline int row_reduce_threads(int64_t units) {
  int tpr = 4;
  while (tpr < 256 && static_cast<int64_t>(tpr) * 8 < units) tpr <<= 1;
  return tpr;
}

template <typename T>
int run_row_reduce(int kind, ReduceParams p, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  if (dev.sm_count == 0) return refuse(B200_E_DEVICE);
  const int kvec = Elem<T>::kVec;
  const bool vec = (p.n % kvec == 0) && (p.ld % kvec == 0) && aligned(p.x, 16) && (!p.v || aligned(p.v, 16));
  const int64_t units = vec ? p.n / kvec : p.n;
  // Threads per row: each thread gets five to eight 16-byte units (rows of up to 32 units share
  // a warp). With up to four units per thread, as before, a row was spread over twice the
  // threads: half the loads in flight per thread and twice the warps to add up per row
  // (GB/s, [65536, 4096] bf16: row_sum 6184 -> 6748, row_dot 4434 -> 5036, matvec 5149 -> 6151;
  // rows of 1536, 3072 and 6144 bf16 values, three units per thread before: row_sum 4.7 -> 6.4-6.6).
  const int tpr = row_reduce_threads(units);
  p.tpr = tpr;
  const int rows_per_cta = 256 / tpr;
  const int64_t wanted = ceil_div(p.m, rows_per_cta);
  return vec ? launch_row_reduce<T, true>(kind, p, wanted, dev.sm_count, stream)
             : launch_row_reduce<T, false>(kind, p, wanted, dev.sm_count, stream);
}

// ---------------------------------------------------------------------------
// Column sums: stage 1 sums a chunk of rows per CTA into partial[s][n] (or out
// directly when there is one chunk); stage 2 adds the chunks in order.
// ---------------------------------------------------------------------------

constexpr int kColThreads = 128;
constexpr int kColTargetCtas = 1024;  // about seven CTAs per SM of a 148-SM part, for strips of 512 columns; 1024 x 512 partial sums = 2 MiB
constexpr int kColMinRows = 64;

struct ColPlan {
  int cols_per_thread;
  int tpr_log2;  // threads side by side on a row (a power of two <= kColThreads); the rest of the CTA takes other rows
  int64_t col_tiles;
  int64_t chunks;
  int64_t rows_per_chunk;
};

// `cpt`: columns per thread (1, 4, or 8 for 16-byte loads of bf16).
ColPlan column_plan(int64_t m, int64_t n, int cpt) {
  ColPlan plan;
  plan.cols_per_thread = cpt;
  const int64_t units = ceil_div(n, static_cast<int64_t>(plan.cols_per_thread));
  // Strips are 512 columns at most (64 threads of 8 bf16 columns, the CTA's other 64 taking
  // every other row): a strip of 1024 left two CTAs per SM, too few bytes in flight for HBM.
  const int side = cpt == 8 ? kColThreads / 2 : kColThreads;
  plan.tpr_log2 = 0;
  while ((1 << plan.tpr_log2) < side && (int64_t(1) << plan.tpr_log2) < units) ++plan.tpr_log2;
  plan.col_tiles = ceil_div(units, int64_t(1) << plan.tpr_log2);
  // Wider strips get fewer row chunks, so the partial sums (chunks x n floats) stay
  // within kColTargetCtas x 512 floats whatever the strip width.
  const int64_t strip = static_cast<int64_t>(cpt) << plan.tpr_log2;
  int64_t chunks = kColTargetCtas * (strip > 512 ? 512 : strip) / strip / (plan.col_tiles > 0 ? plan.col_tiles : 1);
  const int64_t max_chunks = m / kColMinRows;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  plan.rows_per_chunk = ceil_div(m, chunks);
  plan.chunks = ceil_div(m, plan.rows_per_chunk);
  return plan;
}

// A CTA sums `rows_per_chunk` rows of one column tile. Narrow tiles (fewer columns
// than the CTA has threads) are covered by several thread rows that take every
// R-th row each; their partial sums are added in thread-row order at the end, so
// the summation order is fixed.
template <typename T, int CPT, bool MULTI>
__global__ void __launch_bounds__(kColThreads) column_partial_kernel(const T* __restrict__ x, float* __restrict__ dst,
                                                                     int64_t m, int64_t n, int64_t ld,
                                                                     int64_t rows_per_chunk, int tpr_log2) {
  __shared__ float red[MULTI ? kColThreads * CPT : 1];
  // MULTI: the tile is narrower than the CTA, several thread rows share it (else one: plain row loop).
  const int tpr = 1 << tpr_log2, thread_rows = MULTI ? (kColThreads >> tpr_log2) : 1;
  const int tc = threadIdx.x & (tpr - 1), tr = threadIdx.x >> tpr_log2;
  const int64_t col = (static_cast<int64_t>(blockIdx.x) * tpr + tc) * CPT;
  const bool active = col < n;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * rows_per_chunk;
  const int64_t r1 = (r0 + rows_per_chunk < m) ? r0 + rows_per_chunk : m;
  float acc[CPT];
#pragma unroll
  for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
  if (active) {
    const T* p = x + (r0 + tr) * ld + col;
    const int64_t stride = static_cast<int64_t>(thread_rows) * ld;
#pragma unroll 8
    for (int64_t r = r0 + tr; r < r1; r += thread_rows, p += stride) {
      if (CPT == 8) {
        float v[8];
        unpack16(__ldg(reinterpret_cast<const uint4*>(p)), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j];
      } else if (CPT == 4) {
        if (sizeof(T) == 4) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(p));
          acc[0] += q.x;
          acc[1] += q.y;
          acc[2] += q.z;
          acc[3] += q.w;
        } else {
          const uint2 q = __ldg(reinterpret_cast<const uint2*>(p));
          acc[0] += __uint_as_float(q.x << 16);
          acc[1] += __uint_as_float(q.x & 0xffff0000u);
          acc[2] += __uint_as_float(q.y << 16);
          acc[3] += __uint_as_float(q.y & 0xffff0000u);
        }
      } else {
        acc[0] += Elem<T>::load(p);
      }
    }
  }
  if (MULTI) {
#pragma unroll
    for (int j = 0; j < CPT; ++j) red[threadIdx.x * CPT + j] = acc[j];
    __syncthreads();
    if (tr != 0) return;
    for (int other = 1; other < thread_rows; ++other) {
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[j] += red[(other * tpr + tc) * CPT + j];
    }
  }
  if (!active) return;
  float* d = dst + static_cast<int64_t>(blockIdx.y) * n + col;
#pragma unroll
  for (int j = 0; j < CPT; ++j) d[j] = acc[j];
}

// Stage 2: 32 columns x 8 thread rows per CTA. Thread row r adds the partial sums of the
// chunks r, r + 8, ... in ascending order, then the eight rows are added in order: a fixed
// order, and a column's chain of dependent loads is an eighth as long as with one thread
// per column (1048576 x 64: the single CTA of 64 threads took most of the call).
constexpr int kFinalCols = 32, kFinalRows = 8;
__global__ void __launch_bounds__(kFinalCols * kFinalRows)
    column_final_kernel(const float* __restrict__ partial, float* __restrict__ out, int64_t n, int64_t chunks) {
  __shared__ float red[kFinalRows][kFinalCols];
  const int tc = threadIdx.x & (kFinalCols - 1), tr = threadIdx.x / kFinalCols;
  const int64_t col = static_cast<int64_t>(blockIdx.x) * kFinalCols + tc;
  float acc = 0.f;
  if (col < n) {
#pragma unroll 4
    for (int64_t s = tr; s < chunks; s += kFinalRows) acc += partial[s * n + col];
  }
  red[tr][tc] = acc;
  __syncthreads();
  if (tr != 0 || col >= n) return;
#pragma unroll
  for (int r = 1; r < kFinalRows; ++r) acc += red[r][tc];
  out[col] = acc;
}

// Columns per thread: 8 (bf16) or 4 as one 16-byte load, 4 bf16 as an 8-byte load, else 1.
int column_cpt(int32_t dtype, const void* x, int64_t n, int64_t ld) {
  if (dtype == B200_BF16 && n % 8 == 0 && ld % 8 == 0 && aligned(x, 16)) return 8;
  const size_t bytes = 4 * dtype_size(dtype);
  return (n % 4 == 0 && ld % 4 == 0 && aligned(x, bytes)) ? 4 : 1;
}

int column_sum_impl(int32_t dtype, const void* x, float* out, int64_t m, int64_t n, int64_t ld, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream) {
  const int cpt = column_cpt(dtype, x, n, ld);
  const ColPlan plan = column_plan(m, n, cpt);
  float* stage1 = out;
  if (plan.chunks > 1) {
    const size_t need = static_cast<size_t>(plan.chunks) * n * sizeof(float);
    if (!workspace || workspace_bytes < need) return refuse(B200_E_WORKSPACE);
    if (!aligned(workspace, 16)) return refuse(B200_E_ALIGN);
    stage1 = static_cast<float*>(workspace);
  }
  const dim3 grid(static_cast<unsigned>(plan.col_tiles), static_cast<unsigned>(plan.chunks));
  const bool multi = plan.tpr_log2 < 7;  // fewer column threads than the CTA has
  auto launch = [&](auto kernel_multi, auto kernel_single, auto xs) {
    if (multi)
      kernel_multi<<<grid, kColThreads, 0, stream>>>(xs, stage1, m, n, ld, plan.rows_per_chunk, plan.tpr_log2);
    else
      kernel_single<<<grid, kColThreads, 0, stream>>>(xs, stage1, m, n, ld, plan.rows_per_chunk, plan.tpr_log2);
  };
  if (dtype == B200_F32) {
    const float* xs = static_cast<const float*>(x);
    if (cpt == 4)
      launch(column_partial_kernel<float, 4, true>, column_partial_kernel<float, 4, false>, xs);
    else
      launch(column_partial_kernel<float, 1, true>, column_partial_kernel<float, 1, false>, xs);
  } else {
    const __nv_bfloat16* xs = static_cast<const __nv_bfloat16*>(x);
    if (cpt == 8)
      launch(column_partial_kernel<__nv_bfloat16, 8, true>, column_partial_kernel<__nv_bfloat16, 8, false>, xs);
    else if (cpt == 4)
      launch(column_partial_kernel<__nv_bfloat16, 4, true>, column_partial_kernel<__nv_bfloat16, 4, false>, xs);
    else
      launch(column_partial_kernel<__nv_bfloat16, 1, true>, column_partial_kernel<__nv_bfloat16, 1, false>, xs);
  }
  if (plan.chunks > 1) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(n, kFinalCols));
    column_final_kernel<<<blocks, kFinalCols * kFinalRows, 0, stream>>>(stage1, out, n, plan.chunks);
    return launched(2);
  }
  return launched(1);
}

size_t column_sum_workspace(int64_t m, int64_t n) {
  if (m <= 0 || n <= 0) return 0;
  // Whichever vector width the operand's alignment allows at call time.
  int64_t chunks = 1;
  for (int cpt : {1, 4, 8}) {
    const ColPlan plan = column_plan(m, n, cpt);
    if (plan.chunks > chunks) chunks = plan.chunks;
  }
  return chunks > 1 ? static_cast<size_t>(chunks) * n * sizeof(float) : 0;
}

// ---------------------------------------------------------------------------
// Scratch for b200_column_sum_static: a fixed array in the library's own device
// image instead of caller-provided or freshly allocated memory. Every GPU that
// loads the library carries these bytes until the process exits.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = B200_COLUMN_SUM_STATIC_MAX_BYTES;
static __device__ __align__(256) unsigned char g_column_scratch[kStaticScratchBytes];

constexpr int kScratchDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_address[kScratchDevices];  // device address of g_column_scratch, per device (0: not looked up yet)

// The array's name is only a host-side handle here: the address kernels can use
// has to be asked for, once per device and with that device current.
int static_scratch(void** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return -static_cast<int>(err);
  if (device < 0 || device >= kScratchDevices) return B200_E_DEVICE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_address[device]) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_column_scratch);
    if (err != cudaSuccess) {
      cudaGetLastError();
      return -static_cast<int>(err);
    }
    g_scratch_address[device] = address;
  }
  *out = g_scratch_address[device];
  return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_row_reduce(int32_t kind, int32_t dtype, const void* x, const void* v, void* out, int64_t m,
                               int64_t n, int64_t ld, int32_t act, float alpha, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype)) return refuse(B200_E_DTYPE);
  if (kind < 0 || kind > B200_REDUCE_MATVEC || act < 0 || act >= B200_ACT_COUNT_) return refuse(B200_E_ARG);
  if (m < 0 || n < 0) return refuse(B200_E_SHAPE);
  if (m == 0) return finish(0);
  if (!out || (n > 0 && !x) || (kind != B200_REDUCE_ROW_SUM && n > 0 && !v)) return refuse(B200_E_NULL);
  if (ld < n) return refuse(B200_E_STRIDE);
  ReduceParams p{};
  p.x = x;
  p.v = v;
  p.out = out;
  p.m = m;
  p.n = n;
  p.ld = ld;
  p.act = act;
  p.alpha = alpha;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == B200_F32 ? run_row_reduce<float>(kind, p, s) : run_row_reduce<__nv_bfloat16>(kind, p, s);
}

extern "C" int b200_reduce_explain(int32_t kind, int32_t dtype, const void* x, const void* v, int64_t m, int64_t n,
                                   int64_t ld, char* out, size_t out_len) {
  if (!out || out_len == 0) return B200_E_NULL;
  out[0] = 0;
  if (!valid_dtype(dtype)) return B200_E_DTYPE;
  constexpr int kColumnSum = 3;  // beside the B200_REDUCE_* kinds of the row reductions
  if (kind < 0 || kind > kColumnSum) return B200_E_ARG;
  if (m < 1 || n < 1 || ld < n) return B200_E_SHAPE;
  const int size = static_cast<int>(dtype_size(dtype)), kvec = 16 / size;
  if (kind == kColumnSum) {
    const int cpt = column_cpt(dtype, x, n, ld);
    const ColPlan plan = column_plan(m, n, cpt);
    const long long strip = static_cast<long long>(cpt) << plan.tpr_log2;
    if (plan.chunks > 1)
      snprintf(out, out_len,
               "column_partial_kernel: %lld strips of %lld columns (%d per thread) x %lld chunks of %lld rows, then "
               "column_final_kernel adds the chunks in order (%zu bytes of scratch)",
               static_cast<long long>(plan.col_tiles), strip, cpt, static_cast<long long>(plan.chunks),
               static_cast<long long>(plan.rows_per_chunk), static_cast<size_t>(plan.chunks) * n * sizeof(float));
    else
      snprintf(out, out_len, "column_partial_kernel: %lld strips of %lld columns (%d per thread), one chunk of %lld rows",
               static_cast<long long>(plan.col_tiles), strip, cpt, static_cast<long long>(plan.rows_per_chunk));
    return 0;
  }
  const bool vec = (n % kvec == 0) && (ld % kvec == 0) && aligned(x, 16) && (!v || aligned(v, 16));
  const int tpr = row_reduce_threads(vec ? n / kvec : n);
  const bool four = kind == B200_REDUCE_ROW_DOT && size == 2 && vec;
  snprintf(out, out_len, "%s: %d threads per row, %d rows per CTA of 256 threads, %s accesses",
           four ? "row_dot_rows_kernel (four rows per group of threads)" : "row_reduce_kernel", tpr,
           (256 / tpr) * (four ? kDotRows : 1), vec ? "16-byte" : "element");
  return 0;
}

extern "C" size_t b200_column_sum_workspace_bytes(int64_t m, int64_t n) { return column_sum_workspace(m, n); }

extern "C" int b200_column_sum(int32_t dtype, const void* x, float* out, int64_t m, int64_t n, int64_t ld,
                               void* workspace, size_t workspace_bytes, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype)) return refuse(B200_E_DTYPE);
  if (m < 1 || n < 0) return refuse(B200_E_SHAPE);
  if (n == 0) return finish(0);
  if (!x || !out) return refuse(B200_E_NULL);
  if (ld < n) return refuse(B200_E_STRIDE);
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  return column_sum_impl(dtype, x, out, m, n, ld, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

// The size check of b200_column_sum_static, against a given capacity: 0 when the
// partial sums of an m x n column sum fit `capacity` bytes, else B200_E_TOO_LARGE.
// Pure host arithmetic (no device needed).
extern "C" int b200_column_sum_static_fits(int64_t m, int64_t n, size_t capacity) {
  return column_sum_workspace(m, n) > capacity ? B200_E_TOO_LARGE : 0;
}

// Same result as b200_column_sum, for callers that must not allocate and have no
// scratch of their own to lend: the partial sums go to the library's fixed array.
extern "C" int b200_column_sum_static(int32_t dtype, const void* x, float* out, int64_t m, int64_t n, int64_t ld,
                                      void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype)) return refuse(B200_E_DTYPE);
  if (m < 1 || n < 0) return refuse(B200_E_SHAPE);
  if (n == 0) return finish(0);
  if (!x || !out) return refuse(B200_E_NULL);
  if (ld < n) return refuse(B200_E_STRIDE);
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  // The partial sums of this shape must fit the fixed array.
  if (b200_column_sum_static_fits(m, n, kStaticScratchBytes) != 0) return refuse(B200_E_TOO_LARGE);
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != 0) return finish(rc);
  // Nothing in the array has to start at zero: stage 1 writes every partial that
  // stage 2 reads, so whatever an earlier call left behind is overwritten first.
  return column_sum_impl(dtype, x, out, m, n, ld, scratch, kStaticScratchBytes, static_cast<cudaStream_t>(stream));
}
