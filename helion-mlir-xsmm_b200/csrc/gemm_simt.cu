// Exact-f32 FFMA GEMM for sm_100a: the path for every operand the tensor-core
// kernels do not take (f32 inputs, strides TMA cannot describe, tiny problems)
// and the parity yardstick for them. 128x128x16 CTA tiles, 8x8 register tiles,
// operands read in place from any accepted layout with zero fill past M, N, K.
// bf16 operands are widened to f32 on load, products and sums are f32
// (fastmath off), one rounding at the store.
#include "gemm_common.cuh"

namespace b200 {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8;

struct SimtParams {
  GemmOperand a, b;
  GemmEpilogue epi;
  void* c;
  int64_t m, n, k;
  int64_t ldc;
  int64_t stride_a, stride_b, stride_c;
  int32_t splits;        // K splits
  int32_t to_workspace;  // 1: blockIdx.z = batch*splits + s, raw f32 partials to c
  int32_t a_bf16, out_bf16;
  int32_t a_k_contig, b_k_contig;
  int64_t k_per_split;
};

template <typename T>
__device__ __forceinline__ float fetch(const void* base, int64_t off) {
  return Elem<T>::load(static_cast<const T*>(base) + off);
}

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 8x8 outputs each
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
  int64_t batch = blockIdx.z;
  int split_lo = 0, split_hi = p.splits;
  if (p.to_workspace) {
    batch = blockIdx.z / p.splits;
    split_lo = blockIdx.z - batch * p.splits;
    split_hi = split_lo + 1;
  }
  const T* a_base = static_cast<const T*>(p.a.p) + batch * p.stride_a;
  const T* b_base = static_cast<const T*>(p.b.p) + batch * p.stride_b;

  float total[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) total[i][j] = 0.f;

  for (int s = split_lo; s < split_hi; ++s) {
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    const int64_t k_begin = s * p.k_per_split;
    const int64_t k_end = (k_begin + p.k_per_split < p.k) ? k_begin + p.k_per_split : p.k;
    for (int64_t k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
      for (int i = 0; i < (BM * BK) / 256; ++i) {
        int mm, kk;
        if (p.a_k_contig) {
          kk = tid & 15;
          mm = (tid >> 4) + 16 * i;
        } else {
          mm = tid & 127;
          kk = (tid >> 7) + 2 * i;
        }
        const int64_t gm = m0 + mm, gk = k0 + kk;
        As[kk][mm] = (gm < p.m && gk < k_end) ? fetch<T>(a_base, offset_a(p.a, gm, gk)) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < (BN * BK) / 256; ++i) {
        int nn, kk;
        if (p.b_k_contig) {
          kk = tid & 15;
          nn = (tid >> 4) + 16 * i;
        } else {
          nn = tid & 127;
          kk = (tid >> 7) + 2 * i;
        }
        const int64_t gn = n0 + nn, gk = k0 + kk;
        Bs[kk][nn] = (gn < p.n && gk < k_end) ? fetch<T>(b_base, offset_b(p.b, gk, gn)) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        float av[TM], bv[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
        for (int j = 0; j < TN; ++j) bv[j] = Bs[kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
    // The first split initialises the total, so one split adds nothing to the
    // accumulator's bits; later splits are added in ascending order.
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) total[i][j] = (s == split_lo) ? acc[i][j] : total[i][j] + acc[i][j];
  }

  if (p.to_workspace) {
    float* ws = static_cast<float*>(p.c) + (static_cast<int64_t>(split_lo) * (gridDim.z / p.splits) + batch) * p.m * p.n;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int64_t gm = m0 + ty * TM + i;
      if (gm >= p.m) continue;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int64_t gn = n0 + tx * TN + j;
        if (gn < p.n) ws[gm * p.n + gn] = total[i][j];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t gm = m0 + ty * TM + i;
    if (gm >= p.m) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int64_t gn = n0 + tx * TN + j;
      if (gn >= p.n) continue;
      const float r = run_epilogue(p.epi, total[i][j], gn);
      const int64_t off = batch * p.stride_c + gm * p.ldc + gn;
      if (p.out_bf16)
        static_cast<__nv_bfloat16*>(p.c)[off] = __float2bfloat16_rn(r);
      else
        static_cast<float*>(p.c)[off] = r;
    }
  }
}

__global__ void __launch_bounds__(256)
    splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t per_split, int64_t n, void* out,
                         int out_bf16, int64_t ldc, int64_t stride_c, int64_t mn, const GemmEpilogue epi) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < per_split; i += stride) {
    float acc = partial[i];
    for (int s = 1; s < splits; ++s) acc += partial[s * per_split + i];
    const int64_t b = i / mn, rem = i - b * mn;
    const int64_t row = rem / n, col = rem - row * n;
    const float r = run_epilogue(epi, acc, col);
    const int64_t off = b * stride_c + row * ldc + col;
    if (out_bf16)
      static_cast<__nv_bfloat16*>(out)[off] = __float2bfloat16_rn(r);
    else
      static_cast<float*>(out)[off] = r;
  }
}

}  // namespace

int launch_splitk_reduce(const float* partial, int splits, int64_t batch, int64_t m, int64_t n, void* out,
                         int out_bf16, int64_t ldc, int64_t stride_c, const GemmEpilogue& epi, cudaStream_t stream) {
  const int64_t per_split = batch * m * n;
  const int64_t wanted = ceil_div(per_split, 256);
  const int64_t resident = static_cast<int64_t>(device_info().sm_count) * 8;
  const unsigned grid = static_cast<unsigned>(wanted < resident ? wanted : resident);
  splitk_reduce_kernel<<<grid, 256, 0, stream>>>(partial, splits, per_split, n, out, out_bf16, ldc, stride_c, m * n,
                                                 epi);
  return launched();
}

// Runs the FFMA path for a validated descriptor. `splits` > 1 with `workspace`
// uses parallel partial products and the ordered reduction; without it the
// splits run in order inside each CTA.
int run_gemm_simt(const b200_gemm_desc& d, const GemmOperand& a, const GemmOperand& b, const GemmEpilogue& epi,
                  int splits, float* workspace, cudaStream_t stream) {
  SimtParams p{};
  p.a = a;
  p.b = b;
  p.epi = epi;
  p.m = d.m;
  p.n = d.n;
  p.k = d.k;
  p.ldc = d.ldc;
  p.stride_a = d.stride_a;
  p.stride_b = d.stride_b;
  p.stride_c = d.stride_c;
  p.splits = splits < 1 ? 1 : splits;
  p.k_per_split = ceil_div(d.k, p.splits);
  p.a_bf16 = d.dtype == B200_BF16;
  p.out_bf16 = d.out_dtype == B200_BF16;
  p.a_k_contig = a.layout != B200_LAYOUT_COL;
  p.b_k_contig = b.layout == B200_LAYOUT_COL;
  p.to_workspace = (p.splits > 1 && workspace) ? 1 : 0;
  p.c = p.to_workspace ? static_cast<void*>(workspace) : d.c;
  const int64_t z = d.batch * (p.to_workspace ? p.splits : 1);
  if (z > 65535 || ceil_div(d.m, BM) > 65535) return refuse(B200_E_SHAPE);
  const dim3 grid(static_cast<unsigned>(ceil_div(d.n, BN)), static_cast<unsigned>(ceil_div(d.m, BM)),
                  static_cast<unsigned>(z));
  if (d.dtype == B200_F32)
    gemm_simt_kernel<float><<<grid, 256, 0, stream>>>(p);
  else
    gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
  if (!p.to_workspace) return launched();
  const int rc = check_launch();
  if (rc != 0) return finish(rc);
  return launch_splitk_reduce(workspace, p.splits, d.batch, d.m, d.n, d.c, p.out_bf16, d.ldc, d.stride_c, epi,
                              stream);
}

}  // namespace b200
