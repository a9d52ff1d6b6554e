// Elementwise relu / leaky_relu / scalar_mul for sm_100a: one 128-bit load and
// one 128-bit store per 16 bytes, two vectors per thread, one CTA per 512 vectors. Replaces
// _relu_kernel, _leaky_relu_kernel and _scalar_mul_kernel of
// helion_mlir_utils/elementwise.py. Arithmetic is in the tensor's own type as
// torch does for these ops: f32 directly; bf16 through f32 with one rounding.
#include "common.cuh"

namespace b200 {
namespace {

template <int KIND>
__device__ __forceinline__ float elt_op(float x, float param) {
  if (KIND == B200_ELT_RELU) return (x != x) ? x : fmaxf(x, 0.f);
  if (KIND == B200_ELT_LEAKY_RELU) return x > 0.f ? x : x * param;
  return x * param;
}

// AHEAD loads are issued before the first of them is used (a thread with one load in
// flight at a time leaves 2048 threads x 16 bytes = 32 KB per SM in flight).
constexpr int kEltAhead = 2;
template <typename T, int KIND, int AHEAD>
__global__ void __launch_bounds__(256) eltwise_vec_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t vecs,
                                                           float param) {
  constexpr int EPV = Elem<T>::kVec;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += AHEAD * stride) {
    uint4 raw[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u)
      if (i + u * stride < vecs) raw[u] = ld_stream16(x + (i + u * stride) * EPV);
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      if (i + u * stride >= vecs) break;
      float v[EPV];
      unpack16(raw[u], v);
#pragma unroll
      for (int j = 0; j < EPV; ++j) v[j] = elt_op<KIND>(v[j], param);
      st_stream16(y + (i + u * stride) * EPV, pack16(v));
    }
  }
}

template <typename T, int KIND>
__global__ void __launch_bounds__(256) eltwise_scalar_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                              int64_t begin, int64_t count, float param) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = begin + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
    Elem<T>::store(y + i, elt_op<KIND>(Elem<T>::load(x + i), param));
}

template <typename T, int KIND>
int run_eltwise(const void* xv, void* yv, int64_t count, float param, cudaStream_t stream) {
  const DeviceInfo& dev = device_info();
  if (dev.sm_count == 0) return refuse(B200_E_DEVICE);
  const T* x = static_cast<const T*>(xv);
  T* y = static_cast<T*>(yv);
  constexpr int EPV = Elem<T>::kVec;
  const bool vec = aligned(x, 16) && aligned(y, 16);
  const int64_t vecs = vec ? count / EPV : 0;
  int kernels = 0;
  if (vecs > 0) {
    // One CTA per 512 vectors, not a persistent grid: measured on [32768, 4096] f32 / bf16
    // (relu, GB/s read + written): a grid of 8 CTAs per SM striding over the tensor with one
    // load in flight per thread 5848 / 5620, with four loads and 3 CTAs per SM 6121 / 6033,
    // this form with two loads per thread 6666 / 6392 (four: 6550 / 6378, one: 5837 / 5674).
    const int64_t wanted = ceil_div(vecs, int64_t(256) * kEltAhead);
    eltwise_vec_kernel<T, KIND, kEltAhead><<<static_cast<unsigned>(wanted), 256, 0, stream>>>(x, y, vecs, param);
    ++kernels;
  }
  const int64_t done = vecs * EPV;
  if (done < count) {
    const int64_t wanted = ceil_div(count - done, 256);
    const int64_t resident = static_cast<int64_t>(dev.sm_count) * 8;
    eltwise_scalar_kernel<T, KIND><<<static_cast<unsigned>(wanted < resident ? wanted : resident), 256, 0, stream>>>(
        x, y, done, count, param);
    ++kernels;
  }
  return launched(kernels);
}

template <typename T>
int run_eltwise_kind(int kind, const void* x, void* y, int64_t count, float param, cudaStream_t stream) {
  switch (kind) {
    case B200_ELT_RELU:
      return run_eltwise<T, B200_ELT_RELU>(x, y, count, param, stream);
    case B200_ELT_LEAKY_RELU:
      return run_eltwise<T, B200_ELT_LEAKY_RELU>(x, y, count, param, stream);
    default:
      return run_eltwise<T, B200_ELT_SCALAR_MUL>(x, y, count, param, stream);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_eltwise(int32_t kind, int32_t dtype, const void* x, void* y, int64_t count, float param,
                            void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!valid_dtype(dtype)) return refuse(B200_E_DTYPE);
  if (kind < 0 || kind > B200_ELT_SCALAR_MUL) return refuse(B200_E_ARG);
  if (count < 0) return refuse(B200_E_SHAPE);
  if (count == 0) return finish(0);
  if (!x || !y) return refuse(B200_E_NULL);
  if (!aligned(x, dtype_size(dtype)) || !aligned(y, dtype_size(dtype))) return refuse(B200_E_ALIGN);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == B200_F32 ? run_eltwise_kind<float>(kind, x, y, count, param, s)
                           : run_eltwise_kind<__nv_bfloat16>(kind, x, y, count, param, s);
}
