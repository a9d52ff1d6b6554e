// Device memory that the GPUs of one box share: allocation, export to and mapping in
// the other ranks' processes (CUDA IPC). Used by the fused column-sharded linear, whose
// GEMM epilogue stores into every rank's copy of the result (b200_gemm_to_peers).
// Only stores and flag words ever cross to another GPU's memory; nothing is loaded by
// TMA or by a library kernel from it.
#include "common.cuh"

using namespace b200;

extern "C" int b200_symm_alloc(size_t bytes, void** out_ptr, void* out_handle) {
  if (!out_ptr || !out_handle) return refuse(B200_E_NULL);
  *out_ptr = nullptr;
  if (bytes == 0) return refuse(B200_E_SHAPE);
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err == cudaSuccess) err = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t handle;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&handle, p);
  if (err != cudaSuccess) {
    cudaGetLastError();
    if (p) cudaFree(p);
    return finish(-static_cast<int>(err));
  }
  static_assert(sizeof(handle) == B200_IPC_HANDLE_BYTES, "handle size");
  memcpy(out_handle, &handle, sizeof(handle));
  *out_ptr = p;
  return finish(0);
}

extern "C" int b200_symm_open(const void* handle_bytes, void** out_ptr) {
  if (!handle_bytes || !out_ptr) return refuse(B200_E_NULL);
  *out_ptr = nullptr;
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle_bytes, sizeof(handle));
  void* p = nullptr;
  const cudaError_t err = cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }
  *out_ptr = p;
  return finish(0);
}

extern "C" int b200_symm_close(void* ptr) {
  if (!ptr) return refuse(B200_E_NULL);
  const cudaError_t err = cudaIpcCloseMemHandle(ptr);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }
  return finish(0);
}

extern "C" int b200_symm_free(void* ptr) {
  if (!ptr) return refuse(B200_E_NULL);
  const cudaError_t err = cudaFree(ptr);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }
  return finish(0);
}
