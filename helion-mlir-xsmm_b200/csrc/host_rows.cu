// GEMM on host-resident rows: A and C live in (pinned) host memory, B and the
// epilogue vectors on the device. The rows are cut into chunks that move through
// a ring of device staging buffers on three streams:
//
//   copy-in stream   A rows host -> staging
//   caller's stream  b200_gemm on the staged chunk
//   copy-out stream  C rows staging -> host
//
// PCIe carries both directions at once, so a call costs about the larger of the
// two transfers; the GEMM hides behind them. The staging ring, the two copy
// streams and the events belong to the library (one set per device) and persist
// between calls, so back-to-back calls overlap too: the next call's copy-in does
// not wait for the previous call's copy-out, unless it reads host memory that an
// earlier call's copy-out writes (a chained call: the result of one is the input
// of the next). The copy-in stream is not ordered after other work of the caller's
// stream: host rows that such work produces asynchronously must be complete, or the
// caller must have synchronised, before the call is made.
#include <mutex>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kDepth = 4;           // chunks in flight
constexpr int kMaxLaneDevices = 64;
constexpr int64_t kChunkBytes = 16 << 20;  // default staged A bytes per chunk

struct Lanes {
  bool ready = false;
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t copied_in[kDepth], computed[kDepth], copied_out[kDepth];
  bool used[kDepth] = {};
  uint8_t* staging = nullptr;
  size_t staging_bytes = 0;
  size_t a_chunk = 0, c_chunk = 0;  // how the ring is carved at present
  uint64_t next = 0;  // chunks issued so far: slot = next % kDepth
  // Host ranges that copy-outs of earlier calls write, newest last; ranges that fall
  // out of the list are merged into `old_begin..old_end` (a superset: it can only
  // cost an overlap, never miss one). `last_out`: slot of the newest copy-out.
  static constexpr int kRanges = 8;
  uintptr_t out_begin[kRanges] = {}, out_end[kRanges] = {};
  int out_count = 0;
  uintptr_t old_begin = 0, old_end = 0;
  int last_out = -1;
};

bool reads_earlier_output(const Lanes& l, uintptr_t begin, uintptr_t end) {
  if (l.old_begin < end && begin < l.old_end) return true;
  for (int i = 0; i < l.out_count; ++i)
    if (l.out_begin[i] < end && begin < l.out_end[i]) return true;
  return false;
}

void remember_output(Lanes& l, uintptr_t begin, uintptr_t end) {
  if (l.out_count == Lanes::kRanges) {
    if (l.old_end == 0) {
      l.old_begin = l.out_begin[0];
      l.old_end = l.out_end[0];
    } else {
      if (l.out_begin[0] < l.old_begin) l.old_begin = l.out_begin[0];
      if (l.out_end[0] > l.old_end) l.old_end = l.out_end[0];
    }
    for (int i = 1; i < Lanes::kRanges; ++i) {
      l.out_begin[i - 1] = l.out_begin[i];
      l.out_end[i - 1] = l.out_end[i];
    }
    --l.out_count;
  }
  l.out_begin[l.out_count] = begin;
  l.out_end[l.out_count] = end;
  ++l.out_count;
}

Lanes g_lanes[kMaxLaneDevices];
std::mutex g_lanes_mutex;

cudaError_t make_lanes(Lanes& l) {
  cudaError_t err = cudaStreamCreateWithFlags(&l.copy_in, cudaStreamNonBlocking);
  if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&l.copy_out, cudaStreamNonBlocking);
  for (int i = 0; i < kDepth && err == cudaSuccess; ++i) {
    err = cudaEventCreateWithFlags(&l.copied_in[i], cudaEventDisableTiming);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&l.computed[i], cudaEventDisableTiming);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&l.copied_out[i], cudaEventDisableTiming);
  }
  l.ready = err == cudaSuccess;
  return err;
}

// Grows the staging ring. Everything that still uses the old one is waited for first.
cudaError_t reserve_staging(Lanes& l, size_t bytes, cudaStream_t stream) {
  if (bytes <= l.staging_bytes) return cudaSuccess;
  cudaError_t err = cudaStreamSynchronize(l.copy_in);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(l.copy_out);
  if (err != cudaSuccess) return err;
  if (l.staging) cudaFree(l.staging);
  l.staging = nullptr;
  l.staging_bytes = 0;
  l.a_chunk = l.c_chunk = 0;
  for (bool& u : l.used) u = false;
  void* p = nullptr;
  err = cudaMalloc(&p, bytes);
  if (err != cudaSuccess) return err;
  l.staging = static_cast<uint8_t*>(p);
  l.staging_bytes = bytes;
  return cudaSuccess;
}

int64_t default_chunk_rows(int64_t rows, int64_t row_bytes) {
  int64_t chunk = kChunkBytes / (row_bytes > 0 ? row_bytes : 1) / 256 * 256;
  if (chunk < 256) chunk = 256;
  return chunk < rows ? chunk : rows;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_gemm_host_rows(const b200_gemm_desc* desc, const void* a_host, void* c_host, int64_t chunk_rows,
                                   void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (!desc) return refuse(B200_E_NULL);
  const b200_gemm_desc& d = *desc;
  if (d.m < 0 || d.n < 0 || d.k < 0) return refuse(B200_E_SHAPE);
  if (d.m == 0 || d.n == 0) return finish(0);
  if (!a_host || !c_host) return refuse(B200_E_NULL);
  // Whole rows of A move as one block per chunk: A is row-major, one problem.
  if (d.a_layout != B200_LAYOUT_ROW || d.batch != 1) return refuse(B200_E_ARG);
  if (d.lda < d.k || d.ldc < d.n) return refuse(B200_E_STRIDE);
  if (!valid_dtype(d.dtype) || !valid_dtype(d.out_dtype)) return refuse(B200_E_DTYPE);
  const DeviceInfo& dev = device_info();
  if (dev.sm_count == 0 || dev.device < 0 || dev.device >= kMaxLaneDevices) return refuse(B200_E_DEVICE);
  cudaStream_t caller = static_cast<cudaStream_t>(stream);

  const int64_t a_row_bytes = d.lda * static_cast<int64_t>(dtype_size(d.dtype));
  const int64_t c_row_bytes = d.ldc * static_cast<int64_t>(dtype_size(d.out_dtype));
  int64_t chunk = chunk_rows > 0 ? chunk_rows : default_chunk_rows(d.m, a_row_bytes);
  if (chunk > d.m) chunk = d.m;
  const size_t a_chunk = static_cast<size_t>(round_up(chunk * a_row_bytes, 256));
  const size_t c_chunk = static_cast<size_t>(round_up(chunk * c_row_bytes, 256));

  std::lock_guard<std::mutex> lock(g_lanes_mutex);
  Lanes& l = g_lanes[dev.device];
  cudaError_t err = cudaSuccess;
  if (!l.ready) err = make_lanes(l);
  if (err == cudaSuccess) err = reserve_staging(l, kDepth * (a_chunk + c_chunk), caller);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }

  if (err == cudaSuccess && (l.a_chunk != a_chunk || l.c_chunk != c_chunk)) {
    // The ring is carved differently from the last call: new slots overlap old ones,
    // so both writers wait for every reader still in flight.
    for (int s = 0; s < kDepth && err == cudaSuccess; ++s) {
      if (!l.used[s]) continue;
      err = cudaStreamWaitEvent(l.copy_in, l.computed[s], 0);
      if (err == cudaSuccess) err = cudaStreamWaitEvent(l.copy_in, l.copied_out[s], 0);
      if (err == cudaSuccess) err = cudaStreamWaitEvent(caller, l.computed[s], 0);
      if (err == cudaSuccess) err = cudaStreamWaitEvent(caller, l.copied_out[s], 0);
      l.used[s] = false;
    }
    l.a_chunk = a_chunk;
    l.c_chunk = c_chunk;
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }

  // A chained call: these rows are (part of) what an earlier call's copy-out writes.
  // The copy-out stream runs in order, so its newest event covers all earlier ones.
  {
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a_host);
    const uintptr_t a1 = a0 + static_cast<uintptr_t>((d.m - 1) * a_row_bytes + d.k * static_cast<int64_t>(dtype_size(d.dtype)));
    if (l.last_out >= 0 && reads_earlier_output(l, a0, a1)) {
      err = cudaStreamWaitEvent(l.copy_in, l.copied_out[l.last_out], 0);
      if (err != cudaSuccess) {
        cudaGetLastError();
        return finish(-static_cast<int>(err));
      }
    }
  }

  int last_slots[kDepth];
  int issued = 0;
  int gemm_rc = 0;
  for (int64_t begin = 0; begin < d.m; begin += chunk, ++l.next, ++issued) {
    const int64_t rows = d.m - begin < chunk ? d.m - begin : chunk;
    const int slot = static_cast<int>(l.next % kDepth);
    uint8_t* a_dev = l.staging + static_cast<size_t>(slot) * (a_chunk + c_chunk);
    uint8_t* c_dev = a_dev + a_chunk;
    // The slot's previous chunk: its GEMM has read the A stage, its copy-out has read the C stage.
    if (l.used[slot]) {
      err = cudaStreamWaitEvent(l.copy_in, l.computed[slot], 0);
      if (err == cudaSuccess) err = cudaStreamWaitEvent(caller, l.copied_out[slot], 0);
      if (err != cudaSuccess) break;
    }
    err = cudaMemcpyAsync(a_dev, static_cast<const uint8_t*>(a_host) + begin * a_row_bytes,
                          static_cast<size_t>(rows * a_row_bytes), cudaMemcpyHostToDevice, l.copy_in);
    if (err == cudaSuccess) err = cudaEventRecord(l.copied_in[slot], l.copy_in);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(caller, l.copied_in[slot], 0);
    if (err != cudaSuccess) break;
    b200_gemm_desc part = d;
    part.m = rows;
    part.a = a_dev;
    part.c = c_dev;
    gemm_rc = b200_gemm(&part, stream);  // counts itself
    if (gemm_rc != 0) break;
    err = cudaEventRecord(l.computed[slot], caller);
    if (err == cudaSuccess) err = cudaStreamWaitEvent(l.copy_out, l.computed[slot], 0);
    if (err == cudaSuccess)
      err = cudaMemcpyAsync(static_cast<uint8_t*>(c_host) + begin * c_row_bytes, c_dev,
                            static_cast<size_t>(rows * c_row_bytes), cudaMemcpyDeviceToHost, l.copy_out);
    if (err == cudaSuccess) err = cudaEventRecord(l.copied_out[slot], l.copy_out);
    if (err != cudaSuccess) break;
    l.used[slot] = true;
    l.last_out = slot;
    last_slots[issued % kDepth] = slot;
  }
  if (issued > 0) {
    const uintptr_t c0 = reinterpret_cast<uintptr_t>(c_host);
    remember_output(l, c0, c0 + static_cast<uintptr_t>((d.m - 1) * c_row_bytes + d.n * static_cast<int64_t>(dtype_size(d.out_dtype))));
  }
  // The caller's stream sees the host result: it waits for the copy-outs still in flight.
  const int tail = issued < kDepth ? issued : kDepth;
  for (int i = 0; i < tail && err == cudaSuccess; ++i)
    err = cudaStreamWaitEvent(caller, l.copied_out[last_slots[i]], 0);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }
  return gemm_rc;
}

extern "C" int b200_host_rows_release(void) {
  std::lock_guard<std::mutex> lock(g_lanes_mutex);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxLaneDevices) {
    cudaGetLastError();
    return refuse(B200_E_DEVICE);
  }
  Lanes& l = g_lanes[dev];
  if (!l.ready) return 0;
  cudaStreamSynchronize(l.copy_in);
  cudaStreamSynchronize(l.copy_out);
  if (l.staging) cudaFree(l.staging);
  l.staging = nullptr;
  l.staging_bytes = 0;
  for (bool& u : l.used) u = false;
  // both copy streams are idle: no copy-out of an earlier call is in flight any more
  l.out_count = 0;
  l.old_begin = l.old_end = 0;
  l.last_out = -1;
  cudaGetLastError();
  return 0;
}
