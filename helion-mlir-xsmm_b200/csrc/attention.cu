// Softmax attention for sm_100a: out = softmax(scale * Q K^T) V per head, bf16 in
// and out, online over 128-key blocks (the kernel the reference's tests carry as a
// Helion body: tests/harness.py:263-300, tests/test_numerics.py:141-158).
//
// One CTA per (head, 128-query tile), 6 warps:
//   warps 0-3  softmax: thread r owns query row r (TMEM lane r). Per key block it
//              loads its 128 scores from TMEM, keeps a running maximum and sum,
//              writes P = exp2(score * scale * log2e - max) as bf16 into shared memory
//              in the tensor core's K-major swizzled layout, and rescales the output
//              accumulator only when some row's maximum grew by more than 2^8 (the
//              reference body's _RESCALE_THRESHOLD idea: a stale maximum only scales
//              numerator and denominator alike). At the end: O / sum -> bf16 -> global.
//   warp 4     TMA producer: Q once, then K and V blocks through two stages each.
//   warp 5     MMA issuer (one lane): S_j = Q K_j^T into one of two TMEM score
//              buffers, issued one block ahead so that it runs under the softmax of
//              block j-1; then O += P_j V_j.
// TMEM: columns [0,128) and [128,256) scores, [256, 256+D) output accumulator.
//
// Keys past the end of the sequence arrive as zeros from TMA and are masked to
// -inf before the maximum; query rows past the end are computed and not stored.
// Every wait is bounded (status word + CTA-wide abort, as in the GEMM).
#include <cuda.h>

#include <mutex>

#include "umma_ptx.cuh"

namespace b200 {
namespace {

constexpr int kRows = 128;      // queries per CTA
constexpr int kKeys = 128;      // keys per block
constexpr int kStages = 2;      // K and V stages
constexpr int kSoftmaxWarps = 4;
constexpr int kAttnProducerWarp = 4, kAttnMmaWarp = 5;
constexpr int kAttnThreads = 32 * 6;
constexpr uint32_t kScoreCols = 128, kOutCol = 256;
constexpr float kRescaleLog2 = 8.0f;
constexpr int kErrAttnProducer = 32, kErrAttnMma = 64, kErrAttnSoftmax = 128;

struct AttnParams {
  int32_t heads, seq_q, seq_k, dim;
  int32_t tiles_q, key_blocks;
  float scale_log2;  // scale * log2(e)
  __nv_bfloat16* out;
  uint32_t idesc_qk, idesc_pv;
  int32_t* status;
};

struct __align__(8) AttnBarriers {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages];
  uint64_t v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, pv_done;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  constexpr int kChunks = D / 64;                       // 64-element column chunks of a D-wide tile
  constexpr uint32_t kTileBytes = kChunks * 16384;      // 128 rows x D bf16
  constexpr uint32_t kVHalfBytes = kChunks * 8192;      // 64 keys x D bf16 (MN-major chunks of 8 KiB)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + kTileBytes;
  const uint32_t v_smem = k_smem + kStages * kTileBytes;
  const uint32_t p_smem = v_smem + kStages * kTileBytes;  // 2 chunks x 16 KiB
  AttnBarriers* bars = reinterpret_cast<AttnBarriers*>(smem_raw + (p_smem + 32768u - smem_u32(smem_raw)));
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x / p.tiles_q, tile = blockIdx.x - head * p.tiles_q;
  const int q0 = tile * kRows;
  const int nb = p.key_blocks;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars->k_full[s]), 1);
      mbar_init(smem_u32(&bars->k_empty[s]), 1);
      mbar_init(smem_u32(&bars->v_full[s]), 1);
      mbar_init(smem_u32(&bars->v_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bars->s_full[s]), 1);
      mbar_init(smem_u32(&bars->s_empty[s]), kSoftmaxWarps);
    }
    mbar_init(smem_u32(&bars->p_full), kSoftmaxWarps);
    mbar_init(smem_u32(&bars->pv_done), 1);
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == kAttnMmaWarp) {
    tmem_alloc<1>(smem_u32(&bars->tmem_base), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == kAttnProducerWarp) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const uint32_t qf = smem_u32(&bars->q_full);
      mbar_expect_tx(qf, kTileBytes);
      for (int c = 0; c < kChunks; ++c) tma_load_3d(q_smem + c * 16384, &map_q, qf, 64 * c, q0, head);
      bool ok = true;
      uint32_t stage = 0, parity = 1;  // a fresh barrier's preceding phase counts as complete
      int issued = 0;
      for (int j = 0; j < nb && ok; ++j) {
        const int key0 = j * kKeys;
        ok = mbar_wait(smem_u32(&bars->k_empty[stage]), parity, abort_flag, p.status, kErrAttnProducer);
        if (!ok) break;
        const uint32_t kf = smem_u32(&bars->k_full[stage]);
        mbar_expect_tx(kf, kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(k_smem + stage * kTileBytes + c * 16384, &map_k, kf, 64 * c, key0, head);
        ok = mbar_wait(smem_u32(&bars->v_empty[stage]), parity, abort_flag, p.status, kErrAttnProducer);
        if (!ok) {
          // K of this stage is in flight: wait for it below
          ++issued;
          break;
        }
        const uint32_t vf = smem_u32(&bars->v_full[stage]);
        mbar_expect_tx(vf, kTileBytes);
        for (int h = 0; h < 2; ++h)
          for (int c = 0; c < kChunks; ++c)
            tma_load_3d(v_smem + stage * kTileBytes + h * kVHalfBytes + c * 8192, &map_v, vf, 64 * c, key0 + 64 * h,
                        head);
        ++issued;
        if (++stage == kStages) {
          stage = 0;
          parity ^= 1u;
        }
      }
      if (*abort_flag) {
        // Loads this CTA armed may still be in flight: give them (bounded) time to land
        // before the shared memory is given up. On the regular path every block was consumed.
        const unsigned long long start = global_ns();
        while (global_ns() - start < 2000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == kAttnMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t hi = desc_hi(1024);
      bool ok = mbar_wait(smem_u32(&bars->q_full), 0, abort_flag, p.status, kErrAttnMma);
      tc_fence_after();
      const uint64_t q_desc = make_desc(q_smem, 1u, hi);
      // S_j = Q K_j^T: both operands K-major, D/16 MMAs of K = 16 (4 per 64-wide chunk).
      auto issue_scores = [&](int j) -> bool {
        const uint32_t st = j % kStages, buf = j & 1;
        if (!mbar_wait(smem_u32(&bars->k_full[st]), (j / kStages) & 1, abort_flag, p.status, kErrAttnMma)) return false;
        if (!mbar_wait(smem_u32(&bars->s_empty[buf]), ((j >> 1) & 1) ^ 1, abort_flag, p.status, kErrAttnMma))
          return false;
        tc_fence_after();
        const uint64_t k_desc = make_desc(k_smem + st * kTileBytes, 1u, hi);
        uint32_t accumulate = 0;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint64_t step = static_cast<uint64_t>((c * 16384 + i * 32) >> 4);
            umma_bf16<1>(tmem_base + buf * kScoreCols, q_desc + step, k_desc + step, p.idesc_qk, accumulate);
            accumulate = 1;
          }
        }
        umma_commit<1>(smem_u32(&bars->k_empty[st]));
        umma_commit<1>(smem_u32(&bars->s_full[buf]));
        return true;
      };
      if (ok && nb > 0) ok = issue_scores(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) {
          ok = issue_scores(j + 1);
          if (!ok) break;
        }
        // O += P_j V_j: P K-major (two 64-key chunks), V MN-major (64-key halves of D/64 chunks).
        const uint32_t st = j % kStages;
        ok = mbar_wait(smem_u32(&bars->v_full[st]), (j / kStages) & 1, abort_flag, p.status, kErrAttnMma);
        if (ok) ok = mbar_wait(smem_u32(&bars->p_full), j & 1, abort_flag, p.status, kErrAttnMma);
        if (!ok) break;
        tc_fence_after();
        uint32_t accumulate = j > 0 ? 1u : 0u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint64_t p_desc = make_desc(p_smem + h * 16384, 1u, hi);
          const uint64_t v_desc = make_desc(v_smem + st * kTileBytes + h * kVHalfBytes, 8192u >> 4, hi);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            umma_bf16<1>(tmem_base + kOutCol, p_desc + static_cast<uint64_t>((i * 32) >> 4),
                         v_desc + static_cast<uint64_t>((i * 2048) >> 4), p.idesc_pv, accumulate);
            accumulate = 1;
          }
        }
        umma_commit<1>(smem_u32(&bars->v_empty[st]));
        umma_commit<1>(smem_u32(&bars->pv_done));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + output
    const int row = warp * 32 + lane;  // TMEM lane = query row of the tile
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float top = -1.0e30f, total = 0.f;
    bool ok = true;
    const uint32_t p_row = p_smem + row * 128;
    const uint32_t swz = static_cast<uint32_t>(row & 7);
    for (int j = 0; j < nb && ok; ++j) {
      const uint32_t buf = j & 1;
      ok = mbar_wait(smem_u32(&bars->s_full[buf]), (j >> 1) & 1, abort_flag, p.status, kErrAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      tc_fence_after();
      float s[kKeys];
#pragma unroll
      for (int c = 0; c < kKeys / 32; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + lane_addr + buf * kScoreCols + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(raw[i]) * p.scale_log2;
      }
      // The scores are in registers: the MMA warp may overwrite this buffer with S_{j+2}.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->s_empty[buf]));
      const int valid = p.seq_k - j * kKeys;  // keys of this block that exist
      if (valid < kKeys) {
#pragma unroll
        for (int i = 0; i < kKeys; ++i)
          if (i >= valid) s[i] = -INFINITY;
      }
      float block_top = s[0];
#pragma unroll
      for (int i = 1; i < kKeys; ++i) block_top = fmaxf(block_top, s[i]);
      const float new_top = fmaxf(top, block_top);
      bool waited_pv = false;
      if (j == 0) {
        top = new_top;
      } else if (__any_sync(0xffffffffu, new_top - top > kRescaleLog2)) {
        // Some row of this warp outgrew its maximum: rescale the warp's rows of O
        // (after the previous P V has landed there) and their sums.
        ok = mbar_wait(smem_u32(&bars->pv_done), (j - 1) & 1, abort_flag, p.status, kErrAttnSoftmax);
        ok = __all_sync(0xffffffffu, ok) != 0;
        if (!ok) break;
        waited_pv = true;
        tc_fence_after();
        const float alpha = fast_exp2(top - new_top);
        total *= alpha;
        top = new_top;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t raw[32];
          tmem_ld_32x32(tmem_base + lane_addr + kOutCol + c * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
          tmem_st_32x32(tmem_base + lane_addr + kOutCol + c * 32, raw);
        }
        tmem_st_wait();
      }
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < kKeys; ++i) {
        s[i] = fast_exp2(s[i] - top);
        sum += s[i];
      }
      total += sum;
      // P_{j-1} has been consumed (its P V completed) before P_j overwrites it.
      if (j > 0 && !waited_pv) {
        ok = mbar_wait(smem_u32(&bars->pv_done), (j - 1) & 1, abort_flag, p.status, kErrAttnSoftmax);
        ok = __all_sync(0xffffffffu, ok) != 0;
        if (!ok) break;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float* e = &s[h * 64 + u * 8];
          const uint32_t addr = p_row + h * 16384 + ((static_cast<uint32_t>(u) ^ swz) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack2(e[0], e[1])),
                       "r"(pack2(e[2], e[3])), "r"(pack2(e[4], e[5])), "r"(pack2(e[6], e[7]))
                       : "memory");
        }
      }
      fence_proxy_async();  // generic-proxy writes of P become visible to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->p_full));
    }
    if (ok && nb > 0) {
      ok = mbar_wait(smem_u32(&bars->pv_done), (nb - 1) & 1, abort_flag, p.status, kErrAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok) != 0;
    }
    if (ok) {
      tc_fence_after();
      const float inv = nb > 0 ? 1.f / total : 0.f;
      const int64_t q_row = static_cast<int64_t>(q0) + row;
      __nv_bfloat16* dst = p.out + (static_cast<int64_t>(head) * p.seq_q + q_row) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t raw[32];
        if (nb > 0) {
          tmem_ld_32x32(tmem_base + lane_addr + kOutCol + c * 32, raw);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = 0;
        }
        if (q_row < p.seq_q) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack2(__uint_as_float(raw[8 * i]) * inv, __uint_as_float(raw[8 * i + 1]) * inv);
            w.y = pack2(__uint_as_float(raw[8 * i + 2]) * inv, __uint_as_float(raw[8 * i + 3]) * inv);
            w.z = pack2(__uint_as_float(raw[8 * i + 4]) * inv, __uint_as_float(raw[8 * i + 5]) * inv);
            w.w = pack2(__uint_as_float(raw[8 * i + 6]) * inv, __uint_as_float(raw[8 * i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + 8 * i) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kAttnMmaWarp) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

uint32_t attn_idesc(int n, bool b_kmajor) {
  uint32_t d = 0;
  d |= 1u << 4;   // D format f32
  d |= 1u << 7;   // A format bf16
  d |= 1u << 10;  // B format bf16
  d |= (b_kmajor ? 0u : 1u) << 16;
  d |= static_cast<uint32_t>(n >> 3) << 17;
  d |= static_cast<uint32_t>(kRows >> 4) << 24;
  return d;
}

std::once_flag g_attn_attr_once[64];

template <int D>
size_t attn_smem_bytes() {
  return 1024 + static_cast<size_t>(1 + 2 * kStages) * (D / 64) * 16384 + 32768 + sizeof(AttnBarriers);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_attention(int32_t dtype, const void* q, const void* k, const void* v, void* out, int64_t heads,
                              int64_t seq_q, int64_t seq_k, int64_t dim, float scale, void* stream) {
  if (!enabled()) return refuse(B200_E_DISABLED);
  if (dtype != B200_BF16) return refuse(B200_E_DTYPE);
  if (heads < 0 || seq_q < 0 || seq_k < 0) return refuse(B200_E_SHAPE);
  if (dim != 64 && dim != 128) return refuse(B200_E_SHAPE);
  if (heads == 0 || seq_q == 0) return finish(0);
  if (!q || !out || (seq_k > 0 && (!k || !v))) return refuse(B200_E_NULL);
  if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(out, 16)) return refuse(B200_E_ALIGN);
  if (heads > 65535 || seq_q > INT32_MAX - 256 || seq_k > INT32_MAX - 256) return refuse(B200_E_SHAPE);
  const int64_t tiles_q = ceil_div(seq_q, kRows);
  if (heads * tiles_q > INT32_MAX) return refuse(B200_E_SHAPE);
  const DeviceInfo& dev = device_info();
  if (dev.sm_count == 0) return refuse(B200_E_DEVICE);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (seq_k == 0) {
    // softmax over no keys: the reference body leaves 0 / 0; rows of zeros are written here
    const cudaError_t err = cudaMemsetAsync(out, 0, static_cast<size_t>(heads * seq_q * dim) * 2, s);
    return finish(err == cudaSuccess ? 0 : -static_cast<int>(err));
  }
  CUtensorMap map_q, map_k, map_v;
  const bool ok = encode_map(&map_q, q, dim, seq_q, heads, dim, seq_q * dim, 64, kRows) &&
                  encode_map(&map_k, k, dim, seq_k, heads, dim, seq_k * dim, 64, kKeys) &&
                  encode_map(&map_v, v, dim, seq_k, heads, dim, seq_k * dim, 64, 64);
  if (!ok) return refuse(B200_E_DEVICE);

  AttnParams p{};
  p.heads = static_cast<int32_t>(heads);
  p.seq_q = static_cast<int32_t>(seq_q);
  p.seq_k = static_cast<int32_t>(seq_k);
  p.dim = static_cast<int32_t>(dim);
  p.tiles_q = static_cast<int32_t>(tiles_q);
  p.key_blocks = static_cast<int32_t>(ceil_div(seq_k, kKeys));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.idesc_qk = attn_idesc(kKeys, true);
  p.idesc_pv = attn_idesc(static_cast<int>(dim), false);
  p.status = kernel_status_word();

  std::call_once(g_attn_attr_once[dev.device], [] {
    cudaFuncSetAttribute(attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(attn_smem_bytes<64>()));
    cudaFuncSetAttribute(attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(attn_smem_bytes<128>()));
  });
  const unsigned grid = static_cast<unsigned>(heads * tiles_q);
  if (dim == 64)
    attention_kernel<64><<<grid, kAttnThreads, attn_smem_bytes<64>(), s>>>(map_q, map_k, map_v, p);
  else
    attention_kernel<128><<<grid, kAttnThreads, attn_smem_bytes<128>(), s>>>(map_q, map_k, map_v, p);
  return launched();
}
