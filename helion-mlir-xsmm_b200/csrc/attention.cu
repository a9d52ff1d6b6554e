// Softmax attention for sm_100a: out = softmax(scale * Q K^T) V per head, bf16 in
// and out, online over 128-key blocks (the kernel the reference's tests carry as a
// Helion body: tests/harness.py:263-300, tests/test_numerics.py:141-158).
//
// One CTA per (head, 128-query tile), 10 warps:
//   warps 0-3  softmax group 0: the even key blocks.  Thread r owns query row r
//   warps 4-7  softmax group 1: the odd key blocks.   (TMEM lane r) in both groups.
//              Per block a thread loads its 128 scores from the group's TMEM score
//              buffer, keeps the group's running maximum and sum of its row, writes
//              P = exp2(score * scale * log2e - max) as bf16 pairs back into tensor
//              memory over the scores it has just read (tcgen05.st; the second
//              product takes its A operand from there), and rescales
//              the group's output accumulator only when some row's maximum grew by
//              more than 2^8 (the reference body's _RESCALE_THRESHOLD idea: a stale
//              maximum only scales numerator and denominator alike). The two groups
//              are half a block out of phase, so one group's exponentials (MUFU)
//              run under the other's loads, maxima, conversions and stores, and the
//              tensor core always has the other group's products to do.
//              At the end the groups' (maximum, sum, accumulator) are merged:
//              out = (O0 w0 + O1 w1) / (sum0 w0 + sum1 w1), w = 2^(max - common max).
//   warp 8     TMA producers: lane 0 loads Q once and the K blocks, lane 1 the V blocks
//   warp 9     MMA issuer (one lane): O_{j%2} += P_j V_j when the group has written P_j
//              (A from tensor memory, B = V from shared memory), then S_{j+2} = Q K_{j+2}^T
//              into the same score buffer (in issue order after the P V that reads it).
// TMEM: columns [0,128) and [128,256) scores of the two groups, whose first 64 columns
// are reused for P (two bf16 per column); [256, 256+D) and [256+D, 256+2D) the two
// output accumulators. Shared memory holds only Q and the K / V stages.
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
constexpr int kMaxStages = 4;   // K and V stages: 2 at head size 128, 4 at 64
constexpr int kGroupWarps = 4;  // warps of one softmax group
constexpr int kAttnProducerWarp = 8, kAttnMmaWarp = 9;
constexpr int kAttnThreads = 32 * 10;
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
  uint64_t k_full[kMaxStages], k_empty[kMaxStages];
  uint64_t v_full[kMaxStages], v_empty[kMaxStages];
  uint64_t s_full[2];              // per score buffer = per group
  uint64_t p_full[2], pv_done[2];  // per group
  uint64_t merge[4];               // the two warps of a TMEM lane quarter meet here at the end
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
  constexpr int kStages = D == 64 ? 4 : 3;              // K and V stages beside Q in shared memory
  constexpr uint32_t kTileBytes = kChunks * 16384;      // 128 rows x D bf16
  constexpr uint32_t kVHalfBytes = kChunks * 8192;      // 64 keys x D bf16 (MN-major chunks of 8 KiB)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + kTileBytes;
  const uint32_t v_smem = k_smem + kStages * kTileBytes;
  const uint32_t end_smem = v_smem + kStages * kTileBytes;
  AttnBarriers* bars = reinterpret_cast<AttnBarriers*>(smem_raw + (end_smem - smem_u32(smem_raw)));
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x / p.tiles_q, tile = blockIdx.x - head * p.tiles_q;
  const int q0 = tile * kRows;
  const int nb = p.key_blocks;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&bars->k_full[s]), 1);
      mbar_init(smem_u32(&bars->k_empty[s]), 1);
      mbar_init(smem_u32(&bars->v_full[s]), 1);
      mbar_init(smem_u32(&bars->v_empty[s]), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&bars->s_full[g]), 1);
      mbar_init(smem_u32(&bars->p_full[g]), kGroupWarps);
      mbar_init(smem_u32(&bars->pv_done[g]), 1);
    }
    for (int s = 0; s < 4; ++s) mbar_init(smem_u32(&bars->merge[s]), 2);
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
    // ---------------------------------------------------------------- TMA producers
    // Lane 0 loads Q and the K blocks, lane 1 the V blocks, each in its own loop: a K
    // stage is free as soon as its scores are computed, a V stage only after its P V,
    // and neither load may queue behind the other's wait.
    if (lane == 0) {
      const uint32_t qf = smem_u32(&bars->q_full);
      mbar_expect_tx(qf, kTileBytes);
      for (int c = 0; c < kChunks; ++c) tma_load_3d(q_smem + c * 16384, &map_q, qf, 64 * c, q0, head);
      uint32_t stage = 0, parity = 1;  // a fresh barrier's preceding phase counts as complete
      for (int j = 0; j < nb; ++j) {
        if (!mbar_wait(smem_u32(&bars->k_empty[stage]), parity, abort_flag, p.status, kErrAttnProducer)) break;
        const uint32_t kf = smem_u32(&bars->k_full[stage]);
        mbar_expect_tx(kf, kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_3d(k_smem + stage * kTileBytes + c * 16384, &map_k, kf, 64 * c, j * kKeys, head);
        if (++stage == kStages) {
          stage = 0;
          parity ^= 1u;
        }
      }
    } else if (lane == 1) {
      uint32_t stage = 0, parity = 1;
      for (int j = 0; j < nb; ++j) {
        if (!mbar_wait(smem_u32(&bars->v_empty[stage]), parity, abort_flag, p.status, kErrAttnProducer)) break;
        const uint32_t vf = smem_u32(&bars->v_full[stage]);
        mbar_expect_tx(vf, kTileBytes);
        for (int h = 0; h < 2; ++h)
          for (int c = 0; c < kChunks; ++c)
            tma_load_3d(v_smem + stage * kTileBytes + h * kVHalfBytes + c * 8192, &map_v, vf, 64 * c,
                        j * kKeys + 64 * h, head);
        if (++stage == kStages) {
          stage = 0;
          parity ^= 1u;
        }
      }
    }
    if (lane < 2 && *abort_flag) {
      // Loads this CTA armed may still be in flight: give them (bounded) time to land
      // before the shared memory is given up. On the regular path every block was consumed.
      const unsigned long long start = global_ns();
      while (global_ns() - start < 2000000ull) {
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
      // Barriers that are normally complete long before they are needed (the K and V
      // stages) are tested alongside the MMAs issued before them, so that no barrier
      // round trip sits between two groups of MMAs; `k_landed` / `v_landed` carry the result.
      bool k_landed = false, v_landed = false;
      // S_j = Q K_j^T into score buffer j % 2: both operands K-major, D/16 MMAs of K = 16.
      // `peek_v`: the block whose V stage is tested on the way (its P V comes next).
      auto issue_scores = [&](int j, int peek_v) -> bool {
        const uint32_t st = j % kStages, g = j & 1;
        if (!k_landed &&
            !mbar_wait(smem_u32(&bars->k_full[st]), (j / kStages) & 1, abort_flag, p.status, kErrAttnMma))
          return false;
        k_landed = false;
        tc_fence_after();
        const uint64_t k_desc = make_desc(k_smem + st * kTileBytes, 1u, hi);
        const uint32_t d_tmem = tmem_base + g * kScoreCols;
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
          const uint64_t step = static_cast<uint64_t>((c * 16384) >> 4);
          if (c + 1 < kChunks || peek_v < 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              umma_bf16<1>(d_tmem, q_desc + step + static_cast<uint64_t>((i * 32) >> 4),
                           k_desc + step + static_cast<uint64_t>((i * 32) >> 4), p.idesc_qk, (c | i) ? 1u : 0u);
          } else {
            v_landed = umma_bf16_x4_peek<1>(d_tmem, q_desc + step, k_desc + step, 32 >> 4, 32 >> 4, p.idesc_qk,
                                            c ? 1u : 0u, smem_u32(&bars->v_full[peek_v % kStages]),
                                            (peek_v / kStages) & 1) != 0;
          }
        }
        umma_commit<1>(smem_u32(&bars->k_empty[st]));
        umma_commit<1>(smem_u32(&bars->s_full[g]));
        return true;
      };
      if (ok && nb > 0) ok = issue_scores(0, nb > 1 ? -1 : 0);
      if (ok && nb > 1) ok = issue_scores(1, 0);
      for (int j = 0; j < nb && ok; ++j) {
        // O_g += P_j V_j: P from tensor memory (8 columns = 16 keys per MMA), V MN-major
        // in shared memory (64-key halves of D/64 chunks).
        const uint32_t st = j % kStages, g = j & 1;
        if (!v_landed) ok = mbar_wait(smem_u32(&bars->v_full[st]), (j / kStages) & 1, abort_flag, p.status, kErrAttnMma);
        v_landed = false;
        if (ok) ok = mbar_wait(smem_u32(&bars->p_full[g]), (j >> 1) & 1, abort_flag, p.status, kErrAttnMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + kOutCol + g * D, p_tmem = tmem_base + g * kScoreCols;
        const uint64_t v_lo = make_desc(v_smem + st * kTileBytes, 8192u >> 4, hi);
        const uint64_t v_hi = make_desc(v_smem + st * kTileBytes + kVHalfBytes, 8192u >> 4, hi);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          umma_bf16_ts(d_tmem, p_tmem + i * 8, v_lo + static_cast<uint64_t>((i * 2048) >> 4), p.idesc_pv,
                       (j > 1 || i > 0) ? 1u : 0u);
        if (j + 2 < nb) {
          // the second half carries the test of the K stage the next scores need
          const int jn = j + 2;
          k_landed = umma_bf16_ts_x4_peek(d_tmem, p_tmem + 32, v_hi, 2048 >> 4, p.idesc_pv, 1u,
                                          smem_u32(&bars->k_full[jn % kStages]), (jn / kStages) & 1) != 0;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            umma_bf16_ts(d_tmem, p_tmem + 32 + i * 8, v_hi + static_cast<uint64_t>((i * 2048) >> 4), p.idesc_pv, 1u);
        }
        umma_commit<1>(smem_u32(&bars->v_empty[st]));
        umma_commit<1>(smem_u32(&bars->pv_done[g]));
        // The next scores of this group go where P_j lies: issued after the P V that reads
        // it, and the tensor core runs what one thread issues in order. On the way they
        // test the V stage of block j + 1, whose P V is next.
        if (j + 2 < nb) ok = issue_scores(j + 2, j + 1);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + output
    const int quarter = warp & 3, g = warp >> 2;
    const int row = quarter * 32 + lane;  // TMEM lane = query row of the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t score_addr = tmem_base + lane_addr + g * kScoreCols;
    const uint32_t out_addr = tmem_base + lane_addr + kOutCol + g * D;
    float top = -1.0e30f, total = 0.f;
    const bool negative = p.scale_log2 < 0.f;  // then the largest scaled score is the smallest raw one
    bool ok = true;
    const uint32_t s_full = smem_u32(&bars->s_full[g]);
    const uint32_t p_full = smem_u32(&bars->p_full[g]), pv_done = smem_u32(&bars->pv_done[g]);
    int mine = 0;  // blocks this group has taken
    for (int j = g; j < nb && ok; j += 2, ++mine) {
      ok = mbar_wait(s_full, mine & 1, abort_flag, p.status, kErrAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      tc_fence_after();
      // All 128 scores of this row (unscaled), one wait for the four loads.
      float s[kKeys];
      {
        uint32_t(&raw)[kKeys] = reinterpret_cast<uint32_t(&)[kKeys]>(s);
#pragma unroll
        for (int c = 0; c < kKeys / 32; ++c)
          tmem_ld_32x32(score_addr + c * 32, reinterpret_cast<uint32_t(&)[32]>(raw[c * 32]));
        tmem_ld_wait();
      }
      const int valid = p.seq_k - j * kKeys;  // keys of this block that exist
      if (valid < kKeys) {
        const float masked = negative ? INFINITY : -INFINITY;  // times the scale: -inf
#pragma unroll
        for (int i = 0; i < kKeys; ++i)
          if (i >= valid) s[i] = masked;
      }
      // Row maximum of scale * s in eight independent chains.
      float part[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) part[i] = s[i];
      if (!negative) {
#pragma unroll
        for (int i = 8; i < kKeys; ++i) part[i & 7] = fmaxf(part[i & 7], s[i]);
#pragma unroll
        for (int i = 4; i > 0; i >>= 1)
          for (int t = 0; t < i; ++t) part[t] = fmaxf(part[t], part[t + i]);
      } else {
#pragma unroll
        for (int i = 8; i < kKeys; ++i) part[i & 7] = fminf(part[i & 7], s[i]);
#pragma unroll
        for (int i = 4; i > 0; i >>= 1)
          for (int t = 0; t < i; ++t) part[t] = fminf(part[t], part[t + i]);
      }
      const float new_top = fmaxf(top, part[0] * p.scale_log2);
      bool waited_pv = false;
      if (mine == 0) {
        top = new_top;
      } else if (__any_sync(0xffffffffu, new_top - top > kRescaleLog2)) {
        // Some row of this warp outgrew its maximum: rescale the warp's rows of the
        // group's accumulator (after the group's previous P V has landed there) and sums.
        ok = mbar_wait(pv_done, (mine - 1) & 1, abort_flag, p.status, kErrAttnSoftmax);
        ok = __all_sync(0xffffffffu, ok) != 0;
        if (!ok) break;
        waited_pv = true;
        tc_fence_after();
        const float alpha = fast_exp2(top - new_top);
        total *= alpha;
        top = new_top;
#pragma unroll 1
        for (int c = 0; c < D / 16; ++c) {  // 16 columns at a time: the scores hold most registers
          uint32_t raw[16];
          tmem_ld_32x16(out_addr + c * 16, raw);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * alpha);
          tmem_st_32x16(out_addr + c * 16, raw);
        }
        tmem_st_wait();
      }
      // p = 2^(scale * s - top): the multiply-add and the sums on pairs (packed f32x2:
      // one issue slot for two scores; the softmax is bound by instruction issue), one ex2
      // per score, sums in four chains of pairs.
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2), neg_top2 = pack_f32x2(-top, -top);
      uint64_t sums[4] = {0, 0, 0, 0};  // +0.f pairs
#pragma unroll
      for (int i = 0; i < kKeys; i += 2) {
        float x0, x1;
        unpack_f32x2(fma_f32x2(pack_f32x2(s[i], s[i + 1]), scale2, neg_top2), x0, x1);
        s[i] = fast_exp2(x0);
        s[i + 1] = fast_exp2(x1);
        sums[(i >> 1) & 3] = add_f32x2(sums[(i >> 1) & 3], pack_f32x2(s[i], s[i + 1]));
      }
      {
        float lo, hi;
        unpack_f32x2(add_f32x2(add_f32x2(sums[0], sums[1]), add_f32x2(sums[2], sums[3])), lo, hi);
        total += lo + hi;
      }
      // P as bf16 pairs over the first 64 score columns (this thread's lane): keys 2c, 2c+1 in column c.
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t packed[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) packed[c] = pack2(s[h * 64 + 2 * c], s[h * 64 + 2 * c + 1]);
        tmem_st_32x32(score_addr + h * 32, packed);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // The group's last P V has landed in its accumulator. (A group without blocks, which
    // only happens with a single key block, waits for the other group's instead.)
    if (ok) {
      const uint32_t last = mine > 0 ? pv_done : smem_u32(&bars->pv_done[g ^ 1]);
      ok = mbar_wait(last, mine > 0 ? (mine - 1) & 1 : 0, abort_flag, p.status, kErrAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok) != 0;
    }
    // Merge the two groups: each row's (maximum, sum) goes through shared memory, the
    // accumulators are read from TMEM by both warps of the lane quarter, each for its
    // half of the output columns. The statistics reuse the Q tile: whichever group gets
    // here, the tensor core has finished every product that was issued before its last
    // P V, and those include all that read Q.
    float2* stats = reinterpret_cast<float2*>(smem_raw + (q_smem - smem_u32(smem_raw)));
    if (ok) {
      stats[g * kRows + row] = make_float2(top, total);
      tc_fence_before();
      __syncwarp();
      const uint32_t merge = smem_u32(&bars->merge[quarter]);
      if (lane == 0) mbar_arrive(merge);
      ok = mbar_wait(merge, 0, abort_flag, p.status, kErrAttnSoftmax);
      ok = __all_sync(0xffffffffu, ok) != 0;
    }
    if (ok) {
      tc_fence_after();
      const float2 other = stats[(g ^ 1) * kRows + row];
      const int theirs = (nb - (g ^ 1) + 1) >> 1;  // blocks the other group took
      const float common = fmaxf(top, other.x);
      const float w_mine = mine > 0 ? fast_exp2(top - common) : 0.f;
      const float w_theirs = theirs > 0 ? fast_exp2(other.x - common) : 0.f;
      const float inv = 1.f / (total * w_mine + other.y * w_theirs);
      const float a = w_mine * inv, b = w_theirs * inv;
      const int64_t q_row = static_cast<int64_t>(q0) + row;
      __nv_bfloat16* dst = p.out + (static_cast<int64_t>(head) * p.seq_q + q_row) * D;
      const uint32_t theirs_addr = tmem_base + lane_addr + kOutCol + (g ^ 1) * D;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        const int col = g * (D / 2) + c * 32;
        float o[32];
        {
          uint32_t x[32];
          if (mine > 0) {
            tmem_ld_32x32(out_addr + col, x);
            tmem_ld_wait();
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = mine > 0 ? __uint_as_float(x[i]) * a : 0.f;
          if (theirs > 0) {
            tmem_ld_32x32(theirs_addr + col, x);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = fmaf(__uint_as_float(x[i]), b, o[i]);
          }
        }
        if (q_row < p.seq_q) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack2(o[8 * i], o[8 * i + 1]);
            w.y = pack2(o[8 * i + 2], o[8 * i + 3]);
            w.z = pack2(o[8 * i + 4], o[8 * i + 5]);
            w.w = pack2(o[8 * i + 6], o[8 * i + 7]);
            *reinterpret_cast<uint4*>(dst + col + 8 * i) = w;
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
  const size_t stages = D == 64 ? 4 : 3;
  return 1024 + (1 + 2 * stages) * (D / 64) * 16384 + sizeof(AttnBarriers);
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
  // Keys past the end are masked as -inf * scale, which needs a non-zero finite scale.
  if (!(scale != 0.f) || !(fabsf(scale) <= 3.0e38f)) return refuse(B200_E_ARG);
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
