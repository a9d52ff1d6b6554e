// bf16 tensor-core GEMM for sm_100a: tcgen05.mma with the accumulator in tensor
// memory, operands staged in shared memory by TMA, fused epilogue.
//
// One persistent CTA per SM, 10 warps:
//   warps 0-7  epilogue: tcgen05.ld the 128 x BLOCK_N f32 accumulator (warp w owns
//              TMEM lanes 32(w%4)..+31 = tile rows and column half w/4), + bias,
//              * scale, + shift, activation, one rounding, stores to C. Two warps
//              per scheduler: one warp alone cannot hide its own latencies.
//   warp 8     TMA producer: cp.async.bulk.tensor loads of the A and B stage
//              (no cluster multicast: every CTA fetches its own tiles; reuse comes from L2)
//   warp 9     MMA issuer: owns the TMEM allocation; one lane issues
//              tcgen05.mma.cta_group::1.kind::f16 (M=128, N=BLOCK_N, K=16) and
//              commits stage-empty / accumulator-full mbarriers
// The accumulator is double buffered (2 x 256 TMEM columns), so the epilogue of
// one tile overlaps the main loop of the next.
//
// Shared-memory operand tiles use the 128-byte swizzle shared by TMA and the
// UMMA matrix descriptors. Per stage (64 K-elements):
//   K-major operand  (K contiguous in memory): rows x 128 B, 8-row groups 1024 B apart
//   MN-major operand (M or N contiguous): 64-element column chunks of 64 k-rows x 128 B
//                    (8 KiB each), chunk j at j*8 KiB
//
// Every wait is bounded: a wait that runs out ORs a code into the device status
// word, raises a CTA-wide abort flag, and all roles fall through to the common
// teardown (TMEM is released, in-flight TMA stages are drained).
#include <cuda.h>

#include <cstdio>
#include <mutex>

#include "gemm_common.cuh"
#include "umma_ptx.cuh"

namespace b200 {
namespace {

constexpr int kBlockM = 128;
constexpr int kStageK = 64;  // bf16 elements per stage = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kEpilogueWarps = 8;  // warp w: TMEM lane quarter w % 4, column half w / 4
constexpr int kProducerWarp = kEpilogueWarps;
constexpr int kMmaWarp = kEpilogueWarps + 1;
constexpr int kThreads = 32 * (kEpilogueWarps + 2);
constexpr int kMaxStages = 8;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccStride = 256;  // TMEM columns between the two accumulators

// Status bits (also reported through b200_read_kernel_status).
constexpr int kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 4, kErrDrainWait = 8, kErrSelfTest = 16,
              kErrPeerWait = 32;

struct UmmaParams {
  int32_t m, n, k, batch;
  int32_t tiles_m, tiles_n;
  int32_t group_m;        // tile rows per raster group (see tile_of)
  int32_t splits;         // serial K splits per output tile
  int32_t psplits;        // parallel K splits: each is a work item writing its own f32 partial
  int64_t psplit_stride;  // elements of C between the partials of consecutive parallel splits
  int32_t k_blocks;       // 64-wide K blocks per split
  int32_t block_n;
  int32_t stages;
  int32_t a_kmajor, b_kmajor;
  int32_t a_chunked, b_chunked;  // an M- / N-contiguous operand whose 64-column chunks arrive in one 4-D copy
  uint32_t idesc;
  uint32_t a_stage_bytes, b_stage_bytes;
  // matrix descriptor constants: high word and leading-byte-offset field
  uint32_t a_desc_hi, b_desc_hi, a_desc_lbo, b_desc_lbo;
  uint32_t a_kstep, b_kstep;  // descriptor start-address advance (16-byte units) per UMMA K step
  uint32_t a_khalf;           // ... from the first to the third K step of a stage (see umma_bf16_x4_peek)
  GemmEpilogue epi;
  void* c;
  int64_t ldc, stride_c;
  int32_t out_bf16;
  int32_t vec_store;   // rows of C are 16-byte aligned
  int32_t vec_params;  // bias / scale / shift start on 16-byte boundaries
  int32_t* status;
  PeerOut peer;  // PEERS instantiation only: the copies of C on this and the other GPUs
  int32_t peer_staged;  // PEERS: results go through shared memory and leave as whole 128-byte lines
};

struct __align__(8) PipelineBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// Output tile of a work item. Consecutive work items (= the tiles the CTAs of one
// wave run together) walk groups of `group_m` tile rows, M fastest inside a group,
// so that a wave covers a block of the output that shares group_m row panels of A
// and wave / group_m column panels of B in L2 (group_m = 1: N fastest, a wave
// shares a couple of row panels and streams B).
struct Tile {
  int32_t batch, m0, n0, ksplit;
};
__device__ __forceinline__ Tile tile_of(const UmmaParams& p, int64_t work, int rows_per_tile, int row_offset) {
  Tile t;
  t.ksplit = static_cast<int32_t>(work % p.psplits);
  work /= p.psplits;
  const int64_t per_batch = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  t.batch = static_cast<int32_t>(work / per_batch);
  const int64_t r = work - t.batch * per_batch;
  const int64_t group_tiles = static_cast<int64_t>(p.group_m) * p.tiles_n;
  const int64_t group = r / group_tiles, in_group = r - group * group_tiles;
  const int32_t first_row = static_cast<int32_t>(group) * p.group_m;
  const int32_t rows = min(p.group_m, p.tiles_m - first_row);
  const int32_t tile_n = static_cast<int32_t>(in_group / rows);
  t.m0 = (first_row + static_cast<int32_t>(in_group - static_cast<int64_t>(tile_n) * rows)) * rows_per_tile + row_offset;
  t.n0 = tile_n * p.block_n;
  return t;
}

// 32 consecutive entries of a bias / scale / shift vector as floats. `fast`: the
// entries exist (col0 + 32 <= n) and start on a 16-byte boundary, so every lane
// issues the same few vector loads (a broadcast from L1) instead of 32 scalar ones.
__device__ __forceinline__ void load_vec32(const void* p, int64_t col0, int64_t n, bool bf16, bool scalar, bool fast,
                                           float (&out)[32]) {
  if (scalar) {
    const float value = load_vec(p, 0, bf16);
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = value;
  } else if (fast) {
    if (bf16) {
      const uint4* q = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + col0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 w = __ldg(q + j);
        out[8 * j] = __uint_as_float(w.x << 16);
        out[8 * j + 1] = __uint_as_float(w.x & 0xffff0000u);
        out[8 * j + 2] = __uint_as_float(w.y << 16);
        out[8 * j + 3] = __uint_as_float(w.y & 0xffff0000u);
        out[8 * j + 4] = __uint_as_float(w.z << 16);
        out[8 * j + 5] = __uint_as_float(w.z & 0xffff0000u);
        out[8 * j + 6] = __uint_as_float(w.w << 16);
        out[8 * j + 7] = __uint_as_float(w.w & 0xffff0000u);
      }
    } else {
      const float4* q = reinterpret_cast<const float4*>(static_cast<const float*>(p) + col0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 w = __ldg(q + j);
        out[4 * j] = w.x;
        out[4 * j + 1] = w.y;
        out[4 * j + 2] = w.z;
        out[4 * j + 3] = w.w;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = load_vec(p, (col0 + j < n) ? col0 + j : n - 1, bf16);
  }
}

__device__ __forceinline__ void activate32(int act, float alpha, float (&v)[32]) {
  switch (act) {
    case B200_ACT_IDENTITY:
      break;
    case B200_ACT_RELU:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(B200_ACT_RELU, v[j], alpha);
      break;
    case B200_ACT_GELU_ERF:
#pragma unroll
      for (int j = 0; j < 32; j += 2) gelu_erf_pair(v[j], v[j + 1]);
      break;
    case B200_ACT_GELU_TANH:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(B200_ACT_GELU_TANH, v[j], alpha);
      break;
    case B200_ACT_SIGMOID:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(B200_ACT_SIGMOID, v[j], alpha);
      break;
    case B200_ACT_TANH:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(B200_ACT_TANH, v[j], alpha);
      break;
    case B200_ACT_SILU:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(B200_ACT_SILU, v[j], alpha);
      break;
    default:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(B200_ACT_LEAKY_RELU, v[j], alpha);
  }
}

// One rounding and the store of 32 consecutive columns (col0..) of one row of C
// (16-byte stores when the rows allow).
__device__ __forceinline__ void store32(const UmmaParams& p, uint8_t* c_row, int64_t col0, bool full_chunk,
                                        const float (&v)[32]) {
  if (p.out_bf16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(c_row) + col0;
    if (full_chunk && p.vec_store) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 q;
        q.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
        q.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
        q.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
        q.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
        *reinterpret_cast<uint4*>(dst + 8 * j) = q;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.n) dst[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* dst = reinterpret_cast<float*>(c_row) + col0;
    if (full_chunk && p.vec_store) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.n) dst[j] = v[j];
    }
  }
}

template <int CG, bool PEERS = false, bool A_BLOCKED = false>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_umma_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          const UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t stage_bytes = p.a_stage_bytes + p.b_stage_bytes;
  PipelineBarriers* bars = reinterpret_cast<PipelineBarriers*>(smem_aligned + static_cast<size_t>(p.stages) * stage_bytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total_work = static_cast<int64_t>(p.batch) * p.tiles_m * p.tiles_n * p.psplits;
  // A CTA pair (CG == 2) shares one 256-row tile: CTA `rank` owns rows 128*rank.. of it
  // and stages half of the B tile; the even CTA (leader) issues the MMAs for both.
  const int rank = CG == 2 ? static_cast<int>(cluster_cta_rank()) : 0;
  const bool leader = rank == 0;
  const int64_t first_work = blockIdx.x / CG, work_stride = gridDim.x / CG;
  constexpr int kTileRows = kBlockM * CG;
  const bool serial = p.splits > 1;
  const int b_rows = p.block_n / CG;  // columns of the B tile this CTA stages

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->acc_full[a]), 1);
      mbar_init(smem_u32(&bars->acc_empty[a]), kEpilogueWarps * CG);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == kProducerWarp && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == kMmaWarp) {
    tmem_alloc<CG>(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  if (CG == 2)
    cluster_sync_all();  // the peer's barriers are initialised before anything is signalled on them
  else
    __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    // One lane runs the whole loop (the other lanes wait at the __syncwarp below):
    // no per-stage votes, and stage / parity advance by increments, not divisions.
    if (lane == 0) {
      uint32_t stage = 0, parity = 1;  // a fresh barrier's preceding phase counts as complete
      uint32_t issued = 0;
      bool ok = true;
      for (int64_t work = first_work; work < total_work && ok; work += work_stride) {
        const Tile t = tile_of(p, work, kTileRows, rank * kBlockM);
        const int32_t nb = t.n0 + rank * b_rows;  // this CTA's share of the B tile
        for (int s = 0; s < p.splits && ok; ++s) {
          int32_t k0 = (t.ksplit * p.splits + s) * p.k_blocks * kStageK;
          for (int kb = 0; kb < p.k_blocks; ++kb, k0 += kStageK) {
            ok = mbar_wait(smem_u32(&bars->empty[stage]), parity, abort_flag, p.status, kErrProducerWait);
            if (!ok) break;
            const uint32_t full = smem_u32(&bars->full[stage]);
            const uint32_t a_dst = smem_base + stage * stage_bytes;
            const uint32_t b_dst = a_dst + p.a_stage_bytes;
            // The leader's barrier counts the bytes of both CTAs of a pair.
            if (leader) mbar_expect_tx(full, stage_bytes * CG);
            auto load = [&](uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1) {
              if (CG == 2)
                tma_load_3d_pair(dst, map, full, c0, c1, t.batch);
              else
                tma_load_3d(dst, map, full, c0, c1, t.batch);
            };
            if constexpr (A_BLOCKED) {
              // two K blocks of four row blocks each: 128 rows x 64 bytes, 8 KiB apart
              for (int j = 0; j < 2; ++j) {
                if (CG == 2)
                  tma_load_5d_pair(a_dst + j * 8192, &map_a, full, 0, 0, (k0 >> 5) + j, t.m0 >> 5, t.batch);
                else
                  tma_load_5d(a_dst + j * 8192, &map_a, full, 0, 0, (k0 >> 5) + j, t.m0 >> 5, t.batch);
              }
            } else if (p.a_kmajor) {
              load(a_dst, &map_a, k0, t.m0);
            } else if (p.a_chunked) {
              if (CG == 2)
                tma_load_4d_pair(a_dst, &map_a, full, 0, k0, t.m0 >> 6, t.batch);
              else
                tma_load_4d(a_dst, &map_a, full, 0, k0, t.m0 >> 6, t.batch);
            } else {
              for (int j = 0; j < kBlockM / 64; ++j) load(a_dst + j * 8192, &map_a, t.m0 + 64 * j, k0);
            }
            if (p.b_kmajor) {
              load(b_dst, &map_b, k0, nb);
            } else if (p.b_chunked) {
              if (CG == 2)
                tma_load_4d_pair(b_dst, &map_b, full, 0, k0, nb >> 6, t.batch);
              else
                tma_load_4d(b_dst, &map_b, full, 0, k0, nb >> 6, t.batch);
            } else {
              for (int j = 0; j < b_rows / 64; ++j) load(b_dst + j * 8192, &map_b, nb + 64 * j, k0);
            }
            ++issued;
            if (++stage == static_cast<uint32_t>(p.stages)) {
              stage = 0;
              parity ^= 1u;
            }
          }
        }
      }
      // Drain: no stage this CTA armed may still be in flight when its shared memory is
      // given up. (A pair's peer has no barrier of its own to ask: its last loads have
      // landed once the leader's MMAs that read them completed, which its epilogue waits for.)
      if (leader) {
        const uint32_t pending = issued < static_cast<uint32_t>(p.stages) ? issued : p.stages;
        // walk back `pending` stages from the next one to be armed
        uint32_t st = stage, par = parity ^ 1u;  // parity the consumer waits for in the current round
        for (uint32_t j = 0; j < pending; ++j) {
          if (st == 0) {
            st = p.stages;
            par ^= 1u;
          }
          --st;
          int never = 0;
          if (!mbar_wait(smem_u32(&bars->full[st]), par, &never, p.status, kErrDrainWait)) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer (the leader's, for a pair)
    // The tensor core takes a new MMA only as the previous ones drain, so every cycle
    // this thread spends between two MMAs is a cycle the tensor core idles: one lane,
    // no votes, no divisions, descriptors advanced by increments.
    if (lane == 0 && leader) {
      uint32_t stage = 0, parity = 0;
      uint32_t phase = 0;
      bool landed = false;
      const uint32_t stage_step = stage_bytes >> 4;
      bool ok = true;
      for (int64_t work = first_work; work < total_work && ok; work += work_stride) {
        for (int s = 0; s < p.splits && ok; ++s, ++phase) {
          // Without splits the two TMEM halves double-buffer the accumulator; with serial
          // splits the accumulator is half 0 and half 1 holds the running sum of the splits.
          const uint32_t acc = serial ? 0u : (phase & 1u), acc_round = serial ? phase : (phase >> 1);
          ok = mbar_wait(smem_u32(&bars->acc_empty[acc]), (acc_round & 1u) ^ 1u, abort_flag, p.status, kErrMmaWait);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * kAccStride;
          uint32_t accumulate = 0;
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            // `landed`: the previous block's MMAs carried a test of this stage's barrier along
            // (umma_bf16_x4_peek), so the usual case costs no barrier round trip here.
            if (!landed) {
              ok = mbar_wait(smem_u32(&bars->full[stage]), parity, abort_flag, p.status, kErrMmaWait);
              if (!ok) break;
            }
            tc_fence_after();
            const uint64_t a_desc =
                make_desc(smem_base, p.a_desc_lbo, p.a_desc_hi) + static_cast<uint64_t>(stage * stage_step);
            const uint64_t b_desc = make_desc(smem_base + p.a_stage_bytes, p.b_desc_lbo, p.b_desc_hi) +
                                    static_cast<uint64_t>(stage * stage_step);
            const uint32_t this_stage = stage;
            if (++stage == static_cast<uint32_t>(p.stages)) {
              stage = 0;
              parity ^= 1u;
            }
            // (after the last block of the last tile the tested barrier is simply never armed again)
            if constexpr (A_BLOCKED)
              landed = umma_bf16_x4_peek<CG, true>(d_tmem, a_desc, b_desc, p.a_kstep, p.b_kstep, p.idesc, accumulate,
                                                   smem_u32(&bars->full[stage]), parity, p.a_khalf) != 0;
            else
              landed = umma_bf16_x4_peek<CG>(d_tmem, a_desc, b_desc, p.a_kstep, p.b_kstep, p.idesc, accumulate,
                                             smem_u32(&bars->full[stage]), parity) != 0;
            accumulate = 1;
            umma_commit<CG>(smem_u32(&bars->empty[this_stage]));
          }
          if (ok) umma_commit<CG>(smem_u32(&bars->acc_full[acc]));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    uint32_t phase = 0;
    bool ok = true;
    const int quarter = warp & 3, half = warp >> 2;
    const int half_cols = p.block_n >> 1;  // BLOCK_N is a multiple of 64
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    for (int64_t work = first_work; work < total_work && ok; work += work_stride) {
      const Tile t = tile_of(p, work, kTileRows, rank * kBlockM);
      const int64_t row = static_cast<int64_t>(t.m0) + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      uint8_t* c_row = static_cast<uint8_t*>(p.c) +
                       (static_cast<int64_t>(t.ksplit) * p.psplit_stride + static_cast<int64_t>(t.batch) * p.stride_c +
                        row * p.ldc) *
                           (p.out_bf16 ? 2 : 4);
      for (int s = 0; s < p.splits && ok; ++s, ++phase) {
        const uint32_t acc = serial ? 0u : (phase & 1u), acc_round = serial ? phase : (phase >> 1);
        ok = mbar_wait(smem_u32(&bars->acc_full[acc]), acc_round & 1u, abort_flag, p.status, kErrEpilogueWait);
        ok = __all_sync(0xffffffffu, ok) != 0;
        if (!ok) break;
        tc_fence_after();
        const bool last = s == p.splits - 1;
        const int c_begin = half * half_cols, c_end = (half + 1) * half_cols;
        if constexpr (PEERS) {
          // Stores that cross NVLink should be whole 128-byte lines: a thread's own 16-byte
          // pieces of its row (the direct form below) travel as separate small writes (measured
          // on two GPUs: 33.5 MB to the peer in 180 us, a quarter of the link's rate). So the bf16
          // results of 64 columns go through a per-warp tile in shared memory (32 rows x 128
          // bytes, 16-byte pieces XOR-swizzled by row so that neither side conflicts) and leave
          // row-major: eight lanes write one row's 128 bytes, a warp four rows per instruction.
          if (p.peer_staged && static_cast<int64_t>(t.n0) + c_end <= p.n) {
            uint8_t* stage = smem_aligned + static_cast<size_t>(p.stages) * stage_bytes + 1024 + warp * 4096;
            const int64_t row0 = static_cast<int64_t>(t.m0) + quarter * 32;
            uint8_t* c_tile = static_cast<uint8_t*>(p.c) + row0 * p.ldc * 2;  // batch 1, no parallel splits
            for (int c0 = c_begin; c0 < c_end; c0 += 64) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                uint32_t raw[32];
                tmem_ld_32x32(tmem_base + lane_base + acc * kAccStride + c0 + 32 * h, raw);
                tmem_ld_wait();
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                const int64_t col0 = static_cast<int64_t>(t.n0) + c0 + 32 * h;
                const bool vec_fast = p.vec_params != 0;
                if (p.epi.bias) {
                  float w[32];
                  load_vec32(p.epi.bias, col0, p.n, p.epi.vec_bf16, p.epi.bias_scalar, vec_fast, w);
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += w[j];
                }
                if (p.epi.scale) {
                  float w[32];
                  load_vec32(p.epi.scale, col0, p.n, p.epi.vec_bf16, p.epi.scale_scalar, vec_fast, w);
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] *= w[j];
                }
                if (p.epi.shift) {
                  float w[32];
                  load_vec32(p.epi.shift, col0, p.n, p.epi.vec_bf16, p.epi.shift_scalar, vec_fast, w);
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += w[j];
                }
                activate32(p.epi.act, p.epi.alpha, v);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 q;
                  q.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
                  q.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
                  q.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
                  q.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
                  *reinterpret_cast<uint4*>(stage + lane * 128 + (((4 * h + j) ^ (lane & 7)) << 4)) = q;
                }
              }
              if (p.peer.store_maps) {
                // The tile is laid out as TMA's 128-byte swizzle wants it: one bulk tensor store
                // per copy of C moves the 32 x 64 box (rows past M are dropped), issued by one
                // lane, instead of 64 store instructions of the whole warp. The stores read shared
                // memory through the async proxy, hence the fence after the generic writes.
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  const CUtensorMap* maps = static_cast<const CUtensorMap*>(p.peer.store_maps);
                  for (int dest = 0; dest < p.peer.count; ++dest)
                    tma_store_2d(maps + dest, smem_u32(stage), t.n0 + c0, static_cast<int32_t>(row0));
                  tma_store_commit();
                  tma_store_wait_read();  // the tile may be overwritten by the next 64 columns
                }
                __syncwarp();
              } else {
                __syncwarp();
                const int piece = lane & 7;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const int r = 4 * i + (lane >> 3);
                  const uint4 q = *reinterpret_cast<const uint4*>(stage + r * 128 + ((piece ^ (r & 7)) << 4));
                  if (row0 + r < p.m) {
                    uint8_t* to = c_tile + static_cast<int64_t>(r) * p.ldc * 2 + (static_cast<int64_t>(t.n0) + c0) * 2 + piece * 16;
                    for (int dest = 0; dest < p.peer.count; ++dest) *reinterpret_cast<uint4*>(to + p.peer.delta[dest]) = q;
                  }
                }
                __syncwarp();
              }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (CG == 2)
                mbar_arrive_leader(smem_u32(&bars->acc_empty[acc]));
              else
                mbar_arrive(smem_u32(&bars->acc_empty[acc]));
            }
            continue;
          }
        }
        for (int c0 = c_begin; c0 < c_end; c0 += 32) {
          uint32_t raw[32];
          tmem_ld_32x32(tmem_base + lane_base + acc * kAccStride + c0, raw);
          float v[32];
          if (serial) {
            // Ordered split-K: the running sum of the splits lives in the other TMEM
            // half, so partial sums never leave the SM. s = 0 starts it, later splits
            // add to it in ascending order, the last one goes on to the epilogue.
            const uint32_t sum_addr = tmem_base + lane_base + kAccStride + c0;
            uint32_t prev[32];
            if (s > 0) tmem_ld_32x32(sum_addr, prev);
            tmem_ld_wait();
            // This warp's share of the accumulator is in registers once its last chunk
            // is loaded: the MMA warp may overwrite it with the next split.
            if (c0 + 32 >= c_end) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if (CG == 2)
                  mbar_arrive_leader(smem_u32(&bars->acc_empty[acc]));
                else
                  mbar_arrive(smem_u32(&bars->acc_empty[acc]));
              }
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]) + (s > 0 ? __uint_as_float(prev[j]) : 0.f);
            if (!last) {
#pragma unroll
              for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(v[j]);
              tmem_st_32x32(sum_addr, raw);
              tmem_st_wait();
              continue;
            }
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          }
          const int64_t col0 = static_cast<int64_t>(t.n0) + c0;
          if (!row_ok || col0 >= p.n) continue;
          const bool full_chunk = col0 + 32 <= p.n;
          if (last) {
            const bool vec_fast = full_chunk && p.vec_params;
            if (p.epi.bias) {
              float w[32];
              load_vec32(p.epi.bias, col0, p.n, p.epi.vec_bf16, p.epi.bias_scalar, vec_fast, w);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += w[j];
            }
            if (p.epi.scale) {
              float w[32];
              load_vec32(p.epi.scale, col0, p.n, p.epi.vec_bf16, p.epi.scale_scalar, vec_fast, w);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= w[j];
            }
            if (p.epi.shift) {
              float w[32];
              load_vec32(p.epi.shift, col0, p.n, p.epi.vec_bf16, p.epi.shift_scalar, vec_fast, w);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += w[j];
            }
            activate32(p.epi.act, p.epi.alpha, v);
          }
          if constexpr (PEERS) {
            // the same piece into every copy of C (this GPU's and its peers')
            for (int dest = 0; dest < p.peer.count; ++dest) store32(p, c_row + p.peer.delta[dest], col0, full_chunk, v);
          } else {
            store32(p, c_row, col0, full_chunk, v);
          }
        }
        // This warp has read the whole accumulator: hand it back to the MMA warp
        // (with serial splits that happened right after the last chunk was loaded).
        if (!serial) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CG == 2)
              mbar_arrive_leader(smem_u32(&bars->acc_empty[acc]));
            else
              mbar_arrive(smem_u32(&bars->acc_empty[acc]));
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  // Neither CTA of a pair may leave while the other can still read its shared
  // memory (MMA operands) or signal its barriers.
  if constexpr (PEERS) {
    if (warp < kEpilogueWarps) {
      if (p.peer.store_maps && lane == 0) tma_store_wait_all();  // this lane's bulk stores have completed
      __threadfence_system();  // this thread's stores, before the CTA reports
    }
  }
  tc_fence_before();
  if (CG == 2)
    cluster_sync_all();
  else
    __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
  }
  if constexpr (PEERS) {
    // The last CTA to get here has seen every other CTA's report, each made after that
    // CTA's stores were fenced: it resets the counter for the next launch and raises this
    // GPU's flag on every destination.
    if (threadIdx.x == 0) {
      __threadfence_system();
      const uint32_t earlier = atomicAdd(p.peer.done_counter, 1u);
      if (earlier + 1 == gridDim.x) {
        __threadfence_system();
        atomicExch(p.peer.done_counter, 0u);
        for (int dest = 0; dest < p.peer.count; ++dest)
          asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p.peer.flags[dest]), "r"(p.peer.epoch) : "memory");
      }
    }
  }
}

// Waits until every flag of `flags[0..count)` (set by the kernels above, one per GPU of
// the group) has reached `epoch`, or gives up after `budget_ns` and leaves kErrPeerWait in
// the status word. One thread per flag.
__global__ void peer_wait_kernel(const int32_t* flags, int count, int32_t epoch, unsigned long long budget_ns,
                                 int32_t* status) {
  if (static_cast<int>(threadIdx.x) >= count) return;
  const int32_t* flag = flags + threadIdx.x;
  const unsigned long long start = global_ns();
  for (uint32_t spin = 0;; ++spin) {
    int32_t seen;
    asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen - epoch >= 0) return;
    if ((spin & 63u) == 63u && global_ns() - start > budget_ns) {
      if (status) atomicOr(status, kErrPeerWait);
      return;
    }
  }
}

// Waits on a barrier nothing ever arrives on: the wait must run out after
// `budget_ns`, leave kErrSelfTest in the status word and return normally.
__global__ void wait_timeout_selftest_kernel(unsigned long long budget_ns, int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  mbar_wait(smem_u32(&bar), 0, &abort_flag, status, kErrSelfTest, budget_ns);
}

// --------------------------------------------------------------------------- host

uint32_t make_idesc(int block_n, bool a_kmajor, bool b_kmajor, int cta_group) {
  uint32_t d = 0;
  d |= 1u << 4;   // D format f32
  d |= 1u << 7;   // A format bf16
  d |= 1u << 10;  // B format bf16
  d |= (a_kmajor ? 0u : 1u) << 15;
  d |= (b_kmajor ? 0u : 1u) << 16;
  d |= static_cast<uint32_t>(block_n >> 3) << 17;
  d |= static_cast<uint32_t>((kBlockM * cta_group) >> 4) << 24;  // a CTA pair multiplies 256 rows
  return d;
}

std::once_flag g_attr_once[64];

}  // namespace

// Whether the tensor-core path can take `d` (plain ROW/COL layouts of bf16).
// The strides TMA needs: 16-byte aligned bases and row pitches.
int umma_supports(const b200_gemm_desc& d) {
  if (d.dtype != B200_BF16) return B200_E_DTYPE;
  const bool a_blocked = d.a_layout == B200_LAYOUT_BLOCKED;  // read in place through a 5-D tensor map
  if ((d.a_layout > B200_LAYOUT_COL && !a_blocked) || d.b_layout > B200_LAYOUT_COL) return B200_E_ARG;
  if (!aligned(d.a, 16) || !aligned(d.b, 16)) return B200_E_ALIGN;
  if ((!a_blocked && d.lda % 8) || d.ldb % 8 || (d.batch > 1 && (d.stride_a % 8 || d.stride_b % 8))) return B200_E_STRIDE;
  if (d.m > INT32_MAX - 256 || d.n > INT32_MAX - 256 || d.k > INT32_MAX - 256 || d.batch > 65535)
    return B200_E_SHAPE;
  if (d.k < 1) return B200_E_SHAPE;
  return 0;
}

// Tile rows per raster group. While B (n x k) sits in L2 with room to spare, N-fastest
// order (groups of one row) is best: a wave re-reads B from L2 and streams A once.
// A larger B is evicted between tile rows; groups of 16 rows make a wave reuse a few
// column panels of B instead (measured: 4096x16384x4096 1171 -> 1431 TFLOP/s,
// 8192^3 1316 -> 1383, 16384x8192x4096 1341 -> 1415; at 8192x4096x4096, where B is
// 33 MB, grouping costs 2 %).
int raster_group(const b200_gemm_desc& d, int tiles_m) {
  const double b_bytes = static_cast<double>(d.n) * static_cast<double>(d.k) * 2.0;
  int g = b_bytes > 64.0 * 1024 * 1024 ? 16 : 1;
  return g < tiles_m ? g : (tiles_m > 0 ? tiles_m : 1);
}

struct UmmaPlan {
  int cta_group;  // 1: one CTA per 128-row tile; 2: a CTA pair per 256-row tile
  int block_n;
  int stages;
  int splits;   // serial
  int psplits;  // parallel (workspace partials)
  int k_blocks;
  unsigned grid;
  size_t smem;
};

UmmaPlan umma_plan(const b200_gemm_desc& d, int sm_count, bool parallel_splits) {
  UmmaPlan plan;
  const bool b_kmajor = d.b_layout == B200_LAYOUT_COL;
  // BLOCK_N: a multiple of 64 (each half of the columns is read by its epilogue warps
  // 32 at a time; an N-contiguous B arrives in 64-column TMA chunks).
  const int gran = 64;
  int bn = 256;
  // tile_n > 0 is a hint (a Helion config's block_sizes): taken when it asks for at least 128
  // columns, the narrowest tile that keeps the tensor core reasonably busy; smaller hints
  // (written for a CPU's register tiles) leave the choice to the launcher. tile_n < 0 fixes
  // the width to -tile_n (tuning runs).
  const bool fixed_n = d.tile_n < 0 || d.tile_n >= 128;
  if (fixed_n) bn = static_cast<int>(round_up(d.tile_n < 0 ? -static_cast<int64_t>(d.tile_n) : d.tile_n, 64));
  if (bn > 256) bn = 256;
  // Narrow problems: no wider than N needs.
  const int64_t n_cap = round_up(d.n, gran);
  if (bn > n_cap) bn = static_cast<int>(n_cap);
  // Narrower tiles only for a handful of tiles (an eighth of the SMs): a 128-column
  // tile stages two thirds of the bytes of a 256-column one for half its FLOPs, and
  // measured 0.65 of its throughput, so idle SMs cost less than narrow tiles
  // (2048x2048x8192: 1320 TFLOP/s at 256 columns on 128 of 148 SMs, 744 at 128 columns).
  const int64_t psplit_factor = (parallel_splits && d.split_k > 1) ? d.split_k : 1;
  while (!fixed_n && bn > 64 &&
         ceil_div(d.m, kBlockM) * ceil_div(d.n, bn) * d.batch * psplit_factor * 8 < sm_count)
    bn = static_cast<int>(round_up(bn / 2, gran));
  // Short K and less than half a round of 128x256 tiles: what the call costs is the fixed
  // time of one tile (first copies, epilogue of the whole tile), not tensor throughput, so
  // tiles narrow until they occupy the SMs (1024^3: 14.9 -> 12.2 us with 128 tiles of
  // 128x64; 2048x512x1024: 14.4 -> 11.8 us).
  if (!fixed_n && d.k <= 1024 && d.split_k <= 1) {
    const int64_t row_tiles = ceil_div(d.m, kBlockM) * d.batch;
    if (row_tiles * ceil_div(d.n, bn) * 2 <= sm_count) {
      while (bn > 64 && row_tiles * ceil_div(d.n, static_cast<int>(round_up(bn / 2, gran))) <= sm_count)
        bn = static_cast<int>(round_up(bn / 2, gran));
    }
  }
  plan.block_n = bn;
  const int want_splits = d.split_k > 1 ? d.split_k : 1;
  plan.psplits = parallel_splits ? want_splits : 1;
  plan.splits = parallel_splits ? 1 : want_splits;
  const int64_t k_blocks_total = ceil_div(d.k, kStageK);
  plan.k_blocks = static_cast<int>(ceil_div(k_blocks_total, want_splits));
  // CTA pairs halve the B bytes each SM stages per FLOP (deeper pipeline, less L2
  // traffic). Taken when both halves of the B tile are whole 64-column chunks and
  // the pairs' waves do not outlast the single CTAs' (a pair's tile takes about
  // 0.85 of the time of two single tiles).
  const int64_t per_row_tile = ceil_div(d.n, bn) * d.batch * plan.psplits;
  const int64_t work1 = ceil_div(d.m, kBlockM) * per_row_tile, work2 = ceil_div(d.m, 2 * kBlockM) * per_row_tile;
  const int pairs = sm_count / 2;
  const double waves1 = static_cast<double>(ceil_div(work1, sm_count));
  const double waves2 = pairs > 0 ? static_cast<double>(ceil_div(work2, pairs)) : 1e30;
  plan.cta_group = (bn % 128 == 0 && pairs > 0 && waves2 * 0.85 <= waves1) ? 2 : 1;
  if (d.force_kernel == 3) plan.cta_group = 1;
  if (d.force_kernel == 4 && bn % 128 == 0 && pairs > 0) plan.cta_group = 2;
  const int cg = plan.cta_group;
  const size_t stage = static_cast<size_t>(kBlockM) * 128 + static_cast<size_t>(bn / cg) * 128;
  int stages = static_cast<int>((size_t(227) * 1024 - 2048) / stage);
  if (stages > kMaxStages) stages = kMaxStages;
  plan.stages = stages;
  plan.smem = stage * stages + 1024 + sizeof(PipelineBarriers);
  if (cg == 2)
    plan.grid = 2 * static_cast<unsigned>(work2 < pairs ? work2 : pairs);
  else
    plan.grid = static_cast<unsigned>(work1 < sm_count ? work1 : sm_count);
  return plan;
}

// `partials`: NULL, or room for split_k * batch * m * n floats: the K splits then
// run as parallel work items and the ordered reduction applies the epilogue.
// Batches to peel off the end of a batched problem and run as a second launch with
// 128-column tiles, or 0. A persistent grid of CTA pairs runs ceil(tiles / pairs) rounds
// of tiles; when the last round would be less than half full and the batches it holds
// fit one round of half-width tiles, that round costs ~0.7 of a full one instead of 1
// (C5: 256 tiles on 74 pairs are 3.46 rounds, run as 4; peeled: 3 + one round of 72
// half-width tiles).
int64_t tail_batches(const b200_gemm_desc& d, const UmmaPlan& plan, int sm_count) {
  if (d.batch < 2 || plan.cta_group != 2 || plan.block_n != 256 || plan.psplits != 1 || d.tile_n != 0) return 0;
  if (d.n % 256 != 0) return 0;  // the half-width tiles must split every column tile in two
  const int64_t pairs = sm_count / 2;
  const int64_t per_batch = ceil_div(d.m, 2 * kBlockM) * ceil_div(d.n, plan.block_n);
  const int64_t work = per_batch * d.batch;
  const int64_t full_rounds = work / pairs, excess = work - full_rounds * pairs;
  if (full_rounds < 1 || excess == 0 || excess * 2 > pairs) return 0;
  const int64_t peel = ceil_div(excess, per_batch);
  if (peel >= d.batch || peel * per_batch * 2 > pairs) return 0;
  return peel;
}

int run_gemm_umma(const b200_gemm_desc& d, const GemmEpilogue& epi, float* partials, cudaStream_t stream,
                  const PeerOut* peers) {
  const DeviceInfo& dev = device_info();
  if (dev.sm_count == 0) return refuse(B200_E_DEVICE);
  const bool a_kmajor = d.a_layout == B200_LAYOUT_ROW || d.a_layout == B200_LAYOUT_BLOCKED;  // K contiguous
  const bool b_kmajor = d.b_layout == B200_LAYOUT_COL;  // [N,K]: K contiguous
  const bool parallel = partials != nullptr && d.split_k > 1;
  const UmmaPlan plan = umma_plan(d, dev.sm_count, parallel);
  if (const int64_t peel = (parallel || peers) ? 0 : tail_batches(d, plan, dev.sm_count)) {
    b200_gemm_desc head = d, tail = d;
    head.batch = d.batch - peel;
    head.tile_n = -256;  // fixed widths: neither part is planned (or peeled) again
    tail.batch = peel;
    tail.tile_n = -128;
    const int64_t out_size = d.out_dtype == B200_BF16 ? 2 : 4;
    tail.a = static_cast<const uint8_t*>(d.a) + head.batch * d.stride_a * 2;
    tail.b = static_cast<const uint8_t*>(d.b) + head.batch * d.stride_b * 2;
    tail.c = static_cast<uint8_t*>(d.c) + head.batch * d.stride_c * out_size;
    int rc = run_gemm_umma(head, epi, nullptr, stream, nullptr);
    if (rc != 0) return rc;
    rc = run_gemm_umma(tail, epi, nullptr, stream, nullptr);
    if (rc == 0) counters().calls.fetch_sub(1, std::memory_order_relaxed);  // one call, two launches
    return rc;
  }

  CUtensorMap map_a, map_b;
  bool ok, a_chunked = false, b_chunked = false;
  const bool a_blocked = d.a_layout == B200_LAYOUT_BLOCKED;
  if (a_blocked) {
    const int64_t mb = round_up(d.m, 32) / 32, kb = round_up(d.k, 32) / 32;
    ok = encode_map_blocked(&map_a, d.a, mb, kb, d.batch, d.batch > 1 ? d.stride_a : mb * kb * 1024, kBlockM / 32);
  } else if (a_kmajor)
    ok = encode_map(&map_a, d.a, d.k, d.m, d.batch, d.lda, d.batch > 1 ? d.stride_a : d.lda * d.m, kStageK, kBlockM);
  else {
    // [K, M]: with M in whole 64-column chunks both chunks of a stage arrive in one copy
    a_chunked = d.m % 64 == 0 && encode_map_chunked(&map_a, d.a, d.m, d.k, d.batch, d.lda,
                                                    d.batch > 1 ? d.stride_a : d.lda * d.k, kStageK, kBlockM / 64);
    ok = a_chunked ||
         encode_map(&map_a, d.a, d.m, d.k, d.batch, d.lda, d.batch > 1 ? d.stride_a : d.lda * d.k, 64, kStageK);
  }
  if (!ok) return refuse(B200_E_DEVICE);
  if (b_kmajor)
    ok = encode_map(&map_b, d.b, d.k, d.n, d.batch, d.ldb, d.batch > 1 ? d.stride_b : d.ldb * d.n, kStageK,
                    plan.block_n / plan.cta_group);
  else {
    // [K, N]: the same for N
    b_chunked = d.n % 64 == 0 &&
                encode_map_chunked(&map_b, d.b, d.n, d.k, d.batch, d.ldb, d.batch > 1 ? d.stride_b : d.ldb * d.k, kStageK,
                                   static_cast<uint32_t>(plan.block_n / plan.cta_group / 64));
    ok = b_chunked ||
         encode_map(&map_b, d.b, d.n, d.k, d.batch, d.ldb, d.batch > 1 ? d.stride_b : d.ldb * d.k, 64, kStageK);
  }
  if (!ok) return refuse(B200_E_DEVICE);

  UmmaParams p{};
  p.m = static_cast<int32_t>(d.m);
  p.n = static_cast<int32_t>(d.n);
  p.k = static_cast<int32_t>(d.k);
  p.batch = static_cast<int32_t>(d.batch);
  p.tiles_m = static_cast<int32_t>(ceil_div(d.m, kBlockM * plan.cta_group));
  p.tiles_n = static_cast<int32_t>(ceil_div(d.n, plan.block_n));
  p.group_m = raster_group(d, p.tiles_m);
  p.splits = plan.splits;
  p.psplits = plan.psplits;
  p.k_blocks = plan.k_blocks;
  p.block_n = plan.block_n;
  p.stages = plan.stages;
  p.a_kmajor = a_kmajor;
  p.b_kmajor = b_kmajor;
  p.a_chunked = a_chunked;
  p.b_chunked = b_chunked;
  p.idesc = make_idesc(plan.block_n, a_kmajor, b_kmajor, plan.cta_group);
  p.a_stage_bytes = kBlockM * 128;
  p.b_stage_bytes = static_cast<uint32_t>(plan.block_n / plan.cta_group) * 128;  // this CTA's share of the B tile
  // K-major: 8-row groups 1024 B apart, K step = 32 B inside the swizzled row.
  // MN-major: 8-k-row groups 1024 B apart (SBO), 64-column chunks 8 KiB apart (LBO), K step = 16 rows = 2 KiB.
  // Blocked A: rows of 64 bytes (one 32-wide K block) under the 64-byte swizzle, 8-row groups
  // 512 B apart; the stage's second K block starts 8 KiB (128 rows) further on.
  p.a_desc_hi = a_blocked ? desc_hi(512, 4) : desc_hi(1024);
  p.b_desc_hi = desc_hi(1024);
  p.a_desc_lbo = a_kmajor ? 1u : (8192u >> 4);
  p.b_desc_lbo = b_kmajor ? 1u : (8192u >> 4);
  p.a_kstep = a_kmajor ? (32u >> 4) : (2048u >> 4);
  p.b_kstep = b_kmajor ? (32u >> 4) : (2048u >> 4);
  p.a_khalf = a_blocked ? (8192u >> 4) : 2 * p.a_kstep;
  if (parallel) {
    p.epi = GemmEpilogue{};
    p.c = partials;
    p.ldc = d.n;
    p.stride_c = d.m * d.n;
    p.psplit_stride = d.batch * d.m * d.n;
    p.out_bf16 = 0;
  } else {
    p.epi = epi;
    p.c = d.c;
    p.ldc = d.ldc;
    p.stride_c = d.stride_c;
    p.out_bf16 = d.out_dtype == B200_BF16;
  }
  const size_t out_size = p.out_bf16 ? 2 : 4;
  p.vec_store = aligned(p.c, 16) && (p.ldc * out_size) % 16 == 0 && (p.stride_c * out_size) % 16 == 0 &&
                (p.psplit_stride * out_size) % 16 == 0;
  p.vec_params = aligned(epi.bias, 16) && aligned(epi.scale, 16) && aligned(epi.shift, 16);
  p.status = kernel_status_word();
  size_t smem_bytes = plan.smem;
  if (peers) {
    if (parallel || plan.splits > 1 || a_blocked) return refuse(B200_E_ARG);  // one launch, one epilogue per tile; plain A
    p.peer = *peers;
    for (int j = 0; j < peers->count; ++j)  // every copy must take the same kind of stores
      p.vec_store = p.vec_store && (peers->delta[j] % 16 == 0);
    // Staged stores (see the epilogue): bf16 results, 16-byte aligned rows, column halves in
    // whole 64-column pieces. The eight 4 KiB staging tiles take the place of pipeline stages.
    if (p.out_bf16 && p.vec_store && (plan.block_n / 2) % 64 == 0) {
      const size_t stage = static_cast<size_t>(p.a_stage_bytes) + p.b_stage_bytes;
      const size_t staging = static_cast<size_t>(kEpilogueWarps) * 4096;
      while (p.stages > 2 && stage * p.stages + 1024 + sizeof(PipelineBarriers) + 1024 + staging > size_t(227) * 1024) --p.stages;
      smem_bytes = stage * p.stages + 1024 + sizeof(PipelineBarriers) + 1024 + staging;
      p.peer_staged = smem_bytes <= size_t(227) * 1024;
      if (!p.peer_staged) {
        p.stages = plan.stages;
        smem_bytes = plan.smem;
      }
    }
  }

  std::call_once(g_attr_once[dev.device], [] {
    cudaFuncSetAttribute(gemm_umma_bf16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(gemm_umma_bf16_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(gemm_umma_bf16_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(gemm_umma_bf16_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(gemm_umma_bf16_kernel<1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(gemm_umma_bf16_kernel<2, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  });
  if (plan.cta_group == 2) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(plan.grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    config.attrs = &attr;
    config.numAttrs = 1;
    const cudaError_t err = peers       ? cudaLaunchKernelEx(&config, gemm_umma_bf16_kernel<2, true>, map_a, map_b, p)
                            : a_blocked ? cudaLaunchKernelEx(&config, gemm_umma_bf16_kernel<2, false, true>, map_a, map_b, p)
                                        : cudaLaunchKernelEx(&config, gemm_umma_bf16_kernel<2>, map_a, map_b, p);
    if (err != cudaSuccess) {
      cudaGetLastError();
      return finish(-static_cast<int>(err));
    }
  } else {
    if (peers)
      gemm_umma_bf16_kernel<1, true><<<plan.grid, kThreads, smem_bytes, stream>>>(map_a, map_b, p);
    else if (a_blocked)
      gemm_umma_bf16_kernel<1, false, true><<<plan.grid, kThreads, smem_bytes, stream>>>(map_a, map_b, p);
    else
      gemm_umma_bf16_kernel<1><<<plan.grid, kThreads, smem_bytes, stream>>>(map_a, map_b, p);
  }
  if (!parallel) return launched();
  const int rc = check_launch();
  if (rc != 0) return finish(rc);
  return launch_splitk_reduce(partials, plan.psplits, d.batch, d.m, d.n, d.c, d.out_dtype == B200_BF16, d.ldc,
                              d.stride_c, epi, stream);
}

// Encodes one store map per copy of C ([rows, cols] bf16, rows `ld` apart, boxes of 32 rows x
// 64 columns) and writes them to `device_maps` (count x 128 bytes, 64-byte aligned) on the
// current device. Synchronous: a set-up step.
int store_peer_maps(void* device_maps, void* const* c, int count, int64_t rows, int64_t cols, int64_t ld) {
  if (!device_maps || !c || count < 1 || count > B200_MAX_PEERS) return refuse(B200_E_ARG);
  if (!aligned(device_maps, 64) || cols % 8 || ld % 8) return refuse(B200_E_ALIGN);
  CUtensorMap maps[B200_MAX_PEERS];
  for (int j = 0; j < count; ++j) {
    if (!c[j] || !aligned(c[j], 16)) return refuse(B200_E_ALIGN);
    if (!encode_store_map(&maps[j], c[j], cols, rows, ld, 32)) return refuse(B200_E_DEVICE);
  }
  const cudaError_t err = cudaMemcpy(device_maps, maps, sizeof(CUtensorMap) * count, cudaMemcpyHostToDevice);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return finish(-static_cast<int>(err));
  }
  return finish(0);
}

int run_peer_wait(const int32_t* flags, int count, int32_t epoch, unsigned long long budget_ns, cudaStream_t stream) {
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  peer_wait_kernel<<<1, 32, 0, stream>>>(flags, count, epoch, budget_ns, kernel_status_word());
  return launched();
}

int run_wait_timeout_selftest(unsigned long long budget_ns, cudaStream_t stream) {
  if (device_info().sm_count == 0) return refuse(B200_E_DEVICE);
  int32_t* status = kernel_status_word();
  if (!status) return refuse(B200_E_DEVICE);
  wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(budget_ns, status);
  return launched();
}

int explain_gemm_umma(const b200_gemm_desc& d, char* buf, size_t len) {
  const DeviceInfo& dev = device_info();
  const bool parallel = d.workspace != nullptr && d.split_k > 1;
  const UmmaPlan plan = umma_plan(d, dev.sm_count > 0 ? dev.sm_count : 148, parallel);
  const int64_t peel = parallel ? 0 : tail_batches(d, plan, dev.sm_count > 0 ? dev.sm_count : 148);
  int used = snprintf(buf, len, "umma_bf16 cta_group=%d tile=%dx%dx%d stages=%d serial_splits=%d parallel_splits=%d grid=%u smem=%zu",
                      plan.cta_group, kBlockM * plan.cta_group, plan.block_n, kStageK, plan.stages, plan.splits, plan.psplits,
                      plan.grid, plan.smem);
  if (peel > 0 && used > 0 && static_cast<size_t>(used) < len)
    snprintf(buf + used, len - used, " tail_batches=%lld as a second launch with 128-column tiles", static_cast<long long>(peel));
  return 0;
}

}  // namespace b200
