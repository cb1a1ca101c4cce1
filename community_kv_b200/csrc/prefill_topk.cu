// Prefill score-graph emission: causal attention that also reports, for every
// query row, the keys it attends to most (sm_100a, tcgen05 tensor cores + TMEM).
//
// One CTA owns a 128-row tile: 128/G consecutive positions times the G query
// heads of one KV head (the heads of a group share every K/V tile).  Per 128-key
// block:
//   S  = Q K^T   tcgen05.mma (M=128, N=128, K=16 x 8), operands in shared memory
//                in the canonical un-swizzled 8x16-byte core-matrix layout,
//                accumulator in tensor memory;
//   each thread owns one row: it reads the row back with tcgen05.ld, applies the
//   causal mask, feeds the neighbour-candidate queues, updates the running
//   softmax and writes P (bf16) to shared memory;
//   O' = P V     tcgen05.mma again (V is consumed N-major straight from the same
//                [key][dim] staging layout), read back and folded into the
//                thread's fp32 output row.
// K/V tiles are staged with 16-byte cp.async; the next tile's fetch overlaps the
// softmax and the second MMA.  Every wait on a tensor-core completion barrier is
// bounded and reports through the status word.
//
// Neighbour candidates, mode 1 (the reference's rule, community-kv.patch
// hopper/topk_warpselect.h): per row, four classes of columns (class = (j%8)/2)
// each keep their six best packed candidates, key15 = clamp(rn((s+48)*256)) on
// the raw Q.K score, packed = key15 << 17 | j; the row reports the eight largest
// of the 24, probability = exp2(dequant(key15)*scale*log2e - lse*log2e).
// Mode 2 (exact top-m per KV head): per position the group maximum of the scaled
// scores is ranked; each of the G lanes of a position keeps the 16 best of the
// columns j % G == lane, and a second kernel re-scores that short list in the
// fixed fp32 order shared with the CPU oracle and emits the exact top-m.

#include "tc_primitives.cuh"

namespace ckv {

// Returns the key that fell off the end (the candidate itself when it did not enter).
__device__ __forceinline__ uint64_t queue_insert64(uint64_t (&queue)[kExactKeep], uint64_t candidate) {
#pragma unroll
  for (int k = 0; k < kExactKeep; ++k) {
    const uint64_t resident = queue[k];
    const bool greater = candidate > resident;
    queue[k] = greater ? candidate : resident;
    candidate = greater ? resident : candidate;
  }
  return candidate;
}

// One step of a max reduce-scatter over 2 * kWidth columns between lane pairs
// `offset` apart: the lane with `upper` set keeps the upper half of the columns.
template <int kWidth>
__device__ __forceinline__ void butterfly_stage(const float (&in)[2 * kWidth], float (&out)[kWidth],
                                                bool upper, int offset) {
#pragma unroll
  for (int i = 0; i < kWidth; ++i) {
    const float keep = upper ? in[kWidth + i] : in[i];
    const float send = upper ? in[i] : in[kWidth + i];
    out[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, offset));
  }
}

// Ranks kCount group-maximum scores (columns first, first + 1, ...) into the lane's
// list.  `prune`: scores below it cannot be among the position's best 16.  `dropped`
// collects the best score that was turned away.
template <int kCount>
__device__ __forceinline__ void rank_owned(const float (&raw)[kCount], int first, float scale,
                                           float prune, uint64_t (&list)[kExactKeep],
                                           float& dropped) {
  float best = -INFINITY;
#pragma unroll
  for (int i = 0; i < kCount; ++i) {
    best = fmaxf(best, raw[i]);
  }
  const uint64_t last = list[kExactKeep - 1];
  const float own = last == 0ull ? -INFINITY : key32_to_float(static_cast<uint32_t>(last >> 32));
  const float gate = fmaxf(prune, own);
  if (best * scale < gate) {
    dropped = fmaxf(dropped, best * scale);
    return;
  }
#pragma unroll
  for (int i = 0; i < kCount; ++i) {
    const float v = raw[i] * scale;
    if (v >= gate) {
      const uint64_t candidate = (static_cast<uint64_t>(ordered_key32(v)) << 32) |
                                 (0xffffffffu - static_cast<uint32_t>(first + i));
      const uint64_t lost =
          candidate > list[kExactKeep - 1] ? queue_insert64(list, candidate) : candidate;
      if (lost != 0ull) {
        dropped = fmaxf(dropped, key32_to_float(static_cast<uint32_t>(lost >> 32)));
      }
    } else {
      dropped = fmaxf(dropped, v);
    }
  }
}

// kGroup: query heads per KV head (1, 2, 4, 8).  kMode: 0 attention only,
// 1 reference top-8 per query head, 2 candidate lists for the exact top-m.
//
// 256 threads: thread t owns row t % 128 and the column half t / 128 of every
// 128-key block (and the same half of the 128 output dimensions).  K, V and the
// S accumulator are double buffered so that the next block's Q.K^T runs on the
// tensor cores while this block's softmax and candidate bookkeeping run on the
// CUDA cores, and P.V of this block runs under the next block's softmax.
struct PrefillSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = kTileBytes;            // two buffers
  static constexpr int kV = 3 * kTileBytes;        // two buffers
  static constexpr int kP = 5 * kTileBytes;
  static constexpr int kExchange = 6 * kTileBytes;  // float [2][128] row maxima / sums
  static constexpr int kFloors = kExchange + 2 * kPfRows * 4;  // uint32 [2][128] list floors
  static constexpr int kBars = kFloors + 2 * kPfRows * 4;
  static constexpr int kTotal = kBars + 64;  // 7 barriers and the TMEM base slot
};

template <int kGroup, int kMode>
__global__ void __launch_bounds__(kPfThreads, 1)
    prefill_kernel(const ckv_prefill_args a, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* s_q = smem + PrefillSmem::kQ;
  uint8_t* s_k = smem + PrefillSmem::kK;
  uint8_t* s_v = smem + PrefillSmem::kV;
  uint8_t* s_p = smem + PrefillSmem::kP;
  float* exchange = reinterpret_cast<float*>(smem + PrefillSmem::kExchange);
  uint32_t* floor_exchange = reinterpret_cast<uint32_t*>(smem + PrefillSmem::kFloors);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PrefillSmem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);

  constexpr int kPositions = kPfRows / kGroup;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int row = tid & (kPfRows - 1);
  const int half = tid >> 7;            // which 64 of the 128 columns / output dims
  const int col0 = half * 64;
  const int tile = gridDim.x - 1 - blockIdx.x;  // longest rows first
  const int kv_head = blockIdx.y;
  const int batch = blockIdx.z;
  const int pos0 = tile * kPositions;
  const int length = a.seq_len;
  const int row_pos = pos0 + row / kGroup;
  const int row_head = kv_head * kGroup + row % kGroup;
  const bool row_live = row_pos < length;

  const uint32_t bar_s0 = smem_u32(bars);
  const uint32_t bar_s1 = smem_u32(bars + 1);
  const uint32_t bar_o = smem_u32(bars + 2);
  const uint32_t bar_k = smem_u32(bars + 3);  // two barriers: K buffer filled
  const uint32_t bar_v = smem_u32(bars + 5);  // two barriers: V buffer filled
  const int last_pos = min(length, pos0 + kPositions) - 1;
  const int blocks = last_pos / kPfKeys + 1;
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 7; ++i) {
      mbar_init(bar_s0 + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tma_load_tile(smem_u32(s_k), &map_k, bar_k, 0, kv_head, batch);
    tma_load_tile(smem_u32(s_v), &map_v, bar_v, 0, kv_head, batch);
    if (blocks > 1) {
      tma_load_tile(smem_u32(s_k) + kTileBytes, &map_k, bar_k + 8, kPfKeys, kv_head, batch);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  const __nv_bfloat16* q_base = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                                batch * a.q_batch_stride;
  // ---- stage Q once: row r = (position pos0 + r / G, head kv_head*G + r % G) ----
  for (int index = tid; index < kPfRows * 16; index += kPfThreads) {
    const int r = (index & 7) | ((index >> 7) << 3);
    const int chunk = (index >> 3) & 15;
    const int pos = pos0 + r / kGroup;
    const int head = kv_head * kGroup + r % kGroup;
    const bool live = pos < length;
    const __nv_bfloat16* src =
        q_base + (live ? pos : 0) * a.q_row_stride + head * a.q_head_stride + chunk * 8;
    cp_async16(smem_u32(s_q) + core_offset(r, chunk), src, live ? 16u : 0u);
  }
  cp_async_commit();
  cp_async_wait<0>();
  async_proxy_fence();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + (((warp & 3) * 32u) << 16);
  const uint32_t idesc_qk = instruction_descriptor(false);
  const uint32_t idesc_pv = instruction_descriptor(true);

  auto issue_qk = [&](int block) {
    const int buffer = block & 1;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint64_t desc_q = smem_descriptor(smem_u32(s_q) + ks * 4096, 2048, 128);
      const uint64_t desc_k =
          smem_descriptor(smem_u32(s_k) + buffer * kTileBytes + ks * 4096, 2048, 128);
      umma(tmem + buffer * 128u, desc_q, desc_k, idesc_qk, ks > 0 ? 1u : 0u);
    }
    umma_commit(buffer ? bar_s1 : bar_s0);
  };
  bool failed = false;
  if (tid == 0) {
    if (mbar_wait(bar_k, 0)) {
      tc_fence_after();
      issue_qk(0);
    } else {
      failed = true;
    }
  }

  float out[64];  // filled from tensor memory after the last block
  float run_max = -INFINITY;  // of the raw (unscaled) scores, whole row
  float run_sum = 0.f;        // this thread's column half only
  const float scale_log2 = a.softmax_scale * kLog2e;
  uint32_t q32[4][kLocalK];
  uint64_t q64[kExactKeep];
  float dropped = -INFINITY;  // best score this list ever turned away
  if constexpr (kMode == 1) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int k = 0; k < kLocalK; ++k) {
        q32[c][k] = 0u;
      }
    }
  }
  if constexpr (kMode == 2) {
#pragma unroll
    for (int k = 0; k < kExactKeep; ++k) {
      q64[k] = 0ull;
    }
  }
  const int limit = row_live ? min(row_pos, length - 1) : -1;  // last visible key

  // O accumulates in tensor memory over all key blocks (P.V with accumulate); the
  // registers see it twice: when a row's running maximum moves by more than 2^8 (the
  // row is then rescaled in place) and at the very end.
  auto wait_output = [&](int block) {
    if (!mbar_wait(bar_o, block & 1)) {
      failed = true;
    }
    tc_fence_after();
  };

  for (int block = 0; block < blocks; ++block) {
    const int key0 = block * kPfKeys;
    const int buffer = block & 1;
    if (!mbar_wait(buffer ? bar_s1 : bar_s0, (block >> 1) & 1)) {
      failed = true;
    }
    tc_fence_after();
    // ---- this thread's 64 raw scores, kept in registers ----
    float s[64];
    tmem_load64(lane_base + buffer * 128u + col0, s);
    // its K buffer is free again: fetch the block after next into it
    if (tid == 0 && block + 2 < blocks) {
      tma_load_tile(smem_u32(s_k) + buffer * kTileBytes, &map_k, bar_k + 8 * buffer,
                    key0 + 2 * kPfKeys, kv_head, batch);
    }
    // interior block: every key is visible to every row of the tile.  Elsewhere the
    // causal mask is applied once, in place.
    const bool interior = key0 + kPfKeys - 1 <= pos0;
    if (!interior) {
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        s[c] = (key0 + col0 + c) <= limit ? s[c] : -INFINITY;
      }
    }
    float half_max = -INFINITY;
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      half_max = fmaxf(half_max, s[c]);
    }
    exchange[half * kPfRows + row] = half_max;
    if constexpr (kMode == 2) {
      // 16th-best key of this list, maximised over the lists of the position: no
      // list's 16th entry can lie above the position's 16th best, so anything
      // clearly below it is out of the race
      uint32_t floor_key = static_cast<uint32_t>(q64[kExactKeep - 1] >> 32);
#pragma unroll
      for (int offset = 1; offset < kGroup; offset <<= 1) {
        floor_key = max(floor_key, __shfl_xor_sync(0xffffffffu, floor_key, offset));
      }
      floor_exchange[half * kPfRows + row] = floor_key;
    }
    tc_fence_before();
    if (__syncthreads_or(failed ? 1 : 0)) {
      failed = true;
      break;
    }
    // ---- next block's S = Q K^T starts now, under this block's softmax ----
    if (tid == 0 && block + 1 < blocks) {
      if (mbar_wait(bar_k + 8 * (buffer ^ 1), ((block + 1) >> 1) & 1)) {
        tc_fence_after();
        issue_qk(block + 1);
      } else {
        failed = true;
      }
    }
    const float tile_max = fmaxf(half_max, exchange[(half ^ 1) * kPfRows + row]);
    const bool sink_free = key0 >= a.num_sink;

    if constexpr (kMode == 1) {
      if (sink_free) {
        // A key that is below eight keys already held can never reach the output:
        // the second-best entries of the four classes are eight such keys, and so
        // are the top four of the two best classes.
        const uint32_t third0 = q32[0][3], third1 = q32[1][3], third2 = q32[2][3], third3 = q32[3][3];
        const uint32_t second_of_fourths =
            max(min(max(third0, third1), max(third2, third3)),
                max(min(third0, third1), min(third2, third3)));
        const uint32_t row_floor = max(min(min(q32[0][1], q32[1][1]), min(q32[2][1], q32[3][1])),
                                       second_of_fourths);
        // smallest raw score whose quantised key can reach the floor, a little low
        const float gate = (row_floor >> 17) == 0u
                               ? -3.0e38f
                               : (static_cast<float>(row_floor >> 17) - 0.75f) * (1.0f / 256.0f) - 48.0f;
        // Class by class (16 of this thread's 64 columns each): the columns that reach
        // the gate as a bit mask, then insertion in rounds - every lane with a pending
        // column inserts its next one per round - so that the divergent insertion code
        // runs as often as the busiest lane needs, not once per column with a taker.
        if (__any_sync(0xffffffffu, half_max >= gate)) {
#pragma unroll
          for (int cls = 0; cls < 4; ++cls) {
            uint32_t takers = 0u;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int c = (i >> 1) * 8 + cls * 2 + (i & 1);
              takers |= (s[c] >= gate ? 1u : 0u) << i;
            }
            while (__any_sync(0xffffffffu, takers != 0u)) {
              if (takers != 0u) {
                const int i = __ffs(takers) - 1;
                takers &= takers - 1;
                float v = s[cls * 2];
#pragma unroll
                for (int k = 1; k < 16; ++k) {
                  v = i == k ? s[(k >> 1) * 8 + cls * 2 + (k & 1)] : v;
                }
                const int c = (i >> 1) * 8 + cls * 2 + (i & 1);
                const uint32_t candidate = (quantised_key(v) << 17) |
                                           (static_cast<uint32_t>(key0 + col0 + c) & 0x1ffffu);
                if (candidate > q32[cls][kLocalK - 1]) {
                  queue_insert<kLocalK>(q32[cls], candidate);
                }
              }
            }
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int j = key0 + col0 + c;
          if (s[c] > -INFINITY && j >= a.num_sink) {
            const uint32_t candidate =
                (quantised_key(s[c]) << 17) | (static_cast<uint32_t>(j) & 0x1ffffu);
            uint32_t(&queue)[kLocalK] = q32[(c & 7) >> 1];
            if (candidate > queue[kLocalK - 1]) {
              queue_insert<kLocalK>(queue, candidate);
            }
          }
        }
      }
    }
    if constexpr (kMode == 2) {
      // The score of a key for a position is the maximum over the G heads of the
      // group (G adjacent lanes).
      if (interior && sink_free) {
        const uint32_t floor_key =
            max(floor_exchange[row], floor_exchange[kPfRows + row]);  // both halves' lists
        const float prune =
            floor_key == 0u ? -INFINITY : key32_to_float(floor_key) - 2.0f * a.exact_slack;
        float group_max = half_max;
#pragma unroll
        for (int offset = 1; offset < kGroup; offset <<= 1) {
          group_max = fmaxf(group_max, __shfl_xor_sync(0xffffffffu, group_max, offset));
        }
        const float block_best = group_max * a.softmax_scale;
        if (!__any_sync(0xffffffffu, block_best >= prune)) {
          dropped = fmaxf(dropped, block_best);
        } else {
          // reduce-scatter over the group: afterwards every lane holds the group
          // maximum of 64 / G columns of its own
          const int lane = tid & 31;
          if constexpr (kGroup == 1) {
            rank_owned<64>(s, key0 + col0, a.softmax_scale, prune, q64, dropped);
          } else {
            float half32[32];
            butterfly_stage<32>(s, half32, (lane & 1) != 0, 1);
            int first = key0 + col0 + ((lane & 1) ? 32 : 0);
            if constexpr (kGroup == 2) {
              rank_owned<32>(half32, first, a.softmax_scale, prune, q64, dropped);
            } else {
              float quarter[16];
              butterfly_stage<16>(half32, quarter, (lane & 2) != 0, 2);
              first += (lane & 2) ? 16 : 0;
              if constexpr (kGroup == 4) {
                rank_owned<16>(quarter, first, a.softmax_scale, prune, q64, dropped);
              } else {
                float eighth[8];
                butterfly_stage<8>(quarter, eighth, (lane & 4) != 0, 4);
                first += (lane & 4) ? 8 : 0;
                rank_owned<8>(eighth, first, a.softmax_scale, prune, q64, dropped);
              }
            }
          }
        }
      } else {
        // masked or sink-bearing block: lane h of the group ranks the columns j % G == h
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int j = key0 + col0 + c;
          float v = j >= a.num_sink ? s[c] * a.softmax_scale : -INFINITY;
#pragma unroll
          for (int offset = 1; offset < kGroup; offset <<= 1) {
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
          }
          if ((c % kGroup) == (row % kGroup) && v > -INFINITY) {
            const uint64_t candidate = (static_cast<uint64_t>(ordered_key32(v)) << 32) |
                                       (0xffffffffu - static_cast<uint32_t>(j));
            // keep the best score that was ever turned away: the second kernel needs
            // it to prove that the short list is complete
            const uint64_t lost =
                candidate > q64[kExactKeep - 1] ? queue_insert64(q64, candidate) : candidate;
            if (lost != 0ull) {
              dropped = fmaxf(dropped, key32_to_float(static_cast<uint32_t>(lost >> 32)));
            }
          }
        }
      }
    }

    // The running maximum is only moved when the new one lies more than 2^8 above it
    // (probabilities up to 256 are harmless in bf16 / fp32); moving it means rescaling
    // the output row that sits in tensor memory.
    const float new_max = fmaxf(run_max, tile_max);
    const bool move = new_max > run_max && (new_max - run_max) * scale_log2 > 8.0f;
    float corr = 1.f;
    if (move) {
      corr = run_max == -INFINITY ? 0.f : exp2f((run_max - new_max) * scale_log2);
      run_max = new_max;
      run_sum *= corr;
    }
    const float safe_max = run_max == -INFINITY ? 0.f : run_max;

    // ---- probabilities (bf16 pairs; masked keys are -inf and come out as 0) ----
    uint32_t packed[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float p0 = exp2f((s[2 * e] - safe_max) * scale_log2);
      const float p1 = exp2f((s[2 * e + 1] - safe_max) * scale_log2);
      run_sum += p0 + p1;
      packed[e] = pack_bf16(p0, p1);
    }
    // P.V of block-1 ran under the work above; fold it in, which also frees the P tile
    // and that block's V buffer
    if (block > 0) {
      wait_output(block - 1);
      if (__any_sync(0xffffffffu, move)) {
        float o[64];
        tmem_load64(lane_base + 256u + col0, o);
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          o[c] *= corr;
        }
        tmem_store64(lane_base + 256u + col0, o);
      }
    }
    if (tid == 0 && block + 1 < blocks) {
      tma_load_tile(smem_u32(s_v) + (buffer ^ 1) * kTileBytes, &map_v, bar_v + 8 * (buffer ^ 1),
                    key0 + kPfKeys, kv_head, batch);
    }
#pragma unroll
    for (int piece = 0; piece < 8; ++piece) {
      *reinterpret_cast<uint4*>(s_p + core_offset(row, half * 8 + piece)) = make_uint4(
          packed[piece * 4], packed[piece * 4 + 1], packed[piece * 4 + 2], packed[piece * 4 + 3]);
    }
    async_proxy_fence();
    tc_fence_before();
    if (__syncthreads_or(failed ? 1 : 0)) {
      failed = true;
      break;
    }
    // ---- O' = P V, runs under the next block's softmax ----
    if (tid == 0 && !mbar_wait(bar_v + 8 * buffer, (block >> 1) & 1)) {
      failed = true;  // seen by every thread at the next barrier
    } else if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t desc_p = smem_descriptor(smem_u32(s_p) + ks * 4096, 2048, 128);
        const uint64_t desc_v =
            smem_descriptor(smem_u32(s_v) + buffer * kTileBytes + ks * 256, 128, 2048);
        umma(tmem + 256u, desc_p, desc_v, idesc_pv, (ks > 0 || block > 0) ? 1u : 0u);
      }
      umma_commit(bar_o);
    }
  }
  if (!failed) {
    wait_output(blocks - 1);
    tmem_load64(lane_base + 256u + col0, out);
  }
  tc_fence_before();
  const int any_failed = __syncthreads_or(failed ? 1 : 0);
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512)
                 : "memory");
  }
  if (any_failed) {
    if (tid == 0 && a.status != nullptr) {
      atomicOr(a.status, CKV_DEV_WAIT_TIMEOUT);
    }
    return;
  }

  // ---- epilogue: combine the two column halves of every row ----
  exchange[half * kPfRows + row] = run_sum;
  uint32_t* queue_exchange = reinterpret_cast<uint32_t*>(s_p);  // P tile is idle now
  if (half == 1) {
    if constexpr (kMode == 1) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int k = 0; k < kLocalK; ++k) {
          queue_exchange[row * 24 + c * kLocalK + k] = q32[c][k];
        }
      }
    }
    if constexpr (kMode == 2) {
      uint64_t* wide = reinterpret_cast<uint64_t*>(s_p) + row * (kExactKeep + 1);
#pragma unroll
      for (int k = 0; k < kExactKeep; ++k) {
        wide[k] = q64[k];
      }
      wide[kExactKeep] = __float_as_uint(dropped);
    }
  }
  __syncthreads();
  if (!row_live) {
    return;
  }
  const float total = exchange[row] + exchange[kPfRows + row];
  const float inverse = 1.f / total;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.output) + batch * a.o_batch_stride +
                       static_cast<int64_t>(row_pos) * a.o_row_stride + row_head * a.o_head_stride +
                       col0;
#pragma unroll
  for (int d = 0; d < 64; d += 8) {
    uint4 v;
    v.x = pack_bf16(out[d] * inverse, out[d + 1] * inverse);
    v.y = pack_bf16(out[d + 2] * inverse, out[d + 3] * inverse);
    v.z = pack_bf16(out[d + 4] * inverse, out[d + 5] * inverse);
    v.w = pack_bf16(out[d + 6] * inverse, out[d + 7] * inverse);
    *reinterpret_cast<uint4*>(dst + d) = v;
  }
  if (half == 1) {
    return;
  }
  const float lse = run_max * a.softmax_scale + logf(total);
  const int64_t heads_total = static_cast<int64_t>(gridDim.y) * kGroup;
  a.lse[(batch * heads_total + row_head) * length + row_pos] = lse;

  if constexpr (kMode == 1) {
    // fold the other half's class queues into this thread's
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int k = 0; k < kLocalK; ++k) {
        const uint32_t candidate = queue_exchange[row * 24 + c * kLocalK + k];
        if (candidate > q32[c][kLocalK - 1]) {
          queue_insert<kLocalK>(q32[c], candidate);
        }
      }
    }
    const int skip = a.num_sink + kKappa - 1;
    if (row_pos >= skip) {
      // merge the four sorted class queues: eight rounds of "largest head wins"
      int cursor[4] = {0, 0, 0, 0};
      const int64_t base =
          ((batch * heads_total + row_head) * (length - skip) + (row_pos - skip)) * kKappa;
      const float lse_log2 = lse * kLog2e;
#pragma unroll
      for (int rank = 0; rank < kKappa; ++rank) {
        uint32_t best = 0u;
        int winner = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t head = 0u;
#pragma unroll
          for (int k = 0; k < kLocalK; ++k) {
            head = cursor[c] == k ? q32[c][k] : head;
          }
          if (head > best) {
            best = head;
            winner = c;
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          cursor[c] += (c == winner) ? 1 : 0;
        }
        const float dequant = static_cast<float>(best >> 17) / 256.0f - 48.0f;
        a.topk_val[base + rank] = exp2f(dequant * scale_log2 - lse_log2);
        a.topk_idx[base + rank] = static_cast<int32_t>(best & 0x1ffffu);
      }
    }
  }
  if constexpr (kMode == 2) {
    const uint64_t* wide = reinterpret_cast<const uint64_t*>(s_p) + row * (kExactKeep + 1);
    dropped = fmaxf(dropped, __uint_as_float(static_cast<uint32_t>(wide[kExactKeep])));
#pragma unroll
    for (int k = 0; k < kExactKeep; ++k) {
      const uint64_t candidate = wide[k];
      const uint64_t lost =
          candidate > q64[kExactKeep - 1] ? queue_insert64(q64, candidate) : candidate;
      if (lost != 0ull) {
        dropped = fmaxf(dropped, key32_to_float(static_cast<uint32_t>(lost >> 32)));
      }
    }
    // [batch, kv head, position, G lanes, 16 kept + best dropped] for the second kernel
    uint64_t* list = a.candidates +
                     (((static_cast<int64_t>(batch) * gridDim.y + kv_head) * length + row_pos) * kGroup +
                      row % kGroup) * (kExactKeep + 1);
#pragma unroll
    for (int k = 0; k < kExactKeep; ++k) {
      list[k] = q64[k];
    }
    list[kExactKeep] =
        dropped == -INFINITY ? 0ull : static_cast<uint64_t>(ordered_key32(dropped)) << 32;
  }
}

// ---- exact top-m from the candidate lists (mode 2, second kernel) ----
// One warp per (batch, KV head, position).  The G x 16 candidate keys are
// re-scored as max over the group of scale * (q . k) in the fixed fp32 order
// and ranked by (score descending, key index ascending).  A row is flagged when
// a key that was turned away could still belong to the top-m: the best
// approximate score among the dropped keys is within `slack` of the exact m-th.
__global__ void __launch_bounds__(128) exact_edges_kernel(const ckv_prefill_args a, int group) {
  const int warps_per_block = 4;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * warps_per_block + warp;
  const int length = a.seq_len;
  const int skip = a.num_sink + a.edges_per_row - 1;
  const int rows = length - skip;
  const int64_t total = static_cast<int64_t>(a.batch) * a.kv_heads * rows;
  if (item >= total || rows <= 0) {
    return;
  }
  const int pos = skip + static_cast<int>(item % rows);
  const int kv_head = static_cast<int>((item / rows) % a.kv_heads);
  const int batch = static_cast<int>(item / (static_cast<int64_t>(rows) * a.kv_heads));
  const uint64_t* list = a.candidates +
                         ((static_cast<int64_t>(batch) * a.kv_heads + kv_head) * length + pos) *
                             group * (kExactKeep + 1);
  const __nv_bfloat16* q_base = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                                batch * a.q_batch_stride + static_cast<int64_t>(pos) * a.q_row_stride +
                                kv_head * group * a.q_head_stride;
  const __nv_bfloat16* k_base = reinterpret_cast<const __nv_bfloat16*>(a.key) +
                                batch * a.k_batch_stride + kv_head * a.k_head_stride;
  const int candidates = group * kExactKeep;  // <= 128
  // the position's query rows, staged once per warp (every candidate reuses them)
  __shared__ uint4 q_stage[4][8 * 16];
  for (int index = lane; index < group * 16; index += 32) {
    q_stage[warp][index] = *reinterpret_cast<const uint4*>(q_base + (index >> 4) * a.q_head_stride +
                                                           (index & 15) * 8);
  }
  __syncwarp();
  uint64_t best_key[4];
  float best_dropped = -INFINITY;  // best approximate score among the keys turned away
  if (lane < group) {
    const uint64_t lost = list[lane * (kExactKeep + 1) + kExactKeep];
    if (lost != 0ull) {
      best_dropped = key32_to_float(static_cast<uint32_t>(lost >> 32));
    }
  }
#pragma unroll
  for (int slot = 0; slot < 4; ++slot) {
    best_key[slot] = 0ull;
    const int index = lane + 32 * slot;
    if (index >= candidates) {
      continue;
    }
    const uint64_t packed = list[(index / kExactKeep) * (kExactKeep + 1) + index % kExactKeep];
    if (packed == 0ull) {
      continue;
    }
    const int j = static_cast<int>(0xffffffffu - static_cast<uint32_t>(packed));
    const uint4* k_row = reinterpret_cast<const uint4*>(k_base + static_cast<int64_t>(j) * a.k_row_stride);
    uint4 k_reg[16];
#pragma unroll
    for (int piece = 0; piece < 16; ++piece) {
      k_reg[piece] = k_row[piece];
    }
    float score = -INFINITY;
    for (int g = 0; g < group; ++g) {
      // eight slices of 16 sequential mixed-precision FMAs (bf16 x bf16 + fp32, one
      // rounding each), combined in the fixed order
      float part[8];
#pragma unroll
      for (int piece = 0; piece < 8; ++piece) {
        const uint4 q0 = q_stage[warp][g * 16 + 2 * piece];
        const uint4 q1 = q_stage[warp][g * 16 + 2 * piece + 1];
        const uint4 k0 = k_reg[2 * piece];
        const uint4 k1 = k_reg[2 * piece + 1];
        float acc = 0.f;
        acc = fma2_bf16(k0.x, q0.x, acc);
        acc = fma2_bf16(k0.y, q0.y, acc);
        acc = fma2_bf16(k0.z, q0.z, acc);
        acc = fma2_bf16(k0.w, q0.w, acc);
        acc = fma2_bf16(k1.x, q1.x, acc);
        acc = fma2_bf16(k1.y, q1.y, acc);
        acc = fma2_bf16(k1.z, q1.z, acc);
        acc = fma2_bf16(k1.w, q1.w, acc);
        part[piece] = acc;
      }
      const float even = __fadd_rn(__fadd_rn(part[0], part[4]), __fadd_rn(part[2], part[6]));
      const float odd = __fadd_rn(__fadd_rn(part[1], part[5]), __fadd_rn(part[3], part[7]));
      score = fmaxf(score, __fmul_rn(__fadd_rn(even, odd), a.softmax_scale));
    }
    best_key[slot] = (static_cast<uint64_t>(ordered_key32(score)) << 32) |
                     (0xffffffffu - static_cast<uint32_t>(j));
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    best_dropped = fmaxf(best_dropped, __shfl_xor_sync(0xffffffffu, best_dropped, offset));
  }
  const int64_t out_base = ((static_cast<int64_t>(batch) * a.kv_heads + kv_head) * rows + (pos - skip)) *
                           a.edges_per_row;
  float last_score = 0.f;
  for (int rank = 0; rank < a.edges_per_row; ++rank) {
    uint64_t local = 0ull;
#pragma unroll
    for (int slot = 0; slot < 4; ++slot) {
      local = best_key[slot] > local ? best_key[slot] : local;
    }
    const uint64_t winner = warp_max_u64(local);
    if (winner != 0ull) {
#pragma unroll
      for (int slot = 0; slot < 4; ++slot) {
        best_key[slot] = best_key[slot] == winner ? 0ull : best_key[slot];
      }
    }
    last_score = key32_to_float(static_cast<uint32_t>(winner >> 32));
    if (lane == 0) {
      a.edge_idx[out_base + rank] =
          winner == 0ull ? -1 : static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(winner));
      a.edge_score[out_base + rank] = winner == 0ull ? -INFINITY : last_score;
    }
  }
  if (lane == 0 && a.edge_flags != nullptr) {
    const int flagged = (best_dropped + a.exact_slack >= last_score) ? 1 : 0;
    a.edge_flags[item] = flagged;
    if (flagged && a.rescan_list != nullptr) {
      const int slot = atomicAdd(a.rescan_list, 1);
      a.rescan_list[1 + slot] = static_cast<int>(item);
    }
  }
}

// Exact top-m of the rows whose short list could not be proven complete, by a full
// scan of the row's keys.  256 threads per row: every thread scores the keys
// j = tid, tid + 256, ... in the fixed fp32 order and keeps its own sorted top-m; the
// 256 lists are then merged m times by a block-wide maximum.  CTAs take rows from the
// queue exact_edges_kernel filled (or, without a queue, poll every row's flag).
__global__ void __launch_bounds__(256) exact_rescan_kernel(const ckv_prefill_args a, int group) {
  __shared__ uint4 q_stage[8 * 16];
  __shared__ uint64_t lists[256 * kExactKeep];
  __shared__ uint64_t warp_best[8];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int length = a.seq_len;
  const int skip = a.num_sink + a.edges_per_row - 1;
  const int rows = length - skip;
  const int64_t total = static_cast<int64_t>(a.batch) * a.kv_heads * rows;
  const bool queued = a.rescan_list != nullptr;
  const int64_t work = queued ? a.rescan_list[0] : total;
  for (int64_t w = blockIdx.x; w < work; w += gridDim.x) {
    const int64_t item = queued ? a.rescan_list[1 + w] : w;
    if (!queued && a.edge_flags[item] == 0) {
      continue;
    }
    const int pos = skip + static_cast<int>(item % rows);
    const int kv_head = static_cast<int>((item / rows) % a.kv_heads);
    const int batch = static_cast<int>(item / (static_cast<int64_t>(rows) * a.kv_heads));
    const __nv_bfloat16* q_base = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                                  batch * a.q_batch_stride + static_cast<int64_t>(pos) * a.q_row_stride +
                                  kv_head * group * a.q_head_stride;
    const __nv_bfloat16* k_base = reinterpret_cast<const __nv_bfloat16*>(a.key) +
                                  batch * a.k_batch_stride + kv_head * a.k_head_stride;
    __syncthreads();  // the previous row's shared memory is no longer read
    for (int index = tid; index < group * 16; index += 256) {
      q_stage[index] = *reinterpret_cast<const uint4*>(q_base + (index >> 4) * a.q_head_stride +
                                                       (index & 15) * 8);
    }
    __syncthreads();
    uint64_t mine[kExactKeep];
#pragma unroll
    for (int k = 0; k < kExactKeep; ++k) {
      mine[k] = 0ull;
    }
    for (int j = a.num_sink + tid; j <= pos; j += 256) {
      const uint4* k_row = reinterpret_cast<const uint4*>(k_base + static_cast<int64_t>(j) * a.k_row_stride);
      uint4 k_reg[16];
#pragma unroll
      for (int piece = 0; piece < 16; ++piece) {
        k_reg[piece] = k_row[piece];
      }
      float score = -INFINITY;
      for (int g = 0; g < group; ++g) {
        float part[8];
#pragma unroll
        for (int piece = 0; piece < 8; ++piece) {
          const uint4 q0 = q_stage[g * 16 + 2 * piece];
          const uint4 q1 = q_stage[g * 16 + 2 * piece + 1];
          const uint4 k0 = k_reg[2 * piece];
          const uint4 k1 = k_reg[2 * piece + 1];
          float acc = 0.f;
          acc = fma2_bf16(k0.x, q0.x, acc);
          acc = fma2_bf16(k0.y, q0.y, acc);
          acc = fma2_bf16(k0.z, q0.z, acc);
          acc = fma2_bf16(k0.w, q0.w, acc);
          acc = fma2_bf16(k1.x, q1.x, acc);
          acc = fma2_bf16(k1.y, q1.y, acc);
          acc = fma2_bf16(k1.z, q1.z, acc);
          acc = fma2_bf16(k1.w, q1.w, acc);
          part[piece] = acc;
        }
        const float even = __fadd_rn(__fadd_rn(part[0], part[4]), __fadd_rn(part[2], part[6]));
        const float odd = __fadd_rn(__fadd_rn(part[1], part[5]), __fadd_rn(part[3], part[7]));
        score = fmaxf(score, __fmul_rn(__fadd_rn(even, odd), a.softmax_scale));
      }
      const uint64_t packed = (static_cast<uint64_t>(ordered_key32(score)) << 32) |
                              (0xffffffffu - static_cast<uint32_t>(j));
      if (packed > mine[kExactKeep - 1]) {
        queue_insert64(mine, packed);
      }
    }
#pragma unroll
    for (int k = 0; k < kExactKeep; ++k) {
      lists[tid * kExactKeep + k] = mine[k];
    }
    int head = 0;  // next unused entry of this thread's (sorted) list
    const int64_t out_base = item * a.edges_per_row;
    for (int rank = 0; rank < a.edges_per_row; ++rank) {
      const uint64_t offer = head < kExactKeep ? lists[tid * kExactKeep + head] : 0ull;
      const uint64_t best_in_warp = warp_max_u64(offer);
      if (lane == 0) {
        warp_best[warp] = best_in_warp;
      }
      __syncthreads();
      uint64_t winner = warp_best[0];
#pragma unroll
      for (int other = 1; other < 8; ++other) {
        winner = warp_best[other] > winner ? warp_best[other] : winner;
      }
      if (winner != 0ull && offer == winner) {
        head += 1;  // keys are distinct, so exactly one thread advances
      }
      if (tid == 0) {
        a.edge_idx[out_base + rank] =
            winner == 0ull ? -1 : static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(winner));
        a.edge_score[out_base + rank] =
            winner == 0ull ? -INFINITY : key32_to_float(static_cast<uint32_t>(winner >> 32));
      }
      __syncthreads();
    }
  }
}


// ---- candidate lists for the exact top-m, as a kernel of its own (G = 2 or 4) ----
//
// The exact edges rank keys by the maximum of the G heads' scores.  In the attention
// kernel above a row is one (position, head) pair, so that maximum needs a
// reduction across lanes for every key.  Here a row is a POSITION: the G heads of a
// KV head are G separate Q tiles (128 positions x 128 dims each) multiplied against
// the same K tile, their score tiles sit side by side in tensor memory, and the
// thread that owns a position reads the same columns of all G tiles and takes the
// maximum in registers.  No softmax, no P.V: half the tensor work of attention and a
// handful of CUDA-core instructions per key.
//
// 288 threads.  Warp 8 (one lane) is the producer: Q and K tiles by TMA, the
// tcgen05.mma chains, tcgen05.commit onto mbarriers.  Keys are processed in
// sub-blocks of 64; the two worker warpgroups (warps 0-3, 4-7) take even and odd
// sub-blocks, each with its own score buffer in tensor memory (G x 64 columns), so
// the tensor cores fill one buffer while the other is being read.  Every worker
// thread keeps the 16 best (score, key) pairs of its position and its sub-blocks in
// registers, plus the best score it turned away; the two threads of a position tell
// each other their 16th score through shared memory (the position's 16th best is at
// least the larger of the two, so anything clearly below it is turned away at once);
// the two lists go to the candidate array that exact_edges_kernel re-scores.
constexpr int kEdgeThreads = 288;
constexpr int kEdgeSub = 64;  // keys per sub-block

__device__ __forceinline__ uint32_t instruction_descriptor_n64() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((kEdgeSub >> 3) << 17) | ((kPfRows >> 4) << 24);
}

__device__ __forceinline__ void tmem_load16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// Insertion into a descending list by position: every slot decides from two comparisons
// whether it keeps its entry, takes the candidate or takes its left neighbour's entry, so
// the dependency chain is two operations deep whatever the length.  Returns what fell off
// the end (the candidate itself when it did not enter).
template <int kKeep>
__device__ __forceinline__ uint64_t list_insert(uint64_t (&list)[kKeep], uint64_t candidate) {
  bool keeps[kKeep];
#pragma unroll
  for (int k = 0; k < kKeep; ++k) {
    keeps[k] = list[k] >= candidate;
  }
  const uint64_t lost = keeps[kKeep - 1] ? candidate : list[kKeep - 1];
  uint64_t next[kKeep];
  next[0] = keeps[0] ? list[0] : candidate;
#pragma unroll
  for (int k = 1; k < kKeep; ++k) {
    next[k] = keeps[k] ? list[k] : (keeps[k - 1] ? candidate : list[k - 1]);
  }
#pragma unroll
  for (int k = 0; k < kKeep; ++k) {
    list[k] = next[k];
  }
  return lost;
}

struct EdgeSmem {
  static constexpr int kQ = 0;                       // kGroup tiles
  static constexpr int kBarBytes = 128 + 2 * kPfRows * 4;  // barriers, then the floors
  static constexpr int total(int group) { return (group + 2) * kTileBytes + kBarBytes; }
};

template <int kGroup>
__global__ void __launch_bounds__(kEdgeThreads, 1)
    edge_candidates_kernel(const ckv_prefill_args a, const __grid_constant__ CUtensorMap map_q,
                           const __grid_constant__ CUtensorMap map_k) {
  static_assert(kGroup == 2 || kGroup == 4, "two or four heads per KV head");
  constexpr int kKeep = kExactKeep;               // per thread; two threads per position
  constexpr int kBufferColumns = kGroup * kEdgeSub;  // tensor-memory columns of one score buffer
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* s_q = smem;
  uint8_t* s_k = smem + kGroup * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (kGroup + 2) * kTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile float* floors = reinterpret_cast<volatile float*>(bars + 16);  // [2][128]
  const uint32_t bar_q = smem_u32(bars);           // Q tiles landed
  const uint32_t bar_k_full = smem_u32(bars + 1);  // two: K buffer filled
  const uint32_t bar_k_free = smem_u32(bars + 3);  // two: every MMA reading the K buffer is done
  const uint32_t bar_s_full = smem_u32(bars + 5);  // two: score buffer written
  const uint32_t bar_s_free = smem_u32(bars + 7);  // two: score buffer read by its 128 workers

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int tile = gridDim.x - 1 - blockIdx.x;  // longest tiles first
  const int kv_head = blockIdx.y;
  const int batch = blockIdx.z;
  const int length = a.seq_len;
  const int pos0 = tile * kPfRows;
  const int last_pos = min(length, pos0 + kPfRows) - 1;
  const int key_blocks = last_pos / kPfKeys + 1;
  const int sub_total = last_pos / kEdgeSub + 1;

  if (tid < 2 * kPfRows) {
    floors[tid] = -INFINITY;
  }
  if (tid == 0) {
    mbar_init(bar_q, 1);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_k_full + 8 * i, 1);
      mbar_init(bar_k_free + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_s_free + 8 * i, 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  if (warp == 8) {
    // ---- producer: one lane ----
    if (tid == 256) {
      mbar_expect_tx(bar_q, kGroup * kTileBytes);
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        asm volatile(
            "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
            "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(smem_u32(s_q) + h * kTileBytes),
            "l"(&map_q), "r"(0), "r"(pos0), "r"(0), "r"(kv_head * kGroup + h), "r"(batch), "r"(bar_q)
            : "memory");
      }
      tma_load_tile(smem_u32(s_k), &map_k, bar_k_full, 0, kv_head, batch);
      if (key_blocks > 1) {
        tma_load_tile(smem_u32(s_k) + kTileBytes, &map_k, bar_k_full + 8, kPfKeys, kv_head, batch);
      }
      const uint32_t idesc = instruction_descriptor_n64();
      failed = !mbar_wait(bar_q, 0);
      for (int sb = 0; sb < sub_total && !failed; ++sb) {
        const int kb = sb >> 1;
        const int kbuf = kb & 1;
        const int sbuf = sb & 1;
        if ((sb & 1) == 0) {
          // tile kb+1 goes where tile kb-1 was, once the MMAs that read it are done
          if (kb >= 1 && kb + 1 < key_blocks) {
            if (!mbar_wait(bar_k_free + 8 * (kbuf ^ 1), ((kb - 1) >> 1) & 1)) {
              failed = true;
              break;
            }
            tma_load_tile(smem_u32(s_k) + (kbuf ^ 1) * kTileBytes, &map_k, bar_k_full + 8 * (kbuf ^ 1),
                          (kb + 1) * kPfKeys, kv_head, batch);
          }
          if (!mbar_wait(bar_k_full + 8 * kbuf, (kb >> 1) & 1)) {
            failed = true;
            break;
          }
        }
        if (sb >= 2 && !mbar_wait(bar_s_free + 8 * sbuf, ((sb >> 1) - 1) & 1)) {
          failed = true;
          break;
        }
        tc_fence_after();
        // keys [64 * (sb & 1), +64) of the K tile: rows are 16 bytes apart inside a chunk
        const uint32_t k_base = smem_u32(s_k) + kbuf * kTileBytes + (sb & 1) * kEdgeSub * 16;
#pragma unroll
        for (int h = 0; h < kGroup; ++h) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t desc_q =
                smem_descriptor(smem_u32(s_q) + h * kTileBytes + ks * 4096, 2048, 128);
            const uint64_t desc_k = smem_descriptor(k_base + ks * 4096, 2048, 128);
            umma(tmem + sbuf * kBufferColumns + h * kEdgeSub, desc_q, desc_k, idesc, ks > 0 ? 1u : 0u);
          }
        }
        umma_commit(bar_s_full + 8 * sbuf);
        if ((sb & 1) == 1 || sb == sub_total - 1) {
          umma_commit(bar_k_free + 8 * kbuf);
        }
      }
      if (failed && a.status != nullptr) {
        atomicOr(a.status, CKV_DEV_WAIT_TIMEOUT);
      }
    }
  } else {
    // ---- workers: warpgroup `wg` reads score buffer `wg` (sub-blocks wg, wg+2, ...) ----
    const int wg = warp >> 2;
    const int row = tid & (kPfRows - 1);
    const int row_pos = pos0 + row;
    const bool row_live = row_pos < length;
    const uint32_t lane_base = tmem + (((warp & 3) * 32u) << 16) + wg * kBufferColumns;
    uint64_t list[kKeep];
#pragma unroll
    for (int k = 0; k < kKeep; ++k) {
      list[k] = 0ull;
    }
    float dropped = -INFINITY;
    for (int sb = wg; sb < sub_total; sb += 2) {
      if (!mbar_wait(bar_s_full + 8 * wg, (sb >> 1) & 1)) {
        failed = true;
        break;
      }
      tc_fence_after();
      const int key0 = sb * kEdgeSub;
      const bool plain = key0 + kEdgeSub - 1 <= pos0 && key0 >= a.num_sink;  // no mask, no sinks
      const uint64_t last = list[kKeep - 1];
      const float own_floor =
          last == 0ull ? -INFINITY : key32_to_float(static_cast<uint32_t>(last >> 32));
      floors[wg * kPfRows + row] = own_floor;
      // the other list's 16th score, a little low (any earlier value is also valid)
      const float partner_floor = floors[(wg ^ 1) * kPfRows + row] - 2.0f * a.exact_slack;
      float floor_score = fmaxf(own_floor, partner_floor);
      // the next chunk's scores are requested before this chunk's list work and waited
      // for after it
      uint32_t raw[kGroup][16];
#pragma unroll
      for (int h = 0; h < kGroup; ++h) {
        tmem_load16_issue(lane_base + h * kEdgeSub, raw[h]);
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < kEdgeSub; c0 += 16) {
        float best[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float m = __uint_as_float(raw[0][i]);
#pragma unroll
          for (int h = 1; h < kGroup; ++h) {
            m = fmaxf(m, __uint_as_float(raw[h][i]));
          }
          const int j = key0 + c0 + i;
          const bool visible = plain || (j <= row_pos && j >= a.num_sink);
          best[i] = visible ? m * a.softmax_scale : -INFINITY;
        }
        if (c0 + 16 < kEdgeSub) {
#pragma unroll
          for (int h = 0; h < kGroup; ++h) {
            tmem_load16_issue(lane_base + h * kEdgeSub + c0 + 16, raw[h]);
          }
        }
        // Columns that beat the floor, as a bit mask.  The lanes then insert in
        // rounds: in every round each lane that still has such a column inserts its
        // next one, so a chunk costs as many passes over the insertion code as the
        // busiest lane has columns, not as many as there are columns with a taker.
        uint32_t takers = 0u;
        float rejected = -INFINITY;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool take = row_live && best[i] > floor_score;
          takers |= (take ? 1u : 0u) << i;
          rejected = fmaxf(rejected, take ? -INFINITY : best[i]);
        }
        dropped = fmaxf(dropped, rejected);
        while (__any_sync(0xffffffffu, takers != 0u)) {
          if (takers != 0u) {
            const int i = __ffs(takers) - 1;
            takers &= takers - 1;
            // the column's score by a binary tree over the index bits (four selects deep)
            float pick[8];
#pragma unroll
            for (int m = 0; m < 8; ++m) pick[m] = (i & 1) ? best[2 * m + 1] : best[2 * m];
#pragma unroll
            for (int m = 0; m < 4; ++m) pick[m] = (i & 2) ? pick[2 * m + 1] : pick[2 * m];
#pragma unroll
            for (int m = 0; m < 2; ++m) pick[m] = (i & 4) ? pick[2 * m + 1] : pick[2 * m];
            const float v = (i & 8) ? pick[1] : pick[0];
            if (v > floor_score) {
              const uint64_t candidate = (static_cast<uint64_t>(ordered_key32(v)) << 32) |
                                         (0xffffffffu - static_cast<uint32_t>(key0 + c0 + i));
              const uint64_t lost = list_insert<kKeep>(list, candidate);
              if (lost != 0ull) {
                dropped = fmaxf(dropped, key32_to_float(static_cast<uint32_t>(lost >> 32)));
              }
              const uint64_t tail = list[kKeep - 1];
              floor_score = fmaxf(
                  partner_floor,
                  tail == 0ull ? -INFINITY : key32_to_float(static_cast<uint32_t>(tail >> 32)));
            } else {
              dropped = fmaxf(dropped, v);
            }
          }
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      tc_fence_before();
      mbar_arrive(bar_s_free + 8 * wg);
    }
    if (row_live && !failed) {
      // [batch, kv head, position, G lanes, 16 kept + best dropped]: this thread's list
      // is lane `wg` (the other lanes stay empty)
      uint64_t* out = a.candidates +
                      ((static_cast<int64_t>(batch) * gridDim.y + kv_head) * length + row_pos) *
                          kGroup * (kExactKeep + 1);
#pragma unroll
      for (int k = 0; k < kKeep; ++k) {
        out[wg * (kExactKeep + 1) + k] = list[k];
      }
      out[wg * (kExactKeep + 1) + kExactKeep] =
          dropped != -INFINITY ? static_cast<uint64_t>(ordered_key32(dropped)) << 32 : 0ull;
    }
    if (failed && a.status != nullptr) {
      atomicOr(a.status, CKV_DEV_WAIT_TIMEOUT);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512)
                 : "memory");
  }
}

namespace {

// The driver's tensor-map encoder, looked up through the runtime so that the
// library does not link against the driver library.
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 encoder = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) !=
            cudaSuccess ||
        found != cudaDriverEntryPointSuccess) {
      entry = nullptr;
    }
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(entry);
  }();
  return encoder;
}

}  // namespace

// K or V [batch, rows, kv heads, 128] bf16 seen as (8 elements, rows, 16 chunks of
// 16 bytes, kv heads, batch): one box of (8, 128, 16, 1, 1) lands in shared memory as
// 16 chunks of 128 rows x 16 bytes, which is the tensor-core operand layout.
bool tile_map(CUtensorMap* map, const void* base, const ckv_prefill_args& a, int heads,
              int64_t row_stride, int64_t head_stride, int64_t batch_stride, bool swizzled) {
  const auto encoder = tensor_map_encoder();
  if (encoder == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    return false;
  }
  const uint64_t row_bytes = static_cast<uint64_t>(row_stride) * 2;
  // a dimension of extent 1 never uses its stride; give it a legal one
  const uint64_t head_bytes =
      heads > 1 ? static_cast<uint64_t>(head_stride) * 2 : static_cast<uint64_t>(kHeadDim) * 2;
  const uint64_t batch_bytes =
      a.batch > 1 ? static_cast<uint64_t>(batch_stride) * 2 : row_bytes * static_cast<uint64_t>(a.seq_len);
  if (row_stride <= 0 || (row_bytes & 15u) || (head_bytes & 15u) || (batch_bytes & 15u)) {
    return false;
  }
  const cuuint32_t inner = swizzled ? 64 : 8;  // elements per row piece: 128 or 16 bytes
  const cuuint64_t extent[5] = {inner, static_cast<cuuint64_t>(a.seq_len), 128 / inner,
                                static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(a.batch)};
  const cuuint64_t strides[4] = {row_bytes, inner * 2, head_bytes, batch_bytes};
  const cuuint32_t box[5] = {inner, kPfKeys, 128 / inner, 1, 1};
  const cuuint32_t steps[5] = {1, 1, 1, 1, 1};
  return encoder(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), extent, strides,
                 box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

template <int kGroup>
cudaError_t launch_for_group(const ckv_prefill_args& a, cudaStream_t stream) {
  if constexpr (kGroup % 2 == 0) {
    // attention alone or with the top-8 rule: two heads of the group per CTA
    if (a.mode != 2) return launch_prefill_pair(a, stream);
  }
  constexpr int kSmem = PrefillSmem::kTotal;
  const dim3 grid((a.seq_len + kPfRows / kGroup - 1) / (kPfRows / kGroup), a.kv_heads, a.batch);
  CUtensorMap map_k, map_v;
  if (!tile_map(&map_k, a.key, a, a.kv_heads, a.k_row_stride, a.k_head_stride, a.k_batch_stride) ||
      !tile_map(&map_v, a.value, a, a.kv_heads, a.v_row_stride, a.v_head_stride, a.v_batch_stride)) {
    return cudaErrorInvalidValue;
  }
  auto run = [&](auto kernel) -> cudaError_t {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (err != cudaSuccess) return err;
    kernel<<<grid, kPfThreads, kSmem, stream>>>(a, map_k, map_v);
    return cudaGetLastError();
  };
  if (a.mode == 0) return run(prefill_kernel<kGroup, 0>);
  if (a.mode == 1) return run(prefill_kernel<kGroup, 1>);
  return run(prefill_kernel<kGroup, 2>);
}

}  // namespace

// Exact edges with two or four heads per KV head: attention by itself, then the
// candidate lists from the position-per-row kernel.
template <int kGroup>
cudaError_t launch_candidates(const ckv_prefill_args& a, cudaStream_t stream) {
  ckv_prefill_args attention = a;
  attention.mode = 0;
  cudaError_t err = launch_for_group<kGroup>(attention, stream);
  if (err != cudaSuccess) return err;
  CUtensorMap map_q, map_k;
  if (!tile_map(&map_q, a.query, a, a.query_heads, a.q_row_stride, a.q_head_stride, a.q_batch_stride) ||
      !tile_map(&map_k, a.key, a, a.kv_heads, a.k_row_stride, a.k_head_stride, a.k_batch_stride)) {
    return cudaErrorInvalidValue;
  }
  constexpr int kSmem = EdgeSmem::total(kGroup);
  err = cudaFuncSetAttribute(edge_candidates_kernel<kGroup>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (err != cudaSuccess) return err;
  const dim3 grid((a.seq_len + kPfRows - 1) / kPfRows, a.kv_heads, a.batch);
  edge_candidates_kernel<kGroup><<<grid, kEdgeThreads, kSmem, stream>>>(a, map_q, map_k);
  return cudaGetLastError();
}

cudaError_t launch_prefill(const ckv_prefill_args& a, cudaStream_t stream) {
  const int group = a.query_heads / a.kv_heads;
  cudaError_t err;
  if (a.mode == 2 && (group == 2 || group == 4)) {
    err = group == 2 ? launch_candidates<2>(a, stream) : launch_candidates<4>(a, stream);
  } else
  switch (group) {
    case 1: err = launch_for_group<1>(a, stream); break;
    case 2: err = launch_for_group<2>(a, stream); break;
    case 4: err = launch_for_group<4>(a, stream); break;
    case 8: err = launch_for_group<8>(a, stream); break;
    default: return cudaErrorInvalidValue;
  }
  if (err != cudaSuccess || a.mode != 2) {
    return err;
  }
  const int rows = a.seq_len - (a.num_sink + a.edges_per_row - 1);
  if (rows <= 0) {
    return cudaSuccess;
  }
  const int64_t items = static_cast<int64_t>(a.batch) * a.kv_heads * rows;
  exact_edges_kernel<<<static_cast<unsigned>((items + 3) / 4), 128, 0, stream>>>(a, group);
  err = cudaGetLastError();
  if (err != cudaSuccess || a.edge_flags == nullptr) {
    return err;
  }
  const long long rescan_grid = a.rescan_list != nullptr ? (items < 148 * 4 ? items : 148 * 4) : items;
  exact_rescan_kernel<<<static_cast<unsigned>(rescan_grid), 256, 0, stream>>>(a, group);
  return cudaGetLastError();
}

}  // namespace ckv
