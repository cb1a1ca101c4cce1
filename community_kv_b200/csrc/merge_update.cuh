// Device function of the split merge and the online graph update, shared by the
// stand-alone kernel and the fused per-layer cluster kernel (sm_100a).
#pragma once

#include "ckv_device.cuh"

namespace ckv {

constexpr int kMergeThreads = 128;
constexpr int kMaxSplitsInFlight = 8;  // split rows a merging lane fetches at once

struct UpdateDecision {
  int assigned;      // community id the new token joins (clamped to capacity-1)
  int old_size;      // size of that community before the update
  int current;       // cache row of the new token
  int apply;         // 1 when sizes/centroid/labels are to be written
  int valid_position;
  int candidates[kKappa + 1];  // communities the token may join (-1: none), known before the decision
};

// Polls this GPU's arrival counter until the peers' head outputs of this call are
// here (one thread, bounded, system-scope acquire), then takes the count back off.
__device__ __forceinline__ void wait_for_peer_rows(const ckv_layer_args& a) {
  if (a.peer_wait_flag == nullptr || a.peer_wait_expected <= 0 || threadIdx.x != 0) {
    return;
  }
  const uint32_t expected = static_cast<uint32_t>(a.peer_wait_expected);
  constexpr uint32_t kPolls = 1u << 22;  // about two seconds with the back-off below
  for (uint32_t poll = 0; poll < kPolls; ++poll) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.peer_wait_flag) : "memory");
    if (seen >= expected) {
      atomicSub(a.peer_wait_flag, expected);
      return;
    }
    if (poll > 256) {
      __nanosleep(500);
    }
  }
  if (a.status != nullptr) {
    atomicOr(a.status, CKV_DEV_WAIT_TIMEOUT);
  }
}

// Warps 0 .. merge_warps-1 merge the split partials; warp `merge_warps` is the update
// warp: it merges the neighbour candidates and fetches everything the online
// assignment needs while the other warps are still merging, then applies the
// assignment once the first head's log-sum-exp is known.  The CTA has at least
// 128 threads and (merge_warps + 1) warps; `decision` and `lse_s` live in shared
// memory.  Partials are read past the L1 cache: in the fused kernel other CTAs of
// the cluster have just written them.
__device__ __forceinline__ void merge_update_unit(const ckv_layer_args& a, int flat, int merge_warps,
                                                  UpdateDecision& decision, float& lse_s) {
  const Unit u = make_unit(a, flat);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = a.group_size;
  const int splits = a.splits;
  const int capacity = a.community_capacity;
  const bool leader = u.head == u.graph && !(a.flags & CKV_FLAG_SKIP_UPDATE);
  const int64_t graph_slot = static_cast<int64_t>(u.batch) * a.graphs + u.graph;
  // partial rows: dense [unit][split][head][132] unless the caller gives strides
  const int64_t split_stride =
      a.partial_split_stride > 0 ? a.partial_split_stride : static_cast<int64_t>(group) * kPartialStride;
  const int64_t unit_stride = a.partial_unit_stride > 0 ? a.partial_unit_stride : splits * split_stride;
  const float* partial = a.partials + static_cast<int64_t>(flat) * unit_stride;

  // state of the update warp that crosses the barrier
  float my_score = 0.f;
  int my_position = -1;
  int community = -1;
  bool valid = false;
  int active = 0;
  float old_total = 0.f;
  float old_weight = 0.f;
  int current = 0;
  // Graph state of the community this lane's neighbour belongs to (lanes 0-7) or of
  // the next unused community id (lane 8), fetched before the assignment is known:
  // one of these nine is the community the new token will join.
  int spec_community = -1;
  int spec_size = 0, spec_delta = 0, spec_tail = -1;
  int spec_chunk_size = 0, spec_chunk_capacity = 0, spec_chunk_start = 0;
  int free_chunk = 0, free_position = 0;
  // key element of the new token, fetched early by the merging threads
  float key_value = 0.f;

  const bool update_only = (a.flags & CKV_FLAG_UPDATE_ONLY) != 0;
  if (threadIdx.x < kHeadDim && leader) {
    {
      const int position = a.current_position[graph_slot];
      if (a.current_key != nullptr) {
        // [batch, R, 128]: the new token's key for this retrieval head's KV head
        const __nv_bfloat16* key_row = reinterpret_cast<const __nv_bfloat16*>(a.current_key) +
                                       static_cast<int64_t>(flat) * kHeadDim;
        key_value = __bfloat162float(key_row[threadIdx.x]);
      } else if (position >= 0 && position < a.sequence_capacity) {
        const __nv_bfloat16* key_row = reinterpret_cast<const __nv_bfloat16*>(a.key) +
                                       u.batch * a.key_batch_stride + u.kv * a.key_head_stride +
                                       static_cast<int64_t>(position) * a.key_row_stride;
        key_value = __bfloat162float(key_row[threadIdx.x]);
      }
    }
  }
  if (warp < merge_warps) {
    if (update_only) {
      if (threadIdx.x == 0) {
        lse_s = a.lse[static_cast<int64_t>(flat) * group];
      }
    }
    // ---- split merge: warp w takes heads w, w+4, ...; lane s reads split s's
    // (max, sum) pair, every lane then accumulates four output dimensions with
    // independent 16-byte loads ----
    __nv_bfloat16* output = reinterpret_cast<__nv_bfloat16*>(a.output) +
                            static_cast<int64_t>(flat) * group * kHeadDim;
    for (int g = warp; g < group && !update_only; g += merge_warps) {
      // the accumulator rows do not depend on the (max, sum) pairs: fetch both at once
      float4 rows[kMaxSplitsInFlight];
#pragma unroll
      for (int s = 0; s < kMaxSplitsInFlight; ++s) {
        if (s < splits) {
          rows[s] = __ldcg(reinterpret_cast<const float4*>(
              partial + s * split_stride + g * kPartialStride + 4 * lane));
        }
      }
      float my_max = -INFINITY;
      float my_sum = 0.f;
      if (lane < splits) {
        const float2 pair = __ldcg(reinterpret_cast<const float2*>(
            partial + lane * split_stride + g * kPartialStride + kHeadDim));
        my_max = pair.x;
        my_sum = pair.y;
      }
      float best = my_max;
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, offset));
      }
      const float safe = best == -INFINITY ? 0.f : best;
      const float weight = exp2f((my_max - safe) * kLog2e);  // 0 for lanes >= splits
      float denominator = my_sum * weight;
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        denominator += __shfl_xor_sync(0xffffffffu, denominator, offset);
      }
      float4 numerator = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s = 0; s < kMaxSplitsInFlight; ++s) {
        if (s < splits) {
          const float w = __shfl_sync(0xffffffffu, weight, s);
          numerator.x += rows[s].x * w;
          numerator.y += rows[s].y * w;
          numerator.z += rows[s].z * w;
          numerator.w += rows[s].w * w;
        }
      }
      for (int s = kMaxSplitsInFlight; s < splits; ++s) {
        const float w = __shfl_sync(0xffffffffu, weight, s);
        const float4 v = __ldcg(reinterpret_cast<const float4*>(
            partial + s * split_stride + g * kPartialStride + 4 * lane));
        numerator.x += v.x * w;
        numerator.y += v.y * w;
        numerator.z += v.z * w;
        numerator.w += v.w * w;
      }
      if (a.merged != nullptr) {
        float* row = a.merged + (static_cast<int64_t>(flat) * group + g) * kPartialStride;
        *reinterpret_cast<float4*>(row + 4 * lane) = numerator;
        if (lane == 0) {
          row[kHeadDim] = best;
          row[kHeadDim + 1] = denominator;
        }
      }
      const __nv_bfloat162 lo =
          __floats2bfloat162_rn(numerator.x / denominator, numerator.y / denominator);
      const __nv_bfloat162 hi =
          __floats2bfloat162_rn(numerator.z / denominator, numerator.w / denominator);
      uint2 packed;
      packed.x = *reinterpret_cast<const uint32_t*>(&lo);
      packed.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(output + g * kHeadDim + 4 * lane) = packed;
      // the same row, straight into every peer GPU's gathered tensor
      for (int p = 0; p < a.peer_count; ++p) {
        __nv_bfloat16* remote = reinterpret_cast<__nv_bfloat16*>(a.peer_output[p]) +
                                static_cast<int64_t>(flat) * group * kHeadDim;
        *reinterpret_cast<uint2*>(remote + g * kHeadDim + 4 * lane) = packed;
      }
      const float lse = best + logf(denominator);
      if (lane == 0) {
        a.lse[static_cast<int64_t>(flat) * group + g] = lse;
        if (g == 0) {
          lse_s = lse;
        }
      }
    }
  } else if (warp == merge_warps) {
    // ---- update warp, before the barrier: global top-8 of the per-split
    // candidates (every head reports it) and the loads that depend only on it ----
    const int64_t topk_split = a.topk_split_stride > 0 ? a.topk_split_stride : kKappa;
    const int64_t topk_unit = a.topk_unit_stride > 0 ? a.topk_unit_stride : splits * topk_split;
    const uint64_t* candidates = a.partial_topk + static_cast<int64_t>(flat) * topk_unit;
    const int total = splits * kKappa;
    uint64_t mine[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int index = lane + 32 * i;
      mine[i] = (index < total && !update_only)
                    ? __ldcg(candidates + (index / kKappa) * topk_split + (index % kKappa))
                    : 0ull;
    }
    if (leader) {
      active = a.community_counts[flat];
      old_total = a.total_weight[graph_slot];
      current = a.current_position[graph_slot];
      free_chunk = a.next_free_chunk[graph_slot];
      free_position = a.next_free_position[graph_slot];
    }
    // eight rounds of "warp-wide maximum, then retire it"; only the registers that hold
    // candidates take part (two of the eight with up to eight splits)
    for (int k = 0; k < kKappa && !update_only; ++k) {
      uint64_t local = 0ull;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (32 * i < total) {
          local = mine[i] > local ? mine[i] : local;
        }
      }
      const uint64_t best = warp_max_u64(local);
      if (best != 0ull) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (32 * i < total) {
            mine[i] = mine[i] == best ? 0ull : mine[i];
          }
        }
      }
      if (lane == k) {
        my_score = key32_to_float(static_cast<uint32_t>(best >> 32));
        my_position = static_cast<int>(0xffffffffu - static_cast<uint32_t>(best));
        if (a.merged_topk != nullptr) {
          a.merged_topk[static_cast<int64_t>(flat) * kKappa + k] = best;
        }
      }
    }
    if (update_only) {
      if (lane < kKappa) {
        my_score = a.topk_scores[static_cast<int64_t>(flat) * kKappa + lane];
        my_position = a.topk_positions[static_cast<int64_t>(flat) * kKappa + lane];
      }
    } else if (lane < kKappa) {
      a.topk_scores[static_cast<int64_t>(flat) * kKappa + lane] = my_score;
      a.topk_positions[static_cast<int64_t>(flat) * kKappa + lane] = my_position;
    }
    if (leader) {
      valid = lane < kKappa && my_position >= 0 && my_position < a.sequence_capacity;
      if (valid && my_position < a.token_capacity) {
        community = a.token_communities[graph_slot * a.token_capacity + my_position];
      }
      if (valid && community >= 0 && community < capacity) {
        old_weight = a.community_weight[graph_slot * capacity + community];
      }
      spec_community = lane < kKappa ? community : (lane == kKappa ? active : -1);
      if (spec_community >= 0 && spec_community < capacity) {
        const int64_t table = graph_slot * capacity + spec_community;
        spec_size = a.community_sizes[static_cast<int64_t>(flat) * capacity + spec_community];
        spec_delta = a.delta_sizes[table];
        spec_tail = a.community_tail[table];
        if (spec_tail >= 0) {
          const int64_t chunk_base = graph_slot * a.chunks_per_graph;
          spec_chunk_size = a.chunk_size[chunk_base + spec_tail];
          spec_chunk_capacity = a.chunk_capacity[chunk_base + spec_tail];
          spec_chunk_start = a.chunk_start[chunk_base + spec_tail];
        }
      } else {
        spec_community = -1;
      }
    }
    if (lane <= kKappa) {
      decision.candidates[lane] = spec_community;
    }
  }
  __syncthreads();
  if (a.peer_count > 0 && threadIdx.x == 0 && !update_only) {
    // All output rows of this unit were stored before the barrier.  With a local counter
    // (peer_done) a unit only has to order its stores before its count at GPU scope; the
    // last unit of the call, which has observed every other unit's count, then issues ONE
    // system-scope fence (fences are cumulative: it covers the other units' stores too)
    // and signals every peer with relaxed remote adds, which it does not wait for.
    bool signal = true;
    if (a.peer_done != nullptr) {
      __threadfence();
      const uint32_t units = static_cast<uint32_t>(a.batch * a.retrieval_heads);
      const uint32_t before = atomicAdd(a.peer_done, 1u);
      signal = before == units - 1;
      if (signal) {
        atomicExch(a.peer_done, 0u);
      }
    }
    if (signal) {
      __threadfence_system();
      for (int p = 0; p < a.peer_count; ++p) {
        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.peer_flag[p]) : "memory");
      }
    }
  }
  // Centroid bytes of every community the token may join, fetched while the update
  // warp decides: the running-mean update below then needs no further round trip.
  uint8_t centroid_byte[kKappa + 1];
  if (leader && threadIdx.x < kHeadDim) {
    const uint8_t* table = reinterpret_cast<const uint8_t*>(a.centroids) +
                           static_cast<int64_t>(flat) * capacity * kHeadDim + threadIdx.x;
#pragma unroll
    for (int j = 0; j <= kKappa; ++j) {
      const int c = decision.candidates[j];
      centroid_byte[j] = c >= 0 ? table[static_cast<int64_t>(c) * kHeadDim] : 0;
    }
  }

  if (warp == merge_warps && leader) {
    // lanes 0..7 hold rank `lane`; sums run over the ranks in order on every lane
    const float representative_lse = lse_s;
    const float score = valid ? expf(__fsub_rn(my_score, representative_lse)) : 0.f;
    const float direct = __fmul_rn(score, __fmul_rn(a.lam, 0.5f));
    float node_degree = 0.f, score_sum = 0.f, square_sum = 0.f;
    for (int k = 0; k < kKappa; ++k) {
      const float dk = __shfl_sync(0xffffffffu, direct, k);
      const float sk = __shfl_sync(0xffffffffu, score, k);
      node_degree = __fadd_rn(node_degree, dk);
      score_sum = __fadd_rn(score_sum, sk);
      square_sum = __fadd_rn(square_sum, __fmul_rn(sk, sk));
    }
    const float pair_weight =
        __fmul_rn(__fsub_rn(__fmul_rn(score_sum, score_sum), square_sum),
                  __fmul_rn(0.5f, __fsub_rn(1.0f, a.lam)));
    const bool candidate = valid && community >= 0 && community < active;
    float candidate_weight = 0.f;
    int first_rank = kKappa;
    for (int k = 0; k < kKappa; ++k) {
      const int ck = __shfl_sync(0xffffffffu, community, k);
      const int cand_k = __shfl_sync(0xffffffffu, candidate ? 1 : 0, k);
      const float dk = __shfl_sync(0xffffffffu, direct, k);
      if (cand_k && ck == community) {
        candidate_weight = __fadd_rn(candidate_weight, dk);
        first_rank = min(first_rank, k);
      }
    }
    const bool rank_leader = candidate && first_rank == lane;
    const float two_m = fmaxf(__fmul_rn(2.0f, old_total), 1.0f);
    float delta_q = -INFINITY;
    if (candidate && candidate_weight > 0.f) {
      delta_q = __fsub_rn(candidate_weight, __fdiv_rn(__fmul_rn(node_degree, old_weight), two_m));
    }
    float best_delta = delta_q;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      best_delta = fmaxf(best_delta, __shfl_xor_sync(0xffffffffu, best_delta, offset));
    }
    int best_community = (candidate && delta_q == best_delta) ? community : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      best_community = min(best_community, __shfl_xor_sync(0xffffffffu, best_community, offset));
    }
    bool join = best_delta > 0.f;
    int assigned = join ? best_community : active;
    if (a.forced_community != nullptr) {
      // the caller's choice (nearest-centroid variant) replaces the rule's, if it is a live community
      const int forced = a.forced_community[graph_slot];
      if (forced >= 0 && forced < active) {
        join = true;
        assigned = forced;
      }
    }
    const bool community_overflow = assigned >= capacity;
    const int safe_assigned = min(max(assigned, 0), capacity - 1);

    if (!community_overflow && rank_leader) {
      float increment = candidate_weight;
      if (join && community == safe_assigned) {
        increment = __fadd_rn(increment, node_degree);
      }
      a.community_weight[graph_slot * capacity + community] = __fadd_rn(old_weight, increment);
    }
    __syncwarp();
    // the lane that fetched the chosen community's state hands it to lane 0
    const unsigned holders = __ballot_sync(0xffffffffu, spec_community == safe_assigned);
    const int holder = holders ? __ffs(holders) - 1 : 0;
    const bool fetched = holders != 0u && !community_overflow;
    const int got_size = __shfl_sync(0xffffffffu, spec_size, holder);
    const int got_delta = __shfl_sync(0xffffffffu, spec_delta, holder);
    const int got_tail = __shfl_sync(0xffffffffu, spec_tail, holder);
    const int got_chunk_size = __shfl_sync(0xffffffffu, spec_chunk_size, holder);
    const int got_chunk_capacity = __shfl_sync(0xffffffffu, spec_chunk_capacity, holder);
    const int got_chunk_start = __shfl_sync(0xffffffffu, spec_chunk_start, holder);
    if (lane == 0) {
      if (!community_overflow) {
        if (!join) {
          a.community_weight[graph_slot * capacity + safe_assigned] = node_degree;
        }
        a.community_counts[flat] = active + (join ? 0 : 1);
        a.total_weight[graph_slot] = __fadd_rn(__fadd_rn(old_total, node_degree), pair_weight);
      }
      a.assigned[graph_slot] = community_overflow ? -1 : assigned;

      const bool valid_position = current >= 0 && current < a.sequence_capacity;
      bool chunk_overflow = false;
      bool position_overflow = false;
      int old_size = 0;
      if (!community_overflow) {
        const int64_t table = graph_slot * capacity + safe_assigned;
        const int64_t chunk_base = graph_slot * a.chunks_per_graph;
        // normally already in registers (fetched before the decision)
        old_size = fetched ? got_size
                           : a.community_sizes[static_cast<int64_t>(flat) * capacity + safe_assigned];
        const int delta_size = fetched ? got_delta : a.delta_sizes[table];
        const int old_tail = fetched ? got_tail : a.community_tail[table];
        a.community_sizes[static_cast<int64_t>(flat) * capacity + safe_assigned] = old_size + 1;
        if (valid_position && current < a.token_capacity) {
          a.token_communities[graph_slot * a.token_capacity + current] = assigned;
        }
        int old_chunk_size = 0, old_chunk_capacity = 0, old_chunk_start = 0;
        if (old_tail >= 0) {
          old_chunk_size = fetched ? got_chunk_size : a.chunk_size[chunk_base + old_tail];
          old_chunk_capacity = fetched ? got_chunk_capacity : a.chunk_capacity[chunk_base + old_tail];
          old_chunk_start = fetched ? got_chunk_start : a.chunk_start[chunk_base + old_tail];
        }
        const bool allocate = old_tail < 0 || old_chunk_size >= old_chunk_capacity;
        const int new_capacity = old_tail < 0 ? 1 : old_chunk_capacity * 2;
        chunk_overflow = allocate && free_chunk >= a.chunks_per_graph;
        position_overflow = allocate && free_position + new_capacity > a.delta_position_capacity;
        const bool allocation_overflow = chunk_overflow || position_overflow;
        const int chunk = allocate ? free_chunk : old_tail;
        const bool valid_chunk = !allocation_overflow && chunk >= 0 && chunk < a.chunks_per_graph;
        if (allocate && !allocation_overflow) {
          a.next_free_chunk[graph_slot] = free_chunk + 1;
          a.next_free_position[graph_slot] = free_position + new_capacity;
          a.chunk_start[chunk_base + free_chunk] = free_position;
          a.chunk_capacity[chunk_base + free_chunk] = new_capacity;
          a.chunk_previous[chunk_base + free_chunk] = old_tail;
          if (old_tail < 0) {
            a.community_head[table] = free_chunk;
          } else {
            a.chunk_next[chunk_base + old_tail] = free_chunk;
          }
          a.community_tail[table] = free_chunk;
        }
        if (valid_chunk && valid_position) {
          const int target_start = allocate ? free_position : old_chunk_start;
          const int target_slot = allocate ? 0 : old_chunk_size;
          a.delta_positions[graph_slot * a.delta_position_capacity + target_start + target_slot] =
              current;
          a.chunk_size[chunk_base + chunk] = target_slot + 1;
          a.delta_sizes[table] = delta_size + 1;
        }
      }
      const int overflow = (community_overflow ? 1 : 0) | (chunk_overflow ? 2 : 0) |
                           (position_overflow ? 4 : 0) | (valid_position ? 0 : 8);
      a.overflow[graph_slot] = overflow;
      if (overflow == 0) {
        a.current_position[graph_slot] = current + 1;
      }
      decision.assigned = safe_assigned;
      decision.old_size = old_size;
      decision.current = current;
      decision.apply = community_overflow ? 0 : 1;
      decision.valid_position = valid_position ? 1 : 0;
    }
  }
  if (!leader) {
    return;
  }
  __syncthreads();
  // ---- running centroid: fp32 mean stored back as saturating e4m3 ----
  if (threadIdx.x < kHeadDim && decision.apply && decision.valid_position &&
      (a.flags & CKV_FLAG_FP32_CENTROIDS)) {
    // fp32 table: the running mean is stored as it is
    float* centroid = reinterpret_cast<float*>(a.centroids) +
                      (static_cast<int64_t>(flat) * capacity + decision.assigned) * kHeadDim + threadIdx.x;
    *centroid = decision.old_size > 0
                    ? centroid_mean(*centroid, decision.old_size, key_value,
                                    (a.flags & CKV_FLAG_REFERENCE_DIVISION) != 0)
                    : key_value;
  } else if (threadIdx.x < kHeadDim && decision.apply && decision.valid_position) {
    const int d = threadIdx.x;
    __nv_fp8_storage_t* centroid =
        reinterpret_cast<__nv_fp8_storage_t*>(a.centroids) +
        (static_cast<int64_t>(flat) * capacity + decision.assigned) * kHeadDim;
    float updated = key_value;
    if (decision.old_size > 0) {
      uint8_t stored = 0;
      bool have = false;
#pragma unroll
      for (int j = 0; j <= kKappa; ++j) {
        if (!have && decision.candidates[j] == decision.assigned) {
          stored = centroid_byte[j];
          have = true;
        }
      }
      if (!have) {
        stored = centroid[d];
      }
      const __half_raw raw = __nv_cvt_fp8_to_halfraw(stored, __NV_E4M3);
      const float old_value = __half2float(*reinterpret_cast<const __half*>(&raw));
      updated = centroid_mean(old_value, decision.old_size, key_value,
                              (a.flags & CKV_FLAG_REFERENCE_DIVISION) != 0);
    }
    centroid[d] = __nv_cvt_float_to_fp8(updated, __NV_SATFINITE, __NV_E4M3);
  }
}

}  // namespace ckv
