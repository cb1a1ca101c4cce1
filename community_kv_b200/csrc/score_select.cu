// Centroid scoring and exact budgeted community selection (sm_100a).
//
// score_kernel:  scores[b,r,c] = fp16(max over the query group of q . centroid[c]).
//   HBM-bound scan of the e4m3 centroid table (128 B per community).  Eight lanes
//   share one centroid row (16 B each, so a warp reads 512 contiguous bytes per
//   load), every lane keeps four rows in flight, and the 128-long dot product is
//   accumulated in fp32 in one fixed order so that the fp16 result - and with it
//   the selection - is reproducible bit for bit on a CPU.
//
// select_kernel: one CTA per (sequence, retrieval head).  Two weighted 256-bin
//   histograms over the order-preserving 16-bit key give the threshold, an
//   index-ordered block scan compacts the descriptors, and the same CTA then
//   resolves every logical token of the budget to its cache row.

#include "ckv_device.cuh"

namespace ckv {

constexpr int kScoreThreads = 256;
constexpr int kSelectThreads = 1024;
constexpr int kStash = 4608;  // communities whose keys/sizes are staged in shared memory
constexpr int kDescStash = 2048;  // descriptors kept in shared memory for the position search

// Work is counted in 16-row groups.  The groups of all units of the launch are
// laid end to end and every CTA takes an equal contiguous share, so units with
// many communities do not become stragglers.  Inside its share a CTA's eight
// warps stride over the groups and keep the next group's loads in flight while
// they compute the current one.
constexpr int kScoreMaxUnits = 4096;  // units whose group counts fit the shared prefix table

__device__ __forceinline__ void load_group(const uint8_t* table, int row_base, int quad, int slice,
                                           int capacity, uint4 (&raw)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = min(row_base + quad + 4 * i, capacity - 1);
    raw[i] = __ldg(reinterpret_cast<const uint4*>(table + static_cast<int64_t>(row) * kHeadDim) + slice);
  }
}

__device__ __forceinline__ int score_limit(const ckv_layer_args& a, int flat) {
  const int capacity = a.community_capacity;
  if (a.score_cover == nullptr) {
    return capacity;
  }
  const int cover = min(capacity, a.score_cover[flat]);
  return min(capacity, ((cover + kTile - 1) / kTile) * kTile);
}

__global__ void __launch_bounds__(kScoreThreads, 2) score_kernel(const ckv_layer_args a) {
  // query group as fp32, laid out [head][k][slice][4] so that the eight slices
  // of one 16-byte read fall into different banks
  __shared__ __align__(16) float q_s[16 * kHeadDim];
  __shared__ int prefix[kScoreMaxUnits + 1];
  const int units = a.batch * a.retrieval_heads;
  const int group = a.group_size;
  const int capacity = a.community_capacity;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = lane & 7;   // which 16 of the 128 dimensions
  const int quad = lane >> 3;   // row inside a group of four consecutive rows
  pdl_release_dependents();

  // inclusive prefix of the per-unit group counts
  for (int unit = threadIdx.x; unit < units; unit += kScoreThreads) {
    prefix[unit + 1] = (score_limit(a, unit) + 15) / 16;
  }
  if (threadIdx.x == 0) {
    prefix[0] = 0;
  }
  __syncthreads();
  if (warp == 0) {
    const int per_lane = (units + 31) / 32;
    const int lo = min(units, lane * per_lane);
    const int hi = min(units, lo + per_lane);
    int running = 0;
    for (int unit = lo; unit < hi; ++unit) {
      running += prefix[unit + 1];
      prefix[unit + 1] = running;
    }
    int offset = running;
#pragma unroll
    for (int delta = 1; delta < 32; delta <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, offset, delta);
      if (lane >= delta) {
        offset += other;
      }
    }
    offset -= running;
    for (int unit = lo; unit < hi; ++unit) {
      prefix[unit + 1] += offset;
    }
  }
  __syncthreads();
  pdl_wait_for_predecessor();  // the query (and last step's state) come from upstream
  const int total = prefix[units];
  const int my_begin = static_cast<int>(static_cast<int64_t>(blockIdx.x) * total / gridDim.x);
  const int my_end = static_cast<int>(static_cast<int64_t>(blockIdx.x + 1) * total / gridDim.x);
  if (my_begin >= my_end) {
    return;
  }
  int flat = 0;
  {
    int low = 0, high = units - 1;  // last unit whose prefix is <= my_begin
    while (low < high) {
      const int middle = (low + high + 1) >> 1;
      if (prefix[middle] <= my_begin) {
        low = middle;
      } else {
        high = middle - 1;
      }
    }
    flat = low;
  }
  const bool up_a = (slice & 4) != 0;
  const bool up_b = (slice & 2) != 0;
  const int my_row_in_group = quad + 4 * ((up_a ? 2 : 0) + (up_b ? 1 : 0));

  for (; flat < units && prefix[flat] < my_end; ++flat) {
    const int first_group = max(my_begin, prefix[flat]) - prefix[flat];
    const int last_group = min(my_end, prefix[flat + 1]) - prefix[flat];
    if (first_group >= last_group) {
      continue;
    }
    const int limit = score_limit(a, flat);
    const uint8_t* table = reinterpret_cast<const uint8_t*>(a.centroids) +
                           static_cast<int64_t>(flat) * capacity * kHeadDim;
    uint4 raw[4];
    int current = first_group + warp;
    if (current < last_group) {
      load_group(table, current * 16, quad, slice, capacity, raw);
    }
    const __nv_bfloat16* query =
        reinterpret_cast<const __nv_bfloat16*>(a.query) + static_cast<int64_t>(flat) * group * kHeadDim;
    __syncthreads();  // the previous unit's query is no longer read
    for (int i = threadIdx.x; i < group * kHeadDim; i += kScoreThreads) {
      const int g = i >> 7;
      const int dim = i & 127;
      q_s[((g * 4 + ((dim >> 2) & 3)) * 8 + (dim >> 4)) * 4 + (dim & 3)] = __bfloat162float(query[i]);
    }
    __syncthreads();

    const int count = a.community_counts[flat];
    const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
    __half* out = reinterpret_cast<__half*>(a.scores) + static_cast<int64_t>(flat) * capacity;

    for (; current < last_group; current += kScoreThreads / 32) {
      float x[4][16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        fp8x4_to_float(raw[i].x, x[i] + 0);
        fp8x4_to_float(raw[i].y, x[i] + 4);
        fp8x4_to_float(raw[i].z, x[i] + 8);
        fp8x4_to_float(raw[i].w, x[i] + 12);
      }
      const int next = current + kScoreThreads / 32;
      if (next < last_group) {
        load_group(table, next * 16, quad, slice, capacity, raw);
      }
      const int row = current * 16 + my_row_in_group;
      int size = 0;
      if ((slice & 1) == 0 && row < limit) {
        size = __ldg(sizes + row);
      }

      float best = -INFINITY;
      // two heads per pass: eight independent accumulation chains per lane
      for (int g = 0; g < group; g += 2) {
        const bool pair = g + 1 < group;
        float qa[16], qb[16];
        const float4* qp = reinterpret_cast<const float4*>(q_s) + g * 32 + slice;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 v = qp[k * 8];
          const float4 w = pair ? qp[32 + k * 8] : v;
          qa[4 * k + 0] = v.x; qa[4 * k + 1] = v.y; qa[4 * k + 2] = v.z; qa[4 * k + 3] = v.w;
          qb[4 * k + 0] = w.x; qb[4 * k + 1] = w.y; qb[4 * k + 2] = w.z; qb[4 * k + 3] = w.w;
        }
        float pa[4], pb[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float acc_a = __fmul_rn(x[i][0], qa[0]);
          float acc_b = __fmul_rn(x[i][0], qb[0]);
#pragma unroll
          for (int k = 1; k < 16; ++k) {
            acc_a = __fmaf_rn(x[i][k], qa[k], acc_a);
            acc_b = __fmaf_rn(x[i][k], qb[k], acc_b);
          }
          pa[i] = acc_a;
          pb[i] = acc_b;
        }
        // Sum the eight slices of each row: (j, j^4), then (j, j^2), then (j, j^1),
        // folding the four rows onto the lanes on the way (a transposing butterfly).
        float keep0_a = up_a ? pa[2] : pa[0], keep1_a = up_a ? pa[3] : pa[1];
        float keep0_b = up_a ? pb[2] : pb[0], keep1_b = up_a ? pb[3] : pb[1];
        keep0_a = __fadd_rn(keep0_a, __shfl_xor_sync(0xffffffffu, up_a ? pa[0] : pa[2], 4));
        keep1_a = __fadd_rn(keep1_a, __shfl_xor_sync(0xffffffffu, up_a ? pa[1] : pa[3], 4));
        keep0_b = __fadd_rn(keep0_b, __shfl_xor_sync(0xffffffffu, up_a ? pb[0] : pb[2], 4));
        keep1_b = __fadd_rn(keep1_b, __shfl_xor_sync(0xffffffffu, up_a ? pb[1] : pb[3], 4));
        float keep_a = up_b ? keep1_a : keep0_a;
        float keep_b = up_b ? keep1_b : keep0_b;
        keep_a = __fadd_rn(keep_a, __shfl_xor_sync(0xffffffffu, up_b ? keep0_a : keep1_a, 2));
        keep_b = __fadd_rn(keep_b, __shfl_xor_sync(0xffffffffu, up_b ? keep0_b : keep1_b, 2));
        keep_a = __fadd_rn(keep_a, __shfl_xor_sync(0xffffffffu, keep_a, 1));
        keep_b = __fadd_rn(keep_b, __shfl_xor_sync(0xffffffffu, keep_b, 1));
        best = fmaxf(best, keep_a);
        if (pair) {
          best = fmaxf(best, keep_b);
        }
      }
      if ((slice & 1) == 0 && row < limit) {
        const bool live = row < count && size > 0;
        out[row] = __float2half_rn(live ? best : -INFINITY);
      }
    }
  }
}

// ---- block-wide exclusive scan of four counters (1024 threads) ----
struct Quad {
  int high_count;
  int high_mass;
  int equal_count;
  int equal_mass;
};

__device__ __forceinline__ Quad quad_add(Quad x, Quad y) {
  return {x.high_count + y.high_count, x.high_mass + y.high_mass, x.equal_count + y.equal_count,
          x.equal_mass + y.equal_mass};
}
__device__ __forceinline__ Quad quad_shfl_up(Quad v, int delta) {
  return {__shfl_up_sync(0xffffffffu, v.high_count, delta),
          __shfl_up_sync(0xffffffffu, v.high_mass, delta),
          __shfl_up_sync(0xffffffffu, v.equal_count, delta),
          __shfl_up_sync(0xffffffffu, v.equal_mass, delta)};
}

// Returns the exclusive prefix of `value` over the block in thread order and the
// block total in *total.  `scratch` holds one Quad per warp.
__device__ Quad block_scan(Quad value, Quad* scratch, Quad* total) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  Quad inclusive = value;
#pragma unroll
  for (int delta = 1; delta < 32; delta <<= 1) {
    const Quad other = quad_shfl_up(inclusive, delta);
    if (lane >= delta) {
      inclusive = quad_add(inclusive, other);
    }
  }
  if (lane == 31) {
    scratch[warp] = inclusive;
  }
  __syncthreads();
  if (warp == 0) {
    const Quad mine = scratch[lane];
    Quad running = mine;
#pragma unroll
    for (int delta = 1; delta < 32; delta <<= 1) {
      const Quad other = quad_shfl_up(running, delta);
      if (lane >= delta) {
        running = quad_add(running, other);
      }
    }
    scratch[lane] = {running.high_count - mine.high_count, running.high_mass - mine.high_mass,
                     running.equal_count - mine.equal_count, running.equal_mass - mine.equal_mass};
    if (lane == 31) {
      *total = running;
    }
  }
  __syncthreads();
  const Quad base = scratch[warp];
  const Quad result = {base.high_count + inclusive.high_count - value.high_count,
                       base.high_mass + inclusive.high_mass - value.high_mass,
                       base.equal_count + inclusive.equal_count - value.equal_count,
                       base.equal_mass + inclusive.equal_mass - value.equal_mass};
  return result;
}

// Warp 0: scan a 256-bin pair of histograms from the top and find the first bin
// at which either the token mass reaches `budget` or (when limit > 0) the
// community count reaches `limit`.
__device__ __forceinline__ void find_threshold_bin(const int* hist_mass, const int* hist_count,
                                                   int budget, int limit, int start_mass,
                                                   int start_count, int* out_bin, int* out_mass,
                                                   int* out_count) {
  const int lane = threadIdx.x & 31;
  int lane_mass = 0;
  int lane_count = 0;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    lane_mass += hist_mass[lane * 8 + b];
    lane_count += hist_count[lane * 8 + b];
  }
  int suffix_mass = lane_mass;
  int suffix_count = lane_count;
#pragma unroll
  for (int delta = 1; delta < 32; delta <<= 1) {
    const int m = __shfl_down_sync(0xffffffffu, suffix_mass, delta);
    const int c = __shfl_down_sync(0xffffffffu, suffix_count, delta);
    if (lane + delta < 32) {
      suffix_mass += m;
      suffix_count += c;
    }
  }
  int mass = start_mass + suffix_mass - lane_mass;
  int count = start_count + suffix_count - lane_count;
  int found_bin = -1;
  int found_mass = 0;
  int found_count = 0;
#pragma unroll
  for (int b = 7; b >= 0; --b) {
    const int hm = hist_mass[lane * 8 + b];
    const int hc = hist_count[lane * 8 + b];
    const bool hit = (mass + hm >= budget) || (limit > 0 && count + hc >= limit);
    if (hit && found_bin < 0) {
      found_bin = lane * 8 + b;
      found_mass = mass;
      found_count = count;
    }
    mass += hm;
    count += hc;
  }
  const unsigned ballot = __ballot_sync(0xffffffffu, found_bin >= 0);
  if (ballot == 0u) {
    if (lane == 0) {
      *out_bin = 0;
      *out_mass = start_mass;
      *out_count = start_count;
    }
  } else if (lane == 31 - __clz(ballot)) {
    *out_bin = found_bin;
    *out_mass = found_mass;
    *out_count = found_count;
  }
}

__global__ void __launch_bounds__(kSelectThreads, 1) select_kernel(const ckv_layer_args a) {
  __shared__ uint16_t stash_key[kStash];
  __shared__ int stash_size[kStash];
  __shared__ int hist_mass[256];
  __shared__ int hist_count[256];
  __shared__ Quad scan_scratch[32];
  __shared__ Quad scan_total;
  __shared__ int s_bin, s_mass, s_count, s_stored_equal, s_descriptors;
  __shared__ int32_t desc_comm[kDescStash];
  __shared__ int32_t desc_end[kDescStash];

  const int flat = blockIdx.x;
  const Unit u = make_unit(a, flat);
  const int tid = threadIdx.x;
  const int capacity = a.community_capacity;
  const int active = max(0, min(capacity, a.community_counts[flat]));
  const int tile_count = a.token_budget / kTile;
  const int budget = a.token_budget - a.num_sink - 1;
  const int limit = a.max_communities;
  const uint16_t* score_bits =
      reinterpret_cast<const uint16_t*>(a.scores) + static_cast<int64_t>(flat) * capacity;
  const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
  const bool stashed = active <= kStash;
  pdl_release_dependents();

  if (tid < 256) {
    hist_mass[tid] = 0;
    hist_count[tid] = 0;
  }
  if (tid == 0) {
    s_stored_equal = 0;
  }
  pdl_wait_for_predecessor();  // the fp16 scores come from the scoring kernel
  if (stashed) {
#pragma unroll 5
    for (int c = tid; c < active; c += kSelectThreads) {
      const int size = __ldg(sizes + c);
      const uint16_t bits = score_bits[c];  // unconditional: both loads are in flight together
      stash_size[c] = size > 0 ? size : 0;
      stash_key[c] = size > 0 ? ordered_key16(bits) : 0;
    }
  }
  __syncthreads();

  auto item = [&](int c, int& size, int& key) {
    if (stashed) {
      size = stash_size[c];
      key = stash_key[c];
    } else {
      size = sizes[c];
      key = size > 0 ? ordered_key16(score_bits[c]) : 0;
      size = size > 0 ? size : 0;
    }
  };

  // Pass 1: histogram of the high key byte, weighted by community size.
  for (int c = tid; c < active; c += kSelectThreads) {
    int size, key;
    item(c, size, key);
    if (size > 0) {
      atomicAdd(&hist_mass[key >> 8], size);
      atomicAdd(&hist_count[key >> 8], 1);
    }
  }
  __syncthreads();
  if (tid < 32) {
    find_threshold_bin(hist_mass, hist_count, budget, limit, 0, 0, &s_bin, &s_mass, &s_count);
  }
  __syncthreads();
  const int high_bin = s_bin;
  const int mass_above = s_mass;
  const int count_above = s_count;
  __syncthreads();
  if (tid < 256) {
    hist_mass[tid] = 0;
    hist_count[tid] = 0;
  }
  __syncthreads();
  // Pass 2: histogram of the low byte inside the chosen high bin.
  for (int c = tid; c < active; c += kSelectThreads) {
    int size, key;
    item(c, size, key);
    if (size > 0 && (key >> 8) == high_bin) {
      atomicAdd(&hist_mass[key & 0xff], size);
      atomicAdd(&hist_count[key & 0xff], 1);
    }
  }
  __syncthreads();
  if (tid < 32) {
    find_threshold_bin(hist_mass, hist_count, budget, limit, mass_above, count_above, &s_bin,
                       &s_mass, &s_count);
  }
  __syncthreads();
  const int threshold = (high_bin << 8) | s_bin;

  // Pass 3: per-thread totals over a contiguous run of communities, then an
  // index-ordered exclusive scan.
  const int per_thread = (active + kSelectThreads - 1) / kSelectThreads;
  const int first = min(active, tid * per_thread);
  const int last = min(active, first + per_thread);
  Quad mine = {0, 0, 0, 0};
  for (int c = first; c < last; ++c) {
    int size, key;
    item(c, size, key);
    if (size > 0) {
      if (key > threshold) {
        mine.high_count += 1;
        mine.high_mass += size;
      } else if (key == threshold) {
        mine.equal_count += 1;
        mine.equal_mass += size;
      }
    }
  }
  Quad prefix = block_scan(mine, scan_scratch, &scan_total);
  const int total_high_count = scan_total.high_count;
  const int total_high_mass = scan_total.high_mass;

  // Pass 4: emit descriptors in community-index order.
  int32_t* out_comm = a.communities + static_cast<int64_t>(flat) * a.descriptor_capacity;
  int32_t* out_ends = a.cumulative_ends + static_cast<int64_t>(flat) * a.descriptor_capacity;
  int stored_equal = 0;
  for (int c = first; c < last; ++c) {
    int size, key;
    item(c, size, key);
    if (size <= 0) {
      continue;
    }
    if (key > threshold) {
      const int descriptor = prefix.high_count;
      prefix.high_count += 1;
      prefix.high_mass += size;
      if (descriptor < a.descriptor_capacity) {
        out_comm[descriptor] = c;
        out_ends[descriptor] = prefix.high_mass;
        if (descriptor < kDescStash) {
          desc_comm[descriptor] = c;
          desc_end[descriptor] = prefix.high_mass;
        }
      }
    } else if (key == threshold) {
      const int start = total_high_mass + prefix.equal_mass;
      const int rank = total_high_count + prefix.equal_count;
      prefix.equal_count += 1;
      prefix.equal_mass += size;
      const bool stored = start < budget && (limit <= 0 || rank < limit);
      if (stored) {
        if (rank < a.descriptor_capacity) {
          out_comm[rank] = c;
          out_ends[rank] = min(budget, start + size);
          if (rank < kDescStash) {
            desc_comm[rank] = c;
            desc_end[rank] = min(budget, start + size);
          }
        }
        stored_equal += 1;
      }
    }
  }
  if (stored_equal > 0) {
    atomicAdd(&s_stored_equal, stored_equal);
  }
  __syncthreads();
  if (tid == 0) {
    const int descriptors = min(a.descriptor_capacity, total_high_count + s_stored_equal);
    s_descriptors = descriptors;
    a.descriptor_counts[flat] = descriptors;
    if (a.threshold_state != nullptr) {
      a.threshold_state[static_cast<int64_t>(flat) * 4] = threshold;
    }
  }
  __syncthreads();
  const int descriptors = s_descriptors;
  const bool in_smem = descriptors <= kDescStash;
  const int32_t* search_ends = in_smem ? desc_end : out_ends;
  const int32_t* search_comm = in_smem ? desc_comm : out_comm;

  // First descriptor of every 64-token tile.
  for (int tile = tid; tile < tile_count; tile += kSelectThreads) {
    const int offset = max(tile * kTile - a.num_sink, 0);
    int low = 0;
    int high = descriptors;
    while (low < high) {
      const int middle = (low + high) >> 1;
      if (search_ends[middle] <= offset) {
        low = middle + 1;
      } else {
        high = middle;
      }
    }
    a.tile_descriptors[static_cast<int64_t>(flat) * tile_count + tile] =
        max(0, min(low, descriptors - 1));
  }

  // Resolve every logical token of the budget to its cache row.
  // Two logical tokens per thread and pass, so that the two dependent global
  // reads of each (community tables, then the member list) overlap.
  int32_t* positions = a.positions + static_cast<int64_t>(flat) * a.token_budget;
  const int64_t graph_slot = static_cast<int64_t>(u.batch) * a.graphs + u.graph;
  const int32_t* delta_sizes = a.delta_sizes + graph_slot * capacity;
  const int32_t* offsets = a.member_offsets + graph_slot * (capacity + 1);
  const int32_t* members = a.member_positions + graph_slot * a.member_capacity;
  for (int base = 0; base < a.token_budget; base += 2 * kSelectThreads) {
    int logical[2], community[2], member[2], direct[2];
    bool lookup[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      logical[i] = base + i * kSelectThreads + tid;
      lookup[i] = false;
      direct[i] = -1;
      community[i] = 0;
      member[i] = 0;
      if (logical[i] >= a.token_budget) {
        continue;
      }
      if (logical[i] < a.num_sink) {
        direct[i] = a.sink_positions[logical[i]];
      } else if (logical[i] == a.token_budget - 1) {
        direct[i] = a.current_position[graph_slot];
      } else {
        const int offset = logical[i] - a.num_sink;
        int low = 0;
        int high = descriptors;
        while (low < high) {
          const int middle = (low + high) >> 1;
          if (search_ends[middle] <= offset) {
            low = middle + 1;
          } else {
            high = middle;
          }
        }
        if (low < descriptors) {
          lookup[i] = true;
          community[i] = search_comm[low];
          member[i] = offset - (low > 0 ? search_ends[low - 1] : 0);
        }
      }
    }
    int delta_count[2], start[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      delta_count[i] = lookup[i] ? delta_sizes[community[i]] : 0;
      start[i] = lookup[i] ? offsets[community[i]] : 0;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (lookup[i] && member[i] >= delta_count[i]) {
        direct[i] = members[start[i] + member[i] - delta_count[i]];
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (lookup[i] && member[i] < delta_count[i]) {
        direct[i] = delta_member_position(a, graph_slot, community[i], member[i]);
      }
      if (logical[i] < a.token_budget) {
        positions[logical[i]] = direct[i];
      }
    }
  }
}

// Position resolution alone, from descriptors that are already in the workspace.
__global__ void __launch_bounds__(256) resolve_kernel(const ckv_layer_args a) {
  const int flat = blockIdx.y;
  const Unit u = make_unit(a, flat);
  const int logical = blockIdx.x * 256 + threadIdx.x;
  if (logical >= a.token_budget) {
    return;
  }
  const int descriptors = min(a.descriptor_capacity, max(0, a.descriptor_counts[flat]));
  const int64_t base = static_cast<int64_t>(flat) * a.descriptor_capacity;
  a.positions[static_cast<int64_t>(flat) * a.token_budget + logical] =
      resolve_token(a, u, a.cumulative_ends + base, a.communities + base, logical, descriptors);
}

cudaError_t launch_score(const ckv_layer_args& a, cudaStream_t stream) {
  // two CTAs per SM are resident: one wave, but never finer than eight 16-row
  // groups (one per warp) per CTA
  const int units = a.batch * a.retrieval_heads;
  if (units > kScoreMaxUnits) {
    return cudaErrorInvalidConfiguration;
  }
  const long long finest = static_cast<long long>(units) * ((a.community_capacity + 127) / 128);
  const int grid = finest < 1 ? 1 : (finest > 2 * 148 ? 2 * 148 : static_cast<int>(finest));
  return launch_dependent(score_kernel, dim3(grid), dim3(kScoreThreads), 0, stream, a);
}

cudaError_t launch_select(const ckv_layer_args& a, cudaStream_t stream) {
  return launch_dependent(select_kernel, dim3(a.batch * a.retrieval_heads), dim3(kSelectThreads), 0,
                          stream, a);
}

cudaError_t launch_resolve(const ckv_layer_args& a, cudaStream_t stream) {
  const dim3 grid((a.token_budget + 255) / 256, a.batch * a.retrieval_heads);
  resolve_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ckv
