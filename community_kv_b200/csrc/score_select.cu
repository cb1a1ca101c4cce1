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
constexpr int kScoreRowsPerBlock = 128;  // 8 warps x 16 rows
constexpr int kSelectThreads = 1024;
constexpr int kStash = 4608;  // communities whose keys/sizes are staged in shared memory

__global__ void __launch_bounds__(kScoreThreads) score_kernel(const ckv_layer_args a) {
  __shared__ __align__(16) float q_s[16 * kHeadDim];
  const int flat = blockIdx.y;
  const Unit u = make_unit(a, flat);
  const int group = a.group_size;
  const __nv_bfloat16* query = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                               (static_cast<int64_t>(u.batch) * a.retrieval_heads + u.head) *
                                   group * kHeadDim;
  for (int i = threadIdx.x; i < group * kHeadDim; i += kScoreThreads) {
    q_s[i] = __bfloat162float(query[i]);
  }
  __syncthreads();

  const int capacity = a.community_capacity;
  int limit = capacity;
  if (a.score_cover != nullptr) {
    const int cover = min(capacity, a.score_cover[flat]);
    limit = min(capacity, ((cover + kTile - 1) / kTile) * kTile);
  }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = lane & 7;   // which 16 of the 128 dimensions
  const int quad = lane >> 3;   // row inside a group of four consecutive rows
  const int row_base = blockIdx.x * kScoreRowsPerBlock + warp * 16;
  if (row_base >= limit) {
    return;
  }
  const int count = a.community_counts[flat];
  const uint8_t* table =
      reinterpret_cast<const uint8_t*>(a.centroids) + static_cast<int64_t>(flat) * capacity * kHeadDim;

  float x[4][16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = min(row_base + quad + 4 * i, capacity - 1);
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(table + static_cast<int64_t>(row) * kHeadDim) + slice);
    fp8x4_to_float(raw.x, x[i] + 0);
    fp8x4_to_float(raw.y, x[i] + 4);
    fp8x4_to_float(raw.z, x[i] + 8);
    fp8x4_to_float(raw.w, x[i] + 12);
  }

  const bool up_a = (slice & 4) != 0;
  const bool up_b = (slice & 2) != 0;
  float best = -INFINITY;
  for (int g = 0; g < group; ++g) {
    float qv[16];
    const float4* qp = reinterpret_cast<const float4*>(q_s + g * kHeadDim + slice * 16);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 v = qp[k];
      qv[4 * k + 0] = v.x;
      qv[4 * k + 1] = v.y;
      qv[4 * k + 2] = v.z;
      qv[4 * k + 3] = v.w;
    }
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float acc = __fmul_rn(x[i][0], qv[0]);
#pragma unroll
      for (int k = 1; k < 16; ++k) {
        acc = __fmaf_rn(x[i][k], qv[k], acc);
      }
      p[i] = acc;
    }
    // Sum the eight slices of each row: (j, j^4), then (j, j^2), then (j, j^1),
    // folding the four rows onto the lanes on the way (a transposing butterfly).
    float keep0 = up_a ? p[2] : p[0];
    float keep1 = up_a ? p[3] : p[1];
    const float send0 = up_a ? p[0] : p[2];
    const float send1 = up_a ? p[1] : p[3];
    keep0 = __fadd_rn(keep0, __shfl_xor_sync(0xffffffffu, send0, 4));
    keep1 = __fadd_rn(keep1, __shfl_xor_sync(0xffffffffu, send1, 4));
    float keep = up_b ? keep1 : keep0;
    const float send = up_b ? keep0 : keep1;
    keep = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 2));
    keep = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, keep, 1));
    best = fmaxf(best, keep);
  }

  if ((slice & 1) == 0) {
    const int row = row_base + quad + 4 * ((up_a ? 2 : 0) + (up_b ? 1 : 0));
    if (row < limit) {
      const bool live =
          row < count && a.community_sizes[static_cast<int64_t>(flat) * capacity + row] > 0;
      __half* out = reinterpret_cast<__half*>(a.scores) + static_cast<int64_t>(flat) * capacity;
      out[row] = __float2half_rn(live ? best : -INFINITY);
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

__global__ void __launch_bounds__(kSelectThreads) select_kernel(const ckv_layer_args a) {
  __shared__ uint16_t stash_key[kStash];
  __shared__ int stash_size[kStash];
  __shared__ int hist_mass[256];
  __shared__ int hist_count[256];
  __shared__ Quad scan_scratch[32];
  __shared__ Quad scan_total;
  __shared__ int s_bin, s_mass, s_count, s_stored_equal, s_descriptors;

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

  if (tid < 256) {
    hist_mass[tid] = 0;
    hist_count[tid] = 0;
  }
  if (tid == 0) {
    s_stored_equal = 0;
  }
  if (stashed) {
    for (int c = tid; c < active; c += kSelectThreads) {
      const int size = sizes[c];
      stash_size[c] = size > 0 ? size : 0;
      stash_key[c] = size > 0 ? ordered_key16(score_bits[c]) : 0;
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

  // First descriptor of every 64-token tile.
  for (int tile = tid; tile < tile_count; tile += kSelectThreads) {
    const int offset = max(tile * kTile - a.num_sink, 0);
    int low = 0;
    int high = descriptors;
    while (low < high) {
      const int middle = (low + high) >> 1;
      if (out_ends[middle] <= offset) {
        low = middle + 1;
      } else {
        high = middle;
      }
    }
    a.tile_descriptors[static_cast<int64_t>(flat) * tile_count + tile] =
        max(0, min(low, descriptors - 1));
  }

  // Resolve every logical token of the budget to its cache row.
  int32_t* positions = a.positions + static_cast<int64_t>(flat) * a.token_budget;
  for (int logical = tid; logical < a.token_budget; logical += kSelectThreads) {
    positions[logical] = resolve_token(a, u, flat, logical, descriptors);
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
  a.positions[static_cast<int64_t>(flat) * a.token_budget + logical] =
      resolve_token(a, u, flat, logical, descriptors);
}

cudaError_t launch_score(const ckv_layer_args& a, cudaStream_t stream) {
  const dim3 grid((a.community_capacity + kScoreRowsPerBlock - 1) / kScoreRowsPerBlock,
                  a.batch * a.retrieval_heads);
  score_kernel<<<grid, kScoreThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_select(const ckv_layer_args& a, cudaStream_t stream) {
  select_kernel<<<a.batch * a.retrieval_heads, kSelectThreads, 0, stream>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_resolve(const ckv_layer_args& a, cudaStream_t stream) {
  const dim3 grid((a.token_budget + 255) / 256, a.batch * a.retrieval_heads);
  resolve_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ckv
