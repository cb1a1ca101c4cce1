// Device functions of centroid scoring and budgeted community selection, shared by
// the stand-alone kernels and the fused per-layer cluster kernel (sm_100a).
#pragma once

#include <cstddef>

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

// Scores the 16-row groups [first_group, last_group) of one unit: scores[c] =
// fp16(max over the query group of q . centroid[c]).  Every thread of the CTA calls
// it with the same arguments (the query group is staged in `q_s`, 2 * 16 * 128 floats
// of shared memory, 16-byte aligned, behind block barriers); a warp takes every (kThreads / 32)-th
// group and keeps the next group's loads in flight while it computes.
//
// With `slice` set, the keys and sizes of the scored rows are also kept in shared
// memory (index row - slice->row0) and counted into the slice's first-pass
// histogram, which is what a cluster-wide selection starts from.
struct ScoreSlice {
  uint16_t* key;     // order-preserving 16-bit key, 0 for dead rows
  int* size;         // community size, 0 for dead rows
  int* hist_mass;    // 256 bins over the high key byte, weighted by size
  int* hist_count;
  int row0;
  // Speculation: last step's threshold usually falls into the same high-byte bin again.
  // Rows whose key lies in `guess_bin` (-1: none) are also counted by their low byte, so
  // that the second histogram pass of the selection is already done if the guess holds.
  int* low_mass;
  int* low_count;
  int guess_bin;
};

template <int kThreads, bool kNarrow>
__device__ __forceinline__ void score_groups_impl(const ckv_layer_args& a, int flat, int first_group,
                                                  int last_group, float* q_s,
                                                  const ScoreSlice* slice_out) {
  const int group = a.group_size;
  const int capacity = a.community_capacity;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = lane & 7;   // which 16 of the 128 dimensions
  const int quad = lane >> 3;   // row inside a group of four consecutive rows
  const bool up_a = (slice & 4) != 0;
  const bool up_b = (slice & 2) != 0;
  const int my_row_in_group = quad + 4 * ((up_a ? 2 : 0) + (up_b ? 1 : 0));
  const int limit = score_limit(a, flat);
  const uint8_t* table = reinterpret_cast<const uint8_t*>(a.centroids) +
                         static_cast<int64_t>(flat) * capacity * kHeadDim;
  // two groups in flight per warp: with one, the loop runs at one memory round trip
  // per group
  constexpr int kStride = kThreads / 32;
  uint4 raw_even[4], raw_odd[4];
  int size_even = 0, size_odd = 0;  // size of this lane's row, fetched with the group's rows
  const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
  auto load_size = [&](int group_index) {
    const int row = group_index * 16 + my_row_in_group;
    return ((slice & 1) == 0 && row < limit) ? __ldg(sizes + row) : 0;
  };
  int current = first_group + warp;
  if (current < last_group) {
    load_group(table, current * 16, quad, slice, capacity, raw_even);
    size_even = load_size(current);
  }
  if (current + kStride < last_group) {
    load_group(table, (current + kStride) * 16, quad, slice, capacity, raw_odd);
    size_odd = load_size(current + kStride);
  }
  const __nv_bfloat16* query =
      reinterpret_cast<const __nv_bfloat16*>(a.query) + static_cast<int64_t>(flat) * group * kHeadDim;
  __syncthreads();  // the previous unit's query is no longer read
  // Up to four heads: this lane's 16 dimensions of every head stay in registers as
  // packed bf16 (a missing head repeats the last one, which leaves the maximum
  // unchanged).  More heads: the group is staged in shared memory as fp32.
  uint32_t q_bf16[kNarrow ? 4 : 1][8];
  if constexpr (kNarrow) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const uint4* src =
          reinterpret_cast<const uint4*>(query + min(h, group - 1) * kHeadDim + slice * 16);
      const uint4 lo = src[0];
      const uint4 hi = src[1];
      q_bf16[h][0] = lo.x; q_bf16[h][1] = lo.y; q_bf16[h][2] = lo.z; q_bf16[h][3] = lo.w;
      q_bf16[h][4] = hi.x; q_bf16[h][5] = hi.y; q_bf16[h][6] = hi.z; q_bf16[h][7] = hi.w;
    }
  }
  for (int i = threadIdx.x; !kNarrow && i < group * kHeadDim; i += kThreads) {
    const int g = i >> 7;
    const int dim = i & 127;
    // [head][dimension pair of the slice][slice] x {q, q, q', q'}: a warp's eight
    // slices read 128 contiguous bytes, every value arrives already duplicated
    const float value = __bfloat162float(query[i]);
    const int at = ((g * 8 + ((dim & 15) >> 1)) * 8 + (dim >> 4)) * 4 + (dim & 1) * 2;
    q_s[at] = value;
    q_s[at + 1] = value;
  }
  __syncthreads();

  const int count = a.community_counts[flat];
  __half* out = reinterpret_cast<__half*>(a.scores) + static_cast<int64_t>(flat) * capacity;

  auto score_one = [&](uint4 (&raw)[4], int& held_size, int current) {
    // The narrow path widens e4m3 to bf16 with integer operations and feeds
    // mixed-precision FMAs (bf16 x bf16 + fp32, one rounding: the same value as
    // the fp32 FMA of the widened operands); the wide path widens to fp32.
    uint32_t xb[kNarrow ? 4 : 1][8];
    float x[kNarrow ? 1 : 4][16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (kNarrow) {
        e4m3x4_to_bf16x2(raw[i].x, xb[i][0], xb[i][1]);
        e4m3x4_to_bf16x2(raw[i].y, xb[i][2], xb[i][3]);
        e4m3x4_to_bf16x2(raw[i].z, xb[i][4], xb[i][5]);
        e4m3x4_to_bf16x2(raw[i].w, xb[i][6], xb[i][7]);
      } else {
        fp8x4_to_float(raw[i].x, x[i] + 0);
        fp8x4_to_float(raw[i].y, x[i] + 4);
        fp8x4_to_float(raw[i].z, x[i] + 8);
        fp8x4_to_float(raw[i].w, x[i] + 12);
      }
    }
    const int next = current + 2 * kStride;  // this buffer's next group
    const int size = held_size;
    if (next < last_group) {
      load_group(table, next * 16, quad, slice, capacity, raw);
      held_size = load_size(next);
    }
    const int row = current * 16 + my_row_in_group;

    float best;
    if constexpr (kNarrow) {
      // four independent chains (one per head) of 16 sequential FMAs per row;
      // starting from -0 makes the first step the plain product, sign included
      float per_head[4][4];  // [head][row]
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float acc[4] = {-0.0f, -0.0f, -0.0f, -0.0f};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            acc[h] = fma2_bf16(xb[i][j], q_bf16[h][j], acc[h]);
          }
        }
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          per_head[h][i] = acc[h];
        }
      }
      best = -INFINITY;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        // Sum the eight slices of each row: (j, j^4), then (j, j^2), then (j, j^1),
        // folding the four rows onto the lanes on the way (a transposing butterfly).
        const float* pa = per_head[h];
        float keep0 = up_a ? pa[2] : pa[0], keep1 = up_a ? pa[3] : pa[1];
        keep0 = __fadd_rn(keep0, __shfl_xor_sync(0xffffffffu, up_a ? pa[0] : pa[2], 4));
        keep1 = __fadd_rn(keep1, __shfl_xor_sync(0xffffffffu, up_a ? pa[1] : pa[3], 4));
        float keep = up_b ? keep1 : keep0;
        keep = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, up_b ? keep0 : keep1, 2));
        keep = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, keep, 1));
        best = fmaxf(best, keep);
      }
    } else {
      // Rows (0,1) and (2,3) of this lane ride together in packed fp32 pairs: one
      // two-wide FMA advances both rows' chains (each half rounds like a scalar FMA).
      uint64_t x01[16], x23[16];
  #pragma unroll
      for (int k = 0; k < 16; ++k) {
        x01[k] = pack_f32x2(x[0][k], x[1][k]);
        x23[k] = pack_f32x2(x[2][k], x[3][k]);
      }
      best = -INFINITY;
      for (int g = 0; g < group; ++g) {
        // {q, q} pairs of this lane's 16 dimensions, two dimensions per 16-byte read
        const ulonglong2* qp = reinterpret_cast<const ulonglong2*>(q_s) + g * 64 + slice;
        ulonglong2 q2 = qp[0];
        uint64_t acc01 = mul_f32x2(x01[0], q2.x);
        uint64_t acc23 = mul_f32x2(x23[0], q2.x);
        acc01 = fma_f32x2(x01[1], q2.y, acc01);
        acc23 = fma_f32x2(x23[1], q2.y, acc23);
  #pragma unroll
        for (int k2 = 1; k2 < 8; ++k2) {
          q2 = qp[k2 * 8];
          acc01 = fma_f32x2(x01[2 * k2], q2.x, acc01);
          acc23 = fma_f32x2(x23[2 * k2], q2.x, acc23);
          acc01 = fma_f32x2(x01[2 * k2 + 1], q2.y, acc01);
          acc23 = fma_f32x2(x23[2 * k2 + 1], q2.y, acc23);
        }
        float pa[4];
        unpack_f32x2(acc01, pa[0], pa[1]);
        unpack_f32x2(acc23, pa[2], pa[3]);
        // Sum the eight slices of each row: (j, j^4), then (j, j^2), then (j, j^1),
        // folding the four rows onto the lanes on the way (a transposing butterfly).
        float keep0 = up_a ? pa[2] : pa[0], keep1 = up_a ? pa[3] : pa[1];
        keep0 = __fadd_rn(keep0, __shfl_xor_sync(0xffffffffu, up_a ? pa[0] : pa[2], 4));
        keep1 = __fadd_rn(keep1, __shfl_xor_sync(0xffffffffu, up_a ? pa[1] : pa[3], 4));
        float keep = up_b ? keep1 : keep0;
        keep = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, up_b ? keep0 : keep1, 2));
        keep = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, keep, 1));
        best = fmaxf(best, keep);
      }
    }
    if ((slice & 1) == 0 && row < limit) {
      const bool live = row < count && size > 0;
      const __half rounded = __float2half_rn(live ? best : -INFINITY);
      out[row] = rounded;
      if (slice_out != nullptr) {
        const int key = live ? ordered_key16(__half_as_ushort(rounded)) : 0;
        slice_out->key[row - slice_out->row0] = static_cast<uint16_t>(key);
        slice_out->size[row - slice_out->row0] = live ? size : 0;
        if (live) {
          atomicAdd(&slice_out->hist_mass[key >> 8], size);
          atomicAdd(&slice_out->hist_count[key >> 8], 1);
          if ((key >> 8) == slice_out->guess_bin) {
            atomicAdd(&slice_out->low_mass[key & 0xff], size);
            atomicAdd(&slice_out->low_count[key & 0xff], 1);
          }
        }
      }
    }
  };
  for (; current < last_group; current += 2 * kStride) {
    score_one(raw_even, size_even, current);
    if (current + kStride < last_group) {
      score_one(raw_odd, size_odd, current + kStride);
    }
  }
}

// Tensor-core variant of score_groups (CKV_FLAG_TENSOR_SCORES, group size <= 8).
//
// A 16-row group is one mma.m16n8k16 tile: the 16 communities on M, the (padded)
// query group on N = 8, eight k-blocks of 16 dimensions accumulated in ascending
// order in fp32.  The e4m3 rows travel global -> shared memory with 16-byte cp.async
// (no register staging; `stage` holds two groups per warp for four warps) and are
// read back with ldmatrix, which hands thread (g, t) the four bytes 4t..4t+3 of row
// g's 16-byte chunk: after the integer widening to bf16 those are exactly one
// A-fragment pair, so no shuffle is needed.  (The order of the 16 products inside one
// k-block does not change the result of the instruction, so the query fragments use
// the same 4t..4t+3 assignment.)  The sum is the hardware's, not the fixed CUDA-core
// order: a score may differ from the fixed-order one in the last fp16 bit.
template <int kThreads, int kStageBytes>
__device__ __forceinline__ void score_groups_mma(const ckv_layer_args& a, int flat, int first_group,
                                                 int last_group, float* stage_f,
                                                 const ScoreSlice* slice_out) {
  constexpr int kWarps = kThreads / 32;
  constexpr int kGroupBytes = 16 * kHeadDim;                 // one staged group of e4m3 rows
  constexpr int kSlotBytes = kGroupBytes + 64;               // ... followed by the rows' sizes
  constexpr int kRing = kStageBytes / (kWarps * kSlotBytes);   // groups in flight per warp
  static_assert(kRing >= 1 && kRing <= 4, "staging area: one to four groups per warp");
  const int group = a.group_size;
  const int capacity = a.community_capacity;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int limit = score_limit(a, flat);
  const uint8_t* table = reinterpret_cast<const uint8_t*>(a.centroids) +
                         static_cast<int64_t>(flat) * capacity * kHeadDim;
  const uint32_t stage = smem_u32(stage_f) + warp * (kRing * kSlotBytes);
  const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
  __syncthreads();  // the staging area is free (a previous unit's rows have been consumed)

  auto issue = [&](int group_index, int slot) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int piece = lane + 32 * i;
      const int row = piece >> 3;
      const int chunk = piece & 7;
      const int source_row = min(group_index * 16 + row, capacity - 1);
      cp_async16(stage + slot * kSlotBytes + row * kHeadDim + ((chunk ^ (row & 7)) << 4),
                 table + static_cast<int64_t>(source_row) * kHeadDim + chunk * 16, 16u);
    }
    if (lane < 16) {
      cp_async4(stage + slot * kSlotBytes + kGroupBytes + lane * 4,
                sizes + min(group_index * 16 + lane, capacity - 1));
    }
  };
  constexpr int kStride = kWarps;
  int current = first_group + warp;
#pragma unroll
  for (int r = 0; r < kRing; ++r) {
    if (current + r * kStride < last_group) {
      issue(current + r * kStride, r);
    }
    cp_async_commit();
  }

  // B fragments: head g of the group (zero beyond it), dimensions 16j + 4t .. + 3
  uint32_t qb[8][2];
  {
    const __nv_bfloat16* query = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                                 static_cast<int64_t>(flat) * group * kHeadDim;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint2 pair = make_uint2(0u, 0u);
      if (g < group) {
        pair = *reinterpret_cast<const uint2*>(query + g * kHeadDim + 16 * j + 4 * t);
      }
      qb[j][0] = pair.x;
      qb[j][1] = pair.y;
    }
  }
  const int count = a.community_counts[flat];
  __half* out = reinterpret_cast<__half*>(a.scores) + static_cast<int64_t>(flat) * capacity;
  // ldmatrix.x4 row address of this lane: matrix m = lane >> 3 covers rows 8 (m & 1) ..,
  // chunk j + (m >> 1)
  const int lm_row = (lane & 7) + 8 * ((lane >> 3) & 1);
  const int lm_chunk = lane >> 4;

  int slot = 0;
  for (; current < last_group; current += kStride) {
    // lanes t == 0 report row g, lanes t == 1 row g + 8
    const int row = current * 16 + g + 8 * (t & 1);
    cp_async_wait<kRing - 1>();
    __syncwarp();
    int size;
    asm volatile("ld.shared.s32 %0, [%1];"
                 : "=r"(size)
                 : "r"(stage + slot * kSlotBytes + kGroupBytes + (g + 8 * (t & 1)) * 4));
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t base = stage + slot * kSlotBytes + lm_row * kHeadDim;
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4(base + (((j + lm_chunk) ^ (lm_row & 7)) << 4), r0, r1, r2, r3);
      uint32_t a0, a1, a2, a3;
      e4m3x4_to_bf16x2(r0, a0, a2);
      e4m3x4_to_bf16x2(r1, a1, a3);
      mma_bf16_16816(d, a0, a1, a2, a3, qb[j][0], qb[j][1]);
      e4m3x4_to_bf16x2(r2, a0, a2);
      e4m3x4_to_bf16x2(r3, a1, a3);
      mma_bf16_16816(d, a0, a1, a2, a3, qb[j + 1][0], qb[j + 1][1]);
    }
    __syncwarp();  // every lane has read the slot
    if (current + kRing * kStride < last_group) {
      issue(current + kRing * kStride, slot);
    }
    cp_async_commit();
    slot = (slot + 1) % kRing;
    // d0/d1: row g, heads 2t, 2t+1; d2/d3: row g + 8
    const bool head0 = 2 * t < group;
    const bool head1 = 2 * t + 1 < group;
    float low = fmaxf(head0 ? d[0] : -INFINITY, head1 ? d[1] : -INFINITY);
    float high = fmaxf(head0 ? d[2] : -INFINITY, head1 ? d[3] : -INFINITY);
    low = fmaxf(low, __shfl_xor_sync(0xffffffffu, low, 1));
    high = fmaxf(high, __shfl_xor_sync(0xffffffffu, high, 1));
    low = fmaxf(low, __shfl_xor_sync(0xffffffffu, low, 2));
    high = fmaxf(high, __shfl_xor_sync(0xffffffffu, high, 2));
    if (t < 2 && row < limit) {
      const float best = t == 0 ? low : high;
      const bool live = row < count && size > 0;
      const __half rounded = __float2half_rn(live ? best : -INFINITY);
      out[row] = rounded;
      if (slice_out != nullptr) {
        const int key = live ? ordered_key16(__half_as_ushort(rounded)) : 0;
        slice_out->key[row - slice_out->row0] = static_cast<uint16_t>(key);
        slice_out->size[row - slice_out->row0] = live ? size : 0;
        if (live) {
          atomicAdd(&slice_out->hist_mass[key >> 8], size);
          atomicAdd(&slice_out->hist_count[key >> 8], 1);
          if ((key >> 8) == slice_out->guess_bin) {
            atomicAdd(&slice_out->low_mass[key & 0xff], size);
            atomicAdd(&slice_out->low_count[key & 0xff], 1);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
}

// `q_s`: staging area of kStageBytes (>= 16 KB, 128-byte aligned) in shared memory.
template <int kThreads, int kStageBytes = 2 * 16 * kHeadDim * 4>
__device__ __forceinline__ void score_groups(const ckv_layer_args& a, int flat, int first_group,
                                             int last_group, float* q_s,
                                             const ScoreSlice* slice_out = nullptr) {
  if ((a.flags & CKV_FLAG_TENSOR_SCORES) && a.group_size <= 8) {
    score_groups_mma<kThreads, kStageBytes>(a, flat, first_group, last_group, q_s, slice_out);
    return;
  }
  if (a.group_size <= 4) {
    score_groups_impl<kThreads, true>(a, flat, first_group, last_group, q_s, slice_out);
  } else {
    score_groups_impl<kThreads, false>(a, flat, first_group, last_group, q_s, slice_out);
  }
}

// ---- block-wide exclusive scan of four counters ----
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
// block total in *total.  `scratch` holds one Quad per warp (kWarps of them).
template <int kWarps>
__device__ __forceinline__ Quad block_scan(Quad value, Quad* scratch, Quad* total) {
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
    const Quad mine = lane < kWarps ? scratch[lane] : Quad{0, 0, 0, 0};
    Quad running = mine;
#pragma unroll
    for (int delta = 1; delta < 32; delta <<= 1) {
      const Quad other = quad_shfl_up(running, delta);
      if (lane >= delta) {
        running = quad_add(running, other);
      }
    }
    if (lane < kWarps) {
      scratch[lane] = {running.high_count - mine.high_count, running.high_mass - mine.high_mass,
                       running.equal_count - mine.equal_count, running.equal_mass - mine.equal_mass};
    }
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

// Tail of a selection, shared by the one-CTA and the cluster variant: the first
// descriptor of every 64-token tile (when `report_tiles`), then logical tokens
// [token_begin, token_end) -> cache rows, four per thread and pass so that the
// dependent global reads of each overlap.  `search_ends` / `search_comm` hold the
// `descriptors` descriptors (shared or global memory).
template <int kThreads>
__device__ __forceinline__ void resolve_tokens(const ckv_layer_args& a, int flat, const Unit& u,
                                               const int32_t* search_ends, const int32_t* search_comm,
                                               int descriptors, bool report_tiles, int token_begin,
                                               int token_end) {
  const int tid = threadIdx.x;
  const int capacity = a.community_capacity;
  const int tile_count = a.token_budget / kTile;
  // First descriptor of every 64-token tile.
  for (int tile = tid; report_tiles && tile < tile_count; tile += kThreads) {
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

  // This CTA's logical tokens -> cache rows (four per thread and pass, so that the
  // dependent global reads of each overlap).
  int32_t* positions = a.positions + static_cast<int64_t>(flat) * a.token_budget;
  const int64_t graph_slot = static_cast<int64_t>(u.batch) * a.graphs + u.graph;
  const int32_t* delta_sizes = a.delta_sizes + graph_slot * capacity;
  const int32_t* offsets = a.member_offsets + graph_slot * (capacity + 1);
  const int32_t* members = a.member_positions + graph_slot * a.member_capacity;
  for (int base = token_begin; base < token_end; base += 4 * kThreads) {
    int logical[4], community[4], member[4], direct[4];
    bool lookup[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      logical[i] = base + i * kThreads + tid;
      lookup[i] = false;
      direct[i] = -1;
      community[i] = 0;
      member[i] = 0;
      if (logical[i] >= token_end) {
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
    int delta_count[4], start[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      delta_count[i] = lookup[i] ? delta_sizes[community[i]] : 0;
      start[i] = lookup[i] ? offsets[community[i]] : 0;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (lookup[i] && member[i] >= delta_count[i]) {
        direct[i] = members[start[i] + member[i] - delta_count[i]];
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (lookup[i] && member[i] < delta_count[i]) {
        direct[i] = delta_member_position(a, graph_slot, community[i], member[i]);
      }
      if (logical[i] < token_end) {
        positions[logical[i]] = direct[i];
      }
    }
  }
}

// Shared memory of one selection.
struct SelectSmem {
  // keys and sizes of the unit's communities, staged by the caller in (dynamic) shared
  // memory: `stash_capacity` entries each
  uint16_t* stash_key;
  int* stash_size;
  int stash_capacity;
  int* warp_mass;   // optional: one 256-bin histogram per warp (see select_unit), else null
  int* warp_count;
  int hist_mass[256];
  int hist_count[256];
  Quad scan_scratch[32];
  Quad scan_total;
  int bin, mass, count, stored_equal, descriptors;
  int32_t desc_comm[kDescStash];
  int32_t desc_end[kDescStash];
};

// Budgeted community selection of one unit by a CTA of kThreads threads, followed by
// the resolution of logical tokens [token_begin, token_end) to cache rows.  With
// `write_outputs` false the descriptors stay in shared memory only (several CTAs of
// a cluster run the same selection and one of them reports it); the caller then
// makes sure that the descriptors fit `kDescStash`.
template <int kThreads>
__device__ __forceinline__ void select_unit(const ckv_layer_args& a, int flat, SelectSmem& sm,
                                            bool write_outputs, int token_begin, int token_end) {
  const Unit u = make_unit(a, flat);
  const int tid = threadIdx.x;
  const int capacity = a.community_capacity;
  const int active = max(0, min(capacity, a.community_counts[flat]));
  const int budget = a.token_budget - a.num_sink - 1;
  const int limit = a.max_communities;
  const uint16_t* score_bits =
      reinterpret_cast<const uint16_t*>(a.scores) + static_cast<int64_t>(flat) * capacity;
  const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
  const bool stashed = active <= sm.stash_capacity;

  for (int bin = tid; bin < 256; bin += kThreads) {
    sm.hist_mass[bin] = 0;
    sm.hist_count[bin] = 0;
  }
  if (tid == 0) {
    sm.stored_equal = 0;
  }
  if (stashed) {
#pragma unroll 5
    for (int c = tid; c < active; c += kThreads) {
      const int size = __ldg(sizes + c);
      const uint16_t bits = __ldcg(score_bits + c);  // unconditional: both loads are in flight together
      sm.stash_size[c] = size > 0 ? size : 0;
      sm.stash_key[c] = size > 0 ? ordered_key16(bits) : 0;
    }
  }
  __syncthreads();

  auto item = [&](int c, int& size, int& key) {
    if (stashed) {
      size = sm.stash_size[c];
      key = sm.stash_key[c];
    } else {
      size = sizes[c];
      key = size > 0 ? ordered_key16(__ldcg(score_bits + c)) : 0;
      size = size > 0 ? size : 0;
    }
  };

  // A histogram pass.  Scores crowd into a few bins, so atomics on one shared pair of
  // histograms would queue up behind each other across all warps: every warp counts
  // into a histogram of its own (sm.warp_mass / sm.warp_count, when the caller provides
  // them) and the copies are summed afterwards.
  constexpr int kWarps = kThreads / 32;
  const bool privatized = sm.warp_mass != nullptr;
  auto histogram = [&](auto&& bin_of) {
    if (privatized) {
      for (int i = tid; i < kWarps * 256; i += kThreads) {
        sm.warp_mass[i] = 0;
        sm.warp_count[i] = 0;
      }
      __syncthreads();
    }
    int* mass = privatized ? sm.warp_mass + (tid >> 5) * 256 : sm.hist_mass;
    int* count = privatized ? sm.warp_count + (tid >> 5) * 256 : sm.hist_count;
    for (int c = tid; c < active; c += kThreads) {
      int size, key;
      item(c, size, key);
      const int bin = bin_of(key);
      if (size > 0 && bin >= 0) {
        atomicAdd(&mass[bin], size);
        atomicAdd(&count[bin], 1);
      }
    }
    __syncthreads();
    if (privatized) {
      for (int bin = tid; bin < 256; bin += kThreads) {
        int total_mass = 0, total_count = 0;
#pragma unroll 8
        for (int w = 0; w < kWarps; ++w) {
          total_mass += sm.warp_mass[w * 256 + bin];
          total_count += sm.warp_count[w * 256 + bin];
        }
        sm.hist_mass[bin] = total_mass;
        sm.hist_count[bin] = total_count;
      }
      __syncthreads();
    }
  };

  // Pass 1: histogram of the high key byte, weighted by community size.
  histogram([](int key) { return key >> 8; });
  if (tid < 32) {
    find_threshold_bin(sm.hist_mass, sm.hist_count, budget, limit, 0, 0, &sm.bin, &sm.mass, &sm.count);
  }
  __syncthreads();
  const int high_bin = sm.bin;
  const int mass_above = sm.mass;
  const int count_above = sm.count;
  __syncthreads();
  for (int bin = tid; bin < 256; bin += kThreads) {
    sm.hist_mass[bin] = 0;
    sm.hist_count[bin] = 0;
  }
  __syncthreads();
  // Pass 2: histogram of the low byte inside the chosen high bin.
  histogram([high_bin](int key) { return (key >> 8) == high_bin ? (key & 0xff) : -1; });
  if (tid < 32) {
    find_threshold_bin(sm.hist_mass, sm.hist_count, budget, limit, mass_above, count_above, &sm.bin,
                       &sm.mass, &sm.count);
  }
  __syncthreads();
  const int threshold = (high_bin << 8) | sm.bin;

  // Pass 3: per-thread totals over a contiguous run of communities, then an
  // index-ordered exclusive scan.
  const int per_thread = (active + kThreads - 1) / kThreads;
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
  Quad prefix = block_scan<kThreads / 32>(mine, sm.scan_scratch, &sm.scan_total);
  const int total_high_count = sm.scan_total.high_count;
  const int total_high_mass = sm.scan_total.high_mass;

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
        if (write_outputs) {
          out_comm[descriptor] = c;
          out_ends[descriptor] = prefix.high_mass;
        }
        if (descriptor < kDescStash) {
          sm.desc_comm[descriptor] = c;
          sm.desc_end[descriptor] = prefix.high_mass;
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
          if (write_outputs) {
            out_comm[rank] = c;
            out_ends[rank] = min(budget, start + size);
          }
          if (rank < kDescStash) {
            sm.desc_comm[rank] = c;
            sm.desc_end[rank] = min(budget, start + size);
          }
        }
        stored_equal += 1;
      }
    }
  }
  if (stored_equal > 0) {
    atomicAdd(&sm.stored_equal, stored_equal);
  }
  __syncthreads();
  if (tid == 0) {
    const int descriptors = min(a.descriptor_capacity, total_high_count + sm.stored_equal);
    sm.descriptors = descriptors;
    if (write_outputs) {
      a.descriptor_counts[flat] = descriptors;
    }
    if (write_outputs && a.threshold_state != nullptr) {
      a.threshold_state[static_cast<int64_t>(flat) * 4] = threshold;
    }
  }
  __syncthreads();
  const int descriptors = sm.descriptors;
  const bool in_smem = descriptors <= kDescStash;
  const int32_t* search_ends = in_smem ? sm.desc_end : out_ends;
  const int32_t* search_comm = in_smem ? sm.desc_comm : out_comm;

  resolve_tokens<kThreads>(a, flat, u, search_ends, search_comm, descriptors, write_outputs, token_begin,
                           token_end);
}


// ---- selection spread over a thread-block cluster ----
//
// The CTAs of a cluster own contiguous, index-ordered slices of the unit's
// communities (the rows each one scored).  Histograms and per-slice totals are
// summed by reading the other CTAs' shared memory; every CTA ends up with the
// complete descriptor list in its own shared memory, written there by the slices'
// owners.  Same result as select_unit.
__device__ __forceinline__ uint32_t cluster_address(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ int cluster_load(uint32_t address) {
  int value;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(value) : "r"(address) : "memory");
  return value;
}
__device__ __forceinline__ void cluster_store(uint32_t address, int value) {
  asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}
__device__ __forceinline__ void cluster_add(uint32_t address, int value) {
  asm volatile("red.shared::cluster.add.s32 [%0], %1;" ::"r"(address), "r"(value) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

constexpr int kClusterStageBytes = 2 * 16 * kHeadDim * 4 + 2 * kDescStash * 4;  // 32 KB

struct ClusterSelectSmem {
  // Staging area of the scoring phase (query group as fp32 pairs, or a ring of e4m3
  // row groups); the descriptor list, which is only written after every CTA of the
  // cluster has finished scoring, is part of it.
  alignas(128) float query[2 * 16 * kHeadDim];
  int32_t desc_comm[kDescStash];  // the complete list, filled by every slice's owner
  int32_t desc_end[kDescStash];
  uint16_t key[kStash];   // this CTA's slice
  int size[kStash];
  int hist_mass[256];     // slice histograms, read by the other CTAs
  int hist_count[256];
  int low_mass[256];
  int low_count[256];
  int sum_mass[256];      // cluster-wide sums (private)
  int sum_count[256];
  int before_mass[256];   // sums over the slices in front of this one (private)
  int before_count[256];
  Quad scan_scratch[32];
  Quad scan_total;
  int stored_equal;       // stored at-threshold communities of all slices (every owner adds here)
  int bin, mass, count, front_mass, front_count, descriptors;
};
static_assert(offsetof(ClusterSelectSmem, key) == kClusterStageBytes, "staging area must be contiguous");

// Zeroes what scoring accumulates into; call before score_groups, followed by a
// block barrier (score_groups starts with one).
template <int kThreads>
__device__ __forceinline__ void cluster_select_begin(ClusterSelectSmem& sm) {
  for (int bin = threadIdx.x; bin < 256; bin += kThreads) {
    sm.hist_mass[bin] = 0;
    sm.hist_count[bin] = 0;
    sm.low_mass[bin] = 0;
    sm.low_count[bin] = 0;
  }
  if (threadIdx.x == 0) {
    sm.stored_equal = 0;
  }
}

// `row0`, `rows`: this CTA's slice (rows it scored; the stash and the first-pass
// histogram are already filled by score_groups).  Every CTA of the cluster calls
// this; on return sm.desc_* hold all descriptors and the logical tokens
// [token_begin, token_end) are resolved to cache rows.
// `guess_bin`: the high-byte bin score_groups counted the low bytes of (-1: none).
template <int kThreads>
__device__ __forceinline__ void select_cluster(const ckv_layer_args& a, int flat, ClusterSelectSmem& sm,
                                               int rank, int ranks, int row0, int rows,
                                               int token_begin, int token_end, int guess_bin) {
  const Unit u = make_unit(a, flat);
  const int tid = threadIdx.x;
  const int capacity = a.community_capacity;
  const int active = max(0, min(capacity, a.community_counts[flat]));
  const int budget = a.token_budget - a.num_sink - 1;
  const int limit = a.max_communities;
  // The last slice also takes any active rows beyond the scored cover (there are none when
  // the cover is the initial count plus the decode headroom).  They must fit its stash:
  // what does not is left out and reported in the status word.
  if (rank == ranks - 1 && active > row0 + rows) {
    const uint16_t* score_bits =
        reinterpret_cast<const uint16_t*>(a.scores) + static_cast<int64_t>(flat) * capacity;
    const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
    int active_here = active;
    if (active - row0 > kStash) {
      active_here = row0 + kStash;
      if (tid == 0 && a.status != nullptr) {
        atomicOr(a.status, CKV_DEV_STASH_OVERFLOW);
      }
    }
    for (int c = row0 + rows + tid; c < active_here; c += kThreads) {
      const int size = __ldg(sizes + c);
      const int key = size > 0 ? ordered_key16(__ldcg(score_bits + c)) : 0;
      sm.size[c - row0] = size > 0 ? size : 0;
      sm.key[c - row0] = static_cast<uint16_t>(key);
      if (size > 0) {
        atomicAdd(&sm.hist_mass[key >> 8], size);
        atomicAdd(&sm.hist_count[key >> 8], 1);
        if ((key >> 8) == guess_bin) {
          atomicAdd(&sm.low_mass[key & 0xff], size);
          atomicAdd(&sm.low_count[key & 0xff], 1);
        }
      }
    }
    rows = active_here - row0;
  }
  rows = max(0, min(rows, active - row0));
  cluster_sync_all();  // every slice's first-pass histogram is complete
  phase_stamp(a, flat, rank, 2);

  // Sum a pair of 256-bin histograms over the cluster.  Each thread owns
  // 256 / kThreads bins and keeps every slice's values in registers: once the
  // threshold bin is known they also give the totals above it, for all slices and
  // for the slices before this one, without another exchange.
  constexpr int kBins = 256 / kThreads;
  static_assert(kBins * kThreads == 256, "thread count must divide 256");
  // Sum a pair of 256-bin histograms over the cluster.  Each thread owns 256 / kThreads
  // bins and reads every slice's values (all loads in flight together); it writes the sum
  // over all slices and the sum over the slices in front of this one.
  constexpr int kMaxRanks = 8;
  auto gather = [&](const int* mass, const int* count) {
    int part_mass[kBins][kMaxRanks];
    int part_count[kBins][kMaxRanks];
#pragma unroll
    for (int k = 0; k < kBins; ++k) {
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        const bool present = r < ranks;
        part_mass[k][r] = present ? cluster_load(cluster_address(mass + tid + k * kThreads, r)) : 0;
        part_count[k][r] = present ? cluster_load(cluster_address(count + tid + k * kThreads, r)) : 0;
      }
    }
#pragma unroll
    for (int k = 0; k < kBins; ++k) {
      int total_mass = 0, total_count = 0, before_mass = 0, before_count = 0;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        total_mass += part_mass[k][r];
        total_count += part_count[k][r];
        if (r < rank) {
          before_mass += part_mass[k][r];
          before_count += part_count[k][r];
        }
      }
      sm.sum_mass[tid + k * kThreads] = total_mass;
      sm.sum_count[tid + k * kThreads] = total_count;
      sm.before_mass[tid + k * kThreads] = before_mass;
      sm.before_count[tid + k * kThreads] = before_count;
    }
    __syncthreads();
  };
  // Warp 0: the threshold bin of the summed histogram, the totals above it, and the totals
  // above it of the slices in front of this one.
  auto find = [&](int start_mass, int start_count) {
    if (tid < 32) {
      find_threshold_bin(sm.sum_mass, sm.sum_count, budget, limit, start_mass, start_count, &sm.bin,
                         &sm.mass, &sm.count);
      __syncwarp();
      const int bin = sm.bin;
      int mass = 0, count = 0;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (tid * 8 + b > bin) {
          mass += sm.before_mass[tid * 8 + b];
          count += sm.before_count[tid * 8 + b];
        }
      }
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        mass += __shfl_xor_sync(0xffffffffu, mass, offset);
        count += __shfl_xor_sync(0xffffffffu, count, offset);
      }
      if (tid == 0) {
        sm.front_mass = mass;
        sm.front_count = count;
      }
    }
    __syncthreads();
  };

  gather(sm.hist_mass, sm.hist_count);
  find(0, 0);
  const int high_bin = sm.bin;
  const int mass_above = sm.mass;
  const int count_above = sm.count;
  const int coarse_front_mass = sm.front_mass;
  const int coarse_front_count = sm.front_count;
  __syncthreads();  // the find results are read before the next find overwrites them
  // Pass 2: low byte inside the chosen high bin, this slice only - unless scoring has
  // already counted exactly that bin (every CTA sees the same high bin and the same guess,
  // so all of them take the same branch, and the slices' low histograms were complete at
  // the barrier above: no second barrier is needed then).
  if (high_bin != guess_bin) {
    if (guess_bin >= 0) {
      for (int bin = tid; bin < 256; bin += kThreads) {
        sm.low_mass[bin] = 0;
        sm.low_count[bin] = 0;
      }
      __syncthreads();
    }
    for (int i = tid; i < rows; i += kThreads) {
      const int size = sm.size[i];
      const int key = sm.key[i];
      if (size > 0 && (key >> 8) == high_bin) {
        atomicAdd(&sm.low_mass[key & 0xff], size);
        atomicAdd(&sm.low_count[key & 0xff], 1);
      }
    }
    cluster_sync_all();
  }
  phase_stamp(a, flat, rank, 3);
  gather(sm.low_mass, sm.low_count);
  find(mass_above, count_above);
  const int low_bin = sm.bin;
  const int threshold = (high_bin << 8) | low_bin;
  // above the threshold: all slices (the search counted on from the coarse totals), and the
  // slices in front of this one; at the threshold: the slices in front of this one
  const int total_high_count = sm.count;
  const int total_high_mass = sm.mass;
  const Quad before = {coarse_front_count + sm.front_count, coarse_front_mass + sm.front_mass,
                       sm.before_count[low_bin], sm.before_mass[low_bin]};

  // Pass 3: this slice in index order.
  const int per_thread = (rows + kThreads - 1) / kThreads;
  const int first = min(rows, tid * per_thread);
  const int last = min(rows, first + per_thread);
  Quad mine = {0, 0, 0, 0};
  for (int i = first; i < last; ++i) {
    const int size = sm.size[i];
    const int key = sm.key[i];
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
  Quad prefix = block_scan<kThreads / 32>(mine, sm.scan_scratch, &sm.scan_total);
  prefix = quad_add(prefix, before);

  // Pass 4: this slice's descriptors, to the workspace and to every CTA's list.
  int32_t* out_comm = a.communities + static_cast<int64_t>(flat) * a.descriptor_capacity;
  int32_t* out_ends = a.cumulative_ends + static_cast<int64_t>(flat) * a.descriptor_capacity;
  auto publish = [&](int descriptor, int community, int end) {
    if (descriptor < a.descriptor_capacity) {
      out_comm[descriptor] = community;
      out_ends[descriptor] = end;
      if (descriptor < kDescStash) {
        for (int r = 0; r < ranks; ++r) {
          cluster_store(cluster_address(sm.desc_comm + descriptor, r), community);
          cluster_store(cluster_address(sm.desc_end + descriptor, r), end);
        }
      }
    }
  };
  int stored_equal = 0;
  for (int i = first; i < last; ++i) {
    const int size = sm.size[i];
    const int key = sm.key[i];
    if (size <= 0) {
      continue;
    }
    if (key > threshold) {
      const int descriptor = prefix.high_count;
      prefix.high_count += 1;
      prefix.high_mass += size;
      publish(descriptor, row0 + i, prefix.high_mass);
    } else if (key == threshold) {
      const int start = total_high_mass + prefix.equal_mass;
      const int position = total_high_count + prefix.equal_count;
      prefix.equal_count += 1;
      prefix.equal_mass += size;
      if (start < budget && (limit <= 0 || position < limit)) {
        publish(position, row0 + i, min(budget, start + size));
        stored_equal += 1;
      }
    }
  }
  if (stored_equal > 0) {
    // counted into every CTA's own counter: nothing reads another CTA's shared
    // memory after the barrier below, so a CTA may move on and reuse its own
    for (int r = 0; r < ranks; ++r) {
      cluster_add(cluster_address(&sm.stored_equal, r), stored_equal);
    }
  }
  cluster_sync_all();  // the lists are complete everywhere
  phase_stamp(a, flat, rank, 4);
  if (tid == 0) {
    const int descriptors = min(a.descriptor_capacity, total_high_count + sm.stored_equal);
    sm.descriptors = descriptors;
    if (rank == 0) {
      a.descriptor_counts[flat] = descriptors;
      if (a.threshold_state != nullptr) {
        a.threshold_state[static_cast<int64_t>(flat) * 4] = threshold;
      }
    }
  }
  __syncthreads();
  const int descriptors = sm.descriptors;
  phase_stamp(a, flat, rank, 5);
  // The shared-memory list holds the first kDescStash descriptors; a longer list (a large
  // budget spent on very small communities) is searched in the workspace, where every
  // slice's owner stored it before the barrier above.
  const bool in_smem = descriptors <= kDescStash;
  const int32_t* search_ends = in_smem ? sm.desc_end : out_ends;
  const int32_t* search_comm = in_smem ? sm.desc_comm : out_comm;

  resolve_tokens<kThreads>(a, flat, u, search_ends, search_comm, descriptors, rank == 0, token_begin,
                           token_end);
}

}  // namespace ckv
