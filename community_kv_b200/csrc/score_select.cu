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

#include "score_select.cuh"

namespace ckv {

__global__ void __launch_bounds__(kScoreThreads, 2) score_kernel(const ckv_layer_args a) {
  // query group as fp32, every value stored twice, or one staged e4m3 row group per warp
  // (see score_groups)
  constexpr int kStageBytes = (kScoreThreads / 32) * (16 * kHeadDim + 64);
  static_assert(kStageBytes >= 2 * 16 * kHeadDim * 4, "the staging area also holds the fp32 query group");
  __shared__ __align__(128) float q_s[kStageBytes / 4];
  __shared__ int prefix[kScoreMaxUnits + 1];
  const int units = a.batch * a.retrieval_heads;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
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
  for (; flat < units && prefix[flat] < my_end; ++flat) {
    const int first_group = max(my_begin, prefix[flat]) - prefix[flat];
    const int last_group = min(my_end, prefix[flat + 1]) - prefix[flat];
    if (first_group >= last_group) {
      continue;
    }
    score_groups<kScoreThreads, kStageBytes>(a, flat, first_group, last_group, q_s);
  }
}

// fp32 centroid table (CKV_FLAG_FP32_CENTROIDS).  Eight lanes share one centroid row, 16
// dimensions each; every product and every sum is rounded on its own (multiply, then add),
// in the order of the e4m3 path - 16 sequential terms per lane, then lanes (j, j^4),
// (j, j^2), (j, j^1) - so that a CPU reproduces the fp16 score bit for bit.
constexpr int kScoreFp32Threads = 256;

__global__ void __launch_bounds__(kScoreFp32Threads) score_fp32_kernel(const ckv_layer_args a) {
  const int flat = blockIdx.y;
  const int capacity = a.community_capacity;
  const int limit = score_limit(a, flat);
  const int row = blockIdx.x * (kScoreFp32Threads / 8) + (threadIdx.x >> 3);
  const int slice = threadIdx.x & 7;
  const int safe_row = min(row, capacity - 1);  // every lane takes part in the shuffles below
  const float4* source = reinterpret_cast<const float4*>(
      reinterpret_cast<const float*>(a.centroids) +
      (static_cast<int64_t>(flat) * capacity + safe_row) * kHeadDim + slice * 16);
  float x[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = source[i];
    x[4 * i] = v.x;
    x[4 * i + 1] = v.y;
    x[4 * i + 2] = v.z;
    x[4 * i + 3] = v.w;
  }
  const int group = a.group_size;
  const __nv_bfloat16* query = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                               static_cast<int64_t>(flat) * group * kHeadDim + slice * 16;
  float best = -INFINITY;
  for (int g = 0; g < group; ++g) {
    const __nv_bfloat16* q = query + g * kHeadDim;
    float acc = __fmul_rn(x[0], __bfloat162float(q[0]));
#pragma unroll
    for (int k = 1; k < 16; ++k) {
      acc = __fadd_rn(acc, __fmul_rn(x[k], __bfloat162float(q[k])));
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    best = fmaxf(best, acc);
  }
  if (slice == 0 && row < limit) {
    const bool live = row < a.community_counts[flat] &&
                      a.community_sizes[static_cast<int64_t>(flat) * capacity + row] > 0;
    reinterpret_cast<__half*>(a.scores)[static_cast<int64_t>(flat) * capacity + row] =
        __float2half_rn(live ? best : -INFINITY);
  }
}

// Dynamic shared memory: one 256-bin (mass, count) histogram per warp, then the key/size
// stash of `stash_capacity` entries (sizes first).
constexpr int kSelectWarpHistBytes = (kSelectThreads / 32) * 256 * 2 * static_cast<int>(sizeof(int));

__global__ void __launch_bounds__(kSelectThreads, 1) select_kernel(const ckv_layer_args a,
                                                                    int stash_capacity) {
  __shared__ SelectSmem sm;
  extern __shared__ __align__(16) uint8_t dynamic[];
  if (threadIdx.x == 0) {
    sm.warp_mass = reinterpret_cast<int*>(dynamic);
    sm.warp_count = sm.warp_mass + (kSelectThreads / 32) * 256;
    uint8_t* stash = dynamic + kSelectWarpHistBytes;
    sm.stash_size = reinterpret_cast<int*>(stash);
    sm.stash_key = reinterpret_cast<uint16_t*>(stash + static_cast<size_t>(stash_capacity) * sizeof(int));
    sm.stash_capacity = stash_capacity;
  }
  __syncthreads();
  pdl_release_dependents();
  pdl_wait_for_predecessor();  // the fp16 scores come from the scoring kernel
  select_unit<kSelectThreads>(a, blockIdx.x, sm, true, 0, a.token_budget);
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
  if (a.flags & CKV_FLAG_FP32_CENTROIDS) {
    const dim3 grid((a.community_capacity + kScoreFp32Threads / 8 - 1) / (kScoreFp32Threads / 8), units);
    score_fp32_kernel<<<grid, kScoreFp32Threads, 0, stream>>>(a);
    return cudaGetLastError();
  }
  if (units > kScoreMaxUnits) {
    return cudaErrorInvalidConfiguration;
  }
  const long long finest = static_cast<long long>(units) * ((a.community_capacity + 127) / 128);
  const int grid = finest < 1 ? 1 : (finest > 2 * 148 ? 2 * 148 : static_cast<int>(finest));
  return launch_dependent(score_kernel, dim3(grid), dim3(kScoreThreads), 0, stream, a);
}

cudaError_t launch_select(const ckv_layer_args& a, cudaStream_t stream) {
  // Stage every community's key and size in shared memory when they fit (6 bytes each;
  // one CTA per SM, so up to kSelectStashMax communities); beyond that the kernel re-reads
  // them from global memory in every pass.
  constexpr int kSelectStashMax = 20480;
  constexpr int kSelectStashBytes = kSelectStashMax * 6 + kSelectWarpHistBytes;
  static bool configured[64] = {};
  const int device = a.device >= 0 && a.device < 64 ? a.device : 0;
  if (!configured[device]) {
    const cudaError_t err =
        cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelectStashBytes);
    if (err != cudaSuccess) return err;
    configured[device] = true;
  }
  int capacity = ((a.community_capacity + 7) / 8) * 8;
  if (capacity > kSelectStashMax) capacity = kStash;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a.batch * a.retrieval_heads);
  config.blockDim = dim3(kSelectThreads);
  config.dynamicSmemBytes = static_cast<size_t>(capacity) * 6 + kSelectWarpHistBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, select_kernel, a, capacity);
}

cudaError_t launch_resolve(const ckv_layer_args& a, cudaStream_t stream) {
  const dim3 grid((a.token_budget + 255) / 256, a.batch * a.retrieval_heads);
  resolve_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace ckv
