// Split merge (log-sum-exp) + online community assignment + centroid maintenance.
//
// One CTA of 160 threads per (sequence, retrieval head).  Each of the first four
// warps merges the split partials of one query head at a time with independent
// 16-byte loads.  The fifth warp of the CTA whose head leads its graph merges the per-split
// neighbour candidates into the global top-8, applies the modularity-gain rule
// and updates the graph state in place; it is the single writer of that graph.

#include "merge_update.cuh"

namespace ckv {

__global__ void __launch_bounds__(kMergeThreads + 32) merge_update_kernel(const ckv_layer_args a) {
  __shared__ UpdateDecision decision;
  __shared__ float lse_s;
  pdl_release_dependents();
  pdl_wait_for_predecessor();  // partials and candidates come from the attention kernel
  merge_update_unit(a, blockIdx.x, kMergeThreads / 32, decision, lse_s);
  if (blockIdx.x == 0) {
    wait_for_peer_rows(a);
  }
}

// Follower heads of a graph shared by several retrieval heads: apply the
// leader's assignment to their own centroid table.
__global__ void __launch_bounds__(kMergeThreads) sync_shared_kernel(const ckv_layer_args a) {
  const int flat = blockIdx.x;
  const Unit u = make_unit(a, flat);
  if (u.head == u.graph) {
    return;
  }
  const int d = threadIdx.x;
  const int capacity = a.community_capacity;
  const int64_t graph_slot = static_cast<int64_t>(u.batch) * a.graphs + u.graph;
  const int community = a.assigned[graph_slot];
  if (a.overflow[graph_slot] != 0 || community < 0) {
    return;
  }
  const int current = a.current_position[graph_slot] - 1;
  const int64_t size_index = static_cast<int64_t>(flat) * capacity + community;
  const int old_size = a.community_sizes[size_index];
  __syncthreads();
  if (d == 0) {
    a.community_sizes[size_index] = old_size + 1;
    a.community_counts[flat] =
        a.community_counts[static_cast<int64_t>(u.batch) * a.retrieval_heads + u.graph];
  }
  if (current >= 0 && current < a.sequence_capacity) {
    __nv_fp8_storage_t* centroid = reinterpret_cast<__nv_fp8_storage_t*>(a.centroids) +
                                   size_index * kHeadDim;
    const __nv_bfloat16* key_row =
        a.current_key != nullptr
            ? reinterpret_cast<const __nv_bfloat16*>(a.current_key) + static_cast<int64_t>(flat) * kHeadDim
            : reinterpret_cast<const __nv_bfloat16*>(a.key) + u.batch * a.key_batch_stride +
                  u.kv * a.key_head_stride + static_cast<int64_t>(current) * a.key_row_stride;
    const float key_value = __bfloat162float(key_row[d]);
    if (a.flags & CKV_FLAG_FP32_CENTROIDS) {
      float* wide = reinterpret_cast<float*>(a.centroids) + size_index * kHeadDim + d;
      *wide = old_size > 0 ? centroid_mean(*wide, old_size, key_value,
                                           (a.flags & CKV_FLAG_REFERENCE_DIVISION) != 0)
                           : key_value;
      return;
    }
    float updated = key_value;
    if (old_size > 0) {
      const __half_raw raw = __nv_cvt_fp8_to_halfraw(centroid[d], __NV_E4M3);
      const float old_value = __half2float(*reinterpret_cast<const __half*>(&raw));
      updated = centroid_mean(old_value, old_size, key_value, (a.flags & CKV_FLAG_REFERENCE_DIVISION) != 0);
    }
    centroid[d] = __nv_cvt_float_to_fp8(updated, __NV_SATFINITE, __NV_E4M3);
  }
}

// One warp per unit: lanes 0-15 copy the 256-byte key row, lanes 16-31 the value row.
__global__ void __launch_bounds__(128) append_kv_kernel(uint4* key_cache, uint4* value_cache,
                                                        const uint4* new_key, const uint4* new_value,
                                                        int64_t units, int64_t unit_stride_vec,
                                                        const int32_t* row_index, int64_t row_index_stride,
                                                        int64_t row) {
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (unit >= units) {
    return;
  }
  const int lane = threadIdx.x & 31;
  const int64_t target = row_index != nullptr ? row_index[unit * row_index_stride] : row;
  if (target < 0) {
    return;
  }
  const int piece = lane & 15;
  uint4* cache = lane < 16 ? key_cache : value_cache;
  const uint4* fresh = lane < 16 ? new_key : new_value;
  cache[unit * unit_stride_vec + target * (kHeadDim * 2 / 16) + piece] = fresh[unit * (kHeadDim * 2 / 16) + piece];
}

cudaError_t launch_append_kv(void* key_cache, void* value_cache, const void* new_key, const void* new_value,
                             int64_t units, int64_t unit_stride, const int32_t* row_index,
                             int64_t row_index_stride, int64_t row, cudaStream_t stream) {
  append_kv_kernel<<<static_cast<unsigned>((units + 3) / 4), 128, 0, stream>>>(
      static_cast<uint4*>(key_cache), static_cast<uint4*>(value_cache), static_cast<const uint4*>(new_key),
      static_cast<const uint4*>(new_value), units, unit_stride / 8, row_index, row_index_stride, row);
  return cudaGetLastError();
}

// One thread polls this GPU's counter a bounded number of times.
// Launched with programmatic stream serialisation: it may start (and poll) while the
// kernel before it in the stream is still running, and it only ends once that kernel
// has completed, so whatever follows sees both the local and the peers' rows.
__global__ void wait_peers_kernel(uint32_t* flag, uint32_t expected, uint32_t* status) {
  pdl_release_dependents();
  constexpr uint32_t kPolls = 1u << 22;  // about two seconds with the back-off below
  bool arrived = false;
  for (uint32_t poll = 0; poll < kPolls; ++poll) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen >= expected) {
      atomicSub(flag, expected);
      arrived = true;
      break;
    }
    if (poll > 256) {
      __nanosleep(500);
    }
  }
  if (!arrived && status != nullptr) {
    atomicOr(status, CKV_DEV_WAIT_TIMEOUT);
  }
  pdl_wait_for_predecessor();
}

cudaError_t launch_wait_peers(uint32_t* flag, uint32_t expected, uint32_t* status, cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(1);
  config.blockDim = dim3(1);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, wait_peers_kernel, flag, expected, status);
}

// Nearest-centroid assignment variant: per leader head, the live community whose centroid
// has the largest inner product with the key of the token being decoded (the fp16 value the
// scoring kernel would give a query group made of that key; first maximum).  One CTA per
// retrieval head; eight lanes share a centroid row, every product and sum rounded on its own
// in the scoring kernels' fixed order, so a CPU reproduces the choice bit for bit.
constexpr int kNearestThreads = 256;

__global__ void __launch_bounds__(kNearestThreads) nearest_centroid_kernel(const ckv_layer_args a,
                                                                          int32_t* forced) {
  __shared__ unsigned long long warp_best[kNearestThreads / 32];
  const int flat = blockIdx.x;
  const Unit u = make_unit(a, flat);
  if (u.head != u.graph) {
    return;  // followers of a shared graph take the leader's choice
  }
  const int capacity = a.community_capacity;
  const int64_t graph_slot = static_cast<int64_t>(u.batch) * a.graphs + u.graph;
  const int current = min(max(a.current_position[graph_slot], 0), a.sequence_capacity - 1);
  const __nv_bfloat16* key_row =
      a.current_key != nullptr
          ? reinterpret_cast<const __nv_bfloat16*>(a.current_key) + static_cast<int64_t>(flat) * kHeadDim
          : reinterpret_cast<const __nv_bfloat16*>(a.key) + u.batch * a.key_batch_stride +
                u.kv * a.key_head_stride + static_cast<int64_t>(current) * a.key_row_stride;
  const int slice = threadIdx.x & 7;
  float q[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    q[k] = __bfloat162float(key_row[slice * 16 + k]);
  }
  const bool wide = (a.flags & CKV_FLAG_FP32_CENTROIDS) != 0;
  const int count = min(a.community_counts[flat], capacity);
  const int32_t* sizes = a.community_sizes + static_cast<int64_t>(flat) * capacity;
  unsigned long long best = 0ull;  // (ordered fp16 key + 1) << 32 | ~row : the first maximum wins
  for (int base = 0; base < count; base += kNearestThreads / 8) {
    const int row = base + (threadIdx.x >> 3);
    const int safe_row = min(row, capacity - 1);  // every lane takes part in the shuffles
    float x[16];
    if (wide) {
      const float4* source = reinterpret_cast<const float4*>(
          reinterpret_cast<const float*>(a.centroids) +
          (static_cast<int64_t>(flat) * capacity + safe_row) * kHeadDim + slice * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 v = source[i];
        x[4 * i] = v.x;
        x[4 * i + 1] = v.y;
        x[4 * i + 2] = v.z;
        x[4 * i + 3] = v.w;
      }
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint8_t*>(a.centroids) +
          (static_cast<int64_t>(flat) * capacity + safe_row) * kHeadDim + slice * 16);
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const __half_raw half = __nv_cvt_fp8_to_halfraw(
            static_cast<__nv_fp8_storage_t>((words[k >> 2] >> (8 * (k & 3))) & 0xffu), __NV_E4M3);
        x[k] = __half2float(*reinterpret_cast<const __half*>(&half));
      }
    }
    float acc = __fmul_rn(x[0], q[0]);
#pragma unroll
    for (int k = 1; k < 16; ++k) {
      acc = __fadd_rn(acc, __fmul_rn(x[k], q[k]));
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    if (row < count && sizes[row] > 0) {
      uint16_t bits = __half_as_ushort(__float2half_rn(acc));
      bits = bits == 0x8000u ? 0u : bits;  // -0 and +0 compare equal
      const unsigned long long key = static_cast<unsigned long long>(ordered_key16(bits)) + 1ull;
      const unsigned long long packed = (key << 32) | (0xffffffffull - static_cast<unsigned long long>(row));
      best = packed > best ? packed : best;
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, offset);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) {
    warp_best[threadIdx.x >> 5] = best;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kNearestThreads / 32; ++w) {
      best = warp_best[w] > best ? warp_best[w] : best;
    }
    forced[graph_slot] =
        best == 0ull ? -1 : static_cast<int32_t>(0xffffffffull - (best & 0xffffffffull));
  }
}

cudaError_t launch_nearest_centroid(const ckv_layer_args& a, int32_t* forced, cudaStream_t stream) {
  nearest_centroid_kernel<<<a.batch * a.retrieval_heads, kNearestThreads, 0, stream>>>(a, forced);
  return cudaGetLastError();
}

cudaError_t launch_merge_update(const ckv_layer_args& a, cudaStream_t stream) {
  cudaError_t err = launch_dependent(merge_update_kernel, dim3(a.batch * a.retrieval_heads),
                                     dim3(kMergeThreads + 32), 0, stream, a);
  if (err != cudaSuccess) {
    return err;
  }
  if (a.retrieval_heads != a.graphs && !(a.flags & CKV_FLAG_SKIP_UPDATE)) {
    sync_shared_kernel<<<a.batch * a.retrieval_heads, kMergeThreads, 0, stream>>>(a);
    err = cudaGetLastError();
  }
  return err;
}

}  // namespace ckv
