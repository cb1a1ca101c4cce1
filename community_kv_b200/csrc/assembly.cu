// Decode-state assembly from community labels (sm_100a): the step between a finished
// partition and the first decode step.
//
//   ckv_assemble_member_csr   per graph, the non-sink positions grouped by community
//                             (ascending id) and ordered newest first inside a community,
//                             plus the CSR offsets
//                             (reference: build_member_csr, community_kv/graph/partition.py:457-492)
//   ckv_assemble_centroids    per retrieval head, the mean key of every community as
//                             saturating e4m3, and the community sizes
//                             (reference: compute_centroids, partition.py:382-455)
//   ckv_assemble_modularity   per graph, the community weights and the total weight of an
//                             edge list (reference: init_modularity_state, partition.py:495-535)
//
// All integer results are exact.  The member lists are produced without a sort: a warp
// owns a few communities and sweeps the label row from its end, compacting the matching
// positions with a ballot - the order (position descending) falls out of the sweep, and
// the label row (a few hundred KB) stays in L2 for all the warps that read it.  The
// centroid sums are accumulated in ascending position order by ONE lane per dimension,
// which is the order a sequential scatter-add visits the rows, so the e4m3 result is
// reproducible bit for bit; only the modularity weights (floating-point sums over an
// unordered edge list) depend on the order of the atomics, to fp32 rounding.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ckv_b200.h"

namespace ckv {
namespace {

constexpr int kLabelsPerWarp = 4;
constexpr int kFillWarps = 8;

// counts[g][c] = number of non-sink positions of graph g labelled c
__global__ void __launch_bounds__(256) label_count_kernel(const int32_t* labels, int graphs, int length,
                                                          int num_sink, int communities, int32_t* counts) {
  const int graph = blockIdx.y;
  const int32_t* row = labels + static_cast<int64_t>(graph) * length;
  for (int p = num_sink + blockIdx.x * blockDim.x + threadIdx.x; p < length; p += gridDim.x * blockDim.x) {
    const int label = row[p];
    if (label >= 0 && label < communities) {
      atomicAdd(&counts[static_cast<int64_t>(graph) * communities + label], 1);
    }
  }
}

// offsets[g][0..communities] = exclusive prefix of counts[g]; one CTA per graph
__global__ void __launch_bounds__(1024) offsets_scan_kernel(const int32_t* counts, int communities,
                                                            int32_t* offsets) {
  __shared__ int warp_total[32];
  __shared__ int carry;
  const int graph = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int32_t* in = counts + static_cast<int64_t>(graph) * communities;
  int32_t* out = offsets + static_cast<int64_t>(graph) * (communities + 1);
  if (threadIdx.x == 0) {
    carry = 0;
    out[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < communities; base += 1024) {
    const int index = base + threadIdx.x;
    const int value = index < communities ? in[index] : 0;
    int inclusive = value;
#pragma unroll
    for (int delta = 1; delta < 32; delta <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, inclusive, delta);
      if (lane >= delta) inclusive += other;
    }
    if (lane == 31) warp_total[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
      int running = warp_total[lane];
#pragma unroll
      for (int delta = 1; delta < 32; delta <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, running, delta);
        if (lane >= delta) running += other;
      }
      warp_total[lane] = running;  // inclusive over warps
    }
    __syncthreads();
    const int before = carry + (warp > 0 ? warp_total[warp - 1] : 0);
    if (index < communities) {
      out[index + 1] = before + inclusive;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      carry += warp_total[31];
    }
    __syncthreads();
  }
}

// A warp owns kLabelsPerWarp consecutive communities of one graph and sweeps the label row
// from the newest position down; lane i looks at position top - i.
__global__ void __launch_bounds__(kFillWarps * 32) member_fill_kernel(const int32_t* labels, int length,
                                                                      int num_sink, int communities,
                                                                      const int32_t* offsets,
                                                                      int member_capacity,
                                                                      int32_t* member_positions) {
  const int graph = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int first = (blockIdx.x * kFillWarps + warp) * kLabelsPerWarp;
  if (first >= communities) {
    return;
  }
  const int32_t* row = labels + static_cast<int64_t>(graph) * length;
  const int32_t* starts = offsets + static_cast<int64_t>(graph) * (communities + 1);
  int32_t* out = member_positions + static_cast<int64_t>(graph) * member_capacity;
  int cursor[kLabelsPerWarp];
#pragma unroll
  for (int k = 0; k < kLabelsPerWarp; ++k) {
    cursor[k] = first + k < communities ? starts[first + k] : 0;
  }
  const unsigned below = (1u << lane) - 1u;
  for (int top = length - 1; top >= num_sink; top -= 32) {
    const int p = top - lane;
    const int label = p >= num_sink ? __ldg(row + p) : -1;
    const int offset = label - first;
    if (__any_sync(0xffffffffu, offset >= 0 && offset < kLabelsPerWarp)) {
#pragma unroll
      for (int k = 0; k < kLabelsPerWarp; ++k) {
        const unsigned hits = __ballot_sync(0xffffffffu, offset == k);
        if (offset == k) {
          const int slot = cursor[k] + __popc(hits & below);
          if (slot < member_capacity) {
            out[slot] = p;
          }
        }
        cursor[k] += __popc(hits);
      }
    }
  }
}

// One warp per (retrieval head, community); lane l owns dimensions 4l .. 4l+3.
__global__ void __launch_bounds__(256) centroid_kernel(const int32_t* offsets, const int32_t* member_positions,
                                                       int communities, int member_capacity,
                                                       const __nv_bfloat16* keys, int64_t key_head_stride,
                                                       int64_t key_row_stride, const int32_t* retrieval_to_graph,
                                                       const int32_t* retrieval_to_kv, int live, int capacity,
                                                       uint8_t* centroids, int32_t* sizes) {
  const int head = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int community = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (community >= capacity) {
    return;
  }
  const int graph = retrieval_to_graph[head];
  int begin = 0, end = 0;
  if (community < communities) {
    const int32_t* starts = offsets + static_cast<int64_t>(graph) * (communities + 1);
    begin = starts[community];
    end = starts[community + 1];
  }
  const int count = end - begin;
  const int32_t* members = member_positions + static_cast<int64_t>(graph) * member_capacity;
  const __nv_bfloat16* rows = keys + retrieval_to_kv[head] * key_head_stride + 4 * lane;
  float sum[4] = {0.f, 0.f, 0.f, 0.f};
  // the list is newest first; a sequential scatter-add visits the rows oldest first
  for (int base = end - 1; base >= begin; base -= 8) {
    uint2 held[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int index = base - i;
      if (index >= begin) {
        held[i] = __ldg(reinterpret_cast<const uint2*>(rows + static_cast<int64_t>(members[index]) * key_row_stride));
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (base - i >= begin) {
        sum[0] = __fadd_rn(sum[0], __uint_as_float(held[i].x << 16));
        sum[1] = __fadd_rn(sum[1], __uint_as_float(held[i].x & 0xffff0000u));
        sum[2] = __fadd_rn(sum[2], __uint_as_float(held[i].y << 16));
        sum[3] = __fadd_rn(sum[3], __uint_as_float(held[i].y & 0xffff0000u));
      }
    }
  }
  uint32_t packed = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float value = sum[i];
    if (community < live) {
      value = __fdiv_rn(value, static_cast<float>(count > 1 ? count : 1));
    }
    value = fminf(fmaxf(value, -448.0f), 448.0f);
    packed |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
  }
  reinterpret_cast<uint32_t*>(centroids + (static_cast<int64_t>(head) * capacity + community) * CKV_HEAD_DIM)[lane] =
      packed;
  if (lane == 0) {
    sizes[static_cast<int64_t>(head) * capacity + community] = count;
  }
}

__global__ void __launch_bounds__(256) modularity_kernel(const int32_t* labels, int length, int graphs,
                                                         const int64_t* edge_src, const int64_t* edge_dst,
                                                         const float* edge_weight, int64_t edges, int capacity,
                                                         float* community_weight, float* total_weight) {
  for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < edges;
       e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t source = edge_src[e];
    const int64_t destination = edge_dst[e];
    const int64_t graph = source / length;
    if (graph < 0 || graph >= graphs) {
      continue;
    }
    const float weight = edge_weight[e];
    const int from = labels[graph * length + source % length];
    const int to = labels[graph * length + destination % length];
    if (from >= 0 && from < capacity) atomicAdd(&community_weight[graph * capacity + from], weight);
    if (to >= 0 && to < capacity) atomicAdd(&community_weight[graph * capacity + to], weight);
    atomicAdd(&total_weight[graph], 2.0f * weight);
  }
}

int launched() { return cudaGetLastError() == cudaSuccess ? CKV_OK : CKV_ERR_LAUNCH; }

}  // namespace
}  // namespace ckv

extern "C" {

int ckv_assemble_member_csr(const int32_t* labels, int32_t graphs, int32_t length, int32_t num_sink,
                            int32_t communities, int32_t* counts, int32_t* offsets,
                            int32_t* member_positions, int32_t member_capacity, void* cuda_stream) {
  if (!labels || !counts || !offsets || !member_positions) return CKV_ERR_NULL;
  if (graphs <= 0 || graphs > 65535 || length <= 0 || num_sink < 0 || num_sink >= length || communities <= 0 ||
      member_capacity < length - num_sink) {
    return CKV_ERR_SHAPE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * static_cast<size_t>(graphs) * communities, stream) !=
      cudaSuccess) {
    return CKV_ERR_LAUNCH;
  }
  const int blocks = (length - num_sink + 255) / 256;
  ckv::label_count_kernel<<<dim3(blocks > 592 ? 592 : blocks, graphs), 256, 0, stream>>>(
      labels, graphs, length, num_sink, communities, counts);
  if (ckv::launched() != CKV_OK) return CKV_ERR_LAUNCH;
  ckv::offsets_scan_kernel<<<graphs, 1024, 0, stream>>>(counts, communities, offsets);
  if (ckv::launched() != CKV_OK) return CKV_ERR_LAUNCH;
  const int per_block = ckv::kFillWarps * ckv::kLabelsPerWarp;
  ckv::member_fill_kernel<<<dim3((communities + per_block - 1) / per_block, graphs), ckv::kFillWarps * 32, 0,
                            stream>>>(labels, length, num_sink, communities, offsets, member_capacity,
                                      member_positions);
  return ckv::launched();
}

int ckv_assemble_centroids(const int32_t* offsets, const int32_t* member_positions, int32_t communities,
                           int32_t member_capacity, const void* keys, int64_t key_head_stride,
                           int64_t key_row_stride, const int32_t* retrieval_to_graph,
                           const int32_t* retrieval_to_kv, int32_t heads, int32_t live, int32_t capacity,
                           void* centroids, int32_t* sizes, void* cuda_stream) {
  if (!offsets || !member_positions || !keys || !retrieval_to_graph || !retrieval_to_kv || !centroids || !sizes) {
    return CKV_ERR_NULL;
  }
  if (communities <= 0 || member_capacity <= 0 || heads <= 0 || heads > 65535 || live < 0 || capacity < live ||
      capacity < communities || key_row_stride < CKV_HEAD_DIM) {
    return CKV_ERR_SHAPE;
  }
  if ((key_row_stride % 4) || (key_head_stride % 4) || (reinterpret_cast<uintptr_t>(keys) % 8) ||
      (reinterpret_cast<uintptr_t>(centroids) % 4)) {
    return CKV_ERR_ALIGN;
  }
  ckv::centroid_kernel<<<dim3((capacity + 7) / 8, heads), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      offsets, member_positions, communities, member_capacity, static_cast<const __nv_bfloat16*>(keys),
      key_head_stride, key_row_stride, retrieval_to_graph, retrieval_to_kv, live, capacity,
      static_cast<uint8_t*>(centroids), sizes);
  return ckv::launched();
}

int ckv_assemble_modularity(const int32_t* labels, int32_t graphs, int32_t length, const int64_t* edge_src,
                            const int64_t* edge_dst, const float* edge_weight, int64_t edges,
                            int32_t capacity, float* community_weight, float* total_weight,
                            void* cuda_stream) {
  if (!labels || !community_weight || !total_weight) return CKV_ERR_NULL;
  if (graphs <= 0 || length <= 0 || capacity <= 0 || edges < 0) return CKV_ERR_SHAPE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (cudaMemsetAsync(community_weight, 0, sizeof(float) * static_cast<size_t>(graphs) * capacity, stream) !=
          cudaSuccess ||
      cudaMemsetAsync(total_weight, 0, sizeof(float) * static_cast<size_t>(graphs), stream) != cudaSuccess) {
    return CKV_ERR_LAUNCH;
  }
  if (edges == 0) return CKV_OK;
  if (!edge_src || !edge_dst || !edge_weight) return CKV_ERR_NULL;
  const int64_t blocks = (edges + 255) / 256;
  ckv::modularity_kernel<<<static_cast<unsigned>(blocks > 1184 ? 1184 : blocks), 256, 0, stream>>>(
      labels, length, graphs, edge_src, edge_dst, edge_weight, edges, capacity, community_weight, total_weight);
  return ckv::launched();
}

}  // extern "C"
