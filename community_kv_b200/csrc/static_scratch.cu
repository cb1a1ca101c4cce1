// Attention entry point for callers that may not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a serving
// process whose memory pool was carved up at start-up, a plug-in called from
// inside someone else's allocator-owned region, a real-time loop that forbids
// allocation calls after initialisation.  Such a caller can hand over its inputs
// and outputs but has nowhere to put the attention scratch (resolved row
// positions, per-split partials, per-split neighbour candidates).  This file
// keeps that scratch in a fixed array that is part of the loaded module, so the
// entry point below needs no allocation at all - at the price of a hard size
// limit and of every GPU that loads the library holding the array until exit.

#include "ckv_device.cuh"

namespace ckv {
cudaError_t launch_resolve(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_attention(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_merge_update(const ckv_layer_args& a, cudaStream_t stream);
}  // namespace ckv

namespace {

// Limits of the built-in scratch (see ckv_b200.h).
constexpr int kMaxUnits = CKV_STATIC_MAX_UNITS;
constexpr int kMaxBudget = CKV_STATIC_MAX_BUDGET;
constexpr int kMaxSplits = CKV_STATIC_MAX_SPLITS;
constexpr int kMaxGroup = CKV_STATIC_MAX_GROUP;

constexpr size_t kPositionBytes = sizeof(int32_t) * kMaxUnits * kMaxBudget;
constexpr size_t kPartialBytes =
    sizeof(float) * kMaxUnits * kMaxSplits * kMaxGroup * CKV_PARTIAL_STRIDE;
constexpr size_t kTopkBytes = sizeof(uint64_t) * kMaxUnits * kMaxSplits * CKV_KAPPA;
constexpr size_t kScratchBytes = kPositionBytes + kPartialBytes + kTopkBytes;

// Lives in the module image of every device that loads the library.  In host
// code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_attention_scratch[kScratchBytes];

// Device address of the array, looked up once per device.
unsigned char* g_scratch_address[64] = {};

int scratch_for_device(int device, unsigned char** out) {
  if (device < 0 || device >= 64) return CKV_ERR_DEVICE;
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return CKV_ERR_DEVICE;
  if (current != device && cudaSetDevice(device) != cudaSuccess) return CKV_ERR_DEVICE;
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_attention_scratch) != cudaSuccess || address == nullptr) {
      return CKV_ERR_DEVICE;
    }
    g_scratch_address[device] = static_cast<unsigned char*>(address);
  }
  *out = g_scratch_address[device];
  return CKV_OK;
}

}  // namespace

extern "C" int ckv_segmented_attention_static(const ckv_layer_args* args, void* cuda_stream) {
  if (args == nullptr) return CKV_ERR_NULL;
  const ckv_layer_args& in = *args;
  if (in.batch <= 0 || in.retrieval_heads <= 0 || in.graphs <= 0) return CKV_ERR_SHAPE;
  if (in.group_size < 1 || in.token_budget <= 0 || in.token_budget % CKV_TILE) return CKV_ERR_SHAPE;
  if (in.num_sink < 0 || in.num_sink + 1 >= in.token_budget) return CKV_ERR_SHAPE;
  if (in.splits <= 0 || in.splits > in.token_budget / 16) return CKV_ERR_SHAPE;
  // the fixed scratch bounds every extent
  if (static_cast<int64_t>(in.batch) * in.retrieval_heads > kMaxUnits ||
      in.token_budget > kMaxBudget || in.splits > kMaxSplits || in.group_size > kMaxGroup) {
    return CKV_ERR_CAPACITY;
  }
  if (!in.retrieval_to_graph || !in.retrieval_to_kv || !in.query || !in.key || !in.value ||
      !in.output || !in.lse || !in.topk_scores || !in.topk_positions || !in.communities ||
      !in.cumulative_ends || !in.descriptor_counts || !in.member_offsets ||
      !in.member_positions || !in.current_position || !in.delta_positions || !in.chunk_start ||
      !in.chunk_size || !in.chunk_previous || !in.community_tail || !in.delta_sizes) {
    return CKV_ERR_NULL;
  }
  if (in.num_sink > 0 && !in.sink_positions) return CKV_ERR_NULL;
  if (in.member_capacity <= 0 || in.chunks_per_graph <= 0 || in.delta_position_capacity <= 0 ||
      in.sequence_capacity <= 0 || in.token_capacity <= 0 || in.community_capacity <= 0 ||
      in.descriptor_capacity <= 0) {
    return CKV_ERR_SHAPE;
  }
  if ((in.key_row_stride % 8) || (in.value_row_stride % 8) || (in.key_head_stride % 8) ||
      (in.value_head_stride % 8) || (in.key_batch_stride % 8) || (in.value_batch_stride % 8) ||
      (reinterpret_cast<uintptr_t>(in.key) % 16) || (reinterpret_cast<uintptr_t>(in.value) % 16)) {
    return CKV_ERR_ALIGN;
  }
  if (in.key_row_stride < CKV_HEAD_DIM || in.value_row_stride < CKV_HEAD_DIM) return CKV_ERR_SHAPE;
  if (!(in.flags & CKV_FLAG_SKIP_UPDATE)) {
    if (!in.centroids || !in.community_sizes || !in.community_counts || !in.community_weight ||
        !in.total_weight || !in.token_communities || !in.chunk_capacity || !in.chunk_next ||
        !in.community_head || !in.next_free_chunk || !in.next_free_position || !in.assigned ||
        !in.overflow) {
      return CKV_ERR_NULL;
    }
  }

  unsigned char* scratch = nullptr;
  const int ready = scratch_for_device(in.device, &scratch);
  if (ready != CKV_OK) return ready;

  // Same kernels as ckv_segmented_attention; only the three scratch pointers differ.
  ckv_layer_args local = in;
  local.flags &= ~CKV_FLAG_ATTENTION_ONLY;
  local.positions = reinterpret_cast<int32_t*>(scratch);
  local.partials = reinterpret_cast<float*>(scratch + kPositionBytes);
  local.partial_topk = reinterpret_cast<uint64_t*>(scratch + kPositionBytes + kPartialBytes);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (ckv::launch_resolve(local, stream) != cudaSuccess) return CKV_ERR_LAUNCH;
  if (ckv::launch_attention(local, stream) != cudaSuccess) return CKV_ERR_LAUNCH;
  if (ckv::launch_merge_update(local, stream) != cudaSuccess) return CKV_ERR_LAUNCH;
  return CKV_OK;
}
