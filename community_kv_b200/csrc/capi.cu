// C ABI of the sparse-decode path: argument validation and kernel sequencing.

#include "ckv_device.cuh"

namespace ckv {
cudaError_t launch_score(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_select(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_resolve(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_attention(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_merge_update(const ckv_layer_args& a, cudaStream_t stream);
cudaError_t launch_append_kv(void* key_cache, void* value_cache, const void* new_key, const void* new_value,
                             int64_t units, int64_t unit_stride, const int32_t* row_index,
                             int64_t row_index_stride, int64_t row, cudaStream_t stream);
cudaError_t launch_wait_peers(uint32_t* flag, uint32_t expected, uint32_t* status, cudaStream_t stream);
cudaError_t launch_nearest_centroid(const ckv_layer_args& a, int32_t* forced, cudaStream_t stream);
bool fused_layer_supported(const ckv_layer_args& a);
cudaError_t launch_fused_layer(const ckv_layer_args& a, cudaStream_t stream);
int attention_smem_bytes();
cudaError_t launch_prefill(const ckv_prefill_args& a, cudaStream_t stream);

namespace {

int check_common(const ckv_layer_args* a) {
  if (a == nullptr) return CKV_ERR_NULL;
  if (a->batch <= 0 || a->retrieval_heads <= 0 || a->graphs <= 0) return CKV_ERR_SHAPE;
  if (a->group_size < 1 || a->group_size > 16) return CKV_ERR_SHAPE;
  if (a->community_capacity <= 0) return CKV_ERR_SHAPE;
  if (a->token_budget <= 0 || a->token_budget % CKV_TILE) return CKV_ERR_SHAPE;
  if (a->num_sink < 0 || a->num_sink + 1 >= a->token_budget) return CKV_ERR_SHAPE;
  if (static_cast<int64_t>(a->batch) * a->retrieval_heads > 65535) return CKV_ERR_CAPACITY;
  if (a->retrieval_to_graph == nullptr || a->retrieval_to_kv == nullptr) return CKV_ERR_NULL;
  if (a->peer_count < 0 || a->peer_count > CKV_MAX_PEERS) return CKV_ERR_SHAPE;
  for (int p = 0; p < a->peer_count; ++p) {
    if (a->peer_output[p] == nullptr || a->peer_flag[p] == nullptr) return CKV_ERR_NULL;
  }
  return CKV_OK;
}

}  // namespace

// Argument validation shared by every entry point that takes ckv_layer_args (also
// the allocation-free one in static_scratch.cu): nothing is launched, and no CUDA
// call is made, before this returns CKV_OK.
int check(const ckv_layer_args* a, int need) {
  const int common = check_common(a);
  if (common != CKV_OK) return common;
  if (need & kNeedScore) {
    if (!a->query || !a->centroids || !a->community_sizes || !a->community_counts || !a->scores)
      return CKV_ERR_NULL;
  }
  if (need & kNeedSelect) {
    if (!a->scores || !a->community_sizes || !a->community_counts || !a->communities ||
        !a->cumulative_ends || !a->descriptor_counts || !a->tile_descriptors || !a->positions)
      return CKV_ERR_NULL;
    if (a->descriptor_capacity < a->token_budget - a->num_sink - 1) return CKV_ERR_SHAPE;
    if (a->max_communities < 0) return CKV_ERR_SHAPE;
  }
  if (need & (kNeedSelect | kNeedAttention)) {
    if (!a->member_offsets || !a->member_positions || !a->current_position ||
        !a->delta_positions || !a->chunk_start || !a->chunk_size || !a->chunk_previous ||
        !a->community_tail || !a->delta_sizes)
      return CKV_ERR_NULL;
    if (a->num_sink > 0 && !a->sink_positions) return CKV_ERR_NULL;
    if (a->member_capacity <= 0 || a->chunks_per_graph <= 0 || a->delta_position_capacity <= 0)
      return CKV_ERR_SHAPE;
  }
  if (need & kNeedAttention) {
    if (!a->query || !a->key || !a->value || !a->positions || !a->partials || !a->partial_topk ||
        !a->output || !a->lse || !a->topk_scores || !a->topk_positions || !a->communities ||
        !a->cumulative_ends || !a->descriptor_counts)
      return CKV_ERR_NULL;
    if (a->splits <= 0 || a->splits > 32 || a->splits > a->token_budget / 16)
      return CKV_ERR_SHAPE;
    if (a->sequence_capacity <= 0 || a->token_capacity <= 0) return CKV_ERR_SHAPE;
    if ((a->key_row_stride % 8) || (a->value_row_stride % 8) || (a->key_head_stride % 8) ||
        (a->value_head_stride % 8) || (a->key_batch_stride % 8) || (a->value_batch_stride % 8) ||
        (reinterpret_cast<uintptr_t>(a->key) % 16) || (reinterpret_cast<uintptr_t>(a->value) % 16))
      return CKV_ERR_ALIGN;
    if (a->key_row_stride < CKV_HEAD_DIM || a->value_row_stride < CKV_HEAD_DIM)
      return CKV_ERR_SHAPE;
    if (!(a->flags & CKV_FLAG_SKIP_UPDATE)) {
      if (!a->centroids || !a->community_sizes || !a->community_counts || !a->community_weight ||
          !a->total_weight || !a->token_communities || !a->chunk_capacity || !a->chunk_next ||
          !a->community_head || !a->next_free_chunk || !a->next_free_position || !a->assigned ||
          !a->overflow)
        return CKV_ERR_NULL;
    }
  }
  return CKV_OK;
}

namespace {

int select_device(const ckv_layer_args* a) {
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return CKV_ERR_DEVICE;
  if (current != a->device) {
    if (cudaSetDevice(a->device) != cudaSuccess) return CKV_ERR_DEVICE;
  }
  return CKV_OK;
}

int launched(cudaError_t err) { return err == cudaSuccess ? CKV_OK : CKV_ERR_LAUNCH; }

}  // namespace
}  // namespace ckv

extern "C" {

int ckv_version(void) { return 100; }

const char* ckv_status_string(int status) {
  switch (status) {
    case CKV_OK: return "ok";
    case CKV_ERR_NULL: return "a required pointer is null";
    case CKV_ERR_SHAPE: return "a size or stride is out of range";
    case CKV_ERR_ALIGN: return "K/V rows must be 16-byte aligned";
    case CKV_ERR_LAUNCH: return "the CUDA runtime rejected a kernel launch";
    case CKV_ERR_DEVICE: return "the CUDA device cannot be selected";
    case CKV_ERR_UNSUPPORTED: return "unsupported configuration";
    case CKV_ERR_CAPACITY: return "a size exceeds a fixed built-in maximum";
    default: return "unknown status";
  }
}

int ckv_attention_smem_bytes(int group_size) {
  (void)group_size;
  return ckv::attention_smem_bytes();
}

int ckv_score_centroids(const ckv_layer_args* args, void* cuda_stream) {
  int status = ckv::check(args, ckv::kNeedScore);
  if (status != CKV_OK) return status;
  status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  return ckv::launched(ckv::launch_score(*args, static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_select_descriptors(const ckv_layer_args* args, void* cuda_stream) {
  int status = ckv::check(args, ckv::kNeedSelect);
  if (status != CKV_OK) return status;
  status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  return ckv::launched(ckv::launch_select(*args, static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_segmented_attention(const ckv_layer_args* args, void* cuda_stream) {
  int status = ckv::check(args, ckv::kNeedAttention);
  if (status != CKV_OK) return status;
  status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (args->flags & CKV_FLAG_ATTENTION_ONLY) {
    return ckv::launched(ckv::launch_attention(*args, stream));
  }
  status = ckv::launched(ckv::launch_resolve(*args, stream));
  if (status != CKV_OK) return status;
  status = ckv::launched(ckv::launch_attention(*args, stream));
  if (status != CKV_OK) return status;
  return ckv::launched(ckv::launch_merge_update(*args, stream));
}

int ckv_decode_layer(const ckv_layer_args* args, void* cuda_stream) {
  int status =
      ckv::check(args, ckv::kNeedScore | ckv::kNeedSelect | ckv::kNeedAttention);
  if (status != CKV_OK) return status;
  status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (ckv::fused_layer_supported(*args)) {
    // one cluster launch per layer: scoring, selection, attention, merge and update
    if (ckv::launch_fused_layer(*args, stream) == cudaSuccess) return CKV_OK;
    // the cluster shape could not be scheduled on this device: clear the error and
    // run the four kernels instead (same results)
    (void)cudaGetLastError();
  }
  status = ckv::launched(ckv::launch_score(*args, stream));
  if (status != CKV_OK) return status;
  status = ckv::launched(ckv::launch_select(*args, stream));
  if (status != CKV_OK) return status;
  status = ckv::launched(ckv::launch_attention(*args, stream));
  if (status != CKV_OK) return status;
  return ckv::launched(ckv::launch_merge_update(*args, stream));
}

int ckv_append_kv(void* key_cache, void* value_cache, const void* new_key, const void* new_value,
                  int64_t units, int64_t unit_stride, const int32_t* row_index,
                  int64_t row_index_stride, int64_t row, void* cuda_stream) {
  if (!key_cache || !value_cache || !new_key || !new_value) return CKV_ERR_NULL;
  if (units <= 0 || unit_stride <= 0 || (row_index == nullptr && row < 0)) return CKV_ERR_SHAPE;
  if (row_index != nullptr && row_index_stride != 0 && row_index_stride != 1) return CKV_ERR_SHAPE;
  if (unit_stride % 8 || ((reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache) |
                           reinterpret_cast<uintptr_t>(new_key) | reinterpret_cast<uintptr_t>(new_value)) & 15u)) {
    return CKV_ERR_ALIGN;
  }
  return ckv::launched(ckv::launch_append_kv(key_cache, value_cache, new_key, new_value, units, unit_stride,
                                             row_index, row_index_stride, row,
                                             static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_wait_peers(uint32_t* flag, uint32_t expected, uint32_t* status, void* cuda_stream) {
  if (flag == nullptr) return CKV_ERR_NULL;
  if (expected == 0) return CKV_OK;
  return ckv::launched(
      ckv::launch_wait_peers(flag, expected, status, static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_nearest_centroid(const ckv_layer_args* args, int32_t* forced_community, void* cuda_stream) {
  const int common = ckv::check_common(args);
  if (common != CKV_OK) return common;
  const ckv_layer_args& a = *args;
  if (!forced_community || !a.centroids || !a.community_sizes || !a.community_counts ||
      !a.current_position) {
    return CKV_ERR_NULL;
  }
  if (!a.current_key && !a.key) return CKV_ERR_NULL;
  if (a.sequence_capacity <= 0) return CKV_ERR_SHAPE;
  const int status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  return ckv::launched(
      ckv::launch_nearest_centroid(a, forced_community, static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_decode_layer_kernels(const ckv_layer_args* args) {
  if (args == nullptr) return CKV_ERR_NULL;
  if (ckv::fused_layer_supported(*args)) return 1;
  return (args->retrieval_heads != args->graphs && !(args->flags & CKV_FLAG_SKIP_UPDATE)) ? 5 : 4;
}

int ckv_online_update(const ckv_layer_args* args, void* cuda_stream) {
  const int common = ckv::check_common(args);
  if (common != CKV_OK) return common;
  const ckv_layer_args& a = *args;
  if (!a.lse || !a.topk_scores || !a.topk_positions || !a.centroids || !a.community_sizes ||
      !a.community_counts || !a.community_weight || !a.total_weight || !a.token_communities ||
      !a.current_position || !a.delta_positions || !a.chunk_start || !a.chunk_capacity ||
      !a.chunk_size || !a.chunk_next || !a.chunk_previous || !a.community_head ||
      !a.community_tail || !a.delta_sizes || !a.next_free_chunk || !a.next_free_position ||
      !a.assigned || !a.overflow) {
    return CKV_ERR_NULL;
  }
  if (!a.current_key && !a.key) return CKV_ERR_NULL;
  if (a.sequence_capacity <= 0 || a.token_capacity <= 0 || a.chunks_per_graph <= 0 ||
      a.delta_position_capacity <= 0) {
    return CKV_ERR_SHAPE;
  }
  const int status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  ckv_layer_args local = a;
  local.flags = (a.flags | CKV_FLAG_UPDATE_ONLY) & ~CKV_FLAG_SKIP_UPDATE;
  local.splits = 1;
  return ckv::launched(ckv::launch_merge_update(local, static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_merge_partials(const ckv_layer_args* args, void* cuda_stream) {
  const int common = ckv::check_common(args);
  if (common != CKV_OK) return common;
  const ckv_layer_args& a = *args;
  if (!a.partials || !a.partial_topk || !a.output || !a.lse || !a.topk_scores || !a.topk_positions) {
    return CKV_ERR_NULL;
  }
  if (a.splits <= 0 || a.splits > 32) return CKV_ERR_SHAPE;
  if (a.partial_unit_stride < 0 || a.partial_split_stride < 0 || a.topk_unit_stride < 0 ||
      a.topk_split_stride < 0 || (a.partial_unit_stride % 4) || (a.partial_split_stride % 4)) {
    return CKV_ERR_SHAPE;  // rows are read 16 bytes at a time
  }
  if (reinterpret_cast<uintptr_t>(a.partials) % 16 || reinterpret_cast<uintptr_t>(a.partial_topk) % 8) {
    return CKV_ERR_ALIGN;
  }
  if (!(a.flags & CKV_FLAG_SKIP_UPDATE)) {
    if (!a.centroids || !a.community_sizes || !a.community_counts || !a.community_weight ||
        !a.total_weight || !a.token_communities || !a.current_position || !a.delta_positions ||
        !a.chunk_start || !a.chunk_capacity || !a.chunk_size || !a.chunk_next || !a.chunk_previous ||
        !a.community_head || !a.community_tail || !a.delta_sizes || !a.next_free_chunk ||
        !a.next_free_position || !a.assigned || !a.overflow) {
      return CKV_ERR_NULL;
    }
    if (!a.current_key && !a.key) return CKV_ERR_NULL;
    if (a.sequence_capacity <= 0 || a.token_capacity <= 0 || a.chunks_per_graph <= 0 ||
        a.delta_position_capacity <= 0) {
      return CKV_ERR_SHAPE;
    }
  }
  const int status = ckv::select_device(args);
  if (status != CKV_OK) return status;
  ckv_layer_args local = a;
  local.flags = a.flags & ~(CKV_FLAG_UPDATE_ONLY | CKV_FLAG_ATTENTION_ONLY);
  local.merged = nullptr;  // the rows being merged may be the caller's `merged` records themselves
  local.merged_topk = nullptr;
  return ckv::launched(ckv::launch_merge_update(local, static_cast<cudaStream_t>(cuda_stream)));
}

int ckv_prefill_topk(const ckv_prefill_args* args, void* cuda_stream) {
  if (args == nullptr) return CKV_ERR_NULL;
  const ckv_prefill_args& a = *args;
  if (a.batch <= 0 || a.seq_len <= 0 || a.query_heads <= 0 || a.kv_heads <= 0) return CKV_ERR_SHAPE;
  if (a.query_heads % a.kv_heads) return CKV_ERR_SHAPE;
  const int group = a.query_heads / a.kv_heads;
  if (group != 1 && group != 2 && group != 4 && group != 8) return CKV_ERR_UNSUPPORTED;
  if (a.mode < 0 || a.mode > 2 || a.num_sink < 0) return CKV_ERR_SHAPE;
  if (a.kv_heads > 65535 || a.batch > 65535) return CKV_ERR_CAPACITY;
  if (!a.query || !a.key || !a.value || !a.output || !a.lse) return CKV_ERR_NULL;
  if (a.mode == 1) {
    if (!a.topk_val || !a.topk_idx) return CKV_ERR_NULL;
    if (a.seq_len > (1 << 17)) return CKV_ERR_CAPACITY;  /* 17-bit packed key index */
  }
  if (a.mode == 2) {
    if (!a.candidates || !a.edge_idx || !a.edge_score) return CKV_ERR_NULL;
    if (a.edges_per_row < 1 || a.edges_per_row > 16) return CKV_ERR_SHAPE;
  }
  const int64_t strides[] = {a.q_batch_stride, a.q_row_stride, a.q_head_stride, a.k_batch_stride,
                             a.k_row_stride,   a.k_head_stride, a.v_batch_stride, a.v_row_stride,
                             a.v_head_stride,  a.o_batch_stride, a.o_row_stride,  a.o_head_stride};
  for (int64_t stride : strides) {
    if (stride % 8) return CKV_ERR_ALIGN;
  }
  const void* pointers[] = {a.query, a.key, a.value, a.output};
  for (const void* pointer : pointers) {
    if (reinterpret_cast<uintptr_t>(pointer) % 16) return CKV_ERR_ALIGN;
  }
  int current = -1;
  if (cudaGetDevice(&current) != cudaSuccess) return CKV_ERR_DEVICE;
  if (current != a.device && cudaSetDevice(a.device) != cudaSuccess) return CKV_ERR_DEVICE;
  return ckv::launched(ckv::launch_prefill(a, static_cast<cudaStream_t>(cuda_stream)));
}

}  // extern "C"
