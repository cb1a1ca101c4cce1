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

// Device address of the array, looked up once per device.  Two host threads that make
// their first call on a device at the same time both look the address up and store the
// same value, so the table needs no lock.
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
  // the fixed scratch bounds every extent
  if (in.batch > 0 && in.retrieval_heads > 0 &&
      (static_cast<int64_t>(in.batch) * in.retrieval_heads > kMaxUnits ||
       in.token_budget > kMaxBudget || in.splits > kMaxSplits || in.group_size > kMaxGroup)) {
    return CKV_ERR_CAPACITY;
  }
  {
    // the same validation as ckv_segmented_attention (peer fields included), with the
    // three scratch pointers - which this entry point supplies itself - marked present
    ckv_layer_args probe = in;
    probe.positions = reinterpret_cast<int32_t*>(sizeof(int32_t));
    probe.partials = reinterpret_cast<float*>(sizeof(float));
    probe.partial_topk = reinterpret_cast<uint64_t*>(sizeof(uint64_t));
    const int status = ckv::check(&probe, ckv::kNeedAttention);
    if (status != CKV_OK) return status;
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
