// One launch per decode layer: a thread-block cluster per (sequence, retrieval head).
//
// Grid (splits, batch*R), cluster (splits, 1, 1), 128 threads, three CTAs per SM.
// The CTAs of a cluster are co-scheduled, so they can hand work to one another
// through the hardware cluster barrier instead of through kernel boundaries:
//
//   1. every CTA scores a 1/splits share of the unit's centroid rows, writes the
//      fp16 scores to the workspace and keeps its slice's keys, sizes and weighted
//      histogram in shared memory;
//   2. the budgeted selection runs across the cluster (select_cluster: three
//      cluster barriers, histograms and the descriptor list exchanged through
//      distributed shared memory); each CTA then resolves only the logical tokens
//      of its own attention split to cache rows;
//   3. every CTA gathers and attends to its split and writes its partial
//      (acc, max, sum) rows and neighbour candidates;         -- cluster barrier --
//   4. rank 0 merges the partials, writes the output and applies the online
//      graph update; the other CTAs have already left.
//
// The result is bit for bit the one of the four stand-alone kernels: the same
// device functions run in the same order on the same data.  The path needs one
// graph per retrieval head (a graph shared by several heads is updated by its
// leader while followers may still be reading it, which only a kernel boundary
// orders) and per-CTA community slices that fit the selection's shared-memory stash.

#include "merge_update.cuh"
#include "score_select.cuh"
#include "segmented_attention.cuh"

namespace ckv {

constexpr int kFusedThreads = 128;
constexpr int kFusedSmem = AttnSmem::kTotal > static_cast<int>(sizeof(ClusterSelectSmem))
                               ? AttnSmem::kTotal
                               : static_cast<int>(sizeof(ClusterSelectSmem));

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int kBlocks>
__global__ void __launch_bounds__(kFusedThreads, 3) decode_cluster_kernel(const ckv_layer_args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ UpdateDecision decision;
  __shared__ float lse_s;
  const int flat = blockIdx.y;
  const int split = blockIdx.x;  // == rank in the cluster
  pdl_release_dependents();
  // This CTA's share of the centroid table does not come from the kernel before it in
  // the stream (that one produces the query): ask for it in L2 while that kernel is
  // still finishing, before the wait below.
  {
    const int limit = score_limit(a, flat);
    const int groups = (limit + 15) / 16;
    const int first_row = 16 * static_cast<int>(static_cast<int64_t>(split) * groups / a.splits);
    const int last_row = min(limit, 16 * static_cast<int>(static_cast<int64_t>(split + 1) * groups / a.splits));
    const uint8_t* rows = reinterpret_cast<const uint8_t*>(a.centroids) +
                          (static_cast<int64_t>(flat) * a.community_capacity + first_row) * kHeadDim;
    for (int row = threadIdx.x; row < last_row - first_row; row += kFusedThreads) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(rows + static_cast<int64_t>(row) * kHeadDim));
    }
  }
  pdl_wait_for_predecessor();  // the query and last step's state come from upstream
  // ---- 1. centroid scores: this CTA's share of the unit's 16-row groups; the keys
  // stay in shared memory and are counted into the slice's histogram on the way ----
  ClusterSelectSmem& sm = *reinterpret_cast<ClusterSelectSmem*>(smem);
  const int groups = (score_limit(a, flat) + 15) / 16;
  const int first_group = static_cast<int>(static_cast<int64_t>(split) * groups / a.splits);
  const int last_group = static_cast<int>(static_cast<int64_t>(split + 1) * groups / a.splits);
  phase_stamp(a, flat, split, 0);
  cluster_select_begin<kFusedThreads>(sm);
  // last step's threshold of this unit (-1 before the first step): its high byte is the guess
  int guess_bin = -1;
  if (a.threshold_state != nullptr) {
    const int previous = a.threshold_state[static_cast<int64_t>(flat) * 4];
    guess_bin = previous >= 0 ? (previous >> 8) & 0xff : -1;
  }
  {
    const ScoreSlice slice = {sm.key,       sm.size,      sm.hist_mass, sm.hist_count, first_group * 16,
                              sm.low_mass,  sm.low_count, guess_bin};
    score_groups<kFusedThreads, kClusterStageBytes>(a, flat, first_group, last_group, sm.query, &slice);
  }
  __syncthreads();
  phase_stamp(a, flat, split, 1);

  // ---- 2. selection across the cluster, then this split's cache rows ----
  {
    const int steps_total = a.token_budget / kStepTokens;
    const int step_begin = static_cast<int>(static_cast<int64_t>(split) * steps_total / a.splits);
    const int step_end = static_cast<int>(static_cast<int64_t>(split + 1) * steps_total / a.splits);
    const int row0 = first_group * 16;
    const int rows = min(score_limit(a, flat), last_group * 16) - row0;
    select_cluster<kFusedThreads>(a, flat, sm, split, a.splits, row0, rows,
                                  step_begin * kStepTokens, step_end * kStepTokens, guess_bin);
  }
  __syncthreads();  // positions written above are read by other threads of this CTA
  phase_stamp(a, flat, split, 6);

  // ---- 3. gather + attention over this split ----
  attention_split<kBlocks>(a, flat, split, smem);
  phase_stamp(a, flat, split, 7);
  cluster_arrive();  // release at cluster scope: the partials above are visible to rank 0
  if (split != 0) {
    return;
  }
  cluster_wait();
  phase_stamp(a, flat, split, 8);

  // ---- 4. merge, output, online update ----
  merge_update_unit(a, flat, kFusedThreads / 32 - 1, decision, lse_s);
  __syncthreads();
  phase_stamp(a, flat, split, 9);
  if (flat == 0) {
    wait_for_peer_rows(a);
  }
}

bool fused_layer_supported(const ckv_layer_args& a) {
  // every CTA stages the rows it scores: a 1/splits share of the 16-row groups
  const int groups = (a.community_capacity + 15) / 16;
  const int rows_per_cta = 16 * ((groups + a.splits - 1) / (a.splits > 0 ? a.splits : 1));
  return a.graphs == a.retrieval_heads && a.splits >= 1 && a.splits <= 8 && rows_per_cta <= kStash &&
         !(a.flags & (CKV_FLAG_ATTENTION_ONLY | CKV_FLAG_UPDATE_ONLY | CKV_FLAG_UNFUSED |
                      CKV_FLAG_FP32_CENTROIDS));
}

cudaError_t launch_fused_layer(const ckv_layer_args& a, cudaStream_t stream) {
  static bool configured[64] = {};
  const int device = a.device >= 0 && a.device < 64 ? a.device : 0;
  if (!configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(decode_cluster_kernel<1>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmem);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(decode_cluster_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kFusedSmem);
    if (err != cudaSuccess) return err;
    configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(a.splits, a.batch * a.retrieval_heads);
  config.blockDim = dim3(kFusedThreads);
  config.dynamicSmemBytes = kFusedSmem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = a.splits;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = 2;
  if (a.group_size > 8) {
    return cudaLaunchKernelEx(&config, decode_cluster_kernel<2>, a);
  }
  return cudaLaunchKernelEx(&config, decode_cluster_kernel<1>, a);
}

}  // namespace ckv
