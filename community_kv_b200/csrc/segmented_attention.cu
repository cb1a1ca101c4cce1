// Gather + segmented flash-decode attention over the resolved cache rows (sm_100a).
//
// Grid (splits, batch*R), 128 threads, three CTAs per SM.  The T logical tokens of
// one retrieval head are cut into 16-token steps; CTA `split` owns a contiguous
// run of steps and each of its four warps a contiguous quarter of that run.  Every
// warp runs its own two-stage pipeline:
//   * the 16 K rows and 16 V rows of a step (256 bytes each, anywhere in the
//     cache) are fetched with 16-byte cp.async copies, a half-warp per row, so
//     every request is a full coalesced row; completion is tracked with
//     cp.async groups (no barrier objects, nothing to spin on); masked slots are
//     zero-filled without touching memory;
//   * rows land in shared memory at a 272-byte pitch so ldmatrix is conflict free;
//   * S^T = K Q^T and O^T = V^T P^T run on mma.m16n8k16 (bf16 in, fp32 accumulate)
//     with the 16 tokens on the M axis and up to eight query heads on the N axis
//     (two head blocks when the group is larger than eight), P^T moves from the
//     accumulator layout to the operand layout with movmatrix;
//   * the first head of the group is additionally scored on the CUDA cores in the
//     fixed fp32 order shared with the CPU oracle (mixed-precision fma: bf16
//     operands, fp32 accumulate, one rounding); those scores feed the top-8
//     neighbour candidates, so the online labels are reproducible bit for bit;
//   * running (max, sum, acc) per warp, merged across the four warps at the end
//     and written as one partial per (split, head).

#include "segmented_attention.cuh"

namespace ckv {

template <int kBlocks>
__global__ void __launch_bounds__(kAttnThreads, 3) attention_kernel(const ckv_layer_args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_release_dependents();
  pdl_wait_for_predecessor();  // positions (and the query) are produced upstream
  attention_split<kBlocks>(a, blockIdx.y, blockIdx.x, smem);
}

int attention_smem_bytes() { return AttnSmem::kTotal; }

cudaError_t launch_attention(const ckv_layer_args& a, cudaStream_t stream) {
  static bool configured[64] = {};
  const int device = a.device >= 0 && a.device < 64 ? a.device : 0;
  if (!configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(attention_kernel<1>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           AttnSmem::kTotal);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(attention_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnSmem::kTotal);
    if (err != cudaSuccess) return err;
    configured[device] = true;
  }
  const dim3 grid(a.splits, a.batch * a.retrieval_heads);
  if (a.group_size > 8) {
    return launch_dependent(attention_kernel<2>, grid, dim3(kAttnThreads), AttnSmem::kTotal, stream, a);
  }
  return launch_dependent(attention_kernel<1>, grid, dim3(kAttnThreads), AttnSmem::kTotal, stream, a);
}

}  // namespace ckv
