// Gather + segmented flash-decode attention over the resolved cache rows (sm_100a).
//
// Grid (splits, batch*R), 128 threads.  A CTA owns T/splits logical tokens of
// one retrieval head; each of its four warps owns a contiguous quarter and runs
// its own pipeline, 16 tokens per step:
//   * lane i (<16) asks the TMA engine for K row i, lane 16+i for V row i: one
//     256-byte cp.async.bulk per lane per step, completion counted on a per-warp
//     mbarrier (three stages in flight per warp, no multicast, bounded waits);
//   * rows land in shared memory at a 272-byte pitch so ldmatrix is conflict
//     free; Q K^T and P V run on mma.m16n8k16 (bf16 in, fp32 accumulate) with the
//     query group on the M axis;
//   * the first head of the group is additionally scored on the CUDA cores in
//     the fixed fp32 order shared with the CPU oracle; those scores feed the
//     top-8 neighbour candidates, so the online labels are reproducible;
//   * running (max, sum, acc) per warp, merged across the four warps at the end
//     and written as one partial per (split, head).

#include "ckv_device.cuh"

namespace ckv {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = 4;
constexpr int kStages = 3;
constexpr int kRowPitch = 272;                       // bytes between staged rows
constexpr int kStageBytes = 32 * kRowPitch;          // 16 K rows + 16 V rows
constexpr int kWarpBytes = kStages * kStageBytes;    // 26112
constexpr uint32_t kWaitPolls = 1u << 22;

struct AttnSmem {
  // dynamic layout: [warp][stage][32 rows x 272 B], then q_rep, then barriers
  static constexpr int kRowsBytes = kAttnWarps * kWarpBytes;        // 104448
  static constexpr int kQrepOffset = kRowsBytes;                    // 128 floats
  static constexpr int kBarOffset = kQrepOffset + kHeadDim * 4;     // 12 x 8 B
  static constexpr int kTopOffset = kBarOffset + kAttnWarps * kStages * 8;  // 4 x 8 u64
  static constexpr int kTotal = kTopOffset + kAttnWarps * kKappa * 8;
};

__device__ __forceinline__ void top_insert(uint64_t (&list)[kKappa], uint64_t candidate) {
  if (candidate > list[kKappa - 1]) {
#pragma unroll
    for (int k = 0; k < kKappa; ++k) {
      const uint64_t resident = list[k];
      const bool greater = candidate > resident;
      list[k] = greater ? candidate : resident;
      candidate = greater ? resident : candidate;
    }
  }
}

template <bool kHigh>
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const ckv_layer_args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int flat = blockIdx.y;
  const int split = blockIdx.x;
  const Unit u = make_unit(a, flat);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = a.group_size;
  const int tokens_per_cta = a.token_budget / a.splits;
  const int tokens_per_warp = tokens_per_cta / kAttnWarps;
  const int steps = tokens_per_warp / 16;
  const int warp_token0 = split * tokens_per_cta + warp * tokens_per_warp;

  uint8_t* warp_rows = smem + warp * kWarpBytes;
  float* q_rep = reinterpret_cast<float*>(smem + AttnSmem::kQrepOffset);
  const uint32_t bar_base = smem_u32(smem + AttnSmem::kBarOffset) + warp * kStages * 8;
  uint64_t* top_s = reinterpret_cast<uint64_t*>(smem + AttnSmem::kTopOffset);

  const __nv_bfloat16* query = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                               (static_cast<int64_t>(u.batch) * a.retrieval_heads + u.head) *
                                   group * kHeadDim;
  q_rep[threadIdx.x] = __bfloat162float(query[threadIdx.x]);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_base + s * 8, 1);
    }
    mbar_fence_init();
  }
  __syncthreads();

  const int32_t* positions = a.positions + static_cast<int64_t>(flat) * a.token_budget;
  const __nv_bfloat16* key_head = reinterpret_cast<const __nv_bfloat16*>(a.key) +
                                  u.batch * a.key_batch_stride + u.kv * a.key_head_stride;
  const __nv_bfloat16* value_head = reinterpret_cast<const __nv_bfloat16*>(a.value) +
                                    u.batch * a.value_batch_stride + u.kv * a.value_head_stride;
  const int token_lane = lane & 15;
  const bool value_lane = lane >= 16;
  const uint32_t rows_u32 = smem_u32(warp_rows);

  auto issue = [&](int step) {
    const int stage = step % kStages;
    const int pos = positions[warp_token0 + step * 16 + token_lane];
    const int64_t row = pos > 0 ? pos : 0;
    const __nv_bfloat16* src =
        value_lane ? value_head + row * a.value_row_stride : key_head + row * a.key_row_stride;
    const uint32_t bar = bar_base + stage * 8;
    if (lane == 0) {
      mbar_expect_tx(bar, 32 * kHeadDim * 2);
    }
    __syncwarp();
    bulk_copy_g2s(rows_u32 + stage * kStageBytes + lane * kRowPitch, src, kHeadDim * 2, bar);
  };

  const int prologue = steps < kStages ? steps : kStages;
  for (int s = 0; s < prologue; ++s) {
    issue(s);
  }

  // A fragments of the query group: rows g (and g+8) of a 16 x 128 matrix.
  const int g_row = lane >> 2;
  const int t_col = lane & 3;
  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int col = ks * 16 + 2 * t_col;
    qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0u;
    if (g_row < group) {
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(query + g_row * kHeadDim + col);
      qa[ks][2] = *reinterpret_cast<const uint32_t*>(query + g_row * kHeadDim + col + 8);
    }
    if (kHigh && g_row + 8 < group) {
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(query + (g_row + 8) * kHeadDim + col);
      qa[ks][3] = *reinterpret_cast<const uint32_t*>(query + (g_row + 8) * kHeadDim + col + 8);
    }
  }

  float acc[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  }
  float run_max_lo = -INFINITY, run_max_hi = -INFINITY;
  float run_sum_lo = 0.f, run_sum_hi = 0.f;
  uint64_t top[kKappa];
#pragma unroll
  for (int k = 0; k < kKappa; ++k) {
    top[k] = 0ull;
  }
  const float scale = a.softmax_scale;
  bool failed = false;

  for (int step = 0; step < steps; ++step) {
    const int stage = step % kStages;
    const uint32_t parity = (step / kStages) & 1;
    if (!mbar_wait_bounded(bar_base + stage * 8, parity, kWaitPolls)) {
      failed = true;
    }
    if (__any_sync(0xffffffffu, failed)) {
      failed = true;
      break;
    }
    const uint32_t k_u32 = rows_u32 + stage * kStageBytes;
    const uint32_t v_u32 = k_u32 + 16 * kRowPitch;
    const int my_pos = positions[warp_token0 + step * 16 + token_lane];
    const unsigned valid_bits = __ballot_sync(0xffffffffu, my_pos >= 0) & 0xffffu;

    // ---- S = Q K^T for 16 tokens (two 8-token column blocks) ----
    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t b0, b1, b2, b3;
        const uint32_t addr =
            k_u32 + (nb * 8 + (lane & 7)) * kRowPitch + (kk * 4 + (lane >> 3)) * 16;
        ldmatrix_x4(addr, b0, b1, b2, b3);
        mma_bf16_16816(s[nb], qa[2 * kk][0], qa[2 * kk][1], qa[2 * kk][2], qa[2 * kk][3], b0, b1);
        mma_bf16_16816(s[nb], qa[2 * kk + 1][0], qa[2 * kk + 1][1], qa[2 * kk + 1][2],
                       qa[2 * kk + 1][3], b2, b3);
      }
    }
    // scale + mask; columns of s[nb][0..1] are tokens nb*8 + 2t, +1
    float tile_max_lo = -INFINITY, tile_max_hi = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int token = nb * 8 + 2 * t_col + e;
        const bool ok = (valid_bits >> token) & 1u;
        s[nb][e] = ok ? s[nb][e] * scale : -INFINITY;
        s[nb][2 + e] = ok ? s[nb][2 + e] * scale : -INFINITY;
        tile_max_lo = fmaxf(tile_max_lo, s[nb][e]);
        tile_max_hi = fmaxf(tile_max_hi, s[nb][2 + e]);
      }
    }
    tile_max_lo = fmaxf(tile_max_lo, __shfl_xor_sync(0xffffffffu, tile_max_lo, 1));
    tile_max_lo = fmaxf(tile_max_lo, __shfl_xor_sync(0xffffffffu, tile_max_lo, 2));
    if (kHigh) {
      tile_max_hi = fmaxf(tile_max_hi, __shfl_xor_sync(0xffffffffu, tile_max_hi, 1));
      tile_max_hi = fmaxf(tile_max_hi, __shfl_xor_sync(0xffffffffu, tile_max_hi, 2));
    }
    const float new_max_lo = fmaxf(run_max_lo, tile_max_lo);
    const float safe_lo = new_max_lo == -INFINITY ? 0.f : new_max_lo;
    const float corr_lo = exp2f((run_max_lo - safe_lo) * kLog2e);
    run_max_lo = new_max_lo;
    float corr_hi = 1.f, safe_hi = 0.f;
    if (kHigh) {
      const float new_max_hi = fmaxf(run_max_hi, tile_max_hi);
      safe_hi = new_max_hi == -INFINITY ? 0.f : new_max_hi;
      corr_hi = exp2f((run_max_hi - safe_hi) * kLog2e);
      run_max_hi = new_max_hi;
    }
    float p[2][4];
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p[nb][e] = exp2f((s[nb][e] - safe_lo) * kLog2e);
        sum_lo += p[nb][e];
        if (kHigh) {
          p[nb][2 + e] = exp2f((s[nb][2 + e] - safe_hi) * kLog2e);
          sum_hi += p[nb][2 + e];
        } else {
          p[nb][2 + e] = 0.f;
        }
      }
    }
    run_sum_lo = run_sum_lo * corr_lo + sum_lo;
    if (kHigh) {
      run_sum_hi = run_sum_hi * corr_hi + sum_hi;
    }
    const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]);
    const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]);
    const uint32_t pa1 = kHigh ? pack_bf16(p[0][2], p[0][3]) : 0u;
    const uint32_t pa3 = kHigh ? pack_bf16(p[1][2], p[1][3]) : 0u;

    // ---- O = O * corr + P V ----
#pragma unroll
    for (int dd = 0; dd < 8; ++dd) {
      uint32_t b0, b1, b2, b3;
      const uint32_t addr =
          v_u32 + ((lane & 7) + 8 * ((lane >> 3) & 1)) * kRowPitch + (2 * dd + (lane >> 4)) * 16;
      ldmatrix_x4_trans(addr, b0, b1, b2, b3);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float* o = acc[2 * dd + half];
        o[0] *= corr_lo;
        o[1] *= corr_lo;
        if (kHigh) {
          o[2] *= corr_hi;
          o[3] *= corr_hi;
        }
      }
      mma_bf16_16816(acc[2 * dd], pa0, pa1, pa2, pa3, b0, b1);
      mma_bf16_16816(acc[2 * dd + 1], pa0, pa1, pa2, pa3, b2, b3);
    }

    // ---- fixed-order fp32 score of the group's first head (neighbour candidates) ----
    {
      const int half = lane >> 4;  // 0: slices 0,4,2,6   1: slices 1,5,3,7
      const uint8_t* row = warp_rows + stage * kStageBytes + token_lane * kRowPitch;
      float part[4];
#pragma unroll
      for (int idx = 0; idx < 4; ++idx) {
        const int slice = (idx == 0 ? 0 : idx == 1 ? 4 : idx == 2 ? 2 : 6) + half;
        const uint4 r0 = *reinterpret_cast<const uint4*>(row + slice * 32);
        const uint4 r1 = *reinterpret_cast<const uint4*>(row + slice * 32 + 16);
        const float4* qp = reinterpret_cast<const float4*>(q_rep + slice * 16);
        const float4 q0 = qp[0], q1 = qp[1], q2 = qp[2], q3 = qp[3];
        float v = __fmul_rn(bf16_lo(r0.x), q0.x);
        v = __fmaf_rn(bf16_hi(r0.x), q0.y, v);
        v = __fmaf_rn(bf16_lo(r0.y), q0.z, v);
        v = __fmaf_rn(bf16_hi(r0.y), q0.w, v);
        v = __fmaf_rn(bf16_lo(r0.z), q1.x, v);
        v = __fmaf_rn(bf16_hi(r0.z), q1.y, v);
        v = __fmaf_rn(bf16_lo(r0.w), q1.z, v);
        v = __fmaf_rn(bf16_hi(r0.w), q1.w, v);
        v = __fmaf_rn(bf16_lo(r1.x), q2.x, v);
        v = __fmaf_rn(bf16_hi(r1.x), q2.y, v);
        v = __fmaf_rn(bf16_lo(r1.y), q2.z, v);
        v = __fmaf_rn(bf16_hi(r1.y), q2.w, v);
        v = __fmaf_rn(bf16_lo(r1.z), q3.x, v);
        v = __fmaf_rn(bf16_hi(r1.z), q3.y, v);
        v = __fmaf_rn(bf16_lo(r1.w), q3.z, v);
        v = __fmaf_rn(bf16_hi(r1.w), q3.w, v);
        part[idx] = v;
      }
      float total = __fadd_rn(__fadd_rn(part[0], part[1]), __fadd_rn(part[2], part[3]));
      total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, 16));
      if (lane < 16 && my_pos >= 0) {
        const int logical = warp_token0 + step * 16 + token_lane;
        const float candidate = logical < a.num_sink ? -INFINITY : __fmul_rn(total, scale);
        const uint64_t packed = (static_cast<uint64_t>(ordered_key32(candidate)) << 32) |
                                (0xffffffffu - static_cast<uint32_t>(my_pos));
        top_insert(top, packed);
      }
    }

    __syncwarp();
    if (step + kStages < steps) {
      fence_proxy_async();
      issue(step + kStages);
    }
  }

  if (failed) {
    // Give the copies still in flight a bounded chance to land before the
    // shared memory is released, then report and leave without writing.
    for (int s = 0; s < kStages; ++s) {
      mbar_wait_bounded(bar_base + s * 8, 0, 1u << 16);
      mbar_wait_bounded(bar_base + s * 8, 1, 1u << 16);
    }
    if (lane == 0 && a.status != nullptr) {
      atomicOr(a.status, CKV_DEV_WAIT_TIMEOUT);
    }
  }
  const int any_failed = __syncthreads_or(failed ? 1 : 0);
  if (any_failed) {
    return;
  }

  // ---- per-warp epilogue: finish the row sums, park (max, sum, acc) in this
  // warp's (now idle) staging area ----
  run_sum_lo += __shfl_xor_sync(0xffffffffu, run_sum_lo, 1);
  run_sum_lo += __shfl_xor_sync(0xffffffffu, run_sum_lo, 2);
  if (kHigh) {
    run_sum_hi += __shfl_xor_sync(0xffffffffu, run_sum_hi, 1);
    run_sum_hi += __shfl_xor_sync(0xffffffffu, run_sum_hi, 2);
  }
  float* park = reinterpret_cast<float*>(warp_rows);  // [group][130]
  if (g_row < group) {
    float* dst = park + g_row * kPartialStride;
    if (t_col == 0) {
      dst[0] = run_max_lo;
      dst[1] = run_sum_lo;
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      dst[2 + n * 8 + 2 * t_col] = acc[n][0];
      dst[2 + n * 8 + 2 * t_col + 1] = acc[n][1];
    }
  }
  if (kHigh && g_row + 8 < group) {
    float* dst = park + (g_row + 8) * kPartialStride;
    if (t_col == 0) {
      dst[0] = run_max_hi;
      dst[1] = run_sum_hi;
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      dst[2 + n * 8 + 2 * t_col] = acc[n][2];
      dst[2 + n * 8 + 2 * t_col + 1] = acc[n][3];
    }
  }

  // warp-level top-8 of the lanes' sorted lists
  {
    int cursor = 0;
    for (int k = 0; k < kKappa; ++k) {
      uint64_t head = 0ull;
#pragma unroll
      for (int slot = 0; slot < kKappa; ++slot) {
        head = cursor == slot ? top[slot] : head;
      }
      const uint64_t best = warp_max_u64(head);
      if (lane == 0) {
        top_s[warp * kKappa + k] = best;
      }
      if (best != 0ull && head == best) {
        ++cursor;
      }
    }
  }
  __syncthreads();

  // ---- merge the four warps and write one partial per head ----
  const int d = threadIdx.x;  // one output dimension per thread
  float* partial = a.partials + ((static_cast<int64_t>(flat) * a.splits + split) * group) *
                                    kPartialStride;
  for (int g = 0; g < group; ++g) {
    float m[kAttnWarps];
    float best = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      m[w] = reinterpret_cast<const float*>(smem + w * kWarpBytes)[g * kPartialStride];
      best = fmaxf(best, m[w]);
    }
    const float safe = best == -INFINITY ? 0.f : best;
    float sum = 0.f;
    float out = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* src = reinterpret_cast<const float*>(smem + w * kWarpBytes) + g * kPartialStride;
      const float weight = exp2f((m[w] - safe) * kLog2e);
      sum += src[1] * weight;
      out += src[2 + d] * weight;
    }
    float* dst = partial + g * kPartialStride;
    if (d == 0) {
      dst[0] = best;
      dst[1] = sum;
    }
    dst[2 + d] = out;
  }
  if (warp == 0) {
    uint64_t mine = top_s[lane];
    uint64_t* out = a.partial_topk + (static_cast<int64_t>(flat) * a.splits + split) * kKappa;
    for (int k = 0; k < kKappa; ++k) {
      const uint64_t best = warp_max_u64(mine);
      if (lane == 0) {
        out[k] = best;
      }
      if (best != 0ull && mine == best) {
        mine = 0ull;
      }
    }
  }
}

int attention_smem_bytes() { return AttnSmem::kTotal; }

cudaError_t launch_attention(const ckv_layer_args& a, cudaStream_t stream) {
  static bool configured[64] = {};
  const int device = a.device >= 0 && a.device < 64 ? a.device : 0;
  if (!configured[device]) {
    cudaError_t err = cudaFuncSetAttribute(attention_kernel<false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           AttnSmem::kTotal);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(attention_kernel<true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::kTotal);
    if (err != cudaSuccess) return err;
    configured[device] = true;
  }
  const dim3 grid(a.splits, a.batch * a.retrieval_heads);
  if (a.group_size > 8) {
    attention_kernel<true><<<grid, kAttnThreads, AttnSmem::kTotal, stream>>>(a);
  } else {
    attention_kernel<false><<<grid, kAttnThreads, AttnSmem::kTotal, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace ckv
