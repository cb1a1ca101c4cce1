// Device function of the gather + segmented flash-decode attention, shared by the
// stand-alone kernel and the fused per-layer cluster kernel (sm_100a).
#pragma once

#include "ckv_device.cuh"

namespace ckv {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = 4;
constexpr int kStages = 2;
constexpr int kStepTokens = 16;
constexpr int kRowPitch = 272;                     // bytes between staged rows
constexpr int kStageBytes = 32 * kRowPitch;        // 16 K rows + 16 V rows
constexpr int kWarpBytes = kStages * kStageBytes;  // 17408

struct AttnSmem {
  static constexpr int kRowsBytes = kAttnWarps * kWarpBytes;              // 69632
  static constexpr int kQrepOffset = kRowsBytes;                          // 128 bf16
  static constexpr int kTopOffset = kQrepOffset + kHeadDim * 2;           // 4 x 8 u64
  static constexpr int kTotal = kTopOffset + kAttnWarps * kKappa * 8;
};

__device__ __forceinline__ float dot16_bf16(const uint8_t* row, const uint8_t* q) {
  const uint4 r0 = *reinterpret_cast<const uint4*>(row);
  const uint4 r1 = *reinterpret_cast<const uint4*>(row + 16);
  const uint4 q0 = *reinterpret_cast<const uint4*>(q);
  const uint4 q1 = *reinterpret_cast<const uint4*>(q + 16);
  float v = 0.f;
  v = fma2_bf16(r0.x, q0.x, v);
  v = fma2_bf16(r0.y, q0.y, v);
  v = fma2_bf16(r0.z, q0.z, v);
  v = fma2_bf16(r0.w, q0.w, v);
  v = fma2_bf16(r1.x, q1.x, v);
  v = fma2_bf16(r1.y, q1.y, v);
  v = fma2_bf16(r1.z, q1.z, v);
  v = fma2_bf16(r1.w, q1.w, v);
  return v;
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t value) {
  uint32_t out;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(out) : "r"(value));
  return out;
}

// kBlocks = number of 8-head blocks of the query group (1 for G <= 8, 2 for G <= 16).
// One CTA of 128 threads: split `split` of unit `flat`; `smem` is AttnSmem::kTotal
// bytes, 128-byte aligned.  Writes one (acc, max, sum) partial per head and the
// split's eight best neighbour candidates.
template <int kBlocks>
__device__ __forceinline__ void attention_split(const ckv_layer_args& a, int flat, int split,
                                                uint8_t* smem) {
  const Unit u = make_unit(a, flat);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = a.group_size;

  // contiguous runs of 16-token steps: CTA, then warp
  const int steps_total = a.token_budget / kStepTokens;
  const int cta_begin = static_cast<int>(static_cast<int64_t>(split) * steps_total / a.splits);
  const int cta_end = static_cast<int>(static_cast<int64_t>(split + 1) * steps_total / a.splits);
  const int cta_steps = cta_end - cta_begin;
  const int warp_begin = cta_begin + warp * cta_steps / kAttnWarps;
  const int warp_end = cta_begin + (warp + 1) * cta_steps / kAttnWarps;
  const int steps = warp_end - warp_begin;
  const int warp_token0 = warp_begin * kStepTokens;

  uint8_t* warp_rows = smem + warp * kWarpBytes;
  uint8_t* q_rep = smem + AttnSmem::kQrepOffset;
  uint64_t* top_s = reinterpret_cast<uint64_t*>(smem + AttnSmem::kTopOffset);

  const __nv_bfloat16* query = reinterpret_cast<const __nv_bfloat16*>(a.query) +
                               (static_cast<int64_t>(u.batch) * a.retrieval_heads + u.head) *
                                   group * kHeadDim;
  if (threadIdx.x < kHeadDim / 2) {
    reinterpret_cast<uint32_t*>(q_rep)[threadIdx.x] =
        reinterpret_cast<const uint32_t*>(query)[threadIdx.x];
  }
  __syncthreads();

  const int32_t* positions = a.positions + static_cast<int64_t>(flat) * a.token_budget;
  // With a sequence-sharded cache only rows [begin, begin+count) are local: other
  // selected rows become masked slots here and are attended to by their owner.
  // A row at or beyond the cache's capacity (the cursor of a full cache, a corrupt member
  // list) is a masked slot too: it is never read.
  const int row_begin = a.kv_row_count > 0 ? a.kv_row_begin : 0;
  const int row_end = a.kv_row_count > 0 ? min(a.kv_row_begin + a.kv_row_count, a.sequence_capacity)
                                         : a.sequence_capacity;
  auto local_row = [&](int pos) { return (pos >= row_begin && pos < row_end) ? pos - row_begin : -1; };
  const __nv_bfloat16* key_head = reinterpret_cast<const __nv_bfloat16*>(a.key) +
                                  u.batch * a.key_batch_stride + u.kv * a.key_head_stride;
  const __nv_bfloat16* value_head = reinterpret_cast<const __nv_bfloat16*>(a.value) +
                                    u.batch * a.value_batch_stride + u.kv * a.value_head_stride;
  const int token_lane = lane & 15;
  const uint32_t rows_u32 = smem_u32(warp_rows);

  // One step = 32 rows.  Half-warp `lane >> 4` copies rows 2j + (lane >> 4), lane & 15
  // picks the 16-byte piece of the row.  Every lane holds the position of token lane & 15.
  const int piece = lane & 15;
  const int row_half = lane >> 4;
  auto issue = [&](int step, int pos) {
    const uint32_t dst = rows_u32 + (step % kStages) * kStageBytes + piece * 16;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int row = 2 * j + row_half;
      const int row_pos = __shfl_sync(0xffffffffu, pos, row);
      const int64_t safe = row_pos > 0 ? row_pos : 0;
      const uint32_t bytes = row_pos >= 0 ? 16u : 0u;  // 0: zero-fill, nothing is read
      cp_async16(dst + row * kRowPitch, key_head + safe * a.key_row_stride + piece * 8, bytes);
      cp_async16(dst + (16 + row) * kRowPitch, value_head + safe * a.value_row_stride + piece * 8,
                 bytes);
    }
  };

  // positions of the steps in flight (this lane's token) and of the next one
  static_assert(kStages == 2, "the position ring below is written for two stages");
  int pos_even = 0 < steps ? local_row(positions[warp_token0 + token_lane]) : -1;
  int pos_odd = 1 < steps ? local_row(positions[warp_token0 + kStepTokens + token_lane]) : -1;
  if (0 < steps) {
    issue(0, pos_even);
  }
  cp_async_commit();
  if (1 < steps) {
    issue(1, pos_odd);
  }
  cp_async_commit();

  // B fragments of Q^T: b0 = q[head g][16ks + 2t .. +1], b1 = the same + 8
  const int g_row = lane >> 2;
  const int t_col = lane & 3;
  uint32_t qb[kBlocks][8][2];
#pragma unroll
  for (int hb = 0; hb < kBlocks; ++hb) {
    const int head = hb * 8 + g_row;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qb[hb][ks][0] = qb[hb][ks][1] = 0u;
      if (head < group) {
        const __nv_bfloat16* src = query + head * kHeadDim + ks * 16 + 2 * t_col;
        qb[hb][ks][0] = *reinterpret_cast<const uint32_t*>(src);
        qb[hb][ks][1] = *reinterpret_cast<const uint32_t*>(src + 8);
      }
    }
  }

  // O^T accumulators: acc[hb][mb] covers d = 16mb + g (+8), heads 8hb + 2t, +1
  float acc[kBlocks][8][4];
  float run_max[kBlocks][2], run_sum[kBlocks][2];
#pragma unroll
  for (int hb = 0; hb < kBlocks; ++hb) {
    run_max[hb][0] = run_max[hb][1] = -INFINITY;
    run_sum[hb][0] = run_sum[hb][1] = 0.f;
#pragma unroll
    for (int mb = 0; mb < 8; ++mb) {
      acc[hb][mb][0] = acc[hb][mb][1] = acc[hb][mb][2] = acc[hb][mb][3] = 0.f;
    }
  }
  // warp-wide top-8 neighbour candidates: lane j (<8) holds the j-th best
  uint64_t warp_top = 0ull;
  uint64_t warp_floor = 0ull;  // current 8th best (0 while fewer than 8)
  const float scale = a.softmax_scale;

  for (int step = 0; step < steps; ++step) {
    const int stage = step % kStages;
    // position of the token this lane will fetch for step + kStages (prefetch now)
    const int next_step = step + kStages;
    const int next_pos =
        next_step < steps ? local_row(positions[warp_token0 + next_step * kStepTokens + token_lane]) : -1;
    cp_async_wait<kStages - 1>();  // this step's group has landed (one younger group may be pending)
    __syncwarp();
    const uint32_t k_u32 = rows_u32 + stage * kStageBytes;
    const uint32_t v_u32 = k_u32 + 16 * kRowPitch;
    const int my_pos = stage ? pos_odd : pos_even;
    const unsigned valid_bits = __ballot_sync(0xffffffffu, my_pos >= 0) & 0xffffu;
    const bool ok_lo = (valid_bits >> g_row) & 1u;        // token g
    const bool ok_hi = (valid_bits >> (g_row + 8)) & 1u;  // token g + 8

    // ---- S^T = K Q^T : 16 tokens x 8 heads per block, two interleaved chains ----
    float s[kBlocks][4];
    {
      float even[kBlocks][4], odd[kBlocks][4];
#pragma unroll
      for (int hb = 0; hb < kBlocks; ++hb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          even[hb][e] = 0.f;
          odd[hb][e] = 0.f;
        }
      }
      const uint32_t a_base = k_u32 + ((lane & 7) + 8 * ((lane >> 3) & 1)) * kRowPitch + (lane >> 4) * 16;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(a_base + ks * 32, a0, a1, a2, a3);
#pragma unroll
        for (int hb = 0; hb < kBlocks; ++hb) {
          mma_bf16_16816((ks & 1) ? odd[hb] : even[hb], a0, a1, a2, a3, qb[hb][ks][0], qb[hb][ks][1]);
        }
      }
#pragma unroll
      for (int hb = 0; hb < kBlocks; ++hb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[hb][e] = even[hb][e] + odd[hb][e];
        }
      }
    }

    // ---- online softmax per head (heads 2t, 2t+1 of each block live on this lane) ----
    uint32_t pb[kBlocks][2];
    bool rescale = false;
    float corr[kBlocks][2];
#pragma unroll
    for (int hb = 0; hb < kBlocks; ++hb) {
      s[hb][0] = ok_lo ? s[hb][0] * scale : -INFINITY;
      s[hb][1] = ok_lo ? s[hb][1] * scale : -INFINITY;
      s[hb][2] = ok_hi ? s[hb][2] * scale : -INFINITY;
      s[hb][3] = ok_hi ? s[hb][3] * scale : -INFINITY;
      float p[4];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float tile_max = fmaxf(s[hb][e], s[hb][2 + e]);
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
        const float new_max = fmaxf(run_max[hb][e], tile_max);
        const float safe = new_max == -INFINITY ? 0.f : new_max;
        corr[hb][e] = exp2f((run_max[hb][e] - safe) * kLog2e);
        rescale = rescale || (new_max != run_max[hb][e]);
        run_max[hb][e] = new_max;
        p[e] = exp2f((s[hb][e] - safe) * kLog2e);
        p[2 + e] = exp2f((s[hb][2 + e] - safe) * kLog2e);
        run_sum[hb][e] = run_sum[hb][e] * corr[hb][e] + p[e] + p[2 + e];
      }
      // accumulator layout (token g | g+8, heads 2t,2t+1) -> operand layout
      // (tokens 2t,2t+1 | +8, head g)
      pb[hb][0] = movmatrix_trans(pack_bf16(p[0], p[1]));
      pb[hb][1] = movmatrix_trans(pack_bf16(p[2], p[3]));
    }
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
      for (int hb = 0; hb < kBlocks; ++hb) {
#pragma unroll
        for (int mb = 0; mb < 8; ++mb) {
          acc[hb][mb][0] *= corr[hb][0];
          acc[hb][mb][1] *= corr[hb][1];
          acc[hb][mb][2] *= corr[hb][0];
          acc[hb][mb][3] *= corr[hb][1];
        }
      }
    }

    // ---- O^T += V^T P^T ----
    {
      const uint32_t v_base = v_u32 + ((lane & 7) + 8 * (lane >> 4)) * kRowPitch + ((lane >> 3) & 1) * 16;
#pragma unroll
      for (int mb = 0; mb < 8; ++mb) {
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4_trans(v_base + mb * 32, a0, a1, a2, a3);
#pragma unroll
        for (int hb = 0; hb < kBlocks; ++hb) {
          mma_bf16_16816(acc[hb][mb], a0, a1, a2, a3, pb[hb][0], pb[hb][1]);
        }
      }
    }

    // ---- fixed-order fp32 score of the group's first head (neighbour candidates) ----
    {
      const int half = lane >> 4;  // 0: slices 0,4,2,6   1: slices 1,5,3,7
      const uint8_t* row = warp_rows + stage * kStageBytes + token_lane * kRowPitch;
      const float p0 = dot16_bf16(row + (0 + half) * 32, q_rep + (0 + half) * 32);
      const float p1 = dot16_bf16(row + (4 + half) * 32, q_rep + (4 + half) * 32);
      const float p2 = dot16_bf16(row + (2 + half) * 32, q_rep + (2 + half) * 32);
      const float p3 = dot16_bf16(row + (6 + half) * 32, q_rep + (6 + half) * 32);
      float total = __fadd_rn(__fadd_rn(p0, p1), __fadd_rn(p2, p3));
      total = __fadd_rn(total, __shfl_xor_sync(0xffffffffu, total, 16));
      uint64_t candidate = 0ull;
      if (lane < 16 && my_pos >= 0) {
        const int logical = warp_token0 + step * kStepTokens + token_lane;
        const float score = logical < a.num_sink ? -INFINITY : __fmul_rn(total, scale);
        candidate = (static_cast<uint64_t>(ordered_key32(score)) << 32) |
                    (0xffffffffu - static_cast<uint32_t>(my_pos + row_begin));
      }
      unsigned pending = __ballot_sync(0xffffffffu, candidate > warp_floor);
      while (pending) {
        const int src = __ffs(pending) - 1;
        pending &= pending - 1;
        const uint64_t c = (static_cast<uint64_t>(__shfl_sync(0xffffffffu, static_cast<uint32_t>(candidate >> 32), src)) << 32) |
                           __shfl_sync(0xffffffffu, static_cast<uint32_t>(candidate), src);
        const uint32_t up_hi = __shfl_up_sync(0xffffffffu, static_cast<uint32_t>(warp_top >> 32), 1);
        const uint32_t up_lo = __shfl_up_sync(0xffffffffu, static_cast<uint32_t>(warp_top), 1);
        const uint64_t above = (static_cast<uint64_t>(up_hi) << 32) | up_lo;
        if (lane < kKappa && c > warp_top) {
          warp_top = (lane > 0 && above < c) ? above : c;
        }
        warp_floor = (static_cast<uint64_t>(__shfl_sync(0xffffffffu, static_cast<uint32_t>(warp_top >> 32), kKappa - 1)) << 32) |
                     __shfl_sync(0xffffffffu, static_cast<uint32_t>(warp_top), kKappa - 1);
      }
    }

    __syncwarp();
    if (next_step < steps) {
      if (stage) {
        pos_odd = next_pos;
      } else {
        pos_even = next_pos;
      }
      issue(next_step, next_pos);
    }
    cp_async_commit();
  }
  cp_async_wait<0>();

  // ---- per-warp epilogue: finish the row sums, park (max, sum, acc) per head in
  // this warp's (now idle) staging area ----
  float* park = reinterpret_cast<float*>(warp_rows);  // [group][132]: acc[128], max, sum
#pragma unroll
  for (int hb = 0; hb < kBlocks; ++hb) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float sum = run_sum[hb][e];
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      const int head = hb * 8 + 2 * t_col + e;
      if (head < group) {
        float* dst = park + head * kPartialStride;
        if (g_row == 0) {
          dst[kHeadDim] = run_max[hb][e];
          dst[kHeadDim + 1] = sum;
        }
#pragma unroll
        for (int mb = 0; mb < 8; ++mb) {
          dst[mb * 16 + g_row] = acc[hb][mb][e];
          dst[mb * 16 + g_row + 8] = acc[hb][mb][2 + e];
        }
      }
    }
  }
  if (lane < kKappa) {
    top_s[warp * kKappa + lane] = warp_top;
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
      m[w] = reinterpret_cast<const float*>(smem + w * kWarpBytes)[g * kPartialStride + kHeadDim];
      best = fmaxf(best, m[w]);
    }
    const float safe = best == -INFINITY ? 0.f : best;
    float sum = 0.f;
    float out = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float* src = reinterpret_cast<const float*>(smem + w * kWarpBytes) + g * kPartialStride;
      const float weight = exp2f((m[w] - safe) * kLog2e);
      sum += src[kHeadDim + 1] * weight;
      out += src[d] * weight;
    }
    float* dst = partial + g * kPartialStride;
    if (d == 0) {
      dst[kHeadDim] = best;
      dst[kHeadDim + 1] = sum;
    }
    dst[d] = out;
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

}  // namespace ckv
