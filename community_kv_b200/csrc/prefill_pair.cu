// Prefill attention with the reference's top-8 rule, two heads per CTA (sm_100a).
//
// One CTA owns 128 consecutive positions of TWO query heads of one KV group (two
// 128-row tiles that share every K/V tile) and is split into roles:
//   warps 0-3  softmax of tile 0, one thread per row (all 128 columns of a key block);
//   warps 4-7  softmax of tile 1;
//   warp 8     one lane feeds the K and V rings (and Q) with bulk tensor copies;
//   warp 9     one lane issues every tcgen05.mma;
//   warps 10-11 idle: they complete the third warpgroup, which hands most of its
//              registers to the softmax warpgroups (setmaxnreg).
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  A softmax
// thread reads its row of S, and writes the bf16 probabilities back over the first 64
// columns of the same S buffer; O' = P V then takes its A operand straight from tensor
// memory, so P never touches shared memory.  The issuing lane alternates between the two
// tiles - S0, S1, then per key block [P0.V, next S0, P1.V, next S1] - so that one tile's
// softmax runs under the other tile's matrix products.  O stays in tensor memory for
// the whole row; a row's running maximum only moves when the new one is more than 2^8
// above it, and the row of O is then rescaled in place by its own thread.
// Every wait is bounded; a wait that runs out sets the status word and the CTA drains.
//
// The top-8 rule is the one of prefill_topk.cu (community-kv.patch,
// hopper/topk_warpselect.h): per row, four classes of columns (class = (j % 8) / 2)
// keep their six best packed candidates, the row reports the eight largest of the 24.

#include "tc_primitives.cuh"

namespace ckv {

namespace {

constexpr int kPairThreads = 384;  // three warpgroups: two of softmax rows, one of helpers

struct PairSmem {
  static constexpr int kQ = 0;                  // two query tiles
  static constexpr int kK = 2 * kTileBytes;     // two key stages
  static constexpr int kV = 4 * kTileBytes;     // two value stages
  static constexpr int kBars = 6 * kTileBytes;  // barriers, the TMEM slot, the abort flag
  static constexpr int kTotal = kBars + 256;
};

// Operand tiles sit in the 128-byte swizzled layout: [half of the 128 dims][row][128
// bytes], the 16-byte chunks of a row XOR-ed with the row's low three bits (what a bulk
// tensor copy with 128-byte swizzle writes); tiles start on 1024-byte boundaries.

// tcgen05.mma with the descriptors given as 32-bit words (both operands share the high word)
__device__ __forceinline__ void umma_words(uint32_t tmem_d, uint32_t a_low, uint32_t b_low,
                                           uint32_t high, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, {%6, %6, %6, %6}, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_low), "r"(b_low), "r"(high), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_ts_words(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_low,
                                              uint32_t high, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, {%6, %6, %6, %6}, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_low), "r"(high), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(0u)
      : "memory");
}

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two fp32 lanes per instruction (fma.rn.f32x2 / add.f32x2)
__device__ __forceinline__ uint64_t pack_pair(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_pair(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// Bounded wait that also gives up when another role of the CTA already has.  One thread.
// try_wait parks the thread in hardware for a while instead of spinning.
constexpr uint32_t kPairPolls = 1u << 18;
__device__ __forceinline__ bool pair_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort) {
  for (uint32_t poll = 0; poll < kPairPolls; ++poll) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) {
      return true;
    }
    if ((poll & 15u) == 15u && *abort != 0u) {
      return false;
    }
  }
  *abort = 1u;
  return false;
}

// The same for a whole warp: lane 0 polls, the others take its word.  The barrier's
// completion is made visible to the waiting lanes by one successful test of their own.
__device__ __forceinline__ bool pair_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort) {
  bool ok = true;
  if ((threadIdx.x & 31) == 0) {
    ok = pair_wait(bar, parity, abort);
  }
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (ok) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    (void)done;
  }
  return ok;
}

// The candidate key of the top-8 rule, clamp(rn((raw + 48) * 256)) to 15 bits, without the
// conversion instruction (it shares the special-function unit with the other tile's
// exponentials and would queue behind them): adding 1.5 * 2^23 leaves the integer, rounded
// to nearest even, in the low mantissa bits.
__device__ __forceinline__ uint32_t quantised_key_fma(float raw) {
  const float scaled = fminf(fmaxf(fmaf(raw, 256.0f, 12288.0f), 0.0f), 32767.0f);
  return __float_as_uint(scaled + 12582912.0f) & 0x7fffu;
}

// Insertion into a descending list by position: every slot decides by two comparisons
// whether it keeps its entry, takes the candidate or takes its left neighbour's entry.
template <int kDepth>
__device__ __forceinline__ void sorted_insert(uint32_t (&queue)[kDepth], uint32_t candidate) {
  bool keeps[kDepth];
#pragma unroll
  for (int k = 0; k < kDepth; ++k) {
    keeps[k] = queue[k] >= candidate;
  }
  uint32_t next[kDepth];
  next[0] = keeps[0] ? queue[0] : candidate;
#pragma unroll
  for (int k = 1; k < kDepth; ++k) {
    next[k] = keeps[k] ? queue[k] : (keeps[k - 1] ? candidate : queue[k - 1]);
  }
#pragma unroll
  for (int k = 0; k < kDepth; ++k) {
    queue[k] = next[k];
  }
}

template <int kMode>
__global__ void __launch_bounds__(kPairThreads, 1)
    prefill_pair_kernel(const ckv_prefill_args a, const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PairSmem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort = reinterpret_cast<volatile uint32_t*>(bars + 16);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int group = a.query_heads / a.kv_heads;
  const int pairs = group >> 1;
  const int tile = gridDim.x - 1 - blockIdx.x;  // longest rows first
  const int kv_head = blockIdx.y / pairs;
  const int head0 = kv_head * group + 2 * (blockIdx.y % pairs);
  const int batch = blockIdx.z;
  const int length = a.seq_len;
  const int pos0 = tile * kPfRows;
  const int blocks = tile + 1;  // key blocks 0 .. tile; the last one holds the diagonal

  const uint32_t q_addr = smem_u32(smem + PairSmem::kQ);
  const uint32_t k_addr = smem_u32(smem + PairSmem::kK);
  const uint32_t v_addr = smem_u32(smem + PairSmem::kV);
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_k_full = smem_u32(bars + 1);   // two stages
  const uint32_t bar_v_full = smem_u32(bars + 3);   // two stages
  const uint32_t bar_k_free = smem_u32(bars + 5);   // two stages: both tiles' S of that block done
  const uint32_t bar_s_full = smem_u32(bars + 9);   // per tile: S written
  const uint32_t bar_p_full = smem_u32(bars + 11);  // per tile: P written by its four warps
  const uint32_t bar_o_full = smem_u32(bars + 13);  // per tile: P.V folded into O

  // a wait already ran out somewhere in this launch: drain the grid quickly
  const bool drained = a.status != nullptr &&
                       (*reinterpret_cast<volatile uint32_t*>(a.status) & CKV_DEV_WAIT_TIMEOUT) != 0u;
  if (__syncthreads_or(drained ? 1 : 0)) {
    return;
  }
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 11; ++i) {
      mbar_init(bar_q + 8 * i, 1);
    }
    mbar_init(bar_p_full, 4);  // one arrival per softmax warp
    mbar_init(bar_p_full + 8, 4);
    mbar_init(bar_o_full, 1);
    mbar_init(bar_o_full + 8, 1);
    *abort = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool failed = false;

  // Register hand-over between the warpgroups.  setmaxnreg.inc blocks until the registers
  // are free, without any bound: the totals must never exceed what the launch allocated
  // (384 threads x 168 registers = 256 x 216 + 128 x 72).
  static_assert(256 * 216 + 128 * 72 <= kPairThreads * 168, "register hand-over exceeds the launch allocation");
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  }
  if (warp >= 10) {
    // nothing to do
  } else if (warp == 8) {
    // ---- producer ----
    if (lane == 0) {
      mbar_expect_tx(bar_q, 2 * kTileBytes);
      tma_issue_tile(q_addr, &map_q, bar_q, pos0, head0, batch);
      tma_issue_tile(q_addr + kTileBytes, &map_q, bar_q, pos0, head0 + 1, batch);
      for (int block = 0; block < blocks; ++block) {
        const int stage = block & 1;
        // K(block) goes where K(block - 2) was: free once both tiles' S(block - 2) is done
        if (block >= 2 && !pair_wait(bar_k_free + 8 * stage, ((block >> 1) - 1) & 1, abort)) {
          failed = true;
          break;
        }
        tma_load_tile(k_addr + stage * kTileBytes, &map_k, bar_k_full + 8 * stage, block * kPfKeys,
                      kv_head, batch);
        // V(block) goes where V(block - 2) was.  S(block - 1) is committed after both
        // P.V(block - 2) were issued, so that barrier covers the products that read the stage.
        if (block >= 2 && !pair_wait(bar_k_free + 8 * (stage ^ 1), ((block - 1) >> 1) & 1, abort)) {
          failed = true;
          break;
        }
        tma_load_tile(v_addr + stage * kTileBytes, &map_v, bar_v_full + 8 * stage, block * kPfKeys,
                      kv_head, batch);
      }
    }
  } else if (warp == 9) {
    // ---- matrix products ----
    if (lane == 0) {
      const uint32_t idesc_qk = instruction_descriptor(false);
      const uint32_t idesc_pv = instruction_descriptor(true);
      // Descriptors as (low, high) words: the high word (stride between 8-row groups,
      // version, swizzle mode) is the same for every operand, the low word is the
      // address in 16-byte units plus the leading-dimension offset; a step along the
      // reduction only adds a constant to the low word.
      const uint32_t desc_high = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t q_low = ((q_addr & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t k_low = ((k_addr & 0x3ffffu) >> 4) | (1u << 16);
      const uint32_t v_low = ((v_addr & 0x3ffffu) >> 4) | (((kTileBytes / 2) >> 4) << 16);
      auto issue_qk = [&](int t, int stage) {
        const uint32_t a_low = q_low + t * (kTileBytes >> 4);
        const uint32_t b_low = k_low + stage * (kTileBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // dims 16 ks .. 16 ks + 15: 32 bytes into the row of the half that holds them
          const uint32_t within = ((ks >> 2) * (kTileBytes / 2) + (ks & 3) * 32) >> 4;
          umma_words(tmem + t * 128u, a_low + within, b_low + within, desc_high, idesc_qk, ks > 0);
        }
        umma_commit(bar_s_full + 8 * t);
        if (t == 1) {
          umma_commit(bar_k_free + 8 * stage);
        }
      };
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t b_low = v_low + stage * (kTileBytes >> 4);
        // keys 16 ks .. 16 ks + 15: eight packed columns of P, sixteen 128-byte rows of
        // V in each half (the halves are the leading dimension, 8-key groups the stride)
        umma_ts_words(tmem + 256u + t * 128u, tmem + t * 128u, b_low, desc_high, idesc_pv, accumulate);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks) {
          umma_ts_words(tmem + 256u + t * 128u, tmem + t * 128u + ks * 8u, b_low + ks * (2048 >> 4),
                        desc_high, idesc_pv, true);
        }
      };
      if (pair_wait(bar_q, 0, abort) && pair_wait(bar_k_full, 0, abort)) {
        tc_fence_after();
        issue_qk(0, 0);
        issue_qk(1, 0);
        for (int block = 0; block < blocks && !failed; ++block) {
          const int stage = block & 1;
          const bool more = block + 1 < blocks;
          if (!pair_wait(bar_v_full + 8 * stage, (block >> 1) & 1, abort)) {
            failed = true;
            break;
          }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (!pair_wait(bar_p_full + 8 * t, block & 1, abort)) {
              failed = true;
              break;
            }
            tc_fence_after();
            issue_pv(t, stage, block > 0);
            if (!more) {
              umma_commit(bar_o_full + 8 * t);
            } else {
              if (t == 0 && !pair_wait(bar_k_full + 8 * (stage ^ 1), ((block + 1) >> 1) & 1, abort)) {
                failed = true;
                break;
              }
              tc_fence_after();
              issue_qk(t, stage ^ 1);
            }
          }
        }
      } else {
        failed = true;
      }
    }
  } else {
    // ---- softmax of tile t, one thread per row ----
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int t = warp >> 2;
    const int row = tid & (kPfRows - 1);
    const int row_pos = pos0 + row;
    const int row_head = head0 + t;
    const bool row_live = row_pos < length;
    const uint32_t lane_base = tmem + (((warp & 3) * 32u) << 16);
    const uint32_t s_addr = lane_base + t * 128u;
    const uint32_t o_addr = lane_base + 256u + t * 128u;
    const float scale_log2 = a.softmax_scale * kLog2e;
    float run_max = -INFINITY;  // of the raw (unscaled) scores
    float run_sum = 0.f;
    uint32_t q32[4][kLocalK];
    if constexpr (kMode == 1) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int k = 0; k < kLocalK; ++k) {
          q32[c][k] = 0u;
        }
      }
    }

    for (int block = 0; block < blocks; ++block) {
      const int key0 = block * kPfKeys;
      if (!pair_wait_warp(bar_s_full + 8 * t, block & 1, abort)) {
        failed = true;
        break;
      }
      tc_fence_after();
      uint32_t raw[4][32];
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        tmem_load32_issue(s_addr + part * 32u, raw[part]);
      }
      tmem_wait_load();
      float s[128];
#pragma unroll
      for (int c = 0; c < 128; ++c) {
        s[c] = __uint_as_float(raw[c >> 5][c & 31]);
      }
      // only the last block of a tile meets the diagonal: key pos0 + c, row pos0 + row
      if (block == blocks - 1) {
#pragma unroll
        for (int c = 0; c < 128; ++c) {
          s[c] = c <= row ? s[c] : -INFINITY;
        }
      }
      // eight independent chains (the compiler keeps the order of a single one)
      float part_max[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        part_max[i] = fmaxf(s[i], s[i + 8]);
      }
#pragma unroll
      for (int c = 16; c < 128; c += 16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          part_max[i] = fmaxf(part_max[i], fmaxf(s[c + i], s[c + i + 8]));
        }
      }
      const float tile_max = fmaxf(fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])),
                                   fmaxf(fmaxf(part_max[4], part_max[5]), fmaxf(part_max[6], part_max[7])));

      // The running maximum only moves when the new one lies more than 2^8 above it
      // (probabilities up to 256 are harmless in bf16 / fp32); moving it means rescaling
      // the row of O in tensor memory, once the product that still adds to it is done.
      const float new_max = fmaxf(run_max, tile_max);
      const bool move = new_max > run_max && (new_max - run_max) * scale_log2 > 8.0f;
      float corr = 1.f;
      if (move) {
        corr = run_max == -INFINITY ? 0.f : exp2_fast((run_max - new_max) * scale_log2);
        run_max = new_max;
        run_sum *= corr;
      }
      if (block > 0 && __any_sync(0xffffffffu, move)) {
        // P.V of the last block is done: this block's S was committed after it
#pragma unroll
        for (int part = 0; part < 4; ++part) {
          uint32_t o[32];
          tmem_load32_issue(o_addr + part * 32u, o);
          tmem_wait_load();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
          }
          tmem_store32_issue(o_addr + part * 32u, o);
        }
        tmem_wait_store();
      }
      // ---- probabilities, bf16 pairs, over the first 64 columns of this S buffer ----
      const float offset = (run_max == -INFINITY ? 0.f : run_max) * scale_log2;
      const uint64_t scale_pair = pack_pair(scale_log2, scale_log2);
      const uint64_t offset_pair = pack_pair(-offset, -offset);
      uint64_t sum_pair[2] = {0ull, 0ull};
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t packed[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int c = part * 64 + 2 * e;
          float x0, x1;
          unpack_pair(fma_pair(pack_pair(s[c], s[c + 1]), scale_pair, offset_pair), x0, x1);
          const float p0 = exp2_fast(x0);
          const float p1 = exp2_fast(x1);
          sum_pair[e & 1] = add_pair(sum_pair[e & 1], pack_pair(p0, p1));
          packed[e] = pack_bf16(p0, p1);
        }
        tmem_store32_issue(s_addr + part * 32u, packed);
      }
      {
        float a0, a1, b0, b1;
        unpack_pair(sum_pair[0], a0, a1);
        unpack_pair(sum_pair[1], b0, b1);
        run_sum += (a0 + a1) + (b0 + b1);
      }
      tmem_wait_store();
      tc_fence_before();
      // one arrival per warp: 128 arrivals on one barrier word queue up behind each other
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_p_full + 8 * t);
      }

      // The candidate bookkeeping runs from the scores still in registers while the tensor
      // cores work on this tile's P.V and next S: it is off the path between two blocks.
      if constexpr (kMode == 1) {
        if (key0 >= a.num_sink) {
          // A key that is below eight keys already held can never reach the output:
          // the second-best entries of the four classes are eight such keys, and so
          // are the top four of the two best classes.
          const uint32_t third0 = q32[0][3], third1 = q32[1][3], third2 = q32[2][3], third3 = q32[3][3];
          const uint32_t second_of_fourths =
              max(min(max(third0, third1), max(third2, third3)),
                  max(min(third0, third1), min(third2, third3)));
          const uint32_t row_floor = max(min(min(q32[0][1], q32[1][1]), min(q32[2][1], q32[3][1])),
                                         second_of_fourths);
          // smallest raw score whose quantised key can reach the floor, a little low
          const float gate = (row_floor >> 17) == 0u
                                 ? -3.0e38f
                                 : (static_cast<float>(row_floor >> 17) - 0.75f) * (1.0f / 256.0f) - 48.0f;
          // Class by class (32 of the 128 columns each; the larger of two partial maxima
          // is the class maximum, so a class without a taker in any row of the warp costs
          // one vote): the columns that reach the gate as a bit mask, then insertion in
          // rounds - every lane with a pending column inserts its next one per round.
          // Both the pick of the column's score (a binary tree over the index bits) and
          // the insertion (position by comparison) are shallow: one warp runs this alone
          // on its scheduler, so the depth of the dependency chain is what it costs.
#pragma unroll
          for (int cls = 0; cls < 4; ++cls) {
            if (!__any_sync(0xffffffffu, fmaxf(part_max[2 * cls], part_max[2 * cls + 1]) >= gate)) {
              continue;
            }
            uint32_t takers = 0u;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int c = (i >> 1) * 8 + cls * 2 + (i & 1);
              takers |= (s[c] >= gate ? 1u : 0u) << i;
            }
            while (__any_sync(0xffffffffu, takers != 0u)) {
              if (takers != 0u) {
                const int i = __ffs(takers) - 1;
                takers &= takers - 1;
                float pick[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) {
                  pick[m] = (i & 1) ? s[m * 8 + cls * 2 + 1] : s[m * 8 + cls * 2];
                }
#pragma unroll
                for (int width = 8, bit = 2; width >= 1; width >>= 1, bit <<= 1) {
#pragma unroll
                  for (int m = 0; m < width; ++m) {
                    pick[m] = (i & bit) ? pick[2 * m + 1] : pick[2 * m];
                  }
                }
                const int c = (i >> 1) * 8 + cls * 2 + (i & 1);
                const uint32_t candidate =
                    (quantised_key_fma(pick[0]) << 17) | (static_cast<uint32_t>(key0 + c) & 0x1ffffu);
                sorted_insert<kLocalK>(q32[cls], candidate);
              }
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < 128; ++c) {
            const int j = key0 + c;
            if (s[c] > -INFINITY && j >= a.num_sink) {
              const uint32_t candidate =
                  (quantised_key(s[c]) << 17) | (static_cast<uint32_t>(j) & 0x1ffffu);
              uint32_t(&queue)[kLocalK] = q32[(c & 7) >> 1];
              if (candidate > queue[kLocalK - 1]) {
                queue_insert<kLocalK>(queue, candidate);
              }
            }
          }
        }
      }
    }

    if (!failed) {
      if (!pair_wait_warp(bar_o_full + 8 * t, 0, abort)) {
        failed = true;
      }
    }
    if (!failed) {
      tc_fence_after();
      const float inverse = 1.f / run_sum;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.output) + batch * a.o_batch_stride +
                           static_cast<int64_t>(row_live ? row_pos : 0) * a.o_row_stride +
                           row_head * a.o_head_stride;
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        uint32_t o[32];
        tmem_load32_issue(o_addr + part * 32u, o);
        tmem_wait_load();
        if (row_live) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[d]) * inverse, __uint_as_float(o[d + 1]) * inverse);
            v.y = pack_bf16(__uint_as_float(o[d + 2]) * inverse, __uint_as_float(o[d + 3]) * inverse);
            v.z = pack_bf16(__uint_as_float(o[d + 4]) * inverse, __uint_as_float(o[d + 5]) * inverse);
            v.w = pack_bf16(__uint_as_float(o[d + 6]) * inverse, __uint_as_float(o[d + 7]) * inverse);
            *reinterpret_cast<uint4*>(dst + part * 32 + d) = v;
          }
        }
      }
      if (row_live) {
        const float lse = run_max * a.softmax_scale + logf(run_sum);
        const int64_t heads_total = a.query_heads;
        a.lse[(batch * heads_total + row_head) * length + row_pos] = lse;
        if constexpr (kMode == 1) {
          const int skip = a.num_sink + kKappa - 1;
          if (row_pos >= skip) {
            // merge the four sorted class queues: eight rounds of "largest head wins"
            int cursor[4] = {0, 0, 0, 0};
            const int64_t base =
                ((batch * heads_total + row_head) * (length - skip) + (row_pos - skip)) * kKappa;
            const float lse_log2 = lse * kLog2e;
#pragma unroll
            for (int rank = 0; rank < kKappa; ++rank) {
              uint32_t best = 0u;
              int winner = 0;
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint32_t head = 0u;
#pragma unroll
                for (int k = 0; k < kLocalK; ++k) {
                  head = cursor[c] == k ? q32[c][k] : head;
                }
                if (head > best) {
                  best = head;
                  winner = c;
                }
              }
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                cursor[c] += (c == winner) ? 1 : 0;
              }
              const float dequant = static_cast<float>(best >> 17) / 256.0f - 48.0f;
              a.topk_val[base + rank] = exp2f(dequant * scale_log2 - lse_log2);
              a.topk_idx[base + rank] = static_cast<int32_t>(best & 0x1ffffu);
            }
          }
        }
      }
    }
  }

  if (failed && a.status != nullptr) {
    atomicOr(a.status, CKV_DEV_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512)
                 : "memory");
  }
}

}  // namespace

cudaError_t launch_prefill_pair(const ckv_prefill_args& a, cudaStream_t stream) {
  const int group = a.query_heads / a.kv_heads;
  if (group < 2 || (group & 1) != 0 || (a.mode != 0 && a.mode != 1)) {
    return cudaErrorInvalidValue;
  }
  CUtensorMap map_q, map_k, map_v;
  if (!tile_map(&map_q, a.query, a, a.query_heads, a.q_row_stride, a.q_head_stride, a.q_batch_stride, true) ||
      !tile_map(&map_k, a.key, a, a.kv_heads, a.k_row_stride, a.k_head_stride, a.k_batch_stride, true) ||
      !tile_map(&map_v, a.value, a, a.kv_heads, a.v_row_stride, a.v_head_stride, a.v_batch_stride, true)) {
    return cudaErrorInvalidValue;
  }
  const dim3 grid((a.seq_len + kPfRows - 1) / kPfRows, a.kv_heads * (group / 2), a.batch);
  auto run = [&](auto kernel) -> cudaError_t {
    cudaError_t err =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kTotal);
    if (err != cudaSuccess) return err;
    kernel<<<grid, kPairThreads, PairSmem::kTotal, stream>>>(a, map_q, map_k, map_v);
    return cudaGetLastError();
  };
  return a.mode == 0 ? run(prefill_pair_kernel<0>) : run(prefill_pair_kernel<1>);
}

}  // namespace ckv
