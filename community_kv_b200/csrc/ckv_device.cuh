// Device-side helpers shared by the sparse-decode kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ckv_b200.h"

namespace ckv {

constexpr int kHeadDim = CKV_HEAD_DIM;
constexpr int kTile = CKV_TILE;
constexpr int kKappa = CKV_KAPPA;
constexpr int kPartialStride = CKV_PARTIAL_STRIDE;
constexpr int kMaxDeltaWalk = 32;
constexpr float kLog2e = 1.4426950408889634f;

// Host-side argument validation (capi.cu): which groups of fields an entry point needs.
enum Need { kNeedScore = 1, kNeedSelect = 2, kNeedAttention = 4 };
int check(const ckv_layer_args* a, int need);

// One launch covers `batch * retrieval_heads` independent units.
struct Unit {
  int batch;
  int head;
  int graph;
  int kv;
};

__device__ __forceinline__ Unit make_unit(const ckv_layer_args& a, int flat) {
  Unit u;
  u.batch = flat / a.retrieval_heads;
  u.head = flat - u.batch * a.retrieval_heads;
  u.graph = a.retrieval_to_graph[u.head];
  u.kv = a.retrieval_to_kv[u.head];
  return u;
}

__device__ __forceinline__ uint16_t ordered_key16(uint16_t bits) {
  return bits ^ ((bits & 0x8000u) ? 0xffffu : 0x8000u);
}

__device__ __forceinline__ uint32_t ordered_key32(float value) {
  const uint32_t bits = __float_as_uint(value);
  return (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
}

__device__ __forceinline__ float key32_to_float(uint32_t ordered) {
  const uint32_t bits = (ordered & 0x80000000u) ? (ordered ^ 0x80000000u) : ~ordered;
  return __uint_as_float(bits);
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) {
  return __uint_as_float(packed << 16);
}
__device__ __forceinline__ float bf16_hi(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}

// Four e4m3 bytes -> four fp32 values (exact).
__device__ __forceinline__ void fp8x4_to_float(uint32_t word, float* out) {
  const __half2_raw lo =
      __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(word & 0xffffu), __NV_E4M3);
  const __half2_raw hi =
      __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(word >> 16), __NV_E4M3);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  out[0] = a.x;
  out[1] = a.y;
  out[2] = b.x;
  out[3] = b.y;
}

// Packed two-wide fp32 arithmetic (sm_100): each half is an IEEE round-to-nearest
// operation, identical to the scalar instruction.
__device__ __forceinline__ uint64_t pack_f32x2(float low, float high) {
  uint64_t packed;
  asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "f"(low), "f"(high));
  return packed;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t packed, float& low, float& high) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(packed));
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// Four e4m3 bytes -> two packed bf16 pairs (exact; NaN encodings are not handled:
// the saturating centroid update never produces them).  The seven magnitude bits
// go to the top of the bf16 exponent/mantissa field, which reads as the value
// times 2^-120 with e4m3 subnormals landing on bf16 subnormals; a bf16 multiply
// by 2^120 restores the scale.  Integer and FMA pipes only.
__device__ __forceinline__ void e4m3x4_to_bf16x2(uint32_t word, uint32_t& low, uint32_t& high) {
  const uint32_t spread_low = __byte_perm(word, 0u, 0x1404);   // (b1 << 24) | (b0 << 8)
  const uint32_t spread_high = __byte_perm(word, 0u, 0x3424);  // (b3 << 24) | (b2 << 8)
  const uint32_t tiny_low = ((spread_low >> 4) & 0x07f007f0u) | (spread_low & 0x80008000u);
  const uint32_t tiny_high = ((spread_high >> 4) & 0x07f007f0u) | (spread_high & 0x80008000u);
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(low) : "r"(tiny_low), "r"(0x7b807b80u));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(high) : "r"(tiny_high), "r"(0x7b807b80u));
}

// acc += a.lo*b.lo ; acc += a.hi*b.hi  with bf16 operands, fp32 accumulate, each
// step rounded once (the product of two bf16 values is exact in fp32).
__device__ __forceinline__ float fma2_bf16(uint32_t a, uint32_t b, float acc) {
  asm("{\n"
      ".reg .b16 al, ah, bl, bh;\n"
      "mov.b32 {al, ah}, %1;\n"
      "mov.b32 {bl, bh}, %2;\n"
      "fma.rn.f32.bf16 %0, al, bl, %0;\n"
      "fma.rn.f32.bf16 %0, ah, bh, %0;\n"
      "}\n"
      : "+f"(acc)
      : "r"(a), "r"(b));
  return acc;
}

// Running mean of a centroid element, (old * n + key) / (n + 1), before it is stored
// as e4m3.  `reference_division` selects the approximate division the reference's
// compiled kernel uses; otherwise the division is IEEE round-to-nearest.
__device__ __forceinline__ float centroid_mean(float old_value, int old_size, float key_value,
                                               bool reference_division) {
  const float numerator = __fadd_rn(__fmul_rn(old_value, static_cast<float>(old_size)), key_value);
  const float denominator = static_cast<float>(old_size + 1);
  if (reference_division) {
    float quotient;
    asm("div.full.f32 %0, %1, %2;" : "=f"(quotient) : "f"(numerator), "f"(denominator));
    return quotient;
  }
  return __fdiv_rn(numerator, denominator);
}

// Optional phase timestamps of the single-launch decode path (see ckv_layer_args).
__device__ __forceinline__ void phase_stamp(const ckv_layer_args& a, int flat, int rank, int slot) {
  if (a.phase_times != nullptr && threadIdx.x == 0) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    a.phase_times[(static_cast<int64_t>(flat) * 8 + rank) * 16 + slot] = now;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

// Programmatic dependent launch: a kernel lets the next kernel in the stream
// start its prologue early, and waits for its own predecessor's results just
// before it first reads them.
__device__ __forceinline__ void pdl_release_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_for_predecessor() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Host side: launch with the programmatic-serialisation attribute.
template <typename Kernel>
inline cudaError_t launch_dependent(Kernel kernel, dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, const ckv_layer_args& a) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, a);
}

// 16-byte asynchronous global -> shared copy (L2 only); src_bytes 0 zero-fills.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
// 4-byte variant (through L1).
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// ---- warp-level tensor-core helpers (legacy mma path; the decode tiles are
// 16 x 8 and HBM-bound, far below a tcgen05 tile) ----
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float low, float high) {
  const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
  return *reinterpret_cast<const uint32_t*>(&pair);
}

__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t value, int mask) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(value), mask);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, static_cast<uint32_t>(value >> 32), mask);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t value) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const uint64_t other = shfl_xor_u64(value, offset);
    value = other > value ? other : value;
  }
  return value;
}

// Newest-first member of a community's decode-delta chain, or 0 when the chain
// ends early (the same default the reference's masked load yields).
__device__ __forceinline__ int delta_member_position(const ckv_layer_args& a, int64_t graph_slot,
                                                     int community, int member) {
  const int64_t chunk_base = graph_slot * a.chunks_per_graph;
  int chunk = a.community_tail[graph_slot * a.community_capacity + community];
  int remaining = member;
  for (int step = 0; step < kMaxDeltaWalk && chunk >= 0; ++step) {
    const int size = a.chunk_size[chunk_base + chunk];
    if (remaining < size) {
      const int start = a.chunk_start[chunk_base + chunk];
      return a.delta_positions[graph_slot * a.delta_position_capacity + start + size - 1 -
                               remaining];
    }
    remaining -= size;
    chunk = a.chunk_previous[chunk_base + chunk];
  }
  return 0;
}

// Cache row of logical token `logical` (0..T-1) of one unit, -1 when masked.
// `ends` / `comms` are the unit's descriptor arrays (global or shared memory).
__device__ __forceinline__ int resolve_token(const ckv_layer_args& a, const Unit& u,
                                             const int32_t* ends, const int32_t* comms,
                                             int logical, int descriptor_count) {
  const int64_t graph_slot = static_cast<int64_t>(u.batch) * a.graphs + u.graph;
  if (logical < a.num_sink) {
    return a.sink_positions[logical];
  }
  if (logical == a.token_budget - 1) {
    return a.current_position[graph_slot];
  }
  const int offset = logical - a.num_sink;
  int low = 0;
  int high = descriptor_count;
  while (low < high) {
    const int middle = (low + high) >> 1;
    if (ends[middle] <= offset) {
      low = middle + 1;
    } else {
      high = middle;
    }
  }
  if (low >= descriptor_count) {
    return -1;  // budget under-filled: nothing selected for this slot
  }
  const int previous_end = low > 0 ? ends[low - 1] : 0;
  const int member = offset - previous_end;
  const int community = comms[low];
  const int delta_count = a.delta_sizes[graph_slot * a.community_capacity + community];
  if (member < delta_count) {
    return delta_member_position(a, graph_slot, community, member);
  }
  const int start = a.member_offsets[graph_slot * (a.community_capacity + 1) + community];
  return a.member_positions[graph_slot * a.member_capacity + start + member - delta_count];
}

}  // namespace ckv
