// Edge list -> coalesced adjacency (sm_100a): the consumer of the prefill kernel's
// neighbour edges and the producer of the graph that the host-side partitioner works on.
//
// Reference: build_adjacency, community_kv/graph/partition.py:168-249.  Every row of a
// graph contributes kappa direct edges (row position -> neighbour, weight score * lam / 2)
// and, when lam < 1, kappa (kappa + 1) / 2 co-attention edges between its neighbours
// (weight score_a * score_b * (1 - lam), the diagonal included); an edge is stored as
// (min vertex, max vertex) with vertices numbered graph * seq_len + position, duplicates
// are merged by adding their weights, and the result is sorted by (min, max).
//
// The reference sorts with torch.unique and adds with scatter_add_.  Here: the raw edges
// are enumerated in the reference's order (all direct edges, then all co-attention edges),
// sorted by their 64-bit key with a stable least-significant-digit radix sort (8 bits per
// pass, only as many passes as the vertex count needs), and every run of equal keys is
// summed front to back by one thread - a stable sort keeps equal keys in enumeration
// order, so each weight is the same sequence of fp32 additions a sequential scatter-add
// performs: the result is bit-exact and independent of scheduling.  HBM-bound integer work:
// five passes over 12 bytes per raw edge; nothing here is shaped for the tensor cores.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ckv_b200.h"

namespace ckv {
namespace {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;                          // keys per thread and tile
constexpr int kSortTile = kSortThreads * kSortItems;   // 2048
constexpr int kScanThreads = 1024;
constexpr int kScanItems = 4;
constexpr int kScanTile = kScanThreads * kScanItems;   // 4096
constexpr uint64_t kInvalidKey = ~0ull;

// ---- device-wide exclusive scan of uint32 (three small launches) ----
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t value, uint32_t* warp_total, uint32_t* total) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  uint32_t inclusive = value;
#pragma unroll
  for (int delta = 1; delta < 32; delta <<= 1) {
    const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, delta);
    if (lane >= delta) inclusive += other;
  }
  if (lane == 31) warp_total[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    uint32_t running = lane < (blockDim.x >> 5) ? warp_total[lane] : 0u;
#pragma unroll
    for (int delta = 1; delta < 32; delta <<= 1) {
      const uint32_t other = __shfl_up_sync(0xffffffffu, running, delta);
      if (lane >= delta) running += other;
    }
    warp_total[lane] = running;
  }
  __syncthreads();
  const uint32_t before = warp > 0 ? warp_total[warp - 1] : 0u;
  if (total != nullptr) *total = warp_total[(blockDim.x >> 5) - 1];
  __syncthreads();
  return before + inclusive - value;
}

__global__ void __launch_bounds__(kScanThreads) scan_tiles_kernel(const uint32_t* in, uint32_t* out, int64_t n,
                                                                  uint32_t* tile_total) {
  __shared__ uint32_t warp_total[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + threadIdx.x * kScanItems;
  uint32_t item[kScanItems];
  uint32_t sum = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    item[i] = base + i < n ? in[base + i] : 0u;
    sum += item[i];
  }
  uint32_t total;
  uint32_t prefix = block_exclusive_scan(sum, warp_total, &total);
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (base + i < n) out[base + i] = prefix;
    prefix += item[i];
  }
  if (threadIdx.x == 0) tile_total[blockIdx.x] = total;
}

// One CTA: exclusive scan of the tile totals in place, any length.
__global__ void __launch_bounds__(kScanThreads) scan_totals_kernel(uint32_t* tile_total, int64_t tiles) {
  __shared__ uint32_t warp_total[32];
  __shared__ uint32_t carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int64_t base = 0; base < tiles; base += kScanThreads) {
    const int64_t index = base + threadIdx.x;
    const uint32_t value = index < tiles ? tile_total[index] : 0u;
    uint32_t total;
    const uint32_t prefix = block_exclusive_scan(value, warp_total, &total);
    if (index < tiles) tile_total[index] = carry + prefix;
    __syncthreads();
    if (threadIdx.x == 0) carry += total;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kScanThreads) scan_add_kernel(uint32_t* out, int64_t n, const uint32_t* tile_total) {
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile + threadIdx.x * kScanItems;
  const uint32_t add = tile_total[blockIdx.x];
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (base + i < n) out[base + i] += add;
  }
}

cudaError_t exclusive_scan(const uint32_t* in, uint32_t* out, int64_t n, uint32_t* tile_total, cudaStream_t stream) {
  const int64_t tiles = (n + kScanTile - 1) / kScanTile;
  scan_tiles_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, stream>>>(in, out, n, tile_total);
  scan_totals_kernel<<<1, kScanThreads, 0, stream>>>(tile_total, tiles);
  scan_add_kernel<<<static_cast<unsigned>(tiles), kScanThreads, 0, stream>>>(out, n, tile_total);
  return cudaGetLastError();
}

// ---- raw edges in the reference's enumeration order ----
// index < direct: (graph, row, k); else (graph, row, pair) with pairs in row-major upper-triangular order
__global__ void __launch_bounds__(256) edge_keys_kernel(const int32_t* topk_indices, const float* topk_scores,
                                                        const int64_t* query_positions, int64_t rows, int kappa,
                                                        int seq_len, int64_t vertices, float direct_scale,
                                                        float co_scale, int64_t direct, int64_t raw,
                                                        uint64_t* keys, float* weights) {
  const int pairs = kappa * (kappa + 1) / 2;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < raw;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint64_t key = kInvalidKey;
    float weight = 0.f;
    if (i < direct) {
      const int64_t line = i / kappa;  // graph * rows + row
      const int64_t graph = line / rows;
      const int32_t neighbour = topk_indices[i];
      if (neighbour >= 0 && neighbour < seq_len) {
        const int64_t a = query_positions[line] + graph * seq_len;
        const int64_t b = static_cast<int64_t>(neighbour) + graph * seq_len;
        key = static_cast<uint64_t>((a < b ? a : b) * vertices + (a < b ? b : a));
        weight = __fmul_rn(topk_scores[i], direct_scale);
      }
    } else {
      const int64_t j = i - direct;
      const int64_t line = j / pairs;
      int pair = static_cast<int>(j - line * pairs);
      int first = 0;
      while (pair >= kappa - first) {  // row `first` of the upper triangle holds kappa - first pairs
        pair -= kappa - first;
        ++first;
      }
      const int second = first + pair;
      const int64_t graph = line / rows;
      const int32_t u = topk_indices[line * kappa + first];
      const int32_t v = topk_indices[line * kappa + second];
      if (u >= 0 && u < seq_len && v >= 0 && v < seq_len) {
        const int64_t a = static_cast<int64_t>(u) + graph * seq_len;
        const int64_t b = static_cast<int64_t>(v) + graph * seq_len;
        key = static_cast<uint64_t>((a < b ? a : b) * vertices + (a < b ? b : a));
        weight = __fmul_rn(__fmul_rn(topk_scores[line * kappa + first], topk_scores[line * kappa + second]), co_scale);
      }
    }
    keys[i] = key;
    weights[i] = weight;
  }
}

// ---- one stable radix pass: digit = (key >> shift) & 255 ----
// Tile t covers items [t * 2048, (t + 1) * 2048); item order inside a tile is round-major
// (round r holds items r * 256 .. r * 256 + 255), which both kernels below walk in order.
__global__ void __launch_bounds__(kSortThreads) radix_count_kernel(const uint64_t* keys, int64_t n, int shift,
                                                                   int64_t tiles, uint32_t* table) {
  __shared__ uint32_t count[256];
  count[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSortTile;
#pragma unroll
  for (int r = 0; r < kSortItems; ++r) {
    const int64_t index = base + r * kSortThreads + threadIdx.x;
    if (index < n) {
      atomicAdd(&count[(keys[index] >> shift) & 255u], 1u);
    }
  }
  __syncthreads();
  table[static_cast<int64_t>(threadIdx.x) * tiles + blockIdx.x] = count[threadIdx.x];  // digit-major
}

__global__ void __launch_bounds__(kSortThreads) radix_scatter_kernel(const uint64_t* keys, const float* weights,
                                                                     int64_t n, int shift, int64_t tiles,
                                                                     const uint32_t* table, uint64_t* keys_out,
                                                                     float* weights_out) {
  __shared__ uint32_t digit_base[256];                     // where the tile's next item of a digit goes
  __shared__ uint32_t round_base[256];                     // the same, at the start of the current round
  __shared__ uint16_t warp_count[kSortThreads / 32][256];  // this sorting pass, per warp and digit
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  digit_base[threadIdx.x] = table[static_cast<int64_t>(threadIdx.x) * tiles + blockIdx.x];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSortTile;
  for (int r = 0; r < kSortItems; ++r) {
#pragma unroll
    for (int w = 0; w < kSortThreads / 32; ++w) {
      warp_count[w][threadIdx.x] = 0;
    }
    __syncthreads();
    const int64_t index = base + r * kSortThreads + threadIdx.x;
    const bool live = index < n;
    const uint64_t key = live ? keys[index] : 0ull;
    const float weight = live ? weights[index] : 0.f;
    const uint32_t digit = static_cast<uint32_t>(key >> shift) & 255u;
    // lanes of this warp that hold the same digit (eight ballots instead of a match instruction)
    unsigned peers = __ballot_sync(0xffffffffu, live);
#pragma unroll
    for (int bit = 0; bit < 8; ++bit) {
      const unsigned votes = __ballot_sync(0xffffffffu, (digit >> bit) & 1u);
      peers &= ((digit >> bit) & 1u) ? votes : ~votes;
    }
    const uint32_t rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) {
      warp_count[warp][digit] = static_cast<uint16_t>(__popc(peers));
    }
    __syncthreads();
    {
      // thread d: exclusive prefix of digit d's counts over the warps (warp order = item order)
      const int d = threadIdx.x;
      uint32_t sum = 0;
#pragma unroll
      for (int w = 0; w < kSortThreads / 32; ++w) {
        const uint32_t count = warp_count[w][d];
        warp_count[w][d] = static_cast<uint16_t>(sum);
        sum += count;
      }
      round_base[d] = digit_base[d];
      digit_base[d] += sum;
    }
    __syncthreads();
    if (live) {
      const int64_t target = static_cast<int64_t>(round_base[digit]) + warp_count[warp][digit] + rank_in_warp;
      keys_out[target] = key;
      weights_out[target] = weight;
    }
    __syncthreads();
  }
}

// ---- runs of equal keys ----
__global__ void __launch_bounds__(256) run_heads_kernel(const uint64_t* keys, int64_t n, uint32_t* head) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint64_t key = keys[i];
    head[i] = (key != kInvalidKey && (i == 0 || keys[i - 1] != key)) ? 1u : 0u;
  }
}

__global__ void __launch_bounds__(256) run_reduce_kernel(const uint64_t* keys, const float* weights,
                                                         const uint32_t* head, const uint32_t* slot, int64_t n,
                                                         int64_t vertices, int64_t capacity, int32_t* edge_src,
                                                         int32_t* edge_dst, float* edge_weight, int64_t* edge_count) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint64_t key = keys[i];
    if (i == n - 1) {
      *edge_count = static_cast<int64_t>(slot[i]) + head[i];  // runs of valid keys
    }
    if (!head[i]) continue;
    float sum = weights[i];
    for (int64_t j = i + 1; j < n && keys[j] == key; ++j) {
      sum = __fadd_rn(sum, weights[j]);
    }
    const int64_t out = slot[i];
    if (out < capacity) {
      edge_src[out] = static_cast<int32_t>(key / static_cast<uint64_t>(vertices));
      edge_dst[out] = static_cast<int32_t>(key % static_cast<uint64_t>(vertices));
      edge_weight[out] = sum;
    }
  }
}

int64_t align256(int64_t bytes) { return (bytes + 255) / 256 * 256; }

struct Scratch {
  uint64_t* keys[2];
  float* weights[2];
  uint32_t* table;       // radix digit counts [256][tiles]; also run heads / slots [raw]
  uint32_t* table_scan;
  uint32_t* tile_total;
  int64_t bytes;
};

Scratch carve(void* base, int64_t raw) {
  Scratch s = {};
  const int64_t tiles = (raw + kSortTile - 1) / kSortTile;
  const int64_t table_items = raw > 256 * tiles ? raw : 256 * tiles;
  int64_t offset = 0;
  auto take = [&](int64_t bytes) {
    uint8_t* p = base ? static_cast<uint8_t*>(base) + offset : nullptr;
    offset += align256(bytes);
    return p;
  };
  s.keys[0] = reinterpret_cast<uint64_t*>(take(raw * 8));
  s.keys[1] = reinterpret_cast<uint64_t*>(take(raw * 8));
  s.weights[0] = reinterpret_cast<float*>(take(raw * 4));
  s.weights[1] = reinterpret_cast<float*>(take(raw * 4));
  s.table = reinterpret_cast<uint32_t*>(take(table_items * 4));
  s.table_scan = reinterpret_cast<uint32_t*>(take(table_items * 4));
  s.tile_total = reinterpret_cast<uint32_t*>(take(((table_items + kScanTile - 1) / kScanTile + 1) * 4));
  s.bytes = offset;
  return s;
}

}  // namespace
}  // namespace ckv

extern "C" {

int64_t ckv_adjacency_raw_edges(int64_t graphs, int64_t rows, int32_t kappa, double lam) {
  if (graphs <= 0 || rows <= 0 || kappa <= 0) return 0;
  const int64_t per_row = kappa + (lam < 1.0 ? static_cast<int64_t>(kappa) * (kappa + 1) / 2 : 0);
  return graphs * rows * per_row;
}

int64_t ckv_adjacency_scratch_bytes(int64_t graphs, int64_t rows, int32_t kappa, double lam) {
  const int64_t raw = ckv_adjacency_raw_edges(graphs, rows, kappa, lam);
  return raw > 0 ? ckv::carve(nullptr, raw).bytes : 0;
}

int ckv_build_adjacency(const int32_t* topk_indices, const float* topk_scores, const int64_t* query_positions,
                        int32_t graphs, int64_t rows, int32_t kappa, int32_t seq_len, double lam,
                        int32_t* edge_src, int32_t* edge_dst, float* edge_weight, int64_t edge_capacity,
                        int64_t* edge_count, void* scratch, int64_t scratch_bytes, void* cuda_stream) {
  if (!topk_indices || !topk_scores || !query_positions || !edge_src || !edge_dst || !edge_weight ||
      !edge_count || !scratch) {
    return CKV_ERR_NULL;
  }
  if (graphs <= 0 || rows <= 0 || kappa <= 0 || kappa > 64 || seq_len <= 0 || edge_capacity <= 0 ||
      !(lam >= 0.0 && lam <= 1.0)) {
    return CKV_ERR_SHAPE;
  }
  const int64_t vertices = static_cast<int64_t>(graphs) * seq_len;
  if (vertices >= (1ll << 31)) return CKV_ERR_CAPACITY;  // vertex ids are int32 in the output
  const int64_t raw = ckv_adjacency_raw_edges(graphs, rows, kappa, lam);
  if (raw >= (1ll << 32)) return CKV_ERR_CAPACITY;  // positions inside the sort are 32-bit
  const ckv::Scratch s = ckv::carve(scratch, raw);
  if (scratch_bytes < s.bytes) return CKV_ERR_CAPACITY;
  if (reinterpret_cast<uintptr_t>(scratch) % 256) return CKV_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const int64_t direct = static_cast<int64_t>(graphs) * rows * kappa;
  const unsigned wide = static_cast<unsigned>((raw + 255) / 256 > 148 * 16 ? 148 * 16 : (raw + 255) / 256);
  if (cudaMemsetAsync(edge_count, 0, sizeof(int64_t), stream) != cudaSuccess) return CKV_ERR_LAUNCH;
  ckv::edge_keys_kernel<<<wide, 256, 0, stream>>>(topk_indices, topk_scores, query_positions, rows, kappa, seq_len,
                                                  vertices, static_cast<float>(lam / 2.0), static_cast<float>(1.0 - lam), direct, raw,
                                                  s.keys[0],
                                                  s.weights[0]);
  if (cudaGetLastError() != cudaSuccess) return CKV_ERR_LAUNCH;
  // keys are below vertices^2 (the invalid key has every bit set and sorts last in every pass)
  int vertex_bits = 0;
  while ((1ll << vertex_bits) < vertices) ++vertex_bits;
  const int bits = 2 * vertex_bits;
  const int64_t tiles = (raw + ckv::kSortTile - 1) / ckv::kSortTile;
  int from = 0;
  for (int shift = 0; shift < bits; shift += 8) {
    ckv::radix_count_kernel<<<static_cast<unsigned>(tiles), ckv::kSortThreads, 0, stream>>>(
        s.keys[from], raw, shift, tiles, s.table);
    if (ckv::exclusive_scan(s.table, s.table_scan, 256 * tiles, s.tile_total, stream) != cudaSuccess) {
      return CKV_ERR_LAUNCH;
    }
    ckv::radix_scatter_kernel<<<static_cast<unsigned>(tiles), ckv::kSortThreads, 0, stream>>>(
        s.keys[from], s.weights[from], raw, shift, tiles, s.table_scan, s.keys[1 - from], s.weights[1 - from]);
    if (cudaGetLastError() != cudaSuccess) return CKV_ERR_LAUNCH;
    from = 1 - from;
  }
  ckv::run_heads_kernel<<<wide, 256, 0, stream>>>(s.keys[from], raw, s.table);
  if (ckv::exclusive_scan(s.table, s.table_scan, raw, s.tile_total, stream) != cudaSuccess) return CKV_ERR_LAUNCH;
  ckv::run_reduce_kernel<<<wide, 256, 0, stream>>>(s.keys[from], s.weights[from], s.table, s.table_scan, raw,
                                                   vertices, edge_capacity, edge_src, edge_dst, edge_weight,
                                                   edge_count);
  return cudaGetLastError() == cudaSuccess ? CKV_OK : CKV_ERR_LAUNCH;
}

}  // extern "C"
