/*
 * ckv_b200.h - C ABI of the B200 (sm_100a) CommunityKV sparse-decode hot path.
 *
 * Every entry point takes plain pointers and sizes (no framework types), never
 * allocates, never synchronises, and enqueues its kernels on the CUDA stream it
 * is given.  The return value is 0 on success or a negative ckv_status code.
 * Device-side trouble that cannot be known on the host (a bounded wait that ran
 * out) is reported by OR-ing bits into the optional `status` word.
 *
 * All per-sequence tensors carry a leading `batch` dimension and are stored
 * batch-major and contiguous: element [b, ...] lives at b * (product of the
 * remaining extents).  `batch` is the number of independent sequence slots in
 * one launch; with batch == 1 the layouts are exactly the reference's per-layer
 * tensors.  The K/V cache alone uses explicit strides because it belongs to the
 * host framework's cache object.
 *
 * Reference interfaces these entry points stand in for (paths inside the
 * reference project):
 *   ckv_score_centroids      score_centroids(), the Triton launcher
 *                            community_kv/attention/kernels/centroid_selection.py:330-445
 *   ckv_select_descriptors   _selection_native.select_weighted_descriptors
 *                            community_kv/attention/kernels/_csrc/bindings.cpp:3-22
 *                            (descriptor_selection.cu:852-1189)
 *   ckv_segmented_attention  triton_segmented_attention()
 *                            community_kv/attention/kernels/segmented_attention.py:1016-1273
 *   ckv_decode_layer         decode_layer()  community_kv/attention/decode.py:67-111
 *   ckv_prefill_topk         torch.ops.flash_attn_3.fwd(..., exclude_sink_tokens=n)
 *                            community_kv/attention/flash_attention.py:23-51
 *                            (third_party/flash_attention/community-kv.patch)
 *   ckv_append_kv            the cache layer's index_copy_ of the decoded token
 *                            community_kv/attention/cache.py:29-36
 *   ckv_assemble_member_csr, ckv_assemble_centroids, ckv_assemble_modularity
 *                            build_member_csr, compute_centroids, init_modularity_state
 *                            community_kv/graph/partition.py:382-535
 *   ckv_build_adjacency      build_adjacency  community_kv/graph/partition.py:168-249
 * Without a counterpart in the (single-GPU) reference: ckv_online_update, ckv_merge_partials,
 * ckv_wait_peers and the peer_* fields (KV heads or sequence rows sharded over GPUs),
 * ckv_segmented_attention_static, ckv_decode_layer_kernels.
 */
#ifndef CKV_B200_H_
#define CKV_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CKV_HEAD_DIM 128
#define CKV_TILE 64
#define CKV_KAPPA 8
#define CKV_PARTIAL_STRIDE 132 /* floats per (split, head): acc[128], max, sum, 2 pad */

typedef enum ckv_status {
  CKV_OK = 0,
  CKV_ERR_NULL = -1,      /* a required pointer is null */
  CKV_ERR_SHAPE = -2,     /* a size or stride is out of range */
  CKV_ERR_ALIGN = -3,     /* K/V rows are not 16-byte aligned */
  CKV_ERR_LAUNCH = -4,    /* the CUDA runtime rejected a launch */
  CKV_ERR_DEVICE = -5,    /* the device index cannot be selected */
  CKV_ERR_UNSUPPORTED = -6,
  CKV_ERR_CAPACITY = -7   /* a size exceeds a fixed built-in maximum */
} ckv_status;

/* bits OR-ed into *status by the kernels */
#define CKV_DEV_WAIT_TIMEOUT 1u /* a bounded wait gave up */
#define CKV_DEV_STASH_OVERFLOW 2u /* more active communities beyond score_cover than a CTA can stage */

#define CKV_MAX_PEERS 7

/* flags */
#define CKV_FLAG_SKIP_UPDATE 1    /* attention only: leave the graph state untouched */
#define CKV_FLAG_UPDATE_ONLY 4    /* ckv_online_update: take lse / topk_scores / topk_positions
                                     as inputs and only apply the online assignment */
#define CKV_FLAG_ATTENTION_ONLY 2 /* ckv_segmented_attention: launch only the gather+attention
                                     kernel on the positions already in the workspace (no
                                     position resolution, no merge); for kernel timing */
#define CKV_FLAG_UNFUSED 8        /* ckv_decode_layer: run the four stand-alone kernels even when
                                     the single cluster launch is available (same results) */
#define CKV_FLAG_TENSOR_SCORES 32  /* centroid scoring on the tensor cores (group size <= 8): the 128-long
                                     dot products are accumulated by mma.m16n8k16 in fp32 instead of in
                                     the fixed CUDA-core order; a score may differ in its last fp16 bit */
#define CKV_FLAG_FP32_CENTROIDS 64  /* `centroids` is fp32 [batch, R, cap, 128] instead of e4m3: scores are
                                      the fixed-order sum of products rounded one by one, the running
                                      mean is stored unquantised.  ckv_decode_layer then runs the four
                                      stand-alone kernels.  No reference counterpart (its table is e4m3) */
#define CKV_FLAG_REFERENCE_DIVISION 16 /* running centroid mean (old*n + key)/(n+1): divide with the
                                     GPU's approximate full-range division (div.full.f32, at most 2 ulp
                                     off), which is what the reference's Triton kernel compiles `/` to
                                     (segmented_attention.py:708-713), instead of IEEE division, which is
                                     what the reference's CPU test helper computes (tests/community_kv/
                                     graph/test_state.py:32-132).  The two differ when the exact quotient
                                     is a rounding tie of the e4m3 result. */

typedef struct ckv_layer_args {
  /* ---- geometry ---- */
  int32_t device;             /* CUDA device ordinal that owns every pointer */
  int32_t batch;              /* independent sequence slots in this launch */
  int32_t retrieval_heads;    /* R */
  int32_t graphs;             /* number of graphs (R, or 1 when one graph is shared) */
  int32_t group_size;         /* query heads per retrieval head, 1..16 */
  int32_t community_capacity; /* centroid rows per retrieval head */
  int32_t token_budget;       /* T, multiple of 64 */
  int32_t num_sink;
  int32_t sequence_capacity;  /* rows per head in the K/V cache */
  int32_t token_capacity;     /* width of token_communities */
  int32_t member_capacity;    /* width of member_positions */
  int32_t chunks_per_graph;
  int32_t delta_position_capacity;
  int32_t descriptor_capacity; /* width of communities / cumulative_ends, >= T - num_sink - 1 */
  int32_t max_communities;    /* 0: fill the token budget (reference behaviour); k>0: at most k communities */
  int32_t splits;             /* attention CTAs per retrieval head, 1..32 */
  int32_t flags;
  float softmax_scale;
  float lam;
  /* ---- K/V cache, bf16, element strides; a row is 128 contiguous elements ---- */
  int64_t key_batch_stride, key_head_stride, key_row_stride;
  int64_t value_batch_stride, value_head_stride, value_row_stride;
  const void* key;
  const void* value;
  /* ---- per-call inputs ---- */
  const void* query;                 /* bf16 [batch, R*G, 128] */
  const int32_t* sink_positions;     /* [num_sink], shared by the batch */
  const int32_t* retrieval_to_graph; /* [R], shared by the batch */
  const int32_t* retrieval_to_kv;    /* [R], shared by the batch */
  const int32_t* score_cover;        /* [batch, R] or null: score only rows below ceil64(min(capacity, cover)) */
  /* ---- immutable prefill CSR ---- */
  const int32_t* member_offsets;   /* [batch, graphs, capacity+1] */
  const int32_t* member_positions; /* [batch, graphs, member_capacity] */
  /* ---- mutable graph state ---- */
  void* centroids;             /* e4m3 [batch, R, capacity, 128]; fp32 with CKV_FLAG_FP32_CENTROIDS */
  int32_t* community_sizes;    /* [batch, R, capacity] */
  int32_t* community_counts;   /* [batch, R] */
  float* community_weight;     /* [batch, graphs, capacity] */
  float* total_weight;         /* [batch, graphs] */
  int32_t* token_communities;  /* [batch, graphs, token_capacity] */
  int32_t* current_position;   /* [batch, graphs] */
  int32_t* delta_positions;    /* [batch, graphs, delta_position_capacity] */
  int32_t* chunk_start;        /* [batch, graphs, chunks_per_graph] (and the four below) */
  int32_t* chunk_capacity;
  int32_t* chunk_size;
  int32_t* chunk_next;
  int32_t* chunk_previous;
  int32_t* community_head;     /* [batch, graphs, capacity] (and the two below) */
  int32_t* community_tail;
  int32_t* delta_sizes;
  int32_t* next_free_chunk;    /* [batch, graphs] */
  int32_t* next_free_position; /* [batch, graphs] */
  /* ---- selection workspace ---- */
  void* scores;                /* fp16 [batch, R, capacity] */
  int32_t* communities;        /* [batch, R, descriptor_capacity] */
  int32_t* cumulative_ends;    /* [batch, R, descriptor_capacity] */
  int32_t* descriptor_counts;  /* [batch, R] */
  int32_t* tile_descriptors;   /* [batch, R, T/64] */
  int32_t* threshold_state;    /* [batch, R, 4]; slot 0 receives the threshold key */
  /* ---- attention workspace ---- */
  int32_t* positions;          /* [batch, R, T] resolved cache rows, -1 = masked */
  float* partials;             /* [batch, R, splits, G, 132] */
  uint64_t* partial_topk;      /* [batch, R, splits, 8] */
  void* output;                /* bf16 [batch, R*G, 128] */
  float* lse;                  /* [batch, R*G] */
  float* topk_scores;          /* [batch, R, 8] */
  int32_t* topk_positions;     /* [batch, R, 8] */
  int32_t* assigned;           /* [batch, graphs] */
  int32_t* overflow;           /* [batch, graphs] */
  uint32_t* status;            /* one device word, may be null */
  /* ---- sequence sharding (all zero / null when the whole cache is local) ---- */
  int32_t kv_row_begin;        /* first global cache row held in `key` / `value` */
  int32_t kv_row_count;        /* rows held locally; 0 = unsharded.  Selected rows outside
                                  [begin, begin+count) are skipped by the attention kernel */
  float* merged;               /* optional [batch, R, G, 132]: the merged, un-normalised
                                  (acc[128], max, sum) of every head, for a cross-GPU combine */
  const void* current_key;     /* optional bf16 [batch, R, 128]: key of the token being decoded
                                  (row of each retrieval head's KV head), used for the centroid
                                  update instead of a cache read */
  /* ---- head-output exchange between GPUs (peer_count 0: none) ----
   * With KV heads sharded over GPUs every GPU needs all heads' outputs.  Instead of a
   * collective after the layer, the merging CTA stores its output rows straight into
   * each peer's buffer over NVLink (peer_output[p] points at THIS GPU's slot of peer
   * p's gathered tensor, same [batch, R, G, 128] layout as `output`) and then adds 1
   * to peer_flag[p] with system-scope release.  The peer consumes the rows after
   * ckv_wait_peers has seen (its peers' units) increments. */
  int32_t peer_count;
  int32_t peer_wait_expected;  /* with peer_wait_flag: increments this GPU expects per call */
  void* peer_output[CKV_MAX_PEERS];
  uint32_t* peer_flag[CKV_MAX_PEERS];
  uint32_t* peer_done;         /* optional: a counter in THIS GPU's memory (zero before the first
                                  call).  When set, units count themselves here and only the last
                                  unit of the call signals the peers: one increment per peer and
                                  call instead of one per unit (remote atomics on one word are
                                  slow), so the consumer expects (number of peers) per call */
  uint32_t* peer_wait_flag;    /* optional: THIS GPU's counter.  The CTA that merges unit 0 then
                                  polls it (bounded, system-scope acquire) after its own work
                                  until the peers' rows of this call have arrived and subtracts
                                  peer_wait_expected, so that the launch completes only when the
                                  gathered tensor is complete: no separate wait is needed */
  uint64_t* phase_times;       /* optional diagnostic [batch*R, 8, 16]: nanosecond timestamps
                                  (%globaltimer) that thread 0 of every CTA of the single-launch
                                  path writes at its phase boundaries: 0 start, 1 scored,
                                  2..4 after the selection's three cluster exchanges, 5 descriptors
                                  known, 6 cache rows resolved, 7 attended, 8 partials of the whole
                                  cluster visible (rank 0), 9 merged and updated (rank 0) */
  /* ---- partial rows in a foreign layout (all zero / null: the dense local layout) ----
   * ckv_merge_partials can merge rows that were not produced by this GPU's attention
   * kernel, e.g. one merged row set per GPU after an all-gather of sequence shards. */
  int64_t partial_unit_stride;  /* floats between units in `partials`; 0: splits * G * 132 */
  int64_t partial_split_stride; /* floats between the splits of a unit; 0: G * 132 */
  int64_t topk_unit_stride;     /* uint64 elements between units in `partial_topk`; 0: splits * 8 */
  int64_t topk_split_stride;    /* uint64 elements between the splits of a unit; 0: 8 */
  uint64_t* merged_topk;        /* optional [batch, R, 8]: with `merged`, the packed eight best
                                   neighbour candidates of every unit (ordered fp32 score << 32 |
                                   0xffffffff - position; 0: none), for a cross-GPU combine */
  const int32_t* forced_community; /* optional [batch, graphs]: the community the new token joins.
                                  When set and 0 <= value < the leader head's community count,
                                  the online assignment joins it instead of applying the dQ rule
                                  of A5 (weights, sizes, centroid, labels and delta chunks are
                                  updated exactly as for a join the rule had chosen); a negative
                                  value leaves that graph to the rule.  Carries the
                                  nearest-centroid assignment variant: the caller scores the new
                                  token's key against the centroids (ckv_score_centroids) and
                                  passes the arg-max.  No reference counterpart. */
} ckv_layer_args;

/* Arguments of the prefill score-graph kernel.  Q, K, V, O are bf16 with a
 * contiguous last dimension of 128 and element strides for batch, sequence row
 * and head; the reference passes [B, S, H, 128] tensors. */
typedef struct ckv_prefill_args {
  int32_t device;
  int32_t batch;
  int32_t seq_len;
  int32_t query_heads;
  int32_t kv_heads;        /* query_heads / kv_heads must be 1, 2, 4 or 8 */
  int32_t num_sink;        /* keys below this index are never reported as neighbours */
  int32_t mode;            /* 0 attention only; 1 reference top-8 per query head;
                              2 exact top-`edges_per_row` per KV head */
  int32_t edges_per_row;   /* mode 2: 1..16 */
  float softmax_scale;
  float exact_slack;       /* mode 2: margin (in scaled-score units) for the completeness check */
  int64_t q_batch_stride, q_row_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  const void* query;
  const void* key;
  const void* value;
  void* output;            /* bf16, strides above */
  float* lse;              /* [batch, query_heads, seq_len] natural-log sum-exp */
  float* topk_val;         /* mode 1: [batch, query_heads, seq_len - (num_sink+7), 8] */
  int32_t* topk_idx;       /* mode 1: same shape */
  uint64_t* candidates;    /* mode 2 scratch: [batch, kv_heads, seq_len, group, 17] */
  int32_t* edge_idx;       /* mode 2: [batch, kv_heads, seq_len - (num_sink+m-1), m] */
  float* edge_score;       /* mode 2: same shape, scaled scores */
  int32_t* edge_flags;     /* mode 2, optional: [batch, kv_heads, rows]; 1 = row was re-scanned */
  uint32_t* status;        /* one device word, may be null */
  int32_t* rescan_list;    /* mode 2, optional scratch: [1 + batch*kv_heads*rows] int32, element 0
                              zero on entry.  Rows whose short list cannot be proven complete are
                              queued here and re-ranked by a full scan; without it every row's
                              flag is polled instead (slower) */
} ckv_prefill_args;

/* Library version: major*10000 + minor*100 + patch. */
int ckv_version(void);
const char* ckv_status_string(int status);

/* A1.  scores[b,r,c] = fp16(max_g q . centroid); -inf if c >= count or size <= 0. */
int ckv_score_centroids(const ckv_layer_args* args, void* cuda_stream);

/* A2.  Exact weighted threshold selection; fills communities, cumulative_ends,
 * descriptor_counts, tile_descriptors and the resolved `positions`. */
int ckv_select_descriptors(const ckv_layer_args* args, void* cuda_stream);

/* A3+A4+A5.  Resolves positions from the packed descriptors already in the
 * workspace, gathers K/V rows, runs split attention, merges, and (unless
 * CKV_FLAG_SKIP_UPDATE) performs the online assignment and state update. */
int ckv_segmented_attention(const ckv_layer_args* args, void* cuda_stream);

/* A1..A5 back to back: the whole per-layer decode transition.  With one graph per
 * retrieval head, at most eight splits and descriptors that fit the selection's
 * shared-memory list, this is ONE launch: a thread-block cluster per (sequence,
 * retrieval head) scores, selects, attends, merges and updates, synchronising
 * through cluster barriers.  Otherwise (or with CKV_FLAG_UNFUSED) the four
 * stand-alone kernels run back to back.  Results are identical either way. */
int ckv_decode_layer(const ckv_layer_args* args, void* cuda_stream);

/* Writes the decoded token's K and V rows into the caches: cache[u, row, :] = new[u, :]
 * for u < units, where the caches are bf16 [units, rows, 128] with `unit_stride`
 * elements between units and the new rows are contiguous bf16 [units, 128].  The row
 * is `row_index[u * row_index_stride]` when row_index is given (int32, device;
 * stride 0: one device-side cursor shared by all units, stride 1: one row per unit;
 * a negative row skips the unit) and `row` otherwise.  One small launch instead of the
 * arange + two index_copy_ calls of the reference's cache layer
 * (community_kv/attention/cache.py:39-47). */
int ckv_append_kv(void* key_cache, void* value_cache, const void* new_key, const void* new_value,
                  int64_t units, int64_t unit_stride, const int32_t* row_index,
                  int64_t row_index_stride, int64_t row, void* cuda_stream);

/* Waits (on the stream, in a one-thread kernel with a bounded number of polls)
 * until *flag >= expected, then subtracts `expected` from it.  `flag` is this GPU's
 * counter that its peers' ckv_decode_layer calls increment once per unit after
 * storing that unit's head outputs here.  On a timeout the kernel ORs
 * CKV_DEV_WAIT_TIMEOUT into *status (which may be null) and returns.  No reference
 * counterpart: the reference runs on one GPU. */
int ckv_wait_peers(uint32_t* flag, uint32_t expected, uint32_t* status, void* cuda_stream);

/* Nearest-centroid assignment variant (no reference counterpart: the reference assigns by
 * modularity gain, A5).  For every graph writes forced_community[batch, graphs]: the live
 * community (index < community_counts, size > 0) of the graph's leader head whose centroid has
 * the largest inner product with the key of the token being decoded - the fp16 value
 * ckv_score_centroids gives a query group made of that key, fixed summation order; the first
 * maximum wins; -1 when the head has no live community.  The key is current_key[batch, R, 128]
 * when set, else the cache row at current_position.  Pass the array as `forced_community` to
 * ckv_decode_layer / ckv_online_update. */
int ckv_nearest_centroid(const ckv_layer_args* args, int32_t* forced_community, void* cuda_stream);

/* How many kernels ckv_decode_layer launches for these arguments (1, 4 or 5);
 * no reference counterpart, used for launch accounting. */
int ckv_decode_layer_kernels(const ckv_layer_args* args);

/* A5 alone.  Applies the online assignment and centroid update from the
 * `lse`, `topk_scores` and `topk_positions` already in the workspace (for
 * sequence-sharded decoding, where those are combined across GPUs first). */
int ckv_online_update(const ckv_layer_args* args, void* cuda_stream);

/* A4+A5 alone.  Merges the `splits` partial (acc, max, sum) rows per head and the
 * `splits` candidate lists per unit that are already in `partials` / `partial_topk`
 * (addressed with the partial_*_stride / topk_*_stride fields), writes output, lse and the
 * top-8 neighbours, and (unless CKV_FLAG_SKIP_UPDATE) applies the online update.  With
 * sequence-sharded decoding every GPU all-gathers the GPUs' `merged` / `merged_topk`
 * records and calls this with splits = number of GPUs; no reference counterpart. */
int ckv_merge_partials(const ckv_layer_args* args, void* cuda_stream);

/* ---- decode-state assembly from community labels (the step between a finished partition
 * and the first decode step; the reference runs it as torch sort / scatter operations) ---- */

/* Member lists.  labels int32 [graphs, length] (community id of every position; sinks are the
 * first num_sink positions and are left out).  Writes offsets int32 [graphs, communities + 1]
 * and member_positions int32 [graphs, member_capacity >= length - num_sink]: the positions of
 * community c are member_positions[g, offsets[g, c] .. offsets[g, c + 1]), newest first.
 * `counts` is int32 scratch [graphs, communities].  Replaces build_member_csr
 * (community_kv/graph/partition.py:457-492). */
int ckv_assemble_member_csr(const int32_t* labels, int32_t graphs, int32_t length, int32_t num_sink,
                            int32_t communities, int32_t* counts, int32_t* offsets,
                            int32_t* member_positions, int32_t member_capacity, void* cuda_stream);

/* Centroids.  For every retrieval head h and community c < capacity: sizes[h, c] = members of c
 * in graph retrieval_to_graph[h], centroids[h, c, :] = e4m3(clamp(mean of the members' key rows
 * of KV head retrieval_to_kv[h])) (zero rows beyond `live`; the sum runs over the members oldest
 * first in fp32).  keys bf16 [KV heads, rows, 128] with element strides.  Replaces
 * compute_centroids (community_kv/graph/partition.py:382-455). */
int ckv_assemble_centroids(const int32_t* offsets, const int32_t* member_positions, int32_t communities,
                           int32_t member_capacity, const void* keys, int64_t key_head_stride,
                           int64_t key_row_stride, const int32_t* retrieval_to_graph,
                           const int32_t* retrieval_to_kv, int32_t heads, int32_t live, int32_t capacity,
                           void* centroids, int32_t* sizes, void* cuda_stream);

/* Modularity bookkeeping.  Edge e joins flat vertices edge_src[e], edge_dst[e] (graph * length +
 * position, int64) with weight edge_weight[e]: community_weight[g, label] += w for both end
 * points, total_weight[g] += 2 w (both outputs are cleared first).  Replaces
 * init_modularity_state (community_kv/graph/partition.py:495-535). */
int ckv_assemble_modularity(const int32_t* labels, int32_t graphs, int32_t length, const int64_t* edge_src,
                            const int64_t* edge_dst, const float* edge_weight, int64_t edges,
                            int32_t capacity, float* community_weight, float* total_weight,
                            void* cuda_stream);

/* Edge list -> coalesced adjacency: what the host partitioner consumes.  topk_indices int32 and
 * topk_scores fp32 are [graphs, rows, kappa] (neighbour position per row, -1 or >= seq_len:
 * none), query_positions int64 [graphs, rows] the position a row belongs to.  A row contributes
 * kappa direct edges (weight score * lam / 2) and, for lam < 1, kappa (kappa + 1) / 2
 * co-attention edges between its neighbours (weight score_a * score_b * (1 - lam)); edges are
 * stored as (min, max) over vertices graph * seq_len + position, duplicates merged by adding
 * their weights in enumeration order (the scale factors are lam / 2 and 1 - lam rounded to fp32
 * once, as a Python float times an fp32 tensor gives), output sorted by (min, max): edge_src / edge_dst int32,
 * edge_weight fp32, *edge_count the number of distinct edges (device int64; edges beyond
 * edge_capacity are counted but not stored).  scratch: ckv_adjacency_scratch_bytes() bytes,
 * 256-byte aligned.  Replaces build_adjacency (community_kv/graph/partition.py:168-249). */
int64_t ckv_adjacency_raw_edges(int64_t graphs, int64_t rows, int32_t kappa, double lam);
int64_t ckv_adjacency_scratch_bytes(int64_t graphs, int64_t rows, int32_t kappa, double lam);
int ckv_build_adjacency(const int32_t* topk_indices, const float* topk_scores, const int64_t* query_positions,
                        int32_t graphs, int64_t rows, int32_t kappa, int32_t seq_len, double lam,
                        int32_t* edge_src, int32_t* edge_dst, float* edge_weight, int64_t edge_capacity,
                        int64_t* edge_count, void* scratch, int64_t scratch_bytes, void* cuda_stream);

/* P1.  Causal attention (output + lse) that also emits each row's strongest
 * Q.K neighbours: the reference's top-8 rule (mode 1) or exact top-m per KV head
 * (mode 2). */
int ckv_prefill_topk(const ckv_prefill_args* args, void* cuda_stream);

/* Same operation and results as ckv_segmented_attention for callers that cannot
 * allocate device memory (no counterpart in the reference: its Triton launcher
 * always works on caller-allocated workspaces).  `positions`, `partials` and
 * `partial_topk` of `args` are ignored; that scratch lives in a fixed array
 * inside the library instead, CKV_STATIC_SCRATCH_BYTES (about 3.3 MB) on every
 * GPU that loads the library, until the process exits.  Limits, checked up front
 * (CKV_ERR_CAPACITY): batch * retrieval_heads <= CKV_STATIC_MAX_UNITS,
 * token_budget <= CKV_STATIC_MAX_BUDGET, splits <= CKV_STATIC_MAX_SPLITS,
 * group_size <= CKV_STATIC_MAX_GROUP.  Inputs, outputs and graph state are still
 * the caller's.  The first call on a device looks up the array's device address;
 * make that call before any stream capture begins.  All calls share the one
 * array and it keeps the previous call's contents (every element that is read
 * is rewritten first, nothing needs clearing): two calls whose kernels may
 * overlap on the GPU - different streams, or different host threads - race. */
#define CKV_STATIC_MAX_UNITS 64
#define CKV_STATIC_MAX_BUDGET 4096
#define CKV_STATIC_MAX_SPLITS 8
#define CKV_STATIC_MAX_GROUP 8
#define CKV_STATIC_SCRATCH_BYTES                                                        \
  (4 * CKV_STATIC_MAX_UNITS * CKV_STATIC_MAX_BUDGET +                                   \
   4 * CKV_STATIC_MAX_UNITS * CKV_STATIC_MAX_SPLITS * CKV_STATIC_MAX_GROUP *            \
       CKV_PARTIAL_STRIDE +                                                             \
   8 * CKV_STATIC_MAX_UNITS * CKV_STATIC_MAX_SPLITS * CKV_KAPPA)
int ckv_segmented_attention_static(const ckv_layer_args* args, void* cuda_stream);

/* Bytes of dynamic shared memory the attention kernel asks for (for diagnostics). */
int ckv_attention_smem_bytes(int group_size);

#ifdef __cplusplus
}
#endif
#endif /* CKV_B200_H_ */
