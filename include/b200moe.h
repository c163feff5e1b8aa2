/* b200moe — C ABI of the B200 (sm_100a) NVFP4 mixture-of-experts library.
 *
 * Drop-in boundary for the `nvfp4_fused_moe` operator of bcacdwk/KernelSchema
 * (kernel_wiki/aka-cuda-operators-20261030/operators/moe/nvfp4_fused_moe, "NV/" below) and for the dense
 * NVFP4 GEMM next to it (operators/gemm/dense/bf16_nvfp4_gemm, "DG/" below). Plain pointers and sizes only:
 * all pointers are CUDA device pointers unless stated otherwise, `stream` is a cudaStream_t passed as void*.
 * Every function returns 0 on success or a non-zero code (CUDA error numbers < 700; 7xx = argument, shape or
 * tensor-map refusals raised before any launch); b200moe_last_error() gives the text. Nothing throws, nothing
 * traps on the device; bounded device waits report through b200moe_status().
 *
 * Number formats (NV/problem/input.py:53-71, NV/problem/reference.py:28-50): payload = two E2M1 codes per
 * byte, even element in the low nibble; one E4M3 scale byte per 16 elements along K; weights in the published
 * prepared layout (NV/problem/input.py:82-99: rows 32-shuffled, FC1 rows up/gate interleaved, scales in
 * 128-row x 4-column tiles).
 */
#ifndef B200MOE_H
#define B200MOE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 3

/* Scale-factor layouts. */
#define B200MOE_SF_ROW_MAJOR 0 /* [rows, cols/16]                                   */
#define B200MOE_SF_TILED 1     /* [ceil(rows/128), cols/64, 32, 16] (128x4 tiles)   */

typedef struct b200moe_layer* b200moe_handle;

/* Geometry of one MoE layer instance; fixes the workspace the library owns for it. */
typedef struct {
  int32_t struct_size;        /* sizeof(b200moe_config) */
  int32_t hidden;             /* H, multiple of 256 */
  int32_t intermediate;       /* I, multiple of 256 */
  int32_t num_experts;        /* routed experts held by this instance (local experts) */
  int32_t top_k;              /* routed slots per token */
  int32_t num_shared_experts; /* S experts every token also visits with weight 1; stored after the routed ones */
  int32_t max_tokens;         /* largest T a run may pass */
  int32_t tile_n;             /* GEMM tile: 0 = default; 128 or 256 = one CTA per 128 x tile_n tile; 512 = CTA pair per 256 x 256 tile */
  int32_t sm_margin;          /* SMs the persistent GEMM grids leave free (0 = use all): room for a collective that runs beside them */
  int32_t graph_cache;        /* 1 = b200moe_run replays a CUDA graph when it is called again with an identical argument block
                                 on the same stream (captured on the second such call, as the reference's moe_run does,
                                 NV/candidate/nvfp4_moe.cu:9513-9517); 0 = always launch the kernel chain */
  int32_t tma_gather;         /* 0 (default) = the permute pass copies the payload rows of the routed tokens into the workspace and FC1
                                 reads them as plain 128-row boxes; 1 = FC1 fetches its activation rows from hidden_states itself with
                                 TMA tile::gather4 (the reference's activation gather, NV/candidate/nvfp4_moe.cu:244-256) and the
                                 permute pass moves only the scale rows (ignored with tile_n = 512). Same results; measured slower
                                 whenever FC1 is not latency-bound: one gather4 box occupies the TMA unit ~64 cycles */
  int32_t reserved[5];
} b200moe_config;

/* One forward call. Field names follow the reference operator's forward() arguments
 * (NV/problem/reference.py:96; layouts NV/problem/input.py:101-112). */
typedef struct {
  int32_t struct_size;               /* sizeof(b200moe_args) */
  int32_t num_tokens;                /* T */
  const int32_t* topk_ids;           /* [T, top_k]; ids outside [offset, offset+num_experts) are skipped (-1 = none) */
  const float* topk_weights;         /* [T, top_k] */
  const void* hidden_states;         /* uint8 [T, H/2] */
  const void* hidden_states_scale;   /* E4M3 bytes, layout below */
  int32_t hidden_states_scale_layout;/* 2 = row-major [T, H/16] (the reference's value); 1 = 128x4 tiled */
  int32_t activation_type;           /* 3 = gate*sigmoid(alpha*gate)*(up+beta); 10 = SiTU (NV/problem/reference.py:86-89) */
  const void* gemm1_weights;         /* uint8 [E+S, 2I, H/2] prepared */
  const void* gemm1_weights_scale;   /* E4M3 [E+S, 2I, H/16] bytes holding 128x4 tiles */
  const void* gemm2_weights;         /* uint8 [E+S, H, I/2] prepared */
  const void* gemm2_weights_scale;   /* E4M3 [E+S, H, I/16] bytes holding 128x4 tiles */
  const float* gemm1_alpha;          /* [E+S] or NULL (=1) */
  const float* gemm1_beta;           /* [E+S] or NULL (=0) */
  const float* gemm1_clamp_limit;    /* [E+S] or NULL (no clamp) */
  const float* output1_scale_scalar;      /* [E+S] multiplier of the FC1 "up" accumulator, or NULL (=1) */
  const float* output1_scale_gate_scalar; /* [E+S] multiplier of the FC1 "gate" accumulator, or NULL (=1) */
  const float* output2_scale_scalar;      /* [E+S] multiplier of the FC2 accumulator, or NULL (=1) */
  int32_t local_expert_offset;       /* id of this instance's first routed expert */
  int32_t direct_rows;               /* 0 = weighted combine (default). 1 = every token has at most one route (top_k == 1,
                                        no shared experts): FC2 writes bf16(fc2) of the token's route straight into
                                        output[t] (weights ignored, tokens without a route are left untouched) and the
                                        combine pass is skipped; used by the expert-parallel wrapper on received rows */
  void* output;                      /* bf16 [T, H]; the only caller memory that is written */
  int64_t output_stride;             /* elements between output rows (H when contiguous) */
  int64_t hidden_states_stride;      /* bytes between payload rows; 0 = H/2 (contiguous). Multiple of 16 */
  int64_t hidden_states_scale_stride;/* bytes between row-major scale rows; 0 = H/16. Multiple of 4; layout 2 only */
  int64_t topk_stride;               /* elements between the rows of topk_ids / topk_weights; 0 = top_k */
} b200moe_args;

/* Device pointers into the library-owned workspace of a layer, for tests and for the expert-parallel
 * wrapper. Valid until b200moe_destroy. */
typedef struct {
  int32_t* counts;        /* [E+S] routes per expert */
  int32_t* seg_start;     /* [E+S+1] first permuted row of each expert (multiples of 128) */
  int32_t* tile_expert;   /* [tile_capacity] */
  int32_t* tile_row0;     /* [tile_capacity] */
  int32_t* tile_rows;     /* [tile_capacity] */
  int32_t* totals;        /* {m-tiles, permuted rows in use, valid routes, 256-row pair items} */
  int32_t* row_of;        /* [T, top_k+S] permuted row of a route or -1 */
  int32_t* tok_of_row;    /* [row_capacity] token of a permuted row; defined for the first tile_rows[r/128] rows of each 128-row tile */
  float* weight_of_row;   /* [row_capacity] */
  uint8_t* a_q;           /* [row_capacity, H/2] permuted activations */
  uint8_t* a_sf;          /* tiled scales of a_q */
  uint8_t* act_q;         /* [row_capacity, I/2] requantised intermediate */
  uint8_t* act_sf;        /* tiled scales of act_q */
  uint16_t* rout;         /* bf16 [row_capacity, H] per-route FC2 results */
  int64_t row_capacity;
  int64_t tile_capacity;
  int32_t* pair_expert;   /* [tile_capacity] 256-row work items of the CTA-pair GEMM: expert, */
  int32_t* pair_row0;     /*                 first permuted row,                               */
  int32_t* pair_rows;     /*                 valid rows (1..256)                               */
  int32_t* step_ids;      /* [max_tokens, top_k] experts selected by the last b200moe_step */
  float* step_weights;    /* [max_tokens, top_k] and their routing weights */
} b200moe_workspace_view;

int b200moe_abi_version(void);
/* Text of the calling thread's last failure ("" if none). Host memory owned by the library. */
const char* b200moe_last_error(void);

/* (2) bf16 -> NVFP4 quantiser. Replaces quantize() of NV/problem/input.py:53-71 (global_scale == 1) and of
 * DG/problem/input.py:40-64 (global_scale != 1); codes and scale bytes are bit-identical to them.
 * x: bf16 [rows, cols] with row_stride elements between rows; cols % 64 == 0; payload: uint8 [rows, cols/2];
 * scales: layout B200MOE_SF_ROW_MAJOR or B200MOE_SF_TILED (caller sizes it for rows rounded up to 128). */
int b200moe_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int64_t row_stride, float global_scale, void* payload,
                           void* scales, int32_t scale_layout, void* stream);

/* Row-major scale bytes [rows, cols/16] -> 128x4 tiles (the block_scales() step of NV/problem/input.py:82-87
 * for one matrix). dst holds ceil(rows/128)*128 * cols/16 bytes; padding rows become 0. */
int b200moe_scales_to_tiles(const void* scales_row_major, int64_t rows, int64_t cols, void* dst, void* stream);

/* (1) Router. logits fp32 [T, E]; optional bias fp32 [E] added before selection. Replaces the selection part
 * of routes() in NV/problem/input.py:35-36: ids = top-k by logit (descending, ties to the lower index),
 * weights = softmax over the selected logits. ids int32 [T, K], weights fp32 [T, K]. E <= 1024, K <= 32. */
int b200moe_route_topk(const float* logits, const float* bias, int64_t num_tokens, int32_t num_experts, int32_t top_k,
                       int32_t* ids, float* weights, void* stream);
/* Router logits x[T,H] (bf16) times gate[E,H]^T (bf16) in fp32. The reference synthesises its logits
 * (NV/problem/input.py:23-27), so this has no counterpart there. */
int b200moe_router_logits(const void* x, const void* gate_weight, int64_t num_tokens, int32_t hidden, int32_t num_experts,
                          float* logits, void* stream);

/* Dense NVFP4 GEMM: out[M,N] = bf16(alpha * A @ B^T), both operands NVFP4 with tiled scales. Contract of
 * DG/problem/reference.py:10-15 with the A operand quantised by b200moe_quantize_nvfp4; B rows are logical
 * (no shuffle). K % 256 == 0; out 32-byte aligned with out_stride % 16 == 0; tile_n as in b200moe_config (N % tile_n == 0, N % 256 == 0 for 512). status: optional device int32 that receives a non-zero code
 * if a bounded device wait expired. */
int b200moe_gemm_nvfp4(const void* a_q, const void* a_sf_tiled, const void* b_q, const void* b_sf_tiled, float alpha, void* out,
                       int64_t m, int64_t n, int64_t k, int64_t out_stride, int32_t tile_n, int32_t* status, void* stream);

/* Dense GEMM with bf16 activations and NVFP4 weights: out[M,N] = bf16(alpha * A @ decode(B)^T), A NOT quantised. The
 * contract of DG/problem/reference.py:10-15 as the operator publishes it (production entry flashinfer.mm_bf16_fp4,
 * DG/problem/solution.py:11-12): a bf16 [M, K] (a_stride elements between rows), b_q uint8 [N, K/2], b_descale E4M3
 * [N, K/16] row-major (not tiled), alpha a device fp32 scalar or NULL (= 1). K % 256 == 0, N % 128 == 0; out 32-byte
 * aligned with out_stride % 16 == 0. The weights are expanded to bf16 exactly (E2M1 x E4M3 has 6 significant bits), so
 * the result differs from the fp32 reference only by the order of the fp32 additions.
 * workspace (optional, 16-byte aligned device memory of at least b200moe_gemm_bf16_nvfp4_workspace_bytes(m, n, k) bytes;
 * that function returns 0 when none is useful): for M <= 128 it lets several CTAs share the reduction of one output
 * tile (fp32 partial sums added in a fixed order: results stay reproducible). Without it every tile is reduced by one
 * CTA, which leaves most of the device idle at small M. */
int64_t b200moe_gemm_bf16_nvfp4_workspace_bytes(int64_t m, int64_t n, int64_t k);
int b200moe_gemm_bf16_nvfp4(const void* a, int64_t a_stride, const void* b_q, const void* b_descale, const float* alpha, void* out,
                            int64_t m, int64_t n, int64_t k, int64_t out_stride, void* workspace, int64_t workspace_bytes,
                            int32_t* status, void* stream);

/* Layer life cycle. Replaces moe_init / moe_run of NV/candidate/nvfp4_moe.cu:6618, :9496 (bound there through
 * ctypes, NV/candidate/solution.py:96-102). create allocates the workspace on the current device. */
int b200moe_create(const b200moe_config* cfg, b200moe_handle* out);
int b200moe_destroy(b200moe_handle h);
int64_t b200moe_workspace_bytes(const b200moe_config* cfg);
int b200moe_workspace(b200moe_handle h, b200moe_workspace_view* out);

/* (1b) Expert-permutation index build only (route map into the workspace). Replaces k_count / k_scan_tiles /
 * k_scatter_agg of NV/candidate/nvfp4_moe.cu:582, :750, :700. */
int b200moe_route_map(b200moe_handle h, const int32_t* topk_ids, const float* topk_weights, int32_t num_tokens,
                      int32_t local_expert_offset, void* stream);

/* (4) Routing-weighted combine alone: out[t, :] = bf16( sum_s fp32(rows[row_of[t, s], :]) * weight_of_row[row_of[t, s]] ),
 * slots in ascending s, row_of < 0 skipped, every output element written. rows: bf16 [n_rows, hidden] contiguous.
 * Replaces k_finalize of NV/candidate/nvfp4_moe.cu:1464 (NV/problem/reference.py:91-92); the expert-parallel
 * wrapper calls it on the rows returned by the combine all-to-all. */
int b200moe_combine(const void* rows, const int32_t* row_of, const float* weight_of_row, int64_t num_tokens, int32_t slots,
                    int32_t hidden, void* out, int64_t out_stride, void* stream);

/* Expert-parallel dispatch helpers (the reference has no multi-GPU path; no counterpart there).
 * ep_visits: rank_slots[t, r] = r if token t has a route to an expert owned by rank r (experts are sharded
 * contiguously, experts_per_rank each), else -1. Feeding rank_slots to b200moe_route_map of a "plan" layer created with
 * num_experts = world and top_k = world yields the send order (tok_of_row), the 128-row aligned per-rank segments
 * (seg_start) and the position of every (token, rank) pair (row_of).
 * ep_pack: gathers one message row per pair of that plan into `out` ([rows, row_bytes] bytes): payload H/2 | scale
 * bytes H/16 | top_k local expert ids (int32, -1 for experts of other ranks) | top_k weights (fp32); padding rows of a
 * segment get ids = -1. The plan may carry one shared-expert slot (num_shared_experts = 1): its rows follow the last rank's
 * segment, are not messages and are skipped here, but give the caller row_of[:, world] for the locally computed shared
 * row. The receiver runs b200moe_run directly on the message buffer through the *_stride fields. */
int b200moe_ep_visits(const int32_t* topk_ids, int64_t num_tokens, int32_t top_k, int32_t experts_per_rank, int32_t world,
                      int32_t* rank_slots, void* stream);
int b200moe_ep_pack(b200moe_handle plan, const void* hidden_states, const void* hidden_states_scale, const int32_t* topk_ids,
                    const float* topk_weights, int32_t hidden, int32_t top_k, int32_t experts_per_rank, int64_t row_bytes, void* out,
                    void* stream);

/* Route-map build for callers that must not allocate device memory, e.g. code running inside a memory pool
 * it does not own, under a framework allocator that forbids raw cudaMalloc, or in a latency-critical section
 * where an allocation would synchronise the device. This entry point has no counterpart in the reference.
 * It computes exactly what b200moe_route_map computes, but into caller-provided output arrays (sizes as in
 * b200moe_workspace_view, totals holding 4 ints; row_capacity >= (T*(top_k+num_shared)/128 + experts + 1) * 128; the
 * pair items are not produced) and keeps its only
 * scratch, the per-block histograms, in a fixed array inside the library: at most 264 experts (routed + shared)
 * and 524288 routes, larger problems are refused with code 770. It never calls cudaMalloc, cudaFree or any
 * allocating routine. The first call on each device looks up the device address of that array (a host-side
 * query, no allocation); make that first call outside any CUDA stream capture. All calls on one device share the
 * array, so two calls whose kernels may overlap on the GPU (different streams) race; calls on one stream are safe.
 * Nothing in the scratch has to start at zero: every call overwrites the part it reads. Host threads may make a device's
 * first call concurrently (the address cache is an atomic; both look up the same value). */
int b200moe_route_map_noalloc(const int32_t* topk_ids, const float* topk_weights, int32_t num_tokens, int32_t top_k,
                              int32_t num_shared_experts, int32_t num_experts, int32_t local_expert_offset, int32_t* counts,
                              int32_t* seg_start, int32_t* tile_expert, int32_t* tile_row0, int32_t* tile_rows, int32_t* totals,
                              int32_t* row_of, int32_t* tok_of_row, float* weight_of_row, int64_t row_capacity, void* stream);

/* ---- Expert-parallel exchange over peer memory (NVLink). No counterpart in the reference operator, which has no
 * multi-GPU path (it only carries local_expert_offset / local_num_experts, NV/candidate/nvfp4_moe.cu:595-596); the
 * nearest model in the reference catalogue is the in-kernel exchange of OPS/moe/bf16_fused_moe/candidate/kernel.cuh
 * (:365-395 remote stores, :1072-1168 results into the source rank's buffer, :1224-1259 release/acquire flags).
 * One process per GPU. Each rank allocates one shared buffer, passes the 64-byte handle to its peers (any host
 * transport) and opens theirs; kernels of this library then write peers' buffers with plain stores and only ever
 * read or poll their own. Every device-side wait is bounded (about a second) and reports through the layer status. */
#define B200MOE_EP_MAX_RANKS 16
#define B200MOE_EP_CTRL_INTS (4 * B200MOE_EP_MAX_RANKS)   /* int32 words of one control block */
#define B200MOE_EP_FLAG_DISPATCH (2 * B200MOE_EP_MAX_RANKS) /* word offset of the "rows have landed" step counters */
#define B200MOE_EP_FLAG_RETURN (3 * B200MOE_EP_MAX_RANKS)   /* word offset of the "results have landed" step counters */
typedef struct {
  int32_t world, rank;
  void* recv[B200MOE_EP_MAX_RANKS];    /* [d]: this rank's region (seg_len rows) inside rank d's receive buffer */
  int32_t* ctrl[B200MOE_EP_MAX_RANKS]; /* [d]: rank d's control block (B200MOE_EP_CTRL_INTS words, zero before step 1) */
  void* ret[B200MOE_EP_MAX_RANKS];     /* [s]: rank s's return buffer, bf16 rows of `hidden` elements */
} b200moe_ep_peers;
/* cudaMalloc + clear + cudaIpcGetMemHandle (handle: 64 bytes out) / cudaIpcOpenMemHandle / close / free. */
int b200moe_ep_shared_alloc(int64_t bytes, void** ptr, void* ipc_handle);
int b200moe_ep_shared_open(const void* ipc_handle, void** ptr);
int b200moe_ep_shared_close(void* ptr);
int b200moe_ep_shared_free(void* ptr);
/* Dispatch of step `epoch` (1, 2, ...): `plan` is a layer whose "experts" are the ranks (plus one shared slot when
 * shared_slot != 0) and whose route map was built from b200moe_ep_visits output; one message row per (token, rank)
 * pair goes into the destination's receive region, then the segment size, its base row in this rank's return buffer
 * and the dispatch flag. With a shared slot, the plan's row_of[t, world] is pointed at row shared_base + t (weight 1).
 * `counter` is one zero-initialised uint32 in this rank's memory. */
int b200moe_ep_dispatch(b200moe_handle plan, const void* hidden_states, const void* hidden_states_scale, const int32_t* topk_ids,
                        const float* topk_weights, int32_t num_tokens, int32_t hidden, int32_t top_k, int32_t experts_per_rank,
                        int64_t row_bytes, const b200moe_ep_peers* peers, int32_t epoch, int32_t shared_slot, int32_t shared_base,
                        void* counter, void* stream);
/* Waits on the device (bounded) until flags[0..n) >= epoch; an expired wait sets status code 301 on `h`. */
int b200moe_ep_wait(b200moe_handle h, const int32_t* flags, int32_t n, int32_t epoch, void* stream);
/* After everything enqueued before it on `stream`: flag word `field` + rank of every peer's control block = epoch. */
int b200moe_ep_post(const b200moe_ep_peers* peers, int32_t field, int32_t epoch, void* stream);
/* The layer over the world * seg_len token slots of this rank's receive buffer (args->num_tokens = world * seg_len;
 * slots past ctrl[count of the region] are ignored): as b200moe_run, except that the combine pass writes the row of
 * slot (s, i) to row ctrl[ret_base of s] + i of rank s's return buffer instead of args->output. */
int b200moe_run_ep(b200moe_handle h, const b200moe_args* args, const b200moe_ep_peers* peers, const int32_t* ctrl, int32_t seg_len,
                   void* stream);

/* (3)+(4) Whole layer on `stream`, asynchronous: route map, permute, FC1 + activation + NVFP4 requantise,
 * FC2, routing-weighted combine into args->output. Replaces run_pipeline of NV/candidate/nvfp4_moe.cu:9078-9363
 * and matches expected() of NV/problem/reference.py:69-92 within the operator's tolerance. */
int b200moe_run(b200moe_handle h, const b200moe_args* args, void* stream);
/* Same, recording CUDA events between stages and returning their durations in milliseconds (synchronises).
 * stage_ms[0..4] = route map, permute, FC1, FC2, combine. Counterpart of moe_profile, NV/candidate/nvfp4_moe.cu:9678. */
int b200moe_run_profiled(b200moe_handle h, const b200moe_args* args, void* stream, float* stage_ms);
/* The whole step in one call, from bf16 tokens: (2) NVFP4 quantiser with a global scale, (1) router logits x * gate^T,
 * top-k / softmax (optional logit bias), then (3)+(4) the layer as b200moe_run with local_expert_offset 0. The quantised
 * tokens, logits, ids and weights live in the layer's workspace. With b200moe_config.graph_cache the chain of ~10 launches
 * is replayed as one graph from the second identical call on. No counterpart in the reference, whose operator starts from
 * routed NVFP4 inputs (NV/problem/input.py:101-112 generates them on the host side of its boundary). */
typedef struct {
  int32_t struct_size;               /* sizeof(b200moe_step_args) */
  int32_t num_tokens;
  const void* x;                     /* bf16 [T, H] */
  int64_t x_stride;                  /* elements between rows of x (>= H, multiple of 8) */
  const void* gate_weight;           /* bf16 [E, H] router matrix (E = num_experts of the layer) */
  const float* gate_bias;            /* fp32 [E] added to the logits before selection, or NULL */
  float activation_global_scale;     /* global scale of the activation quantiser (> 0) */
  int32_t activation_type;           /* as b200moe_args */
  const void* gemm1_weights;
  const void* gemm1_weights_scale;
  const void* gemm2_weights;
  const void* gemm2_weights_scale;
  const float* gemm1_alpha;
  const float* gemm1_beta;
  const float* gemm1_clamp_limit;
  const float* output1_scale_scalar;
  const float* output1_scale_gate_scalar;
  const float* output2_scale_scalar;
  void* output;                      /* bf16 [T, H] */
  int64_t output_stride;
} b200moe_step_args;
int b200moe_step(b200moe_handle h, const b200moe_step_args* args, void* stream);

/* Host-side counters of a layer (counterpart of the reference's graph_status() / nvfp4_fast.stats(),
 * NV/candidate/nvfp4_moe.cu:9618-9702, NV/candidate/nvfp4_fast.c:139-145). */
typedef struct {
  int64_t runs;             /* b200moe_run calls that launched work */
  int64_t graph_replays;    /* ... of which replayed a cached graph */
  int64_t graph_captures;   /* graphs captured (second identical call) */
  int64_t graph_evictions;  /* cached graphs dropped to make room (the cache holds 4) */
  int64_t eager_in_capture; /* calls made while the caller was capturing `stream` itself: launched into that capture */
  int64_t workspace_bytes;
} b200moe_stats;
int b200moe_get_stats(b200moe_handle h, b200moe_stats* out);

/* Synchronises `stream` and returns the device status word of the layer (0 = no bounded wait expired). */
int b200moe_status(b200moe_handle h, void* stream, int32_t* code);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H */
