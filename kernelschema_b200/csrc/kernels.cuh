// Internal launch interface shared by the kernel files and the C-ABI layer (api.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace b200 {

enum { kGemmDense = 0, kGemmFc1 = 1, kGemmFc2 = 2 };

// True unless the environment says B200MOE_PDL=0 (read once): launches carry the programmatic-stream-serialization
// attribute, so consecutive kernels of the layer overlap launch latency and prologue (see pdl_wait in ptx.cuh).
bool pdl_enabled();

// Multiprocessors of the current device (queried once per device, then cached).
int sm_count();

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (kernel, device) pair: one of these per kernel remembers on
// which devices the opt-in has been made, so that a process driving several GPUs configures each of them.
struct SmemOptIn {
  std::atomic<unsigned long long> done{0};
  template <class Kernel>
  int ensure(Kernel kern, int bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    const unsigned long long bit = 1ull << (dev & 63);
    if (dev < 64 && (done.load(std::memory_order_acquire) & bit)) return 0;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    if (dev < 64) done.fetch_or(bit, std::memory_order_release);
    return 0;
  }
  // which devices have been configured (bit d = device d); for tests of the bookkeeping
  unsigned long long mask() const { return done.load(std::memory_order_acquire); }
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Device buffers produced by the route-map build.
struct RouteMapBuffers {
  int32_t* block_hist;     // [nblk, E'] scratch
  int32_t* counts;         // [E']
  int32_t* seg_start;      // [E' + 1], multiples of 128
  int32_t* tile_expert;    // [tile_capacity]
  int32_t* tile_row0;      // [tile_capacity]
  int32_t* tile_rows;      // [tile_capacity] valid rows of the tile (1..128)
  int32_t* totals;         // {n_tiles, rows in use (multiple of 128), valid routes, n_pairs}
  int32_t* pair_expert;    // [tile_capacity] 256-row items of the CTA-pair GEMM (may be null: not built)
  int32_t* pair_row0;      // [tile_capacity]
  int32_t* pair_rows;      // [tile_capacity] valid rows of the pair (1..256)
  int32_t* row_of;         // [T, K'] permuted row of a route, -1 when invalid
  int32_t* tok_of_row;     // [row_capacity] token of a permuted row; padding rows (past tile_rows of tile row/128) are unspecified
  float* weight_of_row;    // [row_capacity] routing weight of a permuted row
  int64_t row_capacity;
};

struct GemmParams {
  const int32_t* tile_expert;   // null: dense (expert 0, m-tiles are consecutive 128-row blocks)
  const int32_t* tile_row0;
  const int32_t* tile_rows;
  const int32_t* n_tiles_ptr;   // device count of m-tiles, or null -> n_tiles_static
  int n_tiles_static;
  int M;                        // rows of A (dense mode only)
  int64_t rows_hint;            // most rows of A this launch can hold (0 = unknown): picks the epilogue shape, nothing else
  int N;                        // weight rows per expert (2I for FC1, H for FC2)
  int K;                        // reduction length in FP4 elements
  const int32_t* a_tok;         // FC1 only, non-null: the A map covers the TOKEN rows (box {128, 1}) and row r of a tile is fetched from
                                // token a_tok[row0 + r] by TMA gather; null: the A map covers pre-permuted rows
  const uint8_t* sfa;           // A scales, 128x4 tiles [rows/128][K/64][512]
  const uint8_t* sfb;           // B scales, 128x4 tiles [E*N/128][K/64][512]
  uint8_t* act_q;               // FC1 out: packed activations [rows, I/2]
  uint8_t* act_sf;              // FC1 out: activation scales, 128x4 tiles [rows/128][I/64][512]
  __nv_bfloat16* out;           // FC2 / dense out
  int64_t out_stride;           // elements between output rows
  const int32_t* out_row_index; // FC2 only: output row of permuted row r is out_row_index[r] (null = r itself)
  const float* scale_up;        // per expert multipliers of the FC1 accumulators (null = 1)
  const float* scale_gate;
  const float* alpha;           // per expert activation parameters (null = 1 / 0 / no clamp)
  const float* beta;
  const float* limit;
  int act_type;                 // 3 = SwiGLU form gate*sigmoid(alpha*gate)*(up+beta); 10 = SiTU
  const float* out_scale;       // per expert multiplier of the FC2 accumulator (null = 1)
  float dense_alpha;
  int32_t* status;              // device word; first non-zero code sticks (bounded waits report here)
};

int launch_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int64_t row_stride, float gs, void* payload, void* scales,
                          int sf_layout, cudaStream_t st);
int launch_sf_to_tiles(const void* src, int64_t rows, int64_t blocks_per_row, void* dst, cudaStream_t st);
int launch_route_topk(const float* logits, const float* bias, int64_t T, int E, int K, int32_t* ids, float* weights,
                      cudaStream_t st);
int launch_router_logits(const void* x, const void* w, int64_t T, int H, int E, float* logits, cudaStream_t st);
int launch_router_logits_tc(const void* x, const void* w, int64_t T, int H, int E, float* logits, int32_t* status, cudaStream_t st);
// While (token tiles) x (64-expert slices) fit one wave: clusters of blocks split the k-steps and meet in distributed shared
// memory. Returns -1 when the shape does not qualify (the caller then uses launch_router_logits_tc).
int launch_router_logits_ksplit(const void* x, const void* w, int64_t T, int H, int E, float* logits, int32_t* status, cudaStream_t st);
int launch_router_logits_small(const void* x, const void* w, int64_t T, int H, int E, float* logits, cudaStream_t st);   // T <= 16
// seg_len > 0: the T token slots are regions of seg_len consecutive slots and only the first seg_valid[slot / seg_len]
// slots of each region hold a token (the receive buffer of the expert-parallel exchange); the rest count as unrouted.
int launch_route_map(const int32_t* ids, const float* scores, int64_t id_stride, int64_t T, int K, int S, int E, int expert_offset,
                     RouteMapBuffers b, cudaStream_t st, int seg_len = 0, const int32_t* seg_valid = nullptr);
// Route map and permute in ONE launch for batches of at most 8192 routes with row-major token scales (decode sizes):
// `route_gather_fits` says whether a call qualifies.
bool route_gather_fits(int64_t T, int K, int S, int E, int H);
int launch_route_gather(const int32_t* ids, const float* scores, int64_t id_stride, int64_t T, int K, int S, int E, int expert_offset,
                        RouteMapBuffers b, const void* hid_q, const void* hid_sf, int64_t q_stride, int64_t sf_stride, int H, void* a_q,
                        void* a_sf, cudaStream_t st, int seg_len = 0, const int32_t* seg_valid = nullptr);
int launch_route_map_static(const int32_t* ids, const float* scores, int64_t T, int K, int S, int E, int expert_offset,
                            RouteMapBuffers b, cudaStream_t st);
int launch_ep_visits(const int32_t* ids, int64_t T, int K, int experts_per_rank, int world, int32_t* rank_slots, cudaStream_t st);
int launch_ep_pack(const void* hid_q, const void* hid_sf, const int32_t* ids, const float* weights, const int32_t* tok_of_row,
                   const int32_t* tile_expert, const int32_t* tile_rows, const int32_t* totals, int H, int K, int experts_per_rank,
                   int world, int64_t row_bytes, int64_t row_capacity, void* out, cudaStream_t st);
int launch_gather_rows(const void* hid_q, const void* hid_sf, int hid_sf_tiled, int64_t q_stride, int64_t sf_stride,
                       const int32_t* tok_of_row, const int32_t* tile_rows, const int32_t* totals,
                       int H, int64_t row_capacity, void* a_q, void* a_sf, cudaStream_t st);
int launch_finalize(const void* rout, const int32_t* row_of, const float* weight_of_row, int64_t T, int KK, int H, void* out,
                    int64_t out_stride, cudaStream_t st);
int make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                     uint64_t pitch_bytes = 0);   // pitch 0 = rows are contiguous
int launch_gemm_w4a16(const void* a, int64_t a_stride, const void* b_q, const void* b_sf, const float* alpha, int64_t m, int64_t n,
                      int64_t k, void* out, int64_t out_stride, void* workspace, int64_t workspace_bytes, int32_t* status,
                      cudaStream_t st);
int64_t gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k);
int make_sf_map(CUtensorMap* map, const void* base, uint64_t n_chunks);

// ---- expert-parallel exchange over peer memory (ep_exchange.cu)
constexpr int kEpMaxRanks = 16;
// int32 fields of a rank's control block, each kEpMaxRanks wide and indexed by the peer that writes it
constexpr int kEpCount = 0;                           // rows the peer sent (its segment, padded to 128)
constexpr int kEpRetBase = kEpMaxRanks;               // first row of that segment in the peer's return buffer
constexpr int kEpFlagDispatch = 2 * kEpMaxRanks;      // step counter: the peer's rows and the two fields above have landed
constexpr int kEpFlagReturn = 3 * kEpMaxRanks;        // step counter: the peer has written its results into my return buffer
constexpr int kEpCtrlInts = 4 * kEpMaxRanks;
struct EpPeers {                   // addresses for the current step's parity, passed to kernels by value
  int32_t world, rank;
  uint8_t* recv[kEpMaxRanks];      // [d]: this rank's region inside rank d's receive buffer
  int32_t* ctrl[kEpMaxRanks];      // [d]: rank d's control block
  void* ret[kEpMaxRanks];          // [s]: rank s's return buffer (bf16 rows)
};
int launch_ep_dispatch(const void* hid_q, const void* hid_sf, const int32_t* ids, const float* weights, const int32_t* tok_of_row,
                       const int32_t* tile_expert, const int32_t* tile_rows, const int32_t* seg_start, const int32_t* totals, int H,
                       int K, int experts_per_rank, int64_t row_bytes, int64_t row_capacity, const EpPeers& peers, int epoch, int64_t T,
                       int shared_slots, int shared_base, int32_t* row_of, float* weight_of_row, unsigned int* done_counter,
                       cudaStream_t st);
int launch_ep_wait(const int32_t* flags, int n, int epoch, int32_t* status, int code, cudaStream_t st);
int launch_ep_post(const EpPeers& peers, int field, int epoch, cudaStream_t st);
int launch_finalize_ep(const void* rout, const int32_t* row_of, const float* weight_of_row, int64_t T, int KK, int H,
                       const EpPeers& peers, const int32_t* ctrl, int seg_len, cudaStream_t st);
int launch_gemm_nvfp4_pair(int mode, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                           const GemmParams& p, int n_clusters, cudaStream_t st);
int launch_gemm_nvfp4(int mode, int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                      cudaStream_t st);

}  // namespace b200
