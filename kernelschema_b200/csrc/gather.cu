// Permute: copy each routed token's NVFP4 row (payload + scale bytes) into expert order, so that the
// grouped GEMM reads its A operand as plain 128-row TMA boxes. Same role as the reference candidate's
// k_gather_f (moe/nvfp4_fused_moe/candidate/nvfp4_moe.cu:1189). Payload rows are copied with 128-bit
// loads/stores; the row-major token scales [T, H/16] are re-tiled on the fly into the 128x4 layout
// [row/128][H/64][32][16] that tcgen05.cp consumes. Padding rows get zero scales (their products vanish).
// HBM-bound: 2 * H * 9/16 bytes per routed row.
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

__global__ void __launch_bounds__(256) k_gather_rows(const uint8_t* __restrict__ hid_q, const uint8_t* __restrict__ hid_sf,
                                                     int hid_sf_tiled, int64_t q_stride, int64_t sf_stride,
                                                     const int32_t* __restrict__ tok_of_row,
                                                     const int32_t* __restrict__ tile_rows,
                                                     const int32_t* __restrict__ totals, int H, uint8_t* __restrict__ a_q,
                                                     uint8_t* __restrict__ a_sf) {
  // one warp per permuted row, 16 bytes per lane and step
  pdl_trigger();
  pdl_wait();
  const int rows = totals[1];
  const int lane = threadIdx.x & 31;
  const int vec_per_row = H >> 5;      // 16-byte vectors of payload per row (H/2 bytes)
  const int words_per_row = H >> 6;    // 4-byte scale words per row (H/16 bytes)
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    // segments are 128-row aligned and consecutive, so row r belongs to tile r / 128; rows past the tile's count are padding
    const int tok = ((r & 127) < tile_rows[r >> 7]) ? tok_of_row[r] : -1;
    uint32_t* sf_dst = reinterpret_cast<uint32_t*>(a_sf + (size_t)(r >> 7) * words_per_row * 512 + (size_t)(r & 31) * 16 +
                                                   (size_t)((r >> 5) & 3) * 4);
    if (tok < 0) {
      for (int w = lane; w < words_per_row; w += 32) sf_dst[(size_t)w * 128] = 0u;
      continue;
    }
    if (a_q) {                           // null: the GEMM gathers the payload rows itself, only the scales are permuted
      const uint4* src = reinterpret_cast<const uint4*>(hid_q + (size_t)tok * q_stride);
      uint4* dst = reinterpret_cast<uint4*>(a_q + (size_t)r * (H >> 1));
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = __ldg(src + v);
    }
    if (hid_sf_tiled) {
      const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(hid_sf + (size_t)(tok >> 7) * words_per_row * 512 +
                                                                 (size_t)(tok & 31) * 16 + (size_t)((tok >> 5) & 3) * 4);
      for (int w = lane; w < words_per_row; w += 32) sf_dst[(size_t)w * 128] = __ldg(sf_src + (size_t)w * 128);
    } else {
      const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(hid_sf + (size_t)tok * sf_stride);
      for (int w = lane; w < words_per_row; w += 32) sf_dst[(size_t)w * 128] = __ldg(sf_src + w);
    }
  }
}

// Tile form of the permute for row-major token scales: one block of 16 warps per 128-row tile of the permuted buffer. Warps
// 0-3 assemble the tile's scale image ([H/64] chunks of 512 bytes, the layout tcgen05.cp consumes) in shared memory -
// thread r walks the scale bytes of row r's token with 16-byte loads - and store it with full 16-byte coalesced writes
// (written word by word from the rows it would cost one 32-byte sector per 4 bytes). Payload rows are dealt to the warps
// from a shared counter, one row (eight 16-byte vectors per lane in flight) at a time: the other twelve warps start at
// once, the scale warps join when the image is out. Padding rows (past the tile's count) get zero scales and keep whatever
// payload they had. a_q == null: scales only (the GEMM fetches the payload rows of the tokens itself).
__global__ void __launch_bounds__(512, 2) k_gather_tiles(const uint8_t* __restrict__ hid_q, const uint8_t* __restrict__ hid_sf,
                                                         int64_t q_stride, int64_t sf_stride, const int32_t* __restrict__ tok_of_row,
                                                         const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ totals, int H,
                                                         uint8_t* __restrict__ a_q, uint8_t* __restrict__ a_sf) {
  extern __shared__ uint4 s_img4[];                 // [H/64][512 B]
  uint32_t* s_img = reinterpret_cast<uint32_t*>(s_img4);
  __shared__ int s_tok[128];
  __shared__ int s_next;
  pdl_trigger();
  pdl_wait();
  const int n_tiles = totals[0];
  const int lane = threadIdx.x & 31;
  const int chunks = H >> 6;                        // 512-byte scale chunks per tile = 4-byte scale words per row
  const int vec_per_row = H >> 5;                   // 16-byte vectors of payload per row
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int rows = tile_rows[tile];
    const int row0 = tile << 7;
    if (threadIdx.x < 128) s_tok[threadIdx.x] = threadIdx.x < rows ? tok_of_row[row0 + threadIdx.x] : -1;
    if (threadIdx.x == 0) s_next = 0;
    __syncthreads();
    if (threadIdx.x < 128) {
      const int r = threadIdx.x;
      const int tok = s_tok[r];
      uint32_t* dst = s_img + (r & 31) * 4 + (r >> 5);          // word (row, chunk j) lives at j * 128 + (r % 32) * 4 + r / 32
      if (tok >= 0) {
        const uint4* src = reinterpret_cast<const uint4*>(hid_sf + (size_t)tok * sf_stride);
        for (int j0 = 0; j0 < (chunks >> 2); j0 += 4) {          // four 16-byte loads in flight, then their 16 words
          uint4 v[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (j0 + i < (chunks >> 2)) v[i] = __ldg(src + j0 + i);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (j0 + i < (chunks >> 2)) {
              const int j4 = j0 + i;
              dst[(4 * j4 + 0) * 128] = v[i].x;
              dst[(4 * j4 + 1) * 128] = v[i].y;
              dst[(4 * j4 + 2) * 128] = v[i].z;
              dst[(4 * j4 + 3) * 128] = v[i].w;
            }
        }
      } else {
        for (int j = 0; j < chunks; ++j) dst[j * 128] = 0u;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");             // the four scale warps only: the image is complete
      uint4* out = reinterpret_cast<uint4*>(a_sf + (size_t)tile * chunks * 512);
      for (int i = threadIdx.x; i < chunks * 32; i += 128) out[i] = s_img4[i];
    }
    if (a_q) {
      for (;;) {
        int r = 0;
        if (lane == 0) r = atomicAdd(&s_next, 1);
        r = __shfl_sync(0xFFFFFFFFu, r, 0);
        if (r >= rows) break;
        copy_row_batched(reinterpret_cast<const uint4*>(hid_q + (size_t)s_tok[r] * q_stride),
                         reinterpret_cast<uint4*>(a_q + (size_t)(row0 + r) * (H >> 1)), vec_per_row, lane);
      }
    }
    __syncthreads();                                  // s_tok, the counter and the image are reused by the next tile
  }
}

int launch_gather_rows(const void* hid_q, const void* hid_sf, int hid_sf_tiled, int64_t q_stride, int64_t sf_stride,
                       const int32_t* tok_of_row, const int32_t* tile_rows, const int32_t* totals,
                       int H, int64_t row_capacity, void* a_q, void* a_sf, cudaStream_t st) {
  if (row_capacity == 0) return 0;
  const int64_t qs = q_stride > 0 ? q_stride : (int64_t)(H / 2), ss = sf_stride > 0 ? sf_stride : (int64_t)(H / 16);
  const size_t img = (size_t)(H >> 6) * 512;
  if (!hid_sf_tiled && H % 256 == 0 && ss % 16 == 0 && ((uintptr_t)hid_sf & 15) == 0 && img <= 96 * 1024) {
    static SmemOptIn opt_in;
    if (int e = opt_in.ensure(k_gather_tiles, (int)(96 * 1024))) return e;
    int64_t blocks = row_capacity / 128;
    const int64_t resident = (int64_t)sm_count() * 2;      // two 512-thread blocks per SM
    if (blocks > resident) blocks = resident;
    if (blocks < 1) blocks = 1;
    return (int)launch_chain(k_gather_tiles, dim3((unsigned)blocks), dim3(512), img, st, (const uint8_t*)hid_q, (const uint8_t*)hid_sf,
                             qs, ss, tok_of_row, tile_rows, totals, H, (uint8_t*)a_q, (uint8_t*)a_sf);
  }
  // Tiled token scales (or odd strides): one warp per permuted row. Short rows (H <= 4096): a resident grid of 8 blocks per
  // SM walks the rows. Long rows: one warp per row of the capacity; rows past the count in `totals` exit at once.
  int64_t blocks = (row_capacity + 7) / 8;
  if (H <= 4096 && blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  return (int)launch_chain(k_gather_rows, dim3((unsigned)blocks), dim3(256), 0, st, (const uint8_t*)hid_q, (const uint8_t*)hid_sf,
                           hid_sf_tiled, qs, ss, tok_of_row, tile_rows, totals, H, (uint8_t*)a_q, (uint8_t*)a_sf);
}

// ----------------------------------------------------------------------------- expert-parallel dispatch packing
// One message row per (token, destination rank) pair: [payload H/2 | scale bytes H/16 | K local expert ids (int32) |
// K routing weights (fp32)], padded to a multiple of 16 bytes. The pairs come from a route map whose "experts" are
// the destination ranks (segments are 128-row aligned; rows past a tile's count are padding and get ids = -1, so the
// receiver ignores them). One warp per row.
__global__ void __launch_bounds__(256) k_ep_pack(const uint8_t* __restrict__ hid_q, const uint8_t* __restrict__ hid_sf,
                                                 const int32_t* __restrict__ ids, const float* __restrict__ weights,
                                                 const int32_t* __restrict__ tok_of_row, const int32_t* __restrict__ tile_expert,
                                                 const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ totals, int H,
                                                 int K, int experts_per_rank, int world, int64_t row_bytes, uint8_t* __restrict__ out) {
  const int rows = totals[1];
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int q_vecs = H >> 5, sf_words = H >> 6;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int dest = tile_expert[r >> 7];
    if (dest >= world) break;  // rows of the plan's shared-expert slot follow the last rank's segment: not messages
    uint8_t* dst = out + (size_t)r * row_bytes;
    int32_t* id_dst = reinterpret_cast<int32_t*>(dst + (H >> 1) + (H >> 4));
    float* w_dst = reinterpret_cast<float*>(id_dst + K);
    const bool live = (r & 127) < tile_rows[r >> 7];
    if (!live) {
      if (lane < K) id_dst[lane] = -1;
      continue;
    }
    const int tok = tok_of_row[r];
    const uint4* src = reinterpret_cast<const uint4*>(hid_q + (size_t)tok * (H >> 1));
    for (int v = lane; v < q_vecs; v += 32) reinterpret_cast<uint4*>(dst)[v] = __ldg(src + v);
    const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(hid_sf + (size_t)tok * (H >> 4));
    for (int w = lane; w < sf_words; w += 32) reinterpret_cast<uint32_t*>(dst + (H >> 1))[w] = __ldg(sf_src + w);
    if (lane < K) {
      const int g = ids[(size_t)tok * K + lane];
      const bool here = g >= 0 && g / experts_per_rank == dest;
      id_dst[lane] = here ? g - dest * experts_per_rank : -1;
      w_dst[lane] = weights[(size_t)tok * K + lane];
    }
  }
}

// rank_slots[t, r] = r when token t has at least one route to an expert of rank r, else -1.
__global__ void k_ep_visits(const int32_t* __restrict__ ids, int64_t T, int K, int experts_per_rank, int world,
                            int32_t* __restrict__ rank_slots) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * world) return;
  const int64_t t = idx / world;
  const int r = (int)(idx - t * world);
  bool hit = false;
  for (int k = 0; k < K; ++k) {
    const int g = ids[t * K + k];
    hit |= (g >= 0 && g / experts_per_rank == r);
  }
  rank_slots[idx] = hit ? r : -1;
}

int launch_ep_visits(const int32_t* ids, int64_t T, int K, int experts_per_rank, int world, int32_t* rank_slots, cudaStream_t st) {
  const int64_t n = T * world;
  if (n == 0) return 0;
  k_ep_visits<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, T, K, experts_per_rank, world, rank_slots);
  return (int)cudaGetLastError();
}

int launch_ep_pack(const void* hid_q, const void* hid_sf, const int32_t* ids, const float* weights, const int32_t* tok_of_row,
                   const int32_t* tile_expert, const int32_t* tile_rows, const int32_t* totals, int H, int K, int experts_per_rank,
                   int world, int64_t row_bytes, int64_t row_capacity, void* out, cudaStream_t st) {
  if (row_capacity == 0) return 0;
  int64_t blocks = (row_capacity + 7) / 8;
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  k_ep_pack<<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)hid_q, (const uint8_t*)hid_sf, ids, weights, tok_of_row, tile_expert,
                                             tile_rows, totals, H, K, experts_per_rank, world, row_bytes, (uint8_t*)out);
  return (int)cudaGetLastError();
}

}  // namespace b200
