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
                                                     int hid_sf_tiled, const int32_t* __restrict__ tok_of_row,
                                                     const int32_t* __restrict__ tile_rows,
                                                     const int32_t* __restrict__ totals, int H, uint8_t* __restrict__ a_q,
                                                     uint8_t* __restrict__ a_sf) {
  // one warp per permuted row, 16 bytes per lane and step
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
    const uint4* src = reinterpret_cast<const uint4*>(hid_q + (size_t)tok * (H >> 1));
    uint4* dst = reinterpret_cast<uint4*>(a_q + (size_t)r * (H >> 1));
    for (int v = lane; v < vec_per_row; v += 32) dst[v] = __ldg(src + v);
    if (hid_sf_tiled) {
      const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(hid_sf + (size_t)(tok >> 7) * words_per_row * 512 +
                                                                 (size_t)(tok & 31) * 16 + (size_t)((tok >> 5) & 3) * 4);
      for (int w = lane; w < words_per_row; w += 32) sf_dst[(size_t)w * 128] = __ldg(sf_src + (size_t)w * 128);
    } else {
      const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(hid_sf + (size_t)tok * (H >> 4));
      for (int w = lane; w < words_per_row; w += 32) sf_dst[(size_t)w * 128] = __ldg(sf_src + w);
    }
  }
}

int launch_gather_rows(const void* hid_q, const void* hid_sf, int hid_sf_tiled, const int32_t* tok_of_row, const int32_t* tile_rows,
                       const int32_t* totals,
                       int H, int64_t row_capacity, void* a_q, void* a_sf, cudaStream_t st) {
  if (row_capacity == 0) return 0;
  int64_t blocks = (row_capacity + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  k_gather_rows<<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)hid_q, (const uint8_t*)hid_sf, hid_sf_tiled, tok_of_row, tile_rows,
                                                 totals, H, (uint8_t*)a_q, (uint8_t*)a_sf);
  return (int)cudaGetLastError();
}

}  // namespace b200
