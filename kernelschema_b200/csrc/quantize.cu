// bf16 -> NVFP4 quantiser (16-element blocks, E4M3 block scale, optional fp32 global scale).
//
// Follows, bit for bit, the reference input generator's quantize():
//   moe/nvfp4_fused_moe/problem/input.py:53-71            (global scale 1)
//   gemm/dense/bf16_nvfp4_gemm/problem/input.py:40-64     (global scale != 1)
// One thread owns one 16-element block: two 128-bit loads, one 64-bit payload store, one scale byte.
// HBM-bound: 2 B read + 0.5625 B written per element.
#include <math.h>

#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

// Scale byte position inside the 128x4-tiled layout [rows/128][cols/64][32][16]
// (element (row, blk) at [row/128, blk/4, row%32, 4*((row%128)/32) + blk%4]), the layout tcgen05.cp consumes.
DEV size_t sf_tiled_offset(int64_t row, int64_t blk, int64_t chunks_per_row) {
  return ((size_t)(row >> 7) * chunks_per_row + (size_t)(blk >> 2)) * 512 + (size_t)(row & 31) * 16 + (size_t)((row >> 5) & 3) * 4 +
         (size_t)(blk & 3);
}

// GLOBAL_SCALE = false also serves power-of-two global scales: dividing by 2^k is exact, so
// quantize(x, 2^k) == quantize(x * 2^-k, 1) bit for bit and `prescale` = 2^-k is applied to the loaded values.
template <bool GLOBAL_SCALE>
__global__ void __launch_bounds__(256) k_quantize_nvfp4(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                                                        int64_t row_stride, float gs, float prescale, uint8_t* __restrict__ payload,
                                                        uint8_t* __restrict__ scales, int sf_layout) {
  // One block walks rows, its threads walk the 16-element blocks of a row: no integer division anywhere.
  const int blocks_per_row = (int)(cols >> 4);
  pdl_trigger();
  pdl_wait();
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x)
  for (int blk = threadIdx.x; blk < blocks_per_row; blk += blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + row * row_stride + blk * 16);
    uint4 raw[2];
    raw[0] = __ldg(src);
    raw[1] = __ldg(src + 1);
    const uint32_t* w = reinterpret_cast<const uint32_t*>(raw);
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      if (!GLOBAL_SCALE) { v[2 * i] *= prescale; v[2 * i + 1] *= prescale; }
    }
    float peak = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) peak = fmaxf(peak, fabsf(v[i]));
    peak = fmaxf(peak, 9.5367431640625e-07f);                       // clamp_min(2^-20)
    float scale = __fdiv_rn(peak, 6.0f);
    if (GLOBAL_SCALE) scale = __fdiv_rn(scale, gs);
    scale = fminf(fmaxf(scale, 0.001953125f), 448.0f);               // clamp(2^-9, 448)
    const uint32_t sbyte = cvt_e4m3(scale);
    const float sf = e4m3_to_f32(sbyte);
    uint32_t packed[2];
    if (GLOBAL_SCALE) {
      // The divisor stored*gs is an arbitrary fp32 number: only the correctly rounded quotient matches the reference.
      const float d = __fmul_rn(sf, gs);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          word |= cvt_e2m1x2(__fdiv_rn(v[8 * h + 2 * i], d), __fdiv_rn(v[8 * h + 2 * i + 1], d)) << (8 * i);
        packed[h] = word;
      }
    } else {
      // x is bf16 (8 significant bits) and sf has 4, so x/sf is either exactly on an E2M1 midpoint or at least
      // 2^-9 (relative) away from it. One residual-corrected reciprocal multiply is exact on the ties and
      // accurate to ~2^-23 elsewhere, hence yields the same codes as the IEEE division the reference performs.
      const float r = __frcp_rn(sf);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = v[8 * h + 2 * i], b = v[8 * h + 2 * i + 1];
          float qa = a * r, qb = b * r;
          qa = copysignf(fmaf(fmaf(-qa, sf, a), r, qa), a);     // keep -0 and negative underflow: they encode as 8
          qb = copysignf(fmaf(fmaf(-qb, sf, b), r, qb), b);
          word |= cvt_e2m1x2(qa, qb) << (8 * i);
        }
        packed[h] = word;
      }
    }
    *reinterpret_cast<uint2*>(payload + row * (cols >> 1) + (int64_t)blk * 8) = make_uint2(packed[0], packed[1]);
    if (sf_layout == 0)
      scales[row * blocks_per_row + blk] = (uint8_t)sbyte;
    else
      scales[sf_tiled_offset(row, blk, cols >> 6)] = (uint8_t)sbyte;
  }
}

// Row-major scale bytes [rows, cols/16] -> 128x4 tiles; rows beyond `rows` up to the next multiple of 128 become 0.
__global__ void k_sf_to_tiles(const uint8_t* __restrict__ src, int64_t rows, int64_t blocks_per_row, uint8_t* __restrict__ dst) {
  const int64_t rows_pad = (rows + 127) & ~(int64_t)127;
  const int64_t words_per_row = blocks_per_row >> 2;
  const int64_t total = rows_pad * words_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / words_per_row;
    const int64_t wd = idx - row * words_per_row;
    uint32_t val = 0;
    if (row < rows) val = *reinterpret_cast<const uint32_t*>(src + row * blocks_per_row + wd * 4);
    *reinterpret_cast<uint32_t*>(dst + sf_tiled_offset(row, wd * 4, words_per_row)) = val;
  }
}

int launch_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int64_t row_stride, float gs, void* payload, void* scales,
                          int sf_layout, cudaStream_t st) {
  if (rows == 0) return 0;
  const int bpr = (int)(cols >> 4);
  // threads = blocks per row rounded up to a warp, split into equal passes of at most 256 threads
  const int passes = (bpr + 255) / 256;
  int threads = ((bpr + passes - 1) / passes + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  const int64_t blocks = rows < 148LL * 32 ? rows : 148LL * 32;
  int exp2 = 0;
  const bool pow2 = frexpf(gs, &exp2) == 0.5f && exp2 > -100 && exp2 < 100;     // gs = 2^(exp2-1): exact pre-scaling
  if (pow2)
    return (int)launch_chain(k_quantize_nvfp4<false>, dim3((unsigned)blocks), dim3(threads), 0, st, (const __nv_bfloat16*)x, rows, cols,
                             row_stride, gs, ldexpf(1.0f, 1 - exp2), (uint8_t*)payload, (uint8_t*)scales, sf_layout);
  return (int)launch_chain(k_quantize_nvfp4<true>, dim3((unsigned)blocks), dim3(threads), 0, st, (const __nv_bfloat16*)x, rows, cols,
                           row_stride, gs, 1.0f, (uint8_t*)payload, (uint8_t*)scales, sf_layout);
}

int launch_sf_to_tiles(const void* src, int64_t rows, int64_t blocks_per_row, void* dst, cudaStream_t st) {
  const int64_t rows_pad = (rows + 127) & ~(int64_t)127;
  const int64_t total = rows_pad * (blocks_per_row >> 2);
  if (total == 0) return 0;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  k_sf_to_tiles<<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)src, rows, blocks_per_row, (uint8_t*)dst);
  return (int)cudaGetLastError();
}

}  // namespace b200
