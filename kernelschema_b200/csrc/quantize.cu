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

// Quotients x / (stored * gs) without sixteen IEEE divisions per block. With d = RN(stored * gs) (what the reference
// divides by), r = RN(1 / d), q0 = RN(x * r), the residual rem = x - q0 * d is exact in one fma (q0 is within 1.5 ulp of
// x / d and x has only 8 significant bits), and q1 = RN(q0 + rem * r) is the correctly rounded quotient (Markstein's
// residual correction with a correctly rounded reciprocal). The E2M1 code only depends on the side of seven thresholds
// the quotient lies on, so a last-bit error could matter only when x / d is within an ulp of a threshold; the test suite
// sweeps every bf16 value against every E4M3 scale x a set of global scales and compares the codes with true division.
// EXACT_DIV selects IEEE division instead (global scales so small or large that the residual could leave the normal range).
template <bool EXACT_DIV>
__global__ void __launch_bounds__(256) k_quantize_nvfp4(const __nv_bfloat16* __restrict__ x, int64_t rows, int64_t cols,
                                                        int64_t row_stride, float gs, uint8_t* __restrict__ payload,
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
    }
    float peak = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) peak = fmaxf(peak, fabsf(v[i]));
    peak = fmaxf(peak, 9.5367431640625e-07f);                       // clamp_min(2^-20), before the global scale
    float scale = __fdiv_rn(peak, 6.0f);
    if (gs != 1.0f) scale = __fdiv_rn(scale, gs);
    scale = fminf(fmaxf(scale, 0.001953125f), 448.0f);               // clamp(2^-9, 448)
    const uint32_t sbyte = cvt_e4m3(scale);
    const float d = __fmul_rn(e4m3_to_f32(sbyte), gs);               // the reference divides by stored * gs
    uint32_t packed[2];
    if (EXACT_DIV) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          word |= cvt_e2m1x2(__fdiv_rn(v[8 * h + 2 * i], d), __fdiv_rn(v[8 * h + 2 * i + 1], d)) << (8 * i);
        packed[h] = word;
      }
    } else {
      const float r = __frcp_rn(d);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = v[8 * h + 2 * i], b = v[8 * h + 2 * i + 1];
          float qa = a * r, qb = b * r;
          qa = copysignf(fmaf(fmaf(-qa, d, a), r, qa), a);     // keep -0 and negative underflow: they encode as 8
          qb = copysignf(fmaf(fmaf(-qb, d, b), r, qb), b);
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
  const int64_t resident = (int64_t)sm_count() * 32;
  const int64_t blocks = rows < resident ? rows : resident;
  // stored * gs stays a normal number with room for the residual of a bf16 numerator inside 2^-40 .. 2^40
  const bool fast = gs >= 0x1p-40f && gs <= 0x1p40f;
  if (fast)
    return (int)launch_chain(k_quantize_nvfp4<false>, dim3((unsigned)blocks), dim3(threads), 0, st, (const __nv_bfloat16*)x, rows, cols,
                             row_stride, gs, (uint8_t*)payload, (uint8_t*)scales, sf_layout);
  return (int)launch_chain(k_quantize_nvfp4<true>, dim3((unsigned)blocks), dim3(threads), 0, st, (const __nv_bfloat16*)x, rows, cols,
                           row_stride, gs, (uint8_t*)payload, (uint8_t*)scales, sf_layout);
}

int launch_sf_to_tiles(const void* src, int64_t rows, int64_t blocks_per_row, void* dst, cudaStream_t st) {
  const int64_t rows_pad = (rows + 127) & ~(int64_t)127;
  const int64_t total = rows_pad * (blocks_per_row >> 2);
  if (total == 0) return 0;
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
  k_sf_to_tiles<<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)src, rows, blocks_per_row, (uint8_t*)dst);
  return (int)cudaGetLastError();
}

}  // namespace b200
