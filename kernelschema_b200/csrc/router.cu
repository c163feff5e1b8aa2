// Router: top-k selection over expert logits and softmax over the selected logits.
//
// Follows the reference input generator's routes() (moe/nvfp4_fused_moe/problem/input.py:35-41):
//   selected, ids = logits.topk(K); weights = softmax(selected); invalid routes -> id -1, weight 0.
// ids come out in descending-logit order, ties to the lowest expert index. The softmax is evaluated
// in fp64 and rounded once to fp32 so the result does not depend on an exp() implementation.
// One warp per token; each lane keeps E/32 logits in registers.
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kMaxExpertsPerLane = 32;   // E <= 1024

__global__ void __launch_bounds__(256) k_route_topk(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T,
                                                    int E, int K, int32_t* __restrict__ ids, float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (tok >= T) return;
  float v[kMaxExpertsPerLane];
  const int per_lane = (E + 31) >> 5;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = i * 32 + lane;
    float x = -INFINITY;
    if (i < per_lane && e < E) {
      x = logits[tok * E + e];
      if (bias) x = __fadd_rn(x, bias[e]);
    }
    v[i] = x;
  }
  float sel = 0.f;      // lane k keeps the k-th selected logit
  int sel_id = -1;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int best_e = 0x7FFFFFFF;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      if (i < per_lane) {
        const int e = i * 32 + lane;
        if (e < E && (v[i] > best)) { best = v[i]; best_e = e; }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, off);
      const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, off);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (lane == k) { sel = best; sel_id = best_e; }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i)
        if (i == (best_e >> 5)) v[i] = -INFINITY;
    }
  }
  const float top = __shfl_sync(0xFFFFFFFFu, sel, 0);
  double ex = (lane < K) ? exp((double)sel - (double)top) : 0.0;
  double sum = ex;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
  if (lane < K) {
    ids[tok * K + lane] = sel_id;
    weights[tok * K + lane] = (float)(ex / sum);
  }
}

// logits[t, e] = sum_h x[t, h] * w[e, h], bf16 operands, fp32 accumulation. One warp per (token, 8 experts).
__global__ void __launch_bounds__(256) k_router_logits(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                       int64_t T, int H, int E, float* __restrict__ logits) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t tok = blockIdx.x;
  const int e0 = (blockIdx.y * 8 + warp) * 8;
  if (tok >= T || e0 >= E) return;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const uint4* xr = reinterpret_cast<const uint4*>(x + tok * H);
  for (int c = lane; c < (H >> 3); c += 32) {
    const uint4 xv = __ldg(xr + c);
    const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
    float xf[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xf[2 * i] = __uint_as_float(xw[i] << 16);
      xf[2 * i + 1] = __uint_as_float(xw[i] & 0xFFFF0000u);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (e0 + j < E) {
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + (int64_t)(e0 + j) * H) + c);
        const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[j] = fmaf(xf[2 * i], __uint_as_float(ww[i] << 16), acc[j]);
          acc[j] = fmaf(xf[2 * i + 1], __uint_as_float(ww[i] & 0xFFFF0000u), acc[j]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xFFFFFFFFu, acc[j], off);
    if (lane == 0 && e0 + j < E) logits[tok * E + e0 + j] = acc[j];
  }
}

int launch_route_topk(const float* logits, const float* bias, int64_t T, int E, int K, int32_t* ids, float* weights,
                      cudaStream_t st) {
  if (T == 0) return 0;
  const int64_t blocks = (T * 32 + 255) / 256;
  k_route_topk<<<(unsigned)blocks, 256, 0, st>>>(logits, bias, T, E, K, ids, weights);
  return (int)cudaGetLastError();
}

int launch_router_logits(const void* x, const void* w, int64_t T, int H, int E, float* logits, cudaStream_t st) {
  if (T == 0) return 0;
  dim3 grid((unsigned)T, (unsigned)((E + 63) / 64));
  k_router_logits<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, T, H, E, logits);
  return (int)cudaGetLastError();
}

}  // namespace b200
