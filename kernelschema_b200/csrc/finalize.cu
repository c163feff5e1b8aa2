// Routing-weighted combine: out[t, h] = bf16( sum_k fp32(rout[row_of[t, k], h]) * weight[t, k] ), slots in
// ascending k, tokens without any valid route produce zeros, every output element is written.
// Follows reference.py:91-92 of moe/nvfp4_fused_moe/problem (per-route bf16 rounding happens before the
// weight, the sum is fp32, one final bf16 rounding); same role as the candidate's k_finalize
// (candidate/nvfp4_moe.cu:1464). HBM-bound: reads K rows of H bf16 per token, writes one.
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

__global__ void __launch_bounds__(128) k_finalize(const __nv_bfloat16* __restrict__ rout, const int32_t* __restrict__ row_of,
                                                  const float* __restrict__ weight_of_row, int64_t T, int KK, int H,
                                                  __nv_bfloat16* __restrict__ out, int64_t out_stride) {
  const int vecs = H >> 3;
  pdl_trigger();
  pdl_wait();
  for (int64_t t = blockIdx.x; t < T; t += gridDim.x) {
    for (int v = blockIdx.y * blockDim.x + threadIdx.x; v < vecs; v += gridDim.y * blockDim.x) {
      float acc[8];
      combine_slots(rout, row_of + t * KK, weight_of_row, KK, H, v, acc);
      *(reinterpret_cast<uint4*>(out + t * out_stride) + v) = pack_bf16x8(acc);
    }
  }
}

int launch_finalize(const void* rout, const int32_t* row_of, const float* weight_of_row, int64_t T, int KK, int H, void* out,
                    int64_t out_stride, cudaStream_t st) {
  if (T == 0) return 0;
  const int sms = sm_count();
  const int64_t blocks = T < sms * 16 ? T : sms * 16;
  // few tokens: spread each token's row over several blocks so that the whole GPU pulls on HBM
  const int chunks = (H / 8 + 127) / 128;
  const int by = blocks >= sms * 4 ? 1 : (int)(chunks < (sms * 4 + blocks - 1) / blocks ? chunks : (sms * 4 + blocks - 1) / blocks);
  return (int)launch_chain(k_finalize, dim3((unsigned)blocks, (unsigned)by), dim3(128), 0, st, (const __nv_bfloat16*)rout, row_of,
                           weight_of_row, T, KK, H, (__nv_bfloat16*)out, out_stride);
}

}  // namespace b200
