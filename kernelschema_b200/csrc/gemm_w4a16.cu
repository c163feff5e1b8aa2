// Dense GEMM with bf16 activations and NVFP4 weights (W4A16): out = bf16(alpha * A @ decode(B)^T), the contract of
// gemm/dense/bf16_nvfp4_gemm/problem/reference.py:10-15 (A is NOT quantised; B payload [N, K/2] with row-major,
// un-swizzled E4M3 block-16 scales [N, K/16]).
//
// An E2M1 value times an E4M3 scale has at most 6 significant bits and lies in [2^-10, 2688], so it is exactly
// representable in fp16 and in bf16. The weights are therefore expanded to bf16 on the fly, bit-exactly, and the
// product runs on tcgen05.mma kind::f16 (bf16 x bf16, fp32 accumulation in TMEM): the result differs from the fp32
// reference only by the order of the fp32 additions.
//
// Tile: 256 rows of A (two 128-row accumulators) x 128 weight rows, K in steps of 64. One decoded weight tile feeds
// two MMAs, which halves the decoding work per flop; 2 x 2 accumulators of 128 columns fill the 512 TMEM columns, so
// the epilogue of one tile overlaps the k-loop of the next.
// Warp roles: 0 = TMA producer of A (bf16, 128-byte swizzle); 1 = TMEM owner + MMA issuer; 2-5 = weight decoders, one
// thread per weight row: it reads its row's 128-byte line (256 weights) and 16 scale bytes with plain loads, one k-group
// ahead, and writes bf16 into shared memory in the layout a 128-byte-swizzled TMA load would have produced (16-byte
// chunk c of row r at r * 128 + ((c ^ (r & 7)) * 16)), then fence.proxy.async + mbarrier arrive; 6-13 = epilogue.
// Every wait is bounded and reports through the status word.
#include "kernels.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

namespace b200 {

namespace {

constexpr int kWStages = 4;
constexpr int kWABytes = 256 * 128;      // 256 rows x 64 bf16
constexpr int kWBBytes = 128 * 128;      // 128 weight rows x 64 bf16
constexpr int kWSmem = kWStages * (kWABytes + kWBBytes) + 1024 + 256;
constexpr int kWThreads = 32 * 14;

struct W4A16Params {
  const uint8_t* b_q;      // [N, K/2]
  const uint8_t* b_sf;     // [N, K/16] E4M3, row-major
  const float* alpha;      // device scalar or null (= 1)
  __nv_bfloat16* out;
  int64_t out_stride;
  int M, N, K;
  int32_t* status;
};

DEV void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Four bytes of E2M1 pairs -> four fp16x2 words (exact); the low nibble of a byte lands in the low half.
DEV void e2m1x8_to_f16x2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// Two E4M3 bytes (low 16 bits of s) -> fp16x2 (exact).
DEV uint32_t e4m3x2_to_f16x2(uint32_t s) {
  uint32_t h;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h) : "r"(s & 0xFFFFu));
  return h;
}
// fp16x2 (values exactly representable in bf16) -> bf16x2.
DEV uint32_t f16x2_to_bf16x2(uint32_t h) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&b);
}

__global__ void __launch_bounds__(kWThreads, 1)
k_gemm_w4a16(const __grid_constant__ CUtensorMap tm_a, const W4A16Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = base, s_b = s_a + kWStages * kWABytes, s_bar = s_b + kWStages * kWBBytes;
  const uint32_t bar_full_a = s_bar;                       // [stages] TMA bytes of A landed
  const uint32_t bar_full_b = bar_full_a + 8 * kWStages;   // [stages] 4 decoder warps wrote their rows
  const uint32_t bar_empty = bar_full_b + 8 * kWStages;    // [stages] MMAs of the stage retired
  const uint32_t bar_acc_full = bar_empty + 8 * kWStages;  // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;        // [2] 8 epilogue warps
  const uint32_t s_slot = bar_acc_empty + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kWStages; ++s) {
      mbar_init(bar_full_a + 8 * s, 1);
      mbar_init(bar_full_b + 8 * s, 4);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 8);
    }
    mbar_init_fence();
    tma_prefetch_desc(&tm_a);
  }
  if (warp == 1) tmem_alloc<512>(s_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_slot));
  pdl_wait();

  const int n_mt = (p.M + 255) >> 8;        // 256-row tiles of A
  const int n_nt = p.N >> 7;                // 128-row tiles of the weights
  const int nk = p.K >> 6;                  // k-steps of 64
  const int total_items = n_mt * n_nt;      // n fastest: the CTAs of a wave share A's rows and sweep the weights (L2-resident)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer of A
    if (lane == 0) {
      uint32_t s = 0, ph = 1;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int mt = item / n_nt;
        for (int ks = 0; ks < nk; ++ks) {
          if (!mbar_wait(bar_empty + 8 * s, ph)) { if (p.status) atomicCAS(p.status, 0, 121); ok = false; break; }
          mbar_expect_tx(bar_full_a + 8 * s, kWABytes);
          tma_load_2d(s_a + s * kWABytes, &tm_a, bar_full_a + 8 * s, ks * 128, mt * 256);
          if (++s == kWStages) { s = 0; ph ^= 1; }
        }
      }
      pdl_trigger();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 128);
      uint32_t s = 0, ph = 0, it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
        const int mt = item / n_nt;
        const bool second = p.M - mt * 256 > 128;          // rows 128..255 of the tile hold real rows
        const uint32_t buf = it & 1;
        if (!mbar_wait(bar_acc_empty + 8 * buf, ((it >> 1) & 1) ^ 1)) { if (p.status) atomicCAS(p.status, 0, 122); break; }
        tc_fence_after();
        const uint32_t acc = tmem + buf * 256;
        for (int ks = 0; ks < nk; ++ks) {
          if (!mbar_wait(bar_full_a + 8 * s, ph) || !mbar_wait(bar_full_b + 8 * s, ph)) {
            if (p.status) atomicCAS(p.status, 0, 123);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_d = make_desc_sw128(s_a + s * kWABytes), b_d = make_desc_sw128(s_b + s * kWBBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            mma_bf16(acc, a_d + 2 * q, b_d + 2 * q, idesc, (ks | q) ? 1u : 0u);
            if (second) mma_bf16(acc + 128, a_d + (128 * 128 >> 4) + 2 * q, b_d + 2 * q, idesc, (ks | q) ? 1u : 0u);
          }
          mma_commit(bar_empty + 8 * s);
          if (++s == kWStages) { s = 0; ph ^= 1; }
        }
        if (ok) mma_commit(bar_acc_full + 8 * buf);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ weight decoders: thread = weight row of the tile
    const int r = threadIdx.x - 64;                         // 0..127
    const int groups = p.K >> 8;                            // k-groups of 256 weights = one 128-byte line per row
    const uint32_t row_off = (uint32_t)r * 128u;
    const uint32_t sw = (uint32_t)(r & 7);
    uint32_t s = 0, ph = 1;
    bool ok = true;
    uint4 nxt[8];
    uint4 nxt_sf;
    auto fetch = [&](int item, int g) {
      const int nt = item % n_nt;
      const size_t row = (size_t)nt * 128 + r;
      const uint4* q = reinterpret_cast<const uint4*>(p.b_q + row * (size_t)(p.K >> 1)) + (size_t)g * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) nxt[i] = __ldg(q + i);
      nxt_sf = __ldg(reinterpret_cast<const uint4*>(p.b_sf + row * (size_t)(p.K >> 4)) + g);
    };
    if ((int)blockIdx.x < total_items) fetch(blockIdx.x, 0);
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      for (int g = 0; ok && g < groups; ++g) {
        uint32_t cur[32];
        uint32_t cur_sf[4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          cur[4 * i] = nxt[i].x; cur[4 * i + 1] = nxt[i].y; cur[4 * i + 2] = nxt[i].z; cur[4 * i + 3] = nxt[i].w;
        }
        cur_sf[0] = nxt_sf.x; cur_sf[1] = nxt_sf.y; cur_sf[2] = nxt_sf.z; cur_sf[3] = nxt_sf.w;
        // next line: the following k-group of this item, or the first of this CTA's next item
        if (g + 1 < groups) fetch(item, g + 1);
        else if (item + (int)gridDim.x < total_items) fetch(item + gridDim.x, 0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {                       // the four 64-wide k-steps of the group
          int okw = 1;
          if (lane == 0) okw = mbar_wait(bar_empty + 8 * s, ph) ? 1 : 0;
          okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
          if (!okw) { if (lane == 0 && p.status) atomicCAS(p.status, 0, 125); ok = false; break; }
          const uint32_t dst = s_b + s * kWBBytes + row_off;
          const uint32_t sc01 = e4m3x2_to_f16x2(cur_sf[q]), sc23 = e4m3x2_to_f16x2(cur_sf[q] >> 16);
#pragma unroll
          for (int c = 0; c < 8; ++c) {                     // 16-byte chunk = 8 weights = one payload word
            const uint32_t sc_pair = (c & 4) ? sc23 : sc01;
            const uint32_t sc = (c & 2) ? __byte_perm(sc_pair, 0, 0x3232) : __byte_perm(sc_pair, 0, 0x1010);
            uint32_t h[4], o[4];
            e2m1x8_to_f16x2(cur[8 * q + c], h);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __half2 prod = __hmul2(*reinterpret_cast<const __half2*>(&h[i]), *reinterpret_cast<const __half2*>(&sc));
              o[i] = f16x2_to_bf16x2(*reinterpret_cast<const uint32_t*>(&prod));
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (((uint32_t)c ^ sw) << 4)), "r"(o[0]), "r"(o[1]),
                         "r"(o[2]), "r"(o[3])
                         : "memory");
          }
          fence_async_proxy();                              // generic-proxy writes -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full_b + 8 * s);
          if (++s == kWStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 8 warps = 2 accumulators x 4 lane quadrants
    const int quad = warp & 3;
    const int half = (warp - 6) >> 2;
    const float alpha = p.alpha ? *p.alpha : 1.0f;
    uint32_t it = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
      const int mt = item / n_nt, nt = item % n_nt;
      const uint32_t buf = it & 1;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(bar_acc_full + 8 * buf, (it >> 1) & 1) ? 1 : 0;
      okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
      if (!okw) { if (lane == 0 && p.status) atomicCAS(p.status, 0, 124); break; }
      tc_fence_after();
      const int row = mt * 256 + half * 128 + quad * 32 + lane;
      const bool live = row < p.M;
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + buf * 256 + half * 128;
      if (__any_sync(0xFFFFFFFFu, live)) {
        __nv_bfloat16* dst_row = p.out + (size_t)row * p.out_stride + nt * 128;
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          float v[2][32];
          tmem_ld32(taddr + pass * 64, v[0]);
          tmem_ld32(taddr + pass * 64 + 32, v[1]);
          tmem_ld_wait();
          if (pass == 1) {                                  // last read of this accumulator: hand it back before the stores
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
          }
          if (live) {
#pragma unroll
            for (int cb = 0; cb < 2; ++cb) {
              uint32_t o[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const __nv_bfloat162 pr = __floats2bfloat162_rn(v[cb][2 * j] * alpha, v[cb][2 * j + 1] * alpha);
                o[j] = *reinterpret_cast<const uint32_t*>(&pr);
              }
              __nv_bfloat16* d = dst_row + pass * 64 + cb * 32;
#pragma unroll
              for (int j = 0; j < 2; ++j)
                asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(d + 16 * j), "r"(o[8 * j]),
                             "r"(o[8 * j + 1]), "r"(o[8 * j + 2]), "r"(o[8 * j + 3]), "r"(o[8 * j + 4]), "r"(o[8 * j + 5]),
                             "r"(o[8 * j + 6]), "r"(o[8 * j + 7])
                             : "memory");
            }
          }
        }
      } else {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<512>(tmem);
  }
}

}  // namespace

int launch_gemm_w4a16(const void* a, int64_t a_stride, const void* b_q, const void* b_sf, const float* alpha, int64_t m, int64_t n,
                      int64_t k, void* out, int64_t out_stride, int32_t* status, cudaStream_t st) {
  if (m == 0) return 0;
  CUtensorMap ta;
  int rc = make_operand_map(&ta, a, (uint64_t)m, (uint64_t)k * 2, 256, (uint64_t)a_stride * 2);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_w4a16, cudaFuncAttributeMaxDynamicSharedMemorySize, kWSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  W4A16Params p;
  p.b_q = (const uint8_t*)b_q;
  p.b_sf = (const uint8_t*)b_sf;
  p.alpha = alpha;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.M = (int)m;
  p.N = (int)n;
  p.K = (int)k;
  p.status = status;
  const int64_t items = ((m + 255) / 256) * (n / 128);
  return (int)launch_chain(k_gemm_w4a16, dim3((unsigned)(items < sms ? items : sms)), dim3(kWThreads), kWSmem, st, ta, p);
}

}  // namespace b200
