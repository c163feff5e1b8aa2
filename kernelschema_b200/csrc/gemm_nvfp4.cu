// Persistent grouped NVFP4 x NVFP4 GEMM for sm_100a: TMA-staged packed-FP4 tiles and 128x4-tiled E4M3 scale
// factors feed tcgen05.mma kind::mxf4nvf4 (block-scaled, fp32 accumulators in TMEM).
//
// It replaces, on the reference's hot path, FC1 + activation + NVFP4 requantise and FC2
// (moe/nvfp4_fused_moe/problem/reference.py:80-91; candidate kernels k_gemm_f4_ws2 / k_gemm_f4_ws2d,
// candidate/nvfp4_moe.cu:5378-5434) and the dense contract of
// gemm/dense/bf16_nvfp4_gemm/problem/reference.py:10-15 with a quantised A operand.
//
// Work item = (m-tile of 128 permuted rows, n-tile of BN weight rows). The weight operand is consumed in the
// frozen layout the reference publishes (input.py:82-99): rows 32-shuffled and, for FC1, up/gate interleaved,
// scales tiled 128x4. Because payload rows and scale rows share one row map, the MMA runs directly on the
// stored rows; only the epilogue has to know which logical channel an accumulator column is:
//   FC1: inside a 32-column block, column 16c+b is "up" and column 16c+8+b is "gate" of channel 2b+c, so one
//        32-column block is exactly one 16-channel NVFP4 block of the intermediate activation;
//   FC2: column 8a+b is output channel 4b+a.
//
// Warp roles (192 threads, one CTA per SM): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (TMEM lane quadrant = warp & 3). Stage = 256 FP4 of K: A 16 KB, B BN*128 B,
// scale factors 2 KB per 128 rows. Accumulators are double buffered when BN = 128.
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kGemmThreads = 192;
constexpr int kBM = 128;
constexpr int kStageK = 256;             // FP4 elements of K per pipeline stage (128 payload bytes per row)
constexpr int kSfChunk = 512;            // bytes of one (128 rows x 64 K) scale-factor chunk
constexpr int kNumSfBuf = 4;             // TMEM scale-factor buffers in rotation

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 128) ? 6 : 4;
  static constexpr int kAccBufs = (BN == 128) ? 2 : 1;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = BN * 128;
  static constexpr int kSfaBytes = 4 * kSfChunk;
  static constexpr int kSfbBytes = (BN / 128) * 4 * kSfChunk;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSfCols = 16 + 16 * (BN / 128);          // TMEM columns of one scale-factor buffer
  static constexpr int kSfBase = kAccBufs * BN;                  // first scale-factor column
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(kSfBase + kNumSfBuf * kSfCols <= 512, "TMEM budget");
};

DEV void report(int32_t* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

DEV float sigmoid_fast(float x) { return __frcp_rn(1.0f + __expf(-x)); }
DEV float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int MODE, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
k_gemm_nvfp4(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
  using C = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = smem_base;
  const uint32_t s_b = s_a + C::kStages * C::kABytes;
  const uint32_t s_sfa = s_b + C::kStages * C::kBBytes;
  const uint32_t s_sfb = s_sfa + C::kStages * C::kSfaBytes;
  const uint32_t s_bar = s_sfb + C::kStages * C::kSfbBytes;
  const uint32_t bar_full = s_bar;                         // [kStages]
  const uint32_t bar_empty = bar_full + 8 * C::kStages;    // [kStages]
  const uint32_t bar_acc_full = bar_empty + 8 * C::kStages;     // [kAccBufs]
  const uint32_t bar_acc_empty = bar_acc_full + 8 * C::kAccBufs;
  const uint32_t s_tmem_slot = bar_acc_empty + 8 * C::kAccBufs;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < C::kAccBufs; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    mbar_init_fence();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) tmem_alloc<512>(s_tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_tmem_slot));

  const int n_mtiles = p.n_tiles_ptr ? *p.n_tiles_ptr : p.n_tiles_static;
  const int n_ntiles = p.N / BN;
  const int nk = p.K / kStageK;
  const long long total_items = (long long)n_mtiles * n_ntiles;
  const int chunks_per_row = p.K >> 6;     // scale-factor chunks along K

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t g = 0;
      bool ok = true;
      for (long long item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int mt = (int)(item / n_ntiles), nt = (int)(item % n_ntiles);
        const int e = p.tile_expert ? p.tile_expert[mt] : 0;
        const int row0 = p.tile_row0 ? p.tile_row0[mt] : mt * kBM;
        const int brow0 = e * p.N + nt * BN;
        const uint8_t* sfa_src = p.sfa + (size_t)(row0 >> 7) * chunks_per_row * kSfChunk;
        const uint8_t* sfb_src = p.sfb + (size_t)(brow0 >> 7) * chunks_per_row * kSfChunk;
        for (int ks = 0; ks < nk; ++ks, ++g) {
          const uint32_t s = g % C::kStages;
          if (!mbar_wait(bar_empty + 8 * s, ((g / C::kStages) & 1) ^ 1)) { report(p.status, 101); ok = false; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, C::kStageBytes);
          tma_load_2d(s_a + s * C::kABytes, &tm_a, full, ks * 128, row0);
          tma_load_2d(s_b + s * C::kBBytes, &tm_b, full, ks * 128, brow0);
          bulk_load_1d(s_sfa + s * C::kSfaBytes, sfa_src + (size_t)ks * 4 * kSfChunk, 4 * kSfChunk, full);
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
            bulk_load_1d(s_sfb + s * C::kSfbBytes + h * 4 * kSfChunk,
                         sfb_src + ((size_t)h * chunks_per_row + (size_t)ks * 4) * kSfChunk, 4 * kSfChunk, full);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_nvf4(kBM, BN);
      uint32_t g = 0, it = 0;
      bool ok = true;
      for (long long item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
        const uint32_t buf = it % C::kAccBufs;
        if (!mbar_wait(bar_acc_empty + 8 * buf, ((it / C::kAccBufs) & 1) ^ 1)) { report(p.status, 102); break; }
        tc_fence_after();
        const uint32_t acc = tmem + buf * BN;
        for (int ks = 0; ks < nk; ++ks, ++g) {
          const uint32_t s = g % C::kStages;
          if (!mbar_wait(bar_full + 8 * s, (g / C::kStages) & 1)) { report(p.status, 103); ok = false; break; }
          tc_fence_after();
          const uint32_t sf_t = tmem + C::kSfBase + (g % kNumSfBuf) * C::kSfCols;
          const uint32_t sfa_t = sf_t, sfb_t = sf_t + 16;
          const uint32_t sfa_s = s_sfa + s * C::kSfaBytes, sfb_s = s_sfb + s * C::kSfbBytes;
#pragma unroll
          for (int q = 0; q < 4; ++q) tmem_cp_sf(sfa_t + 4 * q, make_desc_sf(sfa_s + q * kSfChunk));
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
#pragma unroll
            for (int q = 0; q < 4; ++q)
              tmem_cp_sf(sfb_t + (BN / 128) * 4 * q + 4 * h, make_desc_sf(sfb_s + (h * 4 + q) * kSfChunk));
          const uint64_t a_d = make_desc_sw128(s_a + s * C::kABytes);
          const uint64_t b_d = make_desc_sw128(s_b + s * C::kBBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            mma_nvf4(acc, a_d + 2 * q, b_d + 2 * q, idesc, sfa_t + 4 * q, sfb_t + (BN / 128) * 4 * q, (ks | q) ? 1u : 0u);
          mma_commit(bar_empty + 8 * s);
        }
        if (ok) mma_commit(bar_acc_full + 8 * buf);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps, one TMEM lane quadrant each)
    const int quad = warp & 3;
    const int r_in_tile = quad * 32 + lane;
    uint32_t it = 0;
    for (long long item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
      const int mt = (int)(item / n_ntiles), nt = (int)(item % n_ntiles);
      const int e = p.tile_expert ? p.tile_expert[mt] : 0;
      const int row0 = p.tile_row0 ? p.tile_row0[mt] : mt * kBM;
      const int rows = p.tile_rows ? p.tile_rows[mt] : min(kBM, p.M - row0);
      const uint32_t buf = it % C::kAccBufs;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(bar_acc_full + 8 * buf, (it / C::kAccBufs) & 1) ? 1 : 0;
      okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
      if (!okw) { if (lane == 0) report(p.status, 104); break; }
      tc_fence_after();
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + buf * BN;
      const bool live = r_in_tile < rows;
      const size_t row = (size_t)row0 + r_in_tile;

      if (MODE == kGemmFc1) {
        const float s_up = p.scale_up ? p.scale_up[e] : 1.0f;
        const float s_gate = p.scale_gate ? p.scale_gate[e] : 1.0f;
        const float alpha = p.alpha ? p.alpha[e] : 1.0f;
        const float beta = p.beta ? p.beta[e] : 0.0f;
        const bool clamp = p.limit != nullptr;
        const float limit = clamp ? p.limit[e] : 0.f;
        const int half_i = p.N >> 2;                       // bytes of one row of packed activations (I / 2)
        uint2 packed[BN / 32];
        uint32_t sfbytes = 0;
        uint32_t sfword[BN / 128];
#pragma unroll
        for (int cb = 0; cb < BN / 32; ++cb) {
          float v[32];
          tmem_ld32(taddr + cb * 32, v);
          tmem_ld_wait();
          float act[16];
          float amax = 0.f;
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int b = 0; b < 8; ++b) {
              float up = v[16 * c + b] * s_up;
              float gate = v[16 * c + 8 + b] * s_gate;
              if (clamp) {
                up = fminf(fmaxf(up, -limit), limit);
                gate = fminf(gate, limit);
              }
              float a;
              if (p.act_type == 10)
                a = alpha * tanh_fast(__fdividef(gate, alpha)) * sigmoid_fast(gate) * (beta * tanh_fast(__fdividef(up, beta)));
              else
                a = gate * sigmoid_fast(alpha * gate) * (up + beta);
              act[2 * b + c] = a;
              amax = fmaxf(amax, fabsf(a));
            }
          // reference.py:40-42: sf = e4m3(clamp(amax * (1/6), 0, 448)); zero scale -> zero block
          const float sfv = fminf(amax * (1.0f / 6.0f), 448.0f);
          const uint32_t sb = cvt_e4m3(sfv);
          const float sff = e4m3_to_f32(sb);
          const float inv = sff > 0.f ? __frcp_rn(sff) : 0.f;
          uint32_t w0 = 0, w1 = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            w0 |= cvt_e2m1x2(act[2 * j] * inv, act[2 * j + 1] * inv) << (8 * j);
            w1 |= cvt_e2m1x2(act[8 + 2 * j] * inv, act[8 + 2 * j + 1] * inv) << (8 * j);
          }
          packed[cb] = make_uint2(w0, w1);
          sfbytes |= sb << (8 * (cb & 3));
          if ((cb & 3) == 3) { sfword[cb >> 2] = sfbytes; sfbytes = 0; }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
        if (live) {
          const int i0 = (nt * BN) >> 1;                   // first intermediate channel of this tile
          uint4* dst = reinterpret_cast<uint4*>(p.act_q + row * half_i + (i0 >> 1));
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            dst[j] = make_uint4(packed[2 * j].x, packed[2 * j].y, packed[2 * j + 1].x, packed[2 * j + 1].y);
          // scale bytes of 64 channels = one 4-byte word of the 128x4-tiled layout [row/128][I/64][32][16]
          const int chunks_i = p.N >> 7;                   // I / 64
#pragma unroll
          for (int j = 0; j < BN / 128; ++j) {
            const size_t off = ((row >> 7) * chunks_i + (size_t)((i0 >> 6) + j)) * kSfChunk + (row & 31) * 16 + ((row >> 5) & 3) * 4;
            *reinterpret_cast<uint32_t*>(p.act_sf + off) = sfword[j];
          }
        }
      } else {
        const float oscale = (MODE == kGemmFc2) ? (p.out_scale ? p.out_scale[e] : 1.0f) : p.dense_alpha;
        __nv_bfloat16* dst_row = p.out + row * p.out_stride + (size_t)nt * BN;
#pragma unroll
        for (int cb = 0; cb < BN / 32; ++cb) {
          float v[32];
          tmem_ld32(taddr + cb * 32, v);
          tmem_ld_wait();
          if (cb == BN / 32 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
          }
          if (live) {
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float x0, x1;
              if (MODE == kGemmFc2) {           // output channel 4b+a lives in column 8a+b
                const int h0 = 2 * j, h1 = 2 * j + 1;
                x0 = v[8 * (h0 & 3) + (h0 >> 2)];
                x1 = v[8 * (h1 & 3) + (h1 >> 2)];
              } else {
                x0 = v[2 * j];
                x1 = v[2 * j + 1];
              }
              const __nv_bfloat162 pr = __floats2bfloat162_rn(x0 * oscale, x1 * oscale);
              o[j] = *reinterpret_cast<const uint32_t*>(&pr);
            }
            uint4* d4 = reinterpret_cast<uint4*>(dst_row + cb * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) d4[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
          }
        }
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

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// 2-D byte tensor [rows, row_bytes] -> boxes of 128 bytes x box_rows rows, 128-byte swizzle.
int make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 701;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700 + (int)r;
}

template <int MODE, int BN>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  auto kern = k_gemm_nvfp4<MODE, BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kGemmThreads, GemmCfg<BN>::kSmemBytes, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

int launch_gemm_nvfp4(int mode, int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                      cudaStream_t st) {
  if (grid <= 0) return 0;
  if (p.K % kStageK != 0 || p.N % bn != 0) return 702;
  if (bn == 128) {
    if (mode == kGemmFc1) return launch_one<kGemmFc1, 128>(ta, tb, p, grid, st);
    if (mode == kGemmFc2) return launch_one<kGemmFc2, 128>(ta, tb, p, grid, st);
    return launch_one<kGemmDense, 128>(ta, tb, p, grid, st);
  }
  if (bn == 256) {
    if (mode == kGemmFc1) return launch_one<kGemmFc1, 256>(ta, tb, p, grid, st);
    if (mode == kGemmFc2) return launch_one<kGemmFc2, 256>(ta, tb, p, grid, st);
    return launch_one<kGemmDense, 256>(ta, tb, p, grid, st);
  }
  return 703;
}

}  // namespace b200
