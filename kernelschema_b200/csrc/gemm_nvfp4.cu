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
// One CTA per SM, warp-specialised: TMA producer, MMA issuer, scale-factor copiers, epilogue warps (roles are listed
// at each kernel). Stage = 256 FP4 of K: A 16 KB, B BN*128 B, scale factors 2 KB per 128 rows.
//
// What bounds the mainloop is the rate at which ONE thread can issue tcgen05 instructions: about 48 cycles per
// instruction (tcgen05.cp, tcgen05.mma and tcgen05.commit alike), measured on B200 with an issue-only loop. A 128 x 256
// stage needs 12 scale-factor copies + 4 MMAs (512 tensor cycles): 16 x 48 = 770 cycles from one thread, 12 x 48 + a
// wait + a commit = 880 from one copier thread beside an MMA thread. Different warps issue concurrently, so the copies
// are split over kCopiers warps (6 each for BN = 256): every issuing thread stays below the 512 cycles of its stage.
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kBM = 128;
constexpr int kStageK = 256;             // FP4 elements of K per pipeline stage (128 payload bytes per row)
constexpr int kSfChunk = 512;            // bytes of one (128 rows x 64 K) scale-factor chunk
constexpr int kCopiers = 2;              // warps that issue the scale-factor copies of a stage, round-robin (a third would make
                                         // 13 or 21 warps: one more warp on an SM sub-partition costs the epilogue its registers)

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
  // one TMEM scale-factor buffer per pipeline stage: a copier can run as far ahead of the MMA thread as the stage ring lets it
  static_assert(kSfBase + kStages * kSfCols <= 512, "TMEM budget");
  static constexpr int kSfCopies = 4 + 4 * (BN / 128);           // tcgen05.cp per stage
};

// Cycle accounting of the MMA thread (where it waits), compiled only into experiment builds (-DB200MOE_PROBE).
#ifdef B200MOE_PROBE
__device__ long long g_probe[1024 * 4];
#define PROBE_DECL long long pr_acc = 0, pr_sf = 0, pr_c = 0; const long long pr_t0 = clock64();
#define PROBE_T(var) const long long var = clock64();
#define PROBE_ADD(acc, t0) acc += clock64() - (t0);
#define PROBE_STORE if (blockIdx.x < 1024) { g_probe[blockIdx.x * 4] = clock64() - pr_t0; g_probe[blockIdx.x * 4 + 1] = pr_acc; g_probe[blockIdx.x * 4 + 2] = pr_sf; g_probe[blockIdx.x * 4 + 3] = pr_c; }
#else
#define PROBE_DECL
#define PROBE_T(var)
#define PROBE_ADD(acc, t0)
#define PROBE_STORE
#endif

DEV void report(int32_t* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

DEV float sigmoid_fast(float x) { return __frcp_rn(1.0f + __expf(-x)); }
DEV float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Epilogue of EC (64 or 128) accumulator columns [col0, col0 + EC) of one tile for the calling warp's 32 TMEM lanes.
// The values are pulled into registers first and `release` is called right after the last TMEM read, so the
// accumulator buffer is free again after a few hundred cycles and the arithmetic, the requantisation and the global
// stores overlap the next tile's mainloop. EC = 64 (16 epilogue warps on a 256-column tile) keeps four warps on every
// scheduler: the activation + requantisation chain is latency-bound with two, which shows when the k-loop of a tile is
// short (K <= 2048: 8 stages, about 4 us); with a long k-loop the eight-warp form (EC = 128) hides it and draws less power.
template <int MODE, int EC, class Release>
DEV void epilogue_cols(const GemmParams& p, uint32_t taddr, int e, size_t row, bool live, int col0, Release release) {
  constexpr int NCB = EC / 32;
  // a warp whose 32 rows are all padding (decode: a few routes per expert) neither reads the accumulator nor computes
  if (!__any_sync(0xFFFFFFFFu, live)) {
    release();
    return;
  }
  float v[NCB][32];
#pragma unroll
  for (int cb = 0; cb < NCB; ++cb) tmem_ld32(taddr + cb * 32, v[cb]);
  tmem_ld_wait();
  release();
  if (MODE == kGemmFc1) {
    const float s_up = p.scale_up ? p.scale_up[e] : 1.0f;
    const float s_gate = p.scale_gate ? p.scale_gate[e] : 1.0f;
    const float alpha = p.alpha ? p.alpha[e] : 1.0f;
    const float beta = p.beta ? p.beta[e] : 0.0f;
    const bool clamp = p.limit != nullptr;
    const float limit = clamp ? p.limit[e] : 0.f;
    uint2 packed[NCB];
    uint32_t sfword = 0;
#pragma unroll
    for (int cb = 0; cb < NCB; ++cb) {
      float act[16];
      float amax = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          float up = v[cb][16 * c + b] * s_up;
          float gate = v[cb][16 * c + 8 + b] * s_gate;
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
      sfword |= sb << (8 * cb);
    }
    if (live) {
      const int half_i = p.N >> 2;                     // bytes of one row of packed activations (I / 2)
      const int i0 = col0 >> 1;                        // first intermediate channel of these columns (multiple of EC / 2)
      // scale bytes of 64 channels = one 4-byte word of the 128x4-tiled layout [row/128][I/64][32][16]
      const size_t off = ((row >> 7) * (size_t)(p.N >> 7) + (size_t)(i0 >> 6)) * kSfChunk + (row & 31) * 16 + ((row >> 5) & 3) * 4;
      if constexpr (NCB == 4) {
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p.act_q + row * half_i + (i0 >> 1)), "r"(packed[0].x),
                     "r"(packed[0].y), "r"(packed[1].x), "r"(packed[1].y), "r"(packed[2].x), "r"(packed[2].y), "r"(packed[3].x),
                     "r"(packed[3].y)
                     : "memory");
        *reinterpret_cast<uint32_t*>(p.act_sf + off) = sfword;
      } else {
        asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p.act_q + row * half_i + (i0 >> 1)), "r"(packed[0].x),
                     "r"(packed[0].y), "r"(packed[1].x), "r"(packed[1].y)
                     : "memory");
        *reinterpret_cast<uint16_t*>(p.act_sf + off + ((i0 >> 5) & 1) * 2) = (uint16_t)sfword;
      }
    }
  } else {
    if (!live) return;
    const float oscale = (MODE == kGemmFc2) ? (p.out_scale ? p.out_scale[e] : 1.0f) : p.dense_alpha;
    const size_t orow = (MODE == kGemmFc2 && p.out_row_index) ? (size_t)p.out_row_index[row] : row;
    __nv_bfloat16* dst_row = p.out + orow * p.out_stride + col0;
#pragma unroll
    for (int cb = 0; cb < NCB; ++cb) {
      uint32_t o[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x0, x1;
        if (MODE == kGemmFc2) {           // output channel 4b+a lives in column 8a+b
          const int h0 = 2 * j, h1 = 2 * j + 1;
          x0 = v[cb][8 * (h0 & 3) + (h0 >> 2)];
          x1 = v[cb][8 * (h1 & 3) + (h1 >> 2)];
        } else {
          x0 = v[cb][2 * j];
          x1 = v[cb][2 * j + 1];
        }
        const __nv_bfloat162 pr = __floats2bfloat162_rn(x0 * oscale, x1 * oscale);
        o[j] = *reinterpret_cast<const uint32_t*>(&pr);
      }
      // 256-bit stores: one full 32-byte sector per thread and instruction
      __nv_bfloat16* d = dst_row + cb * 32;
#pragma unroll
      for (int j = 0; j < 2; ++j)
        asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(d + 16 * j), "r"(o[8 * j]), "r"(o[8 * j + 1]),
                     "r"(o[8 * j + 2]), "r"(o[8 * j + 3]), "r"(o[8 * j + 4]), "r"(o[8 * j + 5]), "r"(o[8 * j + 6]), "r"(o[8 * j + 7])
                     : "memory");
    }
  }
}

// Warp roles: 0 = TMA producer, 1 = TMEM owner + MMA issuer, 2 .. 1 + kCopiers = scale-factor copiers (shared memory ->
// TMEM), then 4 * BN/EC epilogue warps; epilogue warp w owns TMEM lane quadrant w & 3 and the EC-column group
// (w - kFirstEpiWarp) / 4.
constexpr int kFirstEpiWarp = 2 + kCopiers;
// any four consecutive warps own the four TMEM lane quadrants (quadrant = warp & 3), so the epilogue groups may start anywhere
template <int BN, int EC>
constexpr int gemm_threads() { return 32 * (kFirstEpiWarp + 4 * BN / EC); }

// Scale-factor copy j of a stage (j < 4: A scales of k-block j; then B scales, 128-row half h, k-block q) from the
// stage's shared-memory slots into its TMEM buffer.
template <int BN>
DEV void sf_copy(int j, uint32_t sf_t, uint32_t sfa_lo, uint32_t sfb_lo) {
  constexpr uint32_t kHiSf = (128u >> 4) | (1u << 14);                 // SBO 128, descriptor version 1, no swizzle
  if (j < 4) {
    tmem_cp_sf(sf_t + 4 * j, ((uint64_t)kHiSf << 32) | (sfa_lo + j * (kSfChunk >> 4)));
  } else {
    const int h = (j - 4) >> 2, q = (j - 4) & 3;
    tmem_cp_sf(sf_t + 16 + (BN / 128) * 4 * q + 4 * h, ((uint64_t)kHiSf << 32) | (sfb_lo + (h * 4 + q) * (kSfChunk >> 4)));
  }
}

// The scale-factor copies of copier warp C: copies C, C + kCopiers, C + 2 * kCopiers, ... of every stage.
template <int BN, int C>
DEV void copier_loop(const GemmParams& p, uint32_t tmem, uint32_t s_sfa, uint32_t s_sfb, uint32_t bar_full, uint32_t bar_sf,
                     long long total_items, int nk) {
  using Cfg = GemmCfg<BN>;
  const uint32_t sfa_lo0 = (s_sfa >> 4) & 0x3FFF, sfb_lo0 = (s_sfb >> 4) & 0x3FFF;
  uint32_t s = 0, ph = 0;
  for (long long item = blockIdx.x; item < total_items; item += gridDim.x) {
    for (int ks = 0; ks < nk; ++ks) {
      if (!mbar_wait(bar_full + 8 * s, ph)) { report(p.status, 105); return; }
      tc_fence_after();
      const uint32_t sf_t = tmem + Cfg::kSfBase + s * Cfg::kSfCols;
      const uint32_t sfa_lo = sfa_lo0 + s * (Cfg::kSfaBytes >> 4), sfb_lo = sfb_lo0 + s * (Cfg::kSfbBytes >> 4);
#pragma unroll
      for (int j = C; j < Cfg::kSfCopies; j += kCopiers) sf_copy<BN>(j, sf_t, sfa_lo, sfb_lo);
      mma_commit(bar_sf + 8 * s);                      // arrives once this thread's copies have landed
      if (++s == Cfg::kStages) { s = 0; ph ^= 1; }
    }
  }
}

template <int MODE, int BN, int EC>
__global__ void __launch_bounds__(gemm_threads<BN, EC>(), 1)
k_gemm_nvfp4(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
  using C = GemmCfg<BN>;
  constexpr int kEpiWarps = 4 * BN / EC;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = smem_base;
  const uint32_t s_b = s_a + C::kStages * C::kABytes;
  const uint32_t s_sfa = s_b + C::kStages * C::kBBytes;
  const uint32_t s_sfb = s_sfa + C::kStages * C::kSfaBytes;
  const uint32_t s_bar = s_sfb + C::kStages * C::kSfbBytes;
  const uint32_t bar_full = s_bar;                              // [kStages] TMA bytes landed
  const uint32_t bar_sf = bar_full + 8 * C::kStages;            // [kStages] scale factors of the stage are in TMEM (all copiers)
  const uint32_t bar_empty = bar_sf + 8 * C::kStages;           // [kStages] MMAs of the stage retired
  const uint32_t bar_acc_full = bar_empty + 8 * C::kStages;     // [kAccBufs]
  const uint32_t bar_acc_empty = bar_acc_full + 8 * C::kAccBufs;
  const uint32_t s_tmem_slot = bar_acc_empty + 8 * C::kAccBufs;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_sf + 8 * s, kCopiers);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < C::kAccBufs; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, kEpiWarps);
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
  // everything above touches no global memory: it overlaps the previous kernel of the stream
  pdl_wait();

  const int n_mtiles = p.n_tiles_ptr ? *p.n_tiles_ptr : p.n_tiles_static;
  const int n_ntiles = p.N / BN;
  const int nk = p.K / kStageK;
  const long long total_items = (long long)n_mtiles * n_ntiles;
  const int chunks_per_row = p.K >> 6;     // scale-factor chunks along K

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (MODE == kGemmFc1 && p.a_tok) {
      // A rows straight from the token matrix: lane l owns rows 4l .. 4l+3 of the tile and fetches them with one
      // tile::gather4 per stage (four token rows x 128 bytes into 512 bytes of the swizzled A slot). Only the boxes that
      // hold a valid row are issued (rows past the tile's count keep whatever the slot held: their results are never
      // stored), and the stage's expected byte count follows the box count.
      uint32_t s = 0, ph = 1;
      bool ok = true;
      int mt_n = 0, e_n = 0, row0_n = 0, rows_n = 0;
      int4 tok_n = make_int4(0, 0, 0, 0);
      auto fetch = [&](long long item) {
        mt_n = (int)(item / n_ntiles);
        e_n = p.tile_expert[mt_n];
        row0_n = p.tile_row0[mt_n];
        rows_n = p.tile_rows[mt_n];
        tok_n = *reinterpret_cast<const int4*>(p.a_tok + row0_n + 4 * lane);
      };
      if (blockIdx.x < total_items) fetch(blockIdx.x);
      for (long long item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int nt = (int)(item - (long long)mt_n * n_ntiles);
        const int e = e_n, row0 = row0_n, rows = rows_n;
        int4 tok = tok_n;
        if (item + gridDim.x < total_items) fetch(item + gridDim.x);
        const int nbox = max(1, min(kBM / 4, (rows + 3) >> 2));
        // rows of a box past the tile's count repeat the box's first row (entries of padding rows are unspecified)
        if (4 * lane + 1 >= rows) tok.y = tok.x;
        if (4 * lane + 2 >= rows) tok.z = tok.x;
        if (4 * lane + 3 >= rows) tok.w = tok.x;
        if (4 * lane >= rows) tok = make_int4(0, 0, 0, 0);
        const int brow0 = e * p.N + nt * BN;
        const uint8_t* sfa_src = p.sfa + (size_t)(row0 >> 7) * chunks_per_row * kSfChunk;
        const uint8_t* sfb_src = p.sfb + (size_t)(brow0 >> 7) * chunks_per_row * kSfChunk;
        const uint32_t stage_bytes = C::kStageBytes - C::kABytes + (uint32_t)nbox * 512u;
        for (int ks = 0; ks < nk; ++ks) {
          if (lane == 0 && !mbar_wait(bar_empty + 8 * s, ph)) { report(p.status, 101); ok = false; }
          ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * s;
          if (lane == 0) mbar_expect_tx(full, stage_bytes);
          __syncwarp();
          if (lane < nbox) tma_gather4(s_a + s * C::kABytes + 512u * lane, &tm_a, full, ks * 128, tok.x, tok.y, tok.z, tok.w);
          if (lane == 0) {
            tma_load_2d(s_b + s * C::kBBytes, &tm_b, full, ks * 128, brow0);
            bulk_load_1d(s_sfa + s * C::kSfaBytes, sfa_src + (size_t)ks * 4 * kSfChunk, 4 * kSfChunk, full);
#pragma unroll
            for (int h = 0; h < BN / 128; ++h)
              bulk_load_1d(s_sfb + s * C::kSfbBytes + h * 4 * kSfChunk,
                           sfb_src + ((size_t)h * chunks_per_row + (size_t)ks * 4) * kSfChunk, 4 * kSfChunk, full);
          }
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
      if (lane == 0) pdl_trigger();
    } else if (lane == 0) {
      uint32_t s = 0, ph = 1;
      bool ok = true;
      // the tile-table entries of an item are fetched one item ahead, so their latency hides behind a whole k-loop
      int mt_n = 0, e_n = 0, row0_n = 0;
      if (blockIdx.x < total_items) {
        mt_n = (int)(blockIdx.x / n_ntiles);
        e_n = p.tile_expert ? p.tile_expert[mt_n] : 0;
        row0_n = p.tile_row0 ? p.tile_row0[mt_n] : mt_n * kBM;
      }
      for (long long item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int nt = (int)(item - (long long)mt_n * n_ntiles);
        const int e = e_n, row0 = row0_n;
        if (item + gridDim.x < total_items) {
          mt_n = (int)((item + gridDim.x) / n_ntiles);
          e_n = p.tile_expert ? p.tile_expert[mt_n] : 0;
          row0_n = p.tile_row0 ? p.tile_row0[mt_n] : mt_n * kBM;
        }
        const int brow0 = e * p.N + nt * BN;
        const uint8_t* sfa_src = p.sfa + (size_t)(row0 >> 7) * chunks_per_row * kSfChunk;
        const uint8_t* sfb_src = p.sfb + (size_t)(brow0 >> 7) * chunks_per_row * kSfChunk;
        for (int ks = 0; ks < nk; ++ks) {
          if (!mbar_wait(bar_empty + 8 * s, ph)) { report(p.status, 101); ok = false; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, C::kStageBytes);
          tma_load_2d(s_a + s * C::kABytes, &tm_a, full, ks * 128, row0);
          tma_load_2d(s_b + s * C::kBBytes, &tm_b, full, ks * 128, brow0);
          bulk_load_1d(s_sfa + s * C::kSfaBytes, sfa_src + (size_t)ks * 4 * kSfChunk, 4 * kSfChunk, full);
#pragma unroll
          for (int h = 0; h < BN / 128; ++h)
            bulk_load_1d(s_sfb + s * C::kSfbBytes + h * 4 * kSfChunk,
                         sfb_src + ((size_t)h * chunks_per_row + (size_t)ks * 4) * kSfChunk, 4 * kSfChunk, full);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
      // this CTA has asked for its last bytes: the next kernel of the stream may start its prologue under our tail
      pdl_trigger();
    }
  } else if (warp >= 2 && warp < kFirstEpiWarp) {
    // ------------------------------------------------------------------ scale-factor copiers: shared memory -> TMEM
    if (lane == 0) {
      if (warp == 2) copier_loop<BN, 0>(p, tmem, s_sfa, s_sfb, bar_full, bar_sf, total_items, nk);
      else if (warp == 3) copier_loop<BN, 1 % kCopiers>(p, tmem, s_sfa, s_sfb, bar_full, bar_sf, total_items, nk);
      else copier_loop<BN, 2 % kCopiers>(p, tmem, s_sfa, s_sfb, bar_full, bar_sf, total_items, nk);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // One thread feeds the tensor pipe with four instructions per stage: everything is 32-bit, the stage ring is
      // walked with counters and the shared-memory descriptors are base + stage * stride.
      constexpr uint32_t idesc = make_idesc_nvf4(kBM, BN);
      constexpr uint32_t kHiOp = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, SWIZZLE_128B
      const uint32_t a_lo0 = ((s_a >> 4) & 0x3FFF) | (1u << 16), b_lo0 = ((s_b >> 4) & 0x3FFF) | (1u << 16);
      uint32_t s = 0, ph = 0, it = 0;
      bool ok = true;
      PROBE_DECL
      for (long long item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
        const uint32_t buf = it % C::kAccBufs;
        PROBE_T(pr_a)
        if (!mbar_wait(bar_acc_empty + 8 * buf, ((it / C::kAccBufs) & 1) ^ 1)) { report(p.status, 102); break; }
        PROBE_ADD(pr_acc, pr_a)
        tc_fence_after();
        const uint32_t acc = tmem + buf * BN;
        for (int ks = 0; ks < nk; ++ks) {
          // the copiers waited for the stage's TMA bytes before they copied: their barrier covers the operands too
          PROBE_T(pr_b)
          if (!mbar_wait(bar_sf + 8 * s, ph)) { report(p.status, 103); ok = false; break; }
          PROBE_ADD(pr_sf, pr_b)
          tc_fence_after();
          const uint32_t sf_t = tmem + C::kSfBase + s * C::kSfCols;
          const uint32_t a_lo = a_lo0 + s * (C::kABytes >> 4), b_lo = b_lo0 + s * (C::kBBytes >> 4);
          mma_nvf4(acc, ((uint64_t)kHiOp << 32) | a_lo, ((uint64_t)kHiOp << 32) | b_lo, idesc, sf_t, sf_t + 16, ks ? 1u : 0u);
#pragma unroll
          for (int q = 1; q < 4; ++q)
            mma_nvf4(acc, ((uint64_t)kHiOp << 32) | (a_lo + 2 * q), ((uint64_t)kHiOp << 32) | (b_lo + 2 * q), idesc, sf_t + 4 * q,
                     sf_t + 16 + (BN / 128) * 4 * q, 1u);
          mma_commit(bar_empty + 8 * s);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (ok) mma_commit(bar_acc_full + 8 * buf);
      }
      PROBE_STORE
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int group = (warp - kFirstEpiWarp) >> 2;   // which EC accumulator columns
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
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + buf * BN + group * EC;
      epilogue_cols<MODE, EC>(p, taddr, e, (size_t)row0 + r_in_tile, r_in_tile < rows, nt * BN + group * EC, [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      });
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<512>(tmem);
  }
}

// ----------------------------------------------------------------------------- CTA-pair variant (256 x 256 tiles)
// Two CTAs of a cluster work as one tcgen05 cta_group::2 unit: each loads its own 128 rows of A and its own 128
// of the 256 weight rows (no multicast), so one byte fetched from L2 feeds twice the tensor work of a 128 x 256
// single-CTA tile. Work item = (pair of consecutive 128-row m-tiles of one expert, 256 weight rows).
// Barriers: `full` lives in the leader (2 producer arrivals + both CTAs' TMA bytes); `empty` and `acc_full` exist
// in both CTAs and are signalled by the leader's tcgen05.commit to both; `acc_empty` lives in the leader and
// collects the 32 epilogue warps of the pair. The scale-factor copies are issued by kCopiers warps of the leader, half
// of a stage's twelve each (one tcgen05.cp.cta_group::2 copies in both CTAs, each from its own shared memory).
struct PairCfg {
  static constexpr int kStages = 5;
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = 128 * 128;
  static constexpr int kSfaBytes = 4 * kSfChunk;
  static constexpr int kSfbBytes = 2 * 4 * kSfChunk;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // per CTA
  static constexpr int kSfCols = 48;
  static constexpr int kSfBase = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static_assert(kSfBase + kStages * kSfCols <= 512, "TMEM budget: one scale-factor buffer per stage");
};

constexpr int kPairThreads = 32 * (kFirstEpiWarp + 16);    // TMA, MMA, scale-factor copiers, 16 epilogue warps

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
k_gemm_nvfp4_pair(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb, const GemmParams p) {
  using C = PairCfg;
  constexpr int BN = 256;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = smem_base;
  const uint32_t s_b = s_a + C::kStages * C::kABytes;
  const uint32_t s_sfa = s_b + C::kStages * C::kBBytes;
  const uint32_t s_sfb = s_sfa + C::kStages * C::kSfaBytes;
  const uint32_t s_bar = s_sfb + C::kStages * C::kSfbBytes;
  const uint32_t bar_full = s_bar;                            // leader: 2 producer arrivals + both CTAs' TMA bytes
  const uint32_t bar_sf = bar_full + 8 * C::kStages;          // leader: scale factors copied into both CTAs' TMEM
  const uint32_t bar_empty = bar_sf + 8 * C::kStages;         // both CTAs: MMAs of the stage retired
  const uint32_t bar_acc_full = bar_empty + 8 * C::kStages;   // both CTAs
  const uint32_t bar_acc_empty = bar_acc_full + 8;            // leader: 32 epilogue warps of the pair
  const uint32_t s_tmem_slot = bar_acc_empty + 8;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 2);
      mbar_init(bar_sf + 8 * s, kCopiers);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, 32);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc_pair<512>(s_tmem_slot);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_tmem_slot));
  pdl_wait();

  const int n_pairs = p.n_tiles_ptr ? *p.n_tiles_ptr : p.n_tiles_static;
  const int n_ntiles = p.N / BN;
  const int nk = p.K / kStageK;
  const long long total_items = (long long)n_pairs * n_ntiles;
  const int chunks_per_row = p.K >> 6;
  const long long first = blockIdx.x >> 1, stride = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs, own halves)
    if (lane == 0) {
      uint32_t s = 0, ph = 1;
      bool ok = true;
      const uint32_t full0 = map_to_cta(bar_full, 0);
      for (long long item = first; ok && item < total_items; item += stride) {
        const int mt = (int)(item / n_ntiles), nt = (int)(item % n_ntiles);
        const int e = p.tile_expert ? p.tile_expert[mt] : 0;
        const int row0 = (p.tile_row0 ? p.tile_row0[mt] : mt * 256) + (int)rank * 128;
        const int brow0 = e * p.N + nt * BN;
        const int sfa_y = (row0 >> 7) * chunks_per_row;
        const int sfb_y = (brow0 >> 7) * chunks_per_row;
        for (int ks = 0; ks < nk; ++ks) {
          if (!mbar_wait(bar_empty + 8 * s, ph)) { report(p.status, 201); ok = false; break; }
          const uint32_t full = full0 + 8 * s;
          mbar_expect_tx_remote(full, C::kStageBytes);
          tma_load_2d_pair(s_a + s * C::kABytes, &tm_a, full, ks * 128, row0);
          tma_load_2d_pair(s_b + s * C::kBBytes, &tm_b, full, ks * 128, brow0 + (int)rank * 128);
          tma_load_2d_pair(s_sfa + s * C::kSfaBytes, &tm_sfa, full, 0, sfa_y + ks * 4);
          tma_load_2d_pair(s_sfb + s * C::kSfbBytes, &tm_sfb, full, 0, sfb_y + ks * 4);
          tma_load_2d_pair(s_sfb + s * C::kSfbBytes + 4 * kSfChunk, &tm_sfb, full, 0, sfb_y + chunks_per_row + ks * 4);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
      pdl_trigger();
    }
  } else if (warp >= 2 && warp < kFirstEpiWarp) {
    // ------------------------------------------------------------------ scale-factor copiers (leader; every copy acts on both CTAs)
    if (leader && lane == 0) {
      constexpr uint32_t kHiSf = (128u >> 4) | (1u << 14);
      const int j0 = warp - 2;
      const uint32_t sfa_lo0 = (s_sfa >> 4) & 0x3FFF, sfb_lo0 = (s_sfb >> 4) & 0x3FFF;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (long long item = first; ok && item < total_items; item += stride) {
        for (int ks = 0; ks < nk; ++ks) {
          if (!mbar_wait_cluster(bar_full + 8 * s, ph)) { report(p.status, 205); ok = false; break; }
          tc_fence_after();
          const uint32_t sf_t = tmem + C::kSfBase + s * C::kSfCols;
          const uint32_t sfa_lo = sfa_lo0 + s * (C::kSfaBytes >> 4), sfb_lo = sfb_lo0 + s * (C::kSfbBytes >> 4);
          for (int j = j0; j < 12; j += kCopiers) {    // copy j of the stage: 0..3 A scales, then B scales (half h, k-block q)
            if (j < 4) {
              tmem_cp_sf_pair(sf_t + 4 * j, ((uint64_t)kHiSf << 32) | (sfa_lo + j * (kSfChunk >> 4)));
            } else {
              const int h = (j - 4) >> 2, q = (j - 4) & 3;
              tmem_cp_sf_pair(sf_t + 16 + 8 * q + 4 * h, ((uint64_t)kHiSf << 32) | (sfb_lo + (h * 4 + q) * (kSfChunk >> 4)));
            }
          }
          mma_commit_pair_local(bar_sf + 8 * s);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_nvf4(256, BN);
      constexpr uint32_t kHiOp = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t a_lo0 = ((s_a >> 4) & 0x3FFF) | (1u << 16), b_lo0 = ((s_b >> 4) & 0x3FFF) | (1u << 16);
      uint32_t s = 0, ph = 0, it = 0;
      bool ok = true;
      PROBE_DECL
      for (long long item = first; ok && item < total_items; item += stride, ++it) {
        PROBE_T(pr_a)
        if (!mbar_wait_cluster(bar_acc_empty, (it & 1) ^ 1)) { report(p.status, 202); break; }
        PROBE_ADD(pr_acc, pr_a)
        tc_fence_after();
        for (int ks = 0; ks < nk; ++ks) {
          PROBE_T(pr_b)
          if (!mbar_wait(bar_sf + 8 * s, ph)) { report(p.status, 203); ok = false; break; }
          PROBE_ADD(pr_sf, pr_b)
          tc_fence_after();
          const uint32_t sf_t = tmem + C::kSfBase + s * C::kSfCols;
          const uint32_t a_lo = a_lo0 + s * (C::kABytes >> 4), b_lo = b_lo0 + s * (C::kBBytes >> 4);
          mma_nvf4_pair(tmem, ((uint64_t)kHiOp << 32) | a_lo, ((uint64_t)kHiOp << 32) | b_lo, idesc, sf_t, sf_t + 16, ks ? 1u : 0u);
#pragma unroll
          for (int q = 1; q < 4; ++q)
            mma_nvf4_pair(tmem, ((uint64_t)kHiOp << 32) | (a_lo + 2 * q), ((uint64_t)kHiOp << 32) | (b_lo + 2 * q), idesc,
                          sf_t + 4 * q, sf_t + 16 + 8 * q, 1u);
          mma_commit_pair(bar_empty + 8 * s);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (ok) mma_commit_pair(bar_acc_full);
      }
      PROBE_STORE
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs: own 128 rows x 256 columns)
    const int quad = warp & 3;
    const int group = (warp - kFirstEpiWarp) >> 2;
    const int r_in_tile = quad * 32 + lane;
    const uint32_t acc_empty_leader = map_to_cta(bar_acc_empty, 0);
    uint32_t it = 0;
    for (long long item = first; item < total_items; item += stride, ++it) {
      const int mt = (int)(item / n_ntiles), nt = (int)(item % n_ntiles);
      const int e = p.tile_expert ? p.tile_expert[mt] : 0;
      const int row0 = (p.tile_row0 ? p.tile_row0[mt] : mt * 256) + (int)rank * 128;
      const int pair_rows = p.tile_rows ? p.tile_rows[mt] : min(256, p.M - mt * 256);
      const int rows = min(128, max(0, pair_rows - (int)rank * 128));
      int okw = 1;
      if (lane == 0) okw = mbar_wait_cluster(bar_acc_full, it & 1) ? 1 : 0;
      okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
      if (!okw) { if (lane == 0) report(p.status, 204); break; }
      tc_fence_after();
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + group * 64;
      epilogue_cols<MODE, 64>(p, taddr, e, (size_t)row0 + r_in_tile, r_in_tile < rows, nt * BN + group * 64, [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(acc_empty_leader);
      });
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair<512>(tmem);
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
int make_operand_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows, uint64_t pitch_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 701;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {pitch_bytes ? pitch_bytes : row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700 + (int)r;
}

// Scale-factor tiles as a 2-D tensor of 512-byte chunks: [n_chunks, 128 x u32]; a box is 4 consecutive chunks.
int make_sf_map(CUtensorMap* map, const void* base, uint64_t n_chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 701;
  cuuint64_t dims[2] = {128, n_chunks};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 4};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 700 + (int)r;
}

template <int MODE>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                       const GemmParams& p, int grid, cudaStream_t st) {
  auto kern = k_gemm_nvfp4_pair<MODE>;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(kern, PairCfg::kSmemBytes)) return e;
  return (int)launch_chain(kern, dim3(grid), dim3(kPairThreads), PairCfg::kSmemBytes, st, ta, tb, tsa, tsb, p);
}

// grid = 2 CTAs per work-item stream, at most one pair per two SMs
int launch_gemm_nvfp4_pair(int mode, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                           const GemmParams& p, int n_clusters, cudaStream_t st) {
  if (n_clusters <= 0) return 0;
  if (p.K % kStageK != 0 || p.N % 256 != 0) return 702;
  const int grid = 2 * n_clusters;
  if (mode == kGemmFc1) return launch_pair<kGemmFc1>(ta, tb, tsa, tsb, p, grid, st);
  if (mode == kGemmFc2) return launch_pair<kGemmFc2>(ta, tb, tsa, tsb, p, grid, st);
  return launch_pair<kGemmDense>(ta, tb, tsa, tsb, p, grid, st);
}

template <int MODE, int BN, int EC>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  auto kern = k_gemm_nvfp4<MODE, BN, EC>;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(kern, GemmCfg<BN>::kSmemBytes)) return e;
  return (int)launch_chain(kern, dim3(grid), dim3(gemm_threads<BN, EC>()), GemmCfg<BN>::kSmemBytes, st, ta, tb, p);
}

// Epilogue columns per warp. Eight warps x 128 columns win only when the k-loop is long AND the GEMM is tensor-bound
// (DeepSeek-V3 FC1 at T = 8192: 1-2 %). With a short k-loop the eight-warp epilogue is not hidden, and a batch that merely
// streams its weights (rows_hint: at most that many rows of A) wants its accumulator back as early as possible:
// T = 128 over 128 experts at K = 4096 takes 137 us per step with 16 x 64 against 151 us.
static int epilogue_cols_for(int k, int64_t rows_hint) { return (k >= 4096 && (rows_hint == 0 || rows_hint > 8192)) ? 128 : 64; }

template <int MODE>
static int launch_mode(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st) {
  const int ec = epilogue_cols_for(p.K, p.rows_hint);
  if (bn == 128) return ec == 64 ? launch_one<MODE, 128, 64>(ta, tb, p, grid, st) : launch_one<MODE, 128, 128>(ta, tb, p, grid, st);
  if (bn == 256) return ec == 64 ? launch_one<MODE, 256, 64>(ta, tb, p, grid, st) : launch_one<MODE, 256, 128>(ta, tb, p, grid, st);
  return 703;
}

int launch_gemm_nvfp4(int mode, int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                      cudaStream_t st) {
  if (grid <= 0) return 0;
  if (p.K % kStageK != 0 || p.N % bn != 0) return 702;
  if (mode == kGemmFc1) return launch_mode<kGemmFc1>(bn, ta, tb, p, grid, st);
  if (mode == kGemmFc2) return launch_mode<kGemmFc2>(bn, ta, tb, p, grid, st);
  return launch_mode<kGemmDense>(bn, ta, tb, p, grid, st);
}

#ifdef B200MOE_PROBE
extern "C" int b200moe_probe_read(long long* host, int n) {
  return (int)cudaMemcpyFromSymbol(host, g_probe, sizeof(long long) * n);
}
#endif

}  // namespace b200
