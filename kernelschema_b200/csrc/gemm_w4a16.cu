// Dense GEMM with bf16 activations and NVFP4 weights (W4A16): out = bf16(alpha * A @ decode(B)^T), the contract of
// gemm/dense/bf16_nvfp4_gemm/problem/reference.py:10-15 (A is NOT quantised; B payload [N, K/2] with row-major,
// un-swizzled E4M3 block-16 scales [N, K/16]).
//
// An E2M1 value times an E4M3 scale has at most 6 significant bits and lies in [2^-10, 2688], so it is exactly
// representable in bf16. The weights are therefore expanded to bf16 on the fly, bit-exactly, and the
// product runs on tcgen05.mma kind::f16 (bf16 x bf16, fp32 accumulation in TMEM): the result differs from the fp32
// reference only by the order of the fp32 additions.
//
// Tile: 256 rows of A (two 128-row accumulators) x BN weight rows, K in steps of 64; one decoded weight tile feeds two
// MMAs. The kernel is bound by shared-memory bandwidth (per k-step the tile's A and decoded B are written once and read
// by the MMAs), so the wide form BN = 256 is the default when N allows it: 160 KB of shared-memory traffic per
// 256 x 256 x 64 step against 112 KB per 256 x 128 x 64 step. Its two 256-column accumulators fill the 512 TMEM columns,
// so the epilogue of a tile (a few microseconds) is not overlapped; BN = 128 (N % 256 != 0, or M <= 128 where more,
// narrower tiles keep more SMs busy) alternates between two accumulator pairs.
// Warp roles: 0 = TMA producer of A (bf16, 128-byte swizzle); 1 = TMEM owner + MMA issuer; then BN/32 decoder warps, one
// thread per weight row of the tile: it reads the row's 128-byte line (256 weights) and 16 scale bytes with plain loads,
// one k-group ahead, expands them with byte permutes and one bf16 multiply per pair, and writes bf16 into shared memory
// in the layout a 128-byte-swizzled TMA load would have produced (16-byte chunk c of row r at
// r * 128 + ((c ^ (r & 7)) * 16)), then fence.proxy.async + mbarrier arrive; the last 8 warps = epilogue.
// Every wait is bounded and reports through the status word.
#include "kernels.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

namespace b200 {

namespace {

template <int BN>
struct WCfg {
  static constexpr int kStages = BN == 256 ? 3 : 4;
  static constexpr int kABytes = 256 * 128;                // 256 rows x 64 bf16
  static constexpr int kBBytes = BN * 128;                 // BN weight rows x 64 bf16
  static constexpr int kSmem = kStages * (kABytes + kBBytes) + 1024 + 256;
  static constexpr int kDecWarps = BN / 32;                // one decoder thread per weight row
  static constexpr int kEpiWarp0 = 2 + kDecWarps;          // first epilogue warp: 2 mod 4, so warp & 3 walks the lane quadrants
  static constexpr int kThreads = 32 * (kEpiWarp0 + 8);
  static constexpr int kAccBufs = 256 / BN;                // pairs of accumulators that fit the 512 TMEM columns
};

struct W4A16Params {
  const uint8_t* b_q;      // [N, K/2]
  const uint8_t* b_sf;     // [N, K/16] E4M3, row-major
  const float* alpha;      // device scalar or null (= 1)
  __nv_bfloat16* out;
  int64_t out_stride;
  int M, N, K;
  int32_t* status;
  // split-K (small M only): `splits` CTAs share one output tile, each reduces `groups_per_split` k-groups of 256 and
  // writes fp32 partial sums to partial[split][M][N]; k_w4a16_reduce adds them in split order. splits == 1: no workspace.
  int splits;
  int groups_per_split;
  float* partial;
};

DEV void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Two E4M3 bytes (low 16 bits of s) -> bf16x2 (exact: E4M3 has 4 significant bits).
DEV uint32_t e4m3x2_to_bf16x2(uint32_t s) {
  uint32_t h;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h) : "r"(s & 0xFFFFu));
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&b);
}

// Four E2M1 codes (the four nibbles of the low 16 bits of w) -> two bf16x2 words, with byte permutes only: the
// conversion instructions (cvt e2m1x2 -> f16x2 -> f32 -> bf16x2, two per weight) run at a fraction of the ALU rate and
// were the bound of this kernel. The bf16 image of magnitude code c is {0, 0x3F00, 0x3F80, 0x3FC0, 0x4000, 0x4040,
// 0x4080, 0x40C0}[c]: its low and high bytes are looked up with prmt in two 8-byte tables, the sign bits are moved to
// bit 7 of the high bytes with prmt's sign-replication mode, and a last pair of prmt interleaves low and high bytes.
DEV void e2m1x4_to_bf16x2(uint32_t w, uint32_t& v01, uint32_t& v23) {
  const uint32_t sel = w & 0x7777u;
  const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, sel);        // low bytes of codes 0..3 | 4..7
  uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);              // high bytes
  const uint32_t u = w & 0x8888u;                                        // byte k of u: sign of nibble 2k+1 in bit 7, of 2k in bit 3
  const uint32_t sgn = __byte_perm(u, u << 4, 0x9D8Cu);                  // byte i = 0xFF if nibble i is negative (msb replication)
  hi |= sgn & 0x80808080u;
  v01 = __byte_perm(lo, hi, 0x5140u);
  v23 = __byte_perm(lo, hi, 0x7362u);
}

// Half of one k-step (32 of its 64 weights) of one weight row: four payload words and their two scale bytes (low 16
// bits of sf2) -> 64 bytes of bf16. `dst` is the row's base inside the stage; 16-byte chunk c (= c0 + 0..3) goes to
// chunk slot c ^ sw (the 128-byte swizzle, sw = row & 7). Magnitude x scale is exact in bf16 (2 x 4 significant bits).
DEV void decode_half_stage(const uint32_t* w, uint32_t sf2, uint32_t dst, uint32_t sw, uint32_t c0) {
  const uint32_t sc_pair = e4m3x2_to_bf16x2(sf2);
#pragma unroll
  for (int j = 0; j < 4; ++j) {                     // 16-byte chunk = 8 weights = one payload word; two chunks share a scale
    const uint32_t c = c0 + j;
    const uint32_t sc = (j & 2) ? __byte_perm(sc_pair, 0, 0x3232) : __byte_perm(sc_pair, 0, 0x1010);
    uint32_t o[4];
    e2m1x4_to_bf16x2(w[j], o[0], o[1]);
    e2m1x4_to_bf16x2(w[j] >> 16, o[2], o[3]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&o[i]), *reinterpret_cast<const __nv_bfloat162*>(&sc));
      o[i] = *reinterpret_cast<const uint32_t*>(&prod);
    }
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + ((c ^ sw) << 4)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                 : "memory");
  }
}

// BN accumulator columns of the calling warp's 32 lanes -> alpha * x as bf16 at out[row, col0 ...], 64 columns at a
// time; `release` is called right after the last TMEM read. A warp without live rows only releases.
template <int BN, class Release>
DEV void store_cols(const W4A16Params& p, uint32_t taddr, int row, bool live, int col0, float alpha, int split, Release release) {
  if (!__any_sync(0xFFFFFFFFu, live)) {
    release();
    return;
  }
  if (BN == 128 && p.splits > 1) {                   // fp32 partial sums of this split; alpha and the rounding come in the reduce
    float* dst = p.partial + ((size_t)split * p.M + row) * p.N + col0;
#pragma unroll
    for (int pass = 0; pass < BN / 32; ++pass) {
      float v[32];
      tmem_ld32(taddr + pass * 32, v);
      tmem_ld_wait();
      if (pass == BN / 32 - 1) release();
      if (live) {
#pragma unroll
        for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(dst + pass * 32)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    }
    return;
  }
  __nv_bfloat16* dst_row = p.out + (size_t)row * p.out_stride + col0;
#pragma unroll
  for (int pass = 0; pass < BN / 64; ++pass) {
    float v[2][32];
    tmem_ld32(taddr + pass * 64, v[0]);
    tmem_ld32(taddr + pass * 64 + 32, v[1]);
    tmem_ld_wait();
    if (pass == BN / 64 - 1) release();
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
                       "r"(o[8 * j + 1]), "r"(o[8 * j + 2]), "r"(o[8 * j + 3]), "r"(o[8 * j + 4]), "r"(o[8 * j + 5]), "r"(o[8 * j + 6]),
                       "r"(o[8 * j + 7])
                       : "memory");
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(WCfg<BN>::kThreads, 1)
k_gemm_w4a16(const __grid_constant__ CUtensorMap tm_a, const W4A16Params p) {
  using C = WCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = base, s_b = s_a + C::kStages * C::kABytes, s_bar = s_b + C::kStages * C::kBBytes;
  const uint32_t bar_full_a = s_bar;                         // [stages] TMA bytes of A landed
  const uint32_t bar_full_b = bar_full_a + 8 * C::kStages;   // [stages] the decoder warps wrote their rows
  const uint32_t bar_empty = bar_full_b + 8 * C::kStages;    // [stages] MMAs of the stage retired
  const uint32_t bar_acc_full = bar_empty + 8 * C::kStages;  // [kAccBufs]
  const uint32_t bar_acc_empty = bar_acc_full + 16;          // [kAccBufs] 8 epilogue warps
  const uint32_t s_slot = bar_acc_empty + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full_a + 8 * s, 1);
      mbar_init(bar_full_b + 8 * s, C::kDecWarps);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < C::kAccBufs; ++b) {
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
  const int n_nt = p.N / BN;                // BN-row tiles of the weights
  const int groups = p.K >> 8;              // k-groups of 256 weights = one 128-byte line per weight row
  // item = (tile, split), split fastest; tile = (mt, nt), n fastest: the CTAs of a wave share A's rows and sweep the
  // weights (L2-resident). A split covers k-groups [g0, g1).
  const int total_items = n_mt * n_nt * p.splits;
  auto item_tile = [&](int item) { return item / p.splits; };
  auto item_g0 = [&](int item) { return (item % p.splits) * p.groups_per_split; };
  auto item_g1 = [&](int item) { return min(groups, (item % p.splits + 1) * p.groups_per_split); };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer of A
    if (lane == 0) {
      uint32_t s = 0, ph = 1;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const int mt = item_tile(item) / n_nt;
        for (int ks = 4 * item_g0(item); ks < 4 * item_g1(item); ++ks) {
          if (!mbar_wait(bar_empty + 8 * s, ph)) { if (p.status) atomicCAS(p.status, 0, 121); ok = false; break; }
          mbar_expect_tx(bar_full_a + 8 * s, C::kABytes);
          tma_load_2d(s_a + s * C::kABytes, &tm_a, bar_full_a + 8 * s, ks * 128, mt * 256);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
      pdl_trigger();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BN);
      uint32_t s = 0, ph = 0, it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x, ++it) {
        const int mt = item_tile(item) / n_nt;
        const bool second = p.M - mt * 256 > 128;          // rows 128..255 of the tile hold real rows
        const int nk = 4 * (item_g1(item) - item_g0(item));
        const uint32_t buf = it % C::kAccBufs;
        if (!mbar_wait(bar_acc_empty + 8 * buf, ((it / C::kAccBufs) & 1) ^ 1)) { if (p.status) atomicCAS(p.status, 0, 122); break; }
        tc_fence_after();
        const uint32_t acc = tmem + buf * 2 * BN;
        for (int ks = 0; ks < nk; ++ks) {
          if (!mbar_wait(bar_full_a + 8 * s, ph) || !mbar_wait(bar_full_b + 8 * s, ph)) {
            if (p.status) atomicCAS(p.status, 0, 123);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_d = make_desc_sw128(s_a + s * C::kABytes), b_d = make_desc_sw128(s_b + s * C::kBBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            mma_bf16(acc, a_d + 2 * q, b_d + 2 * q, idesc, (ks | q) ? 1u : 0u);
            if (second) mma_bf16(acc + BN, a_d + (128 * 128 >> 4) + 2 * q, b_d + 2 * q, idesc, (ks | q) ? 1u : 0u);
          }
          mma_commit(bar_empty + 8 * s);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
        if (ok) mma_commit(bar_acc_full + 8 * buf);
      }
    }
  } else if (warp < C::kEpiWarp0) {
    // ------------------------------------------------------------------ weight decoders: thread = weight row of the tile
    const int r = threadIdx.x - 64;                         // 0 .. BN-1
    const uint32_t row_off = (uint32_t)r * 128u;
    const uint32_t sw = (uint32_t)(r & 7);
    uint32_t s = 0, ph = 1;
    bool ok = true;
    uint4 nxt[8];
    uint4 nxt_sf;
    auto fetch = [&](int item, int g) {
      const int nt = item_tile(item) % n_nt;
      const size_t row = (size_t)nt * BN + r;
      const uint4* q = reinterpret_cast<const uint4*>(p.b_q + row * (size_t)(p.K >> 1)) + (size_t)g * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) nxt[i] = __ldg(q + i);
      nxt_sf = __ldg(reinterpret_cast<const uint4*>(p.b_sf + row * (size_t)(p.K >> 4)) + g);
    };
    if ((int)blockIdx.x < total_items) fetch(blockIdx.x, item_g0(blockIdx.x));
    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      const int g1 = item_g1(item);
      for (int g = item_g0(item); ok && g < g1; ++g) {
        uint32_t cur[32];
        uint32_t cur_sf[4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          cur[4 * i] = nxt[i].x; cur[4 * i + 1] = nxt[i].y; cur[4 * i + 2] = nxt[i].z; cur[4 * i + 3] = nxt[i].w;
        }
        cur_sf[0] = nxt_sf.x; cur_sf[1] = nxt_sf.y; cur_sf[2] = nxt_sf.z; cur_sf[3] = nxt_sf.w;
        // next line: the following k-group of this item, or the first of this CTA's next item
        if (g + 1 < g1) fetch(item, g + 1);
        else if (item + (int)gridDim.x < total_items) fetch(item + gridDim.x, item_g0(item + gridDim.x));
#pragma unroll
        for (int q = 0; q < 4; ++q) {                       // the four 64-wide k-steps of the group
          int okw = 1;
          if (lane == 0) okw = mbar_wait(bar_empty + 8 * s, ph) ? 1 : 0;
          okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
          if (!okw) { if (lane == 0 && p.status) atomicCAS(p.status, 0, 125); ok = false; break; }
          const uint32_t dst = s_b + s * C::kBBytes + row_off;
          decode_half_stage(cur + 8 * q, cur_sf[q], dst, sw, 0);
          decode_half_stage(cur + 8 * q + 4, cur_sf[q] >> 16, dst, sw, 4);
          fence_async_proxy();                              // generic-proxy writes -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full_b + 8 * s);
          if (++s == C::kStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 8 warps = 2 accumulators x 4 lane quadrants
    const int quad = warp & 3;
    const int half = (warp - C::kEpiWarp0) >> 2;
    const float alpha = p.alpha ? *p.alpha : 1.0f;
    uint32_t it = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
      const int tile = item_tile(item);
      const int mt = tile / n_nt, nt = tile % n_nt;
      const uint32_t buf = it % C::kAccBufs;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(bar_acc_full + 8 * buf, (it / C::kAccBufs) & 1) ? 1 : 0;
      okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
      if (!okw) { if (lane == 0 && p.status) atomicCAS(p.status, 0, 124); break; }
      tc_fence_after();
      const int row = mt * 256 + half * 128 + quad * 32 + lane;
      const bool live = row < p.M;
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + buf * 2 * BN + half * BN;
      store_cols<BN>(p, taddr, row, live, nt * BN, alpha, item % p.splits, [&]() {
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

// out[m, n] = bf16(alpha * sum over splits of partial[s][m][n]), splits added in ascending order (reproducible).
__global__ void __launch_bounds__(256) k_w4a16_reduce(const float* __restrict__ partial, const float* __restrict__ alpha_ptr, int splits,
                                                      int64_t M, int64_t N, __nv_bfloat16* __restrict__ out, int64_t out_stride) {
  pdl_trigger();
  pdl_wait();
  const float alpha = alpha_ptr ? *alpha_ptr : 1.0f;
  const int64_t quads = M * N / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (int64_t)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(partial)[i];
    for (int s = 1; s < splits; ++s) {
      const float4 v = reinterpret_cast<const float4*>(partial + (size_t)s * M * N)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const int64_t m = (i * 4) / N, n = (i * 4) % N;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * alpha, acc.y * alpha), hi = __floats2bfloat162_rn(acc.z * alpha, acc.w * alpha);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + m * out_stride + n) = o;
  }
}

}  // namespace

// Split-K plan for small M: enough CTAs per output tile to occupy the device; 1 = no split (no workspace needed).
static int w4a16_splits(int64_t m, int64_t n, int64_t k, int sms) {
  if (m > 128) return 1;
  const int64_t tiles = n / 128, groups = k / 256;
  int64_t s = sms / tiles;
  if (s > 8) s = 8;
  if (s > groups) s = groups;
  return s < 2 ? 1 : (int)s;
}

int64_t gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  const int s = w4a16_splits(m, n, k, sm_count());
  return s > 1 ? (int64_t)s * m * n * 4 : 0;
}

template <int BN>
static int launch_w4a16(const CUtensorMap& ta, const W4A16Params& p, int sms, cudaStream_t st) {
  auto kern = k_gemm_w4a16<BN>;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(kern, WCfg<BN>::kSmem)) return e;
  const int64_t items = (int64_t)((p.M + 255) / 256) * (p.N / BN) * p.splits;
  return (int)launch_chain(kern, dim3((unsigned)(items < sms ? items : sms)), dim3(WCfg<BN>::kThreads), WCfg<BN>::kSmem, st, ta, p);
}

int launch_gemm_w4a16(const void* a, int64_t a_stride, const void* b_q, const void* b_sf, const float* alpha, int64_t m, int64_t n,
                      int64_t k, void* out, int64_t out_stride, void* workspace, int64_t workspace_bytes, int32_t* status,
                      cudaStream_t st) {
  if (m == 0) return 0;
  const int bn = (n % 256 == 0 && m > 128) ? 256 : 128;
  CUtensorMap ta;
  int rc = make_operand_map(&ta, a, (uint64_t)m, (uint64_t)k * 2, 256, (uint64_t)a_stride * 2);
  if (rc) return rc;
  const int sms = sm_count();
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
  p.splits = 1;
  p.groups_per_split = (int)(k / 256);
  p.partial = nullptr;
  const int want = w4a16_splits(m, n, k, sms);
  if (bn == 128 && want > 1 && workspace && workspace_bytes >= (int64_t)want * m * n * 4) {
    p.groups_per_split = (int)((k / 256 + want - 1) / want);
    p.splits = (int)((k / 256 + p.groups_per_split - 1) / p.groups_per_split);      // no empty split
    p.partial = (float*)workspace;
  }
  rc = bn == 256 ? launch_w4a16<256>(ta, p, sms, st) : launch_w4a16<128>(ta, p, sms, st);
  if (rc || p.splits == 1) return rc;
  const int64_t quads = m * n / 4;
  const int64_t blocks = (quads + 255) / 256;
  return (int)launch_chain(k_w4a16_reduce, dim3((unsigned)(blocks < (int64_t)sms * 8 ? blocks : (int64_t)sms * 8)), dim3(256), 0, st, (const float*)p.partial,
                           alpha, p.splits, m, n, (__nv_bfloat16*)out, out_stride);
}

}  // namespace b200
