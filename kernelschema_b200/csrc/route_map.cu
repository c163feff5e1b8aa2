// Expert-permutation index build: per-expert counts, 128-row-aligned segment starts, the m-tile list,
// and the route <-> permuted-row maps.
//
// Same outputs as the reference candidate's k_count / k_scan_tiles / k_scatter_agg chain
// (moe/nvfp4_fused_moe/candidate/nvfp4_moe.cu:582, :750, :700; specified in
// schema_wiki/.../nvfp4_fused_moe/root.yaml:172-197), with one tightening: the position of a route
// inside its expert segment is its rank in ascending flat index t*K+k (the reference leaves that
// order arbitrary), so every integer output is reproducible and can be compared bit for bit.
// No atomics: three passes (block histograms, scan, stable scatter).
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr int kRouteChunk = 2048;        // routes per block: 32 warps x 2 steps x 32 lanes
constexpr int kRouteWarps = 32;          // these kernels are a few thousand dependent instructions per warp and one block per
                                         // chunk: with 8 warps a block issued one instruction every ~5 cycles per scheduler
constexpr int kRouteThreads = kRouteWarps * 32;
constexpr int kRouteSmemMax = 176 * 1024;  // (32 + 2) x 1024 experts x 4 B + 32 KB of positions (kGatherMaxRoutes x 4 B)

struct RouteView {
  const int32_t* ids;
  int64_t id_stride;  // elements between the id rows of consecutive tokens (>= K)
  int64_t T;
  int K;            // routed slots per token
  int S;            // shared experts: extra always-selected slots
  int E;            // local routed experts
  int expert_offset;
  int seg_len;               // > 0: token slots come in regions of seg_len, of which only the first seg_valid[region] hold a token
  const int32_t* seg_valid;
};

DEV bool slot_holds_token(const RouteView& r, int64_t t) {
  if (r.seg_len <= 0) return true;
  const int64_t s = t / r.seg_len;
  return t - s * r.seg_len < r.seg_valid[s];
}

DEV int route_expert(const RouteView& r, int64_t f, int64_t total) {
  if (f >= total) return -1;
  const int kk = r.K + r.S;
  const int64_t t = f / kk;
  const int k = (int)(f - t * kk);
  if (!slot_holds_token(r, t)) return -1;
  if (k >= r.K) return r.E + (k - r.K);
  const int e = r.ids[t * r.id_stride + k] - r.expert_offset;
  return (e >= 0 && e < r.E) ? e : -1;
}

// Lanes of the warp whose expert equals this lane's: one ballot per bit of the expert id instead of __match_any_sync,
// whose cost grows with the number of distinct values in the warp (close to 32 here). `bits` covers ids below the
// expert count; the extra round on bit `bits` separates the invalid id -1 from the expert made of all ones.
DEV unsigned same_expert_lanes(int e, int bits) {
  unsigned m = 0xFFFFFFFFu;
  for (int b = 0; b <= bits; ++b) {
    const bool set = (e >> b) & 1;
    const unsigned bal = __ballot_sync(0xFFFFFFFFu, set);
    m &= set ? bal : ~bal;
  }
  return m;
}
DEV int expert_bits(int etot) { return etot > 1 ? 32 - __clz(etot - 1) : 0; }

constexpr int kRouteSteps = kRouteChunk / kRouteWarps / 32;   // routes per lane in a chunk
constexpr int kRoutesPerWarp = kRouteSteps * 32;

// Expert of each of this lane's routes in the block's chunk: all loads are issued before any is used.
DEV void load_chunk(const RouteView& r, int64_t total, int64_t chunk_base, int (&e)[kRouteSteps]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t base = chunk_base + warp * kRoutesPerWarp;
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) e[step] = route_expert(r, base + step * 32 + lane, total);
}

// The same for a build whose routes all fit 32-bit indices (the one-block kernel): no 64-bit divisions.
DEV int route_expert32(const RouteView& r, int f, int total) {
  if (f >= total) return -1;
  const int kk = r.K + r.S;
  const int t = f / kk;
  const int k = f - t * kk;
  if (!slot_holds_token(r, t)) return -1;
  if (k >= r.K) return r.E + (k - r.K);
  const int e = r.ids[(int64_t)t * r.id_stride + k] - r.expert_offset;
  return (e >= 0 && e < r.E) ? e : -1;
}

// Per-warp histograms of this block's chunk into hist[warp][e]; each warp owns its row, so no atomics.
template <int STEPS>
DEV void chunk_histogram(const int (&e)[STEPS], int etot, int* hist) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bits = expert_bits(etot);
  for (int i = threadIdx.x; i < (int)(blockDim.x >> 5) * etot; i += blockDim.x) hist[i] = 0;
  __syncthreads();
#pragma unroll
  for (int step = 0; step < STEPS; ++step) {
    if (!__any_sync(0xFFFFFFFFu, e[step] >= 0)) continue;      // a step without a route (decode sizes: most of them)
    const unsigned m = same_expert_lanes(e[step], bits);
    if (e[step] >= 0 && lane == (__ffs(m) - 1)) hist[warp * etot + e[step]] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kRouteThreads) k_route_hist(RouteView r, int etot, int32_t* __restrict__ block_hist) {
  extern __shared__ int hist[];
  pdl_trigger();
  pdl_wait();
  const int64_t total = r.T * (r.K + r.S);
  int ex[kRouteSteps];
  load_chunk(r, total, (int64_t)blockIdx.x * kRouteChunk, ex);
  chunk_histogram(ex, etot, hist);
  for (int e = threadIdx.x; e < etot; e += blockDim.x) {
    int s = 0;
#pragma unroll
    for (int w = 0; w < kRouteWarps; ++w) s += hist[w * etot + e];
    block_hist[(int64_t)blockIdx.x * etot + e] = s;
  }
}

// One block. Turns block_hist into exclusive per-expert prefixes over blocks, then scans experts:
// seg_start (segments padded to 128 rows), the m-tile list, and the totals {n_tiles, r_pad, r_valid}.
__global__ void __launch_bounds__(1024) k_route_scan(int etot, int nblk, int32_t* __restrict__ block_hist,
                                                     int32_t* __restrict__ counts, int32_t* __restrict__ seg_start,
                                                     int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_row0,
                                                     int32_t* __restrict__ tile_rows, int32_t* __restrict__ totals,
                                                     int32_t* __restrict__ pair_expert, int32_t* __restrict__ pair_row0,
                                                     int32_t* __restrict__ pair_rows) {
  __shared__ int warp_pad[32], warp_tiles[32], warp_cnt[32], warp_pairs[32];
  __shared__ int carry[4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x < 4) carry[threadIdx.x] = 0;
  // Exclusive prefix over the blocks, per expert, in a fixed order (reproducible). Two forms, by the number of dependent
  // load rounds: one THREAD per expert with eight loads in flight (ceil(nblk / 8) rounds: many experts, few blocks), or one
  // WARP per expert, lanes on blocks lane, lane + 32, ... and a shuffle scan (ceil(etot / 32) * ceil(nblk / 32) rounds: the
  // receive buffer of an expert-parallel rank, few experts and hundreds of blocks).
  const int rounds_thread = ((nblk + 7) >> 3) * ((etot + (int)blockDim.x - 1) / (int)blockDim.x);
  const int rounds_warp = ((etot + 31) >> 5) * ((nblk + 31) >> 5);
  if (rounds_thread <= rounds_warp) {
    for (int e = threadIdx.x; e < etot; e += blockDim.x) {
      int cnt = 0;
      for (int b0 = 0; b0 < nblk; b0 += 8) {
        int v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (b0 + j < nblk) ? block_hist[(int64_t)(b0 + j) * etot + e] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (b0 + j < nblk) {
            block_hist[(int64_t)(b0 + j) * etot + e] = cnt;
            cnt += v[j];
          }
      }
      counts[e] = cnt;
    }
  } else {
    for (int e = warp; e < etot; e += (int)(blockDim.x >> 5)) {
      int run = 0;
      for (int b0 = 0; b0 < nblk; b0 += 32) {
        const int b = b0 + lane;
        const int v = b < nblk ? block_hist[(int64_t)b * etot + e] : 0;
        int inc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int a = __shfl_up_sync(0xFFFFFFFFu, inc, off);
          if (lane >= off) inc += a;
        }
        if (b < nblk) block_hist[(int64_t)b * etot + e] = run + inc - v;
        run += __shfl_sync(0xFFFFFFFFu, inc, 31);
      }
      if (lane == 0) counts[e] = run;
    }
  }
  __syncthreads();
  for (int e0 = 0; e0 < etot; e0 += blockDim.x) {
    const int e = e0 + threadIdx.x;
    const int cnt = e < etot ? counts[e] : 0;
    const int ntile = (cnt + 127) >> 7;
    const int pad = ntile << 7;
    const int npair = (ntile + 1) >> 1;        // 256-row work items of the CTA-pair GEMM
    int ip = pad, it = ntile, ic = cnt, iq = npair;        // inclusive warp scans
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a = __shfl_up_sync(0xFFFFFFFFu, ip, off);
      const int b = __shfl_up_sync(0xFFFFFFFFu, it, off);
      const int c = __shfl_up_sync(0xFFFFFFFFu, ic, off);
      const int d = __shfl_up_sync(0xFFFFFFFFu, iq, off);
      if (lane >= off) { ip += a; it += b; ic += c; iq += d; }
    }
    if (lane == 31) { warp_pad[warp] = ip; warp_tiles[warp] = it; warp_cnt[warp] = ic; warp_pairs[warp] = iq; }
    __syncthreads();
    int bp = carry[0], bt = carry[1], bq = carry[3];
    for (int w = 0; w < warp; ++w) { bp += warp_pad[w]; bt += warp_tiles[w]; bq += warp_pairs[w]; }
    const int start = bp + ip - pad;
    const int tile0 = bt + it - ntile;
    const int pair0 = bq + iq - npair;
    if (e < etot) {
      seg_start[e] = start;
      for (int j = 0; j < ntile; ++j) {
        tile_expert[tile0 + j] = e;
        tile_row0[tile0 + j] = start + (j << 7);
        tile_rows[tile0 + j] = min(128, cnt - (j << 7));
      }
      if (pair_expert)
        for (int j = 0; j < npair; ++j) {
          pair_expert[pair0 + j] = e;
          pair_row0[pair0 + j] = start + (j << 8);
          pair_rows[pair0 + j] = min(256, cnt - (j << 8));
        }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) {
      int tc = 0;
      for (int w = 0; w < 32; ++w) tc += warp_cnt[w];
      carry[0] = bp + ip;
      carry[1] = bt + it;
      carry[2] += tc;
      carry[3] = bq + iq;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    seg_start[etot] = carry[0];
    totals[0] = carry[1];   // number of 128-row tiles
    totals[1] = carry[0];   // rows of the permuted buffer in use (multiple of 128)
    totals[2] = carry[2];   // valid routes
    totals[3] = carry[3];   // number of 256-row pair items
  }
}

__global__ void __launch_bounds__(kRouteThreads) k_route_scatter(RouteView r, const float* __restrict__ scores, int etot,
                                                       const int32_t* __restrict__ block_base, const int32_t* __restrict__ seg_start,
                                                       int32_t* __restrict__ row_of, int32_t* __restrict__ tok_of_row,
                                                       float* __restrict__ weight_of_row) {
  extern __shared__ int hist[];
  pdl_trigger();
  pdl_wait();
  const int kk = r.K + r.S;
  const int64_t total = r.T * kk;
  int ex[kRouteSteps];
  load_chunk(r, total, (int64_t)blockIdx.x * kRouteChunk, ex);
  chunk_histogram(ex, etot, hist);
  for (int e = threadIdx.x; e < etot; e += blockDim.x) {
    int run = seg_start[e] + block_base[(int64_t)blockIdx.x * etot + e];
#pragma unroll
    for (int w = 0; w < kRouteWarps; ++w) {
      const int c = hist[w * etot + e];
      hist[w * etot + e] = run;
      run += c;
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t base = (int64_t)blockIdx.x * kRouteChunk + warp * (kRouteChunk / kRouteWarps);
  float wt[kRouteSteps];      // all loads before any store
  int32_t tk[kRouteSteps];
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) {
    const int64_t f = base + step * 32 + lane;
    const int64_t t = f / kk;
    const int k = (int)(f - t * kk);
    tk[step] = (int32_t)t;
    wt[step] = (scores && ex[step] >= 0 && k < r.K) ? scores[t * r.id_stride + k] : 1.0f;
  }
  int pos[kRouteSteps];
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) {
    const int e = ex[step];
    pos[step] = -1;
    if (!__any_sync(0xFFFFFFFFu, e >= 0)) continue;
    const unsigned m = same_expert_lanes(e, expert_bits(etot));
    if (e >= 0) pos[step] = hist[warp * etot + e] + __popc(m & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0 && lane == (__ffs(m) - 1)) hist[warp * etot + e] += __popc(m);
    __syncwarp();
  }
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) {
    const int64_t f = base + step * 32 + lane;
    if (f < total) {
      row_of[f] = pos[step];
      if (pos[step] >= 0) {
        tok_of_row[pos[step]] = tk[step];
        weight_of_row[pos[step]] = wt[step];
      }
    }
  }
}

// Whole build in ONE launch for decode-to-medium sizes (up to kFusedMaxBlocks x 2048 routes). Block c scatters chunk c,
// and instead of exchanging histograms with the other blocks it reads ALL expert ids itself (a few tens of KB): that
// gives it every expert's total (segment starts, tile list) and the count in the chunks before its own (its base inside
// the segment). The counts of foreign chunks are accumulated with shared-memory atomics; a count does not depend on the
// order of the additions, so every output stays reproducible. Block 0 also writes the per-expert tables.
constexpr int kFusedMaxBlocks = 8;
constexpr int kGatherMaxRoutes = 8192;           // the fused form that also permutes the rows: 8 routes per lane of ONE chunk

// The permute of one routed row from inside the route-map kernel (small batches): payload with 16-byte vectors, the row's
// scale words straight into the 128x4-tiled image. Scales of padding rows are left as they are: the GEMMs neither store
// nor read across rows, so whatever a padding row computes is dropped.
struct GatherView {
  const uint8_t* hid_q;
  const uint8_t* hid_sf;      // row-major [T, H/16]
  int64_t q_stride, sf_stride;
  int H;
  uint8_t* a_q;               // null: only the scale rows are permuted (the GEMM gathers the payload rows by TMA)
  uint8_t* a_sf;
};

DEV void gather_row(const GatherView& g, int tok, int pos, int lane) {
  const int vecs = g.a_q ? g.H >> 5 : 0, words = g.H >> 6;     // a_q == null: scales only
  const uint4* src = reinterpret_cast<const uint4*>(g.hid_q + (size_t)tok * g.q_stride);
  uint4* dst = reinterpret_cast<uint4*>(g.a_q + (size_t)pos * (g.H >> 1));
  const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(g.hid_sf + (size_t)tok * g.sf_stride);
  uint32_t* sf_dst = reinterpret_cast<uint32_t*>(g.a_sf + (size_t)(pos >> 7) * words * 512 + (size_t)(pos & 31) * 16 +
                                                 (size_t)((pos >> 5) & 3) * 4);
  uint32_t sw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (lane + 32 * i < words) sw[i] = __ldg(sf_src + lane + 32 * i);
  for (int v0 = lane; v0 < vecs; v0 += 32 * 8) {
    uint4 t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v0 + 32 * i < vecs) t[i] = __ldg(src + v0 + 32 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v0 + 32 * i < vecs) dst[v0 + 32 * i] = t[i];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (lane + 32 * i < words) sf_dst[(size_t)(lane + 32 * i) * 128] = sw[i];
  for (int w = lane + 128; w < words; w += 32) sf_dst[(size_t)w * 128] = __ldg(sf_src + w);     // H > 8192
}

// Block-wide scan over the experts, shared by the one-launch kernels. In: hist[w][e] = routes of expert e that warp w of
// this block owns, others[e] = routes of e owned by other blocks, before[e] = those of them that precede this block's.
// Out: segment starts, tile and pair tables and totals (stored by the `writer` block only), and hist[w][e] turned into
// the permuted row of warp w's first route of expert e. Ends with a block barrier.
template <int NW>                                  // NW = warps of the block = rows of hist
DEV void scan_experts(int etot, const int* others, const int* before, int* hist, bool writer, const RouteMapBuffers& b) {
  constexpr int nw = NW;
  __shared__ int warp_pad[kRouteWarps], warp_tiles[kRouteWarps], warp_pairs[kRouteWarps], warp_cnt[kRouteWarps];
  __shared__ int carry[4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < 4) carry[threadIdx.x] = 0;
  __syncthreads();
  for (int e0 = 0; e0 < etot; e0 += blockDim.x) {
    const int e = e0 + threadIdx.x;
    int cnt = 0;
    if (e < etot) {
      cnt = others[e];
#pragma unroll
      for (int w = 0; w < nw; ++w) cnt += hist[w * etot + e];
    }
    const int ntile = (cnt + 127) >> 7, pad = ntile << 7, npair = (ntile + 1) >> 1;
    int ip = pad, it = ntile, ic = cnt, iq = npair;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int a = __shfl_up_sync(0xFFFFFFFFu, ip, off), c2 = __shfl_up_sync(0xFFFFFFFFu, it, off);
      const int c3 = __shfl_up_sync(0xFFFFFFFFu, ic, off), c4 = __shfl_up_sync(0xFFFFFFFFu, iq, off);
      if (lane >= off) { ip += a; it += c2; ic += c3; iq += c4; }
    }
    if (lane == 31) { warp_pad[warp] = ip; warp_tiles[warp] = it; warp_cnt[warp] = ic; warp_pairs[warp] = iq; }
    __syncthreads();
    int bp = carry[0], bt = carry[1], bq = carry[3];
    for (int w = 0; w < warp; ++w) { bp += warp_pad[w]; bt += warp_tiles[w]; bq += warp_pairs[w]; }
    const int start = bp + ip - pad, tile0 = bt + it - ntile, pair0 = bq + iq - npair;
    if (e < etot) {
      if (writer) {
        b.counts[e] = cnt;
        b.seg_start[e] = start;
        for (int j = 0; j < ntile; ++j) {
          b.tile_expert[tile0 + j] = e;
          b.tile_row0[tile0 + j] = start + (j << 7);
          b.tile_rows[tile0 + j] = min(128, cnt - (j << 7));
        }
        if (b.pair_expert)
          for (int j = 0; j < npair; ++j) {
            b.pair_expert[pair0 + j] = e;
            b.pair_row0[pair0 + j] = start + (j << 8);
            b.pair_rows[pair0 + j] = min(256, cnt - (j << 8));
          }
      }
      int run = start + before[e];                   // per-warp bases of this expert, in place of the counts
#pragma unroll
      for (int w = 0; w < nw; ++w) {
        const int c = hist[w * etot + e];
        hist[w * etot + e] = run;
        run += c;
      }
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) {
      int tc = 0;
      for (int w = 0; w < nw; ++w) tc += warp_cnt[w];
      carry[0] = bp + ip;
      carry[1] = bt + it;
      carry[2] += tc;
      carry[3] = bq + iq;
    }
    __syncthreads();
  }
  if (writer && threadIdx.x == 0) {
    b.seg_start[etot] = carry[0];
    b.totals[0] = carry[1];
    b.totals[1] = carry[0];
    b.totals[2] = carry[2];
    b.totals[3] = carry[3];
  }
}

// A chunk's routes are dealt to the block's warps in runs of `rpw` (a multiple of 32, just enough for the chunk), so that a
// small chunk occupies every warp with one step instead of one warp with eight; positions stay in ascending route order.
DEV int routes_per_warp(int chunk_total, int nw = kRouteWarps) { return max(32, (((chunk_total + nw - 1) / nw) + 31) & ~31); }

__global__ void __launch_bounds__(kRouteThreads) k_route_fused(RouteView r, const float* __restrict__ scores, int etot, RouteMapBuffers b) {
  extern __shared__ int hist[];                    // own chunk [kRouteWarps][etot] | all chunks [etot] | chunks before [etot]
  int* others = hist + kRouteWarps * etot;         // routes of expert e in the other chunks
  int* before = others + etot;                     // ... in the chunks before this block's
  const int kk = r.K + r.S;
  const int total = (int)(r.T * kk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool writer = blockIdx.x == 0;
  const int rpw = routes_per_warp(min(kRouteChunk, total - (int)blockIdx.x * kRouteChunk));
  pdl_trigger();
  pdl_wait();
  for (int i = threadIdx.x; i < 2 * etot; i += blockDim.x) others[i] = 0;
  __syncthreads();
  int ex[kRouteSteps];
  float wt[kRouteSteps];                           // routing weight of each own route: fetched with the ids, before any store
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) {
    const int f = (int)blockIdx.x * kRouteChunk + warp * rpw + step * 32 + lane;
    ex[step] = step * 32 < rpw ? route_expert32(r, f, total) : -1;
    wt[step] = 1.0f;
    if (scores && ex[step] >= 0 && ex[step] < r.E) {
      const int t = f / kk;
      wt[step] = scores[(int64_t)t * r.id_stride + (f - t * kk)];
    }
  }
  for (int c = 0; c < (int)gridDim.x; ++c) {
    if (c == (int)blockIdx.x) continue;
    int eo[kRouteSteps];
#pragma unroll
    for (int step = 0; step < kRouteSteps; ++step)
      eo[step] = route_expert32(r, c * kRouteChunk + warp * kRoutesPerWarp + step * 32 + lane, total);
#pragma unroll
    for (int step = 0; step < kRouteSteps; ++step)
      if (eo[step] >= 0) {
        atomicAdd(&others[eo[step]], 1);
        if (c < (int)blockIdx.x) atomicAdd(&before[eo[step]], 1);
      }
  }
  chunk_histogram(ex, etot, hist);                 // own chunk, per warp; its barriers also publish others/before
  scan_experts<kRouteWarps>(etot, others, before, hist, writer, b);
  int pos[kRouteSteps];
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) {
    const int e = ex[step];
    pos[step] = -1;
    if (!__any_sync(0xFFFFFFFFu, e >= 0)) continue;
    const unsigned m = same_expert_lanes(e, expert_bits(etot));
    if (e >= 0) pos[step] = hist[warp * etot + e] + __popc(m & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0 && lane == (__ffs(m) - 1)) hist[warp * etot + e] += __popc(m);
    __syncwarp();
  }
#pragma unroll
  for (int step = 0; step < kRouteSteps; ++step) {
    const int f = (int)blockIdx.x * kRouteChunk + warp * rpw + step * 32 + lane;
    if (step * 32 < rpw && f < total) {
      b.row_of[f] = pos[step];
      if (pos[step] >= 0) {
        b.tok_of_row[pos[step]] = f / kk;
        b.weight_of_row[pos[step]] = wt[step];
      }
    }
  }
}

// Route map AND permute of a decode-sized batch (at most kGatherMaxRoutes routes) in one launch: every block builds the
// whole map for itself in shared memory (a few thousand integer operations), block 0 stores it, and the blocks share the
// row copies, one warp per routed row. The step loops are rolled: a one-wave, latency-bound kernel pays for every
// instruction-cache line it touches, and a decode batch takes one step.
template <int NW>                                  // warps per block: 8 for a handful of routes, kRouteWarps otherwise
__global__ void __launch_bounds__(NW * 32) k_route_gather(RouteView r, const float* __restrict__ scores, int etot, RouteMapBuffers b,
                                                     GatherView gv) {
  extern __shared__ int hist[];                    // [warps][etot] | zeros [etot] | zeros [etot] | expert, then row, of every route
  constexpr int nw = NW;
  int* zeros = hist + nw * etot;
  int* s_pos = zeros + 2 * etot;
  const int kk = r.K + r.S;
  const int total = (int)(r.T * kk);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool writer = blockIdx.x == 0;
  const int rpw = routes_per_warp(total, nw), nsteps = rpw >> 5;
  const int bits = expert_bits(etot);
  pdl_trigger();
  pdl_wait();
  for (int i = threadIdx.x; i < (nw + 2) * etot; i += blockDim.x) hist[i] = 0;
#pragma unroll 4
  for (int step = 0; step < nsteps; ++step) {
    const int f = warp * rpw + step * 32 + lane;
    if (f < total) s_pos[f] = route_expert32(r, f, total);
  }
  __syncthreads();
#pragma unroll 1
  for (int step = 0; step < nsteps; ++step) {
    const int f = warp * rpw + step * 32 + lane;
    const int e = f < total ? s_pos[f] : -1;
    if (!__any_sync(0xFFFFFFFFu, e >= 0)) continue;
    const unsigned m = same_expert_lanes(e, bits);
    if (e >= 0 && lane == (__ffs(m) - 1)) hist[warp * etot + e] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  scan_experts<NW>(etot, zeros, zeros + etot, hist, writer, b);
#pragma unroll 1
  for (int step = 0; step < nsteps; ++step) {
    const int f = warp * rpw + step * 32 + lane;
    const int e = f < total ? s_pos[f] : -1;
    int at = -1;
    if (__any_sync(0xFFFFFFFFu, e >= 0)) {
      const unsigned m = same_expert_lanes(e, bits);
      if (e >= 0) at = hist[warp * etot + e] + __popc(m & ((1u << lane) - 1u));
      __syncwarp();
      if (e >= 0 && lane == (__ffs(m) - 1)) hist[warp * etot + e] += __popc(m);
      __syncwarp();
    }
    if (f < total) {
      s_pos[f] = at;
      if (writer) {
        b.row_of[f] = at;
        if (at >= 0) {
          const int t = f / kk, k = f - t * kk;
          b.tok_of_row[at] = t;
          b.weight_of_row[at] = (scores && k < r.K) ? scores[(int64_t)t * r.id_stride + k] : 1.0f;
        }
      }
    }
  }
  __syncthreads();
  const int warps = (int)gridDim.x * nw;
  for (int f = (int)blockIdx.x * nw + warp; f < total; f += warps) {
    const int at = s_pos[f];
    if (at >= 0) gather_row(gv, f / kk, at, lane);
  }
}

int launch_route_map(const int32_t* ids, const float* scores, int64_t id_stride, int64_t T, int K, int S, int E, int expert_offset,
                     RouteMapBuffers b, cudaStream_t st, int seg_len, const int32_t* seg_valid) {
  const int etot = E + S;
  const int64_t total = T * (K + S);
  const int nblk = (int)((total + kRouteChunk - 1) / kRouteChunk);
  RouteView r{ids, id_stride > 0 ? id_stride : K, T, K, S, E, expert_offset, seg_valid ? seg_len : 0, seg_valid};
  {
    static SmemOptIn fused_opt, hist_opt, scatter_opt;
    if (int e = fused_opt.ensure(k_route_fused, kRouteSmemMax)) return e;
    if (int e = hist_opt.ensure(k_route_hist, kRouteSmemMax)) return e;
    if (int e = scatter_opt.ensure(k_route_scatter, kRouteSmemMax)) return e;
  }
  if (nblk >= 1 && nblk <= kFusedMaxBlocks)
    return (int)launch_chain(k_route_fused, dim3(nblk), dim3(kRouteThreads), sizeof(int) * (kRouteWarps + 2) * (size_t)etot, st, r, scores,
                             etot, b);
  const size_t smem = sizeof(int) * kRouteWarps * (size_t)etot;
  cudaError_t err = cudaSuccess;
  if (nblk > 0) err = launch_chain(k_route_hist, dim3(nblk), dim3(kRouteThreads), smem, st, r, etot, b.block_hist);
  if (err == cudaSuccess)
    err = launch_chain(k_route_scan, dim3(1), dim3(1024), 0, st, etot, nblk, b.block_hist, b.counts, b.seg_start, b.tile_expert,
                       b.tile_row0, b.tile_rows, b.totals, b.pair_expert, b.pair_row0, b.pair_rows);
  if (err == cudaSuccess && nblk > 0)
    err = launch_chain(k_route_scatter, dim3(nblk), dim3(kRouteThreads), smem, st, r, scores, etot, (const int32_t*)b.block_hist,
                       (const int32_t*)b.seg_start, b.row_of, b.tok_of_row, b.weight_of_row);
  return (int)err;
}

bool route_gather_fits(int64_t T, int K, int S, int E, int H) {
  const int64_t total = T * (K + S);
  return total >= 1 && total <= kGatherMaxRoutes && sizeof(int) * ((kRouteWarps + 2) * (size_t)(E + S) + kGatherMaxRoutes) <= kRouteSmemMax &&
         H % 256 == 0;
}

int launch_route_gather(const int32_t* ids, const float* scores, int64_t id_stride, int64_t T, int K, int S, int E, int expert_offset,
                        RouteMapBuffers b, const void* hid_q, const void* hid_sf, int64_t q_stride, int64_t sf_stride, int H, void* a_q,
                        void* a_sf, cudaStream_t st, int seg_len, const int32_t* seg_valid) {
  const int etot = E + S;
  const int64_t total = T * (K + S);
  RouteView r{ids, id_stride > 0 ? id_stride : K, T, K, S, E, expert_offset, seg_valid ? seg_len : 0, seg_valid};
  GatherView gv{(const uint8_t*)hid_q, (const uint8_t*)hid_sf, q_stride > 0 ? q_stride : (int64_t)(H / 2),
                sf_stride > 0 ? sf_stride : (int64_t)(H / 16), H, (uint8_t*)a_q, (uint8_t*)a_sf};
  // a handful of routes (one step of 8 warps): a small block, whose barriers and zeroing cost less (T = 1: 2 us per step)
  const int threads = total <= 256 ? 256 : kRouteThreads;
  int64_t blocks = (total + threads / 32 - 1) / (threads / 32);     // one row per warp while the SMs last
  if (blocks > sm_count()) blocks = sm_count();
  if (threads == 256)       // at most 256 routes: their positions need 1 KB, the whole block stays far below 48 KB
    return (int)launch_chain(k_route_gather<8>, dim3((unsigned)blocks), dim3(256), sizeof(int) * ((8 + 2) * (size_t)etot + 256), st, r,
                             scores, etot, b, gv);
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(k_route_gather<kRouteWarps>, kRouteSmemMax)) return e;
  return (int)launch_chain(k_route_gather<kRouteWarps>, dim3((unsigned)blocks), dim3(kRouteThreads),
                           sizeof(int) * ((kRouteWarps + 2) * (size_t)etot + kGatherMaxRoutes), st, r, scores, etot, b, gv);
}

// ----------------------------------------------------------------------------- allocation-free variant
// Scratch of the route-map build (the per-block histograms) held in a file-scope device array instead of a
// caller- or library-allocated buffer. Sized for kStaticMaxBlocks blocks of 2048 routes and kStaticMaxExperts
// experts: 256 x 264 x 4 B = 264 KiB, resident on every GPU that loads the library until the process exits.
constexpr int kStaticMaxBlocks = 256;      // routes <= 256 * 2048 = 524288
constexpr int kStaticMaxExperts = 264;     // routed + shared experts
static __device__ __align__(256) int32_t g_route_scratch[kStaticMaxBlocks * kStaticMaxExperts];

constexpr int kMaxDevices = 64;
// device address of g_route_scratch, per device, filled on first use; atomic so that host threads making a device's first
// call at the same time both store the same value without a data race
static std::atomic<int32_t*> g_route_scratch_ptr[kMaxDevices];

int launch_route_map_static(const int32_t* ids, const float* scores, int64_t T, int K, int S, int E, int expert_offset,
                            RouteMapBuffers b, cudaStream_t st) {
  const int etot = E + S;
  const int64_t total = T * (K + S);
  const int64_t nblk = (total + kRouteChunk - 1) / kRouteChunk;
  if (etot > kStaticMaxExperts || nblk > kStaticMaxBlocks) return 770;
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return (int)err;
  if (dev < 0 || dev >= kMaxDevices) return 771;
  int32_t* scratch = g_route_scratch_ptr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // The array's name is only a host-side handle: kernels need its device address, looked up once per device
    // with that device current.
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_route_scratch);
    if (err != cudaSuccess) return (int)err;
    scratch = (int32_t*)p;
    g_route_scratch_ptr[dev].store(scratch, std::memory_order_release);
  }
  b.block_hist = scratch;
  return launch_route_map(ids, scores, 0, T, K, S, E, expert_offset, b, st);
}

}  // namespace b200
