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

// PL = logits kept per lane (experts <= 32 * PL); the loops are unrolled for the instantiated size only.
template <int PL>
__global__ void __launch_bounds__(256) k_route_topk(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T,
                                                    int E, int K, int32_t* __restrict__ ids, float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  pdl_trigger();
  pdl_wait();
  if (tok >= T) return;
  float v[PL];
#pragma unroll
  for (int i = 0; i < PL; ++i) {
    const int e = i * 32 + lane;
    float x = -INFINITY;
    if (e < E) {
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
    for (int i = 0; i < PL; ++i) {
      const int e = i * 32 + lane;
      if (e < E && (v[i] > best)) { best = v[i]; best_e = e; }
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
      for (int i = 0; i < PL; ++i)
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

// ----------------------------------------------------------------------------- decode-size router logits (T <= 16)
// With a handful of tokens the product is a stream over the gate matrix (E x H bf16, a few MB): one 128-token tensor-core
// tile walks K serially in a single CTA (34 us at H = 7168, E = 256 against 6 us here at T = 1, 12 us at T = 8), so here the matrix is spread over the device instead: a block
// = 2 experts x 4 quarters of H (one warp each), every warp reads its part of the weight row once and keeps one fp32
// accumulator per token; the four partial sums of an expert are added in a fixed order (reproducible).
template <int TT>
__global__ void __launch_bounds__(256) k_router_logits_small(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                             int T, int H, int E, float* __restrict__ logits) {
  __shared__ float part_sum[4][2][TT];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int el = warp >> 2, part = warp & 3;
  const int e = blockIdx.x * 2 + el;
  pdl_trigger();
  pdl_wait();
  float acc[TT];
#pragma unroll
  for (int t = 0; t < TT; ++t) acc[t] = 0.f;
  if (e < E) {
    const int vecs = H >> 3;
    const uint4* wr = reinterpret_cast<const uint4*>(w + (int64_t)e * H);
    const uint4* xr = reinterpret_cast<const uint4*>(x);
    for (int c = part * 32 + lane; c < vecs; c += 128) {
      const uint4 wv = __ldg(wr + c);
      const uint32_t* ww = reinterpret_cast<const uint32_t*>(&wv);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        wf[2 * i] = __uint_as_float(ww[i] << 16);
        wf[2 * i + 1] = __uint_as_float(ww[i] & 0xFFFF0000u);
      }
#pragma unroll
      for (int t = 0; t < TT; ++t) {
        if (t < T) {
          const uint4 xv = __ldg(xr + (int64_t)t * vecs + c);
          const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[t] = fmaf(__uint_as_float(xw[i] << 16), wf[2 * i], acc[t]);
            acc[t] = fmaf(__uint_as_float(xw[i] & 0xFFFF0000u), wf[2 * i + 1], acc[t]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TT; ++t) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[t] += __shfl_xor_sync(0xFFFFFFFFu, acc[t], off);
    if (lane == 0) part_sum[part][el][t] = acc[t];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * TT; i += blockDim.x) {
    const int ee = i / TT, t = i % TT;
    const int eg = blockIdx.x * 2 + ee;
    if (t < T && eg < E) logits[(int64_t)t * E + eg] = ((part_sum[0][ee][t] + part_sum[1][ee][t]) + part_sum[2][ee][t]) + part_sum[3][ee][t];
  }
}

int launch_router_logits_small(const void* x, const void* w, int64_t T, int H, int E, float* logits, cudaStream_t st) {
  if (T == 0) return 0;
  const dim3 grid((unsigned)((E + 1) / 2));
  if (T <= 8)
    return (int)launch_chain(k_router_logits_small<8>, grid, dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (int)T, H, E,
                             logits);
  return (int)launch_chain(k_router_logits_small<16>, grid, dim3(256), 0, st, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (int)T, H, E,
                           logits);
}

// ----------------------------------------------------------------------------- tensor-core router logits
// Same product on the 5th-gen tensor cores: 128-token tiles, the whole gate matrix (E <= 256 rows) as the B tile,
// K staged 64 bf16 (128 B rows, 128-byte swizzle) at a time by TMA, tcgen05.mma kind::f16 into double-buffered TMEM
// accumulators, fp32 results stored straight from TMEM. Warp roles as in the NVFP4 GEMM.
constexpr int kLgStages = 4;
constexpr int kLgABytes = 128 * 128;
constexpr int kLgBBytes = 256 * 128;
constexpr int kLgSmem = kLgStages * (kLgABytes + kLgBBytes) + 1024 + 128;

__global__ void __launch_bounds__(192, 1)
k_router_logits_tc(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, int T, int H, int E,
                   int e_pad, float* __restrict__ logits, int32_t* status) {
  // e_pad = gate rows of THIS block's tile; blockIdx.y selects which e_pad-row slice of the gate matrix (one slice, or two
  // when a single slice per token tile would leave more than half of the SMs idle)
  const int e0 = (int)blockIdx.y * e_pad;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = base, s_b = s_a + kLgStages * kLgABytes, s_bar = s_b + kLgStages * kLgBBytes;
  const uint32_t bar_full = s_bar, bar_empty = s_bar + 8 * kLgStages, bar_acc_full = bar_empty + 8 * kLgStages,
                 bar_acc_empty = bar_acc_full + 16, s_slot = bar_acc_empty + 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kLgStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 4); }
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc<512>(s_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_slot));
  pdl_trigger();
  pdl_wait();
  const int n_tiles = (T + 127) >> 7;
  const int nk = H >> 6;
  const uint32_t stage_bytes = kLgABytes + (uint32_t)e_pad * 128;
  if (warp == 0) {
    if (lane == 0) {
      uint32_t g = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x)
        for (int ks = 0; ks < nk; ++ks, ++g) {
          const uint32_t s = g % kLgStages;
          if (!mbar_wait(bar_empty + 8 * s, ((g / kLgStages) & 1) ^ 1)) { if (status) atomicCAS(status, 0, 111); ok = false; break; }
          mbar_expect_tx(bar_full + 8 * s, stage_bytes);
          tma_load_2d(s_a + s * kLgABytes, &tm_x, bar_full + 8 * s, ks * 128, tile * 128);
          tma_load_2d(s_b + s * kLgBBytes, &tm_w, bar_full + 8 * s, ks * 128, e0);
        }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, e_pad);
      uint32_t g = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++it) {
        const uint32_t buf = it & 1;
        if (!mbar_wait(bar_acc_empty + 8 * buf, ((it >> 1) & 1) ^ 1)) { if (status) atomicCAS(status, 0, 112); break; }
        tc_fence_after();
        for (int ks = 0; ks < nk; ++ks, ++g) {
          const uint32_t s = g % kLgStages;
          if (!mbar_wait(bar_full + 8 * s, (g / kLgStages) & 1)) { if (status) atomicCAS(status, 0, 113); ok = false; break; }
          tc_fence_after();
          const uint64_t a_d = make_desc_sw128(s_a + s * kLgABytes), b_d = make_desc_sw128(s_b + s * kLgBBytes);
#pragma unroll
          for (int q = 0; q < 4; ++q) mma_bf16(tmem + buf * 256, a_d + 2 * q, b_d + 2 * q, idesc, (ks | q) ? 1u : 0u);
          mma_commit(bar_empty + 8 * s);
        }
        if (ok) mma_commit(bar_acc_full + 8 * buf);
      }
    }
  } else {
    const int quad = warp & 3;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      const uint32_t buf = it & 1;
      int okw = 1;
      if (lane == 0) okw = mbar_wait(bar_acc_full + 8 * buf, (it >> 1) & 1) ? 1 : 0;
      okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
      if (!okw) { if (lane == 0 && status) atomicCAS(status, 0, 114); break; }
      tc_fence_after();
      const int row = tile * 128 + quad * 32 + lane;
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + buf * 256;
      for (int cb = 0; cb < e_pad / 32; ++cb) {
        float v[32];
        tmem_ld32(taddr + cb * 32, v);
        tmem_ld_wait();
        if (row < T) {
          float* dst = logits + (size_t)row * E + e0 + cb * 32;
          if (e0 + cb * 32 + 32 <= E && (E & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (e0 + cb * 32 + j < E) dst[j] = v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tmem_dealloc<512>(tmem); }
}

int launch_router_logits_tc(const void* x, const void* w, int64_t T, int H, int E, float* logits, int32_t* status, cudaStream_t st) {
  if (T == 0) return 0;
  int e_pad = (E + 31) / 32 * 32;
  const int sms = sm_count();
  const int n_tiles = (int)((T + 127) / 128);
  // Every block streams its token tile AND its gate slice once per k-step from L2, at one SM's rate: with at most half of
  // the SMs busy, two blocks per token tile (half of the experts each) halve the gate bytes per block.
  const int n_split = (n_tiles * 2 <= sms && e_pad % 64 == 0) ? 2 : 1;
  e_pad /= n_split;
  CUtensorMap tx, tw;
  int rc = make_operand_map(&tx, x, (uint64_t)T, (uint64_t)H * 2, 128);
  if (rc) return rc;
  rc = make_operand_map(&tw, w, (uint64_t)E, (uint64_t)H * 2, (uint32_t)e_pad);
  if (rc) return rc;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(k_router_logits_tc, kLgSmem)) return e;
  return (int)launch_chain(k_router_logits_tc, dim3(n_tiles < sms ? n_tiles : sms, n_split), dim3(192), kLgSmem, st, tx, tw, (int)T, H, E,
                           e_pad, logits, status);
}

// ----------------------------------------------------------------------------- tensor-core router logits, few token tiles
// A few token tiles: one block per tile walks H / 64 dependent k-steps at one SM's load rate (T = 64, H = 7168, E = 256:
// 35 us for 4.6 MB; 8 us here). A token tile belongs to a CLUSTER of k_split blocks along z, each taking a
// contiguous range of k-steps and (blockIdx.y) a slice of e_slice experts; the partial tiles meet in distributed shared
// memory: block r of the cluster adds rows [128 r / k_split, 128 (r + 1) / k_split) of all partials in rank order
// (reproducible) and stores them. No scratch in global memory, one launch.
constexpr int kLkStages = 8;
constexpr int kLkABytes = 128 * 128;
constexpr int kLkBBytes = 64 * 128;
constexpr int kLkSmem = kLkStages * (kLkABytes + kLkBBytes) + 1024 + 256;

__global__ void __launch_bounds__(192, 1)
k_router_logits_ksplit(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, int T, int H, int E,
                       int e_slice, float* __restrict__ logits, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_a = base, s_b = s_a + kLkStages * kLkABytes, s_bar = s_b + kLkStages * kLkBBytes;
  const uint32_t bar_full = s_bar, bar_empty = s_bar + 8 * kLkStages, bar_acc_full = bar_empty + 8 * kLkStages, s_slot = bar_acc_full + 8;
  const uint32_t s_part = s_a;                    // after the k-loop: this block's partial tile, [e_slice][128] floats
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_split = (int)gridDim.z;
  const uint32_t rank = cluster_ctarank();        // == blockIdx.z: the cluster spans z
  const int tile = (int)blockIdx.x, e0 = (int)blockIdx.y * e_slice;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kLkStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    mbar_init(bar_acc_full, 1);
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc<64>(s_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(s_slot));
  pdl_trigger();
  pdl_wait();
  const int steps = (H >> 6) / k_split, ks0 = (int)rank * steps;
  const uint32_t stage_bytes = kLkABytes + (uint32_t)e_slice * 128;
  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < steps; ++i) {
        const uint32_t s = i % kLkStages;
        if (!mbar_wait(bar_empty + 8 * s, ((i / kLkStages) & 1) ^ 1)) { if (status) atomicCAS(status, 0, 115); break; }
        mbar_expect_tx(bar_full + 8 * s, stage_bytes);
        tma_load_2d(s_a + s * kLkABytes, &tm_x, bar_full + 8 * s, (ks0 + i) * 128, tile * 128);
        tma_load_2d(s_b + s * kLkBBytes, &tm_w, bar_full + 8 * s, (ks0 + i) * 128, e0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, e_slice);
      bool ok = true;
      for (int i = 0; i < steps; ++i) {
        const uint32_t s = i % kLkStages;
        if (!mbar_wait(bar_full + 8 * s, (i / kLkStages) & 1)) { if (status) atomicCAS(status, 0, 116); ok = false; break; }
        tc_fence_after();
        const uint64_t a_d = make_desc_sw128(s_a + s * kLkABytes), b_d = make_desc_sw128(s_b + s * kLkBBytes);
#pragma unroll
        for (int q = 0; q < 4; ++q) mma_bf16(tmem, a_d + 2 * q, b_d + 2 * q, idesc, (i | q) ? 1u : 0u);
        mma_commit(bar_empty + 8 * s);
      }
      if (ok) mma_commit(bar_acc_full);
    }
    __syncwarp();
  } else {
    // accumulator -> this block's partial tile in shared memory, column-major so that the 32 rows of a warp are contiguous
    const int quad = warp & 3;
    int okw = 1;
    if (lane == 0) okw = mbar_wait(bar_acc_full, 0) ? 1 : 0;
    okw = __shfl_sync(0xFFFFFFFFu, okw, 0);
    if (!okw) {
      if (lane == 0 && status) atomicCAS(status, 0, 117);
    } else {
      tc_fence_after();
      const int row = quad * 32 + lane;
      const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
      for (int cb = 0; cb < e_slice / 32; ++cb) {
        float v[32];
        tmem_ld32(taddr + cb * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(s_part + (uint32_t)(((cb * 32 + j) * 128 + row) * 4)), "f"(v[j]) : "memory");
      }
      tc_fence_before();
    }
  }
  cluster_sync_all();                             // every partial tile of the cluster is in place
  {
    const int rows_per = 128 / k_split;
    const int row_base = (int)rank * rows_per;
    for (int i = threadIdx.x; i < rows_per * e_slice; i += blockDim.x) {
      const int r = row_base + i % rows_per, col = i / rows_per;     // rows fastest: neighbouring lanes read neighbouring words
      const uint32_t at = s_part + (uint32_t)((col * 128 + r) * 4);
      float v[8];                                 // all remote loads first (a distributed-shared-memory round trip each), then
#pragma unroll                                    // the sum in rank order
      for (int j = 0; j < 8; ++j) {
        v[j] = 0.f;
        if (j < k_split) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[j]) : "r"(map_to_cta(at, (uint32_t)j)));
      }
      float sum = v[0];
#pragma unroll
      for (int j = 1; j < 8; ++j)
        if (j < k_split) sum += v[j];
      const int row = tile * 128 + r;
      if (row < T && e0 + col < E) logits[(size_t)row * E + e0 + col] = sum;
    }
  }
  cluster_sync_all();                             // nobody leaves while a peer still reads its partial tile
  if (warp == 1) { __syncwarp(); tmem_dealloc<64>(tmem); }
}

// k_split for the cluster form: the largest of 8, 4, 2, 1 that divides the k-steps and keeps the grid within the SMs; 0 = do
// not use it (the grid would not fit one wave, or the shape does not fit).
static int router_ksplit(int64_t T, int H, int E, int* e_slice_out) {
  const int n_tiles = (int)((T + 127) / 128);
  const int e_pad = (E + 31) / 32 * 32;
  if (H % 64 || e_pad > 256) return 0;
  const int e_slice = e_pad % 64 == 0 ? 64 : 32;
  const int slices = e_pad / e_slice;
  const int sms = sm_count();
  for (int ks = 8; ks >= 1; ks >>= 1)            // ks = 1: no split, but 64-expert slices put four blocks on a token tile
    if ((H >> 6) % ks == 0 && n_tiles * slices * ks <= sms) { *e_slice_out = e_slice; return ks; }
  return 0;
}

int launch_router_logits_ksplit(const void* x, const void* w, int64_t T, int H, int E, float* logits, int32_t* status, cudaStream_t st) {
  int e_slice = 0;
  const int k_split = router_ksplit(T, H, E, &e_slice);
  if (!k_split) return -1;                        // caller falls back to the one-block-per-tile kernel
  const int e_pad = (E + 31) / 32 * 32;
  CUtensorMap tx, tw;
  int rc = make_operand_map(&tx, x, (uint64_t)T, (uint64_t)H * 2, 128);
  if (rc) return rc;
  rc = make_operand_map(&tw, w, (uint64_t)E, (uint64_t)H * 2, (uint32_t)e_slice);
  if (rc) return rc;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(k_router_logits_ksplit, kLkSmem)) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((T + 127) / 128), (unsigned)(e_pad / e_slice), (unsigned)k_split);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = kLkSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)k_split;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, k_router_logits_ksplit, tx, tw, (int)T, H, E, e_slice, logits, status);
}

int launch_route_topk(const float* logits, const float* bias, int64_t T, int E, int K, int32_t* ids, float* weights,
                      cudaStream_t st) {
  if (T == 0) return 0;
  const unsigned blocks = (unsigned)((T * 32 + 255) / 256);
  const int per_lane = (E + 31) / 32;
  cudaError_t err;
  if (per_lane <= 1) err = launch_chain(k_route_topk<1>, dim3(blocks), dim3(256), 0, st, logits, bias, T, E, K, ids, weights);
  else if (per_lane <= 2) err = launch_chain(k_route_topk<2>, dim3(blocks), dim3(256), 0, st, logits, bias, T, E, K, ids, weights);
  else if (per_lane <= 4) err = launch_chain(k_route_topk<4>, dim3(blocks), dim3(256), 0, st, logits, bias, T, E, K, ids, weights);
  else if (per_lane <= 8) err = launch_chain(k_route_topk<8>, dim3(blocks), dim3(256), 0, st, logits, bias, T, E, K, ids, weights);
  else if (per_lane <= 16) err = launch_chain(k_route_topk<16>, dim3(blocks), dim3(256), 0, st, logits, bias, T, E, K, ids, weights);
  else err = launch_chain(k_route_topk<32>, dim3(blocks), dim3(256), 0, st, logits, bias, T, E, K, ids, weights);
  return (int)err;
}

int launch_router_logits(const void* x, const void* w, int64_t T, int H, int E, float* logits, cudaStream_t st) {
  if (T == 0) return 0;
  dim3 grid((unsigned)T, (unsigned)((E + 63) / 64));
  k_router_logits<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, T, H, E, logits);
  return (int)cudaGetLastError();
}

}  // namespace b200
