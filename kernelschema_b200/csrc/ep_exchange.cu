// Expert-parallel exchange over peer memory (NVLink): token rows travel to the ranks that own their experts and the
// partial results travel back as plain peer stores issued by this library's own kernels; completion is signalled by
// release stores of a step counter into the receiver's control block, which the receiver polls with acquire loads.
//
// The reference operator has no multi-GPU path (it only carries local_expert_offset / local_num_experts in its ABI,
// candidate/nvfp4_moe.cu:595-596). The nearest model in the reference catalogue is the in-kernel exchange of the bf16
// MoE sibling (moe/bf16_fused_moe/candidate/kernel.cuh:365-395 dispatch by remote stores, :1072-1168 results written
// straight into the source rank's combine buffer, :1224-1259 release/acquire readiness flags). Unlike that code every
// wait here is bounded: after kEpSpinLimit polls it records a status code and carries on, nothing traps.
//
// Memory model of one step (epoch e, parity p = e & 1; every buffer exists twice so that a rank one step ahead never
// overwrites what a slower peer still reads):
//   dispatch   source s -> dest d: message rows into region s of d's receive buffer (fixed region of seg_len rows),
//              then {rows sent, base row of this segment in s's return buffer} into d's control block, then
//              flag_dispatch[s] = e (release.sys) by the last block to finish.
//   experts    d waits for every flag_dispatch (acquire.sys), runs the ordinary layer over the W * seg_len token slots of
//              its receive buffer; slots past a region's row count are invalid. The combine pass writes one bf16 row
//              per received message straight into the source's return buffer (peer stores), then flag_return[d] = e.
//   combine    s waits for every flag_return and adds its rows in slot order.
// Only local memory is ever read by TMA or by a spin loop: peers write, owners read.
#include "kernels.cuh"
#include "ptx.cuh"

namespace b200 {

constexpr uint32_t kEpSpinLimit = 1u << 21;    // polls (with a short sleep between them) before a wait is given up: ~1 s

DEV void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
DEV int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One message row per (token, destination rank) pair of the plan's route map (whose "experts" are the ranks), written
// into the destination's receive buffer: [payload H/2 | scale bytes H/16 | K expert ids local to the destination (-1 =
// lives elsewhere; all -1 on padding rows) | K routing weights]. One warp per row. Also points the plan's shared-expert
// slot of every token at a fixed row of the return buffer, and - by the last block to finish - publishes the segment
// sizes and the dispatch flags.
__global__ void __launch_bounds__(256) k_ep_dispatch(const uint8_t* __restrict__ hid_q, const uint8_t* __restrict__ hid_sf,
                                                     const int32_t* __restrict__ ids, const float* __restrict__ weights,
                                                     const int32_t* __restrict__ tok_of_row, const int32_t* __restrict__ tile_expert,
                                                     const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ seg_start,
                                                     const int32_t* __restrict__ totals, int H, int K, int experts_per_rank,
                                                     int64_t row_bytes, EpPeers peers, int epoch, int64_t T, int shared_slots,
                                                     int shared_base, int32_t* __restrict__ row_of, float* __restrict__ weight_of_row,
                                                     unsigned int* __restrict__ done_counter) {
  const int world = peers.world;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int q_vecs = H >> 5, sf_words = H >> 6;
  // Message rows are grouped by destination. Every rank starts with the segment of the rank after itself and wraps around:
  // walked from row 0 by all ranks at once, all of them would write into rank 0 first, then into rank 1, ... and a
  // destination's inbound link would carry the traffic of the whole machine while the other links idle.
  const int n_msg = seg_start[world];              // rows of the rank segments; the plan's shared-expert slot follows them
  const int first = seg_start[(peers.rank + 1) % world];
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n_msg; i += warps) {
    int r = i + first;
    if (r >= n_msg) r -= n_msg;
    const int dest = tile_expert[r >> 7];
    uint8_t* dst = peers.recv[dest] + (size_t)(r - seg_start[dest]) * row_bytes;
    int32_t* id_dst = reinterpret_cast<int32_t*>(dst + (H >> 1) + (H >> 4));
    float* w_dst = reinterpret_cast<float*>(id_dst + K);
    const bool live = (r & 127) < tile_rows[r >> 7];
    if (!live) {
      if (lane < K) id_dst[lane] = -1;
      continue;
    }
    const int tok = tok_of_row[r];
    copy_row_batched(reinterpret_cast<const uint4*>(hid_q + (size_t)tok * (H >> 1)), reinterpret_cast<uint4*>(dst), q_vecs, lane);
    const uint32_t* sf_src = reinterpret_cast<const uint32_t*>(hid_sf + (size_t)tok * (H >> 4));
    for (int w = lane; w < sf_words; w += 32) reinterpret_cast<uint32_t*>(dst + (H >> 1))[w] = __ldg(sf_src + w);
    if (lane < K) {
      const int g = ids[(size_t)tok * K + lane];
      const bool here = g >= 0 && g / experts_per_rank == dest;
      id_dst[lane] = here ? g - dest * experts_per_rank : -1;
      w_dst[lane] = weights[(size_t)tok * K + lane];
    }
  }
  // the shared experts' rows of this rank's own tokens live at fixed rows of the return buffer, weight 1
  if (shared_slots)
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < T; t += (int64_t)gridDim.x * blockDim.x) {
      row_of[t * (world + 1) + world] = shared_base + (int)t;
      weight_of_row[shared_base + t] = 1.0f;
    }
  // every block: make its peer stores visible system-wide, then count itself; the last one publishes
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;               // ready for the next call on this stream
      __threadfence_system();
      for (int d = 0; d < world; ++d) {
        int32_t* c = peers.ctrl[d];
        c[kEpCount + peers.rank] = seg_start[d + 1] - seg_start[d];
        c[kEpRetBase + peers.rank] = seg_start[d];
        st_release_sys(c + kEpFlagDispatch + peers.rank, epoch);
      }
    }
  }
}

// Thread i < n waits until flags[i] >= epoch (the flags live in THIS rank's memory; peers write them).
__global__ void k_ep_wait(const int32_t* __restrict__ flags, int n, int epoch, int32_t* status, int code) {
  const int i = threadIdx.x;
  if (i >= n) return;
  for (uint32_t it = 0; it < kEpSpinLimit; ++it) {
    if (ld_acquire_sys(flags + i) >= epoch) return;
    __nanosleep(200);
  }
  if (status) atomicCAS(status, 0, code);
}

// After the kernels whose peer stores it covers (stream order): flag field `field` of every peer's control block.
__global__ void k_ep_post(EpPeers peers, int field, int epoch) {
  const int d = threadIdx.x;
  if (d >= peers.world) return;
  __threadfence_system();
  st_release_sys(peers.ctrl[d] + field + peers.rank, epoch);
}

// Routing-weighted combine over this rank's experts of every received message row (as k_finalize: per-route bf16 rows,
// fp32 sum in slot order, one bf16 rounding), written straight into the return buffer of the row's source rank.
// Token slot t = (source s, position i) with s = t / seg_len; slots past the source's row count are skipped.
__global__ void __launch_bounds__(128) k_finalize_ep(const __nv_bfloat16* __restrict__ rout, const int32_t* __restrict__ row_of,
                                                     const float* __restrict__ weight_of_row, int64_t T, int KK, int H, EpPeers peers,
                                                     const int32_t* __restrict__ ctrl, int seg_len) {
  const int vecs = H >> 3;
  pdl_trigger();
  pdl_wait();
  // sources are visited starting with the rank after this one (see k_ep_dispatch: all ranks returning rows to the same source
  // at the same time would share that source's inbound link)
  const int64_t first = (int64_t)((peers.rank + 1) % peers.world) * seg_len;
  for (int64_t tt = blockIdx.x; tt < T; tt += gridDim.x) {
    const int64_t t = tt + first < T ? tt + first : tt + first - T;
    const int s = (int)(t / seg_len);
    const int i = (int)(t - (int64_t)s * seg_len);
    if (i >= ctrl[kEpCount + s]) continue;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(peers.ret[s]) + (size_t)(ctrl[kEpRetBase + s] + i) * H;
    for (int v = blockIdx.y * blockDim.x + threadIdx.x; v < vecs; v += gridDim.y * blockDim.x) {
      float acc[8];
      combine_slots(rout, row_of + t * KK, weight_of_row, KK, H, v, acc);
      *(reinterpret_cast<uint4*>(out) + v) = pack_bf16x8(acc);
    }
  }
}

int launch_ep_dispatch(const void* hid_q, const void* hid_sf, const int32_t* ids, const float* weights, const int32_t* tok_of_row,
                       const int32_t* tile_expert, const int32_t* tile_rows, const int32_t* seg_start, const int32_t* totals, int H,
                       int K, int experts_per_rank, int64_t row_bytes, int64_t row_capacity, const EpPeers& peers, int epoch, int64_t T,
                       int shared_slots, int shared_base, int32_t* row_of, float* weight_of_row, unsigned int* done_counter,
                       cudaStream_t st) {
  int64_t blocks = (row_capacity + 7) / 8;
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  k_ep_dispatch<<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)hid_q, (const uint8_t*)hid_sf, ids, weights, tok_of_row, tile_expert,
                                                 tile_rows, seg_start, totals, H, K, experts_per_rank, row_bytes, peers, epoch, T,
                                                 shared_slots, shared_base, row_of, weight_of_row, done_counter);
  return (int)cudaGetLastError();
}

int launch_ep_wait(const int32_t* flags, int n, int epoch, int32_t* status, int code, cudaStream_t st) {
  k_ep_wait<<<1, 32, 0, st>>>(flags, n, epoch, status, code);
  return (int)cudaGetLastError();
}

int launch_ep_post(const EpPeers& peers, int field, int epoch, cudaStream_t st) {
  k_ep_post<<<1, 32, 0, st>>>(peers, field, epoch);
  return (int)cudaGetLastError();
}

int launch_finalize_ep(const void* rout, const int32_t* row_of, const float* weight_of_row, int64_t T, int KK, int H,
                       const EpPeers& peers, const int32_t* ctrl, int seg_len, cudaStream_t st) {
  if (T == 0) return 0;
  const int sms = sm_count();
  const int64_t blocks = T < sms * 16 ? T : sms * 16;
  const int chunks = (H / 8 + 127) / 128;
  const int by = blocks >= sms * 4 ? 1 : (int)(chunks < (sms * 4 + blocks - 1) / blocks ? chunks : (sms * 4 + blocks - 1) / blocks);
  return (int)launch_chain(k_finalize_ep, dim3((unsigned)blocks, (unsigned)by), dim3(128), 0, st, (const __nv_bfloat16*)rout, row_of,
                           weight_of_row, T, KK, H, peers, ctrl, seg_len);
}

}  // namespace b200
