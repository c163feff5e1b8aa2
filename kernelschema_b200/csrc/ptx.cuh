// Inline-PTX wrappers for sm_100a: mbarrier, TMA (non-multicast), tcgen05 (TMEM alloc, cp, mma, ld, commit).
// Every wait is bounded: after kSpinLimit polls it gives up and reports, so a broken pipeline
// ends the kernel with an error status instead of hanging the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DEV __device__ __forceinline__

namespace b200 {

constexpr uint32_t kSpinLimit = 1u << 24;   // polls of try_wait before a wait is declared dead (~ a few seconds)

DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// Programmatic dependent launch: `pdl_trigger` lets the next kernel of the stream start its prologue while this grid is
// still running; `pdl_wait` blocks until every earlier grid of the stream has finished and its writes are visible.
// Every kernel of the layer chain issues both before it touches global memory, so the only overlap is launch latency
// and prologue (barrier init, TMEM allocation, tensor-map prefetch). Both are no-ops in a kernel launched without the
// attribute.
DEV void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
DEV void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

DEV uint32_t lane_id() { return threadIdx.x & 31; }

// ----------------------------------------------------------------------------- mbarrier
DEV void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
DEV void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
DEV void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
DEV void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Returns false when the phase did not complete within the poll limit.
DEV bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// ----------------------------------------------------------------------------- TMA (bulk async copies, never multicast)
DEV void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// TMA tile::gather4: the map's 128-byte box at byte column x of FOUR rows (tensor dim-1 indices r0..r3) lands in four
// consecutive 128-byte shared slots, the map's swizzle applied per destination row. Map: 2-D, box {128, 1}. Local memory
// only, no multicast.
DEV void tma_gather4(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t r0, int32_t r1, int32_t r2, int32_t r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
DEV void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
DEV void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ----------------------------------------------------------------------------- tcgen05 / TMEM
template <int NCOLS>
DEV void tmem_alloc(uint32_t slot_smem) {   // whole warp, converged
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(NCOLS) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int NCOLS>
DEV void tmem_dealloc(uint32_t taddr) {     // whole warp, converged
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
}
DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand tile with 128-byte rows and the 128-byte swizzle:
// start address >> 4 in bits [0,14), stride-byte-offset (8 rows x 128 B = 1024) >> 4 in [32,46),
// descriptor version 1 in [46,48), layout type 2 (SWIZZLE_128B) in [61,64).
DEV uint64_t make_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// Descriptor of one 32-row x 16-byte scale-factor chunk stored contiguously (512 B), no swizzle:
// 8-row core matrices are 128 B apart.
DEV uint64_t make_desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// Instruction descriptor of tcgen05.mma kind::mxf4nvf4 (block scaled): E2M1 x E2M1 (format code 1),
// both operands K-major, UE4M3 scale format (bit 23 = 0), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc_nvf4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem] with per-16-element E4M3 scales read from TMEM.
DEV void mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                  uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// Instruction descriptor of tcgen05.mma kind::f16 with bf16 operands (format 1), fp32 accumulator (format 1 at bit 4).
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
DEV void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 128 bit from shared memory into 4 TMEM columns, replicated to all four lane quadrants.
DEV void tmem_cp_sf(uint32_t dst_tmem, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(sdesc) : "memory");
}
// mbarrier arrive once every tcgen05 op issued so far by this thread has completed.
DEV void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
DEV void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* u = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr)
      : "memory");
}
DEV void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- CTA pairs (cluster of 2, tcgen05 cta_group::2)
DEV uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
DEV void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) inside CTA `rank` of the cluster
DEV uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// No release semantics needed: the bytes announced here are written by TMA, which orders them with its own completion.
DEV void mbar_expect_tx_remote(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}
DEV void mbar_arrive_remote(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Wait with cluster-scope acquire (the arrivals come from the peer CTA).
DEV bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// TMA tile load into this CTA's shared memory whose completion bytes are counted on a barrier that may live in
// the peer CTA of the pair (cluster address). No multicast: every CTA fetches its own tiles.
DEV void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
template <int NCOLS>
DEV void tmem_alloc_pair(uint32_t slot_smem) {   // same warp index in both CTAs, converged
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(NCOLS) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int NCOLS>
DEV void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
}
// 256 x N tile over the CTA pair: each CTA supplies 128 rows of A and N/2 rows of B from its own shared memory
// and owns 128 lanes x N columns of the accumulator. Issued by one thread of the leader CTA.
DEV void mma_nvf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
DEV void tmem_cp_sf_pair(uint32_t dst_tmem, uint64_t sdesc) {   // in each CTA: own shared memory -> own TMEM
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(sdesc) : "memory");
}
// Arrive on one barrier (cluster address, here always the issuing CTA's own) once all tcgen05 ops issued so far are done.
DEV void mma_commit_pair_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Arrive on the barrier at the same shared-memory offset in both CTAs of the pair once all tcgen05 ops issued so far are done.
DEV void mma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
               : "memory");
}

// ----------------------------------------------------------------------------- number formats
// Two fp32 -> one byte of two E2M1 codes, round-to-nearest-even, saturating at 6; `lo` lands in the low nibble.
DEV uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\tcvt.u32.u8 %0, b;\n\t}" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// fp32 (>= 0, <= 448) -> E4M3 byte, round-to-nearest-even.
DEV uint32_t cvt_e4m3(float x) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
  return (uint32_t)(r & 0xFF);
}
// E4M3 byte (sign bit clear) -> fp32, exact.
DEV float e4m3_to_f32(uint32_t b) {
  uint32_t h;
  asm("{\n\t.reg .b16 s;\n\tcvt.u16.u32 s, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, s;\n\t}" : "=r"(h) : "r"(b & 0xFFu));
  return __half2float(__ushort_as_half((unsigned short)(h & 0xFFFF)));
}

// Routing-weighted sum of one 16-byte vector (8 bf16 columns) over a token's KK slots, fp32, slots in ascending order
// (slots without a row are skipped). Eight slots at a time: their row indices, then their weights, then their vectors are
// each fetched as one batch, so a token costs three dependent memory round trips per eight slots instead of two per slot.
DEV void combine_slots(const __nv_bfloat16* __restrict__ rout, const int32_t* __restrict__ slots, const float* __restrict__ weight_of_row,
                       int KK, int H, int v, float (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < KK; k0 += 8) {
    int row[8];
    float w[8];
    uint4 raw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) row[j] = k0 + j < KK ? slots[k0 + j] : -1;
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = row[j] >= 0 ? weight_of_row[row[j]] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (row[j] >= 0) raw[j] = __ldg(reinterpret_cast<const uint4*>(rout + (size_t)row[j] * H) + v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (row[j] < 0) continue;
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw[j]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] = fmaf(__uint_as_float(u[i] << 16), w[j], acc[2 * i]);
        acc[2 * i + 1] = fmaf(__uint_as_float(u[i] & 0xFFFF0000u), w[j], acc[2 * i + 1]);
      }
    }
  }
}

DEV uint4 pack_bf16x8(const float (&acc)[8]) {
  uint4 o;
  uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    ou[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return o;
}

// One payload row by one warp, eight 16-byte vectors per lane in flight (all loads of a batch before its stores).
DEV void copy_row_batched(const uint4* __restrict__ src, uint4* __restrict__ dst, int vecs, int lane) {
  for (int v0 = lane; v0 < vecs; v0 += 32 * 8) {
    uint4 t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v0 + 32 * i < vecs) t[i] = __ldg(src + v0 + 32 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v0 + 32 * i < vecs) dst[v0 + 32 * i] = t[i];
  }
}

}  // namespace b200
