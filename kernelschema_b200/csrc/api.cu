// C-ABI layer of libb200moe: argument checks, workspace ownership, tensor-map cache and the launch chain.
// Declarations and the reference interfaces they replace are in include/b200moe.h.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/b200moe.h"
#include "kernels.cuh"

using namespace b200;

namespace b200 {
int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 64) {
    const int v = cached[dev].load(std::memory_order_relaxed);
    if (v > 0) return v;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
  if (dev < 64) cached[dev].store(sms, std::memory_order_relaxed);
  return sms;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("B200MOE_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}
}  // namespace b200

static thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
static int cuda_fail(int code, const char* what) {
  if (code == 0) return 0;
  if (code < 700)
    return fail(code, "%s: CUDA error %d (%s)", what, code, cudaGetErrorString((cudaError_t)code));
  return fail(code, "%s: refused with code %d", what, code);
}

struct b200moe_layer {
  b200moe_config cfg;
  int etot;              // E + S
  int kk;                // top_k + S
  int64_t row_capacity;  // permuted rows
  int64_t tile_capacity;
  int sm_count;
  int bn;
  void* base;            // one cudaMalloc
  int64_t bytes;
  RouteMapBuffers rm;
  uint8_t *a_q, *a_sf, *act_q, *act_sf;
  __nv_bfloat16* rout;
  int32_t* status;
  CUtensorMap tm_a1, tm_a2, tm_b1, tm_b2;
  CUtensorMap tm_b1_narrow, tm_b2_narrow;
  CUtensorMap tm_hid;                                 // the caller's token rows as FC1's A operand (TMA gather), box {128, 1}
  const void* hid_ptr;
  int64_t hid_stride;
  uint8_t *step_hq, *step_hs;                         // b200moe_step: quantised tokens,
  float* step_logits;                                 //               router logits,
  int32_t* step_ids;                                  //               selected experts
  float* step_w;                                      //               and their weights             // weight maps with 128-row boxes: small batches run 128 x 128 tiles
  CUtensorMap tm_sfa1, tm_sfa2, tm_sfb1, tm_sfb2;   // scale-factor maps of the CTA-pair GEMM
  int n_clusters;                                    // CTA pairs that can be co-resident
  const void* b1_ptr;
  const void* b2_ptr;
  const void* s1_ptr;
  const void* s2_ptr;
  // graph cache of b200moe_run (cfg.graph_cache): entries keyed on the whole argument block and the stream
  struct Cached {
    uint8_t key[320];         // the argument block of b200moe_run or b200moe_step, fields copied into a zeroed buffer
    int key_bytes;
    cudaStream_t stream;
    cudaGraphExec_t exec;     // null: the key was seen once, the next identical call captures
    uint64_t last_use;
  } cache[4];
  uint64_t tick;
  cudaStream_t capture_stream;   // only ever captured on, never executed on: the caller's stream may be the legacy default
  cudaStream_t side_stream;      // b200moe_step: the quantiser runs here, beside the router kernels on the caller's stream
  cudaEvent_t ev_fork, ev_join;
  b200moe_stats stats;
};

namespace {

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct Plan {
  int64_t row_capacity, tile_capacity, nblk;
  int64_t off_block_hist, off_counts, off_seg, off_texp, off_trow0, off_trows, off_pexp, off_prow0, off_prows, off_totals, off_row_of, off_tok, off_w, off_aq,
      off_asf, off_actq, off_actsf, off_rout, off_status, off_step_hq, off_step_hs, off_step_logits, off_step_ids, off_step_w, total;
};

int check_cfg(const b200moe_config* c) {
  if (!c || c->struct_size != (int32_t)sizeof(b200moe_config)) return fail(710, "config: bad struct_size");
  if (c->hidden <= 0 || c->hidden % 256) return fail(711, "config: hidden=%d must be a positive multiple of 256", c->hidden);
  if (c->intermediate <= 0 || c->intermediate % 256)
    return fail(712, "config: intermediate=%d must be a positive multiple of 256", c->intermediate);
  if (c->num_experts < 0 || c->num_shared_experts < 0 || c->num_experts + c->num_shared_experts <= 0 ||
      c->num_experts + c->num_shared_experts > 1024)
    return fail(713, "config: num_experts + num_shared_experts must be in 1..1024");
  if (c->top_k < 0 || c->top_k > 32 || c->top_k + c->num_shared_experts <= 0) return fail(714, "config: top_k out of range");
  if (c->max_tokens <= 0) return fail(715, "config: max_tokens must be positive");
  if (c->sm_margin < 0 || c->sm_margin > 64) return fail(708, "config: sm_margin must be in 0..64");
  if (c->tile_n != 0 && c->tile_n != 128 && c->tile_n != 256 && c->tile_n != 512)
    return fail(716, "config: tile_n must be 0, 128, 256 or 512");
  if (c->graph_cache != 0 && c->graph_cache != 1) return fail(709, "config: graph_cache must be 0 or 1");
  if (c->tma_gather != 0 && c->tma_gather != 1) return fail(707, "config: tma_gather must be 0 or 1");
  return 0;
}

Plan make_plan(const b200moe_config& c) {
  Plan p;
  const int64_t etot = c.num_experts + c.num_shared_experts, kk = c.top_k + c.num_shared_experts;
  const int64_t routes = (int64_t)c.max_tokens * kk;
  // an expert with c routes owns ceil(c/128) <= c/128 + 1 tiles, so this bounds every routing
  p.tile_capacity = routes / 128 + etot + 1;
  p.row_capacity = p.tile_capacity * 128;
  p.nblk = (routes + 2047) / 2048;
  int64_t o = 0;
  auto take = [&](int64_t bytes) { int64_t at = o; o = align_up(o + bytes, 1024); return at; };
  p.off_block_hist = take(4 * (p.nblk + 1) * etot);
  p.off_counts = take(4 * etot);
  p.off_seg = take(4 * (etot + 1));
  p.off_texp = take(4 * p.tile_capacity);
  p.off_trow0 = take(4 * p.tile_capacity);
  p.off_trows = take(4 * p.tile_capacity);
  p.off_pexp = take(4 * p.tile_capacity);
  p.off_prow0 = take(4 * p.tile_capacity);
  p.off_prows = take(4 * p.tile_capacity);
  p.off_totals = take(16);
  p.off_row_of = take(4 * routes);
  p.off_tok = take(4 * p.row_capacity);
  p.off_w = take(4 * p.row_capacity);
  p.off_aq = take(p.row_capacity * (c.hidden / 2));
  p.off_asf = take(p.row_capacity * (c.hidden / 16));
  p.off_actq = take(p.row_capacity * (c.intermediate / 2));
  p.off_actsf = take(p.row_capacity * (c.intermediate / 16));
  p.off_rout = take(p.row_capacity * c.hidden * 2);
  p.off_status = take(16);
  // buffers of b200moe_step (bf16 tokens in): NVFP4 tokens, router logits over the routed experts, top-k ids and weights
  p.off_step_hq = take((int64_t)c.max_tokens * (c.hidden / 2));
  p.off_step_hs = take((int64_t)c.max_tokens * (c.hidden / 16));
  p.off_step_logits = take((int64_t)c.max_tokens * (c.num_experts > 0 ? c.num_experts : 1) * 4);
  p.off_step_ids = take((int64_t)c.max_tokens * (c.top_k > 0 ? c.top_k : 1) * 4);
  p.off_step_w = take((int64_t)c.max_tokens * (c.top_k > 0 ? c.top_k : 1) * 4);
  p.total = o;
  return p;
}

int check_args(const b200moe_layer* h, const b200moe_args* a) {
  if (!h) return fail(720, "run: null handle");
  if (!a || a->struct_size != (int32_t)sizeof(b200moe_args)) return fail(721, "run: bad args struct_size");
  if (a->num_tokens < 0 || a->num_tokens > h->cfg.max_tokens)
    return fail(722, "run: num_tokens=%d outside 0..max_tokens=%d", a->num_tokens, h->cfg.max_tokens);
  if (a->num_tokens == 0) return 0;
  if (h->cfg.top_k > 0 && (!a->topk_ids || !a->topk_weights)) return fail(723, "run: topk_ids / topk_weights are null");
  if (!a->hidden_states || !a->hidden_states_scale) return fail(724, "run: hidden_states / hidden_states_scale are null");
  if (a->hidden_states_scale_layout != 2 && a->hidden_states_scale_layout != 1)
    return fail(725, "run: hidden_states_scale_layout=%d, expected 2 (row-major) or 1 (tiled)", a->hidden_states_scale_layout);
  if (!a->gemm1_weights || !a->gemm1_weights_scale || !a->gemm2_weights || !a->gemm2_weights_scale)
    return fail(726, "run: weight pointers are null");
  if (a->activation_type != 3 && a->activation_type != 10)
    return fail(727, "run: activation_type=%d, expected 3 or 10", a->activation_type);
  if (!a->output) return fail(728, "run: output is null");
  if (a->output_stride < h->cfg.hidden || a->output_stride % 8)
    return fail(729, "run: output_stride=%lld must be >= hidden and a multiple of 8", (long long)a->output_stride);
  if (((uintptr_t)a->output | (uintptr_t)a->hidden_states | (uintptr_t)a->gemm1_weights | (uintptr_t)a->gemm2_weights |
       (uintptr_t)a->gemm1_weights_scale | (uintptr_t)a->gemm2_weights_scale) & 15)
    return fail(730, "run: tensors must be 16-byte aligned");
  if (((uintptr_t)a->hidden_states_scale) & 3) return fail(731, "run: hidden_states_scale must be 4-byte aligned");
  if (a->hidden_states_stride < 0 || a->hidden_states_stride % 16 || (a->hidden_states_stride && a->hidden_states_stride < h->cfg.hidden / 2))
    return fail(735, "run: hidden_states_stride must be 0 or a multiple of 16 >= hidden/2 bytes");
  if (a->hidden_states_scale_stride < 0 || a->hidden_states_scale_stride % 4 ||
      (a->hidden_states_scale_stride && a->hidden_states_scale_stride < h->cfg.hidden / 16) ||
      (a->hidden_states_scale_stride && a->hidden_states_scale_layout != 2))
    return fail(736, "run: hidden_states_scale_stride must be 0 or a multiple of 4 >= hidden/16 bytes (row-major scales only)");
  if (a->topk_stride < 0 || (a->topk_stride && a->topk_stride < h->cfg.top_k)) return fail(737, "run: topk_stride must be 0 or >= top_k");
  if (a->direct_rows && (h->cfg.top_k != 1 || h->cfg.num_shared_experts != 0))
    return fail(733, "run: direct_rows needs top_k == 1 and no shared experts");
  if (a->direct_rows && (((uintptr_t)a->output & 31) || a->output_stride % 16))
    return fail(734, "run: direct_rows needs a 32-byte aligned output with output_stride %% 16 == 0");
  return 0;
}

struct EpRun {
  EpPeers peers;
  const int32_t* ctrl;     // this rank's control block of the step's parity
  int seg_len;
};

int run_impl(b200moe_layer* h, const b200moe_args* a, cudaStream_t st, cudaEvent_t* ev, const EpRun* ep = nullptr) {
  const b200moe_config& c = h->cfg;
  const int T = a->num_tokens;
  if (T == 0) return 0;
  int rc;
  auto mark = [&](int i) { if (ev) cudaEventRecord(ev[i], st); };
  // cfg.tma_gather: FC1 fetches its A rows from the caller's token matrix by TMA gather and the permute moves only the
  // scale rows; otherwise (and always for the CTA-pair GEMM) the permute also copies the payload rows.
  const bool gather_a = c.tma_gather && h->bn != 512;
  uint8_t* const a_q = gather_a ? nullptr : h->a_q;
  mark(0);
  if (a->hidden_states_scale_layout == 2 && route_gather_fits(T, c.top_k, c.num_shared_experts, c.num_experts, c.hidden)) {
    // decode-sized batch: the route map and the permute are one launch
    rc = launch_route_gather(a->topk_ids, a->topk_weights, a->topk_stride, T, c.top_k, c.num_shared_experts, c.num_experts,
                             a->local_expert_offset, h->rm, a->hidden_states, a->hidden_states_scale, a->hidden_states_stride,
                             a->hidden_states_scale_stride, c.hidden, a_q, h->a_sf, st, ep ? ep->seg_len : 0,
                             ep ? ep->ctrl + kEpCount : nullptr);
    if (rc) return cuda_fail(rc, "route map + permute");
    mark(1);
    mark(2);
  } else {
    rc = launch_route_map(a->topk_ids, a->topk_weights, a->topk_stride, T, c.top_k, c.num_shared_experts, c.num_experts,
                          a->local_expert_offset, h->rm, st, ep ? ep->seg_len : 0, ep ? ep->ctrl + kEpCount : nullptr);
    if (rc) return cuda_fail(rc, "route map");
    mark(1);
    // rows this call can occupy at most (every routing of T tokens fits), not the layer's capacity: sizes the permute grid
    int64_t call_rows = ((int64_t)T * h->kk / 128 + h->etot + 1) * 128;
    if (call_rows > h->row_capacity) call_rows = h->row_capacity;
    rc = launch_gather_rows(a->hidden_states, a->hidden_states_scale, a->hidden_states_scale_layout == 1, a->hidden_states_stride,
                            a->hidden_states_scale_stride, h->rm.tok_of_row, h->rm.tile_rows, h->rm.totals, c.hidden, call_rows, a_q, h->a_sf, st);
    if (rc) return cuda_fail(rc, "permute");
    mark(2);
  }
  if (gather_a && (h->hid_ptr != a->hidden_states || h->hid_stride != a->hidden_states_stride)) {
    rc = make_operand_map(&h->tm_hid, a->hidden_states, (uint64_t)c.max_tokens, c.hidden / 2, 1, (uint64_t)a->hidden_states_stride);
    if (rc) return cuda_fail(rc, "token tensor map");
    h->hid_ptr = a->hidden_states;
    h->hid_stride = a->hidden_states_stride;
  }
  if (h->b1_ptr != a->gemm1_weights || h->s1_ptr != a->gemm1_weights_scale) {
    rc = make_operand_map(&h->tm_b1, a->gemm1_weights, (uint64_t)h->etot * 2 * c.intermediate, c.hidden / 2, h->bn == 512 ? 128 : h->bn);
    if (!rc) rc = make_operand_map(&h->tm_b1_narrow, a->gemm1_weights, (uint64_t)h->etot * 2 * c.intermediate, c.hidden / 2, 128);
    if (!rc && h->bn == 512)
      rc = make_sf_map(&h->tm_sfb1, a->gemm1_weights_scale, (uint64_t)h->etot * 2 * c.intermediate / 128 * (c.hidden / 64));
    if (rc) return cuda_fail(rc, "FC1 weight tensor map");
    h->b1_ptr = a->gemm1_weights;
    h->s1_ptr = a->gemm1_weights_scale;
  }
  if (h->b2_ptr != a->gemm2_weights || h->s2_ptr != a->gemm2_weights_scale) {
    rc = make_operand_map(&h->tm_b2, a->gemm2_weights, (uint64_t)h->etot * c.hidden, c.intermediate / 2, h->bn == 512 ? 128 : h->bn);
    if (!rc) rc = make_operand_map(&h->tm_b2_narrow, a->gemm2_weights, (uint64_t)h->etot * c.hidden, c.intermediate / 2, 128);
    if (!rc && h->bn == 512)
      rc = make_sf_map(&h->tm_sfb2, a->gemm2_weights_scale, (uint64_t)h->etot * c.hidden / 128 * (c.intermediate / 64));
    if (rc) return cuda_fail(rc, "FC2 weight tensor map");
    h->b2_ptr = a->gemm2_weights;
    h->s2_ptr = a->gemm2_weights_scale;
  }
  GemmParams g;
  memset(&g, 0, sizeof(g));
  g.tile_expert = h->rm.tile_expert;
  g.tile_row0 = h->rm.tile_row0;
  g.tile_rows = h->rm.tile_rows;
  g.n_tiles_ptr = h->rm.totals;
  g.status = h->status;
  g.rows_hint = (int64_t)T * h->kk;
  // FC1: [rows, H] x [2I, H]^T -> activation -> NVFP4 [rows, I]
  g.N = 2 * c.intermediate;
  g.K = c.hidden;
  g.sfa = h->a_sf;
  g.a_tok = gather_a ? h->rm.tok_of_row : nullptr;
  g.sfb = (const uint8_t*)a->gemm1_weights_scale;
  g.act_q = h->act_q;
  g.act_sf = h->act_sf;
  g.scale_up = a->output1_scale_scalar;
  g.scale_gate = a->output1_scale_gate_scalar;
  g.alpha = a->gemm1_alpha;
  g.beta = a->gemm1_beta;
  g.limit = a->gemm1_clamp_limit;
  g.act_type = a->activation_type;
  // m-tiles of this call at most: an expert with c routes owns ceil(c / 128) tiles, and no more experts are touched than
  // there are routes. Small batches (decode) are bound by how fast ONE SM can pull its item's weights: when 256-wide
  // tiles would leave half of the SMs without an item, 128-wide tiles double the number of SMs that stream.
  const int64_t routes = (int64_t)T * h->kk;
  const int64_t worst_tiles = routes / 128 + (routes < h->etot ? routes : (int64_t)h->etot);
  auto tile_n_for = [&](int n_cols) {
    if (h->bn != 256 || c.tile_n != 0) return h->bn;
    return worst_tiles * (n_cols / 256) * 2 <= h->sm_count ? 128 : 256;
  };
  {
    const int bn = tile_n_for(g.N);
    const int64_t items = worst_tiles * (g.N / (bn == 512 ? 256 : bn));
    const int grid = (int)(items < h->sm_count ? items : h->sm_count);
    if (bn == 512) {
      GemmParams gp = g;
      gp.tile_expert = h->rm.pair_expert;
      gp.tile_row0 = h->rm.pair_row0;
      gp.tile_rows = h->rm.pair_rows;
      gp.n_tiles_ptr = h->rm.totals + 3;
      rc = launch_gemm_nvfp4_pair(kGemmFc1, h->tm_a1, h->tm_b1, h->tm_sfa1, h->tm_sfb1, gp,
                                  (int)(items < h->n_clusters ? items : h->n_clusters), st);
    } else {
      rc = launch_gemm_nvfp4(kGemmFc1, bn, gather_a ? h->tm_hid : h->tm_a1, bn == h->bn ? h->tm_b1 : h->tm_b1_narrow, g, grid, st);
    }
    if (rc) return cuda_fail(rc, "FC1");
  }
  mark(3);
  // FC2: [rows, I] x [H, I]^T -> bf16 [rows, H]
  g.a_tok = nullptr;
  g.N = c.hidden;
  g.K = c.intermediate;
  g.sfa = h->act_sf;
  g.sfb = (const uint8_t*)a->gemm2_weights_scale;
  g.out = h->rout;
  g.out_stride = c.hidden;
  g.out_scale = a->output2_scale_scalar;
  if (a->direct_rows) {
    g.out = (__nv_bfloat16*)a->output;
    g.out_stride = a->output_stride;
    g.out_row_index = h->rm.tok_of_row;
  }
  {
    const int bn = tile_n_for(g.N);
    const int64_t items = worst_tiles * (g.N / (bn == 512 ? 256 : bn));
    const int grid = (int)(items < h->sm_count ? items : h->sm_count);
    if (bn == 512) {
      GemmParams gp = g;
      gp.tile_expert = h->rm.pair_expert;
      gp.tile_row0 = h->rm.pair_row0;
      gp.tile_rows = h->rm.pair_rows;
      gp.n_tiles_ptr = h->rm.totals + 3;
      rc = launch_gemm_nvfp4_pair(kGemmFc2, h->tm_a2, h->tm_b2, h->tm_sfa2, h->tm_sfb2, gp,
                                  (int)(items < h->n_clusters ? items : h->n_clusters), st);
    } else {
      rc = launch_gemm_nvfp4(kGemmFc2, bn, h->tm_a2, bn == h->bn ? h->tm_b2 : h->tm_b2_narrow, g, grid, st);
    }
    if (rc) return cuda_fail(rc, "FC2");
  }
  mark(4);
  if (a->direct_rows) {
    mark(5);
    return 0;
  }
  if (ep)
    rc = launch_finalize_ep(h->rout, h->rm.row_of, h->rm.weight_of_row, T, h->kk, c.hidden, ep->peers, ep->ctrl, ep->seg_len, st);
  else
    rc = launch_finalize(h->rout, h->rm.row_of, h->rm.weight_of_row, T, h->kk, c.hidden, a->output, a->output_stride, st);
  if (rc) return cuda_fail(rc, "combine");
  mark(5);
  return 0;
}

}  // namespace

extern "C" {

int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }
const char* b200moe_last_error(void) { return g_err; }

int b200moe_quantize_nvfp4(const void* x, int64_t rows, int64_t cols, int64_t row_stride, float global_scale, void* payload,
                           void* scales, int32_t scale_layout, void* stream) {
  if (rows < 0 || cols <= 0 || cols % 64) return fail(740, "quantize: cols=%lld must be a positive multiple of 64", (long long)cols);
  if (row_stride < cols || row_stride % 8) return fail(741, "quantize: row_stride must be >= cols and a multiple of 8");
  if (rows && (!x || !payload || !scales)) return fail(742, "quantize: null pointer");
  if (((uintptr_t)x & 15) || ((uintptr_t)payload & 7)) return fail(743, "quantize: x must be 16-byte and payload 8-byte aligned");
  if (!(global_scale > 0.f)) return fail(744, "quantize: global_scale must be positive");
  if (scale_layout != B200MOE_SF_ROW_MAJOR && scale_layout != B200MOE_SF_TILED) return fail(745, "quantize: unknown scale_layout");
  return cuda_fail(launch_quantize_nvfp4(x, rows, cols, row_stride, global_scale, payload, scales, scale_layout, (cudaStream_t)stream),
                   "quantize");
}

int b200moe_scales_to_tiles(const void* src, int64_t rows, int64_t cols, void* dst, void* stream) {
  if (rows < 0 || cols <= 0 || cols % 64) return fail(746, "scales_to_tiles: cols must be a positive multiple of 64");
  if (rows && (!src || !dst)) return fail(747, "scales_to_tiles: null pointer");
  if (((uintptr_t)src & 3) || ((uintptr_t)dst & 15)) return fail(748, "scales_to_tiles: misaligned pointer");
  return cuda_fail(launch_sf_to_tiles(src, rows, cols / 16, dst, (cudaStream_t)stream), "scales_to_tiles");
}

int b200moe_route_topk(const float* logits, const float* bias, int64_t T, int32_t E, int32_t K, int32_t* ids, float* weights,
                       void* stream) {
  if (T < 0 || E <= 0 || E > 1024 || K <= 0 || K > 32 || K > E) return fail(750, "route_topk: need 0 < K <= min(E, 32), E <= 1024");
  if (T && (!logits || !ids || !weights)) return fail(751, "route_topk: null pointer");
  return cuda_fail(launch_route_topk(logits, bias, T, E, K, ids, weights, (cudaStream_t)stream), "route_topk");
}

static int router_logits_any(const void* x, const void* w, int64_t T, int H, int E, float* logits, cudaStream_t st) {
  // A handful of tokens: the SIMT kernel streams the gate matrix over the whole device (T = 1: 2.4 us at H 2048 / E 128, 6 us
  // at H 7168 / E 256; its cost grows with T, and from T x H ~ 32K elements on the cluster kernel below is faster: 5.5 / 8.3 us
  // up to 256 tokens). It also serves shapes the tensor-core kernels do not take.
  const bool tc_ok = E <= 256 && H % 64 == 0 && E % 8 == 0;
  if (T <= 16 && (!tc_ok || (T <= 8 && T * H <= 32768)))
    return launch_router_logits_small(x, w, T, H, E, logits, st);
  // tensor-core path: whole gate matrix as one B tile (E <= 256), K in 64-element stages, 16-byte aligned rows
  if (tc_ok) {
    const int rc = launch_router_logits_ksplit(x, w, T, H, E, logits, nullptr, st);      // few token tiles: split the k-steps
    return rc >= 0 ? rc : launch_router_logits_tc(x, w, T, H, E, logits, nullptr, st);
  }
  return launch_router_logits(x, w, T, H, E, logits, st);
}

int b200moe_router_logits(const void* x, const void* w, int64_t T, int32_t H, int32_t E, float* logits, void* stream) {
  if (T < 0 || H <= 0 || H % 8 || E <= 0) return fail(752, "router_logits: hidden must be a positive multiple of 8");
  if (T && (!x || !w || !logits)) return fail(753, "router_logits: null pointer");
  if (((uintptr_t)x | (uintptr_t)w) & 15) return fail(754, "router_logits: operands must be 16-byte aligned");
  return cuda_fail(router_logits_any(x, w, T, H, E, logits, (cudaStream_t)stream), "router_logits");
}

int b200moe_gemm_nvfp4(const void* a_q, const void* a_sf, const void* b_q, const void* b_sf, float alpha, void* out, int64_t m,
                       int64_t n, int64_t k, int64_t out_stride, int32_t tile_n, int32_t* status, void* stream) {
  const int bn = tile_n ? tile_n : (n % 256 == 0 ? 256 : 128);
  if (bn != 128 && bn != 256 && bn != 512) return fail(760, "gemm: tile_n must be 0, 128, 256 or 512");
  if (m < 0 || n <= 0 || k <= 0 || k % 256 || n % (bn == 512 ? 256 : bn))
    return fail(761, "gemm: need K %% 256 == 0 and N %% tile_n == 0 (N %% 256 == 0 for the CTA-pair tile)");
  if (m == 0) return 0;
  if (!a_q || !a_sf || !b_q || !b_sf || !out) return fail(762, "gemm: null pointer");
  if (((uintptr_t)a_q | (uintptr_t)a_sf | (uintptr_t)b_q | (uintptr_t)b_sf | (uintptr_t)out) & 15)
    return fail(763, "gemm: operands must be 16-byte aligned");
  if (out_stride < n || out_stride % 16 || ((uintptr_t)out & 31))
    return fail(764, "gemm: out must be 32-byte aligned, out_stride >= N and a multiple of 16");
  CUtensorMap ta, tb;
  int rc = make_operand_map(&ta, a_q, (uint64_t)m, (uint64_t)k / 2, 128);
  if (rc) return cuda_fail(rc, "gemm A tensor map");
  rc = make_operand_map(&tb, b_q, (uint64_t)n, (uint64_t)k / 2, bn == 512 ? 128 : bn);
  if (rc) return cuda_fail(rc, "gemm B tensor map");
  GemmParams g;
  memset(&g, 0, sizeof(g));
  g.n_tiles_static = (int)((m + 127) / 128);
  g.M = (int)m;
  g.N = (int)n;
  g.K = (int)k;
  g.sfa = (const uint8_t*)a_sf;
  g.sfb = (const uint8_t*)b_sf;
  g.out = (__nv_bfloat16*)out;
  g.out_stride = out_stride;
  g.dense_alpha = alpha;
  g.status = status;
  g.rows_hint = m;
  const int sms = sm_count();
  if (bn == 512) {
    CUtensorMap tsa, tsb;
    rc = make_sf_map(&tsa, a_sf, (uint64_t)((m + 127) / 128) * (k / 64));
    if (!rc) rc = make_sf_map(&tsb, b_sf, (uint64_t)(n / 128) * (k / 64));
    if (rc) return cuda_fail(rc, "gemm scale tensor maps");
    g.n_tiles_static = (int)((m + 255) / 256);
    const int64_t pair_items = (int64_t)g.n_tiles_static * (n / 256);
    const int clusters = (int)(pair_items < sms / 2 ? pair_items : sms / 2);
    return cuda_fail(launch_gemm_nvfp4_pair(kGemmDense, ta, tb, tsa, tsb, g, clusters, (cudaStream_t)stream), "gemm");
  }
  const int64_t items = (int64_t)g.n_tiles_static * (n / bn);
  const int grid = (int)(items < sms ? items : sms);
  return cuda_fail(launch_gemm_nvfp4(kGemmDense, bn, ta, tb, g, grid, (cudaStream_t)stream), "gemm");
}

int64_t b200moe_gemm_bf16_nvfp4_workspace_bytes(int64_t m, int64_t n, int64_t k) {
  if (m <= 0 || n <= 0 || k <= 0 || k % 256 || n % 128) return 0;
  return gemm_w4a16_workspace_bytes(m, n, k);
}

int b200moe_gemm_bf16_nvfp4(const void* a, int64_t a_stride, const void* b_q, const void* b_descale, const float* alpha, void* out,
                            int64_t m, int64_t n, int64_t k, int64_t out_stride, void* workspace, int64_t workspace_bytes,
                            int32_t* status, void* stream) {
  if (m < 0 || n <= 0 || k <= 0 || k % 256 || n % 128)
    return fail(765, "gemm_bf16_nvfp4: M=%lld N=%lld K=%lld need K %% 256 == 0 and N %% 128 == 0", (long long)m, (long long)n, (long long)k);
  if (m == 0) return 0;
  if (m > (1 << 30) || n > (1 << 30) || k > (1 << 30)) return fail(765, "gemm_bf16_nvfp4: sizes above 2^30 are not supported");
  if (!a || !b_q || !b_descale || !out) return fail(766, "gemm_bf16_nvfp4: null pointer");
  if (((uintptr_t)a | (uintptr_t)b_q | (uintptr_t)b_descale) & 15) return fail(767, "gemm_bf16_nvfp4: operands must be 16-byte aligned");
  if (a_stride < k || a_stride % 8) return fail(768, "gemm_bf16_nvfp4: a_stride must be >= K and a multiple of 8 elements");
  if (out_stride < n || out_stride % 16 || ((uintptr_t)out & 31))
    return fail(769, "gemm_bf16_nvfp4: out must be 32-byte aligned, out_stride >= N and a multiple of 16");
  if (workspace && ((uintptr_t)workspace & 15)) return fail(769, "gemm_bf16_nvfp4: workspace must be 16-byte aligned");
  return cuda_fail(launch_gemm_w4a16(a, a_stride, b_q, b_descale, alpha, m, n, k, out, out_stride, workspace,
                                     workspace ? workspace_bytes : 0, status, (cudaStream_t)stream),
                   "gemm_bf16_nvfp4");
}

int64_t b200moe_workspace_bytes(const b200moe_config* cfg) {
  if (check_cfg(cfg)) return -1;
  return make_plan(*cfg).total;
}

int b200moe_create(const b200moe_config* cfg, b200moe_handle* out) {
  if (!out) return fail(717, "create: null output handle");
  *out = nullptr;
  int rc = check_cfg(cfg);
  if (rc) return rc;
  const Plan p = make_plan(*cfg);
  b200moe_layer* h = new b200moe_layer();
  memset(h, 0, sizeof(*h));
  h->cfg = *cfg;
  h->etot = cfg->num_experts + cfg->num_shared_experts;
  h->kk = cfg->top_k + cfg->num_shared_experts;
  h->row_capacity = p.row_capacity;
  h->tile_capacity = p.tile_capacity;
  h->bn = cfg->tile_n ? cfg->tile_n : ((2 * cfg->intermediate) % 256 == 0 && cfg->hidden % 256 == 0 ? 256 : 128);
  h->sm_count = sm_count();
  cudaError_t e = cudaMalloc(&h->base, (size_t)p.total);
  if (e != cudaSuccess) {
    delete h;
    return cuda_fail((int)e, "create: workspace allocation");
  }
  if (h->sm_count > 2 * cfg->sm_margin) h->sm_count -= cfg->sm_margin;   // persistent GEMM grids stay off `sm_margin` SMs
  h->bytes = p.total;
  uint8_t* b = (uint8_t*)h->base;
  h->rm.block_hist = (int32_t*)(b + p.off_block_hist);
  h->rm.counts = (int32_t*)(b + p.off_counts);
  h->rm.seg_start = (int32_t*)(b + p.off_seg);
  h->rm.tile_expert = (int32_t*)(b + p.off_texp);
  h->rm.tile_row0 = (int32_t*)(b + p.off_trow0);
  h->rm.tile_rows = (int32_t*)(b + p.off_trows);
  h->rm.totals = (int32_t*)(b + p.off_totals);
  h->rm.pair_expert = (int32_t*)(b + p.off_pexp);
  h->rm.pair_row0 = (int32_t*)(b + p.off_prow0);
  h->rm.pair_rows = (int32_t*)(b + p.off_prows);
  h->rm.row_of = (int32_t*)(b + p.off_row_of);
  h->rm.tok_of_row = (int32_t*)(b + p.off_tok);
  h->rm.weight_of_row = (float*)(b + p.off_w);
  h->rm.row_capacity = p.row_capacity;
  h->a_q = b + p.off_aq;
  h->a_sf = b + p.off_asf;
  h->act_q = b + p.off_actq;
  h->act_sf = b + p.off_actsf;
  h->rout = (__nv_bfloat16*)(b + p.off_rout);
  h->status = (int32_t*)(b + p.off_status);
  h->step_hq = b + p.off_step_hq;
  h->step_hs = b + p.off_step_hs;
  h->step_logits = (float*)(b + p.off_step_logits);
  h->step_ids = (int32_t*)(b + p.off_step_ids);
  h->step_w = (float*)(b + p.off_step_w);
  e = cudaMemset(h->base, 0, (size_t)p.off_aq);   // index tables and status start at zero
  if (e == cudaSuccess) e = cudaMemset(h->status, 0, 16);
  if (e != cudaSuccess) {
    cudaFree(h->base);
    delete h;
    return cuda_fail((int)e, "create: workspace clear");
  }
  rc = make_operand_map(&h->tm_a1, h->a_q, (uint64_t)p.row_capacity, cfg->hidden / 2, 128);
  if (!rc) rc = make_operand_map(&h->tm_a2, h->act_q, (uint64_t)p.row_capacity, cfg->intermediate / 2, 128);
  if (!rc) rc = make_sf_map(&h->tm_sfa1, h->a_sf, (uint64_t)p.row_capacity / 128 * (cfg->hidden / 64));
  if (!rc) rc = make_sf_map(&h->tm_sfa2, h->act_sf, (uint64_t)p.row_capacity / 128 * (cfg->intermediate / 64));
  h->n_clusters = h->sm_count / 2;
  if (rc) {
    cudaFree(h->base);
    delete h;
    return cuda_fail(rc, "create: activation tensor maps");
  }
  *out = h;
  return 0;
}

int b200moe_destroy(b200moe_handle h) {
  if (!h) return 0;
  for (auto& c : h->cache)
    if (c.exec) cudaGraphExecDestroy(c.exec);
  if (h->capture_stream) cudaStreamDestroy(h->capture_stream);
  if (h->side_stream) cudaStreamDestroy(h->side_stream);
  if (h->ev_fork) cudaEventDestroy(h->ev_fork);
  if (h->ev_join) cudaEventDestroy(h->ev_join);
  cudaError_t e = cudaFree(h->base);
  delete h;
  return cuda_fail((int)e, "destroy");
}

int b200moe_workspace(b200moe_handle h, b200moe_workspace_view* v) {
  if (!h || !v) return fail(719, "workspace: null argument");
  v->counts = h->rm.counts;
  v->seg_start = h->rm.seg_start;
  v->tile_expert = h->rm.tile_expert;
  v->tile_row0 = h->rm.tile_row0;
  v->tile_rows = h->rm.tile_rows;
  v->totals = h->rm.totals;
  v->row_of = h->rm.row_of;
  v->tok_of_row = h->rm.tok_of_row;
  v->weight_of_row = h->rm.weight_of_row;
  v->a_q = h->a_q;
  v->a_sf = h->a_sf;
  v->act_q = h->act_q;
  v->act_sf = h->act_sf;
  v->rout = (uint16_t*)h->rout;
  v->row_capacity = h->row_capacity;
  v->tile_capacity = h->tile_capacity;
  v->pair_expert = h->rm.pair_expert;
  v->pair_row0 = h->rm.pair_row0;
  v->pair_rows = h->rm.pair_rows;
  v->step_ids = h->step_ids;
  v->step_weights = h->step_w;
  return 0;
}

int b200moe_route_map(b200moe_handle h, const int32_t* ids, const float* weights, int32_t T, int32_t offset, void* stream) {
  if (!h) return fail(720, "route_map: null handle");
  if (T < 0 || T > h->cfg.max_tokens) return fail(722, "route_map: num_tokens=%d outside 0..max_tokens=%d", T, h->cfg.max_tokens);
  if (T && h->cfg.top_k > 0 && !ids) return fail(723, "route_map: topk_ids is null");
  return cuda_fail(launch_route_map(ids, weights, 0, T, h->cfg.top_k, h->cfg.num_shared_experts, h->cfg.num_experts, offset, h->rm,
                                    (cudaStream_t)stream),
                   "route map");
}

int b200moe_ep_visits(const int32_t* ids, int64_t T, int32_t top_k, int32_t experts_per_rank, int32_t world, int32_t* rank_slots,
                      void* stream) {
  if (T < 0 || top_k <= 0 || experts_per_rank <= 0 || world <= 0) return fail(790, "ep_visits: bad sizes");
  if (T && (!ids || !rank_slots)) return fail(791, "ep_visits: null pointer");
  return cuda_fail(launch_ep_visits(ids, T, top_k, experts_per_rank, world, rank_slots, (cudaStream_t)stream), "ep_visits");
}

int b200moe_ep_pack(b200moe_handle plan, const void* hidden_states, const void* hidden_states_scale, const int32_t* ids,
                    const float* weights, int32_t hidden, int32_t top_k, int32_t experts_per_rank, int64_t row_bytes, void* out,
                    void* stream) {
  if (!plan) return fail(792, "ep_pack: null plan handle");
  if (hidden <= 0 || hidden % 64 || top_k <= 0 || row_bytes % 16 || row_bytes < hidden / 2 + hidden / 16 + 8 * top_k)
    return fail(793, "ep_pack: row_bytes must be a multiple of 16 and hold payload, scales, ids and weights");
  if (!hidden_states || !hidden_states_scale || !ids || !weights || !out) return fail(794, "ep_pack: null pointer");
  if (((uintptr_t)hidden_states | (uintptr_t)out) & 15) return fail(795, "ep_pack: payload and out must be 16-byte aligned");
  return cuda_fail(launch_ep_pack(hidden_states, hidden_states_scale, ids, weights, plan->rm.tok_of_row, plan->rm.tile_expert,
                                  plan->rm.tile_rows, plan->rm.totals, hidden, top_k, experts_per_rank, plan->cfg.num_experts, row_bytes,
                                  plan->row_capacity, out, (cudaStream_t)stream),
                   "ep_pack");
}

int b200moe_combine(const void* rows, const int32_t* row_of, const float* weight_of_row, int64_t T, int32_t slots, int32_t hidden,
                    void* out, int64_t out_stride, void* stream) {
  if (T < 0 || slots <= 0 || hidden <= 0 || hidden % 8) return fail(780, "combine: hidden must be a positive multiple of 8");
  if (T == 0) return 0;
  if (!rows || !row_of || !weight_of_row || !out) return fail(781, "combine: null pointer");
  if (((uintptr_t)rows | (uintptr_t)out) & 15 || out_stride < hidden || out_stride % 8)
    return fail(782, "combine: rows/out must be 16-byte aligned, out_stride >= hidden and a multiple of 8");
  return cuda_fail(launch_finalize(rows, row_of, weight_of_row, T, slots, hidden, out, out_stride, (cudaStream_t)stream), "combine");
}

int b200moe_route_map_noalloc(const int32_t* ids, const float* weights, int32_t T, int32_t top_k, int32_t num_shared,
                              int32_t num_experts, int32_t offset, int32_t* counts, int32_t* seg_start, int32_t* tile_expert,
                              int32_t* tile_row0, int32_t* tile_rows, int32_t* totals, int32_t* row_of, int32_t* tok_of_row,
                              float* weight_of_row, int64_t row_capacity, void* stream) {
  if (T < 0 || top_k < 0 || num_shared < 0 || top_k + num_shared <= 0 || num_experts < 0 || num_experts + num_shared <= 0)
    return fail(772, "route_map_noalloc: bad sizes");
  const int64_t routes = (int64_t)T * (top_k + num_shared);
  const int etot = num_experts + num_shared;
  if (etot > 264 || routes > 256LL * 2048)
    return fail(770, "route_map_noalloc: %d experts / %lld routes exceed the built-in scratch (264 experts, 524288 routes)", etot,
                (long long)routes);
  if (row_capacity < (routes / 128 + etot + 1) * 128)
    return fail(773, "route_map_noalloc: row_capacity=%lld is below (routes/128 + experts + 1) * 128", (long long)row_capacity);
  if (!counts || !seg_start || !tile_expert || !tile_row0 || !tile_rows || !totals || !row_of || !tok_of_row || !weight_of_row ||
      (T && top_k && !ids))
    return fail(774, "route_map_noalloc: null pointer");
  RouteMapBuffers b;
  memset(&b, 0, sizeof(b));
  b.counts = counts;
  b.seg_start = seg_start;
  b.tile_expert = tile_expert;
  b.tile_row0 = tile_row0;
  b.tile_rows = tile_rows;
  b.totals = totals;
  b.row_of = row_of;
  b.tok_of_row = tok_of_row;
  b.weight_of_row = weight_of_row;
  b.row_capacity = row_capacity;
  return cuda_fail(launch_route_map_static(ids, weights, T, top_k, num_shared, num_experts, offset, b, (cudaStream_t)stream),
                   "route_map_noalloc");
}

static int ep_peers_in(const b200moe_ep_peers* in, EpPeers* out, const char* what) {
  if (!in) return fail(796, "%s: null peers", what);
  if (in->world < 1 || in->world > kEpMaxRanks || in->rank < 0 || in->rank >= in->world)
    return fail(796, "%s: world=%d rank=%d outside 1..%d", what, in->world, in->rank, kEpMaxRanks);
  memset(out, 0, sizeof(*out));
  out->world = in->world;
  out->rank = in->rank;
  for (int i = 0; i < in->world; ++i) {
    out->recv[i] = (uint8_t*)in->recv[i];
    out->ctrl[i] = in->ctrl[i];
    out->ret[i] = in->ret[i];
  }
  return 0;
}

int b200moe_ep_shared_alloc(int64_t bytes, void** ptr, void* ipc_handle) {
  if (bytes <= 0 || !ptr || !ipc_handle) return fail(797, "ep_shared_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle((cudaIpcMemHandle_t*)ipc_handle, p);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    return cuda_fail((int)e, "ep_shared_alloc");
  }
  *ptr = p;
  return 0;
}

int b200moe_ep_shared_open(const void* ipc_handle, void** ptr) {
  if (!ipc_handle || !ptr) return fail(797, "ep_shared_open: bad arguments");
  cudaIpcMemHandle_t hnd;
  memcpy(&hnd, ipc_handle, sizeof(hnd));
  return cuda_fail((int)cudaIpcOpenMemHandle(ptr, hnd, cudaIpcMemLazyEnablePeerAccess), "ep_shared_open");
}

int b200moe_ep_shared_close(void* ptr) { return ptr ? cuda_fail((int)cudaIpcCloseMemHandle(ptr), "ep_shared_close") : 0; }
int b200moe_ep_shared_free(void* ptr) { return ptr ? cuda_fail((int)cudaFree(ptr), "ep_shared_free") : 0; }

int b200moe_ep_dispatch(b200moe_handle plan, const void* hidden_states, const void* hidden_states_scale, const int32_t* ids,
                        const float* weights, int32_t num_tokens, int32_t hidden, int32_t top_k, int32_t experts_per_rank,
                        int64_t row_bytes, const b200moe_ep_peers* peers, int32_t epoch, int32_t shared_slot, int32_t shared_base,
                        void* counter, void* stream) {
  if (!plan) return fail(792, "ep_dispatch: null plan handle");
  EpPeers pe;
  int rc = ep_peers_in(peers, &pe, "ep_dispatch");
  if (rc) return rc;
  if (hidden <= 0 || hidden % 64 || top_k <= 0 || row_bytes % 16 || row_bytes < hidden / 2 + hidden / 16 + 8 * top_k)
    return fail(793, "ep_dispatch: row_bytes must be a multiple of 16 and hold payload, scales, ids and weights");
  if (!hidden_states || !hidden_states_scale || !ids || !weights || !counter) return fail(794, "ep_dispatch: null pointer");
  if ((uintptr_t)hidden_states & 15) return fail(795, "ep_dispatch: payload must be 16-byte aligned");
  if (plan->cfg.num_experts != pe.world || plan->cfg.num_shared_experts != (shared_slot ? 1 : 0))
    return fail(798, "ep_dispatch: the plan layer must have world experts and the shared slot asked for");
  if (num_tokens < 0 || num_tokens > plan->cfg.max_tokens || epoch < 1) return fail(798, "ep_dispatch: bad num_tokens / epoch");
  for (int d = 0; d < pe.world; ++d)
    if (!pe.recv[d] || !pe.ctrl[d] || ((uintptr_t)pe.recv[d] & 15)) return fail(799, "ep_dispatch: peer %d has no (aligned) buffers", d);
  return cuda_fail(launch_ep_dispatch(hidden_states, hidden_states_scale, ids, weights, plan->rm.tok_of_row, plan->rm.tile_expert,
                                      plan->rm.tile_rows, plan->rm.seg_start, plan->rm.totals, hidden, top_k, experts_per_rank, row_bytes,
                                      plan->row_capacity, pe, epoch, num_tokens, shared_slot ? 1 : 0, shared_base, plan->rm.row_of,
                                      plan->rm.weight_of_row, (unsigned int*)counter, (cudaStream_t)stream),
                   "ep_dispatch");
}

int b200moe_ep_wait(b200moe_handle h, const int32_t* flags, int32_t n, int32_t epoch, void* stream) {
  if (!h || !flags || n < 1 || n > 32) return fail(796, "ep_wait: bad arguments");
  return cuda_fail(launch_ep_wait(flags, n, epoch, h->status, 301, (cudaStream_t)stream), "ep_wait");
}

int b200moe_ep_post(const b200moe_ep_peers* peers, int32_t field, int32_t epoch, void* stream) {
  EpPeers pe;
  int rc = ep_peers_in(peers, &pe, "ep_post");
  if (rc) return rc;
  if (field != kEpFlagDispatch && field != kEpFlagReturn) return fail(796, "ep_post: unknown flag field");
  for (int d = 0; d < pe.world; ++d)
    if (!pe.ctrl[d]) return fail(799, "ep_post: peer %d has no control block", d);
  return cuda_fail(launch_ep_post(pe, field, epoch, (cudaStream_t)stream), "ep_post");
}

int b200moe_run_ep(b200moe_handle h, const b200moe_args* args, const b200moe_ep_peers* peers, const int32_t* ctrl, int32_t seg_len,
                   void* stream) {
  int rc = check_args(h, args);
  if (rc) return rc;
  EpRun ep;
  rc = ep_peers_in(peers, &ep.peers, "run_ep");
  if (rc) return rc;
  if (!ctrl || seg_len <= 0 || seg_len % 128 || (int64_t)seg_len * ep.peers.world != args->num_tokens)
    return fail(798, "run_ep: num_tokens must be world * seg_len with seg_len a multiple of 128");
  if (args->direct_rows) return fail(798, "run_ep: direct_rows does not apply");
  for (int s = 0; s < ep.peers.world; ++s)
    if (!ep.peers.ret[s] || ((uintptr_t)ep.peers.ret[s] & 15)) return fail(799, "run_ep: peer %d has no (aligned) return buffer", s);
  ep.ctrl = ctrl;
  ep.seg_len = seg_len;
  return run_impl(h, args, (cudaStream_t)stream, nullptr, &ep);
}

// Replay of the layer's launch chain from a CUDA graph. An entry is keyed on the bytes of the argument block and the
// stream: same pointers, sizes and strides mean the same launches (routing and data are read from memory by the
// kernels, tensor maps depend on addresses only). First sighting of a key runs the chain and remembers the key, the
// second captures the chain on the caller's stream and launches the graph, later ones only launch it.
}  // extern "C"

template <class Launch>
static int launch_cached(b200moe_layer* h, const void* key, int key_bytes, cudaStream_t st, Launch launch) {
  static_assert(sizeof(b200moe_args) <= sizeof(h->cache[0].key) && sizeof(b200moe_step_args) <= sizeof(h->cache[0].key), "key buffer");
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    h->stats.eager_in_capture++;
    return launch(st);                           // the caller is capturing: our launches become part of its graph
  }
  b200moe_layer::Cached* hit = nullptr;
  b200moe_layer::Cached* victim = &h->cache[0];
  for (auto& c : h->cache) {
    if (c.last_use && c.stream == st && c.key_bytes == key_bytes && memcmp(c.key, key, key_bytes) == 0) hit = &c;
    if (c.last_use < victim->last_use) victim = &c;
  }
  ++h->tick;
  if (hit && hit->exec) {
    hit->last_use = h->tick;
    h->stats.graph_replays++;
    return cuda_fail((int)cudaGraphLaunch(hit->exec, st), "graph replay");
  }
  if (!hit) {                                    // first sighting: eager, remember the key
    if (victim->exec) {
      cudaGraphExecDestroy(victim->exec);
      h->stats.graph_evictions++;
    }
    memcpy(victim->key, key, key_bytes);
    victim->key_bytes = key_bytes;
    victim->stream = st;
    victim->exec = nullptr;
    victim->last_use = h->tick;
    return launch(st);
  }
  hit->last_use = h->tick;
  // The chain is captured on a stream of the layer's own (nothing ever executes there) and the graph is launched on
  // the caller's stream, which may be the legacy default stream that cannot be captured itself.
  cudaError_t e = cudaSuccess;
  if (!h->capture_stream) e = cudaStreamCreateWithFlags(&h->capture_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamBeginCapture(h->capture_stream, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return launch(st);
  }
  const int rc = launch(h->capture_stream);
  cudaGraph_t graph = nullptr;
  e = cudaStreamEndCapture(h->capture_stream, &graph);
  if (rc || e != cudaSuccess || !graph) {
    if (graph) cudaGraphDestroy(graph);
    cudaGetLastError();
    return rc ? rc : launch(st);
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess || !exec) {
    cudaGetLastError();
    return launch(st);
  }
  hit->exec = exec;
  h->stats.graph_captures++;
  return cuda_fail((int)cudaGraphLaunch(exec, st), "graph launch");
}

static int run_cached(b200moe_layer* h, const b200moe_args* in, cudaStream_t st) {
  // the key is compared as bytes: copy the fields into a zeroed block so that padding never takes part
  b200moe_args key;
  memset(&key, 0, sizeof(key));
#define B200MOE_COPY(f) key.f = in->f
  B200MOE_COPY(struct_size); B200MOE_COPY(num_tokens); B200MOE_COPY(topk_ids); B200MOE_COPY(topk_weights); B200MOE_COPY(hidden_states);
  B200MOE_COPY(hidden_states_scale); B200MOE_COPY(hidden_states_scale_layout); B200MOE_COPY(activation_type); B200MOE_COPY(gemm1_weights);
  B200MOE_COPY(gemm1_weights_scale); B200MOE_COPY(gemm2_weights); B200MOE_COPY(gemm2_weights_scale); B200MOE_COPY(gemm1_alpha);
  B200MOE_COPY(gemm1_beta); B200MOE_COPY(gemm1_clamp_limit); B200MOE_COPY(output1_scale_scalar); B200MOE_COPY(output1_scale_gate_scalar);
  B200MOE_COPY(output2_scale_scalar); B200MOE_COPY(local_expert_offset); B200MOE_COPY(direct_rows); B200MOE_COPY(output);
  B200MOE_COPY(output_stride); B200MOE_COPY(hidden_states_stride); B200MOE_COPY(hidden_states_scale_stride); B200MOE_COPY(topk_stride);
#undef B200MOE_COPY
  return launch_cached(h, &key, (int)sizeof(key), st, [&](cudaStream_t s2) { return run_impl(h, &key, s2, nullptr); });
}

// Whole step from bf16 tokens: quantiser, router logits, top-k / softmax into the layer's own buffers, then the layer.
static int step_impl(b200moe_layer* h, const b200moe_step_args* a, cudaStream_t st) {
  const b200moe_config& c = h->cfg;
  const int T = a->num_tokens;
  // The quantiser and the router kernels both read the tokens and do not depend on each other: from a few thousand
  // tokens on (each kernel then outlasts the two event hops) the quantiser runs on a side stream beside the router; the
  // fork and the join are events, so the pair is captured into the library's graph like any other launch.
  const bool fork = c.top_k > 0 && T >= 2048;
  cudaStream_t qs = st;
  if (fork) {
    cudaError_t e = cudaSuccess;
    if (!h->side_stream) e = cudaStreamCreateWithFlags(&h->side_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess && !h->ev_fork) e = cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess && !h->ev_join) e = cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_fork, st);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(h->side_stream, h->ev_fork, 0);
    if (e != cudaSuccess) return cuda_fail((int)e, "step: side stream");
    qs = h->side_stream;
  }
  int rc = launch_quantize_nvfp4(a->x, T, c.hidden, a->x_stride, a->activation_global_scale, h->step_hq, h->step_hs,
                                 B200MOE_SF_ROW_MAJOR, qs);
  int rc_router = 0;
  const char* where = "step: quantise";
  if (c.top_k > 0) {
    rc_router = router_logits_any(a->x, a->gate_weight, T, c.hidden, c.num_experts, h->step_logits, st);
    if (rc_router) where = "step: router logits";
    if (!rc_router) {
      rc_router = launch_route_topk(h->step_logits, a->gate_bias, T, c.num_experts, c.top_k, h->step_ids, h->step_w, st);
      if (rc_router) where = "step: top-k";
    }
  }
  if (fork) {   // join even when a launch failed: a capture must not end with an unjoined stream
    cudaError_t e = cudaEventRecord(h->ev_join, qs);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st, h->ev_join, 0);
    if (!rc && e != cudaSuccess) rc = (int)e;
  }
  if (rc) return cuda_fail(rc, "step: quantise");
  if (rc_router) return cuda_fail(rc_router, where);
  b200moe_args r;
  memset(&r, 0, sizeof(r));
  r.struct_size = (int32_t)sizeof(r);
  r.num_tokens = T;
  r.topk_ids = h->step_ids;
  r.topk_weights = h->step_w;
  r.hidden_states = h->step_hq;
  r.hidden_states_scale = h->step_hs;
  r.hidden_states_scale_layout = 2;
  r.activation_type = a->activation_type;
  r.gemm1_weights = a->gemm1_weights;
  r.gemm1_weights_scale = a->gemm1_weights_scale;
  r.gemm2_weights = a->gemm2_weights;
  r.gemm2_weights_scale = a->gemm2_weights_scale;
  r.gemm1_alpha = a->gemm1_alpha;
  r.gemm1_beta = a->gemm1_beta;
  r.gemm1_clamp_limit = a->gemm1_clamp_limit;
  r.output1_scale_scalar = a->output1_scale_scalar;
  r.output1_scale_gate_scalar = a->output1_scale_gate_scalar;
  r.output2_scale_scalar = a->output2_scale_scalar;
  r.output = a->output;
  r.output_stride = a->output_stride;
  return run_impl(h, &r, st, nullptr);
}

extern "C" {

int b200moe_step(b200moe_handle h, const b200moe_step_args* a, void* stream) {
  if (!h) return fail(720, "step: null handle");
  if (!a || a->struct_size != (int32_t)sizeof(b200moe_step_args)) return fail(721, "step: bad args struct_size");
  const b200moe_config& c = h->cfg;
  if (a->num_tokens < 0 || a->num_tokens > c.max_tokens)
    return fail(722, "step: num_tokens=%d outside 0..max_tokens=%d", a->num_tokens, c.max_tokens);
  if (a->num_tokens == 0) return 0;
  if (!a->x || ((uintptr_t)a->x & 15) || a->x_stride < c.hidden || a->x_stride % 8)
    return fail(724, "step: x must be 16-byte aligned bf16 rows with x_stride >= hidden and a multiple of 8");
  if (c.top_k > 0 && (!a->gate_weight || ((uintptr_t)a->gate_weight & 15) || c.top_k > c.num_experts))
    return fail(723, "step: gate_weight is null or misaligned, or top_k > num_experts");
  if (!(a->activation_global_scale > 0.f)) return fail(744, "step: activation_global_scale must be positive");
  if (c.hidden % 64) return fail(711, "step: hidden must be a multiple of 64");
  if (!a->gemm1_weights || !a->gemm1_weights_scale || !a->gemm2_weights || !a->gemm2_weights_scale) return fail(726, "step: weight pointers are null");
  if (a->activation_type != 3 && a->activation_type != 10) return fail(727, "step: activation_type=%d, expected 3 or 10", a->activation_type);
  if (!a->output || ((uintptr_t)a->output & 15) || a->output_stride < c.hidden || a->output_stride % 8)
    return fail(728, "step: output must be 16-byte aligned with output_stride >= hidden and a multiple of 8");
  if (((uintptr_t)a->gemm1_weights | (uintptr_t)a->gemm2_weights | (uintptr_t)a->gemm1_weights_scale | (uintptr_t)a->gemm2_weights_scale) & 15)
    return fail(730, "step: tensors must be 16-byte aligned");
  h->stats.runs++;
  if (!c.graph_cache) return step_impl(h, a, (cudaStream_t)stream);
  b200moe_step_args key;
  memset(&key, 0, sizeof(key));
#define B200MOE_COPY(f) key.f = a->f
  B200MOE_COPY(struct_size); B200MOE_COPY(num_tokens); B200MOE_COPY(x); B200MOE_COPY(x_stride); B200MOE_COPY(gate_weight);
  B200MOE_COPY(gate_bias); B200MOE_COPY(activation_global_scale); B200MOE_COPY(activation_type); B200MOE_COPY(gemm1_weights);
  B200MOE_COPY(gemm1_weights_scale); B200MOE_COPY(gemm2_weights); B200MOE_COPY(gemm2_weights_scale); B200MOE_COPY(gemm1_alpha);
  B200MOE_COPY(gemm1_beta); B200MOE_COPY(gemm1_clamp_limit); B200MOE_COPY(output1_scale_scalar); B200MOE_COPY(output1_scale_gate_scalar);
  B200MOE_COPY(output2_scale_scalar); B200MOE_COPY(output); B200MOE_COPY(output_stride);
#undef B200MOE_COPY
  return launch_cached(h, &key, (int)sizeof(key), (cudaStream_t)stream, [&](cudaStream_t s2) { return step_impl(h, &key, s2); });
}

int b200moe_run(b200moe_handle h, const b200moe_args* args, void* stream) {
  int rc = check_args(h, args);
  if (rc) return rc;
  if (args->num_tokens == 0) return 0;
  h->stats.runs++;
  if (h->cfg.graph_cache) return run_cached(h, args, (cudaStream_t)stream);
  return run_impl(h, args, (cudaStream_t)stream, nullptr);
}

int b200moe_get_stats(b200moe_handle h, b200moe_stats* out) {
  if (!h || !out) return fail(719, "get_stats: null argument");
  *out = h->stats;
  out->workspace_bytes = h->bytes;
  return 0;
}

int b200moe_run_profiled(b200moe_handle h, const b200moe_args* args, void* stream, float* stage_ms) {
  int rc = check_args(h, args);
  if (rc) return rc;
  if (!stage_ms) return fail(732, "run_profiled: stage_ms is null");
  cudaEvent_t ev[6];
  for (int i = 0; i < 6; ++i) cudaEventCreate(&ev[i]);
  for (int i = 0; i < 5; ++i) stage_ms[i] = 0.f;
  rc = run_impl(h, args, (cudaStream_t)stream, ev);
  if (!rc && args->num_tokens > 0) {
    cudaError_t e = cudaEventSynchronize(ev[5]);
    if (e != cudaSuccess) rc = cuda_fail((int)e, "run_profiled: synchronize");
    else
      for (int i = 0; i < 5; ++i) cudaEventElapsedTime(&stage_ms[i], ev[i], ev[i + 1]);
  }
  for (int i = 0; i < 6; ++i) cudaEventDestroy(ev[i]);
  return rc;
}

int b200moe_status(b200moe_handle h, void* stream, int32_t* code) {
  if (!h || !code) return fail(719, "status: null argument");
  cudaError_t e = cudaMemcpyAsync(code, h->status, sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  return cuda_fail((int)e, "status");
}

}  // extern "C"
