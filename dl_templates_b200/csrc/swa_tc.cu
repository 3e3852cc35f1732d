// Host side of the tcgen05 kernels: shape qualification, tile planning, TMA tensor
// maps and launches.
#include <cudaTypedefs.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>

#include "swa_tc.cuh"
#include "swa_tc_bwd.cuh"
#include "swa_tc_bwd2.cuh"
#include "swa_tc_fwd.cuh"
#include "swa_tc_fwd2.cuh"

namespace swa {
namespace tc {

namespace {

thread_local char g_tc_err[256] = "";
constexpr uint32_t kSmemLimit = 227 * 1024;

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// 5-D map over a [B, H, N, d] tensor seen as (d, token column, grid row, head, batch); box =
// (64 elements, box_cols, box_rows, 1, 1), 128-byte swizzle, zero fill outside the tensor.
bool make_map(CUtensorMap* m, const swa_tensor_t* t, const swa_geom_t* g, int d, int box_cols, int box_rows) {
  auto fn = encode_fn();
  if (!fn) {
    snprintf(g_tc_err, sizeof(g_tc_err), "cuTensorMapEncodeTiled entry point not available");
    return false;
  }
  const uint64_t Wtok = (uint64_t)g->t_width * g->b_size;
  cuuint64_t dims[5] = {(cuuint64_t)d, Wtok, (cuuint64_t)g->t_height, (cuuint64_t)g->H, (cuuint64_t)g->B};
  cuuint64_t strides[4] = {(cuuint64_t)t->stride[2] * 2, (cuuint64_t)t->stride[2] * 2 * Wtok,
                           (cuuint64_t)t->stride[1] * 2, (cuuint64_t)t->stride[0] * 2};
  // a dimension of extent 1 may carry any stride; give it a legal one
  for (int i = 0; i < 4; ++i)
    if (dims[i + 1] == 1 && (strides[i] == 0 || strides[i] % 16)) strides[i] = 16;
  cuuint32_t box[5] = {64u, (cuuint32_t)box_cols, (cuuint32_t)box_rows, 1u, 1u};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = g->dtype == SWA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(m, dt, 5, t->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_tc_err, sizeof(g_tc_err), "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return false;
  }
  return true;
}

// SMs of the current device (cached per device ordinal).
int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Experiment knobs (environment variables), read ONCE per process -- a launch must not pay for a dozen getenv
// calls -- and again only when refresh_env() is called (tests that vary them do).  -1 / 0 = not set.
struct Knobs {
  int nmax, nxb, kr, kw, stages, nsb, th_all, th[3], trace_it;
  bool no_tabs, disable, verbose, trace;
};
std::mutex g_plan_mu;                 // guards the knobs and the plan cache
bool g_knobs_read = false;
Knobs g_knobs;

int env_raw(const char* name, int dflt) {
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
}
void read_knobs_locked() {
  Knobs k;
  k.nmax = env_raw("SWA_TC_NMAX", 0);
  k.nxb = env_raw("SWA_TC_NXB", 0);
  k.kr = env_raw("SWA_TC_KR", 0);
  k.kw = env_raw("SWA_TC_KW", 0);
  k.stages = env_raw("SWA_TC_STAGES", 0);
  k.nsb = env_raw("SWA_TC_NSB", 0);
  k.th_all = env_raw("SWA_TC_TH", 0);
  k.th[0] = env_raw("SWA_TC_TH_FWD", 0);
  k.th[1] = env_raw("SWA_TC_TH_DQ", 0);
  k.th[2] = env_raw("SWA_TC_TH_DKDV", 0);
  k.trace_it = env_raw("SWA_TC_TRACE_IT", 1);
  k.no_tabs = getenv("SWA_TC_NO_TABS") != nullptr;
  k.disable = getenv("SWA_TC_DISABLE") != nullptr;
  k.verbose = getenv("SWA_TC_VERBOSE") != nullptr;
  k.trace = getenv("SWA_TC_TRACE") != nullptr;
  g_knobs = k;
  g_knobs_read = true;
}
Knobs knobs() {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  if (!g_knobs_read) read_knobs_locked();
  return g_knobs;
}

// Widest halo, in token columns, over all resident-tile columns.
int halo_width(const swa_geom_t* g, int TW) {
  const int Wtok = g->t_width * g->b_size, b = g->b_size;
  int best = 0;
  for (int x0 = 0; x0 < Wtok; x0 += TW) {
    const int lo = (x0 / b - g->col_size) * b;
    const int hi = ((x0 + TW - 1) / b + g->col_size + 1) * b;
    best = hi - lo > best ? hi - lo : best;
  }
  return best;
}

// Choose the resident tile, the streamed-block shape and the pipeline depths.  Tile shapes tried: 16 x 8 first -- a warp's 32 rows then span
// 4 grid rows and skip 3 of the 7 streamed blocks of a 13-row window -- then 8 x 16.
//   tensor memory (512 columns): forward  score buffers at 128-column strides (packed when they do not fit) + two O accumulators;
//                                backward nsb pairs (S, dP) of 2N columns + the accumulators
//   shared memory:               nxb resident-tile buffers + indicator rows + stages x (block + penalty rows [+ lse, delta])
// `v2`: the plan is for the kernels without streamed rotation (swa_tc_fwd2.cuh / swa_tc_bwd2.cuh), whose shared-memory
// block behind the ring differs: no fixed-size penalty tables (they are sized per plan), two more lse / delta slots.
bool make_plan_shape(const swa_geom_t* g, int which, int TH, int TW, uint32_t tab_bytes, Plan* out, long* cost_out = nullptr,
                     bool v2 = false) {
  Plan pl;
  pl.ncb = 1;
  pl.tab_bytes = tab_bytes;
  pl.TH = TH;
  pl.TW = TW;
  const int hw = halo_width(g, pl.TW);
  if (!v2 && hw > kPenCols) return false;     // the kernels with streamed rotation keep a whole halo row per block row
  const int halo_rows = pl.TH + 2 * g->row_size;
  const int qch = (g->d_qk + 63) / 64, vch = (g->d_v + 63) / 64;
  const uint32_t x_bytes = (which == 0 ? qch : qch + vch) * 16384u;
  const uint32_t row_bytes = (qch + vch) * 128u + kXRowBytes;
  const uint32_t stage_extra = which == 0 ? 0u : 1024u;       // lse / delta slots of a streamed block
  const int acc_cols = which == 0 ? 0 : (which == 1 ? 64 * qch : 64 * (qch + vch));
  const int min_stages = 3;
  // alignment pad of the swizzled tiles + the kernel's barrier / exchange / penalty-table block behind the ring
  const uint32_t slack_v1 = 1024u + (((which == 0 ? (uint32_t)sizeof(FwdShared) : (uint32_t)sizeof(BwdShared)) + 15u) & ~15u);
  const uint32_t slack_v2 = 1024u + (((which == 0 ? (uint32_t)sizeof(Fwd2Shared) : (uint32_t)sizeof(Bwd2Shared)) + 15u) & ~15u) +
                            (which == 0 ? 0u : 2048u);
  // per candidate block shape: the v2 kernels' penalty tables take (halo rows + KR + KW) entries of 32 bytes
  auto slack_for = [&](int KR, int KW, int ncb) { return v2 ? slack_v2 + (uint32_t)(halo_rows + KR + KW * ncb) * 32u : slack_v1; };
  {
    // backward: two (S, dP) pairs of 2N columns next to the accumulators (N = 64 always fits: 256 + 256 columns)
    const int nsb = 2;
    int nmax = which == 0 ? 128 : (512 - acc_cols) / (2 * nsb);
    nmax = nmax > 128 ? 128 : nmax;
    const Knobs kn = knobs();
    if (kn.nmax) nmax = kn.nmax;
    for (int nxb = which == 0 ? 2 : (kn.nxb ? kn.nxb : 2); nxb >= (which == 0 ? 2 : 1); --nxb) {
      const uint32_t fixed = nxb * x_bytes + 128u * kXRowBytes + tab_bytes;
      long best_cost = -1;
      // ncb = column blocks per halo row: 1 whenever a block can span the halo; the kernels without streamed
      // rotation also take halos wider than any block and walk them in several column blocks
      for (int ncb = 1; ncb <= (v2 ? 16 : 1) && best_cost < 0; ++ncb)
        for (int KW = (hw + ncb - 1) / ncb; KW <= kPenCols && (ncb == 1 || KW * (ncb - 1) < hw); ++KW)
          for (int KR = 1; KR <= 16; ++KR) {
            const int N = KW * KR;
            if (N > nmax || N % 16) continue;
            if (fixed + min_stages * ((uint32_t)N * row_bytes + stage_extra) + slack_for(KR, KW, ncb) > kSmemLimit) continue;
            const long nblk = (long)((halo_rows + KR - 1) / KR) * ncb;
            const long cost = nblk * N * 16 + nblk * 400;  // executed columns + a per-block overhead
            if (best_cost < 0 || cost < best_cost) {
              best_cost = cost;
              pl.KR = KR; pl.KW = KW; pl.N = N; pl.ncb = ncb;
            }
          }
      if (best_cost < 0) continue;
      if (kn.kr) {
        pl.KR = kn.kr;
        if (kn.kw) pl.KW = kn.kw;
        pl.N = pl.KR * pl.KW;
        pl.ncb = 1;
        // an override must still hold a whole halo row per block row and fit the penalty-table columns
        if (pl.KW < hw || pl.KW > kPenCols || pl.KR > 16) return false;
      }
      const uint32_t stage = (uint32_t)pl.N * row_bytes + stage_extra;
      const uint32_t kSmemSlack = slack_for(pl.KR, pl.KW, pl.ncb);
      pl.pen_rows = halo_rows + pl.KR;
      pl.pen_cols = pl.KW * pl.ncb;
      const int Wtok = g->t_width * g->b_size;
      pl.n_tiles_x = (Wtok + pl.TW - 1) / pl.TW;
      pl.n_tiles_y = (g->t_height + pl.TH - 1) / pl.TH;
      pl.nxb = nxb;
      pl.stages = min_stages;
      while (pl.stages < kMaxStages && fixed + (pl.stages + 1) * stage + kSmemSlack <= kSmemLimit) ++pl.stages;
      if (kn.stages) pl.stages = kn.stages;
      pl.smem_bytes = fixed + pl.stages * stage + kSmemSlack;
      if (which == 0) {
        // forward: score buffers = look-ahead of the score MMAs: 3 next to the two accumulators, 4 (packed at N-column
        // strides) when tensor memory allows and the block ring is deep enough to feed them (measured)
        int n = pl.stages >= 6 ? 4 : 3;
        while (n > 2 && n * pl.N + 2 * 64 * vch > 512) --n;
        pl.nsb = kn.nsb ? kn.nsb : n;
      } else {
        pl.nsb = nsb;
      }
      *out = pl;
      if (cost_out) *cost_out = best_cost;
      // tensor-memory columns of the final plan (the environment overrides above included): a plan beyond the
      // 512-column allocation is refused here, never launched
      const uint32_t fwd_stride = (pl.N <= 128 && pl.nsb * 128 + 2 * 64 * vch <= 512) ? 128u : (uint32_t)pl.N;
      const uint32_t tmem_cols = which == 0 ? pl.nsb * fwd_stride + 2u * 64u * vch : 2u * nsb * pl.N + (uint32_t)acc_cols;
      return pl.smem_bytes <= kSmemLimit && pl.N % 16 == 0 && pl.N >= 16 && pl.N <= 256 && pl.N <= nmax && pl.stages >= 2 &&
             pl.stages <= kMaxStages && pl.nsb >= 2 && pl.nsb <= 4 && tmem_cols <= 512u;
    }
  }
  return false;
}

// Bytes of the cos/sin tables when they are small enough to be staged in shared memory, else 0.
uint32_t rope_table_bytes(const swa_rope_t* rope) {
  if (!rope || !rope->idx) return 0;
  const uint64_t b = (uint64_t)(rope->max_h + rope->max_w) * rope_tab_stride(rope->n_rdim);
  return b <= 48 * 1024 && !knobs().no_tabs ? (uint32_t)((b + 15) & ~15ull) : 0;
}

// Tile shape for one choice of staged-table bytes; *cost = the planner's block cost of the plan taken.
static bool make_plan_tab(const swa_geom_t* g, const swa_rope_t* rope, int which, uint32_t tab, Plan* out, long* cost,
                          bool v2 = false) {
  const Knobs kn = knobs();
  const int th = kn.th[which] ? kn.th[which] : kn.th_all;
  if (th == 8) return make_plan_shape(g, which, 8, 16, tab, out, cost, v2);
  if (th == 16) return make_plan_shape(g, which, 16, 8, tab, out, cost, v2);
  if (which == 2 || (which == 0 && v2)) {
    // dK/dV (K tile resident, Q blocks streamed; its accumulators leave the narrowest blocks): the shape whose
    // blocks cost less by the planner's own measure -- 16 x 8 at the 13 x 13 window with d = 64, 8 x 16 once
    // d_v = 128 or the window grows (measured: 10 % and 13 % faster at 15 x 15 / d_v = 128 and 31 x 31 / d = 128).
    // The forward kernel without streamed rotation: the same rule -- 8 x 16 at the 13 x 13 and 15 x 15 windows (five
    // or six blocks instead of seven or eight), 16 x 8 at the 31 x 31 window with d = 128, where it halves the
    // number of blocks (23 of 80 tokens instead of 38 of 48; measured 3.11 against 3.60 ms at 32 slices)
    Plan a, b;
    long ca = 0, cb = 0;
    const bool oa = make_plan_shape(g, which, 16, 8, tab, &a, &ca, v2), ob = make_plan_shape(g, which, 8, 16, tab, &b, &cb, v2);
    if (!oa && !ob) return false;
    const bool take_a = oa && (!ob || ca <= cb);
    *out = take_a ? a : b;
    *cost = take_a ? ca : cb;
    return true;
  }
  // measured at the 13 x 13 window: with fused RoPE 16 x 8 wins (80-token blocks, every block row shared by
  // two rotating threads), without it 8 x 16 wins for the forward and dQ kernels (fewer, wider blocks)
  // ... and for the dQ kernel also when at most 32 of 64 q/k dims are rotated (measured 12 % faster at d_v = 128
  // with a 15 x 15 window and 3 % at the 13 x 13 window; at d_qk = 128 the 16 x 8 tile stays 27 % ahead)
  const bool wide_first = !(rope && rope->idx) || (which == 1 && rope->n_rdim <= 8 && g->d_qk == 64);
  return wide_first ? (make_plan_shape(g, which, 8, 16, tab, out, cost, v2) || make_plan_shape(g, which, 16, 8, tab, out, cost, v2))
                    : (make_plan_shape(g, which, 16, 8, tab, out, cost, v2) || make_plan_shape(g, which, 8, 16, tab, out, cost, v2));
}

// The cos/sin tables are staged in shared memory when that does not cost block size: a plan with the tables is
// taken only if its blocks are as cheap as those of the plan without them (40 KB of tables beside d = 128 tiles
// would force 48-token instead of 80-token blocks, measured 1.5x slower in the forward kernel).
// Plans are cached: the search below is a few thousand candidate shapes, repeated for the three kernels of every
// step with the same geometry.  Key = everything the planner reads.
using PlanKey = std::tuple<int, int, int, int, int, int, int, int, int, int, int, int, int>;
std::map<PlanKey, std::pair<bool, Plan>> g_plan_cache;

PlanKey plan_key(const swa_geom_t* g, const swa_rope_t* rope, int which, bool v2) {
  const bool has = rope && rope->idx;
  return PlanKey(which + (v2 ? 3 : 0), g->t_height, g->t_width, g->b_size, g->row_size, g->col_size, g->d_qk, g->d_v,
                 has ? rope->n_rdim : 0, has ? rope->max_h : 0, has ? rope->max_w : 0, g->dtype == SWA_BF16 ? 1 : 0, 0);
}
bool cache_lookup(const PlanKey& k, bool* ok, Plan* out) {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  auto it = g_plan_cache.find(k);
  if (it == g_plan_cache.end()) return false;
  *ok = it->second.first;
  *out = it->second.second;
  return true;
}
void cache_store(const PlanKey& k, bool ok, const Plan& pl) {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  if (g_plan_cache.size() > 4096) g_plan_cache.clear();
  g_plan_cache[k] = std::make_pair(ok, pl);
}

bool make_plan_uncached(const swa_geom_t* g, const swa_rope_t* rope, int which, Plan* out) {
  const uint32_t tab = rope_table_bytes(rope);
  Plan with, without;
  long cw = 0, cn = 0;
  const bool ok_n = make_plan_tab(g, rope, which, 0, &without, &cn);
  if (tab && make_plan_tab(g, rope, which, tab, &with, &cw) && (!ok_n || cw <= cn)) {
    *out = with;
    return true;
  }
  if (ok_n) *out = without;
  return ok_n;
}

// Plan of the kernels that rotate no streamed row (rotation handed on between the kernels, or no RoPE): the
// tile shape of the problem without RoPE; the tables (read once per item, in the epilogue) are staged when that
// costs no block size and leaves at least three stages of the ring.
bool make_plan(const swa_geom_t* g, const swa_rope_t* rope, int which, Plan* out) {
  const PlanKey key = plan_key(g, rope, which, false);
  bool ok = false;
  if (cache_lookup(key, &ok, out)) return ok;
  Plan pl{};
  ok = make_plan_uncached(g, rope, which, &pl);
  cache_store(key, ok, pl);
  if (ok) *out = pl;
  return ok;
}

bool make_plan_prerot_uncached(const swa_geom_t* g, const swa_rope_t* rope, int which, Plan* out) {
  const uint32_t tab = rope_table_bytes(rope);
  Plan with, without;
  long cw = 0, cn = 0;
  const bool ok_n = make_plan_tab(g, nullptr, which, 0, &without, &cn, true);
  // (measured: a fourth or fifth stage of the ring is worth nothing here, table rows fetched from L2 inside the
  // epilogue cost 0.2 to 0.3 ms per launch at the default workload)
  if (ok_n && tab && make_plan_tab(g, nullptr, which, tab, &with, &cw, true) && cw <= cn &&
      (with.stages >= without.stages || with.stages >= 3) && with.TH == without.TH) {
    *out = with;
    return true;
  }
  if (ok_n) *out = without;
  return ok_n;
}

// Indicator value a and penalty b (powers of two, exact in fp16 and bf16) of the window mask that
// rides on the score MMA: a*b*scale*log2(e) >= 4000, so exp2 of a masked score is exactly 0.
bool mask_constants(float sm_scale, float* a, float* b) {
  const float need = 4000.f / (sm_scale * kLog2e);
  float bb = 16384.f, aa = 1.f;
  while (aa * bb < need && aa < 16384.f) aa *= 2.f;
  *a = aa;
  *b = bb;
  return aa * bb >= need;
}

bool make_plan_prerot(const swa_geom_t* g, const swa_rope_t* rope, int which, Plan* out) {
  const PlanKey key = plan_key(g, rope, which, true);
  bool ok = false;
  if (cache_lookup(key, &ok, out)) return ok;
  Plan pl{};
  ok = make_plan_prerot_uncached(g, rope, which, &pl);
  cache_store(key, ok, pl);
  if (ok) *out = pl;
  return ok;
}

KParams make_params(const swa_geom_t* g, const swa_rope_t* rope, const Plan& pl, int32_t* status) {
  KParams p;
  p.t_h = g->t_height;
  p.Wtok = g->t_width * g->b_size;
  p.b = g->b_size;
  p.wr = g->row_size;
  p.wc = g->col_size;
  p.H = g->H;
  p.qch = (g->d_qk + 63) / 64;
  p.vch = (g->d_v + 63) / 64;
  p.dqk = g->d_qk;
  p.dv = g->d_v;
  p.sm_scale = g->sm_scale;
  p.scale_log2 = g->sm_scale * kLog2e;
  mask_constants(g->sm_scale, &p.mask_a, &p.mask_b);
  p.pl = pl;
  p.rope = make_rope(rope);
  p.n_items = pl.n_tiles_x * pl.n_tiles_y * g->B * g->H;
  p.status = status;
  // the Python layer hands a 4 KiB status buffer: words 0-3 status, bytes 16.. = 4 roles x 32 clock samples
  const Knobs kn = knobs();
  p.trace = (status != nullptr && kn.trace) ? reinterpret_cast<long long*>(status + 4) : nullptr;
  p.trace_it = kn.trace_it;
  return p;
}

// What a tensor map of these kernels can describe: unit last stride, 16-byte aligned base and rows, and strictly
// positive strides (a batch or head dimension broadcast with stride 0 cannot be encoded; extents of 1 are
// given a legal stride when the map is built).  `B`, `H` = extents of the first two dimensions.
bool tensor_ok(const swa_tensor_t* t, int B, int H) {
  return t->stride[3] == 1 && ((uintptr_t)t->ptr % 16) == 0 && t->stride[0] % 8 == 0 && t->stride[1] % 8 == 0 &&
         t->stride[2] % 8 == 0 && t->stride[2] > 0 && (B == 1 || t->stride[0] > 0) && (H == 1 || t->stride[1] > 0);
}

}  // namespace

const char* last_error() { return g_tc_err; }

void refresh_env() {
  std::lock_guard<std::mutex> lock(g_plan_mu);
  read_knobs_locked();
  g_plan_cache.clear();
}

const char* unsupported_reason(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* const* tensors,
                               int n_tensors, int which, bool prerotated) {
  if (knobs().disable) return "disabled by SWA_TC_DISABLE";
  if (g->dtype != SWA_F16 && g->dtype != SWA_BF16) return "fp32 runs on the SIMT kernels";
  // The kernels work on 64-element chunks of a row.  Those without streamed rotation also take head dims of 32 and
  // 96: the tensor map's innermost extent is the real head dim, so TMA zero-fills the missing half of the last chunk
  // (zero columns of q, k leave every score unchanged, zero columns of v and dO give zero columns of O, dV that are
  // never stored), which costs MMA work on zeros but no HBM traffic and no padded copies.
  {
    const bool v2_dims = prerotated || !(rope && rope->idx);
    auto dim_ok = [&](int d) { return v2_dims ? (d >= 32 && d <= 128 && d % 32 == 0) : (d == 64 || d == 128); };
    if (!dim_ok(g->d_qk) || !dim_ok(g->d_v))
      return v2_dims ? "head dims must be 32, 64, 96 or 128" : "head dims must be 64 or 128 for the kernels that rotate streamed rows";
  }
  if (!(g->sm_scale > 0.f)) return "sm_scale must be positive";
  float ma, mb;
  if (!mask_constants(g->sm_scale, &ma, &mb)) return "sm_scale too small for the MMA-side window mask";
  if (rope && rope->idx && rope->n_rdim != 8 && rope->n_rdim != 16 && rope->n_rdim != 32)
    return "n_rdim must be 8, 16 or 32 (RoPE on 32, 64 or 128 dims)";
  if (g->row_size > 64) return "row window too tall for the penalty tables";
  if ((int64_t)g->t_height * g->t_width * g->b_size > (1 << 30)) return "grid too large";
  Plan pl;
  const bool v2 = prerotated || !(rope && rope->idx);
  if (!(v2 ? make_plan_prerot(g, which == 0 ? nullptr : rope, which, &pl) : make_plan(g, rope, which, &pl)))
    return "no tile plan fits (window too wide for one streamed block of the kernels with streamed rotation)";
  for (int i = 0; i < n_tensors; ++i)
    if (!tensor_ok(tensors[i], g->B, g->H)) return "tensors need unit last stride, positive strides and 16-byte aligned rows";
  return nullptr;
}

bool describe_plan(const swa_geom_t* g, const swa_rope_t* rope, int which, int32_t* out) {
  // which 0..2: the kernel swa_fwd / swa_bwd_dq / swa_bwd_dkdv would run; 3..5: swa_fwd_rot / swa_bwd_dq_rot /
  // swa_bwd_dkdv_rot.  Without RoPE, and for 3..5, these are the kernels without streamed rotation.
  const bool prerot = which >= 3;
  const int kind = which % 3;
  const bool v2 = prerot || !(rope && rope->idx);
  Plan pl;
  if (!(v2 ? make_plan_prerot(g, kind == 0 ? nullptr : rope, kind, &pl) : make_plan(g, rope, kind, &pl))) return false;
  const uint32_t qch = (g->d_qk + 63) / 64, vch = (g->d_v + 63) / 64, N = pl.N;
  const uint32_t pen = v2 ? (uint32_t)(pl.pen_rows + pl.pen_cols) * 32u : 0u;   // v1: inside the kernels' shared block
  uint32_t used = 1023, tmem = 0;   // worst-case pad to the 1024-byte alignment of the swizzled tiles
  if (kind == 0) {
    used += 2 * qch * 16384u + 128u * kXRowBytes + pl.stages * N * ((qch + vch) * 128u + kXRowBytes);
    used += (((v2 ? (uint32_t)sizeof(Fwd2Shared) : (uint32_t)sizeof(FwdShared)) + 15u) & ~15u) + pen;
    const uint32_t o_cols = vch * 64u;
    const uint32_t stride = (N <= 128u && pl.nsb * 128u + 2 * o_cols <= 512u) ? 128u : N;
    tmem = pl.nsb * stride + 2 * o_cols;
    if (stride < N) tmem = 1u << 30;   // a score buffer would not hold a block
  } else {
    used += pl.nxb * (qch + vch) * 16384u + 128u * kXRowBytes + pl.stages * (N * ((qch + vch) * 128u + kXRowBytes) + 1024u);
    used += (((v2 ? (uint32_t)sizeof(Bwd2Shared) : (uint32_t)sizeof(BwdShared)) + 15u) & ~15u) + pen + (v2 ? 2048u : 0u);
    tmem = 2 * 2 * N + 64u * qch + (kind == 2 ? 64u * vch : 0u);
  }
  used += pl.tab_bytes;
  const int32_t v[12] = {pl.TH, pl.TW, pl.KR, pl.KW, pl.N, pl.stages, kind == 0 ? pl.nsb : 2, kind == 0 ? 2 : pl.nxb,
                         (int32_t)pl.tab_bytes, (int32_t)pl.smem_bytes, (int32_t)used, (int32_t)tmem};
  for (int i = 0; i < 12; ++i) out[i] = v[i];
  return true;
}

int launch_fwd(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
               const swa_tensor_t* v, const swa_tensor_t* o, float* lse, int32_t* status, cudaStream_t st) {
  if (!(rope && rope->idx)) return launch_fwd2(g, q, k, v, o, lse, status, st);
  Plan pl;
  if (!make_plan(g, rope, 0, &pl)) {
    snprintf(g_tc_err, sizeof(g_tc_err), "no tile plan");
    return -1;
  }
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q, g, g->d_qk, pl.TW, pl.TH) || !make_map(&tk, k, g, g->d_qk, pl.KW, pl.KR) ||
      !make_map(&tv, v, g, g->d_v, pl.KW, pl.KR))
    return -1;
  const KParams p = make_params(g, rope, pl, status);
  // persistent: one CTA per SM, each walks the items blockIdx.x, blockIdx.x + gridDim.x, ...
  const int n_items = pl.n_tiles_x * pl.n_tiles_y * g->B * g->H;
  const int sms = sm_count();
  dim3 grid(n_items < sms ? n_items : sms), block(kFwdThreads);
  using FwdKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, KParams, View4, float*);
  // the RoPE table width is a template parameter of the kernel (index: n_rdim / 8, 0 = no rotation)
  // ... and so is whether the cos/sin tables are staged in shared memory
  static const FwdKernel fwd_table[2][2][5] = {
      {{fwd_kernel<false, 0, false>, fwd_kernel<false, 1, false>, fwd_kernel<false, 2, false>, nullptr, fwd_kernel<false, 4, false>},
       {fwd_kernel<false, 0, false>, fwd_kernel<false, 1, true>, fwd_kernel<false, 2, true>, nullptr, fwd_kernel<false, 4, true>}},
      {{fwd_kernel<true, 0, false>, fwd_kernel<true, 1, false>, fwd_kernel<true, 2, false>, nullptr, fwd_kernel<true, 4, false>},
       {fwd_kernel<true, 0, false>, fwd_kernel<true, 1, true>, fwd_kernel<true, 2, true>, nullptr, fwd_kernel<true, 4, true>}}};
  const int ni = (rope && rope->idx) ? rope->n_rdim / 8 : 0;
  FwdKernel kern = fwd_table[g->dtype == SWA_BF16 ? 1 : 0][pl.tab_bytes ? 1 : 0][ni];
  if (kern == nullptr) {
    snprintf(g_tc_err, sizeof(g_tc_err), "n_rdim %d has no tensor-core kernel", rope ? rope->n_rdim : 0);
    return -1;
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes);
  if (e != cudaSuccess) {
    snprintf(g_tc_err, sizeof(g_tc_err), "cudaFuncSetAttribute(%u bytes): %s", pl.smem_bytes, cudaGetErrorString(e));
    return -1;
  }
  if (knobs().verbose)
    fprintf(stderr, "[swa2d] fwd plan: tile %dx%d, block %dx%d (N=%d), stages %d, tables %u, smem %u, %d items on %u CTAs\n",
            pl.TH, pl.TW, pl.KR, pl.KW, pl.N, pl.stages, pl.tab_bytes, pl.smem_bytes, n_items, grid.x);
  kern<<<grid, block, pl.smem_bytes, st>>>(tq, tk, tv, p, make_view(o), lse);
  return 0;
}

int launch_fwd2(const swa_geom_t* g, const swa_tensor_t* q, const swa_tensor_t* k, const swa_tensor_t* v,
                const swa_tensor_t* o, float* lse, int32_t* status, cudaStream_t st) {
  Plan pl;
  if (!make_plan_prerot(g, nullptr, 0, &pl)) {      // nothing is rotated: the plan of the problem without RoPE
    snprintf(g_tc_err, sizeof(g_tc_err), "no tile plan");
    return -1;
  }
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q, g, g->d_qk, pl.TW, pl.TH) || !make_map(&tk, k, g, g->d_qk, pl.KW, pl.KR) ||
      !make_map(&tv, v, g, g->d_v, pl.KW, pl.KR))
    return -1;
  const KParams p = make_params(g, nullptr, pl, status);
  const int sms = sm_count();
  dim3 grid(p.n_items < sms ? p.n_items : sms), block(kFwdThreads);   // persistent: one CTA per SM walks the items
  auto kern = g->dtype == SWA_BF16 ? fwd2_kernel<true> : fwd2_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes);
  if (e != cudaSuccess) {
    snprintf(g_tc_err, sizeof(g_tc_err), "cudaFuncSetAttribute(%u bytes): %s", pl.smem_bytes, cudaGetErrorString(e));
    return -1;
  }
  if (knobs().verbose)
    fprintf(stderr, "[swa2d] fwd2 plan: tile %dx%d, block %dx%d (N=%d), stages %d, score buffers %d, smem %u, %d items on %u CTAs\n",
            pl.TH, pl.TW, pl.KR, pl.KW, pl.N, pl.stages, pl.nsb, pl.smem_bytes, p.n_items, grid.x);
  kern<<<grid, block, pl.smem_bytes, st>>>(tq, tk, tv, p, make_view(o), lse);
  return 0;
}

namespace {

// `prerotated`: q and k are rotated copies made by an earlier kernel (the forward kernel of swa_fwd_rot); the
// kernels then run in their no-RoPE structure and only rotate dQ / dK back in the epilogue.
template <bool DKDV>
int launch_bwd(const swa_geom_t* g, const swa_rope_t* rope, bool prerotated, const swa_tensor_t* xqk, const swa_tensor_t* xv,
               const swa_tensor_t* yqk, const swa_tensor_t* yv, const float* lse, const float* delta,
               const swa_tensor_t* out_qk, const swa_tensor_t* out_v, int32_t* status, cudaStream_t st) {
  Plan pl;
  const bool v2 = prerotated || !(rope && rope->idx);      // the kernels without streamed rotation
  if (!(v2 ? make_plan_prerot(g, rope, DKDV ? 2 : 1, &pl) : make_plan(g, rope, DKDV ? 2 : 1, &pl))) {
    snprintf(g_tc_err, sizeof(g_tc_err), "no tile plan");
    return -1;
  }
  CUtensorMap mxqk, mxv, myqk, myv;
  if (!make_map(&mxqk, xqk, g, g->d_qk, pl.TW, pl.TH) || !make_map(&mxv, xv, g, g->d_v, pl.TW, pl.TH) ||
      !make_map(&myqk, yqk, g, g->d_qk, pl.KW, pl.KR) || !make_map(&myv, yv, g, g->d_v, pl.KW, pl.KR))
    return -1;
  const KParams p = make_params(g, rope, pl, status);
  const int sms = sm_count();
  dim3 grid(p.n_items < sms ? p.n_items : sms), block(kBwdThreads);   // persistent: one CTA per SM walks the items
  using BwdKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, KParams, const float*,
                             const float*, View4, View4);
  // [dtype][tables staged][n_rdim / 8]: q / k rotated in shared memory, dQ / dK rotated back in the epilogue
  static const BwdKernel fused_table[2][2][5] = {
      {{nullptr, bwd_kernel<false, DKDV, 1, false>, bwd_kernel<false, DKDV, 2, false>, nullptr, bwd_kernel<false, DKDV, 4, false>},
       {nullptr, bwd_kernel<false, DKDV, 1, true>, bwd_kernel<false, DKDV, 2, true>, nullptr, bwd_kernel<false, DKDV, 4, true>}},
      {{nullptr, bwd_kernel<true, DKDV, 1, false>, bwd_kernel<true, DKDV, 2, false>, nullptr, bwd_kernel<true, DKDV, 4, false>},
       {nullptr, bwd_kernel<true, DKDV, 1, true>, bwd_kernel<true, DKDV, 2, true>, nullptr, bwd_kernel<true, DKDV, 4, true>}}};
  // [dtype][n_rdim / 8]: no RoPE, or inputs already rotated and only the epilogue rotation
  static const BwdKernel prerot_table[2][2][5] = {
      {{bwd2_kernel<false, DKDV, 0, false>, bwd2_kernel<false, DKDV, 1, false>, bwd2_kernel<false, DKDV, 2, false>, nullptr,
        bwd2_kernel<false, DKDV, 4, false>},
       {bwd2_kernel<false, DKDV, 0, false>, bwd2_kernel<false, DKDV, 1, true>, bwd2_kernel<false, DKDV, 2, true>, nullptr,
        bwd2_kernel<false, DKDV, 4, true>}},
      {{bwd2_kernel<true, DKDV, 0, false>, bwd2_kernel<true, DKDV, 1, false>, bwd2_kernel<true, DKDV, 2, false>, nullptr,
        bwd2_kernel<true, DKDV, 4, false>},
       {bwd2_kernel<true, DKDV, 0, false>, bwd2_kernel<true, DKDV, 1, true>, bwd2_kernel<true, DKDV, 2, true>, nullptr,
        bwd2_kernel<true, DKDV, 4, true>}}};
  const int ni = (rope && rope->idx) ? rope->n_rdim / 8 : 0;
  const int bf = g->dtype == SWA_BF16 ? 1 : 0;
  BwdKernel kern = (prerotated || ni == 0) ? prerot_table[bf][pl.tab_bytes ? 1 : 0][ni] : fused_table[bf][pl.tab_bytes ? 1 : 0][ni];
  if (kern == nullptr) {
    snprintf(g_tc_err, sizeof(g_tc_err), "n_rdim %d has no tensor-core kernel", rope ? rope->n_rdim : 0);
    return -1;
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem_bytes);
  if (e != cudaSuccess) {
    snprintf(g_tc_err, sizeof(g_tc_err), "cudaFuncSetAttribute(%u bytes): %s", pl.smem_bytes, cudaGetErrorString(e));
    return -1;
  }
  if (knobs().verbose)
    fprintf(stderr, "[swa2d] %s plan: tile %dx%d, block %dx%d (N=%d), stages %d, nsb %d, nxb %d, tables %u, smem %u, %d items on %u CTAs\n",
            DKDV ? "dkdv" : "dq", pl.TH, pl.TW, pl.KR, pl.KW, pl.N, pl.stages, pl.nsb, pl.nxb, pl.tab_bytes, pl.smem_bytes, p.n_items, grid.x);
  kern<<<grid, block, pl.smem_bytes, st>>>(mxqk, mxv, myqk, myv, p, lse, delta, make_view(out_qk),
                                          out_v ? make_view(out_v) : View4{nullptr, 0, 0, 0, 0});
  return 0;
}

}  // namespace

int launch_dq(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
              const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
              const swa_tensor_t* dq, int32_t* status, cudaStream_t st, bool prerotated) {
  return launch_bwd<false>(g, rope, prerotated, q, d_o, k, v, lse, delta, dq, nullptr, status, st);
}

int launch_dkdv(const swa_geom_t* g, const swa_rope_t* rope, const swa_tensor_t* q, const swa_tensor_t* k,
                const swa_tensor_t* v, const swa_tensor_t* d_o, const float* lse, const float* delta,
                const swa_tensor_t* dk, const swa_tensor_t* dv, int32_t* status, cudaStream_t st, bool prerotated) {
  return launch_bwd<true>(g, rope, prerotated, k, v, q, d_o, lse, delta, dk, dv, status, st);
}

}  // namespace tc
}  // namespace swa
