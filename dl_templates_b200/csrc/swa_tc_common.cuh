// Pieces shared by the three tcgen05 kernels (forward, dQ, dK/dV): the tile plan,
// window bit-masks, in-shared-memory RoPE rotation of 128-byte-swizzled tiles,
// and 16-bit packing.
//
// Geometry.  Tokens of one (batch, head) form a grid of t_h rows by Wtok = t_w*b_size
// token columns (token n = row*Wtok + x).  A CTA owns a "resident" tile of
// TH x TW = 128 tokens (queries in forward and dQ, keys in dK/dV) and streams the
// halo of tokens that can interact with it in blocks of KR rows x KW token columns
// (N = KR*KW <= 128, N % 16 == 0).  The tile-window relation "|row - row'| <= wr and
// |x/b - x'/b| <= wc, both inside the grid" is symmetric, so the same halo and the
// same mask serve all three kernels.
//
// Shared-memory tiles are what a TMA box (64 elements, columns, rows) with the
// 128-byte swizzle produces: row j = jr*cols + jc occupies 128 bytes at j*128, its
// 16-byte unit u stored at position u ^ (j & 7).  A head dim of 128 is two such
// tiles ("chunks") one after the other.
#pragma once

#include "common.cuh"
#include "umma.cuh"

namespace swa {
namespace tc {

constexpr int kTileTokens = 128;  // rows of the resident tile = MMA M
constexpr int kMaxStages = 8;   // depth limit of the streamed-block ring

struct Plan {
  int TH, TW;          // resident tile: rows x token columns (TH*TW == 128)
  int KR, KW, N;       // streamed block: rows x token columns, N = KR*KW
  int ncb;             // column blocks per halo row (1: a block spans the halo; more: only the kernels without
                       // streamed rotation, for halos wider than one block)
  int n_tiles_x, n_tiles_y;
  int stages;          // streamed-block pipeline depth
  int nsb, nxb;        // backward: (S, dP) buffer pairs in tensor memory, resident-tile buffers in shared memory
  int pen_rows, pen_cols;  // entries of the window-mask penalty tables the kernels without streamed rotation keep
  uint32_t tab_bytes;  // cos/sin tables staged in shared memory (0: read from global memory)
  uint32_t smem_bytes;
};

struct KParams {
  int t_h, Wtok, b, wr, wc, H;
  int qch, vch;        // 64-element chunks of a q/k row and of a v row: ceil(d_qk / 64), ceil(d_v / 64)
  int dqk, dv;         // the head dims themselves (multiples of 32): a last chunk that is only half there is zero-filled
                       // by TMA on the way in, and the epilogues store the real columns only
  float scale_log2, sm_scale;
  float mask_a, mask_b;  // window mask through the MMA: indicator value and penalty magnitude (powers of two)
  Plan pl;
  RopeDev rope;
  int n_items;         // persistent kernels: work items = tiles per head x batch x heads
  int32_t* status;
  long long* trace;    // optional per-role clock64() samples of one CTA (performance debugging), else null
  int trace_it;        // which work item of that CTA is sampled
};

// Position of a resident-tile CTA and the halo it streams.
struct TilePos {
  int r0, x0;          // first row / token column of the resident tile
  int hx0;             // first token column of the halo
  int hr_first;        // first halo row (clamped to the grid)
  int hr_last;         // last halo row (clamped to the grid)
  int nblk;            // streamed blocks
};

__device__ __forceinline__ TilePos tile_pos(const KParams& p, int tile_idx) {
  TilePos t;
  const int ty = tile_idx / p.pl.n_tiles_x, tx = tile_idx - ty * p.pl.n_tiles_x;
  t.r0 = ty * p.pl.TH;
  t.x0 = tx * p.pl.TW;
  t.hx0 = (t.x0 / p.b - p.wc) * p.b;
  t.hr_first = max(t.r0 - p.wr, 0);
  t.hr_last = min(t.r0 + p.pl.TH - 1 + p.wr, p.t_h - 1);
  t.nblk = (t.hr_last - t.hr_first + p.pl.KR) / p.pl.KR * p.pl.ncb;
  return t;
}

// Streamed blocks of work item `item`.
__device__ __forceinline__ int item_blocks(const KParams& p, int item, int tiles_per_head) {
  const int tile = item % tiles_per_head, ty = tile / p.pl.n_tiles_x, r0 = ty * p.pl.TH;
  const int first = max(r0 - p.wr, 0), last = min(r0 + p.pl.TH - 1 + p.wr, p.t_h - 1);
  return (last - first + p.pl.KR) / p.pl.KR * p.pl.ncb;
}

// Block j of an item: the blocks walk the halo row band by row band, `ncb` column blocks per band.
__device__ __forceinline__ void block_pos(const Plan& pl, int j, int& band, int& cblk) {
  band = pl.ncb == 1 ? j : j / pl.ncb;
  cblk = j - band * pl.ncb;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (BF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
}

// ---- window mask as extra contraction columns ------------------------------------------------
// The score MMA contracts over 32 extra columns.  The resident token at tile position (i, c)
// carries mask_a in column i (its row in the tile, i < TH) and in column TH+c (its column in the
// tile, c < TW; TH + TW <= 32, both multiples of 8); a streamed token carries -mask_b in column i
// when it is outside the row window of tile row i (or outside the grid) and in column TH+c when it
// is outside the column window of tile column c.  The product adds 0 to every allowed pair and at
// most -mask_a*mask_b to every other pair, so exp2 of the scaled score underflows to exactly 0
// there and the threads that own the rows do no masking work at all.
//
// These "x tiles" are written by threads, not by TMA, in the unswizzled K-major core-matrix
// layout: 16-byte unit u (0..3) of row r at (r/8)*512 + u*128 + (r%8)*16.
constexpr uint32_t kXRowBytes = 64;
constexpr uint32_t kXLbo = 128, kXSbo = 512, kXStepBytes = 256;

__device__ __forceinline__ uint8_t* xtile_unit(uint8_t* tile, int row, int unit) {
  return tile + (row >> 3) * 512 + unit * 128 + (row & 7) * 16;
}

// Units [2*part_lo, 2*part_hi + 2) of the row (a row may be shared by two threads).
template <bool BF16>
__device__ __forceinline__ void write_indicator_row(uint8_t* tile, int row, int part_lo, int part_hi, const KParams& p) {
  const int ti = row / p.pl.TW, tc = row - ti * p.pl.TW;
  const int hot_r = ti, hot_c = p.pl.TH + tc;
  const float a = p.mask_a;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    if ((u >> 1) < part_lo || (u >> 1) > part_hi) continue;
    uint32_t w[4];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const int d0 = u * 8 + 2 * h, d1 = d0 + 1;
      w[h] = pack2<BF16>((d0 == hot_r || d0 == hot_c) ? a : 0.f, (d1 == hot_r || d1 == hot_c) ? a : 0.f);
    }
    *reinterpret_cast<uint4*>(xtile_unit(tile, row, u)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// The penalty row of a streamed token is [row part (TH values) | column part (TW values) | zeros]:
// the row part depends only on the token's halo row, the column part only on its halo column.  Both
// are tabulated once per resident tile; per block a thread only copies 16-byte units.
constexpr int kPenRows = 160;   // >= TH + 2*wr + KR halo rows (wr <= 64)
constexpr int kPenCols = 128;   // >= KW, the widest streamed block (halo width in token columns)
struct PenaltyTables {
  uint4 row[kPenRows][2];       // [halo row - hr_first][tile rows 0-7 | 8-15]
  uint4 col[kPenCols][2];       // [halo column - hx0][tile columns 0-7 | 8-15]
};

template <bool BF16>
__device__ __forceinline__ uint4 penalty_unit(int lo, int hi, float nb) {  // 8 tile positions, allowed range [lo, hi]
  uint32_t w[4];
#pragma unroll
  for (int h = 0; h < 4; ++h)
    w[h] = pack2<BF16>((2 * h >= lo && 2 * h <= hi) ? 0.f : nb, (2 * h + 1 >= lo && 2 * h + 1 <= hi) ? 0.f : nb);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Called by the 128 threads that write the mask tiles, once per resident tile.
template <bool BF16>
__device__ __forceinline__ void build_penalty_tables(PenaltyTables* tab, int t, const KParams& p, const TilePos& tp,
                                                     int nthreads = 128) {
  const float nb = -p.mask_b;
#pragma unroll 1
  for (int hr = t; hr < kPenRows; hr += nthreads) {
    const int yr = tp.hr_first + hr;
    const bool in = yr <= tp.hr_last;                       // hr_first >= 0 and hr_last < t_h by construction
    const int lo = in ? yr - p.wr - tp.r0 : 1, hi = in ? yr + p.wr - tp.r0 : 0;
    tab->row[hr][0] = penalty_unit<BF16>(lo, hi, nb);
    tab->row[hr][1] = penalty_unit<BF16>(lo - 8, hi - 8, nb);
  }
#pragma unroll 1
  for (int jc = t; jc < kPenCols; jc += nthreads) {
    const int yx = tp.hx0 + jc;
    const bool in = yx >= 0 && yx < p.Wtok;
    int lo = 1, hi = 0;
    if (in) {
      const int yc = yx / p.b;
      lo = (yc - p.wc) * p.b - tp.x0;                       // allowed tile columns, inclusive
      hi = (yc + p.wc + 1) * p.b - tp.x0 - 1;
    }
    tab->col[jc][0] = penalty_unit<BF16>(lo, hi, nb);
    tab->col[jc][1] = penalty_unit<BF16>(lo - 8, hi - 8, nb);
  }
}

// The same tables sized for the plan at hand (halo rows of one item, columns of one streamed block) instead of
// for the largest window the kernels accept: 1.7 KB instead of 9 KB at a 13 x 13 window, which is what lets the
// kernels that use them keep one more stage of the block ring.  Entry i of `row` / `col` = two 16-byte units.
struct PenView {
  uint4* row;          // [pen_rows][2]
  uint4* col;          // [pen_cols][2]
  int n_rows, n_cols;
};

template <bool BF16>
__device__ __forceinline__ void build_penalty_view(const PenView& pv, int t, const KParams& p, const TilePos& tp, int nthreads) {
  const float nb = -p.mask_b;
#pragma unroll 1
  for (int hr = t; hr < pv.n_rows; hr += nthreads) {
    const int yr = tp.hr_first + hr;
    const bool in = yr <= tp.hr_last;
    const int lo = in ? yr - p.wr - tp.r0 : 1, hi = in ? yr + p.wr - tp.r0 : 0;
    pv.row[2 * hr] = penalty_unit<BF16>(lo, hi, nb);
    pv.row[2 * hr + 1] = penalty_unit<BF16>(lo - 8, hi - 8, nb);
  }
#pragma unroll 1
  for (int jc = t; jc < pv.n_cols; jc += nthreads) {
    const int yx = tp.hx0 + jc;
    const bool in = yx >= 0 && yx < p.Wtok;
    int lo = 1, hi = 0;
    if (in) {
      const int yc = yx / p.b;
      lo = (yc - p.wc) * p.b - tp.x0;
      hi = (yc + p.wc + 1) * p.b - tp.x0 - 1;
    }
    pv.col[2 * jc] = penalty_unit<BF16>(lo, hi, nb);
    pv.col[2 * jc + 1] = penalty_unit<BF16>(lo - 8, hi - 8, nb);
  }
}

// Whole penalty row (four 16-byte units) of the streamed token at halo row `hr` / block column `jc`.
__device__ __forceinline__ void write_penalty_row_v(uint8_t* tile, int row, const PenView& pv, int hr, int jc, int th8, int tw8) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (u < th8) v = pv.row[2 * hr + u];
    else if (u - th8 < tw8) v = pv.col[2 * jc + (u - th8)];
    *reinterpret_cast<uint4*>(xtile_unit(tile, row, u)) = v;
  }
}

// Everything build_penalty_tables reads, relative to the resident tile: two tiles with the same signature have
// the same tables (all tiles whose halo the grid does not clip, for one).
__device__ __forceinline__ uint64_t penalty_signature(const KParams& p, const TilePos& tp) {
  const uint32_t up = (uint32_t)(tp.r0 - tp.hr_first), down = (uint32_t)(tp.hr_last - tp.r0);
  const uint32_t left = (uint32_t)max(0, -tp.hx0), right = (uint32_t)max(0, tp.hx0 + p.pl.pen_cols - p.Wtok);
  const uint32_t phase = (uint32_t)(tp.x0 - tp.hx0);           // fixes x0 modulo b_size and the window offset
  return ((uint64_t)(up | (down << 8) | (left << 16) | (right << 24))) | ((uint64_t)phase << 32);
}

// Penalty row of the streamed token at halo row index `hr` / halo column `jc` into row `row` of an x tile;
// part 0 = units 0-1, part 1 = units 2-3 (a row may be shared by two threads).  `th8` = TH / 8.
__device__ __forceinline__ void write_penalty_row(uint8_t* tile, int row, int part_lo, int part_hi,
                                                  const PenaltyTables* tab, int hr, int jc, int th8, int tw8) {
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    if ((u >> 1) < part_lo || (u >> 1) > part_hi) continue;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (u < th8) v = tab->row[hr][u];
    else if (u - th8 < tw8) v = tab->col[jc][u - th8];
    *reinterpret_cast<uint4*>(xtile_unit(tile, row, u)) = v;
  }
}

// The same for two rows at once, all table reads before all stores: a warp that writes four rows per lane would
// otherwise wait for every store before its next load (both go through shared memory, and the compiler has to
// assume that they alias).  A row index < 0 is skipped.
__device__ __forceinline__ void write_penalty_rows2(uint8_t* tile, int row0, int row1, const PenaltyTables* tab, int hr0,
                                                    int jc0, int hr1, int jc1, int th8, int tw8) {
  uint4 v[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int hr = i ? hr1 : hr0, jc = i ? jc1 : jc0;
    const bool on = (i ? row1 : row0) >= 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      v[i][u] = make_uint4(0u, 0u, 0u, 0u);
      if (on && u < th8) v[i][u] = ptx::lds128(ptx::smem_u32(&tab->row[hr][u]));
      else if (on && u - th8 < tw8) v[i][u] = ptx::lds128(ptx::smem_u32(&tab->col[jc][u - th8]));
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = i ? row1 : row0;
    if (row < 0) continue;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      ptx::sts128(ptx::smem_u32(xtile_unit(tile, row, u)), v[i][u].x, v[i][u].y, v[i][u].z, v[i][u].w);
  }
}

// Address of 16-byte unit `unit` (0..7) of row `row` in a swizzled 64-element-wide tile.
__device__ __forceinline__ uint8_t* swz(uint8_t* tile, int row, int unit) {
  return tile + row * 128 + ((unit ^ (row & 7)) << 4);
}

// ---- fused RoPE-2D on a swizzled q/k tile in shared memory ---------------------------------
// 128 threads rotate one tile of `rows` rows.  When 2*rows <= 128 two threads share a row (one
// rotates the row-angle pairs, dims [0,R) with [R,2R), the other the column-angle pairs, dims
// [2R,3R) with [3R,4R)); otherwise one thread does both halves of its row.  The cos/sin values
// a thread needs are fetched into registers ahead of time (RopeRow) -- right after it has
// finished its previous row, i.e. while it would otherwise wait for the next tile to arrive --
// because the tables are served by L2 (with ~200 KiB of shared memory per CTA there is hardly
// any L1 left) and a dependent chain of table loads per row would make these warps the
// bottleneck of the whole pipeline.  n_rdim = 8*NI, so the partner of a 16-byte unit is another
// whole unit of the same row.
struct RopeRow {
  float4 cs[16];   // (cos, sin) pairs: [first half handled][second half handled, if it fits]
  int pos[2];      // table rows of the row-angle / column-angle half; negative = not rotated
};

// Which halves a thread handles: [lo, hi].
struct RopeParts {
  int row, lo, hi;
  bool active;
};

// Share of thread t of `nthreads`: the first nthreads - rows rows are split between two threads
// (thread t: row-angle half of row t; thread rows + t: column-angle half), the others are whole.
__device__ __forceinline__ RopeParts rope_parts_n(int t, int rows, int nthreads) {
  RopeParts r;
  const int split = min(rows, nthreads - rows);
  if (t < rows) {
    r.active = true;
    r.row = t;
    r.lo = 0;
    r.hi = t < split ? 0 : 1;
  } else {
    r.row = t - rows;
    r.active = r.row < split;
    r.lo = r.hi = 1;
  }
  return r;
}

template <int NI>
__device__ __forceinline__ void rope_fetch_n(RopeRow& c, const RopeParts& pt, const RopeDev& rp) {
  constexpr int R = 8 * NI;
  const int first = pt.lo;
  const int pos_first = first ? c.pos[1] : c.pos[0];
  if (pos_first >= 0) {
    const float4* t4 = reinterpret_cast<const float4*>((first ? rp.col_cs : rp.row_cs) + (int64_t)pos_first * R * 2);
#pragma unroll
    for (int i = 0; i < NI * 4; ++i) c.cs[i] = __ldg(t4 + i);
  }
  if (NI <= 2 && pt.hi > pt.lo && c.pos[1] >= 0) {
    const float4* t4 = reinterpret_cast<const float4*>(rp.col_cs + (int64_t)c.pos[1] * R * 2);
#pragma unroll
    for (int i = 0; i < NI * 4; ++i) c.cs[(NI * 4 + i) & 15] = __ldg(t4 + i);
  }
}

// Rotate one half (0 = row-angle pairs, 1 = column-angle pairs) of a row with NI*4 float4 of (cos, sin).
template <bool BF16, int NI>
__device__ __forceinline__ void rope_rotate_half(uint8_t* tile, uint32_t chunk_stride, int row, int half,
                                                 const float4* cs) {
  constexpr int R = 8 * NI;
  uint32_t a0[NI], a1[NI];
  uint4 va[NI], vb[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) {  // all loads first
    const int d0 = 2 * half * R + i * 8, d1 = d0 + R;
    a0[i] = ptx::smem_u32(swz(tile + (d0 >> 6) * chunk_stride, row, (d0 & 63) >> 3));
    a1[i] = ptx::smem_u32(swz(tile + (d1 >> 6) * chunk_stride, row, (d1 & 63) >> 3));
    va[i] = ptx::lds128(a0[i]);
    vb[i] = ptx::lds128(a1[i]);
  }
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    uint32_t* pa = reinterpret_cast<uint32_t*>(&va[i]);
    uint32_t* pb = reinterpret_cast<uint32_t*>(&vb[i]);
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float4 c = cs[i * 4 + h];  // (cos, sin) of pairs 2h and 2h+1
      const float2 x0 = unpack2<BF16>(pa[h]), x1 = unpack2<BF16>(pb[h]);
      pa[h] = pack2<BF16>(x0.x * c.x - x1.x * c.y, x0.y * c.z - x1.y * c.w);
      pb[h] = pack2<BF16>(x0.x * c.y + x1.x * c.x, x0.y * c.w + x1.y * c.z);
    }
    ptx::sts128(a0[i], pa[0], pa[1], pa[2], pa[3]);
    ptx::sts128(a1[i], pb[0], pb[1], pb[2], pb[3]);
  }
}

template <bool BF16, int NI>
__device__ __forceinline__ void rope_apply_n(uint8_t* tile, uint32_t chunk_stride, RopeRow& c, const RopeParts& pt,
                                             const RopeDev& rp) {
  const int first = pt.lo;
  if ((first ? c.pos[1] : c.pos[0]) >= 0) rope_rotate_half<BF16, NI>(tile, chunk_stride, pt.row, first, &c.cs[0]);
  if (pt.hi > pt.lo && c.pos[1] >= 0) {
    if constexpr (NI <= 2) {
      rope_rotate_half<BF16, NI>(tile, chunk_stride, pt.row, 1, &c.cs[NI * 4]);
    } else {  // n_rdim 32: the second half did not fit the register cache
      const float4* t4 = reinterpret_cast<const float4*>(rp.col_cs + (int64_t)c.pos[1] * (8 * NI) * 2);
#pragma unroll
      for (int i = 0; i < 16; ++i) c.cs[i] = __ldg(t4 + i);
      rope_rotate_half<BF16, NI>(tile, chunk_stride, pt.row, 1, &c.cs[0]);
    }
  }
}

// Entry points with the table width fixed at compile time (NI = n_rdim / 8; 0 = no rotation): a
// kernel instantiated for one width carries one copy of the rotation code instead of three.
// rope_fetch_t starts fetching the cos/sin rows of the token with packed index `packed` (-1: nothing
// to do), rope_apply_t rotates this thread's share of the tile with the fetched values.
template <int NI>
__device__ __forceinline__ void rope_fetch_t(RopeRow& c, int32_t packed, const RopeParts& pt, const RopeDev& rp) {
  if constexpr (NI > 0) {
    decode_idx(packed, rp.max_h, rp.max_w, c.pos[0], c.pos[1]);
    rope_fetch_n<NI>(c, pt, rp);
  }
}
template <bool BF16, int NI>
__device__ __forceinline__ void rope_apply_t(uint8_t* tile, uint32_t chunk_stride, RopeRow& c, const RopeParts& pt,
                                             const RopeDev& rp) {
  if constexpr (NI > 0) rope_apply_n<BF16, NI>(tile, chunk_stride, c, pt, rp);
}

// ---- the same rotation with the cos/sin tables staged in shared memory ------------------------
// When both tables fit ((max_h + max_w) * n_rdim * 8 bytes), a persistent CTA copies them into
// shared memory once; a rotating thread then reads its (cos, sin) values with shared-memory
// latency, no register cache and no look-ahead are needed, and the rotation code shrinks to one
// loop over the (at most two) halves of a row.
// A staged table row takes n_rdim*8 + 16 bytes: the threads of a warp read the rows of neighbouring
// positions with 16-byte loads, and the 16 bytes of padding spread them over the banks.
struct RopeTabs {
  uint32_t row_addr, col_addr;   // shared-space byte addresses of the row / column table
};
__host__ __device__ __forceinline__ uint32_t rope_tab_stride(int n_rdim) { return (uint32_t)n_rdim * 8u + 16u; }

__device__ __forceinline__ void stage_rope_tables(uint8_t* dst, const RopeDev& rp, int tid, int nthreads) {
  const int per_row = rp.R / 2;                                         // float4 = two (cos, sin) pairs
  const uint32_t stride = rope_tab_stride(rp.R);
  const float4* src_r = reinterpret_cast<const float4*>(rp.row_cs);
  const float4* src_c = reinterpret_cast<const float4*>(rp.col_cs);
  uint8_t* dst_c = dst + (size_t)rp.max_h * stride;
#pragma unroll 1
  for (int i = tid; i < rp.max_h * per_row; i += nthreads) {
    const int r = i / per_row, c = i - r * per_row;
    *reinterpret_cast<float4*>(dst + (size_t)r * stride + c * 16) = __ldg(src_r + i);
  }
#pragma unroll 1
  for (int i = tid; i < rp.max_w * per_row; i += nthreads) {
    const int r = i / per_row, c = i - r * per_row;
    *reinterpret_cast<float4*>(dst_c + (size_t)r * stride + c * 16) = __ldg(src_c + i);
  }
}

template <bool BF16, int NI>
__device__ __forceinline__ void rope_apply_s(uint8_t* tile, uint32_t chunk_stride, int32_t packed, const RopeParts& pt,
                                             const RopeDev& rp, const RopeTabs& tabs) {
  if constexpr (NI > 0) {
    constexpr int R = 8 * NI;
    int pos[2];
    decode_idx(packed, rp.max_h, rp.max_w, pos[0], pos[1]);
#pragma unroll 1
    for (int half = pt.lo; half <= pt.hi; ++half) {
      const int ps = half ? pos[1] : pos[0];
      if (ps < 0) continue;
      const uint32_t cs_addr = (half ? tabs.col_addr : tabs.row_addr) + (uint32_t)ps * rope_tab_stride(R);
      uint32_t a0[NI], a1[NI];
      uint4 va[NI], vb[NI];
#pragma unroll
      for (int i = 0; i < NI; ++i) {  // all loads first
        const int d0 = 2 * half * R + i * 8, d1 = d0 + R;
        a0[i] = ptx::smem_u32(swz(tile + (d0 >> 6) * chunk_stride, pt.row, (d0 & 63) >> 3));
        a1[i] = ptx::smem_u32(swz(tile + (d1 >> 6) * chunk_stride, pt.row, (d1 & 63) >> 3));
        va[i] = ptx::lds128(a0[i]);
        vb[i] = ptx::lds128(a1[i]);
      }
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        uint32_t* pa = reinterpret_cast<uint32_t*>(&va[i]);
        uint32_t* pb = reinterpret_cast<uint32_t*>(&vb[i]);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const uint4 cu = ptx::lds128(cs_addr + (i * 4 + h) * 16);   // (cos, sin) of pairs 2h and 2h+1
          const float cx = __uint_as_float(cu.x), cy = __uint_as_float(cu.y), cz = __uint_as_float(cu.z), cw = __uint_as_float(cu.w);
          const float2 x0 = unpack2<BF16>(pa[h]), x1 = unpack2<BF16>(pb[h]);
          pa[h] = pack2<BF16>(x0.x * cx - x1.x * cy, x0.y * cz - x1.y * cw);
          pb[h] = pack2<BF16>(x0.x * cy + x1.x * cx, x0.y * cw + x1.y * cz);
        }
        ptx::sts128(a0[i], pa[0], pa[1], pa[2], pa[3]);
        ptx::sts128(a1[i], pb[0], pb[1], pb[2], pb[3]);
      }
    }
  }
}

// Performance tracing of one CTA: role `role` stores its k-th clock sample.
// Compiled in only with -DSWA_TC_TRACE: the marks cost instructions in the scalar roles.
__device__ __forceinline__ void trace_mark(const KParams& p, int role, int k) {
#ifdef SWA_TC_TRACE
  if (p.trace != nullptr && blockIdx.x == 37 && blockIdx.y == (gridDim.y > 1 ? 1 : 0) && k < 32) p.trace[role * 32 + k] = clock64();
#endif
}

// Event log of one CTA (performance debugging, -DSWA_TC_TRACE only): one designated thread of a role
// appends (clock << 8 | tag) to that role's row of 256 entries; `n` is the thread's own cursor.
__device__ __forceinline__ void trace_ev(const KParams& p, int role, int& n, bool on, int tag) {
#ifdef SWA_TC_TRACE
  if (on && p.trace != nullptr && blockIdx.x == 37 && n < 256) p.trace[128 + role * 256 + n++] = (clock64() << 8) | (long long)(tag & 255);
#endif
}

// Record a timed-out wait (first one wins) so the host can report it.
__device__ __forceinline__ void report_abort(int32_t* status, int code, int where) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = blockIdx.x;
    status[2] = blockIdx.y;
    status[3] = where;
  }
}

}  // namespace tc
}  // namespace swa
