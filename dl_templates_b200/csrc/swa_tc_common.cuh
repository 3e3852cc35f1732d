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
constexpr int kMaxStages = 4;

struct Plan {
  int TH, TW;          // resident tile: rows x token columns (TH*TW == 128)
  int KR, KW, N;       // streamed block: rows x token columns, N = KR*KW
  int n_tiles_x, n_tiles_y;
  int stages, pbufs;   // streamed-block pipeline depth, buffers for the P/dS operand
  uint32_t smem_bytes;
};

struct KParams {
  int t_h, Wtok, b, wr, wc, H;
  int qch, vch;        // d_qk/64, d_v/64
  float scale_log2, sm_scale;
  Plan pl;
  RopeDev rope;
  int32_t* status;
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
  t.nblk = (t.hr_last - t.hr_first + p.pl.KR) / p.pl.KR;
  return t;
}

// Bit jc of the result: halo column jc (token column hx0+jc) is inside the grid and
// within wc tile columns of token column `x`.  Zero when `x` itself is outside.
__device__ __forceinline__ uint64_t column_mask(const KParams& p, int hx0, int x, bool row_in_grid) {
  if (!row_in_grid || x >= p.Wtok) return 0ull;
  const int c = x / p.b;
  const int lo = max(0, (c - p.wc) * p.b) - hx0;
  const int hi = min(p.Wtok, (c + p.wc + 1) * p.b) - hx0;  // exclusive
  const int n = hi - lo;
  if (n <= 0) return 0ull;
  const uint64_t ones = n >= 64 ? ~0ull : ((1ull << n) - 1ull);
  return ones << lo;
}

// vm (128 bits) |= colmask << shift, 0 <= shift < 128, with static word indexing.
__device__ __forceinline__ void or_shifted(uint32_t (&vm)[4], uint64_t colmask, int shift) {
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const int rel = 32 * w - shift;  // bit `rel` of colmask lands on bit 0 of word w
    uint32_t part;
    if (rel >= 64 || rel <= -32) part = 0u;
    else if (rel >= 0) part = (uint32_t)(colmask >> rel);
    else part = (uint32_t)(colmask << (-rel));
    vm[w] |= part;
  }
}

// Validity bits of the N = KR*KW entries of one streamed block for the resident token
// at row `r` (column validity precomputed in colmask): entry j = jr*KW + jc.
__device__ __forceinline__ void block_mask(uint32_t (&vm)[4], const KParams& p, uint64_t colmask, int brow0, int r,
                                           int hr_last) {
  vm[0] = vm[1] = vm[2] = vm[3] = 0u;
  for (int jr = 0; jr < p.pl.KR; ++jr) {
    const int kr = brow0 + jr;
    if (kr <= hr_last && kr - r <= p.wr && r - kr <= p.wr) or_shifted(vm, colmask, jr * p.pl.KW);
  }
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

// Address of 16-byte unit `unit` (0..7) of row `row` in a swizzled 64-element-wide tile.
__device__ __forceinline__ uint8_t* swz(uint8_t* tile, int row, int unit) {
  return tile + row * 128 + ((unit ^ (row & 7)) << 4);
}

// Rotate, in shared memory, row `row` of a q/k tile (chunks `chunk_stride` bytes
// apart) by the RoPE-2D angles of token `token`.  n_rdim is a multiple of 8 here, so
// the partner of a 16-byte unit is another whole unit of the same row.
template <bool BF16>
__device__ __forceinline__ void rotate_row_smem(uint8_t* tile, uint32_t chunk_stride, int row, int token,
                                                const RopeDev& rp) {
  int irow, icol;
  decode_idx(rp.idx[token], rp.max_h, rp.max_w, irow, icol);
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const int pos = half ? icol : irow;
    if (pos < 0) continue;
    const float* tab = (half ? rp.col_cs : rp.row_cs) + (int64_t)pos * rp.R * 2;
#pragma unroll 1
    for (int i0 = 0; i0 < rp.R; i0 += 8) {
      const int d0 = 2 * half * rp.R + i0, d1 = d0 + rp.R;
      uint8_t* a0 = swz(tile + (d0 >> 6) * chunk_stride, row, (d0 & 63) >> 3);
      uint8_t* a1 = swz(tile + (d1 >> 6) * chunk_stride, row, (d1 & 63) >> 3);
      uint4 va = *reinterpret_cast<uint4*>(a0), vb = *reinterpret_cast<uint4*>(a1);
      uint32_t* pa = reinterpret_cast<uint32_t*>(&va);
      uint32_t* pb = reinterpret_cast<uint32_t*>(&vb);
      const float4* t4 = reinterpret_cast<const float4*>(tab + 2 * i0);
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float4 cs = __ldg(t4 + h);  // (cos, sin) of pairs 2h and 2h+1
        const float2 x0 = unpack2<BF16>(pa[h]), x1 = unpack2<BF16>(pb[h]);
        pa[h] = pack2<BF16>(x0.x * cs.x - x1.x * cs.y, x0.y * cs.z - x1.y * cs.w);
        pb[h] = pack2<BF16>(x0.x * cs.y + x1.x * cs.x, x0.y * cs.w + x1.y * cs.z);
      }
      *reinterpret_cast<uint4*>(a0) = va;
      *reinterpret_cast<uint4*>(a1) = vb;
    }
  }
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
