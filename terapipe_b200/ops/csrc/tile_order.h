// Order in which the CTA pairs of the persistent GEMM walk the output tiles, and the choice of
// that order for the all-gather and reduce-scatter variants.  Plain C++ that compiles for the
// device (the kernel calls pair_tile_coords) and for the host (the entry points choose the
// order; a g++-built test harness walks every tile of an order and checks that the map is a
// bijection onto the tile grid and that the row blocks come in the promised sequence).
#pragma once

#if defined(__CUDACC__)
#define TP_HD __host__ __device__ __forceinline__
#else
#define TP_HD inline
#endif

namespace tp {

// m_major = 0: consecutive tiles walk down a column of the output (tile -> m = tile %
// num_m_tiles), so the CTAs of a wave share few B tiles.  m_major = 1: the columns are taken in
// groups of order_group; inside a group the row blocks are split in two phases: first the
// `order_split` row blocks starting at m_first (wrapping around) for every column of the group,
// then the remaining row blocks for every column, row block fastest in both.
// order_first_only = 1 applies the split to the first group only.  order_pipelined = 1
// interleaves the phases of successive groups (A0 A1 B0 A2 B1 ... B_last): a group's second
// phase then runs one first phase after its own, while its B tiles are still in L2.
struct TileOrder {
  int num_m_tiles, num_n_tiles;
  int m_major, m_first, order_split, order_group, order_first_only, order_pipelined;
};

TP_HD int tile_order_min(int a, int b) { return a < b ? a : b; }

// P: any struct with the fields of TileOrder (the kernel passes its parameter block).
template <class P>
TP_HD void pair_tile_coords(const P& p, int tile, int& m_idx, int& n_idx) {
  if (!p.m_major) {
    m_idx = tile % p.num_m_tiles;
    n_idx = tile / p.num_m_tiles;
    return;
  }
  if (p.order_pipelined) {
    const int G = p.order_group, split = p.order_split, rest = p.num_m_tiles - split;
    const int ng = (p.num_n_tiles + G - 1) / G;
    int t = tile, phase = -1, g = 0;
    const int c0 = tile_order_min(G, p.num_n_tiles);
    if (t < split * c0) {
      phase = 0;
    } else {
      t -= split * c0;
      for (int k = 1; k < ng; ++k) {
        const int ck = tile_order_min(G, p.num_n_tiles - k * G);
        if (t < split * ck) { phase = 0; g = k; break; }
        t -= split * ck;
        if (t < rest * G) { phase = 1; g = k - 1; break; }
        t -= rest * G;
      }
      if (phase < 0) { phase = 1; g = ng - 1; }
    }
    int j;
    if (phase == 0) { j = t % split; n_idx = g * G + t / split; }
    else { j = split + t % rest; n_idx = g * G + t / rest; }
    m_idx = (j + p.m_first) % p.num_m_tiles;
    return;
  }
  const int per_group = p.num_m_tiles * p.order_group;
  const int g = tile / per_group, r = tile % per_group;
  const int cols = tile_order_min(p.order_group, p.num_n_tiles - g * p.order_group);
  int j;
  if (p.order_first_only && g > 0) {
    j = r % p.num_m_tiles;
    n_idx = g * p.order_group + r / p.num_m_tiles;
  } else if (r < p.order_split * cols) {
    j = r % p.order_split;
    n_idx = g * p.order_group + r / p.order_split;
  } else {
    const int r2 = r - p.order_split * cols, cnt = p.num_m_tiles - p.order_split;
    j = p.order_split + r2 % cnt;
    n_idx = g * p.order_group + r2 / cnt;
  }
  m_idx = (j + p.m_first) % p.num_m_tiles;
}

inline TileOrder plain_tile_order(int num_m_tiles, int num_n_tiles) {
  TileOrder o;
  o.num_m_tiles = num_m_tiles; o.num_n_tiles = num_n_tiles;
  o.m_major = 0; o.m_first = 0; o.order_split = 1; o.order_group = 1;
  o.order_first_only = 0; o.order_pipelined = 0;
  return o;
}

// All-gather -> GEMM: rank `rank` holds rows [rank * rows_per_rank, (rank + 1) * rows_per_rank)
// of A locally while the peers' rows are still arriving, so the first wave of tiles (`pairs`
// tiles run at a time) takes row blocks of this rank only; later tiles use the ordinary order.
// tile_rows: rows of one tile.
inline TileOrder ag_tile_order(int num_m_tiles, int num_n_tiles, int tile_rows, int rank,
                               int rows_per_rank, int pairs) {
  TileOrder o = plain_tile_order(num_m_tiles, num_n_tiles);
  const int own_tiles = (rows_per_rank + tile_rows - 1) / tile_rows;
  if (own_tiles < num_m_tiles) {
    o.m_major = 1;
    o.m_first = static_cast<int>((static_cast<long long>(rank) * rows_per_rank) / tile_rows) % num_m_tiles;
    o.order_split = own_tiles;
    o.order_group = (pairs + own_tiles - 1) / own_tiles;
    if (o.order_group > num_n_tiles) o.order_group = num_n_tiles;
    o.order_first_only = 1;
  }
  return o;
}

// GEMM -> reduce-scatter over the rows of an M x N product with inner dimension K: the row
// blocks of the other ranks first (starting after this rank's rows), this rank's own row blocks
// last, so that a partial is always consumed well after the peer produced it.  One column group
// unless the B operand (N x K 16-bit elements) is too large to stay in L2 between the two
// phases: then column groups with the phases of successive groups interleaved, the group sized
// so that about 10 us of other tiles lie between a partial's production and its use.
// tile_rows: rows of one (CTA-pair) tile.
inline TileOrder rs_tile_order(int M, int N, long long K, int num_m_tiles, int num_n_tiles,
                               int tile_rows, int rank, int rows_per_rank, int pairs) {
  TileOrder o = plain_tile_order(num_m_tiles, num_n_tiles);
  o.order_split = 1;
  const long long first_after = static_cast<long long>(rank + 1) * rows_per_rank;
  const long long my_end = first_after < M ? first_after : M;
  const long long my_begin = static_cast<long long>(rank) * rows_per_rank;
  const int own_tiles =
      my_begin >= M ? 0 : static_cast<int>((my_end + tile_rows - 1) / tile_rows - my_begin / tile_rows);
  if (own_tiles > 0 && own_tiles < num_m_tiles) {
    o.m_major = 1;
    o.m_first = first_after >= M ? 0 : static_cast<int>((first_after + tile_rows - 1) / tile_rows) % num_m_tiles;
    o.order_split = num_m_tiles - own_tiles;
    o.order_group = num_n_tiles;
    if (static_cast<long long>(N) * K * 2 > (48ll << 20)) {
      const float tile_us = 0.0046f * static_cast<float>(K);
      int g = static_cast<int>(pairs * 10.0f / (tile_us * o.order_split)) + 1;
      if (g < 2) g = 2;
      if (g < num_n_tiles) {
        const int ng = (num_n_tiles + g - 1) / g;
        o.order_group = (num_n_tiles + ng - 1) / ng;
        o.order_pipelined = 1;
      }
    }
  }
  return o;
}

// Copy an order into a parameter block with the same field names.
template <class P> inline void apply_tile_order(P& p, const TileOrder& o) {
  p.m_major = o.m_major; p.m_first = o.m_first; p.order_split = o.order_split;
  p.order_group = o.order_group; p.order_first_only = o.order_first_only;
  p.order_pipelined = o.order_pipelined;
}

}  // namespace tp
