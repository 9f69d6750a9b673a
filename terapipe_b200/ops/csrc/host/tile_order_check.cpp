// Host-side walk of the GEMM tile orders (tile_order.h is the code the kernels run): for a
// problem size and a rank it builds the order the all-gather / reduce-scatter entry points would
// choose, maps every tile index through pair_tile_coords and reports what it finds.  Used by the
// CPU tests; no CUDA involved.
#include <vector>

#include "../tile_order.h"

extern "C" {

// kind: 0 plain, 1 all-gather -> GEMM, 2 GEMM -> reduce-scatter.
// order_out (8 ints, may be null): the TileOrder fields in declaration order.
// coords_out (2 * num_tiles ints, may be null): (m_idx, n_idx) of tile 0, 1, ...
// Returns the number of tiles, or -(1 + tile) for the first tile whose coordinates fall outside
// the grid or repeat an earlier tile's (i.e. the order is not a bijection).
long long tp_tile_order_walk(int kind, int M, int N, long long K, int tile_rows, int tile_cols,
                             int rank, int rows_per_rank, int pairs, int* order_out,
                             int* coords_out) {
  if (M <= 0 || N <= 0 || tile_rows <= 0 || tile_cols <= 0 || pairs <= 0) return 0;
  const int num_m = (M + tile_rows - 1) / tile_rows, num_n = (N + tile_cols - 1) / tile_cols;
  tp::TileOrder o = tp::plain_tile_order(num_m, num_n);
  if (kind == 1) o = tp::ag_tile_order(num_m, num_n, tile_rows, rank, rows_per_rank, pairs);
  if (kind == 2) o = tp::rs_tile_order(M, N, K, num_m, num_n, tile_rows, rank, rows_per_rank, pairs);
  if (order_out) {
    const int f[8] = {o.num_m_tiles, o.num_n_tiles, o.m_major, o.m_first,
                      o.order_split, o.order_group, o.order_first_only, o.order_pipelined};
    for (int i = 0; i < 8; ++i) order_out[i] = f[i];
  }
  const long long total = static_cast<long long>(num_m) * num_n;
  std::vector<char> seen(static_cast<size_t>(total), 0);
  for (long long t = 0; t < total; ++t) {
    int m = -1, n = -1;
    tp::pair_tile_coords(o, static_cast<int>(t), m, n);
    if (coords_out) { coords_out[2 * t] = m; coords_out[2 * t + 1] = n; }
    if (m < 0 || m >= num_m || n < 0 || n >= num_n) return -(1 + t);
    char& s = seen[static_cast<size_t>(n) * num_m + m];
    if (s) return -(1 + t);
    s = 1;
  }
  return total;
}

}  // extern "C"
