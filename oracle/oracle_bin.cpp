// CPU oracle, stage 2: exact ellipse-to-tile binning and the (tile, depth, index) order. TEST INFRASTRUCTURE ONLY.
// Follows tile_bbox / tile_hit (src/gpu/splat_math.cuh:27-53), the extent and on-screen culls of project_one
// (splat_math.cuh:284-290), the depth key and the two stable sorts of bin_and_sort (src/gpu/binning.cu:10-15,
// 109-145) and tile_ranges_kernel (binning.cu:95-105).
//
// This file is single-precision on purpose: the decisions are a function of fp32 records, and the CUDA kernels
// evaluate the same expression tree with round-to-nearest intrinsics. Build with -ffp-contract=off and no fast-math
// so each operation below rounds exactly once. The reference has no CPU statement of this stage: parity unpinned by
// the reference, pinned here by bit-exact agreement between this file and the kernels on identical records.
#include "oracle_internal.h"

namespace {

inline float fmul(float a, float b) { return a * b; }
inline float fadd(float a, float b) { return a + b; }
inline float fsub(float a, float b) { return a - b; }
inline float fdiv(float a, float b) { return a / b; }
inline float clamp01(float x) { return fminf(fmaxf(x, 0.f), 1.f); }

struct Rec {
  float mx, my, c00, c01, c11, power;
  float ia() const { return fdiv(1.f, fmul(64.f, c00)); }   // per-splat denominators of the closest-point parameters
  float ib() const { return fdiv(1.f, fmul(64.f, c11)); }
};

inline float sigma_at(float px, float py, const Rec& r) {
  const float dx = fsub(px, r.mx), dy = fsub(py, r.my);
  const float q = fadd(fmul(fmul(r.c00, dx), dx), fmul(fmul(r.c11, dy), dy));
  return fadd(fmul(0.5f, q), fmul(fmul(r.c01, dx), dy));
}

// Closest point of the tile rectangle to the ellipse centre in the conic's metric (the StopThePop test).
inline bool tile_hit(int tx, int ty, const Rec& r) {
  const float rmin_x = (float)(tx * orc::TILE), rmin_y = (float)(ty * orc::TILE);
  const float rmax_x = rmin_x + (float)orc::TILE, rmax_y = rmin_y + (float)orc::TILE;
  const bool x_left = r.mx < rmin_x, x_right = r.mx > rmax_x, in_x = !(x_left || x_right);
  const bool y_above = r.my < rmin_y, y_below = r.my > rmax_y, in_y = !(y_above || y_below);
  if (in_x && in_y) return true;
  const float corner_x = x_left ? rmin_x : rmax_x, corner_y = y_above ? rmin_y : rmax_y;
  const float dxf = x_left ? (float)orc::TILE : -(float)orc::TILE, dyf = y_above ? (float)orc::TILE : -(float)orc::TILE;
  const float diff_x = fsub(r.mx, corner_x), diff_y = fsub(r.my, corner_y);
  const float tx_raw = fmul(fmul(dxf, fadd(fmul(r.c00, diff_x), fmul(r.c01, diff_y))), r.ia());
  const float ty_raw = fmul(fmul(dyf, fadd(fmul(r.c01, diff_x), fmul(r.c11, diff_y))), r.ib());
  const float tx_c = in_y ? 0.f : clamp01(tx_raw), ty_c = in_x ? 0.f : clamp01(ty_raw);
  const float px = fadd(corner_x, fmul(tx_c, dxf)), py = fadd(corner_y, fmul(ty_c, dyf));
  return sigma_at(px, py, r) <= r.power;
}

struct Box { int min_x, min_y, max_x, max_y; };

// Returns false when the record is culled by the determinant, extent or on-screen tests.
inline bool tile_box(const Rec& r, int W, int H, Box& b) {
  const float detc = fsub(fmul(r.c00, r.c11), fmul(r.c01, r.c01));
  if (!(detc > 0.f)) return false;
  const float inv = fdiv(1.f, detc);
  const float p2 = fmul(2.f, r.power);
  const float ex = sqrtf(fmul(fmul(p2, r.c11), inv)), ey = sqrtf(fmul(fmul(p2, r.c00), inv));
  if (!(ex >= 0.f && ey >= 0.f)) return false;
  const bool on = fadd(r.mx, ex) > 0.f && fsub(r.mx, ex) < (float)W && fadd(r.my, ey) > 0.f && fsub(r.my, ey) < (float)H;
  if (!on) return false;
  const float tw = (float)orc::TILE, txs = (float)orc::tiles_x(W), tys = (float)orc::tiles_y(H);
  const float cx = fdiv(r.mx, tw), cy = fdiv(r.my, tw), dx = fdiv(ex, tw), dy = fdiv(ey, tw);
  b.min_x = (int)fminf(fmaxf(fsub(cx, dx), 0.f), txs);
  b.min_y = (int)fminf(fmaxf(fsub(cy, dy), 0.f), tys);
  b.max_x = (int)fminf(fmaxf(fadd(fadd(cx, dx), 1.f), 0.f), txs);
  b.max_y = (int)fminf(fmaxf(fadd(fadd(cy, dy), 1.f), 0.f), tys);
  return true;
}

template <class F>
inline int for_each_tile(const Rec& r, int W, int H, F&& f) {
  Box b;
  if (!tile_box(r, W, H, b)) return 0;
  const int tx_n = orc::tiles_x(W);
  int hits = 0;
  for (int ty = b.min_y; ty < b.max_y; ty++)
    for (int tx = b.min_x; tx < b.max_x; tx++)
      if (tile_hit(tx, ty, r)) { f((uint32_t)(ty * tx_n + tx)); hits++; }
  return hits;
}

inline uint32_t float_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

}  // namespace

extern "C" int orc_tiles_of_record(float mx, float my, float c00, float c01, float c11, float power, int W, int H,
                                   uint32_t* tiles, int max_tiles) {
  Rec r{mx, my, c00, c01, c11, power};
  int k = 0;
  return for_each_tile(r, W, H, [&](uint32_t t) { if (tiles && k < max_tiles) tiles[k] = t; k++; });
}

extern "C" int64_t orc_bin(int n, const float* proj0, const float* proj1, int W, int H, uint32_t* tile_count,
                           uint32_t* vals_sorted, uint32_t* keys_sorted, int64_t cap, uint32_t* tile_ranges) {
  const int n_tiles = orc::tiles_x(W) * orc::tiles_y(H);
  auto rec_of = [&](int i) { return Rec{proj0[i * 4], proj0[i * 4 + 1], proj0[i * 4 + 2], proj0[i * 4 + 3], proj1[i * 4], proj1[i * 4 + 3]}; };
#pragma omp parallel for schedule(dynamic, 1024)
  for (int i = 0; i < n; i++) {
    tile_count[i] = 0;
    if (!(proj1[i * 4 + 3] > -0.5f)) continue;  // no record
    tile_count[i] = (uint32_t)for_each_tile(rec_of(i), W, H, [](uint32_t) {});
  }
  // Depth order: ascending raw bits of z, ties by index (key and value of binning.cu:13-14 under a stable sort).
  std::vector<uint32_t> order;
  for (int i = 0; i < n; i++) if (tile_count[i]) order.push_back((uint32_t)i);
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return float_bits(proj1[a * 4 + 2]) < float_bits(proj1[b * 4 + 2]); });
  // Counting sort by tile keeps the depth order inside each tile (the second stable sort, binning.cu:140-142).
  std::vector<int64_t> start((size_t)n_tiles + 1, 0);
  for (uint32_t i : order) for_each_tile(rec_of((int)i), W, H, [&](uint32_t t) { start[t + 1]++; });
  for (int t = 0; t < n_tiles; t++) start[t + 1] += start[t];
  const int64_t total = start[n_tiles];
  for (int t = 0; t < n_tiles; t++) {
    const bool empty = start[t + 1] == start[t];  // untouched tiles keep the zero fill (binning.cu:134)
    tile_ranges[t * 2] = empty ? 0u : (uint32_t)start[t];
    tile_ranges[t * 2 + 1] = empty ? 0u : (uint32_t)start[t + 1];
  }
  std::vector<int64_t> cur(start.begin(), start.end() - 1);
  for (uint32_t i : order)
    for_each_tile(rec_of((int)i), W, H, [&](uint32_t t) {
      const int64_t at = cur[t]++;
      if (at < cap) { if (vals_sorted) vals_sorted[at] = i; if (keys_sorted) keys_sorted[at] = t; }
    });
  return total;
}
