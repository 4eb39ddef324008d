// CPU oracle, stages 3 and 5: front-to-back compositing and its per-pixel reverse replay. TEST INFRASTRUCTURE ONLY.
// Forward follows raster_fwd_kernel (src/gpu/raster_fwd.cu:9-71); the depth accumulator follows the mean-depth mode
// of probe_kernel (src/gpu/probe.cu:30-46). Backward follows raster_bwd_kernel (src/gpu/raster_bwd.cu:11-143).
// The forward is pinned against tests/reference.cpp:84-104 (same compositing, untiled); the backward is pinned by
// central differences of that function.
#include "oracle_internal.h"

using namespace orc;

namespace {
struct Frag { double mx, my, c00, c01, c11, opac, z, power; };
inline Frag frag_of(const double* geo, uint32_t gid) {
  const double* g = geo + (size_t)gid * 8;
  return Frag{g[0], g[1], g[2], g[3], g[4], g[5], g[6], g[7]};
}
}  // namespace

extern "C" void orc_raster_fwd(int W, int H, const double* geo, const double* col, const uint32_t* vals_sorted,
                               uint32_t* tile_ranges, const double* bg, int bwd_info, double* out_rgba, double* out_T,
                               uint32_t* last_idx, double* out_depth) {
  const int txn = tiles_x(W), tyn = tiles_y(H);
#pragma omp parallel for schedule(dynamic, 4)
  for (int tile = 0; tile < txn * tyn; tile++) {
    const int tx = tile % txn, ty = tile / txn;
    const uint32_t r0 = tile_ranges[tile * 2], r1 = tile_ranges[tile * 2 + 1];
    uint32_t max_last = r0;
    for (int ly = 0; ly < TILE; ly++) for (int lx = 0; lx < TILE; lx++) {
      const int px = tx * TILE + lx, py = ty * TILE + ly;
      if (px >= W || py >= H) continue;
      const double pcx = px + 0.5, pcy = py + 0.5;
      double T = 1, r = 0, g = 0, b = 0, zs = 0;
      uint32_t last = r0;
      for (uint32_t idx = r0; idx < r1; idx++) {
        const uint32_t gid = vals_sorted[idx];
        const Frag f = frag_of(geo, gid);
        const double dx = pcx - f.mx, dy = pcy - f.my;
        const double sigma = 0.5 * (f.c00 * dx * dx + f.c11 * dy * dy) + f.c01 * dx * dy;
        if (sigma < 0 || sigma > f.power) continue;
        const double alpha = std::min(ALPHA_MAX, f.opac * std::exp(-sigma));
        const double next_T = T * (1 - alpha);
        if (next_T <= T_CUTOFF) break;
        const double vis = alpha * T;
        const double* c = col + (size_t)gid * 3;
        r += std::max(c[0], 0.0) * vis; g += std::max(c[1], 0.0) * vis; b += std::max(c[2], 0.0) * vis;
        zs += vis * f.z;
        T = next_T;
        last = idx + 1;
      }
      const size_t pix = (size_t)py * W + px;
      out_rgba[pix * 4] = r + T * bg[0]; out_rgba[pix * 4 + 1] = g + T * bg[1]; out_rgba[pix * 4 + 2] = b + T * bg[2]; out_rgba[pix * 4 + 3] = 1 - T;
      out_T[pix] = T;
      if (out_depth) out_depth[pix] = zs;
      if (last_idx) last_idx[pix] = last;
      max_last = std::max(max_last, last);
    }
    if (bwd_info) tile_ranges[tile * 2 + 1] = max_last;
  }
}

// The feature lanes of the forward (src/gpu/raster_fwd.cu:52,62): the same walk as orc_raster_fwd, accumulating
// feat * alpha * T with no clamp. tile_ranges as orc_bin left them (or shrunk: fragments past the shrunk end contribute
// to no pixel). out_feat: [P][3].
extern "C" void orc_raster_feat(int W, int H, const double* geo, const double* feat, const uint32_t* vals_sorted,
                                const uint32_t* tile_ranges, double* out_feat) {
  const int txn = tiles_x(W), tyn = tiles_y(H);
#pragma omp parallel for schedule(dynamic, 4)
  for (int tile = 0; tile < txn * tyn; tile++) {
    const int tx = tile % txn, ty = tile / txn;
    const uint32_t r0 = tile_ranges[tile * 2], r1 = tile_ranges[tile * 2 + 1];
    for (int ly = 0; ly < TILE; ly++) for (int lx = 0; lx < TILE; lx++) {
      const int px = tx * TILE + lx, py = ty * TILE + ly;
      if (px >= W || py >= H) continue;
      const double pcx = px + 0.5, pcy = py + 0.5;
      double T = 1, f0 = 0, f1 = 0, f2 = 0;
      for (uint32_t idx = r0; idx < r1; idx++) {
        const uint32_t gid = vals_sorted[idx];
        const Frag f = frag_of(geo, gid);
        const double dx = pcx - f.mx, dy = pcy - f.my;
        const double sigma = 0.5 * (f.c00 * dx * dx + f.c11 * dy * dy) + f.c01 * dx * dy;
        if (sigma < 0 || sigma > f.power) continue;
        const double alpha = std::min(ALPHA_MAX, f.opac * std::exp(-sigma));
        const double next_T = T * (1 - alpha);
        if (next_T <= T_CUTOFF) break;
        const double vis = alpha * T;
        const double* c = feat + (size_t)gid * 3;
        f0 += c[0] * vis; f1 += c[1] * vis; f2 += c[2] * vis;
        T = next_T;
      }
      const size_t pix = (size_t)py * W + px;
      out_feat[pix * 3] = f0; out_feat[pix * 3 + 1] = f1; out_feat[pix * 3 + 2] = f2;
    }
  }
}

extern "C" void orc_raster_bwd(int n, int W, int H, const double* geo, const double* col, const uint32_t* vals_sorted,
                               const uint32_t* tile_ranges, const double* bg, const double* out_rgba, const double* out_T,
                               const uint32_t* last_idx, const double* v_out, double* v_splat, uint32_t* vis_flag,
                               double* vis_weight) {
  std::memset(v_splat, 0, sizeof(double) * 13 * (size_t)n);
  std::memset(vis_flag, 0, sizeof(uint32_t) * (size_t)n);
  std::memset(vis_weight, 0, sizeof(double) * (size_t)n);
  const int txn = tiles_x(W), tyn = tiles_y(H);
  const double Wf = W, Hf = H;
  // Tiles write to shared per-splat rows: serialise the accumulation per tile batch through per-thread buffers kept
  // sparse (touched rows only), then merge. Simple and deterministic enough for a checker.
#pragma omp parallel
  {
    std::vector<double> acc;         // [touched][14]
    std::vector<uint32_t> ids;
#pragma omp for schedule(dynamic, 4)
    for (int tile = 0; tile < txn * tyn; tile++) {
      const uint32_t r0 = tile_ranges[tile * 2], r1 = tile_ranges[tile * 2 + 1];
      if (r1 <= r0) continue;
      const int tx = tile % txn, ty = tile / txn;
      const uint32_t cnt = r1 - r0;
      acc.assign((size_t)cnt * 14, 0.0);
      ids.assign(cnt, 0u);
      std::vector<uint8_t> touched(cnt, 0);
      for (int ly = 0; ly < TILE; ly++) for (int lx = 0; lx < TILE; lx++) {
        const int px = tx * TILE + lx, py = ty * TILE + ly;
        if (px >= W || py >= H) continue;
        const size_t pix = (size_t)py * W + px;
        const double pcx = px + 0.5, pcy = py + 0.5;
        const double final_a = out_rgba[pix * 4 + 3];
        double T = out_T[pix];
        const uint32_t last = last_idx[pix];
        const double* vo = v_out + pix * 4;
        const double v_o_w = (vo[3] - (bg[0] * vo[0] + bg[1] * vo[1] + bg[2] * vo[2])) * T;
        const double inv_final_a = 1.0 / std::max(final_a, 1e-5);
        double S[3] = {0, 0, 0};
        for (uint32_t idx = std::min(last, r1); idx > r0; idx--) {
          const uint32_t k = idx - 1 - r0;
          const uint32_t gid = vals_sorted[idx - 1];
          const Frag f = frag_of(geo, gid);
          const double dx = pcx - f.mx, dy = pcy - f.my;
          const double sigma = 0.5 * (f.c00 * dx * dx + f.c11 * dy * dy) + f.c01 * dx * dy;
          if (!(sigma >= 0 && sigma <= f.power)) continue;
          const double gauss = std::exp(-sigma);
          const double alpha = std::min(ALPHA_MAX, f.opac * gauss);
          const double ra = 1.0 / (1.0 - alpha);
          const double T_before = T * ra;
          const double vis = alpha * T_before;
          const double* c = col + (size_t)gid * 3;
          const double cc[3] = {std::max(c[0], 0.0), std::max(c[1], 0.0), std::max(c[2], 0.0)};
          double* a = acc.data() + (size_t)k * 14;
          ids[k] = gid; touched[k] = 1;
          for (int ch = 0; ch < 3; ch++) if (c[ch] >= 0) a[5 + ch] += vis * vo[ch];
          double v_alpha = v_o_w * ra;
          for (int ch = 0; ch < 3; ch++) v_alpha += (T_before * cc[ch] - S[ch] * ra) * vo[ch];
          const double v_sigma = -alpha * v_alpha;
          if (f.opac * gauss <= ALPHA_MAX) {
            const double gx = -v_sigma * (f.c00 * dx + f.c01 * dy), gy = -v_sigma * (f.c01 * dx + f.c11 * dy);
            a[0] += gx; a[1] += gy;
            a[2] += 0.5 * v_sigma * dx * dx; a[3] += v_sigma * dx * dy; a[4] += 0.5 * v_sigma * dy * dy;
            a[8] += v_alpha * gauss;
            a[9] += std::sqrt(gx * Wf * gx * Wf + gy * Hf * gy * Hf) * inv_final_a;
          }
          for (int ch = 0; ch < 3; ch++) S[ch] += cc[ch] * vis;
          T = T_before;
          a[13] += vis;
        }
      }
#pragma omp critical
      for (uint32_t k = 0; k < cnt; k++) if (touched[k]) {
        const uint32_t gid = ids[k];
        for (int l = 0; l < 13; l++) v_splat[(size_t)gid * 13 + l] += acc[(size_t)k * 14 + l];
        vis_weight[gid] += acc[(size_t)k * 14 + 13];
        vis_flag[gid] = 1;
      }
    }
  }
}
