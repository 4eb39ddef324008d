// Shared declarations of the CPU oracle. TEST INFRASTRUCTURE ONLY (see oracle.h).
#pragma once
#include "oracle.h"
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace orc {

constexpr int TILE = 8;            // rasteriser tile edge (util.cuh:19)
constexpr double T_CUTOFF = 1e-4;  // splat_math.cuh:8-9
constexpr double ALPHA_MAX = 0.999;

// Everything the projection yields that its backward re-derives (the fields of ProjIntermediates,
// splat_math.cuh:199-217).
struct Proj {
  bool ok = false;
  double mean_c[3];
  double s[3], s2_raw[3], comp_floor;
  double Rq[9];
  double J[6];
  bool clamp_x, clamp_y;
  double cov[3];    // blurred 2D covariance (c00, c01, c11)
  double conic[3];
  double opac, sig, power;
  double mean2d[2];
  double ex, ey;
};

void quat_to_mat(const double q[4], double R[9]);
void sh_basis(int deg, const double v[3], double* b);
void sh_basis_grad(int deg, const double v[3], double (*db)[3]);
bool project_one(const float* po, const float* q, const float* ls, const OrcCamera& cam, Proj& r);

inline int tiles_x(int W) { return (W + TILE - 1) / TILE; }
inline int tiles_y(int H) { return (H + TILE - 1) / TILE; }

}  // namespace orc
