// CPU oracle, stage 1: EWA projection with the 3D-filter floor and SH colour, in double. TEST INFRASTRUCTURE ONLY.
// Follows project_one (src/gpu/splat_math.cuh:224-293), sh_eval (splat_math.cuh:68-117) and the colour clamp of
// project_kernel (src/gpu/project.cu:44-55). The reference's CPU check (tests/reference.cpp:41-77) covers the same
// math without the floor and up to SH degree 3; those parts are pinned against it, the rest is unpinned.
#include "oracle_internal.h"

namespace orc {

void quat_to_mat(const double q[4], double R[9]) {  // q = (w, x, y, z), already normalised
  double w = q[0], x = q[1], y = q[2], z = q[3];
  R[0] = 1 - 2 * (y * y + z * z); R[1] = 2 * (x * y - w * z);     R[2] = 2 * (x * z + w * y);
  R[3] = 2 * (x * y + w * z);     R[4] = 1 - 2 * (x * x + z * z); R[5] = 2 * (y * z - w * x);
  R[6] = 2 * (x * z - w * y);     R[7] = 2 * (y * z + w * x);     R[8] = 1 - 2 * (x * x + y * y);
}

// Real SH basis up to degree 4 in the sign convention the reference uses (splat_math.cuh:120-146).
void sh_basis(int deg, const double v[3], double* b) {
  const double x = v[0], y = v[1], z = v[2];
  b[0] = 0.28209479177387814;
  if (deg < 1) return;
  b[1] = -0.4886025 * y; b[2] = 0.4886025 * z; b[3] = -0.4886025 * x;
  if (deg < 2) return;
  const double z2 = z * z, fc1 = x * x - y * y, fs1 = 2 * x * y;
  b[4] = 0.54627424 * fs1; b[5] = -1.0925485 * z * y; b[6] = 0.9461747 * z2 - 0.31539157;
  b[7] = -1.0925485 * z * x; b[8] = 0.54627424 * fc1;
  if (deg < 3) return;
  const double fc2 = x * fc1 - y * fs1, fs2 = x * fs1 + y * fc1;
  const double f0c = -2.285229 * z2 + 0.4570458, f1b = 1.4453057 * z;
  b[9] = -0.5900436 * fs2; b[10] = f1b * fs1; b[11] = f0c * y; b[12] = z * (1.8658817 * z2 - 1.119529);
  b[13] = f0c * x; b[14] = f1b * fc1; b[15] = -0.5900436 * fc2;
  if (deg < 4) return;
  const double fc3 = x * fc2 - y * fs2, fs3 = x * fs2 + y * fc2;
  const double f0d = z * (-4.683326 * z2 + 2.0071396), f1c = 3.3116114 * z2 - 0.47308735, f2b = -1.7701308 * z;
  b[16] = 0.62583575 * fs3; b[17] = f2b * fs2; b[18] = f1c * fs1; b[19] = f0d * y;
  b[20] = 1.9843135 * z * b[12] - 1.0062306 * b[6];
  b[21] = f0d * x; b[22] = f1c * fc1; b[23] = f2b * fc2; b[24] = 0.62583575 * fc3;
}

// Gradient of every basis value with respect to the (unit) direction: db[k][3].
void sh_basis_grad(int deg, const double v[3], double (*db)[3]) {
  const double x = v[0], y = v[1], z = v[2];
  for (int k = 0; k < (deg + 1) * (deg + 1); k++) db[k][0] = db[k][1] = db[k][2] = 0;
  if (deg < 1) return;
  db[1][1] = -0.4886025; db[2][2] = 0.4886025; db[3][0] = -0.4886025;
  if (deg < 2) return;
  const double z2 = z * z, fc1 = x * x - y * y, fs1 = 2 * x * y;
  const double dfc1[3] = {2 * x, -2 * y, 0}, dfs1[3] = {2 * y, 2 * x, 0};
  for (int a = 0; a < 3; a++) { db[4][a] = 0.54627424 * dfs1[a]; db[8][a] = 0.54627424 * dfc1[a]; }
  db[5][1] = -1.0925485 * z; db[5][2] = -1.0925485 * y;
  db[6][2] = 2 * 0.9461747 * z;
  db[7][0] = -1.0925485 * z; db[7][2] = -1.0925485 * x;
  if (deg < 3) return;
  const double fc2 = x * fc1 - y * fs1, fs2 = x * fs1 + y * fc1;
  double dfc2[3], dfs2[3];
  for (int a = 0; a < 3; a++) {
    dfc2[a] = (a == 0 ? fc1 : 0) + x * dfc1[a] - (a == 1 ? fs1 : 0) - y * dfs1[a];
    dfs2[a] = (a == 0 ? fs1 : 0) + x * dfs1[a] + (a == 1 ? fc1 : 0) + y * dfc1[a];
  }
  const double f0c = -2.285229 * z2 + 0.4570458, f1b = 1.4453057 * z;
  const double df0c_z = -2 * 2.285229 * z, df1b_z = 1.4453057;
  for (int a = 0; a < 3; a++) {
    db[9][a] = -0.5900436 * dfs2[a]; db[15][a] = -0.5900436 * dfc2[a];
    db[10][a] = f1b * dfs1[a] + (a == 2 ? df1b_z * fs1 : 0);
    db[14][a] = f1b * dfc1[a] + (a == 2 ? df1b_z * fc1 : 0);
  }
  db[11][1] = f0c; db[11][2] = df0c_z * y;
  db[13][0] = f0c; db[13][2] = df0c_z * x;
  const double p12 = z * (1.8658817 * z2 - 1.119529), dp12 = 3 * 1.8658817 * z2 - 1.119529;
  db[12][2] = dp12;
  if (deg < 4) return;
  const double fc3 = x * fc2 - y * fs2, fs3 = x * fs2 + y * fc2;
  (void)fc3; (void)fs3;
  double dfc3[3], dfs3[3];
  for (int a = 0; a < 3; a++) {
    dfc3[a] = (a == 0 ? fc2 : 0) + x * dfc2[a] - (a == 1 ? fs2 : 0) - y * dfs2[a];
    dfs3[a] = (a == 0 ? fs2 : 0) + x * dfs2[a] + (a == 1 ? fc2 : 0) + y * dfc2[a];
  }
  const double f0d = z * (-4.683326 * z2 + 2.0071396), df0d = -3 * 4.683326 * z2 + 2.0071396;
  const double f1c = 3.3116114 * z2 - 0.47308735, df1c = 2 * 3.3116114 * z;
  const double f2b = -1.7701308 * z, df2b = -1.7701308;
  for (int a = 0; a < 3; a++) {
    db[16][a] = 0.62583575 * dfs3[a]; db[24][a] = 0.62583575 * dfc3[a];
    db[17][a] = f2b * dfs2[a] + (a == 2 ? df2b * fs2 : 0);
    db[23][a] = f2b * dfc2[a] + (a == 2 ? df2b * fc2 : 0);
    db[18][a] = f1c * dfs1[a] + (a == 2 ? df1c * fs1 : 0);
    db[22][a] = f1c * dfc1[a] + (a == 2 ? df1c * fc1 : 0);
  }
  db[19][1] = f0d; db[19][2] = df0d * y;
  db[21][0] = f0d; db[21][2] = df0d * x;
  db[20][2] = 1.9843135 * (p12 + z * dp12) - 1.0062306 * (2 * 0.9461747 * z);
}

bool project_one(const float* po, const float* q, const float* ls, const OrcCamera& cam, Proj& r) {
  r.ok = false;
  double R[9]; for (int i = 0; i < 9; i++) R[i] = cam.R[i];
  const double mean[3] = {po[0], po[1], po[2]};
  for (int i = 0; i < 3; i++) r.mean_c[i] = R[i * 3] * mean[0] + R[i * 3 + 1] * mean[1] + R[i * 3 + 2] * mean[2] + cam.t[i];
  const double* mc = r.mean_c;
  if (!(std::isfinite(mc[0]) && std::isfinite(mc[1]) && std::isfinite(mc[2]) && mc[2] <= 1e10)) return false;
  if (!(mc[2] >= 0.01)) return false;
  const double f = ls[3], f2 = f * f;
  double s2f[3];
  for (int k = 0; k < 3; k++) { r.s2_raw[k] = std::exp(2.0 * ls[k]); s2f[k] = r.s2_raw[k] + f2; r.s[k] = std::sqrt(s2f[k]); }
  r.comp_floor = f > 0 ? std::sqrt((r.s2_raw[0] * r.s2_raw[1] * r.s2_raw[2]) / (s2f[0] * s2f[1] * s2f[2])) : 1.0;
  if (!(std::isfinite(r.s[0]) && std::isfinite(r.s[1]) && std::isfinite(r.s[2]))) return false;
  const double qn2 = (double)q[0] * q[0] + (double)q[1] * q[1] + (double)q[2] * q[2] + (double)q[3] * q[3];
  if (!(qn2 >= 1e-6 && std::isfinite(qn2))) return false;
  if (!std::isfinite(po[3])) return false;
  const double inv_qn = 1.0 / std::sqrt(qn2);
  const double qn[4] = {q[0] * inv_qn, q[1] * inv_qn, q[2] * inv_qn, q[3] * inv_qn};
  quat_to_mat(qn, r.Rq);
  double M[9];
  for (int i = 0; i < 3; i++) for (int j = 0; j < 3; j++)
    M[i * 3 + j] = (R[i * 3] * r.Rq[j] + R[i * 3 + 1] * r.Rq[3 + j] + R[i * 3 + 2] * r.Rq[6 + j]) * r.s[j];
  const double inv_z = 1.0 / mc[2], rx = mc[0] * inv_z, ry = mc[1] * inv_z;
  const double cxr = std::min(std::max(rx, (double)cam.lim_neg_x), (double)cam.lim_pos_x);
  const double cyr = std::min(std::max(ry, (double)cam.lim_neg_y), (double)cam.lim_pos_y);
  r.clamp_x = !(rx <= cam.lim_pos_x && rx >= cam.lim_neg_x);
  r.clamp_y = !(ry <= cam.lim_pos_y && ry >= cam.lim_neg_y);
  const double dx = cam.fx * inv_z, dy = cam.fy * inv_z;
  r.J[0] = dx; r.J[1] = 0; r.J[2] = -dx * cxr; r.J[3] = 0; r.J[4] = dy; r.J[5] = -dy * cyr;
  double V[6];
  for (int i = 0; i < 2; i++) for (int j = 0; j < 3; j++) V[i * 3 + j] = r.J[i * 3] * M[j] + r.J[i * 3 + 1] * M[3 + j] + r.J[i * 3 + 2] * M[6 + j];
  double c00 = V[0] * V[0] + V[1] * V[1] + V[2] * V[2], c01 = V[0] * V[3] + V[1] * V[4] + V[2] * V[5], c11 = V[3] * V[3] + V[4] * V[4] + V[5] * V[5];
  const double max_abs = std::max(std::fabs(c00), std::max(std::fabs(c01), std::fabs(c11)));
  if (max_abs > 1e18) { const double k = 1e18 / max_abs; c00 *= k; c01 *= k; c11 *= k; }
  const double blur = 0.3;
  r.cov[0] = c00 + blur; r.cov[1] = c01; r.cov[2] = c11 + blur;
  r.sig = 1.0 / (1.0 + std::exp(-(double)po[3]));
  r.opac = r.sig * r.comp_floor;
  if (!(std::isfinite(r.cov[0]) && std::isfinite(r.cov[1]) && std::isfinite(r.cov[2]))) return false;
  const double det = r.cov[0] * r.cov[2] - r.cov[1] * r.cov[1];
  if (!(det > 0)) return false;
  r.conic[0] = r.cov[2] / det; r.conic[1] = -r.cov[1] / det; r.conic[2] = r.cov[0] / det;
  r.mean2d[0] = cam.fx * rx + cam.cx; r.mean2d[1] = cam.fy * ry + cam.cy;
  if (!(r.opac >= 1.0 / 255.0)) return false;
  r.power = std::log(r.opac * 255.0);
  const double detc = r.conic[0] * r.conic[2] - r.conic[1] * r.conic[1];
  if (!(detc > 0)) return false;
  r.ex = std::sqrt(2 * r.power * r.conic[2] / detc);
  r.ey = std::sqrt(2 * r.power * r.conic[0] / detc);
  r.ok = true;
  return true;
}

}  // namespace orc

using namespace orc;

extern "C" void orc_project(int n, int degree, int active_degree, const float* pos_op, const float* quat, const float* lscale,
                            const float* sh, const OrcCamera* cam, double* rec) {
  const int K = (degree + 1) * (degree + 1);
  const int act = std::min(active_degree, degree);
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; i++) {
    double* o = rec + (size_t)i * ORC_REC;
    for (int k = 0; k < ORC_REC; k++) o[k] = 0;
    Proj p;
    if (!project_one(pos_op + i * 4, quat + i * 4, lscale + i * 4, *cam, p)) continue;
    o[ORC_MX] = p.mean2d[0]; o[ORC_MY] = p.mean2d[1]; o[ORC_C00] = p.conic[0]; o[ORC_C01] = p.conic[1]; o[ORC_C11] = p.conic[2];
    o[ORC_OPAC] = p.opac; o[ORC_Z] = p.mean_c[2]; o[ORC_POWER] = p.power; o[ORC_EX] = p.ex; o[ORC_EY] = p.ey; o[ORC_OK] = 1;
    o[ORC_MAXSCREEN] = std::max(p.ex / cam->W, p.ey / cam->H);
    double v[3] = {pos_op[i * 4] - (double)cam->pos[0], pos_op[i * 4 + 1] - (double)cam->pos[1], pos_op[i * 4 + 2] - (double)cam->pos[2]};
    const double vl = std::max(std::sqrt(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]), 1e-12);
    for (int a = 0; a < 3; a++) v[a] /= vl;
    double b[25]; for (int k = 0; k < 25; k++) b[k] = 0;
    sh_basis(act, v, b);
    const int Kact = (act + 1) * (act + 1);
    for (int ch = 0; ch < 3; ch++) {
      double c = 0;
      for (int k = 0; k < Kact; k++) c += b[k] * sh[((size_t)i * K + k) * 3 + ch];
      c += 0.5;
      o[ORC_R + ch] = std::isfinite(c) ? std::min(std::max(c, -100.0), 100.0) : 0.0;
    }
  }
}

extern "C" void orc_min_scale(int n, const float* pos_op, float* lscale, const float* cam_pos, const float* cam_focal, int n_cams) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; i++) {
    double best = INFINITY;
    for (int c = 0; c < n_cams; c++) {
      const double dx = pos_op[i * 4] - (double)cam_pos[c * 3], dy = pos_op[i * 4 + 1] - (double)cam_pos[c * 3 + 1], dz = pos_op[i * 4 + 2] - (double)cam_pos[c * 3 + 2];
      best = std::min(best, std::sqrt(dx * dx + dy * dy + dz * dz) / std::max((double)cam_focal[c], 1e-6));
    }
    lscale[i * 4 + 3] = (float)(std::sqrt(0.1) * best);
  }
}

extern "C" void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

extern "C" int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Per-splat feature lanes (src/gpu/project.cu:62-77). mode 1: pseudo-normal = the local axis of the shortest log
// scale, turned to face the camera, rotated into camera space; mode 2: feat_buffer clamped to +-100, non-finite -> 0.
// feat: [n][3] doubles. Pinned through the reference's normal lane (tests/reference.cpp:67-75,132-140).
extern "C" void orc_features(int n, int mode, const float* pos_op, const float* quat, const float* lscale, const float* feat_buffer,
                             const OrcCamera* cam, double* feat) {
#pragma omp parallel for
  for (int i = 0; i < n; i++) {
    double* f = feat + (size_t)i * 3;
    if (mode == 1) {
      const float* ls = lscale + (size_t)i * 4;
      const int axis = (ls[0] <= ls[1] && ls[0] <= ls[2]) ? 0 : (ls[1] <= ls[2] ? 1 : 2);
      double q[4] = {quat[(size_t)i * 4], quat[(size_t)i * 4 + 1], quat[(size_t)i * 4 + 2], quat[(size_t)i * 4 + 3]};
      const double qn = std::sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
      for (double& c : q) c /= qn;
      double Rq[9];
      orc::quat_to_mat(q, Rq);
      const double a[3] = {Rq[axis], Rq[3 + axis], Rq[6 + axis]};
      const double al = std::max(std::sqrt(a[0] * a[0] + a[1] * a[1] + a[2] * a[2]), 1e-12);
      const double u[3] = {a[0] / al, a[1] / al, a[2] / al};
      const float* p = pos_op + (size_t)i * 4;
      const double face = ((cam->pos[0] - p[0]) * u[0] + (cam->pos[1] - p[1]) * u[1] + (cam->pos[2] - p[2]) * u[2]) >= 0 ? 1.0 : -1.0;
      for (int r = 0; r < 3; r++) f[r] = face * (cam->R[r * 3] * u[0] + cam->R[r * 3 + 1] * u[1] + cam->R[r * 3 + 2] * u[2]);
    } else {
      for (int k = 0; k < 3; k++) {
        const double v = mode == 2 ? (double)feat_buffer[(size_t)i * 3 + k] : 0.0;
        f[k] = std::isfinite(v) ? std::min(std::max(v, -100.0), 100.0) : 0.0;
      }
    }
  }
}
