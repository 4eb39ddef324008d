// CPU oracle, stages 6 and 7: projection backward (screen-space lanes -> parameter gradients) and sparse Adam.
// TEST INFRASTRUCTURE ONLY. Follows optim_kernel (src/gpu/optim.cu:100-297 for the gradient chain, :299-361 for the
// update, adam4 :90-97). The gradient chain is re-derived here in matrix form (T = J Rv Rq diag(s), cov = T T^T) rather
// than step by step; it is pinned by central differences of tests/reference.cpp. The update has no reference test:
// parity unpinned, checked against the CUDA kernel only.
#include "oracle_internal.h"

using namespace orc;

namespace {
inline void mat3_mul(const double* A, const double* B, double* C) {
  for (int i = 0; i < 3; i++) for (int j = 0; j < 3; j++) C[i * 3 + j] = A[i * 3] * B[j] + A[i * 3 + 1] * B[3 + j] + A[i * 3 + 2] * B[6 + j];
}
}  // namespace

extern "C" void orc_proj_bwd(int n, int degree, int active_degree, const float* pos_op, const float* quat, const float* lscale,
                             const float* sh, const OrcCamera* cam_p, const double* v_splat, const uint32_t* vis_flag,
                             const uint32_t* tile_count, double* grad) {
  const OrcCamera& cam = *cam_p;
  const int K = (degree + 1) * (degree + 1), per = 11 + 3 * K;
  const int act = std::min(active_degree, degree), Kact = (act + 1) * (act + 1);
  double Rv[9]; for (int i = 0; i < 9; i++) Rv[i] = cam.R[i];
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; i++) {
    double* o = grad + (size_t)i * per;
    for (int k = 0; k < per; k++) o[k] = 0;
    const double* g = v_splat + (size_t)i * 13;
    const bool visible = vis_flag[i] != 0 && tile_count[i] != 0;
    bool any = false, finite = true;
    for (int k = 0; k < 13; k++) { if (k != 9 && g[k] != 0) any = true; finite = finite && std::isfinite(g[k]); }
    if (!(any && visible && finite)) continue;
    Proj pr;
    if (!project_one(pos_op + i * 4, quat + i * 4, lscale + i * 4, cam, pr)) continue;
    // On-screen cull (splat_math.cuh:288-290) is part of `ok` in the reference; a splat with a gradient has tiles,
    // so it passed.
    const double mean[3] = {pos_op[i * 4], pos_op[i * 4 + 1], pos_op[i * 4 + 2]};
    // --- SH colour and view direction ---
    double u[3] = {mean[0] - cam.pos[0], mean[1] - cam.pos[1], mean[2] - cam.pos[2]};
    const double ul = std::sqrt(u[0] * u[0] + u[1] * u[1] + u[2] * u[2]);
    const double v[3] = {u[0] / ul, u[1] / ul, u[2] / ul};
    double b[25] = {0}; double db[25][3];
    sh_basis(act, v, b); sh_basis_grad(act, v, db);
    const double vc[3] = {g[5], g[6], g[7]};
    double v_v[3] = {0, 0, 0};
    for (int k = 0; k < Kact; k++) {
      const float* c = sh + ((size_t)i * K + k) * 3;
      const double dotc = c[0] * vc[0] + c[1] * vc[1] + c[2] * vc[2];
      for (int a = 0; a < 3; a++) v_v[a] += db[k][a] * dotc;
      for (int ch = 0; ch < 3; ch++) o[11 + k * 3 + ch] = b[k] * vc[ch];
    }
    const double vdot = v[0] * v_v[0] + v[1] * v_v[1] + v[2] * v_v[2];
    double g_pos[3]; for (int a = 0; a < 3; a++) g_pos[a] = (v_v[a] - v[a] * vdot) / ul;
    // --- opacity ---
    const double v_alpha = g[8];
    double g_op = v_alpha * pr.comp_floor * pr.sig * (1 - pr.sig);
    // --- conic -> covariance: dL/dcov = -conic G conic, G the symmetric gradient of the conic ---
    const double G[4] = {g[2], 0.5 * g[3], 0.5 * g[3], g[4]};
    const double X[4] = {pr.conic[0], pr.conic[1], pr.conic[1], pr.conic[2]};
    double XG[4], vcov[4];
    for (int r = 0; r < 2; r++) for (int c = 0; c < 2; c++) XG[r * 2 + c] = X[r * 2] * G[c] + X[r * 2 + 1] * G[2 + c];
    for (int r = 0; r < 2; r++) for (int c = 0; c < 2; c++) vcov[r * 2 + c] = -(XG[r * 2] * X[c] + XG[r * 2 + 1] * X[2 + c]);
    // --- T = J Rv M, M = Rq diag(s) ---
    double M[9], RvM[9], T[6];
    for (int r = 0; r < 3; r++) for (int c = 0; c < 3; c++) M[r * 3 + c] = pr.Rq[r * 3 + c] * pr.s[c];
    mat3_mul(Rv, M, RvM);
    for (int r = 0; r < 2; r++) for (int c = 0; c < 3; c++) T[r * 3 + c] = pr.J[r * 3] * RvM[c] + pr.J[r * 3 + 1] * RvM[3 + c] + pr.J[r * 3 + 2] * RvM[6 + c];
    double vT[6];  // 2 vcov T
    for (int r = 0; r < 2; r++) for (int c = 0; c < 3; c++) vT[r * 3 + c] = 2 * (vcov[r * 2] * T[c] + vcov[r * 2 + 1] * T[3 + c]);
    double vJ[6];  // vT (Rv M)^T
    for (int r = 0; r < 2; r++) for (int c = 0; c < 3; c++) vJ[r * 3 + c] = vT[r * 3] * RvM[c * 3] + vT[r * 3 + 1] * RvM[c * 3 + 1] + vT[r * 3 + 2] * RvM[c * 3 + 2];
    double JR[6];  // J Rv
    for (int r = 0; r < 2; r++) for (int c = 0; c < 3; c++) JR[r * 3 + c] = pr.J[r * 3] * Rv[c] + pr.J[r * 3 + 1] * Rv[3 + c] + pr.J[r * 3 + 2] * Rv[6 + c];
    double vM[9];  // (J Rv)^T vT
    for (int r = 0; r < 3; r++) for (int c = 0; c < 3; c++) vM[r * 3 + c] = JR[r] * vT[c] + JR[3 + r] * vT[3 + c];
    // --- camera-space mean through the pinhole and the clamped Jacobian ---
    const double x = pr.mean_c[0], y = pr.mean_c[1], z = pr.mean_c[2];
    const double iz = 1 / z, iz2 = iz * iz, iz3 = iz2 * iz;
    const double cxr = std::min(std::max(x * iz, (double)cam.lim_neg_x), (double)cam.lim_pos_x);
    const double cyr = std::min(std::max(y * iz, (double)cam.lim_neg_y), (double)cam.lim_pos_y);
    const double v2x = g[0], v2y = g[1];
    double vmc[3];
    vmc[0] = cam.fx * iz * v2x + (pr.clamp_x ? 0.0 : -cam.fx * iz2 * vJ[2]);
    vmc[1] = cam.fy * iz * v2y + (pr.clamp_y ? 0.0 : -cam.fy * iz2 * vJ[5]);
    vmc[2] = -(cam.fx * x * v2x + cam.fy * y * v2y) * iz2 - cam.fx * iz2 * vJ[0] - cam.fy * iz2 * vJ[4]
             + (pr.clamp_x ? cam.fx * cxr * iz2 : 2 * cam.fx * x * iz3) * vJ[2]
             + (pr.clamp_y ? cam.fy * cyr * iz2 : 2 * cam.fy * y * iz3) * vJ[5];
    for (int a = 0; a < 3; a++) g_pos[a] += Rv[a] * vmc[0] + Rv[3 + a] * vmc[1] + Rv[6 + a] * vmc[2];
    // --- scales (through the floor) ---
    const double f2 = (double)lscale[i * 4 + 3] * lscale[i * 4 + 3];
    double g_ls[3];
    for (int c = 0; c < 3; c++) {
      const double vs = pr.Rq[c] * vM[c] + pr.Rq[3 + c] * vM[3 + c] + pr.Rq[6 + c] * vM[6 + c];
      g_ls[c] = vs * pr.s2_raw[c] / pr.s[c] + v_alpha * pr.opac * f2 / (pr.s2_raw[c] + f2);
    }
    // --- rotation: dL/dRq = vM diag(s); then through R(q / |q|) ---
    double vR[9];
    for (int r = 0; r < 3; r++) for (int c = 0; c < 3; c++) vR[r * 3 + c] = vM[r * 3 + c] * pr.s[c];
    const double q0[4] = {quat[i * 4], quat[i * 4 + 1], quat[i * 4 + 2], quat[i * 4 + 3]};
    const double ql = std::sqrt(q0[0] * q0[0] + q0[1] * q0[1] + q0[2] * q0[2] + q0[3] * q0[3]);
    const double qw = q0[0] / ql, qx = q0[1] / ql, qy = q0[2] / ql, qz = q0[3] / ql;
    const double* V = vR;
    double gq[4];
    gq[0] = 2 * (-qz * V[1] + qy * V[2] + qz * V[3] - qx * V[5] - qy * V[6] + qx * V[7]);
    gq[1] = 2 * (qy * V[1] + qz * V[2] + qy * V[3] - 2 * qx * V[4] - qw * V[5] + qz * V[6] + qw * V[7] - 2 * qx * V[8]);
    gq[2] = 2 * (-2 * qy * V[0] + qx * V[1] + qw * V[2] + qx * V[3] + qz * V[5] - qw * V[6] + qz * V[7] - 2 * qy * V[8]);
    gq[3] = 2 * (-2 * qz * V[0] - qw * V[1] + qx * V[2] + qw * V[3] - 2 * qz * V[4] + qy * V[5] + qx * V[6] + qy * V[7]);
    const double qn[4] = {qw, qx, qy, qz};
    const double gd = gq[0] * qw + gq[1] * qx + gq[2] * qy + gq[3] * qz;
    double g_q[4]; for (int a = 0; a < 4; a++) g_q[a] = (gq[a] - qn[a] * gd) / ql;
    bool ok = std::isfinite(g_op);
    for (int a = 0; a < 3; a++) ok = ok && std::isfinite(g_pos[a]) && std::isfinite(g_ls[a]);
    for (int a = 0; a < 4; a++) ok = ok && std::isfinite(g_q[a]);
    if (!ok) { g_op = 0; for (int a = 0; a < 3; a++) g_pos[a] = g_ls[a] = 0; for (int a = 0; a < 4; a++) g_q[a] = 0; }
    o[0] = g_pos[0]; o[1] = g_pos[1]; o[2] = g_pos[2]; o[3] = g_op;
    for (int a = 0; a < 4; a++) o[4 + a] = g_q[a];
    for (int a = 0; a < 3; a++) o[8 + a] = g_ls[a];
  }
}

extern "C" void orc_adam(int n, int degree, float* pos_op, float* quat, float* lscale, float* sh, float* m_pos, float* v_pos,
                         float* m_q, float* v_q, float* m_ls, float* v_ls, float* m_sh, float* v_sh, uint32_t* last_step,
                         const double* grad, const uint8_t* active, const OrcAdam* op) {
  const int K = (degree + 1) * (degree + 1), per = 11 + 3 * K;
  const double b1 = op->beta1, b2 = op->beta2, eps = op->eps;
  const double bc1 = 1 / (1 - std::pow(b1, (double)op->t)), bc2 = 1 / (1 - std::pow(b2, (double)op->t));
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; i++) {
    if (op->sparse && !active[i]) continue;
    const double* g = grad + (size_t)i * per;
    double skipped = 0;
    if (op->sparse) { const uint32_t ls = last_step[i]; skipped = ls == 0 ? 0.0 : std::max((double)op->t - (double)ls - 1.0, 0.0); last_step[i] = (uint32_t)op->t; }
    double d1 = 1, d2 = 1, drift = 0;
    if (skipped > 0) { d1 = std::pow(b1, skipped); d2 = std::pow(b2, skipped); const double r = b1 / std::sqrt(b2); drift = r * (1 - std::pow(r, skipped)) / (1 - r); }
    auto upd = [&](float& p, float& m, float& v, double gr, double lr) {
      double pp = p, mm = m, vv = v;
      if (skipped > 0) { pp -= lr * drift * (mm * bc1) / (std::sqrt(vv * bc2) + eps); mm *= d1; vv *= d2; }
      mm = b1 * mm + (1 - b1) * gr; vv = b2 * vv + (1 - b2) * gr * gr;
      pp -= lr * (mm * bc1) / (std::sqrt(vv * bc2) + eps);
      p = (float)pp; m = (float)mm; v = (float)vv;
    };
    for (int a = 0; a < 3; a++) upd(pos_op[i * 4 + a], m_pos[i * 4 + a], v_pos[i * 4 + a], g[a], op->lr_mean);
    upd(pos_op[i * 4 + 3], m_pos[i * 4 + 3], v_pos[i * 4 + 3], g[3], op->lr_opac);
    for (int a = 0; a < 4; a++) upd(quat[i * 4 + a], m_q[i * 4 + a], v_q[i * 4 + a], g[4 + a], op->lr_rot);
    for (int a = 0; a < 3; a++) upd(lscale[i * 4 + a], m_ls[i * 4 + a], v_ls[i * 4 + a], g[8 + a], op->lr_scale);
    m_ls[i * 4 + 3] = 0; v_ls[i * 4 + 3] = 0;  // the floor lane is frozen (optim.cu:331-335)
    // Adam-mini: one second moment per splat, the EMA of the mean squared SH gradient (optim.cu:337-345).
    double gsq = 0;
    for (int k = 0; k < 3 * K; k++) gsq += g[11 + k] * g[11 + k];
    gsq /= (double)(3 * K);
    const double v_old = (double)v_sh[i] * d2;
    const double denom_old = skipped > 0 ? drift * bc1 / (std::sqrt(v_old * bc2) + eps) : 0.0;
    const double vn = b2 * v_old + (1 - b2) * gsq;
    v_sh[i] = (float)vn;
    const double denom = bc1 / (std::sqrt((double)(float)vn * bc2) + eps);
    for (int k = 0; k < K; k++) {
      const double lrk = k == 0 ? op->lr_dc : op->lr_sh_rest;
      for (int ch = 0; ch < 3; ch++) {
        const size_t at = ((size_t)i * K + k) * 3 + ch;
        double m_old = m_sh[at], p = sh[at];
        if (skipped > 0) { p -= lrk * denom_old * m_old; m_old *= d1; }
        const double m = b1 * m_old + (1 - b1) * g[11 + k * 3 + ch];
        m_sh[at] = (float)m;
        sh[at] = (float)(p - lrk * denom * m);
      }
    }
  }
}

extern "C" double orc_step(int n, int degree, int active_degree, const float* pos_op, const float* quat, const float* lscale,
                           const float* sh, const OrcCamera* cam, const double* bg, const uint32_t* gt, const uint8_t* weights,
                           const OrcLoss* lp, int backward, double* out_rgba_opt, double* grad, int64_t* counters) {
  const int W = cam->W, H = cam->H;
  const size_t P = (size_t)W * H;
  const int n_tiles = tiles_x(W) * tiles_y(H);
  std::vector<double> rec((size_t)n * ORC_REC), geo((size_t)n * 8), col((size_t)n * 3);
  orc_project(n, degree, active_degree, pos_op, quat, lscale, sh, cam, rec.data());
  std::vector<float> p0((size_t)n * 4), p1((size_t)n * 4);
  for (int i = 0; i < n; i++) {
    const double* r = rec.data() + (size_t)i * ORC_REC;
    const bool ok = r[ORC_OK] != 0;
    p0[i * 4] = (float)r[ORC_MX]; p0[i * 4 + 1] = (float)r[ORC_MY]; p0[i * 4 + 2] = (float)r[ORC_C00]; p0[i * 4 + 3] = (float)r[ORC_C01];
    p1[i * 4] = (float)r[ORC_C11]; p1[i * 4 + 1] = (float)r[ORC_OPAC]; p1[i * 4 + 2] = (float)r[ORC_Z]; p1[i * 4 + 3] = ok ? (float)r[ORC_POWER] : -1.f;
    for (int k = 0; k < 8; k++) geo[(size_t)i * 8 + k] = r[k];
    for (int k = 0; k < 3; k++) col[(size_t)i * 3 + k] = r[ORC_R + k];
  }
  std::vector<uint32_t> tile_count(n), ranges((size_t)n_tiles * 2);
  const int64_t total = orc_bin(n, p0.data(), p1.data(), W, H, tile_count.data(), nullptr, nullptr, 0, ranges.data());
  std::vector<uint32_t> vals((size_t)std::max<int64_t>(total, 1));
  orc_bin(n, p0.data(), p1.data(), W, H, tile_count.data(), vals.data(), nullptr, total, ranges.data());
  std::vector<double> rgba_own; double* rgba = out_rgba_opt;
  if (!rgba) { rgba_own.resize(P * 4); rgba = rgba_own.data(); }
  std::vector<double> outT(P); std::vector<uint32_t> last(P);
  orc_raster_fwd(W, H, geo.data(), col.data(), vals.data(), ranges.data(), bg, 1, rgba, outT.data(), last.data(), nullptr);
  double loss = 0;
  std::vector<double> v_out;
  if (gt) { if (backward) v_out.resize(P * 4); loss = orc_loss(W, H, rgba, gt, weights, lp, backward ? v_out.data() : nullptr); }
  if (counters) {
    int64_t V = 0, Ib = 0;
    for (int i = 0; i < n; i++) V += tile_count[i] != 0;
    for (int t = 0; t < n_tiles; t++) Ib += (int64_t)ranges[t * 2 + 1] - ranges[t * 2];
    counters[0] = V; counters[1] = total; counters[2] = Ib;
  }
  if (backward && gt && grad) {
    std::vector<double> v_splat((size_t)n * 13), visw(n); std::vector<uint32_t> vis(n);
    orc_raster_bwd(n, W, H, geo.data(), col.data(), vals.data(), ranges.data(), bg, rgba, outT.data(), last.data(), v_out.data(), v_splat.data(), vis.data(), visw.data());
    orc_proj_bwd(n, degree, active_degree, pos_op, quat, lscale, sh, cam, v_splat.data(), vis.data(), tile_count.data(), grad);
  }
  return loss;
}
