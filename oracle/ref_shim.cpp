// C entry point around the reference's own double-precision CPU check, `reference_loss`
// (tests/reference.cpp:34-143 of the reference tree), so the test suite can call it through ctypes.
// TEST INFRASTRUCTURE ONLY. This file holds no reference code: it includes the reference's header and is linked
// against the reference's unmodified source, compiled where it lies, by the Makefile beside this file.
#include "reference.h"
#include <cstdint>
#include <vector>

extern "C" double ref_reference_loss(int n, int degree, const float* pos, const float* log_scale, const float* quat,
                                     const float* opacity, const float* sh, int W, int H, const float* intr /*fx fy cx cy*/,
                                     const float* R, const float* t, const float* cam_pos, const double* bg, int composite,
                                     int mask, int alpha_lane, double l1_w, double ssim_w, double match_alpha_weight,
                                     double scale, const uint32_t* gt, const uint8_t* wts) {
  b2c::SplatCloud c;
  const int K = (degree + 1) * (degree + 1);
  c.n = (size_t)n; c.sh_degree = degree;
  c.pos.assign(pos, pos + (size_t)n * 3); c.log_scale.assign(log_scale, log_scale + (size_t)n * 3);
  c.quat.assign(quat, quat + (size_t)n * 4); c.opacity.assign(opacity, opacity + n);
  c.sh.assign(sh, sh + (size_t)n * K * 3);
  RefParams p{};
  p.W = W; p.H = H;
  p.cam.width = W; p.cam.height = H; p.cam.fx = intr[0]; p.cam.fy = intr[1]; p.cam.cx = intr[2]; p.cam.cy = intr[3];
  for (int i = 0; i < 9; i++) p.cam.R[i] = R[i];
  for (int i = 0; i < 3; i++) { p.cam.t[i] = t[i]; p.cam.pos[i] = cam_pos[i]; p.bg[i] = bg[i]; }
  p.composite = composite; p.mask = mask; p.alpha_lane = alpha_lane; p.normals = false;
  p.l1_w = l1_w; p.ssim_w = ssim_w; p.match_alpha_weight = match_alpha_weight; p.scale = scale; p.normal_scale = 0;
  std::vector<uint32_t> g(gt, gt + (size_t)W * H), gn;
  std::vector<uint8_t> w;
  p.gt = &g; p.gtn = &gn; p.wts = nullptr;
  if (wts) { w.assign(wts, wts + (size_t)W * H); p.wts = &w; }
  return reference_loss(c, p);
}

// The same call with the reference's normal lane on (tests/reference.cpp:67-75,132-140): gtn is the packed normal
// target (alpha > 127 marks a supervised pixel), normal_scale its weight. With l1_w = ssim_w = 0 and no alpha lane the
// returned loss is a function of the composited feature image alone, which is how the oracle's feature lanes are pinned.
extern "C" double ref_reference_loss_normals(int n, int degree, const float* pos, const float* log_scale, const float* quat,
                                             const float* opacity, const float* sh, int W, int H, const float* intr, const float* R,
                                             const float* t, const float* cam_pos, const double* bg, double l1_w, double ssim_w,
                                             double scale, const uint32_t* gt, const uint32_t* gtn, double normal_scale, const uint8_t* wts) {
  b2c::SplatCloud c;
  const int K = (degree + 1) * (degree + 1);
  c.n = (size_t)n; c.sh_degree = degree;
  c.pos.assign(pos, pos + (size_t)n * 3); c.log_scale.assign(log_scale, log_scale + (size_t)n * 3);
  c.quat.assign(quat, quat + (size_t)n * 4); c.opacity.assign(opacity, opacity + n);
  c.sh.assign(sh, sh + (size_t)n * K * 3);
  RefParams p{};
  p.W = W; p.H = H;
  p.cam.width = W; p.cam.height = H; p.cam.fx = intr[0]; p.cam.fy = intr[1]; p.cam.cx = intr[2]; p.cam.cy = intr[3];
  for (int i = 0; i < 9; i++) p.cam.R[i] = R[i];
  for (int i = 0; i < 3; i++) { p.cam.t[i] = t[i]; p.cam.pos[i] = cam_pos[i]; p.bg[i] = bg[i]; }
  p.composite = false; p.mask = false; p.alpha_lane = false; p.normals = true;
  p.l1_w = l1_w; p.ssim_w = ssim_w; p.match_alpha_weight = 0; p.scale = scale; p.normal_scale = normal_scale;
  std::vector<uint32_t> g(gt, gt + (size_t)W * H), gn(gtn, gtn + (size_t)W * H);
  std::vector<uint8_t> w;
  p.gt = &g; p.gtn = &gn; p.wts = nullptr;
  if (wts) { w.assign(wts, wts + (size_t)W * H); p.wts = &w; }
  return reference_loss(c, p);
}
