// CPU oracle, stage 4: fused L1 + 11-tap SSIM loss with the alpha-match lane, value and per-pixel gradient.
// TEST INFRASTRUCTURE ONLY. Follows photometric_kernel (src/gpu/loss.cu:18-195): Gaussian sigma 1.5, zero padding
// outside the image, variances clamped at 0, SSIM clamped to [-1, 1] with zero gradient where clamped, gradient
// carried by five partial maps blurred back. The loss value is pinned against tests/reference.cpp:106-133; the
// gradient by central differences of that function.
#include "oracle_internal.h"

namespace {

void gauss11(double* w) {
  double sum = 0;
  for (int i = 0; i < 11; i++) { const double x = i - 5.0; w[i] = std::exp(-x * x / (2 * 1.5 * 1.5)); sum += w[i]; }
  for (int i = 0; i < 11; i++) w[i] /= sum;
}

// Separable 11-tap blur with zero padding.
void blur(int W, int H, const double* w, const std::vector<double>& in, std::vector<double>& out) {
  std::vector<double> tmp((size_t)W * H);
#pragma omp parallel for schedule(static)
  for (int y = 0; y < H; y++) for (int x = 0; x < W; x++) {
    double s = 0;
    for (int d = -5; d <= 5; d++) { const int xx = x + d; if (xx >= 0 && xx < W) s += w[d + 5] * in[(size_t)y * W + xx]; }
    tmp[(size_t)y * W + x] = s;
  }
  out.resize((size_t)W * H);
#pragma omp parallel for schedule(static)
  for (int y = 0; y < H; y++) for (int x = 0; x < W; x++) {
    double s = 0;
    for (int d = -5; d <= 5; d++) { const int yy = y + d; if (yy >= 0 && yy < H) s += w[d + 5] * tmp[(size_t)yy * W + x]; }
    out[(size_t)y * W + x] = s;
  }
}

inline double gt_ch(uint32_t p, int c) { return (double)((p >> (8 * c)) & 0xffu) / 255.0; }

}  // namespace

extern "C" double orc_loss(int W, int H, const double* pred, const uint32_t* gt, const uint8_t* weights, const OrcLoss* lp,
                           double* v_out) {
  const size_t P = (size_t)W * H;
  const double C1 = 0.01 * 0.01, C2 = 0.03 * 0.03;
  double w[11]; gauss11(w);
  const double norm = (double)lp->scale / (3.0 * W * H);
  double loss = 0;
  std::vector<double> Mp(P);
  for (size_t i = 0; i < P; i++) {
    const double wp = weights ? weights[i] / 255.0 : 1.0;
    Mp[i] = wp * (lp->mask ? gt_ch(gt[i], 3) : 1.0) * norm;
  }
  if (v_out) std::fill(v_out, v_out + P * 4, 0.0);
  for (int ch = 0; ch < 3; ch++) {
    std::vector<double> X(P), Y(P), X2(P), Y2(P), XY(P);
    for (size_t i = 0; i < P; i++) {
      X[i] = pred[i * 4 + ch];
      Y[i] = gt_ch(gt[i], ch) + (lp->composite ? (1 - gt_ch(gt[i], 3)) * (double)lp->bg[ch] : 0.0);
      X2[i] = X[i] * X[i]; Y2[i] = Y[i] * Y[i]; XY[i] = X[i] * Y[i];
    }
    std::vector<double> mu1, mu2, ex2, ey2, exy;
    blur(W, H, w, X, mu1); blur(W, H, w, Y, mu2); blur(W, H, w, X2, ex2); blur(W, H, w, Y2, ey2); blur(W, H, w, XY, exy);
    std::vector<double> A(P, 0.0), B(P, 0.0), Bm(P, 0.0), C(P, 0.0), Cm(P, 0.0);
    double lsum = 0;
#pragma omp parallel for schedule(static) reduction(+ : lsum)
    for (size_t i = 0; i < P; i++) {
      const double m1 = mu1[i], m2 = mu2[i];
      const double s1_raw = ex2[i] - m1 * m1, s2_raw = ey2[i] - m2 * m2;
      const double s1 = std::max(0.0, s1_raw), s2 = std::max(0.0, s2_raw), s12 = exy[i] - m1 * m2;
      const double A1 = 2 * m1 * m2 + C1, A2 = 2 * s12 + C2, B1 = m1 * m1 + m2 * m2 + C1, B2 = s1 + s2 + C2;
      const double raw = (A1 * A2) / (B1 * B2);
      const double ssim = std::min(std::max(raw, -1.0), 1.0);
      lsum += Mp[i] * ((double)lp->l1_w * std::fabs(X[i] - Y[i]) + (double)lp->ssim_w * ssim);
      if (raw > -1 && raw < 1) {
        const double k = Mp[i] * (double)lp->ssim_w;
        const double d_mu1 = 2 * m2 * A2 / (B1 * B2) - 2 * m1 * ssim / B1;
        const double d_s1 = s1_raw > 0 ? -ssim / B2 : 0.0;
        const double d_s12 = 2 * A1 / (B1 * B2);
        A[i] = k * d_mu1; B[i] = k * d_s1; Bm[i] = B[i] * m1; C[i] = k * d_s12; Cm[i] = C[i] * m2;
      }
    }
    loss += lsum;
    if (v_out) {
      std::vector<double> bA, bB, bBm, bC, bCm;
      blur(W, H, w, A, bA); blur(W, H, w, B, bB); blur(W, H, w, Bm, bBm); blur(W, H, w, C, bC); blur(W, H, w, Cm, bCm);
      for (size_t i = 0; i < P; i++) {
        const double p = X[i], g = Y[i];
        const double sgn = p > g ? 1.0 : (p < g ? -1.0 : 0.0);
        const double grad = Mp[i] * (double)lp->l1_w * sgn + bA[i] + 2 * p * bB[i] - 2 * bBm[i] + g * bC[i] - bCm[i];
        v_out[i * 4 + ch] = grad * (double)lp->grad_scale;
      }
    }
  }
  if (lp->alpha_lane) {
    for (size_t i = 0; i < P; i++) {
      const double wp = weights ? weights[i] / 255.0 : 1.0;
      const double Ma = wp * (double)lp->match_alpha_weight * (double)lp->scale / ((double)W * H);
      const double da = pred[i * 4 + 3] - gt_ch(gt[i], 3);
      loss += Ma * std::fabs(da);
      if (v_out) v_out[i * 4 + 3] = Ma * (da > 0 ? 1.0 : (da < 0 ? -1.0 : 0.0)) * (double)lp->grad_scale;
    }
  }
  return loss;
}
