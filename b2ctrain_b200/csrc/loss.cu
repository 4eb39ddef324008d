// Fused photometric loss: L1 + 11-tap Gaussian SSIM (sigma 1.5, zero padding) + alpha-match lane, value and
// per-pixel gradient in one kernel. Reference semantics: photometric_kernel (src/gpu/loss.cu:18-195),
// accumulate_kernel (loss.cu:317), eval_kernel (loss.cu:241-293).
//
// The work is a stencil: a separable blur of five moments, SSIM and its partial derivatives, the same blur applied
// backwards. It is bound by FP32 issue and shared-memory reads, not by HBM (36 bytes per pixel), so what counts is how
// many blur taps are spent per output. The loss kernel streams down column strips and pays for a halo in one direction
// only; every blur is register-tiled (a thread makes four consecutive outputs from a fourteen-wide sliding window).
#include "common.cuh"

namespace b2k {
namespace {

constexpr int HALO = 5;
constexpr int TILE_PX = LOSS_TILE * LOSS_TILE;
constexpr float C1 = 0.01f * 0.01f, C2 = 0.03f * 0.03f;

struct Gauss { float w[11]; };

Gauss make_gauss() {
  Gauss g; float sum = 0.f;
  for (int i = 0; i < 11; i++) { const float x = (float)i - 5.f; g.w[i] = expf(-x * x / (2.f * 1.5f * 1.5f)); sum += g.w[i]; }
  for (int i = 0; i < 11; i++) g.w[i] /= sum;
  return g;
}

__device__ __forceinline__ float unpack(uint32_t p, int c) { return (float)((p >> (8 * c)) & 0xffu) * (1.f / 255.f); }

struct LossArgs {
  float l1_w, ssim_w, bg[3]; int composite, mask, alpha_lane; float match_alpha_weight, scale, grad_scale;
};

// Eleven-tap sliding window: four consecutive outputs from fourteen consecutive inputs.
__device__ __forceinline__ void window4(const float (&in)[16], const Gauss& g, float (&out)[4]) {
#pragma unroll
  for (int o = 0; o < 4; o++) {
    float a = 0.f;
#pragma unroll
    for (int d = 0; d < 11; d++) a += g.w[d] * in[o + d];
    out[o] = a;
  }
}
__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
#pragma unroll
  for (int q = 0; q < 4; q++) { const float4 t = reinterpret_cast<const float4*>(p)[q]; v[q * 4] = t.x; v[q * 4 + 1] = t.y; v[q * 4 + 2] = t.z; v[q * 4 + 3] = t.w; }
}

// ---- The loss kernel --------------------------------------------------------------------------------------------------
// One CTA owns a strip of STRIP_W output columns, a segment of rows and one colour channel, and walks the segment four
// rows at a time. Both blurs are separable, so only the horizontal direction pays for a halo: the row-blurred moments
// and the derivative maps of the last RING rows live in shared-memory rings, and the four stages of the chain run
// side by side as a pipeline, each on its own warps and on its own rows, with one barrier per four rows:
//   A (2 warps)  rows a..a+3      : effective target and prediction -> five moments blurred along the row
//   B (4 warps)  rows a-9..a-6    : blurred down the column -> SSIM -> derivative maps (three: the two that the chain
//                                   rule multiplies by p and by the target, and the sum of the three it does not)
//   C (2 warps)  rows a-18..a-15  : derivative maps blurred down the column
//   D (2 warps)  rows a-22..a-19  : blurred along the row, chain rule, L1 term, one component of v_out per pixel
// Every thread also fetches one element of the next four input rows while it works. Against one CTA per 16x16 tile (a 36x36 footprint
// blurred for 256 outputs, the reference's shape) this spends about a quarter of the warp instructions per pixel:
// measured 0.41 -> 0.20 ms for a 1920x1080 view.
constexpr int STRIP_W = 54;                   // output columns of a strip
constexpr int STRIP_ST = STRIP_W + 2 * HALO;  // 64 statistics columns
constexpr int STRIP_IN = 76;                  // input columns staged: STRIP_W + 4 * HALO = 74, padded to whole 16-byte words
constexpr int STRIP_ROWS = 4;                 // rows per pipeline step
constexpr int RING = 18;                      // rows of a ring: the 14 a column window of four outputs reads + the 4 being written
constexpr int BV_S = STRIP_ST + 4;            // row stride of stage C's output: the last row window overruns into zero padding
constexpr int STRIP_THREADS = 320;
constexpr int STRIP_CTAS_PER_SM = 4;         // 48 registers per thread; measured faster than 2 or 3 CTAs with more registers
static_assert(STRIP_ST == 64 && STRIP_IN >= STRIP_W + 4 * HALO && STRIP_IN % 4 == 0, "strip geometry");

__device__ __forceinline__ int ring_slot(int row) { return (row + RING * 256) % RING; }

__global__ void __launch_bounds__(STRIP_THREADS, STRIP_CTAS_PER_SM) photometric_strip_kernel(const float4* __restrict__ pred, const uint32_t* __restrict__ gt,
                                                                          const uint8_t* __restrict__ weights, int W, int H, int seg_rows, LossArgs lp,
                                                                          Gauss gauss, float4* __restrict__ v_out, float* __restrict__ loss_accum) {
  __shared__ __align__(16) float s_in[2][2][STRIP_ROWS][STRIP_IN];   // [buffer][prediction, target][row][column]
  __shared__ __align__(16) float s_hb[5][RING][STRIP_ST];            // row-blurred moments
  __shared__ __align__(16) float s_dv[3][RING][STRIP_ST];            // derivative maps
  __shared__ __align__(16) float s_bv[2][3][STRIP_ROWS][BV_S];       // [buffer] derivative maps blurred down the column
  __shared__ float s_red[STRIP_THREADS / 32];
  const int tid = threadIdx.x, warp = tid >> 5, c = blockIdx.z;
  const int x0 = blockIdx.x * STRIP_W, y0 = blockIdx.y * seg_rows, y1 = min(y0 + seg_rows, H);
  const int x_end = min(x0 + STRIP_W, W);
  const float norm = lp.scale / (3.f * (float)W * (float)H);
  const float bg_c = lp.composite ? lp.bg[c] : 0.f;
  const float alpha_norm = lp.match_alpha_weight * lp.scale / ((float)W * (float)H);
  const float* pred_c = reinterpret_cast<const float*>(pred) + c;
  float* out_c = reinterpret_cast<float*>(v_out) + c;

  for (int i = tid; i < 5 * RING * STRIP_ST; i += STRIP_THREADS) (&s_hb[0][0][0])[i] = 0.f;
  for (int i = tid; i < 3 * RING * STRIP_ST; i += STRIP_THREADS) (&s_dv[0][0][0])[i] = 0.f;
  for (int i = tid; i < 2 * 3 * STRIP_ROWS * BV_S; i += STRIP_THREADS) (&s_bv[0][0][0][0])[i] = 0.f;
  // One input element (prediction and effective target, zero outside the image and in the row pad).
  auto fetch = [&](int row0, int e, float& px, float& ty) {
    const int row = e / STRIP_IN, col = e - row * STRIP_IN;
    const int y = row0 + row, x = x0 - 2 * HALO + col;
    px = 0.f; ty = 0.f;
    if (col < STRIP_W + 4 * HALO && y >= 0 && y < H && x >= 0 && x < W) {
      const size_t q = (size_t)y * W + x;
      const uint32_t gp = gt[q];
      px = pred_c[q * 4];
      ty = unpack(gp, c) + (1.f - unpack(gp, 3)) * bg_c;
    }
  };
  for (int e = tid; e < STRIP_ROWS * STRIP_IN; e += STRIP_THREADS) {
    float px, ty;
    fetch(y0 - 2 * HALO, e, px, ty);
    (&s_in[0][0][0][0])[e] = px; (&s_in[0][1][0][0])[e] = ty;
  }
  __syncthreads();

  // Every thread fetches one element of the next four input rows while it does its stage's work (304 elements, 320
  // threads): which element, and whether its column is inside the image, does not change from step to step.
  const int st_row = tid / STRIP_IN, st_col = tid - st_row * STRIP_IN, st_x = x0 - 2 * HALO + st_col;
  const bool st_slot = tid < STRIP_ROWS * STRIP_IN;
  const bool st_ok = st_slot && st_col < STRIP_W + 4 * HALO && st_x >= 0 && st_x < W;
  float loss_local = 0.f;
  const int steps = 8 + (y1 - y0 + STRIP_ROWS - 1) / STRIP_ROWS;
  for (int it = 0; it < steps; it++) {
    const int a = y0 - 2 * HALO + STRIP_ROWS * it, b = a - 9, cr = b - 9, d = cr - STRIP_ROWS;
    const int buf = it & 1;
    const bool more = a + STRIP_ROWS <= y1 - 1 + 2 * HALO;   // stage A has rows to blur in the next step
    float nx = 0.f, ny = 0.f;
    {
      const int y = a + STRIP_ROWS + st_row;
      if (more && st_ok && y >= 0 && y < H) {
        const size_t q = (size_t)y * W + st_x;
        const uint32_t gp = gt[q];
        nx = pred_c[q * 4];
        ny = unpack(gp, c) + (1.f - unpack(gp, 3)) * bg_c;
      }
    }
    if (warp < 2) {
      // A: rows a .. a+3, sixteen groups of four statistics columns each.
      if (a <= y1 - 1 + 2 * HALO) {
        const int row = tid >> 4, g4 = (tid & 15) * 4;
        float x[16], y[16], in[16], out[4];
        load16(&s_in[buf][0][row][g4], x);
        load16(&s_in[buf][1][row][g4], y);
        const int slot = ring_slot(a + row);
        window4(x, gauss, out); *reinterpret_cast<float4*>(&s_hb[0][slot][g4]) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
        for (int k = 0; k < 16; k++) in[k] = x[k] * x[k];
        window4(in, gauss, out); *reinterpret_cast<float4*>(&s_hb[1][slot][g4]) = make_float4(out[0], out[1], out[2], out[3]);
        window4(y, gauss, out); *reinterpret_cast<float4*>(&s_hb[2][slot][g4]) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
        for (int k = 0; k < 16; k++) in[k] = y[k] * y[k];
        window4(in, gauss, out); *reinterpret_cast<float4*>(&s_hb[3][slot][g4]) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
        for (int k = 0; k < 16; k++) in[k] = x[k] * y[k];
        window4(in, gauss, out); *reinterpret_cast<float4*>(&s_hb[4][slot][g4]) = make_float4(out[0], out[1], out[2], out[3]);
      }
    } else if (warp < 6) {
      // B: statistics rows b .. b+3; a thread takes one column and two of the rows.
      if (b + STRIP_ROWS - 1 >= y0 - HALO && b <= y1 - 1 + HALO) {
        const int t = tid - 64, col = t & 63, r2 = (t >> 6) * 2;
        int slots[12];
        slots[0] = ring_slot(b + r2 - HALO);
#pragma unroll
        for (int k = 1; k < 12; k++) slots[k] = slots[k - 1] + 1 == RING ? 0 : slots[k - 1] + 1;
        float st[5][2];
#pragma unroll
        for (int m = 0; m < 5; m++) {
          float in[12];
#pragma unroll
          for (int k = 0; k < 12; k++) in[k] = s_hb[m][slots[k]][col];
          float o0 = 0.f, o1 = 0.f;
#pragma unroll
          for (int dd = 0; dd < 11; dd++) { o0 += gauss.w[dd] * in[dd]; o1 += gauss.w[dd] * in[dd + 1]; }
          st[m][0] = o0; st[m][1] = o1;
        }
        const int xg = x0 - HALO + col;
        const bool x_in = xg >= 0 && xg < W, x_own = xg >= x0 && xg < x_end;
#pragma unroll
        for (int o = 0; o < 2; o++) {
          const int y = b + r2 + o;
          float E0 = 0.f, E1 = 0.f, E2 = 0.f;
          if (x_in && y >= 0 && y < H) {
            const size_t q = (size_t)y * W + xg;
            const float wp = weights ? (float)weights[q] * (1.f / 255.f) : 1.f;
            const float M = wp * (lp.mask ? unpack(gt[q], 3) : 1.f) * norm;
            const float mu1 = st[0][o], mu2 = st[2][o];
            const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
            const float s1_raw = st[1][o] - mu1_sq, s2_raw = st[3][o] - mu2_sq;
            const float sigma1_sq = fmaxf(0.f, s1_raw), sigma2_sq = fmaxf(0.f, s2_raw);
            const float sigma12 = st[4][o] - mu1 * mu2;
            const float A1 = 2.f * mu1 * mu2 + C1, A2 = 2.f * sigma12 + C2, B1 = mu1_sq + mu2_sq + C1, B2 = sigma1_sq + sigma2_sq + C2;
            const float inv_BB = __fdividef(1.f, B1 * B2);   // approximate divisions, as in the reference's fast-math build
            const float raw = A1 * A2 * inv_BB;
            const float ssim = fminf(fmaxf(raw, -1.f), 1.f);
            if (x_own && y >= y0 && y < y1) loss_local += M * lp.ssim_w * ssim;
            if (raw > -1.f && raw < 1.f) {
              const float k = M * lp.ssim_w;
              const float d_mu1 = 2.f * mu2 * A2 * inv_BB - __fdividef(2.f * mu1 * ssim, B1);
              const float d_s1 = s1_raw > 0.f ? -__fdividef(ssim, B2) : 0.f;
              const float d_s12 = 2.f * A1 * inv_BB;
              const float Am = k * d_mu1, Bv = k * d_s1, Cc = k * d_s12;
              // gradient = blur(Am) + 2 p blur(Bv) - 2 blur(Bv mu1) + target blur(Cc) - blur(Cc mu2): the three maps
              // without a per-pixel factor are blurred as one.
              E0 = Am - 2.f * (Bv * mu1) - Cc * mu2; E1 = Bv; E2 = Cc;
            }
          }
          const int slot = slots[HALO + o];
          s_dv[0][slot][col] = E0; s_dv[1][slot][col] = E1; s_dv[2][slot][col] = E2;
        }
      }
    } else {
      const int t = tid - 192;   // 0 .. 127
      if (warp < 8) {
        // C: rows cr .. cr+3 of the three derivative maps blurred down the column, one column per thread.
        if (cr + STRIP_ROWS - 1 >= y0 && cr < y1) {
          const int col = t;
          int slot = ring_slot(cr - HALO);
          int slots[14];
#pragma unroll
          for (int k = 0; k < 14; k++) { slots[k] = slot; slot = slot + 1 == RING ? 0 : slot + 1; }
#pragma unroll
          for (int m = 0; m < 3; m++) {
            float in[16], out[4];
#pragma unroll
            for (int k = 0; k < 14; k++) in[k] = s_dv[m][slots[k]][col];
            in[14] = in[15] = 0.f;
            window4(in, gauss, out);
#pragma unroll
            for (int o = 0; o < 4; o++) s_bv[buf][m][o][col] = out[o];
          }
        }
      } else {
        // D: rows d .. d+3 (stage C wrote them in the step before), fourteen groups of four output columns.
        const int u = t - 64, row = u >> 4, g4 = (u & 15) * 4;
        const int y = d + row;
        if (g4 < STRIP_W && y >= y0 && y < y1) {
          float bl[3][4];
#pragma unroll
          for (int m = 0; m < 3; m++) {
            float in[16];
            load16(&s_bv[buf ^ 1][m][row][g4], in);
            window4(in, gauss, bl[m]);
          }
#pragma unroll
          for (int o = 0; o < 4; o++) {
            const int x = x0 + g4 + o;
            if (x < x_end) {
              const size_t q = (size_t)y * W + x;
              const uint32_t gp = gt[q];
              const float ga = unpack(gp, 3);
              const float wp = weights ? (float)weights[q] * (1.f / 255.f) : 1.f;
              const float M = wp * (lp.mask ? ga : 1.f) * norm;
              float p, pa = 0.f;
              if (c == 0) { const float4 pv = pred[q]; p = pv.x; pa = pv.w; } else p = pred_c[q * 4];
              const float g = unpack(gp, c) + (1.f - ga) * bg_c;
              const float sgn = p > g ? 1.f : (p < g ? -1.f : 0.f);
              loss_local += M * lp.l1_w * fabsf(p - g);
              out_c[q * 4] = (M * lp.l1_w * sgn + bl[0][o] + 2.f * p * bl[1][o] + g * bl[2][o]) * lp.grad_scale;
              if (c == 0) {   // the alpha lane travels with the first channel
                float ga_grad = 0.f;
                if (lp.alpha_lane) {
                  const float da = pa - ga;
                  const float sa = da > 0.f ? 1.f : (da < 0.f ? -1.f : 0.f);
                  const float Ma = wp * alpha_norm;
                  ga_grad = Ma * sa * lp.grad_scale;
                  loss_local += Ma * fabsf(da);
                }
                out_c[q * 4 + 3] = ga_grad;
              }
            }
          }
        }
      }
    }
    if (more && st_slot) { (&s_in[buf ^ 1][0][0][0])[tid] = nx; (&s_in[buf ^ 1][1][0][0])[tid] = ny; }   // consumed by stage A in the next step
    __syncthreads();
  }
  const float s = warp_sum(loss_local);
  if ((tid & 31) == 0) s_red[warp] = s;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < STRIP_THREADS / 32; i++) t += s_red[i];
    if (t != 0.f) atomicAdd(loss_accum, t);
  }
}

// Evaluation metrics (eval_metrics, src/gpu/loss.cu:241-293): squared error and SSIM sums of the 8-bit-quantised
// prediction against the target on a black background, optionally weighted by the target's alpha.
//
// One CTA per 16x16 tile runs the three channels over one staged 26x26 footprint (prediction and target are read from
// global memory once, not once per channel) and both blur passes are register-tiled like the loss kernel's: a thread
// makes four consecutive outputs of all five moments from one fourteen-wide window.
constexpr int EV_W = LOSS_TILE + 2 * HALO;   // 26: footprint of the tile's SSIM windows
constexpr int EV_S = 28;                     // row stride of the footprint planes (aligned 128-bit windows, zero pad)

__global__ void __launch_bounds__(TILE_PX) eval_kernel(const float4* __restrict__ pred, const uint32_t* __restrict__ gt, int W, int H, int tiles_x, int mask_w,
                                                       Gauss gauss, float* __restrict__ accum) {
  __shared__ __align__(16) float s_q[3][EV_W * EV_S];          // quantised prediction per channel
  __shared__ __align__(16) float s_t[3][EV_W * EV_S];          // target per channel
  __shared__ __align__(16) float s_row[5][EV_W][LOSS_TILE];    // horizontally blurred moments of the current channel
  __shared__ float s_part[2][TILE_PX / 32];
  const int tid = threadIdx.x;
  const int x0 = (blockIdx.x % tiles_x) * LOSS_TILE, y0 = (blockIdx.x / tiles_x) * LOSS_TILE;
  for (int i = tid; i < EV_W * EV_S; i += TILE_PX) {
    const int fy = i / EV_S, fx = i % EV_S;
    const int y = y0 + fy - HALO, x = x0 + fx - HALO;
    float q[3] = {0.f, 0.f, 0.f}, t[3] = {0.f, 0.f, 0.f};   // zero padding outside the image and in the row pad
    if (fx < EV_W && y >= 0 && y < H && x >= 0 && x < W) {
      const float4 pv = pred[y * W + x];
      const uint32_t gp = gt[y * W + x];
      const float pc[3] = {pv.x, pv.y, pv.z};
#pragma unroll
      for (int c = 0; c < 3; c++) { q[c] = rintf(fminf(fmaxf(pc[c], 0.f), 1.f) * 255.f) / 255.f; t[c] = unpack(gp, c); }
    }
#pragma unroll
    for (int c = 0; c < 3; c++) { s_q[c][i] = q[c]; s_t[c][i] = t[c]; }
  }
  __syncthreads();
  float se_sum = 0.f, ssim_sum = 0.f;
  for (int c = 0; c < 3; c++) {
    // Horizontal pass: 26 rows x 4 groups of four output columns.
    if (tid < EV_W * 4) {
      const int row = tid >> 2, g4 = (tid & 3) * 4;
      float x[16], y[16], in[16], out[4];
      load16(&s_q[c][row * EV_S + g4], x);
      load16(&s_t[c][row * EV_S + g4], y);
      window4(x, gauss, out); *reinterpret_cast<float4*>(&s_row[0][row][g4]) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
      for (int k = 0; k < 16; k++) in[k] = x[k] * x[k];
      window4(in, gauss, out); *reinterpret_cast<float4*>(&s_row[1][row][g4]) = make_float4(out[0], out[1], out[2], out[3]);
      window4(y, gauss, out); *reinterpret_cast<float4*>(&s_row[2][row][g4]) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
      for (int k = 0; k < 16; k++) in[k] = y[k] * y[k];
      window4(in, gauss, out); *reinterpret_cast<float4*>(&s_row[3][row][g4]) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
      for (int k = 0; k < 16; k++) in[k] = x[k] * y[k];
      window4(in, gauss, out); *reinterpret_cast<float4*>(&s_row[4][row][g4]) = make_float4(out[0], out[1], out[2], out[3]);
    }
    __syncthreads();
    // Vertical pass and the metrics: 16 columns x 4 groups of four output rows.
    if (tid < LOSS_TILE * 4) {
      const int col = tid & (LOSS_TILE - 1), r4 = (tid / LOSS_TILE) * 4;
      float st[5][4];
#pragma unroll
      for (int m = 0; m < 5; m++) {
        float in[16];
#pragma unroll
        for (int k = 0; k < 14; k++) in[k] = s_row[m][r4 + k][col];
        in[14] = in[15] = 0.f;
        window4(in, gauss, st[m]);
      }
#pragma unroll
      for (int o = 0; o < 4; o++) {
        const int y = y0 + r4 + o, x = x0 + col;
        if (y < H && x < W) {
          const float mu_p = st[0][o], mu_t = st[2][o];
          const float var_p = fmaxf(0.f, st[1][o] - mu_p * mu_p), var_t = fmaxf(0.f, st[3][o] - mu_t * mu_t), cov = st[4][o] - mu_p * mu_t;
          const float raw = ((2.f * mu_p * mu_t + C1) * (2.f * cov + C2)) / ((mu_p * mu_p + mu_t * mu_t + C1) * (var_p + var_t + C2));
          const int centre = (r4 + o + HALO) * EV_S + col + HALO;
          const float wgt = mask_w ? unpack(gt[y * W + x], 3) : 1.f;
          const float err = fabsf(s_q[c][centre] - s_t[c][centre]) * wgt;
          se_sum += err * err;
          ssim_sum += fminf(fmaxf(raw, -1.f), 1.f) * wgt;
        }
      }
    }
    __syncthreads();   // s_row is overwritten by the next channel
  }
  const float a = warp_sum(se_sum), b = warp_sum(ssim_sum);
  if ((tid & 31) == 0) { s_part[0][tid >> 5] = a; s_part[1][tid >> 5] = b; }
  __syncthreads();
  if (tid < 2) {
    float total = 0.f;
    for (int i = 0; i < TILE_PX / 32; i++) total += s_part[tid][i];
    atomicAdd(accum + 4 + tid, total);
  }
}

// Running loss sum and view count; also keeps the largest intersection total any view of the step produced, so that
// one readback per step (instead of one per view) tells the host whether a view overflowed its buffers.
__global__ void accumulate_kernel(float* a, uint32_t* num_isect) {
  a[2] += a[0] + a[1]; a[3] += 1.f;
  if (num_isect) num_isect[2] = max(num_isect[2], num_isect[0]);
}
// dst[2] += src[2], dst[3] += src[3]: folds the running loss of a second context (a view in flight on another stream).
__global__ void fold_loss_kernel(float* dst, const float* src) { dst[2] += src[2]; dst[3] += src[3]; }

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" int b2k_loss_photometric(const B2kCtx* c, const B2kLoss* lp, b2k_stream_t stream) {
  B2K_REQUIRE(c && lp && lp->rgba && c->out_rgba && c->v_out && c->loss_accum && c->W > 0 && c->H > 0);
  LossArgs a;
  a.l1_w = lp->l1_w; a.ssim_w = lp->ssim_w; a.bg[0] = lp->bg[0]; a.bg[1] = lp->bg[1]; a.bg[2] = lp->bg[2];
  a.composite = lp->composite; a.mask = lp->mask; a.alpha_lane = lp->alpha_lane;
  a.match_alpha_weight = lp->match_alpha_weight; a.scale = lp->scale; a.grad_scale = lp->grad_scale;
  static const Gauss g = make_gauss();
  // Rows per segment: as many segments as fill the resident CTA slots once (a second, partial wave costs more than the
  // eight pipeline-fill steps a longer segment amortises), in whole steps of four rows.
  const int strips = div_up(c->W, STRIP_W), slots = sm_count() * STRIP_CTAS_PER_SM;
  int segs = slots / (strips * 3);
  segs = segs < 1 ? 1 : segs;
  int seg_rows = div_up(div_up(c->H, segs), STRIP_ROWS) * STRIP_ROWS;
  if (seg_rows < 32) seg_rows = 32;
  const dim3 grid(strips, div_up(c->H, seg_rows), 3);
  photometric_strip_kernel<<<grid, STRIP_THREADS, 0, (cudaStream_t)stream>>>((const float4*)c->out_rgba, lp->rgba, lp->weights, c->W, c->H, seg_rows, a, g,
                                                                            (float4*)c->v_out, c->loss_accum);
  return check_launch();
}

extern "C" int b2k_loss_accumulate(const B2kCtx* c, b2k_stream_t stream) {
  B2K_REQUIRE(c && c->loss_accum);
  accumulate_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(c->loss_accum, c->num_isect);
  return check_launch();
}

extern "C" int b2k_loss_zero(const B2kCtx* c, int32_t first, int32_t count, b2k_stream_t stream) {
  B2K_REQUIRE(c && c->loss_accum && first >= 0 && count >= 0 && first + count <= 16);
  if (count) B2K_CUDA(cudaMemsetAsync(c->loss_accum + first, 0, (size_t)count * sizeof(float), (cudaStream_t)stream));
  return B2K_OK;
}

extern "C" int b2k_step_begin(const B2kCtx* c, b2k_stream_t stream) {
  B2K_REQUIRE(c && c->loss_accum);
  B2K_CUDA(cudaMemsetAsync(c->loss_accum, 0, 16 * sizeof(float), (cudaStream_t)stream));
  if (c->num_isect) B2K_CUDA(cudaMemsetAsync(c->num_isect + 2, 0, sizeof(uint32_t), (cudaStream_t)stream));
  return B2K_OK;
}

extern "C" int b2k_loss_fold(const B2kCtx* dst, const B2kCtx* src, b2k_stream_t stream) {
  B2K_REQUIRE(dst && src && dst->loss_accum && src->loss_accum && dst->loss_accum != src->loss_accum);
  fold_loss_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(dst->loss_accum, src->loss_accum);
  return check_launch();
}

extern "C" int b2k_eval_metrics(const B2kCtx* c, const uint32_t* rgba, int32_t mask_weighted, b2k_stream_t stream) {
  B2K_REQUIRE(c && rgba && c->out_rgba && c->loss_accum && c->W > 0 && c->H > 0);
  const int tiles_x = div_up(c->W, LOSS_TILE), tiles = tiles_x * div_up(c->H, LOSS_TILE);
  static const Gauss g = make_gauss();
  eval_kernel<<<tiles, TILE_PX, 0, (cudaStream_t)stream>>>((const float4*)c->out_rgba, rgba, c->W, c->H, tiles_x, mask_weighted, g, c->loss_accum);
  return check_launch();
}
