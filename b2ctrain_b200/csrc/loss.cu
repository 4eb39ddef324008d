// Fused photometric loss: L1 + 11-tap Gaussian SSIM (sigma 1.5, zero padding) + alpha-match lane, value and
// per-pixel gradient in one kernel. Reference semantics: photometric_kernel (src/gpu/loss.cu:18-195),
// accumulate_kernel (loss.cu:317), eval_kernel (loss.cu:241-293).
//
// One CTA of 256 threads owns a 16x16 pixel tile and runs the three colour channels back to back over one staged
// 36x36 footprint, so the float4 prediction and the packed target are read from global memory once per CTA (the
// reference launches one CTA per channel and reads them three times) and the gradient leaves as one 128-bit store
// per pixel. The work is a shared-memory stencil (forward separable blur of five moments, SSIM and its five partial
// derivative maps, the same blur applied backwards) and shared-memory bandwidth bounds it, so every blur pass is
// register-tiled: a thread produces four consecutive outputs from a fourteen-wide sliding window (3x fewer
// shared-memory reads than one output per thread), fetched with 128-bit loads along rows.
#include "common.cuh"

namespace b2k {
namespace {

constexpr int HALO = 5;
constexpr int STAT_W = LOSS_TILE + 2 * HALO;   // 26: positions whose SSIM statistics reach the tile
constexpr int IN_W = STAT_W + 2 * HALO;        // 36: input footprint
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

// Shared-memory planes of the loss kernel. Rows are padded so that every thread can fetch its sliding window with
// aligned 128-bit loads: 36-wide footprint planes use a stride of 40 floats, 26-wide planes a stride of 28.
constexpr int IN_S = 40, ST_S = 28;
constexpr int H_ROWS = 40;                        // rows of the horizontal-pass planes (36 used; the vertical windows overrun into the pad)
constexpr int OFF_P = 0;                          // [4][36][IN_S]   prediction r, g, b, alpha
constexpr int OFF_GT = OFF_P + 4 * IN_W * IN_S;   // [36][IN_S]      packed target
constexpr int OFF_M = OFF_GT + IN_W * IN_S;       // [26][ST_S]      loss weight M at the statistics positions
constexpr int OFF_H = OFF_M + STAT_W * ST_S;      // [5][H_ROWS][ST_S]
constexpr int OFF_V = OFF_H + 5 * H_ROWS * ST_S;  // [5][26][ST_S]
constexpr int OFF_G = OFF_V + 5 * STAT_W * ST_S;  // [3][256]        per-channel gradients of the tile
constexpr size_t LOSS_SMEM = sizeof(float) * (OFF_G + 3 * TILE_PX);

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

__global__ void __launch_bounds__(TILE_PX) photometric_kernel(const float4* __restrict__ pred, const uint32_t* __restrict__ gt, const uint8_t* __restrict__ weights,
                                                              int W, int H, int tiles_x, LossArgs lp, Gauss gauss, float4* __restrict__ v_out, float* __restrict__ loss_accum) {
  extern __shared__ __align__(16) float smem[];
  float* s_p = smem + OFF_P;
  uint32_t* s_gt = reinterpret_cast<uint32_t*>(smem + OFF_GT);
  float* s_m = smem + OFF_M;
  float* s_h = smem + OFF_H;
  float* s_v = smem + OFF_V;
  float* s_grad = smem + OFF_G;
  __shared__ float s_red[TILE_PX / 32];

  const int tile = blockIdx.x, tid = threadIdx.x;
  const int tx0 = (tile % tiles_x) * LOSS_TILE, ty0 = (tile / tiles_x) * LOSS_TILE;
  const float norm = lp.scale / (3.f * (float)W * (float)H);
  const int ly = tid / LOSS_TILE, lx = tid % LOSS_TILE;
  const int gy = ty0 + ly, gx = tx0 + lx;
  const bool inside = gy < H && gx < W;
  const int pix = inside ? gy * W + gx : 0;
  const int centre = (ly + 2 * HALO) * IN_S + lx + 2 * HALO;
  const int centre_m = (ly + HALO) * ST_S + lx + HALO;

  // Stage the 36x36 footprint (zero outside the image, zero in the row pads).
  float flat_r = 0.f, flat_g = 0.f, flat_b = 0.f;   // per channel: max |pred - target| over the footprint
  for (int i = tid; i < IN_W * IN_S; i += TILE_PX) {
    const int fy = i / IN_S, fx = i % IN_S;
    const int y = ty0 + fy - 2 * HALO, x = tx0 + fx - 2 * HALO;
    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t gp = 0xFF000000u;   // outside the image: opaque black, so the effective target is zero there (zero padding)
    if (fx < IN_W && y >= 0 && y < H && x >= 0 && x < W) {
      const int q = y * W + x;
      p = pred[q];
      gp = gt[q];
      const float ga = unpack(gp, 3);
      float g0 = unpack(gp, 0), g1 = unpack(gp, 1), g2 = unpack(gp, 2);
      if (lp.composite) { g0 += (1.f - ga) * lp.bg[0]; g1 += (1.f - ga) * lp.bg[1]; g2 += (1.f - ga) * lp.bg[2]; }
      flat_r = fmaxf(flat_r, fabsf(p.x - g0)); flat_g = fmaxf(flat_g, fabsf(p.y - g1)); flat_b = fmaxf(flat_b, fabsf(p.z - g2));
      const int sy = fy - HALO, sx = fx - HALO;
      if (sy >= 0 && sy < STAT_W && sx >= 0 && sx < STAT_W) {
        const float wp = weights ? (float)weights[q] * (1.f / 255.f) : 1.f;
        s_m[sy * ST_S + sx] = wp * (lp.mask ? ga : 1.f) * norm;
      }
    } else {
      const int sy = fy - HALO, sx = fx - HALO;
      if (fx < IN_W && sy >= 0 && sy < STAT_W && sx >= 0 && sx < STAT_W) s_m[sy * ST_S + sx] = 0.f;   // outside the image
    }
    s_p[i] = p.x; s_p[IN_W * IN_S + i] = p.y; s_p[2 * IN_W * IN_S + i] = p.z; s_p[3 * IN_W * IN_S + i] = p.w;
    s_gt[i] = gp;
  }
  float gt_a = 0.f, wp_c = 1.f;
  if (inside) {
    gt_a = unpack(gt[pix], 3);
    wp_c = weights ? (float)weights[pix] * (1.f / 255.f) : 1.f;
  }
  __syncthreads();
  if (lp.alpha_lane && inside) flat_r = fmaxf(flat_r, fabsf(s_p[3 * IN_W * IN_S + centre] - gt_a));

  float loss_local = 0.f;
  // Exact early exit per channel: where the prediction equals the effective target on the whole footprint (for the
  // first channel: and alpha matches on the tile) every gradient of that channel is exactly zero and SSIM is exactly
  // one, so only the constant term enters the loss.
  const bool nonflat[3] = {__syncthreads_or(flat_r > 0.f) != 0, __syncthreads_or(flat_g > 0.f) != 0, __syncthreads_or(flat_b > 0.f) != 0};
  for (int c = 0; c < 3; c++) {
    if (!nonflat[c]) {
      if (inside) loss_local += s_m[centre_m] * lp.ssim_w;
      s_grad[c * TILE_PX + tid] = 0.f;
      continue;
    }
    const float* P = s_p + c * IN_W * IN_S;
    const float bg_c = lp.composite ? lp.bg[c] : 0.f;
    // Pass 1, horizontal blur of the five moments. One thread = one row x four output columns (36 x 7 items).
    if (tid < IN_W * 7) {
      const int row = tid / 7, g4 = (tid % 7) * 4;
      float x[16], y[16];
      load16(P + row * IN_S + g4, x);
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const uint4 t = reinterpret_cast<const uint4*>(s_gt + row * IN_S + g4)[q];
        const uint32_t w4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int e = 0; e < 4; e++) y[q * 4 + e] = unpack(w4[e], c) + (1.f - unpack(w4[e], 3)) * bg_c;
      }
      float in[16], out[4];
      float* hb = s_h + row * ST_S + g4;
      window4(x, gauss, out); *reinterpret_cast<float4*>(hb) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
      for (int k = 0; k < 16; k++) in[k] = x[k] * x[k];
      window4(in, gauss, out); *reinterpret_cast<float4*>(hb + H_ROWS * ST_S) = make_float4(out[0], out[1], out[2], out[3]);
      window4(y, gauss, out); *reinterpret_cast<float4*>(hb + 2 * H_ROWS * ST_S) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
      for (int k = 0; k < 16; k++) in[k] = y[k] * y[k];
      window4(in, gauss, out); *reinterpret_cast<float4*>(hb + 3 * H_ROWS * ST_S) = make_float4(out[0], out[1], out[2], out[3]);
#pragma unroll
      for (int k = 0; k < 16; k++) in[k] = x[k] * y[k];
      window4(in, gauss, out); *reinterpret_cast<float4*>(hb + 4 * H_ROWS * ST_S) = make_float4(out[0], out[1], out[2], out[3]);
    }
    __syncthreads();
    // Pass 2, vertical blur -> statistics at 26 x 26, SSIM there, partial derivative maps scaled by M * ssim_w.
    // One thread = one column x four output rows (26 x 7 items).
    if (tid < STAT_W * 7) {
      const int col = tid % STAT_W, r4 = (tid / STAT_W) * 4;
      float st[5][4];
#pragma unroll
      for (int m = 0; m < 5; m++) {
        float in[16];
        const float* hp = s_h + m * H_ROWS * ST_S + r4 * ST_S + col;
#pragma unroll
        for (int k = 0; k < 14; k++) in[k] = hp[k * ST_S];
        in[14] = in[15] = 0.f;
        window4(in, gauss, st[m]);
      }
#pragma unroll
      for (int o = 0; o < 4; o++) {
        const int oy = r4 + o;
        if (oy >= STAT_W) break;
        const float M = s_m[oy * ST_S + col];   // zero outside the image
        float A = 0.f, B = 0.f, Bm = 0.f, Cc = 0.f, Cm = 0.f;
        const int y = ty0 + oy - HALO, xg = tx0 + col - HALO;
        if (y >= 0 && y < H && xg >= 0 && xg < W) {
          const float mu1 = st[0][o], mu2 = st[2][o];
          const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
          const float s1_raw = st[1][o] - mu1_sq, s2_raw = st[3][o] - mu2_sq;
          const float sigma1_sq = fmaxf(0.f, s1_raw), sigma2_sq = fmaxf(0.f, s2_raw);
          const float sigma12 = st[4][o] - mu1 * mu2;
          const float A1 = 2.f * mu1 * mu2 + C1, A2 = 2.f * sigma12 + C2, B1 = mu1_sq + mu2_sq + C1, B2 = sigma1_sq + sigma2_sq + C2;
          const float inv_BB = 1.f / (B1 * B2);
          const float raw = A1 * A2 * inv_BB;
          const float ssim = fminf(fmaxf(raw, -1.f), 1.f);
          if (oy >= HALO && oy < HALO + LOSS_TILE && col >= HALO && col < HALO + LOSS_TILE) {
            const int fi = (oy + HALO) * IN_S + col + HALO;
            const uint32_t gp = s_gt[fi];
            const float gv = unpack(gp, c) + (1.f - unpack(gp, 3)) * bg_c;
            loss_local += M * (lp.l1_w * fabsf(P[fi] - gv) + lp.ssim_w * ssim);
          }
          if (raw > -1.f && raw < 1.f) {
            const float k = M * lp.ssim_w;
            const float d_mu1 = 2.f * mu2 * A2 * inv_BB - 2.f * mu1 * ssim / B1;
            const float d_s1 = s1_raw > 0.f ? -ssim / B2 : 0.f;
            const float d_s12 = 2.f * A1 * inv_BB;
            A = k * d_mu1; B = k * d_s1; Bm = B * mu1; Cc = k * d_s12; Cm = Cc * mu2;
          }
        }
        float* vp = s_v + oy * ST_S + col;
        vp[0] = A; vp[STAT_W * ST_S] = B; vp[2 * STAT_W * ST_S] = Bm; vp[3 * STAT_W * ST_S] = Cc; vp[4 * STAT_W * ST_S] = Cm;
      }
    }
    __syncthreads();
    // Pass 3, backward blur, horizontal: rows 0..25, output columns 0..15. One task = one moment x one row x four columns
    // (520 tasks over the 256 threads: two rounds, where one thread per row and column group would run five in a row).
    for (int task = tid; task < 5 * STAT_W * 4; task += TILE_PX) {
      const int m = task / (STAT_W * 4), rem = task - m * (STAT_W * 4), row = rem >> 2, g4 = (rem & 3) * 4;
      float in[16], out[4];
      load16(s_v + m * STAT_W * ST_S + row * ST_S + g4, in);
      window4(in, gauss, out);
      *reinterpret_cast<float4*>(s_h + m * H_ROWS * ST_S + row * ST_S + g4) = make_float4(out[0], out[1], out[2], out[3]);
    }
    __syncthreads();
    // Pass 4, backward blur, vertical. One task = one moment x one column x four rows (320 tasks, two rounds); the five
    // blurred maps of the tile go to shared memory (the plane pass 3 has finished reading) for the per-pixel chain rule.
    float* s_b = s_v;   // [5][16][16]
    for (int task = tid; task < 5 * LOSS_TILE * 4; task += TILE_PX) {
      const int m = task / (LOSS_TILE * 4), rem = task - m * (LOSS_TILE * 4), col = rem % LOSS_TILE, r4 = (rem / LOSS_TILE) * 4;
      float in[16], out[4];
      const float* hp = s_h + m * H_ROWS * ST_S + r4 * ST_S + col;
#pragma unroll
      for (int k = 0; k < 14; k++) in[k] = hp[k * ST_S];
      in[14] = in[15] = 0.f;
      window4(in, gauss, out);
#pragma unroll
      for (int o = 0; o < 4; o++) s_b[m * TILE_PX + (r4 + o) * LOSS_TILE + col] = out[o];
    }
    __syncthreads();
    {   // the chain rule through the five moments, one pixel per thread
      const int fi = (ly + 2 * HALO) * IN_S + lx + 2 * HALO;
      const uint32_t gp = s_gt[fi];
      const float p = P[fi], g = unpack(gp, c) + (1.f - unpack(gp, 3)) * bg_c;
      const float sgn = p > g ? 1.f : (p < g ? -1.f : 0.f);
      const float M = s_m[centre_m];
      s_grad[c * TILE_PX + tid] = (M * lp.l1_w * sgn + s_b[tid] + 2.f * p * s_b[TILE_PX + tid] - 2.f * s_b[2 * TILE_PX + tid] + g * s_b[3 * TILE_PX + tid] -
                                   s_b[4 * TILE_PX + tid]) * lp.grad_scale;
    }
    __syncthreads();   // s_h / s_v are reused by the next channel; s_grad is read below
  }
  float4 grad = make_float4(s_grad[tid], s_grad[TILE_PX + tid], s_grad[2 * TILE_PX + tid], 0.f);
  if (inside && lp.alpha_lane && nonflat[0]) {
    const float da = s_p[3 * IN_W * IN_S + centre] - gt_a;
    const float sa = da > 0.f ? 1.f : (da < 0.f ? -1.f : 0.f);
    const float Ma = wp_c * lp.match_alpha_weight * lp.scale / ((float)W * (float)H);
    grad.w = Ma * sa * lp.grad_scale;
    loss_local += Ma * fabsf(da);
  }
  if (inside) v_out[pix] = grad;
  const float s = warp_sum(loss_local);
  if ((tid & 31) == 0) s_red[tid >> 5] = s;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < TILE_PX / 32; i++) t += s_red[i];
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

bool g_smem_set[64] = {false};

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" int b2k_loss_photometric(const B2kCtx* c, const B2kLoss* lp, b2k_stream_t stream) {
  B2K_REQUIRE(c && lp && lp->rgba && c->out_rgba && c->v_out && c->loss_accum && c->W > 0 && c->H > 0);
  int dev = 0;
  B2K_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !g_smem_set[dev]) {
    B2K_CUDA(cudaFuncSetAttribute(photometric_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LOSS_SMEM));
    g_smem_set[dev] = true;
  }
  const int tiles_x = div_up(c->W, LOSS_TILE), tiles = tiles_x * div_up(c->H, LOSS_TILE);
  LossArgs a;
  a.l1_w = lp->l1_w; a.ssim_w = lp->ssim_w; a.bg[0] = lp->bg[0]; a.bg[1] = lp->bg[1]; a.bg[2] = lp->bg[2];
  a.composite = lp->composite; a.mask = lp->mask; a.alpha_lane = lp->alpha_lane;
  a.match_alpha_weight = lp->match_alpha_weight; a.scale = lp->scale; a.grad_scale = lp->grad_scale;
  static const Gauss g = make_gauss();
  photometric_kernel<<<tiles, TILE_PX, LOSS_SMEM, (cudaStream_t)stream>>>((const float4*)c->out_rgba, lp->rgba, lp->weights, c->W, c->H, tiles_x, a, g,
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
