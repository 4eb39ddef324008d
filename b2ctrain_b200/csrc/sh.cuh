// Real spherical-harmonic basis up to degree 4 and its direction gradient, in the sign convention of the reference
// (sh_basis, src/gpu/splat_math.cuh:120-146; view-direction VJP, src/gpu/optim.cu:49-88).
#pragma once
#include "common.cuh"

namespace b2k {

#ifdef __CUDACC__

// b[k] for k < (DEG+1)^2. Entries of bands above `active` are zeroed so the caller can use a fixed trip count.
template <int DEG>
__device__ __forceinline__ void sh_basis(const float3 v, int active, float* b) {
  const float x = v.x, y = v.y, z = v.z;
  b[0] = 0.28209479177387814f;
  if constexpr (DEG >= 1) {
    const float m1 = active >= 1 ? 0.4886025f : 0.f;
    b[1] = -m1 * y; b[2] = m1 * z; b[3] = -m1 * x;
  }
  if constexpr (DEG >= 2) {
    const float on = active >= 2 ? 1.f : 0.f;
    const float z2 = z * z, fc1 = x * x - y * y, fs1 = 2.f * x * y;
    b[4] = on * 0.54627424f * fs1; b[5] = on * -1.0925485f * z * y; b[6] = on * (0.9461747f * z2 - 0.31539157f);
    b[7] = on * -1.0925485f * z * x; b[8] = on * 0.54627424f * fc1;
    if constexpr (DEG >= 3) {
      const float on3 = active >= 3 ? 1.f : 0.f;
      const float fc2 = x * fc1 - y * fs1, fs2 = x * fs1 + y * fc1;
      const float f0c = -2.285229f * z2 + 0.4570458f, f1b = 1.4453057f * z;
      const float p12 = z * (1.8658817f * z2 - 1.119529f);
      b[9] = on3 * -0.5900436f * fs2; b[10] = on3 * f1b * fs1; b[11] = on3 * f0c * y; b[12] = on3 * p12;
      b[13] = on3 * f0c * x; b[14] = on3 * f1b * fc1; b[15] = on3 * -0.5900436f * fc2;
      if constexpr (DEG >= 4) {
        const float on4 = active >= 4 ? 1.f : 0.f;
        const float fc3 = x * fc2 - y * fs2, fs3 = x * fs2 + y * fc2;
        const float f0d = z * (-4.683326f * z2 + 2.0071396f), f1c = 3.3116114f * z2 - 0.47308735f, f2b = -1.7701308f * z;
        const float p6 = 0.9461747f * z2 - 0.31539157f;
        b[16] = on4 * 0.62583575f * fs3; b[17] = on4 * f2b * fs2; b[18] = on4 * f1c * fs1; b[19] = on4 * f0d * y;
        b[20] = on4 * (1.9843135f * z * p12 - 1.0062306f * p6);
        b[21] = on4 * f0d * x; b[22] = on4 * f1c * fc1; b[23] = on4 * f2b * fc2; b[24] = on4 * 0.62583575f * fc3;
      }
    }
  }
}

// Gradient of sum_k b[k](v) * w[k] with respect to v, where w[k] = <sh_k, dL/dcolour>. Bands above `active` must carry
// w = 0. Written as explicit partial derivatives of the polynomials above.
template <int DEG>
__device__ __forceinline__ float3 sh_dir_grad(const float3 v, const float* w) {
  const float x = v.x, y = v.y, z = v.z;
  float gx = 0.f, gy = 0.f, gz = 0.f;
  if constexpr (DEG >= 1) { gy += -0.4886025f * w[1]; gz += 0.4886025f * w[2]; gx += -0.4886025f * w[3]; }
  if constexpr (DEG >= 2) {
    const float a = 0.54627424f, c = -1.0925485f;
    gx += 2.f * a * y * w[4] + c * z * w[7] + 2.f * a * x * w[8];
    gy += 2.f * a * x * w[4] + c * z * w[5] - 2.f * a * y * w[8];
    gz += c * y * w[5] + 2.f * 0.9461747f * z * w[6] + c * x * w[7];
  }
  if constexpr (DEG >= 3) {
    const float z2 = z * z, x2 = x * x, y2 = y * y, xy = x * y;
    const float f2a = -0.5900436f, f1b = 1.4453057f * z, f0c = -2.285229f * z2 + 0.4570458f, df0c = -4.570458f * z;
    // fs2 = 3x^2y - y^3, fc2 = x^3 - 3xy^2, fs1 = 2xy, fc1 = x^2 - y^2
    gx += f2a * 6.f * xy * w[9] + f1b * 2.f * y * w[10] + f0c * w[13] + f1b * 2.f * x * w[14] + f2a * 3.f * (x2 - y2) * w[15];
    gy += f2a * 3.f * (x2 - y2) * w[9] + f1b * 2.f * x * w[10] + f0c * w[11] - f1b * 2.f * y * w[14] - f2a * 6.f * xy * w[15];
    gz += 1.4453057f * 2.f * xy * w[10] + df0c * y * w[11] + (5.5976451f * z2 - 1.119529f) * w[12] + df0c * x * w[13] + 1.4453057f * (x2 - y2) * w[14];
  }
  if constexpr (DEG >= 4) {
    const float z2 = z * z, fc1 = x * x - y * y, fs1 = 2.f * x * y, fc2 = x * fc1 - y * fs1, fs2 = x * fs1 + y * fc1;
    const float f3a = 0.62583575f, f2b = -1.7701308f * z, f1c = 3.3116114f * z2 - 0.47308735f, df1c = 6.6232228f * z;
    const float f0d = z * (-4.683326f * z2 + 2.0071396f), df0d = -14.049978f * z2 + 2.0071396f;
    const float p12 = z * (1.8658817f * z2 - 1.119529f), dp12 = 5.5976451f * z2 - 1.119529f;
    const float dp20 = 1.9843135f * (p12 + z * dp12) - 1.0062306f * 1.8923494f * z;
    // d fs3 = (4 fs2, 4 fc2), d fc3 = (4 fc2, -4 fs2); d fs2 = (3 fs1, 3 fc1), d fc2 = (3 fc1, -3 fs1)
    gx += f3a * 4.f * fs2 * w[16] + f2b * 3.f * fs1 * w[17] + f1c * 2.f * y * w[18] + f0d * w[21] + f1c * 2.f * x * w[22] + f2b * 3.f * fc1 * w[23] + f3a * 4.f * fc2 * w[24];
    gy += f3a * 4.f * fc2 * w[16] + f2b * 3.f * fc1 * w[17] + f1c * 2.f * x * w[18] + f0d * w[19] - f1c * 2.f * y * w[22] - f2b * 3.f * fs1 * w[23] - f3a * 4.f * fs2 * w[24];
    gz += -1.7701308f * fs2 * w[17] + df1c * fs1 * w[18] + df0d * y * w[19] + dp20 * w[20] + df0d * x * w[21] + df1c * fc1 * w[22] - 1.7701308f * fc2 * w[23];
  }
  return make_float3(gx, gy, gz);
}

// Colour of splat i seen from the camera at cam_pos: SH up to `active` along the direction camera -> splat, + 0.5,
// clamped to +-100, non-finite -> 0 (src/gpu/project.cu:44-55). One definition, so every caller rounds alike.
template <int DEG>
__device__ __forceinline__ float4 splat_colour(int i, size_t cap, float3 mean, const float* __restrict__ cam_pos, int active,
                                               const float* __restrict__ sh_dc, const float* __restrict__ sh_hi) {
  float3 v = make_float3(mean.x - cam_pos[0], mean.y - cam_pos[1], mean.z - cam_pos[2]);
  const float inv = 1.f / fmaxf(sqrtf(v.x * v.x + v.y * v.y + v.z * v.z), 1e-12f);
  v.x *= inv; v.y *= inv; v.z *= inv;
  constexpr int K = (DEG + 1) * (DEG + 1);
  float b[K];
  sh_basis<DEG>(v, active, b);
  float c[3];
#pragma unroll
  for (int ch = 0; ch < 3; ch++) c[ch] = b[0] * sh_dc[(size_t)ch * cap + i];
  const int kact = (active + 1) * (active + 1);
#pragma unroll
  for (int k = 1; k < K; k++) {
    if (k < kact) {
#pragma unroll
      for (int ch = 0; ch < 3; ch++) c[ch] += b[k] * sh_hi[(size_t)((k - 1) * 3 + ch) * cap + i];
    }
  }
#pragma unroll
  for (int ch = 0; ch < 3; ch++) { const float t = c[ch] + 0.5f; c[ch] = isfinite(t) ? fminf(fmaxf(t, -100.f), 100.f) : 0.f; }
  return make_float4(c[0], c[1], c[2], 0.f);
}

#endif

}  // namespace b2k
