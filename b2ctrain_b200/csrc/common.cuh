// Shared device code of the b2k kernels: constants, status plumbing, the fp32 EWA projection and the exact tile
// decision functions.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/b2k.h"

namespace b2k {

constexpr int RT_W = 8;                 // rasteriser tile edge (reference: src/gpu/util.cuh:19)
constexpr int RT_PX = RT_W * RT_W;
constexpr int LOSS_TILE = 16;           // loss tile edge (util.cuh:17)
constexpr int GRAD_LANES = 13;          // xy 2, conic 3, rgb 3, opacity 1, refine 1, feat 3 (splat_math.cuh:10)
constexpr float ALPHA_CUTOFF = 1.0f / 255.0f;
constexpr float T_CUTOFF = 1e-4f;
constexpr float ALPHA_MAX = 0.999f;
constexpr int NUM_SMS_HINT = 148;       // B200; grids of persistent kernels are sized from the device at run time

extern int g_last_cuda_error;
int check_launch();                     // cudaGetLastError -> status
int sm_count();
// Records, tile boxes and depth keys only (project.cu): the chunked renderer tests tiles and shades later.
int launch_project_lite(const B2kModel* m, const B2kCamera* cam, const B2kRenderOpts* o, const B2kCtx* c, cudaStream_t s);
// One depth chunk of a chunked view, or the whole view when n_chunks <= 1 (raster_fwd.cu).
int launch_raster_fwd(const B2kCtx* c, const B2kRenderOpts* o, int chunk, int n_chunks, uint32_t* alive, cudaStream_t s);

#define B2K_REQUIRE(cond) do { if (!(cond)) return B2K_ERR_ARG; } while (0)
#define B2K_CUDA(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) { b2k::g_last_cuda_error = (int)e_; return B2K_ERR_CUDA; } } while (0)

__host__ __device__ inline int div_up(long long a, int b) { return (int)((a + b - 1) / b); }

// Layout of the caller's sort_tmp scratch. The first words hold the list of splats with large tile boxes, shared by
// the projection (which fills it) and the binning (which emits from it); the radix sort's tables follow.
constexpr size_t BIG_HEADER_WORDS = 16;   // [0] projection's big-splat count, [1] emit's big-splat count
inline uint32_t* big_count_ptr(const B2kCtx* c) { return (uint32_t*)c->sort_tmp; }
inline uint32_t* big_list_ptr(const B2kCtx* c) { return (uint32_t*)c->sort_tmp + BIG_HEADER_WORDS; }
inline uint32_t* big_emit_ptr(const B2kCtx* c) { return (uint32_t*)c->sort_tmp + BIG_HEADER_WORDS + (size_t)c->n_cap; }       // [n_cap][2]
inline uint32_t* sort_tables_ptr(const B2kCtx* c) { return (uint32_t*)c->sort_tmp + BIG_HEADER_WORDS + 3 * (size_t)c->n_cap; }

// Segments of the backward replay. The forward leaves a per-pixel checkpoint (colour sums, transmittance) in
// ctx->bwd_scratch before every SEG_LEN-th fragment of a tile's list and, in a chunked view, where a later depth chunk
// takes a tile over; the backward replays the segments between checkpoints as independent work items.
// Scratch layout: [BWD_HEADER_WORDS] (word 0: item count, word 1: item cursor), [slots] items (range index, segment),
// [slots][64] float4 checkpoints. The checkpoint before fragment range_start + seg * SEG_LEN of range q (= chunk *
// n_tiles + tile) lives in slot (range_start >> SEG_SHIFT) + q + seg: ranges follow each other in the sorted buffer in
// the order of q, which makes the map injective without any table.
#ifndef B2K_SEG_SHIFT
#define B2K_SEG_SHIFT 7
#endif
constexpr int SEG_SHIFT = B2K_SEG_SHIFT, SEG_LEN = 1 << SEG_SHIFT;
constexpr size_t BWD_HEADER_WORDS = 16;
__host__ __device__ inline uint64_t bwd_slots(uint64_t isect_cap, uint64_t n_ranges) { return (((isect_cap >> SEG_SHIFT) + n_ranges + 2) + 1) & ~1ull; }
__host__ __device__ inline uint32_t ckpt_slot(uint32_t range_start, int q, uint32_t seg) { return (range_start >> SEG_SHIFT) + (uint32_t)q + seg; }
inline uint64_t bwd_ranges(const B2kCtx* c) { return (uint64_t)c->n_tiles * (c->n_chunks > 1 ? c->n_chunks : 1); }
inline uint32_t* bwd_work_ptr(const B2kCtx* c) { return (uint32_t*)c->bwd_scratch; }
inline uint2* bwd_items_ptr(const B2kCtx* c) { return (uint2*)((uint32_t*)c->bwd_scratch + BWD_HEADER_WORDS); }
inline float4* bwd_ckpt_ptr(const B2kCtx* c) { return (float4*)(bwd_items_ptr(c) + bwd_slots(c->isect_cap, bwd_ranges(c))); }

struct CamDev {
  float R[9]; float t[3]; float pos[3]; float fx, fy, cx, cy; int W, H; float lim_pos_x, lim_pos_y, lim_neg_x, lim_neg_y;
};
inline CamDev to_camdev(const B2kCamera& c) {
  CamDev d;
  for (int i = 0; i < 9; i++) d.R[i] = c.R[i];
  for (int i = 0; i < 3; i++) { d.t[i] = c.t[i]; d.pos[i] = c.pos[i]; }
  d.fx = c.fx; d.fy = c.fy; d.cx = c.cx; d.cy = c.cy; d.W = c.W; d.H = c.H;
  d.lim_pos_x = c.lim_pos_x; d.lim_pos_y = c.lim_pos_y; d.lim_neg_x = c.lim_neg_x; d.lim_neg_y = c.lim_neg_y;
  return d;
}

#ifdef __CUDACC__

// max-update of a non-negative float statistic that several views may touch at once (bit patterns of non-negative
// floats order like integers).
__device__ __forceinline__ void atomic_max_nonneg(float* p, float v) { atomicMax(reinterpret_cast<int*>(p), __float_as_int(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------------------------------------
// Exact tile decisions. Everything below is a fixed tree of IEEE round-to-nearest single-precision operations (no
// contraction into FMA, no approximate division or square root), so a host evaluation of the same tree in plain
// float arithmetic gives the same tiles bit for bit. Inputs are the fp32 record the projection stored.
// Reference semantics: tile_bbox / tile_hit (src/gpu/splat_math.cuh:27-53), extent and on-screen culls
// (splat_math.cuh:284-290).
// ---------------------------------------------------------------------------------------------------------------
struct TileRec {
  float mx, my, c00, c01, c11, power;
  float ia, ib;   // 1 / (64 c00), 1 / (64 c11): the per-splat denominators of the closest-point parameters
};
__device__ __forceinline__ TileRec make_tile_rec(float mx, float my, float c00, float c01, float c11, float power) {
  TileRec r{mx, my, c00, c01, c11, power, 0.f, 0.f};
  r.ia = __fdiv_rn(1.f, __fmul_rn(64.f, c00));
  r.ib = __fdiv_rn(1.f, __fmul_rn(64.f, c11));
  return r;
}
struct TileBox { int min_x, min_y, max_x, max_y; };

__device__ __forceinline__ float rn_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float rn_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float rn_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float rn_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float clamp01(float x) { return fminf(fmaxf(x, 0.f), 1.f); }

__device__ __forceinline__ bool tile_box(const TileRec& r, int W, int H, int tiles_x, int tiles_y, TileBox& b) {
  const float detc = rn_sub(rn_mul(r.c00, r.c11), rn_mul(r.c01, r.c01));
  if (!(detc > 0.f)) return false;
  const float inv = rn_div(1.f, detc);
  const float p2 = rn_mul(2.f, r.power);
  const float ex = __fsqrt_rn(rn_mul(rn_mul(p2, r.c11), inv)), ey = __fsqrt_rn(rn_mul(rn_mul(p2, r.c00), inv));
  if (!(ex >= 0.f && ey >= 0.f)) return false;
  const bool on = rn_add(r.mx, ex) > 0.f && rn_sub(r.mx, ex) < (float)W && rn_add(r.my, ey) > 0.f && rn_sub(r.my, ey) < (float)H;
  if (!on) return false;
  const float tw = (float)RT_W, txs = (float)tiles_x, tys = (float)tiles_y;
  const float cx = rn_div(r.mx, tw), cy = rn_div(r.my, tw), dx = rn_div(ex, tw), dy = rn_div(ey, tw);
  b.min_x = (int)fminf(fmaxf(rn_sub(cx, dx), 0.f), txs);
  b.min_y = (int)fminf(fmaxf(rn_sub(cy, dy), 0.f), tys);
  b.max_x = (int)fminf(fmaxf(rn_add(rn_add(cx, dx), 1.f), 0.f), txs);
  b.max_y = (int)fminf(fmaxf(rn_add(rn_add(cy, dy), 1.f), 0.f), tys);
  return true;
}

__device__ __forceinline__ bool tile_hit(int tx, int ty, const TileRec& r) {
  const float rmin_x = (float)(tx * RT_W), rmin_y = (float)(ty * RT_W);
  const float rmax_x = rmin_x + (float)RT_W, rmax_y = rmin_y + (float)RT_W;   // exact: small integers
  const bool x_left = r.mx < rmin_x, x_right = r.mx > rmax_x, in_x = !(x_left || x_right);
  const bool y_above = r.my < rmin_y, y_below = r.my > rmax_y, in_y = !(y_above || y_below);
  if (in_x && in_y) return true;
  const float corner_x = x_left ? rmin_x : rmax_x, corner_y = y_above ? rmin_y : rmax_y;
  const float dxf = x_left ? (float)RT_W : -(float)RT_W, dyf = y_above ? (float)RT_W : -(float)RT_W;
  const float diff_x = rn_sub(r.mx, corner_x), diff_y = rn_sub(r.my, corner_y);
  // t = d (c00 diff_x + c01 diff_y) / (d^2 c00) with d = +-8: the division is by a per-splat constant.
  const float tx_raw = rn_mul(rn_mul(dxf, rn_add(rn_mul(r.c00, diff_x), rn_mul(r.c01, diff_y))), r.ia);
  const float ty_raw = rn_mul(rn_mul(dyf, rn_add(rn_mul(r.c01, diff_x), rn_mul(r.c11, diff_y))), r.ib);
  const float tx_c = in_y ? 0.f : clamp01(tx_raw), ty_c = in_x ? 0.f : clamp01(ty_raw);
  const float px = rn_add(corner_x, rn_mul(tx_c, dxf)), py = rn_add(corner_y, rn_mul(ty_c, dyf));
  const float dx = rn_sub(px, r.mx), dy = rn_sub(py, r.my);
  const float q = rn_add(rn_mul(rn_mul(r.c00, dx), dx), rn_mul(rn_mul(r.c11, dy), dy));
  const float sigma = rn_add(rn_mul(0.5f, q), rn_mul(rn_mul(r.c01, dx), dy));
  return sigma <= r.power;
}

// ---------------------------------------------------------------------------------------------------------------
// EWA projection of one splat with the 3D-filter scale floor. Reference semantics: project_one
// (src/gpu/splat_math.cuh:224-293) without its mip branch (rejected by the reference's CLI, main.cpp:26). The
// extent / on-screen culls live in tile_box above so that they are decided from the stored record.
// ---------------------------------------------------------------------------------------------------------------
struct Proj {
  float3 mean_c;
  float3 s, s2_raw;
  float comp_floor;
  float Rq[9];
  float J02, J12, dx, dy;     // J = [[dx, 0, J02], [0, dy, J12]]
  bool clamp_x, clamp_y;
  float c00, c01, c11;        // conic
  float opac, sig;
  float mx, my;
  float power;
};

__device__ __forceinline__ void quat_to_mat(float w, float x, float y, float z, float* R) {
  const float x2 = x * x, y2 = y * y, z2 = z * z, xy = x * y, xz = x * z, yz = y * z, wx = w * x, wy = w * y, wz = w * z;
  R[0] = 1.f - 2.f * (y2 + z2); R[1] = 2.f * (xy - wz);       R[2] = 2.f * (xz + wy);
  R[3] = 2.f * (xy + wz);       R[4] = 1.f - 2.f * (x2 + z2); R[5] = 2.f * (yz - wx);
  R[6] = 2.f * (xz - wy);       R[7] = 2.f * (yz + wx);       R[8] = 1.f - 2.f * (x2 + y2);
}

// The projection of one splat, in the stages the backward walks in reverse (geometry_backward): camera-space mean,
// scales with the 3D-filter floor, rotation, the axes of the splat in camera space, the perspective Jacobian with its
// clamp, the screen covariance with the 0.3 px blur, and its inverse. Returns false where the reference culls
// (src/gpu/splat_math.cuh:224-293); the expression trees are the reference's so that both make the same decisions.
__device__ __forceinline__ bool finite3(const float3 v) { return isfinite(v.x) && isfinite(v.y) && isfinite(v.z); }

__device__ __forceinline__ float3 to_camera(const CamDev& cam, const float4 po) {
  const float* W2C = cam.R;
  return make_float3(W2C[0] * po.x + W2C[1] * po.y + W2C[2] * po.z + cam.t[0], W2C[3] * po.x + W2C[4] * po.y + W2C[5] * po.z + cam.t[1],
                     W2C[6] * po.x + W2C[7] * po.y + W2C[8] * po.z + cam.t[2]);
}

// Squared scales from the log scales, the scales with the floor f folded in, and the opacity compensation of the floor.
__device__ __forceinline__ void floored_scales(const float4 ls, Proj& r) {
  r.s2_raw = make_float3(expf(2.f * ls.x), expf(2.f * ls.y), expf(2.f * ls.z));
  const float floor_sq = ls.w * ls.w;
  const float3 widened = make_float3(r.s2_raw.x + floor_sq, r.s2_raw.y + floor_sq, r.s2_raw.z + floor_sq);
  r.s = make_float3(sqrtf(widened.x), sqrtf(widened.y), sqrtf(widened.z));
  r.comp_floor = ls.w > 0.f ? sqrtf((r.s2_raw.x * r.s2_raw.y * r.s2_raw.z) / (widened.x * widened.y * widened.z)) : 1.f;
}

// axes = R_view * R(q) * diag(s), row-major: column j is the splat's j-th semi-axis in camera space.
__device__ __forceinline__ void camera_axes(const CamDev& cam, const Proj& r, float (&axes)[9]) {
  const float* W2C = cam.R;
#pragma unroll
  for (int row = 0; row < 3; row++) {
    axes[row * 3 + 0] = (W2C[row * 3] * r.Rq[0] + W2C[row * 3 + 1] * r.Rq[3] + W2C[row * 3 + 2] * r.Rq[6]) * r.s.x;
    axes[row * 3 + 1] = (W2C[row * 3] * r.Rq[1] + W2C[row * 3 + 1] * r.Rq[4] + W2C[row * 3 + 2] * r.Rq[7]) * r.s.y;
    axes[row * 3 + 2] = (W2C[row * 3] * r.Rq[2] + W2C[row * 3 + 1] * r.Rq[5] + W2C[row * 3 + 2] * r.Rq[8]) * r.s.z;
  }
}

__device__ __forceinline__ bool project_one(const float4 po, const float4 q, const float4 ls, const CamDev& cam, Proj& r) {
  // 1. camera space, near plane
  r.mean_c = to_camera(cam, po);
  if (!(finite3(r.mean_c) && r.mean_c.z <= 1e10f)) return false;
  if (!(r.mean_c.z >= 0.01f)) return false;
  // 2. scales and rotation
  floored_scales(ls, r);
  if (!finite3(r.s)) return false;
  const float quat_sq = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
  if (!(quat_sq >= 1e-6f && isfinite(quat_sq))) return false;
  if (!isfinite(po.w)) return false;
  const float unit = 1.f / sqrtf(quat_sq);
  quat_to_mat(q.x * unit, q.y * unit, q.z * unit, q.w * unit, r.Rq);
  float axes[9];
  camera_axes(cam, r, axes);
  // 3. perspective Jacobian [[dx, 0, J02], [0, dy, J12]], the ray clamped to the guard band around the image
  const float depth_inv = 1.f / r.mean_c.z;
  const float ray_x = r.mean_c.x * depth_inv, ray_y = r.mean_c.y * depth_inv;
  const float held_x = fminf(fmaxf(ray_x, cam.lim_neg_x), cam.lim_pos_x), held_y = fminf(fmaxf(ray_y, cam.lim_neg_y), cam.lim_pos_y);
  r.clamp_x = !(ray_x <= cam.lim_pos_x && ray_x >= cam.lim_neg_x);
  r.clamp_y = !(ray_y <= cam.lim_pos_y && ray_y >= cam.lim_neg_y);
  r.dx = cam.fx * depth_inv; r.dy = cam.fy * depth_inv;
  r.J02 = -r.dx * held_x; r.J12 = -r.dy * held_y;
  // 4. screen covariance = (J axes)(J axes)^T, kept in range, + 0.3 px of blur
  float JA[6];
#pragma unroll
  for (int j = 0; j < 3; j++) { JA[j] = r.dx * axes[j] + r.J02 * axes[6 + j]; JA[3 + j] = r.dy * axes[3 + j] + r.J12 * axes[6 + j]; }
  float cov_xx = JA[0] * JA[0] + JA[1] * JA[1] + JA[2] * JA[2], cov_xy = JA[0] * JA[3] + JA[1] * JA[4] + JA[2] * JA[5],
        cov_yy = JA[3] * JA[3] + JA[4] * JA[4] + JA[5] * JA[5];
  const float largest = fmaxf(fabsf(cov_xx), fmaxf(fabsf(cov_xy), fabsf(cov_yy)));
  if (largest > 1e18f) { const float shrink = 1e18f / largest; cov_xx *= shrink; cov_xy *= shrink; cov_yy *= shrink; }
  cov_xx += 0.3f; cov_yy += 0.3f;
  // 5. opacity, conic, centre, cut-off radius
  r.sig = 1.f / (1.f + expf(-po.w));
  r.opac = r.sig * r.comp_floor;
  if (!(isfinite(cov_xx) && isfinite(cov_xy) && isfinite(cov_yy))) return false;
  const float cov_det = cov_xx * cov_yy - cov_xy * cov_xy;
  if (!(cov_det > 0.f)) return false;
  const float cov_det_inv = 1.f / cov_det;
  r.c00 = cov_yy * cov_det_inv; r.c01 = -cov_xy * cov_det_inv; r.c11 = cov_xx * cov_det_inv;
  r.mx = cam.fx * ray_x + cam.cx; r.my = cam.fy * ray_y + cam.cy;
  if (!(r.opac >= ALPHA_CUTOFF)) return false;
  r.power = logf(r.opac * 255.f);
  return r.c00 * r.c11 - r.c01 * r.c01 > 0.f;
}

#endif  // __CUDACC__

}  // namespace b2k
