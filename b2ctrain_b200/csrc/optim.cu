// Projection backward (screen-space gradient lanes -> parameter gradients) and sparse Adam with the Adam-mini SH
// second moment. Reference semantics: optim_kernel (src/gpu/optim.cu:100-378), adam4 (optim.cu:90-97).
//
// Three kernels share the device functions below:
//   optim_fused_kernel  the reference's single-view step: gradient and update in one pass over the splats
//   proj_bwd_kernel     gradient half only, ADDED into a dense [n][11+3K] accumulator (several views, then an
//                       all-reduce across GPUs)
//   adam_kernel         update half only, from that accumulator
// All are HBM-bound streams over the model: one thread per splat, 128-bit loads of the float4 parameter and moment
// groups, planar (coalesced) SH lanes.
#include "common.cuh"
#include "dp.cuh"
#include "sh.cuh"
#include <type_traits>

namespace b2k {
namespace {

constexpr int OPT_BLOCK = 128;

struct ParamGrad { float3 pos; float op; float4 q; float3 ls; };

// Matrix form of the chain: T = J Rv M with M = Rq diag(s); cov = T T^T + blur; conic = cov^-1.
__device__ __forceinline__ void geometry_backward(const float* g, const Proj& pr, const CamDev& cam, const float4 qv, const float4 lsv, ParamGrad& o) {
  const float* Rv = cam.R;
  // conic -> covariance: dL/dcov = -X G X, G the symmetric gradient of the conic (off-diagonal lane halved).
  const float G00 = g[2], G01 = 0.5f * g[3], G11 = g[4];
  const float X00 = pr.c00, X01 = pr.c01, X11 = pr.c11;
  const float a00 = X00 * G00 + X01 * G01, a01 = X00 * G01 + X01 * G11, a10 = X01 * G00 + X11 * G01, a11 = X01 * G01 + X11 * G11;
  const float v00 = -(a00 * X00 + a01 * X01), v01 = -(a00 * X01 + a01 * X11), v11 = -(a10 * X01 + a11 * X11);
  float M[9], RvM[9];
#pragma unroll
  for (int r = 0; r < 3; r++) { M[r * 3] = pr.Rq[r * 3] * pr.s.x; M[r * 3 + 1] = pr.Rq[r * 3 + 1] * pr.s.y; M[r * 3 + 2] = pr.Rq[r * 3 + 2] * pr.s.z; }
#pragma unroll
  for (int r = 0; r < 3; r++)
#pragma unroll
    for (int c = 0; c < 3; c++) RvM[r * 3 + c] = Rv[r * 3] * M[c] + Rv[r * 3 + 1] * M[3 + c] + Rv[r * 3 + 2] * M[6 + c];
  float T[6], vT[6];
#pragma unroll
  for (int c = 0; c < 3; c++) { T[c] = pr.dx * RvM[c] + pr.J02 * RvM[6 + c]; T[3 + c] = pr.dy * RvM[3 + c] + pr.J12 * RvM[6 + c]; }
#pragma unroll
  for (int c = 0; c < 3; c++) { vT[c] = 2.f * (v00 * T[c] + v01 * T[3 + c]); vT[3 + c] = 2.f * (v01 * T[c] + v11 * T[3 + c]); }
  // dL/dJ = vT (Rv M)^T: only J00, J11, J02, J12 are live.
  const float vJ00 = vT[0] * RvM[0] + vT[1] * RvM[1] + vT[2] * RvM[2];
  const float vJ02 = vT[0] * RvM[6] + vT[1] * RvM[7] + vT[2] * RvM[8];
  const float vJ11 = vT[3] * RvM[3] + vT[4] * RvM[4] + vT[5] * RvM[5];
  const float vJ12 = vT[3] * RvM[6] + vT[4] * RvM[7] + vT[5] * RvM[8];
  // dL/dM = (J Rv)^T vT.
  float JR[6], vM[9];
#pragma unroll
  for (int c = 0; c < 3; c++) { JR[c] = pr.dx * Rv[c] + pr.J02 * Rv[6 + c]; JR[3 + c] = pr.dy * Rv[3 + c] + pr.J12 * Rv[6 + c]; }
#pragma unroll
  for (int r = 0; r < 3; r++)
#pragma unroll
    for (int c = 0; c < 3; c++) vM[r * 3 + c] = JR[r] * vT[c] + JR[3 + r] * vT[3 + c];
  // Camera-space mean through the pinhole and the clamped Jacobian (optim.cu:186-202).
  const float x = pr.mean_c.x, y = pr.mean_c.y, z = pr.mean_c.z;
  const float iz = 1.f / z, iz2 = iz * iz, iz3 = iz2 * iz;
  const float cxr = fminf(fmaxf(x * iz, cam.lim_neg_x), cam.lim_pos_x), cyr = fminf(fmaxf(y * iz, cam.lim_neg_y), cam.lim_pos_y);
  const float v2x = g[0], v2y = g[1];
  const float vmx = cam.fx * iz * v2x + (pr.clamp_x ? 0.f : -cam.fx * iz2 * vJ02);
  const float vmy = cam.fy * iz * v2y + (pr.clamp_y ? 0.f : -cam.fy * iz2 * vJ12);
  const float vmz = -(cam.fx * x * v2x + cam.fy * y * v2y) * iz2 - cam.fx * iz2 * vJ00 - cam.fy * iz2 * vJ11
                    + (pr.clamp_x ? cam.fx * cxr * iz2 : 2.f * cam.fx * x * iz3) * vJ02
                    + (pr.clamp_y ? cam.fy * cyr * iz2 : 2.f * cam.fy * y * iz3) * vJ12;
  o.pos.x += Rv[0] * vmx + Rv[3] * vmy + Rv[6] * vmz;
  o.pos.y += Rv[1] * vmx + Rv[4] * vmy + Rv[7] * vmz;
  o.pos.z += Rv[2] * vmx + Rv[5] * vmy + Rv[8] * vmz;
  // Scales through s_eff = sqrt(exp(2l) + f^2) and the floor's opacity compensation (optim.cu:219-225).
  const float f2 = lsv.w * lsv.w, v_alpha = g[8];
  const float vs0 = pr.Rq[0] * vM[0] + pr.Rq[3] * vM[3] + pr.Rq[6] * vM[6];
  const float vs1 = pr.Rq[1] * vM[1] + pr.Rq[4] * vM[4] + pr.Rq[7] * vM[7];
  const float vs2 = pr.Rq[2] * vM[2] + pr.Rq[5] * vM[5] + pr.Rq[8] * vM[8];
  o.ls.x = vs0 * pr.s2_raw.x / pr.s.x + v_alpha * pr.opac * f2 / (pr.s2_raw.x + f2);
  o.ls.y = vs1 * pr.s2_raw.y / pr.s.y + v_alpha * pr.opac * f2 / (pr.s2_raw.y + f2);
  o.ls.z = vs2 * pr.s2_raw.z / pr.s.z + v_alpha * pr.opac * f2 / (pr.s2_raw.z + f2);
  // Rotation: dL/dRq = vM diag(s), through R(q / |q|).
  float V[9];
#pragma unroll
  for (int r = 0; r < 3; r++) { V[r * 3] = vM[r * 3] * pr.s.x; V[r * 3 + 1] = vM[r * 3 + 1] * pr.s.y; V[r * 3 + 2] = vM[r * 3 + 2] * pr.s.z; }
  const float ql2 = qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w;
  const float iql = 1.f / sqrtf(ql2);
  const float qw = qv.x * iql, qx = qv.y * iql, qy = qv.z * iql, qz = qv.w * iql;
  const float gw = 2.f * (-qz * V[1] + qy * V[2] + qz * V[3] - qx * V[5] - qy * V[6] + qx * V[7]);
  const float gx = 2.f * (qy * V[1] + qz * V[2] + qy * V[3] - 2.f * qx * V[4] - qw * V[5] + qz * V[6] + qw * V[7] - 2.f * qx * V[8]);
  const float gy = 2.f * (-2.f * qy * V[0] + qx * V[1] + qw * V[2] + qx * V[3] + qz * V[5] - qw * V[6] + qz * V[7] - 2.f * qy * V[8]);
  const float gz = 2.f * (-2.f * qz * V[0] - qw * V[1] + qx * V[2] + qw * V[3] - 2.f * qz * V[4] + qy * V[5] + qx * V[6] + qy * V[7]);
  const float gd = gw * qw + gx * qx + gy * qy + gz * qz;
  o.q = make_float4((gw - qw * gd) * iql, (gx - qx * gd) * iql, (gy - qy * gd) * iql, (gz - qz * gd) * iql);
}

struct SplatGrad {
  bool any;        // the splat has a usable gradient this view
  bool visible;
  ParamGrad pg;
  float3 vc;       // dL/dcolour
  float refine;    // growth statistic lane
};

// Reads and clears the splat's screen-space lanes, updates the refine statistics, and derives the parameter
// gradients. basis[] receives the SH basis (zero above the active degree, and all zero when there is no gradient).
template <int DEG>
__device__ __forceinline__ void splat_gradient(int i, size_t cap, const float4* __restrict__ pos_op, const float4* __restrict__ quat, const float4* __restrict__ lscale,
                                               const float* __restrict__ sh_dc, const float* __restrict__ sh_hi, float* __restrict__ v_splat,
                                               uint32_t* __restrict__ vis_flag, const uint32_t* __restrict__ tile_count, float* __restrict__ refine_norm,
                                               float* __restrict__ vis_count, const CamDev& cam, int active, const float4* pos_ov, const float4* quat_ov,
                                               const float4* ls_ov, SplatGrad& sg, float* basis) {
  constexpr int K = (DEG + 1) * (DEG + 1);
  float g[GRAD_LANES];
  const uint32_t vis = vis_flag[i];
  float* vs = v_splat + (size_t)i * GRAD_LANES;
  if (vis) {
#pragma unroll
    for (int k = 0; k < GRAD_LANES; k++) g[k] = vs[k];
  } else {
#pragma unroll
    for (int k = 0; k < GRAD_LANES; k++) g[k] = 0.f;
  }
  sg.visible = vis != 0u && tile_count[i] != 0u;
  if (vis_count && sg.visible) atomicAdd(vis_count + i, 1.f);   // statistics may be updated by views running on other streams
  sg.refine = isfinite(g[9]) ? fminf(fmaxf(g[9], 0.f), 1e32f) : 0.f;
  if (refine_norm && sg.refine > 0.f) atomic_max_nonneg(refine_norm + i, sg.refine);
  bool any = false, finite = true;
#pragma unroll
  for (int k = 0; k < GRAD_LANES; k++) { if (k != 9 && g[k] != 0.f) any = true; finite = finite && isfinite(g[k]); }
  if (vis) {   // cleared only once the loads have landed: a store issued right behind the load of its own line stalls both
    vis_flag[i] = 0u;
#pragma unroll
    for (int k = 0; k < GRAD_LANES; k++) vs[k] = 0.f;
  }
  sg.any = any && sg.visible && finite;
  sg.pg.pos = make_float3(0.f, 0.f, 0.f); sg.pg.op = 0.f; sg.pg.q = make_float4(0.f, 0.f, 0.f, 0.f); sg.pg.ls = make_float3(0.f, 0.f, 0.f);
  sg.vc = make_float3(0.f, 0.f, 0.f);
#pragma unroll
  for (int k = 0; k < K; k++) basis[k] = 0.f;
  if (!sg.any) return;
  const float4 pv = pos_ov ? pos_ov[i] : pos_op[i];
  const float4 qv = quat_ov ? quat_ov[i] : quat[i];
  const float4 lsv = ls_ov ? ls_ov[i] : lscale[i];
  Proj pr;
  if (!project_one(pv, qv, lsv, cam, pr)) return;
  // SH: colour gradient onto the coefficients (outer product with the basis) and onto the view direction.
  float3 u = make_float3(pv.x - cam.pos[0], pv.y - cam.pos[1], pv.z - cam.pos[2]);
  const float ul = sqrtf(u.x * u.x + u.y * u.y + u.z * u.z), iul = 1.f / ul;
  const float3 v = make_float3(u.x * iul, u.y * iul, u.z * iul);
  sh_basis<DEG>(v, active, basis);
  sg.vc = make_float3(g[5], g[6], g[7]);
  float w[K];
  w[0] = 0.f;
  const int kact = (active + 1) * (active + 1);
#pragma unroll
  for (int k = 1; k < K; k++) {
    w[k] = 0.f;
    if (k < kact) {
      const size_t o = (size_t)((k - 1) * 3) * cap + i;
      w[k] = sh_hi[o] * sg.vc.x + sh_hi[o + cap] * sg.vc.y + sh_hi[o + 2 * cap] * sg.vc.z;
    }
  }
  const float3 v_v = sh_dir_grad<DEG>(v, w);
  const float vdot = v.x * v_v.x + v.y * v_v.y + v.z * v_v.z;
  sg.pg.pos = make_float3((v_v.x - v.x * vdot) * iul, (v_v.y - v.y * vdot) * iul, (v_v.z - v.z * vdot) * iul);
  sg.pg.op = g[8] * pr.comp_floor * pr.sig * (1.f - pr.sig);
  geometry_backward(g, pr, cam, qv, lsv, sg.pg);
  const ParamGrad& p = sg.pg;
  const bool ok = isfinite(p.pos.x) && isfinite(p.pos.y) && isfinite(p.pos.z) && isfinite(p.op) && isfinite(p.ls.x) && isfinite(p.ls.y) && isfinite(p.ls.z) &&
                  isfinite(p.q.x + p.q.y + p.q.z + p.q.w);
  if (!ok) { sg.pg.pos = make_float3(0.f, 0.f, 0.f); sg.pg.op = 0.f; sg.pg.q = make_float4(0.f, 0.f, 0.f, 0.f); sg.pg.ls = make_float3(0.f, 0.f, 0.f); }
  (void)sh_dc;
}

// ---- Adam ----
struct AdamConsts { float b1, b2, eps, bc1, bc2, d1, d2, drift; bool catch_up; };

__device__ __forceinline__ AdamConsts adam_consts(const B2kOptim& op, float skipped) {
  AdamConsts a;
  a.b1 = op.beta1; a.b2 = op.beta2; a.eps = op.eps;
  a.bc1 = 1.f / (1.f - powf(op.beta1, (float)op.t)); a.bc2 = 1.f / (1.f - powf(op.beta2, (float)op.t));
  a.d1 = 1.f; a.d2 = 1.f; a.drift = 0.f; a.catch_up = skipped > 0.f;
  if (a.catch_up) {   // closed form of the zero-gradient steps a lazily updated splat missed (optim.cu:299-313)
    a.d1 = powf(op.beta1, skipped); a.d2 = powf(op.beta2, skipped);
    const float r = op.beta1 / sqrtf(op.beta2);
    a.drift = r * (1.f - powf(r, skipped)) / (1.f - r);
  }
  return a;
}
__device__ __forceinline__ void adam1(float& p, float& m, float& v, float g, float lr, const AdamConsts& a) {
  if (a.catch_up) { p -= lr * a.drift * (m * a.bc1) / (sqrtf(v * a.bc2) + a.eps); m *= a.d1; v *= a.d2; }
  m = a.b1 * m + (1.f - a.b1) * g;
  v = a.b2 * v + (1.f - a.b2) * g * g;
  p -= lr * (m * a.bc1) / (sqrtf(v * a.bc2) + a.eps);
}
__device__ __forceinline__ void adam4(float4& p, float4& m, float4& v, float4 g, float4 lr, const AdamConsts& a) {
  adam1(p.x, m.x, v.x, g.x, lr.x, a); adam1(p.y, m.y, v.y, g.y, lr.y, a); adam1(p.z, m.z, v.z, g.z, lr.z, a); adam1(p.w, m.w, v.w, g.w, lr.w, a);
}

// Random draws of the per-step noise. They must be the reference's, value for value, so that a seeded run makes the same
// perturbations (src/gpu/util.cuh:103-116): the lowbias32 mixer chained over three counters, the top 24 bits as a
// uniform in [0, 1), and a Box-Muller normal from two such uniforms (the second with the last counter moved on).
__device__ __forceinline__ uint32_t lowbias32(uint32_t v) {
  v ^= v >> 16;
  v *= 0x7feb352dU;
  v ^= v >> 15;
  v *= 0x846ca68bU;
  v ^= v >> 16;
  return v;
}
__device__ __forceinline__ float unit_draw(uint32_t key, uint32_t item, uint32_t lane) {
  const uint32_t inner = lowbias32(lane * 0xC2B2AE3DU);
  const uint32_t middle = lowbias32(item * 0x85EBCA77U ^ inner);
  const uint32_t bits = lowbias32(key * 0x9E3779B1U ^ middle);
  return (float)(bits >> 8) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ float normal_draw(uint32_t key, uint32_t item, uint32_t lane) {
  const float radius_u = fmaxf(unit_draw(key, item, lane), 1e-7f);
  const float angle_u = unit_draw(key, item, lane + 0x1234567U);
  return sqrtf(-2.f * __logf(radius_u)) * __cosf(6.28318530718f * angle_u);
}

struct ModelPtrs {
  float4 *pos_op, *quat, *lscale, *m_pos, *v_pos, *m_q, *v_q, *m_ls, *v_ls;
  float *sh_dc, *sh_hi, *m_sh_dc, *m_sh_hi, *v_sh;
  uint32_t* last_step;
  size_t cap;
};

// MCMC noise on the mean of a splat some view saw: a clamped normal step per axis whose size falls with the 150th power
// of (1 - effective opacity), so only near-transparent splats wander (src/gpu/optim.cu:363-376). ls holds the updated
// log scales and the 3D-filter floor, po.w the updated opacity logit.
__device__ __forceinline__ void add_mcmc_noise(float4& po, const float4& ls, int i, const B2kOptim& op, bool visible) {
  if (!visible || !(op.noise_weight > 0.f)) return;
  const float floor_sq = ls.w * ls.w;
  const float3 var = make_float3(__expf(2.f * ls.x), __expf(2.f * ls.y), __expf(2.f * ls.z));
  float floor_comp = 1.f;
  if (ls.w > 0.f) floor_comp = sqrtf((var.x * var.y * var.z) / ((var.x + floor_sq) * (var.y + floor_sq) * (var.z + floor_sq)));
  const float logistic = 1.f / (1.f + __expf(-po.w));
  const float opacity = fminf(fmaxf(logistic * floor_comp, 0.f), 1.f);
  const float size = fminf(fmaxf(powf(1.f - opacity, 150.f), 0.f), 1.f) * op.noise_weight;
  if (!(size > 0.f)) return;
  const uint32_t key = op.seed ^ (op.step * 0x9E3779B9u);
  float* axis = &po.x;
#pragma unroll
  for (uint32_t k = 0; k < 3u; k++) axis[k] += fminf(fmaxf(normal_draw(key, (uint32_t)i, k) * size, -op.noise_clamp), op.noise_clamp);
}

// What the SH lanes of a splat need from its per-splat part of the update.
struct ShStep { float denom, denom_old, d1; bool catch_up; };

__device__ __forceinline__ void adam_sh_lane(float& p, float& m, float g, float lrk, float b1, const ShStep& st) {
  if (st.catch_up) { p -= lrk * st.denom_old * m; m *= st.d1; }
  m = b1 * m + (1.f - b1) * g;
  p -= lrk * st.denom * m;
}

// Everything of one splat's update except its SH lanes: lazy catch-up bookkeeping, means / opacity / rotation / scale,
// the Adam-mini second moment of the SH block (gsq is the mean squared SH gradient), MCMC noise.
__device__ __forceinline__ ShStep adam_geometry(int i, const ModelPtrs& mp, const B2kOptim& op, const ParamGrad& pg, float gsq, bool visible) {
  float skipped = 0.f;
  if (op.sparse) {
    const uint32_t ls = mp.last_step[i];
    skipped = ls == 0u ? 0.f : fmaxf((float)op.t - (float)ls - 1.f, 0.f);
    mp.last_step[i] = (uint32_t)op.t;
  }
  const AdamConsts a = adam_consts(op, skipped);
  // All records are loaded before the first store: the arrays may alias as far as the compiler knows, so a
  // load-update-store sequence per record would run one memory round trip each.
  float4 po = mp.pos_op[i], q = mp.quat[i], ls = mp.lscale[i];
  float4 m_po = mp.m_pos[i], v_po = mp.v_pos[i], m_q = mp.m_q[i], v_q = mp.v_q[i], m_l = mp.m_ls[i], v_l = mp.v_ls[i];
  const float v_sh_in = mp.v_sh[i];
  adam4(po, m_po, v_po, make_float4(pg.pos.x, pg.pos.y, pg.pos.z, pg.op), make_float4(op.lr_mean, op.lr_mean, op.lr_mean, op.lr_opac), a);
  adam4(q, m_q, v_q, pg.q, make_float4(op.lr_rot, op.lr_rot, op.lr_rot, op.lr_rot), a);
  {
    const float keep = ls.w;
    adam4(ls, m_l, v_l, make_float4(pg.ls.x, pg.ls.y, pg.ls.z, 0.f), make_float4(op.lr_scale, op.lr_scale, op.lr_scale, 0.f), a);
    ls.w = keep; m_l.w = 0.f; v_l.w = 0.f;   // the floor lane is a frozen constant
  }
  mp.m_pos[i] = m_po; mp.v_pos[i] = v_po;
  mp.m_q[i] = m_q; mp.v_q[i] = v_q; mp.quat[i] = q;
  mp.m_ls[i] = m_l; mp.v_ls[i] = v_l; mp.lscale[i] = ls;
  // Adam-mini: one second moment per splat, the EMA of the mean squared SH gradient (optim.cu:337-345).
  ShStep st;
  const float v_old = v_sh_in * a.d2;
  st.catch_up = a.catch_up; st.d1 = a.d1;
  st.denom_old = a.catch_up ? a.drift * a.bc1 / (sqrtf(v_old * a.bc2) + a.eps) : 0.f;
  const float v = a.b2 * v_old + (1.f - a.b2) * gsq;
  mp.v_sh[i] = v;
  st.denom = a.bc1 / (sqrtf(v * a.bc2) + a.eps);
  add_mcmc_noise(po, ls, i, op, visible);
  mp.pos_op[i] = po;
  return st;
}

__device__ __forceinline__ float* sh_lane_ptr(float* dc, float* hi, size_t cap, int l, int i) {
  return l < 3 ? dc + (size_t)l * cap + i : hi + (size_t)(l - 3) * cap + i;
}

// Update of one splat by one thread. g_sh(k, ch) yields the SH gradient lane.
template <int DEG, class ShGrad>
__device__ __forceinline__ void adam_update(int i, const ModelPtrs& mp, const B2kOptim& op, const ParamGrad& pg, float gsq, ShGrad g_sh, bool visible) {
  constexpr int K = (DEG + 1) * (DEG + 1);
  const ShStep st = adam_geometry(i, mp, op, pg, gsq, visible);
  constexpr int GROUP = 12;   // lanes whose loads are issued together before the group's stores
#pragma unroll
  for (int l0 = 0; l0 < K * 3; l0 += GROUP) {
    float m_in[GROUP], p_in[GROUP];
#pragma unroll
    for (int u = 0; u < GROUP; u++) {
      const int l = l0 + u;
      if (l < K * 3) { m_in[u] = *sh_lane_ptr(mp.m_sh_dc, mp.m_sh_hi, mp.cap, l, i); p_in[u] = *sh_lane_ptr(mp.sh_dc, mp.sh_hi, mp.cap, l, i); }
    }
#pragma unroll
    for (int u = 0; u < GROUP; u++) {
      const int l = l0 + u;
      if (l < K * 3) {
        adam_sh_lane(p_in[u], m_in[u], g_sh(l / 3, l % 3), l < 3 ? op.lr_dc : op.lr_sh_rest, op.beta1, st);
        *sh_lane_ptr(mp.m_sh_dc, mp.m_sh_hi, mp.cap, l, i) = m_in[u];
        *sh_lane_ptr(mp.sh_dc, mp.sh_hi, mp.cap, l, i) = p_in[u];
      }
    }
  }
}

template <int DEG>
__global__ void __launch_bounds__(OPT_BLOCK) optim_fused_kernel(int n, ModelPtrs mp, float* __restrict__ v_splat, uint32_t* __restrict__ vis_flag,
                                                                const uint32_t* __restrict__ tile_count, float* __restrict__ refine_norm,
                                                                float* __restrict__ vis_count, CamDev cam, B2kOptim op,
                                                                const uint32_t* __restrict__ vis_list, const uint32_t* __restrict__ vis_list_count,
                                                                const uint32_t* __restrict__ isect_total, uint32_t isect_cap) {
  constexpr int K = (DEG + 1) * (DEG + 1);
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (vis_list) { if ((uint32_t)i >= *vis_list_count) return; i = (int)vis_list[i]; }   // sparse walk over the splats the backward touched
  if (i >= n) return;
  SplatGrad sg; float basis[K];
  const int active = op.active_sh_degree < DEG ? (op.active_sh_degree < 0 ? 0 : op.active_sh_degree) : DEG;
  splat_gradient<DEG>(i, mp.cap, mp.pos_op, mp.quat, mp.lscale, mp.sh_dc, mp.sh_hi, v_splat, vis_flag, tile_count, refine_norm, vis_count, cam, active,
                      (const float4*)op.pos_override, (const float4*)op.quat_override, (const float4*)op.lscale_override, sg, basis);
  // A view whose intersections did not fit its buffers was composited from truncated lists: its lanes are consumed
  // (cleared above) but nothing is written from them; the host reads the total later, grows the buffers and redoes it.
  if (isect_total && *isect_total > isect_cap) return;
  if (op.grad_out) {
    if (op.sparse && !sg.any) return;
    float* o = op.grad_out + (size_t)i * (11 + K * 3);
    o[0] = sg.pg.pos.x; o[1] = sg.pg.pos.y; o[2] = sg.pg.pos.z; o[3] = sg.pg.op;
    o[4] = sg.pg.q.x; o[5] = sg.pg.q.y; o[6] = sg.pg.q.z; o[7] = sg.pg.q.w; o[8] = sg.pg.ls.x; o[9] = sg.pg.ls.y; o[10] = sg.pg.ls.z;
#pragma unroll
    for (int k = 0; k < K; k++) { o[11 + k * 3] = basis[k] * sg.vc.x; o[12 + k * 3] = basis[k] * sg.vc.y; o[13 + k * 3] = basis[k] * sg.vc.z; }
    return;
  }
  if (op.sparse && !sg.any) return;
  float bsq = 0.f;
#pragma unroll
  for (int k = 0; k < K; k++) bsq += basis[k] * basis[k];
  const float gsq = bsq * (sg.vc.x * sg.vc.x + sg.vc.y * sg.vc.y + sg.vc.z * sg.vc.z) * (1.f / (float)(K * 3));
  const float3 vc = sg.vc;
  adam_update<DEG>(i, mp, op, sg.pg, gsq, [&](int k, int ch) { return basis[k] * (ch == 0 ? vc.x : (ch == 1 ? vc.y : vc.z)); }, sg.visible);
}

template <int DEG>
__global__ void __launch_bounds__(OPT_BLOCK) proj_bwd_kernel(int n, ModelPtrs mp, float* __restrict__ v_splat, uint32_t* __restrict__ vis_flag,
                                                             const uint32_t* __restrict__ tile_count, float* __restrict__ refine_norm,
                                                             float* __restrict__ vis_count, CamDev cam, B2kOptim op, float* __restrict__ grad,
                                                             const uint32_t* __restrict__ vis_list, const uint32_t* __restrict__ vis_list_count,
                                                             const uint32_t* __restrict__ isect_total, uint32_t isect_cap) {
  constexpr int K = (DEG + 1) * (DEG + 1);
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (vis_list) { if ((uint32_t)i >= *vis_list_count) return; i = (int)vis_list[i]; }
  if (i >= n) return;
  SplatGrad sg; float basis[K];
  const int active = op.active_sh_degree < DEG ? (op.active_sh_degree < 0 ? 0 : op.active_sh_degree) : DEG;
  splat_gradient<DEG>(i, mp.cap, mp.pos_op, mp.quat, mp.lscale, mp.sh_dc, mp.sh_hi, v_splat, vis_flag, tile_count, refine_norm, vis_count, cam, active,
                      (const float4*)op.pos_override, (const float4*)op.quat_override, (const float4*)op.lscale_override, sg, basis);
  if (!sg.any || (isect_total && *isect_total > isect_cap)) return;   // an overflowed view adds nothing (see optim_fused_kernel)
  if (op.touched_out) atomicOr(op.touched_out + (i >> 5), 1u << (i & 31));
  // Several views of a step may be in flight on different streams and add into the same accumulator: reductions
  // (fire-and-forget RED.ADD at the L2), not read-modify-write.
  float* o = grad + (size_t)i * (11 + K * 3);
  atomicAdd(o + 0, sg.pg.pos.x); atomicAdd(o + 1, sg.pg.pos.y); atomicAdd(o + 2, sg.pg.pos.z); atomicAdd(o + 3, sg.pg.op);
  atomicAdd(o + 4, sg.pg.q.x); atomicAdd(o + 5, sg.pg.q.y); atomicAdd(o + 6, sg.pg.q.z); atomicAdd(o + 7, sg.pg.q.w);
  atomicAdd(o + 8, sg.pg.ls.x); atomicAdd(o + 9, sg.pg.ls.y); atomicAdd(o + 10, sg.pg.ls.z);
#pragma unroll
  for (int k = 0; k < K; k++) {
    const float bk = basis[k];
    if (bk != 0.f) { atomicAdd(o + 11 + k * 3, bk * sg.vc.x); atomicAdd(o + 12 + k * 3, bk * sg.vc.y); atomicAdd(o + 13 + k * 3, bk * sg.vc.z); }
  }
}

// The update half of the data-parallel split. The accumulator is row-major [n][PER] (the all-reduce buffer); parameters
// and moments are float4 records per splat plus planar SH lanes. One thread per splat is a long latency-bound chain
// (a hundred loads, a dozen square roots and divisions) with too few warps to hide it: it measured under a third of
// the copy bandwidth. Here FOUR threads share a splat, and a CTA takes 128 splats (64 at SH degree 4):
//   1. all warps stage the accumulator rows through shared memory (coalesced 16-byte loads issued together) and clear
//      them;
//   2. the four threads of a splat each reduce a quarter of its row (touched? sum of squared SH gradients);
//   3. role 0 updates mean + opacity, role 1 the rotation, role 2 the scales, role 3 the Adam-mini second moment of
//      the SH block, whose step size it publishes; every role has already issued the loads of its quarter of the SH
//      lanes (lane l belongs to role l mod 4; a warp holds one role of 32 consecutive splats, so every access is a
//      coalesced 128- or 512-byte run);
//   4. the SH lanes are updated; role 0 adds the MCMC noise (it needs role 2's scales) and stores the mean; role 3
//      stamps last_step, which all four read in step 3.
#ifndef B2K_ADAM_SPLATS
#define B2K_ADAM_SPLATS 128
#endif
#ifndef B2K_ADAM_SHARD_SPLATS
#define B2K_ADAM_SHARD_SPLATS 128
#endif
template <int DEG, bool SHARD = false> struct AdamShape {
  static constexpr int SPLATS = DEG <= 3 ? (SHARD ? B2K_ADAM_SHARD_SPLATS : B2K_ADAM_SPLATS) : 64, THREADS = 4 * SPLATS;
};

// PEERS = NoPeers: the update of this GPU's replica from its own accumulator (rows cleared on the way).
// PEERS = PeerArgs: the sharded data-parallel update (b2k_dp_adam_shard). The rows of this rank's slice are summed from
// every rank's accumulator with peer loads (a reduce-scatter done by the consumer), the update runs once, here, and the
// new parameters are stored into every rank's replica (an all-gather done by the producer); moments stay with the
// owner. Accumulators are left as they are: each rank clears its own afterwards.
struct NoPeers {};
struct PeerArgs {
  int world;
  const float* grad[B2K_DP_MAX_RANKS];
  float4* pos_op[B2K_DP_MAX_RANKS]; float4* quat[B2K_DP_MAX_RANKS]; float4* lscale[B2K_DP_MAX_RANKS];
  float* sh_dc[B2K_DP_MAX_RANKS]; float* sh_hi[B2K_DP_MAX_RANKS];
  const uint32_t* touched[B2K_DP_MAX_RANKS];   // per rank: bit i set when its accumulator holds a row for splat i; used when sparse_rows
  int sparse_rows;
};
__device__ __forceinline__ float4 sum4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

template <int DEG, class PEERS>
__global__ void __launch_bounds__(AdamShape<DEG, !std::is_same<PEERS, NoPeers>::value>::THREADS, 1024 / AdamShape<DEG, !std::is_same<PEERS, NoPeers>::value>::THREADS) adam_kernel(int first, int end, ModelPtrs mp, B2kOptim op, float* __restrict__ grad,
                                                                                                       const PEERS peers) {
  constexpr bool SHARD = !std::is_same<PEERS, NoPeers>::value;
  constexpr int SPLATS = AdamShape<DEG, SHARD>::SPLATS, THREADS = AdamShape<DEG, SHARD>::THREADS;
  constexpr int K = (DEG + 1) * (DEG + 1), L = 3 * K, PER = 11 + L, QUARTER = (PER + 3) / 4, LPT = (L + 3) / 4;
  __shared__ __align__(16) float s_rows[SPLATS * PER];
  __shared__ float s_sq[4][SPLATS], s_denom[SPLATS], s_denom_old[SPLATS];
  __shared__ int s_any[4][SPLATS];
  __shared__ float4 s_ls[SPLATS];
  __shared__ uint32_t s_touch[SHARD ? B2K_DP_MAX_RANKS : 1][SPLATS / 32];
  const int base = first + blockIdx.x * SPLATS;   // first is a multiple of four, which keeps the block 16-byte aligned
  const int rows = end - base < SPLATS ? end - base : SPLATS;
  float* gblock = grad + (size_t)base * PER;
  if (rows == SPLATS) {
    constexpr int WORDS = SPLATS * PER / 4, BATCH = (WORDS + THREADS - 1) / THREADS;   // whole 16-byte words from an aligned start
    float4* s4 = reinterpret_cast<float4*>(s_rows);
    float4 r[BATCH];
    if constexpr (SHARD) {
      // Rows a rank never added to are zero: with the ranks' bitmaps at hand they are not fetched at all (a rank that
      // rendered 8 of a step's 64 views touches about a third of the splats).
      constexpr int TW = SPLATS / 32;
      int row0[BATCH], row1[BATCH];
#pragma unroll
      for (int u = 0; u < BATCH; u++) { const int f = (threadIdx.x + u * THREADS) * 4; row0[u] = f / PER; row1[u] = (f + 3) / PER; }
      if (peers.sparse_rows) {
        if ((int)threadIdx.x < peers.world * TW) s_touch[threadIdx.x / TW][threadIdx.x % TW] = peers.touched[threadIdx.x / TW][base / 32 + threadIdx.x % TW];
        __syncthreads();
      }
      auto wanted = [&](int p, int u) {
        if (!peers.sparse_rows) return true;
        const uint32_t b0 = s_touch[p][row0[u] >> 5] >> (row0[u] & 31), b1 = s_touch[p][row1[u] >> 5] >> (row1[u] & 31);
        return ((b0 | b1) & 1u) != 0u;
      };
#pragma unroll
      for (int u = 0; u < BATCH; u++) r[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      // Two ranks' rows per round, so that twice the loads are in flight over the links; the sums are formed in rank
      // order (every rank would form the same ones).
      for (int p = 0; p < peers.world; p += 2) {
        const bool two = p + 1 < peers.world;
        const float4* ga = reinterpret_cast<const float4*>(peers.grad[p] + (size_t)base * PER);
        const float4* gb = reinterpret_cast<const float4*>(peers.grad[two ? p + 1 : p] + (size_t)base * PER);
        float4 ta[BATCH], tb[BATCH];
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
          const int k = threadIdx.x + u * THREADS;
          const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
          if (k < WORDS) { ta[u] = wanted(p, u) ? __ldcs(ga + k) : zero; tb[u] = two && wanted(p + 1, u) ? __ldcs(gb + k) : zero; }
        }
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
          const int k = threadIdx.x + u * THREADS;
          if (k < WORDS) { r[u] = sum4(r[u], ta[u]); if (two) r[u] = sum4(r[u], tb[u]); }
        }
      }
    } else {
      const float4* g4 = reinterpret_cast<const float4*>(gblock);
#pragma unroll
      for (int u = 0; u < BATCH; u++) { const int k = threadIdx.x + u * THREADS; if (k < WORDS) r[u] = __ldcs(g4 + k); }
    }
#pragma unroll
    for (int u = 0; u < BATCH; u++) { const int k = threadIdx.x + u * THREADS; if (k < WORDS) s4[k] = r[u]; }
  } else if constexpr (SHARD) {
    for (int k = threadIdx.x; k < rows * PER; k += THREADS) {
      float t = 0.f;
      for (int p = 0; p < peers.world; p++) t += peers.grad[p][(size_t)base * PER + k];
      s_rows[k] = t;
    }
  } else {
    for (int k = threadIdx.x; k < rows * PER; k += THREADS) { s_rows[k] = gblock[k]; gblock[k] = 0.f; }
  }
  __syncthreads();
  // The rows are cleared only now, once the loads above have landed: a store issued right behind the load of the same
  // line measured 2.5x slower for the whole kernel than one issued after it.
  if (!SHARD && rows == SPLATS) {
    constexpr int WORDS = SPLATS * PER / 4;
    float4* g4 = reinterpret_cast<float4*>(gblock);
    for (int k = threadIdx.x; k < WORDS; k += THREADS) __stcs(g4 + k, make_float4(0.f, 0.f, 0.f, 0.f));
  }

  const int role = threadIdx.x / SPLATS, sp = threadIdx.x % SPLATS, i = base + sp;
  const float* g = s_rows + sp * PER;
  {
    bool any_q = false; float sq_q = 0.f;
    if (sp < rows) {
#pragma unroll
      for (int u = 0; u < QUARTER; u++) {
        const int k = role * QUARTER + u;
        if (k < PER) { const float x = g[k]; any_q = any_q || x != 0.f; if (k >= 11) sq_q += x * x; }
      }
    }
    s_any[role][sp] = any_q; s_sq[role][sp] = sq_q;
  }
  __syncthreads();
  const bool any = (s_any[0][sp] | s_any[1][sp] | s_any[2][sp] | s_any[3][sp]) != 0;
  const bool live = sp < rows && (!op.sparse || any);   // a splat no view touched is skipped whole in sparse mode
  float m_in[LPT], p_in[LPT];
  AdamConsts a;
  float4 po;
  if (live) {
#pragma unroll
    for (int u = 0; u < LPT; u++) {
      const int l = role + 4 * u;
      if (l < L) { m_in[u] = *sh_lane_ptr(mp.m_sh_dc, mp.m_sh_hi, mp.cap, l, i); p_in[u] = *sh_lane_ptr(mp.sh_dc, mp.sh_hi, mp.cap, l, i); }
    }
    float skipped = 0.f;
    if (op.sparse) {
      const uint32_t ls = mp.last_step[i];
      skipped = ls == 0u ? 0.f : fmaxf((float)op.t - (float)ls - 1.f, 0.f);
    }
    a = adam_consts(op, skipped);
    if (role == 0) {
      po = mp.pos_op[i];
      float4 m = mp.m_pos[i], v = mp.v_pos[i];
      adam4(po, m, v, make_float4(g[0], g[1], g[2], g[3]), make_float4(op.lr_mean, op.lr_mean, op.lr_mean, op.lr_opac), a);
      mp.m_pos[i] = m; mp.v_pos[i] = v;
    } else if (role == 1) {
      float4 q = mp.quat[i], m = mp.m_q[i], v = mp.v_q[i];
      adam4(q, m, v, make_float4(g[4], g[5], g[6], g[7]), make_float4(op.lr_rot, op.lr_rot, op.lr_rot, op.lr_rot), a);
      mp.m_q[i] = m; mp.v_q[i] = v;
      if constexpr (SHARD) { for (int p = 0; p < peers.world; p++) peers.quat[p][i] = q; } else mp.quat[i] = q;
    } else if (role == 2) {
      float4 ls = mp.lscale[i], m = mp.m_ls[i], v = mp.v_ls[i];
      const float keep = ls.w;
      adam4(ls, m, v, make_float4(g[8], g[9], g[10], 0.f), make_float4(op.lr_scale, op.lr_scale, op.lr_scale, 0.f), a);
      ls.w = keep; m.w = 0.f; v.w = 0.f;   // the floor lane is a frozen constant
      mp.m_ls[i] = m; mp.v_ls[i] = v;
      if constexpr (SHARD) { for (int p = 0; p < peers.world; p++) peers.lscale[p][i] = ls; } else mp.lscale[i] = ls;
      s_ls[sp] = ls;
    } else {
      // Adam-mini: one second moment per splat, the EMA of the mean squared SH gradient (optim.cu:337-345).
      const float gsq = (s_sq[0][sp] + s_sq[1][sp] + s_sq[2][sp] + s_sq[3][sp]) * (1.f / (float)L);
      const float v_old = mp.v_sh[i] * a.d2;
      s_denom_old[sp] = a.catch_up ? a.drift * a.bc1 / (sqrtf(v_old * a.bc2) + a.eps) : 0.f;
      const float v = a.b2 * v_old + (1.f - a.b2) * gsq;
      mp.v_sh[i] = v;
      s_denom[sp] = a.bc1 / (sqrtf(v * a.bc2) + a.eps);
    }
  }
  __syncthreads();
  if (!live) return;
  ShStep st;
  st.denom = s_denom[sp]; st.denom_old = s_denom_old[sp]; st.d1 = a.d1; st.catch_up = a.catch_up;
#pragma unroll
  for (int u = 0; u < LPT; u++) {
    const int l = role + 4 * u;
    if (l < L) {
      adam_sh_lane(p_in[u], m_in[u], g[11 + l], l < 3 ? op.lr_dc : op.lr_sh_rest, op.beta1, st);
      *sh_lane_ptr(mp.m_sh_dc, mp.m_sh_hi, mp.cap, l, i) = m_in[u];
      if constexpr (SHARD) { for (int p = 0; p < peers.world; p++) *sh_lane_ptr(peers.sh_dc[p], peers.sh_hi[p], mp.cap, l, i) = p_in[u]; }
      else *sh_lane_ptr(mp.sh_dc, mp.sh_hi, mp.cap, l, i) = p_in[u];
    }
  }
  if (role == 0) {
    add_mcmc_noise(po, s_ls[sp], i, op, any);
    if constexpr (SHARD) { for (int p = 0; p < peers.world; p++) peers.pos_op[p][i] = po; } else mp.pos_op[i] = po;
  } else if (role == 3 && op.sparse) {
    mp.last_step[i] = (uint32_t)op.t;
  }
}

// Indices of the splats whose visibility flag the backward set, appended in no particular order (one atomic per warp).
__global__ void __launch_bounds__(256) compact_vis_kernel(int n, const uint32_t* __restrict__ vis_flag, uint32_t* __restrict__ list, uint32_t* __restrict__ count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool on = i < n && vis_flag[i] != 0u;
  const uint32_t m = __ballot_sync(0xffffffffu, on);
  if (m == 0u) return;
  const int lane = threadIdx.x & 31;
  uint32_t base = 0;
  if (lane == 0) base = atomicAdd(count, (uint32_t)__popc(m));
  base = __shfl_sync(0xffffffffu, base, 0);
  if (on) list[base + __popc(m & ((1u << lane) - 1u))] = (uint32_t)i;
}

int build_vis_list(const B2kCtx* c, int n, cudaStream_t s) {
  B2K_CUDA(cudaMemsetAsync(c->num_isect + 1, 0, sizeof(uint32_t), s));
  compact_vis_kernel<<<div_up(n, 256), 256, 0, s>>>(n, c->vis_flag, c->vis_list, c->num_isect + 1);
  return check_launch();
}

ModelPtrs model_ptrs(const B2kModel* m) {
  ModelPtrs p;
  p.pos_op = (float4*)m->pos_op; p.quat = (float4*)m->quat; p.lscale = (float4*)m->lscale;
  p.m_pos = (float4*)m->m_pos_op; p.v_pos = (float4*)m->v_pos_op; p.m_q = (float4*)m->m_quat; p.v_q = (float4*)m->v_quat;
  p.m_ls = (float4*)m->m_lscale; p.v_ls = (float4*)m->v_lscale;
  p.sh_dc = m->sh_dc; p.sh_hi = m->sh_hi; p.m_sh_dc = m->m_sh_dc; p.m_sh_hi = m->m_sh_hi; p.v_sh = m->v_sh; p.last_step = m->last_step; p.cap = (size_t)m->cap;
  return p;
}

bool has_moments(const B2kModel* m) {
  return m->m_pos_op && m->v_pos_op && m->m_quat && m->v_quat && m->m_lscale && m->v_lscale && m->m_sh_dc && m->v_sh && m->last_step && (m->degree == 0 || m->m_sh_hi);
}

__global__ void min_scale_kernel(int n, const float4* __restrict__ pos, float4* __restrict__ ls, const float* __restrict__ cam_pos, const float* __restrict__ cam_focal, int n_cams) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 p = pos[i];
  float best = INFINITY;
  for (int c = 0; c < n_cams; c++) {
    const float dx = p.x - cam_pos[c * 3], dy = p.y - cam_pos[c * 3 + 1], dz = p.z - cam_pos[c * 3 + 2];
    best = fminf(best, sqrtf(dx * dx + dy * dy + dz * dz) / fmaxf(cam_focal[c], 1e-6f));
  }
  float4 l = ls[i]; l.w = sqrtf(0.1f) * best; ls[i] = l;
}

__global__ void pack_rgba8_kernel(int n, const float4* __restrict__ img, uint32_t* __restrict__ out, int alpha_override) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 v = img[i];
  auto q = [](float x) { return (uint32_t)fminf(fmaxf(x * 255.f + 0.5f, 0.f), 255.f); };
  const uint32_t a = alpha_override >= 0 ? (uint32_t)alpha_override : q(v.w);
  const uint32_t r = min(q(v.x), a), g = min(q(v.y), a), b = min(q(v.z), a);
  out[i] = r | (g << 8) | (b << 16) | (a << 24);
}


// ---- Model::compact (src/model.cu:110-155): stable selection of the kept splats, then a gather of every array ----
constexpr int SEL_BLOCK = 1024;

// Kept entries per block of 1024.
__global__ void __launch_bounds__(SEL_BLOCK) select_count_kernel(int n, const uint32_t* __restrict__ keep, uint32_t* __restrict__ block_counts) {
  const int i = blockIdx.x * SEL_BLOCK + threadIdx.x;
  const int c = __syncthreads_count(i < n && keep[i] != 0u);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = (uint32_t)c;
}
// Exclusive scan of the block counts in place (one CTA), total to *count.
__global__ void __launch_bounds__(1024) select_scan_kernel(int blocks, uint32_t* __restrict__ block_counts, uint32_t* __restrict__ count) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0u;
  __syncthreads();
  for (int b0 = 0; b0 < blocks; b0 += 1024) {
    const int b = b0 + threadIdx.x;
    const uint32_t v = b < blocks ? block_counts[b] : 0u;
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t pre = 0;
    for (int w = 0; w < warp; w++) pre += s_warp[w];
    const uint32_t carry = s_carry;
    if (b < blocks) block_counts[b] = carry + pre + incl - v;
    __syncthreads();
    if (threadIdx.x == 1023) s_carry = carry + pre + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) *count = s_carry;
}
// idx[slot] = i for the kept i, in ascending order.
__global__ void __launch_bounds__(SEL_BLOCK) select_write_kernel(int n, const uint32_t* __restrict__ keep, const uint32_t* __restrict__ block_offsets,
                                                                 uint32_t* __restrict__ idx) {
  __shared__ uint32_t s_warp[SEL_BLOCK / 32];
  const int i = blockIdx.x * SEL_BLOCK + threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool on = i < n && keep[i] != 0u;
  const uint32_t m = __ballot_sync(0xffffffffu, on);
  if (lane == 0) s_warp[warp] = (uint32_t)__popc(m);
  __syncthreads();
  uint32_t pre = block_offsets[blockIdx.x];
  for (int w = 0; w < warp; w++) pre += s_warp[w];
  if (on) idx[pre + __popc(m & ((1u << lane) - 1u))] = (uint32_t)i;
}
// dst[l * stride + j] = src[l * stride + idx[j]] for every lane l (gather_kernel, src/model.cu:112-118), elements of
// WORDS 32-bit words.
template <int WORDS>
__global__ void gather_lanes_kernel(int count, int lanes, size_t stride, const uint32_t* __restrict__ idx, const uint32_t* __restrict__ src,
                                    uint32_t* __restrict__ dst) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= count) return;
  const uint32_t i = idx[j];
  for (int l = 0; l < lanes; l++) {
    if constexpr (WORDS == 4) {
      reinterpret_cast<uint4*>(dst)[(size_t)l * stride + j] = reinterpret_cast<const uint4*>(src)[(size_t)l * stride + i];
    } else {
      dst[(size_t)l * stride + j] = src[(size_t)l * stride + i];
    }
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

#define B2K_DISPATCH_DEG(deg, CALL) \
  switch (deg) { case 0: { constexpr int D = 0; CALL; } break; case 1: { constexpr int D = 1; CALL; } break; case 2: { constexpr int D = 2; CALL; } break; \
                 case 3: { constexpr int D = 3; CALL; } break; default: { constexpr int D = 4; CALL; } break; }

static int check_optim_args(const B2kCtx* c, const B2kModel* m, const B2kOptim* op) {
  B2K_REQUIRE(c && m && op && m->n >= 0 && m->cap >= m->n && m->degree >= 0 && m->degree <= 4);
  B2K_REQUIRE(m->pos_op && m->quat && m->lscale && m->sh_dc && (m->degree == 0 || m->sh_hi));
  B2K_REQUIRE(c->v_splat && c->vis_flag && c->tile_count);
  if (c->n_cap < m->n) return B2K_ERR_CAPACITY;
  return B2K_OK;
}

extern "C" int b2k_optim_fused(const B2kCtx* c, const B2kModel* m, const B2kCamera* cam, const B2kOptim* op, b2k_stream_t stream) {
  int st = check_optim_args(c, m, op);
  if (st) return st;
  B2K_REQUIRE(cam);
  if (m->n == 0) return B2K_OK;
  if (!op->grad_out) B2K_REQUIRE(has_moments(m) && op->t >= 1);
  const CamDev cd = to_camdev(*cam);
  const ModelPtrs mp = model_ptrs(m);
  // The list is complete only for what the sparse update needs: splats the backward touched.
  const uint32_t* list = (c->vis_list && c->num_isect && op->sparse && !op->grad_out) ? c->vis_list : nullptr;
  if (list) { st = build_vis_list(c, m->n, (cudaStream_t)stream); if (st) return st; }
  B2K_DISPATCH_DEG(m->degree, (optim_fused_kernel<D><<<div_up(m->n, OPT_BLOCK), OPT_BLOCK, 0, (cudaStream_t)stream>>>(
      m->n, mp, c->v_splat, c->vis_flag, c->tile_count, m->refine_norm, m->vis_count, cd, *op, list, list ? c->num_isect + 1 : nullptr,
      c->num_isect, (uint32_t)c->isect_cap)));
  return check_launch();
}

extern "C" int b2k_proj_bwd(const B2kCtx* c, const B2kModel* m, const B2kCamera* cam, const B2kOptim* op, float* grad, b2k_stream_t stream) {
  int st = check_optim_args(c, m, op);
  if (st) return st;
  B2K_REQUIRE(cam && grad);
  if (m->n == 0) return B2K_OK;
  const CamDev cd = to_camdev(*cam);
  const ModelPtrs mp = model_ptrs(m);
  const uint32_t* list = (c->vis_list && c->num_isect) ? c->vis_list : nullptr;   // the gradient half only ever needs touched splats
  if (list) { st = build_vis_list(c, m->n, (cudaStream_t)stream); if (st) return st; }
  B2K_DISPATCH_DEG(m->degree, (proj_bwd_kernel<D><<<div_up(m->n, OPT_BLOCK), OPT_BLOCK, 0, (cudaStream_t)stream>>>(
      m->n, mp, c->v_splat, c->vis_flag, c->tile_count, m->refine_norm, m->vis_count, cd, *op, grad, list, list ? c->num_isect + 1 : nullptr,
      c->num_isect, (uint32_t)c->isect_cap)));
  return check_launch();
}

extern "C" int b2k_adam_range(const B2kModel* m, const B2kOptim* op, float* grad, int32_t first, int32_t count, b2k_stream_t stream) {
  B2K_REQUIRE(m && op && grad && m->n >= 0 && m->cap >= m->n && m->degree >= 0 && m->degree <= 4);
  B2K_REQUIRE(m->pos_op && m->quat && m->lscale && m->sh_dc && (m->degree == 0 || m->sh_hi) && has_moments(m) && op->t >= 1);
  B2K_REQUIRE(first >= 0 && count >= 0 && first % 4 == 0 && (int64_t)first + count <= m->n);
  if (count == 0) return B2K_OK;
  const ModelPtrs mp = model_ptrs(m);
  B2K_DISPATCH_DEG(m->degree, (adam_kernel<D, NoPeers><<<div_up(count, AdamShape<D>::SPLATS), AdamShape<D>::THREADS, 0, (cudaStream_t)stream>>>(
      first, first + count, mp, *op, grad, NoPeers{})));
  return check_launch();
}

extern "C" int b2k_dp_adam_shard(B2kDp* dp, const B2kModel* m, const B2kOptim* op, const B2kDpPeers* pr, b2k_stream_t stream) {
  B2K_REQUIRE(dp && m && op && pr && m->n >= 0 && m->cap >= m->n && m->degree >= 0 && m->degree <= 4 && dp->world <= B2K_DP_MAX_RANKS);
  B2K_REQUIRE(m->pos_op && m->quat && m->lscale && m->sh_dc && (m->degree == 0 || m->sh_hi) && has_moments(m) && op->t >= 1);
  PeerArgs pa;
  pa.world = dp->world;
  for (int r = 0; r < dp->world; r++) {
    B2K_REQUIRE(pr->grad[r] && pr->pos_op[r] && pr->quat[r] && pr->lscale[r] && pr->sh_dc[r] && (m->degree == 0 || pr->sh_hi[r]));
    pa.grad[r] = pr->grad[r]; pa.pos_op[r] = (float4*)pr->pos_op[r]; pa.quat[r] = (float4*)pr->quat[r]; pa.lscale[r] = (float4*)pr->lscale[r];
    pa.sh_dc[r] = pr->sh_dc[r]; pa.sh_hi[r] = pr->sh_hi[r];
    pa.touched[r] = pr->touched[r];
  }
  pa.sparse_rows = pr->touched[0] != nullptr;
  for (int r = 0; r < dp->world; r++) B2K_REQUIRE((pr->touched[r] != nullptr) == (pa.sparse_rows != 0));   // all ranks' bitmaps or none
  B2K_REQUIRE(pr->pos_op[dp->rank] == m->pos_op && pr->sh_dc[dp->rank] == m->sh_dc);   // the replica named by `m` is this rank's
  int32_t first = 0, count = 0;
  int st = b2k_dp_slice(m->n, dp->rank, dp->world, &first, &count);
  if (st) return st;
  if (count == 0) return B2K_OK;
  const ModelPtrs mp = model_ptrs(m);
  B2K_DISPATCH_DEG(m->degree, (adam_kernel<D, PeerArgs><<<div_up(count, AdamShape<D, true>::SPLATS), AdamShape<D, true>::THREADS, 0, (cudaStream_t)stream>>>(
      first, first + count, mp, *op, pr->grad[dp->rank], pa)));
  return check_launch();
}

extern "C" int b2k_adam(const B2kModel* m, const B2kOptim* op, float* grad, b2k_stream_t stream) {
  B2K_REQUIRE(m && m->n >= 0);
  return b2k_adam_range(m, op, grad, 0, m->n, stream);
}

extern "C" int b2k_min_scale(const B2kModel* m, const float* cam_pos, const float* cam_focal, int32_t n_cams, b2k_stream_t stream) {
  B2K_REQUIRE(m && m->pos_op && m->lscale && cam_pos && cam_focal && n_cams > 0 && m->n >= 0);
  if (m->n == 0) return B2K_OK;
  min_scale_kernel<<<div_up(m->n, 256), 256, 0, (cudaStream_t)stream>>>(m->n, (const float4*)m->pos_op, (float4*)m->lscale, cam_pos, cam_focal, n_cams);
  return check_launch();
}

// The renderer's 8-bit output (src/render/renderer.cpp:353-358 does it on the host after a float download): every channel
// clamped to [0, 1], scaled by 255 and rounded half away from zero, as lround does; no premultiplied clamp.
__global__ void quantize_rgba8_kernel(int n, const float4* __restrict__ img, uint32_t* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 v = img[i];
  auto q = [](float x) {
    const float p = __fmul_rn(fminf(fmaxf(x, 0.f), 1.f), 255.f);   // the product rounded once, then the exact half test
    const float r = truncf(p);
    return (uint32_t)r + (p - r >= 0.5f ? 1u : 0u);
  };
  out[i] = q(v.x) | (q(v.y) << 8) | (q(v.z) << 16) | (q(v.w) << 24);
}

extern "C" int b2k_quantize_rgba8(const float* rgba, uint32_t* out, int32_t n_pixels, b2k_stream_t stream) {
  B2K_REQUIRE(n_pixels >= 0 && (n_pixels == 0 || (rgba && out)));
  if (n_pixels == 0) return B2K_OK;
  quantize_rgba8_kernel<<<div_up(n_pixels, 256), 256, 0, (cudaStream_t)stream>>>(n_pixels, (const float4*)rgba, out);
  return check_launch();
}

extern "C" int b2k_pack_rgba8(const float* rgba, uint32_t* out, int32_t n_pixels, int32_t alpha_override, b2k_stream_t stream) {
  B2K_REQUIRE(rgba && out && n_pixels >= 0 && alpha_override <= 255);
  if (n_pixels == 0) return B2K_OK;
  pack_rgba8_kernel<<<div_up(n_pixels, 256), 256, 0, (cudaStream_t)stream>>>(n_pixels, (const float4*)rgba, out, alpha_override);
  return check_launch();
}

extern "C" uint64_t b2k_select_tmp_words(int32_t n) { return (uint64_t)(n > 0 ? div_up(n, SEL_BLOCK) : 0) + 1u; }

extern "C" int b2k_select_flagged(const uint32_t* keep, int32_t n, uint32_t* idx, uint32_t* count, uint32_t* tmp, b2k_stream_t stream) {
  B2K_REQUIRE(n >= 0 && count && (n == 0 || (keep && idx && tmp)));
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) { B2K_CUDA(cudaMemsetAsync(count, 0, sizeof(uint32_t), s)); return B2K_OK; }
  const int blocks = div_up(n, SEL_BLOCK);
  select_count_kernel<<<blocks, SEL_BLOCK, 0, s>>>(n, keep, tmp);
  select_scan_kernel<<<1, 1024, 0, s>>>(blocks, tmp, count);
  select_write_kernel<<<blocks, SEL_BLOCK, 0, s>>>(n, keep, tmp, idx);
  return check_launch();
}

extern "C" int b2k_gather_lanes(const void* src, void* dst, const uint32_t* idx, int32_t count, int32_t lanes, uint64_t stride, int32_t elem_bytes,
                                b2k_stream_t stream) {
  B2K_REQUIRE(count >= 0 && lanes >= 0 && (elem_bytes == 4 || elem_bytes == 16) && src != dst);
  if (count == 0 || lanes == 0) return B2K_OK;
  B2K_REQUIRE(src && dst && idx && stride >= (uint64_t)count);
  cudaStream_t s = (cudaStream_t)stream;
  if (elem_bytes == 16) gather_lanes_kernel<4><<<div_up(count, 256), 256, 0, s>>>(count, lanes, (size_t)stride, idx, (const uint32_t*)src, (uint32_t*)dst);
  else gather_lanes_kernel<1><<<div_up(count, 256), 256, 0, s>>>(count, lanes, (size_t)stride, idx, (const uint32_t*)src, (uint32_t*)dst);
  return check_launch();
}
