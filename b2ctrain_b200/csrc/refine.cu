// Device steps of the refinement pass that runs between training steps: prune flags, weighted sampling keys
// (Gumbel top-k), the oversized test, the split of a parent into itself and a child, opacity decay, the floor bake and
// the axis keys of the bounds percentiles. Reference semantics: src/gpu/refine.cu:27-164 (kernels) driven by
// RefineState::run (refine.cu:244-342). The host side (b2ctrain_b200/host/refine.cpp) sequences them; sorting and stream
// compaction are this library's own (b2k_sort_pairs_u32, b2k_select_flagged).
//
// Every kernel is one thread per splat over the float4 parameter groups (HBM streams; the pass runs every few hundred
// steps and is not on the per-step path).
#include "common.cuh"

namespace b2k {
namespace {

constexpr float MIN_OPACITY = 1.f / 255.f;

__device__ __forceinline__ float sigmoid_fast(float x) { return 1.f / (1.f + __expf(-x)); }
// Opacity and scales as rendered, i.e. with the 3D-filter floor folded in (splat_math.cuh:232-237).
__device__ __forceinline__ float effective_opacity(float logit, float4 ls) {
  const float sig = sigmoid_fast(logit);
  if (ls.w <= 0.f) return sig;
  const float f2 = ls.w * ls.w, a = __expf(2.f * ls.x), b = __expf(2.f * ls.y), c = __expf(2.f * ls.z);
  return sig * sqrtf((a * b * c) / ((a + f2) * (b + f2) * (c + f2)));
}
__device__ __forceinline__ float3 effective_scale(float4 ls) {
  const float f2 = ls.w * ls.w;
  return make_float3(sqrtf(__expf(2.f * ls.x) + f2), sqrtf(__expf(2.f * ls.y) + f2), sqrtf(__expf(2.f * ls.z) + f2));
}
__device__ __forceinline__ float logit_of(float o, float lo, float hi) { o = fminf(fmaxf(o, lo), hi); return __logf(o / (1.f - o)); }
__device__ __forceinline__ bool finite4(float4 v, bool with_w) { return isfinite(v.x) && isfinite(v.y) && isfinite(v.z) && (!with_w || isfinite(v.w)); }

// Float -> unsigned whose ascending order is the float's ascending order.
__device__ __forceinline__ uint32_t ascending_key(float f) { const uint32_t u = __float_as_uint(f); return u ^ ((u >> 31) ? 0xFFFFFFFFu : 0x80000000u); }

// The counter hash of the reference's per-step draws (src/gpu/util.cuh:103-111): the same seeds select the same splats.
__device__ __forceinline__ uint32_t mix32(uint32_t x) { x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16; return x; }
__device__ __forceinline__ float uniform_of(uint32_t a, uint32_t b, uint32_t c) {
  const uint32_t h = mix32(a * 0x9E3779B1U ^ mix32(b * 0x85EBCA77U ^ mix32(c * 0xC2B2AE3DU)));
  return (float)(h >> 8) * (1.0f / 16777216.0f);
}

__global__ void flags_kernel(int n, size_t cap, int lanes, const float4* __restrict__ pos, const float4* __restrict__ quat, const float4* __restrict__ ls,
                             const float* __restrict__ sh_dc, const float* __restrict__ sh_hi, float3 center, float max_allowed, const float* __restrict__ vis_weight,
                             float cull_weight, uint32_t* __restrict__ keep, uint32_t* __restrict__ dead, uint32_t* __restrict__ culled) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 p = pos[i], q = quat[i], l = ls[i];
  bool bad = !(finite4(p, true) && finite4(q, true) && finite4(l, false));
  for (int k = 0; k < lanes && !bad; k++) bad = !isfinite(k < 3 ? sh_dc[(size_t)k * cap + i] : sh_hi[(size_t)(k - 3) * cap + i]);
  if (!bad) {
    const float o = effective_opacity(p.w, l);
    const float3 s = effective_scale(l);
    bad = o < MIN_OPACITY || s.x > max_allowed || s.y > max_allowed || s.z > max_allowed || fabsf(p.x - center.x) > max_allowed ||
          fabsf(p.y - center.y) > max_allowed || fabsf(p.z - center.z) > max_allowed;
  }
  const bool cull = !bad && cull_weight > 0.f && vis_weight[i] < cull_weight;   // too little rendered mass since the last pass
  bad = bad || cull;
  keep[i] = bad ? 0u : 1u; dead[i] = bad ? 1u : 0u; culled[i] = cull ? 1u : 0u;
}

// Keys of a weighted draw without replacement: log w + Gumbel noise, largest first. mode 0: w = effective opacity of the
// kept, visible splats (relocation targets); mode 1: w = refine_norm of those above the growth threshold. Stored so that
// an ascending unsigned sort yields descending keys; weight 0 (and excluded splats) sort last.
__global__ void sample_keys_kernel(int n, const uint32_t* __restrict__ keep, const uint32_t* __restrict__ excluded, const float4* __restrict__ pos,
                                   const float4* __restrict__ ls, const float* __restrict__ vis_count, const float* __restrict__ refine_norm, int mode, float threshold,
                                   uint32_t seed, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals, uint32_t* __restrict__ above) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const bool usable = keep[i] != 0u && vis_count[i] > 0.f;
  float w = 0.f;
  if (mode == 0) {
    w = usable ? effective_opacity(pos[i].w, ls[i]) : 0.f;
  } else {
    const bool ab = usable && refine_norm[i] > threshold;
    if (above) above[i] = ab ? 1u : 0u;
    w = ab ? refine_norm[i] : 0.f;
  }
  if (excluded && excluded[i]) w = 0.f;
  float key = -INFINITY;
  if (w > 0.f) {
    const float u = fmaxf(uniform_of(seed, (uint32_t)i, (uint32_t)mode + 7u), 1e-12f);
    key = __logf(w) - __logf(-__logf(u));
  }
  keys[i] = ~ascending_key(key);
  vals[i] = (uint32_t)i;
}

__global__ void oversized_kernel(int n, const uint32_t* __restrict__ keep, const uint32_t* __restrict__ excluded, const float* __restrict__ max_screen,
                                 const float* __restrict__ vis_count, float threshold, uint32_t* __restrict__ flags) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) flags[i] = (keep[i] && !excluded[i] && vis_count[i] > 0.f && max_screen[i] > threshold) ? 1u : 0u;
}

__global__ void mark_kernel(int count, const uint32_t* __restrict__ idx, uint32_t* __restrict__ flags) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) flags[idx[i]] = 1u;
}

struct SplitPtrs {
  float4 *pos, *quat, *ls, *m_pos, *v_pos, *m_q, *v_q, *m_ls, *v_ls;
  float *sh_dc, *sh_hi, *m_sh_dc, *m_sh_hi, *v_sh, *refine_norm, *max_screen, *vis_count;
  uint32_t *last_step, *tile_count;
  size_t cap; int lanes;
};

// Parent k splits into itself and a child: both take 1 - (1 - a)^(1/sqrt 2) of the opacity, shrink along the parent's
// axes (most along its longest, and at least to the screen-size cap) and move apart by what the shrink frees; Adam state
// of both starts over. The child's slot is a reused dead slot while those last, then a new one past the end.
__global__ void split_kernel(int count, const uint32_t* __restrict__ parents, const uint32_t* __restrict__ dead_idx, int from_dead, uint32_t append_base,
                             SplitPtrs m, float split_at_screen_size, uint32_t* __restrict__ children) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= count) return;
  const uint32_t p = parents[k], c = k < from_dead ? dead_idx[k] : append_base + (uint32_t)(k - from_dead);
  children[k] = c;
  const float4 po = m.pos[p], q = m.quat[p], l = m.ls[p];
  const float screen = m.max_screen[p];
  const float a = effective_opacity(po.w, l);
  const float logit = logit_of(1.f - powf(1.f - a, 0.70710678f), 1.f / 255.f, 254.f / 255.f);
  const float3 s = effective_scale(l);
  const float3 s2 = make_float3(s.x * s.x, s.y * s.y, s.z * s.z);
  const float longest = fmaxf(s2.x, fmaxf(s2.y, s2.z));
  float shrink = 0.70710678f;
  if (split_at_screen_size > 0.f && screen > 0.f) shrink = fminf(shrink, split_at_screen_size / screen);
  const float3 kk = make_float3(1.f - s2.x / longest * (1.f - shrink), 1.f - s2.y / longest * (1.f - shrink), 1.f - s2.z / longest * (1.f - shrink));
  const float3 local = make_float3(sqrtf(fmaxf(0.f, 1.f - kk.x * kk.x)) * s.x, sqrtf(fmaxf(0.f, 1.f - kk.y * kk.y)) * s.y, sqrtf(fmaxf(0.f, 1.f - kk.z * kk.z)) * s.z);
  const float inv = rsqrtf(fmaxf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w, 1e-32f));
  const float4 qn = make_float4(q.x * inv, q.y * inv, q.z * inv, q.w * inv);
  float R[9];
  quat_to_mat(qn.x, qn.y, qn.z, qn.w, R);
  const float3 off = make_float3(R[0] * local.x + R[1] * local.y + R[2] * local.z, R[3] * local.x + R[4] * local.y + R[5] * local.z,
                                 R[6] * local.x + R[7] * local.y + R[8] * local.z);
  const float4 nl = make_float4(__logf(s.x * kk.x), __logf(s.y * kk.y), __logf(s.z * kk.z), 0.f);   // the floor is re-attached after the pass
  m.pos[p] = make_float4(po.x - off.x, po.y - off.y, po.z - off.z, logit);
  m.pos[c] = make_float4(po.x + off.x, po.y + off.y, po.z + off.z, logit);
  m.quat[p] = qn; m.quat[c] = qn; m.ls[p] = nl; m.ls[c] = nl;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  m.m_pos[p] = z; m.v_pos[p] = z; m.m_q[p] = z; m.v_q[p] = z; m.m_ls[p] = z; m.v_ls[p] = z;
  m.m_pos[c] = z; m.v_pos[c] = z; m.m_q[c] = z; m.v_q[c] = z; m.m_ls[c] = z; m.v_ls[c] = z;
  for (int j = 0; j < m.lanes; j++) {
    float* par = j < 3 ? m.sh_dc + (size_t)j * m.cap : m.sh_hi + (size_t)(j - 3) * m.cap;
    float* mom = j < 3 ? m.m_sh_dc + (size_t)j * m.cap : m.m_sh_hi + (size_t)(j - 3) * m.cap;
    par[c] = par[p]; mom[p] = 0.f; mom[c] = 0.f;
  }
  m.v_sh[p] = 0.f; m.v_sh[c] = 0.f;
  m.refine_norm[c] = 0.f; m.max_screen[c] = 0.f; m.vis_count[c] = 0.f;
  if (m.tile_count) m.tile_count[c] = 0u;
  m.last_step[c] = 0u; m.last_step[p] = 0u;
}

__global__ void kill_kernel(int count, const uint32_t* __restrict__ idx, float4* __restrict__ pos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) pos[idx[i]].w = -1e6f;   // an opacity nothing renders: the slot is dead until it is reused or compacted away
}

__global__ void opacity_decay_kernel(int n, float4* __restrict__ pos, float delta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) pos[i].w = logit_of(sigmoid_fast(pos[i].w) - delta, 1e-12f, 1.f - 1e-12f);
}

// Folds the floor into the raw parameters and clears it (bake_kernel, refine.cu:40-51).
__global__ void bake_floor_kernel(int n, float4* __restrict__ pos, float4* __restrict__ ls) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float4 l = ls[i];
  if (l.w <= 0.f) return;
  float4 p = pos[i];
  p.w = logit_of(effective_opacity(p.w, l), 1e-6f, 1.f - 1e-6f);
  const float f2 = l.w * l.w;
  l = make_float4(0.5f * __logf(__expf(2.f * l.x) + f2), 0.5f * __logf(__expf(2.f * l.y) + f2), 0.5f * __logf(__expf(2.f * l.z) + f2), 0.f);
  pos[i] = p; ls[i] = l;
}

__global__ void axis_keys_kernel(int n, const float4* __restrict__ pos, int axis, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 p = pos[i];
  const float v = axis == 0 ? p.x : (axis == 1 ? p.y : p.z);
  keys[i] = ascending_key(isfinite(v) ? v : 0.f);
  vals[i] = (uint32_t)i;
}

bool model_ok(const B2kModel* m) { return m && m->n >= 0 && m->cap >= m->n && m->degree >= 0 && m->degree <= 4 && m->pos_op && m->quat && m->lscale && m->sh_dc && (m->degree == 0 || m->sh_hi); }

}  // namespace
}  // namespace b2k

using namespace b2k;

#define LAUNCH_1D(kernel, count, stream, ...) kernel<<<div_up((count), 256), 256, 0, (cudaStream_t)(stream)>>>(__VA_ARGS__)

extern "C" int b2k_refine_flags(const B2kModel* m, const float* center, float max_allowed, float cull_weight, uint32_t* keep, uint32_t* dead, uint32_t* culled,
                                b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m) && center && keep && dead && culled && (cull_weight <= 0.f || m->vis_weight));
  if (m->n == 0) return B2K_OK;
  const int lanes = 3 * (m->degree + 1) * (m->degree + 1);
  LAUNCH_1D(flags_kernel, m->n, s, m->n, (size_t)m->cap, lanes, (const float4*)m->pos_op, (const float4*)m->quat, (const float4*)m->lscale, m->sh_dc, m->sh_hi,
            make_float3(center[0], center[1], center[2]), max_allowed, m->vis_weight, cull_weight, keep, dead, culled);
  return check_launch();
}

extern "C" int b2k_refine_sample_keys(const B2kModel* m, const uint32_t* keep, const uint32_t* excluded, int32_t mode, float threshold, uint32_t seed, uint32_t* keys,
                                      uint32_t* vals, uint32_t* above, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m) && keep && keys && vals && m->vis_count && m->refine_norm && (mode == 0 || mode == 1));
  if (m->n == 0) return B2K_OK;
  LAUNCH_1D(sample_keys_kernel, m->n, s, m->n, keep, excluded, (const float4*)m->pos_op, (const float4*)m->lscale, m->vis_count, m->refine_norm, mode, threshold, seed,
            keys, vals, above);
  return check_launch();
}

extern "C" int b2k_refine_oversized(const B2kModel* m, const uint32_t* keep, const uint32_t* excluded, float threshold, uint32_t* flags, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m) && keep && excluded && flags && m->max_screen && m->vis_count);
  if (m->n == 0) return B2K_OK;
  LAUNCH_1D(oversized_kernel, m->n, s, m->n, keep, excluded, m->max_screen, m->vis_count, threshold, flags);
  return check_launch();
}

extern "C" int b2k_refine_mark(const uint32_t* idx, int32_t count, uint32_t* flags, b2k_stream_t s) {
  B2K_REQUIRE(count >= 0 && (count == 0 || (idx && flags)));
  if (count == 0) return B2K_OK;
  LAUNCH_1D(mark_kernel, count, s, count, idx, flags);
  return check_launch();
}

extern "C" int b2k_refine_split(const B2kModel* m, uint32_t* tile_count, const uint32_t* parents, const uint32_t* dead_idx, int32_t from_dead, int32_t count,
                                float split_at_screen_size, uint32_t* children, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m) && count >= 0 && from_dead >= 0 && from_dead <= count && (count == 0 || (parents && children)) && (from_dead == 0 || dead_idx));
  B2K_REQUIRE(m->m_pos_op && m->v_pos_op && m->m_quat && m->v_quat && m->m_lscale && m->v_lscale && m->m_sh_dc && m->v_sh && m->last_step && (m->degree == 0 || m->m_sh_hi));
  B2K_REQUIRE(m->refine_norm && m->max_screen && m->vis_count);
  if (count == 0) return B2K_OK;
  if ((int64_t)m->n + (count - from_dead) > m->cap) return B2K_ERR_CAPACITY;   // m->n is the count BEFORE the children are appended
  SplitPtrs p;
  p.pos = (float4*)m->pos_op; p.quat = (float4*)m->quat; p.ls = (float4*)m->lscale; p.m_pos = (float4*)m->m_pos_op; p.v_pos = (float4*)m->v_pos_op;
  p.m_q = (float4*)m->m_quat; p.v_q = (float4*)m->v_quat; p.m_ls = (float4*)m->m_lscale; p.v_ls = (float4*)m->v_lscale;
  p.sh_dc = m->sh_dc; p.sh_hi = m->sh_hi; p.m_sh_dc = m->m_sh_dc; p.m_sh_hi = m->m_sh_hi; p.v_sh = m->v_sh; p.refine_norm = m->refine_norm; p.max_screen = m->max_screen;
  p.vis_count = m->vis_count; p.last_step = m->last_step; p.tile_count = tile_count; p.cap = (size_t)m->cap; p.lanes = 3 * (m->degree + 1) * (m->degree + 1);
  LAUNCH_1D(split_kernel, count, s, count, parents, dead_idx, from_dead, (uint32_t)m->n, p, split_at_screen_size, children);
  return check_launch();
}

extern "C" int b2k_refine_kill(const B2kModel* m, const uint32_t* idx, int32_t count, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m) && count >= 0 && (count == 0 || idx));
  if (count == 0) return B2K_OK;
  LAUNCH_1D(kill_kernel, count, s, count, idx, (float4*)m->pos_op);
  return check_launch();
}

extern "C" int b2k_refine_opacity_decay(const B2kModel* m, float delta, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m));
  if (m->n == 0) return B2K_OK;
  LAUNCH_1D(opacity_decay_kernel, m->n, s, m->n, (float4*)m->pos_op, delta);
  return check_launch();
}

extern "C" int b2k_refine_bake_floor(const B2kModel* m, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m));
  if (m->n == 0) return B2K_OK;
  LAUNCH_1D(bake_floor_kernel, m->n, s, m->n, (float4*)m->pos_op, (float4*)m->lscale);
  return check_launch();
}

extern "C" int b2k_refine_axis_keys(const B2kModel* m, int32_t axis, uint32_t* keys, uint32_t* vals, b2k_stream_t s) {
  B2K_REQUIRE(model_ok(m) && axis >= 0 && axis < 3 && keys && vals);
  if (m->n == 0) return B2K_OK;
  LAUNCH_1D(axis_keys_kernel, m->n, s, m->n, (const float4*)m->pos_op, axis, keys, vals);
  return check_launch();
}

extern "C" float b2k_key_to_float(uint32_t ascending_key_bits) {
  const uint32_t u = ascending_key_bits ^ ((ascending_key_bits >> 31) ? 0x80000000u : 0xFFFFFFFFu);
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}
