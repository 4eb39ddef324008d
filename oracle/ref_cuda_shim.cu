// C entry points around the reference's OWN CUDA implementation of the hot path (src/gpu/*.cu, src/model.cu of the
// reference tree), compiled unmodified for sm_100a by the Makefile beside this file into oracle/_ref/librefcuda.so.
// TEST INFRASTRUCTURE ONLY: it is the second oracle (the reference's kernels on the same seeded inputs) and the speed
// incumbent `bench.py` may time beside the product; the product never loads it. This file holds no reference code: it
// includes the reference's headers and calls its public operator API (render.h:97-109, loss.h:32-41, optim.h:50).
#include "gpu/render.h"
#include "gpu/loss.h"
#include "gpu/optim.h"
#include "model.h"
#include "gpu/cage.h"
#include "gpu/deform.h"
#include "gpu/refine.h"
#include "train/evidence.h"
#include <algorithm>
#include <cstring>

// Link-time stand-ins for lanes of the reference that this checker never drives (the evidence pass takes optional rigs,
// always null here; the refinement reads one accessor of the trainer's bounds). They are not reference code.
namespace b2c {
void BodyRig::pose(int, const Model&, cudaStream_t) { throw std::runtime_error("BodyRig::pose is not part of the checker"); }
void CageRig::pose(int, const Model&, cudaStream_t) { throw std::runtime_error("CageRig::pose is not part of the checker"); }
float Bounds::max_extent() const { return std::max(extent[0], std::max(extent[1], extent[2])); }
}

using namespace b2c;

namespace {
struct Handle {
  Model model; RenderCtx ctx; DevBuf<uint32_t> gt; DevBuf<uint8_t> wts; ViewGPU view; DevBuf<float> grads;
  std::string err;
};
Camera camera_of(const float* intr, const float* R, const float* t, int W, int H) {
  Camera c; c.width = W; c.height = H; c.fx = intr[0]; c.fy = intr[1]; c.cx = intr[2]; c.cy = intr[3];
  for (int i = 0; i < 9; i++) c.R[i] = R[i];
  for (int i = 0; i < 3; i++) c.t[i] = t[i];
  c.update_pos();
  return c;
}
RenderParams render_params(const Handle& h, const Camera& cam, const float* bg, int bwd_info) {
  RenderParams rp; rp.cam = CameraGPU::from(cam, h.ctx.W, h.ctx.H);
  for (int k = 0; k < 3; k++) rp.bg[k] = bg[k];
  rp.sh_degree = h.model.degree; rp.bwd_info = bwd_info != 0;
  return rp;
}
template <class F> int guarded(Handle* h, F&& f) {
  try { f(); CUDA_CHECK(cudaDeviceSynchronize()); return 0; } catch (const std::exception& e) { h->err = e.what(); return 1; }
}
}  // namespace

extern "C" {

void* refcu_create(int n, int degree, const float* pos, const float* log_scale, const float* quat, const float* opacity, const float* sh,
                   const float* floor, int W, int H) {
  Handle* h = new Handle();
  try {
    SplatCloud c; c.n = (size_t)n; c.sh_degree = degree;
    const int K = (degree + 1) * (degree + 1);
    c.pos.assign(pos, pos + (size_t)n * 3); c.log_scale.assign(log_scale, log_scale + (size_t)n * 3);
    c.quat.assign(quat, quat + (size_t)n * 4); c.opacity.assign(opacity, opacity + n); c.sh.assign(sh, sh + (size_t)n * K * 3);
    h->model.upload(c);
    if (floor) {   // Model::upload zeroes the floor lane (model.cu:53): write it afterwards
      std::vector<float4> s(n);
      for (int i = 0; i < n; i++) s[i] = make_float4(log_scale[i * 3], log_scale[i * 3 + 1], log_scale[i * 3 + 2], floor[i]);
      CUDA_CHECK(cudaMemcpy(h->model.lscale.ptr, s.data(), (size_t)n * sizeof(float4), cudaMemcpyHostToDevice));
    }
    h->ctx.setup(W, H, h->model.cap, 0);
    CUDA_CHECK(cudaDeviceSynchronize());
  } catch (const std::exception& e) { h->err = e.what(); }
  return h;
}
const char* refcu_error(void* hp) { return ((Handle*)hp)->err.c_str(); }
void refcu_destroy(void* hp) { delete (Handle*)hp; }

int refcu_set_view(void* hp, const uint32_t* gt, const uint8_t* weights) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    const size_t P = (size_t)h->ctx.W * h->ctx.H;
    h->gt.upload(gt, P); h->view.rgba = h->gt; h->view.W = h->ctx.W; h->view.H = h->ctx.H;
    h->view.weights = nullptr;
    if (weights) { h->wts.upload(weights, P); h->view.weights = h->wts; }
  });
}

int refcu_forward(void* hp, const float* intr, const float* R, const float* t, const float* bg, int bwd_info) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] { render_forward(h->ctx, h->model, render_params(*h, camera_of(intr, R, t, h->ctx.W, h->ctx.H), bg, bwd_info), 0); });
}

// lossp: l1_w, ssim_w, bg[3], match_alpha_weight, scale, grad_scale; flags: composite, mask, alpha_lane. Returns the loss in *out.
int refcu_loss(void* hp, const float* lossp, const int* flags, float* out) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    LossParams lp; lp.l1_w = lossp[0]; lp.ssim_w = lossp[1]; lp.bg[0] = lossp[2]; lp.bg[1] = lossp[3]; lp.bg[2] = lossp[4];
    lp.match_alpha_weight = lossp[5]; lp.scale = lossp[6]; lp.grad_scale = lossp[7];
    lp.composite = flags[0]; lp.mask = flags[1]; lp.alpha_lane = flags[2];
    h->ctx.loss_accum.zero(0, 4);
    photometric_loss(h->ctx, h->view, lp, 0);
    std::vector<float> a = h->ctx.loss_accum.download(4);
    *out = a[0];
  });
}

int refcu_backward(void* hp, const float* intr, const float* R, const float* t, const float* bg, int tensor_core, float grad_scale) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    const RenderParams rp = render_params(*h, camera_of(intr, R, t, h->ctx.W, h->ctx.H), bg, 1);
    if (tensor_core) rasterize_backward_tc(h->ctx, h->model, rp, grad_scale, 0); else rasterize_backward(h->ctx, h->model, rp, 0);
  });
}

// Parameter gradients through the debug lane OptimParams::grad_out: out [n][11+3K].
int refcu_grads(void* hp, const float* intr, const float* R, const float* t, float* out) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    const size_t per = 11 + (size_t)h->model.K() * 3, total = (size_t)h->model.n * per;
    h->grads.reserve(total); h->grads.zero();
    OptimParams op; op.cam = CameraGPU::from(camera_of(intr, R, t, h->ctx.W, h->ctx.H), h->ctx.W, h->ctx.H);
    op.active_sh_degree = h->model.degree; op.grad_out = h->grads.ptr;
    optimizer_step(h->ctx, h->model, op, 0);
    CUDA_CHECK(cudaMemcpy(out, h->grads.ptr, total * sizeof(float), cudaMemcpyDeviceToHost));
  });
}

int refcu_optim(void* hp, const float* intr, const float* R, const float* t, int step_t, float lr_mean, int sparse) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    OptimParams op; op.cam = CameraGPU::from(camera_of(intr, R, t, h->ctx.W, h->ctx.H), h->ctx.W, h->ctx.H);
    op.active_sh_degree = h->model.degree; op.t = step_t; op.lr_mean = lr_mean; op.sparse = sparse != 0;
    optimizer_step(h->ctx, h->model, op, 0);
  });
}

// optimizer_step with every Adam / MCMC-noise field of OptimParams the hot path uses (optim.h:10-18,41).
// f: lr_mean, lr_rot, lr_scale, lr_opac, lr_dc, lr_sh_rest, noise_weight, noise_clamp; u: t, sparse, seed, step.
int refcu_optim_full(void* hp, const float* intr, const float* R, const float* t, const float* f, const uint32_t* u) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    OptimParams op; op.cam = CameraGPU::from(camera_of(intr, R, t, h->ctx.W, h->ctx.H), h->ctx.W, h->ctx.H);
    op.active_sh_degree = h->model.degree;
    op.lr_mean = f[0]; op.lr_rot = f[1]; op.lr_scale = f[2]; op.lr_opac = f[3]; op.lr_dc = f[4]; op.lr_sh_rest = f[5];
    op.noise_weight = f[6]; op.noise_clamp = f[7];
    op.t = (int)u[0]; op.sparse = u[1] != 0; op.seed = u[2]; op.step = u[3];
    optimizer_step(h->ctx, h->model, op, 0);
  });
}

// Screen-space gradient lanes and visibility flags as the optimizer's input (what rasterize_backward leaves).
int refcu_set_lanes(void* hp, const float* v_splat, const uint32_t* vis_flag) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    CUDA_CHECK(cudaMemcpy(h->ctx.v_splat.ptr, v_splat, (size_t)h->model.n * 13 * sizeof(float), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(h->ctx.vis_flag.ptr, vis_flag, (size_t)h->model.n * sizeof(uint32_t), cudaMemcpyHostToDevice));
  });
}

// A prediction placed in ctx.out_rgba directly (loss and metric kernels on an arbitrary image).
int refcu_set_image(void* hp, const float* rgba) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] { CUDA_CHECK(cudaMemcpy(h->ctx.out_rgba.ptr, rgba, (size_t)h->ctx.W * h->ctx.H * 4 * sizeof(float), cudaMemcpyHostToDevice)); });
}

// eval_metrics (loss.h:41) on the current ctx.out_rgba: out[0] = sum of squared error, out[1] = sum of SSIM.
int refcu_eval(void* hp, int mask_weighted, float* out) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    CUDA_CHECK(cudaMemset(h->ctx.loss_accum.ptr + 4, 0, 4 * sizeof(float)));
    eval_metrics(h->ctx, h->view, mask_weighted != 0, 0);
    std::vector<float> a = h->ctx.loss_accum.download(8);
    out[0] = a[4]; out[1] = a[5];
  });
}

// The loss gradient image v_out [P][4] of the last refcu_loss.
int refcu_v_out(void* hp, float* dst) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] { CUDA_CHECK(cudaMemcpy(dst, h->ctx.v_out.ptr, (size_t)h->ctx.W * h->ctx.H * 4 * sizeof(float), cudaMemcpyDeviceToHost)); });
}
int refcu_cap(void* hp) { return ((Handle*)hp)->model.cap; }

// what: 0 proj0, 1 proj1, 2 proj2 ([n][4] float), 3 tile_count [n] u32, 4 vals_sorted [num_isect] u32, 5 keys_sorted,
// 6 tile_ranges [tiles][2] u32, 7 out_rgba [P][4], 8 last_idx [P] u32, 9 v_splat [n][13], 10 pos_op, 11 quat, 12 lscale ([n][4]),
// 13 sh_dc [3][cap], 14 sh_hi32 [3(K-1)][cap], 15..20 m/v of pos_op, quat, lscale ([n][4]), 21 m_sh_dc, 22 m_sh_hi32 (planar),
// 23 v_sh [n], 24 last_step [n] u32, 25 vis_count [n], 26 refine_norm [n], 27 out_feat [P][4].
int refcu_download(void* hp, int what, void* dst, size_t bytes) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    const void* src = nullptr;
    switch (what) {
      case 0: src = h->ctx.proj0.ptr; break; case 1: src = h->ctx.proj1.ptr; break; case 2: src = h->ctx.proj2.ptr; break;
      case 3: src = h->ctx.tile_count.ptr; break; case 4: src = h->ctx.vals_sorted.ptr; break; case 5: src = h->ctx.keys_sorted.ptr; break;
      case 6: src = h->ctx.tile_ranges.ptr; break; case 7: src = h->ctx.out_rgba.ptr; break; case 8: src = h->ctx.last_idx.ptr; break;
      case 9: src = h->ctx.v_splat.ptr; break; case 10: src = h->model.pos_op.ptr; break; case 11: src = h->model.quat.ptr; break;
      case 12: src = h->model.lscale.ptr; break;
      case 13: src = h->model.sh_dc.ptr; break; case 14: src = h->model.sh_hi32.ptr; break;
      case 15: src = h->model.m_pos_op.ptr; break; case 16: src = h->model.v_pos_op.ptr; break; case 17: src = h->model.m_quat.ptr; break;
      case 18: src = h->model.v_quat.ptr; break; case 19: src = h->model.m_lscale.ptr; break; case 20: src = h->model.v_lscale.ptr; break;
      case 21: src = h->model.m_sh_dc.ptr; break; case 22: src = h->model.m_sh_hi32.ptr; break; case 23: src = h->model.v_sh.ptr; break;
      case 24: src = h->model.last_step.ptr; break; case 25: src = h->model.vis_count.ptr; break; case 26: src = h->model.refine_norm.ptr; break;
      case 27: src = h->ctx.out_feat.ptr; break;
      default: throw std::runtime_error("bad selector");
    }
    CUDA_CHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
  });
}
uint32_t refcu_num_isect(void* hp) { return ((Handle*)hp)->ctx.num_isect; }

// RefineState::run (gpu/refine.h) on the handle's model with the given statistics ([4][n]: refine_norm, max_screen, vis_count,
// vis_weight) and cameras. fp: growth_grad_threshold, growth_select_fraction, split_at_screen_size, opac_decay, cull_weight;
// up: iter, total, growth_allowed, max_splats, seed, no_new. out: new n, pruned, relocated, grown, split_oversized, culled.
int refcu_refine(void* hp, const float* stats, const float* cam_pos, const float* cam_focal, int n_cams, const float* fp, const uint32_t* up, int* out) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    const size_t n = (size_t)h->model.n;
    float* dst[4] = {h->model.refine_norm.ptr, h->model.max_screen.ptr, h->model.vis_count.ptr, h->model.vis_weight.ptr};
    for (int k = 0; k < 4; k++) CUDA_CHECK(cudaMemcpy(dst[k], stats + k * n, n * sizeof(float), cudaMemcpyHostToDevice));
    RefineState st;
    st.init(h->model, 0);
    st.set_cameras(std::vector<float>(cam_pos, cam_pos + 3 * n_cams), std::vector<float>(cam_focal, cam_focal + n_cams));
    RefineParams p;
    p.growth_grad_threshold = fp[0]; p.growth_select_fraction = fp[1]; p.split_at_screen_size = fp[2]; p.opac_decay = fp[3]; p.cull_weight = fp[4];
    p.iter = up[0]; p.total = up[1]; p.growth_allowed = up[2] != 0; p.max_splats = up[3]; p.seed = up[4]; p.no_new = up[5] != 0;
    const RefineStats r = st.run(h->model, h->ctx, p, 0);
    out[0] = h->model.n; out[1] = r.pruned; out[2] = r.relocated; out[3] = r.grown; out[4] = r.split_oversized; out[5] = r.culled;
  });
}
int refcu_n(void* hp) { return ((Handle*)hp)->model.n; }

// compute_evidence (train/evidence.h) over n_views cameras that share the handle's target view; labels: per-pixel class
// ids or null. out_ev [n][7], out_labels [n][2] (or null). cams: per view intr[4], R[9], t[3] = 16 floats.
int refcu_evidence(void* hp, int n_views, const float* cams, const uint8_t* labels, int masked, int has_alpha, float* out_ev, float* out_labels) {
  Handle* h = (Handle*)hp;
  return guarded(h, [&] {
    DevBuf<uint8_t> lab;
    ViewGPU v = h->view; v.masked = masked != 0; v.has_alpha = has_alpha != 0;
    if (labels) { lab.upload(labels, (size_t)h->ctx.W * h->ctx.H); v.labels = lab; }
    std::vector<ViewGPU> views((size_t)n_views, v);
    std::vector<Camera> cs;
    for (int i = 0; i < n_views; i++) cs.push_back(camera_of(cams + i * 16, cams + i * 16 + 4, cams + i * 16 + 13, h->ctx.W, h->ctx.H));
    Config cfg; cfg.export_labels = labels != nullptr;
    compute_evidence(h->ctx, h->model, views, cs, cfg, 0);
    const std::vector<float> ev = download_evidence(h->model, 0);
    std::memcpy(out_ev, ev.data(), ev.size() * sizeof(float));
    if (out_labels) { const std::vector<float> l = download_labels(h->model, 0); std::memcpy(out_labels, l.data(), l.size() * sizeof(float)); }
  });
}

// One training step of the reference (trainer.cpp:487-529): forward, loss, backward (tensor-core or warp), optimizer.
// Returns the average milliseconds per step over `iters` timed steps (after `warm` untimed ones), CUDA events.
// lr_mean == 0 zeroes every learning rate: the optimizer does all of its work but the scene does not drift between steps.
float refcu_time_steps(void* hp, const float* intr, const float* R, const float* t, const float* bg, int tensor_core, int warm, int iters, float lr_mean) {
  Handle* h = (Handle*)hp;
  float ms = -1.f;
  guarded(h, [&] {
    const Camera cam = camera_of(intr, R, t, h->ctx.W, h->ctx.H);
    const RenderParams rp = render_params(*h, cam, bg, 1);
    LossParams lp; lp.grad_scale = tensor_core ? 3.f * h->ctx.W * h->ctx.H : 1.f;
    cudaEvent_t e0, e1; CUDA_CHECK(cudaEventCreate(&e0)); CUDA_CHECK(cudaEventCreate(&e1));
    for (int it = 0; it < warm + iters; it++) {
      if (it == warm) CUDA_CHECK(cudaEventRecord(e0, 0));
      render_forward(h->ctx, h->model, rp, 0);
      h->ctx.loss_accum.zero(0, 4);
      photometric_loss(h->ctx, h->view, lp, 0);
      accumulate_loss(h->ctx, 0);
      if (tensor_core) rasterize_backward_tc(h->ctx, h->model, rp, lp.grad_scale, 0); else rasterize_backward(h->ctx, h->model, rp, 0);
      OptimParams op; op.cam = rp.cam; op.active_sh_degree = h->model.degree; op.t = ++h->model.adam_t; op.lr_mean = lr_mean; op.sparse = true;
      if (lr_mean == 0.f) op.lr_rot = op.lr_scale = op.lr_opac = op.lr_dc = op.lr_sh_rest = 0.f;   // timing on a scene that stays put
      optimizer_step(h->ctx, h->model, op, 0);
    }
    CUDA_CHECK(cudaEventRecord(e1, 0)); CUDA_CHECK(cudaEventSynchronize(e1));
    CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    ms /= (float)iters;
    cudaEventDestroy(e0); cudaEventDestroy(e1);
  });
  return ms;
}

}  // extern "C"
