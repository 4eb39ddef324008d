// C entry points of the C++ host (libb2chost.so): what a launcher written in another language (the benchmark driver, a
// test) calls to run StepTrainer steps without any of the step loop living on its side. Exceptions of the C++ layer
// become a non-zero return; b2ch_last_error() has the message.
#include "host_c.h"
#include <cstring>
#include <string>
#include "refine.h"
#include "render_io.h"
#include "trainer.h"

using namespace b2c;

namespace {
thread_local std::string g_error;
template <class F> int guarded(F&& f) {
  try { f(); return 0; } catch (const std::exception& e) { g_error = e.what(); return 1; }
}
StepConfig config_of(const B2chConfig& c) {
  StepConfig s;
  s.views_in_flight = c.views_in_flight; s.render_chunks = c.render_chunks; s.isect_cap = (size_t)c.isect_cap; s.ssim_weight = c.ssim_weight;
  s.mask = c.mask != 0; s.alpha_lane = c.alpha_lane != 0; s.composite = c.composite != 0; s.match_alpha_weight = c.match_alpha_weight; s.loss_scale = c.loss_scale;
  for (int k = 0; k < 3; k++) s.bg[k] = c.bg[k];
  s.lr_mean = c.lr_mean; s.lr_rot = c.lr_rot; s.lr_scale = c.lr_scale; s.lr_opac = c.lr_opac; s.lr_dc = c.lr_dc; s.lr_sh_rest = c.lr_sh_rest;
  s.sparse = c.sparse != 0; s.noise_weight = c.noise_weight; s.noise_clamp = c.noise_clamp; s.seed = c.seed; s.shard_update = c.shard_update != 0;
  return s;
}
}  // namespace

extern "C" const char* b2ch_last_error(void) { return g_error.c_str(); }

extern "C" void* b2ch_trainer_create(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh, int32_t W, int32_t H,
                                     const B2chConfig* cfg, int32_t rank, int32_t world, const uint8_t* dp_id) {
  StepTrainer* tr = nullptr;
  const int st = guarded([&] {
    if (!cfg || n < 0 || (n > 0 && (!pos_op || !quat || !lscale || !sh))) throw std::runtime_error("b2ch_trainer_create: bad argument");
    SplatCloud c; c.resize((size_t)n, degree); c.floor.assign((size_t)n, 0.f);
    const int K = c.K();
    for (int i = 0; i < n; i++) {
      for (int k = 0; k < 3; k++) { c.pos[i * 3 + k] = pos_op[i * 4 + k]; c.log_scale[i * 3 + k] = lscale[i * 4 + k]; }
      c.opacity[i] = pos_op[i * 4 + 3]; c.floor[i] = lscale[i * 4 + 3];
      for (int k = 0; k < 4; k++) c.quat[i * 4 + k] = quat[i * 4 + k];
    }
    std::memcpy(c.sh.data(), sh, (size_t)n * K * 3 * sizeof(float));
    tr = new StepTrainer(c, W, H, config_of(*cfg), rank, world, dp_id);
  });
  return st ? nullptr : tr;
}

extern "C" void b2ch_trainer_destroy(void* h) { delete (StepTrainer*)h; }

extern "C" int b2ch_trainer_add_view(void* h, const B2kCamera* cam, const uint32_t* rgba) {
  int idx = -1;
  const int st = guarded([&] {
    StepTrainer& tr = *(StepTrainer*)h;
    Camera c; c.width = cam->W; c.height = cam->H; c.fx = cam->fx; c.fy = cam->fy; c.cx = cam->cx; c.cy = cam->cy;
    for (int i = 0; i < 9; i++) c.R[i] = cam->R[i];
    for (int i = 0; i < 3; i++) { c.t[i] = cam->t[i]; c.pos[i] = cam->pos[i]; }
    idx = tr.add_view(c, rgba);
  });
  return st ? -1 : idx;
}

extern "C" int b2ch_trainer_step(void* h, const int32_t* views, int32_t n_views, void* stream, int32_t from_host) {
  return guarded([&] { ((StepTrainer*)h)->step(std::vector<int>(views, views + n_views), (cudaStream_t)stream, from_host != 0); });
}

extern "C" int b2ch_trainer_read_loss(void* h, float* out16, void* stream) { return guarded([&] { ((StepTrainer*)h)->read_loss(out16, (cudaStream_t)stream); }); }

extern "C" int b2ch_trainer_set_profile(void* h, int32_t on) { ((StepTrainer*)h)->profile = on != 0; return 0; }

extern "C" int b2ch_trainer_info(void* h, uint64_t* out8) {
  return guarded([&] {
    StepTrainer& tr = *(StepTrainer*)h;
    out8[0] = tr.ctxs[0]->isect_cap; out8[1] = (uint64_t)tr.overflow_redos; out8[2] = tr.h2d_bytes; out8[3] = (uint64_t)tr.model.n;
    out8[4] = (uint64_t)tr.model.adam_t; out8[5] = (uint64_t)tr.ctxs.size(); out8[6] = (uint64_t)tr.views.size(); out8[7] = (uint64_t)tr.ctxs[0]->tile_bits;
    std::memcpy(out8 + 8, tr.phase_ms, sizeof tr.phase_ms);   // out8[8..10]: the six phase times of the last profiled step as floats
    tr.h2d_bytes = 0;
  });
}

extern "C" int b2ch_trainer_download(void* h, float* pos_op, float* quat, float* lscale, float* sh) {
  return guarded([&] {
    const SplatCloud c = ((StepTrainer*)h)->model.download(0);
    for (size_t i = 0; i < c.n; i++) {
      for (int k = 0; k < 3; k++) { pos_op[i * 4 + k] = c.pos[i * 3 + k]; lscale[i * 4 + k] = c.log_scale[i * 3 + k]; }
      pos_op[i * 4 + 3] = c.opacity[i]; lscale[i * 4 + 3] = c.floor[i];
      for (int k = 0; k < 4; k++) quat[i * 4 + k] = c.quat[i * 4 + k];
    }
    std::memcpy(sh, c.sh.data(), c.sh.size() * sizeof(float));
  });
}

extern "C" int b2ch_trainer_reduce_statistics(void* h, void* stream) { return guarded([&] { ((StepTrainer*)h)->reduce_statistics((cudaStream_t)stream); }); }

extern "C" uint64_t b2ch_trainer_checksum(void* h, void* stream) {
  uint64_t v = 0;
  guarded([&] { v = ((StepTrainer*)h)->replica_checksum((cudaStream_t)stream); });
  return v;
}

// ---- files: splat PLY and the headless render front end ----
static SplatCloud cloud_of(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh) {
  if (n < 0 || (n > 0 && (!pos_op || !quat || !lscale || !sh))) throw std::runtime_error("bad splat arrays");
  SplatCloud c; c.resize((size_t)n, degree); c.floor.assign((size_t)n, 0.f);
  const int K = c.K();
  for (int i = 0; i < n; i++) {
    for (int k = 0; k < 3; k++) { c.pos[i * 3 + k] = pos_op[i * 4 + k]; c.log_scale[i * 3 + k] = lscale[i * 4 + k]; }
    c.opacity[i] = pos_op[i * 4 + 3]; c.floor[i] = lscale[i * 4 + 3];
    for (int k = 0; k < 4; k++) c.quat[i * 4 + k] = quat[i * 4 + k];
  }
  std::memcpy(c.sh.data(), sh, (size_t)n * K * 3 * sizeof(float));
  return c;
}

extern "C" void* b2ch_renderer_create(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh, int32_t W, int32_t H,
                                      int32_t depth, int32_t render_chunks, int32_t lanes, uint64_t isect_cap) {
  StreamRenderer* r = nullptr;
  const int st = guarded([&] { r = new StreamRenderer(cloud_of(n, degree, pos_op, quat, lscale, sh), W, H, depth != 0, render_chunks, lanes, (size_t)isect_cap); });
  return st ? nullptr : r;
}

extern "C" void b2ch_renderer_destroy(void* h) { delete (StreamRenderer*)h; }

extern "C" int b2ch_renderer_render(void* h, const B2kCamera* cam, const float* background, int32_t sh_degree, uint32_t* host_rgba8, float* host_depth, void* stream) {
  return guarded([&] {
    Camera c; c.width = cam->W; c.height = cam->H; c.fx = cam->fx; c.fy = cam->fy; c.cx = cam->cx; c.cy = cam->cy;
    for (int i = 0; i < 9; i++) c.R[i] = cam->R[i];
    for (int i = 0; i < 3; i++) { c.t[i] = cam->t[i]; c.pos[i] = cam->pos[i]; }
    ((StreamRenderer*)h)->render(c, background, sh_degree, host_rgba8, host_depth, (cudaStream_t)stream);
  });
}

extern "C" int b2ch_renderer_finish(void* h) { return guarded([&] { ((StreamRenderer*)h)->finish(); }); }

extern "C" int b2ch_renderer_info(void* h, uint64_t* out4) {   // five words
  return guarded([&] {
    StreamRenderer& r = *(StreamRenderer*)h;
    out4[0] = r.last_num_isect; out4[1] = r.ctx_of(0).isect_cap; out4[2] = r.d2h_bytes; out4[3] = (uint64_t)r.ctx_of(0).tile_bits;
    out4[4] = (uint64_t)r.redone;
    r.d2h_bytes = 0;
  });
}

extern "C" int b2ch_render_headless(const char* splat, const char* cameras, const char* output_dir, const float* background, int32_t sh_degree, int32_t depth,
                                    int32_t render_chunks, int32_t rank, int32_t world, int32_t* rendered) {
  return guarded([&] {
    HeadlessOptions o;
    if (background) for (int k = 0; k < 3; k++) o.background[k] = background[k];
    o.sh_degree = sh_degree; o.depth = depth != 0; o.render_chunks = render_chunks; o.rank = rank; o.world = world;
    const int n = render_headless(splat, cameras, output_dir, o);
    if (rendered) *rendered = n;
  });
}

// Reads a PLY into caller arrays in two calls: with every pointer NULL it only reports n and the SH degree.
extern "C" int b2ch_ply_read(const char* path, int32_t* n, int32_t* degree, float* pos, float* log_scale, float* quat, float* opacity, float* sh, float* evidence,
                             float* labels, int32_t* flags) {
  return guarded([&] {
    const SplatCloud c = read_ply(path);
    *n = (int32_t)c.n; *degree = c.sh_degree;
    if (flags) *flags = (c.has_scales ? 1 : 0) | (c.has_evidence ? 2 : 0) | (c.has_labels ? 4 : 0);
    auto put = [](float* dst, const std::vector<float>& src) { if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(float)); };
    put(pos, c.pos); put(log_scale, c.log_scale); put(quat, c.quat); put(opacity, c.opacity); put(sh, c.sh); put(evidence, c.evidence); put(labels, c.labels);
  });
}

extern "C" int b2ch_ply_write(const char* path, int32_t n, int32_t degree, const float* pos, const float* log_scale, const float* quat, const float* opacity,
                              const float* sh, const float* evidence, const float* labels, const char* comment) {
  return guarded([&] {
    SplatCloud c;
    c.has_evidence = evidence != nullptr; c.has_labels = labels != nullptr;
    c.resize((size_t)n, degree);
    auto take = [](std::vector<float>& dst, const float* src) { if (src && !dst.empty()) std::memcpy(dst.data(), src, dst.size() * sizeof(float)); };
    take(c.pos, pos); take(c.log_scale, log_scale); take(c.quat, quat); take(c.opacity, opacity); take(c.sh, sh); take(c.evidence, evidence); take(c.labels, labels);
    std::vector<std::string> comments;
    if (comment && *comment) comments.push_back(comment);
    write_ply(path, c, comments);
  });
}

// ---- refinement: one RefineState::run on a model built from host arrays (the pass as a library call; tests drive it) ----
extern "C" int b2ch_refine_once(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh, const float* stats,
                                const float* cam_pos, const float* cam_focal, int32_t n_cams, const float* fp, const uint32_t* up, int32_t W, int32_t H,
                                int32_t* out, int32_t capacity, float* o_pos_op, float* o_quat, float* o_lscale, float* o_sh, uint32_t* o_pairs) {
  return guarded([&] {
    SplatCloud c; c.resize((size_t)n, degree); c.floor.assign((size_t)n, 0.f);
    const int K = c.K();
    for (int i = 0; i < n; i++) {
      for (int k = 0; k < 3; k++) { c.pos[i * 3 + k] = pos_op[i * 4 + k]; c.log_scale[i * 3 + k] = lscale[i * 4 + k]; }
      c.opacity[i] = pos_op[i * 4 + 3]; c.floor[i] = lscale[i * 4 + 3];
      for (int k = 0; k < 4; k++) c.quat[i * 4 + k] = quat[i * 4 + k];
    }
    std::memcpy(c.sh.data(), sh, (size_t)n * K * 3 * sizeof(float));
    Model m; m.upload(c, 0);
    RenderCtx ctx; ctx.setup(W, H, m.cap, 0);
    float* dst[4] = {m.refine_norm.ptr, m.max_screen.ptr, m.vis_count.ptr, m.vis_weight.ptr};
    for (int k = 0; k < 4; k++) B2C_CUDA_CHECK(cudaMemcpy(dst[k], stats + (size_t)k * n, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    RefineState st;
    st.init(m, 0);
    st.set_cameras(std::vector<float>(cam_pos, cam_pos + 3 * n_cams), std::vector<float>(cam_focal, cam_focal + n_cams));
    RefineParams p;
    p.growth_grad_threshold = fp[0]; p.growth_select_fraction = fp[1]; p.split_at_screen_size = fp[2]; p.opac_decay = fp[3]; p.cull_weight = fp[4];
    p.iter = up[0]; p.total = up[1]; p.growth_allowed = up[2] != 0; p.max_splats = up[3]; p.seed = up[4]; p.no_new = up[5] != 0;
    const RefineStats r = st.run(m, ctx, p, 0);
    out[0] = m.n; out[1] = r.pruned; out[2] = r.relocated; out[3] = r.grown; out[4] = r.split_oversized; out[5] = r.culled; out[6] = (int32_t)st.last_pairs;
    if (m.n > capacity) throw std::runtime_error("b2ch_refine_once: output arrays too small");
    const SplatCloud d = m.download(0);
    for (size_t i = 0; i < d.n; i++) {
      for (int k = 0; k < 3; k++) { o_pos_op[i * 4 + k] = d.pos[i * 3 + k]; o_lscale[i * 4 + k] = d.log_scale[i * 3 + k]; }
      o_pos_op[i * 4 + 3] = d.opacity[i]; o_lscale[i * 4 + 3] = d.floor[i];
      for (int k = 0; k < 4; k++) o_quat[i * 4 + k] = d.quat[i * 4 + k];
    }
    std::memcpy(o_sh, d.sh.data(), d.sh.size() * sizeof(float));
    if (o_pairs && st.last_pairs) {
      B2C_CUDA_CHECK(cudaMemcpy(o_pairs, st.sel_parent.ptr, st.last_pairs * sizeof(uint32_t), cudaMemcpyDeviceToHost));
      B2C_CUDA_CHECK(cudaMemcpy(o_pairs + st.last_pairs, st.sel_child.ptr, st.last_pairs * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    }
  });
}

extern "C" int b2ch_trainer_refine(void* h, const float* cam_pos, const float* cam_focal, int32_t n_cams, const float* fp, const uint32_t* up, void* stream, int32_t* out) {
  return guarded([&] {
    StepTrainer& tr = *(StepTrainer*)h;
    if (n_cams > 0) tr.refiner.set_cameras(std::vector<float>(cam_pos, cam_pos + 3 * n_cams), std::vector<float>(cam_focal, cam_focal + n_cams));
    RefineParams p;
    p.growth_grad_threshold = fp[0]; p.growth_select_fraction = fp[1]; p.split_at_screen_size = fp[2]; p.opac_decay = fp[3]; p.cull_weight = fp[4];
    p.iter = up[0]; p.total = up[1]; p.growth_allowed = up[2] != 0; p.max_splats = up[3]; p.seed = up[4]; p.no_new = up[5] != 0;
    const RefineStats r = tr.refine(p, (cudaStream_t)stream);
    out[0] = tr.model.n; out[1] = r.pruned; out[2] = r.relocated; out[3] = r.grown; out[4] = r.split_oversized; out[5] = r.culled;
  });
}
