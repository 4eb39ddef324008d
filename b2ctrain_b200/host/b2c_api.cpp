// Bodies of the reference-named operators over the C ABI (include/b2k.h). Each function fills POD views of the
// caller's objects and makes one b2k_* call; see the header for the interfaces mirrored.
#include "b2c_api.h"
#include <type_traits>
#include "../../include/b2k.h"
#include <algorithm>
#include <cstring>

namespace b2c {

namespace mem {

void* device_block(size_t bytes) {
  void* p = nullptr;
  if (bytes) B2C_CUDA_CHECK(cudaMalloc(&p, bytes));
  return p;
}

void release_device(void* block) noexcept { if (block) cudaFree(block); }

void* regrown(void* old, size_t old_bytes, size_t new_bytes, bool keep, cudaStream_t stream) {
  void* fresh = device_block(new_bytes);
  if (!old) return fresh;
  try {
    if (keep && old_bytes) B2C_CUDA_CHECK(cudaMemcpyAsync(fresh, old, std::min(old_bytes, new_bytes), cudaMemcpyDeviceToDevice, stream));
    B2C_CUDA_CHECK(cudaStreamSynchronize(stream));   // nothing queued on the stream reads the old block any more
  } catch (...) { release_device(fresh); throw; }
  release_device(old);
  return fresh;
}

void clear(void* block, size_t bytes, cudaStream_t stream) { if (block && bytes) B2C_CUDA_CHECK(cudaMemsetAsync(block, 0, bytes, stream)); }

void to_device(void* dst, const void* host_src, size_t bytes, cudaStream_t stream) {
  if (bytes) B2C_CUDA_CHECK(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, stream));
}

void to_host_now(void* host_dst, const void* src, size_t bytes, cudaStream_t stream) {
  if (!bytes) return;
  B2C_CUDA_CHECK(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, stream));
  B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
}

void* pinned_block(size_t bytes) {
  void* p = nullptr;
  if (bytes) B2C_CUDA_CHECK(cudaMallocHost(&p, bytes));
  return p;
}

void release_pinned(void* block) noexcept { if (block) cudaFreeHost(block); }

}  // namespace mem
namespace abi {

void check(int status, const char* what) {
  if (status == B2K_OK) return;
  std::string msg = std::string(what) + ": " + b2k_error_string(status);
  if (status == B2K_ERR_CUDA) msg += std::string(" (") + cudaGetErrorString((cudaError_t)b2k_last_cuda_error()) + ")";
  throw std::runtime_error(msg);
}
[[noreturn]] void unsupported(const char* what) { throw std::runtime_error(std::string(what) + ": unsupported lane"); }

B2kModel view_of(const Model& m) {
  B2kModel v{};
  v.n = m.n; v.cap = m.cap; v.degree = m.degree;
  v.pos_op = (float*)m.pos_op.ptr; v.quat = (float*)m.quat.ptr; v.lscale = (float*)m.lscale.ptr;
  v.sh_dc = m.sh_dc.ptr; v.sh_hi = m.sh_hi32.ptr;
  v.m_pos_op = (float*)m.m_pos_op.ptr; v.v_pos_op = (float*)m.v_pos_op.ptr; v.m_quat = (float*)m.m_quat.ptr; v.v_quat = (float*)m.v_quat.ptr;
  v.m_lscale = (float*)m.m_lscale.ptr; v.v_lscale = (float*)m.v_lscale.ptr;
  v.m_sh_dc = m.m_sh_dc.ptr; v.m_sh_hi = m.m_sh_hi32.ptr; v.v_sh = m.v_sh.ptr;
  v.refine_norm = m.refine_norm.ptr; v.max_screen = m.max_screen.ptr; v.vis_count = m.vis_count.ptr; v.vis_weight = m.vis_weight.ptr;
  v.last_step = m.last_step.ptr;
  return v;
}

B2kCtx view_of(const RenderCtx& c) {
  B2kCtx v{};
  v.W = c.W; v.H = c.H; v.tiles_x = c.tiles_x; v.tiles_y = c.tiles_y; v.n_tiles = c.n_tiles; v.tile_bits = c.tile_bits; v.n_cap = c.n_cap;
  v.proj0 = (float*)c.proj0.ptr; v.proj1 = (float*)c.proj1.ptr; v.proj2 = (float*)c.proj2.ptr;
  v.tile_count = c.tile_count.ptr; v.hit_info = (uint32_t*)c.hit_info.ptr;
  v.depth_keys = c.depth_keys.ptr; v.depth_keys_sorted = c.depth_keys_sorted.ptr; v.order_in = c.order_in.ptr; v.order = c.order.ptr;
  v.tile_off = c.tile_off.ptr;
  v.keys = c.keys.ptr; v.vals = c.vals.ptr; v.keys_sorted = c.keys_sorted.ptr; v.vals_sorted = c.vals_sorted.ptr;
  v.isect_cap = c.isect_cap; v.num_isect = c.d_num_isect.ptr;
  v.sort_tmp = c.cub_tmp.ptr; v.sort_tmp_bytes = c.cub_tmp.count;
  v.tile_ranges = (uint32_t*)c.tile_ranges.ptr;
  v.out_rgba = (float*)c.out_rgba.ptr; v.out_feat = (float*)c.out_feat.ptr; v.out_depth = c.out_depth.ptr;
  v.last_idx = c.last_idx.ptr; v.v_splat = c.v_splat.ptr; v.vis_flag = c.vis_flag.ptr; v.vis_list = c.vis_list.ptr; v.v_out = (float*)c.v_out.ptr;
  v.loss_accum = c.loss_accum.ptr;
  v.n_chunks = c.n_chunks; v.chunk_words = c.chunk_words.ptr; v.proj3 = (float*)c.proj3.ptr;
  v.bwd_scratch = c.bwd_scratch.ptr; v.bwd_scratch_bytes = c.bwd_scratch.count;
  return v;
}

B2kCamera camera_of(const CameraGPU& g) {
  static_assert(sizeof(B2kCamera) == sizeof(CameraGPU), "CameraGPU and B2kCamera share one layout");
  B2kCamera c;
  std::memcpy(&c, &g, sizeof c);
  return c;
}

B2kRenderOpts opts_of(const RenderParams& p, const char* what) {
  if (p.mip || p.warp || p.sh_frame || p.app || p.col_base || p.hollow_z) unsupported(what);
  if ((p.feat == FeatureMode::Buffer) != (p.feat_buffer != nullptr)) unsupported(what);
  B2kRenderOpts o{};
  for (int i = 0; i < 3; i++) o.bg[i] = p.bg[i];
  o.sh_degree = p.sh_degree; o.bwd_info = p.bwd_info ? 1 : 0;
  o.pos_override = (const float*)p.pos_override; o.quat_override = (const float*)p.quat_override; o.lscale_override = (const float*)p.lscale_override;
  o.feat_mode = p.feat == FeatureMode::Normals ? 1 : (p.feat == FeatureMode::Buffer ? 2 : 0); o.feat_buffer = p.feat_buffer;
  return o;
}

B2kOptim optim_of(const OptimParams& op, const char* what) {
  if (op.mip || op.g_pos_out || op.sh_frame || op.frozen || op.update_mask || op.canon_rot || op.spa_z || op.spa_u || op.stretch_w || op.g_app_out) unsupported(what);
  B2kOptim o{};
  o.active_sh_degree = op.active_sh_degree; o.t = op.t; o.beta1 = op.beta1; o.beta2 = op.beta2; o.eps = op.eps;
  o.lr_mean = op.lr_mean; o.lr_rot = op.lr_rot; o.lr_scale = op.lr_scale; o.lr_opac = op.lr_opac; o.lr_dc = op.lr_dc; o.lr_sh_rest = op.lr_sh_rest;
  o.noise_weight = op.noise_weight; o.noise_clamp = op.noise_clamp; o.seed = op.seed; o.step = op.step; o.sparse = op.sparse ? 1 : 0;
  o.pos_override = (const float*)op.pos_override; o.quat_override = (const float*)op.quat_override; o.lscale_override = (const float*)op.lscale_override;
  o.grad_out = op.grad_out;
  return o;
}

void alloc_isect(RenderCtx& c, size_t cap) {
  c.keys.free(); c.vals.free(); c.keys_sorted.free(); c.vals_sorted.free();
  c.keys.reserve(cap); c.vals.reserve(cap); c.keys_sorted.reserve(cap); c.vals_sorted.reserve(cap);
  c.isect_cap = cap;
  c.bwd_scratch.reserve((size_t)b2k_bwd_scratch_bytes(c.W, c.H, c.n_chunks, cap));
}

}  // namespace abi
using namespace abi;

CameraGPU CameraGPU::from(const Camera& c, int W, int H) {
  CameraGPU g;
  for (int i = 0; i < 9; i++) g.R[i] = c.R[i];
  for (int i = 0; i < 3; i++) { g.t[i] = c.t[i]; g.pos[i] = c.pos[i]; }
  const float sx = (float)W / (float)c.width, sy = (float)H / (float)c.height;
  g.fx = c.fx * sx; g.fy = c.fy * sy; g.cx = c.cx * sx; g.cy = c.cy * sy; g.W = W; g.H = H;
  g.lim_pos_x = (1.15f * W - g.cx) / g.fx; g.lim_pos_y = (1.15f * H - g.cy) / g.fy;
  g.lim_neg_x = (-0.15f * W - g.cx) / g.fx; g.lim_neg_y = (-0.15f * H - g.cy) / g.fy;
  return g;
}

void Model::reserve(int want, cudaStream_t stream) {
  if (want <= cap) return;
  int ncap = cap > 0 ? cap : 1024;
  while (ncap < want) ncap *= 2;
  const int hi = (K() - 1) * 3;
  // New buffers first, copies enqueued, one wait, then the old ones go.
  auto grown = [&](auto& b, int lanes) {
    using T = std::remove_reference_t<decltype(*b.ptr)>;
    DevBuf<T> nb;
    nb.reserve((size_t)ncap * (size_t)std::max(lanes, 1)); nb.zero(stream);
    if (b.ptr && n > 0 && lanes > 0)
      B2C_CUDA_CHECK(cudaMemcpy2DAsync(nb.ptr, (size_t)ncap * sizeof(T), b.ptr, (size_t)cap * sizeof(T), (size_t)n * sizeof(T), (size_t)lanes, cudaMemcpyDeviceToDevice, stream));
    return nb;
  };
  auto p0 = grown(pos_op, 1), p1 = grown(quat, 1), p2 = grown(lscale, 1), m0 = grown(m_pos_op, 1), m1 = grown(v_pos_op, 1), m2 = grown(m_quat, 1), m3 = grown(v_quat, 1),
       m4 = grown(m_lscale, 1), m5 = grown(v_lscale, 1);
  auto s0 = grown(sh_dc, 3), s1 = grown(sh_hi32, hi), s2 = grown(m_sh_dc, 3), s3 = grown(m_sh_hi32, hi), s4 = grown(v_sh, 1), t0 = grown(refine_norm, 1),
       t1 = grown(max_screen, 1), t2 = grown(vis_count, 1), t3 = grown(vis_weight, 1);
  auto l0 = grown(last_step, 1);
  B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
  pos_op = std::move(p0); quat = std::move(p1); lscale = std::move(p2); m_pos_op = std::move(m0); v_pos_op = std::move(m1); m_quat = std::move(m2); v_quat = std::move(m3);
  m_lscale = std::move(m4); v_lscale = std::move(m5); sh_dc = std::move(s0); sh_hi32 = std::move(s1); m_sh_dc = std::move(s2); m_sh_hi32 = std::move(s3); v_sh = std::move(s4);
  refine_norm = std::move(t0); max_screen = std::move(t1); vis_count = std::move(t2); vis_weight = std::move(t3); last_step = std::move(l0);
  cap = ncap;
}

void Model::upload(const SplatCloud& c, cudaStream_t stream) {
  if (sh_fp16) unsupported("Model::upload (fp16 SH storage)");
  degree = c.sh_degree; n = (int)c.n;
  cap = 1024; while (cap < n) cap *= 2;   // capacity doubles from 1024 (src/model.cu:10-11)
  const int K = this->K(), hi = (K - 1) * 3;
  std::vector<float4> p(cap, float4{0, 0, 0, 0}), q(cap, float4{0, 0, 0, 0}), s(cap, float4{0, 0, 0, 0});
  std::vector<float> dc((size_t)cap * 3, 0.f), rest((size_t)cap * (hi > 0 ? hi : 1), 0.f);
  for (int i = 0; i < n; i++) {
    p[i] = float4{c.pos[i * 3], c.pos[i * 3 + 1], c.pos[i * 3 + 2], c.opacity[i]};
    q[i] = float4{c.quat[i * 4], c.quat[i * 4 + 1], c.quat[i * 4 + 2], c.quat[i * 4 + 3]};
    s[i] = float4{c.log_scale[i * 3], c.log_scale[i * 3 + 1], c.log_scale[i * 3 + 2], c.floor.empty() ? 0.f : c.floor[i]};
    for (int k = 0; k < 3; k++) dc[(size_t)k * cap + i] = c.sh[(size_t)i * K * 3 + k];
    for (int k = 0; k < hi; k++) rest[(size_t)k * cap + i] = c.sh[(size_t)i * K * 3 + 3 + k];
  }
  for (DevBuf<float4>* b : {&pos_op, &quat, &lscale, &m_pos_op, &v_pos_op, &m_quat, &v_quat, &m_lscale, &v_lscale}) { b->free(); b->reserve(cap); }
  for (DevBuf<float>* b : {&sh_dc, &m_sh_dc}) { b->free(); b->reserve((size_t)cap * 3); }
  for (DevBuf<float>* b : {&sh_hi32, &m_sh_hi32}) { b->free(); b->reserve((size_t)cap * (hi > 0 ? hi : 1)); }
  for (DevBuf<float>* b : {&v_sh, &refine_norm, &max_screen, &vis_count, &vis_weight}) { b->free(); b->reserve(cap); }
  last_step.free(); last_step.reserve(cap);
  pos_op.upload(p, stream); quat.upload(q, stream); lscale.upload(s, stream); sh_dc.upload(dc, stream); sh_hi32.upload(rest, stream);
  B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
  zero_optimizer(stream); zero_stats(stream);
  B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
}

SplatCloud Model::download(cudaStream_t stream) const {
  SplatCloud c; c.resize(n, degree); c.floor.assign(n, 0.f);
  const int K = this->K(), hi = (K - 1) * 3;
  auto p = pos_op.download(n, stream), q = quat.download(n, stream), s = lscale.download(n, stream);
  auto dc = sh_dc.download((size_t)cap * 3, stream);
  std::vector<float> rest; if (hi > 0) rest = sh_hi32.download((size_t)cap * hi, stream);
  for (int i = 0; i < n; i++) {
    c.pos[i * 3] = p[i].x; c.pos[i * 3 + 1] = p[i].y; c.pos[i * 3 + 2] = p[i].z; c.opacity[i] = p[i].w;
    c.quat[i * 4] = q[i].x; c.quat[i * 4 + 1] = q[i].y; c.quat[i * 4 + 2] = q[i].z; c.quat[i * 4 + 3] = q[i].w;
    c.log_scale[i * 3] = s[i].x; c.log_scale[i * 3 + 1] = s[i].y; c.log_scale[i * 3 + 2] = s[i].z; c.floor[i] = s[i].w;
    for (int k = 0; k < 3; k++) c.sh[(size_t)i * K * 3 + k] = dc[(size_t)k * cap + i];
    for (int k = 0; k < hi; k++) c.sh[(size_t)i * K * 3 + 3 + k] = rest[(size_t)k * cap + i];
  }
  return c;
}

void Model::zero_optimizer(cudaStream_t stream) {
  for (DevBuf<float4>* b : {&m_pos_op, &v_pos_op, &m_quat, &v_quat, &m_lscale, &v_lscale}) b->zero(stream);
  m_sh_dc.zero(stream); m_sh_hi32.zero(stream); v_sh.zero(stream); last_step.zero(stream); adam_t = 0;
}
void Model::zero_stats(cudaStream_t stream) { refine_norm.zero(stream); max_screen.zero(stream); vis_count.zero(stream); vis_weight.zero(stream); }

int Model::compact(const uint32_t* keep, const std::vector<DevBuf<float>*>& extras, cudaStream_t stream) {
  if (n == 0) return 0;
  DevBuf<uint32_t> idx, cnt, tmp;
  idx.reserve((size_t)n); cnt.reserve(1); tmp.reserve((size_t)b2k_select_tmp_words(n));
  check(b2k_select_flagged(keep, n, idx.ptr, cnt.ptr, tmp.ptr, stream), "Model::compact");
  const uint32_t kept = cnt.download(1, stream)[0];
  if ((int)kept == n) return n;
  const int hi_lanes = (K() - 1) * 3;
  auto gather = [&](auto& b, int lanes) {   // into a fresh buffer of the same capacity, which then replaces the old
    using T = std::remove_reference_t<decltype(*b.ptr)>;
    if (!b.ptr || lanes == 0) return;
    DevBuf<T> nb; nb.reserve(b.count); nb.zero(stream);
    check(b2k_gather_lanes(b.ptr, nb.ptr, idx.ptr, (int)kept, lanes, (uint64_t)cap, (int)sizeof(T), stream), "Model::compact");
    B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
    b = std::move(nb);
  };
  gather(pos_op, 1); gather(quat, 1); gather(lscale, 1); gather(sh_dc, 3); gather(sh_hi32, hi_lanes);
  gather(m_pos_op, 1); gather(v_pos_op, 1); gather(m_quat, 1); gather(v_quat, 1); gather(m_lscale, 1); gather(v_lscale, 1);
  gather(m_sh_dc, 3); gather(m_sh_hi32, hi_lanes); gather(v_sh, 1);
  gather(refine_norm, 1); gather(max_screen, 1); gather(vis_count, 1); gather(vis_weight, 1); gather(last_step, 1);
  for (DevBuf<float>* e : extras) gather(*e, 1);
  n = (int)kept;
  return n;
}

void RenderCtx::setup(int w, int h, int n, cudaStream_t stream) {
  W = w; H = h; tiles_x = (W + RT_W - 1) / RT_W; tiles_y = (H + RT_W - 1) / RT_W; n_tiles = tiles_x * tiles_y;
  tile_bits = 1; while ((1 << tile_bits) < n_tiles + 1) tile_bits++;
  const size_t nn = (size_t)(n > 0 ? n : 1);
  if ((int)nn > n_cap) {
    proj0.reserve(nn); proj1.reserve(nn); proj2.reserve(nn); proj3.reserve(nn); tile_count.reserve(nn); tile_off.reserve(nn); hit_info.reserve(nn);
    depth_keys.reserve(nn); depth_keys_sorted.reserve(nn); order_in.reserve(nn); order.reserve(nn);
    v_splat.free(); v_splat.reserve(nn * 13); v_splat.zero(stream);   // later clears are the optimizer's job (render.cu:13-14)
    vis_flag.free(); vis_flag.reserve(nn); vis_flag.zero(stream);
    vis_list.free(); vis_list.reserve(nn);
    n_cap = (int)nn;
  }
  tile_ranges.reserve((size_t)n_tiles * (n_chunks > 1 ? n_chunks : 1));
  if (n_chunks > 1) chunk_words.reserve(32 + (size_t)n_tiles + (size_t)(tiles_x + 1) * (tiles_y + 1));
  const size_t npx = (size_t)W * H;
  out_rgba.reserve(npx); out_feat.reserve(npx); last_idx.reserve(npx); v_out.reserve(npx);
  if (want_depth) out_depth.reserve(npx);
  loss_accum.reserve(16);
  if (!d_num_isect.ptr) { d_num_isect.reserve(4); d_num_isect.zero(stream); }
  if (isect_cap == 0) alloc_isect(*this, (size_t)1 << 22);   // starting capacity of the reference (render.cu:20)
  bwd_scratch.reserve((size_t)b2k_bwd_scratch_bytes(W, H, n_chunks, isect_cap));   // grows with the image size too
  cub_tmp.reserve((size_t)b2k_sort_tmp_bytes(n_cap, isect_cap));
}

void project_splats(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream) {
  if (m.n == 0) return;
  const B2kModel mv = view_of(m); const B2kCtx cv = view_of(ctx); const B2kCamera cam = camera_of(p.cam); const B2kRenderOpts o = opts_of(p, "project_splats");
  check(b2k_project(&mv, &cam, &o, &cv, stream), "project_splats");
}

void bin_and_sort(RenderCtx& ctx, const Model& m, cudaStream_t stream) {
  B2kCtx cv = view_of(ctx);
  check(b2k_bin_sort(&cv, m.n, stream), "bin_and_sort");
  uint32_t total = 0;
  int st = b2k_read_num_isect(&cv, stream, &total);   // the reference's 4-byte readback (binning.cu:125-127)
  if (st == B2K_ERR_OVERFLOW) {                        // grow by doubling and redo, as binning.cu:129-133 pre-sizes
    size_t ncap = ctx.isect_cap; while (ncap < total) ncap *= 2;
    alloc_isect(ctx, ncap);
    cv = view_of(ctx);
    check(b2k_bin_sort(&cv, m.n, stream), "bin_and_sort");
    st = b2k_read_num_isect(&cv, stream, &total);
  }
  check(st, "bin_and_sort");
  ctx.num_isect = total;
}

void rasterize_forward(RenderCtx& ctx, const RenderParams& p, cudaStream_t stream) {
  const B2kCtx cv = view_of(ctx); const B2kRenderOpts o = opts_of(p, "rasterize_forward");
  check(b2k_raster_fwd(&cv, &o, stream), "rasterize_forward");
}

void render_forward(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream) {
  if (ctx.n_chunks > 1) {   // front to back in depth chunks: same image and gradients, saturated tiles stop emitting
    for (;;) {
      const B2kModel mv = view_of(m); const B2kCtx cv = view_of(ctx); const B2kCamera cam = camera_of(p.cam); const B2kRenderOpts o = opts_of(p, "render_forward");
      check(b2k_render_chunked(&mv, &cam, &o, &cv, stream), "render_forward");
      uint32_t total = 0;
      const int st = b2k_read_num_isect(&cv, stream, &total);
      ctx.num_isect = total;
      if (st != B2K_ERR_OVERFLOW) { check(st, "render_forward"); return; }
      size_t ncap = ctx.isect_cap; while (ncap < (size_t)total + 32u * (size_t)ctx.n_chunks) ncap *= 2;
      alloc_isect(ctx, ncap);
    }
  }
  project_splats(ctx, m, p, stream);
  bin_and_sort(ctx, m, stream);
  rasterize_forward(ctx, p, stream);
}

void render_forward_async(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream) {
  const B2kModel mv = view_of(m); const B2kCtx cv = view_of(ctx); const B2kCamera cam = camera_of(p.cam); const B2kRenderOpts o = opts_of(p, "render_forward");
  if (ctx.n_chunks > 1) { check(b2k_render_chunked(&mv, &cam, &o, &cv, stream), "render_forward"); return; }
  if (m.n > 0) check(b2k_project(&mv, &cam, &o, &cv, stream), "project_splats");
  check(b2k_bin_sort(&cv, m.n, stream), "bin_and_sort");
  check(b2k_raster_fwd(&cv, &o, stream), "rasterize_forward");
}

bool grow_intersections(RenderCtx& ctx, uint32_t needed) {
  if ((size_t)needed <= ctx.isect_cap) return false;
  size_t ncap = ctx.isect_cap; while (ncap < (size_t)needed + 32u * (size_t)(ctx.n_chunks > 1 ? ctx.n_chunks : 1)) ncap *= 2;
  alloc_isect(ctx, ncap);
  return true;
}

void step_begin(RenderCtx& ctx, cudaStream_t stream) { const B2kCtx cv = view_of(ctx); check(b2k_step_begin(&cv, stream), "step_begin"); }
void fold_loss(RenderCtx& dst, const RenderCtx& src, cudaStream_t stream) {
  const B2kCtx a = view_of(dst), b = view_of(src); check(b2k_loss_fold(&a, &b, stream), "fold_loss");
}

void rasterize_backward(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream) {
  const B2kCtx cv = view_of(ctx); const B2kModel mv = view_of(m); const B2kRenderOpts o = opts_of(p, "rasterize_backward");
  check(b2k_raster_bwd(&cv, &mv, &o, stream), "rasterize_backward");
}

void rasterize_backward_tc(RenderCtx& ctx, const Model& m, const RenderParams& p, float grad_scale, cudaStream_t stream) {
  // The reduction here is fp32 throughout, so the scale is not needed for range; it is honoured as the contract says.
  const B2kCtx cv = view_of(ctx); const B2kModel mv = view_of(m); const B2kRenderOpts o = opts_of(p, "rasterize_backward_tc");
  check(b2k_raster_bwd_scaled(&cv, &mv, &o, grad_scale, stream), "rasterize_backward_tc");
}

void photometric_loss(RenderCtx& ctx, const ViewGPU& view, const LossParams& lp, cudaStream_t stream) {
  if (lp.normal_scale != 0.f) unsupported("photometric_loss (normal lane)");
  const B2kCtx cv = view_of(ctx);
  B2kLoss l{};
  l.rgba = view.rgba; l.weights = view.weights; l.l1_w = lp.l1_w; l.ssim_w = lp.ssim_w;
  for (int i = 0; i < 3; i++) l.bg[i] = lp.bg[i];
  l.composite = lp.composite; l.mask = lp.mask; l.alpha_lane = lp.alpha_lane;
  l.match_alpha_weight = lp.match_alpha_weight; l.scale = lp.scale; l.grad_scale = lp.grad_scale;
  check(b2k_loss_photometric(&cv, &l, stream), "photometric_loss");
}

void normal_loss(RenderCtx&, const ViewGPU&, const LossParams&, cudaStream_t) { unsupported("normal_loss"); }
void hollow_loss(RenderCtx&, float, cudaStream_t) { unsupported("hollow_loss"); }

void accumulate_loss(RenderCtx& ctx, cudaStream_t stream) { const B2kCtx cv = view_of(ctx); check(b2k_loss_accumulate(&cv, stream), "accumulate_loss"); }

void eval_metrics(RenderCtx& ctx, const ViewGPU& view, bool mask_weighted, cudaStream_t stream) {
  const B2kCtx cv = view_of(ctx);
  check(b2k_eval_metrics(&cv, view.rgba, mask_weighted ? 1 : 0, stream), "eval_metrics");
}

void optimizer_step(RenderCtx& ctx, Model& m, const OptimParams& op, cudaStream_t stream) {
  if (m.n == 0) return;
  const B2kCtx cv = view_of(ctx); const B2kModel mv = view_of(m); const B2kCamera cam = camera_of(op.cam); const B2kOptim o = optim_of(op, "optimizer_step");
  check(b2k_optim_fused(&cv, &mv, &cam, &o, stream), "optimizer_step");
}

void projection_backward(RenderCtx& ctx, Model& m, const OptimParams& op, float* grad, cudaStream_t stream, uint32_t* touched) {
  const B2kCtx cv = view_of(ctx); const B2kModel mv = view_of(m); const B2kCamera cam = camera_of(op.cam); B2kOptim o = optim_of(op, "projection_backward");
  o.touched_out = touched;
  check(b2k_proj_bwd(&cv, &mv, &cam, &o, grad, stream), "projection_backward");
}

void adam_step(Model& m, const OptimParams& op, float* grad, cudaStream_t stream) {
  const B2kModel mv = view_of(m); const B2kOptim o = optim_of(op, "adam_step");
  check(b2k_adam(&mv, &o, grad, stream), "adam_step");
}

void update_min_scale(Model& m, const float* cam_pos, const float* cam_focal, int n_cams, cudaStream_t stream) {
  const B2kModel mv = view_of(m);
  check(b2k_min_scale(&mv, cam_pos, cam_focal, n_cams, stream), "update_min_scale");
}

}  // namespace b2c
