// C++ host mirror of the reference's operator interface for the splat hot path, implemented over the C ABI of
// include/b2k.h. Same namespace, type names, member names and free-function signatures as the reference headers
// (src/gpu/util.cuh, src/model.h, src/gpu/render.h, src/gpu/loss.h, src/gpu/optim.h), so a caller written against
// those (the trainer's step loop, the render subcommand, the gradient test harness) compiles against this header.
// Buffers are owned here (DevBuf); the C layer never allocates. Errors throw std::runtime_error, as CUDA_CHECK does in
// the reference (src/gpu/util.cuh:13-15). Lanes that libb2k does not implement throw "unsupported lane".
#pragma once
#include <cuda_runtime.h>
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace b2c {

#define B2C_CUDA_CHECK(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) \
  throw std::runtime_error(std::string("CUDA error ") + cudaGetErrorString(e_) + " at " + __FILE__ + ":" + std::to_string(__LINE__)); } while (0)

// The reference's spelling of the same checks (src/gpu/util.cuh:13-16), for callers written against it.
#ifndef CUDA_CHECK
#define CUDA_CHECK(expr) B2C_CUDA_CHECK(expr)
#define CUDA_KERNEL_CHECK() B2C_CUDA_CHECK(cudaGetLastError())
#endif

constexpr int RT_W = 8;   // rasteriser tile edge
inline int sh_coeffs_for_degree(int d) { return (d + 1) * (d + 1); }

// Byte-level device and pinned-host memory primitives (b2c_api.cpp). Every CUDA failure throws std::runtime_error.
namespace mem {
void* device_block(size_t bytes);
void release_device(void* block) noexcept;
// A block of new_bytes that starts with the first old_bytes of `old` when keep is set; `old` is released once the copy
// (and whatever else is queued on the stream and may still read it) has finished.
void* regrown(void* old, size_t old_bytes, size_t new_bytes, bool keep, cudaStream_t stream);
void clear(void* block, size_t bytes, cudaStream_t stream);
void to_device(void* dst, const void* host_src, size_t bytes, cudaStream_t stream);
void to_host_now(void* host_dst, const void* src, size_t bytes, cudaStream_t stream);   // returns once the bytes have landed
void* pinned_block(size_t bytes);
void release_pinned(void* block) noexcept;
}  // namespace mem

// Owning, grow-only device array: the interface of DevBuf in src/gpu/util.cuh:26-57 (ptr, count, reserve / zero /
// upload / download, implicit conversion to T*), which the reference's callers use directly, over the primitives above.
template <typename T>
struct DevBuf {
  T* ptr = nullptr;
  size_t count = 0;
  DevBuf() = default;
  ~DevBuf() { free(); }
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
  DevBuf(DevBuf&& other) noexcept { exchange(other); }
  DevBuf& operator=(DevBuf&& other) noexcept { DevBuf taken(static_cast<DevBuf&&>(other)); exchange(taken); return *this; }
  void free() noexcept { mem::release_device(ptr); ptr = nullptr; count = 0; }
  void reserve(size_t n, bool keep = false, cudaStream_t stream = 0) {
    if (n <= count) return;
    ptr = static_cast<T*>(mem::regrown(ptr, count * sizeof(T), n * sizeof(T), keep, stream));
    count = n;
  }
  void zero(cudaStream_t stream = 0, size_t n = (size_t)-1) { mem::clear(ptr, std::min(n, count) * sizeof(T), stream); }
  void upload(const T* src, size_t n, cudaStream_t stream = 0) { reserve(n); mem::to_device(ptr, src, n * sizeof(T), stream); }
  void upload(const std::vector<T>& v, cudaStream_t stream = 0) { upload(v.data(), v.size(), stream); }
  std::vector<T> download(size_t n = (size_t)-1, cudaStream_t stream = 0) const {
    std::vector<T> out(n == (size_t)-1 ? count : n);
    mem::to_host_now(out.data(), ptr, out.size() * sizeof(T), stream);
    return out;
  }
  size_t bytes() const { return count * sizeof(T); }
  operator T*() const { return ptr; }

 private:
  void exchange(DevBuf& other) noexcept { std::swap(ptr, other.ptr); std::swap(count, other.count); }
};

// Pinned host array for asynchronous copies in both directions (the role of src/gpu/util.cuh:59-64).
template <typename T>
struct PinnedBuf {
  T* ptr = nullptr;
  size_t count = 0;
  PinnedBuf() = default;
  ~PinnedBuf() { mem::release_pinned(ptr); }
  PinnedBuf(const PinnedBuf&) = delete;
  PinnedBuf& operator=(const PinnedBuf&) = delete;
  void reserve(size_t n) {
    if (n <= count) return;
    mem::release_pinned(ptr);
    ptr = nullptr; count = 0;
    ptr = static_cast<T*>(mem::pinned_block(n * sizeof(T)));
    count = n;
  }
};

// Host splat cloud in the layout of SplatCloud (src/ply.h:12-22).
struct SplatCloud {
  size_t n = 0;
  int sh_degree = 0;
  std::vector<float> pos, log_scale, quat, opacity, sh;   // [n][3], [n][3], [n][4] (w,x,y,z), [n], [n][K][3]
  std::vector<float> floor;                               // [n] 3D-filter floor, empty = none
  bool has_scales = true;                                 // false when the file carried no scale_* columns
  bool has_evidence = false; std::vector<float> evidence; // [n][7] w_in, w_all, err, views, dir xyz (the evidence pass)
  bool has_labels = false; std::vector<float> labels;     // [n][2] class id, winner's share (the label vote)
  int K() const { return (sh_degree + 1) * (sh_degree + 1); }
  void resize(size_t count, int degree) {
    n = count; sh_degree = degree;
    pos.assign(n * 3, 0.f); log_scale.assign(n * 3, 0.f); quat.assign(n * 4, 0.f); opacity.assign(n, 0.f); sh.assign(n * K() * 3, 0.f);
    for (size_t i = 0; i < n; i++) quat[i * 4] = 1.f;
    if (has_evidence) evidence.assign(n * 7, 0.f);
    if (has_labels) labels.assign(n * 2, 0.f);
  }
};

// Splat PLY files (src/ply.h:44-53, src/ply.cpp:80-226) and the camera list of the render subcommand.
constexpr float SH_C0 = 0.28209479177387814f;
extern const char* const EVIDENCE_FIELDS[7];
extern const char* const LABEL_FIELDS[2];
bool ply_is_vertex_only(const std::string& path);
SplatCloud read_ply(const std::string& path);
std::vector<std::string> read_ply_comments(const std::string& path);
void write_ply(const std::string& path, const SplatCloud& c, const std::vector<std::string>& comments);

// Pinhole camera, world-to-camera, OpenCV axes (src/dataset/camera.h:9-16).
struct Camera {
  int width = 0, height = 0;
  float fx = 0, fy = 0, cx = 0, cy = 0;
  float R[9] = {1, 0, 0, 0, 1, 0, 0, 0, 1};
  float t[3] = {0, 0, 0};
  float pos[3] = {0, 0, 0};
  void update_pos() { for (int i = 0; i < 3; i++) pos[i] = -(R[i] * t[0] + R[3 + i] * t[1] + R[6 + i] * t[2]); }
  // World-to-camera pose from a rotation quaternion (normalised here) and a translation.
  void set_w2c_quat(float qw, float qx, float qy, float qz, float tx, float ty, float tz) {
    const float inv = 1.f / std::sqrt(qw * qw + qx * qx + qy * qy + qz * qz);
    const float w = qw * inv, x = qx * inv, y = qy * inv, z = qz * inv;
    const float m[9] = {1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w), 2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                        2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)};
    for (int i = 0; i < 9; i++) R[i] = m[i];
    t[0] = tx; t[1] = ty; t[2] = tz;
    update_pos();
  }
  void rescale(int new_w, int new_h) {   // intrinsics follow the image size
    const float sx = (float)new_w / (float)width, sy = (float)new_h / (float)height;
    fx *= sx; cx *= sx; fy *= sy; cy *= sy; width = new_w; height = new_h;
  }
  float focal_px() const { return 0.5f * (fx + fy); }
};

// Device model (src/model.h:14-40): float4 parameter groups, planar SH with stride cap, moments, refine statistics.
struct Model {
  int n = 0, cap = 0, degree = 3;
  bool sh_fp16 = false;   // not implemented by libb2k: upload() throws when set
  DevBuf<float4> pos_op, quat, lscale;
  DevBuf<float> sh_dc, sh_hi32;
  DevBuf<float4> m_pos_op, v_pos_op, m_quat, v_quat, m_lscale, v_lscale;
  DevBuf<float> m_sh_dc, m_sh_hi32, v_sh;
  DevBuf<float> refine_norm, max_screen, vis_count, vis_weight;
  DevBuf<uint32_t> last_step;
  int adam_t = 0;
  int K() const { return (degree + 1) * (degree + 1); }
  // Capacity for at least `want` splats, contents kept (capacity doubles, src/model.cu:10-11; the planar SH lanes are
  // re-laid out for the new stride).
  void reserve(int want, cudaStream_t stream = 0);
  void upload(const SplatCloud& c, cudaStream_t stream = 0);
  SplatCloud download(cudaStream_t stream = 0) const;
  void zero_optimizer(cudaStream_t stream = 0);
  void zero_stats(cudaStream_t stream = 0);
  // Keeps the splats flagged in `keep` ([n] device words), in order, across every per-splat array and the caller's extra
  // [cap] float arrays (src/model.cu:120-155). Returns the new n.
  int compact(const uint32_t* keep, const std::vector<DevBuf<float>*>& extras, cudaStream_t stream = 0);
};

// src/gpu/render.h:10-24.
struct CameraGPU {
  float R[9]; float t[3]; float pos[3];
  float fx, fy, cx, cy;
  int W, H;
  float lim_pos_x, lim_pos_y, lim_neg_x, lim_neg_y;
  static CameraGPU from(const Camera& c, int W, int H);
};

enum class FeatureMode { None, Normals, Buffer };

// src/gpu/render.h:29-63. Fields of lanes libb2k does not implement are kept so callers compile; setting them throws.
// feat / feat_buffer are implemented in the forward only (out_feat.xyz); the chunked renderer rejects them.
struct RenderParams {
  CameraGPU cam;
  float bg[3] = {0, 0, 0};
  int sh_degree = 3;
  FeatureMode feat = FeatureMode::None;
  const float* feat_buffer = nullptr;
  bool mip = false;
  bool bwd_info = true;
  const float2* warp = nullptr; int warp_w = 0, warp_h = 0;
  const float4* pos_override = nullptr;
  const float4* quat_override = nullptr;
  const float4* lscale_override = nullptr;
  const float4* sh_frame = nullptr;
  const float4* app = nullptr; float4* col_base = nullptr; bool app_add = false;
  const float* hollow_z = nullptr; float hollow_margin = 0.05f; float hollow_lam = 0.f;
};

// src/gpu/render.h:66-95; members the reference's callers read keep their names and element types.
struct RenderCtx {
  int W = 0, H = 0, tiles_x = 0, tiles_y = 0, n_tiles = 0, tile_bits = 0, n_cap = 0;
  DevBuf<float4> proj0, proj1, proj2;
  DevBuf<float2> proj3;              // feature lanes y, z (x rides in proj2.w)
  DevBuf<uint32_t> tile_count, tile_off;
  DevBuf<uint4> hit_info;
  DevBuf<uint32_t> depth_keys, depth_keys_sorted, order_in, order;
  DevBuf<uint32_t> keys, vals, keys_sorted, vals_sorted;
  size_t isect_cap = 0;
  uint32_t num_isect = 0;
  DevBuf<uint32_t> d_num_isect;
  DevBuf<unsigned char> cub_tmp;       // the radix sort's scratch
  DevBuf<uint2> tile_ranges;           // [n_tiles], or [n_chunks][n_tiles] when rendering in chunks
  DevBuf<float4> out_rgba, out_feat;
  DevBuf<float> out_depth;             // optional expected depth (reserve it to enable)
  DevBuf<uint32_t> last_idx;
  DevBuf<float> v_splat;
  DevBuf<uint32_t> vis_flag;
  DevBuf<uint32_t> vis_list;        // splats the backward touched (count in d_num_isect[1]); walked by the sparse optimizer
  DevBuf<float4> v_out;
  DevBuf<float4> v_feat;            // dL/d(feat) per pixel: kept for callers that name it; the feature lanes have no backward here
  DevBuf<float> hollow_pen;         // likewise (hollow loss lane, unsupported)
  DevBuf<float> loss_accum;
  bool want_depth = false;
  int n_chunks = 1;                 // set > 1 before setup(): render_forward composites front to back in depth chunks
  DevBuf<uint32_t> chunk_words;     // scratch of the chunked renderer
  DevBuf<unsigned char> bwd_scratch;   // forward checkpoints + work list of the segmented backward (sized with the intersection buffers)
  void setup(int W, int H, int n_splats, cudaStream_t stream);
};

void render_forward(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream);
void project_splats(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream);
void bin_and_sort(RenderCtx& ctx, const Model& m, cudaStream_t stream);
void rasterize_forward(RenderCtx& ctx, const RenderParams& p, cudaStream_t stream);
void rasterize_backward(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream);
// Same result as rasterize_backward: v_out carries grad_scale and the accumulated lanes are divided by it afterwards.
void rasterize_backward_tc(RenderCtx& ctx, const Model& m, const RenderParams& p, float grad_scale, cudaStream_t stream);

// src/gpu/loss.h:7-30.
struct ViewGPU {
  const uint32_t* rgba = nullptr;
  const uint32_t* normals = nullptr;
  const uint8_t* weights = nullptr;
  const uint8_t* labels = nullptr;
  int W = 0, H = 0;
  bool has_alpha = false, masked = false;
  float alpha_coverage = 1.f;
  float normal_count = 0.f;
  const float2* warp = nullptr; int warp_w = 0, warp_h = 0;
};
struct LossParams {
  float l1_w = 0.8f, ssim_w = -0.2f;
  float bg[3] = {0, 0, 0};
  bool composite = false, mask = false, alpha_lane = false;
  float match_alpha_weight = 0.1f;
  float scale = 1.f;
  float normal_scale = 0.f;
  float grad_scale = 1.f;
};
void photometric_loss(RenderCtx& ctx, const ViewGPU& view, const LossParams& lp, cudaStream_t stream);
// src/gpu/loss.h:35,39: lanes outside this path; declared so callers compile, they throw "unsupported lane".
void normal_loss(RenderCtx& ctx, const ViewGPU& view, const LossParams& lp, cudaStream_t stream);
void hollow_loss(RenderCtx& ctx, float lam, cudaStream_t stream);
void accumulate_loss(RenderCtx& ctx, cudaStream_t stream);
void eval_metrics(RenderCtx& ctx, const ViewGPU& view, bool mask_weighted, cudaStream_t stream);

// src/gpu/optim.h:6-45 (the fields of this path; the cage / deformation lanes throw when set).
struct OptimParams {
  CameraGPU cam;
  bool mip = false;
  int active_sh_degree = 3;
  int t = 1;
  float beta1 = 0.9f, beta2 = 0.999f, eps = 1e-15f;
  float lr_mean = 0.f;
  float lr_rot = 2e-3f, lr_scale = 5e-3f, lr_opac = 0.012f, lr_dc = 2e-3f, lr_sh_rest = 2e-4f;
  float noise_weight = 0.f, noise_clamp = 0.f;
  uint32_t seed = 42, step = 0;
  const float4* pos_override = nullptr;
  float3* g_pos_out = nullptr;
  const float4* quat_override = nullptr;
  const float4* lscale_override = nullptr;
  const float4* sh_frame = nullptr;
  bool frozen = false;
  const uint8_t* update_mask = nullptr;
  const float4* canon_rot = nullptr;
  bool sparse = false;
  const float* spa_z = nullptr; const float* spa_u = nullptr; float spa_rho = 0.f;   // sparsification penalty: throws when set
  const float* stretch_w = nullptr; float stretch_log_tau = 0.f;                     // cage stretch regulariser: throws when set
  float2* g_app_out = nullptr;                                                        // pose-dependent appearance: throws when set
  float* grad_out = nullptr;
};
void optimizer_step(RenderCtx& ctx, Model& m, const OptimParams& op, cudaStream_t stream);
// Data-parallel split of optimizer_step: gradient half adding into grad[n][11+3K], update half from it.
// touched: optional bitmap of (n + 31) / 32 words in which the splats that received a row are marked (B2kOptim.touched_out).
void projection_backward(RenderCtx& ctx, Model& m, const OptimParams& op, float* grad, cudaStream_t stream, uint32_t* touched = nullptr);
void adam_step(Model& m, const OptimParams& op, float* grad, cudaStream_t stream);
void update_min_scale(Model& m, const float* cam_pos, const float* cam_focal, int n_cams, cudaStream_t stream);

// ---- additions for a step that keeps several views in flight (no counterpart in the reference) ----
// render_forward without the host readback of the intersection total: nothing waits for the stream. The total stays in
// ctx.d_num_isect (word 0: this view, word 2: largest since step_begin); grow_intersections() is the reference's
// doubling (src/gpu/binning.cu:129-133) applied afterwards, after which the caller redoes the views.
void render_forward_async(RenderCtx& ctx, const Model& m, const RenderParams& p, cudaStream_t stream);
bool grow_intersections(RenderCtx& ctx, uint32_t needed);
void step_begin(RenderCtx& ctx, cudaStream_t stream);                          // loss_accum and the running maximum = 0
void fold_loss(RenderCtx& dst, const RenderCtx& src, cudaStream_t stream);    // dst.loss_accum[2..3] += src's

}  // namespace b2c

// POD views of the owning objects for direct calls into the C ABI (include/b2k.h).
#include "../../include/b2k.h"
namespace b2c { namespace abi {
void check(int status, const char* what);            // throws std::runtime_error on a non-zero status
B2kModel view_of(const Model& m);
B2kCtx view_of(const RenderCtx& c);
B2kCamera camera_of(const CameraGPU& g);
B2kRenderOpts opts_of(const RenderParams& p, const char* what);
B2kOptim optim_of(const OptimParams& op, const char* what);
void alloc_isect(RenderCtx& c, size_t cap);
} }
