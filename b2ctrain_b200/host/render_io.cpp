// The file side of the reference's `render` subcommand, headless: the camera list (camera_from_json,
// src/render/renderer.cpp:185-197; width / height / cameras[] of cameras.json, renderer.cpp:207-212) and the per-camera
// loop (renderer.cpp:345-363) up to raw buffers on disk: <name>.rgba8 (W x H x 4 bytes, quantised like the reference's
// PNG rows, renderer.cpp:183,366-368) and, on request, <name>.depth.f32 (W x H floats, expected depth). PNG encoding
// stays with whoever consumes the buffers.
#include "render_io.h"
#include <cmath>
#include <fstream>
#include <sstream>
#include "json_min.h"

namespace b2c {

namespace {
std::string slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("failed to open '" + path + "'");
  std::ostringstream ss; ss << f.rdbuf();
  return ss.str();
}
float num(const Json& j) { return (float)j.number(); }
}  // namespace

Camera camera_from_json(const Json& c, int W, int H) {
  Camera cam;
  cam.width = W; cam.height = H;
  cam.fx = num(c.at("fx")); cam.fy = num(c.at("fy")); cam.cx = num(c.at("cx")); cam.cy = num(c.at("cy"));
  // "rotation" is an OpenGL camera-to-world matrix (columns = the camera's axes, Y up, Z backward). The OpenCV
  // world-to-camera rotation is its transpose with the Y and Z axes flipped.
  const Json& rot = c.at("rotation");
  for (int r = 0; r < 3; r++)
    for (int col = 0; col < 3; col++) cam.R[r * 3 + col] = num(rot[(size_t)col][(size_t)r]) * (r == 0 ? 1.f : -1.f);
  const Json& p = c.at("position");
  const float pos[3] = {num(p[0]), num(p[1]), num(p[2])};
  for (int r = 0; r < 3; r++) cam.t[r] = -(cam.R[r * 3] * pos[0] + cam.R[r * 3 + 1] * pos[1] + cam.R[r * 3 + 2] * pos[2]);
  cam.update_pos();
  return cam;
}

CameraList read_cameras_json(const std::string& path) {
  const Json j = Json::parse(slurp(path));
  CameraList out;
  out.W = (int)j.at("width").number(); out.H = (int)j.at("height").number();
  if (out.W <= 0 || out.H <= 0) throw std::runtime_error("cameras: bad image size");
  const Json& cams = j.at("cameras");
  for (size_t i = 0; i < cams.items.size(); i++) {
    const Json& c = cams[i];
    out.names.push_back(c.at("name").string());
    out.cams.push_back(camera_from_json(c, out.W, out.H));
  }
  return out;
}

void write_cameras_json(const std::string& path, const CameraList& list) {
  std::ofstream f(path);
  if (!f) throw std::runtime_error("failed to open '" + path + "' for writing");
  f.precision(9);
  f << "{\"width\": " << list.W << ", \"height\": " << list.H << ", \"cameras\": [";
  for (size_t i = 0; i < list.cams.size(); i++) {
    const Camera& c = list.cams[i];
    f << (i ? ",\n" : "\n") << "  {\"name\": \"" << list.names[i] << "\", \"fx\": " << c.fx << ", \"fy\": " << c.fy << ", \"cx\": " << c.cx << ", \"cy\": " << c.cy
      << ", \"position\": [" << c.pos[0] << ", " << c.pos[1] << ", " << c.pos[2] << "], \"rotation\": [";
    for (int r = 0; r < 3; r++) {   // back to OpenGL camera-to-world: transpose, Y and Z columns flipped
      f << (r ? ", [" : "[");
      for (int col = 0; col < 3; col++) f << (col ? ", " : "") << c.R[col * 3 + r] * (col == 0 ? 1.f : -1.f);
      f << "]";
    }
    f << "]}";
  }
  f << "\n]}\n";
}

StreamRenderer::StreamRenderer(const SplatCloud& cloud, int W_, int H_, bool depth, int render_chunks, int lanes, size_t isect_cap) : W(W_), H(H_) {
  model.upload(cloud, 0);
  B2C_CUDA_CHECK(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
  B2C_CUDA_CHECK(cudaEventCreateWithFlags(&start_, cudaEventDisableTiming));
  for (int l = 0; l < std::max(1, lanes); l++) {
    auto lane = std::make_unique<Lane>();
    lane->ctx = std::make_unique<RenderCtx>();
    lane->ctx->want_depth = depth;
    lane->ctx->n_chunks = render_chunks > 1 ? render_chunks : 1;
    lane->ctx->setup(W, H, model.cap, 0);
    if (isect_cap) abi::alloc_isect(*lane->ctx, isect_cap);
    B2C_CUDA_CHECK(cudaStreamCreateWithFlags(&lane->stream, cudaStreamNonBlocking));
    B2C_CUDA_CHECK(cudaEventCreateWithFlags(&lane->rendered, cudaEventDisableTiming));
    B2C_CUDA_CHECK(cudaEventCreateWithFlags(&lane->copied, cudaEventDisableTiming));
    lane->total.reserve(4);
    lanes_.push_back(std::move(lane));
  }
  B2C_CUDA_CHECK(cudaDeviceSynchronize());
}

StreamRenderer::~StreamRenderer() {
  cudaDeviceSynchronize();
  for (auto& lane : lanes_) {
    if (lane->rendered) cudaEventDestroy(lane->rendered);
    if (lane->copied) cudaEventDestroy(lane->copied);
    if (lane->stream) cudaStreamDestroy(lane->stream);
  }
  if (start_) cudaEventDestroy(start_);
  if (copy_stream_) cudaStreamDestroy(copy_stream_);
}

// Queues the lane's camera: render, intersection total to pinned memory, then (when asked for) quantise / stage and copy out.
void StreamRenderer::issue(Lane& lane, bool wait_total) {
  RenderCtx& ctx = *lane.ctx;
  cudaStream_t s = lane.stream;
  render_forward_async(ctx, model, lane.params, s);
  B2C_CUDA_CHECK(cudaMemcpyAsync(lane.total.ptr, ctx.d_num_isect.ptr, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
  if (wait_total) B2C_CUDA_CHECK(cudaStreamSynchronize(s));
  if (lane.host_rgba8 || lane.host_depth) {
    const size_t P = (size_t)W * H;
    if (lane.staged) B2C_CUDA_CHECK(cudaStreamWaitEvent(s, lane.copied, 0));   // the copies that read the staging buffers last have run
    if (lane.host_rgba8) {
      lane.stage_rgba.reserve(P);
      abi::check(b2k_quantize_rgba8((const float*)ctx.out_rgba.ptr, lane.stage_rgba.ptr, (int32_t)P, s), "b2k_quantize_rgba8");
    }
    if (lane.host_depth) {
      lane.stage_depth.reserve(P);
      B2C_CUDA_CHECK(cudaMemcpyAsync(lane.stage_depth.ptr, ctx.out_depth.ptr, P * sizeof(float), cudaMemcpyDeviceToDevice, s));
    }
    B2C_CUDA_CHECK(cudaEventRecord(lane.rendered, s));
    B2C_CUDA_CHECK(cudaStreamWaitEvent(copy_stream_, lane.rendered, 0));
    if (lane.host_rgba8) { B2C_CUDA_CHECK(cudaMemcpyAsync(lane.host_rgba8, lane.stage_rgba.ptr, P * sizeof(uint32_t), cudaMemcpyDeviceToHost, copy_stream_)); d2h_bytes += P * 4; }
    if (lane.host_depth) { B2C_CUDA_CHECK(cudaMemcpyAsync(lane.host_depth, lane.stage_depth.ptr, P * sizeof(float), cudaMemcpyDeviceToHost, copy_stream_)); d2h_bytes += P * 4; }
    B2C_CUDA_CHECK(cudaEventRecord(lane.copied, copy_stream_));
    lane.staged = true;
  } else {
    B2C_CUDA_CHECK(cudaEventRecord(lane.rendered, s));
  }
}

// The lane's camera is done; if its intersections did not fit, the buffers grow and it is rendered (and copied) again.
void StreamRenderer::settle(Lane& lane) {
  if (!lane.pending) return;
  B2C_CUDA_CHECK(cudaEventSynchronize(lane.rendered));
  for (int guard = 0; guard < 8 && grow_intersections(*lane.ctx, lane.total.ptr[0]); guard++) {
    if (lane.staged) B2C_CUDA_CHECK(cudaEventSynchronize(lane.copied));
    redone++;
    issue(lane, true);
    B2C_CUDA_CHECK(cudaEventSynchronize(lane.rendered));
  }
  lane.ctx->num_isect = lane.total.ptr[0];
  last_num_isect = lane.total.ptr[0];
  lane.pending = false;
}

void StreamRenderer::render(const Camera& cam, const float bg[3], int sh_degree, uint32_t* host_rgba8, float* host_depth, cudaStream_t stream) {
  Lane& lane = *lanes_[next_++ % lanes_.size()];
  settle(lane);
  if (host_depth && !lane.ctx->want_depth) throw std::runtime_error("StreamRenderer: depth was not asked for at construction");
  lane.params = RenderParams();
  lane.params.cam = CameraGPU::from(cam, W, H);
  for (int k = 0; k < 3; k++) lane.params.bg[k] = bg ? bg[k] : 0.f;
  lane.params.sh_degree = sh_degree >= 0 ? std::min(sh_degree, model.degree) : model.degree;
  lane.params.bwd_info = false;
  lane.host_rgba8 = host_rgba8; lane.host_depth = host_depth;
  B2C_CUDA_CHECK(cudaEventRecord(start_, stream));
  B2C_CUDA_CHECK(cudaStreamWaitEvent(lane.stream, start_, 0));
  issue(lane, false);
  lane.pending = true;
}

void StreamRenderer::finish() {
  for (auto& lane : lanes_) settle(*lane);
  B2C_CUDA_CHECK(cudaStreamSynchronize(copy_stream_));
}

int render_headless(const std::string& splat_path, const std::string& cameras_path, const std::string& output_dir, const HeadlessOptions& opt) {
  SplatCloud cloud = read_ply(splat_path);
  if (!cloud.has_scales) throw std::runtime_error("ply '" + splat_path + "' has no scales");
  const CameraList list = read_cameras_json(cameras_path);
  const int W = list.W, H = list.H;
  const size_t P = (size_t)W * H;
  cudaStream_t stream = 0;
  StreamRenderer renderer(cloud, W, H, opt.depth, opt.render_chunks, 1);
  // Two host slots: camera k is written to its files while camera k + 1 renders and reads back.
  PinnedBuf<uint32_t> img[2];
  PinnedBuf<float> dep[2];
  for (int k = 0; k < 2; k++) { img[k].reserve(P); if (opt.depth) dep[k].reserve(P); }
  auto write_out = [&](const std::string& file, int k) {
    std::string name = file;
    const size_t dot = name.rfind('.');
    if (dot != std::string::npos) name = name.substr(0, dot);
    {
      std::ofstream f(output_dir + "/" + name + ".rgba8", std::ios::binary);
      f.write((const char*)img[k].ptr, (std::streamsize)(P * sizeof(uint32_t)));
      if (!f) throw std::runtime_error("failed to write '" + output_dir + "/" + name + ".rgba8'");
    }
    if (opt.depth) {
      std::ofstream f(output_dir + "/" + name + ".depth.f32", std::ios::binary);
      f.write((const char*)dep[k].ptr, (std::streamsize)(P * sizeof(float)));
      if (!f) throw std::runtime_error("failed to write '" + output_dir + "/" + name + ".depth.f32'");
    }
  };
  int count = 0;
  std::string pending;
  for (size_t i = (size_t)opt.rank; i < list.cams.size(); i += (size_t)std::max(1, opt.world)) {   // cameras split round-robin over ranks
    const int k = count & 1;
    renderer.render(list.cams[i], opt.background, opt.sh_degree, img[k].ptr, opt.depth ? dep[k].ptr : nullptr, stream);
    if (count > 0) write_out(pending, k ^ 1);   // the previous camera's copies were waited for below
    renderer.finish();
    pending = list.names[i];
    count++;
  }
  if (count > 0) write_out(pending, (count - 1) & 1);
  return count;
}

}  // namespace b2c
