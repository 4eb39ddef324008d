// File side of the headless render front end: cameras.json and the per-camera render loop to raw buffers
// (src/render/renderer.cpp:185-197, 207-212, 345-368).
#pragma once
#include "b2c_api.h"

namespace b2c {

struct Json;
struct CameraList {
  int W = 0, H = 0;
  std::vector<std::string> names;
  std::vector<Camera> cams;
};
Camera camera_from_json(const Json& c, int W, int H);
CameraList read_cameras_json(const std::string& path);
void write_cameras_json(const std::string& path, const CameraList& list);

struct HeadlessOptions {
  float background[3] = {0.f, 0.f, 0.f};
  int sh_degree = -1;        // < 0: the model's
  bool depth = false;        // also write <name>.depth.f32
  int render_chunks = 1;     // > 1: the front-to-back chunked renderer
  int rank = 0, world = 1;   // cameras rank, rank + world, ... (one process per GPU, no collective)
};
// A renderer for many cameras of one model: the image is quantised on the device and it, and the depth map, leave on a
// copy stream while the next camera renders (two staging slots). Host pointers should be pinned for the copies to overlap.
class StreamRenderer {
 public:
  StreamRenderer(const SplatCloud& cloud, int W, int H, bool depth, int render_chunks);
  ~StreamRenderer();
  StreamRenderer(const StreamRenderer&) = delete;
  StreamRenderer& operator=(const StreamRenderer&) = delete;
  // Renders one camera on `stream`. host_rgba8 (W * H words) and host_depth (W * H floats) may be null: nothing is read back.
  void render(const Camera& cam, const float bg[3], int sh_degree, uint32_t* host_rgba8, float* host_depth, cudaStream_t stream);
  void finish();   // every read-back issued so far has landed
  Model model;
  RenderCtx ctx;
  int W, H;
  uint64_t d2h_bytes = 0;

 private:
  DevBuf<uint32_t> stage_rgba_[2];
  DevBuf<float> stage_depth_[2];
  cudaStream_t copy_stream_ = nullptr;
  cudaEvent_t ready_[2] = {nullptr, nullptr}, free_[2] = {nullptr, nullptr};
  bool used_[2] = {false, false};
  int slot_ = 0;
};

// Renders every camera of this rank's share and writes <output_dir>/<name>.rgba8 (+ .depth.f32). Returns the count.
int render_headless(const std::string& splat_path, const std::string& cameras_path, const std::string& output_dir, const HeadlessOptions& opt);

}  // namespace b2c
