// File side of the headless render front end: cameras.json and the per-camera render loop to raw buffers
// (src/render/renderer.cpp:185-197, 207-212, 345-368).
#pragma once
#include <memory>
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
// A renderer for many cameras of one model. Cameras are dealt to `lanes` render contexts, each on its own stream, so that
// the short kernels and the tails of one camera's launches overlap with another camera's (the same reason the step
// trainer keeps several views in flight). The image is quantised on the device and it, and the depth map, leave on a copy
// stream while later cameras render. Nothing is read back while a camera renders: its intersection total is checked
// when its lane is used again (or at finish), and a camera whose lists did not fit is rendered again with larger
// buffers, so host buffers are valid after finish(). Host pointers should be pinned for the copies to overlap.
class StreamRenderer {
 public:
  // isect_cap: starting capacity of every lane's intersection buffers (0: the reference's 2^22); they grow when a camera needs more.
  StreamRenderer(const SplatCloud& cloud, int W, int H, bool depth, int render_chunks, int lanes = 1, size_t isect_cap = 0);
  ~StreamRenderer();
  StreamRenderer(const StreamRenderer&) = delete;
  StreamRenderer& operator=(const StreamRenderer&) = delete;
  // Renders one camera after whatever is queued on `stream`. host_rgba8 (W * H words) and host_depth (W * H floats) may
  // be null: nothing is read back.
  void render(const Camera& cam, const float bg[3], int sh_degree, uint32_t* host_rgba8, float* host_depth, cudaStream_t stream);
  void finish();   // every camera issued so far is rendered (again, where its buffers had been too small) and read back
  RenderCtx& ctx_of(int lane) { return *lanes_[lane]->ctx; }
  int lanes() const { return (int)lanes_.size(); }
  Model model;
  int W, H;
  uint64_t d2h_bytes = 0;
  uint64_t last_num_isect = 0;   // of the camera settled last
  int redone = 0;                // cameras rendered twice because their intersections did not fit

 private:
  struct Lane {
    std::unique_ptr<RenderCtx> ctx;
    cudaStream_t stream = nullptr;
    cudaEvent_t rendered = nullptr, copied = nullptr;
    DevBuf<uint32_t> stage_rgba;
    DevBuf<float> stage_depth;
    PinnedBuf<uint32_t> total;
    bool pending = false, staged = false;
    RenderParams params;
    uint32_t* host_rgba8 = nullptr;
    float* host_depth = nullptr;
  };
  void issue(Lane& lane, bool wait_total);
  void settle(Lane& lane);
  std::vector<std::unique_ptr<Lane>> lanes_;
  cudaStream_t copy_stream_ = nullptr;
  cudaEvent_t start_ = nullptr;
  size_t next_ = 0;
};

// Renders every camera of this rank's share and writes <output_dir>/<name>.rgba8 (+ .depth.f32). Returns the count.
int render_headless(const std::string& splat_path, const std::string& cameras_path, const std::string& output_dir, const HeadlessOptions& opt);

}  // namespace b2c
