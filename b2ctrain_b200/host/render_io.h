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
// Renders every camera of this rank's share and writes <output_dir>/<name>.rgba8 (+ .depth.f32). Returns the count.
int render_headless(const std::string& splat_path, const std::string& cameras_path, const std::string& output_dir, const HeadlessOptions& opt);

}  // namespace b2c
