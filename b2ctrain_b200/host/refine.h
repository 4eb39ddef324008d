// RefineParams / RefineStats / RefineState with the reference's names (src/gpu/refine.h:8-44): the density-control pass
// that runs between training steps. Under view-level data parallelism every rank holds the same model and, after
// StepTrainer::reduce_statistics(), the same statistics; every draw is a counter hash of (seed, iteration, splat), so
// the pass is deterministic and every rank prunes, relocates, splits and grows identically without further exchange.
#pragma once
#include "b2c_api.h"

namespace b2c {

// src/train/init.h:11.
struct Bounds {
  float min[3] = {0, 0, 0}, max[3] = {0, 0, 0}, center[3] = {0, 0, 0}, extent[3] = {0, 0, 0};
  float max_extent() const { return std::fmax(extent[0], std::fmax(extent[1], extent[2])); }
};

struct RefineParams {
  uint32_t iter = 0, total = 30000;
  bool growth_allowed = true;
  uint32_t max_splats = 10000000;
  float growth_grad_threshold = 0.0025f, growth_select_fraction = 0.25f;
  float split_at_screen_size = 0.5f;
  float opac_decay = 0.004f;
  uint32_t seed = 42;
  bool no_new = false;
  float cull_weight = 0.f;
};
struct RefineStats { int pruned = 0, relocated = 0, grown = 0, split_oversized = 0, culled = 0; };

struct RefineState {
  Bounds bounds{};
  bool accumulate_min_scale = false;
  DevBuf<float> cam_pos, cam_focal; int n_cams = 0;
  DevBuf<uint32_t> keep, dead_flag, dead_idx, selected, above, tmp_idx, sel_parent, sel_child, cull_flag;
  DevBuf<uint32_t> keys, keys_alt, vals, vals_alt, counts, select_tmp;
  DevBuf<unsigned char> sort_tmp;
  int refine_count = 0;
  uint32_t last_pairs = 0;   // sel_parent[k] -> sel_child[k], k < last_pairs: the splats the last run() wrote from a parent

  void init(const Model& m, cudaStream_t stream);
  void set_cameras(const std::vector<float>& pos, const std::vector<float>& focal);
  void update_min_scale(Model& m, cudaStream_t stream);
  void bake_min_scale(Model& m, cudaStream_t stream);
  RefineStats run(Model& m, RenderCtx& ctx, const RefineParams& p, cudaStream_t stream);
  void update_bounds(const Model& m, cudaStream_t stream);
};

}  // namespace b2c
