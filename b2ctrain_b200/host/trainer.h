// One optimisation step of the reference's trainer (the body of train_phase, src/train/trainer.cpp:452-529) as a C++
// class over the operator mirror of b2c_api.h, extended the two ways the reference's design allows but does not use:
// several views of a step in flight on separate streams, and view-level data parallelism over the GPUs of one node.
//
//   * rank r of `world` renders the views r, r + world, ... of a step; every rank holds a full model replica;
//   * each view's projection backward ADDS into a dense accumulator grad[n][11 + 3K] (the layout of the reference's
//     OptimParams::grad_out lane, src/gpu/optim.cu:292-297);
//   * update: with one rank, b2k_adam from the accumulator (or, for a single-view step, the reference's fused
//     optimizer_step); with several ranks either ncclAllReduce + the identical Adam everywhere, or the sharded update
//     (b2k_dp_adam_shard): each rank sums its slice of rows from all ranks through peer memory, updates it and writes
//     the new parameters into every replica.
// Step loss = sum of the per-view losses, whose gradient is the summed accumulator.
#pragma once
#include <memory>
#include "b2c_api.h"
#include "refine.h"

namespace b2c {

struct StepConfig {
  int views_in_flight = 4;        // views of a step processed concurrently, each with its own stream and RenderCtx
  int render_chunks = 1;          // > 1: render front to back in this many depth chunks (b2k_render_chunked)
  size_t isect_cap = 0;           // starting capacity of the intersection buffers (0 = the reference's 2^22)
  float ssim_weight = 0.2f;       // l1_w = 1 - ssim_weight, ssim_w = -ssim_weight (trainer.cpp:493)
  bool mask = false, alpha_lane = false, composite = false;
  float match_alpha_weight = 0.1f, loss_scale = 1.f;
  float bg[3] = {0.f, 0.f, 0.f};
  float lr_mean = 0.f, lr_rot = 2e-3f, lr_scale = 5e-3f, lr_opac = 0.012f, lr_dc = 2e-3f, lr_sh_rest = 2e-4f;
  bool sparse = true;
  float noise_weight = 0.f, noise_clamp = 0.f;   // MCMC noise (trainer.cpp:524)
  uint32_t seed = 42;
  bool shard_update = true;       // several ranks: sharded update over peer memory instead of all-reduce + replicated Adam
};

// A training view: camera and packed RGBA8 target, resident on the device and (optionally) in pinned host memory, from
// where a step can stream it in (the end-to-end measurement).
struct StepView {
  Camera cam;
  DevBuf<uint32_t> rgba;
  PinnedBuf<uint32_t> host_rgba;
};

class StepTrainer {
 public:
  // Collective over the ranks when world > 1 (dp_id = the 128 bytes of b2k_dp_unique_id made by rank 0).
  StepTrainer(const SplatCloud& cloud, int W, int H, const StepConfig& cfg, int rank = 0, int world = 1, const uint8_t* dp_id = nullptr);
  ~StepTrainer();
  StepTrainer(const StepTrainer&) = delete;
  StepTrainer& operator=(const StepTrainer&) = delete;

  int add_view(const Camera& cam, const uint32_t* rgba);   // returns the view's index; every rank registers the views it will render
  // Views of a step this rank takes: positions rank, rank + world, ... of `views`.
  std::vector<int> my_share(const std::vector<int>& views) const;
  // One step over `views` (indices from add_view, the whole step's list on every rank). Work is enqueued on `stream`
  // and on the lanes' own streams, which are joined back into `stream` before the update; the call returns after one
  // host readback per step (the lanes' largest intersection totals), having redone the views with larger buffers if one
  // did not fit. from_host: targets are copied in from pinned memory, double-buffered on a copy stream.
  void step(const std::vector<int>& views, cudaStream_t stream, bool from_host = false);
  // loss_accum of lane 0 after the last step: [0] last view's loss, [2] sum over this rank's views, [3] their count.
  void read_loss(float* out16, cudaStream_t stream);
  // The refinement statistics made global over the ranks (max: refine_norm, max_screen; sum: vis_count, vis_weight).
  void reduce_statistics(cudaStream_t stream);
  // The refinement pass between steps (RefineState::run, src/gpu/refine.cu:244-342) on every rank's replica: first the
  // optimizer state of every splat is made whole on every rank (after the sharded update only its owner holds it) and the
  // statistics are reduced over the ranks; the pass itself is deterministic, so the replicas stay identical without any
  // further exchange. Buffers that grew are shared again and the gradient accumulator follows the new count.
  RefineStats refine(const RefineParams& p, cudaStream_t stream);
  RefineState refiner;
  // Sum of all parameter words of the replica as 64-bit integers: equal on every rank when the replicas are identical.
  uint64_t replica_checksum(cudaStream_t stream);

  Model model;
  std::vector<std::unique_ptr<RenderCtx>> ctxs;
  std::vector<std::unique_ptr<StepView>> views;
  DevBuf<float> grad;
  StepConfig cfg;
  int W, H, rank, world;
  uint32_t step_no = 0;
  int overflow_redos = 0;
  uint64_t h2d_bytes = 0;
  // Of the last step when `profile` is set: views, update, whole step; then the update's parts on several ranks: the barrier
  // before it (which also waits for the slowest rank's views), the sharded kernel, the barrier behind it.
  float phase_ms[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  bool profile = false;

 private:
  void run_views(const std::vector<int>& mine, cudaStream_t stream, bool from_host, bool fused);
  void view_pass(int lane, int view, int slot, cudaStream_t s, bool from_host, bool fused, bool first_of_lane);
  bool overflowed(cudaStream_t stream);
  void update(cudaStream_t stream);
  OptimParams optim_params(const CameraGPU& cam) const;
  const uint32_t* target(int view, int slot, cudaStream_t s, bool from_host);

  void share_buffers();
  size_t grad_words() const;
  uint32_t* touched();
  B2kDp* dp_ = nullptr;
  B2kDpPeers peers_{};
  std::vector<cudaStream_t> streams_;
  cudaStream_t copy_stream_ = nullptr, clear_stream_ = nullptr;
  std::vector<DevBuf<uint32_t>> stage_;
  std::vector<cudaEvent_t> staged_evt_, free_evt_, lane_done_;
  cudaEvent_t start_evt_ = nullptr, cleared_evt_ = nullptr, mark_[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  PinnedBuf<uint32_t> h_isect_;
  bool grad_clear_pending_ = false;
};

}  // namespace b2c
