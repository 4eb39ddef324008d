// StepTrainer: see trainer.h. The sequence per view is the reference's (src/train/trainer.cpp:487-529): render_forward,
// photometric_loss, accumulate_loss, rasterize_backward, then the optimizer (fused for a single-view step, split into
// projection backward + one update per step otherwise).
#include "trainer.h"
#include <algorithm>
#include <cstring>

namespace b2c {
using namespace abi;

namespace {
void cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": CUDA error " + cudaGetErrorString(e));
}
}  // namespace

StepTrainer::StepTrainer(const SplatCloud& cloud, int W_, int H_, const StepConfig& cfg_, int rank_, int world_, const uint8_t* dp_id)
    : cfg(cfg_), W(W_), H(H_), rank(rank_), world(world_) {
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("StepTrainer: bad rank / world");
  model.upload(cloud);
  const int lanes = std::max(1, cfg.views_in_flight);
  for (int l = 0; l < lanes; l++) {
    ctxs.emplace_back(new RenderCtx());
    RenderCtx& c = *ctxs.back();
    c.n_chunks = std::max(1, cfg.render_chunks);
    if (cfg.isect_cap) alloc_isect(c, cfg.isect_cap);
    c.setup(W, H, model.cap, 0);
    c.loss_accum.zero(0);
    cudaStream_t s = nullptr;
    cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "stream");
    streams_.push_back(s);
    cudaEvent_t e = nullptr;
    cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "event");
    lane_done_.push_back(e);
  }
  cuda(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking), "stream");
  cuda(cudaStreamCreateWithFlags(&clear_stream_, cudaStreamNonBlocking), "stream");
  stage_.resize(2 * lanes);
  for (int i = 0; i < 2 * lanes; i++) {
    cudaEvent_t a = nullptr, b = nullptr;
    cuda(cudaEventCreateWithFlags(&a, cudaEventDisableTiming), "event");
    cuda(cudaEventCreateWithFlags(&b, cudaEventDisableTiming), "event");
    staged_evt_.push_back(a); free_evt_.push_back(b);
  }
  cuda(cudaEventCreateWithFlags(&start_evt_, cudaEventDisableTiming), "event");
  cuda(cudaEventCreateWithFlags(&cleared_evt_, cudaEventDisableTiming), "event");
  for (auto& m : mark_) cuda(cudaEventCreate(&m), "event");
  h_isect_.reserve((size_t)lanes);
  grad.reserve(grad_words());
  grad.zero(0);
  cuda(cudaDeviceSynchronize(), "setup");
  if (world > 1) {
    if (!dp_id) throw std::runtime_error("StepTrainer: several ranks need the rendezvous id of rank 0");
    check(b2k_dp_init(&dp_, dp_id, rank, world), "b2k_dp_init");
    if (cfg.shard_update) share_buffers();
  }
  refiner.init(model, 0);
}

// The accumulator [n][11 + 3K], followed by the bitmap of the splats that received a row this step (one allocation, so
// that the peers reach both through one mapping).
size_t StepTrainer::grad_words() const {
  const size_t n = (size_t)std::max(model.n, 1);
  return n * (11 + 3 * (size_t)model.K()) + (n + 31) / 32;
}
uint32_t* StepTrainer::touched() { return reinterpret_cast<uint32_t*>(grad.ptr + (size_t)std::max(model.n, 1) * (11 + 3 * (size_t)model.K())); }

void StepTrainer::share_buffers() {
  check(b2k_dp_share(dp_, grad.ptr, (void**)peers_.grad, 0), "b2k_dp_share(grad)");
  for (int r = 0; r < world; r++) peers_.touched[r] = reinterpret_cast<const uint32_t*>(peers_.grad[r] + (size_t)std::max(model.n, 1) * (11 + 3 * (size_t)model.K()));
  check(b2k_dp_share(dp_, model.pos_op.ptr, (void**)peers_.pos_op, 0), "b2k_dp_share(pos_op)");
  check(b2k_dp_share(dp_, model.quat.ptr, (void**)peers_.quat, 0), "b2k_dp_share(quat)");
  check(b2k_dp_share(dp_, model.lscale.ptr, (void**)peers_.lscale, 0), "b2k_dp_share(lscale)");
  check(b2k_dp_share(dp_, model.sh_dc.ptr, (void**)peers_.sh_dc, 0), "b2k_dp_share(sh_dc)");
  check(b2k_dp_share(dp_, model.sh_hi32.ptr, (void**)peers_.sh_hi, 0), "b2k_dp_share(sh_hi)");
}

RefineStats StepTrainer::refine(const RefineParams& p, cudaStream_t stream) {
  const bool sharded = world > 1 && cfg.shard_update;
  if (grad_clear_pending_) { cuda(cudaStreamWaitEvent(stream, cleared_evt_, 0), "wait"); grad_clear_pending_ = false; }
  if (sharded) {   // moments, the Adam-mini second moment and the lazy-update stamp: whole on every rank again
    const int n = model.n, hi = (model.K() - 1) * 3;
    for (DevBuf<float4>* b : {&model.m_pos_op, &model.v_pos_op, &model.m_quat, &model.v_quat, &model.m_lscale, &model.v_lscale})
      check(b2k_dp_gather_slices(dp_, b->ptr, 16, 1, (uint64_t)model.cap, n, stream), "b2k_dp_gather_slices");
    check(b2k_dp_gather_slices(dp_, model.m_sh_dc.ptr, 4, 3, (uint64_t)model.cap, n, stream), "b2k_dp_gather_slices");
    check(b2k_dp_gather_slices(dp_, model.m_sh_hi32.ptr, 4, hi, (uint64_t)model.cap, n, stream), "b2k_dp_gather_slices");
    check(b2k_dp_gather_slices(dp_, model.v_sh.ptr, 4, 1, (uint64_t)model.cap, n, stream), "b2k_dp_gather_slices");
    check(b2k_dp_gather_slices(dp_, model.last_step.ptr, 4, 1, (uint64_t)model.cap, n, stream), "b2k_dp_gather_slices");
  }
  reduce_statistics(stream);
  const int n_before = model.n;
  const void* before[2] = {model.pos_op.ptr, model.sh_hi32.ptr};
  if (sharded) check(b2k_dp_release_shares(dp_, stream), "b2k_dp_release_shares");   // the pass may reallocate what the peers have mapped
  const RefineStats st = refiner.run(model, *ctxs[0], p, stream);
  for (size_t l = 1; l < ctxs.size(); l++) if (model.cap > ctxs[l]->n_cap) ctxs[l]->setup(W, H, model.cap, stream);
  if (model.n != n_before || model.pos_op.ptr != before[0] || model.sh_hi32.ptr != before[1]) {
    cuda(cudaStreamSynchronize(stream), "sync");
    grad.free();
    grad.reserve(grad_words());
  }
  grad.zero(stream);
  cuda(cudaStreamSynchronize(stream), "sync");
  if (sharded) share_buffers();
  return st;
}

StepTrainer::~StepTrainer() {
  cudaDeviceSynchronize();
  if (dp_) b2k_dp_destroy(dp_);
  for (cudaStream_t s : streams_) cudaStreamDestroy(s);
  if (copy_stream_) cudaStreamDestroy(copy_stream_);
  if (clear_stream_) cudaStreamDestroy(clear_stream_);
  for (cudaEvent_t e : lane_done_) cudaEventDestroy(e);
  for (cudaEvent_t e : staged_evt_) cudaEventDestroy(e);
  for (cudaEvent_t e : free_evt_) cudaEventDestroy(e);
  if (start_evt_) cudaEventDestroy(start_evt_);
  if (cleared_evt_) cudaEventDestroy(cleared_evt_);
  for (cudaEvent_t e : mark_) if (e) cudaEventDestroy(e);
}

int StepTrainer::add_view(const Camera& cam, const uint32_t* rgba) {
  views.emplace_back(new StepView());
  StepView& v = *views.back();
  v.cam = cam;
  const size_t P = (size_t)W * H;
  if (rgba) {
    v.host_rgba.reserve(P);
    std::memcpy(v.host_rgba.ptr, rgba, P * sizeof(uint32_t));
    v.rgba.upload(v.host_rgba.ptr, P, 0);
    cuda(cudaStreamSynchronize(0), "add_view");
  }
  return (int)views.size() - 1;
}

std::vector<int> StepTrainer::my_share(const std::vector<int>& all) const {
  std::vector<int> mine;
  for (size_t j = (size_t)rank; j < all.size(); j += (size_t)world) mine.push_back(all[j]);
  return mine;
}

OptimParams StepTrainer::optim_params(const CameraGPU& cam) const {
  OptimParams op;
  op.cam = cam; op.active_sh_degree = model.degree; op.t = model.adam_t;
  op.lr_mean = cfg.lr_mean; op.lr_rot = cfg.lr_rot; op.lr_scale = cfg.lr_scale; op.lr_opac = cfg.lr_opac; op.lr_dc = cfg.lr_dc; op.lr_sh_rest = cfg.lr_sh_rest;
  op.noise_weight = cfg.noise_weight; op.noise_clamp = cfg.noise_clamp; op.seed = cfg.seed; op.step = step_no; op.sparse = cfg.sparse;
  return op;
}

const uint32_t* StepTrainer::target(int view, int slot, cudaStream_t s, bool from_host) {
  StepView& v = *views[view];
  if (!from_host) return v.rgba.ptr;
  const size_t P = (size_t)W * H;
  DevBuf<uint32_t>& dst = stage_[slot];
  dst.reserve(P);
  cuda(cudaStreamWaitEvent(copy_stream_, free_evt_[slot], 0), "wait");      // the loss that read this slot last has run
  cuda(cudaMemcpyAsync(dst.ptr, v.host_rgba.ptr, P * sizeof(uint32_t), cudaMemcpyHostToDevice, copy_stream_), "target copy");
  cuda(cudaEventRecord(staged_evt_[slot], copy_stream_), "record");
  cuda(cudaStreamWaitEvent(s, staged_evt_[slot], 0), "wait");
  h2d_bytes += P * sizeof(uint32_t);
  return dst.ptr;
}

void StepTrainer::view_pass(int lane, int view, int slot, cudaStream_t s, bool from_host, bool fused, bool first_of_lane) {
  RenderCtx& ctx = *ctxs[lane];
  RenderParams rp;
  rp.cam = CameraGPU::from(views[view]->cam, W, H);
  for (int k = 0; k < 3; k++) rp.bg[k] = cfg.bg[k];
  rp.sh_degree = model.degree; rp.bwd_info = true;
  { const B2kCtx cv = view_of(ctx); check(b2k_loss_zero(&cv, 0, 2, s), "loss_accum.zero"); }
  render_forward_async(ctx, model, rp, s);
  ViewGPU vg; vg.rgba = target(view, slot, s, from_host); vg.W = W; vg.H = H;
  LossParams lp;
  lp.l1_w = 1.f - cfg.ssim_weight; lp.ssim_w = -cfg.ssim_weight;
  for (int k = 0; k < 3; k++) lp.bg[k] = cfg.bg[k];
  lp.composite = cfg.composite; lp.mask = cfg.mask; lp.alpha_lane = cfg.alpha_lane; lp.match_alpha_weight = cfg.match_alpha_weight; lp.scale = cfg.loss_scale;
  photometric_loss(ctx, vg, lp, s);
  if (from_host) cuda(cudaEventRecord(free_evt_[slot], s), "record");
  accumulate_loss(ctx, s);
  rasterize_backward(ctx, model, rp, s);
  const OptimParams op = optim_params(rp.cam);
  if (fused) { optimizer_step(ctx, model, op, s); return; }
  if (first_of_lane && grad_clear_pending_) cuda(cudaStreamWaitEvent(s, cleared_evt_, 0), "wait");   // the accumulator of the last step has been cleared
  projection_backward(ctx, model, op, grad.ptr, s, world > 1 && cfg.shard_update ? touched() : nullptr);
}

void StepTrainer::run_views(const std::vector<int>& mine, cudaStream_t stream, bool from_host, bool fused) {
  for (auto& c : ctxs) step_begin(*c, stream);   // every lane, also the ones that get no view this step
  if (fused) { view_pass(0, mine[0], 0, stream, from_host, true, true); return; }
  const int lanes = (int)ctxs.size();
  if (lanes == 1) {
    for (size_t j = 0; j < mine.size(); j++) view_pass(0, mine[j], (int)(j & 1), stream, from_host, false, j == 0);
    return;
  }
  cuda(cudaEventRecord(start_evt_, stream), "record");
  for (size_t j = 0; j < mine.size(); j++) {
    const int lane = (int)(j % (size_t)lanes);
    if (j < (size_t)lanes) cuda(cudaStreamWaitEvent(streams_[lane], start_evt_, 0), "wait");
    view_pass(lane, mine[j], 2 * lane + (int)((j / (size_t)lanes) & 1), streams_[lane], from_host, false, j < (size_t)lanes);
  }
  const int used = (int)std::min((size_t)lanes, mine.size());
  for (int lane = 0; lane < used; lane++) {
    cuda(cudaEventRecord(lane_done_[lane], streams_[lane]), "record");
    cuda(cudaStreamWaitEvent(stream, lane_done_[lane], 0), "wait");
  }
  for (int lane = 1; lane < used; lane++) fold_loss(*ctxs[0], *ctxs[lane], stream);
}

bool StepTrainer::overflowed(cudaStream_t stream) {
  for (size_t l = 0; l < ctxs.size(); l++)
    cuda(cudaMemcpyAsync(h_isect_.ptr + l, ctxs[l]->d_num_isect.ptr + 2, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream), "readback");
  cuda(cudaStreamSynchronize(stream), "sync");
  bool over = false;
  for (size_t l = 0; l < ctxs.size(); l++) over = grow_intersections(*ctxs[l], h_isect_.ptr[l]) || over;
  return over;
}

void StepTrainer::update(cudaStream_t stream) {
  const OptimParams op = optim_params(CameraGPU{});
  const B2kModel mv = view_of(model);
  const B2kOptim o = optim_of(op, "adam_step");
  if (world == 1) { check(b2k_adam(&mv, &o, grad.ptr, stream), "b2k_adam"); return; }
  if (!cfg.shard_update) {
    check(b2k_dp_allreduce_grads(dp_, grad.ptr, (uint64_t)model.n * (11 + 3 * (uint64_t)model.K()), stream), "b2k_dp_allreduce_grads");
    check(b2k_adam(&mv, &o, grad.ptr, stream), "b2k_adam");
    return;
  }
  check(b2k_dp_barrier(dp_, stream), "b2k_dp_barrier");          // every rank's accumulator is complete
  if (profile) cuda(cudaEventRecord(mark_[3], stream), "record");
  check(b2k_dp_adam_shard(dp_, &mv, &o, &peers_, stream), "b2k_dp_adam_shard");
  if (profile) cuda(cudaEventRecord(mark_[4], stream), "record");
  check(b2k_dp_barrier(dp_, stream), "b2k_dp_barrier");          // every replica is written, every accumulator read
  // This rank's accumulator is cleared beside the start of the next step; the first projection backward waits for it.
  cuda(cudaEventRecord(start_evt_, stream), "record");
  cuda(cudaStreamWaitEvent(clear_stream_, start_evt_, 0), "wait");
  grad.zero(clear_stream_);
  cuda(cudaEventRecord(cleared_evt_, clear_stream_), "record");
  grad_clear_pending_ = true;
}

void StepTrainer::step(const std::vector<int>& all, cudaStream_t stream, bool from_host) {
  if (all.empty()) return;
  model.adam_t++;
  step_no++;
  const std::vector<int> mine = my_share(all);
  const bool fused = world == 1 && all.size() == 1;
  if (profile) cuda(cudaEventRecord(mark_[0], stream), "record");
  for (;;) {
    if (!mine.empty()) run_views(mine, stream, from_host, fused); else for (auto& c : ctxs) step_begin(*c, stream);
    if (!overflowed(stream)) break;
    overflow_redos++;
    if (!fused) {
      if (grad_clear_pending_) cuda(cudaStreamWaitEvent(stream, cleared_evt_, 0), "wait");
      grad.zero(stream);
    }
  }
  if (profile) cuda(cudaEventRecord(mark_[1], stream), "record");
  if (!fused) update(stream);
  if (profile) {
    cuda(cudaEventRecord(mark_[2], stream), "record");
    cuda(cudaEventSynchronize(mark_[2]), "sync");
    cudaEventElapsedTime(&phase_ms[0], mark_[0], mark_[1]);
    cudaEventElapsedTime(&phase_ms[1], mark_[1], mark_[2]);
    cudaEventElapsedTime(&phase_ms[2], mark_[0], mark_[2]);
    phase_ms[3] = phase_ms[4] = phase_ms[5] = 0.f;
    if (!fused && world > 1 && cfg.shard_update) {
      cudaEventElapsedTime(&phase_ms[3], mark_[1], mark_[3]);
      cudaEventElapsedTime(&phase_ms[4], mark_[3], mark_[4]);
      cudaEventElapsedTime(&phase_ms[5], mark_[4], mark_[2]);
    }
  }
}

void StepTrainer::read_loss(float* out16, cudaStream_t stream) {
  cuda(cudaMemcpyAsync(out16, ctxs[0]->loss_accum.ptr, 16 * sizeof(float), cudaMemcpyDeviceToHost, stream), "loss readback");
  cuda(cudaStreamSynchronize(stream), "sync");
}

void StepTrainer::reduce_statistics(cudaStream_t stream) {
  if (world == 1) return;
  check(b2k_dp_allreduce_stat(dp_, model.refine_norm.ptr, (uint64_t)model.n, 1, stream), "refine_norm");
  check(b2k_dp_allreduce_stat(dp_, model.max_screen.ptr, (uint64_t)model.n, 1, stream), "max_screen");
  check(b2k_dp_allreduce_stat(dp_, model.vis_count.ptr, (uint64_t)model.n, 0, stream), "vis_count");
  check(b2k_dp_allreduce_stat(dp_, model.vis_weight.ptr, (uint64_t)model.n, 0, stream), "vis_weight");
}

uint64_t StepTrainer::replica_checksum(cudaStream_t stream) {
  uint64_t sum = 0;
  auto add = [&](const void* p, size_t bytes) {
    std::vector<uint32_t> h(bytes / 4);
    cuda(cudaMemcpyAsync(h.data(), p, bytes, cudaMemcpyDeviceToHost, stream), "checksum");
    cuda(cudaStreamSynchronize(stream), "sync");
    for (uint32_t w : h) sum += w;
  };
  add(model.pos_op.ptr, (size_t)model.n * 16); add(model.quat.ptr, (size_t)model.n * 16); add(model.lscale.ptr, (size_t)model.n * 16);
  add(model.sh_dc.ptr, (size_t)model.cap * 12);
  if (model.K() > 1) add(model.sh_hi32.ptr, (size_t)model.cap * 12 * (size_t)(model.K() - 1));
  return sum;
}

}  // namespace b2c
