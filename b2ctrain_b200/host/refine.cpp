// Host sequence of the refinement pass (RefineState::run, src/gpu/refine.cu:244-342) over the device steps of libb2k
// (csrc/refine.cu), this library's radix sort and its flagged selection. Counts come back to the host where the
// reference reads them back too (how many died, how many are oversized, how many lie above the growth threshold).
#include "refine.h"
#include <algorithm>
#include <cmath>

namespace b2c {
using namespace abi;

namespace {
// Indices of the set flags, in order, into `out`; returns how many (one readback).
uint32_t select_flagged(RefineState& st, const uint32_t* flags, int n, DevBuf<uint32_t>& out, cudaStream_t stream) {
  out.reserve((size_t)std::max(n, 1));
  st.select_tmp.reserve((size_t)b2k_select_tmp_words(n));
  check(b2k_select_flagged(flags, n, out.ptr, st.counts.ptr, st.select_tmp.ptr, stream), "refine: select");
  return st.counts.download(1, stream)[0];
}
void sort_pairs(RefineState& st, int n, cudaStream_t stream) {
  st.sort_tmp.reserve((size_t)b2k_sort_pairs_tmp_bytes());
  check(b2k_sort_pairs_u32(st.keys.ptr, st.vals.ptr, st.keys_alt.ptr, st.vals_alt.ptr, (uint32_t)n, st.sort_tmp.ptr, st.sort_tmp.count, stream), "refine: sort");
}
void copy_words(uint32_t* dst, const uint32_t* src, size_t count, cudaStream_t stream) {
  if (count) B2C_CUDA_CHECK(cudaMemcpyAsync(dst, src, count * sizeof(uint32_t), cudaMemcpyDeviceToDevice, stream));
}
}  // namespace

void RefineState::init(const Model&, cudaStream_t) { counts.reserve(8); }

void RefineState::set_cameras(const std::vector<float>& pos, const std::vector<float>& focal) {
  cam_pos.upload(pos); cam_focal.upload(focal); n_cams = (int)focal.size();
  B2C_CUDA_CHECK(cudaDeviceSynchronize());
}

void RefineState::update_min_scale(Model& m, cudaStream_t stream) {
  if (n_cams == 0 || m.n == 0) return;
  b2c::update_min_scale(m, cam_pos.ptr, cam_focal.ptr, n_cams, stream);
}

void RefineState::bake_min_scale(Model& m, cudaStream_t stream) {
  if (m.n == 0) return;
  const B2kModel mv = view_of(m);
  check(b2k_refine_bake_floor(&mv, stream), "bake_min_scale");
}

// Bounds = the central 80 % of the splats along each axis (refine.cu:187-212).
void RefineState::update_bounds(const Model& m, cudaStream_t stream) {
  const int n = m.n;
  if (n == 0) return;
  counts.reserve(8);
  keys.reserve((size_t)n); keys_alt.reserve((size_t)n); vals.reserve((size_t)n); vals_alt.reserve((size_t)n);
  const float percentile = 0.8f;
  const size_t lo = (size_t)((1.f - percentile) / 2.f * (float)n), hi = std::min<size_t>((size_t)n - 1, (size_t)((1.f + percentile) / 2.f * (float)n));
  const B2kModel mv = view_of(m);
  for (int a = 0; a < 3; a++) {
    check(b2k_refine_axis_keys(&mv, a, keys.ptr, vals.ptr, stream), "update_bounds");
    sort_pairs(*this, n, stream);
    uint32_t k[2];
    B2C_CUDA_CHECK(cudaMemcpyAsync(&k[0], keys.ptr + lo, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
    B2C_CUDA_CHECK(cudaMemcpyAsync(&k[1], keys.ptr + hi, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
    B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
    bounds.min[a] = b2k_key_to_float(k[0]); bounds.max[a] = b2k_key_to_float(k[1]);
    bounds.center[a] = 0.5f * (bounds.min[a] + bounds.max[a]); bounds.extent[a] = bounds.max[a] - bounds.min[a];
  }
}

RefineStats RefineState::run(Model& m, RenderCtx& ctx, const RefineParams& p, cudaStream_t stream) {
  RefineStats stats;
  last_pairs = 0;
  const int n = m.n;
  if (n == 0) return stats;
  refine_count++;
  counts.reserve(8);
  if (accumulate_min_scale) bake_min_scale(m, stream);
  if (bounds.extent[0] == 0.f) update_bounds(m, stream);
  const size_t nn = (size_t)n;
  for (DevBuf<uint32_t>* b : {&keep, &dead_flag, &selected, &above, &cull_flag, &keys, &keys_alt, &vals, &vals_alt}) b->reserve(nn);
  sel_parent.reserve(nn * 2 + 16); sel_child.reserve(nn * 2 + 16);
  B2kModel mv = view_of(m);
  // 1. Which splats die.
  check(b2k_refine_flags(&mv, bounds.center, bounds.max_extent() * 100.f, p.cull_weight, keep.ptr, dead_flag.ptr, cull_flag.ptr, stream), "refine: flags");
  const uint32_t n_dead = select_flagged(*this, dead_flag.ptr, n, dead_idx, stream);
  stats.pruned = (int)n_dead;
  if (p.cull_weight > 0.f) stats.culled = (int)select_flagged(*this, cull_flag.ptr, n, tmp_idx, stream);
  const uint32_t alive = (uint32_t)n - n_dead;
  selected.zero(stream, nn);
  uint32_t n_sel = 0;
  // 2a. Every dead slot is given to a survivor drawn by opacity among the visible ones.
  if (n_dead > 0 && alive > 0 && !p.no_new) {
    check(b2k_refine_sample_keys(&mv, keep.ptr, nullptr, 0, 0.f, p.seed ^ (p.iter * 2654435761u), keys.ptr, vals.ptr, nullptr, stream), "refine: keys");
    sort_pairs(*this, n, stream);
    const uint32_t take = std::min(n_dead, alive);
    copy_words(sel_parent.ptr, vals.ptr, take, stream);
    check(b2k_refine_mark(sel_parent.ptr, (int)take, selected.ptr, stream), "refine: mark");
    n_sel = take; stats.relocated = (int)take;
  }
  // 2b. Splats larger on screen than allowed are split, as far as the budget goes.
  if (p.split_at_screen_size > 0.f && !p.no_new) {
    check(b2k_refine_oversized(&mv, keep.ptr, selected.ptr, p.split_at_screen_size, above.ptr, stream), "refine: oversized");
    uint32_t n_over = select_flagged(*this, above.ptr, n, tmp_idx, stream);
    const uint32_t headroom = alive + n_sel < p.max_splats ? p.max_splats - alive - n_sel : 0;
    n_over = std::min(n_over, headroom);
    copy_words(sel_parent.ptr + n_sel, tmp_idx.ptr, n_over, stream);
    check(b2k_refine_mark(sel_parent.ptr + n_sel, (int)n_over, selected.ptr, stream), "refine: mark");
    n_sel += n_over; stats.split_oversized = (int)n_over;
  }
  // 2c. Growth where the view-space gradient is large: a fraction of those above the threshold, drawn by gradient.
  if (p.growth_allowed && !p.no_new) {
    check(b2k_refine_sample_keys(&mv, keep.ptr, selected.ptr, 1, p.growth_grad_threshold, p.seed ^ (p.iter * 40503u), keys.ptr, vals.ptr, above.ptr, stream), "refine: keys");
    const uint32_t n_above = select_flagged(*this, above.ptr, n, tmp_idx, stream);
    int64_t want = (int64_t)std::lround((double)n_above * p.growth_select_fraction) - (int64_t)n_dead;
    if (want < 0) want = 0;
    const uint32_t headroom = alive + n_sel < p.max_splats ? p.max_splats - alive - n_sel : 0;
    const uint32_t n_grow = std::min((uint32_t)std::min<int64_t>(want, headroom), n_above);
    if (n_grow) { sort_pairs(*this, n, stream); copy_words(sel_parent.ptr + n_sel, vals.ptr, n_grow, stream); }
    n_sel += n_grow; stats.grown = (int)n_grow;
  }
  // 3. Children: into the dead slots first, then appended.
  const uint32_t from_dead = std::min(n_dead, n_sel);
  if (n_sel > 0) {
    const uint32_t appended = n_sel - from_dead;
    const int new_n = n + (int)appended;
    if (new_n > m.cap) m.reserve(new_n, stream);
    if (m.cap > (int)ctx.tile_count.count) ctx.setup(ctx.W, ctx.H, m.cap, stream);
    if (appended) B2C_CUDA_CHECK(cudaMemsetAsync(ctx.tile_count.ptr + n, 0, appended * sizeof(uint32_t), stream));
    mv = view_of(m);   // the buffers may have moved
    check(b2k_refine_split(&mv, ctx.tile_count.ptr, sel_parent.ptr, dead_idx.ptr, (int)from_dead, (int)n_sel, p.split_at_screen_size, sel_child.ptr, stream), "refine: split");
    last_pairs = n_sel;
    m.n = new_n;
    mv = view_of(m);
  }
  if (n_dead > from_dead) check(b2k_refine_kill(&mv, dead_idx.ptr + from_dead, (int)(n_dead - from_dead), stream), "refine: kill");
  // 4. Opacity decay, fading out over the run.
  const float t = std::min(std::max((float)p.iter / (float)std::max(1u, p.total), 0.f), 1.f);
  check(b2k_refine_opacity_decay(&mv, p.opac_decay * (1.f - t), stream), "refine: decay");
  // 5. Bounds and floor; 6. the statistics start over.
  update_bounds(m, stream);
  if ((float)p.iter / (float)std::max(1u, p.total) < 0.9f) update_min_scale(m, stream);
  m.zero_stats(stream);
  return stats;
}

}  // namespace b2c
