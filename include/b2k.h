/* b2k: C ABI of the B200 (sm_100a) splat render-and-backprop path.
 *
 * This is the drop-in boundary: every entry point takes plain structs of raw device pointers and sizes, enqueues its
 * kernels on the caller's CUDA stream and returns an int status (0 = B2K_OK). Nothing here allocates device memory:
 * the caller (the C++ mirror of the reference's host API under b2ctrain_b200/host/, or the ctypes wrapper) owns and
 * sizes every buffer. Each declaration cites the reference interface it stands in for (path:line in the b2ctrain
 * tree).
 */
#ifndef B2K_H
#define B2K_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b2k_stream_t; /* a cudaStream_t */

enum {
  B2K_OK = 0,
  B2K_ERR_ARG = 1,          /* null pointer, bad size, bad degree */
  B2K_ERR_CAPACITY = 2,     /* a caller-provided buffer is too small (message names it) */
  B2K_ERR_UNSUPPORTED = 3,  /* an optional lane of the reference API that this library does not implement */
  B2K_ERR_CUDA = 4,         /* a CUDA runtime call failed; b2k_last_cuda_error() has the code */
  B2K_ERR_OVERFLOW = 5      /* more tile intersections than the intersection buffers hold; grow and redo the view */
};

/* CameraGPU, src/gpu/render.h:10-24 (same fields, same order). */
typedef struct {
  float R[9];
  float t[3];
  float pos[3];
  float fx, fy, cx, cy;
  int32_t W, H;
  float lim_pos_x, lim_pos_y, lim_neg_x, lim_neg_y;
} B2kCamera;

/* Device buffers of Model, src/model.h:14-40. SH is planar: lane (k*3+ch) of splat i lives at sh_dc[lane*cap + i] for
 * lanes 0..2 and at sh_hi[(lane-3)*cap + i] above (fp32; the reference's optional fp16 storage is not implemented).
 * Moment and statistic pointers may be NULL for forward-only use. float4 buffers are passed as float*. */
typedef struct {
  int32_t n, cap, degree;
  float* pos_op;  /* [cap][4] x, y, z, opacity logit */
  float* quat;    /* [cap][4] w, x, y, z (unnormalised) */
  float* lscale;  /* [cap][4] log sx, log sy, log sz, 3D-filter floor f */
  float* sh_dc;   /* [3][cap] */
  float* sh_hi;   /* [3(K-1)][cap] */
  float *m_pos_op, *v_pos_op, *m_quat, *v_quat, *m_lscale, *v_lscale; /* Adam moments, [cap][4] each */
  float *m_sh_dc, *m_sh_hi; /* first moments of SH, planar like the parameters */
  float* v_sh;              /* [cap] Adam-mini second moment, one per splat */
  float *refine_norm, *max_screen, *vis_count, *vis_weight; /* [cap] refine statistics */
  uint32_t* last_step;      /* [cap] lazy sparse Adam bookkeeping */
} B2kModel;

/* Per-view scratch of RenderCtx, src/gpu/render.h:66-95. Names, element types and index meaning follow the
 * reference members that its callers read directly. */
typedef struct {
  int32_t W, H, tiles_x, tiles_y, n_tiles, tile_bits;
  int32_t n_cap;           /* per-splat buffers hold this many entries */
  float* proj0;            /* [n][4] mean2d x, y, conic c00, c01 */
  float* proj1;            /* [n][4] conic c11, opacity, view depth z, power = ln(255 opacity); power = -1: no record */
  float* proj2;            /* [n][4] r, g, b, feature x (0 without a feature mode) */
  uint32_t* tile_count;    /* [n] tiles hit */
  uint32_t* hit_info;      /* [n][4] bit mask (lo, hi) of the hit tiles inside the splat's tile box, row-major; packed box
                              min_x | min_y << 12 | width << 24; unused. Boxes above 64 tiles carry box = 0xFFFFFFFF and are
                              re-tested when emitted (the reference keeps a 32-tile mask, src/gpu/project.cu:33-43) */
  uint32_t* depth_keys;    /* [n] scratch of the depth sort */
  uint32_t* depth_keys_sorted; /* [n] b2k_project leaves the unsorted keys here; b2k_bin_sort sorts them in place */
  uint32_t* order_in;      /* [n] scratch of the depth sort */
  uint32_t* order;         /* [n] after b2k_project: identity; after b2k_bin_sort: splat index by depth rank (culled last) */
  uint32_t* tile_off;      /* [n] inclusive scan of tile counts in depth order */
  uint32_t *keys, *vals, *keys_sorted, *vals_sorted; /* [isect_cap] tile id / splat index before and after the tile sort */
  uint64_t isect_cap;
  uint32_t* num_isect;     /* [4] device words: [0] intersections of this view (may exceed isect_cap: overflow);
                              [1] entries of vis_list; [2] largest [0] since the caller cleared it (b2k_loss_accumulate) */
  void* sort_tmp;          /* scratch of b2k_sort_tmp_bytes() bytes */
  uint64_t sort_tmp_bytes;
  uint32_t* tile_ranges;   /* [n_tiles][2] start, end into vals_sorted; end shrunk by the forward when bwd_info
                              ([n_chunks][n_tiles][2] when n_chunks > 1) */
  float* out_rgba;         /* [P][4] */
  float* out_feat;         /* [P][4] composited feature lanes x, y, z (zero without a feature mode), w = final transmittance */
  float* out_depth;        /* [P] expected depth, or NULL: sum(vis z) / alpha where alpha > 0.05 else +inf (the mean-depth
                              mode of probe_kernel, src/gpu/probe.cu:30-46, fused into the forward) */
  uint32_t* last_idx;      /* [P] one past the last contributing sorted index */
  float* v_splat;          /* [n][13] screen-space gradient lanes, accumulated; cleared by the optimizer */
  uint32_t* vis_flag;      /* [n] set by the backward for splats that contributed; cleared by the optimizer */
  uint32_t* vis_list;      /* [n] scratch or NULL. When present, the sparse optimizer entry points first compact the set
                              visibility flags into this list (count in num_isect[1]) and then walk only those splats
                              instead of all n. */
  float* v_out;            /* [P][4] dL/d(rgba) */
  float* loss_accum;       /* [16] */
  int32_t n_chunks;        /* 0 or 1: the view is binned whole, as the reference does. 2..5: b2k_render_chunked renders it
                              front to back in this many depth chunks; tile_ranges then holds [n_chunks][n_tiles][2] (one
                              range per chunk and tile, indices into vals_sorted) and b2k_raster_bwd walks them all */
  float* proj3;            /* [n][2] feature lanes y, z (x rides in proj2.w), render.h:70; NULL unless a feature mode is used */
  uint32_t* chunk_words;   /* [32 + n_tiles + (tiles_x + 1)(tiles_y + 1)] device scratch of b2k_render_chunked (chunk windows
                              and counts, one "some pixel can still take a fragment" flag per tile, the summed-area table
                              of those flags), or NULL when n_chunks <= 1 */
  void* bwd_scratch;       /* b2k_bwd_scratch_bytes() bytes, needed when the forward runs with bwd_info: per-pixel (colour
                              sums, transmittance) checkpoints the forward leaves every 128 fragments of a tile's list, and
                              the work list of the backward, which replays the segments between checkpoints independently.
                              Takes the place of nothing in the reference (its backward walks a tile's list in one CTA) */
  uint64_t bwd_scratch_bytes;
} B2kCtx;

/* RenderParams, src/gpu/render.h:29-63: the fields this path implements. */
typedef struct {
  float bg[3];
  int32_t sh_degree;                /* active degree <= model degree */
  int32_t bwd_info;
  const float* pos_override;        /* [n][4] or NULL (render.h:42) */
  const float* quat_override;       /* render.h:46 */
  const float* lscale_override;     /* render.h:47 */
  int32_t feat_mode;                /* FeatureMode (render.h:27,33): 0 none, 1 pseudo-normals (shortest-scale axis, camera
                                       facing, camera space; project.cu:63-72), 2 per-splat buffer (project.cu:73-77).
                                       Forward only: the backward of the feature lanes is not implemented. Needs
                                       ctx->proj3; with b2k_render_chunked also ctx->bwd_scratch (16 bytes per pixel) and
                                       bwd_info = 0 */
  const float* feat_buffer;         /* [n][3] when feat_mode == 2 (render.h:34) */
} B2kRenderOpts;

/* ViewGPU + LossParams, src/gpu/loss.h:7-30. */
typedef struct {
  const uint32_t* rgba;    /* packed RGBA8 target */
  const uint8_t* weights;  /* per-pixel loss weight or NULL */
  float l1_w, ssim_w;
  float bg[3];
  int32_t composite, mask, alpha_lane;
  float match_alpha_weight, scale, grad_scale;
} B2kLoss;

/* OptimParams, src/gpu/optim.h:6-45: the fields this path implements. */
typedef struct {
  int32_t active_sh_degree;
  int32_t t;
  float beta1, beta2, eps;
  float lr_mean, lr_rot, lr_scale, lr_opac, lr_dc, lr_sh_rest;
  float noise_weight, noise_clamp;
  uint32_t seed, step;
  int32_t sparse;
  const float* pos_override;
  const float* quat_override;
  const float* lscale_override;
  float* grad_out;         /* [n][11+3K]: write parameter gradients and skip the update (optim.h:44) */
  uint32_t* touched_out;   /* NULL, or a bitmap of (n + 31) / 32 words beside the accumulator of b2k_proj_bwd: bit i is set when a
                              row is added for splat i, so that a reader can skip the rows that are still zero (no counterpart
                              in the reference) */
} B2kOptim;

/* ---- forward ---- */
/* project_splats, src/gpu/render.h:101 (project_kernel, src/gpu/project.cu:9-84). */
int b2k_project(const B2kModel* m, const B2kCamera* cam, const B2kRenderOpts* opts, const B2kCtx* ctx, b2k_stream_t s);
/* The tile-decision half of project_kernel alone (src/gpu/project.cu:31-43 with depth_keys_kernel, src/gpu/binning.cu:10-15):
 * recomputes tile_count, hit_info and the depth sort input from the records already in ctx->proj0 / proj1 (proj1.w <
 * -0.5 = no record). Lets a caller bin records that came from elsewhere (a stage exposed for tests, like the
 * reference's, src/gpu/render.h:100). */
int b2k_count_tiles(const B2kCtx* ctx, int32_t n, b2k_stream_t s);
/* bin_and_sort, src/gpu/render.h:102 (src/gpu/binning.cu:109-145), without the host round trip: the intersection
 * total stays on the device in ctx->num_isect and the later stages read it there. */
int b2k_bin_sort(const B2kCtx* ctx, int32_t n, b2k_stream_t s);
/* b2k_bin_sort with CUDA events between its phases (measurement aid; waits for the stream). ms[10]: [0] depth sort,
 * [1] scan + emit, [2],[3] / [4],[5] / [6],[7] count+row-scan and scatter of tile-sort passes 0 / 1 / 2, [8] tile
 * ranges, [9] whole call. The role of the reference's StageTimer (src/train/trainer.cpp:57-73) at kernel granularity. */
int b2k_bin_sort_profile(const B2kCtx* ctx, int32_t n, b2k_stream_t s, float* ms);
/* The 4-byte count readback of binning.cu:125-127 as its own call: waits for the stream, returns the total and
 * B2K_ERR_OVERFLOW when it exceeds ctx->isect_cap (the caller grows the four buffers and redoes the view). */
int b2k_read_num_isect(const B2kCtx* ctx, b2k_stream_t s, uint32_t* total);
/* b2k_bin_sort for callers that cannot allocate device memory (no counterpart in the reference). Identical results
 * to b2k_bin_sort, but ctx->sort_tmp is ignored: the scratch is a fixed array inside the library, sized for contexts
 * with n_cap <= b2k_static_max_splats() (262,144; larger ones get B2K_ERR_CAPACITY). The first call on a device looks
 * the array's device address up (a synchronising runtime query): make that first call outside any stream capture.
 * All calls on a device share the one array, so two calls whose kernels overlap on the GPU (different streams or
 * threads) race; calls on one stream are safe. Nothing in it needs clearing by the caller.
 * Limits: only the binning scratch is covered. b2k_project and b2k_count_tiles keep the list of splats with large
 * tile boxes in ctx->sort_tmp and still need that buffer from the caller, so a host that cannot allocate at all has
 * to be handed a sort_tmp by whoever owns the memory, or feed this entry records it binned elsewhere. The address
 * looked up on the first call is cached per device ordinal: it is stale after cudaDeviceReset, and two host threads
 * making their first call on one device at once both look it up (harmless: they store the same value). */
int b2k_bin_sort_static(const B2kCtx* ctx, int32_t n, b2k_stream_t s);
uint32_t b2k_static_max_splats(void);
/* rasterize_forward, src/gpu/render.h:103 (raster_fwd_kernel, src/gpu/raster_fwd.cu:9-71). */
int b2k_raster_fwd(const B2kCtx* ctx, const B2kRenderOpts* opts, b2k_stream_t s);
/* render_forward (src/gpu/render.h:97) for dense scenes, with no counterpart in the reference, which always bins every
 * intersection of the view before compositing any: project, then bin + composite the splats in ctx->n_chunks chunks of
 * increasing depth (the nearest 1/4^(C-1) of the visible splats first, each chunk four times the one before). A
 * tile whose pixels have all reached the transmittance cutoff emits no intersections in later chunks, so most of a
 * dense view is never sorted. out_rgba, out_feat.w, out_depth and every gradient of the backward are bit-identical to
 * b2k_project + b2k_bin_sort + b2k_raster_fwd; what differs is the bookkeeping a caller can see: vals_sorted /
 * keys_sorted hold one sorted window per chunk (without the intersections that were skipped), tile_ranges one range
 * per chunk and tile, last_idx an index into that layout with bit 31 set on pixels that reached the cutoff,
 * out_feat.xyz the colour sums without the background (with a feature mode, forward only: the feature lanes, as in the
 * whole-view path; their running sums travel in ctx->bwd_scratch between chunks), num_isect[0] the slots used. Needs last_idx and chunk_words;
 * tile_off and depth_keys are scratch; tile_count holds each splat's
 * tile-box area (an upper bound of its hits: the ellipse-tile tests are made chunk by chunk, only for splats whose box
 * still holds a live tile). Overflow of the intersection buffers is reported like b2k_bin_sort's. */
int b2k_render_chunked(const B2kModel* m, const B2kCamera* cam, const B2kRenderOpts* opts, const B2kCtx* ctx, b2k_stream_t s);
/* Scratch bytes b2k_project and b2k_bin_sort need in ctx->sort_tmp for a context whose per-splat buffers hold n_cap
 * entries (replaces RenderCtx::cub_tmp, src/gpu/render.h:80). */
uint64_t b2k_sort_tmp_bytes(int32_t n_cap, uint64_t isect_cap);

/* ---- loss ---- */
/* photometric_loss, src/gpu/loss.h:33 (photometric_kernel, src/gpu/loss.cu:18-195). */
int b2k_loss_photometric(const B2kCtx* ctx, const B2kLoss* lp, b2k_stream_t s);
/* accumulate_loss, src/gpu/loss.h:37. Also folds this view's intersection total into the running maximum
 * ctx->num_isect[2] (when num_isect is set), which the caller clears at the start of a step. */
int b2k_loss_accumulate(const B2kCtx* ctx, b2k_stream_t s);
/* loss_accum[first .. first + count) = 0 on the stream (the reference's loss_accum.zero(stream, n), src/train/trainer.cpp:
 * 487-491, without a host library in between). */
int b2k_loss_zero(const B2kCtx* ctx, int32_t first, int32_t count, b2k_stream_t s);
/* Start of a training step on this context: loss_accum[0..16) = 0 and the running intersection maximum
 * num_isect[2] = 0 (the loss_accum.zero() of src/train/trainer.cpp:455 plus the overflow bookkeeping). */
int b2k_step_begin(const B2kCtx* ctx, b2k_stream_t s);
/* dst.loss_accum[2..3] += src.loss_accum[2..3]: joins the running loss of a view that was in flight on another stream
 * (no counterpart in the reference, whose step is one view on one stream). */
int b2k_loss_fold(const B2kCtx* dst, const B2kCtx* src, b2k_stream_t s);
/* eval_metrics, src/gpu/loss.h:41 (eval_kernel, src/gpu/loss.cu:241-293). */
int b2k_eval_metrics(const B2kCtx* ctx, const uint32_t* rgba, int32_t mask_weighted, b2k_stream_t s);

/* Bytes of ctx->bwd_scratch for a context of this image size, chunk count (0 or 1: whole view) and intersection capacity. */
uint64_t b2k_bwd_scratch_bytes(int32_t W, int32_t H, int32_t n_chunks, uint64_t isect_cap);

/* ---- backward ---- */
/* rasterize_backward, src/gpu/render.h:106 (raster_bwd_kernel, src/gpu/raster_bwd.cu:11-143). Same gradients; the
 * tile lists are replayed in segments of 128 fragments from the forward's checkpoints in ctx->bwd_scratch. */
int b2k_raster_bwd(const B2kCtx* ctx, const B2kModel* m, const B2kRenderOpts* opts, b2k_stream_t s);
/* rasterize_backward_tc, src/gpu/render.h:107-109 (raster_bwd_tc_kernel, src/gpu/raster_bwd_tc.cu:30-225), as far as its
 * contract goes: the pixel gradients in v_out were produced with LossParams::grad_scale applied and the per-splat
 * lanes leave divided by it (raster_bwd_tc.cu:198). The reference needs the scale to keep fp16 operands in range; the
 * reduction here is fp32 throughout, so this is b2k_raster_bwd with the division folded into its reduction. */
int b2k_raster_bwd_scaled(const B2kCtx* ctx, const B2kModel* m, const B2kRenderOpts* opts, float grad_scale, b2k_stream_t s);
/* optimizer_step, src/gpu/optim.h:50 (optim_kernel, src/gpu/optim.cu:100-378): projection backward fused with
 * sparse Adam; consumes and clears ctx->v_splat / vis_flag. With grad_out set it writes gradients and returns. */
int b2k_optim_fused(const B2kCtx* ctx, const B2kModel* m, const B2kCamera* cam, const B2kOptim* op, b2k_stream_t s);
/* Overflow guard of b2k_optim_fused and b2k_proj_bwd: when ctx->num_isect is set and the view's intersection total
 * num_isect[0] exceeds ctx->isect_cap (the view was composited from truncated lists), the lanes are still consumed and
 * cleared but the model / the accumulator is left untouched, so a host that reads the total only after the step
 * (b2k_read_num_isect, or num_isect[2] once per step) can grow the buffers and redo the view. The reference avoids the
 * case by reading the total inside every bin_and_sort (src/gpu/binning.cu:125-133). */
/* Data-parallel split of optimizer_step. b2k_proj_bwd: the gradient half (optim.cu:100-297) ADDING into a dense
 * accumulator grad[n][11+3K] (the grad_out layout) so several views and, after an all-reduce, several GPUs sum;
 * consumes and clears v_splat / vis_flag. b2k_adam: the update half (optim.cu:299-376) from that accumulator; splats
 * whose accumulated gradient is all zero are skipped when op->sparse; clears the accumulator rows it consumed. */
int b2k_proj_bwd(const B2kCtx* ctx, const B2kModel* m, const B2kCamera* cam, const B2kOptim* op, float* grad, b2k_stream_t s);
int b2k_adam(const B2kModel* m, const B2kOptim* op, float* grad, b2k_stream_t s);
/* b2k_adam on the splats [first, first + count) only (grad is still the whole accumulator; first a multiple of 4), so
 * that the update of one slice can run while the all-reduce of the next slice is in flight. Same device code and the
 * same results as b2k_adam over the whole model (optim.cu:299-376). */
int b2k_adam_range(const B2kModel* m, const B2kOptim* op, float* grad, int32_t first, int32_t count, b2k_stream_t s);

/* ---- refinement (RefineState::run, src/gpu/refine.cu:244-342), as the device steps its host sequence calls ----
 * All index / flag arrays are [n] device words; none of the calls synchronises. */
/* Stable ascending sort of (key, value) pairs on 32-bit keys (the role of cub::DeviceRadixSort in refine.cu:206-223): the
 * sorted pairs end in (keys, vals); (keys_alt, vals_alt) is scratch of the same size; tmp holds b2k_sort_pairs_tmp_bytes(). */
uint64_t b2k_sort_pairs_tmp_bytes(void);
/* Passes the library's LSD radix sort makes over keys of `bits` bits (8-bit digits; 9-bit ones where that saves a pass:
 * 17 or 18 bits, the tile ids of a 4K image). An even count leaves the result in the buffer pair the sort started from. */
int32_t b2k_sort_passes(int32_t bits);
int b2k_sort_pairs_u32(uint32_t* keys, uint32_t* vals, uint32_t* keys_alt, uint32_t* vals_alt, uint32_t n, void* tmp, uint64_t tmp_bytes, b2k_stream_t s);
/* prune_flags_kernel, refine.cu:54-72: keep / dead / culled flags (non-finite, transparent, oversized or far splats; with
 * cull_weight > 0 also those whose vis_weight is below it). center: 3 host floats. */
int b2k_refine_flags(const B2kModel* m, const float* center, float max_allowed, float cull_weight, uint32_t* keep, uint32_t* dead, uint32_t* culled, b2k_stream_t s);
/* gumbel_keys_kernel, refine.cu:75-93: keys of a weighted draw without replacement, stored so that an ASCENDING unsigned
 * sort lists the largest key first (the reference sorts floats descending); vals = the splat index. mode 0: weight =
 * effective opacity of kept visible splats; mode 1: refine_norm above `threshold` (also written to `above` when given). */
int b2k_refine_sample_keys(const B2kModel* m, const uint32_t* keep, const uint32_t* excluded, int32_t mode, float threshold, uint32_t seed, uint32_t* keys,
                           uint32_t* vals, uint32_t* above, b2k_stream_t s);
/* oversized_flags_kernel, refine.cu:95-99. */
int b2k_refine_oversized(const B2kModel* m, const uint32_t* keep, const uint32_t* excluded, float threshold, uint32_t* flags, b2k_stream_t s);
/* mark_kernel, refine.cu:101-104: flags[idx[k]] = 1 for k < count. */
int b2k_refine_mark(const uint32_t* idx, int32_t count, uint32_t* flags, b2k_stream_t s);
/* split_kernel, refine.cu:107-152: parent parents[k] becomes itself + one child, for k < count. The child's slot is
 * dead_idx[k] for k < from_dead and m->n + (k - from_dead) after that (m->n = the count before this call; the caller raises
 * it by count - from_dead afterwards and must have grown the buffers first). children[k] receives the slot;
 * tile_count (a RenderCtx's, may be NULL) is cleared at the child's slot. */
int b2k_refine_split(const B2kModel* m, uint32_t* tile_count, const uint32_t* parents, const uint32_t* dead_idx, int32_t from_dead, int32_t count,
                     float split_at_screen_size, uint32_t* children, b2k_stream_t s);
/* kill_slots_kernel, opacity_decay_kernel, bake_kernel (refine.cu:231, 154-161, 40-51). */
int b2k_refine_kill(const B2kModel* m, const uint32_t* idx, int32_t count, b2k_stream_t s);
int b2k_refine_opacity_decay(const B2kModel* m, float delta, b2k_stream_t s);
int b2k_refine_bake_floor(const B2kModel* m, b2k_stream_t s);
/* axis_kernel, refine.cu:179-185, for the percentile bounds: ascending-sortable keys of one coordinate (non-finite -> 0) and
 * the splat indices; b2k_key_to_float turns a sorted key back into the coordinate (host arithmetic). */
int b2k_refine_axis_keys(const B2kModel* m, int32_t axis, uint32_t* keys, uint32_t* vals, b2k_stream_t s);
float b2k_key_to_float(uint32_t ascending_key_bits);

/* ---- evidence and label vote (forward replays of a rendered view) ----
 * evidence_kernel, src/train/evidence.cu:48-121: for the view just rendered with bwd_info (ranges shrunk, last_idx
 * set), acc[i][0..2] += sum over pixels of vis * (m, m * res, k) with m = target alpha * weight, res the mean absolute
 * colour error of the pixel (+ normal_weight * the normal residual when `normals` is given and the view was rendered
 * with the pseudo-normal feature lane), k = (masked_has_alpha ? target alpha : 1) * weight. acc is [n][3]. */
int b2k_evidence_view(const B2kCtx* ctx, const uint32_t* rgba, const uint32_t* normals, const uint8_t* weights, int32_t masked_has_alpha, float normal_weight,
                      float* acc, b2k_stream_t s);
/* fold_view_kernel, src/train/evidence.cu:123-136: evidence[i][8] += (w_in, w_all, err, -, w_in * dir xyz, w_in^2) of one
 * view's acc, dir the unit vector from the splat to cam_pos (3 host floats). */
int b2k_evidence_fold(const B2kModel* m, const float* acc, const float* cam_pos, float* evidence, b2k_stream_t s);
/* label_vote_kernel, src/train/evidence.cu:142-196: votes[i][class of the pixel] += vis * k over the view's pixels;
 * votes is [n][b2k_label_bins()], class ids at or above the bin count are ignored. */
int b2k_label_vote(const B2kCtx* ctx, const uint32_t* rgba, const uint8_t* labels, const uint8_t* weights, int32_t masked_has_alpha, float* votes, b2k_stream_t s);
int32_t b2k_label_bins(void);

/* ---- data parallelism over the GPUs of one node ----
 * The reference is single-GPU; these entry points shard its step by view (one process or thread per GPU, a full model
 * replica each) as its design allows: views are independent until optimizer_step (src/train/trainer.cpp:464-529).
 * NCCL is loaded at run time (libnccl.so.2) by the first b2k_dp_init; nothing else in the library needs it. */
typedef struct B2kDp B2kDp;
#define B2K_DP_ID_BYTES 128
#define B2K_DP_MAX_RANKS 16
/* Rank 0 makes the rendezvous id and hands the 128 bytes to the other ranks over any host channel. */
int b2k_dp_unique_id(uint8_t* id);
/* Joins the communicator of `world` ranks on the current device (collective: every rank calls it). */
int b2k_dp_init(B2kDp** dp, const uint8_t* id, int32_t rank, int32_t world);
int b2k_dp_destroy(B2kDp* dp);
/* In-place sum over ranks of the dense gradient accumulator grad[count] (count = n * (11 + 3K) floats): the plain
 * ncclAllReduce form of the step, after which every rank runs the identical b2k_adam. */
int b2k_dp_allreduce_grads(B2kDp* dp, float* grad, uint64_t count, b2k_stream_t s);
/* In-place all-reduce of a refinement statistic over ranks: op 0 = sum (vis_count, vis_weight), 1 = max (refine_norm,
 * max_screen; src/gpu/optim.cu:122-124, src/gpu/project.cu:82-83). */
int b2k_dp_allreduce_stat(B2kDp* dp, float* stat, uint64_t count, int32_t op, b2k_stream_t s);
/* Stream-ordered barrier over the ranks (a 4-byte all-reduce): work enqueued after it on any rank starts only when
 * every rank's work enqueued before it has finished. */
int b2k_dp_barrier(B2kDp* dp, b2k_stream_t s);
/* Makes a device buffer of every rank addressable from this one: `base` must be the start of a cudaMalloc allocation
 * of this rank; on return peers[r] is rank r's buffer mapped into this process (peers[rank] == base). Collective;
 * synchronises the stream. The mappings live until b2k_dp_destroy. Needs peer access between the GPUs (NVLink). */
int b2k_dp_share(B2kDp* dp, void* base, void** peers, b2k_stream_t s);
/* Closes every mapping b2k_dp_share opened (after the stream has drained): call it on all ranks before buffers that were
 * shared are freed or reallocated, then share the new ones. */
int b2k_dp_release_shares(B2kDp* dp, b2k_stream_t s);
/* After the sharded update only the owner of a splat holds its current optimizer state. This makes a per-splat array
 * whole again on every rank, in place: for every rank r its slice (b2k_dp_slice) of each of `lanes` lanes (lane l starts
 * at base + l * lane_stride elements) is broadcast from r. Used before anything that moves splats between slices or
 * reads other ranks' moments (refinement, compaction, a checkpoint written by one rank). */
int b2k_dp_gather_slices(B2kDp* dp, void* base, uint64_t elem_bytes, int32_t lanes, uint64_t lane_stride, int32_t n, b2k_stream_t s);
/* The splats [first, first + count) whose update rank `rank` of `world` owns in b2k_dp_adam_shard: contiguous, starts
 * multiples of 128, together covering [0, n) exactly. Pure host arithmetic (no GPU needed). */
int b2k_dp_slice(int32_t n, int32_t rank, int32_t world, int32_t* first, int32_t* count);
/* Replica pointers for b2k_dp_adam_shard, each array indexed by rank (from b2k_dp_share). */
typedef struct {
  float* grad[B2K_DP_MAX_RANKS];     /* every rank's gradient accumulator [n][11+3K] */
  float* pos_op[B2K_DP_MAX_RANKS];   /* every rank's parameter buffers, laid out like B2kModel's */
  float* quat[B2K_DP_MAX_RANKS];
  float* lscale[B2K_DP_MAX_RANKS];
  float* sh_dc[B2K_DP_MAX_RANKS];
  float* sh_hi[B2K_DP_MAX_RANKS];
  const uint32_t* touched[B2K_DP_MAX_RANKS]; /* all NULL: every row of every accumulator is fetched. Else each rank's bitmap
                                                (B2kOptim.touched_out of its b2k_proj_bwd calls): rows whose bit is clear
                                                are zero and are not fetched over the links */
} B2kDpPeers;
/* Reduce-scatter + Adam + all-gather of the data-parallel step as ONE kernel over peer memory: this rank sums the rows
 * of its slice (b2k_dp_slice) from every rank's accumulator with plain peer loads, runs the update of b2k_adam on them
 * (moments, last_step and the Adam-mini second moment live only on the owner) and stores the updated parameters
 * into every rank's replica. Replicas stay bit-identical because each splat is updated by exactly one rank. The caller
 * brackets it with b2k_dp_barrier (before: all ranks' accumulators complete; after: all replicas written) and clears
 * its own accumulator afterwards. Same arithmetic as optim_kernel's update half (src/gpu/optim.cu:299-376). */
int b2k_dp_adam_shard(B2kDp* dp, const B2kModel* m, const B2kOptim* op, const B2kDpPeers* peers, b2k_stream_t s);

/* ---- helpers around the path ---- */
/* min_scale_kernel, src/gpu/refine.cu:27-38: lscale.w = sqrt(0.1) * min over cameras of distance / focal. */
int b2k_min_scale(const B2kModel* m, const float* cam_pos, const float* cam_focal, int32_t n_cams, b2k_stream_t s);
/* Model::compact, src/model.h:33 (src/model.cu:110-155), as its two device steps. b2k_select_flagged: the indices i
 * with keep[i] != 0 in ascending order into idx, their number into *count (device); tmp holds b2k_select_tmp_words(n)
 * words. b2k_gather_lanes: dst[l * stride + j] = src[l * stride + idx[j]] for l < lanes, j < count, with elements of 4
 * or 16 bytes (gather_kernel, src/model.cu:112-118); dst must be a different buffer. The caller reads *count back,
 * gathers every model array into a fresh buffer and swaps, as the reference does. */
uint64_t b2k_select_tmp_words(int32_t n);
int b2k_select_flagged(const uint32_t* keep, int32_t n, uint32_t* idx, uint32_t* count, uint32_t* tmp, b2k_stream_t s);
int b2k_gather_lanes(const void* src, void* dst, const uint32_t* idx, int32_t count, int32_t lanes, uint64_t stride, int32_t elem_bytes,
                     b2k_stream_t s);
/* pack_kernel, src/train/teacher.cu:11-17: float RGBA -> packed RGBA8 target. alpha_override < 0 keeps the image's. */
int b2k_pack_rgba8(const float* rgba, uint32_t* out, int32_t n_pixels, int32_t alpha_override, b2k_stream_t s);
/* The 8-bit image the render front end writes (src/render/renderer.cpp:353-358: lround(clamp(x, 0, 1) * 255) per channel,
 * there on the host after downloading floats), on the device so that a quarter of the bytes cross to the host. */
int b2k_quantize_rgba8(const float* rgba, uint32_t* out, int32_t n_pixels, b2k_stream_t s);

const char* b2k_error_string(int status);
int b2k_last_cuda_error(void);
const char* b2k_version(void);

#ifdef __cplusplus
}
#endif
#endif
