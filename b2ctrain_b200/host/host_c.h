/* C entry points of the C++ host library (libb2chost.so): the step loop of the reference's trainer
 * (src/train/trainer.cpp:452-529), with views in flight and view-level data parallelism, driven from any language.
 * Every function returns 0 on success (creation: a handle, or NULL); b2ch_last_error() describes the last failure of
 * the calling thread. */
#ifndef B2CH_HOST_C_H
#define B2CH_HOST_C_H
#include <stdint.h>
#include "../../include/b2k.h"
#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  int32_t views_in_flight, render_chunks;
  uint64_t isect_cap;
  float ssim_weight;
  int32_t mask, alpha_lane, composite;
  float match_alpha_weight, loss_scale;
  float bg[3];
  float lr_mean, lr_rot, lr_scale, lr_opac, lr_dc, lr_sh_rest;
  int32_t sparse;
  float noise_weight, noise_clamp;
  uint32_t seed;
  int32_t shard_update;
} B2chConfig;

const char* b2ch_last_error(void);
/* Splats in the host layout pos_op [n][4] (xyz, opacity logit), quat [n][4], lscale [n][4] (log scales, floor), sh [n][K][3].
 * Collective over the ranks when world > 1 (dp_id: the 128 bytes of b2k_dp_unique_id from rank 0); uses the current device. */
void* b2ch_trainer_create(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh, int32_t W, int32_t H,
                          const B2chConfig* cfg, int32_t rank, int32_t world, const uint8_t* dp_id);
void b2ch_trainer_destroy(void* trainer);
/* Registers a view (camera record with intrinsics for W x H, packed RGBA8 target on the host); returns its index or -1. */
int b2ch_trainer_add_view(void* trainer, const B2kCamera* cam, const uint32_t* rgba);
/* One optimisation step over the listed views (the whole step's list on every rank). */
int b2ch_trainer_step(void* trainer, const int32_t* views, int32_t n_views, void* stream, int32_t from_host);
int b2ch_trainer_read_loss(void* trainer, float* out16, void* stream);
int b2ch_trainer_set_profile(void* trainer, int32_t on);
/* out[0] intersection capacity, [1] steps redone after an overflow, [2] host-to-device bytes since the last call, [3] n,
 * [4] Adam step, [5] lanes, [6] views, [7] tile bits; out[8..10] hold six floats, ms of the last profiled step: the views,
 * the update, the whole step, and on several ranks the update's parts (the barrier before the sharded kernel, which also
 * waits for the slowest rank's views; the kernel; the barrier behind it). out must hold 11 words. */
int b2ch_trainer_info(void* trainer, uint64_t* out);
int b2ch_trainer_download(void* trainer, float* pos_op, float* quat, float* lscale, float* sh);
int b2ch_trainer_reduce_statistics(void* trainer, void* stream);
uint64_t b2ch_trainer_checksum(void* trainer, void* stream);

/* ---- rendering many cameras of one model ---- */
/* Splats as for b2ch_trainer_create. depth != 0: an expected-depth map is made with every image. render_chunks > 1: the
 * front-to-back chunked renderer. lanes: cameras in flight, each with its own render context and stream (1: one after
 * the other). isect_cap: starting capacity of the intersection buffers (0: 2^22); they grow on demand. Uses the current
 * device. */
void* b2ch_renderer_create(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh, int32_t W, int32_t H,
                           int32_t depth, int32_t render_chunks, int32_t lanes, uint64_t isect_cap);
void b2ch_renderer_destroy(void* renderer);
/* Queues one camera behind whatever is on `stream` and returns without waiting for it. With host_rgba8 (W * H words)
 * and / or host_depth (W * H floats) the image is quantised on the device (b2k_quantize_rgba8) and it, and the depth
 * map, are copied out on a copy stream while later cameras render; the buffers should be pinned and are valid after
 * b2ch_renderer_finish (a camera whose intersections did not fit its buffers is rendered again there, or when its lane
 * comes round again). background: 3 floats or
 * NULL; sh_degree < 0: the model's. */
int b2ch_renderer_render(void* renderer, const B2kCamera* cam, const float* background, int32_t sh_degree, uint32_t* host_rgba8, float* host_depth,
                         void* stream);
int b2ch_renderer_finish(void* renderer);
/* out[0] intersections of the camera checked last, [1] intersection capacity of lane 0, [2] device-to-host bytes since the
 * last call, [3] tile bits, [4] cameras rendered twice because their intersections had not fit. out holds 5 words. */
int b2ch_renderer_info(void* renderer, uint64_t* out5);

/* ---- files ---- */
/* The reference's `render` subcommand without the PNG step (src/render/renderer.cpp:199-368): reads the splat PLY and
 * cameras.json, renders this rank's cameras (rank, rank + world, ...) and writes <output_dir>/<name>.rgba8 (W x H x 4
 * bytes) and, with depth, <name>.depth.f32. background: 3 floats or NULL; sh_degree < 0: the model's. */
int b2ch_render_headless(const char* splat, const char* cameras, const char* output_dir, const float* background, int32_t sh_degree, int32_t depth,
                         int32_t render_chunks, int32_t rank, int32_t world, int32_t* rendered);
/* read_ply / write_ply (src/ply.h:51-53). Reading: call once with the array pointers NULL for n and the degree, then
 * with arrays of [n][3], [n][3], [n][4], [n], [n][K][3], [n][7], [n][2] (any may stay NULL). flags: 1 scales present,
 * 2 evidence columns, 4 label columns. */
int b2ch_ply_read(const char* path, int32_t* n, int32_t* degree, float* pos, float* log_scale, float* quat, float* opacity, float* sh, float* evidence,
                  float* labels, int32_t* flags);
int b2ch_ply_write(const char* path, int32_t n, int32_t degree, const float* pos, const float* log_scale, const float* quat, const float* opacity,
                   const float* sh, const float* evidence, const float* labels, const char* comment);

/* ---- refinement ---- */
/* StepTrainer::refine: the refinement pass on the trainer's model between steps, collective over the ranks (statistics
 * reduced, optimizer state made whole, buffers shared again). Parameters as b2ch_refine_once; out[6]: new n, pruned,
 * relocated, grown, split_oversized, culled. */
int b2ch_trainer_refine(void* trainer, const float* cam_pos, const float* cam_focal, int32_t n_cams, const float* fp, const uint32_t* up, void* stream, int32_t* out);
/* One RefineState::run (src/gpu/refine.cu:244-342) on a model built from the host arrays, with the statistics [4][n]
 * (refine_norm, max_screen, vis_count, vis_weight) and the cameras of the floor. fp: growth_grad_threshold,
 * growth_select_fraction, split_at_screen_size, opac_decay, cull_weight; up: iter, total, growth_allowed, max_splats, seed,
 * no_new. out[7]: new n, pruned, relocated, grown, split_oversized, culled, pairs. The refined splats land in the o_* arrays
 * (room for `capacity` splats); o_pairs (or NULL) receives [2][pairs]: the parents, then the slots of their children. */
int b2ch_refine_once(int32_t n, int32_t degree, const float* pos_op, const float* quat, const float* lscale, const float* sh, const float* stats,
                     const float* cam_pos, const float* cam_focal, int32_t n_cams, const float* fp, const uint32_t* up, int32_t W, int32_t H, int32_t* out,
                     int32_t capacity, float* o_pos_op, float* o_quat, float* o_lscale, float* o_sh, uint32_t* o_pairs);

#ifdef __cplusplus
}
#endif
#endif
