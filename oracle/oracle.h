/* CPU oracle for the splat render-and-backprop path: TEST INFRASTRUCTURE ONLY.
 *
 * A double-precision restatement of the algorithm of b2ctrain's per-step hot path, stage by stage, written to be
 * the checker for the CUDA kernels. Nothing in the product may link, import or call this library: only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity pin: the forward + loss chain (orc_project -> orc_bin -> orc_raster_fwd -> orc_loss) is checked against the
 * reference's own double-precision `reference_loss` (tests/reference.cpp:34-143, compiled unmodified into
 * oracle/_ref/) and the analytic backward chain (orc_raster_bwd -> orc_proj_bwd) against central differences of that
 * same function under the reference's own acceptance rule (tests/tests.cpp:427-435). What the reference's tests never
 * exercise (3D-filter floor, SH degree 4, tile lists and order, the Adam update) is "parity unpinned" by the
 * reference; for those the oracle follows the cited device code and is checked for self-consistency (finite
 * differences of its own forward).
 *
 * Every stage takes plain arrays so a test can feed it either its own upstream output (a pure double chain) or the
 * GPU's upstream output (a stage-isolated comparison).
 */
#ifndef ORACLE_H
#define ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same fields, order and meaning as CameraGPU (src/gpu/render.h:10-24). */
typedef struct {
  float R[9];
  float t[3];
  float pos[3];
  float fx, fy, cx, cy;
  int32_t W, H;
  float lim_pos_x, lim_pos_y, lim_neg_x, lim_neg_y;
} OrcCamera;

/* Same fields as LossParams (src/gpu/loss.h:20-30), flags widened to int32. */
typedef struct {
  float l1_w, ssim_w;
  float bg[3];
  int32_t composite, mask, alpha_lane;
  float match_alpha_weight;
  float scale;
  float grad_scale;
} OrcLoss;

/* Adam hyper-parameters of OptimParams (src/gpu/optim.h:8-17). */
typedef struct {
  int32_t t;
  float beta1, beta2, eps;
  float lr_mean, lr_rot, lr_scale, lr_opac, lr_dc, lr_sh_rest;
  int32_t sparse;
} OrcAdam;

#define ORC_REC 16 /* doubles per projected record, see orc_project */
enum { ORC_MX = 0, ORC_MY, ORC_C00, ORC_C01, ORC_C11, ORC_OPAC, ORC_Z, ORC_POWER, ORC_R, ORC_G, ORC_B, ORC_EX, ORC_EY, ORC_OK, ORC_MAXSCREEN, ORC_PAD };

/* EWA projection with the 3D-filter floor + SH colour (splat_math.cuh:224-293, project.cu:44-55).
 * pos_op/quat/lscale: [n][4] fp32 as in Model (model.h:8-12). sh: [n][K][3] fp32, K = (degree+1)^2 (ply.h:21).
 * rec: [n][ORC_REC] doubles; rec[ORC_OK] = 1 when the splat survives every record-stage cull (depth, finiteness,
 * determinant, opacity >= 1/255), else 0 and the rest is unspecified. */
void orc_project(int n, int degree, int active_degree, const float* pos_op, const float* quat, const float* lscale,
                 const float* sh, const OrcCamera* cam, double* rec);

/* Exact ellipse-to-8x8-tile decision for ONE fp32 record (tile_bbox + tile_hit, splat_math.cuh:27-53; the on-screen
 * and extent culls of splat_math.cuh:284-290). Pure IEEE single-precision arithmetic in a fixed order, no
 * contraction: the CUDA side evaluates the same expression tree with round-to-nearest intrinsics, so the two agree
 * bit for bit. Writes up to `max_tiles` hit tile ids (row-major order) and returns the hit count. */
int orc_tiles_of_record(float mx, float my, float c00, float c01, float c11, float power, int W, int H,
                        uint32_t* tiles, int max_tiles);

/* Binning and ordering (binning.cu:10-15,95-145): per-splat tile counts, the (tile, depth bits, index) order, tile
 * ranges. proj0 = (mx,my,c00,c01), proj1 = (c11,opac,z,power) as fp32 [n][4]; power < -0.5 marks "no record".
 * tile_count: [n]. vals_sorted: capacity `cap` entries (splat index). tile_ranges: [tiles][2]. Returns the number of
 * intersections (which may exceed cap; then nothing past cap is written). */
int64_t orc_bin(int n, const float* proj0, const float* proj1, int W, int H, uint32_t* tile_count,
                uint32_t* vals_sorted, uint32_t* keys_sorted, int64_t cap, uint32_t* tile_ranges);

/* Front-to-back compositing (raster_fwd.cu:9-71). geo: [n][8] doubles (mx,my,c00,c01,c11,opac,z,power); col: [n][3].
 * out_rgba: [P][4]; out_T: [P]; last_idx: [P]; tile_ranges [tiles][2] has .y shrunk in place when bwd_info.
 * out_depth (optional): [P] alpha-weighted depth sum (expected depth = out_depth / alpha, probe.cu:40). */
void orc_raster_fwd(int W, int H, const double* geo, const double* col, const uint32_t* vals_sorted,
                    uint32_t* tile_ranges, const double* bg, int bwd_info, double* out_rgba, double* out_T,
                    uint32_t* last_idx, double* out_depth);

/* Feature lanes (FeatureMode, src/gpu/render.h:27; project.cu:62-77; raster_fwd.cu:52,62): per-splat features [n][3]
 * (mode 1 pseudo-normals, mode 2 the caller's buffer), and their compositing with the walk of orc_raster_fwd. */
void orc_features(int n, int mode, const float* pos_op, const float* quat, const float* lscale, const float* feat_buffer,
                  const OrcCamera* cam, double* feat);
void orc_raster_feat(int W, int H, const double* geo, const double* feat, const uint32_t* vals_sorted,
                     const uint32_t* tile_ranges, double* out_feat);

/* Fused L1 + 11-tap SSIM + alpha lane (loss.cu:18-195). pred: [P][4] doubles; gt: packed RGBA8 [P]; weights: [P] u8
 * or NULL. v_out: [P][4] dL/d(rgba) times grad_scale. Returns the loss. */
double orc_loss(int W, int H, const double* pred, const uint32_t* gt, const uint8_t* weights, const OrcLoss* lp,
                double* v_out);

/* Per-pixel reverse replay (raster_bwd.cu:11-143). v_splat: [n][13] (zeroed here, lanes: xy 2, conic 3, rgb 3,
 * opacity 1, refine 1, feat 3 (always 0)); vis_flag: [n]; vis_weight: [n] (zeroed here). */
void orc_raster_bwd(int n, int W, int H, const double* geo, const double* col, const uint32_t* vals_sorted,
                    const uint32_t* tile_ranges, const double* bg, const double* out_rgba, const double* out_T,
                    const uint32_t* last_idx, const double* v_out, double* v_splat, uint32_t* vis_flag,
                    double* vis_weight);

/* Projection backward (optim.cu:100-297): screen-space lanes -> parameter gradients [n][11+3K]
 * (pos 3, opacity 1, quat 4, log-scale 3, SH K*3), the layout of OptimParams::grad_out (optim.cu:292-297). */
void orc_proj_bwd(int n, int degree, int active_degree, const float* pos_op, const float* quat, const float* lscale,
                  const float* sh, const OrcCamera* cam, const double* v_splat, const uint32_t* vis_flag,
                  const uint32_t* tile_count, double* grad);

/* Sparse Adam with the Adam-mini SH second moment and lazy catch-up (optim.cu:90-97,299-361), no noise.
 * All arrays updated in place: params as above, m_/v_ moments of the same shapes, m_sh [n][K][3], v_sh [n],
 * last_step [n]. grad: [n][11+3K] doubles. `active` [n]: the splat has a gradient this step (optim.cu:125-134). */
void orc_adam(int n, int degree, float* pos_op, float* quat, float* lscale, float* sh, float* m_pos, float* v_pos,
              float* m_q, float* v_q, float* m_ls, float* v_ls, float* m_sh, float* v_sh, uint32_t* last_step,
              const double* grad, const uint8_t* active, const OrcAdam* op);

/* 3D-filter floor (refine.cu:27-38): lscale[i][3] = sqrt(0.1) * min_c |p_i - cam_c| / focal_c. */
void orc_min_scale(int n, const float* pos_op, float* lscale, const float* cam_pos, const float* cam_focal, int n_cams);

/* One fused forward + loss (+ backward) in the pure double chain; the timed CPU baseline. Outputs optional (NULL).
 * Returns the loss. grad: [n][11+3K]. */
double orc_step(int n, int degree, int active_degree, const float* pos_op, const float* quat, const float* lscale,
                const float* sh, const OrcCamera* cam, const double* bg, const uint32_t* gt, const uint8_t* weights,
                const OrcLoss* lp, int backward, double* out_rgba, double* grad, int64_t* counters);

int orc_num_threads(void);
void orc_set_num_threads(int n);   /* OpenMP threads of the loops (overrides an inherited OMP_NUM_THREADS) */

#ifdef __cplusplus
}
#endif
#endif
