// Projection stage: EWA projection with the 3D-filter floor, SH colour, exact tile count and the depth sort key, one
// pass over the splats. Reference semantics: project_kernel (src/gpu/project.cu:9-84) and depth_keys_kernel
// (src/gpu/binning.cu:10-15), fused.
//
// HBM-bound stream: per splat 48 B of float4 parameters + 12 K B of planar SH in, 48 B of records + 12 B of
// count / key / index out. One thread per splat; the three float4 loads are 128-bit and coalesced, the planar SH
// lanes are coalesced across the warp.
#include "common.cuh"
#include "sh.cuh"

namespace b2k {

int g_last_cuda_error = 0;
int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return B2K_ERR_CUDA; }
  return B2K_OK;
}
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NUM_SMS_HINT;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = NUM_SMS_HINT;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

constexpr int PROJ_BLOCK = 256;

// Tile boxes of at most this many tiles are tested by the projecting thread and remembered as a bit mask; larger
// ones go to a list that a warp-per-splat kernel counts (and later emits) cooperatively.
constexpr int MASK_TILES = 64;


// Feature lanes of a splat (src/gpu/project.cu:62-77). Mode 1: pseudo-normal = the local axis of the shortest scale,
// turned to face the camera, in camera space. Mode 2: the caller's per-splat buffer, clamped to +-100, non-finite -> 0.
__device__ __forceinline__ float3 splat_feature(int mode, int i, const float4 po, const float4 ls, const float* Rq, const CamDev& cam,
                                                const float* __restrict__ feat_in) {
  if (mode == 1) {
    const int axis = (ls.x <= ls.y && ls.x <= ls.z) ? 0 : (ls.y <= ls.z ? 1 : 2);
    const float3 a = make_float3(Rq[axis], Rq[3 + axis], Rq[6 + axis]);
    const float inv = 1.f / fmaxf(sqrtf(a.x * a.x + a.y * a.y + a.z * a.z), 1e-12f);
    const float3 u = make_float3(a.x * inv, a.y * inv, a.z * inv);
    const float face = ((cam.pos[0] - po.x) * u.x + (cam.pos[1] - po.y) * u.y + (cam.pos[2] - po.z) * u.z) >= 0.f ? 1.f : -1.f;
    const float3 w = make_float3(u.x * face, u.y * face, u.z * face);
    const float* R = cam.R;
    return make_float3(R[0] * w.x + R[1] * w.y + R[2] * w.z, R[3] * w.x + R[4] * w.y + R[5] * w.z, R[6] * w.x + R[7] * w.y + R[8] * w.z);
  }
  float3 f = make_float3(feat_in[(size_t)i * 3], feat_in[(size_t)i * 3 + 1], feat_in[(size_t)i * 3 + 2]);
  f.x = isfinite(f.x) ? fminf(fmaxf(f.x, -100.f), 100.f) : 0.f;
  f.y = isfinite(f.y) ? fminf(fmaxf(f.y, -100.f), 100.f) : 0.f;
  f.z = isfinite(f.z) ? fminf(fmaxf(f.z, -100.f), 100.f) : 0.f;
  return f;
}

template <int DEG>
__global__ void __launch_bounds__(PROJ_BLOCK) project_kernel(
    int n, size_t cap, const float4* __restrict__ pos_op, const float4* __restrict__ quat, const float4* __restrict__ lscale,
    const float* __restrict__ sh_dc, const float* __restrict__ sh_hi, CamDev cam, int active, int tiles_x, int tiles_y,
    float4* __restrict__ proj0, float4* __restrict__ proj1, float4* __restrict__ proj2, uint32_t* __restrict__ tile_count,
    uint4* __restrict__ hit_info, uint32_t* __restrict__ depth_keys, uint32_t* __restrict__ order_in, float* __restrict__ max_screen,
    uint32_t* __restrict__ big_list, uint32_t* __restrict__ big_count, int feat_mode, const float* __restrict__ feat_in, float2* __restrict__ proj3) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 po = pos_op[i], q = quat[i], ls = lscale[i];
  Proj pr;
  uint32_t hits = 0, mask_lo = 0, mask_hi = 0, box = 0;
  bool shade = false, big = false;
  if (project_one(po, q, ls, cam, pr)) {
    const TileRec rec = make_tile_rec(pr.mx, pr.my, pr.c00, pr.c01, pr.c11, pr.power);
    TileBox bb;
    if (tile_box(rec, cam.W, cam.H, tiles_x, tiles_y, bb)) {
      const int bw = bb.max_x - bb.min_x, bh = bb.max_y - bb.min_y;
      if (bw * bh > MASK_TILES) {
        big = true; shade = true;
        box = 0xFFFFFFFFu;
        big_list[atomicAdd(big_count, 1u)] = (uint32_t)i;
      } else if (bw > 0 && bh > 0) {
        int bit = 0;
        for (int ty = bb.min_y; ty < bb.max_y; ty++)
          for (int tx = bb.min_x; tx < bb.max_x; tx++, bit++)
            if (tile_hit(tx, ty, rec)) { hits++; if (bit < 32) mask_lo |= 1u << bit; else mask_hi |= 1u << (bit - 32); }
        box = (uint32_t)bb.min_x | ((uint32_t)bb.min_y << 12) | ((uint32_t)bw << 24);
        shade = hits != 0;
      }
      const float detc = pr.c00 * pr.c11 - pr.c01 * pr.c01;
      const float ex = sqrtf(2.f * pr.power * pr.c11 / detc), ey = sqrtf(2.f * pr.power * pr.c00 / detc);
      if (max_screen) { const float ms = fmaxf(ex / (float)cam.W, ey / (float)cam.H); if (ms > max_screen[i]) atomic_max_nonneg(max_screen + i, ms); }
    }
    proj0[i] = make_float4(pr.mx, pr.my, pr.c00, pr.c01);
    proj1[i] = make_float4(pr.c11, pr.opac, pr.mean_c.z, pr.power);
    if (shade) {
      float4 col = splat_colour<DEG>(i, cap, make_float3(po.x, po.y, po.z), cam.pos, active, sh_dc, sh_hi);
      if (feat_mode != 0) {
        const float3 f = splat_feature(feat_mode, i, po, ls, pr.Rq, cam, feat_in);
        col.w = f.x;
        proj3[i] = make_float2(f.y, f.z);
      }
      proj2[i] = col;
    }
  } else {
    proj1[i] = make_float4(0.f, 0.f, 0.f, -1.f);   // no record
  }
  hit_info[i] = make_uint4(mask_lo, mask_hi, box, 0u);
  order_in[i] = (uint32_t)i;
  if (!big) {   // big splats get their count and key from count_big_kernel
    tile_count[i] = hits;
    depth_keys[i] = hits ? __float_as_uint(pr.mean_c.z) : 0xFFFFFFFFu;
  }
}


// The projection of the chunked renderer, which decides tiles later and only for the splats whose tile box still holds
// a live tile: records, colours, the tile box, the depth key, the screen-size statistic.
// hit_info = (0, 0, box, height) with box = min_x | min_y << 12 | width << 24 for boxes of at most 64 tiles, and
// (min_x | min_y << 16, width | height << 16, 0xFFFFFFFF, height) above that; height = 0 marks an empty box.
// tile_count holds the box area, an upper bound of the tiles hit (zero exactly when the box is empty).
template <int DEG>
__global__ void __launch_bounds__(PROJ_BLOCK) project_lite_kernel(
    int n, size_t cap, const float4* __restrict__ pos_op, const float4* __restrict__ quat, const float4* __restrict__ lscale,
    const float* __restrict__ sh_dc, const float* __restrict__ sh_hi, int active, CamDev cam, int tiles_x, int tiles_y,
    float4* __restrict__ proj0, float4* __restrict__ proj1, float4* __restrict__ proj2, uint32_t* __restrict__ tile_count, uint4* __restrict__ hit_info,
    uint32_t* __restrict__ depth_keys, uint32_t* __restrict__ order_in, float* __restrict__ max_screen, int feat_mode, const float* __restrict__ feat_in,
    float2* __restrict__ proj3) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 po = pos_op[i], q = quat[i], ls = lscale[i];
  Proj pr;
  uint32_t area = 0, box = 0, bh_out = 0, w0 = 0, w1 = 0;
  if (project_one(po, q, ls, cam, pr)) {
    const TileRec rec = make_tile_rec(pr.mx, pr.my, pr.c00, pr.c01, pr.c11, pr.power);
    TileBox bb;
    if (tile_box(rec, cam.W, cam.H, tiles_x, tiles_y, bb)) {
      const int bw = bb.max_x - bb.min_x, bh = bb.max_y - bb.min_y;
      if (bw > 0 && bh > 0) {
        area = (uint32_t)(bw * bh);
        bh_out = (uint32_t)bh;
        if (area > (uint32_t)MASK_TILES) {
          box = 0xFFFFFFFFu;
          w0 = (uint32_t)bb.min_x | ((uint32_t)bb.min_y << 16); w1 = (uint32_t)bw | ((uint32_t)bh << 16);
        } else {
          box = (uint32_t)bb.min_x | ((uint32_t)bb.min_y << 12) | ((uint32_t)bw << 24);
        }
      }
      const float detc = pr.c00 * pr.c11 - pr.c01 * pr.c01;
      const float ex = sqrtf(2.f * pr.power * pr.c11 / detc), ey = sqrtf(2.f * pr.power * pr.c00 / detc);
      if (max_screen) { const float ms = fmaxf(ex / (float)cam.W, ey / (float)cam.H); if (ms > max_screen[i]) atomic_max_nonneg(max_screen + i, ms); }
    }
    proj0[i] = make_float4(pr.mx, pr.my, pr.c00, pr.c01);
    proj1[i] = make_float4(pr.c11, pr.opac, pr.mean_c.z, pr.power);
    // The colour is evaluated here for every splat with a tile box: this kernel reads the planar SH lanes coalesced,
    // while a colour evaluated later, for the emitting splats only and in depth order, costs one 32-byte sector per
    // lane and splat (it measured slower although it shades a tenth of the splats).
    if (area) {
      float4 col = splat_colour<DEG>(i, cap, make_float3(po.x, po.y, po.z), cam.pos, active, sh_dc, sh_hi);
      if (feat_mode != 0) {
        const float3 f = splat_feature(feat_mode, i, po, ls, pr.Rq, cam, feat_in);
        col.w = f.x;
        proj3[i] = make_float2(f.y, f.z);
      }
      proj2[i] = col;
    }
  } else {
    proj1[i] = make_float4(0.f, 0.f, 0.f, -1.f);   // no record
  }
  hit_info[i] = make_uint4(w0, w1, box, bh_out);
  order_in[i] = (uint32_t)i;
  tile_count[i] = area;
  depth_keys[i] = area ? __float_as_uint(pr.mean_c.z) : 0xFFFFFFFFu;
}

// One warp per listed splat: lanes sweep the tile box 32 tiles at a time.
__global__ void __launch_bounds__(256) count_big_kernel(const uint32_t* __restrict__ big_list, const uint32_t* __restrict__ big_count,
                                                        const float4* __restrict__ proj0, const float4* __restrict__ proj1, int W, int H, int tiles_x,
                                                        int tiles_y, uint32_t* __restrict__ tile_count, uint32_t* __restrict__ depth_keys) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5), count = *big_count;
  for (uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < count; e += warps) {
    const uint32_t i = big_list[e];
    const float4 a = proj0[i], b = proj1[i];
    const TileRec rec = make_tile_rec(a.x, a.y, a.z, a.w, b.x, b.w);
    TileBox bb;
    uint32_t hits = 0;
    if (tile_box(rec, W, H, tiles_x, tiles_y, bb)) {
      const int bw = bb.max_x - bb.min_x, area = bw * (bb.max_y - bb.min_y);
      for (int t0 = 0; t0 < area; t0 += 32) {
        const int t = t0 + lane;
        const bool hit = t < area && tile_hit(bb.min_x + t % bw, bb.min_y + t / bw, rec);
        hits += __popc(__ballot_sync(0xffffffffu, hit));
      }
    }
    if (lane == 0) { tile_count[i] = hits; depth_keys[i] = hits ? __float_as_uint(b.z) : 0xFFFFFFFFu; }
  }
}

// The decision half of the projection on its own: tile counts, hit masks and depth keys recomputed from the records
// already in proj0 / proj1 (power < -0.5 marks "no record").
__global__ void __launch_bounds__(PROJ_BLOCK) count_tiles_kernel(int n, const float4* __restrict__ proj0, const float4* __restrict__ proj1, int W, int H,
                                                                 int tiles_x, int tiles_y, uint32_t* __restrict__ tile_count, uint4* __restrict__ hit_info,
                                                                 uint32_t* __restrict__ depth_keys, uint32_t* __restrict__ order_in,
                                                                 uint32_t* __restrict__ big_list, uint32_t* __restrict__ big_count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float4 a = proj0[i], b = proj1[i];
  uint32_t hits = 0, mask_lo = 0, mask_hi = 0, box = 0;
  bool big = false;
  if (b.w > -0.5f) {
    const TileRec rec = make_tile_rec(a.x, a.y, a.z, a.w, b.x, b.w);
    TileBox bb;
    if (tile_box(rec, W, H, tiles_x, tiles_y, bb)) {
      const int bw = bb.max_x - bb.min_x, bh = bb.max_y - bb.min_y;
      if (bw * bh > MASK_TILES) {
        big = true; box = 0xFFFFFFFFu;
        big_list[atomicAdd(big_count, 1u)] = (uint32_t)i;
      } else if (bw > 0 && bh > 0) {
        int bit = 0;
        for (int ty = bb.min_y; ty < bb.max_y; ty++)
          for (int tx = bb.min_x; tx < bb.max_x; tx++, bit++)
            if (tile_hit(tx, ty, rec)) { hits++; if (bit < 32) mask_lo |= 1u << bit; else mask_hi |= 1u << (bit - 32); }
        box = (uint32_t)bb.min_x | ((uint32_t)bb.min_y << 12) | ((uint32_t)bw << 24);
      }
    }
  }
  hit_info[i] = make_uint4(mask_lo, mask_hi, box, 0u);
  order_in[i] = (uint32_t)i;
  if (!big) { tile_count[i] = hits; depth_keys[i] = hits ? __float_as_uint(b.z) : 0xFFFFFFFFu; }
}

template <int DEG>
int launch(const B2kModel* m, const CamDev& cam, const B2kRenderOpts* o, const B2kCtx* c, cudaStream_t s) {
  const float4* pos = (const float4*)(o->pos_override ? o->pos_override : m->pos_op);
  const float4* quat = (const float4*)(o->quat_override ? o->quat_override : m->quat);
  const float4* lscale = (const float4*)(o->lscale_override ? o->lscale_override : m->lscale);
  const int active = o->sh_degree < m->degree ? o->sh_degree : m->degree;
  uint32_t* big_count = big_count_ptr(c);
  uint32_t* big_list = big_list_ptr(c);
  if (cudaMemsetAsync(big_count, 0, sizeof(uint32_t), s) != cudaSuccess) return check_launch();
  project_kernel<DEG><<<div_up(m->n, PROJ_BLOCK), PROJ_BLOCK, 0, s>>>(
      m->n, (size_t)m->cap, pos, quat, lscale, m->sh_dc, m->sh_hi, cam, active < 0 ? 0 : active, c->tiles_x, c->tiles_y,
      (float4*)c->proj0, (float4*)c->proj1, (float4*)c->proj2, c->tile_count, (uint4*)c->hit_info, c->depth_keys_sorted, c->order, m->max_screen,
      big_list, big_count, o->feat_mode, o->feat_buffer, (float2*)c->proj3);
  count_big_kernel<<<sm_count() * 8, 256, 0, s>>>(big_list, big_count, (const float4*)c->proj0, (const float4*)c->proj1, cam.W, cam.H, c->tiles_x,
                                                  c->tiles_y, c->tile_count, c->depth_keys_sorted);
  return check_launch();
}

}  // namespace

int launch_project_lite(const B2kModel* m, const B2kCamera* cam, const B2kRenderOpts* o, const B2kCtx* c, cudaStream_t s) {
  const float4* pos = (const float4*)(o->pos_override ? o->pos_override : m->pos_op);
  const float4* quat = (const float4*)(o->quat_override ? o->quat_override : m->quat);
  const float4* lscale = (const float4*)(o->lscale_override ? o->lscale_override : m->lscale);
  const int active = o->sh_degree < m->degree ? (o->sh_degree < 0 ? 0 : o->sh_degree) : m->degree;
  const CamDev cd = to_camdev(*cam);
#define L(D) project_lite_kernel<D><<<div_up(m->n, PROJ_BLOCK), PROJ_BLOCK, 0, s>>>(m->n, (size_t)m->cap, pos, quat, lscale, m->sh_dc, m->sh_hi, active, cd, \
      c->tiles_x, c->tiles_y, (float4*)c->proj0, (float4*)c->proj1, (float4*)c->proj2, c->tile_count, (uint4*)c->hit_info, c->depth_keys_sorted, c->order, m->max_screen, \
      o->feat_mode, o->feat_buffer, (float2*)c->proj3)
  switch (m->degree) { case 0: L(0); break; case 1: L(1); break; case 2: L(2); break; case 3: L(3); break; default: L(4); break; }
#undef L
  return check_launch();
}
}  // namespace b2k

using namespace b2k;

extern "C" int b2k_project(const B2kModel* m, const B2kCamera* cam, const B2kRenderOpts* opts, const B2kCtx* ctx, b2k_stream_t s) {
  B2K_REQUIRE(m && cam && opts && ctx);
  if (m->n == 0) return B2K_OK;
  B2K_REQUIRE(m->n > 0 && m->cap >= m->n && m->pos_op && m->quat && m->lscale && m->sh_dc);
  B2K_REQUIRE(m->degree >= 0 && m->degree <= 4 && (m->degree == 0 || m->sh_hi));
  B2K_REQUIRE(ctx->proj0 && ctx->proj1 && ctx->proj2 && ctx->tile_count && ctx->hit_info && ctx->depth_keys_sorted && ctx->order && ctx->sort_tmp);
  if (ctx->sort_tmp_bytes < b2k_sort_tmp_bytes(ctx->n_cap, ctx->isect_cap)) return B2K_ERR_CAPACITY;
  B2K_REQUIRE(cam->W == ctx->W && cam->H == ctx->H && ctx->tiles_x == div_up(ctx->W, RT_W) && ctx->tiles_y == div_up(ctx->H, RT_W));
  B2K_REQUIRE(opts->feat_mode >= 0 && opts->feat_mode <= 2 && (opts->feat_mode == 0 || ctx->proj3) && (opts->feat_mode != 2 || opts->feat_buffer));
  if (ctx->n_cap < m->n) return B2K_ERR_CAPACITY;
  const CamDev cd = to_camdev(*cam);
  cudaStream_t st = (cudaStream_t)s;
  switch (m->degree) {
    case 0: return launch<0>(m, cd, opts, ctx, st);
    case 1: return launch<1>(m, cd, opts, ctx, st);
    case 2: return launch<2>(m, cd, opts, ctx, st);
    case 3: return launch<3>(m, cd, opts, ctx, st);
    default: return launch<4>(m, cd, opts, ctx, st);
  }
}

extern "C" int b2k_count_tiles(const B2kCtx* c, int32_t n, b2k_stream_t stream) {
  B2K_REQUIRE(c && n >= 0);
  if (n == 0) return B2K_OK;
  B2K_REQUIRE(c->proj0 && c->proj1 && c->tile_count && c->hit_info && c->depth_keys_sorted && c->order && c->sort_tmp);
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->tiles_x == div_up(c->W, RT_W) && c->tiles_y == div_up(c->H, RT_W));
  if (c->n_cap < n || c->sort_tmp_bytes < b2k_sort_tmp_bytes(c->n_cap, c->isect_cap)) return B2K_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  uint32_t* big_count = big_count_ptr(c);
  uint32_t* big_list = big_list_ptr(c);
  B2K_CUDA(cudaMemsetAsync(big_count, 0, sizeof(uint32_t), s));
  count_tiles_kernel<<<div_up(n, 256), 256, 0, s>>>(n, (const float4*)c->proj0, (const float4*)c->proj1, c->W, c->H, c->tiles_x, c->tiles_y, c->tile_count,
                                                   (uint4*)c->hit_info, c->depth_keys_sorted, c->order, big_list, big_count);
  count_big_kernel<<<sm_count() * 8, 256, 0, s>>>(big_list, big_count, (const float4*)c->proj0, (const float4*)c->proj1, c->W, c->H, c->tiles_x, c->tiles_y,
                                                  c->tile_count, c->depth_keys_sorted);
  return check_launch();
}

static const char* kErrors[] = {"ok", "bad argument", "buffer capacity exceeded", "unsupported lane", "CUDA error",
                                "intersection buffers overflowed"};
extern "C" const char* b2k_error_string(int status) { return status >= 0 && status <= 5 ? kErrors[status] : "unknown status"; }
extern "C" int b2k_last_cuda_error(void) { return g_last_cuda_error; }
extern "C" const char* b2k_version(void) { return "b2k 0.1 (sm_100a)"; }
