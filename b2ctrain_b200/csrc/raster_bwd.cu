// Backward through compositing: per-pixel reverse replay of the forward, per-fragment gradients reduced across the
// tile and accumulated per splat. Reference semantics: raster_bwd_kernel (src/gpu/raster_bwd.cu:11-143).
//
// Work decomposition (differs from the reference on purpose): a warp owns TWO 8x8 tiles, one per half-warp; each lane
// replays a 2x2 pixel quad. Per fragment the quad is summed in registers first, then the 11 live gradient lanes are
// reduced across the 16 lanes of the half-warp with a halving butterfly (15 shuffles for all lanes together, against
// 5 shuffles per lane and per warp in a plain tree), after which lane L holds the tile's total of lane L and issues
// one global reduction. Fragment records are staged per half-warp in shared memory, so the kernel has no block-wide
// barrier at all: warps (and their tiles) are independent.
//
// FP32-issue bound: ~90 flops, one ex2 and one rcp per contributing fragment-pixel, plus the reduction.
#include "common.cuh"

namespace b2k {
namespace {

constexpr int BWD_WARPS = 2;                 // warps per CTA -> 4 tiles per CTA
constexpr int BWD_BATCH = 16;                // fragments staged per half-warp and batch
constexpr unsigned FULL = 0xffffffffu;

struct Staged { float4 a, c, col; };         // proj0, proj1, proj2 of one fragment

// Halving butterfly over the 16 lanes of a half-warp: on return v[0] of lane L (L = lane & 15) is the sum over the
// half-warp of the callers' v[L].
__device__ __forceinline__ float halfwarp_transpose_sum(float (&v)[16], int lane) {
  {
    const bool hi = lane & 8;
#pragma unroll
    for (int i = 0; i < 8; i++) { const float send = hi ? v[i] : v[i + 8]; const float keep = hi ? v[i + 8] : v[i]; v[i] = keep + __shfl_xor_sync(FULL, send, 8); }
  }
  {
    const bool hi = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; i++) { const float send = hi ? v[i] : v[i + 4]; const float keep = hi ? v[i + 4] : v[i]; v[i] = keep + __shfl_xor_sync(FULL, send, 4); }
  }
  {
    const bool hi = lane & 2;
#pragma unroll
    for (int i = 0; i < 2; i++) { const float send = hi ? v[i] : v[i + 2]; const float keep = hi ? v[i + 2] : v[i]; v[i] = keep + __shfl_xor_sync(FULL, send, 2); }
  }
  {
    const bool hi = lane & 1;
    const float send = hi ? v[0] : v[1]; const float keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(FULL, send, 1);
  }
  return v[0];
}

__global__ void __launch_bounds__(BWD_WARPS * 32) raster_bwd_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ proj2, const float4* __restrict__ out_rgba, const float4* __restrict__ out_feat, const uint32_t* __restrict__ last_idx,
    const float4* __restrict__ v_out, int W, int H, int tiles_x, int n_tiles, float3 bg, float* __restrict__ v_splat, uint32_t* __restrict__ vis_flag,
    float* __restrict__ vis_weight) {
  __shared__ Staged s_frag[BWD_WARPS][2][BWD_BATCH];
  __shared__ uint32_t s_gid[BWD_WARPS][2][BWD_BATCH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = lane >> 4, hl = lane & 15;
  const int tile = (blockIdx.x * BWD_WARPS + warp) * 2 + half;
  const bool tile_ok = tile < n_tiles;
  uint2 range = make_uint2(0u, 0u);
  if (tile_ok) range = tile_ranges[tile];
  if (__ballot_sync(FULL, range.y > range.x) == 0) return;
  const int tx = tile % tiles_x, ty = tile / tiles_x;
  const int qx = tx * RT_W + (hl & 3) * 2, qy = ty * RT_W + (hl >> 2) * 2;   // top-left pixel of this lane's quad

  // Per-pixel state of the quad (index p = dy * 2 + dx).
  float T[4], Sr[4], Sg[4], Sb[4], vr[4], vg[4], vb[4], vow[4], inv_fa[4];
  uint32_t last[4];
#pragma unroll
  for (int p = 0; p < 4; p++) {
    const int px = qx + (p & 1), py = qy + (p >> 1);
    const bool inside = tile_ok && px < W && py < H;
    T[p] = 0.f; Sr[p] = Sg[p] = Sb[p] = 0.f; vr[p] = vg[p] = vb[p] = vow[p] = 0.f; inv_fa[p] = 0.f; last[p] = range.x;
    if (inside) {
      const int pix = py * W + px;
      const float4 vo = v_out[pix];
      T[p] = out_feat[pix].w;
      vr[p] = vo.x; vg[p] = vo.y; vb[p] = vo.z;
      vow[p] = (vo.w - (bg.x * vo.x + bg.y * vo.y + bg.z * vo.z)) * T[p];
      inv_fa[p] = 1.f / fmaxf(out_rgba[pix].w, 1e-5f);
      last[p] = last_idx[pix];
    }
  }
  const float pcx = (float)qx + 0.5f, pcy = (float)qy + 0.5f;
  const float Wf = (float)W, Hf = (float)H;
  Staged* frag = s_frag[warp][half];
  uint32_t* gids = s_gid[warp][half];

  // Both halves walk their own list backwards in lockstep; a half whose list is exhausted idles.
  uint32_t batch_end = range.y;
  while (__ballot_sync(FULL, batch_end > range.x) != 0) {
    const uint32_t remaining = batch_end - range.x;   // 0 when exhausted (batch_end == range.x)
    const uint32_t count = remaining < (uint32_t)BWD_BATCH ? remaining : (uint32_t)BWD_BATCH;
    const uint32_t batch_start = batch_end - count;
    __syncwarp();
    if ((uint32_t)hl < count) {
      const uint32_t gid = vals_sorted[batch_start + hl];
      gids[hl] = gid;
      frag[hl].a = proj0[gid]; frag[hl].c = proj1[gid]; frag[hl].col = proj2[gid];
    }
    __syncwarp();
    const uint32_t max_count = max(count, __shfl_xor_sync(FULL, count, 16));
    for (int j = (int)max_count - 1; j >= 0; j--) {
      const bool have = j < (int)count;
      const uint32_t idx = batch_start + (uint32_t)j;
      float acc[16];
#pragma unroll
      for (int k = 0; k < 16; k++) acc[k] = 0.f;
      bool any = false;
      if (have) {
        const float4 a = frag[j].a, c = frag[j].c, col = frag[j].col;
        const float cr = fmaxf(col.x, 0.f), cg = fmaxf(col.y, 0.f), cb = fmaxf(col.z, 0.f);
#pragma unroll
        for (int p = 0; p < 4; p++) {
          const float dx = pcx + (float)(p & 1) - a.x, dy = pcy + (float)(p >> 1) - a.y;
          const float sigma = 0.5f * (a.z * dx * dx + c.x * dy * dy) + a.w * dx * dy;
          if (idx < last[p] && sigma >= 0.f && sigma <= c.w) {
            any = true;
            const float gauss = __expf(-sigma);
            const float a_raw = c.y * gauss;
            const float alpha = fminf(ALPHA_MAX, a_raw);
            const float ra = 1.f / (1.f - alpha);
            const float Tb = T[p] * ra;
            const float vis = alpha * Tb;
            acc[5] += vis * vr[p]; acc[6] += vis * vg[p]; acc[7] += vis * vb[p];
            const float v_alpha = (Tb * cr - Sr[p] * ra) * vr[p] + (Tb * cg - Sg[p] * ra) * vg[p] + (Tb * cb - Sb[p] * ra) * vb[p] + vow[p] * ra;
            if (a_raw <= ALPHA_MAX) {   // the clamp has zero slope
              const float v_sigma = -alpha * v_alpha;
              const float gx = -v_sigma * (a.z * dx + a.w * dy), gy = -v_sigma * (a.w * dx + c.x * dy);
              acc[0] += gx; acc[1] += gy;
              acc[2] += 0.5f * v_sigma * dx * dx; acc[3] += v_sigma * dx * dy; acc[4] += 0.5f * v_sigma * dy * dy;
              acc[8] += v_alpha * gauss;
              const float sx = gx * Wf, sy = gy * Hf;
              acc[9] += sqrtf(sx * sx + sy * sy) * inv_fa[p];
            }
            Sr[p] += cr * vis; Sg[p] += cg * vis; Sb[p] += cb * vis;
            T[p] = Tb;
            acc[10] += vis;
          }
        }
        if (col.x < 0.f) acc[5] = 0.f;   // colour clamp at zero has zero slope
        if (col.y < 0.f) acc[6] = 0.f;
        if (col.z < 0.f) acc[7] = 0.f;
      }
      const unsigned contrib = __ballot_sync(FULL, any);
      if (contrib == 0) continue;
      const float total = halfwarp_transpose_sum(acc, lane);
      const unsigned mine = half ? (contrib >> 16) : (contrib & 0xffffu);
      if (have && mine != 0) {
        const uint32_t gid = gids[j];
        if (hl < 10) { if (total != 0.f) atomicAdd(v_splat + (size_t)gid * GRAD_LANES + hl, total); }
        else if (hl == 10) { vis_flag[gid] = 1u; if (vis_weight) atomicAdd(vis_weight + gid, total); }
      }
    }
    batch_end = batch_start;
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" int b2k_raster_bwd(const B2kCtx* c, const B2kModel* m, const B2kRenderOpts* o, b2k_stream_t stream) {
  B2K_REQUIRE(c && m && o && c->tile_ranges && c->vals_sorted && c->proj0 && c->proj1 && c->proj2);
  B2K_REQUIRE(c->out_rgba && c->out_feat && c->last_idx && c->v_out && c->v_splat && c->vis_flag);
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->n_tiles == c->tiles_x * c->tiles_y);
  const float3 bg = make_float3(o->bg[0], o->bg[1], o->bg[2]);
  const int tiles_per_cta = BWD_WARPS * 2;
  raster_bwd_kernel<<<div_up(c->n_tiles, tiles_per_cta), BWD_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (const uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, (const float4*)c->proj1, (const float4*)c->proj2,
      (const float4*)c->out_rgba, (const float4*)c->out_feat, c->last_idx, (const float4*)c->v_out, c->W, c->H, c->tiles_x, c->n_tiles, bg,
      c->v_splat, c->vis_flag, m->vis_weight);
  return check_launch();
}
