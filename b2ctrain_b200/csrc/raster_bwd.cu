// Backward through compositing: per-pixel reverse replay of the forward, per-fragment gradients reduced across the
// tile and accumulated per splat. Reference semantics: raster_bwd_kernel (src/gpu/raster_bwd.cu:11-143).
//
// Work decomposition (differs from the reference on purpose): one WARP owns an 8x8 tile, each lane replays two
// horizontally adjacent pixels. Per fragment the pair is summed in registers, then the 11 live gradient lanes are
// reduced across the warp with a halving butterfly (16 shuffles for all lanes together, against 5 shuffles per lane
// in a plain tree), after which lane 2L holds the tile's total of lane L and issues one global reduction. Fragment
// records are staged per warp in shared memory, so the kernel has no block-wide barrier: warps are independent.
// The per-pixel math is branch-free (a non-contributing fragment has alpha = 0 and adds exact zeros), which lets the
// two pixels' dependent chains (ex2, rcp) interleave.
//
// FP32-issue / latency bound: ~90 flops, one ex2 and one rcp per fragment-pixel, plus the reduction.
#include "common.cuh"

namespace b2k {
namespace {

constexpr int BWD_WARPS = 4;                 // warps (tiles) per CTA
constexpr int BWD_BATCH = 32;                // fragments staged per warp and batch
constexpr unsigned FULL = 0xffffffffu;

struct Staged { float4 a, c, col; };         // proj0, proj1, proj2 of one fragment

// Halving butterfly over the warp: on return v[0] of lane l is the warp's sum of the callers' v[(l >> 1) & 15].
__device__ __forceinline__ float warp_transpose_sum(float (&v)[16], int lane) {
  {
    const bool hi = lane & 16;
#pragma unroll
    for (int i = 0; i < 8; i++) { const float send = hi ? v[i] : v[i + 8]; const float keep = hi ? v[i + 8] : v[i]; v[i] = keep + __shfl_xor_sync(FULL, send, 16); }
  }
  {
    const bool hi = lane & 8;
#pragma unroll
    for (int i = 0; i < 4; i++) { const float send = hi ? v[i] : v[i + 4]; const float keep = hi ? v[i + 4] : v[i]; v[i] = keep + __shfl_xor_sync(FULL, send, 8); }
  }
  {
    const bool hi = lane & 4;
#pragma unroll
    for (int i = 0; i < 2; i++) { const float send = hi ? v[i] : v[i + 2]; const float keep = hi ? v[i + 2] : v[i]; v[i] = keep + __shfl_xor_sync(FULL, send, 4); }
  }
  {
    const bool hi = lane & 2;
    const float send = hi ? v[0] : v[1]; const float keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(FULL, send, 2);
  }
  v[0] += __shfl_xor_sync(FULL, v[0], 1);
  return v[0];
}

__device__ __forceinline__ float fast_sqrt(float x) { float r; asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }

struct PixelState { float T, Sr, Sg, Sb, vr, vg, vb, vow, inv_fa; uint32_t last; };

// One fragment against one pixel, branch-free. Adds into acc; returns whether the fragment contributed.
__device__ __forceinline__ bool replay(PixelState& s, float pcx, float pcy, uint32_t idx, const float4 a, const float4 c, float cr, float cg, float cb,
                                       float Wf, float Hf, float (&acc)[16]) {
  const float dx = pcx - a.x, dy = pcy - a.y;
  const float sigma = 0.5f * (a.z * dx * dx + c.x * dy * dy) + a.w * dx * dy;
  const bool on = idx < s.last && sigma >= 0.f && sigma <= c.w;
  const float gauss = __expf(-sigma);
  const float a_raw = c.y * gauss;
  const float alpha = on ? fminf(ALPHA_MAX, a_raw) : 0.f;
  const float ra = __fdividef(1.f, 1.f - alpha);
  const float Tb = s.T * ra;
  const float vis = alpha * Tb;
  acc[5] += vis * s.vr; acc[6] += vis * s.vg; acc[7] += vis * s.vb;
  const float v_alpha = (Tb * cr - s.Sr * ra) * s.vr + (Tb * cg - s.Sg * ra) * s.vg + (Tb * cb - s.Sb * ra) * s.vb + s.vow * ra;
  // The alpha clamp has zero slope: the geometry and opacity lanes vanish where it is active.
  const bool live = on && a_raw <= ALPHA_MAX;
  const float v_sigma = live ? -alpha * v_alpha : 0.f;
  const float gx = -v_sigma * (a.z * dx + a.w * dy), gy = -v_sigma * (a.w * dx + c.x * dy);
  acc[0] += gx; acc[1] += gy;
  acc[2] += 0.5f * v_sigma * dx * dx; acc[3] += v_sigma * dx * dy; acc[4] += 0.5f * v_sigma * dy * dy;
  acc[8] += live ? v_alpha * gauss : 0.f;
  const float sx = gx * Wf, sy = gy * Hf;
  acc[9] += fast_sqrt(sx * sx + sy * sy) * s.inv_fa;
  s.Sr += cr * vis; s.Sg += cg * vis; s.Sb += cb * vis;
  s.T = Tb;
  acc[10] += vis;
  return on;
}

__global__ void __launch_bounds__(BWD_WARPS * 32) raster_bwd_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ proj2, const float4* __restrict__ out_rgba, const float4* __restrict__ out_feat, const uint32_t* __restrict__ last_idx,
    const float4* __restrict__ v_out, int W, int H, int tiles_x, int n_tiles, float3 bg, float* __restrict__ v_splat, uint32_t* __restrict__ vis_flag,
    float* __restrict__ vis_weight) {
  __shared__ Staged s_frag[BWD_WARPS][BWD_BATCH];
  __shared__ uint32_t s_gid[BWD_WARPS][BWD_BATCH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * BWD_WARPS + warp;
  if (tile >= n_tiles) return;
  const uint2 range = tile_ranges[tile];
  if (range.y <= range.x) return;
  const int tx = tile % tiles_x, ty = tile / tiles_x;
  const int px0 = tx * RT_W + (lane & 3) * 2, py = ty * RT_W + (lane >> 2);   // this lane's pixel pair (px0, px0 + 1) on row py

  PixelState st[2];
#pragma unroll
  for (int p = 0; p < 2; p++) {
    const int px = px0 + p;
    PixelState& s = st[p];
    s.T = 0.f; s.Sr = s.Sg = s.Sb = 0.f; s.vr = s.vg = s.vb = s.vow = 0.f; s.inv_fa = 0.f; s.last = range.x;
    if (px < W && py < H) {
      const int pix = py * W + px;
      const float4 vo = v_out[pix];
      s.T = out_feat[pix].w;
      s.vr = vo.x; s.vg = vo.y; s.vb = vo.z;
      s.vow = (vo.w - (bg.x * vo.x + bg.y * vo.y + bg.z * vo.z)) * s.T;
      s.inv_fa = 1.f / fmaxf(out_rgba[pix].w, 1e-5f);
      s.last = last_idx[pix];
    }
  }
  const float pcx = (float)px0 + 0.5f, pcy = (float)py + 0.5f;
  const float Wf = (float)W, Hf = (float)H;
  Staged* frag = s_frag[warp];
  uint32_t* gids = s_gid[warp];

  for (uint32_t batch_end = range.y; batch_end > range.x;) {
    const uint32_t remaining = batch_end - range.x;
    const uint32_t count = remaining < (uint32_t)BWD_BATCH ? remaining : (uint32_t)BWD_BATCH;
    const uint32_t batch_start = batch_end - count;
    __syncwarp();
    if ((uint32_t)lane < count) {
      const uint32_t gid = vals_sorted[batch_start + lane];
      gids[lane] = gid;
      frag[lane].a = proj0[gid]; frag[lane].c = proj1[gid]; frag[lane].col = proj2[gid];
    }
    __syncwarp();
    for (int j = (int)count - 1; j >= 0; j--) {
      const uint32_t idx = batch_start + (uint32_t)j;
      const float4 a = frag[j].a, c = frag[j].c, col = frag[j].col;
      const float cr = fmaxf(col.x, 0.f), cg = fmaxf(col.y, 0.f), cb = fmaxf(col.z, 0.f);
      float acc[16];
#pragma unroll
      for (int k = 0; k < 16; k++) acc[k] = 0.f;
      const bool on0 = replay(st[0], pcx, pcy, idx, a, c, cr, cg, cb, Wf, Hf, acc);
      const bool on1 = replay(st[1], pcx + 1.f, pcy, idx, a, c, cr, cg, cb, Wf, Hf, acc);
      if (__ballot_sync(FULL, on0 || on1) == 0) continue;
      if (col.x < 0.f) acc[5] = 0.f;   // the colour clamp at zero has zero slope
      if (col.y < 0.f) acc[6] = 0.f;
      if (col.z < 0.f) acc[7] = 0.f;
      const float total = warp_transpose_sum(acc, lane);
      if ((lane & 1) == 0) {
        const int k = lane >> 1;
        const uint32_t gid = gids[j];
        if (k < 10) { if (total != 0.f) atomicAdd(v_splat + (size_t)gid * GRAD_LANES + k, total); }
        else if (k == 10) { vis_flag[gid] = 1u; if (vis_weight) atomicAdd(vis_weight + gid, total); }
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
  raster_bwd_kernel<<<div_up(c->n_tiles, BWD_WARPS), BWD_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (const uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, (const float4*)c->proj1, (const float4*)c->proj2,
      (const float4*)c->out_rgba, (const float4*)c->out_feat, c->last_idx, (const float4*)c->v_out, c->W, c->H, c->tiles_x, c->n_tiles, bg,
      c->v_splat, c->vis_flag, m->vis_weight);
  return check_launch();
}
