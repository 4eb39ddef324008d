// Forward compositing: one CTA per 8x8 tile walks the tile's depth-ordered fragment list front to back.
// Reference semantics: raster_fwd_kernel (src/gpu/raster_fwd.cu:9-71); the optional expected-depth output follows
// the mean-depth mode of probe_kernel (src/gpu/probe.cu:30-46).
//
// FP32-issue bound (one ex2 and ~25 flops per fragment-pixel); memory traffic is the gather of 48 B per staged
// fragment, served mostly by L2. Fragments are staged 64 at a time in shared memory with 128-bit loads.
#include "common.cuh"

namespace b2k {
namespace {

template <bool BWD, bool DEPTH>
__global__ void __launch_bounds__(RT_PX) raster_fwd_kernel(
    uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ proj2, int W, int H, int tiles_x, float3 bg, float4* __restrict__ out_rgba, float4* __restrict__ out_feat,
    float* __restrict__ out_depth, uint32_t* __restrict__ last_idx) {
  __shared__ float4 s0[RT_PX], s1[RT_PX], s2[RT_PX];
  __shared__ uint32_t s_max_last;
  const int tile = blockIdx.x;
  const int tx = tile % tiles_x, ty = tile / tiles_x;
  const int lx = threadIdx.x % RT_W, ly = threadIdx.x / RT_W;
  const int px = tx * RT_W + lx, py = ty * RT_W + ly;
  const bool inside = px < W && py < H;
  const float pcx = (float)px + 0.5f, pcy = (float)py + 0.5f;
  const uint2 range = tile_ranges[tile];
  if (threadIdx.x == 0) s_max_last = range.x;
  float T = 1.f, r = 0.f, g = 0.f, b = 0.f, zs = 0.f;
  bool done = !inside;
  uint32_t last = range.x;
  for (uint32_t start = range.x; start < range.y; start += RT_PX) {
    if (__syncthreads_count(done) == RT_PX) break;
    const uint32_t remaining = min((uint32_t)RT_PX, range.y - start);
    if (threadIdx.x < remaining) {
      const uint32_t gid = vals_sorted[start + threadIdx.x];
      s0[threadIdx.x] = proj0[gid]; s1[threadIdx.x] = proj1[gid]; s2[threadIdx.x] = proj2[gid];
    }
    __syncthreads();
    if (!done) {
      for (uint32_t t = 0; t < remaining; t++) {
        const float4 a = s0[t], c = s1[t];
        const float dx = pcx - a.x, dy = pcy - a.y;
        const float sigma = 0.5f * (a.z * dx * dx + c.x * dy * dy) + a.w * dx * dy;
        if (sigma < 0.f || sigma > c.w) continue;          // alpha below 1/255
        const float alpha = fminf(ALPHA_MAX, c.y * __expf(-sigma));
        const float next_T = T * (1.f - alpha);
        if (next_T <= T_CUTOFF) { done = true; break; }    // stop before the fragment that would saturate the pixel
        const float vis = alpha * T;
        const float4 col = s2[t];
        r += fmaxf(col.x, 0.f) * vis; g += fmaxf(col.y, 0.f) * vis; b += fmaxf(col.z, 0.f) * vis;
        if constexpr (DEPTH) zs += vis * c.z;
        T = next_T;
        last = start + t + 1;
      }
    }
  }
  if (inside) {
    const int pix = py * W + px;
    out_rgba[pix] = make_float4(r + T * bg.x, g + T * bg.y, b + T * bg.z, 1.f - T);
    out_feat[pix] = make_float4(0.f, 0.f, 0.f, T);
    if constexpr (DEPTH) out_depth[pix] = (1.f - T) > 0.05f ? zs / (1.f - T) : INFINITY;
    if constexpr (BWD) last_idx[pix] = last;
  }
  if constexpr (BWD) {
    atomicMax(&s_max_last, last);
    __syncthreads();
    if (threadIdx.x == 0) tile_ranges[tile].y = s_max_last;
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" int b2k_raster_fwd(const B2kCtx* c, const B2kRenderOpts* o, b2k_stream_t stream) {
  B2K_REQUIRE(c && o && c->tile_ranges && c->vals_sorted && c->proj0 && c->proj1 && c->proj2 && c->out_rgba && c->out_feat);
  B2K_REQUIRE(!o->bwd_info || c->last_idx);
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->n_tiles == c->tiles_x * c->tiles_y);
  cudaStream_t s = (cudaStream_t)stream;
  const float3 bg = make_float3(o->bg[0], o->bg[1], o->bg[2]);
#define L(B, D) raster_fwd_kernel<B, D><<<c->n_tiles, RT_PX, 0, s>>>((uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, \
    (const float4*)c->proj1, (const float4*)c->proj2, c->W, c->H, c->tiles_x, bg, (float4*)c->out_rgba, (float4*)c->out_feat, c->out_depth, c->last_idx)
  if (o->bwd_info) { if (c->out_depth) L(true, true); else L(true, false); }
  else { if (c->out_depth) L(false, true); else L(false, false); }
#undef L
  return check_launch();
}
