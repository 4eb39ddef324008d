// Backward through compositing: per-pixel reverse replay of the forward, per-fragment gradients reduced across the
// tile and accumulated per splat. Reference semantics: raster_bwd_kernel (src/gpu/raster_bwd.cu:11-143).
//
// Work decomposition (differs from the reference on purpose): one WARP owns an 8x8 tile, each lane replays two
// horizontally adjacent pixels. Per fragment the pair is summed in registers, then the 11 live gradient lanes are
// reduced across the warp with a halving butterfly (16 shuffles for all lanes together, against 5 shuffles per lane
// in a plain tree), after which lane 2L holds the tile's total of lane L and issues one global reduction. Fragment
// records are staged per warp in shared memory, so the kernel has no block-wide barrier: warps are independent.
// A fragment no pixel of the tile sees is rejected after the sigma test; otherwise the pair's math is branch-free (a
// pixel that does not see the fragment has alpha = 0 and adds exact zeros) and runs on packed fp32x2 instructions.
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

// State of this lane's pixel pair, one float2 per quantity: the replay below runs on Blackwell's packed fp32x2
// arithmetic (fma.rn.f32x2 and friends), one instruction for both pixels.
struct PairState { float2 T, Sr, Sg, Sb, vr, vg, vb, vow, inv_fa; uint32_t last0, last1; };

__device__ __forceinline__ float2 f2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float hsum(float2 v) { return v.x + v.y; }

// Tiles in order of decreasing work, approximately: a counting sort on the bit length of the tile's fragment count (all
// chunks together), longest first, tiles without fragments last. The replay kernel hands its warps out in this order,
// so the longest lists start first instead of deciding the kernel's tail, and the four tiles of a CTA are alike.
// One CTA; order[] holds n_tiles entries.
__global__ void __launch_bounds__(1024) tile_order_kernel(const uint2* __restrict__ tile_ranges, int n_tiles, int n_chunks, uint32_t* __restrict__ order) {
  __shared__ uint32_t s_hist[33], s_cursor[33];
  if (threadIdx.x < 33) s_hist[threadIdx.x] = 0u;
  __syncthreads();
  auto bucket_of = [&](int tile) {
    uint32_t len = 0;
    for (int ch = 0; ch < n_chunks; ch++) { const uint2 rg = tile_ranges[(size_t)ch * n_tiles + tile]; len += rg.y > rg.x ? rg.y - rg.x : 0u; }
    return len == 0u ? 0 : 32 - __clz(len);   // 0 for no fragments, else the bit length 1..32
  };
  for (int tile = threadIdx.x; tile < n_tiles; tile += blockDim.x) atomicAdd(&s_hist[bucket_of(tile)], 1u);
  __syncthreads();
  if (threadIdx.x == 0) { uint32_t at = 0; for (int b = 32; b >= 0; b--) { s_cursor[b] = at; at += s_hist[b]; } }
  __syncthreads();
  for (int tile = threadIdx.x; tile < n_tiles; tile += blockDim.x) order[atomicAdd(&s_cursor[bucket_of(tile)], 1u)] = (uint32_t)tile;
}

__global__ void __launch_bounds__(BWD_WARPS * 32) raster_bwd_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ proj2, const float4* __restrict__ out_rgba, const float4* __restrict__ out_feat, const uint32_t* __restrict__ last_idx,
    const float4* __restrict__ v_out, int W, int H, int tiles_x, int n_tiles, float3 bg, float* __restrict__ v_splat, uint32_t* __restrict__ vis_flag,
    float* __restrict__ vis_weight, int n_chunks, const uint32_t* __restrict__ order) {
  __shared__ Staged s_frag[BWD_WARPS][BWD_BATCH];
  __shared__ uint32_t s_gid[BWD_WARPS][BWD_BATCH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = blockIdx.x * BWD_WARPS + warp;
  if (slot >= n_tiles) return;
  const int tile = order ? (int)order[slot] : slot;
  // A view composited in depth chunks has one range per chunk and tile ([chunk][tile]); the replay walks the chunks
  // from the farthest to the nearest, the pixel state running through.
  {
    bool any = false;
    for (int ch = 0; ch < n_chunks; ch++) { const uint2 rg = tile_ranges[(size_t)ch * n_tiles + tile]; any = any || rg.y > rg.x; }
    if (!any) return;
  }
  const int tx = tile % tiles_x, ty = tile / tiles_x;
  const int px0 = tx * RT_W + (lane & 3) * 2, py = ty * RT_W + (lane >> 2);   // this lane's pixel pair (px0, px0 + 1) on row py

  PairState st;
  {
    float T[2] = {0.f, 0.f}, vr[2] = {0.f, 0.f}, vg[2] = {0.f, 0.f}, vb[2] = {0.f, 0.f}, vow[2] = {0.f, 0.f}, ifa[2] = {0.f, 0.f};
    uint32_t last[2] = {0u, 0u};   // outside the image: sees no fragment
#pragma unroll
    for (int p = 0; p < 2; p++) {
      const int px = px0 + p;
      if (px < W && py < H) {
        const int pix = py * W + px;
        const float4 vo = v_out[pix];
        T[p] = out_feat[pix].w;
        vr[p] = vo.x; vg[p] = vo.y; vb[p] = vo.z;
        vow[p] = (vo.w - (bg.x * vo.x + bg.y * vo.y + bg.z * vo.z)) * T[p];
        ifa[p] = 1.f / fmaxf(out_rgba[pix].w, 1e-5f);
        last[p] = last_idx[pix] & 0x7FFFFFFFu;   // a chunked forward keeps its saturation flag in bit 31
      }
    }
    st.T = make_float2(T[0], T[1]); st.Sr = st.Sg = st.Sb = f2(0.f);
    st.vr = make_float2(vr[0], vr[1]); st.vg = make_float2(vg[0], vg[1]); st.vb = make_float2(vb[0], vb[1]);
    st.vow = make_float2(vow[0], vow[1]); st.inv_fa = make_float2(ifa[0], ifa[1]);
    st.last0 = last[0]; st.last1 = last[1];
  }
  const float pcx = (float)px0 + 0.5f, pcy = (float)py + 0.5f;
  const float Wf = (float)W, Hf = (float)H;
  Staged* frag = s_frag[warp];
  uint32_t* gids = s_gid[warp];
#ifdef B2K_BWD_ABLATE_REDUCTION
  float ablate_sink = 0.f;
#endif

  for (int ch = n_chunks - 1; ch >= 0; ch--) {
  const uint2 range = tile_ranges[(size_t)ch * n_tiles + tile];
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
      const float4 a = frag[j].a, c = frag[j].c;
      // sigma for the pair: the two pixels share the row, so dy and the dy terms are scalars.
      const float dy = pcy - a.y;
      const float2 dx = make_float2(pcx - a.x, pcx + 1.f - a.x);
      const float2 sigma = __ffma2_rn(dx, __ffma2_rn(dx, f2(0.5f * a.z), f2(a.w * dy)), f2(0.5f * c.x * dy * dy));
      const bool on0 = idx < st.last0 && sigma.x >= 0.f && sigma.x <= c.w;
      const bool on1 = idx < st.last1 && sigma.y >= 0.f && sigma.y <= c.w;
      if (__ballot_sync(FULL, on0 || on1) == 0) continue;   // nobody in the tile sees this fragment: skip the heavy part
      const float4 col = frag[j].col;
      const float cr = fmaxf(col.x, 0.f), cg = fmaxf(col.y, 0.f), cb = fmaxf(col.z, 0.f);
      // Branch-free from here: a pixel that does not see the fragment has alpha = 0 and adds exact zeros.
      const float2 gauss = make_float2(__expf(-sigma.x), __expf(-sigma.y));
      const float2 a_raw = __fmul2_rn(f2(c.y), gauss);
      const float2 alpha = make_float2(on0 ? fminf(ALPHA_MAX, a_raw.x) : 0.f, on1 ? fminf(ALPHA_MAX, a_raw.y) : 0.f);
      const float2 ra = make_float2(__fdividef(1.f, 1.f - alpha.x), __fdividef(1.f, 1.f - alpha.y));
      const float2 nra = make_float2(-ra.x, -ra.y);
      const float2 Tb = __fmul2_rn(st.T, ra);
      const float2 vis = __fmul2_rn(alpha, Tb);
      float2 va = __fmul2_rn(st.vow, ra);
      va = __ffma2_rn(__ffma2_rn(st.Sr, nra, __fmul2_rn(Tb, f2(cr))), st.vr, va);
      va = __ffma2_rn(__ffma2_rn(st.Sg, nra, __fmul2_rn(Tb, f2(cg))), st.vg, va);
      va = __ffma2_rn(__ffma2_rn(st.Sb, nra, __fmul2_rn(Tb, f2(cb))), st.vb, va);
      // The alpha clamp has zero slope: the geometry and opacity lanes vanish where it is active.
      const bool live0 = on0 && a_raw.x <= ALPHA_MAX, live1 = on1 && a_raw.y <= ALPHA_MAX;
      const float2 av = __fmul2_rn(alpha, va);
      const float2 mvs = make_float2(live0 ? av.x : 0.f, live1 ? av.y : 0.f);          // -v_sigma
      const float2 gx = __fmul2_rn(mvs, __ffma2_rn(dx, f2(a.z), f2(a.w * dy)));
      const float2 gy = __fmul2_rn(mvs, __ffma2_rn(dx, f2(a.w), f2(c.x * dy)));
      const float2 mdx = __fmul2_rn(mvs, dx);
      const float2 og = __fmul2_rn(va, gauss);
      const float2 sx = __fmul2_rn(gx, f2(Wf)), sy = __fmul2_rn(gy, f2(Hf));
      const float2 q = __ffma2_rn(sx, sx, __fmul2_rn(sy, sy));
      const float2 rf = __fmul2_rn(make_float2(fast_sqrt(q.x), fast_sqrt(q.y)), st.inv_fa);
      float acc[16];
      acc[0] = hsum(gx); acc[1] = hsum(gy);
      acc[2] = -0.5f * hsum(__fmul2_rn(mdx, dx)); acc[3] = -hsum(mdx) * dy; acc[4] = -0.5f * dy * dy * hsum(mvs);
      acc[5] = hsum(__fmul2_rn(vis, st.vr)); acc[6] = hsum(__fmul2_rn(vis, st.vg)); acc[7] = hsum(__fmul2_rn(vis, st.vb));
      acc[8] = (live0 ? og.x : 0.f) + (live1 ? og.y : 0.f);
      acc[9] = hsum(rf); acc[10] = hsum(vis);
#pragma unroll
      for (int k = 11; k < 16; k++) acc[k] = 0.f;
      st.Sr = __ffma2_rn(f2(cr), vis, st.Sr); st.Sg = __ffma2_rn(f2(cg), vis, st.Sg); st.Sb = __ffma2_rn(f2(cb), vis, st.Sb);
      st.T = Tb;
      if (col.x < 0.f) acc[5] = 0.f;   // the colour clamp at zero has zero slope
      if (col.y < 0.f) acc[6] = 0.f;
      if (col.z < 0.f) acc[7] = 0.f;
#ifdef B2K_BWD_ABLATE_REDUCTION
      // Ablation build (never shipped): the replay alone, with the cross-lane reduction and the global reductions
      // removed, bounds from above what any other reduction scheme (tensor cores included) could save.
#pragma unroll
      for (int k = 0; k < 11; k++) ablate_sink += acc[k];
      continue;
#endif
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
#ifdef B2K_BWD_ABLATE_REDUCTION
  if (ablate_sink == 123456.789f) v_splat[0] = ablate_sink;   // keeps the replay alive
#endif
}

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" int b2k_raster_bwd(const B2kCtx* c, const B2kModel* m, const B2kRenderOpts* o, b2k_stream_t stream) {
  B2K_REQUIRE(c && m && o && c->tile_ranges && c->vals_sorted && c->proj0 && c->proj1 && c->proj2);
  B2K_REQUIRE(c->out_rgba && c->out_feat && c->last_idx && c->v_out && c->v_splat && c->vis_flag);
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->n_tiles == c->tiles_x * c->tiles_y);
  const float3 bg = make_float3(o->bg[0], o->bg[1], o->bg[2]);
  const int chunks = c->n_chunks > 1 ? c->n_chunks : 1;
  // The unsorted-pair buffer is scratch once the view is binned: it holds the tile order for this launch.
  uint32_t* order = c->keys && c->isect_cap >= (uint64_t)c->n_tiles ? c->keys : nullptr;
  if (order) tile_order_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((const uint2*)c->tile_ranges, c->n_tiles, chunks, order);
  raster_bwd_kernel<<<div_up(c->n_tiles, BWD_WARPS), BWD_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (const uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, (const float4*)c->proj1, (const float4*)c->proj2,
      (const float4*)c->out_rgba, (const float4*)c->out_feat, c->last_idx, (const float4*)c->v_out, c->W, c->H, c->tiles_x, c->n_tiles, bg,
      c->v_splat, c->vis_flag, m->vis_weight, chunks, order);
  return check_launch();
}
