// Forward compositing: one warp per 8x8 tile walks the tile's depth-ordered fragment list front to back, each lane
// carrying two horizontally adjacent pixels. Reference semantics: raster_fwd_kernel (src/gpu/raster_fwd.cu:9-71); the
// optional expected-depth output follows the mean-depth mode of probe_kernel (src/gpu/probe.cu:30-46).
//
// FP32-issue / latency bound (one ex2 and ~25 flops per fragment-pixel); memory traffic is the gather of 48 B per
// staged fragment, served mostly by L2. Fragments are staged 32 at a time per warp in shared memory with 128-bit
// loads, gathered one batch ahead; warps never synchronise with each other.
#include "common.cuh"

namespace b2k {
namespace {

constexpr int FWD_WARPS = 4;
constexpr int FWD_BATCH = 32;
#ifndef B2K_FWD_GROUP
#define B2K_FWD_GROUP 4
#endif
constexpr int FWD_GROUP = B2K_FWD_GROUP;                 // fragments whose state-independent math is issued together

// CHUNKED: the view is composited in depth chunks (chunk `chunk` of `n_chunks`, one launch each, nearest first). Between
// launches a pixel's state lives in the output buffers: the colour sums in out_feat.xyz, the transmittance in
// out_feat.w, and last_idx with bit 31 set once the pixel has reached the cutoff; out_rgba holds the finished pixel
// after every chunk, so a launch only touches tiles that received fragments. With DEPTH the depth sum travels in
// out_depth and the last chunk visits every pixel to divide it out. alive[tile] tells the binning of the next chunk
// whether any pixel of the tile can still take a fragment.
constexpr uint32_t DONE_BIT = 0x80000000u;

template <bool BWD, bool DEPTH, bool CHUNKED, bool FEAT>
__global__ void __launch_bounds__(FWD_WARPS * 32) raster_fwd_kernel(
    uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ proj2, int W, int H, int tiles_x, int n_tiles, float3 bg, float4* __restrict__ out_rgba, float4* __restrict__ out_feat,
    float* __restrict__ out_depth, uint32_t* __restrict__ last_idx, int chunk, int n_chunks, uint32_t* __restrict__ alive,
    const float2* __restrict__ proj3, float4* __restrict__ ckpt, float4* __restrict__ feat_acc) {
  // CHUNKED with FEAT (forward only): between chunks out_feat.xyz carries the colour sums, so the feature sums of a
  // pixel travel in feat_acc and move into out_feat.xyz when the last chunk, which then visits every pixel, is done.
  static_assert(!(FEAT && CHUNKED && BWD), "the chunked backward reads the colour sums from out_feat.xyz");
  __shared__ float4 s0[FWD_WARPS][FWD_BATCH], s1[FWD_WARPS][FWD_BATCH], s2[FWD_WARPS][FWD_BATCH];
  __shared__ float2 s3[FEAT ? FWD_WARPS : 1][FEAT ? FWD_BATCH : 1];
  float f0[2] = {0.f, 0.f}, f1[2] = {0.f, 0.f}, f2[2] = {0.f, 0.f};   // composited feature lanes (raster_fwd.cu:52)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * FWD_WARPS + warp;
  if (tile >= n_tiles) return;
  const int tx = tile % tiles_x, ty = tile / tiles_x;
  const int px0 = tx * RT_W + (lane & 3) * 2, py = ty * RT_W + (lane >> 2);
  const bool in0 = px0 < W && py < H, in1 = px0 + 1 < W && py < H;
  const float pcx = (float)px0 + 0.5f, pcy = (float)py + 0.5f;
  const uint2 range = tile_ranges[tile];
  const bool first = !CHUNKED || chunk == 0, final = !CHUNKED || chunk == n_chunks - 1;
  if (CHUNKED && !first && range.y <= range.x && !(final && (DEPTH || FEAT))) return;   // nothing of this chunk lands here: pixels, state and flag stay
  float T[2] = {1.f, 1.f}, r[2] = {0.f, 0.f}, g[2] = {0.f, 0.f}, b[2] = {0.f, 0.f}, zs[2] = {0.f, 0.f};
  bool done[2] = {!in0, !in1};
  uint32_t last[2] = {range.x, range.x};
  if (CHUNKED && !first) {
#pragma unroll
    for (int p = 0; p < 2; p++) {
      if (p == 0 ? in0 : in1) {
        const int pix = py * W + px0 + p;
        const float4 acc = out_feat[pix];
        r[p] = acc.x; g[p] = acc.y; b[p] = acc.z; T[p] = acc.w;
        if constexpr (DEPTH) zs[p] = out_depth[pix];
        if constexpr (FEAT) { const float4 fa = feat_acc[pix]; f0[p] = fa.x; f1[p] = fa.y; f2[p] = fa.z; }
        const uint32_t l = last_idx[pix];
        done[p] = (l & DONE_BIT) != 0u;
        last[p] = l & ~DONE_BIT;
      }
    }
  }
  // Checkpoints for the backward's segmented replay (see common.cuh): the state a later chunk starts a tile with, and
  // the state before every SEG_LEN-th fragment of the list.
  const int q = CHUNKED ? chunk * n_tiles + tile : tile;
  auto checkpoint = [&](uint32_t seg) {
    float4* dst = ckpt + (size_t)ckpt_slot(range.x, q, seg) * RT_PX + lane * 2;
    dst[0] = make_float4(r[0], g[0], b[0], T[0]); dst[1] = make_float4(r[1], g[1], b[1], T[1]);
  };
  if (BWD && CHUNKED && !first && range.y > range.x) checkpoint(0u);
  // The records of a batch are gathered one batch ahead, into registers: the two dependent loads (list entry, then the
  // splat's records) are in flight while the batch before them is composited.
  float4 n0 = make_float4(0.f, 0.f, 0.f, 0.f), n1 = n0, n2 = n0;
  float2 n3 = make_float2(0.f, 0.f);
  auto gather = [&](uint32_t from) {
    if (from < range.y && (uint32_t)lane < range.y - from) {
      const uint32_t gid = vals_sorted[from + lane];
      n0 = proj0[gid]; n1 = proj1[gid]; n2 = proj2[gid];
      if constexpr (FEAT) n3 = proj3[gid];
    }
  };
  gather(range.x);
  for (uint32_t start = range.x; start < range.y; start += FWD_BATCH) {
    if (__all_sync(0xffffffffu, done[0] && done[1])) break;
    if (BWD && start != range.x && ((start - range.x) & (uint32_t)(SEG_LEN - 1)) == 0u) checkpoint((start - range.x) >> SEG_SHIFT);
    const uint32_t remaining = min((uint32_t)FWD_BATCH, range.y - start);
    __syncwarp();
    if ((uint32_t)lane < remaining) {
      s0[warp][lane] = n0; s1[warp][lane] = n1; s2[warp][lane] = n2;
      if constexpr (FEAT) s3[warp][lane] = n3;
    }
    __syncwarp();
    gather(start + FWD_BATCH);
    // Fragments are taken FWD_GROUP at a time: first everything that does not depend on the pixels' running state (sigma,
    // the hit test, alpha with its exponential) for the whole group, so that those chains overlap, then the short serial
    // part (transmittance and colour sums) fragment by fragment in list order. The arithmetic per pixel is unchanged.
    for (uint32_t t0 = 0; t0 < remaining; t0 += FWD_GROUP) {
      float alpha[FWD_GROUP][2];
      bool inside[FWD_GROUP][2];
#pragma unroll
      for (int u = 0; u < FWD_GROUP; u++) {
        const uint32_t t = min(t0 + (uint32_t)u, remaining - 1u);   // a short last group recomputes its last fragment, unused
        const float4 a = s0[warp][t], c = s1[warp][t];
        // sigma for the pixel pair in one packed fp32x2 chain (the pixels share the row: dy terms are scalars)
        const float dy = pcy - a.y;
        const float2 dx = make_float2(pcx - a.x, pcx + 1.f - a.x);
        const float2 sigma = __ffma2_rn(dx, __ffma2_rn(dx, make_float2(0.5f * a.z, 0.5f * a.z), make_float2(a.w * dy, a.w * dy)),
                                        make_float2(0.5f * c.x * dy * dy, 0.5f * c.x * dy * dy));
        const bool live = t0 + (uint32_t)u < remaining;
        inside[u][0] = live && sigma.x >= 0.f && sigma.x <= c.w;   // alpha >= 1/255
        inside[u][1] = live && sigma.y >= 0.f && sigma.y <= c.w;
        alpha[u][0] = fminf(ALPHA_MAX, c.y * __expf(-sigma.x));
        alpha[u][1] = fminf(ALPHA_MAX, c.y * __expf(-sigma.y));
      }
#pragma unroll
      for (int u = 0; u < FWD_GROUP; u++) {
        const uint32_t t = t0 + (uint32_t)u;
        bool hit[2] = {!done[0] && inside[u][0], !done[1] && inside[u][1]};
        if (!__any_sync(0xffffffffu, hit[0] || hit[1])) continue;
        const float4 col = s2[warp][t];
        const float cr = fmaxf(col.x, 0.f), cg = fmaxf(col.y, 0.f), cb = fmaxf(col.z, 0.f);
        const float cz = s1[warp][t].z;
#pragma unroll
        for (int p = 0; p < 2; p++) {
          const float next_T = T[p] * (1.f - alpha[u][p]);
          if (hit[p] && next_T <= T_CUTOFF) { done[p] = true; hit[p] = false; }   // stop before the fragment that would saturate the pixel
          if (hit[p]) {
            const float vis = alpha[u][p] * T[p];
            r[p] += cr * vis; g[p] += cg * vis; b[p] += cb * vis;
            if constexpr (DEPTH) zs[p] += vis * cz;
            if constexpr (FEAT) { const float2 fz = s3[warp][t]; f0[p] += col.w * vis; f1[p] += fz.x * vis; f2[p] += fz.y * vis; }
            T[p] = next_T;
            last[p] = start + t + 1;
          }
        }
      }
    }
  }
#pragma unroll
  for (int p = 0; p < 2; p++) {
    if (p == 0 ? in0 : in1) {
      const int pix = py * W + px0 + p;
      out_rgba[pix] = make_float4(r[p] + T[p] * bg.x, g[p] + T[p] * bg.y, b[p] + T[p] * bg.z, 1.f - T[p]);
      if constexpr (CHUNKED) {
        if (FEAT && final) out_feat[pix] = make_float4(f0[p], f1[p], f2[p], T[p]);
        else out_feat[pix] = make_float4(r[p], g[p], b[p], T[p]);
        if constexpr (FEAT) { if (!final) feat_acc[pix] = make_float4(f0[p], f1[p], f2[p], 0.f); }
        if constexpr (DEPTH) out_depth[pix] = !final ? zs[p] : ((1.f - T[p]) > 0.05f ? zs[p] / (1.f - T[p]) : INFINITY);
        last_idx[pix] = last[p] | (done[p] ? DONE_BIT : 0u);
      } else {
        out_feat[pix] = make_float4(f0[p], f1[p], f2[p], T[p]);
        if constexpr (DEPTH) out_depth[pix] = (1.f - T[p]) > 0.05f ? zs[p] / (1.f - T[p]) : INFINITY;
        if constexpr (BWD) last_idx[pix] = last[p];
      }
    }
  }
  if (CHUNKED && !final) {
    const bool open = __any_sync(0xffffffffu, !done[0] || !done[1]);
    if (lane == 0) alive[tile] = open ? 1u : 0u;
  }
  if constexpr (BWD) {
    // The backward never needs to look past the last fragment any pixel used. (A pixel whose last fragment lies in an
    // earlier chunk contributes this chunk's start: an empty range.)
    uint32_t m = max(last[0], last[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) tile_ranges[tile].y = CHUNKED ? min(max(m, range.x), range.y) : m;
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

namespace b2k {
// One chunk of a chunked view (n_chunks > 1), or the whole view (n_chunks <= 1).
int launch_raster_fwd(const B2kCtx* c, const B2kRenderOpts* o, int chunk, int n_chunks, uint32_t* alive, cudaStream_t s) {
  const float3 bg = make_float3(o->bg[0], o->bg[1], o->bg[2]);
  uint2* ranges = (uint2*)c->tile_ranges + (n_chunks > 1 ? (size_t)chunk * c->n_tiles : 0);
#define L(B, D, C, F) raster_fwd_kernel<B, D, C, F><<<div_up(c->n_tiles, FWD_WARPS), FWD_WARPS * 32, 0, s>>>(ranges, c->vals_sorted, (const float4*)c->proj0, \
    (const float4*)c->proj1, (const float4*)c->proj2, c->W, c->H, c->tiles_x, c->n_tiles, bg, (float4*)c->out_rgba, (float4*)c->out_feat, c->out_depth, c->last_idx, \
    chunk, n_chunks, alive, (const float2*)c->proj3, o->bwd_info ? bwd_ckpt_ptr(c) : nullptr, (n_chunks > 1 && o->feat_mode != 0) ? (float4*)c->bwd_scratch : nullptr)
  if (n_chunks > 1 && o->feat_mode != 0) {   // forward only (checked by the caller): the scratch of the backward carries the feature sums
    if (c->out_depth) L(false, true, true, true); else L(false, false, true, true);
  } else if (n_chunks > 1) {
    if (o->bwd_info) { if (c->out_depth) L(true, true, true, false); else L(true, false, true, false); }
    else { if (c->out_depth) L(false, true, true, false); else L(false, false, true, false); }
  } else if (o->feat_mode != 0) {
    if (o->bwd_info) { if (c->out_depth) L(true, true, false, true); else L(true, false, false, true); }
    else { if (c->out_depth) L(false, true, false, true); else L(false, false, false, true); }
  } else {
    if (o->bwd_info) { if (c->out_depth) L(true, true, false, false); else L(true, false, false, false); }
    else { if (c->out_depth) L(false, true, false, false); else L(false, false, false, false); }
  }
#undef L
  return check_launch();
}
}  // namespace b2k

extern "C" int b2k_raster_fwd(const B2kCtx* c, const B2kRenderOpts* o, b2k_stream_t stream) {
  B2K_REQUIRE(c && o && c->tile_ranges && c->vals_sorted && c->proj0 && c->proj1 && c->proj2 && c->out_rgba && c->out_feat);
  B2K_REQUIRE(!o->bwd_info || (c->last_idx && c->bwd_scratch));
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->n_tiles == c->tiles_x * c->tiles_y);
  if (o->bwd_info && c->bwd_scratch_bytes < b2k_bwd_scratch_bytes(c->W, c->H, c->n_chunks, c->isect_cap)) return B2K_ERR_CAPACITY;
  B2K_REQUIRE(o->feat_mode >= 0 && o->feat_mode <= 2 && (o->feat_mode == 0 || c->proj3));
  return launch_raster_fwd(c, o, 0, 1, nullptr, (cudaStream_t)stream);
}
