// Backward through compositing: per-pixel reverse replay of the forward, per-fragment gradients reduced across the
// tile and accumulated per splat. Reference semantics: raster_bwd_kernel (src/gpu/raster_bwd.cu:11-143).
//
// Work decomposition (differs from the reference on purpose):
//   * A tile's fragment list is cut into SEGMENTS of 128 fragments. The forward leaves the per-pixel state (colour
//     sums, transmittance) at every segment boundary (and where a depth chunk of a chunked view hands over to the next),
//     so each segment can be replayed on its own: the colour behind a boundary is the final sum minus the checkpoint.
//     A small kernel lists the (range, segment) items; a persistent grid of independent warps pulls them from a
//     counter. The longest list of a view no longer decides the kernel's duration, and no warp slot idles while another
//     warp still has a thousand fragments to go.
//   * One WARP owns an item; each lane replays two horizontally adjacent pixels on packed fp32x2 arithmetic. A fragment
//     no pixel of the tile sees is rejected after the sigma test; otherwise the pair's math is branch-free (a pixel that
//     does not see the fragment has alpha = 0 and adds exact zeros).
//   * Reduction across the tile: every lane stores its eleven per-fragment partial sums as three 16-byte words into
//     a per-warp shared-memory block; once five fragments are pending, thirty lanes each add up sixteen lanes' worth of
//     one 16-byte column (conflict-free: blocks are skewed by one slot), a single shuffle joins the two halves, and the
//     column's owner issues the global reductions. About 15 warp instructions per fragment against 60 for a shuffle
//     butterfly over the warp; warps never synchronise with each other.
//
// FP32-issue bound: ~90 flops, one ex2 and one rcp per fragment-pixel, plus the reduction.
#include "common.cuh"

namespace b2k {
namespace {

#ifndef B2K_BWD_WARPS
#define B2K_BWD_WARPS 4
#endif
constexpr int BWD_WARPS = B2K_BWD_WARPS;     // warps per CTA (independent: the CTA shape only sets the residency granularity)
constexpr int BWD_BATCH = 32;                // fragments staged per warp and batch
#ifndef B2K_BWD_GROUP
#define B2K_BWD_GROUP 2
#endif
constexpr int BWD_GROUP = B2K_BWD_GROUP;                 // fragments whose state-independent math is issued together
constexpr int RED_F = 5;                     // fragments whose partial sums are pending before a column reduction
constexpr int RED_BLOCK = 33 * 3;            // 16-byte words per pending fragment: 32 lanes x 3 words, one slot of skew
constexpr unsigned FULL = 0xffffffffu;

struct Staged { float4 a, c, col; };         // proj0, proj1, proj2 of one fragment

__device__ __forceinline__ float fast_sqrt(float x) { float r; asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float2 f2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float hsum(float2 v) { return v.x + v.y; }
__device__ __forceinline__ float4 add4(float4 a, float4 b) {
  const float2 lo = __fadd2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y)), hi = __fadd2_rn(make_float2(a.z, a.w), make_float2(b.z, b.w));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// Work list of the replay: one item (range index = chunk * n_tiles + tile, segment) per SEG fragments of every
// non-empty range the forward left. Order is irrelevant (items are independent); work[0] receives the count.
__global__ void __launch_bounds__(256) bwd_items_kernel(const uint2* __restrict__ tile_ranges, int n_ranges, uint2* __restrict__ items, uint32_t* __restrict__ work) {
  const int lane = threadIdx.x & 31;
  for (int q0 = (blockIdx.x * blockDim.x + threadIdx.x) & ~31; q0 < n_ranges; q0 += gridDim.x * blockDim.x) {
    const int q = q0 + lane;
    uint32_t segs = 0;
    if (q < n_ranges) { const uint2 rg = tile_ranges[q]; segs = rg.y > rg.x ? (rg.y - rg.x + SEG_LEN - 1) >> SEG_SHIFT : 0u; }
    uint32_t incl = segs;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(FULL, incl, o); if (lane >= o) incl += u; }
    const uint32_t total = __shfl_sync(FULL, incl, 31);
    if (total == 0u) continue;
    uint32_t base = 0;
    if (lane == 31) base = atomicAdd(work, total);
    base = __shfl_sync(FULL, base, 31) + incl - segs;
    for (uint32_t s = 0; s < segs; s++) items[base + s] = make_uint2((uint32_t)q, s);
  }
}

template <bool CHUNKED>
__global__ void __launch_bounds__(BWD_WARPS * 32) raster_bwd_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ proj2, const float4* __restrict__ out_rgba, const float4* __restrict__ out_feat, const uint32_t* __restrict__ last_idx,
    const float4* __restrict__ v_out, int W, int H, int tiles_x, int n_tiles, float3 bg, float* __restrict__ v_splat, uint32_t* __restrict__ vis_flag,
    float* __restrict__ vis_weight, int n_chunks, const uint2* __restrict__ items, uint32_t* __restrict__ work, const float4* __restrict__ ckpt,
    float out_scale) {
  __shared__ Staged s_frag[BWD_WARPS][BWD_BATCH];
  __shared__ uint32_t s_gid[BWD_WARPS][BWD_BATCH];
  __shared__ __align__(16) float4 s_red[BWD_WARPS][RED_F * RED_BLOCK];
  __shared__ uint32_t s_pending[BWD_WARPS][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Staged* frag = s_frag[warp];
  uint32_t* gids = s_gid[warp];
  float4* red = s_red[warp];
  uint32_t* pending_gid = s_pending[warp];
  const float Wf = (float)W, Hf = (float)H;
  // Column reduction roles: lane = half * 16 + (fragment * 3 + word); halves add slots 0..15 and 16..31.
  const int red_idx = lane & 15, red_f = red_idx / 3, red_w = red_idx - 3 * red_f, red_half = lane >> 4;
  const uint32_t n_items = work[0];

  for (;;) {
    uint32_t it = 0;
    if (lane == 0) it = atomicAdd(work + 1, 1u);
    it = __shfl_sync(FULL, it, 0);
    if (it >= n_items) break;
    const uint2 item = items[it];
    const int q = (int)item.x, chunk = q / n_tiles, tile = q - chunk * n_tiles;
    const uint2 range = tile_ranges[q];
    const uint32_t seg_lo = range.x + (item.y << SEG_SHIFT);
    const uint32_t seg_hi = min(seg_lo + (uint32_t)SEG_LEN, range.y);
    // The state behind this segment: the forward's checkpoint at its far boundary; for the last segment of a range,
    // the state with which the next non-empty range of the tile (a later depth chunk) started; else the final state.
    long long slot = -1;
    if (seg_hi < range.y) {
      slot = (long long)ckpt_slot(range.x, q, item.y + 1u);
    } else {
      for (int c2 = chunk + 1; c2 < n_chunks; c2++) {
        const uint2 r2 = tile_ranges[(size_t)c2 * n_tiles + tile];
        if (r2.y > r2.x) { slot = (long long)ckpt_slot(r2.x, c2 * n_tiles + tile, 0u); break; }
      }
    }
    const int tx = tile % tiles_x, ty = tile / tiles_x;
    const int px0 = tx * RT_W + (lane & 3) * 2, py = ty * RT_W + (lane >> 2);   // this lane's pixel pair (px0, px0 + 1) on row py
    float2 T, Sr, Sg, Sb, vr, vg, vb, vow, inv_fa;
    uint32_t last0 = 0u, last1 = 0u;   // outside the image: sees no fragment
    {
      float T_[2] = {0.f, 0.f}, S_[2][3] = {{0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}}, v_[2][3] = {{0.f, 0.f, 0.f}, {0.f, 0.f, 0.f}}, vow_[2] = {0.f, 0.f}, ifa[2] = {0.f, 0.f};
      uint32_t last[2] = {0u, 0u};
#pragma unroll
      for (int p = 0; p < 2; p++) {
        const int px = px0 + p;
        if (px < W && py < H) {
          const int pix = py * W + px;
          const float4 vo = v_out[pix], fin = out_feat[pix], img = out_rgba[pix];
          const float T_fin = fin.w;
          T_[p] = T_fin;
          v_[p][0] = vo.x; v_[p][1] = vo.y; v_[p][2] = vo.z;
          vow_[p] = (vo.w - (bg.x * vo.x + bg.y * vo.y + bg.z * vo.z)) * T_fin;
          ifa[p] = 1.f / fmaxf(img.w, 1e-5f);
          last[p] = last_idx[pix] & 0x7FFFFFFFu;   // a chunked forward keeps its saturation flag in bit 31
          if (slot >= 0 && last[p] > seg_hi) {     // the pixel went on past this segment: fragments behind it hold colour
            const float4 ck = ckpt[(size_t)slot * RT_PX + lane * 2 + p];
            // Final colour sums: a chunked forward keeps them in out_feat; otherwise the image minus the background term.
            const float3 sum = CHUNKED ? make_float3(fin.x, fin.y, fin.z) : make_float3(img.x - T_fin * bg.x, img.y - T_fin * bg.y, img.z - T_fin * bg.z);
            T_[p] = ck.w;
            S_[p][0] = sum.x - ck.x; S_[p][1] = sum.y - ck.y; S_[p][2] = sum.z - ck.z;
          }
        }
      }
      T = make_float2(T_[0], T_[1]);
      Sr = make_float2(S_[0][0], S_[1][0]); Sg = make_float2(S_[0][1], S_[1][1]); Sb = make_float2(S_[0][2], S_[1][2]);
      vr = make_float2(v_[0][0], v_[1][0]); vg = make_float2(v_[0][1], v_[1][1]); vb = make_float2(v_[0][2], v_[1][2]);
      vow = make_float2(vow_[0], vow_[1]); inv_fa = make_float2(ifa[0], ifa[1]);
      last0 = last[0]; last1 = last[1];
    }
    const float pcx = (float)px0 + 0.5f, pcy = (float)py + 0.5f;
    int n_pending = 0;

    // Column sums of the pending fragments' partials, then one global reduction per non-zero lane of each splat.
    auto flush = [&]() {
      __syncwarp();
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const bool mine = red_idx < 3 * RED_F && red_f < n_pending;
      if (mine) {
        const float4* src = red + red_f * RED_BLOCK + red_half * 48 + red_w;
        float4 acc2 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < 16; s += 2) { acc = add4(acc, src[s * 3]); acc2 = add4(acc2, src[s * 3 + 3]); }
        acc = add4(acc, acc2);
      }
      acc.x += __shfl_xor_sync(FULL, acc.x, 16); acc.y += __shfl_xor_sync(FULL, acc.y, 16);
      acc.z += __shfl_xor_sync(FULL, acc.z, 16); acc.w += __shfl_xor_sync(FULL, acc.w, 16);
      if (mine && red_half == 0) {
        const uint32_t gid = pending_gid[red_f];
        float* o = v_splat + (size_t)gid * GRAD_LANES + red_w * 4;
        // out_scale undoes a scale the caller put on the pixel gradients (1 unless asked for); the blend weight is no gradient.
        acc.x *= out_scale; acc.y *= out_scale;
        if (red_w < 2) { acc.z *= out_scale; acc.w *= out_scale; }
        if (red_w < 2) {   // words 0, 1: xy 2 + conic 3 + rgb 3
          if (acc.x != 0.f) atomicAdd(o, acc.x);
          if (acc.y != 0.f) atomicAdd(o + 1, acc.y);
          if (acc.z != 0.f) atomicAdd(o + 2, acc.z);
          if (acc.w != 0.f) atomicAdd(o + 3, acc.w);
        } else {           // word 2: opacity, refine, blend weight
          if (acc.x != 0.f) atomicAdd(o, acc.x);
          if (acc.y != 0.f) atomicAdd(o + 1, acc.y);
          vis_flag[gid] = 1u;
          if (vis_weight) atomicAdd(vis_weight + gid, acc.z);
        }
      }
      __syncwarp();
      n_pending = 0;
    };

    // The records of a batch are gathered one batch ahead, into registers: the two dependent loads (list entry, then the
    // splat's records) are in flight while the batch behind them is replayed.
    uint32_t n_gid = 0u;
    float4 n_a = make_float4(0.f, 0.f, 0.f, 0.f), n_c = n_a, n_col = n_a;
    auto gather = [&](uint32_t end) {   // the batch that ends at `end`
      if (end <= seg_lo) return;
      const uint32_t cnt = min(end - seg_lo, (uint32_t)BWD_BATCH);
      if ((uint32_t)lane < cnt) {
        n_gid = vals_sorted[end - cnt + lane];
        n_a = proj0[n_gid]; n_c = proj1[n_gid]; n_col = proj2[n_gid];
      }
    };
    gather(seg_hi);
    for (uint32_t batch_end = seg_hi; batch_end > seg_lo;) {
      const uint32_t remaining = batch_end - seg_lo;
      const uint32_t count = remaining < (uint32_t)BWD_BATCH ? remaining : (uint32_t)BWD_BATCH;
      const uint32_t batch_start = batch_end - count;
      __syncwarp();
      if ((uint32_t)lane < count) {
        gids[lane] = n_gid;
        frag[lane].a = n_a; frag[lane].c = n_c; frag[lane].col = n_col;
      }
      __syncwarp();
      gather(batch_start);
      // Fragments are replayed BWD_GROUP at a time: first what does not depend on the pixels' running state (sigma, the
      // visibility test, the exponential, alpha and 1 / (1 - alpha)) for the whole group, so that those chains overlap;
      // then the state-dependent part fragment by fragment, back to front. The arithmetic per pixel is unchanged.
      for (int j0 = (int)count - 1; j0 >= 0; j0 -= BWD_GROUP) {
        float2 g_dx[BWD_GROUP], g_gauss[BWD_GROUP], g_araw[BWD_GROUP], g_alpha[BWD_GROUP], g_ra[BWD_GROUP];
        float g_dy[BWD_GROUP];
        bool g_on0[BWD_GROUP], g_on1[BWD_GROUP];
#pragma unroll
        for (int u = 0; u < BWD_GROUP; u++) {
          const int j = max(j0 - u, 0);   // a short last group recomputes fragment 0, unused
          const uint32_t idx = batch_start + (uint32_t)j;
          const float4 a = frag[j].a, c = frag[j].c;
          // sigma for the pair: the two pixels share the row, so dy and the dy terms are scalars.
          const float dy = pcy - a.y;
          const float2 dx = make_float2(pcx - a.x, pcx + 1.f - a.x);
          const float2 sigma = __ffma2_rn(dx, __ffma2_rn(dx, f2(0.5f * a.z), f2(a.w * dy)), f2(0.5f * c.x * dy * dy));
          const bool live = j0 - u >= 0;
          g_on0[u] = live && idx < last0 && sigma.x >= 0.f && sigma.x <= c.w;
          g_on1[u] = live && idx < last1 && sigma.y >= 0.f && sigma.y <= c.w;
          g_dx[u] = dx; g_dy[u] = dy;
          g_gauss[u] = make_float2(__expf(-sigma.x), __expf(-sigma.y));
          g_araw[u] = __fmul2_rn(f2(c.y), g_gauss[u]);
          // a pixel that does not see the fragment has alpha = 0 and adds exact zeros below
          g_alpha[u] = make_float2(g_on0[u] ? fminf(ALPHA_MAX, g_araw[u].x) : 0.f, g_on1[u] ? fminf(ALPHA_MAX, g_araw[u].y) : 0.f);
          g_ra[u] = make_float2(__fdividef(1.f, 1.f - g_alpha[u].x), __fdividef(1.f, 1.f - g_alpha[u].y));
        }
#pragma unroll
        for (int u = 0; u < BWD_GROUP; u++) {
          const int j = j0 - u;
          const bool on0 = g_on0[u], on1 = g_on1[u];
          if (__ballot_sync(FULL, on0 || on1) == 0) continue;   // nobody in the tile sees this fragment: skip the heavy part
          const float4 a = frag[j].a, c = frag[j].c, col = frag[j].col;
          const float dy = g_dy[u];
          const float2 dx = g_dx[u], gauss = g_gauss[u], a_raw = g_araw[u], alpha = g_alpha[u], ra = g_ra[u];
          const float cr = fmaxf(col.x, 0.f), cg = fmaxf(col.y, 0.f), cb = fmaxf(col.z, 0.f);
          const float2 nra = make_float2(-ra.x, -ra.y);
          const float2 Tb = __fmul2_rn(T, ra);
          const float2 vis = __fmul2_rn(alpha, Tb);
          float2 va = __fmul2_rn(vow, ra);
          va = __ffma2_rn(__ffma2_rn(Sr, nra, __fmul2_rn(Tb, f2(cr))), vr, va);
          va = __ffma2_rn(__ffma2_rn(Sg, nra, __fmul2_rn(Tb, f2(cg))), vg, va);
          va = __ffma2_rn(__ffma2_rn(Sb, nra, __fmul2_rn(Tb, f2(cb))), vb, va);
          // The alpha clamp has zero slope: the geometry and opacity lanes vanish where it is active.
          const bool live0 = on0 && a_raw.x <= ALPHA_MAX, live1 = on1 && a_raw.y <= ALPHA_MAX;
          const float2 av = __fmul2_rn(alpha, va);
          const float2 mvs = make_float2(live0 ? av.x : 0.f, live1 ? av.y : 0.f);          // -v_sigma
          const float2 gx = __fmul2_rn(mvs, __ffma2_rn(dx, f2(a.z), f2(a.w * dy)));
          const float2 gy = __fmul2_rn(mvs, __ffma2_rn(dx, f2(a.w), f2(c.x * dy)));
          const float2 mdx = __fmul2_rn(mvs, dx);
          const float2 og = __fmul2_rn(va, gauss);
          const float2 sx = __fmul2_rn(gx, f2(Wf)), sy = __fmul2_rn(gy, f2(Hf));
          const float2 qq = __ffma2_rn(sx, sx, __fmul2_rn(sy, sy));
          const float2 rf = __fmul2_rn(make_float2(fast_sqrt(qq.x), fast_sqrt(qq.y)), inv_fa);
          // The pair's partial sums of the eleven lanes: xy, conic, rgb (zero where the colour clamp at zero is active),
          // opacity, refine, blend weight.
          const float4 w0 = make_float4(hsum(gx), hsum(gy), -0.5f * hsum(__fmul2_rn(mdx, dx)), -hsum(mdx) * dy);
          const float4 w1 = make_float4(-0.5f * dy * dy * hsum(mvs), col.x < 0.f ? 0.f : hsum(__fmul2_rn(vis, vr)), col.y < 0.f ? 0.f : hsum(__fmul2_rn(vis, vg)),
                                        col.z < 0.f ? 0.f : hsum(__fmul2_rn(vis, vb)));
          const float4 w2 = make_float4((live0 ? og.x : 0.f) + (live1 ? og.y : 0.f), hsum(rf), hsum(vis), 0.f);
          float4* dst = red + n_pending * RED_BLOCK + lane * 3;
          dst[0] = w0; dst[1] = w1; dst[2] = w2;
          if (lane == 0) pending_gid[n_pending] = gids[j];
          Sr = __ffma2_rn(f2(cr), vis, Sr); Sg = __ffma2_rn(f2(cg), vis, Sg); Sb = __ffma2_rn(f2(cb), vis, Sb);
          T = Tb;
          if (++n_pending == RED_F) flush();
        }
      }
      batch_end = batch_start;
    }
    if (n_pending) flush();
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" uint64_t b2k_bwd_scratch_bytes(int32_t W, int32_t H, int32_t n_chunks, uint64_t isect_cap) {
  if (W <= 0 || H <= 0) return 0;
  const uint64_t tiles = (uint64_t)div_up(W, RT_W) * div_up(H, RT_W), chunks = n_chunks > 1 ? (uint64_t)n_chunks : 1u;
  const uint64_t slots = bwd_slots(isect_cap, tiles * chunks);
  return sizeof(uint32_t) * BWD_HEADER_WORDS + sizeof(uint2) * slots + sizeof(float4) * RT_PX * slots;
}

extern "C" int b2k_raster_bwd(const B2kCtx* c, const B2kModel* m, const B2kRenderOpts* o, b2k_stream_t stream) {
  return b2k_raster_bwd_scaled(c, m, o, 1.f, stream);
}

extern "C" int b2k_raster_bwd_scaled(const B2kCtx* c, const B2kModel* m, const B2kRenderOpts* o, float grad_scale, b2k_stream_t stream) {
  B2K_REQUIRE(grad_scale > 0.f && isfinite(grad_scale));
  B2K_REQUIRE(c && m && o && c->tile_ranges && c->vals_sorted && c->proj0 && c->proj1 && c->proj2);
  B2K_REQUIRE(c->out_rgba && c->out_feat && c->last_idx && c->v_out && c->v_splat && c->vis_flag);
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->n_tiles == c->tiles_x * c->tiles_y && c->bwd_scratch);
  if (c->bwd_scratch_bytes < b2k_bwd_scratch_bytes(c->W, c->H, c->n_chunks, c->isect_cap)) return B2K_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  const float3 bg = make_float3(o->bg[0], o->bg[1], o->bg[2]);
  const int chunks = c->n_chunks > 1 ? c->n_chunks : 1;
  uint32_t* work = bwd_work_ptr(c);
  uint2* items = bwd_items_ptr(c);
  B2K_CUDA(cudaMemsetAsync(work, 0, 2 * sizeof(uint32_t), s));
  const int n_ranges = chunks * c->n_tiles;
  bwd_items_kernel<<<min(div_up(n_ranges, 256), sm_count() * 4), 256, 0, s>>>((const uint2*)c->tile_ranges, n_ranges, items, work);
  // Persistent grid: as many CTAs as an SM holds (the shared-memory footprint decides).
  static int per_sm[2] = {0, 0};
  if (!per_sm[chunks > 1]) {
    int k = 0;
    const cudaError_t e = chunks > 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&k, raster_bwd_kernel<true>, BWD_WARPS * 32, 0)
                                     : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&k, raster_bwd_kernel<false>, BWD_WARPS * 32, 0);
    per_sm[chunks > 1] = (e == cudaSuccess && k > 0) ? k : 8;
  }
  const int ctas = sm_count() * per_sm[chunks > 1];
#define L(CH) raster_bwd_kernel<CH><<<ctas, BWD_WARPS * 32, 0, s>>>( \
      (const uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, (const float4*)c->proj1, (const float4*)c->proj2, (const float4*)c->out_rgba, \
      (const float4*)c->out_feat, c->last_idx, (const float4*)c->v_out, c->W, c->H, c->tiles_x, c->n_tiles, bg, c->v_splat, c->vis_flag, m->vis_weight, chunks, \
      items, work, bwd_ckpt_ptr(c), 1.f / grad_scale)
  if (chunks > 1) L(true); else L(false);
#undef L
  return check_launch();
}
