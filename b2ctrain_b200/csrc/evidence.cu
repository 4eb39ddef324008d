// Multi-view evidence and label vote: a forward replay of the composited view that accumulates, per splat, how much of
// its rendered weight fell on target pixels, how well those pixels were explained, and which class the pixels under it
// carry. Reference semantics: evidence_kernel, fold_view_kernel, label_vote_kernel (src/train/evidence.cu:48-196).
//
// Same decomposition as the compositing kernels here: one warp per 8x8 tile, two pixels per lane, fragments staged 32 at
// a time per warp, no block barrier. Per fragment the pair's three weights are reduced across the warp by a halving
// butterfly (6 shuffles for all of them) and leave as one global reduction each; the label vote collects the batch in a
// per-warp [32 fragments][32 classes] table in shared memory first (labels are spatially coherent, so a tile touches a
// handful of bins). A chunked view is walked chunk by chunk, the transmittance running through.
#include "common.cuh"

namespace b2k {
namespace {

constexpr int EV_WARPS = 4, EV_BATCH = 32;
constexpr int LABEL_BINS = 32;              // class ids at or above this are ignored (evidence.cu:44)
constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float unpack8(uint32_t p, int c) { return (float)((p >> (8 * c)) & 0xffu) * (1.f / 255.f); }

// Sum over the warp of four per-lane values: on return lanes 0, 8, 16, 24 hold the totals of v[0], v[1], v[2], v[3].
__device__ __forceinline__ float warp_sum4(float v0, float v1, float v2, float v3, int lane) {
  const bool hi16 = lane & 16;
  float a = (hi16 ? v2 : v0) + __shfl_xor_sync(FULL, hi16 ? v0 : v2, 16);   // lanes < 16 keep {v0, v1}, the others {v2, v3}
  float b = (hi16 ? v3 : v1) + __shfl_xor_sync(FULL, hi16 ? v1 : v3, 16);
  const bool hi8 = lane & 8;
  float c = (hi8 ? b : a) + __shfl_xor_sync(FULL, hi8 ? a : b, 8);
  c += __shfl_xor_sync(FULL, c, 4); c += __shfl_xor_sync(FULL, c, 2); c += __shfl_xor_sync(FULL, c, 1);
  return c;   // group (lane >> 3): 0 -> v0, 1 -> v1, 2 -> v2, 3 -> v3
}

struct PixelPair { int px0, py; bool in0, in1; float pcx, pcy; };
__device__ __forceinline__ PixelPair pair_of(int tile, int tiles_x, int lane, int W, int H) {
  PixelPair p;
  p.px0 = (tile % tiles_x) * RT_W + (lane & 3) * 2; p.py = (tile / tiles_x) * RT_W + (lane >> 2);
  p.in0 = p.px0 < W && p.py < H; p.in1 = p.px0 + 1 < W && p.py < H;
  p.pcx = (float)p.px0 + 0.5f; p.pcy = (float)p.py + 0.5f;
  return p;
}

// vis of one fragment for the pair (0 where the pixel does not take it), transmittance advanced.
__device__ __forceinline__ void pair_vis(const float4 a, const float4 c, const PixelPair& pp, uint32_t idx, const uint32_t (&last)[2], float (&T)[2], float (&vis)[2]) {
  const float dy = pp.pcy - a.y;
#pragma unroll
  for (int p = 0; p < 2; p++) {
    vis[p] = 0.f;
    if (idx < last[p]) {
      const float dx = pp.pcx + (float)p - a.x;
      const float sigma = 0.5f * (a.z * dx * dx + c.x * dy * dy) + a.w * dx * dy;
      if (sigma >= 0.f && sigma <= c.w) { const float alpha = fminf(ALPHA_MAX, c.y * __expf(-sigma)); vis[p] = alpha * T[p]; T[p] *= 1.f - alpha; }
    }
  }
}

template <bool NORMALS>
__global__ void __launch_bounds__(EV_WARPS * 32) evidence_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const float4* __restrict__ out_rgba, const float4* __restrict__ out_feat, const uint32_t* __restrict__ last_idx, const uint32_t* __restrict__ gt,
    const uint32_t* __restrict__ gtn, const uint8_t* __restrict__ weights, int W, int H, int tiles_x, int n_tiles, int n_chunks, int masked_has_alpha,
    float normal_weight, float* __restrict__ acc) {
  __shared__ float4 s0[EV_WARPS][EV_BATCH], s1[EV_WARPS][EV_BATCH];
  __shared__ uint32_t s_gid[EV_WARPS][EV_BATCH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * EV_WARPS + warp;
  if (tile >= n_tiles) return;
  const PixelPair pp = pair_of(tile, tiles_x, lane, W, H);
  float m[2] = {0.f, 0.f}, mres[2] = {0.f, 0.f}, k[2] = {0.f, 0.f}, T[2] = {1.f, 1.f};
  uint32_t last[2] = {0u, 0u};
#pragma unroll
  for (int p = 0; p < 2; p++) {
    if (p == 0 ? pp.in0 : pp.in1) {
      const int pix = pp.py * W + pp.px0 + p;
      const uint32_t g = gt[pix];
      const float ga = unpack8(g, 3), wp = weights ? (float)weights[pix] * (1.f / 255.f) : 1.f;
      const float4 o = out_rgba[pix];
      float res = (fabsf(o.x - unpack8(g, 0)) + fabsf(o.y - unpack8(g, 1)) + fabsf(o.z - unpack8(g, 2))) * (1.f / 3.f);
      if constexpr (NORMALS) {   // L1 + (1 - cosine) against the packed normal target where its mask is set (evidence.cu:71-81)
        const uint32_t gn = gtn[pix];
        if (((gn >> 24) & 0xffu) > 127u) {
          const float gx = (float)(gn & 0xffu) * (2.f / 255.f) - 1.f, gy = 1.f - (float)((gn >> 8) & 0xffu) * (2.f / 255.f), gz = 1.f - (float)((gn >> 16) & 0xffu) * (2.f / 255.f);
          const float4 f = out_feat[pix];
          const float pl = fmaxf(sqrtf(f.x * f.x + f.y * f.y + f.z * f.z), 1e-6f), gl = fmaxf(sqrtf(gx * gx + gy * gy + gz * gz), 1e-6f);
          res += normal_weight * (fabsf(f.x - gx) + fabsf(f.y - gy) + fabsf(f.z - gz) + 1.f - (f.x * gx + f.y * gy + f.z * gz) / (pl * gl));
        }
      }
      m[p] = ga * wp; mres[p] = m[p] * res; k[p] = (masked_has_alpha ? ga : 1.f) * wp;
      last[p] = last_idx[pix] & 0x7FFFFFFFu;
    }
  }
  for (int ch = 0; ch < n_chunks; ch++) {
    const uint2 range = tile_ranges[(size_t)ch * n_tiles + tile];
    for (uint32_t start = range.x; start < range.y; start += EV_BATCH) {
      const uint32_t count = min((uint32_t)EV_BATCH, range.y - start);
      __syncwarp();
      if ((uint32_t)lane < count) { const uint32_t gid = vals_sorted[start + lane]; s_gid[warp][lane] = gid; s0[warp][lane] = proj0[gid]; s1[warp][lane] = proj1[gid]; }
      __syncwarp();
      for (uint32_t t = 0; t < count; t++) {
        float vis[2];
        pair_vis(s0[warp][t], s1[warp][t], pp, start + t, last, T, vis);
        if (__ballot_sync(FULL, vis[0] != 0.f || vis[1] != 0.f) == 0u) continue;
        const float total = warp_sum4(vis[0] * m[0] + vis[1] * m[1], vis[0] * mres[0] + vis[1] * mres[1], vis[0] * k[0] + vis[1] * k[1], 0.f, lane);
        if ((lane & 7) == 0 && lane < 24 && total != 0.f) atomicAdd(acc + (size_t)s_gid[warp][t] * 3 + (lane >> 3), total);
      }
    }
  }
}

// ev[i] += this view's (w_in, w_all, err), w_in^2 and the mass-weighted direction to the camera (evidence.cu:123-136).
__global__ void evidence_fold_kernel(int n, const float* __restrict__ acc, const float4* __restrict__ pos, float3 cam, float* __restrict__ ev) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float w_in = acc[i * 3], err = acc[i * 3 + 1], w_all = acc[i * 3 + 2];
  float* e = ev + (size_t)i * 8;
  e[0] += w_in; e[1] += w_all; e[2] += err; e[7] += w_in * w_in;
  if (w_in != 0.f) {
    const float4 p = pos[i];
    const float dx = cam.x - p.x, dy = cam.y - p.y, dz = cam.z - p.z;
    const float inv = w_in / fmaxf(sqrtf(dx * dx + dy * dy + dz * dz), 1e-12f);
    e[4] += dx * inv; e[5] += dy * inv; e[6] += dz * inv;
  }
}

__global__ void __launch_bounds__(EV_WARPS * 32) label_vote_kernel(
    const uint2* __restrict__ tile_ranges, const uint32_t* __restrict__ vals_sorted, const float4* __restrict__ proj0, const float4* __restrict__ proj1,
    const uint32_t* __restrict__ last_idx, const uint32_t* __restrict__ gt, const uint8_t* __restrict__ labels, const uint8_t* __restrict__ weights, int W, int H,
    int tiles_x, int n_tiles, int n_chunks, int masked_has_alpha, float* __restrict__ votes) {
  __shared__ float4 s0[EV_WARPS][EV_BATCH], s1[EV_WARPS][EV_BATCH];
  __shared__ uint32_t s_gid[EV_WARPS][EV_BATCH];
  __shared__ float s_votes[EV_WARPS][EV_BATCH][LABEL_BINS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * EV_WARPS + warp;
  if (tile >= n_tiles) return;
  const PixelPair pp = pair_of(tile, tiles_x, lane, W, H);
  float k[2] = {0.f, 0.f}, T[2] = {1.f, 1.f};
  int bin[2] = {0, 0};
  uint32_t last[2] = {0u, 0u};
#pragma unroll
  for (int p = 0; p < 2; p++) {
    if (p == 0 ? pp.in0 : pp.in1) {
      const int pix = pp.py * W + pp.px0 + p;
      const float wp = weights ? (float)weights[pix] * (1.f / 255.f) : 1.f;
      k[p] = (masked_has_alpha ? unpack8(gt[pix], 3) : 1.f) * wp;
      bin[p] = labels[pix];
      if (bin[p] >= LABEL_BINS) { k[p] = 0.f; bin[p] = 0; }
      // A pixel without voting weight still composites (its transmittance is not needed by anyone): skip it outright.
      last[p] = k[p] != 0.f ? (last_idx[pix] & 0x7FFFFFFFu) : 0u;
    }
  }
  for (int ch = 0; ch < n_chunks; ch++) {
    const uint2 range = tile_ranges[(size_t)ch * n_tiles + tile];
    for (uint32_t start = range.x; start < range.y; start += EV_BATCH) {
      const uint32_t count = min((uint32_t)EV_BATCH, range.y - start);
      __syncwarp();
      if ((uint32_t)lane < count) { const uint32_t gid = vals_sorted[start + lane]; s_gid[warp][lane] = gid; s0[warp][lane] = proj0[gid]; s1[warp][lane] = proj1[gid]; }
      for (int b = lane; b < EV_BATCH * LABEL_BINS; b += 32) (&s_votes[warp][0][0])[b] = 0.f;
      __syncwarp();
      for (uint32_t t = 0; t < count; t++) {
        float vis[2];
        pair_vis(s0[warp][t], s1[warp][t], pp, start + t, last, T, vis);
        if (vis[0] != 0.f) atomicAdd(&s_votes[warp][t][bin[0]], vis[0] * k[0]);
        if (vis[1] != 0.f) atomicAdd(&s_votes[warp][t][bin[1]], vis[1] * k[1]);
      }
      __syncwarp();
      for (int b = lane; b < (int)count * LABEL_BINS; b += 32) {
        const float v = (&s_votes[warp][0][0])[b];
        if (v != 0.f) atomicAdd(votes + (size_t)s_gid[warp][b / LABEL_BINS] * LABEL_BINS + (b % LABEL_BINS), v);
      }
    }
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

static int check_replay_ctx(const B2kCtx* c) {
  B2K_REQUIRE(c && c->tile_ranges && c->vals_sorted && c->proj0 && c->proj1 && c->out_rgba && c->last_idx);
  B2K_REQUIRE(c->W > 0 && c->H > 0 && c->n_tiles == c->tiles_x * c->tiles_y);
  return B2K_OK;
}

extern "C" int b2k_evidence_view(const B2kCtx* c, const uint32_t* rgba, const uint32_t* normals, const uint8_t* weights, int32_t masked_has_alpha, float normal_weight,
                                 float* acc, b2k_stream_t stream) {
  int st = check_replay_ctx(c);
  if (st) return st;
  B2K_REQUIRE(rgba && acc);
  const bool use_normals = normals != nullptr && normal_weight > 0.f;
  B2K_REQUIRE(!use_normals || c->out_feat);
  const int chunks = c->n_chunks > 1 ? c->n_chunks : 1;
  if (use_normals && chunks > 1) return B2K_ERR_UNSUPPORTED;   // a chunked view has no composited feature lanes
#define L(N) evidence_kernel<N><<<div_up(c->n_tiles, EV_WARPS), EV_WARPS * 32, 0, (cudaStream_t)stream>>>( \
      (const uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, (const float4*)c->proj1, (const float4*)c->out_rgba, (const float4*)c->out_feat, c->last_idx, \
      rgba, normals, weights, c->W, c->H, c->tiles_x, c->n_tiles, chunks, masked_has_alpha, normal_weight, acc)
  if (use_normals) L(true); else L(false);
#undef L
  return check_launch();
}

extern "C" int b2k_evidence_fold(const B2kModel* m, const float* acc, const float* cam_pos, float* evidence, b2k_stream_t stream) {
  B2K_REQUIRE(m && m->pos_op && acc && cam_pos && evidence && m->n >= 0);
  if (m->n == 0) return B2K_OK;
  evidence_fold_kernel<<<div_up(m->n, 256), 256, 0, (cudaStream_t)stream>>>(m->n, acc, (const float4*)m->pos_op, make_float3(cam_pos[0], cam_pos[1], cam_pos[2]), evidence);
  return check_launch();
}

extern "C" int b2k_label_vote(const B2kCtx* c, const uint32_t* rgba, const uint8_t* labels, const uint8_t* weights, int32_t masked_has_alpha, float* votes,
                              b2k_stream_t stream) {
  int st = check_replay_ctx(c);
  if (st) return st;
  B2K_REQUIRE(rgba && labels && votes);
  const int chunks = c->n_chunks > 1 ? c->n_chunks : 1;
  label_vote_kernel<<<div_up(c->n_tiles, EV_WARPS), EV_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (const uint2*)c->tile_ranges, c->vals_sorted, (const float4*)c->proj0, (const float4*)c->proj1, c->last_idx, rgba, labels, weights, c->W, c->H, c->tiles_x, c->n_tiles,
      chunks, masked_has_alpha, votes);
  return check_launch();
}

extern "C" int32_t b2k_label_bins(void) { return LABEL_BINS; }
