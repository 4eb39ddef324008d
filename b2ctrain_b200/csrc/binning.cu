// Binning stage (and, at the end of the file, the front-to-back chunked renderer built from the same kernels):
// depth-keyed radix sort of the splats, scan of tile counts in depth order fused with the emission of
// (tile id, splat index) pairs, stable radix sort by tile id, per-tile ranges. Reference semantics: bin_and_sort
// (src/gpu/binning.cu:109-145) with its kernels (:10-105); the two library sorts and the library scan of the
// reference are replaced by the kernels in this file.
//
// Everything here is integer work bound by HBM traffic. Design points:
//  * No host round trip: the element counts of the later stages (intersections) are read from device memory by
//    persistent kernels whose grids are sized from the SM count, so the whole view is one asynchronous chain.
//  * The radix sort is the wait-free three-kernel form (per-block digit counts, row scan, ranked scatter): no kernel
//    ever spins on another block. Each block owns one contiguous segment and walks it tile by tile, so the count
//    table is 256 x (a few hundred) words whatever the input size.
//  * Scatter is staged through shared memory so global writes go out in digit runs (coalesced), keys and values
//    move as 32-bit words, loads are warp-contiguous.
//  * Sorting is LSD with 8-bit digits and is stable, so order = ascending (key, original position): exactly the
//    order the reference's stable sorts define.
#include "common.cuh"
#include <algorithm>

namespace b2k {
namespace {

constexpr int SORT_THREADS = 256;
constexpr int SORT_ITEMS = 16;
constexpr int COUNT_TILE = SORT_THREADS * SORT_ITEMS;   // 4096 keys per counting step of a CTA
constexpr int SORT_TILE = 4096;                         // pairs per scatter tile (a multiple of COUNT_TILE)
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int RADIX_MAX = 512;                 // widest digit (9 bits): sizes the histogram scratch
constexpr int BLOCKS_PER_SM = 2;               // resident scatter CTAs per SM: one wave covers the input

__device__ __forceinline__ uint32_t seg_len(uint32_t n, uint32_t blocks) {
  uint32_t per = (n + blocks - 1) / blocks;
  return ((per + SORT_TILE - 1) / SORT_TILE) * SORT_TILE;
}
__device__ __forceinline__ uint32_t load_n(const uint32_t* n_ptr, uint32_t n_max) {
  const uint32_t n = *n_ptr;
  return n < n_max ? n : n_max;
}
// A sort may work on a window of its buffers that starts `*off_ptr` elements in (a depth chunk of the view): the
// window's length is clamped to what is left of the buffers.
__device__ __forceinline__ uint32_t load_off(const uint32_t* off_ptr) { return off_ptr ? *off_ptr : 0u; }
__device__ __forceinline__ uint32_t load_n(const uint32_t* n_ptr, uint32_t n_max, uint32_t off) {
  return load_n(n_ptr, off < n_max ? n_max - off : 0u);
}

// Pass kernel 1: digit counts of each block's segment. hist is [RADIX][blocks]. Each lane keeps 16 keys in flight
// (four 128-bit loads) so that a few hundred resident warps cover the HBM latency-bandwidth product.
template <int BITS>
__global__ void __launch_bounds__(SORT_THREADS) radix_count_kernel(const uint32_t* __restrict__ keys_base, const uint32_t* __restrict__ n_ptr, uint32_t n_max,
                                                                   int shift, uint32_t mask, uint32_t* __restrict__ hist, const uint32_t* __restrict__ off_ptr) {
  constexpr int RADIX = 1 << BITS;
  __shared__ uint32_t s_hist[SORT_WARPS][RADIX];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < SORT_WARPS * RADIX; i += SORT_THREADS) (&s_hist[0][0])[i] = 0;
  __syncthreads();
  const uint32_t off = load_off(off_ptr);   // a multiple of 32 elements: 128-bit loads stay aligned
  const uint32_t* __restrict__ keys = keys_base + off;
  const uint32_t n = load_n(n_ptr, n_max, off);
  const uint32_t len = seg_len(n, gridDim.x);
  const uint64_t begin64 = (uint64_t)blockIdx.x * len;
  const uint32_t begin = begin64 < n ? (uint32_t)begin64 : n;
  const uint32_t end = (begin64 + len) < n ? (uint32_t)(begin64 + len) : n;
  // Segments start on a multiple of the tile size, so 128-bit loads are aligned.
  for (uint32_t tile = begin + warp * (32 * SORT_ITEMS); tile < end; tile += COUNT_TILE) {   // warp-uniform trip count
    uint32_t k[SORT_ITEMS];
    if (tile + 32 * SORT_ITEMS <= end) {
#pragma unroll
      for (int v = 0; v < SORT_ITEMS / 4; v++) {
        const uint4 q = *reinterpret_cast<const uint4*>(keys + tile + v * 128 + lane * 4);
        k[v * 4] = q.x; k[v * 4 + 1] = q.y; k[v * 4 + 2] = q.z; k[v * 4 + 3] = q.w;
      }
#pragma unroll
      for (int j = 0; j < SORT_ITEMS; j++) atomicAdd(&s_hist[warp][(k[j] >> shift) & mask], 1u);
    } else {
#pragma unroll
      for (int j = 0; j < SORT_ITEMS; j++) { const uint32_t i = tile + j * 32 + lane; k[j] = i < end ? keys[i] : 0u; }
#pragma unroll
      for (int j = 0; j < SORT_ITEMS; j++)
        if (tile + j * 32 + lane < end) atomicAdd(&s_hist[warp][(k[j] >> shift) & mask], 1u);
    }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < RADIX; d += SORT_THREADS) {
    uint32_t t = 0;
#pragma unroll
    for (int w = 0; w < SORT_WARPS; w++) t += s_hist[w][d];
    hist[(size_t)d * gridDim.x + blockIdx.x] = t;
  }
}

// Pass kernel 2: one block per digit turns its row of per-block counts into exclusive offsets and records the row
// total. blocks <= 1024.
__global__ void __launch_bounds__(1024) radix_rows_kernel(uint32_t* __restrict__ hist, int blocks, uint32_t* __restrict__ totals) {
  __shared__ uint32_t s_warp[32];
  const int d = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
  uint32_t v = t < blocks ? hist[(size_t)d * blocks + t] : 0u;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { uint32_t u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = s_warp[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { uint32_t u = __shfl_up_sync(0xffffffffu, wi, o); if (lane >= o) wi += u; }
    s_warp[lane] = wi - w;
    if (lane == 31) totals[d] = wi;
  }
  __syncthreads();
  if (t < blocks) hist[(size_t)d * blocks + t] = s_warp[warp] + incl - v;
}

// Pass kernel 3: ranked, stable scatter of each block's segment. 512 threads x 8 pairs per tile; the next tile's keys
// and this tile's values are in flight while the current tile is ranked, so memory and ranking phases overlap.
constexpr int SCAT_THREADS = 512;
constexpr int SCAT_ITEMS = SORT_TILE / SCAT_THREADS;   // 8
constexpr int SCAT_WARPS = SCAT_THREADS / 32;
constexpr size_t SCAT_SMEM = 2 * SORT_TILE * sizeof(uint32_t);

template <int BITS>
__global__ void __launch_bounds__(SCAT_THREADS, SCAT_THREADS <= 512 ? 2 : 1) radix_scatter_kernel(
    const uint32_t* __restrict__ keys_in_base, const uint32_t* __restrict__ vals_in_base, uint32_t* __restrict__ keys_out_base,
    uint32_t* __restrict__ vals_out_base, const uint32_t* __restrict__ n_ptr, uint32_t n_max, int shift, uint32_t mask,
    const uint32_t* __restrict__ hist, const uint32_t* __restrict__ totals, const uint32_t* __restrict__ off_ptr) {
  const uint32_t off = load_off(off_ptr);
  const uint32_t* __restrict__ keys_in = keys_in_base + off;
  const uint32_t* __restrict__ vals_in = vals_in_base + off;
  uint32_t* __restrict__ keys_out = keys_out_base + off;
  uint32_t* __restrict__ vals_out = vals_out_base + off;
  constexpr int RADIX = 1 << BITS;
  static_assert(RADIX <= SCAT_THREADS, "one thread per digit in the scans below");
  __shared__ uint32_t s_cnt[SCAT_WARPS][RADIX];   // per-warp digit counts, then per-warp offsets inside the digit
  __shared__ uint32_t s_gbase[RADIX];             // running global slot of the digit for this block
  __shared__ uint32_t s_delta[RADIX];             // global slot = s_delta[digit] + local slot (mod 2^32)
  __shared__ uint32_t s_scan[RADIX / 32];
  extern __shared__ uint32_t s_stage[];           // [2][SORT_TILE]: the tile's keys and values in digit order
  uint32_t* s_keys = s_stage;
  uint32_t* s_vals = s_stage + SORT_TILE;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t lane_lt = (1u << lane) - 1u;
  // Global base of (digit, block): exclusive scan of the digit totals + the block's offset inside the digit.
  {
    uint32_t tot = 0, incl = 0;
    if (tid < RADIX) {
      tot = totals[tid]; incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { uint32_t u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
      if (lane == 31) s_scan[warp] = incl;
    }
    __syncthreads();
    if (tid < RADIX) {
      uint32_t pre = 0;
      for (int w = 0; w < warp; w++) pre += s_scan[w];
      s_gbase[tid] = pre + incl - tot + hist[(size_t)tid * gridDim.x + blockIdx.x];
    }
    __syncthreads();
  }
  const uint32_t n = load_n(n_ptr, n_max, off);
  const uint32_t len = seg_len(n, gridDim.x);
  const uint64_t begin64 = (uint64_t)blockIdx.x * len;
  const uint32_t begin = begin64 < n ? (uint32_t)begin64 : n;
  const uint32_t end = (begin64 + len) < n ? (uint32_t)(begin64 + len) : n;
  // Each warp owns 256 consecutive pairs of the tile; item j of lane l is pair j*32 + l of them, so (j, lane) order is
  // input order.
  const uint32_t wbase = warp * (32 * SCAT_ITEMS);
  uint32_t key[SCAT_ITEMS];
#pragma unroll
  for (int j = 0; j < SCAT_ITEMS; j++) { const uint32_t i = begin + wbase + j * 32 + lane; key[j] = i < end ? keys_in[i] : 0xFFFFFFFFu; }
  for (uint32_t tile = begin; tile < end; tile += SORT_TILE) {
    const uint32_t tile_n = end - tile < SORT_TILE ? end - tile : SORT_TILE;
    const bool full = tile_n == SORT_TILE;
    uint32_t val[SCAT_ITEMS], rank[SCAT_ITEMS];
    if (full) {
#pragma unroll
      for (int j = 0; j < SCAT_ITEMS; j++) val[j] = vals_in[tile + wbase + j * 32 + lane];
    } else {
#pragma unroll
      for (int j = 0; j < SCAT_ITEMS; j++) { const uint32_t li = wbase + j * 32 + lane; val[j] = li < tile_n ? vals_in[tile + li] : 0u; }
    }
    for (int i = tid; i < SCAT_WARPS * RADIX; i += SCAT_THREADS) (&s_cnt[0][0])[i] = 0;
    __syncthreads();
    // Rank of every pair among the warp's pairs with the same digit: the lowest lane holding the digit bumps the warp's counter for the digit (one shared-memory atomic) and hands the old value out.
#pragma unroll
    for (int j = 0; j < SCAT_ITEMS; j++) {
      const bool valid = full || wbase + j * 32 + lane < tile_n;
      const uint32_t d = (key[j] >> shift) & mask;
      uint32_t peers = full ? 0xffffffffu : __ballot_sync(0xffffffffu, valid);   // lanes holding the same digit: one vote per digit bit
#pragma unroll                                                                   // (measured 3x cheaper here than match.any)
      for (int b = 0; b < BITS; b++) {
        const bool bit = (d >> b) & 1u;
        const uint32_t vote = __ballot_sync(0xffffffffu, bit);
        peers &= bit ? vote : ~vote;
      }
      const int leader = __ffs(peers) - 1;
      uint32_t old = 0;
      if (valid && lane == leader) old = atomicAdd(&s_cnt[warp][d], (uint32_t)__popc(peers));
      rank[j] = __shfl_sync(0xffffffffu, old, leader) + __popc(peers & lane_lt);
    }
    __syncthreads();
    // Digit `tid`: the digit's first slot in the tile, and for every warp its first slot inside the digit.
    uint32_t total = 0, incl = 0;
    if (tid < RADIX) {
#pragma unroll
      for (int w = 0; w < SCAT_WARPS; w++) total += s_cnt[w][tid];
      incl = total;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { uint32_t u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
      if (lane == 31) s_scan[warp] = incl;
    }
    __syncthreads();
    if (tid < RADIX) {
      uint32_t pre = 0;
      for (int w = 0; w < warp; w++) pre += s_scan[w];
      uint32_t at = pre + incl - total;       // first slot of the digit
      s_delta[tid] = s_gbase[tid] - at;
      s_gbase[tid] += total;
#pragma unroll
      for (int w = 0; w < SCAT_WARPS; w++) { const uint32_t c = s_cnt[w][tid]; s_cnt[w][tid] = at; at += c; }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < SCAT_ITEMS; j++) {
      if (full || wbase + j * 32 + lane < tile_n) {
        const uint32_t slot = s_cnt[warp][(key[j] >> shift) & mask] + rank[j];
        s_keys[slot] = key[j];
        s_vals[slot] = val[j];
      }
    }
    // Prefetch the next tile's keys; they land while this tile is written out.
    {
      const uint32_t next = tile + SORT_TILE;
#pragma unroll
      for (int j = 0; j < SCAT_ITEMS; j++) { const uint64_t i = (uint64_t)next + wbase + j * 32 + lane; key[j] = i < end ? keys_in[i] : 0xFFFFFFFFu; }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < SCAT_ITEMS; j++) {
      const uint32_t slot = j * SCAT_THREADS + tid;
      if (full || slot < tile_n) {
        const uint32_t k = s_keys[slot];
        const uint32_t dst = s_delta[(k >> shift) & mask] + slot;
        keys_out[dst] = k;
        vals_out[dst] = s_vals[slot];
      }
    }
    __syncthreads();
  }
}

// ---- scan of tile counts in depth order, fused with the emission of intersections ----

constexpr int EMIT_THREADS = 256;

__device__ __forceinline__ uint32_t emit_seg_len(uint32_t n, uint32_t blocks) {
  uint32_t per = (n + blocks - 1) / blocks;
  return ((per + EMIT_THREADS - 1) / EMIT_THREADS) * EMIT_THREADS;
}

__global__ void __launch_bounds__(EMIT_THREADS) count_sums_kernel(int n, const uint32_t* __restrict__ order, const uint32_t* __restrict__ tile_count,
                                                                  uint32_t* __restrict__ block_sums) {
  __shared__ uint32_t s_red[EMIT_THREADS / 32];
  const uint32_t len = emit_seg_len((uint32_t)n, gridDim.x);
  const uint64_t begin = (uint64_t)blockIdx.x * len;
  uint32_t acc = 0;
  for (uint64_t r = begin + threadIdx.x; r < begin + len && r < (uint64_t)n; r += EMIT_THREADS) acc += tile_count[order[r]];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) { uint32_t t = 0; for (int w = 0; w < EMIT_THREADS / 32; w++) t += s_red[w]; block_sums[blockIdx.x] = t; }
}

// Scan of the tile counts in depth order fused with the emission of (tile id, splat index) pairs.
// Thread r owns the r-th nearest splat; the block scan gives its slot range. The 32 splats of a warp own a contiguous
// slot range. Each lane walks the set bits of its own hit mask and drops its (tile, splat) pairs into a per-warp
// shared-memory window at slot - window start; the warp then copies the window out, so every global store
// instruction writes 32 consecutive words. Splats with a large tile box (no mask) are appended to a list with their
// first slot; emit_big_kernel, launched next, fills their slots (the window copy leaves stale words there, which
// emit_big_kernel overwrites).
constexpr int EMIT_WINDOW = 1024;   // slots staged per warp at a time
constexpr size_t EMIT_SMEM = (size_t)(EMIT_THREADS / 32) * EMIT_WINDOW * 2 * sizeof(uint32_t);

__global__ void __launch_bounds__(EMIT_THREADS) scan_emit_kernel(
    int n, const uint32_t* __restrict__ order, const uint32_t* __restrict__ tile_count, const uint32_t* __restrict__ block_sums,
    const uint4* __restrict__ hit_info, int tiles_x, uint32_t cap, uint32_t* __restrict__ tile_off, uint32_t* __restrict__ keys,
    uint32_t* __restrict__ vals, uint32_t* __restrict__ num_isect, uint32_t* __restrict__ big_emit, uint32_t* __restrict__ big_emit_count) {
  __shared__ uint32_t s_warp[EMIT_THREADS / 32];
  __shared__ uint32_t s_base;
  extern __shared__ uint32_t s_win[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t* wk = s_win + (size_t)warp * EMIT_WINDOW * 2;
  uint32_t* wv = wk + EMIT_WINDOW;
  {
    uint32_t acc = 0;
    for (int b = tid; b < (int)blockIdx.x; b += EMIT_THREADS) acc += block_sums[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_warp[warp] = acc;
    __syncthreads();
    if (tid == 0) { uint32_t t = 0; for (int w = 0; w < EMIT_THREADS / 32; w++) t += s_warp[w]; s_base = t; }
    __syncthreads();
  }
  uint32_t running = s_base;
  const uint32_t len = emit_seg_len((uint32_t)n, gridDim.x);
  const uint64_t begin = (uint64_t)blockIdx.x * len;
  // The gathers of a chunk (rank -> splat -> count, hit mask) are issued one chunk ahead, so their two dependent
  // global-memory latencies overlap the emission of the current chunk.
  const uint64_t seg_end = (begin + len) < (uint64_t)n ? begin + len : (uint64_t)n;
  uint32_t i_nx = 0, cnt_nx = 0;
  uint4 hi_nx = make_uint4(0u, 0u, 0u, 0u);
  if (begin + tid < seg_end) { i_nx = order[begin + tid]; cnt_nx = tile_count[i_nx]; if (cnt_nx) hi_nx = hit_info[i_nx]; }
  for (uint64_t r0 = begin; r0 < seg_end; r0 += EMIT_THREADS) {
    const uint64_t r = r0 + tid;
    const bool valid = r < seg_end;
    const uint32_t i = i_nx, cnt = valid ? cnt_nx : 0u;
    const uint4 hi = hi_nx;
    {
      const uint64_t rn = r + EMIT_THREADS;
      cnt_nx = 0; hi_nx = make_uint4(0u, 0u, 0u, 0u);
      if (rn < seg_end) { i_nx = order[rn]; cnt_nx = tile_count[i_nx]; if (cnt_nx) hi_nx = hit_info[i_nx]; }
    }
    uint32_t incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { uint32_t u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
    __syncthreads();   // s_warp reuse
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t pre = 0, tile_total = 0;
#pragma unroll
    for (int w = 0; w < EMIT_THREADS / 32; w++) { const uint32_t v = s_warp[w]; if (w < warp) pre += v; tile_total += v; }
    const uint32_t end = running + pre + incl;
    const uint32_t start = end - cnt;
    if (valid) tile_off[r] = end;
    const bool big = cnt != 0 && hi.z == 0xFFFFFFFFu;
    if (big) { const uint32_t e = atomicAdd(big_emit_count, 1u); big_emit[2 * e] = i; big_emit[2 * e + 1] = start; }
    unsigned long long bits = big ? 0ull : ((unsigned long long)hi.y << 32) | hi.x;   // tiles still to emit, row-major inside the box
    const uint32_t bw = hi.z >> 24, min_x = hi.z & 0xFFFu, min_y = (hi.z >> 12) & 0xFFFu;
    const uint32_t inv_bw = bw ? (65536u + bw - 1u) / bw : 0u;                        // exact x / bw for x < 64
    uint32_t cur = start;                                                            // slot of the next tile of this lane
    const uint32_t wstart = __shfl_sync(0xffffffffu, start, 0), wend = __shfl_sync(0xffffffffu, end, 31);
    for (uint32_t w0 = wstart; w0 < wend; w0 += EMIT_WINDOW) {
      const uint32_t w1 = wend - w0 < (uint32_t)EMIT_WINDOW ? wend : w0 + EMIT_WINDOW;
      while (bits != 0ull && cur < w1) {
        const uint32_t bit = (uint32_t)__ffsll((long long)bits) - 1u;
        bits &= bits - 1ull;
        const uint32_t row = (bit * inv_bw) >> 16, col = bit - row * bw;
        wk[cur - w0] = (min_y + row) * (uint32_t)tiles_x + min_x + col;
        wv[cur - w0] = i;
        cur++;
      }
      __syncwarp();
      for (uint32_t s = w0 + lane; s < w1; s += 32)
        if (s < cap) { keys[s] = wk[s - w0]; vals[s] = wv[s - w0]; }
      __syncwarp();
    }
    running += tile_total;
  }
  if (blockIdx.x == gridDim.x - 1 && tid == 0) *num_isect = running;
}

// One warp per listed big splat: the tile box is re-tested 32 tiles at a time in row-major order and the hits are
// written to the splat's slot range in that order.
__global__ void __launch_bounds__(256) emit_big_kernel(const uint32_t* __restrict__ big_emit, const uint32_t* __restrict__ big_emit_count,
                                                       const float4* __restrict__ proj0, const float4* __restrict__ proj1, int W, int H, int tiles_x,
                                                       int tiles_y, uint32_t cap, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5), count = *big_emit_count;
  for (uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < count; e += warps) {
    const uint32_t i = big_emit[2 * e];
    uint32_t at = big_emit[2 * e + 1];
    const float4 a = proj0[i], b = proj1[i];
    const TileRec rec = make_tile_rec(a.x, a.y, a.z, a.w, b.x, b.w);
    TileBox bb;
    if (!tile_box(rec, W, H, tiles_x, tiles_y, bb)) continue;
    const int bw = bb.max_x - bb.min_x, area = bw * (bb.max_y - bb.min_y);
    for (int t0 = 0; t0 < area; t0 += 32) {
      const int t = t0 + lane;
      const int tx = bb.min_x + t % bw, ty = bb.min_y + t / bw;
      const bool hit = t < area && tile_hit(tx, ty, rec);
      const uint32_t m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const uint32_t s = at + __popc(m & ((1u << lane) - 1u));
        if (s < cap) { keys[s] = (uint32_t)(ty * tiles_x + tx); vals[s] = i; }
      }
      at += __popc(m);
    }
  }
}

__global__ void tile_ranges_kernel(const uint32_t* __restrict__ keys_sorted_base, const uint32_t* __restrict__ n_ptr, uint32_t n_max, uint32_t n_tiles,
                                   uint2* __restrict__ ranges, const uint32_t* __restrict__ off_ptr) {
  const uint32_t off = load_off(off_ptr);
  const uint32_t* __restrict__ keys_sorted = keys_sorted_base + off;
  const uint32_t n = load_n(n_ptr, n_max, off);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint32_t tile = keys_sorted[i];
    const uint32_t prev = i == 0 ? 0xFFFFFFFFu : keys_sorted[i - 1];
    if (i == 0 || tile != prev) {
      if (tile < n_tiles) ranges[tile].x = off + i;
      if (i > 0 && prev < n_tiles) ranges[prev].y = off + i;
    }
    if (i == n - 1 && tile < n_tiles) ranges[tile].y = off + n;
  }
}

__global__ void set_word_kernel(uint32_t* p, uint32_t v) { *p = v; }

struct SortScratch { uint32_t* hist; uint32_t* totals; uint32_t* block_sums; uint32_t* n_word; };

int sort_blocks() { int b = sm_count() * BLOCKS_PER_SM; return b > 1024 ? 1024 : b; }

SortScratch carve(const B2kCtx* c, int blocks) {
  SortScratch s;
  s.hist = sort_tables_ptr(c);
  s.totals = s.hist + (size_t)RADIX_MAX * blocks;
  s.block_sums = s.totals + RADIX_MAX;
  s.n_word = s.block_sums + 1024;   // block_sums holds up to 1024 entries (the emit grid differs from the sort grid)
  return s;
}

// Optional timing marks for b2k_bin_sort_profile: when armed, an event is recorded on the stream at each mark.
struct Marks { cudaEvent_t ev[32]; int n = 0; bool armed = false; };
thread_local Marks g_marks;
void mark(cudaStream_t s) { if (g_marks.armed && g_marks.n < 32) cudaEventRecord(g_marks.ev[g_marks.n++], s); }

// Digit width of a sort over `bits` key bits: 8, except where 9 saves a whole pass (17 or 18 bits, the tile ids of a 4K
// image: two passes instead of three).
int sort_digit_bits(int bits) { return (bits > 16 && bits <= 18) ? 9 : 8; }
int sort_passes(int bits) { const int d = sort_digit_bits(bits); return (bits + d - 1) / d; }

template <int BITS>
int radix_pass(uint32_t* k0, uint32_t* v0, uint32_t* k1, uint32_t* v1, const uint32_t* n_ptr, uint32_t n_max, int shift, uint32_t mask, const SortScratch& sc,
               int blocks, cudaStream_t s, const uint32_t* off_ptr) {
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(radix_scatter_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SCAT_SMEM) != cudaSuccess) return check_launch();
    attr_set[dev] = true;
  }
  radix_count_kernel<BITS><<<blocks, SORT_THREADS, 0, s>>>(k0, n_ptr, n_max, shift, mask, sc.hist, off_ptr);
  radix_rows_kernel<<<1 << BITS, 1024, 0, s>>>(sc.hist, blocks, sc.totals);
  mark(s);
  radix_scatter_kernel<BITS><<<blocks, SCAT_THREADS, SCAT_SMEM, s>>>(k0, v0, k1, v1, n_ptr, n_max, shift, mask, sc.hist, sc.totals, off_ptr);
  mark(s);
  return B2K_OK;
}

// LSD radix sort of (key, value) pairs over bits [0, bits). The element count is read from *n_ptr on the device and
// clamped to n_max. Buffers (k0, v0) hold the input; the result lands in (k0, v0) when sort_passes(bits) is even and in
// (k1, v1) when it is odd.
int radix_sort(uint32_t* k0, uint32_t* v0, uint32_t* k1, uint32_t* v1, const uint32_t* n_ptr, uint32_t n_max, int bits, const SortScratch& sc,
               int blocks, cudaStream_t s, const uint32_t* off_ptr = nullptr) {
  const int digit = sort_digit_bits(bits), passes = sort_passes(bits);
  for (int p = 0; p < passes; p++) {
    const int shift = p * digit;
    const int pb = bits - shift < digit ? bits - shift : digit;
    const uint32_t mask = (1u << pb) - 1u;
    const int st = digit == 9 ? radix_pass<9>(k0, v0, k1, v1, n_ptr, n_max, shift, mask, sc, blocks, s, off_ptr)
                              : radix_pass<8>(k0, v0, k1, v1, n_ptr, n_max, shift, mask, sc, blocks, s, off_ptr);
    if (st) return st;
    uint32_t* t = k0; k0 = k1; k1 = t;
    t = v0; v0 = v1; v1 = t;
  }
  return check_launch();
}


// ---- front-to-back rendering in depth chunks ------------------------------------------------------------------------
// The view's splats are taken in a few chunks of increasing depth rank. A chunk is binned (its intersections emitted,
// sorted by tile, ranged) and composited before the next one is touched, and a tile whose pixels have all reached the
// transmittance cutoff emits nothing from then on: in a dense scene most intersections lie behind saturated pixels and
// are never composited, so they need not be sorted either. Chunk c covers the ranks [V b(c-1), V b(c)) of the V
// splats with a tile box, with b = 1/4^(C-1), ..., 1/16, 1/4, 1 (small chunks first: the nearest splats decide most
// pixels, and every chunk costs a dozen launches whatever its size). The projection of this path leaves tile boxes,
// not hit masks: the ellipse-tile tests run per chunk, on the splats whose box still holds a live tile. Every chunk's
// sorted pairs occupy their own window of the key / value buffers, and a tile has one range per chunk. The words that
// chain the chunks live on the device:
//   words[0] = V, words[1 + c] = first slot of chunk c's window, words[16 + c] = pairs of chunk c.
constexpr int MAX_CHUNKS = 5;
constexpr int CW_V = 0, CW_BASE = 1, CW_COUNT = 16, CW_WORDS = 32;   // the tile-alive flags follow the header

__device__ __forceinline__ void chunk_ranks(const uint32_t* words, int lo_num, int hi_num, uint32_t& r0, uint32_t& r1) {
  const uint64_t V = words[CW_V];
  r0 = (uint32_t)((V * (uint64_t)lo_num) >> 8);
  r1 = (uint32_t)((V * (uint64_t)hi_num) >> 8);
}

// V = number of depth-sorted keys that are not the culled marker (they sort last).
__global__ void chunk_prepare_kernel(const uint32_t* __restrict__ keys_sorted, int n, uint32_t* __restrict__ words) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int lo = 0, hi = n;
  while (lo < hi) { const int mid = (lo + hi) >> 1; if (keys_sorted[mid] != 0xFFFFFFFFu) lo = mid + 1; else hi = mid; }
  words[CW_V] = (uint32_t)lo;
  words[CW_BASE] = 0u;
}

// Summed-area table of the tile-alive flags, (tiles_y + 1) x (tiles_x + 1) words with a zero first row and column:
// "is any tile of this box still alive" becomes four loads, which lets the count and emit kernels drop a splat whose
// whole tile box has died without walking its hit mask. Two short launches: a warp per tile row scans along x, then a
// thread per column accumulates down y (loads of a batch issued together, ahead of its stores).
__global__ void __launch_bounds__(32) alive_sat_rows_kernel(const uint32_t* __restrict__ alive, int tiles_x, uint32_t* __restrict__ sat) {
  const int SX = tiles_x + 1, lane = threadIdx.x, y = blockIdx.x;
  if (y == 0) for (int x = lane; x < SX; x += 32) sat[x] = 0u;
  if (lane == 0) sat[(size_t)(y + 1) * SX] = 0u;
  uint32_t carry = 0;
  for (int x0 = 0; x0 < tiles_x; x0 += 32) {
    const int x = x0 + lane;
    uint32_t v = x < tiles_x ? (alive[(size_t)y * tiles_x + x] != 0u ? 1u : 0u) : 0u;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
    if (x < tiles_x) sat[(size_t)(y + 1) * SX + x + 1] = carry + v;
    carry += __shfl_sync(0xffffffffu, v, 31);
  }
}
__global__ void __launch_bounds__(128) alive_sat_cols_kernel(int tiles_x, int tiles_y, uint32_t* __restrict__ sat) {
  const int SX = tiles_x + 1, x = blockIdx.x * blockDim.x + threadIdx.x + 1;
  if (x >= SX) return;
  uint32_t run = 0;
  for (int y0 = 1; y0 <= tiles_y; y0 += 16) {
    uint32_t v[16];
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = y0 + k <= tiles_y ? sat[(size_t)(y0 + k) * SX + x] : 0u;
#pragma unroll
    for (int k = 0; k < 16; k++) { run += v[k]; if (y0 + k <= tiles_y) sat[(size_t)(y0 + k) * SX + x] = run; }
  }
}

__device__ __forceinline__ uint32_t box_alive(const uint32_t* __restrict__ sat, int SX, int x0, int y0, int x1, int y1) {
  return sat[(size_t)y1 * SX + x1] - sat[(size_t)y0 * SX + x1] - sat[(size_t)y1 * SX + x0] + sat[(size_t)y0 * SX + x0];
}

// Hit mask of a splat whose tile box holds at most 64 tiles: bit (row * width + col) set when the ellipse reaches the
// tile and the tile is still alive (alive == nullptr: every tile is). The flag is looked at first: in the later depth
// chunks most tiles of a box are dead, and the ellipse test is the expensive half.
__device__ __forceinline__ unsigned long long box_hit_mask(const TileRec& rec, int min_x, int min_y, int bw, int bh, const uint32_t* __restrict__ alive,
                                                           int tiles_x) {
  unsigned long long m = 0ull;
  int bit = 0;
  for (int ty = min_y; ty < min_y + bh; ty++)
    for (int tx = min_x; tx < min_x + bw; tx++, bit++)
      if ((!alive || alive[ty * tiles_x + tx] != 0u) && tile_hit(tx, ty, rec)) m |= 1ull << bit;
  return m;
}

// First step of a chunk's count, one thread per rank: a splat whose tile box is empty, or holds no live tile (four
// loads of the summed-area table), emits nothing; the others are appended to the list of their kind, masked boxes and
// big boxes, so that the expensive steps below run on dense lists instead of one live lane per warp.
__global__ void __launch_bounds__(256) chunk_filter_kernel(const uint32_t* __restrict__ words, int lo_num, int hi_num, const uint32_t* __restrict__ order,
                                                           const uint4* __restrict__ hit_info, const uint32_t* __restrict__ sat, int tiles_x,
                                                           uint32_t* __restrict__ fcount, uint32_t* __restrict__ live_list, uint32_t* __restrict__ big_list,
                                                           uint32_t* __restrict__ counts) {
  uint32_t r0, r1;
  chunk_ranks(words, lo_num, hi_num, r0, r1);
  const int lane = threadIdx.x & 31;
  const uint32_t span = (r1 - r0 + 31u) & ~31u;   // whole warps, so the votes below are convergent
  const uint32_t T = gridDim.x * blockDim.x;
  constexpr int U = 4;   // ranks per thread and round: three dependent loads each (rank -> splat -> box -> table), kept in flight together
  for (uint32_t q = blockIdx.x * blockDim.x + threadIdx.x; q < span; q += U * T) {
    uint32_t idx[U];
    uint4 hi[U];
    int kind[U];   // 0 emits nothing, 1 masked box, 2 big box
#pragma unroll
    for (int u = 0; u < U; u++) { const uint32_t r = r0 + q + u * T; idx[u] = r < r1 ? order[r] : 0xFFFFFFFFu; }
#pragma unroll
    for (int u = 0; u < U; u++) hi[u] = idx[u] != 0xFFFFFFFFu ? hit_info[idx[u]] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int u = 0; u < U; u++) {
      kind[u] = 0;
      if (hi[u].w != 0u) {
        int x0, y0, x1, y1;
        if (hi[u].z == 0xFFFFFFFFu) { x0 = (int)(hi[u].x & 0xFFFFu); y0 = (int)(hi[u].x >> 16); x1 = x0 + (int)(hi[u].y & 0xFFFFu); y1 = y0 + (int)(hi[u].y >> 16); kind[u] = 2; }
        else { x0 = (int)(hi[u].z & 0xFFFu); y0 = (int)((hi[u].z >> 12) & 0xFFFu); x1 = x0 + (int)(hi[u].z >> 24); y1 = y0 + (int)hi[u].w; kind[u] = 1; }
        if (sat && box_alive(sat, tiles_x + 1, x0, y0, x1, y1) == 0u) kind[u] = 0;
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      if (q + u * T >= span) break;   // warp-uniform: q + u * T and span are whole warps apart
      const uint32_t r = r0 + q + u * T;
      if (r < r1 && kind[u] == 0) fcount[r] = 0u;
#pragma unroll
      for (int k = 1; k <= 2; k++) {   // one atomic per warp and list
        const uint32_t m = __ballot_sync(0xffffffffu, kind[u] == k);
        if (m) {
          uint32_t base = 0;
          if (lane == __ffs(m) - 1) base = atomicAdd(counts + (k - 1), (uint32_t)__popc(m));
          base = __shfl_sync(0xffffffffu, base, __ffs(m) - 1);
          if (kind[u] == k) (k == 1 ? live_list : big_list)[base + __popc(m & ((1u << lane) - 1u))] = r;
        }
      }
    }
  }
}

// Second step, one thread per listed masked-box splat: the ellipse-tile tests the projection left out, the count of
// hits on live tiles, and for a splat that emits its hit mask (kept for the emission).
__global__ void __launch_bounds__(256) chunk_mask_kernel(const uint32_t* __restrict__ live_list, const uint32_t* __restrict__ counts,
                                                         const uint32_t* __restrict__ order, uint4* __restrict__ hit_info, const float4* __restrict__ proj0,
                                                         const float4* __restrict__ proj1, const uint32_t* __restrict__ alive, int tiles_x,
                                                         uint32_t* __restrict__ fcount) {
  const uint32_t count = counts[0];
  for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < count; e += gridDim.x * blockDim.x) {
    const uint32_t r = live_list[e], i = order[r];
    const uint4 hi = hit_info[i];
    const uint32_t bw = hi.z >> 24, min_x = hi.z & 0xFFFu, min_y = (hi.z >> 12) & 0xFFFu, bh = hi.w;
    const float4 a = proj0[i], b = proj1[i];
    const TileRec rec = make_tile_rec(a.x, a.y, a.z, a.w, b.x, b.w);
    // The mask kept for the emission holds the hits on live tiles only: the emission then needs no flag lookups.
    const unsigned long long m = box_hit_mask(rec, (int)min_x, (int)min_y, (int)bw, (int)bh, alive, tiles_x);
    const uint32_t f = (uint32_t)__popcll(m);
    if (f) hit_info[i] = make_uint4((uint32_t)m, (uint32_t)(m >> 32), hi.z, hi.w);
    fcount[r] = f;
  }
}

// The hit words (one ballot per 32 tiles) of the e-th listed big box live in a fixed slot of BALLOT_WORDS words, written
// by the count pass and read back by the emission, which then makes no ellipse tests of its own. Boxes above
// 32 * BALLOT_WORDS tiles, and entries past the end of the buffer, have no slot (0xFFFFFFFF) and are tested twice.
constexpr uint32_t BALLOT_WORDS = 16;
__device__ __forceinline__ uint32_t ballot_slot(uint32_t e, int area, uint32_t cap_words) {
  return (area <= (int)(32u * BALLOT_WORDS) && (uint64_t)(e + 1u) * BALLOT_WORDS <= (uint64_t)cap_words) ? e * BALLOT_WORDS : 0xFFFFFFFFu;
}

// Second step for the listed big-box splats, one warp each: lanes sweep the box 32 tiles at a time.
__global__ void __launch_bounds__(256) chunk_count_big_kernel(const uint32_t* __restrict__ big_list, const uint32_t* __restrict__ counts,
                                                              const uint32_t* __restrict__ order, const uint4* __restrict__ hit_info,
                                                              const float4* __restrict__ proj0, const float4* __restrict__ proj1, int tiles_x,
                                                              const uint32_t* __restrict__ alive, uint32_t* __restrict__ fcount,
                                                              uint32_t* __restrict__ ballots, uint32_t ballot_cap) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5), count = counts[1];
  for (uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < count; e += warps) {
    const uint32_t r = big_list[e], i = order[r];
    const uint4 hi = hit_info[i];
    const float4 a = proj0[i], b = proj1[i];
    const TileRec rec = make_tile_rec(a.x, a.y, a.z, a.w, b.x, b.w);
    const int min_x = (int)(hi.x & 0xFFFFu), min_y = (int)(hi.x >> 16), bw = (int)(hi.y & 0xFFFFu), area = bw * (int)(hi.y >> 16);
    const uint32_t keep = ballot_slot(e, area, ballot_cap);   // where this box's hit words go for its emission
    uint32_t hits = 0;
    for (int t0 = 0; t0 < area; t0 += 32) {
      const int t = t0 + lane;
      const int tx = min_x + t % bw, ty = min_y + t / bw;
      const bool hit = t < area && (!alive || alive[ty * tiles_x + tx] != 0u) && tile_hit(tx, ty, rec);
      const uint32_t m = __ballot_sync(0xffffffffu, hit);
      hits += __popc(m);
      if (keep != 0xFFFFFFFFu && lane == 0) ballots[keep + (uint32_t)(t0 >> 5)] = m;
    }
    if (lane == 0) fcount[r] = hits;
  }
}

__global__ void __launch_bounds__(EMIT_THREADS) chunk_sums_kernel(const uint32_t* __restrict__ words, int lo_num, int hi_num,
                                                                  const uint32_t* __restrict__ fcount, uint32_t* __restrict__ block_sums) {
  __shared__ uint32_t s_red[EMIT_THREADS / 32];
  uint32_t r0, r1;
  chunk_ranks(words, lo_num, hi_num, r0, r1);
  const uint32_t len = emit_seg_len(r1 - r0, gridDim.x);
  const uint64_t begin = (uint64_t)r0 + (uint64_t)blockIdx.x * len;
  uint32_t acc = 0;
  for (uint64_t r = begin + threadIdx.x; r < begin + len && r < (uint64_t)r1; r += EMIT_THREADS) acc += fcount[r];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) { uint32_t t = 0; for (int w = 0; w < EMIT_THREADS / 32; w++) t += s_red[w]; block_sums[blockIdx.x] = t; }
}

// scan_emit_kernel for one chunk: counts come from fcount, the stored masks hold live tiles only, slots start at the
// chunk's window.
// The last block records the chunk's pair count, the next window's first slot (rounded up to 32 so that the sort's
// vector loads stay aligned) and the running total of the view.
__global__ void __launch_bounds__(EMIT_THREADS) chunk_emit_kernel(
    uint32_t* __restrict__ words, int chunk, int lo_num, int hi_num, const uint32_t* __restrict__ order, const uint32_t* __restrict__ fcount,
    const uint32_t* __restrict__ block_sums, const uint4* __restrict__ hit_info, int tiles_x, uint32_t cap,
    uint32_t* __restrict__ big_start, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals, uint32_t* __restrict__ num_isect) {
  __shared__ uint32_t s_warp[EMIT_THREADS / 32];
  __shared__ uint32_t s_base;
  extern __shared__ uint32_t s_win[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t* wk = s_win + (size_t)warp * EMIT_WINDOW * 2;
  uint32_t* wv = wk + EMIT_WINDOW;
  const uint32_t window = words[CW_BASE + chunk];
  {
    uint32_t acc = 0;
    for (int b = tid; b < (int)blockIdx.x; b += EMIT_THREADS) acc += block_sums[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_warp[warp] = acc;
    __syncthreads();
    if (tid == 0) { uint32_t t = 0; for (int w = 0; w < EMIT_THREADS / 32; w++) t += s_warp[w]; s_base = t; }
    __syncthreads();
  }
  uint32_t running = window + s_base;
  uint32_t r0, r1;
  chunk_ranks(words, lo_num, hi_num, r0, r1);
  const uint32_t len = emit_seg_len(r1 - r0, gridDim.x);
  const uint64_t begin = (uint64_t)r0 + (uint64_t)blockIdx.x * len;
  const uint64_t seg_end = (begin + len) < (uint64_t)r1 ? begin + len : (uint64_t)r1;
  uint32_t cnt_nx = begin + tid < seg_end ? fcount[begin + tid] : 0u;   // counts are fetched one group ahead
  for (uint64_t q0 = begin; q0 < seg_end; q0 += EMIT_THREADS) {
    const uint64_t r = q0 + tid;
    const bool valid = r < seg_end;
    const uint32_t cnt = cnt_nx;
    cnt_nx = r + EMIT_THREADS < seg_end ? fcount[r + EMIT_THREADS] : 0u;
    if (!__syncthreads_or(cnt != 0u)) continue;   // in the later chunks most groups of 256 ranks emit nothing at all
    uint32_t i = 0;
    uint4 hi = make_uint4(0u, 0u, 0u, 0u);
    if (valid && cnt) { i = order[r]; hi = hit_info[i]; }
    uint32_t incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { uint32_t u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
    __syncthreads();   // s_warp reuse
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    uint32_t pre = 0, tile_total = 0;
#pragma unroll
    for (int w = 0; w < EMIT_THREADS / 32; w++) { const uint32_t v = s_warp[w]; if (w < warp) pre += v; tile_total += v; }
    const uint32_t end = running + pre + incl;
    const uint32_t start = end - cnt;
    const bool big = cnt != 0 && hi.z == 0xFFFFFFFFu;
    if (big) big_start[r] = start;
    unsigned long long bits = big ? 0ull : ((unsigned long long)hi.y << 32) | hi.x;
    const uint32_t bw = hi.z >> 24, min_x = hi.z & 0xFFFu, min_y = (hi.z >> 12) & 0xFFFu;
    const uint32_t inv_bw = bw ? (65536u + bw - 1u) / bw : 0u;
    uint32_t cur = start;
    const uint32_t wstart = __shfl_sync(0xffffffffu, start, 0), wend = __shfl_sync(0xffffffffu, end, 31);
    for (uint32_t w0 = wstart; w0 < wend; w0 += EMIT_WINDOW) {
      const uint32_t w1 = wend - w0 < (uint32_t)EMIT_WINDOW ? wend : w0 + EMIT_WINDOW;
      while (bits != 0ull && cur < w1) {
        const uint32_t bit = (uint32_t)__ffsll((long long)bits) - 1u;
        bits &= bits - 1ull;
        const uint32_t row = (bit * inv_bw) >> 16, col = bit - row * bw;
        const uint32_t tile = (min_y + row) * (uint32_t)tiles_x + min_x + col;   // the stored mask holds live tiles only
        wk[cur - w0] = tile;
        wv[cur - w0] = i;
        cur++;
      }
      __syncwarp();
      for (uint32_t s = w0 + lane; s < w1; s += 32)
        if (s < cap) { keys[s] = wk[s - w0]; vals[s] = wv[s - w0]; }
      __syncwarp();
    }
    running += tile_total;
  }
  if (blockIdx.x == gridDim.x - 1 && tid == 0) {
    const uint32_t pairs = running - window;
    words[CW_COUNT + chunk] = pairs;
    words[CW_BASE + chunk + 1] = (running + 31u) & ~31u;
    *num_isect = running;
  }
}

__global__ void __launch_bounds__(256) chunk_emit_big_kernel(const uint32_t* __restrict__ big_list, const uint32_t* __restrict__ counts,
                                                             const uint32_t* __restrict__ order, const uint4* __restrict__ hit_info,
                                                             const uint32_t* __restrict__ fcount, const uint32_t* __restrict__ big_start,
                                                             const float4* __restrict__ proj0, const float4* __restrict__ proj1, int tiles_x,
                                                             const uint32_t* __restrict__ alive, uint32_t cap, uint32_t* __restrict__ keys,
                                                             uint32_t* __restrict__ vals, const uint32_t* __restrict__ ballots, uint32_t ballot_cap) {
  const int lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5), count = counts[1];
  for (uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < count; e += warps) {
    const uint32_t r = big_list[e];
    if (fcount[r] == 0u) continue;   // no live tile of the box is hit
    const uint32_t i = order[r];
    uint32_t at = big_start[r];
    const uint4 hi = hit_info[i];
    const float4 a = proj0[i], b = proj1[i];
    const TileRec rec = make_tile_rec(a.x, a.y, a.z, a.w, b.x, b.w);
    const int min_x = (int)(hi.x & 0xFFFFu), min_y = (int)(hi.x >> 16), bw = (int)(hi.y & 0xFFFFu), area = bw * (int)(hi.y >> 16);
    const uint32_t kept = ballot_slot(e, area, ballot_cap);   // the count pass left this box's hit words there, unless it had no room
    for (int t0 = 0; t0 < area; t0 += 32) {
      const int t = t0 + lane;
      const int tx = min_x + t % bw, ty = min_y + t / bw;
      uint32_t m;
      if (kept != 0xFFFFFFFFu) m = ballots[kept + (uint32_t)(t0 >> 5)];
      else m = __ballot_sync(0xffffffffu, t < area && (!alive || alive[ty * tiles_x + tx] != 0u) && tile_hit(tx, ty, rec));
      const bool hit = (m >> lane) & 1u;
      if (hit) {
        const uint32_t s = at + __popc(m & ((1u << lane) - 1u));
        if (s < cap) { keys[s] = (uint32_t)(ty * tiles_x + tx); vals[s] = i; }
      }
      at += __popc(m);
    }
  }
}

}  // namespace
}  // namespace b2k

using namespace b2k;

extern "C" uint64_t b2k_sort_tmp_bytes(int32_t n, uint64_t isect_cap) {
  (void)isect_cap;
  const int blocks = 1024;   // upper bound of sort_blocks()
  const uint64_t n_cap = n > 0 ? (uint64_t)n : 0;
  return (uint64_t)sizeof(uint32_t) * (BIG_HEADER_WORDS + 3 * n_cap + (uint64_t)RADIX_MAX * blocks + RADIX_MAX + blocks + 16);
}

extern "C" int b2k_bin_sort(const B2kCtx* c, int32_t n, b2k_stream_t stream) {
  B2K_REQUIRE(c && n >= 0);
  B2K_REQUIRE(c->tile_ranges && c->num_isect && c->n_tiles == c->tiles_x * c->tiles_y && c->tile_bits >= 1 && c->tile_bits <= 24);
  cudaStream_t s = (cudaStream_t)stream;
  B2K_CUDA(cudaMemsetAsync(c->tile_ranges, 0, sizeof(uint32_t) * 2 * (size_t)c->n_tiles, s));
  if (n == 0) { B2K_CUDA(cudaMemsetAsync(c->num_isect, 0, sizeof(uint32_t), s)); return B2K_OK; }
  B2K_REQUIRE(c->proj0 && c->proj1 && c->tile_count && c->hit_info && c->depth_keys && c->depth_keys_sorted && c->order_in && c->order && c->tile_off);
  B2K_REQUIRE(c->keys && c->vals && c->keys_sorted && c->vals_sorted && c->sort_tmp);
  if (c->n_cap < n) return B2K_ERR_CAPACITY;
  if (c->sort_tmp_bytes < b2k_sort_tmp_bytes(c->n_cap, c->isect_cap) || c->isect_cap == 0 || c->isect_cap > 0xFFFFFFF0ull) return B2K_ERR_CAPACITY;
  const int blocks = sort_blocks();
  const SortScratch sc = carve(c, blocks);
  // 1. Splats by depth: key = bits of view z (culled splats carry 0xFFFFFFFF and land last), value = index. The
  //    projection left its keys and indices in the (depth_keys_sorted, order) pair: with four passes (an even count)
  //    the ping-pong returns to the pair it started from, so the sorted result lands where callers expect it and
  //    (depth_keys, order_in) is the scratch pair.
  set_word_kernel<<<1, 1, 0, s>>>(sc.n_word, (uint32_t)n);
  mark(s);
  int st = radix_sort(c->depth_keys_sorted, c->order, c->depth_keys, c->order_in, sc.n_word, (uint32_t)n, 32, sc, blocks, s);
  if (st) return st;
  // 2 + 3. Scan of the counts in depth order and emission, into the pair the tile sort will read first.
  const int tile_passes = sort_passes(c->tile_bits);
  uint32_t* ek = (tile_passes % 2 == 0) ? c->keys_sorted : c->keys;
  uint32_t* ev = (tile_passes % 2 == 0) ? c->vals_sorted : c->vals;
  uint32_t* ok = (tile_passes % 2 == 0) ? c->keys : c->keys_sorted;
  uint32_t* ov = (tile_passes % 2 == 0) ? c->vals : c->vals_sorted;
  uint32_t* big_emit_count = big_count_ptr(c) + 1;
  B2K_CUDA(cudaMemsetAsync(big_emit_count, 0, sizeof(uint32_t), s));
  const int emit_blocks = sm_count() * 4 > 1024 ? 1024 : sm_count() * 4;
  count_sums_kernel<<<emit_blocks, EMIT_THREADS, 0, s>>>(n, c->order, c->tile_count, sc.block_sums);
  {
    static bool emit_attr[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !emit_attr[dev]) {
      B2K_CUDA(cudaFuncSetAttribute(scan_emit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EMIT_SMEM));
      emit_attr[dev] = true;
    }
  }
  scan_emit_kernel<<<emit_blocks, EMIT_THREADS, EMIT_SMEM, s>>>(n, c->order, c->tile_count, sc.block_sums, (const uint4*)c->hit_info, c->tiles_x,
                                                  (uint32_t)c->isect_cap, c->tile_off, ek, ev, c->num_isect, big_emit_ptr(c), big_emit_count);
  emit_big_kernel<<<sm_count() * 8, 256, 0, s>>>(big_emit_ptr(c), big_emit_count, (const float4*)c->proj0, (const float4*)c->proj1, c->W, c->H,
                                                 c->tiles_x, c->tiles_y, (uint32_t)c->isect_cap, ek, ev);
  mark(s);
  st = check_launch();
  if (st) return st;
  // 4. Stable sort by tile id: depth order survives inside each tile.
  st = radix_sort(ek, ev, ok, ov, c->num_isect, (uint32_t)c->isect_cap, c->tile_bits, sc, blocks, s);
  if (st) return st;
  tile_ranges_kernel<<<sm_count() * 8, 256, 0, s>>>(c->keys_sorted, c->num_isect, (uint32_t)c->isect_cap, (uint32_t)c->n_tiles, (uint2*)c->tile_ranges, nullptr);
  mark(s);
  return check_launch();
}

extern "C" int b2k_render_chunked(const B2kModel* m, const B2kCamera* cam, const B2kRenderOpts* o, const B2kCtx* c, b2k_stream_t stream) {
  B2K_REQUIRE(m && cam && o && c);
  const int C = c->n_chunks;
  B2K_REQUIRE(C >= 2 && C <= MAX_CHUNKS && c->chunk_words && c->last_idx && c->tile_off && c->depth_keys);
  B2K_REQUIRE(!o->bwd_info || c->bwd_scratch);
  if (o->bwd_info && c->bwd_scratch_bytes < b2k_bwd_scratch_bytes(c->W, c->H, C, c->isect_cap)) return B2K_ERR_CAPACITY;
  if (o->feat_mode != 0) {   // out_feat.xyz carries the colour sums between chunks: the feature sums ride in the backward's scratch
    if (o->bwd_info) return B2K_ERR_UNSUPPORTED;
    B2K_REQUIRE(o->feat_mode >= 1 && o->feat_mode <= 2 && c->proj3 && c->bwd_scratch && (o->feat_mode != 2 || o->feat_buffer));
    if (c->bwd_scratch_bytes < sizeof(float4) * (uint64_t)c->W * (uint64_t)c->H) return B2K_ERR_CAPACITY;
  }
  B2K_REQUIRE(c->tile_ranges && c->num_isect && c->n_tiles == c->tiles_x * c->tiles_y && c->tile_bits >= 1 && c->tile_bits <= 24);
  B2K_REQUIRE(c->out_rgba && c->out_feat && c->keys && c->vals && c->keys_sorted && c->vals_sorted && c->sort_tmp);
  cudaStream_t s = (cudaStream_t)stream;
  const int n = m->n;
  B2K_REQUIRE(n >= 0 && m->cap >= n && m->degree >= 0 && m->degree <= 4 && c->proj0 && c->proj1 && c->proj2 && c->tile_count && c->hit_info);
  B2K_REQUIRE(c->depth_keys_sorted && c->order && c->order_in);
  B2K_REQUIRE(cam->W == c->W && cam->H == c->H && c->tiles_x == div_up(c->W, RT_W) && c->tiles_y == div_up(c->H, RT_W));
  int st = B2K_OK;
  if (n > 0) {
    B2K_REQUIRE(m->pos_op && m->quat && m->lscale && m->sh_dc && (m->degree == 0 || m->sh_hi));
    if (c->n_cap < n) return B2K_ERR_CAPACITY;
    st = launch_project_lite(m, cam, o, c, s);
    if (st) return st;
  }
  B2K_CUDA(cudaMemsetAsync(c->tile_ranges, 0, sizeof(uint32_t) * 2 * (size_t)c->n_tiles * C, s));
  if (n == 0) {
    B2K_CUDA(cudaMemsetAsync(c->num_isect, 0, sizeof(uint32_t), s));
    for (int ch = 0; ch < C; ch++) { st = launch_raster_fwd(c, o, ch, C, c->chunk_words + CW_WORDS, s); if (st) return st; }
    return B2K_OK;
  }
  if (c->n_cap < n) return B2K_ERR_CAPACITY;
  if (c->sort_tmp_bytes < b2k_sort_tmp_bytes(c->n_cap, c->isect_cap) || c->isect_cap == 0 || c->isect_cap > 0x7FFFFFF0ull) return B2K_ERR_CAPACITY;
  const int blocks = sort_blocks();
  const SortScratch sc = carve(c, blocks);
  uint32_t* words = c->chunk_words;
  uint32_t* alive = words + CW_WORDS;
  uint32_t* sat = alive + c->n_tiles;
  // Splats by depth, exactly as in b2k_bin_sort.
  set_word_kernel<<<1, 1, 0, s>>>(sc.n_word, (uint32_t)n);
  st = radix_sort(c->depth_keys_sorted, c->order, c->depth_keys, c->order_in, sc.n_word, (uint32_t)n, 32, sc, blocks, s);
  if (st) return st;
  chunk_prepare_kernel<<<1, 32, 0, s>>>(c->depth_keys_sorted, n, words);
  const int tile_passes = sort_passes(c->tile_bits);
  uint32_t* ek = (tile_passes % 2 == 0) ? c->keys_sorted : c->keys;
  uint32_t* ev = (tile_passes % 2 == 0) ? c->vals_sorted : c->vals;
  uint32_t* ok = (tile_passes % 2 == 0) ? c->keys : c->keys_sorted;
  uint32_t* ov = (tile_passes % 2 == 0) ? c->vals : c->vals_sorted;
  uint32_t* fcount = c->depth_keys;          // scratch pair of the depth sort: free from here on
  uint32_t* big_start = c->tile_off;         // first slot of each listed big-box splat, by rank
  uint32_t* live_list = big_emit_ptr(c);                    // ranks of the chunk's masked-box splats with a live tile in the box
  uint32_t* big_list = big_emit_ptr(c) + (size_t)c->n_cap;  // the same for big-box splats
  uint32_t* list_counts = big_count_ptr(c) + 2;             // entries of the two lists
  // Hit words of the big boxes (see ballot_slot) go to the spare key buffer of the tile sort, free until the chunk's sort
  // starts; with an odd number of sort passes that buffer holds the earlier chunks' results, and the emission re-tests.
  uint32_t* ballots = (tile_passes % 2 == 0) ? ok : nullptr;
  const uint32_t ballot_cap = ballots ? (uint32_t)std::min<uint64_t>(c->isect_cap, 0xFFFFFFF0ull) : 0u;
  {
    static bool emit_attr[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !emit_attr[dev]) {
      B2K_CUDA(cudaFuncSetAttribute(chunk_emit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)EMIT_SMEM));
      emit_attr[dev] = true;
    }
  }
  const int emit_blocks = sm_count() * 4 > 1024 ? 1024 : sm_count() * 4;
  for (int ch = 0; ch < C; ch++) {
    const int lo = ch == 0 ? 0 : 256 >> (2 * (C - ch)), hi = 256 >> (2 * (C - 1 - ch));
    const uint32_t* live = ch == 0 ? nullptr : alive;   // the first chunk meets only live tiles
    B2K_CUDA(cudaMemsetAsync(list_counts, 0, 2 * sizeof(uint32_t), s));
    if (live) {
      alive_sat_rows_kernel<<<c->tiles_y, 32, 0, s>>>(live, c->tiles_x, sat);
      alive_sat_cols_kernel<<<div_up(c->tiles_x + 1, 128), 128, 0, s>>>(c->tiles_x, c->tiles_y, sat);
    }
    chunk_filter_kernel<<<sm_count() * 8, 256, 0, s>>>(words, lo, hi, c->order, (const uint4*)c->hit_info, live ? sat : nullptr, c->tiles_x, fcount,
                                                       live_list, big_list, list_counts);
    chunk_mask_kernel<<<sm_count() * 8, 256, 0, s>>>(live_list, list_counts, c->order, (uint4*)c->hit_info, (const float4*)c->proj0,
                                                     (const float4*)c->proj1, live, c->tiles_x, fcount);
    chunk_count_big_kernel<<<sm_count() * 8, 256, 0, s>>>(big_list, list_counts, c->order, (const uint4*)c->hit_info, (const float4*)c->proj0,
                                                          (const float4*)c->proj1, c->tiles_x, live, fcount, ballots, ballot_cap);
    chunk_sums_kernel<<<emit_blocks, EMIT_THREADS, 0, s>>>(words, lo, hi, fcount, sc.block_sums);
    chunk_emit_kernel<<<emit_blocks, EMIT_THREADS, EMIT_SMEM, s>>>(words, ch, lo, hi, c->order, fcount, sc.block_sums, (const uint4*)c->hit_info,
                                                                   c->tiles_x, (uint32_t)c->isect_cap, big_start, ek, ev, c->num_isect);
    chunk_emit_big_kernel<<<sm_count() * 8, 256, 0, s>>>(big_list, list_counts, c->order, (const uint4*)c->hit_info, fcount, big_start,
                                                         (const float4*)c->proj0, (const float4*)c->proj1, c->tiles_x, live, (uint32_t)c->isect_cap, ek, ev,
                                                         ballots, ballot_cap);
    st = check_launch();
    if (st) return st;
    st = radix_sort(ek, ev, ok, ov, words + CW_COUNT + ch, (uint32_t)c->isect_cap, c->tile_bits, sc, blocks, s, words + CW_BASE + ch);
    if (st) return st;
    tile_ranges_kernel<<<sm_count() * 8, 256, 0, s>>>(c->keys_sorted, words + CW_COUNT + ch, (uint32_t)c->isect_cap, (uint32_t)c->n_tiles,
                                                      (uint2*)c->tile_ranges + (size_t)ch * c->n_tiles, words + CW_BASE + ch);
    st = launch_raster_fwd(c, o, ch, C, alive, s);
    if (st) return st;
  }
  return B2K_OK;
}

extern "C" int b2k_bin_sort_profile(const B2kCtx* c, int32_t n, b2k_stream_t stream, float* ms) {
  B2K_REQUIRE(c && ms);
  Marks& mk = g_marks;
  for (int i = 0; i < 32; i++) B2K_CUDA(cudaEventCreate(&mk.ev[i]));
  mk.n = 0; mk.armed = true;
  const int st = b2k_bin_sort(c, n, stream);
  mk.armed = false;
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  // Marks: [0] start, then per depth pass (after count+rows, after scatter) x 4, [9] after emit, then per tile pass x P, last after ranges.
  const int tile_passes = sort_passes(c->tile_bits), expect = 1 + 8 + 1 + 2 * tile_passes + 1;
  for (int i = 0; i < 10; i++) ms[i] = 0.f;
  if (st == B2K_OK && e == cudaSuccess && mk.n == expect && n > 0) {
    auto dt = [&](int a, int b) { float t = 0.f; cudaEventElapsedTime(&t, mk.ev[a], mk.ev[b]); return t; };
    ms[0] = dt(0, 8); ms[1] = dt(8, 9);
    for (int p = 0; p < tile_passes && p < 3; p++) { ms[2 + 2 * p] = dt(9 + 2 * p, 10 + 2 * p); ms[3 + 2 * p] = dt(10 + 2 * p, 11 + 2 * p); }
    ms[8] = dt(9 + 2 * tile_passes, 10 + 2 * tile_passes); ms[9] = dt(0, mk.n - 1);
  }
  for (int i = 0; i < 32; i++) cudaEventDestroy(mk.ev[i]);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; return B2K_ERR_CUDA; }
  return st;
}

// The radix sort above for callers outside the binning (the refinement pass): stable, ascending, 32-bit keys, four
// passes, so the result returns to the pair it started from.
extern "C" int32_t b2k_sort_passes(int32_t bits) { return bits >= 1 && bits <= 32 ? sort_passes(bits) : 0; }

extern "C" uint64_t b2k_sort_pairs_tmp_bytes(void) { return (uint64_t)sizeof(uint32_t) * ((uint64_t)RADIX_MAX * 1024 + RADIX_MAX + 1024 + 16); }

extern "C" int b2k_sort_pairs_u32(uint32_t* keys, uint32_t* vals, uint32_t* keys_alt, uint32_t* vals_alt, uint32_t n, void* tmp, uint64_t tmp_bytes, b2k_stream_t stream) {
  B2K_REQUIRE(n == 0 || (keys && vals && keys_alt && vals_alt && tmp));
  if (n == 0) return B2K_OK;
  if (tmp_bytes < b2k_sort_pairs_tmp_bytes() || n > 0xFFFFFFF0u) return B2K_ERR_CAPACITY;
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = sort_blocks();
  SortScratch sc;
  sc.hist = (uint32_t*)tmp; sc.totals = sc.hist + (size_t)RADIX_MAX * blocks; sc.block_sums = sc.totals + RADIX_MAX; sc.n_word = sc.block_sums + 1024;
  set_word_kernel<<<1, 1, 0, s>>>(sc.n_word, n);
  return radix_sort(keys, vals, keys_alt, vals_alt, sc.n_word, n, 32, sc, blocks, s);
}

extern "C" int b2k_read_num_isect(const B2kCtx* c, b2k_stream_t stream, uint32_t* total) {
  B2K_REQUIRE(c && c->num_isect && total);
  cudaStream_t s = (cudaStream_t)stream;
  B2K_CUDA(cudaMemcpyAsync(total, c->num_isect, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
  B2K_CUDA(cudaStreamSynchronize(s));
  return *total > c->isect_cap ? B2K_ERR_OVERFLOW : B2K_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Binning without any allocation on the caller's side.
//
// b2k_bin_sort needs a scratch buffer (ctx->sort_tmp) that somebody has to cudaMalloc. Some hosts of this library
// cannot: a plugin loaded into a process whose memory pool is owned and fully reserved by the host application, a
// render thread that must never take the allocator's lock, or a caller inside a region where the CUDA allocator is
// off limits. For them the same scratch lives here, inside the library image, as a fixed device array. It is sized
// for contexts of at most B2K_STATIC_MAX_SPLATS per-splat entries (about 5.2 MB, held by every GPU that loads the
// library, until the process exits).
// ---------------------------------------------------------------------------------------------------------------
namespace b2k {
namespace {
constexpr uint32_t STATIC_MAX_SPLATS = 262144;
constexpr size_t STATIC_WORDS = BIG_HEADER_WORDS + 3 * (size_t)STATIC_MAX_SPLATS + (size_t)RADIX_MAX * 1024 + RADIX_MAX + 1024 + 16;
static __device__ __align__(256) uint32_t g_static_sort_tmp[STATIC_WORDS];
// Device address of the array above, per device. In host code the array's name is only a handle for the runtime,
// never a pointer a kernel may be given; the address has to be asked for, once per device, with that device current.
void* g_static_addr[64] = {nullptr};
}  // namespace
}  // namespace b2k

extern "C" uint32_t b2k_static_max_splats(void) { return b2k::STATIC_MAX_SPLATS; }

extern "C" int b2k_bin_sort_static(const B2kCtx* c, int32_t n, b2k_stream_t stream) {
  B2K_REQUIRE(c && n >= 0);
  if (c->n_cap < 0 || (uint32_t)c->n_cap > STATIC_MAX_SPLATS || (uint32_t)n > STATIC_MAX_SPLATS) return B2K_ERR_CAPACITY;
  int dev = 0;
  B2K_CUDA(cudaGetDevice(&dev));
  B2K_REQUIRE(dev >= 0 && dev < 64);
  if (!g_static_addr[dev]) {   // first call on this device: resolve the array's device address
    void* p = nullptr;
    B2K_CUDA(cudaGetSymbolAddress(&p, g_static_sort_tmp));
    B2K_REQUIRE(p != nullptr);
    g_static_addr[dev] = p;
  }
  B2kCtx local = *c;            // same buffers, scratch redirected to the library's own array
  local.sort_tmp = g_static_addr[dev];
  local.sort_tmp_bytes = sizeof(uint32_t) * STATIC_WORDS;
  return b2k_bin_sort(&local, n, stream);
}
