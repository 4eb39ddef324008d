// Test driver for the C++ host mirror, shaped like the reference's gradient-test Harness (tests/tests.cpp:61-102):
// setup() uploads a scene, loss() = render_forward + photometric_loss + readback, analytic() = loss() + backward +
// optimizer_step with grad_out set. Reads a scene file, writes loss, image and parameter gradients to a result file;
// the Python test compares those with the oracle. An optional third argument renders front to back in that many depth
// chunks.
//
// Scene file (little endian): int32 n, degree, W, H, composite, mask, alpha_lane, has_weights; float32 fx, fy, cx, cy,
// R[9], t[3], bg[3], l1_w, ssim_w, match_alpha_weight, scale; then float32 pos[n*3], log_scale[n*3], quat[n*4],
// opacity[n], floor[n], sh[n*K*3]; uint32 gt[W*H]; uint8 weights[W*H] (when has_weights).
#include "b2c_api.h"
#include <cstdio>
#include <cstdlib>

using namespace b2c;

struct Harness {
  Model model; RenderCtx ctx; DevBuf<uint32_t> gt; DevBuf<uint8_t> wts; ViewGPU view; LossParams lp; RenderParams rp; DevBuf<float> grads;
  void setup(const SplatCloud& cloud, const Camera& cam, int W, int H, const std::vector<uint32_t>& g, const std::vector<uint8_t>& w) {
    model.upload(cloud);
    ctx.setup(W, H, model.cap, 0);
    gt.upload(g);
    view.rgba = gt; view.W = W; view.H = H;
    if (!w.empty()) { wts.upload(w); view.weights = wts; }
    rp.cam = CameraGPU::from(cam, W, H);
    for (int k = 0; k < 3; k++) rp.bg[k] = lp.bg[k];
    rp.sh_degree = cloud.sh_degree; rp.bwd_info = true;
  }
  double loss() {
    render_forward(ctx, model, rp, 0);
    ctx.loss_accum.zero(0, 4);
    photometric_loss(ctx, view, lp, 0);
    return (double)ctx.loss_accum.download(4)[0];
  }
  std::vector<float> analytic() {
    const size_t per = 11 + (size_t)model.K() * 3;
    grads.reserve((size_t)model.n * per); grads.zero();
    loss();
    rasterize_backward(ctx, model, rp, 0);
    OptimParams op; op.cam = rp.cam; op.active_sh_degree = model.degree; op.grad_out = grads.ptr;
    optimizer_step(ctx, model, op, 0);
    return grads.download((size_t)model.n * per);
  }
};

template <typename T> static void rd(FILE* f, T* p, size_t n) { if (n && fread(p, sizeof(T), n, f) != n) { fprintf(stderr, "short read\n"); exit(2); } }

int main(int argc, char** argv) {
  if (argc < 3) { fprintf(stderr, "usage: %s scene.bin result.bin [depth chunks]\n", argv[0]); return 2; }
  try {
    FILE* f = fopen(argv[1], "rb"); if (!f) { perror("scene"); return 2; }
    int32_t hdr[8]; rd(f, hdr, 8);
    const int n = hdr[0], degree = hdr[1], W = hdr[2], H = hdr[3];
    float fl[4 + 9 + 3 + 3 + 4]; rd(f, fl, 23);
    SplatCloud c; c.resize(n, degree); c.floor.assign(n, 0.f);
    rd(f, c.pos.data(), c.pos.size()); rd(f, c.log_scale.data(), c.log_scale.size()); rd(f, c.quat.data(), c.quat.size());
    rd(f, c.opacity.data(), c.opacity.size()); rd(f, c.floor.data(), c.floor.size()); rd(f, c.sh.data(), c.sh.size());
    std::vector<uint32_t> gt((size_t)W * H); rd(f, gt.data(), gt.size());
    std::vector<uint8_t> w; if (hdr[7]) { w.resize((size_t)W * H); rd(f, w.data(), w.size()); }
    fclose(f);
    Camera cam; cam.width = W; cam.height = H; cam.fx = fl[0]; cam.fy = fl[1]; cam.cx = fl[2]; cam.cy = fl[3];
    for (int i = 0; i < 9; i++) cam.R[i] = fl[4 + i];
    for (int i = 0; i < 3; i++) cam.t[i] = fl[13 + i];
    cam.update_pos();
    Harness hs;
    if (argc > 3) hs.ctx.n_chunks = atoi(argv[3]);   // > 1: the front-to-back chunked renderer
    for (int i = 0; i < 3; i++) hs.lp.bg[i] = fl[16 + i];
    hs.lp.l1_w = fl[19]; hs.lp.ssim_w = fl[20]; hs.lp.match_alpha_weight = fl[21]; hs.lp.scale = fl[22];
    hs.lp.composite = hdr[4]; hs.lp.mask = hdr[5]; hs.lp.alpha_lane = hdr[6];
    hs.setup(c, cam, W, H, gt, w);
    const std::vector<float> g = hs.analytic();
    const double loss = hs.loss();
    const std::vector<float4> img = hs.ctx.out_rgba.download((size_t)W * H);
    // An unsupported lane must throw, not silently render without it.
    bool threw = false;
    try { RenderParams bad = hs.rp; bad.mip = true; project_splats(hs.ctx, hs.model, bad, 0); } catch (const std::runtime_error&) { threw = true; }
    FILE* o = fopen(argv[2], "wb"); if (!o) { perror("result"); return 2; }
    const uint32_t isect = hs.ctx.num_isect, flag = threw ? 1u : 0u;
    fwrite(&loss, sizeof loss, 1, o); fwrite(&isect, 4, 1, o); fwrite(&flag, 4, 1, o);
    fwrite(img.data(), sizeof(float4), img.size(), o); fwrite(g.data(), sizeof(float), g.size(), o);
    fclose(o);
    printf("loss %.9f intersections %u\n", loss, isect);
  } catch (const std::exception& e) { fprintf(stderr, "error: %s\n", e.what()); return 1; }
  return 0;
}
