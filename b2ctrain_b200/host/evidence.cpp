// Host side of the evidence pass: the per-view loop of compute_evidence (src/train/evidence.cu:200-241) and the two
// downloads (evidence.cu:245-275), over b2k_evidence_view / b2k_evidence_fold / b2k_label_vote.
#include "evidence.h"

namespace b2c {
using namespace abi;

namespace {
constexpr int EV_ACC = 8;   // the exported seven + the sum of w_in^2 from which the effective view count is derived
DevBuf<float> g_evidence, g_view_acc, g_votes;
bool g_votes_valid = false;
}  // namespace

void compute_evidence(RenderCtx& ctx, const Model& m, const std::vector<ViewGPU>& views, const std::vector<Camera>& cams, const EvidenceOptions& cfg, cudaStream_t stream) {
  const int bins = b2k_label_bins();
  g_evidence.reserve((size_t)m.n * EV_ACC); g_evidence.zero(stream, (size_t)m.n * EV_ACC);
  g_view_acc.reserve((size_t)m.n * 3);
  g_votes_valid = cfg.export_labels;
  if (g_votes_valid) { g_votes.reserve((size_t)m.n * bins); g_votes.zero(stream, (size_t)m.n * bins); }
  const B2kModel mv = view_of(m);
  for (size_t v = 0; v < views.size(); v++) {
    const ViewGPU& view = views[v];
    if (view.W != ctx.W || view.H != ctx.H) ctx.setup(view.W, view.H, m.cap, stream);
    RenderParams rp; rp.cam = CameraGPU::from(cams[v], view.W, view.H);
    rp.sh_degree = m.degree; rp.bwd_info = true;
    const bool normals = cfg.evidence_normal_weight > 0.f && view.normals;
    rp.feat = normals ? FeatureMode::Normals : FeatureMode::None;
    render_forward(ctx, m, rp, stream);
    g_view_acc.zero(stream, (size_t)m.n * 3);
    const B2kCtx cv = view_of(ctx);
    const int masked_alpha = view.masked && view.has_alpha ? 1 : 0;
    check(b2k_evidence_view(&cv, view.rgba, normals ? view.normals : nullptr, view.weights, masked_alpha, cfg.evidence_normal_weight, g_view_acc.ptr, stream), "compute_evidence");
    if (g_votes_valid && view.labels) check(b2k_label_vote(&cv, view.rgba, view.labels, view.weights, masked_alpha, g_votes.ptr, stream), "compute_evidence (labels)");
    check(b2k_evidence_fold(&mv, g_view_acc.ptr, cams[v].pos, g_evidence.ptr, stream), "compute_evidence (fold)");
  }
  B2C_CUDA_CHECK(cudaStreamSynchronize(stream));
}

void reduce_evidence(B2kDp* dp, const Model& m, cudaStream_t stream) {
  if (!dp) return;
  check(b2k_dp_allreduce_stat(dp, g_evidence.ptr, (uint64_t)m.n * EV_ACC, 0, stream), "reduce_evidence");
  if (g_votes_valid) check(b2k_dp_allreduce_stat(dp, g_votes.ptr, (uint64_t)m.n * (uint64_t)b2k_label_bins(), 0, stream), "reduce_evidence (labels)");
}

const float* evidence_device(int* stride) { *stride = EV_ACC; return g_evidence.ptr; }

std::vector<float> download_evidence(const Model& m, cudaStream_t stream) {
  std::vector<float> out((size_t)m.n * 7, 0.f);
  if (g_evidence.count < (size_t)m.n * EV_ACC) return out;
  const std::vector<float> acc = g_evidence.download((size_t)m.n * EV_ACC, stream);
  for (size_t i = 0; i < (size_t)m.n; i++) {
    const float* a = &acc[i * EV_ACC];
    float* e = &out[i * 7];
    e[0] = a[0]; e[1] = a[1]; e[2] = a[2];
    e[3] = a[7] > 0.f ? a[0] * a[0] / a[7] : 0.f;   // participation ratio: the number of views the in-mask mass is spread over
    e[4] = a[4]; e[5] = a[5]; e[6] = a[6];
  }
  return out;
}

std::vector<float> download_labels(const Model& m, cudaStream_t stream) {
  std::vector<float> out((size_t)m.n * 2, 0.f);
  const size_t bins = (size_t)b2k_label_bins();
  if (!g_votes_valid || g_votes.count < (size_t)m.n * bins) return out;
  const std::vector<float> acc = g_votes.download((size_t)m.n * bins, stream);
  for (size_t i = 0; i < (size_t)m.n; i++) {
    const float* a = &acc[i * bins];
    float total = 0.f, best = 0.f; int win = 0;
    for (size_t k = 0; k < bins; k++) { total += a[k]; if (a[k] > best) { best = a[k]; win = (int)k; } }
    if (total > 0.f) { out[i * 2] = (float)win; out[i * 2 + 1] = best / total; }
  }
  return out;
}

}  // namespace b2c
