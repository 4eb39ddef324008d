// compute_evidence / download_evidence / download_labels / evidence_device with the reference's names
// (src/train/evidence.h:13-24) over the replay kernels of libb2k. The accumulators live in a module-level state, as
// in the reference (evidence.cu:24-25,39); `EvidenceOptions` stands for the two Config fields the pass reads.
// Under data parallelism each rank passes its share of the views and calls reduce_evidence() before the downloads.
#pragma once
#include "b2c_api.h"

namespace b2c {

struct EvidenceOptions {
  float evidence_normal_weight = 0.f;   // Config::evidence_normal_weight (cli.h:52)
  bool export_labels = false;           // Config::export_labels (cli.h:50)
};
void compute_evidence(RenderCtx& ctx, const Model& m, const std::vector<ViewGPU>& views, const std::vector<Camera>& cams, const EvidenceOptions& cfg, cudaStream_t stream);
// Sums the accumulators over the ranks of `dp` (nullptr or one rank: nothing to do).
void reduce_evidence(B2kDp* dp, const Model& m, cudaStream_t stream);
std::vector<float> download_evidence(const Model& m, cudaStream_t stream);   // [n][7] w_in, w_all, err, views, dir xyz
std::vector<float> download_labels(const Model& m, cudaStream_t stream);     // [n][2] winning class, its share
const float* evidence_device(int* stride);                                   // [n][*stride], w_all at offset 1

}  // namespace b2c
