// Tensor-core attention kernels (placeholder until they land: every shape falls through to the f32 kernels).
#include "common.cuh"

gt_status gt_attention_fwd_tc(gt_ctx*, int, int, int, int, int, int, const float*, const float*, const float*, float*, float*,
                              bool* handled) {
  *handled = false;
  return GT_OK;
}
gt_status gt_attention_bwd_tc(gt_ctx*, int, int, int, int, int, int, const float*, const float*, const float*, const float*,
                              const float*, const float*, float*, int, float*, int, float*, int, bool* handled) {
  *handled = false;
  return GT_OK;
}
