// Tensor-core matrix product (placeholder until it lands: every shape falls through to the f32 kernel).
#include "common.cuh"

gt_status gt_gemm_tc(gt_ctx*, int, int, int, int, int, const float*, const float*, float*, bool* handled) {
  *handled = false;
  return GT_OK;
}
