// Token and mask ingest on the device: the corpus stays resident in HBM in its on-disk form, bare little-endian
// u16 or u32 tokens with no header (src/data/tokens.ts:12-14, 158-185; the supervision mask is read with the same
// width, src/commands/pretrain.ts:416), and a step's input is B window starts instead of B*T ids and B*T targets.
// One integer kernel forms both arrays: ids[b*T + t] = tokens[start_b + t], targets[b*T + t] = tokens[start_b + 1 + t],
// or the ignore marker 0xffffffff where the mask is 0 (maskWindow, src/train/trainer.ts:45-49, applied at start + 1 as
// in src/backend/train-gpu.ts:206-208). Bit-exact by construction: no arithmetic touches a token value.
#include "common.cuh"

namespace {

template <typename TOK>
__global__ void gather_windows_kernel(const TOK* __restrict__ tokens, const TOK* __restrict__ mask, unsigned long long count,
                                      const unsigned long long* __restrict__ starts, int B, int T, uint32_t* __restrict__ ids,
                                      uint32_t* __restrict__ targets, int* __restrict__ bad) {
  const long n = (long)B * T;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const int b = (int)(i / T), t = (int)(i % T);
    const unsigned long long p = starts[b] + (unsigned long long)t;
    if (p + 1 >= count) {          // a window that leaves the corpus: nothing is read there, the row is ignored, the host is told
      ids[i] = 0u;
      targets[i] = 0xffffffffu;
      atomicExch(bad, 1);
      continue;
    }
    ids[i] = (uint32_t)tokens[p];
    const uint32_t tg = (uint32_t)tokens[p + 1];
    targets[i] = (mask != nullptr && mask[p + 1] == (TOK)0) ? 0xffffffffu : tg;
  }
}

// largest token value of the corpus (integer max: exact and order-independent), checked once against the vocabulary
template <typename TOK>
__global__ void token_max_kernel(const TOK* __restrict__ tokens, unsigned long long count, unsigned int* __restrict__ out) {
  unsigned int m = 0;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
       i += (unsigned long long)gridDim.x * blockDim.x)
    m = max(m, (unsigned int)tokens[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}

}  // namespace

extern "C" {

gt_status gt_tokens_max(gt_ctx* ctx, gt_buf tokens, int32_t bytes_per_token, uint64_t count, uint32_t* out_max) {
  GT_REQUIRE(ctx, tokens && out_max && count > 0 && (bytes_per_token == 2 || bytes_per_token == 4),
             "gt_tokens_max: tokens %p count %llu bytes_per_token %d (2 or 4)", gt_ptr<void>(tokens), (unsigned long long)count, bytes_per_token);
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_tokens_max inside a graph capture");
  int* flags = gt_flags(ctx);
  if (!flags) return gt_fail(ctx, GT_ERR_CUDA, "gt_tokens_max: cannot allocate the flag block");
  unsigned int* d = reinterpret_cast<unsigned int*>(flags + GT_FLAG_TOKEN_MAX);
  GT_CUDA(ctx, cudaMemsetAsync(d, 0, sizeof(unsigned int), ctx->stream));
  const int grid = (int)min((unsigned long long)ctx->sm_count * 8, (unsigned long long)((count + 255) / 256));
  if (bytes_per_token == 2) token_max_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(gt_ptr<const uint16_t>(tokens), count, d);
  else token_max_kernel<uint32_t><<<grid, 256, 0, ctx->stream>>>(gt_ptr<const uint32_t>(tokens), count, d);
  GT_LAUNCHED(ctx, "token_max_kernel");
  GT_CUDA(ctx, cudaMemcpyAsync(out_max, d, sizeof(unsigned int), cudaMemcpyDeviceToHost, ctx->stream));
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return GT_OK;
}

gt_status gt_gather_windows(gt_ctx* ctx, gt_buf tokens, gt_buf mask, int32_t bytes_per_token, uint64_t count, gt_buf starts,
                            int32_t B, int32_t T, gt_buf ids, gt_buf targets) {
  GT_REQUIRE(ctx, tokens && starts && ids && targets, "gt_gather_windows: null operand");
  GT_REQUIRE(ctx, B > 0 && T > 0 && (bytes_per_token == 2 || bytes_per_token == 4) && count >= (uint64_t)T + 1,
             "gt_gather_windows: B %d T %d bytes_per_token %d corpus %llu tokens (a window needs T+1)", B, T, bytes_per_token,
             (unsigned long long)count);
  int* flags = gt_flags(ctx);
  int* bad = flags ? flags + GT_FLAG_WINDOW : nullptr;
  if (!bad) return gt_fail(ctx, GT_ERR_STATE, "gt_gather_windows: first use inside a graph capture; call it once eagerly first");
  const long n = (long)B * T;
  const int grid = (int)min((long)ctx->sm_count * 4, (n + 255) / 256);
  const unsigned long long* st = gt_ptr<const unsigned long long>(starts);
  if (bytes_per_token == 2)
    gather_windows_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(gt_ptr<const uint16_t>(tokens), gt_ptr<const uint16_t>(mask), count, st, B, T,
                                                                   gt_ptr<uint32_t>(ids), gt_ptr<uint32_t>(targets), bad);
  else
    gather_windows_kernel<uint32_t><<<grid, 256, 0, ctx->stream>>>(gt_ptr<const uint32_t>(tokens), gt_ptr<const uint32_t>(mask), count, st, B, T,
                                                                   gt_ptr<uint32_t>(ids), gt_ptr<uint32_t>(targets), bad);
  GT_LAUNCHED(ctx, "gather_windows_kernel");
  return GT_OK;
}

}  // extern "C"
