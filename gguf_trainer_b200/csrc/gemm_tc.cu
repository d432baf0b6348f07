// Tensor-core matrix product for sm_100a: tcgen05.mma (kind::tf32, f32 operands read straight from
// shared memory, f32 accumulators in TMEM), operands staged by TMA into 128B-swizzled tiles, a 5/6-stage
// mbarrier pipeline, persistent CTAs (one per SM) with two TMEM accumulators: one elected thread issues TMA, one
// issues MMA, four warps drain the finished accumulator while the next tile is being accumulated.
// Covers the three layouts of WebGPUBackend.gemm (src/backend/webgpu.ts:1654-1671; srcGemm
// src/backend/wgsl.ts:87-196): NT (forward y = x.W^T), NN (dX += dY.W), TN (dW += dY^T.X), with ragged
// edges handled by TMA zero fill and guarded stores, `accum` by a read-modify-write epilogue, and split-K
// (f32 reductions in L2) when a product has few output tiles and a deep K (the dW product, K = rows).
//
// Every wait on an mbarrier is bounded in wall time; on expiry the CTA records a code in a device flag
// the host checks at the next sync, skips its stores, releases its TMEM and exits.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr int BM = 128;          // UMMA M (cta_group::1): accumulator row i lives in TMEM lane i
constexpr int BK = 32;           // f32 elements per stage along K: 128 bytes = one swizzle row
constexpr int UMMA_K = 8;        // tf32: 32 bytes of K per instruction
constexpr int THREADS = 192;     // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue

template <int BN>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 4;   // 16 KB
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN <= 128 ? 5 : 4;
  static constexpr int EPI_BYTES = 4 * 2 * 4096;   // per epilogue warp: two 32x32 f32 staging tiles for the TMA store
  static constexpr int TOTAL = STAGES * STAGE + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr uint32_t TMEM_COLS = 2 * BN <= 256 ? 256 : 512;   // two accumulators
};

// Persistent: each CTA walks output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (n fastest, then m, then the
// split-K slice), so CTAs running at the same time share their A row-blocks in L2. The accumulator is double-buffered
// in TMEM: while the epilogue warps drain tile i, the MMA warp is already accumulating tile i+1.
// A_K: A is K-major in memory (NT, NN); else MN-major ([K, M], TN). B_K: B is K-major (NT); else [K, N] (NN, TN).
template <bool A_K, bool B_K, int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const __grid_constant__ CUtensorMap mapC, float* __restrict__ C, int M, int N, int K, int accum, int ksplit,
                 int use_tma_store, int batch, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = Smem<BN>;
  constexpr int STAGES = S::STAGES;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi = base + STAGES * S::STAGE;    // staging tiles of the epilogue warps
  const uint32_t bars = epi + S::EPI_BYTES;         // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
  const int per_mat = tiles_n * tiles_m * ksplit;
  const int ntiles = per_mat * batch;            // the matrices of a batch are just more tiles
  const int kblocks = (K + BK - 1) / BK;
  const int per = (kblocks + ksplit - 1) / ksplit;   // K blocks per split-K slice

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; b++) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 128); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  bool dead = false;   // set once a bounded wait has expired: later waits are skipped, control flow stays the same
  auto wait = [&](uint32_t bar, uint32_t parity, int code) {
    if (dead) return;
    if (!mbar_wait(bar, parity)) { dead = true; atomicExch(flag, code); }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer ----
      uint32_t it = 0;
      for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int bi = t / per_mat, tt = t % per_mat;
        const int n0 = (tt % tiles_n) * BN, m0 = ((tt / tiles_n) % tiles_m) * BM, z = tt / (tiles_n * tiles_m);
        const int kb0 = z * per, kb1 = min(kblocks, kb0 + per);
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, 1);
          const uint32_t a_dst = base + s * S::STAGE, b_dst = a_dst + S::A_BYTES;
          const int k0 = kb * BK;
          mbar_expect_tx(full_bar(s), S::STAGE);
          if (A_K) tma_load_3d(a_dst, &mapA, k0, m0, bi, full_bar(s));
          else
            for (int c = 0; c < BM / 32; c++) tma_load_3d(a_dst + c * 4096, &mapA, m0 + 32 * c, k0, bi, full_bar(s));
          if (B_K) tma_load_3d(b_dst, &mapB, k0, n0, bi, full_bar(s));
          else
            for (int c = 0; c < BN / 32; c++) tma_load_3d(b_dst + c * 4096, &mapB, n0 + 32 * c, k0, bi, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      constexpr uint32_t idesc = idesc_tf32(!A_K, !B_K, BM, BN);
      uint32_t it = 0, tl = 0;
      for (int t = blockIdx.x; t < ntiles; t += gridDim.x, tl++) {
        const int z = (t % per_mat) / (tiles_n * tiles_m);
        const int kb0 = z * per, kb1 = min(kblocks, kb0 + per);
        const int b = tl & 1;
        wait(acc_empty(b), ((tl >> 1) & 1) ^ 1, 4);   // the epilogue has drained this accumulator
        tc_fence_after();
        const uint32_t d_tmem = tmem + b * BN;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          wait(full_bar(s), (it / STAGES) & 1, 2);
          tc_fence_after();
          const uint32_t a_src = base + s * S::STAGE, b_src = a_src + S::A_BYTES;
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; j++) {
            const uint64_t ad = A_K ? desc_kmajor(a_src + j * 32) : desc_mnmajor(a_src + j * 1024);
            const uint64_t bd = B_K ? desc_kmajor(b_src + j * 32) : desc_mnmajor(b_src + j * 1024);
            umma_tf32(d_tmem, ad, bd, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
        }
        umma_commit(acc_full(b));      // accumulator complete
      }
    }
  } else {
    // ---- epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32) ----
    const int q = warp & 3;
    const bool vec = (N & 3) == 0;
    uint32_t tl = 0, nst = 0;   // nst: TMA stores issued by this warp
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, tl++) {
      const int bi = t / per_mat, tt = t % per_mat;
      const int n0 = (tt % tiles_n) * BN, m0 = ((tt / tiles_n) % tiles_m) * BM, z = tt / (tiles_n * tiles_m);
      const int b = tl & 1;
      const bool have = z * per < kblocks;     // an empty split-K slice issues no MMA and contributes nothing
      const int row = m0 + q * 32 + lane;
      if (have) wait(acc_full(b), (tl >> 1) & 1, 3);
      dead = __any_sync(0xffffffffu, dead);
      tc_fence_after();
      if (have) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;   // uniform across the warp
          float v[32];
          tmem_ld32(tmem + b * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] *= TRUNC_COMP;
          if (use_tma_store) {
            // Stage the warp's 32x32 block in shared memory (128-byte rows, 16-byte chunks XOR (row mod 8), the layout
            // the store's tensor map expects) and let TMA write it: whole 128-byte rows, clipped at M and N, as a
            // plain store or, when accumulating or combining split-K slices, as an f32 reduce-add performed in L2.
            const uint32_t tile = epi + (uint32_t)(q * 2 + (nst & 1)) * 4096u;
            if (nst >= 2) tma_wait_read<1>();        // the tile written two blocks ago has been read out
            __syncwarp();
            uint8_t* tp = smem_raw + (tile - smem_u32(smem_raw)) + lane * 128;
#pragma unroll
            for (int c4 = 0; c4 < 8; c4++)
              *reinterpret_cast<float4*>(tp + ((c4 ^ (lane & 7)) * 16)) = make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && !dead && m0 + q * 32 < M) {
              if (ksplit > 1 || accum) tma_reduce_add_3d(&mapC, tile, col0, m0 + q * 32, bi);
              else tma_store_3d(&mapC, tile, col0, m0 + q * 32, bi);
            }
            if (lane == 0) tma_commit_group();
            nst++;
          } else if (row < M && !dead) {
            float* dst = C + (size_t)bi * M * N + (size_t)row * N + col0;
            if (vec && col0 + 32 <= N) {
              if (ksplit > 1) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) atomicAdd(reinterpret_cast<float4*>(dst + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
              } else if (accum) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  float4 o = *reinterpret_cast<float4*>(dst + j);
                  o.x += v[j]; o.y += v[j + 1]; o.z += v[j + 2]; o.w += v[j + 3];
                  *reinterpret_cast<float4*>(dst + j) = o;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j++) {
                if (col0 + j < N) {
                  if (ksplit > 1) atomicAdd(dst + j, v[j]);
                  else dst[j] = accum ? dst[j] + v[j] : v[j];
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty(b));
    }
    if (lane == 0) tma_wait_all<0>();   // every store of this warp has landed before the CTA's shared memory goes away
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
int* g_flag[64] = {};

template <bool A_K, bool B_K, int BN>
gt_status launch(gt_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int tma_store, float* c, int M, int N,
                 int K, int accum, int ksplit, int batch) {
  auto kern = gemm_tf32_kernel<A_K, B_K, BN>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device]) {
    GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BN>::TOTAL));
    attr_set[ctx->device] = true;
  }
  const long ntiles = (long)gt_cdiv(N, BN) * gt_cdiv(M, BM) * ksplit * batch;
  dim3 grid((unsigned)min((long)ctx->sm_count, ntiles), 1, 1);
  kern<<<grid, THREADS, Smem<BN>::TOTAL, ctx->stream>>>(ma, mb, mc, c, M, N, K, accum, ksplit, tma_store, batch, g_flag[ctx->device]);
  GT_LAUNCHED(ctx, "gemm_tf32_kernel");
  return GT_OK;
}

}  // namespace

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      g_encode = (EncodeTiledFn)fn;
  });
  return g_encode;
}

// 2-D f32 tensor [outer, inner] with `inner` contiguous; box [box_outer, 32]; out-of-range reads give 0.
// kmajor: the tile's rows are K runs (128-byte swizzle); else its rows are MN runs (128-byte swizzle, 32-byte atoms).
}  // namespace

bool tc::make_map_3d(CUtensorMap* map, const float* ptr, uint64_t inner, uint64_t outer, uint64_t batch, uint64_t row_pitch_elems,
                     uint64_t batch_stride_elems, uint32_t box_outer, bool kmajor) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {row_pitch_elems * sizeof(float), batch_stride_elems * sizeof(float)};
  cuuint32_t box[3] = {32, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             kmajor ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tc::make_map_atoms(CUtensorMap* map, const float* ptr, uint64_t inner, uint64_t outer, uint64_t row_pitch_elems,
                        uint32_t box_outer, uint32_t atoms, bool kmajor) {
  EncodeTiledFn enc = encode_fn();
  if (!enc || inner % 32 != 0) return false;
  cuuint64_t dims[3] = {32, outer, inner / 32};
  cuuint64_t strides[2] = {row_pitch_elems * sizeof(float), 32 * sizeof(float)};
  cuuint32_t box[3] = {32, box_outer, atoms};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             kmajor ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tc::make_map_2d(CUtensorMap* map, const float* ptr, uint64_t inner, uint64_t outer, uint64_t row_pitch_elems,
                     uint32_t box_outer, bool kmajor) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_pitch_elems * sizeof(float)};
  cuuint32_t box[2] = {32, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             kmajor ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* tc::device_flag(gt_ctx* ctx) {
  if (ctx->device < 0 || ctx->device >= 64) return nullptr;
  if (!g_flag[ctx->device]) {
    if (ctx->capturing) return nullptr;
    if (cudaMalloc(&g_flag[ctx->device], 65536) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    cudaMemsetAsync(g_flag[ctx->device], 0, 65536, ctx->stream);
  }
  return g_flag[ctx->device];
}

// Reads and clears the device flag the kernels raise when a bounded wait expires.
gt_status gt_gemm_tc_check(gt_ctx* ctx) {
  int* f = g_flag[ctx->device];
  if (!f) return GT_OK;
  int h = 0;
  GT_CUDA(ctx, cudaMemcpyAsync(&h, f, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (h != 0) {
    cudaMemsetAsync(f, 0, sizeof(int), ctx->stream);
    return gt_fail(ctx, GT_ERR_CUDA, "tensor-core kernel: a pipeline wait expired (code %d); results of that launch are invalid", h);
  }
  return GT_OK;
}

// `batch` independent products of the same shape, matrix i of each operand `M*K`, `N*K`, `M*N` elements after matrix i-1.
gt_status gt_gemm_tc_batched(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, int batch,
                             bool* handled) {
  *handled = false;
  if (batch < 1) return GT_OK;
  // Small or oddly aligned products stay on the f32 kernel: TMA needs 16-byte row pitches and bases.
  const bool a_k = kind != GT_GEMM_TN, b_k = kind == GT_GEMM_NT;
  const int a_inner = a_k ? K : M, b_inner = b_k ? K : N;
  if (M < 64 || N < 16 || K < 16) return GT_OK;
  if ((a_inner & 3) || (b_inner & 3)) return GT_OK;
  if ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c)) & 15) return GT_OK;
  if (ctx->device < 0 || ctx->device >= 64) return GT_OK;
  if (!device_flag(ctx)) return GT_OK;
  // tile width: 192 divides the model widths this path is built for (576, 192, 1536, 49152); otherwise 128
  const int bn = (N % 192 == 0 || (N > 128 && (gt_cdiv(N, 192) * 192 - N) < (gt_cdiv(N, 128) * 128 - N))) ? 192 : 128;
  CUtensorMap ma, mb;
  const uint64_t sa = (uint64_t)M * K, sb = (uint64_t)N * K, sc = (uint64_t)M * N;
  const bool oka = a_k ? make_map_3d(&ma, a, K, M, batch, K, sa, BM, true) : make_map_3d(&ma, a, M, K, batch, M, sa, BK, false);
  const bool okb = b_k ? make_map_3d(&mb, b, K, N, batch, K, sb, bn, true) : make_map_3d(&mb, b, N, K, batch, N, sb, BK, false);
  if (!oka || !okb) return GT_OK;
  // the output goes through TMA (32x32 blocks of whole 128-byte rows) whenever its row pitch allows a tensor map
  CUtensorMap mc = ma;
  const int tma_store = ((N & 3) == 0 && make_map_3d(&mc, c, N, M, batch, N, sc, 32, true)) ? 1 : 0;
  // split K when the output has few tiles and K is deep (dW: K = rows); partial sums meet in L2 with f32 adds
  int ksplit = 1;
  const long tiles = (long)gt_cdiv(N, bn) * gt_cdiv(M, BM) * batch;
  const int kblocks = gt_cdiv(K, BK);
  if (tiles < ctx->sm_count && kblocks >= 16) {
    ksplit = (int)min((long)(ctx->sm_count / tiles), (long)(kblocks / 8));
    if (ksplit < 1) ksplit = 1;
  }
  if (ksplit > 1 && !accum) GT_CUDA(ctx, cudaMemsetAsync(c, 0, sizeof(float) * (size_t)M * N * batch, ctx->stream));
  gt_status s;
  if (bn == 192) {
    if (kind == GT_GEMM_NT) s = launch<true, true, 192>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch);
    else if (kind == GT_GEMM_NN) s = launch<true, false, 192>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch);
    else s = launch<false, false, 192>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch);
  } else {
    if (kind == GT_GEMM_NT) s = launch<true, true, 128>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch);
    else if (kind == GT_GEMM_NN) s = launch<true, false, 128>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch);
    else s = launch<false, false, 128>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch);
  }
  if (s) return s;
  *handled = true;
  return GT_OK;
}

gt_status gt_gemm_tc(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, bool* handled) {
  return gt_gemm_tc_batched(ctx, kind, accum, M, N, K, a, b, c, 1, handled);
}

#ifdef GT_ATTN_TRACE
// Development aid (compiled out by default): copies the trace words a traced kernel left behind the device flag.
extern "C" int gtx_debug_trace(gt_ctx* ctx, int* out, int n) {
  int* f = g_flag[ctx->device];
  if (!f) return -1;
  cudaStreamSynchronize(ctx->stream);
  return (int)cudaMemcpy(out, f + 64, sizeof(int) * n, cudaMemcpyDeviceToHost);
}
#endif
