// Tensor-core matrix product for sm_100a: tcgen05.mma (kind::tf32, f32 operands read straight from
// shared memory, f32 accumulators in TMEM), operands staged by TMA into 128B-swizzled tiles, a 4-stage
// mbarrier pipeline, one elected thread issuing TMA, one issuing MMA, four warps draining TMEM.
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

namespace {

constexpr int BM = 128;          // UMMA M (cta_group::1): accumulator row i lives in TMEM lane i
constexpr int BK = 32;           // f32 elements per stage along K: 128 bytes = one swizzle row
constexpr int UMMA_K = 8;        // tf32: 32 bytes of K per instruction
constexpr int STAGES = 4;
constexpr int THREADS = 192;     // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue
constexpr uint64_t WAIT_NS = 2000000000ull;  // 2 s per wait
// kind::tf32 drops the low 13 mantissa bits of each f32 operand (truncation, not rounding), so every product is
// biased low. For operands whose mantissas are log-uniform (generic data) the mean relative truncation error is
// 2^-11 * E[1/m] = 2^-11 / (2 ln 2) = 3.52e-4 per operand: measured -7.05e-4 on the product of two. The
// epilogue multiplies the accumulator by 1 + 2 * 3.52e-4, which removes the systematic part and leaves the
// zero-mean part (relative L2 7.7e-4 -> 3.1e-4 measured). For operands that happen to be exact in tf32 the factor
// itself is the error, the same size as the bias it removes elsewhere and inside the mode's 2e-3 bound.
constexpr float TRUNC_COMP = 1.000704f;

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t gtimer() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// false on timeout
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = gtimer();
  while (!mbar_try(bar, parity)) {
    if (gtimer() - t0 > WAIT_NS) return false;
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the barrier receives one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor. Bits: [0,14) start>>4, [16,30) leading byte offset>>4, [32,46) stride byte
// offset>>4, [46,48) version 1, [61,64) swizzle layout.
// K-major tile (layout 2, 128-byte swizzle in 16-byte units): rows of 128 B (32 f32 of K), 8-row groups 1024 B
//   apart (stride offset); the leading offset is not used for swizzled K-major tiles.
// MN-major tile of 32-bit elements (layout 1, the 128-byte swizzle in 32-byte units, the only one tcgen05 accepts
//   for MN-major tf32; TMA writes it with SWIZZLE_128B_ATOM_32B): chunks of 32 MN-elements x 32 K-rows (4096 B, one
//   TMA box); a K row is 128 B, the swizzle pattern repeats every 4 K rows = 512 B (stride offset), chunks are
//   4096 B apart (leading offset). One MMA (K = 8) reads two such 4-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout << 61;
  return d;
}
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) { return smem_desc(addr, 16, 1024, 2); }
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) { return smem_desc(addr, 4096, 512, 1); }

// Instruction descriptor (kind::tf32, f32 accumulate): [4,6) D format 1 = f32, [7,10) A format 2 = tf32,
// [10,13) B format 2, bit 15 A is MN-major, bit 16 B is MN-major, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn, bool b_mn, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

template <int BN>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 4;   // 16 KB
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int TOTAL = STAGES * STAGE + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// A_K: A is K-major in memory (NT, NN); else MN-major ([K, M], TN). B_K: B is K-major (NT); else [K, N] (NN, TN).
template <bool A_K, bool B_K, int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, float* __restrict__ C,
                 int M, int N, int K, int accum, int ksplit, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = Smem<BN>;
  constexpr uint32_t TMEM_COLS = BN <= 128 ? 128 : 256;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES * S::STAGE;          // full[STAGES], empty[STAGES], done, tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t done_bar = bars + 8u * (2 * STAGES);
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 1);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // split-K: slice z owns K blocks [kb0, kb1)
  const int kblocks = (K + BK - 1) / BK;
  const int per = (kblocks + ksplit - 1) / ksplit;
  const int kb0 = blockIdx.z * per;
  const int kb1 = min(kblocks, kb0 + per);
  const int nk = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(done_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  bool ok = true;

  if (nk > 0) {
    if (warp == 0 && lane == 0) {
      // ---- TMA producer ----
      for (int i = 0; i < nk && ok; i++) {
        const int s = i % STAGES;
        ok = mbar_wait(empty_bar(s), ((i / STAGES) & 1) ^ 1);
        if (!ok) { atomicExch(flag, 1); break; }
        const uint32_t a_dst = base + s * S::STAGE, b_dst = a_dst + S::A_BYTES;
        const int k0 = (kb0 + i) * BK;
        mbar_expect_tx(full_bar(s), S::STAGE);
        if (A_K) tma_load_2d(a_dst, &mapA, k0, m0, full_bar(s));
        else
          for (int c = 0; c < BM / 32; c++) tma_load_2d(a_dst + c * 4096, &mapA, m0 + 32 * c, k0, full_bar(s));
        if (B_K) tma_load_2d(b_dst, &mapB, k0, n0, full_bar(s));
        else
          for (int c = 0; c < BN / 32; c++) tma_load_2d(b_dst + c * 4096, &mapB, n0 + 32 * c, k0, full_bar(s));
      }
    } else if (warp == 1 && lane == 0) {
      // ---- MMA issuer ----
      constexpr uint32_t idesc = make_idesc(!A_K, !B_K, BN);
      for (int i = 0; i < nk && ok; i++) {
        const int s = i % STAGES;
        ok = mbar_wait(full_bar(s), (i / STAGES) & 1);
        if (!ok) { atomicExch(flag, 2); break; }
        tc_fence_after();
        const uint32_t a_src = base + s * S::STAGE, b_src = a_src + S::A_BYTES;
#pragma unroll
        for (int j = 0; j < BK / UMMA_K; j++) {
          const uint64_t ad = A_K ? desc_kmajor(a_src + j * 32) : desc_mnmajor(a_src + j * 1024);
          const uint64_t bd = B_K ? desc_kmajor(b_src + j * 32) : desc_mnmajor(b_src + j * 1024);
          umma_tf32(tmem, ad, bd, idesc, (i > 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
      }
      umma_commit(done_bar);         // accumulator complete
    }
  }

  if (warp >= 2) {
    // ---- epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32) ----
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    bool have = nk > 0;
    if (have) {
      have = mbar_wait(done_bar, 0);
      if (!have && lane == 0) atomicExch(flag, 3);
      have = __all_sync(0xffffffffu, have);
    }
    tc_fence_after();
    if (have) {
      const bool vec = (N & 3) == 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) break;   // uniform across the warp
        float v[32];
        tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
#pragma unroll
        for (int j = 0; j < 32; j++) v[j] *= TRUNC_COMP;
        if (row < M) {
          float* dst = C + (size_t)row * N + col0;
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
            for (int j = 0; j < 32; j++) {
              if (col0 + j >= N) break;
              if (ksplit > 1) atomicAdd(dst + j, v[j]);
              else dst[j] = accum ? dst[j] + v[j] : v[j];
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
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
bool make_map(CUtensorMap* map, const float* ptr, uint64_t inner, uint64_t outer, uint32_t box_outer, bool kmajor) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * sizeof(float)};
  cuuint32_t box[2] = {32, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             kmajor ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int* g_flag[64] = {};

template <bool A_K, bool B_K, int BN>
gt_status launch(gt_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, float* c, int M, int N, int K, int accum, int ksplit) {
  auto kern = gemm_tf32_kernel<A_K, B_K, BN>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device]) {
    GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BN>::TOTAL));
    attr_set[ctx->device] = true;
  }
  dim3 grid(gt_cdiv(N, BN), gt_cdiv(M, BM), ksplit);
  kern<<<grid, THREADS, Smem<BN>::TOTAL, ctx->stream>>>(ma, mb, c, M, N, K, accum, ksplit, g_flag[ctx->device]);
  GT_LAUNCHED(ctx, "gemm_tf32_kernel");
  return GT_OK;
}

}  // namespace

// Reads and clears the device flag the kernels raise when a bounded wait expires.
gt_status gt_gemm_tc_check(gt_ctx* ctx) {
  int* f = g_flag[ctx->device];
  if (!f) return GT_OK;
  int h = 0;
  GT_CUDA(ctx, cudaMemcpyAsync(&h, f, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  GT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (h != 0) {
    cudaMemsetAsync(f, 0, sizeof(int), ctx->stream);
    return gt_fail(ctx, GT_ERR_CUDA, "tensor-core matrix product: a pipeline wait expired (code %d: 1 producer, 2 MMA, 3 epilogue); results of that launch are invalid", h);
  }
  return GT_OK;
}

gt_status gt_gemm_tc(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, bool* handled) {
  *handled = false;
  // Small or oddly aligned products stay on the f32 kernel: TMA needs 16-byte row pitches and bases.
  const bool a_k = kind != GT_GEMM_TN, b_k = kind == GT_GEMM_NT;
  const int a_inner = a_k ? K : M, b_inner = b_k ? K : N;
  if (M < 64 || N < 16 || K < 16) return GT_OK;
  if ((a_inner & 3) || (b_inner & 3)) return GT_OK;
  if ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c)) & 15) return GT_OK;
  if (!encode_fn()) return GT_OK;
  if (ctx->device < 0 || ctx->device >= 64) return GT_OK;
  if (!g_flag[ctx->device]) {
    if (ctx->capturing) return GT_OK;
    GT_CUDA(ctx, cudaMalloc(&g_flag[ctx->device], 256));
    GT_CUDA(ctx, cudaMemsetAsync(g_flag[ctx->device], 0, 256, ctx->stream));
  }
  // tile width: 192 divides the model widths this path is built for (576, 192, 1536, 49152); otherwise 128
  const int bn = (N % 192 == 0 || (N > 128 && (gt_cdiv(N, 192) * 192 - N) < (gt_cdiv(N, 128) * 128 - N))) ? 192 : 128;
  CUtensorMap ma, mb;
  const bool oka = a_k ? make_map(&ma, a, K, M, BM, true) : make_map(&ma, a, M, K, BK, false);
  const bool okb = b_k ? make_map(&mb, b, K, N, bn, true) : make_map(&mb, b, N, K, BK, false);
  if (!oka || !okb) return GT_OK;
  // split K when the output has few tiles and K is deep (dW: K = rows); partial sums meet in L2 with f32 adds
  int ksplit = 1;
  const long tiles = (long)gt_cdiv(N, bn) * gt_cdiv(M, BM);
  const int kblocks = gt_cdiv(K, BK);
  if (tiles < ctx->sm_count && kblocks >= 16) {
    ksplit = (int)min((long)(ctx->sm_count / tiles), (long)(kblocks / 8));
    if (ksplit < 1) ksplit = 1;
  }
  if (ksplit > 1 && !accum) GT_CUDA(ctx, cudaMemsetAsync(c, 0, sizeof(float) * (size_t)M * N, ctx->stream));
  gt_status s;
  if (bn == 192) {
    if (kind == GT_GEMM_NT) s = launch<true, true, 192>(ctx, ma, mb, c, M, N, K, accum, ksplit);
    else if (kind == GT_GEMM_NN) s = launch<true, false, 192>(ctx, ma, mb, c, M, N, K, accum, ksplit);
    else s = launch<false, false, 192>(ctx, ma, mb, c, M, N, K, accum, ksplit);
  } else {
    if (kind == GT_GEMM_NT) s = launch<true, true, 128>(ctx, ma, mb, c, M, N, K, accum, ksplit);
    else if (kind == GT_GEMM_NN) s = launch<true, false, 128>(ctx, ma, mb, c, M, N, K, accum, ksplit);
    else s = launch<false, false, 128>(ctx, ma, mb, c, M, N, K, accum, ksplit);
  }
  if (s) return s;
  *handled = true;
  return GT_OK;
}
