// Flash-style causal attention on the 5th-generation tensor cores (tcgen05, kind::tf32, f32 accumulators in
// TMEM), for head dimensions 32, 64 and 128: grouped-query heads, optional sliding window, sequences batched
// as [nseq*T] rows. Same formulation as the reference's flash kernels (srcAttnFwd/BwdDq/BwdDkv,
// src/backend/wgsl.ts:657-918): exp2-domain scores, running max with a -3e38 sentinel, LSE[h,row] = m + log2(l)
// as the only forward side buffer, backward recomputing p = exp2(s*SCALE2 - LSE) and using D = sum_d dO*O.
// Q, K, V, dO are read as f32 by TMA into swizzled tiles and fed to the tensor cores directly (tf32 drops the
// low mantissa bits; the mean truncation bias is compensated, see tc_common.cuh); softmax, masks and all
// accumulation are f32.
//
// Forward: one CTA owns 128 query rows of one head. Per 64-key block: S = Q.K^T into TMEM (M=128, N=64);
// four warps read it one row per thread (no shuffles), apply mask and online softmax, and write P as the
// A operand of the second product; O_blk = P.V into TMEM; the same threads fold it into their register
// accumulator with the rescale factor. One more warp issues TMA and MMA. K and V of the next block are
// fetched while the current block's softmax runs.
#include "common.cuh"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr float NEG = -3.0e38f;
constexpr int BQ = 128, BKV = 64;

template <int HD>
struct FwdSmem {
  static constexpr int Q_BYTES = BQ * HD * 4;
  static constexpr int K_BYTES = BKV * HD * 4;
  static constexpr int V_BYTES = BKV * HD * 4;
  static constexpr int P_BYTES = BQ * BKV * 4;
  static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + K_BYTES, P_OFF = V_OFF + V_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int TOTAL = BAR_OFF + 128 + 1024;
  static constexpr uint32_t TMEM_COLS = (64 + HD) <= 128 ? 128 : 256;
};

// Q: [rows, Hq*HD]; K, V: [rows, Hkv*HD]. Tensor maps: mapQ box [128 rows, 32], mapK box [64 rows, 32] (both 16-byte-atom
// swizzle), mapV box [64 rows, 32] with the 32-byte-atom swizzle (V is the [keys, hd] operand with hd contiguous).
template <int HD>
__global__ void __launch_bounds__(160, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, float* __restrict__ out, float* __restrict__ lse, int rows, int T,
                   int Hq, int Hkv, int window, float scale2, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = FwdSmem<HD>;
  constexpr int ATOMS = HD / 32;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base + S::Q_OFF, k_s = base + S::K_OFF, v_s = base + S::V_OFF, p_s = base + S::P_OFF;
  const uint32_t bars = base + S::BAR_OFF;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 16, s_full = bars + 24, p_full = bars + 32, o_full = bars + 40;
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + S::BAR_OFF + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ;            // first query position of this tile inside its sequence
  const int h = blockIdx.y, seq = blockIdx.z;
  const int kvh = h / (Hq / Hkv);
  const int row0 = seq * T;                  // first global row of the sequence
  const int q_last = min(q0 + BQ - 1, T - 1);
  const int kb_lo = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / BKV : 0;
  const int kb_hi = q_last / BKV;
  const int nkb = kb_hi - kb_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(v_full, 1); mbar_init(s_full, 1); mbar_init(p_full, 128); mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t tm_s = tmem, tm_o = tmem + 64;

  if (warp == 4) {
    if (lane == 0) {
      // ---- TMA + MMA issue ----
      constexpr uint32_t idesc_s = idesc_tf32(false, false, BQ, BKV);   // S = Q.K^T, both K-major
      constexpr uint32_t idesc_o = idesc_tf32(false, true, BQ, HD);     // O = P.V, V is [keys, hd]
      bool ok = true;
      mbar_expect_tx(q_full, S::Q_BYTES);
      for (int a = 0; a < ATOMS; a++) tma_load_2d(q_s + a * (BQ * 128), &mapQ, h * HD + 32 * a, row0 + q0, q_full);
      auto load_k = [&](int kb) {
        mbar_expect_tx(k_full, S::K_BYTES);
        for (int a = 0; a < ATOMS; a++) tma_load_2d(k_s + a * (BKV * 128), &mapK, kvh * HD + 32 * a, row0 + kb * BKV, k_full);
      };
      auto load_v = [&](int kb) {
        mbar_expect_tx(v_full, S::V_BYTES);
        for (int a = 0; a < ATOMS; a++) tma_load_2d(v_s + a * (BKV * 128), &mapV, kvh * HD + 32 * a, row0 + kb * BKV, v_full);
      };
      load_k(kb_lo);
      load_v(kb_lo);
      ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(flag, 11);
      for (int i = 0; i < nkb && ok; i++) {
        const uint32_t par = i & 1;
        ok = mbar_wait(k_full, par);
        if (!ok) { atomicExch(flag, 12); break; }
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            umma_tf32(tm_s, desc_kmajor(q_s + a * (BQ * 128) + j * 32), desc_kmajor(k_s + a * (BKV * 128) + j * 32), idesc_s,
                      (a > 0 || j > 0) ? 1u : 0u);
        umma_commit(s_full);
        ok = mbar_wait(s_full, par);         // K tile has been read: fetch the next one under the softmax
        if (!ok) { atomicExch(flag, 13); break; }
        if (i + 1 < nkb) load_k(kb_lo + i + 1);
        ok = mbar_wait(v_full, par) && mbar_wait(p_full, par);
        if (!ok) { atomicExch(flag, 14); break; }
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < BKV / 8; j++)
          umma_tf32(tm_o, desc_kmajor(p_s + (j / 4) * (BQ * 128) + (j % 4) * 32), smem_desc(v_s + j * 1024, BKV * 128, 512, 1),
                    idesc_o, j > 0 ? 1u : 0u);
        umma_commit(o_full);
        ok = mbar_wait(o_full, par);         // V and P tiles have been read
        if (!ok) { atomicExch(flag, 15); break; }
        if (i + 1 < nkb) load_v(kb_lo + i + 1);
      }
    }
  } else {
    // ---- softmax + output: thread = one query row; warp w owns TMEM lanes [32w, 32w+32) ----
    const int r = warp * 32 + lane;
    const int tq = q0 + r;
    const bool valid = tq < T;
    float m = NEG, l = 0.f;
    float o[HD];
#pragma unroll
    for (int d = 0; d < HD; d++) o[d] = 0.f;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int i = 0; i < nkb; i++) {
      const uint32_t par = i & 1;
      const int k0 = (kb_lo + i) * BKV;
      if (ok) ok = mbar_wait(s_full, par);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) atomicExch(flag, 16); break; }
      tc_fence_after();
      float s[BKV];
      tmem_ld32(tm_s + lane_base, s);
      tmem_ld32(tm_s + lane_base + 32, s + 32);
      const int lo = (window > 0) ? tq - window + 1 : 0;
      float mx = NEG;
#pragma unroll
      for (int c = 0; c < BKV; c++) {
        const int kg = k0 + c;
        const bool keep = valid && kg <= tq && kg >= lo;
        s[c] = keep ? s[c] * scale2 : NEG;
        mx = fmaxf(mx, s[c]);
      }
      const float mn = fmaxf(m, mx);
      const float alpha = exp2f(m - mn);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < BKV; c++) {
        const float p = (s[c] > -1.0e38f) ? exp2f(s[c] - mn) : 0.f;
        s[c] = p;
        sum += p;
      }
      l = l * alpha + sum;
      m = mn;
      // P as the K-major A operand: atom = 32 keys, row pitch 128 B, 16-byte chunks XOR (row mod 8)
      {
        uint8_t* prow = base_ptr + S::P_OFF + r * 128;
#pragma unroll
        for (int c4 = 0; c4 < BKV / 4; c4++) {
          const int atom = c4 / 8, chunk = (c4 % 8) ^ (r & 7);
          *reinterpret_cast<float4*>(prow + atom * (BQ * 128) + chunk * 16) = make_float4(s[4 * c4], s[4 * c4 + 1], s[4 * c4 + 2], s[4 * c4 + 3]);
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
      if (ok) ok = mbar_wait(o_full, par);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) atomicExch(flag, 17); break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD / 32; c++) {
        float t[32];
        tmem_ld32(tm_o + lane_base + c * 32, t);
#pragma unroll
        for (int d = 0; d < 32; d++) o[c * 32 + d] = o[c * 32 + d] * alpha + t[d];
      }
      tc_fence_before();
    }
    if (ok && valid) {
      const float inv = TRUNC_COMP / l;   // the P.V product carries the truncation bias of both operands
      float* dst = out + (size_t)(row0 + tq) * Hq * HD + (size_t)h * HD;
#pragma unroll
      for (int d = 0; d < HD; d += 4) *reinterpret_cast<float4*>(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
      lse[(size_t)h * rows + row0 + tq] = m + log2f(l);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

template <int HD>
gt_status launch_fwd(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int window, const float* q, const float* k, const float* v,
                     float* out, float* lse, int* flag) {
  CUtensorMap mq, mk, mv;
  if (!make_map_2d(&mq, q, (uint64_t)Hq * HD, rows, (uint64_t)Hq * HD, BQ, true) ||
      !make_map_2d(&mk, k, (uint64_t)Hkv * HD, rows, (uint64_t)Hkv * HD, BKV, true) ||
      !make_map_2d(&mv, v, (uint64_t)Hkv * HD, rows, (uint64_t)Hkv * HD, BKV, false))
    return gt_fail(ctx, GT_ERR_CUDA, "attention: tensor map encoding failed");
  auto kern = attn_fwd_tc_kernel<HD>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device]) {
    GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<HD>::TOTAL));
    attr_set[ctx->device] = true;
  }
  // the S product's truncation bias is folded into the score scale
  const float scale2 = 1.4426950408889634f / sqrtf((float)HD) * TRUNC_COMP;
  dim3 grid(gt_cdiv(T, BQ), Hq, rows / T);
  kern<<<grid, 160, FwdSmem<HD>::TOTAL, ctx->stream>>>(mq, mk, mv, out, lse, rows, T, Hq, Hkv, window, scale2, flag);
  GT_LAUNCHED(ctx, "attn_fwd_tc_kernel");
  return GT_OK;
}

}  // namespace

gt_status gt_attention_fwd_tc(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q, const float* k,
                              const float* v, float* out, float* lse, bool* handled) {
  *handled = false;
  if (hd != 32 && hd != 64 && hd != 128) return GT_OK;
  if (T < 64) return GT_OK;   // tiny sequences stay on the f32 kernels
  if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)out)) & 15) return GT_OK;
  int* flag = device_flag(ctx);
  if (!flag) return GT_OK;
  gt_status s;
  if (hd == 32) s = launch_fwd<32>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);
  else if (hd == 64) s = launch_fwd<64>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);
  else s = launch_fwd<128>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);
  if (s) return s;
  *handled = true;
  return GT_OK;
}

gt_status gt_attention_bwd_tc(gt_ctx*, int, int, int, int, int, int, const float*, const float*, const float*, const float*,
                              const float*, const float*, float*, int, float*, int, float*, int, bool* handled) {
  *handled = false;
  return GT_OK;
}
