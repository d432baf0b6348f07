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
  // Causal work grows with the query position: the heaviest tiles are launched first, and all (head, sequence)
  // pairs of one tile index are adjacent, so the tail of the grid is made of the lightest tiles.
  const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * BQ;   // first query position of this tile inside its sequence
  const int h = blockIdx.x % Hq, seq = blockIdx.x / Hq;
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
  dim3 grid(Hq * (rows / T), gt_cdiv(T, BQ), 1);
  kern<<<grid, 160, FwdSmem<HD>::TOTAL, ctx->stream>>>(mq, mk, mv, out, lse, rows, T, Hq, Hkv, window, scale2, flag);
  GT_LAUNCHED(ctx, "attn_fwd_tc_kernel");
  return GT_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward. D[h,row] = sum_d dO*O first (one warp per (row, head)), then two kernels, as in the reference
// (srcAttnBwdDq, srcAttnBwdDkv): each recomputes S and dP on the tensor cores, forms p and dS in registers
// and feeds them back as the A operand of the gradient products, whose accumulators stay in TMEM for the
// whole loop. Nothing is reduced with atomics: one CTA owns its 128 query rows (dQ) or its 128 key rows
// (dK, dV, summing its GQA group inside the loop), so results are deterministic.
// ---------------------------------------------------------------------------------------------
__global__ void attn_bwd_d_tc_kernel(int rows, int Hq, int hd, const float* __restrict__ go, const float* __restrict__ o,
                                     float* __restrict__ D) {
  const int lane = threadIdx.x & 31;
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (w >= (long)rows * Hq) return;
  const int h = (int)(w % Hq);
  const long row = w / Hq;
  const size_t b = (size_t)row * Hq * hd + (size_t)h * hd;
  float acc = 0.f;
  for (int d = lane; d < hd; d += 32) acc = fmaf(go[b + d], o[b + d], acc);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) D[(size_t)h * rows + row] = acc;
}

// write NC f32 values as row r of a K-major operand tile (atoms of 32 columns, 128 rows each, 128-byte swizzle)
template <int NC>
__device__ __forceinline__ void store_row_kmajor(uint8_t* tile, int r, const float* v) {
#pragma unroll
  for (int c4 = 0; c4 < NC / 4; c4++) {
    const int atom = c4 / 8, chunk = (c4 % 8) ^ (r & 7);
    *reinterpret_cast<float4*>(tile + atom * (128 * 128) + r * 128 + chunk * 16) = make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
  }
}

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, float* v) {
#pragma unroll
  for (int c = 0; c < N / 32; c++) tmem_ld32(taddr + c * 32, v + c * 32);
}

// ---- dK, dV: CTA = 128 keys of one kv head; loop over the group's query heads and over blocks of NQ queries ----
template <int HD, int NQ>
struct DkvSmem {
  static constexpr int KV_BYTES = 128 * HD * 4;          // K, V tiles (K-major A operands)
  static constexpr int QT_BYTES = NQ * HD * 4;           // one copy of a Q or dO tile
  static constexpr int PT_BYTES = 128 * NQ * 4;          // P^T, dS^T (K-major A operands, K = queries)
  static constexpr int K_OFF = 0, V_OFF = KV_BYTES, QK_OFF = 2 * KV_BYTES, DOK_OFF = QK_OFF + QT_BYTES,
                       QM_OFF = DOK_OFF + QT_BYTES, DOM_OFF = QM_OFF + QT_BYTES, P_OFF = DOM_OFF + QT_BYTES,
                       DS_OFF = P_OFF + PT_BYTES, BAR_OFF = DS_OFF + PT_BYTES;
  static constexpr int TOTAL = BAR_OFF + 128 + 1024;
  static constexpr int COLS = 2 * NQ + 2 * HD;
  static constexpr uint32_t TMEM_COLS = COLS <= 128 ? 128 : (COLS <= 256 ? 256 : 512);
};

template <int HD, int NQ>
__global__ void __launch_bounds__(160, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                       const __grid_constant__ CUtensorMap mapQk, const __grid_constant__ CUtensorMap mapQm,
                       const __grid_constant__ CUtensorMap mapGk, const __grid_constant__ CUtensorMap mapGm,
                       const float* __restrict__ lse, const float* __restrict__ Dv, float* gk, int accum_k, float* gv, int accum_v,
                       int rows, int T, int Hq, int Hkv, int window, float scale2, float scale, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = DkvSmem<HD, NQ>;
  constexpr int ATOMS = HD / 32;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t k_s = base + S::K_OFF, v_s = base + S::V_OFF, qk_s = base + S::QK_OFF, gk_s = base + S::DOK_OFF,
                 qm_s = base + S::QM_OFF, gm_s = base + S::DOM_OFF, p_s = base + S::P_OFF, ds_s = base + S::DS_OFF;
  const uint32_t bars = base + S::BAR_OFF;
  const uint32_t kv_full = bars, qk_full = bars + 8, qm_full = bars + 16, s_full = bars + 24, p_full = bars + 32, acc_done = bars + 40;
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + S::BAR_OFF + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.y * 128;            // early keys are read by the most queries: heaviest first
  const int kvh = blockIdx.x % Hkv, seq = blockIdx.x / Hkv;
  const int group = Hq / Hkv;
  const int row0 = seq * T;
  const int k_last = min(k0 + 127, T - 1);
  const int q_max = (window > 0) ? min(T - 1, k_last + window - 1) : T - 1;
  const int qb_lo = k0 / NQ, qb_hi = q_max / NQ;
  const int nqb = qb_hi - qb_lo + 1;
  const int iters = nqb * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qk_full, 1); mbar_init(qm_full, 1); mbar_init(s_full, 1); mbar_init(p_full, 128); mbar_init(acc_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t tm_s = tmem, tm_dp = tmem + NQ, tm_dv = tmem + 2 * NQ, tm_dk = tmem + 2 * NQ + HD;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_tf32(false, false, 128, NQ);   // S^T = K.Q^T and dP^T = V.dO^T
      constexpr uint32_t idesc_g = idesc_tf32(false, true, 128, HD);    // dV += P^T.dO, dK += dS^T.Q
      bool ok = true;
      mbar_expect_tx(kv_full, 2 * S::KV_BYTES);
      for (int a = 0; a < ATOMS; a++) {
        tma_load_2d(k_s + a * (128 * 128), &mapK, kvh * HD + 32 * a, row0 + k0, kv_full);
        tma_load_2d(v_s + a * (128 * 128), &mapV, kvh * HD + 32 * a, row0 + k0, kv_full);
      }
      auto load_k = [&](int it) {   // K-major copies of Q and dO for iteration it
        const int h = kvh * group + it / nqb, qr = row0 + (qb_lo + it % nqb) * NQ;
        mbar_expect_tx(qk_full, 2 * S::QT_BYTES);
        for (int a = 0; a < ATOMS; a++) {
          tma_load_2d(qk_s + a * (NQ * 128), &mapQk, h * HD + 32 * a, qr, qk_full);
          tma_load_2d(gk_s + a * (NQ * 128), &mapGk, h * HD + 32 * a, qr, qk_full);
        }
      };
      auto load_m = [&](int it) {   // [queries, hd] copies (hd contiguous) for the gradient products
        const int h = kvh * group + it / nqb, qr = row0 + (qb_lo + it % nqb) * NQ;
        mbar_expect_tx(qm_full, 2 * S::QT_BYTES);
        for (int a = 0; a < ATOMS; a++) {
          tma_load_2d(qm_s + a * (NQ * 128), &mapQm, h * HD + 32 * a, qr, qm_full);
          tma_load_2d(gm_s + a * (NQ * 128), &mapGm, h * HD + 32 * a, qr, qm_full);
        }
      };
      load_k(0);
      load_m(0);
      ok = mbar_wait(kv_full, 0);
      if (!ok) atomicExch(flag, 21);
      for (int i = 0; i < iters && ok; i++) {
        const uint32_t par = i & 1;
        ok = mbar_wait(qk_full, par);
        if (!ok) { atomicExch(flag, 22); break; }
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t acc = (a > 0 || j > 0) ? 1u : 0u;
            umma_tf32(tm_s, desc_kmajor(k_s + a * (128 * 128) + j * 32), desc_kmajor(qk_s + a * (NQ * 128) + j * 32), idesc_s, acc);
            umma_tf32(tm_dp, desc_kmajor(v_s + a * (128 * 128) + j * 32), desc_kmajor(gk_s + a * (NQ * 128) + j * 32), idesc_s, acc);
          }
        umma_commit(s_full);
        ok = mbar_wait(s_full, par);
        if (!ok) { atomicExch(flag, 23); break; }
        if (i + 1 < iters) load_k(i + 1);
        ok = mbar_wait(qm_full, par) && mbar_wait(p_full, par);
        if (!ok) { atomicExch(flag, 24); break; }
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < NQ / 8; j++) {
          const uint32_t acc = (i > 0 || j > 0) ? 1u : 0u;
          const uint32_t aoff = (j / 4) * (128 * 128) + (j % 4) * 32;
          umma_tf32(tm_dv, desc_kmajor(p_s + aoff), smem_desc(gm_s + j * 1024, NQ * 128, 512, 1), idesc_g, acc);
          umma_tf32(tm_dk, desc_kmajor(ds_s + aoff), smem_desc(qm_s + j * 1024, NQ * 128, 512, 1), idesc_g, acc);
        }
        umma_commit(acc_done);
        ok = mbar_wait(acc_done, par);
        if (!ok) { atomicExch(flag, 25); break; }
        if (i + 1 < iters) load_m(i + 1);
      }
    }
  } else {
    const int r = warp * 32 + lane;          // key row inside the tile
    const int kg = k0 + r;                   // key position in the sequence
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int i = 0; i < iters; i++) {
      const uint32_t par = i & 1;
      const int h = kvh * group + i / nqb;
      const int qpos0 = (qb_lo + i % nqb) * NQ;
      if (ok) ok = mbar_wait(s_full, par);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) atomicExch(flag, 26); break; }
      tc_fence_after();
      float s[NQ], dp[NQ];
      tmem_ld_cols<NQ>(tm_s + lane_base, s);
      tmem_ld_cols<NQ>(tm_dp + lane_base, dp);
      const float* lrow = lse + (size_t)h * rows + row0 + qpos0;
      const float* drow = Dv + (size_t)h * rows + row0 + qpos0;
#pragma unroll
      for (int c = 0; c < NQ; c++) {
        const int tq = qpos0 + c;
        const bool keep = tq < T && kg <= tq && (window == 0 || kg >= tq - window + 1);   // kg <= tq < T
        float p = 0.f, d = 0.f;
        if (keep) {
          p = exp2f(s[c] * scale2 - __ldg(lrow + c));
          d = p * (dp[c] * TRUNC_COMP - __ldg(drow + c)) * scale;
        }
        s[c] = p;
        dp[c] = d;
      }
      if (i > 0) {                            // the previous iteration's gradient products still read P^T / dS^T
        if (ok) ok = mbar_wait(acc_done, (i - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { if (lane == 0) atomicExch(flag, 27); break; }
      }
      store_row_kmajor<NQ>(base_ptr + S::P_OFF, r, s);
      store_row_kmajor<NQ>(base_ptr + S::DS_OFF, r, dp);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok && iters > 0) {
      ok = mbar_wait(acc_done, (iters - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) atomicExch(flag, 28);
    }
    tc_fence_after();
    if (ok) {   // warp-uniform: the TMEM loads are warp-wide instructions, only the stores are per-row
      const bool st = kg < T;
      const size_t off = (size_t)(row0 + (st ? kg : 0)) * Hkv * HD + (size_t)kvh * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; c++) {
        float t[32];
        if (gv) {
          tmem_ld32(tm_dv + lane_base + c * 32, t);
          float* dst = gv + off + c * 32;
#pragma unroll
          for (int d = 0; d < 32 && st; d += 4) {
            float4 o = accum_v ? *reinterpret_cast<float4*>(dst + d) : make_float4(0, 0, 0, 0);
            o.x += t[d] * TRUNC_COMP; o.y += t[d + 1] * TRUNC_COMP; o.z += t[d + 2] * TRUNC_COMP; o.w += t[d + 3] * TRUNC_COMP;
            *reinterpret_cast<float4*>(dst + d) = o;
          }
        }
        if (gk) {
          tmem_ld32(tm_dk + lane_base + c * 32, t);
          float* dst = gk + off + c * 32;
#pragma unroll
          for (int d = 0; d < 32 && st; d += 4) {
            float4 o = accum_k ? *reinterpret_cast<float4*>(dst + d) : make_float4(0, 0, 0, 0);
            o.x += t[d] * TRUNC_COMP; o.y += t[d + 1] * TRUNC_COMP; o.z += t[d + 2] * TRUNC_COMP; o.w += t[d + 3] * TRUNC_COMP;
            *reinterpret_cast<float4*>(dst + d) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

// ---- dQ: CTA = 128 queries of one head; loop over blocks of NK keys ----
template <int HD, int NK>
struct DqSmem {
  static constexpr int Q_BYTES = 128 * HD * 4;           // Q, dO tiles (K-major A operands)
  static constexpr int KT_BYTES = NK * HD * 4;           // one copy of a K or V tile
  static constexpr int DS_BYTES = 128 * NK * 4;
  static constexpr int Q_OFF = 0, DO_OFF = Q_BYTES, KK_OFF = 2 * Q_BYTES, VK_OFF = KK_OFF + KT_BYTES, KM_OFF = VK_OFF + KT_BYTES,
                       DS_OFF = KM_OFF + KT_BYTES, BAR_OFF = DS_OFF + DS_BYTES;
  static constexpr int TOTAL = BAR_OFF + 128 + 1024;
  static constexpr int COLS = 2 * NK + HD;
  static constexpr uint32_t TMEM_COLS = COLS <= 128 ? 128 : (COLS <= 256 ? 256 : 512);
};

template <int HD, int NK>
__global__ void __launch_bounds__(160, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapG,
                      const __grid_constant__ CUtensorMap mapKk, const __grid_constant__ CUtensorMap mapVk,
                      const __grid_constant__ CUtensorMap mapKm, const float* __restrict__ lse, const float* __restrict__ Dv,
                      float* gq, int accum_q, int rows, int T, int Hq, int Hkv, int window, float scale2, float scale,
                      int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = DqSmem<HD, NK>;
  constexpr int ATOMS = HD / 32;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base + S::Q_OFF, g_s = base + S::DO_OFF, kk_s = base + S::KK_OFF, vk_s = base + S::VK_OFF,
                 km_s = base + S::KM_OFF, ds_s = base + S::DS_OFF;
  const uint32_t bars = base + S::BAR_OFF;
  const uint32_t q_full = bars, kk_full = bars + 8, km_full = bars + 16, s_full = bars + 24, p_full = bars + 32, acc_done = bars + 40;
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + S::BAR_OFF + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * 128;   // late queries read the most keys: heaviest first
  const int h = blockIdx.x % Hq, seq = blockIdx.x / Hq;
  const int kvh = h / (Hq / Hkv);
  const int row0 = seq * T;
  const int q_last = min(q0 + 127, T - 1);
  const int kb_lo = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / NK : 0;
  const int kb_hi = q_last / NK;
  const int iters = kb_hi - kb_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(kk_full, 1); mbar_init(km_full, 1); mbar_init(s_full, 1); mbar_init(p_full, 128); mbar_init(acc_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t tm_s = tmem, tm_dp = tmem + NK, tm_dq = tmem + 2 * NK;

  if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_tf32(false, false, 128, NK);   // S = Q.K^T, dP = dO.V^T
      constexpr uint32_t idesc_g = idesc_tf32(false, true, 128, HD);    // dQ += dS.K
      bool ok = true;
      mbar_expect_tx(q_full, 2 * S::Q_BYTES);
      for (int a = 0; a < ATOMS; a++) {
        tma_load_2d(q_s + a * (128 * 128), &mapQ, h * HD + 32 * a, row0 + q0, q_full);
        tma_load_2d(g_s + a * (128 * 128), &mapG, h * HD + 32 * a, row0 + q0, q_full);
      }
      auto load_k = [&](int it) {
        const int kr = row0 + (kb_lo + it) * NK;
        mbar_expect_tx(kk_full, 2 * S::KT_BYTES);
        for (int a = 0; a < ATOMS; a++) {
          tma_load_2d(kk_s + a * (NK * 128), &mapKk, kvh * HD + 32 * a, kr, kk_full);
          tma_load_2d(vk_s + a * (NK * 128), &mapVk, kvh * HD + 32 * a, kr, kk_full);
        }
      };
      auto load_m = [&](int it) {
        const int kr = row0 + (kb_lo + it) * NK;
        mbar_expect_tx(km_full, S::KT_BYTES);
        for (int a = 0; a < ATOMS; a++) tma_load_2d(km_s + a * (NK * 128), &mapKm, kvh * HD + 32 * a, kr, km_full);
      };
      load_k(0);
      load_m(0);
      ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(flag, 31);
      for (int i = 0; i < iters && ok; i++) {
        const uint32_t par = i & 1;
        ok = mbar_wait(kk_full, par);
        if (!ok) { atomicExch(flag, 32); break; }
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t acc = (a > 0 || j > 0) ? 1u : 0u;
            umma_tf32(tm_s, desc_kmajor(q_s + a * (128 * 128) + j * 32), desc_kmajor(kk_s + a * (NK * 128) + j * 32), idesc_s, acc);
            umma_tf32(tm_dp, desc_kmajor(g_s + a * (128 * 128) + j * 32), desc_kmajor(vk_s + a * (NK * 128) + j * 32), idesc_s, acc);
          }
        umma_commit(s_full);
        ok = mbar_wait(s_full, par);
        if (!ok) { atomicExch(flag, 33); break; }
        if (i + 1 < iters) load_k(i + 1);
        ok = mbar_wait(km_full, par) && mbar_wait(p_full, par);
        if (!ok) { atomicExch(flag, 34); break; }
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < NK / 8; j++)
          umma_tf32(tm_dq, desc_kmajor(ds_s + (j / 4) * (128 * 128) + (j % 4) * 32), smem_desc(km_s + j * 1024, NK * 128, 512, 1), idesc_g,
                    (i > 0 || j > 0) ? 1u : 0u);
        umma_commit(acc_done);
        ok = mbar_wait(acc_done, par);
        if (!ok) { atomicExch(flag, 35); break; }
        if (i + 1 < iters) load_m(i + 1);
      }
    }
  } else {
    const int r = warp * 32 + lane;
    const int tq = q0 + r;
    const bool valid = tq < T;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float L = valid ? lse[(size_t)h * rows + row0 + tq] : 0.f;
    const float Dr = valid ? Dv[(size_t)h * rows + row0 + tq] : 0.f;
    const int lo = (window > 0) ? tq - window + 1 : 0;
    bool ok = true;
    for (int i = 0; i < iters; i++) {
      const uint32_t par = i & 1;
      const int kpos0 = (kb_lo + i) * NK;
      if (ok) ok = mbar_wait(s_full, par);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) atomicExch(flag, 36); break; }
      tc_fence_after();
      float s[NK], dp[NK];
      tmem_ld_cols<NK>(tm_s + lane_base, s);
      tmem_ld_cols<NK>(tm_dp + lane_base, dp);
#pragma unroll
      for (int c = 0; c < NK; c++) {
        const int kg = kpos0 + c;
        const bool keep = valid && kg <= tq && kg >= lo;
        float d = 0.f;
        if (keep) {
          const float p = exp2f(s[c] * scale2 - L);
          d = p * (dp[c] * TRUNC_COMP - Dr) * scale;
        }
        s[c] = d;
      }
      if (i > 0) {
        if (ok) ok = mbar_wait(acc_done, (i - 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { if (lane == 0) atomicExch(flag, 37); break; }
      }
      store_row_kmajor<NK>(base_ptr + S::DS_OFF, r, s);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok && iters > 0) {
      ok = mbar_wait(acc_done, (iters - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) atomicExch(flag, 38);
    }
    tc_fence_after();
    if (ok) {   // warp-uniform: the TMEM loads are warp-wide instructions, only the stores are per-row
      float* dst0 = gq + (size_t)(row0 + (valid ? tq : 0)) * Hq * HD + (size_t)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; c++) {
        float t[32];
        tmem_ld32(tm_dq + lane_base + c * 32, t);
        float* dst = dst0 + c * 32;
#pragma unroll
        for (int d = 0; d < 32 && valid; d += 4) {
          float4 o = accum_q ? *reinterpret_cast<float4*>(dst + d) : make_float4(0, 0, 0, 0);
          o.x += t[d] * TRUNC_COMP; o.y += t[d + 1] * TRUNC_COMP; o.z += t[d + 2] * TRUNC_COMP; o.w += t[d + 3] * TRUNC_COMP;
          *reinterpret_cast<float4*>(dst + d) = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

template <int HD, int NQ, int NK>
gt_status launch_bwd(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int window, const float* q, const float* k, const float* v,
                     const float* out, const float* lse, const float* go, float* gq, int accum_q, float* gk, int accum_k, float* gv,
                     int accum_v, int* flag) {
  float* D = nullptr;
  gt_status st = gt_scratch(ctx, sizeof(float) * (size_t)rows * Hq, &D);
  if (st) return st;
  attn_bwd_d_tc_kernel<<<gt_cdiv((long)rows * Hq * 32, 256), 256, 0, ctx->stream>>>(rows, Hq, HD, go, out, D);
  GT_LAUNCHED(ctx, "attn_bwd_d_tc_kernel");
  const float scale = 1.f / sqrtf((float)HD);
  const float scale2 = 1.4426950408889634f * scale * TRUNC_COMP;
  const uint64_t qw = (uint64_t)Hq * HD, kw = (uint64_t)Hkv * HD;
  const int nseq = rows / T;
  if (gk || gv) {
    CUtensorMap mK, mV, mQk, mQm, mGk, mGm;
    if (!make_map_2d(&mK, k, kw, rows, kw, 128, true) || !make_map_2d(&mV, v, kw, rows, kw, 128, true) ||
        !make_map_2d(&mQk, q, qw, rows, qw, NQ, true) || !make_map_2d(&mQm, q, qw, rows, qw, NQ, false) ||
        !make_map_2d(&mGk, go, qw, rows, qw, NQ, true) || !make_map_2d(&mGm, go, qw, rows, qw, NQ, false))
      return gt_fail(ctx, GT_ERR_CUDA, "attention backward: tensor map encoding failed");
    auto kern = attn_bwd_dkv_tc_kernel<HD, NQ>;
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device]) {
      GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<HD, NQ>::TOTAL));
      attr_set[ctx->device] = true;
    }
    dim3 grid(Hkv * nseq, gt_cdiv(T, 128), 1);
    kern<<<grid, 160, DkvSmem<HD, NQ>::TOTAL, ctx->stream>>>(mK, mV, mQk, mQm, mGk, mGm, lse, D, gk, accum_k, gv, accum_v, rows, T, Hq, Hkv,
                                                            window, scale2, scale, flag);
    GT_LAUNCHED(ctx, "attn_bwd_dkv_tc_kernel");
  }
  if (gq) {
    CUtensorMap mQ, mG, mKk, mVk, mKm;
    if (!make_map_2d(&mQ, q, qw, rows, qw, 128, true) || !make_map_2d(&mG, go, qw, rows, qw, 128, true) ||
        !make_map_2d(&mKk, k, kw, rows, kw, NK, true) || !make_map_2d(&mVk, v, kw, rows, kw, NK, true) ||
        !make_map_2d(&mKm, k, kw, rows, kw, NK, false))
      return gt_fail(ctx, GT_ERR_CUDA, "attention backward: tensor map encoding failed");
    auto kern = attn_bwd_dq_tc_kernel<HD, NK>;
    static bool attr_set[64] = {};
    if (!attr_set[ctx->device]) {
      GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<HD, NK>::TOTAL));
      attr_set[ctx->device] = true;
    }
    dim3 grid(Hq * nseq, gt_cdiv(T, 128), 1);
    kern<<<grid, 160, DqSmem<HD, NK>::TOTAL, ctx->stream>>>(mQ, mG, mKk, mVk, mKm, lse, D, gq, accum_q, rows, T, Hq, Hkv, window, scale2,
                                                           scale, flag);
    GT_LAUNCHED(ctx, "attn_bwd_dq_tc_kernel");
  }
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

gt_status gt_attention_bwd_tc(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q, const float* k,
                              const float* v, const float* out, const float* lse, const float* go, float* gq, int accum_q, float* gk,
                              int accum_k, float* gv, int accum_v, bool* handled) {
  *handled = false;
  if (hd != 32 && hd != 64 && hd != 128) return GT_OK;
  if (T < 64) return GT_OK;
  if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)go) | ((uintptr_t)gq) | ((uintptr_t)gk) | ((uintptr_t)gv)) & 15) return GT_OK;
  int* flag = device_flag(ctx);
  if (!flag) return GT_OK;
  gt_status s;
  if (hd == 32) s = launch_bwd<32, 64, 64>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, flag);
  else if (hd == 64) s = launch_bwd<64, 64, 64>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, flag);
  else s = launch_bwd<128, 32, 32>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, flag);
  if (s) return s;
  *handled = true;
  return GT_OK;
}
