// Flash-style causal attention on the 5th-generation tensor cores (tcgen05, kind::tf32, f32 accumulators in
// TMEM), for head dimensions 32, 64, 128 and (as pairs of CTAs, see PairSum) 256: grouped-query heads, optional sliding window, sequences batched
// as [nseq*T] rows. Same formulation as the reference's flash kernels (srcAttnFwd/BwdDq/BwdDkv,
// src/backend/wgsl.ts:657-918): exp2-domain scores, running max with a -3e38 sentinel, LSE[h,row] = m + log2(l)
// as the only forward side buffer, backward recomputing p = exp2(s*SCALE2 - LSE) and using D = sum_d dO*O.
// Q, K, V, dO are read as f32 by TMA into swizzled tiles and fed to the tensor cores directly (tf32 drops the
// low mantissa bits; the mean truncation bias is compensated, see tc_common.cuh); softmax, masks and all
// accumulation are f32.
//
// All three kernels share one shape. A CTA owns 128 rows of the output (queries for forward and dQ, keys for
// dK/dV) and walks the other axis in blocks. In the backward kernels one thread issues the TMA copies and one
// thread of another warp the MMAs, each waiting only on what its own instructions need (with a single issuing
// thread the waits and issue latencies of the two roles added up to more than the tensor time of a block);
// descriptors are formed by one add per operand. Eight warps do the element math, two per TMEM lane quadrant, each
// taking half of a block's columns, one output row per thread (no shuffles). In forward P goes to the second
// product through a shared-memory tile; in backward P^T / dS^T are written back over S^T / dP^T in tensor memory
// and read from there as the A operand of the gradient products. The
// score products of block i+1 are issued before the element math of block i is waited for (their TMEM
// accumulators are double-buffered), so the tensor pipe and the CUDA cores overlap; operand tiles of the next
// block are fetched as soon as the products that read the current ones have completed.
// Waits on mbarriers are bounded in wall time: on expiry a thread raises the device flag and from then on skips
// every wait, so all threads still run the same control flow to the end and release TMEM.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"

using namespace tc;

namespace {

constexpr float NEG = -3.0e38f;
constexpr int ROWS = 128;          // output rows per CTA = TMEM lanes
constexpr int MATH_WARPS = 8;
constexpr int MMA_WARP = MATH_WARPS, TMA_WARP = MATH_WARPS + 1;   // one thread of each issues the products / the copies
constexpr int THREADS = (MATH_WARPS + 2) * 32;
// The forward kernel runs two CTAs per SM and hides its copy latency that way: one control warp issues both the
// copies and the products (with a tenth warp it was a fifth slower).
constexpr int FWD_THREADS = (MATH_WARPS + 1) * 32;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                 "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
}
// issue only: several loads can then share one tmem_wait_ld()
template <int N>
__device__ __forceinline__ void tmem_ld_issue(uint32_t taddr, float* v) {
  static_assert(N == 16 || N % 32 == 0, "column count");
  if constexpr (N == 16) tmem_ld16_issue(taddr, v);
  else {
#pragma unroll
    for (int c = 0; c < N / 32; c++) tmem_ld32_issue(taddr + c * 32, v + c * 32);
  }
}
__device__ __forceinline__ void tmem_st16_issue(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                 "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}
// registers to N columns of this warp's lanes; complete after tmem_wait_st()
template <int N>
__device__ __forceinline__ void tmem_st_issue(uint32_t taddr, const float* v) {
  static_assert(N == 16 || N % 32 == 0, "column count");
  if constexpr (N == 16) tmem_st16_issue(taddr, v);
  else {
#pragma unroll
    for (int c = 0; c < N / 32; c++) tmem_st32_issue(taddr + c * 32, v + c * 32);
  }
}
// A descriptor of the same tile `bytes` further on (the start-address field counts 16-byte units and cannot
// carry: shared memory is smaller than the field's range).
__device__ __forceinline__ uint64_t desc_off(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float* v) {
  static_assert(N == 16 || N % 32 == 0, "column count");
  if constexpr (N == 16) tmem_ld16(taddr, v);
  else {
#pragma unroll
    for (int c = 0; c < N / 32; c++) tmem_ld32(taddr + c * 32, v + c * 32);
  }
}
// The gradient of a rotary embedding in the epilogue of the kernel that produced the gradient of its output: the two
// threads that share a row of a head 2 * HH wide each take half of its HH pairs (j, j + HH). With (c, s) the cosine and
// sine of (position, pair j) the input gradient of a pair is (c.g0 + s.g1, -s.g0 + c.g1). fetch() loads the thread's
// HH / 2 (cos, sin) pairs and is called before the wait for the last products, so the latency of that read (a piece of
// a table row per thread, from L2) is not added to the kernel's tail; store() reads both members of the thread's
// pairs from tensor memory (warp-wide loads: call it under warp-uniform control flow) and writes two runs of HH / 2
// values. Head sizes 64 and 128 (HH / 2 = 16 or 32 columns per load).
template <int HH>
struct RopeRow {
  static constexpr int P = HH / 2;   // pairs per thread
  static_assert(P == 16 || P == 32, "head size 64 or 128");
  float4 cs[P / 2];
  __device__ __forceinline__ void fetch(const float2* __restrict__ row, int half) {
    const float4* src = reinterpret_cast<const float4*>(row + half * P);
#pragma unroll
    for (int i = 0; i < P / 2; i++) cs[i] = __ldg(src + i);
  }
  // acc: tensor-memory address of the head's first column in this thread's lane; dst: the head's first column in
  // this thread's output row
  __device__ __forceinline__ void store(uint32_t acc, float* dst, int half, int accum, bool st, float factor) const {
    float g0[P], g1[P];
    tmem_ld_issue<P>(acc + half * P, g0);
    tmem_ld_issue<P>(acc + HH + half * P, g1);
    tmem_wait_ld();
    if (!st) return;
    float* d0 = dst + half * P;
    float* d1 = d0 + HH;
#pragma unroll
    for (int j = 0; j < P; j += 4) {
      const float4 u = cs[j >> 1], v = cs[(j >> 1) + 1];   // cos, sin of pairs j, j + 1; of pairs j + 2, j + 3
      float4 o0 = accum ? *reinterpret_cast<float4*>(d0 + j) : make_float4(0, 0, 0, 0);
      float4 o1 = accum ? *reinterpret_cast<float4*>(d1 + j) : make_float4(0, 0, 0, 0);
      o0.x += (u.x * g0[j] + u.y * g1[j]) * factor;             o1.x += (u.x * g1[j] - u.y * g0[j]) * factor;
      o0.y += (u.z * g0[j + 1] + u.w * g1[j + 1]) * factor;     o1.y += (u.z * g1[j + 1] - u.w * g0[j + 1]) * factor;
      o0.z += (v.x * g0[j + 2] + v.y * g1[j + 2]) * factor;     o1.z += (v.x * g1[j + 2] - v.y * g0[j + 2]) * factor;
      o0.w += (v.z * g0[j + 3] + v.w * g1[j + 3]) * factor;     o1.w += (v.z * g1[j + 3] - v.w * g0[j + 3]) * factor;
      *reinterpret_cast<float4*>(d0 + j) = o0;
      *reinterpret_cast<float4*>(d1 + j) = o1;
    }
  }
};
__device__ __forceinline__ void pair_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

// A bounded wait that becomes a no-op once any wait of this thread has expired.
struct Waiter {
  bool dead = false;
  int* flag;
  __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity, int code) {
    if (dead) return;
    if (!mbar_wait(bar, parity)) { dead = true; atomicExch(flag, code); }
  }
  __device__ __forceinline__ void wait_cluster(uint32_t bar, uint32_t parity, int code) {
    if (dead) return;
    if (!mbar_wait_cluster(bar, parity)) { dead = true; atomicExch(flag, code); }
  }
};

// Head dimension 256 runs as pairs of CTAs (a cluster of two): each holds one 128-wide half of the head, so its
// tiles are those of a 128-wide head, computes the score products over its half and adds the other CTA's partial
// sums; from there on both hold the same scores and each forms its half of the outputs. Math thread t of one CTA
// and math thread t of the other own the same elements, so a warp exchanges only with the same warp of the other
// CTA and has its own pair of barriers. A CTA has one exchange buffer, written by its peer: a warp's `full` counts
// the peer warp's 32 writers of a block, `free` (on the writer's side) the 32 readers of the block before.
constexpr int PAIR_XCHG_BYTES = 32 * MATH_WARPS * 32 * 4;   // 32 values per math thread
struct PairSum {
  uint32_t buf_peer, full_local, full_peer, free_local, free_peer;
  const float4* buf_local;
  __device__ __forceinline__ void init(uint32_t buf_s, const void* buf_ptr, uint32_t full, uint32_t free_, uint32_t peer) {
    buf_local = reinterpret_cast<const float4*>(buf_ptr);
    buf_peer = cluster_addr_of(buf_s, peer);
    full_local = full; free_local = free_;
    full_peer = cluster_addr_of(full, peer); free_peer = cluster_addr_of(free_, peer);
  }
  // a[0..NA) and b[0..NB) += the peer's values of block i (blocks are exchanged in order, i = 0, 1, 2, ...)
  template <int NA, int NB>
  __device__ __forceinline__ void add(Waiter& w, int i, int t, float* a, float* b, int code) {
    static_assert(NA % 4 == 0 && NB % 4 == 0 && NA + NB <= 32, "exchange size");
    if (i > 0) w.wait_cluster(free_local, (uint32_t)((i - 1) & 1), code);   // the peer has read block i-1
#pragma unroll
    for (int j = 0; j < (NA + NB) / 4; j++) {
      const float* v = j < NA / 4 ? a + 4 * j : b + 4 * (j - NA / 4);
      st_cluster_f32x4(buf_peer + (uint32_t)(j * (MATH_WARPS * 32) + t) * 16u, v[0], v[1], v[2], v[3]);
    }
    mbar_arrive_cluster(full_peer);
    w.wait_cluster(full_local, (uint32_t)(i & 1), code);
#pragma unroll
    for (int j = 0; j < (NA + NB) / 4; j++) {
      float* v = j < NA / 4 ? a + 4 * j : b + 4 * (j - NA / 4);
      const float4 x = buf_local[j * (MATH_WARPS * 32) + t];
      v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
    }
    mbar_arrive_cluster(free_peer);
  }
};

// Write NC consecutive f32 values, starting at column c0 (a multiple of 4), as row r of a K-major operand tile:
// atoms of 32 columns, 128 rows each, rows 128 B apart, 16-byte chunks XOR (row mod 8).
template <int NC>
__device__ __forceinline__ void store_row_kmajor(uint8_t* tile, int r, int c0, const float* v) {
#pragma unroll
  for (int i = 0; i < NC / 4; i++) {
    const int c4 = c0 / 4 + i;
    const int atom = c4 / 8, chunk = (c4 % 8) ^ (r & 7);
    *reinterpret_cast<float4*>(tile + atom * (ROWS * 128) + r * 128 + chunk * 16) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
}

// ---------------------------------------------------------------------------------------------
// Forward. Per 64-key block: S = Q.K^T (M=128, N=64) -> mask, online softmax -> P (A operand) -> O_blk = P.V,
// folded into a register accumulator with the rescale factor. The two warps of a lane quadrant split the 64
// keys for the softmax (exchanging their partial row maxima through shared memory) and the head dimension
// for the accumulator.
// ---------------------------------------------------------------------------------------------
constexpr int BKV = 64;

template <int HD, int SPLIT>
struct FwdSmem {
  static constexpr int Q_BYTES = ROWS * HD * 4, K_BYTES = BKV * HD * 4, V_BYTES = BKV * HD * 4, P_BYTES = ROWS * BKV * 4;
  static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + K_BYTES, P_OFF = V_OFF + V_BYTES, X_OFF = P_OFF + P_BYTES;
  static constexpr int X_BYTES = 2 * 2 * ROWS * 4;   // partial row maxima [parity][half][row]
  static constexpr int XC_OFF = X_OFF + X_BYTES, XC_BYTES = SPLIT == 2 ? PAIR_XCHG_BYTES : 0;   // the peer's partial scores
  static constexpr int BAR_OFF = XC_OFF + XC_BYTES;
  static constexpr int TOTAL = BAR_OFF + (SPLIT == 2 ? 256 : 128) + 1024;   // a pair adds one exchange barrier pair per math warp
  static constexpr uint32_t TMEM_COLS = (2 * BKV + HD) <= 256 ? 256 : 512;
  static_assert(TOTAL <= 232448, "shared memory");
};

template <int HD, int SPLIT>   // HD: columns of the head held by one CTA; the head is HD * SPLIT wide
__global__ void __launch_bounds__(FWD_THREADS, HD <= 64 ? 2 : 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, float* __restrict__ out, float* __restrict__ lse, int rows, int T,
                   int Hq, int Hkv, int window, float scale2, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = FwdSmem<HD, SPLIT>;
  constexpr int ATOMS = HD / 32, HH = HD / 2, HDF = HD * SPLIT;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_s = base + S::Q_OFF, k_s = base + S::K_OFF, v_s = base + S::V_OFF, p_s = base + S::P_OFF;
  float* xch = reinterpret_cast<float*>(base_ptr + S::X_OFF);
  const uint32_t bars = base + S::BAR_OFF;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 16, s_full0 = bars + 24, s_full1 = bars + 32, p_full = bars + 40,
                 o_full = bars + 48, x_full = bars + 128, x_free = bars + 192;
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + S::BAR_OFF + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Causal work grows with the query position: the heaviest tiles are launched first, and all (head, sequence)
  // pairs of one tile index are adjacent, so the tail of the grid is made of the lightest tiles.
  const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * ROWS;
  const int crank = SPLIT == 2 ? (int)(blockIdx.x & 1) : 0, bx = blockIdx.x / SPLIT;   // which half of the head; tile
  const int h = bx % Hq, seq = bx / Hq;
  const int kvh = h / (Hq / Hkv);
  const int row0 = seq * T;
  const int q_last = min(q0 + ROWS - 1, T - 1);
  const int kb_lo = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / BKV : 0;
  const int kb_hi = q_last / BKV;
  const int nkb = kb_hi - kb_lo + 1;

  if (threadIdx.x == 0) {
    tma_prefetch_map(&mapQ); tma_prefetch_map(&mapK); tma_prefetch_map(&mapV);
    mbar_init(q_full, 1); mbar_init(k_full, 1); mbar_init(v_full, 1); mbar_init(s_full0, 1); mbar_init(s_full1, 1);
    mbar_init(p_full, MATH_WARPS * 32); mbar_init(o_full, 1);
    if (SPLIT == 2)
      for (int mw = 0; mw < MATH_WARPS; mw++) { mbar_init(x_full + 8 * mw, 32); mbar_init(x_free + 8 * mw, 32); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  if (SPLIT == 2) cluster_sync_all(); else __syncthreads();   // the peer's barriers exist before anything arrives there
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t tm_o = tmem + 2 * BKV;
  Waiter w{false, flag};
  PairSum xs;
  if (SPLIT == 2 && warp < MATH_WARPS) xs.init(base + S::XC_OFF, base_ptr + S::XC_OFF, x_full + 8 * warp, x_free + 8 * warp, (uint32_t)(crank ^ 1));
  auto s_bar = [&](int it) { return (it & 1) ? s_full1 : s_full0; };
  auto s_par = [&](int it) { return (uint32_t)((it >> 1) & 1); };

  auto load_k = [&](int i) {
    mbar_expect_tx(k_full, S::K_BYTES);
    tma_load_3d(k_s, &mapK, 0, row0 + (kb_lo + i) * BKV, (kvh * SPLIT + crank) * ATOMS, k_full);
  };
  auto load_v = [&](int i) {
    mbar_expect_tx(v_full, S::V_BYTES);
    tma_load_3d(v_s, &mapV, 0, row0 + (kb_lo + i) * BKV, (kvh * SPLIT + crank) * ATOMS, v_full);
  };
  if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_tf32(false, false, ROWS, BKV);   // S = Q.K^T, both K-major
      constexpr uint32_t idesc_o = idesc_tf32(false, true, ROWS, HD);     // O = P.V, V is [keys, hd]
      const uint64_t d_q = desc_kmajor(q_s), d_k = desc_kmajor(k_s), d_p = desc_kmajor(p_s), d_v = smem_desc(v_s, BKV * 128, 512, 1);
      auto mma_s = [&](int i) {
        const uint32_t tm_s = tmem + (i & 1) * BKV;
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            umma_tf32(tm_s, desc_off(d_q, a * (ROWS * 128) + j * 32), desc_off(d_k, a * (BKV * 128) + j * 32), idesc_s,
                      (a > 0 || j > 0) ? 1u : 0u);
        umma_commit(s_bar(i));
      };
      mbar_expect_tx(q_full, S::Q_BYTES);
      tma_load_3d(q_s, &mapQ, 0, row0 + q0, (h * SPLIT + crank) * ATOMS, q_full);
      load_k(0);
      load_v(0);
      w.wait(q_full, 0, 11);
      w.wait(k_full, 0, 12);
      tc_fence_after();
      mma_s(0);
      w.wait(s_full0, 0, 13);
      if (nkb > 1) load_k(1);
      for (int i = 0; i < nkb; i++) {
        if (i + 1 < nkb) {                     // next block's scores, under this block's softmax
          w.wait(k_full, (i + 1) & 1, 12);
          tc_fence_after();
          mma_s(i + 1);
        }
        w.wait(v_full, i & 1, 14);
        w.wait(p_full, i & 1, 14);
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < BKV / 8; j++)
          umma_tf32(tm_o, desc_off(d_p, (j / 4) * (ROWS * 128) + (j % 4) * 32), desc_off(d_v, j * 1024), idesc_o, j > 0 ? 1u : 0u);
        umma_commit(o_full);
        if (i + 2 < nkb) {                     // K tile read: fetch the one after
          w.wait(s_bar(i + 1), s_par(i + 1), 13);
          load_k(i + 2);
        }
        w.wait(o_full, i & 1, 15);             // V and P tiles read
        if (i + 1 < nkb) load_v(i + 1);
      }
    }
  } else if (warp < MATH_WARPS) {
    const int qd = warp & 3, half = warp >> 2;
    const int r = qd * 32 + lane;
    const int tq = q0 + r;
    const bool valid = tq < T;
    const int lo = (window > 0) ? tq - window + 1 : 0;
    float m = NEG, l = 0.f;
    float o[HH];
#pragma unroll
    for (int d = 0; d < HH; d++) o[d] = 0.f;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    for (int i = 0; i < nkb; i++) {
      const int k0 = (kb_lo + i) * BKV + half * 32;
      w.wait(s_bar(i), s_par(i), 16);
      tc_fence_after();
      float s[32];
      const uint32_t tm_s = tmem + (i & 1) * BKV + half * 32 + lane_base;
      tmem_ld<32>(tm_s, s);
      if constexpr (SPLIT == 2) xs.add<32, 0>(w, i, (int)threadIdx.x, s, s, 18);   // + the other half of the head
      // a block strictly below the diagonal and inside the window needs no per-element test
      const bool interior = (k0 + 31 <= q0) && (q0 + ROWS - 1 < T) && (window == 0 || k0 >= q0 + ROWS - window);
      float mx = NEG;
      if (interior) {
#pragma unroll
        for (int c = 0; c < 32; c++) { s[c] *= scale2; mx = fmaxf(mx, s[c]); }
      } else {
#pragma unroll
        for (int c = 0; c < 32; c++) {
          const int kg = k0 + c;
          s[c] = (valid && kg <= tq && kg >= lo) ? s[c] * scale2 : NEG;
          mx = fmaxf(mx, s[c]);
        }
      }
      float* xp = xch + (i & 1) * (2 * ROWS);
      xp[half * ROWS + r] = mx;
      pair_sync(1 + qd);
      mx = fmaxf(mx, xp[(half ^ 1) * ROWS + r]);
      const float mn = fmaxf(m, mx);
      const float alpha = ex2(m - mn);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 32; c++) {
        const float p = (s[c] > -1.0e38f) ? ex2(s[c] - mn) : 0.f;
        s[c] = p;
        sum += p;
      }
      l = l * alpha + sum;
      m = mn;
      // (P passed through tensor memory instead, as in the backward kernels, measured a tenth slower here)
      store_row_kmajor<32>(base_ptr + S::P_OFF, r, half * 32, s);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
      w.wait(o_full, i & 1, 17);
      tc_fence_after();
      float t[HH];
      tmem_ld<HH>(tm_o + half * HH + lane_base, t);
#pragma unroll
      for (int d = 0; d < HH; d++) o[d] = o[d] * alpha + t[d];
      tc_fence_before();
    }
    // total row sum = the two halves' sums (same running max on both sides)
    float* xp = xch;   // every exchange slot was last read before the pair's final sync of the loop
    pair_sync(1 + qd);
    xp[half * ROWS + r] = l;
    pair_sync(1 + qd);
    l += xp[(half ^ 1) * ROWS + r];
    if (!w.dead && valid) {
      const float inv = TRUNC_COMP / l;   // the P.V product carries the truncation bias of both operands
      float* dst = out + (size_t)(row0 + tq) * Hq * HDF + (size_t)h * HDF + crank * HD + half * HH;
#pragma unroll
      for (int d = 0; d < HH; d += 4) *reinterpret_cast<float4*>(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
      if (half == 0 && crank == 0) lse[(size_t)h * rows + row0 + tq] = m + log2f(l);
    }
  }
  tc_fence_before();
  if (SPLIT == 2) cluster_sync_all(); else __syncthreads();   // neither CTA of a pair leaves while the other may still write to it
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Backward. Ds[h,row] = scale * sum_d dO*O first (one warp per (row, head)), then two kernels, as in the
// reference (srcAttnBwdDq, srcAttnBwdDkv): each recomputes S and dP on the tensor cores, forms p and dS in
// registers and feeds them back as the A operand of the gradient products, whose accumulators stay in TMEM for
// the whole loop. Nothing is reduced with atomics: one CTA owns its 128 query rows (dQ) or its 128 key rows
// (dK, dV, summing its GQA group inside the loop), so results are deterministic.
// ---------------------------------------------------------------------------------------------
// HD / 4 lanes per (row, head), one 16-byte load of dO and of O each: the kernel streams both tensors once.
template <int HD>
__global__ void attn_bwd_d_tc_kernel(long nitems, float scale, const float* __restrict__ go, const float* __restrict__ o,
                                     float* __restrict__ D, int rows, int Hq) {
  constexpr int L = HD / 4 < 32 ? HD / 4 : 32;   // lanes per item: 8, 16 or 32
  constexpr int PER = HD / 4 / L;                // 16-byte loads per lane and tensor (2 at HD 256)
  const long gid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long item = gid / L;                  // row * Hq + h
  const int sub = (int)(gid % L);
  float acc = 0.f;
  if (item < nitems) {
#pragma unroll
    for (int e = 0; e < PER; e++) {
      const float4 g = __ldg(reinterpret_cast<const float4*>(go + item * HD) + sub + e * L);
      const float4 v = __ldg(reinterpret_cast<const float4*>(o + item * HD) + sub + e * L);
      acc += g.x * v.x + g.y * v.y + g.z * v.z + g.w * v.w;
    }
  }
#pragma unroll
  for (int off = L / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (item < nitems && sub == 0) {
    const long row = item / Hq;
    const int h = (int)(item % Hq);
    D[(size_t)h * rows + row] = acc * scale;
  }
}

// ---- dK, dV: CTA = 128 keys of one kv head; loop over the group's query heads and over blocks of NQ queries ----
// Transposed products so that keys are the rows: S^T = K.Q^T and dP^T = V.dO^T (M=128 keys, N=NQ queries); then
// dV += P^T.dO and dK += dS^T.Q with P^T, dS^T written to shared memory as K-major A operands (K = queries) and
// dO, Q read a second time as [queries, hd] operands (hd contiguous). KBUF = 2 keeps two blocks of the K-major
// Q / dO copies in flight (their fetch is the longest latency of the loop) where shared memory has the room.
template <int HD, int NQ, int KBUF, int MBUF, int SPLIT>
struct DkvSmem {
  static constexpr int KV_BYTES = ROWS * HD * 4, QT_BYTES = NQ * HD * 4;
  static constexpr int K_OFF = 0, V_OFF = KV_BYTES, QK_OFF = 2 * KV_BYTES, GK_OFF = QK_OFF + KBUF * QT_BYTES,
                       QM_OFF = GK_OFF + KBUF * QT_BYTES, GM_OFF = QM_OFF + MBUF * QT_BYTES, XC_OFF = GM_OFF + MBUF * QT_BYTES,
                       BAR_OFF = XC_OFF + (SPLIT == 2 ? PAIR_XCHG_BYTES : 0);
  static constexpr int TOTAL = BAR_OFF + (SPLIT == 2 ? 256 : 128) + 1024;   // a pair adds one exchange barrier pair per math warp
  static constexpr int COLS = 4 * NQ + 2 * HD;
  static_assert(SPLIT == 1 || NQ <= 32, "a pair exchanges at most 32 values per thread");
  static constexpr uint32_t TMEM_COLS = COLS <= 128 ? 128 : (COLS <= 256 ? 256 : 512);
  static_assert(TOTAL <= 232448, "shared memory");
};

template <int HD, int NQ, int KBUF, int MBUF, int SPLIT>
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                       const __grid_constant__ CUtensorMap mapQk, const __grid_constant__ CUtensorMap mapQm,
                       const __grid_constant__ CUtensorMap mapGk, const __grid_constant__ CUtensorMap mapGm,
                       const float* __restrict__ lse, const float* __restrict__ Ds, float* gk, int accum_k, float* gv, int accum_v,
                       int rows, int T, int Hq, int Hkv, int window, float scale2, float dp_scale, const float2* __restrict__ rope,
                       const int* __restrict__ order, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = DkvSmem<HD, NQ, KBUF, MBUF, SPLIT>;
  constexpr int ATOMS = HD / 32, NH = NQ / 2, HH = HD / 2, HDF = HD * SPLIT;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t k_s = base + S::K_OFF, v_s = base + S::V_OFF, qk_s = base + S::QK_OFF, gk_s = base + S::GK_OFF,
                 qm_s = base + S::QM_OFF, gm_s = base + S::GM_OFF;
  const uint32_t bars = base + S::BAR_OFF;
  const uint32_t kv_full = bars, qk_full0 = bars + 8, qk_full1 = bars + 16, qm_full0 = bars + 24, s_full0 = bars + 32,
                 s_full1 = bars + 40, p_full0 = bars + 48, acc_done0 = bars + 56, all_done = bars + 72, qm_full1 = bars + 80,
                 p_full1 = bars + 88, acc_done1 = bars + 96, x_full = bars + 128, x_free = bars + 192;
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + S::BAR_OFF + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Which (key block, kv head, sequence) this CTA takes. CTAs start in index order as SMs fall free; early key blocks are
  // read by the most queries, so plain index order is heaviest first. `order` (one CTA per tile only) replaces it by
  // the order a packing of the tiles into the SMs prescribes (attn_dkv_order).
  int tile_y = blockIdx.y, tile_x = blockIdx.x;
  if (SPLIT == 1 && order != nullptr) {
    const int lin = order[blockIdx.y * gridDim.x + blockIdx.x];
    tile_y = lin / (int)gridDim.x;
    tile_x = lin % (int)gridDim.x;
  }
  const int k0 = tile_y * ROWS;
  const int crank = SPLIT == 2 ? (int)(tile_x & 1) : 0, bx = tile_x / SPLIT;   // which half of the head; tile
  const int kvh = bx % Hkv, seq = bx / Hkv;
  const int group = Hq / Hkv;
  const int row0 = seq * T;
  const int k_last = min(k0 + ROWS - 1, T - 1);
  const int q_max = (window > 0) ? min(T - 1, k_last + window - 1) : T - 1;
  const int qb_lo = k0 / NQ, qb_hi = q_max / NQ;
  const int nqb = qb_hi - qb_lo + 1;
  const int iters = nqb * group;

  if (threadIdx.x == 0) {
    tma_prefetch_map(&mapK); tma_prefetch_map(&mapV); tma_prefetch_map(&mapQk); tma_prefetch_map(&mapGk);
    tma_prefetch_map(&mapQm); tma_prefetch_map(&mapGm);
    mbar_init(kv_full, 1); mbar_init(qk_full0, 1); mbar_init(qk_full1, 1); mbar_init(qm_full0, 1); mbar_init(qm_full1, 1);
    mbar_init(s_full0, 1);
    mbar_init(s_full1, 1); mbar_init(p_full0, MATH_WARPS * 32); mbar_init(p_full1, MATH_WARPS * 32); mbar_init(acc_done0, 1);
    mbar_init(acc_done1, 1); mbar_init(all_done, 1);
    if (SPLIT == 2)
      for (int mw = 0; mw < MATH_WARPS; mw++) { mbar_init(x_full + 8 * mw, 32); mbar_init(x_free + 8 * mw, 32); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  if (SPLIT == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  // columns: [S^T | dP^T] x 2 buffers, then dV, dK
  const uint32_t tm_dv = tmem + 4 * NQ, tm_dk = tmem + 4 * NQ + HD;
  Waiter w{false, flag};
  PairSum xs;
  if (SPLIT == 2 && warp < MATH_WARPS) xs.init(base + S::XC_OFF, base_ptr + S::XC_OFF, x_full + 8 * warp, x_free + 8 * warp, (uint32_t)(crank ^ 1));
  // barrier and parity of the K-major copies of block `it`, and of its score products
  auto qk_bar = [&](int it) { return (KBUF == 2 && (it & 1)) ? qk_full1 : qk_full0; };
  auto qk_par = [&](int it) { return (uint32_t)((KBUF == 2 ? it >> 1 : it) & 1); };
  // p_full and acc_done alternate between two barriers: their waiters are not throttled by anything else in the
  // loop, and with a single barrier a waiter that fell one phase behind would take the next phase of the same parity
  // for the one it missed and wait for ever. With two, that needs four phases, which the data dependences rule out.
  auto p_bar = [&](int it) { return (it & 1) ? p_full1 : p_full0; };
  auto a_bar = [&](int it) { return (it & 1) ? acc_done1 : acc_done0; };
  auto qm_bar = [&](int it) { return (MBUF == 2 && (it & 1)) ? qm_full1 : qm_full0; };
  auto qm_par = [&](int it) { return (uint32_t)((MBUF == 2 ? it >> 1 : it) & 1); };
  auto s_bar = [&](int it) { return (it & 1) ? s_full1 : s_full0; };
  auto s_par = [&](int it) { return (uint32_t)((it >> 1) & 1); };

  if (warp == TMA_WARP) {
    if (lane == 0) {
      // Both copies are requested block after block, so (head, query block) of the next request is kept by counting:
      // a division by the run-time block count costs this single thread more than the copy instructions themselves.
      int k_h = kvh * group, k_qb = 0, m_h = kvh * group, m_qb = 0;
      auto load_k = [&](int it) {   // K-major copies of Q and dO, block `it` (called with it = 0, 1, 2, ...)
        const int qr = row0 + (qb_lo + k_qb) * NQ;
        const uint32_t bar = qk_bar(it), off = (KBUF == 2 && (it & 1)) ? S::QT_BYTES : 0;
        mbar_expect_tx(bar, 2 * S::QT_BYTES);
        tma_load_3d(qk_s + off, &mapQk, 0, qr, (k_h * SPLIT + crank) * ATOMS, bar);
        tma_load_3d(gk_s + off, &mapGk, 0, qr, (k_h * SPLIT + crank) * ATOMS, bar);
        if (++k_qb == nqb) { k_qb = 0; k_h++; }
      };
      auto load_m = [&](int it) {   // [queries, hd] copies for the gradient products, block `it` (same order)
        const int qr = row0 + (qb_lo + m_qb) * NQ;
        const uint32_t bar = qm_bar(it), off = (MBUF == 2 && (it & 1)) ? S::QT_BYTES : 0;
        mbar_expect_tx(bar, 2 * S::QT_BYTES);
        tma_load_3d(qm_s + off, &mapQm, 0, qr, (m_h * SPLIT + crank) * ATOMS, bar);
        tma_load_3d(gm_s + off, &mapGm, 0, qr, (m_h * SPLIT + crank) * ATOMS, bar);
        if (++m_qb == nqb) { m_qb = 0; m_h++; }
      };
      mbar_expect_tx(kv_full, 2 * S::KV_BYTES);
      tma_load_3d(k_s, &mapK, 0, row0 + k0, (kvh * SPLIT + crank) * ATOMS, kv_full);
      tma_load_3d(v_s, &mapV, 0, row0 + k0, (kvh * SPLIT + crank) * ATOMS, kv_full);
      load_k(0);
      load_m(0);
      if (KBUF == 2 && iters > 1) load_k(1);
      if (MBUF == 2 && iters > 1) load_m(1);
      // waits in the order the products complete: scores of block 0, then scores of block i+1 before the
      // gradient products of block i. Once the scores of a block are done its K-major copies may be replaced.
      w.wait(s_full0, 0, 23);
      if (KBUF < iters) load_k(KBUF);
      for (int i = 0; i < iters; i++) {
        if (i + 1 + KBUF < iters) {
          w.wait(s_bar(i + 1), s_par(i + 1), 23);
          load_k(i + 1 + KBUF);
        }
        w.wait(a_bar(i), s_par(i), 25);           // the gradient products have read the [queries, hd] copies
        if (i + MBUF < iters) load_m(i + MBUF);
      }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_tf32(false, false, ROWS, NQ);
      constexpr uint32_t idesc_g = idesc_tf32(false, true, ROWS, HD);
      const uint64_t d_k = desc_kmajor(k_s), d_v = desc_kmajor(v_s), d_qk = desc_kmajor(qk_s), d_gk = desc_kmajor(gk_s),
                     d_gm = smem_desc(gm_s, NQ * 128, 512, 1), d_qm = smem_desc(qm_s, NQ * 128, 512, 1);
      auto mma_s = [&](int it) {
        const uint32_t tm_s = tmem + (it & 1) * 2 * NQ, tm_dp = tm_s + NQ;
        const uint32_t boff = (KBUF == 2 && (it & 1)) ? S::QT_BYTES : 0;
        // one accumulator at a time: consecutive MMAs into the same TMEM columns pipeline, alternating ones do not
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            umma_tf32(tm_s, desc_off(d_k, a * (ROWS * 128) + j * 32), desc_off(d_qk, boff + a * (NQ * 128) + j * 32), idesc_s,
                      (a > 0 || j > 0) ? 1u : 0u);
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            umma_tf32(tm_dp, desc_off(d_v, a * (ROWS * 128) + j * 32), desc_off(d_gk, boff + a * (NQ * 128) + j * 32), idesc_s,
                      (a > 0 || j > 0) ? 1u : 0u);
        umma_commit(s_bar(it));
      };
      w.wait(kv_full, 0, 21);
      w.wait(qk_full0, 0, 22);
      tc_fence_after();
      mma_s(0);
      for (int i = 0; i < iters; i++) {
        if (i + 1 < iters) {                      // next block's scores, under this block's element math
          w.wait(qk_bar(i + 1), qk_par(i + 1), 22);
          tc_fence_after();
          mma_s(i + 1);
        }
        w.wait(qm_bar(i), qm_par(i), 24);
        w.wait(p_bar(i), s_par(i), 24);
        tc_fence_after();
        const uint32_t tm_p = tmem + (i & 1) * 2 * NQ;   // P^T and dS^T where the math warps wrote them: over S^T, dP^T
        const uint32_t moff = (MBUF == 2 && (i & 1)) ? S::QT_BYTES : 0;
#pragma unroll
        for (int j = 0; j < NQ / 8; j++) umma_tf32_ts(tm_dv, tm_p + j * 8, desc_off(d_gm, moff + j * 1024), idesc_g, (i > 0 || j > 0) ? 1u : 0u);
#pragma unroll
        for (int j = 0; j < NQ / 8; j++)
          umma_tf32_ts(tm_dk, tm_p + NQ + j * 8, desc_off(d_qm, moff + j * 1024), idesc_g, (i > 0 || j > 0) ? 1u : 0u);
        umma_commit(a_bar(i));
      }
      // The end of the accumulation has a barrier of its own, used once (the math warps do not follow acc_done).
      // The issuing thread waits for it too, whatever happened before: no MMA may be in flight when TMEM is freed.
      umma_commit(all_done);
      mbar_wait(all_done, 0);
    }
  } else {
    const int qd = warp & 3, half = warp >> 2;
    const int kg = k0 + qd * 32 + lane;      // key position in the sequence: one row of the tile per thread
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    int c_h = kvh * group, c_qb = 0;         // (head, query block) of block i, kept by counting
    for (int i = 0; i < iters; i++) {
      const int h = c_h;
      const int qpos0 = (qb_lo + c_qb) * NQ + half * NH;         // first query of this thread's columns
      if (++c_qb == nqb) { c_qb = 0; c_h++; }
      const float4* l4 = reinterpret_cast<const float4*>(lse + (size_t)h * rows + row0 + qpos0);
      const float4* d4 = reinterpret_cast<const float4*>(Ds + (size_t)h * rows + row0 + qpos0);
      // every (key, query) pair of the tile kept: keys at or before the first query, queries inside the sequence
      // and, with a window, the last query still within reach of the first key
      const bool interior = (k0 + ROWS - 1 <= qpos0) && (qpos0 + NH - 1 < T) && (window == 0 || k0 >= qpos0 + NH - window) &&
                            (((size_t)h * rows + row0) % 4 == 0);   // and the 16-byte loads of LSE / Ds are aligned
      float4 Lv[NH / 4], Dv[NH / 4];
      if (interior) {                            // fetched under the wait for the products
#pragma unroll
        for (int c4 = 0; c4 < NH / 4; c4++) { Lv[c4] = __ldg(l4 + c4); Dv[c4] = __ldg(d4 + c4); }
      }
      w.wait(s_bar(i), s_par(i), 26);
      tc_fence_after();
      float s[NH], dp[NH];
      const uint32_t tm_s = tmem + (i & 1) * 2 * NQ + half * NH + lane_base;
      tmem_ld_issue<NH>(tm_s, s);
      tmem_ld_issue<NH>(tm_s + NQ, dp);
      tmem_wait_ld();
      if constexpr (SPLIT == 2) xs.add<NH, NH>(w, i, (int)threadIdx.x, s, dp, 29);   // + the other half of the head
      if (interior) {
#pragma unroll
        for (int c4 = 0; c4 < NH / 4; c4++) {
          const float Ls[4] = {Lv[c4].x, Lv[c4].y, Lv[c4].z, Lv[c4].w}, Dd[4] = {Dv[c4].x, Dv[c4].y, Dv[c4].z, Dv[c4].w};
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const int c = c4 * 4 + e;
            const float p = ex2(fmaf(s[c], scale2, -Ls[e]));
            s[c] = p;
            dp[c] = p * fmaf(dp[c], dp_scale, -Dd[e]);
          }
        }
      } else {
        const float* lrow = lse + (size_t)h * rows + row0 + qpos0;
        const float* drow = Ds + (size_t)h * rows + row0 + qpos0;
#pragma unroll
        for (int c = 0; c < NH; c++) {
          const int tq = qpos0 + c;
          const bool keep = tq < T && kg <= tq && (window == 0 || kg >= tq - window + 1);
          float p = 0.f, d = 0.f;
          if (keep) {
            p = ex2(fmaf(s[c], scale2, -__ldg(lrow + c)));
            d = p * fmaf(dp[c], dp_scale, -__ldg(drow + c));
          }
          s[c] = p;
          dp[c] = d;
        }
      }
      // In place: these columns were last read by the gradient products of block i-2, which the tensor pipe
      // finished before it wrote the scores of block i there.
      tmem_st_issue<NH>(tm_s, s);
      tmem_st_issue<NH>(tm_s + NQ, dp);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_bar(i));
    }
    RopeRow<HD >= 64 ? HH : 32> rr;   // (unused below head size 64: the host then launches the rotation's backward itself)
    const bool roped = SPLIT == 1 && HD >= 64 && rope != nullptr && gk != nullptr;
    if (roped) rr.fetch(rope + (size_t)(kg < T ? kg : 0) * HH, half);
    w.wait(all_done, 0, 28);
    tc_fence_after();
    {   // warp-uniform: the TMEM loads are warp-wide instructions, only the stores are per-row
      const bool st = !w.dead && kg < T;
      const size_t off = (size_t)(row0 + (kg < T ? kg : 0)) * Hkv * HDF + (size_t)kvh * HDF + crank * HD + half * HH;
      float t[HH];
      if (gv) {
        tmem_ld<HH>(tm_dv + half * HH + lane_base, t);
        float* dst = gv + off;
        if (st) {
#pragma unroll
          for (int d = 0; d < HH; d += 4) {
            float4 o = accum_v ? *reinterpret_cast<float4*>(dst + d) : make_float4(0, 0, 0, 0);
            o.x += t[d] * TRUNC_COMP; o.y += t[d + 1] * TRUNC_COMP; o.z += t[d + 2] * TRUNC_COMP; o.w += t[d + 3] * TRUNC_COMP;
            *reinterpret_cast<float4*>(dst + d) = o;
          }
        }
      }
      if (roped) {
        if constexpr (SPLIT == 1 && HD >= 64) rr.store(tm_dk + lane_base, gk + off - half * HH, half, accum_k, st, TRUNC_COMP);
      } else if (gk) {
        tmem_ld<HH>(tm_dk + half * HH + lane_base, t);
        float* dst = gk + off;
        if (st) {
#pragma unroll
          for (int d = 0; d < HH; d += 4) {
            float4 o = accum_k ? *reinterpret_cast<float4*>(dst + d) : make_float4(0, 0, 0, 0);
            o.x += t[d] * TRUNC_COMP; o.y += t[d + 1] * TRUNC_COMP; o.z += t[d + 2] * TRUNC_COMP; o.w += t[d + 3] * TRUNC_COMP;
            *reinterpret_cast<float4*>(dst + d) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  if (SPLIT == 2) cluster_sync_all(); else __syncthreads();   // neither CTA of a pair leaves while the other may still write to it
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

// ---- dQ: CTA = 128 queries of one head; loop over blocks of NK keys ----
// S = Q.K^T and dP = dO.V^T (M=128 queries, N=NK keys); dS written as a K-major A operand (K = keys);
// dQ += dS.K with K read a second time as a [keys, hd] operand. KBUF as in the dK/dV kernel.
// SB: one [S | dP] pair in tensor memory instead of two and single-buffered copies, small enough for two CTAs per SM:
// a CTA then runs its products and its element math strictly one after the other, and the second CTA fills the gaps.
template <int HD, int NK, int KBUF, bool SB, int SPLIT>
struct DqSmem {
  static constexpr int Q_BYTES = ROWS * HD * 4, KT_BYTES = NK * HD * 4;
  static constexpr int Q_OFF = 0, G_OFF = Q_BYTES, KK_OFF = 2 * Q_BYTES, VK_OFF = KK_OFF + KBUF * KT_BYTES,
                       KM_OFF = VK_OFF + KBUF * KT_BYTES, XC_OFF = KM_OFF + KT_BYTES, BAR_OFF = XC_OFF + (SPLIT == 2 ? PAIR_XCHG_BYTES : 0);
  static_assert(SPLIT == 1 || NK <= 32, "a pair exchanges at most 32 values per thread");
  static constexpr int SLACK = SB ? 896 : 1024;   // for rounding the base up to 1024 B (two CTAs must fit 228 KB together)
  static constexpr int TOTAL = BAR_OFF + (SPLIT == 2 ? 256 : 128) + SLACK;
  static constexpr int COLS = (SB ? 2 : 4) * NK + HD;
  static constexpr uint32_t TMEM_COLS = COLS <= 128 ? 128 : (COLS <= 256 ? 256 : 512);
  static_assert(TOTAL <= 232448, "shared memory");
};

template <int HD, int NK, int KBUF, bool SB, int SPLIT>
__global__ void __launch_bounds__(THREADS, SB ? 2 : 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapG,
                      const __grid_constant__ CUtensorMap mapKk, const __grid_constant__ CUtensorMap mapVk,
                      const __grid_constant__ CUtensorMap mapKm, const float* __restrict__ lse, const float* __restrict__ Ds,
                      float* gq, int accum_q, int rows, int T, int Hq, int Hkv, int window, float scale2, float dp_scale, const float2* __restrict__ rope,
                      int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = DqSmem<HD, NK, KBUF, SB, SPLIT>;
  constexpr int ATOMS = HD / 32, NH = NK / 2, HH = HD / 2, HDF = HD * SPLIT;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  if (base - smem_u32(smem_raw) > (uint32_t)S::SLACK) {   // cannot happen while dynamic shared memory starts 128-byte aligned
    if (threadIdx.x == 0) atomicExch(flag, 39);
    return;
  }
  const uint32_t q_s = base + S::Q_OFF, g_s = base + S::G_OFF, kk_s = base + S::KK_OFF, vk_s = base + S::VK_OFF, km_s = base + S::KM_OFF;
  const uint32_t bars = base + S::BAR_OFF;
  const uint32_t q_full = bars, kk_full0 = bars + 8, kk_full1 = bars + 16, km_full = bars + 24, s_full0 = bars + 32,
                 s_full1 = bars + 40, p_full0 = bars + 48, acc_done = bars + 56, all_done = bars + 72, p_full1 = bars + 80,
                 x_full = bars + 128, x_free = bars + 192;
  const uint32_t tmem_slot = bars + 64;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + S::BAR_OFF + 64);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = ((int)gridDim.y - 1 - (int)blockIdx.y) * ROWS;   // late queries read the most keys: heaviest first
  const int crank = SPLIT == 2 ? (int)(blockIdx.x & 1) : 0, bx = blockIdx.x / SPLIT;   // which half of the head; tile
  const int h = bx % Hq, seq = bx / Hq;
  const int kvh = h / (Hq / Hkv);
  const int row0 = seq * T;
  const int q_last = min(q0 + ROWS - 1, T - 1);
  const int kb_lo = (window > 0 && q0 - window + 1 > 0) ? (q0 - window + 1) / NK : 0;
  const int kb_hi = q_last / NK;
  const int iters = kb_hi - kb_lo + 1;

  if (threadIdx.x == 0) {
    tma_prefetch_map(&mapQ); tma_prefetch_map(&mapG); tma_prefetch_map(&mapKk); tma_prefetch_map(&mapVk); tma_prefetch_map(&mapKm);
    mbar_init(q_full, 1); mbar_init(kk_full0, 1); mbar_init(kk_full1, 1); mbar_init(km_full, 1); mbar_init(s_full0, 1);
    mbar_init(s_full1, 1); mbar_init(p_full0, MATH_WARPS * 32); mbar_init(p_full1, MATH_WARPS * 32); mbar_init(acc_done, 1);
    mbar_init(all_done, 1);
    if (SPLIT == 2)
      for (int mw = 0; mw < MATH_WARPS; mw++) { mbar_init(x_full + 8 * mw, 32); mbar_init(x_free + 8 * mw, 32); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) tmem_alloc(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  if (SPLIT == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  const uint32_t tm_dq = tmem + (SB ? 2 : 4) * NK;
  PairSum xs;
  if (SPLIT == 2 && warp < MATH_WARPS) xs.init(base + S::XC_OFF, base_ptr + S::XC_OFF, x_full + 8 * warp, x_free + 8 * warp, (uint32_t)(crank ^ 1));
  auto sbuf = [&](int it) { return SB ? 0u : (uint32_t)((it & 1) * 2 * NK); };   // TMEM columns of block it's [S | dP]
  Waiter w{false, flag};
  // two alternating p_full barriers, as in the dK/dV kernel: the math warps may finish block i+1 before the issuing
  // thread has looked at block i's barrier (it may be waiting for the [keys, hd] copy)
  auto p_bar = [&](int it) { return (it & 1) ? p_full1 : p_full0; };
  auto kk_bar = [&](int it) { return (KBUF == 2 && (it & 1)) ? kk_full1 : kk_full0; };
  auto kk_par = [&](int it) { return (uint32_t)((KBUF == 2 ? it >> 1 : it) & 1); };
  auto s_bar = [&](int it) { return (it & 1) ? s_full1 : s_full0; };
  auto s_par = [&](int it) { return (uint32_t)((it >> 1) & 1); };

  if (warp == TMA_WARP) {
    if (lane == 0) {
      auto load_k = [&](int it) {   // K-major copies of K and V
        const int kr = row0 + (kb_lo + it) * NK;
        const uint32_t bar = kk_bar(it), off = (KBUF == 2 && (it & 1)) ? S::KT_BYTES : 0;
        mbar_expect_tx(bar, 2 * S::KT_BYTES);
        tma_load_3d(kk_s + off, &mapKk, 0, kr, (kvh * SPLIT + crank) * ATOMS, bar);
        tma_load_3d(vk_s + off, &mapVk, 0, kr, (kvh * SPLIT + crank) * ATOMS, bar);
      };
      auto load_m = [&](int it) {   // [keys, hd] copy of K for the gradient product
        const int kr = row0 + (kb_lo + it) * NK;
        mbar_expect_tx(km_full, S::KT_BYTES);
        tma_load_3d(km_s, &mapKm, 0, kr, (kvh * SPLIT + crank) * ATOMS, km_full);
      };
      mbar_expect_tx(q_full, 2 * S::Q_BYTES);
      tma_load_3d(q_s, &mapQ, 0, row0 + q0, (h * SPLIT + crank) * ATOMS, q_full);
      tma_load_3d(g_s, &mapG, 0, row0 + q0, (h * SPLIT + crank) * ATOMS, q_full);
      load_k(0);
      load_m(0);
      if (KBUF == 2 && iters > 1) load_k(1);
      w.wait(s_full0, 0, 33);                     // same order of waits as in the dK/dV kernel
      if (KBUF < iters) load_k(KBUF);
      for (int i = 0; i < iters; i++) {
        if (i + 1 + KBUF < iters) {
          w.wait(s_bar(i + 1), s_par(i + 1), 33);
          load_k(i + 1 + KBUF);
        }
        w.wait(acc_done, i & 1, 35);
        if (i + 1 < iters) load_m(i + 1);
      }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_tf32(false, false, ROWS, NK);
      constexpr uint32_t idesc_g = idesc_tf32(false, true, ROWS, HD);
      const uint64_t d_q = desc_kmajor(q_s), d_g = desc_kmajor(g_s), d_kk = desc_kmajor(kk_s), d_vk = desc_kmajor(vk_s),
                     d_km = smem_desc(km_s, NK * 128, 512, 1);
      auto mma_s = [&](int it) {
        const uint32_t tm_s = tmem + sbuf(it), tm_dp = tm_s + NK;
        const uint32_t boff = (KBUF == 2 && (it & 1)) ? S::KT_BYTES : 0;
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            umma_tf32(tm_s, desc_off(d_q, a * (ROWS * 128) + j * 32), desc_off(d_kk, boff + a * (NK * 128) + j * 32), idesc_s,
                      (a > 0 || j > 0) ? 1u : 0u);
#pragma unroll
        for (int a = 0; a < ATOMS; a++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            umma_tf32(tm_dp, desc_off(d_g, a * (ROWS * 128) + j * 32), desc_off(d_vk, boff + a * (NK * 128) + j * 32), idesc_s,
                      (a > 0 || j > 0) ? 1u : 0u);
        umma_commit(s_bar(it));
      };
      w.wait(q_full, 0, 31);
      w.wait(kk_full0, 0, 32);
      tc_fence_after();
      mma_s(0);
      for (int i = 0; i < iters; i++) {
        if (!SB && i + 1 < iters) {               // next block's scores, under this block's element math
          w.wait(kk_bar(i + 1), kk_par(i + 1), 32);
          tc_fence_after();
          mma_s(i + 1);
        }
        w.wait(km_full, i & 1, 34);
        w.wait(p_bar(i), s_par(i), 34);
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < NK / 8; j++)   // dS is read where the math warps wrote it: over S, in tensor memory
          umma_tf32_ts(tm_dq, tmem + sbuf(i) + j * 8, desc_off(d_km, j * 1024), idesc_g, (i > 0 || j > 0) ? 1u : 0u);
        umma_commit(acc_done);
        if (SB && i + 1 < iters) {                // one score buffer: the next scores follow the product that read dS
          w.wait(kk_bar(i + 1), kk_par(i + 1), 32);
          tc_fence_after();
          mma_s(i + 1);
        }
      }
      umma_commit(all_done);   // the end of the accumulation, for the math warps (they do not follow acc_done)
      mbar_wait(all_done, 0);  // and for this thread, whatever happened before: no MMA in flight when TMEM is freed
    }
  } else {
    const int qd = warp & 3, half = warp >> 2;
    const int r = qd * 32 + lane;
    const int tq = q0 + r;
    const bool valid = tq < T;
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    const float L = valid ? lse[(size_t)h * rows + row0 + tq] : 0.f;
    const float Dr = valid ? Ds[(size_t)h * rows + row0 + tq] : 0.f;
    const int lo = (window > 0) ? tq - window + 1 : 0;
    for (int i = 0; i < iters; i++) {
      const int kpos0 = (kb_lo + i) * NK + half * NH;
      w.wait(s_bar(i), s_par(i), 36);
      tc_fence_after();
      float s[NH], dp[NH];
      const uint32_t tm_s = tmem + sbuf(i) + half * NH + lane_base;
      tmem_ld_issue<NH>(tm_s, s);
      tmem_ld_issue<NH>(tm_s + NK, dp);
      tmem_wait_ld();
      if constexpr (SPLIT == 2) xs.add<NH, NH>(w, i, (int)threadIdx.x, s, dp, 37);   // + the other half of the head
      const bool interior = (kpos0 + NH - 1 <= q0) && (q0 + ROWS - 1 < T) && (window == 0 || kpos0 >= q0 + ROWS - window);
      if (interior) {
#pragma unroll
        for (int c = 0; c < NH; c++) {
          const float p = ex2(fmaf(s[c], scale2, -L));
          s[c] = p * fmaf(dp[c], dp_scale, -Dr);
        }
      } else {
#pragma unroll
        for (int c = 0; c < NH; c++) {
          const int kg = kpos0 + c;
          const bool keep = valid && kg <= tq && kg >= lo;
          float d = 0.f;
          if (keep) {
            const float p = ex2(fmaf(s[c], scale2, -L));
            d = p * fmaf(dp[c], dp_scale, -Dr);
          }
          s[c] = d;
        }
      }
      tmem_st_issue<NH>(tm_s, s);               // dS takes the place of S
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_bar(i));
    }
    RopeRow<HD >= 64 ? HH : 32> rr;
    const bool roped = SPLIT == 1 && HD >= 64 && rope != nullptr;
    if (roped) rr.fetch(rope + (size_t)(valid ? tq : 0) * HH, half);
    w.wait(all_done, 0, 38);
    tc_fence_after();
    if (roped) {
      if constexpr (SPLIT == 1 && HD >= 64)
        rr.store(tm_dq + lane_base, gq + (size_t)(row0 + (valid ? tq : 0)) * Hq * HDF + (size_t)h * HDF, half, accum_q, !w.dead && valid, TRUNC_COMP);
    } else {   // warp-uniform TMEM load, per-row store
      float t[HH];
      tmem_ld<HH>(tm_dq + half * HH + lane_base, t);
      if (!w.dead && valid) {
        float* dst = gq + (size_t)(row0 + tq) * Hq * HDF + (size_t)h * HDF + crank * HD + half * HH;
#pragma unroll
        for (int d = 0; d < HH; d += 4) {
          float4 o = accum_q ? *reinterpret_cast<float4*>(dst + d) : make_float4(0, 0, 0, 0);
          o.x += t[d] * TRUNC_COMP; o.y += t[d + 1] * TRUNC_COMP; o.z += t[d + 2] * TRUNC_COMP; o.w += t[d + 3] * TRUNC_COMP;
          *reinterpret_cast<float4*>(dst + d) = o;
        }
      }
    }
  }
  tc_fence_before();
  if (SPLIT == 2) cluster_sync_all(); else __syncthreads();   // neither CTA of a pair leaves while the other may still write to it
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, S::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template <typename K>
gt_status set_smem(gt_ctx* ctx, K kern, int bytes, bool* done) {
  if (!done[ctx->device]) {
    GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done[ctx->device] = true;
  }
  return GT_OK;
}

// <<<grid, threads, smem, stream>>> with the grid's x axis grouped into clusters of `split` CTAs
template <typename... KA, typename... A>
cudaError_t launch_split(void (*kern)(KA...), dim3 grid, int threads, int smem, cudaStream_t stream, int split, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = split;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = split > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KA>(args)...);
}

template <int HD, int SPLIT>
gt_status launch_fwd(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int window, const float* q, const float* k, const float* v,
                     float* out, float* lse, int* flag) {
  CUtensorMap mq, mk, mv;
  const uint64_t qw = (uint64_t)Hq * HD * SPLIT, kw = (uint64_t)Hkv * HD * SPLIT;
  if (!make_map_atoms(&mq, q, qw, rows, qw, ROWS, HD / 32, true) || !make_map_atoms(&mk, k, kw, rows, kw, BKV, HD / 32, true) ||
      !make_map_atoms(&mv, v, kw, rows, kw, BKV, HD / 32, false))
    return gt_fail(ctx, GT_ERR_CUDA, "attention: tensor map encoding failed");
  auto kern = attn_fwd_tc_kernel<HD, SPLIT>;
  using SM = FwdSmem<HD, SPLIT>;
  static bool done[64] = {};
  gt_status st = set_smem(ctx, kern, SM::TOTAL, done);
  if (st) return st;
  // the S product's truncation bias is folded into the score scale
  const float scale2 = 1.4426950408889634f / sqrtf((float)(HD * SPLIT)) * TRUNC_COMP;
  dim3 grid(Hq * (rows / T) * SPLIT, gt_cdiv(T, ROWS), 1);
  if (SPLIT == 1) kern<<<grid, FWD_THREADS, SM::TOTAL, ctx->stream>>>(mq, mk, mv, out, lse, rows, T, Hq, Hkv, window, scale2, flag);
  else GT_CUDA(ctx, launch_split(kern, grid, FWD_THREADS, SM::TOTAL, ctx->stream, SPLIT, mq, mk, mv, out, lse, rows, T, Hq, Hkv, window, scale2, flag));
  GT_LAUNCHED(ctx, "attn_fwd_tc_kernel");
  return GT_OK;
}

// The order in which the tiles of the dK/dV kernel are handed out. A tile's work is its number of (query head, query
// block) iterations, 96 down to 6 at the benchmark shape, and the hardware gives the next tile in index order to whichever
// SM falls free: with the tiles sorted heaviest first that is longest-processing-time-first scheduling, which at 384
// tiles on 148 SMs ends 9 % above the mean load. Here the tiles are first packed into the SMs (first fit decreasing
// under the smallest capacity that fits, found by bisection) and then listed by the time at which the packing starts
// them; handing them out in that order reproduces the packing to within timing noise and ends 3 % above the mean.
// Built once per shape on the host (not during a recording) and kept on the device.
gt_status attn_dkv_order(gt_ctx* ctx, int nkb, int ntx, int group, int T, int NQ, int window, const int** out) {
  std::vector<int> key = {nkb, ntx, group, T, NQ, window, ctx->sm_count};
  auto it = ctx->attn_orders.find(key);
  if (it == ctx->attn_orders.end()) {
    if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "attention backward: the launch order of this shape is built on first use; run the step once eagerly before recording");
    const int n = nkb * ntx, workers = ctx->sm_count;
    std::vector<int> size(n), idx(n);
    double total = 0.0;
    int largest = 0;
    for (int kb = 0; kb < nkb; kb++) {
      const int k0 = kb * ROWS, k_last = min(k0 + ROWS - 1, T - 1);
      const int q_max = window > 0 ? min(T - 1, k_last + window - 1) : T - 1;
      const int w = (q_max / NQ - k0 / NQ + 1) * group + 3;       // iterations, plus about three for the tile's own prologue and epilogue
      for (int x = 0; x < ntx; x++) { size[kb * ntx + x] = w; idx[kb * ntx + x] = kb * ntx + x; }
      total += (double)w * ntx;
      largest = max(largest, w);
    }
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return size[a] > size[b]; });
    std::vector<int> bin_of(n), start(n);
    auto pack = [&](double cap) {
      std::vector<double> load(workers, 0.0);
      for (int j : idx) {
        int b = 0;
        while (b < workers && load[b] + size[j] > cap) b++;
        if (b == workers) return false;
        bin_of[j] = b; start[j] = (int)load[b];
        load[b] += size[j];
      }
      return true;
    };
    double lo = std::max((double)largest, total / workers), hi = 2.0 * lo;
    for (int r = 0; r < 24; r++) {
      const double mid = 0.5 * (lo + hi);
      if (pack(mid)) hi = mid; else lo = mid;
    }
    pack(hi);
    std::vector<int> order(idx);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return start[a] != start[b] ? start[a] < start[b] : size[a] > size[b]; });
    int* dev = nullptr;
    GT_CUDA(ctx, cudaMalloc(&dev, sizeof(int) * n));
    GT_CUDA(ctx, cudaMemcpy(dev, order.data(), sizeof(int) * n, cudaMemcpyHostToDevice));
    ctx->state_bytes += sizeof(int) * n;
    it = ctx->attn_orders.emplace(key, dev).first;
  }
  *out = it->second;
  return GT_OK;
}

template <int HD, int NQ, int NK, int DKV_KBUF, int DKV_MBUF, int DQ_KBUF, bool DQ_SB, int SPLIT>
gt_status launch_bwd(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int window, const float* q, const float* k, const float* v,
                     const float* out, const float* lse, const float* go, float* gq, int accum_q, float* gk, int accum_k, float* gv,
                     int accum_v, const float2* rope, int* flag) {
  float* D = nullptr;
  gt_status st = gt_scratch(ctx, sizeof(float) * (size_t)rows * Hq, &D);
  if (st) return st;
  constexpr int HDF = HD * SPLIT;
  const float scale = 1.f / sqrtf((float)HDF);
  const long nitems = (long)rows * Hq;
  attn_bwd_d_tc_kernel<HDF><<<(unsigned)gt_cdiv(nitems * (HDF / 4 < 32 ? HDF / 4 : 32), 256l), 256, 0, ctx->stream>>>(nitems, scale, go, out, D, rows, Hq);
  GT_LAUNCHED(ctx, "attn_bwd_d_tc_kernel");
  const float scale2 = 1.4426950408889634f * scale * TRUNC_COMP;
  const float dp_scale = scale * TRUNC_COMP;
  const uint64_t qw = (uint64_t)Hq * HDF, kw = (uint64_t)Hkv * HDF;
  const int nseq = rows / T;
  if (gk || gv) {
    CUtensorMap mK, mV, mQk, mQm, mGk, mGm;
    if (!make_map_atoms(&mK, k, kw, rows, kw, ROWS, HD / 32, true) || !make_map_atoms(&mV, v, kw, rows, kw, ROWS, HD / 32, true) ||
        !make_map_atoms(&mQk, q, qw, rows, qw, NQ, HD / 32, true) || !make_map_atoms(&mQm, q, qw, rows, qw, NQ, HD / 32, false) ||
        !make_map_atoms(&mGk, go, qw, rows, qw, NQ, HD / 32, true) || !make_map_atoms(&mGm, go, qw, rows, qw, NQ, HD / 32, false))
      return gt_fail(ctx, GT_ERR_CUDA, "attention backward: tensor map encoding failed");
    constexpr int KBUF = DKV_KBUF, MBUF = DKV_MBUF;
    auto kern = attn_bwd_dkv_tc_kernel<HD, NQ, KBUF, MBUF, SPLIT>;
    using SM = DkvSmem<HD, NQ, KBUF, MBUF, SPLIT>;
    static bool done[64] = {};
    st = set_smem(ctx, kern, SM::TOTAL, done);
    if (st) return st;
    dim3 grid(Hkv * nseq * SPLIT, gt_cdiv(T, ROWS), 1);
    const int* order = nullptr;
    if (SPLIT == 1 && (int)(grid.x * grid.y) > ctx->sm_count && !getenv("GT_ATTN_INDEX_ORDER")) {   // (the variable keeps index order, for comparison)
      st = attn_dkv_order(ctx, (int)grid.y, (int)grid.x, Hq / Hkv, T, NQ, window, &order);
      if (st) return st;
    }
    if (SPLIT == 1)
      kern<<<grid, THREADS, SM::TOTAL, ctx->stream>>>(mK, mV, mQk, mQm, mGk, mGm, lse, D, gk, accum_k, gv, accum_v, rows, T, Hq, Hkv, window, scale2,
                                                      dp_scale, rope, order, flag);
    else
      GT_CUDA(ctx, launch_split(kern, grid, THREADS, SM::TOTAL, ctx->stream, SPLIT, mK, mV, mQk, mQm, mGk, mGm, lse, D, gk, accum_k, gv, accum_v,
                                rows, T, Hq, Hkv, window, scale2, dp_scale, rope, order, flag));
    GT_LAUNCHED(ctx, "attn_bwd_dkv_tc_kernel");
  }
  if (gq) {
    CUtensorMap mQ, mG, mKk, mVk, mKm;
    if (!make_map_atoms(&mQ, q, qw, rows, qw, ROWS, HD / 32, true) || !make_map_atoms(&mG, go, qw, rows, qw, ROWS, HD / 32, true) ||
        !make_map_atoms(&mKk, k, kw, rows, kw, NK, HD / 32, true) || !make_map_atoms(&mVk, v, kw, rows, kw, NK, HD / 32, true) ||
        !make_map_atoms(&mKm, k, kw, rows, kw, NK, HD / 32, false))
      return gt_fail(ctx, GT_ERR_CUDA, "attention backward: tensor map encoding failed");
    auto kern = attn_bwd_dq_tc_kernel<HD, NK, DQ_KBUF, DQ_SB, SPLIT>;
    using SM = DqSmem<HD, NK, DQ_KBUF, DQ_SB, SPLIT>;
    static bool done[64] = {};
    st = set_smem(ctx, kern, SM::TOTAL, done);
    if (st) return st;
    dim3 grid(Hq * nseq * SPLIT, gt_cdiv(T, ROWS), 1);
    if (SPLIT == 1)
      kern<<<grid, THREADS, SM::TOTAL, ctx->stream>>>(mQ, mG, mKk, mVk, mKm, lse, D, gq, accum_q, rows, T, Hq, Hkv, window, scale2, dp_scale, rope, flag);
    else
      GT_CUDA(ctx, launch_split(kern, grid, THREADS, SM::TOTAL, ctx->stream, SPLIT, mQ, mG, mKk, mVk, mKm, lse, D, gq, accum_q, rows, T, Hq, Hkv,
                                window, scale2, dp_scale, rope, flag));
    GT_LAUNCHED(ctx, "attn_bwd_dq_tc_kernel");
  }
  return GT_OK;
}

bool tc_shape_ok(int T, int hd) { return (hd == 32 || hd == 64 || hd == 128 || hd == 256) && T >= 64; }

}  // namespace

gt_status gt_attention_fwd_tc(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q, const float* k,
                              const float* v, float* out, float* lse, bool* handled) {
  *handled = false;
  if (!tc_shape_ok(T, hd)) return GT_OK;   // other head sizes and tiny sequences stay on the f32 kernels
  if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)out)) & 15) return GT_OK;
  int* flag = device_flag(ctx);
  if (!flag) return GT_OK;
  gt_status s;
  if (hd == 32) s = launch_fwd<32, 1>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);
  else if (hd == 64) s = launch_fwd<64, 1>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);
  else if (hd == 128) s = launch_fwd<128, 1>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);
  else s = launch_fwd<128, 2>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, flag);   // 256: pairs of CTAs, half a head each
  if (s) return s;
  *handled = true;
  return GT_OK;
}

gt_status gt_attention_bwd_tc(gt_ctx* ctx, int rows, int T, int Hq, int Hkv, int hd, int window, const float* q, const float* k,
                              const float* v, const float* out, const float* lse, const float* go, float* gq, int accum_q, float* gk,
                              int accum_k, float* gv, int accum_v, const float2* rope, bool* handled) {
  *handled = false;
  if (!tc_shape_ok(T, hd)) return GT_OK;
  if (rope && hd != 64 && hd != 128) return GT_OK;   // (at 256 a CTA of a pair holds half a head: a rotation's pairs straddle the two)
  if ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)out) | ((uintptr_t)go) | ((uintptr_t)gq) | ((uintptr_t)gk) | ((uintptr_t)gv)) & 15)
    return GT_OK;
  int* flag = device_flag(ctx);
  if (!flag) return GT_OK;
  gt_status s;
  if (hd == 32) s = launch_bwd<32, 64, 64, 2, 2, 1, true, 1>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, rope, flag);
  else if (hd == 64) s = launch_bwd<64, 64, 64, 2, 2, 1, true, 1>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, rope, flag);
  else if (hd == 128) s = launch_bwd<128, 32, 32, 2, 1, 2, false, 1>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, rope, flag);
  else s = launch_bwd<128, 32, 32, 1, 1, 1, false, 2>(ctx, rows, T, Hq, Hkv, window, q, k, v, out, lse, go, gq, accum_q, gk, accum_k, gv, accum_v, rope, flag);
  if (s) return s;
  *handled = true;
  return GT_OK;
}
