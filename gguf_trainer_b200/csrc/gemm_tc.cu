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

constexpr int BM1 = 128;         // UMMA M (cta_group::1): accumulator row i lives in TMEM lane i
constexpr int BK = 32;           // f32 elements per stage along K: 128 bytes = one swizzle row
constexpr int UMMA_K = 8;        // tf32: 32 bytes of K per instruction

// Tile shapes. MT = 1: 128 x BN output tile, two TMEM accumulators, so the epilogue of a tile runs under the
// main loop of the next. MT = 2: 256 x BN, two 128-row halves that share every B tile and fill the tensor memory
// (no second buffer: the epilogue is exposed). With 4-byte operands the main loop is bound by shared-memory
// bandwidth, not by the tensor pipe: every stage is written once by TMA and read by the MMAs once per 128-row
// half, at 128 B/clk. A 256-row tile moves fewer bytes per flop (the B tile is fetched once for both halves), which
// pays when the tile count still fills the SMs evenly; the host picks per product.
template <int BN, int MT>
struct Smem {
  static constexpr int BM = BM1 * MT;
  static constexpr int A_BYTES = BM * BK * 4;   // 16 / 32 KB
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = MT == 2 ? 3 : (BN <= 128 ? 5 : 4);
  static constexpr int EPI_WARPS = 4 * MT;
  static constexpr int EPI_TILES = MT == 2 ? 1 : 2;   // 32x32 f32 staging tiles per epilogue warp for the TMA store
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_TILES * 4096;
  static constexpr int TOTAL = STAGES * STAGE + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr uint32_t TMEM_COLS = 2 * BN <= 256 ? 256 : 512;   // two accumulators (MT = 1) or two halves (MT = 2)
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;   // warp 0: TMA, warp 1: MMA + TMEM owner, then the epilogue warps
  static_assert(TOTAL <= 232448, "shared memory");
};

// Persistent: each CTA walks output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (n fastest, then m, then the
// split-K slice), so CTAs running at the same time share their A row-blocks in L2.
// A_K: A is K-major in memory (NT, NN); else MN-major ([K, M], TN). B_K: B is K-major (NT); else [K, N] (NN, TN).
// Operands of one launch: up to MAX_PARTS products A_p.B_p of the same layout, K_p deep, summed into the same output
// tiles. kb_end[p] is the number of K blocks of parts 0..p; only the TMA producer looks at it.
constexpr int MAX_PARTS = 8;
struct PartMaps {
  CUtensorMap a[MAX_PARTS], b[MAX_PARTS];
  int kb_end[MAX_PARTS];
  int nparts;
  // Grouped form (ngroups > 1, one part): group g is its own product A_g.B_g -> C_g of gM[g] x gN[g], all of one
  // layout and one K; its tiles are units [unit_end[g-1], unit_end[g]) of the launch (n fastest, then m, then the
  // split-K slice). c[g] is its output map (c[0] the only one when ngroups == 1).
  CUtensorMap c[MAX_PARTS];
  int ngroups;
  int gM[MAX_PARTS], gN[MAX_PARTS], g_accum[MAX_PARTS], unit_end[MAX_PARTS];
  // Rotary form (EPI_ROPE): the outputs of the groups with g_rope[g] set are rotated as they are written (see the kernel).
  int g_rope[MAX_PARTS];
  const float2* rope_tab;   // [rope_period][32] (cos, sin) of the 32 pairs of a 64-wide head
  int rope_period;          // positions per sequence: row r is position r % rope_period
};
constexpr int EPI_ROPE = 8;   // a value of the kernel's GLU argument that is neither activation

// GLU != 0 (GT_EW_SILU or GT_EW_GELU; NT layout, BN = 192 only): the gated unit of the FFN in the projection that
// feeds it. B is two weight matrices: the tile's first 96 columns are rows [n0/2, n0/2 + 96) of b[0] (gate), the other 96
// the same rows of b[1] (up). The epilogue writes the gate and up projections (backward needs them) through c[0] and
// c[1] and act(gate) * up through c[2], so the separate pass that read both and wrote the product is not launched.
// N_ is 2 x the FFN width.
// GLU == EPI_ROPE (grouped NT launches, BN = 192, heads 64 wide): the rotary embedding that follows the q and k
// projections (src/arch/llama.ts:195-199 records `rope(linear(x, Wq))`) applied to the accumulator on its way out. A
// 192-column tile is three whole heads; the thread that owns a row loads the two 32-column halves of a head, rotates
// pair (j, j + 32) by the angle of (row's position, j) from the table, and both halves go out as they would have.
// The unrotated projection is never written.
template <bool A_K, bool B_K, int BN, int MT, int GLU = 0>
__global__ void __launch_bounds__(Smem<BN, MT>::THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ PartMaps maps, float* __restrict__ C, int M_, int N_,
                 int accum_, int ksplit, int use_tma_store, int batch, float out_scale, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = Smem<BN, MT>;
  const int M = M_, N = N_;   // (of the single product; a grouped launch takes each group's from `maps`)
  constexpr int STAGES = S::STAGES, BM = S::BM;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi = base + STAGES * S::STAGE;    // staging tiles of the epilogue warps
  const uint32_t bars = epi + S::EPI_BYTES;         // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  constexpr bool IS_GLU = GLU == GT_EW_SILU || GLU == GT_EW_GELU;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
  const int per_mat = tiles_n * tiles_m * ksplit;
  const int ngroups = maps.ngroups;
  const int ntiles = ngroups > 1 ? maps.unit_end[ngroups - 1] : per_mat * batch;   // the matrices of a batch are just more tiles
  // where tile t lies: batch matrix (or group), first column, first row (of the 256-row tile when MT = 2), K slice
  struct Where { int bi, g, n0, m0, z; };
  auto where = [&](int t) {
    Where w;
    if (ngroups > 1) {
      int g = 0;
      while (t >= maps.unit_end[g]) g++;
      const int tt = t - (g ? maps.unit_end[g - 1] : 0);
      const int tn = (maps.gN[g] + BN - 1) / BN, tmn = tn * ((maps.gM[g] + BM - 1) / BM);
      const int rem = tt % tmn;
      w.bi = 0; w.g = g; w.z = tt / tmn; w.n0 = (rem % tn) * BN; w.m0 = (rem / tn) * BM;
    } else {
      const int tt = t % per_mat;
      w.bi = t / per_mat; w.g = 0; w.n0 = (tt % tiles_n) * BN; w.m0 = ((tt / tiles_n) % tiles_m) * BM; w.z = tt / (tiles_n * tiles_m);
    }
    return w;
  };
  // Further products of the same layout are accumulated into the same tiles: their K blocks simply follow those of
  // the first in the main loop, read through their own tensor maps.
  const int kblocks = maps.kb_end[maps.nparts - 1];
  const int per = (kblocks + ksplit - 1) / ksplit;   // K blocks per split-K slice
  // TMEM slot of a 128-row accumulator and the parity of its hand-over barriers: with MT = 1 the tiles alternate
  // between two slots, with MT = 2 slot h holds half h of every tile.
  auto slot_of = [&](uint32_t tl, int h) { return MT == 2 ? h : (int)(tl & 1); };
  auto par_of = [&](uint32_t tl) { return MT == 2 ? (tl & 1) : ((tl >> 1) & 1); };

  if (threadIdx.x == 0) {
    for (int p = 0; p < maps.nparts; p++) { tma_prefetch_map(&maps.a[p]); tma_prefetch_map(&maps.b[p]); }
    for (int g = 1; g < ngroups; g++) { tma_prefetch_map(&maps.a[g]); tma_prefetch_map(&maps.b[g]); }
    if (use_tma_store)
      for (int g = 0; g < ngroups; g++) tma_prefetch_map(&maps.c[g]);
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
        const Where wh = where(t);
        const int bi = wh.bi, n0 = wh.n0, m0 = wh.m0, z = wh.z;
        const int kb0 = z * per, kb1 = min(kblocks, kb0 + per);
        int part = wh.g;        // (a grouped launch has one K range per group: the group's operands)
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, 1);
          const uint32_t a_dst = base + s * S::STAGE, b_dst = a_dst + S::A_BYTES;
          if (ngroups == 1) while (kb >= maps.kb_end[part]) part++;
          const CUtensorMap* pa = &maps.a[part];
          const CUtensorMap* pb = &maps.b[part];
          const int k0 = (ngroups == 1 ? kb - (part ? maps.kb_end[part - 1] : 0) : kb) * BK;
          mbar_expect_tx(full_bar(s), S::STAGE);
          if (A_K) tma_load_3d(a_dst, pa, k0, m0, bi, full_bar(s));
          else
            for (int c = 0; c < BM / 32; c++) tma_load_3d(a_dst + c * 4096, pa, m0 + 32 * c, k0, bi, full_bar(s));
          if (IS_GLU) {
            tma_load_3d(b_dst, &maps.b[0], k0, n0 >> 1, bi, full_bar(s));
            tma_load_3d(b_dst + (BN / 2) * 128, &maps.b[1], k0, n0 >> 1, bi, full_bar(s));
          } else if (B_K) tma_load_3d(b_dst, pb, k0, n0, bi, full_bar(s));
          else
            for (int c = 0; c < BN / 32; c++) tma_load_3d(b_dst + c * 4096, pb, n0 + 32 * c, k0, bi, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      constexpr uint32_t idesc = idesc_tf32(!A_K, !B_K, BM1, BN);
      const uint64_t a_desc0 = A_K ? desc_kmajor(base) : desc_mnmajor(base);
      const uint64_t b_desc0 = B_K ? desc_kmajor(base + S::A_BYTES) : desc_mnmajor(base + S::A_BYTES);
      constexpr uint32_t A_STEP = A_K ? 32 : 1024, B_STEP = B_K ? 32 : 1024;   // bytes per K = 8 step
      uint32_t it = 0, tl = 0;
      for (int t = blockIdx.x; t < ntiles; t += gridDim.x, tl++) {
        const int z = where(t).z;
        const int kb0 = z * per, kb1 = min(kblocks, kb0 + per);
        const uint32_t par = par_of(tl) ^ 1;
        wait(acc_empty(slot_of(tl, 0)), par, 4);   // the epilogue has drained this accumulator
        if (MT == 2 && kb0 >= kb1) wait(acc_empty(1), par, 4);
        tc_fence_after();
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          wait(full_bar(s), (it / STAGES) & 1, 2);
          tc_fence_after();
          const uint32_t soff = (uint32_t)(s * S::STAGE) >> 4;
#pragma unroll
          for (int h = 0; h < MT; h++) {
            if (h == 1 && kb == kb0) {             // the second half's accumulator is drained a little later
              wait(acc_empty(1), par, 4);
              tc_fence_after();
            }
            const uint32_t d_tmem = tmem + slot_of(tl, h) * BN;
#pragma unroll
            for (int j = 0; j < BK / UMMA_K; j++)
              umma_tf32(d_tmem, a_desc0 + soff + ((h * 16384 + j * A_STEP) >> 4), b_desc0 + soff + ((j * B_STEP) >> 4), idesc,
                        (kb > kb0 || j > 0) ? 1u : 0u);
            if (kb == kb1 - 1) umma_commit(acc_full(slot_of(tl, h)));   // this accumulator is complete
          }
          umma_commit(empty_bar(s));   // the stage is free once these MMAs have read it
        }
      }
    }
  } else {
    // ---- epilogue: warp w may touch TMEM lanes [32*(w%4), 32*(w%4)+32) ----
    const int q = warp & 3, ew = warp - 2, half = ew >> 2;
    const bool vec = (N & 3) == 0;
    uint32_t tl = 0, nst = 0;   // nst: TMA stores issued by this warp
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, tl++) {
      const Where wh = where(t);
      const int bi = wh.bi, n0 = wh.n0, m0 = wh.m0 + half * BM1, z = wh.z;
      const int M = ngroups > 1 ? maps.gM[wh.g] : M_, N = ngroups > 1 ? maps.gN[wh.g] : N_;
      const int accum = ngroups > 1 ? maps.g_accum[wh.g] : accum_;
      const CUtensorMap* mapC = &maps.c[wh.g];
      const int b = slot_of(tl, half);
      const bool have = z * per < kblocks;     // an empty split-K slice issues no MMA and contributes nothing
      const int row = m0 + q * 32 + lane;
      if (have) wait(acc_full(b), par_of(tl), 3);
      dead = __any_sync(0xffffffffu, dead);
      tc_fence_after();
      if (IS_GLU && have) {
        // gate | up halves of the accumulator: three outputs per 32-column block, each through its own tensor map
        auto put = [&](const float* v, const CUtensorMap* map, int col0) {
          const uint32_t tile = epi + (uint32_t)(ew * S::EPI_TILES + (nst % S::EPI_TILES)) * 4096u;
          if (nst >= S::EPI_TILES) tma_wait_read<S::EPI_TILES - 1>();
          __syncwarp();
          uint8_t* tp = smem_raw + (tile - smem_u32(smem_raw)) + lane * 128;
#pragma unroll
          for (int c4 = 0; c4 < 8; c4++)
            *reinterpret_cast<float4*>(tp + ((c4 ^ (lane & 7)) * 16)) = make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0 && !dead && m0 + q * 32 < M) tma_store_3d(map, tile, col0, m0 + q * 32, bi);
          if (lane == 0) tma_commit_group();
          nst++;
        };
#pragma unroll 1
        for (int c = 0; c < BN / 64; c++) {
          const int col0 = (n0 >> 1) + c * 32;
          if (col0 >= (N >> 1)) break;   // uniform across the warp
          float vg[32], vu[32];
          const uint32_t ta = tmem + b * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32);
          tmem_ld32_issue(ta, vg);
          tmem_ld32_issue(ta + BN / 2, vu);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j++) { vg[j] *= out_scale; vu[j] *= out_scale; }
          put(vg, &maps.c[0], col0);
          put(vu, &maps.c[1], col0);
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const float a = vg[j];
            float act;
            if (GLU == GT_EW_SILU) act = a / (1.f + __expf(-a));
            else act = 0.5f * a * (1.f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
            vg[j] = act * vu[j];
          }
          put(vg, &maps.c[2], col0);
        }
      } else if (GLU == EPI_ROPE && have && maps.g_rope[wh.g]) {
        auto put = [&](const float* v, int col0) {
          const uint32_t tile = epi + (uint32_t)(ew * S::EPI_TILES + (nst % S::EPI_TILES)) * 4096u;
          if (nst >= S::EPI_TILES) tma_wait_read<S::EPI_TILES - 1>();
          __syncwarp();
          uint8_t* tp = smem_raw + (tile - smem_u32(smem_raw)) + lane * 128;
#pragma unroll
          for (int c4 = 0; c4 < 8; c4++)
            *reinterpret_cast<float4*>(tp + ((c4 ^ (lane & 7)) * 16)) = make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
          fence_async_smem();
          __syncwarp();
          if (lane == 0 && !dead && m0 + q * 32 < M) {
            if (ksplit > 1 || accum) tma_reduce_add_3d(mapC, tile, col0, m0 + q * 32, bi);   // (a rotation is linear)
            else tma_store_3d(mapC, tile, col0, m0 + q * 32, bi);
          }
          if (lane == 0) tma_commit_group();
          nst++;
        };
        // (cos, sin) of this row's position, pairs 0..31; rows past M are clipped by the store and read row M - 1's
        const float4* tab4 = reinterpret_cast<const float4*>(maps.rope_tab + (size_t)((row < M ? row : M - 1) % maps.rope_period) * 32);
#pragma unroll 1
        for (int c = 0; c < BN / 64; c++) {
          const int col0 = n0 + c * 64;
          if (col0 >= N) break;   // uniform across the warp
          float v0[32], v1[32];
          const uint32_t ta = tmem + b * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 64);
          tmem_ld32_issue(ta, v0);
          tmem_ld32_issue(ta + 32, v1);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float4 cs = __ldg(tab4 + (j >> 1));   // cos, sin of pair j; cos, sin of pair j + 1
            const float a0 = v0[j] * out_scale, a1 = v1[j] * out_scale, b0 = v0[j + 1] * out_scale, b1 = v1[j + 1] * out_scale;
            v0[j] = a0 * cs.x - a1 * cs.y;
            v1[j] = a0 * cs.y + a1 * cs.x;
            v0[j + 1] = b0 * cs.z - b1 * cs.w;
            v1[j + 1] = b0 * cs.w + b1 * cs.z;
          }
          put(v0, col0);
          put(v1, col0 + 32);
        }
      } else if (have) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;   // uniform across the warp
          float v[32];
          tmem_ld32(tmem + b * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] *= out_scale;   // the caller's factor times the truncation compensation
          if (use_tma_store) {
            // Stage the warp's 32x32 block in shared memory (128-byte rows, 16-byte chunks XOR (row mod 8), the layout
            // the store's tensor map expects) and let TMA write it: whole 128-byte rows, clipped at M and N, as a
            // plain store or, when accumulating or combining split-K slices, as an f32 reduce-add performed in L2.
            const uint32_t tile = epi + (uint32_t)(ew * S::EPI_TILES + (nst % S::EPI_TILES)) * 4096u;
            if (nst >= S::EPI_TILES) tma_wait_read<S::EPI_TILES - 1>();   // the tile's previous contents have been read out
            __syncwarp();
            uint8_t* tp = smem_raw + (tile - smem_u32(smem_raw)) + lane * 128;
#pragma unroll
            for (int c4 = 0; c4 < 8; c4++)
              *reinterpret_cast<float4*>(tp + ((c4 ^ (lane & 7)) * 16)) = make_float4(v[4 * c4], v[4 * c4 + 1], v[4 * c4 + 2], v[4 * c4 + 3]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && !dead && m0 + q * 32 < M) {
              if (ksplit > 1 || accum) tma_reduce_add_3d(mapC, tile, col0, m0 + q * 32, bi);
              else tma_store_3d(mapC, tile, col0, m0 + q * 32, bi);
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
// The same product on CTA pairs (cta_group::2): a cluster of two CTAs on neighbouring SMs owns a 256 x BN output
// tile. Each CTA stages its 128 rows of A and HALF of the B tile (the pair's tensor cores read both halves), so a
// K block costs each SM 16 KB + BN/2 x 128 B of shared-memory writes and as many reads, against 16 KB + BN x 128 B
// for a CTA working alone: with 4-byte operands that traffic, not the tensor pipe, bounds the main loop. Each
// CTA holds its 128 rows of the accumulator, twice (the epilogue of a tile runs under the next tile's main loop).
// Roles per CTA as above; the MMAs are issued by the even CTA only. Barriers: the TMA copies of both CTAs count
// their bytes on the even CTA's `full`; `empty` and `acc_full` receive the MMA completions in both CTAs (multicast
// commit); the epilogue threads of both CTAs arrive on the even CTA's `acc_empty`.
// ---------------------------------------------------------------------------------------------
template <int BN>
struct SmemPair {
  static constexpr int BH = BN / 2;                 // rows of the B tile staged by each CTA
  static constexpr int A_BYTES = BM1 * BK * 4;      // 16 KB
  static constexpr int B_BYTES = BH * BK * 4;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = 4 * 2 * 4096;
  static constexpr int STAGES = (232448 - EPI_BYTES - 1024 - 256) / STAGE;   // 6 for BN = 256 and 192
  static constexpr int TOTAL = STAGES * STAGE + EPI_BYTES + 1024 + 256;
  static constexpr uint32_t TMEM_COLS = 2 * BN <= 256 ? 256 : 512;
  static constexpr int THREADS = 192;
  static_assert(BH % 32 == 0 && STAGES >= 3 && 8 * (2 * STAGES + 5) <= 256, "tile");
};

template <bool A_K, bool B_K, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SmemPair<BN>::THREADS, 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                      const __grid_constant__ CUtensorMap mapC, float* __restrict__ C, int M, int N, int K, int accum, int ksplit,
                      int use_tma_store, int batch, float out_scale, int* __restrict__ flag) {
  extern __shared__ uint8_t smem_raw[];
  using S = SmemPair<BN>;
  constexpr int STAGES = S::STAGES, BM = 2 * BM1;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi = base + STAGES * S::STAGE;
  const uint32_t bars = epi + S::EPI_BYTES;         // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_ctarank();          // 0: issues the MMAs; both stage operands and drain their rows
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
  const int per_mat = tiles_n * tiles_m * ksplit;
  const int ntiles = per_mat * batch;
  const int kblocks = (K + BK - 1) / BK;
  const int per = (kblocks + ksplit - 1) / ksplit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; b++) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 256); }   // 128 epilogue threads per CTA
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, S::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anything is signalled to them
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_ptr;
  bool dead = false;
  auto wait = [&](uint32_t bar, uint32_t parity, int code) {
    if (dead) return;
    if (!mbar_wait(bar, parity)) { dead = true; atomicExch(flag, code); }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer (both CTAs) ----
      uint32_t it = 0;
      for (int t = pair; t < ntiles; t += npairs) {
        const int bi = t / per_mat, tt = t % per_mat;
        const int n0 = (tt % tiles_n) * BN + rank * S::BH, m0 = ((tt / tiles_n) % tiles_m) * BM + rank * BM1, z = tt / (tiles_n * tiles_m);
        const int kb0 = z * per, kb1 = min(kblocks, kb0 + per);
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, 1);
          const uint32_t a_dst = base + s * S::STAGE, b_dst = a_dst + S::A_BYTES;
          const int k0 = kb * BK;
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * S::STAGE);   // both CTAs' stages
          if (A_K) tma_load_3d_pair(a_dst, &mapA, k0, m0, bi, full_bar(s));
          else
            for (int c = 0; c < BM1 / 32; c++) tma_load_3d_pair(a_dst + c * 4096, &mapA, m0 + 32 * c, k0, bi, full_bar(s));
          if (B_K) tma_load_3d_pair(b_dst, &mapB, k0, n0, bi, full_bar(s));
          else
            for (int c = 0; c < S::BH / 32; c++) tma_load_3d_pair(b_dst + c * 4096, &mapB, n0 + 32 * c, k0, bi, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer (even CTA) ----
      constexpr uint32_t idesc = idesc_tf32(!A_K, !B_K, BM, BN);
      const uint64_t a_desc0 = A_K ? desc_kmajor(base) : desc_mnmajor(base);
      const uint64_t b_desc0 = B_K ? desc_kmajor(base + S::A_BYTES) : desc_mnmajor(base + S::A_BYTES);
      constexpr uint32_t A_STEP = A_K ? 32 : 1024, B_STEP = B_K ? 32 : 1024;
      uint32_t it = 0, tl = 0;
      for (int t = pair; t < ntiles; t += npairs, tl++) {
        const int z = (t % per_mat) / (tiles_n * tiles_m);
        const int kb0 = z * per, kb1 = min(kblocks, kb0 + per);
        const int b = tl & 1;
        wait(acc_empty(b), ((tl >> 1) & 1) ^ 1, 4);   // both CTAs have drained this accumulator
        tc_fence_after();
        const uint32_t d_tmem = tmem + b * BN;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          wait(full_bar(s), (it / STAGES) & 1, 2);
          tc_fence_after();
          const uint32_t soff = (uint32_t)(s * S::STAGE) >> 4;
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; j++)
            umma_tf32_pair(d_tmem, a_desc0 + soff + ((j * A_STEP) >> 4), b_desc0 + soff + ((j * B_STEP) >> 4), idesc,
                           (kb > kb0 || j > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(s), 3);   // the stage is free in both CTAs once these MMAs have read it
        }
        if (kb1 > kb0) umma_commit_pair(acc_full(b), 3);
      }
    }
  } else {
    // ---- epilogue (both CTAs): this CTA's 128 rows ----
    const int q = warp & 3;
    uint32_t tl = 0, nst = 0;
    for (int t = pair; t < ntiles; t += npairs, tl++) {
      const int bi = t / per_mat, tt = t % per_mat;
      const int n0 = (tt % tiles_n) * BN, m0 = ((tt / tiles_n) % tiles_m) * BM + rank * BM1, z = tt / (tiles_n * tiles_m);
      const int b = tl & 1;
      const bool have = z * per < kblocks;
      const int row = m0 + q * 32 + lane;
      if (have) wait(acc_full(b), (tl >> 1) & 1, 3);
      dead = __any_sync(0xffffffffu, dead);
      tc_fence_after();
      if (have) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
          const int col0 = n0 + c * 32;
          if (col0 >= N) break;
          float v[32];
          tmem_ld32(tmem + b * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] *= out_scale;   // the caller's factor times the truncation compensation
          if (use_tma_store) {
            const uint32_t tile = epi + (uint32_t)(q * 2 + (nst & 1)) * 4096u;
            if (nst >= 2) tma_wait_read<1>();
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
      tc_fence_before();
      mbar_arrive_leader(acc_empty(b));
    }
    if (lane == 0) tma_wait_all<0>();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, S::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
int* g_flag[64] = {};

template <bool A_K, bool B_K, int BN, int MT, int GLU = 0>
gt_status launch(gt_ctx* ctx, const PartMaps& maps, long ntiles, int tma_store, float* c, int M, int N, int accum, int ksplit,
                 int batch, float out_scale) {
  auto kern = gemm_tf32_kernel<A_K, B_K, BN, MT, GLU>;
  using S = Smem<BN, MT>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device]) {
    GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    attr_set[ctx->device] = true;
  }
  dim3 grid((unsigned)min((long)(ctx->sm_count - ctx->sm_reserved), ntiles), 1, 1);
  kern<<<grid, S::THREADS, S::TOTAL, ctx->stream>>>(maps, c, M, N, accum, ksplit, tma_store, batch, out_scale, g_flag[ctx->device]);
  GT_LAUNCHED(ctx, "gemm_tf32_kernel");
  return GT_OK;
}

template <bool A_K, bool B_K, int BN>
gt_status launch_pair(gt_ctx* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int tma_store, float* c, int M, int N,
                      int K, int accum, int ksplit, int batch, int npairs, float out_scale) {
  auto kern = gemm_tf32_pair_kernel<A_K, B_K, BN>;
  using S = SmemPair<BN>;
  static bool attr_set[64] = {};
  if (!attr_set[ctx->device]) {
    GT_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    attr_set[ctx->device] = true;
  }
  const long ntiles = (long)gt_cdiv(N, BN) * gt_cdiv(M, 2 * BM1) * ksplit * batch;
  dim3 grid(2u * (unsigned)min((long)npairs, ntiles), 1, 1);
  kern<<<grid, S::THREADS, S::TOTAL, ctx->stream>>>(ma, mb, mc, c, M, N, K, accum, ksplit, tma_store, batch, out_scale, g_flag[ctx->device]);
  GT_LAUNCHED(ctx, "gemm_tf32_pair_kernel");
  return GT_OK;
}

template <int BN>
gt_status launch_pair_kind(gt_ctx* ctx, int kind, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int tma_store,
                           float* c, int M, int N, int K, int accum, int ksplit, int batch, int npairs, float out_scale) {
  if (kind == GT_GEMM_NT) return launch_pair<true, true, BN>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch, npairs, out_scale);
  if (kind == GT_GEMM_NN) return launch_pair<true, false, BN>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch, npairs, out_scale);
  return launch_pair<false, false, BN>(ctx, ma, mb, mc, tma_store, c, M, N, K, accum, ksplit, batch, npairs, out_scale);
}

// CTA pairs that can be resident at once (two neighbouring SMs each); 0 when the device cannot run the pair kernel.
int pair_capacity(gt_ctx* ctx) {
  static int cap[64];
  static bool known[64] = {};
  if (!known[ctx->device]) {
    auto kern = gemm_tf32_pair_kernel<true, true, 192>;
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)ctx->sm_count, 1, 1);
    cfg.blockDim = dim3(SmemPair<192>::THREADS, 1, 1);
    cfg.dynamicSmemBytes = SmemPair<192>::TOTAL;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemPair<192>::TOTAL) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cap[ctx->device] = n;
    known[ctx->device] = true;
    if (getenv("GT_GEMM_TILE")) fprintf(stderr, "[gguftrain] resident CTA pairs: %d\n", n);
  }
  return cap[ctx->device];
}

template <int BN, int MT>
gt_status launch_kind(gt_ctx* ctx, int kind, const PartMaps& maps, long ntiles, int tma_store, float* c, int M, int N, int accum,
                      int ksplit, int batch, float out_scale) {
  if (kind == GT_GEMM_NT) return launch<true, true, BN, MT>(ctx, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
  if (kind == GT_GEMM_NN) return launch<true, false, BN, MT>(ctx, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
  return launch<false, false, BN, MT>(ctx, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
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

// Self-test of the bounded wait every pipeline kernel relies on: one thread waits on an mbarrier that nothing will
// ever arrive on, with a caller-chosen limit instead of the kernels' 2 s, gives up when the limit has passed, raises
// the device flag like a pipeline kernel would (code 99) and returns. Nothing spins beyond the limit and the context
// stays usable; the next gt_sync reports the expiry.
__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, int* __restrict__ flag) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint64_t t0 = gtimer();
    bool arrived = mbar_try(bar, 0);
    while (!arrived && gtimer() - t0 <= limit_ns) arrived = mbar_try(bar, 0);
    if (!arrived) atomicExch(flag, 99);
  }
}

extern "C" gt_status gt_selftest_bounded_wait(gt_ctx* ctx, int32_t limit_us) {
  GT_REQUIRE(ctx, limit_us >= 1 && limit_us <= 1000000, "gt_selftest_bounded_wait: limit %d us (1..1000000)", limit_us);
  if (ctx->capturing) return gt_fail(ctx, GT_ERR_STATE, "gt_selftest_bounded_wait inside a graph capture");
  int* flag = device_flag(ctx);
  if (!flag) return gt_fail(ctx, GT_ERR_CUDA, "gt_selftest_bounded_wait: cannot allocate the device flag");
  bounded_wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>((unsigned long long)limit_us * 1000ull, flag);
  GT_LAUNCHED(ctx, "bounded_wait_selftest_kernel");
  return GT_OK;
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
// With nparts > 1 (batch 1 only): c (+)= sum_p op(a_p).op(b_p), every product of the same kind, K_p deep.
static gt_status gemm_tc_dispatch(gt_ctx* ctx, int kind, int accum, int M, int N, int nparts, const int* Ks, const float* const* as,
                                  const float* const* bs, float* c, int batch, float alpha, bool* handled) {
  *handled = false;
  if (batch < 1 || nparts < 1 || nparts > MAX_PARTS || (nparts > 1 && batch != 1)) return GT_OK;
  // Small or oddly aligned products stay on the f32 kernel: TMA needs 16-byte row pitches and bases.
  const bool a_k = kind != GT_GEMM_TN, b_k = kind == GT_GEMM_NT;
  if (M < 16 || N < 16 || Ks[0] < 16) return GT_OK;   // (rows of a tile past M or N are zero-filled by TMA and clipped on store)
  if (((uintptr_t)c) & 15) return GT_OK;
  int kblocks = 0;
  for (int p = 0; p < nparts; p++) {
    const int a_inner = a_k ? Ks[p] : M, b_inner = b_k ? Ks[p] : N;
    if (Ks[p] < 1 || (a_inner & 3) || (b_inner & 3) || ((((uintptr_t)as[p]) | ((uintptr_t)bs[p])) & 15)) return GT_OK;
    kblocks += gt_cdiv(Ks[p], BK);
  }
  if (ctx->device < 0 || ctx->device >= 64) return GT_OK;
  if (!device_flag(ctx)) return GT_OK;
  // Tile shape and split-K factor: the cheapest of the four shapes under a small cost model (cycles of the CTA with
  // the most work: waves x (K blocks x cycles per K block + epilogue)), calibrated on in-kernel cycle counts.
  struct Cfg { int mt, bn; };   // mt 1, 2: 128 / 256 rows on one CTA; mt 3: 256 rows on a CTA pair
  static const Cfg cfgs[6] = {{1, 192}, {1, 128}, {2, 256}, {2, 192}, {3, 192}, {3, 256}};
  const char* force = getenv("GT_GEMM_TILE");   // "mt,bn": forces one tile shape (read per call so tests can switch it)
  const char* ds = getenv("GT_GEMM_DEEP_SPLIT");   // "0": never cut a product that already fills the SMs along K (for comparison)
  const bool deep_split = !(ds && ds[0] == '0');
  const int npairs = max(0, pair_capacity(ctx) - (ctx->sm_reserved + 1) / 2);
  int best = 0, ksplit = 1;
  double best_cost = 1e30;
  int best_deep = 0, ks_deep = 1;      // the best choice that also cuts a product with enough tiles along K (see below)
  double cost_deep = 1e30;
  for (int i = 0; i < 6; i++) {
    const int mt = cfgs[i].mt, bn = cfgs[i].bn, bm = mt == 1 ? BM1 : 2 * BM1;
    if (mt == 3 && (npairs < 8 || nparts > 1)) continue;   // (the pair kernel takes one product)
    if (force) {
      int fm = 0, fb = 0;
      if (sscanf(force, "%d,%d", &fm, &fb) == 2 && (fm != mt || fb != bn)) continue;
    }
    const long workers = mt == 3 ? npairs : ctx->sm_count - ctx->sm_reserved;
    const long tiles = (long)gt_cdiv(N, bn) * gt_cdiv(M, bm) * batch;
    // split K when the output has few tiles and K is deep (dW: K = rows); partial sums meet in L2 with f32 adds
    int ks = 1;
    if (tiles < workers && kblocks >= 16) {
      ks = (int)min((long)(workers / tiles), (long)(kblocks / 8));
      if (ks < 1) ks = 1;
    }
    // One K block costs the slower of its MMAs (N/2 cycles each) and its shared-memory traffic at 128 B/clk: the stage
    // is written once by TMA and read once per 128-row half by the MMAs (measured: 0.9 of that bound). The epilogue
    // of a 256-row tile is exposed, that of a 128-row tile mostly hidden.
    // A CTA of a pair stages 128 rows of A and half of the B tile but still serves both halves of B to the pair's
    // tensor cores: measured 640 (BN 192) and 720 (BN 256) cycles per K block, little better per flop than one CTA
    // with a 256-row tile; what the pair adds is the second accumulator (hidden epilogue) and a deeper pipeline.
    const double tensor = (mt == 2 ? 2 : 1) * 4.0 * (bn / 2);
    const double smem = mt == 3 ? (bn == 192 ? 640.0 : 720.0)
                                : 0.92 * ((bm * 128.0 + bn * 128.0) + mt * (BM1 * 128.0 + bn * 128.0)) / 128.0;
    const double per_kb = tensor > smem ? tensor : smem;
    const double epilogue = mt == 2 ? 14.0 * bn + 900.0 : 1500.0;
    const double cost = gt_cdiv(tiles * ks, workers) * ((double)gt_cdiv(kblocks, ks) * per_kb + epilogue);
    if (cost < best_cost) { best_cost = cost; best = i; ksplit = ks; }
    // A deep product whose tiles fill the SMs unevenly (the readout's dX: 384 tiles of 128 x 192 on 148 SMs are 2.6
    // waves, run as 3) may be cut along K as well when that evens the waves out: as 192 tiles of 256 x 192 in three
    // slices it is 576 units = 3.9 waves of a third of the length. The clear before it and the reduce-adds are
    // charged; the candidate is taken after the loop only if it is predicted well ahead. Measured at rows 16384: the
    // readout's dX (K 49152) 1890 -> 1292 us, dX of gate and up (K 3072) 128 -> 106 us; at K 1536 the same choice
    // measured slower (60.5 -> 67.9 us), hence the depth limit of 64 K blocks.
    if (ks == 1 && tiles >= workers && kblocks >= 64 && deep_split && mt != 3) {
      double best_w = (double)gt_cdiv(tiles, workers);
      int k2best = 1;
      for (int k2 = 2; k2 <= 4; k2++) {
        const double w2 = (double)gt_cdiv(tiles * k2, workers) / k2;
        if (w2 < best_w - 0.05) { best_w = w2; k2best = k2; }
      }
      if (k2best > 1) {
        const double c2 = gt_cdiv(tiles * k2best, workers) * ((double)gt_cdiv(kblocks, k2best) * per_kb + epilogue + 600.0) + 8000.0;
        if (c2 < cost_deep) { cost_deep = c2; best_deep = i; ks_deep = k2best; }
      }
    }
  }
  if (cost_deep < 0.92 * best_cost) { best_cost = cost_deep; best = best_deep; ksplit = ks_deep; }
  if (best_cost >= 1e30) return GT_OK;
  const int mt = cfgs[best].mt, bn = cfgs[best].bn;
  const int a_box = mt == 2 ? 2 * BM1 : BM1, b_box = mt == 3 ? bn / 2 : bn;   // rows one TMA copy brings
  PartMaps maps;
  maps.nparts = nparts;
  int kb_sum = 0;
  for (int p = 0; p < nparts; p++) {
    const int K = Ks[p];
    const uint64_t sa = (uint64_t)M * K, sb = (uint64_t)N * K;
    const bool oka = a_k ? make_map_3d(&maps.a[p], as[p], K, M, batch, K, sa, a_box, true) : make_map_3d(&maps.a[p], as[p], M, K, batch, M, sa, BK, false);
    const bool okb = b_k ? make_map_3d(&maps.b[p], bs[p], K, N, batch, K, sb, b_box, true) : make_map_3d(&maps.b[p], bs[p], N, K, batch, N, sb, BK, false);
    if (!oka || !okb) return GT_OK;
    kb_sum += gt_cdiv(K, BK);
    maps.kb_end[p] = kb_sum;
  }
  for (int p = nparts; p < MAX_PARTS; p++) { maps.a[p] = maps.a[0]; maps.b[p] = maps.b[0]; maps.kb_end[p] = kb_sum; }
  // the output goes through TMA (32x32 blocks of whole 128-byte rows) whenever its row pitch allows a tensor map
  const uint64_t sc = (uint64_t)M * N;
  maps.ngroups = 1;
  maps.c[0] = maps.a[0];
  const int tma_store = ((N & 3) == 0 && make_map_3d(&maps.c[0], c, N, M, batch, N, sc, 32, true)) ? 1 : 0;
  for (int p = 1; p < MAX_PARTS; p++) maps.c[p] = maps.c[0];
  for (int p = 0; p < MAX_PARTS; p++) { maps.gM[p] = M; maps.gN[p] = N; maps.g_accum[p] = accum; maps.unit_end[p] = 0; }
  if (ksplit > 1 && !accum) GT_CUDA(ctx, cudaMemsetAsync(c, 0, sizeof(float) * (size_t)M * N * batch, ctx->stream));
  const float out_scale = alpha * TRUNC_COMP;
  const int K0 = Ks[0];
  const long ntiles = (long)gt_cdiv(N, bn) * gt_cdiv(M, mt == 1 ? BM1 : 2 * BM1) * ksplit * batch;
  gt_status s;
  if (mt == 3 && bn == 192) s = launch_pair_kind<192>(ctx, kind, maps.a[0], maps.b[0], maps.c[0], tma_store, c, M, N, K0, accum, ksplit, batch, npairs, out_scale);
  else if (mt == 3) s = launch_pair_kind<256>(ctx, kind, maps.a[0], maps.b[0], maps.c[0], tma_store, c, M, N, K0, accum, ksplit, batch, npairs, out_scale);
  else if (mt == 1 && bn == 192) s = launch_kind<192, 1>(ctx, kind, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
  else if (mt == 1) s = launch_kind<128, 1>(ctx, kind, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
  else if (bn == 256) s = launch_kind<256, 2>(ctx, kind, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
  else s = launch_kind<192, 2>(ctx, kind, maps, ntiles, tma_store, c, M, N, accum, ksplit, batch, out_scale);
  if (s) return s;
  *handled = true;
  return GT_OK;
}

// ngroups independent products of one layout and one K, each with its own operands, extents and accumulate flag, as
// ONE launch: the weight gradients dW_g = dY_g^T.X_g of several projections (K = rows for all of them). Their tiles
// are so few per product that each would need its own split-K launch with its own tail; together they fill the SMs.
static gt_status gemm_tc_grouped(gt_ctx* ctx, int kind, int ngroups, const int* Ms, const int* Ns, int K, const float* const* as,
                                 const float* const* bs, float* const* cs, const int* accums, const int* ropes, const float2* rope_tab,
                                 int rope_period, float alpha, bool* handled) {
  *handled = false;
  if (ngroups < 2 || ngroups > MAX_PARTS || K < 16) return GT_OK;
  bool any_rope = false;
  for (int g = 0; ropes && g < ngroups; g++) {
    if (!ropes[g]) continue;
    if (kind != GT_GEMM_NT || (Ns[g] & 63) || !rope_tab || rope_period <= 0) return GT_OK;
    any_rope = true;
  }
  const bool a_k = kind != GT_GEMM_TN, b_k = kind == GT_GEMM_NT;
  for (int g = 0; g < ngroups; g++) {
    const int a_inner = a_k ? K : Ms[g], b_inner = b_k ? K : Ns[g];
    if (Ms[g] < 16 || Ns[g] < 16 || (a_inner & 3) || (b_inner & 3) || (Ns[g] & 3)) return GT_OK;
    if ((((uintptr_t)as[g]) | ((uintptr_t)bs[g]) | ((uintptr_t)cs[g])) & 15) return GT_OK;
  }
  if (ctx->device < 0 || ctx->device >= 64 || !device_flag(ctx)) return GT_OK;
  const int kblocks = gt_cdiv(K, BK);
  const long workers = ctx->sm_count - ctx->sm_reserved;
  // 256 x 192 or 128 x 192 tiles; the split-K factor (one for the whole launch) that wastes least of the last wave,
  // among those that leave a slice at least 8 K blocks and add at most 8 partial sums per output element
  int best_mt = 1, best_ks = 1;
  double best_cost = 1e30;
  const char* force = getenv("GT_GEMM_TILE");
  for (int mt = 1; mt <= 2; mt++) {
    if (force) { int fm = 0, fb = 0; if (sscanf(force, "%d,%d", &fm, &fb) == 2 && (fm != mt || fb != 192)) continue; }
    long tiles = 0;
    for (int g = 0; g < ngroups; g++) tiles += (long)gt_cdiv(Ns[g], 192) * gt_cdiv(Ms[g], mt * BM1);
    const double per_kb = 0.92 * ((mt * BM1 * 128.0 + 192 * 128.0) + mt * (BM1 * 128.0 + 192 * 128.0)) / 128.0;
    const double epilogue = mt == 2 ? 14.0 * 192 + 900.0 : 1500.0;
    for (int ks = 1; ks <= 8 && (ks == 1 || kblocks / ks >= 8); ks++) {
      const long waves = gt_cdiv(tiles * ks, workers);
      const double cost = waves * (gt_cdiv(kblocks, ks) * per_kb + epilogue + (ks > 1 ? 600.0 : 0.0));
      if (cost < best_cost) { best_cost = cost; best_mt = mt; best_ks = ks; }
    }
  }
  if (best_cost >= 1e30) return GT_OK;
  const int mt = best_mt, ksplit = best_ks, bm = mt * BM1;
  PartMaps maps;
  maps.nparts = 1;
  maps.ngroups = ngroups;
  int units = 0;
  for (int g = 0; g < ngroups; g++) {
    const int M = Ms[g], N = Ns[g];
    const bool oka = a_k ? make_map_3d(&maps.a[g], as[g], K, M, 1, K, (uint64_t)M * K, bm, true) : make_map_3d(&maps.a[g], as[g], M, K, 1, M, (uint64_t)M * K, BK, false);
    const bool okb = b_k ? make_map_3d(&maps.b[g], bs[g], K, N, 1, K, (uint64_t)N * K, 192, true) : make_map_3d(&maps.b[g], bs[g], N, K, 1, N, (uint64_t)N * K, BK, false);
    const bool okc = make_map_3d(&maps.c[g], cs[g], N, M, 1, N, (uint64_t)M * N, 32, true);
    if (!oka || !okb || !okc) return GT_OK;
    units += gt_cdiv(N, 192) * gt_cdiv(M, bm) * ksplit;
    maps.unit_end[g] = units;
    maps.gM[g] = M; maps.gN[g] = N; maps.g_accum[g] = accums[g];
    maps.g_rope[g] = any_rope ? ropes[g] : 0;
    maps.kb_end[g] = kblocks;
  }
  maps.rope_tab = rope_tab;
  maps.rope_period = rope_period;
  for (int g = ngroups; g < MAX_PARTS; g++) {
    maps.a[g] = maps.a[0]; maps.b[g] = maps.b[0]; maps.c[g] = maps.c[0];
    maps.unit_end[g] = units; maps.gM[g] = Ms[0]; maps.gN[g] = Ns[0]; maps.g_accum[g] = accums[0]; maps.kb_end[g] = kblocks;
    maps.g_rope[g] = 0;
  }
  if (ksplit > 1)
    for (int g = 0; g < ngroups; g++)
      if (!accums[g]) GT_CUDA(ctx, cudaMemsetAsync(cs[g], 0, sizeof(float) * (size_t)Ms[g] * Ns[g], ctx->stream));
  gt_status s;
  if (any_rope)
    s = mt == 1 ? launch<true, true, 192, 1, EPI_ROPE>(ctx, maps, units, 1, cs[0], Ms[0], Ns[0], accums[0], ksplit, 1, alpha * TRUNC_COMP)
                : launch<true, true, 192, 2, EPI_ROPE>(ctx, maps, units, 1, cs[0], Ms[0], Ns[0], accums[0], ksplit, 1, alpha * TRUNC_COMP);
  else
    s = mt == 1 ? launch_kind<192, 1>(ctx, kind, maps, units, 1, cs[0], Ms[0], Ns[0], accums[0], ksplit, 1, alpha * TRUNC_COMP)
                : launch_kind<192, 2>(ctx, kind, maps, units, 1, cs[0], Ms[0], Ns[0], accums[0], ksplit, 1, alpha * TRUNC_COMP);
  if (s) return s;
  *handled = true;
  return GT_OK;
}

// gate = x.Wg^T, up = x.Wu^T and out = act(gate) * up as one launch (see the GLU form of the kernel).
gt_status gt_glu_linear_tc(gt_ctx* ctx, int op, int rows, int ffn, int in, const float* x, const float* wg, const float* wu, float* gate,
                           float* up, float* out, bool* handled) {
  *handled = false;
  if (rows < 16 || ffn < 96 || in < 16 || (in & 3) || (ffn & 3)) return GT_OK;
  if ((((uintptr_t)x) | ((uintptr_t)wg) | ((uintptr_t)wu) | ((uintptr_t)gate) | ((uintptr_t)up) | ((uintptr_t)out)) & 15) return GT_OK;
  if (ctx->device < 0 || ctx->device >= 64 || !device_flag(ctx)) return GT_OK;
  constexpr int BN = 192;
  PartMaps maps;
  maps.nparts = 1;
  maps.ngroups = 1;
  const int kblocks = gt_cdiv(in, BK);
  bool ok = make_map_3d(&maps.a[0], x, in, rows, 1, in, (uint64_t)rows * in, BM1, true);
  ok = ok && make_map_3d(&maps.b[0], wg, in, ffn, 1, in, (uint64_t)ffn * in, BN / 2, true);
  ok = ok && make_map_3d(&maps.b[1], wu, in, ffn, 1, in, (uint64_t)ffn * in, BN / 2, true);
  ok = ok && make_map_3d(&maps.c[0], gate, ffn, rows, 1, ffn, (uint64_t)rows * ffn, 32, true);
  ok = ok && make_map_3d(&maps.c[1], up, ffn, rows, 1, ffn, (uint64_t)rows * ffn, 32, true);
  ok = ok && make_map_3d(&maps.c[2], out, ffn, rows, 1, ffn, (uint64_t)rows * ffn, 32, true);
  if (!ok) return GT_OK;
  for (int p = 0; p < MAX_PARTS; p++) {
    if (p > 0) maps.a[p] = maps.a[0];
    if (p > 1) maps.b[p] = maps.b[0];
    if (p > 2) maps.c[p] = maps.c[0];
    maps.kb_end[p] = kblocks; maps.gM[p] = rows; maps.gN[p] = 2 * ffn; maps.g_accum[p] = 0; maps.unit_end[p] = 0;
  }
  const int N2 = 2 * gt_cdiv(ffn, BN / 2) * (BN / 2);   // whole tiles of 96 + 96 columns; the maps clip at ffn
  const long ntiles = (long)gt_cdiv(N2, BN) * gt_cdiv(rows, BM1);
  gt_status s = op == GT_EW_SILU
                    ? launch<true, true, BN, 1, GT_EW_SILU>(ctx, maps, ntiles, 1, out, rows, N2, 0, 1, 1, TRUNC_COMP)
                    : launch<true, true, BN, 1, GT_EW_GELU>(ctx, maps, ntiles, 1, out, rows, N2, 0, 1, 1, TRUNC_COMP);
  if (s) return s;
  *handled = true;
  return GT_OK;
}

gt_status gt_gemm_tc_grouped(gt_ctx* ctx, int kind, int ngroups, const int* Ms, const int* Ns, int K, const float* const* as,
                             const float* const* bs, float* const* cs, const int* accums, const int* ropes, const float2* rope_tab,
                             int rope_period, float alpha, bool* handled) {
  return gemm_tc_grouped(ctx, kind, ngroups, Ms, Ns, K, as, bs, cs, accums, ropes, rope_tab, rope_period, alpha, handled);
}

gt_status gt_gemm_tc_batched(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, int batch,
                             bool* handled) {
  return gemm_tc_dispatch(ctx, kind, accum, M, N, 1, &K, &a, &b, c, batch, 1.f, handled);
}

gt_status gt_gemm_tc(gt_ctx* ctx, int kind, int accum, int M, int N, int K, const float* a, const float* b, float* c, float alpha,
                     bool* handled) {
  return gemm_tc_dispatch(ctx, kind, accum, M, N, 1, &K, &a, &b, c, 1, alpha, handled);
}

gt_status gt_gemm_tc_multi(gt_ctx* ctx, int kind, int accum, int M, int N, int nparts, const int* Ks, const float* const* as,
                           const float* const* bs, float* c, bool* handled) {
  return gemm_tc_dispatch(ctx, kind, accum, M, N, nparts, Ks, as, bs, c, 1, 1.f, handled);
}
