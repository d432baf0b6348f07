/*
 * libgguftrain_cuda.so - C ABI of the B200 (sm_100a) training backend for gguf-trainer.
 *
 * The library stands in for the WebGPU device behind gguf-trainer's op interface
 * (`OpsBackend` + the `WebGPUBackend` buffer/sync API, src/backend/webgpu.ts). The
 * host (TypeScript through Deno.dlopen, or the Python mirror in this repository)
 * owns the tensors and the tape; this library owns device memory and the kernels.
 *
 * Conventions
 *  - Every function returns a gt_status (0 = ok). gt_last_error() gives the text.
 *    Nothing aborts, nothing throws across the boundary, no device traps.
 *  - gt_buf is a device address inside an allocation made by this library. Adding a
 *    byte offset to it is allowed (the chunked readout addresses row blocks that way).
 *  - All work is enqueued on the context's stream in call order (the WebGPU queue
 *    ordering the reference relies on); only gt_read, gt_sync, gt_graph_end and
 *    gt_profile_stop block.
 *  - Host pointers are borrowed for the duration of the call only.
 *  - One context per process per GPU, called from one thread.
 *  - Layout: row-major f32; activations [rows, features]; weights [out, in]; heads
 *    packed [rows, H*hd]; ids/targets are u32 with 0xffffffff as the ignore marker
 *    (webgpu.ts:1636-1646 maps -1 to it).
 *  - Backward entry points take an `accum` flag per gradient output: 1 adds into the
 *    buffer (the reference's `+=`), 0 overwrites it (what the reference gets from a
 *    cleared buffer followed by `+=`). A zero gradient handle skips that output (a
 *    frozen input, webgpu.ts:898-901).
 */
#ifndef GGUFTRAIN_H
#define GGUFTRAIN_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct gt_ctx gt_ctx;
typedef uint64_t gt_buf;
typedef int32_t gt_status;

enum { GT_OK = 0, GT_ERR_CUDA = 1, GT_ERR_ARG = 2, GT_ERR_OOM = 3, GT_ERR_STATE = 4, GT_ERR_NCCL = 5, GT_ERR_UNSUPPORTED = 6 };
enum { GT_GEMM_NT = 0, GT_GEMM_NN = 1, GT_GEMM_TN = 2 };
enum { GT_PREC_FP32 = 0, GT_PREC_TF32 = 1, GT_PREC_BF16 = 2 };
enum { GT_EW_ADD = 0, GT_EW_MUL = 1, GT_EW_SILU = 2, GT_EW_GELU = 3, GT_EW_SCALE = 4 };

/* ---- construction: initWebGPU / requireGPU / destroy (webgpu.ts:1812-1888, 764-767) ---- */
gt_status gt_init(int32_t device, gt_ctx** out);
gt_status gt_destroy(gt_ctx* ctx);
const char* gt_last_error(gt_ctx* ctx);            /* ctx may be NULL: last init error */
gt_status gt_device_name(gt_ctx* ctx, char* out, int32_t cap); /* adapterName / describeDevice */
/* Matrix-product precision: GT_PREC_FP32 = strict f32 FMA, GT_PREC_TF32 = TF32 tensor cores with f32 accumulation.
 * GT_PREC_BF16 is reserved: no BF16 kernels exist and the call answers GT_ERR_UNSUPPORTED, leaving the mode unchanged. */
gt_status gt_set_precision(gt_ctx* ctx, int32_t mode);
/* Rows handed to the ops are `batch` independent sequences of `seq_len` rows each (RoPE
 * positions wrap, attention is block-diagonal, losses are per sequence). batch=0 restores the
 * reference behaviour: one sequence of however many rows the op is given. */
gt_status gt_set_batch(gt_ctx* ctx, int32_t batch, int32_t seq_len);

/* ---- memory: BufferPool.acquire/release, createStateBuffer, writeBuffer, staging reads
 *      (webgpu.ts:214-262, 1465-1503) ---- */
gt_status gt_alloc(gt_ctx* ctx, uint64_t bytes, gt_buf* out);       /* pooled, contents undefined */
gt_status gt_alloc_state(gt_ctx* ctx, uint64_t bytes, gt_buf* out); /* zero-filled, never pooled */
gt_status gt_free(gt_ctx* ctx, gt_buf buf);                         /* back to the pool */
gt_status gt_write(gt_ctx* ctx, gt_buf dst, const void* host, uint64_t bytes);
gt_status gt_read(gt_ctx* ctx, gt_buf src, void* host, uint64_t bytes); /* blocks until the data is on the host */
/* The same read without blocking the caller or the compute stream (checkpoints taken while training goes on:
 * MuonGpu.syncWeightsToHost / exportState, src/backend/muon-gpu.ts:440-470, built on readStateBuffer,
 * src/backend/webgpu.ts:1492-1503). gt_read_async snapshots `bytes` at `src` as of the work enqueued so far into
 * pinned memory owned by the library, on a copy stream that runs beside later compute. gt_read_fence makes the
 * compute stream wait, on the device, for every read started so far: call it before enqueueing work that overwrites
 * their sources (the next optimizer step). gt_read_finish blocks until that one read has landed and copies it to
 * `host`; the pinned block is then recycled. */
gt_status gt_read_async(gt_ctx* ctx, gt_buf src, uint64_t bytes, uint64_t* out_ticket);
gt_status gt_read_fence(gt_ctx* ctx);
gt_status gt_read_finish(gt_ctx* ctx, uint64_t ticket, void* host, uint64_t bytes);
gt_status gt_zero(gt_ctx* ctx, gt_buf buf, uint64_t bytes);             /* clearBuffer */
gt_status gt_copy(gt_ctx* ctx, gt_buf dst, gt_buf src, uint64_t bytes); /* seedGradFrom, webgpu.ts:748-761 */
gt_status gt_sync(gt_ctx* ctx);                                         /* submit + wait; surfaces latched errors */
/* out[0] pooled bytes, out[1] state bytes, out[2] bytes read back since the last gt_sync,
 * out[3] kernels launched since gt_init (residentBytes / lastSyncReadbackBytes) */
gt_status gt_stats(gt_ctx* ctx, uint64_t* out4);

/* ---- ops (OpsBackend, src/model/autograd.ts:103-151; kernels src/backend/wgsl.ts) ---- */
/* C[M,N] (+)= op(A)*op(B): NT A[M,K] B[N,K]; NN A[M,K] B[K,N]; TN A[K,M] B[K,N]
 * (WebGPUBackend.gemm, webgpu.ts:1654-1671; srcGemm wgsl.ts:87-196). */
gt_status gt_gemm(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t K, gt_buf a, gt_buf b, gt_buf c);
/* The same with a factor on the product: C (+)= alpha * op(A)*op(B) (the alpha/r of a LoRA adapter, applied where
 * the [T, r] intermediate is written instead of by a `scale` pass, src/model/autograd.ts:311-319). */
gt_status gt_gemm_scaled(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t K, gt_buf a, gt_buf b, gt_buf c,
                         float alpha);
/* C[M,N] (+)= op(A)*op(B) + op(A2)*op(B2), both products of layout `kind`, the second K2 deep: the projection with a
 * LoRA adapter, x.W^T + (s.x.A^T).B^T, and its input gradient g.W + (s.g.B).A, as one product each
 * (`linear`, src/model/autograd.ts:311-319, records them as separate ops joined by `add`). */
gt_status gt_gemm2(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t K, gt_buf a, gt_buf b, int32_t K2,
                   gt_buf a2, gt_buf b2, gt_buf c);
/* The general form: C[M,N] (+)= sum over p < nparts (1..8) of op(A_p)*op(B_p), product p being Ks[p] deep, all of
 * layout `kind`. One launch and one write of C where the reference issues nparts accumulating products: the input
 * gradient of an activation that feeds several projections, dX = dQ.Wq + dK.Wk + dV.Wv (each `linear` backward adds
 * its term, src/backend/webgpu.ts:884-903). */
gt_status gt_gemm_multi(gt_ctx* ctx, int32_t kind, int32_t accum, int32_t M, int32_t N, int32_t nparts, const int32_t* Ks,
                        const gt_buf* as, const gt_buf* bs, gt_buf c);
/* ngroups (1..8) independent products of one layout and one depth K as one launch: C_g[Ms[g], Ns[g]] (+)= op(A_g)*op(B_g)
 * with accums[g] per product. The weight gradients dW = dY^T.X of the projections of a layer (every `linear` backward
 * issues its own, src/backend/webgpu.ts:898-901) have few output tiles each and a contraction over all rows; grouped,
 * their tiles share the SMs and one split-K factor instead of each paying a launch, a clear and a last wave. */
gt_status gt_gemm_grouped(gt_ctx* ctx, int32_t kind, int32_t ngroups, const int32_t* Ms, const int32_t* Ns, int32_t K,
                          const gt_buf* as, const gt_buf* bs, const gt_buf* cs, const int32_t* accums);
/* The same with a factor applied to every product as it is written (the thin products x.A^T of the adapters of
 * projections that share an input, src/model/autograd.ts:311-319, carry the adapter scale this way). */
gt_status gt_gemm_grouped_scaled(gt_ctx* ctx, int32_t kind, int32_t ngroups, const int32_t* Ms, const int32_t* Ns, int32_t K,
                                 const gt_buf* as, const gt_buf* bs, const gt_buf* cs, const int32_t* accums, float alpha);
/* add/mul/silu/gelu/scale (webgpu.ts:905-1078, srcElementwise wgsl.ts:199-209) */
gt_status gt_ew_fwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf a, gt_buf b, float c, gt_buf out);
gt_status gt_ew_bwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf a, gt_buf b, float c, gt_buf gout,
                    gt_buf ga, int32_t accum_a, gt_buf gb, int32_t accum_b);
/* Gated unit act(x)*u in one pass, act = GT_EW_SILU or GT_EW_GELU: the reference's silu/gelu followed by mul
 * (webgpu.ts:905-1078 issues them as two dispatches; src/arch/llama.ts:209-211). gx (+)= g*u*act'(x), gu (+)= g*act(x). */
gt_status gt_glu_fwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf x, gt_buf u, gt_buf out);
gt_status gt_glu_bwd(gt_ctx* ctx, int32_t op, uint64_t n, gt_buf x, gt_buf u, gt_buf gout,
                     gt_buf gx, int32_t accum_x, gt_buf gu, int32_t accum_u);
/* The whole entry of a gated FFN: gate = x.Wg^T, up = x.Wu^T (both [rows, ffn], kept for backward) and out = act(gate)*up,
 * x:[rows, in], Wg, Wu:[ffn, in] (src/arch/llama.ts:209-211: two `linear`, an activation and a `mul`). On the tensor
 * cores one launch: each output tile holds 96 gate and the matching 96 up columns and the unit is applied as the tile
 * is written. */
gt_status gt_glu_linear_fwd(gt_ctx* ctx, int32_t op, int32_t rows, int32_t ffn, int32_t in, gt_buf x, gt_buf wg, gt_buf wu, gt_buf gate,
                            gt_buf up, gt_buf out);
/* rmsNorm and rmsNormHeads ([rows, d] view; webgpu.ts:1673-1701, wgsl.ts:217-303) */
gt_status gt_rmsnorm_fwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, float eps, gt_buf y, gt_buf rinv);
gt_status gt_rmsnorm_bwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, gt_buf rinv, gt_buf gy,
                         gt_buf gx, int32_t accum_x, gt_buf gw, int32_t accum_w);
/* The residual add that precedes a norm, in the norm's pass over the row: sum = a + b, y = rmsNorm(sum)
 * (`add` then `rmsNorm`, src/arch/llama.ts:203-208, as one kernel: the sum is not read back). */
gt_status gt_add_rmsnorm_fwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf a, gt_buf b, gt_buf w, float eps, gt_buf sum, gt_buf y,
                             gt_buf rinv);
/* rmsNorm backward whose input-gradient term lands on top of another buffer: gx = gadd + term. `add` backward hands
 * its upstream gradient to both inputs; when the next thing added to it is this term, gadd is that upstream buffer
 * and the copy `add` backward would have made never happens. gw as in gt_rmsnorm_bwd. */
gt_status gt_rmsnorm_bwd_add(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf x, gt_buf w, gt_buf rinv, gt_buf gy, gt_buf gadd, gt_buf gx,
                             gt_buf gw, int32_t accum_w);
/* embedding gather / scatter-add (webgpu.ts:1090-1108, wgsl.ts:305-344); gw always accumulates */
gt_status gt_embedding_fwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf w, gt_buf ids, gt_buf out);
gt_status gt_embedding_bwd(gt_ctx* ctx, int32_t rows, int32_t d, gt_buf gy, gt_buf ids, gt_buf gw);
/* Token and mask ingest. `tokens` (and `mask`, 0 = none) are device copies of a token file as it is on disk: bare
 * little-endian u16 or u32 values, bytes_per_token 2 or 4, `count` tokens (diskTokenSource, src/data/tokens.ts:158-185;
 * the mask is read with the same width, src/commands/pretrain.ts:416). `starts` holds B window starts as u64 on the
 * device. Writes ids[b*T+t] = tokens[start_b+t] and targets[b*T+t] = tokens[start_b+1+t], or 0xffffffff where
 * mask[start_b+1+t] == 0 (maskWindow, src/train/trainer.ts:45-49; window draw src/backend/train-gpu.ts:206-208).
 * A start beyond count-T-1 reads nothing: its rows come out ignored and the next gt_sync reports GT_ERR_ARG.
 * gt_tokens_max returns the largest token value, so the host can refuse a corpus that does not fit the vocabulary
 * once, at upload, instead of checking every window. */
gt_status gt_gather_windows(gt_ctx* ctx, gt_buf tokens, gt_buf mask, int32_t bytes_per_token, uint64_t count, gt_buf starts,
                            int32_t B, int32_t T, gt_buf ids, gt_buf targets);
gt_status gt_tokens_max(gt_ctx* ctx, gt_buf tokens, int32_t bytes_per_token, uint64_t count, uint32_t* out_max);
/* NeoX RoPE, x:[rows, H*hd], position = row (mod seq_len when a batch is set) + pos_offset (wgsl.ts:346-384) */
gt_status gt_rope_fwd(gt_ctx* ctx, int32_t rows, int32_t H, int32_t hd, double base, int32_t pos_offset, gt_buf x, gt_buf y);
gt_status gt_rope_bwd(gt_ctx* ctx, int32_t rows, int32_t H, int32_t hd, double base, int32_t pos_offset, gt_buf gy,
                      gt_buf gx, int32_t accum);
/* causal GQA attention with optional sliding window; lse:[Hq, rows] in log2 units
 * (webgpu.ts:1125-1192; srcAttnFwd/BwdD/BwdDq/BwdDkv wgsl.ts:657-918) */
gt_status gt_attention_fwd(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window,
                           gt_buf q, gt_buf k, gt_buf v, gt_buf out, gt_buf lse);
gt_status gt_attention_bwd(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window,
                           gt_buf q, gt_buf k, gt_buf v, gt_buf out, gt_buf lse, gt_buf gout,
                           gt_buf gq, int32_t accum_q, gt_buf gk, int32_t accum_k, gt_buf gv, int32_t accum_v);
/* The rotary embedding merged into its neighbours (the reference records `rope(linear(x, Wq))`, `rope(linear(x, Wk))`
 * and then `attention`, src/arch/llama.ts:195-201; every op is its own dispatch, src/backend/webgpu.ts:1110-1123).
 * gt_linear_rope_grouped: ngroups (1..8) projections y_g = x.W_g^T of one input x:[rows, K] as one launch; the outputs
 * with heads[g] > 0 (y_g:[rows, heads[g]*hd]) leave the kernel already rotated, so the unrotated projection is never
 * written and the rotation's pass over it is not launched. heads[g] = 0: a plain projection (v).
 * gt_attention_bwd_rope: gt_attention_bwd for q and k that came out of such a rotation; gq and gk receive the
 * gradients with respect to the rotation's inputs (the transposed rotation is applied to the dQ and dK tiles as they
 * are written). Both fall back to the separate launches where the fused kernels do not apply (strict f32, head sizes
 * other than 64 in forward or 256 in backward), with the same results to summation order. */
/* rope(rmsNormHeads(x, w)) as one pass (src/arch/qwen3.ts:169-172, src/arch/gemma3.ts:194-197 record the two ops one after
 * the other): x, y:[rows, H*hd], w:[hd], rinv:[rows*H] as gt_rmsnorm_fwd over rows*H heads would write it. */
gt_status gt_rmsnorm_heads_rope_fwd(gt_ctx* ctx, int32_t rows, int32_t H, int32_t hd, gt_buf x, gt_buf w, float eps, gt_buf y,
                                    gt_buf rinv, double base, int32_t pos_offset);
gt_status gt_linear_rope_grouped(gt_ctx* ctx, int32_t ngroups, int32_t rows, int32_t K, gt_buf x, const int32_t* Ns,
                                 const gt_buf* ws, const gt_buf* ys, const int32_t* heads, int32_t hd, double base,
                                 int32_t pos_offset);
gt_status gt_attention_bwd_rope(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window,
                                gt_buf q, gt_buf k, gt_buf v, gt_buf out, gt_buf lse, gt_buf gout,
                                gt_buf gq, int32_t accum_q, gt_buf gk, int32_t accum_k, gt_buf gv, int32_t accum_v,
                                double base, int32_t pos_offset);
/* No counterpart in the reference. The same f32 attention backward as gt_attention_bwd for callers that
 * cannot allocate device memory (hosts that give all of HBM to their own arena, or steps that cannot afford
 * cudaMalloc's device-wide synchronisation): its only scratch, the per-(head,row) dot products dO.O, sits
 * in a fixed 4 MiB array inside the library, so the call never allocates or frees. Limit: rows*Hq <=
 * 1048576, larger shapes are refused with GT_ERR_ARG. Always f32, whatever gt_set_precision says: it
 * recomputes the probabilities from q, k and lse in f32, so out and lse must come from a forward that ran in
 * GT_PREC_FP32 (row statistics of a TF32 forward do not normalise f32 scores to better than about 1e-3). The
 * first call on a device resolves the array's address, and may be what loads this part of the library onto
 * the device (do it before any stream capture). All calls share the array: calls that overlap on the GPU
 * race, so keep them on one stream. */
gt_status gt_attention_bwd_static(gt_ctx* ctx, int32_t rows, int32_t Hq, int32_t Hkv, int32_t hd, int32_t window,
                                  gt_buf q, gt_buf k, gt_buf v, gt_buf out, gt_buf lse, gt_buf gout,
                                  gt_buf gq, int32_t accum_q, gt_buf gk, int32_t accum_k, gt_buf gv, int32_t accum_v);
/* cross entropy over logits [rows, V] (webgpu.ts:1295-1329; srcCeFwd/Reduce/Bwd wgsl.ts:936-996, 1112-1133).
 * stats: [rows, 2] (row max, 1/sum). loss: [1 + nseq] floats, loss[0] = mean over sequences of the
 * per-sequence kept-row means, loss[1+s] = sequence s; inv_kept: [nseq] = 1/max(kept_s, 1). */
gt_status gt_ce_fwd(gt_ctx* ctx, int32_t rows, int32_t V, gt_buf logits, gt_buf targets, gt_buf stats,
                    gt_buf loss, gt_buf inv_kept);
gt_status gt_ce_bwd(gt_ctx* ctx, int32_t rows, int32_t V, gt_buf logits, gt_buf targets, gt_buf stats,
                    gt_buf inv_kept, gt_buf gloss, gt_buf glogits, int32_t accum);
/* chunked readout+CE (webgpu.ts:1214-1278; srcCeChunkStats/LossFromStats/ChunkGrad wgsl.ts:1153-1247).
 * run: [rows, 3] running (max, sum, target logit); chunk logits [rows, n] cover vocab [v0, v0+n). */
gt_status gt_ce_chunk_stats(gt_ctx* ctx, int32_t rows, int32_t n, int32_t v0, int32_t first, gt_buf chunk,
                            gt_buf targets, gt_buf run);
gt_status gt_ce_loss_from_stats(gt_ctx* ctx, int32_t rows, gt_buf run, gt_buf targets, gt_buf loss, gt_buf inv_kept);
gt_status gt_ce_chunk_grad(gt_ctx* ctx, int32_t rows, int32_t n, int32_t v0, gt_buf chunk, gt_buf targets,
                           gt_buf run, gt_buf inv_kept, gt_buf gloss);
/* sparse-teacher soft CE (webgpu.ts:1331-1378; srcSoftCeFwd/BwdP/BwdQ wgsl.ts:1004-1110).
 * tids/tprobs: [rows, k]; a row whose first id is 0xffffffff is ignored. */
gt_status gt_soft_ce_fwd(gt_ctx* ctx, int32_t rows, int32_t V, int32_t k, gt_buf logits, gt_buf tids, gt_buf tprobs,
                         gt_buf stats, gt_buf loss, gt_buf inv_kept);
gt_status gt_soft_ce_bwd(gt_ctx* ctx, int32_t rows, int32_t V, int32_t k, gt_buf logits, gt_buf tids, gt_buf tprobs,
                         gt_buf stats, gt_buf inv_kept, gt_buf gloss, gt_buf glogits, int32_t accum);

/* ---- optimizers (AdamWGpu src/backend/adamw-gpu.ts:131-251; MuonGpu src/backend/muon-gpu.ts:351-470) ---- */
/* A parameter group: n tensors given as parallel host arrays of device addresses and element counts.
 * Moments are allocated zeroed by the library (createStateBuffer). */
gt_status gt_adamw_create(gt_ctx* ctx, int32_t n, const gt_buf* data, const gt_buf* grad, const uint64_t* sizes,
                          float lr, float beta1, float beta2, float eps, float weight_decay, float clip, uint64_t* out_handle);
gt_status gt_adamw_set_lr(gt_ctx* ctx, uint64_t h, float lr);     /* setLrScale: host passes base*scale */
gt_status gt_adamw_step(gt_ctx* ctx, uint64_t h);                 /* recordStep: clip-norm reduce + fused update */
gt_status gt_adamw_state(gt_ctx* ctx, uint64_t h, int32_t i, gt_buf* m, gt_buf* v); /* exportState/importState buffers */
gt_status gt_adamw_get_t(gt_ctx* ctx, uint64_t h, int32_t* t);
gt_status gt_adamw_set_t(gt_ctx* ctx, uint64_t h, int32_t t);
/* Muon over n matrices [rows_i, cols_i]: momentum, Frobenius normalise, quintic Newton-Schulz, apply. */
gt_status gt_muon_create(gt_ctx* ctx, int32_t n, const gt_buf* data, const gt_buf* grad, const int32_t* rows,
                         const int32_t* cols, float lr, float momentum, int32_t nesterov, int32_t ns_steps,
                         uint64_t* out_handle);
gt_status gt_muon_set_lr(gt_ctx* ctx, uint64_t h, float lr);
gt_status gt_muon_step(gt_ctx* ctx, uint64_t h);
gt_status gt_muon_state(gt_ctx* ctx, uint64_t h, int32_t i, gt_buf* momentum);
/* Data parallel only (after gt_dp_init, on every rank alike): split the Newton-Schulz iterations of each same-shape
 * group of matrices over the ranks and all-gather the orthogonalised matrices, instead of every rank repeating all of
 * them. Results are the same bits on every rank; momentum and the weight update stay replicated. */
gt_status gt_muon_set_sharded(gt_ctx* ctx, uint64_t h, int32_t on);
/* newtonSchulzGpu (muon-gpu.ts:258-282): out[m,n] = NS_steps(g[m,n]) */
gt_status gt_newton_schulz(gt_ctx* ctx, int32_t m, int32_t n, int32_t steps, gt_buf g, gt_buf out);

/* ---- replay: one micro-batch's recorded work as a CUDA graph (the role prepareDispatch plays for
 *      the optimizers, webgpu.ts:1512-1537, extended to the whole forward+backward) ---- */
gt_status gt_graph_begin(gt_ctx* ctx);
gt_status gt_graph_end(gt_ctx* ctx, uint64_t* out_graph);
gt_status gt_graph_launch(gt_ctx* ctx, uint64_t graph);
gt_status gt_graph_destroy(gt_ctx* ctx, uint64_t graph);

/* ---- profiling: startProfile/stopProfile/readProfile (webgpu.ts:817-880). Events on the stream. ---- */
gt_status gt_event_record(gt_ctx* ctx, int32_t slot);            /* slots 0..63 */
gt_status gt_event_elapsed_ms(gt_ctx* ctx, int32_t start_slot, int32_t end_slot, float* ms); /* blocks on end_slot */

/* ---- self-test: no counterpart in the reference. Every wait inside the tensor-core kernels is bounded (2 s) and, on
 *      expiry, raises a device flag that the next gt_sync turns into GT_ERR_CUDA "a pipeline wait expired". This
 *      entry point runs that wait on a barrier nothing arrives on, with a limit of limit_us, so the expiry path can be
 *      exercised without a fault: the kernel returns after limit_us and the next gt_sync reports code 99. ---- */
gt_status gt_selftest_bounded_wait(gt_ctx* ctx, int32_t limit_us);

/* ---- data parallel: no counterpart in the reference (single device). One process per GPU;
 *      gradients are summed across ranks with NCCL on a side stream. ---- */
gt_status gt_dp_unique_id(uint8_t* out128);                       /* rank 0 creates, host broadcasts */
gt_status gt_dp_init(gt_ctx* ctx, int32_t rank, int32_t world, const uint8_t* id128);
/* Start summing count f32 at buf across ranks, ordered after everything enqueued so far on the compute
 * stream; later compute does not wait for it until gt_dp_wait. */
gt_status gt_dp_allreduce_start(gt_ctx* ctx, gt_buf buf, uint64_t count);
gt_status gt_dp_wait(gt_ctx* ctx);                                /* compute stream waits for all started reductions */
/* The same, observed from the host with a limit: returns once every started reduction has completed, or aborts the
 * communicator and returns GT_ERR_NCCL when that takes longer than timeout_ms or NCCL reports an error (a rank that
 * left or hangs). The context stays usable; gt_dp_destroy + gt_dp_init build a new communicator. */
gt_status gt_dp_wait_host(gt_ctx* ctx, int32_t timeout_ms);
/* From now on the persistent kernels size their grids for the device's SMs minus n (0 restores): call it with the
 * number of CTAs the collective uses when the first reduction of a step starts, and with 0 after gt_dp_wait. Grid
 * sizes are recorded into captured graphs, so record under the same setting the replay will run under. */
gt_status gt_dp_reserve_sms(gt_ctx* ctx, int32_t n);
gt_status gt_dp_destroy(gt_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif
