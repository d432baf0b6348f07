// cuda.ts - the B200 backend behind gguf-trainer's op interface, bound to libgguftrain_cuda.so through Deno FFI.
//
// NOT EXECUTED IN THIS REPOSITORY: no TypeScript runtime exists where the library is built and tested. The file is the
// binding a maintainer adds as src/backend/cuda.ts. It is a port of gguf_trainer_b200/backend.py (the Python mirror the
// GPU tests drive through the same C ABI), so every rule below has a test on the Python side: first write to a
// gradient buffer overwrites and later ones accumulate (no clear pass), transients are recycled at sync() or at a
// region's end, a frozen external gets no gradient buffer, -1 ids upload as 0xffffffff.
//
// Public surface: that of WebGPUBackend (src/backend/webgpu.ts:290-1537): install/uninstall, the 14 ops of OpsBackend,
// beginRegion/endRegion/seedGradFrom/regionCount, uploadParams, sync, reclaimStepTransients, residentBytes, destroy,
// buffersFor, keepGradOnDevice, createStateBuffer, writeStateBuffer, readStateBuffer, seedGradFromHost, adapterName,
// describeDevice, timestampSupported, startProfile/stopProfile, gradClearsIssued, lastSyncReadbackBytes, and
// initCuda()/requireGPU() in place of initWebGPU()/requireGPU(). prepareDispatch/prepareGemm have no counterpart:
// AdamWCuda and MuonCuda below call gt_adamw_step / gt_muon_step instead of replaying WGSL dispatches.
//
// The Python mirror also defers some launches so that neighbouring ops run as one kernel (an activation whose only use
// is a product: _gatedUnit; a residual add whose first use is a norm: add/_rmsNormRows; the input-gradient products of
// an activation that feeds several projections: _deferDx; the weight gradients of a layer: _deferDw; projections of
// one input, with the gated unit or the rotary embedding that follows them: _deferLinear, rope; a per-head norm and
// the rotation after it: _deferHeadNorm; add's backward without a copy: _materializeCopy). They change no value, only
// launch counts (550 instead of 1183 per step of a 30-layer model); they are left out here to keep the port short and
// can be carried over method by method: INTEGRATION.md lists the entry point behind each.
import { type OpsBackend, setOpsBackend, Tensor } from "../model/autograd.ts";

const LIB_PATH = Deno.env.get("GGUFTRAIN_CUDA_LIB") ?? new URL("../../libgguftrain_cuda.so", import.meta.url).pathname;

// Every function of include/gguftrain.h. gt_ctx* is an opaque pointer, gt_buf a u64 device address, host arrays are
// borrowed for the duration of the call ("buffer"). Calls that block on the device are declared nonblocking so that
// they return Promises and the event loop keeps running (the reference's sync() is async for the same reason).
const SYMBOLS = {
  gt_init: { parameters: ["i32", "buffer"], result: "i32" },
  gt_destroy: { parameters: ["pointer"], result: "i32" },
  gt_last_error: { parameters: ["pointer"], result: "pointer" },
  gt_device_name: { parameters: ["pointer", "buffer", "i32"], result: "i32" },
  gt_set_precision: { parameters: ["pointer", "i32"], result: "i32" },
  gt_set_batch: { parameters: ["pointer", "i32", "i32"], result: "i32" },
  gt_alloc: { parameters: ["pointer", "u64", "buffer"], result: "i32" },
  gt_alloc_state: { parameters: ["pointer", "u64", "buffer"], result: "i32" },
  gt_free: { parameters: ["pointer", "u64"], result: "i32" },
  gt_write: { parameters: ["pointer", "u64", "buffer", "u64"], result: "i32" },
  gt_read: { parameters: ["pointer", "u64", "buffer", "u64"], result: "i32", nonblocking: true },
  gt_read_async: { parameters: ["pointer", "u64", "u64", "buffer"], result: "i32" },
  gt_read_fence: { parameters: ["pointer"], result: "i32" },
  gt_read_finish: { parameters: ["pointer", "u64", "buffer", "u64"], result: "i32", nonblocking: true },
  gt_zero: { parameters: ["pointer", "u64", "u64"], result: "i32" },
  gt_copy: { parameters: ["pointer", "u64", "u64", "u64"], result: "i32" },
  gt_sync: { parameters: ["pointer"], result: "i32", nonblocking: true },
  gt_stats: { parameters: ["pointer", "buffer"], result: "i32" },
  gt_gemm: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "u64"], result: "i32" },
  gt_gemm_scaled: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "u64", "f32"], result: "i32" },
  gt_gemm2: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "i32", "u64", "u64", "u64"], result: "i32" },
  gt_gemm_multi: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "buffer", "buffer", "buffer", "u64"], result: "i32" },
  gt_gemm_grouped: { parameters: ["pointer", "i32", "i32", "buffer", "buffer", "i32", "buffer", "buffer", "buffer", "buffer"], result: "i32" },
  gt_gemm_grouped_scaled: { parameters: ["pointer", "i32", "i32", "buffer", "buffer", "i32", "buffer", "buffer", "buffer", "buffer", "f32"], result: "i32" },
  gt_ew_fwd: { parameters: ["pointer", "i32", "u64", "u64", "u64", "f32", "u64"], result: "i32" },
  gt_ew_bwd: { parameters: ["pointer", "i32", "u64", "u64", "u64", "f32", "u64", "u64", "i32", "u64", "i32"], result: "i32" },
  gt_glu_fwd: { parameters: ["pointer", "i32", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_glu_bwd: { parameters: ["pointer", "i32", "u64", "u64", "u64", "u64", "u64", "i32", "u64", "i32"], result: "i32" },
  gt_glu_linear_fwd: { parameters: ["pointer", "i32", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_rmsnorm_fwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "f32", "u64", "u64"], result: "i32" },
  gt_rmsnorm_bwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "i32", "u64", "i32"], result: "i32" },
  gt_add_rmsnorm_fwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64", "f32", "u64", "u64", "u64"], result: "i32" },
  gt_rmsnorm_bwd_add: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64", "u64", "i32"], result: "i32" },
  gt_embedding_fwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64"], result: "i32" },
  gt_embedding_bwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64"], result: "i32" },
  gt_gather_windows: { parameters: ["pointer", "u64", "u64", "i32", "u64", "u64", "i32", "i32", "u64", "u64"], result: "i32" },
  gt_tokens_max: { parameters: ["pointer", "u64", "i32", "u64", "buffer"], result: "i32", nonblocking: true },
  gt_rope_fwd: { parameters: ["pointer", "i32", "i32", "i32", "f64", "i32", "u64", "u64"], result: "i32" },
  gt_rope_bwd: { parameters: ["pointer", "i32", "i32", "i32", "f64", "i32", "u64", "u64", "i32"], result: "i32" },
  gt_attention_fwd: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_attention_bwd: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64", "u64", "i32", "u64", "i32", "u64", "i32"], result: "i32" },
  gt_rmsnorm_heads_rope_fwd: { parameters: ["pointer", "i32", "i32", "i32", "u64", "u64", "f32", "u64", "u64", "f64", "i32"], result: "i32" },
  gt_linear_rope_grouped: { parameters: ["pointer", "i32", "i32", "i32", "u64", "buffer", "buffer", "buffer", "buffer", "i32", "f64", "i32"], result: "i32" },
  gt_attention_bwd_rope: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64", "u64", "i32", "u64", "i32", "u64", "i32", "f64", "i32"], result: "i32" },
  gt_attention_bwd_static: { parameters: ["pointer", "i32", "i32", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64", "u64", "i32", "u64", "i32", "u64", "i32"], result: "i32" },
  gt_ce_fwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_ce_bwd: { parameters: ["pointer", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64", "i32"], result: "i32" },
  gt_ce_chunk_stats: { parameters: ["pointer", "i32", "i32", "i32", "i32", "u64", "u64", "u64"], result: "i32" },
  gt_ce_loss_from_stats: { parameters: ["pointer", "i32", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_ce_chunk_grad: { parameters: ["pointer", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_soft_ce_fwd: { parameters: ["pointer", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64"], result: "i32" },
  gt_soft_ce_bwd: { parameters: ["pointer", "i32", "i32", "i32", "u64", "u64", "u64", "u64", "u64", "u64", "u64", "i32"], result: "i32" },
  gt_adamw_create: { parameters: ["pointer", "i32", "buffer", "buffer", "buffer", "f32", "f32", "f32", "f32", "f32", "f32", "buffer"], result: "i32" },
  gt_adamw_set_lr: { parameters: ["pointer", "u64", "f32"], result: "i32" },
  gt_adamw_step: { parameters: ["pointer", "u64"], result: "i32" },
  gt_adamw_state: { parameters: ["pointer", "u64", "i32", "buffer", "buffer"], result: "i32" },
  gt_adamw_get_t: { parameters: ["pointer", "u64", "buffer"], result: "i32" },
  gt_adamw_set_t: { parameters: ["pointer", "u64", "i32"], result: "i32" },
  gt_muon_create: { parameters: ["pointer", "i32", "buffer", "buffer", "buffer", "buffer", "f32", "f32", "i32", "i32", "buffer"], result: "i32" },
  gt_muon_set_lr: { parameters: ["pointer", "u64", "f32"], result: "i32" },
  gt_muon_step: { parameters: ["pointer", "u64"], result: "i32" },
  gt_muon_state: { parameters: ["pointer", "u64", "i32", "buffer"], result: "i32" },
  gt_muon_set_sharded: { parameters: ["pointer", "u64", "i32"], result: "i32" },
  gt_newton_schulz: { parameters: ["pointer", "i32", "i32", "i32", "u64", "u64"], result: "i32" },
  gt_graph_begin: { parameters: ["pointer"], result: "i32" },
  gt_graph_end: { parameters: ["pointer", "buffer"], result: "i32", nonblocking: true },
  gt_graph_launch: { parameters: ["pointer", "u64"], result: "i32" },
  gt_graph_destroy: { parameters: ["pointer", "u64"], result: "i32" },
  gt_event_record: { parameters: ["pointer", "i32"], result: "i32" },
  gt_event_elapsed_ms: { parameters: ["pointer", "i32", "i32", "buffer"], result: "i32", nonblocking: true },
  gt_selftest_bounded_wait: { parameters: ["pointer", "i32"], result: "i32" },
  gt_dp_unique_id: { parameters: ["buffer"], result: "i32" },
  gt_dp_init: { parameters: ["pointer", "i32", "i32", "buffer"], result: "i32", nonblocking: true },
  gt_dp_allreduce_start: { parameters: ["pointer", "u64", "u64"], result: "i32" },
  gt_dp_wait: { parameters: ["pointer"], result: "i32" },
  gt_dp_wait_host: { parameters: ["pointer", "i32"], result: "i32", nonblocking: true },
  gt_dp_reserve_sms: { parameters: ["pointer", "i32"], result: "i32" },
  gt_dp_destroy: { parameters: ["pointer"], result: "i32" },
} as const;

type Lib = Deno.DynamicLibrary<typeof SYMBOLS>["symbols"];
type Buf = bigint; // device address
let lib: Lib | null = null;
function load(): Lib {
  if (!lib) lib = Deno.dlopen(LIB_PATH, SYMBOLS).symbols; // throws when the library is missing: there is no fallback
  return lib;
}

const EW = { add: 0, mul: 1, silu: 2, gelu: 3, scale: 4 } as const;
const KIND = { NT: 0, NN: 1, TN: 2 } as const;
export const PRECISION = { fp32: 0, tf32: 1 } as const;

interface Entry {
  data: Buf;
  grad: Buf; // 0n for a frozen external
  bytes: number;
  external: boolean;
  gradLive: boolean; // has anything been written to grad in the current graph?
}

function cstr(p: Deno.PointerValue): string {
  return p ? new Deno.UnsafePointerView(p).getCString() : "";
}

/** -1 uploads as 0xffffffff, the marker the kernels test for (src/backend/webgpu.ts:1636-1646). */
function asU32(values: ArrayLike<number>): Uint32Array {
  const out = new Uint32Array(values.length);
  for (let i = 0; i < values.length; i++) out[i] = values[i] < 0 ? 0xffffffff : values[i];
  return out;
}

export class CudaBackend implements OpsBackend {
  readonly adapterName: string;
  readonly timestampSupported = true;
  lastSyncReadbackBytes = 0;
  gradClearsIssued = 0;
  private L: Lib;
  private ctx: Deno.PointerValue;
  private entries = new WeakMap<Tensor, Entry>();
  private touched = new Set<Tensor>();
  private keptOnDevice = new WeakSet<Tensor>();
  private transients: { addr: Buf; size: number }[] = [];
  private regionFree: { addr: Buf; size: number }[] = [];
  private regionsOpened = 0;
  private backwardBegun = false;
  private graphSynced = false;
  private graphOpen = false;
  private readback = 0;
  private batch: [number, number] = [0, 0];
  private prof: Map<string, { ms: number; count: number }> | null = null;

  constructor(device = 0, precision: keyof typeof PRECISION = "fp32") {
    this.L = load();
    const out = new BigUint64Array(1);
    const st = this.L.gt_init(device, out);
    if (st !== 0) throw new Error(cstr(this.L.gt_last_error(null)));
    this.ctx = Deno.UnsafePointer.create(out[0]);
    const name = new Uint8Array(256);
    this.check(this.L.gt_device_name(this.ctx, name, 256));
    this.adapterName = new TextDecoder().decode(name.subarray(0, name.indexOf(0)));
    this.check(this.L.gt_set_precision(this.ctx, PRECISION[precision]));
  }

  // ---------------------------------------------------------------- plumbing
  private check(status: number) {
    if (status !== 0) throw new Error(cstr(this.L.gt_last_error(this.ctx)));
  }
  describeDevice(): string[] {
    return [this.adapterName];
  }
  install() {
    setOpsBackend(this);
  }
  uninstall() {
    setOpsBackend(null);
  }
  destroy() {
    this.uninstall();
    if (this.ctx) this.L.gt_destroy(this.ctx);
    this.ctx = null;
  }
  setPrecision(p: keyof typeof PRECISION) {
    this.check(this.L.gt_set_precision(this.ctx, PRECISION[p]));
  }
  /** Rows passed to the ops are `batch` sequences of `seqLen` rows; 0 restores one sequence per call. */
  setBatch(batch: number, seqLen = 0) {
    this.check(this.L.gt_set_batch(this.ctx, batch, seqLen));
    this.batch = [batch, batch ? seqLen : 0];
  }
  private stats() {
    const o = new BigUint64Array(4);
    this.check(this.L.gt_stats(this.ctx, o));
    return { pool: Number(o[0]), state: Number(o[1]), readback: Number(o[2]), launches: Number(o[3]) };
  }
  residentBytes() {
    const s = this.stats();
    return { pool: s.pool, state: s.state, total: s.pool + s.state };
  }
  startProfile() {
    this.prof = new Map();
  }
  stopProfile() {
    const kernels = [...(this.prof ?? new Map()).entries()].map(([label, v]) => ({ label, ms: v.ms, count: v.count }));
    this.prof = null;
    return { kernels, overflow: false };
  }
  /** Runs one enqueueing call; while a profile is open it is bracketed by two events and attributed to `label`. */
  private run(label: string, call: () => number) {
    if (!this.prof) return this.check(call());
    this.check(this.L.gt_event_record(this.ctx, 62));
    this.check(call());
    this.check(this.L.gt_event_record(this.ctx, 63));
    const ms = new Float32Array(1);
    // (gt_event_elapsed_ms is declared nonblocking; a profile is a diagnostic, so block here)
    (this.L.gt_event_elapsed_ms(this.ctx, 62, 63, ms) as unknown as Promise<number>).then(() => {
      const t = this.prof?.get(label) ?? { ms: 0, count: 0 };
      t.ms += ms[0];
      t.count++;
      this.prof?.set(label, t);
    });
  }

  // ---------------------------------------------------------------- memory
  private alloc(bytes: number): { addr: Buf; size: number } {
    const out = new BigUint64Array(1);
    const n = Math.max(bytes, 4);
    this.check(this.L.gt_alloc(this.ctx, BigInt(n), out));
    return { addr: out[0], size: Math.max(256, Math.ceil(n / 256) * 256) };
  }
  private acquirePersistent(bytes: number): Buf {
    return this.alloc(bytes).addr;
  }
  private acquireTransient(bytes: number): Buf {
    const t = this.alloc(bytes);
    this.transients.push(t);
    return t.addr;
  }
  /** Best fit from the region free-list, else a fresh transient. */
  private acquireRecycled(bytes: number): Buf {
    const want = Math.max(256, Math.ceil(Math.max(bytes, 4) / 256) * 256);
    let best = -1;
    for (let i = 0; i < this.regionFree.length; i++) {
      const s = this.regionFree[i].size;
      if (s >= want && (best < 0 || s < this.regionFree[best].size)) best = i;
    }
    if (best < 0) return this.acquireTransient(bytes);
    const [t] = this.regionFree.splice(best, 1);
    this.transients.push(t);
    return t.addr;
  }
  private write(addr: Buf, data: ArrayBufferView) {
    this.check(this.L.gt_write(this.ctx, addr, data, BigInt(data.byteLength)));
  }
  private async read(addr: Buf, out: ArrayBufferView) {
    this.check(await this.L.gt_read(this.ctx, addr, out, BigInt(out.byteLength)));
    this.readback += out.byteLength;
  }
  private uploadU32(values: ArrayLike<number>): Buf {
    const a = asU32(values);
    const addr = this.acquireTransient(a.byteLength);
    this.write(addr, a);
    return addr;
  }
  private uploadF32(values: ArrayLike<number>): Buf {
    const a = Float32Array.from(values);
    const addr = this.acquireTransient(a.byteLength);
    this.write(addr, a);
    return addr;
  }
  /** Externals (parameters, test inputs) get persistent buffers on first use; a frozen one gets no gradient buffer. */
  private entryFor(t: Tensor): Entry {
    let e = this.entries.get(t);
    if (!e) {
      const bytes = t.size * 4;
      e = { data: this.acquirePersistent(bytes), grad: t.requiresGrad ? this.acquirePersistent(bytes) : 0n, bytes, external: true, gradLive: false };
      this.entries.set(t, e);
      this.write(e.data, t.data);
    }
    if (e.external) this.touched.add(t);
    return e;
  }
  private makeOut(shape: number[], prev: Tensor[]): { t: Tensor; e: Entry } {
    const t = Tensor.zeros(shape);
    t._prev = prev;
    const bytes = t.size * 4;
    const e: Entry = { data: this.acquireRecycled(bytes), grad: this.acquireRecycled(bytes), bytes, external: false, gradLive: false };
    this.entries.set(t, e);
    return { t, e };
  }
  /** (grad address or 0, accumulate flag) for a backward kernel about to write into t's gradient. */
  private gradTarget(t: Tensor, e: Entry): [Buf, number] {
    if (e.grad === 0n || (e.external && !t.requiresGrad)) return [0n, 0];
    const acc = e.gradLive ? 1 : 0;
    e.gradLive = true;
    return [e.grad, acc];
  }
  /** The upstream gradient of an op output. Never written means it is exactly zero. */
  private gradSource(e: Entry): Buf {
    if (!e.gradLive) {
      this.check(this.L.gt_zero(this.ctx, e.grad, BigInt(e.bytes)));
      this.gradClearsIssued++;
      e.gradLive = true;
    }
    return e.grad;
  }

  // ---------------------------------------------------------------- data movement
  uploadParams(tensors: Tensor[]) {
    for (const t of tensors) this.write(this.entryFor(t).data, t.data);
  }
  async sync(reads: Tensor[] = []): Promise<void> {
    this.readback = 0;
    for (const t of new Set(reads)) {
      const e = this.entries.get(t);
      if (e) await this.read(e.data, t.data);
    }
    for (const t of this.touched) {
      const e = this.entries.get(t);
      if (!e) continue;
      if (t.requiresGrad && e.grad !== 0n) {
        if (!e.gradLive) { // touched by a forward, never written by a backward: reads back as zeros
          this.check(this.L.gt_zero(this.ctx, e.grad, BigInt(e.bytes)));
          this.gradClearsIssued++;
        }
        if (!this.keptOnDevice.has(t)) await this.read(e.grad, t.grad);
      }
      e.gradLive = false; // the next graph's first writer overwrites
    }
    this.check(await this.L.gt_sync(this.ctx)); // rethrows latched device errors
    this.lastSyncReadbackBytes = this.readback;
    for (const t of this.transients) this.check(this.L.gt_free(this.ctx, t.addr));
    for (const t of this.regionFree) this.check(this.L.gt_free(this.ctx, t.addr));
    this.transients = [];
    this.regionFree = [];
    this.touched.clear();
    this.backwardBegun = false;
    if (this.graphOpen) this.graphSynced = true;
    this.graphOpen = false;
  }
  // deno-lint-ignore require-await
  async reclaimStepTransients(keep: Tensor[] = []): Promise<void> {
    const keepBufs = new Set<Buf>();
    for (const t of keep) {
      const e = this.entries.get(t);
      if (e) keepBufs.add(e.data);
    }
    const retained = [];
    for (const t of this.transients) {
      if (keepBufs.has(t.addr)) retained.push(t);
      else this.check(this.L.gt_free(this.ctx, t.addr));
    }
    this.transients = retained;
    for (const t of this.regionFree) this.check(this.L.gt_free(this.ctx, t.addr));
    this.regionFree = [];
  }

  // ---------------------------------------------------------------- regions (RegionBackend)
  beginRegion(): number {
    this.regionsOpened++;
    return this.transients.length;
  }
  regionCount(): number {
    return this.regionsOpened;
  }
  endRegion(mark: number, keep: Tensor[]): void {
    if (mark > this.transients.length) {
      throw new Error(`endRegion: mark ${mark} is past the ${this.transients.length} live transients; a sync() or reclaim ran inside the region`);
    }
    const keepBufs = new Set<Buf>();
    for (const t of keep) {
      const e = this.entries.get(t);
      if (e) {
        keepBufs.add(e.data);
        keepBufs.add(e.grad);
      }
    }
    const retained = this.transients.slice(0, mark);
    for (const t of this.transients.slice(mark)) (keepBufs.has(t.addr) ? retained : this.regionFree).push(t);
    this.transients = retained;
  }
  seedGradFrom(dst: Tensor, src: Tensor): void {
    this.ensureBackwardBegun();
    const ed = this.entries.get(dst), es = this.entries.get(src);
    if (!ed || !es) throw new Error("seedGradFrom: tensor has no GPU buffers");
    if (dst.size !== src.size) throw new Error(`seedGradFrom: size mismatch ${dst.size} vs ${src.size}`);
    this.check(this.L.gt_copy(this.ctx, ed.grad, this.gradSource(es), BigInt(src.size * 4)));
    ed.gradLive = true;
  }
  seedGradFromHost(t: Tensor) {
    this.ensureBackwardBegun();
    const e = this.entries.get(t);
    if (!e) throw new Error("seedGradFromHost: tensor has no GPU buffers");
    this.write(e.grad, t.grad);
    e.gradLive = true;
  }
  private beginForwardOp() {
    this.backwardBegun = false;
    this.graphSynced = false;
    this.graphOpen = true;
  }
  private ensureBackwardBegun() {
    if (this.backwardBegun) return;
    if (this.graphSynced) {
      throw new Error(
        "backward over a graph built before a sync(): that sync recycled the graph's gradient buffers and discarded " +
          "their clears, so this backward would accumulate into pool garbage",
      );
    }
    this.backwardBegun = true;
  }

  // ---------------------------------------------------------------- raw buffers (optimizers, checkpoints)
  buffersFor(t: Tensor): { data: Buf; grad: Buf } {
    const e = this.entryFor(t);
    return { data: e.data, grad: e.grad };
  }
  keepGradOnDevice(t: Tensor) {
    this.keptOnDevice.add(t);
  }
  createStateBuffer(bytes: number): Buf {
    const out = new BigUint64Array(1);
    this.check(this.L.gt_alloc_state(this.ctx, BigInt(bytes), out));
    return out[0];
  }
  writeStateBuffer(buf: Buf, values: Float32Array) {
    this.write(buf, values);
  }
  async readStateBuffer(buf: Buf, elems: number): Promise<Float32Array> {
    const out = new Float32Array(elems);
    await this.read(buf, out);
    return out;
  }
  /** Checkpoint reads that overlap the next step: start now, fence before the optimizer, finish when convenient. */
  readAsync(buf: Buf, bytes: number): bigint {
    const t = new BigUint64Array(1);
    this.check(this.L.gt_read_async(this.ctx, buf, BigInt(bytes), t));
    return t[0];
  }
  readFence() {
    this.check(this.L.gt_read_fence(this.ctx));
  }
  async readFinish(ticket: bigint, out: ArrayBufferView) {
    this.check(await this.L.gt_read_finish(this.ctx, ticket, out, BigInt(out.byteLength)));
  }
  /** For the optimizers below. */
  _ffi(): { L: Lib; ctx: Deno.PointerValue; check: (s: number) => void } {
    return { L: this.L, ctx: this.ctx, check: (s) => this.check(s) };
  }

  // ---------------------------------------------------------------- ops (OpsBackend)
  private gemm(kind: keyof typeof KIND, accum: number, M: number, N: number, K: number, a: Buf, b: Buf, c: Buf) {
    this.run(`gemm ${kind}`, () => this.L.gt_gemm(this.ctx, KIND[kind], accum, M, N, K, a, b, c));
  }
  linear(x: Tensor, w: Tensor): Tensor {
    this.beginForwardOp();
    const [T, inDim] = x.shape, outDim = w.shape[0];
    const ex = this.entryFor(x), ew = this.entryFor(w);
    const { t: out, e: eo } = this.makeOut([T, outDim], [x, w]);
    this.gemm("NT", 0, T, outDim, inDim, ex.data, ew.data, eo.data);
    out._backward = () => {
      this.ensureBackwardBegun();
      const go = this.gradSource(eo);
      const [gx, ax] = this.gradTarget(x, ex);
      if (gx) this.gemm("NN", ax, T, inDim, outDim, go, ew.data, gx);
      if (w.requiresGrad) { // a frozen base skips dW (src/backend/webgpu.ts:898-901)
        const [gw, aw] = this.gradTarget(w, ew);
        if (gw) this.gemm("TN", aw, outDim, inDim, T, go, ex.data, gw);
      }
    };
    return out;
  }
  private elementwise(op: keyof typeof EW, a: Tensor, b: Tensor | null, c: number): Tensor {
    this.beginForwardOp();
    const ea = this.entryFor(a), eb = b ? this.entryFor(b) : null;
    const { t: out, e: eo } = this.makeOut(a.shape, b ? [a, b] : [a]);
    const n = BigInt(a.size), code = EW[op];
    this.run(op, () => this.L.gt_ew_fwd(this.ctx, code, n, ea.data, eb ? eb.data : 0n, c, eo.data));
    out._backward = () => {
      this.ensureBackwardBegun();
      const go = this.gradSource(eo);
      const [ga, aa] = this.gradTarget(a, ea);
      if (eb && eb === ea) { // add(t,t) / mul(t,t): both contributions land in one write
        this.run(op + " bwd", () => this.L.gt_ew_bwd(this.ctx, code, n, ea.data, ea.data, c, go, ga, aa, ga, aa));
        return;
      }
      const [gb, ab] = eb && b ? this.gradTarget(b, eb) : [0n, 0];
      this.run(op + " bwd", () => this.L.gt_ew_bwd(this.ctx, code, n, ea.data, eb ? eb.data : 0n, c, go, ga, aa, gb, ab));
    };
    return out;
  }
  add(a: Tensor, b: Tensor) {
    return this.elementwise("add", a, b, 0);
  }
  mul(a: Tensor, b: Tensor) {
    return this.elementwise("mul", a, b, 0);
  }
  silu(x: Tensor) {
    return this.elementwise("silu", x, null, 0);
  }
  gelu(x: Tensor) {
    return this.elementwise("gelu", x, null, 0);
  }
  scale(x: Tensor, c: number) {
    return this.elementwise("scale", x, null, c);
  }
  private rmsNormRows(x: Tensor, w: Tensor, rows: number, d: number, eps: number, shape: number[]): Tensor {
    this.beginForwardOp();
    const ex = this.entryFor(x), ew = this.entryFor(w);
    const { t: out, e: eo } = this.makeOut(shape, [x, w]);
    const rinv = this.acquireRecycled(rows * 4);
    this.run("rmsNorm", () => this.L.gt_rmsnorm_fwd(this.ctx, rows, d, ex.data, ew.data, eps, eo.data, rinv));
    out._backward = () => {
      this.ensureBackwardBegun();
      const go = this.gradSource(eo);
      const [gx, ax] = this.gradTarget(x, ex);
      const [gw, aw] = w.requiresGrad ? this.gradTarget(w, ew) : [0n, 0];
      this.run("rmsNorm bwd", () => this.L.gt_rmsnorm_bwd(this.ctx, rows, d, ex.data, ew.data, rinv, go, gx, ax, gw, aw));
    };
    return out;
  }
  rmsNorm(x: Tensor, weight: Tensor, eps: number) {
    const [T, d] = x.shape;
    return this.rmsNormRows(x, weight, T, d, eps, [T, d]);
  }
  rmsNormHeads(x: Tensor, weight: Tensor, T: number, H: number, hd: number, eps: number) {
    return this.rmsNormRows(x, weight, T * H, hd, eps, [T, H * hd]);
  }
  embedding(weight: Tensor, ids: number[]): Tensor {
    this.beginForwardOp();
    const d = weight.shape[1], T = ids.length;
    const ew = this.entryFor(weight);
    const idBuf = this.uploadU32(ids);
    const { t: out, e: eo } = this.makeOut([T, d], [weight]);
    this.run("embedding", () => this.L.gt_embedding_fwd(this.ctx, T, d, ew.data, idBuf, eo.data));
    out._backward = () => {
      this.ensureBackwardBegun();
      if (!weight.requiresGrad || ew.grad === 0n) return;
      const go = this.gradSource(eo);
      if (!ew.gradLive) { // the scatter-add needs a defined starting value
        this.check(this.L.gt_zero(this.ctx, ew.grad, BigInt(ew.bytes)));
        this.gradClearsIssued++;
        ew.gradLive = true;
      }
      this.run("embedding bwd", () => this.L.gt_embedding_bwd(this.ctx, T, d, go, idBuf, ew.grad));
    };
    return out;
  }
  private checkT(T: number, rows: number, where: string) {
    const [b, sl] = this.batch;
    if (b && T !== b * sl) throw new Error(`${where}: T=${T} but the batch is ${b} x ${sl}`);
    if (!b && T !== rows) throw new Error(`${where}: T=${T} but the tensor has ${rows} rows`);
  }
  rope(x: Tensor, T: number, H: number, hd: number, base: number, posOffset: number): Tensor {
    this.beginForwardOp();
    this.checkT(T, x.shape[0], "rope");
    const ex = this.entryFor(x);
    const { t: out, e: eo } = this.makeOut([T, H * hd], [x]);
    this.run("rope", () => this.L.gt_rope_fwd(this.ctx, T, H, hd, base, posOffset, ex.data, eo.data));
    out._backward = () => {
      this.ensureBackwardBegun();
      const go = this.gradSource(eo);
      const [gx, ax] = this.gradTarget(x, ex);
      this.run("rope bwd", () => this.L.gt_rope_bwd(this.ctx, T, H, hd, base, posOffset, go, gx, ax));
    };
    return out;
  }
  attention(q: Tensor, k: Tensor, v: Tensor, T: number, Hq: number, Hkv: number, hd: number, window: number): Tensor {
    this.beginForwardOp();
    this.checkT(T, q.shape[0], "attention");
    const eq = this.entryFor(q), ek = this.entryFor(k), ev = this.entryFor(v);
    const { t: out, e: eo } = this.makeOut([T, Hq * hd], [q, k, v]);
    const lse = this.acquireRecycled(Hq * T * 4);
    this.run("attention", () => this.L.gt_attention_fwd(this.ctx, T, Hq, Hkv, hd, window, eq.data, ek.data, ev.data, eo.data, lse));
    out._backward = () => {
      this.ensureBackwardBegun();
      const go = this.gradSource(eo);
      const [gq, aq] = this.gradTarget(q, eq), [gk, ak] = this.gradTarget(k, ek), [gv, av] = this.gradTarget(v, ev);
      this.run("attention bwd", () =>
        this.L.gt_attention_bwd(this.ctx, T, Hq, Hkv, hd, window, eq.data, ek.data, ev.data, eo.data, lse, go, gq, aq, gk, ak, gv, av));
    };
    return out;
  }
  private nseq() {
    return this.batch[0] || 1;
  }
  /** The scalar loss tensor plus its device-side companions: [1+nseq] losses and [nseq] 1/kept. */
  private lossOut(prev: Tensor[]): { loss: Tensor; e: Entry; invKept: Buf } {
    const loss = Tensor.zeros([1]);
    loss._prev = prev;
    const e: Entry = { data: this.acquireRecycled((1 + this.nseq()) * 4), grad: this.acquireRecycled(4), bytes: 4, external: false, gradLive: false };
    this.entries.set(loss, e);
    return { loss, e, invKept: this.acquireRecycled(this.nseq() * 4) };
  }
  /** backward(loss, seed) wrote the seed into the host grad array; push it to the device (webgpu.ts:1316-1320). */
  private lossGrad(loss: Tensor, e: Entry): Buf {
    if (!e.gradLive) {
      this.write(e.grad, loss.grad.subarray(0, 1));
      e.gradLive = true;
    }
    return e.grad;
  }
  crossEntropy(logits: Tensor, targets: number[], _kept: number): Tensor {
    // `_kept` was counted above the dispatch; the device derives the same count from the uploaded targets
    this.beginForwardOp();
    const [T, V] = logits.shape;
    const el = this.entryFor(logits);
    const tgt = this.uploadU32(targets);
    const stats = this.acquireRecycled(T * 16);
    const { loss, e: eo, invKept } = this.lossOut([logits]);
    this.run("crossEntropy", () => this.L.gt_ce_fwd(this.ctx, T, V, el.data, tgt, stats, eo.data, invKept));
    loss._backward = () => {
      this.ensureBackwardBegun();
      const seed = this.lossGrad(loss, eo);
      const [gl, al] = this.gradTarget(logits, el);
      this.run("crossEntropy bwd", () => this.L.gt_ce_bwd(this.ctx, T, V, el.data, tgt, stats, invKept, seed, gl, al));
    };
    return loss;
  }
  fusedCrossEntropy(hidden: Tensor, w: Tensor, targets: number[], chunk: number, _kept: number): Tensor {
    this.beginForwardOp();
    const [T, H] = hidden.shape, V = w.shape[0];
    const eh = this.entryFor(hidden), ew = this.entryFor(w);
    const tgt = this.uploadU32(targets);
    const run = this.acquireRecycled(T * 12);
    const ch = this.acquireRecycled(T * Math.min(chunk, V) * 4);
    const { loss, e: eo, invKept } = this.lossOut([hidden, w]);
    const rowOf = (v0: number) => ew.data + BigInt(v0 * H * 4); // a byte offset into a gt_buf is allowed
    for (let v0 = 0; v0 < V; v0 += chunk) {
      const n = Math.min(chunk, V - v0);
      this.gemm("NT", 0, T, n, H, eh.data, rowOf(v0), ch);
      this.run("ce chunk stats", () => this.L.gt_ce_chunk_stats(this.ctx, T, n, v0, v0 === 0 ? 1 : 0, ch, tgt, run));
    }
    this.run("ce loss", () => this.L.gt_ce_loss_from_stats(this.ctx, T, run, tgt, eo.data, invKept));
    loss._backward = () => {
      this.ensureBackwardBegun();
      const seed = this.lossGrad(loss, eo);
      let [gh, ah] = this.gradTarget(hidden, eh);
      const [gw, aw] = w.requiresGrad ? this.gradTarget(w, ew) : [0n, 0];
      for (let v0 = 0; v0 < V; v0 += chunk) {
        const n = Math.min(chunk, V - v0);
        this.gemm("NT", 0, T, n, H, eh.data, rowOf(v0), ch);
        this.run("ce chunk grad", () => this.L.gt_ce_chunk_grad(this.ctx, T, n, v0, ch, tgt, run, invKept, seed));
        if (gh) {
          this.gemm("NN", ah, T, H, n, ch, rowOf(v0), gh);
          ah = 1;
        }
        if (gw) this.gemm("TN", aw, n, H, T, ch, eh.data, gw + BigInt(v0 * H * 4)); // each span written by one product
      }
    };
    return loss;
  }
  softCrossEntropy(logits: Tensor, teacherIds: number[], teacherProbs: number[], k: number, _kept: number): Tensor {
    this.beginForwardOp();
    const [T, V] = logits.shape;
    const el = this.entryFor(logits);
    const ids = this.uploadU32(teacherIds), probs = this.uploadF32(teacherProbs);
    const stats = this.acquireRecycled(T * 16);
    const { loss, e: eo, invKept } = this.lossOut([logits]);
    this.run("softCrossEntropy", () => this.L.gt_soft_ce_fwd(this.ctx, T, V, k, el.data, ids, probs, stats, eo.data, invKept));
    loss._backward = () => {
      this.ensureBackwardBegun();
      const seed = this.lossGrad(loss, eo);
      const [gl, al] = this.gradTarget(logits, el);
      this.run("softCrossEntropy bwd", () => this.L.gt_soft_ce_bwd(this.ctx, T, V, k, el.data, ids, probs, stats, invKept, seed, gl, al));
    };
    return loss;
  }
}

/** `initWebGPU()` (src/backend/webgpu.ts:1823-1870): a backend, or null when there is no GPU so suites can SKIP. */
export function initCuda(device = 0, precision: keyof typeof PRECISION = "fp32"): CudaBackend | null {
  try {
    return new CudaBackend(device, precision);
  } catch {
    return null;
  }
}
/** src/backend/webgpu.ts:1812-1821. */
export function requireGPU(purpose: string, device = 0, precision: keyof typeof PRECISION = "fp32"): CudaBackend {
  const gpu = initCuda(device, precision);
  if (!gpu) throw new Error(`no GPU adapter found, and ${purpose} needs one`);
  return gpu;
}

// ------------------------------------------------------------------ optimizers
/** AdamWGpu (src/backend/adamw-gpu.ts:131-251) on gt_adamw_*: same public methods. */
export class AdamWCuda {
  private h: bigint;
  constructor(private gpu: CudaBackend, private params: Tensor[], private baseLr: number,
    o: { beta1?: number; beta2?: number; eps?: number; weightDecay?: number; clip?: number } = {}) {
    const { L, ctx, check } = gpu._ffi();
    const n = params.length;
    const data = new BigUint64Array(n), grad = new BigUint64Array(n), sizes = new BigUint64Array(n);
    params.forEach((p, i) => {
      const b = gpu.buffersFor(p);
      gpu.keepGradOnDevice(p);
      data[i] = b.data; grad[i] = b.grad; sizes[i] = BigInt(p.size);
    });
    const out = new BigUint64Array(1);
    check(L.gt_adamw_create(ctx, n, data, grad, sizes, baseLr, o.beta1 ?? 0.9, o.beta2 ?? 0.999, o.eps ?? 1e-8, o.weightDecay ?? 0, o.clip ?? 1, out));
    this.h = out[0];
  }
  setLrScale(s: number) {
    const { L, ctx, check } = this.gpu._ffi();
    check(L.gt_adamw_set_lr(ctx, this.h, this.baseLr * s));
  }
  zeroGrad() {} // gradients restart at the next step's first write
  recordStep() {
    const { L, ctx, check } = this.gpu._ffi();
    this.gpu.readFence();
    check(L.gt_adamw_step(ctx, this.h));
  }
  async syncWeightsToHost() {
    await this.gpu.sync(this.params);
  }
  async exportState() {
    const { L, ctx, check } = this.gpu._ffi();
    const m: Float32Array[] = [], v: Float32Array[] = [];
    for (let i = 0; i < this.params.length; i++) {
      const a = new BigUint64Array(1), b = new BigUint64Array(1);
      check(L.gt_adamw_state(ctx, this.h, i, a, b));
      m.push(await this.gpu.readStateBuffer(a[0], this.params[i].size));
      v.push(await this.gpu.readStateBuffer(b[0], this.params[i].size));
    }
    const t = new Int32Array(1);
    check(L.gt_adamw_get_t(ctx, this.h, t));
    return { m, v, t: t[0] };
  }
  importState(s: { m: Float32Array[]; v: Float32Array[]; t: number }) {
    const { L, ctx, check } = this.gpu._ffi();
    for (let i = 0; i < this.params.length; i++) {
      const a = new BigUint64Array(1), b = new BigUint64Array(1);
      check(L.gt_adamw_state(ctx, this.h, i, a, b));
      this.gpu.writeStateBuffer(a[0], s.m[i]);
      this.gpu.writeStateBuffer(b[0], s.v[i]);
    }
    check(L.gt_adamw_set_t(ctx, this.h, s.t));
  }
}

/** MuonGpu (src/backend/muon-gpu.ts:351-470) on gt_muon_*: Muon on the hidden matrices, AdamW on the aux group. */
export class MuonCuda {
  private h: bigint;
  readonly aux: AdamWCuda;
  constructor(private gpu: CudaBackend, private muonParams: Tensor[], auxParams: Tensor[],
    o: { lr: number; momentum?: number; nesterov?: boolean; nsSteps?: number; aux: { lr: number; weightDecay?: number; clip?: number; beta1?: number; beta2?: number } }) {
    const { L, ctx, check } = gpu._ffi();
    this.aux = new AdamWCuda(gpu, auxParams, o.aux.lr, o.aux);
    const n = muonParams.length;
    const data = new BigUint64Array(n), grad = new BigUint64Array(n), rows = new Int32Array(n), cols = new Int32Array(n);
    muonParams.forEach((p, i) => {
      const b = gpu.buffersFor(p);
      gpu.keepGradOnDevice(p);
      data[i] = b.data; grad[i] = b.grad; rows[i] = p.shape[0]; cols[i] = p.shape[1];
    });
    const out = new BigUint64Array(1);
    check(L.gt_muon_create(ctx, n, data, grad, rows, cols, o.lr, o.momentum ?? 0.95, (o.nesterov ?? true) ? 1 : 0, o.nsSteps ?? 5, out));
    this.h = out[0];
    this.baseLr = o.lr;
  }
  private baseLr: number;
  setLrScale(s: number) {
    const { L, ctx, check } = this.gpu._ffi();
    check(L.gt_muon_set_lr(ctx, this.h, this.baseLr * s));
    this.aux.setLrScale(s);
  }
  zeroGrad() {}
  recordStep() {
    const { L, ctx, check } = this.gpu._ffi();
    this.gpu.readFence();
    check(L.gt_muon_step(ctx, this.h));
    this.aux.recordStep();
  }
  async syncWeightsToHost() {
    await this.gpu.sync(this.muonParams);
    await this.aux.syncWeightsToHost();
  }
  async exportState() {
    const { L, ctx, check } = this.gpu._ffi();
    const muonMomentum: Float32Array[] = [];
    for (let i = 0; i < this.muonParams.length; i++) {
      const b = new BigUint64Array(1);
      check(L.gt_muon_state(ctx, this.h, i, b));
      muonMomentum.push(await this.gpu.readStateBuffer(b[0], this.muonParams[i].size));
    }
    const a = await this.aux.exportState();
    return { muonMomentum, adamM: a.m, adamV: a.v, adamT: a.t };
  }
  importState(s: { muonMomentum: Float32Array[]; adamM: Float32Array[]; adamV: Float32Array[]; adamT: number }) {
    const { L, ctx, check } = this.gpu._ffi();
    for (let i = 0; i < this.muonParams.length; i++) {
      const b = new BigUint64Array(1);
      check(L.gt_muon_state(ctx, this.h, i, b));
      this.gpu.writeStateBuffer(b[0], s.muonMomentum[i]);
    }
    this.aux.importState({ m: s.adamM, v: s.adamV, t: s.adamT });
  }
}

// ------------------------------------------------------------------ entry points used by other callers
// The remaining functions of the header are reached through CudaBackend._ffi() by the callers that need them:
//   batched replay (src/backend/train-cuda.ts, twin of train-gpu.ts:162-258): gt_set_batch, gt_graph_begin / gt_graph_end /
//     gt_graph_launch / gt_graph_destroy, with ids and targets rewritten by gt_write before each launch;
//   device-resident corpus: gt_tokens_max once at upload, then gt_gather_windows as the first recorded call of the step;
//   data parallel: gt_dp_unique_id, gt_dp_init, gt_dp_allreduce_start per gradient bucket, gt_dp_wait (or gt_dp_wait_host
//     with a limit) before the optimizer, gt_dp_reserve_sms, gt_muon_set_sharded, gt_dp_destroy;
//   adapters: gt_gemm_scaled, gt_gemm_grouped_scaled, gt_gemm2 / gt_gemm_multi (the adapter-carrying projection as one product);
//   fused kernels of the launch-deferring mirror: gt_glu_fwd / gt_glu_bwd, gt_glu_linear_fwd, gt_add_rmsnorm_fwd,
//     gt_rmsnorm_bwd_add, gt_gemm_grouped (projections of one input; the weight gradients of a layer), gt_linear_rope_grouped,
//     gt_rmsnorm_heads_rope_fwd and gt_attention_bwd_rope (the rotary embedding applied by its neighbours);
//   gt_newton_schulz (newtonSchulzGpu, src/backend/muon-gpu.ts:258-282), gt_attention_bwd_static, gt_selftest_bounded_wait.
// gguf_trainer_b200/train.py (CudaStep, DataParallel), ingest.py and lora.py show each sequence of calls.
