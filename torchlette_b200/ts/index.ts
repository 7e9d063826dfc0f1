/**
 * torchlette `cuda` backend for the quantized-weight matmul path.
 *
 * Drop this directory into a torchlette checkout as `src/backend/cuda/`.  It is the TypeScript
 * face of libtlcuda.so (through the N-API addon built from csrc/napi/tl_napi.c) and mirrors,
 * name for name, the pieces of the webgpu backend this path uses:
 *
 *   Backend / BackendOps                      src/backend/types.ts:340-745
 *   matmul seam / matmulQuantizedB            src/backend/webgpu/ops/matmul-ops.ts:42-182
 *   dispatchQuantizedGemvNT                   src/backend/webgpu/matmul/dispatch.ts:875-931
 *   dispatchDequantizeInt8Grouped             src/backend/webgpu/matmul/dispatch.ts:949-1037
 *   dispatchMatmul / dispatchMatmulDirect /
 *     planBareMatmul                          src/backend/webgpu/dispatch.ts:814-1060
 *   route counters                            src/backend/webgpu/matmul/dispatch.ts:833-864, 943-947
 *   per-shape tuning probes                   src/backend/webgpu/matmul/dispatch.ts:79-141
 *   pretuneMatmulShapes / autotune flag       src/backend/webgpu/matmul/dispatch.ts:405-578
 *   exportTuningCache / importTuningCache     src/backend/webgpu/matmul/autotune.ts:309-329
 *   createQuantizedWeight                     src/engine/engine.ts:2041-2149
 *
 * There is no WebGPU or CPU fallback in here: if the addon or a B200 is missing, initCuda()
 * returns false and every op throws.
 *
 * This file has not been executed or type-checked where it was written (no node toolchain
 * there); it is a thin mapping onto the addon, whose argument handling is tested against a
 * fake N-API, and onto the C ABI, which the parity tests exercise from Python.
 */
import type { Backend, BackendOps, BackendTensor, DType, StorageFormat } from "../types";
import { registerBackend } from "../registry";
import type { EpilogueConfig } from "../webgpu/matmul/types";

type Handle = unknown; // an addon external: context or device buffer
type DevPtr = Handle | bigint | null;

// eslint-disable-next-line @typescript-eslint/no-var-requires
let addon: any = null;
let ctx: Handle | null = null;
let initError: string | null = null;

const DTYPE_ID: Record<string, number> = { f32: 0, f16: 1, bf16: 2 };
const DTYPE_BYTES: Record<string, number> = { f32: 4, f16: 2, bf16: 2, u32: 4, u16: 2, i8: 1 };
const UNARY: Record<string, number> = { relu: 1, silu: 2, sigmoid: 3, tanh: 4, gelu: 5, gelu_tanh: 5, gelu_erf: 6 };
const BINARY: Record<string, number> = { add: 1, sub: 2, mul: 3 };
const COUNTER = { qgemv: 0, dequant: 1, gemvEpilogue: 2, qgemm: 3, launches: 4, gemv: 5, tiled: 6 } as const;
const FAMILY_NAME: Record<number, string> = { 1: "qgemv", 2: "qgemm", 3: "matmul" };

/** Device tensor: BackendTensor (types.ts:5-27) + the addon's buffer handle. */
export interface CudaTensor extends BackendTensor {
  buffer: Handle;
  nbytes: number;
  transposed: boolean; // the [K,N] view of a contiguous [N,K] buffer (views.ts:925-933 keeps format/scales)
  scales?: CudaTensor;
}

/** A kernel choice: [family, kernel, p0, p1, p2, p3] (tl_variant). */
export type CudaVariantChoice = [number, number, number, number, number, number];
export interface CudaPlanReceipt {
  family: string; variant: string; choice: CudaVariantChoice; grid: [number, number, number]; block: number;
  splitK: number; fromTuningCache: boolean; epilogueEngaged: boolean;
}

export function initCuda(device = 0): boolean {
  if (ctx !== null) return true;
  try {
    addon = require("./tlcuda.node");
    ctx = addon.ctxCreate(device);
    return true;
  } catch (e) {
    initError = String(e);
    return false;
  }
}
export const getCudaInitError = (): string | null => initError;
export const syncCuda = (): void => addon.sync(need());
export const getGpuUncapturedErrorCount = (): number => addon.asyncErrorCount(need());
export function destroyCuda(): void {
  if (ctx !== null) addon.ctxDestroy(ctx);
  ctx = null;
}
function need(): Handle {
  if (ctx === null) throw new Error(`cuda backend unavailable: ${initError ?? "initCuda() was not called"}`);
  return ctx;
}
const numel = (shape: number[]): number => shape.reduce((a, b) => a * b, 1);

function makeTensor(shape: number[], dtype: string, buffer: Handle, nbytes: number, owns = true): CudaTensor {
  const t: any = { shape: shape.slice(), dtype, buffer, nbytes, ownsBuffer: owns, transposed: false };
  t.toArray = () => Array.from(readSync(t));
  t.destroy = () => {
    // an owning handle frees now; a dropped one is freed by the addon's finalizer
    if (t.ownsBuffer && t.buffer) addon.free(need(), t.buffer);
    t.buffer = null;
  };
  return t as CudaTensor;
}

/** tensorFromArray (types.ts:341-345): typed arrays upload verbatim (their own bytes, views included). */
export function tensorFromArray(values: ArrayBufferView | number[], shape: number[], dtype: string = "f32"): CudaTensor {
  const host: ArrayBufferView = Array.isArray(values) ? Float32Array.from(values) : values;
  const nbytes = host.byteLength;
  if (nbytes !== numel(shape) * DTYPE_BYTES[dtype]) throw new Error(`tensorFromArray: ${nbytes} bytes for shape [${shape}] of ${dtype}`);
  const buf: Handle = addon.alloc(need(), nbytes);
  addon.upload(need(), buf, host);
  return makeTensor(shape, dtype, buf, nbytes);
}
export function empty(shape: number[], dtype: string): CudaTensor {
  const nbytes = numel(shape) * DTYPE_BYTES[dtype];
  return makeTensor(shape, dtype, addon.alloc(need(), nbytes), nbytes);
}
function hostArrayFor(t: CudaTensor): Float32Array | Uint16Array | Uint32Array | Int8Array {
  const n = numel(t.shape);
  return t.dtype === "f32" ? new Float32Array(n) : t.dtype === "u32" ? new Uint32Array(n) : t.dtype === "i8" ? new Int8Array(n) : new Uint16Array(n);
}
/** Blocking read (tests, toArray). */
export function readSync(t: CudaTensor) {
  if (t.transposed) throw new Error("read: materialize the transposed view first (contiguous)");
  const host = hostArrayFor(t);
  addon.download(need(), host, t.buffer);
  return host;
}
/** BackendOps.read (types.ts:346): the JS thread is not blocked while the copy drains. */
export async function read(t: CudaTensor) {
  if (t.transposed) throw new Error("read: materialize the transposed view first (contiguous)");
  return (await addon.downloadAsync(need(), hostArrayFor(t), t.buffer)) as ReturnType<typeof hostArrayFor>;
}
export function transpose(t: CudaTensor): CudaTensor {
  const s = t.shape;
  const v = makeTensor([...s.slice(0, -2), s[s.length - 1], s[s.length - 2]], t.dtype as string, t.buffer, t.nbytes, false);
  v.format = t.format;
  v.scales = t.scales;
  v.transposed = !t.transposed;
  return v;
}

// ---- companion ops: the unfused forms of what the epilogue fuses ---------------------------
function unaryOp(op: number, t: CudaTensor, outDtype?: string): CudaTensor {
  const src = t.transposed ? contiguous(t) : t;
  const out = empty(src.shape, outDtype ?? (src.dtype as string));
  addon.unaryOp(need(), op, src.buffer, DTYPE_ID[src.dtype as string], out.buffer, DTYPE_ID[out.dtype as string], numel(src.shape));
  if (src !== t) src.destroy();
  return out;
}
export const relu = (t: CudaTensor): CudaTensor => unaryOp(UNARY.relu, t);
export const silu = (t: CudaTensor): CudaTensor => unaryOp(UNARY.silu, t);
export const sigmoid = (t: CudaTensor): CudaTensor => unaryOp(UNARY.sigmoid, t);
export const tanh = (t: CudaTensor): CudaTensor => unaryOp(UNARY.tanh, t);
export const gelu = (t: CudaTensor, o?: { approximate?: "tanh" | "none" }): CudaTensor =>
  unaryOp(o?.approximate === "none" ? UNARY.gelu_erf : UNARY.gelu_tanh, t);
export const cast = (t: CudaTensor, dtype: string): CudaTensor => unaryOp(0, t, dtype);
function binaryOp(name: "add" | "sub" | "mul", a: CudaTensor, b: CudaTensor): CudaTensor {
  if (a.transposed || b.transposed) throw new Error(`${name}: materialize transposed views first (contiguous)`);
  const cols = a.shape[a.shape.length - 1];
  const rows = numel(a.shape.slice(0, -1));
  const isRow = a.shape.length > 1 && b.shape.length === 1 && b.shape[0] === cols;
  if (!isRow && (b.shape.length !== a.shape.length || b.shape.some((d, i) => d !== a.shape[i])))
    throw new Error(`${name}: b must have a's shape or be its last dim`);
  const out = empty(a.shape, a.dtype as string);
  addon.binaryOp(need(), BINARY[name], a.buffer, DTYPE_ID[a.dtype as string], b.buffer, DTYPE_ID[b.dtype as string], out.buffer,
                 DTYPE_ID[out.dtype as string], rows, cols, isRow ? 1 : 0);
  return out;
}
export const add = (a: CudaTensor, b: CudaTensor): CudaTensor => binaryOp("add", a, b);
export const sub = (a: CudaTensor, b: CudaTensor): CudaTensor => binaryOp("sub", a, b);
export const mul = (a: CudaTensor, b: CudaTensor): CudaTensor => binaryOp("mul", a, b);
/** contiguous (types.ts): materializes a transposed view; a packed weight has no element-wise transposition. */
export function contiguous(t: CudaTensor): CudaTensor {
  if (t.format?.packing) throw new Error("contiguous: a packed weight has no element-wise transposition");
  if (!t.transposed) return unaryOp(0, t);
  const out = empty(t.shape, t.dtype as string);
  const rows = t.shape[t.shape.length - 1], cols = t.shape[t.shape.length - 2]; // of the stored buffer
  addon.transpose2d(need(), t.buffer, out.buffer, 1, rows, cols, DTYPE_BYTES[t.dtype as string]);
  return out;
}

// ---- the other ops of a decode step (packages/qwen3-browser/src/model.ts:220-420) ------------
/** rmsnorm (src/frontend/tensor.ts:363-367): x * rsqrt(mean(x^2) + eps) * weight over the last dim. */
export function rmsnorm(x: CudaTensor, weight: CudaTensor, eps = 1e-5): CudaTensor {
  const cols = x.shape[x.shape.length - 1];
  const out = empty(x.shape, x.dtype as string);
  addon.rmsnorm(need(), x.buffer, DTYPE_ID[x.dtype as string], weight.buffer, DTYPE_ID[weight.dtype as string], out.buffer,
                DTYPE_ID[out.dtype as string], numel(x.shape) / cols, cols, eps);
  return out;
}
/** fusedRoPE (src/backend/types.ts:593-598; kernel semantics src/backend/webgpu/rope-kernel.ts:1-93). */
export function fusedRoPE(qk: CudaTensor, cos: CudaTensor, sin: CudaTensor,
                          config: { seqLen: number; headDim: number; sinScale?: number; cosOffset?: number; sinOffset?: number }): CudaTensor {
  const out = empty(qk.shape, qk.dtype as string);
  addon.rope(need(), qk.buffer, DTYPE_ID[qk.dtype as string], cos.buffer, sin.buffer, out.buffer,
             numel(qk.shape) / (config.seqLen * config.headDim), config.seqLen, config.headDim, config.sinScale ?? 1, config.cosOffset ?? 0,
             config.sinOffset ?? 0);
  return out;
}
/** One query token per sequence against a KV cache (model.ts:292-312): q [B,H,1,D], caches [B,kvH,cap,D]. */
export function decodeAttention(q: CudaTensor, kCache: CudaTensor, vCache: CudaTensor, kvLen: number, scale: number,
                                mask?: CudaTensor): CudaTensor {
  const [b, h] = q.shape, d = q.shape[q.shape.length - 1];
  const out = empty([b, 1, h * d], q.dtype as string);
  addon.decodeAttention(need(), q.buffer, kCache.buffer, vCache.buffer, out.buffer, DTYPE_ID[q.dtype as string], b, h, kCache.shape[1], d, kvLen,
                        kCache.shape[2], scale, mask ? mask.buffer : null);
  return out;
}

/** S query positions against (a prefix of) a KV cache, causal (model.ts:284-318): q [B,H,S,D] -> [B,S,H*D]. */
export function attention(q: CudaTensor, kCache: CudaTensor, vCache: CudaTensor, kvLen: number, scale: number, causal = true,
                          mask?: CudaTensor): CudaTensor {
  const [b, h, s, d] = q.shape;
  const out = empty([b, s, h * d], q.dtype as string);
  addon.attention(need(), q.buffer, kCache.buffer, vCache.buffer, out.buffer, DTYPE_ID[q.dtype as string], b, h, kCache.shape[1], s, d, kvLen,
                  kCache.shape[2], scale, mask ? mask.buffer : null, causal ? 1 : 0);
  return out;
}

/** createQuantizedWeight (engine.ts:2041-2149): validate, upload, attach format + scales. */
export function createQuantizedWeight(packed: Uint32Array, scalesBits: Uint16Array | Float32Array, n: number, k: number,
                                      format: StorageFormat & { scaleConvention?: "snorm127" | "direct" }): CudaTensor {
  const packing = format.packing;
  if (!packing) throw new Error("createQuantizedWeight: format.packing is required");
  const perWord = (packing.scheme as string) === "int4-grouped" ? 8 : 4; // int4: the reference's planned second scheme
  if (k % perWord !== 0) throw new Error(`createQuantizedWeight: K=${k} must be divisible by ${perWord}`);
  if (packed.length !== n * (k / perWord)) throw new Error(`createQuantizedWeight: packed length ${packed.length} != ${n * (k / perWord)}`);
  const groups = k / packing.groupSize;
  if (scalesBits.length !== n * groups) throw new Error(`createQuantizedWeight: scales length ${scalesBits.length} != ${n * groups}`);
  const buf: Handle = addon.alloc(need(), packed.byteLength);
  addon.upload(need(), buf, packed);
  const w = makeTensor([n, k], format.elementType, buf, packed.byteLength); // logical [N,K] over packed bytes
  w.format = format;
  w.scales = tensorFromArray(scalesBits, [n, groups], scalesBits instanceof Float32Array ? "f32" : "u16");
  return w;
}
/** quantizeLinearWeight (src/backend/quantize.ts:77-131) through the library's host quantizer. */
export function quantizeLinearWeight(weight: Float32Array, n: number, k: number, groupSize = 64, scheme: "int8-grouped" | "int4-grouped" = "int8-grouped") {
  const packed = new Uint32Array(n * (k / (scheme === "int4-grouped" ? 8 : 4)));
  const scales = new Uint16Array(n * (k / groupSize));
  if (scheme === "int4-grouped") addon.quantizeLinearWeightInt4(weight, n, k, groupSize, packed, scales);
  else addon.quantizeLinearWeight(weight, n, k, groupSize, packed, scales);
  return { packed, scales, n, k, groupSize };
}

function encodeEpilogue(epilogue?: EpilogueConfig, inputs: CudaTensor[] = []) {
  if (!epilogue) return undefined;
  const ops = new Int32Array(4 * epilogue.ops.length);
  epilogue.ops.forEach((op: any, i: number) => {
    const kind = { none: 0, bias: 1, unary: 2, binary: 3, cast: 4 }[op.kind as string]!;
    ops[4 * i] = kind;
    ops[4 * i + 1] = op.kind === "unary" ? UNARY[op.op] ?? 99 : op.kind === "binary" ? BINARY[op.op] ?? 99 : 0;
    ops[4 * i + 2] = op.inputIndex ?? 0;
    ops[4 * i + 3] = op.kind === "cast" ? DTYPE_ID[op.toDtype] : 0;
  });
  return { ops, inputs: inputs.map((t) => t.buffer) };
}

/** tl_quant_desc as the addon takes it: Int32Array [scheme, groupSize, scalesDtype, scaleConvention]. */
function qdesc(format: any): Int32Array {
  const p = format.packing;
  if (p.scheme !== "int8-grouped" && p.scheme !== "int4-grouped") throw new Error(`matmulQuantizedB: unsupported scheme ${p.scheme}`);
  return Int32Array.of(p.scheme === "int4-grouped" ? 2 : 1, p.groupSize, DTYPE_ID[p.scalesDtype], format.scaleConvention === "direct" ? 1 : 0);
}
const defaultQdesc = (groupSize: number, scalesDtype: string): Int32Array => Int32Array.of(1, groupSize, scalesDtype === "f32" ? 0 : 1, 0);

function receipt(r: Int32Array): CudaPlanReceipt {
  const choice = Array.from(r.subarray(0, 6)) as CudaVariantChoice;
  return { family: FAMILY_NAME[r[0]] ?? "?", variant: addon.variantName(Int32Array.from(choice)), choice, grid: [r[6], r[7], r[8]],
           block: r[9], splitK: r[10], fromTuningCache: r[11] !== 0, epilogueEngaged: r[12] === 1 };
}

export interface MatmulOptions {
  outBuffer?: CudaTensor; epilogue?: EpilogueConfig; epilogueInputs?: CudaTensor[]; alpha?: number; outputDtype?: string;
  inputCastA?: "f16" | "bf16"; inputCastB?: "f16" | "bf16";
}

/** matmulQuantizedB (matmul-ops.ts:113-182); every M runs a fused-dequant kernel. */
function matmulQuantizedB(a: CudaTensor, b: CudaTensor, o: MatmulOptions = {}): CudaTensor {
  if (!b.format?.packing || !b.scales) throw new Error("matmulQuantizedB: missing packing/scales on B operand");
  if (!b.transposed) throw new Error("matmulQuantizedB: B must be the transposed view of the [N,K] weight");
  const K = b.shape[b.shape.length - 2], N = b.shape[b.shape.length - 1];
  if (a.shape[a.shape.length - 1] !== K) throw new Error("matmul dimension mismatch");
  const M = numel(a.shape.slice(0, -1));
  const outDtype = o.epilogue?.outputDtype ?? o.outputDtype ?? "f32";
  const out = o.outBuffer ?? empty([...a.shape.slice(0, -1), N], outDtype);
  addon.qmatmulNt(need(), a.buffer, DTYPE_ID[a.dtype as string], b.buffer, b.scales.buffer, out.buffer, DTYPE_ID[outDtype],
                  M, N, K, qdesc(b.format), o.alpha ?? 1.0, encodeEpilogue(o.epilogue, o.epilogueInputs));
  return out;
}

/** dispatchQuantizedGemvNT (dispatch.ts:875-931), same positional arguments after `device`. */
export function dispatchQuantizedGemvNT(a: CudaTensor, packedWeight: CudaTensor, scales: CudaTensor, out: CudaTensor, n: number,
                                        k: number, groupSize: number, outputDtype: DType | "bf16" = "f32", alpha = 1.0): void {
  addon.qgemvNt(need(), a.buffer, DTYPE_ID[a.dtype as string], packedWeight.buffer, scales.buffer, out.buffer, DTYPE_ID[outputDtype],
                1, n, k, defaultQdesc(groupSize, scales.dtype as string), alpha, undefined);
}
/** dispatchDequantizeInt8Grouped (dispatch.ts:949-1037). */
export function dispatchDequantizeInt8Grouped(bq: CudaTensor, scales: CudaTensor, out: CudaTensor, n: number, k: number, groupSize: number): void {
  addon.dequantInt8(need(), bq.buffer, scales.buffer, out.buffer, DTYPE_ID[out.dtype as string], n, k, defaultQdesc(groupSize, scales.dtype as string));
}

export interface DirectMatmulConfig {
  m: number; n: number; k: number; transA: boolean; transB: boolean; batchSize: number;
  batchStrideA: number; batchStrideB: number; batchStrideC: number; outShape: number[];
  dtypeA: "f16" | "f32" | "bf16"; dtypeB?: "f16" | "f32" | "bf16"; outputDtype: DType | "bf16";
  epilogueConfig: EpilogueConfig | undefined; epilogueBuffers: Handle[];
  inputCastA?: "f16" | "bf16"; inputCastB?: "f16" | "bf16"; alpha?: number;
}
const CAST = (c?: string): number => (c ? DTYPE_ID[c] : -1);
/** dispatchMatmulDirect (webgpu/dispatch.ts:968-1060): raw buffers + an explicit geometry. */
export function dispatchMatmulDirect(bufA: DevPtr, bufB: DevPtr, c: DirectMatmulConfig, outBuffer?: CudaTensor): CudaTensor {
  const out = outBuffer ?? empty(c.outShape, c.outputDtype);
  const epi = c.epilogueConfig ? { ...encodeEpilogue(c.epilogueConfig, [])!, inputs: c.epilogueBuffers } : undefined;
  addon.matmul(need(), bufA, bufB, out.buffer, c.m, c.n, c.k, c.batchSize, c.batchStrideA, c.batchStrideB, c.batchStrideC,
               c.transA ? 1 : 0, c.transB ? 1 : 0, c.alpha ?? 1.0, DTYPE_ID[c.dtypeA], DTYPE_ID[c.dtypeB ?? c.dtypeA], DTYPE_ID[c.outputDtype],
               CAST(c.inputCastA), CAST(c.inputCastB), epi, 0);
  return out;
}

/** prepareMatmulInputs (webgpu/dispatch.ts:700-812): geometry of a dense product; a transposed view
 * folds into the trans flag, leading dims are the batch, an operand without them is broadcast. */
function denseGeometry(a: CudaTensor, b: CudaTensor, transA: boolean, transB: boolean) {
  const ta = transA !== a.transposed, tb = transB !== b.transposed; // a flag on a view cancels it
  const as = a.shape.length > 1 ? a.shape : [1, ...a.shape];
  const aLog = transA ? [...as.slice(0, -2), as[as.length - 1], as[as.length - 2]] : as;
  const bLog = transB ? [...b.shape.slice(0, -2), b.shape[b.shape.length - 1], b.shape[b.shape.length - 2]] : b.shape;
  let m = aLog[aLog.length - 2]; const k = aLog[aLog.length - 1], n = bLog[bLog.length - 1];
  if (bLog[bLog.length - 2] !== k) throw new Error("matmul dimension mismatch");
  const batchA = aLog.slice(0, -2), batchB = bLog.slice(0, -2);
  if (batchA.length && batchB.length && (batchA.length !== batchB.length || batchA.some((d, i) => d !== batchB[i])))
    throw new Error("matmul: batch dims must match or be absent on one operand");
  const batchDims = batchA.length ? batchA : batchB;
  let batch = numel(batchDims);
  if ((ta && batchA.length) || (tb && batchB.length)) throw new Error("matmul: a transposed view must be a single matrix");
  const outShape = [...batchDims, m, n];
  if (batch > 1 && !batchB.length && !ta) { m *= batch; batch = 1; } // [rows, K] x [K, N]: one matrix
  return { m, n, k, batch, transA: ta, transB: tb, outShape,
           strideA: batchA.length && batch > 1 ? m * k : 0, strideB: batchB.length && batch > 1 ? k * n : 0, strideC: m * n };
}

/** dispatchMatmul (webgpu/dispatch.ts:859-966): dense or packed B, fused epilogue, cast-on-load. */
export function dispatchMatmul(a: CudaTensor, b: CudaTensor, transA = false, transB = false, outBuffer?: CudaTensor,
                               o: { epilogue?: EpilogueConfig; epilogueInputs?: CudaTensor[]; inputCastA?: "f16" | "bf16";
                                    inputCastB?: "f16" | "bf16"; outputDtype?: string; alpha?: number } = {}): CudaTensor {
  if (b.format?.packing) {
    if (transA) throw new Error("cuda dispatchMatmul: transA with a packed B is not served");
    return matmulQuantizedB(a, transB ? transpose(b) : b, { outBuffer, ...o });
  }
  const g = denseGeometry(a, b, transA, transB);
  const outDtype = o.epilogue?.outputDtype ?? o.outputDtype ?? "f32";
  return dispatchMatmulDirect(a.buffer, b.buffer, {
    m: g.m, n: g.n, k: g.k, transA: g.transA, transB: g.transB, batchSize: g.batch, batchStrideA: g.strideA, batchStrideB: g.strideB,
    batchStrideC: g.strideC, outShape: g.outShape, dtypeA: a.dtype as any, dtypeB: b.dtype as any, outputDtype: outDtype as any,
    epilogueConfig: o.epilogue, epilogueBuffers: (o.epilogueInputs ?? []).map((t) => t.buffer), inputCastA: o.inputCastA,
    inputCastB: o.inputCastB, alpha: o.alpha }, outBuffer);
}

/** planBareMatmul (webgpu/dispatch.ts:814-857): what a bare a @ b would run, or why it is not a
 * bare tiled product ("quantized-operand": the seam routes it; this backend never needs a
 * "contiguous-prologue", transposed views fold into the kernel's flags). */
export function planBareMatmul(a: CudaTensor, b: CudaTensor): CudaPlanReceipt | string {
  if (b.format?.packing) return "quantized-operand";
  const g = denseGeometry(a, b, false, false);
  return receipt(addon.matmul(need(), null, null, null, g.m, g.n, g.k, g.batch, g.strideA, g.strideB, g.strideC, g.transA ? 1 : 0,
                              g.transB ? 1 : 0, 1.0, DTYPE_ID[a.dtype as string], DTYPE_ID[b.dtype as string], 0, -1, -1, undefined, 1));
}
/** planTiledMatmul's quantized counterpart: which kernel a packed product of this geometry runs. */
export function planQuantizedMatmul(m: number, n: number, k: number, aDtype: string, outDtype: string, format: any,
                                    epilogue?: EpilogueConfig): CudaPlanReceipt {
  return receipt(addon.planQmatmul(need(), m, n, k, DTYPE_ID[aDtype], DTYPE_ID[outDtype], qdesc(format), encodeEpilogue(epilogue, [])));
}
/** Explicit MatmulKernelConfig analogue (variants.ts:214-236): force one kernel for every following call. */
export const forceVariant = (choice: CudaVariantChoice | null): void => addon.forceVariant(need(), choice ? Int32Array.from(choice) : null);

// ---- route counters and probes (dispatch.ts:79-141, 833-864, 943-947) ----------------------
export const getQuantGemvDispatchCount = (): number => addon.counterGet(need(), COUNTER.qgemv);
export const getDequantI8DispatchCount = (): number => addon.counterGet(need(), COUNTER.dequant);
export const getGemvEpilogueDispatchCount = (): number => addon.counterGet(need(), COUNTER.gemvEpilogue);
export const getGemvDispatchCount = (): number => addon.counterGet(need(), COUNTER.gemv);
export const getQuantGemmDispatchCount = (): number => addon.counterGet(need(), COUNTER.qgemm);
export const getKernelLaunchCount = (): number => addon.counterGet(need(), COUNTER.launches);
export const resetDispatchCounters = (): void => addon.countersReset(need());
export const setAutotuneEnabled = (on: boolean): void => addon.autotuneSetEnabled(need(), on ? 1 : 0);
export const isAutotuneEnabled = (): boolean => addon.autotuneIsEnabled(need()) === 1;
export const getAutotuneRunCount = (): number => addon.tuneRunCount(need());
/** The per-shape cache is keyed by (m, n, k, activation dtype, weight format). */
export function getPerShapeMatmulChoice(m: number, n: number, k: number, dtype: string, format: any): CudaVariantChoice | undefined {
  const v: Int32Array | undefined = addon.tuneGet(need(), m, n, k, DTYPE_ID[dtype], qdesc(format));
  return v ? (Array.from(v) as CudaVariantChoice) : undefined;
}
export function seedPerShapeMatmulChoice(m: number, n: number, k: number, dtype: string, format: any, choice: CudaVariantChoice): void {
  addon.tuneSeed(need(), m, n, k, DTYPE_ID[dtype], qdesc(format), Int32Array.from(choice));
}
/** classifyShape (matmul/types.ts:146-200): the class whose tuned winner a shape falls back to. */
export const classifyShape = (m: number, n: number, k: number, batchSize = 1): string =>
  addon.shapeClassName(addon.classifyShape(m, n, k, batchSize));
export const clearPerShapeMatmulChoices = (): void => addon.tuneClear(need());
export const exportTuningCache = (): string => addon.tuneExportJson(need());
export const importTuningCache = (json: string): void => addon.tuneImportJson(need(), json);

/** Backend.pretuneMatmulShapes (types.ts:681-696). Shapes are [m, n, k]; the weight format must be
 * given (a per-channel format carries groupSize == K, so its shapes share one K).  ONE addon call,
 * handed the whole BigInt64Array: the addon derives the shape count from the array's own length. */
export async function pretuneMatmulShapes(shapes: [number, number, number][], aDtype = "f16", outDtype = "f16",
                                          format?: any): Promise<void> {
  if (shapes.length === 0) return;
  const flat = BigInt64Array.from(shapes.flat().map((v) => BigInt(v)));
  addon.pretune(need(), flat, DTYPE_ID[aDtype], DTYPE_ID[outDtype], format ? qdesc(format) : defaultQdesc(64, "f16"));
}

// ---- replay: a captured CUDA graph stands in for the reference's CompiledPlan replay ----------
export const beginCapture = (): void => addon.graphBegin(need());
export const endCapture = (): bigint => addon.graphEnd(need());
export const replay = (graph: bigint): void => addon.graphLaunch(need(), graph);
export const destroyGraph = (graph: bigint): void => addon.graphDestroy(need(), graph);

const ops: Partial<BackendOps> = {
  tensorFromArray: tensorFromArray as any,
  read: (async (t: BackendTensor) => Array.from(await read(t as CudaTensor))) as any,
  transpose: ((t: BackendTensor) => transpose(t as CudaTensor)) as any,
  contiguous: ((t: BackendTensor) => contiguous(t as CudaTensor)) as any,
  add: ((a: BackendTensor, b: BackendTensor) => add(a as CudaTensor, b as CudaTensor)) as any,
  sub: ((a: BackendTensor, b: BackendTensor) => sub(a as CudaTensor, b as CudaTensor)) as any,
  mul: ((a: BackendTensor, b: BackendTensor) => mul(a as CudaTensor, b as CudaTensor)) as any,
  relu: ((t: BackendTensor) => relu(t as CudaTensor)) as any,
  silu: ((t: BackendTensor) => silu(t as CudaTensor)) as any,
  sigmoid: ((t: BackendTensor) => sigmoid(t as CudaTensor)) as any,
  tanh: ((t: BackendTensor) => tanh(t as CudaTensor)) as any,
  gelu: ((t: BackendTensor, o?: any) => gelu(t as CudaTensor, o)) as any,
  cast: ((t: BackendTensor, dtype: string) => cast(t as CudaTensor, dtype)) as any,
  fusedRoPE: ((qk: BackendTensor, cos: BackendTensor, sin: BackendTensor, config: any) =>
    fusedRoPE(qk as CudaTensor, cos as CudaTensor, sin as CudaTensor, config)) as any,
  // the storage-format seam (matmul-ops.ts:42-59): a packed B goes to the fused-dequant kernels
  matmul: ((a: BackendTensor, b: BackendTensor, options?: { outBuffer?: any }) =>
    dispatchMatmul(a as CudaTensor, b as CudaTensor, false, false, options?.outBuffer)) as any,
};

export const cudaBackend = { name: "cuda", ops: ops as BackendOps, pretuneMatmulShapes } as unknown as Backend;
registerBackend(cudaBackend);
