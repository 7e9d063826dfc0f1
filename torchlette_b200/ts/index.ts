/**
 * torchlette `cuda` backend for the quantized-weight matmul path.
 *
 * Drop this directory into a torchlette checkout as `src/backend/cuda/`.  It is
 * the TypeScript face of libtlcuda.so (through the N-API addon built from
 * csrc/napi/tl_napi.c) and mirrors, name for name, the pieces of the webgpu
 * backend this path uses:
 *
 *   Backend / BackendOps.matmul            src/backend/types.ts:340-745
 *   matmul seam / matmulQuantizedB         src/backend/webgpu/ops/matmul-ops.ts:42-182
 *   dispatchQuantizedGemvNT                src/backend/webgpu/matmul/dispatch.ts:875-931
 *   dispatchDequantizeInt8Grouped          src/backend/webgpu/matmul/dispatch.ts:949-1037
 *   dispatchMatmul (epilogue options)      src/backend/webgpu/dispatch.ts:859-966
 *   route counters                         src/backend/webgpu/matmul/dispatch.ts:833-864, 943-947
 *   pretuneMatmulShapes / autotune flag    src/backend/webgpu/matmul/dispatch.ts:405-578
 *
 * There is no WebGPU or CPU fallback in here: if the addon or a B200 is missing,
 * initCuda() returns false and every op throws.
 *
 * This file could not be executed where it was written (no node toolchain); it
 * is a thin, reviewable 1:1 mapping onto the C ABI, which is what the parity
 * tests exercise from Python.
 */
import type { Backend, BackendOps, BackendTensor, DType, StorageFormat } from "../types";
import { registerBackend } from "../registry";
import type { EpilogueConfig } from "../webgpu/matmul/types";

// eslint-disable-next-line @typescript-eslint/no-var-requires
let addon: any = null;
let ctx: bigint | null = null;
let initError: string | null = null;

const DTYPE_ID: Record<string, number> = { f32: 0, f16: 1, bf16: 2 };
const DTYPE_BYTES: Record<string, number> = { f32: 4, f16: 2, bf16: 2, u32: 4, u16: 2 };
const UNARY: Record<string, number> = { relu: 1, silu: 2, sigmoid: 3, tanh: 4, gelu: 5, gelu_tanh: 5, gelu_erf: 6 };
const BINARY: Record<string, number> = { add: 1, sub: 2, mul: 3 };
const COUNTER = { qgemv: 0, dequant: 1, qgemvEpilogue: 2, qgemm: 3, launches: 4 } as const;

/** Device tensor: BackendTensor (types.ts:5-27) + a raw device pointer. */
export interface CudaTensor extends BackendTensor {
  buffer: bigint; // device pointer
  nbytes: number;
  transposed: boolean; // the [K,N] view of a contiguous [N,K] buffer (views.ts:925-933 keeps format/scales)
  scales?: CudaTensor;
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
function need(): bigint {
  if (ctx === null) throw new Error(`cuda backend unavailable: ${initError ?? "initCuda() was not called"}`);
  return ctx;
}

function makeTensor(shape: number[], dtype: string, buffer: bigint, nbytes: number, owns = true): CudaTensor {
  const t: any = { shape: shape.slice(), dtype, buffer, nbytes, ownsBuffer: owns, transposed: false };
  t.toArray = () => Array.from(read(t));
  t.destroy = () => {
    if (t.ownsBuffer && t.buffer) addon.free(need(), t.buffer);
    t.buffer = 0n;
  };
  return t as CudaTensor;
}

/** tensorFromArray (types.ts:341-345): typed arrays upload verbatim. */
export function tensorFromArray(values: ArrayBufferView | number[], shape: number[], dtype: string = "f32"): CudaTensor {
  const host: ArrayBufferView = Array.isArray(values) ? Float32Array.from(values) : values;
  const nbytes = host.byteLength;
  const buf: bigint = addon.alloc(need(), nbytes);
  addon.upload(need(), buf, host);
  return makeTensor(shape, dtype, buf, nbytes);
}
export function empty(shape: number[], dtype: string): CudaTensor {
  const nbytes = shape.reduce((a, b) => a * b, 1) * DTYPE_BYTES[dtype];
  return makeTensor(shape, dtype, addon.alloc(need(), nbytes), nbytes);
}
export function read(t: CudaTensor): Float32Array | Uint16Array | Uint32Array {
  const n = t.shape.reduce((a, b) => a * b, 1);
  const host = t.dtype === "f32" ? new Float32Array(n) : t.dtype === "u32" ? new Uint32Array(n) : new Uint16Array(n);
  addon.download(need(), host, t.buffer);
  return host;
}
export function transpose(t: CudaTensor): CudaTensor {
  const s = t.shape;
  const v = makeTensor([...s.slice(0, -2), s[s.length - 1], s[s.length - 2]], t.dtype as string, t.buffer, t.nbytes, false);
  v.format = t.format;
  v.scales = t.scales;
  v.transposed = !t.transposed;
  return v;
}

/** createQuantizedWeight (engine.ts:2041-2149): validate, upload, attach format + scales. */
export function createQuantizedWeight(packed: Uint32Array, scalesBits: Uint16Array | Float32Array, n: number, k: number,
                                      format: StorageFormat & { scaleConvention?: "snorm127" | "direct" }): CudaTensor {
  const packing = format.packing;
  if (!packing) throw new Error("createQuantizedWeight: format.packing is required");
  if (k % 4 !== 0) throw new Error(`createQuantizedWeight: K=${k} must be divisible by 4`);
  if (packed.length !== n * (k / 4)) throw new Error(`createQuantizedWeight: packed length ${packed.length} != ${n * (k / 4)}`);
  const groups = k / packing.groupSize;
  if (scalesBits.length !== n * groups) throw new Error(`createQuantizedWeight: scales length ${scalesBits.length} != ${n * groups}`);
  const w = tensorFromArray(packed, [n, k], format.elementType);
  w.format = format;
  w.scales = tensorFromArray(scalesBits, [n, groups], scalesBits instanceof Float32Array ? "f32" : "u16");
  return w;
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
  return { ops, inputs: BigUint64Array.from(inputs.map((t) => t.buffer)) };
}

function qdesc(format: any) {
  const p = format.packing;
  if (p.scheme !== "int8-grouped") throw new Error(`matmulQuantizedB: unsupported scheme ${p.scheme}`);
  return { group: p.groupSize, scalesDtype: DTYPE_ID[p.scalesDtype], convention: format.scaleConvention === "direct" ? 1 : 0 };
}

export interface QuantMatmulOptions { outBuffer?: CudaTensor; epilogue?: EpilogueConfig; epilogueInputs?: CudaTensor[]; alpha?: number; outputDtype?: string }

/** matmulQuantizedB (matmul-ops.ts:113-182); every M runs a fused-dequant kernel. */
function matmulQuantizedB(a: CudaTensor, b: CudaTensor, o: QuantMatmulOptions = {}): CudaTensor {
  if (!b.format?.packing || !b.scales) throw new Error("matmulQuantizedB: missing packing/scales on B operand");
  const K = b.shape[b.shape.length - 2], N = b.shape[b.shape.length - 1];
  if (a.shape[a.shape.length - 1] !== K) throw new Error("matmul dimension mismatch");
  const M = a.shape.slice(0, -1).reduce((x, y) => x * y, 1);
  const outDtype = o.epilogue?.outputDtype ?? o.outputDtype ?? "f32";
  const out = o.outBuffer ?? empty([...a.shape.slice(0, -1), N], outDtype);
  const q = qdesc(b.format);
  addon.qmatmul(need(), a.buffer, DTYPE_ID[a.dtype as string], b.buffer, b.scales.buffer, out.buffer, DTYPE_ID[outDtype],
                M, N, K, q.group, q.scalesDtype, q.convention, o.alpha ?? 1.0, encodeEpilogue(o.epilogue, o.epilogueInputs), 0);
  return out;
}

/** dispatchQuantizedGemvNT (dispatch.ts:875-931), same positional arguments after `device`. */
export function dispatchQuantizedGemvNT(a: CudaTensor, packedWeight: CudaTensor, scales: CudaTensor, out: CudaTensor, n: number,
                                        k: number, groupSize: number, outputDtype: DType | "bf16" = "f32", alpha = 1.0): void {
  addon.qmatmul(need(), a.buffer, DTYPE_ID[a.dtype as string], packedWeight.buffer, scales.buffer, out.buffer, DTYPE_ID[outputDtype],
                1, n, k, groupSize, scales.dtype === "f32" ? 0 : 1, 0, alpha, undefined, 1);
}
/** dispatchDequantizeInt8Grouped (dispatch.ts:949-1037). */
export function dispatchDequantizeInt8Grouped(bq: CudaTensor, scales: CudaTensor, out: CudaTensor, n: number, k: number, groupSize: number): void {
  addon.dequant(need(), bq.buffer, scales.buffer, out.buffer, DTYPE_ID[out.dtype as string], n, k, groupSize, scales.dtype === "f32" ? 0 : 1, 0);
}
/** dispatchMatmul over a packed B with fused epilogue (webgpu/dispatch.ts:859). */
export function dispatchMatmul(a: CudaTensor, b: CudaTensor, transA: boolean, transB: boolean, outBuffer?: CudaTensor,
                               options: { epilogue?: EpilogueConfig; epilogueInputs?: CudaTensor[] } = {}): CudaTensor {
  if (transA) throw new Error("cuda dispatchMatmul: transA is not served on this path");
  const bView = transB ? transpose(b) : b;
  return matmulQuantizedB(a, bView, { outBuffer, ...options });
}

export const getQuantGemvDispatchCount = (): number => addon.counterGet(need(), COUNTER.qgemv);
export const getDequantI8DispatchCount = (): number => addon.counterGet(need(), COUNTER.dequant);
export const getGemvEpilogueDispatchCount = (): number => addon.counterGet(need(), COUNTER.qgemvEpilogue);
export const getQuantGemmDispatchCount = (): number => addon.counterGet(need(), COUNTER.qgemm);
export const setAutotuneEnabled = (on: boolean): void => addon.autotuneSetEnabled(need(), on ? 1 : 0);
export const isAutotuneEnabled = (): boolean => addon.autotuneIsEnabled(need()) === 1;

/** Backend.pretuneMatmulShapes (types.ts:681-696). Shapes are [m, n, k]; the weight format must be given. */
export async function pretuneMatmulShapes(shapes: [number, number, number][], aDtype = "f16", outDtype = "f16",
                                          format?: any): Promise<void> {
  const flat = BigInt64Array.from(shapes.flat().map((v) => BigInt(v)));
  const q = format ? qdesc(format) : { group: 64, scalesDtype: 1, convention: 0 };
  for (let i = 0; i < shapes.length; i++) {
    // per-channel formats carry groupSize == K, which differs per shape
    const g = format ? q.group : 64;
    addon.pretune(need(), flat.subarray(3 * i, 3 * i + 3), DTYPE_ID[aDtype], DTYPE_ID[outDtype], g, q.scalesDtype, q.convention);
  }
}

const ops: Partial<BackendOps> = {
  tensorFromArray: tensorFromArray as any,
  read: (async (t: BackendTensor) => Array.from(read(t as CudaTensor))) as any,
  transpose: ((t: BackendTensor) => transpose(t as CudaTensor)) as any,
  matmul: ((a: BackendTensor, b: BackendTensor, options?: { outBuffer?: any }) => {
    const bt = b as CudaTensor;
    if (bt.format?.packing) return matmulQuantizedB(a as CudaTensor, bt, { outBuffer: options?.outBuffer });
    throw new Error("cuda backend: only a packed (quantized) B operand is served on this path");
  }) as any,
};

export const cudaBackend = { name: "cuda", ops: ops as BackendOps, pretuneMatmulShapes } as unknown as Backend;
registerBackend(cudaBackend);
