"""The lazy graph's epilogue-fusion decision, on a plan of nodes.

Host-side mirror of ``detectMatmulEpilogueCore`` (src/compiler/matmul-epilogue.ts:131-262) with its
helpers ``findChainInput`` (:31-45) and ``getEpilogueOpName`` (:52-62): starting at a matmul node,
walk the plan forward and claim up to four following ops -- casts, bias / residual adds, mul / sub
with another tensor, activations -- as the matmul's epilogue, as long as every link of the chain
has exactly one consumer, is not referenced from outside the plan, and continues the chain.

Two deliberate differences, both on the side of claiming LESS or MORE only where this backend's
kernels differ from the reference's:
  * a unary op is claimed only if the library's epilogue implements it (relu, silu, sigmoid, tanh,
    gelu, gelu_erf -- the set of src/backend/webgpu/matmul/gemv.ts:135-143); the reference's tiled
    kernel also accepts the other element-wise ops of its catalog;
  * a packed (quantized) B operand does not veto the fusion (the reference skips such matmuls,
    src/compiler/graph-compiler.ts:150-152, because its directive path bypasses the format read).
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Set, Union

UNARY_IN_LIBRARY = {"relu", "silu", "sigmoid", "tanh", "gelu", "gelu_erf"}


@dataclass
class PlanNode:
    """A LazyIRNode as far as the decision reads it (src/graph/types.ts): inputs are other
    PlanNodes (pending results) or anything with a ``.shape`` (materialized tensors)."""
    id: int
    op: str
    inputs: List[object] = field(default_factory=list)
    shape: List[int] = field(default_factory=list)
    dtype: Optional[str] = None
    payload: Optional[dict] = None


@dataclass
class EpiloguePlan:
    consumedCount: int          # matmul + claimed ops (reshape skips included)
    epilogueOps: List[dict]
    epilogueInputs: List[object]
    outputDtype: Optional[str]
    outputNode: PlanNode


def consumer_counts(nodes: Sequence[PlanNode]) -> Dict[int, int]:
    counts: Dict[int, int] = {}
    for n in nodes:
        for i in n.inputs:
            if isinstance(i, PlanNode):
                counts[i.id] = counts.get(i.id, 0) + 1
    return counts


def _chain_input(nxt: PlanNode, current_id: int) -> int:
    """Which input of ``nxt`` continues the chain: 0, 1 (add / mul commute) or -1."""
    first = nxt.inputs[0]
    if isinstance(first, PlanNode) and first.id == current_id:
        return 0
    if nxt.op in ("add", "mul") and len(nxt.inputs) == 2:
        second = nxt.inputs[1]
        if isinstance(second, PlanNode) and second.id == current_id:
            return 1
    return -1


def _unary_name(node: PlanNode) -> str:
    if node.op == "gelu":
        return "gelu" if (node.payload or {}).get("approximate") == "tanh" else "gelu_erf"
    return node.op


def detectMatmulEpilogueCore(nodes: Sequence[PlanNode], startIdx: int, consumerCount: Optional[Dict[int, int]] = None,
                             externalNodeIds: Optional[Set[int]] = None) -> Optional[EpiloguePlan]:
    matmul = nodes[startIdx]
    if matmul.op != "matmul":
        return None
    if consumerCount is None:
        consumerCount = consumer_counts(nodes)
    ops: List[dict] = []
    extra: List[object] = []
    claimed = 0
    cur = matmul
    out_dtype = matmul.dtype
    cur_is_reshape_skip = False
    for nxt in nodes[startIdx + 1:]:
        if claimed >= 4 or not nxt.inputs:
            break
        side = _chain_input(nxt, cur.id)
        if side < 0:
            break
        # the link must be private to the chain: no outside reference (a reshape skip already
        # absorbed is exempt), one consumer
        if externalNodeIds and cur.id in externalNodeIds and not cur_is_reshape_skip:
            break
        if consumerCount.get(cur.id, 0) > 1:
            break
        if nxt.op == "reshape":
            a, b = list(cur.shape), list(nxt.shape)
            if len(a) == len(b) + 1 and a[0] == 1 and a[1:] == b:  # [1, M, N] -> [M, N]
                claimed += 1
                cur, cur_is_reshape_skip = nxt, True
                out_dtype = nxt.dtype or out_dtype
                continue
            break
        cur_is_reshape_skip = False
        if nxt.op == "cast":
            to = (nxt.payload or {}).get("dtype")
            if to is None:
                break
            ops.append({"kind": "cast", "toDtype": to})
            out_dtype = to
        elif nxt.op == "add" and len(nxt.inputs) == 2:
            if len(extra) >= 4:
                break
            other = nxt.inputs[1 - side]
            shape = getattr(other, "shape", None)
            if shape is not None and len(shape) == 1:
                ops.append({"kind": "bias", "inputIndex": len(extra)})
            else:
                ops.append({"kind": "binary", "op": "add", "inputIndex": len(extra)})
            extra.append(other)
        elif nxt.op in ("mul", "sub") and len(nxt.inputs) == 2:
            if len(extra) >= 4:
                break
            ops.append({"kind": "binary", "op": nxt.op, "inputIndex": len(extra)})
            extra.append(nxt.inputs[1 - side])
        elif len(nxt.inputs) == 1 and _unary_name(nxt) in UNARY_IN_LIBRARY:
            ops.append({"kind": "unary", "op": _unary_name(nxt)})
        else:
            break
        claimed += 1
        cur = nxt
        out_dtype = nxt.dtype or out_dtype
    if claimed == 0:
        return None
    return EpiloguePlan(1 + claimed, ops, extra, out_dtype, cur)
