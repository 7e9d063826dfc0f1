"""The epilogue-fusion decision on a plan of nodes (torchlette_b200/epilogue_fusion.py) against the
rules of src/compiler/matmul-epilogue.ts:131-262: chain continuity on either input of add / mul,
single consumer, no outside reference (reshape skips exempt), the [1,M,N] -> [M,N] reshape skip,
four claimed ops, four extra inputs, the gelu payload rule, ops outside the library's set."""
from types import SimpleNamespace as T

from torchlette_b200.epilogue_fusion import PlanNode as N
from torchlette_b200.epilogue_fusion import consumer_counts, detectMatmulEpilogueCore as detect


def mm(shape=(4, 8)):
    return N(0, "matmul", [T(shape=[4, 16]), T(shape=[16, 8])], list(shape), "f32")


def test_bias_activation_cast_chain_is_claimed_whole():
    m = mm()
    bias = T(shape=[8])
    a = N(1, "add", [m, bias], [4, 8], "f32")
    g = N(2, "gelu", [a], [4, 8], "f32", {"approximate": "tanh"})
    c = N(3, "cast", [g], [4, 8], "f16", {"dtype": "f16"})
    p = detect([m, a, g, c], 0)
    assert p.consumedCount == 4 and p.outputDtype == "f16" and p.outputNode is c
    assert p.epilogueOps == [{"kind": "bias", "inputIndex": 0}, {"kind": "unary", "op": "gelu"}, {"kind": "cast", "toDtype": "f16"}]
    assert p.epilogueInputs == [bias]


def test_gelu_without_tanh_payload_is_the_erf_form():
    m = mm()
    g = N(1, "gelu", [m], [4, 8], "f32")
    assert detect([m, g], 0).epilogueOps == [{"kind": "unary", "op": "gelu_erf"}]


def test_chain_continues_through_the_second_input_of_add_and_mul_but_not_sub():
    m = mm()
    res = T(shape=[4, 8])
    a = N(1, "add", [res, m], [4, 8], "f32")
    p = detect([m, a], 0)
    assert p.epilogueOps == [{"kind": "binary", "op": "add", "inputIndex": 0}] and p.epilogueInputs == [res]
    mu = N(1, "mul", [res, m], [4, 8], "f32")
    assert detect([m, mu], 0).epilogueOps == [{"kind": "binary", "op": "mul", "inputIndex": 0}]
    s = N(1, "sub", [res, m], [4, 8], "f32")  # res - matmul is not matmul - res
    assert detect([m, s], 0) is None


def test_a_second_consumer_or_an_outside_reference_ends_the_chain():
    m = mm()
    r = N(1, "relu", [m], [4, 8], "f32")
    other = N(2, "neg", [m], [4, 8], "f32")
    assert detect([m, r, other], 0) is None            # matmul has two consumers
    m2 = mm()
    r2 = N(1, "relu", [m2], [4, 8], "f32")
    c2 = N(2, "cast", [r2], [4, 8], "f16", {"dtype": "f16"})
    assert detect([m2, r2, c2], 0, None, {0}) is None  # matmul result is saved elsewhere
    p = detect([m2, r2, c2], 0, None, {1})             # relu result is: the cast is not claimed
    assert p.consumedCount == 2 and p.outputNode is r2


def test_reshape_that_drops_a_leading_one_is_skipped_and_exempt_from_the_outside_reference_rule():
    m = N(0, "matmul", [T(shape=[1, 4, 16]), T(shape=[16, 8])], [1, 4, 8], "f32")
    rs = N(1, "reshape", [m], [4, 8], "f32")
    r = N(2, "relu", [rs], [4, 8], "f32")
    p = detect([m, rs, r], 0, None, {1})
    assert p.consumedCount == 3 and p.epilogueOps == [{"kind": "unary", "op": "relu"}]
    other = N(1, "reshape", [m], [8, 4], "f32")  # any other reshape ends the chain
    assert detect([m, other, N(2, "relu", [other], [8, 4], "f32")], 0) is None


def test_limits_four_ops_four_inputs_and_unknown_ops():
    m = mm()
    chain = [m]
    for i in range(6):
        chain.append(N(i + 1, "relu", [chain[-1]], [4, 8], "f32"))
    assert detect(chain, 0).consumedCount == 5
    m = mm()
    chain = [m]
    for i in range(5):
        chain.append(N(i + 1, "add", [chain[-1], T(shape=[8])], [4, 8], "f32"))
    p = detect(chain, 0)
    assert p.consumedCount == 5 and len(p.epilogueInputs) == 4
    m = mm()
    e = N(1, "exp", [m], [4, 8], "f32")  # element-wise, but not an op of the library's epilogue
    assert detect([m, e], 0) is None
    assert detect([N(0, "add", [T(shape=[1]), T(shape=[1])], [1], "f32")], 0) is None


def test_consumer_counts():
    m = mm()
    r = N(1, "relu", [m], [4, 8], "f32")
    s = N(2, "add", [m, r], [4, 8], "f32")
    assert consumer_counts([m, r, s]) == {0: 2, 1: 1}
