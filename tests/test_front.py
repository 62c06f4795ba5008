"""CPU tests of the boundary: parser, acceptance rules, wiring, recogniser and
the C ABI's error model.  Tables follow the reference's own unit tests
(compiler/src/front/parser.rs:363-607, compiler/src/lower/component_to_graph.rs:
258-498, compiler/src/check/component.rs) but go through the C API, as a
front-end would."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# The reference's own front-end scripts, put there unmodified by `make -C oracle frontend`.
REFERENCE_PY = os.path.join(ROOT, "baseline", "_ref", "ilang-python")


def graph_of(component):
    """Parse the `graph:` section of i_code into (n_inputs, nodes, outputs)."""
    text = component._code()
    head = re.search(r"graph: (\d+) inputs, (\d+) nodes", text)
    nodes = re.findall(r"^  n(\d+) (\w+) (\S+)~\[(\S*)\] <-(.*)$", text, re.M)
    outputs = re.search(r"^  outputs:(.*)$", text, re.M).group(1).split()
    return int(head.group(1)), [(op, pats, out, srcs.split()) for _, op, pats, out, srcs in nodes], outputs


def steps_of(component):
    return re.findall(r"^step \d+: (\w+)", component._code(), re.M)


# ---- parser ---------------------------------------------------------------

@pytest.mark.parametrize("src,op", [
    ("i+i~i", "Add"), ("i*i~i", "Mul"), ("i-i~i", "Sub"), ("i/i~i", "Div"),
    ("i>i~i", "Max"), ("i<i~i", "Min"), ("i^i~i", "Pow"), ("i$i~i", "Log"),
])
def test_parses_binary_ops(ilang, src, op):
    _, nodes, _ = graph_of(ilang.i(src))
    assert nodes[0][0] == op and nodes[0][1] == "[0],[0]" and nodes[0][2] == "0"


@pytest.mark.parametrize("src,op", [
    ("+ij~ij", "Add"), ("*ij~ij", "Mul"), ("-ij~ij", "Sub"), ("/ij~ij", "Div"),
    (">ij~ij", "Max"), ("<ij~ij", "Min"), ("^ij~ij", "Pow"), ("$ij~ij", "Log"),
    ("ij~ij", "Add"),
])
def test_parses_unary_ops(ilang, src, op):
    _, nodes, _ = graph_of(ilang.i(src))
    assert nodes[0][0] == op and nodes[0][1] == "[01]" and nodes[0][2] == "01"


def test_canonical_numbering_outputs_first(ilang):
    # compiler/src/lower/expr_to_node.rs:58-76: `ik*kj~ijk` -> i=0, j=1, k=2.
    _, nodes, _ = graph_of(ilang.i("ik*kj~ijk"))
    assert nodes[0][1] == "[02],[21]" and nodes[0][2] == "012"
    _, nodes, _ = graph_of(ilang.i("ij*jk~ikj"))
    assert nodes[0][1] == "[02],[21]" and nodes[0][2] == "012"


def test_scalar_patterns(ilang):
    _, nodes, _ = graph_of(ilang.i(".*i~i"))
    assert nodes[0][1] == "[.],[0]"
    _, nodes, _ = graph_of(ilang.i("+ij~."))
    assert nodes[0][1] == "[01]" and nodes[0][2] == "."


@pytest.mark.parametrize("src", [
    "ik*kj~ijk|i:2:4,k:8|ik0i'i''k'1j", "+ijk~ij||ij!k0", "+ijk~ij|i:2,k:4|",
    "  ij + i ~ ij |  | i j 1 ", "ij/i~ij|i:2,j:2|iji'j'01",
])
def test_accepts_schedules(ilang, src):
    # Parsing succeeds; staging digits on graph inputs are rejected only later,
    # at compile (see test_graph_input_cannot_be_staged).
    c = ilang.i(src)
    if not re.search(r"[01]", src.split("|")[-1]):
        c._code()


@pytest.mark.parametrize("src,fragment", [
    ("", "expected i-expression"),
    ("ij+ij~ij extra", "unexpected trailing input"),
    ("ij ij~ij", "expected operator after input pattern"),
    ("ij+ij", "expected `~` between inputs and output"),
    ("ij+~ij", "expected pattern"),
    ("+ij~", "expected pattern"),
    ("i.+i~i", "expected operator"),
    (".i+i~i", "scalar pattern must be `.`"),
    ("+ij~i|i:2", "expected second `|` in schedule"),
    ("+ij~i|i2|ij", "expected `:` after split axis"),
    ("+ij~i|i:|ij", "expected integer"),
    ("+ij~i|i:2,i:4|ii'j", "duplicate split entry for axis i"),
    ("ij+ij~ij||ij00", "duplicate compute directive for input 0"),
    ("+ij~i||i!!j", "duplicate output init directive"),
    ("+ij~i||i?j", "expected axis, `!`, or operand in permutation"),
    ("ij+ij~ij||ij2", "expected operand `0` or `1`"),
])
def test_parse_errors(ilang, src, fragment):
    with pytest.raises(RuntimeError) as info:
        ilang.i(src)
    assert "ParseError { offset:" in str(info.value) and fragment in str(info.value)


# ---- acceptance rules (checked at compile, as in the reference) -----------

@pytest.mark.parametrize("src,fragment", [
    ("+ij~ii", "output pattern repeats axis `i`"),
    ("+ij~ik", "output axis `k` does not appear in the input"),
    ("-ij~i", "operator `Sub` is not reducible"),
    ("^ij~i", "operator `Pow` is not reducible"),
    ("ij*jk~ik", "binary operator `Mul` must be pointwise"),
    ("+ij~i|k:2|ij", "split references unknown local axis `k`"),
    ("+ij~i||i", "permutation must list each local axis part exactly once; expected 2, found 1"),
    ("+ij~i|i:2|ijj'", "permutation references nonexistent split part `j'`"),
    ("+ij~i||iij", "permutation repeats axis part `i`"),
    ("ij+ij~ij||ij!", "output init directive is only valid for reductions"),
    ("+ij~i||!ij", "output init cannot appear before output axis part `i`"),
    ("+ij~i||ij1", "permutation references nonexistent input 1"),
])
def test_validation_errors(ilang, src, fragment):
    with pytest.raises(RuntimeError) as info:
        ilang.i(src)._code()
    assert "LowerError { message: \"expr 0: " in str(info.value) and fragment in str(info.value)


def test_expression_numbering_in_errors(ilang):
    c = ilang.i("+ij~i") >> ilang.i("-i~.")
    with pytest.raises(RuntimeError) as info:
        c._compile()
    assert "expr 1: operator `Sub` is not reducible" in str(info.value)


def test_graph_input_cannot_be_staged(ilang):
    # compiler/src/lower/node_to_stage.rs:177-184
    with pytest.raises(RuntimeError) as info:
        ilang.i("ij-i~ij | i:16,j:16 | ji01i'j'")._compile()
    assert "node 0 input 0 is a graph input with a compute site" in str(info.value)



# ---- schedules the reference's planner refuses (csrc/core/schedule.cc) -----------------------------

def compile_error(component):
    with pytest.raises(RuntimeError) as info:
        component._compile()
    return str(info.value)


def test_online_row_sum_without_downstream_accumulator_is_refused(ilang):
    # compiler/src/lower/stage_to_kernel_program.rs:2410-2431, the component of that test: the row
    # sum is consumed inside its own reduction loop by the division, and the division's result is
    # the kernel's output, so nothing can absorb the correction.
    i = ilang.i
    mm_t = i("ik*jk~ijk|i:2,j:2|iji'j'k") >> i("+ijk~ij|i:2,j:2|iji'j'k0")
    mm = i("ik*kj~ijk|i:2,k:2|ik0ji'k'") >> i("+ijk~ij|i:2,k:2|ikji'k'0")
    exp = i("^ij~ij|i:2,j:2|iji'j'0")
    row_sum = i("+ij~i|i:2,j:2|iji'j'0")
    row_div = i("ij/i~ij|i:2,j:2|iji'j'1")
    attention = mm_t >> exp >> (mm & row_sum) >> row_div
    assert compile_error(attention) == (
        'LowerError { message: "online reduction correction reached root without an accumulator" }')


def test_softmax_alone_with_the_fused_loop_orders_is_refused(ilang):
    # The README's fused orders applied to the softmax stages alone (no contraction in front, none
    # behind): with the logits coming from a map rather than a graph input, the online row sum's
    # correction has no `+` accumulator downstream.
    i, I = ilang.i, ilang.I
    logits = i("ij*ij~ij | i:16,j:16 | jii'j'")
    shift = (I & i(">ij~i | i:16,j:16 | ji0i'j'")) >> i("ij-i~ij | i:16,j:16 | ji01i'j'")
    exp = i("^ij~ij | i:16,j:16 | ji0i'j'")
    norm = (I & i("+ij~i | i:16,j:16 | ji0i'j'")) >> i("ij/i~ij | i:16,j:16 | ji01i'j'")
    assert "online reduction correction reached root without an accumulator" in compile_error(
        logits >> shift >> exp >> norm)


def test_staged_producer_must_be_split_like_its_consumer(ilang):
    # compiler/src/lower/node_to_stage.rs:720-745 (case :1390-1421 for the extent kinds).
    i = ilang.i
    assert compile_error(i("+ij~i | i:4 | ii'j") >> i(">i~i | i:2 | ii'0")) == (
        'LowerError { message: "producer extent kind Base([4]) does not match consumer extent kind Base([2])" }')
    assert compile_error(i("+ij~i | i:4 | ii'j") >> i(">i~i || i0")) == (
        'LowerError { message: "producer index 0 has 2 axes but consumer index 0 has 1 axes" }')
    # Same splits: accepted.
    (i("+ij~i | i:4 | ii'j") >> i(">i~i | i:4 | ii'0"))._compile()


def test_online_reductions_other_than_sum_and_max_are_refused(ilang):
    # compiler/src/lower/stage_to_kernel_program.rs:1127-1156: a row minimum consumed inside its
    # own reduction loop.
    i, I = ilang.i, ilang.I
    logits = i("ij*ij~ij | i:16,j:16 | jii'j'")
    c = logits >> (I & i("<ij~i | i:16,j:16 | ji0i'j'")) >> i("ij-i~ij | i:16,j:16 | ji01i'j'")
    assert "requires online reduction lowering: fused reduction axis is consumed before completion" in compile_error(c)


def test_online_max_needs_subtraction_then_exponentiation(ilang):
    # compiler/src/lower/stage_to_kernel_program.rs:1594-1637.
    i, I = ilang.i, ilang.I
    logits = i("ij*ij~ij | i:16,j:16 | jii'j'")
    online_max = I & i(">ij~i | i:16,j:16 | ji0i'j'")
    assert "online max correction requires a subtraction use before exponentiation" in compile_error(
        logits >> online_max >> i("ij*i~ij | i:16,j:16 | ji01i'j'"))
    shifted = logits >> online_max >> i("ij-i~ij | i:16,j:16 | ji01i'j'")
    assert "online max correction requires exponentiation before accumulation" in compile_error(
        shifted >> i("-ij~ij | i:16,j:16 | ji0i'j'") >> i("+ij~i | i:16,j:16 | ji0i'j'"))


def test_accepted_fused_schedules_still_compile(ilang):
    # The README chain, its deferred-normalisation form and the naive five-kernel schedule.
    assert steps_of(readme_attention(ilang)) == ["attention"]
    assert steps_of(naive_attention(ilang)) == ["contract", "row_softmax", "contract"]
    deferred_attention(ilang)._compile()


def test_comparisons_and_logic_compile(ilang):
    # compiler/src/front/parser.rs:270-279, 374-413: every operator token in unary and binary form.
    for tok in (">>", ">=", "<<", "<=", "==", "!=", "&&", "||", "^^"):
        for src in (tok + "ij~ij", "ij" + tok + "ij~ij", "ij" + tok + "j~ij"):
            assert "ib_map" in ilang.i(src)._code()
    assert "ib_map" in ilang.i("!!ij~ij")._code()
    for tok in ("&&", "||", "^^"):
        assert "ib_reduce" in ilang.i(tok + "ij~i")._code()


def test_not_and_comparisons_do_not_reduce(ilang):
    # compiler/src/check/component.rs:407-412
    for src, name in ((">>ij~i", "Gt"), ("==ij~i", "Eq"), ("!!ij~i", "Not")):
        with pytest.raises(RuntimeError) as info:
            ilang.i(src)._compile()
        assert name in str(info.value)


# ---- wiring ---------------------------------------------------------------

def test_identity(ilang):
    n_in, nodes, outs = graph_of(ilang.I)
    assert (n_in, nodes, outs) == (1, [], ["in0"])


def test_pair_concatenates(ilang):
    n_in, nodes, outs = graph_of(ilang.i("ij+i~ij") | ilang.i("+ij~i"))
    assert n_in == 3 and nodes[0][3] == ["in0", "in1"] and nodes[1][3] == ["in2"]
    assert outs == ["n0", "n1"]


def test_chain(ilang):
    n_in, nodes, outs = graph_of(ilang.i("ik*kj~ijk") >> ilang.i("+ijk~ij"))
    assert n_in == 2 and nodes[1][3] == ["n0"] and outs == ["n1"]


def test_chain_mixed_arity(ilang):
    c = (ilang.i("+ij~i") | ilang.i("+ij~j")) >> ilang.i("i~i")
    n_in, nodes, outs = graph_of(c)
    assert n_in == 2 and outs == ["n1", "n2"] and nodes[2][3] == ["n0"]


def test_compose(ilang):
    n_in, nodes, outs = graph_of(ilang.i("ij+i~ij") << ilang.i("+ij~i"))
    assert n_in == 2 and nodes[0][3] == ["in0"] and nodes[1][3] == ["n0", "in1"] and outs == ["n1"]


def test_compose_mixed_arity(ilang):
    c = ilang.i("i+i~i") << (ilang.i("i~i") | ilang.i("i~i"))
    n_in, nodes, outs = graph_of(c)
    assert n_in == 2 and outs == ["n2"] and nodes[2][3] == ["n0", "n1"]


def test_fanout(ilang):
    n_in, nodes, outs = graph_of(ilang.i("+ij~i") & ilang.i("+ij~j"))
    assert n_in == 1 and nodes[0][3] == ["in0"] and nodes[1][3] == ["in0"] and outs == ["n0", "n1"]
    n_in, nodes, _ = graph_of(ilang.i("ij+i~ij") & ilang.i("+ij~i"))
    assert n_in == 2 and nodes[0][3] == ["in0", "in1"] and nodes[1][3] == ["in0"]


def test_swap(ilang):
    _, _, outs = graph_of(~(ilang.i("+ij~i") | ilang.i("+ij~j")))
    assert outs == ["n1", "n0"]
    _, _, outs = graph_of(~ilang.i("+ij~i"))
    assert outs == ["n0"]


def test_nested(ilang):
    i = ilang.i
    c = ~((i("ik*kj~ijk") & i("+ik~i")) >> (i("+ijk~ij") | i("i~i")))
    n_in, nodes, outs = graph_of(c)
    assert n_in == 2 and outs == ["n3", "n2"]


def test_readme_attention_graph(ilang):
    # 3 inputs (Q, K, V appended by chain), 9 nodes in source order.
    n_in, nodes, outs = graph_of(readme_attention(ilang))
    assert n_in == 3 and len(nodes) == 9 and outs == ["n8"]
    assert [n[0] for n in nodes] == ["Mul", "Add", "Max", "Sub", "Pow", "Add", "Div", "Mul", "Add"]
    assert nodes[3][3] == ["n1", "n2"] and nodes[6][3] == ["n4", "n5"] and nodes[7][3] == ["n6", "in2"]


# ---- recogniser -----------------------------------------------------------

def readme_attention(ilang):
    i, I = ilang.i, ilang.I
    mm_t = i("ik*jk~ijk | i:16,j:16 | jii'j'k") >> i("+ijk~ij | i:16,j:16 | jii'j'k0")
    row_max_shift = (I & i(">ij~i | i:16,j:16 | ji0i'j'")) >> i("ij-i~ij | i:16,j:16 | ji01i'j'")
    exp = i("^ij~ij | i:16,j:16 | ji0i'j'")
    row_normalize = (I & i("+ij~i | i:16,j:16 | ji0i'j'")) >> i("ij/i~ij | i:16,j:16 | ji01i'j'")
    mm = i("ij*jk~ikj | i:16,j:16 | ji0i'kj'") >> i("+ikj~ik | i:16,j:16 | jii'kj'0")
    return mm_t >> row_max_shift >> exp >> row_normalize >> mm


def naive_attention(ilang):
    i, I = ilang.i, ilang.I
    mm_t = i("ik*jk~ijk | i:16,j:16 | jii'j'k") >> i("+ijk~ij | i:16,j:16 | jii'j'k0")
    row_max_shift = (I & i(">ij~i | i:16,j:16 | jii'j'")) >> i("ij-i~ij | i:16,j:16 | 1jii'j'")
    exp = i("^ij~ij | i:16,j:16 | jii'j'")
    row_normalize = (I & i("+ij~i | i:16,j:16 | jii'j'")) >> i("ij/i~ij | i:16,j:16 | 1jii'j'")
    mm = i("ij*jk~ikj | i:16,j:16 | jii'kj'") >> i("+ikj~ik | i:16,j:16 | jii'kj'0")
    return mm_t >> row_max_shift >> exp >> row_normalize >> mm


def test_fused_schedule_is_one_attention_kernel(ilang):
    assert steps_of(readme_attention(ilang)) == ["attention"]


def deferred_attention(ilang, shift=False, staged=True):
    """Attention with the division deferred: exp, then (E V) and rowsum(E), then the division —
    the formulation of compiler/src/lower/stage_to_kernel_program.rs:2705-2780 (same strings)."""
    i, I = ilang.i, ilang.I
    mm_t = i("ik*jk~ijk|i:2,j:2|iji'j'k") >> i("+ijk~ij|i:2,j:2|iji'j'k0")
    exp = i("^ij~ij|i:2,j:2|iji'j'0")
    mm = i("ik*kj~ijk|i:2,k:2|ik0i'jk'" if staged else "ik*kj~ijk|i:2,k:2|iki'jk'") \
        >> i("+ijk~ij|i:2,k:2|iki'jk'0")
    row_sum = i("+ij~i|i:2,j:2|ij0i'j'")
    row_div = i("ij/i~ij|i:2|i01i'j")
    chain = mm_t
    if shift:
        chain = chain >> ((I & i(">ij~i|i:2,j:2|ij0i'j'")) >> i("ij-i~ij|i:2,j:2|ij01i'j'"))
    return chain >> exp >> (mm & row_sum) >> row_div


def scaled_attention(ilang, kind="mul_right", batched=False):
    """README attention with one scalar on the logits: (q, k, c, v), or (c, q, k, v) for mul_left
    and rdiv.  `batched` puts two leading axes on every tensor."""
    i, I = ilang.i, ilang.I
    b = "bh" if batched else ""
    mm_t = i(f"{b}ik*{b}jk~{b}ijk | i:16,j:16 | {b}jii'j'k") >> i(f"+{b}ijk~{b}ij | i:16,j:16 | {b}jii'j'k0")
    # The scale is staged into the row maximum's loops, so it carries the same splits
    # (node_to_stage.rs:720-745) and stages its own logits operand the same way.
    scale = {"mul_left": f".*{b}ij~{b}ij | i:16,j:16 | {b}ji1i'j'",
             "mul_right": f"{b}ij*.~{b}ij | i:16,j:16 | {b}ji0i'j'",
             "div": f"{b}ij/.~{b}ij | i:16,j:16 | {b}ji0i'j'",
             "rdiv": f"./{b}ij~{b}ij | i:16,j:16 | {b}ji1i'j'"}[kind]
    logits = ((I | mm_t) if kind in ("mul_left", "rdiv") else (mm_t | I)) >> i(scale)
    row_max_shift = (I & i(f">{b}ij~{b}i | i:16,j:16 | {b}ji0i'j'")) >> i(f"{b}ij-{b}i~{b}ij | i:16,j:16 | {b}ji01i'j'")
    exp = i(f"^{b}ij~{b}ij | i:16,j:16 | {b}ji0i'j'")
    row_normalize = (I & i(f"+{b}ij~{b}i | i:16,j:16 | {b}ji0i'j'")) >> i(f"{b}ij/{b}i~{b}ij | i:16,j:16 | {b}ji01i'j'")
    mm = i(f"{b}ij*{b}jk~{b}ikj | i:16,j:16 | {b}ji0i'kj'") >> i(f"+{b}ikj~{b}ik | i:16,j:16 | {b}jii'kj'0")
    return logits >> row_max_shift >> exp >> row_normalize >> mm


def test_scaled_logits_stay_one_attention_kernel(ilang):
    for kind, text in (("mul_right", "logits * in2"), ("mul_left", "logits * in0"), ("div", "logits / in2")):
        attn = scaled_attention(ilang, kind)
        assert steps_of(attn) == ["attention"], kind
        assert text in attn._code()
    assert steps_of(scaled_attention(ilang, "div", batched=True)) == ["attention"]
    # A scalar over the logits is not a scale on them.
    assert steps_of(scaled_attention(ilang, "rdiv")) == ["contract", "map", "row_softmax", "contract"]
    attn = scaled_attention(ilang)
    q, k, v = (np.zeros(s, np.float32) for s in ((100, 40), (77, 40), (77, 24)))
    assert attn.output_shapes(q, k, np.float32(0.5), v) == [(100, 24)]
    with pytest.raises(RuntimeError, match="scalar"):
        attn.output_shapes(q, k, np.zeros((3,), np.float32), v)


def test_deferred_normalisation_is_one_attention_kernel(ilang):
    assert steps_of(deferred_attention(ilang)) == ["attention"]
    assert steps_of(deferred_attention(ilang, shift=True)) == ["attention"]
    # Without a staged producer in the second contraction nothing fuses across it.
    assert "attention" not in steps_of(deferred_attention(ilang, staged=False))


def test_naive_schedule_keeps_three_kernels(ilang):
    # ilang-python/flash-attn.py:57-65: no staging of P => intermediates stay.
    assert steps_of(naive_attention(ilang)) == ["contract", "row_softmax", "contract"]


def test_batched_attention_letters_do_not_matter(ilang):
    # ilang-python/test.py:75-82 uses b,h axes and other letters.
    i, I = ilang.i, ilang.I
    mm_t = i("bhij*bhkj~bhikj | i:16,k:16 | bhkii'k'j") >> i("+bhikj~bhik | i:16,k:16 | bhkii'k'j0")
    rms = (I & i(">bhik~bhi | i:16,k:16 | bhkii'k'")) >> i("bhik-bhi~bhik | i:16,k:16 | bh1kii'k'")
    exp = i("^bhik~bhik | i:16,k:16 | bhkii'k'")
    rn = (I & i("+bhik~bhi | i:16,k:16 | bhkii'k'")) >> i("bhik/bhi~bhik | i:16,k:16 | bh1kii'k'")
    mm = i("bhik*bhkj~bhijk | i:16,k:16 | bhkii'jk'") >> i("+bhijk~bhij | i:16,k:16 | bhkii'jk'0")
    attn = mm_t >> rms >> exp >> rn >> mm
    assert steps_of(attn) == ["contract", "row_softmax", "contract"]
    q = np.zeros((2, 3, 4, 8), np.float32)
    assert attn.output_shapes(q, q, q) == [(2, 3, 4, 8)]
    assert "batch axes 2" in attn._code()


def test_contraction_forms(ilang):
    i = ilang.i
    assert steps_of(i("ik*jk~ijk") >> i("+ijk~ij")) == ["contract"]
    assert steps_of(i("ik*kj~ijk|i:2,k:2|ii'jkk'") >> i("+ijk~ij|i:2,k:2|ii'j!kk'0")) == ["contract"]
    assert steps_of(i("ij*j~ij") >> i("+ij~i")) == ["contract"]          # matrix-vector
    # A product that is also an output cannot be folded away.
    both = i("ik*jk~ijk") >> (ilang.I & i("+ijk~ij"))
    assert steps_of(both) == ["map", "reduce"]


def test_softmax_alone(ilang):
    i, I = ilang.i, ilang.I
    sm = ((I & i(">ij~i")) >> i("ij-i~ij")) >> i("^ij~ij") >> ((I & i("+ij~i")) >> i("ij/i~ij"))
    assert steps_of(sm) == ["row_softmax"]
    assert sm.output_shapes(np.zeros((5, 9), np.float32)) == [(5, 9)]


def test_pointwise_chains_are_one_kernel(ilang):
    i, I = ilang.i, ilang.I
    bias_relu_gate = i("ij+j~ij") >> i(">ij~ij") >> i("ij*ij~ij")
    assert steps_of(bias_relu_gate) == ["map_chain"]
    assert "in0+in1  >_  _*in2" in bias_relu_gate._code()
    assert bias_relu_gate.output_shapes(*(np.zeros(s, np.float32) for s in ((6, 8), (8,), (6, 8)))) == [(6, 8)]
    assert steps_of(i("bij-bi~bij") >> i("^bij~bij") >> i("bij/bi~bij")) == ["map_chain"]
    assert steps_of(i(".*i~i") >> i("-i~i")) == ["map_chain"]         # scalar operand, rank 1
    # An intermediate that is also an output stays a kernel of its own.
    assert steps_of(i("ij+j~ij") >> (I & i(">ij~ij"))) == ["map", "map"]
    # So does a map that permutes or broadcasts along a leading axis only.
    assert steps_of(i("ij+j~ij") >> i("ij~ji")) == ["map", "map"]
    assert steps_of(i("bij*b~bij") >> i("^bij~bij")) == ["map", "map"]
    # The reading map may take the earlier result on either side, but only once.
    assert steps_of(i("^ij~ij") >> (I & I) >> i("ij*ij~ij")) == ["map", "map"]
    # Nine operators: the ninth starts a new kernel.
    long = i("-i~i")
    for _ in range(8):
        long = long >> i("-i~i")
    assert steps_of(long) == ["map_chain", "map"]
    # Softmax still wins over the generic chain.
    sm = ((I & i(">ij~i")) >> i("ij-i~ij")) >> i("^ij~ij") >> ((I & i("+ij~i")) >> i("ij/i~ij"))
    assert steps_of(sm) == ["row_softmax"]


def test_pointwise_chain_under_a_row_fold_is_one_kernel(ilang):
    i, I = ilang.i, ilang.I
    denom = i("ij-i~ij") >> i("^ij~ij") >> i("+ij~i")
    assert steps_of(denom) == ["chain_reduce"]
    assert "fold `+` of" in denom._code() and "in0-in1  ^_" in denom._code()
    assert denom.output_shapes(np.zeros((6, 8), np.float32), np.zeros((6,), np.float32)) == [(6,)]
    assert steps_of(i("ij>>j~ij") >> i("||ij~i")) == ["chain_reduce"]
    assert steps_of(i("^bij~bij") >> i(">bij~bi")) == ["chain_reduce"]
    assert steps_of(i("-i~i") >> i("+i~.")) == ["chain_reduce"]
    # A product under a sum is still a contraction, a fold of another axis a plain fold.
    assert steps_of(i("ij*ij~ij") >> i("+ij~i")) == ["contract"]
    assert steps_of(i("^ij~ij") >> i("+ij~j")) == ["map", "reduce"]
    assert steps_of(i("^bij~bij") >> i("+bij~b")) == ["map", "reduce"]
    # The pointwise result is needed elsewhere: it is stored, and folded separately.
    assert steps_of(i("^ij~ij") >> (I & i("+ij~i"))) == ["map", "reduce"]


def test_pointwise_operators_on_a_contraction_run_in_its_epilogue(ilang):
    i, I = ilang.i, ilang.I
    mm_t = i("ik*jk~ijk") >> i("+ijk~ij")
    layer = mm_t >> i("ij+j~ij") >> i(">ij~ij")                     # product, bias, rectifier
    assert steps_of(layer) == ["contract"]
    assert "epilogue" in layer._code() and "_+in2  >_" in layer._code()
    shapes = ((6, 5), (8, 5), (8,))
    assert layer.output_shapes(*(np.zeros(s, np.float32) for s in shapes)) == [(6, 8)]
    with pytest.raises(RuntimeError, match="axis extent mismatch"):
        layer.output_shapes(np.zeros((6, 5), np.float32), np.zeros((8, 5), np.float32),
                            np.zeros((7,), np.float32))
    # The product on the right of a subtraction, per-row and full-size operands, batch axes.
    rowwise = (I | mm_t) >> i("i-ij~ij")
    assert steps_of(rowwise) == ["contract"] and "in0-_" in rowwise._code()
    assert steps_of((i("bik*bjk~bijk") >> i("+bijk~bij")) >> i("bij*bij~bij") >> i("<bij~bij")) == ["contract"]
    # Operators outside + - * > < stay a pass of their own, as does a product read twice, one
    # that is also an output, and one stored transposed.
    assert steps_of(mm_t >> i("^ij~ij")) == ["contract", "map"]
    assert steps_of(mm_t >> i("ij+j~ij") >> i("^ij~ij")) == ["contract", "map_chain"]
    assert steps_of(mm_t >> (I & I) >> i("ij*ij~ij")) == ["contract", "map"]
    assert steps_of(mm_t >> (I & i(">ij~ij"))) == ["contract", "map"]
    assert steps_of(i("ik*jk~ijk") >> i("+ijk~ji") >> i(">ji~ji")) == ["contract", "map"]
    squared = mm_t >> i("ij+j~ij") >> (I & I) >> i("ij*ij~ij")      # the bias joins, the square cannot
    assert steps_of(squared) == ["contract", "map"] and "_+in2\n" in squared._code()


def test_output_shapes_follow_inputs(ilang):
    attn = readme_attention(ilang)
    q, k, v = (np.zeros(s, np.float32) for s in ((100, 40), (77, 40), (77, 24)))
    assert attn.output_shapes(q, k, v) == [(100, 24)]
    with pytest.raises(RuntimeError):
        attn.output_shapes(q, k)                       # wrong input count
    with pytest.raises(RuntimeError):
        attn.output_shapes(q, np.zeros((77, 41), np.float32), v)   # extents disagree


# ---- C ABI ----------------------------------------------------------------

def declared_symbols():
    names = []
    for header in ("i.h", "i_b200.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(i_[a-z0-9_]+|ib_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(ilang):
    lib = ilang.core()
    names = declared_symbols()
    assert len([n for n in names if n.startswith("i_") and not n.startswith("i_b200")]) == 19
    for name in names:
        assert hasattr(lib, name), name


def test_error_model(ilang):
    lib = ilang.core()
    assert lib.i_parse(None) is None and b"null source" in lib.i_error()
    assert lib.i_chain(None, None) is None and b"null left component" in lib.i_error()
    assert lib.i_compile(None) is None and b"null component" in lib.i_error()
    assert lib.i_output_count(None) == 0 and b"null program" in lib.i_error()
    assert lib.i_exec_into(None, None, 0, None, 0) == -1
    out = lib.i_exec(None, None, 0)
    assert out.count == 0 and not out.tensors
    lib.i_component_free(None)
    lib.i_program_free(None)
    lib.i_string_free(None)
    c = ilang.i("+ij~i")
    prog = c._compile()
    assert lib.i_exec_into(prog, None, 1, None, 1) == -1 and b"null inputs" in lib.i_error()
    assert lib.i_output_ranks(prog, None) == -1 and b"null ranks" in lib.i_error()


def test_exec_without_gpu_fails_loudly(ilang):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError) as info:
        ilang.i("+ij~i").exec_numpy(np.ones((4, 4), np.float32))
    assert "no usable CUDA device" in str(info.value) and "no CPU path" in str(info.value)


def test_precision_switch(ilang):
    c = ilang.i("ik*jk~ijk") >> ilang.i("+ijk~ij")
    c.set_precision("tf32")
    assert ilang.core().i_b200_program_precision(c._compile()) == 2
    c.set_precision("fp32")
    assert ilang.core().i_b200_program_precision(c._compile()) == 1
    for name, code in (("bf16", 3), ("tf32_f16", 4), ("f16", 5), ("auto", 0)):
        c.set_precision(name)
        assert ilang.core().i_b200_program_precision(c._compile()) == code
    with pytest.raises((ValueError, KeyError, RuntimeError)):
        c.set_precision("fp64")


@pytest.mark.skipif(not os.path.isfile(os.path.join(REFERENCE_PY, "ilang.py")),
                    reason="the reference's front-end has not been fetched (make -C oracle frontend)")
def test_unmodified_reference_frontend_binds_this_library(ilang):
    """The reference's own ilang.py, selected by ILANG_CORE_LIB, builds and
    compiles the README attention against this library (no exec without a GPU)."""
    code = (
        "import numpy as np\n"
        "from ilang import Component as i, I\n"
        "mm_t = i(\"ik*jk~ijk | i:16,j:16 | jii'j'k\") >> i(\"+ijk~ij | i:16,j:16 | jii'j'k0\")\n"
        "rms = (I & i(\">ij~i | i:16,j:16 | ji0i'j'\")) >> i(\"ij-i~ij | i:16,j:16 | ji01i'j'\")\n"
        "ex = i(\"^ij~ij | i:16,j:16 | ji0i'j'\")\n"
        "rn = (I & i(\"+ij~i | i:16,j:16 | ji0i'j'\")) >> i(\"ij/i~ij | i:16,j:16 | ji01i'j'\")\n"
        "mm = i(\"ij*jk~ikj | i:16,j:16 | ji0i'kj'\") >> i(\"+ikj~ik | i:16,j:16 | jii'kj'0\")\n"
        "attn = mm_t >> rms >> ex >> rn >> mm\n"
        "assert 'attention' in attn._code()\n"
        "q = np.zeros((128, 64), np.float32)\n"
        "assert attn.output_shapes(q, q, q) == [(128, 64)]\n"
        "print('bound')\n"
    )
    env = dict(os.environ, ILANG_CORE_LIB=ilang.DEFAULT_LIB, PYTHONPATH=REFERENCE_PY)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
    assert out.returncode == 0 and "bound" in out.stdout, out.stderr


def test_schedule_segment_chooses_the_kernel_geometry(ilang):
    """Splits and loop order reach the plan: i_code names the geometry each step will run with."""
    i = ilang.i

    def mm_t(split, order):
        return i("ik*jk~ijk | %s | %s" % (split, order)) >> i("+ijk~ij | %s | %s0" % (split, order))

    def geometry(component):
        return re.search(r"^\s*geometry: (.*)$", component._code(), re.M).group(1)

    plain = geometry(i("ik*jk~ijk") >> i("+ijk~ij"))
    readme = geometry(mm_t("i:16,j:16", "jii'j'k"))
    narrow = geometry(mm_t("i:128,j:128", "ijj'i'k"))
    wide = geometry(mm_t("i:128,j:256", "jii'j'k"))
    assert plain == readme                     # splits finer than any MMA tile leave the choice open
    assert "128 columns (the schedule's column split)" in narrow and "row by row" in narrow
    assert "256 columns (the schedule's column split)" in wide and "groups of 12" in wide
    assert len({readme, narrow, wide}) == 3
