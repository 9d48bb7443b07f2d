"""CPU: the idiom recogniser (pypto_b200/ir/idioms.py) reads DSL bodies, never runs them, and binds the roles of a
fused operator to a program's own parameter names by data flow."""

import pytest

from pypto_b200 import ir
from pypto_b200.ir import idioms
from pypto_b200.runtime import fused_programs
from tests.dsl_programs import renamed_idioms as progs


def test_swiglu_ffn_is_recognised_under_other_names_orders_and_spellings():
    rec = idioms.recognise(progs.gated_mlp)
    assert rec is not None and rec.idiom == "ffn_swiglu"
    # the weight whose product goes through the sigmoid is the gate, wherever it stands in the signature
    assert rec.roles == {"x": "tokens", "w_gate": "w_act", "w_up": "w_lin", "w_down": "w_out", "out": "y"}
    op = fused_programs.from_idiom(progs.gated_mlp)
    assert op.op_names == ("ffn_swiglu",) and op.names == ("tokens", "w_act", "w_lin", "w_out", "y")
    assert op.matches(progs.gated_mlp) and not op.matches(progs.relu_mlp)


def test_a_program_class_with_kernel_methods_is_followed_through_self():
    prog = progs.GatedMlpProgram
    rec = idioms.recognise(prog.entry, prog)
    assert rec is not None and rec.idiom == "ffn_swiglu"
    assert rec.roles == {"x": "inp", "w_gate": "wa", "w_up": "wb", "w_down": "wc", "out": "res"}
    assert ir.compile(prog, platform="b200").op_names == ("ffn_swiglu",)


def test_rms_norm_is_recognised_with_its_constants():
    rec = idioms.recognise(progs.scaled_norm)
    assert rec is not None and rec.idiom == "rms_norm"
    assert rec.roles == {"x": "rows", "gamma": "weight", "out": "normed"}
    assert rec.constants["eps"] == pytest.approx(progs.EPS) and rec.constants["inv_n"] == pytest.approx(1.0 / 64)
    op = fused_programs.from_idiom(progs.scaled_norm)
    assert op.eps == pytest.approx(progs.EPS) and op.names == ("rows", "weight", "normed")


def test_matrix_products_are_recognised_with_and_without_a_bias():
    rec = idioms.recognise(progs.product)
    assert rec is not None and rec.idiom == "linear" and rec.roles == {"a": "lhs", "b": "rhs", "out": "dst"}
    rec = idioms.recognise(progs.affine)
    assert rec is not None and rec.idiom == "linear"
    assert rec.roles == {"a": "lhs", "b": "rhs", "bias": "offset", "out": "dst"}
    op = fused_programs.from_idiom(progs.affine)
    assert op.op_names == ("linear",) and (op.a, op.b, op.out, op.bias) == ("lhs", "rhs", "dst", "offset")
    assert ir.compile(progs.product, platform="b200").op_names == ("linear",)


def test_one_projection_ffns_are_recognised_with_their_activation():
    rec = idioms.recognise(progs.swish_mlp)
    assert rec is not None and rec.idiom == "ffn_act" and rec.constants["kind"] == 1
    assert rec.constants["alpha"] == pytest.approx(1.0)                      # plain SiLU
    assert rec.roles == {"x": "tokens", "w_in": "w_a", "w_down": "w_b", "out": "y"}
    op = fused_programs.from_idiom(progs.swish_mlp)
    assert op.op_names == ("ffn_act",) and op.names == ("tokens", "w_a", "w_b", "y")


def test_what_is_not_an_idiom_is_refused():
    assert idioms.recognise(progs.relu_mlp) is None          # same shape of program, another activation
    assert idioms.recognise(progs.looped) is None            # a loop is not followed
    with pytest.raises(NotImplementedError, match="no fused kernel registered"):
        ir.compile(progs.relu_mlp, platform="b200")


def test_compile_routes_a_recognised_program_to_the_fused_operator():
    compiled = ir.compile(progs.gated_mlp, platform="b200")
    assert compiled.op_names == ("ffn_swiglu",)
    compiled = ir.compile(progs.scaled_norm, platform="b200")
    assert compiled.op_names == ("rms_norm",)


def test_algebra_is_canonical():
    g, u = idioms.P("g"), idioms.P("u")
    a = idioms.mul(idioms.mul(g, idioms.sigmoid(g)), u)
    b = idioms.mul(u, idioms.mul(idioms.un("recip", idioms.add(idioms.un("exp", idioms.mul(g, idioms.C(-1))), idioms.C(1))), g))
    assert a == b
    assert idioms.add(idioms.C(1), idioms.C(2), g) == idioms.add(g, idioms.C(3))
    assert idioms.mul(g, idioms.C(0)) == idioms.C(0)


def test_the_reference_examples_are_recognised_by_their_bodies():
    """examples/models/01_ffn.py and examples/intermediate/03_normalization.py, loaded unchanged through the ``pypto``
    alias: the recogniser reads their kernels and finds the SwiGLU FFN and the RMSNorm without looking at names;
    the GELU and ReLU FFNs of the same file go to the one-projection FFN; the layer norm has no fused operator and is
    refused."""
    import importlib.util
    import os

    import ref_extract
    if not ref_extract.available():
        pytest.skip("reference tree not mounted")
    from pypto_b200 import compat
    compat.install()

    def load(rel, name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref_extract.REFERENCE_ROOT, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    ffn = load("examples/models/01_ffn.py", "ref_example_01_ffn")
    rec = idioms.recognise(ffn.ffn_swiglu)
    assert rec is not None and rec.idiom == "ffn_swiglu"
    assert rec.roles == {"x": "hidden_states", "w_gate": "gate_proj_weight", "w_up": "up_proj_weight",
                         "w_down": "down_proj_weight", "out": "output"}
    rec = idioms.recognise(ffn.ffn_gelu)
    assert rec is not None and rec.idiom == "ffn_act" and rec.constants["kind"] == 1
    assert rec.constants["alpha"] == pytest.approx(1.702)
    assert rec.roles == {"x": "hidden_states", "w_in": "gate_proj_weight", "w_down": "down_proj_weight", "out": "output"}
    rec = idioms.recognise(ffn.ffn_relu)
    assert rec is not None and rec.idiom == "ffn_act" and rec.constants == {"kind": 2}
    norm = load("examples/intermediate/03_normalization.py", "ref_example_03_norm")
    rec = idioms.recognise(norm.rms_norm)
    assert rec is not None and rec.idiom == "rms_norm" and rec.roles == {"x": "x", "gamma": "gamma", "out": "output"}
    assert rec.constants["eps"] == pytest.approx(1e-5) and rec.constants["inv_n"] == pytest.approx(1.0 / 64)
    assert idioms.recognise(norm.layer_norm) is None
    mm = load("examples/beginner/05_matmul.py", "ref_example_05_matmul")
    rec = idioms.recognise(mm.matmul_64)
    assert rec is not None and rec.idiom == "linear" and rec.roles == {"a": "a", "b": "b", "out": "c"}
    fl = load("examples/intermediate/01_fused_linear.py", "ref_example_01_fused_linear")
    rec = idioms.recognise(fl.fused_matmul_bias)
    assert rec is not None and rec.idiom == "linear" and rec.roles == {"a": "a", "b": "b", "bias": "bias", "out": "c"}
    assert idioms.recognise(fl.fused_linear_relu) is None            # relu(a @ b + bias): no fused operator for it


def test_canonical_forms_do_not_depend_on_operand_order_or_grouping():
    """Property (hypothesis): any way of writing the same product / sum of the same operands gives one canonical
    expression, and a template built one way unifies with an expression built another."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    leaves = [idioms.P(n) for n in "abcd"] + [idioms.un("exp", idioms.P("a")), ("matmul", idioms.P("a"), idioms.P("b"))]

    def build(op, items, splits):
        """Combine `items` with the binary `op` in the grouping that `splits` dictates."""
        items = list(items)
        for sp in splits:
            if len(items) < 2:
                break
            i = sp % (len(items) - 1)
            items[i:i + 2] = [op(items[i], items[i + 1])]
        while len(items) > 1:
            items[0:2] = [op(items[0], items[1])]
        return items[0]

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.sampled_from(leaves), min_size=2, max_size=5), st.randoms(use_true_random=False),
           st.lists(st.integers(0, 7), max_size=4), st.lists(st.integers(0, 7), max_size=4),
           st.sampled_from(["mul", "add"]))
    def check(items, rnd, s1, s2, op_name):
        op = getattr(idioms, op_name)
        shuffled = list(items)
        rnd.shuffle(shuffled)
        assert build(op, items, s1) == build(op, shuffled, s2)

    check()
    # unification across orderings: a template with roles against the same shape written the other way round
    x, w, u = idioms.V("x"), idioms.V("w"), idioms.V("u")
    t = idioms.mul(("matmul", x, w), idioms.sigmoid(("matmul", x, w)), u)
    e = idioms.mul(idioms.P("q"), idioms.mul(idioms.sigmoid(("matmul", idioms.P("p"), idioms.P("r"))), ("matmul", idioms.P("p"), idioms.P("r"))))
    bindings = list(idioms._unify(t, e, {}))
    assert bindings and all(b == {"x": idioms.P("p"), "w": idioms.P("r"), "u": idioms.P("q")} for b in bindings)
