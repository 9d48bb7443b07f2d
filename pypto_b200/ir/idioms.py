"""Idiom recognition over DSL programs: route a program to a fused kernel by what it COMPUTES, not by its name.

The reference lowers every program through its own parser and pass pipeline; this backend runs fused operators and
looks an entry up by name and signature (``runtime/fused_programs.py``).  A program that spells the same computation
with other function or parameter names would miss that table.  This module reads the bodies of the entry and of the
kernels it calls (Python ``ast``; nothing is executed), evaluates them symbolically into one expression per output
tensor and unifies that expression with the algebraic form of a fused operator:

* SwiGLU FFN (examples/models/01_ffn.py:37-131)::

      out = (silu(x @ Wg) * (x @ Wu)) @ Wd,     silu(g) = g * recip(1 + exp(-g))

* RMSNorm (examples/intermediate/03_normalization.py:34-65)::

      out = x / sqrt(c * row_sum(x * x) + eps) * gamma          (or  x * rsqrt(...) * gamma)

* the one-projection FFNs of the same file (examples/models/01_ffn.py:51-62, 80-108, 134-150)::

      out = f(x @ W_in) @ W_down,    f(h) = h * recip(1 + exp(-alpha h))  (GELU: alpha = 1.702)   or   f = relu

* a matrix product, alone or with a full-size bias (examples/beginner/05_matmul.py:29-38,
  examples/intermediate/01_fused_linear.py:60-66)::

      out = a @ b                    out = a @ b + bias

Products and sums are flattened, constants folded and operands matched in any order, so ``mul(up, swish)`` is the same
as ``mul(swish, up)`` and ``sub(0, g)`` the same as ``mul(g, -1)``.  The match binds the roles (x, Wg, Wu, Wd, out, ...)
to the entry's own parameter names and the constants (eps) to their values.  What the evaluator does not follow -- a
loop, a branch, an operation outside the table below -- makes it give up; the caller then reports the program as
unknown.  Tiling arguments of ``load`` / ``store`` (offsets, tile shapes, memory spaces) are ignored: a kernel is read
as acting on whole tensors, which is what the straight-line examples do; the fused operator checks the real shapes
when the program is planned.
"""

from __future__ import annotations

import ast
import itertools
import textwrap

from ..language import Direction, Function


class _GiveUp(Exception):
    pass


# ---------------------------------------------------------------------------------------------------------------
# Expressions: nested tuples.  ("param", name) | ("const", v) | ("var", role) | (op, child, ...)
# "mul" and "add" are n-ary and commutative; every other op keeps its operand order.
# ---------------------------------------------------------------------------------------------------------------

def P(name):
    return ("param", name)


def C(v):
    return ("const", float(v))


def V(role):
    """Pattern variable of a template: binds to an entry parameter ("x", "w_gate", ...) or, for names starting with
    '#', to a constant."""
    return ("var", role)


def _nary(op, items, identity):
    flat, const = [], identity
    for it in items:
        if it[0] == op:
            it_children = it[1:]
        else:
            it_children = (it,)
        for c in it_children:
            if c[0] == "const":
                const = const * c[1] if op == "mul" else const + c[1]
            else:
                flat.append(c)
    if op == "mul" and const == 0.0:
        return C(0.0)
    if const != identity or not flat:
        flat.append(C(const))
    if len(flat) == 1:
        return flat[0]
    return (op, *sorted(flat, key=repr))


def mul(*xs):
    return _nary("mul", xs, 1.0)


def add(*xs):
    return _nary("add", xs, 0.0)


def un(op, x):
    if op == "recip" and x[0] == "const" and x[1] != 0.0:
        return C(1.0 / x[1])
    return (op, x)


def sigmoid(x):
    return un("recip", add(C(1.0), un("exp", mul(C(-1.0), x))))


# ---------------------------------------------------------------------------------------------------------------
# Symbolic evaluation of a DSL body
# ---------------------------------------------------------------------------------------------------------------

_UNARY = {"exp", "recip", "sqrt", "rsqrt", "relu", "abs", "log", "tanh"}
_PASS_THROUGH = {"move", "reshape", "view", "assemble"}          # change layout or placement, not values
_FRESH = {"create_tensor", "create_tile", "create", "zeros_like", "empty"}  # scratch to be written later


class _Evaluator:
    def __init__(self, functions, namespace, depth=0):
        self.functions, self.ns, self.depth = functions, namespace, depth

    # -- values -------------------------------------------------------------------------------------------------
    def number(self, node):
        try:
            v = eval(compile(ast.Expression(node), "<dsl>", "eval"), dict(self.ns))  # noqa: S307 - module constants
        except Exception:
            raise _GiveUp(f"'{ast.unparse(node)}' is neither a tensor value nor a constant")
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise _GiveUp(f"'{ast.unparse(node)}' is not a number")
        return C(v)

    def value(self, node, env):
        if isinstance(node, ast.Name) and node.id in env:
            return env[node.id]
        if isinstance(node, ast.Call):
            return self.call(node, env)
        return self.number(node)

    def callee(self, node):
        if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id == "self":
            return self.functions.get(node.attr)
        if isinstance(node, ast.Name):
            f = self.ns.get(node.id)
            return f if isinstance(f, Function) else None
        return None

    def call(self, node, env):
        fn = self.callee(node.func)
        if fn is not None:
            return self.kernel_call(fn, node, env)
        f = node.func
        root = f.value if isinstance(f, ast.Attribute) else None
        if isinstance(root, ast.Attribute) and root.attr in ("tile", "tensor") and isinstance(root.value, ast.Name):
            root = root.value                           # pl.tile.<op> / pl.tensor.<op>: the same operations, namespaced
        if not (isinstance(root, ast.Name) and root.id in ("pl", "pld")):
            raise _GiveUp(f"call '{ast.unparse(f)}' is not a DSL operation")
        op, a = f.attr, node.args
        if op == "load":
            return self.value(a[0], env)
        if op in _PASS_THROUGH:
            return self.value(a[0], env)
        if op in _FRESH:
            return ("fresh",)
        if op == "store":                               # store(value, offsets, tensor)
            if len(a) < 3 or not isinstance(a[2], ast.Name):
                raise _GiveUp("store without a named destination")
            env[a[2].id] = self.value(a[0], env)
            return env[a[2].id]
        if op in _UNARY:
            return un(op, self.value(a[0], env))
        if op == "neg":
            return mul(C(-1.0), self.value(a[0], env))
        if op in ("mul", "muls"):
            return mul(self.value(a[0], env), self.value(a[1], env))
        if op in ("add", "adds"):
            return add(self.value(a[0], env), self.value(a[1], env))
        if op in ("sub", "subs"):
            return add(self.value(a[0], env), mul(C(-1.0), self.value(a[1], env)))
        if op in ("div", "divs"):
            return mul(self.value(a[0], env), un("recip", self.value(a[1], env)))
        if op == "matmul":
            return ("matmul", self.value(a[0], env), self.value(a[1], env))
        if op in ("row_sum", "row_max"):                # (tile, scratch) -> one value per row
            return (op, self.value(a[0], env))
        if op in ("row_expand_mul", "row_expand_div", "row_expand_add", "row_expand_sub"):
            v = ("per_row", self.value(a[1], env))      # the second operand holds one value per row
            x = self.value(a[0], env)
            return {"row_expand_mul": mul(x, v), "row_expand_div": mul(x, un("recip", v)), "row_expand_add": add(x, v),
                    "row_expand_sub": add(x, mul(C(-1.0), v))}[op]
        if op in ("col_expand_mul", "col_expand_div", "col_expand_add", "col_expand_sub"):
            v = ("per_col", self.value(a[1], env))      # the second operand holds one value per column
            x = self.value(a[0], env)
            return {"col_expand_mul": mul(x, v), "col_expand_div": mul(x, un("recip", v)), "col_expand_add": add(x, v),
                    "col_expand_sub": add(x, mul(C(-1.0), v))}[op]
        raise _GiveUp(f"operation pl.{op} is not in the evaluator's table")

    # -- functions ----------------------------------------------------------------------------------------------
    def kernel_call(self, fn, node, env):
        if self.depth > 8:
            raise _GiveUp("call depth")
        if node.keywords:
            raise _GiveUp("keyword arguments in a kernel call")
        params = [p for p in fn.params]
        if len(node.args) != len(params):
            raise _GiveUp(f"{fn.name}: {len(node.args)} arguments for {len(params)} parameters")
        bound = {}
        for p, a in zip(params, node.args):
            bound[p.name] = self.value(a, env) if p.is_tensor or isinstance(a, ast.Name) and a.id in env else self.number(a)
        outs, ret = evaluate_function(fn, bound, self.functions, self.depth + 1)
        # what the callee stored into its output parameters is what the caller's tensors now hold
        for p, a in zip(params, node.args):
            if p.direction != Direction.In and p.name in outs and isinstance(a, ast.Name):
                env[a.id] = outs[p.name]
        if ret is None:
            written = [outs[p.name] for p in params if p.direction != Direction.In and p.name in outs]
            ret = written[-1] if written else ("fresh",)
        return ret

    def block(self, stmts, env):
        ret = None
        for st in stmts:
            if isinstance(st, ast.Expr) and isinstance(st.value, ast.Constant):
                continue                                                     # docstring
            if isinstance(st, ast.Expr) and isinstance(st.value, ast.Call):
                self.call(st.value, env)
            elif isinstance(st, (ast.Assign, ast.AnnAssign)):
                target = st.targets[0] if isinstance(st, ast.Assign) else st.target
                if (isinstance(st, ast.Assign) and len(st.targets) != 1) or not isinstance(target, ast.Name) or st.value is None:
                    raise _GiveUp("assignment to something other than one name")
                env[target.id] = self.value(st.value, env)
            elif isinstance(st, ast.With):
                ret = self.block(st.body, env)                               # `with pl.at(...)`: placement only
                if ret is not None:
                    return ret
            elif isinstance(st, ast.Return):
                if st.value is None:
                    return ("none",)
                if isinstance(st.value, ast.Name) and st.value.id in env:
                    return env[st.value.id]
                raise _GiveUp("return of something other than a tensor name")
            elif isinstance(st, ast.Pass):
                continue
            else:
                raise _GiveUp(f"statement {type(st).__name__} is not followed")
        return ret


def _namespace(fn) -> dict:
    ns = dict(getattr(fn, "__globals__", {}))
    if getattr(fn, "__closure__", None):
        for name, cell in zip(fn.__code__.co_freevars, fn.__closure__):
            try:
                ns[name] = cell.cell_contents
            except ValueError:
                pass
    return ns


def evaluate_function(fn: Function, bound: dict, functions: dict, depth: int = 0):
    """({output parameter: expression}, returned expression) of ``fn`` with its parameters bound to ``bound``."""
    if not fn.source:
        raise _GiveUp(f"{fn.name}: no source")
    try:
        tree = ast.parse(textwrap.dedent(fn.source))
    except SyntaxError:
        raise _GiveUp(f"{fn.name}: source does not parse")
    fdef = next((n for n in ast.walk(tree) if isinstance(n, ast.FunctionDef)), None)
    if fdef is None:
        raise _GiveUp(f"{fn.name}: no function definition")
    env = dict(bound)
    ret = _Evaluator(functions, _namespace(fn.fn), depth).block(fdef.body, env)
    outs = {p.name: env[p.name] for p in fn.params if p.direction != Direction.In and p.name in env}
    if ret is not None and ret[0] == "none":
        ret = None
    return outs, ret


# ---------------------------------------------------------------------------------------------------------------
# Unification of an expression with a template
# ---------------------------------------------------------------------------------------------------------------

def _unify(t, e, b):
    """Yield every extension of binding ``b`` under which template ``t`` equals expression ``e``."""
    if t[0] == "var":
        role = t[1]
        want_const = role.startswith("#")
        if (e[0] == "const") != want_const or (not want_const and e[0] != "param"):
            return
        if role in b:
            if b[role] == e:
                yield b
            return
        if not want_const and e in b.values():        # two roles never share a tensor
            return
        yield {**b, role: e}
        return
    if t[0] in ("param", "const"):
        if t == e:
            yield b
        return
    if t[0] != e[0] or len(t) != len(e):
        return
    if t[0] in ("mul", "add"):
        for perm in itertools.permutations(e[1:]):
            yield from _unify_seq(t[1:], perm, b)
        return
    yield from _unify_seq(t[1:], e[1:], b)


def _unify_seq(ts, es, b):
    if not ts:
        yield b
        return
    for b1 in _unify(ts[0], es[0], b):
        yield from _unify_seq(ts[1:], es[1:], b1)


def _swiglu_ffn_template():
    x, wg, wu, wd = V("x"), V("w_gate"), V("w_up"), V("w_down")
    gate, up = ("matmul", x, wg), ("matmul", x, wu)
    return ("matmul", mul(gate, sigmoid(gate), up), wd)


def _rms_norm_templates():
    x, gamma = V("x"), V("gamma")
    mean_sq = add(mul(V("#inv_n"), ("row_sum", mul(x, x))), V("#eps"))
    yield mul(x, un("recip", ("per_row", un("sqrt", mean_sq))), ("per_col", gamma))
    yield mul(x, ("per_row", un("rsqrt", mean_sq)), ("per_col", gamma))
    yield mul(x, ("per_row", un("recip", un("sqrt", mean_sq))), ("per_col", gamma))


class Recognised:
    """What a program computes: the fused operator's name, the entry parameter that plays each role, constants."""

    def __init__(self, idiom: str, roles: dict, constants: dict):
        self.idiom, self.roles, self.constants = idiom, roles, constants

    def __repr__(self):
        return f"Recognised({self.idiom}, {self.roles}, {self.constants})"


def recognise(entry: Function, program=None) -> Recognised | None:
    """The idiom ``entry`` computes, or None when its body is not followed or matches no fused operator."""
    functions = dict(getattr(program, "functions", {}) or {})
    tensors = [p for p in entry.params if p.is_tensor]
    outs_decl = [p for p in tensors if p.direction != Direction.In]
    if len(outs_decl) != 1 or len(tensors) != len(entry.params):
        return None
    try:
        outs, ret = evaluate_function(entry, {p.name: P(p.name) for p in tensors}, functions)
    except _GiveUp:
        return None
    out_name = outs_decl[0].name
    expr = outs.get(out_name)
    if expr is None or expr == P(out_name):
        return None
    n_in = len(tensors) - 1

    def finish(idiom, b):
        roles = {r: v[1] for r, v in b.items() if not r.startswith("#")}
        if len(roles) != n_in:                            # every input tensor takes part
            return None
        roles["out"] = out_name
        return Recognised(idiom, roles, {r[1:]: v[1] for r, v in b.items() if r.startswith("#")})

    if n_in == 4:
        for b in _unify(_swiglu_ffn_template(), expr, {}):
            r = finish("ffn_swiglu", b)
            if r is not None:
                return r
    if n_in == 2:
        for t in _rms_norm_templates():
            for b in _unify(t, expr, {}):
                r = finish("rms_norm", b)
                if r is not None:
                    return r
        for b in _unify(("matmul", V("a"), V("b")), expr, {}):
            r = finish("linear", b)
            if r is not None:
                return r
    if n_in == 3:
        h = ("matmul", V("x"), V("w_in"))
        for b in _unify(("matmul", mul(h, un("recip", add(C(1.0), un("exp", mul(V("#neg_alpha"), h))))), V("w_down")), expr, {}):
            r = finish("ffn_act", b)
            if r is not None and r.constants["neg_alpha"] < 0:
                r.constants = {"kind": 1, "alpha": -r.constants["neg_alpha"]}
                return r
        for b in _unify(("matmul", un("relu", h), V("w_down")), expr, {}):
            r = finish("ffn_act", b)
            if r is not None:
                r.constants = {"kind": 2}
                return r
        for b in _unify(add(("matmul", V("a"), V("b")), V("bias")), expr, {}):
            r = finish("linear", b)
            if r is not None:
                return r
    return None
