"""DSL programs that compute what the fused operators compute under names of their own, for the idiom recogniser
(pypto_b200/ir/idioms.py).  Written in the style of the reference's examples (kernels that load tiles, compute and
store; an orchestration that chains them: examples/models/01_ffn.py, examples/intermediate/03_normalization.py),
with other function names, parameter names, parameter orders and algebraic spellings.  Bodies are never executed."""

import pypto_b200.language as pl

EPS = 1e-6


@pl.jit.incore
def product_kernel(lhs: pl.Tensor, rhs: pl.Tensor, dst: pl.Out[pl.Tensor]):
    l1 = pl.load(lhs, [0, 0], [64, 64], target_memory=pl.MemorySpace.Mat)
    r1 = pl.load(rhs, [0, 0], [64, 64], target_memory=pl.MemorySpace.Mat)
    acc = pl.matmul(pl.move(l1, target_memory=pl.MemorySpace.Left), pl.move(r1, target_memory=pl.MemorySpace.Right))
    pl.store(acc, [0, 0], dst)
    return dst


@pl.jit.incore
def gated_kernel(linear_part: pl.Tensor, gated_part: pl.Tensor, dst: pl.Out[pl.Tensor]):
    """dst = linear_part * (gated_part / (1 + exp(0 - gated_part))): the up operand comes FIRST here."""
    lin = pl.load(linear_part, [0, 0], [64, 64])
    g = pl.load(gated_part, [0, 0], [64, 64])
    e = pl.exp(pl.sub(0.0, g))
    swish = pl.div(g, pl.add(1.0, e))
    pl.store(pl.mul(lin, swish), [0, 0], dst)
    return dst


@pl.jit
def gated_mlp(w_out: pl.Tensor, w_lin: pl.Tensor, tokens: pl.Tensor, w_act: pl.Tensor, y: pl.Out[pl.Tensor]):
    """y = ((tokens @ w_lin) * silu(tokens @ w_act)) @ w_out: parameters in an order of its own."""
    a = pl.create_tensor([64, 64], dtype=pl.FP32)
    a = product_kernel(tokens, w_act, a)
    b = pl.create_tensor([64, 64], dtype=pl.FP32)
    b = product_kernel(tokens, w_lin, b)
    h = pl.create_tensor([64, 64], dtype=pl.FP32)
    h = gated_kernel(b, a, h)
    y = product_kernel(h, w_out, y)
    return y


@pl.jit
def scaled_norm(weight: pl.Tensor, rows: pl.Tensor, normed: pl.Out[pl.Tensor]):
    """normed = rows * rsqrt(mean(rows^2) + EPS) * weight, with the reciprocal square root and a module constant."""
    with pl.at(level=pl.Level.CORE_GROUP):
        t = pl.load(rows, [0, 0], [32, 64])
        w = pl.load(weight, [0, 0], [1, 64])
        scratch = pl.create_tile([32, 64], dtype=pl.FP32, target_memory=pl.MemorySpace.Vec)
        ssq = pl.row_sum(pl.mul(t, t), scratch)
        inv = pl.rsqrt(pl.add(pl.mul(ssq, 1.0 / 64), EPS))
        pl.store(pl.col_expand_mul(pl.row_expand_mul(t, inv), w), [0, 0], normed)
    return normed


@pl.jit
def relu_mlp(tokens: pl.Tensor, w_in: pl.Tensor, w_up: pl.Tensor, w_out: pl.Tensor, y: pl.Out[pl.Tensor]):
    """Four inputs and three products like the gated MLP, but another activation: must NOT be taken for SwiGLU."""
    a = pl.create_tensor([64, 64], dtype=pl.FP32)
    a = product_kernel(tokens, w_in, a)
    b = pl.create_tensor([64, 64], dtype=pl.FP32)
    b = product_kernel(tokens, w_up, b)
    h = pl.create_tensor([64, 64], dtype=pl.FP32)
    h = relu_gate_kernel(a, b, h)
    y = product_kernel(h, w_out, y)
    return y


@pl.jit.incore
def relu_gate_kernel(p: pl.Tensor, q: pl.Tensor, dst: pl.Out[pl.Tensor]):
    pl.store(pl.mul(pl.relu(pl.load(p, [0, 0], [64, 64])), pl.load(q, [0, 0], [64, 64])), [0, 0], dst)
    return dst


@pl.jit
def looped(tokens: pl.Tensor, w: pl.Tensor, y: pl.Out[pl.Tensor]):
    """A loop: the evaluator does not follow it and must give up rather than guess."""
    for i in pl.range(4):
        y = product_kernel(tokens, w, y)
    return y


@pl.jit
def product(lhs: pl.Tensor, rhs: pl.Tensor, dst: pl.Out[pl.Tensor]):
    """dst = lhs @ rhs through the kernel above."""
    dst = product_kernel(lhs, rhs, dst)
    return dst


@pl.jit.incore
def shift_kernel(t: pl.Tensor, offset: pl.Tensor, dst: pl.Out[pl.Tensor]):
    pl.store(pl.add(pl.load(offset, [0, 0], [64, 64]), pl.load(t, [0, 0], [64, 64])), [0, 0], dst)
    return dst


@pl.jit
def affine(offset: pl.Tensor, lhs: pl.Tensor, rhs: pl.Tensor, dst: pl.Out[pl.Tensor]):
    """dst = offset + lhs @ rhs: the bias comes first in the signature and first in the sum."""
    tmp = pl.create_tensor([64, 64], dtype=pl.FP32)
    tmp = product_kernel(lhs, rhs, tmp)
    dst = shift_kernel(tmp, offset, dst)
    return dst


@pl.program
class GatedMlpProgram:
    """The gated MLP as a @pl.program class: kernels are methods, the orchestration calls them through `self`."""

    @pl.function(type=pl.FunctionType.InCore)
    def mm(self, p: pl.Tensor[[64, 64], pl.FP32], q: pl.Tensor[[64, 64], pl.FP32],
           r: pl.Out[pl.Tensor[[64, 64], pl.FP32]]) -> pl.Tensor[[64, 64], pl.FP32]:
        acc = pl.matmul(pl.load(p, [0, 0], [64, 64]), pl.load(q, [0, 0], [64, 64]))
        pl.store(acc, [0, 0], r)
        return r

    @pl.function(type=pl.FunctionType.InCore)
    def act(self, g: pl.Tensor[[64, 64], pl.FP32], u: pl.Tensor[[64, 64], pl.FP32],
            r: pl.Out[pl.Tensor[[64, 64], pl.FP32]]) -> pl.Tensor[[64, 64], pl.FP32]:
        tg = pl.tile.load(g, [0, 0], [64, 64])
        sig = pl.recip(pl.add(pl.exp(pl.neg(tg)), 1.0))
        pl.store(pl.mul(pl.mul(tg, sig), pl.load(u, [0, 0], [64, 64])), [0, 0], r)
        return r

    @pl.function(type=pl.FunctionType.Orchestration)
    def run(self, inp: pl.Tensor[[64, 64], pl.FP32], wa: pl.Tensor[[64, 64], pl.FP32], wb: pl.Tensor[[64, 64], pl.FP32],
            wc: pl.Tensor[[64, 64], pl.FP32], res: pl.Out[pl.Tensor[[64, 64], pl.FP32]]) -> pl.Tensor[[64, 64], pl.FP32]:
        ga = pl.tensor.create([64, 64], dtype=pl.FP32)
        ga = self.mm(inp, wa, ga)
        ub = pl.tensor.create([64, 64], dtype=pl.FP32)
        ub = self.mm(inp, wb, ub)
        h = pl.tensor.create([64, 64], dtype=pl.FP32)
        h = self.act(ga, ub, h)
        res = self.mm(h, wc, res)
        return res


@pl.jit.incore
def swish_kernel(t: pl.Tensor, dst: pl.Out[pl.Tensor]):
    v = pl.load(t, [0, 0], [64, 64])
    pl.store(pl.div(v, pl.add(pl.exp(pl.neg(v)), 1.0)), [0, 0], dst)
    return dst


@pl.jit
def swish_mlp(w_b: pl.Tensor, tokens: pl.Tensor, w_a: pl.Tensor, y: pl.Out[pl.Tensor]):
    """y = silu(tokens @ w_a) @ w_b: one projection and an activation, the shape of the reference's ffn_gelu."""
    h = pl.create_tensor([64, 64], dtype=pl.FP32)
    h = product_kernel(tokens, w_a, h)
    a = pl.create_tensor([64, 64], dtype=pl.FP32)
    a = swish_kernel(h, a)
    y = product_kernel(a, w_b, y)
    return y
