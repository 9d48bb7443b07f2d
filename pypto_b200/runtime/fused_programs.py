"""Fused-operator table: orchestration entry -> CUDA kernel launcher.

Each entry knows the parameter list of one reference program (names, order, directions)
and how to turn a call into ``ChipWorker.launch(op, tensors, scalars)``.  A program whose
entry is not in the table has no kernel here and ``lookup`` raises.

(Annotations in this file must be evaluated eagerly -- the program builders below put
shapes from local variables into them -- so postponed evaluation is not enabled here.)
"""

import struct

import torch

from .. import language as pl
from ..language import Direction


class FusedOp:
    op_names: tuple[str, ...] = ()

    def matches(self, entry) -> bool:
        raise NotImplementedError

    def plan(self, compiled, host: dict, worker) -> dict:
        return {}

    def launch(self, worker, dev: dict, host: dict, plan: dict) -> None:
        raise NotImplementedError


def _host_values(t, worker) -> list[int]:
    """Integer contents of a small tensor argument, wherever it lives."""
    from .device_tensor import DeviceTensor
    if isinstance(t, DeviceTensor):
        t = worker.read_tensor(t)
    return [int(v) for v in t.flatten().tolist()]


class PagedAttentionOp(FusedOp):
    """``paged_attention(query, key_cache, value_cache, block_table, context_lens, out, config)``
    (examples/models/04_paged_attention.py:272-283).  ``config`` is the int64 tensor
    [batch, num_heads, kv_head_num, head_dim, block_size, block_num, scale_bits] (:287); an
    optional eighth entry carries q_len (an extension, 1 when absent).  The scale is taken
    from config[6] as the golden does (:489-491)."""

    op_names = ("paged_attention",)
    names = ("query", "key_cache", "value_cache", "block_table", "context_lens", "out", "config")

    def matches(self, entry) -> bool:
        return entry.name in ("paged_attention", "paged_attention_unaligned") and \
            tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        cfg = _host_values(host["config"], worker)
        if len(cfg) < 7:
            raise ValueError("config must hold at least 7 int64 entries")
        batch, heads, kvh, hd, bs, nblk, bits = cfg[:7]
        q_len = cfg[7] if len(cfg) > 7 else 1
        kvh = max(kvh, 1)
        q, out = host["query"], host["out"]
        if q.dtype != torch.bfloat16:
            raise TypeError("query must be bfloat16")
        numel = batch * q_len * heads * hd
        if _numel(q) != numel or _numel(out) != numel:
            raise ValueError(f"query/out hold {_numel(q)}/{_numel(out)} elements; config implies {numel}")
        if _numel(host["block_table"]) != batch * nblk:
            raise ValueError("block_table size does not match batch * block_num from config")
        if _numel(host["context_lens"]) != batch:
            raise ValueError("context_lens size does not match batch from config")
        return dict(scalars=[batch, heads, kvh, hd, bs, nblk, q_len, bits & 0xFFFFFFFF], host_only=("config",))

    def launch(self, worker, dev, host, plan):
        worker.launch("paged_attention", [dev[n] for n in self.names[:6]], plan["scalars"])


def _numel(t) -> int:
    n = 1
    for s in t.shape:
        n *= s
    return n


class PagedGatherOp(FusedOp):
    """``paged_gather(src, indices, block_table, out)`` with block size / column window taken
    from the shapes: out[i, :] = src[block_table[idx // bs] * bs + idx % bs, :size]
    (tests/st/runtime/ops/test_paged_gather.py:14-17).  bs = src rows / block_table length."""

    op_names = ("paged_gather",)
    names = ("src", "indices", "block_table", "out")

    def matches(self, entry) -> bool:
        return entry.name == "paged_gather" and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        src, bt, out = host["src"], host["block_table"], host["out"]
        rows, nb = src.shape[0], _numel(bt)
        if nb == 0 or rows % nb:
            raise ValueError("src rows must be a multiple of the block table length")
        return dict(scalars=[rows // nb, 0, out.shape[-1]])

    def launch(self, worker, dev, host, plan):
        worker.launch("paged_gather", [dev[n] for n in self.names], plan["scalars"])


class PagedAttentionSpmdOp(FusedOp):
    """``paged_attention_spmd(query, key_cache, value_cache, block_table, context_lens, scale, out,
    config)`` (examples/models/09_paged_attention_spmd.py:446-456): the softmax scale is a [1] fp32
    tensor and config[6] is the number of active KV blocks (the golden stops there, :604-607)."""

    op_names = ("paged_attention",)
    names = ("query", "key_cache", "value_cache", "block_table", "context_lens", "scale", "out", "config")

    def matches(self, entry) -> bool:
        return tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        from .device_tensor import DeviceTensor
        cfg = _host_values(host["config"], worker)
        batch, heads, kvh, hd, bs, nblk, active = cfg[:7]
        sc = host["scale"]
        sc = worker.read_tensor(sc) if isinstance(sc, DeviceTensor) else sc
        bits = struct.unpack("I", struct.pack("f", float(sc.flatten()[0])))[0]
        ctx = host["context_lens"]
        extra = {}
        if not isinstance(ctx, DeviceTensor) and int(ctx.max()) > active * bs:
            extra["context_lens"] = torch.clamp(ctx, max=active * bs).contiguous()   # blocks past `active` are not read
        return dict(scalars=[batch, heads, max(kvh, 1), hd, bs, nblk, 1, bits], host_only=("config", "scale"),
                    replace=extra)

    def launch(self, worker, dev, host, plan):
        order = ("query", "key_cache", "value_cache", "block_table", "context_lens", "out")
        worker.launch("paged_attention", [dev[n] for n in order], plan["scalars"])


class FfnSwigluOp(FusedOp):
    """``ffn_swiglu(hidden_states, gate_proj_weight, up_proj_weight, down_proj_weight, output)``
    (examples/models/01_ffn.py:112-131), all fp32 in the ``x @ W`` layout."""

    op_names = ("ffn_swiglu",)
    names = ("hidden_states", "gate_proj_weight", "up_proj_weight", "down_proj_weight", "output")

    def __init__(self, entry=None, names=None):
        # entry + names: a program recognised by what it computes (ir/idioms.py); `names` are ITS parameters in the
        # order x, gate weight, up weight, down weight, output
        self.entry = entry
        if names is not None:
            self.names = tuple(names)

    def matches(self, entry) -> bool:
        if self.entry is not None:
            return entry is self.entry
        return entry.name == "ffn_swiglu" and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        x, wg, wu, wd, out = (host[n] for n in self.names)
        if wg.shape != wu.shape or x.shape[1] != wg.shape[0] or wd.shape[0] != wg.shape[1] or \
                tuple(out.shape) != (x.shape[0], wd.shape[1]):
            raise ValueError("ffn_swiglu: operand shapes do not chain")
        if out.dtype != torch.float32:
            raise TypeError("ffn_swiglu: output must be float32")
        if x.shape[1] % 8 or wg.shape[1] % 32:
            raise ValueError("ffn_swiglu: hidden size must be a multiple of 8 and the intermediate size of 32")
        return {}

    def launch(self, worker, dev, host, plan):
        worker.launch("ffn_swiglu", [dev[n] for n in self.names], [])


class FfnActOp(FusedOp):
    """``ffn_gelu`` / ``ffn_relu(hidden_states, gate_proj_weight, down_proj_weight, output)``
    (examples/models/01_ffn.py:92-108, 134-150): one projection, an elementwise activation, the down projection --
    by those names, or any program recognised as computing ``f(x @ W_in) @ W_down`` with f = h * sigmoid(alpha h) or
    relu (ir/idioms.py), bound to its own parameter names."""

    op_names = ("ffn_act",)
    names = ("hidden_states", "gate_proj_weight", "down_proj_weight", "output")
    KINDS = {"ffn_gelu": (1, 1.702), "ffn_relu": (2, 0.0)}

    def __init__(self, entry=None, names=None, kind=None, alpha=0.0):
        self.entry, self.kind, self.alpha = entry, kind, float(alpha)
        if names is not None:
            self.names = tuple(names)

    def _kind(self, entry):
        return (self.kind, self.alpha) if self.entry is not None else self.KINDS[entry.name]

    def matches(self, entry) -> bool:
        if self.entry is not None:
            return entry is self.entry
        return entry.name in self.KINDS and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        x, wi, wd, out = (host[n] for n in self.names)
        if x.shape[1] != wi.shape[0] or wd.shape[0] != wi.shape[1] or tuple(out.shape) != (x.shape[0], wd.shape[1]):
            raise ValueError("ffn_act: operand shapes do not chain")
        if out.dtype != torch.float32:
            raise TypeError("ffn_act: output must be float32")
        if x.shape[1] % 8 or wi.shape[1] % 8:
            raise ValueError("ffn_act: hidden and intermediate sizes must be multiples of 8")
        kind, alpha = self._kind(compiled.entry)
        return dict(scalars=[kind, _f32_bits(alpha)])

    def launch(self, worker, dev, host, plan):
        worker.launch("ffn_act", [dev[n] for n in self.names], plan["scalars"])


class RmsNormOp(FusedOp):
    """``rms_norm(x, gamma, output)`` (examples/intermediate/03_normalization.py:34-65), eps 1e-5
    (tests/st/examples/02_intermediate/test_rms_norm.py:35)."""

    op_names = ("rms_norm",)
    names = ("x", "gamma", "output")
    eps = 1e-5
    inv_n = None

    def __init__(self, entry=None, names=None, eps=None, inv_n=None):
        # entry + names (+ constants): a program recognised by what it computes (ir/idioms.py); `names` are ITS
        # parameters in the order x, gamma, output; inv_n is the constant it multiplies the row sums by
        self.entry = entry
        if names is not None:
            self.names = tuple(names)
        if eps is not None:
            self.eps = float(eps)
        self.inv_n = inv_n

    def matches(self, entry) -> bool:
        if self.entry is not None:
            return entry is self.entry
        return entry.name == "rms_norm" and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        x, gamma = host[self.names[0]], host[self.names[1]]
        if gamma.dtype != torch.float32:
            raise TypeError("rms_norm: gamma must be float32")
        if self.inv_n is not None and abs(self.inv_n * x.shape[-1] - 1.0) > 1e-6:
            raise ValueError(f"rms_norm: the program scales the row sums by {self.inv_n}, which is not 1 / {x.shape[-1]} "
                             "(the mean over the row the fused kernel computes)")
        return dict(scalars=[struct.unpack("I", struct.pack("f", self.eps))[0]])

    def launch(self, worker, dev, host, plan):
        worker.launch("rms_norm", [dev[n] for n in self.names], plan["scalars"])


class LinearOp(FusedOp):
    """``out = a @ b`` or ``out = a @ b + bias`` of a program recognised by what it computes (ir/idioms.py;
    examples/beginner/05_matmul.py:29-38, examples/intermediate/01_fused_linear.py:60-66): the registered ``linear``
    callable with the program's own parameter names.  fp32 operands are rounded to bf16 for the tensor cores."""

    op_names = ("linear",)

    def __init__(self, entry, a: str, b: str, out: str, bias: str | None = None):
        self.entry, self.a, self.b, self.out, self.bias = entry, a, b, out, bias

    def matches(self, entry) -> bool:
        return entry is self.entry

    def plan(self, compiled, host, worker):
        a, b, out = host[self.a], host[self.b], host[self.out]
        if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0] or tuple(out.shape) != (a.shape[0], b.shape[1]):
            raise ValueError("linear: operand shapes do not chain")
        if out.dtype != torch.float32 or (self.bias is not None and (host[self.bias].dtype != torch.float32 or
                                                                     host[self.bias].shape != out.shape)):
            raise TypeError("linear: output and bias must be float32 of the product's shape")
        if a.shape[1] % 8:
            raise ValueError("linear: the inner size must be a multiple of 8")
        return {}

    def launch(self, worker, dev, host, plan):
        names = [self.a, self.b, self.out] + ([self.bias] if self.bias is not None else [])
        worker.launch("linear", [dev[n] for n in names], [0])


def _f32_bits(v: float) -> int:
    return struct.unpack("I", struct.pack("f", float(v)))[0]


class Qwen3DecodeOp(FusedOp):
    """``qwen3_decode(hidden_states, input_rms_weight, wq, wk, wv, seq_lens, rope_cos, rope_sin, k_cache, v_cache, wo,
    post_rms_weight, w_gate, w_up, w_down, out)`` (examples/models/qwen3_jit/qwen3_decode.py:49-112): one decode
    step of the layer, with grouped-query attention over the contiguous KV cache in the place the example leaves
    open (:95-99).  The caches are updated in place at position seq_len - 1, so they are read back like outputs.
    eps is the example's constant (qwen3_jit/config.py: EPS = 1e-6), the softmax scale 1 / sqrt(head_dim)."""

    op_names = ("decoder_layer",)
    names = ("hidden_states", "input_rms_weight", "wq", "wk", "wv", "seq_lens", "rope_cos", "rope_sin", "k_cache",
             "v_cache", "wo", "post_rms_weight", "w_gate", "w_up", "w_down", "out")
    eps = 1e-6

    def matches(self, entry) -> bool:
        return entry.name == "qwen3_decode" and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        h, cos, wk = host["hidden_states"], host["rope_cos"], host["wk"]
        if h.dtype != torch.bfloat16 or host["out"].dtype != torch.bfloat16:
            raise TypeError("qwen3_decode: hidden_states and out must be bfloat16")
        batch, max_seq, hd = h.shape[0], cos.shape[0], cos.shape[1]
        kvh = wk.shape[1] // hd
        if _numel(host["k_cache"]) != batch * kvh * max_seq * hd:
            raise ValueError("qwen3_decode: k_cache must hold batch * kv_heads * max_seq rows of head_dim")
        if max_seq % 128:
            raise ValueError("qwen3_decode: the cache length per sequence must be a multiple of 128")
        return dict(scalars=[_f32_bits(self.eps), 0], copy_back=("k_cache", "v_cache"))

    def launch(self, worker, dev, host, plan):
        worker.launch("decoder_layer", [dev[n] for n in self.names], plan["scalars"])


class Scope3Op(FusedOp):
    """``scope3(attn_out, hidden_states, wo, post_rms_weight, w_gate, w_up, w_down, out)``
    (tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py:207-250; golden :256-287)."""

    op_names = ("scope3",)
    names = ("attn_out", "hidden_states", "wo", "post_rms_weight", "w_gate", "w_up", "w_down", "out")
    eps = 1e-6

    def matches(self, entry) -> bool:
        return entry.name == "scope3" and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        if any(host[n].dtype != torch.bfloat16 for n in ("attn_out", "hidden_states", "wo", "w_gate", "w_up", "w_down", "out")):
            raise TypeError("scope3: activations and weights must be bfloat16")
        return dict(scalars=[_f32_bits(self.eps)])

    def launch(self, worker, dev, host, plan):
        worker.launch("scope3", [dev[n] for n in self.names], plan["scalars"])


class MatmulMxOp(FusedOp):
    """``orchestrator(a, a_scale, b, b_scale, out, out_acc)`` of the reference's MX matmul program
    (tests/st/runtime/ops/test_matmul_mx.py:203-226): out = matmul_mx(a, a_scale, b, b_scale), out_acc =
    matmul_mx_acc(out, ...).  The scale layouts come from the annotations (``pl.MX_A_ZZ`` / ``pl.MX_B_NN``)."""

    op_names = ("matmul_mx",)
    names = ("a", "a_scale", "b", "b_scale", "out", "out_acc")

    def matches(self, entry) -> bool:
        return tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        a, b = host["a"], host["b"]
        if a.element_size() != 1 or b.element_size() != 1:
            raise TypeError("matmul_mx: operands must be FP8 (the FP4 left operand of the reference's second case is "
                            "cast to FP8E4M3FN before it reaches the matmul)")
        if a.dtype != torch.float8_e4m3fn or b.dtype != torch.float8_e4m3fn:
            raise TypeError("matmul_mx: operands must be float8_e4m3fn")
        by_name = {p.name: p for p in compiled.params}
        la = 1 if getattr(by_name["a_scale"].type, "layout", None) is pl.MX_A_ZZ else 0
        lb = 2 if getattr(by_name["b_scale"].type, "layout", None) is pl.MX_B_NN else 0
        return dict(scalars=[la, lb])

    def launch(self, worker, dev, host, plan):
        worker.launch("matmul_mx", [dev[n] for n in self.names], plan["scalars"])


class LlamaMiniOp(FusedOp):
    """``llama_mini_orch(hidden, causal_mask, cos_emb, sin_emb, wq, wk, wv, w_dense, w_gate, w_up, w_down, w_lm,
    logits)`` (examples/models/08_llama_mini.py:384-483), all fp32: one kernel for the whole forward pass."""

    op_names = ("llama_mini",)
    names = ("hidden", "causal_mask", "cos_emb", "sin_emb", "wq", "wk", "wv", "w_dense", "w_gate", "w_up", "w_down",
             "w_lm", "logits")

    def matches(self, entry) -> bool:
        return entry.name == "llama_mini_orch" and tuple(p.name for p in entry.params) == self.names

    def plan(self, compiled, host, worker):
        if any(host[n].dtype != torch.float32 for n in self.names):
            raise TypeError("llama_mini_orch: every tensor must be float32")
        s, d = host["hidden"].shape
        if d % 2 or 4 * (5 * s * d + s * s) > 200 * 1024:
            raise ValueError("llama_mini_orch: head_dim must be even and 5*S*D + S*S floats must fit in 200 KB of "
                             "shared memory")
        return {}

    def launch(self, worker, dev, host, plan):
        worker.launch("llama_mini", [dev[n] for n in self.names], [])


REGISTRY: list[FusedOp] = [LlamaMiniOp(), PagedAttentionOp(), PagedAttentionSpmdOp(), PagedGatherOp(), FfnSwigluOp(), FfnActOp(), RmsNormOp(),
                           Qwen3DecodeOp(), Scope3Op(), MatmulMxOp()]


def from_idiom(entry, program=None) -> FusedOp | None:
    """A fused operator for a program that matches none by name but computes what one computes (ir/idioms.py):
    the operator is bound to the program's own parameter names."""
    from ..ir import idioms
    rec = idioms.recognise(entry, program)
    if rec is None:
        return None
    r = rec.roles
    if rec.idiom == "ffn_swiglu":
        return FfnSwigluOp(entry, (r["x"], r["w_gate"], r["w_up"], r["w_down"], r["out"]))
    if rec.idiom == "rms_norm":
        return RmsNormOp(entry, (r["x"], r["gamma"], r["out"]), eps=rec.constants.get("eps"), inv_n=rec.constants.get("inv_n"))
    if rec.idiom == "linear":
        return LinearOp(entry, r["a"], r["b"], r["out"], r.get("bias"))
    if rec.idiom == "ffn_act":
        return FfnActOp(entry, (r["x"], r["w_in"], r["w_down"], r["out"]), kind=int(rec.constants["kind"]),
                        alpha=rec.constants.get("alpha", 0.0))
    return None


def lookup(entry) -> FusedOp:
    for op in REGISTRY:
        if op.matches(entry):
            return op
    sig = ", ".join(p.name for p in entry.params)
    raise NotImplementedError(f"no fused kernel registered for program entry '{entry.name}({sig})'; "
                              "this backend runs fused operators only and has no CPU fallback")


# ---------------------------------------------------------------------------
# Programs written against the compatibility surface (same style as the reference
# examples: typed signature, DSL body never executed here).
# ---------------------------------------------------------------------------

def paged_attention_program(batch, num_heads, head_dim, block_size, max_blocks, kv_heads=1, q_len=1,
                            out_dtype=torch.float32, pool_rows=None):
    q_rows = batch * q_len * num_heads
    table = batch * max_blocks
    out_t = pl.dtype_of(out_dtype)
    cfg_len = 8 if q_len != 1 else 7
    kv_shape = [pool_rows, head_dim] if pool_rows else None
    kv_type = pl.Tensor[kv_shape, pl.BF16] if kv_shape else pl.Tensor[pl.BF16]

    @pl.program
    class PagedAttention:
        @pl.function(type=pl.FunctionType.Orchestration)
        def paged_attention(self,
                            query: pl.Tensor[[q_rows, head_dim], pl.BF16],
                            key_cache: kv_type,
                            value_cache: kv_type,
                            block_table: pl.Tensor[[table], pl.INT32],
                            context_lens: pl.Tensor[[batch], pl.INT32],
                            out: pl.Out[pl.Tensor[[q_rows, head_dim], out_t]],
                            config: pl.Tensor[[cfg_len], pl.INT64]):
            ...

    return PagedAttention


def pack_config(d: dict) -> torch.Tensor:
    """int64 config tensor for ``paged_attention_program`` from an input dict
    (batch, num_heads, kv_heads, head_dim, block_size, max_blocks, scale[, q_len])."""
    bits = struct.unpack("I", struct.pack("f", float(d["scale"])))[0]
    vals = [d["batch"], d["num_heads"], d["kv_heads"], d["head_dim"], d["block_size"], d["max_blocks"], bits]
    if d.get("q_len", 1) != 1:
        vals.append(d["q_len"])
    return torch.tensor(vals, dtype=torch.int64)


def time_resident(compiled, d, host, host_out, cfg_t, steps, dev) -> float:
    """Seconds per step with the KV pools resident on the worker as DeviceTensors (the
    reference's own benchmarking recipe: allocate once, register once, loop the handle:
    python/pypto/runtime/bench.py:1267-1340); per step the query, tables and lengths go
    host->device and the output comes back."""
    import time

    from .run_config import RunConfig
    from .worker import ChipWorker
    with ChipWorker(RunConfig(platform="b200", device_id=dev.index or 0)) as w:
        kc = w.alloc_tensor(d["key_cache"].shape, d["key_cache"].dtype, init=d["key_cache"])
        vc = w.alloc_tensor(d["value_cache"].shape, d["value_cache"].dtype, init=d["value_cache"])
        handle = w.register(compiled)
        args = (host["query"], kc, vc, host["block_table"].flatten(), host["context_lens"], host_out, cfg_t)
        handle(*args)
        t0 = time.perf_counter()
        for _ in range(steps):
            handle(*args)
        dt = (time.perf_counter() - t0) / steps
    return dt
