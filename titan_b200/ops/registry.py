"""Dispatcher registration of the sm_100a kernels: ``torch.ops.titan_b200.*``.

Every kernel launcher is also a PyTorch operator with a CUDA implementation (the ctypes call into
``libtitan_b200.so``) and a fake (meta) implementation that only computes output shapes.  That buys three things
a bare ctypes call cannot give:

* **selective activation checkpointing** sees the op: the save list (`parallel.activation_checkpoint`) names
  ``titan_b200::gemm`` and the other contraction ops, so a checkpointed block keeps their outputs instead of running
  every GEMM a second time in backward;
* **`torch.compile(fullgraph=True)`** traces through a converted model (Dynamo inlines the autograd functions of
  `titan_b200.ops.*` and finds operators with fake kernels inside);
* **meta-device runs** (the memory simulator, `--comm.mode fake_backend` dry runs) execute converted models
  without touching the GPU library.

The autograd wiring stays in the `torch.autograd.Function` classes of the op modules; they call the operators
registered here.  The counterpart in the reference is its meta registration of the fused NPU ops
(torchtitan_npu/patches/torch_npu/_meta_registrations.py:9-70).
"""

from __future__ import annotations

import torch

__all__ = ["ops", "dispatcher_ops", "CONTRACTION_OPS"]

_LIB = torch.library.Library("titan_b200", "DEF")
dispatcher_ops = torch.ops.titan_b200
_CUDA_IMPLS: dict = {}


def _define(schema: str, cuda_impl, fake_impl) -> None:
    name = schema.split("(", 1)[0]
    _LIB.define(schema)
    _LIB.impl(name, cuda_impl, "CUDA")
    torch.library.register_fake(f"titan_b200::{name}", fake_impl, lib=_LIB)
    _CUDA_IMPLS[name] = cuda_impl
    _bind(name, cuda_impl)


def _nobody_watches(args) -> bool:
    """True when a call can go straight to the launcher: no dispatch mode on the stack (selective checkpointing,
    fake tensors, the memory tracker), no compiler tracing, and a real CUDA tensor in front."""
    if torch._C._len_torch_dispatch_stack() > 0:
        return False
    for a in args:
        if isinstance(a, torch.Tensor):
            return a.is_cuda
    return False


class _Ops:
    """``ops.<name>(...)``: the dispatcher operator when somebody needs to see the call, the launcher itself otherwise.
    A Python operator call through the dispatcher costs tens of microseconds of host time; launch-bound models (small
    MoE blocks, hyper-connection kernels) feel that, so eager steps without an observer skip it.  ``ops.<name>.op`` is
    the `torch.ops` overload packet (`.default` for save lists and tests).  The attributes are created when an
    operator is defined (nothing is added lazily: a tracer may be looking)."""


ops = _Ops()


def _bind(name: str, impl) -> None:
    op = getattr(dispatcher_ops, name)

    def call(*args, **kwargs):
        if torch.compiler.is_compiling():   # checked first: the tracer folds it and never sees the rest
            return op(*args, **kwargs)
        if _nobody_watches(args):
            return impl(*args, **kwargs)
        return op(*args, **kwargs)

    call.op = op
    call.default = op.default
    call.__name__ = name
    setattr(ops, name, call)


# ---------------------------------------------------------------------------------------------- GEMM
def _gemm_cuda(a, b, a_mn=False, b_mn=False, out_fp32=False):
    from titan_b200.ops.gemm import gemm

    return gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32 if out_fp32 else None)


def _gemm_fake(a, b, a_mn=False, b_mn=False, out_fp32=False):
    m = a.shape[1] if a_mn else a.shape[0]
    n = b.shape[1] if b_mn else b.shape[0]
    return a.new_empty((m, n), dtype=torch.float32 if out_fp32 else a.dtype)


_define("gemm(Tensor a, Tensor b, bool a_mn=False, bool b_mn=False, bool out_fp32=False) -> Tensor", _gemm_cuda,
        _gemm_fake)


def _grouped_gemm_m_cuda(a, b, offs, n, b_mn):
    from titan_b200.ops.moe import _gg_m

    return _gg_m(a, b, offs, n, b_mn)


def _grouped_gemm_m_fake(a, b, offs, n, b_mn):
    return a.new_empty((a.shape[0], n))


_define("grouped_gemm_m(Tensor a, Tensor b, Tensor offs, int n, bool b_mn) -> Tensor", _grouped_gemm_m_cuda,
        _grouped_gemm_m_fake)


def _grouped_gemm_k_cuda(a, b, offs, groups):
    from titan_b200.ops.moe import _gg_k

    return _gg_k(a, b, offs, groups)


def _grouped_gemm_k_fake(a, b, offs, groups):
    return a.new_empty((groups, a.shape[1], b.shape[1]))


_define("grouped_gemm_k(Tensor a, Tensor b, Tensor offs, int groups) -> Tensor", _grouped_gemm_k_cuda,
        _grouped_gemm_k_fake)


# ---------------------------------------------------------------------------------------------- RMSNorm
def _rms_fwd_cuda(x, w, eps):
    from titan_b200.ops.norm import rms_norm_fwd

    return rms_norm_fwd(x, w, eps)


def _rms_fwd_fake(x, w, eps):
    rows = x.numel() // x.shape[-1] if x.shape[-1] else 0
    return torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty((rows,), dtype=torch.float32)


_define("rms_norm_fwd(Tensor x, Tensor w, float eps) -> (Tensor, Tensor)", _rms_fwd_cuda, _rms_fwd_fake)


def _rms_bwd_cuda(g, x, w, rstd):
    from titan_b200.ops.norm import rms_norm_bwd

    return rms_norm_bwd(g, x, w, rstd)


def _rms_bwd_fake(g, x, w, rstd):
    return torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(w)


_define("rms_norm_bwd(Tensor g, Tensor x, Tensor w, Tensor rstd) -> (Tensor, Tensor)", _rms_bwd_cuda, _rms_bwd_fake)


# ---------------------------------------------------------------------------------------------- SwiGLU
def _swiglu_fwd_cuda(gate, up, score, rows, hidden, pitch, limit):
    from titan_b200.ops.swiglu import _fwd

    return _fwd(gate, up if up is not None else gate[:, hidden:], score, rows, hidden, pitch, limit)


def _swiglu_fwd_fake(gate, up, score, rows, hidden, pitch, limit):
    return gate.new_empty((rows, hidden))


_define("swiglu_fwd(Tensor gate, Tensor? up, Tensor? score, int rows, int hidden, int pitch, float limit) -> Tensor",
        _swiglu_fwd_cuda, _swiglu_fwd_fake)


def _swiglu_bwd_cuda(gout, gate, up, score, rows, hidden, pitch, limit):
    from titan_b200.ops.swiglu import _bwd

    return _bwd(gout, gate, up, score, rows, hidden, pitch, limit)


def _swiglu_bwd_fake(gout, gate, up, score, rows, hidden, pitch, limit):
    dgate = torch.empty_like(gate)
    dup = torch.empty_like(up) if up is not None else gate.new_empty((0,))
    dscore = gout.new_empty((rows,), dtype=torch.float32) if score is not None else gout.new_empty((0,))
    return dgate, dup, dscore


_define("swiglu_bwd(Tensor gout, Tensor gate, Tensor? up, Tensor? score, int rows, int hidden, int pitch, "
        "float limit) -> (Tensor, Tensor, Tensor)", _swiglu_bwd_cuda, _swiglu_bwd_fake)


# ---------------------------------------------------------------------------------------------- RoPE
def _rope_cuda(x, cache, positions, interleaved, inverse):
    from titan_b200.ops.rope import _launch

    return _launch(x, cache, positions, interleaved, inverse)


def _rope_fake(x, cache, positions, interleaved, inverse):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


_define("rope(Tensor x, Tensor cache, Tensor? positions, bool interleaved, bool inverse) -> Tensor", _rope_cuda,
        _rope_fake)


# ---------------------------------------------------------------------------------------------- cross-entropy
def _ce_fwd_cuda(x, labels, ignore_index):
    from titan_b200.ops.cross_entropy import _fwd_rows

    return _fwd_rows(x, labels, ignore_index)


def _ce_fwd_fake(x, labels, ignore_index):
    rows = x.shape[0]
    return x.new_empty((rows,), dtype=torch.float32), x.new_empty((rows,), dtype=torch.float32)


_define("cross_entropy_fwd(Tensor x, Tensor labels, int ignore_index) -> (Tensor, Tensor)", _ce_fwd_cuda, _ce_fwd_fake)


def _ce_bwd_cuda(x, labels, lse, gscale, ignore_index):
    from titan_b200.ops.cross_entropy import _bwd_rows

    return _bwd_rows(x, labels, lse, gscale, ignore_index, False)


def _ce_bwd_fake(x, labels, lse, gscale, ignore_index):
    return torch.empty_like(x)


_define("cross_entropy_bwd(Tensor x, Tensor labels, Tensor lse, Tensor gscale, int ignore_index) -> Tensor",
        _ce_bwd_cuda, _ce_bwd_fake)


def _ce_bwd_inplace_cuda(x, labels, lse, gscale, ignore_index):
    from titan_b200.ops.cross_entropy import _bwd_rows

    _bwd_rows(x, labels, lse, gscale, ignore_index, True)


def _ce_bwd_inplace_fake(x, labels, lse, gscale, ignore_index):
    return None


# the gradient overwrites the logits (the vocabulary-sized tensor is not held twice)
_define("cross_entropy_bwd_(Tensor(a!) x, Tensor labels, Tensor lse, Tensor gscale, int ignore_index) -> ()",
        _ce_bwd_inplace_cuda, _ce_bwd_inplace_fake)


# ---------------------------------------------------------------------------------------------- flash attention
def _flash_fwd_cuda(q, k, v, scale, seq_start=None):
    from titan_b200.ops.flash_attention import _flash_fwd_launch

    return _flash_fwd_launch(q, k, v, scale, seq_start)


def _flash_fwd_fake(q, k, v, scale, seq_start=None):
    b, h, s, d = q.shape
    return q.new_empty((b, s, h, v.shape[-1])).transpose(1, 2), q.new_empty((b, h, s), dtype=torch.float32)


_define("flash_attention_fwd(Tensor q, Tensor k, Tensor v, float scale, Tensor? seq_start=None) -> (Tensor, Tensor)",
        _flash_fwd_cuda, _flash_fwd_fake)


def _flash_bwd_cuda(q, k, v, out, lse, g, scale, seq_start=None):
    from titan_b200.ops.flash_attention import _flash_bwd_launch

    return _flash_bwd_launch(q, k, v, out, lse, g, scale, seq_start)


def _flash_bwd_fake(q, k, v, out, lse, g, scale, seq_start=None):
    def like(t):
        b, h, s, d = t.shape
        return t.new_empty((b, s, h, d)).transpose(1, 2)

    return like(q), like(k), like(v)


_define("flash_attention_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, Tensor grad, float scale, "
        "Tensor? seq_start=None) -> (Tensor, Tensor, Tensor)", _flash_bwd_cuda, _flash_bwd_fake)


# ---------------------------------------------------------------------------------------------- sparse attention
def _sparse_mla_fwd_cuda(q, kv, idx, scale, dv, sink=None):
    from titan_b200.ops.sparse_mla import sparse_mla_forward

    return sparse_mla_forward(q, kv, idx, scale, dv, sink)


def _sparse_mla_fwd_fake(q, kv, idx, scale, dv, sink=None):
    s, h, _ = q.shape
    return (q.new_empty((s, h, dv)), q.new_empty((s, h), dtype=torch.float32),
            q.new_empty((s, idx.shape[1]), dtype=torch.float32))


_define("sparse_mla_fwd(Tensor q, Tensor kv, Tensor idx, float scale, int dv, Tensor? sink=None) -> "
        "(Tensor, Tensor, Tensor)", _sparse_mla_fwd_cuda, _sparse_mla_fwd_fake)


def _indexer_topk_cuda(q_idx, weights, k_idx, topk, pos_offset=0, ratio=1):
    from titan_b200.ops.dsa import _indexer_topk_launch

    return _indexer_topk_launch(q_idx, weights, k_idx, topk, pos_offset, ratio)


def _indexer_topk_fake(q_idx, weights, k_idx, topk, pos_offset=0, ratio=1):
    b, s = q_idx.shape[0], q_idx.shape[1]
    return q_idx.new_empty((b, s, topk), dtype=torch.int32), q_idx.new_empty((b, s, topk), dtype=torch.float32)


_define("indexer_topk(Tensor q_idx, Tensor weights, Tensor k_idx, int topk, int pos_offset=0, int ratio=1) -> "
        "(Tensor, Tensor)", _indexer_topk_cuda, _indexer_topk_fake)


# ---------------------------------------------------------------------------------------------- MXFP8 linear
def _mx_linear_fwd_cuda(x2, w, round_mode, need_wgrad, atoms):
    from titan_b200.lowp.mx_linear import _mx_linear_fwd

    return _mx_linear_fwd(x2, w, round_mode, need_wgrad, atoms)


def _mx_linear_fwd_fake(x2, w, round_mode, need_wgrad, atoms):
    m, k = x2.shape
    y = x2.new_empty((m, w.shape[0]))
    if not need_wgrad:
        return y, x2.new_empty((0,), dtype=torch.float8_e4m3fn), x2.new_empty((0,), dtype=torch.uint8)
    return (y, x2.new_empty((k, m), dtype=torch.float8_e4m3fn),
            x2.new_empty((k * m // 32,), dtype=torch.uint8))


_define("mx_linear_fwd(Tensor x, Tensor w, str round_mode, bool need_wgrad, bool atoms) -> (Tensor, Tensor, Tensor)",
        _mx_linear_fwd_cuda, _mx_linear_fwd_fake)


# Ops whose outputs selective activation checkpointing keeps (contractions and the sparse-attention selection:
# recomputing them costs real FLOPs, their outputs are small next to what they read).
CONTRACTION_OPS = (ops.gemm.default, ops.grouped_gemm_m.default, ops.grouped_gemm_k.default,
                   ops.flash_attention_fwd.default, ops.sparse_mla_fwd.default, ops.indexer_topk.default,
                   ops.mx_linear_fwd.default)


# The SwiGLU output is the input of the down projection (needed again for its weight gradient) and the largest tensor
# a checkpointed block would otherwise rebuild: keeping it costs hidden_dim * 2 bytes per token and layer.  Recipes
# opt in (`activation_checkpoint.selective_keep_swiglu`): MoE blocks would keep capacity-sized expert buffers.
SWIGLU_OPS = (ops.swiglu_fwd.default,)


def _register_with_sac() -> None:
    from titan_b200.parallel.activation_checkpoint import register_sac_save_op

    for op in CONTRACTION_OPS:
        register_sac_save_op(op)


_register_with_sac()
