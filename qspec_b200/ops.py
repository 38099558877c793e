"""Tensor-level operators over the C-ABI library.

The function names and argument meaning mirror the reference's native entry points
 so `quarot_nn`-style callers can switch by changing the import:

  layernorm_ops.rms_norm_general_fuse_sum_i4   third-party/kernels/csrc/layernorm.cpp:32-38
  layernorm_ops.rms_norm_general_fuse_sum_fp16 third-party/kernels/csrc/layernorm.cpp:40-42
  quarot._CUDA.fuse_sym_quant                  third-party/QuaRot/quarot/kernels/bindings.cpp:128-146
  faster_fast_hadamard_transform               third-party/fast-hadamard-transform/csrc/fast_hadamard_transform.cpp:69-110
  rowwise_scaled_linear_cutlass_s4s4_unified   third-party/ao/torchao/ops.py:600-636
  bitblas Matmul (W4A16)                       vllm/model_executor/layers/quarot_nn/linear.py:156-211

All outputs are caller-allocated, contiguous, on the same CUDA device; launches go to
torch.cuda.current_stream(). PyTorch is used for memory and streams only.
"""
from __future__ import annotations

from typing import Optional

import os

import torch

from . import _lib

_F16 = torch.float16
_BF16 = torch.bfloat16


def _dt(t: torch.Tensor) -> int:
    if t.dtype == _F16:
        return _lib.DTYPE_F16
    if t.dtype == _BF16:
        return _lib.DTYPE_BF16
    raise ValueError(f"expected float16 or bfloat16 tensor, got {t.dtype}")


def _stream() -> int:
    # the raw handle of the current stream of the current device, without building a torch.cuda.Stream object per launch
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def _chk(t: Optional[torch.Tensor], name: str, dtypes=None, allow_none=False):
    if t is None:
        if allow_none:
            return
        raise ValueError(f"{name} must not be None")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (qspec_b200 has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise ValueError(f"{name}: dtype {t.dtype} not in {dtypes}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_I4 = (torch.int8, torch.uint8)

# ---------------------------------------------------------------------------------------------
# workspaces: one zero-initialised, self-cleaning buffer per (device, kind); grown on demand.
# A workspace that has been handed out is never freed: a CUDA graph captured earlier keeps its pointer (and relies on
# its counter region being zero), so growth allocates a new block and retires the old one alive. Use is single-stream
# per device: two streams running GEMMs of the same kind concurrently would share the tile counters -- give a second
# stream its own workspace through the C ABI (include/qspec_b200.h) instead.
# ---------------------------------------------------------------------------------------------
_workspaces: dict = {}
_retired: list = []


def _workspace(kind: str, nbytes: int, device: torch.device) -> torch.Tensor:
    key = (kind, device.index if device.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reserve_workspaces(max_tokens: int, shapes, device) -> None:
    """Pre-size both GEMM workspaces (call before CUDA-graph capture). shapes = [(N, K), ...]."""
    lib = _lib.load()
    device = torch.device(device)
    n4 = max(lib.qspec_gemm_w4a4_workspace_bytes(max_tokens, n, k) for n, k in shapes)
    n16 = max(lib.qspec_gemm_w4a16_workspace_bytes(m, n, k) for n, k in shapes
              for m in sorted({1, 8, 16, 32, 64, max_tokens}) if m <= max(max_tokens, 1))
    _workspace("w4a4", n4, device)
    _workspace("w4a16", n16, device)


# ---------------------------------------------------------------------------------------------
# (A) norm (+quant)
# ---------------------------------------------------------------------------------------------

def rms_norm_general_fuse_sum_i4(out_q: torch.Tensor, x: torch.Tensor, input_sum: Optional[torch.Tensor],
                                 scaling: torch.Tensor, eps: float, use_per_token_quant: bool = True) -> None:
    if not use_per_token_quant:
        raise NotImplementedError("only the per-token branch is on the QSpec path (layernorm_kernels.cu:903)")
    _chk(x, "input", (_F16,)); _chk(out_q, "out", _I4); _chk(scaling, "scaling", (_F16,))
    _chk(input_sum, "input_sum", (_F16,), allow_none=True)
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if out_q.numel() != rows * K // 2 or scaling.numel() < rows:
        raise ValueError("rms_norm_general_fuse_sum_i4: output shapes do not match the input")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_norm_quant_i4(_ptr(x), _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K,
                                       float(eps), _stream()), "rms_norm_general_fuse_sum_i4")


def add_rms_norm_fuse_sum_i4(out_q: torch.Tensor, x: torch.Tensor, delta: torch.Tensor, input_sum: Optional[torch.Tensor],
                             scaling: torch.Tensor, eps: float) -> None:
    """x += delta (in place), then rms_norm_general_fuse_sum_i4(out_q, x, ...): one launch (quarot_llama.py:380,389)."""
    _chk(x, "input", (_F16,)); _chk(delta, "delta", (_F16,)); _chk(out_q, "out", _I4); _chk(scaling, "scaling", (_F16,))
    _chk(input_sum, "input_sum", (_F16,), allow_none=True)
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if delta.numel() != x.numel() or out_q.numel() != rows * K // 2 or scaling.numel() < rows:
        raise ValueError("add_rms_norm_fuse_sum_i4: shapes do not match the input")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_add_norm_quant_i4(_ptr(x), _ptr(delta), _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K,
                                           float(eps), _stream()), "add_rms_norm_fuse_sum_i4")


def add_rms_norm_fuse_sum_fp16(out: torch.Tensor, x: torch.Tensor, delta: torch.Tensor, eps: float) -> None:
    """x += delta (in place), then rms_norm_general_fuse_sum_fp16(out, x, eps): one launch."""
    _chk(x, "input", (_F16, _BF16)); _chk(delta, "delta", (x.dtype,)); _chk(out, "out", (x.dtype,))
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if out.numel() != x.numel() or delta.numel() != x.numel():
        raise ValueError("add_rms_norm_fuse_sum_fp16: out and delta must have the input's shape")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_add_norm_f16(_ptr(x), _ptr(delta), _ptr(out), rows, K, float(eps), _dt(x), _stream()),
               "add_rms_norm_fuse_sum_fp16")


def tp_two_step(peers, rows: int) -> bool:
    """Which form of the fused all-reduce an exchange of `rows` token rows uses -- a function of (rows, world) only, so every
    rank decides alike. Two-step (row r summed by rank r % world, pushed to the peers) when (world - 1) * rows >=
    QSPEC_TP_SCATTER_MIN. OFF by default: measured on 8 x B200 (profiles/r02s_two_step_ab.md) the one-step form is not bound by
    the (world - 1) x rows x K x 2 bytes every rank reads but by the hand-over latency between GPUs, and the second hand-over of
    the two-step form costs more than its smaller traffic saves (TP = 8: -1 % on the 256-token verify exchanges alone, +10 % with
    the 64-token draft exchanges too; TP = 4: +4 %). Kept as a tested option for larger exchanges (prefill-sized passes)."""
    if not hasattr(peers, "_reduced"):
        return False
    return (peers.world - 1) * rows >= int(os.environ.get("QSPEC_TP_SCATTER_MIN", str(1 << 30))) and rows <= 1024


def tp_add_rms_norm_fuse_sum_i4(out_q: torch.Tensor, x: torch.Tensor, peers, which: int, input_sum: torch.Tensor,
                                scaling: torch.Tensor, eps: float, phases: int = 3, c8: bool = False) -> None:
    """x += sum over ranks of peers.partial(which) (rank order, fp32, one rounding), then the quantising norm:
    the all-reduce of RowParallelLinear.forward (layers/linear.py:1143-1144) fused into the consumer."""
    _chk(x, "input", (_F16,)); _chk(out_q, "out", _I4); _chk(scaling, "scaling", (_F16,)); _chk(input_sum, "input_sum", (_F16,))
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if K != peers.hidden or rows > peers.max_tokens or rows == 0 or peers.buf.dtype != x.dtype:
        raise ValueError("tp_add_rms_norm_fuse_sum_i4: input does not match the peer partial buffers")
    lib = _lib.load()
    _check_container(out_q, rows, K, c8, "tp_add_rms_norm_fuse_sum_i4")
    if c8:
        _lib.check(lib.qspec_tp_add_norm_quant_i4_c8(_ptr(x), peers._partials[which], peers._flags, _ptr(peers.state), peers.world,
                                                     peers.rank, _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K,
                                                     float(eps), _stream()), "tp_add_rms_norm_fuse_sum_i4 (int8 container)")
        return
    if tp_two_step(peers, rows):
        _lib.check(lib.qspec_tp_rs_add_norm_quant_i4(_ptr(x), peers._partials[which], peers._flags, peers._reduced[which],
                                                     peers._row_flags, _ptr(peers.state), peers.world, peers.rank, phases,
                                                     _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K, float(eps),
                                                     _stream()), "tp_add_rms_norm_fuse_sum_i4 (two-step)")
        return
    _lib.check(lib.qspec_tp_add_norm_quant_i4(_ptr(x), peers._partials[which], peers._flags, _ptr(peers.state), peers.world,
                                              peers.rank, _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K,
                                              float(eps), _stream()), "tp_add_rms_norm_fuse_sum_i4")


def tp_add_rms_norm_fuse_sum_fp16(out: torch.Tensor, x: torch.Tensor, peers, which: int, eps: float, phases: int = 3) -> None:
    _chk(x, "input", (_F16, _BF16)); _chk(out, "out", (x.dtype,))
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if K != peers.hidden or rows > peers.max_tokens or rows == 0 or peers.buf.dtype != x.dtype or out.numel() != x.numel():
        raise ValueError("tp_add_rms_norm_fuse_sum_fp16: input does not match the peer partial buffers")
    lib = _lib.load()
    if tp_two_step(peers, rows):
        _lib.check(lib.qspec_tp_rs_add_norm_f16(_ptr(x), peers._partials[which], peers._flags, peers._reduced[which],
                                                peers._row_flags, _ptr(peers.state), peers.world, peers.rank, phases,
                                                _ptr(out), rows, K, float(eps), _dt(x), _stream()),
                   "tp_add_rms_norm_fuse_sum_fp16 (two-step)")
        return
    _lib.check(lib.qspec_tp_add_norm_f16(_ptr(x), peers._partials[which], peers._flags, _ptr(peers.state), peers.world,
                                         peers.rank, _ptr(out), rows, K, float(eps), _dt(x), _stream()),
               "tp_add_rms_norm_fuse_sum_fp16")


def rms_norm_general_fuse_sum_fp16(out: torch.Tensor, x: torch.Tensor, eps: float) -> None:
    _chk(x, "input", (_F16, _BF16)); _chk(out, "out", (x.dtype,))
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if out.numel() != x.numel():
        raise ValueError("rms_norm_general_fuse_sum_fp16: out must have the input's shape")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_norm_f16(_ptr(x), _ptr(out), rows, K, float(eps), _dt(x), _stream()),
               "rms_norm_general_fuse_sum_fp16")


# ---------------------------------------------------------------------------------------------
# quantiser
# ---------------------------------------------------------------------------------------------

def fuse_sym_quant(x: torch.Tensor, scale: torch.Tensor, q: torch.Tensor, input_clip_ratio: float = 1.0) -> None:
    _chk(x, "x", (_F16,)); _chk(scale, "scale", (_F16,)); _chk(q, "q", _I4)
    if x.dim() != 2:
        raise ValueError("fuse_sym_quant: x must be 2-D")
    rows, K = x.shape
    if q.numel() != rows * K // 2 or scale.numel() < rows:
        raise ValueError("fuse_sym_quant: output shapes do not match the input")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_sym_quant_i4(_ptr(x), _ptr(scale), _ptr(q), rows, K, float(input_clip_ratio),
                                      _stream()), "fuse_sym_quant")


# ---------------------------------------------------------------------------------------------
# (B) Hadamard
# ---------------------------------------------------------------------------------------------

def faster_fast_hadamard_transform(x: torch.Tensor, scale: float, out: torch.Tensor) -> torch.Tensor:
    _chk(x, "x", (_F16, _BF16)); _chk(out, "out", (x.dtype,))
    if x.dim() != 2:
        raise ValueError("faster_fast_hadamard_transform: x must be [batch, dim]")
    rows, n = x.shape
    if out.numel() != x.numel():
        raise ValueError("faster_fast_hadamard_transform: out must have x's shape")
    if rows == 0:
        return out
    lib = _lib.load()
    _lib.check(lib.qspec_fht(_ptr(x), _ptr(out), rows, n, float(scale), _dt(x), _stream()),
               "faster_fast_hadamard_transform")
    return out


def _check_container(out_q: Optional[torch.Tensor], rows: int, K: int, c8: bool, who: str) -> None:
    """out_q holds rows x K int4 values: K/2 bytes per row packed, K bytes per row in the int8 container."""
    if out_q is not None and out_q.numel() != rows * (K if c8 else K // 2):
        raise ValueError(f"{who}: out_q has {out_q.numel()} bytes, expected {rows * (K if c8 else K // 2)} "
                         f"({'int8 container' if c8 else 'packed int4'})")


def hadamard_heads(x: torch.Tensor, num_heads: int, head_dim: int, scale: float,
                   out: Optional[torch.Tensor] = None, out_q: Optional[torch.Tensor] = None,
                   scale_out: Optional[torch.Tensor] = None, clip_ratio: float = 1.0, c8: bool = False) -> None:
    """Fused o_proj rotation (+quant): quarot_llama.py:230-238 in one launch. c8: out_q is the int8 container
    ([rows, H*D] int8, one int4 value per byte) instead of the packed format."""
    _chk(x, "x", (_F16,)); _chk(out, "out", (_F16,), True); _chk(out_q, "out_q", _I4, True)
    _chk(scale_out, "scale_out", (_F16,), True)
    rows = x.numel() // (num_heads * head_dim)
    lib = _lib.load()
    _check_container(out_q, rows, num_heads * head_dim, c8, "hadamard_heads")
    _lib.check((lib.qspec_hadamard_heads_c8 if c8 else lib.qspec_hadamard_heads)(_ptr(x), _ptr(out), _ptr(out_q), _ptr(scale_out), rows, num_heads,
                                        head_dim, float(scale), float(clip_ratio), _stream()),
               "hadamard_heads")


def hadamard_k28(x: Optional[torch.Tensor], n: int, scale: float, gate_up: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None, out_q: Optional[torch.Tensor] = None,
                 scale_out: Optional[torch.Tensor] = None, clip_ratio: float = 1.0, c8: bool = False) -> None:
    """Fused down_proj rotation had28 (x) H_n (+SiLU*up in front, +quant behind). c8: out_q is the int8 container."""
    _chk(x, "x", (_F16,), True); _chk(gate_up, "gate_up", (_F16,), True)
    _chk(out, "out", (_F16,), True); _chk(out_q, "out_q", _I4, True); _chk(scale_out, "scale_out", (_F16,), True)
    src = gate_up if gate_up is not None else x
    if src is None:
        raise ValueError("hadamard_k28: x or gate_up is required")
    width = 28 * n * (2 if gate_up is not None else 1)
    rows = src.numel() // width
    lib = _lib.load()
    _check_container(out_q, rows, 28 * n, c8, "hadamard_k28")
    _lib.check((lib.qspec_hadamard_k28_c8 if c8 else lib.qspec_hadamard_k28)(_ptr(x) if gate_up is None else None, _ptr(gate_up), _ptr(out), _ptr(out_q),
                                      _ptr(scale_out), rows, n, float(scale), float(clip_ratio), _stream()),
               "hadamard_k28")


def hadamard_k108(x: Optional[torch.Tensor], n: int, scale: float, gate_up: Optional[torch.Tensor] = None,
                  gate_first: bool = True, out: Optional[torch.Tensor] = None, out_q: Optional[torch.Tensor] = None,
                  scale_out: Optional[torch.Tensor] = None, clip_ratio: float = 1.0) -> None:
    """Qwen2.5-14B down_proj rotation had108 (x) H_128 (+SiLU*mul in front, +quant behind): hadamard_utils.matmul_hadU_cuda
    with K = 108 as Qwen2MLP.forward calls it (qwen2_quarot.py:119-127). gate_up: [gate ; up] (vLLM SiluAndMul) when
    gate_first, else [up ; gate]."""
    _chk(x, "x", (_F16,), True); _chk(gate_up, "gate_up", (_F16,), True)
    _chk(out, "out", (_F16,), True); _chk(out_q, "out_q", _I4, True); _chk(scale_out, "scale_out", (_F16,), True)
    src = gate_up if gate_up is not None else x
    if src is None:
        raise ValueError("hadamard_k108: x or gate_up is required")
    rows = src.numel() // (108 * n * (2 if gate_up is not None else 1))
    lib = _lib.load()
    _lib.check(lib.qspec_hadamard_k108(_ptr(x) if gate_up is None else None, _ptr(gate_up), 1 if gate_first else 0, _ptr(out),
                                       _ptr(out_q), _ptr(scale_out), rows, n, float(scale), float(clip_ratio), _stream()),
               "hadamard_k108")


def hadamard_heads40(x: torch.Tensor, num_heads: int, head_dim: int, scale: float, out: Optional[torch.Tensor] = None,
                     out_q: Optional[torch.Tensor] = None, scale_out: Optional[torch.Tensor] = None,
                     clip_ratio: float = 1.0) -> None:
    """Qwen2.5-14B o_proj rotation (Qwen2Attention.o_had_trans with o_K = 40, qwen2_quarot.py:269-277) (+quant)."""
    _chk(x, "x", (_F16,)); _chk(out, "out", (_F16,), True); _chk(out_q, "out_q", _I4, True)
    _chk(scale_out, "scale_out", (_F16,), True)
    rows = x.numel() // (num_heads * head_dim)
    lib = _lib.load()
    _lib.check(lib.qspec_hadamard_heads40(_ptr(x), _ptr(out), _ptr(out_q), _ptr(scale_out), rows, num_heads, head_dim,
                                          float(scale), float(clip_ratio), _stream()), "hadamard_heads40")


# ---------------------------------------------------------------------------------------------
# GEMMs
# ---------------------------------------------------------------------------------------------

def rowwise_scaled_linear_cutlass_s4s4_unified(input: torch.Tensor, input_scale: torch.Tensor,
                                               weight: torch.Tensor, weight_scale: torch.Tensor,
                                               bias: Optional[torch.Tensor], result: torch.Tensor) -> torch.Tensor:
    """W4A4: result = T(((acc * input_scale[m]) * weight_scale[n]) + bias[n]); exact int32 acc."""
    _chk(input, "input", _I4); _chk(weight, "weight", _I4)
    _chk(result, "result", (_F16, _BF16))
    _chk(input_scale, "input_scale", (result.dtype,)); _chk(weight_scale, "weight_scale", (result.dtype,))
    _chk(bias, "bias", (result.dtype,), True)
    if weight.dim() != 2:
        raise ValueError("expected wq argument to be 2D tensor")
    N, K2 = weight.shape
    if input.shape[-1] != K2:
        raise ValueError(f"expected xq argument to have {K2} columns, but got {input.shape[-1]}")
    M = input.numel() // K2 if K2 else 0
    if input_scale.numel() != M or weight_scale.numel() != N or result.numel() != M * N:
        raise ValueError("rowwise_scaled_linear_cutlass_s4s4_unified: scale/result sizes do not match")
    if bias is not None and bias.numel() != N:
        raise ValueError(f"expected bias argument to have {N} elements")
    if M == 0:
        return result
    lib = _lib.load()
    K = 2 * K2
    need = lib.qspec_gemm_w4a4_workspace_bytes(M, N, K)
    ws = _workspace("w4a4", need, input.device)
    _lib.check(lib.qspec_gemm_w4a4(_ptr(input), _ptr(input_scale), _ptr(weight), _ptr(weight_scale), _ptr(bias),
                                   _ptr(result), M, N, K, _dt(result), _ptr(ws), ws.numel(), _stream()),
               "rowwise_scaled_linear_cutlass_s4s4_unified")
    return result


def gemm_w4a4_acc_i32(input: torch.Tensor, weight: torch.Tensor, acc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Parity/debug entry: raw int32 accumulators of the tcgen05 main loop."""
    _chk(input, "input", _I4); _chk(weight, "weight", _I4)
    N, K2 = weight.shape
    M = input.numel() // K2
    if acc is None:
        acc = torch.empty(M, N, dtype=torch.int32, device=input.device)
    _chk(acc, "acc", (torch.int32,))
    lib = _lib.load()
    need = lib.qspec_gemm_w4a4_workspace_bytes(M, N, 2 * K2)
    ws = _workspace("w4a4", need, input.device)
    _lib.check(lib.qspec_gemm_w4a4_acc_i32(_ptr(input), _ptr(weight), _ptr(acc), M, N, 2 * K2, _ptr(ws),
                                           ws.numel(), _stream()), "gemm_w4a4_acc_i32")
    return acc


def gemm_w4a16(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
               bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """W4A16: out = x @ (int4(weight) * weight_scale[:, None]).T (+ bias); weight is the SAME
    two's-complement packed tensor the W4A4 path reads (no `^ 0x88` copy)."""
    _chk(x, "x", (_F16, _BF16)); _chk(weight, "weight", _I4); _chk(out, "out", (x.dtype,))
    _chk(weight_scale, "weight_scale", (x.dtype,)); _chk(bias, "bias", (x.dtype,), True)
    N, K2 = weight.shape
    K = 2 * K2
    if x.shape[-1] != K:
        raise ValueError(f"gemm_w4a16: x has {x.shape[-1]} columns, weight expects {K}")
    M = x.numel() // K
    if weight_scale.numel() != N or out.numel() != M * N:
        raise ValueError("gemm_w4a16: scale/out sizes do not match")
    if M == 0:
        return out
    lib = _lib.load()
    need = lib.qspec_gemm_w4a16_workspace_bytes(M, N, K)
    ws = _workspace("w4a16", need, x.device)
    _lib.check(lib.qspec_gemm_w4a16(_ptr(x), _ptr(weight), _ptr(weight_scale), _ptr(bias), _ptr(out), M, N, K,
                                    _dt(x), _ptr(ws), ws.numel(), _stream()), "gemm_w4a16")
    return out


# ---------------------------------------------------------------------------------------------
# W4A8 mode (kwargs["w4a8"], off by default in the reference)
#   layernorm_ops.rms_norm_general_fuse_sum_i8   third-party/kernels/csrc/layernorm.cpp:44-50
#   quarot._CUDA.fuse_sym_quant_i8               third-party/QuaRot/quarot/kernels/bindings.cpp:148-164
#   rowwise_scaled_linear_cutlass_s8s4           torchao, as called at quarot_nn/linear.py:98
# ---------------------------------------------------------------------------------------------

def rms_norm_general_fuse_sum_i8(out_q: torch.Tensor, x: torch.Tensor, input_sum: Optional[torch.Tensor],
                                 scaling: torch.Tensor, eps: float, use_per_token_quant: bool = True) -> None:
    if not use_per_token_quant:
        raise NotImplementedError("only the per-token branch is on the QSpec path (normalization.py:96-103)")
    _chk(x, "input", (_F16,)); _chk(out_q, "out", (torch.int8,)); _chk(scaling, "scaling", (_F16,))
    _chk(input_sum, "input_sum", (_F16,), allow_none=True)
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if out_q.numel() != rows * K or scaling.numel() < rows:
        raise ValueError("rms_norm_general_fuse_sum_i8: output shapes do not match the input")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_norm_quant_i8(_ptr(x), _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K,
                                       float(eps), _stream()), "rms_norm_general_fuse_sum_i8")


def fuse_sym_quant_i8(x: torch.Tensor, scale: torch.Tensor, q: torch.Tensor, input_clip_ratio: float = 1.0) -> None:
    _chk(x, "x", (_F16,)); _chk(scale, "scale", (_F16,)); _chk(q, "q", (torch.int8,))
    if x.dim() != 2:
        raise ValueError("fuse_sym_quant_i8: x must be 2-D")
    rows, K = x.shape
    if q.numel() != rows * K or scale.numel() < rows:
        raise ValueError("fuse_sym_quant_i8: output shapes do not match the input")
    if rows == 0:
        return
    lib = _lib.load()
    _lib.check(lib.qspec_sym_quant_i8(_ptr(x), _ptr(scale), _ptr(q), rows, K, float(input_clip_ratio),
                                      _stream()), "fuse_sym_quant_i8")


def rowwise_scaled_linear_cutlass_s8s4(input: torch.Tensor, input_scale: torch.Tensor, weight: torch.Tensor,
                                       weight_scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                                       result: Optional[torch.Tensor] = None) -> torch.Tensor:
    """W4A8: result = T(((acc * input_scale[m]) * weight_scale[n]) + bias[n]); input int8 [M, K], weight packed int4 [N, K/2]."""
    _chk(input, "input", (torch.int8,)); _chk(weight, "weight", _I4)
    _chk(input_scale, "input_scale", (_F16, _BF16)); _chk(weight_scale, "weight_scale", (input_scale.dtype,))
    _chk(bias, "bias", (input_scale.dtype,), True)
    if weight.dim() != 2:
        raise ValueError("expected wq argument to be 2D tensor")
    N, K2 = weight.shape
    K = 2 * K2
    if input.shape[-1] != K:
        raise ValueError(f"expected xq argument to have {K} columns, but got {input.shape[-1]}")
    M = input.numel() // K if K else 0
    if result is None:
        result = torch.empty(*input.shape[:-1], N, dtype=input_scale.dtype, device=input.device)
    _chk(result, "result", (input_scale.dtype,))
    if input_scale.numel() != M or weight_scale.numel() != N or result.numel() != M * N:
        raise ValueError("rowwise_scaled_linear_cutlass_s8s4: scale/result sizes do not match")
    if bias is not None and bias.numel() != N:
        raise ValueError(f"expected bias argument to have {N} elements")
    if M == 0:
        return result
    lib = _lib.load()
    need = lib.qspec_gemm_w4a8_workspace_bytes(M, N, K)
    ws = _workspace("w4a4", need, input.device)
    _lib.check(lib.qspec_gemm_w4a8(_ptr(input), _ptr(input_scale), _ptr(weight), _ptr(weight_scale), _ptr(bias),
                                   _ptr(result), M, N, K, _dt(result), _ptr(ws), ws.numel(), _stream()),
               "rowwise_scaled_linear_cutlass_s8s4")
    return result


def gemm_w4a8_acc_i32(input: torch.Tensor, weight: torch.Tensor, acc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Parity/debug entry: raw int32 accumulators sum_k a_i8[m,k] * w_i4[n,k]."""
    _chk(input, "input", (torch.int8,)); _chk(weight, "weight", _I4)
    N, K2 = weight.shape
    K = 2 * K2
    M = input.numel() // K
    if acc is None:
        acc = torch.empty(M, N, dtype=torch.int32, device=input.device)
    _chk(acc, "acc", (torch.int32,))
    lib = _lib.load()
    need = lib.qspec_gemm_w4a8_workspace_bytes(M, N, K)
    ws = _workspace("w4a4", need, input.device)
    _lib.check(lib.qspec_gemm_w4a8_acc_i32(_ptr(input), _ptr(weight), _ptr(acc), M, N, K, _ptr(ws), ws.numel(),
                                           _stream()), "gemm_w4a8_acc_i32")
    return acc


# ---------------------------------------------------------------------------------------------
# deferred reduction: GEMM leaves per-k-slice partial accumulators, the consuming norm sums them
# ---------------------------------------------------------------------------------------------

class SplitPartials:
    """Raw partial accumulators of one o_proj / down_proj call (qspec_gemm_w4a4_split / qspec_gemm_w4a16_split) plus
    what the consumer needs to finish the GEMM epilogue: [split][M][N] 32-bit words, activation / weight scales, bias."""
    __slots__ = ("buf", "split", "w4a16", "sA", "sW", "bias", "M", "N")

    def __init__(self, buf, split, w4a16, sA, sW, bias, M, N):
        self.buf, self.split, self.w4a16, self.sA, self.sW, self.bias, self.M, self.N = buf, split, w4a16, sA, sW, bias, M, N


def gemm_split_factor(w4a16, M: int, N: int, K: int) -> int:
    """Slices per output element the deferred-reduction GEMM leaves for this shape; 0 = use the plain GEMM.
    w4a16: False / 0 = W4A4 (packed activations), True / 1 = W4A16, 2 = W4A4 from int8-container activations."""
    return int(_lib.load().qspec_gemm_split_factor(int(w4a16), M, N, K))


def gemm_w4a4_c8_split(input: torch.Tensor, input_scale: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                       bias: Optional[torch.Tensor], partials: torch.Tensor) -> SplitPartials:
    """gemm_w4a4_split for int8-container activations ([M, K] int8, one int4 value per byte)."""
    _chk(input, "input", _I4); _chk(weight, "weight", _I4); _chk(partials, "partials", (torch.int32, torch.float32))
    N, K2 = weight.shape
    K = 2 * K2
    M = input.numel() // K
    lib = _lib.load()
    split = lib.qspec_gemm_split_factor(2, M, N, K)
    if split < 1 or partials.numel() < split * M * N:
        raise ValueError(f"gemm_w4a4_c8_split: unsupported shape or partial buffer too small (split={split})")
    ws = _workspace("w4a8", lib.qspec_gemm_w4a8_workspace_bytes(M, N, K), input.device)
    _lib.check(lib.qspec_gemm_w4a8_split(_ptr(input), _ptr(weight), _ptr(partials), partials.numel() * 4, M, N, K, _ptr(ws),
                                         ws.numel(), _stream()), "gemm_w4a4_c8_split")
    return SplitPartials(partials, split, 2, input_scale, weight_scale, bias, M, N)


def gemm_w4a4_split(input: torch.Tensor, input_scale: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                    bias: Optional[torch.Tensor], partials: torch.Tensor) -> SplitPartials:
    """rowwise_scaled_linear_cutlass_s4s4_unified without its cross-CTA reduction and epilogue: raw int32 partial sums
    per k-slice go to `partials` (int32, >= split*M*N elements); the scales travel with the result to the consumer."""
    _chk(input, "input", _I4); _chk(weight, "weight", _I4); _chk(partials, "partials", (torch.int32, torch.float32))
    N, K2 = weight.shape
    M = input.numel() // K2
    K = 2 * K2
    lib = _lib.load()
    split = lib.qspec_gemm_split_factor(0, M, N, K)
    if split < 1 or partials.numel() < split * M * N:
        raise ValueError(f"gemm_w4a4_split: unsupported shape or partial buffer too small (split={split})")
    ws = _workspace("w4a4", lib.qspec_gemm_w4a4_workspace_bytes(M, N, K), input.device)
    _lib.check(lib.qspec_gemm_w4a4_split(_ptr(input), _ptr(weight), _ptr(partials), partials.numel() * 4, M, N, K, _ptr(ws),
                                         ws.numel(), _stream()), "gemm_w4a4_split")
    return SplitPartials(partials, split, False, input_scale, weight_scale, bias, M, N)


def gemm_w4a16_split(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, bias: Optional[torch.Tensor],
                     partials: torch.Tensor) -> SplitPartials:
    _chk(x, "x", (_F16, _BF16)); _chk(weight, "weight", _I4); _chk(partials, "partials", (torch.int32, torch.float32))
    N, K2 = weight.shape
    K = 2 * K2
    M = x.numel() // K
    lib = _lib.load()
    split = lib.qspec_gemm_split_factor(1, M, N, K)
    if split < 1 or partials.numel() < split * M * N:
        raise ValueError(f"gemm_w4a16_split: unsupported shape or partial buffer too small (split={split})")
    ws = _workspace("w4a16", lib.qspec_gemm_w4a16_workspace_bytes(M, N, K), x.device)
    _lib.check(lib.qspec_gemm_w4a16_split(_ptr(x), _ptr(weight), _ptr(partials), partials.numel() * 4, M, N, K, _dt(x),
                                          _ptr(ws), ws.numel(), _stream()), "gemm_w4a16_split")
    return SplitPartials(partials, split, True, None, weight_scale, bias, M, N)


def split_add_rms_norm_fuse_sum_i4(out_q: torch.Tensor, x: torch.Tensor, sp: SplitPartials, input_sum: torch.Tensor,
                                   scaling: torch.Tensor, eps: float, c8: bool = False) -> None:
    """x += epilogue(sum of sp's slices) (in place), then rms_norm_general_fuse_sum_i4: one launch; bit-identical to the
    plain GEMM followed by add_rms_norm_fuse_sum_i4."""
    _chk(x, "input", (_F16,)); _chk(out_q, "out", _I4); _chk(scaling, "scaling", (_F16,)); _chk(input_sum, "input_sum", (_F16,))
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if rows != sp.M or K != sp.N:
        raise ValueError("split_add_rms_norm_fuse_sum_i4: input does not match the partial sums")
    lib = _lib.load()
    _check_container(out_q, rows, K, c8, "split_add_rms_norm_fuse_sum_i4")
    _lib.check((lib.qspec_split_add_norm_quant_i4_c8 if c8 else lib.qspec_split_add_norm_quant_i4)(_ptr(x), _ptr(sp.buf), sp.split, int(sp.w4a16), _ptr(sp.sA), _ptr(sp.sW),
                                                 _ptr(sp.bias), _ptr(out_q), _ptr(scaling), _ptr(input_sum), rows, K, float(eps),
                                                 _stream()), "split_add_rms_norm_fuse_sum_i4")


def split_add_rms_norm_fuse_sum_fp16(out: torch.Tensor, x: torch.Tensor, sp: SplitPartials, eps: float) -> None:
    _chk(x, "input", (_F16, _BF16)); _chk(out, "out", (x.dtype,))
    K = x.shape[-1]
    rows = x.numel() // K if K else 0
    if rows != sp.M or K != sp.N or out.numel() != x.numel():
        raise ValueError("split_add_rms_norm_fuse_sum_fp16: input does not match the partial sums")
    lib = _lib.load()
    _lib.check(lib.qspec_split_add_norm_f16(_ptr(x), _ptr(sp.buf), sp.split, int(sp.w4a16), _ptr(sp.sA), _ptr(sp.sW),
                                            _ptr(sp.bias), _ptr(out), rows, K, float(eps), _dt(x), _stream()),
               "split_add_rms_norm_fuse_sum_fp16")


# ---------------------------------------------------------------------------------------------
# neighbours
# ---------------------------------------------------------------------------------------------

def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _chk(a, "a", (_F16, _BF16)); _chk(b, "b", (a.dtype,)); _chk(out, "out", (a.dtype,))
    lib = _lib.load()
    _lib.check(lib.qspec_add(_ptr(a), _ptr(b), _ptr(out), a.numel(), _dt(a), _stream()), "add")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """gate_up = [up ; gate] (quarot_llama.py:279); out = silu(gate) * up."""
    _chk(gate_up, "gate_up", (_F16, _BF16)); _chk(out, "out", (gate_up.dtype,))
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * inter)
    lib = _lib.load()
    _lib.check(lib.qspec_silu_mul(_ptr(gate_up), _ptr(out), rows, inter, _dt(gate_up), _stream()), "silu_mul")
    return out


def rope_kvcache(qkv: torch.Tensor, cos_sin_cache: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                 cache_k: torch.Tensor, cache_v: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """In-place neox RoPE on q,k of qkv [T, (Hq+2Hkv)*D]; appends k,v to cache [B, S, Hkv, D]."""
    _chk(qkv, "qkv", (_F16,)); _chk(cos_sin_cache, "cos_sin_cache", (_F16,))
    _chk(positions, "positions", (torch.int32,)); _chk(seq_ids, "seq_ids", (torch.int32,))
    _chk(cache_k, "cache_k", (_F16,)); _chk(cache_v, "cache_v", (_F16,))
    T = positions.numel()
    if cos_sin_cache.shape[0] < cache_k.shape[1]:
        raise ValueError(f"rope_kvcache: rotary table has {cos_sin_cache.shape[0]} positions, the KV cache {cache_k.shape[1]}")
    lib = _lib.load()
    _lib.check(lib.qspec_rope_kvcache(_ptr(qkv), _ptr(cos_sin_cache), _ptr(positions), _ptr(seq_ids), _ptr(cache_k),
                                      _ptr(cache_v), T, num_heads, num_kv_heads, head_dim, cache_k.shape[1], _stream()),
               "rope_kvcache")


def rope_qkhad_kvcache(qkv: torch.Tensor, cos_sin_cache: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
                       cache_k: torch.Tensor, cache_v: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                       had_scale: float) -> None:
    """rope_kvcache + the per-head Hadamard of q and k after the rotary embedding (Qwen2Attention.qk_had_trans,
    qwen2_quarot.py:279-288)."""
    _chk(qkv, "qkv", (_F16,)); _chk(cos_sin_cache, "cos_sin_cache", (_F16,))
    _chk(positions, "positions", (torch.int32,)); _chk(seq_ids, "seq_ids", (torch.int32,))
    _chk(cache_k, "cache_k", (_F16,)); _chk(cache_v, "cache_v", (_F16,))
    if cos_sin_cache.shape[0] < cache_k.shape[1]:
        raise ValueError(f"rope_qkhad_kvcache: rotary table has {cos_sin_cache.shape[0]} positions, the KV cache {cache_k.shape[1]}")
    lib = _lib.load()
    _lib.check(lib.qspec_rope_qkhad_kvcache(_ptr(qkv), _ptr(cos_sin_cache), _ptr(positions), _ptr(seq_ids), _ptr(cache_k),
                                            _ptr(cache_v), positions.numel(), num_heads, num_kv_heads, head_dim,
                                            cache_k.shape[1], float(had_scale), _stream()), "rope_qkhad_kvcache")


def decode_attention(qkv: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, positions: torch.Tensor,
                     seq_ids: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                     sm_scale: float) -> torch.Tensor:
    _chk(qkv, "qkv", (_F16,)); _chk(out, "out", (_F16,))
    T = positions.numel()
    lib = _lib.load()
    _lib.check(lib.qspec_decode_attention(_ptr(qkv), _ptr(cache_k), _ptr(cache_v), _ptr(positions), _ptr(seq_ids),
                                          _ptr(out), T, num_heads, num_kv_heads, head_dim, cache_k.shape[1],
                                          float(sm_scale), _stream()), "decode_attention")
    return out


def seq_attention_supported(T: int, num_heads: int, num_kv_heads: int, head_dim: int, cache_len: int) -> bool:
    return bool(_lib.load().qspec_seq_attention_supported(T, num_heads, num_kv_heads, head_dim, cache_len))


def seq_attention(qkv: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, positions: torch.Tensor,
                  seq_ids: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                  sm_scale: float) -> torch.Tensor:
    """decode_attention for passes with many sequences / several tokens per sequence: keys and values of a (sequence, kv head)
    are read once for all its tokens and query heads."""
    _chk(qkv, "qkv", (_F16,)); _chk(out, "out", (_F16,)); _chk(cache_k, "cache_k", (_F16,)); _chk(cache_v, "cache_v", (_F16,))
    _chk(positions, "positions", (torch.int32,)); _chk(seq_ids, "seq_ids", (torch.int32,))
    lib = _lib.load()
    _lib.check(lib.qspec_seq_attention(_ptr(qkv), _ptr(cache_k), _ptr(cache_v), _ptr(positions), _ptr(seq_ids), _ptr(out),
                                       positions.numel(), cache_k.shape[0], num_heads, num_kv_heads, head_dim, cache_k.shape[1],
                                       float(sm_scale), _stream()), "seq_attention")
    return out


def attn_block_supported(T: int, num_heads: int, num_kv_heads: int, head_dim: int, cache_len: int) -> bool:
    return bool(_lib.load().qspec_attn_block_supported(T, num_heads, num_kv_heads, head_dim, cache_len))


def attn_block(qkv: torch.Tensor, cos_sin_cache: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor,
               cache_k: torch.Tensor, cache_v: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
               sm_scale: float, had_scale: float, out: Optional[torch.Tensor] = None, out_q: Optional[torch.Tensor] = None,
               scale_out: Optional[torch.Tensor] = None, attn_out: Optional[torch.Tensor] = None,
               input_clip_ratio: float = 1.0) -> None:
    """rope_kvcache + decode_attention + hadamard_heads (+ quantiser) in one launch (quarot_llama.py:207-238); qkv is
    left untouched. Bit-identical to the chain of the three calls."""
    _chk(qkv, "qkv", (_F16,)); _chk(out, "out", (_F16,), allow_none=True); _chk(out_q, "out_q", _I4, allow_none=True)
    _chk(scale_out, "scale_out", (_F16,), allow_none=True); _chk(attn_out, "attn_out", (_F16,), allow_none=True)
    if positions.dtype != torch.int32 or seq_ids.dtype != torch.int32:
        raise ValueError("attn_block: positions and seq_ids must be int32")
    T = positions.numel()
    if cos_sin_cache.shape[0] < cache_k.shape[1]:
        raise ValueError(f"attn_block: rotary table has {cos_sin_cache.shape[0]} positions, the KV cache {cache_k.shape[1]}")
    lib = _lib.load()
    _lib.check(lib.qspec_attn_block(_ptr(qkv), _ptr(cos_sin_cache), _ptr(positions), _ptr(seq_ids), _ptr(cache_k),
                                    _ptr(cache_v), _ptr(attn_out), _ptr(out), _ptr(out_q), _ptr(scale_out), T, num_heads,
                                    num_kv_heads, head_dim, cache_k.shape[1], float(sm_scale), float(had_scale),
                                    float(input_clip_ratio), _stream()), "attn_block")


def argmax_rows(logits: torch.Tensor, out_val: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row of the logits [rows, V] (float16; bfloat16 / float32 through the sequence-mixer library): int64 indices (lowest index among equal maxima, like
    torch.argmax on distinct values); out_val (f32 [rows], optional) receives the maxima."""
    if not logits.is_cuda or logits.dtype not in (_F16, _BF16, torch.float32):
        raise ValueError("argmax_rows: logits must be a float16 / bfloat16 / float32 CUDA tensor (qspec_b200 has no CPU path)")
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("argmax_rows: logits must be [rows, V] with unit column stride")
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    if rows == 0:
        return out
    if logits.dtype != _F16:                       # bfloat16 / float32 logits: the sequence-mixer library's kernel
        if out_val is not None:
            raise ValueError("argmax_rows: out_val is only available for float16 logits")
        seq = _lib.load_seq()
        _lib.check(seq.qspec_seq_argmax_rows(_ptr(logits), rows, V, logits.stride(0), _ptr(out),
                                             _lib.DTYPE_BF16 if logits.dtype == _BF16 else _lib.DTYPE_F32, _stream()),
                   "argmax_rows", seq)
        return out
    lib = _lib.load()
    ws = _workspace("argmax", lib.qspec_argmax_rows_workspace_bytes(rows), logits.device)
    _lib.check(lib.qspec_argmax_rows(_ptr(logits), rows, V, logits.stride(0), _ptr(out), _ptr(out_val), _ptr(ws), ws.numel(),
                                     _stream()), "argmax_rows")
    return out


def tp_argmax_combine(local_max: torch.Tensor, local_idx: torch.Tensor, index_offset: int, peers,
                      out: Optional[torch.Tensor] = None, phases: int = 3) -> torch.Tensor:
    """Greedy token over a vocab-sharded lm_head through peer memory (no collective call): every rank pushes its
    (max logit, global index) pairs into every peer's table and takes the best of its own in rank order -- what the
    all-gather of the sharded logits (layers/logits_processor.py:84-107) followed by an arg max gives. int64 [rows],
    identical on every rank. phases 1 / 2: the two halves as separate launches (tests/tp_emulation.py)."""
    if not local_max.is_cuda or local_max.dtype != torch.float32 or local_idx.dtype != torch.int64:
        raise ValueError("tp_argmax_combine: local_max must be float32 and local_idx int64 CUDA tensors")
    rows = local_max.numel()
    if rows == 0 or rows != local_idx.numel() or rows > peers.max_tokens:
        raise ValueError("tp_argmax_combine: rows must be 1..peers.max_tokens on every rank")
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=local_max.device)
    lib = _lib.load()
    _lib.check(lib.qspec_tp_argmax_combine(_ptr(local_max), _ptr(local_idx), int(index_offset), rows, peers._amax_slots,
                                           peers._amax_flags, _ptr(peers.amax_state), peers.max_tokens, peers.world,
                                           peers.rank, phases, _ptr(out), _stream()), "tp_argmax_combine")
    return out


def launch_count() -> int:
    return int(_lib.load().qspec_launch_count())


# ---------------------------------------------------------------------------------------------
# Sequence-mixer kernels (include/qspec_b200_seq.h, libqspec_b200_seq.so): bfloat16 / float32
# activations and weights, float32 residual stream. No counterpart in the reference.
# ---------------------------------------------------------------------------------------------
_F32 = torch.float32
_SEQ_ACT = (_BF16, _F32)


def _sdt(t: torch.Tensor) -> int:
    if t.dtype == _BF16:
        return _lib.DTYPE_BF16
    if t.dtype == _F32:
        return _lib.DTYPE_F32
    raise ValueError(f"expected bfloat16 or float32 tensor, got {t.dtype}")


def _seq(status: int, what: str) -> None:
    _lib.check(status, what, _lib.load_seq())


def seq_launch_count() -> int:
    return int(_lib.load_seq().qspec_launch_count())


def seq_embed(table: torch.Tensor, ids: torch.Tensor, x: torch.Tensor) -> None:
    """x[i] = float32(table[ids[i]]); ids int32 [ntok], x float32 [ntok, W]."""
    _chk(table, "table", _SEQ_ACT); _chk(ids, "ids", (torch.int32,)); _chk(x, "x", (_F32,))
    V, W = table.shape
    if x.shape != (ids.numel(), W):
        raise ValueError("seq_embed: x must be [ntok, W]")
    _seq(_lib.load_seq().qspec_seq_embed(_ptr(table), _ptr(ids), _ptr(x), ids.numel(), W, V, _sdt(table), _stream()), "seq_embed")


def seq_norm_conv(x_in: torch.Tensor, meta: torch.Tensor, eps: float, *, out: Optional[torch.Tensor] = None,
                  pre_w: Optional[torch.Tensor] = None, conv_w: Optional[torch.Tensor] = None,
                  tail: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None, y_w: Optional[torch.Tensor] = None,
                  post_w: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None,
                  scratch: Optional[torch.Tensor] = None) -> None:
    """Closes a sublayer (x_out = x_in + zero-centred norm of y, with weight post_w) and opens the next
    (out = h + causal short convolution of h, h = zero-centred norm of the new residual with weight pre_w) in one launch.
    y: [ntok, W] or [ntok, parts, W] (parts summed, each times y_w [ntok, parts] if given). tail: float32
    [2, slots, taps-1, W], read at meta's phase, written at the other. out None: only the residual sum.
    scratch: float32 with room for [ntok, W]; with it, long prompts (256 tokens or more) run as two launches over
    independent rows instead of one that walks the rows of a run in turn; same results."""
    _chk(x_in, "x_in", (_F32,)); _chk(meta, "meta", (torch.int32,))
    ntok, W = x_in.shape
    if meta.shape != (5, ntok):
        raise ValueError("seq_norm_conv: meta must be int32 [5, ntok]")
    for t, n in ((pre_w, "pre_w"), (conv_w, "conv_w"), (tail, "tail"), (y_w, "y_w"), (post_w, "post_w"), (x_out, "x_out")):
        _chk(t, n, (_F32,), allow_none=True)
    _chk(out, "out", _SEQ_ACT, allow_none=True); _chk(y, "y", _SEQ_ACT, allow_none=True)
    parts, pstride, tstride = 1, 0, W
    if y is not None:
        if y.dim() == 3:
            parts, pstride, tstride = y.shape[1], W, y.shape[1] * W
        if y.shape[0] != ntok or y.shape[-1] != W or (y_w is not None and y_w.shape != (ntok, parts)):
            raise ValueError("seq_norm_conv: y / y_w shapes do not match x")
    taps = conv_w.shape[1] if conv_w is not None else 1
    slots = 0
    if conv_w is not None and taps > 1:
        if tail is None or tail.dim() != 4 or tail.shape[0] != 2 or tail.shape[2] != taps - 1 or tail.shape[3] != W:
            raise ValueError("seq_norm_conv: tail must be float32 [2, slots, taps-1, W]")
        slots = tail.shape[1]
    act = out if out is not None else y
    if scratch is not None:
        _chk(scratch, "scratch", (_F32,))
        if scratch.numel() < ntok * W:
            raise ValueError("seq_norm_conv: scratch is smaller than [ntok, W]")
    _seq(_lib.load_seq().qspec_seq_norm_conv(_ptr(x_in), _ptr(x_out), _ptr(y), parts, pstride, tstride, _ptr(y_w), _ptr(post_w),
                                             _ptr(pre_w), _ptr(conv_w), taps, _ptr(tail), slots, _ptr(out), _ptr(meta), ntok, W,
                                             float(eps), _ptr(scratch), _sdt(act), _stream()), "seq_norm_conv")


def seq_qk_norm(qkv: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor, H: int, G: int, D: int, eps: float) -> None:
    """In place: every query and key head of the fused projection rows [q | k | v] <- head / rms(head) * w."""
    _chk(qkv, "qkv", _SEQ_ACT); _chk(q_w, "q_w", (_F32,)); _chk(k_w, "k_w", (_F32,))
    _seq(_lib.load_seq().qspec_seq_qk_norm(_ptr(qkv), qkv.shape[1], _ptr(q_w), _ptr(k_w), qkv.shape[0], H, G, D, float(eps),
                                           _sdt(qkv), _stream()), "seq_qk_norm")


def seq_chunk_attention_tiles_supported(qkv: torch.Tensor, H: int, G: int, D: int, DV: int) -> bool:
    """The tensor-core tile form takes bfloat16 rows that start on 16-byte boundaries and head sizes of 64 or 128."""
    return bool(qkv.dtype == _BF16 and qkv.shape[1] % 8 == 0
                and _lib.load_seq().qspec_seq_chunk_attention_mma_supported(H, G, D, DV))


def seq_chunk_attention(qkv: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, bias: torch.Tensor, out: torch.Tensor,
                        meta: torch.Tensor, H: int, G: int, D: int, DV: int, size: int, scale: float, softcap: float,
                        tiles: bool = False, max_keys: int = 0) -> None:
    """Chunk-local sigmoid attention of a token batch; cache_k [slots, size, G, D], cache_v [slots, size, G, DV].
    tiles=True: the tensor-core form over 64-query tiles (prompt-shaped batches; `seq_chunk_attention_tiles_supported`).
    max_keys: the most keys a token of the batch can see (largest position + 1; 0: unknown) -- the token form spreads the
    keys of a token over a cluster of CTAs when the batch has few tokens with many keys each."""
    for t, n in ((qkv, "qkv"), (cache_k, "cache_k"), (cache_v, "cache_v"), (out, "out")):
        _chk(t, n, (qkv.dtype,))
    _chk(qkv, "qkv", _SEQ_ACT); _chk(bias, "bias", (_F32,)); _chk(meta, "meta", (torch.int32,))
    ntok = qkv.shape[0]
    if out.shape != (ntok, H * DV) or meta.shape != (5, ntok) or cache_k.shape[1:] != (size, G, D) or cache_v.shape[1:] != (size, G, DV):
        raise ValueError("seq_chunk_attention: shapes do not match")
    if tiles:
        _seq(_lib.load_seq().qspec_seq_chunk_attention_mma(_ptr(qkv), qkv.shape[1], _ptr(cache_k), _ptr(cache_v), _ptr(bias), _ptr(out),
                                                           _ptr(meta), ntok, H, G, D, DV, size, float(scale), float(softcap or 0.0),
                                                           _stream()), "seq_chunk_attention (tiles)")
        return
    _seq(_lib.load_seq().qspec_seq_chunk_attention(_ptr(qkv), qkv.shape[1], _ptr(cache_k), _ptr(cache_v), _ptr(bias), _ptr(out),
                                                   _ptr(meta), ntok, H, G, D, DV, size, float(scale), float(softcap or 0.0),
                                                   int(max_keys), _sdt(qkv), _stream()), "seq_chunk_attention")


def seq_cache_append(qkv: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, meta: torch.Tensor, H: int, G: int, D: int,
                     DV: int, size: int) -> None:
    """Writes the step's keys / values of every segment's last chunk into the cache (after the step's attention)."""
    for t, n in ((qkv, "qkv"), (cache_k, "cache_k"), (cache_v, "cache_v")):
        _chk(t, n, (qkv.dtype,))
    _seq(_lib.load_seq().qspec_seq_cache_append(_ptr(qkv), qkv.shape[1], _ptr(cache_k), _ptr(cache_v), _ptr(meta), qkv.shape[0], H, G,
                                                D, DV, size, _sdt(qkv), _stream()), "seq_cache_append")


def seq_relu2(a: torch.Tensor) -> None:
    _chk(a, "a", _SEQ_ACT)
    _seq(_lib.load_seq().qspec_seq_relu2(_ptr(a), a.numel(), _sdt(a), _stream()), "seq_relu2")


def moe_route(h: torch.Tensor, router_w: torch.Tensor, correction: torch.Tensor, idx: torch.Tensor, weight: torch.Tensor) -> None:
    """Softmax router with a choice correction: idx int32 [ntok, top], weight float32 [ntok, top] (plain scores)."""
    _chk(h, "h", _SEQ_ACT); _chk(router_w, "router_w", (_F32,)); _chk(correction, "correction", (_F32,))
    _chk(idx, "idx", (torch.int32,)); _chk(weight, "weight", (_F32,))
    ntok, W = h.shape
    R, top = router_w.shape[0], idx.shape[1]
    if router_w.shape[1] != W or correction.numel() != R or idx.shape != (ntok, top) or weight.shape != (ntok, top):
        raise ValueError("moe_route: shapes do not match")
    _seq(_lib.load_seq().qspec_moe_route(_ptr(h), _ptr(router_w), _ptr(correction), _ptr(idx), _ptr(weight), ntok, W, R, top, _sdt(h),
                                         _stream()), "moe_route")


EXPERT_ACTS = {"gated": 0, "relu2": 1, "silu": 2}       # QSPEC_EXPERT_ACT_* of include/qspec_b200_seq.h


def moe_expert_tokens(h: torch.Tensor, gate_up: Optional[torch.Tensor], down: Optional[torch.Tensor], idx: torch.Tensor,
                      out: torch.Tensor, E: int, F: int, limit: float, act: str = "gated") -> None:
    """Expert outputs per (token, choice), unweighted: out [ntok, top, W]; choices >= E copy h (identity experts).
    act "gated": gate_up [E, 2F, W], the clamped gated activation; "silu": the same rows with silu(gate) * up (limit unused);
    "relu2": gate_up is the up matrix [E, F, W] alone and the activation is the squared ReLU (limit unused)."""
    _chk(h, "h", _SEQ_ACT); _chk(out, "out", (h.dtype,)); _chk(idx, "idx", (torch.int32,))
    _chk(gate_up, "gate_up", (h.dtype,), allow_none=E == 0); _chk(down, "down", (h.dtype,), allow_none=E == 0)
    ntok, W = h.shape
    top = idx.shape[1]
    rows = F if act == "relu2" else 2 * F
    if out.shape != (ntok, top, W) or (E and (gate_up.shape != (E, rows, W) or down.shape != (E, W, F))):
        raise ValueError("moe_expert_tokens: shapes do not match")
    _seq(_lib.load_seq().qspec_moe_expert_tokens_act(_ptr(h), _ptr(gate_up), _ptr(down), _ptr(idx), _ptr(out), ntok, W, F, E, top,
                                                     float(limit), EXPERT_ACTS[act], _sdt(h), _stream()), "moe_expert_tokens")


def moe_grouped_status(device="cuda") -> int:
    """0, or 1 once a CTA of the grouped expert products gave up a bounded wait on its pipeline (its rows were not
    written). Reads the first word of the workspace: synchronises the device."""
    device = torch.device(device)
    ws = _workspaces.get(("moe_grouped", device.index if device.index is not None else torch.cuda.current_device()))
    return 0 if ws is None else int(ws[:4].view(torch.int32).item())


def moe_expert_grouped_supported(h: torch.Tensor, F: int) -> bool:
    return bool(h.dtype == _BF16 and _lib.load_seq().qspec_moe_expert_grouped_supported(h.shape[1], F))


def moe_expert_grouped(h: torch.Tensor, gate_up: Optional[torch.Tensor], down: Optional[torch.Tensor], idx: torch.Tensor,
                       out: torch.Tensor, E: int, F: int, limit: float, act: str = "gated") -> None:
    """`moe_expert_tokens` for many tokens (bfloat16): the (token, choice) pairs are sorted by expert and every expert's rows
    go through tensor-core tiles; same outputs up to the summation order."""
    _chk(h, "h", (_BF16,)); _chk(out, "out", (_BF16,)); _chk(idx, "idx", (torch.int32,))
    _chk(gate_up, "gate_up", (_BF16,), allow_none=E == 0); _chk(down, "down", (_BF16,), allow_none=E == 0)
    ntok, W = h.shape
    top = idx.shape[1]
    rows = F if act == "relu2" else 2 * F
    if out.shape != (ntok, top, W) or (E and (gate_up.shape != (E, rows, W) or down.shape != (E, W, F))):
        raise ValueError("moe_expert_grouped: shapes do not match")
    lib = _lib.load_seq()
    ws = _workspace("moe_grouped", lib.qspec_moe_grouped_workspace_bytes(ntok, top, E, F), h.device)
    _seq(lib.qspec_moe_expert_grouped_act(_ptr(h), _ptr(gate_up), _ptr(down), _ptr(idx), _ptr(out), ntok, W, F, E, top, float(limit),
                                          EXPERT_ACTS[act], _ptr(ws), ws.numel(), _stream()), "moe_expert_grouped")


def moe_route_chosen(h: torch.Tensor, router_w: torch.Tensor, idx: torch.Tensor, weight: torch.Tensor) -> None:
    """Router whose weights are a softmax over the chosen logits only: the `top` largest of router_w h (float32)."""
    _chk(h, "h", _SEQ_ACT); _chk(router_w, "router_w", (_F32,)); _chk(idx, "idx", (torch.int32,)); _chk(weight, "weight", (_F32,))
    ntok, W = h.shape
    R, top = router_w.shape[0], idx.shape[1]
    if router_w.shape[1] != W or idx.shape != (ntok, top) or weight.shape != (ntok, top):
        raise ValueError("moe_route_chosen: shapes do not match")
    _seq(_lib.load_seq().qspec_moe_route_chosen(_ptr(h), _ptr(router_w), _ptr(idx), _ptr(weight), ntok, W, R, top, _sdt(h), _stream()),
         "moe_route_chosen")


def seq_token_shift(x: torch.Tensor, shift: torch.Tensor, prev: torch.Tensor, out: torch.Tensor, meta: torch.Tensor) -> None:
    """out_t = x_t + (x_(t-1) - x_t) * shift; prev float32 [2, slots, W] carries each sequence's last row between steps."""
    _chk(x, "x", (_F32,)); _chk(shift, "shift", (_F32,)); _chk(prev, "prev", (_F32,)); _chk(out, "out", _SEQ_ACT)
    _chk(meta, "meta", (torch.int32,))
    ntok, W = x.shape
    if out.shape != (ntok, W) or shift.numel() != W or prev.dim() != 3 or prev.shape[0] != 2 or prev.shape[2] != W or meta.shape != (5, ntok):
        raise ValueError("seq_token_shift: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_token_shift(_ptr(x), _ptr(shift), _ptr(prev), prev.shape[1], _ptr(out), _ptr(meta), ntok, W, _sdt(out),
                                               _stream()), "seq_token_shift")


def seq_add_norm(y: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, *, kind: str = "layer",
                 x_in: Optional[torch.Tensor] = None, x_out: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 y_w: Optional[torch.Tensor] = None) -> None:
    """r = x_in + norm(sum of y's parts) (x_in None: the norm alone); kind "layer": (v - mean) / sqrt(var + eps) * w + b,
    "rms": v / sqrt(mean(v^2) + eps) * w. y [ntok, W] or [ntok, parts, W] with weights y_w [ntok, parts]. r goes to x_out
    (float32; may be x_in) and, in out's type, to out."""
    _chk(w, "w", (_F32,)); _chk(b, "b", (_F32,), allow_none=True); _chk(x_in, "x_in", (_F32,), allow_none=True)
    _chk(x_out, "x_out", (_F32,), allow_none=True); _chk(out, "out", _SEQ_ACT, allow_none=True); _chk(y_w, "y_w", (_F32,), allow_none=True)
    _chk(y, "y", _SEQ_ACT)
    ntok, W = y.shape[0], y.shape[-1]
    parts, pstride, tstride = (y.shape[1], W, y.shape[1] * W) if y.dim() == 3 else (1, 0, W)
    for t in (x_in, x_out, out):
        if t is not None and t.shape != (ntok, W):
            raise ValueError("seq_add_norm: shapes do not match")
    if w.numel() != W or (y_w is not None and y_w.shape != (ntok, parts)):
        raise ValueError("seq_add_norm: shapes do not match")
    act = _sdt(out) if out is not None else _sdt(y)
    _seq(_lib.load_seq().qspec_seq_add_norm(_ptr(x_in), _ptr(x_out), _ptr(y), parts, pstride, tstride, _ptr(y_w), _ptr(w), _ptr(b),
                                            {"layer": 0, "rms": 1}[kind], _ptr(out), ntok, W, float(eps), _sdt(y), act, _stream()),
         "seq_add_norm")


ROTARY_PAIRINGS = {"halves": 0, "interleaved": 1}      # QSPEC_ROTARY_* of include/qspec_b200_seq.h


def seq_latent_prep(d: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, qn_w: Optional[torch.Tensor], kvn_w: Optional[torch.Tensor],
                    inv_freq: Optional[torch.Tensor], rot_dims: int, cq: Optional[torch.Tensor], cache: Optional[torch.Tensor],
                    meta: torch.Tensor, eps: float, pairing: str = "halves") -> None:
    """Norms of the low-rank query / key-value projections and the rotary key part; with `cache` [slots, cap, kv_rank + rot_dim]
    the step's rows are written at position % cap. q_rank 0: the rows hold no query latent (qn_w and cq None). pairing: which
    entries of the rotary part turn together, (i, i + rot_dims / 2) "halves" or (2i, 2i + 1) "interleaved"."""
    _chk(d, "d", _SEQ_ACT); _chk(cq, "cq", (d.dtype,), allow_none=q_rank == 0); _chk(cache, "cache", (d.dtype,), allow_none=True)
    _chk(qn_w, "qn_w", (_F32,), allow_none=q_rank == 0); _chk(kvn_w, "kvn_w", (_F32,), allow_none=True)
    _chk(inv_freq, "inv_freq", (_F32,), allow_none=True)
    ntok = d.shape[0]
    if (q_rank and cq.shape != (ntok, q_rank)) or (cache is not None and cache.shape[2] != kv_rank + rot_dim):
        raise ValueError("seq_latent_prep: shapes do not match")
    cap = cache.shape[1] if cache is not None else 1
    _seq(_lib.load_seq().qspec_seq_latent_prep_pairing(_ptr(d), d.shape[1], q_rank, kv_rank, rot_dim, _ptr(qn_w), _ptr(kvn_w),
                                                       _ptr(inv_freq), rot_dims, ROTARY_PAIRINGS[pairing], _ptr(cq), _ptr(cache), cap,
                                                       _ptr(meta), ntok, float(eps), _sdt(d), _stream()), "seq_latent_prep")


def seq_rotary(src: torch.Tensor, off: int, dst: torch.Tensor, rot_dims: int, inv_freq: torch.Tensor, meta: torch.Tensor,
               pairing: str = "halves") -> None:
    """dst [ntok, H, n] float32 (a view with a unit last stride will do) = rotary positions on src[t, h, off : off + n]
    (src [ntok, H, head size]); pairing as for `seq_latent_prep`."""
    _chk(src, "src", _SEQ_ACT); _chk(inv_freq, "inv_freq", (_F32,))
    ntok, H, n = dst.shape
    if dst.dtype != _F32 or not dst.is_cuda or dst.stride(2) != 1 or src.shape[:2] != (ntok, H) or off + n > src.shape[2]:
        raise ValueError("seq_rotary: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_rotary_pairing(_ptr(src), H * src.shape[2], src.shape[2], off, dst.data_ptr(), dst.stride(0),
                                                  dst.stride(1), H, n, rot_dims, ROTARY_PAIRINGS[pairing], _ptr(inv_freq), _ptr(meta),
                                                  ntok, _sdt(src), _stream()), "seq_rotary")


def seq_qkv_prep(p: torch.Tensor, HD: int, GD: int, GDV: int, qn_w: torch.Tensor, kn_w: torch.Tensor, qout: torch.Tensor,
                 cache_k: torch.Tensor, cache_v: torch.Tensor, meta: torch.Tensor, eps: float) -> None:
    """Whole-projection norms of q and k of rows [q | k | v | ...]; q to float32 qout, k and v to their ring caches
    [slots, cap, GD] / [slots, cap, GDV] at position % cap."""
    _chk(p, "p", _SEQ_ACT); _chk(qout, "qout", (_F32,)); _chk(cache_k, "cache_k", (p.dtype,)); _chk(cache_v, "cache_v", (p.dtype,))
    _chk(qn_w, "qn_w", (_F32,)); _chk(kn_w, "kn_w", (_F32,))
    ntok = p.shape[0]
    if qout.shape != (ntok, HD) or cache_k.shape[2] != GD or cache_v.shape[2] != GDV or cache_k.shape[:2] != cache_v.shape[:2]:
        raise ValueError("seq_qkv_prep: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_qkv_prep(_ptr(p), p.shape[1], HD, GD, GDV, _ptr(qn_w), _ptr(kn_w), _ptr(qout), _ptr(cache_k),
                                            _ptr(cache_v), cache_k.shape[1], _ptr(meta), ntok, float(eps), _sdt(p), _stream()),
         "seq_qkv_prep")


def seq_window_attention(qa: torch.Tensor, qb: Optional[torch.Tensor], cache_k: torch.Tensor, cache_v: torch.Tensor, out: torch.Tensor,
                         meta: torch.Tensor, window: int, scale: float, sink: Optional[torch.Tensor] = None,
                         gate: Optional[torch.Tensor] = None, gate_per_head: bool = False) -> None:
    """Sliding-window softmax attention with a per-head sink over ring caches.
    qa [ntok, H, DA] and qb [ntok, H, DB] (float32, any strides with a unit last stride): the two parts of the query;
    cache_k [slots, cap, G, DA + DB], cache_v [slots, cap, G, DV] (views with a unit last stride: a latent cache passes two
    views of one buffer); out [ntok, H, DV]; gate [ntok, >= H * DV] (sigmoid applied) or None; gate_per_head: gate is [ntok, >= H],
    one number per head. sink None: an ordinary softmax."""
    import ctypes
    if qa.dtype != _F32 or (qb is not None and qb.dtype != _F32):
        raise ValueError("seq_window_attention: queries are float32")
    if cache_k.dtype != out.dtype or cache_v.dtype != out.dtype or (gate is not None and gate.dtype != out.dtype):
        raise ValueError("seq_window_attention: caches, gate and out share one element type")
    _chk(out, "out", _SEQ_ACT)
    ntok, H, DA = qa.shape
    DB = qb.shape[2] if qb is not None else 0
    slots, cap, G, DK = cache_k.shape
    DV = cache_v.shape[3]
    if DK != DA + DB or out.shape != (ntok, H, DV) or cache_v.shape[:3] != (slots, cap, G) or meta.shape != (5, ntok):
        raise ValueError("seq_window_attention: shapes do not match")
    for t in (qa, qb, cache_k, cache_v):
        if t is not None and t.stride(-1) != 1:
            raise ValueError("seq_window_attention: the last stride must be 1")
    a = _lib.WindowAttnArgs(qa.data_ptr(), qa.stride(0), qa.stride(1), DA,
                            qb.data_ptr() if qb is not None else None, qb.stride(0) if qb is not None else 0,
                            qb.stride(1) if qb is not None else 0, DB,
                            cache_k.data_ptr(), cache_k.stride(0), cache_k.stride(1), cache_k.stride(2),
                            cache_v.data_ptr(), cache_v.stride(0), cache_v.stride(1), cache_v.stride(2), DV,
                            _ptr(sink), gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0,
                            _ptr(out), _ptr(meta), ntok, H, G, int(window), cap, float(scale), int(gate_per_head))
    _seq(_lib.load_seq().qspec_seq_window_attention(ctypes.byref(a), _sdt(out), _stream()), "seq_window_attention")


def seq_window_attention_mma_supported(out_dtype, DA: int, DB: int, DV: int, H: int, G: int, token_rows: bool) -> bool:
    """The tensor-core form takes bfloat16 caches with per-head key parts of 64 or 128 (128 with a shared part of 64) and
    values of 64 or 128; with heads as rows, at most 16 query heads per key/value head."""
    return bool(out_dtype == _BF16 and _lib.load_seq().qspec_seq_window_attention_mma_supported(DA, DB, DV, H, G, int(token_rows)))


def seq_window_attention_mma(q: torch.Tensor, cache_k: torch.Tensor, k_shared: Optional[torch.Tensor], cache_v: torch.Tensor,
                             out: torch.Tensor, meta: torch.Tensor, window: int, scale: float, token_rows: bool,
                             sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                             gate_per_head: bool = False) -> None:
    """`seq_window_attention` on the tensor cores (bfloat16). q [ntok, H, DK] float32; cache_k [slots, cap, G, DA] holds the
    per-head part of the keys and k_shared [slots, cap, DB] (or None) the part all heads share, DK = DA + DB; cache_v
    [slots, cap, G, DV] (views: a slot stride of 0 serves one buffer to every slot). token_rows: False = the rows of the
    products are the query heads of a group, one CTA per (token, key/value head): decoding; True = 16 consecutive batch
    tokens per CTA and head: prompts."""
    import ctypes
    if q.dtype != _F32 or cache_k.dtype != _BF16 or cache_v.dtype != _BF16 or out.dtype != _BF16:
        raise ValueError("seq_window_attention_mma: float32 queries, bfloat16 caches and output")
    _chk(out, "out", (_BF16,))
    ntok, H, DK = q.shape
    slots, cap, G, DA = cache_k.shape
    DB = k_shared.shape[2] if k_shared is not None else 0
    DV = cache_v.shape[3]
    if DK != DA + DB or out.shape != (ntok, H, DV) or cache_v.shape[:3] != (slots, cap, G) or meta.shape != (5, ntok) \
            or (k_shared is not None and k_shared.shape[:2] != (slots, cap)):
        raise ValueError("seq_window_attention_mma: shapes do not match")
    for t in (q, cache_k, cache_v, k_shared):
        if t is not None and t.stride(-1) != 1:
            raise ValueError("seq_window_attention_mma: the last stride must be 1")
    a = _lib.WindowAttnArgs(q.data_ptr(), q.stride(0), q.stride(1), DK, None, 0, 0, 0,
                            cache_k.data_ptr(), cache_k.stride(0), cache_k.stride(1), cache_k.stride(2),
                            cache_v.data_ptr(), cache_v.stride(0), cache_v.stride(1), cache_v.stride(2), DV,
                            _ptr(sink), gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0,
                            _ptr(out), _ptr(meta), ntok, H, G, int(window), cap, float(scale), int(gate_per_head))
    _seq(_lib.load_seq().qspec_seq_window_attention_mma(ctypes.byref(a), k_shared.data_ptr() if k_shared is not None else None,
                                                        k_shared.stride(0) if k_shared is not None else 0,
                                                        k_shared.stride(1) if k_shared is not None else 0, DB, int(token_rows), _stream()),
         "seq_window_attention_mma")


def seq_hgrn2(p: torch.Tensor, f_b: torch.Tensor, lower: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, scratch: torch.Tensor,
              out: torch.Tensor, meta: torch.Tensor, H: int, D: int, DV: int, eps: float, seg_starts: Optional[torch.Tensor] = None) -> None:
    """HGRN2 recurrence over rows [zq | zf | v] with the per-slot state float32 [slots, H, D, DV]; out [ntok, H * DV] after the
    per-head norm; scratch float32 with room for ntok * H * (DV + 3 D) values. seg_starts: int32, the batch row of every segment's first
    token (`BatchMeta.seg_starts`): one CTA per segment instead of one per token."""
    _chk(seg_starts, "seg_starts", (torch.int32,), allow_none=True)
    _chk(p, "p", _SEQ_ACT); _chk(out, "out", (p.dtype,)); _chk(state, "state", (_F32,)); _chk(scratch, "scratch", (_F32,))
    for t, n in ((f_b, "f_b"), (lower, "lower"), (norm_w, "norm_w")):
        _chk(t, n, (_F32,))
    ntok = p.shape[0]
    if out.shape != (ntok, H * DV) or state.shape[1:] != (H, D, DV) or scratch.numel() < ntok * H * (DV + 3 * D) or norm_w.numel() != DV \
            or f_b.numel() != H * D or lower.numel() != H * D:
        raise ValueError("seq_hgrn2: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_hgrn2(_ptr(p), p.shape[1], _ptr(f_b), _ptr(lower), _ptr(norm_w), _ptr(state), _ptr(scratch), _ptr(out),
                                         _ptr(meta), _ptr(seg_starts), 0 if seg_starts is None else seg_starts.numel(), ntok, H, D, DV,
                                         float(eps), _sdt(p), _stream()), "seq_hgrn2")


def seq_side_gate(g: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int) -> None:
    """g [ntok, sd] <- gelu_tanh(g) * table[ids, col0 : col0 + sd], in place."""
    _chk(g, "g", _SEQ_ACT); _chk(table, "table", (g.dtype,)); _chk(ids, "ids", (torch.int32,))
    ntok, sd = g.shape
    _seq(_lib.load_seq().qspec_seq_side_gate(_ptr(g), _ptr(table), _ptr(ids), col0, sd, table.shape[1], table.shape[0], ntok, _sdt(g),
                                             _stream()), "seq_side_gate")


def seq_residual_norm(x_in: torch.Tensor, w: Optional[torch.Tensor], eps: float, *, y: Optional[torch.Tensor] = None,
                      y_w: Optional[torch.Tensor] = None, y2: Optional[torch.Tensor] = None, y2_w: Optional[torch.Tensor] = None,
                      mult: float = 1.0, w_offset: float = 1.0, x_out: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None, y_scale: Optional[torch.Tensor] = None) -> None:
    """r = x_in + mult * y_scale * (sum of y's parts, each times y_w [ntok, parts] if given, + y2_w * y2); out = r / rms(r) *
    (w_offset + w). y_scale: float32 [W], one factor per column (a layer scale), None: ones.
    y [ntok, W] or [ntok, parts, W]; y2 [ntok, W] with one weight per token (y2_w: a float32 vector view, any stride). r goes to
    x_out (float32; may be x_in), the norm to out (activation type). w_offset 1: the weight is stored around zero; 0: plain."""
    _chk(x_in, "x_in", (_F32,)); _chk(w, "w", (_F32,), allow_none=out is None); _chk(x_out, "x_out", (_F32,), allow_none=True)
    _chk(out, "out", _SEQ_ACT, allow_none=True); _chk(y, "y", _SEQ_ACT, allow_none=True); _chk(y_w, "y_w", (_F32,), allow_none=True)
    ntok, W = x_in.shape
    parts, pstride, tstride = 1, 0, W
    if y is not None:
        if y.dim() == 3:
            parts, pstride, tstride = y.shape[1], W, y.shape[1] * W
        if y.shape[0] != ntok or y.shape[-1] != W or (y_w is not None and y_w.shape != (ntok, parts)):
            raise ValueError("seq_residual_norm: y / y_w shapes do not match x")
    w2_stride = 0
    if y2 is not None:
        _chk(y2, "y2", (y.dtype,) if y is not None else _SEQ_ACT)
        if y2.shape != (ntok, W):
            raise ValueError("seq_residual_norm: y2 must be [ntok, W]")
        if y2_w is not None:
            if y2_w.dtype != _F32 or not y2_w.is_cuda or y2_w.dim() != 1 or y2_w.shape[0] != ntok:
                raise ValueError("seq_residual_norm: y2_w must be a float32 vector of ntok entries")
            w2_stride = y2_w.stride(0)
    for t in (x_out, out):
        if t is not None and t.shape != (ntok, W):
            raise ValueError("seq_residual_norm: shapes do not match")
    _chk(y_scale, "y_scale", (_F32,), allow_none=True)
    if (w is not None and w.numel() != W) or (y_scale is not None and y_scale.numel() != W):
        raise ValueError("seq_residual_norm: the norm weight and the column factors have W entries")
    src = y if y is not None else y2
    act = _sdt(out) if out is not None else (_sdt(src) if src is not None and src.dtype != _F32 else _lib.DTYPE_F32)
    ydt = _sdt(src) if src is not None else act
    _seq(_lib.load_seq().qspec_seq_residual_norm_scaled(_ptr(x_in), _ptr(x_out), _ptr(y), parts, pstride, tstride, _ptr(y_w), _ptr(y2),
                                                        y2_w.data_ptr() if y2_w is not None else None, w2_stride, float(mult),
                                                        _ptr(y_scale), _ptr(w), float(w_offset), _ptr(out), ntok, W, float(eps), ydt,
                                                        act, _stream()), "seq_residual_norm")


SEQ_ACTS = {"relu2": 0, "gelu_erf": 1}                 # QSPEC_ACT_* of include/qspec_b200_seq.h


def seq_act(a: torch.Tensor, act: str) -> None:
    """a <- act(a) in place: "relu2" (squared ReLU) or "gelu_erf" (the exact GELU)."""
    _chk(a, "a", _SEQ_ACT)
    _seq(_lib.load_seq().qspec_seq_act(_ptr(a), a.numel(), SEQ_ACTS[act], _sdt(a), _stream()), "seq_act")


def seq_silu_mul(gu: torch.Tensor, out: torch.Tensor) -> None:
    """out [ntok, F] = silu(gu[:, :F]) * gu[:, F:] for rows [gate | up]."""
    _chk(gu, "gu", _SEQ_ACT); _chk(out, "out", (gu.dtype,))
    ntok, F = out.shape
    if gu.shape != (ntok, 2 * F):
        raise ValueError("seq_silu_mul: gu must be [ntok, 2 F]")
    _seq(_lib.load_seq().qspec_seq_silu_mul(_ptr(gu), 2 * F, _ptr(out), ntok, F, _sdt(gu), _stream()), "seq_silu_mul")


def seq_lightning(p: torch.Tensor, decay: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, scratch: torch.Tensor,
                  out: torch.Tensor, meta: torch.Tensor, H: int, D: int, DV: int, eps: float,
                  seg_starts: Optional[torch.Tensor] = None) -> None:
    """Linear attention with one decay per head over rows [zq | zk | zv | zg] (silu on q, k, v; state S <- decay S + k v^T, float32
    [slots, H, D, DV]); out [ntok, H * DV] = the heads normed together, times norm_w and sigmoid(zg). scratch float32 with room for
    ntok * H * (DV + 2 D) values. seg_starts as for `seq_hgrn2`."""
    _chk(seg_starts, "seg_starts", (torch.int32,), allow_none=True)
    _chk(p, "p", _SEQ_ACT); _chk(out, "out", (p.dtype,)); _chk(state, "state", (_F32,)); _chk(scratch, "scratch", (_F32,))
    _chk(decay, "decay", (_F32,)); _chk(norm_w, "norm_w", (_F32,))
    ntok = p.shape[0]
    if out.shape != (ntok, H * DV) or state.shape[1:] != (H, D, DV) or scratch.numel() < ntok * H * (DV + 2 * D) or \
            norm_w.numel() != H * DV or decay.numel() != H or p.shape[1] < 2 * H * (D + DV) or meta.shape != (5, ntok):
        raise ValueError("seq_lightning: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_lightning(_ptr(p), p.shape[1], _ptr(decay), _ptr(norm_w), _ptr(state), _ptr(scratch), _ptr(out),
                                             _ptr(meta), _ptr(seg_starts), 0 if seg_starts is None else seg_starts.numel(), ntok, H, D,
                                             DV, float(eps), _sdt(p), _stream()), "seq_lightning")


def moe_route_grouped(h: torch.Tensor, router_w: torch.Tensor, correction: Optional[torch.Tensor], idx: torch.Tensor,
                      weight: torch.Tensor, *, score: str = "sigmoid", groups: int = 1, keep: int = 1, group_top: int = 2,
                      scale: float = 1.0, extra: Optional[torch.Tensor] = None) -> None:
    """Router with expert groups: scores s = sigmoid or softmax of router_w h (float32), choice = s + correction; the experts form
    `groups` equal groups of neighbours, a group scores the sum of its `group_top` largest choices and only the `keep` best groups
    stay; idx int32 [ntok, top] = the largest remaining choices, weight float32 [ntok, top] = scale * s. Rows of router_w past the
    experts ([R + n, W]) are gate rows: extra float32 [ntok, n] (a view with a unit last stride) receives their sigmoid."""
    _chk(h, "h", _SEQ_ACT); _chk(router_w, "router_w", (_F32,)); _chk(correction, "correction", (_F32,), allow_none=True)
    _chk(idx, "idx", (torch.int32,)); _chk(weight, "weight", (_F32,))
    ntok, W = h.shape
    top = idx.shape[1]
    n_extra = 0
    if extra is not None:
        if extra.dtype != _F32 or not extra.is_cuda or extra.dim() != 2 or extra.shape[0] != ntok or extra.stride(1) != 1:
            raise ValueError("moe_route_grouped: extra must be float32 [ntok, n] with a unit last stride")
        n_extra = extra.shape[1]
    R = router_w.shape[0] - n_extra
    if router_w.shape[1] != W or R < 1 or (correction is not None and correction.numel() != R) or idx.shape != (ntok, top) or \
            weight.shape != (ntok, top):
        raise ValueError("moe_route_grouped: shapes do not match")
    _seq(_lib.load_seq().qspec_moe_route_grouped(_ptr(h), _ptr(router_w), _ptr(correction), _ptr(idx), _ptr(weight),
                                                 extra.data_ptr() if extra is not None else None,
                                                 extra.stride(0) if extra is not None else 0, ntok, W, R, top,
                                                 {"softmax": 0, "sigmoid": 1}[score], int(groups), int(keep), int(group_top),
                                                 float(scale), n_extra, _sdt(h), _stream()), "moe_route_grouped")


def seq_prompt_attention_mma_supported(out_dtype, DA: int, DB: int, DV: int) -> bool:
    """The tile form of a prompt portion takes bfloat16 caches with per-head key parts of 128 (+ a shared part of 64, or none)
    and values of 128, or keys and values of 64."""
    return bool(out_dtype == _BF16 and _lib.load_seq().qspec_seq_prompt_attention_mma_supported(DA, DB, DV))


def seq_prompt_attention_mma(q: torch.Tensor, cache_k: torch.Tensor, k_shared: Optional[torch.Tensor], cache_v: torch.Tensor,
                             out: torch.Tensor, slot: int, pos0: int, window: int, scale: float,
                             sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                             gate_per_head: bool = False) -> None:
    """Softmax attention of one prompt portion on the tensor cores (bfloat16): the rows of q [ntok, H, DK] (float32) are the
    consecutive positions pos0 .. pos0 + ntok - 1 of the sequence in `slot`. 64 tokens and one head per CTA; every visible key /
    value row is read once per 64 queries. cache_k [slots, cap, G, DA], k_shared [slots, cap, DB] or None (DK = DA + DB), cache_v
    [slots, cap, G, DV] as for `seq_window_attention_mma`; window, sink, gate likewise."""
    import ctypes
    if q.dtype != _F32 or cache_k.dtype != _BF16 or cache_v.dtype != _BF16 or out.dtype != _BF16:
        raise ValueError("seq_prompt_attention_mma: float32 queries, bfloat16 caches and output")
    _chk(out, "out", (_BF16,))
    ntok, H, DK = q.shape
    slots, cap, G, DA = cache_k.shape
    DB = k_shared.shape[2] if k_shared is not None else 0
    DV = cache_v.shape[3]
    if DK != DA + DB or out.shape != (ntok, H, DV) or cache_v.shape[:3] != (slots, cap, G) or not 0 <= slot < slots \
            or (k_shared is not None and k_shared.shape[:2] != (slots, cap)) or (gate is not None and gate.dtype != _BF16):
        raise ValueError("seq_prompt_attention_mma: shapes do not match")
    for t in (q, cache_k, cache_v, k_shared):
        if t is not None and t.stride(-1) != 1:
            raise ValueError("seq_prompt_attention_mma: the last stride must be 1")
    a = _lib.WindowAttnArgs(q.data_ptr(), q.stride(0), q.stride(1), DK, None, 0, 0, 0,
                            cache_k.data_ptr(), cache_k.stride(0), cache_k.stride(1), cache_k.stride(2),
                            cache_v.data_ptr(), cache_v.stride(0), cache_v.stride(1), cache_v.stride(2), DV,
                            _ptr(sink), gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0,
                            _ptr(out), None, ntok, H, G, int(window), cap, float(scale), int(gate_per_head))
    _seq(_lib.load_seq().qspec_seq_prompt_attention_mma(ctypes.byref(a), k_shared.data_ptr() if k_shared is not None else None,
                                                        k_shared.stride(0) if k_shared is not None else 0,
                                                        k_shared.stride(1) if k_shared is not None else 0, DB, int(slot), int(pos0),
                                                        _stream()), "seq_prompt_attention_mma")


# ---- mixers whose state is a matrix that every token rewrites; attention with mixed heads ---------------------------------------
def _rows(t: torch.Tensor, name: str, dtypes) -> None:
    """A CUDA matrix view whose rows are contiguous (any leading dimension)."""
    if t is None or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype not in dtypes:
        raise ValueError(f"{name}: a CUDA matrix of {dtypes} with a unit last stride expected")


CONV_ACTS = {None: 0, "none": 0, "silu": 1}            # QSPEC_CONV_ACT_* of include/qspec_b200_seq.h


def seq_conv_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], tail: torch.Tensor, out: torch.Tensor,
                 meta: torch.Tensor, act: Optional[str] = "silu") -> None:
    """Short causal convolution per channel with an activation. x [ntok, C] (a view with any leading dimension), w float32
    [C, taps] (the last column meets the current token), bias float32 [C] or None, tail float32 [2, slots, taps - 1, C] (the
    sequences' last inputs, double-buffered by the step's phase), out [ntok, C] (view) of x's type or float32."""
    _rows(x, "x", _SEQ_ACT); _rows(out, "out", (x.dtype, _F32))
    _chk(w, "w", (_F32,)); _chk(bias, "bias", (_F32,), allow_none=True); _chk(tail, "tail", (_F32,))
    ntok, C = x.shape
    taps = w.shape[1]
    if w.shape[0] != C or out.shape != (ntok, C) or tail.dim() != 4 or tail.shape[0] != 2 or tail.shape[2:] != (taps - 1, C) or \
            (bias is not None and bias.numel() != C) or meta.shape != (5, ntok):
        raise ValueError("seq_conv_act: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_conv_act(x.data_ptr(), x.stride(0), _ptr(w), _ptr(bias), C, taps, CONV_ACTS[act], _ptr(tail),
                                            tail.shape[1], out.data_ptr(), out.stride(0), int(out.dtype == _F32 and x.dtype != _F32),
                                            _ptr(meta), ntok, _sdt(x), _stream()), "seq_conv_act")


def seq_delta_rule(cs: torch.Tensor, ba: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor,
                   gate: Optional[torch.Tensor], state: torch.Tensor, gates: torch.Tensor, o: torch.Tensor, out: torch.Tensor,
                   meta: torch.Tensor, seg_starts: torch.Tensor, H: int, G: int, D: int, DV: int, eps: float, unit_eps: float = 1e-6,
                   q_mult: Optional[float] = None) -> None:
    """Gated delta rule over rows cs = [q (G x D) | k (G x D) | v (H x DV)] (float32, after convolution and activation; q and k
    are made unit vectors in place, q times q_mult, default D^-1/2). ba float32 [ntok, 2 H] = [b | a]: beta = sigmoid(b), decay =
    exp(-exp(A_log) softplus(a + dt_bias)). Per head S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; out [ntok, H *
    DV] = unit_rms(o) * norm_w * silu(gate) (gate [ntok, H * DV] view of out's type, or None). state float32 [slots, H, D, DV];
    scratch: gates float32 >= ntok * (2 H + G), o float32 >= ntok * H * DV."""
    _rows(cs, "cs", (_F32,)); _chk(ba, "ba", (_F32,)); _chk(out, "out", _SEQ_ACT); _chk(state, "state", (_F32,))
    _chk(gates, "gates", (_F32,)); _chk(o, "o", (_F32,)); _chk(seg_starts, "seg_starts", (torch.int32,))
    for t, n in ((A_log, "A_log"), (dt_bias, "dt_bias"), (norm_w, "norm_w")):
        _chk(t, n, (_F32,))
    ntok = cs.shape[0]
    if gate is not None:
        _rows(gate, "gate", (out.dtype,))
    if cs.shape[1] < 2 * G * D + H * DV or ba.shape != (ntok, 2 * H) or out.shape != (ntok, H * DV) or state.shape[1:] != (H, D, DV) or \
            gates.numel() < ntok * (2 * H + G) or o.numel() < ntok * H * DV or A_log.numel() != H or dt_bias.numel() != H or \
            norm_w.numel() != DV or meta.shape != (5, ntok) or (gate is not None and gate.shape != (ntok, H * DV)):
        raise ValueError("seq_delta_rule: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_delta_rule(cs.data_ptr(), cs.stride(0), _ptr(ba), _ptr(A_log), _ptr(dt_bias), _ptr(norm_w),
                                              gate.data_ptr() if gate is not None else None, gate.stride(0) if gate is not None else 0,
                                              _ptr(state), _ptr(gates), _ptr(o), _ptr(out), _ptr(meta), _ptr(seg_starts),
                                              seg_starts.numel(), ntok, H, G, D, DV, float(unit_eps),
                                              float(D ** -0.5 if q_mult is None else q_mult), float(eps), _sdt(out), _stream()),
         "seq_delta_rule")


def seq_selective_scan(x: torch.Tensor, dt_pre: torch.Tensor, dt_bias: torch.Tensor, bc: torch.Tensor, z: torch.Tensor,
                       A_log: torch.Tensor, D_skip: torch.Tensor, state: torch.Tensor, out: torch.Tensor, meta: torch.Tensor,
                       seg_starts: torch.Tensor) -> None:
    """Selective scan: dt = softplus(dt_pre + dt_bias) (float32 [ntok, inner]); per channel and state S <- exp(-dt exp(A_log)) S +
    dt x B, y = S . C + D_skip x; out = y * silu(z). x, z, out [ntok, inner] and bc [ntok, 2 N] = [B | C] are views of the
    activation type; state float32 [slots, inner, N]."""
    _rows(x, "x", _SEQ_ACT)
    for t, n in ((bc, "bc"), (z, "z"), (out, "out")):
        _rows(t, n, (x.dtype,))
    _rows(dt_pre, "dt_pre", (_F32,)); _chk(state, "state", (_F32,)); _chk(seg_starts, "seg_starts", (torch.int32,))
    for t, n in ((dt_bias, "dt_bias"), (A_log, "A_log"), (D_skip, "D_skip")):
        _chk(t, n, (_F32,))
    ntok, inner = x.shape
    N = A_log.shape[1]
    if A_log.shape != (inner, N) or bc.shape != (ntok, 2 * N) or z.shape != (ntok, inner) or out.shape != (ntok, inner) or \
            dt_pre.shape != (ntok, inner) or dt_bias.numel() != inner or D_skip.numel() != inner or state.shape[1:] != (inner, N) or \
            meta.shape != (5, ntok):
        raise ValueError("seq_selective_scan: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_selective_scan(x.data_ptr(), x.stride(0), dt_pre.data_ptr(), dt_pre.stride(0), _ptr(dt_bias),
                                                  bc.data_ptr(), bc.stride(0), z.data_ptr(), z.stride(0), _ptr(A_log), _ptr(D_skip),
                                                  _ptr(state), out.data_ptr(), out.stride(0), _ptr(meta), _ptr(seg_starts),
                                                  seg_starts.numel(), ntok, inner, N, _sdt(x), _stream()), "seq_selective_scan")


def seq_gqa_prep(p: torch.Tensor, qn_w: torch.Tensor, kn_w: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dims: int,
                 qout: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, meta: torch.Tensor, H: int, eps: float, *,
                 v_norm: bool = True, v_first_in: Optional[torch.Tensor] = None, v_first_out: Optional[torch.Tensor] = None,
                 mix: Optional[torch.Tensor] = None) -> None:
    """Grouped-query attention after the fused projection p = [q (H x D) | k (G x D) | v (G x DV)] (biases added): per-head unit-RMS
    norms with the weights qn_w / kn_w [D], rotation of the first rot_dims entries (entry i with i + rot_dims / 2, angle pos *
    inv_freq[i]), values normed without a weight if v_norm, then v <- (1 - mix) v + mix v_first_in if v_first_in is given (mix a
    float32 scalar tensor), else copied to v_first_out if that is given (both float32 [ntok, G * DV]). qout float32 [ntok, H, D];
    cache_k [slots, cap, G, D], cache_v [slots, cap, G, DV] of p's type take row pos % cap."""
    _rows(p, "p", _SEQ_ACT); _chk(qout, "qout", (_F32,)); _chk(cache_k, "cache_k", (p.dtype,)); _chk(cache_v, "cache_v", (p.dtype,))
    _chk(qn_w, "qn_w", (_F32,)); _chk(kn_w, "kn_w", (_F32,)); _chk(inv_freq, "inv_freq", (_F32,), allow_none=rot_dims == 0)
    _chk(v_first_in, "v_first_in", (_F32,), allow_none=True); _chk(v_first_out, "v_first_out", (_F32,), allow_none=True)
    _chk(mix, "mix", (_F32,), allow_none=v_first_in is None)
    ntok = p.shape[0]
    slots, cap, G, D = cache_k.shape
    DV = cache_v.shape[3]
    if cache_v.shape[:3] != (slots, cap, G) or qout.shape != (ntok, H, D) or p.shape[1] < (H + G) * D + G * DV or qn_w.numel() != D or \
            kn_w.numel() != D or meta.shape != (5, ntok) or (rot_dims and inv_freq.numel() != rot_dims // 2) or \
            any(t is not None and t.numel() < ntok * G * DV for t in (v_first_in, v_first_out)):
        raise ValueError("seq_gqa_prep: shapes do not match")
    _seq(_lib.load_seq().qspec_seq_gqa_prep(p.data_ptr(), p.stride(0), _ptr(qn_w), _ptr(kn_w), _ptr(inv_freq), int(rot_dims),
                                            _ptr(v_first_in), _ptr(v_first_out), _ptr(mix), _ptr(qout), _ptr(cache_k), _ptr(cache_v),
                                            cap, _ptr(meta), ntok, H, G, D, DV, float(eps), int(v_norm), _sdt(p), _stream()),
         "seq_gqa_prep")


def seq_talking_attention(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, talk: torch.Tensor, out: torch.Tensor,
                          meta: torch.Tensor, window: int, scale: float, sink: Optional[torch.Tensor] = None,
                          rows_per_cta: int = 1) -> None:
    """Softmax attention whose heads' weights are mixed after the softmax: weight_g(j) = exp(s_g(j)) / (exp(sink[g]) + sum_j
    exp(s_g(j))) with s = scale * q_g . k (sink None: no such term); head h applies sum_g talk[h, g] weight_g to the values of its
    own key/value head. q float32 [ntok, H, D]; cache_k [slots, cap, G, D], cache_v [slots, cap, G, DV] (views with a unit last
    stride, row = position % cap); talk float32 [H, H]; out [ntok, H, DV]; a token at position i sees keys j with 0 <= i - j <
    window. rows_per_cta 4: a CTA takes four consecutive batch rows, which share their key and value loads where they belong to
    one sequence (prompt portions); 1: one row per CTA (decode-shaped batches)."""
    import ctypes
    _chk(q, "q", (_F32,)); _chk(out, "out", _SEQ_ACT); _chk(talk, "talk", (_F32,)); _chk(sink, "sink", (_F32,), allow_none=True)
    if cache_k.dtype != out.dtype or cache_v.dtype != out.dtype or cache_k.stride(-1) != 1 or cache_v.stride(-1) != 1:
        raise ValueError("seq_talking_attention: caches share out's element type and have a unit last stride")
    ntok, H, D = q.shape
    slots, cap, G, DK = cache_k.shape
    DV = cache_v.shape[3]
    if DK != D or out.shape != (ntok, H, DV) or cache_v.shape[:3] != (slots, cap, G) or talk.shape != (H, H) or meta.shape != (5, ntok) \
            or (sink is not None and sink.numel() != H):
        raise ValueError("seq_talking_attention: shapes do not match")
    a = _lib.TalkingAttnArgs(q.data_ptr(), cache_k.data_ptr(), cache_k.stride(0), cache_k.stride(1), cache_k.stride(2),
                             cache_v.data_ptr(), cache_v.stride(0), cache_v.stride(1), cache_v.stride(2), _ptr(talk), _ptr(sink),
                             _ptr(out), _ptr(meta), ntok, H, G, D, DV, int(window), cap, float(scale))
    _seq(_lib.load_seq().qspec_seq_talking_attention(ctypes.byref(a), int(rows_per_cta), _sdt(out), _stream()), "seq_talking_attention")


def seq_glu_clamp(gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float = 1.702) -> None:
    """out [ntok, F] = g * sigmoid(alpha g) * (u + 1) with g = min(gu[:, :F], limit), u = clamp(gu[:, F:], -limit, limit)."""
    _chk(gu, "gu", _SEQ_ACT); _chk(out, "out", (gu.dtype,))
    ntok, F = out.shape
    if gu.shape != (ntok, 2 * F):
        raise ValueError("seq_glu_clamp: gu must be [ntok, 2 F]")
    _seq(_lib.load_seq().qspec_seq_glu_clamp(_ptr(gu), 2 * F, _ptr(out), ntok, F, float(limit), float(alpha), _sdt(gu), _stream()),
         "seq_glu_clamp")


def seq_scale(a: torch.Tensor, s: float) -> None:
    """a <- s * a in place (float32)."""
    _chk(a, "a", (_F32,))
    _seq(_lib.load_seq().qspec_seq_scale_f32(_ptr(a), a.numel(), float(s), _stream()), "seq_scale")
