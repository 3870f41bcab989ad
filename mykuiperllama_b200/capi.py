"""Torch-tensor front end of the kernel C ABI (``include/kuiper_b200.h``).

PyTorch only supplies device memory and streams here; every function hands raw device
pointers to the C ABI, which enqueues the hand-written sm_100a kernel on the current
torch stream.  Shapes and dtypes follow the header: activations fp32, bf16 / fp16
tensors as ``torch.bfloat16`` / ``torch.float16`` (or int16 bit patterns), packed INT4
as int32.
"""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, kernels

ACT_FP32, ACT_FP16, ACT_INT16_BLOCK = 0, 1, 2


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dev(*ts):
    for t in ts:
        if t is not None:
            assert t.is_cuda and t.is_contiguous(), "kuiper kernels take contiguous CUDA tensors"


def set_tuning(key: str, value: int) -> None:
    check(kernels().kuiper_set_tuning(key.encode(), value))


def add(a, b, out=None):
    _dev(a, b, out)
    out = torch.empty_like(a) if out is None else out
    check(kernels().kuiper_add_f32(_ptr(a), _ptr(b), _ptr(out), a.numel(), _stream()))
    return out


def awq_unpack(qweight):
    _dev(qweight)
    K, NW = qweight.shape
    out = torch.empty((K, NW * 8), dtype=torch.uint8, device=qweight.device)
    check(kernels().kuiper_awq_unpack_u8(_ptr(qweight), _ptr(out), K, NW * 8, _stream()))
    return out


def awq_dequant(qweight, qzeros, scales, group=128, dtype=torch.float32):
    _dev(qweight, qzeros, scales)
    K, NW = qweight.shape
    out = torch.empty((K, NW * 8), dtype=dtype, device=qweight.device)
    fn = kernels().kuiper_awq_dequant_f32 if dtype == torch.float32 else kernels().kuiper_awq_dequant_bf16
    check(fn(_ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(out), K, NW * 8, group, _stream()))
    return out


def awq_gemv_workspace(M, K, N, device="cuda"):
    n = kernels().kuiper_awq_gemv_workspace_bytes(M, K, N)
    ws = torch.zeros(max(n, 16), dtype=torch.uint8, device=device)  # zeroed: counters start at 0
    return ws


def awq_gemv(x, qweight, qzeros, scales, workspace=None, residual=None, out=None, group=128, act_mode=ACT_FP16):
    _dev(x, qweight, qzeros, scales, workspace, residual, out)
    M, K = x.shape
    N = qweight.shape[1] * 8
    if workspace is None:
        workspace = awq_gemv_workspace(M, K, N, x.device)
    out = torch.empty((M, N), dtype=torch.float32, device=x.device) if out is None else out
    check(kernels().kuiper_awq_gemv_f32(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(out), _ptr(residual),
                                        M, K, N, group, act_mode, _ptr(workspace), workspace.numel(), _stream()))
    return out


def awq_gemv_accum(x, qweight, qzeros, scales, y, group=128):
    """y += x . W (y holds the addend); returns y."""
    _dev(x, qweight, qzeros, scales, y)
    M, K = x.shape
    N = qweight.shape[1] * 8
    check(kernels().kuiper_awq_gemv_accum_f32(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(y), M, K, N, group,
                                              _stream()))
    return y


def rmsnorm_awq_gemv_accum(h, norm_w, eps, qweight, qzeros, scales, y, group=128):
    """y += RMSNorm(h) . W (y holds the addend); returns y."""
    _dev(h, norm_w, qweight, qzeros, scales, y)
    M, K = h.shape
    N = qweight.shape[1] * 8
    check(kernels().kuiper_rmsnorm_awq_gemv_accum_f32(_ptr(h), _ptr(norm_w), eps, _ptr(qweight), _ptr(qzeros), _ptr(scales),
                                                      _ptr(y), M, K, N, group, _stream()))
    return y


def swiglu_awq_gemv_accum(gate_up, qweight, qzeros, scales, y, group=128):
    """y += (silu(gate) * up) . W with gate_up = [M, 2K]; returns y."""
    _dev(gate_up, qweight, qzeros, scales, y)
    M = gate_up.shape[0]
    K = gate_up.shape[1] // 2
    N = qweight.shape[1] * 8
    check(kernels().kuiper_swiglu_awq_gemv_accum_f32(_ptr(gate_up), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(y), M, K, N,
                                                     group, _stream()))
    return y


def awq_gemv_tickets(device="cuda"):
    """Balance counters of one call site (zeroed once; every launch leaves them at zero)."""
    return torch.zeros(max(kernels().kuiper_awq_gemv_ticket_bytes(), 16), dtype=torch.uint8, device=device)


def awq_gemv_accum_balanced(x, qweight, qzeros, scales, y, tickets=None, norm_w=None, eps=1e-6, swiglu=False, group=128,
                            act_mode=ACT_FP16):
    """y += op(x) . W with the tail of the weight stream handed out by ticket (see kuiper_awq_gemv_accum_balanced_f32)."""
    _dev(x, qweight, qzeros, scales, y, tickets, norm_w)
    M = x.shape[0]
    K = x.shape[1] // (2 if swiglu else 1)
    N = qweight.shape[1] * 8
    check(kernels().kuiper_awq_gemv_accum_balanced_f32(_ptr(x), _ptr(norm_w), eps, int(bool(swiglu)), _ptr(qweight), _ptr(qzeros),
                                                       _ptr(scales), _ptr(y), M, K, N, group, act_mode, _ptr(tickets), _stream()))
    return y


class _GemvItem(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("qweight", ctypes.c_void_p), ("qzeros", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("y", ctypes.c_void_p), ("K", ctypes.c_int32), ("N", ctypes.c_int32)]


class GemvGroup:
    """A list of independent one-row projections y_i += x_i . W_i that runs as one persistent launch.
    items: dicts with x [K] or [1, K], qweight, qzeros, scales, y.  The tensors must stay alive while the group is used."""

    def __init__(self, items, group=128, balanced=False, act_mode=ACT_INT16_BLOCK):
        import numpy as np
        n = len(items)
        arr = (_GemvItem * n)()
        for i, o in enumerate(items):
            _dev(o["x"], o["qweight"], o["qzeros"], o["scales"], o["y"])
            arr[i] = _GemvItem(_ptr(o["x"]), _ptr(o["qweight"]), _ptr(o["qzeros"]), _ptr(o["scales"]), _ptr(o["y"]),
                               o["qweight"].shape[0], o["qweight"].shape[1] * 8)
        host = np.zeros(kernels().kuiper_awq_gemv_group_table_bytes(n), np.uint8)
        units = ctypes.c_int64(0)
        check(kernels().kuiper_awq_gemv_group_plan(ctypes.addressof(arr), n, group, host.ctypes.data, ctypes.byref(units)))
        self.keep = items
        self.n, self.units, self.act_mode = n, units.value, act_mode
        self.table = torch.from_numpy(host).cuda()  # torch allocations are 256-byte aligned
        self.tickets = awq_gemv_tickets() if balanced else None

    def run(self):
        check(kernels().kuiper_awq_gemv_group_f32(_ptr(self.table), self.n, self.units, self.act_mode, _ptr(self.tickets), _stream()))


def awq_gemm_workspace(M, K, device="cuda"):
    n = kernels().kuiper_awq_gemm_workspace_bytes(M, K)
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def awq_gemm(x, qweight, qzeros, scales, y=None, residual=None, accumulate=False, group=128, workspace="auto"):
    """Tensor-core INT4 GEMM for M >= 16 rows: y = x . W (+ residual), or y += x . W.
    workspace: "auto" allocates the fp16 activation copy the kernel reads; a tensor is used as it is."""
    _dev(x, qweight, qzeros, scales)
    M, K = x.shape
    N = qweight.shape[1] * 8
    if y is None:
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    if isinstance(workspace, str):
        workspace = awq_gemm_workspace(M, K, x.device)
    check(kernels().kuiper_awq_gemm_f32(_ptr(x), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(y),
                                        _ptr(residual) if residual is not None else None, int(bool(accumulate)),
                                        M, K, N, group, _ptr(workspace) if workspace is not None else None,
                                        workspace.numel() if workspace is not None else 0, _stream()))
    return y


def awq_gemm_f16in(x16, qweight, qzeros, scales, y=None, residual=None, accumulate=False, group=128):
    """The tensor-core GEMM for activations that already are fp16 [M, K] (no conversion pass, no workspace)."""
    _dev(x16, qweight, qzeros, scales)
    M, K = x16.shape
    N = qweight.shape[1] * 8
    if y is None:
        y = torch.empty((M, N), dtype=torch.float32, device=x16.device)
    check(kernels().kuiper_awq_gemm_f16in_f32(_ptr(x16), _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(y),
                                              _ptr(residual) if residual is not None else None, int(bool(accumulate)),
                                              M, K, N, group, _stream()))
    return y


def awq_gemm_status() -> None:
    check(kernels().kuiper_awq_gemm_status())


def awq_gemv_status() -> None:
    check(kernels().kuiper_awq_gemv_status())


def bf16_gemv(x, W, out=None):
    _dev(x, W, out)
    M, K = x.shape
    N = W.shape[0]
    out = torch.empty((M, N), dtype=torch.float32, device=x.device) if out is None else out
    check(kernels().kuiper_bf16_gemv_f32(_ptr(x), _ptr(W), _ptr(out), M, K, N, _stream()))
    return out


def rmsnorm(x, w, eps=1e-6, out=None):
    _dev(x, w, out)
    M, H = x.shape
    out = torch.empty_like(x) if out is None else out
    check(kernels().kuiper_rmsnorm_f32(_ptr(x), _ptr(w), _ptr(out), M, H, eps, _stream()))
    return out


def rmsnorm_f16(x, w, eps=1e-6):
    """RMSNorm with the result rounded to fp16 (the tensor-core GEMM's activation type)."""
    _dev(x, w)
    M, H = x.shape
    out = torch.empty((M, H), dtype=torch.float16, device=x.device)
    check(kernels().kuiper_rmsnorm_f16(_ptr(x), _ptr(w), _ptr(out), M, H, eps, _stream()))
    return out


def swiglu_f16(gate_up, clear_input=False):
    """silu(gate) * up of gate_up = [M, 2 I], rounded to fp16 [M, I]."""
    _dev(gate_up)
    M, I2 = gate_up.shape
    out = torch.empty((M, I2 // 2), dtype=torch.float16, device=gate_up.device)
    check(kernels().kuiper_swiglu_f16(_ptr(gate_up), _ptr(out), M, I2 // 2, int(bool(clear_input)), _stream()))
    return out


def qknorm_rope_kvwrite(qkv, q_norm_w, k_norm_w, cos_t, sin_t, pos, slot, Nq, Nkv, D, eps, kcache, vcache, clear_input=False,
                        clear_extra=None):
    """kcache / vcache: [n_slots, Nkv, max_seq, D] bf16, updated in place; returns q [M, Nq, D].
    clear_extra: an fp32 tensor the kernel zeroes on the side."""
    _dev(qkv, q_norm_w, k_norm_w, cos_t, sin_t, pos, slot, kcache, vcache, clear_extra)
    M = qkv.shape[0]
    n_slots, _, max_seq, _ = kcache.shape
    q = torch.empty((M, Nq, D), dtype=torch.float32, device=qkv.device)
    check(kernels().kuiper_qknorm_rope_kvwrite(_ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_t), _ptr(sin_t),
                                               _ptr(pos), _ptr(slot), M, Nq, Nkv, D, eps, max_seq, n_slots,
                                               _ptr(q), _ptr(kcache), _ptr(vcache), int(clear_input),
                                               _ptr(clear_extra) if clear_extra is not None else None,
                                               clear_extra.numel() if clear_extra is not None else 0, _stream()))
    return q


def flash_decode_workspace(M, Nq, D, max_seq, device="cuda"):
    n = kernels().kuiper_flash_decode_workspace_bytes(M, Nq, D, max_seq)
    return torch.zeros(max(n, 16), dtype=torch.uint8, device=device)


def flash_decode(q, kcache, vcache, seq_len, slot, workspace=None, out=None, fresh_rows=-1):
    _dev(q, kcache, vcache, seq_len, slot, workspace, out)
    M, Nq, D = q.shape
    n_slots, Nkv, max_seq, _ = kcache.shape
    if workspace is None:
        workspace = flash_decode_workspace(M, Nq, D, max_seq, q.device)
    out = torch.empty_like(q) if out is None else out
    check(kernels().kuiper_flash_decode(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(seq_len), _ptr(slot), _ptr(out),
                                        M, Nq, Nkv, D, max_seq, n_slots, fresh_rows, _ptr(workspace), workspace.numel(),
                                        _stream()))
    return out


def flash_prefill(q, kcache, vcache, pos0, slot, out=None):
    """Causal attention of a prompt chunk: q [M, Nq, D], row m at position pos0 + m of sequence `slot` (rows already in
    the caches); returns [M, Nq, D]."""
    _dev(q, kcache, vcache, out)
    M, Nq, D = q.shape
    n_slots, Nkv, max_seq, _ = kcache.shape
    out = torch.empty_like(q) if out is None else out
    check(kernels().kuiper_flash_prefill(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(out), M, Nq, Nkv, D, max_seq, n_slots,
                                         int(pos0), int(slot), _stream()))
    return out


def rope_flash_decode(qkv, q_norm_w, k_norm_w, cos_t, sin_t, pos, seq_len, slot, Nq, Nkv, D, eps, kcache, vcache,
                      workspace=None, out=None, fresh_rows=-1, clear_input=False, clear_extra=None):
    """q/k-norm + rotary + KV append + flash-decoding in one kernel (decode batches: one row per sequence slot,
    seq_len == pos + 1); returns the attention output [M, Nq, D]."""
    _dev(qkv, q_norm_w, k_norm_w, cos_t, sin_t, pos, seq_len, slot, kcache, vcache, workspace, out, clear_extra)
    M = qkv.shape[0]
    n_slots, _, max_seq, _ = kcache.shape
    if workspace is None:
        workspace = flash_decode_workspace(M, Nq, D, max_seq, qkv.device)
    out = torch.empty((M, Nq, D), dtype=torch.float32, device=qkv.device) if out is None else out
    check(kernels().kuiper_rope_flash_decode(_ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos_t), _ptr(sin_t), _ptr(pos),
                                             _ptr(seq_len), _ptr(slot), _ptr(out), _ptr(kcache), _ptr(vcache), M, Nq, Nkv, D,
                                             eps, max_seq, n_slots, fresh_rows, int(clear_input),
                                             _ptr(clear_extra) if clear_extra is not None else None,
                                             clear_extra.numel() if clear_extra is not None else 0, _ptr(workspace),
                                             workspace.numel(), _stream()))
    return out


def allreduce_buffer(world, max_count, device="cuda"):
    n = kernels().kuiper_allreduce_buffer_bytes(world, max_count)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def allreduce_state(device="cuda"):
    return torch.zeros(kernels().kuiper_allreduce_state_bytes() // 4, dtype=torch.int32, device=device)


def _buffer_ptrs(rank_buffers, world):
    import ctypes
    return (ctypes.c_void_p * world)(*[b if isinstance(b, int) else b.data_ptr() for b in rank_buffers])


def allreduce_sum(partial, rank, world, rank_buffers, max_count, state, residual=None, out=None, clear_partial=False):
    """out = residual + sum over the ranks of `partial` (see kuiper_allreduce_sum_f32); rank_buffers: tensors or raw pointers."""
    _dev(partial, state, residual, out)
    out = torch.empty_like(partial) if out is None else out
    check(kernels().kuiper_allreduce_sum_f32(_ptr(partial), _ptr(residual), _ptr(out), int(clear_partial), partial.numel(), rank, world,
                                             _buffer_ptrs(rank_buffers, world), max_count, _ptr(state), _stream()))
    return out


def argmax_allgather(logits_local, rank, world, rank_buffers, max_count, state):
    """Greedy ids over a vocabulary split across ranks; logits_local: this rank's [M, V_local] slice."""
    _dev(logits_local, state)
    M, V_local = logits_local.shape
    out = torch.empty(M, dtype=torch.int32, device=logits_local.device)
    check(kernels().kuiper_argmax_allgather(_ptr(logits_local), _ptr(out), M, V_local, rank, world, _buffer_ptrs(rank_buffers, world),
                                            max_count, _ptr(state), _stream()))
    return out


def allreduce_status(state, clear=False) -> None:
    check(kernels().kuiper_allreduce_status(_ptr(state), int(clear)))


def swiglu(gate_up, out=None, clear_input=False):
    _dev(gate_up, out)
    M, I2 = gate_up.shape
    out = torch.empty((M, I2 // 2), dtype=torch.float32, device=gate_up.device) if out is None else out
    check(kernels().kuiper_swiglu_f32(_ptr(gate_up), _ptr(out), M, I2 // 2, int(clear_input), _stream()))
    return out


def embedding(tokens, table, out=None):
    _dev(tokens, table, out)
    V, H = table.shape
    M = tokens.numel()
    out = torch.empty((M, H), dtype=torch.float32, device=table.device) if out is None else out
    check(kernels().kuiper_embedding_bf16(_ptr(tokens), _ptr(table), _ptr(out), M, H, V, _stream()))
    return out


def argmax(logits, out=None):
    _dev(logits, out)
    M, V = logits.shape
    out = torch.empty(M, dtype=torch.int32, device=logits.device) if out is None else out
    check(kernels().kuiper_argmax_f32(_ptr(logits), _ptr(out), M, V, _stream()))
    return out
