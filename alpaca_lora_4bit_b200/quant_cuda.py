"""Drop-in for the reference's ``quant_cuda`` extension module (quant_cuda.cpp:204-227).

Same function names, same argument order, same in-place convention: every function returns
``None`` and writes into a caller-allocated tensor; the ``*matmul*`` functions ADD into ``mul``
(the reference kernels ``atomicAdd`` into a pre-zeroed buffer, quant_cuda_kernel.cu:535,974,1040).
Unlike the reference, arguments are validated and launches go to torch's current stream.

The four live decode entry points and the three reconstruct entry points run on the sm_100a
kernels of ``libq4b200.so``.  The reference's 2/3/8-bit GEMVs and ``seq_v2`` are exported by its
binding but never called from its Python code; they raise ``NotImplementedError`` here.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = [
    "vecquant2matmul", "vecquant3matmul", "vecquant4matmul", "vecquant8matmul",
    "vecquant2matmul_faster", "vecquant3matmul_faster", "vecquant4matmul_faster",
    "vecquant4matmul_old_faster", "vecquant4matmul_v1_faster", "vecquant4recons_v1",
    "vecquant4recons_v2", "vecquant2recons_v2", "vecquant4matmul_seq_v2", "vecquant4matmul_g",
]


def _check_int32(t, name):
    if t.dtype != torch.int32:
        raise RuntimeError(f"quant_cuda: {name} must be int32, got {t.dtype}")


def vecquant4recons_v2(mat, res, scales, zeros, g_idx) -> None:
    """``res[K,N] = dequant(mat)``; dtype of ``res`` and ``scales`` half or float (quant_cuda.cpp:143-148)."""
    dev = _lib.require_cuda(mat, res, scales, zeros, g_idx)
    _check_int32(mat, "mat"); _check_int32(zeros, "zeros"); _check_int32(g_idx, "g_idx")
    R, N = mat.shape
    K = R * 8
    if res.shape != (K, N) or res.dtype != scales.dtype:
        raise RuntimeError(f"quant_cuda: res must be [{K},{N}] of {scales.dtype}")
    G = scales.shape[0]
    if scales.shape != (G, N) or zeros.shape != (G, N // 8) or g_idx.numel() < K:
        raise RuntimeError("quant_cuda: scales/zeros/g_idx shapes do not match mat")
    with _lib.on_device(dev):
        _lib.check(_lib.lib().q4_recons_v2(mat.data_ptr(), res.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                           g_idx.data_ptr(), K, N, G, _lib.dtype_code(scales.dtype),
                                           _lib.stream_of(mat)), "recons_v2")


def vecquant4recons_v1(mat, res, scales, zeros) -> None:
    """v1 layers: per-column float scale and zero (quant_cuda.cpp:129-135)."""
    dev = _lib.require_cuda(mat, res, scales, zeros)
    _check_int32(mat, "mat")
    R, N = mat.shape
    K = R * 8
    if res.shape != (K, N) or res.dtype != scales.dtype or zeros.dtype != scales.dtype:
        raise RuntimeError(f"quant_cuda: res must be [{K},{N}] and share the dtype of scales and zeros")
    if scales.numel() != N or zeros.numel() != N:
        raise RuntimeError("quant_cuda: v1 scales and zeros hold one value per column")
    with _lib.on_device(dev):
        _lib.check(_lib.lib().q4_recons_v1(mat.data_ptr(), res.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                           K, N, _lib.dtype_code(scales.dtype), _lib.stream_of(mat)), "recons_v1")


def vecquant2recons_v2(mat, res, scales, zeros, g_idx) -> None:
    """2-bit layers, 16 levels per word (quant_cuda.cpp:156-161)."""
    dev = _lib.require_cuda(mat, res, scales, zeros, g_idx)
    _check_int32(mat, "mat"); _check_int32(zeros, "zeros"); _check_int32(g_idx, "g_idx")
    R, N = mat.shape
    K = R * 16
    G = scales.shape[0]
    if res.shape != (K, N) or res.dtype != scales.dtype:
        raise RuntimeError(f"quant_cuda: res must be [{K},{N}] of {scales.dtype}")
    if scales.shape != (G, N) or zeros.shape != (G, N // 16) or g_idx.numel() < K:
        raise RuntimeError("quant_cuda: scales/zeros/g_idx shapes do not match mat")
    with _lib.on_device(dev):
        _lib.check(_lib.lib().q2_recons_v2(mat.data_ptr(), res.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                           g_idx.data_ptr(), K, N, G, _lib.dtype_code(scales.dtype),
                                           _lib.stream_of(mat)), "recons2_v2")


def gemv(x, qweight, y, scales, zeros, g_idx, groupsize, flags, bias=None) -> None:
    """``y (+)= x @ W`` through ``q4_gemv`` in slabs of at most 16 rows; x, scales fp16.

    This is the per-token path of decode, so the host side is kept short: one stream lookup, one
    cached workspace, one foreign call (shape and pointer checks happen inside the library)."""
    if not (x.is_cuda and x.is_contiguous() and y.is_contiguous() and qweight.is_cuda and scales.is_contiguous()):
        _lib.require_cuda(x, qweight, y, scales, zeros, g_idx, bias)
        raise RuntimeError("quant_cuda: gemv tensors must be contiguous CUDA tensors")
    M, K = x.shape
    N = qweight.shape[1]
    if qweight.shape[0] * 8 != K or y.shape[0] != M or y.shape[1] != N or x.dtype != torch.float16 or scales.dtype != torch.float16:
        raise RuntimeError(f"quant_cuda: shapes x{tuple(x.shape)} mat{tuple(qweight.shape)} mul{tuple(y.shape)} disagree "
                           f"or x / scales are not fp16")
    G = 1 if (flags & _lib.GEMV_V1) else scales.shape[0]
    dev = x.device
    st = torch.cuda.current_stream(dev).cuda_stream
    ws = _lib.workspace_for(dev, st)
    ydt = _lib.Q4_F16 if y.dtype == torch.float16 else _lib.Q4_F32 if y.dtype == torch.float32 else _lib.dtype_code(y.dtype)
    fn = _lib.lib().q4_gemv
    gp = None if g_idx is None else g_idx.data_ptr()
    bp = None if bias is None else bias.data_ptr()
    with _lib.on_device(dev):
        if M <= 16:
            rc = fn(x.data_ptr(), qweight.data_ptr(), y.data_ptr(), scales.data_ptr(), zeros.data_ptr(), gp, bp,
                    M, K, N, G, groupsize, ydt, flags, ws.data_ptr(), ws.numel(), st)
            if rc:
                _lib.check(rc, "gemv")
            return
        row_x, row_y = K * x.element_size(), N * y.element_size()
        for m0 in range(0, M, 16):
            rc = fn(x.data_ptr() + m0 * row_x, qweight.data_ptr(), y.data_ptr() + m0 * row_y, scales.data_ptr(),
                    zeros.data_ptr(), gp, bp, min(16, M - m0), K, N, G, groupsize, ydt, flags, ws.data_ptr(), ws.numel(), st)
            if rc:
                _lib.check(rc, "gemv")


_decode_ws: dict = {}          # (device index, stream handle) -> (pointer, bytes, tensor)

try:                                                      # the handle of the current stream without building a Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:                                    # pragma: no cover - older / newer torch without the private hook
    def _raw_stream(idx):
        return torch.cuda.current_stream(idx).cuda_stream


class _LayerPlan:
    """What the per-token call needs of one layer, looked up by the identity of its ``qweight``."""
    __slots__ = ("handle", "qref", "scales", "zeros", "qptr", "sptr", "zptr", "K", "N", "index", "device", "gs_arg")


_plans: dict = {}              # id(qweight) -> _LayerPlan; the entry dies with the qweight tensor
_F16 = torch.float16
try:
    _current_device = torch._C._cuda_getDevice
except AttributeError:                                    # pragma: no cover
    _current_device = torch.cuda.current_device


_layer_gemv = None             # the per-token foreign call, resolved on first use


def _bind_layer_gemv():
    global _layer_gemv
    _layer_gemv = _lib.layer_gemv_call()
    return _layer_gemv


def _drop_plan(key):
    p = _plans.pop(key, None)
    if p is not None and p.handle:
        _lib.lib().q4_layer_destroy(p.handle)
        p.handle = None


def _make_plan(qweight, scales, zeros, K, N, G, groupsize, gs_arg):
    import ctypes
    import weakref
    h = ctypes.c_void_p()
    _lib.check(_lib.lib().q4_layer_create(ctypes.byref(h), qweight.data_ptr(), scales.data_ptr(), zeros.data_ptr(), K, N, G, groupsize),
               "layer_create")
    p = _LayerPlan()
    key = id(qweight)
    p.handle = h.value
    p.qref = weakref.ref(qweight, lambda _r, key=key: _drop_plan(key))
    p.scales, p.zeros = scales, zeros
    p.qptr, p.sptr, p.zptr = qweight.data_ptr(), scales.data_ptr(), zeros.data_ptr()
    p.K, p.N, p.index, p.device, p.gs_arg = K, N, qweight.device.index, qweight.device, gs_arg
    _drop_plan(key)
    _plans[key] = p


def decode_planned(x, qweight, scales, zeros, groupsize, max_rows):
    """The per-token call for a layer ``decode_v2`` has seen before: ``x @ W`` in a new fp16 tensor, or
    ``None`` when this call is not one the recorded plan covers (the caller then takes the general path).

    A plan is valid for exactly the tensors it was made from: same objects, same storage addresses.
    What is checked per call is what can differ between calls - ``x``, the current device, the
    stream - so that a repeated call costs a dictionary lookup, one allocation and one foreign call
    with seven arguments."""
    p = _plans.get(id(qweight))
    if p is None or p.scales is not scales or p.zeros is not zeros or p.gs_arg != groupsize or p.qref() is not qweight:
        return None
    if x.dtype is not _F16 or x.dim() != 2 or not x.is_contiguous() or x.device != p.device or _current_device() != p.index:
        return None
    M, K = x.shape
    if K != p.K or M < 1 or M > max_rows:
        return None
    if qweight.data_ptr() != p.qptr or scales.data_ptr() != p.sptr or zeros.data_ptr() != p.zptr:
        _drop_plan(id(qweight))                              # storage moved under the same tensor objects
        return None
    y = x.new_empty((M, p.N))
    st = _raw_stream(p.index)
    w = _decode_ws.get((p.index, st))
    if w is None:
        t = _lib.workspace_for(p.device, st)
        w = _decode_ws[(p.index, st)] = (t.data_ptr(), t.numel(), t)
    rc = (_layer_gemv or _bind_layer_gemv())(p.handle, x.data_ptr(), y.data_ptr(), M, w[0], w[1], st)
    if rc:
        _lib.check(rc, "layer_gemv")
    return y


def decode_v2(x, qweight, scales, zeros, groupsize, plan_key=None):
    """``x @ W`` for at most 16 rows on a v2 layer with sequential groups, result in a new fp16 tensor.

    The per-token call of generation: the caller (``matmul_utils_4bit.matmul4bit``) has already
    established that ``x`` is a contiguous 2-D fp16 CUDA tensor and ``scales`` fp16, so what is left
    here is what protects memory - the shapes must describe one layer - and the foreign call.
    With ``plan_key`` (the caller's own ``groupsize`` argument) the validated layer is recorded for
    ``decode_planned``."""
    M, K = x.shape
    R, N = qweight.shape
    G = scales.shape[0]
    if R * 8 != K or scales.shape[1] != N or zeros.shape[0] != G or zeros.shape[1] * 8 != N or M > 16:
        raise RuntimeError(f"quant_cuda: shapes x{tuple(x.shape)} mat{tuple(qweight.shape)} scales{tuple(scales.shape)} "
                           f"zeros{tuple(zeros.shape)} do not describe one layer")
    dev = x.device
    idx = dev.index
    if idx != torch.cuda.current_device() or not (qweight.is_contiguous() and scales.is_contiguous() and zeros.is_contiguous()):
        y = torch.empty((M, N), dtype=torch.float16, device=dev)
        gemv(x, qweight.contiguous(), y, scales.contiguous(), zeros.contiguous(), None, groupsize, 0)
        return y
    y = torch.empty((M, N), dtype=torch.float16, device=dev)
    st = _raw_stream(idx)
    w = _decode_ws.get((idx, st))
    if w is None:
        t = _lib.workspace_for(dev, st)
        w = _decode_ws[(idx, st)] = (t.data_ptr(), t.numel(), t)
    rc = _lib.lib().q4_gemv(x.data_ptr(), qweight.data_ptr(), y.data_ptr(), scales.data_ptr(), zeros.data_ptr(), None, None,
                            M, K, N, G, groupsize, _lib.Q4_F16, 0, w[0], w[1], st)
    if rc:
        _lib.check(rc, "gemv")
    if plan_key is not None and qweight.device == dev and scales.device == dev and zeros.device == dev and zeros.dtype == torch.int32:
        _make_plan(qweight, scales, zeros, K, N, G, groupsize, plan_key)
    return y


_gemm_ws_bytes: dict = {}


_seq_cache: dict = {}        # id(g_idx) -> (weak reference, storage address, version counter, answer)


def groups_are_sequential(g_idx, groups: int) -> bool:
    """True when ``g_idx[k] == k // (K / groups)`` for every row, i.e. the layer was quantised without
    act-order and its groups can be derived from the row index.  One comparison per tensor (it synchronises the
    device), remembered for as long as the tensor lives and is not written to; during a stream capture a tensor
    that has not been looked at yet counts as not sequential."""
    import weakref
    key = id(g_idx)
    hit = _seq_cache.get(key)
    if hit is not None and hit[0]() is g_idx and hit[1] == g_idx.data_ptr() and hit[2] == g_idx._version:
        return hit[3]
    if g_idx.is_cuda and torch.cuda.is_current_stream_capturing():
        return False
    K = g_idx.numel()
    ok = groups > 0 and K % groups == 0
    if ok:
        want = torch.arange(K, device=g_idx.device, dtype=torch.int64) // (K // groups)
        ok = bool(torch.equal(g_idx.reshape(-1).to(torch.int64), want))
    _seq_cache[key] = (weakref.ref(g_idx, lambda _r, key=key: _seq_cache.pop(key, None)), g_idx.data_ptr(), g_idx._version, ok)
    return ok


# Zero terms rn(scale * (zero + 1)) [G, N] of the layers whose backward has run, keyed by the identity of the
# packed zero-point tensor and dropped with it: the table depends on the frozen layer only, a finetune step runs
# every layer's backward once per step, and deriving it ahead of every call is a kernel launch per call
# (2 G N bytes per layer are kept instead, 1.6 % of the packed weights).  ``cache_zero_terms = False`` restores
# the derivation per call.
cache_zero_terms = True
promise_sequential_groups = True     # forward: tell the kernel that group = row / groupsize where that was checked
_zero_term_tables: dict = {}


def _zero_terms(scales, zeros, G, N, st):
    key = id(zeros)
    hit = _zero_term_tables.get(key)
    if hit is not None and hit[1] == (zeros.data_ptr(), scales.data_ptr(), zeros._version, scales._version):
        return hit[0]
    if torch.cuda.is_current_stream_capturing():
        return None                                    # no allocation inside a capture: this call derives the table itself
    import weakref
    table = torch.empty((G, N), dtype=torch.float16, device=scales.device)
    _lib.check(_lib.lib().q4_zero_term_table(scales.data_ptr(), zeros.data_ptr(), table.data_ptr(), G, N, st), "zero_term_table")
    ref = weakref.ref(zeros, lambda _r, key=key: _zero_term_tables.pop(key, None))
    _zero_term_tables[key] = (table, (zeros.data_ptr(), scales.data_ptr(), zeros._version, scales._version), ref)
    return table


def gemm(x, qweight, out, scales, zeros, g_idx, transpose=False, bias=None, lora_u=None, lora_w=None, residual=None) -> None:
    """Fused large-M product on the tensor cores: ``out = x @ W (+ bias)`` or, with ``transpose``,
    ``out = x @ W.T``; ``x``, ``out``, ``scales`` fp16, W never leaves shared memory.

    ``lora_u`` fp16 ``[M, 64]`` (columns beyond the rank zero) with ``lora_w`` adds the low-rank term in
    the same kernel: forward ``+ lora_u[:, :r] @ lora_w.T`` with ``lora_w = lora_B [N, r]``; transpose
    ``+ lora_u[:, :r] @ lora_w`` with ``lora_w = lora_A [r, K]``.  ``residual`` fp16 ``[M, N]`` (forward only) is
    added to the rounded product in the epilogue: ``out = half(half(x @ W + bias) + residual)``."""
    dev = _lib.require_cuda(x, qweight, out, scales, zeros, g_idx, bias, lora_u, lora_w, residual)
    R, N = qweight.shape
    K = R * 8
    M = x.shape[0]
    G = scales.shape[0]
    inner, outer = (N, K) if transpose else (K, N)
    if residual is not None and (transpose or residual.shape != (M, N) or residual.dtype != torch.float16 or not residual.is_contiguous()):
        raise RuntimeError("quant_cuda: gemm takes a contiguous fp16 residual [M, N] with the forward product only")
    if x.shape != (M, inner) or out.shape != (M, outer):
        raise RuntimeError(f"quant_cuda: gemm shapes x{tuple(x.shape)} out{tuple(out.shape)} do not match the layer [{K},{N}]")
    if x.dtype != torch.float16 or out.dtype != torch.float16 or scales.dtype != torch.float16:
        raise RuntimeError("quant_cuda: gemm takes fp16 x, out and scales")
    r = 0
    if lora_u is not None:
        r = lora_w.shape[0] if transpose else lora_w.shape[1]
        want_w = (r, K) if transpose else (N, r)
        if lora_u.shape != (M, 64) or lora_w.shape != want_w or lora_u.dtype != torch.float16 or lora_w.dtype != torch.float16:
            raise RuntimeError(f"quant_cuda: gemm low-rank term needs lora_u [M,64] and lora_w {want_w}, both fp16")
    L = _lib.lib()
    with _lib.on_device(dev):
        st = _lib.stream_of(x)
        need = _gemm_ws_bytes.get((K, N, G))
        if need is None:
            need = _gemm_ws_bytes[(K, N, G)] = int(L.q4_gemm_workspace_bytes(K, N, G))
        ws = _lib.gemm_workspace_for(dev, st, need)
        if transpose:
            zt = _zero_terms(scales, zeros, G, N, st) if cache_zero_terms else None
            if zt is not None:
                rc = L.q4_gemm_bwd_table(x.data_ptr(), qweight.data_ptr(), out.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                         zt.data_ptr(), g_idx.data_ptr(), _lib.ptr(lora_u), _lib.ptr(lora_w), r, M, K, N, G,
                                         ws.data_ptr(), ws.numel(), st)
            else:
                rc = L.q4_gemm_bwd(x.data_ptr(), qweight.data_ptr(), out.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                   g_idx.data_ptr(), _lib.ptr(lora_u), _lib.ptr(lora_w), r, M, K, N, G, ws.data_ptr(), ws.numel(), st)
        else:
            # Sequential groups (checked once per layer): the kernel is given the kept table of zero terms and the word
            # that group = row / groupsize, so that it fetches a task's scales and zero terms ahead with its packed
            # words instead of building shared-memory tables of all groups per tile.  (With act-order every row of a
            # task would need its own pair of loads: measured slower, so the table is not offered.)
            zt, seq_gs = None, 0
            if cache_zero_terms and N % 256 == 0 and K % G == 0 and groups_are_sequential(g_idx, G):
                zt = _zero_terms(scales, zeros, G, N, st)
                seq_gs = K // G if (zt is not None and promise_sequential_groups) else 0
            if zt is not None or residual is not None:
                rc = L.q4_gemm_fwd_residual(x.data_ptr(), qweight.data_ptr(), out.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                            _lib.ptr(zt), g_idx.data_ptr(), _lib.ptr(bias), _lib.ptr(residual), _lib.ptr(lora_u),
                                            _lib.ptr(lora_w), r, M, K, N, G, seq_gs, ws.data_ptr(), ws.numel(), st)
            else:
                rc = L.q4_gemm_fwd(x.data_ptr(), qweight.data_ptr(), out.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                   g_idx.data_ptr(), _lib.ptr(bias), _lib.ptr(lora_u), _lib.ptr(lora_w), r, M, K, N, G,
                                   ws.data_ptr(), ws.numel(), st)
    _lib.check(rc, "gemm")


def gemm_swiglu(x, qweight, out, scales, zeros, g_idx, bias=None) -> None:
    """``out [M, I] = half(silu(half(x @ W_gate))) * half(x @ W_up)`` for a fused ``[K, 2 I]`` gate/up layer in one
    kernel (the SwiGLU product in the GEMM epilogue): what ``gemm`` followed by the element-wise kernel computes,
    without the ``[M, 2 I]`` tensor.  Raises for layers the CTA-pair kernel does not take (``gemm_swiglu_supported``)."""
    dev = _lib.require_cuda(x, qweight, out, scales, zeros, g_idx, bias)
    R, N = qweight.shape
    K, M, G = R * 8, x.shape[0], scales.shape[0]
    if x.shape != (M, K) or out.shape != (M, N // 2):
        raise RuntimeError(f"quant_cuda: gemm_swiglu shapes x{tuple(x.shape)} out{tuple(out.shape)} do not match the layer [{K},{N}]")
    if x.dtype != torch.float16 or out.dtype != torch.float16 or scales.dtype != torch.float16:
        raise RuntimeError("quant_cuda: gemm_swiglu takes fp16 x, out and scales")
    L = _lib.lib()
    with _lib.on_device(dev):
        st = _lib.stream_of(x)
        need = _gemm_ws_bytes.get((K, N, G))
        if need is None:
            need = _gemm_ws_bytes[(K, N, G)] = int(L.q4_gemm_workspace_bytes(K, N, G))
        ws = _lib.gemm_workspace_for(dev, st, need)
        zt, seq_gs = None, 0                    # sequential groups: kept zero-term table and the promise, as in gemm()
        if cache_zero_terms and K % G == 0 and groups_are_sequential(g_idx, G):
            zt = _zero_terms(scales, zeros, G, N, st)
            seq_gs = K // G if (zt is not None and promise_sequential_groups) else 0
        rc = L.q4_gemm_fwd_swiglu(x.data_ptr(), qweight.data_ptr(), out.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                                  _lib.ptr(zt), g_idx.data_ptr(), _lib.ptr(bias), M, K, N, G, seq_gs, ws.data_ptr(), ws.numel(), st)
    _lib.check(rc, "gemm_swiglu")


def gemm_swiglu_supported(K: int, N: int, G: int) -> bool:
    """Layers ``gemm_swiglu`` takes: K % 128 == 0, N % 256 == 0 and scale tables that leave the pair kernel three stages."""
    return K % 128 == 0 and N % 256 == 0 and (1024 + 3 * 32768 + 512 + 2 * G * 128 * 2) <= 227 * 1024


def gemm_supported(K: int, N: int, G: int, transpose: bool) -> bool:
    """Shapes the fused kernels take: K, N multiples of 128; forward scale tables must fit shared memory."""
    if K % 128 or N % 128:
        return False
    return transpose or (1024 + 2 * 49152 + 256 + 2 * G * 128 * 2) <= 227 * 1024


def gemm_set_variant(variant: int) -> None:
    """Which fused GEMM kernel ``gemm`` launches: 0 = chosen per shape (default), 1 = single-CTA kernel,
    2 / 3 = CTA-pair kernel with 256- / 512-row tiles (output columns must be a multiple of 256), 4 = the forward
    kernel with the dequantised weights in tensor memory (sequential groups promised, zero-term table kept),
    5 = chosen per shape among 1-3."""
    _lib.check(_lib.lib().q4_gemm_set_variant(int(variant)), "gemm_set_variant")


def gemv_set_variant(variant: int) -> None:
    """Form of the sequential-group decode kernel, a sum of: bits 0-1 how it gets x (0 = chosen per shape,
    the default; 1 = every unit brings its own slice; 2 = every CTA re-lays the whole of x out once where it
    fits shared memory); 4 = always deal an even share of all units (straddled column tiles meet in the
    workspace); 8 = one-row products in the one-CTA-per-SM form; 32 / 64 = one-row products with 10 / 8 warps
    per CTA in the two-per-SM form."""
    _lib.check(_lib.lib().q4_gemv_set_variant(int(variant)), "gemv_set_variant")


def device_status() -> int:
    """Status of every kernel family on the current device (synchronises): 0 unless a bounded device-side
    wait expired in a fused GEMM kernel (one word per device) or in a decode kernel (one word per decode
    workspace, i.e. per stream that has run a decode product, plus the built-in scratch of
    ``q4_gemv_static``).  A non-zero decode word means the workspace head must be cleared before reuse;
    this function does that for the workspaces this module owns."""
    import ctypes
    L = _lib.lib()
    v = ctypes.c_uint(0)
    _lib.check(L.q4_device_status(ctypes.byref(v)), "device_status")
    status = v.value
    cur = torch.cuda.current_device()
    for (index, _stream), ws in list(_lib._workspaces.items()):
        if index != cur:
            continue
        _lib.check(L.q4_gemv_status(ws.data_ptr(), ws.numel(), ctypes.byref(v)), "gemv_status")
        if v.value:
            ws[:131072].zero_()
            status = status or v.value
    _lib.check(L.q4_gemv_static_status(ctypes.byref(v)), "gemv_static_status")
    return status or v.value


def _half(t):
    return t if t.dtype == torch.float16 else t.half()


def vecquant4matmul(vec, mat, mul, scales, zeros, g_idx) -> None:
    """``mul += vec @ W`` with the group of every row taken from ``g_idx`` (quant_cuda.cpp:41-48).

    The reference computes in the dtype of ``vec`` (float); here activations and scales are
    rounded to fp16 on entry and the sum is kept in fp32.
    """
    _check_int32(mat, "mat"); _check_int32(zeros, "zeros"); _check_int32(g_idx, "g_idx")
    if mul.dtype != vec.dtype:
        raise RuntimeError("quant_cuda: vec and mul must share a dtype")
    K = vec.shape[-1]
    G = scales.shape[0]
    gemv(_half(vec).contiguous(), mat, mul, _half(scales), zeros, g_idx, max(K // G, 1),
         _lib.GEMV_ACCUMULATE | _lib.GEMV_ACT_ORDER)


def vecquant4matmul_g(vec, mat, mul, scales, zeros, g_idx, vec_height=None) -> None:
    """Act-order half GEMV (quant_cuda.cpp:195-202)."""
    vecquant4matmul(vec, mat, mul, scales, zeros, g_idx)


def vecquant4matmul_faster(vec, mat, mul, scales, zeros, g_idx, vec_height=None) -> None:
    """Half GEMV, group from ``g_idx`` (quant_cuda.cpp:101-108); ``mul`` fp16."""
    if vec.dtype != torch.float16 or mul.dtype != torch.float16:
        raise RuntimeError("quant_cuda: vecquant4matmul_faster takes half vec and mul")
    vecquant4matmul(vec, mat, mul, scales, zeros, g_idx)


def vecquant4matmul_old_faster(vec, mat, mul, scales, zeros, groupsize, vec_height=None) -> None:
    """Half-in / float-out GEMV with sequential groups ``k // groupsize`` (quant_cuda.cpp:116-123)."""
    _check_int32(mat, "mat"); _check_int32(zeros, "zeros")
    if vec.dtype != torch.float16 or mul.dtype != torch.float32:
        raise RuntimeError("quant_cuda: vecquant4matmul_old_faster takes half vec and float mul")
    gemv(vec.contiguous(), mat, mul, _half(scales), zeros, None, int(groupsize), _lib.GEMV_ACCUMULATE)


def vecquant4matmul_v1_faster(vec, mat, mul, scales, zeros) -> None:
    """v1-format half GEMV: ``mul += vec @ (scales[n]*q - zeros[n])`` (quant_cuda.cpp:168-174)."""
    _check_int32(mat, "mat")
    if vec.dtype != torch.float16 or mul.dtype != torch.float16:
        raise RuntimeError("quant_cuda: vecquant4matmul_v1_faster takes half vec and mul")
    K = vec.shape[-1]
    gemv(vec.contiguous(), mat, mul, _half(scales).reshape(-1).contiguous(), _half(zeros).reshape(-1).contiguous(),
         None, K, _lib.GEMV_ACCUMULATE | _lib.GEMV_V1)


def _dead(name):
    def f(*args, **kwargs):
        raise NotImplementedError(
            f"quant_cuda.{name}: exported by the reference binding but never called from its Python "
            f"code; not provided by the sm_100a library")
    f.__name__ = name
    return f


vecquant2matmul = _dead("vecquant2matmul")
vecquant3matmul = _dead("vecquant3matmul")
vecquant8matmul = _dead("vecquant8matmul")
vecquant2matmul_faster = _dead("vecquant2matmul_faster")
vecquant3matmul_faster = _dead("vecquant3matmul_faster")
vecquant4matmul_seq_v2 = _dead("vecquant4matmul_seq_v2")
