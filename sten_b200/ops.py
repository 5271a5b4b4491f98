"""Tensor-level entry points: torch tensors in, one C-ABI call, torch tensors out.

torch is used for device memory (caching allocator), the current stream and nothing else; all arithmetic
happens inside ``libnmg_b200.so``.
"""
import functools
import math

import torch

from . import _native as nat

_DTYPES = {torch.float32: nat.NMG_F32, torch.float16: nat.NMG_F16, torch.bfloat16: nat.NMG_BF16}


def _dtype_code(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"grouped n:m kernels support float32, float16 and bfloat16, got {t.dtype}") from None


def _require_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "grouped n:m kernels run on CUDA devices only (there is no CPU fallback); move the tensor with .cuda()")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"operands live on different devices: {dev} and {t.device}")
    return dev


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(dev):
    """Handle of the current stream of ``dev`` (the raw query is several times cheaper than building a Stream object)."""
    if _raw_stream is not None and dev.index is not None:
        return _raw_stream(dev.index)
    return torch.cuda.current_stream(dev).cuda_stream


class _on_device:
    """``torch.cuda.device(dev)`` only when ``dev`` is not already current: the common case costs one integer compare."""

    __slots__ = ("ctx",)

    def __init__(self, dev):
        self.ctx = None if dev.index is None or torch.cuda.current_device() == dev.index else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


def _workspace(nbytes, dev):
    if nbytes == 0:
        return None, 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    return ws, nbytes


def geometry(M, K, n, m, g):
    C = math.comb(m, n)
    cc = C * g
    nb, nc = -(-M // m), -(-K // cc)
    return C, cc, nb, nc


def sparsify(dense3, n, m, g):
    """dense3: [B, M, K] view with unit stride along K.  Returns (val [T, C, g, n], idx [T, C, g, 1])."""
    assert dense3.dim() == 3
    dev = _require_cuda(dense3)
    code = _dtype_code(dense3)
    B, M, K = dense3.shape
    if dense3.stride(2) != 1 or dense3.stride(1) < K or (B > 1 and dense3.stride(0) < M * dense3.stride(1)):
        dense3 = dense3.contiguous()
    # size-1 dims may carry arbitrary strides even in a contiguous tensor: state the packed strides then
    ld, bs = (K, M * K) if dense3.is_contiguous() else (dense3.stride(1), dense3.stride(0))
    C, cc, nb, nc = geometry(M, K, n, m, g)
    T = B * nc * nb
    val = torch.empty((T, C, g, n), dtype=dense3.dtype, device=dev)
    idx = torch.empty((T, C, g, 1), dtype=torch.int16, device=dev)
    with torch.cuda.device(dev):
        nat.check(nat.lib().nmg_sparsify(dense3.data_ptr(), B, M, K, ld, bs, n, m, g, code,
                                         val.data_ptr(), idx.data_ptr(), _stream(dev)))
    return val, idx


def gather_layout(dense3, idx, n, m, g):
    """Values of dense3 [B, M, K] at the positions the layout ``idx`` keeps: val [T, C, g, n] of dense3's dtype."""
    assert dense3.dim() == 3
    dev = _require_cuda(dense3, idx)
    code = _dtype_code(dense3)
    B, M, K = dense3.shape
    if dense3.stride(2) != 1 or dense3.stride(1) < K or (B > 1 and dense3.stride(0) < M * dense3.stride(1)):
        dense3 = dense3.contiguous()
    ld, bs = (K, M * K) if dense3.is_contiguous() else (dense3.stride(1), dense3.stride(0))
    C, cc, nb, nc = geometry(M, K, n, m, g)
    idx = idx.contiguous()
    if idx.numel() != B * nc * nb * cc:
        raise ValueError("idx does not belong to a layout of this shape")
    val = torch.empty((B * nc * nb, C, g, n), dtype=dense3.dtype, device=dev)
    with torch.cuda.device(dev):
        nat.check(nat.lib().nmg_gather(dense3.data_ptr(), idx.data_ptr(), B, M, K, ld, bs, n, m, g, code, val.data_ptr(), _stream(dev)))
    return val


def densify(val, idx, B, M, K, n, m, g):
    """Returns the dense [B, M, K] tensor of a (val, idx) pair."""
    dev = _require_cuda(val, idx)
    code = _dtype_code(val)
    val, idx = val.contiguous(), idx.contiguous()
    out = torch.empty((B, M, K), dtype=val.dtype, device=dev)
    with torch.cuda.device(dev):
        nat.check(nat.lib().nmg_densify(val.data_ptr(), idx.data_ptr(), B, M, K, n, m, g, code, out.data_ptr(), K,
                                        M * K, _stream(dev)))
    return out


def perfect_nm_select(dense, n, m, sparse_dim):
    """Top-n of every block of m along ``sparse_dim``: (val, idx) of shape [..., blocks, n, ...], idx int64."""
    dev = _require_cuda(dense)
    code = _dtype_code(dense)
    dense = dense.contiguous()
    shape = list(dense.shape)
    size = shape[sparse_dim]
    outer, inner = math.prod(shape[:sparse_dim]), math.prod(shape[sparse_dim + 1:])
    blocks = -(-size // m)
    out_shape = shape[:sparse_dim] + [blocks, n] + shape[sparse_dim + 1:]
    val = torch.empty(out_shape, dtype=dense.dtype, device=dev)
    idx = torch.empty(out_shape, dtype=torch.int64, device=dev)
    if val.numel():
        with torch.cuda.device(dev):
            nat.check(nat.lib().nmg_perfect_nm_select(dense.data_ptr(), outer, size, inner, n, m, code, val.data_ptr(), idx.data_ptr(),
                                                      _stream(dev)))
    return val, idx


def perfect_nm_densify(val, idx, n, m, sparse_dim, size):
    """Inverse of perfect_nm_select: the dense tensor with ``size`` elements along ``sparse_dim``."""
    dev = _require_cuda(val, idx)
    code = _dtype_code(val)
    val, idx = val.contiguous(), idx.contiguous()
    shape = list(val.shape)
    outer, inner = math.prod(shape[:sparse_dim]), math.prod(shape[sparse_dim + 2:])
    dense = torch.empty(shape[:sparse_dim] + [size] + shape[sparse_dim + 2:], dtype=val.dtype, device=dev)
    if dense.numel():
        with torch.cuda.device(dev):
            nat.check(nat.lib().nmg_perfect_nm_densify(val.data_ptr(), idx.data_ptr(), outer, size, inner, n, m, code, dense.data_ptr(),
                                                       _stream(dev)))
    return dense


def _row_major_2d(t):
    """(tensor, leading dimension) of a 2-D operand with unit stride along its rows."""
    if t.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        t = t.contiguous()
    return t, (t.shape[1] if t.is_contiguous() else t.stride(0))


def pack(val, idx, M, K, n, m, g):
    """Column-ordered device copy of a weight (opaque uint8 buffer) for the tensor-core and transposed kernels."""
    dev = _require_cuda(val, idx)
    code = _dtype_code(val)
    val, idx = val.contiguous(), idx.contiguous()
    L = nat.lib()
    nbytes = L.nmg_packed_bytes(M, K, n, m, g, code)
    buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        nat.check(L.nmg_pack(val.data_ptr(), idx.data_ptr(), M, K, n, m, g, code, buf.data_ptr(), nbytes, _stream(dev)))
    return buf


@functools.lru_cache(maxsize=4096)
def uses_packed(M, K, tokens, n, m, g, dtype, layout=nat.NMG_ACT_TOKEN_MAJOR, algo=nat.NMG_ALGO_AUTO, transposed=False):
    """Whether spmm (or spmm_t when `transposed`) would read the packed copy for this problem: the fused tensor-core
    kernel and the SIMT transposed kernel do; the two-pass tensor-core variant and the SIMT forward kernel do not."""
    code = {torch.float32: nat.NMG_F32, torch.float16: nat.NMG_F16, torch.bfloat16: nat.NMG_BF16}[dtype]
    return bool(nat.lib().nmg_spmm_uses_packed(M, K, tokens, n, m, g, code, layout, algo, 1 if transposed else 0))


@functools.lru_cache(maxsize=4096)
def _spmm_workspace_bytes(M, K, tokens, n, m, g, code, layout, algo, have_packed):
    return nat.lib().nmg_spmm_workspace_bytes(M, K, tokens, n, m, g, code, layout, algo, have_packed)


def spmm(val, idx, M, K, n, m, g, act, bias=None, layout=nat.NMG_ACT_TOKEN_MAJOR, algo=nat.NMG_ALGO_AUTO, out=None,
         packed=None, activation=None, residual=None):
    """layout TOKEN_MAJOR:          act [tokens, K] -> out [tokens, M] = act @ W^T (+ bias)
       layout K_MAJOR:              act [K, tokens] -> out [M, tokens] = W @ act   (+ bias per row)
       layout TOKEN_MAJOR_OUT_ROWS: act [tokens, K] -> out [M, tokens] = W @ act^T (+ bias per row)
    ``activation="gelu"`` and ``residual`` (a tensor of the output's shape) make it out = activation(product + bias) + residual
    in the same call (fused into the matmul's epilogue on the two-pass tensor-core path)."""
    dev = _require_cuda(val, idx, act, bias)
    code = _dtype_code(val)
    if act.dtype != val.dtype or (bias is not None and bias.dtype != val.dtype):
        raise TypeError(f"activation / bias dtype must match the weight dtype {val.dtype}")
    act, ld_act = _row_major_2d(act)
    token_major = layout != nat.NMG_ACT_K_MAJOR
    tokens = act.shape[0] if token_major else act.shape[1]
    if (act.shape[1] if token_major else act.shape[0]) != K:
        raise ValueError(f"activation shape {tuple(act.shape)} does not match K={K}")
    out_shape = (tokens, M) if layout == nat.NMG_ACT_TOKEN_MAJOR else (M, tokens)
    if out is None:
        out = torch.empty(out_shape, dtype=val.dtype, device=dev)
    else:
        # the kernel writes out_shape[0] rows of out_shape[1] elements, ld_out apart: anything else would land outside `out`
        if out.dtype != val.dtype or out.device != dev:
            raise ValueError(f"out must be a {val.dtype} tensor on {dev}, got {out.dtype} on {out.device}")
        if tuple(out.shape) != out_shape:
            raise ValueError(f"out must have shape {out_shape} for this layout, got {tuple(out.shape)}")
        if out_shape[1] > 1 and out.stride(1) != 1:
            raise ValueError("out must have unit stride along its rows (a transposed view cannot be written in place)")
        if out_shape[0] > 1 and out.stride(0) < out_shape[1]:
            raise ValueError(f"out rows overlap: stride {out.stride(0)} is smaller than the row length {out_shape[1]}")
    ld_out = out.stride(0) if out_shape[0] > 1 else out_shape[1]
    if tokens == 0:
        return out
    val, idx = val.contiguous(), idx.contiguous()
    if bias is not None:
        bias = bias.contiguous()
    L = nat.lib()
    if activation not in (None, "gelu"):
        raise ValueError("activation must be None or 'gelu'")
    fused = activation is not None or residual is not None
    if residual is not None:
        _require_cuda(residual)
        if residual.dtype != val.dtype or tuple(residual.shape) != out_shape or (out_shape[1] > 1 and residual.stride(1) != 1):
            raise ValueError(f"residual must be a {val.dtype} tensor of shape {out_shape} with contiguous rows")
    with _on_device(dev):
        ws, nbytes = _workspace(_spmm_workspace_bytes(M, K, tokens, n, m, g, code, layout, algo, 1 if packed is not None else 0), dev)
        if fused:
            nat.check(L.nmg_spmm_fused(val.data_ptr(), idx.data_ptr(), packed.data_ptr() if packed is not None else None, M, K, n,
                                       m, g, code, act.data_ptr(), ld_act, tokens, bias.data_ptr() if bias is not None else None,
                                       nat.NMG_EPI_GELU if activation == "gelu" else nat.NMG_EPI_NONE,
                                       residual.data_ptr() if residual is not None else None,
                                       (residual.stride(0) if out_shape[0] > 1 else out_shape[1]) if residual is not None else 0,
                                       out.data_ptr(), ld_out, layout, algo, ws.data_ptr() if ws is not None else None, nbytes, _stream(dev)))
        else:
            nat.check(L.nmg_spmm(val.data_ptr(), idx.data_ptr(), packed.data_ptr() if packed is not None else None, M, K, n,
                                 m, g, code, act.data_ptr(), ld_act, tokens,
                                 bias.data_ptr() if bias is not None else None, out.data_ptr(), ld_out, layout, algo,
                                 ws.data_ptr() if ws is not None else None, nbytes, _stream(dev)))
    return out


def expand(val, idx, M, K, n, m, g):
    """Dense 16-bit copy of a weight for ``spmm_expanded`` (opaque uint8 buffer); None when the weight has none (fp32)."""
    dev = _require_cuda(val, idx)
    code = _dtype_code(val)
    nbytes = nat.lib().nmg_expanded_bytes(M, K, n, m, g, code)
    if nbytes == 0:
        return None
    val, idx = val.contiguous(), idx.contiguous()
    buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        nat.check(nat.lib().nmg_expand(val.data_ptr(), idx.data_ptr(), M, K, n, m, g, code, buf.data_ptr(), nbytes, _stream(dev)))
    return buf


def spmm_expanded(expanded, M, K, act, bias=None, activation=None, residual=None, out=None):
    """act [tokens, K] -> out [tokens, M] = activation(act @ W^T + bias) + residual from a kept expanded weight."""
    dev = _require_cuda(expanded, act, bias, residual)
    code = _dtype_code(act)
    act, ld_act = _row_major_2d(act)
    tokens = act.shape[0]
    if out is None:
        out = torch.empty((tokens, M), dtype=act.dtype, device=dev)
    if tokens == 0:
        return out
    if residual is not None and (tuple(residual.shape) != (tokens, M) or residual.stride(1) != 1 or residual.dtype != act.dtype):
        raise ValueError("residual must match the output's shape and dtype, with contiguous rows")
    with _on_device(dev):
        nat.check(nat.lib().nmg_spmm_expanded(expanded.data_ptr(), M, K, code, act.data_ptr(), ld_act, tokens,
                                              bias.contiguous().data_ptr() if bias is not None else None,
                                              nat.NMG_EPI_GELU if activation == "gelu" else nat.NMG_EPI_NONE,
                                              residual.data_ptr() if residual is not None else None,
                                              residual.stride(0) if residual is not None and tokens > 1 else M,
                                              out.data_ptr(), out.stride(0) if tokens > 1 else M, nat.NMG_ACT_TOKEN_MAJOR, _stream(dev)))
    return out


def spmm_replicated(val, idx, M, K, n, m, g, act, out_ptrs, ld_out, bias=None, multicast_ptr=None):
    """C = W @ act^T (+ bias per row) written into every buffer of ``out_ptrs`` (device addresses of [M, ld_out] row
    panels: this GPU's and the peers' mapped copies) by the matmul kernel itself.  The caller keeps the buffers alive and
    synchronises the ranks afterwards.  ``multicast_ptr``: NVSwitch multicast address of the same location, when there is one."""
    import ctypes
    dev = _require_cuda(val, idx, act, bias)
    code = _dtype_code(val)
    if act.dtype != val.dtype or (bias is not None and bias.dtype != val.dtype):
        raise TypeError(f"activation / bias dtype must match the weight dtype {val.dtype}")
    act, ld_act = _row_major_2d(act)
    tokens = act.shape[0]
    if act.shape[1] != K:
        raise ValueError(f"activation shape {tuple(act.shape)} does not match K={K}")
    val, idx = val.contiguous(), idx.contiguous()
    if bias is not None:
        bias = bias.contiguous()
    L = nat.lib()
    ptrs = (ctypes.c_void_p * len(out_ptrs))(*[int(p) for p in out_ptrs])
    with torch.cuda.device(dev):
        ws, nbytes = _workspace(L.nmg_spmm_replicated_workspace_bytes(M, K, tokens, n, m, g, code), dev)
        nat.check(L.nmg_spmm_replicated(val.data_ptr(), idx.data_ptr(), M, K, n, m, g, code, act.data_ptr(), ld_act, tokens,
                                        bias.data_ptr() if bias is not None else None, ptrs, len(out_ptrs),
                                        int(multicast_ptr) if multicast_ptr else None, ld_out,
                                        ws.data_ptr() if ws is not None else None, nbytes, _stream(dev)))


SP24_MIN_TOKENS = 1280  # from here on the transposed product of a 16-bit weight runs on the structured-sparse tensor cores


@functools.lru_cache(maxsize=4096)
def sp24_bytes(M, K, n, m, g, dtype):
    """Size of the compressed transposed copy of a weight, 0 when the weight is outside the 2:4 structure."""
    code = _DTYPES.get(dtype)
    return 0 if code is None else nat.lib().nmg_sp24_bytes(M, K, n, m, g, code)


def pack_sp24(val, idx, M, K, n, m, g):
    """Compressed transposed copy of a 16-bit weight for the structured-sparse transposed product (opaque uint8 buffer)."""
    dev = _require_cuda(val, idx)
    code = _dtype_code(val)
    nbytes = sp24_bytes(M, K, n, m, g, val.dtype)
    if nbytes == 0:
        raise ValueError("this weight is outside the 2:4 structure (needs a 16-bit dtype, n <= 2 and m in {4, 8, 16, 32, 64})")
    val, idx = val.contiguous(), idx.contiguous()
    buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        nat.check(nat.lib().nmg_pack_sp24(val.data_ptr(), idx.data_ptr(), M, K, n, m, g, code, buf.data_ptr(), nbytes, _stream(dev)))
    return buf


def spmm_t(val, idx, M, K, n, m, g, dy, algo=nat.NMG_ALGO_AUTO, packed=None, sp24=None):
    """dy [tokens, M] -> dx [tokens, K] = dy @ W.  ``sp24``: result of pack_sp24 for the same weight; used (and the per-call
    compression skipped) when the call would take the structured-sparse path anyway."""
    dev = _require_cuda(val, idx, dy)
    code = _dtype_code(val)
    if dy.dtype != val.dtype:
        raise TypeError(f"gradient dtype must match the weight dtype {val.dtype}")
    dy, ld_dy = _row_major_2d(dy)
    tokens = dy.shape[0]
    if dy.shape[1] != M:
        raise ValueError(f"gradient shape {tuple(dy.shape)} does not match M={M}")
    dx = torch.empty((tokens, K), dtype=val.dtype, device=dev)
    if tokens == 0:
        return dx
    val, idx = val.contiguous(), idx.contiguous()
    L = nat.lib()
    if (sp24 is not None and tokens >= SP24_MIN_TOKENS and algo in (nat.NMG_ALGO_AUTO, nat.NMG_ALGO_TENSOR)
            and dy.data_ptr() % 16 == 0 and ld_dy % 8 == 0):
        with _on_device(dev):
            nat.check(L.nmg_spmm_t_sp24(sp24.data_ptr(), M, K, n, m, g, code, dy.data_ptr(), ld_dy, tokens, dx.data_ptr(), K, _stream(dev)))
        return dx
    with _on_device(dev):
        ws, nbytes = _workspace(L.nmg_spmm_t_workspace_bytes(M, K, tokens, n, m, g, code, algo,
                                                             1 if packed is not None else 0), dev)
        nat.check(L.nmg_spmm_t(val.data_ptr(), idx.data_ptr(), packed.data_ptr() if packed is not None else None, M, K,
                               n, m, g, code, dy.data_ptr(), ld_dy, tokens,
                               dx.data_ptr(), K, algo, ws.data_ptr() if ws is not None else None, nbytes,
                               _stream(dev)))
    return dx


def copy_2d_async(dst, src, stream=None):
    """Queue a pitched copy between two 2-D tensors of the same shape and dtype whose rows are contiguous (one of them
    typically a column block of a pinned host matrix).  Unlike ``Tensor.copy_`` it never stages through pageable memory."""
    if dst.shape != src.shape or dst.dim() != 2 or dst.dtype != src.dtype:
        raise ValueError("copy_2d_async needs two 2-D tensors of equal shape and dtype")
    if dst.stride(1) != 1 or src.stride(1) != 1:
        raise ValueError("rows must be contiguous")
    es = dst.element_size()
    cuda_side = dst if dst.is_cuda else src
    if not cuda_side.is_cuda:
        raise TypeError("one side must be a CUDA tensor")
    for t in (dst, src):
        if not t.is_cuda and not t.is_pinned():
            raise TypeError("the host side must be pinned memory")
    st = stream.cuda_stream if stream is not None else _stream(cuda_side.device)
    with torch.cuda.device(cuda_side.device):
        nat.check(nat.lib().nmg_memcpy_2d_async(dst.data_ptr(), dst.stride(0) * es, src.data_ptr(), src.stride(0) * es,
                                                dst.shape[1] * es, dst.shape[0], st))


def read_status(dev=None):
    """Synchronise the current stream and raise if any kernel's bounded wait ran out."""
    import ctypes
    dev = dev if dev is not None else torch.device("cuda", torch.cuda.current_device())
    code = ctypes.c_int(0)
    with torch.cuda.device(dev):
        nat.check(nat.lib().nmg_read_status(_stream(dev), ctypes.byref(code)))
    return code.value
