"""Operator layer: the entry points of the reference's ``cuda_kernel/ops.py``
(``__all__`` at :750-775) with the same names, positional order, return shapes
and error behaviour, implemented on the C ABI of ``libw4a4_b200.so``.

Differences that follow from the B200 design (results are unaffected):

* one shape-aware kernel family backs every GEMM entry point, so the ``*_int4``,
  ``*_decode`` and ``*_smallT`` names are aliases of the same call;
* the quant kernel uses IEEE division and therefore equals the reference's
  oracle (``tools/parity/quant_reference.py``) bit for bit;
* there is no Triton or CPU fallback: a missing library raises at import.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .nvtx_shim import traced
from .pack_utils import BCOL, BROW


def _cd(t: torch.Tensor, dtype) -> torch.Tensor:
    """``t`` as a contiguous tensor of ``dtype``; the tensor itself when it already is one (the usual
    case: a no-op ``.to`` still costs most of a microsecond per argument and call)."""
    if t.dtype is not dtype:
        t = t.to(dtype)
    return t if t.is_contiguous() else t.contiguous()

_L = _lib.load()


def reserve_workspace(device, T: int, d_in: int, d_out: int, n_hp_blocks: int = 0) -> None:
    """Allocate the scratch buffer for a shape up front (needed before CUDA-graph
    capture, where allocation is not allowed)."""
    _lib.workspace(torch.device(device), int(T), int(d_in), int(d_out), int(n_hp_blocks))


# ---------------------------------------------------------------------------
# activation_quant   (reference: cuda_kernel/ops.py:223-260)
# ---------------------------------------------------------------------------

@traced("cuda.activation_quant")
def activation_quant_cuda(
    X_fp16: torch.Tensor,
    perm: torch.Tensor,
    bcol: int = BCOL,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-token s4 quantisation: returns ``(X_s4 (T, D/2) int8, scale_x (T,)
    fp16, sum_X (T, D/128) int32)``."""
    assert X_fp16.is_cuda, "activation_quant_cuda requires a CUDA tensor"
    assert X_fp16.dtype == torch.float16, "X must be fp16"
    assert perm.dtype in (torch.int32, torch.int64), "perm must be int32/int64"
    shape = X_fp16.shape
    if X_fp16.dim() == 3:
        T, D = shape[0] * shape[1], shape[2]
    elif X_fp16.dim() == 2:
        T, D = shape
    else:
        raise ValueError(f"X must be 2D or 3D, got shape {shape}")
    if bcol != BCOL:
        raise ValueError(f"bcol must be {BCOL}, got {bcol}")
    if D % bcol != 0:
        raise ValueError(f"d_in ({D}) must be divisible by bcol ({bcol})")
    X_2d = X_fp16.reshape(T, D)
    if X_2d.stride(-1) != 1 or (T > 1 and X_2d.stride(0) < D):
        X_2d = X_2d.contiguous()          # row-strided inputs (a column slice of a wider tensor) go to the kernel as they are
    perm_i32 = _cd(perm if perm.device == X_2d.device else perm.to(X_2d.device), torch.int32)
    dev = X_2d.device
    X_s4 = torch.empty((T, D // 2), dtype=torch.int8, device=dev)
    scale_x = torch.empty((T,), dtype=torch.float16, device=dev)
    sum_X = torch.empty((T, D // bcol), dtype=torch.int32, device=dev)
    if T == 0:
        return X_s4, scale_x, sum_X
    with _lib.on_device(dev):
        _lib.check(_L.w4a4_activation_quant(
            X_2d.data_ptr(), X_2d.stride(0) if T > 1 else D, perm_i32.data_ptr(), X_s4.data_ptr(),
            scale_x.data_ptr(), sum_X.data_ptr(), int(T), int(D), _lib.stream_ptr(dev),
        ), "activation_quant")
    return X_s4, scale_x, sum_X


# ---------------------------------------------------------------------------
# quantisation fused with the element-wise step in front of it (no counterpart in the
# reference, whose layers run RMSNorm / SiLU*mul as separate PyTorch launches)
# ---------------------------------------------------------------------------

def perm_or_none(perm: torch.Tensor, cache_on=None):
    """``None`` when ``perm`` is the identity (the kernels then read rows with 128-bit loads instead of
    gathering), else ``perm`` as contiguous int32.  The check synchronises once; pass the object that
    owns ``perm`` (a weight container) as ``cache_on`` to remember the answer there."""
    if cache_on is not None and getattr(cache_on, "_perm_arg", None) is not None:
        tag, val = cache_on._perm_arg
        if tag == perm.data_ptr():
            return val
    p32 = _cd(perm, torch.int32)
    ident = bool(torch.equal(p32, torch.arange(p32.numel(), dtype=torch.int32, device=p32.device)))
    val = None if ident else p32
    if cache_on is not None:
        cache_on._perm_arg = (perm.data_ptr(), val)
    return val


def _code_format(e4m3) -> int:
    """``False``: s8 codes; ``True``: e4m3 bytes for prepared weights; ``"packed"``: e4m3 bytes in the
    order packed weights are read in (see include/w4a4_b200.h, W4A4_CODES_*)."""
    if isinstance(e4m3, str):
        if e4m3 != "packed":
            raise ValueError(f"e4m3 must be False, True or 'packed', got {e4m3!r}")
        return _lib.CODES_E4M3_PACKED
    return _lib.CODES_E4M3 if e4m3 else _lib.CODES_S8


def _code_flag(e4m3) -> int:
    return (0, _lib.FLAG_CODES_E4M3, _lib.FLAG_CODES_E4M3_PACKED)[_code_format(e4m3)]


def _fused_prologue(which: str, X2: torch.Tensor, K: int, perm, norm_weight, eps: float, expanded: bool, e4m3):
    T = int(X2.shape[0])
    dev = X2.device
    scale_x = torch.empty((T,), dtype=torch.float16, device=dev)
    if expanded:
        XE = torch.empty((int(_L.w4a4_expanded_codes_bytes(T, K)),), dtype=torch.int8, device=dev)
        sumxf = torch.zeros(((T + 15) // 16, K // BCOL, 16), dtype=torch.float32, device=dev)
        outs = (None, scale_x.data_ptr(), None, XE.data_ptr(), sumxf.data_ptr())
        ret = (XE, sumxf, scale_x)
    else:
        X_s4 = torch.empty((T, K // 2), dtype=torch.int8, device=dev)
        sum_X = torch.empty((T, K // BCOL), dtype=torch.int32, device=dev)
        outs = (X_s4.data_ptr(), scale_x.data_ptr(), sum_X.data_ptr(), None, None)
        ret = (X_s4, scale_x, sum_X)
    if T == 0:
        return ret
    pp = None if perm is None else perm.data_ptr()
    with _lib.on_device(dev):
        if which == "rmsnorm":
            w = norm_weight.to(device=dev, dtype=torch.float16).contiguous()
            _lib.check(_L.w4a4_rmsnorm_quant(X2.data_ptr(), X2.stride(0) if T > 1 else K, w.data_ptr(), float(eps), pp, *outs,
                                             _code_format(e4m3), T, K, _lib.stream_ptr(dev)), "rmsnorm_quant")
        else:
            _lib.check(_L.w4a4_silu_mul_quant(X2.data_ptr(), X2.stride(0) if T > 1 else 2 * K, pp, *outs,
                                              _code_format(e4m3), T, K, _lib.stream_ptr(dev)), "silu_mul_quant")
    return ret


def _rows(X: torch.Tensor, width: int) -> torch.Tensor:
    X2 = X.reshape(-1, width)
    if X2.stride(-1) != 1 or (X2.shape[0] > 1 and X2.stride(0) < width):
        X2 = X2.contiguous()
    return X2


def rmsnorm_quant_cuda(X_fp16, norm_weight, eps, perm, *, expanded: bool = False, e4m3=False):
    """RMSNorm and activation quantisation in one launch: quantises
    ``fp16(fp16(x * rsqrt(mean(x^2) + eps)) * norm_weight)``.  Returns ``(X_s4, scale_x, sum_X)`` like
    :func:`activation_quant_cuda`, or with ``expanded=True`` ``(XE, sumxf, scale_x)`` in the layout
    :func:`fused_dense_sparse_expanded_cuda` reads.  ``perm``: int32 permutation, or ``None`` for identity."""
    assert X_fp16.is_cuda and X_fp16.dtype == torch.float16
    K = int(X_fp16.shape[-1])
    if K % BCOL != 0:
        raise ValueError(f"d_in ({K}) must be divisible by {BCOL}")
    if int(norm_weight.numel()) != K:
        raise ValueError(f"norm_weight must have {K} entries, got {int(norm_weight.numel())}")
    return _fused_prologue("rmsnorm", _rows(X_fp16, K), K, perm, norm_weight, eps, expanded, e4m3)


def silu_mul_quant_cuda(gate_up_fp16, perm, *, expanded: bool = False, e4m3=False):
    """``silu(gate) * up`` and activation quantisation in one launch.  ``gate_up_fp16 (..., 2K)`` holds the
    gate in its first K columns and the up projection in the last K (the output of a fused gate/up
    linear); the quantised tensor is ``fp16(fp16(silu(gate)) * up)`` of width K.  Returns as
    :func:`rmsnorm_quant_cuda`."""
    assert gate_up_fp16.is_cuda and gate_up_fp16.dtype == torch.float16
    K2 = int(gate_up_fp16.shape[-1])
    if K2 % (2 * BCOL) != 0:
        raise ValueError(f"the gate/up width ({K2}) must be a multiple of {2 * BCOL}")
    return _fused_prologue("silu_mul", _rows(gate_up_fp16, K2), K2 // 2, perm, None, 0.0, expanded, e4m3)


# ---------------------------------------------------------------------------
# argument preparation shared by the GEMM entry points (ops.py:268-298,419-460)
# ---------------------------------------------------------------------------

def _prep_dense(W_low_packed, X_s4, scale_u4, zero_u4, sum_X, scale_x):
    assert W_low_packed.is_cuda and X_s4.is_cuda
    assert W_low_packed.dtype == torch.int8 and X_s4.dtype == torch.int8
    d_out, d_in_half = W_low_packed.shape
    T = X_s4.shape[0]
    d_in = d_in_half * 2
    ng = d_in // BCOL
    assert X_s4.shape == (T, d_in_half)
    assert scale_u4.shape == (d_out, ng)
    assert zero_u4.shape == (d_out, ng)
    assert sum_X.shape == (T, ng)
    assert scale_x.shape == (T,)
    return (W_low_packed.contiguous(), X_s4.contiguous(),
            _cd(scale_u4, torch.float16), _cd(zero_u4, torch.float16),
            _cd(sum_X, torch.int32), _cd(scale_x, torch.float16),
            int(T), int(d_in), int(d_out))


def _flags(token_major: bool, force: Optional[str]) -> int:
    f = _lib.FLAG_OUT_TOKEN_MAJOR if token_major else 0
    if force == "stream":
        f |= _lib.FLAG_FORCE_STREAM
    elif force == "tensor":
        f |= _lib.FLAG_FORCE_TENSOR
    elif force is not None:
        raise ValueError(f"force must be None, 'stream' or 'tensor', got {force!r}")
    return f


def _out(d_out: int, T: int, device, token_major: bool) -> torch.Tensor:
    shape = (T, d_out) if token_major else (d_out, T)
    return torch.empty(shape, dtype=torch.float16, device=device)


@traced("cuda.dense_gemm")
def dense_gemm_cuda_int4(W_low_packed, X_s4, scale_u4, zero_u4, sum_X, scale_x,
                         *, token_major: bool = False, force: Optional[str] = None) -> torch.Tensor:
    """Dense u4 x s4 GEMM: ``Y_low (d_out, T)`` fp16 (ops.py:314-320)."""
    W, X, s, z, sm, sx, T, K, N = _prep_dense(W_low_packed, X_s4, scale_u4, zero_u4, sum_X, scale_x)
    Y = _out(N, T, W.device, token_major)
    if T == 0:
        return Y
    with _lib.on_device(W.device):
        ws = _lib.workspace(W.device, T, K, N, 0)
        _lib.check(_L.w4a4_dense_gemm(
            W.data_ptr(), X.data_ptr(), s.data_ptr(), z.data_ptr(), sm.data_ptr(), sx.data_ptr(),
            Y.data_ptr(), T, K, N, _flags(token_major, force), ws.data_ptr(), ws.numel(),
            _lib.stream_ptr(W.device)), "dense_gemm")
    return Y


# T-specialised names of the reference map onto the same shape-aware launcher.
dense_gemv_cuda_decode = dense_gemm_cuda_int4
dense_gemm_cuda = dense_gemm_cuda_int4


def dense_gemm_cuda_int8(*args, **kwargs):
    """Archived in the reference (ops.py:306-311); kept as a raising stub."""
    raise RuntimeError(
        "dense_gemm_cuda_int8 is archived; use dense_gemm_cuda_int4 (the production path)."
    )


@traced("cuda.sparse_gemm")
def sparse_gemm_cuda_int4(W_high_blocks_packed, hp_row_offsets, hp_col_indices,
                          X_s4, scale_u4, scale_x, d_out, d_in,
                          *, token_major: bool = False, force: Optional[str] = None) -> torch.Tensor:
    """Block-CSR s4 x s4 GEMM: ``Y_high (d_out, T)`` fp16 WITHOUT the factor 16;
    zeros (and no launch) for an empty block list (ops.py:360-408)."""
    assert X_s4.is_cuda
    T = int(X_s4.shape[0])
    d_out, d_in = int(d_out), int(d_in)
    dev = X_s4.device
    nnz = int(W_high_blocks_packed.shape[0])
    if nnz == 0 or T == 0:
        return torch.zeros((T, d_out) if token_major else (d_out, T), dtype=torch.float16, device=dev)
    Wh = W_high_blocks_packed.contiguous()
    ro = _cd(hp_row_offsets, torch.int32)
    ci = _cd(hp_col_indices, torch.int32)
    X = X_s4.contiguous()
    s = _cd(scale_u4, torch.float16)
    sx = _cd(scale_x, torch.float16)
    _check_bsr(ro, ci, d_out, d_in, nnz)
    Y = _out(d_out, T, dev, token_major)
    with _lib.on_device(dev):
        ws = _lib.workspace(dev, T, d_in, d_out, nnz)
        _lib.check(_L.w4a4_sparse_gemm(
            Wh.data_ptr(), ro.data_ptr(), ci.data_ptr(), X.data_ptr(), s.data_ptr(), sx.data_ptr(),
            Y.data_ptr(), T, d_in, d_out, nnz, _flags(token_major, force), ws.data_ptr(), ws.numel(),
            _lib.stream_ptr(dev)), "sparse_gemm")
    return Y


sparse_gemm_cuda = sparse_gemm_cuda_int4


def sparse_gemm_cuda_int8(*args, **kwargs):
    """Archived in the reference (ops.py:386-391); kept as a raising stub."""
    raise RuntimeError("sparse_gemm_cuda_int8 is archived; use sparse_gemm_cuda_int4.")


def _check_bsr(hp_row_offsets, hp_col_indices, d_out, d_in, nnz):
    nbr = (d_out + BROW - 1) // BROW
    if hp_row_offsets.numel() != nbr + 1:
        raise RuntimeError(
            f"hp_row_offsets must have ceil(d_out/128)+1 = {nbr + 1} entries, got {hp_row_offsets.numel()}"
        )
    if hp_col_indices.numel() != nnz:
        raise RuntimeError(f"hp_col_indices must have {nnz} entries, got {hp_col_indices.numel()}")
    if d_in % BCOL != 0:
        raise RuntimeError(f"d_in ({d_in}) must be divisible by {BCOL}")


def _prep_fused(W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
                X_s4, scale_u4, zero_u4, sum_X, scale_x, d_out, d_in):
    assert W_low_packed.is_cuda and X_s4.is_cuda
    assert W_low_packed.dtype == torch.int8 and X_s4.dtype == torch.int8
    d_out, d_in = int(d_out), int(d_in)
    T = int(X_s4.shape[0])
    ng = d_in // BCOL
    assert X_s4.shape == (T, d_in // 2)
    assert scale_u4.shape == (d_out, ng)
    assert zero_u4.shape == (d_out, ng)
    assert sum_X.shape == (T, ng)
    assert scale_x.shape == (T,)
    if W_high_blocks_packed.numel() == 0:
        W_high_blocks_packed = torch.zeros((0, BROW, BCOL // 2), dtype=torch.int8,
                                           device=W_low_packed.device)
    ro = _cd(hp_row_offsets, torch.int32)
    ci = _cd(hp_col_indices, torch.int32)
    _check_bsr(ro, ci, d_out, d_in, int(W_high_blocks_packed.shape[0]))
    return (W_low_packed.contiguous(), W_high_blocks_packed.contiguous(), ro, ci, X_s4.contiguous(),
            _cd(scale_u4, torch.float16), _cd(zero_u4, torch.float16),
            _cd(sum_X, torch.int32), _cd(scale_x, torch.float16), T, d_in, d_out)


def prepare_weights_cuda(packed: torch.Tensor) -> torch.Tensor:
    """A packed weight array (``W_low_packed`` or ``W_high_blocks_packed``) widened once to one
    byte per code for the many-token tensor-core kernel: same leading shape, last dimension
    doubled, dtype uint8 (e4m3 encodings; see include/w4a4_b200.h).  Pass the results as
    ``prepared=(low, high)`` to the fused operators.  No counterpart in the reference."""
    assert packed.is_cuda and packed.dtype == torch.int8
    src = packed.contiguous()
    out = torch.empty(src.shape[:-1] + (src.shape[-1] * 2,), dtype=torch.uint8, device=src.device)
    if src.numel():
        with _lib.on_device(src.device):
            _lib.check(_L.w4a4_prepare_weights(src.data_ptr(), out.data_ptr(), src.numel(),
                                               _lib.stream_ptr(src.device)), "prepare_weights")
    return out


def dequant_u4_to_fp16_cuda(W_low_packed: torch.Tensor, scale_u4: torch.Tensor, zero_u4: torch.Tensor) -> torch.Tensor:
    """Dense ``(d_out, d_in)`` fp16 copy of the low-precision weights, ``((code - zero) * scale)`` in half precision:
    the reference's ``dequant_u4_to_fp16`` (triton_kernel/dequant_w4_to_fp16.py:131-172), bit for bit."""
    assert W_low_packed.is_cuda and W_low_packed.dtype == torch.int8 and W_low_packed.dim() == 2
    W = W_low_packed.contiguous()
    N, K = int(W.shape[0]), int(W.shape[1]) * 2
    s = _cd(scale_u4, torch.float16)
    z = _cd(zero_u4, torch.float16)
    assert s.shape == (N, K // BCOL) and z.shape == (N, K // BCOL)
    out = torch.empty((N, K), dtype=torch.float16, device=W.device)
    with _lib.on_device(W.device):
        _lib.check(_L.w4a4_dequant_weights_fp16(W.data_ptr(), s.data_ptr(), z.data_ptr(), out.data_ptr(), N, K,
                                                _lib.stream_ptr(W.device)), "dequant_weights")
    return out


def _prepared_ptrs(prepared, W, Wh, nnz):
    """Device pointers of the (low, high) pair made by :func:`prepare_weights_cuda`, checked against the packed arrays."""
    if prepared is None:
        return None, None
    lo, hi = prepared
    assert lo.is_cuda and lo.dtype == torch.uint8 and lo.is_contiguous() and lo.numel() == 2 * W.numel()
    if nnz:
        assert hi is not None and hi.dtype == torch.uint8 and hi.is_contiguous() and hi.numel() == 2 * Wh.numel()
    return lo.data_ptr(), (hi.data_ptr() if nnz else None)


@traced("cuda.fused_dense_sparse")
def fused_dense_sparse_cuda_int4(
    W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
    X_s4, scale_u4, zero_u4, sum_X, scale_x, d_out, d_in,
    *, token_major: bool = False, force: Optional[str] = None, prepared=None,
) -> torch.Tensor:
    """Fused dense + 16 x residual GEMM: ``Y_total (d_out, T)`` fp16 (ops.py:471-481).
    ``prepared``: the pair from :func:`prepare_weights_cuda` for the many-token kernel."""
    (W, Wh, ro, ci, X, s, z, sm, sx, T, K, N) = _prep_fused(
        W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
        X_s4, scale_u4, zero_u4, sum_X, scale_x, d_out, d_in)
    Y = _out(N, T, W.device, token_major)
    if T == 0:
        return Y
    nnz = int(Wh.shape[0])
    with _lib.on_device(W.device):
        ws = _lib.workspace(W.device, T, K, N, nnz)
        plo, phi = _prepared_ptrs(prepared, W, Wh, nnz)
        _lib.check(_L.w4a4_fused_dense_sparse_prepared(
            W.data_ptr(), Wh.data_ptr() if nnz else None, plo, phi, ro.data_ptr(), ci.data_ptr() if nnz else None,
            X.data_ptr(), s.data_ptr(), z.data_ptr(), sm.data_ptr(), sx.data_ptr(), Y.data_ptr(),
            T, K, N, nnz, _flags(token_major, force), ws.data_ptr(), ws.numel(),
            _lib.stream_ptr(W.device)), "fused_dense_sparse")
    return Y


def expand_activations_cuda(X_s4: torch.Tensor, sum_X: torch.Tensor, *, e4m3=False):
    """Quantised activations in the layout the GEMM kernels read: returns
    ``(XE, sumxf)`` - an opaque int8 buffer of expanded codes (group-major, see
    include/w4a4_b200.h) and ``(ceil(T/16), K/128, 16)`` fp32 group sums.  Build once
    and reuse across the linears that share an input (no counterpart in the
    reference).  ``e4m3=True`` writes the codes as e4m3 bytes, the form that goes
    with weights from :func:`prepare_weights_cuda`; ``e4m3="packed"`` writes the e4m3 form the
    tensor-core kernel reads against the packed weights."""
    assert X_s4.is_cuda and X_s4.dtype == torch.int8 and sum_X.dtype == torch.int32
    T, K = int(X_s4.shape[0]), int(X_s4.shape[1]) * 2
    X = X_s4.contiguous()
    sm = sum_X.contiguous()
    XE = torch.empty((int(_L.w4a4_expanded_codes_bytes(T, K)),), dtype=torch.int8, device=X.device)
    sumxf = torch.zeros(((T + 15) // 16, K // BCOL, 16), dtype=torch.float32, device=X.device)
    with _lib.on_device(X.device):
        _lib.check(_L.w4a4_expand_activations_fmt(X.data_ptr(), sm.data_ptr(), XE.data_ptr(), sumxf.data_ptr(),
                                                  T, K, _code_format(e4m3), _lib.stream_ptr(X.device)),
                   "expand_activations")
    return XE, sumxf


def fused_dense_sparse_expanded_cuda(
    W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
    XE, sumxf, scale_u4, zero_u4, scale_x, d_out, d_in,
    *, token_major: bool = False, force: Optional[str] = None, prepared=None, e4m3=False,
) -> torch.Tensor:
    """:func:`fused_dense_sparse_cuda_int4` on activations already expanded by
    :func:`expand_activations_cuda`; a single kernel launch.  ``e4m3`` repeats what ``XE`` was
    expanded with: ``True`` goes with ``prepared`` weights, ``"packed"`` with the packed arrays
    (no ``prepared``); both always run the tensor-core kernel.  A mismatch raises ``ValueError``:
    the bytes of ``XE`` are never reinterpreted silently."""
    d_out, d_in = int(d_out), int(d_in)
    T = int(scale_x.shape[0])
    assert XE.is_cuda and XE.dtype == torch.int8 and XE.is_contiguous()
    assert XE.numel() >= int(_L.w4a4_expanded_codes_bytes(T, d_in)), "XE was built for another shape"
    assert sumxf.dtype == torch.float32 and sumxf.is_contiguous()
    W = W_low_packed.contiguous()
    nnz = int(W_high_blocks_packed.shape[0]) if W_high_blocks_packed.numel() else 0
    Wh = W_high_blocks_packed.contiguous()
    ro = _cd(hp_row_offsets, torch.int32)
    ci = _cd(hp_col_indices, torch.int32)
    _check_bsr(ro, ci, d_out, d_in, nnz)
    s = _cd(scale_u4, torch.float16)
    z = _cd(zero_u4, torch.float16)
    sx = _cd(scale_x, torch.float16)
    Y = _out(d_out, T, W.device, token_major)
    with _lib.on_device(W.device):
        ws = _lib.workspace(W.device, T, d_in, d_out, nnz)
        plo, phi = _prepared_ptrs(prepared, W, Wh, nnz)
        _lib.check(_L.w4a4_fused_dense_sparse_expanded_prepared(
            W.data_ptr(), Wh.data_ptr() if nnz else None, plo, phi, ro.data_ptr(), ci.data_ptr() if nnz else None,
            XE.data_ptr(), sumxf.data_ptr(), s.data_ptr(), z.data_ptr(), sx.data_ptr(), Y.data_ptr(),
            T, d_in, d_out, nnz, _flags(token_major, force) | _code_flag(e4m3),
            ws.data_ptr(), ws.numel(), _lib.stream_ptr(W.device)), "fused_dense_sparse_expanded")
    return Y


fused_gemv_cuda_decode = fused_dense_sparse_cuda_int4
fused_gemv_cuda_smallT = fused_dense_sparse_cuda_int4
fused_dense_sparse_cuda = fused_dense_sparse_cuda_int4


def fused_dense_sparse_cuda_int8(*args, **kwargs):
    """Archived in the reference (ops.py:463-468); kept as a raising stub."""
    raise RuntimeError(
        "fused_dense_sparse_cuda_int8 is archived; use fused_dense_sparse_cuda_int4."
    )


@traced("cuda.fused_dense_sparse_e2e")
def fused_dense_sparse_e2e_cuda(
    X_fp16, perm,
    W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
    scale_u4, zero_u4, d_out, d_in,
    *, token_major: bool = False, force: Optional[str] = None, prepared=None,
) -> torch.Tensor:
    """fp16 activations in, ``Y (d_out, T)`` fp16 out: quantisation and GEMM are
    chained inside one C-ABI call (ops.py:707-747).  ``prepared``: the pair from
    :func:`prepare_weights_cuda` for the many-token kernel."""
    assert X_fp16.is_cuda and X_fp16.dtype == torch.float16
    assert perm.dtype in (torch.int32, torch.int64)
    assert W_low_packed.is_cuda and W_low_packed.dtype == torch.int8
    d_out, d_in = int(d_out), int(d_in)
    if X_fp16.shape[-1] != d_in:
        raise ValueError(f"X last dim ({X_fp16.shape[-1]}) must match d_in ({d_in})")
    X2 = X_fp16 if X_fp16.dim() == 2 else X_fp16.reshape(-1, d_in)
    if not X2.is_contiguous():
        X2 = X2.contiguous()
    T = int(X2.shape[0])
    dev = W_low_packed.device
    W = W_low_packed.contiguous()
    Wh = W_high_blocks_packed.contiguous()
    nnz = int(Wh.shape[0]) if Wh.numel() else 0
    ro = _cd(hp_row_offsets, torch.int32)
    ci = _cd(hp_col_indices, torch.int32)
    _check_bsr(ro, ci, d_out, d_in, nnz)
    s = _cd(scale_u4, torch.float16)
    z = _cd(zero_u4, torch.float16)
    perm_i32 = _cd(perm if perm.device == dev else perm.to(dev), torch.int32)
    Y = _out(d_out, T, dev, token_major)
    if T == 0:
        return Y
    with _lib.on_device(dev):
        ws = _lib.workspace(dev, T, d_in, d_out, nnz)
        plo, phi = _prepared_ptrs(prepared, W, Wh, nnz)
        _lib.check(_L.w4a4_fused_quant_dense_sparse_prepared(
            X2.data_ptr(), X2.stride(0), perm_i32.data_ptr(), W.data_ptr(),
            Wh.data_ptr() if nnz else None, plo, phi, ro.data_ptr(), ci.data_ptr() if nnz else None,
            s.data_ptr(), z.data_ptr(), Y.data_ptr(), T, d_in, d_out, nnz,
            _flags(token_major, force), ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)),
            "fused_quant_dense_sparse")
    return Y


def fused_quant_gemv_cuda(
    X_fp16, perm,
    W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
    scale_u4, zero_u4, d_out, d_in,
) -> torch.Tensor:
    """T == 1 fused quant + GEMV (ops.py:484-517); any d_in is accepted here."""
    T = X_fp16.shape[0]
    if T != 1:
        raise ValueError(f"fused_quant_gemv_cuda requires T == 1, got {T}")
    return fused_dense_sparse_e2e_cuda(X_fp16, perm, W_low_packed, W_high_blocks_packed,
                                       hp_row_offsets, hp_col_indices, scale_u4, zero_u4, d_out, d_in)


@traced("cuda.fused_quant_dense_sparse")
def fused_quant_dense_sparse_cuda_int4(
    X_fp16, perm,
    W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
    scale_u4, zero_u4, d_out, d_in,
) -> torch.Tensor:
    """T >= 2 fused quant + GEMM (ops.py:558-622); the residual is supported."""
    T = X_fp16.shape[0] if X_fp16.dim() == 2 else X_fp16.shape[0] * X_fp16.shape[1]
    if T < 2:
        raise ValueError(
            f"fused_quant_dense_sparse_cuda_int4 requires T >= 2, got {T}; "
            f"use fused_quant_gemv_cuda for T=1."
        )
    return fused_dense_sparse_e2e_cuda(X_fp16, perm, W_low_packed, W_high_blocks_packed,
                                       hp_row_offsets, hp_col_indices, scale_u4, zero_u4, d_out, d_in)


def dump_accumulators(W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices, X_s4,
                      d_out, d_in, *, force: Optional[str] = None, prepared=None, e4m3_packed: bool = False):
    """Parity aid: the exact int32 accumulators of the MMA path, ``acc (ng, d_out,
    T)`` per group and ``acc_hi (nnz, 128, T)`` per residual block.  ``e4m3_packed=True`` runs the
    tensor-core kernel's fp8 instantiation on the packed weights (offset taken out, integers again)."""
    d_out, d_in = int(d_out), int(d_in)
    T = int(X_s4.shape[0])
    dev = X_s4.device
    nnz = int(W_high_blocks_packed.shape[0]) if W_high_blocks_packed is not None else 0
    acc = torch.zeros((d_in // BCOL, d_out, T), dtype=torch.int32, device=dev)
    acc_hi = torch.zeros((nnz, BROW, T), dtype=torch.int32, device=dev)
    W = W_low_packed.contiguous()
    X = X_s4.contiguous()
    # converted copies stay referenced until the call has been issued
    Wh = W_high_blocks_packed.contiguous() if nnz else None
    ro = _cd(hp_row_offsets, torch.int32) if nnz else None
    ci = _cd(hp_col_indices, torch.int32) if nnz else None
    with _lib.on_device(dev):
        ws = _lib.workspace(dev, T, d_in, d_out, nnz)
        plo, phi = _prepared_ptrs(prepared, W, Wh, nnz)
        _lib.check(_L.w4a4_dump_accumulators_prepared(
            W.data_ptr(), Wh.data_ptr() if nnz else None, plo, phi,
            ro.data_ptr() if nnz else None,
            ci.data_ptr() if nnz else None,
            X.data_ptr(), acc.data_ptr(), acc_hi.data_ptr() if nnz else None, T, d_in, d_out, nnz,
            _flags(False, force) | (_lib.FLAG_CODES_E4M3_PACKED if e4m3_packed else 0), ws.data_ptr(), ws.numel(),
            _lib.stream_ptr(dev)), "dump_accumulators")
    return acc, acc_hi


__all__ = [
    "activation_quant_cuda",
    "dense_gemm_cuda",
    "sparse_gemm_cuda",
    "fused_dense_sparse_cuda",
    "dense_gemm_cuda_int8",
    "sparse_gemm_cuda_int8",
    "fused_dense_sparse_cuda_int8",
    "dense_gemm_cuda_int4",
    "sparse_gemm_cuda_int4",
    "fused_dense_sparse_cuda_int4",
    "dense_gemv_cuda_decode",
    "fused_gemv_cuda_decode",
    "fused_gemv_cuda_smallT",
    "fused_quant_gemv_cuda",
    "fused_quant_dense_sparse_cuda_int4",
    "fused_dense_sparse_e2e_cuda",
    "dump_accumulators",
    "prepare_weights_cuda",
    "reserve_workspace",
    "expand_activations_cuda",
    "fused_dense_sparse_expanded_cuda",
    "dequant_u4_to_fp16_cuda",
    "rmsnorm_quant_cuda",
    "silu_mul_quant_cuda",
    "perm_or_none",
]
